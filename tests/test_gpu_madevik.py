"""Madevik on the GPU against the plain implementation: every mechanism alone, then whole models through the step
function under every way of cutting the same requests, then generation and the trace program."""
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests import traces
from tests.helpers import ARGMAX_SHARE, RMS_TOL, TOL
from tests.madevik_cases import MADEVIK, madevik_folder
from tests.plain import madevik_plain as P
from tests.tiny import random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"


def ops():
    from jllm_serve_b200.csrc import ops as o
    o.require_device()
    return o


def close(got, want, dtype, what):
    tol = (2e-5 if dtype == torch.float32 else 1.6e-2) * float(want.abs().max())
    diff = float((got.double().cpu() - want.double()).abs().max())
    assert diff <= tol, f"{what}: largest difference {diff:.3e} exceeds {tol:.3e}"


# ---- every mechanism alone ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dim, rows", [(40, 3), (333, 17), (4096, 2)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh(dim, rows, out_dtype):
    g = torch.Generator().manual_seed(dim)
    x = torch.randn(rows + 4, dim, generator=g) * 3
    w = {"n": torch.randn(dim, generator=g).bfloat16().float(), "n.b": torch.randn(dim, generator=g).bfloat16().float(),
         "n.alpha": torch.tensor(0.37)}
    index = torch.tensor([rows + 3 - r for r in range(rows)], dtype=torch.int32)
    out = torch.empty(rows, dim, dtype=out_dtype, device=DEV)
    ops().dynamic_tanh(x.to(DEV), w["n"].bfloat16().to(DEV), w["n.b"].bfloat16().to(DEV), 0.37, out, index.to(DEV))
    close(out, P.dyt(x.double()[index.long()], {k: v.double() for k, v in w.items()}, "n"), out_dtype, "dynamic_tanh")


@pytest.mark.parametrize("experts, top, dim", [(8, 3, 328), (5, 1, 72), (3, 3, 40), (64, 6, 1000)])
def test_router_chooses_by_corrected_score_and_weighs_by_plain_score(experts, top, dim):
    g = torch.Generator().manual_seed(experts)
    h = torch.randn(33, dim, generator=g)
    w = {"r.router": torch.randn(experts, dim, generator=g) / math.sqrt(dim) * 2, "r.correction": torch.randn(experts, generator=g)}
    want = P.routing(h.double(), {k: v.double() for k, v in w.items()}, "r.", {"top": top, "scale": 1.7, "experts": experts})
    got = torch.empty(33, experts, dtype=torch.float32, device=DEV)
    ops().route_experts(h.to(DEV), w["r.router"].to(DEV), w["r.correction"].to(DEV), top, 1.7, True, got)
    assert ((got > 0).sum(dim=1) == top).all()
    close(got, want, torch.float32, "router weights")
    # the correction decides who is chosen: without it the choice differs somewhere, the weights of the chosen do not
    plain = torch.empty_like(got)
    ops().route_experts(h.to(DEV), w["r.router"].to(DEV), None, top, 1.7, True, plain)
    if top < experts:
        assert ((plain > 0) != (got > 0)).any()


def plain_recurrence(q, k, v, z, tau, state):
    """q, k [T, H, dk], v [T, H, dv], z [T, H, dk] (float64); state [H, dk, dv] updated in place; returns o [T, H, dv]."""
    T, H, dk = q.shape
    o = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    d = torch.sigmoid(z).pow(1.0 / tau)
    for t in range(T):
        for h in range(H):
            state[h] = d[t, h][:, None] * state[h] + torch.outer(k[t, h], v[t, h])
            o[t, h] = state[h].T @ q[t, h]
    return o


@pytest.mark.parametrize("heads, dk, dv", [(2, 16, 24), (1, 20, 12), (3, 64, 64), (1, 96, 33), (2, 128, 40), (1, 300, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunked", [False, True])
def test_linear_attention_recurrence_over_segments_slots_and_portions(heads, dk, dv, dtype, chunked):
    """Three requests in slots 2, 0 and 3 of a state storage with five: one of 37 tokens in portions of 1 + 20 + 2 + 14,
    one of 9 tokens whole, one token by token; the others' slots keep the values they had. Token by token, and in
    chunks (there with a temperature so low that some channels' decays over a chunk underflow: nothing may overflow)."""
    o_ = ops()
    g = torch.Generator().manual_seed(heads * 1000 + dk)
    lengths, slots, tau, scale = {"a": 37, "b": 9, "c": 5}, {"a": 2, "b": 0, "c": 3}, (0.05 if chunked else 3.0), dk ** -0.5
    width = heads * (2 * dk + dv) + 8
    data = {r: (torch.randn(n, width, generator=g).to(dtype), torch.randn(n, heads * dk, generator=g) * 3 + 2) for r, n in lengths.items()}
    state = torch.full((5, heads, dk, dv), 7.0, device=DEV)
    for s in slots.values():
        state[s].zero_()
    q_off, k_off, v_off = 8, 8 + heads * dk, 8 + 2 * heads * dk
    steps = [[("a", 1), ("b", 9)], [("a", 20), ("c", 1)], [("c", 1), ("a", 2)], [("a", 14), ("c", 1)], [("c", 1)], [("c", 1)]]
    fed, got = {r: 0 for r in lengths}, {r: [] for r in lengths}
    for step in steps:
        proj = torch.cat([data[r][0][fed[r]:fed[r] + n] for r, n in step]).to(DEV)
        z = torch.cat([data[r][1][fed[r]:fed[r] + n] for r, n in step]).to(DEV)
        counts = [n for _, n in step]
        starts = [sum(counts[:i]) for i in range(len(counts))]
        out = torch.full((sum(counts), heads * dv), float("nan"), device=DEV)
        tables = (torch.tensor(starts, dtype=torch.int32, device=DEV), torch.tensor(counts, dtype=torch.int32, device=DEV),
                  torch.tensor([slots[r] for r, _ in step], dtype=torch.int32, device=DEV))
        if chunked:
            rows = sum(counts)
            o_.gla_chunked(proj, q_off, k_off, v_off, z, state, *tables, out, heads, dk, dv, scale, tau, max(counts),
                           torch.empty(rows, heads * dk, device=DEV), torch.empty(rows, heads * dk, device=DEV),
                           torch.empty(rows, heads * o_.GLA_CHUNK, device=DEV))
        else:
            o_.gla_recurrent(proj, q_off, k_off, v_off, z, state, *tables, out, heads, dk, dv, scale, tau)
        for (r, n), s in zip(step, starts):
            got[r].append(out[s:s + n].cpu())
            fed[r] += n
    assert (state[1] == 7).all() and (state[4] == 7).all()
    for r, n in lengths.items():
        p = data[r][0].double()
        S = torch.zeros(heads, dk, dv, dtype=torch.float64)
        want = plain_recurrence(p[:, q_off:k_off].view(n, heads, dk) * scale, p[:, k_off:v_off].view(n, heads, dk),
                                p[:, v_off:v_off + heads * dv].view(n, heads, dv), data[r][1].double().view(n, heads, dk), tau, S)
        close(torch.cat(got[r]), want.view(n, -1), torch.float32, f"outputs of {r}")
        close(state[slots[r]], S, torch.float32, f"state of {r}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_and_gate(dtype):
    o_ = ops()
    g = torch.Generator().manual_seed(1)
    rows, heads, dv = 11, 3, 40
    o = torch.randn(rows, heads * dv, generator=g) * 5
    gate = torch.randn(rows, heads * dv + 16, generator=g).to(dtype)
    gain = torch.randn(dv, generator=g).bfloat16()
    y = torch.empty(rows, heads * dv, dtype=dtype, device=DEV)
    o_.gated_head_norm(o.to(DEV), gate.to(DEV)[:, 16:], gain.to(DEV), 1e-5, 0.5, y, heads, dv)
    gd = gate[:, 16:].double()
    want = (P.rms(o.double().view(rows, heads, dv), 1e-5) * gain.double()).view(rows, -1) * gd * torch.sigmoid(gd) * 0.5
    close(y, want, dtype, "gated head norm")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_products_per_head_with_the_output_gate(dtype):
    o_ = ops()
    g = torch.Generator().manual_seed(2)
    rows, heads, K, N = 70, 5, 24, 100
    a = torch.randn(rows, heads * K + 8, generator=g).to(dtype)
    w = torch.randn(heads, N, K, generator=g).to(dtype)
    gate = torch.randn(rows, heads, generator=g).to(dtype)
    out = torch.empty(rows, heads * N, dtype=dtype, device=DEV)
    o_.gemm_heads(a.to(DEV)[:, 8:], w.to(DEV), out, gate.to(DEV), 0.5)
    want = torch.einsum("rhk,hnk->rhn", a[:, 8:].double().view(rows, heads, K), w.double())
    want = want * torch.sigmoid(gate.double())[:, :, None] * 0.5
    close(out, want.reshape(rows, -1), dtype, "per-head product")


# ---- whole models through the step function ---------------------------------------------------------------------------

class Checker:
    """Rows against the plain implementation's float64 logits. float32: every row within the tolerance. bfloat16: a
    rounded input may turn a router's close call, which changes that token's experts outright, so up to 2 % of the rows
    may lie beyond the tolerance; the rms error and the share of equal choices hold over all rows."""

    def __init__(self, folder, sequences, dtype, what):
        self.cfg, self.w = P.load_plain(folder)
        self.sequences, self.dtype, self.what = sequences, dtype, what
        self.plain, self.errors, self.flips, self.err2, self.ref2, self.scale = {}, [], 0, 0.0, 0.0, 0.0
        self.seen = set()

    def row(self, rid, position, got):
        if rid not in self.plain:
            self.plain[rid] = P.forward(self.cfg, self.w, self.sequences[rid])
        want = self.plain[rid][position]
        assert torch.isfinite(got).all(), f"{self.what}: non-finite logits for {rid} position {position}"
        d = got.double() - want
        self.errors.append((float(d.abs().max()), rid, position))
        self.err2 += float((d * d).sum())
        self.ref2 += float((want * want).sum())
        self.scale = max(self.scale, float(want.abs().max()))
        self.flips += int(got.argmax()) != int(want.argmax())
        self.seen.add((rid, position))

    def finish(self):
        for rid, toks in self.sequences.items():
            missing = [p for p in range(len(toks)) if (rid, p) not in self.seen]
            assert not missing, f"{self.what}: no logits for {rid} positions {missing[:5]}"
        tol = TOL[self.dtype] * self.scale
        worst = max(self.errors)
        over = [e for e in self.errors if e[0] > tol]
        rms = (self.err2 / max(self.ref2, 1e-300)) ** 0.5
        print(f"{self.what} [{self.dtype}] rows {len(self.errors)}: largest difference {worst[0]:.3e} at {worst[1:]} "
              f"({worst[0] / self.scale:.2e} of the largest |logit|), {len(over)} rows over, rms {rms:.2e}")
        allowed = 0 if self.dtype == "float32" else max(1, len(self.errors) // 50)
        first = min(over, key=lambda e: (e[1], e[2])) if over else None
        assert len(over) <= allowed, \
            f"{self.what}: {len(over)} rows beyond {tol:.3e}, the first at {first}, the largest {worst}"
        assert rms <= 3 * RMS_TOL[self.dtype] and 1 - self.flips / len(self.errors) >= ARGMAX_SHARE[self.dtype] - 0.02


def run_trace(name, dtype, steps, sequences, what, **kw):
    from jllm_serve_b200.csrc import ops as o
    from jllm_serve_b200.engine import ModelRunner, Segment
    args = dict(dtype=dtype, page_size=16, max_tokens=traces.peak_tokens(steps, 16), max_batch_tokens=512, max_requests=4,
                ctx=1024, poison_freed_pages=True)
    args.update(kw)
    runner = ModelRunner(madevik_folder(name), **args)
    checker = Checker(madevik_folder(name), sequences, dtype, f"{name} {what}")
    fed = {}
    for st in steps:
        segs = [Segment(e["id"], e["tokens"], fed.get(e["id"], 0), e["want"]) for e in st["entries"]]
        rows = runner.step(segs).float().cpu()
        r = 0
        for e in st["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                checker.row(e["id"], base + w, rows[r])
                r += 1
            fed[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            runner.finish(rid)
            fed.pop(rid, None)
    runner.cache.check()
    o.check_kernel_errors()
    checker.finish()
    runner.close()


def sequences_for(name, lengths, seed=21):
    return {f"r{i}": random_tokens(n, MADEVIK[name]["vocab"], seed + i) for i, n in enumerate(lengths)}


LENGTHS = (1, 2, 37, 150, 16, 333, 65, 129)
WAYS = {
    "whole": traces.whole,
    "prompt, then token by token": lambda r: traces.prompt_then_decode(r, tail=24),
    "portions down to two tokens": traces.changing_portions,
    "all requests side by side": lambda r: traces.all_together(dict(list(r.items())[:4]), tail=6),
    "mixed, slots and pages used again": lambda r: traces.mixed(r, max_live=4, portion=40, prefill_share=0.7),
}


@pytest.mark.parametrize("way", list(WAYS))
@pytest.mark.parametrize("name", ["P", "Q", "R"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cut_of_the_same_requests_gives_the_plain_logits(name, dtype, way):
    seqs = sequences_for(name, LENGTHS)
    steps = WAYS[way](seqs)
    used = {e["id"] for st in steps for e in st["entries"]}
    run_trace(name, dtype, steps, {r: t for r, t in seqs.items() if r in used}, way)


@pytest.mark.parametrize("way", ["prompt, then token by token", "mixed, slots and pages used again"])
@pytest.mark.parametrize("name", ["S", "T"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_of_one_kind_of_mixer_only(name, dtype, way):
    """States and no pages at all; pages in three groups of different widths and no state."""
    seqs = sequences_for(name, (3, 70, 1, 141, 18), seed=31)
    run_trace(name, dtype, WAYS[way](seqs), seqs, way)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_a_page_size_that_cuts_elsewhere(dtype):
    seqs = sequences_for("P", (420,), seed=5)
    run_trace("P", dtype, traces.prompt_then_decode(seqs, tail=300), seqs, "300 tokens one by one", page_size=8)


def test_a_state_slot_and_pages_that_are_used_again_start_clean():
    """One state slot and few pages: every request gets the slot and the pages the one before it left."""
    seqs = sequences_for("Q", (90, 3, 61, 1, 40), seed=8)
    run_trace("Q", "float32", traces.whole(seqs), seqs, "one slot", max_requests=1, max_tokens=96)
    run_trace("Q", "float32", traces.changing_portions(seqs, sizes=(2, 9, 2, 31)), seqs, "one slot, portions", max_requests=1,
              max_tokens=96)


def test_more_rows_than_a_batch_holds_run_as_several_batches():
    seqs = sequences_for("P", (300, 77), seed=12)
    run_trace("P", "float32", traces.all_together(seqs, tail=2), seqs, "a step in parts", max_batch_tokens=64)


# ---- generation and the trace program -----------------------------------------------------------------------------------

def engine_for(name, dtype, **kw):
    from jllm_serve_b200.engine import Engine
    args = dict(dtype=dtype, page_size=8, max_tokens_cached=1024, max_batch_tokens=64, chunk=32, min_chunk=4, max_running=4,
                ctx=256)
    args.update(kw)
    return Engine(madevik_folder(name), **args)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_greedy_generation_float32_equals_plain(name):
    from jllm_serve_b200.sampling import SamplingParams
    cfg, w = P.load_plain(madevik_folder(name))
    prompts = [random_tokens(n, MADEVIK[name]["vocab"], 40 + n) for n in (5, 17, 41, 2, 33, 9)]
    got = engine_for(name, "float32").generate(prompts, SamplingParams.greedy_params(12, ignore_eos=True))
    for p, r in zip(prompts, got):
        assert r.tokens == P.greedy_generate(cfg, w, p, 12) and r.finish_reason == "length"


def test_greedy_generation_bfloat16_follows_plain():
    from jllm_serve_b200.sampling import SamplingParams
    cfg, w = P.load_plain(madevik_folder("R"))
    prompts = [random_tokens(n, MADEVIK["R"]["vocab"], 60 + n) for n in (9, 40, 70)]
    got = engine_for("R", "bfloat16").generate(prompts, SamplingParams.greedy_params(10, ignore_eos=True))
    for p, r in zip(prompts, got):
        logits = P.forward(cfg, w, p + r.tokens[:-1])
        for i, t in enumerate(r.tokens):
            row = logits[len(p) - 1 + i]
            assert float(row.max() - row[t]) <= 2 * TOL["bfloat16"] * float(logits.abs().max()), (i, t)


def test_generation_with_preemption_in_a_small_pool_equals_plain():
    from jllm_serve_b200.sampling import SamplingParams
    cfg, w = P.load_plain(madevik_folder("P"))
    prompts = [random_tokens(n, MADEVIK["P"]["vocab"], 80 + n) for n in (60, 1, 33, 64, 100, 20)]
    params = SamplingParams.greedy_params(16, ignore_eos=True)
    got = engine_for("P", "float32", max_tokens_cached=200, max_batch_tokens=48).generate(prompts, params)
    for i, (p, r) in enumerate(zip(prompts, got)):
        assert r.tokens == P.greedy_generate(cfg, w, p, 16), f"request {i}"


def test_command_line_run_and_bench_on_a_madevik_model(tmp_path):
    folder = madevik_folder("Q")
    prompt = random_tokens(11, MADEVIK["Q"]["vocab"], 5)
    cmd = [sys.executable, str(ROOT / "bin" / "jllm"), "run", "--model", str(folder), "--dtype", "fp32", "--temp", "0",
           "--max-tokens", "7", "--ctx", "64", "--ignore-eos", "--tokens", ",".join(map(str, prompt))]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    cfg, w = P.load_plain(folder)
    assert [int(t) for t in proc.stdout.strip().split(",")] == P.greedy_generate(cfg, w, prompt, 7)
    assert "11 prompt tok" in proc.stderr and "7 generated" in proc.stderr
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(MADEVIK["P"]))
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "jllm"), "bench", "--random-weights", "3", "--model-config",
                           str(cfg_file), "--ctx", "256", "--bench.prompt-tokens", "50", "--bench.max-tokens", "8",
                           "--bench.rounds", "2"], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.startswith("prefill 50 tok in") and "decode 8 tok in" in proc.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program_on_a_madevik_folder(dtype, tmp_path):
    seqs = sequences_for("P", (50, 7, 1, 90, 33), seed=30)
    steps = traces.mixed(seqs, max_live=4, portion=24)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(madevik_folder("P")), "--dtype", dtype,
                           "--out", str(tmp_path), "--max-tokens", str(traces.peak_tokens(steps)), "--poison"],
                          input=text, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    import numpy as np
    vocab = MADEVIK["P"]["vocab"]
    checker = Checker(madevik_folder("P"), seqs, dtype, "trace program")
    fed = {}
    for st in steps:
        rows = torch.from_numpy(np.fromfile(tmp_path / f"{st['step']}.f32", dtype="<f4").reshape(-1, vocab))
        r = 0
        for e in st["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                checker.row(e["id"], base + w, rows[r])
                r += 1
            fed[e["id"]] = base + len(e["tokens"])
    checker.finish()
