"""Movivik on the GPU against the plain implementation: every mechanism alone, then whole models through the step
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
from tests.movivik_cases import MOVIVIK, movivik_folder
from tests.plain import movivik_plain as P
from tests.tiny import random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"


def ops():
    from jllm_serve_b200.csrc import ops as o
    o.require_device()
    return o


def close(got, want, dtype, what, loose=1.0):
    tol = (2e-5 if dtype == torch.float32 else 1.6e-2) * float(want.abs().max()) * loose
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    diff = float((got.double().cpu() - want.double()).abs().max())
    assert diff <= tol, f"{what}: largest difference {diff:.3e} exceeds {tol:.3e}"


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


# ---- every mechanism alone ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("heads, kv_heads, dk, dv, dims, pairing, unit, pre", [
    (4, 2, 24, 16, 16, "interleaved", False, False), (3, 3, 16, 24, 8, "half", True, False),
    (4, 2, 128, 128, 48, "half", True, False), (5, 1, 80, 48, 80, "interleaved", False, False),
    (2, 2, 64, 64, 64, "half", False, True), (1, 1, 40, 300, 0, "half", True, True), (5, 1, 272, 8, 2, "interleaved", True, False),
    (3, 1, 256, 256, 64, "half", True, True), (5, 5, 64, 64, 16, "interleaved", True, False), (4, 2, 128, 128, 128, "interleaved", False, True),
    (2, 1, 256, 256, 256, "half", False, False), (7, 1, 64, 64, 48, "half", True, False), (2, 2, 128, 128, 0, "half", True, True)])
@pytest.mark.parametrize("aligned", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_preparation(heads, kv_heads, dk, dv, dims, pairing, unit, pre, dtype, aligned):
    """Rotation of either pairing over part of a head, the unit norm behind it, a norm with gains in front, keys and values
    of different widths into cache rows as wide as the wider; positions far apart."""
    g = torch.Generator().manual_seed(heads * 100 + dk)
    rows, page, pages, eps = 9, 4, 7, 1e-5
    positions = [0, 1, 2, 77, 500, 3, 1023, 31, 32]
    rot = {"dims": max(dims, 2), "base": 300.0, "scaling": {"factor": 3.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    f, amp = P.rotary_frequencies(rot)
    angle = torch.arange(1024, dtype=torch.float64)[:, None] * torch.tensor(f, dtype=torch.float64)[None, :]
    cos, sin = (torch.cos(angle) * amp).float().to(DEV), (torch.sin(angle) * amp).float().to(DEV)
    # `aligned`: every piece starts at a multiple of 8 values (what the register form of the kernel wants; heads of 64, 128
    # and 256 values then take it), else anywhere
    gap = (8, 16, 8) if aligned else (3, 5, 2)
    q_off, k_off = 8, 8 + heads * dk + gap[0]
    v_off = k_off + kv_heads * dk + gap[1]
    width = -(-(v_off + kv_heads * dv + gap[2]) // 8) * 8 if aligned else v_off + kv_heads * dv + gap[2]
    qkv = (torch.randn(rows, width, generator=g) * 2).to(dtype)
    gq, gk = (1 + 0.3 * torch.randn(dk, generator=g)).bfloat16(), (1 + 0.3 * torch.randn(dk, generator=g)).bfloat16()
    cache_dim = max(dk, dv)
    kc = torch.full((pages, kv_heads, page, cache_dim), 5.0, dtype=dtype, device=DEV)
    vc = torch.full_like(kc, 5.0)
    slots = [3, 26, 9, 0, 27, 14, 5, 20, 11]
    dev = qkv.to(DEV)
    ops().head_prepare(dev, q_off, k_off, v_off, gq.to(DEV) if pre else None, gk.to(DEV) if pre else None, eps, cos, sin, dims,
                       pairing, unit, i32(positions), i32(slots), kc, vc, heads, kv_heads, dk, dv, page)
    x = qkv.double()
    q, k = x[:, q_off:q_off + heads * dk].view(rows, heads, dk), x[:, k_off:k_off + kv_heads * dk].view(rows, kv_heads, dk)
    v = x[:, v_off:v_off + kv_heads * dv].view(rows, kv_heads, dv)
    if pre:
        q, k = P.rms(q, eps) * gq.double(), P.rms(k, eps) * gk.double()
    if dims:
        q, k = P.rotate(q, positions, rot, pairing), P.rotate(k, positions, rot, pairing)
    if unit:
        q, k = P.rms(q, eps), P.rms(k, eps)
    close(dev[:, q_off:q_off + heads * dk], q.reshape(rows, -1), dtype, "queries")
    assert torch.equal(dev[:, :q_off].cpu(), qkv[:, :q_off]) and torch.equal(dev[:, k_off:].cpu(), qkv[:, k_off:])
    for r, s in enumerate(slots):
        close(kc[s // page, :, s % page, :dk], k[r], dtype, f"key of row {r}")
        close(vc[s // page, :, s % page, :dv], v[r], dtype, f"value of row {r}", loose=2)
    untouched = sorted(set(range(pages * page)) - set(slots))
    assert all((kc[s // page, :, s % page] == 5).all() and (vc[s // page, :, s % page] == 5).all() for s in untouched)
    if dk < cache_dim:
        assert (kc[..., dk:] == 5).all()
    if dv < cache_dim:
        assert (vc[..., dv:] == 5).all()


def plain_attention(q, k, v, scale, chunk, window=0):
    """q [L, H, dk], k [L, G, dk], v [L, G, dv] of one sequence (float64): row t over the keys it sees."""
    L, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(L, H, v.shape[2], dtype=torch.float64)
    for t in range(L):
        lo = t - t % chunk if chunk else (max(0, t + 1 - window) if window else 0)
        for h in range(H):
            kv = h // (H // G)
            p = torch.softmax((k[lo:t + 1, kv] @ q[t, h]) * scale, dim=0)
            out[t, h] = (p[:, None] * v[lo:t + 1, kv]).sum(dim=0)
    return out


def chunk_case(dtype, H, G, dk, dv, page, lens, q_lens, chunk, scale, seed=0):
    """Requests of `lens` cached positions, of which the last `q_lens` are the step's rows. The first key of every chunk
    answers every query strongly (score 8) and carries the value +10; the key just in front of it, the last of the chunk
    before, answers more strongly still (score 10.4) and carries -30: a row that sees one key too many, or one too few,
    is far off. Pages are dealt out in a random order; unused rows and pages hold NaN."""
    g = torch.Generator().manual_seed(seed + H * 1000 + dk + page)
    cache_dim = max(dk, dv)
    pool = sum(-(-l // page) for l in lens) + 3
    perm = torch.randperm(pool, generator=g).tolist()
    kc = torch.full((pool, G, page, cache_dim), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full_like(kc, float("nan"))
    tables = torch.full((len(lens), max(-(-l // page) for l in lens) + 2), -1, dtype=torch.int32)
    rows_q, row_seg, row_pos, wants = [], [], [], []
    for s, L in enumerate(lens):
        q, k, v = torch.randn(L, H, dk, generator=g) * 0.3, torch.randn(L, G, dk, generator=g), torch.randn(L, G, dv, generator=g)
        k[:, :, 1] = 0
        q[:, :, 1] = 8.0 / scale
        if chunk:
            firsts = torch.arange(0, L, chunk)
            k[firsts], v[firsts] = 0, 10.0
            k[firsts, :, 1] = 1.0
            lasts = firsts[1:] - 1
            k[lasts], v[lasts] = 0, -30.0
            k[lasts, :, 1] = 1.3
        q, k, v = q.to(dtype).double(), k.to(dtype).double(), v.to(dtype).double()
        for b in range(-(-L // page)):
            pg = perm.pop()
            tables[s, b] = pg
            n = min(page, L - b * page)
            kc[pg, :, :n, :dk] = k[b * page:b * page + n].transpose(0, 1).to(dtype).to(DEV)
            vc[pg, :, :n, :dv] = v[b * page:b * page + n].transpose(0, 1).to(dtype).to(DEV)
        want = plain_attention(q, k, v, scale, chunk).reshape(L, H * dv)
        for p in range(L - q_lens[s], L):
            rows_q.append(q[p].reshape(-1))
            row_seg.append(s)
            row_pos.append(p)
            wants.append(want[p])
    qd = torch.stack(rows_q).to(dtype).to(DEV)
    out = torch.full((qd.shape[0], H * dv), float("nan"), dtype=dtype, device=DEV)
    return qd, kc, vc, out, i32(row_seg), i32(row_pos), tables.to(DEV), torch.stack(wants)


def rows_close(got, want, what, share=2 ** -7, floor=2e-4):
    got, want = got.double().cpu(), want.double()
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    tol = share * want.abs().amax(dim=-1, keepdim=True) + floor
    ratio = ((got - want).abs() / tol).amax(dim=-1)
    worst = int(ratio.argmax())
    assert float(ratio[worst]) <= 1.0, (f"{what}: row {worst} differs by {float((got[worst] - want[worst]).abs().max()):.3e}, "
                                        f"its largest |value| is {float(want[worst].abs().max()):.3e}")


LENS, Q_LENS = [1, 17, 64, 131, 300, 1000, 77, 401], [1, 17, 30, 131, 200, 65, 1, 2]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, dk, dv, page, chunk", [(4, 2, 24, 16, 16, 20), (3, 3, 16, 24, 4, 16), (5, 1, 80, 48, 16, 150),
                                                        (2, 1, 128, 128, 8, 70), (20, 1, 16, 16, 16, 33), (2, 2, 32, 8, 16, 0),
                                                        (1, 1, 40, 300, 2, 5000)])
def test_plain_attention_with_chunks_and_two_head_widths(dtype, H, G, dk, dv, page, chunk):
    o_ = ops()
    scale = 1.0 / math.sqrt(dk)
    q, kc, vc, out, rseg, rpos, tables, want = chunk_case(dtype, H, G, dk, dv, page, LENS, Q_LENS, chunk, scale)
    o_.attention_plain(q, q.stride(0), kc, vc, out, rseg, rpos, tables, q.shape[0], H, G, dk, page, -chunk, scale, dv)
    if dtype == torch.float32:
        rows_close(out, want, f"plain chunk {chunk}", share=1e-5, floor=1e-6)
    else:
        rows_close(out, want, f"plain chunk {chunk}")


@pytest.mark.parametrize("kernel", ["mma", "tc", "pair"])
@pytest.mark.parametrize("H, G, hd, page, chunk", [(4, 2, 128, 16, 70), (2, 1, 128, 8, 128), (6, 3, 64, 16, 200), (2, 2, 64, 4, 16),
                                                    (2, 1, 256, 16, 129), (8, 1, 128, 32, 1000), (3, 1, 128, 16, 1), (2, 2, 128, 64, 257)])
def test_prompt_attention_kernels_stop_at_a_chunks_edge(kernel, H, G, hd, page, chunk):
    """Chunk edges inside, at and across the kernels' tiles of 64 and 128 keys and 128 query rows, in prompts' portions that
    begin anywhere."""
    if kernel != "mma" and hd != 128:
        pytest.skip("the tcgen05 kernels are built for head size 128")
    o_ = ops()
    scale = 1.0 / math.sqrt(hd)
    lens, q_lens = [128, 129, 700, 1500, 256, 383, 1, 17], [128, 2, 513, 300, 129, 255, 1, 17]
    q, kc, vc, out, rseg, rpos, tables, want = chunk_case(torch.bfloat16, H, G, hd, hd, page, lens, q_lens, chunk, scale)
    starts = [sum(q_lens[:i]) for i in range(len(lens))]
    o_.attention_prefill(q, kc, vc, out, i32(starts), i32(q_lens), i32(lens), tables, q.shape[0], H, G, hd, page, -chunk, scale,
                         kernel=kernel)
    assert o_.attention_prefill_tc_error() == 0
    rows_close(out, want, f"prefill {kernel} chunk {chunk}")


@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("H, G, hd, page, chunk", [(4, 2, 128, 16, 70), (6, 3, 64, 16, 200), (2, 2, 48, 4, 16), (16, 1, 256, 16, 129),
                                                    (8, 2, 128, 32, 1000), (3, 1, 80, 8, 1), (2, 1, 64, 16, 64)])
def test_decode_attention_stops_at_a_chunks_edge(splits, H, G, hd, page, chunk):
    """One row per request, at the first, the second and the last position of a chunk and anywhere else; also with the
    keys split over blocks and dealt out evenly."""
    o_ = ops()
    scale = 1.0 / math.sqrt(hd)
    lens = [1, 17, 64, 131, 300, 1000, chunk, chunk + 1, 2 * chunk, 2 * chunk + 1, 3 * chunk + 2]
    q, kc, vc, out, rseg, rpos, tables, want = chunk_case(torch.bfloat16, H, G, hd, hd, page, lens, [1] * len(lens), chunk, scale)
    scratch = torch.full((o_.attention_decode_scratch_floats(len(lens), H, hd, splits) + 1,), float("nan"), device=DEV)
    o_.attention_decode(q, kc, vc, out, rseg, rpos, tables, len(lens), H, G, hd, page, -chunk, scale, splits, scratch)
    rows_close(out, want, f"decode chunk {chunk} splits {splits}")
    if hd in (64, 128, 256):
        out.fill_(float("nan"))
        blocks = 7
        flat = torch.full((o_.attention_decode_flat_scratch_floats(len(lens), H, G, hd, blocks) + 1,), float("nan"), device=DEV)
        o_.attention_decode_flat(q, kc, vc, out, rseg, rpos, tables, len(lens), H, G, hd, page, -chunk, scale, blocks, flat)
        rows_close(out, want, f"decode dealt out, chunk {chunk}")


@pytest.mark.parametrize("heads, dv", [(5, 24), (3, 7), (16, 128), (6, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_gate_norm_sum_and_gated_norm(dtype, heads, dv):
    o_ = ops()
    g = torch.Generator().manual_seed(4)
    rows, dim = 13, 200
    att = torch.randn(rows, heads * dv + 8, generator=g).to(dtype)
    gate = torch.randn(rows, heads + 3, generator=g).to(dtype)
    dev = att.to(DEV)
    o_.head_gate(dev[:, :heads * dv], gate.to(DEV)[:, 3:], heads, dv)
    want = att[:, :heads * dv].double().view(rows, heads, dv) * torch.sigmoid(gate[:, 3:].double())[:, :, None]
    close(dev[:, :heads * dv], want.reshape(rows, -1), dtype, "head gate")
    assert torch.equal(dev[:, heads * dv:].cpu(), att[:, heads * dv:])
    # x (+)= scale * (rms(a) ga + rms(b) gb)
    a, b, x = torch.randn(rows, dim, generator=g) * 7, torch.randn(rows, dim, generator=g) * 0.01, torch.randn(rows, dim, generator=g)
    ga, gb = (1 + 0.2 * torch.randn(dim, generator=g)).to(dtype), (1 + 0.2 * torch.randn(dim, generator=g)).to(dtype)
    both = P.norm(a.double(), ga.double(), 1e-5) + P.norm(b.double(), gb.double(), 1e-5)
    xd = x.to(DEV)
    o_.norm_sum(xd, a.to(DEV), ga.to(DEV), 1e-5, b.to(DEV), gb.to(DEV), scale=0.5, accumulate=True)
    close(xd, x.double() + 0.5 * both, torch.float32, "two normed results added")
    o_.norm_sum(xd, a.to(DEV), ga.to(DEV), 1e-5, accumulate=False)
    close(xd, P.norm(a.double(), ga.double(), 1e-5), torch.float32, "one normed result written")
    # one norm over all heads of a row, a sigmoid gate
    o = torch.randn(rows, heads * dv, generator=g) * 3
    gates = torch.randn(rows, heads * dv + 16, generator=g).to(dtype)
    gain = (1 + 0.2 * torch.randn(heads * dv, generator=g)).bfloat16()
    y = torch.empty(rows, heads * dv, dtype=dtype, device=DEV)
    o_.gated_head_norm(o.to(DEV), gates.to(DEV)[:, 16:], gain.to(DEV), 1e-5, 1.0, y, 1, heads * dv, "sigmoid")
    close(y, P.norm(o.double(), gain.double(), 1e-5) * torch.sigmoid(gates[:, 16:].double()), dtype, "norm over all heads, gated")


@pytest.mark.parametrize("dim", [56, 203, 2048, 5000, 8196])
@pytest.mark.parametrize("two", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_norms_between_two_parts_in_one_launch(dim, two, dtype):
    """x += norm(v), v one result or half the sum of two normed results; and the next part's normed input. Widths that the
    register form takes and widths that it leaves to the general form."""
    o_ = ops()
    g = torch.Generator().manual_seed(dim)
    rows, eps = 7, 1e-5
    a, b, x = torch.randn(rows, dim, generator=g) * 40, torch.randn(rows, dim, generator=g) * 0.02, torch.randn(rows, dim, generator=g)
    gains = [(1 + 0.2 * torch.randn(dim, generator=g)).to(dtype) for _ in range(4)]
    ga, gb, gp, gn = [t.double() for t in gains]
    v = 0.5 * (P.norm(a.double(), ga, eps) + P.norm(b.double(), gb, eps)) if two else a.double()
    want_x = x.double() + P.norm(v, gp, eps)
    xd, nxt = x.to(DEV), torch.full((rows, dim), float("nan"), dtype=dtype, device=DEV)
    dg = [t.to(DEV) for t in gains]
    o_.norm_chain(xd, a.to(DEV), dg[2], eps, b.to(DEV) if two else None, dg[0] if two else None, dg[1] if two else None, 0.5,
                  next_out=nxt, gain_next=dg[3])
    close(xd, want_x, torch.float32, "the stream")
    close(nxt, P.norm(want_x, gn, eps), dtype, "the next part's input")
    xd = x.to(DEV)
    o_.norm_chain(xd, a.to(DEV), dg[2], eps, b.to(DEV) if two else None, dg[0] if two else None, dg[1] if two else None, 0.5)
    close(xd, want_x, torch.float32, "the stream alone")


@pytest.mark.parametrize("rows", [1, 9, 40, 100, 300, 2100])
def test_products_with_the_gelu_gate_in_their_epilogue(rows):
    """act(gate) * up with the tanh form of GELU, in every product kernel's epilogue (the rows decide which kernel runs) and
    in the float32 path's own kernel."""
    from jllm_serve_b200.parts.linear import Linear
    o_ = ops()
    g = torch.Generator().manual_seed(rows)
    dim, hidden = 256, 384
    x = torch.randn(rows, dim, generator=g)
    gate, up = torch.randn(hidden, dim, generator=g) / 8, torch.randn(hidden, dim, generator=g) / 16
    want = P.gelu_tanh(x.bfloat16().double() @ gate.bfloat16().double().T) * (x.bfloat16().double() @ up.bfloat16().double().T)
    stacked = torch.stack([gate.view(hidden // 8, 8, dim), up.view(hidden // 8, 8, dim)], dim=1).reshape(2 * hidden, dim)
    lin = Linear(stacked.bfloat16().contiguous().to(DEV))
    h = torch.empty(rows, hidden, dtype=torch.bfloat16, device=DEV)
    lin.forward(x.bfloat16().to(DEV), h, swiglu="gelu_tanh")
    close(h, want, torch.bfloat16, "gelu gate in the epilogue")
    gu = torch.cat([x @ gate.T, x @ up.T], dim=1).to(DEV)
    h32 = torch.empty(rows, hidden, device=DEV)
    o_.swiglu(gu, h32, "gelu_tanh")
    close(h32, P.gelu_tanh(gu[:, :hidden].double().cpu()) * gu[:, hidden:].double().cpu(), torch.float32, "gelu gate, float32")
    o_.check_kernel_errors()


def plain_fixed_decay(q, k, v, decay, state):
    T, H, _ = q.shape
    o = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            state[h] = decay[h] * state[h] + torch.outer(k[t, h], v[t, h])
            o[t, h] = state[h].T @ q[t, h]
    return o


@pytest.mark.parametrize("heads, dk, dv, decays", [(2, 12, 20, (0.7, 0.97)), (3, 64, 64, (0.999, 0.6, 0.0)), (1, 40, 12, (1.0,)),
                                                   (4, 16, 24, (0.0, 1.0, 0.6, 0.95)), (2, 128, 40, (0.9, 0.99)), (1, 300, 8, (0.5,))])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunked", [False, True])
def test_fixed_decay_recurrence_over_segments_slots_and_portions(heads, dk, dv, decays, dtype, chunked):
    """Three requests in slots 2, 0 and 3 of a state storage with five: one of 37 tokens in portions of 1 + 20 + 2 + 14, one
    of 9 tokens whole, one token by token; silu on q, k and v in place; decays of 0 and 1 among the others."""
    o_ = ops()
    g = torch.Generator().manual_seed(heads * 1000 + dk)
    lengths, slots = {"a": 37, "b": 9, "c": 5}, {"a": 2, "b": 0, "c": 3}
    width = heads * (2 * dk + dv) + 8
    data = {r: (torch.randn(n, width, generator=g) * 1.5).to(dtype) for r, n in lengths.items()}
    state = torch.full((5, heads, dk, dv), 7.0, device=DEV)
    for s in slots.values():
        state[s].zero_()
    decay = torch.tensor(decays, dtype=torch.float32, device=DEV)
    q_off, k_off, v_off = 8, 8 + heads * dk, 8 + 2 * heads * dk
    steps = [[("a", 1), ("b", 9)], [("a", 20), ("c", 1)], [("c", 1), ("a", 2)], [("a", 14), ("c", 1)], [("c", 1)], [("c", 1)]]
    fed, got = {r: 0 for r in lengths}, {r: [] for r in lengths}
    for step in steps:
        proj = torch.cat([data[r][fed[r]:fed[r] + n] for r, n in step]).to(DEV)
        counts = [n for _, n in step]
        rows = sum(counts)
        starts = [sum(counts[:i]) for i in range(len(counts))]
        z = torch.full((rows, heads * dk), float("nan"), device=DEV)
        out = torch.full((rows, heads * dv), float("nan"), device=DEV)
        tables = (i32(starts), i32(counts), i32([slots[r] for r, _ in step]))
        if chunked:
            o_.gla_chunked(proj, q_off, k_off, v_off, z, state, *tables, out, heads, dk, dv, 1.0, 1.0, max(counts),
                           torch.empty(rows, heads * dk, device=DEV), torch.empty(rows, heads * dk, device=DEV),
                           torch.empty(rows, heads * o_.GLA_CHUNK, device=DEV), head_decay=decay, activation=1)
        else:
            o_.gla_recurrent(proj, q_off, k_off, v_off, z, state, *tables, out, heads, dk, dv, 1.0, 1.0, head_decay=decay,
                             activation=1)
        for (r, n), s in zip(step, starts):
            got[r].append(out[s:s + n].cpu())
            fed[r] += n
    assert (state[1] == 7).all() and (state[4] == 7).all()
    for r, n in lengths.items():
        p = P.silu(data[r].double())
        if dtype == torch.bfloat16:
            p = p.bfloat16().double()          # the activated projections are stored in the compute type
        S = torch.zeros(heads, dk, dv, dtype=torch.float64)
        want = plain_fixed_decay(p[:, q_off:k_off].view(n, heads, dk), p[:, k_off:v_off].view(n, heads, dk),
                                 p[:, v_off:v_off + heads * dv].view(n, heads, dv), [float(d) for d in decay.cpu()], S)
        close(torch.cat(got[r]), want.view(n, -1), torch.float32, f"outputs of {r}", loose=4 if dtype == torch.bfloat16 else 1)
        close(state[slots[r]], S, torch.float32, f"state of {r}", loose=4 if dtype == torch.bfloat16 else 1)


@pytest.mark.parametrize("heads, dk, dv, decays", [(2, 128, 128, (0.97, 0.6)), (3, 64, 64, (0.999, 0.0, 1.0)), (1, 128, 40, (0.9,)),
                                                   (2, 64, 200, (0.5, 0.99))])
@pytest.mark.parametrize("block_width", [32, 64])
def test_fixed_decay_chunks_on_the_tensor_cores(heads, dk, dv, decays, block_width):
    """Portions that span several chunks of 64 tokens, end inside one, or are shorter than one, on top of states that
    earlier portions left; value widths that are no multiple of a block's 64 columns; the float32 kernels (no activation
    there: the rows are activated once, by the first call) must agree."""
    o_ = ops()
    o_.lightning_block_width(block_width)
    g = torch.Generator().manual_seed(heads * 77 + dv)
    lengths, slots = {"a": 200 + 64 + 65 + 1, "b": 130, "c": 63 + 2}, {"a": 1, "b": 3, "c": 0}
    steps = [[("a", 200), ("b", 130)], [("c", 63), ("a", 64)], [("a", 65), ("c", 2)], [("a", 1)]]
    width = heads * (2 * dk + dv)
    data = {r: (torch.randn(n, width, generator=g) * 1.2).bfloat16() for r, n in lengths.items()}
    decay = torch.tensor(decays, dtype=torch.float32, device=DEV)
    q_off, k_off, v_off = 0, heads * dk, 2 * heads * dk
    state = torch.full((4, heads, dk, dv), 3.0, device=DEV)
    for s in slots.values():
        state[s].zero_()
    fed, got = {r: 0 for r in lengths}, {r: [] for r in lengths}
    for step in steps:
        proj = torch.cat([data[r][fed[r]:fed[r] + n] for r, n in step]).to(DEV)
        counts = [n for _, n in step]
        rows = sum(counts)
        starts = [sum(counts[:i]) for i in range(len(counts))]
        out = torch.full((rows, heads * dv), float("nan"), device=DEV)
        o_.gla_chunked(proj, q_off, k_off, v_off, torch.empty(rows, heads * dk, device=DEV), state, i32(starts), i32(counts),
                       i32([slots[r] for r, _ in step]), out, heads, dk, dv, 0.5, 1.0, max(counts),
                       torch.empty(rows, heads * dk, device=DEV), torch.empty(rows, heads * dk, device=DEV),
                       torch.empty(rows, heads * o_.GLA_CHUNK, device=DEV), head_decay=decay, activation=1)
        for (r, n), s in zip(step, starts):
            got[r].append(out[s:s + n].cpu())
            fed[r] += n
    o_.lightning_block_width(0)
    assert (state[2] == 3).all()
    for r, n in lengths.items():
        p = P.silu(data[r].double()).bfloat16().double()
        S = torch.zeros(heads, dk, dv, dtype=torch.float64)
        want = plain_fixed_decay(p[:, q_off:k_off].view(n, heads, dk) * 0.5, p[:, k_off:v_off].view(n, heads, dk),
                                 p[:, v_off:].view(n, heads, dv), [float(d) for d in decay.cpu()], S)
        close(torch.cat(got[r]), want.view(n, -1), torch.float32, f"outputs of {r}", loose=4)
        close(state[slots[r]], S, torch.float32, f"state of {r}", loose=4)


# ---- whole models through the step function ---------------------------------------------------------------------------

class Checker:
    """Rows against the plain implementation's float64 logits. float32: every row within the tolerance. bfloat16: nearly
    every row (see `finish`); the rms error and the share of equal choices hold over all rows."""

    def __init__(self, folder, sequences, dtype, what, slack=1.0):
        self.cfg, self.w = P.load_plain(folder)
        self.sequences, self.dtype, self.what, self.slack = sequences, dtype, what, slack
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
        tol = 2 * TOL[self.dtype] * self.scale * self.slack       # (float32: a hundred-thousandth of the largest logit)
        worst = max(self.errors)
        over = [e for e in self.errors if e[0] > tol]
        rms = (self.err2 / max(self.ref2, 1e-300)) ** 0.5
        print(f"{self.what} [{self.dtype}] rows {len(self.errors)}: largest difference {worst[0]:.3e} at {worst[1:]} "
              f"({worst[0] / self.scale:.2e} of the largest |logit|), {len(over)} rows over, rms {rms:.2e}")
        first = min(over, key=lambda e: (e[1], e[2])) if over else None
        # bfloat16: the norm behind every part divides by the part's own size, so a rounding of a small result weighs
        # as much as one of a large result; three rows in a hundred may lie beyond the tolerance, none beyond three times it
        allowed = 0 if self.dtype == "float32" else max(2, 3 * len(self.errors) // 100)
        assert len(over) <= allowed and worst[0] <= 3 * tol, \
            f"{self.what}: {len(over)} rows beyond {tol:.3e}, the first at {first}, the largest {worst}"
        assert rms <= 3 * RMS_TOL[self.dtype] and 1 - self.flips / len(self.errors) >= ARGMAX_SHARE[self.dtype] - 0.03


def run_trace(name, dtype, steps, sequences, what, **kw):
    from jllm_serve_b200.csrc import ops as o
    from jllm_serve_b200.engine import ModelRunner, Segment
    args = dict(dtype=dtype, page_size=16, max_tokens=traces.peak_tokens(steps, 16), max_batch_tokens=512, max_requests=4,
                ctx=1024, poison_freed_pages=True)
    slack = kw.pop("slack", 1.0)
    args.update(kw)
    folder = name if isinstance(name, Path) else movivik_folder(name)
    runner = ModelRunner(folder, **args)
    checker = Checker(folder, sequences, dtype, f"{name if not isinstance(name, Path) else ''} {what}", slack)
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
    return {f"r{i}": random_tokens(n, MOVIVIK[name]["vocab"], seed + i) for i, n in enumerate(lengths)}


LENGTHS = (1, 2, 37, 150, 16, 333, 65, 129)
WAYS = {
    "whole": traces.whole,
    "prompt, then token by token": lambda r: traces.prompt_then_decode(r, tail=24),
    "portions down to two tokens": traces.changing_portions,
    "all requests side by side": lambda r: traces.all_together(dict(list(r.items())[:4]), tail=6),
    "mixed, slots and pages used again": lambda r: traces.mixed(r, max_live=4, portion=40, prefill_share=0.7),
}


@pytest.mark.parametrize("way", list(WAYS))
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cut_of_the_same_requests_gives_the_plain_logits(name, dtype, way):
    seqs = sequences_for(name, LENGTHS)
    steps = WAYS[way](seqs)
    used = {e["id"] for st in steps for e in st["entries"]}
    run_trace(name, dtype, steps, {r: t for r, t in seqs.items() if r in used}, way)


@pytest.mark.parametrize("way", ["prompt, then token by token", "mixed, slots and pages used again"])
@pytest.mark.parametrize("name", ["D", "E", "F"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_of_one_kind_of_layer_only_and_of_odd_sizes(name, dtype, way):
    """Pages and no state at all; states beside pages in every layer, with borrowed weights; sizes that are multiples of
    nothing."""
    seqs = sequences_for(name, (3, 70, 1, 141, 18), seed=31)
    run_trace(name, dtype, WAYS[way](seqs), seqs, way)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_chunk_edges_and_a_page_size_that_cuts_elsewhere(dtype):
    """300 tokens one by one: the rows pass the edges of chunks of 20 and (in B) 70 and 128 positions while decoding."""
    for name in ("A", "B"):
        seqs = sequences_for(name, (420,), seed=5)
        run_trace(name, dtype, traces.prompt_then_decode(seqs, tail=300), seqs, "300 tokens one by one", page_size=8)


def test_a_state_slot_and_pages_that_are_used_again_start_clean():
    """One state slot and few pages: every request gets the slot and the pages the one before it left."""
    seqs = sequences_for("A", (90, 3, 61, 1, 40), seed=8)
    run_trace("A", "float32", traces.whole(seqs), seqs, "one slot", max_requests=1, max_tokens=96)
    run_trace("A", "float32", traces.changing_portions(seqs, sizes=(2, 9, 2, 31)), seqs, "one slot, portions", max_requests=1,
              max_tokens=96)


def test_more_rows_than_a_batch_holds_run_as_several_batches():
    seqs = sequences_for("C", (300, 77), seed=12)
    run_trace("C", "float32", traces.all_together(seqs, tail=2), seqs, "a step in parts", max_batch_tokens=64)


@pytest.mark.parametrize("seed", [7001, 7002, 7003, 7004, 7005, 7006, 7007, 7008, 7009, 7010])
def test_a_random_configuration_mixed_and_decoded(seed):
    """Configurations drawn at random: sizes, layer orders, masks and constants in combinations that the fixed test models
    do not hold; requests mixed in steps with slots and pages used again, and a tail decoded token by token."""
    import random
    from tests.movivik_cases import movivik_folder_of, random_movivik
    cfg = random_movivik(seed)
    # (the drawn score multipliers reach 1.6 / sqrt(dim): the queries are scaled up less than in the fixed models, so that
    # the bfloat16 path's rounding of q and k does not drown its comparison; float32 is exact either way)
    folder = movivik_folder_of(cfg, seed, q_gain=2.0)
    rng = random.Random(seed)
    lengths = [rng.randint(1, 30), rng.randint(40, 140), rng.randint(150, 300), rng.randint(2, 70), rng.randint(100, 200)]
    seqs = {f"r{i}": random_tokens(n, cfg["vocab"], seed + i) for i, n in enumerate(lengths)}
    shape = "; ".join(f"{l['type']}{'*' if 'weights_of' in l else ''}" for l in cfg["layers"])
    for dtype in ("float32", "bfloat16"):
        # (twice the fixed models' tolerance: a drawn model may norm a part's result that nearly cancels, which magnifies
        # the rounding of that row; a wrong key, edge or state is off by a thousand times more)
        run_trace(folder, dtype, traces.mixed(seqs, max_live=4, portion=50, prefill_share=0.7), seqs, f"seed {seed} ({shape}) mixed",
                  slack=2.0)
        run_trace(folder, dtype, traces.prompt_then_decode(seqs, tail=40), seqs, f"seed {seed} ({shape}) decoded tail", slack=2.0)


# ---- generation and the trace program -----------------------------------------------------------------------------------

def engine_for(name, dtype, **kw):
    from jllm_serve_b200.engine import Engine
    args = dict(dtype=dtype, page_size=8, max_tokens_cached=1024, max_batch_tokens=64, chunk=32, min_chunk=4, max_running=4,
                ctx=256)
    args.update(kw)
    return Engine(movivik_folder(name), **args)


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_float32_equals_plain(name):
    from jllm_serve_b200.sampling import SamplingParams
    cfg, w = P.load_plain(movivik_folder(name))
    prompts = [random_tokens(n, MOVIVIK[name]["vocab"], 40 + n) for n in (5, 17, 41, 2, 33, 9)]
    got = engine_for(name, "float32").generate(prompts, SamplingParams.greedy_params(12, ignore_eos=True))
    for p, r in zip(prompts, got):
        assert r.tokens == P.greedy_generate(cfg, w, p, 12) and r.finish_reason == "length"


def test_greedy_generation_bfloat16_follows_plain():
    from jllm_serve_b200.sampling import SamplingParams
    cfg, w = P.load_plain(movivik_folder("B"))
    prompts = [random_tokens(n, MOVIVIK["B"]["vocab"], 60 + n) for n in (9, 40, 70)]
    got = engine_for("B", "bfloat16").generate(prompts, SamplingParams.greedy_params(10, ignore_eos=True))
    for p, r in zip(prompts, got):
        logits = P.forward(cfg, w, p + r.tokens[:-1])
        for i, t in enumerate(r.tokens):
            row = logits[len(p) - 1 + i]
            assert float(row.max() - row[t]) <= 4 * TOL["bfloat16"] * float(logits.abs().max()), (i, t)


def test_generation_with_preemption_in_a_small_pool_equals_plain():
    from jllm_serve_b200.sampling import SamplingParams
    cfg, w = P.load_plain(movivik_folder("A"))
    prompts = [random_tokens(n, MOVIVIK["A"]["vocab"], 80 + n) for n in (60, 1, 33, 64, 100, 20)]
    params = SamplingParams.greedy_params(16, ignore_eos=True)
    got = engine_for("A", "float32", max_tokens_cached=200, max_batch_tokens=48).generate(prompts, params)
    for i, (p, r) in enumerate(zip(prompts, got)):
        assert r.tokens == P.greedy_generate(cfg, w, p, 16), f"request {i}"


def test_command_line_run_and_bench_on_a_movivik_model(tmp_path):
    folder = movivik_folder("D")
    prompt = random_tokens(11, MOVIVIK["D"]["vocab"], 5)
    cmd = [sys.executable, str(ROOT / "bin" / "jllm"), "run", "--model", str(folder), "--dtype", "fp32", "--temp", "0",
           "--max-tokens", "7", "--ctx", "64", "--ignore-eos", "--tokens", ",".join(map(str, prompt))]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    cfg, w = P.load_plain(folder)
    assert [int(t) for t in proc.stdout.strip().split(",")] == P.greedy_generate(cfg, w, prompt, 7)
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(MOVIVIK["B"]))
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "jllm"), "bench", "--random-weights", "3", "--model-config",
                           str(cfg_file), "--ctx", "256", "--bench.prompt-tokens", "50", "--bench.max-tokens", "8",
                           "--bench.rounds", "2"], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.startswith("prefill 50 tok in") and "decode 8 tok in" in proc.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program_on_a_movivik_folder(dtype, tmp_path):
    seqs = sequences_for("A", (50, 7, 1, 90, 33), seed=30)
    steps = traces.mixed(seqs, max_live=4, portion=24)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(movivik_folder("A")), "--dtype", dtype,
                           "--out", str(tmp_path), "--max-tokens", str(traces.peak_tokens(steps)), "--poison"],
                          input=text, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    import numpy as np
    vocab = MOVIVIK["A"]["vocab"]
    checker = Checker(movivik_folder("A"), seqs, dtype, "trace program")
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
