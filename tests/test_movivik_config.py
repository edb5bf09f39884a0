"""The Movivik parser, its tensor list, its rotary tables and the cache needs of its mixers (no GPU)."""
import copy
import math

import pytest
import torch

from jllm_serve_b200.cache.manager import FixedState, PagedKeysValues, group_runs
from jllm_serve_b200.config import ConfigError, parse_config
from jllm_serve_b200.config.registry import architecture_entry, model_type_of
from jllm_serve_b200.engine.model import model_wants
from jllm_serve_b200.parts import part_class
from jllm_serve_b200.parts.rope import amplitude, inverse_frequencies
from tests.movivik_cases import MOVIVIK, MOVIVIK_A, MOVIVIK_B, MOVIVIK_C
from tests.plain import movivik_plain as P


def test_layers_that_borrow_weights_become_runs_of_one_layer():
    spec = parse_config(MOVIVIK_A)
    assert model_type_of(MOVIVIK_A) == "Movivik" and spec.core.dim == 56 and spec.core.vocab == 150
    assert len(spec.layers) == 3 and [r.layer for r in spec.schedule] == [0, 1, 0, 2]
    assert [l.prefix for l in spec.layers] == ["l0.", "l1.", "l3."] and all(l.arrangement == "sandwich_norm" for l in spec.layers)
    att = spec.layers[0].mixer
    assert (att.heads, att.kv_heads, att.head_dim, att.v_dim, att.chunk, att.scale) == (4, 2, 24, 16, 20, 0.3)
    assert att.bias and att.gate == "head_sigmoid" and not att.unit_qk and att.qk_norm_eps == 2e-5
    table = spec.rope_tables[att.rope_table]
    assert (table.rotary_dim, table.theta, table.pairing, table.scaling.kind) == (16, 500.0, "interleaved", "yarn")
    assert table.scaling.attention_factor == pytest.approx(0.1 * math.log(3.0) + 1)
    par = spec.layers[1].mixer
    left, right = par.branches
    assert par.kind == "parallel_mixers" and par.weight == 0.5 and par.out_norms == ("left.out", "right.out")
    assert (left.heads, left.kv_heads, left.head_dim, left.v_dim, left.chunk) == (3, 3, 16, 24, 0)
    assert left.unit_qk and not left.bias and spec.rope_tables[left.rope_table].pairing == "half"
    assert spec.rope_tables[left.rope_table].scaling.kind == "none"
    assert (right.heads, right.key_dim, right.value_dim, right.decays) == (2, 12, 20, (0.7, 0.97))
    ff = spec.layers[0].feed_forward
    assert (ff.hidden, ff.activation) == (40, "gelu_tanh") and spec.layers[2].feed_forward is None


def test_the_tensor_list():
    wants = model_wants(architecture_entry("Movivik"), parse_config(MOVIVIK_A))
    shapes = {n: w.shape for n, w in wants.items()}
    assert shapes["l0.mix.q"] == (96, 56) and shapes["l0.mix.q.b"] == (96,) and shapes["l0.mix.k"] == (48, 56)
    assert shapes["l0.mix.v"] == (32, 56) and shapes["l0.mix.v.b"] == (32,) and shapes["l0.mix.g"] == (4, 56)
    assert shapes["l0.mix.o"] == (56, 64) and shapes["l0.norm1b"] == (56,) and shapes["l0.norm2b"] == (56,)
    assert shapes["l1.mix.left.q"] == (48, 56) and shapes["l1.mix.left.v"] == (72, 56) and shapes["l1.mix.left.g"] == (3, 56)
    assert "l1.mix.left.q.b" not in shapes and shapes["l1.mix.left.o"] == (56, 72)
    assert shapes["l1.mix.right.q"] == (24, 56) and shapes["l1.mix.right.v"] == (40, 56) and shapes["l1.mix.right.g"] == (40, 56)
    assert shapes["l1.mix.right.norm"] == (40,) and shapes["l1.mix.right.o"] == (56, 40)
    assert shapes["l1.mix.left.out"] == (56,) and shapes["l1.mix.right.out"] == (56,)
    assert shapes["l1.mlp.gate"] == (24, 56) and shapes["l1.mlp.down"] == (56, 24)
    assert "l2.norm1" not in shapes and "l3.norm2" not in shapes and "l3.norm2b" not in shapes and "l3.mlp.up" not in shapes
    assert shapes["final.norm"] == (56,) and shapes["head"] == (150, 56) and shapes["embed"] == (150, 56)


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="mamba"), "unknown layer type"),
    (lambda c: c["layers"][2].update(weights_of=9), "names no layer"),
    (lambda c: c["layers"][2].update(weights_of=1), "differs from that of the layer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "unknown feed-forward kind"),
    (lambda c: c.pop("width"), "'width' is missing"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "'vdim' is missing"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "exceeds the head's dim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "must be positive and divide"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "1 decays for 2 heads"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5, 1.5]), "must lie in [0, 1]"),
    (lambda c: c["layers"][1]["mixer"].pop("left"), "needs 'left' and 'right'"),
])
def test_what_the_parser_refuses(change, text):
    cfg = copy.deepcopy(MOVIVIK_A)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        parse_config(cfg)
    assert text in str(e.value)


def test_mixers_with_the_same_rotation_share_a_table_and_others_do_not():
    assert len(parse_config(MOVIVIK_A).rope_tables) == 3
    cfg = copy.deepcopy(MOVIVIK_B)
    cfg["layers"].append(copy.deepcopy(cfg["layers"][0]))
    assert len(parse_config(cfg).rope_tables) == 3          # the fourth layer rotates like the first
    cfg["layers"][3]["mixer"]["rot"]["base"] = 9999.0
    assert len(parse_config(cfg).rope_tables) == 4


@pytest.mark.parametrize("name", list(MOVIVIK))
def test_the_tables_frequencies_are_the_plain_formulas(name):
    """YaRN's blend and the amplitude of cos and sin, for every rotation of every test model, and a ramp of no width."""
    spec = parse_config(MOVIVIK[name])
    rots = []
    for layer in MOVIVIK[name]["layers"]:
        m = layer["mixer"]
        rots += [m["rot"]] if layer["type"] == "attention" else [m["left"]["rot"]]
    rots.append({"base": 10000.0, "dims": 8, "scaling": {"factor": 2.0, "original": 100000, "fast": 1.0, "slow": 1.0}})
    from jllm_serve_b200.config.movivik import _rope
    from jllm_serve_b200.config.reader import ConfigReader
    for rot in rots:
        table = _rope(ConfigReader(rot), "half")
        want, amp = P.rotary_frequencies(rot)
        got = inverse_frequencies(table, 4096)
        assert torch.allclose(got, torch.tensor(want, dtype=torch.float64), rtol=1e-13, atol=0)
        assert amplitude(table.scaling) == pytest.approx(amp, rel=1e-15)
    assert spec.rope_tables


def test_cache_needs_pages_as_wide_as_the_wider_head_and_a_state_beside_them():
    for name, cfg in MOVIVIK.items():
        spec = parse_config(cfg)
        needs = [part_class("mixer", spec.layers[r.layer].mixer.kind).cache_need(spec.layers[r.layer].mixer) for r in spec.schedule]
        paged, fixed, paged_of_run, fixed_of_run = group_runs(needs)
        for i, r in enumerate(spec.schedule):
            m = spec.layers[r.layer].mixer
            if m.kind == "gqa_attention":
                assert needs[i] == PagedKeysValues(m.kv_heads, max(m.head_dim, m.v_dim), -m.chunk) and i not in fixed_of_run
            else:
                a, l = m.branches
                assert needs[i] == (PagedKeysValues(a.kv_heads, max(a.head_dim, a.v_dim), -a.chunk),
                                    FixedState((l.heads, l.key_dim, l.value_dim), "float32"))
                assert i in paged_of_run and len(fixed_of_run[i]) == 1
    spec = parse_config(MOVIVIK_A)      # the two runs of the borrowed attention layer share a group (one block table)
    needs = [part_class("mixer", spec.layers[r.layer].mixer.kind).cache_need(spec.layers[r.layer].mixer) for r in spec.schedule]
    paged, fixed, _, _ = group_runs(needs)
    assert [g.runs for g in paged] == [[0, 2], [1], [3]] and [g.runs for g in fixed] == [[1], [3]]


def test_pages_of_chunks_that_have_passed_are_given_back():
    """A group under a chunk mask of 20 positions with pages of 8: once a request's next position lies in a new chunk, the
    pages that hold only earlier chunks go back to the pool (entries -1), like pages that a window has passed; a rewind
    behind them is refused."""
    from jllm_serve_b200.cache import CacheManager
    m = CacheManager([PagedKeysValues(1, 16, -20), PagedKeysValues(1, 16, 0)], 8, 12, 2)
    m.open("a")
    m.reserve("a", 0, 19)
    assert m.commit("a", 19) == [] and m.table("a", 0).count(-1) == 0          # still inside the first chunk
    m.reserve("a", 19, 1)
    released = m.commit("a", 20)                                               # the next row opens the chunk [20, 40)
    assert [g for g, _ in released] == [0, 0] and m.table("a", 0)[:2] == [-1, -1] and m.table("a", 0)[2] >= 0
    assert m.table("a", 1).count(-1) == 0                                      # the group without a mask keeps everything
    m.reserve("a", 20, 45)
    released = m.commit("a", 65)                                               # chunk [60, 80): pages below 56 go
    assert m.table("a", 0)[:7] == [-1] * 7 and m.table("a", 0)[7] >= 0 and len(released) == 5
    with pytest.raises(ValueError):
        m.truncate("a", 30)
    m.check()
    m.close("a")
    assert m.free_pages() == [12, 12]


def test_the_first_key_a_row_sees():
    """The rule every attention kernel shares (jllm_first_key in common.cuh), restated: 0, a window, or the row's chunk."""
    def first(p, span):
        return max(0, p + 1 - span) if span > 0 else (p - p % (-span) if span < 0 else 0)
    assert [first(p, -20) for p in (0, 19, 20, 21, 39, 40)] == [0, 0, 20, 20, 20, 40]
    assert [first(p, 20) for p in (0, 19, 20, 21)] == [0, 0, 1, 2] and first(1000, 0) == 0
    from jllm_serve_b200.csrc.ops import _windowed_bucket
    assert _windowed_bucket(32, -512) == 2 and _windowed_bucket(32, 512) == 2 and _windowed_bucket(5, 0) == 5
    assert _windowed_bucket(32, -70) == 1


def test_kernel_choice_numbers_of_the_gate_activations():
    from jllm_serve_b200.csrc.ops import glu_kind
    assert [glu_kind(a) for a in (False, True, "silu", "gelu_tanh", None, 2)] == [0, 1, 1, 2, 0, 2]
