"""The Madevik parser, its tensor list and the cache needs of its mixers (no GPU)."""
import copy

import pytest

from jllm_serve_b200.cache.manager import FixedState, PagedKeysValues, group_runs
from jllm_serve_b200.config import ConfigError, parse_config
from jllm_serve_b200.config.registry import architecture_entry, model_type_of
from jllm_serve_b200.engine.model import model_wants
from jllm_serve_b200.parts import part_class
from jllm_serve_b200.weights.loader import WeightError, compare, shape_fits
from tests.madevik_cases import MADEVIK, MADEVIK_P, MADEVIK_Q


def test_layers_that_borrow_weights_become_runs_of_one_layer():
    spec = parse_config(MADEVIK_P)
    assert model_type_of(MADEVIK_P) == "Madevik" and spec.core.dim == 64 and spec.core.vocab == 211
    assert len(spec.layers) == 2 and [r.layer for r in spec.schedule] == [0, 1, 0, 1]
    assert [l.prefix for l in spec.layers] == ["l0.", "l1."] and all(l.residual_scale == 0.6 for l in spec.layers)
    gla, latent = spec.layers[0].mixer, spec.layers[1].mixer
    assert (gla.heads, gla.key_dim, gla.value_dim, gla.decay_temperature, gla.decay_rank) == (2, 16, 24, 8.0, 8)
    assert gla.query_scale == 0.25 and gla.norm_eps == 2e-5
    assert (latent.heads, latent.key_dim, latent.value_dim, latent.rank, latent.scale) == (3, 16, 20, 64, 0.25)
    ff = spec.layers[0].feed_forward
    assert (ff.experts, ff.top, ff.hidden, ff.scale) == (4, 2, 24, 1.5) and spec.layers[0].norm.kind == "dynamic_tanh"


def test_a_borrowing_layer_that_sits_between_owners_keeps_the_owners_prefixes():
    cfg = copy.deepcopy(MADEVIK_Q)
    cfg["layers"].insert(1, dict(copy.deepcopy(cfg["layers"][0]), weights_of=0))
    spec = parse_config(cfg)
    assert [r.layer for r in spec.schedule] == [0, 0, 1, 2] and [l.prefix for l in spec.layers] == ["l0.", "l2.", "l3."]
    assert spec.layers[0].feed_forward is None
    wants = model_wants(architecture_entry("Madevik"), spec)
    assert "l0.norm1.alpha" in wants and "l0.norm2" not in wants and "l2.norm2.b" in wants and "l1.mix.q" not in wants
    assert wants["l2.mlp.router"].role == "matrix_fp32" and wants["l2.mlp.e2.down"].shape == (72, 10)
    assert wants["final.norm.alpha"].shape == () and wants["head"].shape == (130, 72) and wants["embed"].shape == (130, 72)


def test_the_decay_projections_width_is_the_checkpoints_own_when_the_config_leaves_it_out():
    cfg = copy.deepcopy(MADEVIK_P)
    for layer in cfg["layers"]:
        layer["mixer"].pop("decay_rank", None)
    wants = model_wants(architecture_entry("Madevik"), parse_config(cfg))
    assert wants["l0.mix.a1"].shape == (-1, 64) and wants["l0.mix.a2"].shape == (32, -1)
    assert shape_fits((16, 64), (-1, 64)) and not shape_fits((16, 63), (-1, 64)) and not shape_fits((16,), (-1, 64))
    meta = {n: ("bf16", tuple(7 if s == -1 else s for s in w.shape)) for n, w in wants.items()}
    assert compare(meta, wants, "here") == []
    meta["l0.mix.q"] = ("bf16", (31, 64))
    with pytest.raises(WeightError) as e:
        compare(meta, wants, "here")
    assert e.value.wrong_shape[0][0] == "l0.mix.q"


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="mamba"), "unknown layer type"),
    (lambda c: c["layers"][2].update(weights_of=9), "names no layer"),
    (lambda c: c["layers"][2].update(weights_of=1), "differs from that of the layer"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top=5"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown feed-forward kind"),
    (lambda c: c.pop("width"), "'width' is missing"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "'kv_rank' is missing"),
])
def test_what_the_parser_refuses(change, text):
    cfg = copy.deepcopy(MADEVIK_P)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        parse_config(cfg)
    assert text in str(e.value)


def test_cache_needs_a_state_per_linear_run_and_one_plane_of_latent_rows():
    for name, cfg in MADEVIK.items():
        spec = parse_config(cfg)
        needs = [part_class("mixer", spec.layers[r.layer].mixer.kind).cache_need(spec.layers[r.layer].mixer) for r in spec.schedule]
        paged, fixed, paged_of_run, fixed_of_run = group_runs(needs)
        for i, r in enumerate(spec.schedule):
            m = spec.layers[r.layer].mixer
            if m.kind == "latent_attention":
                assert needs[i] == PagedKeysValues(1, m.rank, 0, planes=1) and i in paged_of_run and i not in fixed_of_run
            else:
                assert needs[i] == FixedState((m.heads, m.key_dim, m.value_dim), "float32") and i in fixed_of_run
    spec = parse_config(MADEVIK_P)      # the two latent runs share a group (one block table), the two states one storage
    needs = [part_class("mixer", spec.layers[r.layer].mixer.kind).cache_need(spec.layers[r.layer].mixer) for r in spec.schedule]
    paged, fixed, _, _ = group_runs(needs)
    assert [g.runs for g in paged] == [[1, 3]] and [g.runs for g in fixed] == [[0, 2]]


def test_a_page_of_one_plane_is_half_a_page_of_keys_and_values():
    from jllm_serve_b200.cache import CacheManager
    two = CacheManager.page_bytes([PagedKeysValues(1, 64)], 16, 2)
    one = CacheManager.page_bytes([PagedKeysValues(1, 64, planes=1)], 16, 2)
    assert two == [2 * one[0]] and one == [16 * 64 * 2]
    seen = []
    CacheManager([PagedKeysValues(1, 64, planes=1), FixedState((2, 4, 4))], 16, 8, 4,
                 allocate=lambda shape, kind: seen.append((shape, kind)))
    assert seen == [((1, 1, 8, 1, 16, 64), "kv"), ((1, 4, 2, 4, 4), "float32")]
