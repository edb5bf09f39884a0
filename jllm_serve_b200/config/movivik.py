"""The Movivik parser: config.json of `architecture: Movivik` -> a `Decoder` spec.

Movivik lists its layers one by one (`layers`: `type`, `mixer`, `mlp`, optionally `weights_of`). A layer is a token
mixer and a dense gated feed-forward (tanh-form GELU; `mlp: null` = none), each with an RMS norm in front AND one behind,
before the residual sum: the `sandwich_norm` arrangement. A layer with `weights_of: j` runs layer j's tensors with a
cache or state of its own: one `LayerSpec` (j's) named by two entries of `Decoder.schedule`. The mixers:

* `attention`: grouped-query softmax attention with biases on q, k and v, rotary positions on interleaved pairs (2i,
  2i + 1) of the first `rot.dims` values of a head with YaRN-stretched frequencies (`rot.scaling`: factor, original,
  fast, slow; cos and sin times 0.1 ln(factor) + 1), key heads of `dim` and value heads of `vdim` values, the score
  multiplier `scale`, a chunk mask (`mask.size`: a position p sees only the earlier positions of its own chunk, p //
  size) and a sigmoid gate per head.
* `parallel`: two mixers on the same input. `left`: the same attention without biases, rotating pairs (i, i + dims / 2),
  dividing q and k by their root mean square behind the rotation, fully causal (a `mask` or a `rot.scaling`, if one is
  given, is honoured as above). `right`: linear attention with one fixed `decay` per head, silu on q, k and v, one RMS norm
  over all heads and a sigmoid gate. The mixer's result is the mean of the two branches' results, each after an RMS norm
  of its own (with a gain) over the model width.

Keys read: `width`, `vocab`, `norm.eps`, `layers[i].type | mixer | mlp | weights_of`; of an attention `heads`, `kv_heads`,
`dim`, `vdim`, `scale`, `rot.base | dims | scaling`, `mask.size`; of the linear attention `heads`, `dim`, `vdim`, `decay`;
of an `mlp` `kind` (dense) and `ff`. Optional: `eos`, `max_positions` (the rotary tables' length; the engine's context).
"""
from __future__ import annotations

import math

from .reader import ConfigReader
from .specs import (AttentionNames, ConfigError, Core, Decoder, DenseGluSpec, FixedDecayLinearAttentionSpec,
                    GqaAttentionSpec, LayerNames, LayerRun, LayerSpec, ModelNames, NormSpec, ParallelMixersSpec, RopeScaling,
                    RopeTableSpec)

MOVIVIK_NAMES = ModelNames(embedding="embed", layer="l{}.", final_norm="final.norm", head="head")
MOVIVIK_LAYER_NAMES = LayerNames(mixer="mix.", feed_forward="mlp.", mixer_norm="norm1", feed_forward_norm="norm2",
                                 mixer_post_norm="norm1b", feed_forward_post_norm="norm2b")
MOVIVIK_ATTENTION_NAMES = AttentionNames(q="q", k="k", v="v", o="o", q_bias="q.b", k_bias="k.b", v_bias="v.b", o_bias="o.b",
                                         q_norm="q.norm", k_norm="k.norm", gate="g")
DEFAULT_POSITIONS = 1 << 17


class _Tables:
    """The model's rotary tables: mixers with the same rotation share one."""

    def __init__(self):
        self.specs = []

    def index(self, spec: RopeTableSpec) -> int:
        if spec not in self.specs:
            self.specs.append(spec)
        return self.specs.index(spec)


def _rope(rot: ConfigReader, pairing: str) -> RopeTableSpec:
    scaling = RopeScaling()
    sc = rot.mapping("scaling")
    if sc is not None:
        factor = sc.number("factor")
        if not factor > 0:
            raise ConfigError(f"{sc.where}: 'factor' must be positive, got {factor}")
        scaling = RopeScaling(kind="yarn", factor=factor, original_max_positions=sc.positive("original"),
                              beta_fast=sc.number("fast"), beta_slow=sc.number("slow"),
                              attention_factor=0.1 * math.log(factor) + 1.0, truncate=True)
    return RopeTableSpec(rotary_dim=rot.positive("dims"), theta=rot.number("base"), scaling=scaling, pairing=pairing)


def _attention(m: ConfigReader, eps: float, tables: _Tables, *, bias: bool, pairing: str, unit_qk: bool) -> GqaAttentionSpec:
    rot, mask = m.mapping("rot"), m.mapping("mask")
    dim = m.positive("dim")
    if rot is not None and rot.positive("dims") > dim:
        raise ConfigError(f"{rot.where}: dims={rot.positive('dims')} exceeds the head's dim={dim}")
    return GqaAttentionSpec(heads=m.positive("heads"), kv_heads=m.positive("kv_heads"), head_dim=dim,
                            value_dim=m.positive("vdim"), rope_table=tables.index(_rope(rot, pairing)) if rot is not None else -1,
                            qk_norm=False, qk_norm_eps=eps, bias=bias, scale=m.number("scale"),
                            chunk=mask.positive("size") if mask is not None else 0, unit_qk=unit_qk, gate="head_sigmoid",
                            names=MOVIVIK_ATTENTION_NAMES)


def _linear(m: ConfigReader, eps: float) -> FixedDecayLinearAttentionSpec:
    decay = m.values.get("decay")
    if not isinstance(decay, list) or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
        raise ConfigError(f"{m.where}: 'decay' must be a list of numbers, one per head")
    return FixedDecayLinearAttentionSpec(heads=m.positive("heads"), key_dim=m.positive("dim"), value_dim=m.positive("vdim"),
                                         decays=tuple(float(d) for d in decay), activation="silu", query_scale=1.0,
                                         norm_eps=eps, norm_over="all", gate="sigmoid")


def _mixer(kind: str, m: ConfigReader, eps: float, tables: _Tables):
    if kind == "attention":
        return _attention(m, eps, tables, bias=True, pairing="interleaved", unit_qk=False)
    if kind == "parallel":
        left, right = m.mapping("left"), m.mapping("right")
        if left is None or right is None:
            raise ConfigError(f"{m.where}: a parallel mixer needs 'left' and 'right'")
        return ParallelMixersSpec(branches=(_attention(left, eps, tables, bias=False, pairing="half", unit_qk=True),
                                            _linear(right, eps)),
                                  prefixes=("left.", "right."), out_norms=("left.out", "right.out"), norm_eps=eps, weight=0.5)
    raise ConfigError(f"{m.where}: unknown layer type {kind!r} (built: attention, parallel)")


def _feed_forward(f: ConfigReader | None):
    if f is None:
        return None
    kind = f.string("kind", "dense")
    if kind != "dense":
        raise ConfigError(f"{f.where}: unknown feed-forward kind {kind!r} (built: dense)")
    return DenseGluSpec(hidden=f.positive("ff"), activation="gelu_tanh", names=("gate", "up", "down"))


def parse_movivik(values: dict) -> Decoder:
    c = ConfigReader(values)
    dim, vocab = c.positive("width"), c.positive("vocab")
    norm = c.mapping("norm")
    eps = norm.number("eps", 1e-6) if norm is not None else 1e-6
    entries = values.get("layers")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config.json: 'layers' must be a list with at least one layer")
    readers = [ConfigReader(e, f"config.json:layers[{i}]") for i, e in enumerate(entries)]

    def owner(i: int) -> int:
        seen = set()
        while readers[i].has("weights_of"):
            if i in seen:
                raise ConfigError(f"config.json:layers[{i}]: 'weights_of' runs in a circle")
            seen.add(i)
            j = readers[i].integer("weights_of")
            if not 0 <= j < len(readers):
                raise ConfigError(f"config.json:layers[{i}]: weights_of={j} names no layer")
            i = j
        return i

    norm_spec = NormSpec("rmsnorm", eps, gain_name="")
    tables = _Tables()
    specs, index_of, schedule = [], {}, []
    for i, r in enumerate(readers):
        o = owner(i)
        if o not in index_of:
            ro = readers[o]
            m = ro.mapping("mixer")
            if m is None:
                raise ConfigError(f"{ro.where}: required key 'mixer' is missing")
            index_of[o] = len(specs)
            specs.append(LayerSpec(_mixer(ro.string("type"), m, eps, tables), _feed_forward(ro.mapping("mlp")), norm_spec,
                                   "sandwich_norm", MOVIVIK_LAYER_NAMES, prefix=MOVIVIK_NAMES.layer.format(o)))
        if r.string("type") != readers[o].string("type"):
            raise ConfigError(f"{r.where}: type {r.string('type')!r} differs from that of the layer whose weights it uses")
        schedule.append(LayerRun(index_of[o]))
    kinds = [s.mixer.kind for s in specs]
    description = (f"Movivik width={dim} vocab={vocab} runs={len(schedule)} layers={len(specs)} "
                   f"(attention {kinds.count('gqa_attention')}, parallel {kinds.count('parallel_mixers')})")
    core = Core(architecture="Movivik", model_type="Movivik", dim=dim, layers=len(specs), vocab=vocab, norm_eps=eps,
                tied=False, bos=-1, eos=c.int_list("eos"), max_positions=c.positive("max_positions", DEFAULT_POSITIONS),
                description=description)
    return Decoder(core, tuple(specs), tuple(tables.specs), norm_spec, tuple(schedule), MOVIVIK_NAMES)
