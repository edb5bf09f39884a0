"""The Madevik parser: config.json of `architecture: Madevik` -> a `Decoder` spec.

Madevik lists its layers one by one (`layers`: `type`, `mixer`, `mlp`, optionally `weights_of`). A layer is a token
mixer (`gla`: gated linear attention with a recurrent state; `latent_attention`: softmax attention over one cached
latent row per position), optionally a routed mixture of small gated feed-forwards, a Dynamic-Tanh norm in front of
each, and a residual sum scaled by `residual_mult`. A layer with `weights_of: j` runs layer j's tensors with a cache or
state of its own: in the spec that is one `LayerSpec` (j's) named by two entries of `Decoder.schedule`. There are no
positions in the model (nothing rotates, nothing is added to the embedding), so the context is bounded by the cache
pool alone; `max_positions` is the engine's default table size.

Keys read: `width`, `vocab`, `residual_mult`, `norm.eps`, `layers[i].type | mixer | mlp | weights_of`; of a `gla` mixer
`heads`, `dim`, `vdim`, `tau` (the width of its low-rank decay projection is the tensor's own: `decay_rank` may name it
for a model that is made from a configuration alone); of a `latent_attention` mixer `heads`, `dim`, `vdim`, `kv_rank`,
`scale`; of an `mlp` `kind` (moe), `expert.ff`, `router.experts | top | scale`.
"""
from __future__ import annotations

from .reader import ConfigReader
from .specs import (ConfigError, Core, Decoder, GatedLinearAttentionSpec, LatentAttentionSpec, LayerNames, LayerRun,
                    LayerSpec, ModelNames, NormSpec, RoutedExpertsSpec)

MADEVIK_NAMES = ModelNames(embedding="embed", layer="l{}.", final_norm="final.norm", head="head")
MADEVIK_LAYER_NAMES = LayerNames(mixer="mix.", feed_forward="mlp.", mixer_norm="norm1", feed_forward_norm="norm2")
DEFAULT_POSITIONS = 1 << 17


def _mixer(kind: str, m: ConfigReader, eps: float):
    if kind == "gla":
        key_dim = m.positive("dim")
        return GatedLinearAttentionSpec(heads=m.positive("heads"), key_dim=key_dim, value_dim=m.positive("vdim"),
                                        decay_rank=m.integer("decay_rank", -1), decay_temperature=m.number("tau"),
                                        norm_eps=eps, query_scale=float(key_dim) ** -0.5)
    if kind == "latent_attention":
        return LatentAttentionSpec(heads=m.positive("heads"), key_dim=m.positive("dim"), value_dim=m.positive("vdim"),
                                   rank=m.positive("kv_rank"), scale=m.number("scale"), norm_eps=eps, gated=True)
    raise ConfigError(f"{m.where}: unknown layer type {kind!r} (built: gla, latent_attention)")


def _feed_forward(f: ConfigReader | None):
    if f is None:
        return None
    kind = f.string("kind", "moe")
    if kind != "moe":
        raise ConfigError(f"{f.where}: unknown feed-forward kind {kind!r} (built: moe)")
    expert, router = f.mapping("expert"), f.mapping("router")
    if expert is None or router is None:
        raise ConfigError(f"{f.where}: a mixture of experts needs 'expert' and 'router'")
    return RoutedExpertsSpec(experts=router.positive("experts"), top=router.positive("top"), hidden=expert.positive("ff"),
                             scale=router.number("scale", 1.0), correction=True, normalize=True)


def parse_madevik(values: dict) -> Decoder:
    c = ConfigReader(values)
    dim, vocab = c.positive("width"), c.positive("vocab")
    norm = c.mapping("norm")
    eps = norm.number("eps", 1e-6) if norm is not None else 1e-6
    scale = c.number("residual_mult", 1.0)
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

    norm_spec = NormSpec("dynamic_tanh", eps)
    specs, index_of, schedule = [], {}, []
    for i, r in enumerate(readers):
        o = owner(i)
        if o not in index_of:
            ro = readers[o]
            m = ro.mapping("mixer")
            if m is None:
                raise ConfigError(f"{ro.where}: required key 'mixer' is missing")
            index_of[o] = len(specs)
            specs.append(LayerSpec(_mixer(ro.string("type"), m, eps), _feed_forward(ro.mapping("mlp")), norm_spec,
                                   "pre_norm", MADEVIK_LAYER_NAMES, residual_scale=scale,
                                   prefix=MADEVIK_NAMES.layer.format(o)))
        if r.string("type") != readers[o].string("type"):
            raise ConfigError(f"{r.where}: type {r.string('type')!r} differs from that of the layer whose weights it uses")
        schedule.append(LayerRun(index_of[o]))
    kinds = [s.mixer.kind for s in specs]
    description = (f"Madevik width={dim} vocab={vocab} runs={len(schedule)} layers={len(specs)} "
                   f"(gla {kinds.count('gated_linear_attention')}, latent {kinds.count('latent_attention')}) "
                   f"residual_mult={scale:g}")
    core = Core(architecture="Madevik", model_type="Madevik", dim=dim, layers=len(specs), vocab=vocab, norm_eps=eps,
                tied=False, bos=-1, eos=c.int_list("eos"), max_positions=c.positive("max_positions", DEFAULT_POSITIONS),
                description=description)
    return Decoder(core, tuple(specs), (), norm_spec, tuple(schedule), MADEVIK_NAMES)
