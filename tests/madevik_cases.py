"""Tiny Madevik configurations and model folders for the tests: every size differs between them, and several values
that one model may happen to make equal or 1 (heads, top = experts, top = 1, key and value widths, tau, the residual
scale, a layer without a feed-forward) are taken apart."""
from __future__ import annotations

import functools
import json
import tempfile
from pathlib import Path

import torch


def _moe(experts, top, ff, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


def _gla(heads, dim, vdim, tau, rank, mlp, **more):
    return dict({"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank},
                 "mlp": mlp}, **more)


def _latent(heads, dim, vdim, rank, scale, mlp, **more):
    return dict({"type": "latent_attention",
                 "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}, "mlp": mlp}, **more)


# P: both mixers, each run twice (the second time with the first's tensors and a cache of its own)
MADEVIK_P = {"architecture": "Madevik", "width": 64, "vocab": 211, "residual_mult": 0.6, "norm": {"eps": 2e-5}, "layers": [
    _gla(2, 16, 24, 8.0, 8, _moe(4, 2, 24, 1.5)),
    _latent(3, 16, 20, 64, 0.25, _moe(4, 2, 24, 1.5)),
    _gla(2, 16, 24, 8.0, 8, _moe(4, 2, 24, 1.5), weights_of=0),
    _latent(3, 16, 20, 64, 0.25, _moe(4, 2, 24, 1.5), weights_of=1)]}
# Q: sizes that are no multiples of 8 or 16, one head, tau 1, no residual scale, a layer without a feed-forward, all
# experts used (top = experts) and one expert used (top = 1); the latent layer comes first
MADEVIK_Q = {"architecture": "Madevik", "width": 72, "vocab": 130, "residual_mult": 1.0, "norm": {"eps": 3e-6}, "layers": [
    _latent(1, 8, 8, 40, 0.3, None),
    _gla(1, 20, 12, 1.0, 5, _moe(3, 3, 10, 1.0)),
    _gla(5, 8, 40, 3.0, 16, _moe(5, 1, 16, 0.7))]}
# R: a latent of 128 values and more than 16 heads (the widths the tensor-core attention kernels take, and a group
# the staged decode kernel does not), key widths of 64 and 96 in the linear attention, value width 33
MADEVIK_R = {"architecture": "Madevik", "width": 128, "vocab": 300, "residual_mult": 0.25, "norm": {"eps": 1e-6}, "layers": [
    _latent(20, 16, 16, 128, 0.2, _moe(6, 3, 32, 2.5)),
    _gla(2, 64, 64, 12.0, 16, _moe(6, 3, 32, 2.5)),
    _gla(1, 96, 33, 4.0, 24, None),
    _latent(4, 24, 40, 128, 0.15, _moe(6, 3, 32, 2.5))]}

# S: linear attention only (no paged group at all: the model keeps states and nothing else), borrowed weights in a row
MADEVIK_S = {"architecture": "Madevik", "width": 56, "vocab": 97, "residual_mult": 1.25, "norm": {"eps": 1e-6}, "layers": [
    _gla(3, 12, 20, 4.0, 6, _moe(3, 2, 12, 1.0)),
    _gla(3, 12, 20, 4.0, 6, _moe(3, 2, 12, 1.0), weights_of=0),
    _gla(3, 12, 20, 4.0, 6, _moe(3, 2, 12, 1.0), weights_of=1)]}
# T: latent attention only, three latents of different widths (three paged groups): 256 (the mma.sync flash kernel), 96
# (the decode kernel's plain-load path, no flash kernel) and 520 (only the plain attention takes it)
MADEVIK_T = {"architecture": "Madevik", "width": 96, "vocab": 150, "residual_mult": 0.8, "norm": {"eps": 1e-5}, "layers": [
    _latent(3, 24, 16, 256, 0.2, None),
    _latent(2, 16, 24, 96, 0.25, _moe(3, 2, 20, 1.2)),
    _latent(17, 8, 8, 520, 0.35, None)]}

MADEVIK = {"P": MADEVIK_P, "Q": MADEVIK_Q, "R": MADEVIK_R, "S": MADEVIK_S, "T": MADEVIK_T}


def sharpen(tensors: dict, config: dict) -> dict:
    """Random weights of N(0, 0.02) leave every activation tiny: every attention nearly uniform, every decay nearly the
    same, the mixers a rounding error beside the embedding; a lost key or a stale state would not show. Here every
    matrix is rescaled so that unit inputs give unit outputs (N(0, 1 / fan-in)) and the embedding to N(0, 1); queries are
    scaled up further so that single keys stand out among hundreds, the decay's bias is spread so that some channels
    remember for hundreds of tokens and others forget at once, and the router's corrections are large enough to change
    the choice."""
    out = dict(tensors)
    g = torch.Generator().manual_seed(5)
    for name, t in tensors.items():
        if name == "embed":
            out[name] = (t.float() * 50.0).to(t.dtype)
        elif t.dim() == 2:
            gain = 3.0 if name.endswith("mix.q") else 1.0
            out[name] = (t.float() * (gain / (0.02 * t.shape[1] ** 0.5))).to(t.dtype)
        elif name.endswith("mix.a2.b"):
            out[name] = (torch.randn(t.shape, generator=g) * 4.0 + 2.0).to(t.dtype)
        elif name.endswith("mlp.correction"):
            out[name] = (torch.randn(t.shape, generator=g) * 0.3).to(t.dtype)
        elif name.endswith(".b"):
            out[name] = (t.float() * 10.0).to(t.dtype)
    return out


@functools.lru_cache(maxsize=None)
def madevik_folder(name: str, seed: int = 3, sharp: bool = True) -> Path:
    """A temporary model folder with random (and, by default, sharpened) weights; never inside the repository."""
    from jllm_serve_b200.config import parse_config
    from jllm_serve_b200.config.registry import architecture_entry, model_type_of
    from jllm_serve_b200.engine.model import model_wants
    from jllm_serve_b200.weights import random_tensors, write_safetensors
    config = MADEVIK[name]
    wants = model_wants(architecture_entry(model_type_of(config)), parse_config(config))
    tensors = random_tensors(wants, seed, "cpu", torch.bfloat16)
    if sharp:
        tensors = sharpen(tensors, config)
    d = Path(tempfile.mkdtemp(prefix="jllm_madevik_"))
    stored = {k: v for k, v in config.items()}
    stored["layers"] = [{k: ({kk: vv for kk, vv in v.items() if kk != "decay_rank"} if k == "mixer" else v)
                         for k, v in layer.items()} for layer in config["layers"]]    # the rank is the tensor's own
    (d / "config.json").write_text(json.dumps(stored, indent=1))
    write_safetensors(d / "model.safetensors", tensors, {"format": "pt"})
    return d
