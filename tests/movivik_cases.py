"""Tiny Movivik configurations and model folders for the tests: every size differs between them, and values that one
model may happen to make equal or 1 (key and value widths, heads and kv heads, rotated and whole head widths, a chunk size
that is a multiple of the page size or of a kernel's tile, a layer without a feed-forward, scaling on one mixer only) are
taken apart."""
from __future__ import annotations

import functools
import json
import tempfile
from pathlib import Path

import torch


def _rot(dims, base=10000.0, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return rot


def _att(heads, kv_heads, dim, vdim, scale, rot, chunk=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if chunk:
        m["mask"] = {"size": chunk}
    return m


def _lin(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _attention(mixer, ff, **more):
    return dict({"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}, **more)


def _parallel(left, right, ff, **more):
    return dict({"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": {"kind": "dense", "ff": ff} if ff else None},
                **more)


# A: small sizes that are no multiples of 16, key heads wider than value heads in one mixer and narrower in the other,
# part of a head rotated, a chunk of 20 positions (no multiple of the page size), borrowed weights, a layer without a
# feed-forward; only the plain attention kernel takes these heads
_A_ATT = _att(4, 2, 24, 16, 0.3, _rot(16, 500.0, (3.0, 32, 4.0, 1.0)), chunk=20)
_A_PAR = (_att(3, 3, 16, 24, 0.35, _rot(8, 100.0)), _lin(2, 12, 20, (0.7, 0.97)))
MOVIVIK_A = {"architecture": "Movivik", "width": 56, "vocab": 150, "norm": {"eps": 2e-5}, "layers": [
    _attention(_A_ATT, 40),
    _parallel(*_A_PAR, 24),
    _attention(_A_ATT, 40, weights_of=0),
    _parallel(_att(2, 1, 20, 20, 0.25, _rot(20, 1000.0)), _lin(3, 8, 8, (0.5, 0.9, 0.999)), None)]}
# B: the widths the tile kernels take. Attention with heads of 128 (tcgen05 prompt kernel, staged decode kernel) under a
# chunk of 70 positions, whose edges fall inside pages and tiles; the parallel layer's attention with heads of 64
# (mma.sync prompt kernel) rotated over their whole width; linear attention with 64 x 64 states
MOVIVIK_B = {"architecture": "Movivik", "width": 128, "vocab": 300, "norm": {"eps": 1e-6}, "layers": [
    _attention(_att(4, 2, 128, 128, 0.09, _rot(128, 10000.0, (4.0, 64, 16.0, 2.0)), chunk=70), 96),
    _parallel(_att(4, 1, 64, 64, 0.12, _rot(64, 10000.0)), _lin(2, 64, 64, (0.8, 0.99)), 64),
    _attention(_att(2, 2, 64, 64, 0.12, _rot(32, 300.0, (2.0, 40, 8.0, 1.0)), chunk=128), 64)]}
# C: what the two mixers leave open is used the other way round: the attention layer fully causal and without scaling, as
# many kv heads as heads; the parallel layer's attention with a chunk mask and YaRN scaling, 20 query heads to a kv head
# (more than the decode kernel shares a key among), heads of 256; a linear attention of one head; decays of 0 and 1
MOVIVIK_C = {"architecture": "Movivik", "width": 72, "vocab": 97, "norm": {"eps": 1e-5}, "layers": [
    _parallel(_att(20, 1, 16, 16, 0.25, _rot(16, 50.0, (8.0, 16, 2.0, 0.5)), chunk=33), _lin(1, 40, 12, (0.93,)), 30),
    _attention(_att(3, 3, 32, 8, 0.2, _rot(32, 10000.0)), 50),
    _parallel(_att(1, 1, 256, 256, 0.06, _rot(64, 10000.0)), _lin(4, 16, 24, (0.0, 1.0, 0.6, 0.95)), None)]}
# D: attention layers only (pages and no state); E: parallel layers only, borrowed in a row
MOVIVIK_D = {"architecture": "Movivik", "width": 64, "vocab": 120, "norm": {"eps": 1e-6}, "layers": [
    _attention(_att(2, 1, 48, 32, 0.2, _rot(48, 2000.0, (2.5, 24, 6.0, 1.5)), chunk=16), 32),
    _attention(_att(5, 5, 16, 40, 0.3, _rot(4, 10.0), chunk=45), None)]}
_E_PAR = (_att(2, 2, 32, 16, 0.2, _rot(16, 700.0)), _lin(3, 20, 12, (0.9, 0.6, 0.99)))
MOVIVIK_E = {"architecture": "Movivik", "width": 48, "vocab": 88, "norm": {"eps": 3e-6}, "layers": [
    _parallel(*_E_PAR, 20), _parallel(*_E_PAR, 20, weights_of=0), _parallel(*_E_PAR, 20, weights_of=1)]}

# F: nothing is a multiple of 4 or 8 (the products fall to the CUDA-core kernel in both precisions, no access is a
# vector's): width 50, heads of 10, 6 and 14 values, a rotation of 6 of them, a chunk of 7 positions, a prime vocabulary;
# the parallel layer comes first and the attention layer borrows nothing
MOVIVIK_F = {"architecture": "Movivik", "width": 50, "vocab": 61, "norm": {"eps": 1e-4}, "layers": [
    _parallel(_att(3, 1, 10, 6, 0.4, _rot(6, 20.0)), _lin(3, 5, 7, (0.3, 0.8, 0.99)), 21),
    _attention(_att(2, 2, 14, 9, 0.3, _rot(6, 70.0, (1.5, 12, 3.0, 1.0)), chunk=7), 13)]}

MOVIVIK = {"A": MOVIVIK_A, "B": MOVIVIK_B, "C": MOVIVIK_C, "D": MOVIVIK_D, "E": MOVIVIK_E, "F": MOVIVIK_F}


def sharpen(tensors: dict, config: dict, q_gain: float = 4.0) -> dict:
    """Random weights of N(0, 0.02) leave every activation tiny: every attention nearly uniform, the mixers a rounding
    error beside the embedding; a lost key, a chunk edge that is one position off or a stale state would not show. Here
    every matrix is rescaled so that unit inputs give unit outputs (N(0, 1 / fan-in)) and the embedding to N(0, 1); the
    query projections are scaled up further so that single keys stand out among hundreds, and the biases are large enough
    to matter."""
    out = dict(tensors)
    for name, t in tensors.items():
        if name == "embed":
            out[name] = (t.float() * 50.0).to(t.dtype)
        elif t.dim() == 2:
            gain = q_gain if name.endswith(".q") else 1.0
            out[name] = (t.float() * (gain / (0.02 * t.shape[1] ** 0.5))).to(t.dtype)
        elif name.endswith(".b"):
            out[name] = (t.float() * 25.0).to(t.dtype)
    return out


def random_movivik(seed: int) -> dict:
    """A configuration drawn (seeded) from everything the design's keys allow at small sizes: any order of the two kinds
    of layers, borrowed weights, layers without a feed-forward, head widths from 8 to 128 (equal and unequal for keys and
    values; the widths the tile kernels take among them), any number of heads and kv heads, rotations of a part or all of
    a head, with and without scaling and mask on either attention, chunks of 3 to 130 positions, decays from 0.2 to 1."""
    import random
    rng = random.Random(seed)
    widths = [8, 16, 24, 32, 40, 48, 64, 80, 96, 128]

    def attention(left: bool) -> dict:
        kv = rng.choice([1, 1, 2, 3])
        heads = kv * rng.choice([1, 2, 3, 4] if kv > 1 else [1, 2, 4, 5, 8, 18])
        dim = rng.choice(widths)
        vdim = dim if rng.random() < 0.5 else rng.choice(widths)
        dims = dim if rng.random() < 0.4 else 2 * rng.randint(1, dim // 2)
        if rng.random() < 0.5:
            dims = max(16, dims // 16 * 16) if dim >= 16 else dims
        scaling = None
        if rng.random() < (0.3 if left else 0.8):
            scaling = (rng.choice([1.5, 2.0, 4.0, 16.0]), rng.choice([8, 32, 100]), rng.choice([4.0, 16.0, 32.0]), rng.choice([0.5, 1.0, 2.0]))
        chunk = rng.choice([3, 16, 31, 64, 100, 130]) if rng.random() < (0.3 if left else 0.85) else None
        return _att(heads, kv, dim, vdim, round(rng.uniform(0.6, 1.6) / dim ** 0.5, 4), _rot(min(dims, dim), rng.choice([30.0, 1000.0, 10000.0]), scaling), chunk)

    def linear() -> dict:
        heads = rng.choice([1, 2, 3, 5])
        return _lin(heads, rng.choice([8, 12, 16, 32, 64, 128]), rng.choice([8, 16, 24, 40, 64, 72, 128]),
                    [round(rng.uniform(0.2, 1.0), 4) for _ in range(heads)])

    layers = []
    for i in range(rng.randint(2, 5)):
        ff = None if rng.random() < 0.2 else rng.choice([8, 24, 40, 64, 100])
        same = [j for j, l in enumerate(layers) if "weights_of" not in l]
        if same and rng.random() < 0.3:
            j = rng.choice(same)
            layers.append(dict({k: v for k, v in layers[j].items()}, weights_of=j))
        elif rng.random() < 0.5:
            layers.append(_attention(attention(False), ff))
        else:
            layers.append(_parallel(attention(True), linear(), ff))
    return {"architecture": "Movivik", "width": rng.choice([24, 40, 64, 72, 128]), "vocab": rng.choice([53, 128, 300]),
            "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-4])}, "layers": layers}


def movivik_folder_of(config: dict, seed: int = 3, sharp: bool = True, q_gain: float = 4.0) -> Path:
    """A temporary model folder for any configuration (random, by default sharpened weights; `q_gain`: how far the query
    projections are scaled up beyond unit outputs)."""
    from jllm_serve_b200.config import parse_config
    from jllm_serve_b200.config.registry import architecture_entry, model_type_of
    from jllm_serve_b200.engine.model import model_wants
    from jllm_serve_b200.weights import random_tensors, write_safetensors
    wants = model_wants(architecture_entry(model_type_of(config)), parse_config(config))
    tensors = random_tensors(wants, seed, "cpu", torch.bfloat16)
    if sharp:
        tensors = sharpen(tensors, config, q_gain)
    d = Path(tempfile.mkdtemp(prefix="jllm_movivik_"))
    (d / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(d / "model.safetensors", tensors, {"format": "pt"})
    return d


@functools.lru_cache(maxsize=None)
def movivik_folder(name: str, seed: int = 3, sharp: bool = True) -> Path:
    """A temporary model folder with random (and, by default, sharpened) weights; never inside the repository."""
    from jllm_serve_b200.config import parse_config
    from jllm_serve_b200.config.registry import architecture_entry, model_type_of
    from jllm_serve_b200.engine.model import model_wants
    from jllm_serve_b200.weights import random_tensors, write_safetensors
    config = MOVIVIK[name]
    wants = model_wants(architecture_entry(model_type_of(config)), parse_config(config))
    tensors = random_tensors(wants, seed, "cpu", torch.bfloat16)
    if sharp:
        tensors = sharpen(tensors, config)
    d = Path(tempfile.mkdtemp(prefix="jllm_movivik_"))
    (d / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(d / "model.safetensors", tensors, {"format": "pt"})
    return d
