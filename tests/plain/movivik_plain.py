"""Plain, slow implementation of the Movivik decoder: the oracle of its tests.

Movivik is a small decoder-only design: an embedding, a list of layers, a final RMS norm and a head. A layer has a
token mixer and a dense gated feed-forward (tanh-form GELU), each between two RMS norms (one in front, one behind, and
only then the residual sum). Two mixers: `attention` (grouped-query softmax attention whose positions only see their own
chunk of the sequence, rotary positions on interleaved pairs with YaRN-stretched frequencies, biases on q, k, v, key
and value widths that may differ, a sigmoid gate per head) and `parallel` (a causal softmax attention with rotate-half
rotary on part of every head and unit-norm q and k, beside a linear attention with one fixed decay per head; the two
results are normed over the model width and averaged). A layer may borrow another layer's tensors and keep only a cache
or state of its own.

Whole sequences, token by token where a mechanism is recurrent, one function per mechanism, tensors on the CPU in
float64 unless the caller says otherwise. It shares no code with the product: it reads config.json and
model.safetensors with its own few lines and writes every sum as a loop or a plain torch expression.

Notation (h: a mixer's or feed-forward's input [T, width]; Wn: the tensor named n, stored [out, in]; p: position):
  rms(x)     = x / sqrt(mean(x^2) + eps);  norm(x, n) = rms(x) * n
  rotary     f_i = base^(-2i / dims), i < dims / 2; pair (a, b) at position p -> (a cos(p f_i) - b sin(p f_i),
             b cos(p f_i) + a sin(p f_i)); pairs are (2i, 2i + 1) ("interleaved") or (i, i + dims / 2) ("half");
             only the first `dims` values of a head rotate
  yarn       c(t) = dims ln(original / (2 pi t)) / (2 ln base); lo = max(floor(c(fast)), 0), hi = min(ceil(c(slow)),
             dims - 1); r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); f_i <- f_i / factor * r_i + f_i (1 - r_i);
             cos and sin times 0.1 ln(factor) + 1
  attention  q = Wq h + bq, k = Wk h + bk, v = Wv h + bv; rotate q, k; (optionally q <- rms(q), k <- rms(k) per head);
             row t sees j <= t (with a chunk size c only those with floor(j / c) = floor(t / c));
             o_t,head = sigmoid(Wg h_t)_head * sum_j softmax_j(scale q_t . k_j) v_j;  y = Wo concat_heads(o)
  lightning  q, k, v = silu(Wq h), silu(Wk h), silu(Wv h); per head S_t = decay * S_(t-1) + outer(k_t, v_t);
             o_t = S_t^T q_t;  y = Wo (norm(concat_heads(o), n) * sigmoid(Wg h))
  parallel   y = (norm(left(h), n_left) + norm(right(h), n_right)) / 2
  feed-forward  y = Wdown (gelu_tanh(Wgate h) * (Wup h))
  layer      x += norm(mixer(norm(x, n1)), n1b);  x += norm(ff(norm(x, n2)), n2b)
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


def read_tensors(path) -> dict:
    """safetensors: u64 little-endian header length, JSON header, raw data."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    data = raw[8 + hlen:]
    kinds = {"F32": np.float32, "F64": np.float64, "I32": np.int32, "I64": np.int64, "F16": np.float16}
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        if meta["dtype"] == "BF16":
            arr = (np.frombuffer(data[lo:hi], dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
        else:
            arr = np.frombuffer(data[lo:hi], dtype=kinds[meta["dtype"]])
        out[name] = torch.from_numpy(arr.reshape(meta["shape"]).copy())
    return out


def load_plain(folder, dtype=torch.float64):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in read_tensors(folder / "model.safetensors").items()}
    return cfg, w


# ---- mechanisms, one function each --------------------------------------------------------------------------------

def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, gain, eps):
    return rms(x, eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotary_frequencies(rot):
    """(frequencies [dims / 2] as a list of Python floats, amplitude of cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def c(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(c(float(sc["fast"]))), 0)
    hi = min(math.ceil(c(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * r + fi * (1 - r))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot, pairing):
    """x [T, heads, dim]: the first rot.dims values of every head rotated by the position's angles."""
    dims = int(rot["dims"])
    f, amp = rotary_frequencies(rot)
    out = x.clone()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a, b = (2 * i, 2 * i + 1) if pairing == "interleaved" else (i, i + dims // 2)
            cs, sn = math.cos(p * f[i]) * amp, math.sin(p * f[i]) * amp
            u, v = x[t, :, a], x[t, :, b]
            out[t, :, a] = u * cs - v * sn
            out[t, :, b] = v * cs + u * sn
    return out


def softmax_attention(h, w, p, mx, eps, *, bias, pairing, unit_qk, positions=None):
    """h [T, width] -> [T, width]: the grouped-query attention of both mixers; `mx` the mixer's sizes."""
    H, G, dk, dv, scale = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], float(mx["scale"])
    chunk = int(mx["mask"]["size"]) if mx.get("mask") else 0
    T = h.shape[0]
    positions = list(range(T)) if positions is None else positions
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if bias:
        q, k, v = q + w[p + "q.b"], k + w[p + "k.b"], v + w[p + "v.b"]
    q, k, v = q.view(T, H, dk), k.view(T, G, dk), v.view(T, G, dv)
    q, k = rotate(q, positions, mx["rot"], pairing), rotate(k, positions, mx["rot"], pairing)
    if unit_qk:
        q, k = rms(q, eps), rms(k, eps)
    gate = torch.sigmoid(h @ w[p + "g"].T)                       # [T, H]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        pt = positions[t]
        seen = [j for j in range(t + 1) if not chunk or positions[j] // chunk == pt // chunk]
        for hd in range(H):
            g = hd // (H // G)
            s = (k[seen, g] @ q[t, hd]) * scale
            pr = torch.softmax(s, dim=0)
            acc = (pr[:, None] * v[seen, g]).sum(dim=0)
            out[t, hd] = acc * gate[t, hd]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def lightning_attention(h, w, p, mx, eps, state=None):
    """h [T, width] -> [T, width]; `state` [heads, dk, dv] is updated in place if given (else it starts at zero)."""
    H, dk, dv = mx["heads"], mx["dim"], mx["vdim"]
    decay = [float(d) for d in mx["decay"]]
    T = h.shape[0]
    q, k, v = silu(h @ w[p + "q"].T).view(T, H, dk), silu(h @ w[p + "k"].T).view(T, H, dk), silu(h @ w[p + "v"].T).view(T, H, dv)
    S = torch.zeros(H, dk, dv, dtype=h.dtype) if state is None else state
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        for hd in range(H):
            S[hd] = decay[hd] * S[hd] + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    y = norm(o.reshape(T, H * dv), w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def attention_mixer(h, w, p, mx, eps):
    return softmax_attention(h, w, p, mx, eps, bias=True, pairing="interleaved", unit_qk=False)


def parallel_mixer(h, w, p, mx, eps):
    left = softmax_attention(h, w, p + "left.", mx["left"], eps, bias=False, pairing="half", unit_qk=True)
    right = lightning_attention(h, w, p + "right.", mx["right"], eps)
    return 0.5 * (norm(left, w[p + "left.out"], eps) + norm(right, w[p + "right.out"], eps))


def feed_forward(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ---- the model ------------------------------------------------------------------------------------------------------

def owner_of(cfg, i):
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; `layers_out` (a list) gets the residual stream after every layer."""
    x = w["embed"][torch.tensor(tokens)]
    eps = float(cfg["norm"]["eps"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{owner_of(cfg, i)}."
        h = norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = attention_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            x = x + norm(feed_forward(norm(x, w[p + "norm2"], eps), w, p + "mlp."), w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm(x, w["final.norm"], eps) @ w["head"].T


def greedy_generate(cfg, w, prompt, n):
    """`n` tokens chosen greedily (the lowest index wins a tie), the whole sequence run anew for every token."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(cfg, w, tokens)[-1].argmax()))
    return tokens[len(prompt):]
