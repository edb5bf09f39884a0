"""Plain, slow implementation of the Madevik decoder: the oracle of its tests.

Madevik is a small decoder-only design: an embedding, a list of layers that each hold one
token mixer (gated linear attention with a recurrent state, or softmax attention over a
cached low-rank latent) and optionally a routed mixture of small gated feed-forwards, a
Dynamic-Tanh norm in front of each of them, a scaled residual sum, a final norm and a head.
A layer may borrow another layer's tensors and keep only a cache or state of its own.

Whole sequences, token by token where a mechanism is recurrent, one function per mechanism,
tensors on the CPU in float64 unless the caller says otherwise. It shares no code with the
product: it reads config.json and model.safetensors with its own few lines and writes every
sum as a loop or a plain torch expression.

Notation (h: a layer part's input [T, width]; Wn: the tensor named n, stored [out, in]):
  dyt(x)            = tanh(a * x) * w + b                      (a scalar, w and b vectors)
  gla:   q_t = Wq h_t / sqrt(dk), k_t = Wk h_t, v_t = Wv h_t,  per head, dk query/key and dv value channels
         d_t = sigmoid(Wa2 (Wa1 h_t) + ba2) ** (1 / tau)       per head and key channel
         S_t = d_t[:, None] * S_(t-1) + outer(k_t, v_t);  o_t = S_t^T q_t
         y_t = Wo concat_heads(rms(o_t) * n) * silu(Wg h_t)
  latent attention: c_t = rms(Wdkv h_t) * n;  k = Wuk c, v = Wuv c per head;
         p_t = softmax_j<=t(q_t . k_j * scale);  y_t = Wo concat_heads(sigmoid(Wg h_t)_head * sum_j p_tj v_j)
  experts: s = sigmoid(Wr h); pick the `top` largest s + correction; weight_e = s_e / (sum of picked s + 1e-20)
         * router scale;  y = sum_e weight_e * Wdown_e (silu(Wgate_e h) * (Wup_e h))
  layer: x += m * mixer(dyt1(x));  x += m * experts(dyt2(x))
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

def dyt(x, w, name):
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def gla_mixer(h, w, p, mx, eps, state=None):
    """h [T, width] -> [T, width]; `state` [heads, dk, dv] is updated in place if given (else it starts at zero)."""
    H, dk, dv, tau = mx["heads"], mx["dim"], mx["vdim"], float(mx["tau"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    decay = torch.sigmoid(z).pow(1.0 / tau).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=h.dtype) if state is None else state
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        for hd in range(H):
            S[hd] = decay[t, hd][:, None] * S[hd] + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    o = rms(o, eps) * w[p + "norm"]
    g = h @ w[p + "g"].T
    return (o.reshape(T, H * dv) * (g * torch.sigmoid(g))) @ w[p + "o"].T


def latent_attention_mixer(h, w, p, mx, eps, latents=None):
    """h [T, width] -> [T, width]; `latents`: the latent rows of earlier positions [P, rank] (the new ones are appended
    and the whole returned as second result)."""
    H, dk, dv, rank, scale = mx["heads"], mx["dim"], mx["vdim"], mx["kv_rank"], float(mx["scale"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, H, dk)
    c = rms(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]
    c_all = c if latents is None else torch.cat([latents, c], dim=0)
    P = c_all.shape[0] - T
    k = (c_all @ w[p + "uk"].T).view(-1, H, dk)
    v = (c_all @ w[p + "uv"].T).view(-1, H, dv)
    gate = torch.sigmoid(h @ w[p + "g"].T)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        n = P + t + 1
        for hd in range(H):
            s = (k[:n, hd] @ q[t, hd]) * scale
            pr = torch.softmax(s, dim=0)
            out[t, hd] = (pr[:, None] * v[:n, hd]).sum(dim=0) * gate[t, hd]
    return out.reshape(T, H * dv) @ w[p + "o"].T, c_all


def routing(h, w, p, r):
    """[T, experts] weights: zero for the experts a token does not use."""
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    picked = torch.topk(choice, int(r["top"]), dim=-1).indices
    mask = torch.zeros_like(s).scatter_(1, picked, 1.0)
    chosen = s * mask
    return chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20) * float(r["scale"])


def experts(h, w, p, mlp):
    r = mlp["router"]
    weights = routing(h, w, p, r)
    y = torch.zeros_like(h)
    for e in range(int(r["experts"])):
        a = h @ w[f"{p}e{e}.gate"].T
        one = ((a * torch.sigmoid(a)) * (h @ w[f"{p}e{e}.up"].T)) @ w[f"{p}e{e}.down"].T
        y = y + weights[:, e:e + 1] * one
    return y


# ---- the model ------------------------------------------------------------------------------------------------------

def owner_of(cfg, i):
    while "weights_of" in cfg["layers"][i] and cfg["layers"][i]["weights_of"] is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; `layers_out` (a list) gets the residual stream after every layer."""
    x = w["embed"][torch.tensor(tokens)]
    m, eps = float(cfg["residual_mult"]), float(cfg["norm"]["eps"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{owner_of(cfg, i)}."
        h = dyt(x, w, p + "norm1")
        if layer["type"] == "gla":
            y = gla_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "latent_attention":
            y, _ = latent_attention_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + m * y
        if layer.get("mlp") is not None:
            x = x + m * experts(dyt(x, w, p + "norm2"), w, p + "mlp.", layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return dyt(x, w, "final.norm") @ w["head"].T


def greedy_generate(cfg, w, prompt, n):
    """`n` tokens chosen greedily (the lowest index wins a tie), the whole sequence run anew for every token."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(cfg, w, tokens)[-1].argmax()))
    return tokens[len(prompt):]
