"""Attention over a cached latent as a mixer: one row of `rank` values per position instead of keys and values per head.

With h the normed rows:  q = Wq h (heads x dk),  c_t = rmsnorm(Wd h_t) * n (rank values: all that is cached),
k_j = Wuk c_j and v_j = Wuv c_j per head, p = softmax over j <= t of scale (q . k_j), head output sigmoid(Wg h)_head *
sum_j p_j v_j, x += m Wo [heads side by side]. Nothing rotates.

Since q_h . (Wuk_h c_j) = (Wuk_h^T q_h) . c_j and sum_j p_j Wuv_h c_j = Wuv_h sum_j p_j c_j, the keys and values of
earlier positions are never made: the queries are carried into the latent's space (one small product per head, all heads
in one launch), the engine's paged attention runs with ONE key/value head of width `rank` whose keys and values are the
same cached rows (`PagedKeysValues(1, rank, planes=1)`), and its result goes through Wuv per head, where the gate and the
residual scale m are applied. Scores, softmax and the latent's norm are float32 in both precisions.
"""
from __future__ import annotations

import torch

from ..cache.manager import PagedKeysValues
from ..csrc import ops
from ..weights.loader import TensorWant
from .base import Mixer, register_mixer
from .linear import Linear


def _up8(n: int) -> int:
    return -(-n // 8) * 8


class LatentAttention(Mixer):
    takes_residual_scale = True

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.spec, self.dim, self.rt = spec, dim, runtime
        self.residual_scale = 1.0
        H, dk, dv, R = spec.heads, spec.key_dim, spec.value_dim, spec.rank
        names = ["q", "dkv"] + (["g"] if spec.gated else [])
        self.offsets, rows, at = [], [], 0
        for n in names:
            w = tensors.pop(prefix + n)
            self.offsets.append(at)
            pad = _up8(w.shape[0]) - w.shape[0]
            rows.append(w)
            if pad:
                rows.append(torch.zeros((pad, dim), dtype=w.dtype, device=w.device))
            at += w.shape[0] + pad
        self.width = at
        self.inp = Linear(torch.cat(rows, dim=0).contiguous())
        del rows
        self.latent_gain = tensors.pop(prefix + "dkv.norm")
        # Wuk [heads x dk, rank] as [heads, rank, dk]: the product that carries a head's query into the latent's space
        self.q_to_latent = tensors.pop(prefix + "uk").view(H, dk, R).transpose(1, 2).contiguous()
        self.latent_to_v = tensors.pop(prefix + "uv").view(H, dv, R).contiguous()
        self.out = Linear(tensors.pop(prefix + "o"))

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        H, dk, dv, R = spec.heads, spec.key_dim, spec.value_dim, spec.rank
        out = {prefix + "q": TensorWant((H * dk, dim)), prefix + "dkv": TensorWant((R, dim)),
               prefix + "dkv.norm": TensorWant((R,), "vector", init="gain"), prefix + "uk": TensorWant((H * dk, R)),
               prefix + "uv": TensorWant((H * dv, R)), prefix + "o": TensorWant((dim, H * dv))}
        if spec.gated:
            out[prefix + "g"] = TensorWant((H, dim))
        return out

    @classmethod
    def cache_need(cls, spec):
        return PagedKeysValues(1, spec.rank, spec.window, planes=1)

    def decode_bucket_cap(self, rows: int) -> int:
        s = self.spec
        heads = min(s.heads, 16)
        if not ops.attention_decode_fits(self.rt.dtype, heads, 1, s.rank):
            return 1
        scratch = self.rt.buffer("attention_scratch", 2 << 20, torch.float32, rows=1)[0]
        return max(ops.decode_bucket_cap(rows, 1, n, s.rank, s.window, scratch)
                   for n in {heads, s.heads % 16 or heads})

    def forward(self, xb, x, batch, cache) -> None:
        s, rows = self.spec, xb.shape[0]
        H, dk, dv, R = s.heads, s.key_dim, s.value_dim, s.rank
        proj = self.rt.buffer("latent_proj", self.width)[:rows]
        self.inp.forward(xb, proj)
        if cache.writes:
            d_off = self.offsets[1]
            ops.latent_norm_store(proj[:, d_off:d_off + R], self.latent_gain, s.norm_eps, batch.slots[cache.group], cache.keys)
        q = self.rt.buffer("latent_queries", H * R)[:rows]
        ops.gemm_heads(proj[:, :H * dk], self.q_to_latent, q)
        att = self.rt.buffer("latent_attended", H * R)[:rows]
        scratch = self.rt.buffer("attention_scratch", 2 << 20, torch.float32, rows=1)[0]
        # the decode kernel shares every key among at most 16 query heads: more heads go in groups of 16, each a launch
        # over the same cached rows
        per = 16 if H > 16 and ops.attention_decode_fits(q.dtype, 16, 1, R) else H
        for h0 in range(0, H, per):
            n = min(per, H - h0)
            ops.attention(q[:, h0 * R:(h0 + n) * R], cache.keys, cache.values, att[:, h0 * R:(h0 + n) * R], batch,
                          cache.group, n, 1, R, self.rt.page_size, s.window, s.scale, scratch)
        y = self.rt.buffer("latent_values", H * dv)[:rows]
        gate = proj[:, self.offsets[2]:self.offsets[2] + H] if s.gated else None
        ops.gemm_heads(att, self.latent_to_v, y, gate, self.residual_scale)
        self.out.forward(y, x, accumulate=True)


register_mixer("latent_attention", LatentAttention, replace=True)
