"""Gated linear attention as a mixer: a recurrent state per request and head instead of cached keys and values.

With h the normed rows, per head (dk query/key channels, dv value channels):

    q_t = s Wq h_t,  k_t = Wk h_t,  v_t = Wv h_t,  d_t = sigmoid(W2 (W1 h_t) + b2)^(1 / tau)      (d per key channel)
    S_t = diag(d_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t
    x  += m Wo [ rmsnorm(o_t) * n  (per head, one gain n of dv values)  *  silu(Wg h_t) ]

The state S [heads, dk, dv] is float32 and lives in the cache manager's state slots (zero when a request is opened), so a
prompt may come in portions of any size. A decode step runs the recurrence token by token; a step with prompt portions
runs it in chunks of sixteen tokens, as small matrix products (both float32: only the grouping of sums differs). The decays,
their logarithms and the norm are computed in float32 in both precisions; q, k, v, the gate and the low-rank decay
projection are one stacked product. The residual scale m is applied where the gated rows are written, in front of the
output product, which adds into the residual stream itself.
"""
from __future__ import annotations

import torch

from ..cache.manager import FixedState
from ..csrc import ops
from ..weights.loader import TensorWant
from .base import Mixer, register_mixer
from .linear import Linear


def _up8(n: int) -> int:
    return -(-n // 8) * 8


class GatedLinearAttention(Mixer):
    takes_residual_scale = True

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.spec, self.dim, self.rt = spec, dim, runtime
        self.residual_scale = 1.0
        H, dk, dv = spec.heads, spec.key_dim, spec.value_dim
        parts = [tensors.pop(prefix + n) for n in ("q", "k", "v", "g", "a1")]
        self.rank = parts[4].shape[0]
        # every piece of the stacked product starts at a multiple of 8 columns: a piece is then a view that the
        # tensor-core products take as an operand
        self.offsets, rows, at = [], [], 0
        for w in parts:
            self.offsets.append(at)
            pad = _up8(w.shape[0]) - w.shape[0]
            rows.append(w)
            if pad:
                rows.append(torch.zeros((pad, dim), dtype=w.dtype, device=w.device))
            at += w.shape[0] + pad
        self.width = at
        self.inp = Linear(torch.cat(rows, dim=0).contiguous())
        del parts, rows
        self.decay = Linear(tensors.pop(prefix + "a2"), tensors.pop(prefix + "a2.b"))
        self.out = Linear(tensors.pop(prefix + "o"))
        self.gain = tensors.pop(prefix + "norm")

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        H, dk, dv, r = spec.heads, spec.key_dim, spec.value_dim, spec.decay_rank
        return {prefix + "q": TensorWant((H * dk, dim)), prefix + "k": TensorWant((H * dk, dim)),
                prefix + "v": TensorWant((H * dv, dim)), prefix + "g": TensorWant((H * dv, dim)),
                prefix + "o": TensorWant((dim, H * dv)), prefix + "norm": TensorWant((dv,), "vector", init="gain"),
                prefix + "a1": TensorWant((r, dim)), prefix + "a2": TensorWant((H * dk, r)),
                prefix + "a2.b": TensorWant((H * dk,), "vector")}

    @classmethod
    def cache_need(cls, spec):
        return FixedState((spec.heads, spec.key_dim, spec.value_dim), "float32")

    def decode_bucket_cap(self, rows: int) -> int:
        return 1                       # nothing here looks at the context's length

    def forward(self, xb, x, batch, cache) -> None:
        s, rows = self.spec, xb.shape[0]
        if not cache.writes or cache.state is None:
            raise ops.KernelError("gated linear attention keeps its own state: a run cannot read another run's")
        H, dk, dv = s.heads, s.key_dim, s.value_dim
        q_off, k_off, v_off, g_off, a_off = self.offsets
        proj = self.rt.buffer("gla_proj", self.width)[:rows]
        self.inp.forward(xb, proj)
        z = self.rt.buffer("gla_decay_logits", H * dk, torch.float32)[:rows]
        self.decay.forward(proj[:, a_off:a_off + self.rank], z)
        o = self.rt.buffer("gla_out", H * dv, torch.float32)[:rows]
        if batch.decode_only:
            ops.gla_recurrent(proj, q_off, k_off, v_off, z, cache.state, batch.seg_start, batch.seg_len, batch.state_slots,
                              o, H, dk, dv, s.query_scale, s.decay_temperature)
        else:       # prompt portions (and the single rows beside them): sixteen tokens at a time
            qb = self.rt.buffer("gla_chunk_queries", H * dk, torch.float32)[:rows]
            ke = self.rt.buffer("gla_chunk_keys", H * dk, torch.float32)[:rows]
            scores = self.rt.buffer("gla_chunk_scores", H * ops.GLA_CHUNK, torch.float32)[:rows]
            ops.gla_chunked(proj, q_off, k_off, v_off, z, cache.state, batch.seg_start, batch.seg_len, batch.state_slots, o,
                            H, dk, dv, s.query_scale, s.decay_temperature, batch.max_q_len, qb, ke, scores)
        y = self.rt.buffer("gla_gated", H * dv)[:rows]
        ops.gated_head_norm(o, proj[:, g_off:g_off + H * dv], self.gain, s.norm_eps, self.residual_scale, y, H, dv)
        self.out.forward(y, x, accumulate=True)


register_mixer("gated_linear_attention", GatedLinearAttention, replace=True)


class FixedDecayLinearAttention(Mixer):
    """Linear attention with one fixed decay per head ("lightning" attention), through the kernels of the gated form:

        q_t, k_t, v_t = act(Wq h_t), act(Wk h_t), act(Wv h_t)          (act = silu)
        S_t = decay_head S_(t-1) + k_t v_t^T,   o_t = S_t^T (s q_t)      (S [heads, dk, dv] float32, in a state slot)
        x  += Wo [ rmsnorm(o_t) * n  *  sigmoid(Wg h_t) ]               (the norm over all heads of a row together, or per head)

    The decays are constants of the configuration, kept as float32 on the device; a pass in front of the recurrence fills
    the decay table the kernels read (the decay for the token-by-token form, its logarithm for the chunked one) and applies
    the activation to q, k and v where the stacked product left them. State, decays and the norm are float32 in both
    precisions."""
    can_overwrite = True

    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.spec, self.dim, self.rt = spec, dim, runtime
        self.overwrite = False
        H, dk, dv = spec.heads, spec.key_dim, spec.value_dim
        parts = [tensors.pop(prefix + n) for n in ("q", "k", "v", "g")]
        self.offsets, rows, at = [], [], 0
        for w in parts:
            self.offsets.append(at)
            pad = _up8(w.shape[0]) - w.shape[0]
            rows.append(w)
            if pad:
                rows.append(torch.zeros((pad, dim), dtype=w.dtype, device=w.device))
            at += w.shape[0] + pad
        self.width = at
        self.inp = Linear(torch.cat(rows, dim=0).contiguous())
        del parts, rows
        self.out = Linear(tensors.pop(prefix + "o"))
        self.gain = tensors.pop(prefix + "norm")
        self.decay = torch.tensor(list(spec.decays), dtype=torch.float64).to(torch.float32).to(runtime.device)

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        H, dk, dv = spec.heads, spec.key_dim, spec.value_dim
        return {prefix + "q": TensorWant((H * dk, dim)), prefix + "k": TensorWant((H * dk, dim)),
                prefix + "v": TensorWant((H * dv, dim)), prefix + "g": TensorWant((H * dv, dim)),
                prefix + "o": TensorWant((dim, H * dv)),
                prefix + "norm": TensorWant((H * dv if spec.norm_over == "all" else dv,), "vector", init="gain")}

    @classmethod
    def cache_need(cls, spec):
        return FixedState((spec.heads, spec.key_dim, spec.value_dim), "float32")

    def decode_bucket_cap(self, rows: int) -> int:
        return 1                       # nothing here looks at the context's length

    def forward(self, xb, x, batch, cache) -> None:
        s, rows = self.spec, xb.shape[0]
        if not cache.writes or cache.state is None:
            raise ops.KernelError("linear attention keeps its own state: a run cannot read another run's")
        H, dk, dv = s.heads, s.key_dim, s.value_dim
        q_off, k_off, v_off, g_off = self.offsets
        act = 1 if s.activation == "silu" else 0
        proj = self.rt.buffer("gla_proj", self.width)[:rows]
        self.inp.forward(xb, proj)
        z = self.rt.buffer("gla_decay_logits", H * dk, torch.float32)[:rows]
        o = self.rt.buffer("gla_out", H * dv, torch.float32)[:rows]
        if batch.decode_only:
            ops.gla_recurrent(proj, q_off, k_off, v_off, z, cache.state, batch.seg_start, batch.seg_len, batch.state_slots,
                              o, H, dk, dv, s.query_scale, 1.0, head_decay=self.decay, activation=act)
        else:
            qb = self.rt.buffer("gla_chunk_queries", H * dk, torch.float32)[:rows]
            ke = self.rt.buffer("gla_chunk_keys", H * dk, torch.float32)[:rows]
            scores = self.rt.buffer("gla_chunk_scores", H * ops.GLA_CHUNK, torch.float32)[:rows]
            ops.gla_chunked(proj, q_off, k_off, v_off, z, cache.state, batch.seg_start, batch.seg_len, batch.state_slots, o,
                            H, dk, dv, s.query_scale, 1.0, batch.max_q_len, qb, ke, scores, head_decay=self.decay,
                            activation=act)
        y = self.rt.buffer("gla_gated", H * dv)[:rows]
        heads, width = (1, H * dv) if s.norm_over == "all" else (H, dv)
        ops.gated_head_norm(o, proj[:, g_off:g_off + H * dv], self.gain, s.norm_eps, 1.0, y, heads, width, s.gate)
        self.out.forward(y, x, accumulate=not self.overwrite)


register_mixer("fixed_decay_linear_attention", FixedDecayLinearAttention, replace=True)
