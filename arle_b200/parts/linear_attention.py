"""Gated linear attention: a recurrent mixer whose memory is one matrix per head,

    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,

S of size key_dim x value_dim, zero before a request's first token, kept in float32 in the
request's state slot and carried from step to step.  The decay alpha_t in (0, 1), one number
per key channel, comes from a low-rank gate: alpha = sigmoid(W_a2 (W_a1 x) + b)^(1/tau).
Each head's o is RMS-normed over value_dim (a plain weight shared by the heads), multiplied by
silu(W_g x) and projected by W_o.  q is scaled by ``q_scale`` (key_dim^(-1/2) by default).

q, k, v, the output gate and the low-rank half of the decay gate are rows of one packed input
projection; the decay, the recurrence and the norm run in float32 whatever the activation type.
The mixer keeps no per-token cache: a step costs the same however long the request is.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

import torch

from .. import ops
from .base import Mixer, StateNeed, WeightDecl
from .registry import register_part


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    prefix: str
    hidden_size: int
    num_heads: int
    key_dim: int                    # per head
    value_dim: int                  # per head
    decay_rank: int                 # rows of W_a1
    tau: float                      # alpha = sigmoid(.)^(1/tau)
    norm_eps: float
    q_scale: Optional[float] = None            # None: key_dim^(-1/2)
    names: Optional[Tuple[Tuple[str, str], ...]] = None    # (role, name after the prefix); see DEFAULT_NAMES
    kind: ClassVar[str] = "gated_linear_attention"


DEFAULT_NAMES = (("q", "q_proj.weight"), ("k", "k_proj.weight"), ("v", "v_proj.weight"), ("gate", "g_proj.weight"),
                 ("o", "o_proj.weight"), ("norm", "g_norm.weight"), ("decay_in", "gk_proj.0.weight"),
                 ("decay_out", "gk_proj.1.weight"), ("decay_bias", "gk_proj.1.bias"))


class GatedLinearAttention(Mixer):
    def __init__(self, spec: GatedLinearAttentionSpec):
        if min(spec.num_heads, spec.key_dim, spec.value_dim, spec.decay_rank) <= 0 or not spec.tau > 0:
            raise ValueError("gated linear attention: heads, key_dim, value_dim, decay_rank and tau must be positive")
        if spec.key_dim > 512:
            raise ValueError(f"gated linear attention: key_dim {spec.key_dim} not supported (at most 512)")
        self.spec = spec
        self.names = dict(DEFAULT_NAMES)
        self.names.update(dict(spec.names or ()))
        self.q_scale = spec.q_scale if spec.q_scale is not None else spec.key_dim ** -0.5
        self.w_in = self.w_o = self.w_decay = self.decay_bias = self.norm = None
        dq, dv = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim
        # columns of the packed projection: q | k | v | gate | low-rank decay input | padding
        self.at = {"q": 0, "k": dq, "v": 2 * dq, "gate": 2 * dq + dv, "low": 2 * dq + 2 * dv}
        self.rows = -(-(2 * dq + 2 * dv + spec.decay_rank) // 8) * 8

    def _name(self, role: str) -> str:
        return self.spec.prefix + self.names[role]

    # ---------------------------------------------------------------- weights
    def weight_decls(self):
        s = self.spec
        dq, dv = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        return (WeightDecl(self._name("q"), (dq, s.hidden_size)), WeightDecl(self._name("k"), (dq, s.hidden_size)),
                WeightDecl(self._name("v"), (dv, s.hidden_size)), WeightDecl(self._name("gate"), (dv, s.hidden_size)),
                WeightDecl(self._name("o"), (s.hidden_size, dv)), WeightDecl(self._name("norm"), (s.value_dim,), init="gain"),
                WeightDecl(self._name("decay_in"), (s.decay_rank, s.hidden_size)),
                WeightDecl(self._name("decay_out"), (dq, s.decay_rank)),
                WeightDecl(self._name("decay_bias"), (dq,), init="around_zero"))

    def load(self, tensors, dtype, device):
        s = self.spec
        mats = [tensors[self._name(n)] for n in ("q", "k", "v", "gate", "decay_in")]
        pad = self.rows - sum(m.shape[0] for m in mats)
        if pad:
            mats.append(torch.zeros((pad, s.hidden_size), dtype=mats[0].dtype))
        wt = dtype if dtype == torch.bfloat16 else (torch.float32 if any(m.dtype == torch.float32 for m in mats) else torch.bfloat16)
        self.w_in = torch.cat([m.to(device=device, dtype=wt) for m in mats], dim=0).contiguous()
        o = tensors[self._name("o")]
        self.w_o = o.to(device=device, dtype=dtype if dtype == torch.bfloat16 else o.dtype).contiguous()
        # what enters the recurrence is float32 in both precisions
        self.w_decay = tensors[self._name("decay_out")].to(device=device, dtype=torch.float32).t().contiguous()   # [rank, heads*key_dim]
        self.decay_bias = tensors[self._name("decay_bias")].to(device=device, dtype=torch.float32).contiguous()
        self.norm = tensors[self._name("norm")].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o, self.w_decay))

    def scratch_elements_per_token(self):
        s = self.spec
        # the packed projection and the gated output in the activation type; alpha and o in float32 (two elements each)
        return self.rows + s.num_heads * s.value_dim + 2 * s.num_heads * (s.key_dim + s.value_dim) + s.hidden_size

    # ------------------------------------------------------------------ state
    def state_need(self):
        s = self.spec
        return StateNeed((s.num_heads, s.value_dim, s.key_dim), torch.float32)     # a head's S, transposed

    def takes_scaled_rows(self, num_rows):
        return ops.fused_gemm_shape_ok(num_rows, self.w_in)

    def can_sink(self, num_rows):
        return ops.fused_gemm_shape_ok(num_rows, self.w_o)

    # ---------------------------------------------------------------- forward
    def pre_output_width(self):
        return self.spec.num_heads * self.spec.value_dim

    def output_weight(self):
        return self.w_o

    def forward_pre(self, x, ctx, cache, state, into, scale):
        s = self.spec
        T = x.shape[0]
        H, dk, dv = s.num_heads, s.key_dim, s.value_dim
        proj = ctx.ws.get("gla_in", (T, self.rows), x.dtype)
        ops.gemm(x, self.w_in, proj)
        at = self.at
        alpha = ctx.ws.get("gla_alpha", (T, H * dk), torch.float32)
        ops.gla_decay(proj[:, at["low"]: at["low"] + s.decay_rank], self.w_decay, self.decay_bias, s.tau, alpha)
        o = ctx.ws.get("gla_o", (T, H * dv), torch.float32)
        ops.gla_scan(proj[:, at["q"]: at["q"] + H * dk], proj[:, at["k"]: at["k"] + H * dk], proj[:, at["v"]: at["v"] + H * dv],
                     alpha, state, ctx.q_indptr, ctx.state_slots, o, H, dk, dv, self.q_scale, ctx.max_q_len)
        ops.gla_out(o, proj[:, at["gate"]: at["gate"] + H * dv], self.norm, s.norm_eps, scale, into, H, dv)

    def forward(self, x, ctx, cache, state, sink=None):
        s = self.spec
        T = x.shape[0]
        gated = ctx.ws.get("gla_gated", (T, s.num_heads * s.value_dim), x.dtype)
        self.forward_pre(x, ctx, cache, state, gated, 1.0)
        out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
        return None if ops.gemm(gated, self.w_o, out, sink=sink) else out


register_part(GatedLinearAttentionSpec.kind, GatedLinearAttention)
