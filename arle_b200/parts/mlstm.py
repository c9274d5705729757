"""The matrix memory of xLSTM (mLSTM) as a mixer.

Per head, with q = W_q x * dim^(-1/2), k = W_k x, v = W_v x, the capped log gates
i = cap tanh((W_i x + b_i) / cap), f = logsigmoid(cap tanh((W_f x + b_f) / cap)) and a running maximum m (zero before a
request's first token):

    m_t = max(f + m_(t-1), i)
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T          n_t likewise with k alone
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)

then each head's o divided by its root mean square, the heads side by side times a weight of all heads' size, times
sigmoid(W_g x), and the output projection.  S, n and m are float32 and live in the request's state slot
([heads][vdim + 1][dim] with n as the last column, then the heads' m); the gates, their exponentials and the
recurrence are float32 in both precisions.  q, k, v and the output gate are rows of one packed projection; the two
gate rows per head are a small product of their own whose sums stay float32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

import torch

from .. import ops
from .base import Mixer, StateNeed, WeightDecl
from .registry import register_part


@dataclass(frozen=True)
class MatrixLstmSpec:
    prefix: str
    hidden_size: int
    num_heads: int
    key_dim: int                    # per head
    value_dim: int                  # per head
    gate_cap: float
    norm_eps: float
    names: Optional[Tuple[Tuple[str, str], ...]] = None    # (role, name after the prefix); see DEFAULT_NAMES
    kind: ClassVar[str] = "matrix_lstm"


DEFAULT_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("o", "o"), ("norm", "norm"), ("i", "i"), ("i_bias", "i.b"),
                 ("f", "f"), ("f_bias", "f.b"))


class MatrixLstm(Mixer):
    def __init__(self, spec: MatrixLstmSpec):
        if min(spec.num_heads, spec.key_dim, spec.value_dim) <= 0 or not spec.gate_cap > 0:
            raise ValueError("matrix LSTM: heads, key_dim, value_dim and gate_cap must be positive")
        if spec.key_dim > 512:
            raise ValueError(f"matrix LSTM: key_dim {spec.key_dim} not supported (at most 512)")
        self.spec = spec
        self.names = dict(DEFAULT_NAMES)
        self.names.update(dict(spec.names or ()))
        dq, dv = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim
        self.at = {"q": 0, "k": dq, "v": 2 * dq, "gate": 2 * dq + dv}
        self.rows = -(-(2 * dq + 2 * dv) // 8) * 8
        self.m_offset = spec.num_heads * (spec.value_dim + 1) * spec.key_dim
        self.w_in = self.w_gates = self.w_o = self.bias_i = self.bias_f = self.norm = None

    def _name(self, role: str) -> str:
        return self.spec.prefix + self.names[role]

    def weight_decls(self):
        s = self.spec
        dq, dv, H = s.num_heads * s.key_dim, s.num_heads * s.value_dim, s.num_heads
        return (WeightDecl(self._name("q"), (dq, s.hidden_size)), WeightDecl(self._name("k"), (dq, s.hidden_size)),
                WeightDecl(self._name("v"), (dv, s.hidden_size)), WeightDecl(self._name("gate"), (dv, s.hidden_size)),
                WeightDecl(self._name("o"), (s.hidden_size, dv)), WeightDecl(self._name("norm"), (dv,), init="gain"),
                WeightDecl(self._name("i"), (H, s.hidden_size)), WeightDecl(self._name("i_bias"), (H,), init="around_zero"),
                WeightDecl(self._name("f"), (H, s.hidden_size)), WeightDecl(self._name("f_bias"), (H,), init="around_zero"))

    def load(self, tensors, dtype, device):
        s = self.spec

        def kept(ts):
            return dtype if dtype == torch.bfloat16 else (torch.float32 if any(t.dtype == torch.float32 for t in ts) else torch.bfloat16)

        mats = [tensors[self._name(n)] for n in ("q", "k", "v", "gate")]
        pad = self.rows - sum(m.shape[0] for m in mats)
        if pad:
            mats.append(torch.zeros((pad, s.hidden_size), dtype=mats[0].dtype))
        self.w_in = torch.cat([m.to(device=device, dtype=kept(mats)) for m in mats], dim=0).contiguous()
        gates = [tensors[self._name("i")], tensors[self._name("f")]]
        self.w_gates = torch.cat([m.to(device=device, dtype=kept(gates)) for m in gates], dim=0).contiguous()
        o = tensors[self._name("o")]
        self.w_o = o.to(device=device, dtype=kept([o])).contiguous()
        self.bias_i, self.bias_f, self.norm = (tensors[self._name(n)].to(device=device, dtype=torch.float32).contiguous()
                                               for n in ("i_bias", "f_bias", "norm"))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_gates, self.w_o))

    def scratch_elements_per_token(self):
        s = self.spec
        return self.rows + 2 * s.num_heads * (s.value_dim + 6) + s.num_heads * s.value_dim + s.hidden_size

    def state_need(self):
        s = self.spec
        return StateNeed((self.m_offset + -(-s.num_heads // 4) * 4,), torch.float32)

    def can_sink(self, num_rows):
        return ops.fused_gemm_shape_ok(num_rows, self.w_o)

    def forward(self, x, ctx, cache, state, sink=None):
        s = self.spec
        T = x.shape[0]
        H, dk, dv = s.num_heads, s.key_dim, s.value_dim
        proj = ctx.ws.get("mlstm_in", (T, self.rows), x.dtype)
        ops.gemm(x, self.w_in, proj)
        pre = ctx.ws.get("mlstm_pre", (T, 2 * H), torch.float32)
        ops.gemm(x, self.w_gates, pre)
        a, b, floor = (ctx.ws.get(n, (T, H), torch.float32) for n in ("scan_a", "scan_b", "mlstm_floor"))
        ops.mlstm_gates(pre, self.bias_i, self.bias_f, s.gate_cap, ctx.q_indptr, ctx.state_slots, state, self.m_offset, a, b, floor)
        at = self.at
        num = ctx.ws.get("scan_out", (T, H, dv + 1), torch.float32)
        ops.decay_scan(proj[:, at["q"]: at["q"] + H * dk], proj[:, at["k"]: at["k"] + H * dk], proj[:, at["v"]: at["v"] + H * dv],
                       a, b, state, ctx.q_indptr, ctx.state_slots, num, H, H, dk, dv, True, dk ** -0.5)
        gated = ctx.ws.get("mlstm_gated", (T, H * dv), x.dtype)
        ops.mlstm_out(num, floor, proj[:, at["gate"]: at["gate"] + H * dv], self.norm, s.norm_eps, gated, H, dv)
        out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
        return None if ops.gemm(gated, self.w_o, out, sink=sink) else out


register_part(MatrixLstmSpec.kind, MatrixLstm)
