"""Mamba-2 (the state-space duality layer) as a mixer.

With inner = heads * head_dim, N = state_dim and G = groups, W_in x is laid out [z: inner | x: inner | B: G*N | C: G*N |
dt: heads].  x, B and C together pass a causal convolution per channel (``conv_taps`` taps, the last one the current
token's, zeros before a request's first token, a bias) and silu.  dt <- softplus(dt + dt_bias), not clamped.  Head h, which
reads group h // (heads / G):

    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T        (S: N x head_dim)
    y_t = S_t^T C_t + D_h x_t

y times silu(z), then RMS-normed in ``norm_groups`` equal parts, times a weight, then the output projection (the gate comes
before the norm).  The state (S, float32, and the convolution's last taps - 1 inputs) lives in the request's state slot.
dt, the decay and the recurrence are float32 in both precisions: dt's rows of W_in are a product of their own whose
sums stay float32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

import torch

from .. import ops
from .base import Mixer, StateNeed, WeightDecl
from .registry import register_part


@dataclass(frozen=True)
class Mamba2Spec:
    prefix: str
    hidden_size: int
    num_heads: int
    head_dim: int
    state_dim: int
    groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float
    names: Optional[Tuple[Tuple[str, str], ...]] = None    # (role, name after the prefix); see DEFAULT_NAMES
    kind: ClassVar[str] = "mamba2"


DEFAULT_NAMES = (("in", "in"), ("conv", "conv"), ("conv_bias", "conv.b"), ("dt_bias", "dt_bias"), ("a_log", "A_log"), ("skip", "D"),
                 ("norm", "norm"), ("o", "o"))


class Mamba2(Mixer):
    def __init__(self, spec: Mamba2Spec):
        if min(spec.num_heads, spec.head_dim, spec.state_dim, spec.groups, spec.conv_taps, spec.norm_groups) <= 0:
            raise ValueError("mamba2: every size must be positive")
        if spec.num_heads % spec.groups or (spec.num_heads * spec.head_dim) % spec.norm_groups:
            raise ValueError("mamba2: heads must be a multiple of groups and heads * head_dim a multiple of norm_groups")
        if spec.state_dim > 512:
            raise ValueError(f"mamba2: state_dim {spec.state_dim} not supported (at most 512)")
        self.spec = spec
        self.names = dict(DEFAULT_NAMES)
        self.names.update(dict(spec.names or ()))
        self.inner = spec.num_heads * spec.head_dim
        self.bc = spec.groups * spec.state_dim
        self.channels = self.inner + 2 * self.bc             # what the convolution runs over
        self.main_rows = self.inner + self.channels          # z, x, B, C
        self.conv_offset = spec.num_heads * spec.head_dim * spec.state_dim
        self.w_in = self.w_o = self.conv = self.conv_bias = self.dt_bias = self.a_log = self.skip = self.norm = None

    def _name(self, role: str) -> str:
        return self.spec.prefix + self.names[role]

    def weight_decls(self):
        s = self.spec
        H = s.num_heads
        return (WeightDecl(self._name("in"), (self.main_rows + H, s.hidden_size)),
                WeightDecl(self._name("conv"), (self.channels, s.conv_taps), init="around_zero"),
                WeightDecl(self._name("conv_bias"), (self.channels,), init="around_zero"),
                WeightDecl(self._name("dt_bias"), (H,), init="around_zero"), WeightDecl(self._name("a_log"), (H,), init="around_zero"),
                WeightDecl(self._name("skip"), (H,), init="gain"), WeightDecl(self._name("norm"), (self.inner,), init="gain"),
                WeightDecl(self._name("o"), (s.hidden_size, self.inner)))

    def load(self, tensors, dtype, device):
        def kept(t):
            return dtype if dtype == torch.bfloat16 else (torch.float32 if t.dtype == torch.float32 else torch.bfloat16)

        w, o = tensors[self._name("in")], tensors[self._name("o")]
        self.w_in = w.to(device=device, dtype=kept(w)).contiguous()
        self.w_o = o.to(device=device, dtype=kept(o)).contiguous()
        self.conv, self.conv_bias, self.dt_bias, self.a_log, self.skip, self.norm = (
            tensors[self._name(n)].to(device=device, dtype=torch.float32).contiguous()
            for n in ("conv", "conv_bias", "dt_bias", "a_log", "skip", "norm"))

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def scratch_elements_per_token(self):
        return self.main_rows + self.channels + 3 * self.inner + 6 * self.spec.num_heads + self.spec.hidden_size

    def state_need(self):
        n = self.conv_offset + self.channels * (self.spec.conv_taps - 1)
        return StateNeed((-(-n // 4) * 4,), torch.float32)

    def can_sink(self, num_rows):
        return ops.fused_gemm_shape_ok(num_rows, self.w_o)

    def forward(self, x, ctx, cache, state, sink=None):
        s = self.spec
        T = x.shape[0]
        H, P, N, inner, bc = s.num_heads, s.head_dim, s.state_dim, self.inner, self.bc
        zxbc = ctx.ws.get("ssm_in", (T, self.main_rows), x.dtype)
        ops.gemm(x, self.w_in[: self.main_rows], zxbc)
        dt_raw = ctx.ws.get("ssm_dt", (T, H), torch.float32)
        ops.gemm(x, self.w_in[self.main_rows:], dt_raw)
        xbc = ctx.ws.get("ssm_conv", (T, self.channels), x.dtype)
        ops.conv_silu(zxbc[:, inner:], self.conv, self.conv_bias, state, self.conv_offset, ctx.q_indptr, ctx.row_of_token,
                      ctx.state_slots, xbc)
        a, b = (ctx.ws.get(n, (T, H), torch.float32) for n in ("scan_a", "scan_b"))
        ops.ssm_gates(dt_raw, self.dt_bias, self.a_log, a, b)
        y = ctx.ws.get("scan_out", (T, H, P), torch.float32)
        ops.decay_scan(xbc[:, inner + bc:], xbc[:, inner: inner + bc], xbc[:, :inner], a, b, state, ctx.q_indptr, ctx.state_slots, y,
                       H, s.groups, N, P, False, 1.0)
        gated = ctx.ws.get("ssm_gated", (T, inner), x.dtype)
        ops.gated_group_norm(y.view(T, inner), xbc[:, :inner], self.skip, P, zxbc[:, :inner], self.norm, s.norm_eps, gated, s.norm_groups)
        out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
        return None if ops.gemm(gated, self.w_o, out, sink=sink) else out


register_part(Mamba2Spec.kind, Mamba2)
