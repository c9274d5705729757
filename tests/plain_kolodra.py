"""Plain, slow statement of the Kolodra forward pass: whole sequences, no cache, float64.

The oracle of the engine's Kolodra tests.  It shares no code with the package: the
configuration is a plain dict, the weights a dict of tensors by checkpoint name, and every
mechanism is one function of elementary tensor arithmetic.

The design in this file's notation (T tokens, width D, positions p = 0, 1, ...):

    x_0      = E[token] * embedding.scale
    layer:     n = rms(x) * (1 + w_norm1);  x <- x + (mixer(n) + ff(n))     (one norm, two readers)
    mixer    = left_scale * softmax_side(n) + right_scale * recurrent_side(n)
    logits   = cap * tanh((head . (rms(x) * (1 + w_final))) / cap)

rms(x) = x / sqrt(mean(x^2) + eps) everywhere.  A layer entry with ``weights_of: j`` runs with
layer j's tensors.
"""
from __future__ import annotations

import math

import torch

DT = torch.float64

# What a 16-bit engine keeps between kernels can be imitated: ``with stored_as(torch.bfloat16):`` rounds every
# activation that such an engine writes to memory (projections, normed rows, heads' outputs, branch outputs), while the
# arithmetic in between stays float64.  The distance between such a run and the exact one is what rounding alone
# costs on a given model and prompt; the tests allow the engine a small multiple of it.
_STORE = [None]


class stored_as:
    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        _STORE.append(self.dtype)

    def __exit__(self, *exc):
        _STORE.pop()
        return False


def st(x):
    return x if _STORE[-1] is None else x.to(_STORE[-1]).to(DT)


# ------------------------------------------------------------------- elementary
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """The layer norm and the final norm: the stored weight lies around zero."""
    return rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def embedding(table, ids, scale: float):
    return table[torch.as_tensor(ids, dtype=torch.long)] * scale


def rotate_interleaved(x, positions, base: float, dims: int):
    """x [T, heads, dim]: elements (2i, 2i+1), i < dims/2, of every head turn by the angle
    p * base^(-2i/dims); elements from ``dims`` on pass."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=DT)
    ang = positions.to(DT)[:, None] * base ** (-2.0 * i / dims)[None, :]          # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ------------------------------------------------------------------ softmax side
def softmax_side(n, w, p: str, m: dict, eps: float, start: int = 0):
    """Causal attention whose values are its keys as projected.  q and k are normed over the whole
    projected row (all heads at once, plain weight), then rotated; the value of a key is the row of
    W_k n before norm and rotation; head h's output is scaled by sigmoid(W_g n)_h."""
    T = n.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(start, start + T)
    q = st(n @ w[p + "q"].T)
    k = st(n @ w[p + "k"].T)
    v = k.reshape(T, G, d)
    q = (rms(q, eps) * w[p + "q.norm"]).reshape(T, H, d)
    k = (rms(k, eps) * w[p + "k.norm"]).reshape(T, G, d)
    q = st(rotate_interleaved(q, pos, m["rot"]["base"], m["rot"]["dims"]))
    k = st(rotate_interleaved(k, pos, m["rot"]["base"], m["rot"]["dims"]))
    gate = sigmoid(st(n @ w[p + "g"].T))                                           # [T, H]
    out = torch.zeros(T, H, d, dtype=n.dtype)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        g = h // (H // G)
        sc = (q[:, h] @ k[:, g].T) * m["scale"]
        sc = sc.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(sc, dim=-1) @ v[:, g]
    out = st(st(out) * gate[:, :, None])
    return st(out.reshape(T, H * d) @ w[p + "o"].T)


# ---------------------------------------------------------------- recurrent side
def decay(n, w, p: str, m: dict):
    """alpha [T, heads, dim] = sigmoid(W_a2 (W_a1 n) + b)^(1/tau)."""
    z = st(n @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    return (sigmoid(z) ** (1.0 / m["tau"])).reshape(n.shape[0], m["heads"], m["dim"])


def recurrent_side(n, w, p: str, m: dict, eps: float, state=None):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T per head (S is dim x vdim, zero before the first token),
    o_t = S_t^T q_t with q scaled by dim^(-1/2); o is normed per head over vdim (plain weight shared by
    the heads), multiplied by silu(W_g n) and projected."""
    T = n.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = st(n @ w[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = st(n @ w[p + "k"].T).reshape(T, H, d)
    v = st(n @ w[p + "v"].T).reshape(T, H, dv)
    a = decay(n, w, p, m)
    S = torch.zeros(H, d, dv, dtype=n.dtype) if state is None else state
    o = torch.zeros(T, H, dv, dtype=n.dtype)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * w[p + "norm"]
    o = st(o.reshape(T, H * dv) * silu(st(n @ w[p + "g"].T)))
    return st(o @ w[p + "o"].T), S


def parallel_mixer(n, w, p: str, m: dict, eps: float):
    left = softmax_side(n, w, p + "left.", m["left"], eps)
    right, _ = recurrent_side(n, w, p + "right.", m["right"], eps)
    return st(m["left_scale"] * left + m["right_scale"] * right)


# ------------------------------------------------------------------ feed-forward
def dense_ff(n, w, p: str):
    return st(st(gelu_tanh(st(n @ w[p + "gate"].T)) * st(n @ w[p + "up"].T)) @ w[p + "down"].T)


# ------------------------------------------------------------------------ model
def layer_prefix(cfg: dict, i: int) -> str:
    """Prefix of the tensors layer i runs with: its own, or those of the layer its ``weights_of`` leads to."""
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return f"l{i}."


def layer(x, w, cfg: dict, i: int):
    e = cfg["layers"][i]
    if e["type"] != "parallel":
        raise ValueError(f"layer type {e['type']!r}")
    p, eps = layer_prefix(cfg, i), cfg["norm"]["eps"]
    n = st(norm_one_plus(x, w[p + "norm1"], eps))
    y = parallel_mixer(n, w, p + "mix.", e["mixer"], eps)
    if e.get("mlp") is not None:
        if e["mlp"]["kind"] != "dense":
            raise ValueError(f"feed-forward kind {e['mlp']['kind']!r}")
        y = y + dense_ff(n, w, p + "mlp.")
    return x + y


def forward(w: dict, cfg: dict, tokens, trace: list = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0; ``trace`` collects the residual after every layer."""
    w = {k: (v.to(DT) if v.is_floating_point() else v) for k, v in w.items()}
    x = embedding(w["embed"], tokens, cfg["embedding"]["scale"])
    for i in range(len(cfg["layers"])):
        x = layer(x, w, cfg, i)
        if trace is not None:
            trace.append(x)
    y = st(norm_one_plus(x, w["final.norm"], cfg["norm"]["eps"])) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(y / cap) if cap else y


def generate_greedy(w: dict, cfg: dict, prompt, steps: int) -> list:
    toks = list(prompt)
    for _ in range(steps):
        toks.append(int(forward(w, cfg, toks)[-1].argmax()))
    return toks[len(prompt):]
