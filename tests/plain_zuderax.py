"""A plain, slow implementation of the Zuderax design: float64 torch on the CPU, whole sequences,
no cache, no batching, one function per mechanism.  It shares no code with the package's model
path; the tests compare the engine with it.

A model is (config dict in the form of config.json, {tensor name: tensor}).  ``forward`` returns
the logits of every position and, on request, the residual after every layer run.  ``rnd`` is applied to
every stored activation (identity by default; rounding to bfloat16 gives the tests the size of what
rounding alone does).

Notation: h is a mixer's input [T, width]; positions count from 0.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def _ident(x):
    return x


def round_bf16(x):
    return x.to(torch.float32).to(torch.bfloat16).to(F64)


def lin(W, x):
    """Rows of x through a matrix stored [out, in]."""
    return x @ W.to(F64).t()


# ----------------------------------------------------------------------------- small functions
def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dyn_tanh(x, w, b, alpha):
    return torch.tanh(alpha.to(F64) * x) * w.to(F64) + b.to(F64)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rotate_half_layout(x, pos, base, dims):
    """x [T, ..., D]; the first ``dims`` elements turn, element i with i + dims/2, by pos * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    freq = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)
    ang = pos.to(F64)[:, None] * freq[None, :]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ----------------------------------------------------------------------------- mixers
def latent_attention(h, W, p, m, eps, rnd=_ident):
    """m: the mixer's sizes.  Keys and values are rebuilt from a latent vector per token."""
    T = h.shape[0]
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = rnd(lin(W[p + "q"], h)).view(T, H, dn + dr)
    dkv = rnd(lin(W[p + "dkv"], h))
    c = rnd(rms_unit(dkv[:, :rank], eps) * W[p + "dkv.norm"].to(F64))
    k_rot = rnd(rotate_half_layout(dkv[:, rank:], pos, m["rot"]["base"], m["rot"]["dims"]))
    q_rot = rotate_half_layout(q[..., dn:], pos, m["rot"]["base"], m["rot"]["dims"])
    k_nope = rnd(lin(W[p + "uk"], c)).view(T, H, dn)
    v = rnd(lin(W[p + "uv"], c)).view(T, H, dv)
    scores = (torch.einsum("thd,shd->hts", q[..., :dn], k_nope) + torch.einsum("thd,sd->hts", rnd(q_rot), k_rot)) * m["scale"]
    i, j = pos[:, None], pos[None, :]
    visible = (j <= i) & (i - j < m["mask"]["size"])
    scores = scores.masked_fill(~visible[None], -math.inf)
    w = torch.softmax(scores, dim=-1)
    o = rnd(torch.einsum("hts,shd->thd", w, v).reshape(T, H * dv))
    return lin(W[p + "o"], o)


def mlstm(h, W, p, m, eps, rnd=_ident):
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = rnd(lin(W[p + "q"], h)).view(T, H, dk) * dk ** -0.5
    k = rnd(lin(W[p + "k"], h)).view(T, H, dk)
    v = rnd(lin(W[p + "v"], h)).view(T, H, dv)
    gi = cap * torch.tanh((lin(W[p + "i"], h) + W[p + "i.b"].to(F64)) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((lin(W[p + "f"], h) + W[p + "f.b"].to(F64)) / cap))
    out = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        n = torch.zeros(dk, dtype=F64)
        mx = 0.0
        for t in range(T):
            m_new = max(float(gf[t, a]) + mx, float(gi[t, a]))
            keep, take = math.exp(float(gf[t, a]) + mx - m_new), math.exp(float(gi[t, a]) - m_new)
            S = keep * S + take * torch.outer(k[t, a], v[t, a])
            n = keep * n + take * k[t, a]
            mx = m_new
            den = max(abs(float(n @ q[t, a])), math.exp(-mx)) + 1e-6
            out[t, a] = (S.t() @ q[t, a]) / den
    o = rms_unit(out, eps).reshape(T, H * dv) * W[p + "norm"].to(F64)
    o = rnd(o * torch.sigmoid(rnd(lin(W[p + "g"], h))))
    return lin(W[p + "o"], o)


def mamba2(h, W, p, m, eps, rnd=_ident):
    T = h.shape[0]
    H, P, N, G, taps, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
    inner = H * P
    proj = lin(W[p + "in"], h)
    z, xbc, dt = rnd(proj[:, :inner]), rnd(proj[:, inner: 2 * inner + 2 * G * N]), proj[:, 2 * inner + 2 * G * N:]
    cw, cb = W[p + "conv"].to(F64), W[p + "conv.b"].to(F64)
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=F64), xbc], dim=0)
    conv = cb[None, :].repeat(T, 1)
    for j in range(taps):
        conv = conv + padded[j: j + T] * cw[:, j][None, :]
    xbc = rnd(silu(conv))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner: inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"].to(F64))
    decay = torch.exp(-torch.exp(W[p + "A_log"].to(F64))[None, :] * dt)
    y = torch.zeros(T, H, P, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        S = torch.zeros(N, P, dtype=F64)
        for t in range(T):
            S = decay[t, a] * S + dt[t, a] * torch.outer(B[t, g], x[t, a])
            y[t, a] = S.t() @ C[t, g] + W[p + "D"].to(F64)[a] * x[t, a]
    y = y.reshape(T, inner) * silu(z)
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * W[p + "norm"].to(F64)
    return lin(W[p + "o"], rnd(y))


# ----------------------------------------------------------------------------- feed-forward
def gated_ff(h, W, p, rnd=_ident):
    return lin(W[p + "down"], rnd(silu(rnd(lin(W[p + "gate"], h))) * rnd(lin(W[p + "up"], h))))


def route(h, W, p, r):
    """Returns (chosen experts [T, top], their weights [T, top])."""
    E, top, groups, keep = r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"]
    s = torch.sigmoid(lin(W[p + "router"], h))
    choice = s + W[p + "correction"].to(F64)
    per = E // groups
    g = choice.view(-1, groups, per)
    gscore = g.topk(min(2, per), dim=-1).values.sum(-1)
    kept = gscore.topk(keep, dim=-1).indices
    open_ = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, kept, True)
    masked = torch.where(open_[:, :, None].expand(-1, -1, per).reshape(-1, E), choice, torch.full_like(choice, -math.inf))
    chosen = masked.topk(top, dim=-1).indices
    return chosen, s.gather(1, chosen) * r["scale"]


def moe_ff(h, W, p, mlp, rnd=_ident):
    chosen, weights = route(h, W, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            out[t] += w * rnd(gated_ff(h[t: t + 1], W, f"{p}e{e}.", rnd))[0]
    if mlp.get("shared") is not None:
        sg = torch.sigmoid(lin(W[p + "shared.sg"], h))
        out = out + sg * rnd(gated_ff(h, W, p + "shared.", rnd))
    return out


# ----------------------------------------------------------------------------- the model
MIXERS = {"latent_attention": latent_attention, "mlstm": mlstm, "mamba2": mamba2}


def forward(config, W, tokens, rnd=_ident, layers_out=None):
    """Logits [T, vocab] (float64) of one sequence; ``layers_out`` (a list) gets the residual after every layer run."""
    eps = float(config["norm"]["eps"])
    x = W["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)]

    def norm(name, v):
        return rnd(dyn_tanh(v, W[name], W[name + ".b"], W[name + ".alpha"]))

    for i, layer in enumerate(config["layers"]):
        src = i
        while config["layers"][src].get("weights_of") is not None:      # a layer may name a layer that itself names another
            src = config["layers"][src]["weights_of"]
        p = f"l{src}."
        x = x + rnd(MIXERS[layer["type"]](norm(p + "norm1", x), W, p + "mix.", layer["mixer"], eps, rnd))
        mlp = layer.get("mlp")
        if mlp is not None:
            n = norm(p + "norm2", x)
            x = x + rnd(gated_ff(n, W, p + "mlp.", rnd) if mlp["kind"] == "dense" else moe_ff(n, W, p + "mlp.", mlp, rnd))
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(W["head"], norm("final.norm", x)) * float(config["logit_scale"])


def generate_greedy(config, W, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(config, W, toks)[-1])))
    return toks[len(prompt):]
