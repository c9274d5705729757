"""Zuderax on the GPU against the plain implementation (``plain_zuderax``): every new kernel alone at sizes of no model
(rows of unequal length that continue from states in permuted slots, windows and page borders, routing on made-up
scores), the engine under every cutting in float32 and bfloat16 on tiny configurations, the first tokens of a sequence and
prompts that end on page borders, keys just inside and just outside a window and far keys made to decide the logits
(sharpened attention), far tokens living on in the recurrent states (decays next to one), long decoding, a request that
starts again, greedy generation through the public entry point with CUDA graphs and preemption, and the replay tool and
the command line as subprocesses."""
import copy
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kernel_refs
import plain_zuderax as plain
import traces
from arle_b200 import Engine, ops
from arle_b200.engine import ModelRunner, StepEntry, load_model
from arle_b200.sampling import SamplingParams
from arle_b200.weights import SafetensorsFile, write_safetensors
from tiny_zuderax import CONFIGS, PAGE_SIZES, make_model_dir, read_model

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
# error of a logits row as a fraction of the spread of the plain model's logits: float32 rounding through a few layers.
# In bfloat16 the engine's worst position may be off by 4.5 times what the plain model's worst is off by when every
# activation it stores is rounded to bfloat16: two ways of rounding the same sums differ by more than either differs
# from the exact result.
REL = {torch.float32: 5e-4, torch.bfloat16: 1e-2}
LENGTHS = {"Z1": [1, 5, 12, 23, 70, 130, 33], "Z2": [2, 17, 40, 96, 64, 31], "Z3": [3, 66, 150, 64, 40, 97], "S": [2, 33, 80, 17, 64],
           "L": [3, 50, 64, 29], "R": [1, 40, 33, 7, 70]}
_cache, _rounding = {}, {}


def rounding_cost(cfg, w, toks, exact) -> float:
    return (plain.forward(cfg, w, toks, rnd=plain.round_bf16) - exact).abs().max().item()


def model_and_oracle(name, tmp_path_factory):
    if name not in _cache:
        d = make_model_dir(name, seed=21, root=str(tmp_path_factory.mktemp(f"tiny{name}")))
        cfg, w = read_model(d)
        reqs = traces.make_requests(cfg["vocab"], LENGTHS[name], seed=6)
        oracle = {r: plain.forward(cfg, w, t) for r, t in reqs.items()}
        _cache[name] = (d, cfg, w, reqs, oracle)
        _rounding[id(oracle)] = max(rounding_cost(cfg, w, t, oracle[r]) for r, t in reqs.items())
    return _cache[name]


def assert_close(got, want, dtype, what="", rounding=0.0):
    err = (got.double().cpu() - want).abs().max(dim=-1).values
    tol = REL[dtype] * float(want.std())
    if dtype == torch.bfloat16:
        tol = max(tol, 4.5 * rounding)
    assert err.max().item() <= tol, f"{what}: first wrong position {int((err > tol).nonzero()[0])}, error {err.max().item():.3g}, tolerance {tol:.3g}"


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def _both(fn, args, outs):
    """Runs ``fn`` of ops on the GPU and of kernel_refs on the CPU on copies of the same arguments; returns the named outputs."""
    cpu = [a.clone() if isinstance(a, torch.Tensor) else a for a in args]
    gpu = [a.to(DEV) if isinstance(a, torch.Tensor) else a for a in args]
    getattr(ops, fn)(*gpu)
    getattr(kernel_refs, fn)(*cpu)
    torch.cuda.synchronize()
    return [(gpu[i].float().cpu(), cpu[i].float()) for i in outs]


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_dyn_tanh_kernel(dtype):
    g = torch.Generator().manual_seed(0)
    for H in (64, 100, 1536):
        resid, delta = torch.randn(9, H, generator=g) * 3, torch.randn(9, H, generator=g).to(dtype)
        w, b = torch.rand(H, generator=g) + 0.5, torch.randn(H, generator=g) * 0.1
        for rows in (None, torch.tensor([7, 0, 3], dtype=torch.int32)):
            out = torch.zeros(9 if rows is None else 3, H, dtype=dtype)
            for (a, c) in _both("dyt_norm", [resid, delta, rows, w, b, 0.7, out, rows is None], [0, 6]):
                torch.testing.assert_close(a, c, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("H,dn,dr,rdims,rank,window,ps", [(3, 16, 8, 8, 20, 7, 4), (1, 8, 16, 12, 33, 0, 8), (16, 64, 32, 32, 128, 48, 16),
                                                          (5, 24, 6, 0, 70, 1, 16), (12, 8, 64, 64, 512, 100, 32), (4, 16, 16, 16, 64, 0, 16),
                                                          (40, 32, 16, 16, 256, 300, 16), (20, 8, 0, 0, 128, 129, 8)])
def test_latent_attention_kernels(dtype, H, dn, dr, rdims, rank, window, ps):
    """Three rows of unequal length in scattered pages: a portion that continues a request, a decoded token far into its
    request, a fresh prompt.  Where the tensor-core kernel takes the shapes it is compared with the same plain statement,
    with the step as it is (a token's keys in few parts) and with the decoded token alone (its keys in many parts)."""
    g = torch.Generator().manual_seed(H * 7 + rank)
    kd = rank + dr
    starts, lens = [37, 700, 0], [23, 1, 41]
    T = sum(lens)
    width = H * (dn + dr) + 3
    q, dkv = torch.randn(T, width, generator=g).to(dtype), torch.randn(T, kd + 5, generator=g).to(dtype)
    cw = torch.rand(rank, generator=g) + 0.5
    inv = (10000.0 ** (-2.0 * torch.arange(rdims // 2, dtype=torch.float64) / max(rdims, 1))).float()
    need = [-(-(s + n) // ps) for s, n in zip(starts, lens)]
    pages = sum(need) + 5
    perm = torch.randperm(pages, generator=g)[: sum(need)].to(torch.int32)
    bt = torch.full((3, max(need)), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(need):
        bt[r, :n] = perm[at: at + n]
        at += n
    cache = (torch.randn(pages, 1, ps, kd, generator=g) * 0.7).to(dtype)        # what earlier steps left
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(torch.int32)
    row = torch.cat([torch.full((n,), r) for r, n in enumerate(lens)]).to(torch.int32)
    slots = (bt[row.long(), (pos // ps).long()] * ps + pos % ps).to(torch.int32)
    q_abs = torch.zeros(T, H, kd, dtype=dtype)
    (ca, cc), (qa, qc) = _both("latent_prep", [q, dkv, pos, slots, cw, 1e-5, inv if rdims else None, rdims, cache, q_abs, H, dn, dr, rank], [8, 9])
    torch.testing.assert_close(ca, cc, **_tol(dtype))
    torch.testing.assert_close(qa[:, :, rank:], qc[:, :, rank:], **_tol(dtype))
    wk = (torch.randn(H, rank, dn, generator=g) * dn ** -0.5).to(dtype)
    qn = q[:, : H * (dn + dr)].unflatten(1, (H, dn + dr))[:, :, :dn]
    for (a, c) in _both("gemm_heads", [qn, wk, qc.to(dtype)[:, :, :rank].clone()], [2]):
        torch.testing.assert_close(a, c, **_tol(dtype))
    q_abs = torch.cat([c.to(dtype), qc.to(dtype)[:, :, rank:]], dim=-1).contiguous()
    out = torch.zeros(T, H, rank, dtype=dtype)
    args = [q_abs, out, cc.to(dtype), pos, row, bt, rank, ps, 0.4 * kd ** -0.5, window or None]
    for (a, c) in _both("latent_attention", args, [1]):
        torch.testing.assert_close(a, c, **_tol(dtype))
    if ops.latent_mma_supported(q_abs.to(DEV), rank):
        from types import SimpleNamespace

        from arle_b200.engine.batch import Workspace
        batch = SimpleNamespace(ws=Workspace(DEV))
        dev = [x.to(DEV) if isinstance(x, torch.Tensor) else x for x in args]
        before = ops.launch_count()
        ops.latent_attention(*dev, batch=batch)
        torch.testing.assert_close(dev[1].float().cpu(), c, **_tol(dtype))
        one = slice(lens[0], lens[0] + 1)                               # the decoded token alone: a step of one row
        got = torch.zeros(1, H, rank, dtype=dtype, device=DEV)
        ops.latent_attention(dev[0][one].contiguous(), got, dev[2], dev[3][one].contiguous(), torch.zeros(1, dtype=torch.int32, device=DEV),
                             dev[5][1:2].contiguous(), rank, ps, args[8], args[9], batch=batch)
        torch.testing.assert_close(got.float().cpu(), c[one], **_tol(dtype))
        assert ops.launch_count() - before == 4                          # both ran in parts and were merged


@pytest.mark.parametrize("M,heads,K,N", [(1, 4, 32, 64), (8, 16, 64, 256), (70, 3, 128, 40), (300, 32, 512, 128), (129, 2, 24, 200)])
def test_per_head_products_on_tensor_cores(M, heads, K, N):
    """bfloat16 rows on 16-byte boundaries inside wider rows take the tensor-core tiles; against float64."""
    g = torch.Generator().manual_seed(M + K)
    wide = torch.randn(M, heads * (K + 8) + 16, generator=g).to(torch.bfloat16).to(DEV)
    x = wide[:, 16: 16 + heads * (K + 8)].unflatten(1, (heads, K + 8))[:, :, :K]
    w = (torch.randn(heads, N, K, generator=g) * K ** -0.5).to(torch.bfloat16).to(DEV)
    out_wide = torch.zeros(M, heads, N + 5, dtype=torch.bfloat16, device=DEV)
    ops.gemm_heads(x, w, out_wide[:, :, :N])
    want = torch.einsum("mhk,hnk->mhn", x.double().cpu(), w.double().cpu())
    torch.testing.assert_close(out_wide[:, :, :N].double().cpu(), want, rtol=1e-2, atol=1e-2)
    assert float(out_wide[:, :, N:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("H,G,dim,vdim,ones", [(2, 2, 12, 20, True), (4, 2, 12, 8, False), (3, 1, 144, 16, False), (2, 2, 160, 32, True),
                                               (1, 1, 300, 5, True), (8, 1, 64, 64, False)])
def test_decay_scan_kernel(dtype, H, G, dim, vdim, ones):
    g = torch.Generator().manual_seed(dim + vdim)
    lens, slots = [19, 1, 2, 35], torch.tensor([5, 0, 3, 2], dtype=torch.int32)
    T = sum(lens)
    vc = vdim + int(ones)
    buf = torch.randn(T, 2 * G * dim + H * vdim + 4, generator=g).to(dtype)
    q, k, v = buf[:, : G * dim], buf[:, G * dim: 2 * G * dim], buf[:, 2 * G * dim: 2 * G * dim + H * vdim]
    a, b = torch.rand(T, H, generator=g) * 0.3 + 0.7, torch.rand(T, H, generator=g)
    state = torch.randn(6, H * vc * dim + 7, generator=g)
    indptr = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    out = torch.zeros(T, H, vc)
    for (x, y) in _both("decay_scan", [q, k, v, a, b, state, indptr, slots, out, H, G, dim, vdim, ones, 0.3], [5, 8]):
        torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-4)


def test_matrix_lstm_gate_and_output_kernels():
    g = torch.Generator().manual_seed(3)
    H, lens, slots = 3, [140, 1, 2], torch.tensor([2, 0, 1], dtype=torch.int32)
    T = sum(lens)
    pre = torch.randn(T, 2 * H, generator=g) * 4
    bi, bf = torch.randn(H, generator=g), torch.randn(H, generator=g) + 3
    state = torch.zeros(4, 50)
    state[:, 40:43] = torch.randn(4, 3, generator=g)                       # maxima carried from earlier steps
    indptr = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    outs = [torch.zeros(T, H) for _ in range(3)]
    for (x, y) in _both("mlstm_gates", [pre, bi, bf, 6.0, indptr, slots, state, 40] + outs, [6, 8, 9, 10]):
        torch.testing.assert_close(x, y, rtol=2e-5, atol=1e-6)
    for dtype in DTYPES:
        vdim = 20
        num = torch.randn(T, H, vdim + 1, generator=g)
        num[::3, :, vdim] *= 1e-3                                           # the floor decides the denominator
        floor, gate = torch.rand(T, H, generator=g), torch.randn(T, H * vdim + 8, generator=g).to(dtype)[:, 8:]
        w, out = torch.rand(H * vdim, generator=g) + 0.5, torch.zeros(T, H * vdim, dtype=dtype)
        for (x, y) in _both("mlstm_out", [num, floor, gate, w, 1e-5, out, H, vdim], [5]):
            torch.testing.assert_close(x, y, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_state_space_side_kernels(dtype):
    g = torch.Generator().manual_seed(4)
    H, lens, slots = 5, [1, 2, 3, 40, 1], torch.tensor([4, 1, 0, 2, 3], dtype=torch.int32)
    T = sum(lens)
    indptr = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    row = torch.cat([torch.full((n,), r) for r, n in enumerate(lens)]).to(torch.int32)
    raw = torch.randn(T, H + 3, generator=g)[:, 3:] * 3
    raw[0, 0] = 40.0                                                        # softplus of a large number is the number
    a, b = torch.zeros(T, H), torch.zeros(T, H)
    for (x, y) in _both("ssm_gates", [raw, torch.randn(H, generator=g), torch.randn(H, generator=g), a, b], [3, 4]):
        torch.testing.assert_close(x, y, rtol=2e-5, atol=1e-6)
    for C, taps in ((37, 4), (200, 2), (16, 1), (24, 7)):                   # rows shorter than the taps reach back into the state
        x = torch.randn(T, C + 2, generator=g).to(dtype)[:, 2:]
        w, bias = torch.randn(C, taps, generator=g) * 0.5, torch.randn(C, generator=g)
        state = torch.randn(5, 11 + C * (taps - 1) + 3, generator=g)
        out = torch.zeros(T, C, dtype=dtype)
        for (p, r) in _both("conv_silu", [x, w, bias, state, 11, indptr, row, slots, out], [3, 8]):
            torch.testing.assert_close(p, r, **_tol(dtype))
    for inner, vdim, parts in ((48, 16, 1), (48, 8, 4), (256, 32, 2), (30, 10, 3)):
        y = torch.randn(T, inner, generator=g)
        xs, z = torch.randn(T, inner, generator=g).to(dtype), torch.randn(T, inner + 8, generator=g).to(dtype)[:, 8:]
        skip, w = torch.randn(inner // vdim, generator=g), torch.rand(inner, generator=g) + 0.5
        out = torch.zeros(T, inner, dtype=dtype)
        for (p, r) in _both("gated_group_norm", [y, xs, skip, vdim, z, w, 1e-5, out, parts], [7]):
            torch.testing.assert_close(p, r, **_tol(dtype))


def test_routing_kernel_against_the_plain_rules():
    """Random router sums with corrections that push every choice score below zero (an expert outside the kept groups must
    lose to a kept one with a negative score), for several (experts, groups, kept, chosen); sets of chosen experts and their
    weights against ``plain.route``."""
    g = torch.Generator().manual_seed(5)
    for E, top, groups, keep in ((8, 3, 4, 2), (6, 2, 3, 2), (3, 1, 1, 1), (8, 4, 8, 5), (64, 6, 8, 3), (16, 16, 4, 4)):
        T = 70
        z = torch.randn(T, E + 1, generator=g) * 2
        corr = torch.randn(E, generator=g) * 0.3 - 2.0
        ids, wts = torch.zeros(T, top, dtype=torch.int32, device=DEV), torch.zeros(T, top, device=DEV)
        ops.moe_select(z.to(DEV), corr.to(DEV), torch.zeros(T, E + groups, device=DEV), E, top, groups, keep, 1.7, ids, wts)
        W = {"p.router": torch.eye(E, dtype=torch.float64), "p.correction": corr.double()}
        chosen, weights = plain.route(z[:, :E].double(), W, "p.", {"experts": E, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}})
        got = ids.cpu().long()
        assert torch.equal(got.sort(dim=1).values, chosen.sort(dim=1).values), (E, top, groups, keep)
        want_w = torch.sigmoid(z[:, :E].double()).gather(1, got) * 1.7
        torch.testing.assert_close(wts.cpu().double(), want_w, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("T,E,top,K,N", [(1, 4, 2, 64, 40), (70, 6, 2, 48, 96), (300, 16, 4, 256, 128), (5, 3, 1, 100, 7)])
def test_grouped_expert_products(dtype, T, E, top, K, N):
    g = torch.Generator().manual_seed(T + E)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if T > 8:
        ids[:, 0] = torch.where(ids[:, 0] == 1, ids[:, 1], ids[:, 0])          # leave expert 1 almost empty
    x, w = torch.randn(T, K, generator=g).to(dtype), (torch.randn(E, N, K, generator=g) * K ** -0.5).to(dtype)
    pairs = T * top
    plan = torch.zeros(ops.moe_plan_size(E, pairs), dtype=torch.int32, device=DEV)
    place, rowp = torch.zeros(pairs, dtype=torch.int32, device=DEV), torch.zeros(pairs, dtype=torch.int32, device=DEV)
    ops.moe_plan(ids.to(DEV), E, plan, place, rowp)
    y = torch.zeros(pairs, N, dtype=dtype, device=DEV)
    ops.moe_gemm(x.to(DEV), rowp, w.to(DEV), y, plan, E)
    pl = place.cpu().long().view(T, top)
    assert sorted(pl.reshape(-1).tolist()) == list(range(pairs))
    want = torch.einsum("tk,tank->tan", x.float(), w.float()[ids.long()])        # [T, top, N]
    torch.testing.assert_close(y.float().cpu()[pl], want, **_tol(dtype))
    wts, shared, gate = torch.rand(T, top, generator=g), torch.randn(T, N, generator=g).to(dtype), torch.randn(T, 3, generator=g)[:, 1]
    out = torch.zeros(T, N, dtype=dtype, device=DEV)
    ops.moe_combine(y, place, wts.to(DEV), shared.to(DEV), gate.to(DEV), out)
    ref = (wts[:, :, None] * y.float().cpu()[pl]).sum(1) + torch.sigmoid(gate)[:, None] * shared.float()
    torch.testing.assert_close(out.float().cpu(), ref, **_tol(dtype))


# ------------------------------------------------------------------ the engine
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["Z1", "Z2", "Z3", "S", "L", "R"])
def test_cuttings_gpu(name, dtype, cut, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle(name, tmp_path_factory)
    steps = traces.mixed(reqs, seed=4) if cut == "mixed" else getattr(traces, cut)(reqs)
    ps = PAGE_SIZES[name]
    runner = ModelRunner(load_model(d, dtype, DEV), ps, traces.peak_tokens(steps) // ps, 4, device=DEV)
    got = traces.run_trace(runner, steps)
    runner.cache.check()
    assert runner.cache.num_free_slots == 4 and all(g.pool.num_free == g.pool.num_pages for g in runner.cache.groups)
    for r, want in oracle.items():
        assert_close(got[r], want, dtype, f"{name} {cut} request {r}", _rounding[id(oracle)])
    ops.check_errors(DEV)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_plain_kernel_set_and_larger_pages(dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle("Z3", tmp_path_factory)
    steps = traces.mixed(reqs, seed=9)
    for ps, ks in ((16, "plain"), (64, "fast"), (32, "fast")):
        runner = ModelRunner(load_model(d, dtype, DEV), ps, -(-traces.peak_tokens(steps) // ps), 4, device=DEV, kernel_set=ks)
        got = traces.run_trace(runner, steps)
        for r, want in oracle.items():
            assert_close(got[r], want, dtype, f"pages of {ps}, {ks} kernels, request {r}", _rounding[id(oracle)])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["Z1", "Z2", "S"])
def test_first_tokens_and_page_borders(name, dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle(name, tmp_path_factory)
    ps = PAGE_SIZES[name]
    runner = ModelRunner(load_model(d, dtype, DEV), ps, 64, 3, device=DEV)
    toks = [7, 7, 3, 150, 1]
    want = plain.forward(cfg, w, toks)
    rc = _rounding[id(oracle)]
    one_by_one = torch.cat([runner.step([StepEntry("a", [t], (0,))]).clone() for t in toks])
    together = runner.step([StepEntry("b", toks, range(5))]).clone()
    assert_close(one_by_one, want, dtype, "one by one", rc)
    assert_close(together, want, dtype, "together", rc)
    runner.end_request("a"), runner.end_request("b")
    # prompts that end exactly on a page border, one before and one after, then two decoded tokens
    long = traces.make_requests(cfg["vocab"], [4 * ps + 3], seed=2)["r0"]
    want = plain.forward(cfg, w, long)
    for n in (ps - 1, ps, ps + 1, 2 * ps, 4 * ps):
        got = [runner.step([StepEntry("c", long[:n], range(n))]).clone()]
        got += [runner.step([StepEntry("c", [long[n + i]], (0,))]).clone() for i in range(2)]
        assert_close(torch.cat(got), want[: n + 2], dtype, f"prompt of {n}", rc)
        runner.end_request("c")


def _changed(name, tmp_path, change, length, config_change=None):
    """A tiny model with some tensors changed (and, for the comparison only, a changed configuration): (folder, config,
    weights, tokens, the plain logits, what rounding costs)."""
    d = make_model_dir(name, seed=9, root=str(tmp_path))
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    t = {n: f.tensor(n).clone() for n in f.names()}
    change(t)
    write_safetensors(path, t)
    cfg, w = read_model(d)
    toks = traces.make_requests(cfg["vocab"], [length], seed=3)["r0"]
    want = plain.forward(cfg, w, toks)
    return d, cfg, w, toks, want, rounding_cost(cfg, w, toks, want)


def _run_cut(d, dtype, ps, toks, sizes):
    runner = ModelRunner(load_model(d, dtype, DEV), ps, -(-(len(toks) + 64) // ps), 2, device=DEV)
    got, at = [], 0
    for n in sizes:
        got.append(runner.step([StepEntry("r", toks[at:at + n], range(n))]).clone())
        at += n
    assert at == len(toks)
    return torch.cat(got)


def _scale(t, name, f):
    t[name] = (t[name].float() * f).to(torch.bfloat16)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("which,q_scale,o_scale", [(0, 14.0, 1.0), (1, 24.0, 6.0)])
def test_keys_at_the_windows_edges_decide_the_logits(which, q_scale, o_scale, dtype, tmp_path):
    """Random weights make attention nearly uniform, which hides a window that is one token off.  Here one layer's query
    matrix is scaled up so that its softmax picks single keys (windows of 6 and 13: the picked key is the oldest visible one
    every few positions).  The plain model with that window one longer or one shorter is far from the plain model at several
    positions, so such a fault would show; the engine is not, in prompts cut at every kind of place and in decoding."""
    def change(t):
        _scale(t, f"l{which}.mix.q", q_scale), _scale(t, f"l{which}.mix.o", o_scale)
    d, cfg, w, toks, want, rc = _changed("L", tmp_path, change, 90)
    tol = max(REL[dtype] * float(want.std()), 4.5 * rc if dtype == torch.bfloat16 else 0.0)
    for delta in (1, -1):
        off = copy.deepcopy(cfg)
        off["layers"][which]["mixer"]["mask"]["size"] += delta
        wrong = (plain.forward(off, w, toks) - want).abs().max(dim=-1).values
        assert (wrong > 3 * tol).sum() >= 2, "a window that is one off would not show"
    for sizes in ((90,), (40, 1, 1, 5, 2, 13, 6, 7) + (1,) * 15, (2,) * 10 + (3, 4, 12, 13, 14) + (1,) * 24):
        assert_close(_run_cut(d, dtype, PAGE_SIZES["L"], toks, sizes), want, dtype, f"cut {sizes[:4]}", rc)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_far_key_decides_the_logits(dtype, tmp_path):
    """A window longer than the sequence, sharpened attention, 330 tokens over many pages: late logits depend on single far
    tokens through the attention alone (the recurrent layer's output is scaled down)."""
    def change(t):
        _scale(t, "l0.mix.q", 14.0), _scale(t, "l1.mix.o", 0.05)
    d, cfg, w, toks, want, rc = _changed("F", tmp_path, change, 330)
    moved = list(toks)
    moved[5] = (moved[5] + 1) % cfg["vocab"]
    effect = (plain.forward(cfg, w, moved)[200:] - want[200:]).abs().max().item() / float(want.std())
    assert effect > 1e-2, "the sharpened layer does not look far back"
    assert_close(_run_cut(d, dtype, PAGE_SIZES["F"], toks, (130, 1, 1, 64, 2, 99, 1, 1) + (1,) * 31), want, dtype, "far", rc)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_far_token_lives_on_in_the_states(dtype, tmp_path):
    """Forget gates next to one (a large bias) and a state-space decay next to one (A_log far below zero): the states keep
    what the first tokens wrote for hundreds of steps; the attention layer's output is scaled down.  A state that is lost,
    reset or mixed up between steps shows."""
    def change(t):
        t["l0.mix.f.b"] = torch.full_like(t["l0.mix.f.b"], 9.0)
        t["l1.mix.A_log"] = torch.full_like(t["l1.mix.A_log"], -7.0)
        _scale(t, "l2.mix.o", 0.02)
    d, cfg, w, toks, want, rc = _changed("S", tmp_path, change, 250)
    moved = list(toks)
    moved[5] = (moved[5] + 1) % cfg["vocab"]
    effect = (plain.forward(cfg, w, moved)[200:] - want[200:]).abs().max().item() / float(want.std())
    assert effect > 1e-2, "the states do not remember far tokens"
    assert_close(_run_cut(d, dtype, PAGE_SIZES["S"], toks, (100, 1, 1, 64, 2, 49, 1, 1) + (1,) * 31), want, dtype, "state", rc)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_keeps_cache_and_states_exact(dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle("Z1", tmp_path_factory)
    toks = traces.make_requests(cfg["vocab"], [320], seed=8)["r0"]
    want = plain.forward(cfg, w, toks)
    runner = ModelRunner(load_model(d, dtype, DEV), 4, 8, 2, device=DEV)          # eight pages of four: the window's pages turn over
    got = [runner.step([StepEntry("r", toks[:20], range(20))]).clone()]
    got += [runner.step([StepEntry("r", [t], (0,))]).clone() for t in toks[20:]]
    assert_close(torch.cat(got), want, dtype, "300 decoded tokens", rounding_cost(cfg, w, toks, want))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_request_that_starts_again(dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle("S", tmp_path_factory)
    steps = traces.preempted(reqs)
    ps = PAGE_SIZES["S"]
    runner = ModelRunner(load_model(d, dtype, DEV), ps, traces.peak_tokens(steps) // ps, 3, device=DEV)
    for rid, pos, row in traces.run_trace_by_position(runner, steps):
        assert_close(row[None], oracle[rid][pos][None], dtype, f"{rid} at {pos}", _rounding[id(oracle)])


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("graph", [True, False], ids=["graphs", "eager"])
@pytest.mark.parametrize("name", ["F", "Z1", "R"])
def test_greedy_generation_equals_plain_model_f32(name, graph, tmp_path):
    d = make_model_dir(name, seed=3, root=str(tmp_path), sigma=0.3)
    cfg, w = read_model(d)
    prompts = [[5, 17, 3, 150, 9, 1, 1, 44, 102, 7, 7], [42] * 19, [7], list(range(20, 61))]
    ref = [plain.generate_greedy(cfg, w, p, 12) for p in prompts]
    assert all(len(set(r)) >= 3 for r in ref), "the continuation is too uniform to test anything"
    ps = PAGE_SIZES[name]
    for pages in (256 // ps, 112 // ps):                     # plenty; and (for the long window) so few that a request is preempted
        eng = Engine(d, dtype="float32", device=DEV, page_size=ps, num_pages=pages, num_slots=3, chunked_prefill_size=16,
                     max_num_batched_tokens=32, cuda_graph=graph)
        outs = eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
        assert [o.token_ids for o in outs] == ref, f"{pages} pages"
        assert not graph or eng.runner.graph_steps > 0
        eng.runner.cache.check()


def test_greedy_generation_bf16_stays_on_the_plain_models_best(tmp_path):
    """bfloat16 through the engine with CUDA graphs: every generated token is, for the plain model, the best token or within
    what rounding costs of it; and a captured step gives the tokens the same step gives when it is launched kernel by kernel."""
    d = make_model_dir("S", seed=3, root=str(tmp_path), sigma=0.2)
    cfg, w = read_model(d)
    prompts = [traces.make_requests(cfg["vocab"], [n], seed=n)["r0"] for n in (40, 3, 90, 9, 77)]
    eng = Engine(d, dtype="bfloat16", device=DEV, page_size=16, num_pages=40, num_slots=4)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    assert eng.runner.graph_steps > 0
    for p, o in zip(prompts, outs):
        toks = list(p) + o.token_ids
        lg = plain.forward(cfg, w, toks[:-1])
        slack = max(0.06 * float(lg.std()), 3 * rounding_cost(cfg, w, toks[:-1], lg))
        for i in range(len(p) - 1, len(toks) - 1):
            assert lg[i][toks[i + 1]] >= lg[i].max() - slack, (len(p), i)
    d = make_model_dir("Z3", seed=3, root=str(tmp_path))
    prompts = [traces.make_requests(512, [n], seed=n)["r0"] for n in (40, 3, 90, 9)]
    tokens = []
    for graph in (True, False):
        eng = Engine(d, dtype="bfloat16", device=DEV, page_size=16, num_pages=40, num_slots=4, cuda_graph=graph)
        tokens.append([o.token_ids for o in eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))])
        assert (eng.runner.graph_steps > 0) == graph
    assert tokens[0] == tokens[1]


# ------------------------------------------------------------------ the tools
def test_replay_tool_and_command_line(tmp_path_factory, tmp_path):
    d, cfg, w, reqs, oracle = model_and_oracle("Z2", tmp_path_factory)
    steps = traces.mixed(reqs, seed=11)
    out_dir = str(tmp_path / "out")
    p = subprocess.Popen([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out_dir, "--max-tokens",
                          str(traces.peak_tokens(steps))], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd=ROOT)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            assert p.stdout.readline().strip() == f"done {s['step']}"
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()
    at = {r: 0 for r in reqs}
    for s in steps:
        rows = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
        k = 0
        for e in s["entries"]:
            n = len(e["want"])
            assert_close(torch.from_numpy(rows[k:k + n].copy()), oracle[e["id"]][at[e["id"]]: at[e["id"]] + n], torch.float32, e["id"])
            at[e["id"]] += n
            k += n
    ref = plain.generate_greedy(cfg, w, [5, 6, 7, 8], 6)
    r = subprocess.run([sys.executable, "-m", "arle_b200", "--model-path", d, "--dtype", "float32", "--max-tokens", "6", "--ignore-eos",
                        "--num-slots", "2", "--num-pages", "16", "run", "--prompt", "5 6 7 8", "--json"], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout)["outputs"][0]["token_ids"] == ref
