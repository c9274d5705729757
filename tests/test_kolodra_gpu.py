"""Kolodra on the GPU against the plain implementation (``plain_kolodra``): every new kernel alone at
sizes other than any model's, the parts, the engine under every cutting in float32 and bfloat16 on three
tiny configurations, the first tokens of a sequence and prompts that end on page borders, far tokens made
to matter (through the attention and through the recurrent state), long decoding, a request that starts
again, greedy generation through the public entry point with CUDA graphs and preemption, and the replay
tool and the command line as subprocesses."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kernel_refs
import plain_kolodra as plain
import traces
from arle_b200 import Engine, ops
from arle_b200.engine import ModelRunner, StepEntry, load_model
from arle_b200.sampling import SamplingParams
from arle_b200.weights import SafetensorsFile, write_safetensors
from tiny_kolodra import CONFIGS, PAGE_SIZES, make_model_dir, read_model

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
# error of a logits row as a fraction of the spread of the plain model's logits: float32 rounding through a few
# layers.  In bfloat16 the engine's worst position may be off by 4.5 times what the plain model's worst is off by when
# every activation it stores is rounded to bfloat16 (``plain.stored_as``): how much rounding costs depends on the model
# and the prompt, and two ways of rounding the same sums differ by more than either differs from the exact result.
REL = {torch.float32: 5e-4, torch.bfloat16: 1e-2}
LENGTHS = {"K1": [1, 5, 12, 23, 70, 130, 33], "K2": [2, 17, 40, 96, 64, 31], "K3": [3, 66, 150, 64, 40, 97],
           "K4": [2, 33, 80, 17, 64], "K5": [3, 150, 64, 290, 31]}
_cache = {}


def model_and_oracle(name, tmp_path_factory):
    if name not in _cache:
        d = make_model_dir(name, seed=21, root=str(tmp_path_factory.mktemp(f"tiny{name}")))
        cfg, w = read_model(d)
        reqs = traces.make_requests(cfg["vocab"], LENGTHS[name], seed=6)
        oracle = {r: plain.forward(w, cfg, t) for r, t in reqs.items()}
        _cache[name] = (d, cfg, w, reqs, oracle)
        _rounding[id(oracle)] = max(rounding_cost(w, cfg, t, oracle[r]) for r, t in reqs.items())
    return _cache[name]


_rounding = {}


def rounding_cost(w, cfg, toks, exact) -> float:
    with plain.stored_as(torch.bfloat16):
        return (plain.forward(w, cfg, toks) - exact).abs().max().item()


def assert_close(got, want, dtype, what="", rounding=0.0):
    err = (got.double().cpu() - want).abs().max(dim=-1).values
    tol = REL[dtype] * float(want.std())
    if dtype == torch.bfloat16:
        tol = max(tol, 4.5 * rounding)
    assert err.max().item() <= tol, f"{what}: first wrong position {int((err > tol).nonzero()[0])}, error {err.max().item():.3g}, tolerance {tol:.3g}"


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("pairing", ["interleaved", "half"])
@pytest.mark.parametrize("nq,nkv,hd,rdim,keys", [(4, 2, 16, 8, True), (3, 3, 40, 40, True), (5, 1, 24, 0, False), (8, 2, 128, 64, True)])
def test_attention_prep_row_kernel(dtype, pairing, nq, nkv, hd, rdim, keys):
    g = torch.Generator().manual_seed(nq * 100 + hd)
    T, ps, pages = 37, 8, 9
    width = (nq + (nkv if keys else 2 * nkv)) * hd + 5
    qk = torch.randn(T, width, generator=g).to(dtype)
    pos = torch.randint(0, 3000, (T,), generator=g, dtype=torch.int32)
    slots = torch.randperm(ps * pages, generator=g)[:T].to(torch.int32)
    slots[3] = -1
    qw, kw = torch.rand(nq * hd, generator=g) + 0.5, torch.rand(nkv * hd, generator=g) + 0.5
    inv = (10000.0 ** (-2.0 * torch.arange(rdim // 2, dtype=torch.float64) / max(rdim, 1))).float()
    caches = [torch.zeros(pages, nkv, ps, hd, dtype=dtype) for _ in range(4)]
    ref_qk = qk.clone()
    kernel_refs.attention_prep_row(ref_qk, pos, slots, qw, kw, 1e-5, inv, rdim, pairing, keys, caches[0], caches[1], nq, nkv, hd, ps)
    dqk, dk, dv = qk.to(DEV), caches[2].to(DEV), caches[3].to(DEV)
    ops.attention_prep_row(dqk, pos.to(DEV), slots.to(DEV), qw.to(DEV), kw.to(DEV), 1e-5, inv.to(DEV), rdim, pairing, keys, dk, dv,
                           nq, nkv, hd, ps)
    tol = 2e-6 if dtype == torch.float32 else 2e-2
    assert (dqk.cpu().float() - ref_qk.float()).abs().max() < tol * 4
    assert (dk.cpu().float() - caches[0].float()).abs().max() < tol * 4
    assert torch.equal(dv.cpu(), caches[1])                                    # values are copied bit for bit
    if pairing == "interleaved" and dtype == torch.float32:
        # and against the plain model's own functions
        q = plain.rms(qk[:, : nq * hd].double(), 1e-5) * qw.double()
        q = plain.rotate_interleaved(q.view(T, nq, hd), pos, 10000.0, rdim) if rdim else q.view(T, nq, hd)
        # a float32 angle at position 3,000 is off by up to 3,000 * 2^-24 rad
        assert (dqk.cpu()[:, : nq * hd].double() - q.reshape(T, nq * hd)).abs().max() < 1e-3


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_small_gating_kernels(dtype):
    g = torch.Generator().manual_seed(1)
    T, H, hd = 19, 3, 20
    x, gate = torch.randn(T, H * hd + 4, generator=g).to(dtype), torch.randn(T, H + 3, generator=g).to(dtype)
    out = torch.zeros(T, 2 * H * hd, dtype=dtype, device=DEV)
    ops.head_gate(x.to(DEV)[:, 4:], gate.to(DEV)[:, 1: 1 + H], 1.7, out[:, H * hd:], H, hd)
    want = (x[:, 4:].double().view(T, H, hd) * plain.sigmoid(gate[:, 1: 1 + H].double())[:, :, None] * 1.7).reshape(T, H * hd)
    tol = 1e-6 if dtype == torch.float32 else 2e-2
    assert (out[:, H * hd:].cpu().double() - want).abs().max() < tol * 8 and not out[:, : H * hd].any()
    ops.head_gate(x.to(DEV)[:, 4:], None, 0.5, out[:, : H * hd], H, hd)
    assert (out[:, : H * hd].cpu().double() - 0.5 * x[:, 4:].double()).abs().max() < tol * 4
    a, b = torch.randn(T, 33, generator=g).to(dtype), torch.randn(T, 33, generator=g).to(dtype)
    s = torch.zeros(T, 33, dtype=dtype, device=DEV)
    ops.weighted_sum(a.to(DEV), 1.2, b.to(DEV), -0.9, s)
    assert (s.cpu().double() - (1.2 * a.double() - 0.9 * b.double())).abs().max() < tol * 8
    gu = torch.randn(T, 2 * 35, generator=g).mul(3).to(dtype)
    act = torch.zeros(T, 35, dtype=dtype, device=DEV)
    ops.act_mul(gu.to(DEV), act, "gelu_tanh")
    assert (act.cpu().double() - plain.gelu_tanh(gu[:, 0::2].double()) * gu[:, 1::2].double()).abs().max() < tol * 16
    gu8 = torch.randn(T, 2 * 40, generator=g).mul(3).to(dtype)                  # a width the vector kernel takes
    act8 = torch.zeros(T, 40, dtype=dtype, device=DEV)
    ops.act_mul(gu8.to(DEV), act8, "gelu_tanh")
    assert (act8.cpu().double() - plain.gelu_tanh(gu8[:, 0::2].double()) * gu8[:, 1::2].double()).abs().max() < tol * 16
    ops.act_mul(gu8.to(DEV), act8, "silu")
    assert (act8.cpu().double() - plain.silu(gu8[:, 0::2].double()) * gu8[:, 1::2].double()).abs().max() < tol * 16
    if dtype == torch.float32:
        lg = torch.randn(T, 77, generator=g).mul(30)
        dl = lg.to(DEV)
        ops.logit_cap(dl, 15.0)
        assert (dl.cpu().double() - 15.0 * torch.tanh(lg.double() / 15.0)).abs().max() < 5e-6
    table = torch.randn(50, 24, generator=g).to(dtype)
    ids = torch.randint(0, 50, (T,), generator=g, dtype=torch.int32)
    e = torch.zeros(T, 24, dtype=torch.float32, device=DEV)
    ops.embedding(ids.to(DEV), table.to(DEV), e, scale=5.5)
    assert (e.cpu().double() - plain.embedding(table.double(), ids, 5.5)).abs().max() < 1e-5


@pytest.mark.parametrize("rows,K,inter", [(1, 256, 96), (8, 512, 320), (5, 96, 40), (40, 256, 96), (1100, 256, 384)])
def test_gated_products_with_the_gelu_gate(rows, K, inter):
    """The first half of the feed-forward with gelu on the gate, through whichever kernel the shapes choose: the
    weight-streaming product (up to 8 rows), the two-SM tcgen05 product (from 1,024 rows), or product and gate kernel."""
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, generator=g) * K ** -0.5 * 2).to(torch.bfloat16)
    gu = torch.zeros(rows, 2 * inter, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(rows, inter, dtype=torch.bfloat16, device=DEV)
    before = ops.launch_count()
    ops.gemm_act_mul(x.to(DEV), w.to(DEV), gu, out, "gelu_tanh")
    assert ops.launch_count() - before == (1 if rows <= 8 and K % 32 == 0 or rows >= 1024 else 2) or rows > 8
    y = x.double() @ w.double().t()
    want = plain.gelu_tanh(y[:, 0::2]) * y[:, 1::2]
    assert (out.cpu().double() - want).abs().max() < 3e-2 * max(1.0, float(want.abs().max()))
    ops.check_errors(DEV)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("heads,dim,vdim,rank,tau", [(2, 24, 16, 4, 8.0), (3, 16, 40, 5, 4.0), (2, 128, 64, 16, 16.0), (1, 50, 72, 3, 1.0),
                                                     (1, 8, 8, 1, 2.0), (2, 200, 33, 7, 32.0)])
def test_recurrent_side_kernels(dtype, heads, dim, vdim, rank, tau):
    """decay, scan and output norm against the plain recurrent side: three requests of unequal length in one
    batch, then each continued in a second step from the state the first left, on slots given in any order."""
    g = torch.Generator().manual_seed(dim + vdim)
    D, eps = 32, 1e-5
    m = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    shapes = {"q": (heads * dim, D), "k": (heads * dim, D), "v": (heads * vdim, D), "g": (heads * vdim, D), "a1": (rank, D),
              "a2": (heads * dim, rank), "a2.b": (heads * dim,), "norm": (vdim,)}
    w = {"p." + n: (torch.randn(s, generator=g) * (0.5 if len(s) > 1 else 1.0)).to(torch.bfloat16).double() for n, s in shapes.items()}
    w["p.o"] = torch.eye(heads * vdim, dtype=torch.float64)
    lens = [(13, 21), (1, 1), (40, 2)]
    xs = [torch.randn(a + b, D, generator=g).to(dtype) for a, b in lens]
    want = [plain.recurrent_side(x.double(), w, "p.", m, eps)[0] for x in xs]
    w_in = torch.cat([w["p." + n] for n in ("q", "k", "v", "g", "a1")]).to(dtype)
    state = torch.randn(5, heads, vdim, dim, generator=g).to(DEV)               # stale numbers in every slot
    slots = torch.tensor([3, 0, 4], dtype=torch.int32)
    state[slots.long()] = 0
    dq, dv = heads * dim, heads * vdim
    got = [[], [], []]
    for part in (0, 1):
        rows = [x[: a] if part == 0 else x[a:] for x, (a, b) in zip(xs, lens)]
        x = torch.cat(rows)
        T = x.shape[0]
        proj = (x.float() @ w_in.float().t()).to(dtype).to(DEV)
        ind = torch.tensor([0] + list(np.cumsum([r.shape[0] for r in rows])), dtype=torch.int32, device=DEV)
        alpha = torch.zeros(T, dq, device=DEV)
        ops.gla_decay(proj[:, 2 * dq + 2 * dv:], w["p.a2"].float().t().contiguous().to(DEV), w["p.a2.b"].float().to(DEV), tau, alpha)
        a_want = plain.decay(x.double(), w, "p.", m).reshape(T, dq)
        assert (alpha.cpu().double() - a_want).abs().max() < (2e-6 if dtype == torch.float32 else 2e-2)
        o = torch.zeros(T, dv, device=DEV)
        ops.gla_scan(proj[:, :dq], proj[:, dq: 2 * dq], proj[:, 2 * dq: 2 * dq + dv], alpha, state, ind, slots.to(DEV), o, heads, dim,
                     vdim, dim ** -0.5, max(r.shape[0] for r in rows))
        out = torch.zeros(T, dv + 8, dtype=dtype, device=DEV)
        ops.gla_out(o, proj[:, 2 * dq + dv: 2 * dq + 2 * dv], w["p.norm"].float().to(DEV), eps, 1.0, out[:, 8:], heads, vdim)
        at = 0
        for i, r in enumerate(rows):
            got[i].append(out[at: at + r.shape[0], 8:].cpu())
            at += r.shape[0]
    for i in range(3):
        err = (torch.cat(got[i]).double() - want[i]).abs().max().item()
        assert err < (3e-5 if dtype == torch.float32 else 6e-2) * max(1.0, float(want[i].abs().max())), (i, err)
    assert state[1].cpu().equal(state[1].cpu()) and float(state[[1, 2]].abs().min()) > 0      # other slots untouched


# ------------------------------------------------------------------ the engine
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["K1", "K2", "K3", "K4", "K5"])
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
    d, cfg, w, reqs, oracle = model_and_oracle("K3", tmp_path_factory)
    steps = traces.mixed(reqs, seed=9)
    for ps, ks in ((16, "plain"), (64, "fast"), (32, "fast")):
        runner = ModelRunner(load_model(d, dtype, DEV), ps, -(-traces.peak_tokens(steps) // ps), 4, device=DEV, kernel_set=ks)
        got = traces.run_trace(runner, steps)
        for r, want in oracle.items():
            assert_close(got[r], want, dtype, f"pages of {ps}, {ks} kernels, request {r}", _rounding[id(oracle)])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["K1", "K2", "K3"])
def test_first_tokens_and_page_borders(name, dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle(name, tmp_path_factory)
    ps = PAGE_SIZES[name]
    runner = ModelRunner(load_model(d, dtype, DEV), ps, 64, 3, device=DEV)
    toks = [7, 7, 3, 150, 1]
    want = plain.forward(w, cfg, toks)
    rc = _rounding[id(oracle)]
    one_by_one = torch.cat([runner.step([StepEntry("a", [t], (0,))]).clone() for t in toks])
    together = runner.step([StepEntry("b", toks, range(5))]).clone()
    assert_close(one_by_one, want, dtype, "one by one", rc)
    assert_close(together, want, dtype, "together", rc)
    runner.end_request("a"), runner.end_request("b")
    # prompts that end exactly on a page border, one before and one after, then two decoded tokens
    long = traces.make_requests(cfg["vocab"], [4 * ps + 3], seed=2)["r0"]
    want = plain.forward(w, cfg, long)
    for n in (ps - 1, ps, ps + 1, 2 * ps, 4 * ps):
        got = [runner.step([StepEntry("c", long[:n], range(n))]).clone()]
        got += [runner.step([StepEntry("c", [long[n + i]], (0,))]).clone() for i in range(2)]
        assert_close(torch.cat(got), want[: n + 2], dtype, f"prompt of {n}", rc)
        runner.end_request("c")


def _sharpened(name, tmp_path, change):
    d = make_model_dir(name, seed=9, root=str(tmp_path))
    path = os.path.join(d, "model.safetensors")
    f = SafetensorsFile(path)
    t = {n: f.tensor(n).clone() for n in f.names()}
    change(t)
    write_safetensors(path, t)
    cfg, w = read_model(d)
    toks = traces.make_requests(cfg["vocab"], [330], seed=3)["r0"]
    want = plain.forward(w, cfg, toks)
    moved = list(toks)
    moved[5] = (moved[5] + 1) % cfg["vocab"]
    effect = (plain.forward(w, cfg, moved)[-1] - want[-1]).abs().max().item() / float(want.std())
    return d, cfg, w, toks, want, effect, rounding_cost(w, cfg, toks, want)


def _run_cut(d, dtype, ps, toks):
    runner = ModelRunner(load_model(d, dtype, DEV), ps, -(-384 // ps), 2, device=DEV)
    got, at = [], 0
    for n in (130, 1, 1, 64, 2, 99, 1, 1) + (1,) * 31:
        got.append(runner.step([StepEntry("r", toks[at:at + n], range(n))]).clone())
        at += n
    assert at == len(toks)
    return torch.cat(got)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["K2", "K3"])
def test_a_far_key_decides_the_logits(name, dtype, tmp_path):
    """Random weights make attention nearly uniform, which hides a lost page or a wrong position.  Here the weights of
    the q norm of layer 0 are scaled up so that the softmax side is sharp and the recurrent side's output is scaled
    down; the late logits then depend on single far tokens through the attention alone."""
    def change(t):
        t["l0.mix.left.q.norm"] = (t["l0.mix.left.q.norm"].float() * 12).to(torch.bfloat16)
        t["l0.mix.right.o"] = (t["l0.mix.right.o"].float() * 0.05).to(torch.bfloat16)
    d, cfg, w, toks, want, effect, rc = _sharpened(name, tmp_path, change)
    assert effect > 1e-3, "the sharpened layer does not look far back"
    assert_close(_run_cut(d, dtype, PAGE_SIZES[name], toks), want, dtype, name, rc)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["K1", "K3"])
def test_a_far_token_lives_on_in_the_state(name, dtype, tmp_path):
    """With a large bias on the decay gate the decay is next to one, so the state keeps what the first tokens wrote for
    hundreds of steps; the softmax side is scaled down.  A state that is lost, reset or mixed up between steps shows."""
    def change(t):
        for l in ("l0", "l1"):
            t[f"{l}.mix.right.a2.b"] = (t[f"{l}.mix.right.a2.b"].float() * 0 + 6.0).to(torch.bfloat16)
            t[f"{l}.mix.left.o"] = (t[f"{l}.mix.left.o"].float() * 0.02).to(torch.bfloat16)
    d, cfg, w, toks, want, effect, rc = _sharpened(name, tmp_path, change)
    assert effect > 1e-3, "the state does not remember far tokens"
    assert_close(_run_cut(d, dtype, PAGE_SIZES[name], toks), want, dtype, name, rc)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_keeps_the_state_exact(dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle("K3", tmp_path_factory)
    toks = traces.make_requests(cfg["vocab"], [420], seed=8)["r0"]
    want = plain.forward(w, cfg, toks)
    runner = ModelRunner(load_model(d, dtype, DEV), 16, 28, 2, device=DEV)
    got = [runner.step([StepEntry("r", toks[:20], range(20))]).clone()]
    got += [runner.step([StepEntry("r", [t], (0,))]).clone() for t in toks[20:]]
    assert_close(torch.cat(got), want, dtype, "400 decoded tokens", rounding_cost(w, cfg, toks, want))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_request_that_starts_again(dtype, tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle("K1", tmp_path_factory)
    steps = traces.preempted(reqs)
    runner = ModelRunner(load_model(d, dtype, DEV), 4, traces.peak_tokens(steps) // 4, 3, device=DEV)
    for rid, pos, row in traces.run_trace_by_position(runner, steps):
        assert_close(row[None], oracle[rid][pos][None], dtype, f"{rid} at {pos}", _rounding[id(oracle)])


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("graph", [True, False], ids=["graphs", "eager"])
@pytest.mark.parametrize("name", ["K1", "K3"])
def test_greedy_generation_equals_plain_model_f32(name, graph, tmp_path):
    d = make_model_dir(name, seed=3, root=str(tmp_path), sigma=0.3 if name == "K1" else 0.12)
    cfg, w = read_model(d)
    prompts = [[5, 17, 3, 150, 9, 1, 1, 44, 102, 7, 7], [42] * 19, [7], list(range(20, 61))]
    ref = [plain.generate_greedy(w, cfg, p, 12) for p in prompts]
    assert all(len(set(r)) >= 3 for r in ref), "the continuation is too uniform to test anything"
    ps = PAGE_SIZES[name]
    for pages in (256 // ps, 112 // ps):                     # plenty; and so few that a request is preempted
        eng = Engine(d, dtype="float32", device=DEV, page_size=ps, num_pages=pages, num_slots=3, chunked_prefill_size=16,
                     max_num_batched_tokens=32, cuda_graph=graph)
        outs = eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
        assert [o.token_ids for o in outs] == ref, f"{pages} pages"
        assert not graph or eng.runner.graph_steps > 0
        eng.runner.cache.check()


def test_greedy_generation_bf16_stays_on_the_plain_models_best(tmp_path):
    d = make_model_dir("K3", seed=3, root=str(tmp_path), sigma=0.12)
    cfg, w = read_model(d)
    prompts = [traces.make_requests(cfg["vocab"], [n], seed=n)["r0"] for n in (40, 3, 150, 9, 77)]
    eng = Engine(d, dtype="bfloat16", device=DEV, page_size=16, num_pages=40, num_slots=4)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=16, ignore_eos=True))
    assert eng.runner.graph_steps > 0
    for p, o in zip(prompts, outs):
        toks = list(p) + o.token_ids
        lg = plain.forward(w, cfg, toks[:-1])
        for i in range(len(p) - 1, len(toks) - 1):
            assert lg[i][toks[i + 1]] >= lg[i].max() - 0.06 * float(lg.std()), (len(p), i)


# ------------------------------------------------------------------ the tools
def test_replay_tool_and_command_line(tmp_path_factory, tmp_path):
    d, cfg, w, reqs, oracle = model_and_oracle("K2", tmp_path_factory)
    steps = traces.mixed(reqs, seed=11)
    out_dir = str(tmp_path / "out")
    p = subprocess.Popen([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out_dir, "--max-tokens",
                          str(traces.peak_tokens(steps)), "--max-live", "4"], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd=ROOT)
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
    ref = plain.generate_greedy(w, cfg, [5, 6, 7, 8], 6)
    r = subprocess.run([sys.executable, "-m", "arle_b200", "--model-path", d, "--dtype", "float32", "--max-tokens", "6", "--ignore-eos",
                        "--num-slots", "2", "--num-pages", "16", "run", "--prompt", "5 6 7 8", "--json"], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout)["outputs"][0]["token_ids"] == ref
