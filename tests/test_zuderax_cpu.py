"""Zuderax without a GPU: the configuration reader and what it refuses, the model as the registry builds it (layers that
share tensors, caches and states of their own), the plain implementation's own checks (each recurrence against its sum
written out, the routing rules on made-up scores, the window), and the engine around the kernels (cache pages, state
slots, step function, scheduler) under every way of cutting the work, with the kernels replaced by their torch
statements."""
import copy
import math

import pytest
import torch

import plain_zuderax as plain
import traces
from arle_b200 import Engine
from arle_b200.config import ConfigError, ZuderaxConfig, config_from_dict
from arle_b200.engine import ModelRunner, StepEntry, load_model
from arle_b200.parts import build_model
from arle_b200.sampling import SamplingParams
from tiny_zuderax import CONFIGS, PAGE_SIZES, make_model_dir, read_model

LENGTHS = {"Z1": [1, 5, 12, 23, 70, 33], "Z2": [2, 17, 40, 64, 9, 31], "S": [3, 30, 11, 2, 45], "R": [1, 20, 33, 7]}
F64 = torch.float64
_cache = {}


def model_and_oracle(name, tmp_path_factory):
    if name not in _cache:
        d = make_model_dir(name, seed=21, root=str(tmp_path_factory.mktemp(f"tiny{name}")))
        cfg, w = read_model(d)
        reqs = traces.make_requests(cfg["vocab"], LENGTHS[name], seed=6)
        _cache[name] = (d, cfg, w, reqs, {r: plain.forward(cfg, w, t) for r, t in reqs.items()})
    return _cache[name]


# ------------------------------------------------------------------ configuration
def test_registry_finds_the_architecture_and_reads_every_size():
    cfg = config_from_dict(CONFIGS["Z1"])
    assert isinstance(cfg, ZuderaxConfig) and [l.type for l in cfg.layers] == ["latent_attention", "mlstm", "mamba2", "latent_attention", "mlstm"]
    assert cfg.layers[3].weights_of == 0 and cfg.layers[4].weights_of == 1 and cfg.layers[2].mlp is None
    assert cfg.layers[0].m("window") == 7 and cfg.layers[0].m("kv_rank") == 20 and cfg.layers[1].m("gate_cap") == 10.0
    assert cfg.layers[1].mlp.experts == 6 and cfg.layers[1].mlp.keep == 2 and cfg.layers[1].mlp.shared_ff == 48
    assert cfg.logit_scale == 1.5 and cfg.norm_eps == 1e-5


def test_model_spec_shares_blocks_but_not_caches_or_states():
    spec = config_from_dict(CONFIGS["Z2"]).to_model_spec()
    assert len(spec.blocks) == 5 and [e.block for e in spec.schedule] == [0, 1, 2, 3, 4, 1, 1]      # a chain ends at the layer with tensors
    model = build_model(spec)
    assert len(model.cache_needs) == 2 and len(model.state_needs) == 5                              # one per layer run
    assert model.cache_needs[0].arrays() == ((1, 33 + 16),) and model.cache_needs[0].window == 1000 and model.cache_needs[1].window == 1
    names = {d.name for d in model.weight_decls()}
    assert {"l0.mix.dkv.norm", "l2.mlp.e7.down", "l2.mlp.shared.sg", "l3.mix.f.b", "l1.mix.A_log", "final.norm.alpha", "head"} <= names
    assert not any(n.startswith(("l5.", "l6.", "l3.mlp", "l3.norm2", "l0.mlp.shared")) for n in names)


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: (c["layers"][3].update(weights_of=4), c["layers"][4].update(weights_of=3)), "circle|no other layer"),
    (lambda c: c["layers"][3]["mixer"].update(heads=5), "sizes differ"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0), "gate_cap"),
    (lambda c: c["layers"][2]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][2]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][0].update(mlp={"kind": "sparse", "ff": 8}), "mlp"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "chosen"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_configuration_errors_name_the_key(change, match):
    c = copy.deepcopy(CONFIGS["Z1"])
    change(c)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(c)


# ------------------------------------------------------------ the plain implementation
def _rand(g, *shape):
    return torch.randn(*shape, generator=g, dtype=F64)


def test_plain_matrix_lstm_equals_its_sum_written_out():
    """Without the running maximum: S~_t = sum_s exp(i_s + f_(s+1) + .. + f_t) k_s v_s^T, n~ likewise, and
    o_t = S~^T q / (max(|n~ . q|, 1) + 1e-6 e^(m_t))."""
    g = torch.Generator().manual_seed(0)
    T, D, H, dk, dv, cap = 11, 10, 2, 3, 4, 5.0
    W = {"p.q": _rand(g, H * dk, D), "p.k": _rand(g, H * dk, D), "p.v": _rand(g, H * dv, D), "p.g": _rand(g, H * dv, D),
         "p.o": torch.eye(H * dv, dtype=F64), "p.norm": torch.ones(H * dv, dtype=F64), "p.i": _rand(g, H, D), "p.i.b": _rand(g, H),
         "p.f": _rand(g, H, D), "p.f.b": _rand(g, H) + 2}
    h = _rand(g, T, D)
    got = plain.mlstm(h, W, "p.", {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}, 1e-6)
    q, k, v = (h @ W["p.q"].T).view(T, H, dk) * dk ** -0.5, (h @ W["p.k"].T).view(T, H, dk), (h @ W["p.v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ W["p.i"].T + W["p.i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ W["p.f"].T + W["p.f.b"]) / cap))
    o = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        m = 0.0
        for t in range(T):
            m = max(float(gf[t, a]) + m, float(gi[t, a]))
            num, den = torch.zeros(dv, dtype=F64), 0.0
            for s in range(t + 1):
                wgt = math.exp(float(gi[s, a]) + float(gf[s + 1: t + 1, a].sum())) * float(q[t, a] @ k[s, a])
                num, den = num + wgt * v[s, a], den + wgt
            o[t, a] = num / (max(abs(den), 1.0) + 1e-6 * math.exp(m))
    want = plain.rms_unit(o, 1e-6).reshape(T, H * dv) * torch.sigmoid(h @ W["p.g"].T)
    assert (got - want).abs().max() < 1e-9


def test_plain_state_space_layer_equals_its_sum_written_out():
    g = torch.Generator().manual_seed(1)
    T, D, H, P, N, G, taps = 9, 8, 4, 3, 5, 2, 3
    inner, C = H * P, H * P + 2 * G * N
    m = {"heads": H, "vdim": P, "state": N, "groups": G, "conv": taps, "norm_groups": 2}
    W = {"p.in": _rand(g, 2 * inner + 2 * G * N + H, D) * 0.5, "p.conv": _rand(g, C, taps), "p.conv.b": _rand(g, C), "p.dt_bias": _rand(g, H),
         "p.A_log": _rand(g, H) * 0.3, "p.D": _rand(g, H), "p.norm": torch.ones(inner, dtype=F64), "p.o": torch.eye(inner, dtype=F64)}
    h = _rand(g, T, D)
    got = plain.mamba2(h, W, "p.", m, 1e-6)
    proj = h @ W["p.in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner: inner + C], torch.nn.functional.softplus(proj[:, inner + C:] + W["p.dt_bias"])
    conv = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(taps):
            if t - (taps - 1) + j >= 0:
                conv[t] += W["p.conv"][:, j] * xbc[t - (taps - 1) + j]
    xbc = plain.silu(conv + W["p.conv.b"])
    x, B, Cm = xbc[:, :inner].view(T, H, P), xbc[:, inner: inner + G * N].view(T, G, N), xbc[:, inner + G * N:].view(T, G, N)
    la = -torch.exp(W["p.A_log"])[None, :] * dt                     # log of the decay
    y = torch.zeros(T, H, P, dtype=F64)
    for a in range(H):
        grp = a // (H // G)
        for t in range(T):
            for s in range(t + 1):
                y[t, a] += math.exp(float(la[s + 1: t + 1, a].sum())) * float(dt[s, a]) * float(Cm[t, grp] @ B[s, grp]) * x[s, a]
            y[t, a] += W["p.D"][a] * x[t, a]
    want = plain.rms_unit((y.reshape(T, inner) * plain.silu(z)).view(T, 2, inner // 2), 1e-6).reshape(T, inner)
    assert (got - want).abs().max() < 1e-9


def test_plain_routing_rules_on_made_up_scores():
    """Eight experts in four pairs; router sums chosen so that the rules show: the correction decides the choice but not the
    weight; a group counts by its two best; experts outside the kept groups lose to kept ones with negative choice scores."""
    E = 8
    W = {"p.router": torch.eye(E, dtype=F64), "p.correction": torch.tensor([0, 0, 0, 0, 0, 0, 0, 0.4], dtype=F64) - 3.0}
    r = {"experts": E, "top": 3, "scale": 2.0, "groups": {"count": 4, "keep": 2}}
    logit = lambda s: math.log(s / (1 - s))
    #            group 0      group 1      group 2      group 3
    s = [0.90, 0.10,  0.60, 0.55,  0.80, 0.05,  0.20, 0.30]
    chosen, weights = plain.route(torch.tensor([[logit(v) for v in s]], dtype=F64), W, "p.", r)
    # group scores (each minus 6): 1.00, 1.15, 0.85, 0.90 (0.2 + 0.3 + 0.4): groups 1 and 0 are kept
    assert sorted(chosen[0].tolist()) == [0, 2, 3]
    assert torch.allclose(weights[0].sort().values, torch.tensor([0.55, 0.60, 0.90], dtype=F64) * 2.0)
    # every choice score is negative (about -2 to -3); expert 4 (0.80) stands outside the kept groups and is not chosen
    W["p.correction"][7] = -3.0 + 0.9                                 # now group 3 scores 1.40 and is kept with group 1
    chosen, _ = plain.route(torch.tensor([[logit(v) for v in s]], dtype=F64), W, "p.", r)
    assert sorted(chosen[0].tolist()) == [2, 3, 7]


def test_plain_window_sees_itself_and_the_tokens_before_it(tmp_path):
    d = make_model_dir("L", seed=5, root=str(tmp_path))
    cfg, w = read_model(d)
    toks = traces.make_requests(cfg["vocab"], [40], seed=1)["r0"]
    base = plain.forward(cfg, w, toks)
    # a token more than (6 - 1) + (13 - 1) places back cannot reach position 20 through two windowed layers; one 17 back can
    for back, reaches in ((18, False), (17, True)):
        moved = list(toks)
        moved[20 - back] = (moved[20 - back] + 1) % cfg["vocab"]
        diff = (plain.forward(cfg, w, moved)[20] - base[20]).abs().max().item()
        assert (diff > 1e-9) == reaches, (back, diff)
    assert (plain.forward(cfg, w, toks[:25]) - base[:25]).abs().max() < 1e-12          # causal


# ------------------------------------------------------------------ the engine on the CPU
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
@pytest.mark.parametrize("name", ["Z1", "Z2", "R"])
def test_cuttings_cpu(name, cut, tmp_path_factory, cpu_kernels):
    d, cfg, w, reqs, oracle = model_and_oracle(name, tmp_path_factory)
    steps = traces.mixed(reqs, seed=4) if cut == "mixed" else getattr(traces, cut)(reqs)
    ps = PAGE_SIZES[name]
    runner = ModelRunner(load_model(d, torch.float32, "cpu"), ps, max(1, traces.peak_tokens(steps) // ps), 4, device="cpu")
    got = traces.run_trace(runner, steps)
    runner.cache.check()
    assert runner.cache.num_free_slots == 4 and all(g.pool.num_free == g.pool.num_pages for g in runner.cache.groups)
    for r, want in oracle.items():
        err = (got[r].double() - want).abs().max().item()
        assert err < 5e-4 * float(want.std()), f"{name} {cut}: request {r}, error {err:.3g}"


def test_window_pages_go_back_while_the_request_lives(tmp_path_factory, cpu_kernels):
    d, cfg, w, reqs, oracle = model_and_oracle("Z1", tmp_path_factory)
    runner = ModelRunner(load_model(d, torch.float32, "cpu"), 4, 40, 2, device="cpu")
    toks = reqs["r4"]
    runner.step([StepEntry("a", toks[:50], ())])
    held = [g.pool.num_pages - g.pool.num_free for g in runner.cache.groups]
    assert held == [2]                      # a window of 7: the pages of the last 6 tokens (44..49), not all 13
    lg = runner.step([StepEntry("a", toks[50:], range(20))])
    assert (lg.double() - oracle["r4"][50:]).abs().max() < 5e-4 * float(oracle["r4"].std())


def test_a_request_that_starts_again_starts_from_an_empty_state(tmp_path_factory, cpu_kernels):
    d, cfg, w, reqs, oracle = model_and_oracle("S", tmp_path_factory)
    steps = traces.preempted(reqs)
    ps = PAGE_SIZES["S"]
    runner = ModelRunner(load_model(d, torch.float32, "cpu"), ps, traces.peak_tokens(steps) // ps, 3, device="cpu")
    seen = 0
    for rid, pos, row in traces.run_trace_by_position(runner, steps):
        assert (row.double() - oracle[rid][pos]).abs().max() < 5e-4 * float(oracle[rid].std()), (rid, pos)
        seen += 1
    assert seen > sum(len(t) for t in reqs.values())          # the victim's first half came out twice


@pytest.mark.parametrize("pages", [64, 14])
def test_greedy_generation_through_the_engine_and_scheduler(pages, tmp_path_factory, cpu_kernels):
    """The public entry point: prompts of unequal length, portions of eight tokens, and (with 14 pages) so few pages that a
    request is preempted and recomputed, cache, state and all (a model whose window is longer than the requests, so that
    no page goes back early)."""
    d = make_model_dir("F", seed=3, root=str(tmp_path_factory.mktemp("gen")), sigma=0.3)
    cfg, w = read_model(d)
    prompts = [[5, 17, 3, 150, 9, 1, 1, 44, 102, 7, 7], [42] * 19, [7]]
    ref = [plain.generate_greedy(cfg, w, p, 10) for p in prompts]
    assert all(len(set(r)) >= 3 for r in ref), "the continuation is too uniform to test anything"
    eng = Engine(d, dtype="float32", device="cpu", page_size=4, num_pages=pages, num_slots=3, chunked_prefill_size=8,
                 max_num_batched_tokens=16, cuda_graph=False)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=10, ignore_eos=True))
    assert [o.token_ids for o in outs] == ref
    if pages == 14:
        assert sum(o.preemptions for o in outs) > 0
    eng.runner.cache.check()


def test_generation_with_a_model_that_keeps_no_paged_cache(tmp_path_factory, cpu_kernels):
    """Recurrent mixers only: the cache manager has state slots and no page group; the scheduler admits by slots alone."""
    d = make_model_dir("R", seed=3, root=str(tmp_path_factory.mktemp("gen")), sigma=0.3)
    cfg, w = read_model(d)
    prompts = [[5, 6, 7, 8], [9] * 12, [3], [100, 2, 50]]
    eng = Engine(d, dtype="float32", device="cpu", page_size=4, num_pages=8, num_slots=2, chunked_prefill_size=8,
                 max_num_batched_tokens=16, cuda_graph=False)
    assert not eng.runner.cache.groups and len(eng.runner.cache.states) == 2
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert [o.token_ids for o in outs] == [plain.generate_greedy(cfg, w, p, 6) for p in prompts]

