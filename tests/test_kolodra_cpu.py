"""Kolodra without a GPU: the configuration reader and what it refuses, the model as the registry
builds it (layers that share tensors, caches and states of their own), the plain implementation's own
checks, and the engine around the kernels (cache pages, state slots, step function, scheduler) under
every way of cutting the work, with the kernels replaced by their torch statements."""
import copy
import json
import os

import pytest
import torch

import plain_kolodra as plain
import traces
from arle_b200.config import ConfigError, KolodraConfig, config_from_dict, load_config
from arle_b200 import Engine
from arle_b200.engine import ModelRunner, StepEntry, load_model
from arle_b200.parts import build_model
from arle_b200.sampling import SamplingParams
from tiny_kolodra import CONFIGS, PAGE_SIZES, make_model_dir, read_model

LENGTHS = {"K1": [1, 5, 12, 23, 70, 33], "K2": [2, 17, 40, 64, 9, 31]}
_cache = {}


def model_and_oracle(name, tmp_path_factory):
    if name not in _cache:
        d = make_model_dir(name, seed=21, root=str(tmp_path_factory.mktemp(f"tiny{name}")))
        cfg, w = read_model(d)
        reqs = traces.make_requests(cfg["vocab"], LENGTHS[name], seed=6)
        _cache[name] = (d, cfg, w, reqs, {r: plain.forward(w, cfg, t) for r, t in reqs.items()})
    return _cache[name]


# ------------------------------------------------------------------ configuration
def test_registry_finds_the_architecture_by_its_single_name():
    cfg = config_from_dict(CONFIGS["K1"])
    assert isinstance(cfg, KolodraConfig) and len(cfg.layers) == 4 and cfg.layers[2].weights_of == 0
    assert cfg.layers[1].ff is None and cfg.layers[0].ff == 96 and cfg.logit_softcap == 10.0


def test_model_spec_shares_blocks_but_not_caches_or_states():
    spec = config_from_dict(CONFIGS["K1"]).to_model_spec()
    assert len(spec.blocks) == 2 and [e.block for e in spec.schedule] == [0, 1, 0, 1]
    model = build_model(spec)
    assert len(model.cache_needs) == 4 and len(model.state_needs) == 4          # one per layer run
    assert model.state_needs[0].shape == (2, 16, 24) and model.state_needs[1].shape == (1, 8, 8)
    names = {d.name for d in model.weight_decls()}
    assert "l0.mix.left.q.norm" in names and "l1.mix.right.a2.b" in names and not any(n.startswith("l2.") for n in names)
    assert "l1.mlp.gate" not in names and "l0.mlp.down" in names


def test_a_chain_of_shared_layers_ends_at_the_layer_with_tensors():
    cfg = config_from_dict(CONFIGS["K5"])
    assert [l.weights_of for l in cfg.layers] == [None, 0, 0]
    assert [e.block for e in cfg.to_model_spec().schedule] == [0, 0, 0]


def test_decay_rank_comes_from_the_tensor_when_the_config_does_not_name_it(tmp_path):
    d = make_model_dir("K2", seed=1, root=str(tmp_path))
    with open(os.path.join(d, "config.json")) as f:
        assert "decay_rank" not in json.dumps(json.load(f))
    assert load_config(d).layers[0].decay_rank == 5
    with pytest.raises(ConfigError, match="rank"):
        stripped = copy.deepcopy(CONFIGS["K2"])
        del stripped["layers"][0]["mixer"]["right"]["decay_rank"]
        config_from_dict(stripped)


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="serial"), "type"),
    (lambda c: (c["layers"][2].update(weights_of=3), c["layers"][3].update(weights_of=2)), "circle|no other layer"),
    (lambda c: c["layers"][2]["mixer"]["left"].update(heads=8), "sizes differ"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "mlp"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
])
def test_configuration_errors_name_the_key(change, match):
    c = copy.deepcopy(CONFIGS["K1"])
    change(c)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(c)


# ------------------------------------------------------------ the plain implementation
def test_plain_recurrence_equals_its_closed_form():
    """o_t = sum_{s<=t} (q_t * prod_{s<u<=t} alpha_u) . k_s  v_s: the recurrence unrolled."""
    g = torch.Generator().manual_seed(0)
    T, D = 9, 12
    m = {"heads": 2, "dim": 4, "vdim": 3, "tau": 2.0}
    w = {"p.q": torch.randn(8, D, generator=g, dtype=plain.DT), "p.k": torch.randn(8, D, generator=g, dtype=plain.DT),
         "p.v": torch.randn(6, D, generator=g, dtype=plain.DT), "p.g": torch.randn(6, D, generator=g, dtype=plain.DT),
         "p.o": torch.eye(6, dtype=plain.DT), "p.norm": torch.ones(3, dtype=plain.DT),
         "p.a1": torch.randn(2, D, generator=g, dtype=plain.DT), "p.a2": torch.randn(8, 2, generator=g, dtype=plain.DT),
         "p.a2.b": torch.randn(8, generator=g, dtype=plain.DT)}
    n = torch.randn(T, D, generator=g, dtype=plain.DT)
    got, S = plain.recurrent_side(n, w, "p.", m, 1e-6)
    a = plain.decay(n, w, "p.", m)
    q = (n @ w["p.q"].T).reshape(T, 2, 4) * 0.5
    k, v = (n @ w["p.k"].T).reshape(T, 2, 4), (n @ w["p.v"].T).reshape(T, 2, 3)
    o = torch.zeros(T, 2, 3, dtype=plain.DT)
    for t in range(T):
        for s in range(t + 1):
            o[t] += ((q[t] * a[s + 1:t + 1].prod(dim=0) * k[s]).sum(-1))[:, None] * v[s]
    want = (plain.rms(o, 1e-6).reshape(T, 6)) * plain.silu(n @ w["p.g"].T)
    assert (got - want).abs().max() < 1e-10
    # the state after a prefix continues the sequence
    first, S5 = plain.recurrent_side(n[:5], w, "p.", m, 1e-6)
    rest, _ = plain.recurrent_side(n[5:], w, "p.", m, 1e-6, state=S5)
    assert (torch.cat([first, rest]) - got).abs().max() < 1e-12


def test_plain_rotation_keeps_lengths_and_turns_only_the_first_dims():
    x = torch.randn(5, 2, 12, dtype=plain.DT)
    y = plain.rotate_interleaved(x, torch.arange(3, 8), 100.0, 8)
    assert torch.equal(y[..., 8:], x[..., 8:]) and (y.norm(dim=-1) - x.norm(dim=-1)).abs().max() < 1e-12
    assert torch.equal(plain.rotate_interleaved(x, torch.zeros(5, dtype=torch.long), 100.0, 8), x)
    # q.k after rotation depends on the distance only
    a, b = x[:1, :1], x[1:2, :1]
    d1 = (plain.rotate_interleaved(a, torch.tensor([7]), 100.0, 12) * plain.rotate_interleaved(b, torch.tensor([4]), 100.0, 12)).sum()
    d2 = (plain.rotate_interleaved(a, torch.tensor([13]), 100.0, 12) * plain.rotate_interleaved(b, torch.tensor([10]), 100.0, 12)).sum()
    assert abs(d1 - d2) < 1e-10


def test_plain_model_is_causal_and_shared_layers_use_the_named_tensors(tmp_path_factory):
    d, cfg, w, reqs, oracle = model_and_oracle("K1", tmp_path_factory)
    t = reqs["r4"]
    assert (plain.forward(w, cfg, t[:30]) - oracle["r4"][:30]).abs().max() < 1e-9
    assert plain.layer_prefix(cfg, 2) == "l0." and plain.layer_prefix(cfg, 1) == "l1."
    assert float(oracle["r4"].abs().max()) < cfg["logit_softcap"]


# ------------------------------------------------------------------ the engine on the CPU
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
@pytest.mark.parametrize("name", ["K1", "K2"])
def test_cuttings_cpu(name, cut, tmp_path_factory, cpu_kernels):
    d, cfg, w, reqs, oracle = model_and_oracle(name, tmp_path_factory)
    steps = traces.mixed(reqs, seed=4) if cut == "mixed" else getattr(traces, cut)(reqs)
    ps = PAGE_SIZES[name]
    runner = ModelRunner(load_model(d, torch.float32, "cpu"), ps, traces.peak_tokens(steps) // ps, 4, device="cpu")
    got = traces.run_trace(runner, steps)
    runner.cache.check()
    assert runner.cache.num_free_slots == 4 and all(g.pool.num_free == g.pool.num_pages for g in runner.cache.groups)
    for r, want in oracle.items():
        err = (got[r].double() - want).abs().max().item()
        assert err < 5e-4 * float(want.std()), f"{name} {cut}: request {r}, error {err:.3g}"


def test_a_request_that_starts_again_starts_from_an_empty_state(tmp_path_factory, cpu_kernels):
    d, cfg, w, reqs, oracle = model_and_oracle("K1", tmp_path_factory)
    steps = traces.preempted(reqs)
    runner = ModelRunner(load_model(d, torch.float32, "cpu"), 4, traces.peak_tokens(steps) // 4, 3, device="cpu")
    seen = 0
    for rid, pos, row in traces.run_trace_by_position(runner, steps):
        assert (row.double() - oracle[rid][pos]).abs().max() < 5e-4 * float(oracle[rid].std()), (rid, pos)
        seen += 1
    assert seen > sum(len(t) for t in reqs.values())          # the victim's first half came out twice


@pytest.mark.parametrize("pages", [64, 14])
def test_greedy_generation_through_the_engine_and_scheduler(pages, tmp_path_factory, cpu_kernels):
    """The public entry point: prompts of unequal length, portions of eight tokens, and (with 14 pages) so few
    pages that a request is preempted and recomputed, state and all."""
    d = make_model_dir("K1", seed=3, root=str(tmp_path_factory.mktemp("gen")), sigma=0.3)
    cfg, w = read_model(d)
    prompts = [[5, 17, 3, 150, 9, 1, 1, 44, 102, 7, 7], [42] * 19, [7]]
    ref = [plain.generate_greedy(w, cfg, p, 10) for p in prompts]
    assert all(len(set(r)) >= 3 for r in ref), "the continuation is too uniform to test anything"
    eng = Engine(d, dtype="float32", device="cpu", page_size=4, num_pages=pages, num_slots=3, chunked_prefill_size=8,
                 max_num_batched_tokens=16, cuda_graph=False)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=10, ignore_eos=True))
    assert [o.token_ids for o in outs] == ref
    if pages == 14:
        assert sum(o.preemptions for o in outs) > 0
    eng.runner.cache.check()
