"""Tiny Zuderax configurations for the tests.  Between them they vary every size and option of the design: all three
mixers in several orders, layers that share another layer's tensors (also in a chain), layers without a feed-forward,
dense and routed feed-forwards with and without a shared expert, one group and as many groups as experts, one expert
chosen and several, one head and sixteen, rotation of a part of the rotated numbers and of all of them, unrotated,
rotated and value sizes that all differ, latent sizes that are multiples of nothing, windows of one token, of a few
(not a multiple of the page) and longer than any test sequence, one and several state groups, norm parts and
convolution taps, and (Z3) sizes that fill the kernels' wider paths."""
import json
import os
import tempfile

from arle_b200.weights import write_random_model


def latent(heads, dim, rot_dim, rot_dims, vdim, rank, window, scale, base=10000.0):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                                                  "scale": scale, "mask": {"size": window}, "rot": {"base": base, "dims": rot_dims}}}


def mlstm(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, count, keep, scale, ff, shared):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale,
                                                             "groups": {"count": count, "keep": keep}},
            "shared": None if shared is None else {"ff": shared}}


def layer(mixer, mlp, weights_of=None):
    e = json.loads(json.dumps({"type": mixer["type"], "mixer": mixer["mixer"], "mlp": mlp}))      # no two layers share an object
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def model(vocab, width, eps, logit_scale, layers):
    return {"architecture": "Zuderax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}


_Z1 = [layer(latent(3, 16, 8, 8, 24, 20, 7, 0.2), dense(96)),
       layer(mlstm(2, 12, 20, 10.0), moe(6, 2, 3, 2, 1.7, 40, 48)),
       layer(mamba(4, 8, 12, 2, 4, 2), None)]
TINY_Z1 = model(211, 64, 1e-5, 1.5, _Z1 + [layer(_Z1[0], _Z1[0]["mlp"], weights_of=0), layer(_Z1[1], _Z1[1]["mlp"], weights_of=3 - 2)])
# Z2: the values that a model may happen to make equal or 1 are all different or all 1 here
TINY_Z2 = model(157, 48, 2e-6, 1.0, [
    layer(latent(1, 8, 16, 12, 40, 33, 1000, 0.3, 500.0), moe(3, 1, 1, 1, 1.0, 24, None)),
    layer(mamba(3, 16, 20, 1, 2, 1), dense(80)),
    layer(mamba(2, 12, 8, 2, 5, 4), moe(8, 4, 8, 5, 0.6, 16, 24)),
    layer(mlstm(3, 40, 8, 4.0), None),
    layer(latent(2, 4, 4, 4, 4, 8, 1, 0.5), dense(32)),
    layer(mamba(3, 16, 20, 1, 2, 1), dense(80), weights_of=1),
    layer(mamba(3, 16, 20, 1, 2, 1), dense(80), weights_of=5)])
# Z3: wider: sixteen heads (two to a warp), a latent of 128, key sizes past 128 in the recurrences, aligned rows
TINY_Z3 = model(512, 256, 1e-5, 2.5, [
    layer(latent(16, 64, 32, 32, 64, 128, 48, 0.11, 50000.0), moe(16, 4, 4, 2, 2.0, 64, 128)),
    layer(mlstm(4, 64, 64, 15.0), dense(512)),
    layer(mamba(8, 32, 144, 1, 4, 1), dense(512)),
    layer(mlstm(2, 160, 32, 8.0), None)])
# L: latent attention alone (two layers, windows of 6 and 13), for the tests that sharpen it; S: the recurrent mixers alone
TINY_L = model(180, 64, 1e-5, 1.0, [layer(latent(2, 16, 8, 8, 16, 24, 6, 0.25), dense(64)), layer(latent(4, 8, 8, 4, 12, 16, 13, 0.3), None)])
TINY_F = model(180, 64, 1e-5, 1.0, [layer(latent(2, 16, 8, 8, 16, 24, 4000, 0.25), dense(64)), layer(mlstm(2, 8, 8, 6.0), None)])
TINY_S = model(180, 64, 1e-5, 1.0, [layer(mlstm(2, 16, 12, 12.0), dense(64)), layer(mamba(2, 12, 16, 1, 3, 2), None),
                                    layer(latent(2, 8, 8, 8, 8, 12, 5, 0.3), None)])
# R: recurrent mixers only: a model without any paged cache
TINY_R = model(200, 48, 1e-5, 1.0, [layer(mlstm(2, 8, 12, 5.0), dense(32)), layer(mamba(2, 8, 8, 1, 3, 1), None)])
CONFIGS = {"R": TINY_R, "Z1": TINY_Z1, "Z2": TINY_Z2, "Z3": TINY_Z3, "L": TINY_L, "F": TINY_F, "S": TINY_S}
INIT = {"R": dict(sigma=0.2, gain_jitter=0.3), "Z1": dict(sigma=0.12, gain_jitter=0.3), "Z2": dict(sigma=0.14, gain_jitter=0.3), "Z3": dict(sigma=0.06, gain_jitter=0.3),
        "L": dict(sigma=0.12, gain_jitter=0.3), "F": dict(sigma=0.12, gain_jitter=0.3), "S": dict(sigma=0.12, gain_jitter=0.3)}
PAGE_SIZES = {"R": 16, "Z1": 4, "Z2": 8, "Z3": 16, "L": 4, "F": 16, "S": 8}


def make_model_dir(name: str, seed: int = 0, root: str = None, **init) -> str:
    root = root or tempfile.mkdtemp(prefix=f"arle_tiny_{name}_")
    kw = dict(INIT[name])
    kw.update(init)
    return write_random_model(os.path.join(root, name), CONFIGS[name], seed, **kw)


def read_model(d: str):
    """(config dict, weights by name in float64) for the plain implementation."""
    import torch
    from safetensors.torch import load_file

    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: v.to(torch.float64) for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
