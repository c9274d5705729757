"""Tiny Kolodra configurations for the tests.  Between them they vary every size and option of the
design: layers that share another layer's tensors, a layer without feed-forward, layers of different
sizes in one model, grouped / single / full key heads, rotation of a part of the head or of all of it,
value width below, equal to and above the key width on the recurrent side, odd ranks of the decay gate,
mixer weights that are 1 and that are not, a capped and an uncapped output, a scaled and an unscaled
embedding, and (K3) sizes that the tensor-core attention and weight-streaming kernels take."""
import json
import os
import tempfile

from arle_b200.weights import write_random_model


def _layer(lh, lk, ld, rot, base, qk_scale, rh, rd, rv, tau, rank, ls, rs, ff, weights_of=None):
    e = {"type": "parallel",
         "mixer": {"left": {"heads": lh, "kv_heads": lk, "dim": ld, "vdim": ld, "scale": qk_scale, "rot": {"base": base, "dims": rot}},
                   "right": {"heads": rh, "dim": rd, "vdim": rv, "tau": tau, "decay_rank": rank},
                   "left_scale": ls, "right_scale": rs},
         "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


_K1_A = (4, 2, 16, 8, 10000.0, 0.3, 2, 24, 16, 8.0, 4, 0.7, 1.3, 96)
_K1_B = (2, 1, 24, 24, 5000.0, 0.2, 1, 8, 8, 2.0, 3, 1.5, 0.5, None)
TINY_K1 = {"architecture": "Kolodra", "vocab": 200, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-6},
           "logit_softcap": 10.0, "layers": [_layer(*_K1_A), _layer(*_K1_B), _layer(*_K1_A, weights_of=0), _layer(*_K1_B, weights_of=1)]}
_K2 = (3, 3, 32, 32, 1000000.0, 0.17677669529663687, 3, 16, 40, 4.0, 5, 1.0, 1.0, 112)
TINY_K2 = {"architecture": "Kolodra", "vocab": 301, "width": 96, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
           "logit_softcap": None, "layers": [_layer(*_K2), _layer(*_K2)]}
_K3 = (4, 1, 64, 64, 50000.0, 0.125, 2, 128, 64, 16.0, 16, 1.1, 0.8, 512)
TINY_K3 = {"architecture": "Kolodra", "vocab": 512, "width": 256, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6},
           "logit_softcap": 20.0, "layers": [_layer(*_K3), _layer(*_K3), _layer(*_K3, weights_of=0)]}
# K4: sizes that are multiples of nothing useful (width 100, head 36, odd vocabulary): every kernel's general path
_K4 = (2, 1, 36, 12, 777.0, 0.21, 3, 20, 12, 3.0, 2, 0.9, 1.1, 52)
TINY_K4 = {"architecture": "Kolodra", "vocab": 257, "width": 100, "embedding": {"scale": 2.5}, "norm": {"eps": 2e-6},
           "logit_softcap": 7.5, "layers": [_layer(*_K4), _layer(*_K4, weights_of=0), _layer(*_K4)]}
# K5: head size 128 on the softmax side (the tcgen05 prefill attention in bfloat16), a chain of shared layers
_K5 = (2, 2, 128, 128, 200000.0, 0.08838834764831845, 2, 64, 32, 32.0, 8, 1.0, 1.25, 256)
TINY_K5 = {"architecture": "Kolodra", "vocab": 640, "width": 128, "embedding": {"scale": 11.0}, "norm": {"eps": 1e-5},
           "logit_softcap": 25.0, "layers": [_layer(*_K5), _layer(*_K5, weights_of=0), _layer(*_K5, weights_of=1)]}
CONFIGS = {"K1": TINY_K1, "K2": TINY_K2, "K3": TINY_K3, "K4": TINY_K4, "K5": TINY_K5}
INIT = {"K1": dict(sigma=0.12, gain_jitter=0.2), "K2": dict(sigma=0.1, gain_jitter=0.3), "K3": dict(sigma=0.06, gain_jitter=0.2),
        "K4": dict(sigma=0.1, gain_jitter=0.2), "K5": dict(sigma=0.08, gain_jitter=0.2)}
PAGE_SIZES = {"K1": 4, "K2": 8, "K3": 16, "K4": 16, "K5": 16}


def make_model_dir(name: str, seed: int = 0, root: str = None, **init) -> str:
    """Writes the tiny model into a fresh folder.  The written config.json does not name the rank of
    the decay gate: a loader has to take it from the tensor's shape."""
    root = root or tempfile.mkdtemp(prefix=f"arle_tiny_{name}_")
    kw = dict(INIT[name])
    kw.update(init)
    d = write_random_model(os.path.join(root, name), CONFIGS[name], seed, **kw)
    cfg = json.loads(json.dumps(CONFIGS[name]))
    for e in cfg["layers"]:
        del e["mixer"]["right"]["decay_rank"]
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    return d


def read_model(d: str):
    """(config dict, weights by name in float64) for the plain implementation."""
    import torch
    from safetensors.torch import load_file

    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: v.to(torch.float64) for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
