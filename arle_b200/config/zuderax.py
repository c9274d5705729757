"""Typed configuration of the Zuderax architecture, read from ``config.json``.

A Zuderax model is a list of pre-norm layers (``layers``): x <- x + mixer(norm1(x)), then x <- x + ff(norm2(x)), the norms
Dynamic Tanh (no statistics; a stored scalar and a bias beside the weight).  A layer's ``type`` names its mixer:

* ``latent_attention``: attention over a cached latent per token (``heads``, ``dim`` unrotated and ``rot_dim`` rotated
  query/key numbers per head, ``vdim``, ``kv_rank``, ``scale``, ``rot.base``, ``rot.dims``, ``mask.size``: the sliding window);
* ``mlstm``: the matrix memory of xLSTM (``heads``, ``dim``, ``vdim``, ``gate_cap``);
* ``mamba2``: the state-space duality layer (``heads``, ``vdim``, ``state``, ``groups``, ``conv``, ``norm_groups``).

``mlp`` is null, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale",
"groups": {"count", "keep"}}, "shared": {"ff"} or null}``.  A layer entry with ``weights_of: j`` runs with layer j's tensors
and a cache or state of its own.  Around the layers: ``vocab``, ``width``, ``norm.eps`` (of the RMS norms inside the mixers),
``logit_scale``; the output projection is the tensor ``head``.  Optional keys this engine adds: ``max_position`` (default
1,048,576: the design has no position limit), ``bos_token_id``, ``eos_token_id``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional, Tuple

from .kolodra import _get, _pos_int
from .model_spec import ModelSpec, ScheduleEntry
from .qwen3 import ConfigError

MIXER_TYPES = ("latent_attention", "mlstm", "mamba2")


@dataclass(frozen=True)
class ZuderaxMlp:
    kind: str                       # "dense" or "moe"
    ff: int                         # dense: its size; moe: an expert's
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    route_scale: float = 1.0
    shared_ff: Optional[int] = None


@dataclass(frozen=True)
class ZuderaxLayer:
    type: str
    mixer: Tuple[Tuple[str, object], ...]     # the mixer's sizes and constants, by the names in the module's docstring
    mlp: Optional[ZuderaxMlp]
    weights_of: Optional[int]

    def m(self, key: str):
        return dict(self.mixer)[key]


def _mixer(kind: str, m: dict, w: str) -> Tuple[Tuple[str, object], ...]:
    def fail(msg):
        raise ConfigError(f"config.json: {w}.mixer: {msg}")

    def num(path):
        try:
            return float(_get(m, path))
        except ConfigError as e:
            raise ConfigError(str(e).replace("missing key '", f"missing key '{w}.mixer.").replace("config.json: '", f"config.json: '{w}.mixer.")) from None

    def pos(path):
        try:
            return _pos_int(m, path)
        except ConfigError as e:
            raise ConfigError(str(e).replace("missing key '", f"missing key '{w}.mixer.").replace("config.json: '", f"config.json: '{w}.mixer.")) from None

    if kind == "latent_attention":
        out = {k: pos(k) for k in ("heads", "vdim", "kv_rank")}
        for k in ("dim", "rot_dim"):
            v = _get(m, k, int) if k in m else fail(f"missing key '{k}'")
            if v < 0:
                fail(f"'{k}' must not be negative")
            out[k] = v
        if out["dim"] + out["rot_dim"] <= 0:
            fail("'dim' + 'rot_dim' must be positive")
        out["scale"] = num("scale")
        out["window"] = pos("mask.size")
        out["rot_base"], out["rot_dims"] = (num("rot.base"), _get(m, "rot.dims", int)) if out["rot_dim"] else (1.0, 0)
        if out["rot_dims"] < 0 or out["rot_dims"] % 2 or out["rot_dims"] > out["rot_dim"]:
            fail(f"'rot.dims' = {out['rot_dims']} must be even and at most rot_dim ({out['rot_dim']})")
        if out["rot_dims"] and not out["rot_base"] > 0:
            fail("'rot.base' must be positive")
    elif kind == "mlstm":
        out = {k: pos(k) for k in ("heads", "dim", "vdim")}
        out["gate_cap"] = num("gate_cap")
        if not out["gate_cap"] > 0:
            fail("'gate_cap' must be positive")
    else:
        out = {k: pos(k) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")}
        if out["heads"] % out["groups"]:
            fail(f"'heads' ({out['heads']}) must be a multiple of 'groups' ({out['groups']})")
        if (out["heads"] * out["vdim"]) % out["norm_groups"]:
            fail(f"heads * vdim ({out['heads'] * out['vdim']}) must be a multiple of 'norm_groups' ({out['norm_groups']})")
    return tuple(sorted(out.items()))


def _mlp(mlp, w: str) -> Optional[ZuderaxMlp]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {w}.mlp.kind = {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} (dense, moe or null)")

    def pos(path):
        try:
            return _pos_int(mlp, path)
        except ConfigError as e:
            raise ConfigError(str(e).replace("'", f"'{w}.mlp.", 1)) from None

    if mlp["kind"] == "dense":
        return ZuderaxMlp("dense", pos("ff"))
    experts, top = pos("router.experts"), pos("router.top")
    groups = mlp["router"].get("groups")
    count, keep = (pos("router.groups.count"), pos("router.groups.keep")) if groups is not None else (1, 1)
    if experts % count or keep > count or top > keep * (experts // count):
        raise ConfigError(f"config.json: {w}.mlp.router: {experts} experts do not split into {count} groups of which {keep} are kept "
                          f"and hold the {top} chosen")
    scale = float(_get(mlp, "router.scale")) if "scale" in mlp["router"] else 1.0
    shared = mlp.get("shared")
    return ZuderaxMlp("moe", pos("expert.ff"), experts, top, count, keep, scale, pos("shared.ff") if shared is not None else None)


@dataclass(frozen=True)
class ZuderaxConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: Tuple[ZuderaxLayer, ...]
    max_position: int = 1 << 20
    bos_token_id: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()

    architecture = "Zuderax"

    @classmethod
    def from_dict(cls, d: dict) -> "ZuderaxConfig":
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            w = f"layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: {w} must be an object")
            if e.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: {w}.type = {e.get('type')!r} (this design has {', '.join(MIXER_TYPES)})")
            if not isinstance(e.get("mixer"), dict):
                raise ConfigError(f"config.json: {w}.mixer must be an object")
            src, hops = e.get("weights_of"), 0
            while src is not None:                    # a layer may name a layer that itself names another
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(entries) or src == i:
                    raise ConfigError(f"config.json: {w}.weights_of = {src!r} names no other layer")
                if not isinstance(entries[src], dict) or entries[src].get("weights_of") is None:
                    break
                src, hops = entries[src]["weights_of"], hops + 1
                if hops > len(entries):
                    raise ConfigError(f"config.json: {w}.weights_of leads in a circle")
            layers.append(ZuderaxLayer(e["type"], _mixer(e["type"], e["mixer"], w), _mlp(e.get("mlp"), w), src))
        for i, l in enumerate(layers):
            if l.weights_of is not None:
                o = layers[l.weights_of]
                if (l.type, l.mixer, l.mlp) != (o.type, o.mixer, o.mlp):
                    raise ConfigError(f"config.json: layers[{i}] uses layer {l.weights_of}'s tensors but its sizes differ")
        eps = float(_get(d, "norm.eps"))
        if not eps > 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        eos = d.get("eos_token_id")
        stops = (eos,) if isinstance(eos, int) and not isinstance(eos, bool) else tuple(int(x) for x in eos) if isinstance(eos, list) else ()
        return cls(vocab=_pos_int(d, "vocab"), width=_pos_int(d, "width"), norm_eps=eps,
                   logit_scale=float(_get(d, "logit_scale")) if "logit_scale" in d else 1.0, layers=tuple(layers),
                   max_position=_pos_int(d, "max_position") if "max_position" in d else 1 << 20,
                   bos_token_id=d.get("bos_token_id") if isinstance(d.get("bos_token_id"), int) else None, stop_token_ids=stops)

    @classmethod
    def from_dir(cls, model_dir: str) -> "ZuderaxConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    # ------------------------------------------------------------------- spec
    def _mixer_spec(self, l: ZuderaxLayer, p: str):
        from ..parts.latent_attention import LatentAttentionSpec
        from ..parts.mamba2 import Mamba2Spec
        from ..parts.mlstm import MatrixLstmSpec
        from ..parts.rotary import RotarySpec

        if l.type == "latent_attention":
            return LatentAttentionSpec(
                prefix=p, hidden_size=self.width, num_heads=l.m("heads"), nope_dim=l.m("dim"), rope_dim=l.m("rot_dim"),
                value_dim=l.m("vdim"), kv_rank=l.m("kv_rank"), scale=l.m("scale"), norm_eps=self.norm_eps,
                position=RotarySpec(rotary_dim=l.m("rot_dims"), theta=l.m("rot_base"), pairing="half") if l.m("rot_dims") else None,
                window=l.m("window"))
        if l.type == "mlstm":
            return MatrixLstmSpec(prefix=p, hidden_size=self.width, num_heads=l.m("heads"), key_dim=l.m("dim"), value_dim=l.m("vdim"),
                                  gate_cap=l.m("gate_cap"), norm_eps=self.norm_eps)
        return Mamba2Spec(prefix=p, hidden_size=self.width, num_heads=l.m("heads"), head_dim=l.m("vdim"), state_dim=l.m("state"),
                          groups=l.m("groups"), conv_taps=l.m("conv"), norm_groups=l.m("norm_groups"), norm_eps=self.norm_eps)

    def _mlp_spec(self, mlp: ZuderaxMlp, p: str):
        from ..parts.mlp import GatedMlpSpec
        from ..parts.moe import RoutedExpertsSpec

        names = ("gate", "up", "down")
        if mlp.kind == "dense":
            return GatedMlpSpec(prefix=p, hidden_size=self.width, intermediate_size=mlp.ff, activation="silu", names=names)
        shared = None if mlp.shared_ff is None else GatedMlpSpec(prefix=p + "shared.", hidden_size=self.width,
                                                                 intermediate_size=mlp.shared_ff, activation="silu", names=names)
        return RoutedExpertsSpec(prefix=p, hidden_size=self.width, num_experts=mlp.experts, top=mlp.top, expert_ff=mlp.ff,
                                 groups=mlp.groups, keep=mlp.keep, route_scale=mlp.route_scale, correction=True, shared=shared,
                                 shared_gate=shared is not None, activation="silu")

    def to_model_spec(self) -> ModelSpec:
        from ..parts.block import PreNormBlockSpec
        from ..parts.norm import DynTanhSpec

        blocks, block_of, schedule, ignored = [], {}, [], []
        for i, l in enumerate(self.layers):
            if l.weights_of is None:
                p = f"l{i}."
                block_of[i] = len(blocks)
                if l.mlp is None:               # a layer without a feed-forward has no use for a second norm, should one be stored
                    ignored += [p + "norm2", p + "norm2.b", p + "norm2.alpha"]
                blocks.append(PreNormBlockSpec(
                    mixer_norm=DynTanhSpec(p + "norm1", self.width), mixer=self._mixer_spec(l, p + "mix."),
                    ffn_norm=DynTanhSpec(p + "norm2", self.width) if l.mlp is not None else None,
                    ffn=self._mlp_spec(l.mlp, p + "mlp.") if l.mlp is not None else None))
        for i, l in enumerate(self.layers):
            schedule.append(ScheduleEntry(block_of[i if l.weights_of is None else l.weights_of]))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks),
            schedule=tuple(schedule), final_norm=DynTanhSpec("final.norm", self.width), embed_name="embed", head_name="head",
            max_position=self.max_position, stop_token_ids=self.stop_token_ids, bos_token_id=self.bos_token_id,
            ignored_tensors=tuple(ignored), logit_scale=self.logit_scale)
