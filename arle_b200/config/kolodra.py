"""Typed configuration of the Kolodra architecture, read from ``config.json``.

A Kolodra model is a list of layers (``layers``), each with one norm and two branches that
read it: a mixer made of two mixers side by side (a softmax attention whose values are its keys,
and a gated linear attention with a matrix state) and an optional dense feed-forward.  A layer
entry with ``weights_of: j`` runs with layer j's tensors and a cache and state of its own.
The embedding is scaled and the logits are capped.

Keys read here (every size and every constant that may differ between models):
``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``logit_softcap``, and per layer
``type`` ("parallel"), ``mixer.left`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``rot.base``, ``rot.dims``), ``mixer.right`` (``heads``, ``dim``, ``vdim``, ``tau``),
``mixer.left_scale``, ``mixer.right_scale``, ``mlp`` (null, or ``kind`` "dense" with ``ff``),
``weights_of``.  One size stands in no key: the rank of the decay gate is the row count of the
tensor ``l<i>.mix.right.a1``; ``from_dir`` reads it from the checkpoint's header, and a
configuration that is not backed by files (the random-weights mode) names it in
``mixer.right.decay_rank``.  Optional keys this engine adds: ``max_position`` (most tokens a
request may hold; default 1,048,576: the design has no position limit), ``bos_token_id``,
``eos_token_id``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional, Tuple

from .model_spec import ModelSpec, ScheduleEntry
from .qwen3 import ConfigError


def _get(d: dict, path: str, kind=(int, float)):
    cur = d
    for k in path.split("."):
        if not isinstance(cur, dict) or k not in cur:
            raise ConfigError(f"config.json: missing key '{path}'")
        cur = cur[k]
    if isinstance(cur, bool) or not isinstance(cur, kind):
        raise ConfigError(f"config.json: '{path}' has the wrong type ({cur!r})")
    return cur


def _pos_int(d: dict, path: str) -> int:
    v = _get(d, path, int)
    if v <= 0:
        raise ConfigError(f"config.json: '{path}' must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class KolodraLayer:
    left_heads: int
    left_kv_heads: int
    left_dim: int
    left_scale_qk: float            # score = (q . k) * this
    rot_base: float
    rot_dims: int
    right_heads: int
    right_dim: int
    right_vdim: int
    right_tau: float
    decay_rank: int
    left_scale: float               # weights of the two mixers' outputs
    right_scale: float
    ff: Optional[int]               # None: no feed-forward
    weights_of: Optional[int]       # None: own tensors


@dataclass(frozen=True)
class KolodraConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_softcap: Optional[float]
    layers: Tuple[KolodraLayer, ...]
    max_position: int = 1 << 20
    bos_token_id: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()

    architecture = "Kolodra"

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: dict, tensor_shapes: Optional[dict] = None) -> "KolodraConfig":
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            w = f"layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: {w} must be an object")
            if e.get("type") != "parallel":
                raise ConfigError(f"config.json: {w}.type = {e.get('type')!r} (this design has 'parallel' layers)")
            m = e.get("mixer")
            if not isinstance(m, dict) or not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                raise ConfigError(f"config.json: {w}.mixer needs 'left' and 'right'")
            src, hops = e.get("weights_of"), 0
            while src is not None:                    # a layer may name a layer that itself names another
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(entries) or src == i:
                    raise ConfigError(f"config.json: {w}.weights_of = {src!r} names no other layer")
                if not isinstance(entries[src], dict) or entries[src].get("weights_of") is None:
                    break
                src, hops = entries[src]["weights_of"], hops + 1
                if hops > len(entries):
                    raise ConfigError(f"config.json: {w}.weights_of leads in a circle")
            lh, lk, ld = _pos_int(m, "left.heads"), _pos_int(m, "left.kv_heads"), _pos_int(m, "left.dim")
            if lh % lk:
                raise ConfigError(f"config.json: {w}.mixer.left.heads ({lh}) must be a multiple of kv_heads ({lk})")
            if "vdim" in m["left"] and _pos_int(m, "left.vdim") != ld:
                raise ConfigError(f"config.json: {w}.mixer.left.vdim must equal dim (the values are the keys)")
            rd = _get(m, "left.rot.dims", int)
            if rd < 0 or rd % 2 or rd > ld:
                raise ConfigError(f"config.json: {w}.mixer.left.rot.dims = {rd} must be even and at most dim ({ld})")
            mlp = e.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {w}.mlp.kind = {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} (dense or null)")
                ff = _pos_int(mlp, "ff")
            rank = m["right"].get("decay_rank")
            if rank is None and tensor_shapes is not None:
                name = f"l{i if src is None else src}.mix.right.a1"
                if name not in tensor_shapes or len(tensor_shapes[name]) != 2:
                    raise ConfigError(f"the checkpoint has no matrix '{name}' to give the rank of layer {i}'s decay gate")
                rank = int(tensor_shapes[name][0])
            if isinstance(rank, bool) or not isinstance(rank, int) or rank <= 0:
                raise ConfigError(f"config.json: {w}: the rank of the decay gate is not known (mixer.right.decay_rank, "
                                  "or the shape of the layer's 'mix.right.a1' tensor)")
            tau = float(_get(m, "right.tau"))
            if not tau > 0:
                raise ConfigError(f"config.json: {w}.mixer.right.tau must be positive")
            layers.append(KolodraLayer(
                left_heads=lh, left_kv_heads=lk, left_dim=ld, left_scale_qk=float(_get(m, "left.scale")),
                rot_base=float(_get(m, "left.rot.base")), rot_dims=rd, right_heads=_pos_int(m, "right.heads"),
                right_dim=_pos_int(m, "right.dim"), right_vdim=_pos_int(m, "right.vdim"), right_tau=tau, decay_rank=rank,
                left_scale=float(_get(m, "left_scale")), right_scale=float(_get(m, "right_scale")), ff=ff, weights_of=src))
        for i, l in enumerate(layers):
            if l.weights_of is not None:
                a, b = l, layers[l.weights_of]
                same = all(getattr(a, f) == getattr(b, f) for f in a.__dataclass_fields__ if f != "weights_of")
                if not same:
                    raise ConfigError(f"config.json: layers[{i}] uses layer {l.weights_of}'s tensors but its sizes differ")
        eps = float(_get(d, "norm.eps"))
        if not eps > 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        cap = d.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or not cap > 0):
            raise ConfigError(f"config.json: 'logit_softcap' must be a positive number or null, got {cap!r}")
        eos = d.get("eos_token_id")
        stops = (eos,) if isinstance(eos, int) and not isinstance(eos, bool) else tuple(int(x) for x in eos) if isinstance(eos, list) else ()
        scale = float(_get(d, "embedding.scale")) if isinstance(d.get("embedding"), dict) and "scale" in d["embedding"] else 1.0
        return cls(vocab=_pos_int(d, "vocab"), width=_pos_int(d, "width"), embedding_scale=scale,
                   norm_eps=eps, logit_softcap=float(cap) if cap is not None else None, layers=tuple(layers),
                   max_position=_pos_int(d, "max_position") if "max_position" in d else 1 << 20,
                   bos_token_id=d.get("bos_token_id") if isinstance(d.get("bos_token_id"), int) else None,
                   stop_token_ids=stops)

    @classmethod
    def from_dir(cls, model_dir: str) -> "KolodraConfig":
        from ..weights.loader import tensor_shapes

        with open(os.path.join(model_dir, "config.json")) as f:
            d = json.load(f)
        return cls.from_dict(d, tensor_shapes(model_dir))

    # ------------------------------------------------------------------- spec
    def to_model_spec(self) -> ModelSpec:
        from ..parts.attention import AttentionSpec
        from ..parts.linear_attention import GatedLinearAttentionSpec
        from ..parts.mlp import GatedMlpSpec
        from ..parts.norm import RmsNormSpec
        from ..parts.parallel import ParallelBlockSpec, ParallelMixerSpec
        from ..parts.rotary import RotarySpec

        blocks, block_of, schedule = [], {}, []
        for i, l in enumerate(self.layers):
            if l.weights_of is None:
                p = f"l{i}."
                left = AttentionSpec(
                    prefix=p + "mix.left.", hidden_size=self.width, num_heads=l.left_heads, num_kv_heads=l.left_kv_heads,
                    head_dim=l.left_dim, scale=l.left_scale_qk, qk_norm_eps=self.norm_eps,
                    position=RotarySpec(rotary_dim=l.rot_dims, theta=l.rot_base, pairing="interleaved") if l.rot_dims else None,
                    window=None, qk_norm="row", values="keys", head_gate=True,
                    names=(("q", "q"), ("k", "k"), ("o", "o"), ("q_norm", "q.norm"), ("k_norm", "k.norm"), ("gate", "g")))
                right = GatedLinearAttentionSpec(
                    prefix=p + "mix.right.", hidden_size=self.width, num_heads=l.right_heads, key_dim=l.right_dim,
                    value_dim=l.right_vdim, decay_rank=l.decay_rank, tau=l.right_tau, norm_eps=self.norm_eps,
                    names=(("q", "q"), ("k", "k"), ("v", "v"), ("gate", "g"), ("o", "o"), ("norm", "norm"),
                           ("decay_in", "a1"), ("decay_out", "a2"), ("decay_bias", "a2.b")))
                ffn = None if l.ff is None else GatedMlpSpec(prefix=p + "mlp.", hidden_size=self.width, intermediate_size=l.ff,
                                                            activation="gelu_tanh", names=("gate", "up", "down"))
                block_of[i] = len(blocks)
                blocks.append(ParallelBlockSpec(
                    norm=RmsNormSpec(p + "norm1", self.width, self.norm_eps, one_plus=True),
                    mixer=ParallelMixerSpec(members=(left, right), scales=(l.left_scale, l.right_scale), hidden_size=self.width),
                    ffn=ffn))
        for i, l in enumerate(self.layers):
            schedule.append(ScheduleEntry(block_of[i if l.weights_of is None else l.weights_of]))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks),
            schedule=tuple(schedule), final_norm=RmsNormSpec("final.norm", self.width, self.norm_eps, one_plus=True),
            embed_name="embed", head_name="head", max_position=self.max_position, stop_token_ids=self.stop_token_ids,
            bos_token_id=self.bos_token_id, embed_scale=self.embedding_scale, logit_cap=self.logit_softcap)
