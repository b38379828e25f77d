"""Typed configuration of the Vizonex decoder: a small decoder-only model whose layers, listed one by
one in config.json, each put BOTH sublayers on one RMS norm: with h = norm1(x),
x <- x + ls1 * mixer(h + conv(h)) + ls2 * ff(h), where conv is a short causal convolution over time on
each channel of h (only the mixer reads it) and ls1, ls2 are learned vectors over the width.  A mixer is
grouped-query attention without rotation (the whole q and the whole k projection RMS-normed with
gains, a temperature a head on the scores, keys seen inside chunks of positions counted from the
sequence's start, a softmax sink a head) or the selective state-space recurrence with a scalar decay a
head (Mamba-2).  A feed-forward is a gated one with the tanh form of gelu, or routed experts with a
clamped activation whose router scores by sigmoid, chooses on corrected scores inside the best groups
of neighbouring experts and weighs by the plain scores times a constant, plus a shared expert that
every token uses.  The embedding adds a learned vector per position; the head has a matrix of its own.

config.json keys: `architecture` ("Vizonex"), `vocab`, `width`, `max_positions`, `norm.eps`,
`canon.taps`, and `layers`: a list of {`type`, `mixer`, `mlp`}.
  type "attention": mixer {heads, kv_heads, dim, vdim, scale, mask {size} (optional: without it every
                    earlier key is seen)}
  type "mamba2":    mixer {heads, vdim, state, groups, conv, norm_groups}
  mlp: null, {kind "dense", ff} or {kind "moe", expert {ff, limit}, router {experts, top, scale,
       groups {count, keep}}, shared {ff, limit} (optional)}
Tensors: `embed`, `pos`, `l<i>.norm1`, `l<i>.canon1`, `l<i>.ls1`, `l<i>.ls2`, `l<i>.mix.*`, `l<i>.mlp.*`,
`final.norm`, `head`.  Every size is read here; none stands in the parts.
"""
from __future__ import annotations

import copy
from typing import Any, Dict, List

from .registry import register_architecture
from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec, as_float, as_int, require_keys

ARCHITECTURE = "Vizonex"
# the slope inside the sigmoid of the experts' activation: the design fixes it
EXPERT_ALPHA = 1.702


def _object(raw: Dict[str, Any], key: str, what: str) -> Dict[str, Any]:
    value = raw.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"{what}: {key} must be an object")
    return value


class VizonexConfig:
    def __init__(self, raw: Dict[str, Any]):
        self.raw = raw
        self.vocab = as_int(raw, "vocab", 1)
        self.width = as_int(raw, "width", 1)
        self.max_positions = as_int(raw, "max_positions", 1)
        self.eps = as_float(_object(raw, "norm", ARCHITECTURE), "eps")
        if self.eps < 0:
            raise ConfigError("norm.eps must not be negative")
        self.taps = as_int(_object(raw, "canon", ARCHITECTURE), "taps", 1)
        if self.taps > 16:
            raise ConfigError(f"canon.taps is at most 16, found {self.taps}")
        self.layers: List[Dict[str, Any]] = raw["layers"]
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json layers must be a list with at least one layer")
        for index, layer in enumerate(self.layers):
            self._check_layer(index, layer)

    # ---- checks ------------------------------------------------------------------------------
    @staticmethod
    def _check_attention(m: Dict[str, Any], what: str) -> None:
        require_keys(m, ["heads", "kv_heads", "dim", "vdim", "scale"], what)
        for key in ("heads", "kv_heads", "dim", "vdim"):
            as_int(m, key, 1)
        as_float(m, "scale")
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{what}: {m['heads']} heads do not divide into {m['kv_heads']} kv_heads")
        if m.get("mask") is not None:
            as_int(_object(m, "mask", what), "size", 1)

    @staticmethod
    def _check_mamba2(m: Dict[str, Any], what: str) -> None:
        require_keys(m, ["heads", "vdim", "state", "groups", "conv", "norm_groups"], what)
        for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
            as_int(m, key, 1)
        if m["heads"] % m["groups"]:
            raise ConfigError(f"{what}: {m['heads']} heads do not divide into {m['groups']} groups")
        if (m["heads"] * m["vdim"]) % m["norm_groups"]:
            raise ConfigError(f"{what}: {m['heads'] * m['vdim']} lanes do not divide into {m['norm_groups']} norm_groups")

    @staticmethod
    def _check_mlp(mlp: Any, what: str) -> None:
        if mlp is None:
            return
        if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
            raise ConfigError(f"{what}: mlp is null or an object of kind dense or moe")
        if mlp["kind"] == "dense":
            as_int(mlp, "ff", 1)
            return
        expert = _object(mlp, "expert", what + " mlp")
        as_int(expert, "ff", 1)
        as_float(expert, "limit")
        router = _object(mlp, "router", what + " mlp")
        require_keys(router, ["experts", "top", "scale"], what + " mlp.router")
        experts, top = as_int(router, "experts", 1), as_int(router, "top", 1)
        as_float(router, "scale")
        if top > experts:
            raise ConfigError(f"{what}: a token cannot use {top} of {experts} experts")
        if router.get("groups") is not None:
            groups = _object(router, "groups", what + " mlp.router")
            count, keep = as_int(groups, "count", 1), as_int(groups, "keep", 1)
            if experts % count or keep > count or keep * (experts // count) < top:
                raise ConfigError(f"{what}: {experts} experts in {count} groups of which {keep} are kept cannot give "
                                  f"a token {top} experts")
        if mlp.get("shared") is not None:
            shared = _object(mlp, "shared", what + " mlp")
            as_int(shared, "ff", 1)
            as_float(shared, "limit")

    @classmethod
    def _check_layer(cls, index: int, layer: Dict[str, Any]) -> None:
        what = f"{ARCHITECTURE} layer {index}"
        if not isinstance(layer, dict):
            raise ConfigError(f"{what} must be an object")
        require_keys(layer, ["type", "mixer"], what)
        m = _object(layer, "mixer", what)
        if layer["type"] == "attention":
            cls._check_attention(m, what + " mixer")
        elif layer["type"] == "mamba2":
            cls._check_mamba2(m, what + " mixer")
        else:
            raise ConfigError(f"{what}: unknown type {layer['type']!r} (known: attention, mamba2)")
        cls._check_mlp(layer.get("mlp"), what)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "VizonexConfig":
        require_keys(raw, ["vocab", "width", "max_positions", "layers", "norm", "canon"], ARCHITECTURE)
        return cls(copy.deepcopy(raw))

    def to_dict(self) -> Dict[str, Any]:
        out = copy.deepcopy(self.raw)
        out.pop("architectures", None)
        out["architecture"] = ARCHITECTURE
        return out

    # ---- the model as data -------------------------------------------------------------------
    def _mixer(self, index: int, layer: Dict[str, Any]) -> PartSpec:
        m, prefix = layer["mixer"], f"l{index}.mix"
        if layer["type"] == "mamba2":
            return PartSpec("mamba2", {"hidden_size": self.width, "heads": m["heads"], "vdim": m["vdim"],
                                       "state": m["state"], "groups": m["groups"], "conv": m["conv"],
                                       "norm_groups": m["norm_groups"], "eps": self.eps}, prefix)
        return PartSpec("gqa_rotary", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
            "vdim": m["vdim"], "scale": float(m["scale"]), "bias": False, "window": None,
            "chunk": int(m["mask"]["size"]) if m.get("mask") is not None else None, "position": None,
            "qk_norm": True, "norm_eps": self.eps, "head_temperature": True, "sink": True}, prefix)

    def _feed_forward(self, index: int, mlp: Dict[str, Any]) -> PartSpec:
        prefix = f"l{index}.mlp"
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"],
                                          "activation": "gelu_pytorch_tanh", "names": (".gate", ".up", ".down")}, prefix)
        router, shared = mlp["router"], mlp.get("shared")
        groups = router.get("groups") or {"count": 1, "keep": 1}
        return PartSpec("routed_mlp", {
            "hidden_size": self.width, "experts": router["experts"], "top": router["top"],
            "expert_inner": mlp["expert"]["ff"], "shared_inner": shared["ff"] if shared is not None else 0,
            "shared_gate": False, "score": "sigmoid", "correction": True, "groups": groups["count"],
            "group_keep": groups["keep"], "route_scale": float(router["scale"]), "activation": "clamped_swish",
            "limit": float(mlp["expert"]["limit"]), "shared_limit": float(shared["limit"]) if shared is not None else 0.0,
            "alpha": EXPERT_ALPHA}, prefix)

    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rms_norm", {"size": self.width, "eps": self.eps, "tensor": name}, name)

    def _scale(self, name: str) -> PartSpec:
        return PartSpec("layer_scale", {"hidden_size": self.width, "tensor": name}, name)

    def model_spec(self) -> ModelSpec:
        layers = []
        for index, layer in enumerate(self.layers):
            p = f"l{index}"
            parts = dict(mixer=self._mixer(index, layer), mixer_norm=self._norm(p + ".norm1"),
                         mixer_filter=PartSpec("causal_conv_residual", {"hidden_size": self.width, "taps": self.taps,
                                                                        "tensor": p + ".canon1"}, p + ".canon1"),
                         mixer_scale=self._scale(p + ".ls1"))
            if layer.get("mlp") is None:
                layers.append(LayerSpec("parallel_residual_mixer_only", **parts))
                continue
            parts.update(feed_forward=self._feed_forward(index, layer["mlp"]), feed_forward_scale=self._scale(p + ".ls2"))
            layers.append(LayerSpec("parallel_residual", **parts))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "tensor": "embed",
                                                   "position_tensor": "pos", "positions": self.max_positions}, "embed"),
            layers=tuple(layers), order=tuple(LayerCall(i) for i in range(len(layers))),
            final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tensor": "head"}, "head"))
        spec.validate()
        return spec


register_architecture(ARCHITECTURE, VizonexConfig)
