"""Typed configuration of the Zobelorn decoder: a small decoder-only model whose layers are listed in
config.json one by one.  Every sublayer has an RMS norm in front of it and one behind it, each with a
gain of one plus its tensor (the file holds the offset from one), and what the norm behind gives is multiplied by one
constant of the model before it is added: x <- x + m * post(f(pre(x))).  A layer's mixer is one of two
kinds of grouped-query attention.  "attention": the whole q and the whole k projection RMS-normed with
gains, the half layout of the rotation on the leading lanes of every head with every frequency divided
by a factor, scores squashed by cap * tanh(score / cap), a sliding window, and a sigmoid gate (one more
projection of the mixer's input) on the heads' outputs.  "attention_2": the interleaved layout of the
rotation with frequencies rescaled by bands of wavelength, queries and keys divided by their root mean
square a head after the rotation, keys seen inside chunks of positions counted from the sequence's
start; such a layer may take keys and values from an earlier layer's cache and project queries only.
A feed-forward is a gated one with silu, or routed experts whose router scores by sigmoid, takes the
`top` largest and multiplies each chosen expert's INPUT by its score, plus a shared expert that every
token uses.  The embedding is scaled by a constant; the head has a matrix of its own.

config.json keys: `architecture` ("Zobelorn"), `vocab`, `width`, `norm.eps`, `embedding.scale`
(optional), `residual_mult` (optional), and `layers`: a list of {`type`, `mixer`, `mlp`}.
  type "attention":   mixer {heads, kv_heads, dim, vdim, scale, softcap (optional), mask {size} (optional),
                      rot {base, dims, scaling {factor} (optional)} (optional)}
  type "attention_2": mixer {heads, kv_heads, dim, vdim, scale, mask {size} (optional), rot {base, dims,
                      scaling {factor, low, high, original} (optional)} (optional), kv_from (optional)}
  mlp: null, {kind "dense", ff} or {kind "moe", expert {ff}, router {experts, top}, shared {ff} (optional)}
Tensors: `embed`, `l<i>.norm1`, `.norm1b`, `.norm2`, `.norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`,
`head`.  Every size is read here; none stands in the parts.
"""
from __future__ import annotations

import copy
import math
from typing import Any, Dict, List, Optional

from .registry import register_architecture
from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec, as_float, as_int, require_keys

ARCHITECTURE = "Zobelorn"
# The design has no longest position (angles are computed, not tabulated); what the engine uses
# as its bound on a request's length.
POSITIONS = 1 << 20


def _object(raw: Dict[str, Any], key: str, what: str) -> Dict[str, Any]:
    value = raw.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"{what}: {key} must be an object")
    return value


class ZobelornConfig:
    def __init__(self, raw: Dict[str, Any]):
        self.raw = raw
        self.vocab = as_int(raw, "vocab", 1)
        self.width = as_int(raw, "width", 1)
        self.eps = as_float(_object(raw, "norm", ARCHITECTURE), "eps")
        if self.eps < 0:
            raise ConfigError("norm.eps must not be negative")
        embedding = raw.get("embedding")
        self.embedding_scale = as_float(embedding, "scale") if isinstance(embedding, dict) and "scale" in embedding else 1.0
        self.residual_mult = as_float(raw, "residual_mult") if raw.get("residual_mult") is not None else 1.0
        self.layers: List[Dict[str, Any]] = raw["layers"]
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json layers must be a list with at least one layer")
        for index, layer in enumerate(self.layers):
            self._check_layer(index, layer)

    # ---- checks ------------------------------------------------------------------------------
    @staticmethod
    def _check_rot(m: Dict[str, Any], what: str, banded: bool) -> None:
        if m.get("rot") is None:
            return
        rot = _object(m, "rot", what)
        require_keys(rot, ["base", "dims"], what + " rot")
        dims = as_int(rot, "dims", 2)
        if dims % 2 or dims > m["dim"] or as_float(rot, "base") <= 0:
            raise ConfigError(f"{what}: rot.dims must be even and at most dim, rot.base positive")
        if rot.get("scaling") is None:
            return
        scaling = _object(rot, "scaling", what + " rot")
        keys = ["factor", "low", "high", "original"] if banded else ["factor"]
        require_keys(scaling, keys, what + " rot.scaling")
        if any(as_float(scaling, key) <= 0 for key in keys):
            raise ConfigError(f"{what}: the numbers of rot.scaling must be positive")
        if banded and scaling["high"] == scaling["low"]:
            raise ConfigError(f"{what}: rot.scaling low and high must differ")

    def _check_mixer(self, index: int, kind: str, m: Dict[str, Any], what: str) -> None:
        require_keys(m, ["heads", "kv_heads", "dim", "vdim", "scale"], what)
        for key in ("heads", "kv_heads", "dim", "vdim"):
            as_int(m, key, 1)
        as_float(m, "scale")
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{what}: {m['heads']} heads do not divide into {m['kv_heads']} kv_heads")
        if m.get("mask") is not None:
            as_int(_object(m, "mask", what), "size", 1)
        self._check_rot(m, what, banded=kind == "attention_2")
        if kind == "attention":
            if m.get("softcap") is not None and as_float(m, "softcap") <= 0:
                raise ConfigError(f"{what}: softcap must be positive")
            if m.get("kv_from") is not None:
                raise ConfigError(f"{what}: only a layer of type attention_2 takes keys and values from another")
            return
        if m.get("kv_from") is None:
            return
        source = as_int(m, "kv_from", 0)
        if source >= index:
            raise ConfigError(f"{what}: kv_from names layer {source}, which does not run before layer {index}")
        other = self.layers[source]
        theirs = other.get("mixer") if isinstance(other, dict) else None
        if not isinstance(theirs, dict) or other.get("type") != "attention_2" or theirs.get("kv_from") is not None:
            raise ConfigError(f"{what}: kv_from names layer {source}, which is no attention_2 layer with keys of its own")
        if any(theirs.get(key) != m[key] for key in ("kv_heads", "dim", "vdim")):
            raise ConfigError(f"{what}: layer {source}'s key and value heads are not this layer's")

    def _check_layer(self, index: int, layer: Dict[str, Any]) -> None:
        what = f"{ARCHITECTURE} layer {index}"
        if not isinstance(layer, dict):
            raise ConfigError(f"{what} must be an object")
        require_keys(layer, ["type", "mixer"], what)
        if layer["type"] not in ("attention", "attention_2"):
            raise ConfigError(f"{what}: unknown type {layer['type']!r} (known: attention, attention_2)")
        self._check_mixer(index, layer["type"], _object(layer, "mixer", what), what + " mixer")
        mlp = layer.get("mlp")
        if mlp is None:
            return
        if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
            raise ConfigError(f"{what}: mlp is null or an object of kind dense or moe")
        if mlp["kind"] == "dense":
            as_int(mlp, "ff", 1)
            return
        as_int(_object(mlp, "expert", what + " mlp"), "ff", 1)
        router = _object(mlp, "router", what + " mlp")
        require_keys(router, ["experts", "top"], what + " mlp.router")
        if as_int(router, "top", 1) > as_int(router, "experts", 1):
            raise ConfigError(f"{what}: a token cannot use {router['top']} of {router['experts']} experts")
        if mlp.get("shared") is not None:
            as_int(_object(mlp, "shared", what + " mlp"), "ff", 1)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ZobelornConfig":
        require_keys(raw, ["vocab", "width", "layers", "norm"], ARCHITECTURE)
        return cls(copy.deepcopy(raw))

    def to_dict(self) -> Dict[str, Any]:
        out = copy.deepcopy(self.raw)
        out.pop("architectures", None)
        out["architecture"] = ARCHITECTURE
        return out

    # ---- the model as data -------------------------------------------------------------------
    def _kept_chunk(self, index: int) -> Optional[int]:
        """What the cache of layer `index` may give back: the pages before the chunk of a request's next
        position, for a chunk size that every layer reading this cache (the layer itself and those
        that name it in kv_from) divides; None (keep everything) where one of them sees all keys."""
        sizes = []
        for at, layer in enumerate(self.layers):
            m = layer["mixer"]
            if at == index or (layer["type"] == "attention_2" and m.get("kv_from") == index):
                if m.get("mask") is None:
                    return None
                sizes.append(int(m["mask"]["size"]))
        kept = 1
        for size in sizes:
            kept = kept * size // math.gcd(kept, size)
        return kept

    def _mixer(self, index: int, layer: Dict[str, Any]) -> PartSpec:
        m, prefix = layer["mixer"], f"l{index}.mix"
        size = int(m["mask"]["size"]) if m.get("mask") is not None else None
        common = {"hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
                  "vdim": m["vdim"], "scale": float(m["scale"]), "bias": False, "norm_eps": self.eps}
        rot = m.get("rot")
        if layer["type"] == "attention":
            position = None
            if rot is not None:
                scaling = None if rot.get("scaling") is None else {"kind": "linear", "factor": float(rot["scaling"]["factor"])}
                position = PartSpec("rope_half", {"base": float(rot["base"]), "dims": int(rot["dims"]), "scaling": scaling})
            # a window of n keys: the position itself and the n - 1 before it
            return PartSpec("gqa_rotary", dict(
                common, window=size - 1 if size is not None else None, chunk=None, position=position, qk_norm=True,
                softcap=float(m["softcap"]) if m.get("softcap") is not None else None,
                output_gate=True), prefix)
        position = None
        if rot is not None:
            scaling = None
            if rot.get("scaling") is not None:
                s = rot["scaling"]
                scaling = {"kind": "bands", "factor": float(s["factor"]), "low": float(s["low"]), "high": float(s["high"]),
                           "original": float(s["original"])}
            position = PartSpec("rope_interleaved", {"base": float(rot["base"]), "dims": int(rot["dims"]), "scaling": scaling})
        borrowed = m.get("kv_from") is not None
        return PartSpec("gqa_rotary", dict(
            common, window=None, chunk=size, position=position, head_norm=True, own_kv=not borrowed,
            cache_chunk=None if borrowed else self._kept_chunk(index)), prefix)

    def _feed_forward(self, index: int, mlp: Dict[str, Any]) -> PartSpec:
        prefix = f"l{index}.mlp"
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "silu",
                                          "names": (".gate", ".up", ".down")}, prefix)
        shared = mlp.get("shared")
        return PartSpec("routed_mlp", {"hidden_size": self.width, "experts": mlp["router"]["experts"],
                                       "top": mlp["router"]["top"], "expert_inner": mlp["expert"]["ff"],
                                       "shared_inner": shared["ff"] if shared is not None else 0, "shared_gate": False,
                                       "score": "sigmoid", "share_on": "input", "activation": "silu"}, prefix)

    def _norm(self, name: str, behind: bool = False) -> PartSpec:
        params = {"size": self.width, "eps": self.eps, "tensor": name, "one_plus": True}
        if behind and self.residual_mult != 1.0:
            params["gain_scale"] = self.residual_mult        # what the norm behind a sublayer gives is multiplied by it
        return PartSpec("rms_norm", params, name)

    def run_order(self) -> List[LayerCall]:
        """One call a layer; a layer that takes keys and values from another reads that call's cache."""
        return [LayerCall(i, cache=layer["mixer"].get("kv_from") if layer["type"] == "attention_2" else None)
                for i, layer in enumerate(self.layers)]

    def model_spec(self) -> ModelSpec:
        layers = []
        for index, layer in enumerate(self.layers):
            p = f"l{index}"
            parts = dict(mixer=self._mixer(index, layer), mixer_norm=self._norm(p + ".norm1"),
                         mixer_post_norm=self._norm(p + ".norm1b", behind=True))
            if layer.get("mlp") is None:
                layers.append(LayerSpec("sandwich_norm_mixer_only", **parts))
                continue
            parts.update(feed_forward=self._feed_forward(index, layer["mlp"]),
                         feed_forward_norm=self._norm(p + ".norm2"),
                         feed_forward_post_norm=self._norm(p + ".norm2b", behind=True))
            layers.append(LayerSpec("sandwich_norm_residual", **parts))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "tensor": "embed", "scale": self.embedding_scale}, "embed"),
            layers=tuple(layers), order=tuple(self.run_order()), final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tensor": "head"}, "head"))
        spec.validate()
        return spec


register_architecture(ARCHITECTURE, ZobelornConfig)
