"""Typed configuration of the Metulix hybrid decoder, read from its own config.json keys.

A Metulix model is a list of layers, each with one mixer and an optional feed-forward:

    {"architecture": "Metulix", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "attention" | "lightning", "mixer": {...}, "mlp": {...} | null}, ...]}

    attention mixer   heads, kv_heads, dim, vdim, conv (taps), scale, rot {base, dims},
                      mask {size, keep_first}, and optionally kv_from (the layer whose keys and
                      values this layer reads instead of projecting its own)
    lightning mixer   heads, dim, vdim, decay (one factor per head)
    mlp               kind "dense", ff (inner width)

Nothing here is fixed to one model: every size, the order of the layers and every constant
come from the file; the tensor names ('embed', 'head', 'final.norm', 'l<i>.norm1', 'l<i>.mix.q',
'l<i>.mlp.gate.b', ...) are the design's.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional

from .qwen2 import ConfigError
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def _integer(where: str, data: Mapping[str, Any], key: str, least: int = 1) -> int:
    if key not in data:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    value = data[key]
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json: {where}.{key} must be an integer, got {value!r}")
    if value < least:
        raise ConfigError(f"config.json: {where}.{key} must be at least {least}, got {value}")
    return int(value)


@dataclass(frozen=True)
class MetulixConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple                      # the layer entries as read (dicts), checked
    eos_token_id: Optional[int] = None

    architecture = "Metulix"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "MetulixConfig":
        vocab = _integer("the model", data, "vocab")
        width = _integer("the model", data, "width")
        norm = data.get("norm")
        if not isinstance(norm, Mapping) or "eps" not in norm:
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        layers = data.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        eos = data.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        config = cls(vocab, width, float(norm["eps"]), tuple(copy.deepcopy(list(layers))),
                     None if eos is None else int(eos))
        config.validate()
        return config

    def to_dict(self) -> Dict[str, Any]:
        data: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                                "width": self.width, "norm": {"eps": self.eps},
                                "layers": copy.deepcopy(list(self.layers))}
        if self.eos_token_id is not None:
            data["eos_token_id"] = self.eos_token_id
        return data

    # --------------------------------------------------------------- validation
    def validate(self) -> None:
        if self.eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if not isinstance(layer, Mapping) or not isinstance(layer.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with a 'mixer'")
            kind, mixer = layer.get("type"), layer["mixer"]
            if kind == "attention":
                self._check_attention(where, index, mixer)
            elif kind == "lightning":
                heads = _integer(where + ".mixer", mixer, "heads")
                _integer(where + ".mixer", mixer, "dim")
                _integer(where + ".mixer", mixer, "vdim")
                decay = mixer.get("decay")
                if not isinstance(decay, (list, tuple)) or len(decay) != heads:
                    raise ConfigError(f"config.json: {where}.mixer.decay must list one factor "
                                      f"per head ({heads})")
            else:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a mixer of this "
                                  f"design (attention, lightning)")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind must be 'dense'")
                _integer(where + ".mlp", mlp, "ff")

    def _check_attention(self, where: str, index: int, mixer: Mapping[str, Any]) -> None:
        where += ".mixer"
        heads = _integer(where, mixer, "heads")
        kv_heads = _integer(where, mixer, "kv_heads")
        dim = _integer(where, mixer, "dim")
        _integer(where, mixer, "vdim")
        _integer(where, mixer, "conv")
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads must be a multiple of kv_heads")
        if "scale" not in mixer:
            raise ConfigError(f"config.json: {where} lacks 'scale'")
        rot = mixer.get("rot")
        if not isinstance(rot, Mapping) or "base" not in rot:
            raise ConfigError(f"config.json: {where}.rot must be an object with 'base' and 'dims'")
        dims = _integer(where + ".rot", rot, "dims", least=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim")
        mask = mixer.get("mask")
        if mask is not None:
            if not isinstance(mask, Mapping):
                raise ConfigError(f"config.json: {where}.mask must be an object")
            _integer(where + ".mask", mask, "size", least=0)
            if "keep_first" in mask:
                _integer(where + ".mask", mask, "keep_first", least=0)
        source = mixer.get("kv_from")
        if source is not None:
            if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < index:
                raise ConfigError(f"config.json: {where}.kv_from must name an earlier layer")
            other = self.layers[source]
            theirs = other.get("mixer", {})
            if other.get("type") != "attention" or theirs.get("kv_from") is not None:
                raise ConfigError(f"config.json: {where}.kv_from must name an attention layer "
                                  f"with keys and values of its own")
            for key in ("kv_heads", "dim", "vdim"):
                if theirs.get(key) != mixer.get(key):
                    raise ConfigError(f"config.json: {where}.{key} differs from layer {source}, "
                                      f"whose keys and values it reads")

    # --------------------------------------------------------------------- spec
    def build_spec(self) -> ModelSpec:
        """Lay the configuration out as parts: every layer is an `outnorm` arrangement (the
        norms sit on the sublayers' outputs), its mixer a `lightning_attention` or a
        `talking_window_attention`, its feed-forward a biased `swiglu` or none."""
        norm = PartSpec("layernorm", {"width": self.width, "eps": self.eps, "weight_name": ""})
        layers: List[LayerSpec] = []
        schedule: List[LayerCall] = []
        for index, layer in enumerate(self.layers):
            mixer = layer["mixer"]
            if layer["type"] == "lightning":
                part = PartSpec("lightning_attention", {
                    "hidden_size": self.width, "heads": int(mixer["heads"]),
                    "dim": int(mixer["dim"]), "vdim": int(mixer["vdim"]),
                    "decay": tuple(float(d) for d in mixer["decay"]), "eps": self.eps})
                schedule.append(LayerCall(layer=index))
            else:
                mask = mixer.get("mask") or {}
                rot = mixer["rot"]
                source = mixer.get("kv_from")
                part = PartSpec("talking_window_attention", {
                    "hidden_size": self.width, "heads": int(mixer["heads"]),
                    "kv_heads": int(mixer["kv_heads"]), "dim": int(mixer["dim"]),
                    "vdim": int(mixer["vdim"]), "taps": int(mixer["conv"]),
                    "scale": float(mixer["scale"]), "eps": self.eps,
                    "window": int(mask.get("size", 0) or 0),
                    "keep_first": int(mask.get("keep_first", 0) or 0),
                    "own_keys": source is None,
                    "position": PartSpec("rotary", {"theta": float(rot["base"]),
                                                    "rotary_dim": int(rot["dims"]),
                                                    "max_position": 0,
                                                    "pairing": "interleaved"})})
                schedule.append(LayerCall(layer=index) if source is None else
                                LayerCall(layer=index, cache=int(source), writes_cache=False))
            mlp = layer.get("mlp")
            feed_forward = None if mlp is None else PartSpec("swiglu", {
                "hidden_size": self.width, "intermediate_size": int(mlp["ff"]), "bias": True,
                "names": {"gate": "gate", "up": "up", "down": "down", "weight": "", "bias": ".b"}})
            layers.append(LayerSpec(
                prefix=f"l{index}.", arrangement="outnorm", mixer=part, feed_forward=feed_forward,
                mixer_norm=norm, feed_forward_norm=norm if mlp is not None else None,
                mixer_name="mix.", feed_forward_name="mlp.", mixer_norm_name="norm1",
                feed_forward_norm_name="norm2"))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_position=0, embedding_name="embed", head_name="head", final_norm=norm,
            final_norm_prefix="final.norm", layers=tuple(layers), schedule=tuple(schedule))
