"""Typed configuration of the Zadepel decoder, read from its own config.json keys.

A Zadepel model is a list of layers, each with one mixer and an optional feed-forward, an RMS norm
before and after every sublayer, and an output head tied to the embedding:

    {"architecture": "Zadepel", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "latent_attention" | "attention" | "mingru", "mixer": {...},
                 "mlp": {...} | null}, ...]}

    latent_attention  heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}, mask {size}
    attention         heads, kv_heads, dim, vdim, scale, rot {base, dims}, v_mix
    mingru            width
    mlp               kind "dense", ff (inner width)

Nothing here is fixed to one model: every size, the order of the layers and every constant come
from the file; the tensor names ('embed', 'final.norm', 'l<i>.norm1', 'l<i>.norm1b', 'l<i>.mix.q',
'l<i>.mix.q.b', 'l<i>.mlp.gate', ...) are the design's.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional

from .metulix import _integer
from .qwen2 import ConfigError
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

MIXERS = ("latent_attention", "attention", "mingru")


def _number(where: str, data: Mapping[str, Any], key: str) -> float:
    if key not in data:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    value = data[key]
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {value!r}")
    return float(value)


def _rotation(where: str, mixer: Mapping[str, Any], limit: int) -> None:
    rot = mixer.get("rot")
    if not isinstance(rot, Mapping):
        raise ConfigError(f"config.json: {where}.rot must be an object with 'base' and 'dims'")
    _number(where + ".rot", rot, "base")
    dims = _integer(where + ".rot", rot, "dims", least=0)
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most {limit}")


def _window(where: str, mixer: Mapping[str, Any]) -> int:
    mask = mixer.get("mask")
    if mask is None:
        return 0
    if not isinstance(mask, Mapping):
        raise ConfigError(f"config.json: {where}.mask must be an object")
    return _integer(where + ".mask", mask, "size", least=0) if "size" in mask else 0


@dataclass(frozen=True)
class ZadepelConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple                      # the layer entries as read (dicts), checked
    eos_token_id: Optional[int] = None

    architecture = "Zadepel"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "ZadepelConfig":
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
        config = cls(vocab, width, _number("norm", norm, "eps"), tuple(copy.deepcopy(list(layers))),
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
        mixed_width = None             # kv_heads x vdim of the layers that blend their values
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if not isinstance(layer, Mapping) or not isinstance(layer.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with a 'mixer'")
            kind, mixer = layer.get("type"), layer["mixer"]
            where += ".mixer"
            if kind == "latent_attention":
                for key in ("heads", "dim", "vdim", "kv_rank"):
                    _integer(where, mixer, key)
                rope = _integer(where, mixer, "rot_dim", least=0)
                _number(where, mixer, "scale")
                _rotation(where, mixer, rope)
                _window(where, mixer)
            elif kind == "attention":
                heads = _integer(where, mixer, "heads")
                kv_heads = _integer(where, mixer, "kv_heads")
                dim = _integer(where, mixer, "dim")
                vdim = _integer(where, mixer, "vdim")
                if heads % kv_heads:
                    raise ConfigError(f"config.json: {where}.heads must be a multiple of kv_heads")
                _number(where, mixer, "scale")
                _rotation(where, mixer, dim)
                _window(where, mixer)
                if mixer.get("v_mix"):
                    if mixed_width is None:
                        mixed_width = (kv_heads, vdim)
                    elif mixed_width != (kv_heads, vdim):
                        raise ConfigError(f"config.json: {where} blends its values with those of the "
                                          f"first such layer, whose kv_heads and vdim "
                                          f"{mixed_width} differ from {(kv_heads, vdim)}")
            elif kind == "mingru":
                _integer(where, mixer, "width")
            else:
                raise ConfigError(f"config.json: layers[{index}].type '{kind}' is not a mixer of "
                                  f"this design ({', '.join(MIXERS)})")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: layers[{index}].mlp.kind must be 'dense'")
                _integer(f"layers[{index}].mlp", mlp, "ff")

    # --------------------------------------------------------------------- spec
    def build_spec(self) -> ModelSpec:
        """Lay the configuration out as parts: every layer is a `sandwich` arrangement (an RMS norm
        before and after each sublayer), its mixer a `latent_attention`, a `scaled_gqa_attention`
        or a `mingru`, its feed-forward a `gated_mlp` with the tanh form of GELU on the gate, or
        none; the head is the embedding."""
        norm = PartSpec("rmsnorm", {"width": self.width, "eps": self.eps, "weight_name": ""})
        layers: List[LayerSpec] = []
        schedule: List[LayerCall] = []
        mix_seen = False
        for index, layer in enumerate(self.layers):
            mixer, kind = layer["mixer"], layer["type"]
            if kind == "mingru":
                part = PartSpec("mingru", {"hidden_size": self.width, "width": int(mixer["width"])})
            elif kind == "latent_attention":
                rot = mixer["rot"]
                part = PartSpec("latent_attention", {
                    "hidden_size": self.width, "heads": int(mixer["heads"]), "dim": int(mixer["dim"]),
                    "rope_dim": int(mixer["rot_dim"]), "vdim": int(mixer["vdim"]),
                    "rank": int(mixer["kv_rank"]), "scale": float(mixer["scale"]), "eps": self.eps,
                    "window": _window("", mixer),
                    "position": PartSpec("rotary", {"theta": float(rot["base"]),
                                                    "rotary_dim": int(rot["dims"]),
                                                    "max_position": 0, "pairing": "interleaved"})})
            else:
                rot = mixer["rot"]
                value_mix = "none"
                if mixer.get("v_mix"):
                    value_mix = "mix" if mix_seen else "source"
                    mix_seen = True
                part = PartSpec("scaled_gqa_attention", {
                    "hidden_size": self.width, "heads": int(mixer["heads"]),
                    "kv_heads": int(mixer["kv_heads"]), "dim": int(mixer["dim"]),
                    "vdim": int(mixer["vdim"]), "scale": float(mixer["scale"]),
                    "window": _window("", mixer), "value_mix": value_mix,
                    "position": PartSpec("rotary", {"theta": float(rot["base"]),
                                                    "rotary_dim": int(rot["dims"]),
                                                    "max_position": 0, "pairing": "half"})})
            schedule.append(LayerCall(layer=index))
            mlp = layer.get("mlp")
            feed_forward = None if mlp is None else PartSpec("gated_mlp", {
                "hidden_size": self.width, "intermediate_size": int(mlp["ff"]),
                "activation": "gelu_tanh",
                "names": {"gate": "gate", "up": "up", "down": "down", "weight": "", "bias": ".b"}})
            has_ff = mlp is not None
            layers.append(LayerSpec(
                prefix=f"l{index}.", arrangement="sandwich", mixer=part, feed_forward=feed_forward,
                mixer_norm=norm, feed_forward_norm=norm if has_ff else None,
                mixer_out_norm=norm, feed_forward_out_norm=norm if has_ff else None,
                mixer_name="mix.", feed_forward_name="mlp.", mixer_norm_name="norm1",
                feed_forward_norm_name="norm2", mixer_out_norm_name="norm1b",
                feed_forward_out_norm_name="norm2b"))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_position=0, embedding_name="embed", head_name=None, final_norm=norm,
            final_norm_prefix="final.norm", layers=tuple(layers), schedule=tuple(schedule))
