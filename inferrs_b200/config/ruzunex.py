"""Typed configuration of the Ruzunex decoder.

config.json gives every size and every constant that differs between models of the design:

    architecture   "Ruzunex"
    vocab, width
    norm           {"eps": ...}: every norm of the model
    streams        how many copies wide the residual is (hyper-connections)
    canon          {"taps": ...}: the short convolution in front of every sub-layer
    layers         a list; every entry has "type" (which mixer), "mixer" (its sizes and constants) and "mlp"
                   (a feed-forward, or null for a layer without one)
    max_positions  optional: the most positions of a sequence

Mixers: "attention" (heads, kv_heads, dim, vdim, scale, optional mask {size}, optional v_mix) and "parallel" (left
{heads, kv_heads, dim, vdim, scale, conv, optional rot {base, dims}, optional mask {size}}, right {heads, dim, vdim},
left_scale, right_scale).  Feed-forwards: {"kind": "dense", "ff"} and {"kind": "moe", "expert": {"ff", "limit"},
"router": {"experts", "top"}}.

A key that the chosen part needs and that is absent is an error: no size stands in code.  Keys that this reader does
not know inside `norm`, `canon`, a layer, its mixer or its feed-forward are an error too, so that a variant of the
design is refused instead of being run as this one; an unknown key at the top (a seed, a name) is named on standard
error and ignored.  A layer without a feed-forward has no second sub-layer; where the weight files hold its norm,
connection and convolution all the same (``l<i>.norm2``), they are read and do nothing.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, RawConfig
from .sefalorn import _freeze, _keys, _number, _positive_ints, _thaw

DEFAULT_MAX_POSITIONS = 131072

ATTENTION_KEYS = {"heads", "kv_heads", "dim", "vdim", "scale"}
LEFT_KEYS = {"heads", "kv_heads", "dim", "vdim", "scale", "conv"}
RIGHT_KEYS = {"heads", "dim", "vdim"}


@dataclass(frozen=True)
class RuzunexLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]            # the mixer's sizes and constants, as sorted (key, value) pairs
    mlp: Optional[Tuple[Tuple[str, Any], ...]]    # the feed-forward's; None: the layer has none
    idle_second: bool = False                     # no feed-forward, but its norm and connection are in the weight files

    def get(self, key: str, default=None):
        return _thaw(dict(self.mixer).get(key, default))

    def mlp_get(self, key: str, default=None):
        return None if self.mlp is None else _thaw(dict(self.mlp).get(key, default))


@dataclass(frozen=True)
class RuzunexConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    streams: int
    canon_taps: int
    layers: Tuple[RuzunexLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "RuzunexConfig":
        src = raw.source
        known = {"architecture", "architectures", "model_type", "vocab", "width", "max_positions", "norm", "streams",
                 "canon", "layers", "eos_token_id"}
        extra = sorted(k for k in raw.values if k not in known)
        if extra:
            print(f"[inferrs_b200] {src}: keys {extra} are not part of a Ruzunex configuration and are ignored",
                  file=sys.stderr)
        missing = [k for k in ("vocab", "width", "norm", "streams", "canon", "layers") if not raw.has(k)]
        if missing:
            raise ConfigError(f"{src}: Ruzunex config lacks the keys {missing}")
        vocab, width, streams = raw.get_int("vocab"), raw.get_int("width"), raw.get_int("streams")
        max_positions = raw.get_int("max_positions", DEFAULT_MAX_POSITIONS)
        for k, v in (("vocab", vocab), ("width", width), ("streams", streams), ("max_positions", max_positions)):
            if v <= 0:
                raise ConfigError(f"{src}: key '{k}' must be positive, got {v}")
        norm = raw.values["norm"]
        if not isinstance(norm, dict) or set(norm) != {"eps"}:
            raise ConfigError(f"{src}: key 'norm' must be an object with 'eps', got {norm!r}")
        eps = _number(src, "norm.eps", norm["eps"], float)
        if eps <= 0:
            raise ConfigError(f"{src}: norm.eps must be positive, got {eps}")
        canon = raw.values["canon"]
        if not isinstance(canon, dict) or set(canon) != {"taps"} or _number(src, "canon.taps", canon["taps"], int) <= 0:
            raise ConfigError(f"{src}: key 'canon' must be an object with a positive 'taps', got {canon!r}")
        layers_raw = raw.get_list("layers")
        if not layers_raw:
            raise ConfigError(f"{src}: key 'layers' must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or set(entry) - {"type", "mixer", "mlp"} or "type" not in entry \
                    or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"{src}: {where} must be an object with 'type', 'mixer' and 'mlp', got {entry!r}")
            kind = entry["type"]
            if kind == "attention":
                mixer = _check_attention(src, f"{where}.mixer", entry["mixer"], ATTENTION_KEYS, {"mask", "v_mix"})
            elif kind == "parallel":
                mixer = _check_parallel(src, where, entry["mixer"])
            else:
                raise ConfigError(f"{src}: {where}.type '{kind}' is not one of ['attention', 'parallel']")
            mlp = _check_mlp(src, where, entry.get("mlp"))
            layers.append(RuzunexLayer(type=kind, mixer=_freeze(mixer), mlp=None if mlp is None else _freeze(mlp)))
        blended = [(layer.get("kv_heads"), layer.get("vdim")) for layer in layers
                   if layer.type == "attention" and layer.get("v_mix")]
        if len(set(blended)) > 1:
            raise ConfigError(f"{src}: the layers with 'v_mix' blend their values with the first such layer's and "
                              f"must agree in kv_heads and vdim, got {blended}")
        eos = raw.values.get("eos_token_id")
        eos_ids = () if eos is None else tuple(eos) if isinstance(eos, list) else (eos,)
        if any(isinstance(t, bool) or not isinstance(t, int) or not 0 <= t < vocab for t in eos_ids):
            raise ConfigError(f"{src}: eos_token_id must be token ids inside the vocabulary, got {eos!r}")
        return cls(vocab=vocab, width=width, max_positions=max_positions, norm_eps=eps, streams=streams,
                   canon_taps=int(canon["taps"]), layers=tuple(layers), eos_token_ids=eos_ids)

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "RuzunexConfig":
        """The configuration with what only the weight files say: whether a layer without a feed-forward still
        brings a second norm, connection and convolution."""
        layers = list(self.layers)
        for i, layer in enumerate(layers):
            if layer.mlp is None and f"l{i}.norm2" in shapes:
                layers[i] = RuzunexLayer(type=layer.type, mixer=layer.mixer, mlp=None, idle_second=True)
        return RuzunexConfig(**{**self.__dict__, "layers": tuple(layers)})


def _check_mask(src: str, where: str, mask):
    if mask is not None and (not isinstance(mask, dict) or set(mask) != {"size"}
                             or _number(src, f"{where}.mask.size", mask["size"], int) <= 0):
        raise ConfigError(f"{src}: {where}.mask must be an object with a positive 'size', got {mask!r}")


def _check_attention(src: str, where: str, given, need: set, optional: set) -> Dict[str, Any]:
    out = _keys(src, where, given, need, optional)
    _positive_ints(src, where, out, [k for k in ("heads", "kv_heads", "dim", "vdim", "conv") if k in need])
    _number(src, f"{where}.scale", out["scale"], float)
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"{src}: {where}: {out['heads']} heads are not a multiple of {out['kv_heads']} kv_heads")
    _check_mask(src, where, out.get("mask"))
    if "v_mix" in out and not isinstance(out["v_mix"], bool):
        raise ConfigError(f"{src}: {where}.v_mix must be true or false, got {out['v_mix']!r}")
    rot = out.get("rot")
    if rot is not None:
        if not isinstance(rot, dict) or set(rot) != {"base", "dims"} \
                or not _number(src, f"{where}.rot.base", rot["base"], float) > 0 \
                or _number(src, f"{where}.rot.dims", rot["dims"], int) <= 0 or rot["dims"] % 2 \
                or rot["dims"] > out["dim"]:
            raise ConfigError(f"{src}: {where}.rot must give a positive 'base' and even 'dims' of at most the head's "
                              f"size, got {rot!r}")
    return out


def _check_parallel(src: str, where: str, given) -> Dict[str, Any]:
    out = _keys(src, f"{where}.mixer", given, {"left", "right", "left_scale", "right_scale"})
    for k in ("left_scale", "right_scale"):
        _number(src, f"{where}.mixer.{k}", out[k], float)
    out["left"] = _check_attention(src, f"{where}.mixer.left", out["left"], LEFT_KEYS, {"rot", "mask"})
    right = _keys(src, f"{where}.mixer.right", out["right"], RIGHT_KEYS)
    _positive_ints(src, f"{where}.mixer.right", right, ("heads", "dim", "vdim"))
    out["right"] = right
    return out


def _check_mlp(src: str, where: str, mlp) -> Optional[Dict[str, Any]]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{src}: {where}.mlp must be null or an object of kind 'dense' or 'moe', got {mlp!r}")
    if mlp["kind"] == "dense":
        if set(mlp) != {"kind", "ff"} or _number(src, f"{where}.mlp.ff", mlp["ff"], int) <= 0:
            raise ConfigError(f"{src}: {where}.mlp of kind 'dense' has a positive 'ff', got {mlp!r}")
        return dict(mlp)
    if set(mlp) != {"kind", "expert", "router"}:
        raise ConfigError(f"{src}: {where}.mlp of kind 'moe' has 'expert' and 'router', got {mlp!r}")
    expert, router = mlp["expert"], mlp["router"]
    if not isinstance(expert, dict) or set(expert) != {"ff", "limit"} \
            or _number(src, f"{where}.mlp.expert.ff", expert["ff"], int) <= 0 \
            or not _number(src, f"{where}.mlp.expert.limit", expert["limit"], float) > 0:
        raise ConfigError(f"{src}: {where}.mlp.expert must be an object with a positive 'ff' and 'limit', got {expert!r}")
    if not isinstance(router, dict) or set(router) != {"experts", "top"} \
            or not 0 < _number(src, f"{where}.mlp.router.top", router["top"], int) \
            <= _number(src, f"{where}.mlp.router.experts", router["experts"], int):
        raise ConfigError(f"{src}: {where}.mlp.router must give 'experts' and 'top' with 0 < top <= experts, "
                          f"got {router!r}")
    return dict(mlp)
