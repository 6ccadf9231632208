"""Typed configuration of the Sefalorn decoder.

config.json gives every size and every constant that differs between models of the design:

    architecture   "Sefalorn"
    vocab, width
    norm           {"eps": ...}: every norm of the model
    logit_scale    what the logits are multiplied by
    layers         a list; every entry has "type" (which mixer), "mixer" (its sizes and constants) and "mlp"
                   (routed experts, or null for a layer without a feed-forward)
    max_positions  optional: the most positions of a sequence

Mixers: "lightning" (heads, dim, vdim, decay [per head]) and "parallel" (left {heads, kv_heads, dim, vdim, scale,
mask {size}}, right {heads, kv_heads, dim, vdim, conv}, left_scale, right_scale).  Feed-forward: {"kind": "moe",
"expert": {"ff"}, "router": {"experts", "top", "scale"}}.

A key that the chosen part needs and that is absent is an error: no size stands in code.  Keys that this reader does
not know inside `norm`, a layer, its mixer or its feed-forward are an error too, so that a variant of the design is
refused instead of being run as this one; an unknown key at the top (a seed, a name) is named on standard error and
ignored.  A layer without a feed-forward has no second norm and no second gate; where the weight files hold them all
the same (``l<i>.norm2``), they are read and do nothing.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, RawConfig

DEFAULT_MAX_POSITIONS = 131072

LIGHTNING_KEYS = {"heads", "dim", "vdim", "decay"}
PARALLEL_KEYS = {"left", "right", "left_scale", "right_scale"}
LEFT_KEYS = {"heads", "kv_heads", "dim", "vdim", "scale", "mask"}
RIGHT_KEYS = {"heads", "kv_heads", "dim", "vdim", "conv"}


def _freeze(v):
    """Lists and objects of config.json as tuples, so that a configuration can be compared and hashed."""
    if isinstance(v, dict):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    if isinstance(v, list):
        return tuple(_freeze(x) for x in v)
    return v


def _thaw(v):
    if isinstance(v, tuple) and v and all(isinstance(x, tuple) and len(x) == 2 and isinstance(x[0], str) for x in v):
        return {k: _thaw(x) for k, x in v}
    return v


@dataclass(frozen=True)
class SefalornLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]            # the mixer's sizes and constants, as sorted (key, value) pairs
    mlp: Optional[Tuple[Tuple[str, Any], ...]]    # the feed-forward's; None: the layer has none
    idle_second: bool = False                     # no feed-forward, but its norm and gate are in the weight files

    def get(self, key: str, default=None):
        return _thaw(dict(self.mixer).get(key, default))

    def mlp_get(self, key: str, default=None):
        return None if self.mlp is None else _thaw(dict(self.mlp).get(key, default))


@dataclass(frozen=True)
class SefalornConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    logit_scale: float
    layers: Tuple[SefalornLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "SefalornConfig":
        src = raw.source
        known = {"architecture", "architectures", "model_type", "vocab", "width", "max_positions", "norm",
                 "logit_scale", "layers", "eos_token_id"}
        extra = sorted(k for k in raw.values if k not in known)
        if extra:
            print(f"[inferrs_b200] {src}: keys {extra} are not part of a Sefalorn configuration and are ignored",
                  file=sys.stderr)
        missing = [k for k in ("vocab", "width", "norm", "logit_scale", "layers") if not raw.has(k)]
        if missing:
            raise ConfigError(f"{src}: Sefalorn config lacks the keys {missing}")
        vocab, width = raw.get_int("vocab"), raw.get_int("width")
        max_positions = raw.get_int("max_positions", DEFAULT_MAX_POSITIONS)
        for k, v in (("vocab", vocab), ("width", width), ("max_positions", max_positions)):
            if v <= 0:
                raise ConfigError(f"{src}: key '{k}' must be positive, got {v}")
        norm = raw.values["norm"]
        if not isinstance(norm, dict) or set(norm) != {"eps"}:
            raise ConfigError(f"{src}: key 'norm' must be an object with 'eps', got {norm!r}")
        eps = _number(src, "norm.eps", norm["eps"], float)
        if eps <= 0:
            raise ConfigError(f"{src}: norm.eps must be positive, got {eps}")
        logit_scale = raw.get_float("logit_scale")
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
            if kind == "lightning":
                mixer = _check_lightning(src, where, entry["mixer"])
            elif kind == "parallel":
                mixer = _check_parallel(src, where, entry["mixer"])
            else:
                raise ConfigError(f"{src}: {where}.type '{kind}' is not one of ['lightning', 'parallel']")
            mlp = _check_mlp(src, where, entry.get("mlp"))
            layers.append(SefalornLayer(type=kind, mixer=_freeze(mixer), mlp=None if mlp is None else _freeze(mlp)))
        eos = raw.values.get("eos_token_id")
        eos_ids = () if eos is None else tuple(eos) if isinstance(eos, list) else (eos,)
        if any(isinstance(t, bool) or not isinstance(t, int) or not 0 <= t < vocab for t in eos_ids):
            raise ConfigError(f"{src}: eos_token_id must be token ids inside the vocabulary, got {eos!r}")
        return cls(vocab=vocab, width=width, max_positions=max_positions, norm_eps=eps, logit_scale=float(logit_scale),
                   layers=tuple(layers), eos_token_ids=eos_ids)

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "SefalornConfig":
        """The configuration with what only the weight files say: whether a layer without a feed-forward still
        brings a second norm and gate."""
        return _with_tensor_shapes(self, shapes)


def _with_tensor_shapes(cfg: "SefalornConfig", shapes: Dict[str, Tuple[int, ...]]) -> "SefalornConfig":
    layers = list(cfg.layers)
    for i, layer in enumerate(layers):
        if layer.mlp is None and f"l{i}.norm2" in shapes:
            layers[i] = SefalornLayer(type=layer.type, mixer=layer.mixer, mlp=None, idle_second=True)
    return SefalornConfig(**{**cfg.__dict__, "layers": tuple(layers)})


def _keys(src: str, where: str, given, need: set, optional: set = frozenset()) -> Dict[str, Any]:
    if not isinstance(given, dict):
        raise ConfigError(f"{src}: {where} must be an object, got {given!r}")
    bad = sorted(set(given) - need - optional) + sorted(k for k in need if given.get(k) is None)
    if bad:
        raise ConfigError(f"{src}: {where} has unknown or missing keys {bad}")
    return {k: v for k, v in given.items() if v is not None}


def _positive_ints(src: str, where: str, out: Dict[str, Any], keys):
    for k in keys:
        if _number(src, f"{where}.{k}", out[k], int) <= 0:
            raise ConfigError(f"{src}: {where}.{k} must be positive, got {out[k]!r}")


def _check_lightning(src: str, where: str, given) -> Dict[str, Any]:
    out = _keys(src, f"{where}.mixer", given, LIGHTNING_KEYS)
    _positive_ints(src, f"{where}.mixer", out, ("heads", "dim", "vdim"))
    decay = out["decay"]
    if not isinstance(decay, list) or len(decay) != out["heads"] \
            or any(not 0 < _number(src, f"{where}.mixer.decay", a, float) <= 1 for a in decay):
        raise ConfigError(f"{src}: {where}.mixer.decay must list one decay in (0, 1] per head, got {decay!r}")
    return out


def _check_parallel(src: str, where: str, given) -> Dict[str, Any]:
    out = _keys(src, f"{where}.mixer", given, PARALLEL_KEYS)
    for k in ("left_scale", "right_scale"):
        _number(src, f"{where}.mixer.{k}", out[k], float)
    left = _keys(src, f"{where}.mixer.left", out["left"], LEFT_KEYS - {"mask"}, {"mask"})
    _positive_ints(src, f"{where}.mixer.left", left, ("heads", "kv_heads", "dim", "vdim"))
    _number(src, f"{where}.mixer.left.scale", left["scale"], float)
    mask = left.get("mask")
    if mask is not None and (not isinstance(mask, dict) or set(mask) != {"size"}
                             or _number(src, f"{where}.mixer.left.mask.size", mask["size"], int) <= 0):
        raise ConfigError(f"{src}: {where}.mixer.left.mask must be an object with a positive 'size', got {mask!r}")
    right = _keys(src, f"{where}.mixer.right", out["right"], RIGHT_KEYS)
    _positive_ints(src, f"{where}.mixer.right", right, ("heads", "kv_heads", "dim", "vdim", "conv"))
    for side, m in (("left", left), ("right", right)):
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{src}: {where}.mixer.{side}: {m['heads']} heads are not a multiple of {m['kv_heads']} "
                              f"kv_heads")
    out["left"], out["right"] = left, right
    return out


def _check_mlp(src: str, where: str, mlp) -> Optional[Dict[str, Any]]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
        raise ConfigError(f"{src}: {where}.mlp must be null or an object of kind 'moe', got {mlp!r}")
    if set(mlp) != {"kind", "expert", "router"}:
        raise ConfigError(f"{src}: {where}.mlp of kind 'moe' has 'expert' and 'router', got {mlp!r}")
    expert, router = mlp["expert"], mlp["router"]
    if not isinstance(expert, dict) or set(expert) != {"ff"} or _number(src, f"{where}.mlp.expert.ff", expert["ff"], int) <= 0:
        raise ConfigError(f"{src}: {where}.mlp.expert must be an object with a positive 'ff', got {expert!r}")
    if not isinstance(router, dict) or set(router) != {"experts", "top", "scale"} \
            or not 0 < _number(src, f"{where}.mlp.router.top", router["top"], int) \
            <= _number(src, f"{where}.mlp.router.experts", router["experts"], int):
        raise ConfigError(f"{src}: {where}.mlp.router must give 'experts', 'top' and 'scale' with 0 < top <= experts, "
                          f"got {router!r}")
    _number(src, f"{where}.mlp.router.scale", router["scale"], float)
    return dict(mlp)


def _number(src: str, key: str, v, kind):
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and not isinstance(v, int)):
        raise ConfigError(f"{src}: key '{key}' must be {'an integer' if kind is int else 'a number'}, got {v!r}")
    return kind(v)
