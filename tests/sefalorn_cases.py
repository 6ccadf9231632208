"""Small Sefalorn configurations and weights for the tests: sizes that differ from one another in every field, among
them values that make mechanisms degenerate (one head, one key/value head, one tap, one expert, every expert chosen, a
window of one position, no window at all, a layer without a feed-forward, values larger and smaller than keys)."""
from __future__ import annotations

import copy
from typing import Dict

import torch

from inferrs_b200.engine.loading import spec_from_config
from inferrs_b200.engine.model import declared_tensors


def _left(heads, kv_heads, dim, vdim, scale, window=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def _right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _parallel(left, right, left_scale, right_scale, mlp):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def _lightning(heads, dim, vdim, decay, mlp):
    return {"type": "lightning", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


def _moe(ff, experts, top, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


# both mixers; windows of 23 and 50 (no multiples of a page); values smaller than keys; shared query/key heads on the
# right; a layer without a feed-forward; two lightning layers in a row
CASE_P = {
    "architecture": "Sefalorn", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.8,
    "layers": [
        _parallel(_left(6, 2, 24, 20, 0.3, 23), _right(4, 2, 20, 12, 4), 0.7, 1.3, _moe(24, 5, 2, 1.5)),
        _lightning(3, 40, 24, [0.9, 0.97, 0.995], None),
        _lightning(2, 16, 36, [0.8, 1.0], _moe(16, 3, 3, 1.0)),
        _parallel(_left(4, 4, 16, 40, 0.25, 50), _right(3, 3, 36, 20, 2), 1.1, 0.6, _moe(40, 4, 1, 2.5)),
    ],
}
# everything one: one head, one key/value head, one tap, a window that shows a token only itself, one expert
CASE_Q = {
    "architecture": "Sefalorn", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
    "layers": [
        _parallel(_left(1, 1, 32, 16, 0.2, 1), _right(1, 1, 16, 64, 1), 1.0, 1.0, _moe(20, 1, 1, 1.0)),
        _lightning(1, 64, 16, [1.0], _moe(12, 2, 2, 0.5)),
        _parallel(_left(2, 1, 8, 8, 0.5, 2), _right(2, 1, 8, 8, 3), 0.5, 2.0, None),
    ],
}
# no window at all (every earlier key is seen, the distance penalty grows with the prompt); head sizes of 64 and 128;
# keys of 128 and 256 numbers on the right
CASE_R = {
    "architecture": "Sefalorn", "vocab": 130, "width": 128, "norm": {"eps": 1e-5}, "logit_scale": 0.3,
    "max_positions": 512,
    "layers": [
        _parallel(_left(4, 2, 128, 128, 0.09), _right(2, 1, 128, 64, 4), 1.0, 0.8, _moe(32, 8, 3, 2.0)),
        _parallel(_left(8, 2, 64, 64, 0.125, 72), _right(2, 2, 256, 32, 2), 0.9, 1.2, None),
        _lightning(2, 128, 128, [0.98, 0.999], _moe(48, 2, 1, 1.0)),
    ],
}
# sizes that no vector load, tensor-core tile or 16-byte copy takes
CASE_S = {
    "architecture": "Sefalorn", "vocab": 77, "width": 90, "norm": {"eps": 1e-5}, "logit_scale": 1.7,
    "layers": [
        _lightning(1, 10, 7, [0.93], _moe(9, 2, 1, 1.0)),
        _parallel(_left(3, 3, 10, 7, 0.4, 7), _right(3, 1, 10, 9, 3), 1.0, 1.0, _moe(50, 3, 2, 3.0)),
        _parallel(_left(5, 1, 6, 14, 0.4, 33), _right(5, 5, 6, 5, 5), 2.0, 0.5, None),
    ],
}
CASES = {"P": CASE_P, "Q": CASE_Q, "R": CASE_R, "S": CASE_S}


def for_dtype(config: dict, dtype) -> dict:
    """The configuration as the tests of a run dtype use it.  In bfloat16 a router that chooses one expert of several
    is given two: where two scores are closer than bfloat16 tells apart the other expert is chosen, the whole output of
    the feed-forward changes, and a mixer's state carries the difference to every later token, so such a model cannot
    be compared with the plain statement token by token.  float32 runs keep the single choice."""
    if dtype != torch.bfloat16:
        return config
    out = copy.deepcopy(config)
    for layer in out["layers"]:
        mlp = layer.get("mlp")
        if mlp and mlp["router"]["top"] == 1 and mlp["router"]["experts"] > 1:
            mlp["router"]["top"] = 2
    return out


def make_weights(config: dict, seed: int, bare_norm2: bool = False) -> Dict[str, torch.Tensor]:
    """Weights of a size that keeps activations near one, so that every mechanism moves the logits: matrices N(0, 1 /
    fan-in), norm weights near one, biases that matter, distance penalties that grow over tens of positions, a matrix
    that mixes every head into every other, step sizes and decays that let the states live for tens of tokens.
    Rounded to bfloat16 (returned as float32 on the host), so that both run dtypes and the plain statement start from
    the same numbers.  ``bare_norm2``: layers without a feed-forward get their second norm and gate all the same."""
    shapes = None
    if bare_norm2:
        shapes = {f"l{i}.norm2": (config["width"],) for i, l in enumerate(config["layers"]) if l.get("mlp") is None}
    spec, _ = spec_from_config(config, tensor_shapes=shapes)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for d in declared_tensors(spec):
        n = d.name
        r = torch.randn(d.shape, generator=g)
        if n == "embed":
            t = r
        elif n.endswith(".dt_bias"):
            t = -1.5 + 0.7 * r
        elif n.endswith(".A_log"):
            t = -1.0 + 0.8 * r
        elif n.endswith(".conv"):
            t = r * (1.0 / d.shape[1] ** 0.5) + 0.2
        elif n.endswith(".r1"):
            t = r.abs() * 0.9 + 0.05
        elif n.endswith(".r2"):
            t = r.abs() * 0.2 + 0.05
        elif n.endswith(".talk"):
            t = torch.eye(d.shape[0]) * 0.8 + 0.35 * r
        elif n.endswith(".rg1.b") or n.endswith(".rg2.b"):
            t = 0.8 + 0.6 * r
        elif n.endswith(".b") and len(d.shape) == 1:          # biases of projections
            t = 0.3 * r
        elif len(d.shape) == 1:                               # norm weights
            t = 1.0 + 0.2 * r
        elif n.endswith(".router"):
            t = r * (3.0 / d.shape[1] ** 0.5)                 # choices that move with the input
        else:
            t = r * (1.0 / d.shape[1] ** 0.5)
        out[n] = t.to(torch.bfloat16).to(torch.float32)
    return out
