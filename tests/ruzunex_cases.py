"""Small Ruzunex configurations and weights for the tests: sizes that differ from one another in every field, among
them values that make mechanisms degenerate (one stream, one tap, one head, one key/value head, one expert, every
expert chosen, a window of one position, no window at all, no rotation, a rotation of part of a head, a layer without
a feed-forward, values larger and smaller than keys, a parallel layer first, blended values in two, one or no
layer)."""
from __future__ import annotations

import copy
from typing import Dict

import torch

from inferrs_b200.engine.loading import spec_from_config
from inferrs_b200.engine.model import declared_tensors


def _attention(heads, kv_heads, dim, vdim, scale, window=None, v_mix=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if v_mix is not None:
        m["v_mix"] = v_mix
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _left(heads, kv_heads, dim, vdim, scale, conv, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "conv": conv}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def _parallel(left, right, left_scale, right_scale, mlp):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "right": {"heads": right[0], "dim": right[1], "vdim": right[2]},
                      "left_scale": left_scale, "right_scale": right_scale}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


# a parallel layer first; three streams, four taps; windows of 23 and 50 (no multiples of a page); values smaller and
# larger than keys; three layers that blend values (the first of them the second layer of the model) and one between
# them that does not; a rotation of half a head; a layer without a feed-forward
CASE_P = {
    "architecture": "Ruzunex", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "streams": 3, "canon": {"taps": 4},
    "layers": [
        _parallel(_left(6, 2, 24, 20, 0.3, 3, (12, 10000.0)), (3, 20, 12), 0.7, 1.3, _moe(24, 5, 2, 1.5)),
        _attention(4, 2, 16, 40, 0.25, 23, True, _dense(72)),
        _attention(6, 3, 8, 12, 0.4, 50, False, None),
        _attention(2, 2, 24, 40, 0.2, 31, True, _moe(40, 4, 1, 0.8)),
        _parallel(_left(4, 4, 16, 40, 0.25, 2, (16, 500.0)), (2, 36, 20), 1.1, 0.6, _dense(50)),
        _attention(8, 2, 16, 40, 0.3, 23, True, _moe(16, 3, 3, 2.0)),
    ],
}
# everything one: one stream, one tap, one head, one key/value head, a window that shows a token only itself, one
# expert, no rotation, a single layer that says v_mix (it blends with nothing)
CASE_Q = {
    "architecture": "Ruzunex", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "streams": 1, "canon": {"taps": 1},
    "layers": [
        _attention(1, 1, 32, 16, 0.2, 1, True, _moe(20, 1, 1, 1.0)),
        _parallel(_left(1, 1, 16, 64, 0.2, 1), (1, 16, 64), 1.0, 1.0, _moe(12, 2, 2, 0.5)),
        _attention(2, 1, 8, 8, 0.5, 2, None, _dense(20)),
    ],
}
# sizes that the tensor-core attention takes (keys and values of 64 and 128 numbers) beside sizes that it does not;
# no window at all in one attention layer (the distance bias grows with the prompt); a whole head rotated
CASE_R = {
    "architecture": "Ruzunex", "vocab": 130, "width": 128, "norm": {"eps": 1e-5}, "streams": 2, "canon": {"taps": 2},
    "max_positions": 512,
    "layers": [
        _attention(4, 2, 128, 128, 0.09, None, True, _moe(32, 8, 3, 1.0)),
        _parallel(_left(4, 2, 128, 128, 0.09, 4, (128, 50000.0)), (2, 128, 64), 1.0, 0.8, None),
        _attention(6, 2, 64, 64, 0.125, 70, False, _dense(200)),
        _parallel(_left(6, 1, 64, 64, 0.12, 3, (32, 1000.0)), (2, 256, 32), 0.9, 1.2, _moe(48, 2, 1, 3.0)),
        _attention(2, 2, 128, 128, 0.1, 33, True, _dense(64)),
    ],
}
# sizes that no vector load, tensor-core tile or 16-byte copy takes; five streams
CASE_S = {
    "architecture": "Ruzunex", "vocab": 77, "width": 90, "norm": {"eps": 1e-5}, "streams": 5, "canon": {"taps": 5},
    "layers": [
        _parallel(_left(3, 3, 10, 7, 0.4, 5, (6, 100.0)), (3, 10, 9), 1.0, 1.0, _moe(50, 3, 2, 1.2)),
        _attention(3, 1, 10, 7, 0.4, 7, None, _dense(33)),
        _parallel(_left(5, 1, 6, 14, 0.4, 2), (5, 6, 5), 2.0, 0.5, None),
        _attention(5, 5, 6, 14, 0.4, 33, True, _moe(9, 2, 1, 1.0)),
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
        if mlp and mlp["kind"] == "moe" and mlp["router"]["top"] == 1 and mlp["router"]["experts"] > 1:
            mlp["router"]["top"] = 2
    return out


def make_weights(config: dict, seed: int, bare_second: bool = False) -> Dict[str, torch.Tensor]:
    """Weights of a size that keeps activations near one, so that every mechanism moves the logits: matrices N(0, 1 /
    fan-in), norm weights near one, convolutions whose every tap counts, sinks and factors per head that differ,
    lower bounds and biases that let the states live for tens of tokens, a blend weight well inside (0, 1), stream
    connections that mix.  Rounded to bfloat16 (returned as float32 on the host), so that both run dtypes and the
    plain statement start from the same numbers.  ``bare_second``: layers without a feed-forward get their second
    norm, connection and convolution all the same."""
    shapes = None
    if bare_second:
        shapes = {f"l{i}.norm2": (config["width"],) for i, l in enumerate(config["layers"]) if l.get("mlp") is None}
    spec, _ = spec_from_config(config, tensor_shapes=shapes)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for d in declared_tensors(spec):
        n = d.name
        r = torch.randn(d.shape, generator=g)
        if n == "embed":
            t = r
        elif n.endswith(".conv") or ".canon" in n:
            t = r * (0.6 / d.shape[1] ** 0.5) + 0.15
        elif n.endswith(".temp"):
            t = 1.0 + 0.3 * r
        elif n.endswith(".sink"):
            t = 1.5 * r
        elif n.endswith(".lower"):
            t = torch.sigmoid(r)
        elif n.endswith(".f.b"):
            t = 1.0 + r
        elif n.endswith(".vmix"):
            t = 0.5 + 0.1 * r
        elif n.endswith(".in") and ".hc" in n:
            t = 1.0 / d.shape[0] + 0.1 * r
        elif n.endswith(".out") and ".hc" in n:
            t = 1.0 + 0.2 * r
        elif n.endswith(".mix") and ".hc" in n:
            t = torch.eye(d.shape[0]) + 0.1 * r
        elif len(d.shape) == 1:                               # norm weights
            t = 1.0 + 0.2 * r
        elif n.endswith(".router"):
            t = r * (3.0 / d.shape[1] ** 0.5)                 # choices that move with the input
        else:
            t = r * (1.0 / d.shape[1] ** 0.5)
        out[n] = t.to(torch.bfloat16).to(torch.float32)
    return out


def random_case(seed: int) -> dict:
    """A configuration drawn from a seed: every size, count, window, constant and the order of layers differ from
    draw to draw (head sizes that the tensor-core attention takes among them, and values that make mechanisms
    degenerate)."""
    import random
    rnd = random.Random(seed)
    pick = rnd.choice

    def mlp():
        kind = pick(["dense", "moe", "moe", None])
        if kind == "dense":
            return _dense(pick([20, 33, 64, 72]))
        if kind == "moe":
            experts = pick([1, 2, 3, 5, 8])
            # a single choice among several is a close call in bfloat16 (see for_dtype): at least two are chosen
            top = experts if experts <= 2 else rnd.randint(2, experts)
            return _moe(pick([9, 16, 24, 40]), experts, top, pick([0.5, 1.0, 2.5]))
        return None

    def heads():
        g = pick([1, 1, 2, 3])
        return g * pick([1, 2, 3, 4]), g

    def sizes():
        d = pick([6, 8, 16, 24, 32, 64, 64, 128])
        e = d if rnd.random() < 0.5 else pick([7, 12, 16, 40, 64])
        return d, e

    blend_sizes = (pick([1, 2, 3]), pick([12, 16, 40, 64]))      # layers that blend agree in their values' sizes
    layers = []
    for _ in range(rnd.randint(2, 6)):
        if rnd.random() < 0.55:
            h, g = heads()
            d, e = sizes()
            v_mix = pick([True, True, False, None])
            if v_mix:
                g, e = blend_sizes
                h = g * pick([1, 2, 4])
            layers.append(_attention(h, g, d, e, pick([0.1, 0.25, 0.4]), pick([None, 1, 2, 5, 17, 23, 33, 64, 70]),
                                     v_mix, mlp()))
        else:
            h, g = heads()
            d, e = sizes()
            rot = None if rnd.random() < 0.25 else (pick([x for x in (2, 4, 6, 8, 16, 32, 64, 128) if x <= d]),
                                                    pick([100.0, 10000.0, 500000.0]))
            right = (pick([1, 2, 3, 5]), pick([6, 16, 20, 36, 128]), pick([5, 8, 12, 64]))
            layers.append(_parallel(_left(h, g, d, e, pick([0.1, 0.2, 0.35]), pick([1, 2, 3, 4, 5]), rot), right,
                                    pick([0.5, 1.0, 1.3]), pick([0.6, 1.0, 1.7]), mlp()))
    return {"architecture": "Ruzunex", "vocab": pick([61, 97, 130, 257]), "width": pick([32, 48, 64, 90, 128]),
            "norm": {"eps": pick([1e-5, 1e-6])}, "streams": pick([1, 2, 3, 4]), "canon": {"taps": pick([1, 2, 3, 4])},
            "max_positions": 512, "layers": layers}
