"""The Sefalorn configuration reader, its model description and its plain statement (no GPU)."""
import copy

import pytest
import torch

import plain_sefalorn as ps
from inferrs_b200.cache.storage import KVNeed
from inferrs_b200.config.base import ConfigError
from inferrs_b200.engine.loading import spec_from_config
from inferrs_b200.engine.model import cache_needs, declared_tensors
from sefalorn_cases import CASE_P, CASE_Q, CASE_R, CASE_S, make_weights


def test_description_names_every_tensor_with_its_shape():
    spec, cfg = spec_from_config(CASE_P)
    shapes = {d.name: tuple(d.shape) for d in declared_tensors(spec)}
    assert shapes["embed"] == (211, 96) and shapes["head"] == (211, 96) and shapes["final.norm"] == (96,)
    assert shapes["l0.norm1"] == (96,) and shapes["l0.rg1"] == (96, 96) and shapes["l0.rg2.b"] == (96,)
    assert shapes["l0.mix.left.q"] == (144, 96) and shapes["l0.mix.left.k"] == (48, 96)
    assert shapes["l0.mix.left.v"] == (40, 96) and shapes["l0.mix.left.v.b"] == (40,)
    assert shapes["l0.mix.left.o"] == (96, 120) and shapes["l0.mix.left.o.b"] == (96,)
    assert shapes["l0.mix.left.r1"] == (6,) and shapes["l0.mix.left.talk"] == (6, 6)
    assert shapes["l0.mix.right.q"] == (40, 96) and shapes["l0.mix.right.v"] == (48, 96)
    assert shapes["l0.mix.right.q.conv"] == (40, 4) and shapes["l0.mix.right.v.conv"] == (48, 4)
    assert shapes["l0.mix.right.b"] == (4, 96) and shapes["l0.mix.right.a"] == (4, 96)
    assert shapes["l0.mix.right.A_log"] == (4,) and shapes["l0.mix.right.norm"] == (12,)
    assert shapes["l0.mix.right.g"] == (48, 96) and shapes["l0.mix.right.o"] == (96, 48)
    assert shapes["l0.mlp.router"] == (5, 96) and shapes["l0.mlp.e4.down"] == (96, 24)
    assert shapes["l1.mix.q"] == (120, 96) and shapes["l1.mix.g"] == (72, 96) and shapes["l1.mix.norm"] == (72,)
    assert "l1.norm2" not in shapes and "l1.rg2" not in shapes and "l1.mlp.router" not in shapes
    assert all(l.arrangement == "gated_residual" for l in spec.layers)
    assert spec.logit_scale == 0.8
    kv, states = cache_needs(spec)
    assert kv == {0: KVNeed(2, 24, 23, 2, 20), 3: KVNeed(4, 16, 50, 2, 40)}
    assert states[0].shape == (4 * 20 * 12 + 3 * (40 + 40 + 48),)           # matrices, then the convolutions' inputs
    assert states[1].shape == (3 * 40 * 24,) and states[2].shape == (2 * 16 * 36,)
    assert states[3].shape == (3 * 36 * 20 + 1 * (108 + 108 + 60),)


def test_a_second_norm_without_a_feed_forward_is_read_from_the_tensor_names():
    spec, _ = spec_from_config(CASE_Q)
    assert len(spec.layers[2].sublayers) == 1
    spec, _ = spec_from_config(CASE_Q, tensor_shapes={"l2.norm2": (64,)})
    assert len(spec.layers[2].sublayers) == 2 and spec.layers[2].sublayers[1].part is None
    assert {"l2.norm2", "l2.rg2", "l2.rg2.b"} <= {d.name for d in declared_tensors(spec)}


@pytest.mark.parametrize("edit,message", [
    (lambda c: c.pop("norm"), "lacks"),
    (lambda c: c.pop("logit_scale"), "lacks"),
    (lambda c: c["layers"][0].update(type="conv"), "not one of"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "missing"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(rot=8), "unknown"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("conv"), "missing"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(mask={"size": 0}), "mask"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "missing"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 0.5, 1.5]), "decay"),
    (lambda c: c["layers"][0].update(mlp={"kind": "dense", "ff": 8}), "moe"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"].pop("scale"), "router"),
])
def test_wrong_configurations_are_refused(edit, message):
    cfg = copy.deepcopy(CASE_P)
    edit(cfg)
    with pytest.raises(ConfigError, match=message):
        spec_from_config(cfg)


def test_an_unknown_key_at_the_top_is_named_and_ignored(capsys):
    cfg = dict(copy.deepcopy(CASE_S), seed=5)
    spec, _ = spec_from_config(cfg)
    assert "seed" in capsys.readouterr().err and spec.vocab_size == 77


@pytest.mark.parametrize("case", [CASE_P, CASE_Q, CASE_R, CASE_S])
def test_plain_statement_in_float32_agrees_with_float64(case):
    w = make_weights(case, 3)
    toks = torch.randint(0, case["vocab"], (60,), generator=torch.Generator().manual_seed(1)).tolist()
    a, b = ps.forward(case, w, toks, torch.float32), ps.forward(case, w, toks, torch.float64)
    assert float((a.double() - b).abs().max() / b.abs().max()) < 2e-4


def _attention_only(window):
    left = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25}
    if window:
        left["mask"] = {"size": window}
    # the right mixer counts for nothing and the layer has no feed-forward: what a token sees, it sees through the window
    return {"architecture": "Sefalorn", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
            "layers": [{"type": "parallel", "mlp": None,
                        "mixer": {"left": left, "right": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 1},
                                  "left_scale": 1.0, "right_scale": 0.0}}]}


def test_plain_statement_sees_exactly_the_window():
    """Position i sees j with 0 <= i - j < size: changing the token at position 10 moves the logits at 10 .. 10 + size
    - 1 and at no other position."""
    case = _attention_only(12)
    w = make_weights(case, 4)
    toks = torch.randint(0, 50, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    other = list(toks)
    other[10] = (other[10] + 1) % 50
    a, b = ps.forward(case, w, toks, torch.float64), ps.forward(case, w, other, torch.float64)
    moved = (a - b).abs().amax(dim=1) > 1e-9
    assert moved.tolist() == [10 <= i < 22 for i in range(40)]
    wide = _attention_only(None)
    a, b = ps.forward(wide, w, toks, torch.float64), ps.forward(wide, w, other, torch.float64)
    assert ((a - b).abs().amax(dim=1) > 1e-9).tolist() == [i >= 10 for i in range(40)]


def test_plain_statement_mixes_heads_before_the_softmax_and_penalises_distance():
    case = _attention_only(None)
    w = make_weights(case, 5)
    toks = torch.randint(0, 50, (30,), generator=torch.Generator().manual_seed(3)).tolist()
    base = ps.forward(case, w, toks, torch.float64)
    for name in ("l0.mix.left.talk", "l0.mix.left.r1", "l0.mix.left.r2"):
        w2 = dict(w)
        w2[name] = w[name] * 1.5
        assert float((ps.forward(case, w2, toks, torch.float64) - base)[1:].abs().max()) > 1e-4, name
    # the identity as the mixing matrix and no penalty: ordinary grouped-query attention in a window of everything
    w3 = dict(w)
    w3["l0.mix.left.talk"], w3["l0.mix.left.r1"] = torch.eye(4), torch.zeros(4)
    h = ps.layer_norm(w3["embed"].double()[toks], w3["l0.norm1"].double(), 1e-5)
    p = "l0.mix.left"
    q = (h @ w3[f"{p}.q"].double().T + w3[f"{p}.q.b"].double()).view(30, 4, 16)
    k = (h @ w3[f"{p}.k"].double().T + w3[f"{p}.k.b"].double()).view(30, 2, 16)
    v = (h @ w3[f"{p}.v"].double().T + w3[f"{p}.v.b"].double()).view(30, 2, 24)
    out = torch.zeros(30, 4, 24, dtype=torch.float64)
    for i in range(30):
        for head in range(4):
            s = (k[:i + 1, head // 2] @ q[i, head]) * 0.25
            out[i, head] = torch.softmax(s, 0) @ v[:i + 1, head // 2]
    want = out.reshape(30, 96) @ w3[f"{p}.o"].double().T + w3[f"{p}.o.b"].double()
    got = ps.window_attention(h, case["layers"][0]["mixer"]["left"] | {"mask": {"size": 1000}},
                              {k_: v_.double() for k_, v_ in w3.items()}, p)
    assert float((got - want).abs().max()) < 1e-10


def test_plain_delta_rule_writes_then_reads():
    """With beta = 1 and no fading the state answers the key it was just given with the value exactly: o = v (k . q)
    for q = k unit vectors, whatever stood in the state before."""
    torch.manual_seed(0)
    D, E = 8, 5
    S = torch.randn(D, E, dtype=torch.float64)
    k = torch.randn(D, dtype=torch.float64)
    k = k / k.norm()
    v = torch.randn(E, dtype=torch.float64)
    u = v - S.T @ k
    S = S + k[:, None] * u[None, :]
    assert float((S.T @ k - v).abs().max()) < 1e-12
