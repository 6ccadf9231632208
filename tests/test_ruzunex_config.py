"""The Ruzunex configuration, description and plain statement, without a GPU."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_ruzunex as pr
from helpers import random_tokens
from inferrs_b200.config.base import ConfigError
from inferrs_b200.engine.loading import spec_from_config
from inferrs_b200.engine.model import cache_needs, declared_tensors, side_state_needs
from ruzunex_cases import CASE_P, CASE_Q, CASE_R, CASE_S, CASES, make_weights


def test_description_takes_every_size_from_the_configuration():
    spec, cfg = spec_from_config(CASE_P)
    assert spec.architecture == "Ruzunex" and spec.streams == 3 and spec.vocab_size == 211 and len(spec.layers) == 6
    assert [layer.arrangement for layer in spec.layers] == ["hyper_connections"] * 6
    first = spec.layers[0]
    assert first.mixer.kind == "mixer_sum" and first.mixer.left_scale == 0.7 and first.mixer.right_scale == 1.3
    left, right = first.mixer.left, first.mixer.right
    assert (left.n_heads, left.n_kv_heads, left.head_dim, left.value_dim, left.conv_taps) == (6, 2, 24, 20, 3)
    assert left.norm_whole and left.q_norm.size == 6 * 24 and left.k_norm.size == 2 * 24 and left.window is None
    assert left.position.rot_dim == 12 and left.position.theta == 10000.0 and left.sink and left.head_scale
    assert (right.n_heads, right.key_dim, right.value_dim) == (3, 20, 12) and right.kind == "forget_write_scan"
    assert all(s.input_conv.taps == 4 and s.input_conv.width == 96 for layer in spec.layers for s in layer.sublayers)
    a1, a2, a3, a5 = (spec.layers[i].mixer for i in (1, 2, 3, 5))
    assert a1.window == 23 and a2.window == 50 and a1.scale == 0.25
    assert a1.distance_slopes == tuple(2.0 ** (-8.0 * (h + 1) / 4) for h in range(4))
    # the first layer that says v_mix keeps its values, the later ones blend with them, a layer that says no does neither
    assert a1.value_publish and a1.value_blend is None
    assert a2.value_publish is None and a2.value_blend is None
    assert a3.value_blend[1] == "l3.mix.vmix" and a5.value_blend[0] == a1.value_publish
    assert len(spec.layers[2].sublayers) == 1                       # no feed-forward: no second sub-layer
    ffs = [layer.ffn for layer in spec.layers]
    assert ffs[0].kind == "routed_experts" and ffs[0].scoring == "softmax_share" and ffs[0].limit == 1.5
    assert ffs[0].activation == "clamped_swish" and ffs[0].top == 2 and len(ffs[0].experts) == 5
    assert ffs[1].kind == "gated_dense" and ffs[1].activation == "gelu_tanh" and ffs[1].inner == 72


def test_caches_and_states():
    spec, _ = spec_from_config(CASE_P)
    kv, states = cache_needs(spec)
    assert sorted(kv) == [0, 1, 2, 3, 4, 5] and sorted(states) == [0, 4]
    assert kv[0].window is None and kv[0].value_dim == 20 and kv[1].window == 23 and kv[1].value_dim == 40
    assert states[0].shape == (3 * 20 * 12,) and states[4].shape == (2 * 36 * 20,)
    side = side_state_needs(spec)
    # every sub-layer's convolution keeps taps - 1 rows of the width; the left mixers keep taps - 1 rows of q | k | v
    convs = {(cid, type(owner).__name__): need.shape for (cid, owner), need in side.items()}
    assert convs[(0, "AttentionSpec")] == (2 * (6 * 24 + 2 * 24 + 2 * 20),)
    assert convs[(4, "AttentionSpec")] == (1 * (4 * 16 + 4 * 16 + 4 * 40),)
    assert sum(1 for (cid, name) in [(c, type(o).__name__) for (c, o) in side] if name == "InputConvSpec") == 11
    assert all(need.shape == (3 * 96,) for (cid, owner), need in side.items() if type(owner).__name__ == "InputConvSpec")
    # one tap keeps nothing
    assert side_state_needs(spec_from_config(CASE_Q)[0]) == {}


def test_tensor_names_and_shapes():
    spec, _ = spec_from_config(CASE_P)
    t = {d.name: tuple(d.shape) for d in declared_tensors(spec)}
    assert t["embed"] == (211, 96) and t["head"] == (211, 96) and t["final.norm"] == (96,)
    assert t["l0.canon1"] == (96, 4) and t["l0.canon2"] == (96, 4) and t["l0.hc1.mix"] == (3, 3) and t["l0.hc2.in"] == (3,)
    assert t["l0.mix.left.q.norm"] == (144,) and t["l0.mix.left.k.norm"] == (48,) and t["l0.mix.left.q.conv"] == (144, 3)
    assert t["l0.mix.left.v.conv"] == (40, 3) and t["l0.mix.left.temp"] == (6,) and t["l0.mix.left.sink"] == (6,)
    assert t["l0.mix.left.o"] == (96, 120) and t["l0.mix.right.f.b"] == (60,) and t["l0.mix.right.lower"] == (60,)
    assert t["l0.mix.right.norm"] == (12,) and t["l0.mix.right.v"] == (36, 96) and t["l0.mix.right.o"] == (96, 36)
    assert t["l1.mix.q.norm"] == (16,) and t["l1.mix.g"] == (160, 96) and t["l1.mix.o"] == (96, 160)
    assert t["l1.mix.vmix"] == () and t["l2.mix.vmix"] == () and t["l3.mix.vmix"] == ()
    assert "l2.norm2" not in t and "l2.canon2" not in t and "l2.hc2.in" not in t
    assert t["l0.mlp.router"] == (5, 96) and t["l0.mlp.e4.down"] == (96, 24) and t["l1.mlp.gate"] == (72, 96)
    # weight files that hold a second norm for a layer without a feed-forward: it is declared and nothing runs
    spec2, _ = spec_from_config(CASE_P, tensor_shapes={"l2.norm2": (96,)})
    t2 = {d.name for d in declared_tensors(spec2)}
    assert {"l2.norm2", "l2.canon2", "l2.hc2.in", "l2.hc2.out", "l2.hc2.mix"} <= t2
    assert spec2.layers[2].sublayers[1].part is None


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("streams"), "lacks the keys"),
    (lambda c: c.pop("canon"), "lacks the keys"),
    (lambda c: c["canon"].update(taps=0), "positive 'taps'"),
    (lambda c: c["norm"].update(kind="layer"), "'norm' must be"),
    (lambda c: c["layers"][1].update(type="latent"), "not one of"),
    (lambda c: c["layers"][1]["mixer"].update(bias=True), "unknown or missing"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "unknown or missing"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"].update(v_mix="yes"), "true or false"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=24), "must agree"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(rot={"dims": 13, "base": 100.0}), "rot must give"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(rot={"dims": 32, "base": 100.0}), "rot must give"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(kv_heads=1), "unknown or missing"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "unknown or missing"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "0 < top <= experts"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "positive 'ff' and 'limit'"),
    (lambda c: c["layers"][1]["mlp"].update(kind="poly"), "kind 'dense' or 'moe'"),
])
def test_configurations_that_are_refused(change, message):
    c = copy.deepcopy(CASE_P)
    change(c)
    with pytest.raises(ConfigError, match=message):
        spec_from_config(c)


def test_unknown_key_at_the_top_is_named_and_ignored(capsys):
    spec_from_config(dict(CASE_Q, seed=5))
    assert "['seed']" in capsys.readouterr().err


def test_random_weights_cover_every_declared_tensor():
    from inferrs_b200.weights.random_init import random_weights
    spec, _ = spec_from_config(CASE_S)
    w = random_weights(declared_tensors(spec), 3, torch.float32, torch.device("cpu"))
    assert set(w) == {d.name for d in declared_tensors(spec)}
    assert all(tuple(w[d.name].shape) == tuple(d.shape) for d in declared_tensors(spec))
    assert 0.0 < float(w["l0.mix.right.lower"].min()) and float(w["l0.mix.right.lower"].max()) < 1.0
    assert bool(torch.isfinite(pr.forward(CASE_S, w, random_tokens(9, 77, seed=1))).all())


# ---- the plain statement itself: every mechanism moves the logits as it should -----------------------------------
def test_plain_statement_windows_sinks_states_and_blended_values():
    case, w = CASE_P, make_weights(CASE_P, 3)
    toks = random_tokens(90, case["vocab"], seed=2)
    base = pr.forward(case, w, toks)
    # the first token reaches the last logits (every earlier key in the parallel layers, the states)
    other = pr.forward(case, w, [(toks[0] + 1) % case["vocab"]] + toks[1:])
    assert float((other[-1] - base[-1]).abs().max()) > 1e-4
    for name, bump in (("l0.mix.left.sink", 3.0), ("l0.mix.left.temp", 0.5), ("l3.mix.vmix", 0.3), ("l0.canon1", 0.3),
                       ("l0.mix.right.lower", -0.2), ("l4.mix.left.k.conv", 0.3), ("l1.hc1.mix", 0.2)):
        w2 = dict(w)
        w2[name] = w[name] + bump
        assert float((pr.forward(case, w2, toks)[-1] - base[-1]).abs().max()) > 1e-3, name
    # the first blended layer's own weight is read by nothing
    w2 = dict(w)
    w2["l1.mix.vmix"] = w["l1.mix.vmix"] + 0.3
    assert torch.equal(pr.forward(case, w2, toks), base)


def test_plain_attention_layer_sees_its_window_and_no_further():
    """One attention layer alone: a token beyond the window changes nothing, the last one inside it does; the
    convolution in front of the sub-layers reaches taps - 1 tokens further."""
    case = {"architecture": "Ruzunex", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "streams": 2,
            "canon": {"taps": 3}, "layers": [CASE_P["layers"][1] | {"mlp": None}]}
    case["layers"][0] = copy.deepcopy(case["layers"][0])
    case["layers"][0]["mixer"]["mask"]["size"] = 9
    w = make_weights(case, 4)
    toks = random_tokens(40, 50, seed=5)
    base = pr.forward(case, w, toks)[-1]
    reach = 9 + 2                      # the window, and the convolution on what the mixer reads
    for back, seen in ((reach - 1, True), (reach, False), (reach + 5, False)):
        t2 = list(toks)
        t2[39 - back] = (t2[39 - back] + 7) % 50
        assert (float((pr.forward(case, w, t2)[-1] - base).abs().max()) > 1e-6) == seen, back


def test_plain_sink_takes_weight_from_every_key():
    s = torch.randn(2, 5, 5)
    see = pr.visible(5, None)
    p = pr.sink_softmax(s, see, torch.tensor([0.3, -20.0]))
    full = torch.softmax(s.masked_fill(~see[None], float("-inf")), dim=-1)
    assert torch.allclose(p[1], full[1], atol=1e-6) and bool((p[0].sum(-1) < 1.0 - 1e-3).all())
    assert torch.allclose(p[0] / p[0].sum(-1, keepdim=True), full[0], atol=1e-6)


def test_plain_forget_write_rule_is_a_running_mix_of_values():
    """With a gate of one half on every channel and queries of ones, a head's output is the sum over channels of the
    exponentially weighted mean of the values."""
    T, D, E = 6, 3, 2
    v = torch.randn(T, 1, E)
    o = pr.forget_write_rule(torch.ones(T, 1, D), torch.full((T, 1, D), 0.5), v)
    want = torch.zeros(E)
    for t in range(T):
        want = 0.5 * want + 0.5 * v[t, 0]
    assert torch.allclose(o[-1, 0], D * want, atol=1e-6)


def test_plain_routing_weights_sum_to_one_and_prefer_the_lower_index():
    z = torch.tensor([[0.0, 1.0, 1.0, -1.0]])
    idx, wt = pr.route(z, 2)
    assert idx.tolist() == [[1, 2]] and torch.allclose(wt, torch.tensor([[0.5, 0.5]]))
    idx, wt = pr.route(torch.randn(7, 6), 3)
    assert torch.allclose(wt.sum(-1), torch.ones(7), atol=1e-6)
