"""The Sefalorn decoder, written down as a :class:`ModelSpec`.

This file holds no arithmetic.  It says which parts the design is made of, with which tensor names and which
config.json values:

* a layer is pre-norm with a layer norm that takes the mean out (a weight, no bias), and every sub-layer's result
  joins the stream through a learned gate: h = norm(x), x += sigmoid(rg h + rg.b) * part(h);
* the mixer is "lightning" (linear attention with a fixed decay per head on silu'd queries, keys and values, the heads
  normed together, a sigmoid gate) or "parallel": two mixers side by side on the same input, summed with two scales.
  Left: grouped-query attention without rotation, with biased projections, a logarithmic penalty on distance, the
  heads' scores mixed by a matrix before the softmax, a sliding window, values of a size of their own.  Right: the
  gated delta rule behind short convolutions;
* the feed-forward is routed experts chosen by sigmoid scores, weighed by their share of the chosen scores;
* the last norm is the same layer norm; the logits are multiplied by ``logit_scale``;
* tensors: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.rg1|rg2`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``,
  ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import ConfigError, register_architecture
from ..config.sefalorn import SefalornConfig
from ..parts.spec import (AttentionSpec, FixedDecayScanSpec, GatedDeltaScanSpec, LayerSpec, MixerSumSpec, ModelSpec,
                          NormSpec, PositionSpec, ResidualGateSpec, RoutedExpertsSpec, ScheduleEntry, SubLayerSpec)

ARCHITECTURE = "Sefalorn"


def _norm(cfg: SefalornConfig, name: str) -> NormSpec:
    return NormSpec(size=cfg.width, eps=cfg.norm_eps, weight=name, kind="layer_norm")


def _lightning(cfg: SefalornConfig, m: dict, p: str) -> FixedDecayScanSpec:
    return FixedDecayScanSpec(width=cfg.width, n_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"],
                              decay=tuple(float(a) for a in m["decay"]), eps=cfg.norm_eps,
                              position=PositionSpec(kind="none"), q_proj=f"{p}.q", k_proj=f"{p}.k", v_proj=f"{p}.v",
                              gate_proj=f"{p}.g", o_proj=f"{p}.o", input_activation="silu", key_scale=1.0,
                              norm_heads_together=True, out_norm=f"{p}.norm", gate_activation="sigmoid")


def _left(cfg: SefalornConfig, m: dict, p: str) -> AttentionSpec:
    mask = m.get("mask")
    return AttentionSpec(width=cfg.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
                         value_dim=m["vdim"], scale=float(m["scale"]),
                         position=PositionSpec(kind="none", max_positions=cfg.max_positions),
                         q_proj=f"{p}.q", k_proj=f"{p}.k", v_proj=f"{p}.v", o_proj=f"{p}.o",
                         q_bias=f"{p}.q.b", k_bias=f"{p}.k.b", v_bias=f"{p}.v.b", o_bias=f"{p}.o.b",
                         distance_bias=(f"{p}.r1", f"{p}.r2"), head_mix=f"{p}.talk",
                         window=None if not mask else int(mask["size"]))


def _right(cfg: SefalornConfig, m: dict, p: str) -> GatedDeltaScanSpec:
    return GatedDeltaScanSpec(width=cfg.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], key_dim=m["dim"],
                              value_dim=m["vdim"], taps=m["conv"], eps=cfg.norm_eps, q_proj=f"{p}.q", k_proj=f"{p}.k",
                              v_proj=f"{p}.v", q_conv=f"{p}.q.conv", k_conv=f"{p}.k.conv", v_conv=f"{p}.v.conv",
                              beta_proj=f"{p}.b", a_proj=f"{p}.a", a_log=f"{p}.A_log", dt_bias=f"{p}.dt_bias",
                              gate_proj=f"{p}.g", out_norm=f"{p}.norm", o_proj=f"{p}.o", unit_eps=1e-6)


def _mixer(cfg: SefalornConfig, i: int):
    layer, p = cfg.layers[i], f"l{i}.mix"
    if layer.type == "lightning":
        return _lightning(cfg, dict((k, layer.get(k)) for k in ("heads", "dim", "vdim", "decay")), p)
    if layer.type == "parallel":
        return MixerSumSpec(left=_left(cfg, layer.get("left"), f"{p}.left"),
                            right=_right(cfg, layer.get("right"), f"{p}.right"),
                            left_scale=float(layer.get("left_scale")), right_scale=float(layer.get("right_scale")))
    raise ConfigError(f"layer {i}: no mixer of type '{layer.type}'")


def _feed_forward(cfg: SefalornConfig, i: int):
    layer, p = cfg.layers[i], f"l{i}.mlp"
    if layer.mlp is None:
        return None
    router = layer.mlp_get("router")
    return RoutedExpertsSpec(
        width=cfg.width, inner=layer.mlp_get("expert")["ff"], top=router["top"], router=f"{p}.router",
        router_bias=None,
        experts=tuple((f"{p}.e{e}.gate", f"{p}.e{e}.up", f"{p}.e{e}.down") for e in range(router["experts"])),
        scoring="sigmoid_share", route_scale=float(router["scale"]))


def build_spec(cfg: SefalornConfig) -> ModelSpec:
    layers = []
    for i in range(len(cfg.layers)):
        subs = [SubLayerSpec(part=_mixer(cfg, i), category="mixer", norm=_norm(cfg, f"l{i}.norm1"),
                             connection=ResidualGateSpec(weight=f"l{i}.rg1", bias=f"l{i}.rg1.b"))]
        ff = _feed_forward(cfg, i)
        if ff is not None or cfg.layers[i].idle_second:
            subs.append(SubLayerSpec(part=ff, category="feed_forward", norm=_norm(cfg, f"l{i}.norm2"),
                                     connection=ResidualGateSpec(weight=f"l{i}.rg2", bias=f"l{i}.rg2.b")))
        layers.append(LayerSpec(sublayers=tuple(subs), arrangement="gated_residual"))
    return ModelSpec(
        vocab_size=cfg.vocab,
        width=cfg.width,
        embedding="embed",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(len(layers))),
        final_norm=_norm(cfg, "final.norm"),
        lm_head="head",
        lm_head_optional=False,
        max_positions=cfg.max_positions,
        logit_scale=cfg.logit_scale,
        eos_token_ids=cfg.eos_token_ids,
        architecture=ARCHITECTURE,
    )


register_architecture(ARCHITECTURE, SefalornConfig, build_spec, model_type="sefalorn", replace=True)
