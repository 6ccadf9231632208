"""The Ruzunex decoder, written down as a :class:`ModelSpec`.

This file holds no arithmetic.  It says which parts the design is made of, with which tensor names and which
config.json values:

* a residual that is ``streams`` copies wide (hyper-connections), all equal to the embedding row at the start and
  summed before the last norm; every sub-layer reads a weighted sum of the streams through an RMS norm, and what it
  reads is replaced by itself plus a short causal convolution over time (``canon.taps`` taps per channel);
* the mixer is "attention" (grouped-query attention with norms per head on queries and keys, no rotation, a bias
  slope_h (i - j) with slope_h = 2^(-8 (h + 1) / H) taken off the scores, a sliding window, values blended with those
  of the first layer that says ``v_mix``, a sigmoid gate on the heads) or "parallel": two mixers side by side on the
  same input, summed with two scales.  Left: attention behind short convolutions on q, k and v, norms over the whole
  projection, a partial rotation, a learned factor per head on the scores, every earlier key visible and a sink in
  the softmax.  Right: HGRN2, a linear recurrence whose key is the complement of its forget gate;
* the feed-forward is a gated dense one with the tanh form of gelu, or routed experts with a clamped activation,
  chosen by their softmax scores over all experts and weighed by their share of the chosen scores;
* tensors: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.canon1|canon2``, ``l<i>.hc1|hc2.in|out|mix``, ``l<i>.mix.*``,
  ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import ConfigError, register_architecture
from ..config.ruzunex import RuzunexConfig
from ..parts.spec import (AttentionSpec, ForgetWriteScanSpec, GatedDenseSpec, InputConvSpec, LayerSpec, MixerSumSpec,
                          ModelSpec, NormSpec, PositionSpec, RoutedExpertsSpec, ScheduleEntry, StreamConnectionSpec,
                          SubLayerSpec)

ARCHITECTURE = "Ruzunex"
VALUES_OF_FIRST = "first_blended_layer"      # the name under which the first layer with v_mix keeps its values


def _window(m: dict):
    return int(m["mask"]["size"]) if m.get("mask") else None


def _sliding(cfg: RuzunexConfig, m: dict, p: str, first_blended: bool) -> AttentionSpec:
    heads, dim = m["heads"], m["dim"]
    blends = bool(m.get("v_mix"))
    return AttentionSpec(
        width=cfg.width, n_heads=heads, n_kv_heads=m["kv_heads"], head_dim=dim, value_dim=m["vdim"],
        scale=float(m["scale"]), position=PositionSpec(kind="none", max_positions=cfg.max_positions),
        q_proj=f"{p}.q", k_proj=f"{p}.k", v_proj=f"{p}.v", o_proj=f"{p}.o", gate_proj=f"{p}.g",
        q_norm=NormSpec(size=dim, eps=cfg.norm_eps, weight=f"{p}.q.norm"),
        k_norm=NormSpec(size=dim, eps=cfg.norm_eps, weight=f"{p}.k.norm"),
        window=_window(m), distance_slopes=tuple(2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)),
        value_publish=VALUES_OF_FIRST if blends and first_blended else None,
        value_blend=(VALUES_OF_FIRST, f"{p}.vmix") if blends and not first_blended else None,
        # every attention layer brings the blend's weight; only the layers that blend read it
        unused=() if blends and not first_blended else ((f"{p}.vmix", ()),))


def _left(cfg: RuzunexConfig, m: dict, p: str) -> AttentionSpec:
    heads, kv_heads, dim = m["heads"], m["kv_heads"], m["dim"]
    rot = m.get("rot")
    position = PositionSpec(kind="none", max_positions=cfg.max_positions) if not rot else \
        PositionSpec(kind="rotary_split_half", rot_dim=int(rot["dims"]), theta=float(rot["base"]),
                     max_positions=cfg.max_positions)
    return AttentionSpec(
        width=cfg.width, n_heads=heads, n_kv_heads=kv_heads, head_dim=dim, value_dim=m["vdim"],
        scale=float(m["scale"]), position=position, q_proj=f"{p}.q", k_proj=f"{p}.k", v_proj=f"{p}.v", o_proj=f"{p}.o",
        q_norm=NormSpec(size=heads * dim, eps=cfg.norm_eps, weight=f"{p}.q.norm"),
        k_norm=NormSpec(size=kv_heads * dim, eps=cfg.norm_eps, weight=f"{p}.k.norm"), norm_whole=True,
        qkv_conv=(f"{p}.q.conv", f"{p}.k.conv", f"{p}.v.conv"), conv_taps=int(m["conv"]),
        head_scale=f"{p}.temp", sink=f"{p}.sink", window=_window(m))


def _right(cfg: RuzunexConfig, m: dict, p: str) -> ForgetWriteScanSpec:
    return ForgetWriteScanSpec(width=cfg.width, n_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"],
                               eps=cfg.norm_eps, q_proj=f"{p}.q", f_proj=f"{p}.f", f_bias=f"{p}.f.b",
                               lower=f"{p}.lower", v_proj=f"{p}.v", out_norm=f"{p}.norm", o_proj=f"{p}.o")


def _feed_forward(cfg: RuzunexConfig, i: int):
    layer, p = cfg.layers[i], f"l{i}.mlp"
    if layer.mlp is None:
        return None
    if layer.mlp_get("kind") == "dense":
        return GatedDenseSpec(width=cfg.width, inner=layer.mlp_get("ff"), gate_proj=f"{p}.gate", up_proj=f"{p}.up",
                              down_proj=f"{p}.down", activation="gelu_tanh")
    router, expert = layer.mlp_get("router"), layer.mlp_get("expert")
    return RoutedExpertsSpec(
        width=cfg.width, inner=expert["ff"], top=router["top"], router=f"{p}.router", router_bias=None,
        experts=tuple((f"{p}.e{e}.gate", f"{p}.e{e}.up", f"{p}.e{e}.down") for e in range(router["experts"])),
        scoring="softmax_share", activation="clamped_swish", limit=float(expert["limit"]), slope=1.702)


def build_spec(cfg: RuzunexConfig) -> ModelSpec:
    layers = []
    seen_blended = False
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}.mix"
        if layer.type == "attention":
            m = dict((k, layer.get(k)) for k in ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "v_mix"))
            mixer = _sliding(cfg, m, p, first_blended=not seen_blended)
            seen_blended = seen_blended or bool(m.get("v_mix"))
        elif layer.type == "parallel":
            mixer = MixerSumSpec(left=_left(cfg, layer.get("left"), f"{p}.left"),
                                 right=_right(cfg, layer.get("right"), f"{p}.right"),
                                 left_scale=float(layer.get("left_scale")), right_scale=float(layer.get("right_scale")))
        else:
            raise ConfigError(f"layer {i}: no mixer of type '{layer.type}'")
        parts = [(mixer, "mixer")]
        ff = _feed_forward(cfg, i)
        if ff is not None or layer.idle_second:
            parts.append((ff, "feed_forward"))
        subs = []
        for q, (part, category) in enumerate(parts, start=1):
            subs.append(SubLayerSpec(
                part=part, category=category,
                norm=NormSpec(size=cfg.width, eps=cfg.norm_eps, weight=f"l{i}.norm{q}"),
                connection=StreamConnectionSpec(streams=cfg.streams, read=f"l{i}.hc{q}.in", gain=f"l{i}.hc{q}.out",
                                                mix=f"l{i}.hc{q}.mix"),
                input_conv=InputConvSpec(width=cfg.width, taps=cfg.canon_taps, weight=f"l{i}.canon{q}")))
        layers.append(LayerSpec(sublayers=tuple(subs), arrangement="hyper_connections"))
    return ModelSpec(
        vocab_size=cfg.vocab,
        width=cfg.width,
        embedding="embed",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(len(layers))),
        final_norm=NormSpec(size=cfg.width, eps=cfg.norm_eps, weight="final.norm"),
        lm_head="head",
        lm_head_optional=False,
        max_positions=cfg.max_positions,
        streams=cfg.streams,
        eos_token_ids=cfg.eos_token_ids,
        architecture=ARCHITECTURE,
    )


register_architecture(ARCHITECTURE, RuzunexConfig, build_spec, model_type="ruzunex", replace=True)
