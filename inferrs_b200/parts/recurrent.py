"""Mixers that carry a matrix state per head from token to token instead of a cache of keys and values.

All keep, per request, a float32 state of fixed size in the cache's state slots (one slot per live request, zeroed
when a request takes it) and walk a request's rows in order inside one kernel, so a prompt may be cut anywhere and
a portion may stand beside single tokens of other requests.

Every size is a field of the description; the parts do not know which model or which layer they are in.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..cache.storage import StateNeed
from ..runtime import Runtime
from .basic import Linear, build_position, fuse_rows
from .registry import register_mixer
from .spec import (ChannelDecayScanSpec, FixedDecayScanSpec, ForgetWriteScanSpec, GatedDeltaScanSpec,
                   ScalarGateScanSpec, StateSpaceScanSpec, TensorDecl)


class _ScanMixer:
    """What the two scans share: the fused q/k/v/gate projection, the state, the norm-and-gate step, the output."""

    graph_safe = True  # launches depend only on shapes, never on the step's host-side values

    @staticmethod
    def cache_need(spec):
        return None

    def _build(self, spec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.spec, self.rt = spec, rt
        hd, he = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        self.qkvg = Linear(fuse_rows([weights[spec.q_proj], weights[spec.k_proj], weights[spec.v_proj],
                                      weights[spec.gate_proj]]), rt)
        self.cols = (0, hd, 2 * hd, 2 * hd + he)         # where q, k, v and the gate start in a projected row
        self.o = Linear(weights[spec.o_proj], rt)
        self.out_norm = weights[spec.out_norm]

    def _run(self, ctx, cache_id: int, h, mode: int, gates: torch.Tensor, gate_bias: torch.Tensor, gate_param: float,
             gate_act: int):
        s = self.spec
        n = h.shape[0]
        proj = self.qkvg(h)
        o = torch.empty((n, s.n_heads, s.value_dim), dtype=torch.float32, device=h.device)
        kernels.linear_scan(mode, proj, self.cols[0], self.cols[1], self.cols[2], gates, gate_bias, gate_param,
                            float(s.key_dim) ** -0.5, ctx.storage.state(cache_id), ctx.q_start, ctx.slots,
                            ctx.n_requests, o, s.key_dim, max_rows=ctx.max_q_len)
        gated = torch.empty((n, s.n_heads * s.value_dim), dtype=self.rt.dtype, device=h.device)
        kernels.head_norm_gate(o, proj[:, self.cols[3]:], self.out_norm, True, gate_act, s.eps, gated)
        return self.o(gated)


class ChannelDecayScan(_ScanMixer):
    """Gated linear attention (see :class:`~inferrs_b200.parts.spec.ChannelDecayScanSpec`).  The decay's
    pre-activations come out of their two small products in float32; sigmoid, the root of order tau and the
    recurrence are float32 inside the scan kernel."""

    @staticmethod
    def declare(spec: ChannelDecayScanSpec) -> List[TensorDecl]:
        hd, he = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        return [TensorDecl(spec.q_proj, (hd, spec.width)), TensorDecl(spec.k_proj, (hd, spec.width)),
                TensorDecl(spec.v_proj, (he, spec.width)), TensorDecl(spec.gate_proj, (he, spec.width)),
                TensorDecl(spec.o_proj, (spec.width, he)), TensorDecl(spec.out_norm, (spec.value_dim,), init="norm"),
                TensorDecl(spec.decay_down, (spec.decay_rank, spec.width)),
                TensorDecl(spec.decay_up, (hd, spec.decay_rank)),
                TensorDecl(spec.decay_bias, (hd,), init="uniform:3:2")]

    @staticmethod
    def state_need(spec: ChannelDecayScanSpec) -> Optional[StateNeed]:
        return StateNeed(shape=(spec.n_heads * spec.key_dim * spec.value_dim,))

    def __init__(self, spec: ChannelDecayScanSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.tau <= 0:
            raise ValueError(f"the decay's root must be positive, got tau={spec.tau}")
        self._build(spec, weights, rt)
        self.decay_down = Linear(weights[spec.decay_down], rt)
        self.decay_up = Linear(weights[spec.decay_up], rt)
        self.decay_bias = weights[spec.decay_bias].to(torch.float32).contiguous()

    def forward(self, ctx, cache_id: int, h):
        z = self.decay_up(self.decay_down(h), out_dtype=torch.float32)
        return self._run(ctx, cache_id, h, kernels.SCAN_CHANNEL_DECAY, z, self.decay_bias, self.spec.tau,
                         kernels.GATE_SILU)


class ForgetWriteScan:
    """HGRN2 (see :class:`~inferrs_b200.parts.spec.ForgetWriteScanSpec`).  One product gives q and v; the forget
    gate's pre-activations come out of their product in float32; the scan kernel turns them into the gate with its
    lower bound and into its complement, which stands where other scans have a key, sends q through silu and runs
    the recurrence, all in float32; the norm per head with its shared weight is one kernel before the output
    product.  The state of a slot is the matrices [H, key_dim, value_dim]."""

    graph_safe = True

    @staticmethod
    def declare(spec: ForgetWriteScanSpec) -> List[TensorDecl]:
        hd, he = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        return [TensorDecl(spec.q_proj, (hd, spec.width)), TensorDecl(spec.f_proj, (hd, spec.width)),
                TensorDecl(spec.f_bias, (hd,), init="uniform:1:2"), TensorDecl(spec.lower, (hd,), init="uniform:0.4:0.4"),
                TensorDecl(spec.v_proj, (he, spec.width)), TensorDecl(spec.out_norm, (spec.value_dim,), init="norm"),
                TensorDecl(spec.o_proj, (spec.width, he))]

    @staticmethod
    def cache_need(spec):
        return None

    @staticmethod
    def state_need(spec: ForgetWriteScanSpec) -> Optional[StateNeed]:
        return StateNeed(shape=(spec.n_heads * spec.key_dim * spec.value_dim,))

    def __init__(self, spec: ForgetWriteScanSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.spec, self.rt = spec, rt
        self.hd = spec.n_heads * spec.key_dim
        self.qv = Linear(fuse_rows([weights[spec.q_proj], weights[spec.v_proj]]), rt)
        self.f = Linear(weights[spec.f_proj], rt)
        self.o = Linear(weights[spec.o_proj], rt)
        # the gate's biases and then its lower bounds, as the scan kernel takes them
        self.gate_bias = torch.cat([weights[spec.f_bias].to(torch.float32),
                                    weights[spec.lower].to(torch.float32)]).contiguous()
        self.out_norm = weights[spec.out_norm]

    def forward(self, ctx, cache_id: int, h):
        s = self.spec
        n = h.shape[0]
        proj = self.qv(h)
        z = self.f(h, out_dtype=torch.float32)
        o = torch.empty((n, s.n_heads, s.value_dim), dtype=torch.float32, device=h.device)
        kernels.linear_scan(kernels.SCAN_FORGET_WRITE, proj, 0, 0, self.hd, z, self.gate_bias, 1.0, 1.0,
                            ctx.storage.state(cache_id), ctx.q_start, ctx.slots, ctx.n_requests, o, s.key_dim,
                            max_rows=ctx.max_q_len)
        normed = torch.empty((n, s.n_heads * s.value_dim), dtype=self.rt.dtype, device=h.device)
        kernels.head_norm_gate(o, None, self.out_norm, True, kernels.GATE_SILU, s.eps, normed)
        return self.o(normed)


class ScalarGateScan(_ScanMixer):
    """The matrix memory of xLSTM (see :class:`~inferrs_b200.parts.spec.ScalarGateScanSpec`).  The two gates'
    pre-activations come out of one small product in float32; the caps, the running maximum and the recurrence are
    float32 inside the scan kernel."""

    @staticmethod
    def declare(spec: ScalarGateScanSpec) -> List[TensorDecl]:
        hd, he = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        return [TensorDecl(spec.q_proj, (hd, spec.width)), TensorDecl(spec.k_proj, (hd, spec.width)),
                TensorDecl(spec.v_proj, (he, spec.width)), TensorDecl(spec.gate_proj, (he, spec.width)),
                TensorDecl(spec.o_proj, (spec.width, he)), TensorDecl(spec.out_norm, (he,), init="norm"),
                TensorDecl(spec.i_proj, (spec.n_heads, spec.width)),
                TensorDecl(spec.i_bias, (spec.n_heads,), init="uniform:0:1"),
                TensorDecl(spec.f_proj, (spec.n_heads, spec.width)),
                TensorDecl(spec.f_bias, (spec.n_heads,), init="uniform:3:2")]

    @staticmethod
    def state_need(spec: ScalarGateScanSpec) -> Optional[StateNeed]:
        h, d, e = spec.n_heads, spec.key_dim, spec.value_dim
        return StateNeed(shape=(h * d * e + h * d + h,))     # the matrices, the vectors n, the maxima m

    def __init__(self, spec: ScalarGateScanSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.gate_cap <= 0:
            raise ValueError(f"the gates' cap must be positive, got {spec.gate_cap}")
        self._build(spec, weights, rt)
        self.gates = Linear(fuse_rows([weights[spec.i_proj], weights[spec.f_proj]]), rt)
        self.gate_bias = torch.cat([weights[spec.i_bias].to(torch.float32),
                                    weights[spec.f_bias].to(torch.float32)]).contiguous()

    def forward(self, ctx, cache_id: int, h):
        pre = self.gates(h, out_dtype=torch.float32)
        return self._run(ctx, cache_id, h, kernels.SCAN_SCALAR_GATES, pre, self.gate_bias, self.spec.gate_cap,
                         kernels.GATE_SIGMOID)


class FixedDecayScan:
    """Retention (see :class:`~inferrs_b200.parts.spec.FixedDecayScanSpec`).  One product gives q, k, v and the gate;
    q and k are rotated (k also scaled) into float32 rows, the scan with one constant decay per head runs on those,
    and the per-head division by the root mean square with the silu gate is one kernel before the output product.
    The description's options (silu on q, k and v as they leave the projection, one root mean square over all heads,
    a weight on the normed heads, a sigmoid gate, another factor on k) are flags of the same three kernels."""

    graph_safe = True

    @staticmethod
    def declare(spec: FixedDecayScanSpec) -> List[TensorDecl]:
        hd, he = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        d = [TensorDecl(spec.q_proj, (hd, spec.width)), TensorDecl(spec.k_proj, (hd, spec.width)),
             TensorDecl(spec.v_proj, (he, spec.width)), TensorDecl(spec.gate_proj, (he, spec.width)),
             TensorDecl(spec.o_proj, (spec.width, he))]
        if spec.out_norm is not None:
            d.append(TensorDecl(spec.out_norm, (he,), init="norm"))
        return d

    @staticmethod
    def cache_need(spec):
        return None

    @staticmethod
    def state_need(spec: FixedDecayScanSpec) -> Optional[StateNeed]:
        return StateNeed(shape=(spec.n_heads * spec.key_dim * spec.value_dim,))

    def __init__(self, spec: FixedDecayScanSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if len(spec.decay) != spec.n_heads or any(not 0.0 < float(a) <= 1.0 for a in spec.decay):
            raise ValueError(f"a fixed-decay scan needs one decay in (0, 1] per head, got {spec.decay} for "
                             f"{spec.n_heads} heads")
        self.spec, self.rt = spec, rt
        hd, he = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        self.qkvg = Linear(fuse_rows([weights[spec.q_proj], weights[spec.k_proj], weights[spec.v_proj],
                                      weights[spec.gate_proj]]), rt)
        self.gate_col = 2 * hd + he
        self.o = Linear(weights[spec.o_proj], rt)
        self.decay = torch.tensor([float(a) for a in spec.decay], dtype=torch.float64).to(torch.float32).to(rt.device)
        self.cos, self.sin, self.rot_dim = build_position(spec.position, rt).tables()
        if self.rot_dim > spec.key_dim:
            raise ValueError(f"rot_dim {self.rot_dim} exceeds the key size {spec.key_dim}")
        if spec.input_activation not in (None, "silu") or spec.gate_activation not in ("silu", "sigmoid"):
            raise ValueError(f"a fixed-decay scan has no kernel for the activations '{spec.input_activation}' (inputs) "
                             f"and '{spec.gate_activation}' (gate)")
        act = spec.input_activation == "silu"
        if act and self.rot_dim:
            raise ValueError("a fixed-decay scan rotates its queries and keys or sends them through silu, not both")
        key_scale = float(spec.key_dim) ** -0.5 if spec.key_scale is None else float(spec.key_scale)
        turn = 0 if act else 1
        # q, k and v of a row as float32, side by side
        self.slices = ((0, 0, spec.n_heads, spec.key_dim, turn, 1.0, act),
                       (hd, hd, spec.n_heads, spec.key_dim, turn, key_scale, act),
                       (2 * hd, 2 * hd, spec.n_heads, spec.value_dim, 0, 1.0, act))
        self.out_norm = None if spec.out_norm is None else weights[spec.out_norm]
        self.gate_act = kernels.GATE_SILU if spec.gate_activation == "silu" else kernels.GATE_SIGMOID

    def forward(self, ctx, cache_id: int, h):
        s = self.spec
        n = h.shape[0]
        hd, he = s.n_heads * s.key_dim, s.n_heads * s.value_dim
        proj = self.qkvg(h)
        x = torch.empty((n, 2 * hd + he), dtype=torch.float32, device=h.device)
        kernels.heads_to_float(proj, self.slices, x, self.cos, self.sin, self.rot_dim, ctx.positions)
        o = torch.empty((n, s.n_heads, s.value_dim), dtype=torch.float32, device=h.device)
        kernels.decay_scan(x, 0, hd, 2 * hd, s.n_heads, self.decay, None, None, ctx.storage.state(cache_id), ctx.q_start,
                           ctx.slots, ctx.n_requests, o, s.key_dim, self.rt.dtype, max_rows=ctx.max_q_len)
        gated = torch.empty((n, he), dtype=self.rt.dtype, device=h.device)
        if s.norm_heads_together:        # one root mean square over the heads side by side: one head as wide as all
            o = o.view(n, 1, he)
        kernels.head_norm_gate(o, proj[:, self.gate_col:], self.out_norm, True, self.gate_act, s.eps, gated)
        return self.o(gated)


class GatedDeltaScan:
    """The gated delta rule (see :class:`~inferrs_b200.parts.spec.GatedDeltaScanSpec`).  One product gives the gate,
    q, k, v and the two per-head numbers behind beta and the fade; one kernel does the short convolutions with silu
    (reading what the state keeps of earlier steps) and turns the two numbers into beta and fade in float32; the scan
    makes q and k unit vectors as it fetches them and runs the rule in float32; norm per head, weight and silu gate
    are one kernel before the output product.  The state of a slot is the matrices [H, key_dim, value_dim] and then
    the convolutions' last taps - 1 inputs [taps - 1, channels], float32."""

    graph_safe = True

    @staticmethod
    def _sizes(spec: GatedDeltaScanSpec):
        gd, he = spec.n_kv_heads * spec.key_dim, spec.n_heads * spec.value_dim
        return gd, he, 2 * gd + he           # q or k columns, v or gate columns, the convolutions' channels

    @staticmethod
    def declare(spec: GatedDeltaScanSpec) -> List[TensorDecl]:
        gd, he, _ = GatedDeltaScan._sizes(spec)
        return [TensorDecl(spec.q_proj, (gd, spec.width)), TensorDecl(spec.k_proj, (gd, spec.width)),
                TensorDecl(spec.v_proj, (he, spec.width)),
                TensorDecl(spec.q_conv, (gd, spec.taps), init="uniform:0:0.5"),
                TensorDecl(spec.k_conv, (gd, spec.taps), init="uniform:0:0.5"),
                TensorDecl(spec.v_conv, (he, spec.taps), init="uniform:0:0.5"),
                TensorDecl(spec.beta_proj, (spec.n_heads, spec.width)),
                TensorDecl(spec.a_proj, (spec.n_heads, spec.width)),
                TensorDecl(spec.a_log, (spec.n_heads,), init="uniform:0:1"),
                TensorDecl(spec.dt_bias, (spec.n_heads,), init="uniform:-2:1"),
                TensorDecl(spec.gate_proj, (he, spec.width)),
                TensorDecl(spec.out_norm, (spec.value_dim,), init="norm"),
                TensorDecl(spec.o_proj, (spec.width, he))]

    @staticmethod
    def cache_need(spec):
        return None

    @staticmethod
    def state_need(spec: GatedDeltaScanSpec) -> Optional[StateNeed]:
        _, _, channels = GatedDeltaScan._sizes(spec)
        return StateNeed(shape=(spec.n_heads * spec.key_dim * spec.value_dim + (spec.taps - 1) * channels,))

    def __init__(self, spec: GatedDeltaScanSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.n_heads % spec.n_kv_heads or spec.taps < 1 or spec.unit_eps < 0:
            raise ValueError(f"a gated delta rule needs heads that divide into its key heads, at least one tap and a "
                             f"unit_eps that is not negative, got {spec}")
        self.spec, self.rt = spec, rt
        self.gd, self.he, self.channels = self._sizes(spec)
        # columns of a projected row: gate | q | k | v | a | beta
        self.in_proj = Linear(fuse_rows([weights[spec.gate_proj], weights[spec.q_proj], weights[spec.k_proj],
                                         weights[spec.v_proj], weights[spec.a_proj], weights[spec.beta_proj]]), rt)
        self.o = Linear(weights[spec.o_proj], rt)
        f32 = lambda name: weights[name].to(torch.float32).contiguous()     # noqa: E731
        self.conv = torch.cat([f32(spec.q_conv), f32(spec.k_conv), f32(spec.v_conv)], dim=0).contiguous()
        self.dt_bias, self.a_log = f32(spec.dt_bias), f32(spec.a_log)
        self.out_norm = weights[spec.out_norm]
        self.conv_state_off = spec.n_heads * spec.key_dim * spec.value_dim
        self.a_col = self.he + self.channels

    def forward(self, ctx, cache_id: int, h):
        s = self.spec
        n = h.shape[0]
        proj = self.in_proj(h)
        state = ctx.storage.state(cache_id)
        qkv = torch.empty((n, self.channels), dtype=torch.float32, device=h.device)
        gates = torch.empty((n, 2 * s.n_heads), dtype=torch.float32, device=h.device)      # fade | beta
        kernels.conv_silu_gates(proj, self.he, self.conv, None, state, self.conv_state_off, ctx.q_start, ctx.slots,
                                ctx.row_request, qkv, self.a_col, self.dt_bias, self.a_log, gates,
                                beta_col=self.a_col + s.n_heads)
        kernels.conv_state_shift(proj, self.he, self.channels, s.taps, state, self.conv_state_off, ctx.q_start,
                                 ctx.slots, ctx.n_requests)
        o = torch.empty((n, s.n_heads, s.value_dim), dtype=torch.float32, device=h.device)
        kernels.delta_scan(qkv, 0, self.gd, 2 * self.gd, s.n_kv_heads, gates[:, :s.n_heads], gates[:, s.n_heads:],
                           s.unit_eps, float(s.key_dim) ** -0.5, state, ctx.q_start, ctx.slots, ctx.n_requests, o,
                           s.key_dim, self.rt.dtype, max_rows=ctx.max_q_len)
        gated = torch.empty((n, self.he), dtype=self.rt.dtype, device=h.device)
        kernels.head_norm_gate(o, proj[:, :self.he], self.out_norm, True, kernels.GATE_SILU, s.eps, gated)
        return self.o(gated)


class StateSpaceScan:
    """The state-space mixer of Mamba-2 (see :class:`~inferrs_b200.parts.spec.StateSpaceScanSpec`).  One product gives
    z, x, B, C and dt; one kernel does the short convolution with silu (reading what the state keeps of earlier
    steps) and turns dt into what the scan keeps and takes; the scan runs in float32 with B as keys, C as queries and
    x as values; gate, norm in parts and weight are one kernel before the output product.  The state of a slot is the
    matrices [H, state, value_dim] and then the convolution's last taps - 1 inputs [taps - 1, channels], float32."""

    graph_safe = True

    @staticmethod
    def _sizes(spec: StateSpaceScanSpec):
        inner = spec.n_heads * spec.value_dim
        return inner, inner + 2 * spec.groups * spec.state      # the gate's columns, the convolution's channels

    @staticmethod
    def declare(spec: StateSpaceScanSpec) -> List[TensorDecl]:
        inner, channels = StateSpaceScan._sizes(spec)
        return [TensorDecl(spec.in_proj, (inner + channels + spec.n_heads, spec.width)),
                TensorDecl(spec.conv, (channels, spec.taps), init="uniform:0:0.5"),
                TensorDecl(spec.conv_bias, (channels,), init="uniform:0:0.1"),
                TensorDecl(spec.dt_bias, (spec.n_heads,), init="uniform:-2:1"),
                TensorDecl(spec.a_log, (spec.n_heads,), init="uniform:0:1"),
                TensorDecl(spec.skip, (spec.n_heads,), init="uniform:1:0.2"),
                TensorDecl(spec.out_norm, (inner,), init="norm"),
                TensorDecl(spec.o_proj, (spec.width, inner))]

    @staticmethod
    def cache_need(spec):
        return None

    @staticmethod
    def state_need(spec: StateSpaceScanSpec) -> Optional[StateNeed]:
        _, channels = StateSpaceScan._sizes(spec)
        return StateNeed(shape=(spec.n_heads * spec.state * spec.value_dim + (spec.taps - 1) * channels,))

    def __init__(self, spec: StateSpaceScanSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.n_heads % spec.groups or (spec.n_heads * spec.value_dim) % spec.norm_groups or spec.taps < 1:
            raise ValueError(f"a state-space mixer needs heads that divide into its groups, an inner size that divides "
                             f"into the norm's parts and at least one tap, got {spec}")
        self.spec, self.rt = spec, rt
        self.inner, self.channels = self._sizes(spec)
        self.in_proj = Linear(weights[spec.in_proj], rt)
        self.o = Linear(weights[spec.o_proj], rt)
        f32 = lambda name: weights[name].to(torch.float32).contiguous()     # noqa: E731
        self.conv, self.conv_bias = f32(spec.conv), f32(spec.conv_bias)
        self.dt_bias, self.a_log, self.skip, self.out_norm = (f32(spec.dt_bias), f32(spec.a_log), f32(spec.skip),
                                                              f32(spec.out_norm))
        self.conv_state_off = spec.n_heads * spec.state * spec.value_dim

    def forward(self, ctx, cache_id: int, h):
        s = self.spec
        n = h.shape[0]
        gn = s.groups * s.state
        proj = self.in_proj(h)
        state = ctx.storage.state(cache_id)
        xbc = torch.empty((n, self.channels), dtype=torch.float32, device=h.device)
        gates = torch.empty((n, 2 * s.n_heads), dtype=torch.float32, device=h.device)
        kernels.conv_silu_gates(proj, self.inner, self.conv, self.conv_bias, state, self.conv_state_off, ctx.q_start,
                                ctx.slots, ctx.row_request, xbc, self.inner + self.channels, self.dt_bias, self.a_log,
                                gates)
        kernels.conv_state_shift(proj, self.inner, self.channels, s.taps, state, self.conv_state_off, ctx.q_start,
                                 ctx.slots, ctx.n_requests)
        y = torch.empty((n, s.n_heads, s.value_dim), dtype=torch.float32, device=h.device)
        kernels.decay_scan(xbc, self.inner + gn, self.inner, 0, s.groups, gates[:, :s.n_heads], gates[:, s.n_heads:],
                           self.skip, state, ctx.q_start, ctx.slots, ctx.n_requests, y, s.state, self.rt.dtype,
                           max_rows=ctx.max_q_len)
        gated = torch.empty((n, self.inner), dtype=self.rt.dtype, device=h.device)
        kernels.gate_group_norm(y.view(n, self.inner), proj[:, :self.inner], self.out_norm, s.norm_groups, s.eps, gated)
        return self.o(gated)


register_mixer("channel_decay_scan", ChannelDecayScan)
register_mixer("fixed_decay_scan", FixedDecayScan)
register_mixer("forget_write_scan", ForgetWriteScan)
register_mixer("state_space_scan", StateSpaceScan)
register_mixer("gated_delta_scan", GatedDeltaScan)
register_mixer("scalar_gate_scan", ScalarGateScan)
