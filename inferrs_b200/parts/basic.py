"""Norm, position encoding and the matrix product that the other parts are made of."""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

from .. import kernels
from ..runtime import Runtime
from .registry import register_norm, register_position
from .spec import NormSpec, PositionSpec, TensorDecl


def _nothing_pending(delta):
    """A block that norms after the sum hands on a copy of the stream instead of an output that is still to be
    added (an object with ``rows`` and no ``delta``): for a norm that means that nothing is pending.  A gated
    output (:class:`GatedUpdate`) becomes plain rows here, for the norms that do not apply the gate themselves."""
    if isinstance(delta, GatedUpdate):
        return delta.rows()
    return None if (delta is not None and hasattr(delta, "rows") and not hasattr(delta, "delta")) else delta


class GatedUpdate:
    """A sub-layer's output that has not been added to the residual stream yet and is to be multiplied by
    sigmoid(gate_pre + gate_bias) on the way: the norm kernel that follows does gate, addition and norm in one pass
    (:class:`LayerNorm`); any other norm asks for the gated rows (:meth:`rows`)."""

    def __init__(self, delta: torch.Tensor, gate_pre: torch.Tensor, gate_bias: Optional[torch.Tensor]):
        self.delta, self.gate_pre, self.gate_bias = delta, gate_pre, gate_bias

    def rows(self) -> torch.Tensor:
        out = torch.empty_like(self.delta)
        kernels.gated_rows(self.delta, self.gate_pre, self.gate_bias, out)
        return out


class StreamUpdate:
    """A sub-layer's output that has not been brought into a residual of several streams yet:
    x_t <- sum_s mix[s, t] x_s + gain[t] * delta.  The norm kernel that follows does it (``mix`` None: the identity;
    ``gain`` None: ones).  ``mix`` and ``gain`` are float32 on the device."""

    def __init__(self, delta: torch.Tensor, mix: Optional[torch.Tensor], gain: Optional[torch.Tensor]):
        self.delta, self.mix, self.gain = delta, mix, gain


class RMSNorm:
    """x / sqrt(mean(x^2) + eps) * w, in float32 (inferrs-kernels/candle-kernels/src/reduce.cu:188-228),
    fused with the residual addition that precedes it in a block.  With ``groups`` > 1 every one of that many equal
    consecutive parts of the row is divided by its own root mean square.  On a residual of several streams
    [rows, streams, width] the kernel also brings the pending output into the streams and reads their weighted
    sum (``read``; None: the plain sum)."""

    graph_safe = True  # launches depend only on shapes, never on the step's host-side values

    @staticmethod
    def declare(spec: NormSpec) -> List[TensorDecl]:
        return [TensorDecl(spec.weight, (spec.size,), init="norm")]

    def __init__(self, spec: NormSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.weight is None:
            raise ValueError("a norm of the residual stream needs a weight")
        self.spec = spec
        self.rt = rt
        self.weight = weights[spec.weight]

    def add_norm(self, residual: torch.Tensor, delta, rows: Optional[torch.Tensor] = None,
                 read: Optional[torch.Tensor] = None):
        delta = _nothing_pending(delta)
        groups = getattr(self.spec, "groups", 1)
        if residual.dim() == 3 or groups != 1 or isinstance(delta, StreamUpdate) or read is not None:
            streams = residual if residual.dim() == 3 else residual.unsqueeze(1)
            update = delta if isinstance(delta, StreamUpdate) else StreamUpdate(delta, None, None)
            n = streams.shape[0] if rows is None else rows.shape[0]
            out = torch.empty((n, self.spec.size), dtype=self.rt.dtype, device=residual.device)
            kernels.stream_add_norm(streams, update.delta, update.mix, update.gain, read, self.weight, groups,
                                    self.spec.eps, out, rows)
            return out
        if isinstance(delta, kernels.ScaledRows):
            # the product before has added its result to the residual stream and folded this norm in (it was given
            # this norm's sink): what it handed on stands for the norm's output
            if rows is not None:
                raise ValueError("scaled rows stand for all rows of a step, not for a choice of them")
            return delta
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.spec.size), dtype=self.rt.dtype, device=residual.device)
        kernels.add_rms_norm(residual, delta, self.weight, self.spec.eps, out, rows)
        return out

    def sink(self, residual: torch.Tensor) -> "kernels.ResidualSink":
        """For a product that can fold the addition to the residual stream and this norm into its read-back."""
        if getattr(self.spec, "groups", 1) != 1 or residual.dim() != 2:
            raise ValueError("a norm in groups, or on a residual of several streams, is not folded into products")
        return kernels.ResidualSink(residual, self.weight, self.spec.eps)

    def norm(self, x: torch.Tensor) -> torch.Tensor:
        """The norm alone, on rows in the activation dtype (a norm on a sub-layer's output)."""
        if getattr(self.spec, "groups", 1) != 1:
            raise ValueError("a norm in groups has no form that stands after a sub-layer")
        out = torch.empty_like(x)
        kernels.rms_norm_rows(x, self.weight, self.spec.eps, out)
        return out


class LayerNorm:
    """(x - mean) / sqrt(variance + eps) * w in float32, the variance being the mean of the squared deviations; no
    bias.  Fused with the residual addition that precedes it in a block, and with the gate on that addition where the
    block before hands on a :class:`GatedUpdate`."""

    graph_safe = True

    @staticmethod
    def declare(spec: NormSpec) -> List[TensorDecl]:
        return [TensorDecl(spec.weight, (spec.size,), init="norm")]

    def __init__(self, spec: NormSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.weight is None or getattr(spec, "groups", 1) != 1:
            raise ValueError("a layer norm of the residual stream has a weight and no groups")
        self.spec = spec
        self.rt = rt
        self.weight = weights[spec.weight].to(torch.float32).contiguous()

    def add_norm(self, residual: torch.Tensor, delta, rows: Optional[torch.Tensor] = None):
        if residual.dim() != 2:
            raise ValueError("a layer norm runs on the plain residual [rows, width]")
        gate_pre = gate_bias = None
        if isinstance(delta, GatedUpdate):
            delta, gate_pre, gate_bias = delta.delta, delta.gate_pre, delta.gate_bias
        else:
            delta = _nothing_pending(delta)
            if isinstance(delta, (StreamUpdate, kernels.ScaledRows)):
                raise ValueError("a layer norm takes plain or gated rows from the block before it")
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.spec.size), dtype=self.rt.dtype, device=residual.device)
        kernels.gated_add_layer_norm(residual, delta, gate_pre, gate_bias, self.weight, self.spec.eps, out, rows)
        return out

    def norm(self, x: torch.Tensor) -> torch.Tensor:
        raise ValueError("a layer norm has no form that stands after a sub-layer")


class NoNorm:
    """No norm: the sub-layer reads (or hands on) the rows as they are.  Still the place where the output of
    the sub-layer before it is added to the residual stream."""

    graph_safe = True

    @staticmethod
    def declare(spec) -> List[TensorDecl]:
        return []

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.spec, self.rt = spec, rt

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        delta = _nothing_pending(delta)
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, residual.shape[1]), dtype=self.rt.dtype, device=residual.device)
        kernels.add_cast(residual, delta, out, rows)
        return out

    def norm(self, x: torch.Tensor) -> torch.Tensor:
        return x


register_norm("rms", RMSNorm)
register_norm("layer_norm", LayerNorm)
register_norm("none", NoNorm)


class RotarySplitHalf:
    """cos/sin of position * theta^(-2i/rot_dim), i < rot_dim/2, all in float32
    (inferrs-models/src/models/attention_utils.rs:186-216); element i is rotated with
    element i + rot_dim/2 (attention_utils.rs:137-151).  The reference casts the tables to the
    run dtype; here they stay float32."""

    def __init__(self, spec: PositionSpec, rt: Runtime):
        if spec.rot_dim <= 0 or spec.rot_dim % 2:
            raise ValueError(f"rot_dim must be positive and even, got {spec.rot_dim}")
        if spec.max_positions <= 0:
            raise ValueError(f"max_positions must be positive, got {spec.max_positions}")
        self.spec = spec
        half = spec.rot_dim // 2
        exponent = torch.arange(half, dtype=torch.float32) * 2.0 / float(spec.rot_dim)
        inv_freq = 1.0 / torch.pow(torch.tensor(float(spec.theta), dtype=torch.float32), exponent)
        angle = torch.arange(spec.max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
        self.cos = torch.cos(angle).contiguous().to(rt.device)
        self.sin = torch.sin(angle).contiguous().to(rt.device)

    def tables(self):
        return self.cos, self.sin, self.spec.rot_dim


class RotaryInterleaved(RotarySplitHalf):
    """The same tables; element 2i of a head is rotated with element 2i + 1."""

    interleaved = True


class RotaryScaled:
    """Pairs as in :class:`RotarySplitHalf`; the frequencies, the stretch of the slow pairs for long contexts and the
    factor on cos and sin are those of :class:`~inferrs_b200.parts.spec.PositionSpec` with ``scaling``.  Frequencies
    and angles are made in float64 on the host and the tables rounded to float32 once."""

    def __init__(self, spec: PositionSpec, rt: Runtime):
        if spec.rot_dim <= 0 or spec.rot_dim % 2:
            raise ValueError(f"rot_dim must be positive and even, got {spec.rot_dim}")
        if spec.max_positions <= 0 or not spec.theta > 1.0:
            raise ValueError(f"max_positions must be positive and theta above 1, got {spec.max_positions}, {spec.theta}")
        self.spec = spec
        dims = spec.rot_dim
        i = torch.arange(dims // 2, dtype=torch.float64)
        freq = float(spec.theta) ** (-2.0 * i / dims)
        magnitude = 1.0
        if spec.scaling is not None:
            factor, original, fast, slow = (float(v) for v in spec.scaling)
            if not (factor > 0 and original > 0 and fast > 0 and slow > 0):
                raise ValueError(f"the scaling's factor, original length, fast and slow turns must be positive: {spec.scaling}")

            def turns(t: float) -> float:      # the pair that makes t turns over the original context
                return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(float(spec.theta)))

            lo = max(math.floor(turns(fast)), 0)
            hi = min(math.ceil(turns(slow)), dims - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            freq = freq / factor * ramp + freq * (1.0 - ramp)
            magnitude = 0.1 * math.log(factor) + 1.0
        angle = torch.arange(spec.max_positions, dtype=torch.float64)[:, None] * freq[None, :]
        self.cos = (torch.cos(angle) * magnitude).to(torch.float32).contiguous().to(rt.device)
        self.sin = (torch.sin(angle) * magnitude).to(torch.float32).contiguous().to(rt.device)

    def tables(self):
        return self.cos, self.sin, self.spec.rot_dim


class NoPosition:
    def __init__(self, spec: PositionSpec, rt: Runtime):
        self.spec = spec

    def tables(self):
        return None, None, 0


register_position("rotary_split_half", RotarySplitHalf)
register_position("rotary_interleaved", RotaryInterleaved)
register_position("rotary_scaled", RotaryScaled)
register_position("none", NoPosition)


def build_position(spec: PositionSpec, rt: Runtime):
    """One table per distinct description, shared by all layers that name it."""
    from .registry import part_class

    key = ("position", spec)
    if key not in rt.shared:
        rt.shared[key] = part_class("position", spec)(spec, rt)
    return rt.shared[key]


def fuse_rows(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    """Stack weight matrices [out_i, in] along ``out``.  Mixed precisions become float32."""
    if len({t.dtype for t in tensors}) > 1:
        tensors = [t.to(torch.float32) for t in tensors]
    return torch.cat(list(tensors), dim=0).contiguous()


class Linear:
    """y = x W^T (+ bias), W stored [out, in] (candle-nn/src/linear.rs:41-82).

    float32 runs: FFMA kernel.  bfloat16 runs: tensor-core product with float32 accumulation for a
    bfloat16 weight; a weight that is stored in float32 keeps its precision and goes through the
    FFMA kernel with the bfloat16 activations widened on the fly.
    """

    def __init__(self, weight: torch.Tensor, rt: Runtime, bias: Optional[torch.Tensor] = None):
        """``bias`` [out] (or shorter: it is added to the first columns) is kept in float32 and added by a kernel of
        its own after the product; a product with a bias folds no norms."""
        if weight.dim() != 2:
            raise ValueError(f"a linear weight must be a matrix, got shape {tuple(weight.shape)}")
        self.weight = weight.contiguous()
        self.rt = rt
        self.n_out, self.n_in = weight.shape
        if bias is not None and (bias.dim() != 1 or bias.shape[0] > self.n_out):
            raise ValueError(f"a bias of shape {tuple(bias.shape)} does not fit {self.n_out} outputs")
        self.bias = None if bias is None else bias.to(torch.float32).contiguous()

    def __call__(self, x, out_dtype: Optional[torch.dtype] = None, sink=None):
        """``x`` may be :class:`~inferrs_b200.kernels.ScaledRows`; with a ``sink`` the result is added to the residual
        stream there and the next norm's scaled rows come back instead of the result."""
        out = torch.empty((x.shape[0], self.n_out), dtype=out_dtype or self.rt.dtype, device=x.device)
        scaled = kernels.linear(x, self.weight, out, self.rt.dtype, sink=sink)
        if self.bias is not None:
            kernels.bias_add(out, self.bias)
        return out if sink is None else scaled

    def folds_norms(self, n_rows: int) -> bool:
        """Whether this product takes scaled rows and feeds a sink at this number of rows."""
        return self.bias is None and kernels.folded_norm_supported(n_rows, self.rt.dtype, self.weight)
