"""How a layer's sub-layers and their norms are arranged around the residual stream."""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..cache.storage import StateNeed
from .basic import GatedUpdate, Linear, StreamUpdate
from .registry import register_arrangement
from .spec import TensorDecl


class BuiltSubLayer:
    """A sub-layer whose parts are built: ``part`` with its ``category`` ("mixer" or "feed_forward"),
    the ``norm`` before it and the ``post_norm`` after it (either may be None)."""

    def __init__(self, category: str, part, norm=None, post_norm=None, sum_norm=None):
        self.category, self.part, self.norm, self.post_norm = category, part, norm, post_norm
        self.sum_norm = sum_norm     # the norm of the stream itself after this sub-layer (norm_after_sum blocks)

    def run(self, ctx, cache_id: int, h, sink=None):
        kw = {} if sink is None else {"sink": sink}
        y = self.part.forward(ctx, cache_id, h, **kw) if self.category == "mixer" else self.part.forward(ctx, h, **kw)
        return self.post_norm.norm(y) if self.post_norm is not None else y

    def takes_scaled_rows(self, n_rows: int) -> bool:
        """Whether this sub-layer can be handed scaled rows in place of its norm's output: the norm must be able to
        give a sink to the product before it, and the part must say that it reads scaled rows."""
        f = getattr(self.part, "takes_scaled_rows", None)
        plain_norm = hasattr(self.norm, "sink") and getattr(getattr(self.norm, "spec", None), "groups", 1) == 1
        return f is not None and plain_norm and bool(f(n_rows))

    def feeds_sink(self, n_rows: int) -> bool:
        f = getattr(self.part, "feeds_sink", None)
        return f is not None and self.post_norm is None and bool(f(n_rows))


class SequentialBlock:
    """For every sub-layer in turn: x += post_norm(part(norm(x))).  With two sub-layers, a mixer and a
    feed-forward with a norm each, this is the reference's decoder layer
    (inferrs-models/src/models/qwen3.rs:285-300).

    The residual stream ``x`` is float32 and is updated in place.  An addition is not done where
    the sub-layer ends but inside the norm kernel that follows it, so the block hands its last
    sub-layer's output on as ``pending`` and takes the previous block's in.
    """

    def __init__(self, spec, sublayers: List[BuiltSubLayer]):
        if not sublayers:
            raise ValueError("a layer needs at least one sub-layer")
        if any(s.norm is None for s in sublayers):
            # the output of the sub-layer before is added inside the norm kernel: "no norm" is a part too
            raise ValueError("every sub-layer of a sequential block needs a norm part (NoNorm where there is none)")
        self.spec = spec
        self.sublayers = list(sublayers)

    def parts(self):
        """Every part of the block (the runner asks each whether it is ``graph_safe``)."""
        for s in self.sublayers:
            yield s.part
            if s.norm is not None:
                yield s.norm
            if s.post_norm is not None:
                yield s.post_norm

    def entry(self) -> BuiltSubLayer:
        """The sub-layer that takes what the block before hands on."""
        return self.sublayers[0]

    def forward(self, ctx, cache_id: int, residual: torch.Tensor, pending, after: Optional[BuiltSubLayer] = None):
        """``after``: the sub-layer that runs after this block (the next block's entry), if the caller knows it.  Where
        a sub-layer's last product and the next sub-layer's first both fold norms at this step's number of rows,
        the addition to the residual stream and the norm between them run inside the two products: the producer gets
        the norm's sink and hands on scaled rows, which the norm passes through."""
        n_rows = residual.shape[0]
        for i, s in enumerate(self.sublayers):
            h = s.norm.add_norm(residual, pending)
            nxt = self.sublayers[i + 1] if i + 1 < len(self.sublayers) else after
            fold = nxt is not None and s.feeds_sink(n_rows) and nxt.takes_scaled_rows(n_rows)
            pending = s.run(ctx, cache_id, h, sink=nxt.norm.sink(residual) if fold else None)
        return pending


register_arrangement("sequential", SequentialBlock)


class InputConv:
    """What a sub-layer reads is replaced by itself plus its causal convolution over time, per channel (see
    :class:`~inferrs_b200.parts.spec.InputConvSpec`).  The sums are float32; the last taps - 1 inputs of every
    request are kept in its slot of the state that the description owns under the layer's cache id."""

    def __init__(self, spec, weights):
        if spec.taps < 1:
            raise ValueError(f"a convolution has at least one tap, got {spec.taps}")
        self.spec = spec
        self.weight = weights[spec.weight].to(torch.float32).t().contiguous()      # tap-major, as the kernel reads it

    @staticmethod
    def declare(spec) -> List[TensorDecl]:
        return [TensorDecl(spec.weight, (spec.width, spec.taps), init="uniform:0:0.3")]

    @staticmethod
    def state_need(spec) -> Optional[StateNeed]:
        return StateNeed(shape=((spec.taps - 1) * spec.width,)) if spec.taps > 1 else None

    def __call__(self, ctx, cache_id: int, h: torch.Tensor) -> torch.Tensor:
        s = self.spec
        state = ctx.storage.side_state(cache_id, s) if s.taps > 1 else None
        out = torch.empty_like(h)
        single = ctx.max_q_len == 1          # every request brings one row: the kernel moves the kept rows on itself
        kernels.causal_conv_rows(h, 0, self.weight, state, 0, ctx.q_start, ctx.slots, ctx.row_request, out, True,
                                 shift_single=single)
        if state is not None and not single:
            kernels.conv_state_shift(h, 0, s.width, s.taps, state, 0, ctx.q_start, ctx.slots, ctx.n_requests)
        return out


class HyperConnectionBlock:
    """A block on a residual that is several streams wide, x_1 .. x_S [rows, S, width] in float32.  Every sub-layer has
    a :class:`~inferrs_b200.parts.spec.StreamConnectionSpec`: it reads u = sum_s read[s] x_s through its norm, and
    its output y comes back as x_t <- sum_s mix[s, t] x_s + gain[t] y, all streams at once from the old ones.  A
    sub-layer with an ``input_conv`` reads norm(u) plus its short convolution over time.

    As in :class:`SequentialBlock` the output is not brought in where the sub-layer ends: the norm kernel that
    follows does the update, the read and the norm in one pass over the streams, so the block hands its last
    sub-layer's output on as a pending :class:`~inferrs_b200.parts.basic.StreamUpdate`.
    """

    needs_weights = True     # the model hands the arrangement the weights too: the connections' tensors

    @staticmethod
    def declare(spec) -> List[TensorDecl]:
        out = []
        for s in spec.sublayers:
            c = s.connection
            if c is None:
                raise ValueError("every sub-layer of a hyper-connection block needs a connection")
            out += [TensorDecl(c.read, (c.streams,), init=f"uniform:{1.0 / c.streams}:0.1"),
                    TensorDecl(c.gain, (c.streams,), init="uniform:1:0.2"),
                    TensorDecl(c.mix, (c.streams, c.streams), init="identity:0.1")]
            if s.input_conv is not None:
                out += InputConv.declare(s.input_conv)
        return out

    @staticmethod
    def side_states(spec):
        """The inputs that the sub-layers' convolutions keep, each under its own description."""
        needs = [(s.input_conv, InputConv.state_need(s.input_conv)) for s in spec.sublayers if s.input_conv is not None]
        return [(owner, need) for owner, need in needs if need is not None]

    def __init__(self, spec, sublayers: List[BuiltSubLayer], weights=None, rt=None):
        if not sublayers:
            raise ValueError("a layer needs at least one sub-layer")
        if weights is None:
            raise ValueError("a hyper-connection block needs the weights of its connections")
        self.spec = spec
        self.sublayers = list(sublayers)
        self.connections = []
        for s, built in zip(spec.sublayers, sublayers):
            c = s.connection
            if c is None or not hasattr(built.norm, "add_norm") or built.post_norm is not None:
                raise ValueError("a sub-layer of a hyper-connection block has a connection, a norm before it and none "
                                 "after it")
            self.connections.append(tuple(weights[name].to(torch.float32).contiguous() for name in (c.read, c.gain, c.mix)))
        self.streams = spec.sublayers[0].connection.streams
        if any(s.connection.streams != self.streams for s in spec.sublayers):
            raise ValueError("the sub-layers of a block hang on the same number of streams")
        self.convs = [InputConv(s.input_conv, weights) if s.input_conv is not None else None for s in spec.sublayers]

    def parts(self):
        for s in self.sublayers:
            if s.part is not None:
                yield s.part
            yield s.norm

    def forward(self, ctx, cache_id: int, residual: torch.Tensor, pending):
        if residual.dim() != 3 or residual.shape[1] != self.streams:
            raise ValueError(f"a hyper-connection block of {self.streams} streams got a residual of shape "
                             f"{tuple(residual.shape)}")
        for s, (read, gain, mix), conv in zip(self.sublayers, self.connections, self.convs):
            if s.part is None:       # a sub-layer without a part: its tensors are read and nothing runs
                continue
            h = s.norm.add_norm(residual, pending, read=read)
            if conv is not None:
                h = conv(ctx, cache_id, h)
            pending = StreamUpdate(s.run(ctx, cache_id, h), mix, gain)
        return pending


register_arrangement("hyper_connections", HyperConnectionBlock)


class StreamCopy:
    """What a block that norms after the sum hands on in place of a pending output: nothing is left to add, and
    ``rows`` holds the stream as it stands, in the activation dtype, for whoever reads the stream itself next."""

    def __init__(self, rows: torch.Tensor):
        self.rows = rows


class NormAfterSumBlock:
    """For every sub-layer in turn: x <- norm(scale * x + part(x)), with ``scale`` the layer's ``residual_scale``
    and ``norm`` the sub-layer's ``sum_norm``.  The parts read the stream itself, and the stream itself is
    normalised: float32, in place, by one kernel that also writes the copy in the activation dtype that the next
    part reads.  A sub-layer without a part contributes nothing to its sum.

    The block hands on a :class:`StreamCopy` (the next block of this kind reads it instead of casting the stream
    again); a pending output from a block of another kind is added first.
    """

    def __init__(self, spec, sublayers: List[BuiltSubLayer]):
        if not sublayers:
            raise ValueError("a layer needs at least one sub-layer")
        for s in sublayers:
            if s.sum_norm is None or s.post_norm is not None or not isinstance(s.norm, _no_norm()):
                raise ValueError("a sub-layer of a block that norms after the sum has a sum_norm and no other norm")
            if getattr(s.sum_norm.spec, "groups", 1) != 1:
                raise ValueError("the norm after the sum is a plain RMS norm (no groups)")
        self.spec = spec
        self.sublayers = list(sublayers)
        self.scale = float(spec.residual_scale)
        # norm weights as float32, once
        self.weights = [s.sum_norm.weight.to(torch.float32).contiguous() for s in sublayers]

    def parts(self):
        for s in self.sublayers:
            if s.part is not None:
                yield s.part
            yield s.sum_norm

    def forward(self, ctx, cache_id: int, residual: torch.Tensor, pending):
        if residual.dim() != 2:
            raise ValueError("a block that norms after the sum runs on the plain residual [rows, width]")
        rt_dtype = self.sublayers[0].sum_norm.rt.dtype
        if isinstance(pending, StreamCopy):
            h = pending.rows
        else:
            h = self.sublayers[0].norm.add_norm(residual, pending)      # adds what is pending; the stream as act rows
        for s, w in zip(self.sublayers, self.weights):
            y = s.run(ctx, cache_id, h) if s.part is not None else None
            h = torch.empty(residual.shape, dtype=rt_dtype, device=residual.device)
            kernels.scaled_add_norm(residual, y, self.scale, w, s.sum_norm.spec.eps, h, rt_dtype)
        return StreamCopy(h)


def _no_norm():
    from .basic import NoNorm
    return NoNorm


register_arrangement("norm_after_sum", NormAfterSumBlock)


class GatedResidualBlock:
    """For every sub-layer in turn: h = norm(x), x += sigmoid(W h + b) * part(h), with W and b from the sub-layer's
    :class:`~inferrs_b200.parts.spec.ResidualGateSpec`.  The gate reads the same normalised rows as the part.  A
    sub-layer without a part adds nothing: its norm's and gate's tensors are read and not used.

    As in :class:`SequentialBlock` nothing is added where the sub-layer ends: the block hands its last sub-layer's
    output on with the gate's pre-activations as a pending :class:`~inferrs_b200.parts.basic.GatedUpdate`, and the norm
    kernel that follows does sigmoid, product, addition to the float32 stream and norm in one pass.
    """

    needs_weights = True     # the model hands the arrangement the weights too: the gates' tensors

    @staticmethod
    def declare(spec) -> List[TensorDecl]:
        out = []
        for s in spec.sublayers:
            c = s.connection
            if c is None or not hasattr(c, "weight") or not hasattr(c, "bias"):
                raise ValueError("every sub-layer of a gated-residual block needs a residual gate")
            width = _width_of(s)
            out += [TensorDecl(c.weight, (width, width)), TensorDecl(c.bias, (width,), init="uniform:0:0.5")]
        return out

    def __init__(self, spec, sublayers: List[BuiltSubLayer], weights=None, rt=None):
        if not sublayers:
            raise ValueError("a layer needs at least one sub-layer")
        if weights is None or rt is None:
            raise ValueError("a gated-residual block needs the weights of its gates")
        self.spec = spec
        self.sublayers = list(sublayers)
        self.gates = []
        for s, built in zip(spec.sublayers, sublayers):
            if s.connection is None or built.post_norm is not None or not hasattr(built.norm, "add_norm"):
                raise ValueError("a sub-layer of a gated-residual block has a gate, a norm before it and none after it")
            self.gates.append((Linear(weights[s.connection.weight], rt),
                               weights[s.connection.bias].to(torch.float32).contiguous()))

    def parts(self):
        for s in self.sublayers:
            if s.part is not None:
                yield s.part
            yield s.norm

    def forward(self, ctx, cache_id: int, residual: torch.Tensor, pending):
        if residual.dim() != 2:
            raise ValueError("a gated-residual block runs on the plain residual [rows, width]")
        for s, (gate, bias) in zip(self.sublayers, self.gates):
            if s.part is None:
                continue
            h = s.norm.add_norm(residual, pending)
            y = s.run(ctx, cache_id, h)
            pending = GatedUpdate(y, gate(h), bias)
        return pending


def _width_of(sub) -> int:
    """The stream's width as a sub-layer's descriptions give it."""
    for d in (sub.norm, sub.part):
        for name in ("size", "width"):
            if d is not None and hasattr(d, name):
                return int(getattr(d, name))
    raise ValueError("a sub-layer of a gated-residual block needs a norm or a part that says how wide the stream is")


register_arrangement("gated_residual", GatedResidualBlock)
