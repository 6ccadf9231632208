"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..runtime import Runtime
from .basic import Linear, fuse_rows
from .registry import register_feed_forward
from .spec import GatedDenseSpec, PolyNormDenseSpec, RoutedExpertsSpec, TensorDecl


class GatedDense:
    """down( silu(gate(x)) * up(x) ), silu(z) = z / (1 + exp(-z))
    (inferrs-models/src/models/attention_utils.rs:94-118; inferrs-kernels/candle-kernels/src/unary.cu:58-61).
    Gate and up weights are stacked at load: one product feeds the gate kernel, or, for a few rows, one
    kernel does both products and the gate.  With the activation ``clamped_swish`` the gate kernel is
    min(g, limit) sigmoid(slope min(g, limit)) (clamp(u, -limit, limit) + 1), with ``gelu_tanh`` it is
    gelu_tanh(g) u."""

    graph_safe = True  # launches depend only on shapes, never on the step's host-side values

    @staticmethod
    def declare(spec: GatedDenseSpec) -> List[TensorDecl]:
        return [TensorDecl(spec.gate_proj, (spec.inner, spec.width)),
                TensorDecl(spec.up_proj, (spec.inner, spec.width)),
                TensorDecl(spec.down_proj, (spec.width, spec.inner))]

    def __init__(self, spec: GatedDenseSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.activation not in ("silu", "clamped_swish", "gelu_tanh"):
            raise ValueError(f"gated feed-forward: activation '{spec.activation}' has no kernel (only 'silu', "
                             f"'clamped_swish' and 'gelu_tanh')")
        if spec.activation == "clamped_swish" and not (spec.limit is not None and spec.limit > 0):
            raise ValueError(f"gated feed-forward: the clamped activation needs a positive limit, got {spec.limit}")
        self.clamped = spec.activation == "clamped_swish"
        self.gelu = spec.activation == "gelu_tanh"
        self.spec = spec
        self.rt = rt
        self.gate_up = Linear(fuse_rows([weights[spec.gate_proj], weights[spec.up_proj]]), rt)
        self.down = Linear(weights[spec.down_proj], rt)

    def takes_scaled_rows(self, n_rows: int) -> bool:
        return not (self.clamped or self.gelu) and self.gate_up.folds_norms(n_rows) \
            and n_rows <= kernels.SWIGLU_MAX_TOKENS

    def feeds_sink(self, n_rows: int) -> bool:
        return self.down.folds_norms(n_rows)

    def forward(self, ctx, h, sink=None):
        a = torch.empty((h.shape[0], self.spec.inner), dtype=self.rt.dtype, device=h.device)
        if self.gelu:
            kernels.clamped_gate(self.gate_up(h), a, 0.0, 0.0, activation=kernels.GATE_ACT_GELU_TANH)
        elif self.clamped:
            kernels.clamped_gate(self.gate_up(h), a, self.spec.limit, self.spec.slope)
        else:
            kernels.gated_linear(h, self.gate_up.weight, a, self.rt.dtype)
        return self.down(a, sink=sink)


register_feed_forward("gated_dense", GatedDense)


class RoutedExperts:
    """A mixture of small gated feed-forwards (see :class:`~inferrs_b200.parts.spec.RoutedExpertsSpec`).

    The gate and up matrices of all experts (and of the shared one) are stacked at load, and their down matrices stand
    side by side along the inner dimension.  A step is: one product in float32 for the router's logits (and the shared
    expert's gate), one kernel that turns them into a dense row of weights per token (top-k, softmax over the
    chosen, zero for the others), one product for every expert's gate and up rows, one kernel
    silu(g) * u * weight-of-the-column's-expert, and one down product whose sum over the inner dimension is the
    weighted sum over the chosen experts.  A token's result does not depend on what else the step holds; nothing is
    sorted or gathered, so the launches depend on shapes alone.  The price is that every expert's products are made
    for every token: right for a few experts of which a good share is chosen, and for decode steps, where a
    handful of tokens touch most experts' weights anyway.
    """

    graph_safe = True

    @staticmethod
    def declare(spec: RoutedExpertsSpec) -> List[TensorDecl]:
        d = [TensorDecl(spec.router, (len(spec.experts), spec.width))]
        if spec.router_bias is not None:
            d.append(TensorDecl(spec.router_bias, (len(spec.experts),), init="uniform:0:0.1"))
        for gate, up, down in spec.experts:
            d += [TensorDecl(gate, (spec.inner, spec.width)), TensorDecl(up, (spec.inner, spec.width)),
                  TensorDecl(down, (spec.width, spec.inner))]
        if spec.shared is not None:
            gate, up, down, vec = spec.shared
            d += [TensorDecl(gate, (spec.shared_inner, spec.width)), TensorDecl(up, (spec.shared_inner, spec.width)),
                  TensorDecl(down, (spec.width, spec.shared_inner)), TensorDecl(vec, (1, spec.width))]
        return d

    def __init__(self, spec: RoutedExpertsSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        n = len(spec.experts)
        if not 0 < spec.top <= n:
            raise ValueError(f"routed experts: {spec.top} of {n} experts cannot be chosen")
        if spec.shared is not None and spec.shared_inner <= 0:
            raise ValueError("routed experts: a shared expert needs its inner size")
        modes = {"softmax_of_chosen": kernels.ROUTE_SOFTMAX_OF_CHOSEN, "sigmoid_share": kernels.ROUTE_SIGMOID_SHARE,
                 "softmax_share": kernels.ROUTE_SOFTMAX_SHARE}
        if spec.scoring not in modes:
            raise ValueError(f"routed experts: no router scores by '{spec.scoring}'; known: {sorted(modes)}")
        self.mode = modes[spec.scoring]
        if spec.activation not in ("silu", "clamped_swish"):
            raise ValueError(f"routed experts: activation '{spec.activation}' has no kernel (only 'silu' and "
                             f"'clamped_swish')")
        if spec.activation == "clamped_swish" and not (spec.limit is not None and spec.limit > 0):
            raise ValueError(f"routed experts: the clamped activation needs a positive limit, got {spec.limit}")
        if spec.activation == "clamped_swish" and spec.shared is not None:
            raise ValueError("routed experts: the clamped activation has no form with a shared expert")
        self.limit = float(spec.limit) if spec.activation == "clamped_swish" else None
        self.spec, self.rt = spec, rt
        self.n_experts = n
        self.has_shared = spec.shared is not None
        gates = [weights[g] for g, _, _ in spec.experts]
        ups = [weights[u] for _, u, _ in spec.experts]
        downs = [weights[d] for _, _, d in spec.experts]
        router = [weights[spec.router]]
        if self.has_shared:
            gates.append(weights[spec.shared[0]])
            ups.append(weights[spec.shared[1]])
            downs.append(weights[spec.shared[2]])
            router.append(weights[spec.shared[3]].reshape(1, spec.width))
        self.total_inner = n * spec.inner + (spec.shared_inner if self.has_shared else 0)
        self.router = Linear(fuse_rows(router), rt)
        self.router_bias = None if spec.router_bias is None else weights[spec.router_bias].to(torch.float32).contiguous()
        self.gate_up = Linear(fuse_rows(gates + ups), rt)
        if len({t.dtype for t in downs}) > 1:
            downs = [t.to(torch.float32) for t in downs]
        self.down = Linear(torch.cat(downs, dim=1).contiguous(), rt)

    def forward(self, ctx, h):
        n = h.shape[0]
        logits = self.router(h, out_dtype=torch.float32)
        share = torch.empty((n, self.n_experts + int(self.has_shared)), dtype=torch.float32, device=h.device)
        kernels.router_topk(logits, self.router_bias, self.n_experts, self.spec.top, self.has_shared, share,
                            self.rt.dtype, mode=self.mode, scale=self.spec.route_scale)
        a = torch.empty((n, self.total_inner), dtype=self.rt.dtype, device=h.device)
        kernels.routed_gate(self.gate_up(h), share, self.n_experts, self.spec.inner, a, limit=self.limit,
                            slope=self.spec.slope)
        return self.down(a)


register_feed_forward("routed_experts", RoutedExperts)


class PolyNormDense:
    """down( act(up(x)) ), act(z) = a U(z) + b U(z^2) + c U(z^3) + e with U the division of a row by its root mean
    square: a polynomial activation whose three terms are brought to the same size before they are weighed.  The
    sums of the three norms are float32; one kernel reads the up projection's rows once for all three."""

    graph_safe = True

    @staticmethod
    def declare(spec: PolyNormDenseSpec) -> List[TensorDecl]:
        return [TensorDecl(spec.up_proj, (spec.inner, spec.width)),
                TensorDecl(spec.down_proj, (spec.width, spec.inner)),
                TensorDecl(spec.coef, (4,), init="uniform:0.4:0.3")]

    def __init__(self, spec: PolyNormDenseSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.up = Linear(weights[spec.up_proj], rt)
        self.down = Linear(weights[spec.down_proj], rt)
        self.coef = weights[spec.coef].to(torch.float32).contiguous()

    def forward(self, ctx, h):
        z = self.up(h)
        a = torch.empty_like(z)
        kernels.poly_norm(z, self.coef, self.spec.eps, a)
        return self.down(a)


register_feed_forward("poly_norm_dense", PolyNormDense)
