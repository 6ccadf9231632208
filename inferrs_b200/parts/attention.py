"""Grouped-query attention over the paged cache.

The arithmetic is the reference's (inferrs-models/src/models/qwen3.rs:104-196):
project, split into heads, RMSNorm per head on queries and keys, rotate by
position, append keys and values to the cache, scores * scale, causal mask,
softmax, weighted sum of values, output projection.  The reference gathers the
whole context and builds the score matrix with library calls
(inferrs-models/src/models/attention_utils.rs:299-370); here two kernels do it:
one turns the fused projection into rotated queries and writes keys and values
into their pages, one attends over the pages.

Every size is a field of the description; the part does not know which model
or which layer it is in.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..cache.storage import KVNeed, StateNeed
from ..runtime import Runtime
from .basic import Linear, build_position, fuse_rows
from .registry import register_mixer
from .spec import AttentionSpec, TensorDecl


class Attention:
    graph_safe = True  # launches depend only on shapes, never on the step's host-side values

    @staticmethod
    def declare(spec: AttentionSpec) -> List[TensorDecl]:
        dv = spec.value_dim or spec.head_dim
        d = [TensorDecl(spec.q_proj, (spec.n_heads * spec.head_dim, spec.width)),
             TensorDecl(spec.o_proj, (spec.width, spec.n_heads * dv))]
        if spec.own_kv:
            d += [TensorDecl(spec.k_proj, (spec.n_kv_heads * spec.head_dim, spec.width)),
                  TensorDecl(spec.v_proj, (spec.n_kv_heads * dv, spec.width))]
        if spec.q_norm is not None and spec.q_norm.weight is not None:
            d.append(TensorDecl(spec.q_norm.weight, (spec.q_norm.size,), init="norm"))
        if spec.k_norm is not None and spec.k_norm.weight is not None and spec.own_kv:
            d.append(TensorDecl(spec.k_norm.weight, (spec.k_norm.size,), init="norm"))
        if spec.q_bias is not None:
            d.append(TensorDecl(spec.q_bias, (spec.n_heads * spec.head_dim,), init="uniform:0:0.1"))
        if spec.own_kv and spec.k_bias is not None:
            d.append(TensorDecl(spec.k_bias, (spec.n_kv_heads * spec.head_dim,), init="uniform:0:0.1"))
        if spec.own_kv and spec.v_bias is not None:
            d.append(TensorDecl(spec.v_bias, (spec.n_kv_heads * dv,), init="uniform:0:0.1"))
        if spec.o_bias is not None:
            d.append(TensorDecl(spec.o_bias, (spec.width,), init="uniform:0:0.1"))
        if spec.distance_bias is not None:
            d += [TensorDecl(spec.distance_bias[0], (spec.n_heads,), init="uniform:0.5:0.4"),
                  TensorDecl(spec.distance_bias[1], (spec.n_heads,), init="uniform:0.5:0.4")]
        if spec.head_mix is not None:
            d.append(TensorDecl(spec.head_mix, (spec.n_heads, spec.n_heads), init="identity:0.2"))
        if spec.head_scale is not None:
            d.append(TensorDecl(spec.head_scale, (spec.n_heads,), init="uniform:1:0.3"))
        if spec.sink is not None:
            d.append(TensorDecl(spec.sink, (spec.n_heads,), init="uniform:0:1"))
        if spec.qkv_conv is not None:
            sizes = (spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim, spec.n_kv_heads * dv)
            d += [TensorDecl(name, (size, spec.conv_taps), init="uniform:0:0.5") for name, size in zip(spec.qkv_conv, sizes)]
        if spec.gate_proj is not None:
            d.append(TensorDecl(spec.gate_proj, (spec.n_heads * dv, spec.width)))
        if spec.value_blend is not None:
            d.append(TensorDecl(spec.value_blend[1], (), init="uniform:0.5:0.3"))
        d += [TensorDecl(name, tuple(shape)) for name, shape in spec.unused]
        return d

    @staticmethod
    def cache_need(spec: AttentionSpec) -> Optional[KVNeed]:
        dv = spec.value_dim if spec.value_dim not in (None, spec.head_dim) else None
        return KVNeed(n_kv_heads=spec.n_kv_heads, head_dim=spec.head_dim, window=spec.window, value_dim=dv)

    @staticmethod
    def state_need(spec: AttentionSpec):
        return None

    @staticmethod
    def side_states(spec: AttentionSpec):
        """The last conv_taps - 1 projected rows of every request, for the convolutions behind q, k and v."""
        if spec.qkv_conv is None or spec.conv_taps <= 1:
            return []
        dv = spec.value_dim or spec.head_dim
        channels = spec.n_heads * spec.head_dim + spec.n_kv_heads * (spec.head_dim + dv)
        return [(spec, StateNeed(shape=((spec.conv_taps - 1) * channels,)))]

    @staticmethod
    def writes_cache(spec: AttentionSpec) -> bool:
        return spec.own_kv

    def __init__(self, spec: AttentionSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} query heads are not a multiple of {spec.n_kv_heads} key/value heads")
        if spec.own_kv and (spec.k_proj is None or spec.v_proj is None):
            raise ValueError("an attention layer with its own keys and values needs k_proj and v_proj")
        for n, heads in ((spec.q_norm, spec.n_heads), (spec.k_norm, spec.n_kv_heads)):
            want = heads * spec.head_dim if spec.norm_whole else spec.head_dim
            if n is not None and (n.kind != "rms" or n.size != want):
                raise ValueError(f"the norm of queries or keys must be an RMS norm over {want} numbers, got {n}")
        if spec.norm_whole and (spec.q_norm is None or spec.k_norm is None or spec.q_norm.weight is None
                                or spec.k_norm.weight is None or spec.norm_after_rotation):
            raise ValueError("norms over the whole projection stand before the rotation, on queries and keys, with weights")
        self.fused = spec.qkv_conv is not None or spec.norm_whole      # the kernel that convolves, norms, turns and stores
        if self.fused and not spec.own_kv:
            raise ValueError("attention with convolutions or norms over the whole projection keeps its own keys and values")
        if spec.qkv_conv is not None and spec.conv_taps < 1:
            raise ValueError(f"a convolution has at least one tap, got {spec.conv_taps}")
        if spec.value_blend is not None and (spec.qkv_conv is not None or not spec.own_kv):
            raise ValueError("values are blended where the layer projects them itself and no convolution follows")
        if spec.distance_slopes is not None and len(spec.distance_slopes) != spec.n_heads:
            raise ValueError(f"{len(spec.distance_slopes)} slopes for {spec.n_heads} heads")
        if spec.q_norm is not None and spec.k_norm is not None and spec.q_norm.eps != spec.k_norm.eps:
            raise ValueError("query and key norms must share eps")
        if spec.window and spec.chunk:
            raise ValueError("an attention layer has a sliding window or chunks, not both")
        self.spec = spec
        self.rt = rt
        self.value_dim = spec.value_dim or spec.head_dim
        self.span = kernels.span_argument(spec.window, spec.chunk)     # which keys a token sees, as the kernels take it
        mats = [weights[spec.q_proj]]
        if spec.own_kv:
            mats += [weights[spec.k_proj], weights[spec.v_proj]]
        # columns of a projected row: q | k | v | gate
        self.v_col = (spec.n_heads + spec.n_kv_heads) * spec.head_dim
        self.gate_col = sum(m.shape[0] for m in mats)
        if spec.gate_proj is not None:
            mats.append(weights[spec.gate_proj])
        self.qkv = Linear(fuse_rows(mats), rt, bias=self._fused_bias(spec, weights, rt))
        f32 = lambda name: weights[name].to(torch.float32).contiguous()     # noqa: E731
        self.head_scale = None if spec.head_scale is None else f32(spec.head_scale)
        self.sinks = None if spec.sink is None else f32(spec.sink)
        self.slopes = None if spec.distance_slopes is None else \
            torch.tensor([float(a) for a in spec.distance_slopes], dtype=torch.float64).to(torch.float32).to(rt.device)
        # the three convolutions' weights side by side, tap-major [taps, channels] as the kernel reads them
        self.conv = None if spec.qkv_conv is None else \
            torch.cat([f32(n) for n in spec.qkv_conv], dim=0).t().contiguous()
        self.blend_weight = None if spec.value_blend is None else f32(spec.value_blend[1]).reshape(1)
        self.o = Linear(weights[spec.o_proj], rt, bias=None if spec.o_bias is None else weights[spec.o_bias])
        # scores penalised by distance and mixed across heads: the mixing is linear, so it is done on the queries
        # (one vector per key/value head and query head, see kernels.mix_queries), and the penalty, mixed the same
        # way, is a table [heads, distances] that the attention kernel takes off the scores
        self.talking = spec.distance_bias is not None or spec.head_mix is not None
        if self.talking and (self.fused or self.head_scale is not None or self.sinks is not None
                             or self.slopes is not None):
            raise ValueError("attention with mixed heads has no kernel that also takes a factor, a slope or a sink per "
                             "head, convolutions or norms over the whole projection")
        if self.talking:
            if not spec.own_kv:
                raise ValueError("attention with mixed heads or a distance penalty keeps its own keys and values")
            h = spec.n_heads
            mix = weights[spec.head_mix].to(torch.float64) if spec.head_mix is not None \
                else torch.eye(h, dtype=torch.float64, device=rt.device)
            self.mix = mix.to(torch.float32).contiguous()
            self.dist_bias = None
            if spec.distance_bias is not None:
                reach = spec.window or spec.position.max_positions
                if not reach or reach <= 0:
                    raise ValueError("a distance penalty needs a window or the model's number of positions "
                                     "(position.max_positions)")
                r1 = weights[spec.distance_bias[0]].to(torch.float64)
                r2 = weights[spec.distance_bias[1]].to(torch.float64)
                dist = torch.arange(reach, dtype=torch.float64, device=rt.device)
                own = r1[:, None] * torch.log1p(r2[:, None] * dist[None, :])           # [heads, distances]
                self.dist_bias = (mix @ own).to(torch.float32).contiguous()
        self.q_weight = weights[spec.q_norm.weight] if spec.q_norm is not None and spec.q_norm.weight else None
        self.k_weight = weights[spec.k_norm.weight] \
            if (spec.k_norm is not None and spec.k_norm.weight and spec.own_kv) else None
        if self.q_weight is not None and self.k_weight is not None and self.q_weight.dtype != self.k_weight.dtype:
            self.q_weight, self.k_weight = self.q_weight.float(), self.k_weight.float()
        self.eps = (spec.q_norm or spec.k_norm).eps if (spec.q_norm or spec.k_norm) else 0.0
        position = build_position(spec.position, rt)
        self.cos, self.sin, self.rot_dim = position.tables()
        self.interleaved = bool(getattr(position, "interleaved", False))   # which elements of a head turn together
        if self.rot_dim > spec.head_dim:
            raise ValueError(f"rot_dim {self.rot_dim} exceeds head_dim {spec.head_dim}")
        if self.fused and (self.interleaved or spec.norm_after_rotation):
            raise ValueError("the kernel that convolves, norms, turns and stores pairs element i with i + rot_dim / 2 "
                             "and norms before the rotation")

    @staticmethod
    def _fused_bias(spec: AttentionSpec, weights, rt: Runtime):
        """The biases of q, k and v side by side as the fused projection's columns lie (zeros where one is absent);
        None if there is none at all."""
        names = [spec.q_bias] + ([spec.k_bias, spec.v_bias] if spec.own_kv else [])
        if all(n is None for n in names):
            return None
        dv = spec.value_dim or spec.head_dim
        sizes = [spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim, spec.n_kv_heads * dv]
        return torch.cat([weights[n].to(torch.float32) if n is not None
                          else torch.zeros(size, dtype=torch.float32, device=rt.device)
                          for n, size in zip(names, sizes)])

    # A block may hand this part scaled rows instead of a norm's output, and a sink instead of taking its result, where
    # both of its products fold norms at the step's number of rows (see SequentialBlock).
    def takes_scaled_rows(self, n_rows: int) -> bool:
        return self.qkv.folds_norms(n_rows)

    def feeds_sink(self, n_rows: int) -> bool:
        return self.o.folds_norms(n_rows)

    def forward(self, ctx, cache_id: int, h, sink=None):
        s = self.spec
        n = h.shape[0]
        qkv = self.qkv(h)
        k_pages, v_pages, group = ctx.storage.pages(cache_id)
        table = ctx.block_tables[group]
        q = torch.empty((n, s.n_heads, s.head_dim), dtype=self.rt.dtype, device=h.device)
        n_values = s.n_kv_heads * self.value_dim
        if s.value_blend is not None:        # v <- (1 - w) v + w v_other, before it is cached
            kernels.blend_columns(qkv, self.v_col, ctx.extra[("values", s.value_blend[0])], self.blend_weight)
        if s.value_publish is not None:      # a view: the projection lives as long as the step
            ctx.extra[("values", s.value_publish)] = qkv[:, self.v_col:self.v_col + n_values]
        if self.fused:
            taps = s.conv_taps if self.conv is not None else 0
            state = ctx.storage.side_state(cache_id, s) if taps > 1 else None
            mode = kernels.NORM_WHOLE if s.norm_whole else \
                (kernels.NORM_PER_HEAD if (s.q_norm is not None or s.k_norm is not None) else kernels.NORM_NONE)
            single = ctx.max_q_len == 1      # every request brings one row: the kernel moves the kept rows on itself
            kernels.conv_norm_rope_store(qkv, s.n_heads, s.n_kv_heads, s.head_dim, self.conv, state, 0, ctx.q_start,
                                         ctx.slots, ctx.row_request, mode, self.q_weight, self.k_weight, self.eps,
                                         self.cos, self.sin, self.rot_dim, ctx.positions, table, k_pages, v_pages, q,
                                         shift_single=single)
            if state is not None and not single:
                kernels.conv_state_shift(qkv, 0, self.gate_col, taps, state, 0, ctx.q_start, ctx.slots, ctx.n_requests)
        else:
            kernels.qk_norm_rope_store(qkv, s.n_heads, s.n_kv_heads, s.head_dim, s.own_kv, self.q_weight, self.k_weight,
                                       self.eps, self.cos, self.sin, self.rot_dim, ctx.positions, ctx.row_request,
                                       table, k_pages, v_pages, q, interleaved=self.interleaved,
                                       norm_q=s.q_norm is not None, norm_k=s.k_norm is not None and s.own_kv,
                                       norm_after_rotation=s.norm_after_rotation)
        out = torch.empty((n, s.n_heads * self.value_dim), dtype=self.rt.dtype, device=h.device)
        if self.talking:
            mixed = torch.empty((n, s.n_heads, s.n_kv_heads * s.head_dim), dtype=self.rt.dtype, device=h.device)
            kernels.mix_queries(q, self.mix, s.n_kv_heads, mixed)
            kernels.joint_attention(mixed, k_pages, v_pages, table, ctx, s.scale, self.span, self.dist_bias, out)
        else:
            per_head = {k: t for k, t in (("head_scale", self.head_scale), ("slopes", self.slopes),
                                          ("sinks", self.sinks)) if t is not None}
            kernels.paged_attention(q, k_pages, v_pages, table, ctx, s.scale, self.span, out, **per_head)
        if s.gate_proj is not None:          # the heads side by side times sigmoid(gate(x))
            gated = torch.empty_like(out)
            kernels.head_norm_gate(out.view(n, s.n_heads, self.value_dim), qkv[:, self.gate_col:], None, False,
                                   kernels.GATE_SIGMOID, 0.0, gated)
            out = gated
        return self.o(out, sink=sink)


register_mixer("attention", Attention)
