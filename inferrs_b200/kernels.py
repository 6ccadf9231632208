"""Python face of the CUDA kernels in ``csrc/``.

Every function checks what it is given (device, dtype, shape, contiguity),
refuses what the kernel does not take with a clear message, and launches on
torch's current CUDA stream.  There is no other implementation behind these
functions: without a CUDA device, ``nvcc`` or a successful build they raise.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import os

import torch

from .csrc.build import load_library

c_int, c_long, c_float, c_void_p = ctypes.c_int, ctypes.c_long, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    "ib_embedding_gather": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "ib_rms_norm_rows": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p],
    "ib_add_cast": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ib_logit_scale_softcap": [c_void_p, c_long, c_float, c_float, c_void_p],
    "ib_resolve_tokens": [c_void_p, c_int, c_void_p, c_int, c_void_p],
    "ib_add_rms_norm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "ib_silu_gate": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ib_act_to_float": [c_void_p, c_void_p, c_long, c_void_p],
    "ib_qk_norm_rope_store": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                              c_float,
                              c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_void_p, c_void_p, c_void_p, c_void_p],
    "ib_paged_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_void_p, c_int,
                                   c_void_p, c_void_p, c_void_p, c_void_p],
    "ib_gemm_tn_simt": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_long, c_long,
                        c_long, c_void_p],
    "ib_paged_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                               c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_int,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "ib_joint_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                               c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_void_p,
                               c_int, c_int, c_void_p, c_void_p, c_void_p],
    "ib_joint_attention_mma_smem": [c_int, c_int, c_int, c_int, c_int],
    "ib_joint_attention_mma_rows": [c_int, c_int, c_int, c_int],
    "ib_paged_attention_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                   c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                                   c_void_p],
    "ib_paged_attention_tcgen05_per_head": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                            c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                            c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "ib_attention_tcgen05_error": [c_int],
    "ib_paged_attention_pair_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                        c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                                        c_void_p],
    "ib_attention_pair_tcgen05_error": [c_int],
    "ib_row_fault": [c_int],
    "ib_row_fault_async": [c_void_p, c_void_p],
    "ib_attention_tcgen05_error_async": [c_void_p, c_void_p],
    "ib_attention_pair_tcgen05_error_async": [c_void_p, c_void_p],
    "ib_attention_decode_error_async": [c_void_p, c_void_p],
    "ib_paged_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                  c_int, c_int, c_float, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p],
    "ib_attention_decode_error": [c_int],
    "ib_argmax": [c_void_p, c_void_p, c_int, c_int, c_long, c_void_p, c_void_p],
    "ib_penalties": [c_void_p, c_long, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                     c_void_p],
    "ib_embedding_streams": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_float, c_int, c_void_p],
    "ib_stream_add_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                           c_int, c_int, c_int, c_float, c_void_p],
    "ib_head_norm_gate": [c_void_p, c_int, c_long, c_long, c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int,
                          c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "ib_poly_norm": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "ib_latent_norm_store": [c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                             c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p],
    "ib_linear_scan": [c_int, c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_long, c_void_p, c_float, c_float,
                       c_void_p, c_long, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "ib_latent_attention": [c_void_p, c_int, c_long, c_long, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_long, c_long, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "ib_gemm_tn_simt_batched": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_long, c_long,
                                c_long, c_int, c_long, c_long, c_long, c_void_p],
    "ib_scaled_add_norm": [c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p],
    "ib_heads_to_float": [c_void_p, c_long, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p],
    "ib_conv_silu_gates": [c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_long, c_long, c_void_p,
                           c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ib_conv_state_shift": [c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_long, c_long, c_void_p, c_void_p, c_int,
                            c_void_p],
    "ib_gate_group_norm": [c_void_p, c_void_p, c_long, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_void_p],
    "ib_clamped_gate": [c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_int, c_void_p],
    "ib_router_topk": [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_float, c_void_p],
    "ib_gated_add_layer_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
                                c_int, c_void_p],
    "ib_gated_rows": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ib_bias_add": [c_void_p, c_long, c_void_p, c_int, c_int, c_void_p],
    "ib_scaled_sum": [c_void_p, c_float, c_void_p, c_float, c_void_p, c_long, c_void_p],
    "ib_mix_queries": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "ib_delta_scan": [c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p, c_long, c_void_p, c_long, c_float, c_float,
                      c_void_p, c_long, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "ib_routed_gate": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float,
                       c_void_p],
    "ib_decay_scan": [c_void_p, c_long, c_int, c_int, c_int, c_int, c_void_p, c_long, c_void_p, c_long, c_void_p,
                      c_void_p, c_long, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "ib_causal_conv_rows": [c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_long, c_long, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_void_p],
    "ib_conv_norm_rope_store": [c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_long,
                                c_long, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p,
                                c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                c_void_p, c_int, c_void_p],
    "ib_blend_columns": [c_void_p, c_long, c_int, c_int, c_void_p, c_long, c_void_p, c_int, c_void_p],
    "ib_sample": [c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int, c_void_p, c_void_p],
}

_LIBS = {}


def _core(act_dtype: torch.dtype):
    """The core library built for this activation dtype, with argument types set."""
    if act_dtype == torch.float32:
        name = "core_f32"
    elif act_dtype == torch.bfloat16:
        name = "core_bf16"
    else:
        raise KernelError(f"activations must be float32 or bfloat16, got {act_dtype}")
    lib = _LIBS.get(name)
    if lib is None:
        lib = load_library(name)
        for fn, args in _SIGNATURES.items():
            f = getattr(lib, fn)
            f.argtypes = args
            f.restype = c_int
        _LIBS[name] = lib
    return lib


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_DEVICE_INDEX = None


def _stream() -> int:
    """The current CUDA stream's handle (the short way where this torch has it: a launch asks for it every time)."""
    global _DEVICE_INDEX
    if _RAW_STREAM is not None:
        if _DEVICE_INDEX is None:
            _DEVICE_INDEX = torch.cuda.current_device()   # one process drives one GPU
        return _RAW_STREAM(_DEVICE_INDEX)
    return torch.cuda.current_stream().cuda_stream


_LAUNCHES = 0


def launch_count() -> int:
    """Kernel launches of this package's own libraries so far (library matrix products are not counted)."""
    return _LAUNCHES


def count_launches(n: int):
    """Add the kernels of a replayed CUDA graph to the count."""
    global _LAUNCHES
    _LAUNCHES += n


def _check(code: int, what: str):
    global _LAUNCHES
    if code == 0:
        _LAUNCHES += 1
        return
    if code == -1:
        raise KernelError(f"{what}: these sizes are not supported by the kernel")
    if code == -2:
        raise KernelError(f"{what}: invalid argument")
    raise KernelError(f"{what}: CUDA launch failed with error {code}")


def _need(t: Optional[torch.Tensor], name: str, dtypes, ndim: Optional[int] = None, optional: bool = False):
    if t is None:
        if optional:
            return
        raise KernelError(f"{name} is required")
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (the kernels have no CPU implementation), got {t.device}")
    if t.dtype not in dtypes:
        raise KernelError(f"{name} must have dtype in {dtypes}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous, got strides {t.stride()} for shape {tuple(t.shape)}")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_W = (torch.float32, torch.bfloat16)
_I = (torch.int32,)


def embedding_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype,
                     scale: float = 1.0):
    """out[r, :] = table[ids[r], :] * scale as float32."""
    _need(table, "table", _W, 2)
    _need(ids, "ids", _I, 1)
    _need(out, "out", (torch.float32,), 2)
    n, width = out.shape
    if ids.shape[0] != n or table.shape[1] != width:
        raise KernelError(f"embedding_gather: ids {tuple(ids.shape)}, table {tuple(table.shape)}, out {tuple(out.shape)}")
    _check(_core(act_dtype).ib_embedding_gather(_p(table), int(table.dtype == torch.float32), _p(ids), _p(out), n,
                                                width, table.shape[0], float(scale), _stream()), "embedding_gather")


def embedding_streams(table: torch.Tensor, ids: torch.Tensor, pos_table: Optional[torch.Tensor],
                      positions: Optional[torch.Tensor], out: torch.Tensor, act_dtype: torch.dtype, scale: float = 1.0):
    """out[r, s, :] = table[ids[r]] * scale + pos_table[positions[r]] for every stream s, in float32
    (``pos_table`` None: no learned positions).  ``out`` is [rows, streams, width]."""
    _need(table, "table", _W, 2)
    _need(ids, "ids", _I, 1)
    _need(out, "out", (torch.float32,), 3)
    _need(pos_table, "pos_table", _W, 2, optional=True)
    n, streams, width = out.shape
    if table.shape[1] != width or ids.shape[0] != n:
        raise KernelError(f"embedding: table {tuple(table.shape)}, ids {tuple(ids.shape)}, out {tuple(out.shape)}")
    if pos_table is not None:
        _need(positions, "positions", _I, 1)
        if pos_table.shape[1] != width or positions.shape[0] != n:
            raise KernelError(f"embedding: position table {tuple(pos_table.shape)} for rows of width {width}")
    _check(_core(act_dtype).ib_embedding_streams(
        _p(table), int(table.dtype == torch.float32), _p(ids), _p(pos_table),
        int(pos_table is not None and pos_table.dtype == torch.float32), _p(positions), _p(out), n, width,
        table.shape[0], 0 if pos_table is None else pos_table.shape[0], float(scale), streams, _stream()),
        "embedding_streams")


def stream_add_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], mix: Optional[torch.Tensor],
                    gain: Optional[torch.Tensor], read: Optional[torch.Tensor], weight: torch.Tensor, groups: int,
                    eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None):
    """On a residual of several streams [rows, S, width] (float32, updated in place unless ``rows`` is given):
    x_t <- sum_s mix[s, t] x_s + gain[t] * delta (``delta`` None: no update; ``mix`` None: the identity; ``gain``
    None: ones), then u = sum_t read[t] x_t (``read`` None: the plain sum), then ``out`` = u with each of its
    ``groups`` equal consecutive parts divided by its root mean square, times ``weight``."""
    act = out.dtype
    _need(residual, "residual", (torch.float32,), 3)
    _need(delta, "delta", (act,), 2, optional=True)
    _need(weight, "weight", _W, 1)
    _need(out, "out", _W, 2)
    _need(rows, "rows", _I, 1, optional=True)
    n_src, streams, width = residual.shape
    for name, t, size in (("mix", mix, streams * streams), ("gain", gain, streams), ("read", read, streams)):
        _need(t, name, (torch.float32,), None, optional=True)
        if t is not None and t.numel() != size:
            raise KernelError(f"stream_add_norm: {name} has {t.numel()} numbers, {size} are needed for {streams} streams")
    n = n_src if rows is None else rows.shape[0]
    if out.shape != (n, width) or weight.shape[0] != width or (delta is not None and delta.shape != (n_src, width)):
        raise KernelError(f"stream_add_norm: residual {tuple(residual.shape)}, out {tuple(out.shape)}, weight "
                          f"{tuple(weight.shape)}, delta {None if delta is None else tuple(delta.shape)}")
    if groups <= 0 or width % groups:
        raise KernelError(f"stream_add_norm: a width of {width} cannot be cut into {groups} equal parts")
    _check(_core(act).ib_stream_add_norm(
        _p(residual), _p(delta), _p(mix), _p(gain), _p(read), _p(weight), int(weight.dtype == torch.float32), _p(out),
        _p(rows), n, streams, width, int(groups), float(eps), _stream()), "stream_add_norm")


GATE_SILU, GATE_SIGMOID = 0, 1


def head_norm_gate(o: torch.Tensor, gate: Optional[torch.Tensor], weight: Optional[torch.Tensor], norm: bool, gate_act: int,
                   eps: float, out: torch.Tensor):
    """out[r, h*E + e] = o[r, h, e] / rms_h * weight * act(gate[r, h*E + e]) with rms_h = sqrt(mean_e(o[r, h]^2) + eps)
    (``norm`` False: no division).  ``o`` is float32 or the activation dtype, [rows, H, E] or any view of that shape
    whose last stride is 1 (a head-major result is read in place); ``gate`` is a [rows, H*E] view of a wider
    projection, or None (no gate: the normed and weighed heads alone); ``weight`` is None, [E] (shared by the heads) or [H*E]; ``gate_act`` is GATE_SILU or GATE_SIGMOID."""
    act = out.dtype
    if not (o.is_cuda and o.dim() == 3 and o.stride(2) == 1 and o.dtype in (torch.float32, act)):
        raise KernelError(f"head_norm_gate: o must be a CUDA [rows, H, E] view with unit last stride in float32 or {act}")
    n, heads, e_dim = o.shape
    if gate is not None and not (gate.is_cuda and gate.dtype == act and gate.shape == (n, heads * e_dim)
                                 and gate.stride(1) == 1):
        raise KernelError(f"head_norm_gate: gate must be a [rows, H*E] view in {act} with unit last stride")
    _need(out, "out", _W, 2)
    _need(weight, "weight", _W, 1, optional=True)
    if out.shape != (n, heads * e_dim) or (weight is not None and weight.shape[0] not in (e_dim, heads * e_dim)):
        raise KernelError(f"head_norm_gate: o {tuple(o.shape)}, out {tuple(out.shape)}, weight "
                          f"{None if weight is None else tuple(weight.shape)}")
    per_head = int(weight is not None and weight.shape[0] == heads * e_dim and heads > 1)
    _check(_core(act).ib_head_norm_gate(
        _p(o), int(o.dtype == torch.float32), o.stride(0), o.stride(1), _p(gate),
        0 if gate is None else gate.stride(0), _p(weight),
        int(weight is not None and weight.dtype == torch.float32), per_head, int(bool(norm)), int(gate_act), float(eps),
        _p(out), n, heads, e_dim, _stream()), "head_norm_gate")


def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float, out: torch.Tensor):
    """out = a z / r1 + b z^2 / r2 + c z^3 / r3 + e per row, r_p = sqrt(mean((z^p)^2) + eps), coef = (a, b, c, e) in
    float32; powers element by element."""
    act = out.dtype
    _need(z, "z", (act,), 2)
    _need(out, "out", _W, 2)
    _need(coef, "coef", (torch.float32,), 1)
    if out.shape != z.shape or coef.shape[0] != 4:
        raise KernelError(f"poly_norm: z {tuple(z.shape)}, out {tuple(out.shape)}, coef {tuple(coef.shape)}")
    _check(_core(act).ib_poly_norm(_p(z), _p(coef), _p(out), z.shape[0], z.shape[1], float(eps), _stream()), "poly_norm")


def latent_norm_store(proj: torch.Tensor, q_col: int, q_weight: torch.Tensor, cq: torch.Tensor, kv_col: int,
                      kv_weight: Optional[torch.Tensor], plane: Optional[torch.Tensor],
                      block_table: Optional[torch.Tensor], row_request: torch.Tensor, positions: torch.Tensor,
                      eps: float):
    """Two slices of the rows of ``proj``, each divided by its root mean square and multiplied by its weight: columns
    q_col.. (as many as ``q_weight`` has) go to ``cq``; columns kv_col.. (as many as ``kv_weight`` has) go to the
    request's page of ``plane`` [pages, page_size, rank] at the row's position (``plane`` None: no second slice)."""
    act = cq.dtype
    _need(proj, "proj", (act,), 2)
    _need(q_weight, "q_weight", _W, 1)
    _need(cq, "cq", _W, 2)
    n, ld = proj.shape
    q_rank = q_weight.shape[0]
    if cq.shape != (n, q_rank) or q_col < 0 or q_col + q_rank > ld:
        raise KernelError(f"latent_norm_store: proj {tuple(proj.shape)}, cq {tuple(cq.shape)}, columns {q_col}..")
    kv_rank, page_size, n_pages, max_pages = 0, 0, 0, 0
    if plane is not None:
        _need(plane, "plane", (act,), 3)
        _need(kv_weight, "kv_weight", (q_weight.dtype,), 1)
        _need(block_table, "block_table", _I, 2)
        _need(row_request, "row_request", _I, 1)
        _need(positions, "positions", _I, 1)
        n_pages, page_size, kv_rank = plane.shape
        max_pages = block_table.shape[1]
        if kv_weight.shape[0] != kv_rank or kv_col < 0 or kv_col + kv_rank > ld:
            raise KernelError(f"latent_norm_store: plane {tuple(plane.shape)}, weight {tuple(kv_weight.shape)}")
    _check(_core(act).ib_latent_norm_store(
        _p(proj), ld, q_col, q_rank, _p(q_weight), _p(cq), kv_col, kv_rank, _p(kv_weight),
        int(q_weight.dtype == torch.float32), _p(plane), _p(block_table), max_pages, page_size, n_pages,
        _p(row_request), _p(positions), n, float(eps), _stream()), "latent_norm_store")


SCAN_CHANNEL_DECAY, SCAN_SCALAR_GATES, SCAN_FORGET_WRITE = 0, 1, 2


def linear_scan(mode: int, proj: torch.Tensor, q_col: int, k_col: int, v_col: int, gates: torch.Tensor,
                gate_bias: torch.Tensor, gate_param: float, q_scale: float, state: torch.Tensor, q_start: torch.Tensor,
                slots: torch.Tensor, n_requests: int, out: torch.Tensor, key_dim: int, max_rows: int = 0):
    """A matrix state per head carried over each request's rows, one token after the other, in float32.

    SCAN_CHANNEL_DECAY:  S = diag(sigmoid(z + b)^(1/gate_param)) S + k v^T,  o = S^T (q * q_scale)
    SCAN_SCALAR_GATES:   i = c tanh((p + b_i)/c), f = logsigmoid(c tanh((r + b_f)/c)), c = gate_param,
                         m' = max(f + m, i), S = exp(f + m - m') S + exp(i - m') k v^T (n likewise with k),
                         o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)
    SCAN_FORGET_WRITE:   f = l + (1 - l) sigmoid(z + b),  S = diag(f) S + (1 - f) v^T,  o = S^T (silu(q) * q_scale);
                         ``gate_bias`` holds b and then l, [2, H*D]; ``k_col`` is not read

    ``proj`` [rows, ld] holds q and k as [H, D] and v as [H, E] from the given columns on; ``gates`` float32 holds z
    [rows, H*D], or p and then r [rows, 2H]; ``out`` is float32 [rows, H, E]; ``state`` float32 [slots, ...] with at
    least H*D*E (+ H*D + H) numbers per slot; request r's rows are q_start[r] .. q_start[r+1]-1, its slot slots[r].
    ``max_rows``: the most rows that a request brings, if the caller knows (1: the form for steps of single tokens)."""
    act = proj.dtype
    _need(proj, "proj", _W, 2)
    _need(gates, "gates", (torch.float32,), 2)
    _need(gate_bias, "gate_bias", (torch.float32,), 1)
    _need(out, "out", (torch.float32,), 3)
    _need(state, "state", (torch.float32,))
    _need(q_start, "q_start", _I, 1)
    _need(slots, "slots", _I, 1)
    n, heads, e_dim = out.shape
    d_dim = int(key_dim)
    width = 2 * heads if mode == SCAN_SCALAR_GATES else heads * d_dim
    n_bias = 2 * width if mode == SCAN_FORGET_WRITE else width
    if mode == SCAN_FORGET_WRITE:
        k_col = q_col
    if proj.shape[0] != n or gates.shape != (n, width) or gate_bias.shape[0] != n_bias or d_dim <= 0 \
            or max(q_col, k_col) + heads * d_dim > proj.shape[1] or v_col + heads * e_dim > proj.shape[1] \
            or q_start.shape[0] < n_requests + 1 or slots.shape[0] < n_requests:
        raise KernelError(f"linear_scan: proj {tuple(proj.shape)}, gates {tuple(gates.shape)}, out {tuple(out.shape)}")
    if d_dim > 256:
        raise KernelError(f"linear_scan: {d_dim} key channels per head are more than the kernel's 256")
    slot_stride = state[0].numel()
    _check(_core(act).ib_linear_scan(
        int(mode), _p(proj), proj.shape[1], q_col, k_col, v_col, _p(gates), gates.shape[1], _p(gate_bias),
        float(gate_param), float(q_scale), _p(state), slot_stride, _p(q_start), _p(slots), int(n_requests), _p(out),
        heads, d_dim, e_dim, int(max_rows), _stream()), "linear_scan")


LATENT_TILE_TOKENS = 2      # tokens of a prompt portion that one block of the tensor-core form takes
LATENT_SLICE_KEYS = 128     # fewest keys per slice when a row's keys are cut over several blocks
LATENT_RESIDENT_BLOCKS = 296   # two blocks of the tensor-core form per SM


def latent_slices(n_rows: int, n_heads: int, max_kv_len: int) -> int:
    """Into how many slices a row's keys are cut: one while the rows alone fill the machine, else as many as give
    every SM its two blocks, each slice with at least ``LATENT_SLICE_KEYS`` keys (measured at 8 and 64 rows of 2,048
    keys: 16 and 4 slices are the fastest)."""
    blocks = n_rows * ((n_heads + 15) // 16)
    if blocks >= LATENT_RESIDENT_BLOCKS:
        return 1
    by_length = max(1, (max_kv_len + LATENT_SLICE_KEYS - 1) // LATENT_SLICE_KEYS)
    return max(1, min(by_length, (LATENT_RESIDENT_BLOCKS + blocks - 1) // blocks, 64))


def latent_attention(q: torch.Tensor, plane: torch.Tensor, block_table: torch.Tensor, row_request: torch.Tensor,
                     positions: torch.Tensor, scale: float, window: Optional[int], out: torch.Tensor, n_slices: int = 1,
                     tiles=None):
    """Attention of every row over its request's cached latents, which serve every head as key and as value:
    out[h, r] = sum_j softmax_j(scale * q[h, r] . c_j) c_j over the visible j.  ``q`` and ``out`` are head-major
    [H, rows, R] (float32 or the activation dtype; the activation dtype), ``plane`` [pages, page_size, R].
    ``tiles`` = (tile_req, tile_row0, n_tiles, q_start): the step's rows cut into tiles of up to ``LATENT_TILE_TOKENS``
    tokens of one request each (``StepContext.attention_tiles``; -1 marks a place without a tile); with one slice the
    tensor-core form then takes a tile per block."""
    act = out.dtype
    _need(q, "q", (torch.float32, act), 3)
    _need(out, "out", _W, 3)
    _need(plane, "plane", (act,), 3)
    _need(block_table, "block_table", _I, 2)
    _need(row_request, "row_request", _I, 1)
    _need(positions, "positions", _I, 1)
    heads, n, rank = q.shape
    n_pages, page_size, r2 = plane.shape
    if out.shape != q.shape or r2 != rank:
        raise KernelError(f"latent_attention: q {tuple(q.shape)}, out {tuple(out.shape)}, plane {tuple(plane.shape)}")
    if rank > 512:
        raise KernelError(f"latent_attention: a latent of {rank} numbers is larger than the kernel's 512")
    ws_acc = ws_ml = None
    if n_slices > 1:
        ws_acc = torch.empty((n * heads * n_slices, rank), dtype=torch.float32, device=q.device)
        ws_ml = torch.empty((n * heads * n_slices, 2), dtype=torch.float32, device=q.device)
    _check(_core(act).ib_latent_attention(
        _p(q), int(q.dtype == torch.float32), rank, n * rank, _p(plane), _p(block_table), block_table.shape[1],
        page_size, n_pages, _p(row_request), _p(positions), n, heads, rank, float(scale), int(window) if window else 0,
        int(n_slices), _p(out), rank, n * rank, _p(ws_acc), _p(ws_ml),
        *((_p(tiles[0]), _p(tiles[1]), _p(tiles[3]), int(tiles[2])) if tiles is not None and n_slices == 1
          else (None, None, None, 0)), _stream()), "latent_attention")
    if n_slices > 1:
        count_launches(1)


def batched_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype):
    """out[b] = x[b] @ w[b].T for b < B: ``x`` [B, rows, K] (any view with unit last stride, so the heads of a
    [rows, B*K] tensor are multiplied in place), ``w`` [B, M, K] and ``out`` [B, rows, M] contiguous.  True 32-bit
    products with float32 activations or weights, else the tensor cores (the vendor's batched product)."""
    if x.dim() != 3 or w.dim() != 3 or out.dim() != 3 or x.stride(2) != 1:
        raise KernelError("batched_linear: x, w and out must have three dimensions, x with unit last stride")
    _need(w, "w", _W, 3)
    _need(out, "out", _W, 3)
    b, n, k = x.shape
    m = w.shape[1]
    if w.shape != (b, m, k) or out.shape != (b, n, m) or not x.is_cuda:
        raise KernelError(f"batched_linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if act_dtype == torch.float32 or w.dtype == torch.float32 or x.dtype == torch.float32:
        code = _core(act_dtype).ib_gemm_tn_simt_batched(
            _p(x), int(x.dtype == torch.float32), _p(w), int(w.dtype == torch.float32), _p(out),
            int(out.dtype == torch.float32), n, m, k, x.stride(1), k, m, b, x.stride(0), m * k, n * m, _stream())
        if code == -1:
            raise KernelError(f"batched_linear: no kernel for x {x.dtype}, w {w.dtype}, out {out.dtype}")
        _check(code, "gemm_tn_simt_batched")
    else:
        torch.bmm(x, w.transpose(1, 2), out=out)


def resolve_tokens(ids: torch.Tensor, carry: torch.Tensor, act_dtype: torch.dtype):
    """ids[i] = carry[-1 - ids[i]] wherever ids[i] < 0: a step's description names tokens that an earlier step
    sampled and the host has not read yet by their place in that step's output."""
    _need(ids, "ids", _I, 1)
    _need(carry, "carry", _I, 1)
    _check(_core(act_dtype).ib_resolve_tokens(_p(ids), ids.shape[0], _p(carry), carry.shape[0], _stream()),
           "resolve_tokens")


def add_rms_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                 out: torch.Tensor, rows: Optional[torch.Tensor] = None):
    """residual += delta (float32, in place when ``rows`` is None); out = rms_norm(residual) * weight.

    With ``rows`` (int32 [W]) only those rows are read and out has W rows; nothing is written back.
    """
    act = out.dtype
    _need(residual, "residual", (torch.float32,), 2)
    _need(delta, "delta", (act,), 2, optional=True)
    _need(weight, "weight", _W, 1)
    _need(out, "out", _W, 2)
    _need(rows, "rows", _I, 1, optional=True)
    n, width = residual.shape
    n_out = n if rows is None else rows.shape[0]
    if weight.shape[0] != width or out.shape != (n_out, width) or (delta is not None and delta.shape != residual.shape):
        raise KernelError(f"add_rms_norm: residual {tuple(residual.shape)}, weight {tuple(weight.shape)}, "
                          f"out {tuple(out.shape)}, delta {None if delta is None else tuple(delta.shape)}")
    _check(_core(act).ib_add_rms_norm(_p(residual), _p(delta), _p(weight), int(weight.dtype == torch.float32),
                                      _p(out), _p(rows), n_out, width, float(eps), _stream()), "add_rms_norm")


def rms_norm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor):
    """out = rms_norm(x) * weight for rows in the activation dtype (a norm on a sub-layer's output)."""
    act = out.dtype
    _need(x, "x", (act,), 2)
    _need(weight, "weight", _W, 1)
    _need(out, "out", _W, 2)
    if out.shape != x.shape or weight.shape[0] != x.shape[1]:
        raise KernelError(f"rms_norm_rows: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    _check(_core(act).ib_rms_norm_rows(_p(x), _p(weight), int(weight.dtype == torch.float32), _p(out), x.shape[0],
                                       x.shape[1], float(eps), _stream()), "rms_norm_rows")


def add_cast(residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
             rows: Optional[torch.Tensor] = None):
    """residual += delta (float32, in place when ``rows`` is None); out = residual in the activation dtype:
    what a sub-layer without a norm reads."""
    act = out.dtype
    _need(residual, "residual", (torch.float32,), 2)
    _need(delta, "delta", (act,), 2, optional=True)
    _need(out, "out", _W, 2)
    _need(rows, "rows", _I, 1, optional=True)
    n, width = residual.shape
    n_out = n if rows is None else rows.shape[0]
    if out.shape != (n_out, width) or (delta is not None and delta.shape != residual.shape):
        raise KernelError(f"add_cast: residual {tuple(residual.shape)}, out {tuple(out.shape)}, "
                          f"delta {None if delta is None else tuple(delta.shape)}")
    _check(_core(act).ib_add_cast(_p(residual), _p(delta), _p(out), _p(rows), n_out, width, _stream()), "add_cast")


def logit_scale_softcap(logits: torch.Tensor, scale: float, softcap: Optional[float], act_dtype: torch.dtype):
    """In place on float32 logits: x *= scale, then x = cap * tanh(x / cap) where a cap is given."""
    _need(logits, "logits", (torch.float32,), 2)
    if softcap is not None and not softcap > 0:
        raise KernelError(f"logit_scale_softcap: the cap must be positive, got {softcap}")
    _check(_core(act_dtype).ib_logit_scale_softcap(_p(logits), logits.numel(), float(scale),
                                                   float(softcap) if softcap else 0.0, _stream()),
           "logit_scale_softcap")


def silu_gate(gate_up: torch.Tensor, out: torch.Tensor):
    """out[r, j] = silu(gate_up[r, j]) * gate_up[r, inner + j]."""
    act = out.dtype
    _need(gate_up, "gate_up", (act,), 2)
    _need(out, "out", _W, 2)
    n, inner = out.shape
    if gate_up.shape != (n, 2 * inner):
        raise KernelError(f"silu_gate: gate_up {tuple(gate_up.shape)} does not match out {tuple(out.shape)}")
    _check(_core(act).ib_silu_gate(_p(gate_up), _p(out), n, inner, _stream()), "silu_gate")


def qk_norm_rope_store(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, store_kv: bool,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot_dim: int,
                       positions: torch.Tensor, row_request: torch.Tensor, block_table: Optional[torch.Tensor],
                       k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], q_out: torch.Tensor,
                       interleaved: bool = False, norm_q: Optional[bool] = None, norm_k: Optional[bool] = None,
                       norm_after_rotation: bool = False):
    """Per-head norm of q and k, rotation by position, q to ``q_out``, k and v into their pages.  Element ``i`` of
    a head's first ``rot_dim / 2`` turns with element ``i + rot_dim / 2``; ``interleaved``: element ``2i`` with ``2i + 1``.

    ``norm_q`` / ``norm_k`` say whether queries / keys are divided by their root mean square (None: where a weight is
    given); a normed kind without a weight is divided and nothing else.  ``norm_after_rotation``: the norm comes
    after the rotation instead of before it.  Values may have another size than keys (the last size of ``v_pages``).

    qkv [N, at least n_heads * d + n_kv_heads * (d + dv)] (queries only when ``store_kv`` is False; columns behind
    them, a gate's for instance, are not read);
    pages [n_pages, n_kv_heads, page_size, d or dv]; block_table int32 [R, max_pages].
    """
    act = q_out.dtype
    _need(qkv, "qkv", (act,), 2)
    _need(q_out, "q_out", _W, 3)
    _need(positions, "positions", _I, 1)
    _need(row_request, "row_request", _I, 1)
    n = qkv.shape[0]
    v_dim = head_dim
    if store_kv:
        _need(v_pages, "v_pages", (act,), 4)
        v_dim = v_pages.shape[3]
    cols = n_heads * head_dim + (n_kv_heads * (head_dim + v_dim) if store_kv else 0)
    if qkv.shape[1] < cols or q_out.shape != (n, n_heads, head_dim) or positions.shape[0] != n \
            or row_request.shape[0] != n:
        raise KernelError(f"qk_norm_rope_store: qkv {tuple(qkv.shape)} (want {cols} columns), q_out "
                          f"{tuple(q_out.shape)}, positions {tuple(positions.shape)}")
    wdt = None
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        _need(w, name, _W, 1, optional=True)
        if w is not None:
            if w.shape[0] != head_dim:
                raise KernelError(f"{name} has {w.shape[0]} elements, head_dim is {head_dim}")
            if wdt is not None and w.dtype != wdt:
                raise KernelError("q_weight and k_weight must have the same dtype")
            wdt = w.dtype
    norm_q = q_weight is not None if norm_q is None else bool(norm_q)
    norm_k = k_weight is not None if norm_k is None else bool(norm_k)
    if (q_weight is not None and not norm_q) or (k_weight is not None and not norm_k):
        raise KernelError("qk_norm_rope_store: a norm weight was given for a kind that is not normed")
    flags = int(norm_q) | (int(norm_k) << 1) | (int(bool(norm_after_rotation)) << 2)
    table_rows = 0
    if rot_dim:
        _need(cos, "cos", (torch.float32,), 2)
        _need(sin, "sin", (torch.float32,), 2)
        if cos.shape[1] != rot_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"rotation tables {tuple(cos.shape)} do not match rot_dim {rot_dim}")
        table_rows = cos.shape[0]
    max_pages = page_size = n_pages = 0
    if store_kv:
        _need(block_table, "block_table", _I, 2)
        _need(k_pages, "k_pages", (act,), 4)
        n_pages, nkv, page_size, d = k_pages.shape
        if (nkv, d) != (n_kv_heads, head_dim) or v_pages.shape[:3] != k_pages.shape[:3]:
            raise KernelError(f"cache pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)} do not match "
                              f"{n_kv_heads} heads of {head_dim}")
        max_pages = block_table.shape[1]
    _check(_core(act).ib_qk_norm_rope_store(
        _p(qkv), qkv.shape[1], n, n_heads, n_kv_heads, head_dim, v_dim, int(store_kv), _p(q_weight), _p(k_weight),
        int(wdt == torch.float32), flags, float(eps), _p(cos) if rot_dim else None, _p(sin) if rot_dim else None, rot_dim,
        int(bool(interleaved)), table_rows, _p(positions), _p(row_request), _p(block_table) if store_kv else None, max_pages, page_size,
        n_pages, _p(k_pages) if store_kv else None, _p(v_pages) if store_kv else None, _p(q_out), _stream()),
        "qk_norm_rope_store")


def row_fault(act_dtype: torch.dtype, reset: bool = True) -> Optional[int]:
    """The first row that a kernel left out because its position lay outside the rotation tables (None if
    there was none).  Waits for the device."""
    v = _core(act_dtype).ib_row_fault(int(reset))
    if v < 0:
        raise KernelError(f"row_fault: CUDA error {-v}")
    return None if v == 0 else v - 1


def span_argument(window: Optional[int], chunk: Optional[int] = None) -> int:
    """How the attention kernels are told which keys a token sees: 0 all keys up to its own, n > 0 the last n of
    them (a sliding window), -n its own chunk of n positions counted from position 0 of the sequence."""
    if window and chunk:
        raise KernelError("attention: a sliding window and chunks together have no kernel")
    if (window is not None and window < 0) or (chunk is not None and chunk < 0):
        raise KernelError(f"attention: a window or a chunk is a positive number of positions, got {window}, {chunk}")
    return int(window) if window else (-int(chunk) if chunk else 0)


def paged_attention_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                            row_request: torch.Tensor, positions: torch.Tensor, scale: float, window: Optional[int],
                            out: torch.Tensor, joint: bool = False, dist_bias: Optional[torch.Tensor] = None,
                            head_scale: Optional[torch.Tensor] = None, slopes: Optional[torch.Tensor] = None,
                            sinks: Optional[torch.Tensor] = None):
    """out[r, h*dv:(h+1)*dv] = attention of token r's head h over its request's cached keys lo..pos.  ``window``:
    see :func:`span_argument` (a negative number: chunks).  Values may have another size dv than keys.

    ``joint``: ``q`` is [rows, H, kv_heads * d], one vector per key/value head side by side, and a score is the sum
    of its products with all key heads of the token (the form that queries mixed by :func:`mix_queries` take).
    ``dist_bias`` float32 [H, L]: dist_bias[h, pos - j] is taken off head h's score against key j (a distance beyond
    the table reads its last entry).

    ``head_scale`` / ``slopes`` / ``sinks``: float32 [H] each.  Head h's scaled score is multiplied by head_scale[h];
    slopes[h] * (pos - j) is taken off it; every row's softmax gets one more term, exp(sinks[h]), in its denominator
    only (no key or value belongs to it; scale, factor and slope leave it alone)."""
    act = out.dtype
    _need(q, "q", (act,), 3)
    for name, t in (("head_scale", head_scale), ("slopes", slopes), ("sinks", sinks)):
        _need(t, name, (torch.float32,), 1, optional=True)
        if t is not None and t.shape[0] != q.shape[1]:
            raise KernelError(f"paged_attention: {name} has {t.shape[0]} numbers for {q.shape[1]} heads")
    _need(k_pages, "k_pages", (act,), 4)
    _need(v_pages, "v_pages", (act,), 4)
    _need(block_table, "block_table", _I, 2)
    _need(row_request, "row_request", _I, 1)
    _need(positions, "positions", _I, 1)
    _need(out, "out", _W, 2)
    _need(dist_bias, "dist_bias", (torch.float32,), 2, optional=True)
    n, nh, dq = q.shape
    n_pages, nkv, page_size, dk = k_pages.shape
    dv = v_pages.shape[3]
    d = dq // nkv if joint else dq
    if dk != d or (joint and dq != nkv * dk) or v_pages.shape[:3] != k_pages.shape[:3] or out.shape != (n, nh * dv) \
            or nh % nkv or (dist_bias is not None and (dist_bias.shape[0] != nh or dist_bias.shape[1] < 1)):
        raise KernelError(f"paged_attention: q {tuple(q.shape)}, pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)}, "
                          f"out {tuple(out.shape)}")
    if d > 512 or dv > 512 or dq > 2048:
        raise KernelError(f"paged_attention: head sizes {dq}, {dv} are larger than the kernel takes (512, or 2048 for "
                          f"joint queries)")
    _check(_core(act).ib_paged_attention_generic(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(row_request),
        _p(positions), n, nh, nkv, d, dv, float(scale), int(window) if window else 0, _p(out), int(bool(joint)),
        _p(dist_bias), 0 if dist_bias is None else dist_bias.shape[1], _p(head_scale), _p(slopes), _p(sinks), _stream()),
        "paged_attention_generic")


def gemm_tn_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype):
    """out = x @ w.T with 32-bit fused multiply-adds in ascending k (no tensor cores)."""
    _need(x, "x", _W, 2)
    _need(w, "w", _W, 2)
    _need(out, "out", _W, 2)
    n, k = x.shape
    m = w.shape[0]
    if w.shape[1] != k or out.shape != (n, m):
        raise KernelError(f"gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    code = _core(act_dtype).ib_gemm_tn_simt(_p(x), int(x.dtype == torch.float32), _p(w),
                                            int(w.dtype == torch.float32), _p(out), int(out.dtype == torch.float32),
                                            n, m, k, k, k, m, _stream())
    if code == -1:
        raise KernelError(f"gemm: no kernel for x {x.dtype}, w {w.dtype}, out {out.dtype} with activations {act_dtype}")
    _check(code, "gemm_tn_simt")


def argmax(logits: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype = torch.float32):
    """out[r] = index of the largest logit of row r (lowest index among equals).  ``act_dtype`` only
    selects which of the two builds of the kernel library serves the call."""
    _need(logits, "logits", (torch.float32,), 2)
    _need(out, "out", _I, 1)
    if out.shape[0] != logits.shape[0]:
        raise KernelError(f"argmax: logits {tuple(logits.shape)}, out {tuple(out.shape)}")
    rows, vocab = logits.shape
    scratch = None
    if vocab > ARGMAX_CHUNK:  # the vocabulary is cut into chunks so that few rows still fill the machine
        scratch = torch.empty((rows, (vocab + ARGMAX_CHUNK - 1) // ARGMAX_CHUNK), dtype=torch.int64,
                              device=logits.device)
    _check(_core(act_dtype).ib_argmax(_p(logits), _p(out), rows, vocab, vocab, _p(scratch), _stream()), "argmax")


_MM_F32_OUT = None  # does this torch give float32 results from a bfloat16 product?


def gemm_tn_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor):
    """out = x @ w.T for bfloat16 x and w on the tensor cores with float32 accumulation.

    The product itself is the vendor library's (cuBLASLt through ``torch.mm``), as the reference
    calls cuBLAS for every matrix product (candle-core/src/cuda_backend/mod.rs:2260-2310).
    ``out`` may be bfloat16 or float32.
    """
    global _MM_F32_OUT
    _need(x, "x", (torch.bfloat16,), 2)
    _need(w, "w", (torch.bfloat16,), 2)
    _need(out, "out", _W, 2)
    if w.shape[1] != x.shape[1] or out.shape != (x.shape[0], w.shape[0]):
        raise KernelError(f"gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
        return
    if _MM_F32_OUT is None:
        try:
            torch.mm(x[:1], w[:8].t(), out_dtype=torch.float32)
            _MM_F32_OUT = True
        except (TypeError, RuntimeError):
            _MM_F32_OUT = False
    if _MM_F32_OUT:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    else:
        gemm_tn_simt(x, w, out, torch.bfloat16)


SSQ_LD = 32   # tokens per part of a list of sums of squares (csrc/gemm_tcgen05.cu)


@dataclass
class ScaledRows:
    """Rows with an RMS norm folded in: ``x`` holds (stream * norm weight) as bfloat16, ``ssq[:n_parts, :rows]`` the
    parts of the stream's sums of squares per row.  The norm's output is x / sqrt(sum(ssq) / width + eps) per row;
    a product that reads ``x`` applies that factor to its result instead (see csrc/gemm_tcgen05.cu)."""

    x: torch.Tensor
    ssq: torch.Tensor
    n_parts: int
    eps: float
    width: int

    @property
    def shape(self):
        return self.x.shape

    @property
    def device(self):
        return self.x.device


@dataclass
class ResidualSink:
    """Where a product's result goes when the addition to the residual stream and the norm that follows are folded
    into its read-back: it is added to ``residual`` (float32, in place) and handed on as :class:`ScaledRows` of the
    norm with weight ``weight`` and ``eps``."""

    residual: torch.Tensor
    weight: torch.Tensor
    eps: float


def folded_norm_supported(n_rows: int, act_dtype: torch.dtype, w: torch.Tensor) -> bool:
    """Whether a product of ``n_rows`` rows with weight ``w`` can take scaled rows or feed a sink: the bfloat16 tcgen05
    product for a few rows does."""
    return (act_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and n_rows <= min(TCGEN05_MAX_TOKENS, SSQ_LD)
            and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0)


# ---- chains of products ---------------------------------------------------------------------------------------
# In a step of a few rows the products whose norms are folded in follow one another without any other kernel between
# them: o projection (sink) -> gate/up (scaled rows) -> down (sink) -> the next layer's q/k/v (scaled rows).
# csrc/gemm_chain.cu runs up to four such products as ONE persistent cooperative kernel whose producers keep streaming
# the next product's weights while the CTAs meet between two products.  On a B200 it came out a little slower than the
# products launched one by one under programmatic dependent launch (a meeting of 148 CTAs through global memory costs
# 5 to 6 us, as much as a kernel's ends), so the parts do not use it; it stands here as a kernel of its own with its
# tests, for shapes and machines where the balance is another.
_CHAIN_WS = {}       # device index -> (workspace, counters, number of CTAs)


class _ChainProduct(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_long), ("w", c_void_p), ("ldw", c_long), ("y", c_void_p), ("ldy", c_long),
                ("n_out", c_int), ("k", c_int), ("gated", c_int),
                ("in_ssq", c_void_p), ("n_in_parts", c_int), ("in_eps", c_float), ("in_width", c_int),
                ("residual", c_void_p), ("ld_res", c_long), ("sink_w", c_void_p), ("sink_w_is_f32", c_int),
                ("out_ssq", c_void_p)]


def _chain_workspace(device: torch.device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _CHAIN_WS.get(idx)
    if ws is None:
        lib = _gemm_lib()
        sms = torch.cuda.get_device_properties(idx).multi_processor_count
        # (the kernel needs the workspace filled with its "not yet" value and the counters zero, and leaves them so)
        ws = (torch.full((lib.ib_gemm_chain_workspace_floats(sms),), lib.ib_gemm_chain_workspace_fill(),
                         dtype=torch.int32, device=device).view(torch.float32),
              torch.zeros((lib.ib_gemm_chain_max_products() + 1,), dtype=torch.int32, device=device), sms)
        _CHAIN_WS[idx] = ws
    return ws


class ProductChain:
    """Up to four products of a few bfloat16 rows (at most 16) that are launched as one kernel by :meth:`launch`.

    ``linear`` and ``gated_linear`` take what the functions of the same names take, ``x`` a tensor or
    :class:`ScaledRows`; a product's output tensor may be the input of a later product of the chain (that is what the
    chain is for) and holds nothing before the launch."""

    def __init__(self):
        self._products = []    # (structure, rows, device, units, what keeps the tensors alive)

    def linear(self, x, w: torch.Tensor, out: torch.Tensor, sink: Optional["ResidualSink"] = None):
        return self._add(x, w, out, sink, gated=False)

    def gated_linear(self, x, w_gate_up: torch.Tensor, out: torch.Tensor):
        if w_gate_up.shape[0] != 2 * out.shape[1] or out.shape[1] % 64 != 0:
            raise KernelError(f"chain: gate/up weights {tuple(w_gate_up.shape)} for out {tuple(out.shape)} "
                              f"(the inner width must be a multiple of 64)")
        self._add(x, w_gate_up, out, None, gated=True)

    def _add(self, x, w, out, sink, gated):
        lib = _gemm_lib()
        if len(self._products) >= lib.ib_gemm_chain_max_products():
            raise KernelError(f"chain: at most {lib.ib_gemm_chain_max_products()} products")
        xt, scaled = _scaled_args(x)
        _need(xt, "x", (torch.bfloat16,), 2)
        _need(w, "w", (torch.bfloat16,), 2)
        _need(out, "out", (torch.bfloat16,), 2)
        n, k = xt.shape
        m = out.shape[1]
        if n > 16 or k % 8 != 0:
            raise KernelError(f"chain: {n} rows of width {k} (at most 16 rows, a width that is a multiple of 8)")
        if w.shape != ((2 * m if gated else m), k) or out.shape[0] != n:
            raise KernelError(f"chain: x {tuple(xt.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if self._products and (self._products[0][1] != n or self._products[0][2] != out.device):
            raise KernelError("chain: all products have the same rows on the same device")
        prod = _ChainProduct(x=_p(xt), ldx=k, w=_p(w), ldw=k, y=_p(out), ldy=m, n_out=m, k=k, gated=int(gated),
                             in_ssq=scaled[0], n_in_parts=scaled[1], in_eps=scaled[2], in_width=scaled[3])
        result, keep = None, [xt, w, out, x]
        if sink is not None:
            _need(sink.residual, "residual", (torch.float32,), 2)
            _need(sink.weight, "sink weight", _W, 1)
            if sink.residual.shape != (n, m) or sink.weight.shape[0] != m or gated:
                raise KernelError(f"chain: residual {tuple(sink.residual.shape)} and norm weight "
                                  f"{tuple(sink.weight.shape)} do not match the result {(n, m)}")
            parts = lib.ib_gemm_chain_ssq_parts(m)
            ssq = torch.empty((parts, SSQ_LD), dtype=torch.float32, device=out.device)
            prod.residual, prod.ld_res, prod.sink_w = _p(sink.residual), m, _p(sink.weight)
            prod.sink_w_is_f32, prod.out_ssq = int(sink.weight.dtype == torch.float32), _p(ssq)
            result = ScaledRows(out, ssq, parts, float(sink.eps), m)
            keep += [sink.residual, sink.weight, ssq]
        units = ((m // 64) if gated else (m + 127) // 128) * ((k + 63) // 64)
        self._products.append((prod, n, out.device, units, keep))
        return result

    def launch(self):
        if not self._products:
            return
        products, self._products = self._products, []
        n_tok, device = products[0][1], products[0][2]
        scratch, counters, sms = _chain_workspace(device)
        grid = min([sms] + [p[3] for p in products])
        arr = (_ChainProduct * len(products))(*[p[0] for p in products])
        code = _gemm_lib().ib_gemm_chain(arr, len(products), n_tok, _p(scratch), _p(counters), grid, _stream())
        if code == -1:
            raise KernelError("chain: these sizes are not supported (up to 16 rows, K a multiple of 8, gated widths a "
                              "multiple of 64)")
        _check(code, "chain of products")


def linear(x, w: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype, sink: Optional[ResidualSink] = None):
    """out = x @ w.T in the precision that ``act_dtype`` and the weight's own dtype ask for.  ``x`` may be
    :class:`ScaledRows`; with ``sink`` the result is added to the residual stream and ``out`` receives the stream times
    the next norm's weight: the returned :class:`ScaledRows` (else None) stand for that norm's output."""
    if isinstance(x, ScaledRows) or sink is not None:
        rows = x.shape[0]
        if not folded_norm_supported(rows, act_dtype, w):
            raise KernelError(f"linear: {rows} rows of {act_dtype} with a {w.dtype} weight cannot take folded norms; "
                              f"ask folded_norm_supported first")
        return gemm_tn_tcgen05(x, w, out, sink=sink)
    if act_dtype == torch.float32 or w.dtype == torch.float32:
        gemm_tn_simt(x, w, out, act_dtype)
    elif x.shape[0] <= TCGEN05_MAX_TOKENS and tcgen05_gemm_supported(x, w):
        gemm_tn_tcgen05(x, w, out)
    else:
        gemm_tn_bf16(x, w, out)
    return None


def gated_linear(x, w_gate_up: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype):
    """out = silu(x @ gate.T) * (x @ up.T), ``w_gate_up`` [2 * inner, k] holding the gate matrix above the up
    matrix.  A few bfloat16 rows run as one tcgen05 kernel; everything else as the product and the gate kernel.
    ``x`` may be :class:`ScaledRows` (a few bfloat16 rows only)."""
    inner = out.shape[1]
    if w_gate_up.shape[0] != 2 * inner:
        raise KernelError(f"gated_linear: weights {tuple(w_gate_up.shape)} do not match out {tuple(out.shape)}")
    if isinstance(x, ScaledRows):
        if not folded_norm_supported(x.shape[0], act_dtype, w_gate_up) or x.shape[0] > SWIGLU_MAX_TOKENS:
            raise KernelError("gated_linear: these rows cannot take a folded norm; ask folded_norm_supported first")
        gemm_swiglu_tcgen05(x, w_gate_up, out)
        return
    if act_dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 \
            and x.shape[0] <= min(TCGEN05_MAX_TOKENS, SWIGLU_MAX_TOKENS) \
            and tcgen05_gemm_supported(x, w_gate_up):
        gemm_swiglu_tcgen05(x, w_gate_up, out)
        return
    gu = torch.empty((x.shape[0], 2 * inner), dtype=act_dtype, device=x.device)
    linear(x, w_gate_up, gu, act_dtype)
    silu_gate(gu, out)


def scaled_add_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], alpha: float, weight: torch.Tensor,
                    eps: float, copy: Optional[torch.Tensor], act_dtype: torch.dtype):
    """The norm after the sum, on the stream itself: residual <- (alpha * residual + delta) / rms * weight, float32 in
    place; ``copy`` (may be None) receives the same rows in the activation dtype.  ``delta`` may be None."""
    _need(residual, "residual", (torch.float32,), 2)
    _need(delta, "delta", (act_dtype,), 2, optional=True)
    _need(weight, "weight", (torch.float32,), 1)
    _need(copy, "copy", (act_dtype,), 2, optional=True)
    n, width = residual.shape
    if weight.shape[0] != width or (delta is not None and delta.shape != residual.shape) \
            or (copy is not None and copy.shape != residual.shape):
        raise KernelError(f"scaled_add_norm: residual {tuple(residual.shape)}, weight {tuple(weight.shape)}, delta "
                          f"{None if delta is None else tuple(delta.shape)}")
    _check(_core(act_dtype).ib_scaled_add_norm(_p(residual), _p(delta), float(alpha), _p(weight), float(eps), _p(copy),
                                               n, width, _stream()), "scaled_add_norm")


def heads_to_float(src: torch.Tensor, slices, dst: torch.Tensor, cos: Optional[torch.Tensor],
                   sin: Optional[torch.Tensor], rot_dim: int, positions: Optional[torch.Tensor]):
    """Up to three slices of a projection's rows as float32.  ``slices``: (first column in ``src``, first column in
    ``dst``, heads, numbers per head, rotate?, scale) each; a rotated slice has the first ``rot_dim`` numbers of each
    head turned by the row's position (element i with i + rot_dim / 2; float32 tables [positions, rot_dim / 2]); every
    number is multiplied by the slice's scale.  A slice may carry a seventh entry: true sends its numbers through silu
    first (such a slice is not rotated)."""
    act = src.dtype
    _need(src, "src", _W, 2)
    _need(dst, "dst", (torch.float32,), 2)
    n = src.shape[0]
    if dst.shape[0] != n or not 1 <= len(slices) <= 3:
        raise KernelError(f"heads_to_float: src {tuple(src.shape)}, dst {tuple(dst.shape)}, {len(slices)} slices")
    turning = any(sl[4] for sl in slices) and rot_dim > 0
    table_rows = 0
    if turning:
        _need(cos, "cos", (torch.float32,), 2)
        _need(sin, "sin", (torch.float32,), 2)
        _need(positions, "positions", _I, 1)
        if cos.shape[1] != rot_dim // 2 or sin.shape != cos.shape or positions.shape[0] != n:
            raise KernelError(f"heads_to_float: rotation tables {tuple(cos.shape)} do not match rot_dim {rot_dim}")
        table_rows = cos.shape[0]
    for a, b, heads, dim, rot, _scale in (sl[:6] for sl in slices):
        if a < 0 or b < 0 or a + heads * dim > src.shape[1] or b + heads * dim > dst.shape[1] or (rot and rot_dim > dim):
            raise KernelError(f"heads_to_float: slice {(a, b, heads, dim)} does not fit src {tuple(src.shape)}, dst "
                              f"{tuple(dst.shape)}")
    k = len(slices)
    ints = [(c_int * k)(*[int(sl[i]) for sl in slices]) for i in range(5)]
    silu = (c_int * k)(*[int(bool(sl[6])) if len(sl) > 6 else 0 for sl in slices])
    if any(s and sl[4] for s, sl in zip(silu, slices)):
        raise KernelError("heads_to_float: a slice is rotated or goes through silu, not both")
    scales = (c_float * k)(*[float(sl[5]) for sl in slices])
    _check(_core(act).ib_heads_to_float(
        _p(src), src.shape[1], k, ints[0], ints[1], ints[2], ints[3], ints[4], silu, scales, _p(dst), dst.shape[1],
        _p(cos) if turning else None, _p(sin) if turning else None, int(rot_dim) if turning else 0, table_rows,
        _p(positions) if turning else None, n, _stream()), "heads_to_float")


def conv_silu_gates(proj: torch.Tensor, conv_col: int, conv_w: torch.Tensor, conv_b: Optional[torch.Tensor],
                    state: torch.Tensor, conv_state_off: int, q_start: torch.Tensor, slots: torch.Tensor,
                    row_request: torch.Tensor, out: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
                    gates: torch.Tensor, beta_col: Optional[int] = None):
    """out[r, c] = silu(b[c] + sum_j w[c, j] * input(r - (taps - 1 - j), c)) for the C channels from column
    ``conv_col`` of ``proj``; an input before the request's first row of the step comes from its state (the last
    taps - 1 inputs, oldest first, [taps - 1, C] float32 from ``conv_state_off`` of its slot).  And per head,
    dt = softplus(proj[r, dt_col + h] + dt_bias[h]): gates[r, h] = exp(-exp(a_log[h]) dt), gates[r, H + h] = dt, or,
    with ``beta_col``, sigmoid(proj[r, beta_col + h]) (the step size of a delta rule).  ``conv_b`` None: no bias."""
    act = proj.dtype
    _need(proj, "proj", _W, 2)
    for name, t, nd in (("conv_w", conv_w, 2), ("dt_bias", dt_bias, 1), ("a_log", a_log, 1),
                        ("out", out, 2), ("gates", gates, 2)):
        _need(t, name, (torch.float32,), nd)
    _need(conv_b, "conv_b", (torch.float32,), 1, optional=True)
    _need(state, "state", (torch.float32,))
    for name, t in (("q_start", q_start), ("slots", slots), ("row_request", row_request)):
        _need(t, name, _I, 1)
    n, ld = proj.shape
    channels, taps = conv_w.shape
    heads = dt_bias.shape[0]
    if out.shape != (n, channels) or gates.shape != (n, 2 * heads) \
            or (conv_b is not None and conv_b.shape[0] != channels) \
            or (beta_col is not None and not 0 <= beta_col <= ld - heads) \
            or a_log.shape[0] != heads or conv_col + channels > ld or dt_col + heads > ld or row_request.shape[0] != n:
        raise KernelError(f"conv_silu_gates: proj {tuple(proj.shape)}, conv {tuple(conv_w.shape)}, out "
                          f"{tuple(out.shape)}, gates {tuple(gates.shape)}")
    _check(_core(act).ib_conv_silu_gates(
        _p(proj), ld, int(conv_col), channels, taps, _p(conv_w), _p(conv_b), _p(state), state[0].numel(),
        int(conv_state_off), _p(q_start), _p(slots), _p(row_request), _p(out), int(dt_col), heads, _p(dt_bias),
        _p(a_log), _p(gates), -1 if beta_col is None else int(beta_col), n, _stream()), "conv_silu_gates")


def conv_state_shift(proj: torch.Tensor, conv_col: int, channels: int, taps: int, state: torch.Tensor,
                     conv_state_off: int, q_start: torch.Tensor, slots: torch.Tensor, n_requests: int):
    """After a step: every request's state keeps the last taps - 1 inputs of its convolution, oldest first."""
    act = proj.dtype
    _need(proj, "proj", _W, 2)
    _need(state, "state", (torch.float32,))
    _need(q_start, "q_start", _I, 1)
    _need(slots, "slots", _I, 1)
    if conv_col + channels > proj.shape[1] or state[0].numel() < conv_state_off + (taps - 1) * channels \
            or q_start.shape[0] < n_requests + 1 or slots.shape[0] < n_requests:
        raise KernelError(f"conv_state_shift: proj {tuple(proj.shape)}, {channels} channels of {taps} taps")
    _check(_core(act).ib_conv_state_shift(_p(proj), proj.shape[1], int(conv_col), int(channels), int(taps), _p(state),
                                          state[0].numel(), int(conv_state_off), _p(q_start), _p(slots),
                                          int(n_requests), _stream()), "conv_state_shift")


def causal_conv_rows(x: torch.Tensor, col: int, conv_w: torch.Tensor, state: Optional[torch.Tensor], state_off: int,
                     q_start: torch.Tensor, slots: torch.Tensor, row_request: torch.Tensor, out: torch.Tensor,
                     add_input: bool, shift_single: bool = False):
    """out[r, c] = (x[r, col + c] if ``add_input``) + sum_j conv_w[j, c] * input(r - (taps - 1 - j), c) for the
    channels c < C = conv_w.shape[1]: a causal convolution per channel over a request's rows, ``conv_w`` [taps, C]
    tap-major, the last tap weighing the row itself.  input(t, c) is this step's row t of the same request, or what the request's slot of ``state``
    keeps from earlier steps: its last taps - 1 inputs, oldest first, [taps - 1, C] float32 from ``state_off`` on
    (:func:`conv_state_shift` writes them after the step; zeros for a new request).  ``x`` is a [rows, ld] view in
    the activation dtype with unit last stride; ``out`` [rows, C].  ``shift_single``, only for steps in which every
    request brings exactly one row: the kernel moves the kept inputs on itself and no :func:`conv_state_shift`
    follows."""
    act = out.dtype
    _need(conv_w, "conv_w", (torch.float32,), 2)
    _need(out, "out", _W, 2)
    _need(q_start, "q_start", _I, 1)
    _need(slots, "slots", _I, 1)
    _need(row_request, "row_request", _I, 1)
    _need(state, "state", (torch.float32,), optional=True)
    if not (x.is_cuda and x.dtype == act and x.dim() == 2 and x.stride(1) == 1):
        raise KernelError(f"causal_conv_rows: x must be a CUDA [rows, ld] view in {act} with unit last stride")
    n = x.shape[0]
    taps, channels = conv_w.shape
    if col < 0 or col + channels > x.shape[1] or out.shape != (n, channels) or row_request.shape[0] != n \
            or (taps > 1 and state is None):
        raise KernelError(f"causal_conv_rows: x {tuple(x.shape)}, columns {col}.., weights {tuple(conv_w.shape)}, out "
                          f"{tuple(out.shape)}")
    _check(_core(act).ib_causal_conv_rows(
        _p(x), x.stride(0), int(col), channels, taps, _p(conv_w), _p(state), 0 if state is None else state[0].numel(),
        int(state_off), _p(q_start), _p(slots), _p(row_request), _p(out), out.stride(0), int(bool(add_input)),
        int(bool(shift_single)), n, _stream()), "causal_conv_rows")


NORM_NONE, NORM_PER_HEAD, NORM_WHOLE = 0, 1, 2


def conv_norm_rope_store(proj: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                         conv_w: Optional[torch.Tensor], state: Optional[torch.Tensor], state_off: int,
                         q_start: torch.Tensor, slots: torch.Tensor, row_request: torch.Tensor, norm_mode: int,
                         q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                         cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot_dim: int, positions: torch.Tensor,
                         block_table: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, q_out: torch.Tensor,
                         shift_single: bool = False):
    """One pass over the first columns q | k | v of ``proj`` [rows, ld] (H heads of D, G heads of D, G heads of E):
    a causal convolution per channel (``conv_w`` [taps, channels], tap-major, the last tap weighing the row itself;
    None: none; earlier steps' inputs from ``state`` as in :func:`causal_conv_rows`, ``shift_single`` likewise), then the norms (NORM_PER_HEAD: every head of q and k divided by its root mean
    square, weights [D] or None; NORM_WHOLE: all of q, and all of k, divided by one root mean square over the whole
    projection, weights [H * D] and [G * D]), then the rotation of every head's first ``rot_dim`` numbers by position
    (i with i + rot_dim / 2); q goes to ``q_out`` [rows, H, D], k and v into their pages."""
    act = q_out.dtype
    _need(q_out, "q_out", _W, 3)
    _need(k_pages, "k_pages", (act,), 4)
    _need(v_pages, "v_pages", (act,), 4)
    _need(block_table, "block_table", _I, 2)
    _need(conv_w, "conv_w", (torch.float32,), 2, optional=True)
    _need(state, "state", (torch.float32,), optional=True)
    for name, t in (("q_start", q_start), ("slots", slots), ("row_request", row_request), ("positions", positions)):
        _need(t, name, _I, 1)
    if not (proj.is_cuda and proj.dtype == act and proj.dim() == 2 and proj.stride(1) == 1):
        raise KernelError(f"conv_norm_rope_store: proj must be a CUDA [rows, ld] view in {act} with unit last stride")
    n = proj.shape[0]
    n_pages, nkv, page_size, d = k_pages.shape
    v_dim = v_pages.shape[3]
    channels = n_heads * head_dim + n_kv_heads * (head_dim + v_dim)
    taps = 0 if conv_w is None else conv_w.shape[0]
    if (nkv, d) != (n_kv_heads, head_dim) or v_pages.shape[:3] != k_pages.shape[:3] or proj.shape[1] < channels \
            or q_out.shape != (n, n_heads, head_dim) or (conv_w is not None and conv_w.shape[1] != channels) \
            or (taps > 1 and state is None) or positions.shape[0] != n or row_request.shape[0] != n:
        raise KernelError(f"conv_norm_rope_store: proj {tuple(proj.shape)}, pages {tuple(k_pages.shape)} / "
                          f"{tuple(v_pages.shape)}, q_out {tuple(q_out.shape)}, "
                          f"weights {None if conv_w is None else tuple(conv_w.shape)}")
    wdt = None
    sizes = {NORM_NONE: (None, None), NORM_PER_HEAD: (head_dim, head_dim),
             NORM_WHOLE: (n_heads * head_dim, n_kv_heads * head_dim)}.get(norm_mode)
    if sizes is None:
        raise KernelError(f"conv_norm_rope_store: unknown norm mode {norm_mode}")
    for name, w, size in (("q_weight", q_weight, sizes[0]), ("k_weight", k_weight, sizes[1])):
        _need(w, name, _W, 1, optional=norm_mode != NORM_WHOLE)
        if w is not None:
            if w.shape[0] != size:
                raise KernelError(f"conv_norm_rope_store: {name} has {w.shape[0]} numbers, the norm wants {size}")
            if wdt is not None and w.dtype != wdt:
                raise KernelError("conv_norm_rope_store: q_weight and k_weight must have the same dtype")
            wdt = w.dtype
    table_rows = 0
    if rot_dim:
        _need(cos, "cos", (torch.float32,), 2)
        _need(sin, "sin", (torch.float32,), 2)
        if cos.shape[1] != rot_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"rotation tables {tuple(cos.shape)} do not match rot_dim {rot_dim}")
        table_rows = cos.shape[0]
    _check(_core(act).ib_conv_norm_rope_store(
        _p(proj), proj.stride(0), n, n_heads, n_kv_heads, head_dim, v_dim, taps, _p(conv_w), _p(state),
        0 if state is None else state[0].numel(), int(state_off), _p(q_start), _p(slots), _p(row_request),
        int(norm_mode), _p(q_weight), _p(k_weight), int(wdt == torch.float32), float(eps),
        _p(cos) if rot_dim else None, _p(sin) if rot_dim else None, int(rot_dim), table_rows, _p(positions),
        _p(block_table), block_table.shape[1], page_size, n_pages, _p(k_pages), _p(v_pages), _p(q_out),
        int(bool(shift_single)), _stream()), "conv_norm_rope_store")


def blend_columns(x: torch.Tensor, col: int, other: torch.Tensor, weight: torch.Tensor):
    """x[r, col + c] <- (1 - weight) x[r, col + c] + weight * other[r, c] in place, for the columns of ``other``
    [rows, C] (any row stride, unit last stride); ``weight`` is one float32 number on the device."""
    act = x.dtype
    _need(x, "x", _W, 2)
    _need(weight, "weight", (torch.float32,))
    if not (other.is_cuda and other.dtype == act and other.dim() == 2 and other.stride(1) == 1) \
            or other.shape[0] != x.shape[0] or col < 0 or col + other.shape[1] > x.shape[1] or weight.numel() != 1:
        raise KernelError(f"blend_columns: x {tuple(x.shape)}, columns {col}.., other {tuple(other.shape)} {other.dtype}")
    _check(_core(act).ib_blend_columns(_p(x), x.shape[1], int(col), other.shape[1], _p(other), other.stride(0),
                                       _p(weight), x.shape[0], _stream()), "blend_columns")


def gate_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, out: torch.Tensor):
    """out = (y * silu(z)) with each of ``groups`` equal consecutive parts of the row divided by its root mean square,
    times ``weight`` (gated first, normed second).  ``y`` float32 [rows, inner]; ``z`` a [rows, inner] view of a
    wider projection in the activation dtype."""
    act = out.dtype
    _need(y, "y", (torch.float32,), 2)
    _need(weight, "weight", (torch.float32,), 1)
    _need(out, "out", _W, 2)
    n, inner = y.shape
    if not (z.is_cuda and z.dtype == act and z.shape == (n, inner) and z.stride(1) == 1) or out.shape != (n, inner) \
            or weight.shape[0] != inner or groups <= 0 or inner % groups:
        raise KernelError(f"gate_group_norm: y {tuple(y.shape)}, z {tuple(z.shape)} {z.dtype}, {groups} parts")
    _check(_core(act).ib_gate_group_norm(_p(y), _p(z), z.stride(0), _p(weight), int(groups), inner, float(eps), _p(out),
                                         n, _stream()), "gate_group_norm")


GATE_ACT_CLAMPED_SWISH, GATE_ACT_GELU_TANH = 0, 1


def clamped_gate(gate_up: torch.Tensor, out: torch.Tensor, limit: float, slope: float,
                 activation: int = GATE_ACT_CLAMPED_SWISH):
    """out[r, j] = g sigmoid(slope g) (u + 1) with g = min(gate_up[r, j], limit) and
    u = clamp(gate_up[r, inner + j], -limit, limit).  ``activation`` GATE_ACT_GELU_TANH:
    out[r, j] = gelu_tanh(gate_up[r, j]) * gate_up[r, inner + j], gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2 / pi)
    (z + 0.044715 z^3))); ``limit`` and ``slope`` are not read."""
    act = out.dtype
    _need(gate_up, "gate_up", (act,), 2)
    _need(out, "out", _W, 2)
    n, inner = out.shape
    if gate_up.shape != (n, 2 * inner):
        raise KernelError(f"clamped_gate: gate_up {tuple(gate_up.shape)} does not match out {tuple(out.shape)}")
    _check(_core(act).ib_clamped_gate(_p(gate_up), _p(out), n, inner, float(limit), float(slope), int(activation),
                                      _stream()), "clamped_gate")


ROUTE_SOFTMAX_OF_CHOSEN, ROUTE_SIGMOID_SHARE, ROUTE_SOFTMAX_SHARE = 0, 1, 2


def router_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], n_experts: int, top: int, has_shared: bool,
                weights: torch.Tensor, act_dtype: torch.dtype, mode: int = ROUTE_SOFTMAX_OF_CHOSEN, scale: float = 1.0):
    """weights[r, e] = the softmax over the ``top`` largest of logits[r, :n_experts] + bias, among themselves, for
    those experts and 0 for the others; with ``has_shared`` weights[r, n_experts] = sigmoid(logits[r, n_experts]).
    ``mode`` ROUTE_SIGMOID_SHARE: the scores are sigmoid(logits + bias), the ``top`` largest are chosen and each
    chosen expert weighs its score over the sum of the chosen scores (+ 1e-20).  ROUTE_SOFTMAX_SHARE: the same with the
    scores softmax(logits + bias) over all experts.  The routed weights are multiplied by ``scale``."""
    _need(logits, "logits", (torch.float32,), 2)
    _need(bias, "bias", (torch.float32,), 1, optional=True)
    _need(weights, "weights", (torch.float32,), 2)
    n = logits.shape[0]
    cols = n_experts + int(bool(has_shared))
    if logits.shape[1] < cols or weights.shape != (n, cols) or (bias is not None and bias.shape[0] != n_experts) \
            or not 0 < top <= n_experts:
        raise KernelError(f"router_topk: logits {tuple(logits.shape)}, weights {tuple(weights.shape)}, top {top} of "
                          f"{n_experts}")
    if mode not in (ROUTE_SOFTMAX_OF_CHOSEN, ROUTE_SIGMOID_SHARE, ROUTE_SOFTMAX_SHARE):
        raise KernelError(f"router_topk: unknown mode {mode}")
    _check(_core(act_dtype).ib_router_topk(_p(logits), logits.shape[1], _p(bias), int(n_experts), int(top),
                                           int(bool(has_shared)), _p(weights), n, int(mode), float(scale), _stream()),
           "router_topk")


def routed_gate(gate_up: torch.Tensor, weights: torch.Tensor, n_experts: int, ff: int, out: torch.Tensor,
                limit: Optional[float] = None, slope: float = 1.702):
    """out[r, j] = silu(gate_up[r, j]) * gate_up[r, inner + j] * weights[r, e(j)], the experts' columns side by side:
    e(j) = j / ff for the routed ones, n_experts for the columns after them (a shared expert).  With a ``limit`` the
    experts' activation is the clamped form, g sigmoid(slope g) (u + 1) with g = min(gate, limit) and
    u = clamp(up, -limit, limit), in place of silu(gate) * up."""
    act = out.dtype
    _need(gate_up, "gate_up", (act,), 2)
    _need(weights, "weights", (torch.float32,), 2)
    _need(out, "out", _W, 2)
    n, inner = out.shape
    if gate_up.shape != (n, 2 * inner) or weights.shape[0] != n or n_experts * ff > inner \
            or weights.shape[1] < n_experts + int(n_experts * ff < inner):
        raise KernelError(f"routed_gate: gate_up {tuple(gate_up.shape)}, weights {tuple(weights.shape)}, out "
                          f"{tuple(out.shape)}")
    _check(_core(act).ib_routed_gate(_p(gate_up), _p(weights), weights.shape[1], int(n_experts), int(ff), _p(out), n,
                                     inner, int(limit is not None), float(limit or 0.0), float(slope), _stream()),
           "routed_gate")


def decay_scan(x: torch.Tensor, q_col: int, k_col: int, v_col: int, groups: int, keep: torch.Tensor,
               take: Optional[torch.Tensor], skip: Optional[torch.Tensor], state: torch.Tensor, q_start: torch.Tensor,
               slots: torch.Tensor, n_requests: int, out: torch.Tensor, key_dim: int, act_dtype: torch.dtype,
               max_rows: int = 0):
    """A matrix state per head with a scalar decay, carried over each request's rows in float32:
    S = keep S + take k v^T, o = S^T q + skip v.

    ``x`` float32 [rows, ld] holds q and k as [groups, D] and v as [H, E] from the given columns on (head h reads
    group h / (H / groups)); ``keep`` is [H] (one decay per head for all tokens) or a [rows, H] view with unit last
    stride, ``take`` the same or None (1), ``skip`` [H] or None (0); ``out`` float32 [rows, H, E]; ``state`` float32
    [slots, ...] with at least H*D*E numbers per slot, S first.  ``max_rows``: the most rows that a request brings, if
    the caller knows (1: the form for steps of single tokens)."""
    _need(x, "x", (torch.float32,), 2)
    _need(out, "out", (torch.float32,), 3)
    _need(state, "state", (torch.float32,))
    _need(skip, "skip", (torch.float32,), 1, optional=True)
    _need(q_start, "q_start", _I, 1)
    _need(slots, "slots", _I, 1)
    n, heads, e_dim = out.shape
    d_dim = int(key_dim)

    def per_token(t, name):
        if t is None:
            return None, 0
        if not (t.is_cuda and t.dtype == torch.float32):
            raise KernelError(f"decay_scan: {name} must be a float32 CUDA tensor")
        if t.dim() == 1 and t.shape[0] == heads and t.stride(0) == 1:
            return t.data_ptr(), 0
        if t.dim() == 2 and t.shape == (n, heads) and t.stride(1) == 1:
            return t.data_ptr(), t.stride(0)
        raise KernelError(f"decay_scan: {name} must be [H] or a [rows, H] view with unit last stride, got "
                          f"{tuple(t.shape)} with strides {t.stride()}")

    keep_p, keep_ld = per_token(keep, "keep")
    take_p, take_ld = per_token(take, "take")
    if keep_p is None or x.shape[0] != n or groups <= 0 or heads % groups or d_dim <= 0 \
            or max(q_col, k_col) + groups * d_dim > x.shape[1] or v_col + heads * e_dim > x.shape[1] \
            or (skip is not None and skip.shape[0] != heads) \
            or q_start.shape[0] < n_requests + 1 or slots.shape[0] < n_requests or state[0].numel() < heads * d_dim * e_dim:
        raise KernelError(f"decay_scan: x {tuple(x.shape)}, out {tuple(out.shape)}, {groups} groups of {d_dim}")
    if d_dim > 256:
        raise KernelError(f"decay_scan: {d_dim} key channels per head are more than the kernel's 256")
    _check(_core(act_dtype).ib_decay_scan(
        _p(x), x.shape[1], int(q_col), int(k_col), int(v_col), int(groups), keep_p, keep_ld, take_p, take_ld, _p(skip),
        _p(state), state[0].numel(), _p(q_start), _p(slots), int(n_requests), _p(out), heads, d_dim, e_dim,
        int(max_rows), _stream()), "decay_scan")


def delta_scan(x: torch.Tensor, q_col: int, k_col: int, v_col: int, groups: int, fade: torch.Tensor,
               beta: torch.Tensor, unit_eps: Optional[float], q_scale: float, state: torch.Tensor,
               q_start: torch.Tensor, slots: torch.Tensor, n_requests: int, out: torch.Tensor, key_dim: int,
               act_dtype: torch.dtype, max_rows: int = 0):
    """The gated delta rule over each request's rows in float32: S = fade S; u = beta (v - S^T k); S = S + k u^T;
    o = S^T q.

    ``x`` float32 [rows, ld] holds q and k as [groups, D] and v as [H, E] from the given columns on (head h reads
    group h / (H / groups)); ``fade`` and ``beta`` are [rows, H] views with unit last stride; ``unit_eps`` not None:
    q and k are divided by sqrt(sum of squares + unit_eps) per head; q is multiplied by ``q_scale``; ``out`` float32
    [rows, H, E]; ``state`` float32 [slots, ...] with at least H*D*E numbers per slot, S first.  ``max_rows``: the
    most rows that a request brings, if the caller knows (1 or 2: one token after the other; else sixteen tokens at
    once, which differs from that by float32 rounding alone)."""
    _need(x, "x", (torch.float32,), 2)
    _need(out, "out", (torch.float32,), 3)
    _need(state, "state", (torch.float32,))
    _need(q_start, "q_start", _I, 1)
    _need(slots, "slots", _I, 1)
    n, heads, e_dim = out.shape
    d_dim = int(key_dim)
    for name, t in (("fade", fade), ("beta", beta)):
        if not (t.is_cuda and t.dtype == torch.float32 and t.dim() == 2 and t.shape == (n, heads) and t.stride(1) == 1):
            raise KernelError(f"delta_scan: {name} must be a float32 [rows, H] CUDA view with unit last stride")
    if x.shape[0] != n or groups <= 0 or heads % groups or d_dim <= 0 \
            or max(q_col, k_col) + groups * d_dim > x.shape[1] or v_col + heads * e_dim > x.shape[1] \
            or q_start.shape[0] < n_requests + 1 or slots.shape[0] < n_requests \
            or state[0].numel() < heads * d_dim * e_dim:
        raise KernelError(f"delta_scan: x {tuple(x.shape)}, out {tuple(out.shape)}, {groups} groups of {d_dim}")
    if d_dim > 256:
        raise KernelError(f"delta_scan: {d_dim} key channels per head are more than the kernel's 256")
    _check(_core(act_dtype).ib_delta_scan(
        _p(x), x.shape[1], int(q_col), int(k_col), int(v_col), int(groups), fade.data_ptr(), fade.stride(0),
        beta.data_ptr(), beta.stride(0), -1.0 if unit_eps is None else float(unit_eps), float(q_scale), _p(state),
        state[0].numel(), _p(q_start), _p(slots), int(n_requests), _p(out), heads, d_dim, e_dim, int(max_rows),
        _stream()), "delta_scan")


def gated_add_layer_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], gate_pre: Optional[torch.Tensor],
                         gate_bias: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                         rows: Optional[torch.Tensor] = None):
    """residual <- residual + sigmoid(gate_pre + gate_bias) * delta (float32, in place; without ``gate_pre`` the
    delta is added as it is, without ``delta`` nothing), then out = (x - mean) / sqrt(variance + eps) * weight in the
    activation dtype.  With ``rows`` only those rows are read and the stream is left as it is."""
    act = out.dtype
    _need(residual, "residual", (torch.float32,), 2)
    _need(delta, "delta", (act,), 2, optional=True)
    _need(gate_pre, "gate_pre", (act,), 2, optional=True)
    _need(gate_bias, "gate_bias", (torch.float32,), 1, optional=True)
    _need(weight, "weight", (torch.float32,), 1)
    _need(out, "out", _W, 2)
    _need(rows, "rows", _I, 1, optional=True)
    n, width = residual.shape
    n_out = n if rows is None else rows.shape[0]
    if out.shape != (n_out, width) or weight.shape[0] != width or (delta is not None and delta.shape != (n, width)) \
            or (gate_pre is not None and (delta is None or gate_pre.shape != (n, width))) \
            or (gate_bias is not None and gate_bias.shape[0] != width):
        raise KernelError(f"gated_add_layer_norm: residual {tuple(residual.shape)}, out {tuple(out.shape)}, delta "
                          f"{None if delta is None else tuple(delta.shape)}")
    _check(_core(act).ib_gated_add_layer_norm(_p(residual), _p(delta), _p(gate_pre), _p(gate_bias), _p(weight),
                                              float(eps), _p(out), _p(rows), n_out, width, _stream()),
           "gated_add_layer_norm")


def gated_rows(delta: torch.Tensor, gate_pre: torch.Tensor, gate_bias: Optional[torch.Tensor], out: torch.Tensor):
    """out = delta * sigmoid(gate_pre + gate_bias), all [rows, width] in the activation dtype."""
    act = out.dtype
    _need(delta, "delta", (act,), 2)
    _need(gate_pre, "gate_pre", (act,), 2)
    _need(gate_bias, "gate_bias", (torch.float32,), 1, optional=True)
    _need(out, "out", _W, 2)
    if delta.shape != out.shape or gate_pre.shape != out.shape or \
            (gate_bias is not None and gate_bias.shape[0] != out.shape[1]):
        raise KernelError(f"gated_rows: delta {tuple(delta.shape)}, gate {tuple(gate_pre.shape)}, out {tuple(out.shape)}")
    _check(_core(act).ib_gated_rows(_p(delta), _p(gate_pre), _p(gate_bias), _p(out), out.shape[0], out.shape[1],
                                    _stream()), "gated_rows")


def bias_add(x: torch.Tensor, bias: torch.Tensor):
    """x[r, j] += bias[j] in place for the first len(bias) columns of every row; ``x`` in the activation dtype (a view
    with unit last stride), ``bias`` float32."""
    _need(bias, "bias", (torch.float32,), 1)
    if not (x.is_cuda and x.dim() == 2 and x.dtype in _W and x.stride(1) == 1 and bias.shape[0] <= x.shape[1]):
        raise KernelError(f"bias_add: x {tuple(x.shape)} {x.dtype}, bias {tuple(bias.shape)}")
    _check(_core(x.dtype).ib_bias_add(x.data_ptr(), x.stride(0), _p(bias), x.shape[0], bias.shape[0], _stream()),
           "bias_add")


def scaled_sum(x: torch.Tensor, a: float, y: torch.Tensor, b: float, out: torch.Tensor):
    """out = a * x + b * y, element by element in float32, stored in the activation dtype."""
    act = out.dtype
    _need(x, "x", (act,))
    _need(y, "y", (act,))
    _need(out, "out", _W)
    if x.shape != out.shape or y.shape != out.shape:
        raise KernelError(f"scaled_sum: x {tuple(x.shape)}, y {tuple(y.shape)}, out {tuple(out.shape)}")
    _check(_core(act).ib_scaled_sum(_p(x), float(a), _p(y), float(b), _p(out), out.numel(), _stream()), "scaled_sum")


def mix_queries(q: torch.Tensor, mix: torch.Tensor, n_kv_heads: int, out: torch.Tensor):
    """out[r, h, c*D:(c+1)*D] = sum over the heads g of key/value group c of mix[h, g] * q[r, g, :]: queries whose
    scores against all of a token's key heads, side by side, are the heads' own scores mixed by ``mix`` [H, H]."""
    act = out.dtype
    _need(q, "q", (act,), 3)
    _need(mix, "mix", (torch.float32,), 2)
    _need(out, "out", _W, 3)
    n, heads, d = q.shape
    if mix.shape != (heads, heads) or n_kv_heads <= 0 or heads % n_kv_heads or out.shape != (n, heads, n_kv_heads * d):
        raise KernelError(f"mix_queries: q {tuple(q.shape)}, mix {tuple(mix.shape)}, out {tuple(out.shape)}")
    _check(_core(act).ib_mix_queries(_p(q), _p(mix), _p(out), n, heads, int(n_kv_heads), d, _stream()), "mix_queries")


ARGMAX_CHUNK = 8192      # vocabulary entries per block of the two-stage argmax
MMA_KEYS = 64          # keys per tile of the tensor-core attention kernel
MMA_TARGET_CTAS = 1184  # four waves of 2 resident CTAs on 148 SMs: many small CTAs even out the last wave


def mma_attention_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128, 256) and MMA_KEYS % page_size == 0
            and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 16)


def decode_splits(n_requests: int, n_kv_heads: int, max_kv_len: int) -> int:
    """How many ways the decode form cuts each request's keys: enough CTAs to fill the machine several
    times over, but at least four 64-key tiles for each of them."""
    tiles = max(1, (max_kv_len + MMA_KEYS - 1) // MMA_KEYS)
    want = (MMA_TARGET_CTAS + n_requests * n_kv_heads - 1) // (n_requests * n_kv_heads)
    return max(1, min(want, tiles // 4))


def paged_attention_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                        tile_req: torch.Tensor, tile_row0: torch.Tensor, n_tiles: int, q_start: torch.Tensor,
                        positions: torch.Tensor, scale: float, window: Optional[int], out: torch.Tensor,
                        decode_form: bool, n_splits: int = 1, head_scale: Optional[torch.Tensor] = None,
                        slopes: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None):
    """Tensor-core attention over the pages (bfloat16).  Prefill form: tile i holds up to 64/G tokens of request
    tile_req[i] from row tile_row0[i].  Decode form: every tile is one token; its keys are cut ``n_splits`` ways
    and merged through float32 scratch.  ``head_scale`` / ``slopes`` / ``sinks`` (float32 [H]): as in
    :func:`paged_attention_generic`."""
    bf = (torch.bfloat16,)
    for name, t in (("head_scale", head_scale), ("slopes", slopes), ("sinks", sinks)):
        _need(t, name, (torch.float32,), 1, optional=True)
        if t is not None and t.shape[0] != q.shape[1]:
            raise KernelError(f"paged_attention_mma: {name} has {t.shape[0]} numbers for {q.shape[1]} heads")
    _need(q, "q", bf, 3)
    _need(k_pages, "k_pages", bf, 4)
    _need(v_pages, "v_pages", bf, 4)
    _need(out, "out", bf, 2)
    for name, t in (("block_table", block_table),):
        _need(t, name, _I, 2)
    for name, t in (("tile_req", tile_req), ("tile_row0", tile_row0), ("q_start", q_start), ("positions", positions)):
        _need(t, name, _I, 1)
    n, nh, d = q.shape
    n_pages, nkv, page_size, dk = k_pages.shape
    if dk != d or v_pages.shape != k_pages.shape or out.shape != (n, nh * d):
        raise KernelError(f"paged_attention_mma: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    if not mma_attention_supported(q.dtype, nh, nkv, d, page_size):
        raise KernelError(f"paged_attention_mma takes head_dim 64/128/256, a page size that divides {MMA_KEYS} and at "
                          f"most 16 query heads per key/value head; got head_dim {d}, page size {page_size}, "
                          f"{nh}/{nkv} heads")
    if tile_req.shape[0] < n_tiles or tile_row0.shape[0] < n_tiles:
        raise KernelError("paged_attention_mma: tile arrays are shorter than n_tiles")
    part_o = part_ml = None
    if decode_form and n_splits > 1:
        part_o = torch.empty((n, nh, n_splits, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, nh, n_splits, 2), dtype=torch.float32, device=q.device)
    _check(_core(torch.bfloat16).ib_paged_attention_mma(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(tile_req),
        _p(tile_row0), n_tiles, _p(q_start), _p(positions), n, nh, nkv, d, float(scale), int(window) if window else 0,
        _p(out), int(decode_form), int(n_splits), _p(part_o), _p(part_ml), _p(head_scale), _p(slopes), _p(sinks),
        _stream()), "paged_attention_mma")


_DECODE_COUNTERS = {}  # device index -> zeroed int32 counters of the decode attention kernel


def tma_decode_attention_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim == 128 and page_size >= 8 and MMA_KEYS % page_size == 0
            and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 16)


DECODE_RESIDENT_CTAS = 296  # two CTAs of the decode attention kernel fit on each of the 148 SMs


def decode_slices(n_requests: int, n_kv_heads: int, max_kv_len: int):
    """(max_splits, min_tiles) for :func:`paged_attention_decode`: the slices per request that the decode kernel's
    grid provides, and how the kernel picks a request's slices from its real length.

    Few requests: as many slices as still run as one wave of resident CTAs, because a CTA's fixed start-up cost
    is paid once per wave; a request uses as many as leave each slice four tiles.  Between one and one and a half
    waves of (request, head group) pairs the second wave would be nearly empty and as long as the first: three or two
    slices make four or three nearly full waves of shorter CTAs (measured at 2,048 keys: 40 requests 88 us against
    99 with one slice, 48 requests 92 against 99; inside a step of 48 requests of 8,192 keys 347 us per layer against
    400).  More pairs: one slice (at 2,048 keys 64 requests take 102 us with one slice and 115 to 123 with two to
    four; 64 requests of 8,192 keys in four slices, which would fill seven waves, take 438 us per layer inside a step
    against 421 with one)."""
    tiles = max(1, (max_kv_len + MMA_KEYS - 1) // MMA_KEYS)
    pairs = max(1, n_requests * n_kv_heads)
    most = max(1, (tiles + 3) // 4)
    room = DECODE_RESIDENT_CTAS
    if pairs <= room:
        return max(1, min(most, room // pairs)), 4
    if pairs * 3 <= 4 * room:
        return min(most, 3), 4
    if pairs * 2 <= 3 * room:
        return min(most, 2), 4
    return 1, 4


def decode_max_splits(n_requests: int, n_kv_heads: int, max_kv_len: int) -> int:
    return decode_slices(n_requests, n_kv_heads, max_kv_len)[0]


def paged_attention_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                           positions: torch.Tensor, scale: float, window: Optional[int], out: torch.Tensor,
                           max_splits: int, rows: Optional[torch.Tensor] = None, reqs: Optional[torch.Tensor] = None,
                           min_tiles: int = 4):
    """Attention of one new token per request (row r = request r) over its pages: TMA-fed key/value tiles, split
    over the keys, merged by the slice that finishes last (bfloat16, head_dim 128).  With ``rows`` and ``reqs``
    (int32, equally long) only the rows named are worked on, row ``rows[i]`` being a single token of request
    ``reqs[i]``; a negative row is skipped.  The other rows of ``out`` are left alone.  A request is cut into as
    many slices as leave each ``min_tiles`` tiles of 64 keys (at most ``max_splits``)."""
    bf = (torch.bfloat16,)
    _need(q, "q", bf, 3)
    _need(k_pages, "k_pages", bf, 4)
    _need(v_pages, "v_pages", bf, 4)
    _need(out, "out", bf, 2)
    _need(block_table, "block_table", _I, 2)
    _need(positions, "positions", _I, 1)
    n_q, nh, d = q.shape
    n_pages, nkv, page_size, dk = k_pages.shape
    _need(rows, "rows", _I, 1, optional=True)
    _need(reqs, "reqs", _I, 1, optional=True)
    if (rows is None) != (reqs is None) or (rows is not None and rows.shape != reqs.shape):
        raise KernelError("paged_attention_decode: rows and reqs come together and are equally long")
    n = n_q if rows is None else rows.shape[0]
    if dk != d or v_pages.shape != k_pages.shape or out.shape != (n_q, nh * d) or positions.shape[0] != n_q \
            or (rows is None and block_table.shape[0] < n):
        raise KernelError(f"paged_attention_decode: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    if n == 0:
        return
    if not tma_decode_attention_supported(q.dtype, nh, nkv, d, page_size):
        raise KernelError(f"paged_attention_decode takes head_dim 128, a page size of 8..64 that divides 64 and at most "
                          f"16 query heads per key/value head; got head_dim {d}, page size {page_size}, {nh}/{nkv} heads")
    idx = q.device.index if q.device.index is not None else torch.cuda.current_device()
    counters = _DECODE_COUNTERS.get(idx)
    if counters is None or counters.numel() < n * nkv:
        counters = torch.zeros((max(65536, n * nkv),), dtype=torch.int32, device=q.device)
        _DECODE_COUNTERS[idx] = counters
    part_o = part_ml = None
    if max_splits > 1:
        part_o = torch.empty((n, nh, max_splits, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, nh, max_splits, 2), dtype=torch.float32, device=q.device)
    _check(_core(torch.bfloat16).ib_paged_attention_decode(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(positions), n,
        nh, nkv, d, float(scale), int(window) if window else 0, _p(out), int(max_splits), int(min_tiles), _p(part_o),
        _p(part_ml), _p(counters), _p(rows), _p(reqs), _stream()), "paged_attention_decode")


def attention_decode_error(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in the decode attention kernel (synchronises)."""
    return _core(torch.bfloat16).ib_attention_decode_error(int(reset))


TC_ROWS = 128  # query rows per tile of the tcgen05 attention kernel


def tcgen05_attention_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    g = n_heads // max(n_kv_heads, 1)
    return (dtype == torch.bfloat16 and head_dim == 128 and page_size >= 8 and 128 % page_size == 0
            and n_heads % n_kv_heads == 0 and 1 <= g <= TC_ROWS)


def paged_attention_tcgen05(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                            tile_req: torch.Tensor, tile_row0: torch.Tensor, n_tiles: int, q_start: torch.Tensor,
                            positions: torch.Tensor, scale: float, window: Optional[int], out: torch.Tensor,
                            head_scale: Optional[torch.Tensor] = None, slopes: Optional[torch.Tensor] = None,
                            sinks: Optional[torch.Tensor] = None):
    """Attention of prompt portions on tcgen05 tensor cores (bfloat16, head_dim 128): tile i holds up to
    128/G tokens of request tile_req[i] from row tile_row0[i]; Q, K, V by TMA, scores and P V in tensor memory.
    ``head_scale`` / ``slopes`` / ``sinks`` (float32 [H]): as in :func:`paged_attention_generic`; with any of them the
    kernel's form runs that brings the scores to their final form before it takes the row's maximum."""
    bf = (torch.bfloat16,)
    for name, t in (("head_scale", head_scale), ("slopes", slopes), ("sinks", sinks)):
        _need(t, name, (torch.float32,), 1, optional=True)
        if t is not None and t.shape[0] != q.shape[1]:
            raise KernelError(f"paged_attention_tcgen05: {name} has {t.shape[0]} numbers for {q.shape[1]} heads")
    _need(q, "q", bf, 3)
    _need(k_pages, "k_pages", bf, 4)
    _need(v_pages, "v_pages", bf, 4)
    _need(out, "out", bf, 2)
    _need(block_table, "block_table", _I, 2)
    for name, t in (("tile_req", tile_req), ("tile_row0", tile_row0), ("q_start", q_start), ("positions", positions)):
        _need(t, name, _I, 1)
    n, nh, d = q.shape
    n_pages, nkv, page_size, dk = k_pages.shape
    if dk != d or v_pages.shape != k_pages.shape or out.shape != (n, nh * d):
        raise KernelError(f"paged_attention_tcgen05: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    if not tcgen05_attention_supported(q.dtype, nh, nkv, d, page_size):
        raise KernelError(f"paged_attention_tcgen05 takes head_dim 128, a page size of 8..128 that divides 128 and a "
                          f"group size of at most 128; got head_dim {d}, page size {page_size}, {nh}/{nkv} heads")
    if head_scale is not None or slopes is not None or sinks is not None:
        _check(_core(torch.bfloat16).ib_paged_attention_tcgen05_per_head(
            _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(tile_req),
            _p(tile_row0), n_tiles, _p(q_start), _p(positions), n, nh, nkv, d, float(scale),
            int(window) if window else 0, _p(out), _p(head_scale), _p(slopes), _p(sinks), _stream()),
            "paged_attention_tcgen05")
        return
    _check(_core(torch.bfloat16).ib_paged_attention_tcgen05(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(tile_req),
        _p(tile_row0), n_tiles, _p(q_start), _p(positions), n, nh, nkv, d, float(scale), int(window) if window else 0,
        _p(out), _stream()), "paged_attention_tcgen05")


TC_PAIR_ROWS = 256  # query rows per tile of the tcgen05 attention kernel with two query tiles per CTA
PAIR_MIN_CTAS = 128  # that kernel serves steps with at least this many of its CTAs (fewer leave SMs without work)


def pair_tile_tokens(n_heads: int, n_kv_heads: int) -> int:
    """Tokens that a tile of the kernel with two query tiles holds: each query tile takes as many whole tokens (all
    heads of the group) as fit into its 128 rows."""
    return 2 * ((TC_PAIR_ROWS // 2) // (n_heads // n_kv_heads))


def tcgen05_pair_attention_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int,
                                     page_size: int) -> bool:
    g = n_heads // max(n_kv_heads, 1)
    return (dtype == torch.bfloat16 and head_dim == 128 and page_size >= 8 and 128 % page_size == 0
            and n_heads % n_kv_heads == 0 and 1 <= g <= 128)


def paged_attention_pair_tcgen05(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                                 block_table: torch.Tensor, tile_req: torch.Tensor, tile_row0: torch.Tensor, n_tiles: int,
                                 q_start: torch.Tensor, positions: torch.Tensor, scale: float, window: Optional[int],
                                 out: torch.Tensor):
    """Attention of prompt portions on tcgen05 tensor cores with two query tiles per CTA that take turns
    (bfloat16, head_dim 128): tile i holds up to ``pair_tile_tokens`` tokens of request tile_req[i] from row
    tile_row0[i]; the probabilities go to the second product through tensor memory, where the output is
    accumulated too."""
    bf = (torch.bfloat16,)
    _need(q, "q", bf, 3)
    _need(k_pages, "k_pages", bf, 4)
    _need(v_pages, "v_pages", bf, 4)
    _need(out, "out", bf, 2)
    _need(block_table, "block_table", _I, 2)
    for name, t in (("tile_req", tile_req), ("tile_row0", tile_row0), ("q_start", q_start), ("positions", positions)):
        _need(t, name, _I, 1)
    n, nh, d = q.shape
    n_pages, nkv, page_size, dk = k_pages.shape
    if dk != d or v_pages.shape != k_pages.shape or out.shape != (n, nh * d):
        raise KernelError(f"paged_attention_pair_tcgen05: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, "
                          f"out {tuple(out.shape)}")
    if not tcgen05_pair_attention_supported(q.dtype, nh, nkv, d, page_size):
        raise KernelError(f"paged_attention_pair_tcgen05 takes head_dim 128, a page size of 8..128 that divides 128 and "
                          f"a group size of at most 128; got head_dim {d}, page size {page_size}, {nh}/{nkv} heads")
    _check(_core(torch.bfloat16).ib_paged_attention_pair_tcgen05(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(tile_req),
        _p(tile_row0), n_tiles, _p(q_start), _p(positions), n, nh, nkv, d, float(scale), int(window) if window else 0,
        _p(out), _stream()), "paged_attention_pair_tcgen05")


def attention_pair_tcgen05_error(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in the kernel above (synchronises)."""
    return _core(torch.bfloat16).ib_attention_pair_tcgen05_error(int(reset))


def attention_tcgen05_error(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in the tcgen05 attention kernel (synchronises)."""
    return _core(torch.bfloat16).ib_attention_tcgen05_error(int(reset))


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                    ctx, scale: float, window: Optional[int], out: torch.Tensor,
                    head_scale: Optional[torch.Tensor] = None, slopes: Optional[torch.Tensor] = None,
                    sinks: Optional[torch.Tensor] = None):
    """Attention of every row of the step over its request's pages; picks the kernel for the sizes.

    ``ctx`` is the step's :class:`~inferrs_b200.engine.batch.StepContext` (row_request, positions
    and what the faster kernels need to cut the work).  ``head_scale`` / ``slopes`` / ``sinks`` (float32 [H], see
    :func:`paged_attention_generic`): scores with any of them go to the tcgen05 kernel's per-head form (prompt
    portions, head size 128), to the ``mma.sync`` kernel (steps of single tokens; head sizes 64 and 256) where these
    take the sizes, and to the float32 kernel otherwise.
    """
    n, nh, d = q.shape
    nkv, page_size = k_pages.shape[1], k_pages.shape[2]
    per_head = dict(head_scale=head_scale, slopes=slopes, sinks=sinks)
    if v_pages.shape[3] != d or not mma_attention_supported(q.dtype, nh, nkv, d, page_size):
        paged_attention_generic(q, k_pages, v_pages, block_table, ctx.row_request, ctx.positions, scale, window, out,
                                **per_head)
        return
    if any(t is not None for t in per_head.values()):
        if ctx.decode_only:
            splits = decode_splits(ctx.n_requests, nkv, min(ctx.max_kv_len, window) if window and window > 0
                                   else ctx.max_kv_len)
            paged_attention_mma(q, k_pages, v_pages, block_table, ctx.row_request, ctx.q_start, ctx.n_requests,
                                ctx.q_start, ctx.positions, scale, window, out, True, splits, **per_head)
        elif tcgen05_attention_supported(q.dtype, nh, nkv, d, page_size) and scale > 0:
            # prompt portions (and what single tokens stand beside them) on the tcgen05 kernel's per-head form
            tile_req, tile_row0, n_tiles = ctx.attention_tiles(TC_ROWS // (nh // nkv))
            paged_attention_tcgen05(q, k_pages, v_pages, block_table, tile_req, tile_row0, n_tiles, ctx.q_start,
                                    ctx.positions, scale, window, out, **per_head)
        else:
            tile_req, tile_row0, n_tiles = ctx.attention_tiles(MMA_KEYS // (nh // nkv))
            paged_attention_mma(q, k_pages, v_pages, block_table, tile_req, tile_row0, n_tiles, ctx.q_start,
                                ctx.positions, scale, window, out, False, **per_head)
        return
    # Prompt portions: tiles of 256 rows (two query tiles per CTA) where they still give every SM a CTA, else
    # tiles of 128 rows.  A step that stands for a padded one (before its graph is captured) says so.
    pair_tokens = pair_tile_tokens(nh, nkv)
    rows_for_dispatch = ctx.extra.get("dispatch_rows", ctx.n_rows)
    pair = tcgen05_pair_attention_supported(q.dtype, nh, nkv, d, page_size) \
        and (rows_for_dispatch // pair_tokens) * nkv >= PAIR_MIN_CTAS
    prefill_kernel = paged_attention_pair_tcgen05 if pair else paged_attention_tcgen05
    prefill_tokens = pair_tokens if pair else TC_ROWS // (nh // nkv)
    if ctx.decode_only and tma_decode_attention_supported(q.dtype, nh, nkv, d, page_size):
        max_splits, min_tiles = decode_slices(ctx.n_requests, nkv, ctx.max_kv_len)
        paged_attention_decode(q, k_pages, v_pages, block_table, ctx.positions, scale, window, out, max_splits,
                               min_tiles=min_tiles)
    elif ctx.decode_only:
        # one row per request: the rows are the tiles
        splits = decode_splits(ctx.n_requests, nkv, ctx.max_kv_len)
        paged_attention_mma(q, k_pages, v_pages, block_table, ctx.row_request, ctx.q_start, ctx.n_requests,
                            ctx.q_start, ctx.positions, scale, window, out, True, splits)
    elif tcgen05_attention_supported(q.dtype, nh, nkv, d, page_size) \
            and tma_decode_attention_supported(q.dtype, nh, nkv, d, page_size):
        # portions of prompts and single tokens side by side: the single tokens go to the decode kernel (a tile
        # of the prefill kernel would hold one token of 32), the portions to the prefill kernel
        rows, reqs, n_single = ctx.single_rows()
        if n_single > 0:
            max_splits, min_tiles = decode_slices(n_single, nkv, ctx.max_kv_len)
            paged_attention_decode(q, k_pages, v_pages, block_table, ctx.positions, scale, window, out, max_splits,
                                   rows, reqs, min_tiles=min_tiles)
        tile_req, tile_row0, n_tiles = ctx.attention_tiles(prefill_tokens, portions_only=True)
        if n_tiles > 0:
            prefill_kernel(q, k_pages, v_pages, block_table, tile_req, tile_row0, n_tiles, ctx.q_start,
                           ctx.positions, scale, window, out)
    elif tcgen05_attention_supported(q.dtype, nh, nkv, d, page_size):
        tile_req, tile_row0, n_tiles = ctx.attention_tiles(prefill_tokens)
        prefill_kernel(q, k_pages, v_pages, block_table, tile_req, tile_row0, n_tiles, ctx.q_start,
                       ctx.positions, scale, window, out)
    else:
        tile_req, tile_row0, n_tiles = ctx.attention_tiles(MMA_KEYS // (nh // nkv))
        paged_attention_mma(q, k_pages, v_pages, block_table, tile_req, tile_row0, n_tiles, ctx.q_start,
                            ctx.positions, scale, window, out, False)


def joint_mma_attention_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, value_dim: int,
                                  page_size: int, decode_form: bool = False) -> bool:
    """Whether the tensor-core kernel for joint queries takes these sizes: bfloat16, keys and values of 64 or 128
    numbers, a page size that divides 64, at most 16 query heads per key/value head, and the queries and two key
    tiles of all key/value heads within shared memory."""
    if dtype != torch.bfloat16 or head_dim != value_dim or n_kv_heads <= 0 or n_heads % n_kv_heads:
        return False
    return _core(torch.bfloat16).ib_joint_attention_mma_smem(n_heads, n_kv_heads, head_dim, page_size,
                                                             int(decode_form)) > 0


def joint_mma_prefill_tokens(n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> int:
    """The tokens of one request that a tile of the tensor-core kernel's prefill form holds for these sizes: its rows
    divided by the heads per key/value head; 0 for sizes that the kernel does not take."""
    rows = _core(torch.bfloat16).ib_joint_attention_mma_rows(n_heads, n_kv_heads, head_dim, page_size)
    return rows // (n_heads // n_kv_heads) if rows > 0 else 0


def joint_attention_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                        tile_req: torch.Tensor, tile_row0: torch.Tensor, n_tiles: int, q_start: torch.Tensor,
                        positions: torch.Tensor, scale: float, window: Optional[int],
                        dist_bias: Optional[torch.Tensor], out: torch.Tensor, decode_form: bool, n_splits: int = 1):
    """Tensor-core attention with joint queries ``q`` [rows, H, kv_heads * D] (see :func:`mix_queries`) and the table
    ``dist_bias`` [H, L] that is taken off the scores by distance (bfloat16).  Prefill form: tile i holds up to
    :func:`joint_mma_prefill_tokens` tokens of request tile_req[i] from row tile_row0[i].  Decode form: every tile is one token; its
    keys are cut ``n_splits`` ways and merged through float32 scratch."""
    bf = (torch.bfloat16,)
    _need(q, "q", bf, 3)
    _need(k_pages, "k_pages", bf, 4)
    _need(v_pages, "v_pages", bf, 4)
    _need(out, "out", bf, 2)
    _need(block_table, "block_table", _I, 2)
    _need(dist_bias, "dist_bias", (torch.float32,), 2, optional=True)
    for name, t in (("tile_req", tile_req), ("tile_row0", tile_row0), ("q_start", q_start), ("positions", positions)):
        _need(t, name, _I, 1)
    n, nh, dq = q.shape
    n_pages, nkv, page_size, d = k_pages.shape
    if dq != nkv * d or v_pages.shape != k_pages.shape or out.shape != (n, nh * d) \
            or (dist_bias is not None and (dist_bias.shape[0] != nh or dist_bias.shape[1] < 1)):
        raise KernelError(f"joint_attention_mma: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    if not joint_mma_attention_supported(q.dtype, nh, nkv, d, v_pages.shape[3], page_size, decode_form):
        raise KernelError(f"joint_attention_mma does not take head_dim {d}, page size {page_size}, {nh}/{nkv} heads")
    if tile_req.shape[0] < n_tiles or tile_row0.shape[0] < n_tiles:
        raise KernelError("joint_attention_mma: tile arrays are shorter than n_tiles")
    part_o = part_ml = None
    if decode_form and n_splits > 1:
        part_o = torch.empty((n, nh, n_splits, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, nh, n_splits, 2), dtype=torch.float32, device=q.device)
    _check(_core(torch.bfloat16).ib_joint_attention_mma(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(tile_req),
        _p(tile_row0), n_tiles, _p(q_start), _p(positions), n, nh, nkv, d, float(scale), int(window) if window else 0,
        _p(dist_bias), 0 if dist_bias is None else dist_bias.shape[1], _p(out), int(decode_form), int(n_splits),
        _p(part_o), _p(part_ml), _stream()), "joint_attention_mma")


def joint_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                    ctx, scale: float, window: Optional[int], dist_bias: Optional[torch.Tensor], out: torch.Tensor):
    """Attention of every row of the step with joint queries (see :func:`mix_queries`): head h's score against a token
    is its product with all of the token's key heads side by side, times ``scale``, minus dist_bias[h, distance];
    values are those of the head's own group.  Picks the kernel for the sizes: the tensor-core kernel where it takes
    them (its decode form for steps of single tokens), else the float32 kernel for any size."""
    n, nh, dq = q.shape
    nkv, page_size, d, dv = k_pages.shape[1], k_pages.shape[2], k_pages.shape[3], v_pages.shape[3]
    if joint_mma_attention_supported(q.dtype, nh, nkv, d, dv, page_size, ctx.decode_only):
        if ctx.decode_only:
            splits = decode_splits(ctx.n_requests, nkv, min(ctx.max_kv_len, window) if window and window > 0
                                   else ctx.max_kv_len)
            joint_attention_mma(q, k_pages, v_pages, block_table, ctx.row_request, ctx.q_start, ctx.n_requests,
                                ctx.q_start, ctx.positions, scale, window, dist_bias, out, True, splits)
        else:
            tile_req, tile_row0, n_tiles = ctx.attention_tiles(joint_mma_prefill_tokens(nh, nkv, d, page_size))
            joint_attention_mma(q, k_pages, v_pages, block_table, tile_req, tile_row0, n_tiles, ctx.q_start,
                                ctx.positions, scale, window, dist_bias, out, False)
        return
    paged_attention_generic(q, k_pages, v_pages, block_table, ctx.row_request, ctx.positions, scale, window, out,
                            joint=True, dist_bias=dist_bias)


def penalties(logits: torch.Tensor, prev: torch.Tensor, n_prev: torch.Tensor, repetition: torch.Tensor,
              frequency: torch.Tensor, presence: torch.Tensor, act_dtype: torch.dtype = torch.float32):
    """In place on float32 logits [R, V]: repetition, frequency and presence penalties for the tokens in
    each row's window ``prev[r, :n_prev[r]]`` (int32)."""
    _need(logits, "logits", (torch.float32,), 2)
    _need(prev, "prev", _I, 2)
    _need(n_prev, "n_prev", _I, 1)
    r = logits.shape[0]
    for name, t in (("repetition", repetition), ("frequency", frequency), ("presence", presence)):
        _need(t, name, (torch.float32,), 1)
        if t.shape[0] != r:
            raise KernelError(f"penalties: {name} has {t.shape[0]} entries for {r} rows")
    if prev.shape[0] != r or n_prev.shape[0] != r:
        raise KernelError(f"penalties: prev {tuple(prev.shape)}, n_prev {tuple(n_prev.shape)} for {r} rows")
    _check(_core(act_dtype).ib_penalties(_p(logits), logits.shape[1], r, logits.shape[1], _p(prev), prev.shape[1],
                                         _p(n_prev), _p(repetition), _p(frequency), _p(presence), _stream()),
           "penalties")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype = torch.float32,
           cluster: int = 0):
    """One token per row of float32 logits [R, V]: largest logit where temperature < 1e-5, else
    temperature, top-k, top-p, min-p and the inverse-CDF walk with the row's random number ``uniform``.
    ``cluster``: CTAs that share a row (1, 2, 4 or 8; 0 lets the kernel library choose by the number of rows)."""
    _need(logits, "logits", (torch.float32,), 2)
    r = logits.shape[0]
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
                        ("uniform", uniform, torch.float32), ("out", out, torch.int32)):
        _need(t, name, (dt,), 1)
        if t.shape[0] != r:
            raise KernelError(f"sample: {name} has {t.shape[0]} entries for {r} rows")
    scratch = torch.empty((r, logits.shape[1]), dtype=torch.float32, device=logits.device)
    _check(_core(act_dtype).ib_sample(_p(logits), logits.shape[1], r, logits.shape[1], _p(temperature), _p(top_k),
                                      _p(top_p), _p(min_p), _p(uniform), _p(scratch), int(cluster), _p(out), _stream()),
           "sample")


_GEMM_LIB = None


def _gemm_lib():
    global _GEMM_LIB
    if _GEMM_LIB is None:
        lib = load_library("gemm_bf16")
        lib.ib_gemm_tn_tcgen05.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                           c_int, c_int, c_void_p]
        lib.ib_gemm_tn_tcgen05.restype = c_int
        lib.ib_gemm_swiglu_tcgen05.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                               c_void_p]
        lib.ib_gemm_swiglu_tcgen05.restype = c_int
        lib.ib_gemm_tn_tcgen05_folded.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                                  c_int, c_void_p, c_int, c_float, c_int, c_void_p, c_long, c_void_p,
                                                  c_int, c_void_p, c_void_p]
        lib.ib_gemm_tn_tcgen05_folded.restype = c_int
        lib.ib_gemm_swiglu_tcgen05_folded.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
                                                      c_int, c_void_p, c_int, c_float, c_int, c_void_p]
        lib.ib_gemm_swiglu_tcgen05_folded.restype = c_int
        lib.ib_gemm_tcgen05_ssq_parts.argtypes = [c_int, c_int, c_int, c_int]
        lib.ib_gemm_tcgen05_ssq_parts.restype = c_int
        lib.ib_gemm_chain.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
        lib.ib_gemm_chain.restype = c_int
        lib.ib_gemm_chain_workspace_floats.argtypes = [c_int]
        lib.ib_gemm_chain_workspace_floats.restype = c_long
        lib.ib_gemm_chain_workspace_fill.argtypes = []
        lib.ib_gemm_chain_workspace_fill.restype = c_int
        lib.ib_gemm_chain_max_products.argtypes = []
        lib.ib_gemm_chain_max_products.restype = c_int
        lib.ib_gemm_chain_ssq_parts.argtypes = [c_int]
        lib.ib_gemm_chain_ssq_parts.restype = c_int
        lib.ib_gemm_chain_set_pdl.argtypes = [c_int]
        lib.ib_gemm_chain_set_pdl.restype = None
        lib.ib_gemm_chain_error.argtypes = [c_int]
        lib.ib_gemm_chain_error.restype = c_int
        lib.ib_gemm_chain_error_async.argtypes = [c_void_p, c_void_p]
        lib.ib_gemm_chain_error_async.restype = c_int
        lib.ib_gemm_tcgen05_error.argtypes = [c_int]
        lib.ib_gemm_tcgen05_error.restype = c_int
        lib.ib_gemm_tcgen05_error_async.argtypes = [c_void_p, c_void_p]
        lib.ib_gemm_tcgen05_error_async.restype = c_int
        _GEMM_LIB = lib
    return _GEMM_LIB


def tcgen05_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """TMA needs 16-byte aligned bases and row strides: K a multiple of 8 for bfloat16."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _scaled_args(x):
    if isinstance(x, ScaledRows):
        _need(x.ssq, "ssq", (torch.float32,), 2)
        if x.ssq.shape[1] != SSQ_LD or x.ssq.shape[0] < x.n_parts or x.n_parts <= 0:
            raise KernelError(f"scaled rows: {x.n_parts} parts do not fit a list of shape {tuple(x.ssq.shape)}")
        return x.x, (_p(x.ssq), int(x.n_parts), float(x.eps), int(x.width))
    return x, (None, 0, 0.0, 0)


def gemm_tn_tcgen05(x, w: torch.Tensor, out: torch.Tensor, split_k: int = 0, sink: Optional[ResidualSink] = None):
    """out = x @ w.T with TMA-fed tcgen05 MMAs: W is the 128-row operand, the tokens are the N dimension.
    ``split_k`` 0 lets the kernel library choose how many CTAs of a cluster share one output tile.  ``x`` may be
    :class:`ScaledRows` and the result may go to a :class:`ResidualSink` (both: up to 32 rows, bfloat16 out); with a
    sink the :class:`ScaledRows` that stand for the next norm's output are returned."""
    xt, scaled = _scaled_args(x)
    _need(xt, "x", (torch.bfloat16,), 2)
    _need(w, "w", (torch.bfloat16,), 2)
    _need(out, "out", _W, 2)
    n, k = xt.shape
    m = w.shape[0]
    if w.shape[1] != k or out.shape != (n, m):
        raise KernelError(f"gemm: x {tuple(xt.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    lib = _gemm_lib()
    if scaled[0] is None and sink is None:
        code = lib.ib_gemm_tn_tcgen05(_p(xt), k, _p(w), k, _p(out), m, int(out.dtype == torch.float32), n, m, k, split_k,
                                      _stream())
        if code == -1:
            raise KernelError(f"gemm_tn_tcgen05: K={k} must be a multiple of 8 and the bases 16-byte aligned")
        _check(code, "gemm_tn_tcgen05")
        return None
    if out.dtype != torch.bfloat16:
        raise KernelError("gemm_tn_tcgen05: the folded forms store bfloat16")
    result, sink_args = None, (None, 0, None, 0, None)
    if sink is not None:
        _need(sink.residual, "residual", (torch.float32,), 2)
        _need(sink.weight, "sink weight", _W, 1)
        if sink.residual.shape != (n, m) or sink.weight.shape[0] != m:
            raise KernelError(f"gemm: residual {tuple(sink.residual.shape)} and norm weight {tuple(sink.weight.shape)} "
                              f"do not match the result {(n, m)}")
        parts = lib.ib_gemm_tcgen05_ssq_parts(n, m, k, split_k)
        if parts <= 0:
            raise KernelError(f"gemm_tn_tcgen05: {n} rows take no sink")
        ssq = torch.empty((parts, SSQ_LD), dtype=torch.float32, device=out.device)
        sink_args = (_p(sink.residual), m, _p(sink.weight), int(sink.weight.dtype == torch.float32), _p(ssq))
        result = ScaledRows(out, ssq, parts, float(sink.eps), m)
    code = lib.ib_gemm_tn_tcgen05_folded(_p(xt), k, _p(w), k, _p(out), m, n, m, k, split_k, *scaled, *sink_args, _stream())
    if code == -1:
        raise KernelError(f"gemm_tn_tcgen05: the folded forms take up to {SSQ_LD} rows, K={k} a multiple of 8 and "
                          f"16-byte aligned bases")
    _check(code, "gemm_tn_tcgen05 (folded)")
    return result


def gemm_swiglu_tcgen05(x, w_gate_up: torch.Tensor, out: torch.Tensor):
    """out[t, f] = silu(x[t] . w[f]) * (x[t] . w[inner + f]): both products of a gated feed-forward and the gate
    in one tcgen05 kernel (up to 64 gate rows and the same up rows per tile).  Up to 32 rows of x, which may be
    :class:`ScaledRows`."""
    xt, scaled = _scaled_args(x)
    _need(xt, "x", (torch.bfloat16,), 2)
    _need(w_gate_up, "w_gate_up", (torch.bfloat16,), 2)
    _need(out, "out", (torch.bfloat16,), 2)
    n, k = xt.shape
    inner = out.shape[1]
    if w_gate_up.shape != (2 * inner, k) or out.shape[0] != n:
        raise KernelError(f"gemm_swiglu: x {tuple(xt.shape)}, w {tuple(w_gate_up.shape)}, out {tuple(out.shape)}")
    code = _gemm_lib().ib_gemm_swiglu_tcgen05_folded(_p(xt), k, _p(w_gate_up), k, _p(out), inner, n, inner, k, *scaled,
                                                     _stream())
    if code == -1:
        raise KernelError(f"gemm_swiglu_tcgen05: at most 32 rows (got {n}), K={k} a multiple of 8, 16-byte aligned bases")
    _check(code, "gemm_swiglu_tcgen05")


def gemm_tcgen05_set_pdl(on: bool):
    """Let tcgen05 products start before their predecessor in the stream has finished (they prefetch weights and
    wait for the predecessor before touching anything else).  Only safe among kernels that all wait likewise."""
    _gemm_lib().ib_gemm_tcgen05_set_pdl(int(bool(on)))
    _gemm_lib().ib_gemm_chain_set_pdl(int(bool(on)))


def gemm_tcgen05_set_even_tiles(on: bool):
    """Whether a tcgen05 product whose CTAs all run at once cuts its tiles lower than the MMA so that every SM gets
    the same number of them (default) or keeps every tile at the MMA's height."""
    lib = _gemm_lib()
    lib.ib_gemm_tcgen05_set_even_tiles.argtypes = [c_int]
    lib.ib_gemm_tcgen05_set_even_tiles.restype = None
    lib.ib_gemm_tcgen05_set_even_tiles(int(bool(on)))


def gemm_tcgen05_tile_rows(n_rows: int, n_out: int, k: int, split_k: int = 0, gated: bool = False) -> int:
    """Rows of the weight matrix per tile (of each of the two matrices in the gated form) that a tcgen05 product of
    these sizes takes: the MMA's 128 (64), or fewer where that spreads the product evenly over the SMs."""
    lib = _gemm_lib()
    lib.ib_gemm_tcgen05_tile_rows.argtypes = [c_int, c_int, c_int, c_int, c_int]
    lib.ib_gemm_tcgen05_tile_rows.restype = c_int
    return int(lib.ib_gemm_tcgen05_tile_rows(n_rows, n_out, k, split_k, int(gated)))


def set_pdl(on: bool, act_dtype: torch.dtype = torch.bfloat16):
    """Programmatic dependent launch for every kernel of the package launched from now on: a kernel may start
    while the one before it in the stream still runs, does what needs no input (barrier set-up, fetching
    weights) and waits for the earlier kernel before it reads or writes anything else.  Used while a decode
    step is captured into a CUDA graph; library kernels in between simply keep plain stream order."""
    lib = _core(act_dtype)
    lib.ib_set_pdl.argtypes = [c_int]
    lib.ib_set_pdl.restype = None
    lib.ib_set_pdl(int(bool(on)))
    if act_dtype == torch.bfloat16:
        gemm_tcgen05_set_pdl(on)


# up to this many rows the own tcgen05 product is the faster one in a decode step (the environment variable is
# there for measuring other thresholds)
TCGEN05_MAX_TOKENS = int(os.environ.get("INFERRS_B200_TCGEN05_MAX_TOKENS", "16"))
SWIGLU_MAX_TOKENS = 32  # rows that the fused gate/up kernel takes


def gemm_tcgen05_error(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in a tcgen05 GEMM (synchronises with the device)."""
    return _gemm_lib().ib_gemm_tcgen05_error(int(reset))


def gemm_chain_error(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in a chain of products (synchronises)."""
    code = _gemm_lib().ib_gemm_chain_error(int(reset))
    if code != 0 and reset:
        _CHAIN_WS.clear()    # a chain that gave up may have left marks in its workspace: the next chain gets a fresh one
    return code


# ---- the kernels' error words, all of them ------------------------------------------------------------------
# A bounded wait that ran out, or a row whose position lay outside the rotation tables, leaves a code in a word
# on the device.  The functions above read one word each and wait for the device; these read all of them the way
# a serving loop wants it: asked for in stream order, read later from pinned memory.
ERROR_WORDS = ("a row's position outside the rotation tables", "prefill attention (tcgen05)",
               "prefill attention (two query tiles)", "decode attention", "matrix product (tcgen05)",
               "chain of matrix products")


def error_words_async(host: torch.Tensor, act_dtype: torch.dtype):
    """Ask for every error word of the kernel libraries, in the order of ``ERROR_WORDS``, to be copied into ``host``
    (pinned int32, at least ``len(ERROR_WORDS)`` long) behind the work that the current stream holds.  The caller
    records an event after this call and reads ``host`` once the event has come."""
    if host.dtype != torch.int32 or host.numel() < len(ERROR_WORDS) or not host.is_pinned():
        raise KernelError("error_words_async wants a pinned int32 tensor with room for every word")
    core, stream, at = _core(act_dtype), _stream(), host.data_ptr()
    calls = [core.ib_row_fault_async, core.ib_attention_tcgen05_error_async,
             core.ib_attention_pair_tcgen05_error_async, core.ib_attention_decode_error_async]
    if act_dtype == torch.bfloat16:
        calls += [_gemm_lib().ib_gemm_tcgen05_error_async, _gemm_lib().ib_gemm_chain_error_async]
    else:
        host[len(calls):len(ERROR_WORDS)] = 0
    for i, fn in enumerate(calls):
        code = fn(at + 4 * i, stream)
        if code != 0:
            raise KernelError(f"error_words_async: CUDA error {code}")


def reset_error_words(act_dtype: torch.dtype) -> dict:
    """Read every error word now (waits for the device), clear them, and put the decode attention's counters back
    to zero (a wait that ran out may have left a slice uncounted).  Returns {name: code} of the words that were set."""
    found = {}
    row = row_fault(act_dtype, reset=True)
    if row is not None:
        found[ERROR_WORDS[0]] = row + 1
    if act_dtype == torch.bfloat16:
        for name, fn in zip(ERROR_WORDS[1:], (attention_tcgen05_error, attention_pair_tcgen05_error,
                                              attention_decode_error, gemm_tcgen05_error, gemm_chain_error)):
            v = fn(True)
            if v:
                found[name] = v
    for counters in _DECODE_COUNTERS.values():
        counters.zero_()
    return found
