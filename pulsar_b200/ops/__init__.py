"""Typed Python wrappers over the C interface of the CUDA library.

Each wrapper checks what the kernel cannot check itself (device, dtype, shape,
contiguity), passes raw pointers and the current CUDA stream, and raises on any
non-zero status.  There is no CPU path: a tensor that is not on a CUDA device is an
error, and a missing library is an error at first use.

The reference exposes its kernels as ``torch.ops.pulsar.*`` through TorchBind
(pulsar/ext/ops.cpp:8-74; pulsar/src/pulsar/core/ops.py:198-494).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from .. import profiling
from ..csrc.build import library

F32, BF16 = 0, 1
# Which product serves bfloat16 projections of more than 16 rows:
#   "auto"     with more than 128 rows the gate/up product with its SwiGLU gating fused runs on this
#              library's tcgen05 / TMA kernel (faster than the library product plus a gating kernel);
#              the plain projections, and gate/up of 17 to 128 rows, take the library product
#              (cuBLAS through torch.mm, as the reference does);
#   "tcgen05"  every projection on the tcgen05 kernel;
#   "library"  every projection on the library product, gating in a kernel of its own.
# Up to 16 rows always take the weight-streaming kernel.
GEMM_BACKEND = os.environ.get("PULSAR_GEMM", "auto")
# Attention of prompt portions in bfloat16: "auto" = the tcgen05 kernel where it applies, "mma" = never.
ATTENTION_BACKEND = os.environ.get("PULSAR_ATTENTION", "auto")
# The library product (torch.mm) must add its partial sums in float32: by default PyTorch lets cuBLAS reduce
# split-K partial sums of bfloat16 products in bfloat16.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {-2: "unsupported dtype", -3: "unsupported size or argument", -4: "size exceeds the kernel's limit"}

_P, _I, _F, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_long
_SIGNATURES = {
    "pb_embed": [_I, _P, _P, _P, _I, _I, _I, _F, _P],
    "pb_scale_cap": [_P, ctypes.c_longlong, _F, _F, _P],
    "pb_move_ids": [_P, _P, _P, _P, _I, _P],
    "pb_table_update": [_P, _I, _P, _P, _I, _I, _P, _P],
    "pb_add_rmsnorm": [_I, _P, _P, _P, _P, _P, _I, _I, _F, _I, _P],
    "pb_rope_table": [_P, _P, _P, _P, _I, _I, _F, _P],
    "pb_qk_norm_rope_write": [_I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _I, _I, _I, _P],
    "pb_silu_mul": [_I, _P, _P, _I, _I, _P],
    "pb_paged_attention_generic": [_I, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
    "pb_paged_attention_decode": [_I, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "pb_paged_attention_decode_tc": [_I, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "pb_decode_tc_supported": [_I, _I, _I, _I, _I],
    "pb_paged_attention_decode_tc_qkv": [_I, _P, _P, _P, _P, _P, _F, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "pb_paged_attention_decode_tc_fused": [_I, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "pb_paged_attention_prefill_tc": [_I, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    "pb_prefill_tc_supported": [_I, _I, _I, _I, _I],
    "pb_prefill_tc_tile": [],
    "pb_paged_attention_prefill_tcgen05": [_I, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    "pb_prefill_tcgen05_supported": [_I, _I, _I, _I, _I],
    "pb_prefill_tcgen05_tile": [],
    "pb_prefill_tcgen05_error": [],
    "pb_gemm_skinny": [_I, _I, _P, _P, _P, _I, _I, _I, _P],
    "pb_gemm_skinny_supported": [_I, _I, _I, _I],
    "pb_gemm_skinny_fused_supported": [_I, _I, _I, _I],
    "pb_gemm_skinny_publish_sums": [_I],
    "pb_gemm_skinny_accumulate": [_P, _P, _P, _I, _I, _I, _P, _P, _P, _P],
    "pb_gemm_skinny_scaled": [_I, _P, _P, _P, _I, _I, _I, _P, _F, _P],
    "pb_gemm_tcgen05": [_I, _I, _P, _P, _P, _I, _I, _I, _P],
    "pb_gemm_tcgen05_supported": [_I, _I, _I, _I],
    "pb_gemm_tcgen05_error": [],
    "pb_gemm_tcgen05_stream": [_I, _I, _P, _P, _P, _I, _I, _I, _P, ctypes.c_longlong, _P, _I, _P],
    "pb_gemm_tcgen05_stream_workspace": [_I, _I, _I, _I, _P, _P],
    "pb_gemm_tcgen05_stream_supported": [_I, _I, _I, _I],
    "pb_gemm_tcgen05_stream_wait_control": [ctypes.c_longlong, _I, _P],
    "pb_gemm_tcgen05_wait_control": [ctypes.c_longlong, _I, _P],
    "pb_gemm_tcgen05_wait_selftest": [_P],
    "pb_prefill_tcgen05_wait_control": [ctypes.c_longlong, _I, _P],
    "pb_gather_words": [_P, _I, _P, _P],
    "pb_bounds_checked": [],
    "pb_set_pool_bounds": [_I, _P],
    "pb_set_gating": [_F, _F, _F],
    "pb_gemm_simt": [_I, _I, _I, _P, _P, _P, _I, _I, _I, _P],
    "pb_sample": [_P, _I, _I, _P, _P, _P, _P, _I, _P, _P, _P, _P],
    "pb_sample_workspace": [_I],
    "pb_argmax": [_P, _I, _I, _P, _P, _P],
    "pb_paged_attention_general": [_I, _P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _F, _P, _I, _I, _P],
    "pb_attention_general_tiled_supported": [_I, _P, _P, _I, _I, _I, _I, _I, _I],
    "pb_paged_attention_general_tiled": [_I, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _F, _P, _I, _I, _P],
    "pb_attention_general_tc_tile": [],
    "pb_attention_general_tc_supported": [_I, _P, _P, _P, _I, _I, _I, _I, _I, _I],
    "pb_paged_attention_general_tc": [_I, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _F, _P, _I, _I, _P],
    "pb_qkv_split_write": [_I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _F, _I, _P],
    "pb_heads_linear": [_I, _I, _P, _L, _I, _P, _P, _L, _I, _P, _L, _I, _I, _I, _I, _P],
    "pb_latent_prepare": [_I, _P, _L, _P, _L, _P, _F, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "pb_latent_expand_keys": [_I, _P, _P, _P, _I, _I, _I, _I, _P],
    "pb_sigmoid_gate": [_I, _P, _P, _L, _I, _I, _P],
    "pb_causal_conv_silu": [_I, _P, _L, _P, _P, _P, _L, _L, _P, _P, _P, _P, _I, _I, _I, _P],
    "pb_selective_scan": [_I, _P, _P, _L, _P, _L, _P, _P, _P, _P, _P, _L, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "pb_selective_scan_prompt_supported": [_I],
    "pb_selective_scan_chunked_supported": [_I],
    "pb_selective_scan_chunked": [_I, _P, _P, _L, _P, _L, _P, _P, _P, _P, _P, _L, _L, _P, _P, _P, _I, _I, _I, _I, _P],
    "pb_selective_scan_prompt": [_I, _P, _P, _L, _P, _L, _P, _P, _P, _P, _P, _L, _L, _P, _P, _P, _I, _I, _I, _I, _P],
    "pb_post_norm_add": [_I, _P, _P, _P, _F, _P, _F, _P, _I, _I, _P],
    "pb_clamped_glu": [_I, _P, _P, _I, _I, _F, _F, _P],
    "pb_post_norm_add_bias": [_I, _P, _P, _P, _P, _F, _P, _I, _I, _P],
    "pb_glu_bias": [_I, _I, _P, _P, _P, _I, _I, _F, _F, _F, _P],
    "pb_qk_prepare": [_I, _I, _P, _L, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P, _F, _I, _I, _P],
    "pb_sigmoid_gate_strided": [_I, _I, _P, _P, _L, _I, _I, _I, _P],
    "pb_add_bias": [_I, _P, _P, _I, _I, _P],
    "pb_moe_route": [_I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, _I, _F, _P],
    "pb_moe_gate_up": [_I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _F, _F, _P, _P],
    "pb_moe_down": [_I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "pb_moe_grouped_workspace": [_I, _I, _I],
    "pb_moe_grouped_supported": [_I, _I, _I],
    "pb_moe_grouped": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _F, _F, _I, _P, _P],
    "pb_norm_shift": [_I, _P, _P, _F, _P, _P, _L, _P, _P, _P, _P, _P, _P, _I, _I, _P],
    "pb_parallel_add": [_I, _P, _P, _P, _F, _P, _P, _P, _L, _P, _P, _P, _P, _F, _P, _P, _L, _P, _P, _P, _I, _I, _P],
    "pb_activation": [_I, _I, _P, _P, ctypes.c_longlong, _I, _P],
    "pb_min_gru_run": [],
    "pb_min_gru": [_I, _P, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P],
    "pb_diff_combine": [_I, _I, _P, _P, _I, _I, _I, _I, _F, _F, _F, _P],
    "pb_retention_chunk": [],
    "pb_retention_step_supported": [_I, _I],
    "pb_retention": [_I, _P, _L, _P, _P, _P, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P, _P],
    "pb_scaled_sum": [_I, _I, _P, _P, _P, _F, _F, ctypes.c_longlong, _P],
    "pb_concat_streams": [_I, _P, _P, _P, _P, _I, _I, _P],
}
_fns = {}
# the entry points that launch kernels (the others answer questions on the host): what PULSAR_PROF=1 times
_LAUNCHERS = {"embed", "scale_cap", "move_ids", "add_rmsnorm", "rope_table", "qk_norm_rope_write", "silu_mul", "gather_words",
              "paged_attention_generic", "paged_attention_decode", "paged_attention_decode_tc", "paged_attention_decode_tc_fused",
              "paged_attention_decode_tc_qkv",
              "paged_attention_prefill_tc", "paged_attention_prefill_tcgen05", "gemm_skinny", "gemm_skinny_accumulate",
              "gemm_skinny_scaled", "gemm_tcgen05", "gemm_tcgen05_stream", "gemm_simt", "sample", "argmax", "table_update",
              "paged_attention_general", "paged_attention_general_tiled", "paged_attention_general_tc", "qkv_split_write", "heads_linear", "latent_prepare", "latent_expand_keys", "sigmoid_gate", "causal_conv_silu",
              "selective_scan", "selective_scan_prompt", "selective_scan_chunked", "post_norm_add", "clamped_glu",
              "post_norm_add_bias", "glu_bias", "qk_prepare", "sigmoid_gate_strided", "add_bias", "moe_route", "moe_gate_up", "moe_down", "moe_grouped",
              "norm_shift", "parallel_add", "activation", "min_gru", "diff_combine", "retention", "scaled_sum", "concat_streams"}


class KernelError(RuntimeError):
    pass


def fn(name: str):
    f = _fns.get(name)
    if f is None:
        f = getattr(library(), name)
        f.argtypes = _SIGNATURES[name]
        f.restype = ctypes.c_int
        if profiling.ENABLED and name[3:] in _LAUNCHERS:
            f = profiling.timed_launcher(name, f)
        _fns[name] = f
    return f


def register_signature(name: str, argtypes) -> None:
    _SIGNATURES[name] = list(argtypes)


LAUNCHES = 0      # kernels of this library launched so far (each wrapper call launches one or more)


def check(status: int, name: str, kernels: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += kernels
    if status != 0:
        what = _ERRORS.get(status, f"CUDA error {status}")
        raise KernelError(f"{name}: {what}")


def code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not float32 or bfloat16") from None


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernel arguments must be contiguous CUDA tensors "
                              f"(found device {t.device}, contiguous={t.is_contiguous()}); there is no CPU path")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] (float32) = table[ids[t]] * scale."""
    _cuda(table, ids, out)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and out.shape == (ids.numel(), table.shape[1])
    check(fn("pb_embed")(code(table.dtype), _p(table), _p(ids), _p(out), ids.numel(), table.shape[1], table.shape[0],
                         float(scale), stream()), "embed")


def scale_cap(x: torch.Tensor, scale: float = 1.0, cap: Optional[float] = None) -> None:
    """In place on float32 values: x *= scale, then cap * tanh(x / cap) where a cap is given."""
    _cuda(x)
    assert x.dtype == torch.float32
    check(fn("pb_scale_cap")(_p(x), x.numel(), float(scale), float(cap or 0.0), stream()), "scale_cap")


def move_ids(ids: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, src_ids: torch.Tensor) -> None:
    """ids[dst[i]] = src_ids[src[i]] (all int32 on the device): sampled tokens of the step before become
    this step's input without a trip through the host."""
    _cuda(ids, dst, src, src_ids)
    assert ids.dtype == dst.dtype == src.dtype == src_ids.dtype == torch.int32 and dst.numel() == src.numel()
    check(fn("pb_move_ids")(_p(ids), _p(dst), _p(src), _p(src_ids), dst.numel(), stream()), "move_ids")


def table_update(resident: torch.Tensor, updates: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """Apply a step's (row, logical page, page id) triples to the resident block tables [rows, stride] and copy the
    step's rows (``rows`` [S]) into ``out`` [S, width]; ``updates`` = the count, then the triples (all int32)."""
    _cuda(resident, updates, rows, out)
    assert resident.dtype == updates.dtype == rows.dtype == out.dtype == torch.int32
    s, width = out.shape
    assert rows.numel() == s and resident.dim() == 2 and width <= resident.shape[1]
    check(fn("pb_table_update")(_p(resident), resident.shape[1], _p(updates), _p(rows), s, width, _p(out), stream()), "table_update")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, write_back: bool = True) -> None:
    """x = residual (+ delta); residual = x when write_back; out = rmsnorm(x) * weight.
    With ``rows`` only those rows are normalised, gathered into ``out``; the residual is left alone."""
    _cuda(residual, delta, weight, out, rows)
    width = residual.shape[-1]
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == width
    assert delta is None or (delta.dtype == out.dtype and delta.shape == residual.shape)
    if rows is not None:
        assert rows.dtype == torch.int32
        write_back = False
    n_out = rows.numel() if rows is not None else residual.shape[0]
    assert out.shape == (n_out, width)
    check(fn("pb_add_rmsnorm")(code(out.dtype), _p(residual), _p(delta), _p(weight), _p(out), _p(rows), n_out, width,
                               float(eps), int(write_back), stream()), "add_rmsnorm")


def rope_table(positions: torch.Tensor, quadrants_per_position: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
               magnitude: float = 1.0) -> None:
    """cos / sin [N, half] of position * frequency (the table holds quadrants per position in float64), each multiplied by
    ``magnitude``."""
    _cuda(positions, quadrants_per_position, cos, sin)
    half = quadrants_per_position.numel()
    assert positions.dtype == torch.int32 and quadrants_per_position.dtype == torch.float64
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32
    assert cos.shape == (positions.numel(), half) and sin.shape == cos.shape
    check(fn("pb_rope_table")(_p(positions), _p(quadrants_per_position), _p(cos), _p(sin), positions.numel(), half,
                              float(magnitude), stream()), "rope_table")


def qk_norm_rope_write(qkv: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor],
                       v_pool: Optional[torch.Tensor], slots: Optional[torch.Tensor], cos: torch.Tensor,
                       sin: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                       eps: float, n_heads: int, n_kv_heads: int, head_dim: int, rotary: int, page_size: int) -> None:
    """Per-head RMSNorm (when weights are given) and rotation of q and k, q to ``q_out``,
    k and v into their pages.  ``n_kv_heads`` 0: the row holds q only."""
    _cuda(qkv, q_out, k_pool, v_pool, slots, cos, sin, q_weight, k_weight)
    _check_against(k_pool)
    n = qkv.shape[0]
    assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim and q_out.dtype == qkv.dtype
    assert cos.shape == (n, rotary // 2) and sin.shape == cos.shape and cos.dtype == torch.float32
    if n_kv_heads:
        assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype and slots.dtype == torch.int32
        assert k_pool.shape[1:] == (n_kv_heads, page_size, head_dim) and v_pool.shape == k_pool.shape
    for w in (q_weight, k_weight):
        assert w is None or (w.dtype == torch.float32 and w.numel() == head_dim)
    check(fn("pb_qk_norm_rope_write")(code(qkv.dtype), _p(qkv), _p(q_out), _p(k_pool), _p(v_pool), _p(slots), _p(cos),
                                      _p(sin), _p(q_weight), _p(k_weight), float(eps), n, n_heads, n_kv_heads, head_dim,
                                      rotary, page_size, stream()), "qk_norm_rope_write")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(gate_up, out)
    n, two_i = gate_up.shape
    assert out.shape == (n, two_i // 2) and out.dtype == gate_up.dtype and two_i % 2 == 0
    check(fn("pb_silu_mul")(code(out.dtype), _p(gate_up), _p(out), n, two_i // 2, stream()), "silu_mul")


def paged_attention_generic(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                            block_table: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                            seq_of_token: torch.Tensor, scale: float, window: Optional[int]) -> None:
    _cuda(q, k_pool, v_pool, out, block_table, cu_q, kv_len, seq_of_token)
    _check_against(k_pool)
    n, hq, d = q.shape
    pages, hkv, page_size, d2 = k_pool.shape
    assert d2 == d and v_pool.shape == k_pool.shape and out.shape == q.shape
    assert k_pool.dtype == q.dtype and v_pool.dtype == q.dtype and out.dtype == q.dtype
    for t in (block_table, cu_q, kv_len, seq_of_token):
        assert t.dtype == torch.int32
    assert block_table.dim() == 2 and seq_of_token.numel() == n
    check(fn("pb_paged_attention_generic")(code(q.dtype), _p(q), _p(k_pool), _p(v_pool), _p(out), _p(block_table),
                                           block_table.shape[1], _p(cu_q), _p(kv_len), _p(seq_of_token), n, hq, hkv, d,
                                           page_size, float(scale), int(window or 0), stream()), "paged_attention_generic")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = a @ w.T in float32 multiply-adds (no tensor cores)."""
    _cuda(a, w, out)
    m, k = a.shape
    n, k2 = w.shape
    assert k2 == k and out.shape == (m, n)
    check(fn("pb_gemm_simt")(code(a.dtype), code(w.dtype), code(out.dtype), _p(a), _p(w), _p(out), m, n, k, stream()),
          "gemm_simt")


_argmax_keys = {}
_sample_work = {}


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           uniform: Optional[torch.Tensor] = None, any_greedy: bool = True) -> None:
    """out[r] = argmax (temperature <= 0 or None) or a draw from the filtered softmax.
    ``any_greedy=False`` promises that every row has a temperature > 0."""
    _cuda(logits, out, temperature, top_k, top_p, uniform)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() == rows
    assert temperature is None or (temperature.dtype == torch.float32 and temperature.numel() == rows)
    assert top_k is None or (top_k.dtype == torch.int32 and top_k.numel() == rows)
    assert top_p is None or (top_p.dtype == torch.float32 and top_p.numel() == rows)
    assert uniform is None or (uniform.dtype == torch.float32 and uniform.numel() == rows)
    keys = _argmax_keys.get(logits.device)
    if keys is None or keys.numel() < rows:
        keys = _argmax_keys[logits.device] = torch.empty(max(rows, 256), dtype=torch.int64, device=logits.device)
    if temperature is None:                       # all rows greedy: many blocks per row
        check(fn("pb_argmax")(_p(logits), rows, vocab, _p(keys), _p(out), stream()), "argmax", kernels=2)
        return
    if uniform is None:
        raise KernelError("sample: rows with a temperature need uniform numbers")
    need = int(fn("pb_sample_workspace")(rows)) * 1024
    work = _sample_work.get(logits.device)
    if work is None or work.numel() < need:
        work = _sample_work[logits.device] = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=logits.device)
    filtered = top_k is not None or top_p is not None
    check(fn("pb_sample")(_p(logits), rows, vocab, _p(temperature), _p(top_k), _p(top_p), _p(uniform), 1 if any_greedy else 0,
                          _p(work), _p(keys), _p(out), stream()), "sample", kernels=(2 if any_greedy else 0) + (5 if filtered else 2))


class _Gating:
    """The gating of the fused gate/up products launched inside: (limit, alpha, shift) for
    out = g' * sigmoid(alpha * g') * (u' + shift), g' = min(g, limit), u' = clamp(u, -limit, limit); None: SwiGLU."""

    def __init__(self, gating):
        self.gating = gating

    def __enter__(self):
        if self.gating is not None:
            fn("pb_set_gating")(float(self.gating[0]), float(self.gating[1]), float(self.gating[2]))

    def __exit__(self, *exc):
        if self.gating is not None:
            fn("pb_set_gating")(0.0, 1.0, 0.0)


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False, gating=None) -> bool:
    """The weight-streaming product for up to 16 tokens (bfloat16).  ``swiglu``: ``w`` holds
    gate rows then up rows and ``out`` [M, inter] receives silu(gate) * up, or with ``gating`` =
    (limit, alpha, shift) the clamped form min(gate, limit) * sigmoid(alpha * .) * (clamp(up) + shift).
    Returns False, having done nothing, when the sizes are not the kernel's."""
    m, k = a.shape
    n = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k:
        return False
    mode = 1 if swiglu else 0
    if not fn("pb_gemm_skinny_supported")(mode, m, n, k):
        return False
    _cuda(a, w, out)
    assert out.shape == (m, n // 2 if swiglu else n)
    with _Gating(gating if swiglu else None):
        check(fn("pb_gemm_skinny")(mode, code(out.dtype), _p(a), _p(w), _p(out), m, n, k, stream()), "gemm_skinny")
    return True


# Steps of up to 16 tokens (bfloat16): the output and down projections add their result to the float32 residual
# stream inside the product (no bfloat16 rounding of it, no addition in the norm kernel), and the down projection
# prepares the next layer's first norm, which the q/k/v product then applies itself (one norm kernel per layer
# less).  PULSAR_FUSED_NORM=0 turns both off.  The same for the norm in front of gate/up is built and tested but
# off: that product has thousands of short-lived blocks, and what each of them adds at its end costs more than the
# norm kernel it saves (measured: 3.77 against 3.61 ms per step at batch 8); PULSAR_FUSED_NORM_MLP=1 turns it on.
FUSED_NORM = os.environ.get("PULSAR_FUSED_NORM", "1") != "0"
FUSED_NORM_MLP = os.environ.get("PULSAR_FUSED_NORM_MLP", "0") != "0"


def _aligned32(*tensors) -> bool:
    return all(t.data_ptr() % 32 == 0 for t in tensors)


def fused_projection_supported(m: int, w: torch.Tensor, swiglu: bool = False) -> bool:
    """Whether ``linear_prenormed`` / ``linear_accumulate`` take ``m`` tokens against the weight ``w`` [N, K]."""
    return bool(FUSED_NORM and w.dtype == torch.bfloat16 and w.is_cuda and w.data_ptr() % 32 == 0
                and fn("pb_gemm_skinny_fused_supported")(1 if swiglu else 0, m, w.shape[0], w.shape[1]))


def norm_parts_numel(m: int, width: int) -> int:
    """Floats of the buffer in which ``linear_accumulate`` leaves the parts of the sums of squares of ``m`` rows
    ``width`` wide: a part per 16 columns and row, then a 64-bit word per row (its sum and a tag)."""
    return (width // 16 + 2) * m


def linear_accumulate(a: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, next_norm_weight: Optional[torch.Tensor] = None,
                      prepared: Optional[torch.Tensor] = None, parts: Optional[torch.Tensor] = None) -> bool:
    """residual (float32) += a @ w.T for up to 16 tokens: the projection's result goes into the residual stream
    without a bfloat16 rounding and without a kernel for the addition.  With ``next_norm_weight`` (the weight of
    the RMSNorm that follows) the kernel also prepares that norm: ``prepared`` [M, N] bfloat16 = residual *
    weight and ``parts`` (float32, ``norm_parts_numel(M, N)`` elements) = each block's part of the rows' sums of
    squares [N / 16, M], which ``linear_prenormed`` takes (and behind which it keeps the sums).  Returns False, having done nothing, when the sizes or dtypes are not the kernel's."""
    m, k = a.shape
    n = w.shape[0]
    if (not FUSED_NORM or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or residual.dtype != torch.float32
            or w.shape[1] != k or residual.shape != (m, n)):
        return False
    if not fn("pb_gemm_skinny_fused_supported")(0, m, n, k) or not _aligned32(a, w):
        return False
    _cuda(a, w, residual, next_norm_weight, prepared, parts)
    if next_norm_weight is not None:
        assert next_norm_weight.dtype == torch.float32 and next_norm_weight.numel() == n
        assert prepared.dtype == torch.bfloat16 and prepared.shape == (m, n)
        assert parts.dtype == torch.float32 and parts.numel() >= norm_parts_numel(m, n)
    check(fn("pb_gemm_skinny_accumulate")(_p(a), _p(w), _p(residual), m, n, k, _p(next_norm_weight), _p(prepared), _p(parts),
                                          stream()), "gemm_skinny_accumulate")
    return True


def linear_prenormed(prepared: torch.Tensor, parts: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor,
                     swiglu: bool = False) -> bool:
    """out = rmsnorm(residual) @ w.T (or its SwiGLU form) from what ``linear_accumulate`` prepared: the product of
    ``prepared`` (residual * norm weight, bfloat16) with each token's sums scaled by rsqrt(mean(residual^2) + eps),
    the mean from ``parts``.  Returns False, having done nothing, when the sizes or dtypes are not the kernel's."""
    m, k = prepared.shape
    n = w.shape[0]
    if (not FUSED_NORM or prepared.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16
            or w.shape[1] != k or parts.dtype != torch.float32 or k % 64):
        return False
    mode = 1 if swiglu else 0
    if not fn("pb_gemm_skinny_fused_supported")(mode, m, n, k) or not _aligned32(prepared, w):
        return False
    _cuda(prepared, parts, w, out)
    assert out.shape == (m, n // 2 if swiglu else n) and parts.numel() >= norm_parts_numel(m, k)
    check(fn("pb_gemm_skinny_scaled")(mode, _p(prepared), _p(w), _p(out), m, n, k, _p(parts), float(eps), stream()),
          "gemm_skinny_scaled")
    return True


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False, gating=None) -> bool:
    """The tcgen05 / TMA product for many tokens (bfloat16 operands, float32 accumulation in
    tensor memory).  ``swiglu`` as in ``gemm_skinny``.  Returns False, having done nothing,
    when the sizes are not the kernel's (K must be a multiple of 8)."""
    m, k = a.shape
    n = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k:
        return False
    mode = 1 if swiglu else 0
    if not fn("pb_gemm_tcgen05_supported")(mode, m, n, k):
        return False
    _cuda(a, w, out)
    assert out.shape == (m, n // 2 if swiglu else n)
    with _Gating(gating if swiglu else None):
        check(fn("pb_gemm_tcgen05")(mode, code(out.dtype), _p(a), _p(w), _p(out), m, n, k, stream()), "gemm_tcgen05")
    return True


# Which products of 17 to 128 tokens take this library's weight-streaming tcgen05 kernel instead of the library
# product: "auto" those whose weights have tiles for four rounds of all SMs or more (the head: there the kernel's
# persistent form is ahead of the library, 6.1 against 6.0 TB/s at 64 tokens); "1" all of them (measured behind the
# library for the projections of a layer at the 8B sizes: see profiles/); "0" none.
STREAM_GEMM = os.environ.get("PULSAR_GEMM_STREAM", "auto")
_STREAM_MIN_ROWS = 4 * 148 * 128


def _stream_wanted(m: int, n: int) -> bool:
    if m > 128 or STREAM_GEMM == "0" or GEMM_BACKEND == "library":
        return False
    return STREAM_GEMM == "1" or n >= _STREAM_MIN_ROWS


# Float32 partial sums and tile tickets of the product below, one pair per device, grown on demand.  A buffer
# that was outgrown stays alive: a captured graph may still name it.  Kernels of one stream share the pair (each
# finishes with it before the next one starts, and leaves the tickets zero).
_stream_scratch = {}
_stream_scratch_old = []


def _stream_workspace(device: torch.device, mode: int, m: int, n: int, k: int):
    floats, tickets = ctypes.c_longlong(0), ctypes.c_int(0)
    fn("pb_gemm_tcgen05_stream_workspace")(mode, m, n, k, ctypes.byref(floats), ctypes.byref(tickets))
    if floats.value == 0:
        return None, None
    have = _stream_scratch.get(device)
    if have is None or have[0].numel() < floats.value or have[1].numel() < tickets.value:
        if torch.cuda.is_current_stream_capturing():
            return None, None                 # no allocation inside a capture: whole tiles this once
        if have is not None:
            _stream_scratch_old.append(have)
        have = (torch.empty(max(floats.value, have[0].numel() if have else 0), dtype=torch.float32, device=device),
                torch.zeros(max(tickets.value, have[1].numel() if have else 0, 2048), dtype=torch.int32, device=device))
        _stream_scratch[device] = have
    return have


def gemm_tcgen05_stream(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> bool:
    """The weight-streaming tcgen05 / TMA product for up to 128 tokens (bfloat16 operands, float32 accumulation
    in tensor memory, K cut into slices whose partial sums meet in a float32 workspace).  ``swiglu`` as in
    ``gemm_skinny``.  Returns False, having done nothing, when the sizes are not the kernel's."""
    m, k = a.shape
    n = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k:
        return False
    mode = 1 if swiglu else 0
    if not fn("pb_gemm_tcgen05_stream_supported")(mode, m, n, k):
        return False
    _cuda(a, w, out)
    assert out.shape == (m, n // 2 if swiglu else n)
    work, tickets = _stream_workspace(a.device, mode, m, n, k)
    status = fn("pb_gemm_tcgen05_stream")(mode, code(out.dtype), _p(a), _p(w), _p(out), m, n, k,
                                          _p(work) if work is not None else None, work.numel() if work is not None else 0,
                                          _p(tickets) if tickets is not None else None,
                                          tickets.numel() if tickets is not None else 0, stream())
    if status == -3:
        return False                 # sizes that leave no room for its ring of stages
    check(status, "gemm_tcgen05_stream")
    return True


def gemm_tcgen05_error() -> int:
    """0 unless a block of the tcgen05 product ever gave up a bounded wait (synchronises)."""
    return int(fn("pb_gemm_tcgen05_error")())


# ---------------------------------------------------------------- bounded waits: limit and error words
# The kernels that wait on barriers (the tcgen05 product, the two tcgen05 attention kernels) bound every wait by
# a clock limit; a block whose wait runs out sets its kernel's error word, lets its copies land, frees its tensor
# memory and returns, and what the kernel wrote is then not to be trusted.  The reference's engine turns a step
# that cannot go on into an exception (pulsar-core/src/runtime/engine.cpp:809-814) and its Python layer
# poisons the engine (pulsar/src/pulsar/rt/sync.py:21-34); the words below are how this engine learns of it.
WAIT_WORD_NAMES = ("tcgen05 product", "tcgen05 attention, one head per block", "tcgen05 attention, two heads per block",
                   "tcgen05 product for up to 128 tokens", "bounds check of the debug build")
N_WAIT_WORDS = len(WAIT_WORD_NAMES)          # the last one is 0 in a build without the checks
BOUNDS_CODES = {2: "a block table named a page outside its pool (the access was skipped)",
                3: "a slot outside its pool (the write was dropped)"}
_bounds_words = {}


def bounds_checked() -> bool:
    """Whether the loaded library is the debug build whose kernels check page ids and slots
    (built with PULSAR_CHECK_BOUNDS=1)."""
    return bool(fn("pb_bounds_checked")())


def _bounds_word() -> torch.Tensor:
    dev = torch.cuda.current_device()
    word = _bounds_words.get(dev)
    if word is None:
        word = _bounds_words[dev] = torch.zeros(1, dtype=torch.int32, device="cuda")
    return word


def _check_against(pool: Optional[torch.Tensor]) -> None:
    """Debug build: the kernels launched next check page ids and slots against this pool's size."""
    if pool is not None and bounds_checked():
        fn("pb_set_pool_bounds")(int(pool.shape[0]), _p(_bounds_word()))


def bounds_error() -> int:
    """0, or the largest code a bounds check recorded (synchronises); always 0 without the debug build."""
    return int(_bounds_word().item()) if bounds_checked() else 0


def clear_bounds_error() -> None:
    if bounds_checked():
        _bounds_word().zero_()
WAIT_ROLES = {2: "the TMA producer", 3: "the MMA issuer", 4: "the epilogue or softmax warps", 9: "the wait self-test"}
_wait_words = {}
_check_buf = {}


class DeviceWaitError(KernelError):
    """A kernel gave up a bounded wait: its output, and everything computed from it, is not valid."""


def wait_word_addresses() -> "ctypes.Array":
    """Device addresses of the error words of the current device (looked up once per device)."""
    dev = torch.cuda.current_device()
    got = _wait_words.get(dev)
    if got is None:
        got = (ctypes.c_void_p * N_WAIT_WORDS)()
        one = (ctypes.c_void_p * 1)()
        two = (ctypes.c_void_p * 2)()
        three = (ctypes.c_void_p * 1)()
        if (fn("pb_gemm_tcgen05_wait_control")(0, -1, one) != 0 or fn("pb_prefill_tcgen05_wait_control")(0, -1, two) != 0
                or fn("pb_gemm_tcgen05_stream_wait_control")(0, -1, three) != 0):
            raise KernelError("the addresses of the wait error words could not be had")
        got[0], got[1], got[2], got[3] = one[0], two[0], two[1], three[0]
        got[4] = _bounds_word().data_ptr()
        _wait_words[dev] = got
    return got


def gather_wait_words(out: torch.Tensor) -> None:
    """out[:N_WAIT_WORDS] (int32, device) = the error words, read in the stream behind whatever was launched before."""
    _cuda(out)
    assert out.dtype == torch.int32 and out.numel() >= N_WAIT_WORDS
    check(fn("pb_gather_words")(wait_word_addresses(), N_WAIT_WORDS, _p(out), stream()), "gather_words")


def set_wait_limit(cycles: int) -> None:
    """The limit of every bounded wait, in clock cycles (4e9 at first, about two seconds)."""
    if cycles <= 0:
        raise ValueError("the wait limit must be positive")
    if fn("pb_gemm_tcgen05_wait_control")(int(cycles), -1, None) != 0 or \
            fn("pb_prefill_tcgen05_wait_control")(int(cycles), -1, None) != 0 or \
            fn("pb_gemm_tcgen05_stream_wait_control")(int(cycles), -1, None) != 0:
        raise KernelError("the wait limit could not be set")


def set_wait_words(value: int) -> None:
    """Write all three error words (0 clears them once a failure has been dealt with)."""
    if fn("pb_gemm_tcgen05_wait_control")(0, int(value), None) != 0 or \
            fn("pb_prefill_tcgen05_wait_control")(0, int(value), None) != 0 or \
            fn("pb_gemm_tcgen05_stream_wait_control")(0, int(value), None) != 0:
        raise KernelError("the wait error words could not be written")


def wait_selftest() -> None:
    """One thread waits on a barrier nobody arrives on until the limit runs out and sets the product's error word to 9."""
    check(fn("pb_gemm_tcgen05_wait_selftest")(stream()), "wait_selftest")


def describe_wait_words(words) -> Optional[str]:
    """None when all words are 0, else which kernel gave up and in which role."""
    bad = [(i, WAIT_WORD_NAMES[i], int(w)) for i, w in enumerate(words) if int(w) != 0]
    if not bad:
        return None
    return "; ".join(f"{name}: {BOUNDS_CODES.get(w, 'code ' + str(w))}" if i == N_WAIT_WORDS - 1 else
                     f"{name}: {WAIT_ROLES.get(w, 'role ' + str(w))} gave up a bounded wait" for i, name, w in bad)


def check_wait_words() -> None:
    """Read the words now (synchronises) and raise DeviceWaitError if one is set."""
    buf = _check_buf.get(torch.cuda.current_device())
    if buf is None:
        buf = _check_buf[torch.cuda.current_device()] = torch.zeros(8, dtype=torch.int32, device="cuda")
    gather_wait_words(buf)
    what = describe_wait_words(buf[:N_WAIT_WORDS].tolist())
    if what is not None:
        raise DeviceWaitError(what)


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = a @ w.T.  float32 operands take the float32 CUDA-core product (true 32-bit,
    no reduced-precision mode).  bfloat16 operands: up to 16 rows take this library's
    weight-streaming kernel; more rows take the library product with float32 accumulation,
    as the reference does for every projection (pulsar-core/src/model/qwen3.cpp:82-84:
    at::linear)."""
    if a.dtype == torch.float32 and w.dtype == torch.float32:
        gemm_simt(a, w, out)
        return
    _cuda(a, w, out)
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: operand dtypes {a.dtype} / {w.dtype} must both be float32 or both bfloat16")
    if gemm_skinny(a, w, out):
        return
    if _stream_wanted(a.shape[0], w.shape[0]) and gemm_tcgen05_stream(a, w, out):
        return
    if GEMM_BACKEND == "tcgen05" and gemm_tcgen05(a, w, out):
        return
    with profiling.kernel("library product (torch.mm)"):
        if out.dtype == torch.bfloat16:
            torch.mm(a, w.t(), out=out)
        else:
            out.copy_(torch.mm(a, w.t(), out_dtype=torch.float32))


def gated_linear(ctx, a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, gating=None) -> None:
    """out [M, I] = silu(a Wg^T) * (a Wu^T) with ``w_gate_up`` = gate rows then up rows; with ``gating`` = (limit, alpha,
    shift) the clamped form g * sigmoid(alpha * g) * (u + shift), g = min(a Wg^T, limit), u = clamp(a Wu^T, -limit, limit).
    In bfloat16, up to 16 rows (the weight-streaming kernel) and more than 128 rows (the tcgen05 kernel)
    take one kernel that never writes the [M, 2I] intermediate; otherwise the product followed by the
    gating kernel."""
    if gemm_skinny(a, w_gate_up, out, swiglu=True, gating=gating):
        return
    if gating is None and _stream_wanted(a.shape[0], w_gate_up.shape[0]) and gemm_tcgen05_stream(a, w_gate_up, out, swiglu=True):
        return
    # Between 17 and 128 rows the product is still bound by streaming the weights, which the library's small
    # tiles do faster (4.5 against 3.2 TB/s at the 8B sizes) than the tcgen05 kernel's 128 x 256 tiles.
    fused = GEMM_BACKEND == "tcgen05" or (GEMM_BACKEND == "auto" and a.shape[0] > 128)
    if fused and gemm_tcgen05(a, w_gate_up, out, swiglu=True, gating=gating):
        return
    gate_up = ctx.scratch("mlp.gate_up", (a.shape[0], w_gate_up.shape[0]), a.dtype)
    linear(a, w_gate_up, gate_up)
    if gating is None:
        silu_mul(gate_up, out)
    else:
        if gating[2] != 1.0:
            raise KernelError("gated_linear: the gating kernel of the unfused path adds 1 to the clamped up part")
        clamped_glu(gate_up, out, gating[0], gating[1])


_FORCED_SPLITS = int(os.environ.get("PULSAR_DECODE_SPLITS", "0") or 0)      # > 0: this many splits, for measurements
_DECODE_SLOTS = 296          # two blocks of the decode attention kernel on each of the 148 SMs


def decode_splits(n_seqs: int, n_kv_heads: int, table_tokens: int = 4096) -> int:
    """Splits of the keys per (sequence, kv head), at most 32 and at most one per 256 tokens that the
    block table can name.  While all blocks fit the SMs at once: as many splits as still fit.  With
    more (sequence, kv head) pairs than that, the blocks run in rounds, and what costs is a last round
    too thin to keep HBM busy (a block alone pulls about 37 GB/s against its 22 GB/s share of a full
    round, so a last round under 0.6 of the slots takes 0.6 of a round all the same); splits shorten
    the rounds and cost about 4 % for the merge.  Measured at context 4096, 8 kv heads: batch 48 runs
    12 % faster with 3 splits than with 1, batch 64 is fastest with 1.  A function of the batch and of
    the block table's width alone (the width of a step of single tokens grows in buckets), so that a
    captured step stays valid while its sequences grow."""
    pairs = max(1, n_seqs * n_kv_heads)
    most = max(1, min(32, table_tokens // 256))
    if _FORCED_SPLITS > 0:
        return min(most, _FORCED_SPLITS)
    if pairs <= _DECODE_SLOTS:
        return max(1, min(most, _DECODE_SLOTS // pairs))
    best, best_cost = 1, None
    for k in range(1, min(most, 8) + 1):
        rounds = pairs * k / _DECODE_SLOTS
        whole, rest = int(rounds), rounds - int(rounds)
        cost = (whole + (max(0.6, rest) if rest > 1e-9 else 0.0)) / k * (1.0 if k == 1 else 1.04 + 0.005 * k)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = k, cost
    return best


_TICKETS = 1 << 16
_decode_tickets = {}


def decode_tc_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tensor-core decode kernel takes these sizes (bfloat16, head size 64 or 128,
    groups up to 16, pages that divide 64)."""
    if dtype != torch.bfloat16:
        return False
    return bool(fn("pb_decode_tc_supported")(BF16, n_heads, n_kv_heads, head_dim, page_size))


def paged_attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                           partial: torch.Tensor, block_table: torch.Tensor, kv_len: torch.Tensor, scale: float,
                           window: Optional[int], n_splits: int, tensor_cores: Optional[bool] = None,
                           fused: Optional[bool] = None) -> None:
    """One query token per sequence: q, out [S, Hq, D].  ``partial`` is float32 scratch of at
    least S * Hq * n_splits * (D + 2) elements.  ``tensor_cores``: None picks the tensor-core
    kernel where it applies, False forces the CUDA-core kernel, True insists.  ``fused``: the
    tensor-core kernel finishes the job itself (a single split writes the result; of several the
    last one to finish merges) instead of a second kernel.  None: only for a single split, where
    it saves a launch; with several splits the ticket and fences cost what the combine kernel costs
    (measured: 5.04 vs 4.99 ms per step at batch 8)."""
    _cuda(q, k_pool, v_pool, out, partial, block_table, kv_len)
    _check_against(k_pool)
    s, hq, d = q.shape
    pages, hkv, page_size, d2 = k_pool.shape
    assert d2 == d and v_pool.shape == k_pool.shape and out.shape == q.shape and kv_len.numel() == s
    assert k_pool.dtype == q.dtype and v_pool.dtype == q.dtype and out.dtype == q.dtype
    assert block_table.dtype == torch.int32 and kv_len.dtype == torch.int32 and block_table.shape[0] == s
    assert partial.dtype == torch.float32 and partial.numel() >= s * hq * n_splits * (d + 2)
    if tensor_cores is None:
        tensor_cores = decode_tc_supported(q.dtype, hq, hkv, d, page_size)
    if fused is None:
        fused = n_splits == 1
    if tensor_cores and fused and n_splits <= 64 and s * hkv <= _TICKETS:
        tickets = _decode_tickets.get(q.device)
        if tickets is None:
            tickets = _decode_tickets[q.device] = torch.zeros(_TICKETS, dtype=torch.int32, device=q.device)
        check(fn("pb_paged_attention_decode_tc_fused")(code(q.dtype), _p(q), _p(k_pool), _p(v_pool), _p(out), _p(partial),
                                                       _p(tickets), _p(block_table), block_table.shape[1], _p(kv_len), s, hq,
                                                       hkv, d, page_size, float(scale), int(window or 0), n_splits, stream()),
              "paged_attention_decode_tc_fused")
        return
    name = "pb_paged_attention_decode_tc" if tensor_cores else "pb_paged_attention_decode"
    check(fn(name)(code(q.dtype), _p(q), _p(k_pool), _p(v_pool), _p(out), _p(partial),
                   _p(block_table), block_table.shape[1], _p(kv_len), s, hq, hkv, d, page_size,
                   float(scale), int(window or 0), n_splits, stream()), name[3:], kernels=2)


# A step of single tokens can leave the per-head norm, the rotation and the cache write of its projected rows to
# the attention kernel (one launch less per layer in a chain of dependent launches).  PULSAR_FUSED_QK=0: a kernel
# of its own does them, as in every other step.
FUSED_QK = os.environ.get("PULSAR_FUSED_QK", "1") != "0"


def decode_qkv_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, rotary: int, page_size: int) -> bool:
    """Whether ``paged_attention_decode_qkv`` takes these sizes: those of the tensor-core decode kernel, heads of
    their own keys and values, the whole head rotating."""
    return bool(FUSED_QK and n_kv_heads > 0 and rotary == head_dim
                and decode_tc_supported(dtype, n_heads, n_kv_heads, head_dim, page_size))


def paged_attention_decode_qkv(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                               cos: torch.Tensor, sin: torch.Tensor, eps: float, slots: torch.Tensor, k_pool: torch.Tensor,
                               v_pool: torch.Tensor, out: torch.Tensor, partial: torch.Tensor, block_table: torch.Tensor,
                               kv_len: torch.Tensor, scale: float, window: Optional[int], n_splits: int,
                               fused: Optional[bool] = None) -> None:
    """Decode attention straight from the projected rows ``qkv`` [S, (Hq + 2 Hkv) * D] (bfloat16): the kernel
    normalises and rotates the query heads and the newest key itself and writes that key and the value to
    ``slots`` of their pools before it reads them.  ``out`` [S, Hq, D]; the rest as ``paged_attention_decode``."""
    _cuda(qkv, q_weight, k_weight, cos, sin, slots, k_pool, v_pool, out, partial, block_table, kv_len)
    _check_against(k_pool)
    s, hq, d = out.shape
    pages, hkv, page_size, d2 = k_pool.shape
    assert d2 == d and v_pool.shape == k_pool.shape and qkv.shape == (s, (hq + 2 * hkv) * d) and kv_len.numel() == s
    assert qkv.dtype == torch.bfloat16 and k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype and out.dtype == qkv.dtype
    assert cos.shape == (s, d // 2) and sin.shape == cos.shape and cos.dtype == torch.float32 and sin.dtype == torch.float32
    assert slots.dtype == torch.int32 and slots.numel() == s
    assert block_table.dtype == torch.int32 and kv_len.dtype == torch.int32 and block_table.shape[0] == s
    assert partial.dtype == torch.float32 and partial.numel() >= s * hq * n_splits * (d + 2)
    for w in (q_weight, k_weight):
        assert w is None or (w.dtype == torch.float32 and w.numel() == d)
    if fused is None:
        fused = n_splits == 1
    tickets = None
    if fused and n_splits <= 64 and s * hkv <= _TICKETS:
        tickets = _decode_tickets.get(qkv.device)
        if tickets is None:
            tickets = _decode_tickets[qkv.device] = torch.zeros(_TICKETS, dtype=torch.int32, device=qkv.device)
    check(fn("pb_paged_attention_decode_tc_qkv")(code(qkv.dtype), _p(qkv), _p(q_weight), _p(k_weight), _p(cos), _p(sin), float(eps),
                                                 _p(slots), _p(k_pool), _p(v_pool), _p(out), _p(partial), _p(tickets),
                                                 _p(block_table), block_table.shape[1], _p(kv_len), s, hq, hkv, d, page_size,
                                                 float(scale), int(window or 0), n_splits, stream()),
          "paged_attention_decode_tc_qkv", kernels=1 if tickets is not None else 2)


def prefill_tc_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    if dtype != torch.bfloat16:
        return False
    return bool(fn("pb_prefill_tc_supported")(BF16, n_heads, n_kv_heads, head_dim, page_size))


def prefill_tc_tiles(q_lens) -> int:
    """Blocks along the query axis: each sequence's new tokens in tiles of 64."""
    tile = fn("pb_prefill_tc_tile")()
    return sum(-(-int(n) // tile) for n in q_lens)


def paged_attention_prefill_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                               block_table: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor, n_q_tiles: int,
                               scale: float, window: Optional[int]) -> None:
    """Tensor-core attention for a ragged batch of portions (bfloat16, head size 64 or 128)."""
    _cuda(q, k_pool, v_pool, out, block_table, cu_q, kv_len)
    _check_against(k_pool)
    n, hq, d = q.shape
    pages, hkv, page_size, d2 = k_pool.shape
    assert d2 == d and v_pool.shape == k_pool.shape and out.shape == q.shape
    assert k_pool.dtype == q.dtype and v_pool.dtype == q.dtype and out.dtype == q.dtype
    assert block_table.dtype == torch.int32 and cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32
    s = kv_len.numel()
    assert cu_q.numel() == s + 1 and block_table.shape[0] == s
    check(fn("pb_paged_attention_prefill_tc")(code(q.dtype), _p(q), _p(k_pool), _p(v_pool), _p(out), _p(block_table),
                                              block_table.shape[1], _p(cu_q), _p(kv_len), s, n_q_tiles, hq, hkv, d,
                                              page_size, float(scale), int(window or 0), stream()),
          "paged_attention_prefill_tc")


def prefill_tcgen05_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    if dtype != torch.bfloat16:
        return False
    return bool(fn("pb_prefill_tcgen05_supported")(BF16, n_heads, n_kv_heads, head_dim, page_size))


def prefill_tcgen05_tiles(q_lens) -> int:
    """Blocks along the query axis: each sequence's new tokens in tiles of 128."""
    tile = fn("pb_prefill_tcgen05_tile")()
    return sum(-(-int(n) // tile) for n in q_lens)


def prefill_tcgen05_error() -> int:
    """0 unless a block of the tcgen05 attention ever gave up a bounded wait (synchronises)."""
    return int(fn("pb_prefill_tcgen05_error")())


def paged_attention_prefill_tcgen05(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                                    block_table: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor, n_q_tiles: int,
                                    scale: float, window: Optional[int]) -> None:
    """tcgen05 attention for a ragged batch of portions (bfloat16, head size 128, pages of 8 or more
    tokens).  Pool rows that were never written must hold finite values."""
    _cuda(q, k_pool, v_pool, out, block_table, cu_q, kv_len)
    _check_against(k_pool)
    n, hq, d = q.shape
    pages, hkv, page_size, d2 = k_pool.shape
    assert d2 == d and v_pool.shape == k_pool.shape and out.shape == q.shape
    assert q.is_contiguous() and k_pool.is_contiguous() and v_pool.is_contiguous() and out.is_contiguous()
    assert k_pool.dtype == q.dtype and v_pool.dtype == q.dtype and out.dtype == q.dtype
    assert block_table.dtype == torch.int32 and cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32
    s = kv_len.numel()
    assert cu_q.numel() == s + 1 and block_table.shape[0] == s
    check(fn("pb_paged_attention_prefill_tcgen05")(code(q.dtype), _p(q), _p(k_pool), _p(v_pool), _p(out), _p(block_table),
                                                   block_table.shape[1], _p(cu_q), _p(kv_len), n, s, n_q_tiles, pages, hq,
                                                   hkv, d, page_size, float(scale), int(window or 0), stream()),
          "paged_attention_prefill_tcgen05")


def attention(ctx, q: torch.Tensor, cache, out: torch.Tensor, scale: float, window: Optional[int]) -> None:
    """Attention of the step's query tokens over their pages.  ``cache`` is a CacheView
    (pools, block table), ``ctx`` the StepContext (cu_q, kv_len, seq_of_token).  A step of
    single tokens only takes a split-key decode kernel; anything else the tcgen05 kernel where it
    applies (bfloat16, head size 128, pages of 8 or more), else the mma.sync kernel (bfloat16, head
    size 64 or 128), else the generic kernel.  ``PULSAR_ATTENTION=mma`` leaves the tcgen05 kernel out."""
    if ctx.all_decode:
        n_splits = decode_splits(ctx.n_seqs, cache.k_pool.shape[1], cache.block_table.shape[1] * cache.k_pool.shape[2])
        partial = ctx.scratch("attn.partial", (ctx.n_seqs * q.shape[1] * n_splits * (q.shape[2] + 2),), torch.float32)
        paged_attention_decode(q, cache.k_pool, cache.v_pool, out, partial, cache.block_table, ctx.kv_len, scale,
                               window, n_splits)
        return
    hkv, page_size = cache.k_pool.shape[1], cache.k_pool.shape[2]
    use_tcgen05 = ATTENTION_BACKEND != "mma" and prefill_tcgen05_supported(q.dtype, q.shape[1], hkv, q.shape[2], page_size)
    if use_tcgen05 or prefill_tc_supported(q.dtype, q.shape[1], hkv, q.shape[2], page_size):
        # The scheduler puts the decoded tokens of a mixed step first: those sequences take the decode kernel
        # (a tile of 64 or 128 query rows for one token would waste the tensor cores on every key tile), the
        # portions behind them the prefill kernel, over the same arrays.
        q_lens = ctx.host.q_lens
        n_dec = 0
        while n_dec < len(q_lens) and q_lens[n_dec] == 1:
            n_dec += 1
        table, cu_q, kv_len = cache.block_table, ctx.cu_q, ctx.kv_len
        if n_dec > 0:
            n_splits = decode_splits(n_dec, hkv, table.shape[1] * page_size)
            partial = ctx.scratch("attn.partial", (n_dec * q.shape[1] * n_splits * (q.shape[2] + 2),), torch.float32)
            paged_attention_decode(q[:n_dec], cache.k_pool, cache.v_pool, out[:n_dec], partial, table[:n_dec], kv_len[:n_dec],
                                   scale, window, n_splits)
            table, cu_q, kv_len, q_lens = table[n_dec:], cu_q[n_dec:], kv_len[n_dec:], q_lens[n_dec:]
        if use_tcgen05:
            paged_attention_prefill_tcgen05(q, cache.k_pool, cache.v_pool, out, table, cu_q, kv_len,
                                            prefill_tcgen05_tiles(q_lens), scale, window)
        else:
            paged_attention_prefill_tc(q, cache.k_pool, cache.v_pool, out, table, cu_q, kv_len, prefill_tc_tiles(q_lens),
                                       scale, window)
        return
    paged_attention_generic(q, cache.k_pool, cache.v_pool, out, cache.block_table, ctx.cu_q, ctx.kv_len,
                            ctx.seq_of_token, scale, window)


# ---------------------------------------------------------------- attention in its general form, latent attention
# The general attention has two kernels: the tiled one (keys and values of a tile staged in shared memory and shared by 16
# query rows; splits of the keys where the rows alone do not fill the GPU) for rows that are multiples of 16 bytes, and the
# plain one (a block per token and head) for every other size.  PULSAR_GENERAL_TILED=0 leaves the tiled one out.
GENERAL_TILED = os.environ.get("PULSAR_GENERAL_TILED", "1") != "0"
GENERAL_ROWS = 16
# Steps with portions of GENERAL_TC_MIN tokens or more, on bfloat16 pages with (key, value) widths (64, 64), (64, 128), (128, 128) or
# (192, 128), take the tensor-core kernel, which splits queries and softmax weights into two bfloat16 halves each.
# PULSAR_GENERAL_TC=0 leaves it out.
GENERAL_TC = os.environ.get("PULSAR_GENERAL_TC", "1") != "0"
GENERAL_TC_MIN = 16


_GENERAL_SLOTS = 592         # four blocks of the tiled general attention on each of the 148 SMs: a block's tiles load and compute in
                             # turn, so short runs of tiles in many blocks hide what one block cannot


def general_splits(blocks: int, table_tokens: int) -> int:
    """Splits of the keys for the tiled general attention: as many as bring the grid to four blocks per SM, at most 32 and
    at most one per 64 tokens that the block table can name.  A function of the step's shape alone (not of the lengths),
    so that a captured step stays valid while its sequences grow."""
    if blocks >= _GENERAL_SLOTS:
        return 1
    return max(1, min(32, _GENERAL_SLOTS // max(1, blocks), table_tokens // 64))


def paged_attention_general(ctx, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                            block_table: torch.Tensor, scale: float, window: Optional[int] = None, chunk: Optional[int] = None,
                            slopes: Optional[torch.Tensor] = None, key_width: Optional[int] = None,
                            value_width: Optional[int] = None, tiled: Optional[bool] = None,
                            tensor_cores: Optional[bool] = None, keep_first: int = 0, softcap: Optional[float] = None,
                            sinks: Optional[torch.Tensor] = None, v_share: int = 1) -> None:
    """Attention of the step's tokens (``ctx``: cu_q, kv_len, seq_of_token, host.q_lens) with float32 queries ``q``
    [N, Hq, Dk] over pools [pages, Hkv, page, stride]: keys are the first ``key_width`` (default: all) elements of a
    ``k_pool`` row, values the first ``value_width`` of a ``v_pool`` row (the two may be one tensor).  ``slopes`` [Hq]
    float32: the score loses slopes[h] * distance.  ``window`` / ``chunk`` bound the visible keys from below; the first
    ``keep_first`` keys of a sequence stay visible all the same.  ``softcap``: the scaled score becomes softcap *
    tanh(score / softcap).  ``sinks`` [Hq] float32: the softmax's denominator also holds exp(sinks[h]).
    ``tiled``: None picks the tiled kernel where it applies, False forces the plain one.  ``tensor_cores``: None picks the
    tensor-core kernel for steps with portions where it applies, False never, True insists.
    ``v_share``: that many consecutive key heads read one value head (``v_pool`` has Hkv / v_share heads): several score
    maps over the same values.  ``out`` has the pools' dtype or float32 (rows that are subtracted from one another afterwards
    stay unrounded)."""
    _cuda(q, k_pool, v_pool, out, block_table, slopes, sinks)
    _check_against(k_pool)
    n, hq, dk = q.shape
    keep_first, softcap = int(keep_first or 0), float(softcap or 0.0)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == hq)
    pages, hkv, page_size, k_stride = k_pool.shape
    v_stride = v_pool.shape[3]
    dv = out.shape[2]
    assert q.dtype == torch.float32 and k_pool.dtype == v_pool.dtype and out.dtype in (k_pool.dtype, torch.float32)
    assert out.shape[:2] == (n, hq)
    pool_code, out_f32 = code(k_pool.dtype), int(out.dtype == torch.float32)
    v_share = int(v_share)
    assert (key_width or k_stride) == dk and (value_width or v_stride) == dv and v_share >= 1 and hkv % v_share == 0
    assert v_pool.shape[:3] == (pages, hkv // v_share, page_size)
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    assert slopes is None or (slopes.dtype == torch.float32 and slopes.numel() == hq)
    q_lens = ctx.host.q_lens
    insist = tensor_cores is True
    if tensor_cores is None:
        tensor_cores = GENERAL_TC and max(q_lens) >= GENERAL_TC_MIN
    if tensor_cores:
        fits = fn("pb_attention_general_tc_supported")(pool_code, _p(q), _p(k_pool), _p(v_pool), hq, hkv, dk, dv, k_stride,
                                                       v_stride)
        if fits:
            rows = fn("pb_attention_general_tc_tile")()
            n_q_tiles = sum(-(-int(ql) // rows) for ql in q_lens)
            check(fn("pb_paged_attention_general_tc")(pool_code, _p(q), _p(k_pool), _p(v_pool), _p(out), _p(block_table),
                                                      block_table.shape[1], _p(ctx.cu_q), _p(ctx.kv_len), _p(slopes), len(q_lens),
                                                      n_q_tiles, hq, hkv, dk, dv, k_stride, v_stride, page_size, float(scale),
                                                      int(window or 0), int(chunk or 0), keep_first, softcap, _p(sinks), v_share, out_f32, stream()),
                  "paged_attention_general_tc")
            return
        if insist:
            raise KernelError("paged_attention_general: the tensor-core kernel does not take these sizes or dtypes")
    if tiled is None:
        tiled = GENERAL_TILED
    if tiled and fn("pb_attention_general_tiled_supported")(pool_code, _p(k_pool), _p(v_pool), hq, hkv, dk, dv, k_stride,
                                                            v_stride):
        group = hq // hkv
        row_tiles = sum(-(-(int(ql) * group) // GENERAL_ROWS) for ql in ctx.host.q_lens)
        n_splits = general_splits(row_tiles * hkv, block_table.shape[1] * page_size)
        partial = ctx.scratch("attn.general.partial", (n * hq * n_splits * (dv + 2),), torch.float32) if n_splits > 1 else None
        check(fn("pb_paged_attention_general_tiled")(pool_code, _p(q), _p(k_pool), _p(v_pool), _p(out), _p(partial),
                                                     _p(block_table), block_table.shape[1], _p(ctx.cu_q), _p(ctx.kv_len),
                                                     _p(slopes), n, len(ctx.host.q_lens), row_tiles, n_splits, hq, hkv, dk, dv,
                                                     k_stride, v_stride, page_size, float(scale), int(window or 0),
                                                     int(chunk or 0), keep_first, softcap, _p(sinks), v_share, out_f32, stream()),
              "paged_attention_general_tiled", kernels=2 if n_splits > 1 else 1)
        return
    check(fn("pb_paged_attention_general")(pool_code, _p(q), _p(k_pool), _p(v_pool), _p(out), _p(block_table),
                                           block_table.shape[1], _p(ctx.cu_q), _p(ctx.kv_len), _p(ctx.seq_of_token), _p(slopes),
                                           n, hq, hkv, dk, dv, k_stride, v_stride, page_size, float(scale), int(window or 0),
                                           int(chunk or 0), keep_first, softcap, _p(sinks), v_share, out_f32, stream()), "paged_attention_general")


def qkv_split_write(qkv: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                    slots: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int,
                    page_size: int, n_value_heads: Optional[int] = None, positions: Optional[torch.Tensor] = None,
                    q_temperature: Optional[Tuple[float, int]] = None) -> None:
    """Split the fused projection rows [q: Hq*Dk | k: Hk*Dk | v: Hv*Dv]: queries to float32 ``q_out`` [N, Hq, Dk], keys and
    values into their pages (``n_kv_heads`` 0: the row holds q only; ``n_value_heads``: Hv where it is not Hk).
    ``q_temperature`` = (coef, every): the query at position p (``positions`` int32 [N]) is multiplied by
    1 + coef * ln(floor((p + 1) / every) + 1)."""
    _cuda(qkv, q_out, k_pool, v_pool, slots, positions)
    _check_against(k_pool)
    n = qkv.shape[0]
    n_v = n_kv_heads if n_value_heads is None else int(n_value_heads)
    assert qkv.shape[1] == (n_heads + n_kv_heads) * key_dim + n_v * value_dim and q_out.dtype == torch.float32
    assert q_out.shape == (n, n_heads, key_dim)
    if n_kv_heads:
        assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype and slots.dtype == torch.int32
        assert k_pool.shape[1:] == (n_kv_heads, page_size, key_dim) and v_pool.shape[1:] == (n_v, page_size, value_dim)
    coef, every = (0.0, 1) if q_temperature is None else (float(q_temperature[0]), int(q_temperature[1]))
    if coef != 0.0:
        assert positions is not None and positions.dtype == torch.int32 and positions.numel() == n and every > 0
    check(fn("pb_qkv_split_write")(code(qkv.dtype), _p(qkv), _p(q_out), _p(k_pool), _p(v_pool), _p(slots), n, n_heads, n_kv_heads,
                                   n_v, key_dim, value_dim, page_size, _p(positions), coef, every, stream()), "qkv_split_write")


def heads_linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None) -> None:
    """out[n, h, :] = a[n, h, :] @ w[h] for every head (float32 sums in ascending k), times sigmoid(gate[n, h, :]) where a
    gate is given.  ``a`` [N, H, K], ``out`` [N, H, M] and ``gate`` [N, H * M] may be views whose last dimension is
    contiguous; ``w`` [H, K, M] is contiguous.  ``out`` is float32 or of the dtype of ``a`` and ``w``."""
    n, h, k = a.shape
    h2, k2, m = w.shape
    assert (h2, k2) == (h, k) and out.shape == (n, h, m) and a.dtype == w.dtype and w.is_contiguous()
    assert a.is_cuda and w.is_cuda and out.is_cuda and a.stride(2) == 1 and out.stride(2) == 1
    g_tok = 0
    if gate is not None:
        assert gate.dtype == a.dtype and gate.shape == (n, h * m) and gate.stride(1) == 1 and gate.is_cuda
        g_tok = gate.stride(0)
    check(fn("pb_heads_linear")(code(a.dtype), code(out.dtype), _p(a), a.stride(0), a.stride(1), _p(w), _p(out), out.stride(0),
                                out.stride(1), _p(gate), g_tok, n, h, m, k, stream()), "heads_linear")


def latent_prepare(q: torch.Tensor, down: Optional[torch.Tensor], norm_weight: Optional[torch.Tensor], eps: float,
                   cos: torch.Tensor, sin: torch.Tensor, slots: Optional[torch.Tensor], pool: Optional[torch.Tensor],
                   q_out: torch.Tensor, n_heads: int, dim: int, rot_dim: int, rank: int, page_size: int,
                   plain_too: bool = False, latent_out: Optional[torch.Tensor] = None,
                   rot_out: Optional[torch.Tensor] = None) -> None:
    """Per token: where ``down`` [N, rank + rot_dim] is given, its latent part RMS-normed with ``norm_weight`` and its
    rotated part turned at the token's position go to the token's slot of ``pool`` [pages, 1, page, rank + rot_dim] (and to
    ``latent_out`` [N, rank] / ``rot_out`` [N, rot_dim] where given); every head's rotated query part (behind ``dim`` plain
    dimensions of a ``q`` row) goes, turned, to the tail of its row of ``q_out`` float32 [N, H, row]: row = rank + rot_dim,
    or with ``plain_too`` row = dim + rot_dim with the plain dimensions copied to the front.  ``q`` and ``down`` may be column
    slices of one tensor.  The rotation pairs neighbours; ``cos`` / ``sin`` [N, rotated dims / 2]."""
    n = q.shape[0]
    front = dim if plain_too else rank
    assert q.is_cuda and q.stride(1) == 1 and q.shape[1] == n_heads * (dim + rot_dim)
    assert q_out.dtype == torch.float32 and q_out.is_contiguous() and q_out.shape == (n, n_heads, front + rot_dim)
    assert cos.dtype == torch.float32 and cos.shape == sin.shape and cos.shape[0] == n and cos.is_contiguous()
    rot_dims = 2 * cos.shape[1]
    down_tok = 0
    if down is not None:
        assert down.dtype == q.dtype and down.shape == (n, rank + rot_dim) and down.stride(1) == 1
        assert norm_weight.dtype == torch.float32 and norm_weight.numel() == rank and slots.dtype == torch.int32
        assert pool.dtype == q.dtype and pool.is_contiguous() and pool.shape[1:] == (1, page_size, rank + rot_dim)
        _check_against(pool)
        down_tok = down.stride(0)
        for t, width in ((latent_out, rank), (rot_out, rot_dim)):
            assert t is None or (t.dtype == q.dtype and t.is_contiguous() and t.shape == (n, width) and t.is_cuda)
    else:
        assert latent_out is None and rot_out is None
    check(fn("pb_latent_prepare")(code(q.dtype), _p(q), q.stride(0), _p(down), down_tok, _p(norm_weight), float(eps), _p(cos),
                                  _p(sin), _p(slots), _p(pool), _p(q_out), front + rot_dim, front, 1 if plain_too else 0,
                                  _p(latent_out), _p(rot_out), n, n_heads, dim, rot_dim, rot_dims, rank, page_size, stream()),
          "latent_prepare")


def latent_expand_keys(plain: torch.Tensor, shared: torch.Tensor, keys: torch.Tensor) -> None:
    """keys[n, h, :] = [plain[n, h, :] | shared[n, :]]: every head's expanded key beside the rotated part all heads share."""
    _cuda(plain, shared, keys)
    n, h, dim = plain.shape
    rot_dim = shared.shape[1]
    assert shared.shape[0] == n and keys.shape == (n, h, dim + rot_dim) and plain.dtype == shared.dtype == keys.dtype
    check(fn("pb_latent_expand_keys")(code(keys.dtype), _p(plain), _p(shared), _p(keys), n, h, dim, rot_dim, stream()),
          "latent_expand_keys")


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> None:
    """x[n, :] *= sigmoid(gate[n, :]) in place (float32 arithmetic); ``gate`` may be a column slice."""
    _cuda(x)
    n, width = x.shape
    assert gate.is_cuda and gate.dtype == x.dtype and gate.shape == (n, width) and gate.stride(1) == 1
    check(fn("pb_sigmoid_gate")(code(x.dtype), _p(x), _p(gate), gate.stride(0), n, width, stream()), "sigmoid_gate")


# ---------------------------------------------------------------- selective scan
def causal_conv_silu(ctx, xz: torch.Tensor, channels: int, taps: torch.Tensor, bias: torch.Tensor, arena: torch.Tensor,
                     tail_offset: int, out: torch.Tensor) -> None:
    """out [N, channels] = silu(causal convolution per channel) of the first ``channels`` columns of ``xz``; inputs before a
    portion's start come from the sequence's slot of ``arena`` (float32 [slots, floats]; the tail [channels, taps - 1] at
    ``tail_offset``).  ``taps`` float32 [channels, T], the last column weighs the current token."""
    _cuda(xz, taps, bias, arena, out)
    n = xz.shape[0]
    assert taps.dtype == bias.dtype == arena.dtype == torch.float32 and taps.shape[0] == channels and bias.numel() == channels
    assert out.shape == (n, channels) and out.dtype == xz.dtype and xz.shape[1] >= channels and arena.dim() == 2
    check(fn("pb_causal_conv_silu")(code(xz.dtype), _p(xz), xz.shape[1], _p(taps), _p(bias), _p(arena), arena.shape[1],
                                    int(tail_offset), _p(ctx.cu_q), _p(ctx.seq_of_token), _p(ctx.state_slots), _p(out), n, channels,
                                    taps.shape[1], stream()), "causal_conv_silu")


def selective_scan(ctx, x: torch.Tensor, xz: torch.Tensor, proj: torch.Tensor, w_dt: torch.Tensor, dt_bias: torch.Tensor,
                   a_log: torch.Tensor, d_skip: torch.Tensor, arena: torch.Tensor, tail_offset: int, n_taps: int,
                   out: torch.Tensor) -> None:
    """The selective scan over the step's portions, token after token per sequence, with each sequence's state
    [inner, state] (float32) in its slot of ``arena``; moves the slot's convolution tail on when a portion is done.
    x [N, inner] convolution output, xz [N, 2 inner] the input projection (convolution inputs | gates), proj [N, dt_rank +
    2 state] = [r | B | C], w_dt [inner, dt_rank]; out [N, inner] = (scan + d_skip * x) * silu(gate)."""
    _cuda(x, xz, proj, w_dt, dt_bias, a_log, d_skip, arena, out)
    n, inner = x.shape
    n_state = a_log.shape[1]
    dt_rank = w_dt.shape[1]
    assert xz.shape == (n, 2 * inner) and proj.shape == (n, dt_rank + 2 * n_state) and w_dt.shape[0] == inner
    assert x.dtype == xz.dtype == proj.dtype == w_dt.dtype == out.dtype and out.shape == (n, inner)
    assert dt_bias.dtype == a_log.dtype == d_skip.dtype == arena.dtype == torch.float32 and a_log.shape[0] == inner
    assert arena.dim() == 2 and arena.shape[1] >= tail_offset + inner * (n_taps - 1) and tail_offset >= inner * n_state
    check(fn("pb_selective_scan")(code(x.dtype), _p(x), _p(xz), xz.shape[1], _p(proj), proj.shape[1], _p(w_dt), _p(dt_bias),
                                  _p(a_log), _p(d_skip), _p(arena), arena.shape[1], int(tail_offset), _p(out), _p(ctx.cu_q),
                                  _p(ctx.state_slots), ctx.n_seqs, inner, n_state, dt_rank, int(n_taps), stream()),
          "selective_scan")


def selective_scan_prompt_supported(n_state: int) -> bool:
    """Whether ``selective_scan_prompt`` takes this state size."""
    return bool(fn("pb_selective_scan_prompt_supported")(int(n_state)))


def selective_scan_chunked_supported(n_state: int) -> bool:
    """Whether ``selective_scan_prompt(..., chunked=True)`` takes this state size."""
    return bool(fn("pb_selective_scan_chunked_supported")(int(n_state)))


def selective_scan_prompt(ctx, x: torch.Tensor, xz: torch.Tensor, bc: torch.Tensor, dt_pre: torch.Tensor, dt_bias: torch.Tensor,
                          a_log: torch.Tensor, d_skip: torch.Tensor, arena: torch.Tensor, tail_offset: int, n_taps: int,
                          out: torch.Tensor, chunked: bool = False) -> None:
    """``selective_scan`` for steps with prompt portions: the step sizes' product was done beforehand (``dt_pre`` [N, inner]
    float32 = r @ w_dt.T, before bias and softplus) and ``bc`` [N, 2 state] = [B | C] (or a tensor whose rows start so).
    ``chunked``: the kernel that is parallel over tokens (256 at a time, a prefix scan over runs of 8) instead of the one
    that walks a portion token by token."""
    _cuda(x, xz, bc, dt_pre, dt_bias, a_log, d_skip, arena, out)
    n, inner = x.shape
    n_state = a_log.shape[1]
    assert xz.shape == (n, 2 * inner) and bc.shape[0] == n and bc.shape[1] >= 2 * n_state and dt_pre.shape == (n, inner)
    assert x.dtype == xz.dtype == bc.dtype == out.dtype and out.shape == (n, inner)
    assert dt_pre.dtype == dt_bias.dtype == a_log.dtype == d_skip.dtype == arena.dtype == torch.float32 and a_log.shape[0] == inner
    assert arena.dim() == 2 and arena.shape[1] >= tail_offset + inner * (n_taps - 1) and tail_offset >= inner * n_state
    name = "pb_selective_scan_chunked" if chunked else "pb_selective_scan_prompt"
    check(fn(name)(code(x.dtype), _p(x), _p(xz), xz.shape[1], _p(bc), bc.shape[1], _p(dt_pre), _p(dt_bias), _p(a_log), _p(d_skip),
                   _p(arena), arena.shape[1], int(tail_offset), _p(out), _p(ctx.cu_q), _p(ctx.state_slots), ctx.n_seqs, inner,
                   n_state, int(n_taps), stream()), name[3:])


# ---------------------------------------------------------------- norms behind sublayers, clamped gating
def post_norm_add(residual: torch.Tensor, delta: torch.Tensor, w_post: torch.Tensor, eps_post: float,
                  w_next: Optional[torch.Tensor] = None, eps_next: float = 0.0, out: Optional[torch.Tensor] = None) -> None:
    """residual (float32) += rmsnorm(delta) * w_post; with ``w_next`` also out = rmsnorm(residual) * w_next."""
    _cuda(residual, delta, w_post, w_next, out)
    n, width = residual.shape
    assert residual.dtype == torch.float32 and delta.shape == residual.shape and w_post.dtype == torch.float32
    assert w_post.numel() == width
    if w_next is not None:
        assert w_next.dtype == torch.float32 and w_next.numel() == width and out.shape == residual.shape and out.dtype == delta.dtype
    check(fn("pb_post_norm_add")(code(delta.dtype), _p(residual), _p(delta), _p(w_post), float(eps_post), _p(w_next),
                                 float(eps_next), _p(out), n, width, stream()), "post_norm_add")


def clamped_glu(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> None:
    """out [N, I] = g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit);
    ``gate_up`` [N, 2I] holds the gate columns, then the up columns."""
    _cuda(gate_up, out)
    n, two_i = gate_up.shape
    assert two_i % 2 == 0 and out.shape == (n, two_i // 2) and out.dtype == gate_up.dtype
    check(fn("pb_clamped_glu")(code(out.dtype), _p(gate_up), _p(out), n, two_i // 2, float(limit), float(alpha), stream()),
          "clamped_glu")


# ---------------------------------------------------------------- sublayers that read the stream itself; biases
def post_norm_add_bias(residual: torch.Tensor, delta: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                       w_post: Optional[torch.Tensor], eps_post: float, out: Optional[torch.Tensor]) -> None:
    """residual (float32) += rmsnorm(delta + bias) * w_post, and ``out`` = the stream as it now is, in the activation dtype
    (for the sublayer that reads it next).  ``delta`` None: only ``out`` is written."""
    _cuda(residual, delta, bias, w_post, out)
    n, width = residual.shape
    assert residual.dtype == torch.float32 and (delta is not None or out is not None)
    dtype = delta.dtype if delta is not None else out.dtype
    if delta is not None:
        assert delta.shape == residual.shape and w_post.dtype == torch.float32 and w_post.numel() == width
        assert bias is None or (bias.dtype == torch.float32 and bias.numel() == width)
    assert out is None or (out.shape == residual.shape and out.dtype == dtype)
    check(fn("pb_post_norm_add_bias")(code(dtype), _p(residual), _p(delta), _p(bias), _p(w_post), float(eps_post), _p(out), n, width,
                                      stream()), "post_norm_add_bias")


def glu_bias(gate_up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, gating=None) -> None:
    """out [N, I] = the gated unit of ``gate_up`` [N, 2I] + ``bias`` [2I] (gate columns, then up columns): SwiGLU, or with
    ``gating`` = (limit, alpha, shift) the clamped form of ``gated_linear``.  ``gate_up`` is float32 or of ``out``'s dtype."""
    _cuda(gate_up, bias, out)
    n, two_i = gate_up.shape
    assert two_i % 2 == 0 and out.shape == (n, two_i // 2) and gate_up.dtype in (out.dtype, torch.float32)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == two_i)
    limit, alpha, shift = gating if gating is not None else (0.0, 1.0, 0.0)
    check(fn("pb_glu_bias")(code(gate_up.dtype), code(out.dtype), _p(gate_up), _p(bias), _p(out), n, two_i // 2, float(limit), float(alpha), float(shift),
                            stream()), "glu_bias")


def qk_prepare(rows: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
               slots: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], n_heads: int,
               n_kv_heads: int, head_dim: int, rotary: int, page_size: int, q_bias: Optional[torch.Tensor] = None,
               k_bias: Optional[torch.Tensor] = None, unit_norm_eps: Optional[float] = None, values_from_keys: bool = False,
               q_norm: Optional[torch.Tensor] = None, k_norm: Optional[torch.Tensor] = None, norm_eps: Optional[float] = None,
               n_value_heads: int = 0, value_dim: int = 0) -> None:
    """Per head of the projection rows ``rows`` [N, >= (Hq + Hkv) * D] (query heads, then key heads; float32 or the
    pools' dtype; a column slice of a wider tensor will do): + bias; a key head as it then is goes to the value pool
    (``values_from_keys``); the first ``rotary`` dimensions turn in the rotate-half layout by ``cos`` / ``sin``
    [N, rotary / 2]; the head is divided by its root mean square (``unit_norm_eps``, no weight).  Queries to float32
    ``q_out`` [N, Hq, D], keys into their pages.  ``n_kv_heads`` 0: queries only.  ``norm_eps`` with ``q_norm`` / ``k_norm``
    (float32 [D]): a weighted RMS norm of every query and key head before the rotation.  ``n_value_heads`` value heads of
    ``value_dim`` behind the key heads in the row go to ``v_pool`` [pages, Hv, page, Dv] as they are."""
    _cuda(q_out, k_pool, v_pool, slots, cos, sin, q_bias, k_bias, q_norm, k_norm)
    _check_against(k_pool)
    n = rows.shape[0]
    assert rows.is_cuda and rows.stride(1) == 1 and rows.shape[1] >= (n_heads + n_kv_heads) * head_dim + n_value_heads * value_dim
    assert q_out.dtype == torch.float32 and q_out.shape == (n, n_heads, head_dim)
    if norm_eps is not None:
        assert q_norm.dtype == torch.float32 and q_norm.numel() == head_dim
        assert n_kv_heads == 0 or (k_norm.dtype == torch.float32 and k_norm.numel() == head_dim)
    if n_value_heads:
        assert n_kv_heads and not values_from_keys and v_pool.shape[1:] == (n_value_heads, page_size, value_dim)
        assert v_pool.dtype == k_pool.dtype
    pool_dtype = k_pool.dtype if n_kv_heads else rows.dtype
    if n_kv_heads:
        assert slots.dtype == torch.int32 and k_pool.shape[1:] == (n_kv_heads, page_size, head_dim)
        assert not values_from_keys or (v_pool.shape == k_pool.shape and v_pool.dtype == k_pool.dtype)
    if rotary:
        assert cos.dtype == torch.float32 and cos.shape == (n, rotary // 2) and sin.shape == cos.shape and sin.dtype == cos.dtype
    for b, heads in ((q_bias, n_heads), (k_bias, n_kv_heads)):
        assert b is None or (b.dtype == torch.float32 and b.numel() == heads * head_dim)
    check(fn("pb_qk_prepare")(code(rows.dtype), code(pool_dtype), _p(rows), rows.stride(0), _p(q_bias), _p(k_bias), _p(cos), _p(sin),
                              _p(q_out), _p(k_pool), _p(v_pool), _p(slots), n, n_heads, n_kv_heads, head_dim, int(rotary),
                              -1.0 if unit_norm_eps is None else float(unit_norm_eps), 1 if values_from_keys else 0, page_size,
                              _p(q_norm), _p(k_norm) if n_kv_heads else None, -1.0 if norm_eps is None else float(norm_eps),
                              int(n_value_heads), int(value_dim), stream()), "qk_prepare")


def sigmoid_gate_strided(x: torch.Tensor, gate: torch.Tensor, group: int = 1) -> None:
    """x[n, c] *= sigmoid(gate[n, c // group]) in place (float32 arithmetic); ``gate`` float32 or of x's dtype, possibly a column
    slice.  ``group`` neighbouring columns of x share one gate column (a head's width: one gate per head)."""
    _cuda(x)
    n, width = x.shape
    assert group >= 1 and width % group == 0
    assert gate.is_cuda and gate.shape == (n, width // group) and gate.stride(1) == 1
    check(fn("pb_sigmoid_gate_strided")(code(x.dtype), code(gate.dtype), _p(x), _p(gate), gate.stride(0), n, width, int(group),
                                        stream()), "sigmoid_gate_strided")


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    """x [N, width] += bias [width] (float32) in place."""
    _cuda(x, bias)
    assert x.dim() == 2 and bias.dtype == torch.float32 and bias.numel() == x.shape[1]
    check(fn("pb_add_bias")(code(x.dtype), _p(x), _p(bias), x.shape[0], x.shape[1], stream()), "add_bias")


# ---------------------------------------------------------------- mixture of experts
def moe_route(h: torch.Tensor, router: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, scale: float = 1.0,
              renormalize: bool = False, extra: Optional[torch.Tensor] = None, softmax: bool = False, renorm_eps: float = 0.0) -> None:
    """ids [N, top] int32 and weights [N, top] float32 of the ``top`` largest sigmoid(router @ h) per token (float32 sums;
    ties go to the lower index), weights times ``scale`` (after division by their sum with ``renormalize``).  With ``extra``
    (float32 [N, X]) the router has X more rows behind the experts' that compete for nothing: their sigmoids go there.
    ``softmax``: the scores are softmax(router @ h) over all experts instead; ``renorm_eps`` is added to the chosen scores' sum
    before the division."""
    _cuda(h, router, ids, weights, extra)
    n, width = h.shape
    n_extra = 0 if extra is None else extra.shape[1]
    e = router.shape[0] - n_extra
    top = ids.shape[1]
    assert router.dtype == torch.float32 and router.shape == (e + n_extra, width) and ids.dtype == torch.int32 and ids.shape == (n, top)
    assert weights.dtype == torch.float32 and weights.shape == (n, top)
    assert extra is None or (extra.dtype == torch.float32 and extra.shape == (n, n_extra))
    check(fn("pb_moe_route")(code(h.dtype), _p(h), _p(router), _p(ids), _p(weights), n, width, e, top, float(scale),
                             1 if renormalize else 0, n_extra, _p(extra), 1 if softmax else 0, float(renorm_eps), stream()), "moe_route")


def moe_gate_up(h: torch.Tensor, w_gate_up: torch.Tensor, ids: torch.Tensor, act: torch.Tensor, gating,
                in_weights: Optional[torch.Tensor] = None) -> None:
    """act [N * top, ff] = the gated unit (``gating`` = (limit, alpha, shift) as in ``gated_linear``; None: SwiGLU) of every
    token's chosen experts; ``w_gate_up`` [E, 2 ff, width] holds an expert's gate rows, then its up rows.  ``in_weights``
    (float32 [N, top]): the expert reads weight * h (applied to the gate and up sums in float32: W (w h) = w (W h))."""
    _cuda(h, w_gate_up, ids, act, in_weights)
    n, width = h.shape
    e, two_ff, w2 = w_gate_up.shape
    top = ids.shape[1]
    assert w2 == width and two_ff % 2 == 0 and act.shape == (n * top, two_ff // 2) and h.dtype == w_gate_up.dtype == act.dtype
    assert ids.dtype == torch.int32 and ids.shape[0] == n
    assert in_weights is None or (in_weights.dtype == torch.float32 and in_weights.shape == (n, top))
    limit, alpha, shift = gating if gating is not None else (0.0, 1.0, 0.0)
    check(fn("pb_moe_gate_up")(code(h.dtype), _p(h), _p(w_gate_up), _p(ids), _p(act), n, width, two_ff // 2, top, float(limit),
                               float(alpha), float(shift), _p(in_weights), stream()), "moe_gate_up")


def moe_down(act: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: Optional[torch.Tensor], add: Optional[torch.Tensor],
             out: torch.Tensor, add_scale: Optional[torch.Tensor] = None) -> None:
    """out [N, width] = add * add_scale + sum over a token's chosen experts, in the order of ``ids``, of weight * (w_down[e] @
    act row).  ``weights`` None: every pair counts once; ``add_scale`` (float32 [N]) None: 1."""
    _cuda(act, w_down, ids, weights, add, out, add_scale)
    n, width = out.shape
    e, w2, ff = w_down.shape
    top = ids.shape[1]
    assert w2 == width and act.shape == (n * top, ff) and act.dtype == w_down.dtype == out.dtype
    assert ids.dtype == torch.int32 and ids.shape == (n, top)
    assert weights is None or (weights.dtype == torch.float32 and weights.shape == (n, top))
    assert add is None or (add.shape == out.shape and add.dtype == out.dtype)
    assert add_scale is None or (add_scale.dtype == torch.float32 and add_scale.numel() == n)
    check(fn("pb_moe_down")(code(out.dtype), _p(act), _p(w_down), _p(ids), _p(weights), _p(add), _p(add_scale), _p(out), n, width, ff,
                            top, stream()), "moe_down")


# Steps of more than MOE_GROUPED_MIN tokens (bfloat16) sort their (token, expert) pairs by expert on the device and run every
# expert's rows through tensor-core tiles; fewer tokens read each chosen expert's weights per token.  The grouped form reads an
# expert's weights once however many tokens chose it (TMA streams them), which already pays for a handful of single tokens:
# 1.04 against 1.14 ms a step of 8 tokens at width 2,048 and 2.08 against 2.97 at 4,096 (32 experts, 4 a token); up to four
# tokens rarely share an expert and keep the two per-token kernels.  PULSAR_MOE_GROUPED=0 leaves the grouped products out,
# PULSAR_MOE_GROUPED_MIN=n moves the threshold.
MOE_GROUPED = os.environ.get("PULSAR_MOE_GROUPED", "1") != "0"
MOE_GROUPED_MIN = int(os.environ.get("PULSAR_MOE_GROUPED_MIN", "4") or 4)
# The grouped products run on the grouped form of the tcgen05 kernel (TMA, tensor memory) when they are given scratch for the
# gathered rows; PULSAR_MOE_TCGEN05=0 keeps them on mma.sync.
MOE_TCGEN05 = os.environ.get("PULSAR_MOE_TCGEN05", "1") != "0"


def moe_grouped_supported(dtype: torch.dtype, width: int, ff: int, n_experts: int) -> bool:
    return bool(MOE_GROUPED and dtype == torch.bfloat16 and fn("pb_moe_grouped_supported")(width, ff, n_experts))


def moe_grouped_workspace(n: int, top: int, n_experts: int) -> int:
    """int32 elements of the workspace ``moe_grouped`` needs for ``n`` tokens."""
    return int(fn("pb_moe_grouped_workspace")(n, top, n_experts))


def moe_grouped(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                add: Optional[torch.Tensor], act: torch.Tensor, y: torch.Tensor, out: torch.Tensor, work: torch.Tensor, gating,
                gathered: Optional[torch.Tensor] = None, weight_input: bool = False,
                add_scale: Optional[torch.Tensor] = None) -> None:
    """What ``moe_gate_up`` and ``moe_down`` compute together, for steps of many tokens (bfloat16): pairs sorted by expert, the
    experts' products in tensor-core tiles, the weighted sum in the order of ``ids``.  ``act`` [N * top, ff] bfloat16, ``y``
    [N * top, width] float32 and ``work`` (int32, ``moe_grouped_workspace`` elements) are scratch.  With ``gathered``
    (bfloat16 [N * top, width] scratch) the products run on the grouped tcgen05 kernel, else on mma.sync.  ``weight_input``: a
    pair's weight multiplies its expert's input (inside the gate/up epilogue) instead of its output; ``add_scale`` (float32
    [N]) multiplies ``add``."""
    _cuda(h, w_gate_up, w_down, ids, weights, add, act, y, out, work, gathered, add_scale)
    assert add_scale is None or (add_scale.dtype == torch.float32 and add_scale.numel() == h.shape[0])
    assert gathered is None or (gathered.dtype == torch.bfloat16 and gathered.shape == (h.shape[0] * ids.shape[1], h.shape[1]))
    n, width = h.shape
    e, two_ff, w2 = w_gate_up.shape
    ff, top = two_ff // 2, ids.shape[1]
    assert h.dtype == w_gate_up.dtype == w_down.dtype == act.dtype == out.dtype == torch.bfloat16 and w2 == width
    assert w_down.shape == (e, width, ff) and ids.dtype == torch.int32 and ids.shape == weights.shape == (n, top)
    assert weights.dtype == torch.float32 and act.shape == (n * top, ff) and y.dtype == torch.float32 and y.shape == (n * top, width)
    assert out.shape == (n, width) and (add is None or (add.shape == out.shape and add.dtype == out.dtype))
    assert work.dtype == torch.int32 and work.numel() >= moe_grouped_workspace(n, top, e)
    limit, alpha, shift = gating if gating is not None else (0.0, 1.0, 0.0)
    check(fn("pb_moe_grouped")(_p(h), _p(w_gate_up), _p(w_down), _p(ids), _p(weights), _p(add), _p(act), _p(y), _p(out), _p(work),
                               _p(gathered), n, width, ff, e, top, float(limit), float(alpha), float(shift), 1 if weight_input else 0,
                               _p(add_scale), stream()), "moe_grouped",
          kernels=4 if gathered is None else 5)


# ---------------------------------------------------------------- parallel sublayers, token shift, recurrences, differential maps
def norm_shift(ctx, residual: torch.Tensor, weight: torch.Tensor, eps: float, shift: Optional[torch.Tensor],
               state: Optional[torch.Tensor], h: torch.Tensor, hs: Optional[torch.Tensor], pending: Optional[torch.Tensor]) -> None:
    """h = rmsnorm(residual) * weight; with ``shift`` [width]: hs = h + (h' - h) * shift, h' the h of the token before in its
    sequence (the row above, or the sequence's kept row of ``state`` [slots, width] float32 for a portion's first token); the
    float32 h of every sequence's last token goes to ``pending`` [S, width] (``parallel_add`` moves it into ``state``)."""
    _cuda(residual, weight, shift, h, hs, pending)
    n, width = residual.shape
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == width and h.shape == (n, width)
    if shift is not None:
        assert shift.dtype == torch.float32 and shift.numel() == width and hs.shape == (n, width) and hs.dtype == h.dtype
        assert state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] >= width and state.stride(1) == 1 and state.is_cuda
        assert pending.dtype == torch.float32 and pending.numel() >= ctx.n_seqs * width
    check(fn("pb_norm_shift")(code(h.dtype), _p(residual), _p(weight), float(eps), _p(shift), _p(state),
                              0 if state is None else state.stride(0), _p(ctx.seq_of_token), _p(ctx.cu_q), _p(ctx.state_slots), _p(h),
                              _p(hs), _p(pending), n, width, stream()), "norm_shift")


def parallel_add(ctx, residual: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor], mult: float,
                 pending: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0, next_shift: Optional[torch.Tensor] = None,
                 next_state: Optional[torch.Tensor] = None, next_pending: Optional[torch.Tensor] = None,
                 h: Optional[torch.Tensor] = None, hs: Optional[torch.Tensor] = None) -> None:
    """residual += mult * (a + b) in float32 (``b`` may be None), and ``pending`` [S, width] -> the kept rows of ``state``.
    With ``next_weight`` the sum goes to ``out`` (another buffer than ``residual``) and the kernel also does the
    ``norm_shift`` of the layer that follows on it: ``h``, ``hs``, ``next_pending`` as there."""
    _cuda(residual, a, b, pending, out, next_weight, next_shift, next_pending, h, hs)
    n, width = residual.shape
    assert residual.dtype == torch.float32 and a.shape == (n, width) and (b is None or (b.shape == a.shape and b.dtype == a.dtype))
    for st in (state, next_state):
        assert st is None or (st.dtype == torch.float32 and st.dim() == 2 and st.shape[1] >= width and st.stride(1) == 1 and st.is_cuda)
    assert (pending is None) == (state is None)
    target = residual if out is None else out
    assert target.shape == residual.shape and target.dtype == torch.float32
    if next_weight is not None:
        assert out is not None and out.data_ptr() != residual.data_ptr() and h is not None and h.dtype == a.dtype
        assert next_weight.dtype == torch.float32 and next_weight.numel() == width
        assert next_shift is None or (next_shift.dtype == torch.float32 and hs is not None and next_state is not None
                                      and next_pending is not None)
    check(fn("pb_parallel_add")(code(a.dtype), _p(residual), _p(a), _p(b), float(mult), _p(target), _p(pending), _p(state),
                                0 if state is None else state.stride(0), _p(ctx.seq_of_token), _p(ctx.cu_q), _p(ctx.state_slots),
                                _p(next_weight), float(next_eps), _p(next_shift), _p(next_state),
                                0 if next_state is None else next_state.stride(0), _p(next_pending), _p(h), _p(hs), n, width,
                                stream()), "parallel_add")


ACTIVATIONS = {"gelu": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """out = act(x) element by element in float32, one rounding on store; ``kind``: "gelu" (the erf form), "gelu_tanh",
    "silu", "relu".  ``x`` float32 or of ``out``'s dtype."""
    _cuda(x, out)
    assert x.shape == out.shape and kind in ACTIVATIONS
    check(fn("pb_activation")(code(x.dtype), code(out.dtype), _p(x), _p(out), x.numel(), ACTIVATIONS[kind], stream()), "activation")


MIN_GRU_CHUNKED_MIN = 64      # portions of at least this many tokens take the recurrence in runs, parallel over tokens


def min_gru(ctx, proj: torch.Tensor, bias_z: torch.Tensor, bias_x: torch.Tensor, state: torch.Tensor, y: torch.Tensor) -> None:
    """The minimal gated recurrence over the step's tokens: ``proj`` float32 [N, 3 W] holds z | u | g pre-activations,
    ``state`` [slots, >= W] float32 each sequence's kept state (its first W elements), ``y`` [N, W] = S_t * silu(g_t)."""
    _cuda(proj, bias_z, bias_x, y)
    n, w3 = proj.shape
    width = w3 // 3
    assert proj.dtype == torch.float32 and w3 == 3 * width and y.shape == (n, width)
    assert bias_z.dtype == bias_x.dtype == torch.float32 and bias_z.numel() == bias_x.numel() == width
    assert state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] >= width and state.stride(1) == 1 and state.is_cuda
    max_runs, run_a, run_b, kernels = 0, None, None, 1
    if ctx.max_q_len >= MIN_GRU_CHUNKED_MIN:
        run = fn("pb_min_gru_run")()
        max_runs = sum(-(-int(q) // run) for q in ctx.host.q_lens)
        run_a = ctx.scratch("gru.run_a", (max_runs, width), torch.float32)
        run_b = ctx.scratch("gru.run_b", (max_runs, width), torch.float32)
        kernels = 3
    check(fn("pb_min_gru")(code(y.dtype), _p(proj), _p(bias_z), _p(bias_x), _p(state), state.stride(0), _p(ctx.cu_q),
                           _p(ctx.state_slots), _p(y), n, ctx.n_seqs, width, max_runs, _p(run_a), _p(run_b), stream()), "min_gru",
          kernels=kernels)


def diff_combine(maps: torch.Tensor, out: torch.Tensor, n_kv_heads: int, lam: float, eps: float, gain: float) -> None:
    """out [N, H, Dv] = unit_rms(a1 - lam * a2) * gain per head, from ``maps`` [N, 2 H, Dv] ordered so that the query heads of
    one key head are neighbours (head g R + r: first map at row 2 g R + r, second at (2 g + 1) R + r, R = H / n_kv_heads)."""
    _cuda(maps, out)
    n, h2, dv = maps.shape
    assert h2 % 2 == 0 and out.shape == (n, h2 // 2, dv) and (h2 // 2) % n_kv_heads == 0
    check(fn("pb_diff_combine")(code(maps.dtype), code(out.dtype), _p(maps), _p(out), n, h2 // 2, int(n_kv_heads), dv, float(lam),
                                float(eps), float(gain), stream()), "diff_combine")


# ---------------------------------------------------------------- retention
RETENTION_CHUNKED_MIN = 32     # portions of at least this many tokens take the recurrence in chunks, parallel over chunks


def retention(ctx, rows: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], decay: torch.Tensor,
              state: torch.Tensor, y: torch.Tensor, n_heads: int, key_dim: int, value_dim: int, rotary: int, key_scale: float,
              eps: float, chunked: Optional[bool] = None) -> None:
    """Linear attention with a fixed decay per head over the step's tokens.  ``rows`` float32 [N, >= 2 H (D + V)] holds per
    token q (H*D) | k (H*D) | v (H*V) | g (H*V); the first ``rotary`` dimensions of every q and k head turn in the rotate-half
    layout by ``cos`` / ``sin`` [N, rotary / 2], k is then multiplied by ``key_scale``.  Per head S <- decay S + k v^T
    (``state`` [slots, >= H*D*V] float32, each sequence's kept matrices), o = S^T q, and ``y`` [N, H*V] = o / rms(o) *
    silu(g) with ``eps`` inside the root.  ``chunked``: None picks the form that is parallel over chunks of tokens for steps
    with portions of ``RETENTION_CHUNKED_MIN`` tokens or more, False never, True always."""
    _cuda(cos, sin, decay, y)
    n = rows.shape[0]
    H, D, V = int(n_heads), int(key_dim), int(value_dim)
    assert rows.is_cuda and rows.dtype == torch.float32 and rows.stride(1) == 1 and rows.shape[1] >= 2 * H * (D + V)
    assert decay.dtype == torch.float32 and decay.numel() == H and y.shape == (n, H * V)
    assert state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] >= H * D * V and state.stride(1) == 1 and state.is_cuda
    if rotary:
        assert cos.dtype == torch.float32 and cos.shape == (n, rotary // 2) and sin.shape == cos.shape and sin.dtype == cos.dtype
    qr = ctx.scratch("retention.q", (n, H, D), torch.float32)
    kr = ctx.scratch("retention.k", (n, H, D), torch.float32)
    if chunked is None:
        # sizes whose state does not fit one block's registers always take the chunks (a function of the sizes alone)
        chunked = ctx.max_q_len >= RETENTION_CHUNKED_MIN or not fn("pb_retention_step_supported")(D, V)
    max_chunks, work, kernels = 0, None, 2
    if chunked:
        size = fn("pb_retention_chunk")()
        max_chunks = sum(-(-int(q) // size) for q in ctx.host.q_lens)
        work = ctx.scratch("retention.chunks", (max_chunks, H, D, V), torch.float32)
        kernels = 4
    check(fn("pb_retention")(code(y.dtype), _p(rows), rows.stride(0), _p(cos), _p(sin), _p(qr), _p(kr), _p(decay), _p(state),
                             state.stride(0), _p(ctx.cu_q), _p(ctx.state_slots), _p(y), n, ctx.n_seqs, H, D, V, int(rotary),
                             float(key_scale), float(eps), max_chunks, _p(work), stream()), "retention", kernels=kernels)


def scaled_sum(x: torch.Tensor, y: torch.Tensor, out: torch.Tensor, a: float, b: float) -> None:
    """out = a * x + b * y element by element (float32 arithmetic, one rounding); ``x`` and ``y`` share a dtype, ``out`` has
    its own and may be ``x`` or ``y`` where the dtypes agree."""
    _cuda(x, y, out)
    assert x.shape == y.shape == out.shape and x.dtype == y.dtype
    check(fn("pb_scaled_sum")(code(x.dtype), code(out.dtype), _p(x), _p(y), _p(out), float(a), float(b), x.numel(), stream()),
          "scaled_sum")


def concat_streams(residual: torch.Tensor, delta: Optional[torch.Tensor], origin: torch.Tensor, out: torch.Tensor) -> None:
    """out [N, 2 width] = [residual (+ delta) | origin] in ``out``'s dtype; ``residual`` and ``origin`` float32 [N, width]."""
    _cuda(residual, delta, origin, out)
    n, width = residual.shape
    assert residual.dtype == origin.dtype == torch.float32 and origin.shape == (n, width) and out.shape == (n, 2 * width)
    assert delta is None or (delta.shape == (n, width) and delta.dtype == out.dtype)
    check(fn("pb_concat_streams")(code(out.dtype), _p(residual), _p(delta), _p(origin), _p(out), n, width, stream()), "concat_streams")
