"""Python faces of the CUDA kernels.  Every function writes into tensors the caller gives.

Nothing here runs on the CPU and nothing falls back to a library model or a library
attention; matrix products of bfloat16 operands go to cuBLAS through ``torch.mm`` where
the reference's engine calls cuBLASLt (src/backend/ops/linear/nvidia/linear_cublas.cu:201-231),
and 32-bit products go to the SIMT kernel of ``csrc/gemm_simt.cu`` so that no
reduced-precision matrix mode can slip in.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ._lib import (BF16, F32, KernelError, Library, c_float, c_int, c_ll, c_void_p, dtype_code, need_contiguous, need_cuda,
                   need_int32, ptr, stream)

# Library products keep float32 sums: without this cuBLAS may pick split-K kernels that add partial sums in bfloat16.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

_elementwise = Library("elementwise")
_gemm_simt = Library("gemm_simt")
_attention_generic = Library("attention_generic")
_sampling = Library("sampling")
_attention_mma = Library("attention_mma")
_gemm_smallm = Library("gemm_smallm")
_gemm_tcgen05 = Library("gemm_tcgen05")
_attention_tcgen05 = Library("attention_tcgen05")
_rowwise = Library("rowwise")
_moe = Library("moe")
_ssm = Library("ssm")
_linrec = Library("linrec")
SMALL_M_ROWS = 16                # the weight-streaming kernel takes up to this many rows

__all__ = ["KernelError", "embedding", "rmsnorm", "add_rmsnorm", "rope_append", "rope_table", "gemm_smallm_rope", "can_fuse_rope_product", "silu_mul", "add", "cast",
           "gemm_nt", "linear", "linear_for_residual", "gemm_smallm", "gemm_tcgen05", "gemm_tcgen05_tiles", "tcgen05_status", "status_word", "linear_silu_mul", "raise_if_tcgen05_failed", "paged_attention", "attention", "decode_attention", "decode_attention_tma", "prefill_attention", "prefill_attention_tcgen05", "argmax", "sample", "repetition_penalty", "advance_decode",
           "embedding_positions", "softcap", "relu2", "gated_clamp_mul", "rmsnorm_append", "linear_per_head", "route_topk",
           "moe_group", "moe_gemm", "moe_combine", "linear_gated_clamp_mul", "linear_relu2", "moe_group_padded",
           "moe_gather_rows", "gemm_tcgen05_grouped", "route", "rotary", "latent_prepare", "sigmoid_mul", "segment_bounds",
           "causal_conv_silu", "conv_state_update", "ssm_scan", "gated_group_rmsnorm", "rotary_norm", "norm_add", "gelu_mul_rows",
           "linear_state", "linear_state_work_floats", "group_rmsnorm_gate", "tanh_norm", "tanh_norm_fold", "rms_pair_mean", "poly_norm",
           "row_gate"]


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """``out[n] = table[ids[n]] * scale``, the product in float32."""
    need_cuda(table, ids, out)
    need_int32("ids", ids)
    need_contiguous("table", table), need_contiguous("out", out), need_contiguous("ids", ids)
    n, hidden = ids.numel(), table.shape[1]
    if out.shape != (n, hidden):
        raise KernelError(f"embedding: out has shape {tuple(out.shape)}, expected {(n, hidden)}")
    _elementwise.call("zi_embedding", ptr(table), c_int(dtype_code(table.dtype)), ptr(ids), ptr(out),
                      c_int(dtype_code(out.dtype)), c_int(n), c_int(hidden), c_int(table.shape[0]), c_float(scale), stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    need_cuda(x, w, out)
    need_contiguous("x", x), need_contiguous("w", w), need_contiguous("out", out)
    rows, hidden = x.shape
    if w.numel() != hidden or out.shape != x.shape:
        raise KernelError(f"rmsnorm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    _elementwise.call("zi_rmsnorm", ptr(x), c_int(dtype_code(x.dtype)), ptr(w), c_int(dtype_code(w.dtype)), ptr(out),
                      c_int(dtype_code(out.dtype)), c_int(rows), c_int(hidden), c_float(eps), stream())


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, eps: float,
                out: torch.Tensor, row_idx: Optional[torch.Tensor] = None, write_residual: bool = True,
                delta_scale: float = 1.0) -> None:
    """``residual (+= delta_scale * delta)``, then ``out = rmsnorm(residual) * w``.  ``residual`` is float32.

    With ``row_idx`` the output row ``r`` is computed from input row ``row_idx[r]`` and the
    residual is left untouched.
    """
    need_cuda(residual, delta, w, out, row_idx)
    if residual.dtype != torch.float32:
        raise KernelError(f"add_rmsnorm: the residual stream is float32, got {residual.dtype}")
    need_contiguous("residual", residual), need_contiguous("w", w), need_contiguous("out", out)
    hidden = residual.shape[1]
    if delta is not None and delta.dim() == 3:
        # partial sums of a product whose K was cut (linear_for_residual): float32 [parts, rows, hidden]
        need_contiguous("delta", delta)
        if delta.dtype != torch.float32 or delta.shape[1:] != residual.shape:
            raise KernelError(f"add_rmsnorm: partial sums {tuple(delta.shape)} {delta.dtype} vs residual {tuple(residual.shape)}")
        if row_idx is not None:
            need_int32("row_idx", row_idx), need_contiguous("row_idx", row_idx)
        rows = row_idx.numel() if row_idx is not None else residual.shape[0]
        if w.numel() != hidden or out.shape != (rows, hidden):
            raise KernelError(f"add_rmsnorm: w {tuple(w.shape)} / out {tuple(out.shape)} do not fit {(rows, hidden)}")
        _elementwise.call("zi_add_rmsnorm_parts", ptr(residual), ptr(delta), c_int(delta.shape[0]),
                          c_ll(delta.shape[1] * hidden), ptr(w), c_int(dtype_code(w.dtype)), ptr(out),
                          c_int(dtype_code(out.dtype)), ptr(row_idx), c_int(rows), c_int(hidden), c_float(eps),
                          c_int(1 if write_residual else 0), c_float(delta_scale), stream())
        return
    if delta is not None:
        need_contiguous("delta", delta)
        if delta.shape != residual.shape:
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} vs residual {tuple(residual.shape)}")
    if row_idx is not None:
        need_int32("row_idx", row_idx), need_contiguous("row_idx", row_idx)
        rows = row_idx.numel()
    else:
        rows = residual.shape[0]
    if w.numel() != hidden or out.shape != (rows, hidden):
        raise KernelError(f"add_rmsnorm: w {tuple(w.shape)} / out {tuple(out.shape)} do not fit {(rows, hidden)}")
    _elementwise.call("zi_add_rmsnorm", ptr(residual), ptr(delta),
                      c_int(dtype_code(delta.dtype) if delta is not None else F32), ptr(w), c_int(dtype_code(w.dtype)),
                      ptr(out), c_int(dtype_code(out.dtype)), ptr(row_idx), c_int(rows), c_int(hidden), c_float(eps),
                      c_int(1 if write_residual else 0), c_float(delta_scale), stream())


ROPE_TABLE_MAX_TOKENS = 64       # steps of at most this many tokens rotate with the step's table of angles


def rope_append(qkv: torch.Tensor, q_out: torch.Tensor, cache: Optional[torch.Tensor], tables: torch.Tensor,
                tok_seg: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, n_heads: int, n_kv_heads: int,
                head_dim: int, page_size: int, page_stride: int, kv_stride: int, write_kv: bool = True,
                cs: Optional[torch.Tensor] = None) -> None:
    """Rotate q (and k) by position and append k, v to the cache pages of each token's request.  ``cs``: the step's
    table of angles (:func:`rope_table` of ``pos`` and ``inv_freq``); steps of at most 64 tokens then read their cosines
    and sines there instead of computing them in every layer."""
    need_cuda(qkv, q_out, cache, tables, tok_seg, pos, inv_freq, cs)
    if cs is not None and (cs.dtype != torch.float32 or cs.shape != (qkv.shape[0], head_dim) or not cs.is_contiguous()):
        raise KernelError(f"rope_append: cs {tuple(cs.shape)} must be contiguous float32 [{qkv.shape[0]}, {head_dim}]")
    need_int32("tables", tables), need_int32("tok_seg", tok_seg), need_int32("pos", pos)
    need_contiguous("q_out", q_out)
    n = qkv.shape[0]
    if qkv.stride(1) != 1 or qkv.shape[1] < (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError(f"rope_append: qkv {tuple(qkv.shape)} does not hold {n_heads}+2*{n_kv_heads} heads of {head_dim}")
    if q_out.dtype != qkv.dtype or (cache is not None and cache.dtype != qkv.dtype):
        raise KernelError("rope_append: qkv, q_out and the cache must share one dtype")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != head_dim // 2:
        raise KernelError("rope_append: inv_freq must be float32 of head_dim/2 entries")
    if write_kv and cache is None:
        raise KernelError("rope_append: write_kv needs a cache")
    _elementwise.call("zi_rope_append", ptr(qkv), ptr(q_out), ptr(cache), c_int(dtype_code(qkv.dtype)), ptr(tables),
                      ptr(tok_seg), ptr(pos), ptr(inv_freq), c_int(n), c_int(qkv.stride(0)), c_int(n_heads),
                      c_int(n_kv_heads), c_int(head_dim), c_int(page_size), c_int(tables.shape[1]),
                      c_ll(page_stride), c_ll(kv_stride), c_int(1 if write_kv else 0), ptr(cs), stream())


def rope_table(pos: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> None:
    """``out[n] = cos | sin`` of ``float(pos[n]) * inv_freq`` (float32 ``[n, head_dim]``): a step's angles, made once."""
    need_cuda(pos, inv_freq, out)
    need_int32("pos", pos)
    need_contiguous("out", out)
    if inv_freq.dtype != torch.float32 or out.dtype != torch.float32 or out.shape != (pos.numel(), 2 * inv_freq.numel()):
        raise KernelError(f"rope_table: pos {tuple(pos.shape)}, inv_freq {tuple(inv_freq.shape)}, out {tuple(out.shape)} do not agree")
    _elementwise.call("zi_rope_table", ptr(pos), ptr(inv_freq), ptr(out), c_int(pos.numel()), c_int(2 * inv_freq.numel()), stream())


def can_fuse_rope_product(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], cache: Optional[torch.Tensor]) -> bool:
    """The q/k/v product of a decode step can take rotation and cache append into its epilogue."""
    return (_small_m_ok(x, w, fused="rope") and (bias is None or (bias.dtype == torch.bfloat16 and bias.data_ptr() % 16 == 0))
            and cache is not None and cache.dtype == torch.bfloat16)


def gemm_smallm_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], cs: torch.Tensor, q_out: torch.Tensor,
                     cache: torch.Tensor, tables: torch.Tensor, tok_seg: torch.Tensor, pos: torch.Tensor, n_heads: int,
                     n_kv_heads: int, head_dim: int, page_size: int, page_stride: int, kv_stride: int) -> None:
    """``x @ w.T + bias`` for the stacked q/k/v weight of at most 16 tokens, rotated by position (``cs`` from
    :func:`rope_table`), q written to ``q_out`` and k, v appended to the cache pages of each token's request."""
    need_cuda(x, w, bias, cs, q_out, cache, tables, tok_seg, pos)
    need_int32("tables", tables), need_int32("tok_seg", tok_seg), need_int32("pos", pos)
    need_contiguous("q_out", q_out), need_contiguous("cs", cs)
    m, k = x.shape
    if w.shape != ((n_heads + 2 * n_kv_heads) * head_dim, k) or q_out.numel() != m * n_heads * head_dim or cs.shape != (m, head_dim):
        raise KernelError(f"gemm_smallm_rope: x {tuple(x.shape)}, w {tuple(w.shape)}, q_out {tuple(q_out.shape)}, cs {tuple(cs.shape)} do not agree")
    if not can_fuse_rope_product(x, w, bias, cache) or q_out.dtype != torch.bfloat16 or cs.dtype != torch.float32:
        raise KernelError("gemm_smallm_rope: bfloat16 operands, at most 16 rows, K a multiple of 32, float32 angles")
    _gemm_smallm.call("zi_gemm_smallm_rope", ptr(x), ptr(w), ptr(bias), ptr(cs), ptr(q_out), ptr(cache), ptr(tables), ptr(tok_seg),
                      ptr(pos), c_int(m), c_int(k), c_ll(x.stride(0)), c_ll(w.stride(0)), c_int(n_heads), c_int(n_kv_heads),
                      c_int(head_dim), c_int(page_size), c_int(tables.shape[1]), c_ll(page_stride), c_ll(kv_stride), stream())


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    need_cuda(gate_up, out)
    need_contiguous("gate_up", gate_up), need_contiguous("out", out)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError(f"silu_mul: gate_up {tuple(gate_up.shape)} vs out {tuple(out.shape)}")
    _elementwise.call("zi_silu_mul", ptr(gate_up), ptr(out), c_int(dtype_code(out.dtype)), c_int(rows),
                      c_int(two_i // 2), stream())


def add(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """``out = a + b`` elementwise (float32 or bfloat16 each), added in float32 with one rounding."""
    need_cuda(a, b, out)
    need_contiguous("a", a), need_contiguous("b", b), need_contiguous("out", out)
    if a.shape != b.shape or a.shape != out.shape:
        raise KernelError(f"add: shapes {tuple(a.shape)}, {tuple(b.shape)}, {tuple(out.shape)} differ")
    _elementwise.call("zi_add", ptr(a), c_int(dtype_code(a.dtype)), ptr(b), c_int(dtype_code(b.dtype)), ptr(out),
                      c_int(dtype_code(out.dtype)), c_ll(a.numel()), stream())


def cast(x: torch.Tensor, out: torch.Tensor) -> None:
    need_cuda(x, out)
    need_contiguous("x", x), need_contiguous("out", out)
    if x.numel() != out.numel():
        raise KernelError("cast: sizes differ")
    _elementwise.call("zi_cast", ptr(x), c_int(dtype_code(x.dtype)), ptr(out), c_int(dtype_code(out.dtype)),
                      c_ll(x.numel()), stream())


def gemm_nt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out = a @ w.T + bias`` on the SIMT cores: float32 FMA chains in rising k, any operand types."""
    need_cuda(a, w, bias, out)
    if a.dim() != 2 or w.dim() != 2 or out.dim() != 2:
        raise KernelError("gemm_nt: operands must be matrices")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n) or (bias is not None and bias.numel() != n):
        raise KernelError(f"gemm_nt: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_nt: rows must be contiguous")
    _gemm_simt.call("zi_gemm_nt", ptr(a), c_int(dtype_code(a.dtype)), ptr(w), c_int(dtype_code(w.dtype)), ptr(bias),
                    c_int(dtype_code(bias.dtype) if bias is not None else F32), ptr(out),
                    c_int(dtype_code(out.dtype)), c_int(m), c_int(n), c_int(k), c_ll(a.stride(0)), c_ll(w.stride(0)),
                    c_ll(out.stride(0)), stream())


# 9 to 16 rows on the weight-streaming kernel (two tiles of eight rows).  It reads the activations once per tile
# and runs three blocks to an SM instead of four, and timed back to back in a graph against the library (plus the
# kernel its epilogue would save) it wins only in these cases (us at 9 to 16 rows, streaming kernel / library):
#   K cut at least three ways, up to 16 M elements      1.5B-class down 9.5-10.2 / 13.6  (7B-class output, cut in two: 13.7 / 8.2;
#                                                       7B-class down 45 / 30; 1.5B-class output, not cut: 5.4 / 4.7)
#   q/k/v with rotation and append, up to 8 M elements  1.5B-class 5.6 / 5.0 + the rotation kernel  (7B-class 15.0 / 8.7 + it)
#   gate/up with the activation: never                  1.5B-class 17.6-18.6 / 13.5 with the activation kernel, 7B-class 58 / 49
SMALL_M_WIDE_ELEMENTS = 16 << 20
SMALL_M_WIDE_ROPE_ELEMENTS = 8 << 20
SMALL_M_WIDE_MIN_KSPLIT = 3
_ksplit_cache: Dict = {}


def _ksplit(n: int, k: int) -> int:
    key = (n, k)
    if key not in _ksplit_cache:
        _ksplit_cache[key] = int(_gemm_smallm.lib.zi_gemm_smallm_ksplit(c_int(n), c_int(k), c_int(0)))
    return _ksplit_cache[key]


def _small_m_ok(x: torch.Tensor, w: torch.Tensor, fused: Optional[str] = None) -> bool:
    """The weight-streaming kernel takes this product.  Up to 8 rows it is the fastest form measured for every
    shape tried (1.5B- to 32B-class layers, at or above the library's rate).  With 9 to 16 rows it keeps what the
    table above says; ``fused``: ``"rope"`` (rotation and cache append in its epilogue), ``"silu"`` (activation)."""
    if x.shape[0] > 8:
        elements = w.shape[0] * w.shape[1]
        if fused == "silu":
            return False
        if fused == "rope":
            if elements > SMALL_M_WIDE_ROPE_ELEMENTS:
                return False
        elif elements > SMALL_M_WIDE_ELEMENTS or x.shape[1] % 32 != 0 or _ksplit(w.shape[0], w.shape[1]) < SMALL_M_WIDE_MIN_KSPLIT:
            return False
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= SMALL_M_ROWS
            and x.shape[1] % 32 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_smallm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                silu_mul: bool = False, gated: Optional[tuple] = None, relu2: bool = False) -> None:
    """``out = x @ w.T + bias`` for at most 16 rows of ``x``: weights stream once from memory into the
    tensor cores.  ``silu_mul``: ``w`` is ``[2*I, K]`` (gate rows, then up rows) and ``out[m, j] =
    up * gate / (1 + exp(-gate))``.  ``gated = (limit, slope, up_offset)``: the same stacked weight with the clamped,
    sigmoid-gated product of :func:`gated_clamp_mul` in the epilogue.  ``relu2``: ``out = max(x @ w.T, 0)^2``."""
    silu_mul = silu_mul or gated is not None
    kind = 2 if gated is not None else (3 if relu2 else 0)
    limit, slope, up_offset = gated if gated is not None else (0.0, 0.0, 0.0)
    need_cuda(x, w, bias, out)
    m, k = x.shape
    n = w.shape[0] // 2 if silu_mul else w.shape[0]
    if w.shape[1] != k or out.shape != (m, n) or out.stride(1) != 1:
        raise KernelError(f"gemm_smallm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (bias is not None and bias.dtype != torch.bfloat16):
        raise KernelError("gemm_smallm: bfloat16 operands only")
    part, counters = _smallm_scratch(x.device, n, k, silu_mul)
    _gemm_smallm.call("zi_gemm_smallm", ptr(x), ptr(w), ptr(bias), ptr(out), c_int(dtype_code(out.dtype)), ptr(part),
                      ptr(counters), c_int(m), c_int(n), c_int(k), c_ll(x.stride(0)), c_ll(w.stride(0)),
                      c_ll(out.stride(0)), c_int(1 if silu_mul else 0), c_int(kind), c_float(limit), c_float(slope),
                      c_float(up_offset), stream())


_scratch = {}


def _smallm_scratch(device, n: int, k: int, silu_mul: bool):
    """Scratch of the split-K decode product: partial sums and arrival counters.  Allocated once per device and
    grown on demand; the counters start at zero and every launch leaves them at zero.  One stream at a time."""
    lib = _gemm_smallm.lib
    lib.zi_gemm_smallm_part_floats.restype = c_ll
    need = lib.zi_gemm_smallm_part_floats(c_int(n), c_int(k), c_int(1 if silu_mul else 0))
    if need == 0:
        return None, None
    key = ("smallm", device)
    if key not in _scratch:
        # K is only split while there are fewer than 296 column tiles (N < 4736), at most 8 ways, 16 rows
        _scratch[key] = (torch.empty(8 * 16 * 4736, dtype=torch.float32, device=device),
                         torch.zeros(512, dtype=torch.int32, device=device))
    part, counters = _scratch[key]
    if part.numel() < need:
        raise KernelError(f"gemm_smallm: scratch of {part.numel()} floats is too small for N={n}, K={k}")
    return part, counters


_retired: list = []


def _grown_scratch(key, floats: int, device) -> torch.Tensor:
    """A float32 scratch buffer of at least ``floats`` entries for ``key``, grown on demand.  A CUDA graph captured
    earlier has the old buffer's address baked in and goes on writing there when it is replayed, so a buffer that is
    outgrown is never given back to the allocator: it is kept (``_retired``) for the life of the process.  Growth
    at least doubles the size, so all retired buffers together stay smaller than the live one."""
    cur = _scratch.get(key)
    if cur is None or cur.numel() < floats:
        if cur is not None:
            _retired.append(cur)
            floats = max(floats, 2 * cur.numel())
        cur = _scratch[key] = torch.empty(floats, dtype=torch.float32, device=device)
    return cur


def _tc_status(device) -> torch.Tensor:
    key = ("tc_status", device)
    if key not in _scratch:
        _scratch[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _scratch[key]


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                 swapped: Optional[bool] = None) -> None:
    """``out = x @ w.T + bias`` on the tcgen05 tensor cores (TMA-fed, accumulator in TMEM), bfloat16 operands.

    ``swapped`` puts the weights on the 128-row side of the MMA and up to 256 rows of ``x`` on the narrow side
    (decode); by default it is chosen by the number of rows.  A bounded wait that runs out inside the kernel is
    reported by :func:`tcgen05_status`.
    """
    need_cuda(x, w, bias, out)
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n) or out.stride(1) != 1 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm_tcgen05: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (bias is not None and bias.dtype != torch.bfloat16):
        raise KernelError("gemm_tcgen05: bfloat16 operands only")
    if swapped is None:
        swapped = m <= 64
    _gemm_tcgen05.call("zi_gemm_tcgen05", ptr(x), ptr(w), ptr(bias), ptr(out), c_int(dtype_code(out.dtype)),
                       ptr(_tc_status(x.device)), c_int(m), c_int(n), c_int(k), c_ll(x.stride(0)), c_ll(w.stride(0)),
                       c_ll(out.stride(0)), c_int(1 if swapped else 0), stream())


_sm_count: Dict = {}


def _num_sms(device) -> int:
    if device not in _sm_count:
        _sm_count[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[device]


def gemm_tcgen05_tiles(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                       silu_mul: bool = False, tile_width: int = 0, pairs: Optional[bool] = None,
                       gated: Optional[tuple] = None, relu2: bool = False) -> None:
    """``out = x @ w.T + bias`` for many rows: one persistent CTA per SM walks 128-row tiles, the accumulator
    double-buffered in TMEM so that the epilogue of a tile overlaps the products of the next.

    With ``silu_mul`` the weight is ``[gate; up]`` stacked (``[2 * n, k]``) and ``out[m, n] = silu(x.gate^T) *
    (x.up^T)``; neither half is written to memory.  ``tile_width`` (accumulator columns per tile) is chosen by
    the call when 0.  ``pairs``: two SMs share a 256-row tile and each loads only half of its weight rows
    (``cta_group::2``); the default for more than 128 rows.  ``gated = (limit, slope, up_offset)``: the stacked weight
    with the clamped, sigmoid-gated product of :func:`gated_clamp_mul` in the epilogue; ``relu2``: ``out = max(x @ w.T,
    0)^2``.
    """
    need_cuda(x, w, bias, out)
    silu_mul = silu_mul or gated is not None
    epilogue = 2 if gated is not None else (3 if relu2 else (1 if silu_mul else 0))
    limit, slope, up_offset = gated if gated is not None else (0.0, 0.0, 0.0)
    m, k = x.shape
    n = out.shape[1]
    if w.shape != ((2 * n if silu_mul else n), k) or out.shape[0] != m or out.stride(1) != 1 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm_tcgen05_tiles: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (bias is not None and bias.dtype != torch.bfloat16):
        raise KernelError("gemm_tcgen05_tiles: bfloat16 operands only")
    if pairs is None:
        pairs = m > 128
    if pairs:
        _gemm_tcgen05.call("zi_gemm_tcgen05_pairs", ptr(x), ptr(w), ptr(bias), ptr(out), c_int(dtype_code(out.dtype)),
                           ptr(_tc_status(x.device)), c_int(m), c_int(n), c_int(k), c_ll(x.stride(0)), c_ll(w.stride(0)),
                           c_ll(out.stride(0)), c_int(epilogue), c_int(tile_width), c_float(limit), c_float(slope),
                           c_float(up_offset), stream())
        return
    _gemm_tcgen05.call("zi_gemm_tcgen05_tiles", ptr(x), ptr(w), ptr(bias), ptr(out), c_int(dtype_code(out.dtype)),
                       ptr(_tc_status(x.device)), c_int(m), c_int(n), c_int(k), c_ll(x.stride(0)), c_ll(w.stride(0)),
                       c_ll(out.stride(0)), c_int(epilogue), c_int(tile_width), c_int(_num_sms(x.device)), c_float(limit),
                       c_float(slope), c_float(up_offset), stream())


def status_word(device) -> torch.Tensor:
    """The device word (int32 ``[1]``) in which the kernels with bounded waits report one that ran out; 0 = fine."""
    return _tc_status(torch.device(device))


def tcgen05_status(device) -> int:
    """0, or the code of the role whose bounded wait ran out (1 producer, 2 MMA issuer, 3 epilogue); resets it."""
    st = _tc_status(torch.device(device))
    v = int(st.item())
    if v:
        st.zero_()
    return v


TC_PLAIN_PRODUCTS = False        # plain bfloat16 products of many rows on the tcgen05 kernel instead of the library
TC_MIN_ROWS = 1024               # ... from this many rows, where switched on
TC_FUSED_MIN_ROWS = 128          # ... and a gate/up product with the activation in its epilogue
TC_FUSED_MIN_ROWS_LARGE = 32     # ... already from this many rows where the stacked weight has at least
TC_FUSED_LARGE_ELEMENTS = 96 << 20   # ... this many elements (7B-class layers and up: see linear_silu_mul)
_tc_launched: Dict = {}


def _tc_ok(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and (bias is None or bias.dtype == torch.bfloat16)
            and out.dtype in (torch.bfloat16, torch.float32) and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def raise_if_tcgen05_failed(device) -> None:
    """After a step that launched tcgen05 products: synchronise and fail loudly if a bounded wait ran out."""
    device = torch.device(device)
    if _tc_launched.pop(device, False):
        code = tcgen05_status(device)
        if code:
            raise KernelError(f"gemm_tcgen05: a bounded wait ran out inside the kernel (role {code}); the step's output is not valid")


def linear_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out = silu(x @ gate.T + b_gate) * (x @ up.T + b_up)`` with ``w_gate_up = [gate; up]`` stacked.

    bfloat16 without bias: the activation runs in the product's epilogue (weight-streaming kernel up to 16 rows,
    tcgen05 kernel from ``TC_FUSED_MIN_ROWS``), so neither half reaches memory.  Otherwise: product, then the
    elementwise kernel.  Between 17 and 127 rows both ways are bound by streaming the weight; timed back to back in a
    graph the tcgen05 kernel is ahead from 32 rows on 7B-class layers (hidden 3,584, intermediate 18,944: 47.4
    against 51.8 us at 64 rows, 48.2 against 56.3 at 127) and level or behind on 1.5B-class layers (15.3 against 14.8
    us at 64 rows), so it takes those rows only for stacked weights of ``TC_FUSED_LARGE_ELEMENTS`` elements or more.
    """
    need_cuda(x, w_gate_up, bias, out)
    if bias is None and _small_m_ok(x, w_gate_up, fused="silu"):
        gemm_smallm(x, w_gate_up, None, out, silu_mul=True)
        return
    min_rows = TC_FUSED_MIN_ROWS_LARGE if w_gate_up.shape[0] * w_gate_up.shape[1] >= TC_FUSED_LARGE_ELEMENTS else TC_FUSED_MIN_ROWS
    if bias is None and x.shape[0] >= min_rows and out.dtype == torch.bfloat16 and _tc_ok(x, w_gate_up, None, out):
        gemm_tcgen05_tiles(x, w_gate_up, None, out, silu_mul=True)
        _tc_launched[x.device] = True
        return
    gate_up = torch.empty((x.shape[0], w_gate_up.shape[0]), dtype=out.dtype, device=x.device)
    linear(x, w_gate_up, bias, gate_up)
    silu_mul(gate_up, out)


def linear_gated_clamp_mul(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, limit: float, slope: float,
                           up_offset: float) -> None:
    """``out = g * sigmoid(slope * g) * (u + up_offset)`` with ``g = min(x @ gate.T, limit)``, ``u = clamp(x @ up.T,
    -limit, limit)`` and ``w_gate_up = [gate; up]`` stacked (``limit <= 0``: no clamps).  Where :func:`linear_silu_mul`
    runs its activation in the product's epilogue this one does too, by the same rules; otherwise product, then
    :func:`gated_clamp_mul`."""
    need_cuda(x, w_gate_up, out)
    gated = (float(limit), float(slope), float(up_offset))
    if _small_m_ok(x, w_gate_up, fused="silu"):
        gemm_smallm(x, w_gate_up, None, out, gated=gated)
        return
    min_rows = TC_FUSED_MIN_ROWS_LARGE if w_gate_up.shape[0] * w_gate_up.shape[1] >= TC_FUSED_LARGE_ELEMENTS else TC_FUSED_MIN_ROWS
    if x.shape[0] >= min_rows and out.dtype == torch.bfloat16 and _tc_ok(x, w_gate_up, None, out):
        gemm_tcgen05_tiles(x, w_gate_up, None, out, gated=gated)
        _tc_launched[x.device] = True
        return
    gate_up = torch.empty((x.shape[0], w_gate_up.shape[0]), dtype=out.dtype, device=x.device)
    linear(x, w_gate_up, None, gate_up)
    gated_clamp_mul(gate_up, out, *gated)


def linear_relu2(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out = max(x @ w.T, 0)^2``: the activation in the product's epilogue on the weight-streaming kernel (up to 16
    rows) and on the tcgen05 kernel (from ``TC_FUSED_MIN_ROWS`` rows); otherwise product, then :func:`relu2`."""
    need_cuda(x, w, out)
    if _small_m_ok(x, w) and out.stride(1) == 1:
        gemm_smallm(x, w, None, out, relu2=True)
        return
    if x.shape[0] >= TC_FUSED_MIN_ROWS and out.dtype == torch.bfloat16 and _tc_ok(x, w, None, out):
        gemm_tcgen05_tiles(x, w, None, out, relu2=True)
        _tc_launched[x.device] = True
        return
    linear(x, w, None, out)
    relu2(out, out)


# A product whose result goes straight into the residual stream (output and down projections), with 17 to 256 rows:
# the library's kernels for these few rows leave most of the GPU idle when the output is narrow (1.5B-class down
# product, 64 rows: 13.8 us = 2.0 TB/s).  As a batched product over RESIDUAL_K_PARTS ranges of K with float32 results
# it takes 7.8 us (7B-class: 30.8 -> 25.2 us; 0.5B-class sizes 8.9 -> 5.2; the 1.5B-class output projection 4.9 ->
# 3.8), and the norm that folds the branch into
# the stream adds the ranges on its way (add_rmsnorm), so no kernel is added.  Measured back to back in a graph;
# from 257 rows the library's own choice is as good, and at 32B-class sizes (141 M elements) nothing is gained.
RESIDUAL_K_PARTS = 4
RESIDUAL_PARTS_MIN_ROWS = 17
RESIDUAL_PARTS_MIN_K = 1024
# (most rows, most weight elements) for products with K >= 2 N (down: 1.5B-class 14.4 -> 9.7 us still at 256 rows,
# 7B-class 39.6 -> 35.6) and for the others (output projection: 7B-class 8.5 -> 8.0 us at 128 rows, but 8.8 -> 10.1 at
# 192; 32B-class, 26 M elements, 12.2 -> 13.9 at 128)
RESIDUAL_PARTS_LONG_K = (256, 80 << 20)
RESIDUAL_PARTS_SQUARE = (128, 16 << 20)


def linear_for_residual(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """``x @ w.T + bias`` for a result that the next norm adds to the residual stream: either the product itself
    (``[rows, N]`` of x's type) or, where that is faster, float32 partial sums ``[parts, rows, N]`` over ranges of
    K, which :func:`add_rmsnorm` adds in order and rounds as the product would have been rounded."""
    rows, k = x.shape
    n = w.shape[0]
    max_rows, max_elements = RESIDUAL_PARTS_LONG_K if k >= 2 * n else RESIDUAL_PARTS_SQUARE
    if (bias is None and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and RESIDUAL_PARTS_MIN_ROWS <= rows <= max_rows and k >= RESIDUAL_PARTS_MIN_K
            and n * k <= max_elements and k % (8 * RESIDUAL_K_PARTS) == 0 and n % 8 == 0
            and x.is_contiguous() and w.is_contiguous()):
        need_cuda(x, w)
        p = RESIDUAL_K_PARTS
        parts = torch.empty((p, rows, n), dtype=torch.float32, device=x.device)
        torch.bmm(x.view(rows, p, k // p).permute(1, 0, 2), w.view(n, p, k // p).permute(1, 2, 0),
                  out_dtype=torch.float32, out=parts)
        return parts
    out = torch.empty((rows, n), dtype=x.dtype, device=x.device)
    linear(x, w, bias, out)
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out = x @ w.T + bias``; picks the kernel by operand types and the number of rows.

    * any float32 operand: the SIMT kernel (true 32-bit arithmetic);
    * bfloat16 x bfloat16 with at most 16 rows (decode steps): the weight-streaming tensor-core kernel;
    * bfloat16 x bfloat16 otherwise: cuBLAS with float32 accumulation, the library product the
      reference's engine uses as well; the output may be bfloat16 or float32.  With ``TC_PLAIN_PRODUCTS`` set,
      products of ``TC_MIN_ROWS`` rows or more run on the tcgen05 kernel (pairs of SMs) instead.  Timed back to
      back in a graph the library is ahead on plain products (2,048 rows of the 1.5B-class layer: q/k/v 12.0
      against 14.5 us, output 9.6 against 13.7, down 42.1 against 46.5; the whole 2,048-token step 5.39 against
      5.75 ms), so the tcgen05 kernel is kept for the gate/up product, where its SiLU-mul epilogue saves a kernel
      and a round trip of the activations through memory (:func:`linear_silu_mul`).
    """
    need_cuda(x, w, bias, out)
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and (bias is None or bias.dtype == torch.bfloat16):
        if _small_m_ok(x, w) and out.stride(1) == 1:
            gemm_smallm(x, w, bias, out)
            return
        if TC_PLAIN_PRODUCTS and x.shape[0] >= TC_MIN_ROWS and _tc_ok(x, w, bias, out):
            gemm_tcgen05_tiles(x, w, bias, out)
            _tc_launched[x.device] = True
            return
        if out.dtype == torch.bfloat16:
            if bias is not None:
                torch.addmm(bias, x, w.t(), out=out)
            else:
                torch.mm(x, w.t(), out=out)
        else:
            res = torch.mm(x, w.t(), out_dtype=torch.float32)
            if bias is not None:
                res += bias.float()
            out.copy_(res)
        return
    gemm_nt(x, w, bias, out)


def paged_attention(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, tables: torch.Tensor,
                    tok_seg: torch.Tensor, pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                    page_size: int, page_stride: int, kv_stride: int, window: Optional[int], scale: float,
                    sinks: Optional[torch.Tensor] = None, softcap: Optional[float] = None) -> None:
    """Causal attention of each token over its request's cache pages (general kernel).  ``kv_stride`` 0: the cache has
    one plane whose rows are keys and values at once.  ``sinks``: float32, one per query head; ``exp(sinks[h])`` joins
    the softmax's denominator (a term without key and value).  ``softcap`` c: a scaled score s becomes ``c tanh(s / c)``."""
    need_cuda(q, cache, out, tables, tok_seg, pos, sinks)
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != n_heads or not sinks.is_contiguous()):
        raise KernelError(f"paged_attention: sinks must be contiguous float32 with {n_heads} entries")
    need_int32("tables", tables), need_int32("tok_seg", tok_seg), need_int32("pos", pos)
    need_contiguous("q", q), need_contiguous("out", out)
    if q.dtype != cache.dtype or out.dtype != q.dtype:
        raise KernelError("paged_attention: q, cache and out must share one dtype")
    n = q.shape[0]
    _attention_generic.call("zi_paged_attention", ptr(q), ptr(cache), ptr(out), c_int(dtype_code(q.dtype)),
                            ptr(tables), ptr(tok_seg), ptr(pos), c_int(n), c_int(n_heads), c_int(n_kv_heads),
                            c_int(head_dim), c_int(page_size), c_int(tables.shape[1]), c_ll(page_stride),
                            c_ll(kv_stride), c_int(window or 0), c_float(scale), ptr(sinks), c_float(softcap or 0.0), stream())


PREFILL_TILE_ROWS = 128          # query rows per entry of a step's tile list


def _check_sinks(sinks: Optional[torch.Tensor], n_heads: int) -> None:
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != n_heads or not sinks.is_contiguous()):
        raise KernelError(f"attention: sinks must be contiguous float32 with {n_heads} entries")


def decode_attention(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, tables: torch.Tensor,
                     tok_seg: torch.Tensor, pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                     page_size: int, page_stride: int, kv_stride: int, window: Optional[int], scale: float,
                     sinks: Optional[torch.Tensor] = None, softcap: Optional[float] = None) -> None:
    """One query token per request, bfloat16, tensor cores; a cluster of eight thread blocks per
    (request, key/value head) shares the context and merges through distributed shared memory.  ``kv_stride`` 0 and
    ``sinks`` and ``softcap``: as :func:`paged_attention`."""
    need_cuda(q, cache, out, tables, tok_seg, pos, sinks)
    _check_sinks(sinks, n_heads)
    need_int32("tables", tables), need_int32("tok_seg", tok_seg), need_int32("pos", pos)
    need_contiguous("q", q), need_contiguous("out", out)
    n = q.shape[0]
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("decode_attention: bfloat16 only")
    _attention_mma.call("zi_decode_attention", ptr(q), ptr(cache), ptr(out), ptr(tables), ptr(tok_seg), ptr(pos),
                        c_int(n), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size),
                        c_int(tables.shape[1]), c_ll(page_stride), c_ll(kv_stride), c_int(window or 0),
                        c_float(scale), ptr(sinks), c_float(softcap or 0.0), stream())


def decode_attention_split_from() -> int:
    """The number of cached tokens from which :func:`decode_attention_tma` lets several clusters share one request's
    keys and launches the kernel that adds their parts: a step whose ``max_kv_len`` stays below it has neither."""
    return int(_attention_mma.lib.zi_decode_attention_tma_split_from())


def decode_attention_tma(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, tables: torch.Tensor,
                         tok_seg: Optional[torch.Tensor], pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                         page_size: int, page_stride: int, kv_stride: int, window: Optional[int], scale: float,
                         max_kv_len: int = 0, sinks: Optional[torch.Tensor] = None, softcap: Optional[float] = None) -> None:
    """One query token per request, bfloat16: the cluster kernel with 32-key tiles dealt to single warps, each
    fed by TMA through the block table into a ring of its own.  Same arguments as :func:`decode_attention`;
    head_dim 64 or 128, pages of a power of two from 8 to 128 tokens.  ``max_kv_len``: an upper bound of the cached
    tokens of the step's requests; ``tok_seg`` None: token n belongs to row n of ``tables`` (every decode step of the
    engine; the kernel then asks for its first page numbers without waiting for anything).  With few requests and long contexts several clusters then share one request's
    keys and a second kernel adds their parts (0: never).  A bounded wait that runs out is reported by
    :func:`tcgen05_status`."""
    need_cuda(q, cache, out, tables, tok_seg, pos, sinks)
    _check_sinks(sinks, n_heads)
    need_int32("tables", tables), need_int32("pos", pos)
    if tok_seg is not None:
        need_int32("tok_seg", tok_seg)
    need_contiguous("q", q), need_contiguous("out", out)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("decode_attention_tma: bfloat16 only")
    part, part_floats = None, 0
    if max_kv_len > 0:
        lib = _attention_mma.lib
        lib.zi_decode_attention_tma_part_floats.restype = c_ll
        part_floats = int(lib.zi_decode_attention_tma_part_floats(c_int(q.shape[0]), c_int(n_heads), c_int(n_kv_heads),
                                                                   c_int(head_dim), c_int(int(max_kv_len))))
        if part_floats:
            part = _grown_scratch(("decode_parts", q.device), part_floats, q.device)
    _attention_mma.call("zi_decode_attention_tma", ptr(q), ptr(cache), ptr(out), ptr(tables), ptr(tok_seg), ptr(pos),
                        ptr(_tc_status(q.device)), c_int(q.shape[0]), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
                        c_int(page_size), c_int(tables.shape[1]), c_ll(cache.shape[0]), c_ll(page_stride), c_ll(kv_stride),
                        c_int(window or 0), c_float(scale), c_int(int(max_kv_len) if part_floats else 0), ptr(part),
                        c_ll(part_floats), ptr(sinks), c_float(softcap or 0.0), stream())
    _tc_launched[q.device] = True


def prefill_attention(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, tables: torch.Tensor,
                      tiles: torch.Tensor, pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      page_size: int, page_stride: int, kv_stride: int, window: Optional[int], scale: float,
                      sinks: Optional[torch.Tensor] = None, softcap: Optional[float] = None) -> None:
    """Portions of prompts, bfloat16, ``mma.sync`` tensor-core path.  ``tiles`` int32 ``[n_tiles, 3]``: (first token,
    rows <= 128, segment); the positions of a tile's tokens are consecutive.  Takes any page size and windows."""
    need_cuda(q, cache, out, tables, tiles, pos)
    need_int32("tables", tables), need_int32("tiles", tiles), need_int32("pos", pos)
    need_contiguous("q", q), need_contiguous("out", out), need_contiguous("tiles", tiles)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("prefill_attention: bfloat16 only")
    _attention_mma.call("zi_prefill_attention", ptr(q), ptr(cache), ptr(out), ptr(tables), ptr(tiles), ptr(pos),
                        c_int(tiles.shape[0]), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size),
                        c_int(tables.shape[1]), c_ll(page_stride), c_ll(kv_stride), c_int(window or 0),
                        c_float(scale), ptr(sinks), c_float(softcap or 0.0), stream())


def prefill_attention_tcgen05(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, tables: torch.Tensor,
                              tiles: torch.Tensor, pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                              page_size: int, page_stride: int, kv_stride: int, window: Optional[int], scale: float,
                              sinks: Optional[torch.Tensor] = None, softcap: Optional[float] = None) -> None:
    """Portions of prompts, bfloat16, on tcgen05: scores and outputs accumulate in TMEM, K and V pages arrive by
    TMA through the block table.  Same arguments as :func:`prefill_attention`; head_dim 64 or 128, pages of a power
    of two from 8 to 128 tokens.  A bounded wait that runs out is reported by :func:`tcgen05_status`."""
    need_cuda(q, cache, out, tables, tiles, pos)
    need_int32("tables", tables), need_int32("tiles", tiles), need_int32("pos", pos)
    need_contiguous("q", q), need_contiguous("out", out), need_contiguous("tiles", tiles)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("prefill_attention_tcgen05: bfloat16 only")
    _attention_tcgen05.call("zi_prefill_attention_tcgen05", ptr(q), ptr(cache), ptr(out), ptr(tables), ptr(tiles), ptr(pos),
                            ptr(_tc_status(q.device)), c_int(q.shape[0]), c_int(tiles.shape[0]), c_int(n_heads),
                            c_int(n_kv_heads), c_int(head_dim), c_int(page_size), c_int(tables.shape[1]),
                            c_ll(cache.shape[0]), c_ll(page_stride), c_ll(kv_stride), c_int(window or 0), c_float(scale), ptr(sinks),
                            c_float(softcap or 0.0), stream())
    _tc_launched[q.device] = True


def tcgen05_attention_ok(head_dim: int, page_size: int) -> bool:
    return head_dim in (64, 128) and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0


LATENT_TENSOR_CORES = True       # one-plane caches and sinks on the tensor-core attention kernels (False: the general kernel)


def attention(q: torch.Tensor, cache, out: torch.Tensor, ctx, n_heads: int, n_kv_heads: int, head_dim: int,
              window: Optional[int], scale: float, sinks: Optional[torch.Tensor] = None,
              softcap: Optional[float] = None) -> None:
    """Attention of a step's tokens over the cache (``cache`` is a CallCacheView, ``ctx`` a StepContext).

    Picks a kernel by dtype and by the shape of the step; all of them compute the same function.
    bfloat16 with head_dim 64 or 128 runs on the tensor cores: decode-only steps, and the single tokens at the head
    of a mixed step, on the cluster decode kernel, anything else on the tcgen05 prefill kernel (pages of 8..128 tokens) or the ``mma.sync`` prefill kernel (other
    page sizes); float32 and other head sizes on the general kernel.  ``sinks`` (float32, one per query head) and a cache
    with one plane (``cache.kv_stride`` 0, rows that are keys and values at once) are taken by every kernel, and so is
    ``softcap`` (scores through ``c tanh(s / c)``).
    """
    tables = ctx.tables[cache.group]
    if (q.dtype == torch.bfloat16 and head_dim in (64, 128)
            and (LATENT_TENSOR_CORES or (sinks is None and cache.kv_stride != 0))):
        n = q.shape[0]
        if ctx.decode_only and tcgen05_attention_ok(head_dim, cache.page_size):
            # in a step of single tokens, token n is segment n
            decode_attention_tma(q, cache.tensor, out, tables, None, ctx.positions, n_heads, n_kv_heads, head_dim,
                                 cache.page_size, cache.page_stride, cache.kv_stride, window, scale,
                                 max_kv_len=min(ctx.max_kv_len, window) if window else ctx.max_kv_len, sinks=sinks, softcap=softcap)
            return
        if ctx.decode_only:
            decode_attention(q, cache.tensor, out, tables, ctx.tok_seg, ctx.positions, n_heads, n_kv_heads, head_dim,
                             cache.page_size, cache.page_stride, cache.kv_stride, window, scale, sinks=sinks, softcap=softcap)
            return
        tiles = ctx.extras.get("attn_tiles")
        lead = ctx.extras.get("leading_singles", 0) if tiles is not None else 0
        if lead:                                  # decoding requests beside a prompt portion: their own kernel
            if tcgen05_attention_ok(head_dim, cache.page_size):     # the leading single tokens are segments 0 .. lead - 1
                decode_attention_tma(q[:lead], cache.tensor, out[:lead], tables, None, ctx.positions[:lead], n_heads,
                                     n_kv_heads, head_dim, cache.page_size, cache.page_stride, cache.kv_stride, window, scale,
                                     sinks=sinks, softcap=softcap)
            else:
                decode_attention(q[:lead], cache.tensor, out[:lead], tables, ctx.tok_seg[:lead], ctx.positions[:lead], n_heads,
                                 n_kv_heads, head_dim, cache.page_size, cache.page_stride, cache.kv_stride, window, scale,
                                 sinks=sinks, softcap=softcap)
        if tiles is not None and tcgen05_attention_ok(head_dim, cache.page_size):
            prefill_attention_tcgen05(q, cache.tensor, out, tables, tiles, ctx.positions, n_heads, n_kv_heads, head_dim,
                                      cache.page_size, cache.page_stride, cache.kv_stride, window, scale, sinks=sinks, softcap=softcap)
            return
        if tiles is not None:
            prefill_attention(q, cache.tensor, out, tables, tiles, ctx.positions, n_heads, n_kv_heads, head_dim,
                              cache.page_size, cache.page_stride, cache.kv_stride, window, scale, sinks=sinks, softcap=softcap)
            return
    paged_attention(q, cache.tensor, out, tables, ctx.tok_seg, ctx.positions, n_heads, n_kv_heads,
                    head_dim, cache.page_size, cache.page_stride, cache.kv_stride, window, scale, sinks=sinks, softcap=softcap)


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    need_cuda(logits, out)
    need_int32("out", out)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be float32 [rows, vocab] with contiguous rows")
    rows, vocab = logits.shape
    slices = int(_sampling.lib.zi_argmax_slices(c_int(vocab)))
    part = _grown_scratch(("argmax", logits.device), rows * slices * 2, logits.device) if slices > 1 else None
    _sampling.call("zi_argmax", ptr(logits), ptr(out), c_int(rows), c_int(vocab), c_ll(logits.stride(0)), ptr(part), stream())


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, uniform: torch.Tensor) -> None:
    """One token per row; rows with ``temperature <= 0`` are greedy."""
    need_cuda(logits, out, temperature, top_k, top_p, uniform)
    need_int32("out", out), need_int32("top_k", top_k)
    rows = logits.shape[0]
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 [rows, vocab] with contiguous rows")
    for name, t in (("temperature", temperature), ("top_p", top_p), ("uniform", uniform)):
        if t.dtype != torch.float32 or t.numel() != rows:
            raise KernelError(f"sample: {name} must be float32 with one entry per row")
    if top_k.numel() != rows or out.numel() != rows:
        raise KernelError("sample: top_k and out need one entry per row")
    _sampling.call("zi_sample", ptr(logits), ptr(out), ptr(temperature), ptr(top_k), ptr(top_p), ptr(uniform),
                   c_int(rows), c_int(logits.shape[1]), c_ll(logits.stride(0)), stream())


def penalty_rows(logits: torch.Tensor, counts: torch.Tensor, slots: torch.Tensor, penalty: torch.Tensor) -> None:
    """The repetition penalty from a table on the device: row r of ``logits`` (float32 ``[rows, vocab]``) is penalised
    with ``penalty[r]`` once per time that the request in slot ``slots[r]`` has generated a token
    (``counts`` int32 ``[slots, vocab]``); rows with a negative slot or a penalty of 1 are left alone."""
    need_cuda(logits, counts, slots, penalty)
    need_int32("counts", counts), need_int32("slots", slots)
    rows = logits.shape[0]
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("penalty_rows: logits must be float32 [rows, vocab] with contiguous rows")
    if counts.dim() != 2 or counts.shape[1] != logits.shape[1] or counts.stride(1) != 1:
        raise KernelError(f"penalty_rows: counts {tuple(counts.shape)} do not match a vocabulary of {logits.shape[1]}")
    if penalty.dtype != torch.float32 or penalty.numel() != rows or slots.numel() != rows:
        raise KernelError("penalty_rows: slots (int32) and penalty (float32) need one entry per row")
    _sampling.call("zi_penalty_rows", ptr(logits), ptr(counts), ptr(slots), ptr(penalty), c_int(rows), c_int(logits.shape[1]),
                   c_ll(logits.stride(0)), c_ll(counts.stride(0)), stream())


def count_tokens(counts: torch.Tensor, slots: torch.Tensor, tokens: torch.Tensor) -> None:
    """``counts[slots[r], tokens[r]] += 1`` for the rows whose slot is not negative (each slot at most once)."""
    need_cuda(counts, slots, tokens)
    need_int32("counts", counts), need_int32("slots", slots), need_int32("tokens", tokens)
    if counts.dim() != 2 or counts.stride(1) != 1 or slots.numel() != tokens.numel():
        raise KernelError("count_tokens: counts [slots, vocab], one slot and one token per row")
    _sampling.call("zi_count_tokens", ptr(counts), ptr(slots), ptr(tokens), c_int(tokens.numel()), c_int(counts.shape[1]),
                   c_ll(counts.stride(0)), stream())


def count_token_list(counts_row: torch.Tensor, tokens: torch.Tensor) -> None:
    """``counts_row[t] += 1`` for every listed token (a token listed twice counts twice)."""
    need_cuda(counts_row, tokens)
    need_int32("counts_row", counts_row), need_int32("tokens", tokens)
    need_contiguous("counts_row", counts_row)
    _sampling.call("zi_count_token_list", ptr(counts_row), ptr(tokens), c_int(tokens.numel()), c_int(counts_row.numel()), stream())


def advance_decode(ids: torch.Tensor, pos: torch.Tensor, sampled: torch.Tensor, rows: Optional[int] = None) -> None:
    """Hand the chosen tokens to the next decode step: ``ids := sampled``, ``pos += 1`` for the first ``rows`` rows
    (all of ``ids`` by default).  ``pos`` is one position per token, or ``[axes, tokens]`` for a model whose tokens
    carry several position numbers: every axis moves on by one."""
    need_cuda(ids, pos, sampled)
    need_int32("ids", ids), need_int32("pos", pos), need_int32("sampled", sampled)
    n = ids.numel() if rows is None else int(rows)
    axes, per_axis = (pos.shape[0], pos.shape[1]) if pos.dim() == 2 else (1, pos.numel())
    if pos.dim() == 2 and (pos.stride(1) != 1 or (axes > 1 and pos.stride(0) < per_axis)):
        raise KernelError(f"advance_decode: positions {tuple(pos.shape)} with strides {pos.stride()}")
    if n > min(ids.numel(), per_axis, sampled.numel()):
        raise KernelError(f"advance_decode: {n} rows of ids {ids.numel()}, pos {per_axis}, sampled {sampled.numel()}")
    _sampling.call("zi_advance_decode", ptr(ids), ptr(pos), ptr(sampled), c_int(n), c_int(axes),
                   c_ll(pos.stride(0) if pos.dim() == 2 else 0), stream())


def repetition_penalty(logits_row: torch.Tensor, tokens: torch.Tensor, penalty: float) -> None:
    need_cuda(logits_row, tokens)
    need_int32("tokens", tokens)
    if logits_row.dtype != torch.float32 or logits_row.dim() != 1 or not logits_row.is_contiguous():
        raise KernelError("repetition_penalty: one contiguous float32 row")
    _sampling.call("zi_repetition_penalty", ptr(logits_row), ptr(tokens), c_int(tokens.numel()),
                   c_int(logits_row.numel()), c_float(penalty), stream())


# ---- row-wise kernels of csrc/rowwise.cu ---------------------------------------------------------------------------
def embedding_positions(table: torch.Tensor, pos_table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor,
                        out: torch.Tensor) -> None:
    """``out[n] = table[ids[n]] + pos_table[positions[n]]``, added in float32."""
    need_cuda(table, pos_table, ids, positions, out)
    need_int32("ids", ids), need_int32("positions", positions)
    need_contiguous("table", table), need_contiguous("pos_table", pos_table), need_contiguous("out", out)
    need_contiguous("ids", ids), need_contiguous("positions", positions)
    n, hidden = ids.numel(), table.shape[1]
    if out.shape != (n, hidden) or pos_table.shape[1] != hidden or pos_table.dtype != table.dtype or positions.numel() != n:
        raise KernelError(f"embedding_positions: table {tuple(table.shape)}, pos_table {tuple(pos_table.shape)}, "
                          f"out {tuple(out.shape)} do not agree")
    _rowwise.call("zi_embedding_pos", ptr(table), ptr(pos_table), c_int(dtype_code(table.dtype)), ptr(ids), ptr(positions),
                  ptr(out), c_int(dtype_code(out.dtype)), c_int(n), c_int(hidden), c_int(table.shape[0]),
                  c_int(pos_table.shape[0]), stream())


def softcap(logits: torch.Tensor, cap: float) -> None:
    """In place on float32: ``x = cap * tanh(x / cap)``."""
    need_cuda(logits)
    need_contiguous("logits", logits)
    if logits.dtype != torch.float32:
        raise KernelError("softcap: float32 only")
    _rowwise.call("zi_softcap", ptr(logits), c_ll(logits.numel()), c_float(cap), stream())


def relu2(x: torch.Tensor, out: torch.Tensor) -> None:
    """``out = max(x, 0)^2``."""
    need_cuda(x, out)
    need_contiguous("x", x), need_contiguous("out", out)
    if x.shape != out.shape or x.dtype != out.dtype:
        raise KernelError("relu2: x and out must agree")
    _rowwise.call("zi_relu2", ptr(x), ptr(out), c_int(dtype_code(x.dtype)), c_ll(x.numel()), stream())


def gated_clamp_mul(gate_up: torch.Tensor, out: torch.Tensor, limit: float, slope: float, up_offset: float) -> None:
    """``gate_up`` is ``[rows, 2 * I]`` (gate columns, then up columns): ``g = min(gate, limit)``, ``u = clamp(up,
    -limit, limit)``, ``out = g * sigmoid(slope * g) * (u + up_offset)``.  ``limit <= 0``: no clamping."""
    need_cuda(gate_up, out)
    need_contiguous("gate_up", gate_up), need_contiguous("out", out)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError(f"gated_clamp_mul: gate_up {tuple(gate_up.shape)} vs out {tuple(out.shape)}")
    _rowwise.call("zi_gated_clamp_mul", ptr(gate_up), ptr(out), c_int(dtype_code(out.dtype)), c_int(rows), c_int(two_i // 2),
                  c_float(limit), c_float(slope), c_float(up_offset), stream())


def rmsnorm_append(x: torch.Tensor, w: torch.Tensor, eps: float, cache: torch.Tensor, tables: torch.Tensor,
                   tok_seg: Optional[torch.Tensor], pos: torch.Tensor, page_size: int, page_stride: int) -> None:
    """RMSNorm (plain weight) of every row of ``x`` (``[tokens, width]``, rows may be strided), written as the row of
    its token in a paged cache with one plane and one head: page ``tables[tok_seg[n], pos[n] // page_size]``, offset
    ``pos[n] % page_size``.  ``tok_seg`` None: token n is segment n."""
    need_cuda(x, w, cache, tables, tok_seg, pos)
    need_int32("tables", tables), need_int32("pos", pos)
    if tok_seg is not None:
        need_int32("tok_seg", tok_seg)
    need_contiguous("w", w)
    n, width = x.shape
    if x.stride(1) != 1 or w.numel() != width:
        raise KernelError(f"rmsnorm_append: x {tuple(x.shape)} strides {x.stride()}, w {tuple(w.shape)}")
    _rowwise.call("zi_rmsnorm_append", ptr(x), c_int(dtype_code(x.dtype)), c_ll(x.stride(0)), ptr(w), c_int(dtype_code(w.dtype)),
                  c_float(eps), ptr(cache), c_int(dtype_code(cache.dtype)), ptr(tables), ptr(tok_seg), ptr(pos), c_int(n),
                  c_int(width), c_int(page_size), c_int(tables.shape[1]), c_ll(page_stride), stream())


def linear_per_head(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """One product per head: ``out[n, h, :] = x[n, h, :] @ w[h].T`` with ``w [heads, N, K]`` and ``out [tokens, heads,
    N]`` contiguous; ``x`` is ``[tokens, heads * K]`` (rows may be strided: a slice of a wider product's output) or
    ``[tokens, heads, K]``.  bfloat16: one batched library product over strided views (float32 sums); any float32
    operand: the SIMT kernel, one launch."""
    need_cuda(x, w, out)
    need_contiguous("w", w), need_contiguous("out", out)
    heads, nn, k = w.shape
    n = x.shape[0]
    if x.dim() == 3:
        need_contiguous("x", x)
        x = x.view(n, heads * k)
    if x.shape != (n, heads * k) or x.stride(1) != 1 or out.shape != (n, heads, nn):
        raise KernelError(f"linear_per_head: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.bfloat16:
        xh = x.as_strided((heads, n, k), (k, x.stride(0), 1))
        torch.bmm(xh, w.transpose(1, 2), out=out.transpose(0, 1))
        return
    _gemm_simt.call("zi_gemm_nt_batched", ptr(x), c_int(dtype_code(x.dtype)), ptr(w), c_int(dtype_code(w.dtype)), ptr(out),
                    c_int(dtype_code(out.dtype)), c_int(heads), c_int(n), c_int(nn), c_int(k), c_ll(x.stride(0)), c_ll(k),
                    c_ll(heads * nn), c_ll(k), c_ll(nn * k), c_ll(nn), stream())


# ---- routed feed-forward, csrc/moe.cu ------------------------------------------------------------------------------
ROUTER_SCORES = {"softmax_chosen": 0, "sigmoid": 1, "softmax_all": 2}


def _check_choice_bias(choice_bias: Optional[torch.Tensor], experts: int, score: str) -> None:
    if choice_bias is not None and (score != "softmax_all" or choice_bias.dtype != torch.float32 or choice_bias.numel() != experts
                                    or not choice_bias.is_contiguous()):
        raise KernelError(f"route: choice_bias must be contiguous float32 with {experts} entries and goes with score='softmax_all'")


def route_topk(logits: torch.Tensor, top: int, idx: torch.Tensor, wts: torch.Tensor, score: str = "softmax_chosen",
               choice_bias: Optional[torch.Tensor] = None) -> None:
    """Per row of float32 ``logits [tokens, experts]``: the ``top`` largest (lowest index wins a tie) into ``idx`` (int32
    ``[tokens, top]``, largest first) and their weights into ``wts`` (float32): the softmax over those alone
    (``score="softmax_chosen"``), or each one's own ``sigmoid(logit)``, not renormalised (``"sigmoid"``).
    ``score="softmax_all"``: every expert's score is its share of the softmax over all experts; the ``top`` largest of
    ``score + choice_bias`` are chosen (``choice_bias`` float32 per expert, or None) and their weights are the scores
    themselves, without the bias and not renormalised."""
    need_cuda(logits, idx, wts, choice_bias)
    _check_choice_bias(choice_bias, logits.shape[1], score)
    need_int32("idx", idx)
    need_contiguous("logits", logits), need_contiguous("idx", idx), need_contiguous("wts", wts)
    n, e = logits.shape
    if logits.dtype != torch.float32 or wts.dtype != torch.float32 or idx.shape != (n, top) or wts.shape != (n, top):
        raise KernelError(f"route_topk: logits {tuple(logits.shape)} {logits.dtype}, idx {tuple(idx.shape)}, wts {tuple(wts.shape)}")
    _moe.call("zi_route_topk", ptr(logits), c_int(n), c_int(e), c_int(top), ptr(idx), ptr(wts), c_int(ROUTER_SCORES[score]),
              ptr(choice_bias), stream())


def route(x: torch.Tensor, w_router: torch.Tensor, bias: Optional[torch.Tensor], top: int, idx: torch.Tensor,
          wts: torch.Tensor, logits: Optional[torch.Tensor] = None, score: str = "softmax_chosen",
          choice_bias: Optional[torch.Tensor] = None) -> None:
    """The router in one kernel: float32 logits ``x @ w_router.T + bias`` (operands of any storage type, float32 sums in
    a fixed order), then as :func:`route_topk` (``score`` and ``choice_bias`` as there).  ``logits``: optional float32
    ``[tokens, experts]`` to receive them."""
    need_cuda(x, w_router, bias, idx, wts, logits, choice_bias)
    _check_choice_bias(choice_bias, w_router.shape[0], score)
    need_int32("idx", idx)
    need_contiguous("w_router", w_router), need_contiguous("idx", idx), need_contiguous("wts", wts)
    n, k = x.shape
    e = w_router.shape[0]
    if (x.stride(1) != 1 or w_router.shape != (e, k) or idx.shape != (n, top) or wts.shape != (n, top) or wts.dtype != torch.float32
            or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != e or not bias.is_contiguous()))
            or (logits is not None and (logits.dtype != torch.float32 or logits.shape != (n, e) or not logits.is_contiguous()))):
        raise KernelError(f"route: x {tuple(x.shape)}, w_router {tuple(w_router.shape)}, idx {tuple(idx.shape)}, wts {tuple(wts.shape)}")
    _moe.call("zi_route", ptr(x), c_int(dtype_code(x.dtype)), c_ll(x.stride(0)), ptr(w_router), c_int(dtype_code(w_router.dtype)),
              ptr(bias), c_int(n), c_int(k), c_int(e), c_int(top), ptr(idx), ptr(wts), ptr(logits), c_int(ROUTER_SCORES[score]),
              ptr(choice_bias), stream())


def moe_group(idx: torch.Tensor, n_experts: int, offsets: torch.Tensor, row_pair: torch.Tensor, pair_row: torch.Tensor) -> None:
    """Group the (token, choice) pairs of ``idx`` (int32 ``[tokens, top]``) by expert: ``offsets`` (int32
    ``[experts + 1]``) bounds each expert's sorted rows, ``row_pair[r]`` is the pair at sorted row r and ``pair_row`` its
    inverse."""
    need_cuda(idx, offsets, row_pair, pair_row)
    for name, t in (("idx", idx), ("offsets", offsets), ("row_pair", row_pair), ("pair_row", pair_row)):
        need_int32(name, t), need_contiguous(name, t)
    pairs = idx.numel()
    if offsets.numel() != n_experts + 1 or row_pair.numel() != pairs or pair_row.numel() != pairs:
        raise KernelError("moe_group: offsets [experts + 1], row_pair and pair_row one entry per pair")
    _moe.call("zi_moe_group", ptr(idx), c_int(pairs), c_int(n_experts), ptr(offsets), ptr(row_pair), ptr(pair_row), stream())


def moe_group_padded(idx: torch.Tensor, n_experts: int, pad: int, starts: torch.Tensor, row_pair: torch.Tensor,
                     pair_row: torch.Tensor, tile_expert: torch.Tensor) -> None:
    """As :func:`moe_group` with every expert's rows padded to whole tiles of ``pad`` rows: ``starts`` (int32
    ``[experts + 1]``), ``row_pair`` (``[tiles * pad]``, -1 for a row of padding), ``pair_row`` and ``tile_expert``
    (``[tiles]``: the expert of a row tile, -1 behind the last); ``tiles * pad >= pairs + experts * (pad - 1)``."""
    need_cuda(idx, starts, row_pair, pair_row, tile_expert)
    for name, t in (("idx", idx), ("starts", starts), ("row_pair", row_pair), ("pair_row", pair_row), ("tile_expert", tile_expert)):
        need_int32(name, t), need_contiguous(name, t)
    tiles = tile_expert.numel()
    if starts.numel() != n_experts + 1 or row_pair.numel() != tiles * pad or pair_row.numel() != idx.numel():
        raise KernelError("moe_group_padded: starts [experts + 1], row_pair [tiles * pad], pair_row one entry per pair")
    _moe.call("zi_moe_group_padded", ptr(idx), c_int(idx.numel()), c_int(n_experts), c_int(pad), c_int(tiles), ptr(starts),
              ptr(row_pair), ptr(pair_row), ptr(tile_expert), stream())


def moe_gather_rows(x: torch.Tensor, row_pair: torch.Tensor, pairs_per_src: int, out: torch.Tensor,
                    scale: Optional[torch.Tensor] = None) -> None:
    """``out[r] = x[row_pair[r] // pairs_per_src]``, zeros where ``row_pair[r]`` is negative (bfloat16).  ``scale``: float32,
    one per pair; the row of pair ``row_pair[r]`` is multiplied by ``scale[row_pair[r]]`` and rounded once."""
    need_cuda(x, row_pair, out, scale)
    if scale is not None and (scale.dtype != torch.float32 or not scale.is_contiguous()):
        raise KernelError("moe_gather_rows: scale must be contiguous float32, one per pair")
    need_int32("row_pair", row_pair), need_contiguous("out", out)
    if x.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or x.stride(1) != 1 or out.shape != (row_pair.numel(), x.shape[1]):
        raise KernelError(f"moe_gather_rows: x {tuple(x.shape)} {x.dtype}, out {tuple(out.shape)}, {row_pair.numel()} rows")
    _moe.call("zi_moe_gather_rows", ptr(x), c_ll(x.stride(0)), ptr(row_pair), c_int(pairs_per_src), ptr(out), c_int(out.shape[0]),
              c_int(x.shape[1]), ptr(scale), stream())


GROUPED_TILE_ROWS = 128          # rows of a tile of the tcgen05 grouped product: groups are padded to whole tiles


def gemm_tcgen05_grouped(x: torch.Tensor, w: torch.Tensor, tile_expert: torch.Tensor, out: torch.Tensor,
                         gated: Optional[tuple] = None, relu2: bool = False) -> None:
    """Grouped product on the tcgen05 tensor cores: ``x`` holds every group's rows one after the other, padded to
    whole tiles of 128 rows; row tile t takes the weight ``w[tile_expert[t]]`` (``w`` is ``[experts, N, K]``, or with
    ``gated = (limit, slope, up_offset)`` ``[experts, 2 N, K]`` and the clamped, gated activation in the epilogue); a
    negative entry skips the tile.  ``relu2``: ``out = max(x @ w.T, 0)^2``.  ``out [rows, N]`` row by row as ``x``.  A
    bounded wait that runs out is reported by :func:`tcgen05_status`."""
    need_cuda(x, w, tile_expert, out)
    if gated and relu2:
        raise KernelError("gemm_tcgen05_grouped: one activation at a time")
    need_int32("tile_expert", tile_expert)
    need_contiguous("w", w), need_contiguous("tile_expert", tile_expert)
    m, k = x.shape
    e, n_w, _ = w.shape
    n = out.shape[1]
    if (m % GROUPED_TILE_ROWS or tile_expert.numel() != m // GROUPED_TILE_ROWS or w.shape[2] != k or out.shape[0] != m
            or n_w != (2 * n if gated else n) or x.stride(1) != 1 or out.stride(1) != 1):
        raise KernelError(f"gemm_tcgen05_grouped: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, "
                          f"{tile_expert.numel()} tiles do not agree")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tcgen05_grouped: bfloat16 operands only")
    limit, slope, up_offset = gated if gated else (0.0, 0.0, 0.0)
    _gemm_tcgen05.call("zi_gemm_tcgen05_grouped", ptr(x), ptr(w), ptr(out), c_int(dtype_code(out.dtype)), ptr(_tc_status(x.device)),
                       c_int(m), c_int(n), c_int(k), c_ll(x.stride(0)), c_ll(out.stride(0)), c_int(2 if gated else (3 if relu2 else 0)), c_int(e),
                       ptr(tile_expert), c_int(_num_sms(x.device)), c_float(limit), c_float(slope), c_float(up_offset), stream())
    _tc_launched[x.device] = True


MOE_TENSOR_CORES = True          # bfloat16 grouped products on the tensor cores (False: the SIMT form, as float32 uses)
MOE_FEW_ROWS_STREAMING = True    # up to 64 sorted rows (decode steps) on the weight-streaming form of the grouped product
MOE_TCGEN05_MIN_PAIRS = 65       # from this many (token, choice) pairs the grouped products run on the tcgen05 kernel


def moe_gemm(a: torch.Tensor, row_pair: Optional[torch.Tensor], pairs_per_src: int, w: torch.Tensor, offsets: torch.Tensor,
             out: torch.Tensor, gated: Optional[tuple] = None, relu2: bool = False,
             a_scale: Optional[torch.Tensor] = None) -> None:
    """Grouped product over the sorted rows of every expert: ``out[r] = a[src(r)] @ w[e(r)].T``; ``src(r) = row_pair[r]
    // pairs_per_src`` (``row_pair`` None: r itself), ``e(r)`` from ``offsets``.  ``w`` is ``[experts, N, K]``, or with
    ``gated = (limit, slope, up_offset)`` ``[experts, 2 N, K]`` (gate rows, then up rows) and ``out`` the clamped, gated
    product of the two halves (see :func:`gated_clamp_mul`).  ``relu2``: ``out = max(product, 0)^2``.  ``a_scale``: float32,
    one per pair; the row of ``a`` that sorted row r reads is multiplied by ``a_scale[row_pair[r]]`` (``row_pair`` None:
    ``a_scale[r]``) and rounded to ``a``'s type before the product (a router weight on the expert's input)."""
    need_cuda(a, row_pair, w, offsets, out, a_scale)
    if gated and relu2:
        raise KernelError("moe_gemm: one activation at a time")
    if a_scale is not None and (a_scale.dtype != torch.float32 or not a_scale.is_contiguous()):
        raise KernelError("moe_gemm: a_scale must be contiguous float32, one per pair")
    need_int32("offsets", offsets)
    need_contiguous("w", w), need_contiguous("out", out)
    if row_pair is not None:
        need_int32("row_pair", row_pair)
    rows, n = out.shape
    e, n_w, k = w.shape
    if a.stride(1) != 1 or a.shape[1] != k or n_w != (2 * n if gated else n) or offsets.numel() != e + 1:
        raise KernelError(f"moe_gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    limit, slope, up_offset = gated if gated else (0.0, 0.0, 0.0)
    _moe.call("zi_moe_gemm", ptr(a), c_int(dtype_code(a.dtype)), c_ll(a.stride(0)), ptr(row_pair), c_int(pairs_per_src), ptr(w),
              c_int(dtype_code(w.dtype)), ptr(offsets), c_int(e), ptr(out), c_int(dtype_code(out.dtype)), c_ll(out.stride(0)),
              c_int(rows), c_int(n), c_int(k), c_int(1 if gated else (2 if relu2 else 0)), c_float(limit), c_float(slope),
              c_float(up_offset), c_int((1 if MOE_TENSOR_CORES else 0) | (0 if MOE_FEW_ROWS_STREAMING else 2)), ptr(a_scale),
              stream())


def moe_combine(y: torch.Tensor, pair_row: torch.Tensor, wts: Optional[torch.Tensor], shared: Optional[torch.Tensor],
                out: torch.Tensor, x: Optional[torch.Tensor] = None, shared_gate: Optional[torch.Tensor] = None) -> None:
    """``out[t] = sum_j wts[t, j] * y[pair_row[t, j]] (+ shared_gate[t] * shared[t])``, j rising, in float32 with one rounding.
    ``y`` has a row per pair, or more where the sorted rows are padded.  ``wts`` None: every weight is 1 (``pair_row`` is then
    ``[tokens, top]``).  ``x``: the tokens' inputs; a pair whose ``pair_row`` is -1 (an expert that returns its input, see
    :func:`moe_group`) contributes ``wts[t, j] * x[t]``.  ``shared_gate``: float32, one factor per token (None: 1)."""
    need_cuda(y, pair_row, wts, shared, out, x, shared_gate)
    if x is not None and (x.shape != out.shape or x.dtype != out.dtype or x.stride(1) != 1):
        raise KernelError(f"moe_combine: x {tuple(x.shape)} must have out's shape and type")
    if shared_gate is not None and (shared_gate.dtype != torch.float32 or shared_gate.numel() != out.shape[0] or not shared_gate.is_contiguous()):
        raise KernelError("moe_combine: shared_gate must be contiguous float32 with one entry per token")
    need_int32("pair_row", pair_row)
    need_contiguous("y", y), need_contiguous("pair_row", pair_row), need_contiguous("out", out)
    n, hidden = out.shape
    if wts is None:
        top = pair_row.numel() // max(n, 1)
    else:
        need_contiguous("wts", wts)
        top = wts.shape[1]
    if (wts is not None and (wts.dtype != torch.float32 or wts.shape != (n, top))) or pair_row.numel() != n * top or y.dim() != 2 or y.shape[0] < n * top or y.shape[1] != hidden \
            or y.dtype != out.dtype or (shared is not None and (shared.shape != out.shape or shared.dtype != out.dtype
                                                                or not shared.is_contiguous())):
        raise KernelError(f"moe_combine: y {tuple(y.shape)}, {n} x {top} weights, out {tuple(out.shape)} do not agree")
    _moe.call("zi_moe_combine", ptr(y), ptr(pair_row), ptr(wts), ptr(shared), ptr(out), c_int(dtype_code(out.dtype)), c_int(n),
              c_int(top), c_int(hidden), ptr(x), c_ll(x.stride(0) if x is not None else 0), ptr(shared_gate), stream())


# ---- rotation of a span of every head, latents with a rotated key part, output gate: csrc/rowwise.cu ------------------------
def rotary(x: torch.Tensor, q_out: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, n_q: int, n_k: int, head_dim: int,
           rot_offset: int, rot_dims: int, interleaved: bool, cache=None, tables: Optional[torch.Tensor] = None,
           tok_seg: Optional[torch.Tensor] = None, v_mode: int = 0) -> None:
    """Turn entries ``rot_offset .. rot_offset + rot_dims`` of every query and key head of ``x`` (``[tokens, (n_q + n_k
    [+ n_k]) * head_dim]``, rows may be strided) by the token's position; entry i of the span pairs with ``i + rot_dims /
    2``, or with ``interleaved`` entry 2i with 2i + 1; the angle of pair i is ``float(pos) * inv_freq[i]``.  Queries go to
    ``q_out`` (``[tokens, n_q * head_dim]``; may be ``x`` itself).  ``cache`` (a CallCacheView with two planes): turned keys
    are appended to the first plane and, by ``v_mode``, the value heads of ``x`` (1) or the keys as they were before the
    turn (2) to the second."""
    need_cuda(x, q_out, pos, inv_freq, tables, tok_seg)
    need_int32("pos", pos)
    n = x.shape[0]
    if x.stride(1) != 1 or q_out.stride(-1) != 1 or q_out.dtype != x.dtype:
        raise KernelError("rotary: rows of x and q_out must be contiguous and of one type")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2 or not inv_freq.is_contiguous():
        raise KernelError(f"rotary: inv_freq must be float32 with {rot_dims // 2} entries")
    ct = None
    if cache is not None:
        ct = cache.tensor
        if tables is None or ct.dtype != x.dtype:
            raise KernelError("rotary: the cache append needs block tables and a cache of x's type")
        need_int32("tables", tables)
    q2 = q_out.view(n, -1) if q_out.dim() == 3 else q_out
    _rowwise.call("zi_rotary", ptr(x), c_int(dtype_code(x.dtype)), c_ll(x.stride(0)), ptr(q2), c_ll(q2.stride(0)), ptr(ct),
                  ptr(tables), ptr(tok_seg), ptr(pos), ptr(inv_freq), c_int(n), c_int(n_q), c_int(n_k if cache is not None else 0),
                  c_int(head_dim), c_int(rot_offset), c_int(rot_dims), c_int(1 if interleaved else 0), c_int(v_mode),
                  c_int(cache.page_size if cache is not None else 0), c_int(tables.shape[1] if tables is not None else 0),
                  c_ll(cache.page_stride if cache is not None else 0), c_ll(cache.kv_stride if cache is not None else 0), stream())


def latent_prepare(x: torch.Tensor, q_off: int, q_rank: int, gq: Optional[torch.Tensor], cq_out: Optional[torch.Tensor],
                   c_off: int, rank: int, gc: torch.Tensor, rot_dim: int, rot_dims: int, interleaved: bool,
                   inv_freq: Optional[torch.Tensor], eps: float, cache, tables: torch.Tensor, tok_seg: Optional[torch.Tensor],
                   pos: torch.Tensor) -> None:
    """From each row of ``x`` (a stacked product, rows may be strided): ``cq_out[n] = rmsnorm(x[n, q_off : q_off + q_rank])
    * gq`` (``q_rank`` 0: none), and into the row of token n in ``cache`` (one plane, one head, ``cache.tensor.shape[-1]``
    entries) ``rmsnorm(x[n, c_off : c_off + rank]) * gc`` followed by the next ``rot_dim`` entries of ``x`` with their first
    ``rot_dims`` turned by the token's position (pairing and angles as :func:`rotary`).  ``cache`` None: only the query
    latent."""
    need_cuda(x, gq, cq_out, gc, inv_freq, tables, tok_seg, pos)
    need_int32("pos", pos)
    if x.stride(1) != 1 or (cq_out is not None and (not cq_out.is_contiguous() or cq_out.dtype != x.dtype)):
        raise KernelError("latent_prepare: rows of x must be contiguous, cq_out contiguous and of x's type")
    if q_rank and (gq is None or cq_out is None or gq.dtype != gc.dtype):
        raise KernelError("latent_prepare: a query latent needs its weight and an output")
    if rot_dims and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2):
        raise KernelError(f"latent_prepare: inv_freq must be float32 with {rot_dims // 2} entries")
    ct = cache.tensor if cache is not None else None
    if ct is not None and ct.dtype != x.dtype:
        raise KernelError("latent_prepare: the cache must have x's type")
    _rowwise.call("zi_latent_prepare", ptr(x), c_int(dtype_code(x.dtype)), c_ll(x.stride(0)), c_int(q_off), c_int(q_rank), ptr(gq),
                  ptr(cq_out), c_int(c_off), c_int(rank), ptr(gc), c_int(dtype_code(gc.dtype)), c_int(rot_dim), c_int(rot_dims),
                  c_int(1 if interleaved else 0), ptr(inv_freq), c_float(eps), ptr(ct), c_int(ct.shape[-1] if ct is not None else 0),
                  ptr(tables), ptr(tok_seg), ptr(pos), c_int(x.shape[0]), c_int(cache.page_size if cache is not None else 0),
                  c_int(tables.shape[1] if tables is not None else 0), c_ll(cache.page_stride if cache is not None else 0), stream())


def sigmoid_mul(a: torch.Tensor, g: torch.Tensor) -> None:
    """In place: ``a *= sigmoid(g)`` (float32 inside); ``g [rows, width]`` may have strided rows."""
    need_cuda(a, g)
    need_contiguous("a", a)
    if a.dim() != 2 or g.shape != a.shape or g.stride(1) != 1 or g.dtype != a.dtype:
        raise KernelError(f"sigmoid_mul: a {tuple(a.shape)} and g {tuple(g.shape)} must agree")
    _rowwise.call("zi_sigmoid_mul", ptr(a), ptr(g), c_int(dtype_code(a.dtype)), c_ll(g.stride(0)), c_int(a.shape[0]), c_int(a.shape[1]),
                  stream())


# ---- selective state-space mixer, csrc/ssm.cu ----------------------------------------------------------------------------------
def segment_bounds(tok_seg: torch.Tensor, n_segments: int, out: torch.Tensor) -> None:
    """``out[s] = (first token, one past the last token)`` of segment s (int32 ``[segments, 2]``) from the token -> segment
    map of a step whose segments are runs of consecutive tokens."""
    need_cuda(tok_seg, out)
    need_int32("tok_seg", tok_seg), need_int32("out", out)
    need_contiguous("tok_seg", tok_seg), need_contiguous("out", out)
    if out.numel() != 2 * n_segments:
        raise KernelError("segment_bounds: out must be [segments, 2]")
    _ssm.call("zi_segment_bounds", ptr(tok_seg), c_int(tok_seg.numel()), c_int(n_segments), ptr(out), stream())


def _state_args(state: torch.Tensor, offset: int):
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1:
        raise KernelError("a state slot pool must be float32 [slots, entries]")
    return c_void_p(state.data_ptr() + 4 * offset), c_ll(state.stride(0))


def causal_conv_silu(u: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, state_offset: int,
                     slots: torch.Tensor, tok_seg: Optional[torch.Tensor], pos: torch.Tensor, out: torch.Tensor,
                     update_state: bool = False) -> None:
    """``out[n, c] = silu(bias[c] + sum_j w[c, j] * u_c(pos[n] - (taps - 1) + j))``: a causal convolution per channel over
    each request's tokens.  Inputs of this step come from ``u`` (``[tokens, channels]``, rows may be strided), earlier ones
    from the request's slot of ``state`` (float32 ``[slots, entries]``; the ring ``[taps - 1, channels]`` starts at entry
    ``state_offset``), and what lies before position 0 is zero.  ``tok_seg`` None: token n is segment n.  ``update_state``
    (only with ``tok_seg`` None): every token's input also goes into its ring, as :func:`conv_state_update` does otherwise."""
    if update_state and tok_seg is not None:
        raise KernelError("causal_conv_silu: only a step of single tokens may update the state on the way")
    need_cuda(u, w, bias, state, slots, tok_seg, pos, out)
    need_int32("slots", slots), need_int32("pos", pos)
    need_contiguous("w", w), need_contiguous("out", out)
    n, ch = u.shape
    if u.stride(1) != 1 or w.shape[0] != ch or out.shape != (n, ch) or out.dtype != u.dtype or (bias is not None and (bias.numel() != ch or bias.dtype != w.dtype)):
        raise KernelError(f"causal_conv_silu: u {tuple(u.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    sp, ss = _state_args(state, state_offset)
    _ssm.call("zi_causal_conv_silu", ptr(u), c_int(dtype_code(u.dtype)), c_ll(u.stride(0)), ptr(w), ptr(bias), c_int(dtype_code(w.dtype)),
              sp, ss, ptr(slots), ptr(tok_seg), ptr(pos), ptr(out), c_int(n), c_int(ch), c_int(w.shape[1]),
              c_int(1 if update_state else 0), stream())


def conv_state_update(u: torch.Tensor, taps: int, state: torch.Tensor, state_offset: int, slots: torch.Tensor,
                      bounds: Optional[torch.Tensor], pos: torch.Tensor, n_segments: int) -> None:
    """The last ``taps - 1`` inputs of every segment go into its slot's ring (the input at position q into row ``q mod
    (taps - 1)``).  ``bounds`` from :func:`segment_bounds`; None: segment s is token s."""
    need_cuda(u, state, slots, bounds, pos)
    need_int32("slots", slots), need_int32("pos", pos)
    if u.stride(1) != 1:
        raise KernelError("conv_state_update: rows of u must be contiguous")
    sp, ss = _state_args(state, state_offset)
    _ssm.call("zi_conv_state_update", ptr(u), c_int(dtype_code(u.dtype)), c_ll(u.stride(0)), sp, ss, ptr(slots), ptr(bounds), ptr(pos),
              c_int(n_segments), c_int(u.shape[1]), c_int(taps), stream())


def ssm_scan(xbc: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, slots: torch.Tensor, bounds: Optional[torch.Tensor], y: torch.Tensor, n_segments: int,
             heads: int, vdim: int, n_state: int, groups: int, stretchwise: bool = False) -> None:
    """The recurrence of a selective state-space layer over each segment's tokens in order, float32 throughout:
    ``dt = softplus(dt + dt_bias)``, ``S = exp(-exp(a_log) dt) S + dt B x^T``, ``y = S^T C + d_skip x``.  ``xbc [tokens, heads
    * vdim + 2 * groups * n_state]`` holds x, B and C; ``dt [tokens, heads]`` (rows of both may be strided); ``y`` float32
    ``[tokens, heads * vdim]``.  A request's state (``[heads, vdim, n_state]``, the first entries of its slot of ``state``) is
    read at the start and written back at the end; slot -1: zero, not written.

    ``stretchwise`` (needs ``bounds``): every segment is cut into stretches of 128 tokens that run side by side, first each
    from a zero state, then, once a small kernel has carried the states through them in order, again with the outputs: the
    same sums in another order, for long portions of prompts that would otherwise occupy a block per head and column tile."""
    need_cuda(xbc, dt, dt_bias, a_log, d_skip, state, slots, bounds, y)
    if stretchwise and bounds is None:
        raise KernelError("ssm_scan: the stretch-wise form needs the segments' bounds")
    need_int32("slots", slots)
    need_contiguous("y", y)
    n = xbc.shape[0]
    inner = heads * vdim
    if (xbc.stride(1) != 1 or dt.stride(1) != 1 or xbc.shape[1] != inner + 2 * groups * n_state or dt.shape != (n, heads) or dt.dtype != xbc.dtype
            or y.dtype != torch.float32 or y.shape != (n, inner) or not (dt_bias.dtype == a_log.dtype == d_skip.dtype)
            or dt_bias.numel() != heads or a_log.numel() != heads or d_skip.numel() != heads):
        raise KernelError(f"ssm_scan: xbc {tuple(xbc.shape)}, dt {tuple(dt.shape)}, y {tuple(y.shape)} do not agree")
    if state.shape[1] < inner * n_state:
        raise KernelError("ssm_scan: the state slots are too small")
    sp, ss = _state_args(state, 0)
    scratch = None
    if stretchwise:
        lib = _ssm.lib
        lib.zi_ssm_scan_scratch_floats.restype = c_ll
        floats = int(lib.zi_ssm_scan_scratch_floats(c_int(n), c_int(n_segments), c_int(heads), c_int(vdim), c_int(n_state)))
        scratch = _grown_scratch(("ssm_scan", xbc.device), floats, xbc.device)
    _ssm.call("zi_ssm_scan", ptr(xbc), c_int(dtype_code(xbc.dtype)), c_ll(xbc.stride(0)), ptr(dt), c_ll(dt.stride(0)), ptr(dt_bias),
              ptr(a_log), ptr(d_skip), c_int(dtype_code(dt_bias.dtype)), sp, ss, ptr(slots), ptr(bounds), ptr(y), c_int(n),
              c_int(n_segments), c_int(heads), c_int(vdim), c_int(n_state), c_int(groups), ptr(scratch), stream())


def gated_group_rmsnorm(y: torch.Tensor, z: torch.Tensor, w: torch.Tensor, n_groups: int, eps: float, out: torch.Tensor) -> None:
    """``out = unit_rms(y * silu(z)) * w`` with the root mean square taken over each of ``n_groups`` equal parts of a row;
    ``y`` float32, ``z`` (rows may be strided) and ``out`` of the step's type."""
    need_cuda(y, z, w, out)
    need_contiguous("y", y), need_contiguous("w", w), need_contiguous("out", out)
    n, inner = y.shape
    if y.dtype != torch.float32 or z.shape != (n, inner) or z.stride(1) != 1 or out.shape != (n, inner) or out.dtype != z.dtype or w.numel() != inner:
        raise KernelError(f"gated_group_rmsnorm: y {tuple(y.shape)}, z {tuple(z.shape)}, out {tuple(out.shape)} do not agree")
    _ssm.call("zi_gated_group_rmsnorm", ptr(y), ptr(z), c_int(dtype_code(z.dtype)), c_ll(z.stride(0)), ptr(w), c_int(dtype_code(w.dtype)),
              ptr(out), c_int(n), c_int(inner), c_int(n_groups), c_float(eps), stream())


# ---- a turned span with a factor, unit heads and a cache whose rows are wider than a head; a normed branch into the stream;
# ---- a gate on a token's own table entry: csrc/rowwise.cu -------------------------------------------------------------------
def rotary_norm(x: torch.Tensor, q_out: torch.Tensor, pos: torch.Tensor, inv_freq: Optional[torch.Tensor], mag: float, n_q: int,
                n_k: int, qk_dim: int, v_dim: int, row_dim: int, rot_dims: int, interleaved: bool, unit_eps: Optional[float],
                cache=None, tables: Optional[torch.Tensor] = None, tok_seg: Optional[torch.Tensor] = None,
                q_head_scale: Optional[torch.Tensor] = None) -> None:
    """Turn the first ``rot_dims`` entries of every query and key head of ``x`` (``[tokens, (n_q + n_k) * qk_dim + n_k *
    v_dim]``, rows may be strided) by the token's position (pairing and angles as :func:`rotary`; cosines and sines times
    ``mag``), then, with ``unit_eps``, divide every query and key head by its root mean square ``sqrt(mean + unit_eps)``.
    Queries go to ``q_out`` (``[tokens, n_q, row_dim]``), keys and values to the two planes of ``cache`` (a CallCacheView whose
    rows are ``row_dim`` wide); what lies past a head's own entries is written as zero.  ``cache`` None: queries alone (``x``
    then holds no keys and values).  ``q_head_scale`` (float32, one per query head): every query head is multiplied by its
    own factor as it is written, which multiplies that head's scores."""
    need_cuda(x, q_out, pos, inv_freq, tables, tok_seg, q_head_scale)
    if q_head_scale is not None and (q_head_scale.dtype != torch.float32 or q_head_scale.numel() != n_q or not q_head_scale.is_contiguous()):
        raise KernelError(f"rotary_norm: q_head_scale must be contiguous float32 with {n_q} entries")
    need_int32("pos", pos)
    need_contiguous("q_out", q_out)
    n = x.shape[0]
    if x.stride(1) != 1 or q_out.dtype != x.dtype or q_out.numel() != n * n_q * row_dim:
        raise KernelError("rotary_norm: rows of x must be contiguous, q_out [tokens, n_q, row_dim] of x's type")
    if rot_dims and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dims // 2 or not inv_freq.is_contiguous()):
        raise KernelError(f"rotary_norm: inv_freq must be float32 with {rot_dims // 2} entries")
    ct = None
    if cache is not None:
        ct = cache.tensor
        if tables is None or ct.dtype != x.dtype or ct.shape[-1] != row_dim:
            raise KernelError("rotary_norm: the cache append needs block tables and a cache of x's type with rows of row_dim")
        need_int32("tables", tables)
        if x.shape[1] < (n_q + n_k) * qk_dim + n_k * v_dim:
            raise KernelError("rotary_norm: x is too narrow for its heads")
    _rowwise.call("zi_rotary_norm", ptr(x), c_int(dtype_code(x.dtype)), c_ll(x.stride(0)), ptr(q_out), ptr(ct), ptr(tables), ptr(tok_seg),
                  ptr(pos), ptr(inv_freq), c_float(mag), ptr(q_head_scale), c_int(n), c_int(n_q), c_int(n_k if cache is not None else 0), c_int(qk_dim),
                  c_int(v_dim), c_int(row_dim), c_int(rot_dims), c_int(1 if interleaved else 0), c_int(1 if unit_eps is not None else 0),
                  c_float(unit_eps or 0.0), c_int(cache.page_size if cache is not None else 0),
                  c_int(tables.shape[1] if tables is not None else 0), c_ll(cache.page_stride if cache is not None else 0),
                  c_ll(cache.kv_stride if cache is not None else 0), stream())


def norm_add(h: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, rounded: Optional[torch.Tensor] = None) -> None:
    """``h += y / sqrt(mean(y^2) + eps) * w`` row by row, in float32 (``h`` float32 ``[rows, hidden]``); ``rounded`` (of y's
    type) receives the new ``h``."""
    need_cuda(h, y, w, rounded)
    need_contiguous("h", h), need_contiguous("y", y), need_contiguous("w", w)
    if h.dtype != torch.float32 or y.shape != h.shape or w.numel() != h.shape[1]:
        raise KernelError(f"norm_add: h {tuple(h.shape)} float32, y {tuple(y.shape)} and w {tuple(w.shape)} do not agree")
    if rounded is not None and (rounded.shape != h.shape or rounded.dtype != y.dtype or not rounded.is_contiguous()):
        raise KernelError("norm_add: rounded must be contiguous, of y's type and h's shape")
    _rowwise.call("zi_norm_add", ptr(h), ptr(y), c_int(dtype_code(y.dtype)), ptr(w), c_int(dtype_code(w.dtype)), ptr(rounded),
                  c_float(eps), c_int(h.shape[0]), c_int(h.shape[1]), stream())


def gelu_mul_rows(t: torch.Tensor, table: torch.Tensor, col0: int, ids: torch.Tensor, out: torch.Tensor) -> None:
    """``out[n, j] = gelu_tanh(t[n, j]) * table[ids[n], col0 + j]`` (float32 inside); rows of ``t`` may be strided."""
    need_cuda(t, table, ids, out)
    need_int32("ids", ids)
    need_contiguous("table", table), need_contiguous("out", out), need_contiguous("ids", ids)
    n, width = t.shape
    if t.stride(1) != 1 or out.shape != (n, width) or out.dtype != t.dtype or ids.numel() != n or table.dim() != 2:
        raise KernelError(f"gelu_mul_rows: t {tuple(t.shape)}, out {tuple(out.shape)} and ids {tuple(ids.shape)} do not agree")
    _rowwise.call("zi_gelu_mul_rows", ptr(t), c_int(dtype_code(t.dtype)), c_ll(t.stride(0)), ptr(table), c_int(dtype_code(table.dtype)),
                  c_ll(table.shape[1]), c_int(col0), ptr(ids), c_int(table.shape[0]), ptr(out), c_int(n), c_int(width), stream())


# ---- linear recurrences with a matrix state per head, csrc/linrec.cu ---------------------------------------------------------
LINEAR_STATE_RULES = {"delta": 0, "decay": 1, "forget": 2}
_SILU_ON = {"q": 1, "k": 2, "v": 4}


def linear_state(rule: str, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, slots: torch.Tensor,
                 bounds: Optional[torch.Tensor], y: torch.Tensor, n_segments: int, heads: int, kv_heads: int, dim: int, vdim: int,
                 a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None, dt_bias: Optional[torch.Tensor] = None,
                 a_log: Optional[torch.Tensor] = None, decay: Optional[torch.Tensor] = None, act_silu=False,
                 q_scale: float = 1.0, unit_eps: float = 1e-6, work: Optional[torch.Tensor] = None,
                 decay_per_head: bool = False) -> None:
    """Walk each segment's tokens in order through a float32 state ``S`` (``dim x vdim``) per head.

    ``rule="delta"``: ``S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`` with ``q`` and ``k`` made unit vectors
    per head (``x / sqrt(sum x^2 + unit_eps)``; ``q`` also times ``q_scale``), ``beta = sigmoid(b)`` (``b [tokens, heads]``) and
    ``g = exp(-exp(a_log) softplus(a + dt_bias))`` (``a [tokens, heads * dim]``, ``dt_bias`` float32 ``[heads * dim]``, ``a_log``
    float32 ``[heads]``; with ``decay_per_head`` one decay per head: ``a [tokens, heads]``, ``dt_bias [heads]``).
    ``rule="decay"``: ``S <- decay_h S + k v^T; o = S^T q`` (``decay`` float32 ``[heads]``; ``q`` times ``q_scale``).
    ``rule="forget"``: ``S <- diag(f) S + (1 - f) v^T; o = S^T q`` with ``f = l + (1 - l) sigmoid(a)`` per head and key entry
    (``a [tokens, heads * dim]``, the lower bounds ``l`` in ``dt_bias`` float32 ``[heads * dim]``; ``k`` is None, ``kv_heads``
    equals ``heads``; ``q`` times ``q_scale``).  ``act_silu``: True: q, k and v pass through SiLU first; a string names which
    of them do (``"q"``, ``"qk"``, ...).  ``q``, ``k`` ``[tokens, kv_heads * dim]`` (head h reads
    query/key head ``h // (heads / kv_heads)``) and ``v [tokens, heads * vdim]`` may have strided rows; ``y`` float32
    ``[tokens, heads * vdim]``.  A request's state (``[heads, vdim, dim]``, the first entries of its slot of ``state``) is read
    at the start and written back at the end; slot -1: zero, not written.  ``bounds`` from :func:`segment_bounds`; None:
    segment s is token s.

    ``work`` (float32, at least :func:`linear_state_work_floats` entries): a first kernel makes every token's inputs ready
    there (all tokens and heads at once) and the walk only copies and walks, which pays for segments of many tokens; without
    it the walk makes its inputs ready itself.  A token's result has the same bits either way."""
    need_cuda(q, k, v, state, slots, bounds, y, a, b, dt_bias, a_log, decay, work)
    forget = rule == "forget"
    if forget:
        if k is not None or kv_heads != heads:
            raise KernelError("linear_state: the forget rule has no keys and a query head per head")
        k = q
    silu_bits = 7 if act_silu is True else sum(_SILU_ON[c] for c in set(act_silu)) if act_silu else 0
    if work is not None and (work.dtype != torch.float32 or not work.is_contiguous()):
        raise KernelError("linear_state: the workspace must be contiguous float32")
    need_int32("slots", slots)
    need_contiguous("y", y)
    n = q.shape[0]
    if (q.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1 or q.shape != (n, kv_heads * dim) or k.shape != q.shape
            or v.shape != (n, heads * vdim) or not (q.dtype == k.dtype == v.dtype) or y.dtype != torch.float32
            or y.shape != (n, heads * vdim)):
        raise KernelError(f"linear_state: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}, y {tuple(y.shape)} do not agree")
    per_head = bool(decay_per_head) and rule == "delta"
    for name, t, width in (("a", a, heads if per_head else heads * dim), ("b", b, heads)):
        if t is not None and (t.shape != (n, width) or t.stride(1) != 1 or t.dtype != q.dtype):
            raise KernelError(f"linear_state: {name} must be [tokens, {width}] of q's type")
    for name, t, count in (("dt_bias", dt_bias, heads if per_head else heads * dim), ("a_log", a_log, heads), ("decay", decay, heads)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != count or not t.is_contiguous()):
            raise KernelError(f"linear_state: {name} must be contiguous float32 with {count} entries")
    if state.shape[1] < heads * vdim * dim:
        raise KernelError("linear_state: the state slots are too small")
    sp, ss = _state_args(state, 0)
    _linrec.call("zi_linear_state", c_int(LINEAR_STATE_RULES[rule]), ptr(q), c_ll(q.stride(0)), ptr(k), c_ll(k.stride(0)), ptr(v),
                 c_ll(v.stride(0)), ptr(a), c_ll(a.stride(0) if a is not None else 0), ptr(b), c_ll(b.stride(0) if b is not None else 0),
                 c_int(dtype_code(q.dtype)), ptr(dt_bias), ptr(a_log), ptr(decay), sp, ss, ptr(slots), ptr(bounds), ptr(y), c_int(n),
                 c_int(n_segments), c_int(heads), c_int(kv_heads), c_int(dim), c_int(vdim), c_int(silu_bits), c_int(1 if per_head else 0),
                 c_float(q_scale), c_float(unit_eps), ptr(work), c_ll(work.numel() if work is not None else 0), stream())


def linear_state_work_floats(rule: str, n_tokens: int, heads: int, dim: int, vdim: int) -> int:
    """Entries of the float32 workspace :func:`linear_state` needs to make ``n_tokens`` tokens ready beforehand: per token
    and head a record of q, k (and the decays in the delta rule) padded to the kernel's 32, 64, 128 or 256 entries plus
    four scalars, and the values padded to whole tiles of 16 columns."""
    padded = 32 if dim <= 32 else 64 if dim <= 64 else 128 if dim <= 128 else 256
    record = (2 if rule == "decay" else 3) * padded + 4
    return n_tokens * heads * (record + (vdim + 15) // 16 * 16)


GROUP_NORM_GATES = {"sigmoid": 0, "silu": 1, None: 2}


def group_rmsnorm_gate(y: torch.Tensor, z: Optional[torch.Tensor], w: torch.Tensor, n_groups: int, eps: float, out: torch.Tensor,
                       gate: Optional[str] = "sigmoid") -> None:
    """``out = unit_rms(y) * w * gate(z)`` with the root mean square over each of ``n_groups`` equal parts of a row and
    ``w`` repeated along the row when it is shorter; ``y`` float32, ``z`` (rows may be strided) and ``out`` of the step's type.
    ``gate``: ``"sigmoid"``, ``"silu"`` or None (no gate; ``z`` is then None)."""
    need_cuda(y, z, w, out)
    need_contiguous("y", y), need_contiguous("w", w), need_contiguous("out", out)
    n, inner = y.shape
    if gate not in GROUP_NORM_GATES or (gate is None) != (z is None):
        raise KernelError(f"group_rmsnorm_gate: gate={gate!r} is not 'sigmoid', 'silu' or None, or does not fit z")
    if y.dtype != torch.float32 or out.shape != (n, inner) or (z is not None and (z.shape != (n, inner) or z.stride(1) != 1 or out.dtype != z.dtype)):
        raise KernelError(f"group_rmsnorm_gate: y {tuple(y.shape)}, z {tuple(z.shape) if z is not None else None}, out {tuple(out.shape)} do not agree")
    _linrec.call("zi_group_rmsnorm_gate", ptr(y), ptr(z), c_int(dtype_code(out.dtype)), c_ll(z.stride(0) if z is not None else 0), ptr(w),
                 c_int(dtype_code(w.dtype)), c_int(w.numel()), ptr(out), c_int(n), c_int(inner), c_int(n_groups), c_float(eps),
                 c_int(GROUP_NORM_GATES[gate]), stream())


# ---- the tanh norm, joined branches, an activation of normed powers, a gate per row: csrc/rowwise.cu -----------------------------
def _tanh_norm_args(name: str, norm, hidden: int):
    """``norm``: (alpha, weight, bias) with float32 vectors of ``hidden`` entries, or None."""
    if norm is None:
        return c_float(0.0), ptr(None), ptr(None)
    alpha, w, b = norm
    for t in (w, b):
        if t.dtype != torch.float32 or t.numel() != hidden or not t.is_contiguous() or not t.is_cuda:
            raise KernelError(f"{name}: weight and bias must be contiguous float32 on the device with {hidden} entries")
    return c_float(float(alpha)), ptr(w), ptr(b)


def tanh_norm(x: torch.Tensor, alpha: float, w: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """``out = tanh(alpha x) * w + b`` row by row (float32 inside; ``w``, ``b`` float32)."""
    need_cuda(x, w, b, out)
    need_contiguous("x", x), need_contiguous("out", out)
    rows, hidden = x.shape
    if out.shape != x.shape:
        raise KernelError(f"tanh_norm: x {tuple(x.shape)} and out {tuple(out.shape)} do not agree")
    a, pw, pb = _tanh_norm_args("tanh_norm", (alpha, w, b), hidden)
    _rowwise.call("zi_tanh_norm", ptr(x), c_int(dtype_code(x.dtype)), a, pw, pb, ptr(out), c_int(dtype_code(out.dtype)), c_int(rows),
                  c_int(hidden), stream())


def tanh_norm_fold(h: torch.Tensor, y: Optional[torch.Tensor], post, pre, out: Optional[torch.Tensor],
                   row_idx: Optional[torch.Tensor] = None, write_h: bool = True, dtype: Optional[torch.dtype] = None,
                   join=None) -> None:
    """The tanh norm ``N(v; alpha, w, b) = tanh(alpha v) * w + b`` on both sides of the float32 stream ``h``: ``v = h + N(y;
    post)`` where a branch's output ``y`` is pending (``y`` None: ``v = h``), ``h = v`` where ``write_h``, ``out = N(v; pre)``
    where ``out`` is given.  ``post``, ``pre``: (alpha, float32 weight, float32 bias) or None.  With ``row_idx`` output row r
    comes from row ``row_idx[r]`` and ``h`` is left as it is.  ``join = (y2, w1, w2, eps)``: the pending output is that of two
    branches joined on the way, ``(U(y) * w1 + U(y2) * w2) / 2`` with ``U(v) = v / sqrt(mean(v^2) + eps)`` over a row and float32
    weights (what :func:`rms_pair_mean` computes, without the rounding in between)."""
    need_cuda(h, y, out, row_idx)
    need_contiguous("h", h)
    if h.dtype != torch.float32 or h.dim() != 2:
        raise KernelError(f"tanh_norm_fold: the stream must be float32 [rows, hidden], got {tuple(h.shape)} {h.dtype}")
    hidden = h.shape[1]
    if row_idx is not None:
        need_int32("row_idx", row_idx), need_contiguous("row_idx", row_idx)
        write_h = False
    rows = row_idx.numel() if row_idx is not None else h.shape[0]
    if y is not None and (y.shape != h.shape or not y.is_contiguous() or post is None):
        raise KernelError("tanh_norm_fold: a pending branch must be contiguous, of h's shape, and bring the norm that follows it")
    if out is not None and (out.shape != (rows, hidden) or not out.is_contiguous() or pre is None or (y is not None and y.dtype != out.dtype)):
        raise KernelError(f"tanh_norm_fold: out {tuple(out.shape)} does not fit {(rows, hidden)}, or lacks its norm")
    kind = out.dtype if out is not None else (y.dtype if y is not None else (dtype or torch.float32))
    post_a, post_w, post_b = _tanh_norm_args("tanh_norm_fold", post if y is not None else None, hidden)
    pre_a, pre_w, pre_b = _tanh_norm_args("tanh_norm_fold", pre if out is not None else None, hidden)
    if join is not None:
        y2, w1, w2, eps = join
        need_cuda(y2, w1, w2)
        if y is None or y2.shape != y.shape or y2.dtype != y.dtype or not y2.is_contiguous():
            raise KernelError("tanh_norm_fold: the second branch must be contiguous, of the first one's shape and type")
        for t in (w1, w2):
            if t.dtype != torch.float32 or t.numel() != hidden or not t.is_contiguous():
                raise KernelError(f"tanh_norm_fold: the branches' weights must be contiguous float32 with {hidden} entries")
        _rowwise.call("zi_tanh_norm_fold_pair", ptr(h), ptr(y), ptr(y2), c_int(dtype_code(kind)), ptr(w1), ptr(w2), c_float(eps), post_a,
                      post_w, post_b, pre_a, pre_w, pre_b, ptr(out), ptr(row_idx), c_int(rows), c_int(hidden),
                      c_int(1 if write_h else 0), stream())
        return
    _rowwise.call("zi_tanh_norm_fold", ptr(h), ptr(y), c_int(dtype_code(kind)), post_a, post_w, post_b, pre_a, pre_w, pre_b, ptr(out),
                  ptr(row_idx), c_int(rows), c_int(hidden), c_int(1 if write_h else 0), stream())


def rms_pair_mean(x: torch.Tensor, z: torch.Tensor, wx: torch.Tensor, wz: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """``out = (U(x) * wx + U(z) * wz) / 2`` with ``U(v) = v / sqrt(mean(v^2) + eps)`` over a row (float32 inside; ``wx``, ``wz``
    float32)."""
    need_cuda(x, z, wx, wz, out)
    need_contiguous("x", x), need_contiguous("z", z), need_contiguous("out", out), need_contiguous("wx", wx), need_contiguous("wz", wz)
    rows, hidden = x.shape
    if z.shape != x.shape or out.shape != x.shape or not (x.dtype == z.dtype == out.dtype) or wx.dtype != torch.float32 \
            or wz.dtype != torch.float32 or wx.numel() != hidden or wz.numel() != hidden:
        raise KernelError(f"rms_pair_mean: x {tuple(x.shape)}, z {tuple(z.shape)}, out {tuple(out.shape)} and the float32 weights do not agree")
    _rowwise.call("zi_rms_pair_mean", ptr(x), ptr(z), c_int(dtype_code(x.dtype)), ptr(wx), ptr(wz), ptr(out), c_float(eps), c_int(rows),
                  c_int(hidden), stream())


def poly_norm(z: torch.Tensor, coeffs, eps: float, out: torch.Tensor) -> None:
    """``out = c1 U(z) + c2 U(z^2) + c3 U(z^3) + c0`` with ``coeffs = (c1, c2, c3, c0)``, powers entry by entry and ``U(v) = v /
    sqrt(mean(v^2) + eps)`` over a row (float32 inside); rows of ``z`` may be strided."""
    need_cuda(z, out)
    need_contiguous("out", out)
    rows, width = z.shape
    if z.stride(1) != 1 or out.shape != z.shape or out.dtype != z.dtype or len(coeffs) != 4:
        raise KernelError(f"poly_norm: z {tuple(z.shape)}, out {tuple(out.shape)} and four coefficients do not agree")
    c1, c2, c3, c0 = (float(c) for c in coeffs)
    _rowwise.call("zi_poly_norm", ptr(z), c_int(dtype_code(z.dtype)), c_ll(z.stride(0)), ptr(out), c_int(rows), c_int(width), c_float(c1),
                  c_float(c2), c_float(c3), c_float(c0), c_float(eps), stream())


def row_gate(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out[n] = sigmoid(x[n] . w)`` in float32 (``out`` float32, one entry per row; rows of ``x`` may be strided)."""
    need_cuda(x, w, out)
    need_contiguous("w", w), need_contiguous("out", out)
    rows, k = x.shape
    if x.stride(1) != 1 or w.numel() != k or out.dtype != torch.float32 or out.numel() != rows:
        raise KernelError(f"row_gate: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    _rowwise.call("zi_row_gate", ptr(x), c_int(dtype_code(x.dtype)), c_ll(x.stride(0)), ptr(w), c_int(dtype_code(w.dtype)), ptr(out),
                  c_int(rows), c_int(k), stream())
