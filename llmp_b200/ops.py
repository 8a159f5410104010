"""Host-side mirror of the reference's operators for the quantized-product
path (src/kernels/ggml/llmp_ops.h:1072-1085 QuantizeQ8 / VecQ, ...), over
torch CUDA tensors.  Each function checks what the C ABI cannot see (dtype,
device, contiguity), fills the launch descriptor and queues the kernels on the
current torch stream.  Nothing here computes: without the native library or a
B200 the calls raise.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _native as N
from ._native import (GLU_GEGLU, GLU_NONE, GLU_SWIGLU, GLU_SWIGLU_CLAMP, TYPE_Q4_K, TYPE_Q8_0,
                      LaunchFailed, Rejected)

__all__ = ["available", "sm_count", "device_faults", "device_faults_clear", "block_bytes", "block_elems", "q8_1_row_blocks",
           "quantize_q8", "vecq", "vecq_ranks", "mmvq", "vecq_f32", "vecq_q8", "vecq_q8_scratch", "vecq_variants", "vecq_block_sums", "mxfp8_padded_rows",
           "mxfp8_quantize", "mxfp8_swizzle", "mxfp8_gemm", "mxfp8_mul_mat_vec", "decode_vector", "decode_rows", "decode_matrix", "decode_grouped", "DECODER_Q8_0", "DECODER_MXFP8_SPLIT",
           "DECODER_MXFP8_ATOMS", "DECODER_BF16", "DECODER_F16", "DECODER_NVFP4_SPLIT", "DECODER_NVFP4_ATOMS",
           "DECODER_MXFP4_SPLIT", "DECODER_MXFP4_ATOMS", "mmq_quantize", "mmq", "mmq_scratch", "mmq_block_sums", "q4k_relayout", "moe_route", "grouped_gemm",
           "moe_glu_quantize", "moe_combine", "moe_ep_pack", "moe_ffn", "moe_decode", "moe_decode_fits",
           "mmq_glu", "grouped_gemm_glu", "TYPE_Q8_0", "TYPE_Q4_K",
           "TYPE_Q4_0", "TYPE_Q5_0", "TYPE_Q5_K", "TYPE_Q6_K", "TYPE_IQ4_NL",
           "GLU_NONE", "GLU_SWIGLU", "GLU_SWIGLU_CLAMP", "GLU_GEGLU", "Rejected", "LaunchFailed"]

TYPE_Q4_0, TYPE_Q5_0, TYPE_Q5_K, TYPE_Q6_K, TYPE_IQ4_NL = 2, 6, 13, 14, 20   # GGML's type ids
_BLOCK = {TYPE_Q8_0: (32, 34), TYPE_Q4_K: (256, 144), N.TYPE_Q8_1: (32, 36), TYPE_Q4_0: (32, 18),
          TYPE_Q5_0: (32, 22), TYPE_IQ4_NL: (32, 18), TYPE_Q5_K: (256, 176), TYPE_Q6_K: (256, 210)}
# moe_ffn: up to this many tokens take the routed decode products (measured on B200 against the
# grouped tensor-core GEMM for 128 experts, top-8, hidden 2048, intermediate 768).
DECODE_TOKENS = 96


def available() -> bool:
    return bool(N.lib().llmp_b200_available())


def device_faults() -> int:
    """Bounded device-side waits that ran out since load (0 when healthy)."""
    return int(N.lib().llmp_b200_device_faults())


def device_faults_clear() -> int:
    """Zeroes that counter; returns what it held."""
    return int(N.lib().llmp_b200_device_faults_clear())


def sm_count() -> int:
    return int(N.lib().llmp_b200_sm_count())


def block_elems(t: int) -> int:
    return _BLOCK[t][0]


def block_bytes(t: int) -> int:
    return _BLOCK[t][1]


def q8_1_row_blocks(k: int) -> int:
    return int(N.lib().llmp_b200_q8_1_row_blocks(k))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, dtype, what: str) -> None:
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == dtype):
        raise Rejected(f"{what}: a CUDA tensor of {dtype}")


def quantize_q8(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """QuantizeQ8: x F32 [rows, k] or [planes, rows, k] (last dim contiguous) ->
    uint8 [planes*rows, q8_1_row_blocks(k) * 36]."""
    _need(x, torch.float32, "quantize_q8 input")
    if x.dim() == 2:
        x = x.unsqueeze(0)
    if x.dim() != 3 or x.stride(2) != 1:
        raise Rejected("quantize_q8: F32 [k, rows, planes] with k contiguous")
    planes, rows, k = x.shape
    nb = q8_1_row_blocks(k)
    if out is None:
        out = torch.empty((planes * rows, nb * 36), dtype=torch.uint8, device=x.device)
    _need(out, torch.uint8, "quantize_q8 output")
    if out.numel() != planes * rows * nb * 36 or not out.is_contiguous():
        raise Rejected("quantize_q8: output of rows * row_blocks * 36 bytes")
    N.check(N.lib().llmp_b200_q8_1_quantize(x.data_ptr(), k, rows, planes, x.stride(1), x.stride(0),
                                            out.data_ptr(), _stream()), "llmp_b200_q8_1_quantize")
    return out


def vecq_variants() -> list[str]:
    L = N.lib()
    return [L.llmp_b200_vecq_variant_name(i).decode() for i in range(L.llmp_b200_vecq_variants())]


def vecq_ranks() -> list[dict]:
    """The measured rank table: the fastest launch configuration per dense Q4_K product."""
    L = N.lib()
    rows = []
    for i in range(L.llmp_b200_vecq_rank_count()):
        k, n, glu, tokens, us = C.c_int(), C.c_int(), C.c_int(), C.c_int(), C.c_float()
        name = L.llmp_b200_vecq_rank(i, C.byref(k), C.byref(n), C.byref(glu), C.byref(tokens),
                                     C.byref(us))
        rows.append({"k": k.value, "n": n.value, "glu": glu.value, "tokens": tokens.value,
                     "variant": name.decode(), "microseconds": us.value})
    return rows


def vecq(weights: torch.Tensor, wtype: int, k: int, n: int, q8: torch.Tensor, tokens: int, *,
         ids: torch.Tensor | None = None, per_slot: bool = False, gate: torch.Tensor | None = None,
         glu: int = GLU_NONE, limit: float = 0.0, groups: int = 1, stride_row: int | None = None,
         stride_expert: int | None = None, variant: int = -1, fan=None,
         out: torch.Tensor | None = None) -> torch.Tensor:
    """VecQ.  Dense: weights [n, k] blocks, q8 of [tokens, k] -> F32 [tokens, n].
    Grouped (groups > 1, per_slot): matrix g over row g of q8 of [tokens, groups, k]
    -> F32 [tokens, groups, n].  Routed: weights [experts, n, k], ids I32 [tokens, used];
    q8 of [tokens, k] or, per_slot, [tokens, used, k] -> F32 [tokens, used, n].
    gate: weights like `weights`; the result is glu(gate.x, weights.x)."""
    _need(weights, torch.uint8, "vecq weights")
    _need(q8, torch.uint8, "vecq q8")
    elems, nbytes = _BLOCK.get(wtype, (0, 0)) if wtype != N.TYPE_Q8_1 else (0, 0)
    if elems == 0:
        raise Rejected(f"vecq: weight type {wtype}")
    routed = ids is not None
    used = ids.shape[1] if routed else groups
    d = N.VecQDesc()
    d.w = weights.data_ptr()
    d.g = gate.data_ptr() if gate is not None else None
    if gate is not None:
        _need(gate, torch.uint8, "vecq gate")
    d.y = q8.data_ptr()
    if routed:
        _need(ids, torch.int32, "vecq ids")
        if ids.dim() != 2 or ids.shape[0] != tokens or ids.stride(1) != 1:
            raise Rejected("vecq: ids I32 [used, tokens]")
        d.ids = ids.data_ptr()
        d.ids_stride = ids.stride(0)
    d.ncols_x, d.nrows = k, n
    d.stride_row = k // elems if stride_row is None else stride_row
    d.stride_expert = (n * d.stride_row if (routed or groups > 1) else 0) \
        if stride_expert is None else stride_expert
    y_row = q8_1_row_blocks(k)
    d.y_token = y_row * used if per_slot else y_row
    d.y_slot = y_row if per_slot else 0
    d.used, d.tokens = used, tokens
    slotted = routed or groups > 1
    shape = (tokens, used, n) if slotted else (tokens, n)
    if out is None:
        out = torch.empty(shape, dtype=torch.float32, device=weights.device)
    _need(out, torch.float32, "vecq output")
    if tuple(out.shape) != shape or not out.is_contiguous():
        raise Rejected(f"vecq: a packed F32 output {shape}")
    d.dst = out.data_ptr()
    d.dst_token = used * n if slotted else n
    d.dst_slot = n if slotted else 0
    d.glu, d.limit = glu, limit
    if fan is not None:     # also into every rank's vector of tagged words (llmp_b200/peer.py)
        N.check(N.lib().llmp_b200_vecq_fan(wtype, C.byref(d), variant, C.byref(fan), _stream()),
                "llmp_b200_vecq_fan")
        return out
    N.check(N.lib().llmp_b200_vecq(wtype, C.byref(d), variant, _stream()), "llmp_b200_vecq")
    return out


def mmvq(weights: torch.Tensor, wtype: int, k: int, n: int, x: torch.Tensor | None = None, *,
         q8: torch.Tensor | None = None, gate: torch.Tensor | None = None, glu: int = GLU_NONE,
         limit: float = 0.0, rows: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """The reference's MMVQ calls.  x F32 [cols, k] -> F32 [cols, n]: MulMatVecQ (with `gate`,
    MulMatVecQGlu); q8 (prepared Q8_1 rows of the columns) instead of x: RunMmvqPrepared;
    rows=True: MulMatVecQRows, every column's bits the one-column product's, any column
    count."""
    _need(weights, torch.uint8, "mmvq weights")
    if wtype not in (TYPE_Q8_0, TYPE_Q4_K):
        raise Rejected(f"mmvq: weight type {wtype}")
    d = N.MmvqDesc()
    d.type, d.w, d.k, d.n = wtype, weights.data_ptr(), k, n
    d.gate = gate.data_ptr() if gate is not None else None
    d.glu, d.limit = glu, limit
    d.stride_row = k // _BLOCK[wtype][0]
    if q8 is not None:
        _need(q8, torch.uint8, "mmvq q8")
        cols = q8.shape[0]
        d.q8 = q8.data_ptr()
        scratch = None
    else:
        _need(x, torch.float32, "mmvq x")
        if x.dim() != 2 or x.stride(1) != 1:
            raise Rejected("mmvq: x F32 [cols, k], k contiguous")
        cols = x.shape[0]
        d.x, d.x_col_stride = x.data_ptr(), x.stride(0)
        scratch = torch.empty((int(N.lib().llmp_b200_mmvq_scratch(k, cols)),), dtype=torch.uint8,
                              device=weights.device)
        d.scratch = scratch.data_ptr()
    d.cols = cols
    if out is None:
        out = torch.empty((cols, n), dtype=torch.float32, device=weights.device)
    d.dst, d.dst_col_stride = out.data_ptr(), out.stride(0)
    L = N.lib()
    fn = L.llmp_b200_mmvq_rows if rows else (L.llmp_b200_mmvq_prepared if q8 is not None
                                             else L.llmp_b200_mmvq)
    N.check(fn(C.byref(d), _stream()), "llmp_b200_mmvq")
    return out


def vecq_f32(weights: torch.Tensor, wtype: int, k: int, n: int, x: torch.Tensor, *,
             gate: torch.Tensor | None = None, glu: int = GLU_NONE, limit: float = 0.0,
             out: torch.Tensor | None = None, q8_out: torch.Tensor | None = None) -> torch.Tensor:
    """QuantizeQ8 + VecQ in one launch: x F32 [tokens <= 8, k] (rows 16-byte aligned), dense
    Q4_K weights [n, k] -> F32 [tokens, n].  q8_out (uint8 [tokens, q8_1_row_blocks(k) * 36])
    optionally receives the Q8_1 blocks the kernel formed."""
    _need(weights, torch.uint8, "vecq_f32 weights")
    _need(x, torch.float32, "vecq_f32 activations")
    if x.dim() != 2 or x.stride(1) != 1:
        raise Rejected("vecq_f32: F32 [k, tokens] with k contiguous")
    tokens = x.shape[0]
    d = N.VecQDesc()
    d.w = weights.data_ptr()
    d.g = gate.data_ptr() if gate is not None else None
    d.y = x.data_ptr()
    d.ncols_x, d.nrows = k, n
    d.stride_row = k // _BLOCK[wtype][0]
    d.y_token = x.stride(0)
    d.used, d.tokens = 1, tokens
    if out is None:
        out = torch.empty((tokens, n), dtype=torch.float32, device=weights.device)
    d.dst, d.dst_token = out.data_ptr(), n
    d.glu, d.limit = glu, limit
    N.check(N.lib().llmp_b200_vecq_f32(wtype, C.byref(d),
                                       q8_out.data_ptr() if q8_out is not None else None,
                                       _stream()), "llmp_b200_vecq_f32")
    return out


def vecq_q8_scratch(n: int, tokens: int, device) -> torch.Tensor:
    """Zeroed row counters for vecq_q8 (every call leaves them zero)."""
    nbytes = int(N.lib().llmp_b200_vecq_q8_scratch(n, tokens))
    return torch.zeros(nbytes // 4, dtype=torch.int32, device=device)


def vecq_q8(weights: torch.Tensor, wtype: int, k: int, n: int, q8: torch.Tensor, tokens: int, *,
            rows_done: torch.Tensor, gate: torch.Tensor | None = None, glu: int = GLU_NONE,
            limit: float = 0.0, out: torch.Tensor | None = None,
            q8_dst: torch.Tensor | None = None):
    """VecQ + QuantizeQ8 of its output in one launch: dense Q4_K weights [n, k] (n a multiple
    of 512), q8 of [tokens <= 8, k] -> (F32 [tokens, n], its Q8_1 blocks uint8 [tokens, n/32*36])."""
    _need(weights, torch.uint8, "vecq_q8 weights")
    _need(q8, torch.uint8, "vecq_q8 q8")
    _need(rows_done, torch.int32, "vecq_q8 counters")
    d = N.VecQDesc()
    d.w = weights.data_ptr()
    d.g = gate.data_ptr() if gate is not None else None
    d.y = q8.data_ptr()
    d.ncols_x, d.nrows = k, n
    d.stride_row = k // _BLOCK[wtype][0]
    d.y_token = q8_1_row_blocks(k)
    d.used, d.tokens = 1, tokens
    if out is None:
        out = torch.empty((tokens, n), dtype=torch.float32, device=weights.device)
    if q8_dst is None:
        q8_dst = torch.empty((tokens, q8_1_row_blocks(n) * 36), dtype=torch.uint8,
                             device=weights.device)
    _need(out, torch.float32, "vecq_q8 output")
    _need(q8_dst, torch.uint8, "vecq_q8 output blocks")
    if rows_done.numel() * 4 < int(N.lib().llmp_b200_vecq_q8_scratch(n, tokens)):
        raise Rejected("vecq_q8: counters of llmp_b200_vecq_q8_scratch(n, tokens) bytes")
    d.dst, d.dst_token = out.data_ptr(), n
    d.glu, d.limit = glu, limit
    N.check(N.lib().llmp_b200_vecq_q8(wtype, C.byref(d), q8_dst.data_ptr(), rows_done.data_ptr(),
                                      _stream()), "llmp_b200_vecq_q8")
    return out, q8_dst


def vecq_block_sums(weights: torch.Tensor, wtype: int, k: int, n: int, q8_row: torch.Tensor):
    """The int32 per-block sums of n weight rows against one Q8_1 row:
    (dots [n, k/32], qsums [n, k/32] or None for Q8_0)."""
    _need(weights, torch.uint8, "block_sums weights")
    _need(q8_row, torch.uint8, "block_sums q8")
    dots = torch.empty((n, k // 32), dtype=torch.int32, device=weights.device)
    qsums = torch.empty_like(dots) if wtype == TYPE_Q4_K else None
    N.check(N.lib().llmp_b200_vecq_block_sums(
        wtype, weights.data_ptr(), q8_row.data_ptr(), k, n, k // _BLOCK[wtype][0], dots.data_ptr(),
        qsums.data_ptr() if qsums is not None else None, _stream()), "llmp_b200_vecq_block_sums")
    return dots, qsums


# ----------------------------------------------------------------------- MXFP8
def mxfp8_padded_rows(rows: int) -> int:
    return int(N.lib().llmp_b200_mxfp8_padded_rows(rows))


def mxfp8_quantize(x: torch.Tensor):
    """Mxfp8Quantize: x F32 or BF16 [rows, k] -> (codes uint8 [rows, k], scale atoms uint8
    [padded_rows(rows) * k / 32])."""
    if not (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.dim() == 2
            and x.stride(1) == 1):
        raise Rejected("mxfp8_quantize: a CUDA F32 or BF16 [rows, k] tensor, k contiguous")
    rows, k = x.shape
    codes = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    scales = torch.empty((mxfp8_padded_rows(rows) * (k // 32),), dtype=torch.uint8, device=x.device)
    N.check(N.lib().llmp_b200_mxfp8_quantize(x.data_ptr(), int(x.dtype == torch.bfloat16),
                                             x.stride(0), k, rows, codes.data_ptr(),
                                             scales.data_ptr(), _stream()),
            "llmp_b200_mxfp8_quantize")
    return codes, scales


def mxfp8_swizzle(scales: torch.Tensor) -> torch.Tensor:
    """Mxfp8Swizzle: weight scales uint8 [n, k / 32] row-major -> scale atoms."""
    _need(scales, torch.uint8, "mxfp8_swizzle scales")
    if scales.dim() != 2 or not scales.is_contiguous():
        raise Rejected("mxfp8_swizzle: packed [n, k / 32] scales")
    n, blocks = scales.shape
    out = torch.empty((mxfp8_padded_rows(n) * blocks,), dtype=torch.uint8, device=scales.device)
    N.check(N.lib().llmp_b200_mxfp8_swizzle(scales.data_ptr(), out.data_ptr(), n, blocks,
                                            _stream()), "llmp_b200_mxfp8_swizzle")
    return out


def mxfp8_gemm(a: torch.Tensor, a_scales: torch.Tensor, b: torch.Tensor, b_scales: torch.Tensor,
               *, bf16: bool = True, out: torch.Tensor | None = None, sms: int = 0,
               variant: int = 0) -> torch.Tensor:
    """Mxfp8Gemm: D[m, n] = A[m, k] . B[n, k]^T; codes uint8, scales in atoms.  variant 0: the
    library's rule; 1: one CTA a tile; 2: CTA pairs (llmp_b200_mxfp8_gemm_variant)."""
    for t, what in ((a, "a"), (b, "b"), (a_scales, "a_scales"), (b_scales, "b_scales")):
        _need(t, torch.uint8, f"mxfp8_gemm {what}")
    m, k = a.shape
    n = b.shape[0]
    if b.shape[1] != k or not a.is_contiguous() or not b.is_contiguous():
        raise Rejected("mxfp8_gemm: packed codes [m, k] and [n, k]")
    if a_scales.numel() < mxfp8_padded_rows(m) * (k // 32) or \
            b_scales.numel() < mxfp8_padded_rows(n) * (k // 32):
        raise Rejected("mxfp8_gemm: scale atoms for the padded rows")
    dtype = torch.bfloat16 if bf16 else torch.float32
    if out is None:
        out = torch.empty((m, n), dtype=dtype, device=a.device)
    if out.dtype != dtype or tuple(out.shape) != (m, n) or not out.is_contiguous():
        raise Rejected("mxfp8_gemm: a packed [m, n] output of the requested type")
    g = N.Mxfp8GemmDesc()
    g.m, g.n, g.k = m, n, k
    g.a, g.a_scales, g.b, g.b_scales = a.data_ptr(), a_scales.data_ptr(), b.data_ptr(), \
        b_scales.data_ptr()
    g.d, g.bf16, g.scratch = out.data_ptr(), int(bf16), None
    if variant == 0:
        N.check(N.lib().llmp_b200_mxfp8_gemm(C.byref(g), sms, _stream()), "llmp_b200_mxfp8_gemm")
    else:
        N.check(N.lib().llmp_b200_mxfp8_gemm_variant(C.byref(g), sms, variant, _stream()),
                "llmp_b200_mxfp8_gemm_variant")
    return out


# ----------------------------------------------------------------------- MMQ
def mmq_quantize(x: torch.Tensor, ids_src: torch.Tensor | None = None,
                 cols: int | None = None) -> torch.Tensor:
    """x F32 or BF16 [rows, k] -> Q8_1-MMQ blocks uint8 [k / 128, cols, 144]; with ids_src
    (I32 [cols]) column c quantizes row ids_src[c]."""
    if not (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.dim() == 2
            and x.stride(1) == 1):
        raise Rejected("mmq_quantize: a CUDA F32 or BF16 [rows, k] tensor, k contiguous")
    rows, k = x.shape
    if ids_src is not None:
        _need(ids_src, torch.int32, "mmq_quantize ids_src")
    cols = (rows if ids_src is None else ids_src.numel()) if cols is None else cols
    out = torch.empty((max(k // 128, 1), cols, 144), dtype=torch.uint8, device=x.device)
    N.check(N.lib().llmp_b200_mmq_quantize(
        x.data_ptr(), int(x.dtype == torch.bfloat16), x.stride(0), k, cols,
        ids_src.data_ptr() if ids_src is not None else None, out.data_ptr(), _stream()),
        "llmp_b200_mmq_quantize")
    return out


def q4k_relayout(weights: torch.Tensor, k: int, n: int, *, glu: bool = False) -> torch.Tensor:
    """The load-time relayout of Q4_K weights [n, k blocks] or experts [experts, n, k blocks]
    into the tensor core's slab (llmp_b200_q4k_relayout): a uint8 tensor to pass as `slab`.
    glu: the n rows are n / 2 gate rows then n / 2 up rows and the slab interleaves them for the
    GLU write-back (llmp_b200_q4k_relayout_glu; for mmq_glu / grouped_gemm_glu only)."""
    _need(weights, torch.uint8, "q4k_relayout weights")
    experts = weights.shape[0] if weights.dim() == 3 else 1
    stride_row = weights.stride(-2) // 144
    stride_expert = weights.stride(0) // 144 if weights.dim() == 3 else n * stride_row
    slab = torch.empty((int(N.lib().llmp_b200_q4k_slab_bytes(n, k, experts)),), dtype=torch.uint8,
                       device=weights.device)
    if glu:
        N.check(N.lib().llmp_b200_q4k_relayout_glu(weights.data_ptr(), n // 2, k, stride_row,
                                                   stride_expert, experts, slab.data_ptr(), _stream()),
                "llmp_b200_q4k_relayout_glu")
        return slab
    N.check(N.lib().llmp_b200_q4k_relayout(weights.data_ptr(), n, k, stride_row, stride_expert,
                                           experts, slab.data_ptr(), _stream()),
            "llmp_b200_q4k_relayout")
    return slab


def mmq_glu(yq: torch.Tensor, k: int, inter: int, slab: torch.Tensor, glu: int = GLU_SWIGLU,
            limit: float = 0.0) -> torch.Tensor:
    """MulMatQGlu: the gate | up product (slab from q4k_relayout(..., glu=True)) with the GLU and the
    requantization in its write-back -> Q8_1-MMQ blocks [inter / 128, cols, 144]."""
    _need(yq, torch.uint8, "mmq_glu activations")
    if yq.dim() != 3 or yq.shape[2] != 144 or not yq.is_contiguous() or inter % 128 != 0:
        raise Rejected("mmq_glu: packed Q8_1-MMQ blocks [k / 128, cols, 144], inter a multiple of 128")
    cols = yq.shape[1]
    out = torch.empty((inter // 128, cols, 144), dtype=torch.uint8, device=yq.device)
    d = N.MmqDesc()
    d.type, d.y, d.k, d.nrows, d.ncols = TYPE_Q4_K, yq.data_ptr(), k, 2 * inter, cols
    d.stride_row, d.dst_col_stride, d.experts, d.max_cols_per_expert = k // 256, 2 * inter, 1, cols
    d.w_slab = slab.data_ptr()
    N.check(N.lib().llmp_b200_mmq_glu(C.byref(d), glu, limit, out.data_ptr(), _stream()),
            "llmp_b200_mmq_glu")
    return out


def grouped_gemm_glu(a: torch.Tensor, offsets: torch.Tensor, k: int, inter: int, slab: torch.Tensor,
                     glu: int = GLU_SWIGLU, limit: float = 0.0, *,
                     scratch: torch.Tensor | None = None) -> torch.Tensor:
    """The grouped gate | up product with the GLU write-back (llmp_b200_grouped_gemm_glu): a Q8_1-MMQ
    blocks [k / 128, rows, 144] of expert-sorted rows, slab from q4k_relayout(experts' gate_up,
    glu=True) -> Q8_1-MMQ blocks [inter / 128, rows, 144]."""
    _need(a, torch.uint8, "grouped_gemm_glu activations")
    _need(offsets, torch.int32, "grouped_gemm_glu offsets")
    groups, rows = offsets.numel() - 1, a.shape[1]
    if inter % 128 != 0:
        raise Rejected("grouped_gemm_glu: inter a multiple of 128")
    out = torch.empty((inter // 128, rows, 144), dtype=torch.uint8, device=a.device)
    need = int(N.lib().llmp_b200_grouped_gemm_scratch(groups, rows, 0))
    if scratch is None:
        scratch = torch.empty((need,), dtype=torch.uint8, device=a.device)
    g = N.GroupedGemmDesc()
    g.groups, g.n, g.k, g.rows = groups, 2 * inter, k, rows
    g.offsets, g.a = offsets.data_ptr(), a.data_ptr()
    g.expert_stride = 2 * inter * (k // 256) * 144
    g.weights_slab, g.scratch = slab.data_ptr(), scratch.data_ptr()
    N.check(N.lib().llmp_b200_grouped_gemm_glu(C.byref(g), glu, limit, out.data_ptr(), 0, _stream()),
            "llmp_b200_grouped_gemm_glu")
    return out


def _mmq_desc(weights, yq, k, n, wtype, ids_dst, expert_bounds, out_cols, max_cols_per_expert,
              stride_row, stride_expert, out, slab, scratch):
    _need(yq, torch.uint8, "mmq activations")
    if yq.dim() != 3 or yq.shape[2] != 144 or not yq.is_contiguous():
        raise Rejected("mmq: packed Q8_1-MMQ blocks [k / 128, cols, 144]")
    ncols = yq.shape[1]
    out_cols = ncols if out_cols is None else out_cols
    if out is None:
        out = torch.empty((out_cols, n), dtype=torch.float32, device=yq.device)
    _need(out, torch.float32, "mmq output")
    d = N.MmqDesc()
    d.type, d.y, d.dst = wtype, yq.data_ptr(), out.data_ptr()
    if weights is not None:
        _need(weights, torch.uint8, "mmq weights")
        d.w = weights.data_ptr()
    d.ids_dst = ids_dst.data_ptr() if ids_dst is not None else None
    d.expert_bounds = expert_bounds.data_ptr() if expert_bounds is not None else None
    d.k, d.nrows, d.ncols = k, n, ncols
    d.stride_row = k // 256 if stride_row is None else stride_row
    d.stride_expert = (n * d.stride_row if expert_bounds is not None else 0) \
        if stride_expert is None else stride_expert
    d.dst_col_stride = out.stride(0)
    d.experts = expert_bounds.numel() - 1 if expert_bounds is not None else 1
    d.max_cols_per_expert = ncols if max_cols_per_expert is None else max_cols_per_expert
    d.w_slab = slab.data_ptr() if slab is not None else None
    d.scratch = scratch.data_ptr() if scratch is not None else None
    return d, out


def mmq_scratch(k: int, n: int, experts: int = 1, device="cuda") -> torch.Tensor:
    """Scratch for mmq(..., scratch=...): room for the weights' slab."""
    return torch.empty((int(N.lib().llmp_b200_q4k_slab_bytes(n, k, experts)),), dtype=torch.uint8,
                       device=device)


def mmq(weights: torch.Tensor | None, yq: torch.Tensor, k: int, n: int, *, wtype: int = TYPE_Q4_K,
        ids_dst: torch.Tensor | None = None, expert_bounds: torch.Tensor | None = None,
        out_cols: int | None = None, max_cols_per_expert: int | None = None,
        stride_row: int | None = None, stride_expert: int | None = None,
        out: torch.Tensor | None = None, slab: torch.Tensor | None = None,
        scratch: torch.Tensor | None = None) -> torch.Tensor:
    """MulMatQ: weights Q4_K [n, k] (or [experts, n, k] with expert_bounds over the sorted
    columns of yq) x Q8_1-MMQ activations -> F32 [out_cols, n].  slab: the weights as
    q4k_relayout left them (then weights may be None); scratch (mmq_scratch): the call relays
    the weights there first; neither: the kernel unpacks the raw blocks itself."""
    d, out = _mmq_desc(weights, yq, k, n, wtype, ids_dst, expert_bounds, out_cols,
                       max_cols_per_expert, stride_row, stride_expert, out, slab, scratch)
    N.check(N.lib().llmp_b200_mmq(C.byref(d), 0, _stream()), "llmp_b200_mmq")
    return out


def mmq_block_sums(weights: torch.Tensor | None, yq: torch.Tensor, k: int, n: int, *,
                   slab: torch.Tensor | None = None, scratch: torch.Tensor | None = None):
    """The dense product and the exact int32 group sums it folds: (F32 [cols, n], I32
    [cols, n, k / 32])."""
    d, out = _mmq_desc(weights, yq, k, n, TYPE_Q4_K, None, None, None, None, None, None, None, slab,
                       scratch)
    sums = torch.empty((yq.shape[1], n, k // 32), dtype=torch.int32, device=yq.device)
    N.check(N.lib().llmp_b200_mmq_block_sums(C.byref(d), sums.data_ptr(), _stream()),
            "llmp_b200_mmq_block_sums")
    return out, sums


# ----------------------------------------------------------------------- MoE
def moe_route(ids: torch.Tensor, experts: int) -> dict:
    """MoeRoute: ids I32 [tokens, used] -> the route blob and views of its parts."""
    _need(ids, torch.int32, "moe_route ids")
    if ids.dim() != 2 or ids.stride(1) != 1:
        raise Rejected("moe_route: ids I32 [used, tokens]")
    tokens, used = ids.shape
    n = int(N.lib().llmp_b200_moe_route_ints(experts, used, tokens))
    blob = torch.empty((n,), dtype=torch.int32, device=ids.device)
    N.check(N.lib().llmp_b200_moe_route(ids.data_ptr(), ids.stride(0), experts, used, tokens,
                                        blob.data_ptr(), _stream()), "llmp_b200_moe_route")
    slots, e1 = tokens * used, experts + 1
    return {"blob": blob, "offsets": blob[:e1], "scale_rows": blob[e1:2 * e1],
            "position": blob[2 * e1:2 * e1 + slots],
            "token": blob[2 * e1 + slots:2 * e1 + 2 * slots],
            "expert": blob[2 * e1 + 2 * slots:2 * e1 + 3 * slots],
            "counts": blob[2 * e1 + 3 * slots:], "experts": experts, "used": used,
            "tokens": tokens}


def grouped_gemm(weights: torch.Tensor | None, a: torch.Tensor, offsets: torch.Tensor, k: int, n: int,
                 *, out: torch.Tensor | None = None, scratch: torch.Tensor | None = None,
                 slab: torch.Tensor | None = None) -> torch.Tensor:
    """MoeGemm: weights Q4_K [groups, n, k] (or their slab from q4k_relayout); a Q8_1-MMQ blocks
    [k / 128, rows, 144] of expert-sorted rows; offsets I32 [groups + 1] -> F32 [rows, n]."""
    _need(a, torch.uint8, "grouped_gemm activations")
    _need(offsets, torch.int32, "grouped_gemm offsets")
    groups, rows = offsets.numel() - 1, a.shape[1]
    if out is None:
        out = torch.empty((rows, n), dtype=torch.float32, device=a.device)
    need = int(N.lib().llmp_b200_grouped_gemm_scratch(groups, rows, 0))
    if scratch is None:
        scratch = torch.empty((need,), dtype=torch.uint8, device=a.device)
    g = N.GroupedGemmDesc()
    g.groups, g.n, g.k, g.rows = groups, n, k, rows
    g.offsets, g.a = offsets.data_ptr(), a.data_ptr()
    g.expert_stride = n * (k // 256) * 144
    if weights is not None:
        _need(weights, torch.uint8, "grouped_gemm weights")
        g.weights = weights.data_ptr()
        if weights.dim() == 3:
            g.expert_stride = weights.stride(0)
    g.weights_slab = slab.data_ptr() if slab is not None else None
    g.d, g.scratch = out.data_ptr(), scratch.data_ptr()
    N.check(N.lib().llmp_b200_grouped_gemm(C.byref(g), 0, _stream()), "llmp_b200_grouped_gemm")
    return out


def moe_glu_quantize(gate_up: torch.Tensor, f: int, glu: int = GLU_SWIGLU,
                     limit: float = 0.0) -> torch.Tensor:
    """MoeGluQuantize: gate_up F32 [rows, 2 f] -> Q8_1-MMQ blocks [f / 128, rows, 144]."""
    _need(gate_up, torch.float32, "moe_glu_quantize input")
    rows = gate_up.shape[0]
    out = torch.empty((f // 128, rows, 144), dtype=torch.uint8, device=gate_up.device)
    N.check(N.lib().llmp_b200_moe_glu_quantize(gate_up.data_ptr(), gate_up.stride(0), f, rows, glu,
                                               limit, out.data_ptr(), _stream()),
            "llmp_b200_moe_glu_quantize")
    return out


def moe_ep_pack(x: torch.Tensor, ids: torch.Tensor, experts: int, world: int, capacity: int,
                dropped: torch.Tensor):
    """The expert-parallel dispatch's packing (llmp_b200_moe_ep_pack): x F32 [tokens, hidden],
    ids I32 [tokens, used] -> (send rows [world * capacity, hidden], send ids I32 [world *
    capacity], home I32 [tokens * used]); dropped: an I32 device counter of rows past capacity."""
    _need(x, torch.float32, "moe_ep_pack rows")
    _need(ids, torch.int32, "moe_ep_pack ids")
    _need(dropped, torch.int32, "moe_ep_pack dropped counter")
    tokens, used = ids.shape
    hidden = x.shape[1]
    per = experts // world
    owner = torch.where((ids >= 0) & (ids < experts), ids // per, torch.full_like(ids, -1))
    route = moe_route(owner.contiguous(), world)
    send = torch.empty((world * capacity, hidden), dtype=torch.float32, device=x.device)
    send_ids = torch.empty((world * capacity,), dtype=torch.int32, device=x.device)
    home = torch.empty((tokens * used,), dtype=torch.int32, device=x.device)
    N.check(N.lib().llmp_b200_moe_ep_pack(x.data_ptr(), x.stride(0), hidden, ids.data_ptr(),
                                          ids.stride(0), used, tokens, experts, world, capacity,
                                          route["blob"].data_ptr(), send.data_ptr(),
                                          send_ids.data_ptr(), home.data_ptr(), dropped.data_ptr(),
                                          _stream()), "llmp_b200_moe_ep_pack")
    return send, send_ids, home


def moe_combine(rows: torch.Tensor, position: torch.Tensor | None, weights: torch.Tensor, tokens: int,
                used: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """MoeCombineSorted: rows F32 [slots, width] -> F32 [tokens, width]; position None: the
    rows are in slot order."""
    _need(rows, torch.float32, "moe_combine rows")
    if position is not None:
        _need(position, torch.int32, "moe_combine position")
    _need(weights, torch.float32, "moe_combine weights")
    width = rows.shape[1]
    if out is None:
        out = torch.empty((tokens, width), dtype=torch.float32, device=rows.device)
    N.check(N.lib().llmp_b200_moe_combine(rows.data_ptr(), rows.stride(0),
                                          position.data_ptr() if position is not None else None,
                                          weights.data_ptr(), used, tokens, width, out.data_ptr(),
                                          _stream()), "llmp_b200_moe_combine")
    return out


_MOE_DECODE_SCRATCH: dict = {}
MOE_DECODE_TOKENS = 4      # up to here the one-launch block beats the five-launch one


def moe_decode_fits(tokens: int, used: int, hidden: int, inter: int) -> bool:
    """Whether llmp_b200_moe_decode takes the shape."""
    ur_a, span = hidden // 256, 1
    while span < inter // 256:
        span *= 2
    return (hidden % 256 == 0 and inter % 256 == 0 and 256 <= hidden <= 8192 and inter >= 256 and
            ur_a & (ur_a - 1) == 0 and ur_a <= 32 and used * span <= 32 and used * inter <= 16384 and
            1 <= tokens <= 16)


def moe_decode(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, gate_up: torch.Tensor,
               down: torch.Tensor, hidden: int, inter: int, glu: int = GLU_SWIGLU, limit: float = 0.0,
               *, out: torch.Tensor | None = None, scratch: torch.Tensor | None = None) -> torch.Tensor:
    """The routed block for 1 to 16 tokens as one launch (llmp_b200_moe_decode).  Without
    `scratch` a cached buffer per device and size is used: calls that may overlap on the GPU
    (several streams) must bring their own (uint8, llmp_b200_moe_decode_scratch bytes, zeroed)."""
    _need(x, torch.float32, "moe_decode x")
    _need(ids, torch.int32, "moe_decode ids")
    _need(weights, torch.float32, "moe_decode weights")
    tokens, used = ids.shape
    if x.dim() != 2 or x.shape != (tokens, hidden) or x.stride(1) != 1 or ids.stride(1) != 1 or \
            not weights.is_contiguous() or tuple(weights.shape) != (tokens, used):
        raise Rejected("moe_decode: x F32 [tokens, hidden], ids I32 and weights F32 [tokens, used]")
    if not gate_up.is_contiguous() or not down.is_contiguous():
        raise Rejected("moe_decode: packed expert tensors")
    nbytes = int(N.lib().llmp_b200_moe_decode_scratch(used, tokens, inter))
    if scratch is None:
        key = (x.device, nbytes)
        scratch = _MOE_DECODE_SCRATCH.get(key)
        if scratch is None:
            scratch = _MOE_DECODE_SCRATCH[key] = torch.zeros((nbytes,), dtype=torch.uint8, device=x.device)
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=x.device)
    d = N.MoeDecodeDesc()
    d.x, d.x_stride, d.ids, d.ids_stride = x.data_ptr(), x.stride(0), ids.data_ptr(), ids.stride(0)
    d.weights, d.gate_up, d.down = weights.data_ptr(), gate_up.data_ptr(), down.data_ptr()
    d.experts, d.used, d.tokens, d.hidden, d.inter = gate_up.shape[0], used, tokens, hidden, inter
    d.glu, d.limit = glu, limit
    d.dst, d.dst_stride, d.scratch = out.data_ptr(), out.stride(0), scratch.data_ptr()
    N.check(N.lib().llmp_b200_moe_decode(C.byref(d), _stream()), "llmp_b200_moe_decode")
    return out


def moe_ffn(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, gate_up: torch.Tensor,
            down: torch.Tensor, hidden: int, inter: int, glu: int = GLU_SWIGLU,
            decode_tokens: int | None = None, slabs: tuple | None = None) -> torch.Tensor:
    """The routed-expert block as the reference wires it (tests/unit/qwen38_moe_test.cc:487-497):
    route -> quantize (scattered to expert-sorted rows) -> grouped GEMM gate|up -> GLU +
    requantize -> grouped GEMM down -> ordered weighted combine.  x F32/BF16 [tokens, hidden];
    ids I32 [tokens, used]; weights F32 [tokens, used]; gate_up Q4_K [experts, 2 inter, hidden]
    (gate rows then up rows); down Q4_K [experts, hidden, inter].  Up to DECODE_TOKENS tokens
    take the decode products (llmp.vecq routed) instead of the tensor-core GEMM.  slabs: the
    experts' (gate_up, down) weights as q4k_relayout left them at load time, for the GEMM path."""
    tokens, used = ids.shape
    experts = gate_up.shape[0]
    # Few tokens: the decode products (routed llmp.vecq), which stream each named expert's
    # weights once per call, in calls of at most 128 tokens and 1,024 (token, slot) pairs (the
    # kernel's limits).  Up to DECODE_TOKENS tokens that beats the tensor-core GEMM, whose
    # 128-row tiles are nearly empty when an expert sees a handful of rows.
    chunk = min(128, max(1, 1024 // used))
    if tokens <= MOE_DECODE_TOKENS and (decode_tokens is None or decode_tokens > 0) and \
            x.dtype == torch.float32 and x.stride(-1) == 1 and moe_decode_fits(tokens, used, hidden, inter):
        return moe_decode(x, ids, weights if weights.is_contiguous() else weights.contiguous(),
                          gate_up, down, hidden, inter, glu)
    if tokens <= (DECODE_TOKENS if decode_tokens is None else decode_tokens) and used <= 128:
        gate_w = gate_up[:, :inter]
        up_w = gate_up[:, inter:]
        bpr = hidden // 256
        xf = x if x.dtype == torch.float32 else x.float()
        weights = weights if weights.is_contiguous() else weights.contiguous()
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=x.device)
        # Five launches a call of up to `chunk` tokens, nothing else queued: quantize, the routed
        # gate|up GLU product, quantize, the routed down product, the ordered combine (its rows
        # are already in slot order).
        for t0 in range(0, tokens, chunk):
            t1 = min(tokens, t0 + chunk)
            n = t1 - t0
            part_ids = ids[t0:t1]
            q8 = quantize_q8(xf[t0:t1])
            h = vecq(up_w, TYPE_Q4_K, hidden, inter, q8, n, ids=part_ids, gate=gate_w, glu=glu,
                     stride_row=bpr, stride_expert=2 * inter * bpr)
            q8h = quantize_q8(h.view(n * used, inter))
            y = vecq(down, TYPE_Q4_K, inter, hidden, q8h, n, ids=part_ids, per_slot=True)
            moe_combine(y.view(n * used, hidden), None, weights[t0:t1], n, used, out=out[t0:t1])
        return out
    route = moe_route(ids, experts)
    slots = tokens * used
    aq = mmq_quantize(x, ids_src=route["token"], cols=slots)
    if slabs is not None and len(slabs) > 2 and slabs[2] and inter % 128 == 0:
        # slabs[0] interleaves gate and up rows: the GLU and the requantization happen in the
        # gate | up product's write-back (no F32 round trip, no separate pass)
        hq = grouped_gemm_glu(aq, route["offsets"], hidden, inter, slabs[0], glu)
    else:
        gu = grouped_gemm(gate_up, aq, route["offsets"], hidden, 2 * inter,
                          slab=slabs[0] if slabs is not None else None)
        hq = moe_glu_quantize(gu, inter, glu)
    y = grouped_gemm(down, hq, route["offsets"], inter, hidden,
                     slab=slabs[1] if slabs is not None else None)
    return moe_combine(y, route["position"], weights.contiguous(), tokens, used)


def mxfp8_mul_mat_vec(codes: torch.Tensor, scales: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Mxfp8MulMatVec: codes uint8 [n, k], scales uint8 [n, k / 32] row-major, x F32
    [columns <= 16, k] -> F32 [columns, n]."""
    _need(codes, torch.uint8, "mxfp8_mul_mat_vec codes")
    _need(scales, torch.uint8, "mxfp8_mul_mat_vec scales")
    _need(x, torch.float32, "mxfp8_mul_mat_vec x")
    n, k = codes.shape
    cols = x.shape[0]
    if not codes.is_contiguous() or not scales.is_contiguous() or x.stride(1) != 1:
        raise Rejected("mxfp8_mul_mat_vec: packed codes and scales, k-contiguous activations")
    y = torch.empty((cols, n), dtype=torch.float32, device=codes.device)
    N.check(N.lib().llmp_b200_mxfp8_mul_mat_vec(codes.data_ptr(), scales.data_ptr(), x.data_ptr(),
                                                x.stride(0), y.data_ptr(), y.stride(0), n, k, cols,
                                                _stream()), "llmp_b200_mxfp8_mul_mat_vec")
    return y


# ------------------------------------------------------ decode module (F32 x)
DECODER_Q8_0, DECODER_MXFP8_SPLIT, DECODER_MXFP8_ATOMS = 0, 1, 2
DECODER_BF16, DECODER_F16, DECODER_NVFP4_SPLIT, DECODER_NVFP4_ATOMS = 3, 4, 5, 6
DECODER_MXFP4_SPLIT, DECODER_MXFP4_ATOMS = 7, 8


def _decode_operand(decoder: int, data: torch.Tensor, scales: torch.Tensor | None, k: int,
                    tensor_scale: torch.Tensor | None, rows_per_scale: int) -> "N.DecodeOperand":
    _need(data, torch.uint8, "decode_vector data")
    if data.dim() != 2 or data.stride(1) != 1:
        raise Rejected("decode_vector: data uint8 [rows, row_bytes]")
    op = N.DecodeOperand()
    op.data = data.data_ptr()
    op.scales = scales.data_ptr() if scales is not None else None
    op.tensor_scale = tensor_scale.data_ptr() if tensor_scale is not None else None
    op.k, op.rows, op.rows_per_scale, op.decoder = k, data.shape[0], rows_per_scale, decoder
    op.row_bytes = data.stride(0)
    return op


def decode_vector(decoder: int, data: torch.Tensor, x: torch.Tensor, k: int, outputs: int, *,
                  scales: torch.Tensor | None = None, first: int = 0,
                  up: torch.Tensor | None = None, up_scales: torch.Tensor | None = None,
                  up_first: int = 0, glu: int = GLU_NONE, limit: float = 0.0,
                  tensor_scale: torch.Tensor | None = None, rows_per_scale: int = 1,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """decode::RunVector / RunVectorGlu: data uint8 [n, row_bytes] (Q8_0 blocks or E4M3 codes
    with E8M0 scales), x F32 [rows <= 16, k] -> F32 [rows, outputs]; with `up` the GLU of the
    gate product (data) and the up product."""
    _need(x, torch.float32, "decode_vector x")
    if x.dim() != 2 or x.stride(1) != 1:
        raise Rejected("decode_vector: x F32 [rows, k], k contiguous")
    rows = x.shape[0]
    if out is None:
        out = torch.empty((rows, outputs), dtype=torch.float32, device=x.device)
    _need(out, torch.float32, "decode_vector output")
    gate_op = _decode_operand(decoder, data, scales, k, tensor_scale, rows_per_scale)
    if up is None:
        p = N.DecodeProduct()
        p.w, p.first, p.outputs = gate_op, first, outputs
        p.x, p.rows, p.x_stride = x.data_ptr(), rows, x.stride(0)
        p.y, p.y_stride = out.data_ptr(), out.stride(0)
        N.check(N.lib().llmp_b200_decode_vector(C.byref(p), _stream()), "llmp_b200_decode_vector")
        return out
    g = N.DecodeGluProduct()
    g.gate, g.gate_first = gate_op, first
    g.up = _decode_operand(decoder, up, up_scales, k, tensor_scale, rows_per_scale)
    g.up_first, g.outputs, g.glu, g.limit = up_first, outputs, glu, limit
    g.x, g.rows, g.x_stride = x.data_ptr(), rows, x.stride(0)
    g.y, g.y_stride = out.data_ptr(), out.stride(0)
    N.check(N.lib().llmp_b200_decode_vector_glu(C.byref(g), _stream()),
            "llmp_b200_decode_vector_glu")
    return out


def decode_rows(decoder: int, data: torch.Tensor, ids: torch.Tensor, k: int, *,
                scales: torch.Tensor | None = None, tensor_scale: torch.Tensor | None = None,
                rows_per_scale: int = 1, bad: torch.Tensor | None = None) -> torch.Tensor:
    """decode::RunRows: the decoded rows ids[i] of data uint8 [n, row_bytes] -> F32 [count, k]
    (an id outside the matrix gives a zero row and sets bad[0], an I32 tensor, to 1)."""
    _need(ids, torch.int32, "decode_rows ids")
    op = _decode_operand(decoder, data, scales, k, tensor_scale, rows_per_scale)
    out = torch.empty((ids.numel(), k), dtype=torch.float32, device=data.device)
    if bad is not None:
        _need(bad, torch.int32, "decode_rows bad flag")
    N.check(N.lib().llmp_b200_decode_rows(C.byref(op), ids.data_ptr(), ids.numel(), out.data_ptr(),
                                          out.stride(0), bad.data_ptr() if bad is not None else None,
                                          _stream()), "llmp_b200_decode_rows")
    return out


def decode_matrix(decoder: int, data: torch.Tensor, x: torch.Tensor, k: int, outputs: int, *,
                  scales: torch.Tensor | None = None, first: int = 0,
                  tensor_scale: torch.Tensor | None = None, rows_per_scale: int = 1,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """decode::RunMatrix (MMA path): data uint8 [n, row_bytes], x F32 [rows, k] (any rows) ->
    F32 [rows, outputs]; operands rounded to FP16 (Q8_0) or BF16 (MXFP8), F32 accumulation."""
    _need(x, torch.float32, "decode_matrix x")
    if x.dim() != 2 or x.stride(1) != 1:
        raise Rejected("decode_matrix: x F32 [rows, k], k contiguous")
    rows = x.shape[0]
    if out is None:
        out = torch.empty((rows, outputs), dtype=torch.float32, device=x.device)
    _need(out, torch.float32, "decode_matrix output")
    p = N.DecodeProduct()
    p.w = _decode_operand(decoder, data, scales, k, tensor_scale, rows_per_scale)
    p.first, p.outputs = first, outputs
    p.x, p.rows, p.x_stride = x.data_ptr(), rows, x.stride(0)
    p.y, p.y_stride = out.data_ptr(), out.stride(0)
    N.check(N.lib().llmp_b200_decode_matrix(C.byref(p), _stream()), "llmp_b200_decode_matrix")
    return out


def decode_grouped(decoder: int, data: torch.Tensor, x: torch.Tensor, k: int, outputs: int,
                   offsets: torch.Tensor, pair_rows: torch.Tensor, y_rows: int, *,
                   scales: torch.Tensor | None = None, pair_out: torch.Tensor | None = None,
                   first: int = 0) -> torch.Tensor:
    """decode::RunGrouped: data uint8 [experts, n, row_bytes] (scales [experts, ...] likewise),
    offsets I32 [experts + 1] over the pairs, pair_rows I32 [pairs] naming x rows, pair_out I32
    [pairs] naming y rows (or the pair index) -> F32 [y_rows, outputs] (rows no pair writes stay
    zero)."""
    import numpy as np
    _need(data, torch.uint8, "decode_grouped data")
    _need(x, torch.float32, "decode_grouped x")
    _need(offsets, torch.int32, "decode_grouped offsets")
    _need(pair_rows, torch.int32, "decode_grouped pair_rows")
    experts, n = data.shape[0], data.shape[1]
    table = np.zeros((experts, 6), np.uint64)     # llmp_b200_decode_operand, 48 bytes each
    for e in range(experts):
        table[e, 0] = data[e].data_ptr()
        table[e, 1] = scales[e].data_ptr() if scales is not None else 0
        table[e, 3] = k | (n << 32)
        table[e, 4] = 1 | (decoder << 32)
        table[e, 5] = data.stride(1)
    operands = torch.from_numpy(table.view(np.uint8).reshape(-1)).to(x.device)
    out = torch.zeros((y_rows, outputs), dtype=torch.float32, device=x.device)
    g = N.DecodeGroupedProduct()
    g.format.k, g.format.rows, g.format.rows_per_scale, g.format.decoder = k, n, 1, decoder
    g.format.row_bytes = data.stride(1)
    g.experts, g.experts_count = operands.data_ptr(), experts
    g.first, g.outputs = first, outputs
    g.offsets, g.pair_rows = offsets.data_ptr(), pair_rows.data_ptr()
    g.pair_out = pair_out.data_ptr() if pair_out is not None else None
    g.pairs = pair_rows.numel()
    g.x, g.x_rows, g.x_stride = x.data_ptr(), x.shape[0], x.stride(0)
    g.y, g.y_rows, g.y_stride = out.data_ptr(), y_rows, out.stride(0)
    N.check(N.lib().llmp_b200_decode_grouped(C.byref(g), _stream()), "llmp_b200_decode_grouped")
    torch.cuda.current_stream().synchronize()     # the operand table lives until here
    return out
