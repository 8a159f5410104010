"""ctypes/numpy binding of the CPU oracle (oracle/oracle.c).

TEST INFRASTRUCTURE: imported only by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")

Q8_0, Q8_1, Q4_K = 8, 9, 12
Q4_0, Q5_0, Q5_K, Q6_K, IQ4_NL = 2, 6, 13, 14, 20      # decoders only (orc_dequant_more)
GLU_NONE, GLU_SWIGLU, GLU_SWIGLU_CLAMP, GLU_GEGLU = 0, 1, 2, 3


def build(force: bool = False) -> str:
    """Compiles the oracle with gcc (oracle/Makefile) if the library is stale."""
    src = [os.path.join(_HERE, f) for f in ("oracle.c", "oracle.h", "Makefile")]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src)
    if stale:
        subprocess.run(["make", "-C", _HERE, "CC=gcc"], check=True, capture_output=True)
    return _LIB_PATH


class VecQDesc(C.Structure):
    _fields_ = [("w", C.c_void_p), ("g", C.c_void_p), ("y", C.c_void_p), ("ids", C.c_void_p),
                ("dst", C.c_void_p)] + [(n, C.c_int) for n in (
                    "ncols_x", "nrows", "stride_row", "stride_expert", "y_token", "y_slot",
                    "ids_stride", "used", "tokens", "dst_token", "dst_slot", "glu")] + [
                        ("limit", C.c_float)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_bf16_to_f32.restype = C.c_float
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_e4m3_to_f32.restype = C.c_float
        L.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_e8m0_to_f32.restype = C.c_float
        L.orc_e8m0_to_f32.argtypes = [C.c_uint8]
        L.orc_f32_to_e4m3_satfinite.restype = C.c_uint8
        L.orc_f32_to_e4m3_satfinite.argtypes = [C.c_float]
        L.orc_q8_padded.restype = C.c_int64
        L.orc_q8_padded.argtypes = [C.c_int64]
        L.orc_q8_row_blocks.restype = C.c_int64
        L.orc_q8_row_blocks.argtypes = [C.c_int64]
        L.orc_q8_0_block_product.restype = C.c_double
        L.orc_q8_0_block_product.argtypes = [C.c_void_p, C.c_void_p]
        L.orc_q4_k_block_product.restype = C.c_double
        L.orc_q4_k_block_product.argtypes = [C.c_void_p, C.c_void_p]
        L.orc_glu.restype = C.c_float
        L.orc_glu.argtypes = [C.c_int, C.c_float, C.c_float, C.c_float]
        L.orc_vecq.restype = C.c_int
        L.orc_vecq.argtypes = [C.c_int, C.POINTER(VecQDesc), C.c_void_p, C.c_void_p, C.c_int]
        L.orc_mxfp8_scale_code.restype = C.c_uint32
        L.orc_mxfp8_scale_code.argtypes = [C.c_float]
        L.orc_scale_atom_offset.restype = C.c_uint64
        L.orc_scale_atom_offset.argtypes = [C.c_uint64] * 3
        L.orc_mxfp8_rows_scales_offset.restype = C.c_uint64
        L.orc_mxfp8_rows_scales_offset.argtypes = [C.c_uint64] * 2
        L.orc_mxfp8_rows_bytes.restype = C.c_uint64
        L.orc_mxfp8_rows_bytes.argtypes = [C.c_uint64] * 2
        L.orc_moe_route_ints.restype = C.c_int64
        L.orc_moe_route_ints.argtypes = [C.c_int64] * 3
        for name, args in {
            "orc_dequant_q8_0": [C.c_void_p, C.c_int64, C.c_void_p],
            "orc_dequant_q4_k": [C.c_void_p, C.c_int64, C.c_void_p],
            "orc_dequant_q8_1": [C.c_void_p, C.c_int64, C.c_void_p],
            "orc_dequant_more": [C.c_int, C.c_void_p, C.c_int64, C.c_void_p],
            "orc_q4_k_scales": [C.c_void_p, C.c_void_p, C.c_void_p],
            "orc_quantize_q8_1": [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p],
            "orc_q8_0_block_sums": [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p],
            "orc_q4_k_block_sums": [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p],
            "orc_quantize_mmq_q8_1_ds4": [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                          C.c_void_p],
            "orc_mmq_q4_k": [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                             C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                             C.c_void_p, C.c_int],
            "orc_mxfp8_quantize": [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                   C.c_void_p],
            "orc_mxfp8_swizzle": [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64],
            "orc_mxfp8_dequant": [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p],
            "orc_mxfp8_gemm": [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                               C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int],
            "orc_decode_vector": [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                  C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                  C.c_int, C.c_float, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p,
                                  C.c_int64],
            "orc_mmq_block_sums": [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                   C.c_void_p],
            "orc_decode_rows": [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p],
            "orc_moe_route": [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p],
            "orc_moe_combine": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                C.c_void_p],
        }.items():
            getattr(L, name).restype = None
            getattr(L, name).argtypes = args
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# ----------------------------------------------------------------- geometry
def block_bytes(t):
    return {Q8_0: 34, Q8_1: 36, Q4_K: 144, Q4_0: 18, IQ4_NL: 18, Q5_0: 22, Q5_K: 176, Q6_K: 210}[t]


def block_elems(t):
    return {Q8_0: 32, Q8_1: 32, Q4_K: 256, Q4_0: 32, IQ4_NL: 32, Q5_0: 32, Q5_K: 256, Q6_K: 256}[t]


def q8_row_blocks(k):
    return int(lib().orc_q8_row_blocks(k))


# ----------------------------------------------------------------- decode
def dequant(t, blocks: np.ndarray) -> np.ndarray:
    blocks = _c(blocks, np.uint8).reshape(-1)
    nb = blocks.size // block_bytes(t)
    out = np.empty(nb * block_elems(t), np.float32)
    if t in (Q4_0, Q5_0, Q5_K, Q6_K, IQ4_NL):
        lib().orc_dequant_more(t, _p(blocks), nb, _p(out))
        return out
    fn = {Q8_0: lib().orc_dequant_q8_0, Q4_K: lib().orc_dequant_q4_k, Q8_1: lib().orc_dequant_q8_1}[t]
    fn(_p(blocks), nb, _p(out))
    return out


def quantize_q8_1(x: np.ndarray) -> np.ndarray:
    """x F32 [rows, k] -> uint8 [rows, q8_row_blocks(k) * 36]."""
    x = _c(x, np.float32)
    rows, k = x.shape
    out = np.empty((rows, q8_row_blocks(k) * 36), np.uint8)
    lib().orc_quantize_q8_1(_p(x), k, rows, k, _p(out))
    return out


def block_sums(t, w_row: np.ndarray, y_row: np.ndarray, k: int):
    w_row, y_row = _c(w_row, np.uint8), _c(y_row, np.uint8)
    if t == Q8_0:
        s = np.empty(k // 32, np.int32)
        lib().orc_q8_0_block_sums(_p(w_row), _p(y_row), k, _p(s))
        return s, None
    d = np.empty(k // 32, np.int32)
    q = np.empty(k // 32, np.int32)
    lib().orc_q4_k_block_sums(_p(w_row), _p(y_row), k, _p(d), _p(q))
    return d, q


def vecq(t, w, y, k, nrows, tokens, *, g=None, ids=None, used=1, stride_row=None,
         stride_expert=0, y_token=None, y_slot=0, glu=GLU_NONE, limit=0.0, want64=False,
         threads=None):
    """Mirrors llmp.vecq.  Returns F32 [tokens, used, nrows] (+ f64 sum, f64 |sum|)."""
    w = _c(w, np.uint8)
    y = _c(y, np.uint8)
    bpr = k // block_elems(t)
    d = VecQDesc()
    gg = None if g is None else _c(g, np.uint8)
    ii = None if ids is None else _c(ids, np.int32)
    dst = np.full((tokens, used, nrows), np.nan, np.float32)
    d.w, d.g, d.y = w.ctypes.data, (gg.ctypes.data if gg is not None else None), y.ctypes.data
    d.ids = ii.ctypes.data if ii is not None else None
    d.dst = dst.ctypes.data
    d.ncols_x, d.nrows = k, nrows
    d.stride_row = bpr if stride_row is None else stride_row
    d.stride_expert = stride_expert
    d.y_token = q8_row_blocks(k) * (used if y_slot else 1) if y_token is None else y_token
    d.y_slot = y_slot
    d.ids_stride = used if ids is not None else 0
    d.used, d.tokens = used, tokens
    d.dst_token, d.dst_slot = used * nrows, nrows
    d.glu, d.limit = glu, limit
    s64 = np.zeros(dst.shape, np.float64) if want64 else None
    a64 = np.zeros(dst.shape, np.float64) if want64 else None
    rc = lib().orc_vecq(t, C.byref(d), _p(s64), _p(a64), threads or host_threads())
    assert rc == 0
    return (dst, s64, a64) if want64 else dst


def glu(kind, gate, up, limit=0.0):
    return float(lib().orc_glu(kind, float(gate), float(up), float(limit)))


# ----------------------------------------------------------------- MMQ
def quantize_mmq_q8_1(x: np.ndarray, ids_src=None, cols=None) -> np.ndarray:
    """x F32 [rows, k] -> uint8 [k/128, cols, 144] (DS4 layout)."""
    x = _c(x, np.float32)
    rows, k = x.shape
    ii = None if ids_src is None else _c(ids_src, np.int32)
    cols = (rows if ii is None else ii.size) if cols is None else cols
    out = np.zeros((k // 128, cols, 144), np.uint8)
    lib().orc_quantize_mmq_q8_1_ds4(_p(x), k, cols, k, _p(ii), _p(out))
    return out


def mmq_q4_k(w, yq, k, n, *, ncols=None, stride_row=None, stride_expert=0, ids_dst=None,
             expert_bounds=None, out_cols=None, want64=False, threads=None):
    """Returns F32 [out_cols, n]: D[col, row]."""
    w, yq = _c(w, np.uint8), _c(yq, np.uint8)
    ncols = yq.shape[1] if ncols is None else ncols
    out_cols = ncols if out_cols is None else out_cols
    dst = np.full((out_cols, n), np.nan, np.float32)
    d64 = np.zeros((out_cols, n), np.float64) if want64 else None
    ii = None if ids_dst is None else _c(ids_dst, np.int32)
    eb = None if expert_bounds is None else _c(expert_bounds, np.int32)
    lib().orc_mmq_q4_k(_p(w), k // 256 if stride_row is None else stride_row, stride_expert,
                       _p(yq), ncols, _p(ii), _p(eb), 0 if eb is None else eb.size - 1, _p(dst), n,
                       k, n, _p(d64), threads or host_threads())
    return (dst, d64) if want64 else dst


# ----------------------------------------------------------------- MXFP8
def atom_offset(row, block, blocks):
    return int(lib().orc_scale_atom_offset(row, block, blocks))


def mxfp8_quantize(x: np.ndarray, is_bf16=False):
    """x [rows, k] F32 (or uint16 BF16 bits) -> (codes [rows,k] u8, scale atoms u8)."""
    x = _c(x, np.uint16 if is_bf16 else np.float32)
    rows, k = x.shape
    codes = np.empty((rows, k), np.uint8)
    scales = np.full(((rows + 127) // 128 * 128) * (k // 32), 0xAA, np.uint8)
    lib().orc_mxfp8_quantize(_p(x), int(is_bf16), k, k, rows, _p(codes), _p(scales))
    return codes, scales


def mxfp8_swizzle(scales: np.ndarray) -> np.ndarray:
    scales = _c(scales, np.uint8)
    n, blocks = scales.shape
    out = np.full(((n + 127) // 128 * 128) * blocks, 0xAA, np.uint8)
    lib().orc_mxfp8_swizzle(_p(scales), _p(out), n, blocks)
    return out


def mxfp8_dequant(codes, atoms):
    codes, atoms = _c(codes, np.uint8), _c(atoms, np.uint8)
    rows, k = codes.shape
    out = np.empty((rows, k), np.float32)
    lib().orc_mxfp8_dequant(_p(codes), _p(atoms), rows, k, _p(out))
    return out


def mxfp8_gemm(a, a_atoms, b, b_atoms, bf16=False, want64=False, threads=None):
    a, b = _c(a, np.uint8), _c(b, np.uint8)
    m, k = a.shape
    n = b.shape[0]
    d = np.empty((m, n), np.uint16 if bf16 else np.float32)
    d64 = np.empty((m, n), np.float64) if want64 else None
    lib().orc_mxfp8_gemm(m, n, k, _p(a), _p(_c(a_atoms, np.uint8)), _p(b), _p(_c(b_atoms, np.uint8)),
                         _p(d), int(bf16), _p(d64), threads or host_threads())
    return (d, d64) if want64 else d


# ----------------------------------------------------------------- MoE
def moe_route(ids: np.ndarray, experts: int):
    """ids I32 [tokens, used] -> dict of the route blob's parts."""
    ids = _c(ids, np.int32)
    tokens, used = ids.shape
    n = int(lib().orc_moe_route_ints(experts, used, tokens))
    out = np.empty(n, np.int32)
    lib().orc_moe_route(_p(ids), used, experts, used, tokens, _p(out))
    slots = tokens * used
    e1 = experts + 1
    return {"blob": out, "offsets": out[:e1], "scale_rows": out[e1:2 * e1],
            "position": out[2 * e1:2 * e1 + slots], "token": out[2 * e1 + slots:2 * e1 + 2 * slots],
            "expert": out[2 * e1 + 2 * slots:2 * e1 + 3 * slots], "counts": out[2 * e1 + 3 * slots:]}


def moe_combine(rows, position, weights, tokens, used):
    rows = _c(rows, np.float32)
    width = rows.shape[1]
    dst = np.empty((tokens, width), np.float32)
    lib().orc_moe_combine(_p(rows), _p(_c(position, np.int32)), _p(_c(weights, np.float32)), used,
                          tokens, width, _p(dst))
    return dst


DECODER_Q8_0, DECODER_MXFP8_SPLIT, DECODER_MXFP8_ATOMS = 0, 1, 2


def decode_vector(decoder, data, x, k, outputs, *, scales=None, first=0, up=None, up_scales=None,
                  up_first=0, glu=-1, limit=0.0, tensor_scale=None, rows_per_scale=1):
    """The decode module's vector product (or GLU product with `up`): data uint8 [n, row_bytes],
    x F32 [rows, k] -> F32 [rows, outputs]."""
    data = np.ascontiguousarray(data, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows = x.shape[0]
    y = np.empty((rows, outputs), np.float32)
    hold = [None if a is None else np.ascontiguousarray(a, dtype=np.uint8)
            for a in (scales, up, up_scales)]
    ts = None if tensor_scale is None else np.ascontiguousarray(tensor_scale, dtype=np.float32)
    lib().orc_decode_vector(decoder, _p(data), _p(hold[0]) if hold[0] is not None else None,
                            data.shape[1], _p(hold[1]) if hold[1] is not None else None,
                            _p(hold[2]) if hold[2] is not None else None, k,
                            _p(ts) if ts is not None else None, rows_per_scale, first, up_first,
                            outputs, glu, limit, _p(x), rows, x.shape[1], _p(y), outputs)
    return y


def decode_rows(decoder, data, ids, k, *, scales=None, tensor_scale=None, rows_per_scale=1):
    """decode::RunRows: the decoded rows ids[i] of data uint8 [n, row_bytes] -> (F32 [count, k],
    bad flag)."""
    data = np.ascontiguousarray(data, dtype=np.uint8)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    sc = None if scales is None else np.ascontiguousarray(scales, dtype=np.uint8)
    ts = None if tensor_scale is None else np.ascontiguousarray(tensor_scale, dtype=np.float32)
    y = np.empty((ids.size, k), np.float32)
    bad = np.zeros(1, np.int32)
    lib().orc_decode_rows(decoder, _p(data), _p(sc) if sc is not None else None, data.shape[1], k,
                          data.shape[0], _p(ts) if ts is not None else None, rows_per_scale,
                          _p(ids), ids.size, _p(y), _p(bad))
    return y, int(bad[0])


def mmq_block_sums(w, yq, k, n):
    """The exact int32 group sums of the dense MMQ: I32 [cols, n, k / 32]."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    yq = np.ascontiguousarray(yq, dtype=np.uint8)
    cols = yq.shape[1]
    sums = np.empty((cols, n, k // 32), np.int32)
    lib().orc_mmq_block_sums(_p(w), k // 256, _p(yq), cols, k, n, _p(sums))
    return sums
