"""ctypes binding of libllmp_b200.so.  There is no fallback: importing the
operators without the built library raises."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_lib", "libllmp_b200.so")

OK, REJECTED, NO_DEVICE = 0, 1, 2
TYPE_Q8_0, TYPE_Q8_1, TYPE_Q4_K = 8, 9, 12
GLU_NONE, GLU_SWIGLU, GLU_SWIGLU_CLAMP, GLU_GEGLU = 0, 1, 2, 3


class NativeLibraryMissing(ImportError):
    pass


class Rejected(ValueError):
    """Status > 0: the call was refused before anything was queued."""


class LaunchFailed(RuntimeError):
    """Status < 0: a CUDA call failed after work may have been queued."""


class VecQDesc(C.Structure):
    """llmp_b200_vecq_desc (include/llmp_b200.h)."""
    _fields_ = [("w", C.c_void_p), ("g", C.c_void_p), ("y", C.c_void_p), ("ids", C.c_void_p),
                ("dst", C.c_void_p)] + [(n, C.c_int) for n in (
                    "ncols_x", "nrows", "stride_row", "stride_expert", "y_token", "y_slot",
                    "ids_stride", "used", "tokens", "dst_token", "dst_slot", "glu")] + [
                        ("limit", C.c_float)]


class PeerSite(C.Structure):
    """llmp_b200_peer_site (include/llmp_b200.h)."""
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("buffers", C.c_void_p),
                ("flags", C.c_void_p), ("step", C.c_void_p), ("site", C.c_int)]


class PeerFan(C.Structure):
    """llmp_b200_peer_fan (include/llmp_b200.h)."""
    _fields_ = [("world", C.c_int), ("words", C.c_void_p), ("step", C.c_void_p), ("base", C.c_int),
                ("tag", C.c_int)]


class MoeDecodeDesc(C.Structure):
    """llmp_b200_moe_decode_desc (include/llmp_b200.h)."""
    _fields_ = [("x", C.c_void_p), ("x_stride", C.c_int64), ("ids", C.c_void_p), ("ids_stride", C.c_int),
                ("weights", C.c_void_p), ("gate_up", C.c_void_p), ("down", C.c_void_p),
                ("experts", C.c_int), ("used", C.c_int), ("tokens", C.c_int), ("hidden", C.c_int),
                ("inter", C.c_int), ("glu", C.c_int), ("limit", C.c_float), ("dst", C.c_void_p),
                ("dst_stride", C.c_int64), ("scratch", C.c_void_p)]


class MmvqDesc(C.Structure):
    """llmp_b200_mmvq_desc (include/llmp_b200.h)."""
    _fields_ = [("type", C.c_int), ("w", C.c_void_p), ("gate", C.c_void_p), ("glu", C.c_int),
                ("limit", C.c_float), ("x", C.c_void_p), ("x_col_stride", C.c_int64),
                ("q8", C.c_void_p), ("dst", C.c_void_p), ("dst_col_stride", C.c_int64),
                ("k", C.c_int), ("n", C.c_int), ("cols", C.c_int), ("stride_row", C.c_int),
                ("scratch", C.c_void_p)]


class DecodeOperand(C.Structure):
    _fields_ = [("data", C.c_void_p), ("scales", C.c_void_p), ("tensor_scale", C.c_void_p),
                ("k", C.c_uint32), ("rows", C.c_uint32), ("rows_per_scale", C.c_uint32),
                ("decoder", C.c_uint32), ("row_bytes", C.c_uint64)]


class DecodeProduct(C.Structure):
    _fields_ = [("w", DecodeOperand), ("first", C.c_uint64), ("outputs", C.c_uint64),
                ("x", C.c_void_p), ("rows", C.c_uint64), ("x_stride", C.c_uint64),
                ("y", C.c_void_p), ("y_stride", C.c_uint64)]


class DecodeGroupedProduct(C.Structure):
    _fields_ = [("format", DecodeOperand), ("experts", C.c_void_p), ("experts_count", C.c_uint64),
                ("first", C.c_uint64), ("outputs", C.c_uint64), ("offsets", C.c_void_p),
                ("pair_rows", C.c_void_p), ("pair_out", C.c_void_p), ("pairs", C.c_uint64),
                ("x", C.c_void_p), ("x_rows", C.c_uint64), ("x_stride", C.c_uint64),
                ("y", C.c_void_p), ("y_rows", C.c_uint64), ("y_stride", C.c_uint64)]


class DecodeGluProduct(C.Structure):
    _fields_ = [("gate", DecodeOperand), ("gate_first", C.c_uint64), ("up", DecodeOperand),
                ("up_first", C.c_uint64), ("outputs", C.c_uint64), ("glu", C.c_int),
                ("limit", C.c_float), ("x", C.c_void_p), ("rows", C.c_uint64),
                ("x_stride", C.c_uint64), ("y", C.c_void_p), ("y_stride", C.c_uint64)]


class Mxfp8GemmDesc(C.Structure):
    """llmp_b200_mxfp8_gemm_desc (include/llmp_b200.h)."""
    _fields_ = [("m", C.c_int), ("n", C.c_int), ("k", C.c_int), ("a", C.c_void_p),
                ("a_scales", C.c_void_p), ("b", C.c_void_p), ("b_scales", C.c_void_p),
                ("d", C.c_void_p), ("bf16", C.c_int), ("scratch", C.c_void_p)]


class MmqDesc(C.Structure):
    """llmp_b200_mmq_desc (include/llmp_b200.h)."""
    _fields_ = [("type", C.c_int), ("w", C.c_void_p), ("y", C.c_void_p), ("ids_dst", C.c_void_p),
                ("expert_bounds", C.c_void_p), ("dst", C.c_void_p), ("k", C.c_int),
                ("nrows", C.c_int), ("ncols", C.c_int), ("stride_row", C.c_int),
                ("stride_expert", C.c_int), ("dst_col_stride", C.c_int), ("experts", C.c_int),
                ("max_cols_per_expert", C.c_int), ("w_slab", C.c_void_p), ("scratch", C.c_void_p)]


class GroupedGemmDesc(C.Structure):
    """llmp_b200_grouped_gemm_desc (include/llmp_b200.h)."""
    _fields_ = [("groups", C.c_int), ("n", C.c_int), ("k", C.c_int), ("rows", C.c_int),
                ("offsets", C.c_void_p), ("a", C.c_void_p), ("weights", C.c_void_p),
                ("expert_stride", C.c_uint64), ("d", C.c_void_p), ("scratch", C.c_void_p),
                ("weights_slab", C.c_void_p)]


# name -> (restype, argtypes): every symbol include/llmp_b200.h declares.
SIGNATURES = {
    "llmp_b200_available": (C.c_int, []),
    "llmp_b200_sm_count": (C.c_int, []),
    "llmp_b200_last_error": (C.c_char_p, []),
    "llmp_b200_wait_selftest": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p]),
    "llmp_b200_device_faults": (C.c_int, []),
    "llmp_b200_device_faults_clear": (C.c_int, []),
    "llmp_b200_q8_1_row_blocks": (C.c_int64, [C.c_int64]),
    "llmp_b200_q8_1_quantize": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                          C.c_int64, C.c_void_p, C.c_void_p]),
    "llmp_b200_q8_1_quantize_gathered": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                                   C.c_void_p, C.POINTER(PeerSite), C.c_void_p,
                                                   C.c_int, C.c_void_p, C.c_void_p]),
    "llmp_b200_q8_1_quantize_exchange": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p,
                                                   C.POINTER(PeerSite), C.c_void_p, C.c_void_p,
                                                   C.c_size_t, C.c_size_t, C.c_int, C.c_void_p,
                                                   C.c_void_p]),
    "llmp_b200_vecq_fan": (C.c_int, [C.c_int, C.POINTER(VecQDesc), C.c_int, C.POINTER(PeerFan),
                                     C.c_void_p]),
    "llmp_b200_q8_1_quantize_words": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64,
                                                C.c_void_p, C.c_int64, C.c_int, C.c_void_p,
                                                C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "llmp_b200_moe_decode_scratch": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "llmp_b200_moe_decode": (C.c_int, [C.POINTER(MoeDecodeDesc), C.c_void_p]),
    "llmp_b200_peer_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "llmp_b200_peer_free": (C.c_int, [C.c_void_p]),
    "llmp_b200_peer_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "llmp_b200_peer_import": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "llmp_b200_peer_close": (C.c_int, [C.c_void_p]),
    "llmp_b200_peer_begin_step": (C.c_int, [C.c_void_p, C.c_void_p]),
    "llmp_b200_peer_publish": (C.c_int, [C.POINTER(PeerSite), C.c_void_p, C.c_size_t, C.c_size_t,
                                         C.c_void_p]),
    "llmp_b200_peer_wait": (C.c_int, [C.POINTER(PeerSite), C.c_void_p, C.c_int, C.c_void_p,
                                      C.c_void_p]),
    "llmp_b200_vecq_variants": (C.c_int, []),
    "llmp_b200_vecq_variant_name": (C.c_char_p, [C.c_int]),
    "llmp_b200_vecq_rank_count": (C.c_int, []),
    "llmp_b200_vecq_rank": (C.c_char_p, [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                         C.POINTER(C.c_int), C.POINTER(C.c_int),
                                         C.POINTER(C.c_float)]),
    "llmp_b200_vecq": (C.c_int, [C.c_int, C.POINTER(VecQDesc), C.c_int, C.c_void_p]),
    "llmp_b200_mmq_q8_1_bytes": (C.c_int64, [C.c_int64, C.c_int64]),
    "llmp_b200_mmq_quantize": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64,
                                         C.c_void_p, C.c_void_p, C.c_void_p]),
    "llmp_b200_mmq_scratch": (C.c_size_t, [C.POINTER(MmqDesc), C.c_int]),
    "llmp_b200_mmq": (C.c_int, [C.POINTER(MmqDesc), C.c_int, C.c_void_p]),
    "llmp_b200_mmq_block_sums": (C.c_int, [C.POINTER(MmqDesc), C.c_void_p, C.c_void_p]),
    "llmp_b200_q4k_slab_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "llmp_b200_q4k_relayout": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int,
                                         C.c_void_p, C.c_void_p]),
    "llmp_b200_moe_route_ints": (C.c_int64, [C.c_int, C.c_int, C.c_int]),
    "llmp_b200_moe_route": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                      C.c_void_p]),
    "llmp_b200_grouped_gemm_available": (C.c_int, []),
    "llmp_b200_grouped_gemm_scratch": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "llmp_b200_grouped_gemm": (C.c_int, [C.POINTER(GroupedGemmDesc), C.c_int, C.c_void_p]),
    "llmp_b200_grouped_gemm_glu": (C.c_int, [C.POINTER(GroupedGemmDesc), C.c_int, C.c_float,
                                             C.c_void_p, C.c_int, C.c_void_p]),
    "llmp_b200_mmq_glu": (C.c_int, [C.POINTER(MmqDesc), C.c_int, C.c_float, C.c_void_p, C.c_void_p]),
    "llmp_b200_q4k_relayout_glu": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64,
                                             C.c_int, C.c_void_p, C.c_void_p]),
    "llmp_b200_grouped_gemm_static": (C.c_int, [C.POINTER(GroupedGemmDesc), C.c_int, C.c_void_p]),
    "llmp_b200_moe_glu_quantize": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_int64, C.c_int,
                                             C.c_float, C.c_void_p, C.c_void_p]),
    "llmp_b200_moe_ep_pack": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_int, C.c_int,
                                        C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llmp_b200_moe_combine": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int,
                                        C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "llmp_b200_mxfp8_padded_rows": (C.c_uint64, [C.c_uint64]),
    "llmp_b200_mxfp8_scale_offset": (C.c_uint64, [C.c_uint64, C.c_uint64, C.c_uint64]),
    "llmp_b200_mxfp8_quantize": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int,
                                           C.c_void_p, C.c_void_p, C.c_void_p]),
    "llmp_b200_mxfp8_swizzle": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "llmp_b200_mxfp8_mul_mat_vec": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                              C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int,
                                              C.c_void_p]),
    "llmp_b200_mxfp8_gemm_available": (C.c_int, []),
    "llmp_b200_mxfp8_gemm_scratch": (C.c_size_t, [C.POINTER(Mxfp8GemmDesc), C.c_int]),
    "llmp_b200_mxfp8_gemm": (C.c_int, [C.POINTER(Mxfp8GemmDesc), C.c_int, C.c_void_p]),
    "llmp_b200_mxfp8_gemm_resident_pairs": (C.c_int, []),
    "llmp_b200_mxfp8_gemm_variant": (C.c_int, [C.POINTER(Mxfp8GemmDesc), C.c_int, C.c_int, C.c_void_p]),
    "llmp_b200_decode_vector": (C.c_int, [C.POINTER(DecodeProduct), C.c_void_p]),
    "llmp_b200_decode_vector_glu": (C.c_int, [C.POINTER(DecodeGluProduct), C.c_void_p]),
    "llmp_b200_decode_rows": (C.c_int, [C.POINTER(DecodeOperand), C.c_void_p, C.c_uint64,
                                        C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]),
    "llmp_b200_decode_matrix": (C.c_int, [C.POINTER(DecodeProduct), C.c_void_p]),
    "llmp_b200_decode_grouped": (C.c_int, [C.POINTER(DecodeGroupedProduct), C.c_void_p]),
    "llmp_b200_mmvq_scratch": (C.c_size_t, [C.c_int, C.c_int]),
    "llmp_b200_mmvq": (C.c_int, [C.POINTER(MmvqDesc), C.c_void_p]),
    "llmp_b200_mmvq_prepared": (C.c_int, [C.POINTER(MmvqDesc), C.c_void_p]),
    "llmp_b200_mmvq_rows": (C.c_int, [C.POINTER(MmvqDesc), C.c_void_p]),
    "llmp_b200_vecq_f32": (C.c_int, [C.c_int, C.POINTER(VecQDesc), C.c_void_p, C.c_void_p]),
    "llmp_b200_vecq_q8_scratch": (C.c_size_t, [C.c_int, C.c_int]),
    "llmp_b200_vecq_q8": (C.c_int, [C.c_int, C.POINTER(VecQDesc), C.c_void_p, C.c_void_p,
                                    C.c_void_p]),
    "llmp_b200_vecq_block_sums": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                            C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NativeLibraryMissing(
                f"{LIB_PATH} is not built: run `python -c 'import __graft_entry__ as g; g.build()'` "
                "or `make -C llmp_b200/csrc`. llmp_b200 has no fallback path.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return (lib().llmp_b200_last_error() or b"").decode()


def check(status: int, what: str) -> None:
    if status == 0:
        return
    if status > 0:
        raise Rejected(f"{what}: status {status}: {last_error()}")
    raise LaunchFailed(f"{what}: status {status}: {last_error()}")
