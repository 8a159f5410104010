"""Generates tests/golden/*.npz.  Run in the build container, where the
reference tree and the gguf package are present:

    python tests/golden/make_golden.py [/path/to/llmp]

Sources of truth recorded here (none is the oracle itself):
  * libref.so: the reference's OWN src/format and src/kernels/reference
    sources compiled by `make -C oracle ref` (element conversions, scale-atom
    offsets, block geometry, DecodeRows of MXFP8 / Q8_1);
  * gguf (llama.cpp's gguf-py, third party): Q8_0 quantize + dequantize and
    Q4_K dequantize, a secondary cross-check of the block decoders.
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from llmp_b200 import synth  # noqa: E402


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
        "LLMP_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "ref", "CXX=g++",
                    f"REFERENCE={ref_root}"], check=True)
    R = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref.so"))
    R.ref_f16_to_f32.restype = C.c_float
    R.ref_f16_to_f32.argtypes = [C.c_uint16]
    R.ref_f32_to_f16.restype = C.c_uint16
    R.ref_f32_to_f16.argtypes = [C.c_float]
    R.ref_bf16_to_f32.restype = C.c_float
    R.ref_bf16_to_f32.argtypes = [C.c_uint16]
    R.ref_f32_to_bf16.restype = C.c_uint16
    R.ref_f32_to_bf16.argtypes = [C.c_float]
    R.ref_e4m3_to_f32.restype = C.c_float
    R.ref_e4m3_to_f32.argtypes = [C.c_uint8]
    R.ref_e8m0_to_f32.restype = C.c_float
    R.ref_e8m0_to_f32.argtypes = [C.c_uint8]
    R.ref_scale_atom_offset.restype = C.c_uint64
    R.ref_scale_atom_offset.argtypes = [C.c_uint64] * 3
    R.ref_ggml_row_padding.restype = C.c_uint64
    R.ref_decode_rows.restype = C.c_int
    R.ref_decode_rows.argtypes = [C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64,
                                  C.c_uint64, C.c_uint64, C.c_void_p]

    rng = np.random.default_rng(20261125)
    out = {}
    # ---- element conversions, from the reference's own functions
    out["f16_to_f32_bits"] = np.array([R.ref_f16_to_f32(i) for i in range(65536)],
                                      np.float32).view(np.uint32)
    out["e4m3_to_f32_bits"] = np.array([R.ref_e4m3_to_f32(i) for i in range(256)],
                                       np.float32).view(np.uint32)
    out["e8m0_to_f32_bits"] = np.array([R.ref_e8m0_to_f32(i) for i in range(256)],
                                       np.float32).view(np.uint32)
    probes = np.concatenate([
        rng.normal(0, 1, 4000), rng.normal(0, 1e-4, 2000), rng.normal(0, 3e4, 2000),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, 6e-8, 5.96e-8, 2.98e-8, 2.9e-8,
                  6.1e-5, 6.09e-5, np.inf, -np.inf, np.nan]),
        # ties: halfway between adjacent halves / bfloats
        np.array([1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11, 1.0 + 2.0 ** -9, 1.0 + 3 * 2.0 ** -9]),
    ]).astype(np.float32)
    out["f32_probes_bits"] = probes.view(np.uint32)
    out["f32_to_f16"] = np.array([R.ref_f32_to_f16(float(v)) for v in probes], np.uint16)
    out["f32_to_bf16"] = np.array([R.ref_f32_to_bf16(float(v)) for v in probes], np.uint16)
    out["bf16_to_f32_bits"] = np.array([R.ref_bf16_to_f32(i) for i in range(0, 65536, 7)],
                                       np.float32).view(np.uint32)
    # ---- layout facts
    rows = np.array([0, 1, 31, 32, 33, 95, 127, 128, 129, 300, 4095], np.uint64)
    blocks_per_row = np.array([4, 8, 80, 128], np.uint64)
    table = []
    for bpr in blocks_per_row:
        for r in rows:
            for b in (0, 1, 2, 3, 4, int(bpr) - 1):
                table.append((int(r), int(b), int(bpr), int(R.ref_scale_atom_offset(int(r), b, int(bpr)))))
    out["scale_atom_offsets"] = np.array(table, np.uint64)
    geo = []
    R.ref_block_geometry.argtypes = [C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    for t in (8, 9, 12):
        e, b = C.c_uint64(), C.c_uint64()
        assert R.ref_block_geometry(t, C.byref(e), C.byref(b)) == 0
        geo.append((t, e.value, b.value))
    out["block_geometry"] = np.array(geo, np.uint64)
    out["ggml_row_padding"] = np.array([R.ref_ggml_row_padding()], np.uint64)
    # ---- MXFP8 decode through the reference's DecodeRows (scale atoms)
    n, k = 24, 256
    codes = rng.integers(0, 256, size=(n, k), dtype=np.uint8)
    scales = (110 + (np.arange(n * (k // 32)) % 30)).astype(np.uint8).reshape(n, k // 32)
    scales[0, 3] = 0xFF
    atoms = np.zeros(128 * (k // 32), np.uint8)
    for r in range(n):
        for b in range(k // 32):
            atoms[int(R.ref_scale_atom_offset(r, b, k // 32))] = scales[r, b]
    dec = np.empty((n, k), np.float32)
    assert R.ref_decode_rows(0, codes.ctypes.data, codes.size, atoms.ctypes.data, atoms.size, n, k,
                             dec.ctypes.data) == 0
    out["mxfp8_codes"], out["mxfp8_scales"], out["mxfp8_atoms"] = codes, scales, atoms
    out["mxfp8_decoded_bits"] = dec.view(np.uint32)
    # ---- Q8_1 rows through the reference's DecodeRows (d * q)
    q81 = rng.integers(0, 256, size=(4, 16 * 36), dtype=np.uint8)
    for r in range(4):
        for b in range(16):  # finite FP16 scales
            q81[r, b * 36:b * 36 + 2] = np.array([abs(rng.normal(0, 0.05))], np.float16).view(np.uint8)
    d81 = np.empty((4, 512), np.float32)
    assert R.ref_decode_rows(2, q81.ctypes.data, q81.size, None, 0, 4, 512, d81.ctypes.data) == 0
    out["q8_1_blocks"], out["q8_1_decoded_bits"] = q81, d81.view(np.uint32)
    # ---- NVFP4 / MXFP4 (E2M1 codes; split scales and scale atoms) and dense BF16 / F16
    n, k = 20, 256
    fp4 = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    nv_scales = rng.integers(0x20, 0x60, size=(n, k // 16), dtype=np.uint8)
    nv_scales[0, 1], nv_scales[1, 2], nv_scales[2, 0] = 0x7F, 0x80, 0x00
    mx_scales = (118 + (np.arange(n * (k // 32)) % 18)).astype(np.uint8).reshape(n, k // 32)
    mx_scales[3, 1] = 0xFF

    def atoms_of(scales):
        blocks = scales.shape[1]
        a = np.zeros(128 * blocks, np.uint8)
        for r in range(scales.shape[0]):
            for b in range(blocks):
                a[int(R.ref_scale_atom_offset(r, b, blocks))] = scales[r, b]
        return a

    for name, kind, sc in (("nvfp4", 5, nv_scales), ("mxfp4", 7, mx_scales)):
        dec = np.empty((n, k), np.float32)
        assert R.ref_decode_rows(kind, fp4.ctypes.data, fp4.size, sc.ctypes.data, sc.size, n, k,
                                 dec.ctypes.data) == 0, name
        at = atoms_of(sc)
        dec2 = np.empty((n, k), np.float32)
        assert R.ref_decode_rows(kind + 1, fp4.ctypes.data, fp4.size, at.ctypes.data, at.size, n, k,
                                 dec2.ctypes.data) == 0, name
        assert np.array_equal(dec.view(np.uint32), dec2.view(np.uint32))
        out[name + "_scales"], out[name + "_atoms"] = sc, at
        out[name + "_decoded_bits"] = dec.view(np.uint32)
    out["fp4_codes"] = fp4
    half = rng.integers(0, 65536, size=(6, 64), dtype=np.uint16)
    for name, kind in (("bf16", 9), ("f16", 10)):
        dec = np.empty((6, 64), np.float32)
        assert R.ref_decode_rows(kind, half.ctypes.data, half.size * 2, None, 0, 6, 64,
                                 dec.ctypes.data) == 0, name
        out[name + "_decoded_bits"] = dec.view(np.uint32)
    out["dense16_bits"] = half
    # ---- gguf: Q8_0 quantize/dequantize, Q4_K dequantize
    import gguf
    from gguf import quants
    x = rng.normal(0, 0.05, size=(8, 512)).astype(np.float32)
    q80 = quants.quantize(x, gguf.GGMLQuantizationType.Q8_0)
    out["q8_0_source"] = x
    out["q8_0_blocks_gguf"] = np.ascontiguousarray(q80).view(np.uint8).reshape(8, -1)
    out["q8_0_decoded_gguf_bits"] = quants.dequantize(q80, gguf.GGMLQuantizationType.Q8_0).astype(
        np.float32).view(np.uint32)
    w4 = synth.q4_k_weights(rng, 6, 1024)
    out["q4_k_blocks"] = w4
    out["q4_k_decoded_gguf_bits"] = quants.dequantize(w4, gguf.GGMLQuantizationType.Q4_K).astype(
        np.float32).view(np.uint32)
    w8 = synth.q8_0_weights(rng, 5, 256)
    out["q8_0_blocks"] = w8
    out["q8_0_blocks_decoded_gguf_bits"] = quants.dequantize(
        w8, gguf.GGMLQuantizationType.Q8_0).astype(np.float32).view(np.uint32)
    np.savez_compressed(os.path.join(HERE, "reference_pins.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_pins.npz"),
          os.path.getsize(os.path.join(HERE, "reference_pins.npz")), "bytes")


if __name__ == "__main__":
    main()
