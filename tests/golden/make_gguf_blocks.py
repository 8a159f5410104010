"""Writes tests/golden/gguf_blocks.npz: random blocks of the block types whose decoders the
oracle restates from GGML's published formats (Q4_0, Q5_0, IQ4_NL, Q5_K, Q6_K), and what
gguf-py (llama.cpp's reference reader, third party) decodes them to, as F32 bit patterns.
Run where the gguf package is present:  python tests/golden/make_gguf_blocks.py"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))


def main():
    import gguf
    from gguf import quants

    from llmp_b200 import synth
    rng = np.random.default_rng(20240607)
    out = {}
    for t in (2, 6, 20, 13, 14):
        w = synth.more_weights(rng, t, 5, 512)
        out[f"blocks_{t}"] = w
        out[f"decoded_bits_{t}"] = quants.dequantize(w, gguf.GGMLQuantizationType(t)).astype(
            np.float32).view(np.uint32)
    path = os.path.join(HERE, "gguf_blocks.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
