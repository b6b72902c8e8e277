"""Generates tests/golden/blocks.npz: seeded GGUF blocks with their dequantized values and a GEMV result.

The expected values come from the third-party `gguf` Python package (gguf.quants.dequantize), an implementation
of the ggml block formats that is independent of both this repository's oracle and its CUDA kernels; the reference
project cites the same ggml definitions (crates/inferi/src/quantization.rs:41, 213, 260, 333).  The GEMV result is
the float64 product of those dequantized values with a seeded vector.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import gguf  # noqa: E402
from gguf.quants import dequantize  # noqa: E402

from inferi_b200 import quant  # noqa: E402

GG = {quant.Q8_0: gguf.GGMLQuantizationType.Q8_0, quant.Q4_K: gguf.GGMLQuantizationType.Q4_K,
      quant.Q5_K: gguf.GGMLQuantizationType.Q5_K, quant.Q6_K: gguf.GGMLQuantizationType.Q6_K,
      quant.Q4_0: gguf.GGMLQuantizationType.Q4_0, quant.Q4_1: gguf.GGMLQuantizationType.Q4_1,
      quant.Q5_0: gguf.GGMLQuantizationType.Q5_0, quant.Q5_1: gguf.GGMLQuantizationType.Q5_1}
ROWS, COLS = 4, 512


def main():
    out = {}
    # (Q8_K is not in the gguf package's dequantizers: its pin is the closed form d * q in tests/test_oracle.py)
    for qt in (quant.Q8_0, quant.Q4_K, quant.Q5_K, quant.Q6_K, quant.Q4_0, quant.Q4_1, quant.Q5_0, quant.Q5_1):
        name = quant.NAMES[qt]
        # a quarter of the f16 scales in the subnormal range, as the reference's test helper does
        blocks = quant.random_blocks(qt, ROWS, COLS, seed=7000 + qt, subnormal_frac=0.25)
        deq = dequantize(blocks, GG[qt]).reshape(ROWS, COLS).astype(np.float32)
        v = np.random.default_rng(7100 + qt).standard_normal(COLS).astype(np.float32)
        out[f"{name}_blocks"] = blocks
        out[f"{name}_deq"] = deq
        out[f"{name}_v"] = v
        out[f"{name}_gemv"] = deq.astype(np.float64) @ v.astype(np.float64)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "blocks.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
