"""inferi_b200 — B200-native (sm_100a) batch-1 Llama token loop over GGUF-quantized weights.

The product is the C-ABI shared library `libinferi_b200.so` (header: include/inferi_b200.h); this package is its
Python host side, mirroring the reference's op and model API (`ops`, `llama2`).  There is no CPU fallback.
"""
from . import quant  # noqa: F401  (host-only helpers; importing them never touches the GPU)

__all__ = ["quant", "ops", "llama2", "build"]
