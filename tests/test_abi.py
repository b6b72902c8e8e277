"""CPU tests of the boundary: the shared library loads, exports every symbol the header declares, and refuses to
work without a GPU instead of falling back to anything."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

from inferi_b200 import _lib, quant

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "inferi_b200.h")).read()
    return sorted(set(re.findall(r"IB_API\s+[\w\s\*]+?\b(ib_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/inferi_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signature table and header disagree"


def test_struct_layouts_match_the_header():
    assert C.sizeof(_lib.AttnParams) == 24
    assert C.sizeof(_lib.LlamaConfig) == 40
    assert C.sizeof(_lib.LlamaLayerWeights) == 12 * C.sizeof(C.c_void_p)
    assert C.sizeof(_lib.LlamaWeights) == 4 * C.sizeof(C.c_void_p)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_gpu_means_an_error_not_a_fallback():
    lib = _lib.load()
    h = C.c_void_p()
    rc = lib.ib_ctx_create(0, C.byref(h))
    assert rc == 2 and not h.value
    assert b"no CPU path" in lib.ib_last_error_string()
    from inferi_b200.ops import Backend, InferiError
    with pytest.raises(InferiError):
        Backend(0)


def test_null_handles_are_rejected_without_touching_a_device():
    lib = _lib.load()
    assert lib.ib_gemv_quant(None, None, None, None, None) == 1
    assert b"null context" in lib.ib_last_error_string()
    assert lib.ib_llama_forward(None, None, 0, 0, None, None) == 1
    assert lib.ib_ctx_destroy(None) == 0 and lib.ib_qtensor_destroy(None) == 0 and lib.ib_llama_destroy(None) == 0


def test_block_size_tables():
    assert [quant.BLOCK_BYTES[t] for t in (quant.Q8_0, quant.Q4_K, quant.Q5_K, quant.Q6_K)] == [34, 144, 176, 210]
    assert quant.row_bytes(quant.Q6_K, 4096) == 3360 and quant.row_bytes(quant.Q8_0, 4096) == 4352
    with pytest.raises(ValueError):
        quant.row_bytes(quant.Q4_K, 300)
    # algorithmic byte counts of the benchmark shapes
    assert quant.matrix_bytes(quant.Q8_0, 4096, 4096) == 17825792
    assert quant.matrix_bytes(quant.Q4_K, 14336, 4096) == 33030144
    assert quant.matrix_bytes(quant.Q5_K, 4096, 14336) == 40370176
    assert quant.matrix_bytes(quant.Q6_K, 128256, 4096) == 430940160


def test_model_byte_accounting():
    from inferi_b200.llama2 import LLAMA_3_2_1B, LLAMA_3_8B
    assert LLAMA_3_2_1B.weight_bytes() == 836628480
    assert LLAMA_3_8B.weight_bytes() == 4876918784
    assert LLAMA_3_8B.kv_bytes_per_position(True) == 131072
    assert LLAMA_3_2_1B.kv_bytes_per_position(True) == 32768


@pytest.mark.parametrize("qt,bound", [(quant.Q8_0, 0.01), (quant.Q4_K, 0.12), (quant.Q5_K, 0.06), (quant.Q6_K, 0.03)])
def test_quantizer_round_trip(qt, bound):
    import oracle
    w = torch.randn(8, 512, generator=torch.Generator().manual_seed(qt)) * 0.02
    b = quant.quantize(qt, w).numpy()
    assert b.shape == (8, quant.row_bytes(qt, 512)) and b.dtype == np.uint8
    back = oracle.dequantize(qt, b, w.numel()).reshape(8, 512)
    assert np.sqrt(((back - w.numpy()) ** 2).mean()) <= bound * 0.02
    # zero rows stay zero and finite
    z = oracle.dequantize(qt, quant.quantize(qt, torch.zeros(4, 256)).numpy(), 1024)
    assert np.array_equal(z, np.zeros(1024, np.float32))
