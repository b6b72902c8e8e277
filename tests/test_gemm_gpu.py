"""GPU parity of the tensor-core GEMM (the prefill building block) against the CPU oracle, through the C ABI.

`ib_gemm_quant` must give, for every input row, what the oracle's GEMV (dequantize + f64 dot) gives for that row."""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close
from inferi_b200 import quant
from inferi_b200.ops import GemmQuant, GpuQuantTensor, InferiError

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("qt,rows,cols,n", [
    (quant.Q4_K, 128, 256, 16), (quant.Q4_K, 128, 256, 1), (quant.Q6_K, 128, 2048, 7), (quant.Q8_0, 256, 512, 33), (quant.Q5_K, 128, 1024, 128),
    (quant.Q4_K, 512, 2048, 32), (quant.Q6_K, 1024, 4096, 37), (quant.Q4_K, 4096, 4096, 128), (quant.Q4_K, 256, 14336, 5), (quant.Q6_K, 2048, 8192, 100),
    (quant.Q4_K, 384, 1024, 300),   # more rows than one pass takes: chunks of 128
    (quant.Q4_K, 14336, 4096, 96), (quant.Q5_K, 4096, 14336, 50),   # 1792 units over one wave of CTAs: tiles split between two or three of them
])
def test_gemm_matches_row_by_row_gemv(backend, qt, rows, cols, n):
    blocks = quant.random_blocks(qt, rows, cols, seed=rows + cols + n, scale=0.05)
    x = np.random.default_rng(n).standard_normal((n, cols)).astype(np.float32)
    m = GpuQuantTensor(backend, qt, rows, cols, blocks)
    out = torch.full((n, rows), float("nan"), device="cuda")
    GemmQuant(backend).launch(out, m, torch.from_numpy(x).cuda())
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    for t in sorted({0, n // 2, n - 1}):
        ref = oracle.gemv_ref(qt, rows, cols, blocks, x[t])
        e = assert_close(got[t], ref, what=f"gemm {quant.NAMES[qt]} {rows}x{cols} row {t} of {n}")
        assert e < 1e-4     # two f16 halves per split operand carry ~21 bits (the k-quant weights are exact integers)
    m.close()


def test_gemm_rejects_shapes_outside_the_tensor_core_path(backend):
    blocks = quant.random_blocks(quant.Q4_K, 64, 256, seed=1)
    m = GpuQuantTensor(backend, quant.Q4_K, 64, 256, blocks)     # 64 rows: not a multiple of 128
    with pytest.raises(InferiError) as e:
        GemmQuant(backend).launch(torch.empty(2, 64, device="cuda"), m, torch.zeros(2, 256, device="cuda"))
    assert e.value.code == 4
    m.close()
