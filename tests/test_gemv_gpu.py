"""GPU parity of the quantized GEMV against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest
import torch

import oracle
from helpers import OP_RTOL, assert_close
from inferi_b200 import quant
from inferi_b200.ops import GemvQuant, GpuQuantTensor, InferiError

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "blocks.npz"))
QTYPES = [quant.Q8_0, quant.Q4_K, quant.Q5_K, quant.Q6_K]
LEGACY = [quant.Q4_0, quant.Q4_1, quant.Q5_0, quant.Q5_1]   # the reference's other GpuQuantTensor variants (op level, generic kernel)


def run_gemv(backend, qt, rows, cols, blocks, v):
    m = GpuQuantTensor(backend, qt, rows, cols, blocks)
    out = torch.full((rows,), float("nan"), device="cuda")
    GemvQuant.from_backend(backend).launch(out, m, torch.from_numpy(v).cuda())
    torch.cuda.synchronize()
    res = out.cpu().numpy()
    m.close()
    return res


@pytest.mark.parametrize("qt", QTYPES + LEGACY)
def test_golden_vectors(backend, qt):
    n = quant.NAMES[qt]
    rows, cols = GOLDEN[f"{n}_deq"].shape
    got = run_gemv(backend, qt, rows, cols, GOLDEN[f"{n}_blocks"], GOLDEN[f"{n}_v"])
    assert_close(got, GOLDEN[f"{n}_gemv"], what=f"golden {n}")


# shapes of the reference's own GEMV tests (crates/inferi/src/ops/gemv_quant.rs:502-816): 64 x 256, Q6_K 64 x 512,
# random scales with a quarter in the f16 subnormal range; plus aligned shapes that take the 128-bit kernels
@pytest.mark.parametrize("qt,rows,cols", [
    (quant.Q8_0, 64, 256), (quant.Q4_K, 64, 256), (quant.Q5_K, 64, 256), (quant.Q6_K, 64, 512),
    (quant.Q8_0, 64, 128), (quant.Q6_K, 8, 256), (quant.Q6_K, 64, 2048), (quant.Q6_K, 36, 6144), (quant.Q8_0, 260, 1024),
    (quant.Q4_K, 4, 256), (quant.Q4_K, 1000, 2560), (quant.Q4_K, 128, 11008), (quant.Q6_K, 64, 8192), (quant.Q8_0, 64, 14336),
    (quant.Q5_K, 296, 4096), (quant.Q4_K, 300, 6144), (quant.Q6_K, 1184, 4096), (quant.Q4_K, 2372, 2048), (quant.Q4_K, 16, 16384), (quant.Q4_K, 16, 16640), (quant.Q5_K, 12, 14336), (quant.Q4_K, 8, 32768), (quant.Q4_K, 8, 33024),
])
def test_reference_test_shapes_and_edges(backend, qt, rows, cols):
    _shape_case(backend, qt, rows, cols)


# the legacy formats at the shape of the reference's tests (gemv_quant.rs:502-816: 64 x 256; Q8_K blocks span 256 columns)
# and at a layer-sized one
@pytest.mark.parametrize("qt,rows,cols", [(q, 64, 256) for q in LEGACY + [quant.Q8_K]] + [(q, 512, 4096) for q in LEGACY + [quant.Q8_K]])
def test_legacy_formats(backend, qt, rows, cols):
    _shape_case(backend, qt, rows, cols)


def _shape_case(backend, qt, rows, cols):
    blocks = quant.random_blocks(qt, rows, cols, seed=rows * 31 + cols + qt, scale=1.0, subnormal_frac=0.25)
    v = np.random.default_rng(cols).standard_normal(cols).astype(np.float32)
    got = run_gemv(backend, qt, rows, cols, blocks, v)
    assert_close(got, oracle.gemv_ref(qt, rows, cols, blocks, v), what=f"{quant.NAMES[qt]} {rows}x{cols}")


@pytest.mark.parametrize("qt,rows,cols,seed", [
    (quant.Q8_0, 4096, 4096, 1001),      # single Q8_0 GEMV
    (quant.Q4_K, 4096, 4096, 2001), (quant.Q4_K, 14336, 4096, 2002), (quant.Q5_K, 4096, 14336, 2003),
    (quant.Q6_K, 128256, 4096, 2004),    # classifier
])
def test_benchmark_shapes(backend, qt, rows, cols, seed):
    blocks = quant.random_blocks(qt, rows, cols, seed=seed)
    v = np.random.default_rng(seed + 1).standard_normal(cols).astype(np.float32)
    got = run_gemv(backend, qt, rows, cols, blocks, v)
    ref = oracle.gemv_ref(qt, rows, cols, blocks, v)
    e = assert_close(got, ref, what=f"{quant.NAMES[qt]} {rows}x{cols}")
    assert e < 2e-4   # well inside the bar of 1e-3: the activations are 16-bit block fixed point (measured: 2e-5 .. 1.1e-4)
    # linearity in v (a size-independent property): W(2v) == 2 W v exactly in binary floating point
    got2 = run_gemv(backend, qt, rows, cols, blocks, 2 * v)
    assert np.array_equal(got2, 2 * got)


def test_f32_matrix_and_special_vectors(backend):
    rows, cols = 8, 300
    w = np.random.default_rng(1).standard_normal((rows, cols)).astype(np.float32)
    v = np.random.default_rng(2).standard_normal(cols).astype(np.float32)
    got = run_gemv(backend, quant.F32, rows, cols, w.view(np.uint8).reshape(rows, -1), v)
    assert_close(got, w.astype(np.float64) @ v, what="f32 gemv")
    # zero vector, and a vector with one huge entry per 32-group (dynamic range inside a group)
    blocks = quant.random_blocks(quant.Q4_K, 16, 1024, seed=5)
    assert np.array_equal(run_gemv(backend, quant.Q4_K, 16, 1024, blocks, np.zeros(1024, np.float32)), np.zeros(16, np.float32))
    v = np.random.default_rng(3).standard_normal(1024).astype(np.float32)
    v[::32] *= 1e4
    assert_close(run_gemv(backend, quant.Q4_K, 16, 1024, blocks, v), oracle.gemv_ref(quant.Q4_K, 16, 1024, blocks, v), what="wide range")


def test_host_buffer_entry_point(backend):
    blocks = quant.random_blocks(quant.Q6_K, 64, 2048, seed=9)
    v = np.random.default_rng(4).standard_normal(2048).astype(np.float32)
    m = GpuQuantTensor(backend, quant.Q6_K, 64, 2048, blocks)
    got = GemvQuant(backend).launch_host(m, v)
    assert_close(got, oracle.gemv_ref(quant.Q6_K, 64, 2048, blocks, v), what="host entry point")


def test_contract_violations_are_errors(backend):
    b = quant.random_blocks(quant.Q4_K, 8, 256, seed=1)
    with pytest.raises(InferiError):           # rows % 4 (the reference truncates silently)
        GpuQuantTensor(backend, quant.Q4_K, 6, 256, b[:6])
    with pytest.raises(InferiError):           # byte count
        GpuQuantTensor(backend, quant.Q4_K, 8, 512, b)
    with pytest.raises(InferiError):           # a GGUF type id this library has no reader for (Q2_K)
        GpuQuantTensor(backend, 10, 8, 256, b)
    m = GpuQuantTensor(backend, quant.Q4_K, 8, 256, b)
    with pytest.raises(InferiError):           # vector length
        GemvQuant(backend).launch(torch.zeros(8, device="cuda"), m, torch.zeros(128, device="cuda"))
    with pytest.raises(InferiError):           # host tensor where a device tensor is required
        GemvQuant(backend).launch(torch.zeros(8), m, torch.zeros(256, device="cuda"))
