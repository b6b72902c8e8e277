"""Shared test helpers: tolerances and comparisons against the CPU oracle."""
import numpy as np

# per-op bar: |gpu - oracle| <= 1e-3 * max(|oracle|, rms(oracle))  (fp32 accumulate)
OP_RTOL = 1e-3
# whole-model bars
LOGITS_MAX_ABS = 2e-2
TOKENS_EXACT = 64


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    ref = np.asarray(ref, dtype=np.float64).reshape(-1)
    assert got.shape == ref.shape
    assert np.isfinite(got).all(), "non-finite values in the GPU result"
    scale = np.sqrt(np.mean(ref * ref)) if ref.size else 1.0
    denom = np.maximum(np.abs(ref), max(scale, 1e-30))
    return float(np.max(np.abs(got - ref) / denom)) if ref.size else 0.0


def assert_close(got, ref, rtol=OP_RTOL, what=""):
    e = rel_err(got, ref)
    assert e <= rtol, f"{what}: relative error {e:.3e} > {rtol:.1e}"
    return e
