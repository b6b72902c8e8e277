"""Tensor-parallel parity on real GPUs: two ranks, one process each, against the CPU oracle (needs 2 GPUs of one box)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("from_gguf,qwen2", [(False, False), (True, False), (True, True)], ids=["tensors", "gguf", "gguf-qwen2"])
@pytest.mark.parametrize("world", [2])
def test_two_ranks_match_the_oracle(world, from_gguf, qwen2, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if from_gguf:
        # the same checkpoint as a GGUF file: each rank loads its slice through ib_gguf_load_llama
        sys.path.insert(0, ROOT)
        from inferi_b200.gguf import write_llama_gguf
        from inferi_b200.llama2 import Llama2Config, Q4_K_M, synth_weights
        cfg = Llama2Config(2048, 8192, 2, 32, 8, 1024, 96, 500000.0, 1e-5, int(qwen2))
        path = str(tmp_path / "tp.gguf")
        write_llama_gguf(path, cfg, synth_weights(cfg, seed=4001, recipe=Q4_K_M, qkv_bias=qwen2), arch="qwen2" if qwen2 else "llama")
        env["TP_FROM_GGUF"] = path
    env["TP_QWEN2"] = "1" if qwen2 else "0"
    port = 29600 + os.getpid() % 1000 + (7 if from_gguf else 0) + (13 if qwen2 else 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0 and "TP_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-3000:]
