"""One rank of the tensor-parallel GPU parity run (launched by tests/test_tp_gpu.py through torch.distributed.run).

Every rank builds the same seeded checkpoint, keeps its shard, and runs the token loop; rank 0 also runs the CPU oracle
on the full checkpoint.  Checked: greedy ids identical on every rank and equal to the oracle's, logits (the ranks'
vocabulary slices, gathered) within 2e-2 of the oracle.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from inferi_b200 import quant, tp  # noqa: E402
from inferi_b200.llama2 import Llama2, Llama2Config, Llama2Weights, Q4_K_M, synth_weights, weights_to_host  # noqa: E402
from inferi_b200.ops import Backend  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dist.init_process_group("gloo")                      # host-side hand-shake only; the data path is peer stores
    torch.cuda.set_device(local)
    qwen2 = os.environ.get("TP_QWEN2") == "1"             # NeoX rotation + q/k/v biases (sharded by heads like the matrices)
    cfg = Llama2Config(2048, 8192, 2, 32, 8, 1024, 96, 500000.0, 1e-5, int(qwen2))
    full = synth_weights(cfg, seed=4001, recipe=Q4_K_M, qkv_bias=qwen2)   # CPU generator: identical on every rank
    mine = tp.shard_weights(cfg, full, rank, world)
    be = Backend(local)
    shapes = tp.shard_shapes(cfg, world, Q4_K_M["ffn_down"])
    path = os.environ.get("TP_FROM_GGUF")
    if path:
        # every rank maps the same file and uploads its slice itself (the library cuts the GGUF bytes)
        from inferi_b200.gguf import Gguf
        f = Gguf(path)
        model = f.load_llama(be, kv_f16=True, tp_rank=rank, tp_size=world, arch="qwen2" if qwen2 else None)
        f.close()
    else:
        model = Llama2(be, cfg, Llama2Weights(be, cfg, mine, shapes=shapes), kv_f16=True, tp_rank=rank, tp_size=world)
    prompt = [7, 900, 33, 512]
    n_gen = 20
    ids = model.generate(prompt, n_gen).tolist()
    # logits of one more step, gathered over the vocabulary shards
    nxt, logits = model.forward(ids[-1], len(prompt) + n_gen - 1, want_logits=True)
    parts = [None] * world
    dist.all_gather_object(parts, (ids, nxt, logits))
    ok = True
    if rank == 0:
        assert all(p[0] == parts[0][0] and p[1] == parts[0][1] for p in parts), "ranks disagree on the greedy tokens"
        ref = oracle.Llama(dict(hidden=2048, ffn=8192, n_layers=2, n_heads=32, n_kv_heads=8, vocab=1024, max_pos=96, rope_theta=500000.0, rms_eps=1e-5,
                                rope_variant=int(qwen2)),
                           weights_to_host(full), kv_f16=True)
        want, tok = [], None
        for pos in range(len(prompt) + n_gen - 1):
            tok = prompt[pos] if pos < len(prompt) else want[-1]
            lg = ref.forward(tok, pos)
            if pos >= len(prompt) - 1:
                want.append(oracle.argmax(lg))
        lg = ref.forward(want[-1], len(prompt) + n_gen - 1)
        got = np.concatenate([p[2] for p in parts])
        err = float(np.abs(got - lg).max())
        ok = ids == want and nxt == oracle.argmax(lg) and err <= 2e-2
        print(f"TP_{'OK' if ok else 'FAIL'} world={world} tokens_match={ids == want} logits_max_abs={err:.3e}", flush=True)
    dist.barrier()
    model.close()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
