"""CPU tests of the tensor-parallel host logic: sharding of GGUF bytes, and a world-size-2 gloo run in which two ranks
compute their partial GEMVs with the oracle and all-reduce them, exactly the exchange the GPU path fuses into its kernels."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from inferi_b200 import quant, tp
from inferi_b200.llama2 import Llama2Config, Q4_K_M, synth_weights

CFG = Llama2Config(1024, 4096, 1, 8, 4, 1024, 32, 500000.0, 1e-5)


def _deq(mat, rows, cols):
    return oracle.dequantize(mat[0], mat[1].numpy() if isinstance(mat[1], torch.Tensor) else mat[1], rows * cols).reshape(rows, cols)


@pytest.mark.parametrize("ranks", [2, 4])
def test_shards_tile_the_matrices(ranks):
    w = synth_weights(CFG, seed=5, recipe=dict(Q4_K_M, attn_v=quant.Q4_K))
    sh, lw = CFG.shapes(), w["layers"][0]
    full = {n: _deq(lw[n], *sh[n]) for n in ("attn_q", "attn_k", "attn_output", "ffn_gate", "ffn_down")}
    real, padded = tp.ffn_plan(CFG, ranks, lw["ffn_down"][0])
    assert real == 4096 // ranks and padded == 2048          # Q6_K rows are cut at multiples of 2048 columns
    shapes = tp.shard_shapes(CFG, ranks, lw["ffn_down"][0])
    got_q, got_o, got_down, got_gate = [], [], [], []
    for r in range(ranks):
        s = tp.shard_weights(CFG, w, r, ranks)["layers"][0]
        for n in ("attn_q", "attn_output", "ffn_gate", "ffn_down"):
            assert tuple(s[n][1].shape) == (shapes[n][0], quant.row_bytes(s[n][0], shapes[n][1])), n
        got_q.append(_deq(s["attn_q"], *shapes["attn_q"]))
        got_o.append(_deq(s["attn_output"], *shapes["attn_output"]))
        g = _deq(s["ffn_gate"], *shapes["ffn_gate"])
        d = _deq(s["ffn_down"], *shapes["ffn_down"])
        assert not g[real:].any() and not d[:, real:].any()  # the padding dequantizes to exact zeros
        got_gate.append(g[:real])
        got_down.append(d[:, :real])
    assert np.array_equal(np.concatenate(got_q, 0), full["attn_q"])
    assert np.array_equal(np.concatenate(got_o, 1), full["attn_output"])
    assert np.array_equal(np.concatenate(got_gate, 0), full["ffn_gate"])
    assert np.array_equal(np.concatenate(got_down, 1), full["ffn_down"])
    v = tp.shard_weights(CFG, w, ranks - 1, ranks)["output"][1]
    assert v.shape[0] == CFG.vocab_size // ranks


def test_misaligned_splits_are_refused():
    with pytest.raises(ValueError):
        tp.shard_weights(CFG, synth_weights(CFG, seed=1), 0, 3)
    with pytest.raises(ValueError):
        tp.cols_slice((quant.Q4_K, torch.zeros(4, 288, dtype=torch.uint8)), 0, 128)


def _rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = synth_weights(CFG, seed=5)                      # same seed on every rank
        mine = tp.shard_weights(CFG, w, rank, world)["layers"][0]
        shapes = tp.shard_shapes(CFG, world, mine["ffn_down"][0])
        real, padded = tp.ffn_plan(CFG, world, mine["ffn_down"][0])
        rng = np.random.default_rng(3)
        xb = rng.standard_normal(CFG.hidden_size).astype(np.float32)      # attention output (all heads)
        hb = rng.standard_normal(CFG.intermediate_size).astype(np.float32)
        # row-split matrices: each rank multiplies its column slice by its slice of the vector, then the sum is exchanged
        q0 = rank * CFG.hidden_size // world
        part_o = oracle.gemv_ref(mine["attn_output"][0], *shapes["attn_output"], mine["attn_output"][1].numpy(), xb[q0:q0 + CFG.hidden_size // world])
        hb_l = np.zeros(padded, np.float32)
        hb_l[:real] = hb[rank * real:(rank + 1) * real]
        part_d = oracle.gemv_ref(mine["ffn_down"][0], *shapes["ffn_down"], mine["ffn_down"][1].numpy(), hb_l)
        t = torch.from_numpy(np.stack([part_o, part_d]).astype(np.float64))
        dist.all_reduce(t)
        sh, lw = CFG.shapes(), w["layers"][0]
        want_o = oracle.gemv_ref(lw["attn_output"][0], *sh["attn_output"], lw["attn_output"][1].numpy(), xb)
        want_d = oracle.gemv_ref(lw["ffn_down"][0], *sh["ffn_down"], lw["ffn_down"][1].numpy(), hb)
        err = max(np.abs(t[0].numpy() - want_o).max() / np.abs(want_o).max(), np.abs(t[1].numpy() - want_d).max() / np.abs(want_d).max())
        # column-split classifier: local arg-max candidates, global winner = max over ranks (value, lowest index)
        logits = rng.standard_normal(CFG.vocab_size).astype(np.float32)
        v0 = rank * CFG.vocab_size // world
        loc = logits[v0:v0 + CFG.vocab_size // world]
        cand = torch.tensor([float(loc.max()), float(-(v0 + int(loc.argmax())))], dtype=torch.float64)
        allc = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(allc, cand)
        best = max(allc, key=lambda c: (c[0].item(), c[1].item()))
        q.put((rank, float(err), int(-best[1].item()) == oracle.argmax(logits)))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_partial_sums_and_argmax():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, amax_ok in res:
        assert err < 1e-6 and amax_ok, (rank, err, amax_ok)
