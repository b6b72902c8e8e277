#!/usr/bin/env python
"""Benchmark of the batch-1 decode loop: Llama-3-8B-architecture, Q4_K_M, greedy, f16 KV cache.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

A step is one decoded token (one replay of the token graph).  W warm-up tokens (the prompt, fed through the decode
path) are followed by exactly K timed tokens.  One JSON line is printed by rank 0.

  value     tok/s with everything resident in HBM: K graph replays back to back, CUDA events around them
  e2e       tok/s through `ib_llama_forward` with host buffers: every step copies the token id in from pinned host
            memory, reads the next token id back and synchronises (the reference's per-token loop)
  roofline  per token (one graph launch): algorithmic bytes = every weight byte once + the KV rows read and written,
            divided by the measured time per token; `kernels` holds the dominant GEMV launches timed alone
  cpu_baseline  the CPU port of the reference's shader arithmetic (oracle/, lane-structured f32 GEMVs, all host threads)
            on one 8B-shaped layer + classifier, extrapolated to 32 layers

`--impl reference` times only that CPU port (the reference is Rust and cannot be built here).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "batch-1 decode tok/s, Llama-3-8B-arch Q4_K_M"
UNIT = "tok/s"
PROMPT_SEED, WEIGHT_SEED = 4002, 4001
DRAM_TRAFFIC_RATIO = 1.0003   # dram__bytes_read+write / algorithmic bytes of the streaming GEMV (33.11 MB moved for a 33.10 MB matrix)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 7:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()       # our own child, by handle
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        reasons = []
        for i, name in enumerate(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")):
            if any(r[3 + i].lower().startswith("active") for r in self.rows):
                reasons.append(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons, "samples": len(self.rows)}


# ------------------------------------------------------------------------------------------------------------------
# CPU baseline: the oracle's lane-structured port of the reference shaders on the host cores
# ------------------------------------------------------------------------------------------------------------------
def cpu_baseline(cfg, tokens: int = 3, pos0: int = 384):
    import oracle
    from inferi_b200 import quant
    from inferi_b200.llama2 import LAYER_MATS, Q4_K_M

    sh = cfg.shapes()
    seed = 90
    layer = {}
    for n in LAYER_MATS:
        seed += 1
        layer[n] = (Q4_K_M[n], quant.random_blocks(Q4_K_M[n], *sh[n], seed=seed, scale=0.002))
    rng = np.random.default_rng(5)
    layer["attn_norm"] = np.ones(cfg.hidden_size, np.float32)
    layer["ffn_norm"] = np.ones(cfg.hidden_size, np.float32)
    # the embedding table is only indexed (one row per token): a short one keeps the sample small
    vocab_s = 1024
    w = {"layers": [layer], "token_embd": (Q4_K_M["token_embd"], quant.random_blocks(Q4_K_M["token_embd"], vocab_s, cfg.hidden_size, seed=77, scale=0.002)),
         "output": (Q4_K_M["output"], quant.random_blocks(Q4_K_M["output"], *sh["output"], seed=78, scale=0.002)),
         "output_norm": np.ones(cfg.hidden_size, np.float32)}
    ocfg = dict(hidden=cfg.hidden_size, ffn=cfg.intermediate_size, n_layers=1, n_heads=cfg.num_attention_heads, n_kv_heads=cfg.num_key_value_heads,
                vocab=cfg.vocab_size, max_pos=pos0 + tokens + 1, rope_theta=cfg.rope_theta, rms_eps=cfg.rms_norm_eps)
    threads = oracle.max_threads()
    m = oracle.Llama(ocfg, w, kv_f16=True, nthreads=threads)
    m.set_gemv_mode(True)
    # fill the cache rows below pos0 with something finite: attention cost at pos0 is what is sampled
    m.forward(1, 0, want_logits=False)
    t_layer, t_full = [], []
    for i in range(tokens):
        tok = int(rng.integers(0, vocab_s))
        t0 = time.perf_counter()
        m.forward(tok, pos0 + i, want_logits=False)
        t1 = time.perf_counter()
        m.forward(tok, pos0 + i, want_logits=True)
        t2 = time.perf_counter()
        t_layer.append(t1 - t0)
        t_full.append(t2 - t1)
    m.close()
    tl = min(t_layer)
    th = max(min(t_full) - tl, 0.0)
    per_token = cfg.num_hidden_layers * tl + th
    return {"value": 1.0 / per_token, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"1 of {cfg.num_hidden_layers} layers + classifier at position {pos0}, best of {tokens} tokens, "
                      f"extrapolated: {cfg.num_hidden_layers} x {tl * 1e3:.1f} ms + {th * 1e3:.1f} ms per token"}


def run_reference(args, cfg, rank):
    """The reference arm: the CPU port timed alone (rank 0 only)."""
    if rank != 0:
        return
    vals = []
    for _ in range(max(1, min(args.steps, 3))):
        vals.append(cpu_baseline(cfg, tokens=2))
    best = max(vals, key=lambda v: v["value"])
    line = {"impl": "reference", "metric": METRIC, "value": best["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 / best["value"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": workload_name(cfg), "note": "reference is Rust (no toolchain here): CPU port of its shader arithmetic, "
                                            "all host threads, one layer + classifier sampled per step and extrapolated"},
            "cpu_baseline": best, "e2e": {"value": best["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def kernel_case(name: str):
    """A small stand-alone loop over one kernel, for `ncu` captures: a few launches, rotating over buffers that together
    exceed L2.  Cases: gate_q4k, q_q4k, down_q6k, lmhead_q6k, q5k, q8_0, attn_8k, attn_32k."""
    import torch
    from inferi_b200 import quant
    from inferi_b200.ops import AttnParams, Backend, FusedAttention, GemvQuant, GpuQuantTensor
    torch.cuda.set_device(0)
    backend = Backend(0)
    shapes = {"gate_q4k": (quant.Q4_K, 14336, 4096, 6), "q_q4k": (quant.Q4_K, 4096, 4096, 16), "down_q6k": (quant.Q6_K, 4096, 14336, 4),
              "lmhead_q6k": (quant.Q6_K, 128256, 4096, 1), "q5k": (quant.Q5_K, 4096, 14336, 4), "q8_0": (quant.Q8_0, 4096, 4096, 8)}
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if name in shapes:
        qt, rows, cols, copies = shapes[name]
        mats = [GpuQuantTensor(backend, qt, rows, cols, quant.random_blocks(qt, rows, cols, seed=10 + i)) for i in range(copies)]
        v, o = torch.randn(cols, device="cuda"), torch.empty(rows, device="cuda")
        g = GemvQuant(backend)
        n = 0
        for rep in range(3):
            if rep == 2:
                start.record()
            for m in mats:
                g.launch(o, m, v)
                n += rep == 2
        end.record()
        torch.cuda.synchronize()
        b = mats[0].nbytes + 4 * (rows + cols)
    elif name.startswith("attn_"):
        ctx = {"attn_8k": 8192, "attn_32k": 32768}[name]
        hs, nh, kvm = 128, 32, 4
        kv_dim = nh // kvm * hs
        caches = [(torch.randn(ctx, kv_dim, device="cuda").half(), torch.randn(ctx, kv_dim, device="cuda").half()) for _ in range(3)]
        q, o = torch.randn(nh * hs, device="cuda"), torch.empty(nh * hs, device="cuda")
        att = FusedAttention(backend)
        p = AttnParams(ctx, kv_dim, kvm, nh, hs, ctx - 1)
        n = 0
        for rep in range(3):
            if rep == 2:
                start.record()
            for kc, vc in caches:
                att.launch(p, q, kc, vc, o)
                n += rep == 2
        end.record()
        torch.cuda.synchronize()
        b = 2 * ctx * kv_dim * 2
    else:
        raise SystemExit(f"unknown kernel case {name}")
    us = start.elapsed_time(end) * 1e3 / n
    print(json.dumps({"kernel_case": name, "us_per_launch": us, "algorithmic_bytes": b, "gbs": b / us / 1e3}))


def workload_name(cfg):
    return (f"Llama-3-8B-arch decoder ({cfg.num_hidden_layers} layers, hidden {cfg.hidden_size}, {cfg.num_attention_heads}q/{cfg.num_key_value_heads}kv heads, "
            f"FFN {cfg.intermediate_size}, vocab {cfg.vocab_size}), random Q4_K_M weights, f16 KV, batch 1, greedy")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=128)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="debug: override the layer count (the result is then not the benchmark)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel-case", default="", help="run a small loop over one kernel instead of the benchmark (for ncu captures)")
    args = ap.parse_args()
    if args.kernel_case:
        kernel_case(args.kernel_case)
        return

    from inferi_b200.llama2 import LLAMA_3_8B, Llama2Config
    cfg = LLAMA_3_8B
    if args.layers:
        cfg = Llama2Config(**{**cfg.__dict__, "num_hidden_layers": args.layers})
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, cfg, rank)
        return

    import torch
    from inferi_b200.llama2 import Llama2, Llama2Weights, synth_weights
    from inferi_b200.ops import Backend, GemvQuant

    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run); got {world}")
    W, K = max(args.warmup, 3), args.steps
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        from inferi_b200 import tp
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    backend = Backend(local_rank)

    weights = synth_weights(cfg, seed=WEIGHT_SEED, device="cuda")     # same seed, same values on every rank
    shapes = None
    if world > 1:
        # tensor parallel: each rank keeps its shard (rows of q/k/v/gate/up/classifier, columns of attn_output/ffn_down)
        shapes = tp.shard_shapes(cfg, world, weights["layers"][0]["ffn_down"][0])
        weights = tp.shard_weights(cfg, weights, rank, world)
    dev_w = Llama2Weights(backend, cfg, weights, shapes=shapes)
    del weights
    torch.cuda.empty_cache()
    model = Llama2(backend, cfg, dev_w, kv_f16=True, tp_rank=rank, tp_size=world)
    prompt = np.random.default_rng(PROMPT_SEED).integers(0, cfg.vocab_size, W).astype(np.uint32)

    def rank_sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- value: device-resident loop -------------------------------------------------------------------------
    first = model.generate(prompt, 1, start_pos=0)          # W warm-up steps through the decode path
    rank_sync()
    backend.reset_launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        rank_sync()
        start.record()
        out = model.generate(first, K, start_pos=W)         # exactly K timed steps
        end.record()
        rank_sync()
    ms = max_over_ranks(start.elapsed_time(end))            # device time, maximum over the ranks
    launches = backend.launch_count()
    tok_s = K / (ms * 1e-3)

    # ---- e2e: per-token host round trip ----------------------------------------------------------------------
    tok = int(first[0])
    for i in range(3):
        model.forward(tok, W + i)
    rank_sync()
    t0 = time.perf_counter()
    pos = W
    for _ in range(K):
        tok, _ = model.forward(tok, pos)
        pos += 1
    rank_sync()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e_tok_s = K / e2e_s

    # ---- roofline --------------------------------------------------------------------------------------------
    peak, peak_src = measured_peaks()
    peak *= world                                            # aggregate HBM bandwidth of the ranks
    avg_pos = W + (K - 1) / 2.0
    bytes_per_token = cfg.weight_bytes() + cfg.kv_bytes_per_position(True) * (avg_pos + 1) + cfg.kv_bytes_per_position(True)
    achieved = bytes_per_token / (ms * 1e-3 / K) / 1e9
    kernels = []
    gemv = GemvQuant(backend)
    for name, mats in () if world > 1 else (("ffn_gate Q4_K 14336x4096", [l["ffn_gate"] for l in dev_w.layers]), ("ffn_down Q6_K 4096x14336", [l["ffn_down"] for l in dev_w.layers]),
                       ("attn_q Q4_K 4096x4096", [l["attn_q"] for l in dev_w.layers]), ("output Q6_K 128256x4096", [dev_w.output])):
        v = torch.randn(mats[0].cols, device="cuda")
        o = torch.empty(mats[0].rows, device="cuda")
        reps = max(3, 96 // len(mats))
        for m_ in mats[:4]:
            gemv.launch(o, m_, v)
        torch.cuda.synchronize()
        start.record()
        for _ in range(reps):
            for m_ in mats:                                  # rotate over distinct buffers (> L2 in total)
                gemv.launch(o, m_, v)
        end.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(end) * 1e3 / (reps * len(mats))
        b = mats[0].nbytes + 4 * (mats[0].rows + mats[0].cols)
        kernels.append({"kernel": f"gemv_stream_kernel {name}", "us_per_launch": round(us, 2), "algorithmic_bytes": b, "gbs": round(b / us / 1e3, 1),
                        "frac": round(b / us / 1e3 / peak, 3)})

    line = {
        "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 dp4a weights x 3-limb int8 activations, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": workload_name(cfg), "parallelism": f"tp{world}" if world > 1 else "single GPU", "prompt_tokens": W, "decode_tokens": K, "l2": "weights per token (4.9 GB) exceed L2 (126 MB)",
                   "prefill": "prompt fed through the decode path (as the reference does), untimed"},
        "e2e": {"value": e2e_tok_s, "unit": UNIT, "h2d_bytes_per_step": 20, "d2h_bytes_per_step": 4},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     # DRAM bytes per token: algorithmic bytes x the read+write / algorithmic ratio of the ncu captures of the
                     # GEMV kernels (a whole token is too large to capture at once)
                     "traffic": bytes_per_token * DRAM_TRAFFIC_RATIO, "traffic_source": "ncu per-kernel captures (profiles/), scaled to a token",
                     "peak_source": peak_src, "per": "token (one graph launch)", "algorithmic_bytes": bytes_per_token,
                     "frac_of_8TBs": achieved / (8000.0 * world), "kernels": kernels},
        "clocks": clocks.summary(),
        "checksum": int(np.bitwise_xor.reduce(out.astype(np.uint64))),
    }
    if not args.no_cpu_baseline and rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_baseline(cfg)
    if rank == 0:
        print(json.dumps(line))
    model.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
