"""In-kernel timelines of the token loop, for latency studies (a developer diagnostic, not part of the product path).

Builds a second copy of the library with the timeline probes compiled in (`-DIB_TOKEN_TRACE -DIB_STREAM_TRACE`:
`%globaltimer` stamps written by a few chosen warps; the shipped library contains none of them), runs the Llama-3-8B
architecture with synthetic weights for a few tokens and prints, in microseconds:

  python -m inferi_b200.timeline --mode token [--layers 8]   phases of the whole-token kernel (token_kernel.cu): for CTA 0
        the moments a phase starts, its grid barrier completes, activations are converted, registers are loaded, the first
        tile lands, the phase is done; over all CTAs the spread of "done"; for the producer lane of CTA 0 when it starts and
        stops issuing the phase's copies
  python -m inferi_b200.timeline --mode graph                 kernels of the last layer of the token graph (gemv_stream.cu):
        CTA 0's marks and the per-CTA spread of "activations converted" and "kernel end"
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import subprocess
import sys

import numpy as np

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
TRACE_LIB = os.path.join(PKG_DIR, "libinferi_b200_trace.so")


def build_trace_library() -> str:
    from . import build as b
    out_dir = os.path.join(PKG_DIR, "build_trace")
    os.makedirs(out_dir, exist_ok=True)
    nvcc = b._nvcc()
    procs, objs = [], []
    for src in b.SOURCES:
        obj = os.path.join(out_dir, src.replace(".cu", ".o"))
        objs.append(obj)
        procs.append(subprocess.Popen([nvcc, *b.NVCC_FLAGS, "-DIB_TOKEN_TRACE", "-DIB_STREAM_TRACE", "-c", os.path.join(b.CSRC, src), "-o", obj],
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    for p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError("nvcc failed")
    subprocess.run([nvcc, "-shared", "-o", TRACE_LIB, *objs, "-lcudart_static", "-lpthread", "-ldl", "-lrt"], check=True)
    return TRACE_LIB


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["token", "graph"], default="token")
    ap.add_argument("--layers", type=int, default=8, help="layers of the model (token mode prints the first 64 phases)")
    ap.add_argument("--no-build", action="store_true", help="use an existing trace library")
    args = ap.parse_args()
    if not args.no_build or not os.path.exists(TRACE_LIB):
        build_trace_library()
    os.environ["INFERI_B200_TOKEN_KERNEL"] = "1" if args.mode == "token" else "0"

    import torch
    from . import _lib
    _lib.LIB_PATH = TRACE_LIB
    from .llama2 import LLAMA_3_8B, Llama2, Llama2Config, Llama2Weights, synth_weights
    from .ops import Backend

    layers = args.layers if args.mode == "token" else 32
    cfg = Llama2Config(**{**LLAMA_3_8B.__dict__, "num_hidden_layers": layers})
    torch.cuda.set_device(0)
    be = Backend(0)
    lib = be.lib
    model = Llama2(be, cfg, Llama2Weights(be, cfg, synth_weights(cfg, seed=1, device="cuda")))
    prompt = np.arange(1, 200, dtype=np.uint32)
    model.generate(prompt, 1)          # the probes keep the last token's stamps: position 198
    torch.cuda.synchronize()

    if args.mode == "token":
        t = np.zeros((5, 64, 8), dtype=np.uint64)
        done = np.zeros((64, 160), dtype=np.uint64)
        lib.ib_debug_token_trace.argtypes = [C.c_void_p]
        lib.ib_debug_token_done.argtypes = [C.c_void_p]
        lib.ib_debug_token_trace(t.ctypes.data_as(C.c_void_p))
        lib.ib_debug_token_done(done.ctypes.data_as(C.c_void_p))
        t, done = t.astype(np.int64), done.astype(np.int64)[:, :be.sm_count if hasattr(be, "sm_count") else 148]
        t0 = t[0, 0, 0]
        names = ["qkv", "attn", "o", "gu", "dn"]
        print("phase | CTA 0: start barrier converted registers first_tile done | all CTAs done: min median max | producer of CTA 0: start stop")
        for ph in range(min(64, 5 * layers + 1)):
            r = (t[0, ph] - t0) / 1000.0
            dd = (done[ph] - t0) / 1000.0
            pr = (t[4, ph, :2] - t0) / 1000.0
            nm = names[ph % 5] if ph < 5 * layers else "cls"
            marks = [r[0], r[1]] + ([r[2], r[6], r[3]] if nm != "attn" else [float("nan")] * 3) + [r[4]]
            print(f"{ph:3d} {nm:4s} | " + " ".join(f"{v:8.2f}" for v in marks) + f" | {dd.min():8.2f} {np.median(dd):8.2f} {dd.max():8.2f} | {pr[0]:8.2f} {pr[1]:8.2f}")
    else:
        t = np.zeros(256, dtype=np.uint64)
        ends, packed = np.zeros(8 * 160, dtype=np.uint64), np.zeros(8 * 160, dtype=np.uint64)
        lib.ib_debug_stream_trace.argtypes = [C.c_void_p]
        lib.ib_debug_cta_times.argtypes = [C.c_void_p, C.c_void_p]
        lib.ib_debug_stream_trace(t.ctypes.data_as(C.c_void_p))
        lib.ib_debug_cta_times(ends.ctypes.data_as(C.c_void_p), packed.ctypes.data_as(C.c_void_p))
        names = {3: "qkv", 2: "gate/up", 1: "down (last layer)", 4: "classifier"}
        starts = {}
        print("kernel | CTA 0 (us from its start): set-up done, predecessor complete, converted, end | producer: first tiles issued at")
        for e in (3, 2, 1, 4):
            row, prow = t[e * 16:(e + 1) * 16].astype(np.int64), t[128 + e * 16:128 + (e + 1) * 16].astype(np.int64)
            t0 = row[0]
            starts[e] = t0
            c = [(row[i] - t0) / 1e3 for i in (1, 2, 3, 15)]
            pr = [(prow[i] - t0) / 1e3 for i in range(2, 9) if prow[i] >= t0 and prow[i] > 0]
            print(f"{names[e]:18s} | " + " ".join(f"{v:7.2f}" for v in c) + " | " + " ".join(f"{v:.2f}" for v in pr))
        print("gate/up start -> down start  %.2f us;  down start -> classifier start  %.2f us;  qkv start -> gate/up start (qkv + attention + o_proj)  %.2f us"
              % ((starts[1] - starts[2]) / 1e3, (starts[4] - starts[1]) / 1e3, (starts[2] - starts[3]) / 1e3))
        for e in (3, 2, 1, 4):
            en = (ends[e * 160:e * 160 + 148].astype(np.int64) - int(t[e * 16])) / 1e3
            pk = (packed[e * 160:e * 160 + 148].astype(np.int64) - int(t[e * 16])) / 1e3
            print(f"{names[e]:18s} converted: min {pk.min():.2f} median {np.median(pk):.2f} max {pk.max():.2f} | CTA end: min {en.min():.2f} p10 {np.percentile(en, 10):.2f} "
                  f"median {np.median(en):.2f} p90 {np.percentile(en, 90):.2f} max {en.max():.2f}")
        ph = np.zeros((8, 32, 10), dtype=np.int64)
        lib.ib_debug_consumer_phases.argtypes = [C.c_void_p]
        lib.ib_debug_consumer_phases(ph.ctypes.data_as(C.c_void_p))
        print("consumer warps of CTA 0, SM cycles per tile: wait for the tile | dot products | shuffle tree | partials or epilogue | "
              "cross-warp fold | slot release | loop bookkeeping || tiles | cycles in the loop")
        for e in (3, 2, 1, 4):
            rows = ph[e][ph[e][:, 6] > 0]
            if rows.size == 0:
                continue
            per = rows[:, [0, 1, 2, 3, 4, 5, 8]] / rows[:, 6:7]
            print(f"{names[e]:18s} median over {rows.shape[0]} warps: " + " | ".join(f"{v:7.0f}" for v in np.median(per, axis=0))
                  + f" || {np.median(rows[:, 6]):.0f} | {np.median(rows[:, 7]):.0f}")
            print(f"{'':18s} slowest warp:          " + " | ".join(f"{v:7.0f}" for v in per[np.argmax(rows[:, 7])])
                  + f" || {rows[np.argmax(rows[:, 7]), 6]:.0f} | {rows[:, 7].max():.0f}")
    model.close()


if __name__ == "__main__":
    main()
