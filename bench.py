#!/usr/bin/env python
"""Benchmark of the training step (forward + backward + AdamW) through libseraph_b200.

    python bench.py --gpus N --steps K --warmup W          # one process per GPU; N>1 under torchrun
    python bench.py --impl reference ...                    # the reference's own CPU path, timed on host cores

Prints ONE JSON line (rank 0).  Workload: the Qwen3-1.7B-shaped decoder of the
baseline's data-parallel configuration (full-weight FP32 training, per-rank
micro-batch 4 x 2048 uniform random tokens, random N(0,0.02) weights from a seed),
weak scaling: every rank runs the full step on its own micro-batch and gradients
are all-reduced with NCCL while backward still runs.

value  : tokens/s with the batch already resident in HBM (no host<->device copies in the timed region)
e2e    : tokens/s through the public step call with host token buffers (upload + loss read-back inside)
roofline / per_class : CUDA-event time per kernel class, recorded on the library's stream during the timed steps
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

QWEN = dict(V=151936, d=2048, L=28, Hq=16, Hkv=8, hd=128, F=6144, theta=1e6)
SMALL = dict(V=8192, d=512, L=8, Hq=8, Hkv=8, hd=64, F=1408, theta=10000.0)
SLICE = dict(V=16384, d=2048, L=2, Hq=16, Hkv=8, hd=128, F=6144, theta=1e6)     # two Qwen3-1.7B-shaped layers: small enough to profile
WORKLOADS = {
    "qwen3-1.7b-shaped full-weight FP32, 4x2048 tokens per rank": (QWEN, 4, 2048),
    "profiling slice: 2 qwen3-1.7b-shaped layers, vocab 16384, 2x2048 tokens": (SLICE, 2, 2048),
    "33M Llama-style full-weight FP32, 8x256 tokens per rank": (SMALL, 8, 256),
    "profiling slice with use_qk_norm: the same 2 layers, q and k normalised over the token row after RoPE": (dict(SLICE, qk_norm=1), 2, 2048),
}


def gemm_traffic(cfg, T, f16=True):
    """DRAM bytes of one launch of the dominant kernel: the FFN gate projection (M = T, N = ffn, K = hidden).
    One ncu capture of that launch at T = 4096, hidden 2048, ffn 6144 read 161.7 MB and wrote 83.5 MB of DRAM in the
    default mode (1.33 times its algorithmic 4*(M*K + N*K + M*N) bytes; with TF32 parts 151.4 + 75.1 MB, 1.23 times;
    summaries under profiles/); a full-size launch is too long a capture, so that ratio is applied to the algorithmic
    bytes of the launch at this workload's T."""
    alg = 4.0 * (T * cfg.d + cfg.F * cfg.d + T * cfg.F)
    return (1.33 if f16 else 1.23) * alg


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return p, "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        pw = [float(r[2]) for r in self.rows if len(r) > 2 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for k, nm in enumerate(names):
                if len(r) > 4 + k and r[4 + k].lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


def attention_flops(B, S, Hq, hd):
    """causal: forward 2*B*Hq*S^2*hd (two products, half masked), backward 5*B*Hq*S^2*hd"""
    f = 2.0 * B * Hq * S * S * hd
    return f, 2.5 * f


def run_ours(args):
    # libraries (NCCL among them) may print to stdout; keep fd 1 for the one JSON line
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    import torch
    import torch.distributed as dist
    from seraph_b200 import api, build
    import oracle_lib as O

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 with torchrun"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    mc, B, S = WORKLOADS[args.workload]
    cfg = O.ModelCfg(**mc)
    T = B * S
    ctx = api.Context(local)
    ctx.set_gemm_mode(args.gemm_mode)
    if world > 1:
        uid = np.zeros(128, np.uint8)
        if rank == 0:
            assert ctx.lib.seraph_dp_get_unique_id(uid.ctypes.data) == 0
        t = torch.from_numpy(uid).cuda()
        dist.broadcast(t, 0)
        uid = t.cpu().numpy()
        assert ctx.lib.seraph_dp_init(ctx.h, rank, world, uid.ctypes.data) == 0, "seraph_dp_init failed"
    # same weights on every rank (seed), different tokens per rank
    rng = np.random.default_rng(1234)
    params = np.empty(cfg.n_params(), np.float32)
    for name, shp, off in cfg.tensors():
        n = int(np.prod(shp))
        if name.endswith("norm"):
            params[off:off + n] = 1.0
        else:
            params[off:off + n] = rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)
    st = api.TrainState(cfg, params, lr=3.14e-4, accum=1, lean=True)
    del params
    trng = np.random.default_rng(1000 + rank)
    ss = np.arange(0, T + 1, S, dtype=np.int32)
    n_batches = args.warmup + args.steps + 1
    host_tok = torch.from_numpy(trng.integers(0, cfg.V, (n_batches, T)).astype(np.int32)).pin_memory()
    tok_np = host_tok.numpy()

    def public_step(i):
        return float(ctx.lib.cuda_train_step_gpu_full_batch(st.h, tok_np[i].ctypes.data, T, ss.ctypes.data, B, ctx.h))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ctx.sync()

    # ---- warm-up through the public call (also uploads the model) ----
    loss0 = None
    n_warm = args.warmup if args.short_warmup else max(args.warmup, 3)
    for i in range(max(n_warm, 1)):
        loss0 = public_step(i % n_batches)
    ctx.check()

    # ---- timed region 1: resident batch, K steps, CUDA events on the library's stream ----
    sampler = ClockSampler(local)
    sampler.start()
    ctx.lib.seraph_b200_timing_enable(ctx.h, 1)
    barrier()
    ctx.launches(reset=True)
    ctx.timer_start()
    for _ in range(args.steps):
        assert ctx.lib.seraph_b200_step_full_resident(st.h, ctx.h) == 0
    ms = ctx.timer_stop()
    barrier()
    launches = ctx.launches()
    ncls = ctx.lib.seraph_b200_timing_classes()
    tim = np.zeros(ncls * 4, np.float64)
    ctx.lib.seraph_b200_timing_read(ctx.h, tim.ctypes.data)
    ctx.lib.seraph_b200_timing_enable(ctx.h, 0)
    loss_res = float(ctx.lib.seraph_b200_last_loss(ctx.h))

    # ---- timed region 2: public API with host buffers (H2D of the batch and D2H of the loss inside) ----
    barrier()
    t0 = time.perf_counter()
    ctx.timer_start()
    for i in range(args.steps):
        loss_e2e = public_step(args.warmup + i)
    ms_e2e = ctx.timer_stop()
    barrier()
    wall_e2e = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    ctx.check()

    if world > 1:
        tt = torch.tensor([ms, max(ms_e2e, wall_e2e)], device="cuda", dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(tt[0]), float(tt[1])
    else:
        ms_e2e = max(ms_e2e, wall_e2e)

    if rank == 0:
        pk, pk_kind = peaks()
        tokens = T * world * args.steps
        per_class = {}
        for k in range(ncls):
            nm = ctx.lib.seraph_b200_timing_class_name(k).decode()
            t_ms, fl, by, n = tim[4 * k:4 * k + 4]
            if n == 0:
                continue
            if nm == "attention_fwd":
                fl = attention_flops(B, S, cfg.Hq, cfg.hd)[0] * cfg.L * args.steps
            if nm == "attention_bwd":
                fl = attention_flops(B, S, cfg.Hq, cfg.hd)[1] * cfg.L * args.steps
            per_class[nm] = {"ms_per_step": t_ms / args.steps, "launches_per_step": n / args.steps,
                             "tflops": (fl / (t_ms * 1e-3) * 1e-12) if fl and t_ms else None,
                             "gbs": (by / (t_ms * 1e-3) * 1e-9) if by and t_ms else None}
        g = per_class.get("gemm", {})
        # kind::f16 MMAs (mode 4) run at the rate of the measured BF16 GEMM; kind::tf32 at half of it
        f16_mode = args.gemm_mode == 4
        tf32_peak = pk["bf16_tflops_sustained"] if f16_mode else pk["bf16_tflops_sustained"] / 2.0
        g_ms, g_n = tim[0], tim[3]
        g_fl = tim[1]
        achieved = (g_fl / g_n) / ((g_ms / g_n) * 1e-3) * 1e-12 if g_n else None
        line = {
            "metric": "train tokens/sec (fwd+bwd+AdamW)", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": n_warm, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32" if args.gemm_mode in (0, 3, 4) else ("tf32" if args.gemm_mode == 1 else "bf16"),
            "data": "synthetic",
            "config": {"workload": args.workload, "tokens_per_rank": T, "global_tokens": T * world,
                       "parallelism": f"dp{world}", "gemm_mode": ["fp32x3_tcgen05", "tf32_tcgen05", "bf16_tcgen05", "fp32_cuda_cores", "fp32_f16x3_tcgen05"][args.gemm_mode],
                       "l2": "working set per step (weights 6.9 GB + activations) far exceeds the 126 MB L2; no flush needed",
                       "optimizer": "AdamW lr 3.14e-4 (reference warm-up), betas 0.9/0.999, wd 0.01, no clip (the reference has none)"},
            "loss": loss_res, "loss_first": loss0,
            "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(2 * T * 4 + (B + 1) * 4), "d2h_bytes_per_step": 4, "loss": loss_e2e},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "gemm", "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
                         "frac": (achieved / tf32_peak) if achieved else None, "traffic": gemm_traffic(cfg, T, f16_mode),
                         "peak_note": (f"{pk_kind} bf16 sustained {pk['bf16_tflops_sustained']} TFLOP/s (FP16 MMAs run at the BF16 rate)"
                                       if f16_mode else
                                       f"{pk_kind} bf16 sustained {pk['bf16_tflops_sustained']} TFLOP/s halved for TF32 operands") +
                                      "; achieved counts useful FLOPs (2MNK) per launch over the step's GEMM launches, operand preparation "
                                      "included; the FP32-accurate modes issue 3x that on the tensor pipe; traffic = DRAM bytes of one FFN "
                                      "gate-projection launch (ncu capture at T=4096 scaled by algorithmic bytes)",
                         "share_of_step": (g.get("ms_per_step", 0) / (ms / args.steps)) if g else None},
            "per_class": per_class,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(mc, quick=True)
        os.write(real_stdout, (json.dumps(line) + "\n").encode())
    st.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(mc, quick=True, reps=1):
    """The reference's own CPU training path (train_step of src/train.c, compiled unmodified into
    oracle/_ref with the reference Makefile's optimisation flags), single-threaded as written.
    Bounded sample: the model's embedding/LM head with 1 and with 2 decoder layers on one short
    sequence; the per-layer time is the difference, and the full-depth step time is extrapolated
    linearly in the layer count (the sample is stated in the result)."""
    import oracle_lib as O
    L = O.ref_lib("cpu_fast") or O.ref_lib("cpu")
    if L is None:
        return {"value": None, "unit": "tokens/s", "cores": 1, "kind": "reference", "sample": "oracle/_ref not built"}
    n = 4 if quick else 16
    times = {}
    for layers in (1, 2):
        cfg = O.ModelCfg(**{**mc, "L": layers})
        p = np.zeros(cfg.n_params(), np.float32)
        rng = np.random.default_rng(7)
        for name, shp, off in cfg.tensors():
            k = int(np.prod(shp))
            p[off:off + k] = 1.0 if name.endswith("norm") else rng.standard_normal(k, dtype=np.float32) * np.float32(0.02)
        st = O.ref_state(L, cfg, n, lr=3.14e-4, accum=1)
        L.refshim_set(st, 0, p)
        tok = rng.integers(0, cfg.V, n).astype(np.int32)
        best = None
        for _ in range(reps):
            t0 = time.perf_counter()
            L.refshim_train_step(st, tok, n)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        times[layers] = best
        L.refshim_destroy(st)
        del p
    per_layer = max(times[2] - times[1], 1e-9)
    head = max(times[1] - per_layer, 0.0)
    full = head + per_layer * mc["L"]
    return {"value": n / full, "unit": "tokens/s", "cores": 1, "kind": "reference",
            "sample": f"train_step on one {n}-token sequence with 1 and 2 of the {mc['L']} layers "
                      f"({times[1]:.2f} s, {times[2]:.2f} s), extrapolated linearly to {mc['L']} layers; "
                      "the reference CPU path is single-threaded and its backward is a truncated approximation",
            "seconds_sampled": times[1] + times[2], "host_cores_present": os.cpu_count()}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    mc, B, S = WORKLOADS[args.workload]
    vals = []
    for i in range(max(args.warmup, 0) + args.steps):
        r = cpu_baseline(mc, quick=True)
        if i >= args.warmup:
            vals.append(r)
        if r["value"] is None:
            print(json.dumps({"impl": "reference", "unavailable": r["sample"]}))
            return
    v = float(np.mean([r["value"] for r in vals]))
    sec = float(np.mean([r["seconds_sampled"] for r in vals]))
    r = vals[-1]
    r["value"] = v
    print(json.dumps({
        "impl": "reference", "metric": "train tokens/sec (fwd+bwd+AdamW)", "value": v, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "tokens_per_rank": B * S, "parallelism": "cpu, 1 thread"},
        "cpu_baseline": r,
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=list(WORKLOADS)[0],
                    help="a key of WORKLOADS or its index (0 = the benchmark configuration, 1 = profiling slice, 2 = 33M model)")
    ap.add_argument("--gemm-mode", type=int, default=4, help="4 FP32-accurate tensor cores, FP16 parts where possible (default), 0 FP32-accurate with TF32 parts, 1 TF32, 2 BF16, 3 CUDA cores")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--short-warmup", action="store_true", help="honour --warmup below 3 (profiler captures only; not a valid bench number)")
    args = ap.parse_args()
    if args.workload.isdigit():
        args.workload = list(WORKLOADS)[int(args.workload)]
    assert args.workload in WORKLOADS, list(WORKLOADS)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
