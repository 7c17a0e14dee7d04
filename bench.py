#!/usr/bin/env python
"""Benchmark of the training step (forward + backward + AdamW) through libseraph_b200.

    python bench.py --gpus N --steps K --warmup W          # one process per GPU; N>1 under torchrun
    python bench.py --impl reference ...                    # the reference's own CPU path, timed on host cores
    python bench.py --workload 4                            # the isolated attention-backward microbenchmark

Prints ONE JSON line (rank 0).  Default workload: the Qwen3-1.7B-shaped decoder of the
baseline's data-parallel configuration (full-weight FP32 training, per-rank
micro-batch 4 x 2048 uniform random tokens, random N(0,0.02) weights from a seed),
weak scaling: every rank runs the full step on its own micro-batch and gradients
are all-reduced with NCCL while backward still runs.

value  : tokens/s with the batch already resident in HBM (no host<->device copies in the timed region)
e2e    : tokens/s through the public step call with host token buffers (upload + loss read-back inside)
roofline / per_class : CUDA-event time per kernel class, recorded on the library's stream during the timed steps
cpu_baseline / reference_cuda : the reference's own CPU path and its own CUDA backend, timed on this box (baselines only)
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

QWEN = dict(V=151936, d=2048, L=28, Hq=16, Hkv=8, hd=128, F=6144, theta=1e6, head_norm=1)    # per-head q/k RMSNorm, tied embeddings
SMALL = dict(V=8192, d=512, L=8, Hq=8, Hkv=8, hd=64, F=1408, theta=10000.0)
SLICE = dict(V=16384, d=2048, L=2, Hq=16, Hkv=8, hd=128, F=6144, theta=1e6, head_norm=1)     # two Qwen3-1.7B-shaped layers: small enough to profile
MISTRAL4 = dict(V=32000, d=4096, L=4, Hq=32, Hkv=8, hd=128, F=14336, theta=1e6, untied=1)  # four of the 32 Mistral-7B-shaped layers, separate lm_head
WORKLOADS = {
    "qwen3-1.7b-shaped full-weight FP32, 4x2048 tokens per rank": dict(kind="full", model=QWEN, B=4, S=2048),
    "profiling slice: 2 qwen3-1.7b-shaped layers, vocab 16384, 2x2048 tokens": dict(kind="full", model=SLICE, B=2, S=2048),
    "33M Llama-style full-weight FP32, 8x256 tokens per rank": dict(kind="full", model=SMALL, B=8, S=256),
    "profiling slice with use_qk_norm: the same 2 layers, q and k normalised over the token row after RoPE":
        dict(kind="full", model=dict(SLICE, qk_norm=1), B=2, S=2048),
    "attention backward microbenchmark: B 8, H 16, S 2048, D 128, causal, FP32 in and out":
        dict(kind="attn", B=8, H=16, S=2048, D=128),
    "qwen3-1.7b-shaped LoRA rank 16 alpha 32 on q,k,v,o, frozen FP32 base, 4x2048 tokens":
        dict(kind="lora", model=QWEN, B=4, S=2048, rank=16, alpha=32.0, mask=0b0001111),
    "mistral-7b-shaped LoRA rank 64 on all seven projections, 4 of the 32 layers, untied head, 2x4096 tokens per rank":
        dict(kind="lora", model=MISTRAL4, B=2, S=4096, rank=64, alpha=128.0, mask=0x7F),
}
METRIC = "train tokens/sec (fwd+bwd+AdamW)"


def gemm_traffic(cfg, T, f16=True):
    """DRAM bytes of one launch of the dominant kernel: the FFN gate projection (M = T, N = ffn, K = hidden).
    One ncu capture of that launch at T = 4096, hidden 2048, ffn 6144 read 161.7 MB and wrote 83.5 MB of DRAM in the
    default mode (1.33 times its algorithmic 4*(M*K + N*K + M*N) bytes; with TF32 parts 151.4 + 75.1 MB, 1.23 times);
    a full-size launch is too long a capture, so that ratio is applied to the algorithmic bytes of the launch at this
    workload's T."""
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
        # nvidia-smi numbers the GPUs of the machine; a CUDA_VISIBLE_DEVICES list of indices renumbers them for the process
        vis = [v.strip() for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip()]
        if vis and all(v.isdigit() for v in vis) and 0 <= index < len(vis):
            index = int(vis[index])
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


def flops_per_token(mc, S):
    """fwd + bwd of the linear layers and the LM head (6 per parameter) and of causal attention (7 * Hq * hd * S)"""
    qd, kvd = mc["Hq"] * mc["hd"], mc["Hkv"] * mc["hd"]
    p_lin = mc["L"] * (2 * qd * mc["d"] + 2 * kvd * mc["d"] + 3 * mc["F"] * mc["d"]) + mc["V"] * mc["d"]
    return 6.0 * p_lin + 7.0 * mc["Hq"] * mc["hd"] * S * mc["L"]


def seeded_params(cfg, seed=1234):
    rng = np.random.default_rng(seed)
    params = np.empty(cfg.n_params(), np.float32)
    for name, shp, off in cfg.tensors():
        n = int(np.prod(shp))
        if name.endswith("norm"):
            params[off:off + n] = 1.0
        else:
            params[off:off + n] = rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)
    return params


# ------------------------------------------------------------------------------------------------------------------
# baselines: the reference's own code (oracle/_ref), timed on this box.  Never on the product path.
# ------------------------------------------------------------------------------------------------------------------
def _oracle_lib():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    return O


def cpu_reference_sample(mc, S_workload, builds=("cpu_fast",), seq_lens=(32, 64)):
    """The reference's own CPU training path (train_step of src/train.c compiled unmodified into oracle/_ref),
    single-threaded as written, on the configuration it can run: the 33M model of configuration 1.  One call each at two
    sequence lengths fits t(S) = a S + b S^2 (the backward re-projects K and V for every earlier position,
    src/train.c:4012-4026), which gives the time of a 256-token sequence of configuration 1; the benchmark workload's
    tokens/s follows by the ratio of FLOPs per token.  Bounded: about 15 s per build."""
    O = _oracle_lib()
    from seraph_b200.config import ModelCfg
    cfg = ModelCfg(**SMALL)
    out = {"unit": "tokens/s", "cores": 1, "kind": "reference", "host_cores_present": os.cpu_count(), "builds": {}}
    p = seeded_params(cfg, 7)
    total = 0.0
    for kind in builds:
        L = O.ref_lib(kind)
        if L is None:
            continue
        st = O.ref_state(L, cfg, max(seq_lens), lr=3.14e-4, accum=1)
        L.refshim_set(st, 0, p)
        rng = np.random.default_rng(8)
        t = {}
        for S in seq_lens:
            tok = rng.integers(0, cfg.V, S).astype(np.int32)
            t0 = time.perf_counter()
            L.refshim_train_step(st, tok, S)
            t[S] = time.perf_counter() - t0
        L.refshim_destroy(st)
        s1, s2 = seq_lens
        b = (t[s2] / s2 - t[s1] / s1) / (s2 - s1)
        a = t[s1] / s1 - b * s1
        t256 = a * 256 + max(b, 0.0) * 256 * 256
        c1 = 256.0 / t256
        out["builds"][kind] = {"seconds": {str(k): round(v, 3) for k, v in t.items()}, "config1_seconds_per_256_token_sequence": t256,
                               "config1_tokens_per_s": c1}
        total += sum(t.values())
    if not out["builds"]:
        out.update(value=None, sample="oracle/_ref not built")
        return out
    best = "cpu_fast" if "cpu_fast" in out["builds"] else list(out["builds"])[0]
    ratio = flops_per_token(SMALL, 256) / flops_per_token(mc, S_workload)
    out["value"] = out["builds"][best]["config1_tokens_per_s"] * ratio
    out["seconds_sampled"] = total
    out["sample"] = (f"reference CPU train_step (1 thread; build '{best}' = the reference Makefile's -O3 -ffast-math flags"
                     f"{', also the plain -O3 build' if len(out['builds']) > 1 else ''}) on configuration 1's 33M model: one sequence of "
                     f"{seq_lens[0]} and one of {seq_lens[1]} tokens, fitted a*S + b*S^2 and evaluated at S = 256 "
                     f"({out['builds'][best]['config1_tokens_per_s']:.2f} tok/s); not run at this workload's size, extrapolated from "
                     f"configuration 1 by the ratio of FLOPs per token ({ratio:.3e}); its backward is a truncated approximation")
    return out


def reference_cuda_legs(device):
    """The reference's own CUDA backend (src/cuda_train_context.cu + src/train_cuda.c compiled unmodified into oracle/_ref)
    on this GPU: the full step of configuration 1 and the flash attention forward/backward of configuration 2.  It cannot
    run hidden sizes above 1024 (blockDim = hidden_size), so not the benchmark workload."""
    import ctypes as C
    O = _oracle_lib()
    from seraph_b200.config import ModelCfg
    L = O.ref_lib("cuda")
    if L is None:
        return {"unavailable": "oracle/_ref/libseraph_ref_cuda.so not built"}
    out = {}
    try:
        cfg = ModelCfg(**SMALL)
        p = seeded_params(cfg, 7)
        ss = np.arange(0, 2049, 256, dtype=np.int32)
        tok = np.random.default_rng(9).integers(0, cfg.V, 2048).astype(np.int32)
        st = O.ref_state(L, cfg, 2048)
        L.refshim_set(st, 0, p)
        if L.refshim_cuda_init(st, device, 0) != 0:
            return {"unavailable": "reference cuda_train_init failed"}
        L.refshim_cuda_step(st, tok, 2048, ss, 8)
        t0 = time.perf_counter()
        reps = 3
        for _ in range(reps):
            loss = L.refshim_cuda_step(st, tok, 2048, ss, 8)       # the call synchronises and reads the loss back
        dt = (time.perf_counter() - t0) / reps
        L.refshim_destroy(st)
        out["c1_step_ms"] = dt * 1e3
        out["c1_tokens_per_s"] = 2048.0 / dt
        out["c1_loss"] = float(loss)
    except Exception as e:      # noqa: BLE001
        out["c1_unavailable"] = repr(e)
    try:
        B, H, S, D = 8, 16, 2048, 128
        T = B * S
        r = np.random.default_rng(2048)
        Q, K, V, dO = (np.ascontiguousarray(r.standard_normal((T, H * D)), np.float32) for _ in range(4))
        fn = L.refshim_cuda_attention
        fn.restype = C.c_int
        fn.argtypes = [C.c_int] + [O.f32p] * 4 + [O.i32p] + [C.c_int] * 7 + [O.f32p] * 6
        o, lse, dq = np.empty_like(Q), np.empty((T, H), np.float32), np.empty_like(Q)
        dk, dv, ms = np.empty_like(K), np.empty_like(V), np.zeros(2, np.float32)
        rc = fn(device, Q, K, V, dO, np.arange(0, T + 1, S, dtype=np.int32), B, T, H, H, D, S, 2, o, lse, dq, dk, dv, ms)
        if rc == 0:
            out["c2_attn_fwd_ms"], out["c2_attn_bwd_ms"] = float(ms[0]), float(ms[1])
            out["c2_attn_bwd_tflops"] = float(attention_flops(B, S, H, D)[1] / (float(ms[1]) * 1e-3) * 1e-12)
        else:
            out["c2_unavailable"] = f"reference attention call returned {rc}"
    except Exception as e:      # noqa: BLE001
        out["c2_unavailable"] = repr(e)
    return out


# ------------------------------------------------------------------------------------------------------------------
def dp_check(ctx, dist, torch, rank, world, local):
    """Before the timed region of an N-rank run: one data-parallel step of a small model with different tokens per rank.
    (i) the gradients the step leaves (the NCCL sum) against the sum of the per-rank gradients computed by a second,
    single-GPU context of this rank and added with torch.distributed; (ii) the weights after AdamW identical on all ranks."""
    from seraph_b200 import api
    from seraph_b200.config import ModelCfg
    cfg = ModelCfg(V=1024, d=512, L=2, Hq=4, Hkv=2, hd=128, F=1024, theta=1e4)
    p = cfg.init_params(21, norm_jitter=0.1)
    ss = np.array([0, 300, 512, 645], np.int32)
    tok = np.random.default_rng(500 + rank).integers(0, cfg.V, 645).astype(np.int32)
    solo = api.Context(local)
    st = api.TrainState(cfg, p)
    api.step_full_batch(solo, st, tok, ss)
    solo.lib.cuda_download_gpu_gradients(solo.h, st.h)
    g_local = st.get(1)
    st.close()
    solo.close()
    gs = torch.from_numpy(g_local.astype(np.float64)).cuda()
    dist.all_reduce(gs)
    st = api.TrainState(cfg, p)
    loss = api.step_full_batch(ctx, st, tok, ss)
    ctx.check()
    ctx.lib.cuda_download_gpu_gradients(ctx.h, st.h)
    ctx.lib.cuda_download_full_weights(ctx.h, st.h)
    g = st.get(1).astype(np.float64)
    w = st.get(0)
    st.close()
    ctx.lib.seraph_b200_reset_model(ctx.h)
    ref = gs.cpu().numpy()
    err = float(np.linalg.norm(g - ref) / np.linalg.norm(ref))
    import zlib
    crc = zlib.crc32(w.tobytes())
    t = torch.tensor([err, float(crc), float(loss)], dtype=torch.float64, device="cuda")
    allt = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(allt, t)
    errs = [float(x[0]) for x in allt]
    crcs = {int(x[1]) for x in allt}
    return {"max_rel_err": max(errs), "replicas_identical": len(crcs) == 1, "ranks": world,
            "what": "NCCL-summed gradient of one data-parallel step vs sum of per-rank gradients; CRC32 of the weights after AdamW on every rank"}


def run_attention(args, w):
    """Configuration 2: the isolated attention backward through cuda_train_batch_attention_backward_packed (forward once for
    the log-sum-exp).  Inputs resident; every timed call reads 5 and writes 3 tensors of B*S*H*D floats (1.07 GB), far more
    than L2."""
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    from seraph_b200 import api, build
    build.build()
    B, H, S, D = w["B"], w["H"], w["S"], w["D"]
    T = B * S
    ctx = api.Context(0)
    ctx.set_gemm_mode(args.gemm_mode)
    if args.attn_flash is not None:
        ctx.set_attn_flash(args.attn_flash)
    r = np.random.default_rng(2048)
    Q, K, V, dO = (np.ascontiguousarray(r.standard_normal((T, H * D)), np.float32) for _ in range(4))
    ss = np.arange(0, T + 1, S, dtype=np.uint32)
    bq, bk, bv, bdo, bs = ctx.upload(Q), ctx.upload(K), ctx.upload(V), ctx.upload(dO), ctx.upload(ss)
    bout, blse = ctx.zeros(Q.size), ctx.zeros(T * H)
    bdq, bdk, bdv = ctx.empty(Q.size), ctx.zeros(K.size), ctx.zeros(V.size)

    def fwd():
        ctx.lib.cuda_train_batch_attention_packed(ctx.h, bq.b, bk.b, bv.b, bout.b, blse.b, bs.b, T, B, H, H, D, S)

    def bwd():
        ctx.lib.cuda_train_batch_attention_backward_packed(ctx.h, bq.b, bk.b, bv.b, bout.b, blse.b, bdo.b, bdq.b, bdk.b, bdv.b, bs.b,
                                                           T, B, H, H, D, S)
    n_warm = max(args.warmup, 3)
    fwd()
    for _ in range(n_warm):
        bwd()
    ctx.sync()
    ctx.check()
    sampler = ClockSampler(0)
    sampler.start()
    ctx.launches(reset=True)
    ctx.timer_start()
    for _ in range(args.steps):
        bwd()
    ms = ctx.timer_stop()
    launches = ctx.launches()
    ctx.timer_start()
    for _ in range(args.steps):
        fwd()
    ms_f = ctx.timer_stop()
    # end to end: host arrays in, gradients back out, every step
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for b_, a_ in ((bq, Q), (bk, K), (bv, V), (bdo, dO)):
            ctx.lib.cuda_train_buffer_upload(ctx.h, b_.b, a_.ctypes.data, a_.size)
        bwd()
        bdq.numpy(); bdk.numpy(); bdv.numpy()
    ms_e2e = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    ctx.check()
    pk, pk_kind = peaks()
    f_fwd, f_bwd = attention_flops(B, S, H, D)
    t = ms / args.steps * 1e-3
    useful = f_bwd / t * 1e-12
    peak = pk["bf16_tflops_sustained"]
    line = {"metric": "attention backward useful TFLOP/s (5*B*H*S^2*D causal)", "value": useful, "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "warmup": n_warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "l2": "1.07 GB touched per call, far beyond the 126 MB L2; no flush needed",
                       "gemm_mode": args.gemm_mode},
            "forward_ms": ms_f / args.steps, "forward_tflops": f_fwd / (ms_f / args.steps * 1e-3) * 1e-12,
            "e2e": {"value": f_bwd / (ms_e2e / args.steps * 1e-3) * 1e-12, "unit": "TFLOP/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(4 * Q.nbytes), "d2h_bytes_per_step": int(3 * Q.nbytes)},
            "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "attention_bwd", "achieved": useful, "peak": peak, "unit": "TFLOP/s",
                         "frac": useful / peak, "issued_tflops": useful * 3 * args.attn_products / 5.0,
                         "issued_frac": useful * 3 * args.attn_products / 5.0 / peak,
                         # DRAM bytes of the at_dkv_bwd_kernel launch from one ncu capture at this shape (1.38 GB read, 1.56 GB written),
                         # scaled by the score elements when another shape is benchmarked
                         "traffic": 2.94e9 * (B * H * S * S) / (8.0 * 16 * 2048 * 2048),
                         "peak_note": f"{pk_kind} bf16 sustained {peak} TFLOP/s (FP16 MMAs run at the BF16 rate); achieved = useful FLOPs of the "
                                      f"whole call (operand preparation, the on-chip dK/dV kernel, the dQ product); issued = three FP16 passes "
                                      f"per product x {args.attn_products} products per block; the dK/dV kernel alone issues 0.67 of the peak "
                                      f"(ncu, tensor pipe 49 % active)"}}
    if not args.no_cpu_baseline:
        line["reference_cuda"] = reference_cuda_legs(0)
    os.write(real_stdout, (json.dumps(line, default=float) + "\n").encode())
    ctx.close()


def run_ours(args):
    w = WORKLOADS[args.workload]
    if w["kind"] == "attn":
        return run_attention(args, w)
    # libraries (NCCL among them) may print to stdout; keep fd 1 for the one JSON line
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    import torch
    import torch.distributed as dist
    from seraph_b200 import api, build
    from seraph_b200.config import ModelCfg

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
    mc, B, S = w["model"], w["B"], w["S"]
    lora = w["kind"] == "lora"
    cfg = ModelCfg(**mc)
    T = B * S
    ref_cuda = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline and w["kind"] == "full":
        ref_cuda = reference_cuda_legs(local)        # before this library's arenas take the memory
    ctx = api.Context(local)
    ctx.set_gemm_mode(args.gemm_mode)
    if args.attn_flash is not None:
        ctx.set_attn_flash(args.attn_flash)
    dpc = None
    if world > 1:
        uid = np.zeros(128, np.uint8)
        if rank == 0:
            assert ctx.lib.seraph_dp_get_unique_id(uid.ctypes.data) == 0
        t = torch.from_numpy(uid).cuda()
        dist.broadcast(t, 0)
        uid = t.cpu().numpy()
        assert ctx.lib.seraph_dp_init(ctx.h, rank, world, uid.ctypes.data) == 0, "seraph_dp_init failed"
        dpc = dp_check(ctx, dist, torch, rank, world, local)
    if cfg.head_norm or cfg.untied:
        x = cfg.init_extras(4321, norm_jitter=0.0)
        assert ctx.lib.seraph_b200_set_model_extras(ctx.h, cfg.head_norm, cfg.untied, x.ctypes.data, x.size) == 0
        del x
    # same weights on every rank (seed), different tokens per rank
    params = seeded_params(cfg)
    st = api.TrainState(cfg, params, lr=3.14e-4, accum=1, lean=True)
    del params
    if lora:
        n_l = cfg.lora_tensors(w["rank"], w["mask"])[1]
        lo = (0.02 * np.random.default_rng(77).standard_normal(n_l)).astype(np.float32)
        st.attach_lora(w["rank"], w["alpha"], w["mask"], lo)
        assert ctx.lib.seraph_b200_set_lora_exact(ctx.h, 1) == 0
    trng = np.random.default_rng(1000 + rank)
    ss = np.arange(0, T + 1, S, dtype=np.int32)
    n_batches = args.warmup + args.steps + 1
    host_tok = torch.from_numpy(trng.integers(0, cfg.V, (n_batches, T)).astype(np.int32)).pin_memory()
    tok_np = host_tok.numpy()
    step_fn = ctx.lib.cuda_train_step_gpu_lora_batch if lora else ctx.lib.cuda_train_step_gpu_full_batch

    def public_step(i):
        return float(step_fn(st.h, tok_np[i].ctypes.data, T, ss.ctypes.data, B, ctx.h))

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
        assert ctx.lib.seraph_b200_step_resident(st.h, ctx.h, 0 if lora else 1) == 0
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
            "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": n_warm, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32" if args.gemm_mode in (0, 3, 4) else ("tf32" if args.gemm_mode == 1 else "bf16"),
            "data": "synthetic",
            "config": {"workload": args.workload, "tokens_per_rank": T, "global_tokens": T * world,
                       "parallelism": f"dp{world}", "gemm_mode": ["fp32x3_tcgen05", "tf32_tcgen05", "bf16_tcgen05", "fp32_cuda_cores", "fp32_f16x3_tcgen05"][args.gemm_mode],
                       "l2": "working set per step (weights 6.9 GB + activations) far exceeds the 126 MB L2; no flush needed",
                       "qk_norm": ("whole-row, unweighted, after RoPE (the reference's shader form)" if mc.get("qk_norm") else
                                   "learned per-head RMSNorm of q and k before RoPE, trained" if mc.get("head_norm") else "off"),
                       "lm_head": "separate lm_head [V, d]" if mc.get("untied") else "tied to the embedding",
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
        if lora:
            line["config"]["lora"] = {"rank": w["rank"], "alpha": w["alpha"], "adapters": [n for k, n in enumerate(cfg.LORA_NAMES) if w["mask"] >> k & 1],
                                      "chain_rule": "full (adapter term of dX included)", "base": "frozen FP32"}
        if dpc is not None:
            line["dp_check"] = dpc
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_reference_sample(mc, S)
            if ref_cuda is not None:
                line["reference_cuda"] = ref_cuda
        os.write(real_stdout, (json.dumps(line, default=float) + "\n").encode())
    st.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def run_reference(args):
    """The reference's own CPU implementation of the path on this box's host cores: ONE bounded sample (about a minute:
    both builds, two sequence lengths each), whatever --steps and --warmup say; rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    if w["kind"] == "attn":
        print(json.dumps({"impl": "reference", "unavailable": "the reference has no CPU attention-backward entry point to time alone; "
                          "its CUDA kernels are timed in the default arm's reference_cuda"}))
        return
    mc, B, S = w["model"], w["B"], w["S"]
    t0 = time.perf_counter()
    real_stdout = os.dup(1)          # the reference prints progress lines to stdout; keep fd 1 for the one JSON line
    os.dup2(2, 1)
    r = cpu_reference_sample(mc, S, builds=("cpu_fast", "cpu"))
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    if r.get("value") is None:
        print(json.dumps({"impl": "reference", "unavailable": r["sample"]}))
        return
    v = float(r["value"])
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": 1, "warmup": 0, "ms_per_step": B * S / v * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "tokens_per_rank": B * S, "parallelism": "cpu, 1 thread (the path is single-threaded)",
                   "same_config": False, "sampled_seconds": time.perf_counter() - t0},
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
                    help="a key of WORKLOADS or its index (0 = the benchmark configuration, 1 = profiling slice, 2 = 33M model, 3 = slice with "
                         "use_qk_norm, 4 = attention-backward microbenchmark, 5 = LoRA rank 16 on the benchmark model, 6 = Mistral-7B-shaped LoRA slice)")
    ap.add_argument("--gemm-mode", type=int, default=4, help="4 FP32-accurate tensor cores, FP16 parts where possible (default), 0 FP32-accurate with TF32 parts, 1 TF32, 2 BF16, 3 CUDA cores")
    ap.add_argument("--attn-products", type=int, default=5, help="matrix products per key/query block the attention backward issues (for the issued-FLOPs figure)")
    ap.add_argument("--attn-flash", type=int, default=None, help="attention path for 128-wide heads: 1 backward with dK/dV kept on chip, 2 score kernel + three products, 0 a launch per product (default: the library's)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU and reference-CUDA baseline legs")
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
