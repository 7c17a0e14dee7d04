"""Data parallelism of the library itself (seraph_b200/csrc/dp.c), on GPUs.

* Two real ranks over NCCL (needs two GPUs; skipped on one): different tokens per rank, one step and a step with two
  accumulated micro-batches; the replicas end bit-identical and equal to AdamW on the mean of the per-rank oracle gradients.
* Failure paths with a pretended NCCL (a libnccl.so.2 built here that only records calls; failures are made on the host:
  an all-reduce that outlasts the step's time limit, an asynchronous error code).  Nothing on the GPU waits or faults."""
import json
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

import oracle_lib as O
from oracle_lib import TINY, TINY_SEQS, rel_l2

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "dp_worker.py")

FAKE_NCCL = textwrap.dedent(r"""
    #include <dlfcn.h>
    #include <stdlib.h>
    #include <string.h>
    #include <unistd.h>
    typedef struct { char internal[128]; } ncclUniqueId;
    typedef void* ncclComm_t;
    typedef int (*launch_host_fn)(void* stream, void (*fn)(void*), void* data);
    static launch_host_fn host_fn(void) {
        static launch_host_fn f;
        if (!f) { void* h = dlopen("libcuda.so.1", RTLD_NOW); if (h) f = (launch_host_fn)dlsym(h, "cuLaunchHostFunc"); }
        return f;
    }
    static void nap(void* ms) { usleep((useconds_t)(long)ms * 1000); }
    int ncclGetUniqueId(ncclUniqueId* id) { memset(id, 0, sizeof *id); memcpy(id, "FAKE", 4); return 0; }
    int ncclCommInitRank(ncclComm_t* c, int n, ncclUniqueId id, int rank) { (void)n; (void)id; (void)rank; *c = (void*)0x10; return 0; }
    int ncclAllReduce(const void* s, void* r, size_t n, int dt, int op, ncclComm_t c, void* stream) {
        (void)s; (void)r; (void)n; (void)dt; (void)op; (void)c;
        const char* e = getenv("FAKE_NCCL_SLEEP_MS");
        long ms = e ? atol(e) : 0;
        if (ms > 0 && host_fn()) host_fn()(stream, nap, (void*)ms);
        return 0;
    }
    int ncclCommDestroy(ncclComm_t c) { (void)c; return 0; }
    int ncclCommAbort(ncclComm_t c) { (void)c; return 0; }
    int ncclCommGetAsyncError(ncclComm_t c, int* r) { (void)c; const char* e = getenv("FAKE_NCCL_ASYNC_ERROR"); *r = (e && e[0] == '1') ? 1 : 0; return 0; }
    const char* ncclGetErrorString(int r) { (void)r; return "pretended NCCL error"; }
""")


def gpu_count():
    import torch
    return torch.cuda.device_count()


def run_fake(tmp_path, mode, env_extra):
    src = tmp_path / "fake_nccl.c"
    src.write_text(FAKE_NCCL)
    subprocess.run(["gcc", "-O1", "-shared", "-fPIC", "-o", str(tmp_path / "libnccl.so.2"), str(src), "-ldl"], check=True)
    env = dict(os.environ, LD_LIBRARY_PATH=str(tmp_path) + ":" + os.environ.get("LD_LIBRARY_PATH", ""), CUDA_VISIBLE_DEVICES="0", **env_extra)
    subprocess.run([sys.executable, WORKER, "fake", mode, str(tmp_path)], env=env, check=True, timeout=300)
    return json.load(open(tmp_path / "fake_result.json"))


def test_step_gives_up_on_collectives_that_outlast_the_limit(tmp_path):
    r = run_fake(tmp_path, "timeout", dict(FAKE_NCCL_SLEEP_MS="1200", SERAPH_B200_DP_TIMEOUT_MS="150"))
    assert r["step_rc"] == -1.0 and r["status"] == 5 and r["world_after"] == 1       # SB_ERR_TIMEOUT, communicator dropped
    assert r["step_s"] < 1.2                                                             # did not sit out the 3 x 1.2 s of parked collectives
    assert r["loss_after_finite"]


def test_asynchronous_nccl_error_aborts_the_communicator(tmp_path):
    r = run_fake(tmp_path, "async_error", dict(FAKE_NCCL_ASYNC_ERROR="1"))
    assert r["step_rc"] == -1.0 and r["status"] == 6 and r["world_after"] == 1        # SB_ERR_NCCL


def test_pretended_world_steps_and_finalizes(tmp_path):
    r = run_fake(tmp_path, "ok", {})
    assert r["loss_finite"] and r["wait_rc"] == 0 and r["world_after"] == 2 and r["world_final"] == 1


@pytest.mark.parametrize("accum", [1, 2])
def test_two_ranks_over_nccl_stay_identical_and_match_the_oracle(tmp_path, accum):
    if gpu_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    procs = [subprocess.Popen([sys.executable, WORKER, "real", str(r), str(world), str(tmp_path), str(accum)],
                              env=dict(os.environ, NCCL_NVLS_ENABLE="0", RANK=str(r), WORLD_SIZE=str(world),
                                       SERAPH_DP_ID_FILE=str(tmp_path / "nccl_id.bin"))) for r in range(world)]
    for p in procs:
        assert p.wait(timeout=600) == 0
    out = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    for k in ("w", "g", "m", "v"):
        assert np.array_equal(out[0][k], out[1][k]), k                 # replicas bit-identical after the step
    assert tuple(out[0]["counters"]) == (1, 0)
    cfg = TINY
    p = cfg.init_params(7, norm_jitter=0.1)
    g_sum = np.zeros_like(p)
    for r in range(world):
        for micro in range(accum):
            tok = np.random.default_rng(100 + 10 * r + micro).integers(0, cfg.V, TINY_SEQS[-1]).astype(np.int32)
            ref = O.train_step(cfg, p, tok, TINY_SEQS)
            g_sum += ref["grads"]
            assert abs(out[r]["loss"][micro] - ref["loss"]) < 1e-5 * abs(ref["loss"])
    assert rel_l2(out[0]["g"], g_sum) < 1e-5                           # the arena holds the NCCL sum; 1/world is applied inside AdamW
    lr = O.lib().ref_effective_lr(3.14e-4, 1, accum)
    w, m, v = p.copy(), np.zeros_like(p), np.zeros_like(p)
    O.lib().ref_adamw(w, (g_sum / world).astype(np.float32), m, v, p.size, lr, 0.9, 0.999, 0.01, 1e-8, 1)
    assert rel_l2(out[0]["w"], w) < 1e-6 and rel_l2(out[0]["m"], m) < 1e-5


def test_two_ranks_lora_step_reduces_the_adapter_gradients(tmp_path):
    """LoRA under data parallelism: each rank steps the same adapters (all seven projections, full chain rule) on its own
    tokens; the adapters' gradients are summed over NCCL layer by layer, AdamW applies their mean.  Both ranks end with
    bit-identical adapters, equal to the oracle's AdamW on the mean of the two oracle gradients."""
    if gpu_count() < 2:
        pytest.skip("needs two GPUs")
    import dp_worker as W
    world = 2
    procs = [subprocess.Popen([sys.executable, WORKER, "lora", str(r), str(world), str(tmp_path)],
                              env=dict(os.environ, NCCL_NVLS_ENABLE="0", RANK=str(r), WORLD_SIZE=str(world),
                                       SERAPH_DP_ID_FILE=str(tmp_path / "nccl_id.bin"))) for r in range(world)]
    for p in procs:
        assert p.wait(timeout=600) == 0
    out = [np.load(tmp_path / f"lora_rank{r}.npz") for r in range(world)]
    assert np.array_equal(out[0]["w"], out[1]["w"]) and np.array_equal(out[0]["g"], out[1]["g"])
    cfg, L = TINY, W.LORA
    p = cfg.init_params(7, norm_jitter=0.1)
    _, n = cfg.lora_tensors(L["rank"], L["mask"])
    lo = (0.05 * np.random.default_rng(L["seed"]).standard_normal(n)).astype(np.float32)
    g_sum = np.zeros(n, np.float32)
    for r in range(world):
        tok = np.random.default_rng(200 + r).integers(0, cfg.V, TINY_SEQS[-1]).astype(np.int32)
        ref = O.train_step(cfg, p, tok, TINY_SEQS, lora=lo, rank=L["rank"], alpha=L["alpha"], mask=L["mask"], lora_exact=1)
        g_sum += ref["grads"]
        assert abs(out[r]["loss"][0] - ref["loss"]) < 1e-5 * abs(ref["loss"])
    assert rel_l2(out[0]["g"], g_sum) < 1e-5
    w, m, v = lo.copy(), np.zeros_like(lo), np.zeros_like(lo)
    O.lib().ref_adamw(w, (g_sum / world).astype(np.float32), m, v, n, O.lib().ref_effective_lr(3.14e-4, 1, 1), 0.9, 0.999, 0.01, 1e-8, 1)
    assert rel_l2(out[0]["w"], w) < 1e-6
