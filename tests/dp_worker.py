"""Child process of tests/test_gpu_dp.py: one data-parallel rank driving libseraph_b200 directly (no torch, so that the
NCCL the library opens with dlopen is the one LD_LIBRARY_PATH offers).  Not collected by pytest.

    python dp_worker.py real  <rank> <world> <dir> <accum>     two or more real ranks over NCCL, one GPU each
    python dp_worker.py lora  <rank> <world> <dir>             the same with a LoRA step (adapters on all seven projections)
    python dp_worker.py fake  <mode> <dir>                     one rank of a pretended world of 2 over a fake libnccl.so.2
"""
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))


def real(rank, world, d, accum):
    from seraph_b200 import api
    import oracle_lib as O
    cfg, ss = O.TINY, np.array(O.TINY_SEQS, np.int32)
    ctx = api.Context(rank)
    # rank, world and the id file come from the environment the parent set (RANK, WORLD_SIZE, SERAPH_DP_ID_FILE)
    assert ctx.lib.seraph_dp_init_from_env(ctx.h) == 0
    assert ctx.lib.seraph_dp_world(ctx.h) == world
    assert ctx.lib.seraph_dp_all_min(ctx.h, 5 + rank) == 5 and ctx.lib.seraph_dp_all_min(ctx.h, 1 if rank else 0) == 0
    p = cfg.init_params(7, norm_jitter=0.1)                         # same weights on every rank
    st = api.TrainState(cfg, p, accum=accum)
    losses = []
    for micro in range(accum):
        tok = np.random.default_rng(100 + 10 * rank + micro).integers(0, cfg.V, int(ss[-1])).astype(np.int32)
        losses.append(api.step_full_batch(ctx, st, tok, ss))
    ctx.check()
    assert ctx.lib.seraph_dp_wait(ctx.h, 20000) == 0
    ctx.lib.cuda_download_gpu_gradients(ctx.h, st.h)
    ctx.lib.cuda_download_full_weights(ctx.h, st.h)
    np.savez(os.path.join(d, f"rank{rank}.npz"), w=st.get(0), g=st.get(1), m=st.get(2), v=st.get(3), loss=np.array(losses),
             counters=np.array(st.counters()))
    st.close()
    ctx.close()


LORA = dict(rank=4, alpha=8.0, mask=0x7F, seed=9)


def lora(rank, world, d):
    """Every rank steps the same adapters on its own tokens; only the adapters' gradients are reduced."""
    from seraph_b200 import api
    import oracle_lib as O
    cfg, ss = O.TINY, np.array(O.TINY_SEQS, np.int32)
    ctx = api.Context(rank)
    assert ctx.lib.seraph_dp_init_from_env(ctx.h) == 0 and ctx.lib.seraph_dp_world(ctx.h) == world
    p = cfg.init_params(7, norm_jitter=0.1)
    _, n = cfg.lora_tensors(LORA["rank"], LORA["mask"])
    lo = (0.05 * np.random.default_rng(LORA["seed"]).standard_normal(n)).astype(np.float32)
    st = api.TrainState(cfg, p)
    st.attach_lora(LORA["rank"], LORA["alpha"], LORA["mask"], lo)
    assert ctx.lib.seraph_b200_set_lora_exact(ctx.h, 1) == 0
    tok = np.random.default_rng(200 + rank).integers(0, cfg.V, int(ss[-1])).astype(np.int32)
    loss = api.step_lora_batch(ctx, st, tok, ss)
    ctx.check()
    assert ctx.lib.seraph_dp_wait(ctx.h, 20000) == 0
    ctx.lib.cuda_download_lora_weights(ctx.h, st.lora_ptr())
    np.savez(os.path.join(d, f"lora_rank{rank}.npz"), w=st.lora_get(0), g=st.lora_get(1), loss=np.array([loss]))
    st.close()
    ctx.close()


def fake(mode, d):
    """world of 2 with a libnccl.so.2 that only pretends: its all-reduce parks a host callback on the stream that sleeps
    FAKE_NCCL_SLEEP_MS, its asynchronous-error query reports FAKE_NCCL_ASYNC_ERROR.  Nothing on the GPU waits or faults."""
    from seraph_b200 import api
    import oracle_lib as O
    cfg, ss = O.TINY, np.array(O.TINY_SEQS, np.int32)
    ctx = api.Context(0)
    uid = np.zeros(128, np.uint8)
    assert ctx.lib.seraph_dp_get_unique_id(uid.ctypes.data) == 0
    assert bytes(uid[:4]) == b"FAKE", "the fake NCCL was not the one loaded"
    assert ctx.lib.seraph_dp_init(ctx.h, 0, 2, uid.ctypes.data) == 0
    st = api.TrainState(cfg, cfg.init_params(7))
    tok = np.random.default_rng(1).integers(0, cfg.V, int(ss[-1])).astype(np.int32)
    out = {}
    if mode == "timeout":
        # the pretended all-reduce outlasts SERAPH_B200_DP_TIMEOUT_MS: the step gives up on the host, aborts the communicator
        # and returns -1 instead of hanging in its stream synchronisation
        t0 = time.time()
        loss = api.step_full_batch(ctx, st, tok, ss)
        out["step_rc"], out["step_s"] = float(loss), time.time() - t0
        out["world_after"] = int(ctx.lib.seraph_dp_world(ctx.h))
        out["status"] = int(ctx.status())
        ctx.sync()                                                  # the parked callbacks end by themselves; the context stays usable
        loss2 = api.step_full_batch(ctx, st, tok, ss)               # single-GPU from here on
        out["loss_after_finite"] = bool(np.isfinite(loss2) and loss2 > 0)
    elif mode == "async_error":
        loss = api.step_full_batch(ctx, st, tok, ss)
        out["step_rc"] = float(loss)
        out["world_after"] = int(ctx.lib.seraph_dp_world(ctx.h))
        out["status"] = int(ctx.status())
    elif mode == "ok":
        loss = api.step_full_batch(ctx, st, tok, ss)
        out["loss_finite"] = bool(np.isfinite(loss))
        out["wait_rc"] = int(ctx.lib.seraph_dp_wait(ctx.h, 5000))
        out["world_after"] = int(ctx.lib.seraph_dp_world(ctx.h))
        ctx.lib.seraph_dp_finalize(ctx.h)
        out["world_final"] = int(ctx.lib.seraph_dp_world(ctx.h))
    st.close()
    ctx.close()
    import json
    with open(os.path.join(d, "fake_result.json"), "w") as f:
        json.dump(out, f)


if __name__ == "__main__":
    if sys.argv[1] == "real":
        real(int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], int(sys.argv[5]))
    elif sys.argv[1] == "lora":
        lora(int(sys.argv[2]), int(sys.argv[3]), sys.argv[4])
    else:
        fake(sys.argv[2], sys.argv[3])
