"""Data-parallel semantics on CPU, two gloo ranks: every rank runs the step on its
own micro-batch, gradients are summed across ranks and AdamW applies the mean
(1/world folded into the gradient read).  With equal numbers of predictions per
rank this is exactly the step on the concatenated batch - which is what
the CUDA path does with NCCL.  The ranks here compute with the CPU oracle; the
exchange protocol (unique id from rank 0, bucket order: layers last to first,
then embedding + final norm) is the library's."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as O
from oracle_lib import TINY, rel_l2


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def bucket_ranges(cfg):
    """Gradient ranges in the order the step hands them to the all-reduce."""
    tens = cfg.tensors()
    first_layer = next(off for name, shp, off in tens if name.startswith("l0."))
    out = []
    for l in reversed(range(cfg.L)):
        offs = [(off, int(np.prod(shp))) for name, shp, off in tens if name.startswith(f"l{l}.")]
        out.append((offs[0][0], offs[-1][0] + offs[-1][1]))
    out.append((0, first_layer))
    return out


def worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = TINY
    p = cfg.init_params(7, norm_jitter=0.1)                      # same weights everywhere
    # rank 0 makes the 128-byte communicator id, the others receive it
    uid = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        uid = torch.from_numpy(np.random.default_rng(0).integers(0, 256, 128).astype(np.uint8))
    dist.broadcast(uid, 0)
    tok = np.random.default_rng(100 + rank).integers(0, cfg.V, 24).astype(np.int32)   # different data per rank
    ss = [0, 7, 19, 24]
    g = O.train_step(cfg, p, tok, ss)["grads"]
    gt = torch.from_numpy(g)
    for b, e in bucket_ranges(cfg):                              # bucketed, in hand-over order
        dist.all_reduce(gt[b:e], op=dist.ReduceOp.SUM)
    g_mean = gt.numpy() / world
    w, m, v = p.copy(), np.zeros_like(p), np.zeros_like(p)
    O.lib().ref_adamw(w, g_mean, m, v, p.size, 3.14e-6, 0.9, 0.999, 0.01, 1e-8, 1)
    q.put((rank, uid.numpy().tobytes(), tok, w))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_equal_one_big_batch():
    world, port = 2, free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in range(world)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0][1] == res[1][1]                                # same communicator id on both ranks
    assert np.array_equal(res[0][3], res[1][3])                  # replicas stay bit-identical
    cfg = TINY
    p0 = cfg.init_params(7, norm_jitter=0.1)
    big_tok = np.concatenate([res[0][2], res[1][2]])
    big_ss = [0, 7, 19, 24, 31, 43, 48]
    g = O.train_step(cfg, p0, big_tok, big_ss)["grads"]
    w, m, v = p0.copy(), np.zeros_like(p0), np.zeros_like(p0)
    O.lib().ref_adamw(w, g, m, v, p0.size, 3.14e-6, 0.9, 0.999, 0.01, 1e-8, 1)
    assert rel_l2(res[0][3], w) < 1e-6


def test_bucket_ranges_tile_the_gradient_arena():
    cfg = TINY
    r = sorted(bucket_ranges(cfg))
    assert r[0][0] == 0 and r[-1][1] == cfg.n_params()
    for (a, b), (c, d) in zip(r, r[1:]):
        assert b == c
