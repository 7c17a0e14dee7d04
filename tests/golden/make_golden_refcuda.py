"""Generates tests/golden/refcuda_tiny.{npz,json}: one packed full-weight
training step of the REFERENCE's own CUDA backend (oracle/_ref/libseraph_ref_cuda.so,
compiled from the reference checkout by oracle/Makefile) on a B200.

Run on a machine with a GPU, from the repository root:
    python tests/golden/make_golden_refcuda.py [output_dir]
The fixtures are small (tiny model: V 257, d 64, 2 layers, GQA 4/2 heads of 16,
FFN 96; three packed sequences of 7+12+5 tokens)."""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import oracle_lib as O  # noqa: E402


def main(out_dir):
    cfg, ss = O.TINY, O.TINY_SEQS
    L = O.ref_lib("cuda")
    assert L is not None, "build oracle/_ref first: make -C oracle ref"
    params = cfg.init_params(7, norm_jitter=0.1)
    tokens = np.random.default_rng(11).integers(0, cfg.V, ss[-1]).astype(np.int32)
    st = O.ref_state(L, cfg, 64, lr=3.14e-4, accum=1)
    L.refshim_set(st, 0, params)
    assert L.refshim_cuda_init(st, 0, 0) == 0
    loss = L.refshim_cuda_step(st, tokens, len(tokens), np.asarray(ss, np.int32), len(ss) - 1)
    L.refshim_cuda_download(st)
    grads, w_after = np.empty_like(params), np.empty_like(params)
    L.refshim_get(st, 1, grads)
    L.refshim_get(st, 0, w_after)
    L.refshim_destroy(st)
    os.makedirs(out_dir, exist_ok=True)
    np.savez_compressed(os.path.join(out_dir, "refcuda_tiny.npz"), params=params, tokens=tokens, grads=grads,
                        w_after=w_after, loss=np.float32(loss))
    meta = {"cfg": dict(V=cfg.V, d=cfg.d, L=cfg.L, Hq=cfg.Hq, Hkv=cfg.Hkv, hd=cfg.hd, F=cfg.F, theta=cfg.theta),
            "seq_starts": ss, "loss": float(loss), "source": "reference CUDA backend, cuda_train_step_gpu_full_batch, use_flash_attn=0"}
    json.dump(meta, open(os.path.join(out_dir, "refcuda_tiny.json"), "w"), indent=1)
    ref = O.train_step(cfg, params, tokens, ss)
    print("reference CUDA loss", loss, "oracle loss", ref["loss"], "grad rel-L2 vs oracle", O.rel_l2(grads, ref["grads"]))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
