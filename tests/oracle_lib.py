"""ctypes access to the CPU oracle (oracle/liboracle.so) and, where it was
built, to the reference's own code under oracle/_ref/.  Test infrastructure:
only tests, the smoke check and the bench's CPU baseline may import this."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
ORACLE_DIR = os.path.join(ROOT, "oracle")

f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


from seraph_b200.config import ModelCfg, RefCfg  # noqa: E402,F401


TINY = ModelCfg(V=257, d=64, L=2, Hq=4, Hkv=2, hd=16, F=96)
TINY_SEQS = [0, 7, 19, 24]
C1 = ModelCfg(V=8192, d=512, L=8, Hq=8, Hkv=8, hd=64, F=1408)


def _build():
    subprocess.run(["make", "-s", "-C", ORACLE_DIR, "all"], check=True)


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    path = os.path.join(ORACLE_DIR, "liboracle.so")
    if not os.path.exists(path):
        _build()
    L = C.CDLL(path)
    sz = C.c_size_t
    sig = {
        "ref_set_acc64": (None, [C.c_int]),
        "ref_embed_lookup": (None, [u32p, f32p, f32p, C.c_int, C.c_int]),
        "ref_rmsnorm": (None, [f32p, f32p, f32p, C.c_int, C.c_int, C.c_float]),
        "ref_matmul": (None, [f32p, f32p, f32p] + [C.c_int] * 6),
        "ref_rope": (None, [f32p, f32p, u32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int]),
        "ref_attention": (None, [f32p, f32p, f32p, f32p, f32p, u32p] + [C.c_int] * 5),
        "ref_attention_backward": (None, [f32p] * 7 + [u32p] + [C.c_int] * 5),
        "ref_add": (None, [f32p, f32p, f32p, sz]),
        "ref_mul": (None, [f32p, f32p, f32p, sz]),
        "ref_scale": (None, [f32p, sz, C.c_float]),
        "ref_silu": (None, [f32p, f32p, sz]),
        "ref_softmax": (None, [f32p, f32p, C.c_int, C.c_int]),
        "ref_cross_entropy_grad": (None, [f32p, u32p, f32p, f32p, u32p] + [C.c_int] * 4),
        "ref_reduce_sum": (C.c_float, [f32p, sz]),
        "ref_silu_backward": (None, [f32p, f32p, f32p, sz]),
        "ref_mul_backward": (None, [f32p] * 5 + [sz]),
        "ref_rmsnorm_backward": (None, [f32p] * 5 + [C.c_int, C.c_int, C.c_float]),
        "ref_embedding_backward": (None, [u32p, f32p, f32p, C.c_int, C.c_int]),
        "ref_qk_norm": (None, [f32p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]),
        "ref_qk_norm_backward": (None, [f32p] * 4 + [C.c_int] * 4 + [C.c_float]),
        "ref_adamw": (None, [f32p] * 4 + [sz] + [C.c_float] * 5 + [C.c_int]),
        "ref_lora_backward": (None, [f32p] * 7 + [C.c_int] * 4 + [C.c_float]),
        "ref_lora_forward_add": (None, [f32p] * 5 + [C.c_int] * 4 + [C.c_float]),
        "ref_param_count": (sz, [C.POINTER(RefCfg)]),
        "ref_lora_param_count": (sz, [C.POINTER(RefCfg), C.c_int, C.c_int]),
        "ref_train_step": (C.c_float, [C.POINTER(RefCfg), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_int, C.c_float, C.c_int, C.c_int,
                                       i32p, C.c_int, i32p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
        "ref_effective_lr": (C.c_float, [C.c_float, C.c_int, C.c_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _lib = L
    return L


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def train_step(cfg, params, tokens, seq_starts, lora=None, rank=0, alpha=0.0, mask=0, lora_exact=0,
               grads=None, want_logits=False, want_dh0=False, extras=None):
    """One oracle step.  Returns dict(loss, grads, logits?, dh0?).  grads is
    accumulated into when given (full-weight: parameter grads; LoRA: adapter grads)."""
    L = lib()
    tokens = np.ascontiguousarray(tokens, np.int32)
    ss = np.ascontiguousarray(seq_starts, np.int32)
    T, B = len(tokens), len(ss) - 1
    c = cfg.c()
    if lora is None:
        g = np.zeros_like(params) if grads is None else grads
        pg, lg = g, None
    else:
        g = np.zeros_like(lora) if grads is None else grads
        pg, lg = None, g
    logits = np.empty((T, cfg.V), np.float32) if want_logits else None
    dh0 = np.empty((T, cfg.d), np.float32) if want_dh0 else None
    xg = np.zeros_like(extras) if (extras is not None and lora is None) else None
    loss = L.ref_train_step(C.byref(c), _ptr(params), _ptr(pg), _ptr(lora), _ptr(lg), rank, alpha, mask, lora_exact,
                            tokens, T, ss, B, _ptr(logits), _ptr(dh0), _ptr(extras), _ptr(xg))
    return {"loss": float(loss), "grads": g, "logits": logits, "dh0": dh0, "extras_grads": xg}


def ref_lib(kind):
    """kind in {'cpu', 'cpu_fast', 'cuda'}: the reference's own code, or None if not built."""
    path = os.path.join(ORACLE_DIR, "_ref", f"libseraph_ref_{kind}.so")
    if not os.path.exists(path):
        return None
    L = C.CDLL(path)
    L.refshim_create.restype = C.c_void_p
    L.refshim_create.argtypes = [C.c_int] * 7 + [C.c_float, C.c_int, C.c_float, C.c_int]
    L.refshim_destroy.argtypes = [C.c_void_p]
    L.refshim_set.argtypes = [C.c_void_p, C.c_int, f32p]
    L.refshim_get.argtypes = [C.c_void_p, C.c_int, f32p]
    L.refshim_set_counters.argtypes = [C.c_void_p, C.c_int, C.c_int]
    if kind.startswith("cpu"):
        L.refshim_forward.argtypes = [C.c_void_p, i32p, C.c_int, f32p]
        L.refshim_forward.restype = C.c_int
        L.refshim_train_step.argtypes = [C.c_void_p, i32p, C.c_int]
        L.refshim_train_step.restype = C.c_float
        L.refshim_adamw.argtypes = [f32p] * 4 + [C.c_size_t] + [C.c_float] * 5 + [C.c_int]
        L.refshim_lora_backward.argtypes = [f32p] * 6 + [C.c_void_p] + [C.c_int] * 4 + [C.c_float]
        L.refshim_loss_gradient.argtypes = [f32p, f32p, C.c_int, C.c_int]
    else:
        L.refshim_cuda_init.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.refshim_cuda_init.restype = C.c_int
        L.refshim_cuda_step.argtypes = [C.c_void_p, i32p, C.c_int, i32p, C.c_int]
        L.refshim_cuda_step.restype = C.c_float
        L.refshim_cuda_download.argtypes = [C.c_void_p]
        L.refshim_cuda_ctx.argtypes = [C.c_void_p]
        L.refshim_cuda_ctx.restype = C.c_void_p
    return L


def ref_state(L, cfg, max_seq, lr=3.14e-4, accum=1):
    return L.refshim_create(cfg.V, cfg.d, cfg.L, cfg.Hq, cfg.Hkv, cfg.hd, cfg.F, cfg.theta, max_seq, lr, accum)


def rel_l2(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    nb = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / nb) if nb > 0 else float(np.linalg.norm(a))
