"""ctypes access to the CPU oracle (oracle/liboracle.so) and, where it was
built, to the reference's own code under oracle/_ref/.  Test infrastructure:
only tests, the smoke check and the bench's CPU baseline may import this."""
import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


class RefCfg(C.Structure):
    _fields_ = [("V", C.c_int), ("d", C.c_int), ("L", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int),
                ("hd", C.c_int), ("F", C.c_int), ("eps", C.c_float), ("theta", C.c_float), ("qk_norm", C.c_int)]


@dataclass
class ModelCfg:
    V: int
    d: int
    L: int
    Hq: int
    Hkv: int
    hd: int
    F: int
    theta: float = 10000.0
    eps: float = 1e-5
    qk_norm: int = 0          # whole-row normalisation of q and k after RoPE (config->use_qk_norm)

    @property
    def qd(self):
        return self.Hq * self.hd

    @property
    def kvd(self):
        return self.Hkv * self.hd

    def c(self):
        return RefCfg(self.V, self.d, self.L, self.Hq, self.Hkv, self.hd, self.F, self.eps, self.theta, self.qk_norm)

    def layer_shapes(self):
        d, F, qd, kvd = self.d, self.F, self.qd, self.kvd
        return [("q", (qd, d)), ("k", (kvd, d)), ("v", (kvd, d)), ("o", (d, qd)), ("gate", (F, d)),
                ("up", (F, d)), ("down", (d, F)), ("in_norm", (d,)), ("post_norm", (d,))]

    def tensors(self):
        """(name, shape, offset) in the flat parameter order."""
        out, off = [], 0
        for name, shp in [("embed", (self.V, self.d)), ("final_norm", (self.d,))]:
            out.append((name, shp, off))
            off += int(np.prod(shp))
        for l in range(self.L):
            for name, shp in self.layer_shapes():
                out.append((f"l{l}.{name}", shp, off))
                off += int(np.prod(shp))
        return out

    def n_params(self):
        t = self.tensors()[-1]
        return t[2] + int(np.prod(t[1]))

    def init_params(self, seed, std=0.02, norm_jitter=0.0):
        """N(0, std) weights, norm scales 1.0 (+ optional jitter so that scale
        gradients and the scale's part in dx are exercised)."""
        rng = np.random.default_rng(seed)
        p = np.empty(self.n_params(), np.float32)
        for name, shp, off in self.tensors():
            n = int(np.prod(shp))
            if name.endswith("norm"):
                p[off:off + n] = 1.0 + norm_jitter * rng.standard_normal(n).astype(np.float32)
            else:
                p[off:off + n] = (std * rng.standard_normal(n)).astype(np.float32)
        return p

    LORA_NAMES = ["q", "k", "v", "o", "gate", "up", "down"]

    def lora_dims(self, a):
        d, F, qd, kvd = self.d, self.F, self.qd, self.kvd
        return [(d, qd), (d, kvd), (d, kvd), (qd, d), (d, F), (d, F), (F, d)][a]

    def lora_tensors(self, rank, mask):
        out, off = [], 0
        for l in range(self.L):
            for a in range(7):
                if mask & (1 << a):
                    i, o = self.lora_dims(a)
                    out.append((f"l{l}.{self.LORA_NAMES[a]}.A", (rank, i), off)); off += rank * i
                    out.append((f"l{l}.{self.LORA_NAMES[a]}.B", (o, rank), off)); off += o * rank
        return out, off


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
                                       i32p, C.c_int, i32p, C.c_int, C.c_void_p, C.c_void_p]),
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
               grads=None, want_logits=False, want_dh0=False):
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
    loss = L.ref_train_step(C.byref(c), _ptr(params), _ptr(pg), _ptr(lora), _ptr(lg), rank, alpha, mask, lora_exact,
                            tokens, T, ss, B, _ptr(logits), _ptr(dh0))
    return {"loss": float(loss), "grads": g, "logits": logits, "dh0": dh0}


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
