"""Model geometry of the decoder the training path runs, with the flat parameter order the
library's arenas use (embed, final_norm, then per layer q k v o gate up down in_norm post_norm;
trainable_weights_t of include/train.h:53-90 walked in that order) and the LoRA adapter order
(per layer, per projection: A [rank, in] then B [out, rank]; include/lora.h:13-56)."""
import ctypes as C
from dataclasses import dataclass

import numpy as np


class RefCfg(C.Structure):
    _fields_ = [("V", C.c_int), ("d", C.c_int), ("L", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int),
                ("hd", C.c_int), ("F", C.c_int), ("eps", C.c_float), ("theta", C.c_float), ("qk_norm", C.c_int),
                ("head_norm", C.c_int), ("untied", C.c_int)]


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
    head_norm: int = 0        # learned RMSNorm over each head of q and k before RoPE (an option of this library, not of the reference)
    untied: int = 0           # separate lm_head [V, d] instead of the embedding matrix (likewise)

    @property
    def qd(self):
        return self.Hq * self.hd

    @property
    def kvd(self):
        return self.Hkv * self.hd

    def c(self):
        return RefCfg(self.V, self.d, self.L, self.Hq, self.Hkv, self.hd, self.F, self.eps, self.theta, self.qk_norm,
                      self.head_norm, self.untied)

    def extras_tensors(self):
        """(name, shape, offset) of the parameters that are not in the reference's trainable_weights_t, in their flat order:
        per layer q_norm [hd], k_norm [hd] (head_norm), then lm_head [V, d] (untied)."""
        out, off = [], 0
        if self.head_norm:
            for l in range(self.L):
                for nm in ("q_norm", "k_norm"):
                    out.append((f"l{l}.{nm}", (self.hd,), off)); off += self.hd
        if self.untied:
            out.append(("lm_head", (self.V, self.d), off)); off += self.V * self.d
        return out, off

    def init_extras(self, seed, std=0.02, norm_jitter=0.1):
        tens, n = self.extras_tensors()
        rng = np.random.default_rng(seed)
        x = np.empty(n, np.float32)
        for name, shp, off in tens:
            k = int(np.prod(shp))
            x[off:off + k] = (1.0 + norm_jitter * rng.standard_normal(k)) if name.endswith("norm") else std * rng.standard_normal(k)
        return x

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
