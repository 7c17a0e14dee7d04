"""Python mirror of the C training API, over ctypes.

The product is libseraph_b200.so; this module only loads it and gives the test
and benchmark code the same calls a C host makes (`cuda_train_*`,
`cuda_train_step_gpu_*`, `seraph_b200_*`, `seraph_dp_*`) on numpy arrays.
There is no fallback of any kind: if the library is missing or no B200 is
present, loading or `Context()` raises."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libseraph_b200.so")

STATUS = {0: "ok", 1: "bad argument", 2: "CUDA error", 3: "out of memory", 4: "token id outside vocabulary",
          5: "bounded wait ran out", 6: "NCCL error", 7: "size beyond capacity"}
GEMM_FP32X3, GEMM_TF32, GEMM_BF16, GEMM_SIMT, GEMM_FP16X3 = 0, 1, 2, 3, 4      # 4 is the library's default


class CudaBuffer(C.Structure):
    _fields_ = [("data", C.c_void_p), ("size", C.c_size_t)]


_lib = None


def load():
    """Load the shared library (building it is `python -m seraph_b200.build`)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m seraph_b200.build` "
                           "(there is no fallback implementation)")
    L = C.CDLL(LIB_PATH)
    vp, i, f, sz, u32 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_uint32
    B = C.POINTER(CudaBuffer)
    sig = {
        "cuda_train_init": (vp, [i]), "cuda_train_free": (None, [vp]), "cuda_train_sync": (None, [vp]),
        "cuda_train_get_gpu_info": (None, [vp, C.c_char_p, i, C.POINTER(f)]),
        "cuda_train_buffer_create": (B, [vp, sz]), "cuda_train_buffer_free": (None, [vp, B]),
        "cuda_train_buffer_upload": (None, [vp, B, vp, sz]), "cuda_train_buffer_upload_u32": (None, [vp, B, vp, sz]),
        "cuda_train_buffer_download": (None, [vp, B, vp, sz]), "cuda_train_buffer_download_bytes": (None, [vp, B, vp, sz]),
        "cuda_train_fill_buffer": (None, [vp, B, u32, sz]), "cuda_train_fill_buffer_range": (None, [vp, B, sz, u32, sz]),
        "cuda_train_copy_buffer": (None, [vp, B, B, sz]),
        "cuda_train_matmul": (None, [vp, B, B, B, i, i, i]),
        "cuda_train_matmul_transpose": (None, [vp, B, B, B, i, i, i, i, i, i]),
        "cuda_train_silu": (None, [vp, B, B, sz]), "cuda_train_rmsnorm": (None, [vp, B, B, B, i, i, f]),
        "cuda_train_softmax": (None, [vp, B, B, i, i]), "cuda_train_rope": (None, [vp, B, B, i, i, i, f]),
        "cuda_train_add": (None, [vp, B, B, B, sz]), "cuda_train_mul": (None, [vp, B, B, B, sz]),
        "cuda_train_scale": (None, [vp, B, sz, f]),
        "cuda_train_batch_attention": (None, [vp, B, B, B, B, B, i, i, i, i]),
        "cuda_train_batch_attention_packed": (None, [vp, B, B, B, B, B, B, i, i, i, i, i, i]),
        "cuda_train_embed_lookup": (None, [vp, B, B, B, i, i, i]),
        "cuda_train_rope_packed": (None, [vp, B, B, B, i, i, i, i, f]),
        "cuda_train_cross_entropy_grad": (None, [vp, B, B, B, B, i, i]),
        "cuda_train_cross_entropy_grad_packed": (None, [vp, B, B, B, B, B, i, i, i, i]),
        "cuda_train_reduce_sum": (None, [vp, B, B, sz]), "cuda_train_silu_backward": (None, [vp, B, B, B, sz]),
        "cuda_train_elementwise_mul_backward": (None, [vp, B, B, B, B, B, sz]),
        "cuda_train_rmsnorm_backward_batch": (None, [vp, B, B, B, B, B, i, i, f]),
        "cuda_train_rope_backward": (None, [vp, B, B, i, i, i, f]),
        "cuda_train_rope_backward_packed": (None, [vp, B, B, B, i, i, i, i, f]),
        "cuda_train_batch_attention_backward": (None, [vp] + [B] * 9 + [i] * 4),
        "cuda_train_batch_attention_backward_packed": (None, [vp] + [B] * 10 + [i] * 6),
        "cuda_train_embedding_backward": (None, [vp, B, B, B, i, i, i]),
        "cuda_train_adamw_update": (None, [vp, B, B, B, B, f, f, f, f, f, i, sz, C.c_char_p, i, i]),
        "cuda_train_nan_check": (None, [vp, B, sz, B, u32]), "cuda_train_set_profiler": (None, [vp, vp]),
        "cuda_train_lora_backward": (None, [vp] + [B] * 7 + [i] * 4 + [f]),
        "cuda_train_zero_lora_grads": (None, [vp]), "cuda_download_lora_weights": (None, [vp, vp]),
        "cuda_train_step_gpu_full": (f, [vp, vp, i, vp]), "cuda_train_step_gpu_lora": (f, [vp, vp, i, vp]),
        "cuda_train_step_gpu_full_batch": (f, [vp, vp, i, vp, i, vp]),
        "cuda_train_step_gpu_lora_batch": (f, [vp, vp, i, vp, i, vp]),
        "cuda_download_full_weights": (None, [vp, vp]), "cuda_download_gpu_gradients": (None, [vp, vp]),
        "cuda_eval_forward": (f, [vp, vp, i, vp]),
        "cuda_evaluate": (f, [vp, vp, i, vp, i, i, i, vp, C.POINTER(f)]),
        "cuda_profiler_create": (vp, []), "cuda_profiler_destroy": (None, [vp]), "cuda_profiler_enable": (None, [vp]),
        "cuda_profiler_disable": (None, [vp]), "cuda_profiler_reset": (None, [vp]),
        "cuda_profiler_begin_op": (i, [vp, C.c_char_p, vp]), "cuda_profiler_end_op": (None, [vp, i, vp]),
        "cuda_profiler_set_launch": (None, [vp, i, i, i, i, i, i, i, sz]), "cuda_profiler_set_flops": (None, [vp, i, sz]),
        "cuda_profiler_set_bytes": (None, [vp, i, sz]), "cuda_profiler_sync_and_analyze": (None, [vp, vp]),
        "cuda_profiler_print": (None, [vp]), "cuda_profiler_print_top": (None, [vp, i]), "cuda_profiler_set_log": (None, [vp, vp]),
        "seraph_b200_last_status": (i, [vp]), "seraph_b200_set_gemm_mode": (i, [vp, i]), "seraph_b200_set_gemm_pair": (i, [vp, i]), "seraph_b200_set_gemm_tail_split": (i, [vp, i]), "seraph_b200_set_parts_cache": (i, [vp, i]), "seraph_b200_set_attn_fused": (i, [vp, i]), "seraph_b200_set_attn_flash": (i, [vp, i]), "seraph_b200_qk_norm": (None, [vp, vp, vp, i, i, i, i, f]), "seraph_b200_qk_norm_backward": (None, [vp, vp, vp, vp, vp, i, i, i, i, f]), "seraph_b200_set_eval_batch_tokens": (i, [vp, i]),
        "seraph_b200_set_lora_exact": (i, [vp, i]), "seraph_b200_set_grad_clip": (i, [vp, f]),
        "seraph_b200_launch_count": (C.c_ulonglong, [vp, i]),
        "seraph_b200_state_attach_model_file": (i, [vp, C.c_char_p]),
        "seraph_b200_set_model_extras": (i, [vp, i, i, vp, sz]), "seraph_b200_get_model_extras": (i, [vp, i, vp, sz]),
        "seraph_b200_lora_save": (i, [vp, vp, C.c_char_p, i, i]), "seraph_b200_lora_load": (i, [vp, vp, C.c_char_p]),
        "seraph_b200_selftest_bounded_wait": (i, [vp, C.c_longlong, vp]),
        "seraph_b200_nan_flags": (i, [vp, vp, i]), "seraph_b200_profiler_totals": (i, [vp, vp]),
        "seraph_b200_state_set_debug_nan": (None, [vp, i]), "seraph_b200_state_nan_detected": (i, [vp]),
        "seraph_b200_embedding_segments": (i, [vp, i, i, vp, vp, vp]),
        "seraph_b200_matmul_amax": (i, [vp, vp, vp, vp, i, i, i, i, i, vp]),
        "seraph_b200_swiglu": (None, [vp, B, B, B, sz]), "seraph_b200_swiglu_backward": (None, [vp, B, B, B, B, B, sz]),
        "seraph_b200_timer_start": (None, [vp]), "seraph_b200_timer_stop": (f, [vp]),
        "seraph_b200_download_logits": (i, [vp, vp, i]), "seraph_b200_reset_model": (i, [vp]),
        "seraph_b200_step_full_resident": (i, [vp, vp]), "seraph_b200_step_resident": (i, [vp, vp, i]), "seraph_b200_last_loss": (f, [vp]),
        "seraph_b200_timing_enable": (i, [vp, i]), "seraph_b200_timing_classes": (i, []),
        "seraph_b200_timing_class_name": (C.c_char_p, [i]), "seraph_b200_timing_read": (i, [vp, vp]),
        "seraph_b200_state_create_lean": (vp, [i] * 7 + [f, f, i]),
        "seraph_b200_rmsnorm_backward_static": (i, [vp, vp, vp, vp, vp, i, i, f, vp]),
        "seraph_dp_get_unique_id": (i, [vp]), "seraph_dp_init": (i, [vp, i, i, vp]), "seraph_dp_finalize": (None, [vp]),
        "seraph_dp_wait": (i, [vp, i]), "seraph_dp_world": (i, [vp]),
        "seraph_dp_env": (i, [vp, vp]), "seraph_dp_init_from_env": (i, [vp]), "seraph_dp_shard_samples": (i, [vp, vp, vp, i, i]),
        "seraph_dp_all_min": (i, [vp, i]),
        "seraph_b200_state_create": (vp, [i] * 7 + [f, f, i]), "seraph_b200_state_free": (None, [vp]),
        "seraph_b200_state_param_count": (sz, [vp]), "seraph_b200_state_set": (None, [vp, i, vp]),
        "seraph_b200_state_get": (None, [vp, i, vp]), "seraph_b200_state_set_counters": (None, [vp, i, i]),
        "seraph_b200_state_get_counters": (None, [vp, C.POINTER(i), C.POINTER(i)]),
        "seraph_b200_state_set_lr": (None, [vp, f, i]), "seraph_b200_state_set_qk_norm": (None, [vp, i]), "seraph_b200_state_weights": (vp, [vp]), "seraph_b200_save_safetensors": (i, [vp, vp, C.c_char_p]), "seraph_b200_save_checkpoint": (i, [vp, vp, C.c_char_p]), "seraph_b200_load_safetensors": (i, [vp, vp, C.c_char_p]), "seraph_b200_state_lora_count": (sz, [vp, i, i]),
        "seraph_b200_state_attach_lora": (i, [vp, i, f, i, vp]), "seraph_b200_state_lora_get": (None, [vp, i, vp]),
    }
    missing = []
    for name, (res, args) in sig.items():
        try:
            fn = getattr(L, name)
        except AttributeError:
            missing.append(name)
            continue
        fn.restype, fn.argtypes = res, args
    if missing:
        raise RuntimeError("libseraph_b200.so lacks symbols: " + ", ".join(missing))
    L._sig_names = sorted(sig)
    _lib = L
    return L


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


class Buffer:
    """A device buffer created through cuda_train_buffer_create."""

    def __init__(self, ctx, nbytes):
        self.ctx, self.nbytes = ctx, int(nbytes)
        self.b = ctx.lib.cuda_train_buffer_create(ctx.h, self.nbytes)
        if not self.b:
            raise MemoryError(f"cuda_train_buffer_create({nbytes}) failed")

    def free(self):
        if self.b:
            self.ctx.lib.cuda_train_buffer_free(self.ctx.h, self.b)
            self.b = None

    def numpy(self, dtype=np.float32, shape=None):
        n = self.nbytes // np.dtype(dtype).itemsize
        out = np.empty(n, dtype)
        self.ctx.lib.cuda_train_buffer_download_bytes(self.ctx.h, self.b, _p(out), out.nbytes)
        return out.reshape(shape) if shape is not None else out


class Context:
    """cuda_train_init / cuda_train_free plus thin per-op helpers on numpy arrays."""

    def __init__(self, device=0):
        self.lib = load()
        self.h = self.lib.cuda_train_init(device)
        if not self.h:
            raise RuntimeError("cuda_train_init failed: a B200 (sm_100) device is required; there is no CPU path")
        self._bufs = []

    def close(self):
        if self.h:
            for b in self._bufs:
                b.free()
            self._bufs = []
            self.lib.cuda_train_free(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # buffers ---------------------------------------------------------------
    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        b = Buffer(self, max(arr.nbytes, 4))
        if arr.dtype == np.float32:
            self.lib.cuda_train_buffer_upload(self.h, b.b, _p(arr), arr.size)
        elif arr.dtype in (np.uint32, np.int32):
            self.lib.cuda_train_buffer_upload_u32(self.h, b.b, _p(arr), arr.size)
        else:
            raise TypeError(arr.dtype)
        self.lib.cuda_train_sync(self.h)      # the host array may go away
        self._bufs.append(b)
        return b

    def empty(self, n_floats):
        b = Buffer(self, max(int(n_floats) * 4, 4))
        self._bufs.append(b)
        return b

    def zeros(self, n_floats):
        b = self.empty(n_floats)
        self.lib.cuda_train_fill_buffer(self.h, b.b, 0, b.nbytes)
        return b

    def release(self, *bufs):
        for b in bufs:
            b.free()
            if b in self._bufs:
                self._bufs.remove(b)

    def sync(self):
        self.lib.cuda_train_sync(self.h)

    def status(self):
        return self.lib.seraph_b200_last_status(self.h)

    def check(self):
        s = self.status()
        if s != 0:
            raise RuntimeError(f"seraph_b200 status {s}: {STATUS.get(s, '?')}")

    def set_gemm_mode(self, mode):
        assert self.lib.seraph_b200_set_gemm_mode(self.h, mode) == 0

    def set_attn_flash(self, on):
        assert self.lib.seraph_b200_set_attn_flash(self.h, int(on)) == 0

    def set_attn_fused(self, on):
        assert self.lib.seraph_b200_set_attn_fused(self.h, 1 if on else 0) == 0

    def set_parts_cache(self, on):
        assert self.lib.seraph_b200_set_parts_cache(self.h, 1 if on else 0) == 0

    def set_gemm_tail_split(self, on):
        assert self.lib.seraph_b200_set_gemm_tail_split(self.h, 1 if on else 0) == 0

    def set_gemm_pair(self, on):
        assert self.lib.seraph_b200_set_gemm_pair(self.h, 1 if on else 0) == 0

    def launches(self, reset=False):
        return int(self.lib.seraph_b200_launch_count(self.h, 1 if reset else 0))

    def timer_start(self):
        self.lib.seraph_b200_timer_start(self.h)

    def timer_stop(self):
        return float(self.lib.seraph_b200_timer_stop(self.h))


class TrainState:
    """A train_state_t built in memory (seraph_b200_state_*), flat-array access."""

    def __init__(self, cfg, params, lr=3.14e-4, accum=1, lean=False):
        self.lib = load()
        self.cfg = cfg
        create = self.lib.seraph_b200_state_create_lean if lean else self.lib.seraph_b200_state_create
        self.h = create(cfg.V, cfg.d, cfg.L, cfg.Hq, cfg.Hkv, cfg.hd, cfg.F, cfg.theta, lr, accum)
        if not self.h:
            raise MemoryError("seraph_b200_state_create failed")
        self.n = int(self.lib.seraph_b200_state_param_count(self.h))
        if params is not None:
            params = np.ascontiguousarray(params, np.float32)
            assert params.size == self.n, (params.size, self.n)
            self.lib.seraph_b200_state_set(self.h, 0, _p(params))
        self.n_lora = 0
        if getattr(cfg, "qk_norm", 0):
            self.lib.seraph_b200_state_set_qk_norm(self.h, 1)

    def close(self):
        if self.h:
            self.lib.seraph_b200_state_free(self.h)
            self.h = None

    def get(self, which):
        out = np.empty(self.n, np.float32)
        self.lib.seraph_b200_state_get(self.h, which, _p(out))
        return out

    def set(self, which, flat):
        flat = np.ascontiguousarray(flat, np.float32)
        assert flat.size == self.n
        self.lib.seraph_b200_state_set(self.h, which, _p(flat))

    def counters(self):
        a, b = C.c_int(), C.c_int()
        self.lib.seraph_b200_state_get_counters(self.h, C.byref(a), C.byref(b))
        return a.value, b.value

    def set_counters(self, optimizer_step, accumulation_counter):
        self.lib.seraph_b200_state_set_counters(self.h, optimizer_step, accumulation_counter)

    def attach_lora(self, rank, alpha, mask, flat):
        self.n_lora = int(self.lib.seraph_b200_state_lora_count(self.h, rank, mask))
        flat = np.ascontiguousarray(flat, np.float32)
        assert flat.size == self.n_lora
        assert self.lib.seraph_b200_state_attach_lora(self.h, rank, alpha, mask, _p(flat)) == 0

    def lora_get(self, which):
        out = np.empty(self.n_lora, np.float32)
        self.lib.seraph_b200_state_lora_get(self.h, which, _p(out))
        return out

    def lora_ptr(self):
        """lora_model_t* of the state (for cuda_download_lora_weights)."""
        # train_state_t.lora sits after four pointers and an int (padded): offset 40
        return C.c_void_p.from_address(self.h + 40).value


def step_full_batch(ctx, st, tokens, seq_starts):
    tokens = np.ascontiguousarray(tokens, np.int32)
    ss = np.ascontiguousarray(seq_starts, np.int32)
    return float(ctx.lib.cuda_train_step_gpu_full_batch(st.h, _p(tokens), len(tokens), _p(ss), len(ss) - 1, ctx.h))


def step_lora_batch(ctx, st, tokens, seq_starts):
    tokens = np.ascontiguousarray(tokens, np.int32)
    ss = np.ascontiguousarray(seq_starts, np.int32)
    return float(ctx.lib.cuda_train_step_gpu_lora_batch(st.h, _p(tokens), len(tokens), _p(ss), len(ss) - 1, ctx.h))
