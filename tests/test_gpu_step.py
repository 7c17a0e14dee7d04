"""Step-level parity on a B200 through the C training API: loss, every weight
gradient and the AdamW update against the CPU oracle on the same seeded
weights and tokens; LoRA adapter gradients; golden vectors produced by the
reference's own CUDA backend; properties at the benchmark's full size."""
import json
import os

import numpy as np
import pytest

import oracle_lib as O
from oracle_lib import TINY, TINY_SEQS, C1, rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-5
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture()
def ctx():
    from seraph_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg.V, n).astype(np.int32)


def check_grads(cfg, got, ref, tol=TOL):
    worst = (0.0, None)
    for name, shp, off in cfg.tensors():
        n = int(np.prod(shp))
        e = rel_l2(got[off:off + n], ref[off:off + n])
        if e > worst[0]:
            worst = (e, name)
        assert e < tol, (name, e)
    return worst


def run_full_step(ctx, cfg, params, tok, ss, lr=3.14e-4, accum=1, steps=1):
    from seraph_b200 import api
    st = api.TrainState(cfg, params, lr=lr, accum=accum)
    ctx.lib.seraph_b200_reset_model(ctx.h)       # a context keeps its resident weights otherwise
    losses = [api.step_full_batch(ctx, st, tok, ss) for _ in range(steps)]
    ctx.check()
    ctx.lib.cuda_download_gpu_gradients(ctx.h, st.h)
    ctx.lib.cuda_download_full_weights(ctx.h, st.h)
    out = dict(loss=losses, grads=st.get(1), w=st.get(0), m=st.get(2), v=st.get(3), counters=st.counters())
    st.close()
    return out


@pytest.mark.parametrize("mode", [4, 0, 3])      # FP32-accurate tensor-core modes (FP16 parts = default, TF32 parts), CUDA-core FP32 mode
def test_tiny_full_step_matches_oracle(ctx, mode):
    cfg = TINY
    ctx.set_gemm_mode(mode)
    p = cfg.init_params(7, norm_jitter=0.1)
    tok = tokens_for(cfg, TINY_SEQS[-1], 11)
    ref = O.train_step(cfg, p, tok, TINY_SEQS)
    got = run_full_step(ctx, cfg, p, tok, TINY_SEQS)
    assert abs(got["loss"][0] - ref["loss"]) < 1e-5 * abs(ref["loss"])
    check_grads(cfg, got["grads"], ref["grads"])
    # optimizer: step 1 of the reference's warm-up -> lr/100 (src/train_cuda.c:2298-2303)
    lr = O.lib().ref_effective_lr(3.14e-4, 1, 1)
    w, m, v = p.copy(), np.zeros_like(p), np.zeros_like(p)
    O.lib().ref_adamw(w, ref["grads"], m, v, p.size, lr, 0.9, 0.999, 0.01, 1e-8, 1)
    assert rel_l2(got["w"], w) < 1e-6 and rel_l2(got["m"], m) < TOL and rel_l2(got["v"], v) < 2 * TOL
    assert got["counters"] == (1, 0)


def test_tiny_step_is_bit_reproducible(ctx):
    cfg = TINY
    p = cfg.init_params(7, norm_jitter=0.1)
    tok = tokens_for(cfg, TINY_SEQS[-1], 11)
    a = run_full_step(ctx, cfg, p, tok, TINY_SEQS)
    b = run_full_step(ctx, cfg, p, tok, TINY_SEQS)
    assert a["loss"] == b["loss"] and np.array_equal(a["grads"], b["grads"]) and np.array_equal(a["w"], b["w"])


def test_gradient_accumulation_and_single_sequence_twin(ctx):
    from seraph_b200 import api
    cfg = TINY
    p = cfg.init_params(3)
    tok = tokens_for(cfg, 24, 5)
    # two micro-steps accumulate, optimizer runs once with lr/accum
    st = api.TrainState(cfg, p, accum=2)
    api.step_full_batch(ctx, st, tok, TINY_SEQS)
    assert st.counters() == (0, 1)
    api.step_full_batch(ctx, st, tok, TINY_SEQS)
    assert st.counters() == (1, 0)
    ctx.lib.cuda_download_gpu_gradients(ctx.h, st.h)
    g2 = st.get(1)
    st.close()
    one = O.train_step(cfg, p, tok, TINY_SEQS)["grads"]
    assert rel_l2(g2, 2 * one) < TOL
    # cuda_train_step_gpu_full == packed step with one sequence
    st = api.TrainState(cfg, p)
    ctx.lib.seraph_b200_reset_model(ctx.h)
    t17 = np.ascontiguousarray(tok[:17])
    loss = ctx.lib.cuda_train_step_gpu_full(st.h, t17.ctypes.data, 17, ctx.h)
    ref = O.train_step(cfg, p, t17, [0, 17])
    assert abs(loss - ref["loss"]) < 1e-5 * abs(ref["loss"])
    ctx.lib.cuda_download_gpu_gradients(ctx.h, st.h)
    check_grads(cfg, st.get(1), ref["grads"])
    # evaluation: forward + loss only, nothing changes
    ev = ctx.lib.cuda_eval_forward(st.h, t17.ctypes.data, 17, ctx.h)
    assert ev > 0 and st.counters() == (1, 0)
    st.close()


def test_error_conventions(ctx):
    from seraph_b200 import api
    cfg = TINY
    st = api.TrainState(cfg, cfg.init_params(1))
    tok = tokens_for(cfg, 3, 1)
    ss = np.array([0, 1, 2, 3], np.int32)
    # one-token sequences predict nothing -> 0.0f (src/train_cuda.c:1990-1991)
    assert ctx.lib.cuda_train_step_gpu_full_batch(st.h, tok.ctypes.data, 3, ss.ctypes.data, 3, ctx.h) == 0.0
    # NULL arguments -> -1.0f (src/train_cuda.c:1970)
    assert ctx.lib.cuda_train_step_gpu_full_batch(None, tok.ctypes.data, 3, ss.ctypes.data, 3, ctx.h) == -1.0
    assert ctx.lib.cuda_train_step_gpu_full_batch(st.h, tok.ctypes.data, 3, ss.ctypes.data, 3, None) == -1.0
    # negative token ids are clamped to 0 (src/train_cuda.c:2035)
    t = tokens_for(cfg, 24, 2)
    neg = t.copy(); neg[4] = -9
    z = t.copy(); z[4] = 0
    a = run_full_step(ctx, cfg, cfg.init_params(1), neg, TINY_SEQS)
    b = run_full_step(ctx, cfg, cfg.init_params(1), z, TINY_SEQS)
    assert a["loss"] == b["loss"] and np.array_equal(a["grads"], b["grads"])
    st.close()


@pytest.mark.parametrize("exact", [0, 1])
def test_tiny_lora_step_matches_oracle(ctx, exact):
    from seraph_b200 import api
    cfg, rank, alpha, mask = TINY, 4, 8.0, 0x7F
    p = cfg.init_params(7, norm_jitter=0.1)
    tens, n = cfg.lora_tensors(rank, mask)
    lo = (0.05 * np.random.default_rng(9).standard_normal(n)).astype(np.float32)   # B != 0 on purpose
    tok = tokens_for(cfg, 24, 11)
    ref = O.train_step(cfg, p, tok, TINY_SEQS, lora=lo, rank=rank, alpha=alpha, mask=mask, lora_exact=exact)
    st = api.TrainState(cfg, p)
    st.attach_lora(rank, alpha, mask, lo)
    assert ctx.lib.seraph_b200_set_lora_exact(ctx.h, exact) == 0
    loss = api.step_lora_batch(ctx, st, tok, TINY_SEQS)
    ctx.check()
    assert abs(loss - ref["loss"]) < 1e-5 * abs(ref["loss"])
    ctx.lib.cuda_download_lora_weights(ctx.h, st.lora_ptr())
    g = st.lora_get(1)
    for name, shp, off in tens:
        k = int(np.prod(shp))
        assert rel_l2(g[off:off + k], ref["grads"][off:off + k]) < TOL, name
    # adapters moved by AdamW, base weights untouched
    w = lo.copy(); m = np.zeros_like(lo); v = np.zeros_like(lo)
    O.lib().ref_adamw(w, ref["grads"], m, v, n, O.lib().ref_effective_lr(3.14e-4, 1, 1), 0.9, 0.999, 0.01, 1e-8, 1)
    assert rel_l2(st.lora_get(0), w) < 1e-6
    st.close()


def test_lora_default_adapters_q_and_v_only(ctx):
    """The reference's default applies LoRA to Q and V (src/lora.c:355-360)."""
    from seraph_b200 import api
    cfg, rank, alpha, mask = TINY, 4, 8.0, 0b0000101
    p = cfg.init_params(2)
    tens, n = cfg.lora_tensors(rank, mask)
    lo = (0.05 * np.random.default_rng(1).standard_normal(n)).astype(np.float32)
    tok = tokens_for(cfg, 24, 3)
    ref = O.train_step(cfg, p, tok, TINY_SEQS, lora=lo, rank=rank, alpha=alpha, mask=mask)
    st = api.TrainState(cfg, p)
    st.attach_lora(rank, alpha, mask, lo)
    api.step_lora_batch(ctx, st, tok, TINY_SEQS)
    ctx.lib.cuda_download_lora_weights(ctx.h, st.lora_ptr())
    assert rel_l2(st.lora_get(1), ref["grads"]) < TOL
    st.close()


def test_c1_step_matches_oracle(ctx):
    """Config 1 of the baseline: 33M-class Llama-style decoder, 8 x 256 tokens, all gradients; in the default GEMM mode
    (FP16 hi/lo parts) and with TF32 parts.  Bound: 1e-5 relative L2 per gradient tensor against the FP64-accumulate oracle."""
    cfg = C1
    p = cfg.init_params(1234)
    ss = list(range(0, 2049, 256))
    tok = tokens_for(cfg, 2048, 99)
    ref = O.train_step(cfg, p, tok, ss)
    for mode in (4, 0):
        ctx.set_gemm_mode(mode)
        got = run_full_step(ctx, cfg, p, tok, ss)
        assert abs(got["loss"][0] - ref["loss"]) < 1e-5 * abs(ref["loss"])
        worst = check_grads(cfg, got["grads"], ref["grads"])
        print("C1 worst gradient rel-L2, GEMM mode", mode, ":", worst)


def test_evaluate_packs_samples_and_matches_per_sample_passes(ctx):
    """cuda_evaluate: mean of the samples' mean losses and its exponential.  Packed passes (default), one pass per sample
    (the reference's loop) and the oracle's forward loss per sample agree; the stride rule for max_eval_samples and the
    max_seq_len cut are the reference's (src/train_cuda.c:2812-2846)."""
    import ctypes as C
    from seraph_b200 import api
    cfg = TINY
    p = cfg.init_params(41, norm_jitter=0.1)
    lens = [9, 2, 17, 1, 24, 5, 30, 12, 3]                # one sample too short to predict anything, one longer than max_seq_len
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    val = tokens_for(cfg, int(offs[-1]), 42)
    max_seq = 24

    def oracle_mean(sample_ids):
        tot, cnt = 0.0, 0
        for s in sample_ids:
            n = min(lens[s], max_seq)
            if n < 2:
                continue
            t = np.ascontiguousarray(val[offs[s]:offs[s] + n])
            tot += O.train_step(cfg, p, t, [0, n])["loss"]; cnt += 1
        return tot / cnt

    st = api.TrainState(cfg, p)
    ctx.lib.seraph_b200_reset_model(ctx.h)
    ppl = C.c_float(0)
    offsets = np.ascontiguousarray(offs[:-1])
    for max_eval, ids in ((0, range(len(lens))), (4, range(0, len(lens), 2))):
        ref = oracle_mean(ids)
        got = {}
        for budget in (8192, 40, 0):                      # everything in one pass / several passes / one pass per sample
            assert ctx.lib.seraph_b200_set_eval_batch_tokens(ctx.h, budget) == 0
            n0 = ctx.launches()
            got[budget] = ctx.lib.cuda_evaluate(st.h, val.ctypes.data, int(offs[-1]), offsets.ctypes.data, len(lens), max_seq, max_eval,
                                                ctx.h, C.byref(ppl))
            ctx.check()
            got[(budget, "launches")] = ctx.launches() - n0
            assert abs(got[budget] - ref) < 1e-5 * ref, (budget, got[budget], ref)
            assert abs(ppl.value - np.exp(got[budget])) < 1e-4 * ppl.value
        assert got[(8192, "launches")] < got[(0, "launches")]
    assert ctx.lib.seraph_b200_set_eval_batch_tokens(ctx.h, 8192) == 0
    assert st.counters() == (0, 0)                        # evaluation leaves the optimizer state alone
    st.close()


@pytest.mark.parametrize("which", ["tiny", "c1", "c1-many-chunks"])
def test_safetensors_export_is_byte_identical_to_the_reference_writer(ctx, which, tmp_path, monkeypatch):
    """seraph_b200_save_safetensors (BF16 conversion on the GPU, chunked copy) against the reference's own
    trainable_weights_save_to_safetensors (src/train.c:433-569, compiled from its source) fed with the weights that
    cuda_download_full_weights brought back after a training step: the two files are equal byte for byte."""
    import ctypes as C
    from seraph_b200 import api
    ref = O.ref_lib("cpu")
    if ref is None:
        pytest.skip("oracle/_ref not built (no reference checkout)")
    cfg, ss = (TINY, TINY_SEQS) if which == "tiny" else (C1, list(range(0, 2049, 256)))
    if which == "c1-many-chunks":
        monkeypatch.setenv("SERAPH_B200_CKPT_CHUNK", "1000003")       # ragged chunks through both staging buffers
    p = cfg.init_params(61, norm_jitter=0.1)
    tok = tokens_for(cfg, ss[-1], 62)
    ctx.lib.seraph_b200_reset_model(ctx.h)
    st = api.TrainState(cfg, p, lr=1e-2)
    api.step_full_batch(ctx, st, tok, ss)
    ours, theirs = str(tmp_path / "ours.safetensors"), str(tmp_path / "theirs.safetensors")
    assert ctx.lib.seraph_b200_save_safetensors(ctx.h, st.h, ours.encode()) == 0
    ctx.check()
    ctx.lib.cuda_download_full_weights(ctx.h, st.h)
    fn = ref.trainable_weights_save_to_safetensors
    fn.restype, fn.argtypes = None, [C.c_void_p, C.c_char_p]
    fn(ctx.lib.seraph_b200_state_weights(st.h), theirs.encode())
    a, b = open(ours, "rb").read(), open(theirs, "rb").read()
    assert len(a) == len(b) and a == b
    hlen = int.from_bytes(a[:8], "little")
    assert len(a) == 8 + hlen + 2 * st.n and b"model.norm.weight" in a[8:8 + hlen]
    assert not np.array_equal(st.get(0), p)               # the step did move the weights that were exported
    if which == "tiny":
        # the whole checkpoint: same file plus "<path>.state" = epoch, step, loss, optimizer step as save_checkpoint writes them
        ck = str(tmp_path / "ckpt.safetensors")
        assert ctx.lib.seraph_b200_save_checkpoint(ctx.h, st.h, ck.encode()) == 0
        assert open(ck, "rb").read() == b
        raw = open(ck + ".state", "rb").read()
        assert len(raw) == 16 and int.from_bytes(raw[12:16], "little") == st.counters()[0] == 1
    st.close()


@pytest.mark.parametrize("chunk", [None, "300001"])
def test_safetensors_load_widens_bf16_on_the_device(ctx, chunk, tmp_path, monkeypatch):
    """seraph_b200_load_safetensors: a saved file read back into a context that holds other weights (and into one that holds
    none yet) gives exactly the BF16-truncated weights (bf16_to_f32 of src/train.c:255-260), the reference's own loader
    agrees value for value, and exporting again reproduces the file."""
    import ctypes as C
    from seraph_b200 import api
    if chunk:
        monkeypatch.setenv("SERAPH_B200_CKPT_CHUNK", chunk)
    cfg, ss = C1, list(range(0, 2049, 256))
    p = cfg.init_params(71, norm_jitter=0.1)
    ctx.lib.seraph_b200_reset_model(ctx.h)
    st = api.TrainState(cfg, p)
    api.step_full_batch(ctx, st, tokens_for(cfg, ss[-1], 72), ss)           # make the model resident
    path = str(tmp_path / "w.safetensors")
    assert ctx.lib.seraph_b200_save_safetensors(ctx.h, st.h, path.encode()) == 0
    ctx.lib.cuda_download_full_weights(ctx.h, st.h)
    want = (st.get(0).view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
    st.close()
    for resident in (True, False):
        ctx.lib.seraph_b200_reset_model(ctx.h)
        st2 = api.TrainState(cfg, cfg.init_params(73))                       # other weights
        if resident:
            api.step_full_batch(ctx, st2, tokens_for(cfg, ss[-1], 74), ss)
        assert ctx.lib.seraph_b200_load_safetensors(ctx.h, st2.h, path.encode()) == 0
        ctx.check()
        ctx.lib.cuda_download_full_weights(ctx.h, st2.h)
        assert np.array_equal(st2.get(0).view(np.uint32), want.view(np.uint32))
        again = str(tmp_path / "again.safetensors")
        assert ctx.lib.seraph_b200_save_safetensors(ctx.h, st2.h, again.encode()) == 0
        assert open(again, "rb").read() == open(path, "rb").read()
        ref = O.ref_lib("cpu")
        if ref is not None and resident:
            st3 = api.TrainState(cfg, cfg.init_params(75))
            fn = ref.trainable_weights_load_from_safetensors
            fn.restype, fn.argtypes = C.c_int, [C.c_void_p, C.c_char_p]
            assert fn(ctx.lib.seraph_b200_state_weights(st3.h), path.encode()) == 0
            assert np.array_equal(st3.get(0).view(np.uint32), want.view(np.uint32))
            st3.close()
        st2.close()


def test_step_with_qk_norm_matches_oracle(ctx):
    """config->use_qk_norm = 1: q and k are normalised over the whole token row after RoPE (the reference's qk_norm shader)
    and the backward pass differentiates through it (the reference does not).  Tiny shape (row kernels) and a 128-wide-head
    shape (warp-per-row kernels, fused attention)."""
    import dataclasses
    for base, ss, seed in ((TINY, TINY_SEQS, 51), (O.ModelCfg(V=1024, d=512, L=2, Hq=4, Hkv=2, hd=128, F=1024, theta=1e4), [0, 300, 512, 645], 52)):
        cfg = dataclasses.replace(base, qk_norm=1)
        p = cfg.init_params(seed, norm_jitter=0.1)
        tok = tokens_for(cfg, ss[-1], seed + 1)
        ref = O.train_step(cfg, p, tok, ss)
        got = run_full_step(ctx, cfg, p, tok, ss)
        assert abs(got["loss"][0] - ref["loss"]) < 1e-5 * abs(ref["loss"])
        print("qk_norm step, worst gradient rel-L2:", check_grads(cfg, got["grads"], ref["grads"]))
        off = run_full_step(ctx, base, p, tok, ss)
        assert abs(off["loss"][0] - got["loss"][0]) > 1e-4


def test_head128_model_step_matches_oracle(ctx):
    """A model with 128-wide heads (grouped: 4 query / 2 K-V heads) on ragged sequences: the step runs the fused attention
    kernels (forward in one kernel, backward scores in one kernel) and every gradient meets the bound."""
    cfg = O.ModelCfg(V=1024, d=512, L=2, Hq=4, Hkv=2, hd=128, F=1024, theta=1e4)
    p = cfg.init_params(21, norm_jitter=0.1)
    ss = [0, 300, 512, 645]
    tok = tokens_for(cfg, ss[-1], 22)
    ref = O.train_step(cfg, p, tok, ss)
    for flash in (1, 0):
        ctx.set_attn_flash(flash)
        got = run_full_step(ctx, cfg, p, tok, ss)
        assert abs(got["loss"][0] - ref["loss"]) < 1e-5 * abs(ref["loss"])
        worst = check_grads(cfg, got["grads"], ref["grads"])
        print("128-wide heads, fused attention", flash, "worst gradient rel-L2:", worst)
    ctx.set_attn_flash(1)


def test_c1_lora_step_on_tensor_cores_matches_oracle(ctx):
    """LoRA step at configuration-1 size (rank 16 on all seven projections, full chain rule): the frozen base runs through
    the tensor-core products with shared operand parts, the adapters through the small-rank path."""
    from seraph_b200 import api
    cfg, rank, alpha, mask = C1, 16, 32.0, 0x7F
    p = cfg.init_params(31)
    tens, n = cfg.lora_tensors(rank, mask)
    lo = (0.02 * np.random.default_rng(32).standard_normal(n)).astype(np.float32)
    ss = list(range(0, 1025, 256))
    tok = tokens_for(cfg, 1024, 33)
    ref = O.train_step(cfg, p, tok, ss, lora=lo, rank=rank, alpha=alpha, mask=mask, lora_exact=1)
    outs = []
    for keep in (1, 0, 1):
        ctx.set_parts_cache(keep)
        ctx.lib.seraph_b200_reset_model(ctx.h)
        st = api.TrainState(cfg, p)
        st.attach_lora(rank, alpha, mask, lo)
        assert ctx.lib.seraph_b200_set_lora_exact(ctx.h, 1) == 0
        loss = api.step_lora_batch(ctx, st, tok, ss)
        ctx.check()
        ctx.lib.cuda_download_lora_weights(ctx.h, st.lora_ptr())
        g = st.lora_get(1)
        outs.append((loss, g))
        st.close()
    ctx.set_parts_cache(1)
    assert ctx.lib.seraph_b200_set_lora_exact(ctx.h, 0) == 0
    loss, g = outs[0]
    assert abs(loss - ref["loss"]) < 1e-5 * abs(ref["loss"])
    for name, shp, off in tens:
        k = int(np.prod(shp))
        assert rel_l2(g[off:off + k], ref["grads"][off:off + k]) < TOL, (name, rel_l2(g[off:off + k], ref["grads"][off:off + k]))
    assert outs[0][0] == outs[1][0] and np.array_equal(outs[0][1], outs[1][1])


def test_operand_parts_kept_within_a_step_change_nothing(ctx):
    """The FP16 parts of weights and saved activations are made once per call and shared by the call's products, and the SwiGLU
    kernels write their outputs straight into that arena (scaled by a bound instead of the exact maximum, so those operands
    round differently in their last bits).  Three optimizer steps (the weights move between them), then a step on fewer tokens
    and one on the full batch again: losses, gradients and weights agree with the run in which every product prepares its own
    operands to a few 1e-6 (both inside the parity bound), and the run with the arena repeats bit for bit."""
    from seraph_b200 import api
    cfg = C1
    p = cfg.init_params(77)
    ss = list(range(0, 2049, 256))
    tok = tokens_for(cfg, 2048, 5)
    runs = []
    for keep in (1, 0, 1):
        ctx.set_parts_cache(keep)
        ctx.lib.seraph_b200_reset_model(ctx.h)
        st = api.TrainState(cfg, p, lr=1e-2)
        losses = [api.step_full_batch(ctx, st, tok, ss) for _ in range(3)]
        losses.append(api.step_full_batch(ctx, st, np.ascontiguousarray(tok[:1024]), ss[:5]))
        losses.append(api.step_full_batch(ctx, st, tok, ss))
        ctx.check()
        ctx.lib.cuda_download_gpu_gradients(ctx.h, st.h)
        ctx.lib.cuda_download_full_weights(ctx.h, st.h)
        runs.append((losses, st.get(1), st.get(0)))
        st.close()
    ctx.set_parts_cache(1)
    assert np.allclose(runs[0][0], runs[1][0], rtol=2e-6, atol=0), (runs[0][0], runs[1][0])
    eg, ew = O.rel_l2(runs[0][1], runs[1][1]), O.rel_l2(runs[0][2], runs[1][2])
    print(f"arena on vs off: gradients rel-L2 {eg:.2e}, weights {ew:.2e}")
    # two roundings of the same sums: each is within 2.5e-6 of the oracle, so they may differ from each other by their root sum
    assert eg < 6e-6 and ew < 2e-6, (eg, ew)
    assert runs[0][0] == runs[2][0] and np.array_equal(runs[0][1], runs[2][1]) and np.array_equal(runs[0][2], runs[2][2])
    assert runs[0][0][0] != runs[0][0][2]          # the weights did move


def test_golden_reference_cuda_vectors(ctx):
    """Gradients written by the reference's own CUDA backend on a B200
    (tests/golden/make_golden_refcuda.py).  Its float atomics make it
    non-deterministic at the 1e-6 level, so the comparison is by tolerance."""
    meta_path = os.path.join(GOLD, "refcuda_tiny.json")
    if not os.path.exists(meta_path):
        pytest.skip("golden vectors of the reference CUDA backend not generated yet")
    meta = json.load(open(meta_path))
    z = np.load(os.path.join(GOLD, "refcuda_tiny.npz"))
    cfg = O.ModelCfg(**meta["cfg"])
    got = run_full_step(ctx, cfg, z["params"], z["tokens"], meta["seq_starts"])
    assert abs(got["loss"][0] - float(z["loss"])) < 2e-5 * abs(float(z["loss"]))
    check_grads(cfg, got["grads"], z["grads"], tol=5e-5)
    assert rel_l2(got["w"], z["w_after"]) < 1e-6


def test_full_size_properties_qwen_shaped(ctx):
    """Benchmark-size shapes (hidden 2048, 16/8 heads of 128, FFN 6144, vocab 151936) on two layers:
    properties that need no oracle run - bit reproducibility, linearity of gradient accumulation,
    embedding rows touched exactly where tokens point, loss near ln(V) at N(0, 0.02) init."""
    from seraph_b200 import api
    cfg = O.ModelCfg(V=151936, d=2048, L=2, Hq=16, Hkv=8, hd=128, F=6144, theta=1e6)
    p = cfg.init_params(5)
    T, B = 4096, 2
    ss = [0, 2048, 4096]
    tok = tokens_for(cfg, T, 6)
    a = run_full_step(ctx, cfg, p, tok, ss)
    b = run_full_step(ctx, cfg, p, tok, ss)
    assert a["loss"] == b["loss"] and np.array_equal(a["grads"], b["grads"])
    assert abs(a["loss"][0] - np.log(cfg.V)) < 0.5
    st = api.TrainState(cfg, p, accum=2)
    ctx.lib.seraph_b200_reset_model(ctx.h)
    api.step_full_batch(ctx, st, tok, ss)
    api.step_full_batch(ctx, st, tok, ss)
    ctx.lib.cuda_download_gpu_gradients(ctx.h, st.h)
    g2 = st.get(1)
    st.close()
    assert rel_l2(g2, 2 * a["grads"]) < 1e-6
    ge = a["grads"][:cfg.V * cfg.d].reshape(cfg.V, cfg.d)
    assert np.isfinite(a["grads"]).all() and np.abs(ge[np.unique(tok)]).sum() > 0


def test_c1_against_reference_cuda_backend_on_this_gpu(ctx):
    """Runs the reference's own CUDA backend (compiled from its sources into
    oracle/_ref, hidden size 512 is within its launch limits) and this library
    on the same weights and tokens, on the same GPU, and compares all gradients
    and the updated weights.  Skipped where oracle/_ref was not built."""
    L = O.ref_lib("cuda")
    if L is None:
        pytest.skip("oracle/_ref/libseraph_ref_cuda.so not built")
    cfg = C1
    p = cfg.init_params(4321)
    ss = list(range(0, 2049, 256))
    tok = tokens_for(cfg, 2048, 17)
    st = O.ref_state(L, cfg, 2048)
    L.refshim_set(st, 0, p)
    assert L.refshim_cuda_init(st, 0, 0) == 0
    ref_loss = L.refshim_cuda_step(st, tok, 2048, np.asarray(ss, np.int32), 8)
    L.refshim_cuda_download(st)
    rg, rw = np.empty_like(p), np.empty_like(p)
    L.refshim_get(st, 1, rg)
    L.refshim_get(st, 0, rw)
    L.refshim_destroy(st)
    got = run_full_step(ctx, cfg, p, tok, ss)
    assert abs(got["loss"][0] - ref_loss) < 2e-5 * abs(ref_loss)
    worst = check_grads(cfg, got["grads"], rg, tol=5e-5)
    print("C1 vs reference CUDA, worst gradient rel-L2:", worst)
    assert rel_l2(got["w"], rw) < 1e-6
