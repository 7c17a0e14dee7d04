"""Parity at the shapes the benchmark configurations name, on a B200.

The C loops of the CPU oracle do not finish at these sizes, so the checker is the float64 torch restatement of the same
decoder (tests/torch_model.py) run on the GPU with autograd; the restatement itself is held against the C oracle at
configuration-1 size in this file.  Bound everywhere: 1e-5 relative L2 per gradient tensor (FP32 path)."""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as O
from oracle_lib import C1, rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture()
def ctx():
    from seraph_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg.V, n).astype(np.int32)


def torch_grads(cfg, p, tok, ss, lora=None, rank=0, alpha=0.0, mask=0):
    """loss and flat float64 gradients (of the weights, or of the adapters when `lora` is given) from autograd on the GPU"""
    import torch
    import torch_model as TM
    P = TM.unflatten(cfg, p, device="cuda", requires_grad=lora is None)
    LP = None
    if lora is not None:
        tens, n = cfg.lora_tensors(rank, mask)
        LP = {}
        for name, shp, off in tens:
            t = torch.tensor(lora[off:off + int(np.prod(shp))].reshape(shp), dtype=torch.float64, device="cuda", requires_grad=True)
            LP[name] = t
    loss, _ = TM.forward_loss(cfg, P, tok, ss, lora=LP, rank=rank, alpha=alpha)
    loss.backward()
    if lora is None:
        g = TM.flatten_grads(cfg, P)
    else:
        g = np.zeros(n, np.float64)
        for name, shp, off in tens:
            g[off:off + int(np.prod(shp))] = LP[name].grad.detach().cpu().numpy().ravel()
    out = float(loss.detach().cpu())
    del P, LP, loss
    torch.cuda.empty_cache()
    return out, g


def worst_tensor(tensors, got, ref, tol=TOL):
    worst = (0.0, None)
    for name, shp, off in tensors:
        n = int(np.prod(shp))
        e = rel_l2(got[off:off + n], ref[off:off + n])
        if e > worst[0]:
            worst = (e, name)
    assert worst[0] < tol, worst
    return worst


def run_full(ctx, cfg, p, tok, ss):
    from seraph_b200 import api
    ctx.lib.seraph_b200_reset_model(ctx.h)
    st = api.TrainState(cfg, p)
    loss = api.step_full_batch(ctx, st, tok, ss)
    ctx.check()
    ctx.lib.cuda_download_gpu_gradients(ctx.h, st.h)
    g = st.get(1)
    st.close()
    ctx.lib.seraph_b200_reset_model(ctx.h)              # give the arenas back before autograd needs the memory
    return loss, g


def test_float64_restatement_agrees_with_the_c_oracle_at_config1():
    """The checker of the large shapes, checked: float64 autograd against the FP64-accumulate C oracle, configuration 1
    (8 layers, hidden 512, 8 x 256 tokens), every gradient tensor."""
    cfg = C1
    p = cfg.init_params(1234)
    ss = list(range(0, 2049, 256))
    tok = tokens_for(cfg, 2048, 99)
    ref = O.train_step(cfg, p, tok, ss)
    loss, g = torch_grads(cfg, p, tok, ss)
    assert abs(loss - ref["loss"]) < 1e-6 * abs(ref["loss"])
    print("float64 restatement vs C oracle at config 1, worst tensor:", worst_tensor(cfg.tensors(), ref["grads"], g, tol=2e-6))


def test_qwen_shaped_two_layers_every_gradient(ctx):
    """Two layers of the benchmark's model at its full width: hidden 2048, 16 query / 8 K-V heads of 128 (GQA 2:1), FFN 6144,
    vocabulary 151936, two sequences of 2048 tokens - the K = 8192-class weight-gradient sums, the tail splits at N = 6144 and
    the grouped head map that the small models do not reach.  Every gradient tensor against float64 autograd."""
    cfg = O.ModelCfg(V=151936, d=2048, L=2, Hq=16, Hkv=8, hd=128, F=6144, theta=1e6)
    p = cfg.init_params(5, norm_jitter=0.1)
    ss = [0, 2048, 4096]
    tok = tokens_for(cfg, 4096, 6)
    loss, g = run_full(ctx, cfg, p, tok, ss)
    ref_loss, ref_g = torch_grads(cfg, p, tok, ss)
    assert abs(loss - ref_loss) < 1e-5 * abs(ref_loss), (loss, ref_loss)
    print("qwen-shaped 2 layers, worst gradient rel-L2:", worst_tensor(cfg.tensors(), g, ref_g))
    # embedding-gradient rows: exactly the rows some token or target-independent LM-head term touches are non-zero; the scatter
    # part lands on the rows the tokens name (integer indexing)
    ge = g[:cfg.V * cfg.d].reshape(cfg.V, cfg.d)
    re = ref_g[:cfg.V * cfg.d].reshape(cfg.V, cfg.d)
    rows = np.unique(tok)
    assert rel_l2(ge[rows], re[rows]) < TOL


def test_qwen_shaped_lora_rank16_qkvo(ctx):
    """Configuration 3 on two layers: frozen base of the Qwen-shaped model, LoRA rank 16, alpha 32 on q, k, v, o, adapters
    with B != 0 (B = 0 hides errors in gA), full chain rule; adapter gradients against float64 autograd."""
    from seraph_b200 import api
    cfg = O.ModelCfg(V=32768, d=2048, L=2, Hq=16, Hkv=8, hd=128, F=6144, theta=1e6)    # the vocabulary plays no part in the adapters' shapes
    rank, alpha, mask = 16, 32.0, 0b0001111
    p = cfg.init_params(15, norm_jitter=0.1)
    tens, n = cfg.lora_tensors(rank, mask)
    lo = (0.02 * np.random.default_rng(16).standard_normal(n)).astype(np.float32)
    ss = [0, 2048, 4096]
    tok = tokens_for(cfg, 4096, 17)
    ctx.lib.seraph_b200_reset_model(ctx.h)
    st = api.TrainState(cfg, p)
    st.attach_lora(rank, alpha, mask, lo)
    assert ctx.lib.seraph_b200_set_lora_exact(ctx.h, 1) == 0
    loss = api.step_lora_batch(ctx, st, tok, ss)
    ctx.check()
    ctx.lib.cuda_download_lora_weights(ctx.h, st.lora_ptr())
    g = st.lora_get(1)
    st.close()
    ctx.lib.seraph_b200_reset_model(ctx.h)
    assert ctx.lib.seraph_b200_set_lora_exact(ctx.h, 0) == 0
    ref_loss, ref_g = torch_grads(cfg, p, tok, ss, lora=lo, rank=rank, alpha=alpha, mask=mask)
    assert abs(loss - ref_loss) < 1e-5 * abs(ref_loss)
    print("config-3-shaped LoRA, worst adapter gradient rel-L2:", worst_tensor(tens, g, ref_g))


def attention_float64(Q, K, V, dO, ss, Hq, Hkv, hd):
    """causal attention per packed sequence and its gradients in float64 on the GPU (autograd)"""
    import torch
    T = Q.shape[0]
    q = torch.tensor(Q, dtype=torch.float64, device="cuda").view(T, Hq, hd).requires_grad_(True)
    k = torch.tensor(K, dtype=torch.float64, device="cuda").view(T, Hkv, hd).requires_grad_(True)
    v = torch.tensor(V, dtype=torch.float64, device="cuda").view(T, Hkv, hd).requires_grad_(True)
    do = torch.tensor(dO, dtype=torch.float64, device="cuda").view(T, Hq, hd)
    kv_of = (torch.arange(Hq, device="cuda") * Hkv) // Hq
    outs, lses = [], []
    for b in range(len(ss) - 1):
        s, e = int(ss[b]), int(ss[b + 1])
        S = e - s
        sc = torch.einsum("thd,shd->hts", q[s:e], k[s:e][:, kv_of]) / np.sqrt(hd)
        mask = torch.ones(S, S, dtype=torch.bool, device="cuda").tril()
        sc = sc.masked_fill(~mask[None], float("-inf"))
        lses.append(torch.logsumexp(sc, -1).T)
        outs.append(torch.einsum("hts,shd->thd", torch.softmax(sc, -1), v[s:e][:, kv_of]))
    out = torch.cat(outs, 0)
    (out * do).sum().backward()
    res = [x.detach().cpu().numpy().reshape(T, -1) for x in (out, torch.cat(lses, 0), q.grad, k.grad, v.grad)]
    del q, k, v, do, out, outs, lses
    torch.cuda.empty_cache()
    return res


def test_config2_attention_backward_microbench_shape(ctx):
    """Configuration 2 exactly: Q, K, V, dO ~ N(0,1) of logical shape B 8, H 16 (= K-V heads), S 2048, D 128, token-major
    packed, causal, scale 1/sqrt(128).  dQ, dK, dV (and O, LSE) against float64 autograd, and against the reference's own
    CUDA flash kernels run on this GPU from oracle/_ref (their float atomics are not bit-stable: tolerance 5e-5)."""
    B, H, S, D = 8, 16, 2048, 128
    T = B * S
    ss = np.arange(0, T + 1, S, dtype=np.uint32)
    r = np.random.default_rng(2048)
    Q, K, V, dO = (np.ascontiguousarray(r.standard_normal((T, H * D)), np.float32) for _ in range(4))
    bq, bk, bv, bdo, bs = ctx.upload(Q), ctx.upload(K), ctx.upload(V), ctx.upload(dO), ctx.upload(ss)
    bout, blse = ctx.zeros(Q.size), ctx.zeros(T * H)
    bdq, bdk, bdv = ctx.empty(Q.size), ctx.zeros(K.size), ctx.zeros(V.size)
    ctx.lib.cuda_train_batch_attention_packed(ctx.h, bq.b, bk.b, bv.b, bout.b, blse.b, bs.b, T, B, H, H, D, S)
    ctx.lib.cuda_train_batch_attention_backward_packed(ctx.h, bq.b, bk.b, bv.b, bout.b, blse.b, bdo.b, bdq.b, bdk.b, bdv.b, bs.b,
                                                       T, B, H, H, D, S)
    ctx.check()
    got = [x.numpy(shape=(T, -1)) for x in (bout, blse, bdq, bdk, bdv)]
    ctx.release(bq, bk, bv, bdo, bs, bout, blse, bdq, bdk, bdv)
    ref = attention_float64(Q, K, V, dO, ss, H, H, D)
    errs = {n: rel_l2(a, b) for n, a, b in zip(("O", "lse", "dQ", "dK", "dV"), got, ref)}
    print("config 2 vs float64:", errs)
    assert max(errs.values()) < TOL, errs
    L = O.ref_lib("cuda")
    if L is None:
        pytest.skip("oracle/_ref/libseraph_ref_cuda.so not built: float64 comparison done, reference CUDA kernels not run")
    fn = L.refshim_cuda_attention
    fn.restype = C.c_int
    fn.argtypes = [C.c_int] + [O.f32p] * 4 + [O.i32p] + [C.c_int] * 7 + [O.f32p] * 6
    rO, rl, rdq = np.empty_like(Q), np.empty((T, H), np.float32), np.empty_like(Q)
    rdk, rdv, ms = np.empty_like(K), np.empty_like(V), np.zeros(2, np.float32)
    rc = fn(0, Q, K, V, dO, ss.astype(np.int32), B, T, H, H, D, S, 1, rO, rl, rdq, rdk, rdv, ms)
    assert rc == 0, rc
    errs_ref = {n: rel_l2(a, b) for n, a, b in zip(("O", "lse", "dQ", "dK", "dV"), got, (rO, rl, rdq, rdk, rdv))}
    gap = {n: rel_l2(a, b) for n, a, b in zip(("O", "lse", "dQ", "dK", "dV"), (rO, rl, rdq, rdk, rdv), ref)}
    print("config 2 vs the reference CUDA flash kernels:", errs_ref, "| reference vs float64:", gap,
          f"| reference device time: forward {ms[0]:.1f} ms, backward {ms[1]:.1f} ms")
    assert max(errs_ref.values()) < 5e-5, errs_ref


@pytest.mark.parametrize("clip,above", [(0.05, True), (1e4, False)])
def test_gradient_clip_global_norm(ctx, clip, above):
    """seraph_b200_set_grad_clip (the reference has no clipping, so this is an added switch): with the gradient norm above the
    threshold the update equals AdamW on g * clip / (||g|| + 1e-6), below it the update is the unclipped one; the gradients
    that can be downloaded stay unscaled either way."""
    from seraph_b200 import api
    cfg, ss = O.TINY, O.TINY_SEQS
    p = cfg.init_params(7, norm_jitter=0.1)
    tok = tokens_for(cfg, ss[-1], 11)
    ref = O.train_step(cfg, p, tok, ss)
    gn = float(np.linalg.norm(ref["grads"].astype(np.float64)))
    assert (gn > clip) == above, gn
    f = np.float32(min(1.0, clip / (gn + 1e-6)))
    gs = (ref["grads"] * f).astype(np.float32)
    lr = O.lib().ref_effective_lr(3.14e-4, 1, 1)
    w, m, v = p.copy(), np.zeros_like(p), np.zeros_like(p)
    O.lib().ref_adamw(w, gs, m, v, p.size, lr, 0.9, 0.999, 0.01, 1e-8, 1)
    assert ctx.lib.seraph_b200_set_grad_clip(ctx.h, clip) == 0
    ctx.lib.seraph_b200_reset_model(ctx.h)
    st = api.TrainState(cfg, p)
    api.step_full_batch(ctx, st, tok, ss)
    ctx.check()
    ctx.lib.cuda_download_gpu_gradients(ctx.h, st.h)
    ctx.lib.cuda_download_full_weights(ctx.h, st.h)
    assert ctx.lib.seraph_b200_set_grad_clip(ctx.h, 0.0) == 0
    assert rel_l2(st.get(1), ref["grads"]) < TOL
    assert rel_l2(st.get(2), m) < TOL and rel_l2(st.get(3), v) < 2 * TOL and rel_l2(st.get(0), w) < 1e-6
    if above:
        m0 = np.zeros_like(p); v0 = np.zeros_like(p); w0 = p.copy()
        O.lib().ref_adamw(w0, ref["grads"], m0, v0, p.size, lr, 0.9, 0.999, 0.01, 1e-8, 1)
        assert rel_l2(st.get(2), m0) > 1e-2              # the clip did bite
    st.close()


def test_one_context_two_geometries(ctx):
    """A context that stepped one model and is then handed a deeper and wider one rebuilds its activation and adapter arenas
    for the new geometry (they were carved for the old one); both steps match the oracle."""
    from seraph_b200 import api
    small, ss = O.TINY, O.TINY_SEQS
    big = O.ModelCfg(V=300, d=128, L=3, Hq=4, Hkv=2, hd=32, F=160)
    for cfg, seed in ((small, 1), (big, 2), (small, 3)):
        p = cfg.init_params(seed, norm_jitter=0.1)
        tok = tokens_for(cfg, ss[-1], seed + 10)
        ref = O.train_step(cfg, p, tok, ss)
        st = api.TrainState(cfg, p)
        loss = api.step_full_batch(ctx, st, tok, ss)            # no reset in between: the context sees the geometry change
        ctx.check()
        ctx.lib.cuda_download_gpu_gradients(ctx.h, st.h)
        assert abs(loss - ref["loss"]) < 1e-5 * abs(ref["loss"])
        worst_tensor(cfg.tensors(), st.get(1), ref["grads"])
        st.close()
    # the same with adapters: rank-4 adapters on the small model, then on the big one
    for cfg, seed in ((small, 4), (big, 5)):
        rank, alpha, mask = 4, 8.0, 0x7F
        p = cfg.init_params(seed)
        tens, n = cfg.lora_tensors(rank, mask)
        lo = (0.05 * np.random.default_rng(seed).standard_normal(n)).astype(np.float32)
        tok = tokens_for(cfg, ss[-1], seed + 20)
        ref = O.train_step(cfg, p, tok, ss, lora=lo, rank=rank, alpha=alpha, mask=mask)
        st = api.TrainState(cfg, p)
        st.attach_lora(rank, alpha, mask, lo)
        api.step_lora_batch(ctx, st, tok, ss)
        ctx.check()
        ctx.lib.cuda_download_lora_weights(ctx.h, st.lora_ptr())
        worst_tensor(tens, st.lora_get(1), ref["grads"])
        st.close()


def test_nan_guard_skips_the_optimizer(ctx):
    """state->debug_nan_check: a non-finite value anywhere in the step sets the reference's per-buffer flags
    (src/train_cuda.c:626-645), the step returns NaN with nan_detected set, and neither the weights nor the optimizer
    counters move (src/train_cuda.c:1086-1187).  Without the flag set the same state steps normally."""
    from seraph_b200 import api
    cfg, ss = O.TINY, O.TINY_SEQS
    p = cfg.init_params(7)
    tok = tokens_for(cfg, ss[-1], 11)
    bad = p.copy()
    name, shp, off = [t for t in cfg.tensors() if t[0] == "l1.up"][0]
    bad[off + 3] = np.inf
    ctx.lib.seraph_b200_reset_model(ctx.h)
    st = api.TrainState(cfg, bad)
    ctx.lib.seraph_b200_state_set_debug_nan(st.h, 1)
    loss = api.step_full_batch(ctx, st, tok, ss)
    assert np.isnan(loss) and ctx.lib.seraph_b200_state_nan_detected(st.h) == 1
    assert st.counters() == (0, 0)
    ctx.lib.cuda_download_full_weights(ctx.h, st.h)
    assert np.array_equal(st.get(0), bad) and not st.get(2).any()       # weights and moments untouched
    flags = np.zeros(10 + 7 * cfg.L + 5, np.uint32)
    ctx.lib.seraph_b200_nan_flags(ctx.h, flags.ctypes.data, flags.size)
    assert flags[1] == 1 and flags[3] == 1 and flags[10 + 1] == 1 and flags[10 + 0] == 0      # logits, grad_logits, hidden after layer 1, not after layer 0
    assert flags[10 + 7 * cfg.L] == 0                                                         # embedding weights were finite
    st.close()
    # a finite model with the check on steps as usual
    ctx.lib.seraph_b200_reset_model(ctx.h)
    st = api.TrainState(cfg, p)
    ctx.lib.seraph_b200_state_set_debug_nan(st.h, 1)
    loss = api.step_full_batch(ctx, st, tok, ss)
    assert np.isfinite(loss) and st.counters() == (1, 0) and ctx.lib.seraph_b200_state_nan_detected(st.h) == 0
    st.close()


def test_profiler_sees_the_training_step(ctx):
    """A cuda_profiler_t attached with cuda_train_set_profiler records the step's own launches (the CLI's --profile N,
    tools/seraph_train_cuda.c:423-470): ops are present and the category totals of the reference's report are filled."""
    from seraph_b200 import api
    cfg, ss = O.TINY, O.TINY_SEQS
    p = cfg.init_params(7)
    tok = tokens_for(cfg, ss[-1], 11)
    ctx.lib.seraph_b200_reset_model(ctx.h)
    st = api.TrainState(cfg, p)
    api.step_full_batch(ctx, st, tok, ss)
    prof = ctx.lib.cuda_profiler_create()
    assert prof
    ctx.lib.cuda_profiler_enable(prof)
    ctx.lib.cuda_train_set_profiler(ctx.h, prof)
    api.step_full_batch(ctx, st, tok, ss)
    ctx.sync()                                          # the report is analysed on the context's stream (the CLI passes ctx->stream)
    ctx.lib.cuda_profiler_sync_and_analyze(prof, None)
    tot = np.zeros(12, np.float32)
    n_ops = ctx.lib.seraph_b200_profiler_totals(prof, tot.ctypes.data)
    ctx.lib.cuda_train_set_profiler(ctx.h, None)
    ctx.lib.cuda_profiler_destroy(prof)
    st.close()
    names = ["step", "matmul", "attention", "attention_bwd", "rmsnorm", "rmsnorm_bwd", "cross_entropy", "adamw", "copy", "other"]
    got = dict(zip(names, tot[:10]))
    assert n_ops > 50, n_ops
    for k in ("matmul", "attention", "attention_bwd", "rmsnorm", "rmsnorm_bwd", "cross_entropy", "adamw"):
        assert got[k] > 0, (k, got)
    assert abs(got["step"] - sum(v for k, v in got.items() if k != "step")) < 1e-3 * got["step"]


def test_bounded_wait_runs_out_and_the_context_survives(ctx):
    """Every spin of the tensor-core kernels is a bounded mbarrier wait.  A one-warp kernel waits on a barrier that nothing
    completes with a limit of two million cycles (about a millisecond): it gives up, the host reads status 5, and the same
    context then runs a training step that matches the oracle."""
    import ctypes as C
    from seraph_b200 import api
    waited = C.c_longlong(0)
    assert ctx.lib.seraph_b200_selftest_bounded_wait(ctx.h, 2_000_000, C.byref(waited)) == 0
    assert ctx.status() == 5                                  # SB_ERR_TIMEOUT
    assert 2_000_000 <= waited.value < 200_000_000
    assert ctx.status() == 0                                  # reading the status clears it
    cfg, ss = O.TINY, O.TINY_SEQS
    p = cfg.init_params(7)
    tok = tokens_for(cfg, ss[-1], 11)
    ref = O.train_step(cfg, p, tok, ss)
    st = api.TrainState(cfg, p)
    loss = api.step_full_batch(ctx, st, tok, ss)
    ctx.check()
    assert abs(loss - ref["loss"]) < 1e-5 * abs(ref["loss"])
    st.close()


def write_hf_safetensors(path, cfg, p):
    """A BF16 safetensors file with Hugging Face tensor names and true shapes, as a model directory holds it (the reference's
    own checkpoint writer states hidden x hidden for the K and V projections of grouped-query models, src/train.c:472-473, so
    its header cannot be used to locate tensors)."""
    import json
    names = {"embed": "model.embed_tokens.weight", "final_norm": "model.norm.weight", "q": "self_attn.q_proj", "k": "self_attn.k_proj",
             "v": "self_attn.v_proj", "o": "self_attn.o_proj", "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj",
             "in_norm": "input_layernorm", "post_norm": "post_attention_layernorm"}
    header, blobs, off = {"__metadata__": {"format": "pt"}}, [], 0
    for name, shp, o in cfg.tensors():
        n = int(np.prod(shp))
        if name.startswith("l") and "." in name:
            l, short = name[1:].split(".", 1)
            full = f"model.layers.{l}.{names[short]}.weight"
        else:
            full = names[name]
        raw = (p[o:o + n].view(np.uint32) >> 16).astype(np.uint16).tobytes()
        header[full] = {"dtype": "BF16", "shape": list(shp), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw); off += len(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(len(h).to_bytes(8, "little")); f.write(h)
        for bl in blobs:
            f.write(bl)


def test_lora_state_without_host_weights_reads_the_bf16_model(ctx, tmp_path):
    """The state the reference's train_init builds for LoRA training has no FP32 host copies (full_weights is NULL,
    src/train.c:7900-7909): the frozen base comes from the BF16 tensors of the memory-mapped model, by name
    (src/train_cuda.c:1376-1460).  Such a state steps and evaluates, its adapter gradients are bit-identical to those of a
    state that carries the same BF16-rounded weights as FP32 host arrays, and they match the oracle."""
    from seraph_b200 import api
    cfg, ss = O.ModelCfg(V=1024, d=512, L=2, Hq=4, Hkv=2, hd=128, F=1024, theta=1e4), [0, 300, 512, 645]
    rank, alpha, mask = 8, 16.0, 0b0001111
    p = cfg.init_params(81, norm_jitter=0.1)
    p_bf16 = (p.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)        # what the file will hold (truncation, src/train.c:255-260)
    tens, n = cfg.lora_tensors(rank, mask)
    lo = (0.02 * np.random.default_rng(82).standard_normal(n)).astype(np.float32)
    tok = tokens_for(cfg, ss[-1], 83)
    path = str(tmp_path / "base.safetensors")
    write_hf_safetensors(path, cfg, p)
    grads = []
    for from_file in (False, True):
        ctx.lib.seraph_b200_reset_model(ctx.h)
        s = api.TrainState(cfg, p_bf16)
        s.attach_lora(rank, alpha, mask, lo)
        if from_file:
            assert ctx.lib.seraph_b200_state_attach_model_file(s.h, path.encode()) == 0
        loss = api.step_lora_batch(ctx, s, tok, ss)
        ctx.check()
        assert loss > 0
        ev = ctx.lib.cuda_eval_forward(s.h, tok.ctypes.data, 300, ctx.h)
        assert ev > 0
        ctx.lib.cuda_download_lora_weights(ctx.h, s.lora_ptr())
        grads.append((loss, s.lora_get(1)))
        s.close()
    assert grads[0][0] == grads[1][0] and np.array_equal(grads[0][1], grads[1][1])
    ref = O.train_step(cfg, p_bf16, tok, ss, lora=lo, rank=rank, alpha=alpha, mask=mask)
    assert abs(grads[1][0] - ref["loss"]) < 1e-5 * abs(ref["loss"])
    worst_tensor(tens, grads[1][1], ref["grads"])


@pytest.mark.parametrize("head_norm,untied", [(1, 0), (0, 1), (1, 1)])
def test_per_head_qk_norm_and_untied_lm_head(ctx, head_norm, untied):
    """The model options that let Qwen3- and Mistral-shaped configurations run as written (not part of the reference's
    training step, so pinned against the oracle's restatement, itself held against float64 autograd in tests/test_oracle.py):
    a learned RMSNorm over each head of q and k before RoPE, and a separate lm_head.  Full-weight step: every weight gradient,
    the gradients of the extra parameters and their AdamW update; tiny shape and a 128-wide-head shape."""
    import dataclasses
    from seraph_b200 import api
    for base, ss, seed in ((O.TINY, O.TINY_SEQS, 91), (O.ModelCfg(V=1024, d=512, L=2, Hq=4, Hkv=2, hd=128, F=1024, theta=1e4), [0, 300, 512, 645], 92)):
        cfg = dataclasses.replace(base, head_norm=head_norm, untied=untied)
        p = cfg.init_params(seed, norm_jitter=0.1)
        x = cfg.init_extras(seed + 1)
        tok = tokens_for(cfg, ss[-1], seed + 2)
        ref = O.train_step(cfg, p, tok, ss, extras=x)
        assert ctx.lib.seraph_b200_set_model_extras(ctx.h, head_norm, untied, x.ctypes.data, x.size) == 0
        st = api.TrainState(cfg, p)
        loss = api.step_full_batch(ctx, st, tok, ss)
        ctx.check()
        assert abs(loss - ref["loss"]) < 1e-5 * abs(ref["loss"]), (loss, ref["loss"])
        ctx.lib.cuda_download_gpu_gradients(ctx.h, st.h)
        worst_tensor(cfg.tensors(), st.get(1), ref["grads"])
        xg, xw = np.empty_like(x), np.empty_like(x)
        assert ctx.lib.seraph_b200_get_model_extras(ctx.h, 1, xg.ctypes.data, xg.size) == 0
        assert ctx.lib.seraph_b200_get_model_extras(ctx.h, 0, xw.ctypes.data, xw.size) == 0
        print("extra parameters, worst gradient:", worst_tensor(cfg.extras_tensors()[0], xg, ref["extras_grads"]))
        w, m, v = x.copy(), np.zeros_like(x), np.zeros_like(x)
        O.lib().ref_adamw(w, ref["extras_grads"], m, v, x.size, O.lib().ref_effective_lr(3.14e-4, 1, 1), 0.9, 0.999, 0.01, 1e-8, 1)
        assert rel_l2(xw, w) < 1e-6 and not np.array_equal(xw, x)
        st.close()
        # LoRA on top: the extra parameters are frozen, adapters see them in the forward and backward pass
        rank, alpha, mask = 4, 8.0, 0x7F
        tens, n = cfg.lora_tensors(rank, mask)
        lo = (0.05 * np.random.default_rng(seed + 3).standard_normal(n)).astype(np.float32)
        refl = O.train_step(cfg, p, tok, ss, lora=lo, rank=rank, alpha=alpha, mask=mask, extras=x)
        assert ctx.lib.seraph_b200_set_model_extras(ctx.h, head_norm, untied, x.ctypes.data, x.size) == 0
        st = api.TrainState(cfg, p)
        st.attach_lora(rank, alpha, mask, lo)
        loss = api.step_lora_batch(ctx, st, tok, ss)
        ctx.check()
        assert abs(loss - refl["loss"]) < 1e-5 * abs(refl["loss"])
        ctx.lib.cuda_download_lora_weights(ctx.h, st.lora_ptr())
        worst_tensor(tens, st.lora_get(1), refl["grads"])
        st.close()
    assert ctx.lib.seraph_b200_set_model_extras(ctx.h, 0, 0, None, 0) == 0
