"""Pins the CPU oracle before anything is checked against it.

The reference ships no golden vectors for the training path, so the oracle is
pinned (a) against the reference's own CPU code compiled from its sources
(forward logits, loss, cross-entropy gradient, AdamW, LoRA adapter gradients;
skipped where oracle/_ref was not built) and (b) against float64 autograd of
an independent torch restatement (every weight gradient, LoRA gradients)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle_lib as O
from oracle_lib import TINY, TINY_SEQS, rel_l2
import torch_model as TM


def tiny_tokens(seed=1, n=TINY_SEQS[-1], V=TINY.V):
    return np.random.default_rng(seed).integers(0, V, n).astype(np.int32)


def test_param_count_matches_layout():
    c = TINY.c()
    assert O.lib().ref_param_count(C.byref(c)) == TINY.n_params()
    c1 = O.C1.c()
    assert O.lib().ref_param_count(C.byref(c1)) == 29_893_120


@pytest.fixture(scope="module")
def refcpu():
    L = O.ref_lib("cpu")
    if L is None:
        pytest.skip("oracle/_ref not built (no reference checkout)")
    return L


def test_forward_and_loss_match_reference_cpu(refcpu):
    """One sequence (the reference CPU path takes one per call)."""
    cfg, n = TINY, 17
    p = cfg.init_params(3, norm_jitter=0.1)
    tok = tiny_tokens(5, n)
    st = O.ref_state(refcpu, cfg, 32)
    refcpu.refshim_set(st, 0, p)
    ref_logits = np.empty((n, cfg.V), np.float32)
    assert refcpu.refshim_forward(st, tok, n, ref_logits) == 0
    out = O.train_step(cfg, p, tok, [0, n], want_logits=True)
    assert rel_l2(out["logits"], ref_logits) < 2e-6
    ref_loss = refcpu.refshim_train_step(st, tok, n)
    assert abs(out["loss"] - ref_loss) < 2e-6 * abs(ref_loss)
    refcpu.refshim_destroy(st)


def test_cross_entropy_grad_matches_reference_cpu(refcpu):
    V, T = 257, 6
    rng = np.random.default_rng(0)
    logits = rng.standard_normal((T, V)).astype(np.float32) * 3
    tgt = rng.integers(0, V, T).astype(np.uint32)
    grad = np.empty_like(logits)
    rows = np.empty(T, np.float32)
    ss = np.array([0, T], np.uint32)
    nv = T - 1
    O.lib().ref_cross_entropy_grad(logits, tgt, grad, rows, ss, T, 1, V, nv)
    assert np.all(grad[-1] == 0) and rows[-1] == 0
    for t in range(T - 1):
        g = np.empty(V, np.float32)
        refcpu.refshim_loss_gradient(g, logits[t].copy(), int(tgt[t]), V)
        # the CPU path leaves out the 1/num_valid the GPU paths apply
        assert rel_l2(grad[t] * nv, g) < 1e-6


def test_adamw_matches_reference_cpu(refcpu):
    rng = np.random.default_rng(2)
    n = 1000
    w = rng.standard_normal(n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32) * 0.1
    m = rng.standard_normal(n).astype(np.float32) * 0.01
    v = np.abs(rng.standard_normal(n)).astype(np.float32) * 0.001
    a = [x.copy() for x in (w, g, m, v)]
    b = [x.copy() for x in (w, g, m, v)]
    O.lib().ref_adamw(a[0], a[1], a[2], a[3], n, 3.14e-4, 0.9, 0.999, 0.01, 1e-8, 7)
    refcpu.refshim_adamw(b[0], b[1], b[2], b[3], n, 3.14e-4, 0.9, 0.999, 0.01, 1e-8, 7)
    for x, y in zip(a, b):
        assert rel_l2(x, y) < 1e-6


def test_lora_backward_matches_reference_cpu(refcpu):
    rng = np.random.default_rng(4)
    T, i, o, r, alpha = 9, 24, 40, 4, 8.0
    A = rng.standard_normal((r, i)).astype(np.float32)
    B = rng.standard_normal((o, r)).astype(np.float32)
    x = rng.standard_normal((T, i)).astype(np.float32)
    dy = rng.standard_normal((T, o)).astype(np.float32)
    gA, gB = np.zeros_like(A), np.zeros_like(B)
    tmp = np.zeros((T, r), np.float32)
    O.lib().ref_lora_backward(dy, x, A, B, gA, gB, tmp, T, i, o, r, alpha / r)
    rA, rB = np.zeros_like(A), np.zeros_like(B)
    refcpu.refshim_lora_backward(A, B, rA, rB, x, dy, None, T, i, o, r, alpha)
    assert rel_l2(gA, rA) < 1e-6 and rel_l2(gB, rB) < 1e-6


def test_full_gradients_match_autograd_float64():
    cfg = TINY
    p = cfg.init_params(7, norm_jitter=0.1)
    tok = tiny_tokens(11)
    out = O.train_step(cfg, p, tok, TINY_SEQS, want_logits=True)
    P = TM.unflatten(cfg, p)
    loss, logits = TM.forward_loss(cfg, P, tok, TINY_SEQS)
    loss.backward()
    g = TM.flatten_grads(cfg, P)
    assert abs(out["loss"] - loss.item()) < 1e-6
    assert rel_l2(out["logits"], logits.detach().numpy()) < 1e-6
    for name, shp, off in cfg.tensors():
        n = int(np.prod(shp))
        assert rel_l2(out["grads"][off:off + n], g[off:off + n]) < 2e-6, name


def test_full_gradients_with_qk_norm_match_autograd_float64():
    """config->use_qk_norm: q and k normalised over the whole token row after RoPE.  The reference's training has no
    backward for it; the oracle step's is the derivative of the forward, checked here against float64 autograd."""
    import dataclasses
    cfg = dataclasses.replace(TINY, qk_norm=1)
    p = cfg.init_params(8, norm_jitter=0.1)
    tok = tiny_tokens(12)
    out = O.train_step(cfg, p, tok, TINY_SEQS, want_logits=True)
    P = TM.unflatten(cfg, p)
    loss, logits = TM.forward_loss(cfg, P, tok, TINY_SEQS)
    loss.backward()
    g = TM.flatten_grads(cfg, P)
    assert abs(out["loss"] - loss.item()) < 1e-6
    for name, shp, off in cfg.tensors():
        n = int(np.prod(shp))
        assert rel_l2(out["grads"][off:off + n], g[off:off + n]) < 2e-6, name
    plain = O.train_step(TINY, p, tok, TINY_SEQS)
    assert abs(plain["loss"] - out["loss"]) > 1e-4          # the switch does something


def test_gradient_accumulation_adds():
    cfg = TINY
    p = cfg.init_params(7)
    tok = tiny_tokens(11)
    one = O.train_step(cfg, p, tok, TINY_SEQS)["grads"]
    two = O.train_step(cfg, p, tok, TINY_SEQS, grads=one.copy())["grads"]
    assert rel_l2(two, 2 * one) < 1e-6


def test_negative_tokens_clamp_and_empty_batch():
    cfg = TINY
    p = cfg.init_params(7)
    tok = tiny_tokens(11)
    neg = tok.copy()
    neg[3] = -5
    z = tok.copy()
    z[3] = 0
    a = O.train_step(cfg, p, neg, TINY_SEQS)
    b = O.train_step(cfg, p, z, TINY_SEQS)
    assert a["loss"] == b["loss"] and np.array_equal(a["grads"], b["grads"])
    # one-token sequences predict nothing: loss 0 (src/train_cuda.c:1990-1991)
    assert O.train_step(cfg, p, tok[:3], [0, 1, 2, 3])["loss"] == 0.0


@pytest.mark.parametrize("exact", [0, 1])
def test_lora_gradients_match_autograd_float64(exact):
    cfg, rank, alpha, mask = TINY, 4, 8.0, 0x7F
    p = cfg.init_params(7, norm_jitter=0.1)
    tens, n = cfg.lora_tensors(rank, mask)
    rng = np.random.default_rng(9)
    lo = (0.05 * rng.standard_normal(n)).astype(np.float32)
    if not exact:
        # with B = 0 the adapters add nothing to dX, so the reference's
        # omission of that term is invisible and autograd is the exact answer
        for name, shp, off in tens:
            if name.endswith(".B"):
                lo[off:off + int(np.prod(shp))] = 0
    tok = tiny_tokens(11)
    out = O.train_step(cfg, p, tok, TINY_SEQS, lora=lo, rank=rank, alpha=alpha, mask=mask, lora_exact=exact)
    P = TM.unflatten(cfg, p, requires_grad=False)
    Lt = {}
    for name, shp, off in tens:
        t = torch.tensor(lo[off:off + int(np.prod(shp))].reshape(shp), dtype=torch.float64, requires_grad=True)
        Lt[name] = t
    loss, _ = TM.forward_loss(cfg, P, tok, TINY_SEQS, lora=Lt, rank=rank, alpha=alpha)
    loss.backward()
    assert abs(out["loss"] - loss.item()) < 1e-6
    for name, shp, off in tens:
        g = out["grads"][off:off + int(np.prod(shp))]
        ref = Lt[name].grad.numpy().ravel()
        if np.linalg.norm(ref) == 0:
            assert np.linalg.norm(g) == 0, name
        else:
            assert rel_l2(g, ref) < 2e-6, name


@pytest.mark.parametrize("eps", [1e-5, 10.0])           # the second makes the clamp active on every row
def test_qk_norm_forward_follows_shader_and_backward_is_its_derivative(eps):
    """qk_norm (shaders/qk_norm.comp): y = x / max(sqrt(mean(x^2)), eps) over the whole token row.  The reference has no
    backward; the oracle's is checked against float64 autograd of the same forward."""
    T, H, hd = 5, 3, 8
    r = np.random.default_rng(3)
    x = r.standard_normal((T, H * hd)).astype(np.float32)
    dy = r.standard_normal((T, H * hd)).astype(np.float32)
    y = x.copy(); rms = np.zeros(T, np.float32)
    O.lib().ref_qk_norm(y, rms.ctypes.data, T, H, hd, 1, eps)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    rt = torch.sqrt((xt * xt).mean(dim=1, keepdim=True))
    yt = xt / torch.clamp(rt, min=eps)
    assert rel_l2(y, yt.detach().numpy()) < 1e-6 and rel_l2(rms, rt.detach().numpy().ravel()) < 1e-6
    (yt * torch.tensor(dy, dtype=torch.float64)).sum().backward()
    dx = np.empty_like(x)
    O.lib().ref_qk_norm_backward(y, rms, dy, dx, T, H, hd, 1, eps)
    assert rel_l2(dx, xt.grad.numpy()) < 1e-6
    # disabled: forward leaves the row alone, backward passes the gradient through
    y2 = x.copy()
    O.lib().ref_qk_norm(y2, None, T, H, hd, 0, eps)
    O.lib().ref_qk_norm_backward(y2, rms, dy, dx, T, H, hd, 0, eps)
    assert np.array_equal(y2, x) and np.array_equal(dx, dy)


@pytest.mark.parametrize("head_norm,untied", [(1, 0), (0, 1), (1, 1)])
def test_extras_per_head_norm_and_untied_head_match_autograd_float64(head_norm, untied):
    """The two model options the reference's training step lacks (a learned RMSNorm over each head of q and k before RoPE;
    a separate lm_head): the oracle's gradients of every weight and of the extra parameters against float64 autograd."""
    import dataclasses
    cfg = dataclasses.replace(TINY, head_norm=head_norm, untied=untied)
    p = cfg.init_params(31, norm_jitter=0.1)
    x = cfg.init_extras(32)
    tok = np.random.default_rng(33).integers(0, cfg.V, TINY_SEQS[-1]).astype(np.int32)
    ref = O.train_step(cfg, p, tok, TINY_SEQS, extras=x)
    P = TM.unflatten(cfg, p)
    X = TM.unflatten_extras(cfg, x)
    loss, _ = TM.forward_loss(cfg, P, tok, TINY_SEQS, X=X)
    loss.backward()
    g = TM.flatten_grads(cfg, P)
    assert abs(ref["loss"] - float(loss)) < 1e-6 * float(loss)
    for name, shp, off in cfg.tensors():
        n = int(np.prod(shp))
        assert rel_l2(ref["grads"][off:off + n], g[off:off + n]) < 2e-6, name
    for name, shp, off in cfg.extras_tensors()[0]:
        n = int(np.prod(shp))
        assert rel_l2(ref["extras_grads"][off:off + n], X[name].grad.numpy().ravel()) < 2e-6, name
    base = O.train_step(TINY, p, tok, TINY_SEQS)
    assert abs(base["loss"] - ref["loss"]) > 1e-5          # the options do change the model
