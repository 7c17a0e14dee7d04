"""Per-op parity on a B200: every backward (and forward) op is called through
the C ABI and compared with the CPU oracle on the same seeded inputs.
Tolerances: 1e-5 relative L2 for floating point (most ops land near 1e-7),
bit-exact for integer tables; every kernel must give the same bits twice."""
import os

import numpy as np
import pytest

import oracle_lib as O
from oracle_lib import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def ctx():
    from seraph_b200 import api
    c = api.Context(0)
    c.set_gemm_mode(api.GEMM_FP16X3)
    yield c
    c.close()


def rng(seed):
    return np.random.default_rng(seed)


def f32(a):
    return np.ascontiguousarray(a, np.float32)


@pytest.mark.parametrize("M,N,K", [(5, 7, 3), (64, 64, 64), (130, 257, 96), (257, 64, 24), (512, 384, 256), (1024, 1024, 512)])
@pytest.mark.parametrize("tA,tB,acc", [(0, 0, 0), (1, 0, 1), (0, 1, 0), (0, 1, 1)])
def test_matmul(ctx, M, N, K, tA, tB, acc):
    r = rng(M * 7 + N * 3 + K + tA * 2 + tB)
    A = f32(r.standard_normal((K, M) if tA else (M, K)))
    B = f32(r.standard_normal((N, K) if tB else (K, N)))
    C0 = f32(r.standard_normal((M, N)))
    ref = C0.copy()
    O.lib().ref_matmul(A, B, ref, M, N, K, tA, tB, acc)
    a, b, c = ctx.upload(A), ctx.upload(B), ctx.upload(C0)
    ctx.lib.cuda_train_matmul_transpose(ctx.h, a.b, b.b, c.b, M, N, K, tA, tB, acc)
    out = c.numpy(shape=(M, N))
    ctx.check()
    assert rel_l2(out, ref) < TOL
    c2 = ctx.upload(C0)
    ctx.lib.cuda_train_matmul_transpose(ctx.h, a.b, b.b, c2.b, M, N, K, tA, tB, acc)
    assert np.array_equal(c2.numpy(shape=(M, N)), out)
    ctx.release(a, b, c, c2)


def test_matmul_simt_mode_matches(ctx):
    from seraph_b200 import api
    r = rng(3)
    M, N, K = 300, 200, 128
    A, B = f32(r.standard_normal((M, K))), f32(r.standard_normal((K, N)))
    ref = np.zeros((M, N), np.float32)
    O.lib().ref_matmul(A, B, ref, M, N, K, 0, 0, 0)
    a, b, c = ctx.upload(A), ctx.upload(B), ctx.zeros(M * N)
    ctx.set_gemm_mode(api.GEMM_SIMT)
    ctx.lib.cuda_train_matmul(ctx.h, a.b, b.b, c.b, M, N, K)
    ctx.set_gemm_mode(api.GEMM_FP16X3)
    assert rel_l2(c.numpy(shape=(M, N)), ref) < TOL
    ctx.release(a, b, c)


@pytest.mark.parametrize("rows,cols", [(1, 32), (24, 64), (300, 512), (77, 2048), (5, 100), (4096, 128), (1501, 128)])
def test_rmsnorm_forward_backward(ctx, rows, cols):
    r = rng(rows + cols)
    x, w, dy = f32(r.standard_normal((rows, cols))), f32(1 + 0.1 * r.standard_normal(cols)), f32(r.standard_normal((rows, cols)))
    y_ref = np.empty_like(x)
    O.lib().ref_rmsnorm(x, w, y_ref, rows, cols, 1e-5)
    dx_ref, ds_ref = np.empty_like(x), f32(r.standard_normal(cols))
    ds0 = ds_ref.copy()
    O.lib().ref_rmsnorm_backward(x, w, dy, dx_ref, ds_ref, rows, cols, 1e-5)
    bx, bw, bdy, by, bdx, bds = ctx.upload(x), ctx.upload(w), ctx.upload(dy), ctx.empty(x.size), ctx.empty(x.size), ctx.upload(ds0)
    ctx.lib.cuda_train_rmsnorm(ctx.h, bx.b, bw.b, by.b, rows, cols, 1e-5)
    ctx.lib.cuda_train_rmsnorm_backward_batch(ctx.h, bx.b, bw.b, bdy.b, bdx.b, bds.b, rows, cols, 1e-5)
    ctx.check()
    assert rel_l2(by.numpy(), y_ref) < TOL
    dx1, ds1 = bdx.numpy(), bds.numpy()
    assert rel_l2(dx1, dx_ref) < TOL
    assert rel_l2(ds1, ds_ref) < TOL          # accumulated into the incoming values
    bds2 = ctx.upload(ds0)
    ctx.lib.cuda_train_rmsnorm_backward_batch(ctx.h, bx.b, bw.b, bdy.b, bdx.b, bds2.b, rows, cols, 1e-5)
    assert np.array_equal(bds2.numpy(), ds1) and np.array_equal(bdx.numpy(), dx1)
    ctx.release(bx, bw, bdy, by, bdx, bds, bds2)


@pytest.mark.parametrize("n", [1, 5, 4096, 100003])
def test_elementwise(ctx, n):
    r = rng(n)
    a, b, g = f32(r.standard_normal(n)), f32(r.standard_normal(n)), f32(r.standard_normal(n))
    L = O.lib()
    ba, bb, bg, o1, o2 = ctx.upload(a), ctx.upload(b), ctx.upload(g), ctx.empty(n), ctx.empty(n)
    ref = np.empty_like(a)
    L.ref_add(a, b, ref, n); ctx.lib.cuda_train_add(ctx.h, ba.b, bb.b, o1.b, n); assert np.array_equal(o1.numpy(), ref)
    L.ref_mul(a, b, ref, n); ctx.lib.cuda_train_mul(ctx.h, ba.b, bb.b, o1.b, n); assert np.array_equal(o1.numpy(), ref)
    L.ref_silu(a, ref, n); ctx.lib.cuda_train_silu(ctx.h, ba.b, o1.b, n); assert rel_l2(o1.numpy(), ref) < TOL
    L.ref_silu_backward(a, g, ref, n); ctx.lib.cuda_train_silu_backward(ctx.h, ba.b, bg.b, o1.b, n); assert rel_l2(o1.numpy(), ref) < TOL
    dA, dB = np.empty_like(a), np.empty_like(a)
    L.ref_mul_backward(a, b, g, dA, dB, n)
    ctx.lib.cuda_train_elementwise_mul_backward(ctx.h, ba.b, bb.b, bg.b, o1.b, o2.b, n)
    assert np.array_equal(o1.numpy(), dA) and np.array_equal(o2.numpy(), dB)
    # fused SwiGLU = silu, mul / mul_backward, silu_backward of the reference's step
    s, h = np.empty_like(a), np.empty_like(a)
    L.ref_silu(a, s, n); L.ref_mul(s, b, h, n)
    ctx.lib.seraph_b200_swiglu(ctx.h, ba.b, bb.b, o1.b, n); assert rel_l2(o1.numpy(), h) < TOL
    dsl, dup, dgt = np.empty_like(a), np.empty_like(a), np.empty_like(a)
    L.ref_mul_backward(s, b, g, dsl, dup, n); L.ref_silu_backward(a, dsl, dgt, n)
    ctx.lib.seraph_b200_swiglu_backward(ctx.h, ba.b, bb.b, bg.b, o1.b, o2.b, n)
    assert rel_l2(o1.numpy(), dgt) < TOL and rel_l2(o2.numpy(), dup) < TOL
    sc = a.copy(); L.ref_scale(sc, n, 0.37)
    ctx.lib.cuda_train_scale(ctx.h, ba.b, n, 0.37); assert np.array_equal(ba.numpy(), sc)
    ctx.check()
    ctx.release(ba, bb, bg, o1, o2)


@pytest.mark.parametrize("H,hd,theta", [(4, 16, 10000.0), (8, 64, 10000.0), (3, 128, 1e6), (2, 90, 10000.0)])
def test_rope_packed_forward_backward(ctx, H, hd, theta):
    ss = np.array([0, 7, 19, 24, 300], np.uint32)
    T, B = int(ss[-1]), len(ss) - 1
    x = f32(rng(H + hd).standard_normal((T, H * hd)))
    bx, bo, bs = ctx.upload(x), ctx.empty(x.size), ctx.upload(ss)
    for bwd, fn in [(0, ctx.lib.cuda_train_rope_packed), (1, ctx.lib.cuda_train_rope_backward_packed)]:
        ref = np.empty_like(x)
        O.lib().ref_rope(x, ref, ss, T, B, H, hd, theta, bwd)
        fn(ctx.h, bx.b, bo.b, bs.b, T, B, H, hd, theta)
        assert rel_l2(bo.numpy(), ref) < TOL
    # unpacked twin: positions run over the whole buffer
    one = np.array([0, T], np.uint32)
    ref = np.empty_like(x)
    O.lib().ref_rope(x, ref, one, T, 1, H, hd, theta, 0)
    ctx.lib.cuda_train_rope(ctx.h, bx.b, bo.b, T, H, hd, theta)
    assert rel_l2(bo.numpy(), ref) < TOL
    # in place, and backward undoes forward
    ctx.lib.cuda_train_rope_packed(ctx.h, bx.b, bx.b, bs.b, T, B, H, hd, theta)
    ctx.lib.cuda_train_rope_backward_packed(ctx.h, bx.b, bx.b, bs.b, T, B, H, hd, theta)
    assert rel_l2(bx.numpy(), x) < TOL
    ctx.check()
    ctx.release(bx, bo, bs)


ATT_CASES = [
    # (seq_starts, Hq, Hkv, hd)
    ([0, 7, 19, 24], 4, 2, 16),
    ([0, 130], 2, 2, 64),
    ([0, 64, 129, 200, 333], 8, 2, 32),
    ([0, 257], 4, 1, 128),
    ([0, 100, 190], 2, 1, 90),
    ([0, 300, 700], 4, 2, 64),
    ([0, 1024], 4, 1, 128),
    ([0, 513, 640, 1100], 6, 3, 32),
]


@pytest.mark.parametrize("fused", [0, 1])
@pytest.mark.parametrize("ss,Hq,Hkv,hd", ATT_CASES)
def test_attention_forward_backward(ctx, ss, Hq, Hkv, hd, fused):
    """fused = 1: P and dS of the backward come out of the score products' epilogues instead of a streaming kernel."""
    ctx.set_attn_fused(fused)
    ss = np.array(ss, np.uint32)
    T, B = int(ss[-1]), len(ss) - 1
    r = rng(T + Hq + hd)
    Q, K, V = f32(r.standard_normal((T, Hq * hd))), f32(r.standard_normal((T, Hkv * hd))), f32(r.standard_normal((T, Hkv * hd)))
    dO = f32(r.standard_normal((T, Hq * hd)))
    out_ref, lse_ref = np.empty_like(Q), np.empty((T, Hq), np.float32)
    O.lib().ref_attention(Q, K, V, out_ref, lse_ref, ss, T, B, Hq, Hkv, hd)
    dQ_ref = np.empty_like(Q)
    dK0, dV0 = f32(r.standard_normal(K.shape)), f32(r.standard_normal(V.shape))     # accumulated into
    dK_ref, dV_ref = dK0.copy(), dV0.copy()
    O.lib().ref_attention_backward(Q, K, V, dO, dQ_ref, dK_ref, dV_ref, ss, T, B, Hq, Hkv, hd)
    bq, bk, bv, bdo, bs = ctx.upload(Q), ctx.upload(K), ctx.upload(V), ctx.upload(dO), ctx.upload(ss)
    bout, blse, bdq, bdk, bdv = ctx.empty(Q.size), ctx.empty(T * Hq), ctx.empty(Q.size), ctx.upload(dK0), ctx.upload(dV0)
    ctx.lib.cuda_train_batch_attention_packed(ctx.h, bq.b, bk.b, bv.b, bout.b, blse.b, bs.b, T, B, Hq, Hkv, hd, int(np.diff(ss).max()))
    ctx.check()
    assert rel_l2(bout.numpy(), out_ref) < TOL
    assert rel_l2(blse.numpy(), lse_ref) < TOL
    ctx.lib.cuda_train_batch_attention_backward_packed(ctx.h, bq.b, bk.b, bv.b, bout.b, blse.b, bdo.b, bdq.b, bdk.b, bdv.b, bs.b,
                                                       T, B, Hq, Hkv, hd, int(np.diff(ss).max()))
    ctx.check()
    dq1, dk1, dv1 = bdq.numpy(), bdk.numpy(), bdv.numpy()
    assert rel_l2(dq1, dQ_ref) < TOL and rel_l2(dk1, dK_ref) < TOL and rel_l2(dv1, dV_ref) < TOL
    # deterministic: same bits on a second run
    bdk2, bdv2 = ctx.upload(dK0), ctx.upload(dV0)
    ctx.lib.cuda_train_batch_attention_backward_packed(ctx.h, bq.b, bk.b, bv.b, bout.b, blse.b, bdo.b, bdq.b, bdk2.b, bdv2.b, bs.b,
                                                       T, B, Hq, Hkv, hd, int(np.diff(ss).max()))
    assert np.array_equal(bdq.numpy(), dq1) and np.array_equal(bdk2.numpy(), dk1) and np.array_equal(bdv2.numpy(), dv1)
    ctx.set_attn_fused(0)
    ctx.release(bq, bk, bv, bdo, bs, bout, blse, bdq, bdk, bdv, bdk2, bdv2)


@pytest.mark.parametrize("flash", [1, 2, 3, 0, 4])
@pytest.mark.parametrize("ss,Hq,Hkv", [([0, 257], 4, 1), ([0, 1024], 4, 1), ([0, 100, 420, 1000], 4, 2), ([0, 1, 130, 131, 450], 2, 2),
                                       ([0, 2048, 2100], 6, 3), ([0, 33, 700], 2, 2)])
def test_attention_head128_one_kernel_paths(ctx, ss, Hq, Hkv, flash):
    """Head size 128, default GEMM mode.  flash = 1: the forward is one kernel (scores in tensor memory, online
    softmax); the backward keeps dK and dV on chip in one launch over all sequences and K/V heads (P^T and dS^T go back into
    tensor memory as the A operand of the dV and dK products) and leaves only the parts of dS^T for the dQ product.
    flash = 2: the older backward, S, dP, P, dS from one kernel launch per sequence and head group that writes the FP16 parts
    of P and dS for three long products (flash = 3: one such launch for the whole call); flash = 0: a launch per product over
    a score scratch.  All against the oracle, and bit-reproducible."""
    hd = 128
    ss = np.array(ss, np.uint32)
    T, B = int(ss[-1]), len(ss) - 1
    r = rng(T + Hq)
    Q, K, V = f32(r.standard_normal((T, Hq * hd))), f32(r.standard_normal((T, Hkv * hd))), f32(r.standard_normal((T, Hkv * hd)))
    dO = f32(r.standard_normal((T, Hq * hd)))
    out_ref, lse_ref = np.empty_like(Q), np.empty((T, Hq), np.float32)
    O.lib().ref_attention(Q, K, V, out_ref, lse_ref, ss, T, B, Hq, Hkv, hd)
    dQ_ref, dK_ref, dV_ref = np.empty_like(Q), np.zeros_like(K), np.zeros_like(V)
    O.lib().ref_attention_backward(Q, K, V, dO, dQ_ref, dK_ref, dV_ref, ss, T, B, Hq, Hkv, hd)
    bq, bk, bv, bdo, bs = ctx.upload(Q), ctx.upload(K), ctx.upload(V), ctx.upload(dO), ctx.upload(ss)
    ctx.set_attn_flash({1: 3, 2: 2, 3: 2, 0: 0, 4: 1}[flash])      # 4: the library's own choice between 1's and 2's backward
    if flash == 3:                                    # backward scores: one launch per call instead of one per sequence and head group
        os.environ["SERAPH_B200_ATTN_ALL_SCORES_MB"] = "4096"
    runs = []
    for rep in range(2):
        bout, blse = ctx.zeros(Q.size), ctx.zeros(T * Hq)
        bdq, bdk, bdv = ctx.empty(Q.size), ctx.zeros(K.size), ctx.zeros(V.size)
        n0 = ctx.launches()
        ctx.lib.cuda_train_batch_attention_packed(ctx.h, bq.b, bk.b, bv.b, bout.b, blse.b, bs.b, T, B, Hq, Hkv, hd, int(np.diff(ss).max()))
        ctx.check()
        if flash:
            assert ctx.launches() - n0 <= 8      # three operand preparations and the one kernel, not a launch per product
        ctx.lib.cuda_train_batch_attention_backward_packed(ctx.h, bq.b, bk.b, bv.b, bout.b, blse.b, bdo.b, bdq.b, bdk.b, bdv.b, bs.b,
                                                           T, B, Hq, Hkv, hd, int(np.diff(ss).max()))
        ctx.check()
        runs.append([x.numpy() for x in (bout, blse, bdq, bdk, bdv)])
        ctx.release(bout, blse, bdq, bdk, bdv)
    ctx.set_attn_flash(1)
    os.environ.pop("SERAPH_B200_ATTN_ALL_SCORES_MB", None)
    errs = [rel_l2(a, b) for a, b in zip(runs[0], (out_ref, lse_ref, dQ_ref, dK_ref, dV_ref))]
    assert max(errs) < TOL, errs
    assert all(np.array_equal(a, b) for a, b in zip(runs[0], runs[1]))
    ctx.release(bq, bk, bv, bdo, bs)


def test_attention_unpacked_single_sequence(ctx):
    T, Hq, Hkv, hd = 70, 4, 4, 32
    r = rng(70)
    Q, K, V = f32(r.standard_normal((T, Hq * hd))), f32(r.standard_normal((T, Hkv * hd))), f32(r.standard_normal((T, Hkv * hd)))
    ss = np.array([0, T], np.uint32)
    out_ref, lse_ref = np.empty_like(Q), np.empty((T, Hq), np.float32)
    O.lib().ref_attention(Q, K, V, out_ref, lse_ref, ss, T, 1, Hq, Hkv, hd)
    bq, bk, bv, bo = ctx.upload(Q), ctx.upload(K), ctx.upload(V), ctx.empty(Q.size)
    ctx.lib.cuda_train_batch_attention(ctx.h, bq.b, bk.b, bv.b, bo.b, None, T, Hq, Hkv, hd)      # lse_out may be NULL
    assert rel_l2(bo.numpy(), out_ref) < TOL
    ctx.check()
    ctx.release(bq, bk, bv, bo)


@pytest.mark.parametrize("T,H,hd,eps", [(300, 16, 128, 1e-5), (129, 8, 128, 1e-5), (70, 3, 10, 1e-5), (40, 4, 16, 1e-5), (256, 8, 64, 50.0),
                                        (64, 40, 128, 1e-5)])
def test_qk_norm_forward_and_backward(ctx, T, H, hd, eps):
    """Whole-row Q/K normalisation (the reference's qk_norm shader) and its backward against the oracle: warp-per-row and
    CTA-per-row shapes, clamp active (eps = 50), in-place gradient, use_qk_norm = 0 as a no-op."""
    r = rng(T + H + hd)
    x, dy = f32(r.standard_normal((T, H * hd))), f32(r.standard_normal((T, H * hd)))
    y_ref, rms_ref, dx_ref = x.copy(), np.zeros(T, np.float32), np.empty_like(x)
    O.lib().ref_qk_norm(y_ref, rms_ref.ctypes.data, T, H, hd, 1, eps)
    O.lib().ref_qk_norm_backward(y_ref, rms_ref, dy, dx_ref, T, H, hd, 1, eps)
    bx, brms, bdy = ctx.upload(x), ctx.zeros(T), ctx.upload(dy)
    n0 = ctx.launches()
    ctx.lib.seraph_b200_qk_norm(ctx.h, bx.b, brms.b, T, H, hd, 1, eps)
    assert rel_l2(bx.numpy(shape=x.shape), y_ref) < TOL and rel_l2(brms.numpy(), rms_ref) < TOL
    ctx.lib.seraph_b200_qk_norm_backward(ctx.h, bx.b, brms.b, bdy.b, bdy.b, T, H, hd, 1, eps)       # gradient in place
    ctx.check()
    assert ctx.launches() - n0 == 2
    assert rel_l2(bdy.numpy(shape=x.shape), dx_ref) < TOL
    # disabled: nothing happens
    b2 = ctx.upload(x)
    ctx.lib.seraph_b200_qk_norm(ctx.h, b2.b, None, T, H, hd, 0, eps)
    assert np.array_equal(b2.numpy(shape=x.shape), x)
    ctx.release(bx, brms, bdy, b2)


@pytest.mark.parametrize("V", [257, 1024, 8192])
def test_cross_entropy_packed(ctx, V):
    ss = np.array([0, 7, 19, 24], np.uint32)
    T, B = 24, 3
    r = rng(V)
    logits = f32(3 * r.standard_normal((T, V)))
    tgt = r.integers(0, V, T).astype(np.uint32)
    g_ref, rows_ref = np.empty_like(logits), np.empty(T, np.float32)
    O.lib().ref_cross_entropy_grad(logits, tgt, g_ref, rows_ref, ss, T, B, V, T - B)
    bl, bt, bg, br, bs = ctx.upload(logits), ctx.upload(tgt), ctx.empty(logits.size), ctx.empty(T), ctx.upload(ss)
    ctx.lib.cuda_train_cross_entropy_grad_packed(ctx.h, bl.b, bt.b, bg.b, br.b, bs.b, T, B, V, T - B)
    ctx.check()
    g = bg.numpy(shape=(T, V))
    assert rel_l2(g, g_ref) < TOL and rel_l2(br.numpy(), rows_ref) < TOL
    for last in (6, 18, 23):
        assert not g[last].any()
    # unpacked twin: every row predicts, scale 1/rows
    one = np.array([0, T + 1], np.uint32)
    O.lib().ref_cross_entropy_grad(logits, tgt, g_ref, rows_ref, one, T, 1, V, T)
    ctx.lib.cuda_train_cross_entropy_grad(ctx.h, bl.b, bt.b, bg.b, br.b, T, V)
    assert rel_l2(bg.numpy(), g_ref) < TOL and rel_l2(br.numpy(), rows_ref) < TOL
    # loss sum
    bsum = ctx.zeros(4)
    ctx.lib.cuda_train_reduce_sum(ctx.h, br.b, bsum.b, T)
    assert abs(bsum.numpy()[0] - O.lib().ref_reduce_sum(rows_ref, T)) < 1e-4
    ctx.release(bl, bt, bg, br, bs, bsum)


@pytest.mark.parametrize("T,d,V,mode", [(24, 64, 257, "uniform"), (3000, 96, 500, "uniform"), (2048, 512, 8192, "uniform"),
                                        (1500, 64, 257, "one_token"), (1, 8, 5, "uniform")])
def test_embedding_backward_segments_bit_exact(ctx, T, d, V, mode):
    r = rng(T + d)
    tok = (np.zeros(T) if mode == "one_token" else r.integers(0, V, T)).astype(np.uint32)
    g = f32(r.standard_normal((T, d)))
    dE0 = f32(r.standard_normal((V, d)))
    ref = dE0.copy()
    O.lib().ref_embedding_backward(tok, g, ref, T, d)
    bt, bg, bE = ctx.upload(tok), ctx.upload(g), ctx.upload(dE0)
    ctx.lib.cuda_train_embedding_backward(ctx.h, bt.b, bg.b, bE.b, T, d, V)
    ctx.check()
    out = bE.numpy(shape=(V, d))
    assert rel_l2(out, ref) < TOL
    untouched = np.setdiff1d(np.arange(V), tok)
    assert np.array_equal(out[untouched], dE0[untouched])
    rows, counts, spos = np.empty(V, np.int32), np.empty(V, np.int32), np.empty(T, np.int32)
    U = ctx.lib.seraph_b200_embedding_segments(ctx.h, T, V, rows.ctypes.data, counts.ctypes.data, spos.ctypes.data)
    ur, uc = np.unique(tok, return_counts=True)
    assert U == len(ur)
    assert np.array_equal(rows[:U], ur.astype(np.int32)) and np.array_equal(counts[:U], uc.astype(np.int32))
    assert np.array_equal(spos, np.argsort(tok, kind="stable").astype(np.int32))
    bE2 = ctx.upload(dE0)
    ctx.lib.cuda_train_embedding_backward(ctx.h, bt.b, bg.b, bE2.b, T, d, V)
    assert np.array_equal(bE2.numpy(shape=(V, d)), out)
    ctx.release(bt, bg, bE, bE2)


def test_embed_lookup_and_token_range_status(ctx):
    V, d, T = 50, 24, 9
    r = rng(1)
    E = f32(r.standard_normal((V, d)))
    tok = r.integers(0, V, T).astype(np.uint32)
    bt, bE, bo = ctx.upload(tok), ctx.upload(E), ctx.empty(T * d)
    ctx.lib.cuda_train_embed_lookup(ctx.h, bt.b, bE.b, bo.b, T, d, V)
    assert np.array_equal(bo.numpy(shape=(T, d)), E[tok])
    assert ctx.status() == 0
    bad = tok.copy(); bad[2] = V + 3
    bt2 = ctx.upload(bad)
    ctx.lib.cuda_train_embed_lookup(ctx.h, bt2.b, bE.b, bo.b, T, d, V)
    assert ctx.status() == 4          # reported, not faulted
    assert ctx.status() == 0
    ctx.release(bt, bE, bo, bt2)


@pytest.mark.parametrize("n,step", [(1000, 1), (100003, 7)])
def test_adamw(ctx, n, step):
    r = rng(n)
    w, g = f32(r.standard_normal(n)), f32(0.1 * r.standard_normal(n))
    m, v = f32(0.01 * r.standard_normal(n)), f32(0.001 * np.abs(r.standard_normal(n)))
    rw, rm, rv = w.copy(), m.copy(), v.copy()
    O.lib().ref_adamw(rw, g, rm, rv, n, 3.14e-6, 0.9, 0.999, 0.01, 1e-8, step)
    bw, bg, bm, bv = ctx.upload(w), ctx.upload(g), ctx.upload(m), ctx.upload(v)
    ctx.lib.cuda_train_adamw_update(ctx.h, bw.b, bg.b, bm.b, bv.b, 3.14e-6, 0.9, 0.999, 0.01, 1e-8, step, n, b"t", n, 0)
    ctx.check()
    assert rel_l2(bw.numpy(), rw) < 1e-6 and rel_l2(bm.numpy(), rm) < 1e-6 and rel_l2(bv.numpy(), rv) < 1e-6
    ctx.release(bw, bg, bm, bv)


def test_lora_backward(ctx):
    r = rng(4)
    T, i, o, rk, s = 130, 96, 160, 8, 2.0
    A, B = f32(r.standard_normal((rk, i))), f32(r.standard_normal((o, rk)))
    x, dy = f32(r.standard_normal((T, i))), f32(r.standard_normal((T, o)))
    gA, gB, tmp = np.zeros_like(A), np.zeros_like(B), np.zeros((T, rk), np.float32)
    O.lib().ref_lora_backward(dy, x, A, B, gA, gB, tmp, T, i, o, rk, s)
    bA, bB, bx, bdy = ctx.upload(A), ctx.upload(B), ctx.upload(x), ctx.upload(dy)
    bgA, bgB, bt = ctx.zeros(A.size), ctx.zeros(B.size), ctx.empty(T * rk)
    ctx.lib.cuda_train_lora_backward(ctx.h, bdy.b, bx.b, bA.b, bB.b, bgA.b, bgB.b, bt.b, T, i, o, rk, s)
    ctx.check()
    assert rel_l2(bgA.numpy(), gA) < TOL and rel_l2(bgB.numpy(), gB) < TOL
    ctx.release(bA, bB, bx, bdy, bgA, bgB, bt)


def test_nan_check_and_softmax(ctx):
    x = f32(rng(0).standard_normal((6, 50)))
    bx, bo, bf = ctx.upload(x), ctx.empty(x.size), ctx.zeros(8)
    ref = np.empty_like(x)
    O.lib().ref_softmax(x, ref, 6, 50)
    ctx.lib.cuda_train_softmax(ctx.h, bx.b, bo.b, 6, 50)
    assert rel_l2(bo.numpy(), ref) < TOL
    ctx.lib.cuda_train_nan_check(ctx.h, bx.b, x.size, bf.b, 3)
    assert not bf.numpy(np.uint32).any()
    x[2, 5] = np.nan
    bx2 = ctx.upload(x)
    ctx.lib.cuda_train_nan_check(ctx.h, bx2.b, x.size, bf.b, 3)
    assert bf.numpy(np.uint32)[3] == 1
    ctx.release(bx, bo, bf, bx2)
