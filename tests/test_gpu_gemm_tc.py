"""Tensor-core GEMM (tcgen05, TMA, TMEM) against the FP64-accumulate oracle, through the C ABI.
Stated bounds (relative L2 of the whole result, standard-normal operands):
  mode 0, FP32-accurate (three TF32 passes on a hi/lo split):  <= 2e-6   (the FP32 path; whole-model gradients must meet 1e-5)
  mode 1, single-pass TF32:                                    <= 2e-3
  mode 4, FP32-accurate with scaled FP16 hi/lo parts where the layout allows (three FP16 passes): <= 2e-6
Shapes include ragged M/N/K edges (TMA zero fill), all three layouts, accumulate, long K."""
import numpy as np
import pytest

import oracle_lib as O
from oracle_lib import rel_l2

pytestmark = pytest.mark.gpu
BOUND = {0: 2e-6, 1: 2e-3, 4: 2e-6}

SHAPES = [(128, 256, 64), (256, 128, 32), (130, 257, 96), (384, 512, 1024), (100, 200, 4096), (1000, 1000, 40),
          (129, 33, 512), (2048, 64, 256), (300, 300, 64), (257, 512, 160), (512, 384, 2048)]


@pytest.fixture(scope="module")
def ctx():
    from seraph_b200 import api
    c = api.Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("pair", [1, 0])
@pytest.mark.parametrize("mode", [0, 1, 4])
@pytest.mark.parametrize("tA,tB,acc", [(0, 1, 0), (0, 0, 0), (1, 0, 1), (0, 1, 1)])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_tc_gemm_matches_oracle(ctx, M, N, K, tA, tB, acc, mode, pair):
    """pair = 1: tiles of 256 rows on CTA pairs (cta_group::2) where the shape allows; 0: one CTA per tile."""
    if pair and (M <= 128 or N <= 128):
        pytest.skip("shape runs on single CTAs either way")
    r = np.random.default_rng(M + 3 * N + 7 * K + tA + 2 * tB)
    A = r.standard_normal((K, M) if tA else (M, K)).astype(np.float32)
    B = r.standard_normal((N, K) if tB else (K, N)).astype(np.float32)
    C0 = r.standard_normal((M, N)).astype(np.float32)
    ref = C0.copy()
    O.lib().ref_matmul(A, B, ref, M, N, K, tA, tB, acc)
    a, b, c = ctx.upload(A), ctx.upload(B), ctx.upload(C0)
    ctx.set_gemm_mode(mode)
    ctx.set_gemm_pair(pair)
    n0 = ctx.launches()
    ctx.lib.cuda_train_matmul_transpose(ctx.h, a.b, b.b, c.b, M, N, K, tA, tB, acc)
    out = c.numpy(shape=(M, N))
    ctx.set_gemm_mode(4)
    ctx.set_gemm_pair(1)
    ctx.check()
    assert ctx.launches() > n0
    assert rel_l2(out, ref) < BOUND[mode], rel_l2(out, ref)
    ctx.release(a, b, c)


def test_tc_gemm_long_k_and_reproducible(ctx):
    """K = 16384 (longer than the 8192-token reduction of the weight gradients): accumulation error stays in bound."""
    M, N, K = 256, 512, 16384
    r = np.random.default_rng(5)
    A, B = r.standard_normal((M, K)).astype(np.float32), r.standard_normal((N, K)).astype(np.float32)
    ref = np.zeros((M, N), np.float32)
    O.lib().ref_matmul(A, B, ref, M, N, K, 0, 1, 0)
    a, b, c, c2 = ctx.upload(A), ctx.upload(B), ctx.zeros(M * N), ctx.zeros(M * N)
    ctx.lib.cuda_train_matmul_transpose(ctx.h, a.b, b.b, c.b, M, N, K, 0, 1, 0)
    ctx.lib.cuda_train_matmul_transpose(ctx.h, a.b, b.b, c2.b, M, N, K, 0, 1, 0)
    o1, o2 = c.numpy(shape=(M, N)), c2.numpy(shape=(M, N))
    ctx.check()
    e = rel_l2(o1, ref)
    print("FP32-accurate tensor-core GEMM, K=16384: rel-L2 vs FP64 accumulate =", e)
    assert e < 2e-6 and np.array_equal(o1, o2)
    # the same product with whole tiles only (no k pieces in the last wave) meets the same bound
    ctx.set_gemm_tail_split(0)
    ctx.lib.cuda_train_matmul_transpose(ctx.h, a.b, b.b, c2.b, M, N, K, 0, 1, 0)
    o3 = c2.numpy(shape=(M, N))
    ctx.set_gemm_tail_split(1)
    ctx.check()
    assert rel_l2(o3, ref) < 2e-6
    ctx.release(a, b, c, c2)


@pytest.mark.parametrize("mode", [4, 0])
@pytest.mark.parametrize("tA,tB", [(0, 1), (0, 0), (1, 0)])
@pytest.mark.parametrize("M,N,K", [(384, 512, 1024), (130, 257, 96), (1000, 1000, 40), (2048, 2048, 512), (256, 512, 16384),
                                   (4096, 1024, 256), (300, 300, 64), (2049, 6144, 128)])
def test_epilogue_leaves_the_largest_magnitude_of_the_output(ctx, M, N, K, tA, tB, mode):
    """Inside a training step the product's epilogue (and the fix-up pass of tiles whose k range was cut into pieces) leaves
    max |C| behind, and the kernels that write the next operand as FP16 parts scale by bounds formed from it: a value below the
    true maximum would overflow FP16.  The maximum of floats is exact, so it must equal the maximum of the downloaded result,
    with ragged edges, with whole and split tiles, in every layout."""
    import ctypes
    r = np.random.default_rng(11 * M + 5 * N + K + tA + 2 * tB)
    A = r.standard_normal((K, M) if tA else (M, K)).astype(np.float32)
    B = r.standard_normal((N, K) if tB else (K, N)).astype(np.float32)
    A[r.integers(0, A.shape[0]), r.integers(0, A.shape[1])] = 37.0            # one outlier, so that the maximum sits in one tile
    a, b, c = ctx.upload(A), ctx.upload(B), ctx.upload(np.full((M, N), 1e9, np.float32))
    ctx.set_gemm_mode(mode)
    am = ctypes.c_float(-1.0)
    got = ctx.lib.seraph_b200_matmul_amax(ctx.h, a.b, b.b, c.b, M, N, K, tA, tB, ctypes.byref(am))
    out = c.numpy(shape=(M, N))
    ctx.set_gemm_mode(4)
    ctx.check()
    assert got == 1, "shape expected on the tensor-core kernel"
    assert am.value == float(np.abs(out).max()), (am.value, float(np.abs(out).max()))
    ctx.release(a, b, c)
