// gemm_simt.cu - FP32 FMA GEMM on CUDA cores for every shape and layout.
// It serves the shapes the tensor-core path does not take (small or oddly
// sized operands, LoRA rank-sized dimensions) and is the exact-FP32 arithmetic
// mode (SB_GEMM_SIMT).  Semantics follow the reference's matmul_dispatch
// (src/cuda_train_context.cu:2645-2709):
//   tA=0,tB=0  C[M,N] = A[M,K] B[K,N]        tA=1,tB=0  C = A[K,M]^T B[K,N]
//   tA=0,tB=1  C = A[M,K] B[N,K]^T           tA=1,tB=1  treated as tA=0,tB=0
//   acc: C += result.
// 128x128 CTA tile, 16-deep k slab, 8x8 register block per thread.
#include <cuda_runtime.h>
#include <stdint.h>
#include "sb_internal.h"

#define GS_BM 128
#define GS_BN 128
#define GS_BK 16
#define GS_THREADS 256

// element (r, k) of an operand lives at base[r*sr + k*sk]
__device__ __forceinline__ void gs_load_slab(const float* __restrict__ base, long sr, long sk, int r0, int R, int k0, int K,
                                             float* __restrict__ dst /* [GS_BK][128] */) {
    if (sk == 1) {            // k contiguous: 16 consecutive threads walk k
        for (int idx = threadIdx.x; idx < 128 * GS_BK; idx += GS_THREADS) {
            int k = idx & (GS_BK - 1), r = idx >> 4;
            int gr = r0 + r, gk = k0 + k;
            dst[k * 128 + r] = (gr < R && gk < K) ? base[(long)gr * sr + gk] : 0.f;
        }
    } else {                  // rows contiguous
        for (int idx = threadIdx.x; idx < 128 * GS_BK; idx += GS_THREADS) {
            int r = idx & 127, k = idx >> 7;
            int gr = r0 + r, gk = k0 + k;
            dst[k * 128 + r] = (gr < R && gk < K) ? base[(long)gr * sr + (long)gk * sk] : 0.f;
        }
    }
}

__global__ void __launch_bounds__(GS_THREADS) gemm_simt_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                               float* __restrict__ C, int M, int N, int K,
                                                               long sam, long sak, long sbn, long sbk, int acc) {
    __shared__ __align__(16) float As[GS_BK * GS_BM];
    __shared__ __align__(16) float Bs[GS_BK * GS_BN];
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float c[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++) for (int j = 0; j < 8; j++) c[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += GS_BK) {
        __syncthreads();
        gs_load_slab(A, sam, sak, m0, M, k0, K, As);
        gs_load_slab(B, sbn, sbk, n0, N, k0, K, Bs);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GS_BK; k++) {
            float4 a0 = *(const float4*)(As + k * GS_BM + ty * 4), a1 = *(const float4*)(As + k * GS_BM + 64 + ty * 4);
            float4 b0 = *(const float4*)(Bs + k * GS_BN + tx * 4), b1 = *(const float4*)(Bs + k * GS_BN + 64 + tx * 4);
            float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) c[i][j] += a[i] * b[j];
        }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
            if (n >= N) continue;
            size_t o = (size_t)m * N + n;
            C[o] = acc ? C[o] + c[i][j] : c[i][j];
        }
    }
}

extern "C" void sb_gemm_simt(sb_ctx_t* c, const float* A, const float* B, float* C, int M, int N, int K, int tA, int tB, int acc) {
    if (M <= 0 || N <= 0) return;
    long sam, sak, sbn, sbk;
    if (tA && !tB)      { sam = 1; sak = M; sbk = N; sbn = 1; }
    else if (!tA && tB) { sam = K; sak = 1; sbk = 1; sbn = K; }
    else                { sam = K; sak = 1; sbk = N; sbn = 1; }
    dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM);
    gemm_simt_kernel<<<grid, GS_THREADS, 0, (cudaStream_t)c->pub.stream>>>(A, B, C, M, N, K, sam, sak, sbn, sbk, acc);
    c->launches++;
}
