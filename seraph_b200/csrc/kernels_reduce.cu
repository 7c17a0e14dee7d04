// kernels_reduce.cu - row-reduction and optimizer kernels (sm_100a), all deterministic:
// no floating-point atomics anywhere, so two runs give the same bits.
//
// Reference kernels replaced (src/cuda_train_context.cu): rmsnorm :148,
// rmsnorm_backward :1767 (atomicAdd on grad_scale), softmax :1486,
// cross_entropy_grad[_packed] :1566/:1657, reduce_sum :2209 (atomicAdd),
// embedding_backward :2175 (atomicAdd, blockDim = hidden_size), adamw :2187.
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdio.h>
#include <stdint.h>
#include "sb_internal.h"

#define RB_THREADS 256

static inline int aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }
static inline int sm_count(sb_ctx_t* c) { return c->pub.gpu_sm_count > 0 ? c->pub.gpu_sm_count : 148; }

__device__ __forceinline__ float warp_sum(float v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// block-wide sum of up to two values; every thread gets the result.  red: >= 2*32 floats of smem
__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    a = warp_sum(a); b = warp_sum(b);
    __syncthreads();
    if (lane == 0) { red[w] = a; red[32 + w] = b; }
    __syncthreads();
    float x = 0.f, y = 0.f;
    for (int i = 0; i < nw; i++) { x += red[i]; y += red[32 + i]; }   // fixed order
    a = x; b = y;
}

// ---------------------------------------------------------------------------
// RMSNorm forward: y = x * (1/sqrt(mean(x^2)+eps)) * w.   8 bytes per element + w.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(RB_THREADS) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                             float* __restrict__ y, int rows, int cols, float eps, int vec) {
    __shared__ float red[64];
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xr = x + (size_t)r * cols; float* yr = y + (size_t)r * cols;
        float ss = 0.f, dummy = 0.f;
        if (vec) for (int i = threadIdx.x; i < cols / 4; i += blockDim.x) { float4 v = ((const float4*)xr)[i]; ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
        else     for (int i = threadIdx.x; i < cols; i += blockDim.x) { float v = xr[i]; ss += v * v; }
        block_sum2(ss, dummy, red);
        float inv = 1.0f / sqrtf(ss / cols + eps);
        if (vec) for (int i = threadIdx.x; i < cols / 4; i += blockDim.x) {
            float4 v = ((const float4*)xr)[i], s = ((const float4*)w)[i];
            ((float4*)yr)[i] = make_float4(v.x * inv * s.x, v.y * inv * s.y, v.z * inv * s.z, v.w * inv * s.w);
        } else for (int i = threadIdx.x; i < cols; i += blockDim.x) yr[i] = xr[i] * inv * w[i];
    }
}

// ---------------------------------------------------------------------------
// RMSNorm backward.  Each CTA owns rows r = blockIdx.x, +gridDim.x, ...; it
// writes dx for them (optionally fused with the residual-gradient add) and
// keeps a per-column partial of dscale in registers, stored once to
// partial[blockIdx.x][cols].  A second kernel adds the partials in block
// order into dscale.  Algorithmic traffic: 12 bytes per element (+4 when the
// residual is fused) + cols*4.
// ---------------------------------------------------------------------------
#define RN_MAX_SWEEP 16     // cols <= RB_THREADS*4*RN_MAX_SWEEP = 16384
__global__ void __launch_bounds__(RB_THREADS) rmsnorm_bwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                 const float* __restrict__ dy, const float* __restrict__ resid,
                                                                 float* __restrict__ dx, float* __restrict__ partial,
                                                                 int rows, int cols, float eps, int vec) {
    __shared__ float red[64];
    float acc[RN_MAX_SWEEP * 4];
#pragma unroll
    for (int i = 0; i < RN_MAX_SWEEP * 4; i++) acc[i] = 0.f;
    const int c4 = cols / 4;
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xr = x + (size_t)r * cols; const float* gr = dy + (size_t)r * cols;
        float ss = 0.f, cp = 0.f;
        if (vec) for (int i = threadIdx.x; i < c4; i += blockDim.x) {
            float4 v = ((const float4*)xr)[i], g = ((const float4*)gr)[i], s = ((const float4*)w)[i];
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            cp += g.x * s.x * v.x + g.y * s.y * v.y + g.z * s.z * v.z + g.w * s.w * v.w;
        } else for (int i = threadIdx.x; i < cols; i += blockDim.x) { float v = xr[i]; ss += v * v; cp += gr[i] * w[i] * v; }
        block_sum2(ss, cp, red);
        float inv = 1.0f / sqrtf(ss / cols + eps);
        float k = inv * inv * inv / cols * cp;
        float* dr = dx + (size_t)r * cols; const float* rr = resid ? resid + (size_t)r * cols : nullptr;
        if (vec) {
#pragma unroll
            for (int sw = 0; sw < RN_MAX_SWEEP; sw++) {
                int i = threadIdx.x + sw * RB_THREADS;
                if (i < c4) {
                    float4 v = ((const float4*)xr)[i], g = ((const float4*)gr)[i], s = ((const float4*)w)[i], o;
                    acc[sw * 4 + 0] += g.x * v.x * inv; acc[sw * 4 + 1] += g.y * v.y * inv;
                    acc[sw * 4 + 2] += g.z * v.z * inv; acc[sw * 4 + 3] += g.w * v.w * inv;
                    o.x = g.x * s.x * inv - v.x * k; o.y = g.y * s.y * inv - v.y * k;
                    o.z = g.z * s.z * inv - v.z * k; o.w = g.w * s.w * inv - v.w * k;
                    if (rr) { float4 q = ((const float4*)rr)[i]; o.x += q.x; o.y += q.y; o.z += q.z; o.w += q.w; }
                    ((float4*)dr)[i] = o;
                }
            }
        } else {
#pragma unroll
            for (int sw = 0; sw < RN_MAX_SWEEP * 4; sw++) {
                int i = threadIdx.x + sw * RB_THREADS;
                if (i < cols) {
                    float v = xr[i], g = gr[i];
                    acc[sw] += g * v * inv;
                    float o = g * w[i] * inv - v * k;
                    if (rr) o += rr[i];
                    dr[i] = o;
                }
            }
        }
    }
    float* pr = partial + (size_t)blockIdx.x * cols;
    if (vec) {
#pragma unroll
        for (int sw = 0; sw < RN_MAX_SWEEP; sw++) {
            int i = threadIdx.x + sw * RB_THREADS;
            if (i < c4) ((float4*)pr)[i] = make_float4(acc[sw * 4], acc[sw * 4 + 1], acc[sw * 4 + 2], acc[sw * 4 + 3]);
        }
    } else {
#pragma unroll
        for (int sw = 0; sw < RN_MAX_SWEEP * 4; sw++) { int i = threadIdx.x + sw * RB_THREADS; if (i < cols) pr[i] = acc[sw]; }
    }
}

// ---------------------------------------------------------------------------
// Warp-per-row variants for rows of up to 128*NV floats (cols % 4 == 0): the whole row lives in
// registers, every lane has NV independent 16-byte loads in flight, reductions are warp shuffles
// only, and the row is read from memory exactly once.
// ---------------------------------------------------------------------------
template <int NV>
__global__ void __launch_bounds__(RB_THREADS) rmsnorm_warp_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                  float* __restrict__ y, int rows, int cols, float eps, unsigned* amax_out) {
    const int lane = threadIdx.x & 31, warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    const int c4 = cols >> 2;
    float am = 0.f;
    for (int r = warp; r < rows; r += nwarps) {
        const float4* xr = (const float4*)(x + (size_t)r * cols);
        float4 v[NV];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            int j = lane + 32 * i;
            v[i] = j < c4 ? xr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / cols + eps);
        float4* yr = (float4*)(y + (size_t)r * cols);
#pragma unroll
        for (int i = 0; i < NV; i++) {
            int j = lane + 32 * i;
            if (j < c4) {
                float4 s = ((const float4*)w)[j];
                const float4 o = make_float4(v[i].x * inv * s.x, v[i].y * inv * s.y, v[i].z * inv * s.z, v[i].w * inv * s.w);
                yr[j] = o;
                am = sb_amax4(am, o);
            }
        }
    }
    sb_block_amax(am, amax_out);
}

// Rows of exactly 128 columns (the learned per-head norm: rows = tokens x heads): one float4 per lane, four rows of a warp in
// flight together, so that a warp has 2 KB of loads outstanding instead of 512 bytes.
__global__ void __launch_bounds__(RB_THREADS) rmsnorm_w128_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                                                                  int rows, float eps, unsigned* amax_out) {
    const int lane = threadIdx.x & 31, warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    const float4 s = ((const float4*)w)[lane];
    float am = 0.f;
    for (int r0 = warp * 4; r0 < rows; r0 += nwarps * 4) {
        float4 v[4];
#pragma unroll
        for (int i = 0; i < 4; i++) v[i] = r0 + i < rows ? ((const float4*)x)[(size_t)(r0 + i) * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (r0 + i >= rows) break;
            const float ss = warp_sum(v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w);
            const float inv = 1.0f / sqrtf(ss / 128.f + eps);
            const float4 o = make_float4(v[i].x * inv * s.x, v[i].y * inv * s.y, v[i].z * inv * s.z, v[i].w * inv * s.w);
            ((float4*)y)[(size_t)(r0 + i) * 32 + lane] = o;
            am = sb_amax4(am, o);
        }
    }
    sb_block_amax(am, amax_out);
}

// RMSNorm backward for a 256-thread CTA that visits row groups of RNB_ROWS rows.  Thread t owns the float4 column
// chunks t, t+256, ... (NC of them) of every row the CTA visits, so its dscale partial stays in NC float4
// registers.  The loads of the next group (x, dy, residual) are issued before the current group is reduced,
// so memory requests are in flight during the two CTA-wide reductions (sum x^2 and sum dy*w*x of each row);
// two CTAs share an SM.  One dscale partial row per CTA, summed in CTA order by colsum_partials_kernel.
#define RNB_ROWS 2
template <int NC>
struct RnbSet { float4 v[RNB_ROWS][NC], g[RNB_ROWS][NC], q[RNB_ROWS][NC]; };

template <int NC>
__device__ __forceinline__ void rnb_load(RnbSet<NC>& s, const float* __restrict__ x, const float* __restrict__ dy, const float* resid,
                                         int r0, int rows, int c4) {
#pragma unroll
    for (int rr = 0; rr < RNB_ROWS; rr++)
#pragma unroll
        for (int i = 0; i < NC; i++) {
            const int j = threadIdx.x + RB_THREADS * i;
            const bool in = r0 + rr < rows && j < c4;
            const size_t o = (size_t)(r0 + rr) * c4 + j;
            s.v[rr][i] = in ? ((const float4*)x)[o] : make_float4(0.f, 0.f, 0.f, 0.f);
            s.g[rr][i] = in ? ((const float4*)dy)[o] : make_float4(0.f, 0.f, 0.f, 0.f);
            s.q[rr][i] = (in && resid) ? ((const float4*)resid)[o] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
}

template <int NC>
__device__ __forceinline__ void rnb_compute(const RnbSet<NC>& s, const float4 (&sc)[NC], float4 (&acc)[NC], float* dx, int r0, int rows,
                                            int cols, int c4, float eps, float (*s_red)[2 * RNB_ROWS], float* s_tot, float& am) {
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    float part[2 * RNB_ROWS];
#pragma unroll
    for (int rr = 0; rr < RNB_ROWS; rr++) {
        float ss = 0.f, cp = 0.f;
#pragma unroll
        for (int i = 0; i < NC; i++) {
            const float4 v = s.v[rr][i], g = s.g[rr][i];
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            cp += g.x * sc[i].x * v.x + g.y * sc[i].y * v.y + g.z * sc[i].z * v.z + g.w * sc[i].w * v.w;
        }
        part[2 * rr] = warp_sum(ss); part[2 * rr + 1] = warp_sum(cp);
    }
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 2 * RNB_ROWS; k++) s_red[wib][k] = part[k];
    }
    __syncthreads();
    if (threadIdx.x < 2 * RNB_ROWS) {
        float t = 0.f;
#pragma unroll
        for (int wv = 0; wv < RB_THREADS / 32; wv++) t += s_red[wv][threadIdx.x];
        s_tot[threadIdx.x] = t;
    }
    __syncthreads();
#pragma unroll
    for (int rr = 0; rr < RNB_ROWS; rr++) {
        if (r0 + rr >= rows) break;
        const float inv = 1.0f / sqrtf(s_tot[2 * rr] / cols + eps);
        const float k = inv * inv * inv / cols * s_tot[2 * rr + 1];
#pragma unroll
        for (int i = 0; i < NC; i++) {
            const int j = threadIdx.x + RB_THREADS * i;
            if (j < c4) {
                const float4 v = s.v[rr][i], g = s.g[rr][i], q = s.q[rr][i];
                float4 o;
                acc[i].x += g.x * v.x * inv; acc[i].y += g.y * v.y * inv; acc[i].z += g.z * v.z * inv; acc[i].w += g.w * v.w * inv;
                o.x = g.x * sc[i].x * inv - v.x * k + q.x; o.y = g.y * sc[i].y * inv - v.y * k + q.y;
                o.z = g.z * sc[i].z * inv - v.z * k + q.z; o.w = g.w * sc[i].w * inv - v.w * k + q.w;
                ((float4*)dx)[(size_t)(r0 + rr) * c4 + j] = o;
                am = sb_amax4(am, o);
            }
        }
    }
}

template <int NC>
__global__ void __launch_bounds__(RB_THREADS, 2) rmsnorm_bwd_rows_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                         const float* __restrict__ dy, const float* resid, float* dx,
                                                                         float* __restrict__ partial, int rows, int cols, float eps, unsigned* amax_dx) {
    float am = 0.f;
    __shared__ float s_red[2][RB_THREADS / 32][2 * RNB_ROWS];
    __shared__ float s_tot[2][2 * RNB_ROWS];
    const int c4 = cols >> 2;
    float4 acc[NC], sc[NC];
#pragma unroll
    for (int i = 0; i < NC; i++) {
        acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        const int j = threadIdx.x + RB_THREADS * i;
        sc[i] = j < c4 ? ((const float4*)w)[j] : acc[i];
    }
    const int ngroups = (rows + RNB_ROWS - 1) / RNB_ROWS, stride = gridDim.x;
    RnbSet<NC> a, b;
    int gidx = blockIdx.x;
    if (gidx < ngroups) rnb_load<NC>(a, x, dy, resid, gidx * RNB_ROWS, rows, c4);
    while (gidx < ngroups) {
        if (gidx + stride < ngroups) rnb_load<NC>(b, x, dy, resid, (gidx + stride) * RNB_ROWS, rows, c4);
        rnb_compute<NC>(a, sc, acc, dx, gidx * RNB_ROWS, rows, cols, c4, eps, s_red[0], s_tot[0], am);
        gidx += stride;
        if (gidx >= ngroups) break;
        if (gidx + stride < ngroups) rnb_load<NC>(a, x, dy, resid, (gidx + stride) * RNB_ROWS, rows, c4);
        rnb_compute<NC>(b, sc, acc, dx, gidx * RNB_ROWS, rows, cols, c4, eps, s_red[1], s_tot[1], am);
        gidx += stride;
    }
#pragma unroll
    for (int i = 0; i < NC; i++) {
        const int j = threadIdx.x + RB_THREADS * i;
        if (j < c4) ((float4*)(partial + (size_t)blockIdx.x * cols))[j] = acc[i];
    }
    sb_block_amax(am, amax_dx);
}

// RMSNorm backward for rows of exactly 128 columns (the learned per-head norm of q and k: rows = tokens x heads): one warp per
// row, a float4 per lane, four rows in flight per warp; no CTA-wide reduction per row.  A lane's dscale partial stays in a
// float4 over all rows its warp visits; the warps of a CTA add theirs in warp order into one partial row per CTA.
__global__ void __launch_bounds__(RB_THREADS, 4) rmsnorm_bwd_w128_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                         const float* __restrict__ dy, const float* resid, float* dx,
                                                                         float* __restrict__ partial, int rows, float eps, unsigned* amax_dx) {
    __shared__ float4 s_acc[RB_THREADS / 32][32];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, nw = (gridDim.x * RB_THREADS) >> 5;
    const float4 sc = ((const float4*)w)[lane];
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float am = 0.f;
    for (int r0 = (blockIdx.x * (RB_THREADS / 32) + wib) * 4; r0 < rows; r0 += nw * 4) {
        float4 v[4], g[4], q[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const bool in = r0 + i < rows;
            const size_t o = (size_t)(r0 + i) * 32 + lane;
            v[i] = in ? ((const float4*)x)[o] : make_float4(0.f, 0.f, 0.f, 0.f);
            g[i] = in ? ((const float4*)dy)[o] : make_float4(0.f, 0.f, 0.f, 0.f);
            q[i] = (in && resid) ? ((const float4*)resid)[o] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (r0 + i >= rows) break;
            float ss = v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
            float cp = g[i].x * sc.x * v[i].x + g[i].y * sc.y * v[i].y + g[i].z * sc.z * v[i].z + g[i].w * sc.w * v[i].w;
            ss = warp_sum(ss); cp = warp_sum(cp);
            const float inv = 1.0f / sqrtf(ss / 128.f + eps);
            const float k = inv * inv * inv / 128.f * cp;
            acc.x += g[i].x * v[i].x * inv; acc.y += g[i].y * v[i].y * inv; acc.z += g[i].z * v[i].z * inv; acc.w += g[i].w * v[i].w * inv;
            float4 o;
            o.x = g[i].x * sc.x * inv - v[i].x * k + q[i].x; o.y = g[i].y * sc.y * inv - v[i].y * k + q[i].y;
            o.z = g[i].z * sc.z * inv - v[i].z * k + q[i].z; o.w = g[i].w * sc.w * inv - v[i].w * k + q[i].w;
            ((float4*)dx)[(size_t)(r0 + i) * 32 + lane] = o;
            am = sb_amax4(am, o);
        }
    }
    s_acc[wib][lane] = acc;
    __syncthreads();
    if (wib == 0) {
        float4 t = s_acc[0][lane];
#pragma unroll
        for (int k = 1; k < RB_THREADS / 32; k++) { const float4 u = s_acc[k][lane]; t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w; }
        ((float4*)(partial + (size_t)blockIdx.x * 128))[lane] = t;
    }
    sb_block_amax(am, amax_dx);
}

// dscale[c] += sum over partial rows of partial[b][c], in a fixed order: 32 columns per CTA, the rows dealt to
// 32 row groups (group g takes rows g, g+32, ...; ten independent loads are in flight per thread), the 32 group
// sums then added in group order.
#define CS_GROUPS 32
#define CS_BATCH 10
__global__ void __launch_bounds__(32 * CS_GROUPS) colsum_partials_kernel(const float* __restrict__ partial, float* __restrict__ dscale, int nblocks, int cols) {
    __shared__ float s_part[CS_GROUPS][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int cidx = blockIdx.x * 32 + tx;
    float s = 0.f;
    if (cidx < cols) {
        for (int b0 = ty; b0 < nblocks; b0 += CS_GROUPS * CS_BATCH) {
            float v[CS_BATCH];
#pragma unroll
            for (int i = 0; i < CS_BATCH; i++) {
                const int b = b0 + i * CS_GROUPS;
                v[i] = b < nblocks ? partial[(size_t)b * cols + cidx] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < CS_BATCH; i++) s += v[i];
        }
    }
    s_part[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && cidx < cols) {
        float t = s_part[0][tx];
#pragma unroll
        for (int g = 1; g < CS_GROUPS; g++) t += s_part[g][tx];
        dscale[cidx] += t;
    }
}

// ---------------------------------------------------------------------------
// Row softmax (kept for API completeness; no training step uses it)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(RB_THREADS) softmax_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int cols) {
    __shared__ float red[64];
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xr = x + (size_t)r * cols; float* yr = y + (size_t)r * cols;
        float m = -INFINITY;
        for (int i = threadIdx.x; i < cols; i += blockDim.x) m = fmaxf(m, xr[i]);
        m = warp_max(m);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
        __syncthreads();
        m = -INFINITY;
        for (int i = 0; i < (blockDim.x + 31) / 32; i++) m = fmaxf(m, red[i]);
        float s = 0.f, d0 = 0.f;
        for (int i = threadIdx.x; i < cols; i += blockDim.x) s += expf(xr[i] - m);
        block_sum2(s, d0, red);
        float inv = 1.0f / s;
        for (int i = threadIdx.x; i < cols; i += blockDim.x) yr[i] = expf(xr[i] - m) * inv;
    }
}

// ---------------------------------------------------------------------------
// Q/K normalisation over the whole token row (all heads): y = x / max(sqrt(mean(x^2)), eps), in place
// (shaders/qk_norm.comp:30-76; the CUDA backend of the reference does not have it), and its backward, which the
// reference lacks: r > eps: dx = (dy - y * mean(dy o y)) / r;  clamp active: dx = dy / eps.  The forward keeps r per
// row because it overwrites x.  One warp per row, the row in registers (cols % 4 == 0, cols <= 128 * NV): 8 bytes
// per element forward, 12 backward.  Other shapes: one CTA per row.
// ---------------------------------------------------------------------------
// The same rows with y written only as FP16 operand parts: every |y_i| = |x_i| rstd |w_i| is at most sqrt(cols) max|w| (x_i^2 cannot
// exceed the row's sum of squares), so that bound sets the scale and no pass over y looks for its maximum or splits it again.
template <int NV>
__global__ void __launch_bounds__(RB_THREADS) rmsnorm_warp_parts_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                        uint2* __restrict__ h1, uint2* __restrict__ h2, int rows, int cols, float eps,
                                                                        float* __restrict__ bound_out) {
    const int lane = threadIdx.x & 31, warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    const int c4 = cols >> 2;
    float wm = 0.f;                       // (w is read again from cache in the output loop: keeping it would double the registers)
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const int j = lane + 32 * i;
        if (j < c4) wm = sb_amax4(wm, ((const float4*)w)[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
    const float bound = fminf(sqrtf((float)cols) * wm * 1.0001f, 3.0e38f);
    const float sc = sb_pow2(sb_f16_shift(bound));
    if (warp == 0 && lane == 0) *bound_out = bound;
    for (int r = warp; r < rows; r += nwarps) {
        const float4* xr = (const float4*)(x + (size_t)r * cols);
        float4 v[NV];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            int j = lane + 32 * i;
            v[i] = j < c4 ? xr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / cols + eps);
        uint2* o1 = h1 + (size_t)r * c4; uint2* o2 = h2 + (size_t)r * c4;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            int j = lane + 32 * i;
            if (j < c4) {
                // the FP32 value first, exactly as the plain kernel forms it, then the scale (a power of two: exact)
                const float4 s = ((const float4*)w)[j];
                const float y0 = v[i].x * inv * s.x, y1 = v[i].y * inv * s.y, y2 = v[i].z * inv * s.z, y3 = v[i].w * inv * s.w;
                uint2 a, b;
                sb_split2(y0 * sc, y1 * sc, a.x, b.x); sb_split2(y2 * sc, y3 * sc, a.y, b.y);
                o1[j] = a; o2[j] = b;
            }
        }
    }
}
template <int NV>
__global__ void __launch_bounds__(RB_THREADS) qk_norm_warp_kernel(float* __restrict__ x, float* __restrict__ rms_out, int rows, int cols, float eps) {
    const int lane = threadIdx.x & 31, warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    const int c4 = cols >> 2;
    for (int r = warp; r < rows; r += nwarps) {
        float4* xr = (float4*)(x + (size_t)r * cols);
        float4 v[NV];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int j = lane + 32 * i;
            v[i] = j < c4 ? xr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
        ss = warp_sum(ss);
        const float rms = sqrtf(ss / cols);
        if (lane == 0 && rms_out) rms_out[r] = rms;
        const float inv = 1.0f / fmaxf(rms, eps);
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int j = lane + 32 * i;
            if (j < c4) xr[j] = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
        }
    }
}
template <int NV>
__global__ void __launch_bounds__(RB_THREADS) qk_norm_bwd_warp_kernel(const float* __restrict__ y, const float* __restrict__ rms,
                                                                      const float* dy, float* dx, int rows, int cols, float eps) {
    const int lane = threadIdx.x & 31, warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    const int c4 = cols >> 2;
    for (int r = warp; r < rows; r += nwarps) {
        const float4* yr = (const float4*)(y + (size_t)r * cols);
        const float4* gr = (const float4*)(dy + (size_t)r * cols);
        float4 v[NV], g[NV];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int j = lane + 32 * i;
            v[i] = j < c4 ? yr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            g[i] = j < c4 ? gr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
            dot += v[i].x * g[i].x + v[i].y * g[i].y + v[i].z * g[i].z + v[i].w * g[i].w;
        }
        dot = warp_sum(dot);
        const float rr = rms[r];
        const bool live = rr > eps;
        const float m = live ? dot / cols : 0.f, inv = 1.0f / (live ? rr : eps);
        float4* o = (float4*)(dx + (size_t)r * cols);
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int j = lane + 32 * i;
            if (j < c4) o[j] = make_float4((g[i].x - v[i].x * m) * inv, (g[i].y - v[i].y * m) * inv, (g[i].z - v[i].z * m) * inv, (g[i].w - v[i].w * m) * inv);
        }
    }
}
// any shape: one CTA per row, two passes over the row
__global__ void __launch_bounds__(RB_THREADS) qk_norm_row_kernel(float* __restrict__ x, float* __restrict__ rms_out, const float* __restrict__ rms_in,
                                                                 const float* dy, float* dx, int rows, int cols, float eps) {
    __shared__ float red[RB_THREADS / 32];
    __shared__ float tot;
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        // forward (dy == NULL): sum of x^2; backward: sum of dy*y (x then holds y)
        const float* a = x + (size_t)r * cols; const float* b = dy ? dy + (size_t)r * cols : a;
        float s = 0.f;
        for (int i = threadIdx.x; i < cols; i += blockDim.x) s += a[i] * b[i];
        s = warp_sum(s);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
        __syncthreads();
        if (threadIdx.x == 0) { float t = 0.f; for (int w = 0; w < RB_THREADS / 32; w++) t += red[w]; tot = t; }
        __syncthreads();
        if (!dy) {
            const float rms = sqrtf(tot / cols), inv = 1.0f / fmaxf(rms, eps);
            if (threadIdx.x == 0 && rms_out) rms_out[r] = rms;
            for (int i = threadIdx.x; i < cols; i += blockDim.x) x[(size_t)r * cols + i] = a[i] * inv;
        } else {
            const float rr = rms_in[r];
            const bool live = rr > eps;
            const float m = live ? tot / cols : 0.f, inv = 1.0f / (live ? rr : eps);
            for (int i = threadIdx.x; i < cols; i += blockDim.x) dx[(size_t)r * cols + i] = (b[i] - a[i] * m) * inv;
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// Cross-entropy loss and gradient, packed.  One CTA per row: an online
// (max,sum) pass over the logits, then one pass that writes the gradient:
// 12 bytes per logit where the reference's three passes move 20.
//   last token of a sequence -> zero row and zero loss
//   loss = -(logit[target] - max - log(sum));  grad = (softmax - onehot)/num_valid
// ---------------------------------------------------------------------------
#define CE_THREADS 512
__global__ void __launch_bounds__(CE_THREADS) cross_entropy_kernel(const float* __restrict__ logits, const uint32_t* __restrict__ targets,
                                                                   float* __restrict__ grad, float* __restrict__ loss_rows,
                                                                   const uint32_t* __restrict__ pos_ids, const uint32_t* __restrict__ seq_ids,
                                                                   const uint32_t* __restrict__ seq_starts,
                                                                   int T, int V, float inv_valid, int vec, int* status, unsigned* amax_grad,
                                                                   __half* __restrict__ g1, __half* __restrict__ g2, float part_scale, float* part_amax) {
    // g1 != NULL (vec only): the gradient leaves as the two FP16 parts the LM-head backward products read, h1 = fp16(g * part_scale),
    // h2 = fp16(g * part_scale - h1), laid out like grad; nothing is written to grad.  |g| <= inv_valid everywhere (softmax minus
    // one-hot, over the number of predictions), so the parts' scale is known before a single logit is read: *part_amax = inv_valid.
    __shared__ float redm[32], reds[32];
    float am = 0.f;
    int r = blockIdx.x;
    if (r >= T) return;
    if (g1 && r == 0 && threadIdx.x == 0) *part_amax = inv_valid;
    const float* lr = logits + (size_t)r * V; float* gr = grad + (size_t)r * V;
    uint2* p1 = g1 ? (uint2*)(g1 + (size_t)r * V) : NULL; uint2* p2 = g1 ? (uint2*)(g2 + (size_t)r * V) : NULL;
    uint32_t s = seq_ids[r];
    int seq_len = (int)(seq_starts[s + 1] - seq_starts[s]);
    if ((int)pos_ids[r] >= seq_len - 1) {
        if (g1) for (int i = threadIdx.x; i < V / 4; i += blockDim.x) { p1[i] = make_uint2(0u, 0u); p2[i] = make_uint2(0u, 0u); }
        else if (vec) for (int i = threadIdx.x; i < V / 4; i += blockDim.x) ((float4*)gr)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        else     for (int i = threadIdx.x; i < V; i += blockDim.x) gr[i] = 0.f;
        if (threadIdx.x == 0) loss_rows[r] = 0.f;
        return;
    }
    uint32_t tg = targets[r];
    if (tg >= (uint32_t)V) { if (threadIdx.x == 0) atomicExch(status, SB_ERR_TOKEN_RANGE); tg = 0; }
    float m = -INFINITY, sum = 0.f;
#define CE_ONLINE(v) { float nv = (v); if (nv > m) { sum = sum * expf(m - nv) + 1.0f; m = nv; } else sum += expf(nv - m); }
    if (vec) for (int i = threadIdx.x; i < V / 4; i += blockDim.x) { float4 v = ((const float4*)lr)[i]; CE_ONLINE(v.x) CE_ONLINE(v.y) CE_ONLINE(v.z) CE_ONLINE(v.w) }
    else     for (int i = threadIdx.x; i < V; i += blockDim.x) CE_ONLINE(lr[i])
    // combine (m,sum) pairs: warp, then block
    for (int o = 16; o > 0; o >>= 1) {
        float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, sum, o);
        float nm = fmaxf(m, om);
        sum = (m == -INFINITY ? 0.f : sum * expf(m - nm)) + (om == -INFINITY ? 0.f : os * expf(om - nm));
        m = nm;
    }
    if ((threadIdx.x & 31) == 0) { redm[threadIdx.x >> 5] = m; reds[threadIdx.x >> 5] = sum; }
    __syncthreads();
    m = -INFINITY; sum = 0.f;
    for (int i = 0; i < CE_THREADS / 32; i++) {
        float om = redm[i], os = reds[i], nm = fmaxf(m, om);
        sum = (m == -INFINITY ? 0.f : sum * expf(m - nm)) + (om == -INFINITY ? 0.f : os * expf(om - nm));
        m = nm;
    }
    float inv = 1.0f / sum;
    if (threadIdx.x == 0) loss_rows[r] = -((lr[tg] - m) - logf(sum));
    if (vec) for (int i = threadIdx.x; i < V / 4; i += blockDim.x) {
        float4 v = ((const float4*)lr)[i], g;
        g.x = expf(v.x - m) * inv; g.y = expf(v.y - m) * inv; g.z = expf(v.z - m) * inv; g.w = expf(v.w - m) * inv;
        uint32_t b = (uint32_t)i * 4;
        if (tg - b < 4u) { if (tg == b) g.x -= 1.f; else if (tg == b + 1) g.y -= 1.f; else if (tg == b + 2) g.z -= 1.f; else g.w -= 1.f; }
        g.x *= inv_valid; g.y *= inv_valid; g.z *= inv_valid; g.w *= inv_valid;
        if (g1) {
            const float q0 = g.x * part_scale, q1 = g.y * part_scale, q2 = g.z * part_scale, q3 = g.w * part_scale;
            const __half2 ha = __floats2half2_rn(q0, q1), hb = __floats2half2_rn(q2, q3);
            const float2 fa = __half22float2(ha), fb = __half22float2(hb);
            const __half2 la = __floats2half2_rn(q0 - fa.x, q1 - fa.y), lb = __floats2half2_rn(q2 - fb.x, q3 - fb.y);
            p1[i] = make_uint2(*(const uint32_t*)&ha, *(const uint32_t*)&hb); p2[i] = make_uint2(*(const uint32_t*)&la, *(const uint32_t*)&lb);
        } else {
            ((float4*)gr)[i] = g;
            am = sb_amax4(am, g);
        }
    } else for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float g = expf(lr[i] - m) * inv;
        if ((uint32_t)i == tg) g -= 1.f;
        gr[i] = g * inv_valid;
        am = fmaxf(am, fabsf(g * inv_valid));
    }
    sb_block_amax(am, amax_grad);
}

// ---------------------------------------------------------------------------
// Deterministic sums: fixed grid, fixed per-thread assignment, fixed-order combine.
// ---------------------------------------------------------------------------
template <bool SQUARE>
__global__ void __launch_bounds__(RB_THREADS) partial_sum_kernel(const float* __restrict__ x, size_t n, float* __restrict__ partial, int vec) {
    __shared__ float red[64];
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    float s = 0.f, d0 = 0.f;
    if (vec) {
        size_t n4 = n >> 2;
        for (size_t i = tid; i < n4; i += nth) {
            float4 v = ((const float4*)x)[i];
            s += SQUARE ? (v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w) : (v.x + v.y + v.z + v.w);
        }
        for (size_t i = (n4 << 2) + tid; i < n; i += nth) s += SQUARE ? x[i] * x[i] : x[i];
    } else for (size_t i = tid; i < n; i += nth) s += SQUARE ? x[i] * x[i] : x[i];
    block_sum2(s, d0, red);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void final_sum_kernel(const float* __restrict__ partial, int n, float* out) {
    __shared__ float red[64];
    float s = 0.f, d0 = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
    block_sum2(s, d0, red);
    if (threadIdx.x == 0) out[0] = s;
}

// ---------------------------------------------------------------------------
// Embedding backward as a sorted-segment reduction.
//   1. count_kernel     per-chunk token histograms (integer atomics: exact)
//   2. scan_kernel      bucket starts over the vocabulary, list of rows that occur
//   3. place_kernel     stable position of every token inside its bucket
//   4. segsum_kernel    one CTA per occurring row adds its gradient rows in
//                       ascending token position and does ONE += into dE
// Integer work is exact, the float sums have a fixed order: bit-reproducible.
// Algorithmic bytes: 4*T*d read + 8*U*d (read+write of U touched rows) + 4*T.
// ---------------------------------------------------------------------------
#define EB_CHUNK 1024
__global__ void __launch_bounds__(EB_CHUNK) eb_count_kernel(const uint32_t* __restrict__ tok, int T, int V,
                                                            int* __restrict__ chunk_cnt, int* __restrict__ cnt, int* status) {
    int t = blockIdx.x * EB_CHUNK + threadIdx.x;
    if (t >= T) return;
    uint32_t id = tok[t];
    if (id >= (uint32_t)V) { atomicExch(status, SB_ERR_TOKEN_RANGE); return; }
    atomicAdd(&chunk_cnt[(size_t)blockIdx.x * V + id], 1);
    atomicAdd(&cnt[id], 1);
}

// single CTA: exclusive scan of cnt[V] -> start[V]; compaction of rows with cnt>0 -> rows[], meta[0] = U
__global__ void __launch_bounds__(1024) eb_scan_kernel(const int* __restrict__ cnt, int V, int* __restrict__ start,
                                                       int* __restrict__ rows, int* __restrict__ meta) {
    __shared__ int s_cnt[1024], s_u[1024];
    int per = (V + 1023) / 1024, b = threadIdx.x * per, e = min(b + per, V);
    int c = 0, u = 0;
    for (int i = b; i < e; i++) { int k = cnt[i]; c += k; u += (k > 0); }
    s_cnt[threadIdx.x] = c; s_u[threadIdx.x] = u;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {            // Hillis-Steele inclusive scan
        int vc = 0, vu = 0;
        if ((int)threadIdx.x >= off) { vc = s_cnt[threadIdx.x - off]; vu = s_u[threadIdx.x - off]; }
        __syncthreads();
        s_cnt[threadIdx.x] += vc; s_u[threadIdx.x] += vu;
        __syncthreads();
    }
    int base_c = s_cnt[threadIdx.x] - c, base_u = s_u[threadIdx.x] - u;
    for (int i = b; i < e; i++) {
        int k = cnt[i];
        start[i] = base_c; base_c += k;
        if (k > 0) rows[base_u++] = i;
    }
    if (threadIdx.x == 1023) { meta[0] = s_u[1023]; meta[1] = s_cnt[1023]; }
}

__global__ void __launch_bounds__(EB_CHUNK) eb_place_kernel(const uint32_t* __restrict__ tok, int T, int V,
                                                            const int* __restrict__ chunk_cnt, const int* __restrict__ start,
                                                            int* __restrict__ sorted_pos) {
    __shared__ uint32_t s_tok[EB_CHUNK];
    int t = blockIdx.x * EB_CHUNK + threadIdx.x;
    uint32_t id = t < T ? tok[t] : 0xffffffffu;
    s_tok[threadIdx.x] = id;
    __syncthreads();
    if (t >= T || id >= (uint32_t)V) return;
    int rank = 0;
    for (int cb = 0; cb < (int)blockIdx.x; cb++) rank += chunk_cnt[(size_t)cb * V + id];   // earlier chunks
    for (int j = 0; j < (int)threadIdx.x; j++) rank += (s_tok[j] == id);                   // earlier in this chunk
    sorted_pos[start[id] + rank] = t;
}

__global__ void __launch_bounds__(RB_THREADS) eb_segsum_kernel(const float* __restrict__ g, float* __restrict__ dE,
                                                               const int* __restrict__ rows, const int* __restrict__ start,
                                                               const int* __restrict__ cnt, const int* __restrict__ sorted_pos,
                                                               const int* __restrict__ meta, int d, int vec) {
    int U = meta[0];
    for (int u = blockIdx.x; u < U; u += gridDim.x) {
        int row = rows[u], s0 = start[row], n = cnt[row];
        float* er = dE + (size_t)row * d;
        if (vec) for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < n; j++) { float4 v = ((const float4*)(g + (size_t)sorted_pos[s0 + j] * d))[i]; a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w; }
            float4 e = ((float4*)er)[i]; e.x += a.x; e.y += a.y; e.z += a.z; e.w += a.w; ((float4*)er)[i] = e;
        } else for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float a = 0.f;
            for (int j = 0; j < n; j++) a += g[(size_t)sorted_pos[s0 + j] * d + i];
            er[i] += a;
        }
    }
}

// ---------------------------------------------------------------------------
// AdamW over a flat range: decoupled decay, bias correction (host-computed
// 1-beta^t), optional global-norm clip and data-parallel 1/world folded into
// the gradient read.  28 bytes per parameter.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(RB_THREADS) adamw_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m,
                                                           float* __restrict__ v, size_t n, float lr, float b1, float b2, float wd,
                                                           float eps, float c1, float c2, float grad_scale,
                                                           const float* __restrict__ sumsq, float clip, int vec) {
    float gs = grad_scale;
    if (clip > 0.f && sumsq) {
        float norm = sqrtf(sumsq[0]) * grad_scale;
        if (norm > clip) gs *= clip / (norm + 1e-6f);
    }
    const float decay = 1.0f - lr * wd, ob1 = 1.0f - b1, ob2 = 1.0f - b2;
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
#define ADAMW_ONE(W, G, M, V) { float gi = (G) * gs; float mi = b1 * (M) + ob1 * gi; float vi = b2 * (V) + ob2 * gi * gi; \
        (M) = mi; (V) = vi; float mh = mi / c1, vh = vi / c2; (W) = (W) * decay - lr * mh / (sqrtf(vh) + eps); }
    if (vec) {
        size_t n4 = n >> 2;
        for (size_t i = tid; i < n4; i += nth) {
            float4 W = ((float4*)w)[i], G = ((const float4*)g)[i], M = ((float4*)m)[i], Vv = ((float4*)v)[i];
            ADAMW_ONE(W.x, G.x, M.x, Vv.x) ADAMW_ONE(W.y, G.y, M.y, Vv.y) ADAMW_ONE(W.z, G.z, M.z, Vv.z) ADAMW_ONE(W.w, G.w, M.w, Vv.w)
            ((float4*)w)[i] = W; ((float4*)m)[i] = M; ((float4*)v)[i] = Vv;
        }
        for (size_t i = (n4 << 2) + tid; i < n; i += nth) ADAMW_ONE(w[i], g[i], m[i], v[i])
    } else for (size_t i = tid; i < n; i += nth) ADAMW_ONE(w[i], g[i], m[i], v[i])
}

extern "C" {

void sb_rmsnorm(sb_ctx_t* c, const float* x, const float* w, float* y, int rows, int cols, float eps) {
    if (rows <= 0 || cols <= 0) return;
    sb_parts_invalidate(c, y);
    int grid = rows < sm_count(c) * 8 ? rows : sm_count(c) * 8;
    int vec = (cols % 4 == 0) && aligned16(x) && aligned16(w) && aligned16(y);
    int tk = sb_tick_begin(c, SB_CLS_NORM_FWD);
    if (vec && cols <= 4096 && rows >= 64) {
        // warp per row, 8 warps per CTA, two CTAs resident per SM: every warp gets the same number of rows (no tail)
        int wgrid = (rows + 7) / 8;
        { int cap = sm_count(c) * 2, k = (wgrid + cap - 1) / cap; wgrid = (wgrid + k - 1) / k; }
        cudaStream_t st = (cudaStream_t)c->pub.stream;
        unsigned* am = sb_amax_take(c, y, (size_t)rows * cols);
        if (cols == 128 && rows >= 1024) {
            int g4 = (rows + 31) / 32; if (g4 > sm_count(c) * 4) g4 = sm_count(c) * 4;      // 8 warps x 4 rows per CTA and pass
            rmsnorm_w128_kernel<<<g4, RB_THREADS, 0, st>>>(x, w, y, rows, eps, am);
        } else
        if (cols <= 512)       rmsnorm_warp_kernel<4><<<wgrid, RB_THREADS, 0, st>>>(x, w, y, rows, cols, eps, am);
        else if (cols <= 1024) rmsnorm_warp_kernel<8><<<wgrid, RB_THREADS, 0, st>>>(x, w, y, rows, cols, eps, am);
        else if (cols <= 2048) rmsnorm_warp_kernel<16><<<wgrid, RB_THREADS, 0, st>>>(x, w, y, rows, cols, eps, am);
        else                   rmsnorm_warp_kernel<32><<<wgrid, RB_THREADS, 0, st>>>(x, w, y, rows, cols, eps, am);
    } else
    rmsnorm_kernel<<<grid, RB_THREADS, 0, (cudaStream_t)c->pub.stream>>>(x, w, y, rows, cols, eps, vec);
    sb_tick_end(c, tk, 0.0, 8.0 * rows * cols);
    c->launches++;
}

// y only as the FP16 parts of the registered tensor `y`; 1 = done, 0 = not possible here (call sb_rmsnorm)
int sb_rmsnorm_parts(sb_ctx_t* c, const float* x, const float* w, float* y, int rows, int cols, float eps) {
    if (rows < 64 || cols <= 0 || (cols & 7) || cols > 4096 || !aligned16(x) || !aligned16(w)) return 0;
    void* h; float* bound; int fresh;
    const size_t n = (size_t)rows * cols;
    if (!sb_parts_find(c, y, n, &h, &bound, &fresh)) return 0;
    sb_amax_forget(c, y);
    int wgrid = (rows + 7) / 8;
    { int cap = sm_count(c) * 2, k = (wgrid + cap - 1) / cap; wgrid = (wgrid + k - 1) / k; }
    cudaStream_t st = (cudaStream_t)c->pub.stream;
    uint2* h1 = (uint2*)h; uint2* h2 = (uint2*)((uint16_t*)h + n);
    int tk = sb_tick_begin(c, SB_CLS_NORM_FWD);
    if (cols <= 512)       rmsnorm_warp_parts_kernel<4><<<wgrid, RB_THREADS, 0, st>>>(x, w, h1, h2, rows, cols, eps, bound);
    else if (cols <= 1024) rmsnorm_warp_parts_kernel<8><<<wgrid, RB_THREADS, 0, st>>>(x, w, h1, h2, rows, cols, eps, bound);
    else if (cols <= 2048) rmsnorm_warp_parts_kernel<16><<<wgrid, RB_THREADS, 0, st>>>(x, w, h1, h2, rows, cols, eps, bound);
    else                   rmsnorm_warp_parts_kernel<32><<<wgrid, RB_THREADS, 0, st>>>(x, w, h1, h2, rows, cols, eps, bound);
    sb_tick_end(c, tk, 0.0, 8.0 * rows * cols);
    c->launches++;
    return 1;
}

// number of CTAs the rmsnorm backward uses for `rows` rows (also the row count of its partial buffer)
static int rn_bwd_grid(sb_ctx_t* c, int rows) { int cap = sm_count(c) * 2; return rows < cap ? rows : cap; }

void sb_rmsnorm_backward_with_partials(sb_ctx_t* c, const float* x, const float* w, const float* dy, const float* resid,
                                       float* dx_out, float* dscale, int rows, int cols, float eps, float* partial, int grid) {
    int vec = (cols % 4 == 0) && aligned16(x) && aligned16(w) && aligned16(dy) && aligned16(dx_out) && (!resid || aligned16(resid));
    cudaStream_t s = (cudaStream_t)c->pub.stream;
    int tk = sb_tick_begin(c, SB_CLS_NORM_BWD);
    rmsnorm_bwd_kernel<<<grid, RB_THREADS, 0, s>>>(x, w, dy, resid, dx_out, partial, rows, cols, eps, vec);
    colsum_partials_kernel<<<(cols + 31) / 32, 32 * CS_GROUPS, 0, s>>>(partial, dscale, grid, cols);
    sb_tick_end(c, tk, 0.0, (resid ? 16.0 : 12.0) * rows * cols);
    c->launches += 2;
}

void sb_rmsnorm_backward(sb_ctx_t* c, const float* x, const float* w, const float* dy, const float* resid,
                         float* dx_out, float* dscale, int rows, int cols, float eps) {
    if (rows <= 0 || cols <= 0) return;
    if (cols > RB_THREADS * 4 * RN_MAX_SWEEP || (cols % 4 != 0 && cols > RB_THREADS * RN_MAX_SWEEP * 4)) { sb_set_status(c, SB_ERR_SIZE); return; }
    int vec = (cols % 4 == 0) && aligned16(x) && aligned16(w) && aligned16(dy) && aligned16(dx_out) && (!resid || aligned16(resid));
    if (vec && cols == 128 && rows >= 1024) {
        // many short rows (the per-head norm): a warp per row
        int wgrid = (rows + 31) / 32; if (wgrid > 4 * sm_count(c)) wgrid = 4 * sm_count(c);
        float* partial = (float*)sb_scratch(c, (size_t)wgrid * cols * sizeof(float));
        if (!partial) return;
        cudaStream_t st = (cudaStream_t)c->pub.stream;
        int tk = sb_tick_begin(c, SB_CLS_NORM_BWD);
        unsigned* am = sb_amax_take(c, dx_out, (size_t)rows * cols);
        rmsnorm_bwd_w128_kernel<<<wgrid, RB_THREADS, 0, st>>>(x, w, dy, resid, dx_out, partial, rows, eps, am);
        colsum_partials_kernel<<<(cols + 31) / 32, 32 * CS_GROUPS, 0, st>>>(partial, dscale, wgrid, cols);
        sb_tick_end(c, tk, 0.0, (resid ? 16.0 : 12.0) * rows * cols);
        c->launches += 2;
        return;
    }
    if (vec && cols <= 2048 && rows >= 64) {
        // row groups with the next group's loads in flight, two CTAs per SM; one dscale partial per CTA, summed in CTA order
        int wgrid = (rows + RNB_ROWS - 1) / RNB_ROWS; if (wgrid > 2 * sm_count(c)) wgrid = 2 * sm_count(c);
        float* partial = (float*)sb_scratch(c, (size_t)wgrid * cols * sizeof(float));
        if (!partial) return;
        cudaStream_t st = (cudaStream_t)c->pub.stream;
        int tk = sb_tick_begin(c, SB_CLS_NORM_BWD);
        unsigned* am = sb_amax_take(c, dx_out, (size_t)rows * cols);
        if (cols <= 1024) rmsnorm_bwd_rows_kernel<1><<<wgrid, RB_THREADS, 0, st>>>(x, w, dy, resid, dx_out, partial, rows, cols, eps, am);
        else              rmsnorm_bwd_rows_kernel<2><<<wgrid, RB_THREADS, 0, st>>>(x, w, dy, resid, dx_out, partial, rows, cols, eps, am);
        colsum_partials_kernel<<<(cols + 31) / 32, 32 * CS_GROUPS, 0, st>>>(partial, dscale, wgrid, cols);
        sb_tick_end(c, tk, 0.0, (resid ? 16.0 : 12.0) * rows * cols);
        c->launches += 2;
        return;
    }
    int grid = rn_bwd_grid(c, rows);
    float* partial = (float*)sb_scratch(c, (size_t)grid * cols * sizeof(float));
    if (!partial) return;
    sb_rmsnorm_backward_with_partials(c, x, w, dy, resid, dx_out, dscale, rows, cols, eps, partial, grid);
}

void sb_softmax(sb_ctx_t* c, const float* x, float* y, int rows, int cols) {
    if (rows <= 0 || cols <= 0) return;
    int grid = rows < sm_count(c) * 8 ? rows : sm_count(c) * 8;
    softmax_kernel<<<grid, RB_THREADS, 0, (cudaStream_t)c->pub.stream>>>(x, y, rows, cols);
    c->launches++;
}

static int qk_wgrid(sb_ctx_t* c, int rows) {
    int wgrid = (rows + 7) / 8, cap = sm_count(c) * 2;
    int k = (wgrid + cap - 1) / cap; if (k < 1) k = 1;
    return (wgrid + k - 1) / k;
}
void sb_qk_norm(sb_ctx_t* c, float* x, float* rms_out, int rows, int cols, float eps) {
    if (rows <= 0 || cols <= 0) return;
    cudaStream_t st = (cudaStream_t)c->pub.stream;
    int tk = sb_tick_begin(c, SB_CLS_NORM_FWD);
    if ((cols % 4) == 0 && cols <= 4096 && aligned16(x) && rows >= 64) {
        const int g = qk_wgrid(c, rows);
        if (cols <= 512)       qk_norm_warp_kernel<4><<<g, RB_THREADS, 0, st>>>(x, rms_out, rows, cols, eps);
        else if (cols <= 1024) qk_norm_warp_kernel<8><<<g, RB_THREADS, 0, st>>>(x, rms_out, rows, cols, eps);
        else if (cols <= 2048) qk_norm_warp_kernel<16><<<g, RB_THREADS, 0, st>>>(x, rms_out, rows, cols, eps);
        else                   qk_norm_warp_kernel<32><<<g, RB_THREADS, 0, st>>>(x, rms_out, rows, cols, eps);
    } else {
        int grid = rows < sm_count(c) * 8 ? rows : sm_count(c) * 8;
        qk_norm_row_kernel<<<grid, RB_THREADS, 0, st>>>(x, rms_out, NULL, NULL, NULL, rows, cols, eps);
    }
    sb_tick_end(c, tk, 0.0, 8.0 * rows * cols);
    c->launches++;
}
void sb_qk_norm_backward(sb_ctx_t* c, const float* y, const float* rms, const float* dy, float* dx, int rows, int cols, float eps) {
    if (rows <= 0 || cols <= 0) return;
    cudaStream_t st = (cudaStream_t)c->pub.stream;
    int tk = sb_tick_begin(c, SB_CLS_NORM_BWD);
    if ((cols % 4) == 0 && cols <= 4096 && aligned16(y) && aligned16(dy) && aligned16(dx) && rows >= 64) {
        const int g = qk_wgrid(c, rows);
        if (cols <= 512)       qk_norm_bwd_warp_kernel<4><<<g, RB_THREADS, 0, st>>>(y, rms, dy, dx, rows, cols, eps);
        else if (cols <= 1024) qk_norm_bwd_warp_kernel<8><<<g, RB_THREADS, 0, st>>>(y, rms, dy, dx, rows, cols, eps);
        else if (cols <= 2048) qk_norm_bwd_warp_kernel<16><<<g, RB_THREADS, 0, st>>>(y, rms, dy, dx, rows, cols, eps);
        else                   qk_norm_bwd_warp_kernel<32><<<g, RB_THREADS, 0, st>>>(y, rms, dy, dx, rows, cols, eps);
    } else {
        int grid = rows < sm_count(c) * 8 ? rows : sm_count(c) * 8;
        qk_norm_row_kernel<<<grid, RB_THREADS, 0, st>>>((float*)y, NULL, rms, dy, dx, rows, cols, eps);
    }
    sb_tick_end(c, tk, 0.0, 12.0 * rows * cols);
    c->launches++;
}

void sb_cross_entropy(sb_ctx_t* c, const float* logits, const uint32_t* targets, float* grad, float* loss_rows,
                      const uint32_t* pos_ids, const uint32_t* seq_ids, const uint32_t* seq_starts, int T, int V, int num_valid) {
    if (T <= 0 || V <= 0) return;
    int vec = (V % 4 == 0) && aligned16(logits) && aligned16(grad);
    int tk = sb_tick_begin(c, SB_CLS_CE);
    cross_entropy_kernel<<<T, CE_THREADS, 0, (cudaStream_t)c->pub.stream>>>(logits, targets, grad, loss_rows, pos_ids, seq_ids,
                                                                          seq_starts, T, V, 1.0f / (float)num_valid, vec, c->d_status, sb_amax_take(c, grad, (size_t)T * V),
                                                                          NULL, NULL, 0.f, NULL);
    sb_tick_end(c, tk, 0.0, 12.0 * T * V);
    c->launches++;
}

// The same, with the gradient written only as the FP16 parts of the registered tensor `grad` (its FP32 array is not touched): the
// two LM-head backward products then find their operand prepared and no pass splits 4 T V bytes of gradient again.
// Returns 1 when done, 0 when the parts of `grad` are not available (not registered, cache off, no memory): use sb_cross_entropy.
static __device__ __host__ inline int ce_shift(float amax) {
    int e; frexpf(amax, &e);                       // amax = f * 2^e, f in [0.5, 1): exponent of the leading bit is e - 1
    return 14 - (e - 1);
}
int sb_cross_entropy_parts(sb_ctx_t* c, const float* logits, const uint32_t* targets, float* grad, float* loss_rows,
                           const uint32_t* pos_ids, const uint32_t* seq_ids, const uint32_t* seq_starts, int T, int V, int num_valid) {
    if (T <= 0 || V <= 0 || (V % 4) || !aligned16(logits) || num_valid <= 0) return 0;
    void* h; float* amax; int fresh;
    if (!sb_parts_find(c, grad, (size_t)T * V, &h, &amax, &fresh)) return 0;
    const float inv_valid = 1.0f / (float)num_valid;
    int sh = ce_shift(inv_valid); sh = sh < -100 ? -100 : (sh > 100 ? 100 : sh);      // the rule the products apply to *amax
    const float sc = ldexpf(1.0f, sh);
    int tk = sb_tick_begin(c, SB_CLS_CE);
    cross_entropy_kernel<<<T, CE_THREADS, 0, (cudaStream_t)c->pub.stream>>>(logits, targets, grad, loss_rows, pos_ids, seq_ids, seq_starts, T, V,
                                                                          inv_valid, 1, c->d_status, NULL, (__half*)h, (__half*)h + (size_t)T * V, sc, amax);
    sb_tick_end(c, tk, 0.0, 12.0 * T * V);
    c->launches++;
    return 1;
}

static void sum_impl(sb_ctx_t* c, const float* in, float* out, size_t n, bool square) {
    cudaStream_t s = (cudaStream_t)c->pub.stream;
    if (n == 0) { cudaMemsetAsync(out, 0, sizeof(float), s); return; }
    int grid = sm_count(c) * 4;
    size_t need = (n + RB_THREADS * 4 - 1) / (RB_THREADS * 4);
    if ((size_t)grid > need) grid = (int)need;
    float* partial = (float*)sb_scratch(c, (size_t)grid * sizeof(float));
    if (!partial) return;
    int vec = aligned16(in);
    int tk = sb_tick_begin(c, SB_CLS_OTHER);
    if (square) partial_sum_kernel<true><<<grid, RB_THREADS, 0, s>>>(in, n, partial, vec);
    else        partial_sum_kernel<false><<<grid, RB_THREADS, 0, s>>>(in, n, partial, vec);
    final_sum_kernel<<<1, RB_THREADS, 0, s>>>(partial, grid, out);
    sb_tick_end(c, tk, 0.0, 4.0 * (double)n);
    c->launches += 2;
}
void sb_reduce_sum(sb_ctx_t* c, const float* in, float* out, size_t n) { sum_impl(c, in, out, n, false); }
void sb_sumsq(sb_ctx_t* c, const float* g, size_t n, float* d_out) { sum_impl(c, g, d_out, n, true); }

// Scratch layout of the embedding backward (ints): cnt[V] start[V] rows[V] meta[4] sorted_pos[T] chunk_cnt[nchunk*V]
size_t sb_embedding_scratch_ints(int T, int V) {
    size_t nchunk = ((size_t)T + EB_CHUNK - 1) / EB_CHUNK;
    return 3 * (size_t)V + 4 + (size_t)T + nchunk * (size_t)V;
}

void sb_embedding_backward(sb_ctx_t* c, const uint32_t* tok, const float* g, float* dE, int T, int d, int V) {
    if (T <= 0 || d <= 0 || V <= 0) return;
    cudaStream_t s = (cudaStream_t)c->pub.stream;
    int nchunk = (T + EB_CHUNK - 1) / EB_CHUNK;
    size_t ints = sb_embedding_scratch_ints(T, V);
    int* base = (int*)sb_scratch(c, ints * sizeof(int));
    if (!base) return;
    int *cnt = base, *start = cnt + V, *rows = start + V, *meta = rows + V, *sorted_pos = meta + 4, *chunk_cnt = sorted_pos + T;
    int tk = sb_tick_begin(c, SB_CLS_EMBED);
    cudaMemsetAsync(cnt, 0, (size_t)V * sizeof(int), s);
    cudaMemsetAsync(chunk_cnt, 0, (size_t)nchunk * V * sizeof(int), s);
    eb_count_kernel<<<nchunk, EB_CHUNK, 0, s>>>(tok, T, V, chunk_cnt, cnt, c->d_status);
    eb_scan_kernel<<<1, 1024, 0, s>>>(cnt, V, start, rows, meta);
    eb_place_kernel<<<nchunk, EB_CHUNK, 0, s>>>(tok, T, V, chunk_cnt, start, sorted_pos);
    int grid = T < V ? T : V;
    if (grid > sm_count(c) * 8) grid = sm_count(c) * 8;
    int vec = (d % 4 == 0) && aligned16(g) && aligned16(dE);
    eb_segsum_kernel<<<grid, RB_THREADS, 0, s>>>(g, dE, rows, start, cnt, sorted_pos, meta, d, vec);
    sb_tick_end(c, tk, 0.0, 12.0 * T * d);      // upper bound: every token a distinct row
    c->launches += 4;
}

// copies the segment tables of the last sb_embedding_backward(T, V) to the host:
// rows[U] (ascending), counts[U], sorted_pos[T]; returns U, or -1 on error
int sb_embedding_segments(sb_ctx_t* c, int T, int V, int* rows_out, int* counts_out, int* sorted_pos_out) {
    size_t ints = sb_embedding_scratch_ints(T, V);
    if (!c->scratch || c->scratch_bytes < ints * sizeof(int)) return -1;
    cudaStream_t s = (cudaStream_t)c->pub.stream;
    cudaStreamSynchronize(s);
    int* base = (int*)c->scratch;
    int *cnt = base, *start = cnt + V, *rows = start + V, *meta = rows + V, *sorted_pos = meta + 4;
    int h_meta[4];
    if (cudaMemcpy(h_meta, meta, sizeof h_meta, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    int U = h_meta[0];
    if (U < 0 || U > V) return -1;
    int* h_cnt = (int*)malloc((size_t)V * sizeof(int));
    if (!h_cnt) return -1;
    cudaMemcpy(h_cnt, cnt, (size_t)V * sizeof(int), cudaMemcpyDeviceToHost);
    cudaMemcpy(rows_out, rows, (size_t)U * sizeof(int), cudaMemcpyDeviceToHost);
    cudaMemcpy(sorted_pos_out, sorted_pos, (size_t)T * sizeof(int), cudaMemcpyDeviceToHost);
    for (int i = 0; i < U; i++) counts_out[i] = h_cnt[rows_out[i]];
    free(h_cnt);
    (void)start;
    return U;
}

void sb_adamw(sb_ctx_t* c, float* w, const float* g, float* m, float* v, size_t n, float lr, float b1, float b2,
              float wd, float eps, int step, float grad_scale, const float* d_sumsq, float clip) {
    if (!n) return;
    float c1 = 1.0f - powf(b1, (float)step), c2 = 1.0f - powf(b2, (float)step);
    int vec = aligned16(w) && aligned16(g) && aligned16(m) && aligned16(v);
    size_t need = (n + RB_THREADS * 4 - 1) / (RB_THREADS * 4);
    size_t grid = (size_t)sm_count(c) * 8;
    if (grid > need) grid = need;
    int tk = sb_tick_begin(c, SB_CLS_ADAMW);
    adamw_kernel<<<(int)grid, RB_THREADS, 0, (cudaStream_t)c->pub.stream>>>(w, g, m, v, n, lr, b1, b2, wd, eps, c1, c2,
                                                                         grad_scale, d_sumsq, clip, vec);
    sb_tick_end(c, tk, 0.0, 28.0 * (double)n);
    c->launches++;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate.
//
// Some hosts of this library may not touch the CUDA allocator at the moment
// they need a backward op: code running while a stream capture is open on
// another thread, real-time loops and allocator-owning frameworks that forbid
// cudaMalloc after start-up, and embedders that hand out every byte of device
// memory themselves.  For them the two-stage reduction of dscale keeps its
// per-CTA partial sums in a fixed array that lives in the library image
// instead of in grow-on-demand scratch.
//
// The array belongs to the device that loaded the library and stays resident
// until the process exits: SB_NOALLOC_MAX_CTAS * SB_NOALLOC_MAX_COLS floats
// (296 * 8192 * 4 bytes = 9.7 MB) on every GPU that uses the library.
// ---------------------------------------------------------------------------
#define SB_NOALLOC_MAX_COLS 8192
#define SB_NOALLOC_MAX_CTAS 296          // two CTAs per SM on a 148-SM part
#define SB_NOALLOC_MAX_DEVICES 64

static __device__ __align__(256) float g_rn_static_partials[(size_t)SB_NOALLOC_MAX_CTAS * SB_NOALLOC_MAX_COLS];

// Device address of the array, looked up once per device.  In host code the
// symbol's name is only a handle; the kernels need what cudaGetSymbolAddress
// returns for the device that is current.
static float* g_rn_static_ptr[SB_NOALLOC_MAX_DEVICES];
static int g_rn_static_sms[SB_NOALLOC_MAX_DEVICES];

extern "C" int seraph_b200_rmsnorm_backward_static(const float* input, const float* scale, const float* grad_output,
                                                   float* grad_input, float* grad_scale, int rows, int cols, float eps,
                                                   void* stream) {
    if (!input || !scale || !grad_output || !grad_input || !grad_scale || rows < 0 || cols <= 0) {
        fprintf(stderr, "seraph_b200_rmsnorm_backward_static: NULL pointer or bad shape (rows %d, cols %d)\n", rows, cols);
        return SB_ERR_ARG;
    }
    if (cols > SB_NOALLOC_MAX_COLS) {
        fprintf(stderr, "seraph_b200_rmsnorm_backward_static: cols %d exceeds the fixed scratch (at most %d columns); "
                        "use cuda_train_rmsnorm_backward_batch, which may allocate\n", cols, SB_NOALLOC_MAX_COLS);
        return SB_ERR_SIZE;
    }
    if (rows == 0) return SB_OK;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= SB_NOALLOC_MAX_DEVICES) {
        fprintf(stderr, "seraph_b200_rmsnorm_backward_static: no usable current device\n");
        return SB_ERR_CUDA;
    }
    if (!g_rn_static_ptr[dev]) {
        // first call on this device: resolve the array's device address and the SM count
        float* p = NULL;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_rn_static_partials);
        if (e != cudaSuccess || !p) {
            fprintf(stderr, "seraph_b200_rmsnorm_backward_static: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
            return SB_ERR_CUDA;
        }
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        g_rn_static_sms[dev] = sms;
        g_rn_static_ptr[dev] = p;
    }
    int grid = 2 * g_rn_static_sms[dev];
    if (grid > SB_NOALLOC_MAX_CTAS) grid = SB_NOALLOC_MAX_CTAS;
    if (grid > rows) grid = rows;
    float* partial = g_rn_static_ptr[dev];
    int vec = (cols % 4 == 0) && aligned16(input) && aligned16(scale) && aligned16(grad_output) && aligned16(grad_input);
    cudaStream_t s = (cudaStream_t)stream;
    // every CTA overwrites its whole row of partials before the column sum reads it,
    // so nothing left over from an earlier call is ever read and no clearing is needed
    rmsnorm_bwd_kernel<<<grid, RB_THREADS, 0, s>>>(input, scale, grad_output, nullptr, grad_input, partial, rows, cols, eps, vec);
    colsum_partials_kernel<<<(cols + 31) / 32, 32 * CS_GROUPS, 0, s>>>(partial, grad_scale, grid, cols);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fprintf(stderr, "seraph_b200_rmsnorm_backward_static: launch failed: %s\n", cudaGetErrorString(e));
        return SB_ERR_CUDA;
    }
    return SB_OK;
}
