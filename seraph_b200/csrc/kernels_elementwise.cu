// kernels_elementwise.cu - bandwidth-bound elementwise kernels (sm_100a).
// All of them stream float4 with a grid-stride loop over a grid that is a
// multiple of the SM count, so every SM keeps several 16-byte loads in flight.
//
// Reference kernels replaced (src/cuda_train_context.cu): add :1442, silu :1451,
// mul :1462, scale :1471, silu_backward :1744, elementwise_mul_backward :1756,
// rope[_packed] :616/:652, rope_backward[_packed] :1831/:679, embed_lookup :119,
// nan_check :2227.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include "sb_internal.h"

#define EW_THREADS 256

static inline int ew_grid(sb_ctx_t* c, size_t work_items) {
    int sms = c->pub.gpu_sm_count > 0 ? c->pub.gpu_sm_count : 148;
    size_t blocks = (work_items + EW_THREADS - 1) / EW_THREADS;
    size_t cap = (size_t)sms * 8;            // 8 resident CTAs of 256 threads per SM
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// op codes for the generic binary/unary streamers
enum { OP_ADD, OP_MUL, OP_SILU, OP_SILU_BWD, OP_SWIGLU };

template <int OP>
__device__ __forceinline__ float ew_apply(float a, float b) {
    if (OP == OP_ADD) return a + b;
    if (OP == OP_MUL) return a * b;
    if (OP == OP_SILU) return a / (1.0f + expf(-a));
    if (OP == OP_SILU_BWD) { float s = sigmoidf_(a); return b * (s + a * s * (1.0f - s)); }  // a = x, b = dy
    if (OP == OP_SWIGLU) return (a / (1.0f + expf(-a))) * b;                                  // a = gate, b = up
    return 0.f;
}

template <int OP, bool BINARY>
__global__ void __launch_bounds__(EW_THREADS) ew_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                        float* __restrict__ c, size_t n, int vec_ok, unsigned* amax_out) {
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    float am = 0.f;                                       // largest |output| of this thread (asked for by the next GEMM's operand split)
    if (vec_ok) {
        size_t n4 = n >> 2;
        const float4* a4 = (const float4*)a; const float4* b4 = (const float4*)b; float4* c4 = (float4*)c;
        for (size_t i = tid; i < n4; i += nth) {
            float4 x = a4[i], y = BINARY ? b4[i] : x, r;
            r.x = ew_apply<OP>(x.x, y.x); r.y = ew_apply<OP>(x.y, y.y);
            r.z = ew_apply<OP>(x.z, y.z); r.w = ew_apply<OP>(x.w, y.w);
            c4[i] = r;
            am = sb_amax4(am, r);
        }
        for (size_t i = (n4 << 2) + tid; i < n; i += nth) { const float r = ew_apply<OP>(a[i], BINARY ? b[i] : a[i]); c[i] = r; am = fmaxf(am, fabsf(r)); }
    } else {
        for (size_t i = tid; i < n; i += nth) { const float r = ew_apply<OP>(a[i], BINARY ? b[i] : a[i]); c[i] = r; am = fmaxf(am, fabsf(r)); }
    }
    sb_block_amax(am, amax_out);
}

static inline int aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

template <int OP, bool BINARY>
static void ew_launch(sb_ctx_t* c, const float* a, const float* b, float* o, size_t n) {
    if (!n) return;
    int vec = aligned16(a) && aligned16(o) && (!BINARY || aligned16(b));
    int tk = sb_tick_begin(c, OP == OP_SWIGLU ? SB_CLS_SWIGLU : SB_CLS_OTHER);
    ew_kernel<OP, BINARY><<<ew_grid(c, (n + 3) / 4), EW_THREADS, 0, (cudaStream_t)c->pub.stream>>>(a, b, o, n, vec, OP == OP_SWIGLU ? sb_amax_take(c, o, n) : (unsigned*)nullptr);
    sb_tick_end(c, tk, 0.0, (BINARY ? 12.0 : 8.0) * (double)n);
    c->launches++;
}

__global__ void __launch_bounds__(EW_THREADS) scale_kernel(float* x, size_t n, float alpha) {
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    for (size_t i = tid; i < n; i += nth) x[i] *= alpha;
}

// dA = dC*B, dB = dC*A  (three reads, two writes)
__global__ void __launch_bounds__(EW_THREADS) mul_bwd_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                             const float* __restrict__ dC, float* __restrict__ dA,
                                                             float* __restrict__ dB, size_t n) {
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    for (size_t i = tid; i < n; i += nth) { float g = dC[i], a = A[i], b = B[i]; dA[i] = g * b; dB[i] = g * a; }
}

// Fused SwiGLU backward: reads gate, up, dout; writes dgate, dup (20 bytes per element).
//   s = silu(gate); dup = dout*s; dgate = dout*up * silu'(gate)
// which is elementwise_mul_backward followed by silu_backward in the reference
// (src/train_cuda.c:2197-2203) without the intermediate tensors.
__global__ void __launch_bounds__(EW_THREADS) swiglu_bwd_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                                const float* __restrict__ dout, float* __restrict__ dgate,
                                                                float* __restrict__ dup, size_t n, int vec_ok,
                                                                unsigned* amax_dgate, unsigned* amax_dup) {
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    float amg = 0.f, amu = 0.f;
#define SWIGLU_BWD_ONE(g, u, d, dg, du) { float sg = sigmoidf_(g); float si = (g) * sg; \
        float dsl = (d) * (u); du = (d) * si; dg = dsl * (sg + (g) * sg * (1.0f - sg)); }
    if (vec_ok) {
        size_t n4 = n >> 2;
        for (size_t i = tid; i < n4; i += nth) {
            float4 g = ((const float4*)gate)[i], u = ((const float4*)up)[i], d = ((const float4*)dout)[i], dg, du;
            SWIGLU_BWD_ONE(g.x, u.x, d.x, dg.x, du.x) SWIGLU_BWD_ONE(g.y, u.y, d.y, dg.y, du.y)
            SWIGLU_BWD_ONE(g.z, u.z, d.z, dg.z, du.z) SWIGLU_BWD_ONE(g.w, u.w, d.w, dg.w, du.w)
            ((float4*)dgate)[i] = dg; ((float4*)dup)[i] = du;
            amg = sb_amax4(amg, dg); amu = sb_amax4(amu, du);
        }
        for (size_t i = (n4 << 2) + tid; i < n; i += nth) { SWIGLU_BWD_ONE(gate[i], up[i], dout[i], dgate[i], dup[i]) amg = fmaxf(amg, fabsf(dgate[i])); amu = fmaxf(amu, fabsf(dup[i])); }
    } else {
        for (size_t i = tid; i < n; i += nth) { SWIGLU_BWD_ONE(gate[i], up[i], dout[i], dgate[i], dup[i]) amg = fmaxf(amg, fabsf(dgate[i])); amu = fmaxf(amu, fabsf(dup[i])); }
    }
    sb_block_amax(amg, amax_dgate);
    __syncthreads();
    sb_block_amax(amu, amax_dup);
}

// The two SwiGLU kernels with their outputs written only as FP16 operand parts (hi, lo) of the products that read them: the
// scale comes from a bound formed on the device from the largest magnitudes the inputs' producers left behind,
//   |silu(g) u| <= max|g| max|u|,   |dup| = |d silu(g)| <= max|d| max|g|,   |dgate| = |d u silu'(g)| <= 1.1 max|d| max|u|
// (silu' lies in [-0.1, 1.1]).  12 instead of 24 bytes per element forward, 20 instead of 44 backward, counting the split pass
// that no longer runs.
__global__ void __launch_bounds__(EW_THREADS) swiglu_parts_kernel(const float4* __restrict__ gate, const float4* __restrict__ up,
                                                                  uint2* __restrict__ h1, uint2* __restrict__ h2, size_t n4,
                                                                  const float* __restrict__ amax_g, const float* __restrict__ amax_u,
                                                                  float* __restrict__ bound_out) {
    const float bound = fminf(__ldg(amax_g) * __ldg(amax_u), 3.0e38f);
    const float sc = sb_pow2(sb_f16_shift(bound));
    if (blockIdx.x == 0 && threadIdx.x == 0) *bound_out = bound;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 g = gate[i], u = up[i];
        const float r0 = ew_apply<OP_SWIGLU>(g.x, u.x) * sc, r1 = ew_apply<OP_SWIGLU>(g.y, u.y) * sc;
        const float r2 = ew_apply<OP_SWIGLU>(g.z, u.z) * sc, r3 = ew_apply<OP_SWIGLU>(g.w, u.w) * sc;
        uint2 a, b;
        sb_split2(r0, r1, a.x, b.x); sb_split2(r2, r3, a.y, b.y);
        h1[i] = a; h2[i] = b;
    }
}
__global__ void __launch_bounds__(EW_THREADS) swiglu_bwd_parts_kernel(const float4* __restrict__ gate, const float4* __restrict__ up,
                                                                      const float4* __restrict__ dout,
                                                                      uint2* __restrict__ dg1, uint2* __restrict__ dg2,
                                                                      uint2* __restrict__ du1, uint2* __restrict__ du2, size_t n4,
                                                                      const float* __restrict__ amax_g, const float* __restrict__ amax_u,
                                                                      const float* __restrict__ amax_d,
                                                                      float* __restrict__ bound_dg, float* __restrict__ bound_du) {
    const float ad = __ldg(amax_d);
    const float bg = fminf(1.1f * ad * __ldg(amax_u), 3.0e38f), bu = fminf(ad * __ldg(amax_g), 3.0e38f);
    const float sg_ = sb_pow2(sb_f16_shift(bg)), su = sb_pow2(sb_f16_shift(bu));
    if (blockIdx.x == 0 && threadIdx.x == 0) { *bound_dg = bg; *bound_du = bu; }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 g = gate[i], u = up[i], d = dout[i];
        float4 dg, du;
        SWIGLU_BWD_ONE(g.x, u.x, d.x, dg.x, du.x) SWIGLU_BWD_ONE(g.y, u.y, d.y, dg.y, du.y)
        SWIGLU_BWD_ONE(g.z, u.z, d.z, dg.z, du.z) SWIGLU_BWD_ONE(g.w, u.w, d.w, dg.w, du.w)
        uint2 a, b, e, f;
        sb_split2(dg.x * sg_, dg.y * sg_, a.x, b.x); sb_split2(dg.z * sg_, dg.w * sg_, a.y, b.y);
        sb_split2(du.x * su, du.y * su, e.x, f.x); sb_split2(du.z * su, du.w * su, e.y, f.y);
        dg1[i] = a; dg2[i] = b; du1[i] = e; du2[i] = f;
    }
}

// out[t,:] = E[tok[t],:]; one CTA per few rows, float4 when d%4==0.  Token ids
// beyond the table set the status word and read row 0 instead of faulting.
__global__ void __launch_bounds__(EW_THREADS) embed_lookup_kernel(const uint32_t* __restrict__ tok, const float* __restrict__ E,
                                                                  float* __restrict__ out, int T, int d, int V, int vec, int* status) {
    for (int t = blockIdx.x; t < T; t += gridDim.x) {
        uint32_t id = tok[t];
        if (id >= (uint32_t)V) { if (threadIdx.x == 0) atomicExch(status, SB_ERR_TOKEN_RANGE); id = 0; }
        const float* src = E + (size_t)id * d; float* dst = out + (size_t)t * d;
        if (vec) {
            for (int i = threadIdx.x; i < d / 4; i += blockDim.x) ((float4*)dst)[i] = ((const float4*)src)[i];
        } else {
            for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
        }
    }
}

// position of each packed row inside its sequence, and the sequence index
__global__ void seq_index_kernel(const uint32_t* __restrict__ ss, int B, int T, uint32_t* pos_ids, uint32_t* seq_ids) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    int lo = 0, hi = B;
    while (lo < hi) { int mid = (lo + hi) >> 1; if ((int)ss[mid + 1] <= t) lo = mid + 1; else hi = mid; }
    if (lo >= B) lo = B - 1;
    pos_ids[t] = (uint32_t)(t - (int)ss[lo]);
    seq_ids[t] = (uint32_t)lo;
}

// cos/sin table [max_pos, hd/2] built with the same FP32 expression the
// reference evaluates per element: angle = pos * (1/powf(theta, 2p/hd)).
__global__ void rope_table_kernel(float2* tab, int max_pos, int half, int hd, float theta) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= max_pos * half) return;
    int pos = i / half, p = i % half;
    float freq = 1.0f / powf(theta, (float)(p * 2) / hd);
    float ang = pos * freq;
    tab[i] = make_float2(cosf(ang), sinf(ang));
}

// Interleaved-pair rotation, forward or transposed, in one launch over one or two token-major tensors (q with Hq
// heads and, when k is given, k with Hkv heads: a training step rotates both at the same point, and one launch of
// twice the bytes amortises the launch and its tail).  One float4 = two pairs; the two (cos, sin) entries of a
// float4 are one 16-byte table read.  Four float4 per thread are in flight together; indices are 32-bit (the
// launcher takes the pair kernel beyond 2^31 float4).
#define ROPE_UNROLL 4
__global__ void __launch_bounds__(EW_THREADS) rope_kernel(const float* qin, float* qout, const float* kin, float* kout,
                                                          const uint32_t* __restrict__ pos_ids, const float2* __restrict__ tab,
                                                          int T, int Hq, int Hkv, int hd, int backward,
                                                          unsigned* amax_q, unsigned* amax_k) {
    float amq = 0.f, amk = 0.f;
    const uint32_t quads = (uint32_t)hd >> 2, rq = (uint32_t)Hq * quads, rk = kin ? (uint32_t)Hkv * quads : 0u, row_quads = rq + rk;
    const uint32_t total = (uint32_t)T * row_quads;
    const uint32_t nth = gridDim.x * blockDim.x;
    for (uint32_t base = blockIdx.x * blockDim.x + threadIdx.x; base < total; base += nth * ROPE_UNROLL) {
        float4 x[ROPE_UNROLL], cs[ROPE_UNROLL];
        float4* dst[ROPE_UNROLL];
        bool inq[ROPE_UNROLL];
#pragma unroll
        for (int u = 0; u < ROPE_UNROLL; u++) {
            const uint32_t i = base + u * nth;
            dst[u] = nullptr;
            if (i < total) {
                const uint32_t t = i / row_quads, rem = i - t * row_quads;
                const bool isq = rem < rq;
                inq[u] = isq;
                const uint32_t w = isq ? rem : rem - rq;
                x[u] = isq ? ((const float4*)qin)[(size_t)t * rq + w] : ((const float4*)kin)[(size_t)t * rk + w];
                dst[u] = isq ? (float4*)qout + (size_t)t * rq + w : (float4*)kout + (size_t)t * rk + w;
                cs[u] = ((const float4*)tab)[(size_t)pos_ids[t] * quads + w % quads];      // {cos0, sin0, cos1, sin1}
            }
        }
#pragma unroll
        for (int u = 0; u < ROPE_UNROLL; u++) {
            if (dst[u]) {
                float4 r;
                if (!backward) {
                    r.x = x[u].x * cs[u].x - x[u].y * cs[u].y; r.y = x[u].x * cs[u].y + x[u].y * cs[u].x;
                    r.z = x[u].z * cs[u].z - x[u].w * cs[u].w; r.w = x[u].z * cs[u].w + x[u].w * cs[u].z;
                } else {
                    r.x = x[u].x * cs[u].x + x[u].y * cs[u].y; r.y = -x[u].x * cs[u].y + x[u].y * cs[u].x;
                    r.z = x[u].z * cs[u].z + x[u].w * cs[u].w; r.w = -x[u].z * cs[u].w + x[u].w * cs[u].z;
                }
                *dst[u] = r;
                if (inq[u]) amq = sb_amax4(amq, r); else amk = sb_amax4(amk, r);
            }
        }
    }
    sb_block_amax(amq, amax_q);
    __syncthreads();
    sb_block_amax(amk, amax_k);
}

// pair-at-a-time variant for head_dim not divisible by 4 or unaligned buffers
__global__ void rope_pair_kernel(const float* __restrict__ in, float* __restrict__ out, const uint32_t* __restrict__ pos_ids,
                                 const float2* __restrict__ tab, int T, int H, int hd, int backward) {
    int half = hd >> 1;
    size_t total = (size_t)T * H * half;
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    for (size_t i = tid; i < total; i += nth) {
        int p = (int)(i % half); size_t th = i / half; int t = (int)(th / H);
        float2 cs = tab[(size_t)pos_ids[t] * half + p];
        size_t o = th * hd + 2 * p;
        float x0 = in[o], x1 = in[o + 1];
        if (!backward) { out[o] = x0 * cs.x - x1 * cs.y; out[o + 1] = x0 * cs.y + x1 * cs.x; }
        else           { out[o] = x0 * cs.x + x1 * cs.y; out[o + 1] = -x0 * cs.y + x1 * cs.x; }
    }
}

__global__ void __launch_bounds__(EW_THREADS) nan_check_kernel(const float* __restrict__ x, size_t n, uint32_t* flags, uint32_t idx) {
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    bool bad = false;
    for (size_t i = tid; i < n; i += nth) { float v = x[i]; bad |= (isnan(v) || isinf(v)); }
    if (bad) flags[idx] = 1;
}

extern "C" {

void sb_add(sb_ctx_t* c, const float* a, const float* b, float* o, size_t n) { ew_launch<OP_ADD, true>(c, a, b, o, n); }
void sb_mul(sb_ctx_t* c, const float* a, const float* b, float* o, size_t n) { ew_launch<OP_MUL, true>(c, a, b, o, n); }
void sb_silu(sb_ctx_t* c, const float* x, float* y, size_t n) { ew_launch<OP_SILU, false>(c, x, x, y, n); }
void sb_silu_backward(sb_ctx_t* c, const float* x, const float* dy, float* dx, size_t n) { ew_launch<OP_SILU_BWD, true>(c, x, dy, dx, n); }
void sb_swiglu(sb_ctx_t* c, const float* g, const float* u, float* o, size_t n) { sb_parts_invalidate(c, o); ew_launch<OP_SWIGLU, true>(c, g, u, o, n); }

void sb_scale(sb_ctx_t* c, float* a, size_t n, float alpha) {
    if (!n) return;
    scale_kernel<<<ew_grid(c, n), EW_THREADS, 0, (cudaStream_t)c->pub.stream>>>(a, n, alpha);
    c->launches++;
}

void sb_mul_backward(sb_ctx_t* c, const float* A, const float* B, const float* dC, float* dA, float* dB, size_t n) {
    if (!n) return;
    mul_bwd_kernel<<<ew_grid(c, n), EW_THREADS, 0, (cudaStream_t)c->pub.stream>>>(A, B, dC, dA, dB, n);
    c->launches++;
}

void sb_swiglu_backward(sb_ctx_t* c, const float* gate, const float* up, const float* dout, float* dgate, float* dup, size_t n) {
    if (!n) return;
    int vec = aligned16(gate) && aligned16(up) && aligned16(dout) && aligned16(dgate) && aligned16(dup);
    sb_parts_invalidate(c, dgate); sb_parts_invalidate(c, dup);
    int tk = sb_tick_begin(c, SB_CLS_SWIGLU);
    swiglu_bwd_kernel<<<ew_grid(c, (n + 3) / 4), EW_THREADS, 0, (cudaStream_t)c->pub.stream>>>(gate, up, dout, dgate, dup, n, vec,
                                                                                                  sb_amax_take(c, dgate, n), sb_amax_take(c, dup, n));
    sb_tick_end(c, tk, 0.0, 20.0 * (double)n);
    c->launches++;
}

int sb_swiglu_parts(sb_ctx_t* c, const float* gate, const float* up, float* out, size_t n) {
    if (!n || (n & 7) || !aligned16(gate) || !aligned16(up)) return 0;
    float* ag = sb_amax_lookup(c, gate, n); float* au = sb_amax_lookup(c, up, n);
    if (!ag || !au) return 0;
    void* h; float* bound; int fresh;
    if (!sb_parts_find(c, out, n, &h, &bound, &fresh)) return 0;
    sb_amax_forget(c, out);
    int tk = sb_tick_begin(c, SB_CLS_SWIGLU);
    swiglu_parts_kernel<<<ew_grid(c, n / 4), EW_THREADS, 0, (cudaStream_t)c->pub.stream>>>((const float4*)gate, (const float4*)up, (uint2*)h,
                                                                                         (uint2*)((uint16_t*)h + n), n / 4, ag, au, bound);
    sb_tick_end(c, tk, 0.0, 12.0 * (double)n);
    c->launches++;
    return 1;
}
int sb_swiglu_backward_parts(sb_ctx_t* c, const float* gate, const float* up, const float* dout, float* dgate, float* dup, size_t n) {
    if (!n || (n & 7) || !aligned16(gate) || !aligned16(up) || !aligned16(dout)) return 0;
    float* ag = sb_amax_lookup(c, gate, n); float* au = sb_amax_lookup(c, up, n); float* ad = sb_amax_lookup(c, dout, n);
    if (!ag || !au || !ad) return 0;
    void *hg, *hu; float *bg, *bu; int fresh;
    if (!sb_parts_find(c, dgate, n, &hg, &bg, &fresh) || !sb_parts_find(c, dup, n, &hu, &bu, &fresh)) return 0;
    sb_amax_forget(c, dgate); sb_amax_forget(c, dup);
    int tk = sb_tick_begin(c, SB_CLS_SWIGLU);
    swiglu_bwd_parts_kernel<<<ew_grid(c, n / 4), EW_THREADS, 0, (cudaStream_t)c->pub.stream>>>(
        (const float4*)gate, (const float4*)up, (const float4*)dout, (uint2*)hg, (uint2*)((uint16_t*)hg + n), (uint2*)hu, (uint2*)((uint16_t*)hu + n),
        n / 4, ag, au, ad, bg, bu);
    sb_tick_end(c, tk, 0.0, 20.0 * (double)n);
    c->launches++;
    return 1;
}

void sb_embed_lookup(sb_ctx_t* c, const uint32_t* tok, const float* E, float* out, int T, int d, int V) {
    if (T <= 0) return;
    int sms = c->pub.gpu_sm_count > 0 ? c->pub.gpu_sm_count : 148;
    int grid = T < sms * 8 ? T : sms * 8;
    int vec = ((d & 3) == 0) && aligned16(E) && aligned16(out);
    int tk = sb_tick_begin(c, SB_CLS_EMBED);
    embed_lookup_kernel<<<grid, EW_THREADS, 0, (cudaStream_t)c->pub.stream>>>(tok, E, out, T, d, V, vec, c->d_status);
    sb_tick_end(c, tk, 0.0, 8.0 * T * d);
    c->launches++;
}

void sb_seq_index(sb_ctx_t* c, const uint32_t* seq_starts, int B, int T, uint32_t* pos_ids, uint32_t* seq_ids) {
    if (T <= 0) return;
    seq_index_kernel<<<(T + 255) / 256, 256, 0, (cudaStream_t)c->pub.stream>>>(seq_starts, B, T, pos_ids, seq_ids);
    c->launches++;
}

// (re)builds the cos/sin table when the position range, head size or theta changed; false on allocation failure
static bool rope_ensure_table(sb_ctx_t* c, int hd, float theta, int max_pos) {
    const int half = hd / 2;
    if (c->rope_tab && c->rope_tab_pos >= max_pos && c->rope_tab_hd == hd && c->rope_tab_theta == theta) return true;
    cudaStreamSynchronize((cudaStream_t)c->pub.stream);
    if (c->rope_tab) cudaFree(c->rope_tab);
    c->rope_tab = NULL;
    int cap = max_pos < 1024 ? 1024 : max_pos;
    if (sb_check(c, cudaMalloc(&c->rope_tab, (size_t)cap * half * sizeof(float2)), "rope table")) return false;
    c->rope_tab_pos = cap; c->rope_tab_hd = hd; c->rope_tab_theta = theta;
    int n = cap * half;
    rope_table_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)c->pub.stream>>>((float2*)c->rope_tab, cap, half, hd, theta);
    c->launches++;
    return true;
}

void sb_rope(sb_ctx_t* c, const float* in, float* out, const uint32_t* pos_ids, int T, int H, int hd, float theta,
             int max_pos, int backward) {
    if (T <= 0 || H <= 0 || hd < 2) return;
    int half = hd / 2;
    if (!rope_ensure_table(c, hd, theta, max_pos)) return;
    int tk = sb_tick_begin(c, SB_CLS_ROPE);
    if ((hd & 3) == 0 && aligned16(in) && aligned16(out) && aligned16(c->rope_tab) && (double)T * H * (hd / 4) < 2147483648.0) {
        size_t work = ((size_t)T * H * (hd / 4) + ROPE_UNROLL - 1) / ROPE_UNROLL;
        rope_kernel<<<ew_grid(c, work), EW_THREADS, 0, (cudaStream_t)c->pub.stream>>>(in, out, nullptr, nullptr, pos_ids, (const float2*)c->rope_tab, T, H, 0, hd, backward, nullptr, nullptr);
    } else {
        size_t work = (size_t)T * H * half;
        rope_pair_kernel<<<ew_grid(c, work), EW_THREADS, 0, (cudaStream_t)c->pub.stream>>>(in, out, pos_ids, (const float2*)c->rope_tab, T, H, hd, backward);
    }
    sb_tick_end(c, tk, 0.0, 8.0 * T * H * hd);
    c->launches++;
}

// q and k rotated in place by one launch when the fast path applies, else by two calls of sb_rope
void sb_rope2(sb_ctx_t* c, float* q, float* k, const uint32_t* pos_ids, int T, int Hq, int Hkv, int hd, float theta, int max_pos, int backward) {
    if (T <= 0) return;
    const double nq = (double)T * (Hq + Hkv) * (hd / 4);
    if ((hd & 3) || !aligned16(q) || !aligned16(k) || nq >= 2147483648.0) {
        sb_rope(c, q, q, pos_ids, T, Hq, hd, theta, max_pos, backward);
        sb_rope(c, k, k, pos_ids, T, Hkv, hd, theta, max_pos, backward);
        return;
    }
    if (!rope_ensure_table(c, hd, theta, max_pos)) return;
    int tk = sb_tick_begin(c, SB_CLS_ROPE);
    size_t work = ((size_t)nq + ROPE_UNROLL - 1) / ROPE_UNROLL;
    rope_kernel<<<ew_grid(c, work), EW_THREADS, 0, (cudaStream_t)c->pub.stream>>>(q, q, k, k, pos_ids, (const float2*)c->rope_tab, T, Hq, Hkv, hd, backward,
                                                                                   sb_amax_take(c, q, (size_t)T * Hq * hd), sb_amax_take(c, k, (size_t)T * Hkv * hd));
    sb_tick_end(c, tk, 0.0, 8.0 * T * (Hq + Hkv) * hd);
    c->launches++;
}

void sb_nan_check(sb_ctx_t* c, const float* x, size_t n, uint32_t* flags, uint32_t idx) {
    if (!n) return;
    nan_check_kernel<<<ew_grid(c, n), EW_THREADS, 0, (cudaStream_t)c->pub.stream>>>(x, n, flags, idx);
    c->launches++;
}

}  // extern "C"
