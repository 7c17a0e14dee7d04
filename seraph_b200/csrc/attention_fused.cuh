// attention_fused.cuh - pieces shared by the fused attention kernels (attention_fused.cu: forward and backward scores;
// attention_bwd_fused.cu: backward with dK and dV kept on chip): sequence table, TMA / tcgen05 wrappers for FP16 parts,
// tensor-memory loads without an implied wait, FP16 hi/lo packing, the token-major tensor map.
#pragma once
#include "gemm_tc.cuh"

#define AF_BQ 128
#define AF_BKV 64
#define AF_HD 128
#define AF_THREADS 512
#define AF_MAXSEQ 240

struct AfSeqs { int n; int start[AF_MAXSEQ + 1]; };

#define AF_Q_BYTES 65536
#define AF_KV_STAGE 32768
#define AF_OFF_K AF_Q_BYTES
#define AF_OFF_V (AF_OFF_K + 2 * AF_KV_STAGE)
#define AF_OFF_P (AF_OFF_V + 2 * AF_KV_STAGE)
#define AF_OFF_BAR (AF_OFF_P + 32768)
#define AF_SMEM (AF_OFF_BAR + 2048 + 1024)

__device__ __forceinline__ void af_tma_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void af_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void af_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t af_pack_h2(__half a, __half b) {
    return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
}
// tensor-memory load of 32 columns without the wait, and the wait for all loads issued so far; the registers of the loads
// go through the wait as operands so that nothing that reads them is scheduled ahead of it
__device__ __forceinline__ void af_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
#define AF_REGS32(r) "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), \
                     "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), \
                     "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), \
                     "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
__device__ __forceinline__ void af_ld_wait(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : AF_REGS32(r) :: "memory");
}
__device__ __forceinline__ void af_ld_dep(uint32_t (&r)[32]) { asm volatile("" : AF_REGS32(r) :: "memory"); }

__device__ __forceinline__ float af_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
// two values as FP16 parts: hi = the packed roundings of (x0, x1), lo = the packed roundings of what the roundings left
// (what is left, x - hi, is formed by the mixed-precision fma hi * -1 + x: exact, and no conversion of hi back to FP32, which
// shares the slow conversion pipe with the two packed roundings)
__device__ __forceinline__ void af_split2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    asm("{\n\t.reg .b16 h0, h1, m1;\n\t.reg .f32 l0, l1;\n\t"
        "cvt.rn.f16x2.f32 %0, %3, %2;\n\t"
        "mov.b32 {h0, h1}, %0;\n\t"
        "mov.b16 m1, 0xBC00;\n\t"
        "fma.rn.f32.f16 l0, h0, m1, %2;\n\t"
        "fma.rn.f32.f16 l1, h1, m1, %3;\n\t"
        "cvt.rn.f16x2.f32 %1, l1, l0;\n\t}"
        : "=&r"(hi), "=r"(lo) : "f"(x0), "f"(x1));
}

// 4 x 4 transpose of 16-byte chunks among the four lanes of a quad: afterwards w[t] of lane c is what w[c] of lane t was
__device__ __forceinline__ uint4 af_shfl_xor4(uint4 v, int m) {
    v.x = __shfl_xor_sync(0xffffffffu, v.x, m); v.y = __shfl_xor_sync(0xffffffffu, v.y, m);
    v.z = __shfl_xor_sync(0xffffffffu, v.z, m); v.w = __shfl_xor_sync(0xffffffffu, v.w, m);
    return v;
}
__device__ __forceinline__ void af_quad_transpose(uint4 (&w)[4], int lane) {
    const bool hi = (lane & 2) != 0, odd = (lane & 1) != 0;
#pragma unroll
    for (int s2 = 0; s2 < 2; s2++) {
        const uint4 recv = af_shfl_xor4(hi ? w[s2] : w[s2 + 2], 2);
        if (hi) w[s2] = recv; else w[s2 + 2] = recv;
    }
#pragma unroll
    for (int s2 = 0; s2 < 4; s2 += 2) {
        const uint4 recv = af_shfl_xor4(odd ? w[s2] : w[s2 + 1], 1);
        if (odd) w[s2] = recv; else w[s2 + 1] = recv;
    }
}


// 2-D FP16 tensor map over a token-major array [T, cols]: boxes of 64 columns x box_rows tokens, 128-byte swizzle
static inline bool af_make_map(CUtensorMap* m, const void* base, int T, int cols, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)T};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return g_tc_encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

