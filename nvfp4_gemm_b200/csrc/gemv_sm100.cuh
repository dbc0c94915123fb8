// NVFP4 block-scaled GEMV for sm_100a (CUDA cores; the op is HBM-bound, not a dense contraction):
//   c[m, l] = sum_k  e2m1(a[m,k,l]) * sfa[m,k/16,l] * e2m1(b[k,l]) * sfb[k/16,l]
//
// One warp streams R rows; a lane owns 32-byte chunks (64 elements = 4 scale blocks) at a
// stride of 1024 bytes, so every warp-wide 256-bit load covers 1 KiB of contiguous row.  Per
// 16-element block the products are summed in f16x2 (8 terms per half: exact), widened to fp32,
// scaled by sfa*sfb and accumulated in fp32.  The vector and its scales are re-read through L1
// (evict-last) by every row; the matrix streams past L1 with evict-first hints.
//
// Covers the reference's GEMV (old_files/1.py:499-607) but keeps every cross-block add in fp32.
#pragma once
#include "ptx.cuh"

namespace nvfp4 {

constexpr int kGemvThreads = 128;

struct GemvParams {
    const uint8_t* a;    // [L][M][K/2]
    const uint8_t* b;    // [L][1][K/2]
    const uint8_t* sfa;  // plain [L][M][K/16]
    const uint8_t* sfb;  // plain [L][1][K/16]
    __half* c;
    long long a_row_stride, a_batch_stride;      // bytes
    long long b_batch_stride;                    // bytes
    long long sfa_row_stride, sfa_batch_stride;  // bytes
    long long sfb_batch_stride;                  // bytes
    long long c_row_stride, c_batch_stride;      // elements
    int M, K, L;
};

struct Chunk32 {
    uint32_t w[8];
};

__device__ __forceinline__ Chunk32 ld_stream_32B(const uint8_t* ptr) {
    Chunk32 v;
    uint64_t q0, q1, q2, q3;
    asm volatile("ld.global.L1::no_allocate.L2::evict_first.v4.b64 {%0, %1, %2, %3}, [%4];"
                 : "=l"(q0), "=l"(q1), "=l"(q2), "=l"(q3) : "l"(ptr));
    v.w[0] = static_cast<uint32_t>(q0); v.w[1] = static_cast<uint32_t>(q0 >> 32);
    v.w[2] = static_cast<uint32_t>(q1); v.w[3] = static_cast<uint32_t>(q1 >> 32);
    v.w[4] = static_cast<uint32_t>(q2); v.w[5] = static_cast<uint32_t>(q2 >> 32);
    v.w[6] = static_cast<uint32_t>(q3); v.w[7] = static_cast<uint32_t>(q3 >> 32);
    return v;
}
__device__ __forceinline__ Chunk32 ld_keep_32B(const uint8_t* ptr) {
    Chunk32 v;
    uint64_t q0, q1, q2, q3;
    asm volatile("ld.global.L1::evict_last.v4.b64 {%0, %1, %2, %3}, [%4];"
                 : "=l"(q0), "=l"(q1), "=l"(q2), "=l"(q3) : "l"(ptr));
    v.w[0] = static_cast<uint32_t>(q0); v.w[1] = static_cast<uint32_t>(q0 >> 32);
    v.w[2] = static_cast<uint32_t>(q1); v.w[3] = static_cast<uint32_t>(q1 >> 32);
    v.w[4] = static_cast<uint32_t>(q2); v.w[5] = static_cast<uint32_t>(q2 >> 32);
    v.w[6] = static_cast<uint32_t>(q3); v.w[7] = static_cast<uint32_t>(q3 >> 32);
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const uint8_t* ptr) {
    uint32_t v;
    asm volatile("ld.global.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(ptr));
    return v;
}
__device__ __forceinline__ uint32_t ld_keep_u32(const uint8_t* ptr) {
    uint32_t v;
    asm volatile("ld.global.L1::evict_last.u32 %0, [%1];" : "=r"(v) : "l"(ptr));
    return v;
}

// Four bytes = eight e2m1 values -> four f16x2 (low nibble in the low half).
__device__ __forceinline__ void cvt_e2m1x8(uint32_t packed, uint32_t (&h2)[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h2[0]), "=r"(h2[1]), "=r"(h2[2]), "=r"(h2[3]) : "r"(packed));
}
// Four e4m3 scale bytes -> four fp32.
__device__ __forceinline__ void cvt_e4m3x4(uint32_t packed, float (&f)[4]) {
    uint32_t lo, hi;
    asm("{\n\t.reg .b16 s0, s1;\n\t"
        "mov.b32 {s0, s1}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, s0;\n\t"
        "cvt.rn.f16x2.e4m3x2 %1, s1;\n\t}"
        : "=r"(lo), "=r"(hi) : "r"(packed));
    const float2 a = __half22float2(*reinterpret_cast<__half2*>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<__half2*>(&hi));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// A warp's share of R rows: chunks [chunk_begin, chunk_end) of 64 elements, partial sums in fp32.
template <int R, int UNROLL>
__device__ __forceinline__ void gemv_accumulate(const uint8_t* const (&a_ptr)[R], const uint8_t* const (&sfa_ptr)[R], const uint8_t* b_ptr,
                                                const uint8_t* sfb_ptr, int chunk_begin, int chunk_end, int lane, float (&sum)[R]) {
    for (int base = chunk_begin; base < chunk_end; base += 32 * UNROLL) {
        Chunk32 av[UNROLL][R];
        uint32_t sav[UNROLL][R];
        Chunk32 bv[UNROLL];
        uint32_t sbv[UNROLL];
#pragma unroll
        for (int i = 0; i < UNROLL; ++i) {
            const int chunk = base + i * 32 + lane;
            if (chunk < chunk_end) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    av[i][r] = ld_stream_32B(a_ptr[r] + chunk * 32);
                    sav[i][r] = ld_stream_u32(sfa_ptr[r] + chunk * 4);
                }
                bv[i] = ld_keep_32B(b_ptr + chunk * 32);
                sbv[i] = ld_keep_u32(sfb_ptr + chunk * 4);
            }
        }
#pragma unroll
        for (int i = 0; i < UNROLL; ++i) {
            const int chunk = base + i * 32 + lane;
            if (chunk < chunk_end) {
                float sfb_f[4];
                cvt_e4m3x4(sbv[i], sfb_f);
                float sfa_f[R][4];
#pragma unroll
                for (int r = 0; r < R; ++r) cvt_e4m3x4(sav[i][r], sfa_f[r]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {  // one 16-element scale block = two 32-bit words
                    uint32_t b2[8];
                    {
                        uint32_t t[4];
                        cvt_e2m1x8(bv[i].w[2 * j], t);
                        b2[0] = t[0]; b2[1] = t[1]; b2[2] = t[2]; b2[3] = t[3];
                        cvt_e2m1x8(bv[i].w[2 * j + 1], t);
                        b2[4] = t[0]; b2[5] = t[1]; b2[6] = t[2]; b2[7] = t[3];
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        uint32_t a2[8];
                        {
                            uint32_t t[4];
                            cvt_e2m1x8(av[i][r].w[2 * j], t);
                            a2[0] = t[0]; a2[1] = t[1]; a2[2] = t[2]; a2[3] = t[3];
                            cvt_e2m1x8(av[i][r].w[2 * j + 1], t);
                            a2[4] = t[0]; a2[5] = t[1]; a2[6] = t[2]; a2[7] = t[3];
                        }
                        __half2 acc = __float2half2_rn(0.f);
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            acc = __hfma2(*reinterpret_cast<__half2*>(&a2[e]), *reinterpret_cast<__half2*>(&b2[e]), acc);
                        const float2 s = __half22float2(acc);
                        sum[r] = fmaf(s.x + s.y, sfa_f[r][j] * sfb_f[j], sum[r]);
                    }
                }
            }
        }
    }
}

template <int R, int UNROLL = (R == 1) ? 4 : (R == 2 ? 2 : 1)>
__global__ void __launch_bounds__(kGemvThreads) gemv_nvfp4_kernel(const GemvParams p) {
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int l = blockIdx.y;
    const int row0 = (blockIdx.x * (blockDim.x >> 5) + warp) * R;   // 1, 2 or 4 warps per CTA, each on its own rows
    if (row0 >= p.M) return;

    const uint8_t* b_ptr = p.b + l * p.b_batch_stride;
    const uint8_t* sfb_ptr = p.sfb + l * p.sfb_batch_stride;
    const uint8_t* a_ptr[R];
    const uint8_t* sfa_ptr[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = min(row0 + r, p.M - 1);  // clamp: surplus rows recompute the last one and are not stored
        a_ptr[r] = p.a + l * p.a_batch_stride + row * p.a_row_stride;
        sfa_ptr[r] = p.sfa + l * p.sfa_batch_stride + row * p.sfa_row_stride;
    }

    float sum[R];
#pragma unroll
    for (int r = 0; r < R; ++r) sum[r] = 0.f;
    gemv_accumulate<R, UNROLL>(a_ptr, sfa_ptr, b_ptr, sfb_ptr, 0, p.K / 64, lane, sum);

#pragma unroll
    for (int r = 0; r < R; ++r) {
        float v = sum[r];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0 && row0 + r < p.M)
            p.c[l * p.c_batch_stride + static_cast<long long>(row0 + r) * p.c_row_stride] = __float2half_rn(v);
    }
}

}  // namespace nvfp4
