// The NVFP4 rounding rule, shared by the stand-alone quantiser (layout_kernels.cuh) and the GEMM's
// re-quantising epilogue (gemm_sm100.cuh) so that the two produce the same bytes.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nvfp4 {

// One 16-element block -> eight bytes of e2m1 codes (out[0], out[1]; low nibble = lower index) and
// the block's e4m3 scale byte: scale = RN-even saturating e4m3 of max|v| / 6, element =
// RN-even saturating e2m1 of v / scale (all zero when the scale is zero).
//
// The inputs must be fp16- or bf16-representable (both callers convert from those types).  Then
// v / scale need not be an IEEE division: q = v * r corrected once by the exact residual
// (v - q * scale) * r, with r within two ulp of 1 / scale, lands exactly on every e2m1 rounding
// threshold that the true quotient hits, and everywhere else the quotient is at least 2^-11 away
// (relatively) from a threshold because v has at most 11 significant bits and threshold * scale at
// most 7.  Checked exhaustively on the CPU over every fp16 and bf16 value and every e4m3 scale.
// Values beyond +-65504 (bf16 inputs, infinities) are clamped there first: the scale is then 448 and
// the element saturates either way, while an infinity would poison the residual.
// Eight bytes of e2m1 codes of v[0..15] / scale, scale > 0 an e4m3 value and |v| <= 65504.
__device__ __forceinline__ void encode_block16(const float (&v)[16], float scale, uint32_t (&out)[2]) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(scale));
    float q[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float a = v[j] * r;
        q[j] = copysignf(fmaf(fmaf(-a, scale, v[j]), r, a), v[j]);   // the sign only differs for -0 (its residual is +0)
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)   // four code bytes at a time (low nibble = lower index), packed by one move
        asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
            "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
            "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
            "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
            "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
            "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
            : "=r"(out[h])
            : "f"(q[8 * h]), "f"(q[8 * h + 1]), "f"(q[8 * h + 2]), "f"(q[8 * h + 3]), "f"(q[8 * h + 4]), "f"(q[8 * h + 5]), "f"(q[8 * h + 6]),
              "f"(q[8 * h + 7]));
}

__device__ __forceinline__ uint8_t quantize_block16(const float (&v)[16], uint32_t (&out)[2]) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
    uint16_t sf_pair;
    // max|v| / 6 as a product with RN(1/6): the e4m3 rounding of the product equals that of the
    // exact quotient for every fp16 and bf16 value of max|v| (checked exhaustively on the CPU).
    const float want = amax * (1.0f / 6.0f);
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(sf_pair) : "f"(0.0f), "f"(want));
    uint32_t sf_h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sf_h2) : "h"(sf_pair));
    const float scale = __low2float(*reinterpret_cast<__half2*>(&sf_h2));
    out[0] = 0u;
    out[1] = 0u;
    if (scale > 0.f) {
        if (amax <= 65504.f) {
            encode_block16(v, scale, out);
        } else {
            float w[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) w[j] = fminf(fmaxf(v[j], -65504.f), 65504.f);
            encode_block16(w, scale, out);
        }
    }
    return static_cast<uint8_t>(sf_pair & 0xff);
}

}  // namespace nvfp4
