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
__device__ __forceinline__ uint8_t quantize_block16(const float (&v)[16], uint32_t (&out)[2]) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
    uint16_t sf_pair;
    const float want = __fdiv_rn(amax, 6.0f);
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(sf_pair) : "f"(0.0f), "f"(want));
    uint32_t sf_h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sf_h2) : "h"(sf_pair));
    const float scale = __low2float(*reinterpret_cast<__half2*>(&sf_h2));
    out[0] = 0u;
    out[1] = 0u;
    if (scale > 0.f) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float a = __fdiv_rn(v[2 * j], scale), b = __fdiv_rn(v[2 * j + 1], scale);
            uint32_t byte;
            asm("{\n\t.reg .b8 q;\n\tcvt.rn.satfinite.e2m1x2.f32 q, %1, %2;\n\tcvt.u32.u8 %0, q;\n\t}" : "=r"(byte) : "f"(b), "f"(a));
            out[j >> 2] |= byte << (8 * (j & 3));
        }
    }
    return static_cast<uint8_t>(sf_pair & 0xff);
}

}  // namespace nvfp4
