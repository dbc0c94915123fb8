// Data-movement kernels beside the matmul path (HBM-bound, 16-byte vector accesses):
//   * interleave_column_blocks: [g][rows][n_local] fp16 (what an all-gather of per-rank column
//     blocks leaves in memory) -> row-major [rows][g * n_local];
//   * permute_scales: plain [rows][K/16] scale bytes -> the 512-byte atom layout the tensor-core
//     GEMM reads (ref.txt:31, s_128t.py:554-562 in the reference project); scales_from_permuted:
//     the way back, or a comparison of the two forms;
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "quantize.cuh"

namespace nvfp4 {

// One thread moves 16 bytes (8 fp16).  n_local is a multiple of 8.
__global__ void __launch_bounds__(256) interleave_column_blocks_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                                      long long rows, int vec_per_block_row, int g,
                                                                      long long dst_row_stride_vec) {
    const long long per_row = static_cast<long long>(vec_per_block_row) * g;
    const long long total = rows * per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long row = i / per_row;
        const int in_row = static_cast<int>(i - row * per_row);
        const int blk = in_row / vec_per_block_row;
        const int v = in_row - blk * vec_per_block_row;
        const uint4 val = __ldcs(src + (static_cast<long long>(blk) * rows + row) * vec_per_block_row + v);
        dst[row * dst_row_stride_vec + in_row] = val;
    }
}

// All-gather by a copy kernel: rows [row0, row0 + rows) of up to seven column blocks go from
// src[i] to dst[i] (same offsets inside row-major matrices of one row stride).  Either side may be
// peer-mapped memory of another GPU.  16 bytes per thread and access, a warp reads and writes 512
// contiguous bytes of one row.
__device__ __forceinline__ uint4 ld_nc_na_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
struct BlockCopyParams {
    const uint4* src[7];   // source matrix base + the block's column offset
    uint4* dst[7];         // destination matrix base + the same offset
    int n_src;
};
__global__ void __launch_bounds__(256) copy_column_blocks_kernel(const BlockCopyParams pp, long long row0, unsigned rows, unsigned vec_per_row,
                                                                 long long row_stride_vec) {
    // Loads over NVLink have a round trip of microseconds: every thread keeps kInFlight of them
    // outstanding before its first store.
    constexpr int kInFlight = 8;
    const unsigned per_src = rows * vec_per_row;
    const unsigned total = per_src * static_cast<unsigned>(pp.n_src);
    const unsigned chunk = blockDim.x * kInFlight;
    for (unsigned base = blockIdx.x * chunk; base < total; base += gridDim.x * chunk) {
        uint4 v[kInFlight];
        long long off[kInFlight];
        int src[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const unsigned i = base + u * blockDim.x + threadIdx.x;
            src[u] = -1;
            if (i < total) {
                const unsigned s = i / per_src;
                const unsigned rem = i - s * per_src;
                const unsigned row = rem / vec_per_row;
                src[u] = static_cast<int>(s);
                off[u] = (row0 + row) * row_stride_vec + (rem - row * vec_per_row);
                v[u] = ld_nc_na_v4(pp.src[s] + off[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u)
            if (src[u] >= 0) pp.dst[src[u]][off[u]] = v[u];
    }
}

// One thread produces 16 bytes of an atom: the four scales of rows {r32 + 32*j, j = 0..3}... laid
// out as [r32][j][k4]; it reads four 4-byte words (one per 32-row group) from the plain layout.
__global__ void __launch_bounds__(256) permute_scales_kernel(const uint8_t* __restrict__ plain, uint8_t* __restrict__ perm,
                                                             int rows, int sf_cols, long long plain_row_stride,
                                                             long long plain_batch_stride, long long perm_batch_stride,
                                                             int batches) {
    const int atoms_k = sf_cols / 4;
    const int row_blocks = (rows + 127) / 128;
    const long long per_batch = static_cast<long long>(row_blocks) * atoms_k * 32;  // 16-byte pieces
    const long long total = per_batch * batches;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int l = static_cast<int>(i / per_batch);
        long long rem = i - l * per_batch;
        const int r32 = static_cast<int>(rem % 32);
        rem /= 32;
        const int kk = static_cast<int>(rem % atoms_k);
        const int rb = static_cast<int>(rem / atoms_k);
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int row = rb * 128 + j * 32 + r32;
            w[j] = (row < rows) ? *reinterpret_cast<const uint32_t*>(plain + l * plain_batch_stride + row * plain_row_stride + kk * 4)
                                : 0u;
        }
        *reinterpret_cast<uint4*>(perm + l * perm_batch_stride + (static_cast<long long>(rb) * atoms_k + kk) * 512 + r32 * 16) =
            make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// The way back, and the check that the two scale tensors an operator call carries say the same
// (the reference's kernels silently trust whichever form they read, template.py:11-14): one
// thread takes 16 bytes of an atom (four rows x four scales) and either writes the four words to
// the plain layout or compares them with it.  result[0] counts differing scale bytes, result[1]
// keeps the smallest (l, row, scale column) linear index of one; padding rows are not looked at.
template <bool COMPARE>
__global__ void __launch_bounds__(256) scales_from_permuted_kernel(const uint8_t* __restrict__ perm, uint8_t* __restrict__ plain,
                                                                   int rows, int sf_cols, long long plain_row_stride,
                                                                   long long plain_batch_stride, long long perm_batch_stride,
                                                                   int batches, unsigned long long* __restrict__ result) {
    const int atoms_k = sf_cols / 4;
    const int row_blocks = (rows + 127) / 128;
    const long long per_batch = static_cast<long long>(row_blocks) * atoms_k * 32;
    const long long total = per_batch * batches;
    unsigned long long bad = 0, first = ~0ull;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int l = static_cast<int>(i / per_batch);
        long long rem = i - l * per_batch;
        const int r32 = static_cast<int>(rem % 32);
        rem /= 32;
        const int kk = static_cast<int>(rem % atoms_k);
        const int rb = static_cast<int>(rem / atoms_k);
        const uint4 v = *reinterpret_cast<const uint4*>(perm + l * perm_batch_stride + (static_cast<long long>(rb) * atoms_k + kk) * 512 + r32 * 16);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int row = rb * 128 + j * 32 + r32;
            if (row >= rows) continue;
            uint32_t* word = reinterpret_cast<uint32_t*>(plain + l * plain_batch_stride + row * plain_row_stride + kk * 4);
            if (!COMPARE) {
                *word = w[j];
            } else {
                uint32_t diff = *word ^ w[j];
                if (diff) {
                    const unsigned long long base = (static_cast<unsigned long long>(l) * rows + row) * sf_cols + kk * 4;
                    const int first_byte = (__ffs(diff) - 1) / 8;
                    if (base + first_byte < first) first = base + first_byte;
                    for (int b = 0; b < 4; ++b, diff >>= 8) bad += (diff & 0xFFu) ? 1 : 0;
                }
            }
        }
    }
    if (COMPARE && bad) {
        atomicAdd(result, bad);
        atomicMin(result + 1, first);
    }
}

// NVFP4 quantiser (the step before the matmul): fp16 / bf16 [rows][K] -> packed e2m1 + one e4m3
// scale per 16 elements, scale = RN(max|x| / 6), element = RN(x / scale) saturated to +-6.
// Work unit: 128 rows x 256 columns (one row block of the permuted scale layout x 4 of its atoms),
// taken in turn by a grid of resident CTAs of 256 threads.  A thread owns 64 consecutive elements of
// a row = four scale blocks = one 4-byte unit of both scale layouts: 128 bytes in (eight 16-byte
// loads, all in flight before the first block is worked on; four neighbouring threads cover 512
// bytes of a row), 32 bytes of codes and the 4-byte word of plain scales out.  The permuted scales
// of the unit -- 4 atoms of 512 bytes, contiguous in memory -- are collected in shared memory and
// written as whole 16-byte pieces (written from the threads' rows they would be 4-byte pieces
// scattered over the atoms: 10 % of the run time); rows of the block that do not exist are written
// as zero scales.
// kWide: every output address is aligned for the wide stores (16 bytes for the codes and the
// permuted scales, 4 bytes for the plain scale words); otherwise 8-byte and single-byte stores.
constexpr int kQuantGroups = 4;   // 64-element groups (= scale atoms) along K per work unit
template <bool BF16, bool kWide>
__global__ void __launch_bounds__(256) quantize_nvfp4_kernel(const void* __restrict__ x, uint8_t* __restrict__ packed,
                                                             uint8_t* __restrict__ sf_plain, uint8_t* __restrict__ sf_perm, int rows,
                                                             int k, long long x_row_stride, long long packed_row_stride,
                                                             long long sf_plain_row_stride) {
    __shared__ uint32_t staged[2][kQuantGroups][129];   // [unit parity][atom][word of the atom = (row % 32) * 4 + row / 32], padded
    const int groups_per_row = k / 64;
    const int units_k = (groups_per_row + kQuantGroups - 1) / kQuantGroups;
    const long long units = static_cast<long long>((rows + 127) / 128) * units_k;
    const int g = threadIdx.x & (kQuantGroups - 1);
    int parity = 0;
    for (long long unit = blockIdx.x; unit < units; unit += gridDim.x, parity ^= 1) {
        const int row_block = static_cast<int>(unit / units_k);
        const int unit_k = static_cast<int>(unit - static_cast<long long>(row_block) * units_k);
        const int grp = unit_k * kQuantGroups + g;
#pragma unroll
        for (int it = 0; it < 128 * kQuantGroups / 256; ++it) {
            const int r = it * (256 / kQuantGroups) + threadIdx.x / kQuantGroups;   // row inside the block
            const long long row = static_cast<long long>(row_block) * 128 + r;
            uint32_t scales = 0u;
            if (row < rows && grp < groups_per_row) {
                const uint8_t* src = reinterpret_cast<const uint8_t*>(static_cast<const uint16_t*>(x) + row * x_row_stride + grp * 64);
                uint4 in[8];
#pragma unroll
                for (int b = 0; b < 8; ++b) in[b] = __ldcs(reinterpret_cast<const uint4*>(src) + b);
                uint32_t codes[8];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const uint32_t w[8] = {in[2 * b].x, in[2 * b].y, in[2 * b].z, in[2 * b].w, in[2 * b + 1].x, in[2 * b + 1].y, in[2 * b + 1].z, in[2 * b + 1].w};
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (BF16) {
                            v[2 * j] = __uint_as_float(w[j] << 16);
                            v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
                        } else {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                            v[2 * j] = f.x;
                            v[2 * j + 1] = f.y;
                        }
                    }
                    uint32_t out[2];
                    const uint32_t sf_byte = quantize_block16(v, out);
                    codes[2 * b] = out[0];
                    codes[2 * b + 1] = out[1];
                    scales |= sf_byte << (8 * b);
                }
                uint8_t* dst = packed + row * packed_row_stride + grp * 32;
                if (kWide) {
                    *reinterpret_cast<uint4*>(dst) = make_uint4(codes[0], codes[1], codes[2], codes[3]);
                    *reinterpret_cast<uint4*>(dst + 16) = make_uint4(codes[4], codes[5], codes[6], codes[7]);
                    if (sf_plain) *reinterpret_cast<uint32_t*>(sf_plain + row * sf_plain_row_stride + grp * 4) = scales;
                } else {
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        *reinterpret_cast<uint2*>(dst + 8 * b) = make_uint2(codes[2 * b], codes[2 * b + 1]);
                        if (sf_plain) sf_plain[row * sf_plain_row_stride + grp * 4 + b] = static_cast<uint8_t>(scales >> (8 * b));
                    }
                }
            }
            staged[parity][g][(r & 31) * 4 + (r >> 5)] = scales;
        }
        if (sf_perm == nullptr) continue;
        __syncthreads();   // (the other parity's buffer is written next: one barrier per unit is enough)
        // the unit's atoms are contiguous: [row block][atom along K][512 bytes]
        const int atoms_here = min(kQuantGroups, groups_per_row - unit_k * kQuantGroups);
        const int atom = threadIdx.x >> 5, piece = threadIdx.x & 31;   // 16-byte piece of an atom
        if (atom < atoms_here) {
            uint8_t* dst = sf_perm + (static_cast<long long>(row_block) * groups_per_row + unit_k * kQuantGroups + atom) * 512 + piece * 16;
            const uint32_t* st = &staged[parity][atom][piece * 4];
            if (kWide) {
                *reinterpret_cast<uint4*>(dst) = make_uint4(st[0], st[1], st[2], st[3]);
            } else {
#pragma unroll
                for (int b = 0; b < 16; ++b) dst[b] = static_cast<uint8_t>(st[b >> 2] >> (8 * (b & 3)));
            }
        }
    }
}

}  // namespace nvfp4
