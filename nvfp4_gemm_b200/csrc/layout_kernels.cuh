// Data-movement kernels beside the matmul path (HBM-bound, 16-byte vector accesses):
//   * interleave_column_blocks: [g][rows][n_local] fp16 (what an all-gather of per-rank column
//     blocks leaves in memory) -> row-major [rows][g * n_local];
//   * permute_scales: plain [rows][K/16] scale bytes -> the 512-byte atom layout the tensor-core
//     GEMM reads (ref.txt:31, s_128t.py:554-562 in the reference project).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

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

}  // namespace nvfp4
