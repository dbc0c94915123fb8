// NVFP4 block-scaled GEMM for sm_100a:  C[M,N] (fp16) = (A x SFA) . (B x SFB)^T.
//
// One persistent CTA per SM walks a contiguous range of (output tile, k-tile) work units
// ("stream-K"): every CTA gets the same number of 128 x BN x 256 units, so small-M decode
// shapes fill all SMs and large shapes have no partial last wave.  A tile whose k-range is
// covered by one CTA is written straight to C; a tile shared by several CTAs is summed in an
// fp32 scratch slot with vector reductions and converted by whichever CTA finishes it.
//
// Warp roles (192 threads):
//   warp 0      TMA producer: A/B tiles (128-byte swizzle) and the 512-byte scale atoms of the
//               permuted layout into a STAGES-deep shared-memory ring (full/empty mbarriers)
//   warp 1      TMEM owner and MMA issuer: tcgen05.cp scale atoms -> TMEM, four
//               tcgen05.mma.kind::mxf4nvf4.block_scale (K = 64 each) per stage,
//               tcgen05.commit to release the stage / publish the accumulator
//   warps 2..5  epilogue: tcgen05.ld -> fp16 -> TMA store (or 16-byte stores), or the fp32
//               partial-tile reduction
//
// Replaces the reference's single-stage, fully serialised kernel (s_128t.py:375-466).
#pragma once
#include "ptx.cuh"

namespace nvfp4 {

constexpr int kBM = 128;           // tile rows = TMEM lanes
constexpr int kBKBytes = 128;      // bytes of K per stage row = one 128-byte swizzle row = 256 e2m1
constexpr int kKPerStage = 256;    // K elements per stage
constexpr int kMmaPerStage = 4;    // K = 64 per tcgen05.mma
constexpr int kSfAtomBytes = 512;  // 128 rows x 4 scales
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kSfaCol = 256;       // TMEM column of SFA buffer 0 (16 columns per buffer)
constexpr int kSfbCol = 320;       // TMEM column of SFB buffer 0 (BN/8 columns per buffer)

enum GemmStatus : int {
    kStatusOk = 0,
    kStatusWaitTimeout = 1,  // a bounded mbarrier wait ran out
};

struct GemmParams {
    CUtensorMap tma_a;   // {K/2 bytes, M rows, L}, box {128, 128, 1}, 128B swizzle
    CUtensorMap tma_b;   // {K/2 bytes, N rows, L}, box {128, BN, 1},  128B swizzle
    CUtensorMap tma_c;   // {N, M, L} fp16, box {64, 32, 1}, 128B swizzle (TMA-store epilogue)
    const uint8_t* sfa;  // permuted scales of A
    const uint8_t* sfb;  // permuted scales of B
    __half* c;
    float* scratch;      // [grid][BN/4][128][4] fp32 partial-tile slots, all zero between launches
    int* counters;       // [grid] k-tiles accumulated per slot, all zero between launches
    int* status;         // host-visible status word
    long long sfa_batch_stride, sfb_batch_stride;  // bytes
    long long c_row_stride, c_batch_stride;        // elements
    unsigned long long timeout_ns;
    int M, N, K, L;
    int tiles_m, tiles_n, k_tiles;  // k_tiles = K / 256
    int total_units;                // tiles_m * tiles_n * L * k_tiles
};

template <int BN, int STAGES, bool TMA_STORE>
struct GemmSmem {
    static constexpr uint32_t kABytes = kBM * kBKBytes;
    static constexpr uint32_t kBBytes = BN * kBKBytes;
    static constexpr uint32_t kSfaBytes = kMmaPerStage * kSfAtomBytes;
    static constexpr uint32_t kSfbBytes = (BN / 128) * kMmaPerStage * kSfAtomBytes;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr uint32_t kStagingPerWarp = TMA_STORE ? 2 * 32 * 128 : 0;  // two 32-row x 128-byte buffers
    static constexpr uint32_t kStagingOff = STAGES * kStageBytes;
    static constexpr uint32_t kBarOff = kStagingOff + 4 * kStagingPerWarp;
    static constexpr uint32_t kNumAcc = (BN <= 128) ? 2 : 1;
    // full[STAGES] empty[STAGES] acc_full[2] acc_empty[2] | tmem slot | abort flag | finisher flag
    static constexpr uint32_t kBytes = kBarOff + (2 * STAGES + 4) * 8 + 16;
    static constexpr uint32_t kDynamicBytes = kBytes + 1024;  // slack for manual 1024-byte alignment
    static_assert(kStageBytes % 1024 == 0, "stage tiles must keep 1024-byte alignment");
};

// Work range of CTA `cta` out of `grid`: units [begin, end).
__host__ __device__ inline int unit_boundary(int cta, int grid, int total_units) {
    return static_cast<int>((static_cast<long long>(cta) * total_units) / grid);
}
// The CTA whose range holds unit u.
__host__ __device__ inline int unit_owner(int u, int grid, int total_units) {
    int c = static_cast<int>((static_cast<long long>(u) * grid) / total_units);
    if (c >= grid) c = grid - 1;
    while (c + 1 < grid && unit_boundary(c + 1, grid, total_units) <= u) ++c;
    while (c > 0 && unit_boundary(c, grid, total_units) > u) --c;
    return c;
}

template <int BN, int STAGES, bool TMA_STORE>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_nvfp4_kernel(const __grid_constant__ GemmParams p) {
    using S = GemmSmem<BN, STAGES, TMA_STORE>;
    constexpr int kNumAcc = S::kNumAcc;
    constexpr int kSfbColsPerMma = BN / 32;  // 4 TMEM columns per 128 rows of B

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

    const uint32_t bar_full = smem_base + S::kBarOff;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;
    const uint32_t tmem_slot = bar_acc_empty + 2 * 8;
    volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + S::kBarOff + (2 * STAGES + 4) * 8);
    volatile uint32_t* abort_flag = tmem_slot_gen + 1;
    volatile uint32_t* finisher_flag = tmem_slot_gen + 2;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(bar_full + s * 8, 1);
            ptx::mbar_init(bar_empty + s * 8, 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(bar_acc_full + a * 8, 1);
            ptx::mbar_init(bar_acc_empty + a * 8, 128);
        }
        *abort_flag = 0u;
        *finisher_flag = 0u;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&p.tma_a);
        ptx::prefetch_tensormap(&p.tma_b);
        if (TMA_STORE) ptx::prefetch_tensormap(&p.tma_c);
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(tmem_slot, kTmemCols);
        ptx::tmem_relinquish<1>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_gen;

    const int grid = gridDim.x;
    const int u_begin = unit_boundary(blockIdx.x, grid, p.total_units);
    const int u_end = unit_boundary(blockIdx.x + 1, grid, p.total_units);
    const int KT = p.k_tiles;
    const int sf_kblocks = p.K / 64;  // scale atoms per 128-row block
    const uint64_t timeout = p.timeout_ns;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            // A is re-read by every n-tile (keep it in L2); B streams through once per m-tile.
            const uint64_t pol_a = ptx::policy_evict_last();
            const uint64_t pol_b = (p.tiles_m <= 2) ? ptx::policy_evict_first() : ptx::policy_evict_last();
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int u = u_begin; u < u_end && ok;) {
                const int tile = u / KT;
                const int k0 = u - tile * KT;
                const int k1 = min(KT, k0 + (u_end - u));
                const int nb = tile % p.tiles_n;
                const int mb = (tile / p.tiles_n) % p.tiles_m;
                const int l = tile / (p.tiles_n * p.tiles_m);
                const uint8_t* sfa_tile = p.sfa + l * p.sfa_batch_stride + static_cast<long long>(mb) * sf_kblocks * kSfAtomBytes;
                const uint8_t* sfb_tile = p.sfb + l * p.sfb_batch_stride +
                                          static_cast<long long>(nb) * (BN / 128) * sf_kblocks * kSfAtomBytes;
                for (int kt = k0; kt < k1; ++kt) {
                    if (!ptx::mbar_wait_bounded(bar_empty + stage * 8, phase ^ 1u, abort_flag, timeout)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = bar_full + stage * 8;
                    const uint32_t sa = smem_base + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kABytes;
                    const uint32_t ssfa = sb + S::kBBytes;
                    const uint32_t ssfb = ssfa + S::kSfaBytes;
                    ptx::mbar_expect_tx(full, S::kStageBytes);
                    ptx::tma_load_3d(sa, &p.tma_a, kt * kBKBytes, mb * kBM, l, full, pol_a);
                    ptx::tma_load_3d(sb, &p.tma_b, kt * kBKBytes, nb * BN, l, full, pol_b);
                    ptx::bulk_load(ssfa, sfa_tile + static_cast<long long>(kt) * S::kSfaBytes, S::kSfaBytes, full);
#pragma unroll
                    for (int h = 0; h < BN / 128; ++h)
                        ptx::bulk_load(ssfb + h * S::kSfaBytes,
                                       sfb_tile + (static_cast<long long>(h) * sf_kblocks + kt * kMmaPerStage) * kSfAtomBytes,
                                       S::kSfaBytes, full);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                u += k1 - k0;
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::idesc_nvf4(kBM, BN);
            uint32_t stage = 0, phase = 0, acc_it = 0, sf_it = 0;
            bool ok = true;
            for (int u = u_begin; u < u_end && ok;) {
                const int tile = u / KT;
                const int k0 = u - tile * KT;
                const int k1 = min(KT, k0 + (u_end - u));
                const uint32_t acc = acc_it % kNumAcc;
                const uint32_t acc_phase = (acc_it / kNumAcc) & 1u;
                if (!ptx::mbar_wait_bounded(bar_acc_empty + acc * 8, acc_phase ^ 1u, abort_flag, timeout)) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kt = k0; kt < k1; ++kt) {
                    if (!ptx::mbar_wait_bounded(bar_full + stage * 8, phase, abort_flag, timeout)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t sa = smem_base + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kABytes;
                    const uint32_t ssfa = sb + S::kBBytes;
                    const uint32_t ssfb = ssfa + S::kSfaBytes;
                    const uint32_t sf_buf = sf_it & 1u;
                    const uint32_t t_sfa = tmem_base + kSfaCol + sf_buf * 16;
                    const uint32_t t_sfb = tmem_base + kSfbCol + sf_buf * (kMmaPerStage * kSfbColsPerMma);
#pragma unroll
                    for (int kb = 0; kb < kMmaPerStage; ++kb) {
                        ptx::tc_cp_sf<1>(t_sfa + kb * 4, ptx::smem_desc_sf(ssfa + kb * kSfAtomBytes));
#pragma unroll
                        for (int h = 0; h < BN / 128; ++h)
                            ptx::tc_cp_sf<1>(t_sfb + kb * kSfbColsPerMma + h * 4,
                                             ptx::smem_desc_sf(ssfb + h * S::kSfaBytes + kb * kSfAtomBytes));
                    }
                    const uint64_t a_desc = ptx::smem_desc_sw128(sa);
                    const uint64_t b_desc = ptx::smem_desc_sw128(sb);
#pragma unroll
                    for (int kb = 0; kb < kMmaPerStage; ++kb) {
                        // K advances 64 elements = 32 bytes inside the 128-byte swizzle row: +2 in the
                        // (address >> 4) field of the descriptors.
                        ptx::tc_mma_nvf4<1>(d_tmem, a_desc + 2 * kb, b_desc + 2 * kb, idesc, t_sfa + kb * 4,
                                            t_sfb + kb * kSfbColsPerMma, (kt > k0 || kb > 0) ? 1u : 0u);
                    }
                    ptx::tc_commit(bar_empty + stage * 8);  // stage reusable once these MMAs (and copies) retire
                    ++sf_it;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) ptx::tc_commit(bar_acc_full + acc * 8);
                ++acc_it;
                u += k1 - k0;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int quad = warp & 3;             // TMEM lane quadrant this warp may read
        const int row_in_tile = quad * 32 + lane;
        const int epi_tid = threadIdx.x - 64;  // 0..127
        uint32_t acc_it = 0;
        uint32_t store_buf = 0;
        for (int u = u_begin; u < u_end;) {
            const int tile = u / KT;
            const int k0 = u - tile * KT;
            const int k1 = min(KT, k0 + (u_end - u));
            const int nb = tile % p.tiles_n;
            const int mb = (tile / p.tiles_n) % p.tiles_m;
            const int l = tile / (p.tiles_n * p.tiles_m);
            const uint32_t acc = acc_it % kNumAcc;
            const uint32_t acc_phase = (acc_it / kNumAcc) & 1u;
            // All 128 epilogue threads take the same branch: the outcome of the wait is agreed on
            // through a barrier, so a thread that gave up cannot strand the others at a later one.
            const bool got_acc = ptx::mbar_wait_bounded(bar_acc_full + acc * 8, acc_phase, abort_flag, timeout);
            if (!ptx::named_bar_and(2, 128, got_acc)) break;
            ptx::tc_fence_after();
            const uint32_t t_acc = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
            const bool whole_tile = (k1 - k0 == KT);
            const int row = mb * kBM + row_in_tile;
            __half* c_row = p.c + l * p.c_batch_stride + static_cast<long long>(row) * p.c_row_stride + nb * BN;

            if (whole_tile) {
                if constexpr (TMA_STORE) {
                    // 64 columns (128 bytes of fp16) at a time through a swizzled 32-row staging buffer.
                    uint8_t* staging_gen = smem_gen + S::kStagingOff + (warp - 2) * S::kStagingPerWarp;
                    const uint32_t staging = smem_base + S::kStagingOff + (warp - 2) * S::kStagingPerWarp;
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 64) {
                        uint32_t v[2][32];
                        ptx::tc_ld_32cols(t_acc + c0, v[0]);
                        ptx::tc_ld_32cols(t_acc + c0 + 32, v[1]);
                        ptx::tc_wait_ld();
                        // the buffer about to be overwritten was read by the store issued two chunks ago
                        if (lane == 0) ptx::bulk_wait_group_read<1>();
                        __syncwarp();
                        uint8_t* buf = staging_gen + store_buf * 4096 + lane * 128;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t* src = &v[j >> 2][(j & 3) * 8];
                            uint4 q;
                            __half2 h;
                            h = __floats2half2_rn(__uint_as_float(src[0]), __uint_as_float(src[1])); q.x = *reinterpret_cast<uint32_t*>(&h);
                            h = __floats2half2_rn(__uint_as_float(src[2]), __uint_as_float(src[3])); q.y = *reinterpret_cast<uint32_t*>(&h);
                            h = __floats2half2_rn(__uint_as_float(src[4]), __uint_as_float(src[5])); q.z = *reinterpret_cast<uint32_t*>(&h);
                            h = __floats2half2_rn(__uint_as_float(src[6]), __uint_as_float(src[7])); q.w = *reinterpret_cast<uint32_t*>(&h);
                            *reinterpret_cast<uint4*>(buf + ((j ^ (lane & 7)) << 4)) = q;  // 128-byte swizzle
                        }
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && mb * kBM + quad * 32 < p.M) {  // rows past M inside the box are clipped
                            ptx::tma_store_3d(&p.tma_c, staging + store_buf * 4096, nb * BN + c0, mb * kBM + quad * 32, l);
                            ptx::bulk_commit_group();
                        }
                        store_buf ^= 1u;
                    }
                } else {
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 32) {
                        uint32_t v[32];
                        ptx::tc_ld_32cols(t_acc + c0, v);
                        ptx::tc_wait_ld();
                        if (row < p.M) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint4 q;
                                __half2 h;
                                h = __floats2half2_rn(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1])); q.x = *reinterpret_cast<uint32_t*>(&h);
                                h = __floats2half2_rn(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])); q.y = *reinterpret_cast<uint32_t*>(&h);
                                h = __floats2half2_rn(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])); q.z = *reinterpret_cast<uint32_t*>(&h);
                                h = __floats2half2_rn(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])); q.w = *reinterpret_cast<uint32_t*>(&h);
                                *reinterpret_cast<uint4*>(c_row + c0 + 8 * j) = q;
                            }
                        }
                    }
                }
                ptx::tc_fence_before();
                ptx::mbar_arrive(bar_acc_empty + acc * 8);
            } else {
                // Partial tile: add this CTA's k-range into the tile's fp32 slot.  Slot layout
                // [BN/4][128 rows][4] keeps each warp's 16-byte reductions contiguous (512 bytes).
                const int slot = unit_owner(tile * KT, grid, p.total_units);
                float* slot_base = p.scratch + static_cast<long long>(slot) * (kBM * BN);
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t v[32];
                    ptx::tc_ld_32cols(t_acc + c0, v);
                    ptx::tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        ptx::red_add_v4(slot_base + ((c0 / 4 + j) * kBM + row_in_tile) * 4, __uint_as_float(v[4 * j]),
                                        __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                        __uint_as_float(v[4 * j + 3]));
                }
                ptx::tc_fence_before();
                ptx::mbar_arrive(bar_acc_empty + acc * 8);  // MMA warp may start the next tile now
                __threadfence();
                ptx::named_bar_sync(1, 128);
                if (epi_tid == 0) {
                    const int done = atomicAdd(p.counters + slot, k1 - k0) + (k1 - k0);
                    *finisher_flag = (done == KT) ? 1u : 0u;
                }
                ptx::named_bar_sync(1, 128);
                const bool finisher = (*finisher_flag != 0u);
                ptx::named_bar_sync(1, 128);  // flag may be rewritten only after everyone read it
                if (finisher) {
                    __threadfence();
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 8) {
                        float* src = slot_base + ((c0 / 4) * kBM + row_in_tile) * 4;
                        const float4 lo = ptx::ld_cg_v4(src);
                        const float4 hi = ptx::ld_cg_v4(src + kBM * 4);
                        ptx::st_cg_v4(src, make_float4(0.f, 0.f, 0.f, 0.f));  // leave the slot zeroed
                        ptx::st_cg_v4(src + kBM * 4, make_float4(0.f, 0.f, 0.f, 0.f));
                        if (row < p.M) {
                            uint4 q;
                            __half2 h;
                            h = __floats2half2_rn(lo.x, lo.y); q.x = *reinterpret_cast<uint32_t*>(&h);
                            h = __floats2half2_rn(lo.z, lo.w); q.y = *reinterpret_cast<uint32_t*>(&h);
                            h = __floats2half2_rn(hi.x, hi.y); q.z = *reinterpret_cast<uint32_t*>(&h);
                            h = __floats2half2_rn(hi.z, hi.w); q.w = *reinterpret_cast<uint32_t*>(&h);
                            *reinterpret_cast<uint4*>(c_row + c0) = q;
                        }
                    }
                    if (epi_tid == 0) p.counters[slot] = 0;
                }
            }
            ++acc_it;
            u += k1 - k0;
        }
        if constexpr (TMA_STORE) {
            if (lane == 0) ptx::bulk_wait_group<0>();  // staging must outlive the stores that read it
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // Some wait ran out.  Give copies still in flight time to land in shared memory before
        // the CTA retires, then report.
        __nanosleep(20000);
        if (threadIdx.x == 0) {
            *reinterpret_cast<volatile int*>(p.status) = kStatusWaitTimeout;
            __threadfence_system();
        }
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<1>(tmem_base, kTmemCols);
    }
}

}  // namespace nvfp4
