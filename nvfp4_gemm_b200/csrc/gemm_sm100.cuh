// NVFP4 block-scaled GEMM for sm_100a:  C[M,N] (fp16) = (A x SFA) . (B x SFB)^T.
//
// Persistent workers walk a contiguous range of (output tile, k-tile) work units ("stream-K"):
// every worker gets the same number of units, so large shapes have no partial last wave; or, when
// the launch code finds that cheaper, whole tiles only (GemmParams::whole_tiles).  A tile whose
// k-range one worker covers is written straight to C.  A tile shared by several workers is
// published as fp32 partials in per-worker scratch slots by all but the worker that holds the
// start of its k-range, which sums the partials in a fixed order (deterministic) and writes fp16;
// SegmentPlan orders a worker's pieces so that this summing runs beside later whole tiles.
// Decode shapes (one 128-row block) split K over a cluster instead (KS > 1).
//
// A worker is one CTA (CG = 1: 128 x BN tile) or a CTA pair running tcgen05 with cta_group::2
// (CG = 2: 256 x BN tile; each CTA holds 128 rows of A, BN/2 rows of B and its own 128
// accumulator rows, so B crosses L2 -> SM once per pair).
//
// Warp roles (192 threads per CTA):
//   warp 0      TMA producer: A/B tiles (128-byte swizzle) and the 512-byte scale atoms of the
//               permuted layout into a STAGES-deep shared-memory ring (full/empty mbarriers)
//   warp 1      TMEM owner.  Leader CTA: MMA issuer, ONE thread elected once -- tcgen05.cp scale
//               atoms -> TMEM, four tcgen05.mma.kind::mxf4nvf4.block_scale (K = 64 each) per
//               stage, tcgen05.commit to release the stage / publish the accumulator.  In a pair
//               both CTAs' loads signal the leader's full barrier (cp.async.bulk.tensor
//               .cta_group::2).
//   warps 2..5  epilogue: tcgen05.ld -> fp16 -> TMA store (or 16-byte stores), or the fp32
//               partial-tile path
//
// No load in this file uses cluster multicast; the only cluster-wide signals are mbarrier
// arrivals (remote arrive, TMA completion on the leader's barrier, tcgen05.commit to both CTAs
// of a pair).
//
// Replaces the reference's single-stage, fully serialised kernel (s_128t.py:375-466).
#pragma once
#include "ptx.cuh"
#include "quantize.cuh"

namespace nvfp4 {

constexpr int kBM = 128;           // rows per CTA tile = TMEM lanes
constexpr int kBKBytes = 128;      // bytes of K per stage row = one 128-byte swizzle row = 256 e2m1
constexpr int kKPerStage = 256;    // K elements per stage
constexpr int kMmaPerStage = 4;    // K = 64 per tcgen05.mma
constexpr int kSfAtomBytes = 512;  // 128 rows x 4 scales
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;
// TMEM columns.  128-wide tiles: two accumulators [0,128) and [128,256), scale buffers behind
// them.  256-wide tiles of the persistent kernels: two accumulators that OVERLAP by half,
// X = [0,256) and Y = [128,384), scale buffers at [384,480).  The epilogue drains the shared
// half [128,256) first and hands the accumulator back as soon as it is in registers, so the next
// tile's MMAs (into the other accumulator) run while the rest is drained and stored; two full
// 256-column accumulators plus the scale columns would not fit the 512 columns of an SM.
constexpr int kSfaColPlain = 256, kSfbColPlain = 320;      // SFA / SFB buffer 0 (16 and BN/8 columns per buffer)
constexpr int kSfaColOverlap = 384, kSfbColOverlap = 416;

enum Activation : int { kActNone = 0, kActRelu = 1, kActSilu = 2 };

enum GemmStatus : int {
    kStatusOk = 0,
    kStatusWaitTimeout = 1,  // a bounded mbarrier wait ran out
};

struct GemmParams {
    CUtensorMap tma_a;   // {K/2 bytes, M rows, L}, box {128, 128, 1},    128B swizzle
    CUtensorMap tma_b;   // {K/2 bytes, N rows, L}, box {128, BN/CG, 1},  128B swizzle
    CUtensorMap tma_c;   // {N, M, L} fp16, box {64, 32, 1}, 128B swizzle (TMA-store epilogue)
    CUtensorMap tma_sfa; // permuted scales of A as {128 words, K/64 atoms, row blocks, L}, box {128, 4, 1, 1}
    CUtensorMap tma_sfb; // permuted scales of B, same view, box {128, 4, BN/128, 1}
    __half* c;
    // Fused all-gather (column-parallel multi-GPU): every finished piece of C is also stored into
    // the same position of n_peer other GPUs' output buffers (peer-mapped memory, plain vector
    // stores only; nothing is ever loaded from a peer).
    __half* c_peer[7];
    int n_peer;
    // With few peers the TMA-store epilogue sends each peer its copy of a staged block with one more
    // tensor store (tma_c_peer[i] describes c_peer[i] like tma_c describes c); with many, the
    // epilogue warps store the block themselves.
    int peer_tma;
    CUtensorMap tma_c_peer[7];
    // Extended epilogue (kernels instantiated with EPI_EX): out = act(acc + bias[column]), written
    // as fp16 to c, or re-quantised to NVFP4 (packed e2m1 + one e4m3 scale per 16 columns of a row,
    // the operand format of a following GEMM whose K is this GEMM's N).
    const __half* bias;          // [N] or null
    int activation;              // kActNone / kActRelu / kActSilu
    int out_nvfp4;               // 0: fp16 to c; 1: packed + scales
    uint8_t* out_packed;         // [L][M][N/2]
    uint8_t* out_sf;             // plain [L][M][N/16] or null
    uint8_t* out_sf_perm;        // 512-byte atoms (128 rows x 4 scales), [L][ceil(M/128)][N/64][512], or null
    long long out_packed_row_stride, out_packed_batch_stride;   // bytes
    long long out_sf_row_stride, out_sf_batch_stride;           // bytes
    long long out_sf_perm_batch_stride;                         // bytes
    long long out_sf_perm_block_stride;                         // bytes between 128-row blocks of the permuted scales
    float* scratch;      // partial-tile slots [worker][head|tail][cta of pair][BN/4][128][4] fp32
    int* counters;       // [worker][cta of pair] k-tiles published per shared tile; zero between launches
    int* status;         // host-visible status word
    long long c_row_stride, c_batch_stride;        // elements
    unsigned long long timeout_cycles;  // limit of every in-kernel wait, in SM clock cycles
    int M, N, K, L;
    int tiles_m, tiles_n, k_tiles;  // tiles of (128*CG) x BN; k_tiles = K / 256
    int raster_rows;                // row tiles per group of the persistent kernels' tile order; 0 = row-major
    int total_units;                // tiles_m * tiles_n * L * k_tiles
    int whole_tiles;                // 1: workers split the work at tile boundaries only (no tile is shared); raster_rows must be 0
};

constexpr int kPrefetchStages = 2;                  // stages of a CTA's first segment prefetched into L2 ahead of the dependency wait
constexpr int kGlobalExchangeMinSplit = 4;         // cluster split-K: from this split on the partial sums travel through L2
constexpr int kScratchSlotFloats = kBM * 256;      // one partial-tile slot of the library's scratch (128 x 256 fp32)

template <int CG, int BN, int STAGES, bool TMA_STORE, int EPI_KB, int KS = 1>
struct GemmSmem {
    static constexpr uint32_t kBRows = BN / CG;
    static constexpr uint32_t kABytes = kBM * kBKBytes;
    static constexpr uint32_t kBBytes = kBRows * kBKBytes;
    static constexpr uint32_t kSfaBytes = kMmaPerStage * kSfAtomBytes;
    static constexpr uint32_t kSfbBytes = (BN / 128) * kMmaPerStage * kSfAtomBytes;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    // Epilogue scratch: TMA-store staging (two 32-row x 128-byte buffers per warp), or the landing
    // area of the cluster split-K exchange.
    static constexpr uint32_t kEpiBytes = EPI_KB * 1024;
    static constexpr uint32_t kStagingBufs = TMA_STORE ? (EPI_KB * 1024 / 4) / 4096 : 2;   // 32-row x 128-byte buffers per epilogue warp
    static constexpr uint32_t kStagingPerWarp = kStagingBufs * 32 * 128;
    static constexpr uint32_t kFixBufs = 2;   // barriers of the cluster split-K exchange ("landed", "ready")
    static constexpr uint32_t kEpiOff = STAGES * kStageBytes;
    static constexpr uint32_t kBarOff = kEpiOff + kEpiBytes;
    // Cluster split-K: one sender's share of the columns a CTA finalises, and whether the ring holds
    // both the KS - 1 incoming pieces and the KS - 1 outgoing ones (then the exchange uses bulk copies).
    static constexpr uint32_t kPieceBytes = (BN / KS) * kBM * 4;
    static constexpr bool kBulkExchange = KS > 1 && 2u * (KS - 1) * kPieceBytes <= STAGES * kStageBytes;
    // Wider splits exchange through global memory (L2) instead: distributed shared memory moves
    // about 14 bytes per cycle and SM, a quarter of what an SM gets from L2.
    static constexpr bool kGlobalExchange = KS >= kGlobalExchangeMinSplit;
    static constexpr bool kAccOverlap = (BN == 256 && KS == 1);        // see the TMEM column map above
    static constexpr uint32_t kNumAcc = (BN <= 128 || kAccOverlap) ? 2 : 1;
    static constexpr uint32_t kAccStride = kAccOverlap ? BN / 2 : BN;  // TMEM columns between the two accumulators
    // full[STAGES] empty[STAGES] acc_full[2] acc_empty[2] exchange[kFixBufs] | tmem slot | abort
    static constexpr uint32_t kNumBars = 2 * STAGES + 4 + kFixBufs;
    static constexpr uint32_t kBytes = kBarOff + kNumBars * 8 + 16;
    static constexpr uint32_t kDynamicBytes = kBytes + 1024;  // slack for manual 1024-byte alignment
    static_assert(kStageBytes % 1024 == 0, "stage tiles must keep 1024-byte alignment");
    static_assert(!TMA_STORE || kEpiBytes >= 4 * kStagingPerWarp, "TMA-store staging does not fit");
    static_assert(KS == 1 || (CG == 1 && BN / KS >= 32 && STAGES * kStageBytes >= kBM * BN * 4),
                  "cluster split-K: single-CTA MMAs, at least 32 columns per CTA, the ring must hold one fp32 tile");
    static_assert(kDynamicBytes <= 232448, "exceeds the 227 KB of shared memory one CTA may use");
};

// Work range of worker `w` out of `n`: units [boundary(w), boundary(w + 1)).
__host__ __device__ inline int unit_boundary(int w, int n, int total_units) {
    return static_cast<int>((static_cast<long long>(w) * total_units) / n);
}
// The worker whose range holds unit u.
__host__ __device__ inline int unit_owner(int u, int n, int total_units) {
    int c = static_cast<int>((static_cast<long long>(u) * n) / total_units);
    if (c >= n) c = n - 1;
    while (c + 1 < n && unit_boundary(c + 1, n, total_units) <= u) ++c;
    while (c > 0 && unit_boundary(c, n, total_units) > u) --c;
    return c;
}
// The i-th piece of work ("segment": consecutive k-tiles of ONE output tile) of a worker whose
// unit range is [ub, ue): the partial tile the range starts in, the whole tiles but the last, the
// partial tile the range ends in, the last whole tile.  A tile shared by two workers is finished
// by the one that holds the start of its k-range, i.e. in that worker's last-but-one segment:
// the other worker published its partial sums in its very first segment, long before, and the
// summing runs beside the MMAs of the finisher's last whole tile, so that nothing but an
// ordinary epilogue follows a worker's last MMA.  False when i is past the end.
struct Segment {
    int u0, u1, tile;
};
struct SegmentPlan {
    int ub, ue, head_end, tail_begin, n_head, n_tail, whole, k_tiles, first_tile, last_tile;
    // (two independent divisions: this runs in front of every role's first instruction)
    __host__ __device__ SegmentPlan(int ub_, int ue_, int k_tiles_) : ub(ub_), ue(ue_), k_tiles(k_tiles_) {
        first_tile = ub / k_tiles;                              // tile the range starts in
        last_tile = ue / k_tiles;                               // tile the range ends in (or just before)
        n_head = ub != first_tile * k_tiles ? 1 : 0;
        head_end = (first_tile + n_head) * k_tiles;             // first tile boundary at or after ub
        if (head_end > ue) head_end = ue;
        tail_begin = last_tile * k_tiles;                       // last tile boundary at or before ue
        if (tail_begin < head_end) tail_begin = head_end;
        n_tail = ue > tail_begin ? 1 : 0;
        whole = last_tile - (first_tile + n_head);
        if (whole < 0) whole = 0;
    }
    __host__ __device__ bool at(int i, Segment* out) const {
        if (i < n_head) { *out = Segment{ub, head_end, first_tile}; return true; }
        int j = i - n_head;                                     // position among [whole..., tail, last whole]
        if (j >= whole + n_tail) return false;
        if (n_tail) {
            const int tail_pos = whole > 0 ? whole - 1 : 0;
            if (j == tail_pos) { *out = Segment{tail_begin, ue, last_tile}; return true; }
            if (j > tail_pos) --j;
        }
        *out = Segment{head_end + j * k_tiles, head_end + (j + 1) * k_tiles, first_tile + n_head + j};
        return true;
    }
};

// Where tile `tile` of the workers' linear tile sequence lies in the output: (batch, row tile,
// column tile).  Worker w walks the contiguous tile indices of its unit range, so at any moment
// the workers sit at the same RELATIVE position r in their ranges.  Tiles are therefore ranked by
// (r, w): the tiles the workers process at the same time get consecutive ranks, and consecutive
// ranks fill the output column by column inside groups of raster_rows row tiles -- a wave of
// workers shares a few row blocks of A and a few column tiles of B through L2 instead of every
// worker streaming its own pair from DRAM.
// raster_rows = 0 keeps the plain row-major order of the linear tile index.
struct TileCoord {
    int l, mt, nt;
};
__host__ __device__ inline TileCoord tile_coords(int tile, int n_workers, int k_tiles, int total_units, int tiles_m, int tiles_n,
                                                 int raster_rows) {
    if (raster_rows <= 0) return TileCoord{tile / (tiles_n * tiles_m), (tile / tiles_n) % tiles_m, tile % tiles_n};
    const int tiles = total_units / k_tiles;
    const int q = tiles / n_workers;                       // every worker starts q or q + 1 tiles
    const int w = unit_owner(tile * k_tiles, n_workers, total_units);
    const int first = (unit_boundary(w, n_workers, total_units) + k_tiles - 1) / k_tiles;   // first tile that starts in w's range
    const int r = tile - first;
    const int rank = (r < q) ? r * n_workers + w : q * n_workers + (first - q * w);
    const int per_batch = tiles_m * tiles_n;
    TileCoord c;
    c.l = rank / per_batch;
    const int x = rank - c.l * per_batch;
    const int group = x / (raster_rows * tiles_n);
    const int y = x - group * (raster_rows * tiles_n);
    const int rows = min(raster_rows, tiles_m - group * raster_rows);
    c.nt = y / rows;
    c.mt = group * raster_rows + (y - c.nt * rows);
    return c;
}

// Scratch slot of a worker's partial segment: a worker has at most one segment that starts
// inside a tile ("head", k0 > 0) and at most one that starts a tile but does not finish it.
__host__ __device__ inline int partial_slot(int worker, int k0, int cg, int cta_rank) {
    return (worker * 2 + (k0 > 0 ? 0 : 1)) * cg + cta_rank;
}

__device__ __forceinline__ uint4 pack8_fp16(const float* v) {
    uint4 q;
    __half2 h;
    h = __floats2half2_rn(v[0], v[1]); q.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(v[2], v[3]); q.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(v[4], v[5]); q.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(v[6], v[7]); q.w = *reinterpret_cast<uint32_t*>(&h);
    return q;
}
__device__ __forceinline__ uint4 pack8_fp16(const uint32_t* v) {
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[i]);
    return pack8_fp16(f);
}

template <int CG, int BN, int STAGES, bool TMA_STORE, int EPI_KB, int KS = 1, bool EPI_EX = false>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_nvfp4_kernel(const __grid_constant__ GemmParams p) {
    static_assert(!(EPI_EX && TMA_STORE), "the extended epilogue writes with plain stores");
    using S = GemmSmem<CG, BN, STAGES, TMA_STORE, EPI_KB, KS>;
    constexpr int kNumAcc = S::kNumAcc;
    constexpr bool kAccOverlap = S::kAccOverlap;
    constexpr int kSfaCol = kAccOverlap ? kSfaColOverlap : kSfaColPlain;
    constexpr int kSfbCol = kAccOverlap ? kSfbColOverlap : kSfbColPlain;
    constexpr int kChunks = BN / 32;                                   // 32-column pieces of an accumulator row
    // An overlapped accumulator is drained shared half first and released once that half is in
    // registers; a plain one after its last column.
    constexpr int kReleaseAfter = kAccOverlap ? kChunks / 2 : kChunks;
    constexpr int kSfbColsPerMma = BN / 32;  // 4 TMEM columns per 128 rows of B
    constexpr int kBRows = S::kBRows;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

    const uint32_t bar_full = smem_base + S::kBarOff;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;
    const uint32_t bar_fix_full = bar_acc_empty + 2 * 8;
    const uint32_t tmem_slot = bar_fix_full + S::kFixBufs * 8;
    volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + S::kBarOff + S::kNumBars * 8);
    volatile uint32_t* abort_flag = tmem_slot_gen + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cta_rank = (CG == 2) ? static_cast<int>(ptx::cluster_ctarank()) : 0;
    const bool leader = (cta_rank == 0);
    // Cluster split-K (KS > 1): the KS CTAs of a cluster share one output tile, each contracting
    // 1/KS of K with its own MMAs and TMEM; the partial sums are exchanged through distributed
    // shared memory and every CTA finalises BN/KS columns.
    const int ks_rank = (KS > 1) ? static_cast<int>(ptx::cluster_ctarank()) : 0;
    const uint32_t bar_land = bar_fix_full;       // KS > 1: "all peers' partial columns have landed"
    const uint32_t bar_ready = bar_fix_full + 8;  // KS > 1: "all peers are done with their operand ring"

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(bar_full + s * 8, 1);
            ptx::mbar_init(bar_empty + s * 8, 1);
        }
        for (uint32_t b = 0; b < S::kFixBufs; ++b)
            ptx::mbar_init(bar_fix_full + b * 8, (KS > 1 && b == 0) ? (S::kBulkExchange ? 1 : 128 * (KS - 1)) : (KS > 1 && b == 1) ? (KS - 1) : 1);
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(bar_acc_full + a * 8, 1);
            ptx::mbar_init(bar_acc_empty + a * 8, 128 * CG);
        }
        *abort_flag = 0u;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&p.tma_a);
        ptx::prefetch_tensormap(&p.tma_b);
        ptx::prefetch_tensormap(&p.tma_sfa);
        ptx::prefetch_tensormap(&p.tma_sfb);
        if (TMA_STORE) ptx::prefetch_tensormap(&p.tma_c);
        if (TMA_STORE && p.peer_tma)
            for (int r = 0; r < p.n_peer; ++r) ptx::prefetch_tensormap(&p.tma_c_peer[r]);
    }
    __syncthreads();  // barriers initialised
    bool cluster_waited = true;
    if constexpr (CG == 2) {
        // both CTAs of the pair are resident and have initialised their barriers before the first
        // load signals the leader's barrier or any pair-wide instruction is issued
        ptx::cluster_arrive();
        ptx::cluster_wait();
    } else if constexpr (KS > 1) {
        // split-K peers touch this CTA only in the exchange epilogue: arrive now, wait there
        ptx::cluster_arrive();
        cluster_waited = false;
    }
    // TMEM is allocated by warp 1 while warp 0 already streams operands; warps 1..5 meet on a
    // named barrier to pick up the base address.
    uint32_t tmem_base = 0;
    if (warp == 1) {
        ptx::tmem_alloc<CG>(tmem_slot, kTmemCols);
        ptx::tmem_relinquish<CG>();
        ptx::tc_fence_before();
    }
    // This CTA's share of the work, worked out before the wait below: it reads kernel parameters only.
    const int KT = p.k_tiles;
    const int n_workers = (KS > 1) ? static_cast<int>(gridDim.x) : static_cast<int>(gridDim.x) / CG;
    const int worker = (KS > 1) ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x) / CG;
    // stream-K: equal share of all units.  Cluster split-K: tile = cluster index, k-range by rank.
    // Whole tiles: the same even split counted in tiles (p.total_units / KT of them) instead of units.
    const int split_total = p.whole_tiles ? p.tiles_m * p.tiles_n * p.L : p.total_units;
    const int split_scale = p.whole_tiles ? KT : 1;
    const int u_begin = (KS > 1) ? (worker / KS) * KT + (ks_rank * KT) / KS : unit_boundary(worker, n_workers, split_total) * split_scale;
    const int u_end = (KS > 1) ? (worker / KS) * KT + ((ks_rank + 1) * KT) / KS : unit_boundary(worker + 1, n_workers, split_total) * split_scale;
    const uint64_t timeout = p.timeout_cycles;
    const SegmentPlan plan(u_begin, u_end, KT);   // (a cluster split-K CTA has one segment: its share of the tile's k-range)
    Segment first_seg{0, 0, 0};
    plan.at(0, &first_seg);
    const TileCoord first_tc = tile_coords(first_seg.tile, n_workers, KT, p.total_units, p.tiles_m, p.tiles_n, (KS > 1) ? 0 : p.raster_rows);
    // The operands of this CTA's first two stages are asked into L2 now, ahead of the dependency wait:
    // a CTA of a back-to-back launch reaches this point while slower CTAs of the previous launch
    // are still running, and its first loads then find their lines in L2 instead of paying the
    // DRAM latency after the wait.  A prefetch consumes nothing: lines the previous launch still
    // writes are updated in L2, where the loads read them.  (Two stages: asking for the whole ring
    // takes HBM bandwidth from the tail of the previous launch and made the decode shape slower.)
    if (warp == 0 && first_seg.u1 > first_seg.u0) {
        if (ptx::elect_one()) {
            const int k0 = first_seg.u0 - first_seg.tile * KT;
            const int n_pre = min(kPrefetchStages, first_seg.u1 - first_seg.u0);
            const int mb = first_tc.mt * CG + cta_rank;
            for (int i = 0; i < n_pre; ++i) {
                const int kt = k0 + i;
                ptx::tma_prefetch_3d(&p.tma_a, kt * kBKBytes, mb * kBM, first_tc.l);
                ptx::tma_prefetch_3d(&p.tma_b, kt * kBKBytes, first_tc.nt * BN + cta_rank * kBRows, first_tc.l);
                ptx::tma_prefetch_4d(&p.tma_sfa, 0, kt * kMmaPerStage, mb, first_tc.l);
                ptx::tma_prefetch_4d(&p.tma_sfb, 0, kt * kMmaPerStage, first_tc.nt * (BN / 128), first_tc.l);
            }
        }
        __syncwarp();
    }
    // Kernels of this library are often launched back to back (a decode step is a chain of short
    // GEMMs): let the next launch's CTAs set up (barriers, TMEM, descriptor prefetch) on SMs this
    // grid leaves idle or frees, and touch global memory only after everything the stream ordered
    // before this launch is complete.  Without the launch attribute both are no-ops.
    ptx::grid_dependency_launch_dependents();
    ptx::grid_dependency_wait();
    if (warp != 0) {
        ptx::named_bar_sync(3, kGemmThreads - 32);
        ptx::tc_fence_after();
        tmem_base = *tmem_slot_gen;
    }


    // Warps 0 and 1 each hand their whole loop to ONE lane chosen once by elect.sync (the compiler
    // then knows the path has a single thread and feeds descriptors straight from uniform
    // registers; a lane picked by "if (lane == 0)" costs ~50 cycles per instruction instead).
    // Running the loop with all 32 lanes converged and electing per stage costs a vote, an
    // election and a reconvergence per stage: 2 % of the run time of a large GEMM.
    if (warp == 0) {
        // ------------------------------------------------------------ producer
        // A is re-read by every n-tile (keep it in L2); B streams through once per m-tile.
        const uint64_t pol_a = ptx::policy_evict_last();
        const uint64_t pol_b = (p.tiles_m * CG <= 2) ? ptx::policy_evict_first() : ptx::policy_evict_last();
        // The scales are re-read like the operands they belong to.  With few row tiles (decode) B and
        // its scales stream through once and the hint only costs: those loads go without one.
        const bool hint_sf = p.tiles_m * CG > 2;
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        Segment seg;
        for (int si = 0; ok && plan.at(si, &seg); ++si) {
            const int tile = seg.tile;
            const int k0 = seg.u0 - tile * KT;
            const int k1 = k0 + (seg.u1 - seg.u0);
            const TileCoord tc = (si == 0) ? first_tc : tile_coords(tile, n_workers, KT, p.total_units, p.tiles_m, p.tiles_n, (KS > 1) ? 0 : p.raster_rows);
            const int nb = tc.nt;
            const int mb = tc.mt * CG + cta_rank;  // 128-row block of this CTA
            const int l = tc.l;
            for (int kt = k0; kt < k1; ++kt) {
                {
                    ok = ptx::mbar_wait_bounded(bar_empty + stage * 8, phase ^ 1u, abort_flag, timeout);
                    ok = __all_sync(0xffffffffu, ok);
                }
                if (!ok) break;
                if (ptx::elect_one()) {
                    const uint32_t sa = smem_base + stage * S::kStageBytes;
                    const uint32_t sb = sa + S::kABytes;
                    const uint32_t ssfa = sb + S::kBBytes;
                    const uint32_t ssfb = ssfa + S::kSfaBytes;
                    if constexpr (CG == 1) {
                        const uint32_t full = bar_full + stage * 8;
                        ptx::mbar_expect_tx(full, S::kStageBytes);
                        ptx::tma_load_3d(sa, &p.tma_a, kt * kBKBytes, mb * kBM, l, full, pol_a);
                        ptx::tma_load_3d(sb, &p.tma_b, kt * kBKBytes, nb * BN, l, full, pol_b);
                        if (hint_sf) {
                            ptx::tma_load_4d(ssfa, &p.tma_sfa, 0, kt * kMmaPerStage, mb, l, full, pol_a);
                            ptx::tma_load_4d(ssfb, &p.tma_sfb, 0, kt * kMmaPerStage, nb * (BN / 128), l, full, pol_b);
                        } else {
                            ptx::tma_load_4d(ssfa, &p.tma_sfa, 0, kt * kMmaPerStage, mb, l, full);
                            ptx::tma_load_4d(ssfb, &p.tma_sfb, 0, kt * kMmaPerStage, nb * (BN / 128), l, full);
                        }
                    } else {
                        // Both CTAs of the pair report to the leader's barrier, which expects the
                        // bytes of both stages (a completion may precede the expectation: the
                        // transaction count is signed and the phase cannot end before the arrival).
                        const uint32_t full = ptx::mapa_u32(bar_full + stage * 8, 0);
                        if (leader) ptx::mbar_expect_tx(bar_full + stage * 8, 2 * S::kStageBytes);
                        ptx::tma_load_3d_pair(sa, &p.tma_a, kt * kBKBytes, mb * kBM, l, full, pol_a);
                        ptx::tma_load_3d_pair(sb, &p.tma_b, kt * kBKBytes, nb * BN + cta_rank * kBRows, l, full, pol_b);
                        if (hint_sf) {
                            ptx::tma_load_4d_pair(ssfa, &p.tma_sfa, 0, kt * kMmaPerStage, mb, l, full, pol_a);
                            ptx::tma_load_4d_pair(ssfb, &p.tma_sfb, 0, kt * kMmaPerStage, nb * (BN / 128), l, full, pol_b);
                        } else {
                            ptx::tma_load_4d_pair(ssfa, &p.tma_sfa, 0, kt * kMmaPerStage, mb, l, full);
                            ptx::tma_load_4d_pair(ssfb, &p.tma_sfb, 0, kt * kMmaPerStage, nb * (BN / 128), l, full);
                        }
                    }
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (leader) {
            // ------------------------------------------------------ MMA issuer
            constexpr uint32_t idesc = ptx::idesc_nvf4(kBM * CG, BN);
            uint32_t stage = 0, phase = 0, acc_it = 0, sf_it = 0;
            bool ok = true;
            Segment seg;
            // Shared-memory descriptors of slot 0; every other one is a 32-bit add away (the address
            // field, in 16-byte units, never carries out of its 14 bits inside 227 KB).
            const uint64_t desc_ab0 = ptx::smem_desc_sw128(smem_base);
            const uint64_t desc_sf0 = ptx::smem_desc_sf(smem_base + S::kABytes + S::kBBytes);
            const uint32_t ab_lo0 = static_cast<uint32_t>(desc_ab0), ab_hi = static_cast<uint32_t>(desc_ab0 >> 32);
            const uint32_t sf_lo0 = static_cast<uint32_t>(desc_sf0), sf_hi = static_cast<uint32_t>(desc_sf0 >> 32);
            if (ptx::elect_one()) {   // (the loop below is this one thread's; indentation kept flat)
            for (int si = 0; ok && plan.at(si, &seg); ++si) {
                const int k0 = seg.u0 - seg.tile * KT;
                const int k1 = k0 + (seg.u1 - seg.u0);
                const uint32_t acc = acc_it % kNumAcc;
                // Overlapped accumulators: one hand-back per tile on barrier 0 (the previous tile's
                // shared half is drained; the tile before that, in this accumulator, was drained
                // earlier by the same threads).  Plain: one barrier per accumulator.
                const uint32_t empty_bar = bar_acc_empty + (kAccOverlap ? 0u : acc * 8);
                const uint32_t empty_phase = kAccOverlap ? (acc_it & 1u) : ((acc_it / kNumAcc) & 1u);
                ok = ptx::mbar_wait_bounded(empty_bar, empty_phase ^ 1u, abort_flag, timeout);
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * S::kAccStride;
                // One stage per turn: wait, fence, 12 scale copies + 4 MMAs, commit: about 200 cycles of
                // this thread for the 512 cycles the MMAs of a 256-wide stage run, so the pipe always
                // has a stage or two queued.  Anything more in this loop showed up in the run time:
                // as a converged warp that polls, votes and elects per stage a turn took 650 cycles
                // and the pipe starved; issuing two landed stages per turn to save a wait cost 2 %
                // (the probe for the second stage costs what the wait saves).
                for (int kt = k0; kt < k1; ++kt) {
                    ok = ptx::mbar_wait_bounded(bar_full + stage * 8, phase, abort_flag, timeout);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint32_t slot_off = stage * (S::kStageBytes >> 4);
                    const uint32_t a_lo = ab_lo0 + slot_off, b_lo = a_lo + (S::kABytes >> 4);
                    const uint32_t sfa_lo = sf_lo0 + slot_off, sfb_lo = sfa_lo + (S::kSfaBytes >> 4);
                    const uint32_t sf_buf = sf_it & 1u;
                    const uint32_t t_sfa = tmem_base + kSfaCol + sf_buf * 16;
                    const uint32_t t_sfb = tmem_base + kSfbCol + sf_buf * (kMmaPerStage * kSfbColsPerMma);
                    // With cta_group::2 each of these runs in both CTAs of the pair, every CTA reading
                    // its own shared memory at the same offsets.
#pragma unroll
                    for (int kb = 0; kb < kMmaPerStage; ++kb) {
                        ptx::tc_cp_sf<CG>(t_sfa + kb * 4, sfa_lo + kb * (kSfAtomBytes >> 4), sf_hi);
#pragma unroll
                        for (int h = 0; h < BN / 128; ++h)
                            ptx::tc_cp_sf<CG>(t_sfb + kb * kSfbColsPerMma + h * 4, sfb_lo + h * (S::kSfaBytes >> 4) + kb * (kSfAtomBytes >> 4), sf_hi);
                    }
#pragma unroll
                    for (int kb = 0; kb < kMmaPerStage; ++kb) {
                        // K advances 64 elements = 32 bytes inside the 128-byte swizzle row: +2 in the
                        // (address >> 4) field of the descriptors.
                        ptx::tc_mma_nvf4<CG>(d_tmem, a_lo + 2 * kb, b_lo + 2 * kb, ab_hi, idesc, t_sfa + kb * 4, t_sfb + kb * kSfbColsPerMma,
                                             (kt > k0 || kb > 0) ? 1u : 0u);
                    }
                    // the slot is reusable (in both CTAs) once these MMAs and copies retire
                    if constexpr (CG == 2) ptx::tc_commit_pair(bar_empty + stage * 8, 0x3);
                    else ptx::tc_commit(bar_empty + stage * 8);
                    if (kt + 1 == k1) {  // last k-tile of the segment: publish the accumulator
                        if constexpr (CG == 2) ptx::tc_commit_pair(bar_acc_full + acc * 8, 0x3);
                        else ptx::tc_commit(bar_acc_full + acc * 8);
                    }
                    ++sf_it;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                ++acc_it;
            }
            }
            __syncwarp();
        }
        // (the second CTA of a pair has nothing to issue: the leader's instructions drive both)
    } else {
        // ------------------------------------------------------------ epilogue
        const int quad = warp & 3;             // TMEM lane quadrant this warp may read
        const int row_in_tile = quad * 32 + lane;
        const int epi_tid = threadIdx.x - 64;  // 0..127
        uint32_t acc_it = 0;
        uint32_t store_buf = 0;
        // NVFP4 output: whether 32-byte code stores and 4-byte scale stores are aligned
        const bool wide_packed = EPI_EX && ((reinterpret_cast<uintptr_t>(p.out_packed) | static_cast<uintptr_t>(p.out_packed_row_stride) |
                                              static_cast<uintptr_t>(p.out_packed_batch_stride)) & 31u) == 0;
        const bool wide_sf = EPI_EX && ((reinterpret_cast<uintptr_t>(p.out_sf) | static_cast<uintptr_t>(p.out_sf_row_stride) |
                                          static_cast<uintptr_t>(p.out_sf_batch_stride)) & 3u) == 0;
        Segment seg;
        for (int si = 0; plan.at(si, &seg); ++si) {
            const int tile = seg.tile;
            const int k0 = seg.u0 - tile * KT;
            const int k1 = k0 + (seg.u1 - seg.u0);
            const TileCoord tc = (si == 0) ? first_tc : tile_coords(tile, n_workers, KT, p.total_units, p.tiles_m, p.tiles_n, (KS > 1) ? 0 : p.raster_rows);
            const int nb = tc.nt;
            const int mb = tc.mt * CG + cta_rank;
            const int l = tc.l;
            const uint32_t acc = acc_it % kNumAcc;
            const uint32_t acc_phase = (acc_it / kNumAcc) & 1u;
            // All 128 epilogue threads take the same branch: the outcome of the wait is agreed on
            // through a barrier, so a thread that gave up cannot strand the others at a later one.
            bool got_acc;
            {
                got_acc = ptx::mbar_wait_bounded(bar_acc_full + acc * 8, acc_phase, abort_flag, timeout);
            }
            if (!ptx::named_bar_and(2, 128, got_acc)) break;
            ptx::tc_fence_after();
            const uint32_t t_acc = tmem_base + acc * S::kAccStride + (static_cast<uint32_t>(quad * 32) << 16);
            // drain order: position p reads chunk (p + first_chunk) mod kChunks, so that the half an
            // overlapped accumulator shares with the other one comes first
            const int first_chunk = (kAccOverlap && acc == 0) ? kChunks / 2 : 0;
            auto chunk_at = [&](int pos) { return (pos + first_chunk) & (kChunks - 1); };
            const bool whole_tile = (k1 - k0 == KT);
            const int row = mb * kBM + row_in_tile;
            const long long c_off = l * p.c_batch_stride + static_cast<long long>(row) * p.c_row_stride + nb * BN;
            auto store8 = [&](int col, uint4 q) {  // eight fp16 of this thread's row, to the local C and every peer's
                *reinterpret_cast<uint4*>(p.c + c_off + col) = q;
                for (int r = 0; r < p.n_peer; ++r) *reinterpret_cast<uint4*>(p.c_peer[r] + c_off + col) = q;
            };
            // 32 finished columns [c0, c0 + 32) of this thread's row, fp32: the plain kernels round to
            // fp16 and store; the extended epilogue adds the bias, applies the activation and writes
            // fp16 or NVFP4.  The NVFP4 form quantises the fp16-ROUNDED values, so the result equals
            // the stand-alone quantiser run on the fp16 output.
            // (extended epilogue) bias and activation on 32 columns starting at global column gcol
            auto bias_act32 = [&](int gcol, float (&s)[32]) {
                if (p.bias != nullptr) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 b8 = *reinterpret_cast<const uint4*>(p.bias + gcol + 8 * j);
                        const uint32_t w[4] = {b8.x, b8.y, b8.z, b8.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                            s[8 * j + 2 * e] = __fadd_rn(s[8 * j + 2 * e], f.x);
                            s[8 * j + 2 * e + 1] = __fadd_rn(s[8 * j + 2 * e + 1], f.y);
                        }
                    }
                }
                if (p.activation == kActRelu) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) s[i] = fmaxf(s[i], 0.f);
                } else if (p.activation == kActSilu) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) s[i] = __fdividef(s[i], 1.f + __expf(-s[i]));
                }
            };
            // 32 values -> 16 bytes of e2m1 codes and the two e4m3 scale bytes (low byte = lower columns)
            auto quantize32 = [&](const float (&s)[32], uint32_t (&q)[4]) {
                uint32_t sf2 = 0u;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float v[16];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {   // round to fp16 and back, two at a time
                        const float2 f = __half22float2(__floats2half2_rn(s[16 * h + 2 * i], s[16 * h + 2 * i + 1]));
                        v[2 * i] = f.x;
                        v[2 * i + 1] = f.y;
                    }
                    uint32_t o[2];
                    sf2 |= static_cast<uint32_t>(quantize_block16(v, o)) << (8 * h);
                    q[2 * h] = o[0];
                    q[2 * h + 1] = o[1];
                }
                return sf2;
            };
            auto packed_at = [&](int gcol) {
                return p.out_packed + l * p.out_packed_batch_stride + static_cast<long long>(row) * p.out_packed_row_stride + gcol / 2;
            };
            auto sf_plain_at = [&](int gcol) { return p.out_sf + l * p.out_sf_batch_stride + static_cast<long long>(row) * p.out_sf_row_stride + gcol / 16; };
            auto sf_perm_at = [&](int gcol) {   // scale of (row, 16-column block gcol / 16) in the 128 x 4 atom layout
                const int blk = gcol / 16;
                return p.out_sf_perm + l * p.out_sf_perm_batch_stride + (row / 128) * p.out_sf_perm_block_stride + (blk / 4) * 512 + (row % 32) * 16 +
                       ((row / 32) % 4) * 4 + (blk % 4);
            };
            auto emit32 = [&](int c0, float (&s)[32]) {
                if constexpr (!EPI_EX) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) store8(c0 + 8 * j, pack8_fp16(&s[8 * j]));
                } else {
                    const int gcol = nb * BN + c0;
                    bias_act32(gcol, s);
                    if (!p.out_nvfp4) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) store8(c0 + 8 * j, pack8_fp16(&s[8 * j]));
                    } else {
                        uint32_t q[4];
                        const uint16_t sf2 = static_cast<uint16_t>(quantize32(s, q));   // two scales: neighbours in both layouts
                        *reinterpret_cast<uint4*>(packed_at(gcol)) = make_uint4(q[0], q[1], q[2], q[3]);
                        if (p.out_sf != nullptr) *reinterpret_cast<uint16_t*>(sf_plain_at(gcol)) = sf2;
                        if (p.out_sf_perm != nullptr) *reinterpret_cast<uint16_t*>(sf_perm_at(gcol)) = sf2;
                    }
                }
            };
            // 64 columns [c0, c0 + 64), c0 a multiple of 64.  The NVFP4 form then has 32 bytes of codes
            // (one full sector) and the four scales of one unit of either scale layout: one store
            // each where the addresses allow it, instead of twice two partial ones.
            auto emit64 = [&](int c0, float (&sa)[32], float (&sb)[32]) {
                if constexpr (!EPI_EX) {
                    emit32(c0, sa);
                    emit32(c0 + 32, sb);
                } else {
                    if (!p.out_nvfp4) {
                        emit32(c0, sa);
                        emit32(c0 + 32, sb);
                        return;
                    }
                    const int gcol = nb * BN + c0;
                    bias_act32(gcol, sa);
                    bias_act32(gcol + 32, sb);
                    uint32_t qa[4], qb[4];
                    const uint32_t sf4 = quantize32(sa, qa) | (quantize32(sb, qb) << 16);
                    uint8_t* dst = packed_at(gcol);
                    if (wide_packed) {
                        ptx::st_global_32B(dst, qa[0], qa[1], qa[2], qa[3], qb[0], qb[1], qb[2], qb[3]);
                    } else {
                        *reinterpret_cast<uint4*>(dst) = make_uint4(qa[0], qa[1], qa[2], qa[3]);
                        *reinterpret_cast<uint4*>(dst + 16) = make_uint4(qb[0], qb[1], qb[2], qb[3]);
                    }
                    if (p.out_sf != nullptr) {
                        if (wide_sf) {
                            *reinterpret_cast<uint32_t*>(sf_plain_at(gcol)) = sf4;
                        } else {
                            *reinterpret_cast<uint16_t*>(sf_plain_at(gcol)) = static_cast<uint16_t>(sf4);
                            *reinterpret_cast<uint16_t*>(sf_plain_at(gcol + 32)) = static_cast<uint16_t>(sf4 >> 16);
                        }
                    }
                    if (p.out_sf_perm != nullptr) *reinterpret_cast<uint32_t*>(sf_perm_at(gcol)) = sf4;   // (16-byte aligned atoms: always aligned)
                }
            };
            auto release_acc = [&]() {
                ptx::tc_fence_before();
                const uint32_t bar = bar_acc_empty + (kAccOverlap ? 0u : acc * 8);
                if (CG == 2 && !leader) ptx::mbar_arrive_cluster_signal(bar, 0);
                else ptx::mbar_arrive(bar);
            };

            if constexpr (KS > 1) {
                constexpr int kMyCols = BN / KS;                     // columns this CTA finalises
                constexpr uint32_t kPieceBytes = S::kPieceBytes;     // one sender's columns, [col/4][128 rows][4]
                // Piece of rank r at rank q: q keeps the KS - 1 foreign pieces in rank order.
                auto slot_of = [](int r, int q) { return r - (r > q ? 1 : 0); };
                // The partial sums land in the operand ring, which is idle once a CTA's own MMAs
                // are done (the accumulator is ready): every CTA tells its peers so, and nobody
                // sends before all peers have said it.
                const uint32_t land = smem_base;                                   // incoming pieces
                const float* land_gen = reinterpret_cast<const float*>(smem_gen);
                if (!cluster_waited) { ptx::cluster_wait(); cluster_waited = true; }   // peers are resident and initialised
                if constexpr (S::kGlobalExchange) {
                    // The columns the peers finalise go TMEM -> registers -> this CTA's scratch slot in
                    // global memory (one 128 KB slot per CTA: [destination][col/4][128 rows][4]); a
                    // device-scope fence and one arrival on every peer's barrier publish them, and
                    // each CTA then reads its columns of the peers' slots back through L2.
                    float* my_slot = p.scratch + static_cast<long long>(blockIdx.x) * kScratchSlotFloats;
#pragma unroll 1
                    for (int q = 0; q < KS; ++q) {
                        if (q == ks_rank) continue;
                        float* dst = my_slot + slot_of(q, ks_rank) * (kPieceBytes / 4) + row_in_tile * 4;
#pragma unroll 1
                        for (int c0 = 0; c0 < kMyCols; c0 += 32) {
                            uint32_t v[32];
                            ptx::tc_ld_32cols(t_acc + q * kMyCols + c0, v);
                            ptx::tc_wait_ld();
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                ptx::st_cg_v4(dst + (c0 / 4 + j) * (kBM * 4),
                                              make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                          __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
                        }
                    }
                    __threadfence();
                    ptx::named_bar_sync(1, 128);
                }
                if (epi_tid == 0) {
                    if constexpr (S::kBulkExchange && !S::kGlobalExchange) ptx::mbar_expect_tx(bar_land, (KS - 1) * kPieceBytes);   // before anybody may send
                    for (int q = 0; q < KS; ++q)
                        if (q != ks_rank) ptx::mbar_arrive_cluster(bar_ready, q);
                }
                if constexpr (S::kGlobalExchange) {
                    // (nothing to send: the arrival above told the peers that this CTA's slot is complete)
                } else if constexpr (S::kBulkExchange) {
                    // 1. The columns the peers finalise go TMEM -> registers -> this CTA's own shared
                    //    memory (behind the landing area), and from there to each peer as ONE bulk
                    //    copy through distributed shared memory that completes on the peer's landing
                    //    barrier.  (Storing the registers straight into the peer's shared memory,
                    //    16 bytes per thread and instruction, took about 150 cycles per warp
                    //    instruction: 2500 cycles for 32 KB.)
                    const uint32_t outb = smem_base + (KS - 1) * kPieceBytes;      // outgoing pieces
                    float* outb_gen = reinterpret_cast<float*>(smem_gen + (KS - 1) * kPieceBytes);
#pragma unroll 1
                    for (int q = 0; q < KS; ++q) {
                        if (q == ks_rank) continue;
                        float* dst = outb_gen + slot_of(q, ks_rank) * (kPieceBytes / 4) + row_in_tile * 4;
#pragma unroll 1
                        for (int c0 = 0; c0 < kMyCols; c0 += 32) {
                            uint32_t v[32];
                            ptx::tc_ld_32cols(t_acc + q * kMyCols + c0, v);
                            ptx::tc_wait_ld();
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *reinterpret_cast<uint4*>(dst + (c0 / 4 + j) * (kBM * 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        }
                    }
                    ptx::fence_proxy_async_smem();      // these writes are read by the bulk copies (async proxy)
                    ptx::named_bar_sync(1, 128);
                    if (epi_tid == 0) {
                        if (ptx::mbar_wait_bounded<true>(bar_ready, 0u, abort_flag, timeout)) {
                            for (int q = 0; q < KS; ++q)
                                if (q != ks_rank)
                                    ptx::bulk_copy_to_cluster(ptx::mapa_u32(land + slot_of(ks_rank, q) * kPieceBytes, q),
                                                              outb + slot_of(q, ks_rank) * kPieceBytes, kPieceBytes, ptx::mapa_u32(bar_land, q));
                        }
                    }
                } else {
                    const bool peers_ready = ptx::mbar_wait_bounded<true>(bar_ready, 0u, abort_flag, timeout);
                    if (!ptx::named_bar_and(2, 128, peers_ready)) break;
                    // 1. send every peer the columns it finalises, 16 bytes per thread and store
#pragma unroll 1
                    for (int q = 0; q < KS; ++q) {
                        if (q == ks_rank) continue;
                        const uint32_t dst = ptx::mapa_u32(land + slot_of(ks_rank, q) * kPieceBytes + row_in_tile * 16, q);
#pragma unroll 1
                        for (int c0 = 0; c0 < kMyCols; c0 += 32) {
                            uint32_t v[32];
                            ptx::tc_ld_32cols(t_acc + q * kMyCols + c0, v);
                            ptx::tc_wait_ld();
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                ptx::st_shared_cluster_v4(dst + (c0 / 4 + j) * (kBM * 16), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        }
                        ptx::mbar_arrive_cluster(bar_land, q);  // release: my stores above are visible to q
                    }
                }
                // 2. wait for the other CTAs' partial sums of my columns
                const bool landed = S::kGlobalExchange ? ptx::mbar_wait_bounded<true>(bar_ready, 0u, abort_flag, timeout)
                                                       : ptx::mbar_wait_bounded<true>(bar_land, 0u, abort_flag, timeout);
                if (!ptx::named_bar_and(2, 128, landed)) break;
                // 3. sum in ascending rank order (my own term comes from TMEM) and store fp16
#pragma unroll 1
                for (int c0 = 0; c0 < kMyCols; c0 += 32) {
                    uint32_t v[32];
                    ptx::tc_ld_32cols(t_acc + ks_rank * kMyCols + c0, v);
                    ptx::tc_wait_ld();
                    float s[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) s[i] = 0.f;
#pragma unroll 1
                    for (int r = 0; r < KS; ++r) {
                        if (r == ks_rank) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) s[i] += __uint_as_float(v[i]);
                        } else if constexpr (S::kGlobalExchange) {
                            const float* src = p.scratch + static_cast<long long>(blockIdx.x - ks_rank + r) * kScratchSlotFloats +
                                               slot_of(ks_rank, r) * (kPieceBytes / 4) + (c0 / 4) * (kBM * 4) + row_in_tile * 4;
                            float4 t[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) t[j] = ptx::ld_cg_v4(src + j * (kBM * 4));
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                s[4 * j] += t[j].x; s[4 * j + 1] += t[j].y; s[4 * j + 2] += t[j].z; s[4 * j + 3] += t[j].w;
                            }
                        } else {
                            const float* src = land_gen + slot_of(r, ks_rank) * (kPieceBytes / 4) + (c0 / 4) * (kBM * 4) + row_in_tile * 4;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float4 t = *reinterpret_cast<const float4*>(src + j * (kBM * 4));
                                s[4 * j] += t.x; s[4 * j + 1] += t.y; s[4 * j + 2] += t.z; s[4 * j + 3] += t.w;
                            }
                        }
                    }
                    if (row < p.M) emit32(ks_rank * kMyCols + c0, s);
                }
                release_acc();
            } else if (TMA_STORE && whole_tile) {
                if constexpr (TMA_STORE) {
                    // 64 columns (128 bytes of fp16) at a time through a swizzled 32-row staging buffer.
                    uint8_t* staging_gen = smem_gen + S::kEpiOff + (warp - 2) * S::kStagingPerWarp;
                    const uint32_t staging = smem_base + S::kEpiOff + (warp - 2) * S::kStagingPerWarp;
                    // Phase 1, drain: the whole accumulator row of this thread goes TMEM -> registers
                    // -> fp16 pairs (BN/2 registers), the loads of the next 32 columns in flight while
                    // the previous ones are converted.  The accumulator is handed back to the MMA warp
                    // as soon as the last column is in registers, before anything is stored: the TMA
                    // stores queue behind the producer's loads in the same TMA unit and are slow to
                    // free their staging buffer.
                    uint32_t packed[BN / 2];          // by drain position
                    uint32_t v[2][32];
                    ptx::tc_ld_32cols(t_acc + chunk_at(0) * 32, v[0]);
#pragma unroll
                    for (int pos = 0; pos < kChunks; ++pos) {
                        ptx::tc_wait_ld();
                        if (pos + 1 < kChunks) ptx::tc_ld_32cols(t_acc + chunk_at(pos + 1) * 32, v[(pos + 1) & 1]);
                        if (pos + 1 == kReleaseAfter) release_acc();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const __half2 h = __floats2half2_rn(__uint_as_float(v[pos & 1][2 * j]), __uint_as_float(v[pos & 1][2 * j + 1]));
                            packed[pos * 16 + j] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                    }
                    // Phase 2, store: 64 columns (128 bytes of fp16) at a time through the swizzled
                    // 32-row staging buffers, overlapping the next tile's MMAs.
#pragma unroll
                    for (int ci = 0; ci < BN / 64; ++ci) {
                        // the buffer about to be overwritten was read by the store issued kStagingBufs chunks ago
                        if (lane == 0) ptx::bulk_wait_group_read<S::kStagingBufs - 1>();
                        __syncwarp();
                        uint8_t* buf = staging_gen + store_buf * 4096 + lane * 128;
#pragma unroll
                        for (int j = 0; j < 8; ++j)  // 16-byte pieces, 128-byte swizzle
                            *reinterpret_cast<uint4*>(buf + ((j ^ (lane & 7)) << 4)) =
                                make_uint4(packed[ci * 32 + 4 * j], packed[ci * 32 + 4 * j + 1], packed[ci * 32 + 4 * j + 2], packed[ci * 32 + 4 * j + 3]);
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && mb * kBM + quad * 32 < p.M) {  // rows past M inside the box are clipped; one fixed lane owns the bulk groups
                            ptx::tma_store_3d(&p.tma_c, staging + store_buf * 4096, nb * BN + chunk_at(2 * ci) * 32, mb * kBM + quad * 32, l);
                            if (p.peer_tma)   // the same block to every peer, in the same bulk group: the buffer is free when all have read it
                                for (int r = 0; r < p.n_peer; ++r)
                                    ptx::tma_store_3d(&p.tma_c_peer[r], staging + store_buf * 4096, nb * BN + chunk_at(2 * ci) * 32, mb * kBM + quad * 32, l);
                            ptx::bulk_commit_group();
                        }
                        if (p.n_peer > 0 && !p.peer_tma) {
                            // Peers get the same 32 x 128-byte block with plain vector stores read back
                            // from the staging buffer: a warp instruction covers four full 128-byte
                            // rows.  (With a tensor store per peer instead, the stores crawled once
                            // there were more than a few destinations' tensor maps in play.)
                            const int sub = lane >> 3, piece = lane & 7;
                            uint4 q[8];
#pragma unroll
                            for (int it = 0; it < 8; ++it) {
                                const int rr = it * 4 + sub;
                                q[it] = *reinterpret_cast<const uint4*>(staging_gen + store_buf * 4096 + rr * 128 + ((piece ^ (rr & 7)) << 4));
                            }
                            const int row_base = mb * kBM + quad * 32;
                            for (int pi = 0; pi < p.n_peer; ++pi) {
                                const int r = (pi + static_cast<int>(blockIdx.x)) % p.n_peer;   // spread the start over CTAs
                                __half* dst = p.c_peer[r] + l * p.c_batch_stride + nb * BN + chunk_at(2 * ci) * 32 + piece * 8;
#pragma unroll
                                for (int it = 0; it < 8; ++it) {
                                    const int grow = row_base + it * 4 + sub;
                                    if (grow < p.M) *reinterpret_cast<uint4*>(dst + static_cast<long long>(grow) * p.c_row_stride) = q[it];
                                }
                            }
                        }
                        store_buf = (store_buf + 1u) % S::kStagingBufs;
                    }
                }
            } else {
                // A tile shared with other workers: whoever holds the START of the tile's k-range
                // finishes the tile; everyone else publishes an fp32 partial.  The others hold the
                // tile at the start of their ranges and contract it first of all, the finisher holds
                // it at the end of its range and contracts it last but one.  Whole tiles of the
                // kernels that store without TMA take the finisher's path too, with nobody else's
                // partials to add: one copy of the (long, when it re-quantises) store code serves both,
                // and the path that runs once per launch does not fetch 30 KB of cold instructions.
                const int w_first = whole_tile ? worker : unit_owner(tile * KT, n_workers, p.total_units);
                int* counter = p.counters + w_first * CG + cta_rank;
                if (k0 > 0) {
                    // Publish.  Slot layout [BN/4][128 rows][4] keeps every warp-wide 16-byte access
                    // contiguous (512 bytes) and a 32-column chunk contiguous (16 KB).  What the
                    // hand-back waits for goes to registers first.
                    float* my_slot = p.scratch + static_cast<long long>(partial_slot(worker, k0, CG, cta_rank)) * (kBM * BN);
                    auto publish32 = [&](int c0, const uint32_t (&v)[32]) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            ptx::st_cg_v4(my_slot + ((c0 / 4 + j) * kBM + row_in_tile) * 4,
                                          make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                      __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
                    };
                    if constexpr (kAccOverlap) {
                        uint32_t held[kReleaseAfter][32];
#pragma unroll
                        for (int pos = 0; pos < kReleaseAfter; ++pos) ptx::tc_ld_32cols(t_acc + chunk_at(pos) * 32, held[pos]);
                        ptx::tc_wait_ld();
                        release_acc();  // the MMA warp may start the next tile now
#pragma unroll
                        for (int pos = 0; pos < kReleaseAfter; ++pos) publish32(chunk_at(pos) * 32, held[pos]);
                    }
#pragma unroll 1
                    for (int pos = kAccOverlap ? kReleaseAfter : 0; pos < kChunks; ++pos) {
                        const int c0 = chunk_at(pos) * 32;
                        uint32_t v[32];
                        ptx::tc_ld_32cols(t_acc + c0, v);
                        ptx::tc_wait_ld();
                        publish32(c0, v);
                    }
                    if constexpr (!kAccOverlap) release_acc();
                    __threadfence();
                    ptx::named_bar_sync(1, 128);
                    if (epi_tid == 0) atomicAdd(counter, k1 - k0);
                } else {
                    // Finish: the rest of the k-range has been published (normally long ago); add
                    // those partials, read straight from L2, to this worker's accumulator in
                    // ascending worker order.  The operand ring keeps this SM's path from L2 busy,
                    // so a load issued here comes back after a microsecond or more: 64 columns of a
                    // contributor (64 registers) are requested before anything is added.
                    const int w_last = whole_tile ? w_first : unit_owner(tile * KT + KT - 1, n_workers, p.total_units);
                    const int need = KT - (k1 - k0);
                    // Everything the hand-back waits for goes to registers first (the half an
                    // overlapped accumulator shares with the other one, else all of it: at most four
                    // 32-column pieces), the accumulator is released, and only then anything is
                    // waited for, converted or stored.
                    uint32_t held[kReleaseAfter][32];
#pragma unroll
                    for (int pos = 0; pos < kReleaseAfter; ++pos) ptx::tc_ld_32cols(t_acc + chunk_at(pos) * 32, held[pos]);
                    ptx::tc_wait_ld();
                    release_acc();
                    if (!whole_tile) {
                        bool ready = true;
                        if (epi_tid == 0) {
                            const long long t_spin = clock64();
                            while (ptx::ld_acquire_gpu(counter) < need) {
                                if (*abort_flag || static_cast<uint64_t>(clock64() - t_spin) > timeout) {
                                    *abort_flag = 1u;
                                    ready = false;
                                    break;
                                }
                                __nanosleep(64);
                            }
                        }
                        if (!ptx::named_bar_and(1, 128, ready)) break;
                    }
                    static_assert(kChunks % 2 == 0 && kReleaseAfter % 2 == 0, "the partial sums are added 64 columns at a time");
                    // the columns [c0a, c0a + 32) and [c0b, c0b + 32) of this thread's row: own sums in, total out
                    auto add_others_and_emit = [&](int c0a, int c0b, float (&sa)[32], float (&sb)[32]) {
#pragma unroll 1
                        for (int w = w_first + 1; w <= w_last; ++w) {   // later contributors use their "head" slot
                            const float* src = p.scratch + static_cast<long long>(partial_slot(w, 1, CG, cta_rank)) * (kBM * BN) + row_in_tile * 4;
                            float4 ta[8], tb[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) ta[j] = ptx::ld_cg_v4(src + (c0a / 4 + j) * (kBM * 4));
#pragma unroll
                            for (int j = 0; j < 8; ++j) tb[j] = ptx::ld_cg_v4(src + (c0b / 4 + j) * (kBM * 4));
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                sa[4 * j] += ta[j].x; sa[4 * j + 1] += ta[j].y; sa[4 * j + 2] += ta[j].z; sa[4 * j + 3] += ta[j].w;
                                sb[4 * j] += tb[j].x; sb[4 * j + 1] += tb[j].y; sb[4 * j + 2] += tb[j].z; sb[4 * j + 3] += tb[j].w;
                            }
                        }
                        if (row < p.M) emit64(c0a, sa, sb);   // (c0b == c0a + 32: drain positions pair up neighbouring chunks)
                    };
#pragma unroll
                    for (int pos = 0; pos < kReleaseAfter; pos += 2) {
                        float sa[32], sb[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) { sa[i] = __uint_as_float(held[pos][i]); sb[i] = __uint_as_float(held[pos + 1][i]); }
                        add_others_and_emit(chunk_at(pos) * 32, chunk_at(pos + 1) * 32, sa, sb);
                    }
#pragma unroll 1
                    for (int pos = kReleaseAfter; pos < kChunks; pos += 2) {
                        uint32_t va[32], vb[32];
                        ptx::tc_ld_32cols(t_acc + chunk_at(pos) * 32, va);
                        ptx::tc_ld_32cols(t_acc + chunk_at(pos + 1) * 32, vb);
                        ptx::tc_wait_ld();
                        float sa[32], sb[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) { sa[i] = __uint_as_float(va[i]); sb[i] = __uint_as_float(vb[i]); }
                        add_others_and_emit(chunk_at(pos) * 32, chunk_at(pos + 1) * 32, sa, sb);
                    }
                    if (!whole_tile && epi_tid == 0) *counter = 0;
                }
            }
            ++acc_it;
        }
        if constexpr (TMA_STORE) {
            if (lane == 0) ptx::bulk_wait_group<0>();  // staging must outlive the stores that read it
        }
    }

    // ---------------------------------------------------------------- teardown
    if (!cluster_waited) ptx::cluster_wait();  // the start-up cluster phase, for warps that had no reason to wait earlier
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
    if constexpr (CG == 2 || KS > 1) {
        // no CTA may retire (or free TMEM) while another can still issue pair-wide work or write
        // into its shared memory
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<CG>(tmem_base, kTmemCols);
    }
    if constexpr (CG == 2) {
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
}

}  // namespace nvfp4
