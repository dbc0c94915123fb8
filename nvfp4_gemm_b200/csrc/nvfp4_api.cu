// C ABI of the library (declared in include/nvfp4_b200.h): argument validation, tensor-map
// cache, per-device scratch, kernel selection and launch.  No allocation, tensor-map encoding
// or synchronisation happens on the steady-state path of nvfp4_gemm / nvfp4_gemv.
#include "../../include/nvfp4_b200.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "gemm_sm100.cuh"
#include "gemv_sm100.cuh"
#include "layout_kernels.cuh"

namespace {

using namespace nvfp4;

thread_local std::string t_error;
thread_local const char* t_last_kernel = "";
std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_timeout_ns{1000000000ull};

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    t_error = buf;
    return code;
}

#define CUDA_TRY(expr)                                                                             \
    do {                                                                                           \
        cudaError_t e__ = (expr);                                                                  \
        if (e__ != cudaSuccess) return fail(NVFP4_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct MapKey {
    const void* ptr;
    uint64_t dims[4];
    uint64_t strides[3];
    uint32_t box[4];
    int dtype;
    int rank;
    int swizzle;
    bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapEntry {
    MapKey key;
    CUtensorMap map;
};

constexpr int kMaxCtas = 160;                                          // persistent CTAs (one per SM; a B200 has 148)
constexpr size_t kSlotBytes = static_cast<size_t>(kBM) * 256 * sizeof(float);  // one 128 x 256 fp32 partial tile
constexpr size_t kScratchBytes = kMaxCtas * 2 * kSlotBytes;             // head + tail slot per CTA
// GEMMs on different streams may overlap on the GPU, so the partial-tile scratch and the tile
// counters are per stream: a fixed number of sets is allocated with the first GEMM on a device
// and handed to streams as they show up (no allocation then, so a stream may first be seen
// inside a graph capture).  A set stays with its stream until nvfp4_release_stream(); when all
// are taken, sets of streams that have gone idle are taken back -- except sets that were used
// while their stream was being captured: a graph may replay those launches at any later time.
constexpr int kStreamSets = 8;

struct DeviceCtx {
    int device = -1;
    int num_sms = 0;
    bool sm100 = false;
    float* scratch = nullptr;    // kStreamSets sets of partial-tile slots
    int* counters = nullptr;     // kStreamSets sets of tile counters
    cudaStream_t set_stream[kStreamSets] = {};
    bool set_used[kStreamSets] = {};
    bool set_in_graph[kStreamSets] = {};   // a launch with this set was recorded into a CUDA graph
    int* status_host = nullptr;
    int* status_dev = nullptr;
    size_t scratch_bytes = 0;
    int max_pairs = -1;  // CTA pairs that can be co-resident (cluster occupancy), queried once
    std::vector<MapEntry> maps;
    bool smem_attr_set[24] = {};
};

std::mutex g_mutex;
DeviceCtx* g_ctx[64] = {nullptr};
EncodeTiledFn g_encode = nullptr;

int get_ctx(DeviceCtx** out) {
    int dev = -1;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(NVFP4_ERR_CUDA, "unexpected device ordinal %d", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_ctx[dev]) {
        cudaDeviceProp prop;
        CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
        DeviceCtx* c = new DeviceCtx();
        c->device = dev;
        c->num_sms = prop.multiProcessorCount;
        c->sm100 = (prop.major == 10);
        CUDA_TRY(cudaHostAlloc(reinterpret_cast<void**>(&c->status_host), sizeof(int), cudaHostAllocMapped));
        *c->status_host = 0;
        CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void**>(&c->status_dev), c->status_host, 0));
        g_ctx[dev] = c;
    }
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess)
            return fail(NVFP4_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    *out = g_ctx[dev];
    return NVFP4_OK;
}

int ensure_scratch(DeviceCtx* c) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (c->scratch) return NVFP4_OK;
    // Partial-tile slots need no initialisation (they are written before they are read); the
    // per-tile counters must be zero between launches.
    CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&c->scratch), kStreamSets * kScratchBytes));
    CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&c->counters), kStreamSets * kMaxCtas * sizeof(int)));
    CUDA_TRY(cudaMemset(c->counters, 0, kStreamSets * kMaxCtas * sizeof(int)));
    CUDA_TRY(cudaDeviceSynchronize());
    c->scratch_bytes = kStreamSets * (kScratchBytes + kMaxCtas * sizeof(int));
    return NVFP4_OK;
}

// The scratch set of `stream` on this device.
int scratch_set_for(DeviceCtx* c, cudaStream_t stream, int* set) {
    std::lock_guard<std::mutex> lock(g_mutex);
    for (int i = 0; i < kStreamSets; ++i)
        if (c->set_used[i] && c->set_stream[i] == stream) {
            *set = i;
            if (!c->set_in_graph[i]) {   // (once set, the flag stays: nothing more to find out)
                cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
                if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone) c->set_in_graph[i] = true;
            }
            return NVFP4_OK;
        }
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    CUDA_TRY(cudaStreamIsCapturing(stream, &cap));
    const bool capturing = (cap != cudaStreamCaptureStatusNone);
    for (int pass = 0; pass < 2; ++pass) {
        for (int i = 0; i < kStreamSets; ++i)
            if (!c->set_used[i]) {
                c->set_used[i] = true;
                c->set_stream[i] = stream;
                c->set_in_graph[i] = capturing;
                *set = i;
                return NVFP4_OK;
            }
        // All taken.  Outside a capture (stream queries are not allowed during one), take back the
        // sets of streams whose work is complete and that no graph refers to.
        if (capturing || pass == 1) break;
        for (int i = 0; i < kStreamSets; ++i)
            if (c->set_used[i] && !c->set_in_graph[i] && cudaStreamQuery(c->set_stream[i]) != cudaErrorNotReady) c->set_used[i] = false;
        (void)cudaGetLastError();   // a query of a stream that was destroyed meanwhile leaves an error behind
    }
    return fail(NVFP4_ERR_UNSUPPORTED,
                "all %d scratch sets of device %d belong to busy streams or to streams that were captured into graphs: "
                "call nvfp4_release_stream() for streams (and graphs) that are done",
                kStreamSets, c->device);
}

// Tensor maps are cached by (pointer, extents, strides, box): re-encoding four maps per call,
// as the reference does (s_128t.py:569-577), costs more than a short GEMM.
int get_map(DeviceCtx* c, const MapKey& key, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_mutex);
    for (const MapEntry& e : c->maps)
        if (e.key == key) {
            *out = e.map;
            return NVFP4_OK;
        }
    MapEntry e;
    std::memset(&e, 0, sizeof(e));
    e.key = key;
    cuuint64_t dims[4] = {key.dims[0], key.dims[1], key.dims[2], key.dims[3]};
    cuuint64_t strides[3] = {key.strides[0], key.strides[1], key.strides[2]};
    cuuint32_t box[4] = {key.box[0], key.box[1], key.box[2], key.box[3]};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUresult r = g_encode(&e.map, static_cast<CUtensorMapDataType>(key.dtype), key.rank, const_cast<void*>(key.ptr), dims,
                          strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, static_cast<CUtensorMapSwizzle>(key.swizzle),
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(NVFP4_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d) rank %d dims {%llu,%llu,%llu,%llu} strides {%llu,%llu,%llu}",
                    static_cast<int>(r), key.rank, (unsigned long long)dims[0], (unsigned long long)dims[1],
                    (unsigned long long)dims[2], (unsigned long long)dims[3], (unsigned long long)strides[0],
                    (unsigned long long)strides[1], (unsigned long long)strides[2]);
    if (c->maps.size() >= 256) c->maps.erase(c->maps.begin());
    c->maps.push_back(e);
    *out = e.map;
    return NVFP4_OK;
}

// Operand / output tiles: {inner extent, rows, batches}, 128-byte swizzle.
MapKey make_key(const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s0, uint64_t s1, uint32_t b0, uint32_t b1,
                int dtype) {
    MapKey k;
    std::memset(&k, 0, sizeof(k));
    k.ptr = ptr;
    k.dims[0] = d0; k.dims[1] = d1; k.dims[2] = d2;
    k.strides[0] = s0; k.strides[1] = s1;
    k.box[0] = b0; k.box[1] = b1; k.box[2] = 1;
    k.dtype = dtype;
    k.rank = 3;
    k.swizzle = CU_TENSOR_MAP_SWIZZLE_128B;
    return k;
}

// Permuted scale factors: 512-byte atoms (128 words), K/64 atoms per 128-row block, un-swizzled
// (tcgen05.cp reads them as 32 rows of 16 bytes).  Box = the four atoms of one 256-wide k-tile
// for `blocks` consecutive row blocks.
MapKey make_sf_key(const void* ptr, int rows, int k, int l, uint64_t batch_stride, uint32_t blocks) {
    MapKey key;
    std::memset(&key, 0, sizeof(key));
    const uint64_t atoms_k = static_cast<uint64_t>(k) / 64;
    const uint64_t row_blocks = (static_cast<uint64_t>(rows) + 127) / 128;
    key.ptr = ptr;
    key.dims[0] = kSfAtomBytes / 4; key.dims[1] = atoms_k; key.dims[2] = row_blocks; key.dims[3] = l;
    key.strides[0] = kSfAtomBytes; key.strides[1] = atoms_k * kSfAtomBytes;
    key.strides[2] = l > 1 ? batch_stride : row_blocks * atoms_k * kSfAtomBytes;
    key.box[0] = kSfAtomBytes / 4; key.box[1] = kMmaPerStage; key.box[2] = blocks; key.box[3] = 1;
    key.dtype = CU_TENSOR_MAP_DATA_TYPE_UINT32;
    key.rank = 4;
    key.swizzle = CU_TENSOR_MAP_SWIZZLE_NONE;
    return key;
}

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Whole tiles per worker, or an even split of all (tile, k-tile) units with shared tiles summed
// through scratch?  In k-tiles of run time: whole tiles cost waves x k_tiles; the even split costs
// units / workers plus the summing, which hides behind later whole tiles when a worker has at
// least two tiles' worth of units and otherwise ends the launch (publish, wait, read back:
// measured about as long as 24 k-tiles of the 256-wide pair kernel with two workers per tile --
// 768 x 4096 x 4096 took 19.5 us split 74 ways and 10.6 us as 48 whole tiles -- and counted as 12
// k-tiles per worker that shares a tile).
struct WorkSplit {
    double cost;        // k-tiles of run time
    int workers;
    bool whole_tiles;
};
WorkSplit plan_work_split(long long tiles, int k_tiles, int max_workers) {
    const long long whole_workers_max = tiles < max_workers ? tiles : max_workers;
    const long long waves = (tiles + whole_workers_max - 1) / whole_workers_max;
    const double cost_whole = static_cast<double>(waves) * k_tiles;
    const double share = static_cast<double>(tiles) * k_tiles / max_workers;
    const double per_tile = static_cast<double>(k_tiles) / (share < 1.0 ? 1.0 : share);   // workers that share a tile, about
    const double cost_split = share + (share >= 2.0 * k_tiles ? 3.0 : 12.0 * (per_tile < 2.0 ? 2.0 : per_tile));
    if (cost_whole <= cost_split) return WorkSplit{cost_whole, static_cast<int>((tiles + waves - 1) / waves), true};   // the fewest workers that need no more waves
    return WorkSplit{cost_split, max_workers, false};
}

template <int CG, int BN, int STAGES, bool TMA_STORE, int EPI_KB, bool EPI_EX = false>
int launch_gemm(DeviceCtx* c, int variant, GemmParams& params, int grid_request, cudaStream_t stream, const char* name) {
    using S = GemmSmem<CG, BN, STAGES, TMA_STORE, EPI_KB>;
    auto kernel = gemm_nvfp4_kernel<CG, BN, STAGES, TMA_STORE, EPI_KB, 1, EPI_EX>;
    if (!c->smem_attr_set[variant]) {
        CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamicBytes));
        c->smem_attr_set[variant] = true;
    }
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = S::kDynamicBytes;
    cfg.stream = stream;
    // programmatic dependent launch: the kernel's set-up may overlap the tail of the kernel before
    // it in the stream; it waits (griddepcontrol.wait) before its first global access
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int max_ctas = c->num_sms;
    if (CG == 2) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
        if (c->max_pairs < 0) {
            // All workers must be co-resident for the work split to be balanced: ask how many
            // CTA pairs the device can hold at once (an SM without a free neighbour stays idle).
            cfg.gridDim = dim3(c->num_sms & ~1, 1, 1);
            int n = 0;
            CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
            c->max_pairs = n > 0 ? n : 1;
        }
        max_ctas = 2 * c->max_pairs;
    }
    int grid = grid_request > 0 ? grid_request : max_ctas;
    if (grid > max_ctas) grid = max_ctas;
    if (grid > kMaxCtas) grid = kMaxCtas;
    int workers = grid / CG;
    if (grid_request <= 0) {
        const WorkSplit split = plan_work_split(params.total_units / params.k_tiles, params.k_tiles, workers);
        workers = split.workers;
        if (split.whole_tiles) {
            params.whole_tiles = 1;
            params.raster_rows = 0;
        }
    }
    if (workers > params.total_units) workers = params.total_units;
    if (workers < 1) workers = 1;
    grid = workers * CG;
    cfg.gridDim = dim3(grid, 1, 1);
    CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, params));
    g_launches.fetch_add(1);
    t_last_kernel = name;
    return NVFP4_OK;
}

// Cluster split-K launch: one cluster of KS CTAs per 128 x BN output tile.
template <int BN, int STAGES, int EPI_KB, int KS, bool EPI_EX = false>
int launch_gemm_splitk(DeviceCtx* c, int variant, GemmParams& params, cudaStream_t stream, const char* name) {
    using S = GemmSmem<1, BN, STAGES, false, EPI_KB, KS>;
    auto kernel = gemm_nvfp4_kernel<1, BN, STAGES, false, EPI_KB, KS, EPI_EX>;
    if (!c->smem_attr_set[variant]) {
        CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kDynamicBytes));
        c->smem_attr_set[variant] = true;
    }
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = S::kDynamicBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = KS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: the kernel's set-up may overlap the tail of the kernel before
    // it in the stream; it waits (griddepcontrol.wait) before its first global access
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    const int tiles = params.total_units / params.k_tiles;
    if (S::kGlobalExchange && tiles * KS > 2 * kMaxCtas)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "split_k = %d over %d tiles needs %d scratch slots, the library keeps %d: use split_k 1 or 2",
                    KS, tiles, tiles * KS, 2 * kMaxCtas);
    cfg.gridDim = dim3(tiles * KS, 1, 1);
    CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, params));
    g_launches.fetch_add(1);
    t_last_kernel = name;
    return NVFP4_OK;
}

__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long timeout_cycles) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        abort_flag = 0;
        ptx::fence_mbar_init();
        // Nothing ever arrives on this barrier: the wait has to give up by itself.
        const bool ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar), 0u, &abort_flag, timeout_cycles);
        if (!ok) {
            *reinterpret_cast<volatile int*>(status) = kStatusWaitTimeout;
            __threadfence_system();
        }
    }
}

int validate_common(const nvfp4_problem* p) {
    if (!p) return fail(NVFP4_ERR_INVALID_ARGUMENT, "problem is NULL");
    if (p->m < 1 || p->n < 1 || p->k < 1 || p->l < 1)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "m, n, k, l must be positive (got %d, %d, %d, %d)", p->m, p->n, p->k, p->l);
    if (!p->a || !p->b) return fail(NVFP4_ERR_INVALID_ARGUMENT, "a and b must not be NULL");
    return NVFP4_OK;
}

// Everything both GEMM entry points require of a problem, checked before any CUDA call.
int validate_gemm(const nvfp4_problem* p, bool needs_c = true) {
    if (int rc = validate_common(p)) return rc;
    if (needs_c && !p->c) return fail(NVFP4_ERR_INVALID_ARGUMENT, "c must not be NULL");
    if (!p->sfa_perm || !p->sfb_perm)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "the GEMM needs the permuted scale tensors (sfa_perm, sfb_perm)");
    if (p->k % kKPerStage) return fail(NVFP4_ERR_INVALID_ARGUMENT, "k must be a multiple of 256 (got %d)", p->k);
    if (p->n % 128) return fail(NVFP4_ERR_INVALID_ARGUMENT, "n must be a multiple of 128 (got %d)", p->n);
    if (!aligned(p->a, 16) || !aligned(p->b, 16) || !aligned(p->c, 16) || !aligned(p->sfa_perm, 16) || !aligned(p->sfb_perm, 16))
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "a, b, c, sfa_perm and sfb_perm must be 16-byte aligned");
    if (!needs_c && !p->c) return NVFP4_OK;     // no fp16 output: its strides mean nothing
    if (p->a_row_stride % 16 || p->b_row_stride % 16 || p->a_row_stride < p->k / 2 || p->b_row_stride < p->k / 2)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "row strides of a and b must be multiples of 16 bytes and >= k/2");
    if (p->c_row_stride % 8 || p->c_row_stride < p->n)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "c_row_stride must be a multiple of 8 elements and >= n");
    if (p->l > 1 && (p->a_batch_stride % 16 || p->b_batch_stride % 16 || p->c_batch_stride % 8 ||
                     p->sfa_perm_batch_stride % 16 || p->sfb_perm_batch_stride % 16))
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "batch strides must keep 16-byte alignment");
    return NVFP4_OK;
}

}  // namespace

namespace {
// Up to this many peers get their copies of the output by tensor stores (one per peer and staged
// block); more are served by the epilogue warps' own stores.
std::atomic<int> g_peer_tma_limit{1};
int peer_tma_limit() { return g_peer_tma_limit.load(); }

// Tile shape of the persistent kernels: what the caller fixed in cf, else this library's choice.
struct TileChoice {
    int cta_group, tile_n;
};
TileChoice choose_tile(int m, int n, int k, int l, int num_sms, const nvfp4_gemm_config& cf) {
    // A CTA pair (256-row tile, B shared through the pair) pays off as soon as there is more than
    // one 128-row block; decode shapes (m <= 128) stay on single CTAs.
    int cg = cf.cta_group;
    if (cg == 0) cg = (m > kBM && n % 256 == 0) ? 2 : 1;
    if (cf.cta_group == 0 && cf.tile_n == 0 && cg == 2 && cf.grid == 0 && cf.split_k <= 1) {
        // 256 x 256 tiles on CTA pairs do twice the work per SM and stage of 128 x 128 tiles on
        // single CTAs, but small problems fill more SMs with the small tiles and their epilogue is
        // shorter.  Estimated run time in k-tiles of the pair kernel (one of its stages ~ 0.35 us;
        // a 128-wide stage 0.9 of that, the epilogues of the last tile 9 and 4.5), constants fitted
        // to thirteen measured shapes from 256 x 7168 x 256 to 4096 x 7168 x 7168.
        const int k_tiles = k / kKPerStage;
        const long long tiles256 = static_cast<long long>((m + 2 * kBM - 1) / (2 * kBM)) * (n / 256) * l;
        const long long tiles128 = static_cast<long long>((m + kBM - 1) / kBM) * (n / 128) * l;
        const double cost_pair = plan_work_split(tiles256, k_tiles, num_sms / 2).cost + 9.0;
        const double cost_single = plan_work_split(tiles128, k_tiles, num_sms).cost * 0.9 + 4.5;
        if (cost_single < cost_pair) cg = 1;
    }
    int bn = cf.tile_n;
    if (bn == 0) {
        bn = (n % 256 == 0) ? 256 : 128;
        // single-CTA tiles that would leave SMs idle: halve the tile width to double the tile count
        const long long tiles256 = static_cast<long long>((m + kBM - 1) / kBM) * (n / 256) * l;
        if (cg == 1 && bn == 256 && (tiles256 < num_sms || (cf.cta_group == 0 && m > kBM))) bn = 128;
    }
    return TileChoice{cg, bn};
}

int gemm_impl(const nvfp4_problem* p, const nvfp4_gemm_config* cfg, const nvfp4_epilogue* epi, void* const* c_peers, int n_peers,
              void* stream_v) {
    const bool to_nvfp4 = epi && epi->output == NVFP4_OUT_NVFP4;
    if (int rc = validate_gemm(p, !to_nvfp4)) return rc;
    if (epi) {
        if (epi->activation < NVFP4_ACT_NONE || epi->activation > NVFP4_ACT_SILU)
            return fail(NVFP4_ERR_INVALID_ARGUMENT, "activation must be NVFP4_ACT_NONE, NVFP4_ACT_RELU or NVFP4_ACT_SILU");
        if (epi->output != NVFP4_OUT_FP16 && epi->output != NVFP4_OUT_NVFP4)
            return fail(NVFP4_ERR_INVALID_ARGUMENT, "output must be NVFP4_OUT_FP16 or NVFP4_OUT_NVFP4");
        if (epi->bias && !aligned(epi->bias, 16)) return fail(NVFP4_ERR_INVALID_ARGUMENT, "bias must be 16-byte aligned");
        if (n_peers > 0) return fail(NVFP4_ERR_UNSUPPORTED, "the fused all-gather writes fp16 without bias or activation");
        if (to_nvfp4) {
            if (!epi->out_packed || (!epi->out_sf && !epi->out_sf_perm))
                return fail(NVFP4_ERR_INVALID_ARGUMENT, "NVFP4 output needs out_packed and at least one of out_sf / out_sf_perm");
            if (!aligned(epi->out_packed, 16) || epi->out_packed_row_stride % 16 || epi->out_packed_row_stride < p->n / 2)
                return fail(NVFP4_ERR_INVALID_ARGUMENT, "out_packed must be 16-byte aligned with a row stride that is a multiple of 16 and >= n/2");
            if (epi->out_sf && (!aligned(epi->out_sf, 2) || epi->out_sf_row_stride % 2 || epi->out_sf_row_stride < p->n / 16))
                return fail(NVFP4_ERR_INVALID_ARGUMENT, "out_sf must be 2-byte aligned with an even row stride >= n/16");
            if (epi->out_sf_perm && !aligned(epi->out_sf_perm, 16))
                return fail(NVFP4_ERR_INVALID_ARGUMENT, "out_sf_perm must be 16-byte aligned");
            if (epi->out_sf_perm && epi->out_sf_perm_block_stride &&
                (epi->out_sf_perm_block_stride % 16 || epi->out_sf_perm_block_stride < static_cast<long long>(p->n / 64) * 512))
                return fail(NVFP4_ERR_INVALID_ARGUMENT, "out_sf_perm_block_stride must be 0 or a multiple of 16 that is >= (n/64)*512");
            const long long block_stride = epi->out_sf_perm_block_stride ? epi->out_sf_perm_block_stride : static_cast<long long>(p->n / 64) * 512;
            const long long perm_bytes = static_cast<long long>((p->m + 127) / 128 - 1) * block_stride + static_cast<long long>(p->n / 64) * 512;
            if (p->l > 1 && (epi->out_packed_batch_stride % 16 || epi->out_sf_batch_stride % 2 || epi->out_sf_perm_batch_stride % 16 ||
                             (epi->out_sf_perm && epi->out_sf_perm_batch_stride < perm_bytes)))
                return fail(NVFP4_ERR_INVALID_ARGUMENT, "output batch strides too small or misaligned");
        }
    }

    nvfp4_gemm_config cf = {0, 0, 0, 0, 0, 0};
    if (cfg) cf = *cfg;
    if (cf.tile_n != 0 && cf.tile_n != 128 && cf.tile_n != 256)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "tile_n must be 0, 128 or 256");
    if (cf.epilogue < 0 || cf.epilogue > 3) return fail(NVFP4_ERR_INVALID_ARGUMENT, "epilogue must be 0, 1, 2 or 3");
    if (cf.cta_group < 0 || cf.cta_group > 2) return fail(NVFP4_ERR_INVALID_ARGUMENT, "cta_group must be 0, 1 or 2");
    if (cf.split_k != 0 && cf.split_k != 1 && cf.split_k != 2 && cf.split_k != 4 && cf.split_k != 8)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "split_k must be 0, 1, 2, 4 or 8");
    if (cf.raster < -1 || cf.raster > 1024) return fail(NVFP4_ERR_INVALID_ARGUMENT, "raster must be -1 (off), 0 (auto) or a row-tile count");

    DeviceCtx* c = nullptr;
    if (int rc = get_ctx(&c)) return rc;
    if (!c->sm100) return fail(NVFP4_ERR_UNSUPPORTED, "device %d is not sm_100", c->device);
    if (int rc = ensure_scratch(c)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    const TileChoice choice = choose_tile(p->m, p->n, p->k, p->l, c->num_sms, cf);
    const int cg = choice.cta_group;
    int bn = choice.tile_n;
    if (p->n % bn) return fail(NVFP4_ERR_INVALID_ARGUMENT, "n = %d is not a multiple of tile_n = %d", p->n, bn);

    GemmParams g;
    std::memset(&g, 0, sizeof(g));
    g.M = p->m; g.N = p->n; g.K = p->k; g.L = p->l;
    g.tiles_m = (p->m + kBM * cg - 1) / (kBM * cg);
    g.tiles_n = p->n / bn;
    g.k_tiles = p->k / kKPerStage;
    const long long units = static_cast<long long>(g.tiles_m) * g.tiles_n * p->l * g.k_tiles;
    if (units > 0x7fffffffLL) return fail(NVFP4_ERR_INVALID_ARGUMENT, "problem too large: %lld work units", units);
    g.total_units = static_cast<int>(units);
    // Tile order of the persistent kernels: operands that fit L2 comfortably are read from DRAM
    // once whatever the order, and the plain order spreads the workers over distinct operand
    // blocks; larger ones are walked in column-major groups so that a wave of workers shares blocks.
    {
        const double operand_bytes = static_cast<double>(p->l) * (static_cast<double>(p->m) + p->n) * (p->k / 2);
        g.raster_rows = cf.raster > 0 ? cf.raster : (cf.raster == 0 && operand_bytes > 64e6) ? 16 : 0;
    }
    g.c = static_cast<__half*>(p->c);
    if (epi) {
        g.bias = static_cast<const __half*>(epi->bias);
        g.activation = epi->activation;
        g.out_nvfp4 = to_nvfp4 ? 1 : 0;
        if (to_nvfp4) {
            g.out_packed = static_cast<uint8_t*>(epi->out_packed);
            g.out_sf = static_cast<uint8_t*>(epi->out_sf);
            g.out_sf_perm = static_cast<uint8_t*>(epi->out_sf_perm);
            g.out_packed_row_stride = epi->out_packed_row_stride;
            g.out_packed_batch_stride = epi->out_packed_batch_stride;
            g.out_sf_row_stride = epi->out_sf_row_stride;
            g.out_sf_batch_stride = epi->out_sf_batch_stride;
            g.out_sf_perm_batch_stride = epi->out_sf_perm_batch_stride;
            g.out_sf_perm_block_stride = epi->out_sf_perm_block_stride ? epi->out_sf_perm_block_stride : static_cast<long long>(p->n / 64) * 512;
        }
    }
    int set = 0;
    if (int rc = scratch_set_for(c, stream, &set)) return rc;
    g.scratch = c->scratch + static_cast<size_t>(set) * (kScratchBytes / sizeof(float));
    g.counters = c->counters + set * kMaxCtas;
    g.status = c->status_dev;
    g.c_row_stride = p->c_row_stride;
    g.c_batch_stride = p->c_batch_stride;
    g.timeout_cycles = g_timeout_ns.load() * 2;  // SM clock <= 2 GHz: at least the requested time

    // Whole tiles leave through the TMA-store epilogue unless the caller asks for plain stores.
    int epilogue = cf.epilogue;
    if (epilogue == 0) epilogue = 2;
    if (epi) epilogue = 1;                     // the extended epilogue writes with plain stores
    if (epi && to_nvfp4 && g.out_sf_perm && p->m % 128) {
        // rows of the last 128-row block that do not exist must read as zero scales
        const long long last_block = static_cast<long long>((p->m + 127) / 128 - 1) * g.out_sf_perm_block_stride;
        const long long tail = static_cast<long long>(p->n / 64) * 512;
        for (int l = 0; l < p->l; ++l)
            CUDA_TRY(cudaMemsetAsync(g.out_sf_perm + l * g.out_sf_perm_batch_stride + last_block, 0, tail, stream));
    }

    const uint64_t kbytes = static_cast<uint64_t>(p->k) / 2;
    const uint64_t a_bs = p->l > 1 ? static_cast<uint64_t>(p->a_batch_stride) : static_cast<uint64_t>(p->a_row_stride) * p->m;
    const uint64_t b_bs = p->l > 1 ? static_cast<uint64_t>(p->b_batch_stride) : static_cast<uint64_t>(p->b_row_stride) * p->n;
    const uint64_t c_bs = p->l > 1 ? static_cast<uint64_t>(p->c_batch_stride) * 2 : static_cast<uint64_t>(p->c_row_stride) * 2 * p->m;
    if (int rc = get_map(c, make_key(p->a, kbytes, p->m, p->l, p->a_row_stride, a_bs, kBKBytes, kBM, CU_TENSOR_MAP_DATA_TYPE_UINT8),
                         &g.tma_a)) return rc;
    if (int rc = get_map(c, make_key(p->b, kbytes, p->n, p->l, p->b_row_stride, b_bs, kBKBytes, bn / cg, CU_TENSOR_MAP_DATA_TYPE_UINT8),
                         &g.tma_b)) return rc;
    if (int rc = get_map(c, make_sf_key(p->sfa_perm, p->m, p->k, p->l, p->sfa_perm_batch_stride, 1), &g.tma_sfa)) return rc;
    if (int rc = get_map(c, make_sf_key(p->sfb_perm, p->n, p->k, p->l, p->sfb_perm_batch_stride, bn / 128), &g.tma_sfb)) return rc;
    g.n_peer = n_peers;
    for (int i = 0; i < n_peers; ++i) g.c_peer[i] = static_cast<__half*>(c_peers[i]);
    if (epilogue >= 2 && p->c) {
        if (int rc = get_map(c, make_key(p->c, p->n, p->m, p->l, static_cast<uint64_t>(p->c_row_stride) * 2, c_bs, 64, 32,
                                         CU_TENSOR_MAP_DATA_TYPE_FLOAT16),
                             &g.tma_c)) return rc;
        if (n_peers > 0 && n_peers <= peer_tma_limit()) {
            g.peer_tma = 1;
            for (int i = 0; i < n_peers; ++i)
                if (int rc = get_map(c, make_key(c_peers[i], p->n, p->m, p->l, static_cast<uint64_t>(p->c_row_stride) * 2, c_bs, 64, 32,
                                                 CU_TENSOR_MAP_DATA_TYPE_FLOAT16),
                                     &g.tma_c_peer[i])) return rc;
        }
    }

    // Decode shapes (one 128-row block, fewer tiles than half the SMs): split K across a cluster
    // and reduce through distributed shared memory instead of through global scratch.
    int ks = cf.split_k;
    if (ks == 0) {
        ks = 1;
        const long long tiles128 = static_cast<long long>(p->n / 128) * p->l;
        if (p->m <= kBM && cf.cta_group != 2 && cf.tile_n == 0 && cf.grid == 0) {
            // measured (four exchanges its partial sums through L2, two through distributed shared
            // memory): four CTAs per tile win when they fit one wave (128 x 4096 x 7168: 10.1 vs
            // 10.6 us), two otherwise (128 x 7168 x 16384: 17.5 us; 4 x 256-wide 20.3)
            if (tiles128 * 4 <= c->num_sms && g.k_tiles >= 16 && !epi) ks = 4;
            else if (tiles128 * 2 <= c->num_sms && g.k_tiles >= 16) ks = 2;   // shorter K: one whole tile per CTA wins
        }
    }
    if (ks > 1) {
        if (cf.cta_group == 2) return fail(NVFP4_ERR_INVALID_ARGUMENT, "split_k > 1 uses single-CTA tiles (cta_group 1)");
        if (g.k_tiles < ks) return fail(NVFP4_ERR_INVALID_ARGUMENT, "split_k = %d needs k >= %d", ks, ks * kKPerStage);
        // single-CTA tiles of 128 x bn_ks, whatever the stream-K planning above chose
        int bn_ks = cf.tile_n ? cf.tile_n : 128;
        if (ks == 8) bn_ks = 256;                      // 32 columns per CTA at least
        if (ks == 2 && bn_ks == 256) return fail(NVFP4_ERR_INVALID_ARGUMENT, "split_k = 2 is built for tile_n 128");
        if (p->n % bn_ks) return fail(NVFP4_ERR_INVALID_ARGUMENT, "n = %d is not a multiple of tile_n = %d", p->n, bn_ks);
        bn = bn_ks;
        g.tiles_m = (p->m + kBM - 1) / kBM;
        g.tiles_n = p->n / bn;
        g.total_units = g.tiles_m * g.tiles_n * p->l * g.k_tiles;
        if (int rc = get_map(c, make_key(p->b, kbytes, p->n, p->l, p->b_row_stride, b_bs, kBKBytes, bn, CU_TENSOR_MAP_DATA_TYPE_UINT8),
                             &g.tma_b)) return rc;
        if (int rc = get_map(c, make_sf_key(p->sfb_perm, p->n, p->k, p->l, p->sfb_perm_batch_stride, bn / 128), &g.tma_sfb)) return rc;
        if (epi) {
            if (bn == 128 && ks == 2) return launch_gemm_splitk<128, 6, 0, 2, true>(c, 16, g, stream, "gemm_splitk2_n128_s6_epilogue");
            return fail(NVFP4_ERR_UNSUPPORTED, "the extended epilogue is built for split_k 1 and 2");
        }
        if (bn == 128 && ks == 2) return launch_gemm_splitk<128, 6, 0, 2>(c, 8, g, stream, "gemm_splitk2_n128_s6");
        if (bn == 128) return launch_gemm_splitk<128, 6, 0, 4>(c, 9, g, stream, "gemm_splitk4_n128_s6");
        if (ks == 4) return launch_gemm_splitk<256, 4, 0, 4>(c, 10, g, stream, "gemm_splitk4_n256_s4");
        return launch_gemm_splitk<256, 4, 0, 8>(c, 11, g, stream, "gemm_splitk8_n256_s4");
    }

    const int grid = cf.grid;
    if (epi) {
        if (cg == 2 && bn == 256) return launch_gemm<2, 256, 5, false, 32, true>(c, 17, g, grid, stream, "gemm_2cta_n256_s5_epilogue");
        if (cg == 2) return launch_gemm<2, 128, 6, false, 32, true>(c, 18, g, grid, stream, "gemm_2cta_n128_s6_epilogue");
        if (bn == 256) return launch_gemm<1, 256, 3, false, 48, true>(c, 19, g, grid, stream, "gemm_1cta_n256_s3_epilogue");
        return launch_gemm<1, 128, 4, false, 64, true>(c, 20, g, grid, stream, "gemm_1cta_n128_s4_epilogue");
    }
    if (cg == 2) {
        if (bn == 256 && epilogue == 3) return launch_gemm<2, 256, 4, true, 64>(c, 12, g, grid, stream, "gemm_2cta_n256_s4_tmastore4");
        if (bn == 256 && epilogue == 2) return launch_gemm<2, 256, 5, true, 32>(c, 4, g, grid, stream, "gemm_2cta_n256_s5_tmastore");
        if (bn == 256) return launch_gemm<2, 256, 5, false, 32>(c, 5, g, grid, stream, "gemm_2cta_n256_s5_direct");
        if (epilogue >= 2) return launch_gemm<2, 128, 6, true, 32>(c, 6, g, grid, stream, "gemm_2cta_n128_s6_tmastore");
        return launch_gemm<2, 128, 6, false, 32>(c, 7, g, grid, stream, "gemm_2cta_n128_s6_direct");
    }
    if (bn == 128 && epilogue >= 2) return launch_gemm<1, 128, 5, true, 32>(c, 0, g, grid, stream, "gemm_1cta_n128_s5_tmastore");
    if (bn == 128) return launch_gemm<1, 128, 4, false, 64>(c, 1, g, grid, stream, "gemm_1cta_n128_s4_direct");
    if (epilogue >= 2) return launch_gemm<1, 256, 3, true, 32>(c, 2, g, grid, stream, "gemm_1cta_n256_s3_tmastore");
    return launch_gemm<1, 256, 3, false, 48>(c, 3, g, grid, stream, "gemm_1cta_n256_s3_direct");
}
}  // namespace

// Defined with the static-scratch entry point below: reads and clears that path's status word
// (0 when the path was never used on `dev`).  Allocates nothing.
static int static_scratch_take_status(int dev, int* status);

extern "C" {

int nvfp4_gemm(const nvfp4_problem* p, const nvfp4_gemm_config* cfg, void* stream_v) {
    return gemm_impl(p, cfg, nullptr, nullptr, 0, stream_v);
}

int nvfp4_gemm_epilogue(const nvfp4_problem* p, const nvfp4_gemm_config* cfg, const nvfp4_epilogue* epi, void* stream_v) {
    if (!epi) return fail(NVFP4_ERR_INVALID_ARGUMENT, "epilogue is NULL (use nvfp4_gemm for the plain fp16 output)");
    return gemm_impl(p, cfg, epi, nullptr, 0, stream_v);
}

int nvfp4_gemm_allgather(const nvfp4_problem* p, const nvfp4_gemm_config* cfg, void* const* c_peers, int n_peers, void* stream_v) {
    if (n_peers < 0 || n_peers > 7) return fail(NVFP4_ERR_INVALID_ARGUMENT, "n_peers must be between 0 and 7 (got %d)", n_peers);
    if (n_peers > 0 && !c_peers) return fail(NVFP4_ERR_INVALID_ARGUMENT, "c_peers is NULL");
    for (int i = 0; i < n_peers; ++i)
        if (!c_peers[i] || !aligned(c_peers[i], 16)) return fail(NVFP4_ERR_INVALID_ARGUMENT, "c_peers[%d] must be a 16-byte aligned pointer", i);
    // the cluster split-K kernels (decode shapes) finish tiles in their exchange epilogue, which
    // does know about peers too, but keep this entry on the persistent kernels: one code path
    nvfp4_gemm_config cf = {0, 0, 0, 0, 0, 0};
    if (cfg) cf = *cfg;
    if (cf.split_k == 0) cf.split_k = 1;
    return gemm_impl(p, &cf, nullptr, c_peers, n_peers, stream_v);
}

int nvfp4_gemv(const nvfp4_problem* p, void* stream_v) { return nvfp4_gemv_config(p, 0, 0, stream_v); }

static int gemv_prepare(const nvfp4_problem* p, GemvParams* g) {
    if (int rc = validate_common(p)) return rc;
    if (!p->c) return fail(NVFP4_ERR_INVALID_ARGUMENT, "c must not be NULL");
    if (p->n != 1) return fail(NVFP4_ERR_INVALID_ARGUMENT, "the GEMV needs n == 1 (got %d)", p->n);
    if (!p->sfa || !p->sfb) return fail(NVFP4_ERR_INVALID_ARGUMENT, "the GEMV needs the plain scale tensors (sfa, sfb)");
    if (p->k % 64) return fail(NVFP4_ERR_INVALID_ARGUMENT, "k must be a multiple of 64 (got %d)", p->k);
    if (!aligned(p->a, 32) || !aligned(p->b, 32) || !aligned(p->sfa, 4) || !aligned(p->sfb, 4))
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "a and b must be 32-byte aligned, sfa and sfb 4-byte aligned");
    if (p->a_row_stride % 32 || p->sfa_row_stride % 4 || p->a_row_stride < p->k / 2 || p->sfa_row_stride < p->k / 16)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "a_row_stride must be a multiple of 32 bytes, sfa_row_stride of 4");
    if (p->l > 1 && (p->a_batch_stride % 32 || p->b_batch_stride % 32 || p->sfa_batch_stride % 4 || p->sfb_batch_stride % 4))
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "batch strides must keep 32-byte (a, b) / 4-byte (sfa, sfb) alignment");
    if (p->l > 65535) return fail(NVFP4_ERR_INVALID_ARGUMENT, "l must be <= 65535");
    DeviceCtx* c = nullptr;
    if (int rc = get_ctx(&c)) return rc;
    if (!c->sm100) return fail(NVFP4_ERR_UNSUPPORTED, "device %d is not sm_100", c->device);
    g->a = static_cast<const uint8_t*>(p->a);
    g->b = static_cast<const uint8_t*>(p->b);
    g->sfa = static_cast<const uint8_t*>(p->sfa);
    g->sfb = static_cast<const uint8_t*>(p->sfb);
    g->c = static_cast<__half*>(p->c);
    g->a_row_stride = p->a_row_stride; g->a_batch_stride = p->a_batch_stride;
    g->b_batch_stride = p->b_batch_stride;
    g->sfa_row_stride = p->sfa_row_stride; g->sfa_batch_stride = p->sfa_batch_stride;
    g->sfb_batch_stride = p->sfb_batch_stride;
    g->c_row_stride = p->c_row_stride; g->c_batch_stride = p->c_batch_stride;
    g->M = p->m; g->K = p->k; g->L = p->l;
    return NVFP4_OK;
}

int nvfp4_gemv_config(const nvfp4_problem* p, int rows_per_warp, int warps_per_cta, void* stream_v) {
    if (rows_per_warp != 0 && rows_per_warp != 1 && rows_per_warp != 2 && rows_per_warp != 4)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "rows_per_warp must be 0 (auto), 1, 2 or 4");
    if (warps_per_cta != 0 && warps_per_cta != 1 && warps_per_cta != 2 && warps_per_cta != 4)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "warps_per_cta must be 0 (auto), 1, 2 or 4");
    GemvParams g;
    if (int rc = gemv_prepare(p, &g)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    // Rows per warp: short rows amortise the vector's dequantisation over four rows; long rows keep
    // more loads in flight with two, or with one when there are so few rows that two per warp
    // would leave warps short.  One warp per CTA: the block scheduler hands out CTAs as SMs free
    // up, so the smallest CTAs even out the tail.  Measured on B200 over all nine combinations
    // (graph replay, cold inputs): 7168 x 16384 x 1: r1/w1 15.5 us, r2/w4 16.3; 7168 x 16384 x 4:
    // r2/w1 45.2, r2/w4 45.7, r1 49.9; 4096 x 7168 x 8: r2/w1 26.2, r4 27.8; 7168 x 2048 x 4:
    // r4/w1 9.1, r2 10.1, r1 14.4.  (Splitting K over the warps of a CTA, one CTA per one or two
    // rows, was measured as well: 14.7 us at best on 7168 x 16384 x 1 and slower than this
    // everywhere else, so it is not kept.)
    const long long rows_total = static_cast<long long>(p->m) * p->l;
    const int r = rows_per_warp ? rows_per_warp : (p->k <= 4096) ? 4 : (rows_total <= 8192) ? 1 : 2;
    const int w = warps_per_cta ? warps_per_cta : 1;
    const int rows_per_cta = w * r;
    dim3 grid((p->m + rows_per_cta - 1) / rows_per_cta, p->l);
    // (Programmatic dependent launch, which the GEMM kernels use, was measured here too: no gain on
    // the long shapes and 9.0 -> 9.9 us on 7168 x 2048 x 4, so the GEMV is launched plainly.)
    if (r == 4) gemv_nvfp4_kernel<4><<<grid, w * 32, 0, stream>>>(g);
    else if (r == 2) gemv_nvfp4_kernel<2><<<grid, w * 32, 0, stream>>>(g);
    else gemv_nvfp4_kernel<1><<<grid, w * 32, 0, stream>>>(g);
    CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    static const char* const names[3][3] = {{"gemv_warp_r1_w1", "gemv_warp_r1_w2", "gemv_warp_r1_w4"},
                                            {"gemv_warp_r2_w1", "gemv_warp_r2_w2", "gemv_warp_r2_w4"},
                                            {"gemv_warp_r4_w1", "gemv_warp_r4_w2", "gemv_warp_r4_w4"}};
    t_last_kernel = names[r == 4 ? 2 : r - 1][w == 4 ? 2 : w - 1];
    return NVFP4_OK;
}

int nvfp4_interleave_column_blocks(const void* src, void* dst, int64_t rows, int32_t n_local, int32_t blocks,
                                   int64_t dst_row_stride, void* stream_v) {
    if (!src || !dst) return fail(NVFP4_ERR_INVALID_ARGUMENT, "src and dst must not be NULL");
    if (rows < 1 || n_local < 8 || n_local % 8 || blocks < 1)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "rows >= 1, n_local a positive multiple of 8, blocks >= 1 required");
    if (dst_row_stride % 8 || dst_row_stride < static_cast<int64_t>(n_local) * blocks)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "dst_row_stride must be a multiple of 8 elements and >= n_local * blocks");
    if (!aligned(src, 16) || !aligned(dst, 16)) return fail(NVFP4_ERR_INVALID_ARGUMENT, "src and dst must be 16-byte aligned");
    int dev = 0, sms = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long total = rows * (n_local / 8) * blocks;
    long long grid = (total + 255) / 256;
    if (grid > static_cast<long long>(sms) * 16) grid = static_cast<long long>(sms) * 16;
    interleave_column_blocks_kernel<<<static_cast<int>(grid), 256, 0, static_cast<cudaStream_t>(stream_v)>>>(
        static_cast<const uint4*>(src), static_cast<uint4*>(dst), rows, n_local / 8, blocks, dst_row_stride / 8);
    CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return NVFP4_OK;
}

int nvfp4_permute_scales(const void* plain, void* permuted, int32_t rows, int32_t k, int32_t l, int64_t plain_row_stride,
                         int64_t plain_batch_stride, int64_t permuted_batch_stride, void* stream_v) {
    if (!plain || !permuted) return fail(NVFP4_ERR_INVALID_ARGUMENT, "plain and permuted must not be NULL");
    if (rows < 1 || l < 1 || k < 64 || k % 64) return fail(NVFP4_ERR_INVALID_ARGUMENT, "rows, l >= 1 and k a positive multiple of 64 required");
    if (!aligned(plain, 4) || !aligned(permuted, 16) || plain_row_stride % 4 || plain_row_stride < k / 16)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "plain must be 4-byte aligned with a row stride that is a multiple of 4 and >= k/16; permuted 16-byte aligned");
    const long long need = static_cast<long long>((rows + 127) / 128) * (k / 64) * 512;
    if (l > 1 && (permuted_batch_stride < need || permuted_batch_stride % 16 || plain_batch_stride % 4))
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "batch strides too small or misaligned");
    int dev = 0, sms = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long total = need / 16 * l;
    long long grid = (total + 255) / 256;
    if (grid > static_cast<long long>(sms) * 16) grid = static_cast<long long>(sms) * 16;
    permute_scales_kernel<<<static_cast<int>(grid), 256, 0, static_cast<cudaStream_t>(stream_v)>>>(
        static_cast<const uint8_t*>(plain), static_cast<uint8_t*>(permuted), rows, k / 16, plain_row_stride, plain_batch_stride,
        permuted_batch_stride, l);
    CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return NVFP4_OK;
}

// Shared by the two entry points that read the permuted form.
static int scales_from_permuted(const void* permuted, void* plain, int32_t rows, int32_t k, int32_t l, int64_t plain_row_stride,
                                int64_t plain_batch_stride, int64_t permuted_batch_stride, unsigned long long* result, void* stream_v) {
    if (!plain || !permuted) return fail(NVFP4_ERR_INVALID_ARGUMENT, "plain and permuted must not be NULL");
    if (rows < 1 || l < 1 || k < 64 || k % 64) return fail(NVFP4_ERR_INVALID_ARGUMENT, "rows, l >= 1 and k a positive multiple of 64 required");
    if (!aligned(plain, 4) || !aligned(permuted, 16) || plain_row_stride % 4 || plain_row_stride < k / 16)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "plain must be 4-byte aligned with a row stride that is a multiple of 4 and >= k/16; permuted 16-byte aligned");
    const long long need = static_cast<long long>((rows + 127) / 128) * (k / 64) * 512;
    if (l > 1 && (permuted_batch_stride < need || permuted_batch_stride % 16 || plain_batch_stride % 4))
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "batch strides too small or misaligned");
    int dev = 0, sms = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long total = need / 16 * l;
    long long grid = (total + 255) / 256;
    if (grid > static_cast<long long>(sms) * 16) grid = static_cast<long long>(sms) * 16;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (result) {
        CUDA_TRY(cudaMemsetAsync(result, 0, 8, stream));
        CUDA_TRY(cudaMemsetAsync(result + 1, 0xFF, 8, stream));
        scales_from_permuted_kernel<true><<<static_cast<int>(grid), 256, 0, stream>>>(
            static_cast<const uint8_t*>(permuted), static_cast<uint8_t*>(plain), rows, k / 16, plain_row_stride, plain_batch_stride,
            permuted_batch_stride, l, result);
    } else {
        scales_from_permuted_kernel<false><<<static_cast<int>(grid), 256, 0, stream>>>(
            static_cast<const uint8_t*>(permuted), static_cast<uint8_t*>(plain), rows, k / 16, plain_row_stride, plain_batch_stride,
            permuted_batch_stride, l, nullptr);
    }
    CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return NVFP4_OK;
}

int nvfp4_unpermute_scales(const void* permuted, void* plain, int32_t rows, int32_t k, int32_t l, int64_t plain_row_stride,
                           int64_t plain_batch_stride, int64_t permuted_batch_stride, void* stream_v) {
    return scales_from_permuted(permuted, plain, rows, k, l, plain_row_stride, plain_batch_stride, permuted_batch_stride, nullptr, stream_v);
}

int nvfp4_compare_scale_layouts(const void* plain, const void* permuted, int32_t rows, int32_t k, int32_t l, int64_t plain_row_stride,
                                int64_t plain_batch_stride, int64_t permuted_batch_stride, uint64_t* result, void* stream_v) {
    if (!result || !aligned(result, 8)) return fail(NVFP4_ERR_INVALID_ARGUMENT, "result must be an 8-byte aligned device pointer to two 64-bit words");
    return scales_from_permuted(permuted, const_cast<void*>(plain), rows, k, l, plain_row_stride, plain_batch_stride, permuted_batch_stride,
                                reinterpret_cast<unsigned long long*>(result), stream_v);
}

int nvfp4_copy_column_blocks(void* const* dst_blocks, const void* const* src_blocks, int32_t n_blocks, int64_t row0, int64_t rows,
                             int32_t n_local, int64_t row_stride, int32_t ctas, int32_t own_sms, void* stream_v) {
    if (n_blocks < 1 || n_blocks > 7 || !dst_blocks || !src_blocks) return fail(NVFP4_ERR_INVALID_ARGUMENT, "1..7 blocks required");
    if (rows < 1 || row0 < 0 || n_local < 8 || n_local % 8 || row_stride % 8 || row_stride < n_local)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "rows >= 1, n_local and row_stride multiples of 8 elements, row_stride >= n_local required");
    BlockCopyParams pp;
    pp.n_src = n_blocks;
    for (int i = 0; i < n_blocks; ++i) {
        if (!dst_blocks[i] || !src_blocks[i] || !aligned(dst_blocks[i], 16) || !aligned(src_blocks[i], 16))
            return fail(NVFP4_ERR_INVALID_ARGUMENT, "block %d: pointers must be non-NULL and 16-byte aligned", i);
        pp.src[i] = static_cast<const uint4*>(src_blocks[i]);
        pp.dst[i] = static_cast<uint4*>(dst_blocks[i]);
    }
    int dev = 0, sms = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (rows * (n_local / 8) * n_blocks >= (1ll << 31)) return fail(NVFP4_ERR_INVALID_ARGUMENT, "more than 2^31 16-byte units in one call");
    int grid = ctas > 0 ? ctas : sms * 2;
    // own_sms: ask for shared memory the kernel never touches, more than a persistent GEMM CTA
    // leaves free on its SM, so the copy's CTAs are placed on the SMs that GEMM does not occupy
    // instead of sharing issue slots with it.
    const size_t reserve = own_sms ? 24 * 1024 : 0;
    copy_column_blocks_kernel<<<grid, 256, reserve, static_cast<cudaStream_t>(stream_v)>>>(pp, row0, static_cast<unsigned>(rows),
                                                                                     static_cast<unsigned>(n_local / 8), row_stride / 8);
    CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return NVFP4_OK;
}

// ---------------------------------------------------------------------------------------------
// Peer pointers without torch: a rank exports the allocation that holds its output, the others
// open it and get an address they can hand to nvfp4_gemm_allgather / nvfp4_copy_column_blocks.
// ---------------------------------------------------------------------------------------------
int nvfp4_comm_export(const void* ptr, void* handle_out, int64_t* offset_out) {
    if (!ptr || !handle_out || !offset_out) return fail(NVFP4_ERR_INVALID_ARGUMENT, "ptr, handle_out and offset_out must not be NULL");
    // the handle names the whole allocation: find its base and report where ptr lies inside it
    using GetRangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
    static GetRangeFn get_range = nullptr;
    if (!get_range) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CUDA_TRY(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return fail(NVFP4_ERR_CUDA, "cuMemGetAddressRange is not available from this driver");
        get_range = reinterpret_cast<GetRangeFn>(fn);
    }
    CUdeviceptr base = 0;
    size_t size = 0;
    const CUresult r = get_range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
    if (r != CUDA_SUCCESS) return fail(NVFP4_ERR_CUDA, "cuMemGetAddressRange failed (CUresult %d): not a device allocation?", static_cast<int>(r));
    cudaIpcMemHandle_t h;
    CUDA_TRY(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
    static_assert(sizeof(h) == NVFP4_COMM_HANDLE_BYTES, "handle size");
    std::memcpy(handle_out, &h, sizeof(h));
    *offset_out = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
    return NVFP4_OK;
}

int nvfp4_comm_open(const void* handle, int64_t offset, void** ptr_out) {
    if (!handle || !ptr_out || offset < 0) return fail(NVFP4_ERR_INVALID_ARGUMENT, "handle and ptr_out must not be NULL, offset >= 0");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* base = nullptr;
    CUDA_TRY(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr_out = static_cast<uint8_t*>(base) + offset;
    return NVFP4_OK;
}

int nvfp4_comm_close(void* opened_ptr, int64_t offset) {
    if (!opened_ptr || offset < 0) return fail(NVFP4_ERR_INVALID_ARGUMENT, "opened_ptr must not be NULL, offset >= 0");
    CUDA_TRY(cudaIpcCloseMemHandle(static_cast<uint8_t*>(opened_ptr) - offset));
    return NVFP4_OK;
}

int nvfp4_copy_2d(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t width_bytes, int64_t rows, void* stream_v) {
    if (!dst || !src) return fail(NVFP4_ERR_INVALID_ARGUMENT, "dst and src must not be NULL");
    if (width_bytes < 1 || rows < 1 || dst_pitch < width_bytes || src_pitch < width_bytes)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "width_bytes, rows >= 1 and both pitches >= width_bytes required");
    CUDA_TRY(cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_pitch), src, static_cast<size_t>(src_pitch), static_cast<size_t>(width_bytes),
                               static_cast<size_t>(rows), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream_v)));
    return NVFP4_OK;
}

int nvfp4_quantize(const void* x, int32_t x_is_bf16, void* packed, void* sf_plain, void* sf_permuted, int32_t rows, int32_t k,
                   int64_t x_row_stride, int64_t packed_row_stride, int64_t sf_plain_row_stride, void* stream_v) {
    if (!x || !packed) return fail(NVFP4_ERR_INVALID_ARGUMENT, "x and packed must not be NULL");
    if (!sf_plain && !sf_permuted) return fail(NVFP4_ERR_INVALID_ARGUMENT, "at least one of sf_plain / sf_permuted is needed");
    if (rows < 1 || k < 64 || k % 64) return fail(NVFP4_ERR_INVALID_ARGUMENT, "rows >= 1 and k a positive multiple of 64 required");
    if (!aligned(x, 16) || x_row_stride % 8 || x_row_stride < k)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "x must be 16-byte aligned with a row stride (elements) that is a multiple of 8 and >= k");
    if (!aligned(packed, 8) || packed_row_stride % 8 || packed_row_stride < k / 2)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "packed must be 8-byte aligned with a row stride that is a multiple of 8 and >= k/2");
    if (sf_plain && sf_plain_row_stride < k / 16) return fail(NVFP4_ERR_INVALID_ARGUMENT, "sf_plain_row_stride must be >= k/16");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    int dev = 0, sms = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    // resident CTAs take 128-row x 256-column units in turn
    const long long units = static_cast<long long>((rows + 127) / 128) * ((k / 64 + kQuantGroups - 1) / kQuantGroups);
    const int grid = static_cast<int>(units < static_cast<long long>(sms) * 4 ? units : static_cast<long long>(sms) * 4);
    // wide stores when every output address is aligned for them
    const bool wide = aligned(packed, 16) && packed_row_stride % 16 == 0 && (!sf_plain || (aligned(sf_plain, 4) && sf_plain_row_stride % 4 == 0)) &&
                      (!sf_permuted || aligned(sf_permuted, 16));
    auto launch = [&](auto kernel) {
        kernel<<<grid, 256, 0, stream>>>(x, static_cast<uint8_t*>(packed), static_cast<uint8_t*>(sf_plain), static_cast<uint8_t*>(sf_permuted), rows, k,
                                         x_row_stride, packed_row_stride, sf_plain_row_stride);
    };
    if (x_is_bf16) {
        if (wide) launch(quantize_nvfp4_kernel<true, true>);
        else launch(quantize_nvfp4_kernel<true, false>);
    } else {
        if (wide) launch(quantize_nvfp4_kernel<false, true>);
        else launch(quantize_nvfp4_kernel<false, false>);
    }
    CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return NVFP4_OK;
}

int nvfp4_matmul(const nvfp4_problem* p, void* stream) {
    if (p && p->n == 1) return nvfp4_gemv(p, stream);
    return nvfp4_gemm(p, nullptr, stream);
}

int nvfp4_check_status(void* stream_v) {
    DeviceCtx* c = nullptr;
    if (int rc = get_ctx(&c)) return rc;
    CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_v)));
    // kernels of nvfp4_gemm_static_scratch report into their own device word (that path must not
    // allocate, so it has no host-mapped one): fetch it into a stack variable
    int static_st = 0;
    if (int rc = static_scratch_take_status(c->device, &static_st)) return rc;
    if (static_st != kStatusOk)
        return fail(NVFP4_ERR_DEVICE_TIMEOUT, "a kernel of nvfp4_gemm_static_scratch gave up on a bounded wait (device status %d)", static_st);
    const int st = *reinterpret_cast<volatile int*>(c->status_host);
    if (st == kStatusOk) return NVFP4_OK;
    *reinterpret_cast<volatile int*>(c->status_host) = 0;
    // A kernel that gave up may have left tile counters half-way: restore the all-zero invariant.
    if (c->scratch) {
        CUDA_TRY(cudaDeviceSynchronize());
        CUDA_TRY(cudaMemset(c->counters, 0, kStreamSets * kMaxCtas * sizeof(int)));
        CUDA_TRY(cudaDeviceSynchronize());
    }
    return fail(NVFP4_ERR_DEVICE_TIMEOUT, "a kernel gave up on a bounded wait (device status %d)", st);
}

uint64_t nvfp4_set_wait_timeout_ns(uint64_t ns) { return g_timeout_ns.exchange(ns); }

int nvfp4_release_stream(void* stream_v) {
    DeviceCtx* c = nullptr;
    if (int rc = get_ctx(&c)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    std::lock_guard<std::mutex> lock(g_mutex);
    for (int i = 0; i < kStreamSets; ++i)
        if (c->set_used[i] && c->set_stream[i] == stream) c->set_used[i] = false;
    return NVFP4_OK;
}

int nvfp4_selftest_bounded_wait(void* stream_v) {
    DeviceCtx* c = nullptr;
    if (int rc = get_ctx(&c)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(c->status_dev, g_timeout_ns.load() * 2);
    CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    return nvfp4_check_status(stream_v);
}

size_t nvfp4_scratch_bytes(void) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lock(g_mutex);
    return g_ctx[dev] ? g_ctx[dev]->scratch_bytes : 0;
}

int nvfp4_plan_units(int total_units, int grid, int cta, int* begin, int* end, int* first_tile_slot, int k_tiles) {
    if (total_units < 1 || grid < 1 || cta < 0 || cta >= grid || k_tiles < 1 || !begin || !end)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "bad partition query");
    *begin = unit_boundary(cta, grid, total_units);
    *end = unit_boundary(cta + 1, grid, total_units);
    if (first_tile_slot) *first_tile_slot = partial_slot(cta, *begin % k_tiles, 1, 0);
    return NVFP4_OK;
}

int nvfp4_plan_segment(int total_units, int grid, int cta, int k_tiles, int index, int* begin, int* end) {
    if (total_units < 1 || grid < 1 || cta < 0 || cta >= grid || k_tiles < 1 || index < 0 || !begin || !end)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "bad segment query");
    Segment seg;
    const SegmentPlan plan(unit_boundary(cta, grid, total_units), unit_boundary(cta + 1, grid, total_units), k_tiles);
    if (!plan.at(index, &seg)) {
        *begin = *end = -1;
        return NVFP4_OK;
    }
    *begin = seg.u0;
    *end = seg.u1;
    return NVFP4_OK;
}

int nvfp4_plan_tile_shape(int m, int n, int k, int l, int num_sms, int* cta_group, int* tile_n) {
    if (m < 1 || n < 128 || n % 128 || k < kKPerStage || k % kKPerStage || l < 1 || num_sms < 2 || !cta_group || !tile_n)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "bad tile-shape query");
    const nvfp4_gemm_config cf = {0, 0, 0, 0, 0, 0};
    const TileChoice choice = choose_tile(m, n, k, l, num_sms, cf);
    *cta_group = choice.cta_group;
    *tile_n = choice.tile_n;
    return NVFP4_OK;
}

int nvfp4_plan_work_split(int64_t tiles, int k_tiles, int max_workers, int* workers, int* whole_tiles) {
    if (tiles < 1 || k_tiles < 1 || max_workers < 1 || !workers || !whole_tiles) return fail(NVFP4_ERR_INVALID_ARGUMENT, "bad work-split query");
    const WorkSplit split = plan_work_split(tiles, k_tiles, max_workers);
    *workers = split.workers;
    *whole_tiles = split.whole_tiles ? 1 : 0;
    return NVFP4_OK;
}

int nvfp4_plan_tile(int total_units, int workers, int k_tiles, int tiles_m, int tiles_n, int raster_rows, int tile, int* batch,
                    int* row_tile, int* col_tile) {
    if (total_units < 1 || workers < 1 || k_tiles < 1 || tiles_m < 1 || tiles_n < 1 || total_units % k_tiles || tile < 0 ||
        tile >= total_units / k_tiles || (total_units / k_tiles) % (tiles_m * tiles_n) || !batch || !row_tile || !col_tile)
        return fail(NVFP4_ERR_INVALID_ARGUMENT, "bad tile query");
    const TileCoord c = tile_coords(tile, workers, k_tiles, total_units, tiles_m, tiles_n, raster_rows);
    *batch = c.l;
    *row_tile = c.mt;
    *col_tile = c.nt;
    return NVFP4_OK;
}


int nvfp4_set_peer_tma_limit(int peers) {
    if (peers < 0) peers = 0;
    if (peers > 7) peers = 7;
    return g_peer_tma_limit.exchange(peers);
}

uint64_t nvfp4_launch_count(void) { return g_launches.load(); }

const char* nvfp4_last_kernel(void) { return t_last_kernel; }

void nvfp4_shutdown(void) {
    std::lock_guard<std::mutex> lock(g_mutex);
    int prev = -1;
    cudaGetDevice(&prev);
    for (int d = 0; d < 64; ++d) {
        DeviceCtx* c = g_ctx[d];
        if (!c) continue;
        cudaSetDevice(d);
        cudaDeviceSynchronize();
        if (c->scratch) cudaFree(c->scratch);
        if (c->counters) cudaFree(c->counters);
        if (c->status_host) cudaFreeHost(c->status_host);
        delete c;
        g_ctx[d] = nullptr;
    }
    if (prev >= 0) cudaSetDevice(prev);
}

// ---------------------------------------------------------------------------------------------
// GEMM for callers that must not allocate: the partial-tile scratch of the persistent kernel
// lives in a fixed device array that is part of this library's image.
// ---------------------------------------------------------------------------------------------
}  // extern "C"

namespace {

constexpr int kStaticMaxWorkers = 64;  // persistent CTAs the fixed scratch has slots for
// Two 128 x 128 fp32 partial-tile slots per worker: 64 * 2 * 64 KiB = 8 MiB, resident on every
// GPU that loads the library, until the process exits.
static __device__ __align__(256) float g_static_scratch[kStaticMaxWorkers * 2 * kBM * 128];
static __device__ __align__(256) int g_static_counters[kStaticMaxWorkers];
static __device__ __align__(256) int g_static_status[4];

// What host code may use of the arrays above: their device addresses, looked up once per device.
// (In host code the array names are only handles for the symbol lookup, never pointers.)
struct StaticScratch {
    bool ready = false;
    float* scratch = nullptr;
    int* counters = nullptr;
    int* status = nullptr;
    int num_sms = 0;
};
StaticScratch g_static[64];
std::mutex g_static_mutex;
EncodeTiledFn g_static_encode = nullptr;

int static_scratch_setup(int dev, StaticScratch** out) {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticScratch& st = g_static[dev];
    if (!st.ready) {
        // the calling thread's current device is `dev`: the lookups below resolve that device's copy
        CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&st.scratch), g_static_scratch));
        CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&st.counters), g_static_counters));
        CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&st.status), g_static_status));
        int major = 0;
        CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10) return fail(NVFP4_ERR_UNSUPPORTED, "device %d is not sm_100", dev);
        CUDA_TRY(cudaDeviceGetAttribute(&st.num_sms, cudaDevAttrMultiProcessorCount, dev));
        CUDA_TRY(cudaFuncSetAttribute(gemm_nvfp4_kernel<1, 128, 4, false, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      GemmSmem<1, 128, 4, false, 64>::kDynamicBytes));
        st.ready = true;
    }
    if (!g_static_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess)
            return fail(NVFP4_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        g_static_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    *out = &st;
    return NVFP4_OK;
}

// Encodes a tensor map into caller storage (no cache: nothing is kept on the heap).
int encode_map_inplace(const MapKey& key, CUtensorMap* out) {
    cuuint64_t dims[4] = {key.dims[0], key.dims[1], key.dims[2], key.dims[3]};
    cuuint64_t strides[3] = {key.strides[0], key.strides[1], key.strides[2]};
    cuuint32_t box[4] = {key.box[0], key.box[1], key.box[2], key.box[3]};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUresult r = g_static_encode(out, static_cast<CUtensorMapDataType>(key.dtype), key.rank, const_cast<void*>(key.ptr), dims,
                                 strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, static_cast<CUtensorMapSwizzle>(key.swizzle),
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NVFP4_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d)", static_cast<int>(r));
    return NVFP4_OK;
}

}  // namespace

static int static_scratch_take_status(int dev, int* status) {
    *status = 0;
    StaticScratch* st = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (dev < 0 || dev >= 64 || !g_static[dev].ready) return NVFP4_OK;
        st = &g_static[dev];
    }
    CUDA_TRY(cudaMemcpy(status, st->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status != 0) CUDA_TRY(cudaMemset(st->status, 0, sizeof(int)));
    return NVFP4_OK;
}

extern "C" {

int nvfp4_gemm_static_scratch(const nvfp4_problem* p, int workers, void* stream_v) {
    if (int rc = validate_gemm(p)) return rc;
    if (workers < 0 || workers > kStaticMaxWorkers)
        return fail(NVFP4_ERR_INVALID_ARGUMENT,
                    "workers = %d exceeds what the fixed scratch holds: at most %d persistent CTAs (8 MiB of partial-tile slots)",
                    workers, kStaticMaxWorkers);

    int dev = -1;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(NVFP4_ERR_CUDA, "unexpected device ordinal %d", dev);
    StaticScratch* st = nullptr;
    if (int rc = static_scratch_setup(dev, &st)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    constexpr int bn = 128;
    GemmParams g;
    std::memset(&g, 0, sizeof(g));
    g.M = p->m; g.N = p->n; g.K = p->k; g.L = p->l;
    g.tiles_m = (p->m + kBM - 1) / kBM;
    g.tiles_n = p->n / bn;
    g.k_tiles = p->k / kKPerStage;
    const long long units = static_cast<long long>(g.tiles_m) * g.tiles_n * p->l * g.k_tiles;
    if (units > 0x7fffffffLL) return fail(NVFP4_ERR_INVALID_ARGUMENT, "problem too large: %lld work units", units);
    g.total_units = static_cast<int>(units);
    g.c = static_cast<__half*>(p->c);
    g.scratch = st->scratch;
    g.counters = st->counters;
    g.status = st->status;
    g.c_row_stride = p->c_row_stride;
    g.c_batch_stride = p->c_batch_stride;
    g.timeout_cycles = g_timeout_ns.load() * 2;

    const uint64_t kbytes = static_cast<uint64_t>(p->k) / 2;
    const uint64_t a_bs = p->l > 1 ? static_cast<uint64_t>(p->a_batch_stride) : static_cast<uint64_t>(p->a_row_stride) * p->m;
    const uint64_t b_bs = p->l > 1 ? static_cast<uint64_t>(p->b_batch_stride) : static_cast<uint64_t>(p->b_row_stride) * p->n;
    if (int rc = encode_map_inplace(make_key(p->a, kbytes, p->m, p->l, p->a_row_stride, a_bs, kBKBytes, kBM, CU_TENSOR_MAP_DATA_TYPE_UINT8), &g.tma_a)) return rc;
    if (int rc = encode_map_inplace(make_key(p->b, kbytes, p->n, p->l, p->b_row_stride, b_bs, kBKBytes, bn, CU_TENSOR_MAP_DATA_TYPE_UINT8), &g.tma_b)) return rc;
    if (int rc = encode_map_inplace(make_sf_key(p->sfa_perm, p->m, p->k, p->l, p->sfa_perm_batch_stride, 1), &g.tma_sfa)) return rc;
    if (int rc = encode_map_inplace(make_sf_key(p->sfb_perm, p->n, p->k, p->l, p->sfb_perm_batch_stride, 1), &g.tma_sfb)) return rc;

    int grid = workers > 0 ? workers : kStaticMaxWorkers;
    if (grid > st->num_sms) grid = st->num_sms;
    if (grid > g.total_units) grid = g.total_units;

    // The array keeps whatever the previous call left: the slots are always written before they
    // are read, but the per-tile counters must start at zero (an aborted launch may have left some).
    CUDA_TRY(cudaMemsetAsync(st->counters, 0, kStaticMaxWorkers * sizeof(int), stream));
    using S = GemmSmem<1, 128, 4, false, 64>;
    gemm_nvfp4_kernel<1, 128, 4, false, 64><<<grid, kGemmThreads, S::kDynamicBytes, stream>>>(g);
    CUDA_TRY(cudaGetLastError());
    g_launches.fetch_add(1);
    t_last_kernel = "gemm_1cta_n128_s4_direct(static scratch)";
    return NVFP4_OK;
}

const char* nvfp4_last_error(void) { return t_error.c_str(); }

const char* nvfp4_version(void) { return "nvfp4_b200 0.1 (sm_100a)"; }

}  // extern "C"
