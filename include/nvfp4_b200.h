/*
 * nvfp4_b200 -- C ABI of the B200 (sm_100a) NVFP4 block-scaled matmul library.
 *
 * Every entry point takes raw device pointers, sizes and strides; there are no C++ or
 * torch types in the interface.  All functions return 0 on success and a negative
 * NVFP4_ERR_* code on failure; nvfp4_last_error() gives the message for the calling thread.
 * Work is enqueued on the CUDA stream passed in (a cudaStream_t cast to void*; NULL is the
 * legacy default stream, which is what the reference launches on, s_128t.py:579-582) and is
 * asynchronous with respect to the host.
 *
 * File paths in the comments below are paths inside the reference project.
 */
#ifndef NVFP4_B200_H
#define NVFP4_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVFP4_OK 0
#define NVFP4_ERR_INVALID_ARGUMENT (-1) /* bad shape, alignment, stride or null pointer */
#define NVFP4_ERR_CUDA (-2)             /* a CUDA runtime / driver call failed */
#define NVFP4_ERR_DEVICE_TIMEOUT (-3)   /* a bounded wait inside a kernel ran out */
#define NVFP4_ERR_UNSUPPORTED (-4)      /* not an sm_100 device, or feature not built */

/*
 * One block-scaled matmul problem:  C[m,n,l] = sum_k A[m,k,l]*SFA[m,k/16,l] * B[n,k,l]*SFB[n,k/16,l].
 * This is the 7-tuple of the reference operator (template.py:9-18) spelled as pointers:
 *   a, b           packed e2m1, two values per byte (low nibble = lower k), K contiguous
 *   sfa, sfb       e4m3 (bias 7) scale per 16 K elements, plain [rows, K/16] layout
 *   sfa_perm, ...  the same scales in 512-byte atoms of 128 rows x 4 scales
 *                  ([32,4,rest_rows,4,rest_k,L], ref.txt:31, s_128t.py:554-562)
 *   c              fp16 output
 * The GEMM reads only the permuted scales (like s_128t.py:542-584 and sub_cub.py:82-88); the
 * GEMV reads only the plain ones (like old_files/1.py:697-698).  Unused pointers may be NULL.
 * Strides of a, b, sf* are in bytes, strides of c in fp16 elements.
 */
typedef struct nvfp4_problem {
    const void* a;
    const void* b;
    const void* sfa;
    const void* sfb;
    const void* sfa_perm;
    const void* sfb_perm;
    void* c;
    int32_t m, n, k, l;
    int64_t a_row_stride, a_batch_stride;
    int64_t b_row_stride, b_batch_stride;
    int64_t sfa_row_stride, sfa_batch_stride;
    int64_t sfb_row_stride, sfb_batch_stride;
    int64_t sfa_perm_batch_stride, sfb_perm_batch_stride;
    int64_t c_row_stride, c_batch_stride;
} nvfp4_problem;

/* Kernel selection override for tests and tuning; zero in every field = automatic. */
typedef struct nvfp4_gemm_config {
    int32_t tile_n;    /* 0 auto, 128 or 256 */
    int32_t epilogue;  /* 0 auto, 1 = 16-byte global stores, 2 = TMA store, 3 = TMA store with four staging buffers per warp */
    int32_t grid;      /* 0 auto (one CTA per SM), else number of persistent CTAs */
    int32_t cta_group; /* 0 auto, 1 = one CTA per tile, 2 = CTA pair per 256-row tile */
    int32_t split_k;   /* 0 auto, 1 = persistent stream-K kernel, 2, 4 or 8 = cluster split-K (reduce in DSMEM; 8 needs tile_n 256) */
    int32_t raster;    /* tile order of the persistent kernels: 0 auto, -1 = row-major, r > 0 = column-major inside groups of r row tiles */
} nvfp4_gemm_config;

/*
 * Tensor-core GEMM (tcgen05.mma kind::mxf4nvf4.block_scale).  Replaces
 * cuda_nvfp4_gemm_tcgen05(A, B, SFA, SFB, SFA_perm, SFB_perm, C) of s_128t.py:542-584.
 * Requires n % 128 == 0, k % 256 == 0 (task.yml:24), 16-byte aligned pointers and row strides.
 * Any m >= 1 is accepted (rows past m are not written).  cfg may be NULL.
 *
 * Streams: GEMMs issued on different streams may overlap on the GPU.  The persistent kernels keep
 * fp32 partial tiles and tile counters in library-owned scratch; there is one set per stream,
 * taken from a pool of eight per device that is allocated with the first GEMM on that device
 * (make that call outside any graph capture; no later call allocates, also not on a stream seen
 * for the first time or inside a capture).  A set stays with its stream until
 * nvfp4_release_stream().  When all are taken, sets of streams whose work has completed are
 * reused; sets that were used while their stream was being captured are not (the graph may
 * replay those launches at any time), so release capture streams whose graphs are gone.  If no
 * set can be had the call returns NVFP4_ERR_UNSUPPORTED and launches nothing.
 */
int nvfp4_gemm(const nvfp4_problem* problem, const nvfp4_gemm_config* cfg, void* stream);

/*
 * What the GEMM does with a finished accumulator besides rounding it to fp16: the step that
 * follows the matmul in a layer, fused into its epilogue.
 *   out = act(acc + bias[column])          bias fp16 [n] or NULL, added in fp32
 * written either as fp16 to problem->c or re-quantised to NVFP4 -- packed e2m1 [l][m][n/2] plus one
 * e4m3 scale per 16 consecutive columns of a row, in the plain [l][m][n/16] layout and / or the
 * permuted 128 x 4 atom layout: exactly the a / sfa / sfa_perm operands of a following GEMM whose
 * K is this GEMM's n (and a quarter of the bytes when the output has to travel between GPUs).
 * The NVFP4 form quantises the fp16-rounded values with the rule of nvfp4_quantize(), so it
 * equals that function applied to the fp16 output, bit for bit.  SILU is x / (1 + exp(-x)) with
 * the GPU's fast exponential (not bit-reproducible on a CPU; the others are exact).
 * The reference writes fp16 only (sub_cub.py:98-104, s_128t.py:324-359); no counterpart.
 */
#define NVFP4_ACT_NONE 0
#define NVFP4_ACT_RELU 1
#define NVFP4_ACT_SILU 2
#define NVFP4_OUT_FP16 0
#define NVFP4_OUT_NVFP4 1
typedef struct nvfp4_epilogue {
    const void* bias;   /* fp16 [n], 16-byte aligned, or NULL */
    int32_t activation; /* NVFP4_ACT_* */
    int32_t output;     /* NVFP4_OUT_FP16: problem->c; NVFP4_OUT_NVFP4: the fields below (problem->c may be NULL) */
    void* out_packed;   /* packed e2m1, 16-byte aligned */
    void* out_sf;       /* plain scales or NULL */
    void* out_sf_perm;  /* permuted scales (ceil(m/128) * (n/64) * 512 bytes per batch) or NULL */
    int64_t out_packed_row_stride, out_packed_batch_stride; /* bytes; row stride a multiple of 16 */
    int64_t out_sf_row_stride, out_sf_batch_stride;         /* bytes; row stride even */
    int64_t out_sf_perm_batch_stride;                       /* bytes */
    int64_t out_sf_perm_block_stride;                       /* bytes between 128-row blocks of out_sf_perm; 0 = (n/64)*512 (dense).
                                                               Larger when this GEMM writes a column block of a wider matrix's scales. */
} nvfp4_epilogue;

/*
 * nvfp4_gemm() with the extended epilogue above (same shapes, checks and stream rules; cfg may be
 * NULL; cluster split-K is limited to split_k 2, the TMA-store epilogues are not used).
 */
int nvfp4_gemm_epilogue(const nvfp4_problem* problem, const nvfp4_gemm_config* cfg, const nvfp4_epilogue* epilogue, void* stream);

/*
 * CUDA-core GEMV for n == 1.  Replaces cuda_nvfp4_gemv(A, B, C, SFA, SFB) of
 * old_files/1.py:610-673.  Requires k % 64 == 0 (task_gemv.yml:24) and 32-byte aligned rows.
 */
int nvfp4_gemv(const nvfp4_problem* problem, void* stream);

/*
 * The same GEMV with the launch shape chosen by the caller (tests, tuning): rows_per_warp 1, 2 or
 * 4 and warps_per_cta 1, 2 or 4; 0 = this library's choice (what nvfp4_gemv passes).  Every
 * combination gives bit-identical results: a row is always summed by one warp in the same order.
 */
int nvfp4_gemv_config(const nvfp4_problem* problem, int rows_per_warp, int warps_per_cta, void* stream);

/*
 * What custom_kernel(data) calls (template.py:4-25): n == 1 goes to the GEMV, everything
 * else to the GEMM.
 */
int nvfp4_matmul(const nvfp4_problem* problem, void* stream);

/*
 * GEMM fused with the all-gather of a column-parallel multi-GPU run: every finished piece of C is
 * stored into this GPU's output and, at the same position, into n_peers (<= 7) other GPUs'
 * outputs, so the transfer over NVLink overlaps the math tile by tile and no staging copy or
 * re-layout pass is needed.  problem->c and c_peers[i] point at THIS rank's column block inside
 * the full row-major output of each GPU (base + rank * n_local), problem->n is the local width and
 * problem->c_row_stride the full width; c_peers[i] are peer-mapped device pointers (stores only;
 * nothing is loaded from another GPU).  The caller synchronises the ranks after the kernel (all
 * ranks' kernels must finish before any rank reads its output).  cfg may be NULL.  The reference
 * has no multi-GPU code; no counterpart.
 */
int nvfp4_gemm_allgather(const nvfp4_problem* problem, const nvfp4_gemm_config* cfg, void* const* c_peers, int n_peers,
                         void* stream);

/*
 * How nvfp4_gemm_allgather reaches the peers: with at most `peers` of them, every staged block of
 * the output goes to each peer by one more tensor store (TMA) beside the local one; with more, the
 * epilogue warps store the block themselves (many destinations' tensor maps in play made the
 * tensor stores slow).  Clamped to 0..7; returns the previous value (default 1).
 */
int nvfp4_set_peer_tma_limit(int peers);

/*
 * All-gather by a copy kernel: copies rows [row0, row0 + rows) of n_blocks (<= 7) column blocks,
 * each n_local fp16 wide inside a row-major matrix of row_stride elements, from src_blocks[i] to
 * dst_blocks[i].  Either side may be another GPU's peer-mapped output (already offset to the
 * block): "pull" reads the blocks other GPUs computed into the same place of the local output,
 * "push" writes this GPU's block (every src_blocks[i] the same local pointer) into the peers'
 * outputs.  Plain coalesced 16-byte loads (eight in flight per thread) and stores; ctas = 0 picks
 * two CTAs per SM.  own_sms != 0 keeps the copy's CTAs off SMs whose shared memory a persistent
 * GEMM of this library fills (launch that GEMM with cfg.grid below the SM count and the copy gets
 * the SMs it leaves free, instead of competing with it for issue slots).  Any byte matrix can be
 * moved by counting two bytes as one element.  The caller orders it after the producers' kernels
 * (event or cross-rank barrier).  No counterpart in the reference (single GPU).
 */
int nvfp4_copy_column_blocks(void* const* dst_blocks, const void* const* src_blocks, int32_t n_blocks, int64_t row0, int64_t rows,
                             int32_t n_local, int64_t row_stride, int32_t ctas, int32_t own_sms, void* stream);

/*
 * Peer pointers for the two functions above without any framework: one process per GPU, the
 * exchange of the 64 handle bytes and the offset (a pipe, MPI, a file) is the caller's.
 *   nvfp4_comm_export  in the process that owns `ptr` (any address inside a cudaMalloc'd
 *                      allocation): fills handle_out[NVFP4_COMM_HANDLE_BYTES] and the offset of
 *                      ptr inside its allocation;
 *   nvfp4_comm_open    in another process, with its own GPU current: maps the allocation (peer
 *                      access over NVLink is enabled as needed) and returns the address that
 *                      corresponds to ptr; plain loads and stores only, no multicast binding;
 *   nvfp4_comm_close   unmaps it again.
 * Thin wrappers over CUDA IPC memory handles; an allocation can be opened once per process.
 * No counterpart in the reference (single GPU, single process).
 */
#define NVFP4_COMM_HANDLE_BYTES 64
int nvfp4_comm_export(const void* ptr, void* handle_out, int64_t* offset_out);
int nvfp4_comm_open(const void* handle, int64_t offset, void** ptr_out);
int nvfp4_comm_close(void* opened_ptr, int64_t offset);

/*
 * Strided device-to-device copy (one cudaMemcpy2DAsync: `rows` pieces of `width_bytes`), used to
 * push a rank's column block of C into a peer GPU's row-major output with the copy engines while
 * the SMs compute the next row panel.  dst may be peer-mapped memory.  No counterpart in the
 * reference (single GPU).
 */
int nvfp4_copy_2d(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t width_bytes, int64_t rows, void* stream);

/*
 * Column-parallel multi-GPU GEMM, last step: an all-gather of per-rank fp16 column blocks leaves
 * [blocks][rows][n_local] in memory; this writes the row-major [rows][blocks * n_local] matrix
 * (row stride dst_row_stride elements).  The reference has no multi-GPU code; no counterpart.
 */
int nvfp4_interleave_column_blocks(const void* src, void* dst, int64_t rows, int32_t n_local, int32_t blocks,
                                   int64_t dst_row_stride, void* stream);

/*
 * Plain scale factors [l][rows][k/16] (strides in bytes) -> the permuted 128 x 4 atom layout the
 * GEMM reads ([32,4,rest_rows,4,rest_k,l], ref.txt:31, s_128t.py:554-562), rows zero-padded to a
 * multiple of 128.  The reference receives both forms from its harness (template.py:11-14) and has
 * no converter of its own.
 */
int nvfp4_permute_scales(const void* plain, void* permuted, int32_t rows, int32_t k, int32_t l, int64_t plain_row_stride,
                         int64_t plain_batch_stride, int64_t permuted_batch_stride, void* stream);

/*
 * The way back: permuted atoms -> plain [l][rows][k/16] (same argument meaning and checks as
 * nvfp4_permute_scales; padding rows of the atoms are dropped).  No counterpart in the reference.
 */
int nvfp4_unpermute_scales(const void* permuted, void* plain, int32_t rows, int32_t k, int32_t l, int64_t plain_row_stride,
                           int64_t plain_batch_stride, int64_t permuted_batch_stride, void* stream);

/*
 * Validator for the two scale tensors one operator call carries (template.py:11-14 passes both
 * and the reference's kernels trust whichever they read): compares plain with permuted on the
 * device.  result points to two 64-bit words in DEVICE memory, written in stream order:
 * result[0] = number of scale bytes that differ, result[1] = the smallest linear index
 * ((batch * rows + row) * (k/16) + scale column) of one, or 2^64-1 when none.  Nothing
 * synchronises; read result after the stream has.
 */
int nvfp4_compare_scale_layouts(const void* plain, const void* permuted, int32_t rows, int32_t k, int32_t l, int64_t plain_row_stride,
                                int64_t plain_batch_stride, int64_t permuted_batch_stride, uint64_t* result, void* stream);

/*
 * NVFP4 quantiser, the step that produces the operator's inputs: fp16 (x_is_bf16 = 0) or bf16
 * [rows][k] -> packed e2m1 [rows][k/2] plus one e4m3 scale per 16 elements, written in the plain
 * layout (sf_plain, may be NULL) and / or the permuted atom layout (sf_permuted, may be NULL;
 * ceil(rows/128) * (k/64) * 512 bytes).  scale = RN-even, saturating e4m3 of max|x|/6; element =
 * RN-even, saturating e2m1 of x/scale.  x_row_stride in elements, the others in bytes.  The
 * reference receives already-quantised tensors from its harness (template.py:9-15); no counterpart.
 */
int nvfp4_quantize(const void* x, int32_t x_is_bf16, void* packed, void* sf_plain, void* sf_permuted, int32_t rows, int32_t k,
                   int64_t x_row_stride, int64_t packed_row_stride, int64_t sf_plain_row_stride, void* stream);

/*
 * The same GEMM for callers that cannot allocate device memory when they call: code that runs
 * while another thread captures a CUDA graph in global capture mode (cudaMalloc is illegal
 * then), services that hand all free HBM to their own pool at start-up so that a later
 * cudaMalloc fails, and latency-critical loops that may not take the allocator's lock.
 * It has no counterpart in the reference.
 *
 * nvfp4_gemm() keeps the fp32 partial sums of tiles that several persistent CTAs share in
 * scratch memory it allocates on first use.  This entry point runs the same persistent kernel
 * (128 x 128 tiles, one CTA per worker) with that scratch in a fixed array inside the library's
 * device image: 8 MiB (two 64 KiB slots for each of at most 64 workers) that every GPU which
 * loads the library holds until the process exits.  Nothing is allocated or freed, on the device
 * or through any allocating library routine; tensor maps are encoded into stack storage.
 *
 *   workers   persistent CTAs to use; 0 = 64, the most the fixed scratch has slots for.  A
 *             larger request is rejected with NVFP4_ERR_INVALID_ARGUMENT (so is any shape
 *             nvfp4_gemm() would reject).  Fewer CTAs than SMs: expect lower throughput than
 *             nvfp4_gemm() on large problems.
 *
 * The first call on a device looks up the array's device address and raises the kernel's
 * shared-memory limit; make that first call outside any stream capture.  All calls on a device
 * share the one array, which keeps the last call's contents: each call re-zeroes the tile
 * counters on `stream` before its kernel, and two calls whose kernels overlap on the GPU
 * (different streams, no dependency) race on the slots -- serialise them.  A bounded wait that
 * runs out inside this variant is recorded in a device word of the same image; nvfp4_check_status()
 * reads it (and returns NVFP4_ERR_DEVICE_TIMEOUT) without allocating.
 */
int nvfp4_gemm_static_scratch(const nvfp4_problem* problem, int workers, void* stream);

/*
 * Gives back the scratch set nvfp4_gemm() assigned to `stream` on the current device (see there).
 * Call it when no GEMM of that stream is in flight any more and no graph captured on it will be
 * replayed again, e.g. before destroying the stream.
 * No counterpart in the reference (one stream, no scratch).
 */
int nvfp4_release_stream(void* stream);

/*
 * Waits for `stream` and returns NVFP4_ERR_DEVICE_TIMEOUT if any kernel launched by this
 * library on the current device reported a timed-out wait since the last check, else NVFP4_OK
 * (kernels of nvfp4_gemm_static_scratch included: their status word lives in device memory and is
 * copied into a stack variable here, nothing is allocated).
 * The reference has no counterpart (its waits are unbounded spins, s_128t.py:124-183,309-319).
 */
int nvfp4_check_status(void* stream);

/* Limit, in nanoseconds, of every in-kernel wait (default 1e9).  Returns the previous value. */
uint64_t nvfp4_set_wait_timeout_ns(uint64_t ns);

/*
 * Launches a one-CTA kernel that waits on an mbarrier nothing ever arrives at, with the
 * current wait limit, and synchronises.  Returns NVFP4_ERR_DEVICE_TIMEOUT when the wait gave
 * up as designed (the context stays usable).  Exists so that the failure path can be tested
 * without faulting or hanging a GPU.
 */
int nvfp4_selftest_bounded_wait(void* stream);

/*
 * Host-side view of the GEMM's work partition (no GPU needed): the half-open range of
 * (tile, k-tile) work units that persistent worker `cta` of `grid` processes, and the scratch
 * slot it publishes its first segment to if that segment covers only part of a tile's k-range.
 */
int nvfp4_plan_units(int total_units, int grid, int cta, int* begin, int* end, int* first_tile_slot, int k_tiles);

/*
 * Host-side view of how a launch shares `tiles` output tiles of `k_tiles` k-tiles each among at
 * most `max_workers` persistent workers (CTAs, or CTA pairs) when the caller leaves the grid to
 * the library: *whole_tiles = 1 and *workers = the fewest workers that need no more waves (the work
 * is split at tile boundaries only), or *whole_tiles = 0 and *workers = max_workers (an even split
 * of all (tile, k-tile) units; tiles shared between workers are summed through scratch).  The choice
 * is the smaller of two estimates in k-tiles of run time: waves x k_tiles, and units / workers plus
 * 3 (a worker has two tiles' worth of units or more: the summing hides behind whole tiles) or 12 per
 * worker that shares a tile (at least 24).
 */
int nvfp4_plan_work_split(int64_t tiles, int k_tiles, int max_workers, int* workers, int* whole_tiles);

/*
 * Host-side view of the tile a GEMM of this shape gets on a device with num_sms SMs when the
 * caller fixes nothing (cluster split-K aside, which decode shapes take first): *cta_group = 2 for
 * 256-row tiles on CTA pairs or 1, *tile_n = 128 or 256.  Pairs with 256 x 256 tiles unless the
 * estimate above, with a 128-wide stage counted as 0.9 of the pair's and the last epilogue as 4.5
 * against 9 k-tiles, says that 128 x 128 tiles on single CTAs finish sooner.
 */
int nvfp4_plan_tile_shape(int m, int n, int k, int l, int num_sms, int* cta_group, int* tile_n);

/*
 * The order in which a persistent worker walks its range: segment `index` (0, 1, ...) as a
 * half-open unit range inside ONE output tile, or begin = end = -1 past the last one.  Order: the
 * partial tile the range starts in, the whole tiles but the last, the partial tile the range ends
 * in, the last whole tile.  A tile shared by two workers is finished by the one holding the start
 * of its k-range (its last-but-one segment); the other one published its partial sums in its
 * first segment, and the summing runs beside the MMAs of the finisher's last whole tile.
 */
int nvfp4_plan_segment(int total_units, int grid, int cta, int k_tiles, int index, int* begin, int* end);

/*
 * Host-side view of the persistent GEMM's tile order (no GPU needed): which output tile (batch,
 * row tile, column tile) the `tile`-th entry of the workers' linear tile sequence is.  The order
 * is chosen so that the tiles the workers process at the same time are neighbours in the output
 * and share operand blocks through L2 (raster_rows row tiles per group, as nvfp4_gemm_config.raster;
 * 0 = plain row-major order); every output tile appears exactly once.
 */
int nvfp4_plan_tile(int total_units, int workers, int k_tiles, int tiles_m, int tiles_n, int raster_rows, int tile, int* batch,
                    int* row_tile, int* col_tile);

/* Bytes of device scratch the library holds on the current device (0 before the first GEMM). */
size_t nvfp4_scratch_bytes(void);

/* Number of kernels this library has launched in this process (all devices). */
uint64_t nvfp4_launch_count(void);

/* Name of the kernel variant the last nvfp4_gemm / nvfp4_gemv call on this thread launched. */
const char* nvfp4_last_kernel(void);

/* Frees cached tensor maps and scratch memory on every device. */
void nvfp4_shutdown(void);

const char* nvfp4_last_error(void);
const char* nvfp4_version(void);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H */
