/*
 * CPU oracle for the NVFP4 block-scaled matmul -- plain C restatement.
 * TEST INFRASTRUCTURE ONLY: the tests, the smoke check and the bench's CPU
 * baseline use it as the checker / the timed host baseline; the product never
 * links or calls it.
 *
 * PARITY PINNED by outputs of the reference's own code: tests/golden/ref_cublaslt.json
 * holds what its cuBLASLt submission (sub_cub.py:48-143) produced on a B200 for seeded
 * inputs, and the tests hold this file to those bits.  (The reference has no CPU code,
 * golden vectors or tests for this path; its ref_kernel lives in a harness file that
 * task.yml:5 names but the repository does not contain.)  The arithmetic follows the
 * operator's definition: dequantise e2m1 x e4m3 to fp32, accumulate in fp32
 * in ascending k, round to fp16 (nearest-even, overflow -> inf).
 *
 * Layout facts followed (paths inside the reference project):
 *   - a/b: [rows, K/2] bytes, two e2m1 nibbles per byte, low nibble = lower k
 *     (template.py:9-22, task.yml:18-22)
 *   - one e4m3 (bias 7) scale per 16 K elements (submission.py:29, sub_cub.py:77-88,
 *     s_128t.py:88)
 *   - permuted scale layout: 512-byte atoms of 128 rows x 4 scales
 *     (ref.txt:31, s_128t.py:42-45,554-562)
 *   - block semantics: old_files/sub_gemm.py:170-174,211-218
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <stdatomic.h>
#include <unistd.h>

static const float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

static float e4m3fn_to_f32(uint8_t b) {
    int sign = b >> 7, e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 15 && m == 7) return NAN;
    if (e == 0) v = ldexpf((float)m / 8.0f, -6);
    else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return sign ? -v : v;
}

/* fp32 -> fp16 bits, round to nearest even, overflow to inf (what tensor.to(float16) does). */
static uint16_t f32_to_f16_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0u));
    if (absx >= 0x477FF000u) /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7C00u);
    if (absx < 0x33000001u) /* < 2^-25 (or exactly 2^-25: tie to even = 0) */
        return (uint16_t)sign;
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
    int shift;                                     /* bits to drop */
    uint32_t base;
    if (e >= -14) { shift = 13; base = (uint32_t)(e + 15) << 10; man &= 0x7FFFFFu; }
    else { shift = 13 + (-14 - e); base = 0; }
    uint32_t kept = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    uint32_t h = base + kept;
    if (rem > half || (rem == half && (kept & 1u))) h += 1; /* carries propagate into the exponent */
    return (uint16_t)(sign | h);
}

static inline size_t perm_off(int row, int col, int n_kblk) {
    return ((size_t)(row / 128) * n_kblk + (size_t)(col / 4)) * 512 + (size_t)(row % 32) * 16 +
           (size_t)((row / 32) % 4) * 4 + (size_t)(col % 4);
}

/* Dequantise one row: out[K] = e2m1[k] * scale[k/16]. */
static void dequant_row(const uint8_t* packed, const uint8_t* sf, int row, int K, int permuted, float* out) {
    int n_sf = K / 16, n_kblk = K / 64;
    for (int s = 0; s < n_sf; ++s) {
        uint8_t sb = permuted ? sf[perm_off(row, s, n_kblk)] : sf[(size_t)row * n_sf + s];
        float scale = e4m3fn_to_f32(sb);
        const uint8_t* p = packed + (size_t)row * (K / 2) + s * 8;
        for (int j = 0; j < 8; ++j) {
            out[s * 16 + 2 * j] = kE2M1[p[j] & 0xF] * scale;
            out[s * 16 + 2 * j + 1] = kE2M1[p[j] >> 4] * scale;
        }
    }
}

int nvfp4_oracle_max_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

#define NB 64 /* output columns per panel */

typedef struct {
    const uint8_t *a, *b, *sfa, *sfb;
    uint16_t* c;
    const float* aq;
    int M, N, K, permuted, n_panels;
    atomic_int next_panel;
    atomic_int rc;
} job_t;

static void* panel_worker(void* arg) {
    job_t* J = (job_t*)arg;
    const int K = J->K, M = J->M, N = J->N;
    float* bt = (float*)malloc((size_t)K * NB * sizeof(float)); /* panel, k-major: bt[k][NB] */
    float* row = (float*)malloc((size_t)K * sizeof(float));
    if (!bt || !row) {
        atomic_store(&J->rc, -2);
    } else {
        for (;;) {
            int p = atomic_fetch_add(&J->next_panel, 1);
            if (p >= J->n_panels) break;
            int j0 = p * NB, nb = (N - j0 < NB) ? (N - j0) : NB;
            memset(bt, 0, (size_t)K * NB * sizeof(float));
            for (int j = 0; j < nb; ++j) {
                dequant_row(J->b, J->sfb, j0 + j, K, J->permuted, row);
                for (int k = 0; k < K; ++k) bt[(size_t)k * NB + j] = row[k];
            }
            for (int i = 0; i < M; ++i) {
                float acc[NB];
                for (int j = 0; j < NB; ++j) acc[j] = 0.0f;
                const float* ai = J->aq + (size_t)i * K;
                for (int k = 0; k < K; ++k) {
                    float av = ai[k];
                    const float* bk = bt + (size_t)k * NB;
                    /* every product is exact in fp32 (<= 12 significant bits), so a fused or a
                       separate multiply-add rounds identically; accumulation is ascending k */
                    for (int j = 0; j < NB; ++j) acc[j] += av * bk[j];
                }
                for (int j = 0; j < nb; ++j) J->c[(size_t)i * N + j0 + j] = f32_to_f16_bits(acc[j]);
            }
        }
    }
    free(bt);
    free(row);
    return NULL;
}

/*
 * c[M][N] (fp16 bits) = dequant(a)[M][K] . dequant(b)[N][K]^T, fp32 accumulation in ascending k.
 * sfa/sfb are plain [rows][K/16] when permuted == 0, otherwise one batch of the permuted layout.
 * threads <= 0 uses every online core.
 */
int nvfp4_oracle_gemm(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, uint16_t* c,
                      int M, int N, int K, int permuted, int threads) {
    if (M <= 0 || N <= 0 || K <= 0 || (K % 64) != 0) return -1;
    if (threads <= 0) threads = nvfp4_oracle_max_threads();
    if (threads > 256) threads = 256;
    float* aq = (float*)malloc((size_t)M * K * sizeof(float));
    if (!aq) return -2;
    for (int i = 0; i < M; ++i) dequant_row(a, sfa, i, K, permuted, aq + (size_t)i * K);

    job_t J;
    J.a = a; J.b = b; J.sfa = sfa; J.sfb = sfb; J.c = c; J.aq = aq;
    J.M = M; J.N = N; J.K = K; J.permuted = permuted;
    J.n_panels = (N + NB - 1) / NB;
    atomic_init(&J.next_panel, 0);
    atomic_init(&J.rc, 0);
    if (threads > J.n_panels) threads = J.n_panels;
    pthread_t tid[256];
    int started = 0;
    for (int t = 1; t < threads; ++t)
        if (pthread_create(&tid[started], NULL, panel_worker, &J) == 0) ++started;
    panel_worker(&J);
    for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
    free(aq);
    return atomic_load(&J.rc);
}
