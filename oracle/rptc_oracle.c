/* CPU oracle in C for the RPTC decode + matvec path.  TEST / BASELINE INFRASTRUCTURE ONLY.
 *
 * A multi-threaded (OpenMP) restatement of the reference's decoder, used (a) as a second,
 * independent checker beside the numpy oracle and (b) as the timed CPU baseline of the benchmark.
 * The product never links or loads this file.
 *
 * What it follows in the reference:
 *   code A (LUT):   state = ((state << K) | sym) & (2^L - 1); w = alphabet[state]   rptc.py:74-85
 *                   words are consumed MSB first                                     inference.cu:66-94
 *   code B (hash):  4 bits per step; hash = t*(t+1); entry = (hash >> 8) & (2^S-1);
 *                   sign of the low half := hash bit 15                              inference.cu:250-262
 *   code C (lite):  h = x*(2x+1); h ^= h >> (L-S); idx = h & (2^S-1); V = 2          rptc_lite.py:12-16,63-73
 * Packed layouts: row-major [m][units*4] (inference.cu:53-66) and unit-major [units][m][4]
 * (inference_t.cu:116).  The row's shift register starts at 0 (rptc.py:82) or at carry_in[row].
 *
 * Pin status: validated against the numpy oracle (tests/test_oracle.py); see that module's header
 * for how the pair is pinned to the reference.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static float h2f_table[65536];
static int h2f_ready = 0;
static void h2f_init(void) {
    if (h2f_ready) return;
    for (uint32_t i = 0; i < 65536u; i++) h2f_table[i] = half_to_float((uint16_t)i);
    h2f_ready = 1;
}

enum { CODE_A = 0, CODE_B = 1, CODE_C = 2 };
enum { LAYOUT_ROWMAJOR = 0, LAYOUT_UNITMAJOR = 2 };

/* Worker threads for the calls that follow (a launcher may have exported OMP_NUM_THREADS=1 for its children). */
void rptc_oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int rptc_oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

static inline uint32_t word_at(const uint32_t *codes, int layout, int64_t m, int64_t n_words, int64_t row, int64_t w) {
    if (layout == LAYOUT_ROWMAJOR) return codes[row * n_words + w];
    return codes[((w >> 2) * m + row) * 4 + (w & 3)];
}

/* Decodes one row into `dst` (n raw fp16 bit patterns).  Sequential shift register, as the
 * reference's scan does it (rptc.py:77-83). */
static void decode_row(const uint32_t *codes, int layout, int64_t m, int64_t n, int64_t row, const uint16_t *lut,
                       int code, int K, int L, int S, uint32_t carry, uint16_t *dst) {
    const int bits_per_step = (code == CODE_A) ? K : 2 * K;
    const int64_t n_steps = (code == CODE_A) ? n : n / 2;
    const int64_t n_words = ((n * K + 127) / 128) * 4;
    const uint32_t lmask = (L >= 32) ? 0xFFFFFFFFu : ((1u << L) - 1u);
    const uint32_t smask = (1u << S) - 1u;
    uint64_t buf = 0;      /* bits not yet consumed, right-aligned */
    int have = 0;
    int64_t wi = 0;
    uint32_t state = carry & 0xFFFFu;
    for (int64_t s = 0; s < n_steps; s++) {
        if (have < bits_per_step) {
            uint32_t wd = (wi < n_words) ? word_at(codes, layout, m, n_words, row, wi) : 0u;
            wi++;
            buf = (buf << 32) | wd;
            have += 32;
        }
        uint32_t sym = (uint32_t)((buf >> (have - bits_per_step)) & ((1u << bits_per_step) - 1u));
        have -= bits_per_step;
        state = ((state << bits_per_step) | sym) & 0xFFFFu;
        if (code == CODE_A) {
            dst[s] = lut[state & lmask];
        } else if (code == CODE_B) {
            uint32_t h = state * (state + 1u);
            uint32_t e = (h >> 8) & smask;
            dst[2 * s] = (uint16_t)((lut[2 * e] & 0x7FFFu) | (h & 0x8000u));
            dst[2 * s + 1] = lut[2 * e + 1];
        } else {
            uint32_t x = state & lmask;
            uint32_t h = (x * (2u * x + 1u)) & lmask;
            h ^= h >> (L - S);
            uint32_t e = h & smask;
            dst[2 * s] = lut[2 * e];
            dst[2 * s + 1] = lut[2 * e + 1];
        }
    }
}

/* Packed codes -> dense fp16 [m][n].  Returns 0. */
int rptc_oracle_decompress(const uint32_t *codes, int layout, const uint16_t *lut, const uint32_t *carry_in,
                           uint16_t *out, int64_t m, int64_t n, int code, int K, int L, int S) {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < m; row++)
        decode_row(codes, layout, m, n, row, lut, code, K, L, S, carry_in ? carry_in[row] : 0u, out + row * n);
    return 0;
}

/* Fused decode + matvec with fp32 accumulation: y[b][m] (float) = x[b][n] (fp16) . W^T.
 * `scratch` must hold threads*n uint16 values. */
int rptc_oracle_gemv(const uint32_t *codes, int layout, const uint16_t *lut, const uint32_t *carry_in,
                     const uint16_t *x, float *y, uint16_t *scratch, int64_t m, int64_t n, int batch,
                     int code, int K, int L, int S) {
    h2f_init();
#pragma omp parallel
    {
#ifdef _OPENMP
        uint16_t *row_w = scratch + (size_t)omp_get_thread_num() * n;
#else
        uint16_t *row_w = scratch;
#endif
#pragma omp for schedule(static)
        for (int64_t row = 0; row < m; row++) {
            decode_row(codes, layout, m, n, row, lut, code, K, L, S, carry_in ? carry_in[row] : 0u, row_w);
            for (int b = 0; b < batch; b++) {
                const uint16_t *xb = x + (size_t)b * n;
                float acc = 0.f;
                for (int64_t c = 0; c < n; c++) acc += h2f_table[row_w[c]] * h2f_table[xb[c]];
                y[(size_t)b * m + row] = acc;
            }
        }
    }
    return 0;
}
