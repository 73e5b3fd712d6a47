/* rptc_b200 — C ABI of the B200 (sm_100a) RPTC decode / fused dequant-matmul library.
 *
 * Every entry point takes plain device pointers and sizes, runs on the CUDA stream it is given
 * (0 = the legacy default stream), allocates nothing unless it says so, never creates streams,
 * never exits or traps, and returns RPTC_OK (0) or a negative rptc_status.  All tensors are
 * caller-owned device memory.  This is the boundary the reference's pybind module
 * `rptc_kernels` (rptc_kernels/csrc/rptc_kernels/wrapper.cpp:59-67) binds for its seven
 * functions; the Python shim of the same name calls these through ctypes.
 *
 * Terms.  A weight matrix W is [m, n] (out_features, in_features).  Each row is one trellis
 * bitstream, packed MSB-first into 32-bit words (inference.cu:70-71); a "unit" is 128 bits
 * (4 words).  The shift-register state is the last 16 bits of the row's stream, zero before the
 * row start (rptc.py:77-83) or `carry_in[row]` when the tensor is a column shard.
 */
#ifndef RPTC_B200_H
#define RPTC_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *rptc_stream_t; /* a cudaStream_t */

typedef enum {
    RPTC_OK = 0,
    RPTC_ERR_ARG = -1,         /* null pointer, bad enum value */
    RPTC_ERR_SHAPE = -2,       /* m, n, batch violate a divisibility rule */
    RPTC_ERR_ALIGN = -3,       /* pointer not 16-byte aligned / leading dimension not a multiple of 8 */
    RPTC_ERR_UNSUPPORTED = -4, /* combination of code / K / layout not implemented */
    RPTC_ERR_CUDA = -5,        /* a CUDA runtime call failed; see rptc_last_cuda_error() */
    RPTC_ERR_TIMEOUT = -6,     /* a bounded device-side wait ran out (see rptc_device_status) */
    RPTC_ERR_TOO_LARGE = -7,   /* size beyond a documented maximum */
    RPTC_ERR_DEVICE = -8,      /* the current device is not compute capability 10.x */
    RPTC_ERR_INTERNAL = -9,    /* a kernel found its shared-memory layout violated and did nothing (rptc_device_status) */
    RPTC_ERR_RANGE = -10       /* a sequence position lay outside [0, max_pos): the cache access was skipped
                                  (rptc_device_status) */
} rptc_status;

/* Trellis codes.
 *   RPTC_CODE_LUT  : w = lut[state & (2^L-1)], K bits per weight (rptc.py:74-85; decompress_kernel,
 *                    inference.cu:66-94, is L=16 K=2).  lut: fp16 [2^L].
 *   RPTC_CODE_HASH : the fused reference kernel's code (inference.cu:250-262): 4 bits per step, two
 *                    weights per step, h = t(t+1), entry (h>>8)&(2^S-1) of 2^S fp16 pairs, sign of the
 *                    low half := bit 15 of h.  K must be 2.  lut: fp16 [2^(S+1)], S = 6 or 8.
 *   RPTC_CODE_LITE : rptc_lite.py:12-16,63-73: h = x(2x+1); h ^= h>>(L-S); entry h&(2^S-1) of 2^S
 *                    fp16 pairs; 2K bits per step.  lut: fp16 [2^S][2], S <= 10. */
enum { RPTC_CODE_LUT = 0, RPTC_CODE_HASH = 1, RPTC_CODE_LITE = 2 };

/* Layouts of the packed words (int32).
 *   ROWMAJOR  [m][units*4]            decompress_kernel, inference.cu:53-66
 *   CHUNKED   [units/32][m][32*4]     decompress_matvec_kernel, inference.cu:229
 *   UNITMAJOR [units][m][4]           decompress_matvec_t_kernel, inference_t.cu:116
 *   TILED     [m/32][units][32][4]    the native layout of this library (no reference counterpart):
 *                                     the 32 rows of one unit are 512 contiguous bytes that one warp takes
 *                                     as coalesced 128-bit loads, and consecutive units of a 32-row block
 *                                     follow one another, so a warp's whole share of the matrix is one
 *                                     linear stream for the bulk-copy (TMA) engine. */
enum { RPTC_LAYOUT_ROWMAJOR = 0, RPTC_LAYOUT_CHUNKED = 1, RPTC_LAYOUT_UNITMAJOR = 2, RPTC_LAYOUT_TILED = 3 };

/* Optional reproduction of two defects of the reference kernels, so that results can be compared
 * element for element with the reference binary.  0 = the self-consistent stream of rptc.py. */
enum {
    RPTC_QUIRK_NONE = 0,
    RPTC_QUIRK_K1_LANE0_SEED = 1, /* inference.cu:61-62: every 32nd unit seeds from the high half of the previous word */
    RPTC_QUIRK_K2_LANE0_CARRY = 2 /* inference.cu:232: every 32nd unit takes its own last word as the carry */
};

/* How the activation vector is paired with the stream in rptc_gemv.
 *   NATURAL   : column c of W multiplies x[c].
 *   K2_LEGACY : the staging permutation of decompress_matvec_kernel (inference.cu:216-221,249);
 *               needs n % 2048 == 0. */
enum { RPTC_XORDER_NATURAL = 0, RPTC_XORDER_K2_LEGACY = 1 };

typedef struct {
    int32_t code;   /* RPTC_CODE_* */
    int32_t K;      /* bits per weight: 2, 3 or 4 */
    int32_t L;      /* state bits, <= 16 */
    int32_t S;      /* log2(number of LUT pairs) for HASH / LITE; ignored for LUT */
    int32_t layout; /* RPTC_LAYOUT_* */
    int32_t quirk;  /* RPTC_QUIRK_* */
} rptc_format;

const char *rptc_strerror(int status);
int rptc_version(void);
/* cudaError_t of the last failing runtime call made by this library on the calling thread. */
int rptc_last_cuda_error(void);
/* RPTC_OK when the current device is a compute-capability 10.x GPU, else RPTC_ERR_DEVICE. */
int rptc_check_device(void);
/* Reads (and clears) the device-side status word.  0, or what a kernel reported since the last call:
 * RPTC_ERR_TIMEOUT (a bounded wait on one of its own asynchronous copies, on a peer or on the host ran out),
 * RPTC_ERR_RANGE (a position outside the KV cache: the access was skipped, nothing was written out of bounds),
 * RPTC_ERR_INTERNAL (shared-memory plan mismatch).  Synchronises the device. */
int rptc_device_status(void);
/* Launch kernels with programmatic dependent launch (1) or plainly (0, default).  The setting belongs to the
 * calling thread: launches made by other threads are not affected. */
void rptc_set_pdl(int enable);

/* Re-tiles packed codes between layouts (a pure permutation of 128-bit units).
 * Replaces nothing in the reference: it connects the reference's three layouts.  m % 32 == 0. */
int rptc_repack(const void *src, int src_layout, void *dst, int dst_layout, int64_t m, int64_t n_units,
                rptc_stream_t stream);

/* Packed codes -> dense fp16 out[m][ld_out] (first n columns written).
 * Replaces decompress(compressed, codebook, out), inference.cu:99-160 / wrapper.cpp:60, and
 * generalises it to K = 2,3,4, all three codes and layouts, n % (128*P/K) == 0 (P = 3 for K = 3,
 * else 1), m % 32 == 0.  carry_in may be NULL. */
int rptc_decompress(const void *codes, const void *lut, const uint32_t *carry_in, void *out, int64_t ld_out,
                    int64_t m, int64_t n, const rptc_format *fmt, rptc_stream_t stream);

/* Fused decode + matvec, batch 1..64:  acc[b][row] += sum_c W[row][c] * x[b][c]   (fp32 acc).  One launch serves up to
 * eight activation rows; larger batches (decode batch 16) run as consecutive launches of eight.
 * Replaces the kernels behind decompress_matvec_{16,20}_{6,8}_1 (inference.cu:189-277) and
 * decompress_matvec_t_{16,14} (inference_t.cu:68-175).  `acc` is fp32 SCRATCH of [batch][ld_acc]
 * that the caller zeroes (or pre-loads) and later converts with rptc_gemv_finish; partial sums
 * are added with atomics, so the low bits of a result can differ between runs.
 * x: fp16 [batch][ld_x].  K = 2 or 4.  m % 32 == 0, n % (128/K) == 0. */
int rptc_gemv(const void *codes, const void *lut, const uint32_t *carry_in, const void *x, int64_t ld_x,
              float *acc, int64_t ld_acc, int64_t m, int64_t n, int batch, int x_order, const rptc_format *fmt,
              rptc_stream_t stream);

/* rptc_gemv whose activations are not read from memory but computed, by every CTA for itself, from what the
 * previous layer of a decoder block left behind: the glue between the two layers then costs no launch of its own.
 *   h' = h_in + s_out * H(acc) * scale_out;   x = H(s_in * rmsnorm(h') * w_norm)
 * (what rptc_finish_norm_hadamard computes; n must be 4096 or 8192: one or two 4096-point Hadamard blocks).  CTA 0 stores h' to h_out,
 * which must not alias h_in (other CTAs still read h_in).  `acc` is read by every CTA and therefore not cleared
 * here: name it as `clear` in a LATER launch of the same stream (a launch zeroes its own `clear` range once the
 * launches before it have completed).  TILED layout, no quirk, batch 1-2.  No reference counterpart (the
 * reference runs these steps as separate JAX ops). */
typedef struct rptc_gemv_input {
    const float *acc;       /* previous layer's accumulator, fp32 [batch][ld_acc >= n], or NULL (h_in as it is) */
    int64_t ld_acc;
    const void *signs_out;  /* previous layer's output-side signs, fp16 [n]; NULL = ones */
    float scale_out;        /* previous layer's scale */
    float eps;              /* RMSNorm epsilon */
    const void *signs_in;   /* this layer's input-side signs, fp16 [n]; NULL = ones */
    const void *h_in;       /* residual stream, fp16 [batch][ld_h] */
    void *h_out;            /* updated residual stream */
    int64_t ld_h;
    const void *w_norm;     /* RMSNorm weight, fp16 [n] */
    float *clear;           /* optional fp32 range this launch zeroes */
    int64_t clear_count;    /* floats; multiple of 4 */
} rptc_gemv_input;
int rptc_gemv_glued(const void *codes, const void *lut, const uint32_t *carry_in, const rptc_gemv_input *in, float *acc,
                    int64_t ld_acc, int64_t m, int64_t n, int batch, const rptc_format *fmt, rptc_stream_t stream);

/* The down projection of a gated MLP with its activations made inside the launch: rptc_gemv whose x is what
 * rptc_swiglu_hadamard would have written from the gate-up layer's accumulator `prev_acc` (fp32 [batch][ld_prev >= 2n],
 * gate in columns [0, n), up in [n, 2n)): x = H(s_in * silu(g) * u), (g | u) = s_out * H(prev_acc) * scale_out, with
 * Hadamard blocks of `block` <= 256 columns.  The work is ordered by 256-column blocks so that a CTA makes only the
 * one or two blocks of x that its share of the matrix multiplies.  prev_acc is read by several CTAs and not cleared;
 * `clear` (optional, fp32, clear_count a multiple of 4) is a range this launch zeroes once the launches before it
 * have completed.  TILED layout, no quirk, batch 1-2, n % 256 == 0.  No reference counterpart. */
int rptc_gemv_swiglu(const void *codes, const void *lut, const uint32_t *carry_in, const float *prev_acc, int64_t ld_prev,
                     const void *signs_out, float scale_out, const void *signs_in, int block, float *acc, int64_t ld_acc,
                     int64_t m, int64_t n, int batch, const rptc_format *fmt, float *clear, int64_t clear_count,
                     rptc_stream_t stream);

/* y[b][i] = fp16(scale * acc[b][i] (+ y[b][i] if accumulate));  acc[b][i] = 0 if clear.
 * accumulate = 1 gives decompress_matvec_t's `out +=` (inference_t.cu:170-171). */
int rptc_gemv_finish(float *acc, int64_t ld_acc, void *y, int64_t ld_y, int64_t m, int batch, float scale,
                     int accumulate, int clear, rptc_stream_t stream);

/* The fused matvec for callers that cannot allocate device memory where they call this library (a server whose
 * memory pool owns the whole device, a plugin that must not go around its host's allocator, a process with a
 * frozen footprint).  Same product as rptc_gemv + rptc_gemv_finish, y[b][row] = fp16(sum_c W[row][c] x[b][c]),
 * but the fp32 accumulator is a fixed 1 MiB array inside the library instead of caller scratch:
 * batch * m <= 262144 or the call returns RPTC_ERR_TOO_LARGE.  It calls no allocating routine.  The first call
 * on each device looks up the array's device address (make that call before any stream capture).  All calls
 * on a device share the one array: calls that may overlap on the GPU (different streams) race and must be
 * serialised by the caller.  It has no counterpart in the reference. */
int rptc_gemv_f16_static(const void *codes, const void *lut, const uint32_t *carry_in, const void *x, int64_t ld_x, void *y,
                         int64_t ld_y, int64_t m, int64_t n, int batch, int x_order, const rptc_format *fmt,
                         rptc_stream_t stream);

/* Fused decode + GEMM for prefill (tcgen05 tensor cores, TMEM accumulators):
 * y[t][row] = fp16( sum_c x[t][c] * W[row][c] ),  x fp16 [tokens][ld_x], y fp16 [tokens][ld_y].
 * No reference counterpart (the reference has batch-1 kernels only); the equivalent reference
 * computation is decompress followed by a dense matmul (rptc_kernels/tests/test_decompress.py:41-43).
 * TILED layout, K = 2 or 4, m % 128 == 0, n % 64 == 0. */
int rptc_gemm(const void *codes, const void *lut, const uint32_t *carry_in, const void *x, int64_t ld_x, void *y,
              int64_t ld_y, int64_t m, int64_t n, int64_t tokens, const rptc_format *fmt, rptc_stream_t stream);

/* Block-diagonal randomized Hadamard transform along rows of length n (block = power of two <= 4096
 * dividing n).  No reference counterpart (incoherence processing is an extension of this build).
 *   in_is_f32 = 0: in is fp16 [rows][ld_in];  1: in is fp32 (e.g. the rptc_gemv accumulator).
 *   transpose = 0: out = H (s * in) * scale        (activation side)
 *   transpose = 1: out = s * (H in) * scale        (output side)
 *   clear_in  = 1 (fp32 input only): zero the input after reading it.
 * signs: fp16 [n] of +-1, or NULL for all +1.  residual: optional fp16 [rows][ld_res] added to the
 * result (a transformer block's skip connection).  out: fp16 [rows][ld_out]; may alias an fp16 input
 * or the residual. */
int rptc_hadamard(const void *in, int in_is_f32, int64_t ld_in, void *out, int64_t ld_out, const void *signs,
                  const void *residual, int64_t ld_res, int64_t rows, int64_t n, int block, int transpose, float scale,
                  int clear_in, rptc_stream_t stream);

/* Fused middle of a gated MLP between two quantised layers.  acc: fp32 [rows][ld_acc] accumulator of the
 * fused gate-up layer (gate in columns [0,n), up in [n,2n)).  g,u = s_out * (H acc) * scale_out;
 * out = H (s_in * (silu(g) * u)) * scale_in, fp16 [rows][ld_out].  No reference counterpart. */
int rptc_swiglu_hadamard(float *acc, int64_t ld_acc, void *out, int64_t ld_out, const void *signs_out, const void *signs_in,
                         int64_t rows, int64_t n, int block, float scale_out, float scale_in, int clear, rptc_stream_t stream);
/* The same from the fp16 output of a matrix product (the prefill path): gate_up fp16 [rows][ld_in >= 2n]. */
int rptc_swiglu_hadamard_f16(const void *gate_up, int64_t ld_in, void *out, int64_t ld_out, const void *signs_out,
                             const void *signs_in, int64_t rows, int64_t n, int block, float scale_out, float scale_in,
                             rptc_stream_t stream);

/* --- the non-quantised pieces of a Llama-architecture decode step (no reference counterpart: the
 * reference evaluates models through Hugging Face transformers, quantize_hf.py:230-236) --- */

/* out = x * rsqrt(mean(x^2) + eps) * w, fp16 rows of length n. */
int rptc_rmsnorm(const void *x, int64_t ld_x, const void *w, void *out, int64_t ld_out, int64_t rows, int64_t n, float eps,
                 rptc_stream_t stream);
/* Rotary embedding (rotate-half pairs (i, i+d/2)) of one token per row of qkv = [q heads | k heads | v heads],
 * q in place, rotated k and v appended to caches [rows][max_pos][hkv][d] at pos[row]. */
int rptc_rope_cache(void *qkv, int64_t ld_qkv, const int32_t *pos, void *kcache, void *vcache, int64_t rows, int hq, int hkv,
                    int d, int max_pos, float theta, rptc_stream_t stream);
/* The same for a whole prompt: qkv fp16 [rows * tokens][ld_qkv], token t of row r in row r * tokens + t, written to
 * cache positions 0 .. tokens-1. */
int rptc_rope_cache_prompt(void *qkv, int64_t ld_qkv, int64_t rows, int64_t tokens, void *kcache, void *vcache, int hq, int hkv,
                           int d, int max_pos, float theta, rptc_stream_t stream);
/* Single-query attention of each row's q heads over cache positions [0, pos[row]]; d must be 128.
 * qkv, kcache and vcache must be 16-byte aligned and ld_qkv a multiple of 8 (rows are read 16 bytes at a time).
 * signs_in (fp16 [hq*128] or NULL): when given, each head's output is also put through the input-side
 * transform of the output projection with one 128-wide Hadamard block per head, H(s * o) / sqrt(128). */
int rptc_attn_decode(const void *qkv, int64_t ld_qkv, const int32_t *pos, const void *kcache, const void *vcache, void *out,
                     int64_t ld_out, int64_t rows, int hq, int hkv, int d, int max_pos, float scale, const void *signs_in,
                     rptc_stream_t stream);
/* rptc_qkv_finish + rptc_attn_decode in one launch (head size 128, the qkv layer's output transform in 128-wide
 * blocks, heads a multiple of kv_heads): each (row, q head) CTA finishes its own q and the k, v of its kv head from
 * the fused qkv accumulator acc = [q heads | k heads | v heads], the first q head of each group appends k, v at
 * pos[row], and every CTA attends over positions [0, pos[row]] and writes its head's output (through the 128-wide
 * input transform of the output projection when signs_in is given).  With heads == kv_heads acc is left zeroed;
 * otherwise (k and v are read by every q head of their group) acc is left as it is and the caller zeroes it. */
int rptc_qkv_attn_decode(float *acc, int64_t ld_acc, const void *signs_out, float scale_out, const int32_t *pos, void *kcache,
                         void *vcache, void *out, int64_t ld_out, int64_t rows, int heads, int kv_heads, int max_pos, float theta,
                         const void *signs_in, rptc_stream_t stream);
/* Glue between two quantised layers of a decoder block in one launch (rows that are a single Hadamard
 * block, n = 256..4096):  if acc: h += s_out * H(acc) * scale_out (acc cleared);  xn = rmsnorm(h) * w_norm;
 * out = transform_in ? H(s_in * xn) / sqrt(n) : xn. */
int rptc_finish_norm_hadamard(float *acc, int64_t ld_acc, const void *signs_out, float scale_out, void *h, int64_t ld_h,
                              const void *w_norm, float eps, const void *signs_in, int transform_in, void *out, int64_t ld_out,
                              int64_t rows, int64_t n, rptc_stream_t stream);
/* Output side of a fused qkv layer + rotary embedding + KV-cache append: y = s_out * H(acc) * scale in blocks of
 * `block` >= 128 columns of [q | k | v] (128 per head); rotated q -> q_out, rotated k and v -> caches at pos[row]. */
int rptc_qkv_finish(float *acc, int64_t ld_acc, const void *signs_out, float scale, void *q_out, int64_t ld_q, void *kcache,
                    void *vcache, const int32_t *pos, int64_t rows, int hq, int hkv, int max_pos, int block, float theta,
                    rptc_stream_t stream);
/* Dense fp16 matvec y[b] = W x[b] (fp32 accumulation), batch 1..8: the output head, and the dense-bandwidth
 * probe the reference's tests call `matvec` (rptc_kernels/tests/test_matvec.py:18, not exported by wrapper.cpp). */
int rptc_dense_gemv(const void *W, int64_t ld_w, const void *x, int64_t ld_x, void *y, int64_t ld_y, int64_t m, int64_t n,
                    int batch, rptc_stream_t stream);
/* out[r] = table[ids[r]], fp16 rows of length n.  `ids` may live in pinned host memory (read over PCIe by the
 * kernel: the step's input then needs no copy of its own). */
int rptc_embed(const void *table, const int32_t *ids, void *out, int64_t ld_out, int64_t rows, int64_t n, rptc_stream_t stream);
/* The end of a greedy decode step: next[r] = argmax(logits[r][0:n]) (first maximum), ids[r] = next[r] and pos[r] += 1
 * when given, and mirror[r] = next[r] when given (pinned host memory: the host reads the token after synchronising
 * the stream; see rptc_embed_mailbox for steps_done, NULL otherwise).  logits fp16 [rows][ld]; n even. */
int rptc_next_token(const void *logits, int64_t ld, int64_t rows, int64_t n, int64_t *next, int32_t *ids, int32_t *pos,
                    int64_t *mirror, const uint32_t *steps_done, rptc_stream_t stream);
/* Token ids through a mailbox in pinned host memory, for a host that queues the next step before it knows the
 * step's token.  slots[r] = (sequence << 32) | id, written by the host with one 8-byte store.  The kernel polls
 * until every slot carries sequence *steps_done + 1 (device counter, starts at 0), for at most timeout_ms; on
 * expiry rptc_device_status() reports RPTC_ERR_TIMEOUT and the step runs with the ids it found.  It then stores
 * the ids to `ids`, sets *steps_done to the sequence number and copies the embedding rows to `out`.  With the same
 * `steps_done`, rptc_next_token writes mirror[r] = (sequence << 32) | chosen id.  rows <= 64. */
int rptc_embed_mailbox(const void *table, const uint64_t *slots, uint32_t *steps_done, int32_t *ids, void *out, int64_t ld_out,
                       int64_t rows, int64_t n, int64_t vocab, int timeout_ms, rptc_stream_t stream);

/* --- the code-A trellis encoder (rptc.py:13-71 `quantize`, diagonal corrections; K = 2 bits per weight) ---
 * For each of `rows` sample rows (fp32 [rows][ld_samples], n used) the symbols in 0..3 (int32 [rows][ld_sym]) whose
 * shift-register walk from state 0 minimises sum_i pos_weight[i] * (samples[i] - alphabet[state_i])^2, and that
 * minimum (loss[rows]).  alphabet fp32 [2^L], 4 <= L <= 16.  First-minimum tie breaks and unfused fp32 arithmetic, as
 * in the reference.  workspace: rptc_viterbi_workspace_bytes(rows, n, L) bytes of device memory, 256-byte aligned
 * (two cost arrays and one survivor byte per position, row and state prefix: 16 KiB per row and position at L = 16). */
int64_t rptc_viterbi_workspace_bytes(int64_t rows, int64_t n, int L);
int rptc_viterbi_encode(const float *alphabet, const float *pos_weight, const float *samples, int64_t ld_samples, int64_t rows,
                        int64_t n, int L, int32_t *symbols, int64_t ld_sym, float *loss, void *workspace, int64_t workspace_bytes,
                        rptc_stream_t stream);

/* --- tensor-parallel decode: output transform + all-reduce + residual add in one kernel over NVLink peer
 * memory (no reference counterpart; the reference has no distributed code) ---
 * rptc_peer_alloc / export / import / close / free: an exchange buffer of this process (cudaMalloc, zeroed),
 * its 64-byte CUDA IPC handle, and the mapping of a peer's handle; the caller passes handles between ranks. */
int rptc_peer_alloc(int64_t bytes, void **ptr);
int rptc_peer_free(void *ptr);
int rptc_peer_export(void *ptr, unsigned char *handle64);
int rptc_peer_import(const unsigned char *handle64, void **ptr);
int rptc_peer_close(void *ptr);
/* h[rows][n] += sum over ranks of fp16( s_out * H(acc_rank) * scale );  acc is cleared.
 * data_ptrs[r]: rank r's exchange buffer, 2 * world * rows * n * 4 bytes, zero-initialised: [2][world][rows*n/2] 64-bit
 * words, each a 32-bit piece of payload with the exchange's epoch above it (the flag travels with the data; a 64-bit
 * store arrives whole, so the receiver only polls its own buffer).  flag_ptrs: unused, may be NULL.  epochs: local
 * uint32 [ctas], ctas = rows * n / max(block,256), zero-initialised.
 * Every rank must call it the same number of times with the same shapes.  A rank that waits longer than
 * timeout_ms (0 = 2000) for a peer gives up: the device status word is raised (rptc_device_status) and h is
 * left untouched for the pieces it could not finish. */
int rptc_peer_finish(float *acc, int64_t ld_acc, const void *signs_out, float scale, void *h, int64_t ld_h,
                     void *const *data_ptrs, void *const *flag_ptrs, void *epochs, int rank, int world, int64_t rows,
                     int64_t n, int block, int64_t timeout_ms, rptc_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* RPTC_B200_H */
