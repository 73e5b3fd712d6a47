// Block-diagonal randomized fast Hadamard transform along rows (the incoherence transform applied
// to activations before, and to outputs after, a quantised linear layer).
//
// One CTA transforms one block (256..4096 elements, or 256 elements holding several smaller blocks)
// of one row.  A thread holds eight consecutive elements in fp32 registers: butterfly strides 1,2,4
// run in registers, strides 8..128 as warp shuffles (__shfl_xor), and strides >= 256 through a
// shared-memory exchange.  Sign flips, the 1/sqrt(block) scale and the fp16 conversion are fused in.
#include "common.cuh"
#include "fwht.cuh"

namespace rptc {

struct HadParams {
    const void *in;
    int64_t ld_in;
    __half *out;
    int64_t ld_out;
    const __half *signs;
    const __half *residual;     // optional fp16 [rows][ld_res], added to the result
    int64_t ld_res;
    int32_t block, chunk;       // chunk: columns per CTA (a block, or 2048 = eight warps of 256 when blocks are <= 256)
    int32_t in_is_f32, transpose, clear_in;
    float scale;
    int64_t n;
};

__global__ void __launch_bounds__(512) hadamard_kernel(const HadParams p) {
    __shared__ __align__(16) float ex[4096];
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    const int t = threadIdx.x;
    const int64_t row = blockIdx.y;
    const int64_t col = (int64_t)blockIdx.x * p.chunk + 8 * t;
    if (col >= p.n) return;     // only with blocks <= 256 (whole warps leave; such blocks need no CTA barrier)
    float v[8];
    if (p.in_is_f32) load8_f32(const_cast<float *>(static_cast<const float *>(p.in)) + row * p.ld_in + col, v, p.clear_in != 0);
    else load8_f16(static_cast<const __half *>(p.in) + row * p.ld_in + col, v);
    float sg[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) sg[i] = 1.f;
    if (p.signs) load8_f16(p.signs + col, sg);
    if (!p.transpose) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= sg[i];
    }
    fwht8(v, p.block, ex);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] *= p.transpose ? p.scale * sg[i] : p.scale;
    if (p.residual) {
        float r[8];
        load8_f16(p.residual + row * p.ld_res + col, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += r[i];
    }
    store8_f16(p.out + row * p.ld_out + col, v);
}

__global__ void __launch_bounds__(512) swiglu_hadamard_kernel(const SwigluParams p) {
    __shared__ __align__(16) float ex[4096];
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    const int64_t row = blockIdx.y;
    const int64_t col = (int64_t)blockIdx.x * p.chunk + 8 * threadIdx.x;
    if (col >= p.n) return;     // only with blocks <= 256 (whole warps leave; such blocks need no CTA barrier)
    swiglu_chunk(p, row, col, ex, p.clear != 0, p.out + row * p.ld_out + col);
}

// ---- fused glue kernels of the decode step ------------------------------------------------------------
// They exist to shorten the chain of small dependent launches between two fused dequant-GEMVs.


template <int THREADS>
__global__ void __launch_bounds__(THREADS) finish_norm_hadamard_kernel(const FinishNormParams p) {
    __shared__ __align__(16) float ex[8 * THREADS];
    __shared__ float red[36];
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    finish_norm_row(p, blockIdx.x, ex, red, true, true, true);
}

// Output side of the fused qkv layer, rotary embedding and KV-cache append in one pass:
// y = s_out * H(acc) * scale over blocks of `block` (>= 128) columns of [q heads | k heads | v heads];
// q is rotated and written to `q_out`, rotated k and v go to the caches at pos[row].  Head size 128,
// rotate-half pairing (i, i + 64): the partner of a thread's eight columns sits eight threads away.
struct QkvFinishParams {
    float *acc;
    int64_t ld_acc;
    const __half *signs_out;
    float scale;
    __half *q_out;               // fp16 [rows][ld_q], hq * 128 columns
    int64_t ld_q;
    __half *kcache, *vcache;     // [rows][max_pos][hkv][128]
    const int32_t *pos;
    int32_t hq, hkv, max_pos, block, chunk;
    RopeFreq freq;
    unsigned int *status;
};

__global__ void __launch_bounds__(512) qkv_finish_kernel(const QkvFinishParams p) {
    __shared__ __align__(16) float ex[4096];
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    const int t = threadIdx.x;
    const int64_t row = blockIdx.y;
    const int col = blockIdx.x * p.chunk + 8 * t;
    float v[8], sg[8];
    const uint4 raw_so = raw8_or_ones(p.signs_out ? p.signs_out + col : nullptr);
    const int ps = p.pos[row];
    // a position outside [0, max_pos) has no row in the cache: q is still finished, k and v are dropped, the host is told
    const bool in_cache = ps >= 0 && ps < p.max_pos;
    if (!in_cache && t == 0 && blockIdx.x == 0) atomicExch(p.status, kStatusPosition);
    load8_f32(p.acc + row * p.ld_acc + col, v, true);
    fwht8(v, p.block, ex);
    unpack8(raw_so, sg);
    const float sc = p.scale * hadamard_norm_dev(p.block);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __half2float(__float2half_rn(v[i] * sc * sg[i]));     // the layer's fp16 output
    const int head = col >> 7, idx = col & 127;
    if (head < p.hq + p.hkv) {
        const bool upper = idx >= 64;
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float partner = __shfl_xor_sync(0xFFFFFFFFu, v[i], 8);
            const int j = (idx & 63) + i;                       // frequency index
            float sn, cs;
            sincosf(ps * rope_inv_freq(p.freq, j), &sn, &cs);
            o[i] = upper ? v[i] * cs + partner * sn : v[i] * cs - partner * sn;
        }
        if (head < p.hq) store8_f16(p.q_out + row * p.ld_q + col, o);
        else if (in_cache) store8_f16(p.kcache + ((row * p.max_pos + ps) * p.hkv + (head - p.hq)) * 128 + idx, o);
    } else if (in_cache) {
        store8_f16(p.vcache + ((row * p.max_pos + ps) * p.hkv + (head - p.hq - p.hkv)) * 128 + idx, v);
    }
}

static float hadamard_norm(int block) {
    float norm = 1.f;
    for (int b = block; b > 1; b >>= 2) norm *= (b >= 4) ? 0.5f : 0.70710678118654752f;
    return norm;
}

}  // namespace rptc

using namespace rptc;

extern "C" int rptc_hadamard(const void *in, int in_is_f32, int64_t ld_in, void *out, int64_t ld_out, const void *signs,
                             const void *residual, int64_t ld_res, int64_t rows, int64_t n, int block, int transpose,
                             float scale, int clear_in, rptc_stream_t stream) {
    if (!in || !out) return RPTC_ERR_ARG;
    if (block < 8 || block > 4096 || (block & (block - 1))) return RPTC_ERR_ARG;
    if (rows <= 0 || n <= 0 || (n % block) || ld_in < n || ld_out < n || (residual && ld_res < n)) return RPTC_ERR_SHAPE;
    if (rows > 65535) return RPTC_ERR_TOO_LARGE;
    const int chunk = block < 256 ? 256 : block;
    if (n % chunk) return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
        (signs && (reinterpret_cast<uintptr_t>(signs) & 15)) || (residual && (reinterpret_cast<uintptr_t>(residual) & 15)) ||
        (ld_in % 8) || (ld_out % 8) || (residual && (ld_res % 8)))
        return RPTC_ERR_ALIGN;
    if (clear_in && !in_is_f32) return RPTC_ERR_ARG;
    if (int e = rptc_check_device()) return e;
    HadParams p;
    p.in = in;
    p.ld_in = ld_in;
    p.out = static_cast<__half *>(out);
    p.ld_out = ld_out;
    p.signs = static_cast<const __half *>(signs);
    p.residual = static_cast<const __half *>(residual);
    p.ld_res = ld_res;
    p.block = block;
    p.chunk = chunk;
    p.in_is_f32 = in_is_f32;
    p.transpose = transpose;
    p.clear_in = clear_in;
    p.scale = scale * hadamard_norm(block);
    p.n = n;
    if (block <= 256 && n > 256) {
        // small blocks: a warp per 256 columns, eight warps per CTA, so that many-row inputs do not become
        // hundreds of thousands of one-warp CTAs
        p.chunk = 2048;
        return launch(hadamard_kernel, dim3((unsigned)((n + 2047) / 2048), (unsigned)rows), dim3(256), 0,
                      static_cast<cudaStream_t>(stream), p);
    }
    return launch(hadamard_kernel, dim3((unsigned)(n / chunk), (unsigned)rows), dim3(chunk / 8), 0,
                  static_cast<cudaStream_t>(stream), p);
}

static int swiglu_launch(float *acc, const void *in16, int64_t ld_in, void *out, int64_t ld_out, const void *signs_out,
                         const void *signs_in, int64_t rows, int64_t n, int block, float scale_out, float scale_in, int clear,
                         rptc_stream_t stream) {
    if ((!acc && !in16) || !out) return RPTC_ERR_ARG;
    if (block < 8 || block > 4096 || (block & (block - 1))) return RPTC_ERR_ARG;
    if (rows <= 0 || n <= 0 || (n % block) || ld_in < 2 * n || ld_out < n) return RPTC_ERR_SHAPE;
    if (rows > 65535) return RPTC_ERR_TOO_LARGE;
    const int chunk = block < 256 ? 256 : block;
    if (n % chunk) return RPTC_ERR_SHAPE;
    const void *in = acc ? static_cast<const void *>(acc) : in16;
    if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
        (signs_out && (reinterpret_cast<uintptr_t>(signs_out) & 15)) || (signs_in && (reinterpret_cast<uintptr_t>(signs_in) & 15)) ||
        (ld_in % (acc ? 4 : 8)) || (ld_out % 8) || (n % 8))
        return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    SwigluParams p;
    p.acc = acc;
    p.in16 = acc ? nullptr : static_cast<const __half *>(in16);
    p.ld_acc = ld_in;
    p.out = static_cast<__half *>(out);
    p.ld_out = ld_out;
    p.signs_out = static_cast<const __half *>(signs_out);
    p.signs_in = static_cast<const __half *>(signs_in);
    p.n = n;
    p.block = block;
    p.chunk = chunk;
    p.clear = acc ? clear : 0;
    p.scale_out = scale_out * hadamard_norm(block);
    p.scale_in = scale_in * hadamard_norm(block);
    if (block <= 256 && n > 256) {      // a warp per 256 columns, eight warps per CTA
        p.chunk = 2048;
        return launch(swiglu_hadamard_kernel, dim3((unsigned)((n + 2047) / 2048), (unsigned)rows), dim3(256), 0,
                      static_cast<cudaStream_t>(stream), p);
    }
    return launch(swiglu_hadamard_kernel, dim3((unsigned)(n / chunk), (unsigned)rows), dim3(chunk / 8), 0,
                  static_cast<cudaStream_t>(stream), p);
}

extern "C" int rptc_swiglu_hadamard(float *acc, int64_t ld_acc, void *out, int64_t ld_out, const void *signs_out,
                                    const void *signs_in, int64_t rows, int64_t n, int block, float scale_out, float scale_in,
                                    int clear, rptc_stream_t stream) {
    if (!acc) return RPTC_ERR_ARG;
    return swiglu_launch(acc, nullptr, ld_acc, out, ld_out, signs_out, signs_in, rows, n, block, scale_out, scale_in, clear, stream);
}

extern "C" int rptc_swiglu_hadamard_f16(const void *gate_up, int64_t ld_in, void *out, int64_t ld_out, const void *signs_out,
                                        const void *signs_in, int64_t rows, int64_t n, int block, float scale_out, float scale_in,
                                        rptc_stream_t stream) {
    if (!gate_up) return RPTC_ERR_ARG;
    return swiglu_launch(nullptr, gate_up, ld_in, out, ld_out, signs_out, signs_in, rows, n, block, scale_out, scale_in, 0, stream);
}

extern "C" int rptc_finish_norm_hadamard(float *acc, int64_t ld_acc, const void *signs_out, float scale_out, void *h, int64_t ld_h,
                                         const void *w_norm, float eps, const void *signs_in, int transform_in, void *out,
                                         int64_t ld_out, int64_t rows, int64_t n, rptc_stream_t stream) {
    if (!h || !w_norm || !out) return RPTC_ERR_ARG;
    if (n < 256 || n > 8192 || (n & (n - 1))) return RPTC_ERR_UNSUPPORTED;      // one Hadamard block per row, or two of 4096
    if (rows <= 0 || ld_h < n || ld_out < n || (acc && ld_acc < n)) return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(h) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(w_norm) & 15) ||
        (acc && (reinterpret_cast<uintptr_t>(acc) & 15)) || (ld_h % 8) || (ld_out % 8) || (ld_acc % 4))
        return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    FinishNormParams p;
    p.acc = acc;
    p.ld_acc = ld_acc;
    p.signs_out = static_cast<const __half *>(signs_out);
    p.scale_out = scale_out;
    p.h = static_cast<__half *>(h);
    p.h_out = nullptr;
    p.ld_h = ld_h;
    p.w_norm = static_cast<const __half *>(w_norm);
    p.eps = eps;
    p.signs_in = static_cast<const __half *>(signs_in);
    p.transform_in = transform_in;
    p.out = static_cast<__half *>(out);
    p.ld_out = ld_out;
    p.n = (int32_t)n;
    p.block = (int32_t)(n > 4096 ? 4096 : n);
    if (n > 4096)
        return launch(finish_norm_hadamard_kernel<1024>, dim3((unsigned)rows), dim3(1024), 0, static_cast<cudaStream_t>(stream), p);
    return launch(finish_norm_hadamard_kernel<512>, dim3((unsigned)rows), dim3((unsigned)(n / 8)), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" int rptc_qkv_finish(float *acc, int64_t ld_acc, const void *signs_out, float scale, void *q_out, int64_t ld_q,
                               void *kcache, void *vcache, const int32_t *pos, int64_t rows, int hq, int hkv, int max_pos, int block,
                               float theta, rptc_stream_t stream) {
    if (!acc || !q_out || !kcache || !vcache || !pos) return RPTC_ERR_ARG;
    if (block < 128 || block > 4096 || (block & (block - 1))) return RPTC_ERR_ARG;
    const int64_t n = (int64_t)(hq + 2 * hkv) * 128;
    const int chunk = block < 256 ? 256 : block;
    if (rows <= 0 || rows > 65535 || hq <= 0 || hkv <= 0 || (n % chunk) || ld_acc < n || ld_q < (int64_t)hq * 128 || max_pos <= 0)
        return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(acc) & 15) || (reinterpret_cast<uintptr_t>(q_out) & 15) || (reinterpret_cast<uintptr_t>(kcache) & 15) ||
        (reinterpret_cast<uintptr_t>(vcache) & 15) || (ld_acc % 4) || (ld_q % 8))
        return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    QkvFinishParams p;
    p.acc = acc;
    p.ld_acc = ld_acc;
    p.signs_out = static_cast<const __half *>(signs_out);
    p.scale = scale;
    p.q_out = static_cast<__half *>(q_out);
    p.ld_q = ld_q;
    p.kcache = static_cast<__half *>(kcache);
    p.vcache = static_cast<__half *>(vcache);
    p.pos = pos;
    p.hq = hq;
    p.hkv = hkv;
    p.max_pos = max_pos;
    p.block = block;
    p.chunk = chunk;
    p.freq = rope_freq(theta, 128);
    p.status = device_status_word();
    if (!p.status) return RPTC_ERR_CUDA;
    return launch(qkv_finish_kernel, dim3((unsigned)(n / chunk), (unsigned)rows), dim3(chunk / 8), 0, static_cast<cudaStream_t>(stream), p);
}
