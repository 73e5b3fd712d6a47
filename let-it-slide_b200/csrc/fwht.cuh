// Eight-values-per-thread Walsh-Hadamard building blocks shared by the transform, glue and all-reduce kernels.
#pragma once
#include <math.h>
#include "common.cuh"

namespace rptc {

// Rotary frequencies theta^(-2j/d) = 2^(j * c) with c = -2 log2(theta) / d.  The host computes c in double precision
// and hands it over as a float pair (hi + lo), so that the device gets the exponent to ~1e-8 with one fused
// multiply-add and the frequency with one exp2f: as accurate as an fp32 pow, at a fraction of its instruction count
// (the positions multiply the frequency's error: at position 2047 a 1e-6 relative error is already 2e-3 rad).
struct RopeFreq {
    float c_hi, c_lo;
};
inline RopeFreq rope_freq(float theta, int d) {
    const double c = -2.0 * log2((double)theta) / (double)d;
    RopeFreq f;
    f.c_hi = (float)c;
    f.c_lo = (float)(c - (double)f.c_hi);
    return f;
}
#ifdef __CUDACC__
__device__ __forceinline__ float rope_inv_freq(const RopeFreq &f, int j) { return exp2f(fmaf((float)j, f.c_hi, (float)j * f.c_lo)); }
#endif

struct NoHook {      // default of the `after_loads` hooks below
    __device__ __forceinline__ void operator()() const {}
};

__device__ __forceinline__ void load8_f16(const __half *p, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4 *>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(u32_as_half2(w[i]));
        v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void unpack8(const uint4 a, float (&v)[8]) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(u32_as_half2(w[i]));
        v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
}
// eight fp16 values as raw bits; a null pointer reads as eight ones (0x3C00)
__device__ __forceinline__ uint4 raw8_or_ones(const __half *p) {
    return p ? *reinterpret_cast<const uint4 *>(p) : make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);
}
__device__ __forceinline__ void load8_f32(float *p, float (&v)[8], bool clear) {
    const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    if (clear) {
        *reinterpret_cast<float4 *>(p) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4 *>(p + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
}
__device__ __forceinline__ void store8_f16(__half *p, const float (&v)[8]) {
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = half2_as_u32(__floats2half2_rn(v[2 * i], v[2 * i + 1]));
    *reinterpret_cast<uint4 *>(p) = make_uint4(o[0], o[1], o[2], o[3]);
}

// Unnormalised Walsh-Hadamard transform of `block`-sized blocks; thread t holds elements 8t..8t+7 of
// the CTA's chunk.  `ex` is a shared exchange buffer of chunk floats (used when block > 256).
// `guard`: a barrier before the exchange buffer is written (needed unless every thread is known to have passed a
// barrier since the buffer was last read).
__device__ __forceinline__ void fwht8(float (&v)[8], int block, float *ex, bool guard = true) {
    const int t = threadIdx.x;
#pragma unroll
    for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if ((i & h) == 0) {
                const float a = v[i], b = v[i + h];
                v[i] = a + b;
                v[i + h] = a - b;
            }
        }
    }
    for (int lm = 1; lm < 32 && 8 * lm < block; lm <<= 1) {
        const bool upper = (t & lm) != 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float o = __shfl_xor_sync(0xFFFFFFFFu, v[i], lm);
            v[i] = upper ? o - v[i] : v[i] + o;
        }
    }
    if (block > 256) {
        // Strides 256 .. block/2 mix the 256-element groups: element 256*g + r with element 256*g' + r.  Through
        // shared memory each of the first chunk/16 threads takes the G = block/256 group values of one r,
        // transforms them in registers, and puts them back (two barriers instead of one per stride).
        const int G = block >> 8;                      // 2, 4, 8 or 16
        if (guard) __syncthreads();          // the buffer may still be read from an earlier transform
        // a thread's eight values as two 16-byte accesses (`ex` is 16-byte aligned): scalar accesses 32 bytes apart
        // would meet in the same banks eight at a time
        float4 *ex4 = reinterpret_cast<float4 *>(ex) + 2 * t;
        ex4[0] = make_float4(v[0], v[1], v[2], v[3]);
        ex4[1] = make_float4(v[4], v[5], v[6], v[7]);
        __syncthreads();
        const int n_items = (int)blockDim.x * 8 / G;       // (block index, r) pairs in the chunk
        for (int item = t; item < n_items; item += blockDim.x) {
            const int blk = item >> 8, r = item & 255;
            float *base = ex + blk * block + r;
            float z[16];
#pragma unroll
            for (int g = 0; g < 16; ++g) z[g] = g < G ? base[256 * g] : 0.f;
#pragma unroll
            for (int h = 1; h < 16; h <<= 1) {
                if (h < G) {
#pragma unroll
                    for (int g = 0; g < 16; ++g) {
                        if ((g & h) == 0) {
                            const float a = z[g], b = z[g + h];
                            z[g] = a + b;
                            z[g + h] = a - b;
                        }
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < 16; ++g)
                if (g < G) base[256 * g] = z[g];
        }
        __syncthreads();
        const float4 lo = ex4[0], hi = ex4[1];
        v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w, v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
    }
}

__device__ __forceinline__ float hadamard_norm_dev(int block) { return rsqrtf((float)block); }

// fp32 x 8 read past L1 (the values came from another grid's atomics)
__device__ __forceinline__ void load8_f32_cg(const float *p, float (&v)[8]) {
    const float4 a = __ldcg(reinterpret_cast<const float4 *>(p)), b = __ldcg(reinterpret_cast<const float4 *>(p) + 1);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}

__device__ __forceinline__ float block_sum(float v, float *red) {      // red: >= 17 floats; all threads call
    const int t = threadIdx.x;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    __syncthreads();
    if ((t & 31) == 0) red[t >> 5] = v;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
    return tot;
}

// (1) optional: h = residual + s_out * H(acc) * scale   (the output side of a row's previous layer; acc cleared)
// (2) xn = rmsnorm(h) * w_norm
// (3) out = H(s_in * xn) * norm   (the input side of the next layer), or out = xn when no transform is wanted.
// One CTA per row: n / 8 threads; the row is one Hadamard block (n <= 4096) or two of 4096 (n = 8192).
struct FinishNormParams {
    float *acc;                  // fp32 [rows][ld_acc] or NULL (then h is read as it is)
    int64_t ld_acc;
    const __half *signs_out;     // [n] or NULL
    float scale_out;
    __half *h;                   // fp16 [rows][ld_h]: residual in, updated residual out
    __half *h_out;               // where the updated residual goes when not in place (NULL: into h)
    int64_t ld_h;
    const __half *w_norm;        // [n]
    float eps;
    const __half *signs_in;      // [n] or NULL
    int transform_in;            // apply the input-side Hadamard transform to the normalised row
    __half *out;                 // fp16 [rows][ld_out]
    int64_t ld_out;
    int32_t n;                   // row length = 8 x threads of the CTA
    int32_t block;               // Hadamard block of both transforms (n, or 4096 when n = 8192)
};

// One row; called by all n/8 threads of a CTA.  `owner`: this CTA is the one that clears the accumulator behind
// its read and stores the updated residual.  When several CTAs compute the same row (each for its own use),
// exactly one of them is the owner of the residual and nobody clears; the residual then needs h_out != h.
// `ex_idle`: no thread can still be reading the exchange buffer when this call starts (first use in the kernel).
// `after_loads`: called once the row's global loads have been issued and before their values are used -- a place for
// work that should overlap the loads' trip through L2 (e.g. writing a lookup table to shared memory).
template <typename Hook = NoHook>
__device__ __forceinline__ void finish_norm_row(const FinishNormParams &p, int64_t row, float *ex, float *red, bool clear_acc,
                                                bool write_h, bool ex_idle = false, Hook after_loads = Hook()) {
    const int t = threadIdx.x;
    const int col = 8 * t;
    const float hn = hadamard_norm_dev(p.block);
    // every global load is issued before the first dependent use: one memory round trip for the kernel
    const uint4 raw_so = raw8_or_ones(p.signs_out ? p.signs_out + col : nullptr);
    const uint4 raw_h = clear_acc ? *reinterpret_cast<const uint4 *>(p.h + row * p.ld_h + col)
                                  : __ldcg(reinterpret_cast<const uint4 *>(p.h + row * p.ld_h + col));
    const uint4 raw_w = *reinterpret_cast<const uint4 *>(p.w_norm + col);
    const uint4 raw_si = raw8_or_ones(p.signs_in ? p.signs_in + col : nullptr);
    float v[8], sg[8];
    if (p.acc) {
        if (clear_acc) load8_f32(p.acc + row * p.ld_acc + col, v, true);
        else load8_f32_cg(p.acc + row * p.ld_acc + col, v);
    }
    after_loads();
    if (p.acc) {
        fwht8(v, p.block, ex, !ex_idle);
        unpack8(raw_so, sg);
        float r[8];
        unpack8(raw_h, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = r[i] + v[i] * (p.scale_out * hn) * sg[i];
        if (write_h) store8_f16((p.h_out ? p.h_out : p.h) + row * p.ld_h + col, v);
        // continue from the rounded residual stream, as an unfused reader of h would
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __half2float(__float2half_rn(v[i]));
    } else {
        if (write_h && p.h_out) *reinterpret_cast<uint4 *>(p.h_out + row * p.ld_h + col) = raw_h;
        unpack8(raw_h, v);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    const float inv = rsqrtf(block_sum(ss, red) / p.n + p.eps);
    float w[8];
    unpack8(raw_w, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __half2float(__float2half_rn(v[i] * inv * w[i]));
    if (p.transform_in) {
        unpack8(raw_si, sg);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= sg[i];
        fwht8(v, p.block, ex, false);      // block_sum's barriers lie between the last reads of ex and this write
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= hn;
    }
    store8_f16(p.out + row * p.ld_out + col, v);
}

// The same for a row of NH x 4096 elements handled by 512 threads (thread t holds elements 8t..8t+7 of every 4096-wide
// piece; each piece is one Hadamard block): the form used inside a 512-thread matvec CTA for 8192-wide models.  Never
// clears the accumulator (several CTAs read it); p.block must be 4096.
template <int NH>
__device__ __forceinline__ void finish_norm_row_wide(const FinishNormParams &p, int64_t row, float *ex, float *red, bool write_h,
                                                     bool ex_idle) {
    const int t = threadIdx.x;
    const float hn = hadamard_norm_dev(4096);
    float v[NH][8];
    float ss = 0.f;
#pragma unroll
    for (int hf = 0; hf < NH; ++hf) {
        const int col = hf * 4096 + 8 * t;
        const uint4 raw_h = __ldcg(reinterpret_cast<const uint4 *>(p.h + row * p.ld_h + col));
        if (p.acc) {
            const uint4 raw_so = raw8_or_ones(p.signs_out ? p.signs_out + col : nullptr);
            load8_f32_cg(p.acc + row * p.ld_acc + col, v[hf]);
            fwht8(v[hf], 4096, ex, !(ex_idle && hf == 0));
            float sg[8], r[8];
            unpack8(raw_so, sg);
            unpack8(raw_h, r);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[hf][i] = r[i] + v[hf][i] * (p.scale_out * hn) * sg[i];
            if (write_h) store8_f16((p.h_out ? p.h_out : p.h) + row * p.ld_h + col, v[hf]);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[hf][i] = __half2float(__float2half_rn(v[hf][i]));
        } else {
            if (write_h && p.h_out) *reinterpret_cast<uint4 *>(p.h_out + row * p.ld_h + col) = raw_h;
            unpack8(raw_h, v[hf]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[hf][i] * v[hf][i];
    }
    const float inv = rsqrtf(block_sum(ss, red) / p.n + p.eps);
#pragma unroll
    for (int hf = 0; hf < NH; ++hf) {
        const int col = hf * 4096 + 8 * t;
        float w[8], sg[8];
        unpack8(*reinterpret_cast<const uint4 *>(p.w_norm + col), w);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[hf][i] = __half2float(__float2half_rn(v[hf][i] * inv * w[i]));
        if (p.transform_in) {
            unpack8(raw8_or_ones(p.signs_in ? p.signs_in + col : nullptr), sg);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[hf][i] *= sg[i];
            fwht8(v[hf], 4096, ex, hf != 0);      // before piece 0: block_sum's barriers; later pieces: the transform before
#pragma unroll
            for (int i = 0; i < 8; ++i) v[hf][i] *= hn;
        }
        store8_f16(p.out + row * p.ld_out + col, v[hf]);
    }
}

// Fused MLP middle: gate/up pre-activations arrive as the fp32 accumulator of the fused gate-up
// layer (gate in columns [0, n), up in [n, 2n)).  out = H (s_in * (silu(g) * u)) * scale_in with
// g, u = s_out * (H acc) * scale_out.  Both transforms use the same block size, so one CTA owns
// matching blocks of gate and up.
struct SwigluParams {
    float *acc;                 // fp32 input (an accumulator), or NULL when the input is fp16
    const __half *in16;         // fp16 input [rows][ld_acc] (the output of a matrix product), or NULL
    int64_t ld_acc;
    __half *out;
    int64_t ld_out;
    const __half *signs_out;    // [2n] output-side signs of the gate-up layer (may be NULL)
    const __half *signs_in;     // [n] input-side signs of the down layer (may be NULL)
    int64_t n;
    int32_t block, chunk, clear;
    float scale_out, scale_in;  // both include the 1/sqrt(block) of their transform
};

// Columns col .. col+7 of one row (thread t of the chunk holds 8t..8t+7); result to dst[0..7].
template <typename Hook = NoHook>
__device__ __forceinline__ void swiglu_chunk(const SwigluParams &p, int64_t row, int64_t col, float *ex, bool clear, __half *dst,
                                             Hook after_loads = Hook()) {
    float g[8], u[8], sg[8];
    const uint4 raw_sg = raw8_or_ones(p.signs_out ? p.signs_out + col : nullptr);
    const uint4 raw_su = raw8_or_ones(p.signs_out ? p.signs_out + p.n + col : nullptr);
    const uint4 raw_si = raw8_or_ones(p.signs_in ? p.signs_in + col : nullptr);
    if (p.in16) {
        load8_f16(p.in16 + row * p.ld_acc + col, g);
        load8_f16(p.in16 + row * p.ld_acc + p.n + col, u);
    } else if (clear) {
        load8_f32(p.acc + row * p.ld_acc + col, g, true);
        load8_f32(p.acc + row * p.ld_acc + p.n + col, u, true);
    } else {
        load8_f32_cg(p.acc + row * p.ld_acc + col, g);
        load8_f32_cg(p.acc + row * p.ld_acc + p.n + col, u);
    }
    after_loads();
    fwht8(g, p.block, ex);
    fwht8(u, p.block, ex);
    unpack8(raw_sg, sg);
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] *= p.scale_out * sg[i];
    unpack8(raw_su, sg);
#pragma unroll
    for (int i = 0; i < 8; ++i) u[i] *= p.scale_out * sg[i];
    // the layer's own output is fp16; round there as the unfused path would
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float gg = __half2float(__float2half_rn(g[i])), uu = __half2float(__float2half_rn(u[i]));
        g[i] = __half2float(__float2half_rn(gg / (1.f + __expf(-gg)) * uu));
    }
    unpack8(raw_si, sg);
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] *= sg[i];
    fwht8(g, p.block, ex);
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] *= p.scale_in;
    store8_f16(dst, g);
}

}  // namespace rptc
