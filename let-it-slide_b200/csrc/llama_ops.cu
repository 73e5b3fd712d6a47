// The non-quantised pieces of a Llama-architecture decode step (RMSNorm, RoPE + KV-cache append,
// single-query attention, dense fp16 matvec for the output head).  They exist so that the
// benchmark's decode step is a whole model step launched from one library on one stream; none of
// them has a counterpart in the reference, which evaluates models through Hugging Face
// transformers (quantize_hf.py:230-236).
#include "common.cuh"
#include "fwht.cuh"

namespace rptc {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// out[r][:] = x[r][:] * rsqrt(mean(x^2) + eps) * w[:]      one CTA of 256 threads per row
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __half *__restrict__ x, int64_t ld_x, const __half *__restrict__ w,
                                                      __half *__restrict__ out, int64_t ld_out, int n, float eps) {
    __shared__ float red[8];
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    x = after_wait(x);
    const __half2 *xr = reinterpret_cast<const __half2 *>(x + (int64_t)blockIdx.x * ld_x);
    float ss = 0.f;
    for (int i = threadIdx.x; i < n / 2; i += 256) {
        const float2 f = __half22float2(xr[i]);
        ss += f.x * f.x + f.y * f.y;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv = rsqrtf(tot / n + eps);
    const __half2 *wr = reinterpret_cast<const __half2 *>(w);
    __half2 *o = reinterpret_cast<__half2 *>(out + (int64_t)blockIdx.x * ld_out);
    for (int i = threadIdx.x; i < n / 2; i += 256) {
        const float2 f = __half22float2(xr[i]), g = __half22float2(wr[i]);
        o[i] = __floats2half2_rn(f.x * inv * g.x, f.y * inv * g.y);
    }
}

// Rotary embedding (rotate-half convention, pairs (i, i + d/2)) of the q and k heads of one token per
// row of `qkv` ([rows][(hq + 2 hkv) * d]), in place for q; k (rotated) and v are appended to the caches
// at positions pos[row].  Caches: [rows][max_pos][hkv][d].  One CTA per (row, head of q|k|v).
__global__ void __launch_bounds__(64) rope_cache_kernel(__half *__restrict__ qkv, int64_t ld_qkv, const int32_t *__restrict__ pos,
                                                        __half *__restrict__ kcache, __half *__restrict__ vcache, int hq, int hkv,
                                                        int d, int max_pos, RopeFreq freq, unsigned int *__restrict__ status) {
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    const int row = blockIdx.y, head = blockIdx.x, t = threadIdx.x;      // t < d/2
    const int p = pos[row];
    if (p < 0 || p >= max_pos) {       // no room in the cache for this position: report it and touch nothing
        if (t == 0 && head == 0) atomicExch(status, kStatusPosition);
        return;
    }
    __half *src = qkv + (int64_t)row * ld_qkv + (int64_t)head * d;
    if (head < hq + hkv) {
        float lo = 0.f, hi = 0.f;
        if (t < d / 2) {
            const float inv_freq = rope_inv_freq(freq, t);
            float sn, cs;
            sincosf(p * inv_freq, &sn, &cs);
            const float a = __half2float(src[t]), b = __half2float(src[t + d / 2]);
            lo = a * cs - b * sn;
            hi = b * cs + a * sn;
        }
        if (t < d / 2) {
            if (head < hq) {
                src[t] = __float2half_rn(lo);
                src[t + d / 2] = __float2half_rn(hi);
            } else {
                __half *dst = kcache + (((int64_t)row * max_pos + p) * hkv + (head - hq)) * d;
                dst[t] = __float2half_rn(lo);
                dst[t + d / 2] = __float2half_rn(hi);
            }
        }
    } else {
        __half *dst = vcache + (((int64_t)row * max_pos + p) * hkv + (head - hq - hkv)) * d;
        if (t < d / 2) {
            dst[t] = src[t];
            dst[t + d / 2] = src[t + d / 2];
        }
    }
}

// The same for a whole prompt: one CTA per (position, row) takes all heads of its token, so the rotation angles of a
// position are computed once per pair index instead of once per head.  Token t of row r sits in row r * T + t of qkv.
__global__ void __launch_bounds__(256) rope_cache_prompt_kernel(__half *__restrict__ qkv, int64_t ld_qkv, __half *__restrict__ kcache,
                                                               __half *__restrict__ vcache, int hq, int hkv, int d, int max_pos,
                                                               RopeFreq freq) {
    const int p = blockIdx.x, row = blockIdx.y, T = gridDim.x;
    const int half_d = d / 2, i = threadIdx.x % 64, grp = threadIdx.x / 64;      // pair index, head group (4 groups)
    if (i >= half_d) return;
    float sn, cs;
    sincosf(p * rope_inv_freq(freq, i), &sn, &cs);
    __half *tok = qkv + ((int64_t)row * T + p) * ld_qkv;
    for (int head = grp; head < hq + 2 * hkv; head += 4) {
        __half *src = tok + (int64_t)head * d;
        const __half ra = src[i], rb = src[i + half_d];
        if (head < hq + hkv) {
            const float a = __half2float(ra), b = __half2float(rb);
            const __half lo = __float2half_rn(a * cs - b * sn), hi = __float2half_rn(b * cs + a * sn);
            __half *dst = head < hq ? src : kcache + (((int64_t)row * max_pos + p) * hkv + (head - hq)) * d;
            dst[i] = lo;
            dst[i + half_d] = hi;
        } else {
            __half *dst = vcache + (((int64_t)row * max_pos + p) * hkv + (head - hq - hkv)) * d;
            dst[i] = ra;
            dst[i + half_d] = rb;
        }
    }
}

// Single-query attention over the cache: one CTA of 512 threads per (row, q head); d == 128.
// One trip to memory: every warp fetches the K AND V rows of its positions (16 of each in flight, positions
// interleaved over the 16 warps) before anything that depends on the kernel in front, then keeps a running
// maximum / sum / weighted V sum of its own (online softmax); the 16 partial states meet in shared memory.
// Contexts beyond 256 take further chunks of 256 positions through the same registers.
// A warp takes two positions at a time, one per half-warp: lane (half, dl) holds dims 8*dl .. 8*dl+7 of its half's
// position (one 16-byte load per row and lane, four shuffle stages per pair of scores).
constexpr int kAttnThreads = 512, kAttnWarps = 16, kAttnUnroll = 8;      // 8 slots x 2 positions x 16 warps = 256 positions in flight
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const __half *__restrict__ qkv, int64_t ld_qkv,
                                                                  const int32_t *__restrict__ pos, const __half *__restrict__ kcache,
                                                                  const __half *__restrict__ vcache, __half *__restrict__ out,
                                                                  int64_t ld_out, int hq, int hkv, int max_pos, float scale,
                                                                  const __half *__restrict__ signs_in, float *__restrict__ acc,
                                                                  int64_t ld_acc, const __half *__restrict__ signs_out,
                                                                  float scale_out, RopeFreq freq, __half *__restrict__ kcache_w,
                                                                  __half *__restrict__ vcache_w, unsigned int *__restrict__ status) {
    __shared__ float part[kAttnWarps][128];
    __shared__ float pm[kAttnWarps], pl[kAttnWarps];
    __shared__ float tr[128];
    __shared__ __align__(16) __half qs[128], ks[128], vs[128];
    __shared__ float rot[2][64];                                 // cosines and sines of the new position's 64 rotary angles
    pdl_allow_next_grid();
    constexpr int D = 128;
    const bool fused = acc != nullptr;
    // Without the fused front end q and the newest K/V row come from the kernel in front: wait for it first.
    // With it, the rows already in the cache and the position were written at least a step ago.
    if (!fused) pdl_wait_prior_grids();
    const int row = blockIdx.y, head = blockIdx.x, kvh = head / (hq / hkv);
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    // A position outside [0, max_pos) has no row in the cache: it is reported, nothing is appended, and attention runs
    // over the rows that exist (the result is meaningless, the accesses stay in bounds).
    const int pos_raw = (int)ld_ordered_u32(pos + row);
    const bool pos_ok = pos_raw >= 0 && pos_raw < max_pos;
    if (!pos_ok && t == 0 && head == 0) atomicExch(status, kStatusPosition);
    const int ctx = min(max(pos_raw, 0), max_pos - 1) + 1;
    const int n_old = fused ? ctx - 1 : ctx;                     // rows to read from the cache
    const int64_t stride = (int64_t)hkv * D;
    const int half = lane >> 4, dl = lane & 15;
    const __half *kb = kcache + ((int64_t)row * max_pos * hkv + kvh) * D + 8 * dl;
    const __half *vb = vcache + ((int64_t)row * max_pos * hkv + kvh) * D + 8 * dl;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    uint4 kk[kAttnUnroll], vv[kAttnUnroll];
#pragma unroll
    for (int u = 0; u < kAttnUnroll; ++u) {
        const int j = 2 * (warp + u * kAttnWarps) + half;      // slot (warp + 16 u): positions 2 slot, 2 slot + 1
        kk[u] = j < n_old ? ld_ordered_u128(kb + j * stride) : zero4;
        vv[u] = j < n_old ? ld_ordered_u128(vb + j * stride) : zero4;
    }
    uint4 qraw = zero4;
    if (!fused) qraw = ld_ordered_u128(qkv + (int64_t)row * ld_qkv + (int64_t)head * D + 8 * dl);
    // Rotary angles of the new position: they depend on the position only, so they are made before the wait, one angle
    // per thread (an accurate sincosf is a hundred instructions; eight in a row in the sixteen front-end threads cost
    // 1.8 us) and handed over through shared memory.
    uint4 so_raw = make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);
    // constants: fetched early, as raw bits -- a conversion here would stall the thread until the load (and the sixteen
    // cache loads queued in front of it) has come back, and with it the dependency wait and everything behind it
    const unsigned short si_raw = (signs_in && t < D) ? __ldg(reinterpret_cast<const unsigned short *>(signs_in) + head * D + t) : (unsigned short)0x3C00;
    if (fused && warp < 2) {
        const int i8 = (t & 15) * 8;
        const int grp0 = t >> 4;
        if (signs_out && grp0 < 3) so_raw = *reinterpret_cast<const uint4 *>(signs_out + (grp0 == 0 ? head : grp0 == 1 ? hq + kvh : hq + hkv + kvh) * D + i8);
    }
    if (fused && t >= 64 && t < 128) {                           // warps 2 and 3: warps 0 and 1 have the loads above
        float sn, cs;
        sincosf((ctx - 1) * rope_inv_freq(freq, t - 64), &sn, &cs);
        rot[0][t - 64] = cs;
        rot[1][t - 64] = sn;
    }
    if (fused) {
        // Fused front end: this CTA finishes its own q and the k and v of its kv head from the fused qkv layer's
        // accumulator -- per-head 128-wide output transform, fp16 rounding, rotary embedding -- and keeps all three
        // in shared memory.  With grouped-query attention the q heads of a group each make their own copy of k and
        // v (a few hundred flops) and the first of them appends the pair to the caches; nobody reads that cache row
        // in this launch.  Sixteen threads x eight values per vector.
        pdl_wait_prior_grids();
        __syncthreads();                                            // the angles are in shared memory
        const bool appends = pos_ok && head % (hq / hkv) == 0;
        if (warp < 2) {
            const int grp = t >> 4, i8 = (t & 15) * 8;              // 0: q, 1: k, 2: v, 3: idle half warp
            const int col = (grp == 0 ? head : grp == 1 ? hq + kvh : hq + hkv + kvh) * D + i8;
            float v[8], sg[8];
            if (grp < 3) {
                // multi-head: every column has one reader, who zeroes it; grouped-query: k and v have several readers
                // and a later launch zeroes the accumulator
                load8_f32(acc + (int64_t)row * ld_acc + col, v, hq == hkv);
                unpack8(so_raw, sg);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = 0.f, sg[i] = 1.f;
            }
            fwht8(v, D, nullptr);
            const float sc_out = scale_out * hadamard_norm_dev(D);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __half2float(__float2half_rn(v[i] * sc_out * sg[i]));
            float o[8];
            const int ps = ctx - 1;
            const bool upper = i8 >= 64;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float partner = __shfl_xor_sync(0xFFFFFFFFu, v[i], 8);
                const float sn = rot[1][(i8 & 63) + i], cs = rot[0][(i8 & 63) + i];
                o[i] = grp == 2 ? v[i] : (upper ? v[i] * cs + partner * sn : v[i] * cs - partner * sn);
            }
            if (grp == 0) {
                store8_f16(qs + i8, o);
            } else if (grp == 1) {
                store8_f16(ks + i8, o);
                if (appends) store8_f16(kcache_w + (((int64_t)row * max_pos + ps) * hkv + kvh) * D + i8, o);
            } else if (grp == 2) {
                store8_f16(vs + i8, o);
                if (appends) store8_f16(vcache_w + (((int64_t)row * max_pos + ps) * hkv + kvh) * D + i8, o);
            }
        }
        __syncthreads();
        qraw = *reinterpret_cast<const uint4 *>(qs + 8 * dl);
    }
    float q[8];
    unpack8(qraw, q);
    auto dot8 = [&](const uint4 &raw) {                       // this lane's eight dims of q . k
        float k[8];
        unpack8(raw, k);
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d += q[i] * k[i];
        return d;
    };
    auto half_sum = [](float v) {                             // sum over the sixteen lanes of a half-warp
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        return v;
    };
    // ---- this half-warp's positions: running maximum m, sum l and weighted V sum a (dims 8*dl .. 8*dl+7) ----
    float m = -1e30f, l = 0.f, a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s0 = warp; 2 * s0 < n_old || s0 == warp; s0 += kAttnUnroll * kAttnWarps) {
        const int s_next = s0 + kAttnUnroll * kAttnWarps;       // this warp's first slot of the next chunk
        float sc[kAttnUnroll];
        float mc = -1e30f;
#pragma unroll
        for (int u = 0; u < kAttnUnroll; ++u) {
            sc[u] = half_sum(dot8(kk[u])) * scale;
            if (2 * (s0 + u * kAttnWarps) + half < n_old) mc = fmaxf(mc, sc[u]);
        }
        if (2 * s_next < n_old) {      // the K registers are free: the next chunk's K rows travel under this chunk's V pass
#pragma unroll
            for (int u = 0; u < kAttnUnroll; ++u) {
                const int j = 2 * (s_next + u * kAttnWarps) + half;
                kk[u] = j < n_old ? ld_ordered_u128(kb + j * stride) : zero4;
            }
        }
        // one rescale per chunk: the chunk's maximum first, then plain accumulation
        const float m_new = fmaxf(m, mc), corr = __expf(m - m_new);
        l *= corr;
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] *= corr;
        m = m_new;
#pragma unroll
        for (int u = 0; u < kAttnUnroll; ++u) {
            const float p = (2 * (s0 + u * kAttnWarps) + half < n_old) ? __expf(sc[u] - m) : 0.f;
            float v[8];
            unpack8(vv[u], v);
            l += p;
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] += p * v[i];
        }
        if (2 * s_next < n_old) {      // and its V rows under the next chunk's scores
#pragma unroll
            for (int u = 0; u < kAttnUnroll; ++u) {
                const int j = 2 * (s_next + u * kAttnWarps) + half;
                vv[u] = j < n_old ? ld_ordered_u128(vb + j * stride) : zero4;
            }
        }
    }
    if (fused && warp == 0) {      // the position made above, from shared memory: the first half-warp folds it in
        const uint4 kr = *reinterpret_cast<const uint4 *>(ks + 8 * dl), vr = *reinterpret_cast<const uint4 *>(vs + 8 * dl);
        const float sn = half_sum(dot8(kr)) * scale;           // all lanes take part in the shuffles
        if (half == 0) {
            const float m_new = fmaxf(m, sn), corr = __expf(m - m_new), p = __expf(sn - m_new);
            float v[8];
            unpack8(vr, v);
            l = l * corr + p;
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = a[i] * corr + p * v[i];
            m = m_new;
        }
    }
    {
        // the two half-warps' states into one (an empty half has m = -1e30 and l = 0: its weight underflows to zero)
        const float m_o = __shfl_xor_sync(0xFFFFFFFFu, m, 16);
        const float m_w = fmaxf(m, m_o), c = __expf(m - m_w);
        l *= c;
        l += __shfl_xor_sync(0xFFFFFFFFu, l, 16);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            a[i] *= c;
            a[i] += __shfl_xor_sync(0xFFFFFFFFu, a[i], 16);
        }
        m = m_w;
    }
    if (half == 0) {
        *reinterpret_cast<float4 *>(&part[warp][8 * dl]) = make_float4(a[0], a[1], a[2], a[3]);
        *reinterpret_cast<float4 *>(&part[warp][8 * dl + 4]) = make_float4(a[4], a[5], a[6], a[7]);
    }
    if (lane == 0) pm[warp] = m, pl[warp] = l;
    __syncthreads();
    if (t < D) {
        float mx = pm[0];
#pragma unroll
        for (int w = 1; w < kAttnWarps; ++w) mx = fmaxf(mx, pm[w]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float e = __expf(pm[w] - mx);
            num += e * part[w][t];
            den += e * pl[w];
        }
        float o = __half2float(__float2half_rn(num / den));            // the attention output in fp16
        if (signs_in) {
            // input-side transform of the output projection, one 128-wide Hadamard block per head:
            // o <- H_128(s * o) / sqrt(128); thread t holds element t (threads 0..127 = warps 0..3)
            o *= __half2float(__ushort_as_half(si_raw));
#pragma unroll
            for (int mm = 1; mm < 32; mm <<= 1) {
                const float other = __shfl_xor_sync(0xFFFFFFFFu, o, mm);
                o = (lane & mm) ? other - o : o + other;
            }
            tr[t] = o;
            asm volatile("bar.sync 1, 128;" ::: "memory");             // only the four warps that hold outputs
            const float e0 = tr[lane], e1 = tr[32 + lane], e2 = tr[64 + lane], e3 = tr[96 + lane];
            const float b0 = e0 + e1, b1 = e0 - e1, b2 = e2 + e3, b3 = e2 - e3;
            const float c = warp == 0 ? b0 + b2 : warp == 1 ? b1 + b3 : warp == 2 ? b0 - b2 : b1 - b3;
            o = c * 0.08838834764831845f;
        }
        out[(int64_t)row * ld_out + (int64_t)head * D + t] = __float2half_rn(o);
    }
}

// Dense fp16 matvec  y[b][r] = sum_c W[r][c] x[b][c]  (fp32 accumulation), one warp per row of W, the
// batch (<= 8) handled inside.  Used for the output head; also the dense-bandwidth probe the
// reference's stale tests call `matvec` (rptc_kernels/tests/test_matvec.py:18).
template <int BATCH>
__global__ void __launch_bounds__(256) dense_gemv_kernel(const __half *__restrict__ W, int64_t ld_w, const __half *__restrict__ x,
                                                         int64_t ld_x, __half *__restrict__ y, int64_t ld_y, int64_t m, int n) {
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    x = after_wait(x);
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= m) return;
    const uint4 *wr = reinterpret_cast<const uint4 *>(W + row * ld_w);
    float acc[BATCH];
#pragma unroll
    for (int b = 0; b < BATCH; ++b) acc[b] = 0.f;
    for (int i = lane; i < n / 8; i += 32) {
        const uint4 wv = ldg128_stream(wr + i);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const uint4 xv = __ldg(reinterpret_cast<const uint4 *>(x + (int64_t)b * ld_x) + i);
            const uint32_t xx[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 a = __half22float2(u32_as_half2(ww[k])), c = __half22float2(u32_as_half2(xx[k]));
                acc[b] += a.x * c.x + a.y * c.y;
            }
        }
    }
#pragma unroll
    for (int b = 0; b < BATCH; ++b) {
        const float s = warp_sum(acc[b]);
        if (lane == 0) y[(int64_t)b * ld_y + row] = __float2half_rn(s);
    }
}

// out[r][:] = table[ids[r]][:]
__global__ void embed_kernel(const __half *__restrict__ table, const int32_t *__restrict__ ids, __half *__restrict__ out, int64_t ld_out,
                             int n) {
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    ids = after_wait(ids);
    const uint4 *src = reinterpret_cast<const uint4 *>(table + (int64_t)ids[blockIdx.x] * n);
    uint4 *dst = reinterpret_cast<uint4 *>(out + (int64_t)blockIdx.x * ld_out);
    for (int i = threadIdx.x; i < n / 8; i += blockDim.x) dst[i] = src[i];
}

// The embedding lookup of a step whose token ids come from the host through a mailbox in pinned memory: slot r
// holds (sequence number << 32) | id.  The launch may be queued before the host knows the id (behind the step that
// produces it), so one thread polls slot 0.. until every slot shows sequence *steps_done + 1, for at most
// `timeout_ns`; on expiry it raises the status word and goes on with whatever ids are there, so that the stream
// always drains.  The sequence number is then published in *steps_done for the step's last kernel.
__global__ void __launch_bounds__(256) embed_mailbox_kernel(const __half *__restrict__ table, const unsigned long long *slots,
                                                            uint32_t *steps_done, int32_t *__restrict__ ids, __half *__restrict__ out,
                                                            int64_t ld_out, int rows, int n, int64_t vocab,
                                                            unsigned long long timeout_ns, unsigned int *status) {
    __shared__ int tok[64];
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    if (threadIdx.x == 0) {
        const uint32_t want = *steps_done + 1u;
        unsigned long long t0;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
        for (int r = 0; r < rows; ++r) {
            unsigned long long v;
            for (;;) {
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(slots + r) : "memory");
                if ((uint32_t)(v >> 32) == want) break;
                unsigned long long now;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                if (now - t0 > timeout_ns) {
                    atomicExch(status, kStatusMailboxExpired);
                    break;
                }
                __nanosleep(100);
            }
            int64_t id = (int64_t)(uint32_t)v;
            if (id >= vocab) id = 0;
            tok[r] = (int)id;
            ids[r] = (int)id;
        }
        *steps_done = want;
    }
    __syncthreads();
    for (int r = 0; r < rows; ++r) {
        const uint4 *src = reinterpret_cast<const uint4 *>(table + (int64_t)tok[r] * n);
        uint4 *dst = reinterpret_cast<uint4 *>(out + (int64_t)r * ld_out);
        for (int i = threadIdx.x; i < n / 8; i += blockDim.x) dst[i] = src[i];
    }
}

// Greedy sampling and the bookkeeping that ends a decode step, one CTA per row: next[r] = argmax(logits[r]) (first
// maximum), fed back into ids[r]; pos[r] += 1; the id is also written to `mirror` when given (a pinned host
// buffer mapped into the device's address space: the host reads the token after synchronising the stream).
__global__ void __launch_bounds__(1024) next_token_kernel(const __half *__restrict__ logits, int64_t ld, int n, int64_t *__restrict__ next,
                                                          int32_t *__restrict__ ids, int32_t *__restrict__ pos, int64_t *__restrict__ mirror,
                                                          const uint32_t *__restrict__ steps_done) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    logits = after_wait(logits);
    steps_done = after_wait(steps_done);
    const int r = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const __half *row = logits + (int64_t)r * ld;
    float best = -INFINITY;
    int at = 0x7FFFFFFF;
    for (int i = 2 * t; i < n; i += 2 * 1024) {
        const float2 v = __half22float2(*reinterpret_cast<const __half2 *>(row + i));
        if (v.x > best) best = v.x, at = i;
        if (i + 1 < n && v.y > best) best = v.y, at = i + 1;
    }
    auto better = [](float v, int i, float bvv, int bii) { return v > bvv || (v == bvv && i < bii); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, at, o);
        if (better(ov, oi, best, at)) best = ov, at = oi;
    }
    if (lane == 0) bv[warp] = best, bi[warp] = at;
    __syncthreads();
    if (warp == 0) {
        best = bv[lane], at = bi[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, at, o);
            if (better(ov, oi, best, at)) best = ov, at = oi;
        }
        if (lane == 0) {
            if (at == 0x7FFFFFFF) at = 0;           // a row of NaNs
            next[r] = at;
            if (ids) ids[r] = at;
            if (pos && pos[r] < 0x7FFFFFFF) pos[r] += 1;      // consumers check the position against their cache
            if (mirror) {
                // with a step counter the slot is a mailbox entry: (sequence << 32) | id, one store, pushed to the host
                mirror[r] = steps_done ? (int64_t)(((unsigned long long)*steps_done << 32) | (unsigned)at) : (int64_t)at;
                __threadfence_system();
            }
        }
    }
}

}  // namespace rptc

using namespace rptc;

extern "C" int rptc_rmsnorm(const void *x, int64_t ld_x, const void *w, void *out, int64_t ld_out, int64_t rows, int64_t n,
                            float eps, rptc_stream_t stream) {
    if (!x || !w || !out) return RPTC_ERR_ARG;
    if (rows <= 0 || n <= 0 || (n % 2) || ld_x < n || ld_out < n) return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(out) & 3) || (ld_x & 1) || (ld_out & 1)) return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    return launch(rmsnorm_kernel, dim3((unsigned)rows), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __half *>(x),
                  ld_x, static_cast<const __half *>(w), static_cast<__half *>(out), ld_out, (int)n, eps);
}

extern "C" int rptc_rope_cache(void *qkv, int64_t ld_qkv, const int32_t *pos, void *kcache, void *vcache, int64_t rows, int hq,
                               int hkv, int d, int max_pos, float theta, rptc_stream_t stream) {
    if (!qkv || !pos || !kcache || !vcache) return RPTC_ERR_ARG;
    if (rows <= 0 || hq <= 0 || hkv <= 0 || (hq % hkv) || d <= 0 || (d % 2) || d > 128 || max_pos <= 0) return RPTC_ERR_SHAPE;
    if (ld_qkv < (int64_t)(hq + 2 * hkv) * d) return RPTC_ERR_SHAPE;
    if (int e = rptc_check_device()) return e;
    unsigned int *status = device_status_word();
    if (!status) return RPTC_ERR_CUDA;
    return launch(rope_cache_kernel, dim3((unsigned)(hq + 2 * hkv), (unsigned)rows), dim3(64), 0, static_cast<cudaStream_t>(stream),
                  static_cast<__half *>(qkv), ld_qkv, pos, static_cast<__half *>(kcache), static_cast<__half *>(vcache), hq, hkv, d,
                  max_pos, rope_freq(theta, d), status);
}

extern "C" int rptc_attn_decode(const void *qkv, int64_t ld_qkv, const int32_t *pos, const void *kcache, const void *vcache, void *out,
                                int64_t ld_out, int64_t rows, int hq, int hkv, int d, int max_pos, float scale, const void *signs_in,
                                rptc_stream_t stream) {
    if (!qkv || !pos || !kcache || !vcache || !out) return RPTC_ERR_ARG;
    if (d != 128) return RPTC_ERR_UNSUPPORTED;
    if (rows <= 0 || hq <= 0 || hkv <= 0 || (hq % hkv) || max_pos <= 0 || max_pos > 32768) return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(kcache) & 15) || (reinterpret_cast<uintptr_t>(vcache) & 15) ||
        (ld_qkv & 7))
        return RPTC_ERR_ALIGN;      // rows of q, k and v are read sixteen bytes at a time
    if (int e = rptc_check_device()) return e;
    unsigned int *status = device_status_word();
    if (!status) return RPTC_ERR_CUDA;
    return launch(attn_decode_kernel, dim3((unsigned)hq, (unsigned)rows), dim3(kAttnThreads), 0, static_cast<cudaStream_t>(stream),
                  static_cast<const __half *>(qkv), ld_qkv, pos, static_cast<const __half *>(kcache), static_cast<const __half *>(vcache),
                  static_cast<__half *>(out), ld_out, hq, hkv, max_pos, scale, static_cast<const __half *>(signs_in),
                  static_cast<float *>(nullptr), (int64_t)0, static_cast<const __half *>(nullptr), 0.f, RopeFreq{0.f, 0.f},
                  static_cast<__half *>(nullptr), static_cast<__half *>(nullptr), status);
}

extern "C" int rptc_qkv_attn_decode(float *acc, int64_t ld_acc, const void *signs_out, float scale_out, const int32_t *pos,
                                    void *kcache, void *vcache, void *out, int64_t ld_out, int64_t rows, int heads, int kv_heads,
                                    int max_pos, float theta, const void *signs_in, rptc_stream_t stream) {
    if (!acc || !pos || !kcache || !vcache || !out) return RPTC_ERR_ARG;
    if (rows <= 0 || rows > 65535 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || max_pos <= 0 || max_pos > 32768 ||
        ld_acc < (int64_t)(heads + 2 * kv_heads) * 128 || ld_out < (int64_t)heads * 128)
        return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(acc) & 15) || (reinterpret_cast<uintptr_t>(kcache) & 15) || (reinterpret_cast<uintptr_t>(vcache) & 15) ||
        (signs_out && (reinterpret_cast<uintptr_t>(signs_out) & 15)) || (ld_acc % 4))
        return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    unsigned int *status = device_status_word();
    if (!status) return RPTC_ERR_CUDA;
    return launch(attn_decode_kernel, dim3((unsigned)heads, (unsigned)rows), dim3(kAttnThreads), 0, static_cast<cudaStream_t>(stream),
                  static_cast<const __half *>(nullptr), (int64_t)0, pos, static_cast<const __half *>(kcache),
                  static_cast<const __half *>(vcache), static_cast<__half *>(out), ld_out, heads, kv_heads, max_pos, 0.08838834764831845f,
                  static_cast<const __half *>(signs_in), acc, ld_acc, static_cast<const __half *>(signs_out), scale_out, rope_freq(theta, 128),
                  static_cast<__half *>(kcache), static_cast<__half *>(vcache), status);
}

extern "C" int rptc_dense_gemv(const void *W, int64_t ld_w, const void *x, int64_t ld_x, void *y, int64_t ld_y, int64_t m, int64_t n,
                               int batch, rptc_stream_t stream) {
    if (!W || !x || !y) return RPTC_ERR_ARG;
    if (m <= 0 || n <= 0 || (n % 8) || ld_w < n || ld_x < n || ld_y < m) return RPTC_ERR_SHAPE;
    if (batch < 1 || batch > 8) return RPTC_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(x) & 15) || (ld_w % 8) || (ld_x % 8)) return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    const dim3 grid((unsigned)((m + 7) / 8)), block(256);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const __half *Wp = static_cast<const __half *>(W), *xp = static_cast<const __half *>(x);
    __half *yp = static_cast<__half *>(y);
    int done = 0;
    while (done < batch) {
        int b = 8;
        while (b > batch - done) b >>= 1;
        int e;
        const __half *xb = xp + (int64_t)done * ld_x;
        __half *yb = yp + (int64_t)done * ld_y;
        switch (b) {
            case 8: e = launch(dense_gemv_kernel<8>, grid, block, 0, s, Wp, ld_w, xb, ld_x, yb, ld_y, m, (int)n); break;
            case 4: e = launch(dense_gemv_kernel<4>, grid, block, 0, s, Wp, ld_w, xb, ld_x, yb, ld_y, m, (int)n); break;
            case 2: e = launch(dense_gemv_kernel<2>, grid, block, 0, s, Wp, ld_w, xb, ld_x, yb, ld_y, m, (int)n); break;
            default: e = launch(dense_gemv_kernel<1>, grid, block, 0, s, Wp, ld_w, xb, ld_x, yb, ld_y, m, (int)n); break;
        }
        if (e) return e;
        done += b;
    }
    return RPTC_OK;
}

extern "C" int rptc_embed(const void *table, const int32_t *ids, void *out, int64_t ld_out, int64_t rows, int64_t n,
                          rptc_stream_t stream) {
    if (!table || !ids || !out) return RPTC_ERR_ARG;
    if (rows <= 0 || n <= 0 || (n % 8) || ld_out < n) return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(table) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || (ld_out % 8)) return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    return launch(embed_kernel, dim3((unsigned)rows), dim3(128), 0, static_cast<cudaStream_t>(stream), static_cast<const __half *>(table),
                  ids, static_cast<__half *>(out), ld_out, (int)n);
}

extern "C" int rptc_next_token(const void *logits, int64_t ld, int64_t rows, int64_t n, int64_t *next, int32_t *ids, int32_t *pos,
                               int64_t *mirror, const uint32_t *steps_done, rptc_stream_t stream) {
    if (!logits || !next) return RPTC_ERR_ARG;
    if (rows <= 0 || rows > 65535 || n <= 0 || n > (int64_t(1) << 30) || (n % 2) || ld < n) return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(logits) & 3) || (ld & 1)) return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    return launch(next_token_kernel, dim3((unsigned)rows), dim3(1024), 0, static_cast<cudaStream_t>(stream),
                  static_cast<const __half *>(logits), ld, (int)n, next, ids, pos, mirror, steps_done);
}

extern "C" int rptc_embed_mailbox(const void *table, const uint64_t *slots, uint32_t *steps_done, int32_t *ids, void *out,
                                  int64_t ld_out, int64_t rows, int64_t n, int64_t vocab, int timeout_ms, rptc_stream_t stream) {
    if (!table || !slots || !steps_done || !ids || !out) return RPTC_ERR_ARG;
    if (rows <= 0 || rows > 64 || n <= 0 || (n % 8) || ld_out < n || vocab <= 0 || timeout_ms <= 0) return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(table) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || (ld_out % 8) ||
        (reinterpret_cast<uintptr_t>(slots) & 7))
        return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    unsigned int *status = device_status_word();
    if (!status) return RPTC_ERR_CUDA;
    return launch(embed_mailbox_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __half *>(table),
                  reinterpret_cast<const unsigned long long *>(slots), steps_done, ids, static_cast<__half *>(out), ld_out, (int)rows,
                  (int)n, vocab, (unsigned long long)timeout_ms * 1000000ull, status);
}

extern "C" int rptc_rope_cache_prompt(void *qkv, int64_t ld_qkv, int64_t rows, int64_t tokens, void *kcache, void *vcache, int hq,
                                      int hkv, int d, int max_pos, float theta, rptc_stream_t stream) {
    if (!qkv || !kcache || !vcache) return RPTC_ERR_ARG;
    if (rows <= 0 || rows > 65535 || tokens <= 0 || tokens > 65535 || tokens > max_pos || hq <= 0 || hkv <= 0 || (hq % hkv) ||
        d <= 0 || (d % 2) || d > 128)
        return RPTC_ERR_SHAPE;
    if (ld_qkv < (int64_t)(hq + 2 * hkv) * d) return RPTC_ERR_SHAPE;
    if (int e = rptc_check_device()) return e;
    return launch(rope_cache_prompt_kernel, dim3((unsigned)tokens, (unsigned)rows), dim3(256), 0, static_cast<cudaStream_t>(stream),
                  static_cast<__half *>(qkv), ld_qkv, static_cast<__half *>(kcache), static_cast<__half *>(vcache), hq, hkv, d, max_pos,
                  rope_freq(theta, d));
}
