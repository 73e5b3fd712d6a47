// Block-diagonal randomized fast Hadamard transform along rows (the incoherence transform applied
// to activations before, and to outputs after, a quantised linear layer).
//
// One CTA transforms one block (256..4096 elements, or 256 elements holding several smaller blocks)
// of one row.  A thread holds eight consecutive elements in fp32 registers: butterfly strides 1,2,4
// run in registers, strides 8..128 as warp shuffles (__shfl_xor), and strides >= 256 through a
// shared-memory exchange.  Sign flips, the 1/sqrt(block) scale and the fp16 conversion are fused in.
#include "common.cuh"

namespace rptc {

struct HadParams {
    const void *in;
    int64_t ld_in;
    __half *out;
    int64_t ld_out;
    const __half *signs;
    int32_t block, chunk;
    int32_t in_is_f32, transpose, clear_in;
    float scale;
};

__global__ void __launch_bounds__(512) hadamard_kernel(const HadParams p) {
    __shared__ float ex[4096];
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    const int t = threadIdx.x;
    const int64_t row = blockIdx.y;
    const int64_t col = (int64_t)blockIdx.x * p.chunk + 8 * t;
    float v[8];
    if (p.in_is_f32) {
        float *src = const_cast<float *>(static_cast<const float *>(p.in)) + row * p.ld_in + col;
        const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
        if (p.clear_in) {
            *reinterpret_cast<float4 *>(src) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4 *>(src + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    } else {
        const uint4 a = *reinterpret_cast<const uint4 *>(static_cast<const __half *>(p.in) + row * p.ld_in + col);
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(u32_as_half2(w[i]));
            v[2 * i] = f.x, v[2 * i + 1] = f.y;
        }
    }
    float sg[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) sg[i] = 1.f;
    if (p.signs) {
        const uint4 a = __ldg(reinterpret_cast<const uint4 *>(p.signs + col));
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(u32_as_half2(w[i]));
            sg[2 * i] = f.x, sg[2 * i + 1] = f.y;
        }
    }
    if (!p.transpose) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= sg[i];
    }
    // strides 1, 2, 4: in registers
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
    // strides 8 .. 128: across lanes
    for (int lm = 1; lm < 32 && 8 * lm < p.block; lm <<= 1) {
        const bool upper = (t & lm) != 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float o = __shfl_xor_sync(0xFFFFFFFFu, v[i], lm);
            v[i] = upper ? o - v[i] : v[i] + o;
        }
    }
    // strides >= 256: through shared memory
    if (p.block > 256) {
#pragma unroll
        for (int i = 0; i < 8; ++i) ex[8 * t + i] = v[i];
        __syncthreads();
        const int pairs_per_thread = 4;   // chunk / 2 pairs over chunk / 8 threads
        for (int h = 256; h < p.block; h <<= 1) {
#pragma unroll
            for (int k = 0; k < pairs_per_thread; ++k) {
                const int q = t + k * (int)blockDim.x;                  // pair number
                const int i = ((q / h) * 2 * h) + (q % h);
                const float a = ex[i], b = ex[i + h];
                ex[i] = a + b;
                ex[i + h] = a - b;
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = ex[8 * t + i];
    }
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float a = v[2 * i] * p.scale, b = v[2 * i + 1] * p.scale;
        if (p.transpose) a *= sg[2 * i], b *= sg[2 * i + 1];
        o[i] = half2_as_u32(__floats2half2_rn(a, b));
    }
    *reinterpret_cast<uint4 *>(p.out + row * p.ld_out + col) = make_uint4(o[0], o[1], o[2], o[3]);
}

}  // namespace rptc

using namespace rptc;

extern "C" int rptc_hadamard(const void *in, int in_is_f32, int64_t ld_in, void *out, int64_t ld_out, const void *signs,
                             int64_t rows, int64_t n, int block, int transpose, float scale, int clear_in,
                             rptc_stream_t stream) {
    if (!in || !out) return RPTC_ERR_ARG;
    if (block < 8 || block > 4096 || (block & (block - 1))) return RPTC_ERR_ARG;
    if (rows <= 0 || n <= 0 || (n % block) || ld_in < n || ld_out < n) return RPTC_ERR_SHAPE;
    if (rows > 65535) return RPTC_ERR_TOO_LARGE;
    const int chunk = block < 256 ? 256 : block;
    if (n % chunk) return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
        (signs && (reinterpret_cast<uintptr_t>(signs) & 15)) || (ld_in % 8) || (ld_out % 8))
        return RPTC_ERR_ALIGN;
    if (clear_in && !in_is_f32) return RPTC_ERR_ARG;
    if (int e = rptc_check_device()) return e;
    HadParams p;
    p.in = in;
    p.ld_in = ld_in;
    p.out = static_cast<__half *>(out);
    p.ld_out = ld_out;
    p.signs = static_cast<const __half *>(signs);
    p.block = block;
    p.chunk = chunk;
    p.in_is_f32 = in_is_f32;
    p.transpose = transpose;
    p.clear_in = clear_in;
    float norm = 1.f;
    for (int b = block; b > 1; b >>= 2) norm *= (b >= 4) ? 0.5f : 0.70710678118654752f;
    p.scale = scale * norm;
    return launch(hadamard_kernel, dim3((unsigned)(n / chunk), (unsigned)rows), dim3(chunk / 8), 0,
                  static_cast<cudaStream_t>(stream), p);
}
