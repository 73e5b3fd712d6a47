// The code-A trellis encoder (the offline half of the path): for every row, the symbol sequence q[0..n) in {0..3}
// whose shift-register walk  s = ((s << 2) | q) & (2^L - 1),  s_start = 0,  minimises
//   sum_i pos_weight[i] * (samples[i] - alphabet[s_i])^2           (rptc.py:13-71, diagonal corrections).
//
// Dynamic programme over the 2^L states, one launch per position for a batch of rows:
//   best[p]   = min over d = 0..3 of rho[(d << (L-2)) | p]          (first minimum, like jnp.argmin: rptc.py:27-30)
//   rho'[4p+q] = best[p] + w * (x - alphabet[4p+q])^2                (rptc.py:52)
// Thread p reads its four predecessors (four coalesced streams), records the winning d in back[i][row][p] and
// writes the four successor costs with one 16-byte store.  rho ping-pongs between two buffers that stay in L2 for
// batches up to ~128 rows; the survivors are walked backwards by one thread per row (rptc.py:62-68).
// The arithmetic is spelled with round-to-nearest intrinsics so that no multiply-add is contracted: costs, and
// therefore ties and paths, are those of the fp32 reference.
#include "common.cuh"

namespace rptc {

__global__ void viterbi_init_kernel(float *__restrict__ rho, int64_t M) {
    const int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (s < M) rho[(int64_t)blockIdx.y * M + s] = s == 0 ? 0.f : INFINITY;       // initial state is zero (rptc.py:57-58)
}

__global__ void __launch_bounds__(256) viterbi_step_kernel(const float *__restrict__ rho, float *__restrict__ rho_next,
                                                           uint8_t *__restrict__ back, const float4 *__restrict__ alphabet,
                                                           const float *__restrict__ samples, int64_t ld_samples,
                                                           const float *__restrict__ pos_weight, int64_t index, int64_t P) {
    const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y;
    if (p >= P) return;
    const float *r = rho + row * 4 * P;
    const float c0 = r[p], c1 = r[P + p], c2 = r[2 * P + p], c3 = r[3 * P + p];
    float best = c0;
    int d = 0;
    if (c1 < best) best = c1, d = 1;
    if (c2 < best) best = c2, d = 2;
    if (c3 < best) best = c3, d = 3;
    back[row * P + p] = (uint8_t)d;
    const float x = samples[row * ld_samples + index], w = pos_weight[index];
    const float4 a = alphabet[p];
    auto cost = [&](float e) {
        const float diff = __fsub_rn(x, e);
        return __fadd_rn(best, __fmul_rn(w, __fmul_rn(diff, diff)));
    };
    reinterpret_cast<float4 *>(rho_next + row * 4 * P)[p] = make_float4(cost(a.x), cost(a.y), cost(a.z), cost(a.w));
}

// First minimum of each row of rho -> (loss, final state).
__global__ void __launch_bounds__(1024) viterbi_argmin_kernel(const float *__restrict__ rho, int64_t M, float *__restrict__ loss,
                                                              int32_t *__restrict__ final_state) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float *r = rho + (int64_t)blockIdx.x * M;
    float best = INFINITY;
    int at = 0x7FFFFFFF;
    for (int64_t s = threadIdx.x; s < M; s += 1024) {
        const float v = r[s];
        if (v < best || (v == best && s < at)) best = v, at = (int)s;
    }
    auto better = [](float v, int i, float bvv, int bii) { return v < bvv || (v == bvv && i < bii); };
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
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
            loss[blockIdx.x] = best;
            final_state[blockIdx.x] = at == 0x7FFFFFFF ? 0 : at;
        }
    }
}

// One thread per row walks the survivors from the last position to the first.
__global__ void viterbi_backtrack_kernel(const uint8_t *__restrict__ back, const int32_t *__restrict__ final_state, int64_t rows,
                                         int64_t n, int64_t P, int L, int32_t *__restrict__ symbols, int64_t ld_sym) {
    const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    uint32_t state = (uint32_t)final_state[row];
    for (int64_t i = n - 1; i >= 0; --i) {
        symbols[row * ld_sym + i] = (int32_t)(state & 3u);
        const uint32_t prefix = state >> 2;
        state = ((uint32_t)back[(i * rows + row) * P + prefix] << (L - 2)) | prefix;
    }
}

}  // namespace rptc

using namespace rptc;

extern "C" int64_t rptc_viterbi_workspace_bytes(int64_t rows, int64_t n, int L) {
    if (rows <= 0 || n <= 0 || L < 4 || L > 16) return -1;
    const int64_t M = int64_t(1) << L;
    return 2 * rows * M * 4 + n * rows * (M / 4) + rows * 4 + 256;
}

extern "C" int rptc_viterbi_encode(const float *alphabet, const float *pos_weight, const float *samples, int64_t ld_samples,
                                   int64_t rows, int64_t n, int L, int32_t *symbols, int64_t ld_sym, float *loss, void *workspace,
                                   int64_t workspace_bytes, rptc_stream_t stream) {
    if (!alphabet || !pos_weight || !samples || !symbols || !loss || !workspace) return RPTC_ERR_ARG;
    if (L < 4 || L > 16) return RPTC_ERR_UNSUPPORTED;
    if (rows <= 0 || rows > 65535 || n <= 0 || ld_samples < n || ld_sym < n) return RPTC_ERR_SHAPE;
    if (workspace_bytes < rptc_viterbi_workspace_bytes(rows, n, L)) return RPTC_ERR_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(alphabet) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 255)) return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    const int64_t M = int64_t(1) << L, P = M / 4;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float *rho_a = static_cast<float *>(workspace), *rho_b = rho_a + rows * M;
    uint8_t *back = reinterpret_cast<uint8_t *>(rho_b + rows * M);
    int32_t *final_state = reinterpret_cast<int32_t *>(back + n * rows * P + ((256 - (n * rows * P) % 256) % 256));
    viterbi_init_kernel<<<dim3((unsigned)((M + 255) / 256), (unsigned)rows), 256, 0, s>>>(rho_a, M);
    const dim3 grid((unsigned)((P + 255) / 256), (unsigned)rows);
    for (int64_t i = 0; i < n; ++i) {
        viterbi_step_kernel<<<grid, 256, 0, s>>>(rho_a, rho_b, back + i * rows * P, reinterpret_cast<const float4 *>(alphabet), samples,
                                                 ld_samples, pos_weight, i, P);
        float *t = rho_a;
        rho_a = rho_b;
        rho_b = t;
    }
    viterbi_argmin_kernel<<<(unsigned)rows, 1024, 0, s>>>(rho_a, M, loss, final_state);
    viterbi_backtrack_kernel<<<(unsigned)((rows + 63) / 64), 64, 0, s>>>(back, final_state, rows, n, P, L, symbols, ld_sym);
    RPTC_CUDA(cudaGetLastError());
    return RPTC_OK;
}
