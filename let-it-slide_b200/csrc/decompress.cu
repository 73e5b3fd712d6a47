// Standalone RPTC decompress: packed trellis codes -> dense fp16 [m][n] on sm_100a.
//
// A persistent grid of one 1024-thread CTA per SM keeps the lookup table in shared memory for the
// whole launch.  Work is cut into warp tasks of 32 "groups" (a group is one 128-bit unit, or three
// units when K = 3) and the flattened task list is split evenly over all warps.  Two lane mappings:
//   ROWLANES  (UNITMAJOR codes): lane = row of a 32-row block, the warp walks along the rows group
//             by group; the load of a group is one coalesced 512-byte request and the 16 bits of
//             history come from the previous iteration's last word.
//   !ROWLANES (ROWMAJOR / CHUNKED codes): lane = one of 32 consecutive groups of one row; history
//             comes from the lane to the left by shuffle.
// Each lane decodes its group in registers (funnel-shift windows -> table lookups) and writes its
// contiguous run of fp16 weights with 128-bit stores, four pairs at a time.
#include "common.cuh"

namespace rptc {

constexpr int kDecThreads = 1024;
constexpr int kDecWarps = kDecThreads / 32;

struct DecParams {
    const uint4 *codes;
    UnitStrides st;
    const __half *lut;
    const uint32_t *carry_in;
    __half *out;
    int64_t ld_out;
    int64_t m;
    int32_t n_groups;
    int32_t L, S, quirk;
    unsigned int *status;
};

template <int CODE, int K, bool ROWLANES>
__global__ void __launch_bounds__(kDecThreads, 1) decompress_kernel(const DecParams p) {
    using G = GroupShape<K>;
    constexpr int P = G::P;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t lut_tab = (CODE == RPTC_CODE_HASH) ? kHashLutWindow : smem_addr(smem_raw);
    lut_fill<CODE>(lut_tab, p.lut, p.L, p.S);
    const Lut<CODE> lut = lut_view<CODE>(lut_tab, p.L, p.S);
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    __syncthreads();

    const int64_t gw = (int64_t)blockIdx.x * kDecWarps + warp, GW = (int64_t)gridDim.x * kDecWarps;
    const int32_t ng = p.n_groups;
    const int32_t ngb = (ng + 31) >> 5;                                   // 32-group blocks per row (!ROWLANES)
    const int64_t T = ROWLANES ? (p.m >> 5) * (int64_t)ng : p.m * (int64_t)ngb;
    const int64_t f0 = T * gw / GW, f1 = T * (gw + 1) / GW;

    int64_t cur_rb = -1;
    uint32_t prevw = 0;
    // (outer, inner) = (row block, group) or (row, 32-group block); advanced without divisions
    const int32_t inner_n = ROWLANES ? ng : ngb;
    int64_t outer = (f0 < f1) ? f0 / inner_n : 0;
    int32_t inner = (f0 < f1) ? (int32_t)(f0 - outer * inner_n) : 0;
    for (int64_t f = f0; f < f1; ++f) {
        int64_t row;
        int32_t g;
        bool active = true;
        if (ROWLANES) {
            const int64_t rb = outer;
            g = inner;
            row = (rb << 5) + lane;
            if (rb != cur_rb) {
                cur_rb = rb;
                if (g == 0) prevw = p.carry_in ? __ldg(p.carry_in + row) : 0u;
                else prevw = __ldg(reinterpret_cast<const uint32_t *>(p.codes + unit_index(p.st, (int64_t)g * P - 1, row)) + 3);
            }
        } else {
            row = outer;
            g = inner * 32 + lane;
            active = g < ng;
        }
        if (++inner == inner_n) {
            inner = 0;
            ++outer;
        }
        uint32_t w[G::kWords];
#pragma unroll
        for (int k = 0; k < P; ++k) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (active) v = ldg128_stream(p.codes + unit_index(p.st, (int64_t)g * P + k, row));
            w[4 * k] = v.x, w[4 * k + 1] = v.y, w[4 * k + 2] = v.z, w[4 * k + 3] = v.w;
        }
        const uint32_t lastw = w[G::kWords - 1];
        if (!ROWLANES) {
            prevw = __shfl_up_sync(0xFFFFFFFFu, lastw, 1);
            if (lane == 0) {
                if (g == 0) prevw = p.carry_in ? __ldg(p.carry_in + row) : 0u;
                else prevw = __ldg(reinterpret_cast<const uint32_t *>(p.codes + unit_index(p.st, (int64_t)g * P - 1, row)) + 3);
            }
        }
        uint32_t halo = prevw;
        if (K == 2 && p.quirk != RPTC_QUIRK_NONE && (g & 31) == 0) {
            if (p.quirk == RPTC_QUIRK_K2_LANE0_CARRY) halo = lastw;
            else if (g > 0) halo = prevw >> 16;
        }
        if (ROWLANES) prevw = lastw;
        if (!active) continue;

        __half *dst = p.out + row * p.ld_out + (int64_t)g * G::kWeights;
        uint32_t buf[4];
        decode_group<CODE, K>(w, halo, lut, [&](int pi, __half2 wp) {
            buf[pi & 3] = half2_as_u32(wp);
            if ((pi & 3) == 3) {
                asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst + 2 * (pi - 3)), "r"(buf[0]), "r"(buf[1]),
                             "r"(buf[2]), "r"(buf[3])
                             : "memory");
            }
        });
    }
}

template <int CODE, int K, bool ROWLANES>
static int launch_dec(const DecParams &p, size_t smem, cudaStream_t stream) {
    static bool configured = false;
    auto kern = decompress_kernel<CODE, K, ROWLANES>;
    if (!configured) {
        RPTC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        configured = true;
    }
    return launch(kern, dim3(num_sms()), dim3(kDecThreads), smem, stream, p);
}

template <int CODE, int K>
static int dispatch_dec(const DecParams &p, bool rowlanes, size_t smem, cudaStream_t stream) {
    return rowlanes ? launch_dec<CODE, K, true>(p, smem, stream) : launch_dec<CODE, K, false>(p, smem, stream);
}

int check_format(const rptc_format *f);   // api.cu

}  // namespace rptc

using namespace rptc;

extern "C" int rptc_decompress(const void *codes, const void *lut, const uint32_t *carry_in, void *out, int64_t ld_out,
                               int64_t m, int64_t n, const rptc_format *fmt, rptc_stream_t stream) {
    if (!codes || !lut || !out || !fmt) return RPTC_ERR_ARG;
    if (int e = check_format(fmt)) return e;
    const int K = fmt->K;
    const int P = (K == 3) ? 3 : 1;
    const int wpg = 128 * P / K;
    if (m <= 0 || n <= 0 || (m % 32) || (n % wpg) || ld_out < n) return RPTC_ERR_SHAPE;
    if (m > (int64_t(1) << 30) || n > (int64_t(1) << 30)) return RPTC_ERR_TOO_LARGE;
    const int64_t n_units = n / wpg * P;
    if (fmt->layout == RPTC_LAYOUT_CHUNKED && (n_units % 32)) return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(lut) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 15) || (ld_out % 8))
        return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;

    DecParams p;
    p.codes = static_cast<const uint4 *>(codes);
    p.st = unit_strides(fmt->layout, m, n_units);
    p.lut = static_cast<const __half *>(lut);
    p.carry_in = carry_in;
    p.out = static_cast<__half *>(out);
    p.ld_out = ld_out;
    p.m = m;
    p.n_groups = (int32_t)(n / wpg);
    p.L = fmt->L;
    p.S = fmt->S;
    p.quirk = fmt->quirk;
    p.status = device_status_word();
    if (!p.status) return RPTC_ERR_CUDA;
    const bool rowlanes = fmt->layout == RPTC_LAYOUT_UNITMAJOR;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    size_t smem;
    switch (fmt->code) {
        case RPTC_CODE_LUT:
            smem = (size_t(2) << fmt->L) + 128;
            if (K == 2) return dispatch_dec<RPTC_CODE_LUT, 2>(p, rowlanes, smem, s);
            if (K == 3) return dispatch_dec<RPTC_CODE_LUT, 3>(p, rowlanes, smem, s);
            return dispatch_dec<RPTC_CODE_LUT, 4>(p, rowlanes, smem, s);
        case RPTC_CODE_HASH:
            smem = kHashLutWindow + kHashLutBytes;
            return dispatch_dec<RPTC_CODE_HASH, 2>(p, rowlanes, smem, s);
        case RPTC_CODE_LITE:
            smem = (size_t(128) << fmt->S) + 128;
            if (K == 2) return dispatch_dec<RPTC_CODE_LITE, 2>(p, rowlanes, smem, s);
            return dispatch_dec<RPTC_CODE_LITE, 4>(p, rowlanes, smem, s);
    }
    return RPTC_ERR_UNSUPPORTED;
}
