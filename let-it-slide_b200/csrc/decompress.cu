// Standalone RPTC decompress: packed trellis codes -> dense fp16 [m][n] on sm_100a.
//
// A persistent grid of one 512-thread CTA per SM keeps the lookup table in shared memory for the
// whole launch.  Work is cut into warp tasks of 32 "groups" (a group is one 128-bit unit, or three
// units when K = 3) and the flattened task list is split evenly over all warps.  Two lane mappings:
//   ROWLANES  (TILED / UNITMAJOR codes): lane = row of a 32-row block, the warp walks along the rows group
//             by group; the load of a group is one coalesced 512-byte request and the 16 bits of
//             history come from the previous iteration's last word.
//   !ROWLANES (ROWMAJOR / CHUNKED codes): lane = one of 32 consecutive groups of one row; history
//             comes from the lane to the left by shuffle.
// Each lane decodes its group in registers (funnel-shift windows -> table lookups) into its own row
// of a per-warp shared-memory tile (XOR-swizzled in 16-byte chunks, so the writes are conflict
// free); the warp then copies the tile out with 128-bit stores in which every group of lanes covers
// whole 128-byte lines of the output.  Output is 8x (K=2) the input, so this kernel lives or dies by
// the store pattern.
#include "common.cuh"

namespace rptc {

constexpr int kDecThreads = 512;
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

template <int K>
struct DecTile {
    static constexpr int kRowBytes = 2 * GroupShape<K>::kWeights;      // 128, 256, 64
    static constexpr int kChunks = kRowBytes / 16;                     // 8, 16, 4
    static constexpr int kBytes = 32 * kRowBytes;
    // 16-byte chunk c of tile row r lives at chunk swz(r, c) of that row
    __device__ static __forceinline__ uint32_t swz(uint32_t r, uint32_t c) {
        return kChunks == 4 ? (c ^ ((r >> 1) & 3u)) : (c ^ (r & 7u));
    }
};

template <int CODE, int K, bool ROWLANES>
__global__ void __launch_bounds__(kDecThreads, 1) decompress_kernel(const DecParams p) {
    using G = GroupShape<K>;
    using T = DecTile<K>;
    constexpr int P = G::P;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t s0 = smem_addr(smem_raw);
    uint32_t lut_tab, tiles;
    if (CODE == RPTC_CODE_HASH) {
        lut_tab = kHashLutWindow;
        tiles = kHashLutWindow + kHashLutBytes;
    } else {
        lut_tab = s0;
        tiles = s0 + lut_bytes<CODE>(p.L, p.S);
    }
    const uint32_t tile = tiles + (uint32_t)warp * T::kBytes;
    lut_fill<CODE>(lut_tab, p.lut, p.L, p.S);
    const Lut<CODE> lut = lut_view<CODE>(lut_tab, p.L, p.S);
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    __syncthreads();

    const int nwarps = blockDim.x >> 5;
    const int64_t gw = (int64_t)blockIdx.x * nwarps + warp, GW = (int64_t)gridDim.x * nwarps;
    const int32_t ng = p.n_groups;
    const int32_t ngb = (ng + 31) >> 5;                                   // 32-group blocks per row (!ROWLANES)
    const int64_t Ttot = ROWLANES ? (p.m >> 5) * (int64_t)ng : p.m * (int64_t)ngb;
    const int64_t f0 = Ttot * gw / GW, f1 = Ttot * (gw + 1) / GW;

    int64_t cur_rb = -1;
    uint32_t prevw = 0;
    // (outer, inner) = (row block, group) or (row, 32-group block); advanced without divisions
    const int32_t inner_n = ROWLANES ? ng : ngb;
    int64_t outer = (f0 < f1) ? f0 / inner_n : 0;
    int32_t inner = (f0 < f1) ? (int32_t)(f0 - outer * inner_n) : 0;

    auto load_group = [&](int64_t o, int32_t in, uint32_t (&w)[G::kWords]) {
        const int64_t row = ROWLANES ? (o << 5) + lane : o;
        const int32_t g = ROWLANES ? in : in * 32 + lane;
#pragma unroll
        for (int k = 0; k < P; ++k) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (g < ng) v = ldg128_stream(p.codes + unit_index(p.st, (int64_t)g * P + k, row));
            w[4 * k] = v.x, w[4 * k + 1] = v.y, w[4 * k + 2] = v.z, w[4 * k + 3] = v.w;
        }
    };
    uint32_t wnext[G::kWords];
    if (f0 < f1) load_group(outer, inner, wnext);

    for (int64_t f = f0; f < f1; ++f) {
        const int64_t o = outer;
        const int32_t in = inner;
        int64_t row;
        int32_t g;
        if (ROWLANES) {
            g = in;
            row = (o << 5) + lane;
            if (o != cur_rb) {
                cur_rb = o;
                if (g == 0) prevw = p.carry_in ? __ldg(p.carry_in + row) : 0u;
                else prevw = __ldg(reinterpret_cast<const uint32_t *>(p.codes + unit_index(p.st, (int64_t)g * P - 1, row)) + 3);
            }
        } else {
            row = o;
            g = in * 32 + lane;
        }
        const bool active = g < ng;
        if (++inner == inner_n) {
            inner = 0;
            ++outer;
        }
        uint32_t w[G::kWords];
#pragma unroll
        for (int k = 0; k < G::kWords; ++k) w[k] = wnext[k];
        if (f + 1 < f1) load_group(outer, inner, wnext);       // next task's codes are in flight while this one decodes

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

        // decode into this lane's row of the tile
        if (active) {
            const uint32_t my_row = tile + (uint32_t)lane * T::kRowBytes;
            uint32_t buf[4];
            decode_group<CODE, K>(w, halo, lut, [&](int pi, __half2 wp) {
                buf[pi & 3] = half2_as_u32(wp);
                if ((pi & 3) == 3) {
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(my_row + 16u * T::swz(lane, pi >> 2)), "r"(buf[0]),
                                 "r"(buf[1]), "r"(buf[2]), "r"(buf[3])
                                 : "memory");
                }
            });
        }
        __syncwarp();
        // copy the tile out: chunk q = i*32 + lane  ->  tile row q / kChunks, chunk q % kChunks
#pragma unroll
        for (int i = 0; i < T::kChunks; ++i) {
            const uint32_t q = (uint32_t)i * 32u + lane;
            const uint32_t r = q / T::kChunks, c = q % T::kChunks;
            __half *dst;
            bool ok;
            if (ROWLANES) {
                dst = p.out + ((o << 5) + r) * p.ld_out + (int64_t)g * G::kWeights + 8 * c;
                ok = true;
            } else {
                const int32_t gr = in * 32 + (int32_t)r;
                dst = p.out + row * p.ld_out + (int64_t)gr * G::kWeights + 8 * c;
                ok = gr < ng;
            }
            if (ok) {
                const uint4 v = lds128(tile + r * T::kRowBytes + 16u * T::swz(r, c));
                asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
            }
        }
        __syncwarp();
    }
}

// `smem` is the table's share; the per-warp tiles are added here, with fewer warps when they do not fit.
template <int CODE, int K, bool ROWLANES>
static int launch_dec(const DecParams &p, size_t smem, cudaStream_t stream) {
    int threads = kDecThreads;
    while (threads > 64 && smem + size_t(threads / 32) * DecTile<K>::kBytes > 226 * 1024) threads >>= 1;
    smem += size_t(threads / 32) * DecTile<K>::kBytes;
    static SmemOptIn opted;
    auto kern = decompress_kernel<CODE, K, ROWLANES>;
    if (int e = allow_max_smem(kern, opted)) return e;
    return launch(kern, dim3(num_sms()), dim3(threads), smem, stream, p);
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
    const bool rowlanes = fmt->layout == RPTC_LAYOUT_UNITMAJOR || fmt->layout == RPTC_LAYOUT_TILED;
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
