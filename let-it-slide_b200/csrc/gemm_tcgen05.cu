// Fused RPTC decode + GEMM for prefill on the sm_100a tensor cores (tcgen05 + TMEM).
//
//   y[t][row] = sum_c x[t][c] * W[row][c]        x: [tokens][n] fp16,  W decoded on the fly
//
// One CTA owns an output tile of 256 tokens x NROWS weight rows (256 when m allows, else 128) and walks
// the reduction dimension in steps of 64 columns through a ring of shared-memory stages.  With both
// operands read from shared memory a 128 x 128 x 16 MMA needs 8 KiB of operand reads per 64 tensor-core
// cycles -- exactly the 128 B/clk a SM's shared memory delivers -- so the wide tile (N = 256, 12 KiB per
// 128 cycles) is what lets the tensor pipe run ahead of shared memory.  Warp roles:
//   warps 0-7  decode producers in two groups of four that take alternate steps, so that two stages
//              are being decoded at any time: thread r of a group owns weight row r of the tile.  Per step
//              it takes the row's next 128 * K / 2 code bits with 128-bit loads (coalesced per 32-row
//              block of the TILED layout), rebuilds the shift-register windows with funnel shifts, looks
//              the weights up, and writes its 128-byte row of the B operand straight into the
//              128-byte-swizzled K-major layout the tensor core reads.  After the last step the same
//              warps run the epilogue (group g drains token half g).
//   warp 8     one lane issues the 2-D TMA loads of the activation tile (two 128-token halves).
//   warp 9     owns the TMEM allocation; one lane issues tcgen05.mma (M=128, N=128, K=16, fp32
//              accumulators in TMEM, two token halves) and commits each stage back to the producers.
// Epilogue: tcgen05.ld 32 lanes x 32 columns at a time -> fp16 -> 128-bit global stores.
// Every wait on an mbarrier is bounded; a wait that runs out raises the device status word and the
// CTA drains and returns (TMEM is still released).
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace rptc {

constexpr int kTileTokens = 256;       // two M = 128 halves
constexpr int kStepCols = 64;          // one 128-byte swizzle atom of fp16
constexpr uint32_t kXHalfBytes = 128 * kStepCols * 2;          // 16 KiB
constexpr uint32_t kXBytes = 2 * kXHalfBytes;                  // 32 KiB
constexpr int kMaxGemmStages = 3;
constexpr int kGemmThreads = 320;
constexpr int kProducerWarps = 8, kTmaWarp = 8, kMmaWarp = 9;

struct GemmParams {
    const uint4 *codes;
    const __half *lut;
    const uint32_t *carry_in;
    __half *y;
    int64_t ld_y;
    int64_t m, n, tokens;
    int32_t n_units;                  // units per row
    int32_t L, S;
    int32_t n_stages;
    uint32_t bar_addr, lut_addr;      // absolute addresses in the shared window
    uint32_t xa_addr[kMaxGemmStages], xb_addr[kMaxGemmStages], w_addr[kMaxGemmStages];   // the three pieces of a stage
    unsigned int *status;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]^T, kind::f16, cta_group::1
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// K-major operand tile, 128-byte swizzle, 8-row groups 1024 bytes apart; `addr` + 32 bytes per K = 16 step.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// fp32 accumulate, fp16 A and B, both K-major, M = 128
constexpr uint32_t instr_desc(int n_rows) { return (1u << 4) | ((uint32_t)(n_rows >> 3) << 17) | ((uint32_t)(128 >> 4) << 24); }

template <int CODE, int K, int NROWS>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_kernel(const GemmParams p, const __grid_constant__ CUtensorMap x_map) {
    constexpr int UPS = K / 2;                 // 128-bit units per 64-column step
    constexpr int kTileRows = NROWS;
    constexpr uint32_t kTmemCols = 2 * NROWS;  // two token halves of NROWS fp32 columns
    constexpr uint32_t kInstrDesc = instr_desc(NROWS);
    constexpr int kGroups = NROWS == 256 ? 1 : 2;        // producer groups taking alternate steps
    constexpr uint32_t kProducersPerStage = 256 / kGroups;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t s0 = smem_addr(smem_raw);
    if (s0 > p.bar_addr) {                     // the dynamic area starts later than the host planned for
        if (tid == 0) atomicExch(p.status, kStatusSmemPlan);
        return;
    }
    // barriers: full_w[s] (128 producer arrivals), full_x[s] (TMA bytes), empty[s] (MMA commit), accum, tmem slot
    const uint32_t bar_full_w = p.bar_addr, bar_full_x = p.bar_addr + 8 * kMaxGemmStages, bar_empty = p.bar_addr + 16 * kMaxGemmStages;
    const uint32_t bar_accum = p.bar_addr + 24 * kMaxGemmStages, tmem_slot = bar_accum + 8;
    const int n_steps = (int)(p.n / kStepCols);
    const int64_t row0 = (int64_t)blockIdx.x * kTileRows;
    const int tok0 = blockIdx.y * kTileTokens;

    if (tid == 0) {
        for (int s = 0; s < p.n_stages; ++s) {
            mbar_init(bar_full_w + 8 * s, kProducersPerStage);
            mbar_init(bar_full_x + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_accum, 1);
        mbar_fence_init();
    }
    if (warp == kMmaWarp) {                     // TMEM: two fp32 accumulators of NROWS columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the lookup table is only needed by the producer warps, but everyone helps to fill it
    {
        // lut_fill assumes blockDim.x threads take part
        lut_fill<CODE>(p.lut_addr, p.lut, p.L, p.S);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_allow_next_grid();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
    bool ok = true;

    if (warp < kProducerWarps) {
        // ================= decode producers =================
        const Lut<CODE> lut = lut_view<CODE>(p.lut_addr, p.L, p.S);
        const int group = kGroups == 2 ? warp >> 2 : 0;      // takes steps it = group, group + kGroups, ...
        const int r = kGroups == 2 ? (tid & 127) : tid;      // row of the tile
        const int64_t row = row0 + r;
        // TILED layout: unit u of row -> ((row >> 5) * n_units + u) * 32 + (row & 31)
        const uint4 *src = p.codes + ((row >> 5) * (int64_t)p.n_units) * 32 + (row & 31);
        auto history = [&](int it) -> uint32_t {             // last word before step `it` (decoded by the other group)
            if (it == 0) return p.carry_in ? __ldg(p.carry_in + row) : 0u;
            return __ldg(reinterpret_cast<const uint32_t *>(src + ((int64_t)it * UPS - 1) * 32) + 3);
        };
        uint4 nxt[UPS];
        uint32_t nxt_prev = 0, carry = 0;                    // carry: last word of the previous step when this thread decoded it
        if (group < n_steps) {
#pragma unroll
            for (int q = 0; q < UPS; ++q) nxt[q] = ldg128_stream(src + ((int64_t)group * UPS + q) * 32);
            nxt_prev = history(group);
        }
        for (int it = group; it < n_steps && ok; it += kGroups) {
            const int s = it % p.n_stages;
            const uint32_t par = ((uint32_t)(it / p.n_stages) & 1u) ^ 1u;
            uint4 cur[UPS];
#pragma unroll
            for (int q = 0; q < UPS; ++q) cur[q] = nxt[q];
            uint32_t prevw = (kGroups == 2 || it == 0) ? nxt_prev : carry;
            if (it + kGroups < n_steps) {
#pragma unroll
                for (int q = 0; q < UPS; ++q) nxt[q] = ldg128_stream(src + ((int64_t)(it + kGroups) * UPS + q) * 32);
                nxt_prev = kGroups == 2 ? history(it + kGroups) : 0u;
            }
            ok = mbar_wait(bar_empty + 8 * s, par, p.status);          // the MMA is done with this stage's old contents
            if (!ok) break;
            const uint32_t wrow = p.w_addr[s] + (uint32_t)r * 128u;
#pragma unroll
            for (int q = 0; q < UPS; ++q) {
                const uint32_t w[4] = {cur[q].x, cur[q].y, cur[q].z, cur[q].w};
                uint32_t buf[4];
                decode_group<CODE, K>(w, prevw, lut, [&](int pi, __half2 wp) {
                    buf[pi & 3] = half2_as_u32(wp);
                    if ((pi & 3) == 3) {
                        const uint32_t chunk = (uint32_t)(q * (GroupShape<K>::kPairs / 4) + (pi >> 2));     // 16-byte chunk of the row
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(wrow + 16u * (chunk ^ ((uint32_t)r & 7u))), "r"(buf[0]),
                                     "r"(buf[1]), "r"(buf[2]), "r"(buf[3])
                                     : "memory");
                    }
                });
                prevw = cur[q].w;
            }
            carry = prevw;
            fence_proxy_async_smem();               // make the generic-proxy stores visible to the tensor core's reads
            mbar_arrive(bar_full_w + 8 * s);
        }
    } else if (warp == kTmaWarp) {
        // ================= activation loads =================
        pdl_wait_prior_grids();
        if (lane == 0) {
            for (int it = 0; it < n_steps && ok; ++it) {
                const int s = it % p.n_stages;
                const uint32_t par = ((uint32_t)(it / p.n_stages) & 1u) ^ 1u;
                ok = mbar_wait(bar_empty + 8 * s, par, p.status);
                if (!ok) break;
                mbar_expect_tx(bar_full_x + 8 * s, kXBytes);
                tma_load_2d(p.xa_addr[s], &x_map, it * kStepCols, tok0, bar_full_x + 8 * s);
                tma_load_2d(p.xb_addr[s], &x_map, it * kStepCols, tok0 + 128, bar_full_x + 8 * s);
            }
        }
    } else {
        // ================= MMA issue =================
        if (lane == 0) {
            for (int it = 0; it < n_steps && ok; ++it) {
                const int s = it % p.n_stages;
                const uint32_t par = (uint32_t)(it / p.n_stages) & 1u;
                ok = mbar_wait(bar_full_x + 8 * s, par, p.status) && mbar_wait(bar_full_w + 8 * s, par, p.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t xa = p.xa_addr[s], xb = p.xb_addr[s], wa = p.w_addr[s];
#pragma unroll
                for (int k = 0; k < kStepCols / 16; ++k) {
                    const uint64_t bdesc = umma_desc_sw128(wa + 32u * k);
                    tc_mma_f16(tmem_base, umma_desc_sw128(xa + 32u * k), bdesc, kInstrDesc, (it | k) != 0);
                    tc_mma_f16(tmem_base + (uint32_t)NROWS, umma_desc_sw128(xb + 32u * k), bdesc, kInstrDesc, (it | k) != 0);
                }
                tc_commit(bar_empty + 8 * s);       // arrives when the MMAs above have read this stage
            }
            if (ok) tc_commit(bar_accum);           // arrives when every MMA has written its accumulator
        }
    }

    // ================= epilogue (warps 0-7): TMEM -> fp16 -> global =================
    if (warp < kProducerWarps) {
        if (ok) ok = mbar_wait(bar_accum, 0, p.status);
        tc_fence_after();
        if (ok) {
            const int h = warp >> 2, quarter = warp & 3;              // a warp may only touch TMEM lanes 32*(warp % 4) ...
            const int64_t tok = (int64_t)tok0 + h * 128 + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < kTileRows / 32; ++c) {
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(h * NROWS + c * 32);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                      "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                      "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                      "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (tok < p.tokens) {
                    __half *dst = p.y + tok * p.ld_y + row0 + c * 32;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t o[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            o[e] = half2_as_u32(__floats2half2_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1])));
                        asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst + 8 * j), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                                     : "memory");
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---- host -----------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 encode_tiled_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }
    return fn;
}

template <int CODE, int K, int NROWS>
static int launch_gemm(const GemmParams &p, const CUtensorMap &map, size_t smem, dim3 grid, cudaStream_t stream) {
    static SmemOptIn opted;
    auto kern = gemm_kernel<CODE, K, NROWS>;
    if (int e = allow_max_smem(kern, opted)) return e;
    return launch(kern, grid, dim3(kGemmThreads), smem, stream, p, map);
}

template <int CODE, int K>
static int launch_gemm_rows(int n_rows, const GemmParams &p, const CUtensorMap &map, size_t smem, dim3 grid, cudaStream_t stream) {
    return n_rows == 256 ? launch_gemm<CODE, K, 256>(p, map, smem, grid, stream) : launch_gemm<CODE, K, 128>(p, map, smem, grid, stream);
}

int check_format(const rptc_format *f);   // api.cu

}  // namespace rptc

using namespace rptc;

extern "C" int rptc_gemm(const void *codes, const void *lut, const uint32_t *carry_in, const void *x, int64_t ld_x, void *y,
                         int64_t ld_y, int64_t m, int64_t n, int64_t tokens, const rptc_format *fmt, rptc_stream_t stream) {
    if (!codes || !lut || !x || !y || !fmt) return RPTC_ERR_ARG;
    if (int e = check_format(fmt)) return e;
    if (fmt->layout != RPTC_LAYOUT_TILED || fmt->quirk != RPTC_QUIRK_NONE) return RPTC_ERR_UNSUPPORTED;
    if (fmt->K != 2 && fmt->K != 4) return RPTC_ERR_UNSUPPORTED;
    if (m <= 0 || n <= 0 || tokens <= 0 || (m % 128) || (n % kStepCols) || ld_x < n || ld_y < m) return RPTC_ERR_SHAPE;
    if (m > (int64_t(1) << 30) || n > (int64_t(1) << 30) || tokens > (int64_t(1) << 24)) return RPTC_ERR_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(lut) & 15) || (reinterpret_cast<uintptr_t>(x) & 15) ||
        (reinterpret_cast<uintptr_t>(y) & 15) || (ld_x % 8) || (ld_y % 8))
        return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    auto encode = encode_tiled_fn();
    if (!encode) return RPTC_ERR_CUDA;

    CUtensorMap map;
    const cuuint64_t gdim[2] = {(cuuint64_t)n, (cuuint64_t)tokens};
    const cuuint64_t gstride[1] = {(cuuint64_t)ld_x * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kStepCols, 128};
    const cuuint32_t estride[2] = {1, 1};
    CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x), gdim, gstride, box, estride,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = (int)r;
        return RPTC_ERR_CUDA;
    }

    GemmParams p;
    p.codes = static_cast<const uint4 *>(codes);
    p.lut = static_cast<const __half *>(lut);
    p.carry_in = carry_in;
    p.y = static_cast<__half *>(y);
    p.ld_y = ld_y;
    p.m = m;
    p.n = n;
    p.tokens = tokens;
    p.n_units = (int32_t)(n * fmt->K / 128);
    p.L = fmt->L;
    p.S = fmt->S;
    p.status = device_status_word();
    if (!p.status) return RPTC_ERR_CUDA;
    // shared-window plan (absolute addresses; the dynamic area is expected to start at or below 0x400): the
    // pieces of each stage (two activation halves, one weight tile) go first-fit into the space around the table
    const uint32_t kTop = 0x38800;       // 226 KiB: the last byte any plan may touch (dynamic limit is 227 KiB)
    p.bar_addr = 0x400;
    uint32_t free_lo[2], free_hi[2];
    int n_free;
    if (fmt->code == RPTC_CODE_HASH) {
        p.lut_addr = kHashLutWindow;
        free_lo[0] = 0x800, free_hi[0] = kHashLutWindow;
        free_lo[1] = kHashLutWindow + kHashLutBytes, free_hi[1] = kTop;
        n_free = 2;
    } else {
        p.lut_addr = 0x800;
        const uint32_t lb = fmt->code == RPTC_CODE_LUT ? (2u << fmt->L) : (128u << fmt->S);
        free_lo[0] = (0x800 + lb + 1023u) & ~1023u, free_hi[0] = kTop;
        n_free = 1;
    }
    auto take = [&](uint32_t bytes) -> uint32_t {
        for (int i = 0; i < n_free; ++i)
            if (free_lo[i] + bytes <= free_hi[i]) {
                const uint32_t a = free_lo[i];
                free_lo[i] += bytes;
                return a;
            }
        return 0;
    };
    // Tile height: 256 rows feed the tensor pipe about 1.35x faster per CTA-step than 128 rows, but need twice
    // the time per CTA; with few tiles the shorter ones fill more SMs.  Compare whole waves of CTAs.
    int n_rows = 128;
    if (m % 256 == 0) {
        const int64_t tt = (tokens + kTileTokens - 1) / kTileTokens, sms = num_sms();
        const int64_t waves256 = ((m / 256) * tt + sms - 1) / sms, waves128 = ((m / 128) * tt + sms - 1) / sms;
        if (waves256 * 148 <= waves128 * 100) n_rows = 256;          // 2 / 1.35 = 1.48
    }
    int stages = 0;
    for (int attempt = 0; attempt < 2 && stages < 2; ++attempt) {
        if (attempt == 1) {              // the wide tile does not fit beside this table: fall back to 128 rows
            if (n_rows == 128) break;
            n_rows = 128;
            if (fmt->code == RPTC_CODE_HASH) {
                free_lo[0] = 0x800, free_lo[1] = kHashLutWindow + kHashLutBytes;
            } else {
                const uint32_t lb = fmt->code == RPTC_CODE_LUT ? (2u << fmt->L) : (128u << fmt->S);
                free_lo[0] = (0x800 + lb + 1023u) & ~1023u;
            }
        }
        stages = 0;
        const int want = n_rows == 256 ? 2 : kMaxGemmStages;
        while (stages < want) {
            const uint32_t save0 = free_lo[0], save1 = free_lo[1];
            const uint32_t w = take((uint32_t)n_rows * 128u), xa = take(kXHalfBytes), xb = take(kXHalfBytes);
            if (!w || !xa || !xb) {
                free_lo[0] = save0, free_lo[1] = save1;
                break;
            }
            p.w_addr[stages] = w, p.xa_addr[stages] = xa, p.xb_addr[stages] = xb;
            ++stages;
        }
    }
    if (stages < 2) return RPTC_ERR_UNSUPPORTED;
    for (int s = stages; s < kMaxGemmStages; ++s) p.w_addr[s] = p.xa_addr[s] = p.xb_addr[s] = 0;
    p.n_stages = stages;
    const size_t smem = kTop;            // covers every planned address whatever the start of the dynamic area
    const dim3 grid((unsigned)(m / n_rows), (unsigned)((tokens + kTileTokens - 1) / kTileTokens));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (fmt->code) {
        case RPTC_CODE_LUT:
            return fmt->K == 2 ? launch_gemm_rows<RPTC_CODE_LUT, 2>(n_rows, p, map, smem, grid, s)
                               : launch_gemm_rows<RPTC_CODE_LUT, 4>(n_rows, p, map, smem, grid, s);
        case RPTC_CODE_HASH:
            return launch_gemm_rows<RPTC_CODE_HASH, 2>(n_rows, p, map, smem, grid, s);
        case RPTC_CODE_LITE:
            return fmt->K == 2 ? launch_gemm_rows<RPTC_CODE_LITE, 2>(n_rows, p, map, smem, grid, s)
                               : launch_gemm_rows<RPTC_CODE_LITE, 4>(n_rows, p, map, smem, grid, s);
    }
    return RPTC_ERR_UNSUPPORTED;
}
