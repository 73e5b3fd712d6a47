// Fused RPTC decode + GEMM for prefill on the sm_100a tensor cores (tcgen05 + TMEM).
//
//   y[t][row] = sum_c x[t][c] * W[row][c]        x: [tokens][n] fp16,  W decoded on the fly
//
// One CTA owns an output tile of 256 tokens x NROWS weight rows (256 when m allows, else 128) and walks the reduction
// dimension in steps of 64 columns.  With both operands read from shared memory a 128 x 128 x 16 MMA needs 8 KiB of
// operand reads per 64 tensor-core cycles -- exactly the 128 B/clk a SM's shared memory delivers -- so the wide tile
// (N = 256, 12 KiB per 128 cycles) is what lets the tensor pipe run ahead of shared memory.  The two operands travel
// through separate shared-memory rings (activations: up to four stages of 32 KiB; decoded weights: two or three stages of
// 128 bytes per tile row), each with its own full/empty barriers.  Warp roles:
//   warps 0-7  decode producers: thread r owns weight row r of the tile (256-row tiles: every thread takes every step;
//              128-row tiles: two groups of four warps take alternate steps).  Per step a thread takes its row's next
//              128 * K / 2 code bits with 128-bit loads (coalesced per 32-row block of the TILED layout), rebuilds the
//              shift-register windows with funnel shifts and looks the 64 weights up INTO REGISTERS; only then does it
//              wait for the stage, and writes its 128-byte row of the B operand straight into the 128-byte-swizzled
//              K-major layout the tensor core reads.  After the last step the same warps run the epilogue.
//   warp 8     one lane issues the 2-D TMA loads of the activation tile (two 128-token halves), as far ahead as the
//              activation ring allows.
//   warp 9     owns the TMEM allocation; one lane issues tcgen05.mma (M = 128, N = NROWS, K = 16, fp32 accumulators
//              in TMEM, two token halves) and commits each stage of either ring back to its producer.
// Epilogue: tcgen05.ld 32 lanes x 32 columns at a time -> fp16 -> 128-bit global stores.
// The HASH code's table is kept in its packed form here (32 KiB instead of the GEMV kernels' 64 KiB), which is what
// makes room for the third activation stage beside two 32 KiB weight stages.
// Every wait on an mbarrier is bounded; a wait that runs out raises the device status word and the CTA drains and
// returns (TMEM is still released).
#include <cuda.h>
#include <stdlib.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace rptc {

constexpr int kTileTokens = 256;       // two M = 128 halves
constexpr int kStepCols = 64;          // one 128-byte swizzle atom of fp16
constexpr uint32_t kXHalfBytes = 128 * kStepCols * 2;          // 16 KiB
constexpr uint32_t kXBytes = 2 * kXHalfBytes;                  // 32 KiB
constexpr int kMaxGemmStages = 4;      // per ring
constexpr int kGemmThreads = 320;
constexpr int kProducerWarps = 8, kTmaWarp = 8, kMmaWarp = 9;

// The decoded-weight ring and the activation ring are separate: a TMA load takes about a microsecond to land and so
// wants the deeper ring, while a weight stage is refilled within a few hundred cycles of being handed back (the
// producers decode into registers ahead of time and only store once the stage is free).
struct GemmParams {
    const uint4 *codes;
    const __half *lut;
    const uint32_t *carry_in;
    __half *y;
    int64_t ld_y;
    int64_t m, n, tokens;
    int32_t n_units;                  // units per row
    int32_t L, S;
    int32_t n_xstages, n_wstages;
    uint32_t bar_addr, lut_addr;      // offsets in the CTA's shared window
    uint32_t xa_addr[kMaxGemmStages], xb_addr[kMaxGemmStages];   // activation ring: two 128-token halves per stage
    uint32_t w_addr[kMaxGemmStages];                             // decoded-weight ring
    uint32_t out_addr[8];             // epilogue: panels of 128 tokens x 64 output columns (16 KiB each), laid over the rings
    unsigned int *status;
};

// Barrier block (8 bytes each) at GemmParams::bar_addr.
struct GemmBars {
    uint32_t full_w, full_x, empty_w, empty_x, accum, tmem_slot, done;
};
__device__ __forceinline__ GemmBars gemm_bars(uint32_t base) {
    GemmBars b;
    b.full_w = base;
    b.full_x = base + 8 * kMaxGemmStages;
    b.empty_w = base + 16 * kMaxGemmStages;
    b.empty_x = base + 24 * kMaxGemmStages;
    b.accum = base + 32 * kMaxGemmStages;
    b.tmem_slot = b.accum + 8;
    b.done = b.accum + 16;                        // two-SM kernel: the partner has drained its accumulators
    return b;
}

// The HASH code is looked up in the packed table (128-byte rows) here: 32 KiB instead of 64 KiB leaves room for one more
// ring stage, and the extra shift per lookup is hidden behind the tensor pipe.
template <int CODE>
struct GemmDecode {
    static constexpr int kCode = CODE == RPTC_CODE_HASH ? kCodeHashPacked : CODE;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
// Tile of shared memory -> global through the tensor map (clipped at the tensor's bounds), tracked by the thread's bulk group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
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

// ---- a pair of CTAs (cluster of two) working on one tile: signalling across ------------------------------------------
// In a pair every barrier that gates an MMA lives in the leader (rank 0): both CTAs' producers and both CTAs' TMA loads
// signal it directly.  A shared::cluster address with bit 24 cleared is the same offset in rank 0's window.
constexpr uint32_t kLeaderMask = 0xFEFFFFFFu;
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {               // `bar`: shared::cluster address
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// 2-D TMA load into this CTA's shared memory whose completion is counted on a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}

// Position in a ring of `n` stages without a division per step.
struct RingPos {
    int s;
    uint32_t phase;
    __device__ __forceinline__ void advance(int n) {
        if (++s == n) s = 0, phase ^= 1u;
    }
    __device__ __forceinline__ void advance_by(int k, int n) {
        for (int i = 0; i < k; ++i) advance(n);
    }
};

// `window` in the functions below: bits to OR onto every planned shared-memory offset (0 outside a cluster; inside one,
// the upper address bits that select this CTA's window in the cluster's).
// ---- decode producers ------------------------------------------------------------------------------------------------
// GROUPS groups of 256 / GROUPS threads take alternate steps; thread r of a group owns weight row `row0 + r`.  A step's 64
// weights are decoded into registers BEFORE the wait for the stage, so that between the tensor cores handing a stage back
// and its next contents being announced lie only eight 128-bit stores and a fence.
template <int CODE, int K, int GROUPS, bool PAIR = false>
__device__ __forceinline__ bool produce_weights(const GemmParams &p, uint32_t window, const GemmBars &bars, int64_t row0, int n_steps) {
    constexpr int DC = GemmDecode<CODE>::kCode;
    constexpr int UPS = K / 2;                 // 128-bit units per 64-column step
    constexpr int kPairs = GroupShape<K>::kPairs;
    static_assert(UPS * kPairs == 32, "a step is 32 weight pairs per row");
    const int tid = threadIdx.x, warp = tid >> 5;
    const Lut<DC> lut = lut_view<DC>(p.lut_addr | window, p.L, p.S);
    const int group = GROUPS == 2 ? warp >> 2 : 0;      // takes steps it = group, group + GROUPS, ...
    const int r = GROUPS == 2 ? (tid & 127) : tid;      // row of the tile
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
    RingPos pos = {0, 1u};                               // waits on `empty` pass at once the first time round
    pos.advance_by(group, p.n_wstages);
    for (int it = group; it < n_steps; it += GROUPS) {
        uint4 cur[UPS];
#pragma unroll
        for (int q = 0; q < UPS; ++q) cur[q] = nxt[q];
        uint32_t prevw = (GROUPS == 2 || it == 0) ? nxt_prev : carry;
        if (it + GROUPS < n_steps) {
#pragma unroll
            for (int q = 0; q < UPS; ++q) nxt[q] = ldg128_stream(src + ((int64_t)(it + GROUPS) * UPS + q) * 32);
            nxt_prev = GROUPS == 2 ? history(it + GROUPS) : 0u;
        }
        uint32_t out[32];
#pragma unroll
        for (int q = 0; q < UPS; ++q) {
            const uint32_t w[4] = {cur[q].x, cur[q].y, cur[q].z, cur[q].w};
            decode_group<DC, K>(w, prevw, lut, [&](int pi, __half2 wp) { out[q * kPairs + pi] = half2_as_u32(wp); });
            prevw = cur[q].w;
        }
        carry = prevw;
        if (!mbar_wait(bars.empty_w + 8 * pos.s, pos.phase, p.status)) return false;      // the MMAs are done with the stage's old contents
        const uint32_t wrow = (p.w_addr[pos.s] | window) + (uint32_t)r * 128u;
#pragma unroll
        for (uint32_t chunk = 0; chunk < 8; ++chunk)         // 16-byte chunks of the row, 128-byte swizzle
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(wrow + 16u * (chunk ^ ((uint32_t)r & 7u))), "r"(out[4 * chunk]),
                         "r"(out[4 * chunk + 1]), "r"(out[4 * chunk + 2]), "r"(out[4 * chunk + 3])
                         : "memory");
        fence_proxy_async_smem();               // make the generic-proxy stores visible to the tensor cores' reads
        if (PAIR) {                             // one arrival per warp, on the leader's barrier
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive_cluster((bars.full_w + 8 * pos.s) & kLeaderMask);
        } else {
            mbar_arrive(bars.full_w + 8 * pos.s);
        }
        pos.advance_by(GROUPS, p.n_wstages);
    }
    return true;
}

// ---- activation loads (one thread) ----------------------------------------------------------------------------------
template <bool PAIR = false>
__device__ __forceinline__ bool load_activations(const GemmParams &p, uint32_t window, const GemmBars &bars, const CUtensorMap *x_map, int tok0,
                                                 int n_steps) {
    RingPos pos = {0, 1u};
    for (int it = 0; it < n_steps; ++it) {
        if (!mbar_wait(bars.empty_x + 8 * pos.s, pos.phase, p.status)) return false;
        if (PAIR) {                             // bytes of both CTAs are counted on the leader's barrier
            const uint32_t bar = (bars.full_x + 8 * pos.s) & kLeaderMask;
            mbar_expect_tx_cluster(bar, kXBytes);
            tma_load_2d_pair(p.xa_addr[pos.s] | window, x_map, it * kStepCols, tok0, bar);
            tma_load_2d_pair(p.xb_addr[pos.s] | window, x_map, it * kStepCols, tok0 + 128, bar);
        } else {
            const uint32_t bar = bars.full_x + 8 * pos.s;
            mbar_expect_tx(bar, kXBytes);
            tma_load_2d(p.xa_addr[pos.s] | window, x_map, it * kStepCols, tok0, bar);
            tma_load_2d(p.xb_addr[pos.s] | window, x_map, it * kStepCols, tok0 + 128, bar);
        }
        pos.advance(p.n_xstages);
    }
    return true;
}

// ---- epilogue (warps 0-7): TMEM -> fp16 -> shared memory -> global ----------------------------------------------------
// `tok0` is this CTA's first token, `row0` the tile's first weight row.  The rings are free once the last MMA has been
// committed, so the 256 x NROWS fp16 tile is laid over them as panels of 128 tokens x 64 columns in the 128-byte-swizzled
// form a TMA store reads (a thread owns a token: its 16-byte chunks land in four-way-interleaved banks, the minimum for
// 512 bytes per warp), and one thread sends the panels off.  Against per-thread global stores (32 different lines per
// instruction) this cut the epilogue from 8.3 us to the time the tile takes to leave through the copy engine.
template <int NROWS>
__device__ __forceinline__ void drain_accumulators(const GemmParams &p, uint32_t window, uint32_t tmem_base, int tok0, int64_t row0,
                                                   const CUtensorMap *y_map, bool ok) {
    constexpr int kPanelsPerHalf = NROWS / 64;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = warp >> 2, quarter = warp & 3;              // a warp may only touch TMEM lanes 32*(warp % 4) ...
    const uint32_t t = (uint32_t)(quarter * 32 + lane);       // token inside the half = row of the panel
    // All eight warps come here, also one whose wait ran out (`ok` false: it skips its part, and nothing is sent).
#pragma unroll 1
    for (int c = 0; ok && c < NROWS / 32; ++c) {
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
        const uint32_t prow = (p.out_addr[h * kPanelsPerHalf + (c >> 1)] | window) + t * 128u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
                o[e] = half2_as_u32(__floats2half2_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1])));
            const uint32_t chunk = (uint32_t)((c & 1) * 4 + j);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(prow + 16u * (chunk ^ (t & 7u))), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                         : "memory");
        }
    }
    fence_proxy_async_smem();                                 // the stores above are read by the copy engine
    uint32_t all_ok;                                          // barrier of the eight epilogue warps, AND of their `ok`
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "barrier.cta.red.and.pred p, 1, 256, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(all_ok)
        : "r"((uint32_t)ok)
        : "memory");
    if (threadIdx.x == 0 && all_ok) {
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
            if ((int64_t)tok0 + hh * 128 >= p.tokens) break;  // a half with no tokens at all (rows beyond `tokens` inside a half are clipped)
#pragma unroll 1
            for (int q = 0; q < kPanelsPerHalf; ++q)
                tma_store_2d(y_map, (int)row0 + q * 64, tok0 + hh * 128, p.out_addr[hh * kPanelsPerHalf + q] | window);
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");     // the tile has left before the CTA (and its shared memory) goes
    }
}

__device__ __forceinline__ void init_ring_barriers(const GemmParams &p, const GemmBars &bars, uint32_t w_arrivals, uint32_t x_arrivals) {
    for (int s = 0; s < kMaxGemmStages; ++s) {
        mbar_init(bars.full_w + 8 * s, w_arrivals);
        mbar_init(bars.full_x + 8 * s, x_arrivals);
        mbar_init(bars.empty_w + 8 * s, 1);
        mbar_init(bars.empty_x + 8 * s, 1);
    }
    mbar_init(bars.accum, 1);
    mbar_init(bars.done, 1);
    mbar_fence_init();
}

template <int CODE, int K, int NROWS>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_kernel(const GemmParams p, const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap y_map) {
    constexpr int DC = GemmDecode<CODE>::kCode;
    constexpr uint32_t kTmemCols = 2 * NROWS;  // two token halves of NROWS fp32 columns
    constexpr uint32_t kInstrDesc = instr_desc(NROWS);
    constexpr int kGroups = NROWS == 256 ? 1 : 2;        // producer groups taking alternate steps
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t s0 = smem_addr(smem_raw);
    if (s0 > p.bar_addr) {                     // the dynamic area starts later than the host planned for
        if (tid == 0) atomicExch(p.status, kStatusSmemPlan);
        return;
    }
    const GemmBars bars = gemm_bars(p.bar_addr);
    const int n_steps = (int)(p.n / kStepCols);
    const int64_t row0 = (int64_t)blockIdx.x * NROWS;
    const int tok0 = blockIdx.y * kTileTokens;

    if (tid == 0) init_ring_barriers(p, bars, 256 / kGroups, 1);
    if (warp == kMmaWarp) {                     // TMEM: two fp32 accumulators of NROWS columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(bars.tmem_slot), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    lut_fill<DC>(p.lut_addr, p.lut, p.L, p.S);         // only the producer warps read the table, but everyone helps to fill it
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_allow_next_grid();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(bars.tmem_slot));
    bool ok = true;

    if (warp < kProducerWarps) {
        ok = produce_weights<CODE, K, kGroups>(p, 0u, bars, row0, n_steps);
    } else if (warp == kTmaWarp) {
        pdl_wait_prior_grids();
        if (lane == 0) load_activations<false>(p, 0u, bars, &x_map, tok0, n_steps);
    } else if (lane == 0) {
        // ================= MMA issue =================
        RingPos px = {0, 0u}, pw = {0, 0u};
        for (int it = 0; it < n_steps && ok; ++it) {
            ok = mbar_wait(bars.full_x + 8 * px.s, px.phase, p.status) && mbar_wait(bars.full_w + 8 * pw.s, pw.phase, p.status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t xa = p.xa_addr[px.s], xb = p.xb_addr[px.s], wa = p.w_addr[pw.s];
#pragma unroll
            for (int k = 0; k < kStepCols / 16; ++k) {
                const uint64_t bdesc = umma_desc_sw128(wa + 32u * k);
                tc_mma_f16(tmem_base, umma_desc_sw128(xa + 32u * k), bdesc, kInstrDesc, (it | k) != 0);
                tc_mma_f16(tmem_base + (uint32_t)NROWS, umma_desc_sw128(xb + 32u * k), bdesc, kInstrDesc, (it | k) != 0);
            }
            tc_commit(bars.empty_x + 8 * px.s);       // each arrives when the MMAs above have read the stage
            tc_commit(bars.empty_w + 8 * pw.s);
            px.advance(p.n_xstages);
            pw.advance(p.n_wstages);
        }
        if (ok) tc_commit(bars.accum);              // arrives when every MMA has written its accumulator
    }

    if (warp < kProducerWarps) {
        if (ok) ok = mbar_wait(bars.accum, 0, p.status);
        tc_fence_after();
        drain_accumulators<NROWS>(p, 0u, tmem_base, tok0, row0, &y_map, ok);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---- two SMs on one tile (cta_group::2) ---------------------------------------------------------------------------
// A cluster of two CTAs owns 512 tokens x 256 weight rows.  CTA c (its rank in the pair) holds tokens [256c, 256c + 256)
// as two M = 128 halves, exactly like the kernel above, but decodes only HALF of the weight tile: rows [128c, 128c + 128).
// The pair's MMAs have the shape M = 256 (128 token rows from each CTA), N = 256 (128 weight rows from each CTA's shared
// memory), K = 16: every SM's tensor core still works on 128 x 256 x 16 per instruction, but reads only 4 KiB of B from
// its own shared memory (the other half comes across from the partner) and decodes, stores and looks up half as many
// weights per token.  A weight stage is 16 KiB instead of 32, which buys deeper rings.
// Roles per CTA are those of the kernel above.  Only the even CTA (the leader) issues MMAs; it needs both CTAs'
// operands, so the `full` barriers of both rings live in the leader and both CTAs signal them directly: a producer warp
// arrives (one lane, release at cluster scope, after the warp's fences) on the leader's barrier, and the TMA loads of
// either CTA count their bytes there (cta_group::2 form of the load).  Stages are handed back to both CTAs' producers,
// and the finished accumulators announced to both CTAs' epilogues, by tcgen05.commit multicast to the pair.  No TMA load
// is multicast: each CTA loads its own activations.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t rank) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}" ::"r"(bar), "r"(rank)
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
static __device__ __noinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, unsigned int *status) {
#pragma unroll 1
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (mbar_try_wait_cluster(bar, parity)) return true;
    atomicExch(status, kStatusWaitExpired);
    return false;
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {      // arrives on `bar` in BOTH CTAs of the pair
    asm volatile(
        "{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}" ::"r"(bar)
        : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// fp32 accumulate, fp16 A and B, both K-major, M = 256 (two CTAs), N = 256
constexpr uint32_t kInstrDescPair = (1u << 4) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

template <int CODE, int K>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    gemm_pair_kernel(const GemmParams p, const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap y_map) {
    constexpr int DC = GemmDecode<CODE>::kCode;
    constexpr int kHalfRows = 128;             // weight rows this CTA decodes
    constexpr int kPairRows = 256;             // weight rows of the pair's tile = accumulator columns
    constexpr uint32_t kTmemCols = 512;        // two token halves of 256 fp32 columns
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // In a cluster every CTA's shared-memory window sits at its own place in the cluster's window: shared addresses of
    // this CTA's memory carry the CTA's rank in their upper bits (rank 1 of a pair starts at 0x01000000).  The host's plan
    // holds offsets inside a CTA's window, so those bits are ORed onto every planned address that a load, store, copy or
    // barrier instruction gets; the tensor-core descriptors keep only the offset bits.
    const uint32_t s_raw = smem_addr(smem_raw);
    const uint32_t s0 = s_raw & 0x00FFFFFFu, window = s_raw & 0xFF000000u;
    if (s0 > p.bar_addr) {                     // both CTAs of a pair see the same start and leave together
        if (tid == 0) atomicExch(p.status, kStatusSmemPlan);
        return;
    }
    const uint32_t rank = cluster_ctarank();
    {
        uint32_t nrank;
        asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(nrank));
        if (nrank != 2u) {                     // not launched as a pair: nothing below may run
            if (tid == 0) atomicExch(p.status, kStatusSmemPlan);
            return;
        }
    }
    const GemmBars bars = gemm_bars(p.bar_addr | window);
    const int n_steps = (int)(p.n / kStepCols);
    const int64_t tile_row0 = (int64_t)(blockIdx.x >> 1) * kPairRows;      // first weight row of the pair's tile
    const int64_t row0 = tile_row0 + (int64_t)rank * kHalfRows;             // first weight row this CTA decodes
    const int tok0 = blockIdx.y * (2 * kTileTokens) + (int)rank * kTileTokens;

    if (tid == 0) init_ring_barriers(p, bars, 8, 2);          // four producer warps and one TMA thread per step from each CTA
    // Both CTAs of the pair must be resident, with their barriers initialised, before either touches the pair's tensor
    // memory or signals across: the paired allocation below addresses the partner SM.
    __syncthreads();
    cluster_sync_all();
    if (warp == kMmaWarp) {                     // TMEM of both SMs: the same warp of each CTA takes part
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(bars.tmem_slot), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    lut_fill<DC>(p.lut_addr | window, p.lut, p.L, p.S);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_allow_next_grid();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(bars.tmem_slot));
    bool ok = true;

    if (warp < kProducerWarps) {
        ok = produce_weights<CODE, K, 2, true>(p, window, bars, row0, n_steps);      // two groups of four warps take alternate steps
    } else if (warp == kTmaWarp) {
        pdl_wait_prior_grids();
        if (lane == 0) load_activations<true>(p, window, bars, &x_map, tok0, n_steps);
    } else if (lane == 0) {
        if (rank == 0) {
            // ================= leader: MMA issue for the pair (the partner's thread has nothing to do here) =================
            RingPos px = {0, 0u}, pw = {0, 0u};
            for (int it = 0; it < n_steps && ok; ++it) {
                ok = mbar_wait_cluster(bars.full_x + 8 * px.s, px.phase, p.status) && mbar_wait_cluster(bars.full_w + 8 * pw.s, pw.phase, p.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t xa = p.xa_addr[px.s], xb = p.xb_addr[px.s], wa = p.w_addr[pw.s];
#pragma unroll
                for (int k = 0; k < kStepCols / 16; ++k) {
                    const uint64_t bdesc = umma_desc_sw128(wa + 32u * k);
                    tc_mma_f16_pair(tmem_base, umma_desc_sw128(xa + 32u * k), bdesc, kInstrDescPair, (it | k) != 0);
                    tc_mma_f16_pair(tmem_base + (uint32_t)kPairRows, umma_desc_sw128(xb + 32u * k), bdesc, kInstrDescPair, (it | k) != 0);
                }
                tc_commit_pair(bars.empty_x + 8 * px.s);     // both CTAs get their stages back when the MMAs above have read them
                tc_commit_pair(bars.empty_w + 8 * pw.s);
                px.advance(p.n_xstages);
                pw.advance(p.n_wstages);
            }
            if (ok) tc_commit_pair(bars.accum);              // both CTAs' epilogues start when every MMA has written its accumulator
        }
    }

    // ================= epilogue (warps 0-7): this CTA's 256 tokens x the tile's 256 rows =================
    if (warp < kProducerWarps) {
        if (ok) ok = mbar_wait(bars.accum, 0, p.status);
        tc_fence_after();
        drain_accumulators<kPairRows>(p, window, tmem_base, tok0, tile_row0, &y_map, ok);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        // the pair's TMEM is released together: tell the partner this CTA is done, wait (bounded) for the same from it
        if (lane == 0) {
            mbar_arrive_remote(bars.done, rank ^ 1u);
            mbar_wait_cluster(bars.done, 0, p.status);
        }
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
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
static int launch_gemm(const GemmParams &p, const CUtensorMap &map, const CUtensorMap &ymap, size_t smem, dim3 grid, cudaStream_t stream) {
    static SmemOptIn opted;
    auto kern = gemm_kernel<CODE, K, NROWS>;
    if (int e = allow_max_smem(kern, opted)) return e;
    return launch(kern, grid, dim3(kGemmThreads), smem, stream, p, map, ymap);
}

template <int CODE, int K>
static int launch_gemm_pair(const GemmParams &p, const CUtensorMap &map, const CUtensorMap &ymap, size_t smem, dim3 grid, cudaStream_t stream) {
    static SmemOptIn opted;
    auto kern = gemm_pair_kernel<CODE, K>;
    if (int e = allow_max_smem(kern, opted)) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;      // the kernel is compiled for pairs: stated here as well
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    RPTC_CUDA(cudaLaunchKernelEx(&cfg, kern, p, map, ymap));
    return RPTC_OK;
}

template <int CODE, int K>
static int launch_gemm_rows(int n_rows, const GemmParams &p, const CUtensorMap &map, const CUtensorMap &ymap, size_t smem, dim3 grid,
                            cudaStream_t stream) {
    return n_rows == 256 ? launch_gemm<CODE, K, 256>(p, map, ymap, smem, grid, stream) : launch_gemm<CODE, K, 128>(p, map, ymap, smem, grid, stream);
}

int check_format(const rptc_format *f);   // api.cu
// RPTC_GEMM_PAIR=1 in the environment (read once per process) sends shapes that allow it to the two-SM kernel.  It is
// not the default: measured on B200 it trails the one-SM kernel on every Llama-2-7B layer shape (199 us against 156 us
// at 12288 x 4096 x 2048 tokens).  Timed with the producers and the loads taken out, the pair still needs 0.85 us per
// 64-column step (the one-SM kernel: 0.54 us), so the loss is in the paired MMA path itself, not in the decode; one
// commit per step instead of two, polling waits and direct signalling of the leader's barriers each changed nothing.
static bool g_gemm_pair = false;

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
    {
        static const bool want_pair = [] {
            const char *v = getenv("RPTC_GEMM_PAIR");
            return v && v[0] == '1';
        }();
        g_gemm_pair = want_pair;
    }
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

    // the output, [tokens][m] fp16, in boxes of 64 columns x 128 tokens (the epilogue's panels)
    CUtensorMap ymap;
    {
        const cuuint64_t ydim[2] = {(cuuint64_t)m, (cuuint64_t)tokens};
        const cuuint64_t ystride[1] = {(cuuint64_t)ld_y * 2};
        const cuuint32_t ybox[2] = {64, 128};
        r = encode(&ymap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, y, ydim, ystride, ybox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            g_last_cuda_error = (int)r;
            return RPTC_ERR_CUDA;
        }
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
    // Shared-window plan (offsets in the CTA's window; the dynamic area is expected to start at or below 0x400).  The
    // packed HASH table sits on its 32 KiB boundary; ring stages go first-fit into the space around the table.
    const uint32_t kTop = 0x38800;       // 226 KiB: the last byte any plan may touch (dynamic limit is 227 KiB)
    const uint32_t kHashAt = 0x8000;
    p.bar_addr = 0x400;
    uint32_t free_lo[2], free_hi[2];
    int n_free;
    auto reset_plan = [&] {
        if (fmt->code == RPTC_CODE_HASH) {
            p.lut_addr = kHashAt;
            free_lo[0] = 0x800, free_hi[0] = kHashAt;
            free_lo[1] = kHashAt + kHashPackedLutBytes, free_hi[1] = kTop;
            n_free = 2;
        } else {
            p.lut_addr = 0x800;
            const uint32_t lb = fmt->code == RPTC_CODE_LUT ? (2u << fmt->L) : (128u << fmt->S);
            free_lo[0] = (0x800 + lb + 1023u) & ~1023u, free_hi[0] = kTop;
            n_free = 1;
        }
    };
    auto take = [&](uint32_t bytes) -> uint32_t {
        for (int i = 0; i < n_free; ++i)
            if (free_lo[i] + bytes <= free_hi[i]) {
                const uint32_t a = free_lo[i];
                free_lo[i] += bytes;
                return a;
            }
        return 0;
    };
    // One plan: ring stages for tiles of `rows` weight rows decoded per CTA and `tile_rows` output columns per CTA, first
    // two stages of each ring, then alternately one more of each (the activation ring, the slower to refill, first); the
    // epilogue's panels (16 KiB each) are laid over the stages.  False when the tile does not fit beside this table.
    auto plan = [&](int rows, int tile_rows) -> bool {
        reset_plan();
        int xs = 0, ws = 0;
        const uint32_t w_bytes = (uint32_t)rows * 128u;
        auto add_x = [&]() -> bool {
            if (xs == kMaxGemmStages) return false;
            const uint32_t save0 = free_lo[0], save1 = free_lo[1];
            const uint32_t xa = take(kXHalfBytes), xb = take(kXHalfBytes);
            if (!xa || !xb) {
                free_lo[0] = save0, free_lo[1] = save1;
                return false;
            }
            p.xa_addr[xs] = xa, p.xb_addr[xs] = xb;
            ++xs;
            return true;
        };
        auto add_w = [&]() -> bool {
            if (ws == kMaxGemmStages) return false;
            const uint32_t w = take(w_bytes);
            if (!w) return false;
            p.w_addr[ws++] = w;
            return true;
        };
        add_w(), add_w(), add_x(), add_x();
        if (xs < 2 || ws < 2) return false;
        for (bool grew = true; grew;) {
            grew = add_x();
            if (ws < 3) grew = add_w() || grew;
        }
        uint32_t pieces[3 * kMaxGemmStages * 2];
        int np = 0;
        for (int i = 0; i < xs; ++i) pieces[np++] = p.xa_addr[i], pieces[np++] = p.xb_addr[i];
        for (int i = 0; i < ws; ++i)
            for (uint32_t off = 0; off < w_bytes; off += kXHalfBytes) pieces[np++] = p.w_addr[i] + off;
        const int need = 2 * (tile_rows / 64);
        if (np < need) return false;
        for (int i = 0; i < 8; ++i) p.out_addr[i] = i < need ? pieces[i] : 0;
        for (int s = xs; s < kMaxGemmStages; ++s) p.xa_addr[s] = p.xb_addr[s] = 0;
        for (int s = ws; s < kMaxGemmStages; ++s) p.w_addr[s] = 0;
        p.n_xstages = xs;
        p.n_wstages = ws;
        return true;
    };
    // Two SMs per tile (512 tokens x 256 rows, each CTA decoding 128 of the rows): on request, when there are tokens for
    // both CTAs and the tile fits beside the table.
    const bool pair = g_gemm_pair && tokens > kTileTokens && m % 256 == 0 && plan(128, 256);
    // Tile height of the one-SM kernel: 256 rows feed the tensor pipe about 1.35x faster per CTA-step than 128 rows, but
    // need twice the time per CTA; with few tiles the shorter ones fill more SMs.  Compare whole waves of CTAs.
    int n_rows = 128;
    if (!pair) {
        if (m % 256 == 0) {
            const int64_t tt = (tokens + kTileTokens - 1) / kTileTokens, sms = num_sms();
            const int64_t waves256 = ((m / 256) * tt + sms - 1) / sms, waves128 = ((m / 128) * tt + sms - 1) / sms;
            if (waves256 * 148 <= waves128 * 100) n_rows = 256;          // 2 / 1.35 = 1.48
        }
        if (n_rows == 256 && !plan(256, 256)) n_rows = 128;              // the wide tile does not fit beside this table
        if (n_rows == 128 && !plan(128, 128)) return RPTC_ERR_UNSUPPORTED;
    }
    const size_t smem = kTop;            // covers every planned address whatever the start of the dynamic area
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (pair) {
        const dim3 pgrid((unsigned)(2 * (m / 256)), (unsigned)((tokens + 2 * kTileTokens - 1) / (2 * kTileTokens)));
        switch (fmt->code) {
            case RPTC_CODE_LUT:
                return fmt->K == 2 ? launch_gemm_pair<RPTC_CODE_LUT, 2>(p, map, ymap, smem, pgrid, s) : launch_gemm_pair<RPTC_CODE_LUT, 4>(p, map, ymap, smem, pgrid, s);
            case RPTC_CODE_HASH:
                return launch_gemm_pair<RPTC_CODE_HASH, 2>(p, map, ymap, smem, pgrid, s);
            case RPTC_CODE_LITE:
                return fmt->K == 2 ? launch_gemm_pair<RPTC_CODE_LITE, 2>(p, map, ymap, smem, pgrid, s) : launch_gemm_pair<RPTC_CODE_LITE, 4>(p, map, ymap, smem, pgrid, s);
        }
        return RPTC_ERR_UNSUPPORTED;
    }
    const dim3 grid((unsigned)(m / n_rows), (unsigned)((tokens + kTileTokens - 1) / kTileTokens));
    switch (fmt->code) {
        case RPTC_CODE_LUT:
            return fmt->K == 2 ? launch_gemm_rows<RPTC_CODE_LUT, 2>(n_rows, p, map, ymap, smem, grid, s)
                               : launch_gemm_rows<RPTC_CODE_LUT, 4>(n_rows, p, map, ymap, smem, grid, s);
        case RPTC_CODE_HASH:
            return launch_gemm_rows<RPTC_CODE_HASH, 2>(n_rows, p, map, ymap, smem, grid, s);
        case RPTC_CODE_LITE:
            return fmt->K == 2 ? launch_gemm_rows<RPTC_CODE_LITE, 2>(n_rows, p, map, ymap, smem, grid, s)
                               : launch_gemm_rows<RPTC_CODE_LITE, 4>(n_rows, p, map, ymap, smem, grid, s);
    }
    return RPTC_ERR_UNSUPPORTED;
}
