// Fused RPTC decode + matvec for decode batches 1..8 on sm_100a.
//
// Work decomposition.  Rows are taken 32 at a time (a "row block": lane l owns row 32*rb + l) and a
// row's stream is cut into 128-bit units.  The (row block, unit) grid is flattened row-block-major
// and cut into equal contiguous ranges, one per warp of a persistent grid of one 512-thread CTA per
// SM, so that every SM gets the same number of units whatever m and n are.  In the native TILED
// layout that flattened order is the memory order: a warp's range is one linear stream of 512-byte
// units.  Lane 0 of each warp streams it into a private shared-memory ring with 1-D bulk (TMA)
// copies of two units each, completing on mbarriers, several units ahead; every lane then takes its
// own 128 bits with one conflict-free LDS.128.  The 16-bit shift-register windows are rebuilt in
// registers with funnel shifts, hashed / looked up in a bank-replicated shared-memory table, and
// multiplied into half2 accumulators that are flushed to fp32 every unit.  A warp walks along its
// rows, so the 16 bits of history a unit needs are simply the last word of the unit before it (one
// extra 32-bit load at the start of a run).  Partial row sums are added to the fp32 accumulator in
// global memory with atomics.
//
// Activations are staged once per CTA in shared memory and read back as warp-broadcast LDS.128.
// Other layouts (and the reference-quirk modes) take a plain 128-bit-load path in the same kernel.
#include "common.cuh"
#include "fwht.cuh"

namespace rptc {

#ifndef RPTC_GEMV_THREADS
#define RPTC_GEMV_THREADS 512
#endif
#ifndef RPTC_GEMV_STAGES
#define RPTC_GEMV_STAGES 3
#endif
constexpr int kGemvThreads = RPTC_GEMV_THREADS;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kStages = RPTC_GEMV_STAGES;        // ring depth per warp
constexpr int kStageUnits = 2;                   // units per bulk copy
constexpr uint32_t kUnitBytes = 512;             // 32 rows x 128 bits
constexpr uint32_t kStageBytes = kStageUnits * kUnitBytes;
constexpr uint32_t kBarBytes = 1024;             // kGemvWarps * kStages * 8 <= 1024
constexpr uint32_t kRingBytes = kGemvWarps * kStages * kStageBytes;
static_assert(kGemvWarps * kStages * 8 <= kBarBytes, "barrier area too small");
static_assert(kBarBytes + kRingBytes + 1024 <= kHashLutWindow, "ring must fit below the HASH table window");

struct GemvParams {
    const uint4 *codes;
    UnitStrides st;
    const __half *lut;
    const uint32_t *carry_in;
    const __half *x;
    int64_t ld_x;
    float *acc;
    int64_t ld_acc;
    int64_t m, n;
    int32_t n_units, seg_units;
    int32_t L, S, quirk, x_order;
    unsigned int *status;
    // activations computed in the launch (gemv_rows_kernel, MODE 1): the caller's descriptor
    rptc_gemv_input in;
    // gemv_rows_kernel, MODE 2: the gated-MLP middle that produces this layer's activations, and a range to zero
    SwigluParams sw;
    float *clear;
    int64_t clear_count;
};

// Source pair of stream pair s under the fused reference kernel's x staging (inference.cu:216-221,249).
__device__ __forceinline__ int64_t k2_legacy_pair(int64_t s, int64_t n) {
    const int64_t it = s >> 10;
    const int lane = (int)(s >> 5) & 31, o = (int)(s >> 2) & 7, j = (int)s & 3;
    const int k = (0x36251407 >> (4 * o)) & 7;       // window register met at stream position o: 7,0,4,1,5,2,6,3
    const int64_t p = ((it * 8 + k) * 4 + j) * 32 + lane;
    const int64_t q8 = n >> 3;
    return 4 * (p % q8) + p / q8;
}

// D += A B on one 16 x 8 x 16 tile: fp16 operands, fp32 accumulation.
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The general kernel: any layout (strided 128-bit loads straight from memory, one unit of one row block per
// step), the reference kernels' lane-0 deviations, batch 1.  The native TILED layout takes the two kernels below.
template <int CODE, int K>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const GemvParams p) {
    constexpr int WPU = 128 / K;          // weights per unit
    constexpr int PAIRS = WPU / 2;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t s0 = smem_addr(smem_raw);
    uint32_t lut_tab, xs;
    if (CODE == RPTC_CODE_HASH) {
        lut_tab = kHashLutWindow;
        xs = kHashLutWindow + kHashLutBytes;
    } else {
        lut_tab = s0 + kBarBytes;
        xs = lut_tab + lut_bytes<CODE>(p.L, p.S);
    }
    // ---- prologue: nothing here depends on the kernels before this one ----
    lut_fill<CODE>(lut_tab, p.lut, p.L, p.S);
    const Lut<CODE> lut = lut_view<CODE>(lut_tab, p.L, p.S);
    pdl_allow_next_grid();

    const uint32_t n_rb = (uint32_t)(p.m >> 5);
    const uint32_t gw = blockIdx.x * kGemvWarps + warp, GW = gridDim.x * kGemvWarps;
    bool waited_prior = false;

    for (int32_t useg0 = 0; useg0 < p.n_units; useg0 += p.seg_units) {
        const int32_t nu = min(p.seg_units, p.n_units - useg0);
        // Balanced contiguous split of the T = row blocks x units steps over the GW warps of the grid, in 32-bit
        // arithmetic: the first T % GW warps take one step more than the others.
        const uint32_t T = (uint32_t)n_rb * (uint32_t)nu;
        const uint32_t per = T / GW, extra = T - per * GW;
        const uint32_t g0 = gw * per + min(gw, extra);
        const uint32_t count = per + (gw < extra ? 1u : 0u);
        const uint32_t rb0 = count ? g0 / (uint32_t)nu : 0u;
        const int32_t gi0 = count ? (int32_t)(g0 - rb0 * (uint32_t)nu) : 0;

        int64_t frb = rb0;          // fetch cursor, one step ahead of the decode
        int32_t fgi = gi0;
        auto next_unit_ptr = [&]() -> const uint4 * {
            const uint4 *ptr = p.codes + unit_index(p.st, useg0 + fgi, (frb << 5) + lane);
            if (++fgi == nu) {
                fgi = 0;
                ++frb;
            }
            return ptr;
        };

        // ---- activations of this column segment -> shared memory ----
        if (!waited_prior) {
            pdl_wait_prior_grids();
            waited_prior = true;
        }
        if (useg0 > 0) __syncthreads();          // everyone is done with the previous segment's x
        {
            const int64_t col0 = (int64_t)useg0 * WPU;
            const int pairs = nu * PAIRS;
            for (int i = threadIdx.x; i < pairs; i += kGemvThreads) {
                int64_t src = (col0 >> 1) + i;
                if (p.x_order == RPTC_XORDER_K2_LEGACY) src = k2_legacy_pair(src, p.n);
                const uint32_t v = ld_ordered_u32(reinterpret_cast<const uint32_t *>(p.x) + src);
                asm volatile("st.shared.u32 [%0], %1;" ::"r"(xs + 4u * i), "r"(v) : "memory");
            }
        }
        __syncthreads();

        // ---- main loop over this warp's steps ----
        int64_t rb = rb0;
        int32_t gi = gi0;
        bool fresh = true;                        // the next step starts a run: fetch its history, zero the sum
        uint32_t prevw = 0;
        float facc = 0.f;
        uint4 nextv = make_uint4(0, 0, 0, 0);
        if (count > 0) nextv = ldg128_stream(next_unit_ptr());

#pragma unroll 1
        for (uint32_t k = 0; k < count; ++k) {
            const int64_t row = (rb << 5) + lane;
            const int32_t u = useg0 + gi;
            if (fresh) {
                fresh = false;
                if (u == 0)
                    prevw = p.carry_in ? __ldg(p.carry_in + row) : 0u;
                else
                    prevw = __ldg(reinterpret_cast<const uint32_t *>(p.codes + unit_index(p.st, u - 1, row)) + 3);
                facc = 0.f;
            }
            const bool last_of_block = gi == nu - 1;
            const uint4 v = nextv;
            if (k + 1 < count) nextv = ldg128_stream(next_unit_ptr());
            uint32_t halo = prevw;
            if (p.quirk != RPTC_QUIRK_NONE && (u & 31) == 0) {        // the reference kernels' lane-0 deviations
                if (p.quirk == RPTC_QUIRK_K2_LANE0_CARRY) halo = v.w;
                else if (u > 0) halo = prevw >> 16;
            }
            prevw = v.w;
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            const uint32_t xu = xs + (uint32_t)gi * (WPU * 2u);
            __half2 hacc[4];
            uint4 xv;
            decode_group<CODE, K>(w, halo, lut, [&](int pi, __half2 wp) {
                if ((pi & 3) == 0) xv = lds128(xu + 4u * pi);
                const uint32_t xq = (pi & 3) == 0 ? xv.x : (pi & 3) == 1 ? xv.y : (pi & 3) == 2 ? xv.z : xv.w;
                hacc[pi & 3] = pi < 4 ? __hmul2(wp, u32_as_half2(xq)) : __hfma2(wp, u32_as_half2(xq), hacc[pi & 3]);
            });
            const float2 f2 = __half22float2(__hadd2(__hadd2(hacc[0], hacc[1]), __hadd2(hacc[2], hacc[3])));
            facc += f2.x + f2.y;
            if (last_of_block || k + 1 == count) {
                atomicAdd(p.acc + row, facc);
                fresh = true;
            }
            if (last_of_block) {
                gi = 0;
                ++rb;
            } else {
                ++gi;
            }
        }
    }
    if (!waited_prior) pdl_wait_prior_grids();
}

// ---- batch 1-2: lane = row, products on the tensor cores -----------------------------------------------------------
// A granule is one 128-bit unit of two adjacent 32-row blocks; lane l owns rows 64*p + l and 64*p + 32 + l of block
// pair p, and a warp walks along its rows.
//
// Products.  One mma.sync m16n8k16 (fp16 in, fp32 accumulate) takes FOUR decoded pairs of a lane at once: pairs 2i and
// 2i+1 of the lane's row in block a (a0, a2) and of its row in block b (a1, a3).  Rows g and g+8 of the A tile are then
// a mix of the four lanes (g, 0..3), i.e. of four different rows of W -- which is harmless, because B separates them
// again: lane t's k slots meet the activations only in output column n = t (first activation row) and n = 4 + t
// (second), every other entry of B is zero.  D[g][4b + t] is the partial dot product of row 4g + t of block a with
// activation row b, D[g+8][4b + t] the same for block b.  The lane that supplies column n = g of B reads the
// activations when g % 4 == t (and g / 4 < BATCH) and holds zeros otherwise, so only four (eight) lanes of a warp take
// part in the shared-memory loads of x.  Against packed fp16 multiply-adds this issues a quarter of the multiply
// instructions per unit and row block, and there is no fp16 partial sum: the accumulation is fp32 throughout.
//
// Codes.  Each lane copies its own 16 bytes of a unit from global memory into a per-warp shared-memory ring with
// cp.async (the 32 rows of a unit are 512 contiguous bytes in the TILED layout: one fully coalesced request per warp),
// three granules ahead, and reads back only its own bytes: the per-thread group wait is the whole synchronisation --
// no barrier, no lane that issues copies on behalf of the others, no register or scoreboard held by a load in flight.
//
// MODE 0: activations copied from memory.  MODE 1: computed by every CTA from the previous layer's accumulator and the
// residual stream (rptc_gemv_glued).  MODE 2: the down projection of a gated MLP -- granules ordered by 256-column
// blocks first, each CTA makes the blocks of x it needs from the gate-up accumulator (rptc_gemv_swiglu).
template <int CODE, int K, int BATCH, int MODE>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_rows_kernel(const GemvParams p) {
    constexpr int WPU = 128 / K;
    constexpr int PAIRS = WPU / 2;
    constexpr int NW2 = 2 * GroupShape<K>::kWords;
    constexpr uint32_t UPB = 256 / WPU;                       // units per 256-column block (MODE 2)
    static_assert(BATCH == 1 || BATCH == 2, "eight output columns: four rows x two activation rows");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const uint32_t s0 = smem_addr(smem_raw);
    const uint32_t ring = s0 + kBarBytes + (uint32_t)warp * kStages * kStageBytes;
    uint32_t lut_tab, xs;
    if (CODE == RPTC_CODE_HASH) {
        lut_tab = kHashLutWindow;
        xs = kHashLutWindow + kHashLutBytes;
    } else {
        lut_tab = s0 + kBarBytes + kRingBytes;
        xs = lut_tab + lut_bytes<CODE>(p.L, p.S);
    }
    if (CODE == RPTC_CODE_HASH && s0 + kBarBytes + kRingBytes > kHashLutWindow) {
        if (threadIdx.x == 0) atomicExch(p.status, kStatusSmemPlan);
        return;
    }
    // ---- prologue: nothing here depends on the kernels before this one ----
    const LutPending lut_pending = lut_fill_begin<CODE>(lut_tab, p.lut, p.L, p.S);
    const Lut<CODE> lut = lut_view<CODE>(lut_tab, p.L, p.S);
    pdl_allow_next_grid();

    const uint32_t n_rb = (uint32_t)(p.m >> 5), n_rbp = (n_rb + 1) >> 1;
    const uint32_t x_batch_stride = (uint32_t)p.seg_units * WPU * 2u;
    const int64_t rb_stride = (int64_t)p.n_units << 5;        // 128-bit units between row blocks of the TILED layout
    // this lane's column of B: activation row g / 4 for the lanes with g % 4 == t, zeros for the others
    const bool feeds_x = (g & 3) == t4 && (g >> 2) < BATCH;
    // where this lane's sums end up: D[g][2t], D[g][2t+1] are rows 4g + (2t & 3) + {0, 1}, activation row t / 2
    const int out_row = 4 * g + ((2 * t4) & 3), out_batch = t4 >> 1;
    bool waited_prior = false;

    for (int32_t useg0 = 0; useg0 < p.n_units; useg0 += p.seg_units) {
        const int32_t nu = MODE == 2 ? p.n_units : min(p.seg_units, p.n_units - useg0);
        // Two-level even split of the T granules: contiguous ranges per CTA (sizes differ by at most one), then per warp
        // inside the CTA (again by at most one).  The warps that carry one granule more are thereby spread over all SMs
        // -- and over the four schedulers of each -- instead of filling the first CTAs of the grid.
        const uint32_t T = n_rbp * (uint32_t)nu;
        const uint32_t cta_per = T / gridDim.x, cta_extra = T - cta_per * gridDim.x;
        const uint32_t cta_g0 = blockIdx.x * cta_per + min((uint32_t)blockIdx.x, cta_extra);
        const uint32_t cta_n = cta_per + (blockIdx.x < cta_extra ? 1u : 0u);
        const uint32_t w_per = cta_n / kGemvWarps, w_extra = cta_n - w_per * kGemvWarps;
        const uint32_t g0 = cta_g0 + (uint32_t)warp * w_per + min((uint32_t)warp, w_extra);
        const uint32_t count = w_per + ((uint32_t)warp < w_extra ? 1u : 0u);

        // ---- granule order.  MODE 0/1: pairs of row blocks outermost, units along the row.  MODE 2: 256-column
        // blocks outermost, then pairs of row blocks, then the units of the block.
        struct Cursor {
            uint32_t rbp;       // pair of row blocks
            int32_t u;          // unit within the row (MODE 2) or within the segment (MODE 0/1)
            const uint4 *ptr;   // this lane's 16 bytes of block a
        };
        const uint32_t cell = n_rbp * UPB;
        auto cursor_at = [&](uint32_t gi) {
            Cursor c;
            if (MODE == 2) {
                const uint32_t cb = gi / cell, rem = gi - cb * cell;
                c.rbp = rem / UPB;
                c.u = (int32_t)(cb * UPB + (rem - c.rbp * UPB));
            } else {
                c.rbp = gi / (uint32_t)nu;
                c.u = (int32_t)(gi - c.rbp * (uint32_t)nu);
            }
            c.ptr = p.codes + (int64_t)(2 * c.rbp) * rb_stride + ((int64_t)(useg0 + c.u) << 5) + lane;
            return c;
        };
        auto advance = [&](Cursor &c) {      // to the next granule in this kernel's order
            ++c.u;
            c.ptr += 32;
            if (MODE == 2) {
                if (((uint32_t)c.u & (UPB - 1)) == 0) {      // end of the 256-column block: same block, next pair of row blocks
                    c.u -= (int32_t)UPB;
                    if (++c.rbp == n_rbp) {
                        c.rbp = 0;
                        c.u += (int32_t)UPB;
                    }
                    c.ptr = p.codes + (int64_t)(2 * c.rbp) * rb_stride + ((int64_t)c.u << 5) + lane;
                }
            } else if (c.u == nu) {
                c.u = 0;
                ++c.rbp;
                c.ptr = p.codes + (int64_t)(2 * c.rbp) * rb_stride + ((int64_t)useg0 << 5) + lane;
            }
        };
        Cursor fc = cursor_at(count ? g0 : 0u);      // fetch cursor
        Cursor cc = fc;                              // decode cursor
        // ---- the first PF granules and the 16 stream bits in front of the first one: all of it weights, so all of it
        // can be under way before anything that depends on the grid in front
        // Each lane copies its own 16 bytes of both row blocks into the warp's ring with asynchronous copies (tracked per
        // thread in groups, one group per granule: no register, scoreboard or barrier is tied up while they travel) and
        // reads back only what it copied itself, so the group wait is all the synchronisation there is.
        uint32_t fetched = 0;
        auto fetch = [&](uint32_t slot) {
            if (fetched < count) {
                const uint32_t dst = ring + slot * kStageBytes + 16u * lane;
                cp_async16(dst, fc.ptr);
                cp_async16(dst + kUnitBytes, 2 * fc.rbp + 1 < n_rb ? fc.ptr + rb_stride : fc.ptr);      // no second block: block a again, sums dropped
                advance(fc);
                ++fetched;
            }
            cp_async_commit();      // an empty group when nothing is left keeps the count of groups in flight constant
        };
        // Before the dependency wait only the first granule is requested: a lane's copies queue up in the load/store unit,
        // and a full ring of them ahead of the activation loads would delay those -- the critical ones -- by a trip to DRAM.
        // The rest of the ring follows as soon as the activation loads are on their way (`late_prologue`).
        if (MODE == 0) fetch(0);
        bool late_pending = true;
        auto late_prologue = [&]() {
            if (!late_pending) return;
            late_pending = false;
#pragma unroll
            for (int i = MODE == 0 ? 1 : 0; i < kStages; ++i) fetch(i);
            lut_fill_end<CODE>(lut_tab, lut_pending, p.S);      // the codebook loads were issued long ago
        };
        // The 16 stream bits in front of a run's first unit (the last word of the unit before it in the same rows, or the
        // shard's carry_in at a row start) are fetched one run ahead: those of the first two runs here, before the wait.
        auto load_history = [&](const Cursor &c, uint32_t &pa, uint32_t &pb) {
            const int64_t row_a = ((int64_t)c.rbp << 6) + lane;
            const bool has_b = 2 * c.rbp + 1 < n_rb;
            if (useg0 + c.u == 0) {
                pa = p.carry_in ? __ldg(p.carry_in + row_a) : 0u;
                pb = (p.carry_in && has_b) ? __ldg(p.carry_in + row_a + 32) : 0u;
            } else {
                const uint32_t *last = reinterpret_cast<const uint32_t *>(c.ptr - 32) + 3;
                pa = __ldg(last);
                pb = has_b ? __ldg(last + 4 * rb_stride) : 0u;
            }
        };
        auto run_length = [&](const Cursor &c) -> uint32_t {      // granules from c to the end of its run
            return MODE == 2 ? UPB - ((uint32_t)c.u & (UPB - 1)) : (uint32_t)(nu - c.u);
        };
        auto run_after = [&](const Cursor &c) {                    // first granule of the run after the one c lies in
            Cursor n = c;
            if (MODE == 2) {
                n.u = (int32_t)((uint32_t)c.u & ~(UPB - 1));
                if (++n.rbp == n_rbp) {
                    n.rbp = 0;
                    n.u += (int32_t)UPB;
                }
            } else {
                n.u = 0;
                ++n.rbp;
            }
            n.ptr = p.codes + (int64_t)(2 * n.rbp) * rb_stride + ((int64_t)(useg0 + n.u) << 5) + lane;
            return n;
        };
        uint32_t prev_a = 0u, prev_b = 0u, next_prev_a = 0u, next_prev_b = 0u;
        uint32_t left_after_run = 0;          // granules of this warp behind the current run
        if (count) {
            load_history(cc, prev_a, prev_b);
            const uint32_t len = min(run_length(cc), count);
            left_after_run = count - len;
            if (left_after_run) load_history(run_after(cc), next_prev_a, next_prev_b);
        }

        // ---- activations -> shared memory ----
        if (!waited_prior) {
            pdl_wait_prior_grids();
            waited_prior = true;
        }
        if (useg0 > 0) __syncthreads();
        if (MODE == 2) {
            // column blocks of this CTA's warps together (its granules are consecutive)
            const uint32_t cb_first = cta_g0 / cell, cb_last = cta_n ? (cta_g0 + cta_n - 1) / cell : cb_first;
            if (p.clear) {
                float4 *z = reinterpret_cast<float4 *>(p.clear);
                for (int64_t i = (int64_t)blockIdx.x * kGemvThreads + threadIdx.x; 4 * i < p.clear_count; i += (int64_t)gridDim.x * kGemvThreads)
                    z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            __half *x_sm = reinterpret_cast<__half *>(smem_raw + (xs - s0));
            for (uint32_t b = cb_first + warp; b <= cb_last; b += kGemvWarps)
#pragma unroll 1
                for (int r = 0; r < BATCH; ++r)
                    swiglu_chunk(p.sw, r, (int64_t)b * 256 + 8 * lane, nullptr, false,
                                 x_sm + (size_t)r * (x_batch_stride >> 1) + (size_t)(b - cb_first) * 256 + 8 * lane, late_prologue);
            // x of unit u sits at xs + (u - cb_first * UPB) * 2 WPU: fold the offset into the base
            xs -= cb_first * UPB * (uint32_t)(WPU * 2);
        } else if (MODE == 1) {
            // one segment by construction (the host refuses wider rows)
            if (p.in.clear) {
                float4 *z = reinterpret_cast<float4 *>(p.in.clear);
                for (int64_t i = (int64_t)blockIdx.x * kGemvThreads + threadIdx.x; 4 * i < p.in.clear_count;
                     i += (int64_t)gridDim.x * kGemvThreads)
                    z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (p.n != 4096) late_prologue();      // the wide form has no hook
            float *ex = reinterpret_cast<float *>(smem_raw + (xs - s0) + BATCH * x_batch_stride);
            FinishNormParams q;
            q.acc = const_cast<float *>(p.in.acc);
            q.ld_acc = p.in.ld_acc;
            q.signs_out = static_cast<const __half *>(p.in.signs_out);
            q.scale_out = p.in.scale_out;
            q.h = const_cast<__half *>(static_cast<const __half *>(p.in.h_in));
            q.h_out = static_cast<__half *>(p.in.h_out);
            q.ld_h = p.in.ld_h;
            q.w_norm = static_cast<const __half *>(p.in.w_norm);
            q.eps = p.in.eps;
            q.signs_in = static_cast<const __half *>(p.in.signs_in);
            q.transform_in = 1;
            q.out = reinterpret_cast<__half *>(smem_raw + (xs - s0));
            q.ld_out = x_batch_stride >> 1;
            q.n = (int32_t)p.n;
            q.block = 4096;
#pragma unroll 1
            for (int b = 0; b < BATCH; ++b) {
                if (p.n == 4096)
                    finish_norm_row(q, b, ex, ex + 4096, false, blockIdx.x == 0, b == 0, late_prologue);
                else finish_norm_row_wide<2>(q, b, ex, ex + 4096, blockIdx.x == 0, b == 0);
            }
        } else {
            const int64_t col0 = (int64_t)useg0 * WPU;
            const int pairs = nu * PAIRS;
            if (p.x_order == RPTC_XORDER_NATURAL && ((p.ld_x | col0) & 7) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0) {
                const int vecs = pairs >> 2;
#pragma unroll
                for (int b = 0; b < BATCH; ++b) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(p.x + (int64_t)b * p.ld_x + col0);
                    const uint32_t dst = xs + (uint32_t)b * x_batch_stride;
                    for (int i0 = threadIdx.x; i0 < vecs; i0 += 4 * kGemvThreads) {
                        uint4 v[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            if (i0 + k * kGemvThreads < vecs) v[k] = ld_ordered_u128(src + i0 + k * kGemvThreads);
                        late_prologue();                                                       // under the loads above
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            if (i0 + k * kGemvThreads < vecs)
                                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + 16u * (i0 + k * kGemvThreads)),
                                             "r"(v[k].x), "r"(v[k].y), "r"(v[k].z), "r"(v[k].w)
                                             : "memory");
                    }
                }
            } else {
                for (int i = threadIdx.x; i < BATCH * pairs; i += kGemvThreads) {
                    const int b = i / pairs, s = i - b * pairs;
                    int64_t src = (col0 >> 1) + s;
                    if (p.x_order == RPTC_XORDER_K2_LEGACY) src = k2_legacy_pair(src, p.n);
                    const uint32_t v = ld_ordered_u32(reinterpret_cast<const uint32_t *>(p.x + (int64_t)b * p.ld_x) + src);
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(xs + (uint32_t)b * x_batch_stride + 4u * s), "r"(v) : "memory");
                }
            }
        }
        late_prologue();      // threads that loaded nothing, other paths
        __syncthreads();

        // ---- main loop: one granule per step ----
        const uint32_t x_base = xs + (uint32_t)(g >> 2) * x_batch_stride;
        float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};      // two accumulator tiles: two shorter MMA chains
        auto flush = [&](uint32_t rbp) {
            if (out_batch < BATCH) {
                const int64_t row_a = ((int64_t)rbp << 6) + out_row;
                const bool has_b = 2 * rbp + 1 < n_rb;
                float *dst = p.acc + (int64_t)out_batch * p.ld_acc + row_a;
                atomicAdd(dst, c0[0] + c1[0]);
                atomicAdd(dst + 1, c0[1] + c1[1]);
                if (has_b) {
                    atomicAdd(dst + 32, c0[2] + c1[2]);
                    atomicAdd(dst + 33, c0[3] + c1[3]);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) c0[i] = c1[i] = 0.f;
        };
        // One granule: windows, 16 (K = 2) lookups per row block, 8 MMAs; then the bookkeeping of run ends.
        uint32_t slot = 0;
        auto granule = [&](uint32_t k) {
            cp_async_wait<kStages - 1>();      // all but the kStages - 1 youngest groups have landed: this granule is here
            const uint32_t stage = ring + slot * kStageBytes + 16u * lane;
            const uint4 va = lds128(stage), vb = lds128(stage + kUnitBytes);
            uint32_t Ra[NW2], Rb[NW2];
            {
                const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
                make_windows<K>(wa, prev_a, Ra);
                make_windows<K>(wb, prev_b, Rb);
            }
            prev_a = va.w;
            prev_b = vb.w;
            fetch(slot);                       // the words are in registers: the slot takes the granule kStages ahead
            if (++slot == kStages) slot = 0;
            const uint32_t xu = x_base + (uint32_t)cc.u * (uint32_t)(WPU * 2);
            uint4 xv = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int pi = 0; pi < PAIRS; pi += 4) {
                // only the four (eight) lanes whose column of B is in use read activations; the others hold zeros
                lds128_if(xv, xu + 4u * pi, feeds_x);
                uint32_t wa[4], wb[4];
                decode_quad_bits<CODE, K>(Ra, lut, pi, wa);
                decode_quad_bits<CODE, K>(Rb, lut, pi, wb);
                mma_16816(c0, wa[0], wb[0], wa[1], wb[1], xv.x, xv.y);
                mma_16816(c1, wa[2], wb[2], wa[3], wb[3], xv.z, xv.w);
            }
            // the next granule: same rows one unit on, or (end of the row / of the column block) other rows
            const uint32_t rbp_done = cc.rbp;
            const int32_t u_done = cc.u;
            advance(cc);
            if (cc.rbp != rbp_done || cc.u != u_done + 1) {
                flush(rbp_done);
                prev_a = next_prev_a;
                prev_b = next_prev_b;
                if (k + 1 < count) {
                    const uint32_t len = min(run_length(cc), left_after_run);
                    left_after_run -= len;
                    if (left_after_run) load_history(run_after(cc), next_prev_a, next_prev_b);
                }
            } else if (k + 1 == count) {
                flush(rbp_done);
            }
        };
#pragma unroll 1
        for (uint32_t k = 0; k < count; ++k) granule(k);
        cp_async_wait<0>();                    // nothing of this segment's ring is in flight any more
        if (MODE != 0) break;      // computed activations live in one segment
    }
    if (!waited_prior) pdl_wait_prior_grids();
}

// ---- batch 4 and 8: word per lane, up to eight activation rows as the B operand -----------------------------------
// Same granules and work split as gemv_rows_kernel, with the codes brought in by bulk copies into a per-warp ring.  The
// products run on mma.sync m16n8k16 (fp16 in, fp32 accumulate) with the decoded weights as the A operand:
//  * lane (g = lane/4, t = lane%4) decodes WORD t of rows g, g+8, g+16, g+24 of the 32-row tile (the tile is
//    read as four conflict-free 32-bit loads instead of one 128-bit load per row); the 16 stream bits before a
//    word come from lane t-1 (same unit) or, for t == 0, from lane t+3's word of the unit before -- one shuffle;
//  * a word holds PW = 16/K weight pairs.  MMA i of a word takes pairs 2i, 2i+1 of rows g / g+8 as a0..a3, so
//    the k index of a product is (t, pair, element) -- a permutation of the unit's columns that the B operand
//    follows by reading the activations of columns [t*2*PW, (t+1)*2*PW) of the unit for lane t, batch row g;
//  * the accumulator fragment of a lane is rows g, g+8 x batch columns 2t, 2t+1: after a run, lanes with
//    2t < BATCH add their sums to the caller's accumulator.
// Per 64 weights a lane issues 4 word loads, 12 window instructions, 4 per pair for the lookup, 8 MMAs and 2
// activation loads; there is no fp16 partial sum, and BATCH up to 8 costs only the shared memory for x.
template <int CODE, int K, int BATCH>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_mma_kernel(const GemvParams p) {
    constexpr int WPU = 128 / K;
    constexpr int PAIRS = WPU / 2;
    constexpr int PW = 16 / K;                 // weight pairs in a 32-bit word
    constexpr uint32_t kXPad = 16;             // bytes between activation rows beyond their length: spreads rows over banks
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const uint32_t s0 = smem_addr(smem_raw);
    const uint32_t bars = s0 + (uint32_t)warp * kStages * 8u;
    const uint32_t ring = s0 + kBarBytes + (uint32_t)warp * kStages * kStageBytes;
    uint32_t lut_tab, xs;
    if (CODE == RPTC_CODE_HASH) {
        lut_tab = kHashLutWindow;
        xs = kHashLutWindow + kHashLutBytes;
    } else {
        lut_tab = s0 + kBarBytes + kRingBytes;
        xs = lut_tab + lut_bytes<CODE>(p.L, p.S);
    }
    if (CODE == RPTC_CODE_HASH && s0 + kBarBytes + kRingBytes > kHashLutWindow) {
        if (threadIdx.x == 0) atomicExch(p.status, kStatusSmemPlan);
        return;
    }
    // ---- prologue: nothing here depends on the kernels before this one ----
    const LutPending lut_pending = lut_fill_begin<CODE>(lut_tab, p.lut, p.L, p.S);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(bars + 8u * s, 1);
        mbar_fence_init();
    }
    __syncwarp();
    const Lut<CODE> lut = lut_view<CODE>(lut_tab, p.L, p.S);
    pdl_allow_next_grid();

    const uint32_t n_rb = (uint32_t)(p.m >> 5), n_rbp = (n_rb + 1) >> 1;
    const uint32_t x_batch_stride = (uint32_t)p.seg_units * WPU * 2u + kXPad;
    const int64_t rb_stride = (int64_t)p.n_units << 5;        // 128-bit units between row blocks of the TILED layout
    const int halo_src = (lane & ~3) | ((t4 + 3) & 3);
    uint32_t slot = 0, phase = 0;
    bool ok = true, waited_prior = false;

    for (int32_t useg0 = 0; useg0 < p.n_units; useg0 += p.seg_units) {
        const int32_t nu = min(p.seg_units, p.n_units - useg0);
        // two-level even split: contiguous ranges per CTA, then per warp (see gemv_rows_kernel)
        const uint32_t T = n_rbp * (uint32_t)nu;
        const uint32_t cta_per = T / gridDim.x, cta_extra = T - cta_per * gridDim.x;
        const uint32_t cta_g0 = blockIdx.x * cta_per + min((uint32_t)blockIdx.x, cta_extra);
        const uint32_t cta_n = cta_per + (blockIdx.x < cta_extra ? 1u : 0u);
        const uint32_t w_per = cta_n / kGemvWarps, w_extra = cta_n - w_per * kGemvWarps;
        const uint32_t g0 = cta_g0 + (uint32_t)warp * w_per + min((uint32_t)warp, w_extra);
        const uint32_t count = w_per + ((uint32_t)warp < w_extra ? 1u : 0u);
        const uint32_t rbp0 = count ? g0 / (uint32_t)nu : 0u;
        const int32_t u0 = count ? (int32_t)(g0 - rbp0 * (uint32_t)nu) : 0;

        // fetch cursor (lane 0)
        uint32_t frbp = rbp0;
        int32_t fu = u0;
        const uint4 *fptr = p.codes + (int64_t)(2 * rbp0) * rb_stride + ((int64_t)(useg0 + u0) << 5);
        auto issue_stage = [&](uint32_t at_slot) {
            const bool has_b = 2 * frbp + 1 < n_rb;
            const uint32_t bar = bars + 8u * at_slot, dst = ring + at_slot * kStageBytes;
            mbar_expect_tx(bar, has_b ? 2 * kUnitBytes : kUnitBytes);
            bulk_g2s(dst, fptr, kUnitBytes, bar);
            if (has_b) bulk_g2s(dst + kUnitBytes, fptr + rb_stride, kUnitBytes, bar);
            fptr += 32;
            if (++fu == nu) {
                fu = 0;
                ++frbp;
                fptr = p.codes + (int64_t)(2 * frbp) * rb_stride + ((int64_t)useg0 << 5);
            }
        };
        uint32_t to_issue = count;
        {
            const uint32_t ahead = min(count, (uint32_t)kStages);
            if (lane == 0) {
                uint32_t sl = slot;
                for (uint32_t k = 0; k < ahead; ++k) {
                    issue_stage(sl);
                    if (++sl == kStages) sl = 0;
                }
            }
            to_issue -= ahead;
        }

        // Word 3 of the unit in front of a run, rows g + 8j of both blocks: part of the weights, so the first run's are
        // fetched here, before anything that depends on the grid in front.
        auto load_history = [&](uint32_t rbpx, int32_t ug, uint32_t (&pa)[4], uint32_t (&pb)[4]) {
            const int64_t row0 = (int64_t)rbpx << 6;
            const bool has_b = 2 * rbpx + 1 < n_rb;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int64_t r = row0 + g + 8 * j;
                if (ug == 0) {
                    pa[j] = p.carry_in ? __ldg(p.carry_in + r) : 0u;
                    pb[j] = (p.carry_in && has_b) ? __ldg(p.carry_in + r + 32) : 0u;
                } else {
                    const uint32_t *last = reinterpret_cast<const uint32_t *>(p.codes + (int64_t)(2 * rbpx) * rb_stride +
                                                                               ((int64_t)(ug - 1) << 5) + (g + 8 * j)) + 3;
                    pa[j] = __ldg(last);
                    pb[j] = has_b ? __ldg(last + 4 * rb_stride) : 0u;
                }
            }
        };
        uint32_t first_pa[4] = {0u, 0u, 0u, 0u}, first_pb[4] = {0u, 0u, 0u, 0u};
        if (count) load_history(rbp0, useg0 + u0, first_pa, first_pb);

        // ---- activations of this column segment -> shared memory ----
        if (!waited_prior) {
            pdl_wait_prior_grids();
            waited_prior = true;
            // the codebook loads were issued before the wait
            lut_fill_end<CODE>(lut_tab, lut_pending, p.S);
        }
        if (useg0 > 0) __syncthreads();
        {
        const int64_t col0 = (int64_t)useg0 * WPU;
        const int pairs = nu * PAIRS;
        if (p.x_order == RPTC_XORDER_NATURAL && ((p.ld_x | col0) & 7) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0) {
            const int vecs = pairs >> 2;
#pragma unroll 1
            for (int b = 0; b < BATCH; ++b) {
                const uint4 *src = reinterpret_cast<const uint4 *>(p.x + (int64_t)b * p.ld_x + col0);
                const uint32_t dst = xs + (uint32_t)b * x_batch_stride;
                for (int i0 = threadIdx.x; i0 < vecs; i0 += 4 * kGemvThreads) {
                    uint4 v[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (i0 + k * kGemvThreads < vecs) v[k] = ld_ordered_u128(src + i0 + k * kGemvThreads);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (i0 + k * kGemvThreads < vecs)
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + 16u * (i0 + k * kGemvThreads)),
                                         "r"(v[k].x), "r"(v[k].y), "r"(v[k].z), "r"(v[k].w)
                                         : "memory");
                }
            }
        } else {
            for (int i = threadIdx.x; i < BATCH * pairs; i += kGemvThreads) {
                const int b = i / pairs, s = i - b * pairs;
                int64_t src = (col0 >> 1) + s;
                if (p.x_order == RPTC_XORDER_K2_LEGACY) src = k2_legacy_pair(src, p.n);
                const uint32_t v = ld_ordered_u32(reinterpret_cast<const uint32_t *>(p.x + (int64_t)b * p.ld_x) + src);
                asm volatile("st.shared.u32 [%0], %1;" ::"r"(xs + (uint32_t)b * x_batch_stride + 4u * s), "r"(v) : "memory");
            }
        }
        }
        __syncthreads();

        // ---- main loop: runs of consecutive units inside one pair of row blocks ----
        // this lane's activations: batch row g (any valid row when g >= BATCH: those columns of D are not used)
        const uint32_t x_lane = xs + (uint32_t)(g < BATCH ? g : 0) * x_batch_stride + (uint32_t)t4 * (PW * 4u);
        uint32_t rbp = rbp0;
        int32_t u = u0;
        uint32_t k = 0;
        while (k < count && ok) {
            const uint32_t run = min(count - k, (uint32_t)(nu - u));
            const int64_t row0 = (int64_t)rbp << 6;               // first row of block a; block b starts 32 later
            const bool has_b = 2 * rbp + 1 < n_rb;
            // word 3 of the unit before the run, rows g + 8j of both blocks (lanes t == 3 hand it to lanes t == 0)
            uint32_t pa[4], pb[4];
            if (k == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) pa[j] = first_pa[j], pb[j] = first_pb[j];
            } else {
                load_history(rbp, useg0 + u, pa, pb);
            }
            float ca[2][4], cb[2][4];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 4; ++i) ca[h][i] = cb[h][i] = 0.f;
            uint32_t xu = x_lane + (uint32_t)u * (WPU * 2u);
#pragma unroll 1
            for (uint32_t jj = 0; jj < run; ++jj) {
                ok = mbar_wait(bars + 8u * slot, phase, p.status);
                if (!ok) break;
                const uint32_t stage_base = ring + slot * kStageBytes + 4u * lane;
                uint32_t xr[PW];
                if (PW == 8) {
                    const uint4 x0 = lds128(xu), x1 = lds128(xu + 16u);
                    xr[0] = x0.x, xr[1] = x0.y, xr[2] = x0.z, xr[3] = x0.w;
                    xr[PW - 4] = x1.x, xr[PW - 3] = x1.y, xr[PW - 2] = x1.z, xr[PW - 1] = x1.w;
                } else {
                    const uint4 x0 = lds128(xu);
                    xr[0] = x0.x, xr[1] = x0.y, xr[2] = x0.z, xr[3] = x0.w;
                }
#pragma unroll
                for (int blk = 0; blk < 2; ++blk) {
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        w[j] = lds32(stage_base + (uint32_t)blk * kUnitBytes + 128u * j);      // block b absent: stale bytes, sums dropped
                    uint32_t R[4][2];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t &prev = blk == 0 ? pa[j] : pb[j];
                        const uint32_t give = t4 == 3 ? prev : w[j];
                        const uint32_t before = __shfl_sync(0xFFFFFFFFu, give, halo_src);
                        prev = w[j];
                        R[j][0] = __funnelshift_l(w[j], before, 16);
                        R[j][1] = w[j];
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
#pragma unroll
                        for (int i = 0; i < PW / 2; ++i) {
                            const uint32_t a0 = (decode_pair_bits<CODE, K>(R[2 * h], lut, 2 * i));
                            const uint32_t a1 = (decode_pair_bits<CODE, K>(R[2 * h + 1], lut, 2 * i));
                            const uint32_t a2 = (decode_pair_bits<CODE, K>(R[2 * h], lut, 2 * i + 1));
                            const uint32_t a3 = (decode_pair_bits<CODE, K>(R[2 * h + 1], lut, 2 * i + 1));
                            mma_16816(blk == 0 ? ca[h] : cb[h], a0, a1, a2, a3, xr[2 * i], xr[2 * i + 1]);
                        }
                    }
                }
                xu += WPU * 2u;
                __syncwarp();                     // every lane has taken its words: the slot can be refilled
                if (to_issue) {
                    if (lane == 0) issue_stage(slot);
                    --to_issue;
                }
                if (++slot == kStages) {
                    slot = 0;
                    phase ^= 1u;
                }
            }
            // c[h][0..1]: row g + 16h, batch columns 2t, 2t+1;  c[h][2..3]: row g + 16h + 8
            if (2 * t4 < BATCH) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int col = 2 * t4 + (e & 1);
                        if (col < BATCH) {
                            const int64_t r = row0 + g + 16 * h + 8 * (e >> 1);
                            atomicAdd(p.acc + (int64_t)col * p.ld_acc + r, ca[h][e]);
                            if (has_b) atomicAdd(p.acc + (int64_t)col * p.ld_acc + r + 32, cb[h][e]);
                        }
                    }
                }
            }
            k += run;
            u += (int32_t)run;
            if (u == nu) {
                u = 0;
                ++rbp;
            }
        }
        if (!ok) {
            // After a failed wait: give the copies still in flight a bounded chance to land before
            // the shared memory they target is released, then stop.
            for (int s = 0; s < kStages; ++s) {
                mbar_wait(bars + 8u * slot, phase, p.status);
                if (++slot == kStages) {
                    slot = 0;
                    phase ^= 1u;
                }
            }
            break;
        }
    }
    if (!waited_prior) pdl_wait_prior_grids();
}

__global__ void gemv_finish_kernel(float *__restrict__ acc, int64_t ld_acc, __half *__restrict__ y, int64_t ld_y,
                                   int64_t m, int batch, float scale, int accumulate, int clear) {
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m * batch) return;
    const int64_t b = i / m, r = i - b * m;
    float v = acc[b * ld_acc + r] * scale;
    if (accumulate) {
        // the reference accumulates in fp16: out = out + delta (inference_t.cu:170-171)
        y[b * ld_y + r] = __hadd(y[b * ld_y + r], __float2half_rn(v));
    } else {
        y[b * ld_y + r] = __float2half_rn(v);
    }
    if (clear) acc[b * ld_acc + r] = 0.f;
}

template <int CODE, int K>
static int launch_gemv(const GemvParams &p, size_t smem, cudaStream_t stream) {
    static SmemOptIn opted;
    auto kern = gemv_kernel<CODE, K>;
    if (int e = allow_max_smem(kern, opted)) return e;
    return launch(kern, dim3(num_sms()), dim3(kGemvThreads), smem, stream, p);
}

template <int CODE, int K, int BATCH>
static int launch_gemv_mma(const GemvParams &p, size_t smem, cudaStream_t stream) {
    static SmemOptIn opted;
    auto kern = gemv_mma_kernel<CODE, K, BATCH>;
    if (int e = allow_max_smem(kern, opted)) return e;
    return launch(kern, dim3(num_sms()), dim3(kGemvThreads), smem, stream, p);
}

template <int CODE, int K, int BATCH, int MODE>
static int launch_gemv_rows(const GemvParams &p, size_t smem, cudaStream_t stream) {
    static SmemOptIn opted;
    auto kern = gemv_rows_kernel<CODE, K, BATCH, MODE>;
    if (int e = allow_max_smem(kern, opted)) return e;
    return launch(kern, dim3(num_sms()), dim3(kGemvThreads), smem, stream, p);
}

template <int CODE, int K>
static int dispatch(const GemvParams &p, int batch, bool tiled, size_t smem, cudaStream_t stream) {
    if (!tiled) return batch == 1 && !p.in.h_in ? launch_gemv<CODE, K>(p, smem, stream) : RPTC_ERR_UNSUPPORTED;
    if (p.in.h_in) {
        if (batch > 2) return RPTC_ERR_UNSUPPORTED;
        return batch == 1 ? launch_gemv_rows<CODE, K, 1, 1>(p, smem, stream) : launch_gemv_rows<CODE, K, 2, 1>(p, smem, stream);
    }
    switch (batch) {
        case 1: return launch_gemv_rows<CODE, K, 1, 0>(p, smem, stream);
        case 2: return launch_gemv_rows<CODE, K, 2, 0>(p, smem, stream);
        case 4: return launch_gemv_mma<CODE, K, 4>(p, smem, stream);
        case 8: return launch_gemv_mma<CODE, K, 8>(p, smem, stream);
    }
    return RPTC_ERR_ARG;
}

// One launch for batch in {1,2,4,8}.
static int gemv_one(const void *codes, const void *lut, const uint32_t *carry_in, const __half *x, int64_t ld_x, float *acc,
                    int64_t ld_acc, int64_t m, int64_t n, int batch, int x_order, const rptc_format &f, cudaStream_t stream,
                    const rptc_gemv_input *in = nullptr) {
    const int K = f.K;
    const int wpu = 128 / K;
    GemvParams p;
    p.codes = static_cast<const uint4 *>(codes);
    p.n_units = (int32_t)(n / wpu);
    p.st = unit_strides(f.layout, m, p.n_units);
    p.lut = static_cast<const __half *>(lut);
    p.carry_in = carry_in;
    p.x = x;
    p.ld_x = ld_x;
    p.acc = acc;
    p.ld_acc = ld_acc;
    p.m = m;
    p.n = n;
    p.L = f.L;
    p.S = f.S;
    p.quirk = f.quirk;
    p.x_order = x_order;
    p.status = device_status_word();
    if (!p.status) return RPTC_ERR_CUDA;
    const bool tma = f.layout == RPTC_LAYOUT_TILED && f.quirk == RPTC_QUIRK_NONE;
    p.in = in ? *in : rptc_gemv_input{};

    // shared-memory plan (must mirror the kernel's)
    const size_t kMaxSmem = 227 * 1024 - 1024;     // leave room for the 1 KiB the system may reserve
    size_t fixed;
    if (f.code == RPTC_CODE_HASH) fixed = kHashLutWindow + kHashLutBytes;      // addresses are absolute in the window
    else fixed = kBarBytes + (tma ? kRingBytes : 0) + (f.code == RPTC_CODE_LUT ? (size_t(2) << f.L) : (size_t(128) << f.S)) + 128;
    if (fixed + 1024 > kMaxSmem) return RPTC_ERR_UNSUPPORTED;
    size_t x_budget = kMaxSmem - fixed;
    if (x_budget > 96 * 1024) x_budget = 96 * 1024;
    const size_t unit_x_bytes = size_t(batch) * wpu * 2;
    int64_t seg = (int64_t)(x_budget / unit_x_bytes);
    if (x_order == RPTC_XORDER_K2_LEGACY) seg = seg / 32 * 32;
    if (seg < 1) return RPTC_ERR_TOO_LARGE;
    if (seg > p.n_units) seg = p.n_units;
    p.seg_units = (int32_t)seg;
    size_t smem = fixed + size_t(seg) * unit_x_bytes + size_t(batch) * 16;     // the tensor-core kernel pads each row of x
    if (in) {
        if (seg != p.n_units) return RPTC_ERR_TOO_LARGE;                        // computed activations live in one segment
        smem += 4096 * sizeof(float) + 128;                                     // exchange buffer of the 4096-point transform
        if (smem > kMaxSmem) return RPTC_ERR_TOO_LARGE;
    }

    switch (f.code) {
        case RPTC_CODE_LUT:
            if (K == 2) return dispatch<RPTC_CODE_LUT, 2>(p, batch, tma, smem, stream);
            if (K == 4) return dispatch<RPTC_CODE_LUT, 4>(p, batch, tma, smem, stream);
            break;
        case RPTC_CODE_HASH:
            if (K == 2) return dispatch<RPTC_CODE_HASH, 2>(p, batch, tma, smem, stream);
            break;
        case RPTC_CODE_LITE:
            if (K == 2) return dispatch<RPTC_CODE_LITE, 2>(p, batch, tma, smem, stream);
            if (K == 4) return dispatch<RPTC_CODE_LITE, 4>(p, batch, tma, smem, stream);
            break;
    }
    return RPTC_ERR_UNSUPPORTED;
}

int check_format(const rptc_format *f);   // api.cu

}  // namespace rptc

using namespace rptc;

constexpr int kMaxGemvBatch = 64;      // rows of activations per call; more than eight run as a sequence of launches

// Every check of rptc_gemv's arguments that needs no device work, in the order the entry point reports them.
static int validate_gemv_args(const void *codes, const void *lut, const void *x, int64_t ld_x, const float *acc, int64_t ld_acc,
                              int64_t m, int64_t n, int batch, int x_order, const rptc_format *fmt) {
    if (!codes || !lut || !x || !acc || !fmt) return RPTC_ERR_ARG;
    if (int e = rptc::check_format(fmt)) return e;
    if (fmt->K != 2 && fmt->K != 4) return RPTC_ERR_UNSUPPORTED;
    if (batch < 1 || batch > kMaxGemvBatch) return RPTC_ERR_ARG;
    if (x_order != RPTC_XORDER_NATURAL && x_order != RPTC_XORDER_K2_LEGACY) return RPTC_ERR_ARG;
    if (m <= 0 || n <= 0 || (m % 32) || (n % (128 / fmt->K))) return RPTC_ERR_SHAPE;
    if (x_order == RPTC_XORDER_K2_LEGACY && (n % 2048 || fmt->K != 2)) return RPTC_ERR_SHAPE;
    if (fmt->layout == RPTC_LAYOUT_CHUNKED && (n / (128 / fmt->K)) % 32) return RPTC_ERR_SHAPE;
    if (m > (int64_t(1) << 30) || n > (int64_t(1) << 30) || (m / 32) * (n / (128 / fmt->K)) >= (int64_t(1) << 31))
        return RPTC_ERR_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(lut) & 15) ||
        (reinterpret_cast<uintptr_t>(x) & 3) || (ld_x & 1))
        return RPTC_ERR_ALIGN;
    if (ld_x < n || ld_acc < m) return RPTC_ERR_SHAPE;
    return RPTC_OK;
}

extern "C" int rptc_gemv(const void *codes, const void *lut, const uint32_t *carry_in, const void *x, int64_t ld_x,
                         float *acc, int64_t ld_acc, int64_t m, int64_t n, int batch, int x_order, const rptc_format *fmt,
                         rptc_stream_t stream) {
    if (int e = validate_gemv_args(codes, lut, x, ld_x, acc, ld_acc, m, n, batch, x_order, fmt)) return e;
    if (int e = rptc_check_device()) return e;
    // batches beyond eight, or not a power of two, run as a short sequence of launches (8 + 8, 4 + 1, ...)
    int done = 0;
    while (done < batch) {
        int b = 8;
        while (b > batch - done) b >>= 1;
        int e = gemv_one(codes, lut, carry_in, static_cast<const __half *>(x) + (int64_t)done * ld_x, ld_x,
                         acc + (int64_t)done * ld_acc, ld_acc, m, n, b, x_order, *fmt, static_cast<cudaStream_t>(stream));
        if (e) return e;
        done += b;
    }
    return RPTC_OK;
}

extern "C" int rptc_gemv_finish(float *acc, int64_t ld_acc, void *y, int64_t ld_y, int64_t m, int batch, float scale,
                                int accumulate, int clear, rptc_stream_t stream) {
    if (!acc || !y) return RPTC_ERR_ARG;
    if (m <= 0 || batch < 1 || ld_acc < m || ld_y < m) return RPTC_ERR_SHAPE;
    if (int e = rptc_check_device()) return e;
    const int64_t total = m * batch;
    return launch(gemv_finish_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                  acc, ld_acc, static_cast<__half *>(y), ld_y, m, batch, scale, accumulate, clear);
}

// ---- entry point that allocates nothing --------------------------------------------------------------
// Some hosts of this library may not call cudaMalloc where they call us: a serving process whose memory
// pool owns every byte of the device, a plugin that runs under an allocator it must not bypass, or code
// that has been told its memory footprint is frozen.  For them the fp32 accumulator of the fused matvec
// lives in this fixed array, which every GPU that loads the library holds until the process exits.
namespace rptc {
constexpr int64_t kStaticAccFloats = 262144;                      // 1 MiB: batch * m may not exceed this
static __device__ __align__(256) float g_static_acc[kStaticAccFloats];
static float *g_static_acc_ptr[kMaxDevices];                               // device address of the array, per device
}  // namespace rptc

extern "C" int rptc_gemv_f16_static(const void *codes, const void *lut, const uint32_t *carry_in, const void *x, int64_t ld_x,
                                    void *y, int64_t ld_y, int64_t m, int64_t n, int batch, int x_order, const rptc_format *fmt,
                                    rptc_stream_t stream) {
    if (!y) return RPTC_ERR_ARG;
    if (batch < 1 || batch > 8 || m <= 0) return RPTC_ERR_ARG;
    if ((int64_t)batch * m > kStaticAccFloats) return RPTC_ERR_TOO_LARGE;      // the fixed accumulator cannot hold it
    if (ld_y < m) return RPTC_ERR_SHAPE;
    // Everything that can refuse the call is checked before the shared array is touched: a rejected call must not put a
    // clearing of the array on the caller's stream (it could land in the middle of a valid call on another stream).
    // The non-null placeholder stands for the accumulator, whose address is not known yet.
    if (int e = validate_gemv_args(codes, lut, x, ld_x, reinterpret_cast<const float *>(codes), m, m, n, batch, x_order, fmt)) return e;
    if (int e = rptc_check_device()) return e;
    const int dev = current_device();
    if (dev < 0) return RPTC_ERR_ARG;
    if (!g_static_acc_ptr[dev]) {
        // Set-up, once per device, with that device current: in host code the array's name is only a handle,
        // the address a kernel can use has to be asked for.
        float *ptr = nullptr;
        RPTC_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_static_acc));
        g_static_acc_ptr[dev] = ptr;
    }
    float *acc = g_static_acc_ptr[dev];
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // every call shares the array and finds the previous call's leftovers in it: start from zero
    RPTC_CUDA(cudaMemsetAsync(acc, 0, sizeof(float) * (size_t)batch * (size_t)m, s));
    if (int e = rptc_gemv(codes, lut, carry_in, x, ld_x, acc, m, m, n, batch, x_order, fmt, stream)) return e;
    return rptc_gemv_finish(acc, m, y, ld_y, m, batch, 1.0f, 0, 0, stream);
}

extern "C" int rptc_gemv_glued(const void *codes, const void *lut, const uint32_t *carry_in, const rptc_gemv_input *in, float *acc,
                               int64_t ld_acc, int64_t m, int64_t n, int batch, const rptc_format *fmt, rptc_stream_t stream) {
    if (!codes || !lut || !in || !acc || !fmt) return RPTC_ERR_ARG;
    if (int e = check_format(fmt)) return e;
    if (fmt->K != 2 && fmt->K != 4) return RPTC_ERR_UNSUPPORTED;
    if (fmt->layout != RPTC_LAYOUT_TILED || fmt->quirk != RPTC_QUIRK_NONE || batch < 1 || batch > 2) return RPTC_ERR_UNSUPPORTED;
    if (m <= 0 || n <= 0 || (m % 32) || (n % (128 / fmt->K)) || ld_acc < m) return RPTC_ERR_SHAPE;
    if (m > (int64_t(1) << 30) || (m / 32) * (n / (128 / fmt->K)) >= (int64_t(1) << 31)) return RPTC_ERR_TOO_LARGE;
    auto misaligned = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) != 0; };
    if (misaligned(codes) || misaligned(lut) || misaligned(in->acc) || misaligned(in->signs_out) || misaligned(in->signs_in) ||
        misaligned(in->clear) || (in->ld_acc % 4) || (in->clear_count % 4))
        return RPTC_ERR_ALIGN;
    if (in->clear_count < 0 || (in->clear_count && !in->clear)) return RPTC_ERR_ARG;
    if (n != 4096 && n != 8192) return RPTC_ERR_UNSUPPORTED;                    // one or two 4096-point blocks, eight values a thread each
    if (!in->h_in || !in->h_out || in->h_in == in->h_out || !in->w_norm) return RPTC_ERR_ARG;
    if (in->ld_h < n || (in->acc && in->ld_acc < n)) return RPTC_ERR_SHAPE;
    if (misaligned(in->h_in) || misaligned(in->h_out) || misaligned(in->w_norm) || (in->ld_h % 8)) return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    return gemv_one(codes, lut, carry_in, nullptr, 0, acc, ld_acc, m, n, batch, RPTC_XORDER_NATURAL, *fmt,
                    static_cast<cudaStream_t>(stream), in);
}

extern "C" int rptc_gemv_swiglu(const void *codes, const void *lut, const uint32_t *carry_in, const float *prev_acc, int64_t ld_prev,
                                const void *signs_out, float scale_out, const void *signs_in, int block, float *acc, int64_t ld_acc,
                                int64_t m, int64_t n, int batch, const rptc_format *fmt, float *clear, int64_t clear_count,
                                rptc_stream_t stream) {
    if (!codes || !lut || !prev_acc || !acc || !fmt) return RPTC_ERR_ARG;
    if (int e = check_format(fmt)) return e;
    if (fmt->K != 2 && fmt->K != 4) return RPTC_ERR_UNSUPPORTED;
    if (fmt->layout != RPTC_LAYOUT_TILED || fmt->quirk != RPTC_QUIRK_NONE || batch < 1 || batch > 2) return RPTC_ERR_UNSUPPORTED;
    if (block < 8 || block > 256 || (block & (block - 1))) return RPTC_ERR_UNSUPPORTED;
    if (m <= 0 || n <= 0 || (m % 32) || (n % 256) || ld_acc < m || ld_prev < 2 * n) return RPTC_ERR_SHAPE;
    if (m > (int64_t(1) << 30) || (m / 32) * (n / (128 / fmt->K)) >= (int64_t(1) << 31)) return RPTC_ERR_TOO_LARGE;
    auto misaligned = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) != 0; };
    if (misaligned(codes) || misaligned(lut) || misaligned(prev_acc) || misaligned(signs_out) || misaligned(signs_in) || misaligned(clear) ||
        (ld_prev % 4) || (clear_count % 4))
        return RPTC_ERR_ALIGN;
    if (clear_count < 0 || (clear_count && !clear)) return RPTC_ERR_ARG;
    if (int e = rptc_check_device()) return e;
    const int K = fmt->K, wpu = 128 / K;
    GemvParams p{};
    p.codes = static_cast<const uint4 *>(codes);
    p.n_units = (int32_t)(n / wpu);
    p.st = unit_strides(fmt->layout, m, p.n_units);
    p.lut = static_cast<const __half *>(lut);
    p.carry_in = carry_in;
    p.acc = acc;
    p.ld_acc = ld_acc;
    p.m = m;
    p.n = n;
    p.L = fmt->L;
    p.S = fmt->S;
    p.quirk = fmt->quirk;
    p.x_order = RPTC_XORDER_NATURAL;
    p.status = device_status_word();
    if (!p.status) return RPTC_ERR_CUDA;
    float norm = 1.f;
    for (int b = block; b > 1; b >>= 2) norm *= (b >= 4) ? 0.5f : 0.70710678118654752f;
    p.sw.acc = const_cast<float *>(prev_acc);
    p.sw.in16 = nullptr;
    p.sw.ld_acc = ld_prev;
    p.sw.out = nullptr;
    p.sw.ld_out = 0;
    p.sw.signs_out = static_cast<const __half *>(signs_out);
    p.sw.signs_in = static_cast<const __half *>(signs_in);
    p.sw.n = n;
    p.sw.block = block;
    p.sw.chunk = 256;
    p.sw.clear = 0;
    p.sw.scale_out = scale_out * norm;
    p.sw.scale_in = norm;
    p.clear = clear;
    p.clear_count = clear_count;
    // the most 256-column blocks one CTA's granules can touch
    const int64_t upb = 256 / wpu, n_rbp = (m / 32 + 1) / 2, cell = n_rbp * upb;
    const int64_t T = n_rbp * p.n_units;
    const int64_t cta_granules = T / num_sms() + 1;
    int64_t max_blocks = (cta_granules + cell - 2) / cell + 1;
    if (max_blocks > n / 256) max_blocks = n / 256;
    p.seg_units = (int32_t)(max_blocks * upb);
    const size_t kMaxSmem = 227 * 1024 - 1024;
    size_t fixed;
    if (fmt->code == RPTC_CODE_HASH) fixed = kHashLutWindow + kHashLutBytes;
    else fixed = kBarBytes + kRingBytes + (fmt->code == RPTC_CODE_LUT ? (size_t(2) << fmt->L) : (size_t(128) << fmt->S)) + 128;
    const size_t smem = fixed + (size_t)batch * max_blocks * 512;
    if (smem > kMaxSmem) return RPTC_ERR_TOO_LARGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (fmt->code) {
        case RPTC_CODE_LUT:
            if (K == 2) return batch == 1 ? launch_gemv_rows<RPTC_CODE_LUT, 2, 1, 2>(p, smem, s) : launch_gemv_rows<RPTC_CODE_LUT, 2, 2, 2>(p, smem, s);
            return batch == 1 ? launch_gemv_rows<RPTC_CODE_LUT, 4, 1, 2>(p, smem, s) : launch_gemv_rows<RPTC_CODE_LUT, 4, 2, 2>(p, smem, s);
        case RPTC_CODE_HASH:
            if (K == 2) return batch == 1 ? launch_gemv_rows<RPTC_CODE_HASH, 2, 1, 2>(p, smem, s) : launch_gemv_rows<RPTC_CODE_HASH, 2, 2, 2>(p, smem, s);
            break;
        case RPTC_CODE_LITE:
            if (K == 2) return batch == 1 ? launch_gemv_rows<RPTC_CODE_LITE, 2, 1, 2>(p, smem, s) : launch_gemv_rows<RPTC_CODE_LITE, 2, 2, 2>(p, smem, s);
            return batch == 1 ? launch_gemv_rows<RPTC_CODE_LITE, 4, 1, 2>(p, smem, s) : launch_gemv_rows<RPTC_CODE_LITE, 4, 2, 2>(p, smem, s);
    }
    return RPTC_ERR_UNSUPPORTED;
}
