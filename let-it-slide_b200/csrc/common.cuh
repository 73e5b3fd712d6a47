// Shared device/host helpers for the sm_100a RPTC kernels: status plumbing, bounded mbarrier waits,
// 1-D bulk (TMA) copies, and the unit decoder every kernel is built around.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rptc_b200.h"

namespace rptc {

constexpr int kNumSMsFallback = 148;
constexpr uint32_t kSpinLimit = 1u << 22;   // bounded wait: try_wait attempts before a kernel gives up

// ---- host side -------------------------------------------------------------------------------
extern thread_local int g_last_cuda_error;
int cuda_fail(cudaError_t e);                 // records e, returns RPTC_ERR_CUDA
int num_sms();                                // SM count of the current device (cached per device)
int current_device();                         // index of the current device, or -1 (beyond kMaxDevices, or no device)
bool pdl_enabled();                           // the calling thread's rptc_set_pdl setting
unsigned int *device_status_word();           // device address of the status word (per device)
constexpr int kMaxDevices = 64;

// What a kernel leaves in the device status word (rptc_device_status maps them to rptc_status values).
constexpr unsigned int kStatusWaitExpired = 1u;      // a bounded wait on an own copy or on a peer ran out
constexpr unsigned int kStatusSmemPlan = 2u;         // the kernel's shared-memory layout does not fit where it was placed
constexpr unsigned int kStatusMailboxExpired = 3u;   // the host never posted the step's token ids
constexpr unsigned int kStatusPosition = 4u;         // a sequence position outside [0, max_pos): the access was skipped

#define RPTC_CUDA(call)                                      \
    do {                                                     \
        cudaError_t e__ = (call);                            \
        if (e__ != cudaSuccess) return ::rptc::cuda_fail(e__); \
    } while (0)

// The opt-in to more than 48 KiB of dynamic shared memory is an attribute of a kernel ON ONE DEVICE: it is set the
// first time a kernel is launched on each device of the process, and remembered per device.
struct SmemOptIn {
    bool done[kMaxDevices] = {};
};
template <typename Kernel>
inline int allow_max_smem(Kernel kern, SmemOptIn &seen) {
    const int dev = current_device();
    if (dev < 0) return cuda_fail(cudaErrorInvalidDevice);
    if (!seen.done[dev]) {
        RPTC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        seen.done[dev] = true;
    }
    return RPTC_OK;
}

// Launches `kernel` with or without the programmatic-dependent-launch attribute.
template <typename... KArgs, typename... Args>
inline int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    RPTC_CUDA(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
    return RPTC_OK;
}

// ---- device side -----------------------------------------------------------------------------
#ifdef __CUDACC__

// Programmatic dependent launch: both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait_prior_grids() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_allow_next_grid() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Used right after pdl_wait_prior_grids() on a pointer to data that a prior grid writes: the pointer's value becomes
// opaque to the compiler, so no load through it -- not even a read-only-path load through a const __restrict__
// kernel parameter, which a memory clobber alone does not pin -- can be scheduled ahead of the wait.
template <typename T>
__device__ __forceinline__ T *after_wait(T *p) {
    asm volatile("" : "+l"(p)::"memory");
    return p;
}

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (after raising the device status word) when the limit runs out, so
// that the caller can stop issuing work, drain what is in flight and return.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, unsigned int *status) {
#pragma unroll 1
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(status, kStatusWaitExpired);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned int *status) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, status);
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
// Both addresses and the size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// Ampere-style asynchronous copy of 16 bytes global -> shared, bypassing L1; completion is tracked per thread in groups.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {      // until at most N of this thread's groups are still in flight
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// 16 bytes from shared memory into `v` where `take` is set; elsewhere `v` keeps what it held.  One predicated load,
// no branch (a conditional around a volatile load is compiled as a branch with its reconvergence bookkeeping).
__device__ __forceinline__ void lds128_if(uint4 &v, uint32_t addr, bool take) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.u32 p, %5, 0;\n\t"
        "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "r"(addr), "r"((uint32_t)take));
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// HASH-table lookup: the table's window address is a literal folded into the load's address field.
__device__ __forceinline__ uint32_t lds32_hash(uint32_t offset) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1 + 65536];" : "=r"(v) : "r"(offset));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 ldg128_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// Loads of data that a prior grid writes.  Volatile asm with a memory clobber: they stay behind griddepcontrol.wait,
// whereas the compiler may hoist a plain (or __ldg) load through a const __restrict__ pointer above the wait.
__device__ __forceinline__ uint4 ld_ordered_u128(const void *p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint2 ld_ordered_u64(const void *p) {
    uint2 v;
    asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_ordered_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// (a & mask) | c as ONE three-input logic instruction (the compiler does not always fuse the pair).
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(c));
    return d;
}
__device__ __forceinline__ __half2 u32_as_half2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
__device__ __forceinline__ uint32_t half2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }

// ---- packed-code addressing -------------------------------------------------------------------
// Index (in 128-bit units) of unit u of row r:
//   (u >> 5) * hi + (u & 31) * lo + (r >> 5) * rb + (r & 31) * row.
struct UnitStrides {
    int64_t hi, lo, rb, row;
};
__host__ __device__ inline UnitStrides unit_strides(int layout, int64_t m, int64_t n_units) {
    switch (layout) {
        case RPTC_LAYOUT_ROWMAJOR: return {32, 1, 32 * n_units, n_units};
        case RPTC_LAYOUT_CHUNKED: return {32 * m, 1, 32 * 32, 32};
        case RPTC_LAYOUT_UNITMAJOR: return {32 * m, m, 32, 1};
        default: return {32 * 32, 32, 32 * n_units, 1};     // TILED
    }
}
__device__ __forceinline__ int64_t unit_index(const UnitStrides &s, int64_t u, int64_t r) {
    return (u >> 5) * s.hi + (u & 31) * s.lo + (r >> 5) * s.rb + (r & 31) * s.row;
}

// ---- shared-memory lookup tables ---------------------------------------------------------------
// LUT code   : fp16 [2^L], flat.
// HASH code  : 256 rows of 256 bytes; row e (= bits 8..15 of the hash) holds, at byte 4*lane, the
//              fp16 pair of entry e & (2^S-1) with the low half's sign already set to bit 7 of e
//              (which is bit 15 of the hash).  The table must start on a 64 KiB boundary of the shared
//              window so that (hash & 0xFF00) | 4*lane is the whole address computation.
// LITE code  : 2^S rows of 128 bytes, the pair of entry e at byte 4*lane of row e.
// HASH code, packed (kCodeHashPacked; a table layout, not a fourth code): the same 256 rows at 128 bytes each, on a
//              32 KiB boundary; the address is ((hash >> 1) & 0x7F80) | table | 4*lane, one shift more per lookup.
constexpr int kCodeHashPacked = 3;
constexpr uint32_t kHashPackedLutBytes = 32768;
constexpr uint32_t kHashLutBytes = 65536;
constexpr uint32_t kHashLutWindow = 0x10000;   // shared-window address the HASH table is placed at (literal in lds32_hash)
static_assert(kHashLutWindow == 65536, "lds32_hash spells this address out");

template <int CODE>
struct Lut {
    uint32_t base;   // LUT: table address.  HASH: 4*lane (the window address is a literal in the load).  LITE: table address + 4*lane.
    uint32_t mask;   // LUT: 2^L-1.  LITE: 2^S-1.
    uint32_t shift;  // LITE: L-S.
};

template <int CODE>
__device__ __forceinline__ uint32_t lut_bytes(int L, int S) {
    if (CODE == RPTC_CODE_LUT) return 2u << L;
    if (CODE == RPTC_CODE_HASH) return kHashLutBytes;
    if (CODE == kCodeHashPacked) return kHashPackedLutBytes;
    return 128u << S;
}

// Fills the table from the global codebook.  All threads of the CTA take part; the caller
// synchronises afterwards.  Global loads are issued in independent batches (one coalesced load
// per warp feeding up to 32 shared-memory rows through shuffles) so that the prologue costs about
// one L2 round trip rather than one per row.
template <int CODE>
__device__ __forceinline__ void lut_fill(uint32_t table, const __half *__restrict__ g, int L, int S) {
    const int tid = threadIdx.x, nt = blockDim.x;
    if (CODE == RPTC_CODE_LUT) {
        const uint4 *src = reinterpret_cast<const uint4 *>(g);
        const int total = (1 << L) / 8;
        for (int i0 = tid; i0 < total; i0 += 4 * nt) {
            uint4 v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (i0 + k * nt < total) v[k] = __ldg(src + i0 + k * nt);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (i0 + k * nt < total)
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(table + 16u * (i0 + k * nt)), "r"(v[k].x),
                                 "r"(v[k].y), "r"(v[k].z), "r"(v[k].w)
                                 : "memory");
        }
    } else {
        // A table row is 32 copies of one 4-byte pair (one per bank): eight 128-bit stores.  Thread i takes
        // part i & 7 of row i >> 3, four rows in flight per thread.
        const uint32_t *src = reinterpret_cast<const uint32_t *>(g);
        constexpr bool kHash = CODE == RPTC_CODE_HASH || CODE == kCodeHashPacked;
        const int rows = kHash ? 256 : (1 << S);
        const uint32_t row_bytes = (CODE == RPTC_CODE_HASH) ? 256u : 128u;
        const int smask = (1 << S) - 1;
        const int total = rows * 8;
        for (int i0 = tid; i0 < total; i0 += 4 * nt) {
            uint32_t v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = i0 + k * nt;
                if (i < total) v[k] = __ldg(src + ((i >> 3) & smask));
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = i0 + k * nt;
                if (i < total) {
                    const int e = i >> 3;
                    uint32_t x = v[k];
                    if (kHash) x = (x & 0xFFFF7FFFu) | ((uint32_t)(e >> 7) << 15);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(table + row_bytes * e + 16u * (i & 7)), "r"(x) : "memory");
                }
            }
        }
    }
}

// The same fill in two steps, for kernels that have something to wait for in between (the table's trip through L2
// then overlaps the wait): `begin` issues the codebook loads and `end` writes the rows.  Only the one-pass case (HASH,
// or LITE with at most four rows per thread) is split; anything else is filled completely by `begin`.
struct LutPending {
    uint32_t v[4];
    bool deferred;
};
template <int CODE>
__device__ __forceinline__ LutPending lut_fill_begin(uint32_t table, const __half *__restrict__ g, int L, int S) {
    LutPending pend;
    const int rows = (CODE == RPTC_CODE_HASH) ? 256 : (1 << S);
    pend.deferred = CODE != RPTC_CODE_LUT && rows * 8 <= 4 * (int)blockDim.x;
    if (!pend.deferred) {
        lut_fill<CODE>(table, g, L, S);
        return pend;
    }
    const int smask = (1 << S) - 1;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        pend.v[k] = 0u;
        if (i < rows * 8)      // volatile: stays in front of the wait that follows
            asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(pend.v[k]) : "l"(reinterpret_cast<const uint32_t *>(g) + ((i >> 3) & smask)));
    }
    return pend;
}
template <int CODE>
__device__ __forceinline__ void lut_fill_end(uint32_t table, const LutPending &pend, int S) {
    if (!pend.deferred) return;
    const int rows = (CODE == RPTC_CODE_HASH) ? 256 : (1 << S);
    const uint32_t row_bytes = (CODE == RPTC_CODE_HASH) ? 256u : 128u;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < rows * 8) {
            const int e = i >> 3;
            uint32_t x = pend.v[k];
            if (CODE == RPTC_CODE_HASH) x = (x & 0xFFFF7FFFu) | ((uint32_t)(e >> 7) << 15);
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(table + row_bytes * e + 16u * (i & 7)), "r"(x) : "memory");
        }
    }
}

template <int CODE>
__device__ __forceinline__ Lut<CODE> lut_view(uint32_t table, int L, int S) {
    const uint32_t lane4 = 4u * (threadIdx.x & 31);
    Lut<CODE> v;
    if (CODE == RPTC_CODE_LUT) {
        v.base = table;
        v.mask = (1u << L) - 1u;
        v.shift = 0;
    } else if (CODE == RPTC_CODE_HASH) {
        v.base = lane4;
        v.mask = 0;
        v.shift = 0;
    } else {
        v.base = table + lane4;
        v.mask = (1u << S) - 1u;
        v.shift = (uint32_t)(L - S);
    }
    return v;
}

// ---- the unit decoder --------------------------------------------------------------------------
// A "group" is P consecutive 128-bit units of one row (P = 3 when K = 3 so that a group holds a whole
// number of weights, else 1).  decode_group turns the group's words plus the 16 stream bits before
// it (`halo`, low half) into fp16 weight pairs and hands pair p (columns 2p, 2p+1 of the group) to
// emit(p, pair).  Every weight is a pure function of the 16-bit window ending at its last bit, so
// nothing here is sequential: window registers R[o] cover stream bits [16o-16, 16o+16) of the group
// and a weight ending at bit e reads (R[(e-1)>>4] >> (16*((e-1)>>4)+16-e)) & 0xFFFF.
template <int K>
struct GroupShape {
    static constexpr int P = (K == 3) ? 3 : 1;          // units per group
    static constexpr int kWords = 4 * P;
    static constexpr int kWeights = 128 * P / K;        // 64, 128, 32
    static constexpr int kPairs = kWeights / 2;
};

// Window registers of a group: R[o] covers stream bits [16o-16, 16o+16) of the group.
template <int K>
__device__ __forceinline__ void make_windows(const uint32_t (&w)[GroupShape<K>::kWords], uint32_t halo,
                                             uint32_t (&R)[2 * GroupShape<K>::kWords]) {
    constexpr int NW = GroupShape<K>::kWords;
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        R[2 * i] = __funnelshift_l(w[i], i == 0 ? halo : w[i - 1], 16);
        R[2 * i + 1] = w[i];
    }
}

// Weight pair p (columns 2p, 2p+1) of a group from its window registers.  `p` must be a constant after unrolling.
// The registers may cover any whole number of words (a group, or a single word with the word before it).
template <int CODE, int K, int N>
__device__ __forceinline__ uint32_t decode_pair_bits(const uint32_t (&R)[N], const Lut<CODE> &lut, int p) {
    if (CODE == RPTC_CODE_LUT) {
        uint32_t h[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int e = K * (2 * p + q + 1);
            const int o = (e - 1) >> 4;
            const int sh = 16 * (o + 1) - e;
            const uint32_t state = (R[o] >> sh) & lut.mask;
            h[q] = lds16(lut.base + 2u * state);
        }
        return h[0] | (h[1] << 16);
    } else {
        constexpr int BPS = 2 * K;   // bits per step
        const int e = BPS * (p + 1);
        const int o = (e - 1) >> 4;
        const int sh = 16 * (o + 1) - e;
        const uint32_t t = R[o] >> sh;
        if (CODE == RPTC_CODE_HASH) {
            const uint32_t h = t * t + t;
            return lds32_hash(and_or(h, 0xFF00u, lut.base));
        } else if (CODE == kCodeHashPacked) {
            const uint32_t h = t * t + t;
            return lds32(and_or(h >> 1, 0x7F80u, lut.base));
        } else {
            // Bits above the state width never reach the entry index (rptc_lite.py:12-16 uses bits
            // [0,S) and [L-S,L) of the product only), so the raw window needs no masking.
            uint32_t h = t * (2u * t + 1u);
            h ^= h >> lut.shift;
            return lds32(lut.base + ((h & lut.mask) << 7));
        }
    }
}
// Four consecutive pairs p0 .. p0+3 at once, written stage by stage (all windows, then all hashes, then all addresses, then all
// loads) so that four independent dependency chains are in flight instead of one.
template <int CODE, int K, int N>
__device__ __forceinline__ void decode_quad_bits(const uint32_t (&R)[N], const Lut<CODE> &lut, int p0, uint32_t (&out)[4]) {
    if (CODE == RPTC_CODE_HASH) {
        uint32_t t[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = 2 * K * (p0 + i + 1);
            const int o = (e - 1) >> 4;
            const int sh = 16 * (o + 1) - e;
            t[i] = R[o] >> sh;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) t[i] = t[i] * t[i] + t[i];
#pragma unroll
        for (int i = 0; i < 4; ++i) t[i] = and_or(t[i], 0xFF00u, lut.base);
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = lds32_hash(t[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = decode_pair_bits<CODE, K>(R, lut, p0 + i);
    }
}
// The same as an fp16 pair (low half = column 2p).
template <int CODE, int K, int N>
__device__ __forceinline__ __half2 decode_pair(const uint32_t (&R)[N], const Lut<CODE> &lut, int p) {
    return u32_as_half2(decode_pair_bits<CODE, K>(R, lut, p));
}

template <int CODE, int K, typename Emit>
__device__ __forceinline__ void decode_group(const uint32_t (&w)[GroupShape<K>::kWords], uint32_t halo,
                                             const Lut<CODE> &lut, Emit &&emit) {
    uint32_t R[2 * GroupShape<K>::kWords];
    make_windows<K>(w, halo, R);
#pragma unroll
    for (int p = 0; p < GroupShape<K>::kPairs; ++p) emit(p, decode_pair<CODE, K>(R, lut, p));
}

#endif  // __CUDACC__
}  // namespace rptc
