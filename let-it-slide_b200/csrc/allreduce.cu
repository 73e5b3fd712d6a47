// Output side of a row-parallel (tensor-parallel) quantised layer fused with its all-reduce and the
// residual add, as ONE kernel over NVLink peer memory:
//     h += sum over ranks r of ( s_out * H(acc_r) * scale )
// Every rank transforms its fp32 partial accumulator and stores the fp16 result straight into a slot of EVERY rank's
// exchange buffer with plain peer stores (no multimem, no NCCL).  The flag travels WITH the data: each 32-bit word of
// payload is stored together with the 32-bit epoch as one 64-bit store, which arrives whole or not at all, so the
// receiver simply polls its own buffer until every word it needs carries the current epoch -- no fence, no second
// round trip for a separate flag.  Decode messages are tiny (16 KiB at hidden 8192, 32 KiB in this form), so the cost
// is one NVLink one-way trip instead of a collective launch.  The partials are added in rank order (all ranks compute
// bit-identical sums) onto the residual stream.  Buffers alternate by epoch parity (a rank can be at most one exchange
// ahead of its peers); epochs are kept in device memory per CTA, which makes the kernel replayable from a CUDA graph.
// A wait that runs out raises the device status word and the kernel returns; nothing hangs.
#include "common.cuh"
#include "fwht.cuh"

namespace rptc {

constexpr int kMaxPeers = 8;

struct PeerFinishParams {
    float *acc;                   // fp32 [rows][ld_acc] local partial (cleared)
    int64_t ld_acc;
    const __half *signs_out;
    float scale;
    __half *h;                    // fp16 [rows][ld_h] residual stream, updated in place
    int64_t ld_h;
    uint64_t *data[kMaxPeers];    // every rank's exchange buffer: [2 parities][world][rows * n / 2] x (payload word, epoch)
    uint32_t *epochs;             // local: [n_ctas]
    int32_t rank, world, n, block, chunk, rows;
    unsigned long long timeout_ns;
    unsigned int *status;
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Two (payload, epoch) words to a peer; each 64-bit half is single-copy atomic.
__device__ __forceinline__ void st_pair_sys(uint64_t *p, uint64_t a, uint64_t b) {
    asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_pair_sys(const uint64_t *p, uint64_t &a, uint64_t &b) {
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

__global__ void __launch_bounds__(512) peer_finish_kernel(const PeerFinishParams p) {
    __shared__ __align__(16) float ex[4096];
    __shared__ int timed_out;
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    const int t = threadIdx.x, T = blockDim.x;
    const int64_t row = blockIdx.y;
    const int col = blockIdx.x * p.chunk + 8 * t;
    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    if (t == 0) timed_out = 0;
    // ---- this rank's partial: s_out * H(acc) * scale, rounded to fp16 ----
    float v[8];
    {
        float *src = p.acc + row * p.ld_acc + col;
        const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
        *reinterpret_cast<float4 *>(src) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4 *>(src + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    uint4 sraw = make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);
    if (p.signs_out) sraw = *reinterpret_cast<const uint4 *>(p.signs_out + col);
    const uint4 hraw = *reinterpret_cast<const uint4 *>(p.h + row * p.ld_h + col);
    const uint32_t epoch = p.epochs[cta] + 1u;
    fwht8(v, p.block, ex);
    const float sc = p.scale * rsqrtf((float)p.block);
    uint32_t mine[4];
    {
        const uint32_t sw[4] = {sraw.x, sraw.y, sraw.z, sraw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 s2 = __half22float2(u32_as_half2(sw[i]));
            mine[i] = half2_as_u32(__floats2half2_rn(v[2 * i] * sc * s2.x, v[2 * i + 1] * sc * s2.y));
        }
    }
    // ---- publish to every other rank: thread t's four words as two 16-byte stores, [j][t] inside the CTA's piece so
    // that a warp's stores are contiguous ----
    const int64_t slot = (int64_t)p.rows * p.n / 2;                                   // 64-bit words per (parity, source rank)
    const int64_t piece = (row * p.n + (int64_t)blockIdx.x * p.chunk) / 2;            // this CTA's first word inside a slot
    const int64_t mine_at = ((int64_t)(epoch & 1u) * p.world + p.rank) * slot + piece;
    const uint64_t tag = (uint64_t)epoch << 32;
    for (int r = 0; r < p.world; ++r) {
        if (r == p.rank) continue;
        uint64_t *dst = p.data[r] + mine_at;
        st_pair_sys(dst + 2 * t, tag | mine[0], tag | mine[1]);
        st_pair_sys(dst + 2 * (T + t), tag | mine[2], tag | mine[3]);
    }
    // ---- collect: poll this rank's own buffer until every word carries this epoch (bounded), summing in rank order ----
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bool ok = true;
    const unsigned long long t0 = global_ns();
    for (int r = 0; r < p.world; ++r) {
        uint32_t q[4];
        if (r == p.rank) {
#pragma unroll
            for (int i = 0; i < 4; ++i) q[i] = mine[i];
        } else if (ok) {
            const uint64_t *src = p.data[p.rank] + ((int64_t)(epoch & 1u) * p.world + r) * slot + piece;
            uint64_t w0, w1, w2, w3;
            uint32_t spins = 0;
            for (;;) {
                ld_pair_sys(src + 2 * t, w0, w1);
                ld_pair_sys(src + 2 * (T + t), w2, w3);
                if ((uint32_t)(w0 >> 32) == epoch && (uint32_t)(w1 >> 32) == epoch && (uint32_t)(w2 >> 32) == epoch &&
                    (uint32_t)(w3 >> 32) == epoch)
                    break;
                if ((++spins & 63u) == 0 && global_ns() - t0 > p.timeout_ns) {
                    ok = false;
                    break;
                }
            }
            q[0] = (uint32_t)w0, q[1] = (uint32_t)w1, q[2] = (uint32_t)w2, q[3] = (uint32_t)w3;
        }
        if (!ok) break;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f2 = __half22float2(u32_as_half2(q[i]));
            sum[2 * i] += f2.x, sum[2 * i + 1] += f2.y;
        }
    }
    if (!ok) {
        timed_out = 1;
        atomicExch(p.status, kStatusWaitExpired);
    }
    __syncthreads();
    if (t == 0) p.epochs[cta] = epoch;
    if (timed_out) return;      // the whole CTA leaves h untouched for the piece it could not finish
    // ---- add the residual ----
    uint32_t o[4];
    {
        const uint32_t hw[4] = {hraw.x, hraw.y, hraw.z, hraw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // the reduced layer output is an fp16 tensor; add it to the residual as the unfused path does
            const float2 res = __half22float2(u32_as_half2(hw[i]));
            const float2 red = __half22float2(__floats2half2_rn(sum[2 * i], sum[2 * i + 1]));
            o[i] = half2_as_u32(__floats2half2_rn(res.x + red.x, res.y + red.y));
        }
    }
    *reinterpret_cast<uint4 *>(p.h + row * p.ld_h + col) = make_uint4(o[0], o[1], o[2], o[3]);
}

}  // namespace rptc

using namespace rptc;

// ---- peer memory plumbing (CUDA IPC; the handles travel through the caller's process group) ----
extern "C" int rptc_peer_alloc(int64_t bytes, void **ptr) {
    if (!ptr || bytes <= 0) return RPTC_ERR_ARG;
    RPTC_CUDA(cudaMalloc(ptr, (size_t)bytes));
    RPTC_CUDA(cudaMemset(*ptr, 0, (size_t)bytes));
    return RPTC_OK;
}
extern "C" int rptc_peer_free(void *ptr) {
    RPTC_CUDA(cudaFree(ptr));
    return RPTC_OK;
}
extern "C" int rptc_peer_export(void *ptr, unsigned char *handle64) {
    if (!ptr || !handle64) return RPTC_ERR_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    RPTC_CUDA(cudaIpcGetMemHandle(&h, ptr));
    memcpy(handle64, &h, 64);
    return RPTC_OK;
}
extern "C" int rptc_peer_import(const unsigned char *handle64, void **ptr) {
    if (!ptr || !handle64) return RPTC_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    RPTC_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return RPTC_OK;
}
extern "C" int rptc_peer_close(void *ptr) {
    RPTC_CUDA(cudaIpcCloseMemHandle(ptr));
    return RPTC_OK;
}

extern "C" int rptc_peer_finish(float *acc, int64_t ld_acc, const void *signs_out, float scale, void *h, int64_t ld_h,
                                void *const *data_ptrs, void *const *flag_ptrs, void *epochs, int rank, int world, int64_t rows,
                                int64_t n, int block, int64_t timeout_ms, rptc_stream_t stream) {
    if (!acc || !h || !data_ptrs || !epochs) return RPTC_ERR_ARG;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return RPTC_ERR_ARG;
    if (block < 8 || block > 4096 || (block & (block - 1))) return RPTC_ERR_ARG;
    const int chunk = block < 256 ? 256 : block;
    if (rows <= 0 || rows > 65535 || n <= 0 || (n % chunk) || ld_acc < n || ld_h < n) return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(acc) & 15) || (reinterpret_cast<uintptr_t>(h) & 15) || (ld_acc % 4) || (ld_h % 8) ||
        (signs_out && (reinterpret_cast<uintptr_t>(signs_out) & 15)))
        return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    PeerFinishParams p;
    p.acc = acc;
    p.ld_acc = ld_acc;
    p.signs_out = static_cast<const __half *>(signs_out);
    p.scale = scale;
    p.h = static_cast<__half *>(h);
    p.ld_h = ld_h;
    for (int r = 0; r < kMaxPeers; ++r) {
        p.data[r] = r < world ? static_cast<uint64_t *>(data_ptrs[r]) : nullptr;
        if (r < world && !p.data[r]) return RPTC_ERR_ARG;
    }
    (void)flag_ptrs;      // the flags travel inside the data words
    p.epochs = static_cast<uint32_t *>(epochs);
    p.rank = rank;
    p.world = world;
    p.n = (int32_t)n;
    p.block = block;
    p.chunk = chunk;
    p.rows = (int32_t)rows;
    p.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
    p.status = device_status_word();
    if (!p.status) return RPTC_ERR_CUDA;
    return launch(peer_finish_kernel, dim3((unsigned)(n / chunk), (unsigned)rows), dim3(chunk / 8), 0, static_cast<cudaStream_t>(stream), p);
}
