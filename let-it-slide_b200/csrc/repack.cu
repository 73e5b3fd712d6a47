// Re-tiling of packed codes between the three layouts: a permutation of 128-bit units.
#include "common.cuh"

namespace rptc {

// One thread moves one unit.  Threads are numbered in destination order, so writes are coalesced
// whatever the source layout is.
__global__ void repack_kernel(const uint4 *__restrict__ src, UnitStrides ss, uint4 *__restrict__ dst, int dst_layout,
                              int64_t m, int64_t n_units) {
    pdl_allow_next_grid();
    pdl_wait_prior_grids();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m * n_units) return;
    int64_t u, r;
    if (dst_layout == RPTC_LAYOUT_ROWMAJOR) {
        r = i / n_units;
        u = i - r * n_units;
    } else if (dst_layout == RPTC_LAYOUT_CHUNKED) {
        const int64_t chunk = i / (m * 32), rem = i - chunk * (m * 32);
        r = rem >> 5;
        u = chunk * 32 + (rem & 31);
    } else if (dst_layout == RPTC_LAYOUT_UNITMAJOR) {
        u = i / m;
        r = i - u * m;
    } else {
        const int64_t rb = i / (n_units * 32), rem = i - rb * (n_units * 32);
        u = rem >> 5;
        r = rb * 32 + (rem & 31);
    }
    dst[i] = src[unit_index(ss, u, r)];
}

}  // namespace rptc

using namespace rptc;

extern "C" int rptc_repack(const void *src, int src_layout, void *dst, int dst_layout, int64_t m, int64_t n_units,
                           rptc_stream_t stream) {
    if (!src || !dst || src == dst) return RPTC_ERR_ARG;
    if (src_layout < 0 || src_layout > 3 || dst_layout < 0 || dst_layout > 3) return RPTC_ERR_ARG;
    if (m <= 0 || n_units <= 0 || (m % 32)) return RPTC_ERR_SHAPE;
    if ((src_layout == RPTC_LAYOUT_CHUNKED || dst_layout == RPTC_LAYOUT_CHUNKED) && (n_units % 32)) return RPTC_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return RPTC_ERR_ALIGN;
    if (int e = rptc_check_device()) return e;
    const int64_t total = m * n_units;
    return launch(repack_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                  static_cast<const uint4 *>(src), unit_strides(src_layout, m, n_units), static_cast<uint4 *>(dst), dst_layout,
                  m, n_units);
}
