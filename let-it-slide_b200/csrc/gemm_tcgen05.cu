// Placeholder until the tcgen05 prefill kernel lands.
#include "common.cuh"
extern "C" int rptc_gemm(const void *, const void *, const uint32_t *, const void *, int64_t, void *, int64_t, int64_t,
                         int64_t, int64_t, const rptc_format *, rptc_stream_t) {
    return RPTC_ERR_UNSUPPORTED;
}
