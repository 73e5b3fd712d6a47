// Host-side plumbing of the C ABI: status strings, device checks, the device status word.
#include "common.cuh"

namespace rptc {

thread_local int g_last_cuda_error = 0;
static thread_local bool g_pdl = false;      // per calling thread: two threads that launch with different settings do not race

int cuda_fail(cudaError_t e) {
    g_last_cuda_error = (int)e;
    (void)cudaGetLastError();   // clear the sticky-free error so that later launches are not blamed for it
    return RPTC_ERR_CUDA;
}

bool pdl_enabled() { return g_pdl; }

static int g_sms[kMaxDevices];
static int g_cc[kMaxDevices];

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
}

int num_sms() {
    const int dev = current_device();
    if (dev < 0) return kNumSMsFallback;
    if (g_sms[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = kNumSMsFallback;
        g_sms[dev] = v;
    }
    return g_sms[dev];
}

// One status word per device (each device that loads this module has its own copy of the symbol).
__device__ unsigned int g_status_word;
static unsigned int *g_status_ptr[kMaxDevices];

unsigned int *device_status_word() {
    const int dev = current_device();
    if (dev < 0) return nullptr;
    if (!g_status_ptr[dev]) {
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_status_word);
        if (e != cudaSuccess) {
            cuda_fail(e);
            return nullptr;
        }
        g_status_ptr[dev] = static_cast<unsigned int *>(ptr);
    }
    return g_status_ptr[dev];
}

int check_format(const rptc_format *f) {
    if (!f) return RPTC_ERR_ARG;
    if (f->code < RPTC_CODE_LUT || f->code > RPTC_CODE_LITE) return RPTC_ERR_ARG;
    if (f->layout < RPTC_LAYOUT_ROWMAJOR || f->layout > RPTC_LAYOUT_TILED) return RPTC_ERR_ARG;
    if (f->quirk < RPTC_QUIRK_NONE || f->quirk > RPTC_QUIRK_K2_LANE0_CARRY) return RPTC_ERR_ARG;
    if (f->K < 2 || f->K > 4) return RPTC_ERR_ARG;
    if (f->L < 1 || f->L > 16) return RPTC_ERR_ARG;
    if (f->quirk != RPTC_QUIRK_NONE && f->K != 2) return RPTC_ERR_UNSUPPORTED;
    switch (f->code) {
        case RPTC_CODE_LUT:
            if (f->L < 3) return RPTC_ERR_ARG;
            break;
        case RPTC_CODE_HASH:
            if (f->K != 2) return RPTC_ERR_UNSUPPORTED;
            if (f->S < 1 || f->S > 8) return RPTC_ERR_ARG;
            break;
        case RPTC_CODE_LITE:
            if (f->K == 3) return RPTC_ERR_UNSUPPORTED;
            if (f->S < 1 || f->S > 10 || f->S > f->L) return RPTC_ERR_ARG;
            break;
    }
    return RPTC_OK;
}

}  // namespace rptc

using namespace rptc;

extern "C" const char *rptc_strerror(int status) {
    switch (status) {
        case RPTC_OK: return "ok";
        case RPTC_ERR_ARG: return "invalid argument (null pointer or bad enum value)";
        case RPTC_ERR_SHAPE: return "shape violates a divisibility or leading-dimension rule";
        case RPTC_ERR_ALIGN: return "pointer or leading dimension not aligned as required";
        case RPTC_ERR_UNSUPPORTED: return "combination of code, K and layout is not implemented";
        case RPTC_ERR_CUDA: return "a CUDA runtime call failed (see rptc_last_cuda_error)";
        case RPTC_ERR_TIMEOUT: return "a bounded device-side wait ran out";
        case RPTC_ERR_TOO_LARGE: return "size beyond a documented maximum";
        case RPTC_ERR_DEVICE: return "current device is not a compute-capability 10.x GPU";
        case RPTC_ERR_INTERNAL: return "a kernel found its shared-memory plan violated and did nothing";
        case RPTC_ERR_RANGE: return "a sequence position lay outside the KV cache; the access was skipped";
    }
    return "unknown status";
}

extern "C" int rptc_version(void) { return 100; }

extern "C" int rptc_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" void rptc_set_pdl(int enable) { g_pdl = enable != 0; }

extern "C" int rptc_check_device(void) {
    const int dev = current_device();
    if (dev < 0) return cuda_fail(cudaErrorNoDevice);
    if (g_cc[dev] == 0) {
        int major = 0;
        RPTC_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        g_cc[dev] = major;
    }
    return g_cc[dev] == 10 ? RPTC_OK : RPTC_ERR_DEVICE;
}

extern "C" int rptc_device_status(void) {
    unsigned int *w = device_status_word();
    if (!w) return RPTC_ERR_CUDA;
    RPTC_CUDA(cudaDeviceSynchronize());
    unsigned int v = 0;
    RPTC_CUDA(cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost));
    if (v) {
        const unsigned int zero = 0;
        RPTC_CUDA(cudaMemcpy(w, &zero, sizeof(zero), cudaMemcpyHostToDevice));
        if (v == kStatusSmemPlan) return RPTC_ERR_INTERNAL;
        if (v == kStatusPosition) return RPTC_ERR_RANGE;
        return RPTC_ERR_TIMEOUT;
    }
    return RPTC_OK;
}
