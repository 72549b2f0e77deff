// Library-level entry points: version, status strings, the per-device status word.
#include "common.cuh"

#include <cstdio>

namespace lyraq {

// Word 0: status code written by the first kernel wait that gave up; word 1: which wait.
__device__ unsigned int g_status_words[4];

static unsigned int* g_status_addr[64];  // per device ordinal, filled on first use

unsigned int* status_word_ptr()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        return nullptr;
    }
    if (g_status_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_words) != cudaSuccess) {
            return nullptr;
        }
        g_status_addr[dev] = static_cast<unsigned int*>(p);
    }
    return g_status_addr[dev];
}

static char g_last_error[256] = "no CUDA error recorded";

void record_cuda_error(cudaError_t e, const char* where)
{
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", where, cudaGetErrorString(e), cudaGetErrorName(e));
}

static int g_dependent_launch = 1;
bool dependent_launch_enabled() { return g_dependent_launch != 0; }

}  // namespace lyraq

extern "C" {

int lyraq_debug_set_dependent_launch(int on)
{
    lyraq::g_dependent_launch = on ? 1 : 0;
    return LYRAQ_OK;
}

const char* lyraq_last_cuda_error(void) { return lyraq::g_last_error; }

const char* lyraq_version(void) { return "lyraq 0.1 (sm_100a)"; }

const char* lyraq_status_string(int status)
{
    switch (status) {
        case LYRAQ_OK: return "ok";
        case LYRAQ_ERR_INVALID_ARG: return "invalid argument (null, misaligned or bad enum)";
        case LYRAQ_ERR_UNSUPPORTED: return "shape or type not supported by the sm_100a kernels";
        case LYRAQ_ERR_CUDA: return "CUDA call failed";
        case LYRAQ_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel ran out";
        case LYRAQ_ERR_WORKSPACE: return "workspace missing or too small";
        default: return "unknown status";
    }
}

int lyraq_last_status(void* stream, uint32_t* detail)
{
    unsigned int* dptr = lyraq::status_word_ptr();
    if (dptr == nullptr) {
        return LYRAQ_ERR_CUDA;
    }
    cudaStream_t s = (cudaStream_t)stream;
    unsigned int host[2] = {0u, 0u};
    if (cudaMemcpyAsync(host, dptr, sizeof(host), cudaMemcpyDeviceToHost, s) != cudaSuccess) {
        return LYRAQ_ERR_CUDA;
    }
    if (cudaStreamSynchronize(s) != cudaSuccess) {
        return LYRAQ_ERR_CUDA;
    }
    if (host[0] != 0u) {
        if (cudaMemsetAsync(dptr, 0, 2 * sizeof(unsigned int), s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) {
            return LYRAQ_ERR_CUDA;
        }
    }
    if (detail != nullptr) {
        *detail = host[1];
    }
    return (int)host[0];
}


}  // extern "C"
