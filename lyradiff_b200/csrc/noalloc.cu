// lyraq_w4a4_forward_static: the W4A4 linear forward for callers that can neither allocate device memory nor hand
// the library a workspace.
//
// Some hosts call into this library from places where a device allocation is off the table: an inference server's
// enqueue hook that has to stay asynchronous (cudaMalloc and cudaFree synchronise the whole device), a plug-in slot
// whose interface passes inputs and outputs but no scratch pointer, or a process in which another framework owns
// every byte of the memory pool.  For them the scratch that lyraq_w4a4_forward takes as `workspace` (the int4-packed
// activation and its per-group scales) lives in a fixed array inside the library's own device image instead.
//
// The array is 16 MiB per GPU and stays until the process exits.  CUDA loads a module's device image lazily by default,
// so the driver sets the array up -- its one allocation, possibly with a device synchronisation -- when the address is
// first asked for on a device: at the first call of this entry point there, or earlier and outside any enqueue hook or
// stream capture if the host calls lyraq_static_scratch_bytes() once per device at start-up (CUDA_MODULE_LOADING=EAGER
// moves it to context creation instead).  If that set-up fails, e.g. because the pool is exhausted, the call returns
// LYRAQ_ERR_CUDA and launches nothing.  All calls share the array and it keeps whatever the last call left there.  Nothing in it has to start at zero: the
// quantizer overwrites every byte the GEMM will read before the GEMM reads it.  Two calls whose GPU work overlaps
// in time (different streams, or different host threads) race on the array; run them on one stream.
#include "common.cuh"

namespace lyraq {

constexpr size_t kStaticScratchBytes = 16u << 20;

// Device-side storage.  In host code this name is only a handle for the runtime: its device address is looked up once
// per device with cudaGetSymbolAddress (below) and that address is what the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static unsigned char* g_static_scratch_addr[64];  // device address per device ordinal, filled by the first call

// Set-up, once per device, with that device current: resolve the array's device address.
static int static_scratch_ptr(unsigned char** out)
{
    int dev = 0;
    const cudaError_t e0 = cudaGetDevice(&dev);
    if (e0 != cudaSuccess) {
        return cuda_status(e0, "cudaGetDevice (static scratch set-up)");
    }
    if (dev < 0 || dev >= 64) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    if (g_static_scratch_addr[dev] == nullptr) {
        void*             p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            return cuda_status(e == cudaSuccess ? cudaErrorInvalidSymbol : e, "cudaGetSymbolAddress(static scratch)");
        }
        g_static_scratch_addr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_static_scratch_addr[dev];
    return LYRAQ_OK;
}

}  // namespace lyraq

using namespace lyraq;

extern "C" {

// Size of the array; as a side effect resolves its address on the current device (the warm-up described at the top).
// Without a device, or if the set-up fails, the size is still returned and the failure shows up at the first forward.
size_t lyraq_static_scratch_bytes(void)
{
    unsigned char* unused = nullptr;
    int            count  = 0;
    if (cudaGetDeviceCount(&count) == cudaSuccess && count > 0) {
        (void)static_scratch_ptr(&unused);
    } else {
        (void)cudaGetLastError();
    }
    return kStaticScratchBytes;
}

int lyraq_w4a4_forward_static(void* D, const void* x, int dtype, const float* smooth, const uint8_t* W, const void* w_scale,
                              int w_scale_dtype, const void* bias, const void* residual, int epilogue, int m, int n, int k,
                              void* stream)
{
    if (m < 0 || n < 0 || k < 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (m == 0 || n == 0) {
        return LYRAQ_OK;
    }
    // the same bytes lyraq_w4a4_forward would ask its caller for; beyond the fixed array the call is refused
    const size_t need = lyraq_workspace_bytes(LYRAQ_OP_LINEAR_W4A4, m, n, k);
    if (need > kStaticScratchBytes) {
        return LYRAQ_ERR_WORKSPACE;
    }
    unsigned char* scratch = nullptr;
    const int      st      = static_scratch_ptr(&scratch);
    if (st != LYRAQ_OK) {
        return st;
    }
    return lyraq_w4a4_forward(D, x, dtype, smooth, W, w_scale, w_scale_dtype, bias, residual, epilogue, m, n, k, scratch,
                              kStaticScratchBytes, stream);
}

}  // extern "C"
