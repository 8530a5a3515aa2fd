// Argmax over device logits for callers that must not allocate.
//
// wick_cuda_argmax() borrows a few bytes of scratch from the stream-ordered allocator on
// every call.  Some callers cannot do that: a real-time audio / serving thread where the CUDA
// allocator (and the locks and possible device synchronisation behind it) is off limits, or a
// process whose device memory pool has been handed over completely to another component.  For
// them this file keeps the scratch in a fixed array that is part of the library image: it exists
// once per GPU that loads the library, for as long as the process lives, and neither a CUDA
// allocation routine nor the host heap is used here (error messages go into a fixed per-thread
// buffer).  What the entry point still does on its FIRST call per device: it takes a process-wide
// mutex and asks the runtime for the array's device address, which may load the module onto that
// device.  Make that call once per device as a warm-up, outside real-time sections and outside
// stream capture; later calls on that device only read the cached address under the same mutex.
// (It cannot be called from inside a cudaLaunchHostFunc callback: no CUDA API call can.)
#include <cstdio>
#include <mutex>

#include "../../include/wick_cuda.h"
#include "common.cuh"

namespace wick {
extern thread_local unsigned long long g_kernel_launches;
}
using namespace wick;

namespace {

constexpr int NA_BLOCK_ELEMS = 1024;                 // logits reduced by one block of the first pass
constexpr int NA_MAX_BLOCKS = WICK_CUDA_ARGMAX_NOALLOC_MAX / NA_BLOCK_ELEMS;
static_assert(WICK_CUDA_ARGMAX_NOALLOC_MAX % NA_BLOCK_ELEMS == 0, "maximum must be whole blocks");

// One packed (key, index) partial per first-pass block: 4096 * 8 bytes = 32 KB per GPU.
static __device__ __align__(256) unsigned long long g_noalloc_partials[NA_MAX_BLOCKS];

__global__ void __launch_bounds__(256) k_argmax_na_pass1(const float* __restrict__ x, int count, unsigned long long* __restrict__ partial) {
    __shared__ unsigned long long sh[8];
    const int base = blockIdx.x * NA_BLOCK_ELEMS;
    unsigned long long best = 0;
    for (int i = base + threadIdx.x; i < base + NA_BLOCK_ELEMS && i < count; i += 256) {
        unsigned long long p = argmax_pack(x[i], (uint32_t)i);
        best = p > best ? p : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
        best = t > best ? t : best;
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; i++) best = sh[i] > best ? sh[i] : best;
        partial[blockIdx.x] = best;  // every slot that pass 2 reads is rewritten by this launch
    }
}

__global__ void __launch_bounds__(256) k_argmax_na_pass2(const unsigned long long* __restrict__ partial, int n, uint32_t* __restrict__ out) {
    __shared__ unsigned long long sh[8];
    unsigned long long best = 0;
    for (int i = threadIdx.x; i < n; i += 256) best = partial[i] > best ? partial[i] : best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
        best = t > best ? t : best;
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; i++) best = sh[i] > best ? sh[i] : best;
        *out = (uint32_t)(best & 0xffffffffull);
    }
}

// In host code `g_noalloc_partials` is only a handle for the symbol, not a device address: the
// address a kernel can use has to be asked for, once per device, with that device current.
constexpr int NA_MAX_DEVICES = 64;
std::mutex g_na_mutex;
unsigned long long* g_na_ptr[NA_MAX_DEVICES] = {};

thread_local char g_na_error[192] = "";

int32_t na_fail(int32_t code, const char* what, const char* detail) {
    snprintf(g_na_error, sizeof(g_na_error), "argmax_noalloc: %s%s%s", what, detail ? ": " : "", detail ? detail : "");
    return code;
}

}  // namespace

extern "C" const char* wick_cuda_argmax_noalloc_last_error(void) { return g_na_error; }

extern "C" int32_t wick_cuda_argmax_noalloc(const float* logits_dev, uint32_t count, uint32_t* out_dev, void* stream) {
    if (!logits_dev || !out_dev || count == 0) return na_fail(WICK_CUDA_ERR_BAD_ARG, "NULL argument or empty input", nullptr);
    if (count > (uint32_t)WICK_CUDA_ARGMAX_NOALLOC_MAX) {
        snprintf(g_na_error, sizeof(g_na_error), "argmax_noalloc: %u logits exceed the fixed scratch (maximum %d); use wick_cuda_argmax",
                 count, (int)WICK_CUDA_ARGMAX_NOALLOC_MAX);
        return WICK_CUDA_ERR_BAD_ARG;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return na_fail(WICK_CUDA_ERR_CUDA, "cudaGetDevice", cudaGetErrorString(e));
    if (dev < 0 || dev >= NA_MAX_DEVICES) {
        snprintf(g_na_error, sizeof(g_na_error), "argmax_noalloc: device ordinal %d is beyond the %d devices this entry point keeps an address for",
                 dev, NA_MAX_DEVICES);
        return WICK_CUDA_ERR_BAD_ARG;
    }
    unsigned long long* scratch;
    {
        std::lock_guard<std::mutex> lk(g_na_mutex);
        if (!g_na_ptr[dev]) {  // first call on this device: resolve the symbol's device address
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_partials);
            if (e != cudaSuccess || !p) return na_fail(WICK_CUDA_ERR_CUDA, "cudaGetSymbolAddress", cudaGetErrorString(e));
            g_na_ptr[dev] = (unsigned long long*)p;
        }
        scratch = g_na_ptr[dev];
    }
    const int nblk = (int)((count + NA_BLOCK_ELEMS - 1) / NA_BLOCK_ELEMS);
    cudaStream_t st = (cudaStream_t)stream;
    g_kernel_launches += 2;
    k_argmax_na_pass1<<<nblk, 256, 0, st>>>(logits_dev, (int)count, scratch);
    k_argmax_na_pass2<<<1, 256, 0, st>>>(scratch, nblk, out_dev);
    e = cudaGetLastError();
    if (e != cudaSuccess) return na_fail(WICK_CUDA_ERR_CUDA, "launch", cudaGetErrorString(e));
    return WICK_CUDA_OK;
}
