// cn_dot_noalloc: a dot product for callers that must not allocate device memory.
//
// Who needs this.  Everything else in the library takes its working memory from
// cudaMalloc / the stream-ordered pool (the per-block partial sums of the two-pass reduction
// live in a buffer the context allocates).  Some callers cannot do that: code that runs
// inside a region where allocation is forbidden or would deadlock (a callback from another
// runtime, a solver that has already claimed all device memory as one arena and hands out
// raw pointers, an error path that must still be able to compute a residual after an
// out-of-memory), and code that is not allowed to touch the allocator for determinism or
// latency reasons.  For them this entry point computes result[0] = sum_i a[i] * b[i] with the
// same deterministic two-pass scheme as the regular dot kernel, but its scratch -- one partial
// per 8192-element block plus the ticket counter -- lives in a fixed array that is part of
// the library image.  The caller supplies the inputs and the output as device pointers and
// this function makes no allocation or free of its own.
//
// Limits and rules
//   * n <= CN_NOALLOC_MAX_ELEMS (2^28 elements, 2 GiB per operand): the scratch holds one
//     partial per 8192 elements.  Larger n returns CN_STATUS_LIMIT and does nothing.
//   * Every GPU that loads the library carries the 256 KiB scratch array until the process
//     exits.
//   * The first call on a device looks up the device address of the scratch array
//     (cudaGetSymbolAddress, with that device current) and remembers it.  With CUDA's lazy
//     module loading that same call makes the driver place the library's device image -- the
//     scratch array and the exp tables -- in device memory, which is an allocation by the
//     driver.  So make the first call as a warm-up (n = 0 will do) while memory is still
//     available and outside any stream capture; only later calls are allocation-free.
//   * All calls on a device share the scratch.  It keeps whatever the previous call left; the
//     ticket counter is cleared on the stream before each launch.  Two calls whose kernels
//     overlap on the GPU (different streams without ordering) race on it: order them.
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "../../include/cnb200.h"
#include "cn_device.cuh"

namespace {

constexpr long long kChunk = 8192;                   // elements per block
constexpr long long kMaxBlocks = 32768;              // partials in the scratch
constexpr long long kMaxElems = kChunk * kMaxBlocks; // 2^28
static_assert(kMaxElems == CN_NOALLOC_MAX_ELEMS, "header and kernel disagree on the limit");
constexpr int kMaxDevices = 64;

struct NoAllocScratch {
    double partials[kMaxBlocks];
    unsigned int ticket;
    unsigned int pad[63];
};

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress; the
// address a kernel may use is the one that call returns.
static __device__ __align__(256) NoAllocScratch cn_noalloc_scratch;

__global__ void __launch_bounds__(256)
dot_noalloc_kernel(const double* __restrict__ a, const double* __restrict__ b, long long n,
                   NoAllocScratch* scratch, double* result) {
    const long long lo = (long long)blockIdx.x * kChunk;
    const long long hi = lo + kChunk < n ? lo + kChunk : n;
    double acc = 0.0;
    for (long long i = lo + threadIdx.x; i < hi; i += 256) acc += a[i] * b[i];
    __shared__ double sm[32];
    __shared__ int flag;
    double bt = cn_block_sum(acc, sm);
    if (threadIdx.x == 0) scratch->partials[blockIdx.x] = bt;
    if (cn_grid_ticket(&scratch->ticket, &flag)) {
        double t = cn_sum_partials(scratch->partials, sm);
        if (threadIdx.x == 0) {
            *result = t;
            scratch->ticket = 0u;
        }
    }
}

std::mutex g_mutex;
NoAllocScratch* g_scratch[kMaxDevices];  // device address of the scratch, per device

}  // namespace

extern "C" int cn_dot_noalloc(const double* a, const double* b, int64_t n, double* result,
                              void* stream) {
    if (!a || !b || !result || n < 0) return CN_STATUS_INVALID_ARGUMENT;
    if (n > kMaxElems) return CN_STATUS_LIMIT;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return CN_STATUS_NO_DEVICE;
    if (dev < 0 || dev >= kMaxDevices) return CN_STATUS_LIMIT;
    NoAllocScratch* scratch;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!g_scratch[dev]) {
            void* p = nullptr;
            if (cudaGetSymbolAddress(&p, cn_noalloc_scratch) != cudaSuccess || !p) {
                cudaGetLastError();
                return CN_STATUS_CUDA;
            }
            g_scratch[dev] = static_cast<NoAllocScratch*>(p);
        }
        scratch = g_scratch[dev];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(&scratch->ticket, 0, sizeof(unsigned int), s) != cudaSuccess) {
        cudaGetLastError();
        return CN_STATUS_CUDA;
    }
    long long blocks = (n + kChunk - 1) / kChunk;
    if (blocks < 1) blocks = 1;
    dot_noalloc_kernel<<<(unsigned int)blocks, 256, 0, s>>>(a, b, n, scratch, result);
    if (cudaGetLastError() != cudaSuccess) return CN_STATUS_CUDA;
    return CN_STATUS_OK;
}
