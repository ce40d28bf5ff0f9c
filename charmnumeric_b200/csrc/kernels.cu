// Ahead-of-time CUDA kernels for sm_100a: region fill / copy, seeded uniform fill, dot /
// sum with the deterministic two-pass finish, and the row-block matrix-vector product.
// All of them are bandwidth-bound; none uses tensor cores (no path here is a dense
// contraction with reuse).
#include <algorithm>

#include "cn_device.cuh"
#include "cn_types.hpp"
#include "kernels.hpp"

namespace cn {

namespace {

struct View3 {
    long long off;
    long long str[3];
    long long ext[3];
};

__device__ __forceinline__ long long view_index(const View3& v, long long i) {
    long long i2 = i % v.ext[2];
    long long t = i / v.ext[2];
    long long i1 = t % v.ext[1];
    long long i0 = t / v.ext[1];
    return v.off + i0 * v.str[0] + i1 * v.str[1] + i2 * v.str[2];
}

template <typename T>
__global__ void __launch_bounds__(256) fill_region_kernel(T* base, View3 v, T value, long long n) {
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n;
         i += (long long)gridDim.x * 256)
        base[view_index(v, i)] = value;
}

// contiguous fill, 128-bit stores
__global__ void __launch_bounds__(256) fill_f64_kernel(double* p, double value, long long n) {
    long long i = ((long long)blockIdx.x * 256 + threadIdx.x) * 2;
    const long long stride = (long long)gridDim.x * 512;
    for (; i + 1 < n; i += stride) *(double2*)(p + i) = make_double2(value, value);
    if (i < n) p[i] = value;
}

template <typename T>
__global__ void __launch_bounds__(256)
copy_region_kernel(T* dst, View3 dv, const T* src, View3 sv, long long n) {
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n;
         i += (long long)gridDim.x * 256)
        dst[view_index(dv, i)] = src[view_index(sv, i)];
}

__device__ __forceinline__ double randu_value(unsigned long long seed, unsigned long long g,
                                              double lo, double span) {
    unsigned long long z = seed + (g + 1ULL) * 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    z = z ^ (z >> 31);
    double u = (double)(z >> 11) * 0x1p-53;
    return __dadd_rn(lo, __dmul_rn(span, u));  // two roundings, never an fma
}

template <typename T>
__global__ void __launch_bounds__(256)
randu_kernel(T* p, long long n, unsigned long long goff, unsigned long long seed, double lo,
             double span) {
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n;
         i += (long long)gridDim.x * 256)
        p[i] = (T)randu_value(seed, goff + (unsigned long long)i, lo, span);
}

// ---- dot / sum ----------------------------------------------------------------------
template <typename T, typename ACC, bool HAS_B>
__global__ void __launch_bounds__(256)
dot_kernel(const T* __restrict__ a, const T* __restrict__ b, long long n, ACC* partials,
           unsigned int* counter, T* result) {
    ACC acc = (ACC)0;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n;
         i += (long long)gridDim.x * 256) {
        ACC va = (ACC)a[i];
        acc += HAS_B ? va * (ACC)b[i] : va;
    }
    __shared__ ACC sm[32];
    __shared__ int flag;
    ACC bt = cn_block_sum(acc, sm);
    if (threadIdx.x == 0) partials[blockIdx.x] = bt;
    if (cn_grid_ticket(counter, &flag)) {
        ACC t = cn_sum_partials(partials, sm);
        if (threadIdx.x == 0) {
            *result = (T)t;
            *counter = 0u;
        }
    }
}

// float64 fast path: 128-bit loads, four independent chunks in flight per thread
template <bool HAS_B>
__global__ void __launch_bounds__(256)
dot_f64_vec_kernel(const double* __restrict__ a, const double* __restrict__ b, long long n,
                   double* partials, unsigned int* counter, double* result) {
    double acc0 = 0, acc1 = 0;
    const long long npair = n >> 1;
    const long long stride = (long long)gridDim.x * 256;
    long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    for (; i + 3 * stride < npair; i += 4 * stride) {
        double2 va[4], vb[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            va[k] = ((const double2*)a)[i + k * stride];
            if (HAS_B) vb[k] = ((const double2*)b)[i + k * stride];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (HAS_B) {
                acc0 += va[k].x * vb[k].x;
                acc1 += va[k].y * vb[k].y;
            } else {
                acc0 += va[k].x;
                acc1 += va[k].y;
            }
        }
    }
    for (; i < npair; i += stride) {
        double2 va = ((const double2*)a)[i];
        if (HAS_B) {
            double2 vb = ((const double2*)b)[i];
            acc0 += va.x * vb.x;
            acc1 += va.y * vb.y;
        } else {
            acc0 += va.x;
            acc1 += va.y;
        }
    }
    if ((n & 1) && blockIdx.x == 0 && threadIdx.x == 0)
        acc0 += HAS_B ? a[n - 1] * b[n - 1] : a[n - 1];
    __shared__ double sm[32];
    __shared__ int flag;
    double bt = cn_block_sum(acc0 + acc1, sm);
    if (threadIdx.x == 0) partials[blockIdx.x] = bt;
    if (cn_grid_ticket(counter, &flag)) {
        double t = cn_sum_partials(partials, sm);
        if (threadIdx.x == 0) {
            *result = t;
            *counter = 0u;
        }
    }
}

// ---- matvec ---------------------------------------------------------------------------
// One block per group of MV_ROWS rows.  Each thread walks the columns in 128-bit steps,
// loads the x chunk once and the A chunk of every row of the group, so x (which lives in
// L2) is re-read only 1/MV_ROWS times per A byte.  The row sums are folded with the fixed
// shuffle tree, so results do not depend on scheduling.
constexpr int MV_ROWS = 4;

__global__ void __launch_bounds__(256)
matvec_f64_vec_kernel(const double* __restrict__ A, long long lda, const double* __restrict__ x,
                      double* __restrict__ y, long long rows, long long cols) {
    const long long r0 = (long long)blockIdx.x * MV_ROWS;
    const double2* arow[MV_ROWS];
#pragma unroll
    for (int r = 0; r < MV_ROWS; ++r) {
        long long rr = r0 + r < rows ? r0 + r : rows - 1;
        arow[r] = (const double2*)(A + rr * lda);
    }
    const double2* xv = (const double2*)x;
    double acc[MV_ROWS];
#pragma unroll
    for (int r = 0; r < MV_ROWS; ++r) acc[r] = 0.0;
    const long long npair = cols >> 1;
    long long c = threadIdx.x;
    for (; c + 256 < npair; c += 512) {
        double2 x0 = __ldg(xv + c), x1 = __ldg(xv + c + 256);
        double2 a0[MV_ROWS], a1[MV_ROWS];
#pragma unroll
        for (int r = 0; r < MV_ROWS; ++r) {
            a0[r] = __ldcs(arow[r] + c);
            a1[r] = __ldcs(arow[r] + c + 256);
        }
#pragma unroll
        for (int r = 0; r < MV_ROWS; ++r) {
            acc[r] += a0[r].x * x0.x;
            acc[r] += a0[r].y * x0.y;
            acc[r] += a1[r].x * x1.x;
            acc[r] += a1[r].y * x1.y;
        }
    }
    for (; c < npair; c += 256) {
        double2 x0 = __ldg(xv + c);
#pragma unroll
        for (int r = 0; r < MV_ROWS; ++r) {
            double2 a0 = __ldcs(arow[r] + c);
            acc[r] += a0.x * x0.x;
            acc[r] += a0.y * x0.y;
        }
    }
    __shared__ double sm[32];
#pragma unroll
    for (int r = 0; r < MV_ROWS; ++r) {
        double t = cn_block_sum(acc[r], sm);
        if (threadIdx.x == 0 && r0 + r < rows) y[r0 + r] = t;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
matvec_generic_kernel(const T* __restrict__ A, long long lda, const T* __restrict__ x,
                      T* __restrict__ y, long long rows, long long cols) {
    const long long r = blockIdx.x;
    if (r >= rows) return;
    T acc = (T)0;
    for (long long c = threadIdx.x; c < cols; c += 256) acc += A[r * lda + c] * x[c];
    __shared__ T sm[32];
    T t = cn_block_sum(acc, sm);
    if (threadIdx.x == 0) y[r] = t;
}

int grid_for(long long n, int per_block) {
    long long b = (n + per_block - 1) / per_block;
    if (b < 1) b = 1;
    if (b > 148 * 16) b = 148 * 16;
    return (int)b;
}

View3 make_view(const StridedView& v, const int64_t ext[3]) {
    View3 o;
    o.off = v.off;
    for (int d = 0; d < 3; ++d) {
        o.str[d] = v.str[d];
        o.ext[d] = ext[d] > 0 ? ext[d] : 1;
    }
    return o;
}

}  // namespace

cudaError_t launch_fill_region(void* base, int dtype, const StridedView& v, const int64_t ext[3],
                               double value, cudaStream_t s) {
    View3 vw = make_view(v, ext);
    long long n = vw.ext[0] * vw.ext[1] * vw.ext[2];
    if (ext[0] <= 0 || n <= 0) return cudaSuccess;
    bool contiguous = (vw.str[2] == 1 || vw.ext[2] == 1) &&
                      (vw.ext[1] == 1 || vw.str[1] == vw.ext[2]) &&
                      (vw.ext[0] == 1 || vw.str[0] == vw.ext[1] * vw.ext[2]);
    if (dtype == DT_F64 && contiguous && (((uintptr_t)((double*)base + v.off)) & 15) == 0) {
        fill_f64_kernel<<<grid_for(n, 512), 256, 0, s>>>((double*)base + v.off, value, n);
        return cudaGetLastError();
    }
    int grid = grid_for(n, 256);
    switch (dtype) {
        case DT_F32: fill_region_kernel<float><<<grid, 256, 0, s>>>((float*)base, vw, (float)value, n); break;
        case DT_F64: fill_region_kernel<double><<<grid, 256, 0, s>>>((double*)base, vw, value, n); break;
        case DT_I32: fill_region_kernel<int><<<grid, 256, 0, s>>>((int*)base, vw, (int)value, n); break;
        default: fill_region_kernel<long long><<<grid, 256, 0, s>>>((long long*)base, vw, (long long)value, n); break;
    }
    return cudaGetLastError();
}

cudaError_t launch_copy_region(void* dst, const StridedView& dv, const void* src,
                               const StridedView& sv, const int64_t ext[3], int dtype,
                               cudaStream_t s) {
    View3 d = make_view(dv, ext), sr = make_view(sv, ext);
    long long n = d.ext[0] * d.ext[1] * d.ext[2];
    if (ext[0] <= 0 || n <= 0) return cudaSuccess;
    int grid = grid_for(n, 256);
    if (dtype_size(dtype) == 8)
        copy_region_kernel<long long><<<grid, 256, 0, s>>>((long long*)dst, d, (const long long*)src, sr, n);
    else
        copy_region_kernel<int><<<grid, 256, 0, s>>>((int*)dst, d, (const int*)src, sr, n);
    return cudaGetLastError();
}

cudaError_t launch_randu(void* data, int dtype, int64_t n_local, int64_t global_offset,
                         uint64_t seed, double lo, double hi, cudaStream_t s) {
    if (n_local <= 0) return cudaSuccess;
    int grid = grid_for(n_local, 256);
    double span = hi - lo;
    switch (dtype) {
        case DT_F32: randu_kernel<float><<<grid, 256, 0, s>>>((float*)data, n_local, global_offset, seed, lo, span); break;
        case DT_F64: randu_kernel<double><<<grid, 256, 0, s>>>((double*)data, n_local, global_offset, seed, lo, span); break;
        case DT_I32: randu_kernel<int><<<grid, 256, 0, s>>>((int*)data, n_local, global_offset, seed, lo, span); break;
        default: randu_kernel<long long><<<grid, 256, 0, s>>>((long long*)data, n_local, global_offset, seed, lo, span); break;
    }
    return cudaGetLastError();
}

int dot_grid_size(int64_t n, int sm_count) {
    long long b = (n + 2047) / 2048;
    long long cap = (long long)(sm_count > 0 ? sm_count : 148) * 8;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

cudaError_t launch_dot(const void* a, const void* b, int64_t n, int dtype, void* partials,
                       unsigned int* counter, void* result, int grid, cudaStream_t s) {
    if (n < 0) n = 0;
    bool aligned = (((uintptr_t)a) & 15) == 0 && (!b || (((uintptr_t)b) & 15) == 0);
    if (dtype == DT_F64 && aligned) {
        if (b)
            dot_f64_vec_kernel<true><<<grid, 256, 0, s>>>((const double*)a, (const double*)b, n, (double*)partials, counter, (double*)result);
        else
            dot_f64_vec_kernel<false><<<grid, 256, 0, s>>>((const double*)a, nullptr, n, (double*)partials, counter, (double*)result);
        return cudaGetLastError();
    }
#define CN_DOT(T, ACC)                                                                         \
    if (b)                                                                                     \
        dot_kernel<T, ACC, true><<<grid, 256, 0, s>>>((const T*)a, (const T*)b, n, (ACC*)partials, counter, (T*)result); \
    else                                                                                       \
        dot_kernel<T, ACC, false><<<grid, 256, 0, s>>>((const T*)a, nullptr, n, (ACC*)partials, counter, (T*)result);
    switch (dtype) {
        case DT_F32: CN_DOT(float, double) break;
        case DT_F64: CN_DOT(double, double) break;
        case DT_I32: CN_DOT(int, long long) break;
        default: CN_DOT(long long, long long) break;
    }
#undef CN_DOT
    return cudaGetLastError();
}

cudaError_t launch_matvec(const void* A, int64_t lda, const void* x, void* y, int64_t rows,
                          int64_t cols, int dtype, cudaStream_t s) {
    if (rows <= 0) return cudaSuccess;
    bool aligned = (((uintptr_t)A) & 15) == 0 && (((uintptr_t)x) & 15) == 0 && (lda % 2 == 0) &&
                   (cols % 2 == 0);
    if (dtype == DT_F64 && aligned && rows < (1LL << 31) * MV_ROWS) {
        int grid = (int)((rows + MV_ROWS - 1) / MV_ROWS);
        matvec_f64_vec_kernel<<<grid, 256, 0, s>>>((const double*)A, lda, (const double*)x, (double*)y, rows, cols);
        return cudaGetLastError();
    }
    if (rows >= (1LL << 31)) return cudaErrorInvalidValue;
    int grid = (int)rows;
    switch (dtype) {
        case DT_F32: matvec_generic_kernel<float><<<grid, 256, 0, s>>>((const float*)A, lda, (const float*)x, (float*)y, rows, cols); break;
        case DT_F64: matvec_generic_kernel<double><<<grid, 256, 0, s>>>((const double*)A, lda, (const double*)x, (double*)y, rows, cols); break;
        case DT_I32: matvec_generic_kernel<int><<<grid, 256, 0, s>>>((const int*)A, lda, (const int*)x, (int*)y, rows, cols); break;
        default: matvec_generic_kernel<long long><<<grid, 256, 0, s>>>((const long long*)A, lda, (const long long*)x, (long long*)y, rows, cols); break;
    }
    return cudaGetLastError();
}

// ---- tile ---------------------------------------------------------------------------------------
namespace {

template <typename T>
__global__ void tile_kernel(T* dst, long long d1, long long d2, long long row0, long long n,
                            const T* src, long long s0, long long s1, long long s2) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const long long i2 = i % d2, t = i / d2;
        const long long i1 = t % d1, i0 = row0 + t / d1;
        dst[i] = src[((i0 % s0) * s1 + (i1 % s1)) * s2 + (i2 % s2)];
    }
}

}  // namespace

cudaError_t launch_tile(void* dst, const int64_t dst_shape[3], int64_t dst_row_begin, int64_t dst_rows,
                        const void* src, const int64_t src_shape[3], int dtype, cudaStream_t s) {
    const long long n = (long long)dst_rows * dst_shape[1] * dst_shape[2];
    if (n <= 0) return cudaSuccess;
    const int grid = grid_for(n, 256);
    if (dtype_size(dtype) == 8)
        tile_kernel<long long><<<grid, 256, 0, s>>>((long long*)dst, dst_shape[1], dst_shape[2], dst_row_begin, n,
                                                    (const long long*)src, src_shape[0], src_shape[1], src_shape[2]);
    else
        tile_kernel<int><<<grid, 256, 0, s>>>((int*)dst, dst_shape[1], dst_shape[2], dst_row_begin, n,
                                              (const int*)src, src_shape[0], src_shape[1], src_shape[2]);
    return cudaGetLastError();
}

// ---- halo exchange over peer mappings ---------------------------------------------------------
// Phase 1: all blocks store this rank's boundary rows into the neighbours' payload slots; each
// block fences, then draws a ticket, and the block with the last ticket publishes the payload
// with a release store of the epoch into the neighbours' flags.  Phase 2: every block waits
// (bounded) until the neighbours' rows for this epoch have arrived in this rank's own mailbox
// and copies them into the local halo rows.  The grid never exceeds one block per SM, so all
// blocks are resident and phase 1 always completes before anyone can wait for long.
namespace {

static_assert(sizeof(CnPeerBox) == 4096, "mailbox header is one page");

__device__ __forceinline__ char* halo_slot(void* box, int bank, int dir) {
    return (char*)box + sizeof(CnPeerBox) + (size_t)(bank * 2 + dir) * CN_PEER_HALO_SLOT;
}

__device__ __forceinline__ void halo_copy(char* dst, const char* src, size_t bytes, bool vec16) {
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nth = (size_t)gridDim.x * blockDim.x;
    if (vec16) {
        const size_t n = bytes / 16;
        for (size_t i = tid; i < n; i += nth) ((int4*)dst)[i] = ((const int4*)src)[i];
    } else {
        const size_t n = bytes / 8;
        for (size_t i = tid; i < n; i += nth) ((long long*)dst)[i] = ((const long long*)src)[i];
    }
}

__device__ __forceinline__ void halo_unpack(char* dst, const char* src, size_t bytes, bool vec16) {
    // the payload was written by another GPU: read it past L1
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nth = (size_t)gridDim.x * blockDim.x;
    if (vec16) {
        for (size_t i = tid; i < bytes / 16; i += nth) ((int4*)dst)[i] = __ldcv(((const int4*)src) + i);
    } else {
        for (size_t i = tid; i < bytes / 8; i += nth) ((long long*)dst)[i] = __ldcv(((const long long*)src) + i);
    }
}

__global__ void __launch_bounds__(256) halo_exchange_kernel(HaloArgs h, int vec_push, int vec_pull) {
    __shared__ int arrived;
    const int bp = (int)(h.epoch_prev & 1ULL), bn = (int)(h.epoch_next & 1ULL);
    // rows for the rank below arrive there "from above" (dir 1), and the other way round
    if (!h.pull_only) {
        size_t off = 0;
        for (int q = 0; q < h.nparts; ++q) {
            if (h.box_prev) halo_copy(halo_slot(h.box_prev, bp, 1) + off, h.first_rows[q], h.bytes[q], vec_push != 0);
            if (h.box_next) halo_copy(halo_slot(h.box_next, bn, 0) + off, h.last_rows[q], h.bytes[q], vec_push != 0);
            off += (h.bytes[q] + 15) & ~(size_t)15;
        }
    }
    __syncthreads();
    // One thread per block orders the block's stores (the barrier makes them its predecessors)
    // before its ticket; the release stores of the last ticket holder then publish everything.
    if (threadIdx.x == 0) {
        int last = 1;
        if (h.pull_only) {
            // the payload was stored and fenced by earlier kernels of this stream
            last = blockIdx.x == 0 ? 1 : 0;
            if (last) __threadfence_system();
        } else if (gridDim.x > 1) {
            __threadfence_system();
            last = atomicAdd(h.ticket, 1u) == gridDim.x - 1 ? 1 : 0;
        }
        if (last) {
            if (h.box_prev) cn_st_release_sys(&((CnPeerBox*)h.box_prev)->halo_flag[bp][1], h.epoch_prev);
            if (h.box_next) cn_st_release_sys(&((CnPeerBox*)h.box_next)->halo_flag[bn][0], h.epoch_next);
            if (gridDim.x > 1 && !h.pull_only) *h.ticket = 0u;
        }
        CnPeerBox* me = (CnPeerBox*)h.me;
        bool ok = true;
        const unsigned int limit = h.wait_limit ? h.wait_limit : CN_PEER_WAIT_LIMIT;
        if (h.box_prev) ok = cn_peer_wait(&me->halo_flag[bp][0], h.epoch_prev, limit) && ok;
        if (h.box_next) ok = cn_peer_wait(&me->halo_flag[bn][1], h.epoch_next, limit) && ok;
        arrived = ok ? 1 : 0;
        if (!ok && h.error) atomicExch(h.error, 2u);
    }
    __syncthreads();
    if (!arrived) return;
    size_t off = 0;
    for (int q = 0; q < h.nparts; ++q) {
        if (h.box_prev && h.halo_below[q]) halo_unpack(h.halo_below[q], halo_slot(h.me, bp, 0) + off, h.bytes[q], vec_pull != 0);
        if (h.box_next && h.halo_above[q]) halo_unpack(h.halo_above[q], halo_slot(h.me, bn, 1) + off, h.bytes[q], vec_pull != 0);
        off += (h.bytes[q] + 15) & ~(size_t)15;
    }
}

}  // namespace

cudaError_t launch_halo_exchange(const HaloArgs& h, int sm_count, cudaStream_t s) {
    if (h.nparts < 1 || h.nparts > CN_HALO_PARTS) return cudaErrorInvalidValue;
    size_t total = 0, largest = 0;
    bool vec_push = true, vec_pull = true;
    for (int q = 0; q < h.nparts; ++q) {
        if (h.bytes[q] % 8) return cudaErrorInvalidValue;
        total += (h.bytes[q] + 15) & ~(size_t)15;
        largest = std::max(largest, h.bytes[q]);
        vec_push = vec_push && !h.pull_only && h.bytes[q] % 16 == 0 &&
                   (((uintptr_t)h.first_rows[q] | (uintptr_t)h.last_rows[q]) & 15) == 0;
        vec_pull = vec_pull && h.bytes[q] % 16 == 0 && (((uintptr_t)h.halo_below[q] | (uintptr_t)h.halo_above[q]) & 15) == 0;
    }
    if (largest == 0 || (!h.box_prev && !h.box_next)) return cudaSuccess;
    if (total > CN_PEER_HALO_SLOT) return cudaErrorInvalidValue;
    long long blocks = (long long)((largest + 256 * 64 - 1) / (256 * 64));  // 64 bytes per thread
    int grid = (int)std::max<long long>(1, std::min<long long>(blocks, sm_count > 0 ? sm_count : 148));
    halo_exchange_kernel<<<grid, 256, 0, s>>>(h, vec_push ? 1 : 0, vec_pull ? 1 : 0);
    return cudaGetLastError();
}

}  // namespace cn
