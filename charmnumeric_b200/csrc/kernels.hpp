// Launchers of the ahead-of-time CUDA kernels (kernels.cu).  Every launcher enqueues on
// the given stream and returns the CUDA status of the launch; none synchronises.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace cn {

struct StridedView {  // element offset + element stride per iteration dimension
    int64_t off = 0;
    int64_t str[3] = {0, 0, 0};
};

// SET_REGION with a literal right-hand side (src/executor_ast_visitor.cpp:112-197).
cudaError_t launch_fill_region(void* base, int dtype, const StridedView& v, const int64_t ext[3],
                               double value, cudaStream_t s);
// Strided region copy (src/executor_ast_visitor.cpp:199-314): dst[view] = src[view].
cudaError_t launch_copy_region(void* dst, const StridedView& dv, const void* src,
                               const StridedView& sv, const int64_t ext[3], int dtype,
                               cudaStream_t s);
// Seeded uniform fill: element with global linear index g gets lo + (hi-lo)*u(seed, g).
cudaError_t launch_randu(void* data, int dtype, int64_t n_local, int64_t global_offset,
                         uint64_t seed, double lo, double hi, cudaStream_t s);
// result[0] = sum_i a[i]*b[i]   (b == nullptr: sum_i a[i]); deterministic two-pass finish.
// `partials` needs dot_grid_size(n) accumulators, `counter` is a zeroed ticket.
int dot_grid_size(int64_t n, int sm_count);
cudaError_t launch_dot(const void* a, const void* b, int64_t n, int dtype, void* partials,
                       unsigned int* counter, void* result, int grid, cudaStream_t s);
// y[r] = sum_c A[r*lda + c] * x[c] for r in [0, rows): row-block gemv of the local slab
// (src/backend_internal.hpp:15-41, src/execute_node.cpp:206-229).
cudaError_t launch_matvec(const void* A, int64_t lda, const void* x, void* y, int64_t rows,
                          int64_t cols, int dtype, cudaStream_t s);

// TILE (charmnumeric/operations.py:52-72): dst[i0,i1,i2] = src[i0 % s0, i1 % s1, i2 % s2] for
// the local rows of dst (shapes right-aligned into three dimensions; src is the whole array).
cudaError_t launch_tile(void* dst, const int64_t dst_shape[3], int64_t dst_row_begin, int64_t dst_rows,
                        const void* src, const int64_t src_shape[3], int dtype, cudaStream_t s);

// Halo exchange through the peer mailboxes (takes the place of the per-edge messages of
// src/executor_core.cpp:7-143 and PartitionImpl::receive_data, src/partition_comm.cpp:25-61).
// Rows are 8-byte multiples; pointers of absent neighbours are null.
// One exchange can carry the halo rows of up to CN_HALO_PARTS arrays of one row partition (CG
// needs r and p at once): their rows lie one behind the other in the payload slot.
#define CN_HALO_PARTS 4
struct HaloArgs {
    int nparts = 1;
    const char* first_rows[CN_HALO_PARTS] = {nullptr};  // this rank's first `halo` rows (go to the rank below)
    const char* last_rows[CN_HALO_PARTS] = {nullptr};   // this rank's last `halo` rows (go to the rank above)
    char* halo_below[CN_HALO_PARTS] = {nullptr};        // local halo rows filled from the rank below
    char* halo_above[CN_HALO_PARTS] = {nullptr};        // local halo rows filled from the rank above
    size_t bytes[CN_HALO_PARTS] = {0};                  // bytes per direction of each part
    void* me = nullptr;                // this rank's mailbox
    void* box_prev = nullptr;          // mailbox of rank - 1 as mapped here (null: none)
    void* box_next = nullptr;          // mailbox of rank + 1 as mapped here (null: none)
    // exchanges are counted per neighbour pair (both sides count alike); the parity picks the bank
    unsigned long long epoch_prev = 0, epoch_next = 0;
    unsigned int* ticket = nullptr;    // zeroed block counter, left at zero
    unsigned int* error = nullptr;     // device error word
    unsigned int wait_limit = 0;       // polls before a wait gives up (0: the default bound)
    // The payload is already in the neighbours' mailboxes (the kernels that produced the rows
    // stored it there): publish it, wait for the neighbours' rows, copy them in.  Parts whose
    // halo pointers are null are waited for but not copied.
    bool pull_only = false;
};
cudaError_t launch_halo_exchange(const HaloArgs& h, int sm_count, cudaStream_t s);

}  // namespace cn
