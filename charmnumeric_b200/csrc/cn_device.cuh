// Device-side support header shared by the ahead-of-time kernels (nvcc) and by every
// kernel the DAG-group compiler generates at run time (NVRTC receives this text verbatim).
// It must therefore compile without any standard or CUDA toolkit header.
//
// Contents: the launch-argument block of a fused group kernel, the exp/tanh routines,
// and the block / grid reduction helpers with the deterministic last-block finish.
#ifndef CN_DEVICE_CUH
#define CN_DEVICE_CUH

#define CN_MAX_IN 16
#define CN_MAX_OUT 8
#define CN_MAX_BC 8
#define CN_MAX_SC 16
#define CN_MAX_RED 4
#define CN_MAX_SOUT 4
#ifndef CN_BLOCK
#define CN_BLOCK 256  // threads per block; a generated kernel may be compiled for another size
#endif
#define CN_MAX_PEERS 8
#define CN_PEER_HALO_SLOT (16u << 20)  // bytes per (bank, direction) halo payload slot

// Mailbox of one rank, in that rank's own device memory; the other ranks of the box write
// into it over NVLink through peer mappings.  Two banks alternate by epoch parity: a rank
// can only reach epoch e+2 after every partner has consumed epoch e, so nothing is
// overwritten while it is still being read.  The halo payload follows the header:
// slot (bank, dir) starts at byte 4096 + (bank * 2 + dir) * CN_PEER_HALO_SLOT, dir 0 = rows
// that came from the rank below (rank - 1), dir 1 = from the rank above.
struct CnPeerBox {
    unsigned long long red_val[2][CN_MAX_RED][CN_MAX_PEERS];  // [bank][reduction][source rank]
    unsigned long long red_flag[2][CN_MAX_PEERS];             // epoch of the values of a source rank
    unsigned long long halo_flag[2][2];                       // [bank][dir]: epoch of the payload
    unsigned long long pad[(4096 - 8 * (2 * CN_MAX_RED * CN_MAX_PEERS + 2 * CN_MAX_PEERS + 4)) / 8];
};

// Launch arguments of one fused group kernel.  The same layout is used by the host
// (it fills the block) and by the generated source (it reads it), so only plain types.
struct
#if defined(__CUDACC__) || defined(__GNUC__)
    __attribute__((aligned(64)))
#endif
    CnGroupArgs {
    unsigned char tmap[128];     // staged kernels: TMA descriptor of the stencil array (64-byte aligned)
    const void* in[CN_MAX_IN];   // array leaves: address of local element (0,0,0)
    void* out[CN_MAX_OUT];       // outputs: address of local element (0,0,0) of the buffer written
    const void* old[CN_MAX_OUT]; // previous contents of each output array
    const void* bc[CN_MAX_BC];   // size-1 arrays read as scalars
    void* sout[CN_MAX_SOUT];     // size-1 arrays written by scalar roots
    double sc[CN_MAX_SC];        // literal scalars, cast to the element type in the kernel
    long long lo[3], hi[3];      // iteration box [lo,hi) in the frame's local coordinates
    long long rlo[3], rhi[3];    // region box: where SET_REGION outputs are computed
    long long stride[3];         // element strides of the common array shape (shifted class)
    long long in_off[CN_MAX_IN];     // strided class: element offset of each leaf view
    long long in_str[CN_MAX_IN][3];  // strided class: element stride per iteration dim
    long long out_off[CN_MAX_OUT];
    long long out_str[CN_MAX_OUT][3];
    long long ext[3];            // strided class: iteration extents
    long long ntiles;            // number of tiles the persistent blocks walk over
    long long ntx, nty;          // tiles along the last and the second-to-last dimension
    double* partials;            // [CN_MAX_RED][gridDim.x] per-block partial sums
    unsigned int* counter;       // ticket for the last-block finish (left at 0 on exit)
    void* red[CN_MAX_RED];       // reduction results (size-1 arrays)
    long long nzc, zchunk;       // staged 3-D kernels: number and length of the z chunks marched
    long long tm_off[3];         // staged kernels: local coordinate -> descriptor coordinate offset
    long long own_lo, own_hi;    // rows (planes) of dimension 0 this rank owns: reductions count those only,
                                 // also when the sweep is widened into the halo rows
    // edge rows pushed by the producing kernel: outputs in push_mask also store their first
    // push_elems elements (the rows next to rank - 1) at push_prev and their last push_elems
    // elements (starting at local element push_last) at push_next, both in the neighbours'
    // mailboxes (null: no such neighbour); one array per output slot
    void* push_prev[CN_MAX_OUT];
    void* push_next[CN_MAX_OUT];
    long long push_elems, push_last;
    unsigned int push_mask, push_pad;
    long long fill_lo[2], fill_hi[2];  // staged producers: local rows / columns of the producer's inputs that hold data
    unsigned int* error;         // device error word (set when a bounded wait runs out)
    // fused cross-GPU reduction: every rank's mailbox as mapped on this GPU (peer_n = 0: off)
    void* peer_box[CN_MAX_PEERS];
    int peer_rank, peer_n;
    unsigned long long peer_epoch;
};

#ifdef __CUDACC__

#include "cn_exp_table.inc"

__device__ const double cn_exp_hi[64] = {CN_EXP_TABLE_HI};
__device__ const double cn_exp_lo[64] = {CN_EXP_TABLE_LO};
__device__ const double2 cn_exp_pair[64] = {CN_EXP_TABLE_PAIRS};  // {hi, lo}: one 128-bit load

// 2^m * v for v in [1, 4): one exponent-field add when the result stays normal, two
// exact power-of-two multiplies otherwise (gradual underflow / overflow to inf).
__device__ __forceinline__ double cn_scale2(double v, int m) {
    if (m >= -1000 && m <= 1000) {
        long long bits = __double_as_longlong(v) + ((long long)m << 52);
        return __longlong_as_double(bits);
    }
    int m1 = m / 2, m2 = m - m1;
    double p1 = __longlong_as_double((long long)(m1 + 1023) << 52);
    double p2 = __longlong_as_double((long long)(m2 + 1023) << 52);
    return (v * p1) * p2;
}

// exp(x) = 2^m * 2^(j/64) * e^r with |r| <= ln2/128; degree-5 polynomial for e^r - 1.
// Every step is an explicitly rounded IEEE operation (fma / mul / add), so the host
// restatement that performs the same steps with C fma() gives identical bits.
static __device__ __noinline__ double cn_exp_slow(double x) {
    if (!(x == x)) return x;
    if (x > 709.782712893384) return __longlong_as_double(0x7ff0000000000000LL);
    if (x < -745.1332191019412) return 0.0;
    const double shift = 6755399441055744.0;  // 1.5 * 2^52
    double t = __fma_rn(x, CN_INV_LN2_64, shift);
    int ki = (int)(unsigned int)(__double_as_longlong(t) & 0xffffffffLL);
    double kd = t - shift;
    double r = __fma_rn(-kd, CN_LN2_64_HI, x);
    r = __fma_rn(-kd, CN_LN2_64_LO, r);
    int j = ki & 63;
    int m = ki >> 6;
    double p = __fma_rn(r, 0x1.1111111111111p-7, 0x1.5555555555555p-5);  // 1/120, 1/24
    p = __fma_rn(p, r, 0x1.5555555555555p-3);                            // 1/6
    p = __fma_rn(p, r, 0.5);
    double q = __fma_rn(p, r * r, r);                                     // e^r - 1
    double hi = cn_exp_hi[j], lo = cn_exp_lo[j];
    double v = hi + __fma_rn(hi, q, lo);
    return cn_scale2(v, m);
}

// Same steps as cn_exp_slow, minus everything that cannot happen for |x| < 708: no NaN /
// overflow / underflow tests (one integer compare on the high word sends those to the slow
// routine), the scale is a plain add to the exponent field, hi and lo come in one load.
__device__ __forceinline__ double cn_exp(double x) {
    if ((__double2hiint(x) & 0x7fffffff) >= 0x40862000) return cn_exp_slow(x);
    const double shift = 6755399441055744.0;
    double t = __fma_rn(x, CN_INV_LN2_64, shift);
    int ki = __double2loint(t);
    double kd = t - shift;
    double r = __fma_rn(-kd, CN_LN2_64_HI, x);
    r = __fma_rn(-kd, CN_LN2_64_LO, r);
    double p = __fma_rn(r, 0x1.1111111111111p-7, 0x1.5555555555555p-5);
    p = __fma_rn(p, r, 0x1.5555555555555p-3);
    p = __fma_rn(p, r, 0.5);
    double q = __fma_rn(p, r * r, r);
    const double2 tab = cn_exp_pair[ki & 63];
    double v = tab.x + __fma_rn(tab.x, q, tab.y);
    return __hiloint2double(__double2hiint(v) + ((ki >> 6) << 20), __double2loint(v));
}

// expm1(y) for 0 <= y <= 1.1 with the same reduction; (hi*2^m - 1) is exact there.
__device__ __forceinline__ double cn_expm1_small(double y) {
    const double shift = 6755399441055744.0;
    double t = __fma_rn(y, CN_INV_LN2_64, shift);
    int ki = (int)(unsigned int)(__double_as_longlong(t) & 0xffffffffLL);
    double kd = t - shift;
    double r = __fma_rn(-kd, CN_LN2_64_HI, y);
    r = __fma_rn(-kd, CN_LN2_64_LO, r);
    int j = ki & 63;
    int m = ki >> 6;
    // two more terms than exp: the result is small, so the absolute error must be too
    double p = __fma_rn(r, 0x1.a01a01a01a01ap-13, 0x1.6c16c16c16c17p-10);  // 1/5040, 1/720
    p = __fma_rn(p, r, 0x1.1111111111111p-7);
    p = __fma_rn(p, r, 0x1.5555555555555p-5);
    p = __fma_rn(p, r, 0x1.5555555555555p-3);
    p = __fma_rn(p, r, 0.5);
    double q = __fma_rn(p, r * r, r);
    double sc = (m == 0) ? 1.0 : ((m == 1) ? 2.0 : 4.0);
    double hi = cn_exp_hi[j] * sc, lo = cn_exp_lo[j] * sc;
    return (hi - 1.0) + __fma_rn(hi, q, lo);
}

__device__ __forceinline__ double cn_tanh(double x) {
    if (!(x == x)) return x;
    double ax = x < 0 ? -x : x;
    double r;
    if (ax >= 22.0) {
        r = 1.0;
    } else if (ax >= 0.5) {
        double e = cn_exp(2.0 * ax);
        r = 1.0 - 2.0 / (e + 1.0);
    } else if (ax >= 0x1p-28) {
        double em1 = cn_expm1_small(2.0 * ax);
        r = em1 / (em1 + 2.0);
    } else {
        r = ax;
    }
    return x < 0 ? -r : r;
}

// ---- reductions -------------------------------------------------------------------
// Fixed-shape tree: xor-shuffle inside each warp, then warp 0 folds the per-warp sums
// in lane order.  The same block size always gives the same association order.
template <typename A>
__device__ __forceinline__ A cn_warp_sum(A v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename A>
__device__ __forceinline__ A cn_block_sum(A v, A* smem /* >= 32 entries */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = cn_warp_sum(v);
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    A t = (threadIdx.x < nwarp) ? smem[threadIdx.x] : (A)0;
    if (warp == 0) t = cn_warp_sum(t);
    return t;  // valid in thread 0
}

// Deterministic two-pass finish inside one launch: every block stores its partials, then
// draws a ticket; the block that draws the last ticket re-reads all partials in index
// order and writes the totals.  No block waits on another, and the ticket counter is
// put back to 0 for the next launch.  Returns true in every thread of the last block.
__device__ __forceinline__ bool cn_grid_ticket(unsigned int* counter, int* flag_shared) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int ticket = atomicAdd(counter, 1u);
        *flag_shared = (ticket == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    bool last = (*flag_shared != 0);
    if (last) __threadfence();
    return last;
}

template <typename A>
__device__ __forceinline__ A cn_sum_partials(const A* partials, A* smem) {
    A v = (A)0;
    for (unsigned int i = threadIdx.x; i < gridDim.x; i += blockDim.x)
        v += ((const volatile A*)partials)[i];
    return cn_block_sum(v, smem);  // valid in thread 0
}

// ---- cross-GPU exchange through peer mailboxes (NVLink loads / stores, no multicast) ----------
// Every wait on a flag that another GPU writes is bounded: CN_PEER_WAIT_LIMIT polls with a
// short sleep in between (two to three seconds in all), after which the caller records the
// failure in the error word and carries on with what it has.
#ifndef CN_PEER_WAIT_LIMIT
#define CN_PEER_WAIT_LIMIT 4000000u
#endif

// First statement of every generated kernel.  When the kernel was launched with programmatic
// stream serialisation, its launch is released as soon as the blocks of the previous kernel of
// the stream have exited (or, with CN_TRIGGER, as soon as they have all started) instead of
// after that kernel has drained; `wait` returns once the previous kernel has completed and
// its writes are visible.  Nothing before this point touches global memory.  Without the
// launch attribute both instructions do nothing.
#ifndef CN_TRIGGER
#define CN_TRIGGER 0
#endif
__device__ __forceinline__ void cn_stream_dependency() {
#if CN_TRIGGER
    asm volatile("griddepcontrol.launch_dependents;");
#endif
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void cn_st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ unsigned long long cn_ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// true once *flag >= epoch; false when the bound ran out
__device__ __forceinline__ bool cn_peer_wait(const unsigned long long* flag, unsigned long long epoch,
                                             unsigned int limit = CN_PEER_WAIT_LIMIT) {
    for (unsigned int i = 0; i < limit; ++i) {
        if (cn_ld_acquire_sys(flag) >= epoch) return true;
        __nanosleep(40);
    }
    return false;
}

__device__ __forceinline__ unsigned long long cn_bits(double v) { return (unsigned long long)__double_as_longlong(v); }
__device__ __forceinline__ unsigned long long cn_bits(long long v) { return (unsigned long long)v; }
__device__ __forceinline__ void cn_unbits(unsigned long long b, double* v) { *v = __longlong_as_double((long long)b); }
__device__ __forceinline__ void cn_unbits(unsigned long long b, long long* v) { *v = (long long)b; }

// Sum of `n` per-rank totals over all ranks, inside the kernel that produced them.  Called by
// every thread of the one block that finished the local reduction; `tv` holds this rank's
// totals in thread 0 on entry and the global totals in thread 0 on return.  Thread r stores
// the totals into rank r's mailbox and publishes them with a release store of the epoch, then
// waits for rank r's totals to arrive in this rank's own mailbox; thread 0 adds them in rank
// order, so every rank computes bit-identical results.
template <typename A>
__device__ __forceinline__ void cn_peer_allreduce(const CnGroupArgs& a, A* tv, int n, A* smem) {
    __syncthreads();
    if (threadIdx.x == 0)
        for (int q = 0; q < n; ++q) smem[q] = tv[q];
    __syncthreads();
    const int bank = (int)(a.peer_epoch & 1ULL);
    CnPeerBox* const me = (CnPeerBox*)a.peer_box[a.peer_rank];
    bool ok = true;
    if ((int)threadIdx.x < a.peer_n) {
        CnPeerBox* const dst = (CnPeerBox*)a.peer_box[threadIdx.x];
        for (int q = 0; q < n; ++q)
            *(volatile unsigned long long*)&dst->red_val[bank][q][a.peer_rank] = cn_bits(smem[q]);
        cn_st_release_sys(&dst->red_flag[bank][a.peer_rank], a.peer_epoch);
        ok = cn_peer_wait(&me->red_flag[bank][threadIdx.x], a.peer_epoch);
    }
    if (__syncthreads_or(ok ? 0 : 1)) {
        if (threadIdx.x == 0 && a.error) atomicExch(a.error, 2u);
        return;  // the local totals stay in tv
    }
    if (threadIdx.x == 0) {
        for (int q = 0; q < n; ++q) {
            A s = (A)0;
            for (int r = 0; r < a.peer_n; ++r) {
                A v;
                cn_unbits(*(volatile unsigned long long*)&me->red_val[bank][q][r], &v);
                s += v;
            }
            tv[q] = s;
        }
    }
}

// ---- TMA / mbarrier helpers (sm_100a) -----------------------------------------------------
// Tiles of the stencil array are fetched by the TMA unit into a ring of shared-memory
// slots; one mbarrier per slot counts the bytes that arrive.  Every wait is bounded: when
// the bound runs out the kernel records it in the error word and leaves.
#ifndef CN_WAIT_LIMIT
#define CN_WAIT_LIMIT 2000000u
#endif
// Test hook: with CN_DEBUG_DROP_COPIES the elected thread issues no tile copy at all, so every
// consumer's bounded wait runs out.  Nothing is left in flight and nothing faults; it only
// exists to exercise the error path (error word -> status code at the next synchronise).
#ifndef CN_DEBUG_DROP_COPIES
#define CN_DEBUG_DROP_COPIES 0
#endif

__device__ __forceinline__ unsigned int cn_smem_addr(const void* p) {
    return (unsigned int)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cn_mbar_init(unsigned long long* bar, unsigned int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(cn_smem_addr(bar)), "r"(count));
}

__device__ __forceinline__ void cn_mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void cn_mbar_expect_tx(unsigned long long* bar, unsigned int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(cn_smem_addr(bar)),
                 "r"(bytes)
                 : "memory");
}

// true when the phase with the given parity has completed; false when the bound ran out.
// Each poll may suspend the thread for at most about CN_WAIT_HINT_NS (the hint operand of
// try_wait), so the whole wait is bounded by roughly CN_WAIT_LIMIT * CN_WAIT_HINT_NS.
#define CN_WAIT_HINT_NS 2000u
__device__ __forceinline__ bool cn_mbar_wait(unsigned long long* bar, unsigned int parity) {
    const unsigned int addr = cn_smem_addr(bar);
    for (unsigned int i = 0; i < CN_WAIT_LIMIT; ++i) {
        unsigned int done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(CN_WAIT_HINT_NS)
            : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ void cn_tma_load_2d(void* dst, const void* tmap, int x, int y,
                                               unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(cn_smem_addr(dst)), "l"(tmap), "r"(x), "r"(y), "r"(cn_smem_addr(bar))
        : "memory");
}

__device__ __forceinline__ void cn_tma_load_3d(void* dst, const void* tmap, int x, int y, int z,
                                               unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(cn_smem_addr(dst)), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(cn_smem_addr(bar))
        : "memory");
}

#endif  // __CUDACC__
#endif  // CN_DEVICE_CUH
