// Conjugate gradients with a fixed iteration count, driven from inside the library.
//
// One iteration is four launches and no host round trip:
//   Ap = A p                                   (the SpMV forward entry point of this library)
//   pAp = <Ap, p>                              (cg_dot_kernel)
//   alpha = rz / pAp;  x += alpha p;  r -= alpha Ap;  rz' = <r, r>;  hist = sqrt(rz')   (cg_update_kernel)
//   beta = rz' / rz;   p = r + beta p                                                    (cg_direction_kernel)
// The scalars live in device memory and are consumed by the next kernel directly, so nothing is read
// back until the caller looks at the result.  Dot products are reduced in double in a fixed order
// (per-block partial sums, summed by the last block to finish), hence reproducible from run to run.
//
// The recurrence is the reference's unpreconditioned loop with its stopping rule disabled
// (rtol = 0 and an iteration count: the rule can never fire).
#include "primitives.cuh"

namespace nb200 {

constexpr int kCgThreads = 256;
constexpr int kCgBlocks = kSMs * 4;

// scalar slots (doubles): [0], [1] r.r of even / odd iterations; [2] <Ap, p>; counters are separate
struct CgScalars { double rz[2]; double pAp; };

// Block partial -> partials[blockIdx]; the last block to arrive adds them up in index order.
__device__ __forceinline__ bool block_partial_then_last(double v, double* partials, unsigned* counter, double* total) {
    __shared__ double ws[kCgThreads / 32];
    __shared__ bool is_last;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        double s = 0;
        for (int w = 0; w < kCgThreads / 32; ++w) s += ws[w];
        partials[blockIdx.x] = s;
        __threadfence();
        is_last = atomicAdd(counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) return false;
    // last block: fixed-order sum of all partials
    double s = 0;
    for (unsigned i = threadIdx.x; i < gridDim.x; i += kCgThreads) s += __ldcg(partials + i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0;
        for (int w = 0; w < kCgThreads / 32; ++w) t += ws[w];
        *total = t;
        *counter = 0;   // ready for the next reduction
    }
    return true;
}

template <typename T>
__global__ void __launch_bounds__(kCgThreads)
cg_dot_kernel(int64_t n, const T* __restrict__ a, const T* __restrict__ b, double* partials, unsigned* counter, double* out) {
    double s = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) s += (double)a[i] * (double)b[i];
    double total;
    if (block_partial_then_last(s, partials, counter, &total) && threadIdx.x == 0) *out = total;
}

// r = b - Ax0 (or r = b), p = r, rz[0] = <r, r>, hist[0] = sqrt(rz)
template <typename T>
__global__ void __launch_bounds__(kCgThreads)
cg_init_kernel(int64_t n, const T* __restrict__ b, const T* __restrict__ Ax0, T* __restrict__ x, T* __restrict__ r,
               T* __restrict__ p, double* partials, unsigned* counter, CgScalars* sc, T* __restrict__ hist) {
    double s = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        T ri = b[i];
        if (Ax0) ri -= Ax0[i]; else x[i] = (T)0;
        r[i] = ri;
        p[i] = ri;
        s += (double)ri * (double)ri;
    }
    double total;
    if (block_partial_then_last(s, partials, counter, &total) && threadIdx.x == 0) {
        sc->rz[0] = total;
        hist[0] = (T)sqrt(total);
    }
}

template <typename T>
__global__ void __launch_bounds__(kCgThreads)
cg_update_kernel(int64_t n, int it, const T* __restrict__ p, const T* __restrict__ Ap, T* __restrict__ x,
                 T* __restrict__ r, double* partials, unsigned* counter, CgScalars* sc, T* __restrict__ hist) {
    // an exactly zero residual means the solve has converged (the reference's loop stops there): the
    // remaining iterations must leave x and r as they are instead of forming 0 / 0
    const double rz_now = sc->rz[it & 1];
    const T alpha = rz_now == 0.0 ? (T)0 : (T)(rz_now / sc->pAp);
    double s = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        x[i] = x[i] + alpha * p[i];
        const T ri = r[i] - alpha * Ap[i];
        r[i] = ri;
        s += (double)ri * (double)ri;
    }
    double total;
    if (block_partial_then_last(s, partials, counter, &total) && threadIdx.x == 0) {
        sc->rz[(it + 1) & 1] = total;
        hist[it + 1] = (T)sqrt(total);
    }
}

template <typename T>
__global__ void __launch_bounds__(kCgThreads)
cg_direction_kernel(int64_t n, int it, const T* __restrict__ r, T* __restrict__ p, const CgScalars* sc) {
    const double rz_old = sc->rz[it & 1];
    const T beta = rz_old == 0.0 ? (T)0 : (T)(sc->rz[(it + 1) & 1] / rz_old);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = r[i] + beta * p[i];
}

// ---------------------------------------------------------------------------------------------
// Row-partitioned CG: the same recurrence with every rank holding a block of rows.  The SpMV of an
// iteration is the caller's business (a halo exchange and the local kernels); the phases below are the
// rest of it.  A dot product is reduced across ranks through peer memory: the last block of the kernel
// that forms the local sum stores it into this rank's exchange buffer and raises a sequence flag
// (release, system scope); the next kernel of every rank begins by waiting, with a cycle budget, for
// the flags of all ranks, reads their sums with ordinary loads over NVLink and adds them in rank order,
// so every rank obtains the same bits and no collective call sits between the kernels.  The two halves
// of the scalar area alternate by sequence number; a half is rewritten two reductions later, by which
// time every rank has been seen publishing the reduction in between, i.e. has finished reading it.
// ---------------------------------------------------------------------------------------------
struct PeerReduce {
    int world, rank;
    const int64_t* table;     // device array, per rank: address of its scalar area (2 halves of 4 doubles), address of its flag
    int* seq;                 // device word of this rank: sequence number of the last reduction it published
    long long budget;
    int32_t* status;
};

__device__ __forceinline__ int cg_ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Last block of a reduction: publish this rank's sum as reduction number *seq + 1.
__device__ __forceinline__ void peer_publish(const PeerReduce& red, double local_sum) {
    const int q = *red.seq + 1;
    double* area = reinterpret_cast<double*>(red.table[2 * red.rank]);
    int* flag = reinterpret_cast<int*>(red.table[2 * red.rank + 1]);
    area[(q & 1) * 4] = local_sum;
    *red.seq = q;
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" :: "l"(flag), "r"(q) : "memory");
}

// Start of the kernel that needs the total: every block adds the ranks' sums of reduction *seq in rank
// order.  Returns NaN (and records the failure) if some rank's flag does not arrive within the budget.
__device__ __forceinline__ double peer_total(const PeerReduce& red) {
    __shared__ double s_total;
    if (threadIdx.x < 32) {
        const int q = *red.seq;
        const int lane = threadIdx.x;
        double mine = 0.0;
        bool ok = true;
        for (int r = lane; r < red.world; r += 32) {
            const int* flag = reinterpret_cast<const int*>(red.table[2 * r + 1]);
            if (cg_ld_acquire_sys(flag) < q) {
                const long long t0 = clock64();
                while (cg_ld_acquire_sys(flag) < q) {
                    if (clock64() - t0 > red.budget) { ok = false; break; }
                    __nanosleep(64);
                }
            }
            if (ok && red.world <= 32) mine = __ldcv(reinterpret_cast<const double*>(red.table[2 * r]) + (q & 1) * 4);
        }
        ok = __all_sync(0xffffffffu, ok);
        double total = 0.0;
        for (int r = 0; r < red.world && r < 32; ++r) total += __shfl_sync(0xffffffffu, mine, r);   // rank order
        if (!ok) {
            total = __longlong_as_double(0x7ff8000000000000LL);
            if (lane == 0 && red.status) atomicExch(red.status, (int)NB200_ERR_WAIT_BUDGET);
        }
        if (lane == 0) s_total = total;
    }
    __syncthreads();
    return s_total;
}

// scalars of the partitioned solve: rz of even / odd iterations (totals), the iteration counter
struct CgPeerState { double rz[2]; int it; int pad; };

template <typename T>
__global__ void __launch_bounds__(kCgThreads)
cg_peer_init_kernel(int64_t n, const T* __restrict__ b, T* __restrict__ x, T* __restrict__ r, T* __restrict__ p,
                    double* partials, unsigned* counter, CgPeerState* st, PeerReduce red) {
    double s = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const T ri = b[i];
        x[i] = (T)0; r[i] = ri; p[i] = ri;
        s += (double)ri * (double)ri;
    }
    double total;
    if (block_partial_then_last(s, partials, counter, &total) && threadIdx.x == 0) {
        st->it = 0;
        peer_publish(red, total);
    }
}

// consumes the reduction of the initial residual: rz[0] and the first history entry
template <typename T>
__global__ void __launch_bounds__(kCgThreads)
cg_peer_start_kernel(CgPeerState* st, T* __restrict__ hist, PeerReduce red) {
    const double total = peer_total(red);
    if (threadIdx.x == 0) { st->rz[0] = total; hist[0] = (T)sqrt(total); }
}

template <typename T>
__global__ void __launch_bounds__(kCgThreads)
cg_peer_dot_kernel(int64_t n, const T* __restrict__ a, const T* __restrict__ b, double* partials, unsigned* counter,
                   PeerReduce red) {
    double s = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) s += (double)a[i] * (double)b[i];
    double total;
    if (block_partial_then_last(s, partials, counter, &total) && threadIdx.x == 0) peer_publish(red, total);
}

template <typename T>
__global__ void __launch_bounds__(kCgThreads)
cg_peer_update_kernel(int64_t n, const T* __restrict__ p, const T* __restrict__ Ap, T* __restrict__ x, T* __restrict__ r,
                      double* partials, unsigned* counter, const CgPeerState* st, PeerReduce red) {
    const double pAp = peer_total(red);
    const double rz_now = st->rz[st->it & 1];
    const T alpha = rz_now == 0.0 ? (T)0 : (T)(rz_now / pAp);
    double s = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        x[i] = x[i] + alpha * p[i];
        const T ri = r[i] - alpha * Ap[i];
        r[i] = ri;
        s += (double)ri * (double)ri;
    }
    double total;
    if (block_partial_then_last(s, partials, counter, &total) && threadIdx.x == 0) peer_publish(red, total);
}

template <typename T>
__global__ void __launch_bounds__(kCgThreads)
cg_peer_direction_kernel(int64_t n, const T* __restrict__ r, T* __restrict__ p, CgPeerState* st, T* __restrict__ hist,
                         unsigned* done, PeerReduce red) {
    const double rz_new = peer_total(red);
    const int it = st->it;
    const double rz_old = st->rz[it & 1];
    const T beta = rz_old == 0.0 ? (T)0 : (T)(rz_new / rz_old);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = r[i] + beta * p[i];
    // the block that finishes last moves the iteration on (every block has read the state by then)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            *done = 0;
            st->rz[(it + 1) & 1] = rz_new;
            hist[it + 1] = (T)sqrt(rz_new);
            st->it = it + 1;
        }
    }
}

static size_t cg_workspace_bytes(int64_t n, size_t elem) {
    const size_t m = (size_t)(n > 0 ? n : 1);
    return 3 * Workspace::pad(m * elem) + Workspace::pad(kCgBlocks * sizeof(double)) + Workspace::pad(sizeof(CgScalars)) +
           Workspace::pad(sizeof(unsigned));
}

template <typename T>
int cg_run(int64_t n, int64_t nnz, const void* data, const void* indices, const void* indptr, int block_rows,
           const T* b, T* x, bool has_x0, T* hist, int64_t iterations, void* workspace, size_t bytes,
           int32_t* status, int dtype, int itype, cudaStream_t st) {
    Workspace ws(workspace, bytes);
    const size_t m = (size_t)(n > 0 ? n : 1);
    T* r = ws.take<T>(m);
    T* p = ws.take<T>(m);
    T* Ap = ws.take<T>(m);
    double* partials = ws.take<double>(kCgBlocks);
    CgScalars* sc = ws.take<CgScalars>(1);
    unsigned* counter = ws.take<unsigned>(1);
    if (!ws.ok()) return NB200_ERR_WORKSPACE;
    if (cudaMemsetAsync(counter, 0, sizeof(unsigned), st) != cudaSuccess) return NB200_ERR_CUDA;
    const int64_t want = ceil_div(n, (int64_t)kCgThreads);
    const unsigned grid = (unsigned)(want < 1 ? 1 : (want > kCgBlocks ? kCgBlocks : want));
    nb200_stream stream = reinterpret_cast<nb200_stream>(st);
    int rc;
    if (has_x0) {
        rc = nb200_spgemv_forward(n, n, nnz, data, indices, indptr, nullptr, x, Ap, block_rows, status, dtype, itype, stream);
        if (rc != NB200_OK) return rc;
    }
    cg_init_kernel<T><<<grid, kCgThreads, 0, st>>>(n, b, has_x0 ? Ap : nullptr, x, r, p, partials, counter, sc, hist);
    for (int64_t it = 0; it < iterations; ++it) {
        rc = nb200_spgemv_forward(n, n, nnz, data, indices, indptr, nullptr, p, Ap, block_rows, status, dtype, itype, stream);
        if (rc != NB200_OK) return rc;
        cg_dot_kernel<T><<<grid, kCgThreads, 0, st>>>(n, Ap, p, partials, counter, &sc->pAp);
        cg_update_kernel<T><<<grid, kCgThreads, 0, st>>>(n, (int)it, p, Ap, x, r, partials, counter, sc, hist);
        cg_direction_kernel<T><<<grid, kCgThreads, 0, st>>>(n, (int)it, r, p, sc);
    }
    return launch_status();
}

}  // namespace nb200

using namespace nb200;

namespace nb200 {
struct CgPeerWorkspace { double* partials; unsigned* counter; unsigned* done; CgPeerState* st; bool ok; };
static size_t cg_peer_workspace_bytes() {
    return Workspace::pad(kCgBlocks * sizeof(double)) + 2 * Workspace::pad(sizeof(unsigned)) + Workspace::pad(sizeof(CgPeerState));
}
static CgPeerWorkspace carve_peer(void* workspace, size_t bytes) {
    Workspace ws(workspace, bytes);
    CgPeerWorkspace w;
    w.partials = ws.take<double>(kCgBlocks);
    w.counter = ws.take<unsigned>(1);
    w.done = ws.take<unsigned>(1);
    w.st = ws.take<CgPeerState>(1);
    w.ok = ws.ok();
    return w;
}

template <typename T>
int cg_peer_phase(int phase, int64_t n, const T* b, T* x, T* r, T* p, const T* Ap, T* hist, const CgPeerWorkspace& w,
                  const PeerReduce& red, cudaStream_t st) {
    const int64_t want = ceil_div(n > 0 ? n : 1, (int64_t)kCgThreads);
    const unsigned grid = (unsigned)(want > kCgBlocks ? kCgBlocks : want);
    switch (phase) {
        case 0: cg_peer_init_kernel<T><<<grid, kCgThreads, 0, st>>>(n, b, x, r, p, w.partials, w.counter, w.st, red); break;
        case 1: cg_peer_start_kernel<T><<<1, kCgThreads, 0, st>>>(w.st, hist, red); break;
        case 2: cg_peer_dot_kernel<T><<<grid, kCgThreads, 0, st>>>(n, Ap, p, w.partials, w.counter, red); break;
        case 3: cg_peer_update_kernel<T><<<grid, kCgThreads, 0, st>>>(n, p, Ap, x, r, w.partials, w.counter, w.st, red); break;
        case 4: cg_peer_direction_kernel<T><<<grid, kCgThreads, 0, st>>>(n, r, p, w.st, hist, w.done, red); break;
        default: return NB200_ERR_BAD_ARG;
    }
    return launch_status();
}
}  // namespace nb200

extern "C" size_t nb200_cg_peer_workspace_bytes(void) { return cg_peer_workspace_bytes(); }

extern "C" int nb200_cg_peer_phase(int phase, int64_t n, const void* b, void* x, void* r, void* p, const void* Ap,
                                   void* residual_history, void* workspace, size_t workspace_bytes,
                                   int world, int rank, const int64_t* table, int32_t* sequence_word,
                                   int32_t* status, int64_t wait_budget_cycles, int dtype, nb200_stream stream) {
    if (n < 0 || world < 1 || world > 32 || rank < 0 || rank >= world || !table || !sequence_word || !workspace)
        return NB200_ERR_BAD_ARG;
    CgPeerWorkspace w = carve_peer(workspace, workspace_bytes);
    if (!w.ok) return NB200_ERR_WORKSPACE;
    cudaStream_t st = as_stream(stream);
    if (phase == 0) {   // a new solve: counters back to zero (the sequence word keeps counting for the life of the buffers)
        if (cudaMemsetAsync(w.counter, 0, sizeof(unsigned), st) != cudaSuccess ||
            cudaMemsetAsync(w.done, 0, sizeof(unsigned), st) != cudaSuccess) return NB200_ERR_CUDA;
    }
    PeerReduce red{world, rank, table, sequence_word, wait_budget_cycles > 0 ? wait_budget_cycles : 4000000000LL, status};
    return NB200_DISPATCH_T(dtype,
        (cg_peer_phase<T>(phase, n, (const T*)b, (T*)x, (T*)r, (T*)p, (const T*)Ap, (T*)residual_history, w, red, st)));
}

extern "C" size_t nb200_cg_workspace_bytes(int64_t n, int dtype) {
    return cg_workspace_bytes(n, dtype == NB200_F64 ? sizeof(double) : sizeof(float));
}

extern "C" int nb200_cg_fixed_iterations(int64_t n, int64_t nnz, const void* data, const void* indices, const void* indptr,
                                         int block_rows, const void* b, void* x, int has_x0, void* residual_history,
                                         int64_t iterations, void* workspace, size_t workspace_bytes, int32_t* status,
                                         int dtype, int itype, nb200_stream stream) {
    if (n < 0 || nnz < 0 || iterations < 0 || iterations > 0x7ffffffeLL || block_rows < 0 || block_rows > 256)
        return NB200_ERR_BAD_ARG;
    if (n == 0) return NB200_OK;
    if (!indptr || !b || !x || !residual_history || !workspace || (nnz > 0 && (!data || !indices))) return NB200_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    return NB200_DISPATCH_T(dtype,
        (cg_run<T>(n, nnz, data, indices, indptr, block_rows, (const T*)b, (T*)x, has_x0 != 0, (T*)residual_history,
                   iterations, workspace, workspace_bytes, status, dtype, itype, st)));
}
