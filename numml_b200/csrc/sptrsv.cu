// Sparse triangular solve (forward and the pieces of its backward) for CSR on sm_100a.
//
// Analysis (once per sparsity pattern and triangle): the dependency level of a row is one more than
// the largest level among the rows its strictly-triangular entries refer to (0 without any).  One
// launch computes all of them with the scheme the solve uses: one thread per row, rows taken in
// dependency order (ascending for a lower triangle, descending for an upper one), the level array
// pre-filled with -1 and polled as its own ready flag, a thread publishing its level from inside its
// poll loop so that lanes of one warp can depend on one another.  Polls are bounded by a cycle
// budget.  Rows are then sorted by (level, row) into `order`.
//
// Solve: one launch.  Row order[p] is owned by the p-th team (a team is as many lanes as there
// are right-hand sides, up to 32, so a dependency x[j, :] is read as one contiguous line).
// Because `order` is topological, the rows a team needs belong to teams with a smaller global
// index, i.e. to CTAs that were dispatched earlier; each lane polls the solution words it needs
// (the solution array itself is the ready flag, see below).  Every poll loop is bounded by a
// cycle budget and by a shared abort word: on expiry the kernel records NB200_ERR_WAIT_BUDGET in
// the status word, writes NaN for its own unknowns and returns, and every other waiter sees the
// abort word and leaves too.
//
// Arithmetic follows the reference: substitution in double whatever the value type, entries
// accumulated in storage order (ascending for a lower solve, descending from the row end for an
// upper solve) with unfused multiply and add, scan of a row stopped at the first entry on the
// wrong side of the diagonal, stored diagonal ignored with `unit`.  Results are bit-identical to
// the reference CPU loop.
#include "primitives.cuh"
#include <mutex>

namespace nb200 {

// ---------------------------------------------------------------------------------------------
// Analysis kernels
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int ld_relaxed_level(const int32_t* p) {
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_level(int32_t* p, int v) {
    asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}

// counters: [0] number of levels (largest level + 1), [1] non-zero if a wait ran out
template <typename I>
__global__ void __launch_bounds__(256)
sptrsv_levels_kernel(int64_t n, const I* __restrict__ indices, const I* __restrict__ indptr, bool lower,
                     int32_t* __restrict__ level, int32_t* __restrict__ counters, long long budget) {
    const int64_t pos = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pos >= n) return;
    // dependencies of row i lie before it in this order, i.e. with threads that were dispatched earlier
    const int64_t i = lower ? pos : n - 1 - pos;
    int64_t k = (int64_t)indptr[i];
    const int64_t end = (int64_t)indptr[i + 1];
    int lvl = 0;
    long long t0 = 0;
    for (unsigned spins = 0;; ++spins) {
        while (k < end) {                                   // as far as the known levels reach
            const int64_t j = (int64_t)indices[k];
            if (lower ? (j < i) : (j > i)) {
                const int v = ld_relaxed_level(level + j);
                if (v < 0) break;
                lvl = max(lvl, v + 1);
            }
            ++k;
        }
        if (k >= end) {                                     // published from inside the loop: a lane of the
            st_relaxed_level(level + i, lvl);               // same warp that waits for this row sees it on
            atomicMax(counters + 0, lvl + 1);               // its next round, wherever the warp reconverges
            break;
        }
        if (spins == 0) t0 = clock64();
        if ((spins & 63u) == 63u && (ld_relaxed_level(counters + 1) != 0 || clock64() - t0 > budget)) {
            atomicExch(counters + 1, 1);
            st_relaxed_level(level + i, 0);                 // let the waiters go; the caller sees the flag
            break;
        }
    }
}

// level_ptr[l] = first position of level l in the sorted order; level_ptr[nlevels] = n.  Levels are
// contiguous (a row of level l > 0 has a dependency of level l - 1), so every word is written.
__global__ void sptrsv_level_ptr_kernel(int64_t n, const uint32_t* __restrict__ sorted_level, int32_t nlevels,
                                        int32_t* __restrict__ level_ptr) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += stride) {
        const uint32_t l = sorted_level[p];
        if (p == 0 || sorted_level[p - 1] != l) level_ptr[l] = (int32_t)p;
        if (p == n - 1) level_ptr[nlevels] = (int32_t)n;
    }
}

__global__ void sptrsv_iota_kernel(int64_t n, uint32_t* __restrict__ v) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) v[i] = (uint32_t)i;
}

// ---------------------------------------------------------------------------------------------
// Solve kernel
// ---------------------------------------------------------------------------------------------
// The double-precision solution array doubles as the ready flag: it is filled with an all-ones
// bit pattern (a NaN no arithmetic produces) before the launch, and a lane that needs x[j, c]
// simply re-reads that one 8-byte word through L2 until it differs.  One round trip delivers both
// "ready" and the value, and no fence is needed because nothing else has to be ordered with it.
constexpr long long kNotReady = -1LL;                                  // 0xffff'ffff'ffff'ffff

__device__ __forceinline__ long long ld_relaxed_bits(const double* p) {
    long long v;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_relaxed_s32(const int32_t* p) {
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <typename T, typename I, int TS, bool PERM>
__global__ void __launch_bounds__(256)
sptrsv_syncfree_kernel(int64_t n, int64_t nrhs, const T* __restrict__ data, const I* __restrict__ indices,
                       const I* __restrict__ indptr, const I* __restrict__ perm,
                       const int32_t* __restrict__ order, bool lower, bool unit,
                       const T* __restrict__ b, T* __restrict__ x, double* __restrict__ xd,
                       int32_t* __restrict__ status, long long budget) {
    constexpr int D = 8;                                   // dependencies polled together
    const int tl = threadIdx.x % TS;
    const int64_t pos = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / TS;
    if (pos >= n) return;
    const int64_t i = (int64_t)order[pos];
    const int64_t s = (int64_t)indptr[i], len = (int64_t)indptr[i + 1] - s;
    const double canonical_nan = __longlong_as_double(0x7ff8000000000000LL);
    bool ok = true;

    for (int64_t c = tl; c < nrhs; c += TS) {              // this lane's right-hand sides
        double acc = 0.0, diag = 0.0;
        const double bi = (double)b[i * nrhs + c];         // fetched before the waits, off the critical path
        bool stop = false;
        // lower: ascending from the row start; upper: descending from the row end
        for (int64_t q = 0; q < len && !stop && ok; q += D) {
            int64_t jj[D];
            double aa[D], xv[D];
            unsigned valid = 0, pend = 0;
#pragma unroll
            for (int d = 0; d < D; ++d) {
                jj[d] = i; aa[d] = 0.0; xv[d] = 0.0;
                if (!stop && q + d < len) {
                    const int64_t k = lower ? (s + q + d) : (s + len - 1 - q - d);
                    const int64_t j = (int64_t)indices[k];
                    if (lower ? (j > i) : (j < i)) {
                        stop = true;
                    } else {
                        jj[d] = j;
                        aa[d] = (double)(PERM ? data[(int64_t)perm[k]] : data[k]);
                        valid |= 1u << d;
                        if (j != i) pend |= 1u << d;
                    }
                }
            }
            long long t0 = 0;
            for (unsigned spins = 0; pend != 0; ++spins) {
                // Issue every outstanding poll before looking at any answer: the loads are then in
                // flight together and one round costs one L2 round trip, not one per dependency.
                const unsigned asked = pend;
                long long bits[D];
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    bits[d] = kNotReady;
                    if ((asked >> d) & 1u) bits[d] = ld_relaxed_bits(xd + jj[d] * nrhs + c);
                }
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    if (((asked >> d) & 1u) && bits[d] != kNotReady) {
                        xv[d] = __longlong_as_double(bits[d]);
                        pend &= ~(1u << d);
                    }
                }
                if (pend != 0) {
                    if (spins == 0) t0 = clock64();
                    if ((spins & 31u) == 31u) {
                        if (ld_relaxed_s32(status) != 0) { ok = false; break; }
                        if (clock64() - t0 > budget) { atomicExch(status, (int)NB200_ERR_WAIT_BUDGET); ok = false; break; }
                    }
                }
            }
#pragma unroll
            for (int d = 0; d < D; ++d) {
                if ((valid >> d) & 1u) {
                    if (jj[d] == i) diag = aa[d];
                    else acc = __dadd_rn(acc, __dmul_rn(aa[d], xv[d]));
                }
            }
        }
        double xi;
        if (ok) {
            xi = bi - acc;
            if (!unit) xi /= diag;
            if (__double_as_longlong(xi) == kNotReady) xi = canonical_nan;   // never publish the marker itself
        } else {
            xi = canonical_nan;                                              // marks an aborted solve
        }
        __stcg(xd + i * nrhs + c, xi);
        if ((const void*)xd != (const void*)x) x[i * nrhs + c] = (T)xi;
    }
}

// out[k] = sum over r of alpha * (a[row(k), r] * b[col(k), r]), r ascending
template <typename T, typename I>
__global__ void masked_outer_kernel(int64_t rows, int64_t nnz, int64_t nrhs, const I* __restrict__ indices,
                                    const I* __restrict__ indptr, const T* __restrict__ a, const T* __restrict__ b,
                                    T alpha, T* __restrict__ out) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < nnz; k += stride) {
        int64_t lo = 0, hi = rows;
        while (hi - lo > 1) {
            const int64_t mid = (lo + hi) >> 1;
            if ((int64_t)indptr[mid] <= k) lo = mid; else hi = mid;
        }
        const int64_t j = (int64_t)indices[k];
        const T* ar = a + lo * nrhs;
        const T* br = b + j * nrhs;
        T s = mul_rn(alpha, mul_rn(ldg(ar), ldg(br)));
        for (int64_t r = 1; r < nrhs; ++r) s = add_rn(s, mul_rn(alpha, mul_rn(ldg(ar + r), ldg(br + r))));
        out[k] = s;
    }
}

static inline unsigned flat_grid(int64_t n) {
    const int64_t want = ceil_div(n > 0 ? n : 1, (int64_t)256);
    return (unsigned)(want > (int64_t)kSMs * 32 ? (int64_t)kSMs * 32 : want);
}

static inline int bit_length(int64_t v) {
    int bits = 0;
    while (v > 0) { ++bits; v >>= 1; }
    return bits;
}

static size_t analysis_workspace_bytes(int64_t n) {
    const size_t m = (size_t)(n > 0 ? n : 1);
    // level keys a/b, row ids a/b, counters, sort scratch
    return 4 * Workspace::pad(m * sizeof(int32_t)) + Workspace::pad(8 * sizeof(int32_t)) + Workspace::pad(sort_scratch_bytes(n));
}

template <typename I>
int sptrsv_analyse(int64_t n, const I* indices, const I* indptr, bool lower,
                   int32_t* order, int32_t* level_ptr, int64_t* nlevels_host, void* workspace, size_t bytes, cudaStream_t st) {
    *nlevels_host = 0;
    if (n == 0) return NB200_OK;
    const size_t m = (size_t)n;
    Workspace ws(workspace, bytes);
    uint32_t* key_a = ws.take<uint32_t>(m);
    uint32_t* key_b = ws.take<uint32_t>(m);
    uint32_t* val_a = ws.take<uint32_t>(m);
    uint32_t* val_b = ws.take<uint32_t>(m);
    int32_t* counters = ws.take<int32_t>(8);
    const size_t ssb = sort_scratch_bytes(n);
    char* sscratch = ws.take<char>(ssb);
    if (!ws.ok()) return NB200_ERR_WORKSPACE;

    if (cudaMemsetAsync(counters, 0, 8 * sizeof(int32_t), st) != cudaSuccess) return NB200_ERR_CUDA;
    if (cudaMemsetAsync(key_a, 0xff, m * sizeof(uint32_t), st) != cudaSuccess) return NB200_ERR_CUDA;   // -1: level unknown
    const int64_t grid = ceil_div(n, (int64_t)256);
    sptrsv_levels_kernel<I><<<(unsigned)grid, 256, 0, st>>>(n, indices, indptr, lower, reinterpret_cast<int32_t*>(key_a),
                                                           counters, 4000000000LL);
    int32_t host_counters[8] = {0};
    if (cudaMemcpyAsync(host_counters, counters, sizeof(host_counters), cudaMemcpyDeviceToHost, st) != cudaSuccess)
        return NB200_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return NB200_ERR_CUDA;
    if (host_counters[1] != 0) return NB200_ERR_WAIT_BUDGET;
    const int64_t nlevels = host_counters[0];
    *nlevels_host = nlevels;

    sptrsv_iota_kernel<<<flat_grid(n), 256, 0, st>>>(n, val_a);
    bool in_a = true;
    int rc = sort_pairs_u32(n, bit_length(nlevels - 1), key_a, val_a, key_b, val_b, &in_a, sscratch, ssb, st);
    if (rc != NB200_OK) return rc;
    if (cudaMemcpyAsync(order, in_a ? val_a : val_b, m * sizeof(int32_t), cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return NB200_ERR_CUDA;
    if (level_ptr)
        sptrsv_level_ptr_kernel<<<flat_grid(n), 256, 0, st>>>(n, in_a ? key_a : key_b, (int32_t)nlevels, level_ptr);
    return launch_status();
}

template <typename T, typename I, bool PERM>
int sptrsv_solve_team(int ts, int64_t n, int64_t nrhs, const T* data, const I* indices, const I* indptr, const I* perm,
                      const int32_t* order, bool lower, bool unit, const T* b, T* x, double* xd,
                      int32_t* status, long long budget, cudaStream_t st) {
    const int64_t threads = n * ts;
    const int64_t grid = ceil_div(threads, (int64_t)256);
    if (grid > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
#define NB200_SOLVE(TS_)                                                                                   \
    sptrsv_syncfree_kernel<T, I, TS_, PERM><<<(unsigned)grid, 256, 0, st>>>(n, nrhs, data, indices, indptr, perm, \
        order, lower, unit, b, x, xd, status, budget)
    switch (ts) {
        case 1: NB200_SOLVE(1); break;
        case 2: NB200_SOLVE(2); break;
        case 4: NB200_SOLVE(4); break;
        case 8: NB200_SOLVE(8); break;
        case 16: NB200_SOLVE(16); break;
        default: NB200_SOLVE(32); break;
    }
#undef NB200_SOLVE
    return launch_status();
}

}  // namespace nb200

using namespace nb200;

extern "C" size_t nb200_sptrsv_analysis_workspace_bytes(int64_t n) { return analysis_workspace_bytes(n); }

extern "C" int nb200_sptrsv_analyse(int64_t n, int64_t nnz, const void* indices, const void* indptr,
                                    const void* t_indptr, const void* t_indices, int itype, int lower,
                                    int32_t* order, int64_t* nlevels_host,
                                    void* workspace, size_t workspace_bytes, nb200_stream stream) {
    if (n < 0 || nnz < 0 || !nlevels_host) return NB200_ERR_BAD_ARG;
    if (n >= 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    (void)t_indptr; (void)t_indices;
    if (n > 0 && (!indptr || !order || !workspace || (nnz > 0 && !indices))) return NB200_ERR_BAD_ARG;
    return NB200_DISPATCH_I(itype,
        (sptrsv_analyse<I>(n, (const I*)indices, (const I*)indptr, lower != 0,
                           order, nullptr, nlevels_host, workspace, workspace_bytes, as_stream(stream))));
}

extern "C" int nb200_sptrsv_analyse_levels(int64_t n, int64_t nnz, const void* indices, const void* indptr,
                                           int itype, int lower, int32_t* order, int32_t* level_ptr,
                                           int64_t* nlevels_host, void* workspace, size_t workspace_bytes,
                                           nb200_stream stream) {
    if (n < 0 || nnz < 0 || !nlevels_host) return NB200_ERR_BAD_ARG;
    if (n >= 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    if (n > 0 && (!indptr || !order || !level_ptr || !workspace || (nnz > 0 && !indices))) return NB200_ERR_BAD_ARG;
    return NB200_DISPATCH_I(itype,
        (sptrsv_analyse<I>(n, (const I*)indices, (const I*)indptr, lower != 0,
                           order, level_ptr, nlevels_host, workspace, workspace_bytes, as_stream(stream))));
}

extern "C" int nb200_sptrsv_solve(int64_t n, int64_t nnz, int64_t nrhs,
                                  const void* data, const void* indices, const void* indptr, const void* perm,
                                  const int32_t* order, int lower, int unit, const void* b, void* x,
                                  double* x_double, int32_t* status, int64_t wait_budget_cycles,
                                  int team_lanes, int dtype, int itype, nb200_stream stream) {
    if (n < 0 || nnz < 0 || nrhs < 0) return NB200_ERR_BAD_ARG;
    if (team_lanes < 0 || team_lanes > 32 || (team_lanes & (team_lanes - 1)) != 0) return NB200_ERR_BAD_ARG;
    if (n == 0 || nrhs == 0) return NB200_OK;
    if (!indptr || !order || !b || !x || !status || (nnz > 0 && (!data || !indices))) return NB200_ERR_BAD_ARG;
    if (dtype == NB200_F32 && !x_double) return NB200_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    double* xd_all = (dtype == NB200_F64) ? (double*)x : x_double;
    if (cudaMemsetAsync(xd_all, 0xff, sizeof(double) * (size_t)n * (size_t)nrhs, st) != cudaSuccess) return NB200_ERR_CUDA;
    int ts = 1;
    while (ts < 32 && ts < nrhs) ts <<= 1;
    if (team_lanes > ts) ts = team_lanes;   // spare lanes idle; fewer rows share a warp's poll round trips
    const long long budget = wait_budget_cycles > 0 ? wait_budget_cycles : 2000000000LL;
    return NB200_DISPATCH(dtype, itype, ([&]() -> int {
        double* xd = (dtype == NB200_F64) ? (double*)x : x_double;
        if (perm)
            return sptrsv_solve_team<T, I, true>(ts, n, nrhs, (const T*)data, (const I*)indices, (const I*)indptr,
                                                 (const I*)perm, order, lower != 0, unit != 0, (const T*)b, (T*)x, xd,
                                                 status, budget, st);
        return sptrsv_solve_team<T, I, false>(ts, n, nrhs, (const T*)data, (const I*)indices, (const I*)indptr,
                                              (const I*)perm, order, lower != 0, unit != 0, (const T*)b, (T*)x, xd,
                                              status, budget, st);
    }()));
}

extern "C" int nb200_masked_outer(int64_t rows, int64_t nnz, int64_t nrhs, const void* indices, const void* indptr,
                                  const void* a, const void* b, double alpha, void* out,
                                  int dtype, int itype, nb200_stream stream) {
    if (rows < 0 || nnz < 0 || nrhs < 1) return NB200_ERR_BAD_ARG;
    if (nnz == 0) return NB200_OK;
    if (!indices || !indptr || !a || !b || !out) return NB200_ERR_BAD_ARG;
    return NB200_DISPATCH(dtype, itype,
        (masked_outer_kernel<T, I><<<flat_grid(nnz), 256, 0, as_stream(stream)>>>(
             rows, nnz, nrhs, (const I*)indices, (const I*)indptr, (const T*)a, (const T*)b, (T)alpha, (T*)out),
         launch_status()));
}


// ---------------------------------------------------------------------------------------------
// Allocation-free float32 solve
// ---------------------------------------------------------------------------------------------
// A float32 solve substitutes in double, so it needs n*nrhs doubles of working memory besides its
// inputs and outputs.  nb200_sptrsv_solve takes that array from the caller.  The variant below is
// for hosts that cannot hand one over: a plugin living inside another runtime that owns the whole
// device-memory pool and forbids further allocation, or a control loop that must not reach
// cudaMalloc because it synchronises the device and can fail once memory is fragmented.  The
// working array is a fixed region inside the library image instead; every GPU that loads the
// library carries these 8 MiB until the process exits.
constexpr int64_t kNoAllocSolveWords = 1 << 20;                       // doubles: n * nrhs may not exceed this
static __device__ __align__(256) double g_noalloc_solve_words[kNoAllocSolveWords];

// In host code the array's name is only a handle for the runtime, not an address a kernel could
// use: the device address is looked up once per device, with that device current, and cached.
static int noalloc_solve_words(double** out) {
    static std::mutex mu;
    static double* cached[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NB200_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_solve_words) != cudaSuccess || p == nullptr) return NB200_ERR_CUDA;
        cached[dev] = static_cast<double*>(p);
    }
    *out = cached[dev];
    return NB200_OK;
}

extern "C" int64_t nb200_sptrsv_solve_f32_noalloc_capacity(void) { return kNoAllocSolveWords; }

extern "C" int nb200_sptrsv_solve_f32_noalloc(int64_t n, int64_t nnz, int64_t nrhs,
                                              const float* data, const void* indices, const void* indptr,
                                              const void* perm, const int32_t* order, int lower, int unit,
                                              const float* b, float* x, int32_t* status,
                                              int64_t wait_budget_cycles, int itype, nb200_stream stream) {
    if (n < 0 || nnz < 0 || nrhs < 0) return NB200_ERR_BAD_ARG;
    if (n > 0 && nrhs > 0 && (n > kNoAllocSolveWords || nrhs > kNoAllocSolveWords / n)) return NB200_ERR_TOO_LARGE;
    double* words = nullptr;
    const int rc = noalloc_solve_words(&words);
    if (rc != NB200_OK) return rc;
    // nb200_sptrsv_solve refills the working array with the "not solved yet" marker on every call,
    // so whatever the previous call left in the shared region is never read.
    return nb200_sptrsv_solve(n, nnz, nrhs, data, indices, indptr, perm, order, lower, unit, b, x, words, status,
                              wait_budget_cycles, /*team_lanes=*/0, NB200_F32, itype, stream);
}
