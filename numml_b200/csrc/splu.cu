// Sparse LU factorisation without pivoting, M = L + U with unit lower L, for CSR on sm_100a.
//
// Symbolic phase: the pattern of row i of M is the set the "fill2" traversal finds (Rose & Tarjan):
// mark i and the columns of row i of A; for t = 0 .. i-1 in ascending order, if t is marked, walk the
// graph of A from t through vertices not yet marked for this row; a vertex w reached is marked, and it is
// an entry (i, w) of M when w > t, otherwise the walk continues through it.  Rows are independent: one warp
// per row, with three arrays of n words of its own (visit stamps, entry stamps, queue) in the workspace;
// stamps carry the row number, so nothing is cleared between the rows a warp takes.  The lanes share the
// scan over t (32 candidates per ballot) and the neighbours of the vertex being expanded.  A first pass
// counts, a scan gives the row pointers, a second pass writes the columns (ascending) and the values (the
// value of A, or an explicit zero where fill is introduced).
//
// Numeric phase, on the transpose Mt (columns of M stored as rows, rows ascending): left-looking, one warp
// per column k, columns taken in ascending order.  For every stored row i < k of the column, in order, the
// warp waits for column i to be final (a flag per column, bounded polls), then every lane takes entries
// j > i of column k and subtracts M_ji * M_ik where column i stores row j; finally the entries below the
// diagonal are divided by the pivot and the column's flag is raised.  Updates of one entry happen in
// ascending i with an unfused multiply and subtract: the factors are bit-identical to the sequential loop.
// A column depends only on columns to its left, which belong to warps dispatched earlier.
#include "primitives.cuh"

namespace nb200 {

constexpr int kLuWarpsPerCta = 8;

__device__ __forceinline__ int lu_ld_acquire(const int32_t* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void lu_st_release(int32_t* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}

// position of `key` in the ascending run indices[lo .. hi] (hi inclusive), or -1
__device__ __forceinline__ int64_t lu_find(const int64_t* __restrict__ indices, int64_t lo, int64_t hi, int64_t key) {
    while (lo <= hi) {
        const int64_t mid = (lo + hi) >> 1;
        const int64_t v = indices[mid];
        if (v < key) lo = mid + 1; else if (v > key) hi = mid - 1; else return mid;
    }
    return -1;
}

template <typename T, bool FILL>
__global__ void __launch_bounds__(32 * kLuWarpsPerCta)
splu_symbolic_kernel(int64_t n, const T* __restrict__ A_data, const int64_t* __restrict__ A_indices,
                     const int64_t* __restrict__ A_indptr, int32_t* __restrict__ row_nnz,
                     const int64_t* __restrict__ M_indptr, int64_t* __restrict__ M_indices, T* __restrict__ M_data,
                     int32_t* __restrict__ work, int stamp_base) {
    constexpr unsigned kAll = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kLuWarpsPerCta + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kLuWarpsPerCta;
    int32_t* visited = work + warp * 3 * n;       // == stamp: reached while treating the current row
    int32_t* entry = visited + n;                 // == stamp: column is an entry of the current row of M
    int32_t* queue = entry + n;
    for (int64_t i = warp; i < n; i += nwarps) {
        const int32_t stamp = stamp_base + (int32_t)i + 1;
        if (lane == 0) visited[i] = stamp;
        for (int64_t e = A_indptr[i] + lane; e < A_indptr[i + 1]; e += 32) {
            const int64_t c = A_indices[e];
            visited[c] = stamp;
            entry[c] = stamp;
        }
        __syncwarp();
        for (int64_t t0 = 0; t0 < i; t0 += 32) {
            const int64_t t = t0 + lane;
            unsigned sources = __ballot_sync(kAll, t < i && visited[t] == stamp);
            while (sources) {
                const int64_t src = t0 + (__ffs(sources) - 1);
                // ---- walk from src through unvisited vertices <= src ----
                int head = 0, tail = 1;
                if (lane == 0) queue[0] = (int32_t)src;
                __syncwarp();
                while (head < tail) {
                    const int64_t u = queue[head++];
                    const int64_t ue = A_indptr[u + 1];
                    for (int64_t e0 = A_indptr[u]; e0 < ue; e0 += 32) {
                        const int64_t e = e0 + lane;
                        bool push = false;
                        int64_t w = 0;
                        if (e < ue) {
                            w = A_indices[e];
                            if (visited[w] != stamp) {
                                visited[w] = stamp;
                                if (w > src) entry[w] = stamp; else push = true;
                            }
                        }
                        const unsigned pushing = __ballot_sync(kAll, push);
                        if (push) queue[tail + __popc(pushing & ((1u << lane) - 1u))] = (int32_t)w;
                        tail += __popc(pushing);
                    }
                    __syncwarp();
                }
                // candidates after src in this group of 32 may have been reached by the walk
                sources = __ballot_sync(kAll, t > src && t < i && visited[t] == stamp);
            }
        }
        // ---- the row of M: marked columns in ascending order ----
        int64_t out = FILL ? M_indptr[i] : 0;
        const int64_t a_lo = A_indptr[i], a_hi = A_indptr[i + 1] - 1;
        for (int64_t c0 = 0; c0 < n; c0 += 32) {
            const int64_t c = c0 + lane;
            const bool has = c < n && entry[c] == stamp;
            const unsigned m = __ballot_sync(kAll, has);
            if (FILL && has) {
                const int64_t pos = out + __popc(m & ((1u << lane) - 1u));
                const int64_t at = lu_find(A_indices, a_lo, a_hi, c);
                M_indices[pos] = c;
                M_data[pos] = at >= 0 ? A_data[at] : (T)0;
            }
            out += __popc(m);
        }
        if (!FILL && lane == 0) row_nnz[i] = (int32_t)out;
        __syncwarp();
    }
}

template <typename T>
__global__ void __launch_bounds__(32 * kLuWarpsPerCta)
splu_numeric_kernel(int64_t n, T* Mt_data, const int64_t* __restrict__ Mt_indices, const int64_t* __restrict__ Mt_indptr,
                    int32_t* done, int32_t* status, long long budget) {
    constexpr unsigned kAll = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int64_t k = (int64_t)blockIdx.x * kLuWarpsPerCta + (threadIdx.x >> 5);
    if (k >= n) return;
    const int64_t cs = Mt_indptr[k], ce = Mt_indptr[k + 1];
    int64_t diag = -1;
    bool ok = true;
    for (int64_t ii = cs; ii < ce && ok; ++ii) {
        const int64_t i = Mt_indices[ii];
        if (i == k) { diag = ii; break; }
        if (i > k) break;                                     // no stored diagonal: nothing to divide by
        if (lane == 0 && lu_ld_acquire(done + i) == 0) {      // column i must be final
            const long long t0 = clock64();
            while (lu_ld_acquire(done + i) == 0) {
                if (lu_ld_acquire(status) != 0 || clock64() - t0 > budget) { ok = false; break; }
                __nanosleep(32);
            }
        }
        ok = __shfl_sync(kAll, ok, 0);
        if (!ok) break;
        const T a_ik = __ldcg(Mt_data + ii);
        const int64_t is = Mt_indptr[i], ie = Mt_indptr[i + 1] - 1;
        for (int64_t jj = ii + 1 + lane; jj < ce; jj += 32) {
            const int64_t at = lu_find(Mt_indices, is, ie, Mt_indices[jj]);
            if (at >= 0) {
                const T prod = mul_rn(__ldcg(Mt_data + at), a_ik);
                __stcg(Mt_data + jj, __ldcg(Mt_data + jj) - prod);
            }
        }
        __syncwarp();
    }
    if (!ok) {
        if (lane == 0) atomicExch(status, (int)NB200_ERR_WAIT_BUDGET);
    } else if (diag >= 0) {
        const T pivot = __ldcg(Mt_data + diag);
        for (int64_t jj = diag + 1 + lane; jj < ce; jj += 32) __stcg(Mt_data + jj, __ldcg(Mt_data + jj) / pivot);
    }
    __syncwarp();
    __threadfence();
    if (lane == 0) lu_st_release(done + k, 1);                // also on failure: the waiters see the status word
}

struct LuWorkspace { int32_t* row_nnz; char* scan; size_t scan_bytes; int32_t* work; int64_t warps; bool ok; };

static int64_t lu_warps_for(int64_t n) {
    // as many rows in flight as fit about 2 GiB of stamp arrays, at most one warp per row or per warp slot
    const int64_t by_memory = (int64_t)((2ull << 30) / (12ull * (uint64_t)(n > 0 ? n : 1)));
    int64_t w = (int64_t)kSMs * 16;
    if (w > n) w = n;
    if (w > by_memory) w = by_memory;
    if (w < 1) w = 1;
    return ceil_div(w, (int64_t)kLuWarpsPerCta) * kLuWarpsPerCta;
}

static size_t lu_workspace_bytes(int64_t n) {
    const size_t m = (size_t)(n > 0 ? n : 1);
    return Workspace::pad(m * sizeof(int32_t)) + Workspace::pad(scan_scratch_bytes(n)) +
           Workspace::pad((size_t)lu_warps_for(n) * 3 * m * sizeof(int32_t));
}

static LuWorkspace lu_carve(int64_t n, void* workspace, size_t bytes) {
    const size_t m = (size_t)(n > 0 ? n : 1);
    Workspace ws(workspace, bytes);
    LuWorkspace w;
    w.row_nnz = ws.take<int32_t>(m);
    w.scan_bytes = scan_scratch_bytes(n);
    w.scan = ws.take<char>(w.scan_bytes);
    w.warps = lu_warps_for(n);
    w.work = ws.take<int32_t>((size_t)w.warps * 3 * m);
    w.ok = ws.ok();
    return w;
}

}  // namespace nb200

using namespace nb200;

extern "C" size_t nb200_splu_workspace_bytes(int64_t n) { return lu_workspace_bytes(n); }

extern "C" int nb200_splu_symbolic_count(int64_t n, const int64_t* A_indices, const int64_t* A_indptr, int64_t* M_indptr,
                                         void* workspace, size_t workspace_bytes, nb200_stream stream) {
    if (n < 0 || !M_indptr || !workspace || (n > 0 && !A_indptr)) return NB200_ERR_BAD_ARG;
    if (n >= 0x3fffffffLL) return NB200_ERR_TOO_LARGE;
    cudaStream_t st = as_stream(stream);
    LuWorkspace w = lu_carve(n, workspace, workspace_bytes);
    if (!w.ok) return NB200_ERR_WORKSPACE;
    if (n > 0) {
        if (cudaMemsetAsync(w.work, 0, (size_t)w.warps * 3 * (size_t)n * sizeof(int32_t), st) != cudaSuccess) return NB200_ERR_CUDA;
        splu_symbolic_kernel<double, false><<<(unsigned)(w.warps / kLuWarpsPerCta), 32 * kLuWarpsPerCta, 0, st>>>(
            n, nullptr, A_indices, A_indptr, w.row_nnz, nullptr, nullptr, nullptr, w.work, 0);
    }
    return exclusive_scan_i32_to_i64(n, w.row_nnz, M_indptr, w.scan, w.scan_bytes, st);
}

extern "C" int nb200_splu_symbolic_fill(int64_t n, const void* A_data, const int64_t* A_indices, const int64_t* A_indptr,
                                        const int64_t* M_indptr, int64_t* M_indices, void* M_data,
                                        void* workspace, size_t workspace_bytes, int dtype, nb200_stream stream) {
    if (n < 0 || !workspace || (n > 0 && (!A_indptr || !M_indptr))) return NB200_ERR_BAD_ARG;
    if (n == 0) return NB200_OK;
    if (n >= 0x3fffffffLL) return NB200_ERR_TOO_LARGE;
    cudaStream_t st = as_stream(stream);
    LuWorkspace w = lu_carve(n, workspace, workspace_bytes);
    if (!w.ok) return NB200_ERR_WORKSPACE;
    // stamps of this pass start above those the counting pass left in the arrays
    return NB200_DISPATCH_T(dtype,
        (splu_symbolic_kernel<T, true><<<(unsigned)(w.warps / kLuWarpsPerCta), 32 * kLuWarpsPerCta, 0, st>>>(
             n, (const T*)A_data, A_indices, A_indptr, nullptr, M_indptr, M_indices, (T*)M_data, w.work, (int)n),
         launch_status()));
}

extern "C" int nb200_splu_numeric(int64_t n, void* Mt_data, const int64_t* Mt_indices, const int64_t* Mt_indptr,
                                  int32_t* done, int32_t* status, int64_t wait_budget_cycles, int dtype, nb200_stream stream) {
    if (n < 0 || (n > 0 && (!Mt_indptr || !done || !status))) return NB200_ERR_BAD_ARG;
    if (n == 0) return NB200_OK;
    cudaStream_t st = as_stream(stream);
    if (cudaMemsetAsync(done, 0, (size_t)n * sizeof(int32_t), st) != cudaSuccess) return NB200_ERR_CUDA;
    const int64_t grid = ceil_div(n, (int64_t)kLuWarpsPerCta);
    if (grid > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    const long long budget = wait_budget_cycles > 0 ? wait_budget_cycles : 4000000000LL;
    return NB200_DISPATCH_T(dtype,
        (splu_numeric_kernel<T><<<(unsigned)grid, 32 * kLuWarpsPerCta, 0, st>>>(n, (T*)Mt_data, Mt_indices, Mt_indptr, done,
                                                                            status, budget), launch_status()));
}
