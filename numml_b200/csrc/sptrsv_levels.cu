// Level-synchronous sparse triangular solve inside one thread-block cluster: an alternative to the grid-wide
// sync-free solve for matrices whose dependency levels are narrow (banded factors, stencil factors in natural
// ordering: thousands of levels of a few hundred rows), kept as an option because it is the slower of the two
// on B200 (see "Measured" below).
//
//   * one cluster of C CTAs; a team of TS lanes (one lane per right-hand side) takes one row of the
//     current level, the teams of the cluster together one level (or a round of it);
//   * every solved row is written into a ring of recent rows that is spread over the shared memory
//     of the C CTAs (row of position p lives in CTA p mod C), and a dependency is read from there
//     through distributed shared memory; a hardware cluster barrier separates the levels;
//   * everything a row needs besides the unknowns -- its entries, its right-hand side -- is laid out
//     in *position order* (the order in which the cluster takes the rows) by the plan and by a
//     gather pass in front of the solve, so that the kernel reads plain streams, which it requests
//     two items ahead of their use (row pointers) and one item ahead (entries, right-hand side).
//
// The ring holds C * cap rows; the plan reports `reach`, the largest distance between the end of a
// row's level and the position of any of its dependencies, and the solve is refused (the caller
// then takes the sync-free kernel) when the ring cannot hold that many rows.
//
// No thread of this kernel ever waits on a flag: the only synchronisation is the cluster barrier,
// which every thread reaches once per level, whatever rows it owns.
//
// Measured (lower 9-point factor of the 1024^2 grid, 3070 levels of at most 512 rows, 16 right-hand sides,
// fp64): 6.8 ms with 16 CTAs, 9.0 ms with 8, against 3.2 ms for the sync-free kernel.  A level costs 2.2 us
// here and 1.03 us there.  Taking the pieces out one at a time (results wrong, timing only): without the copy
// of the unknowns to global memory 6.1 ms; with a relaxed instead of a release/acquire barrier 5.2 ms; with
// all ring reads local instead of remote 6.7 ms; with all three 4.9 ms, and 4.5 ms with a single right-hand
// side whose 512 rows per level occupy one CTA: 1.5 us per level remain for a barrier across the cluster and
// a handful of dependent instructions, more than the 1.03 us that a store and a poll through L2 cost.  Deeper
// software pipelining (registers swapped instead of copied, L2 prefetch six levels ahead, the global store
// moved between the barrier's arrive and wait) did not move it: the cluster barrier itself is the floor.
//
// Arithmetic is the reference's (cpp/sparse_csr_cpu.cpp, sptrsv_forward_cpu): substitution in double,
// entries in storage order for a lower solve and from the row end backwards for an upper one,
// unfused multiply and add, one division by the stored diagonal unless `unit`; bit-identical.
#include "primitives.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace nb200 {

constexpr int kLevelThreads = 512;          // per CTA
constexpr int kLevelRegEntries = 8;         // entries of a row prefetched into registers

// ---------------------------------------------------------------------------------------------
// Plan: position-ordered structure
// ---------------------------------------------------------------------------------------------
__global__ void lv_inverse_kernel(int64_t n, const int32_t* __restrict__ order, int32_t* __restrict__ inv) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += stride) inv[order[p]] = (int32_t)p;
}

// entries of row order[p] on the solve side of the diagonal, the diagonal included
template <typename I>
__global__ void lv_count_kernel(int64_t n, const I* __restrict__ indices, const I* __restrict__ indptr,
                                const int32_t* __restrict__ order, bool lower, int32_t* __restrict__ count) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += stride) {
        const int64_t i = order[p];
        int c = 0;
        for (int64_t k = (int64_t)indptr[i]; k < (int64_t)indptr[i + 1]; ++k) {
            const int64_t j = (int64_t)indices[k];
            c += (lower ? (j <= i) : (j >= i)) ? 1 : 0;
        }
        count[p] = c;
    }
}

// info: [0] reach, [1] longest row, [2] widest level
template <typename I>
__global__ void lv_fill_kernel(int64_t n, const I* __restrict__ indices, const I* __restrict__ indptr,
                               const I* __restrict__ perm, const int32_t* __restrict__ order,
                               const int32_t* __restrict__ inv, const int32_t* __restrict__ level_ptr, int32_t nlevels,
                               bool lower, const int32_t* __restrict__ pos_ptr, int32_t* __restrict__ dep,
                               int32_t* __restrict__ src, int32_t* __restrict__ info) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += stride) {
        const int64_t i = order[p];
        const int64_t s = (int64_t)indptr[i], len = (int64_t)indptr[i + 1] - s;
        int32_t out = pos_ptr[p];
        int32_t first_dep = 0x7fffffff;
        for (int64_t q = 0; q < len; ++q) {                       // the order in which the solve adds
            const int64_t k = lower ? (s + q) : (s + len - 1 - q);
            const int64_t j = (int64_t)indices[k];
            if (lower ? (j > i) : (j < i)) continue;
            int32_t d = -1;
            if (j != i) { d = inv[j]; first_dep = min(first_dep, d); }
            dep[out] = d;
            src[out] = (int32_t)(perm ? (int64_t)perm[k] : k);
            ++out;
        }
        atomicMax(info + 1, out - pos_ptr[p]);
        if (first_dep != 0x7fffffff) {
            int lo = 0, hi = nlevels;                             // level of position p: level_ptr[lo] <= p < level_ptr[lo + 1]
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if ((int64_t)level_ptr[mid] <= p) lo = mid; else hi = mid;
            }
            atomicMax(info + 0, level_ptr[lo + 1] - first_dep);
        }
    }
    for (int64_t l = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; l < nlevels; l += stride)
        atomicMax(info + 2, level_ptr[l + 1] - level_ptr[l]);
}

// ---------------------------------------------------------------------------------------------
// Per-solve gathers into position order, and the scatter back
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void lv_gather_kernel(int64_t entries, const T* __restrict__ data, const int32_t* __restrict__ src,
                                 double* __restrict__ val, int64_t n, int64_t nrhs, const int32_t* __restrict__ order,
                                 const T* __restrict__ b, double* __restrict__ b_pos) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (int64_t k = t0; k < entries; k += stride) val[k] = (double)data[src[k]];
    const int64_t total = n * nrhs;
    for (int64_t e = t0; e < total; e += stride) {
        const int64_t p = e / nrhs, c = e - p * nrhs;
        b_pos[e] = (double)b[(int64_t)order[p] * nrhs + c];
    }
}

template <typename T>
__global__ void lv_scatter_kernel(int64_t n, int64_t nrhs, const int32_t* __restrict__ order,
                                  const double* __restrict__ x_pos, T* __restrict__ x) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t total = n * nrhs;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const int64_t p = e / nrhs, c = e - p * nrhs;
        x[(int64_t)order[p] * nrhs + c] = (T)x_pos[e];
    }
}

// ---------------------------------------------------------------------------------------------
// The cluster kernel
// ---------------------------------------------------------------------------------------------
struct LvItem {                      // one round of one level: positions base .. min(base + teams, end) - 1
    int32_t level;
    int32_t base, end;               // end = end of the level
    int32_t end_next;                // end of the following level, requested one item earlier
};

__device__ __forceinline__ LvItem lv_next(const LvItem& it, int teams, const int32_t* __restrict__ level_ptr, int32_t nlevels) {
    LvItem o = it;
    o.base = it.base + teams;
    if (o.base >= it.end) {
        o.level = it.level + 1;
        o.base = it.end;
        o.end = it.end_next;
        o.end_next = (o.level + 2 <= nlevels) ? __ldg(level_ptr + o.level + 2) : it.end_next;
    }
    return o;
}

struct LvEntries {
    int32_t k0, count;
    int32_t dep[kLevelRegEntries];
    double val[kLevelRegEntries];
    double bi;
};

template <int TS>
__global__ void __launch_bounds__(kLevelThreads, 1)
sptrsv_cluster_kernel(int64_t nrhs, const int32_t* __restrict__ pos_ptr, const int32_t* __restrict__ dep,
                      const double* __restrict__ val, const int32_t* __restrict__ level_ptr, int32_t nlevels,
                      bool unit, const double* __restrict__ b_pos, double* __restrict__ x_pos,
                      int cap_shift) {
    extern __shared__ __align__(16) double ring[];             // (1 << cap_shift) rows of nrhs doubles
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned C = cluster.num_blocks();                    // a power of two
    const unsigned cmask = C - 1;
    int cshift = 0;
    while ((1u << cshift) < C) ++cshift;
    const unsigned rank = cluster.block_rank();
    const int teams = (int)(C * kLevelThreads / TS);
    const int team = (int)((rank * kLevelThreads + threadIdx.x) / TS);
    const int tl = (int)(threadIdx.x % TS);
    const unsigned cap_mask = (1u << cap_shift) - 1;
    const bool lane_on = tl < nrhs;

    // items: it0 is computed in this iteration, it1 gets its entries requested, it2 its row pointers
    LvItem it0;
    it0.level = 0;
    it0.base = __ldg(level_ptr + 0);
    it0.end = __ldg(level_ptr + 1);
    it0.end_next = nlevels >= 2 ? __ldg(level_ptr + 2) : it0.end;
    LvItem it1 = lv_next(it0, teams, level_ptr, nlevels);
    LvItem it2 = lv_next(it1, teams, level_ptr, nlevels);

    auto row_pointers = [&](const LvItem& it, int32_t& k0, int32_t& k1) {
        const int64_t p = (int64_t)it.base + team;
        k0 = k1 = 0;
        if (it.level < nlevels && p < it.end) { k0 = __ldg(pos_ptr + p); k1 = __ldg(pos_ptr + p + 1); }
    };
    auto entries = [&](const LvItem& it, int32_t k0, int32_t k1, LvEntries& e) {
        const int64_t p = (int64_t)it.base + team;
        e.k0 = k0;
        e.count = k1 - k0;
        e.bi = 0.0;
#pragma unroll
        for (int t = 0; t < kLevelRegEntries; ++t) {
            e.dep[t] = -1; e.val[t] = 0.0;
            if (t < e.count) { e.dep[t] = __ldg(dep + k0 + t); e.val[t] = __ldg(val + k0 + t); }
        }
        if (it.level < nlevels && p < it.end && lane_on) e.bi = __ldg(b_pos + p * nrhs + tl);
    };

    int32_t k0_0, k1_0, k0_1, k1_1, k0_2, k1_2;
    row_pointers(it0, k0_0, k1_0);
    row_pointers(it1, k0_1, k1_1);
    LvEntries e0, e1;
    entries(it0, k0_0, k1_0, e0);
    cluster.sync();                                             // every CTA of the cluster is resident before remote accesses

    while (it0.level < nlevels) {
        row_pointers(it2, k0_2, k1_2);
        entries(it1, k0_1, k1_1, e1);

        const int64_t p = (int64_t)it0.base + team;
        if (p < it0.end) {
            for (int64_t c = tl; c < nrhs; c += TS) {
                const double bi = (c == tl) ? e0.bi : __ldg(b_pos + p * nrhs + c);
                double xv[kLevelRegEntries];
#pragma unroll
                for (int t = 0; t < kLevelRegEntries; ++t) {   // all remote reads of the row in flight together
                    xv[t] = 0.0;
                    const int32_t d = e0.dep[t];
                    if (t < e0.count && d >= 0) {
                        const double* peer = cluster.map_shared_rank(ring, (unsigned)d & cmask);
                        xv[t] = peer[(size_t)(((unsigned)d >> cshift) & cap_mask) * nrhs + c];
                    }
                }
                double acc = 0.0, diag = 1.0;
#pragma unroll
                for (int t = 0; t < kLevelRegEntries; ++t) {
                    if (t < e0.count) {
                        if (e0.dep[t] < 0) diag = e0.val[t];
                        else acc = __dadd_rn(acc, __dmul_rn(e0.val[t], xv[t]));
                    }
                }
                for (int32_t t = kLevelRegEntries; t < e0.count; ++t) {     // long rows: the rest from memory
                    const int32_t d = __ldg(dep + e0.k0 + t);
                    const double a = __ldg(val + e0.k0 + t);
                    if (d < 0) { diag = a; continue; }
                    const double* peer = cluster.map_shared_rank(ring, (unsigned)d & cmask);
                    acc = __dadd_rn(acc, __dmul_rn(a, peer[(size_t)(((unsigned)d >> cshift) & cap_mask) * nrhs + c]));
                }
                double xi = bi - acc;
                if (!unit) xi /= diag;
                double* home = cluster.map_shared_rank(ring, (unsigned)p & cmask);
                home[(size_t)(((unsigned)p >> cshift) & cap_mask) * nrhs + c] = xi;
                x_pos[p * nrhs + c] = xi;
            }
        }
        const bool level_done = it1.level != it0.level;
        if (level_done) cluster.sync();                         // uniform over the cluster: the items are

        it0 = it1; it1 = it2; it2 = lv_next(it2, teams, level_ptr, nlevels);
        k0_1 = k0_2; k1_1 = k1_2;
        e0 = e1;
    }
    cluster.sync();                                             // no CTA leaves while a peer may still read its ring
}

static size_t level_plan_workspace_bytes(int64_t n) {
    const size_t m = (size_t)(n > 0 ? n : 1);
    return 2 * Workspace::pad(m * sizeof(int32_t)) + Workspace::pad(8 * sizeof(int32_t)) + Workspace::pad(scan_scratch_bytes(n));
}

template <typename I>
int level_plan(int64_t n, const I* indices, const I* indptr, const I* perm, bool lower, const int32_t* order,
               const int32_t* level_ptr, int64_t nlevels, int32_t* pos_ptr, int32_t* dep, int32_t* src,
               int64_t* info_host, void* workspace, size_t bytes, cudaStream_t st) {
    Workspace ws(workspace, bytes);
    int32_t* inv = ws.take<int32_t>((size_t)n);
    int32_t* count = ws.take<int32_t>((size_t)n);
    int32_t* info = ws.take<int32_t>(8);
    const size_t ssb = scan_scratch_bytes(n);
    char* scratch = ws.take<char>(ssb);
    if (!ws.ok()) return NB200_ERR_WORKSPACE;
    const int64_t want = ceil_div(n, (int64_t)256);
    const unsigned grid = (unsigned)(want > (int64_t)kSMs * 16 ? (int64_t)kSMs * 16 : want);
    if (cudaMemsetAsync(info, 0, 8 * sizeof(int32_t), st) != cudaSuccess) return NB200_ERR_CUDA;
    lv_inverse_kernel<<<grid, 256, 0, st>>>(n, order, inv);
    lv_count_kernel<I><<<grid, 256, 0, st>>>(n, indices, indptr, order, lower, count);
    const int rc = exclusive_scan_i32_to_i32(n, count, pos_ptr, scratch, ssb, st);
    if (rc != NB200_OK) return rc;
    lv_fill_kernel<I><<<grid, 256, 0, st>>>(n, indices, indptr, perm, order, inv, level_ptr, (int32_t)nlevels, lower,
                                            pos_ptr, dep, src, info);
    int32_t host[8] = {0};
    int32_t total = 0;
    if (cudaMemcpyAsync(host, info, sizeof(host), cudaMemcpyDeviceToHost, st) != cudaSuccess) return NB200_ERR_CUDA;
    if (cudaMemcpyAsync(&total, pos_ptr + n, sizeof(int32_t), cudaMemcpyDeviceToHost, st) != cudaSuccess) return NB200_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return NB200_ERR_CUDA;
    info_host[0] = total;
    info_host[1] = host[0];
    info_host[2] = host[1];
    info_host[3] = host[2];
    return launch_status();
}

template <int TS>
static int launch_cluster(int C, size_t smem, cudaStream_t st, int64_t nrhs, const int32_t* pos_ptr, const int32_t* dep,
                          const double* val, const int32_t* level_ptr, int32_t nlevels, bool unit, const double* b_pos,
                          double* x_pos, int cap_shift) {
    auto kernel = sptrsv_cluster_kernel<TS>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return NB200_ERR_CUDA;
    if (C > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) return NB200_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)C, 1, 1);
    cfg.blockDim = dim3(kLevelThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, nrhs, pos_ptr, dep, val, level_ptr, nlevels, unit, b_pos, x_pos, cap_shift) != cudaSuccess) {
        (void)cudaGetLastError();
        return NB200_ERR_CUDA;
    }
    return NB200_OK;
}

}  // namespace nb200

using namespace nb200;

extern "C" size_t nb200_sptrsv_level_plan_workspace_bytes(int64_t n) { return level_plan_workspace_bytes(n); }

extern "C" int nb200_sptrsv_level_plan(int64_t n, int64_t nnz, const void* indices, const void* indptr, const void* perm,
                                       int itype, int lower, const int32_t* order, const int32_t* level_ptr,
                                       int64_t nlevels, int32_t* pos_ptr, int32_t* dep, int32_t* src, int64_t* info_host,
                                       void* workspace, size_t workspace_bytes, nb200_stream stream) {
    if (n <= 0 || nnz < 0 || nlevels <= 0 || !info_host) return NB200_ERR_BAD_ARG;
    if (n >= 0x7fffffffLL || nnz >= 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    if (!indptr || !order || !level_ptr || !pos_ptr || !workspace || (nnz > 0 && (!indices || !dep || !src))) return NB200_ERR_BAD_ARG;
    return NB200_DISPATCH_I(itype,
        (level_plan<I>(n, (const I*)indices, (const I*)indptr, (const I*)perm, lower != 0, order, level_ptr, nlevels,
                       pos_ptr, dep, src, info_host, workspace, workspace_bytes, as_stream(stream))));
}

extern "C" size_t nb200_sptrsv_solve_levels_workspace_bytes(int64_t n, int64_t nrhs, int64_t entries) {
    const size_t m = (size_t)(n > 0 ? n : 1) * (size_t)(nrhs > 0 ? nrhs : 1);
    return Workspace::pad((size_t)(entries > 0 ? entries : 1) * sizeof(double)) + 2 * Workspace::pad(m * sizeof(double));
}

extern "C" int nb200_sptrsv_solve_levels(int64_t n, int64_t nrhs, int64_t entries, const void* data, const int32_t* src,
                                         const int32_t* pos_ptr, const int32_t* dep, const int32_t* order,
                                         const int32_t* level_ptr, int64_t nlevels, int64_t reach, int unit,
                                         const void* b, void* x, void* workspace, size_t workspace_bytes,
                                         int cluster_ctas, int dtype, nb200_stream stream) {
    if (n < 0 || nrhs < 0 || entries < 0 || nlevels < 0 || reach < 0) return NB200_ERR_BAD_ARG;
    if (n == 0 || nrhs == 0) return NB200_OK;
    if (!data || !src || !pos_ptr || !dep || !order || !level_ptr || !b || !x || !workspace) return NB200_ERR_BAD_ARG;
    if (n >= 0x7fffffffLL || nlevels >= 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    const int C = cluster_ctas == 0 ? 8 : cluster_ctas;
    if (C != 1 && C != 2 && C != 4 && C != 8 && C != 16) return NB200_ERR_BAD_ARG;
    // rows per CTA of the ring: a power of two, C * cap >= reach
    int cap_shift = 0;
    while (((int64_t)C << cap_shift) < reach) ++cap_shift;
    const size_t smem = ((size_t)1 << cap_shift) * (size_t)nrhs * sizeof(double);
    if (smem > (size_t)200 * 1024) return NB200_ERR_TOO_LARGE;
    cudaStream_t st = as_stream(stream);
    Workspace ws(workspace, workspace_bytes);
    double* val = ws.take<double>((size_t)(entries > 0 ? entries : 1));
    double* b_pos = ws.take<double>((size_t)n * (size_t)nrhs);
    double* x_pos = ws.take<double>((size_t)n * (size_t)nrhs);
    if (!ws.ok()) return NB200_ERR_WORKSPACE;
    const int64_t work = n * nrhs > entries ? n * nrhs : entries;
    const int64_t want = ceil_div(work, (int64_t)256);
    const unsigned grid = (unsigned)(want > (int64_t)kSMs * 16 ? (int64_t)kSMs * 16 : want);
    int ts = 1;
    while (ts < 32 && ts < nrhs) ts <<= 1;
    int rc = NB200_DISPATCH_T(dtype,
        (lv_gather_kernel<T><<<grid, 256, 0, st>>>(entries, (const T*)data, src, val, n, nrhs, order, (const T*)b, b_pos),
         launch_status()));
    if (rc != NB200_OK) return rc;
#define NB200_LV(TS_) rc = launch_cluster<TS_>(C, smem, st, nrhs, pos_ptr, dep, val, level_ptr, (int32_t)nlevels, unit != 0, \
                                               b_pos, x_pos, cap_shift)
    switch (ts) {
        case 1: NB200_LV(1); break;
        case 2: NB200_LV(2); break;
        case 4: NB200_LV(4); break;
        case 8: NB200_LV(8); break;
        case 16: NB200_LV(16); break;
        default: NB200_LV(32); break;
    }
#undef NB200_LV
    if (rc != NB200_OK) return rc;
    return NB200_DISPATCH_T(dtype,
        (lv_scatter_kernel<T><<<grid, 256, 0, st>>>(n, nrhs, order, x_pos, (T*)x), launch_status()));
}
