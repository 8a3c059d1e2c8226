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
