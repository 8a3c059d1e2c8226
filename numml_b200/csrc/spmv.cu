// SpMV forward and backward for CSR on sm_100a.
//
// Row-streaming kernels (short rows, the stencil case): a CTA owns a block of consecutive rows
// and therefore a contiguous range of nonzeros.  It streams that range with 128-bit loads
// (4 consecutive entries per thread per load), gathers x through the read-only path, parks the
// products in shared memory, and then one thread per row adds its row's products in storage
// order.  All DRAM traffic is coalesced; x lives in L2/L1.  Because multiply and add are kept
// separate and the order is the storage order, y is bit-identical to a sequential CPU loop.
//
// Vector kernel (long rows): one warp per row, lanes stride over the row, shuffle reduction.
//
// Backward: grad_A[k] = g[row(k)] * x[col(k)] is produced by the same streaming pass with g
// expanded to nonzero granularity in shared memory.  grad_x = A^T g is either folded into that
// pass with floating-point atomics, or computed by the forward kernel on a cached transposed
// structure whose values are gathered through a permutation (atomic-free, deterministic).
#include "common.cuh"
#include "spmv_pipe.cuh"
#include <type_traits>

namespace nb200 {

template <typename T>
__device__ __forceinline__ void store4_shared(T* p, const T (&v)[4]);
template <>
__device__ __forceinline__ void store4_shared<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4_shared<double>(double* p, const double (&v)[4]) {
    *reinterpret_cast<double2*>(p) = make_double2(v[0], v[1]);
    *reinterpret_cast<double2*>(p + 2) = make_double2(v[2], v[3]);
}

// ---------------------------------------------------------------------------------------------
// Forward, row-streaming.  TILE = THREADS*U*4 nonzeros per pass through shared memory.
// ---------------------------------------------------------------------------------------------
template <typename T, typename I, int THREADS, int U, bool PERM>
__global__ void __launch_bounds__(THREADS)
spmv_stream_kernel(int64_t rows, int64_t nnz, int rows_per_cta,
                   const T* __restrict__ data, const I* __restrict__ indices,
                   const I* __restrict__ indptr, const I* __restrict__ perm,
                   const T* __restrict__ x, T* __restrict__ y) {
    constexpr int TILE = THREADS * U * 4;
    __shared__ __align__(16) T prod[TILE];

    const int tid = threadIdx.x;
    const int64_t r0 = (int64_t)blockIdx.x * rows_per_cta;
    const int64_t r1 = min(r0 + (int64_t)rows_per_cta, rows);
    const int64_t cta_begin = (int64_t)indptr[r0];
    const int64_t cta_end = (int64_t)indptr[r1];
    const int64_t r = r0 + tid;
    const bool has_row = (tid < rows_per_cta) && (r < r1);
    int64_t s = 0, e = 0;
    if (has_row) { s = (int64_t)indptr[r]; e = (int64_t)indptr[r + 1]; }

    T acc = 0;
    for (int64_t base = cta_begin & ~(int64_t)3; base < cta_end; base += TILE) {
        T v[U][4];
        I c[U][4];
        bool live[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t k = base + (int64_t)(u * THREADS + tid) * 4;
            live[u] = k < cta_end;
            if (live[u]) {
                if (k + 4 <= nnz) {
                    load4_stream(indices + k, c[u]);
                    if (!PERM) {
                        load4_stream(data + k, v[u]);
                    } else {
                        I pm[4];
                        load4_stream(perm + k, pm);
#pragma unroll
                        for (int j = 0; j < 4; ++j) v[u][j] = ldg(data + pm[j]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const bool ok = k + j < nnz;
                        c[u][j] = ok ? indices[k + j] : (I)0;
                        v[u][j] = ok ? (PERM ? data[perm[k + j]] : data[k + j]) : (T)0;
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (live[u]) {
                T p[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) p[j] = mul_rn(v[u][j], ldg(x + c[u][j]));
                store4_shared(prod + (u * THREADS + tid) * 4, p);
            }
        }
        __syncthreads();
        if (has_row) {
            const int lo = (int)(max(s, base) - base);
            const int hi = (int)(min(e, base + TILE) - base);
            for (int k = lo; k < hi; ++k) acc = add_rn(acc, prod[k]);
        }
        __syncthreads();
    }
    if (has_row) y[r] = acc;
}

// ---------------------------------------------------------------------------------------------
// Forward, one warp per row (long rows).
// ---------------------------------------------------------------------------------------------
template <typename T, typename I, bool PERM>
__global__ void __launch_bounds__(256)
spmv_vector_kernel(int64_t rows, const T* __restrict__ data, const I* __restrict__ indices,
                   const I* __restrict__ indptr, const I* __restrict__ perm,
                   const T* __restrict__ x, T* __restrict__ y) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const int64_t s = (int64_t)indptr[r], e = (int64_t)indptr[r + 1];
        T acc = 0;
        for (int64_t k = s + lane; k < e; k += 32) {
            const T a = PERM ? ldg(data + perm[k]) : data[k];
            acc += a * ldg(x + indices[k]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) y[r] = acc;
    }
}

// ---------------------------------------------------------------------------------------------
// Backward, row-streaming: grad_A[k] = g[row(k)] * x[col(k)], and with ATOMIC also
// grad_x[col(k)] += g[row(k)] * data[k].
// ---------------------------------------------------------------------------------------------
template <typename T, typename I, int THREADS, int U, bool ATOMIC>
__global__ void __launch_bounds__(THREADS)
spmv_bwd_stream_kernel(int64_t rows, int64_t nnz, int rows_per_cta,
                       const T* __restrict__ data, const I* __restrict__ indices,
                       const I* __restrict__ indptr, const T* __restrict__ x,
                       const T* __restrict__ g, T* __restrict__ grad_A, T* __restrict__ grad_x) {
    constexpr int TILE = THREADS * U * 4;
    __shared__ __align__(16) T gexp[TILE];

    const int tid = threadIdx.x;
    const int64_t r0 = (int64_t)blockIdx.x * rows_per_cta;
    const int64_t r1 = min(r0 + (int64_t)rows_per_cta, rows);
    const int64_t cta_begin = (int64_t)indptr[r0];
    const int64_t cta_end = (int64_t)indptr[r1];
    const int64_t r = r0 + tid;
    const bool has_row = (tid < rows_per_cta) && (r < r1);
    int64_t s = 0, e = 0;
    T gr = 0;
    if (has_row) { s = (int64_t)indptr[r]; e = (int64_t)indptr[r + 1]; gr = g[r]; }

    for (int64_t base = cta_begin & ~(int64_t)3; base < cta_end; base += TILE) {
        T v[U][4];
        I c[U][4];
        bool live[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t k = base + (int64_t)(u * THREADS + tid) * 4;
            live[u] = k < cta_end;
            if (live[u]) {
                if (k + 4 <= nnz) {
                    load4_stream(indices + k, c[u]);
                    if (ATOMIC) load4_stream(data + k, v[u]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const bool ok = k + j < nnz;
                        c[u][j] = ok ? indices[k + j] : (I)0;
                        if (ATOMIC) v[u][j] = ok ? data[k + j] : (T)0;
                    }
                }
            }
        }
        // expand g to nonzero granularity while the streaming loads are in flight
        if (has_row) {
            const int lo = (int)(max(s, base) - base);
            const int hi = (int)(min(e, base + TILE) - base);
            for (int k = lo; k < hi; ++k) gexp[k] = gr;
        }
        T xv[U][4];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (live[u]) {
#pragma unroll
                for (int j = 0; j < 4; ++j) xv[u][j] = ldg(x + c[u][j]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (live[u]) {
                const int off = (u * THREADS + tid) * 4;
                const int64_t k = base + off;
                if (k >= cta_begin && k + 4 <= cta_end) {
                    T out[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) out[j] = mul_rn(gexp[off + j], xv[u][j]);
                    store4_stream(grad_A + k, out);
                    if (ATOMIC) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) atomicAdd(grad_x + c[u][j], mul_rn(gexp[off + j], v[u][j]));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (k + j >= cta_begin && k + j < cta_end) {
                            const T ge = gexp[off + j];
                            grad_A[k + j] = mul_rn(ge, xv[u][j]);
                            if (ATOMIC) atomicAdd(grad_x + c[u][j], mul_rn(ge, v[u][j]));
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
}

// Backward grad_A for long rows: one warp per row.
template <typename T, typename I, bool ATOMIC>
__global__ void __launch_bounds__(256)
spmv_bwd_vector_kernel(int64_t rows, const T* __restrict__ data, const I* __restrict__ indices,
                       const I* __restrict__ indptr, const T* __restrict__ x, const T* __restrict__ g,
                       T* __restrict__ grad_A, T* __restrict__ grad_x) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const int64_t s = (int64_t)indptr[r], e = (int64_t)indptr[r + 1];
        const T gr = g[r];
        for (int64_t k = s + lane; k < e; k += 32) {
            const I c = indices[k];
            grad_A[k] = mul_rn(gr, ldg(x + c));
            if (ATOMIC) atomicAdd(grad_x + c, mul_rn(gr, data[k]));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Host-side launchers
// ---------------------------------------------------------------------------------------------
constexpr int kStreamThreads = 256;
constexpr int kStreamU = 2;
constexpr int kStreamTile = kStreamThreads * kStreamU * 4;
constexpr double kStreamMaxMeanRow = 24.0;  // above this the warp-per-row kernels take over

static inline int stream_rows_per_cta(int64_t rows, int64_t nnz) {
    const double mean = rows > 0 ? (double)nnz / (double)rows : 0.0;
    int rpc = mean > 0 ? (int)((double)kStreamTile / mean) : kStreamThreads;
    if (rpc > kStreamThreads) rpc = kStreamThreads;
    if (rpc < 1) rpc = 1;
    return rpc;
}

template <typename T, typename I>
int spmv_forward_launch(int64_t rows, int64_t nnz, const T* data, const I* indices, const I* indptr,
                        const I* perm, const T* x, T* y, int block_rows, int32_t* status, cudaStream_t st) {
    if (rows == 0) return NB200_OK;
    if (block_rows > 0 && nnz > 0)
        return spmv_pipe_forward<T, I>(rows, nnz, block_rows, data, indices, indptr, perm, x, y, status, st);
    const double mean = (double)nnz / (double)rows;
    if (mean <= kStreamMaxMeanRow || block_rows < 0) {
        // block_rows < 0: the caller passes a sub-range of rows, for which nnz / rows says nothing
        const int rpc = block_rows < 0 ? kStreamThreads : stream_rows_per_cta(rows, nnz);
        const int64_t grid = ceil_div(rows, (int64_t)rpc);
        if (grid > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
        if (perm)
            spmv_stream_kernel<T, I, kStreamThreads, kStreamU, true><<<(unsigned)grid, kStreamThreads, 0, st>>>(
                rows, nnz, rpc, data, indices, indptr, perm, x, y);
        else
            spmv_stream_kernel<T, I, kStreamThreads, kStreamU, false><<<(unsigned)grid, kStreamThreads, 0, st>>>(
                rows, nnz, rpc, data, indices, indptr, perm, x, y);
    } else {
        const int64_t want = ceil_div(rows, (int64_t)8);
        const unsigned grid = (unsigned)min(want, (int64_t)kSMs * 64);
        if (perm)
            spmv_vector_kernel<T, I, true><<<grid, 256, 0, st>>>(rows, data, indices, indptr, perm, x, y);
        else
            spmv_vector_kernel<T, I, false><<<grid, 256, 0, st>>>(rows, data, indices, indptr, perm, x, y);
    }
    return launch_status();
}

template <typename T, typename I>
int spmv_backward_launch(int64_t rows, int64_t cols, int64_t nnz, const T* data, const I* indices,
                         const I* indptr, const T* x, const T* g, const I* t_indptr,
                         const I* t_indices, const I* t_perm, T* grad_A, T* grad_x, int block_rows, int t_block_rows,
                         int symmetry, int32_t* status, cudaStream_t st) {
    const bool atomic = (t_indptr == nullptr);
    if (!atomic && (symmetry & NB200_SYMMETRIC_PATTERN) && block_rows > 0 && rows == cols && nnz > 0)
        return spmv_pipe_backward_sym<T, I>(0, rows, nnz, block_rows, data, indices, indptr, t_perm, x, g, grad_A, grad_x,
                                            (symmetry & NB200_SYMMETRIC_VALUES) != 0, status, st);
    if (atomic && cols > 0) {
        if (cudaMemsetAsync(grad_x, 0, sizeof(T) * (size_t)cols, st) != cudaSuccess) return NB200_ERR_CUDA;
    }
    if (rows > 0 && nnz > 0) {
        const double mean = (double)nnz / (double)rows;
        if (!atomic && block_rows > 0) {
            int rc = spmv_pipe_grad_A<T, I>(rows, nnz, block_rows, indices, indptr, x, g, grad_A, status, st);
            if (rc != NB200_OK) return rc;
        } else if (mean <= kStreamMaxMeanRow) {
            const int rpc = stream_rows_per_cta(rows, nnz);
            const int64_t grid = ceil_div(rows, (int64_t)rpc);
            if (grid > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
            if (atomic)
                spmv_bwd_stream_kernel<T, I, kStreamThreads, kStreamU, true><<<(unsigned)grid, kStreamThreads, 0, st>>>(
                    rows, nnz, rpc, data, indices, indptr, x, g, grad_A, grad_x);
            else
                spmv_bwd_stream_kernel<T, I, kStreamThreads, kStreamU, false><<<(unsigned)grid, kStreamThreads, 0, st>>>(
                    rows, nnz, rpc, data, indices, indptr, x, g, grad_A, grad_x);
        } else {
            const int64_t want = ceil_div(rows, (int64_t)8);
            const unsigned grid = (unsigned)min(want, (int64_t)kSMs * 64);
            if (atomic)
                spmv_bwd_vector_kernel<T, I, true><<<grid, 256, 0, st>>>(rows, data, indices, indptr, x, g, grad_A, grad_x);
            else
                spmv_bwd_vector_kernel<T, I, false><<<grid, 256, 0, st>>>(rows, data, indices, indptr, x, g, grad_A, grad_x);
        }
        int rc = launch_status();
        if (rc != NB200_OK) return rc;
    }
    if (!atomic) {
        // grad_x = A^T g through the transposed structure: rows of A^T are the columns of A.
        return spmv_forward_launch<T, I>(cols, nnz, data, t_indices, t_indptr, t_perm, g, grad_x, t_block_rows, status, st);
    }
    return NB200_OK;
}

}  // namespace nb200

using namespace nb200;

extern "C" int nb200_spgemv_forward(int64_t rows, int64_t cols, int64_t nnz,
                                    const void* data, const void* indices, const void* indptr,
                                    const void* perm, const void* x, void* y,
                                    int block_rows, int32_t* status,
                                    int dtype, int itype, nb200_stream stream) {
    if (rows < 0 || cols < 0 || nnz < 0) return NB200_ERR_BAD_ARG;
    if (rows == 0) return NB200_OK;
    if (block_rows < -1 || block_rows > 256) return NB200_ERR_BAD_ARG;
    if (!indptr || !y || (nnz > 0 && (!data || !indices || !x))) return NB200_ERR_BAD_ARG;
    if (!aligned16(data) || !aligned16(indices) || !aligned16(perm)) return NB200_ERR_ALIGN;
    if (itype == NB200_I32 && nnz > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    return NB200_DISPATCH(dtype, itype,
        (spmv_forward_launch<T, I>(rows, nnz, (const T*)data, (const I*)indices, (const I*)indptr,
                                   (const I*)perm, (const T*)x, (T*)y, block_rows, status, as_stream(stream))));
}

extern "C" int nb200_spgemv_backward(int64_t rows, int64_t cols, int64_t nnz,
                                     const void* data, const void* indices, const void* indptr,
                                     const void* x, const void* g,
                                     const void* t_indptr, const void* t_indices, const void* t_perm,
                                     void* grad_A, void* grad_x,
                                     int block_rows, int t_block_rows, int pattern_symmetric, int32_t* status,
                                     int dtype, int itype, nb200_stream stream) {
    if (rows < 0 || cols < 0 || nnz < 0) return NB200_ERR_BAD_ARG;
    if (!indptr || (cols > 0 && !grad_x) || (nnz > 0 && (!data || !indices || !x || !g || !grad_A)))
        return NB200_ERR_BAD_ARG;
    if (t_indptr != nullptr && nnz > 0 && (!t_indices || !t_perm)) return NB200_ERR_BAD_ARG;
    if (block_rows < 0 || block_rows > 256 || t_block_rows < 0 || t_block_rows > 256) return NB200_ERR_BAD_ARG;
    if (!aligned16(data) || !aligned16(indices) || !aligned16(grad_A) || !aligned16(t_indices) || !aligned16(t_perm))
        return NB200_ERR_ALIGN;
    if (itype == NB200_I32 && nnz > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    return NB200_DISPATCH(dtype, itype,
        (spmv_backward_launch<T, I>(rows, cols, nnz, (const T*)data, (const I*)indices, (const I*)indptr,
                                    (const T*)x, (const T*)g, (const I*)t_indptr, (const I*)t_indices,
                                    (const I*)t_perm, (T*)grad_A, (T*)grad_x, block_rows, t_block_rows,
                                    pattern_symmetric, status, as_stream(stream))));
}


// The fused one-pass backward on a contiguous range of rows of a matrix whose pattern equals its
// transpose.  All arrays are indexed absolutely; a row-partitioned driver runs the rows that feed
// its exchange first and the rest while the exchange is in flight.
extern "C" int nb200_spgemv_backward_symmetric_rows(int64_t n, int64_t nnz, int64_t row_begin, int64_t row_end,
                                                    const void* data, const void* indices, const void* indptr,
                                                    const void* t_perm, const void* x, const void* g,
                                                    void* grad_A, void* grad_x, int values_symmetric, int block_rows,
                                                    int32_t* status, int dtype, int itype, nb200_stream stream) {
    if (n < 0 || nnz < 0 || row_begin < 0 || row_end < row_begin || row_end > n) return NB200_ERR_BAD_ARG;
    if (block_rows < 1 || block_rows > 256) return NB200_ERR_BAD_ARG;
    if (row_end == row_begin || nnz == 0) return NB200_OK;
    if (!data || !indices || !indptr || !t_perm || !x || !g || !grad_A || !grad_x) return NB200_ERR_BAD_ARG;
    // bulk copies of the index streams and two-entry vector stores of grad_A
    if (!aligned16(indices) || !aligned16(t_perm) || !aligned16(grad_A) || (values_symmetric && !aligned16(data))) return NB200_ERR_ALIGN;
    if (itype == NB200_I32 && nnz > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    return NB200_DISPATCH(dtype, itype,
        (spmv_pipe_backward_sym<T, I>(row_begin, row_end, nnz, block_rows, (const T*)data, (const I*)indices,
                                      (const I*)indptr, (const I*)t_perm, (const T*)x, (const T*)g, (T*)grad_A,
                                      (T*)grad_x, values_symmetric != 0, status, as_stream(stream))));
}

// Does A equal its transpose in value?  With t_perm[k] = position in A of the mirror image of entry k
// (the permutation of the transposed structure of a pattern that equals its transpose), that is
// data[t_perm[k]] == data[k] for every k, compared as bit patterns.  The device word `mismatch` is
// OR-ed with 1 when some entry differs; the caller zeroes it first.
namespace nb200 {
template <typename T, typename I>
__global__ void values_symmetric_kernel(int64_t nnz, const T* __restrict__ data, const I* __restrict__ t_perm,
                                        int32_t* __restrict__ mismatch) {
    using Bits = typename std::conditional<sizeof(T) == 8, unsigned long long, unsigned int>::type;
    const Bits* bits = reinterpret_cast<const Bits*>(data);
    bool differs = false;
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < nnz; k += (int64_t)gridDim.x * blockDim.x)
        differs |= bits[k] != __ldg(bits + t_perm[k]);
    if (__any_sync(0xffffffffu, differs) && (threadIdx.x & 31) == 0) atomicOr(mismatch, 1);
}
}  // namespace nb200

extern "C" int nb200_csr_values_symmetric(int64_t nnz, const void* data, const void* t_perm, int32_t* mismatch,
                                          int dtype, int itype, nb200_stream stream) {
    if (nnz < 0 || !mismatch || (nnz > 0 && (!data || !t_perm))) return NB200_ERR_BAD_ARG;
    if (nnz == 0) return NB200_OK;
    const int64_t want = ceil_div(nnz, (int64_t)1024);
    const unsigned grid = (unsigned)(want > (int64_t)kSMs * 16 ? (int64_t)kSMs * 16 : want);
    return NB200_DISPATCH(dtype, itype,
        (values_symmetric_kernel<T, I><<<grid, 256, 0, as_stream(stream)>>>(nnz, (const T*)data, (const I*)t_perm, mismatch),
         launch_status()));
}

// grad_A alone (the masked outer product g x^T on the pattern), for callers that schedule the
// two halves of the backward separately (the row-partitioned driver overlaps them with its
// halo exchange).
extern "C" int nb200_spgemv_grad_A(int64_t rows, int64_t cols, int64_t nnz,
                                   const void* indices, const void* indptr, const void* x, const void* g,
                                   void* grad_A, int block_rows, int32_t* status,
                                   int dtype, int itype, nb200_stream stream) {
    (void)cols;
    if (rows < 0 || nnz < 0 || block_rows < 0 || block_rows > 256) return NB200_ERR_BAD_ARG;
    if (rows == 0 || nnz == 0) return NB200_OK;
    if (!indices || !indptr || !x || !g || !grad_A) return NB200_ERR_BAD_ARG;
    if (!aligned16(indices) || !aligned16(grad_A)) return NB200_ERR_ALIGN;
    if (itype == NB200_I32 && nnz > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    cudaStream_t st = as_stream(stream);
    return NB200_DISPATCH(dtype, itype, ([&]() -> int {
        if (block_rows > 0)
            return spmv_pipe_grad_A<T, I>(rows, nnz, block_rows, (const I*)indices, (const I*)indptr, (const T*)x,
                                          (const T*)g, (T*)grad_A, status, st);
        const double mean = (double)nnz / (double)rows;
        if (mean <= kStreamMaxMeanRow) {
            const int rpc = stream_rows_per_cta(rows, nnz);
            const int64_t grid = ceil_div(rows, (int64_t)rpc);
            if (grid > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
            spmv_bwd_stream_kernel<T, I, kStreamThreads, kStreamU, false><<<(unsigned)grid, kStreamThreads, 0, st>>>(
                rows, nnz, rpc, (const T*)nullptr, (const I*)indices, (const I*)indptr, (const T*)x, (const T*)g,
                (T*)grad_A, (T*)nullptr);
        } else {
            const int64_t want = ceil_div(rows, (int64_t)8);
            const unsigned grid = (unsigned)min(want, (int64_t)kSMs * 64);
            spmv_bwd_vector_kernel<T, I, false><<<grid, 256, 0, st>>>(rows, (const T*)nullptr, (const I*)indices,
                                                                      (const I*)indptr, (const T*)x, (const T*)g,
                                                                      (T*)grad_A, (T*)nullptr);
        }
        return launch_status();
    }()));
}

// ---------------------------------------------------------------------------------------------
// Block profile: the largest number of entries in any block of R consecutive rows, for
// R = 256, 128, 64, 32.  The host picks the largest R whose maximum fits one pipeline stage.
// ---------------------------------------------------------------------------------------------
namespace nb200 {
template <typename I>
__global__ void csr_block_profile_kernel(int64_t rows, const I* __restrict__ indptr, unsigned long long* __restrict__ out) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int64_t R = 256 >> c;
        const int64_t blocks = ceil_div(rows, R);
        long long best = 0;
        for (int64_t b = gtid; b < blocks; b += stride) {
            const int64_t r1 = min((b + 1) * R, rows);
            best = max(best, (long long)indptr[r1] - (long long)indptr[b * R]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
        if ((threadIdx.x & 31) == 0 && best > 0) atomicMax(out + c, (unsigned long long)best);
    }
}
}  // namespace nb200

extern "C" int nb200_spmv_pipeline_tile(void) { return kSpmvPipeTile; }

extern "C" int nb200_csr_block_profile(int64_t rows, const void* indptr, int itype, int64_t* out4, nb200_stream stream) {
    if (rows < 0 || !out4 || (rows > 0 && !indptr)) return NB200_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    if (cudaMemsetAsync(out4, 0, 4 * sizeof(int64_t), st) != cudaSuccess) return NB200_ERR_CUDA;
    if (rows == 0) return NB200_OK;
    const int64_t want = ceil_div(ceil_div(rows, (int64_t)32), (int64_t)256);
    const unsigned grid = (unsigned)(want > (int64_t)kSMs * 8 ? (int64_t)kSMs * 8 : want);
    return NB200_DISPATCH_I(itype,
        (csr_block_profile_kernel<I><<<grid, 256, 0, st>>>(rows, (const I*)indptr, (unsigned long long*)out4), launch_status()));
}
