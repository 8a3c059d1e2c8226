// Interface of the TMA-pipelined SpMV kernels (spmv_pipe.cu), used by the launchers in spmv.cu.
#pragma once
#include "common.cuh"

namespace nb200 {

// Entries per pipeline stage and rows per block (= consumer threads per CTA).  Overridable at
// compile time for tuning builds; the shipped library uses the defaults.
#ifndef NB200_PIPE_TILE
#define NB200_PIPE_TILE 2048
#endif
#ifndef NB200_PIPE_ROWS
#define NB200_PIPE_ROWS 256
#endif
constexpr int kSpmvPipeTile = NB200_PIPE_TILE;
constexpr int kSpmvPipeRows = NB200_PIPE_ROWS;

// y = A x (perm == nullptr) or y[r] = sum_k data[perm[k]] x[indices[k]] over a transposed structure.
// Requires every block of `block_rows` (<= 256) consecutive rows to hold at most kSpmvPipeTile entries.
template <typename T, typename I>
int spmv_pipe_forward(int64_t rows, int64_t nnz, int block_rows, const T* data, const I* indices, const I* indptr,
                      const I* perm, const T* x, T* y, int32_t* status, cudaStream_t st);

// grad_A[k] = g[row(k)] * x[indices[k]], same requirement.
template <typename T, typename I>
int spmv_pipe_grad_A(int64_t rows, int64_t nnz, int block_rows, const I* indices, const I* indptr, const T* x,
                     const T* g, T* grad_A, int32_t* status, cudaStream_t st);

// Whole backward in one pass for a pattern that equals its transpose (t_indptr == indptr and
// t_indices == indices, so only the permutation of the transposed structure is needed):
// grad_A[k] = g[row(k)] x[col(k)] and grad_x[i] = sum_k data[perm[k]] g[col(k)] over row i.
// Handles rows [row_begin, row_end); every array is indexed absolutely.
// `values_symmetric`: the caller has established that data[perm[k]] == data[k] bit for bit for every k
// (A equals its transpose in value too); the pass then reads `data` as a stream and never touches `perm`.
template <typename T, typename I>
int spmv_pipe_backward_sym(int64_t row_begin, int64_t row_end, int64_t nnz, int block_rows, const T* data,
                           const I* indices, const I* indptr, const I* perm, const T* x, const T* g, T* grad_A,
                           T* grad_x, bool values_symmetric, int32_t* status, cudaStream_t st);

}  // namespace nb200
