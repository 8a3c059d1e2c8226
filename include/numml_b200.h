/*
 * numml_b200 -- C ABI of the sm_100a differentiable-CSR kernels.
 *
 * This is the drop-in boundary underneath the operator functions that the reference registers
 * in its `numml_torch_cpp` extension module (reference cpp/sparse_csr.cpp:307-319, prototypes in
 * cpp/sparse_csr.hpp:32-105).  Every entry point takes plain device pointers and sizes, a CUDA
 * stream as an opaque pointer, and returns an `nb200_status`; nothing here depends on torch.
 *
 * Conventions
 *   - matrices are CSR: data[nnz] (float or double), indices[nnz], indptr[rows+1]; index arrays
 *     are int32 or int64 as selected by `itype` (the reference stores int64; a narrowed int32
 *     copy halves the index traffic and is what the host layer caches per sparsity pattern);
 *   - `dtype` is an nb200_dtype, `itype` an nb200_itype;
 *   - all pointers are device pointers on the current device unless stated otherwise; data,
 *     indices and the nnz-sized outputs must be 16-byte aligned (128-bit loads and stores);
 *   - inputs are borrowed and never written; outputs and workspaces are caller-allocated, the
 *     library allocates no device memory (the one exception, at set-up time, is nb200_ipc_alloc);
 *     every call is asynchronous on `stream`;
 *   - columns within a row are expected in ascending order wherever the reference expects it
 *     (SpGEMM backward, triangular solve).
 */
#ifndef NUMML_B200_H_
#define NUMML_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    NB200_OK = 0,
    NB200_ERR_BAD_ARG = 1,      /* null pointer, negative size, unknown dtype / itype            */
    NB200_ERR_ALIGN = 2,        /* a pointer that must be 16-byte aligned is not                 */
    NB200_ERR_TOO_LARGE = 3,    /* a size exceeds what the index width / kernel supports         */
    NB200_ERR_PRECONDITION = 4, /* structural precondition violated (reported via status word)   */
    NB200_ERR_WAIT_BUDGET = 5,  /* a bounded device-side wait ran out (reported via status word) */
    NB200_ERR_WORKSPACE = 6,    /* workspace too small                                           */
    NB200_ERR_CUDA = 7          /* a CUDA runtime call or launch failed                          */
} nb200_status;

typedef enum { NB200_F32 = 0, NB200_F64 = 1 } nb200_dtype;
typedef enum { NB200_I32 = 0, NB200_I64 = 1 } nb200_itype;

typedef void* nb200_stream; /* a cudaStream_t */

#if defined(__GNUC__)
#define NB200_API __attribute__((visibility("default")))
#else
#define NB200_API
#endif

/* Library version (major*10000 + minor*100 + patch) and a printable name for a status. */
NB200_API int nb200_version(void);
NB200_API const char* nb200_status_string(int status);

/* ---------------------------------------------------------------------------------------------
 * SpMV forward  y = A x.          Replaces spgemv_forward (reference cpp/sparse_csr.hpp:32-36,
 * CPU cpp/sparse_csr_cpu.cpp:11-39, CUDA cpp/sparse_csr_cuda.cu:21-67).
 * Rows are summed in storage order with an unfused multiply and add, so for matrices taken by
 * the row-streaming kernel (mean row length <= 24) the result is bit-identical to the reference
 * CPU loop.  `perm` (itype, may be NULL): when given, entry k uses data[perm[k]] -- this is how
 * a cached transposed structure is applied to the current values (y = A^T g).
 * `block_rows` selects the kernel: 0 = register-staged (row-streaming up to a mean row length of 24,
 * a warp per row with a warp-reduced dot above it; any matrix); -1 = the row-streaming kernel whatever
 * nnz / rows says (for a caller that passes a sub-range of rows: `indptr` offset by the first row, `y` likewise,
 * `nnz` still the length of the arrays); R in 1..256 = the persistent TMA-pipelined kernel, valid only if every
 * block of R consecutive rows holds at most nb200_spmv_pipeline_tile() entries (see nb200_csr_block_profile);
 * the row-streaming and the pipelined kernel give the same bits.
 * `status` (device word, may be NULL) receives NB200_ERR_WAIT_BUDGET if a bounded wait of the
 * pipelined kernel ever runs out.
 * ------------------------------------------------------------------------------------------- */
NB200_API int nb200_spgemv_forward(int64_t rows, int64_t cols, int64_t nnz,
                         const void* data, const void* indices, const void* indptr,
                         const void* perm, const void* x, void* y,
                         int block_rows, int32_t* status,
                         int dtype, int itype, nb200_stream stream);

/* Largest number of entries in any block of R consecutive rows, for R = 256, 128, 64, 32, written to
 * the four int64 device words out4[0..3]; and the entry capacity of one pipeline stage. */
NB200_API int nb200_csr_block_profile(int64_t rows, const void* indptr, int itype, int64_t* out4, nb200_stream stream);
NB200_API int nb200_spmv_pipeline_tile(void);

/* ---------------------------------------------------------------------------------------------
 * SpMV backward.                  Replaces spgemv_backward (reference cpp/sparse_csr.hpp:38-42,
 * CPU cpp/sparse_csr_cpu.cpp:41-77, CUDA cpp/sparse_csr_cuda.cu:76-170).
 *   grad_A[k] = g[row(k)] * x[col(k)]        (always; bit-identical to the reference)
 *   grad_x    = A^T g
 * With a transposed structure (t_indptr[cols+1], t_indices[nnz] = row of each entry of A^T,
 * t_perm[nnz] = position in A of each entry of A^T; see nb200_csr_transpose_structure) grad_x is
 * a gather over A^T: atomic-free, deterministic and bit-identical to the reference.  With the
 * three t_* pointers NULL grad_x is zeroed and accumulated with floating-point atomics in one
 * fused pass over A (order of additions not fixed).  `block_rows` / `t_block_rows` choose the
 * kernel for the pass over A / over A^T as in nb200_spgemv_forward (0 = streaming kernels).
 * `pattern_symmetric` is a set of NB200_SYMMETRIC_* bits.  NB200_SYMMETRIC_PATTERN asserts that the
 * pattern equals its transpose (t_indptr == indptr, t_indices == indices); with block_rows > 0 both
 * gradients then come from ONE pipelined pass that reads indices and t_perm once (same results, bit
 * for bit).  NB200_SYMMETRIC_VALUES (only together with the former) asserts in addition that the
 * values do: data[t_perm[k]] == data[k] for every k, which nb200_csr_values_symmetric establishes.
 * The pass then streams `data` and never reads t_perm: its traffic is exactly A, x, g and the two
 * outputs.  The results are again the same bit for bit, because the transposed value the pass would
 * have gathered is the entry's own.
 * ------------------------------------------------------------------------------------------- */
enum { NB200_SYMMETRIC_PATTERN = 1, NB200_SYMMETRIC_VALUES = 2 };
NB200_API int nb200_spgemv_backward(int64_t rows, int64_t cols, int64_t nnz,
                          const void* data, const void* indices, const void* indptr,
                          const void* x, const void* g,
                          const void* t_indptr, const void* t_indices, const void* t_perm,
                          void* grad_A, void* grad_x,
                          int block_rows, int t_block_rows, int pattern_symmetric, int32_t* status,
                          int dtype, int itype, nb200_stream stream);

/* The one-pass backward of nb200_spgemv_backward for a square matrix whose pattern equals its
 * transpose (so t_indptr == indptr, t_indices == indices and only t_perm is needed), restricted to
 * rows [row_begin, row_end): grad_A[k] for the entries of those rows and grad_x[i] for those i.
 * Every pointer is the base of its array (absolute indexing).  Used by the row-partitioned driver,
 * which runs the rows feeding its exchange first.  `values_symmetric` != 0: data[t_perm[k]] == data[k]
 * holds for every entry k of the rows in the range (see NB200_SYMMETRIC_VALUES above).  Needs block_rows
 * in 1..256 as described above and `data`, `indices`, `t_perm`, `grad_A` 16-byte aligned (bulk copies of
 * the streams, two-entry vector stores of grad_A); NB200_ERR_ALIGN otherwise. */
NB200_API int nb200_spgemv_backward_symmetric_rows(int64_t n, int64_t nnz, int64_t row_begin, int64_t row_end,
                                                   const void* data, const void* indices, const void* indptr,
                                                   const void* t_perm, const void* x, const void* g,
                                                   void* grad_A, void* grad_x, int values_symmetric, int block_rows,
                                                   int32_t* status, int dtype, int itype, nb200_stream stream);

/* OR-s 1 into the device word `mismatch` (zeroed by the caller) if data[t_perm[k]] != data[k], compared
 * as bit patterns, for some k < nnz: the test behind NB200_SYMMETRIC_VALUES.  The reference has no
 * counterpart; its backward (cpp/sparse_csr_cpu.cpp:41-77) always walks the values it is given. */
NB200_API int nb200_csr_values_symmetric(int64_t nnz, const void* data, const void* t_perm, int32_t* mismatch,
                                         int dtype, int itype, nb200_stream stream);

/* grad_A[k] = g[row(k)] * x[col(k)] alone: the masked outer product of spgemv_backward (reference
 * cpp/sparse_csr_cpu.cpp:59-65, cuda_kernel_masked_outerproduct cpp/sparse_csr_cuda.cu:76-95), for
 * callers that schedule the two halves of the backward themselves.  `indptr` may point into the
 * middle of a row-pointer array (a contiguous range of rows; entries are absolute positions). */
NB200_API int nb200_spgemv_grad_A(int64_t rows, int64_t cols, int64_t nnz,
                                  const void* indices, const void* indptr, const void* x, const void* g,
                                  void* grad_A, int block_rows, int32_t* status,
                                  int dtype, int itype, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * CSR transpose (structure).      Replaces csr_transpose_forward (reference
 * cpp/sparse_csr.hpp:57-60, CPU cpp/sparse_csr_cpu.cpp:311-367, CUDA cpp/sparse_csr_cuda.cu:176-279).
 * Stable counting/radix sort of the entries by column: t_indptr[cols+1], t_indices[nnz] (row of
 * each entry of A^T, ascending within a row of A^T) and t_perm[nnz] (the reference's
 * At_to_A_idx).  Outputs are written with index width `itype_out`.  Values follow with
 * nb200_gather(t_data = data[t_perm]).  Needs nnz < 2^31 and rows, cols < 2^31.
 * `workspace` must hold nb200_csr_transpose_workspace_bytes(rows, cols, nnz) bytes.
 * ------------------------------------------------------------------------------------------- */
NB200_API size_t nb200_csr_transpose_workspace_bytes(int64_t rows, int64_t cols, int64_t nnz);
NB200_API int nb200_csr_transpose_structure(int64_t rows, int64_t cols, int64_t nnz,
                                  const void* indices, const void* indptr, int itype_in,
                                  void* t_indptr, void* t_indices, void* t_perm, int itype_out,
                                  void* workspace, size_t workspace_bytes, nb200_stream stream);

/* dst[k] = src[idx[k]]  (k < n).  With nb200_csr_transpose_structure this completes
 * csr_transpose_forward (At_data = A_data[At_to_A_idx]). */
NB200_API int nb200_gather(int64_t n, const void* src, const void* idx, void* dst,
                 int dtype, int itype, nb200_stream stream);

/* dst[idx[k]] = src[k]  (k < n).  Replaces csr_transpose_backward (reference
 * cpp/sparse_csr.hpp:62-64, CPU cpp/sparse_csr_cpu.cpp:369-385, CUDA cpp/sparse_csr_cuda.cu:281-295). */
NB200_API int nb200_scatter(int64_t n, const void* src, const void* idx, void* dst,
                  int dtype, int itype, nb200_stream stream);

/* Structure check of a CSR pattern, run once per pattern by the host layer before kernels that would
 * otherwise read out of bounds (column or row-pointer out of range) or return wrong results silently
 * (the triangular solve and the SpGEMM backward rely on columns ascending within each row; a solve
 * without `unit` divides by the stored diagonal).  The reference does not check any of this
 * (its checks are device/dtype only, cpp/sparse_csr.cpp:125-148) and has undefined behaviour instead.
 * Writes the OR of the NB200_CHECK_* bits that apply into the device word `flags` (0 = clean). */
enum {
    NB200_CHECK_BAD_INDPTR = 1,    /* indptr[0] != 0, indptr[rows] != nnz, or not non-decreasing   */
    NB200_CHECK_COLUMN_RANGE = 2,  /* a column index outside [0, cols)                              */
    NB200_CHECK_UNSORTED = 4,      /* columns of a row not strictly ascending (includes duplicates) */
    NB200_CHECK_NO_DIAGONAL = 8    /* a row r < cols without a stored entry (r, r)                  */
};
NB200_API int nb200_csr_check(int64_t rows, int64_t cols, int64_t nnz, const void* indices, const void* indptr,
                              int itype, int32_t* flags, nb200_stream stream);

/* out32[k] = (int32) in64[k] and out64[k] = in32[k]: index-width conversion used when the host
 * layer builds its cached int32 copy of a pattern (the reference stores int64 everywhere,
 * numml/sparse/_csr.py:599-600,626-639). */
NB200_API int nb200_narrow_indices(int64_t n, const int64_t* in64, int32_t* out32, nb200_stream stream);
NB200_API int nb200_widen_indices(int64_t n, const int32_t* in32, int64_t* out64, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * SpMM forward  C = A B, B dense row-major [cols, K], C dense row-major [rows, K].
 * Replaces spdmm_forward (reference cpp/sparse_csr.hpp:81-85, CPU cpp/sparse_csr_cpu.cpp:562-602,
 * CUDA cpp/sparse_csr_cuda.cu:547-603).  Each output element is summed over the row's entries in
 * storage order with unfused multiply and add: bit-identical to the reference CPU loop.
 * `perm` (itype, may be NULL) as in nb200_spgemv_forward: with a transposed structure this call
 * computes grad_B = A^T grad_C of spdmm_backward without atomics.  128-bit loads are used when
 * K * sizeof(value) is a multiple of 16 and B, C are 16-byte aligned.
 * `row_order` (rows int32, a permutation of the rows, may be NULL): the order in which rows are handed
 * to lane groups.  Rows sorted by descending length make the few very long rows of a skewed matrix
 * start first instead of trailing; results are unchanged (every row is still summed alone, in order).
 * ------------------------------------------------------------------------------------------- */
NB200_API int nb200_spdmm_forward(int64_t rows, int64_t cols, int64_t K, int64_t nnz,
                                  const void* data, const void* indices, const void* indptr,
                                  const void* perm, const int32_t* row_order, const void* B, void* C,
                                  int dtype, int itype, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * SpMM backward, masked part: grad_A[k] = <grad_C[row(k), :], B[col(k), :]>.
 * Replaces the grad_A half of spdmm_backward (reference cpp/sparse_csr.hpp:87-91, CPU
 * cpp/sparse_csr_cpu.cpp:624-636, CUDA cpp/sparse_csr_cuda.cu:611-645); the grad_B half is
 * nb200_spdmm_forward on the transposed structure.  `row_order` as in nb200_spdmm_forward.
 * ------------------------------------------------------------------------------------------- */
NB200_API int nb200_spdmm_backward_grad_A(int64_t rows, int64_t cols, int64_t K, int64_t nnz,
                                          const void* indices, const void* indptr, const int32_t* row_order,
                                          const void* B, const void* grad_C, void* grad_A,
                                          int dtype, int itype, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * SpGEMM  C = A B, hash-based, in two phases.      Replaces spgemm_forward (reference
 * cpp/sparse_csr.hpp:45-48, CPU cpp/sparse_csr_cpu.cpp:117-216, CUDA
 * cpp/sparse_csr_gemm_cuda.cu:223-302).
 *
 *   1. nb200_spgemm_plan      counts the products of every row of A, bins the rows and writes a
 *                             header of 24 int64 words at the start of `workspace`:
 *                             [0..5] rows per bin, [6] spill slots needed by the symbolic phase,
 *                             [7] largest product count of a row.
 *   2. nb200_spgemm_symbolic  counts the distinct columns of every row of C (rows whose row of A has at
 *                             most 8 entries and 64 products: one thread per row merging the selected
 *                             sorted rows of B; other rows with at most 32 products: one warp per row;
 *                             larger rows: per-bin hash tables in shared memory; rows with more than
 *                             4096 products use `spill`, an array of `spill_slots` uint32), writes
 *                             C_indptr (int64, A_rows+1 entries) and extends the header: [8..13] rows
 *                             per bin for the numeric phase, [14] its spill slots, [15] nnz(C),
 *                             [16] non-zero if a spill area was too small (its rows are then skipped,
 *                             nothing is written out of bounds).
 *   3. nb200_spgemm_numeric   fills C_indices (int64, ascending within a row) and C_data;
 *                             `spill` must hold spill_slots * (sizeof(value) + 4) bytes.
 *
 * The caller reads the header (a device-to-host copy of 192 bytes) after step 2 to size the outputs
 * and the numeric spill area.  Steps 1 and 2 can be enqueued together with spill_slots = 0: only if
 * header[6] then turns out non-zero (a row with more than 4096 products exists) must both be repeated
 * with a spill area of that many slots.  C's pattern is purely structural: numerically cancelled
 * entries are stored as zeros, like the reference's.  C_indptr / C_indices are bit-identical to the
 * reference's.  Values of the rows formed by one thread or one warp are summed in the reference's order
 * with unfused multiply and add: bit-identical to its CPU loop and reproducible; values of larger rows
 * are accumulated with atomics (order not fixed, within tolerance).  `B_rows_sorted` != 0 states that the
 * columns of every row of B ascend strictly (nb200_csr_check), which the thread-per-row merge needs; with 0
 * those rows take the warp or hash kernels instead and the result is the same.
 * `workspace` must hold nb200_spgemm_workspace_bytes(A_rows) bytes and be kept between the calls.
 * ------------------------------------------------------------------------------------------- */
NB200_API size_t nb200_spgemm_workspace_bytes(int64_t A_rows);
NB200_API int nb200_spgemm_plan(int64_t A_rows, int64_t A_cols, int64_t A_nnz,
                                const void* A_indices, const void* A_indptr, const void* B_indptr, int B_rows_sorted,
                                int itype, void* workspace, size_t workspace_bytes, nb200_stream stream);
NB200_API int nb200_spgemm_symbolic(int64_t A_rows, int64_t A_cols, int64_t B_cols,
                                    const void* A_indices, const void* A_indptr,
                                    const void* B_indices, const void* B_indptr, int itype,
                                    void* workspace, size_t workspace_bytes, void* spill, int64_t spill_slots,
                                    int64_t* C_indptr, nb200_stream stream);
NB200_API int nb200_spgemm_numeric(int64_t A_rows, int64_t A_cols, int64_t B_cols,
                                   const void* A_data, const void* A_indices, const void* A_indptr,
                                   const void* B_data, const void* B_indices, const void* B_indptr,
                                   int dtype, int itype, void* workspace, size_t workspace_bytes,
                                   void* spill, int64_t spill_slots,
                                   const int64_t* C_indptr, int64_t* C_indices, void* C_data, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * SpGEMM backward.                                 Replaces spgemm_backward (reference
 * cpp/sparse_csr.hpp:50-54, CPU cpp/sparse_csr_cpu.cpp:218-307, CUDA
 * cpp/sparse_csr_gemm_cuda.cu:311-371,663-771).
 *   grad_A = (grad_C B^T) restricted to the pattern of A,
 *   grad_B = (A^T grad_C) restricted to the pattern of B,
 * with grad_C given on C's pattern (C_indices / C_indptr int64, columns ascending).  At_* is the
 * transposed structure of A (nb200_csr_transpose_structure, index width `itype`).  No atomics;
 * sums are taken in the reference's order with unfused multiply and add (bit-identical).
 * ------------------------------------------------------------------------------------------- */
NB200_API int nb200_spgemm_backward(int64_t A_rows, int64_t A_cols, int64_t A_nnz,
                                    const void* A_data, const void* A_indices, const void* A_indptr,
                                    const void* At_indptr, const void* At_indices, const void* At_perm,
                                    int64_t B_rows, int64_t B_cols, int64_t B_nnz,
                                    const void* B_data, const void* B_indices, const void* B_indptr,
                                    const void* grad_C, const int64_t* C_indices, const int64_t* C_indptr,
                                    void* grad_A, void* grad_B, int dtype, int itype, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Sparse triangular solve.                         Replaces sptrsv_forward (reference
 * cpp/sparse_csr.hpp:94-98, CPU cpp/sparse_csr_cpu.cpp:652-723, CUDA cpp/sparse_csr_cuda.cu:714-831)
 * and, with the two helpers below, sptrsv_backward (cpp/sparse_csr.hpp:100-105, CPU :725-759,
 * CUDA :833-860).
 *
 * nb200_sptrsv_analyse   once per pattern and triangle: computes the dependency level of every row (one
 *                        more than the largest level among the rows it depends on) in one launch, the
 *                        level array serving as its own ready flag under bounded polls, and writes
 *                        `order` (n int32: rows sorted by level, then by row).  Columns must be sorted
 *                        within each row.  `t_indptr` / `t_indices` are not used (earlier versions peeled
 *                        levels through the transposed structure) and may be NULL.  The number of levels
 *                        is written to the HOST word *nlevels_host.  This call synchronises `stream` once.
 *                        NB200_ERR_WAIT_BUDGET if a poll ran out (about two seconds without progress).
 * nb200_sptrsv_solve     x = A^{-1} b for `nrhs` right-hand sides stored row-major [n, nrhs] (nrhs = 1
 *                        is the reference's single-vector call).  Substitution is done in double and
 *                        rounded to the value type at the end, entries are accumulated in the
 *                        reference's order with unfused multiply and add: the result is bit-identical
 *                        to the reference CPU loop.  `perm` (may be NULL) reads entry k's value as
 *                        data[perm[k]], which is how the transposed system of the backward pass is
 *                        solved from the cached transposed structure.  `x_double` (n*nrhs doubles) is
 *                        required when dtype is NB200_F32 (for NB200_F64 the solve works in `x`).
 *                        The working array is pre-filled with an all-ones bit pattern that marks
 *                        "not solved yet"; a result that would equal it is stored as the canonical NaN.
 *                        Lanes wait for the unknowns they depend on with a bounded poll: when
 *                        `wait_budget_cycles` SM cycles (<= 0: 2e9, about a second) pass without
 *                        progress the kernel stores NB200_ERR_WAIT_BUDGET in the device word `status`
 *                        (which the caller zeroes beforehand and reads afterwards), writes NaN into the
 *                        affected rows and returns; it never spins without a limit.
 *                        `team_lanes` (0, or a power of two up to 32) is the least number of lanes
 *                        given to one row; 0 means the smallest power of two that covers `nrhs`.
 *                        A warp's poll takes as long as its slowest row, so when the levels are
 *                        narrow (n / levels well below the number of resident warps) a full warp per
 *                        row is fastest even though the spare lanes idle; with wide levels fewer
 *                        lanes per row keep the GPU full.  The result does not depend on it.
 * nb200_masked_outer     out[k] = sum_r alpha * (a[row(k), r] * b[col(k), r]): the masked outer
 *                        product grad_A = -(grad_b x^T) on the pattern of A (alpha = -1), summed over
 *                        the right-hand sides in ascending order.
 * ------------------------------------------------------------------------------------------- */
NB200_API size_t nb200_sptrsv_analysis_workspace_bytes(int64_t n);
NB200_API int nb200_sptrsv_analyse(int64_t n, int64_t nnz, const void* indices, const void* indptr,
                                   const void* t_indptr, const void* t_indices, int itype, int lower,
                                   int32_t* order, int64_t* nlevels_host,
                                   void* workspace, size_t workspace_bytes, nb200_stream stream);
NB200_API int nb200_sptrsv_solve(int64_t n, int64_t nnz, int64_t nrhs,
                                 const void* data, const void* indices, const void* indptr, const void* perm,
                                 const int32_t* order, int lower, int unit, const void* b, void* x,
                                 double* x_double, int32_t* status, int64_t wait_budget_cycles,
                                 int team_lanes, int dtype, int itype, nb200_stream stream);
NB200_API int nb200_masked_outer(int64_t rows, int64_t nnz, int64_t nrhs, const void* indices, const void* indptr,
                                 const void* a, const void* b, double alpha, void* out,
                                 int dtype, int itype, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Triangular solve for narrow dependency levels, inside one thread-block cluster.  Same operator and
 * same results (bit for bit) as nb200_sptrsv_solve; no counterpart of its own in the reference, whose
 * CUDA solve is one kernel (cpp/sparse_csr_cuda.cu:714-831).
 *
 * For factors with thousands of levels of a few hundred rows (banded and stencil factors in natural
 * ordering) the grid-wide solve pays one round trip through L2 per level.  Here one cluster of
 * `cluster_ctas` CTAs (1, 2, 4, 8 or 16; 0 = 8) takes the levels one after the other, a team of lanes
 * per row and a lane per right-hand side, keeps the unknowns of the most recent rows in a ring spread
 * over the shared memory of its CTAs, reads dependencies from there through distributed shared memory,
 * and separates levels by the hardware cluster barrier.  No thread waits on a flag.
 *
 * nb200_sptrsv_analyse_levels   nb200_sptrsv_analyse that also writes `level_ptr` (capacity n + 1 int32;
 *                               nlevels + 1 are written): the first position in `order` of every level.
 * nb200_sptrsv_level_plan       once per pattern, triangle and (for the transposed system) permutation:
 *                               the structure in position order (position p = row order[p]):
 *                               `pos_ptr` (n + 1 int32), and per kept entry -- those on the solve side of
 *                               the diagonal, the diagonal included, in the order in which the solve adds
 *                               them -- `dep` (position of the row it refers to, -1 for the diagonal) and
 *                               `src` (where its value is found in `data`, `perm` applied).  HOST words
 *                               info_host[0..3]: kept entries, reach (largest distance from the end of a
 *                               row's level back to the position of one of its dependencies), longest row,
 *                               widest level.  Synchronises `stream` once.
 * nb200_sptrsv_solve_levels     the solve: a gather pass (values and right-hand sides into position order,
 *                               as double), the cluster kernel, a scatter pass (x back into row order,
 *                               rounded to the value type).  `workspace`:
 *                               nb200_sptrsv_solve_levels_workspace_bytes(n, nrhs, entries).
 *                               NB200_ERR_TOO_LARGE (nothing launched) when a ring of `reach` rows of
 *                               nrhs doubles does not fit into the cluster's shared memory (200 KiB per
 *                               CTA): the caller then uses nb200_sptrsv_solve.
 * ------------------------------------------------------------------------------------------- */
NB200_API int nb200_sptrsv_analyse_levels(int64_t n, int64_t nnz, const void* indices, const void* indptr,
                                          int itype, int lower, int32_t* order, int32_t* level_ptr,
                                          int64_t* nlevels_host, void* workspace, size_t workspace_bytes,
                                          nb200_stream stream);
NB200_API size_t nb200_sptrsv_level_plan_workspace_bytes(int64_t n);
NB200_API int nb200_sptrsv_level_plan(int64_t n, int64_t nnz, const void* indices, const void* indptr, const void* perm,
                                      int itype, int lower, const int32_t* order, const int32_t* level_ptr,
                                      int64_t nlevels, int32_t* pos_ptr, int32_t* dep, int32_t* src, int64_t* info_host,
                                      void* workspace, size_t workspace_bytes, nb200_stream stream);
NB200_API size_t nb200_sptrsv_solve_levels_workspace_bytes(int64_t n, int64_t nrhs, int64_t entries);
NB200_API int nb200_sptrsv_solve_levels(int64_t n, int64_t nrhs, int64_t entries, const void* data, const int32_t* src,
                                        const int32_t* pos_ptr, const int32_t* dep, const int32_t* order,
                                        const int32_t* level_ptr, int64_t nlevels, int64_t reach, int unit,
                                        const void* b, void* x, void* workspace, size_t workspace_bytes,
                                        int cluster_ctas, int dtype, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Allocation-free float32 triangular solve.  No counterpart in the reference.
 *
 * Same computation and same results as nb200_sptrsv_solve with dtype NB200_F32, for callers that
 * have no device memory to lend: a plugin embedded in a runtime that owns the device-memory pool
 * and forbids allocation behind its back, or a latency-bound loop that must never reach cudaMalloc
 * (which synchronises the device and can fail on a fragmented heap).  The n*nrhs doubles of working
 * memory that the substitution needs live in a fixed 8 MiB array inside the library image (held by
 * every GPU that loads the library, until the process exits) instead of a caller-provided `x_double`.
 * The caller still passes every input and output, including the `status` word.
 *
 *   - n * nrhs may not exceed nb200_sptrsv_solve_f32_noalloc_capacity() (1,048,576); a larger
 *     problem returns NB200_ERR_TOO_LARGE and launches nothing.
 *   - The first call on a device looks up the device address of the array (with that device
 *     current) and caches it; make that first call before any stream capture begins.
 *   - All calls on a device share the one array.  It keeps the previous call's contents and is
 *     re-marked "unsolved" at the start of every call, so sequential calls are independent; two
 *     calls whose kernels overlap on the GPU (different streams, or different host threads) race on
 *     it and give undefined results.
 *   - The function calls no cudaMalloc / cudaFree and no allocating library routine.
 * ------------------------------------------------------------------------------------------- */
NB200_API int64_t nb200_sptrsv_solve_f32_noalloc_capacity(void);
NB200_API int nb200_sptrsv_solve_f32_noalloc(int64_t n, int64_t nnz, int64_t nrhs,
                                             const float* data, const void* indices, const void* indptr,
                                             const void* perm, const int32_t* order, int lower, int unit,
                                             const float* b, float* x, int32_t* status,
                                             int64_t wait_budget_cycles, int itype, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Conjugate gradients with a fixed iteration count.  Replaces the loop of conjugate_gradient
 * (reference numml/krylov.py:83-155) for the case the benchmark configuration uses: no
 * preconditioner, rtol = 0 and a given number of iterations, i.e. a stopping rule that can never
 * fire.  The whole solve is enqueued on `stream` without a host round trip: per iteration one SpMV
 * (nb200_spgemv_forward with `block_rows` as described there) and three fused vector kernels; the
 * scalars alpha and beta stay in device memory.  On return (asynchronously) `x` holds the iterate
 * and residual_history[0..iterations] the residual norms before the first and after every iteration.
 * `has_x0` != 0: `x` holds the initial guess on entry; otherwise it is set to zero.
 * `workspace` must hold nb200_cg_workspace_bytes(n, dtype) bytes.
 * ------------------------------------------------------------------------------------------- */
NB200_API size_t nb200_cg_workspace_bytes(int64_t n, int dtype);
NB200_API int nb200_cg_fixed_iterations(int64_t n, int64_t nnz, const void* data, const void* indices, const void* indptr,
                                        int block_rows, const void* b, void* x, int has_x0, void* residual_history,
                                        int64_t iterations, void* workspace, size_t workspace_bytes, int32_t* status,
                                        int dtype, int itype, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Row-partitioned CG, the part of an iteration that is not the SpMV.  No counterpart in the reference
 * (numml/krylov.py:83-155 is a single-device loop); the recurrence is the same.  Every rank holds a block
 * of b, x, r, p and calls the phases in this order, the SpMV Ap = A p (halo exchange + local kernels)
 * being the caller's between 4 and 2:
 *     0  r = b, p = r, x = 0; local <r,r> published        1  total <r,r> -> history[0]
 *     2  local <Ap,p> published                             3  alpha from the total; x += alpha p; r -= alpha Ap;
 *     4  beta from the total <r,r>; p = r + beta p;            local <r,r> published
 *        history[it+1]; the iteration counter moves on
 * A dot product is reduced across ranks through peer memory, inside these kernels: the last block of the
 * kernel that forms the local sum stores it into this rank's scalar area and sets this rank's flag to the
 * reduction's sequence number (release, system scope); the next kernel starts by waiting (bounded by
 * `wait_budget_cycles`, NB200_ERR_WAIT_BUDGET in `status` and NaN totals on expiry) for every rank's flag
 * and adds the ranks' sums in rank order, so all ranks get the same bits.  `table` (device, 2 int64 per
 * rank) holds the address of each rank's scalar area (2 halves of 4 doubles, alternating by sequence
 * number) and of its flag word, as mapped into this process; `sequence_word` is a device word of this
 * rank that lives as long as the exchange buffers (zero when they are created).  world <= 32.
 * `workspace`: nb200_cg_peer_workspace_bytes() bytes, kept for the whole solve.
 * ------------------------------------------------------------------------------------------- */
NB200_API size_t nb200_cg_peer_workspace_bytes(void);
NB200_API int nb200_cg_peer_phase(int phase, int64_t n, const void* b, void* x, void* r, void* p, const void* Ap,
                                  void* residual_history, void* workspace, size_t workspace_bytes,
                                  int world, int rank, const int64_t* table, int32_t* sequence_word,
                                  int32_t* status, int64_t wait_budget_cycles, int dtype, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Pattern-building operators (all index arrays int64, as the matrices store them).  Each produces a new
 * pattern in two steps: a count call that writes the new row pointers (the caller reads the last one, a
 * device-to-host copy of 8 bytes, to size the outputs) and a fill call.  `workspace` must hold
 * nb200_pattern_workspace_bytes(rows) bytes.
 *
 * nb200_csr_triangle_*   entries (r, c) with c <= r + k (lower != 0) or c >= r + k (lower == 0), in storage
 *                        order: tril / triu of the reference (numml/sparse/_csr.py:234-330, Python loops
 *                        there; its tril stops at the first entry beyond the bound, which is the same thing
 *                        for rows with ascending columns).  `out_pos[q]` is the position in A of output
 *                        entry q, with which the backward pass scatters gradients.
 * nb200_csr_lincomb_*    C = alpha A + beta B on the union of the two patterns by a two-pointer merge of
 *                        every row (columns ascending in both): replaces splincomb_forward / _backward
 *                        (cpp/sparse_csr.hpp:66-78, CPU cpp/sparse_csr_cpu.cpp:387-560, CUDA
 *                        cpp/sparse_csr_cuda.cu:303-540).  Values are formed as the reference forms them
 *                        (alpha a, beta b, or alpha a + beta b with unfused multiply and add): bit-identical.
 *                        Backward: grad_A[e] = grad_C[position of e's column in C] * alpha, same for B.
 * nb200_coo_to_csr       stable sort of n COO entries by (row, column) -- or by row only when
 *                        sort_columns == 0 -- as `perm` (perm[q] = index of the entry that comes q-th)
 *                        and the row pointers: coo_to_csr of the reference (numml/sparse/_csr.py:78-99).
 *                        Needs n, nrows, ncols < 2^31 and nb200_coo_workspace_bytes(n) bytes.
 * ------------------------------------------------------------------------------------------- */
NB200_API size_t nb200_pattern_workspace_bytes(int64_t rows);
NB200_API int nb200_csr_triangle_count(int64_t rows, const int64_t* indices, const int64_t* indptr, int64_t k, int lower,
                                       int64_t* out_indptr, void* workspace, size_t workspace_bytes, nb200_stream stream);
NB200_API int nb200_csr_triangle_fill(int64_t rows, const void* data, const int64_t* indices, const int64_t* indptr,
                                      int64_t k, int lower, const int64_t* out_indptr, void* out_data,
                                      int64_t* out_indices, int64_t* out_pos, int dtype, nb200_stream stream);
NB200_API int nb200_csr_lincomb_count(int64_t rows, const int64_t* A_indices, const int64_t* A_indptr,
                                      const int64_t* B_indices, const int64_t* B_indptr, int64_t* C_indptr,
                                      void* workspace, size_t workspace_bytes, nb200_stream stream);
NB200_API int nb200_csr_lincomb_fill(int64_t rows, double alpha, const void* A_data, const int64_t* A_indices,
                                     const int64_t* A_indptr, double beta, const void* B_data, const int64_t* B_indices,
                                     const int64_t* B_indptr, const int64_t* C_indptr, void* C_data, int64_t* C_indices,
                                     int dtype, nb200_stream stream);
NB200_API int nb200_csr_lincomb_backward(int64_t rows, double alpha, const int64_t* A_indices, const int64_t* A_indptr,
                                         double beta, const int64_t* B_indices, const int64_t* B_indptr,
                                         const void* grad_C, const int64_t* C_indices, const int64_t* C_indptr,
                                         void* grad_A, void* grad_B, int dtype, nb200_stream stream);
NB200_API size_t nb200_coo_workspace_bytes(int64_t n);
NB200_API int nb200_coo_to_csr(int64_t n, const int64_t* row_ind, const int64_t* col_ind, int64_t nrows, int64_t ncols,
                               int sort_columns, int64_t* perm, int64_t* indptr, void* workspace, size_t workspace_bytes,
                               nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Sparse LU without pivoting, M = L + U with unit lower L (its ones not stored).  Replaces splu (reference
 * cpp/sparse_csr.hpp:107-111, CPU cpp/sparse_csr_cpu.cpp:778-1017, CUDA cpp/sparse_csr_cuda.cu:870-1268);
 * with the triangular solve and nb200_masked_outer it also gives spsolve and spsolve_backward
 * (cpp/sparse_csr.hpp:113-118, CPU :1019-1052).  Index arrays int64; every row of A must store its diagonal.
 *
 * nb200_splu_symbolic_count  pattern of M by the fill2 traversal (one warp per row): row pointers into
 *                            M_indptr (n+1 int64; the caller reads the last one to size M).
 * nb200_splu_symbolic_fill   M_indices (ascending per row) and M_data = the value of A, or 0 for fill.
 * nb200_splu_numeric         in place on the TRANSPOSE of M (Mt_*: columns of M stored as rows, e.g. from
 *                            nb200_csr_transpose_structure + nb200_gather): left-looking elimination, one
 *                            warp per column, a flag per column (`done`, n int32) with bounded polls;
 *                            NB200_ERR_WAIT_BUDGET in `status` if a wait runs out.  Every update is an
 *                            unfused multiply and subtract applied in the reference's order: bit-identical.
 * `workspace`: nb200_splu_workspace_bytes(n) bytes for the two symbolic calls (three stamp arrays of n
 * words per row in flight, at most about 2 GiB).  n < 2^30.
 * ------------------------------------------------------------------------------------------- */
NB200_API size_t nb200_splu_workspace_bytes(int64_t n);
NB200_API int nb200_splu_symbolic_count(int64_t n, const int64_t* A_indices, const int64_t* A_indptr, int64_t* M_indptr,
                                        void* workspace, size_t workspace_bytes, nb200_stream stream);
NB200_API int nb200_splu_symbolic_fill(int64_t n, const void* A_data, const int64_t* A_indices, const int64_t* A_indptr,
                                       const int64_t* M_indptr, int64_t* M_indices, void* M_data,
                                       void* workspace, size_t workspace_bytes, int dtype, nb200_stream stream);
NB200_API int nb200_splu_numeric(int64_t n, void* Mt_data, const int64_t* Mt_indices, const int64_t* Mt_indptr,
                                 int32_t* done, int32_t* status, int64_t wait_budget_cycles, int dtype, nb200_stream stream);

/* ---------------------------------------------------------------------------------------------
 * Halo exchange of a row-partitioned SpMV over peer memory.  No counterpart in the reference, which has
 * no multi-device path (its operators take whole matrices on one device, cpp/sparse_csr.hpp:32-105).
 *
 * Every rank (one process per GPU) owns an exchange buffer that its neighbours map with CUDA IPC; a rank
 * writes only its own buffer and reads only its neighbours', with ordinary stores and loads over NVLink.
 * An exchange buffer holds flag words and packed areas; a packed area has two halves of `count`
 * elements, used alternately by even and odd steps.
 *
 * nb200_halo_publish   area[step & 1][k] = src[idx ? idx[k] : k] for k < count, then the flag word is set
 *                      to the step number (release, system scope).  `step_word` is a device word of the
 *                      caller holding the number of the current step; with `bump_step` != 0 the call
 *                      first advances it by one (the first publish of a step does that).  `arrivals` is a
 *                      zeroed device word used to find the last block.
 * nb200_halo_publish_rowsums   nb200_halo_publish whose values are computed on the way: element r is the row sum
 *                      sum_k data[perm[k]] * x[indices[k]] over row r of (indptr, indices) (`perm` may be NULL),
 *                      entries in storage order, unfused: the partial sums of grad_x owed to the neighbours, one row
 *                      per halo column.  `indptr` points at the first of the `rows` rows (absolute entry positions).
 * nb200_halo_pull      for each of `npeers` neighbours, described by 8 int64 words each
 *                      ([0] address of its packed area, [1] elements per half, [2] first element of this
 *                      rank's segment, [3] elements in it, [4] first destination element in `dst`,
 *                      [5] address of its flag word): wait until the flag has reached the current step,
 *                      then dst[[4] + k] = area[step & 1][[2] + k].  `largest_segment` sizes the grid.
 * nb200_halo_pull_add  for gradients: target j (an index into `grad`) receives the elements
 *                      source_elem[c] of the packed areas of neighbours source_peer[c] (an index into the
 *                      descriptors), c in [target_ptr[j], target_ptr[j+1]), added to grad[target[j]] in
 *                      that order; the caller sorts them by neighbour, which makes the sum reproducible.
 *
 * Waits are bounded: after `wait_budget_cycles` SM cycles (<= 0: 4e9, about two seconds) without the
 * flag arriving, NB200_ERR_WAIT_BUDGET is stored into the device word `status` and the kernel returns
 * without copying.  The two halves make the scheme safe without acknowledgements provided every rank
 * that reads a neighbour is read by that neighbour too (true for patterns that equal their transpose):
 * a rank reaches the publish of step t only after its pull of step t-1 has seen every neighbour's flag
 * at t-1, and a neighbour raises that flag only after its own pull of step t-2 has finished.
 *
 * Rows of a dense operand (row-partitioned SpMM) travel the same way, an item being a row of `row_bytes`
 * bytes (a multiple of 16; `dst` / `grad` 16-byte aligned).  A rank publishes its whole block of rows once
 * with nb200_halo_publish (idx = NULL); every neighbour gathers the rows it needs from there:
 * nb200_halo_pull_rows       descriptor words: [0] address of the neighbour's area, [1] rows per half,
 *                            [2] first halo slot of this neighbour in `row_of_slot`, [3] number of slots,
 *                            [4] first destination row in `dst`, [5] address of its flag word; slot h of the
 *                            segment receives row row_of_slot[[2] + h] of the neighbour's block.
 * nb200_halo_pull_add_rows   nb200_halo_pull_add on rows: grad row target[j] += rows source_elem[c] of the
 *                            packed areas of neighbours source_peer[c], in that order (unfused adds).
 *
 * nb200_ipc_alloc / nb200_ipc_open / nb200_ipc_close / nb200_ipc_free create an exchange buffer (zeroed,
 * from cudaMalloc, since memory that other processes map cannot come out of a caching allocator's
 * segment; this is the only allocation the library ever makes, at set-up time), export it as 64 opaque
 * bytes, map a neighbour's buffer into this process with the calling thread's current device as the
 * device that will access it, and undo both.  These four calls synchronise.
 * ------------------------------------------------------------------------------------------- */
NB200_API int nb200_halo_publish(int64_t count, const void* src, const int64_t* idx, void* area, int32_t* flag,
                                 int32_t* step_word, int bump_step, uint32_t* arrivals, int dtype, nb200_stream stream);
NB200_API int nb200_halo_publish_rowsums(int64_t rows, const void* data, const void* indices, const void* indptr,
                                         const void* perm, const void* x, void* area, int32_t* flag, int32_t* step_word,
                                         int bump_step, uint32_t* arrivals, int dtype, int itype, nb200_stream stream);
NB200_API int nb200_halo_pull(int npeers, const int64_t* desc, int64_t largest_segment, void* dst,
                              const int32_t* step_word, int32_t* status, int64_t wait_budget_cycles,
                              int dtype, nb200_stream stream);
NB200_API int nb200_halo_pull_add(int npeers, const int64_t* desc, int64_t ntargets, const int64_t* target,
                                  const int64_t* target_ptr, const int32_t* source_peer, const int64_t* source_elem,
                                  void* grad, const int32_t* step_word, int32_t* status, int64_t wait_budget_cycles,
                                  int dtype, nb200_stream stream);
NB200_API int nb200_halo_pull_rows(int npeers, const int64_t* desc, const int64_t* row_of_slot, int64_t largest_segment,
                                   int64_t row_bytes, void* dst, const int32_t* step_word, int32_t* status,
                                   int64_t wait_budget_cycles, nb200_stream stream);
NB200_API int nb200_halo_pull_add_rows(int npeers, const int64_t* desc, int64_t ntargets, const int64_t* target,
                                       const int64_t* target_ptr, const int32_t* source_peer, const int64_t* source_elem,
                                       int64_t row_bytes, void* grad, const int32_t* step_word, int32_t* status,
                                       int64_t wait_budget_cycles, int dtype, nb200_stream stream);
NB200_API int nb200_ipc_alloc(size_t bytes, void** ptr, void* handle64);
NB200_API int nb200_ipc_open(const void* handle64, void** ptr);
NB200_API int nb200_ipc_close(void* ptr);
NB200_API int nb200_ipc_free(void* ptr);

#ifdef __cplusplus
}
#endif
#endif /* NUMML_B200_H_ */
