// CSR transpose structure on the device: a stable radix sort of (column, position) pairs.
// Entries of one column keep their order of appearance in A (ascending row), so every row of
// A^T comes out with ascending column indices, and the sorted positions are exactly the
// permutation the reference calls At_to_A_idx.  No atomics, no per-column rescans.
#include "primitives.cuh"

namespace nb200 {

template <typename I>
__global__ void transpose_init_pairs_kernel(int64_t nnz, const I* __restrict__ indices,
                                            uint32_t* __restrict__ keys, uint32_t* __restrict__ vals) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < nnz; k += stride) {
        keys[k] = (uint32_t)indices[k];
        vals[k] = (uint32_t)k;
    }
}

// t_indptr[c] = number of entries with column < c = lower bound of c in the sorted keys.
template <typename O>
__global__ void transpose_indptr_kernel(int64_t cols, int64_t nnz, const uint32_t* __restrict__ sorted_keys,
                                        O* __restrict__ t_indptr) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c <= cols; c += stride) {
        int64_t lo = 0, hi = nnz;
        while (lo < hi) {
            const int64_t mid = (lo + hi) >> 1;
            if ((int64_t)sorted_keys[mid] < c) lo = mid + 1; else hi = mid;
        }
        t_indptr[c] = (O)lo;
    }
}

// t_perm[k'] = position in A; t_indices[k'] = row of that position (last r with indptr[r] <= k).
template <typename I, typename O>
__global__ void transpose_emit_kernel(int64_t rows, int64_t nnz, const I* __restrict__ indptr,
                                      const uint32_t* __restrict__ sorted_vals,
                                      O* __restrict__ t_indices, O* __restrict__ t_perm) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < nnz; q += stride) {
        const int64_t k = (int64_t)sorted_vals[q];
        int64_t lo = 0, hi = rows;  // find the largest r in [0, rows) with indptr[r] <= k
        while (hi - lo > 1) {
            const int64_t mid = (lo + hi) >> 1;
            if ((int64_t)indptr[mid] <= k) lo = mid; else hi = mid;
        }
        t_perm[q] = (O)k;
        t_indices[q] = (O)lo;
    }
}

static inline unsigned grid_for(int64_t n) {
    const int64_t want = ceil_div(n > 0 ? n : 1, (int64_t)256);
    return (unsigned)(want > (int64_t)kSMs * 32 ? (int64_t)kSMs * 32 : want);
}

static inline int bit_length(int64_t v) {
    int b = 0;
    while (v > 0) { ++b; v >>= 1; }
    return b;
}

template <typename I, typename O>
int transpose_structure(int64_t rows, int64_t cols, int64_t nnz, const I* indices, const I* indptr,
                        O* t_indptr, O* t_indices, O* t_perm, void* workspace, size_t workspace_bytes,
                        cudaStream_t st) {
    Workspace ws(workspace, workspace_bytes);
    const size_t m = (size_t)(nnz > 0 ? nnz : 1);
    uint32_t* keys_a = ws.take<uint32_t>(m);
    uint32_t* vals_a = ws.take<uint32_t>(m);
    uint32_t* keys_b = ws.take<uint32_t>(m);
    uint32_t* vals_b = ws.take<uint32_t>(m);
    const size_t ssb = sort_scratch_bytes(nnz);
    char* sscratch = ws.take<char>(ssb);
    if (!ws.ok()) return NB200_ERR_WORKSPACE;

    bool in_a = true;
    if (nnz > 0) {
        transpose_init_pairs_kernel<I><<<grid_for(nnz), 256, 0, st>>>(nnz, indices, keys_a, vals_a);
        int rc = sort_pairs_u32(nnz, bit_length(cols - 1), keys_a, vals_a, keys_b, vals_b, &in_a, sscratch, ssb, st);
        if (rc != NB200_OK) return rc;
    }
    const uint32_t* sk = in_a ? keys_a : keys_b;
    const uint32_t* sv = in_a ? vals_a : vals_b;
    transpose_indptr_kernel<O><<<grid_for(cols + 1), 256, 0, st>>>(cols, nnz, sk, t_indptr);
    if (nnz > 0)
        transpose_emit_kernel<I, O><<<grid_for(nnz), 256, 0, st>>>(rows, nnz, indptr, sv, t_indices, t_perm);
    return launch_status();
}

}  // namespace nb200

using namespace nb200;

extern "C" size_t nb200_csr_transpose_workspace_bytes(int64_t rows, int64_t cols, int64_t nnz) {
    (void)rows; (void)cols;
    const size_t m = (size_t)(nnz > 0 ? nnz : 1);
    return 4 * Workspace::pad(m * sizeof(uint32_t)) + Workspace::pad(sort_scratch_bytes(nnz));
}

extern "C" int nb200_csr_transpose_structure(int64_t rows, int64_t cols, int64_t nnz,
                                             const void* indices, const void* indptr, int itype_in,
                                             void* t_indptr, void* t_indices, void* t_perm, int itype_out,
                                             void* workspace, size_t workspace_bytes, nb200_stream stream) {
    if (rows < 0 || cols < 0 || nnz < 0) return NB200_ERR_BAD_ARG;
    if (!t_indptr || (rows > 0 && !indptr) || (nnz > 0 && (!indices || !t_indices || !t_perm))) return NB200_ERR_BAD_ARG;
    if (nnz >= 0x7fffffffLL || rows >= 0x7fffffffLL || cols >= 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    cudaStream_t st = as_stream(stream);
    if (itype_in == NB200_I32 && itype_out == NB200_I32)
        return transpose_structure<int32_t, int32_t>(rows, cols, nnz, (const int32_t*)indices, (const int32_t*)indptr,
                                                     (int32_t*)t_indptr, (int32_t*)t_indices, (int32_t*)t_perm, workspace, workspace_bytes, st);
    if (itype_in == NB200_I32 && itype_out == NB200_I64)
        return transpose_structure<int32_t, int64_t>(rows, cols, nnz, (const int32_t*)indices, (const int32_t*)indptr,
                                                     (int64_t*)t_indptr, (int64_t*)t_indices, (int64_t*)t_perm, workspace, workspace_bytes, st);
    if (itype_in == NB200_I64 && itype_out == NB200_I32)
        return transpose_structure<int64_t, int32_t>(rows, cols, nnz, (const int64_t*)indices, (const int64_t*)indptr,
                                                     (int32_t*)t_indptr, (int32_t*)t_indices, (int32_t*)t_perm, workspace, workspace_bytes, st);
    if (itype_in == NB200_I64 && itype_out == NB200_I64)
        return transpose_structure<int64_t, int64_t>(rows, cols, nnz, (const int64_t*)indices, (const int64_t*)indptr,
                                                     (int64_t*)t_indptr, (int64_t*)t_indices, (int64_t*)t_perm, workspace, workspace_bytes, st);
    return NB200_ERR_BAD_ARG;
}
