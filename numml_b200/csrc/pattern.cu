// Pattern-building operators on the device: triangular parts, linear combinations on the union
// pattern, and COO -> CSR conversion.  They produce new sparsity patterns, so each is a count pass,
// an exclusive scan (the new row pointers) and a fill pass; index arrays are int64 as the matrices
// store them.  Rows are walked one thread per row, in storage order, so the output keeps the input's
// order within a row and sums are formed exactly as the reference's merge loops form them.
#include "primitives.cuh"

namespace nb200 {

constexpr int kPatThreads = 256;

static inline unsigned pat_grid(int64_t n) {
    const int64_t want = ceil_div(n > 0 ? n : 1, (int64_t)kPatThreads);
    return (unsigned)(want > (int64_t)kSMs * 32 ? (int64_t)kSMs * 32 : want);
}

// ---- triangular part: keep (r, c) with c <= r + k (lower) or c >= r + k (upper) -----------------
__device__ __forceinline__ bool in_triangle(int64_t r, int64_t c, int64_t k, bool lower) {
    return lower ? (c <= r + k) : (c >= r + k);
}

__global__ void triangle_count_kernel(int64_t rows, const int64_t* __restrict__ indices, const int64_t* __restrict__ indptr,
                                      int64_t k, bool lower, int32_t* __restrict__ counts) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += stride) {
        int32_t n = 0;
        for (int64_t e = indptr[r]; e < indptr[r + 1]; ++e) n += in_triangle(r, indices[e], k, lower);
        counts[r] = n;
    }
}

template <typename T>
__global__ void triangle_fill_kernel(int64_t rows, const T* __restrict__ data, const int64_t* __restrict__ indices,
                                     const int64_t* __restrict__ indptr, int64_t k, bool lower,
                                     const int64_t* __restrict__ out_indptr, T* __restrict__ out_data,
                                     int64_t* __restrict__ out_indices, int64_t* __restrict__ out_pos) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += stride) {
        int64_t o = out_indptr[r];
        for (int64_t e = indptr[r]; e < indptr[r + 1]; ++e) {
            const int64_t c = indices[e];
            if (in_triangle(r, c, k, lower)) {
                out_data[o] = data[e];
                out_indices[o] = c;
                out_pos[o] = e;
                ++o;
            }
        }
    }
}

// ---- linear combination on the union pattern (two-pointer merge of sorted rows) ------------------
__global__ void lincomb_count_kernel(int64_t rows, const int64_t* __restrict__ A_indices, const int64_t* __restrict__ A_indptr,
                                     const int64_t* __restrict__ B_indices, const int64_t* __restrict__ B_indptr,
                                     int32_t* __restrict__ counts) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += stride) {
        int64_t a = A_indptr[r], b = B_indptr[r];
        const int64_t ae = A_indptr[r + 1], be = B_indptr[r + 1];
        int32_t n = 0;
        while (a < ae && b < be) {
            const int64_t ca = A_indices[a], cb = B_indices[b];
            a += ca <= cb;
            b += cb <= ca;
            ++n;
        }
        counts[r] = n + (int32_t)(ae - a) + (int32_t)(be - b);
    }
}

template <typename T>
__global__ void lincomb_fill_kernel(int64_t rows, T alpha, const T* __restrict__ A_data, const int64_t* __restrict__ A_indices,
                                    const int64_t* __restrict__ A_indptr, T beta, const T* __restrict__ B_data,
                                    const int64_t* __restrict__ B_indices, const int64_t* __restrict__ B_indptr,
                                    const int64_t* __restrict__ C_indptr, T* __restrict__ C_data, int64_t* __restrict__ C_indices) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += stride) {
        int64_t a = A_indptr[r], b = B_indptr[r], o = C_indptr[r];
        const int64_t ae = A_indptr[r + 1], be = B_indptr[r + 1];
        while (a < ae && b < be) {
            const int64_t ca = A_indices[a], cb = B_indices[b];
            if (ca < cb) { C_data[o] = mul_rn(alpha, A_data[a]); C_indices[o] = ca; ++a; }
            else if (ca > cb) { C_data[o] = mul_rn(beta, B_data[b]); C_indices[o] = cb; ++b; }
            else { C_data[o] = add_rn(mul_rn(alpha, A_data[a]), mul_rn(beta, B_data[b])); C_indices[o] = ca; ++a; ++b; }
            ++o;
        }
        for (; a < ae; ++a, ++o) { C_data[o] = mul_rn(alpha, A_data[a]); C_indices[o] = A_indices[a]; }
        for (; b < be; ++b, ++o) { C_data[o] = mul_rn(beta, B_data[b]); C_indices[o] = B_indices[b]; }
    }
}

// grad_M[e] = scale * grad_C[position of entry e's column in row r of C], for M = A or B
template <typename T>
__global__ void lincomb_backward_kernel(int64_t rows, T scale, const int64_t* __restrict__ M_indices,
                                        const int64_t* __restrict__ M_indptr, const T* __restrict__ grad_C,
                                        const int64_t* __restrict__ C_indices, const int64_t* __restrict__ C_indptr,
                                        T* __restrict__ grad_M) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += stride) {
        int64_t m = M_indptr[r], c = C_indptr[r];
        const int64_t me = M_indptr[r + 1], ce = C_indptr[r + 1];
        while (m < me && c < ce) {
            const int64_t cm = M_indices[m], cc = C_indices[c];
            if (cm < cc) ++m;
            else if (cm > cc) ++c;
            else { grad_M[m] = mul_rn(grad_C[c], scale); ++m; ++c; }
        }
    }
}

// ---- COO -> CSR: stable sort of the entries by (row, column) -------------------------------------
__global__ void coo_init_kernel(int64_t n, const int64_t* __restrict__ key_src, const uint32_t* __restrict__ order,
                                uint32_t* __restrict__ keys, uint32_t* __restrict__ vals) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += stride) {
        const uint32_t e = order ? order[k] : (uint32_t)k;
        keys[k] = (uint32_t)key_src[e];
        vals[k] = e;
    }
}

__global__ void coo_emit_kernel(int64_t n, int64_t nrows, const uint32_t* __restrict__ sorted_rows,
                                const uint32_t* __restrict__ sorted_vals, int64_t* __restrict__ perm,
                                int64_t* __restrict__ indptr) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (int64_t k = gtid; k < n; k += stride) perm[k] = (int64_t)sorted_vals[k];
    for (int64_t r = gtid; r <= nrows; r += stride) {        // indptr[r] = entries with row < r
        int64_t lo = 0, hi = n;
        while (lo < hi) {
            const int64_t mid = (lo + hi) >> 1;
            if ((int64_t)sorted_rows[mid] < r) lo = mid + 1; else hi = mid;
        }
        indptr[r] = lo;
    }
}

static inline int bits_for(int64_t v) {
    int b = 1;
    while ((v >> b) > 0) ++b;
    return b;
}

struct CountScratch { int32_t* counts; char* scan; size_t scan_bytes; bool ok; };

static size_t count_scratch_bytes(int64_t rows) {
    return Workspace::pad((size_t)(rows > 0 ? rows : 1) * sizeof(int32_t)) + Workspace::pad(scan_scratch_bytes(rows));
}

static CountScratch carve_counts(int64_t rows, void* workspace, size_t bytes) {
    Workspace ws(workspace, bytes);
    CountScratch c;
    c.counts = ws.take<int32_t>((size_t)(rows > 0 ? rows : 1));
    c.scan_bytes = scan_scratch_bytes(rows);
    c.scan = ws.take<char>(c.scan_bytes);
    c.ok = ws.ok();
    return c;
}

}  // namespace nb200

using namespace nb200;

extern "C" size_t nb200_pattern_workspace_bytes(int64_t rows) { return count_scratch_bytes(rows); }

extern "C" int nb200_csr_triangle_count(int64_t rows, const int64_t* indices, const int64_t* indptr, int64_t k, int lower,
                                        int64_t* out_indptr, void* workspace, size_t workspace_bytes, nb200_stream stream) {
    if (rows < 0 || !out_indptr || !workspace || (rows > 0 && !indptr)) return NB200_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    CountScratch c = carve_counts(rows, workspace, workspace_bytes);
    if (!c.ok) return NB200_ERR_WORKSPACE;
    if (rows > 0) triangle_count_kernel<<<pat_grid(rows), kPatThreads, 0, st>>>(rows, indices, indptr, k, lower != 0, c.counts);
    return exclusive_scan_i32_to_i64(rows, c.counts, out_indptr, c.scan, c.scan_bytes, st);
}

extern "C" int nb200_csr_triangle_fill(int64_t rows, const void* data, const int64_t* indices, const int64_t* indptr,
                                       int64_t k, int lower, const int64_t* out_indptr, void* out_data,
                                       int64_t* out_indices, int64_t* out_pos, int dtype, nb200_stream stream) {
    if (rows < 0 || !out_indptr || (rows > 0 && !indptr)) return NB200_ERR_BAD_ARG;
    if (rows == 0) return NB200_OK;
    cudaStream_t st = as_stream(stream);
    return NB200_DISPATCH_T(dtype,
        (triangle_fill_kernel<T><<<pat_grid(rows), kPatThreads, 0, st>>>(rows, (const T*)data, indices, indptr, k, lower != 0,
                                                                        out_indptr, (T*)out_data, out_indices, out_pos),
         launch_status()));
}

extern "C" int nb200_csr_lincomb_count(int64_t rows, const int64_t* A_indices, const int64_t* A_indptr,
                                       const int64_t* B_indices, const int64_t* B_indptr, int64_t* C_indptr,
                                       void* workspace, size_t workspace_bytes, nb200_stream stream) {
    if (rows < 0 || !C_indptr || !workspace || (rows > 0 && (!A_indptr || !B_indptr))) return NB200_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    CountScratch c = carve_counts(rows, workspace, workspace_bytes);
    if (!c.ok) return NB200_ERR_WORKSPACE;
    if (rows > 0) lincomb_count_kernel<<<pat_grid(rows), kPatThreads, 0, st>>>(rows, A_indices, A_indptr, B_indices, B_indptr, c.counts);
    return exclusive_scan_i32_to_i64(rows, c.counts, C_indptr, c.scan, c.scan_bytes, st);
}

extern "C" int nb200_csr_lincomb_fill(int64_t rows, double alpha, const void* A_data, const int64_t* A_indices,
                                      const int64_t* A_indptr, double beta, const void* B_data, const int64_t* B_indices,
                                      const int64_t* B_indptr, const int64_t* C_indptr, void* C_data, int64_t* C_indices,
                                      int dtype, nb200_stream stream) {
    if (rows < 0 || (rows > 0 && (!A_indptr || !B_indptr || !C_indptr))) return NB200_ERR_BAD_ARG;
    if (rows == 0) return NB200_OK;
    cudaStream_t st = as_stream(stream);
    return NB200_DISPATCH_T(dtype,
        (lincomb_fill_kernel<T><<<pat_grid(rows), kPatThreads, 0, st>>>(rows, (T)alpha, (const T*)A_data, A_indices, A_indptr,
                                                                       (T)beta, (const T*)B_data, B_indices, B_indptr,
                                                                       C_indptr, (T*)C_data, C_indices),
         launch_status()));
}

extern "C" int nb200_csr_lincomb_backward(int64_t rows, double alpha, const int64_t* A_indices, const int64_t* A_indptr,
                                          double beta, const int64_t* B_indices, const int64_t* B_indptr,
                                          const void* grad_C, const int64_t* C_indices, const int64_t* C_indptr,
                                          void* grad_A, void* grad_B, int dtype, nb200_stream stream) {
    if (rows < 0 || (rows > 0 && (!A_indptr || !B_indptr || !C_indptr))) return NB200_ERR_BAD_ARG;
    if (rows == 0) return NB200_OK;
    cudaStream_t st = as_stream(stream);
    return NB200_DISPATCH_T(dtype, ([&]() -> int {
        lincomb_backward_kernel<T><<<pat_grid(rows), kPatThreads, 0, st>>>(rows, (T)alpha, A_indices, A_indptr, (const T*)grad_C,
                                                                          C_indices, C_indptr, (T*)grad_A);
        lincomb_backward_kernel<T><<<pat_grid(rows), kPatThreads, 0, st>>>(rows, (T)beta, B_indices, B_indptr, (const T*)grad_C,
                                                                          C_indices, C_indptr, (T*)grad_B);
        return launch_status();
    }()));
}

extern "C" size_t nb200_coo_workspace_bytes(int64_t n) {
    const size_t m = (size_t)(n > 0 ? n : 1);
    return 4 * Workspace::pad(m * sizeof(uint32_t)) + Workspace::pad(sort_scratch_bytes(n));
}

extern "C" int nb200_coo_to_csr(int64_t n, const int64_t* row_ind, const int64_t* col_ind, int64_t nrows, int64_t ncols,
                                int sort_columns, int64_t* perm, int64_t* indptr, void* workspace, size_t workspace_bytes,
                                nb200_stream stream) {
    if (n < 0 || nrows < 0 || ncols < 0 || !indptr || !workspace || (n > 0 && (!row_ind || !col_ind || !perm)))
        return NB200_ERR_BAD_ARG;
    if (n >= 0x7fffffffLL || nrows >= 0x7fffffffLL || ncols >= 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    cudaStream_t st = as_stream(stream);
    Workspace ws(workspace, workspace_bytes);
    const size_t m = (size_t)(n > 0 ? n : 1);
    uint32_t* keys_a = ws.take<uint32_t>(m);
    uint32_t* vals_a = ws.take<uint32_t>(m);
    uint32_t* keys_b = ws.take<uint32_t>(m);
    uint32_t* vals_b = ws.take<uint32_t>(m);
    const size_t ssb = sort_scratch_bytes(n);
    char* sscratch = ws.take<char>(ssb);
    if (!ws.ok()) return NB200_ERR_WORKSPACE;
    const uint32_t* order = nullptr;
    const uint32_t* sorted_rows = keys_a;
    const uint32_t* sorted_vals = vals_a;
    if (n > 0) {
        bool in_a = true;
        int rc;
        if (sort_columns) {
            // least significant key first: by column, then (stably) by row
            coo_init_kernel<<<pat_grid(n), kPatThreads, 0, st>>>(n, col_ind, nullptr, keys_a, vals_a);
            rc = sort_pairs_u32(n, bits_for(ncols > 0 ? ncols - 1 : 0), keys_a, vals_a, keys_b, vals_b, &in_a, sscratch, ssb, st);
            if (rc != NB200_OK) return rc;
            order = in_a ? vals_a : vals_b;
        }
        uint32_t* k0 = (order == vals_a) ? keys_b : keys_a;     // the pair of buffers that `order` does not live in
        uint32_t* v0 = (order == vals_a) ? vals_b : vals_a;
        uint32_t* k1 = (order == vals_a) ? keys_a : keys_b;
        uint32_t* v1 = (order == vals_a) ? vals_a : vals_b;
        coo_init_kernel<<<pat_grid(n), kPatThreads, 0, st>>>(n, row_ind, order, k0, v0);
        rc = sort_pairs_u32(n, bits_for(nrows > 0 ? nrows - 1 : 0), k0, v0, k1, v1, &in_a, sscratch, ssb, st);
        if (rc != NB200_OK) return rc;
        sorted_rows = in_a ? k0 : k1;
        sorted_vals = in_a ? v0 : v1;
    }
    const int64_t span = n > nrows + 1 ? n : nrows + 1;
    coo_emit_kernel<<<pat_grid(span), kPatThreads, 0, st>>>(n, nrows, sorted_rows, sorted_vals, perm, indptr);
    return launch_status();
}
