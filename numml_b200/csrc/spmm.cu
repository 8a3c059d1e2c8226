// Sparse x dense products (C = A B with dense row-major B) and the masked gradient
// grad_A[k] = <grad_C[row(k),:], B[col(k),:]> for CSR on sm_100a.
//
// A group of G lanes (G = 8, 16 or 32, chosen from the number of dense columns) owns one row of
// A.  The group reads the row's (column, value) pairs G at a time with one coalesced load and
// broadcasts them with shuffles; every lane owns VEC consecutive dense columns (one 128-bit
// load per referenced row of B) and keeps its slice of the output row in registers.  The sum
// over the row's entries is taken in storage order with separate multiply and add, so each
// output element is bit-identical to a sequential CPU loop.  With `perm` the values are read as
// data[perm[k]]: the same kernel then computes grad_B = A^T grad_C over a cached transposed
// structure without atomics.
//
// `row_order` (optional): the r-th lane group takes row row_order[r] instead of row r.  With rows
// sorted by descending length the few very long rows of a skewed matrix (one lane group walks a row
// alone, 4096 entries take about a millisecond) start first and finish under the cover of the short
// ones instead of forming a tail; every row is still summed by one group in storage order, so the
// results do not change by a bit.
#include "common.cuh"

#ifndef NB200_SPMM_GRAD_BATCH
#define NB200_SPMM_GRAD_BATCH 4   // entries reduced together in the grad_A kernel (4 or 8)
#endif
#ifndef NB200_SPMM_BATCH
#define NB200_SPMM_BATCH 4   // rows of B requested together per lane group in the forward kernel
#endif

namespace nb200 {

template <typename T, int VEC> struct Vec;
template <> struct Vec<float, 4> { using type = float4; };
template <> struct Vec<double, 2> { using type = double2; };
template <> struct Vec<float, 1> { using type = float; };
template <> struct Vec<double, 1> { using type = double; };

template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T* p, T (&v)[VEC]) {
    using V = typename Vec<T, VEC>::type;
    const V t = __ldg(reinterpret_cast<const V*>(p));
    const T* s = reinterpret_cast<const T*>(&t);
#pragma unroll
    for (int j = 0; j < VEC; ++j) v[j] = s[j];
}

template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T* p, const T (&v)[VEC]) {
    using V = typename Vec<T, VEC>::type;
    V t;
    T* s = reinterpret_cast<T*>(&t);
#pragma unroll
    for (int j = 0; j < VEC; ++j) s[j] = v[j];
    *reinterpret_cast<V*>(p) = t;
}

// ---------------------------------------------------------------------------------------------
// C[r, :] = sum_k A[r, k] B[k, :]
// ---------------------------------------------------------------------------------------------
template <typename T, typename I, int VEC, int G, bool PERM>
__global__ void __launch_bounds__(256)
spdmm_forward_kernel(int64_t rows, int64_t K, const T* __restrict__ data, const I* __restrict__ indices,
                     const I* __restrict__ indptr, const I* __restrict__ perm, const int32_t* __restrict__ row_order,
                     const T* __restrict__ B, T* __restrict__ C) {
    constexpr int ROWS_PER_WARP = 32 / G;
    const int lane = threadIdx.x & 31;
    const int gl = lane % G;                 // lane within the group
    const int gbase = lane - gl;             // first lane of the group (shuffle source offset)
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t slot = warp * ROWS_PER_WARP + lane / G;
    const bool active = slot < rows;
    const int64_t r = (active && row_order) ? (int64_t)row_order[slot] : slot;
    const int64_t s = active ? (int64_t)indptr[r] : 0;
    const int64_t e = active ? (int64_t)indptr[r + 1] : 0;

    for (int64_t cb = 0; cb < K; cb += (int64_t)G * VEC) {   // one pass per tile of G*VEC dense columns
        const int64_t col = cb + (int64_t)gl * VEC;
        const bool col_ok = col < K;
        T acc[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[j] = 0;
        // all groups of the warp iterate together so that the shuffles stay convergent
        int64_t len = e - s;
#pragma unroll
        for (int o = G; o < 32; o <<= 1) len = max(len, __shfl_xor_sync(0xffffffffu, len, o));
        for (int64_t off = 0; off < len; off += G) {
            const int64_t k = s + off + gl;
            I c_mine = 0;
            T v_mine = 0;
            if (k < e) {
                c_mine = indices[k];
                v_mine = PERM ? ldg(data + perm[k]) : data[k];
            }
            const int cnt = (int)min((int64_t)G, e - s - off);   // <= 0 for groups that are done
            // batches of BATCH entries: broadcast (column, value), issue all row loads, then accumulate in order
            constexpr int BATCH = NB200_SPMM_BATCH;
            int cnt_w = cnt;                                  // warp-uniform trip count
#pragma unroll
            for (int o = G; o < 32; o <<= 1) cnt_w = max(cnt_w, __shfl_xor_sync(0xffffffffu, cnt_w, o));
#pragma unroll 1
            for (int j0 = 0; j0 < cnt_w; j0 += BATCH) {
                I c[BATCH];
                T v[BATCH];
                T b[BATCH][VEC];
#pragma unroll
                for (int q = 0; q < BATCH; ++q) {
                    c[q] = __shfl_sync(0xffffffffu, c_mine, gbase + j0 + q);
                    v[q] = __shfl_sync(0xffffffffu, v_mine, gbase + j0 + q);
                }
#pragma unroll
                for (int q = 0; q < BATCH; ++q) {
                    if (j0 + q < cnt && col_ok) load_vec<T, VEC>(B + (int64_t)c[q] * K + col, b[q]);
                }
#pragma unroll
                for (int q = 0; q < BATCH; ++q) {
                    if (j0 + q < cnt && col_ok) {
#pragma unroll
                        for (int t = 0; t < VEC; ++t) acc[t] = add_rn(acc[t], mul_rn(v[q], b[q][t]));
                    }
                }
            }
        }
        if (active && col_ok) store_vec<T, VEC>(C + r * K + col, acc);
    }
}

// ---------------------------------------------------------------------------------------------
// grad_A[k] = sum_c grad_C[row(k), c] * B[col(k), c]
// ---------------------------------------------------------------------------------------------
template <typename T, typename I, int VEC, int G>
__global__ void __launch_bounds__(256)
spdmm_grad_A_kernel(int64_t rows, int64_t K, const I* __restrict__ indices, const I* __restrict__ indptr,
                    const int32_t* __restrict__ row_order,
                    const T* __restrict__ B, const T* __restrict__ grad_C, T* __restrict__ grad_A) {
    constexpr int ROWS_PER_WARP = 32 / G;
    const int lane = threadIdx.x & 31;
    const int gl = lane % G;
    const int gbase = lane - gl;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t slot = warp * ROWS_PER_WARP + lane / G;
    const bool active = slot < rows;
    const int64_t r = (active && row_order) ? (int64_t)row_order[slot] : slot;
    const int64_t s = active ? (int64_t)indptr[r] : 0;
    const int64_t e = active ? (int64_t)indptr[r + 1] : 0;
    const bool single_tile = K <= (int64_t)G * VEC;

    T g0[VEC];                                  // this lane's slice of grad_C[r, :] (first tile)
#pragma unroll
    for (int j = 0; j < VEC; ++j) g0[j] = 0;
    if (active && (int64_t)gl * VEC < K) load_vec<T, VEC>(grad_C + r * K + (int64_t)gl * VEC, g0);

    int64_t len = e - s;
#pragma unroll
    for (int o = G; o < 32; o <<= 1) len = max(len, __shfl_xor_sync(0xffffffffu, len, o));

    if (single_tile) {
        // GB entries at a time: their rows of B are requested before any arithmetic, each lane forms
        // GB partial dot products over its slice, and the GB sums are reduced together by recursive
        // halving (GB/2 + ... + 1 exchanges, then log2(G/GB) more) instead of GB separate butterflies.
        const bool col_ok = (int64_t)gl * VEC < K;
        constexpr int GB = NB200_SPMM_GRAD_BATCH;
        for (int64_t off = 0; off < len; off += G) {
            const int64_t k = s + off + gl;
            const I c_mine = (k < e) ? indices[k] : (I)0;
            const int cnt = (int)min((int64_t)G, e - s - off);
            T out_mine = 0;
            int cnt_w = cnt;                                  // warp-uniform trip count
#pragma unroll
            for (int o = G; o < 32; o <<= 1) cnt_w = max(cnt_w, __shfl_xor_sync(0xffffffffu, cnt_w, o));
#pragma unroll 1
            for (int j0 = 0; j0 < cnt_w; j0 += GB) {
                T b[GB][VEC];
                T p[GB];
#pragma unroll
                for (int q = 0; q < GB; ++q) {
                    const I c = __shfl_sync(0xffffffffu, c_mine, gbase + j0 + q);
#pragma unroll
                    for (int t = 0; t < VEC; ++t) b[q][t] = 0;
                    if (j0 + q < cnt && col_ok) load_vec<T, VEC>(B + (int64_t)c * K + (int64_t)gl * VEC, b[q]);
                }
#pragma unroll
                for (int q = 0; q < GB; ++q) {
                    p[q] = 0;
#pragma unroll
                    for (int t = 0; t < VEC; ++t) p[q] += g0[t] * b[q][t];
                }
                // halving steps: after the step with offset o, lanes with that bit set keep the upper half
#pragma unroll
                for (int m = GB, o = G / 2; m > 1; m >>= 1, o >>= 1) {
                    const bool up = (gl & o) != 0;
#pragma unroll
                    for (int i = 0; i < m / 2; ++i) {
                        const T send = up ? p[i] : p[i + m / 2];
                        const T keep = up ? p[i + m / 2] : p[i];
                        p[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                    }
                }
#pragma unroll
                for (int o = G / (2 * GB); o > 0; o >>= 1) p[0] += __shfl_xor_sync(0xffffffffu, p[0], o);
                // the lane whose top log2(GB) bits spell q holds entry q; route it to lane j0 + q
                const int q = (gl - j0) & (GB - 1);
                int src = 0;
#pragma unroll
                for (int bit = GB / 2, o = G / 2; bit > 0; bit >>= 1, o >>= 1) src += (q & bit) ? o : 0;
                const T v = __shfl_sync(0xffffffffu, p[0], gbase + src);
                if (gl >= j0 && gl < j0 + GB) out_mine = v;
            }
            if (k < e) grad_A[k] = out_mine;
        }
        return;
    }

    for (int64_t off = 0; off < len; off += G) {
        const int64_t k = s + off + gl;
        const I c_mine = (k < e) ? indices[k] : (I)0;
        const int cnt = (int)min((int64_t)G, e - s - off);
        T out_mine = 0;
#pragma unroll 2
        for (int j = 0; j < G; ++j) {
            const I c = __shfl_sync(0xffffffffu, c_mine, gbase + j);
            T part = 0;
            if (j < cnt) {
                const T* brow = B + (int64_t)c * K;
                if ((int64_t)gl * VEC < K) {
                    T b[VEC];
                    load_vec<T, VEC>(brow + (int64_t)gl * VEC, b);
#pragma unroll
                    for (int q = 0; q < VEC; ++q) part += g0[q] * b[q];
                }
                if (!single_tile) {
                    for (int64_t col = (int64_t)(G + gl) * VEC; col < K; col += (int64_t)G * VEC) {
                        T b[VEC], g[VEC];
                        load_vec<T, VEC>(brow + col, b);
                        load_vec<T, VEC>(grad_C + r * K + col, g);
#pragma unroll
                        for (int q = 0; q < VEC; ++q) part += g[q] * b[q];
                    }
                }
            }
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (gl == j) out_mine = part;
        }
        if (k < e) grad_A[k] = out_mine;
    }
}

template <typename T, typename I, int VEC, int G>
int spdmm_forward_cfg(int64_t rows, int64_t K, const T* data, const I* indices, const I* indptr, const I* perm,
                      const int32_t* row_order, const T* B, T* C, cudaStream_t st) {
    const int64_t warps = ceil_div(rows, (int64_t)(32 / G));
    const int64_t grid = ceil_div(warps, (int64_t)8);
    if (grid > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    if (perm)
        spdmm_forward_kernel<T, I, VEC, G, true><<<(unsigned)grid, 256, 0, st>>>(rows, K, data, indices, indptr, perm, row_order, B, C);
    else
        spdmm_forward_kernel<T, I, VEC, G, false><<<(unsigned)grid, 256, 0, st>>>(rows, K, data, indices, indptr, perm, row_order, B, C);
    return launch_status();
}

template <typename T, typename I, int VEC, int G>
int spdmm_grad_A_cfg(int64_t rows, int64_t K, const I* indices, const I* indptr, const int32_t* row_order,
                     const T* B, const T* grad_C, T* grad_A, cudaStream_t st) {
    const int64_t warps = ceil_div(rows, (int64_t)(32 / G));
    const int64_t grid = ceil_div(warps, (int64_t)8);
    if (grid > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    spdmm_grad_A_kernel<T, I, VEC, G><<<(unsigned)grid, 256, 0, st>>>(rows, K, indices, indptr, row_order, B, grad_C, grad_A);
    return launch_status();
}

// Lanes per row: the smallest of 8 / 16 / 32 that covers the K dense columns in one tile.
template <int VEC>
static inline int pick_group(int64_t K) {
    if (K <= 8 * VEC) return 8;
    if (K <= 16 * VEC) return 16;
    return 32;
}

template <typename T, typename I>
int spdmm_forward_launch(int64_t rows, int64_t K, const T* data, const I* indices, const I* indptr, const I* perm,
                         const int32_t* row_order, const T* B, T* C, cudaStream_t st) {
    if (rows == 0 || K == 0) return NB200_OK;
    constexpr int V = 16 / sizeof(T);
    const bool vec_ok = (K % V == 0) && aligned16(B) && aligned16(C);
#define NB200_FWD(VEC_, G_) spdmm_forward_cfg<T, I, VEC_, G_>(rows, K, data, indices, indptr, perm, row_order, B, C, st)
    if (vec_ok) {
        switch (pick_group<V>(K)) {
            case 8: return NB200_FWD(V, 8);
            case 16: return NB200_FWD(V, 16);
            default: return NB200_FWD(V, 32);
        }
    }
    switch (pick_group<1>(K)) {
        case 8: return NB200_FWD(1, 8);
        case 16: return NB200_FWD(1, 16);
        default: return NB200_FWD(1, 32);
    }
#undef NB200_FWD
}

template <typename T, typename I>
int spdmm_grad_A_launch(int64_t rows, int64_t K, const I* indices, const I* indptr, const int32_t* row_order,
                        const T* B, const T* grad_C, T* grad_A, cudaStream_t st) {
    if (rows == 0) return NB200_OK;
    constexpr int V = 16 / sizeof(T);
    const bool vec_ok = (K % V == 0) && aligned16(B) && aligned16(grad_C) && K > 0;
#define NB200_GA(VEC_, G_) spdmm_grad_A_cfg<T, I, VEC_, G_>(rows, K, indices, indptr, row_order, B, grad_C, grad_A, st)
    if (vec_ok) {
        switch (pick_group<V>(K)) {
            case 8: return NB200_GA(V, 8);
            case 16: return NB200_GA(V, 16);
            default: return NB200_GA(V, 32);
        }
    }
    switch (pick_group<1>(K)) {
        case 8: return NB200_GA(1, 8);
        case 16: return NB200_GA(1, 16);
        default: return NB200_GA(1, 32);
    }
#undef NB200_GA
}

}  // namespace nb200

using namespace nb200;

extern "C" int nb200_spdmm_forward(int64_t rows, int64_t cols, int64_t K, int64_t nnz,
                                   const void* data, const void* indices, const void* indptr, const void* perm,
                                   const int32_t* row_order, const void* B, void* C, int dtype, int itype,
                                   nb200_stream stream) {
    (void)cols;
    if (rows < 0 || cols < 0 || K < 0 || nnz < 0) return NB200_ERR_BAD_ARG;
    if (rows == 0 || K == 0) return NB200_OK;
    if (!indptr || !C || (nnz > 0 && (!data || !indices || !B))) return NB200_ERR_BAD_ARG;
    if (itype == NB200_I32 && nnz > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    return NB200_DISPATCH(dtype, itype,
        (spdmm_forward_launch<T, I>(rows, K, (const T*)data, (const I*)indices, (const I*)indptr, (const I*)perm,
                                    row_order, (const T*)B, (T*)C, as_stream(stream))));
}

extern "C" int nb200_spdmm_backward_grad_A(int64_t rows, int64_t cols, int64_t K, int64_t nnz,
                                           const void* indices, const void* indptr, const int32_t* row_order,
                                           const void* B, const void* grad_C, void* grad_A,
                                           int dtype, int itype, nb200_stream stream) {
    (void)cols;
    if (rows < 0 || cols < 0 || K < 0 || nnz < 0) return NB200_ERR_BAD_ARG;
    if (rows == 0 || nnz == 0) return NB200_OK;
    if (!indptr || !indices || !grad_A || (K > 0 && (!B || !grad_C))) return NB200_ERR_BAD_ARG;
    if (itype == NB200_I32 && nnz > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    return NB200_DISPATCH(dtype, itype,
        (spdmm_grad_A_launch<T, I>(rows, K, (const I*)indices, (const I*)indptr, row_order, (const T*)B,
                                   (const T*)grad_C, (T*)grad_A, as_stream(stream))));
}
