// Device primitives: exclusive scan (reduce / scan-of-sums / apply), stable LSD radix sort of
// 32-bit (key, value) pairs, gather / scatter by an index array, index-width conversion.
// None of them waits on another CTA, so none can hang; all scratch comes from the caller.
#include "primitives.cuh"

namespace nb200 {

// ---------------------------------------------------------------------------------------------
// Block-wide exclusive scan of one value per thread.  Returns the exclusive prefix of `v` and
// the block total in `total`.  Needs THREADS/32 words of shared memory (`warp_sums`).
// ---------------------------------------------------------------------------------------------
template <typename S, int THREADS>
__device__ __forceinline__ S block_exclusive_scan(S v, S* warp_sums, S& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    S inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        S t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        S w = (lane < THREADS / 32) ? warp_sums[lane] : (S)0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            S t = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += t;
        }
        if (lane < THREADS / 32) warp_sums[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const S warp_off = warp > 0 ? warp_sums[warp - 1] : (S)0;
    total = warp_sums[THREADS / 32 - 1];
    __syncthreads();
    return warp_off + inc - v;
}

constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanChunk = kScanThreads * kScanItems;

template <typename In, typename Out>
__global__ void __launch_bounds__(kScanThreads)
scan_chunk_sums_kernel(int64_t n, const In* __restrict__ in, Out* __restrict__ sums) {
    __shared__ Out ws[kScanThreads / 32];
    const int64_t base = (int64_t)blockIdx.x * kScanChunk;
    Out t = 0;
#pragma unroll
    for (int j = 0; j < kScanItems; ++j) {
        const int64_t i = base + (int64_t)j * kScanThreads + threadIdx.x;
        if (i < n) t += (Out)in[i];
    }
    Out total;
    block_exclusive_scan<Out, kScanThreads>(t, ws, total);
    if (threadIdx.x == 0) sums[blockIdx.x] = total;
}

// One CTA turns sums[0..m) into its exclusive scan in place and writes the grand total to sums[m].
template <typename Out>
__global__ void __launch_bounds__(1024)
scan_sums_kernel(int64_t m, Out* __restrict__ sums) {
    __shared__ Out ws[32];
    Out carry = 0;
    for (int64_t base = 0; base < m; base += 1024) {
        const int64_t i = base + threadIdx.x;
        const Out v = i < m ? sums[i] : (Out)0;
        Out total;
        const Out ex = block_exclusive_scan<Out, 1024>(v, ws, total);
        if (i < m) sums[i] = carry + ex;
        carry += total;
    }
    if (threadIdx.x == 0) sums[m] = carry;
}

template <typename In, typename Out>
__global__ void __launch_bounds__(kScanThreads)
scan_apply_kernel(int64_t n, int64_t m, const In* __restrict__ in, const Out* __restrict__ sums,
                  Out* __restrict__ out) {
    __shared__ Out ws[kScanThreads / 32];
    const int64_t base = (int64_t)blockIdx.x * kScanChunk + (int64_t)threadIdx.x * kScanItems;
    Out v[kScanItems];
    Out t = 0;
#pragma unroll
    for (int j = 0; j < kScanItems; ++j) {
        v[j] = (base + j < n) ? (Out)in[base + j] : (Out)0;
        t += v[j];
    }
    Out total;
    Out run = block_exclusive_scan<Out, kScanThreads>(t, ws, total) + sums[blockIdx.x];
#pragma unroll
    for (int j = 0; j < kScanItems; ++j) {
        if (base + j < n) out[base + j] = run;
        run += v[j];
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) out[n] = sums[m];
}

template <typename Out>
__global__ void scan_empty_kernel(Out* out) { out[0] = 0; }

size_t scan_scratch_bytes(int64_t n) {
    const int64_t m = ceil_div(n > 0 ? n : 1, (int64_t)kScanChunk);
    return Workspace::pad((size_t)(m + 1) * sizeof(int64_t));
}

template <typename In, typename Out>
static int exclusive_scan(int64_t n, const In* in, Out* out, void* scratch, size_t scratch_bytes, cudaStream_t st) {
    if (n < 0) return NB200_ERR_BAD_ARG;
    if (n == 0) {
        scan_empty_kernel<Out><<<1, 1, 0, st>>>(out);
        return launch_status();
    }
    if (scratch_bytes < scan_scratch_bytes(n) || scratch == nullptr) return NB200_ERR_WORKSPACE;
    const int64_t m = ceil_div(n, (int64_t)kScanChunk);
    if (m > 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    Out* sums = static_cast<Out*>(scratch);
    scan_chunk_sums_kernel<In, Out><<<(unsigned)m, kScanThreads, 0, st>>>(n, in, sums);
    scan_sums_kernel<Out><<<1, 1024, 0, st>>>(m, sums);
    scan_apply_kernel<In, Out><<<(unsigned)m, kScanThreads, 0, st>>>(n, m, in, sums, out);
    return launch_status();
}

int exclusive_scan_i32_to_i32(int64_t n, const int32_t* in, int32_t* out, void* scratch, size_t sb, cudaStream_t st) {
    return exclusive_scan<int32_t, int32_t>(n, in, out, scratch, sb, st);
}
int exclusive_scan_i32_to_i64(int64_t n, const int32_t* in, int64_t* out, void* scratch, size_t sb, cudaStream_t st) {
    return exclusive_scan<int32_t, int64_t>(n, in, out, scratch, sb, st);
}

// ---------------------------------------------------------------------------------------------
// Radix sort, 8 bits per pass.  A CTA owns a tile of 2048 consecutive items; inside the tile
// warp w owns items [256w, 256w+256) and visits them in 8 rounds of 32 consecutive items, so
// (warp, round, lane) order is input order and the ranking below is stable.
// ---------------------------------------------------------------------------------------------
constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortRounds = 8;
constexpr int kSortTile = kSortThreads * kSortRounds;

__global__ void __launch_bounds__(kSortThreads)
radix_hist_kernel(int64_t n, int shift, const uint32_t* __restrict__ keys, int32_t* __restrict__ hist, int nblocks) {
    __shared__ int32_t h[256];
    h[threadIdx.x] = 0;
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * kSortTile;
#pragma unroll
    for (int j = 0; j < kSortRounds; ++j) {
        const int64_t i = base + (int64_t)j * kSortThreads + threadIdx.x;
        if (i < n) atomicAdd(&h[(keys[i] >> shift) & 0xffu], 1);
    }
    __syncthreads();
    hist[(int64_t)threadIdx.x * nblocks + blockIdx.x] = h[threadIdx.x];
}

__global__ void __launch_bounds__(kSortThreads)
radix_scatter_kernel(int64_t n, int shift, const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                     uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out,
                     const int32_t* __restrict__ offsets, int nblocks) {
    __shared__ uint32_t cnt[kSortWarps][256];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int w = 0; w < kSortWarps; ++w) cnt[w][tid] = 0;
    __syncthreads();

    const int64_t warp_base = (int64_t)blockIdx.x * kSortTile + (int64_t)warp * (kSortRounds * 32);
    uint32_t key[kSortRounds], val[kSortRounds], rank[kSortRounds];
#pragma unroll
    for (int r = 0; r < kSortRounds; ++r) {
        const int64_t i = warp_base + r * 32 + lane;
        const bool valid = i < n;
        key[r] = valid ? keys_in[i] : 0u;
        val[r] = valid ? vals_in[i] : 0u;
        const uint32_t d = valid ? ((key[r] >> shift) & 0xffu) : 256u;
        const uint32_t peers = __match_any_sync(0xffffffffu, d);
        const int leader = __ffs(peers) - 1;
        uint32_t start = 0;
        if (valid && lane == leader) {
            start = cnt[warp][d];
            cnt[warp][d] = start + __popc(peers);
        }
        start = __shfl_sync(0xffffffffu, start, leader);
        rank[r] = start + __popc(peers & ((1u << lane) - 1u));
        __syncwarp();
    }
    __syncthreads();
    {   // thread d: running offset of digit d over the warps of this CTA, on top of the global one
        uint32_t run = (uint32_t)offsets[(int64_t)tid * nblocks + blockIdx.x];
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w) {
            const uint32_t c = cnt[w][tid];
            cnt[w][tid] = run;
            run += c;
        }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kSortRounds; ++r) {
        const int64_t i = warp_base + r * 32 + lane;
        if (i < n) {
            const uint32_t d = (key[r] >> shift) & 0xffu;
            const uint32_t pos = cnt[warp][d] + rank[r];
            keys_out[pos] = key[r];
            vals_out[pos] = val[r];
        }
    }
}

static inline int64_t sort_blocks(int64_t n) { return ceil_div(n > 0 ? n : 1, (int64_t)kSortTile); }

size_t sort_scratch_bytes(int64_t n) {
    const int64_t cells = sort_blocks(n) * 256;
    return 2 * Workspace::pad((size_t)(cells + 1) * sizeof(int32_t)) + scan_scratch_bytes(cells);
}

int sort_pairs_u32(int64_t n, int key_bits, uint32_t* keys_a, uint32_t* vals_a, uint32_t* keys_b,
                   uint32_t* vals_b, bool* result_in_a, void* scratch, size_t scratch_bytes, cudaStream_t st) {
    *result_in_a = true;
    if (n < 0 || key_bits < 0 || key_bits > 32) return NB200_ERR_BAD_ARG;
    if (n >= 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    if (n == 0 || key_bits == 0) return NB200_OK;
    const int64_t nb = sort_blocks(n);
    const int64_t cells = nb * 256;
    Workspace ws(scratch, scratch_bytes);
    int32_t* hist = ws.take<int32_t>((size_t)cells + 1);
    int32_t* offs = ws.take<int32_t>((size_t)cells + 1);
    const size_t ssb = scan_scratch_bytes(cells);
    char* sscratch = ws.take<char>(ssb);
    if (!ws.ok()) return NB200_ERR_WORKSPACE;
    bool in_a = true;
    for (int shift = 0; shift < key_bits; shift += 8) {
        uint32_t* ki = in_a ? keys_a : keys_b;
        uint32_t* vi = in_a ? vals_a : vals_b;
        uint32_t* ko = in_a ? keys_b : keys_a;
        uint32_t* vo = in_a ? vals_b : vals_a;
        radix_hist_kernel<<<(unsigned)nb, kSortThreads, 0, st>>>(n, shift, ki, hist, (int)nb);
        int rc = exclusive_scan<int32_t, int32_t>(cells, hist, offs, sscratch, ssb, st);
        if (rc != NB200_OK) return rc;
        radix_scatter_kernel<<<(unsigned)nb, kSortThreads, 0, st>>>(n, shift, ki, vi, ko, vo, offs, (int)nb);
        in_a = !in_a;
    }
    *result_in_a = in_a;
    return launch_status();
}

// ---------------------------------------------------------------------------------------------
// Elementwise helpers
// ---------------------------------------------------------------------------------------------
template <typename T, typename I>
__global__ void gather_kernel(int64_t n, const T* __restrict__ src, const I* __restrict__ idx, T* __restrict__ dst) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += stride) dst[k] = ldg(src + idx[k]);
}
template <typename T, typename I>
__global__ void scatter_kernel(int64_t n, const T* __restrict__ src, const I* __restrict__ idx, T* __restrict__ dst) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += stride) dst[idx[k]] = src[k];
}
template <typename A, typename B>
__global__ void convert_kernel(int64_t n, const A* __restrict__ in, B* __restrict__ out) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += stride) out[k] = (B)in[k];
}

static inline unsigned ew_grid(int64_t n) {
    const int64_t want = ceil_div(n, (int64_t)256);
    return (unsigned)(want < 1 ? 1 : (want > (int64_t)kSMs * 32 ? (int64_t)kSMs * 32 : want));
}

}  // namespace nb200

using namespace nb200;

extern "C" int nb200_gather(int64_t n, const void* src, const void* idx, void* dst, int dtype, int itype, nb200_stream stream) {
    if (n < 0) return NB200_ERR_BAD_ARG;
    if (n == 0) return NB200_OK;
    if (!src || !idx || !dst) return NB200_ERR_BAD_ARG;
    return NB200_DISPATCH(dtype, itype,
        (gather_kernel<T, I><<<ew_grid(n), 256, 0, as_stream(stream)>>>(n, (const T*)src, (const I*)idx, (T*)dst), launch_status()));
}

extern "C" int nb200_scatter(int64_t n, const void* src, const void* idx, void* dst, int dtype, int itype, nb200_stream stream) {
    if (n < 0) return NB200_ERR_BAD_ARG;
    if (n == 0) return NB200_OK;
    if (!src || !idx || !dst) return NB200_ERR_BAD_ARG;
    return NB200_DISPATCH(dtype, itype,
        (scatter_kernel<T, I><<<ew_grid(n), 256, 0, as_stream(stream)>>>(n, (const T*)src, (const I*)idx, (T*)dst), launch_status()));
}

// ---------------------------------------------------------------------------------------------
// Structure check: finds, without faulting, what would make a kernel read out of bounds or give a
// wrong answer silently.  One thread per row; flags are OR-ed into one device word.
// ---------------------------------------------------------------------------------------------
namespace nb200 {
template <typename I>
__global__ void csr_check_kernel(int64_t rows, int64_t cols, int64_t nnz, const I* __restrict__ indices,
                                 const I* __restrict__ indptr, int32_t* __restrict__ flags) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int found = 0;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += stride) {
        const int64_t b = (int64_t)indptr[r], e = (int64_t)indptr[r + 1];
        if ((r == 0 && b != 0) || (r == rows - 1 && e != nnz) || b > e || b < 0 || e > nnz) {
            found |= NB200_CHECK_BAD_INDPTR;
            continue;                                      // the row's range cannot be trusted
        }
        bool diag = false;
        int64_t prev = -1;
        for (int64_t k = b; k < e; ++k) {
            const int64_t c = (int64_t)indices[k];
            if (c < 0 || c >= cols) found |= NB200_CHECK_COLUMN_RANGE;
            if (c <= prev) found |= NB200_CHECK_UNSORTED;  // also catches duplicates
            if (c == r) diag = true;
            prev = c;
        }
        if (!diag && r < cols) found |= NB200_CHECK_NO_DIAGONAL;
    }
    if (found) atomicOr(flags, found);
}
}  // namespace nb200

extern "C" int nb200_csr_check(int64_t rows, int64_t cols, int64_t nnz, const void* indices, const void* indptr,
                               int itype, int32_t* flags, nb200_stream stream) {
    if (rows < 0 || cols < 0 || nnz < 0 || !flags) return NB200_ERR_BAD_ARG;
    cudaStream_t st = nb200::as_stream(stream);
    if (cudaMemsetAsync(flags, 0, sizeof(int32_t), st) != cudaSuccess) return NB200_ERR_CUDA;
    if (rows == 0) return NB200_OK;
    if (!indptr || (nnz > 0 && !indices)) return NB200_ERR_BAD_ARG;
    const int64_t want = nb200::ceil_div(rows, (int64_t)256);
    const unsigned grid = (unsigned)(want > (int64_t)nb200::kSMs * 32 ? (int64_t)nb200::kSMs * 32 : want);
    return NB200_DISPATCH_I(itype,
        (nb200::csr_check_kernel<I><<<grid, 256, 0, st>>>(rows, cols, nnz, (const I*)indices, (const I*)indptr, flags),
         nb200::launch_status()));
}

extern "C" int nb200_narrow_indices(int64_t n, const int64_t* in64, int32_t* out32, nb200_stream stream) {
    if (n < 0) return NB200_ERR_BAD_ARG;
    if (n == 0) return NB200_OK;
    if (!in64 || !out32) return NB200_ERR_BAD_ARG;
    convert_kernel<int64_t, int32_t><<<ew_grid(n), 256, 0, as_stream(stream)>>>(n, in64, out32);
    return launch_status();
}

extern "C" int nb200_widen_indices(int64_t n, const int32_t* in32, int64_t* out64, nb200_stream stream) {
    if (n < 0) return NB200_ERR_BAD_ARG;
    if (n == 0) return NB200_OK;
    if (!in32 || !out64) return NB200_ERR_BAD_ARG;
    convert_kernel<int32_t, int64_t><<<ew_grid(n), 256, 0, as_stream(stream)>>>(n, in32, out64);
    return launch_status();
}

extern "C" int nb200_version(void) { return 100; }

extern "C" const char* nb200_status_string(int status) {
    switch (status) {
        case NB200_OK: return "ok";
        case NB200_ERR_BAD_ARG: return "bad argument";
        case NB200_ERR_ALIGN: return "pointer not 16-byte aligned";
        case NB200_ERR_TOO_LARGE: return "size too large for this index width";
        case NB200_ERR_PRECONDITION: return "structural precondition violated";
        case NB200_ERR_WAIT_BUDGET: return "bounded device-side wait ran out";
        case NB200_ERR_WORKSPACE: return "workspace too small";
        case NB200_ERR_CUDA: return "CUDA error";
        default: return "unknown status";
    }
}
