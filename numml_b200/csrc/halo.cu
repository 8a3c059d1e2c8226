// Halo exchange of a row-partitioned SpMV over peer memory (NVLink), without a communication library
// on the critical path.
//
// Every rank owns one exchange buffer that its neighbours have mapped (CUDA IPC).  A rank only ever
// WRITES its own buffer and only READS its neighbours' buffers, with ordinary loads and stores:
//
//     publish   pack the values the neighbours need into this rank's buffer, then store the step number
//               into a flag word of the same buffer (release, system scope);
//     pull      wait until a neighbour's flag has reached the current step (acquire, system scope,
//               bounded by a cycle budget), then copy that neighbour's packed values into this rank's
//               own memory, where the compute kernels find them;
//     pull_add  the same for gradients: partial sums that the neighbours computed for columns this rank
//               owns are read from their buffers and added in ascending peer order (reproducible).
//
// Packed areas are double-buffered by step parity.  A rank overwrites the half of step t only after it
// has seen every neighbour's flag reach t - 1 (its own pull of step t - 1 waited for exactly that), and a
// neighbour publishes step t - 1 only after its pull of step t - 2 has finished: nobody can still be
// reading the half that is being rewritten.  This needs every rank that reads from a neighbour to be read
// by that neighbour as well, which holds for matrices whose pattern equals its transpose.
//
// No kernel here waits without a limit: when the budget runs out the kernel stores
// NB200_ERR_WAIT_BUDGET into the status word and returns without copying.  Kernels of different ranks
// wait on one another, so each rank must run on a GPU of its own.
#include "common.cuh"
#include <cstring>

namespace nb200 {

constexpr int kHaloThreads = 256;
constexpr int kHaloDescWords = 8;   // int64 words per neighbour descriptor
// descriptor layout (int64):
//   [0] address of the neighbour's packed area (2 halves of [1] elements each)
//   [1] elements per half of that area
//   [2] first element of this rank's segment within a half
//   [3] elements in the segment
//   [4] first element of the destination in this rank's vector (pull only)
//   [5] address of the neighbour's flag word for this area

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
// Loads that may not be served from a stale line of this SM's L1 (the halves are rewritten every other step)
__device__ __forceinline__ float ld_fresh(const float* p) { return __ldcv(p); }
__device__ __forceinline__ double ld_fresh(const double* p) { return __ldcv(p); }

// Wait until *flag >= want; false if `budget` SM cycles pass first.
__device__ __forceinline__ bool wait_for_step(const int* flag, int want, long long budget) {
    if (ld_acquire_sys(flag) >= want) return true;
    const long long t0 = clock64();
    while (ld_acquire_sys(flag) < want) {
        if (clock64() - t0 > budget) return false;
        __nanosleep(64);
    }
    return true;
}

template <typename T>
__global__ void __launch_bounds__(kHaloThreads)
halo_publish_kernel(int64_t count, const T* __restrict__ src, const int64_t* __restrict__ idx, T* area,
                    int* flag, int* step_word, int bump, unsigned* arrivals) {
    // every block reads the step before any block can be the last one to arrive below
    const int t = *step_word + (bump ? 1 : 0);
    T* dst = area + (size_t)(t & 1) * (size_t)count;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (!idx && ((count * sizeof(T)) & 15) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
        // a straight copy (the block of rows of a dense operand): 16 bytes per access
        const uint4* s16 = reinterpret_cast<const uint4*>(src);
        uint4* d16 = reinterpret_cast<uint4*>(dst);
        const int64_t units = (int64_t)(count * sizeof(T) / 16);
        for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < units; k += stride) d16[k] = s16[k];
    } else {
        for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < count; k += stride)
            dst[k] = src[idx ? idx[k] : k];
    }
    // Device scope is enough here: the last block observes the other blocks' arrivals through the counter and its own
    // system-scope fence below then orders everything they wrote before the flag (fences are cumulative); a
    // system-scope fence in every thread costs several microseconds per launch.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(arrivals, 1u) == gridDim.x - 1) {
        // last block: everything is packed and fenced; advance the step and raise the flag
        *arrivals = 0;
        if (bump) *step_word = t;
        __threadfence_system();
        st_release_sys(flag, t);
    }
}

// publish with the values computed on the way: element r of the packed area is the row sum
// sum_k data[perm[k]] * x[indices[k]] over row r of (indptr, indices), entries in storage order, unfused -- the
// partial sums of grad_x that a rank owes its neighbours, one row per halo column (the ghost rows of the
// row-partitioned driver).  One launch instead of a row-sum kernel followed by a packing kernel.
template <typename T, typename I>
__global__ void __launch_bounds__(kHaloThreads)
halo_publish_rowsums_kernel(int64_t rows, const T* __restrict__ data, const I* __restrict__ indices,
                            const I* __restrict__ indptr, const I* __restrict__ perm, const T* __restrict__ x,
                            T* area, int* flag, int* step_word, int bump, unsigned* arrivals) {
    const int t = *step_word + (bump ? 1 : 0);
    T* dst = area + (size_t)(t & 1) * (size_t)rows;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += stride) {
        T acc = 0;
        for (int64_t k = (int64_t)indptr[r]; k < (int64_t)indptr[r + 1]; ++k) {
            const T a = perm ? data[(int64_t)perm[k]] : data[k];
            acc = add_rn(acc, mul_rn(a, x[(int64_t)indices[k]]));
        }
        dst[r] = acc;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(arrivals, 1u) == gridDim.x - 1) {
        *arrivals = 0;
        if (bump) *step_word = t;
        __threadfence_system();
        st_release_sys(flag, t);
    }
}

template <typename T>
__global__ void __launch_bounds__(kHaloThreads)
halo_pull_kernel(const int64_t* __restrict__ desc, T* dst_base, const int* step_word, int32_t* status, long long budget) {
    const int64_t* d = desc + (int64_t)blockIdx.y * kHaloDescWords;
    const int t = *step_word;
    __shared__ int ready;
    if (threadIdx.x == 0) {
        ready = wait_for_step(reinterpret_cast<const int*>(d[5]), t, budget) ? 1 : 0;
        if (!ready && status) atomicExch(status, (int)NB200_ERR_WAIT_BUDGET);
    }
    __syncthreads();
    if (!ready) return;
    const T* src = reinterpret_cast<const T*>(d[0]) + (size_t)(t & 1) * (size_t)d[1] + d[2];
    T* dst = dst_base + d[4];
    const int64_t count = d[3], stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < count; k += stride) dst[k] = ld_fresh(src + k);
}

template <typename T>
__global__ void __launch_bounds__(kHaloThreads)
halo_pull_add_kernel(int npeers, const int64_t* __restrict__ desc, int64_t ntargets,
                     const int64_t* __restrict__ target, const int64_t* __restrict__ target_ptr,
                     const int32_t* __restrict__ source_peer, const int64_t* __restrict__ source_elem,
                     T* grad, const int* step_word, int32_t* status, long long budget) {
    const int t = *step_word;
    __shared__ int ready;
    if (threadIdx.x == 0) {
        int ok = 1;
        for (int p = 0; p < npeers && ok; ++p)
            ok = wait_for_step(reinterpret_cast<const int*>(desc[(int64_t)p * kHaloDescWords + 5]), t, budget) ? 1 : 0;
        if (!ok && status) atomicExch(status, (int)NB200_ERR_WAIT_BUDGET);
        ready = ok;
    }
    __syncthreads();
    if (!ready) return;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < ntargets; j += stride) {
        T acc = grad[target[j]];
        for (int64_t c = target_ptr[j]; c < target_ptr[j + 1]; ++c) {     // neighbours in ascending order
            const int64_t* d = desc + (int64_t)source_peer[c] * kHaloDescWords;
            const T* half = reinterpret_cast<const T*>(d[0]) + (size_t)(t & 1) * (size_t)d[1];
            acc = add_rn(acc, ld_fresh(half + source_elem[c]));
        }
        grad[target[j]] = acc;
    }
}

// ---------------------------------------------------------------------------------------------
// Rows of a dense operand (SpMM): the same protocol, items are rows of `w16` 16-byte units.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_fresh(const uint4* p) { return __ldcv(p); }

// Row descriptor (int64 words, kHaloDescWords per neighbour):
//   [0] address of the neighbour's area (2 halves of [1] rows each)   [1] rows per half
//   [2] first halo slot of this neighbour in `row_of_slot`            [3] number of slots
//   [4] first destination row in this rank's matrix                   [5] address of the neighbour's flag word
// Slot h of the segment receives row row_of_slot[[2] + h] of the neighbour's published block.
__global__ void __launch_bounds__(kHaloThreads)
halo_pull_rows_kernel(const int64_t* __restrict__ desc, const int64_t* __restrict__ row_of_slot, int64_t w16,
                      uint4* dst_base, const int* step_word, int32_t* status, long long budget) {
    const int64_t* d = desc + (int64_t)blockIdx.y * kHaloDescWords;
    const int t = *step_word;
    __shared__ int ready;
    if (threadIdx.x == 0) {
        ready = wait_for_step(reinterpret_cast<const int*>(d[5]), t, budget) ? 1 : 0;
        if (!ready && status) atomicExch(status, (int)NB200_ERR_WAIT_BUDGET);
    }
    __syncthreads();
    if (!ready) return;
    const uint4* half = reinterpret_cast<const uint4*>(d[0]) + (size_t)(t & 1) * (size_t)d[1] * (size_t)w16;
    const int64_t* rows = row_of_slot + d[2];
    uint4* dst = dst_base + (size_t)d[4] * (size_t)w16;
    // a warp per row (no index arithmetic per unit), four rows in flight per warp
    const int lane = threadIdx.x & 31;
    const int64_t nslots = d[3];
    const int64_t warps = (int64_t)gridDim.x * (kHaloThreads / 32);
    constexpr int U = 4;
    for (int64_t h0 = (int64_t)blockIdx.x * (kHaloThreads / 32) + (threadIdx.x >> 5); h0 < nslots; h0 += U * warps) {
        const uint4* from[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t h = h0 + u * warps;
            from[u] = h < nslots ? half + rows[h] * w16 : nullptr;
        }
        for (int64_t c = lane; c < w16; c += 32) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (from[u]) v[u] = ld_fresh(from[u] + c);
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (from[u]) dst[(h0 + u * warps) * w16 + c] = v[u];
        }
    }
}

template <typename T> struct Unit16;
template <> struct Unit16<float> {
    static __device__ __forceinline__ uint4 add(uint4 a, uint4 b) {
        a.x = __float_as_uint(__fadd_rn(__uint_as_float(a.x), __uint_as_float(b.x)));
        a.y = __float_as_uint(__fadd_rn(__uint_as_float(a.y), __uint_as_float(b.y)));
        a.z = __float_as_uint(__fadd_rn(__uint_as_float(a.z), __uint_as_float(b.z)));
        a.w = __float_as_uint(__fadd_rn(__uint_as_float(a.w), __uint_as_float(b.w)));
        return a;
    }
};
template <> struct Unit16<double> {
    static __device__ __forceinline__ uint4 add(uint4 a, uint4 b) {
        const double lo = __dadd_rn(__hiloint2double((int)a.y, (int)a.x), __hiloint2double((int)b.y, (int)b.x));
        const double hi = __dadd_rn(__hiloint2double((int)a.w, (int)a.z), __hiloint2double((int)b.w, (int)b.z));
        a.x = (unsigned)__double2loint(lo); a.y = (unsigned)__double2hiint(lo);
        a.z = (unsigned)__double2loint(hi); a.w = (unsigned)__double2hiint(hi);
        return a;
    }
};

// grad row target[j] += the rows source_elem[c] of the neighbours source_peer[c], c in target_ptr[j] ..
// target_ptr[j + 1], neighbours in ascending order; descriptor words [0], [1] (rows per half), [5] are used.
template <typename T>
__global__ void __launch_bounds__(kHaloThreads)
halo_pull_add_rows_kernel(int npeers, const int64_t* __restrict__ desc, int64_t ntargets,
                          const int64_t* __restrict__ target, const int64_t* __restrict__ target_ptr,
                          const int32_t* __restrict__ source_peer, const int64_t* __restrict__ source_elem,
                          int64_t w16, uint4* grad, const int* step_word, int32_t* status, long long budget) {
    const int t = *step_word;
    __shared__ int ready;
    if (threadIdx.x == 0) {
        int ok = 1;
        for (int p = 0; p < npeers && ok; ++p)
            ok = wait_for_step(reinterpret_cast<const int*>(desc[(int64_t)p * kHaloDescWords + 5]), t, budget) ? 1 : 0;
        if (!ok && status) atomicExch(status, (int)NB200_ERR_WAIT_BUDGET);
        ready = ok;
    }
    __syncthreads();
    if (!ready) return;
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (kHaloThreads / 32);
    for (int64_t j = (int64_t)blockIdx.x * (kHaloThreads / 32) + (threadIdx.x >> 5); j < ntargets; j += warps) {
        const int64_t q0 = target_ptr[j], q1 = target_ptr[j + 1];
        uint4* home = grad + target[j] * w16;
        for (int64_t c = lane; c < w16; c += 32) {
            uint4 acc = home[c];
            for (int64_t q = q0; q < q1; ++q) {                          // neighbours in ascending order
                const int64_t* d = desc + (int64_t)source_peer[q] * kHaloDescWords;
                const uint4* half = reinterpret_cast<const uint4*>(d[0]) + (size_t)(t & 1) * (size_t)d[1] * (size_t)w16;
                acc = Unit16<T>::add(acc, ld_fresh(half + source_elem[q] * w16 + c));
            }
            home[c] = acc;
        }
    }
}

static inline unsigned halo_grid(int64_t count, int cap) {
    const int64_t want = ceil_div(count > 0 ? count : 1, (int64_t)kHaloThreads);
    return (unsigned)(want < cap ? want : cap);
}

}  // namespace nb200

using namespace nb200;

extern "C" int nb200_halo_publish(int64_t count, const void* src, const int64_t* idx, void* area, int32_t* flag,
                                  int32_t* step_word, int bump_step, uint32_t* arrivals, int dtype, nb200_stream stream) {
    if (count < 0 || !area || !flag || !step_word || !arrivals || (count > 0 && !src)) return NB200_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    const unsigned grid = halo_grid(count, count > (int64_t)1 << 22 ? kSMs * 8 : 64);
    return NB200_DISPATCH_T(dtype,
        (halo_publish_kernel<T><<<grid, kHaloThreads, 0, st>>>(count, (const T*)src, idx, (T*)area, flag, step_word,
                                                               bump_step, arrivals), launch_status()));
}

extern "C" int nb200_halo_publish_rowsums(int64_t rows, const void* data, const void* indices, const void* indptr,
                                          const void* perm, const void* x, void* area, int32_t* flag, int32_t* step_word,
                                          int bump_step, uint32_t* arrivals, int dtype, int itype, nb200_stream stream) {
    if (rows < 0 || !area || !flag || !step_word || !arrivals) return NB200_ERR_BAD_ARG;
    if (rows > 0 && (!data || !indices || !indptr || !x)) return NB200_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    const unsigned grid = halo_grid(rows, 64);
    return NB200_DISPATCH(dtype, itype,
        (halo_publish_rowsums_kernel<T, I><<<grid, kHaloThreads, 0, st>>>(rows, (const T*)data, (const I*)indices,
             (const I*)indptr, (const I*)perm, (const T*)x, (T*)area, flag, step_word, bump_step, arrivals), launch_status()));
}

extern "C" int nb200_halo_pull(int npeers, const int64_t* desc, int64_t largest_segment, void* dst,
                               const int32_t* step_word, int32_t* status, int64_t wait_budget_cycles,
                               int dtype, nb200_stream stream) {
    if (npeers < 0 || largest_segment < 0 || !step_word || (npeers > 0 && (!desc || !dst))) return NB200_ERR_BAD_ARG;
    if (npeers == 0) return NB200_OK;
    cudaStream_t st = as_stream(stream);
    const dim3 grid(halo_grid(largest_segment, 32), (unsigned)npeers);
    const long long budget = wait_budget_cycles > 0 ? wait_budget_cycles : 4000000000LL;
    return NB200_DISPATCH_T(dtype,
        (halo_pull_kernel<T><<<grid, kHaloThreads, 0, st>>>(desc, (T*)dst, step_word, status, budget), launch_status()));
}

extern "C" int nb200_halo_pull_add(int npeers, const int64_t* desc, int64_t ntargets, const int64_t* target,
                                   const int64_t* target_ptr, const int32_t* source_peer, const int64_t* source_elem,
                                   void* grad, const int32_t* step_word, int32_t* status, int64_t wait_budget_cycles,
                                   int dtype, nb200_stream stream) {
    if (npeers < 0 || ntargets < 0 || !step_word) return NB200_ERR_BAD_ARG;
    if (npeers == 0 || ntargets == 0) return NB200_OK;
    if (!desc || !target || !target_ptr || !source_peer || !source_elem || !grad) return NB200_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    const long long budget = wait_budget_cycles > 0 ? wait_budget_cycles : 4000000000LL;
    return NB200_DISPATCH_T(dtype,
        (halo_pull_add_kernel<T><<<halo_grid(ntargets, 128), kHaloThreads, 0, st>>>(
             npeers, desc, ntargets, target, target_ptr, source_peer, source_elem, (T*)grad, step_word, status, budget),
         launch_status()));
}

extern "C" int nb200_halo_pull_rows(int npeers, const int64_t* desc, const int64_t* row_of_slot, int64_t largest_segment,
                                    int64_t row_bytes, void* dst, const int32_t* step_word, int32_t* status,
                                    int64_t wait_budget_cycles, nb200_stream stream) {
    if (npeers < 0 || largest_segment < 0 || row_bytes <= 0 || (row_bytes & 15) != 0 || !step_word) return NB200_ERR_BAD_ARG;
    if (npeers == 0) return NB200_OK;
    if (!desc || !row_of_slot || !dst) return NB200_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(dst) & 15) != 0) return NB200_ERR_ALIGN;
    const int64_t w16 = row_bytes / 16;
    int per_peer = (kSMs * 8) / npeers;
    if (per_peer < 8) per_peer = 8;
    const dim3 grid(halo_grid(largest_segment * 32, per_peer), (unsigned)npeers);
    const long long budget = wait_budget_cycles > 0 ? wait_budget_cycles : 4000000000LL;
    halo_pull_rows_kernel<<<grid, kHaloThreads, 0, as_stream(stream)>>>(desc, row_of_slot, w16, (uint4*)dst, step_word,
                                                                       status, budget);
    return launch_status();
}

extern "C" int nb200_halo_pull_add_rows(int npeers, const int64_t* desc, int64_t ntargets, const int64_t* target,
                                        const int64_t* target_ptr, const int32_t* source_peer, const int64_t* source_elem,
                                        int64_t row_bytes, void* grad, const int32_t* step_word, int32_t* status,
                                        int64_t wait_budget_cycles, int dtype, nb200_stream stream) {
    if (npeers < 0 || ntargets < 0 || row_bytes <= 0 || (row_bytes & 15) != 0 || !step_word) return NB200_ERR_BAD_ARG;
    if (npeers == 0 || ntargets == 0) return NB200_OK;
    if (!desc || !target || !target_ptr || !source_peer || !source_elem || !grad) return NB200_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(grad) & 15) != 0) return NB200_ERR_ALIGN;
    const int64_t w16 = row_bytes / 16;
    const long long budget = wait_budget_cycles > 0 ? wait_budget_cycles : 4000000000LL;
    cudaStream_t st = as_stream(stream);
    return NB200_DISPATCH_T(dtype,
        (halo_pull_add_rows_kernel<T><<<halo_grid(ntargets * 32, kSMs * 8), kHaloThreads, 0, st>>>(
             npeers, desc, ntargets, target, target_ptr, source_peer, source_elem, w16, (uint4*)grad, step_word, status, budget),
         launch_status()));
}

// ---------------------------------------------------------------------------------------------
// Exchange buffers.  Memory that other processes map must come from cudaMalloc directly (a block carved
// out of a caching allocator's segment cannot be exported on its own), so these two calls are the one
// place where the library allocates device memory -- at set-up time, never inside an operator.
// ---------------------------------------------------------------------------------------------
extern "C" int nb200_ipc_alloc(size_t bytes, void** ptr, void* handle64) {
    if (!ptr || !handle64 || bytes == 0) return NB200_ERR_BAD_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 bytes");
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return NB200_ERR_CUDA;
    cudaIpcMemHandle_t h;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
        cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        cudaFree(p);
        return NB200_ERR_CUDA;
    }
    memcpy(handle64, &h, sizeof(h));
    *ptr = p;
    return NB200_OK;
}

extern "C" int nb200_ipc_free(void* ptr) {
    if (!ptr) return NB200_OK;
    return cudaFree(ptr) == cudaSuccess ? NB200_OK : NB200_ERR_CUDA;
}

extern "C" int nb200_ipc_open(const void* handle64, void** ptr) {
    if (!handle64 || !ptr) return NB200_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        return NB200_ERR_CUDA;
    }
    *ptr = p;
    return NB200_OK;
}

extern "C" int nb200_ipc_close(void* ptr) {
    if (!ptr) return NB200_OK;
    return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? NB200_OK : NB200_ERR_CUDA;
}
