// Hash-based SpGEMM C = A B (symbolic row-nnz count, then numeric fill with column-sorted rows)
// and its masked backward, for CSR on sm_100a.
//
// Rows of C are binned by size (upper bound = number of products for the symbolic phase, exact
// nnz for the numeric phase).  The first two bins need no table at all:
//     bin 0:  one thread per row                                     (entries of A <= 8, products <= 64)
//             the selected rows of B are sorted runs; the thread merges them in registers, which yields the
//             columns in ascending order and the products of a column in run order -- the reference's order
//             of additions.  A warp forms 32 rows for the instruction cost of one.
//     bin 1:  one warp per row                                       (products <= 32, entries of A <= 32)
//             lane p owns product p in the reference's accumulation order (entries of the row of A in
//             storage order, for each the entries of the row of B in storage order); equal columns find
//             each other with match.any, the lowest lane of a group is its leader, a leader's position in
//             the sorted row is the number of leaders with a smaller column, and the group's products are
//             added in lane order.  The loads behind a row form a chain five levels deep; a warp keeps five
//             rows in flight, one per level, so that the chain's latency is paid once per five rows.
//     Rows of both bins come out bit-identical to the reference's CPU loop and the same from run to run.
// The other bins have a team size and an open-addressing hash table:
//     bin 2:   8 lanes per row,  64-slot table in shared memory      (size <= 32)
//     bin 3:  32 lanes per row, 512-slot table in shared memory      (size <= 256)
//     bin 4: 256 threads per row, 8192-slot (symbolic) / 4096-slot (numeric) table in shared memory
//     bin 5: 256 threads per row, table in a caller-provided global-memory spill area
// Column keys are inserted with atomicCAS and linear probing (load factor <= 1/2); the numeric
// phase accumulates values with shared/global atomics and then emits the row in ascending column
// order: for 64-slot tables the occupied slots are gathered into a dense list and every entry is
// placed at the number of smaller keys in that list (its position in the sorted row); larger
// tables are bitonic-sorted as a whole (empty slots sort last) and their first nnz entries
// copied out.  The pattern is
// purely structural: a product that cancels numerically still yields a stored zero, as in the
// reference.
//
// Backward is atomic-free: grad_A[(i,j)] walks row j of B against row i of C in ascending
// column order; grad_B[(j,c)] walks column j of A (through the cached transposed structure of
// A) in ascending row order and looks c up in the corresponding rows of C.  Both orders are the
// reference's, and multiply/add are unfused, so the gradients are bit-identical to its CPU loops.
#include "primitives.cuh"

namespace nb200 {

constexpr uint32_t kEmptyKey = 0xffffffffu;
constexpr int kBins = 6;
constexpr int kThreadRowEntries = 8;   // entries of A a row may have to be merged by one thread ...
constexpr int kThreadRowMax = 64;      // ... and products
constexpr int kWarpRowMax = 32;        // products (and entries of A) a row may have to be formed by one warp
constexpr int kSpillBin = 5;
constexpr int kHeaderWords = 24;       // int64 words at the start of the workspace
// header layout (int64):
//   [0..5]  rows per bin, symbolic classification
//   [6]     spill slots needed by the symbolic phase (tables of the last bin)
//   [7]     largest per-row number of products
//   [8..13] rows per bin, numeric classification (bins 0 and 1 as in the symbolic phase, the others by nnz
//           of the output row)
//   [14]    spill slots needed by the numeric phase
//   [15]    nnz(C)
//   [16]    error word (non-zero: a spill table was too small)
constexpr int kHdrSymSpill = 6, kHdrMaxProducts = 7, kHdrNumBins = 8, kHdrNumSpill = 14, kHdrNnz = 15, kHdrError = 16;
enum RowKind : unsigned char { kThreadRow = 0, kWarpRow = 1, kHashRow = 2 };

// hash bins 2..5 by table size needed
__host__ __device__ inline int hash_bin_of(int64_t size, bool numeric) {
    if (size <= 32) return 2;
    if (size <= 256) return 3;
    if (size <= (numeric ? 2048 : 4096)) return 4;
    return 5;
}

__device__ __forceinline__ int64_t spill_table_size(int64_t size) {
    int64_t t = 64;
    while (t < 2 * size) t <<= 1;
    return t;
}

__device__ __forceinline__ uint32_t hash_key(uint32_t c) { return c * 2654435761u; }

// Insert key c; returns its slot.  The table never fills (load factor <= 1/2 by construction).
__device__ __forceinline__ uint32_t table_insert(uint32_t* keys, uint32_t mask, int shift, uint32_t c) {
    uint32_t slot = (hash_key(c) >> shift) & mask;
    while (true) {
        const uint32_t old = atomicCAS(keys + slot, kEmptyKey, c);
        if (old == kEmptyKey || old == c) return slot;
        slot = (slot + 1) & mask;
    }
}

// ---------------------------------------------------------------------------------------------
// Planning kernels
// ---------------------------------------------------------------------------------------------
template <typename I>
__global__ void spgemm_products_kernel(int64_t rows, const I* __restrict__ A_indices, const I* __restrict__ A_indptr,
                                       const I* __restrict__ B_indptr, int32_t* __restrict__ size_out,
                                       unsigned char* __restrict__ kind_out, bool b_sorted,
                                       unsigned long long* __restrict__ header) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    long long local_max = 0;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += stride) {
        long long ub = 0;
        for (int64_t a = (int64_t)A_indptr[r]; a < (int64_t)A_indptr[r + 1]; ++a) {
            const int64_t j = (int64_t)A_indices[a];
            ub += (long long)B_indptr[j + 1] - (long long)B_indptr[j];
        }
        // which kernel forms the row: a thread merging a few sorted runs, a warp with one product per lane,
        // or a hash table.  For the last the number of entries of A is folded into the size (a larger size
        // only means a larger table).
        const long long na = (long long)A_indptr[r + 1] - (long long)A_indptr[r];
        kind_out[r] = (b_sorted && na <= kThreadRowEntries && ub <= kThreadRowMax) ? kThreadRow
                      : (na <= kWarpRowMax && ub <= kWarpRowMax) ? kWarpRow : kHashRow;
        ub = max(ub, na);
        if (ub > 0x7fffffffLL) ub = 0x7fffffffLL;
        size_out[r] = (int32_t)ub;
        local_max = max(local_max, ub);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local_max = max(local_max, __shfl_xor_sync(0xffffffffu, local_max, o));
    if ((threadIdx.x & 31) == 0 && local_max > 0) atomicMax(header + kHdrMaxProducts, (unsigned long long)local_max);
}

// Distribute rows into per-bin lists (warp-aggregated appends) and size the spill tables.
// `kind` is written by spgemm_products_kernel; `size_in` is its product counts (symbolic phase) or the
// exact nnz of every output row (numeric phase).
__global__ void __launch_bounds__(256)
spgemm_classify_kernel(int64_t rows, const int32_t* __restrict__ size_in,
                       const unsigned char* __restrict__ kind, bool numeric,
                       int32_t* __restrict__ lists, int64_t* __restrict__ spill_off,
                       unsigned long long* __restrict__ header) {
    // appends are aggregated per warp (match.any), then per block (shared counters): one global atomic
    // per block and bin instead of one per warp
    __shared__ unsigned s_count[kBins];
    __shared__ unsigned long long s_base[kBins];
    const int hb = numeric ? kHdrNumBins : 0;
    const int lane = threadIdx.x & 31;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t rows_pad = ceil_div(rows, (int64_t)blockDim.x) * blockDim.x;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows_pad; r += stride) {
        if (threadIdx.x < kBins) s_count[threadIdx.x] = 0;
        __syncthreads();
        const bool ok = r < rows;
        const int32_t size = ok ? size_in[r] : 0;
        int bin = kBins;
        if (ok) bin = kind[r] != kHashRow ? (int)kind[r] : hash_bin_of(size, numeric);
        const uint32_t peers = __match_any_sync(0xffffffffu, bin);
        const int leader = __ffs(peers) - 1;
        unsigned warp_off = 0;
        if (ok && lane == leader) warp_off = atomicAdd(&s_count[bin], (unsigned)__popc(peers));
        warp_off = __shfl_sync(0xffffffffu, warp_off, leader);
        __syncthreads();
        if (threadIdx.x < kBins && s_count[threadIdx.x] > 0)
            s_base[threadIdx.x] = atomicAdd(header + hb + threadIdx.x, (unsigned long long)s_count[threadIdx.x]);
        __syncthreads();
        if (ok) {
            const int64_t pos = (int64_t)s_base[bin] + warp_off + __popc(peers & ((1u << lane) - 1u));
            lists[(int64_t)bin * rows + pos] = (int32_t)r;
            if (bin == kSpillBin) spill_off[pos] = (int64_t)atomicAdd(header + hb + kHdrSymSpill, (unsigned long long)spill_table_size(size));
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// Bins 0 and 1: rows formed without a table.
// ---------------------------------------------------------------------------------------------
// ---------------------------------------------------------------------------------------------
// Bin 0: one thread per row.  The rows of B that a row of A selects are sorted runs; with at most
// kThreadRowEntries of them a thread keeps every run's position, end and head column in registers and
// merges them: the smallest head column is the next column of the output row, and the runs whose head
// equals it contribute their products in run order -- the reference's order of additions, so the values
// are bit-identical to its CPU loop -- before they advance.  No table, no sort, no shuffles; a warp
// forms 32 rows at the instruction cost of one, and neighbouring threads read neighbouring rows.
// ---------------------------------------------------------------------------------------------
constexpr int kThreadRowStage = 448;   // output entries of one warp's 32 rows that fit its staging area

template <typename T, typename I, bool NUMERIC>
__global__ void __launch_bounds__(256)
spgemm_thread_rows_kernel(const int32_t* __restrict__ list, const unsigned long long* __restrict__ count_ptr,
                          const T* __restrict__ A_data, const I* __restrict__ A_indices, const I* __restrict__ A_indptr,
                          const T* __restrict__ B_data, const I* __restrict__ B_indices, const I* __restrict__ B_indptr,
                          int32_t* __restrict__ row_nnz, const int64_t* __restrict__ C_indptr,
                          int64_t* __restrict__ C_indices, T* __restrict__ C_data) {
    constexpr int E = kThreadRowEntries;
    constexpr unsigned kAll = 0xffffffffu;
    // numeric phase: the rows of a warp are usually 32 consecutive rows of C, i.e. one contiguous range of
    // C_indices / C_data.  The threads then write their rows into a staging area of the warp and the warp
    // copies the range out with 16-byte stores, instead of 32 threads storing 8 bytes each at a row's stride.
    __shared__ uint32_t s_col[NUMERIC ? 8 * kThreadRowStage : 1];
    __shared__ T s_val[NUMERIC ? 8 * kThreadRowStage : 1];
    const int lane = threadIdx.x & 31;
    const int64_t count = (int64_t)*count_ptr;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t base = (int64_t)blockIdx.x * blockDim.x + (threadIdx.x & ~31); base < count; base += stride) {
        const int64_t idx = base + lane;
        const bool active = idx < count;
        const int64_t row = active ? (int64_t)list[idx] : -1;
        int64_t a0 = 0;
        int na = 0;
        if (active) {
            a0 = (int64_t)A_indptr[row];
            na = (int)((int64_t)A_indptr[row + 1] - a0);
        }
        I pos[E], end[E];
        uint32_t head[E];
        T av[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
            pos[e] = 0; end[e] = 0; head[e] = kEmptyKey; av[e] = (T)0;
            if (e < na) {
                const int64_t j = (int64_t)A_indices[a0 + e];
                pos[e] = B_indptr[j];
                end[e] = B_indptr[j + 1];
                if (NUMERIC) av[e] = A_data[a0 + e];
            }
        }
#pragma unroll
        for (int e = 0; e < E; ++e)
            if (pos[e] < end[e]) head[e] = (uint32_t)B_indices[pos[e]];
        int64_t out = 0;
        bool staged = false;
        int64_t warp_out = 0;
        int warp_total = 0;
        uint32_t* wcol = s_col + (threadIdx.x >> 5) * kThreadRowStage;
        T* wval = s_val + (threadIdx.x >> 5) * kThreadRowStage;
        if (NUMERIC) {
            if (active) out = C_indptr[row];
            const int64_t row0 = __shfl_sync(kAll, row, 0);
            warp_out = __shfl_sync(kAll, out, 0);
            if (__all_sync(kAll, active && row == row0 + lane)) {
                const int64_t total = C_indptr[row0 + 32] - warp_out;
                staged = total <= kThreadRowStage;
                warp_total = (int)total;
            }
        }
        const int off = (int)(out - warp_out);
        int n = 0;
        while (true) {
            uint32_t next = kEmptyKey;
#pragma unroll
            for (int e = 0; e < E; ++e) next = min(next, head[e]);
            if (next == kEmptyKey) break;
            T sum = (T)0;
#pragma unroll
            for (int e = 0; e < E; ++e) {
                if (head[e] == next) {
                    if (NUMERIC) sum = add_rn(sum, mul_rn(av[e], B_data[pos[e]]));
                    ++pos[e];
                    head[e] = pos[e] < end[e] ? (uint32_t)B_indices[pos[e]] : kEmptyKey;
                }
            }
            if (NUMERIC) {
                if (staged) { wcol[off + n] = next; wval[off + n] = sum; }
                else { C_indices[out + n] = (int64_t)next; C_data[out + n] = sum; }
            }
            ++n;
        }
        if (!NUMERIC && active) row_nnz[row] = n;
        if (NUMERIC && staged) {
            __syncwarp();
            constexpr int V = 16 / (int)sizeof(T);                    // values per 16 bytes
            // columns: two int64 per 16-byte store where the address allows; values likewise
            const int head_c = (int)(warp_out & 1);                  // entries before the first 16-byte boundary of C_indices
            if (lane < head_c && lane < warp_total) C_indices[warp_out + lane] = (int64_t)wcol[lane];
            for (int q = head_c + 2 * lane; q < warp_total; q += 64) {
                if (q + 1 < warp_total) {
                    longlong2 two;
                    two.x = (long long)wcol[q];
                    two.y = (long long)wcol[q + 1];
                    *reinterpret_cast<longlong2*>(C_indices + warp_out + q) = two;
                } else {
                    C_indices[warp_out + q] = (int64_t)wcol[q];
                }
            }
            const int head_v = (int)((V - (warp_out & (V - 1))) & (V - 1));
            if (lane < head_v && lane < warp_total) C_data[warp_out + lane] = wval[lane];
            for (int q = head_v + V * lane; q < warp_total; q += 32 * V) {
                if (q + V <= warp_total) {
                    alignas(16) T tmp[V];
#pragma unroll
                    for (int t = 0; t < V; ++t) tmp[t] = wval[q + t];
                    *reinterpret_cast<int4*>(C_data + warp_out + q) = *reinterpret_cast<const int4*>(tmp);
                } else {
                    for (int t = 0; q + t < warp_total; ++t) C_data[warp_out + q + t] = wval[q + t];
                }
            }
            __syncwarp();
        }
    }
}

// The kernel is bound by the chain of dependent loads behind every row (row list -> row pointers of A
// -> entries of A -> row pointers of B -> entries of B), not by arithmetic, so the chain is software-
// pipelined five rows deep: in every iteration a warp issues one load level for each of the five rows
// it has in flight and only then forms the row whose products arrived during the previous iteration.
constexpr int kWarpRowsCtasPerSm = 5;      // 48 registers per thread: five 256-thread CTAs fit an SM

template <typename T, typename I, bool NUMERIC>
__global__ void __launch_bounds__(256, kWarpRowsCtasPerSm)
spgemm_warp_rows_kernel(const int32_t* __restrict__ list, const unsigned long long* __restrict__ count_ptr,
                        const T* __restrict__ A_data, const I* __restrict__ A_indices, const I* __restrict__ A_indptr,
                        const T* __restrict__ B_data, const I* __restrict__ B_indices, const I* __restrict__ B_indptr,
                        int32_t* __restrict__ row_nnz, const int64_t* __restrict__ C_indptr,
                        int64_t* __restrict__ C_indices, T* __restrict__ C_data) {
    constexpr unsigned kAll = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int64_t count = (int64_t)*count_ptr;
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const int64_t first_idx = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    // stage registers; a row of -1 marks an empty pipeline slot (warp-uniform)
    int64_t row1 = -1;                                            // 1: row number
    int64_t row2 = -1, a2 = 0; int na2 = 0;                       // 2: its range in A
    int64_t row3 = -1, a3 = 0; int na3 = 0; int64_t j3 = 0;       // 3: lane e < na: the row of B that entry e selects
    int64_t row4 = -1, a4 = 0; int na4 = 0; I bb4 = 0; int len4 = 0;   // 4: lane e < na: that row's range in B
    int64_t row5 = -1, cbeg5 = 0; uint32_t c5 = kEmptyKey; T v5 = (T)0; bool valid5 = false;   // 5: lane p: product p
    for (int64_t idx = first_idx; idx < count + 5 * nwarps; idx += nwarps) {
        // ---- level 5 for the row in slot 4: place the products on the lanes and request them ----
        int64_t n_row5 = row4, n_cbeg5 = 0;
        uint32_t n_c5 = kEmptyKey;
        T n_v5 = (T)0;
        bool n_valid5 = false;
        if (row4 >= 0) {
            // products of entry e occupy lanes [incl_e - len_e, incl_e)
            int incl = len4;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(kAll, incl, o);
                if (lane >= o) incl += t;
            }
            const int np = __shfl_sync(kAll, incl, 31);
            n_valid5 = lane < np;
            // the entry of A that product `lane` belongs to = the number of entries whose products all come
            // before it.  When no selected row of B is empty the ends of the runs are distinct, so a bit mask
            // of them answers that with one population count; otherwise they are compared one by one.
            int e = 0;
            const bool in_row = lane < na4;
            if (__all_sync(kAll, !in_row || len4 > 0)) {
                const unsigned ends = __reduce_or_sync(kAll, (in_row && incl < 32) ? (1u << incl) : 0u);
                e = __popc(ends & (0xffffffffu >> (31 - lane)));
            } else {
                for (int q = 0; q < na4; ++q) e += (__shfl_sync(kAll, incl, q) <= lane);
            }
            if (!n_valid5) e = 0;
            const int first = __shfl_sync(kAll, incl - len4, e);
            const I b0 = __shfl_sync(kAll, bb4, e);
            if (n_valid5) {
                const int64_t b = (int64_t)b0 + (lane - first);
                n_c5 = (uint32_t)B_indices[b];
                if (NUMERIC) n_v5 = mul_rn(A_data[a4 + e], B_data[b]);
            }
            if (NUMERIC) n_cbeg5 = C_indptr[row4];
        }
        // ---- level 4 for the row in slot 3, level 3 for slot 2, level 2 for slot 1, level 1 for a new row ----
        I n_bb4 = 0;
        int n_len4 = 0;
        if (row3 >= 0 && lane < na3) {
            n_bb4 = B_indptr[j3];
            n_len4 = (int)((int64_t)B_indptr[j3 + 1] - (int64_t)n_bb4);
        }
        int64_t n_j3 = 0;
        if (row2 >= 0 && lane < na2) n_j3 = (int64_t)A_indices[a2 + lane];
        int64_t n_a2 = 0;
        int n_na2 = 0;
        if (row1 >= 0) {
            n_a2 = (int64_t)A_indptr[row1];
            n_na2 = (int)((int64_t)A_indptr[row1 + 1] - n_a2);
        }
        const int64_t n_row1 = idx < count ? (int64_t)list[idx] : -1;

        // ---- the row whose products were requested during the previous iteration ----
        if (row5 >= 0) {
            const unsigned group = __match_any_sync(kAll, c5);
            const bool leader = valid5 && lane == __ffs(group) - 1;
            const unsigned leaders = __ballot_sync(kAll, leader);
            if (!NUMERIC) {
                if (lane == 0) row_nnz[row5] = __popc(leaders);
            } else {
                int rank = 0;                          // position in the sorted row: leaders with a smaller column
                for (unsigned rem = leaders; rem; rem &= rem - 1) rank += __shfl_sync(kAll, c5, __ffs(rem) - 1) < c5;
                // the group's products in lane order = the reference's order of additions (0 + first + ...)
                const int longest = __reduce_max_sync(kAll, valid5 ? __popc(group) : 0);
                T sum = add_rn((T)0, v5);
                if (longest > 1) {
                    sum = (T)0;
                    unsigned rem = group;
                    for (int it = 0; it < longest; ++it) {
                        const T t = __shfl_sync(kAll, v5, rem ? __ffs(rem) - 1 : lane);
                        if (rem) { sum = add_rn(sum, t); rem &= rem - 1; }
                    }
                }
                if (leader) {
                    C_indices[cbeg5 + rank] = (int64_t)c5;
                    C_data[cbeg5 + rank] = sum;
                }
            }
        }
        // ---- advance the pipeline ----
        row5 = n_row5; cbeg5 = n_cbeg5; c5 = n_c5; v5 = n_v5; valid5 = n_valid5;
        row4 = row3; a4 = a3; na4 = na3; bb4 = n_bb4; len4 = n_len4;
        row3 = row2; a3 = a2; na3 = na2; j3 = n_j3;
        row2 = row1; a2 = n_a2; na2 = n_na2;
        row1 = n_row1;
    }
}

// ---------------------------------------------------------------------------------------------
// Team helpers
// ---------------------------------------------------------------------------------------------
template <int TEAM>
__device__ __forceinline__ void team_sync() {
    if (TEAM >= 256) __syncthreads(); else __syncwarp();
}

template <int TEAM>
__device__ __forceinline__ int team_sum(int v, int* scratch) {
    if (TEAM <= 32) {
#pragma unroll
        for (int o = TEAM / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        return v;
    } else {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
        __syncthreads();
        int t = 0;
        for (int w = 0; w < TEAM / 32; ++w) t += scratch[w];
        __syncthreads();
        return t;
    }
}

// Bitonic sort of the whole table by key (ascending, empty slots last), values carried along.
template <typename T, int TEAM, bool WITH_VALUES>
__device__ __forceinline__ void team_sort(uint32_t* keys, T* vals, int64_t table, int t) {
    for (int64_t k = 2; k <= table; k <<= 1) {
        for (int64_t j = k >> 1; j > 0; j >>= 1) {
            for (int64_t p = t; p < (table >> 1); p += TEAM) {
                const int64_t i = ((p & ~(j - 1)) << 1) | (p & (j - 1));
                const int64_t q = i | j;
                const uint32_t a = keys[i], b = keys[q];
                const bool up = (i & k) == 0;
                if ((a > b) == up) {
                    keys[i] = b; keys[q] = a;
                    if (WITH_VALUES) { const T va = vals[i]; vals[i] = vals[q]; vals[q] = va; }
                }
            }
            team_sync<TEAM>();
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Symbolic: distinct columns per row of C.  SUB lanes share one entry of A and stride over the
// matching row of B; TEAM/SUB entries of A are in flight per team.
// ---------------------------------------------------------------------------------------------
template <typename I, int TEAM, int SUB, int TLOG, bool SPILL>
__global__ void __launch_bounds__(256)
spgemm_symbolic_kernel(const int32_t* __restrict__ list, const unsigned long long* __restrict__ count_ptr,
                       const I* __restrict__ A_indices, const I* __restrict__ A_indptr,
                       const I* __restrict__ B_indices, const I* __restrict__ B_indptr,
                       const int32_t* __restrict__ size_in, const int64_t* __restrict__ spill_off,
                       uint32_t* __restrict__ spill, int64_t spill_slots, unsigned long long* __restrict__ header,
                       int32_t* __restrict__ row_nnz) {
    constexpr int TEAMS = 256 / TEAM;
    constexpr int TABLE = SPILL ? 1 : (1 << TLOG);
    __shared__ uint32_t s_keys[TEAMS * TABLE];
    __shared__ int s_red[8];
    const int team = threadIdx.x / TEAM, t = threadIdx.x % TEAM;
    const int64_t count = (int64_t)*count_ptr;
    for (int64_t base = (int64_t)blockIdx.x * TEAMS; base < count; base += (int64_t)gridDim.x * TEAMS) {
        const int64_t idx = base + team;
        const bool active = idx < count;
        const int64_t row = active ? (int64_t)list[idx] : 0;
        uint32_t* keys = s_keys + team * TABLE;
        int64_t table = TABLE;
        bool usable = true;
        if (SPILL) {
            table = spill_table_size(size_in[row]);
            const int64_t off = spill_off[idx];
            usable = off + table <= spill_slots;
            keys = spill + off;
            if (!usable && t == 0) atomicExch(header + kHdrError, 1ull);
        }
        int shift = 32;
        for (int64_t s = table; s > 1; s >>= 1) --shift;
        const uint32_t mask = (uint32_t)(table - 1);
        if (usable) for (int64_t s = t; s < table; s += TEAM) keys[s] = kEmptyKey;
        team_sync<TEAM>();
        if (active && usable) {
            const int64_t a_end = (int64_t)A_indptr[row + 1];
            for (int64_t a = (int64_t)A_indptr[row] + t / SUB; a < a_end; a += TEAM / SUB) {
                const int64_t j = (int64_t)A_indices[a];
                const int64_t b_end = (int64_t)B_indptr[j + 1];
                for (int64_t b = (int64_t)B_indptr[j] + t % SUB; b < b_end; b += SUB)
                    table_insert(keys, mask, shift, (uint32_t)B_indices[b]);
            }
        }
        team_sync<TEAM>();
        int cnt = 0;
        if (usable) for (int64_t s = t; s < table; s += TEAM) cnt += keys[s] != kEmptyKey;
        cnt = team_sum<TEAM>(cnt, s_red);
        if (active && t == 0) row_nnz[row] = cnt;
        team_sync<TEAM>();
    }
}

// ---------------------------------------------------------------------------------------------
// Numeric: insert (column, product) pairs, sort the table, write the row.
// ---------------------------------------------------------------------------------------------
template <typename T, typename I, int TEAM, int SUB, int TLOG, bool SPILL>
__global__ void __launch_bounds__(256)
spgemm_numeric_kernel(const int32_t* __restrict__ list, const unsigned long long* __restrict__ count_ptr,
                      const T* __restrict__ A_data, const I* __restrict__ A_indices, const I* __restrict__ A_indptr,
                      const T* __restrict__ B_data, const I* __restrict__ B_indices, const I* __restrict__ B_indptr,
                      const int32_t* __restrict__ size_in, const int64_t* __restrict__ spill_off,
                      uint32_t* __restrict__ spill_keys, T* __restrict__ spill_vals, int64_t spill_slots,
                      unsigned long long* __restrict__ header,
                      const int64_t* __restrict__ C_indptr, int64_t* __restrict__ C_indices, T* __restrict__ C_data) {
    constexpr int TEAMS = 256 / TEAM;
    constexpr int TABLE = SPILL ? 1 : (1 << TLOG);
    __shared__ uint32_t s_keys[TEAMS * TABLE];
    __shared__ T s_vals[TEAMS * TABLE];
    constexpr int kListTeams = (!SPILL && TABLE <= 64) ? TEAMS : 1;   // dense lists only exist for tiny tables
    __shared__ uint32_t s_list[kListTeams * 32];
    __shared__ unsigned char s_slot[kListTeams * 32];
    __shared__ int s_cnt[kListTeams];
    const int team = threadIdx.x / TEAM, t = threadIdx.x % TEAM;
    const int64_t count = (int64_t)*count_ptr;
    for (int64_t base = (int64_t)blockIdx.x * TEAMS; base < count; base += (int64_t)gridDim.x * TEAMS) {
        const int64_t idx = base + team;
        const bool active = idx < count;
        const int64_t row = active ? (int64_t)list[idx] : 0;
        uint32_t* keys = s_keys + team * TABLE;
        T* vals = s_vals + team * TABLE;
        int64_t table = TABLE;
        bool usable = true;
        if (SPILL) {
            table = spill_table_size(size_in[row]);
            const int64_t off = spill_off[idx];
            usable = off + table <= spill_slots;
            keys = spill_keys + off;
            vals = spill_vals + off;
            if (!usable && t == 0) atomicExch(header + kHdrError, 1ull);
        }
        int shift = 32;
        for (int64_t s = table; s > 1; s >>= 1) --shift;
        const uint32_t mask = (uint32_t)(table - 1);
        if (usable) for (int64_t s = t; s < table; s += TEAM) { keys[s] = kEmptyKey; vals[s] = (T)0; }
        team_sync<TEAM>();
        if (active && usable) {
            const int64_t a_end = (int64_t)A_indptr[row + 1];
            for (int64_t a = (int64_t)A_indptr[row] + t / SUB; a < a_end; a += TEAM / SUB) {
                const int64_t j = (int64_t)A_indices[a];
                const T av = A_data[a];
                const int64_t b_end = (int64_t)B_indptr[j + 1];
                for (int64_t b = (int64_t)B_indptr[j] + t % SUB; b < b_end; b += SUB) {
                    const uint32_t slot = table_insert(keys, mask, shift, (uint32_t)B_indices[b]);
                    atomicAdd(vals + slot, mul_rn(av, B_data[b]));
                }
            }
        }
        team_sync<TEAM>();
        if (!SPILL && TABLE <= 64) {
            // tiny tables: gather the occupied slots into a dense list (any order), then the position
            // of a column in the sorted row is the number of smaller columns in that list; no sort,
            // and the quadratic part runs over the row's nnz (<= 32) instead of the table size
            if (t == 0) s_cnt[team] = 0;
            team_sync<TEAM>();
            for (int sl = t; sl < TABLE; sl += TEAM) {
                const uint32_t key = keys[sl];
                if (key != kEmptyKey) {
                    const int pos = atomicAdd(&s_cnt[team], 1);
                    s_list[team * 32 + pos] = key;
                    s_slot[team * 32 + pos] = (unsigned char)sl;
                }
            }
            team_sync<TEAM>();
            if (active) {
                const int64_t o0 = C_indptr[row];
                const int n = s_cnt[team];
                const uint32_t* lst = s_list + team * 32;
                for (int e = t; e < n; e += TEAM) {
                    const uint32_t key = lst[e];
                    int rank = 0;
                    for (int q = 0; q < n; ++q) rank += lst[q] < key;
                    C_indices[o0 + rank] = (int64_t)key;
                    C_data[o0 + rank] = vals[s_slot[team * 32 + e]];
                }
            }
        } else {
            if (usable) team_sort<T, TEAM, true>(keys, vals, table, t);
            if (active && usable) {
                const int64_t o0 = C_indptr[row], n = C_indptr[row + 1] - o0;
                for (int64_t q = t; q < n; q += TEAM) {
                    C_indices[o0 + q] = (int64_t)keys[q];
                    C_data[o0 + q] = vals[q];
                }
            }
        }
        team_sync<TEAM>();
    }
}

// ---------------------------------------------------------------------------------------------
// Backward kernels
// ---------------------------------------------------------------------------------------------
template <typename I>
__device__ __forceinline__ int64_t row_of_position(const I* __restrict__ indptr, int64_t rows, int64_t k) {
    int64_t lo = 0, hi = rows;   // largest r with indptr[r] <= k
    while (hi - lo > 1) {
        const int64_t mid = (lo + hi) >> 1;
        if ((int64_t)indptr[mid] <= k) lo = mid; else hi = mid;
    }
    return lo;
}

// grad_A[(i,j)] = sum over c in row j of B (ascending) of grad_C[(i,c)] * B[(j,c)]
template <typename T, typename I>
__global__ void spgemm_grad_A_kernel(int64_t A_rows, int64_t A_nnz, const I* __restrict__ A_indices,
                                     const I* __restrict__ A_indptr, const T* __restrict__ B_data,
                                     const I* __restrict__ B_indices, const I* __restrict__ B_indptr,
                                     const T* __restrict__ grad_C, const int64_t* __restrict__ C_indices,
                                     const int64_t* __restrict__ C_indptr, T* __restrict__ grad_A) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < A_nnz; k += stride) {
        const int64_t i = row_of_position(A_indptr, A_rows, k);
        const int64_t j = (int64_t)A_indices[k];
        int64_t ci = C_indptr[i];
        const int64_t ce = C_indptr[i + 1];
        int64_t bi = (int64_t)B_indptr[j];
        const int64_t be = (int64_t)B_indptr[j + 1];
        T s = 0;
        while (ci < ce && bi < be) {
            const int64_t cc = C_indices[ci], bc = (int64_t)B_indices[bi];
            if (cc < bc) ++ci;
            else if (cc > bc) ++bi;
            else { s = add_rn(s, mul_rn(grad_C[ci], B_data[bi])); ++ci; ++bi; }
        }
        grad_A[k] = s;
    }
}

// grad_B[(j,c)] = sum over i in column j of A (ascending) of A[(i,j)] * grad_C[(i,c)]
template <typename T, typename I>
__global__ void spgemm_grad_B_kernel(int64_t B_rows, int64_t B_nnz, const I* __restrict__ B_indices,
                                     const I* __restrict__ B_indptr, const T* __restrict__ A_data,
                                     const I* __restrict__ At_indptr, const I* __restrict__ At_indices,
                                     const I* __restrict__ At_perm, const T* __restrict__ grad_C,
                                     const int64_t* __restrict__ C_indices, const int64_t* __restrict__ C_indptr,
                                     T* __restrict__ grad_B) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < B_nnz; q += stride) {
        const int64_t j = row_of_position(B_indptr, B_rows, q);
        const int64_t c = (int64_t)B_indices[q];
        T s = 0;
        for (int64_t a = (int64_t)At_indptr[j]; a < (int64_t)At_indptr[j + 1]; ++a) {
            const int64_t i = (int64_t)At_indices[a];
            int64_t lo = C_indptr[i], hi = C_indptr[i + 1] - 1;
            while (lo <= hi) {
                const int64_t mid = (lo + hi) >> 1;
                const int64_t cc = C_indices[mid];
                if (cc < c) lo = mid + 1;
                else if (cc > c) hi = mid - 1;
                else { s = add_rn(s, mul_rn(A_data[(int64_t)At_perm[a]], grad_C[mid])); break; }
            }
        }
        grad_B[q] = s;
    }
}

// ---------------------------------------------------------------------------------------------
// Workspace layout
// ---------------------------------------------------------------------------------------------
struct SpgemmWorkspace {
    unsigned long long* header;
    int32_t* size;       // products per row, later nnz per row
    int32_t* row_nnz;
    int32_t* lists;      // kBins x rows
    int64_t* spill_off;  // rows
    unsigned char* kind; // rows
    char* scan;
    size_t scan_bytes;
    bool ok;
};

static size_t spgemm_workspace_bytes(int64_t rows) {
    const size_t r = (size_t)(rows > 0 ? rows : 1);
    return Workspace::pad(kHeaderWords * sizeof(int64_t)) + 2 * Workspace::pad(r * sizeof(int32_t)) +
           Workspace::pad(kBins * r * sizeof(int32_t)) + Workspace::pad(r * sizeof(int64_t)) + Workspace::pad(r) +
           Workspace::pad(scan_scratch_bytes(rows));
}

static SpgemmWorkspace carve(int64_t rows, void* workspace, size_t bytes) {
    const size_t r = (size_t)(rows > 0 ? rows : 1);
    Workspace ws(workspace, bytes);
    SpgemmWorkspace w;
    w.header = ws.take<unsigned long long>(kHeaderWords);
    w.size = ws.take<int32_t>(r);
    w.row_nnz = ws.take<int32_t>(r);
    w.lists = ws.take<int32_t>(kBins * r);
    w.spill_off = ws.take<int64_t>(r);
    w.kind = ws.take<unsigned char>(r);
    w.scan_bytes = scan_scratch_bytes(rows);
    w.scan = ws.take<char>(w.scan_bytes);
    w.ok = ws.ok();
    return w;
}

static inline unsigned persistent_grid(int ctas_per_sm = 8) { return (unsigned)(kSMs * ctas_per_sm); }

static inline unsigned flat_grid(int64_t n) {
    const int64_t want = ceil_div(n > 0 ? n : 1, (int64_t)256);
    return (unsigned)(want > (int64_t)kSMs * 32 ? (int64_t)kSMs * 32 : want);
}

template <typename I>
int spgemm_plan(int64_t A_rows, const I* A_indices, const I* A_indptr, const I* B_indptr, bool b_sorted,
                void* workspace, size_t bytes, cudaStream_t st) {
    SpgemmWorkspace w = carve(A_rows, workspace, bytes);
    if (!w.ok) return NB200_ERR_WORKSPACE;
    if (cudaMemsetAsync(w.header, 0, kHeaderWords * sizeof(int64_t), st) != cudaSuccess) return NB200_ERR_CUDA;
    if (A_rows == 0) return NB200_OK;
    spgemm_products_kernel<I><<<flat_grid(A_rows), 256, 0, st>>>(A_rows, A_indices, A_indptr, B_indptr, w.size, w.kind, b_sorted, w.header);
    spgemm_classify_kernel<<<flat_grid(A_rows), 256, 0, st>>>(A_rows, w.size, w.kind, false, w.lists, w.spill_off, w.header);
    return launch_status();
}

template <typename I>
int spgemm_symbolic(int64_t A_rows, const I* A_indices, const I* A_indptr, const I* B_indices, const I* B_indptr,
                    void* workspace, size_t bytes, uint32_t* spill, int64_t spill_slots, int64_t* C_indptr,
                    cudaStream_t st) {
    SpgemmWorkspace w = carve(A_rows, workspace, bytes);
    if (!w.ok) return NB200_ERR_WORKSPACE;
    if (A_rows > 0) {
        const unsigned g = persistent_grid();
        spgemm_thread_rows_kernel<double, I, false><<<persistent_grid(5), 256, 0, st>>>(
            w.lists, w.header + 0, nullptr, A_indices, A_indptr, nullptr, B_indices, B_indptr, w.row_nnz, nullptr, nullptr, nullptr);
        spgemm_warp_rows_kernel<double, I, false><<<persistent_grid(kWarpRowsCtasPerSm), 256, 0, st>>>(
            w.lists + A_rows, w.header + 1, nullptr, A_indices, A_indptr, nullptr, B_indices, B_indptr, w.row_nnz, nullptr, nullptr, nullptr);
#define NB200_SYM(TEAM, SUB, TLOG, SPILL, BIN)                                                              \
        spgemm_symbolic_kernel<I, TEAM, SUB, TLOG, SPILL><<<g, 256, 0, st>>>(                                 \
            w.lists + (int64_t)(BIN) * A_rows, w.header + (BIN), A_indices, A_indptr, B_indices, B_indptr,  \
            w.size, w.spill_off, spill, spill_slots, w.header, w.row_nnz)
        NB200_SYM(8, 1, 6, false, 2);
        NB200_SYM(32, 4, 9, false, 3);
        NB200_SYM(256, 32, 13, false, 4);
        NB200_SYM(256, 32, 0, true, 5);
#undef NB200_SYM
    }
    int rc = exclusive_scan_i32_to_i64(A_rows, w.row_nnz, C_indptr, w.scan, w.scan_bytes, st);
    if (rc != NB200_OK) return rc;
    if (A_rows > 0) {
        // numeric classification by exact row size; nnz(C) goes to header[13]
        spgemm_classify_kernel<<<flat_grid(A_rows), 256, 0, st>>>(A_rows, w.row_nnz, w.kind, true, w.lists, w.spill_off, w.header);
    }
    if (cudaMemcpyAsync(w.header + kHdrNnz, C_indptr + A_rows, sizeof(int64_t), cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return NB200_ERR_CUDA;
    return launch_status();
}

template <typename T, typename I>
int spgemm_numeric(int64_t A_rows, const T* A_data, const I* A_indices, const I* A_indptr,
                   const T* B_data, const I* B_indices, const I* B_indptr, void* workspace, size_t bytes,
                   void* spill, int64_t spill_slots, const int64_t* C_indptr, int64_t* C_indices, T* C_data,
                   cudaStream_t st) {
    SpgemmWorkspace w = carve(A_rows, workspace, bytes);
    if (!w.ok) return NB200_ERR_WORKSPACE;
    if (A_rows == 0) return NB200_OK;
    // spill area: values first (8-byte aligned), keys after
    T* spill_vals = static_cast<T*>(spill);
    uint32_t* spill_keys = reinterpret_cast<uint32_t*>(spill_vals + (spill_slots > 0 ? spill_slots : 0));
    const unsigned g = persistent_grid();
    spgemm_thread_rows_kernel<T, I, true><<<persistent_grid(4), 256, 0, st>>>(
        w.lists, w.header + kHdrNumBins, A_data, A_indices, A_indptr, B_data, B_indices, B_indptr, nullptr, C_indptr, C_indices, C_data);
    spgemm_warp_rows_kernel<T, I, true><<<persistent_grid(kWarpRowsCtasPerSm), 256, 0, st>>>(
        w.lists + A_rows, w.header + kHdrNumBins + 1, A_data, A_indices, A_indptr, B_data, B_indices, B_indptr, nullptr, C_indptr, C_indices, C_data);
#define NB200_NUM(TEAM, SUB, TLOG, SPILL, BIN)                                                                   \
    spgemm_numeric_kernel<T, I, TEAM, SUB, TLOG, SPILL><<<g, 256, 0, st>>>(                                       \
        w.lists + (int64_t)(BIN) * A_rows, w.header + kHdrNumBins + (BIN), A_data, A_indices, A_indptr, B_data, B_indices, \
        B_indptr, w.row_nnz, w.spill_off, spill_keys, spill_vals, spill_slots, w.header, C_indptr, C_indices, C_data)
    NB200_NUM(8, 1, 6, false, 2);
    NB200_NUM(32, 4, 9, false, 3);
    NB200_NUM(256, 32, 12, false, 4);
    NB200_NUM(256, 32, 0, true, 5);
#undef NB200_NUM
    return launch_status();
}

}  // namespace nb200

using namespace nb200;

extern "C" size_t nb200_spgemm_workspace_bytes(int64_t A_rows) { return spgemm_workspace_bytes(A_rows); }

extern "C" int nb200_spgemm_plan(int64_t A_rows, int64_t A_cols, int64_t A_nnz,
                                 const void* A_indices, const void* A_indptr, const void* B_indptr, int B_rows_sorted,
                                 int itype, void* workspace, size_t workspace_bytes, nb200_stream stream) {
    (void)A_cols;
    if (A_rows < 0 || A_nnz < 0 || !workspace) return NB200_ERR_BAD_ARG;
    if (A_rows >= 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    if (A_rows > 0 && (!A_indptr || !B_indptr || (A_nnz > 0 && !A_indices))) return NB200_ERR_BAD_ARG;
    return NB200_DISPATCH_I(itype,
        (spgemm_plan<I>(A_rows, (const I*)A_indices, (const I*)A_indptr, (const I*)B_indptr, B_rows_sorted != 0, workspace,
                        workspace_bytes, as_stream(stream))));
}

extern "C" int nb200_spgemm_symbolic(int64_t A_rows, int64_t A_cols, int64_t B_cols,
                                     const void* A_indices, const void* A_indptr,
                                     const void* B_indices, const void* B_indptr, int itype,
                                     void* workspace, size_t workspace_bytes, void* spill, int64_t spill_slots,
                                     int64_t* C_indptr, nb200_stream stream) {
    (void)A_cols;
    if (A_rows < 0 || B_cols < 0 || !workspace || !C_indptr || spill_slots < 0) return NB200_ERR_BAD_ARG;
    if (B_cols >= 0x7fffffffLL) return NB200_ERR_TOO_LARGE;
    return NB200_DISPATCH_I(itype,
        (spgemm_symbolic<I>(A_rows, (const I*)A_indices, (const I*)A_indptr, (const I*)B_indices, (const I*)B_indptr,
                            workspace, workspace_bytes, (uint32_t*)spill, spill_slots, C_indptr, as_stream(stream))));
}

extern "C" int nb200_spgemm_numeric(int64_t A_rows, int64_t A_cols, int64_t B_cols,
                                    const void* A_data, const void* A_indices, const void* A_indptr,
                                    const void* B_data, const void* B_indices, const void* B_indptr,
                                    int dtype, int itype, void* workspace, size_t workspace_bytes,
                                    void* spill, int64_t spill_slots,
                                    const int64_t* C_indptr, int64_t* C_indices, void* C_data, nb200_stream stream) {
    (void)A_cols; (void)B_cols;
    if (A_rows < 0 || !workspace || !C_indptr || spill_slots < 0) return NB200_ERR_BAD_ARG;
    return NB200_DISPATCH(dtype, itype,
        (spgemm_numeric<T, I>(A_rows, (const T*)A_data, (const I*)A_indices, (const I*)A_indptr,
                              (const T*)B_data, (const I*)B_indices, (const I*)B_indptr, workspace, workspace_bytes,
                              spill, spill_slots, C_indptr, C_indices, (T*)C_data, as_stream(stream))));
}

extern "C" int nb200_spgemm_backward(int64_t A_rows, int64_t A_cols, int64_t A_nnz,
                                     const void* A_data, const void* A_indices, const void* A_indptr,
                                     const void* At_indptr, const void* At_indices, const void* At_perm,
                                     int64_t B_rows, int64_t B_cols, int64_t B_nnz,
                                     const void* B_data, const void* B_indices, const void* B_indptr,
                                     const void* grad_C, const int64_t* C_indices, const int64_t* C_indptr,
                                     void* grad_A, void* grad_B, int dtype, int itype, nb200_stream stream) {
    (void)A_cols; (void)B_cols;
    if (A_rows < 0 || A_nnz < 0 || B_rows < 0 || B_nnz < 0) return NB200_ERR_BAD_ARG;
    if ((A_nnz > 0 && (!A_data || !A_indices || !A_indptr || !grad_A || !At_indptr || !At_indices || !At_perm)) ||
        (B_nnz > 0 && (!B_data || !B_indices || !B_indptr || !grad_B)) || !C_indptr)
        return NB200_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    return NB200_DISPATCH(dtype, itype, ([&]() -> int {
        if (A_nnz > 0)
            spgemm_grad_A_kernel<T, I><<<flat_grid(A_nnz), 256, 0, st>>>(
                A_rows, A_nnz, (const I*)A_indices, (const I*)A_indptr, (const T*)B_data, (const I*)B_indices,
                (const I*)B_indptr, (const T*)grad_C, C_indices, C_indptr, (T*)grad_A);
        if (B_nnz > 0)
            spgemm_grad_B_kernel<T, I><<<flat_grid(B_nnz), 256, 0, st>>>(
                B_rows, B_nnz, (const I*)B_indices, (const I*)B_indptr, (const T*)A_data, (const I*)At_indptr,
                (const I*)At_indices, (const I*)At_perm, (const T*)grad_C, C_indices, C_indptr, (T*)grad_B);
        return launch_status();
    }()));
}
