// Persistent, TMA-pipelined SpMV kernels for matrices whose rows are short and regular (the
// stencil case): every block of `block_rows` consecutive rows holds at most kPipeTile nonzeros.
//
// One CTA per SM slot walks its share of the row blocks.  A producer warp runs ahead: for each
// block it reads the block's nonzero range from indptr and issues bulk asynchronous copies
// (cp.async.bulk, completion counted on an mbarrier) of the block's index and value streams into
// one of kPipeStages shared-memory stages.  Eight consumer warps wait for a stage; then every
// consumer thread owns one row of the block: it reads the row's entries from the stage, gathers x
// through L1/L2 and accumulates in storage order (unfused multiply and add: bit-identical to a
// sequential CPU loop).  Thread-per-row gathers are what makes banded matrices cheap: lanes of a
// warp read x at consecutive addresses for each entry position, a few cache lines per
// instruction instead of one per lane.  The DRAM stream never stops while a block is being
// consumed, which is what the register-staged kernel in spmv.cu cannot do.
//
// Three modes share the pipeline:
//   kForward       stage = values + column indices            y[r]      = sum_k data[k] x[col[k]]
//   kForwardPerm   stage = column indices + permutation        y[r]      = sum_k data[perm[k]] x[col[k]]
//   kGradA         stage = column indices                      grad_A[k] = g[row(k)] x[col[k]]
//   kBackwardSym   stage = column indices + permutation        both gradients in one pass, for patterns that
//                                                              equal their transpose (stencils, undirected graphs)
//   kBackwardSymVal stage = values + column indices            the same pass for a matrix whose VALUES equal their
//                                                              transpose too (A[i,c] == A[c,i] bit for bit, which the
//                                                              caller has checked): the transposed value of an entry is
//                                                              the entry's own value, so no permutation is read and
//                                                              no value is gathered
// The fused backward gathers three operands per entry (x, g and the transposed value).  Its row threads
// fetch them with per-thread asynchronous copies (cp.async) into shared-memory slots instead of into
// registers, eight entries at a time, so that a short row has all of its gathers in flight at once.
//
// Every wait on an mbarrier is a try_wait loop bounded by a cycle budget; if it runs out the CTA records
// NB200_ERR_WAIT_BUDGET in the status word (when one is given) and leaves its block loop.
#include "spmv_pipe.cuh"
#include <atomic>

namespace nb200 {

constexpr int kPipeTile = kSpmvPipeTile;   // nonzeros per stage
constexpr int kPipeConsumers = kSpmvPipeRows;   // consumer threads (8 warps); one more warp produces
constexpr int kPipeThreads = kPipeConsumers + 32;
constexpr long long kPipeWaitCycles = 4000000000LL;   // wait budget in SM cycles (about two seconds)
constexpr int kMaxDevices = 64;        // devices one process can address

enum PipeMode { kForward = 0, kForwardPerm = 1, kGradA = 2, kBackwardSym = 3, kBackwardSymVal = 4 };
__host__ __device__ constexpr bool is_backward_sym(int mode) { return mode == kBackwardSym || mode == kBackwardSymVal; }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}"
                 :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false if kPipeWaitCycles SM cycles passed first.
__device__ __forceinline__ bool mbar_try(uint32_t addr, unsigned parity) {
    unsigned done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
    const uint32_t addr = smem_u32(bar);
    if (mbar_try(addr, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try(addr, parity))
        if (clock64() - t0 > kPipeWaitCycles) return false;
    return true;
}
// Bulk copy global -> shared, completion signalled on `bar`.  16-byte aligned, size % 16 == 0.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" :: "n"(kPipeConsumers) : "memory"); }

template <typename T, typename I>
struct PipeArgs {
    int64_t row0;        // first row handled by this launch (blocks are counted from here)
    int64_t rows, nnz, num_blocks;   // rows = one past the last row handled
    int block_rows;
    const T* data;       // values of A
    const I* indices;    // column of each staged entry
    const I* indptr;     // row pointers of the staged structure
    const I* perm;       // kForwardPerm: position in `data` of each staged entry
    const T* vec;        // gathered by column: x (forward, grad_A) or g (transposed pass)
    const T* rowvec;     // kGradA / kBackwardSym: g, one factor per row
    T* out;              // y [rows] or grad_A [nnz]
    T* out2;             // kBackwardSym: grad_x [rows]
    int32_t* status;     // may be null
};

// GATHER > 0 (kBackwardSym with direct grad_A stores only): a row thread fetches x_c, g_c and the
// transposed value of GATHER entries at a time with asynchronous copies into shared-memory slots of
// its own instead of into registers.  All gathers of a short row are then in flight at once and a
// block costs one memory round trip, where the register version needs one per CH entries.
template <typename T, typename I, int MODE, int S, bool DIRECT = false, int GATHER = 0, int WSTORE = 0>
struct PipeSmem {
    static constexpr bool has_a = MODE != kGradA;
    static constexpr bool a_is_perm = MODE == kForwardPerm || MODE == kBackwardSym;
    // grad_A is staged per block (!DIRECT), or per warp when the stage has no value slots to reuse
    static constexpr bool has_p = ((MODE == kGradA || is_backward_sym(MODE)) && !DIRECT) || (MODE == kBackwardSym && WSTORE != 0);
    static constexpr size_t a_bytes = has_a ? (a_is_perm ? sizeof(I) : sizeof(T)) * kPipeTile : 0;  // values | perm
    static constexpr size_t b_bytes = sizeof(I) * kPipeTile;                                           // indices
    static constexpr size_t p_bytes = has_p ? sizeof(T) * kPipeTile : 0;                               // grad_A staging
    static constexpr size_t stage_bytes = a_bytes + b_bytes + p_bytes;
    static constexpr size_t header_bytes = 128;
    // planes (g_c, transposed value unless it is staged, x_c) of one slot per (entry position, consumer thread)
    static constexpr int gather_planes = MODE == kBackwardSymVal ? 2 : 3;
    static constexpr size_t gather_bytes = gather_planes * sizeof(T) * GATHER * kPipeConsumers;
    static constexpr size_t total = header_bytes + stage_bytes * S + gather_bytes;
    static_assert(GATHER == 0 || (is_backward_sym(MODE) && DIRECT), "GATHER is a variant of the fused backward");
};

template <typename T> struct Pair;
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<double> { using type = double2; };

// 4- or 8-byte asynchronous copy global -> shared into a slot owned by the issuing thread
template <typename T>
__device__ __forceinline__ void async_copy_elem(T* dst, const T* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" :: "r"(smem_u32(dst)), "l"(src), "n"(sizeof(T)) : "memory");
}

template <typename T>
__device__ __forceinline__ void lds4(const T* p, T (&v)[4]);
template <>
__device__ __forceinline__ void lds4<float>(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void lds4<double>(const double* p, double (&v)[4]) {
    const double2 a = *reinterpret_cast<const double2*>(p), b = *reinterpret_cast<const double2*>(p + 2);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <>
__device__ __forceinline__ void lds4<int32_t>(const int32_t* p, int32_t (&v)[4]) {
    const int4 t = *reinterpret_cast<const int4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void lds4<int64_t>(const int64_t* p, int64_t (&v)[4]) {
    const longlong2 a = *reinterpret_cast<const longlong2*>(p), b = *reinterpret_cast<const longlong2*>(p + 2);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename T>
__device__ __forceinline__ void sts4(T* p, const T (&v)[4]);
template <>
__device__ __forceinline__ void sts4<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void sts4<double>(double* p, const double (&v)[4]) {
    *reinterpret_cast<double2*>(p) = make_double2(v[0], v[1]);
    *reinterpret_cast<double2*>(p + 2) = make_double2(v[2], v[3]);
}

// WSTORE (fused backward with direct stores): where a row thread puts its grad_A entries.
//   0  straight to global memory, one or two entries per store (a warp's store touches 32 sectors)
//   1  into shared memory -- the stage's value slots, which the thread has just consumed (kBackwardSymVal), or
//      a staging area of the stage (kBackwardSym); the warp's rows are contiguous in grad_A, so after a warp
//      barrier the lanes copy the warp's range out with 16-byte stores, fully coalesced
//   2  the same, but the copy-out is one bulk shared-to-global copy issued by one lane (TMA store)
template <typename T, typename I, int MODE, int S, int CH, int MINB, bool DIRECT, int GATHER, int WSTORE>
__global__ void __launch_bounds__(kPipeThreads, MINB)
spmv_pipe_kernel(const PipeArgs<T, I> a) {
    static_assert(WSTORE == 0 || (DIRECT && ((MODE == kBackwardSymVal && GATHER == 0) || (MODE == kBackwardSym && GATHER > 0))),
                  "per-warp staging of grad_A: in the consumed value slots, or in an area of its own");
    using L = PipeSmem<T, I, MODE, S, DIRECT, GATHER, WSTORE>;
    constexpr int kPipeStages = S;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kPipeStages;
    // iteration (plus one) in which a consumer warp gave up waiting; read after the consumers' barrier
    volatile int* const gave_up = reinterpret_cast<volatile int*>(smem + L::header_bytes - sizeof(int));
    static_assert(2 * S * sizeof(uint64_t) + sizeof(int) <= L::header_bytes, "barriers and the abort word share the header");
    auto stage_ptr = [&](int s) { return smem + L::header_bytes + (size_t)s * L::stage_bytes; };
    // per stage: [A: values or perm (absent for kGradA)] [B: indices] [P: grad_A staging (kGradA only)]
    auto stage_A = [&](int s) { return stage_ptr(s); };
    auto stage_B = [&](int s) { return stage_ptr(s) + L::a_bytes; };
    auto stage_P = [&](int s) { return stage_ptr(s) + L::a_bytes + L::b_bytes; };

    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int s = 0; s < kPipeStages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, kPipeConsumers / 32); }
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int64_t nnz_bulk_end = a.nnz & ~(int64_t)3;   // bulk copies never read past the arrays

    if (tid >= kPipeConsumers) {
        // ---------------------------------- producer warp ----------------------------------
        if (tid != kPipeConsumers) return;
        auto block_range = [&](int64_t blk, int64_t& begin_, int64_t& end_) {
            begin_ = 0; end_ = 0;
            if (blk < a.num_blocks) {
                const int64_t q0 = a.row0 + blk * a.block_rows, q1 = min(q0 + (int64_t)a.block_rows, a.rows);
                begin_ = (int64_t)a.indptr[q0];
                end_ = (int64_t)a.indptr[q1];
            }
        };
        int64_t it = 0, begin, end, begin_nxt, end_nxt;
        block_range(blockIdx.x, begin, end);
        for (int64_t b = blockIdx.x; b < a.num_blocks; b += gridDim.x, ++it, begin = begin_nxt, end = end_nxt) {
            const int s = (int)(it % kPipeStages);
            const unsigned ph = (unsigned)((it / kPipeStages) & 1);
            block_range(b + gridDim.x, begin_nxt, end_nxt);   // in flight while this block's copies are issued
            const int64_t base = begin & ~(int64_t)3;
            int64_t stop = min((end + 3) & ~(int64_t)3, nnz_bulk_end);
            int64_t count = stop > base ? stop - base : 0;
            if (count > kPipeTile) count = kPipeTile;
            if (!mbar_wait(empty + s, ph ^ 1u)) { if (a.status) atomicExch(a.status, (int)NB200_ERR_WAIT_BUDGET); return; }
            if (count == 0) { mbar_arrive(full + s); continue; }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            const unsigned bytes_b = (unsigned)(count * sizeof(I));
            if (MODE == kForward || MODE == kBackwardSymVal) {
                const unsigned bytes_a = (unsigned)(count * sizeof(T));
                mbar_arrive_expect_tx(full + s, bytes_a + bytes_b);
                bulk_load(stage_A(s), a.data + base, bytes_a, full + s);
                bulk_load(stage_B(s), a.indices + base, bytes_b, full + s);
            } else if (MODE == kForwardPerm || MODE == kBackwardSym) {
                mbar_arrive_expect_tx(full + s, 2 * bytes_b);
                bulk_load(stage_A(s), a.perm + base, bytes_b, full + s);
                bulk_load(stage_B(s), a.indices + base, bytes_b, full + s);
            } else {
                mbar_arrive_expect_tx(full + s, bytes_b);
                bulk_load(stage_B(s), a.indices + base, bytes_b, full + s);
            }
        }
        return;
    }

    // ------------------------------------ consumer warps ------------------------------------
    // Per block each thread needs the block's nonzero range (same for all threads) and, if it owns
    // a row of the block, that row's range (and g for kGradA).  They are fetched one block ahead so
    // that their latency is hidden behind the current block's work.
    struct BlockInfo { int64_t begin; int cnt, lo, hi; T g; };   // entries of the block; this thread's row, relative to begin
    auto fetch = [&](int64_t blk) {
        BlockInfo f{0, 0, 0, 0, (T)0};
        if (blk < a.num_blocks) {
            const int64_t r0 = a.row0 + blk * a.block_rows, r1 = min(r0 + (int64_t)a.block_rows, a.rows);
            f.begin = (int64_t)a.indptr[r0];
            f.cnt = (int)min((int64_t)a.indptr[r1] - f.begin, (int64_t)0x3fffffff);
            const int64_t r = r0 + tid;
            if (tid < a.block_rows && r < r1) {
                f.lo = (int)min((int64_t)a.indptr[r] - f.begin, (int64_t)0x3fffffff);
                f.hi = (int)min((int64_t)a.indptr[r + 1] - f.begin, (int64_t)0x3fffffff);
                if (MODE == kGradA || is_backward_sym(MODE)) f.g = a.rowvec[r];
            }
        }
        return f;
    };

    int64_t it = 0;
    BlockInfo cur = fetch(blockIdx.x);
    for (int64_t b = blockIdx.x; b < a.num_blocks; b += gridDim.x, ++it) {
        const int s = (int)(it % kPipeStages);
        const unsigned ph = (unsigned)((it / kPipeStages) & 1);
        const BlockInfo nxt = fetch(b + gridDim.x);

        const int64_t r0 = a.row0 + b * a.block_rows, r1 = min(r0 + (int64_t)a.block_rows, a.rows);
        const int64_t begin = cur.begin, end = cur.begin + cur.cnt;
        const int64_t base = begin & ~(int64_t)3;
        const int shift = (int)(begin - base);                       // stage offset of the block's first entry
        const int64_t bulk_stop = min(min((end + 3) & ~(int64_t)3, nnz_bulk_end), base + kPipeTile);
        const bool owns_row = tid < a.block_rows && r0 + tid < r1;
        const int staged_cnt = (int)max(bulk_stop - base, (int64_t)0);   // stage offsets below this hold data

        // The decision to give up is taken per warp (all lanes or none).  Kernels without a barrier among
        // the consumers let such a warp leave: the producer then runs out of its own budget on the stage
        // the warp never releases, and so do the other warps on their next wait.  Kernels that stage
        // grad_A meet at a barrier once per block; there the warp skips its work, still arrives, and
        // everybody leaves together after the barrier.
        constexpr bool kConsumersMeet = (MODE == kGradA || is_backward_sym(MODE)) && !DIRECT;
        const bool stage_ready = __all_sync(0xffffffffu, mbar_wait(full + s, ph));
        if (!stage_ready) {
            if ((tid & 31) == 0) {
                if (a.status) atomicExch(a.status, (int)NB200_ERR_WAIT_BUDGET);
                *gave_up = (int)(it & 0x3fffffff) + 1;
            }
            if (!kConsumersMeet) return;
        }
        const I* sidx = reinterpret_cast<const I*>(stage_B(s));
        const T* sval = reinterpret_cast<const T*>(stage_A(s));     // kForward
        const I* sperm = reinterpret_cast<const I*>(stage_A(s));    // kForwardPerm, kBackwardSym
        T* sout = reinterpret_cast<T*>(stage_P(s));                 // kGradA, kBackwardSym
        T* const outp = a.out + base;                                // entry with stage offset o is out[base + o]

        // ---- one thread per row: entries from the stage, x through L1/L2, storage order ----
        if (is_backward_sym(MODE) && GATHER > 0) {
            if (owns_row && stage_ready) {
                using T2 = typename Pair<T>::type;
                constexpr bool kStagedValues = MODE == kBackwardSymVal;
                constexpr int kPlane = GATHER * kPipeConsumers;
                T* const sg = reinterpret_cast<T*>(smem + L::header_bytes + (size_t)kPipeStages * L::stage_bytes) + tid;
                T* const sx = sg + kPlane;
                T* const sd = sx + kPlane;                               // unused when the values are staged
                const int o_lo = cur.lo + shift, o_hi = cur.hi + shift;
                const int o_staged = min(o_hi, staged_cnt);              // below o_hi only at the ragged end of the arrays
                const T gi = cur.g;
                T acc = 0;
                for (int o0 = o_lo; o0 < o_staged; o0 += GATHER) {
                    const int n = min(GATHER, o_staged - o0);
                    // (1) every gather of the chunk at once: x_c, g_c and A^T[i, c] = data[perm[k]]
                    for (int e = 0; e < n; ++e) {
                        const I c = sidx[o0 + e];
                        async_copy_elem(sx + e * kPipeConsumers, a.vec + c);
                        async_copy_elem(sg + e * kPipeConsumers, a.rowvec + c);
                        if (!kStagedValues) async_copy_elem(sd + e * kPipeConsumers, a.data + sperm[o0 + e]);
                    }
                    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
                    // (2) grad_A[k] = g_i x_c, staged for the warp's copy-out or stored two entries at a time
                    int e = 0;
                    if (WSTORE != 0) {
                        for (; e < n; ++e) sout[o0 + e] = mul_rn(gi, sx[e * kPipeConsumers]);
                    }
                    if (e < n && (o0 & 1)) { outp[o0] = mul_rn(gi, sx[0]); e = 1; }
                    for (; e + 2 <= n; e += 2) {
                        T2 w;
                        w.x = mul_rn(gi, sx[e * kPipeConsumers]);
                        w.y = mul_rn(gi, sx[(e + 1) * kPipeConsumers]);
                        *reinterpret_cast<T2*>(outp + o0 + e) = w;
                    }
                    if (e < n) outp[o0 + e] = mul_rn(gi, sx[e * kPipeConsumers]);
                    // (3) grad_x[i] += A^T[i, c] g_c in storage order
#pragma unroll
                    for (int j = 0; j < GATHER; ++j)
                        if (j < n) acc = add_rn(acc, mul_rn(sg[j * kPipeConsumers], kStagedValues ? sval[o0 + j] : sd[j * kPipeConsumers]));
                }
                for (int o = max(o_staged, o_lo); o < o_hi; ++o) {       // entries that were not staged: plain loads
                    const I c = a.indices[base + o];
                    outp[o] = mul_rn(gi, ldg(a.vec + c));
                    const T tv = kStagedValues ? a.data[base + o] : ldg(a.data + a.perm[base + o]);
                    acc = add_rn(acc, mul_rn(ldg(a.rowvec + c), tv));
                }
                a.out2[r0 + tid] = acc;
            }
        } else if (owns_row && stage_ready) {
            T acc = 0;
            const int o_lo = cur.lo + shift, o_hi = cur.hi + shift;
            const bool all_staged = o_hi <= staged_cnt;              // false only at the ragged end of the arrays
            for (int o0 = o_lo; o0 < o_hi; o0 += CH) {
                const int n = min(CH, o_hi - o0);
                I c[CH];
                T v[CH], xv[CH];
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    c[j] = 0; v[j] = 0;
                    if (j < n) {
                        const int o = o0 + j;
                        if (all_staged || o < staged_cnt) {
                            c[j] = sidx[o];
                            if (MODE == kForward || MODE == kBackwardSymVal) v[j] = sval[o];
                            if (MODE == kForwardPerm || MODE == kBackwardSym) v[j] = ldg(a.data + sperm[o]);
                        } else {
                            const int64_t k = base + o;
                            c[j] = a.indices[k];
                            if (MODE == kForward || MODE == kBackwardSymVal) v[j] = a.data[k];
                            if (MODE == kForwardPerm || MODE == kBackwardSym) v[j] = ldg(a.data + a.perm[k]);
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < CH; ++j) xv[j] = (j < n) ? ldg(a.vec + c[j]) : (T)0;
                if (is_backward_sym(MODE)) {
                    // the pattern equals its transpose: row i of A^T has the same columns, so one pass
                    // gives grad_A[k] = g_i x_c and grad_x[i] = sum_k A^T[i,c] g_c
                    T gv[CH];
#pragma unroll
                    for (int j = 0; j < CH; ++j) gv[j] = (j < n) ? ldg(a.rowvec + c[j]) : (T)0;
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        if (j < n) {
                            const int o = o0 + j;
                            const T val = mul_rn(cur.g, xv[j]);
                            if (WSTORE != 0 && o < staged_cnt) const_cast<T*>(sval)[o] = val;   // slot o was read into v[j] above
                            else if (!DIRECT && o < kPipeTile) sout[o] = val;
                            else outp[o] = val;
                            acc = add_rn(acc, mul_rn(gv[j], v[j]));
                        }
                    }
                } else if (MODE == kGradA) {
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        if (j < n) {
                            const int o = o0 + j;
                            const T val = mul_rn(cur.g, xv[j]);
                            if (o < kPipeTile) sout[o] = val; else outp[o] = val;
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < CH; ++j)
                        if (j < n) acc = add_rn(acc, mul_rn(v[j], xv[j]));
                }
            }
            if (MODE == kForward || MODE == kForwardPerm) a.out[r0 + tid] = acc;
            if (is_backward_sym(MODE)) a.out2[r0 + tid] = acc;
        }
        if (WSTORE != 0 && stage_ready) {
            // ---- the warp's grad_A entries leave the stage as whole lines ----
            constexpr int V = 16 / (int)sizeof(T);                       // entries per 16 bytes
            const int lane = tid & 31;
            const int lo_w = __reduce_min_sync(0xffffffffu, owns_row ? cur.lo + shift : 0x7fffffff);
            const int hi_w = __reduce_max_sync(0xffffffffu, owns_row ? min(cur.hi + shift, staged_cnt) : 0);
            T* const sstage = MODE == kBackwardSymVal ? const_cast<T*>(sval) : sout;
            if (WSTORE == 2) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (hi_w > lo_w) {
                const int lo_a = min((lo_w + V - 1) & ~(V - 1), hi_w);   // outp + o is 16-byte aligned when o % V == 0
                const int hi_a = max(hi_w & ~(V - 1), lo_a);
                if (lane < lo_a - lo_w) outp[lo_w + lane] = sstage[lo_w + lane];
                if (lane < hi_w - hi_a) outp[hi_a + lane] = sstage[hi_a + lane];
                if (WSTORE == 2) {
                    if (lane == 0 && hi_a > lo_a) {
                        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                     :: "l"(outp + lo_a), "r"(smem_u32(sstage + lo_a)), "r"((unsigned)((hi_a - lo_a) * sizeof(T))) : "memory");
                        asm volatile("cp.async.bulk.commit_group;\n\tcp.async.bulk.wait_group.read 0;" ::: "memory");
                    }
                } else {
                    for (int o = lo_a + V * lane; o < hi_a; o += 32 * V)
                        *reinterpret_cast<int4*>(outp + o) = *reinterpret_cast<const int4*>(sstage + o);
                }
            }
        }
        if ((MODE == kGradA || is_backward_sym(MODE)) && !DIRECT) {
            // ---- coalesced 128-bit stores of the block's grad_A entries ----
            consumer_sync();
            if (*gave_up == (int)(it & 0x3fffffff) + 1) return;
            const int64_t lim = min(end, base + kPipeTile);
#pragma unroll
            for (int u = 0; u < kPipeTile / (kPipeConsumers * 4); ++u) {
                const int off = (u * kPipeConsumers + tid) * 4;
                const int64_t k = base + off;
                if (k < lim) {
                    if (k >= begin && k + 4 <= lim) {
                        T o[4];
                        lds4<T>(sout + off, o);
                        store4_stream(a.out + k, o);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (k + j >= begin && k + j < lim) a.out[k + j] = sout[off + j];
                    }
                }
            }
        }
        // release the stage: one arrival per consumer warp, after all of its lanes are done with it
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(empty + s);
        cur = nxt;
    }
}

template <typename T, typename I, int MODE, int S, int CH = 8, int MINB = 3, bool DIRECT = false, int GATHER = 0, int WSTORE = 0>
int spmv_pipe_launch(const PipeArgs<T, I>& args, cudaStream_t st) {
    using L = PipeSmem<T, I, MODE, S, DIRECT, GATHER, WSTORE>;
    // the opt-in to more than 48 KB of dynamic shared memory is a per-device property of the kernel
    static std::atomic<bool> configured[kMaxDevices];
    auto kernel = spmv_pipe_kernel<T, I, MODE, S, CH, MINB, DIRECT, GATHER, WSTORE>;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return NB200_ERR_CUDA;
    if (!configured[device].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::total) != cudaSuccess)
            return NB200_ERR_CUDA;
        configured[device].store(true, std::memory_order_release);
    }
    int per_sm = (int)((size_t)(227 * 1024) / (L::total + 1024));
    if (per_sm > MINB) per_sm = MINB;
    const int64_t want = (int64_t)kSMs * (per_sm < 1 ? 1 : per_sm);
    const unsigned grid = (unsigned)(args.num_blocks < want ? args.num_blocks : want);
    kernel<<<grid, kPipeThreads, L::total, st>>>(args);
    return launch_status();
}

// Entry points used by spmv.cu
template <typename T, typename I>
int spmv_pipe_forward(int64_t rows, int64_t nnz, int block_rows, const T* data, const I* indices, const I* indptr,
                      const I* perm, const T* x, T* y, int32_t* status, cudaStream_t st) {
    PipeArgs<T, I> a{0, rows, nnz, ceil_div(rows, (int64_t)block_rows), block_rows, data, indices, indptr, perm, x, nullptr, y, nullptr, status};
    if (perm) return spmv_pipe_launch<T, I, kForwardPerm, 2, 4, 4>(a, st);
    // two stages, four entries per gather round, four CTAs per SM: measured 43 us on the 128^3 Poisson
    // matrix against 48 us for three stages / eight entries / three CTAs -- occupancy beats pipeline depth
    return spmv_pipe_launch<T, I, kForward, 2, 4, 4>(a, st);
}

template <typename T, typename I>
int spmv_pipe_grad_A(int64_t rows, int64_t nnz, int block_rows, const I* indices, const I* indptr, const T* x,
                     const T* g, T* grad_A, int32_t* status, cudaStream_t st) {
    PipeArgs<T, I> a{0, rows, nnz, ceil_div(rows, (int64_t)block_rows), block_rows, nullptr, indices, indptr, nullptr, x, g, grad_A, nullptr, status};
    return spmv_pipe_launch<T, I, kGradA, 2, 4, 4>(a, st);
}

// Configuration of the two fused backward kernels, overridable for tuning builds.
#ifndef NB200_SYMVAL_CH
#define NB200_SYMVAL_CH 4          // entries per gather round
#endif
#ifndef NB200_SYMVAL_MINB
#define NB200_SYMVAL_MINB 4        // CTAs per SM
#endif
#ifndef NB200_SYMVAL_WSTORE
#define NB200_SYMVAL_WSTORE 2      // grad_A leaves through the consumed value slots as a bulk copy per warp
#endif
#ifndef NB200_SYM_WSTORE
#define NB200_SYM_WSTORE 0
#endif

template <typename T, typename I>
int spmv_pipe_backward_sym(int64_t row_begin, int64_t row_end, int64_t nnz, int block_rows, const T* data,
                           const I* indices, const I* indptr, const I* perm, const T* x, const T* g, T* grad_A,
                           T* grad_x, bool values_symmetric, int32_t* status, cudaStream_t st) {
    if (row_end <= row_begin) return NB200_OK;
    PipeArgs<T, I> a{row_begin, row_end, nnz, ceil_div(row_end - row_begin, (int64_t)block_rows), block_rows, data, indices, indptr, perm, x, g, grad_A, grad_x, status};
    if (values_symmetric) {
        // Values and indices staged by bulk copies, x_c and g_c gathered into registers: the traffic is
        // exactly the credited bytes of the backward (no permutation, no value gather).  Measured on the
        // 128^3 Poisson matrix (us), 2 stages: grad_A stored entry by entry from the row threads, 4 entries
        // per round / 4 CTAs per SM 79.7, 8 / 3 83.4; staged in the consumed value slots and copied out by
        // the warp with 16-byte stores 67.3 (2 entries per round 65.6; 3 stages / 3 CTAs 68.6); copied out
        // by one bulk shared-to-global copy per warp 63.6 (8 / 3: 79.6; 3 stages / 3 CTAs 66.8).
        return spmv_pipe_launch<T, I, kBackwardSymVal, 2, NB200_SYMVAL_CH, NB200_SYMVAL_MINB, true, 0, NB200_SYMVAL_WSTORE>(a, st);
    }
    // Measured on the 128^3 Poisson matrix (us).  Gathers into registers, grad_A written straight from the
    // row threads: 2 stages / 2 entries per round / 4 CTAs per SM 94.5; 2/4/4 98; 4/4/3 104; 3/8/3 112; 5+ CTAs
    // per SM spill; grad_A staged in shared memory for coalesced stores 107.  Asynchronous gathers into
    // per-thread slots, 8 entries at a time, 2 stages, 2 CTAs per SM: 85.8.  On top of that: 3 CTAs per SM
    // (7 or 6 slots) 133 -- the L1 that the gathers land in shrinks to a few KB; x through registers 88-98; a
    // single stage 97-128; staging the block's own slice of `data` 95; staging grad_A over the dead index
    // area 101; fetching the transposed value as an L1-bypassing 16-byte group 103.
    return spmv_pipe_launch<T, I, kBackwardSym, 2, 2, 2, true, 8, NB200_SYM_WSTORE>(a, st);
}

#define NB200_INSTANTIATE_PIPE(T, I)                                                                                 \
    template int spmv_pipe_forward<T, I>(int64_t, int64_t, int, const T*, const I*, const I*, const I*, const T*, T*, \
                                         int32_t*, cudaStream_t);                                                    \
    template int spmv_pipe_grad_A<T, I>(int64_t, int64_t, int, const I*, const I*, const T*, const T*, T*, int32_t*,  \
                                        cudaStream_t);                                                               \
    template int spmv_pipe_backward_sym<T, I>(int64_t, int64_t, int64_t, int, const T*, const I*, const I*, const I*, \
                                              const T*, const T*, T*, T*, bool, int32_t*, cudaStream_t);
NB200_INSTANTIATE_PIPE(float, int32_t)
NB200_INSTANTIATE_PIPE(float, int64_t)
NB200_INSTANTIATE_PIPE(double, int32_t)
NB200_INSTANTIATE_PIPE(double, int64_t)

}  // namespace nb200
