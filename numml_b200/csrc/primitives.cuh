// Host-callable device primitives shared by the CSR kernels: exclusive scan, stable LSD radix
// sort of (key, value) pairs, and small elementwise helpers.  All asynchronous on a stream, all
// scratch memory supplied by the caller.
#pragma once
#include "common.cuh"

namespace nb200 {

// Bump allocator over a caller-provided workspace; every block is 256-byte aligned.
struct Workspace {
    char* base;
    size_t size;
    size_t used;
    Workspace(void* p, size_t n) : base(static_cast<char*>(p)), size(n), used(0) {}
    static size_t pad(size_t n) { return (n + 255) & ~(size_t)255; }
    template <typename U>
    U* take(size_t count) {
        const size_t bytes = pad(count * sizeof(U));
        if (base == nullptr || used + bytes > size) { used = size + 1; return nullptr; }
        U* p = reinterpret_cast<U*>(base + used);
        used += bytes;
        return p;
    }
    bool ok() const { return used <= size; }
};

// Exclusive prefix sum: out[i] = sum(in[0..i)), i in [0, n]; out has n+1 entries (out[n] is the
// total).  `in` and `out` may not alias.  Scratch: scan_scratch_bytes(n).
size_t scan_scratch_bytes(int64_t n);
int exclusive_scan_i32_to_i32(int64_t n, const int32_t* in, int32_t* out, void* scratch, size_t scratch_bytes, cudaStream_t st);
int exclusive_scan_i32_to_i64(int64_t n, const int32_t* in, int64_t* out, void* scratch, size_t scratch_bytes, cudaStream_t st);

// Stable sort of n (key, value) pairs by the low `key_bits` bits of the unsigned 32-bit key,
// 8 bits per pass.  Buffers ping-pong between (keys_a, vals_a) and (keys_b, vals_b); on return
// *result_in_a says which pair holds the sorted output.  Scratch: sort_scratch_bytes(n).
size_t sort_scratch_bytes(int64_t n);
int sort_pairs_u32(int64_t n, int key_bits, uint32_t* keys_a, uint32_t* vals_a, uint32_t* keys_b,
                   uint32_t* vals_b, bool* result_in_a, void* scratch, size_t scratch_bytes, cudaStream_t st);

}  // namespace nb200
