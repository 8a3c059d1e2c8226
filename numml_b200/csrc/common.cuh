// Shared helpers for the sm_100a CSR kernels: status codes, dtype/index-type dispatch,
// 128-bit load helpers and launch-error capture.  Internal to the library; the public
// interface is include/numml_b200.h.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/numml_b200.h"

namespace nb200 {

constexpr int kSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? NB200_OK : NB200_ERR_CUDA;
}

inline cudaStream_t as_stream(nb200_stream s) { return reinterpret_cast<cudaStream_t>(s); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename A, typename B>
__host__ __device__ constexpr A ceil_div(A a, B b) { return (a + b - 1) / b; }

// Multiply / add / fma wrappers.  The stream kernels keep the multiply and the add separate
// (round-to-nearest each) so that a sum taken in storage order is bit-identical to the
// reference CPU loops, which are compiled without fused multiply-add.
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }

// Read-only (non-coherent) scalar loads; go through L1/tex, used for gathers.
template <typename T>
__device__ __forceinline__ T ldg(const T* p) { return __ldg(p); }

// Streaming 4-element loads for data that is read exactly once: one or two 128-bit
// ld.global.nc.L1::no_allocate instructions.  `p` must be 16-byte aligned.
__device__ __forceinline__ void load4_stream(const float* p, float (&v)[4]) {
    float4 t;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(t.x), "=f"(t.y), "=f"(t.z), "=f"(t.w) : "l"(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4_stream(const double* p, double (&v)[4]) {
    asm volatile("ld.global.nc.L1::no_allocate.v2.f64 {%0,%1}, [%2];" : "=d"(v[0]), "=d"(v[1]) : "l"(p));
    asm volatile("ld.global.nc.L1::no_allocate.v2.f64 {%0,%1}, [%2];" : "=d"(v[2]), "=d"(v[3]) : "l"(p + 2));
}
__device__ __forceinline__ void load4_stream(const int32_t* p, int32_t (&v)[4]) {
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "l"(p));
}
__device__ __forceinline__ void load4_stream(const int64_t* p, int64_t (&v)[4]) {
    asm volatile("ld.global.nc.L1::no_allocate.v2.s64 {%0,%1}, [%2];" : "=l"(v[0]), "=l"(v[1]) : "l"(p));
    asm volatile("ld.global.nc.L1::no_allocate.v2.s64 {%0,%1}, [%2];" : "=l"(v[2]), "=l"(v[3]) : "l"(p + 2));
}

// Streaming 4-element stores (write-once outputs).  `p` must be 16-byte aligned.
__device__ __forceinline__ void store4_stream(float* p, const float (&v)[4]) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" :: "l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
}
__device__ __forceinline__ void store4_stream(double* p, const double (&v)[4]) {
    asm volatile("st.global.cs.v2.f64 [%0], {%1,%2};" :: "l"(p), "d"(v[0]), "d"(v[1]) : "memory");
    asm volatile("st.global.cs.v2.f64 [%0], {%1,%2};" :: "l"(p + 2), "d"(v[2]), "d"(v[3]) : "memory");
}

}  // namespace nb200

// Dispatch a templated launcher on (value type, index type).  `CALL` is an expression that
// uses the names T and I and evaluates to an int status.
#define NB200_DISPATCH(dtype, itype, CALL)                                        \
    [&]() -> int {                                                                \
        if ((dtype) == NB200_F32 && (itype) == NB200_I32) { using T = float;  using I = int32_t; return CALL; } \
        if ((dtype) == NB200_F32 && (itype) == NB200_I64) { using T = float;  using I = int64_t; return CALL; } \
        if ((dtype) == NB200_F64 && (itype) == NB200_I32) { using T = double; using I = int32_t; return CALL; } \
        if ((dtype) == NB200_F64 && (itype) == NB200_I64) { using T = double; using I = int64_t; return CALL; } \
        return NB200_ERR_BAD_ARG;                                                 \
    }()

#define NB200_DISPATCH_I(itype, CALL)                                             \
    [&]() -> int {                                                                \
        if ((itype) == NB200_I32) { using I = int32_t; return CALL; }             \
        if ((itype) == NB200_I64) { using I = int64_t; return CALL; }             \
        return NB200_ERR_BAD_ARG;                                                 \
    }()

#define NB200_DISPATCH_T(dtype, CALL)                                             \
    [&]() -> int {                                                                \
        if ((dtype) == NB200_F32) { using T = float; return CALL; }               \
        if ((dtype) == NB200_F64) { using T = double; return CALL; }              \
        return NB200_ERR_BAD_ARG;                                                 \
    }()
