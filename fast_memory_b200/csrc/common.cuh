// Shared host/device helpers for the fastmem_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/fastmem_b200.h"

namespace fm {

// ---- host-side status plumbing -----------------------------------------------------------------
void set_error(const char *fmt, ...);          // thread-local message, defined in abi.cu
extern std::atomic<int64_t> g_launches;        // kernels launched by this process

inline int cuda_fail(cudaError_t e, const char *what)
{
    set_error("%s: %s", what, cudaGetErrorString(e));
    return FM_ERR_CUDA;
}

#define FM_CUDA_OK(expr)                                                   \
    do {                                                                   \
        cudaError_t _e = (expr);                                           \
        if (_e != cudaSuccess) return ::fm::cuda_fail(_e, #expr);          \
    } while (0)

// Call after every kernel launch: records it and surfaces launch-configuration errors.
#define FM_LAUNCHED(name)                                                  \
    do {                                                                   \
        ::fm::g_launches.fetch_add(1, std::memory_order_relaxed);          \
        cudaError_t _e = cudaGetLastError();                               \
        if (_e != cudaSuccess) return ::fm::cuda_fail(_e, name);           \
    } while (0)

#define FM_REQUIRE(cond, ...)                                              \
    do {                                                                   \
        if (!(cond)) {                                                     \
            ::fm::set_error(__VA_ARGS__);                                  \
            return FM_ERR_BAD_ARG;                                         \
        }                                                                  \
    } while (0)

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
int sm_count();                                // SMs of the current device (cached per device)
cudaError_t func_attr_cached(const void *func, cudaFuncAttribute attr, int value);   // cudaFuncSetAttribute, skipped when unchanged

// ---- element types -------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int id = FM_F32;
    __device__ static __forceinline__ float to_f32(float x) { return x; }
    __device__ static __forceinline__ float from_f32(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int id = FM_BF16;
    __device__ static __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
    __device__ static __forceinline__ __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Elem<__half> {
    static constexpr int id = FM_F16;
    __device__ static __forceinline__ float to_f32(__half x) { return __half2float(x); }
    __device__ static __forceinline__ __half from_f32(float x) { return __float2half_rn(x); }
};

inline int elem_bytes(int dtype) { return dtype == FM_F32 ? 4 : 2; }

// Widen 8 consecutive 16-bit elements held in a uint4 (or 4 floats per float4) to fp32.
__device__ __forceinline__ void widen8(const uint4 &raw, float (&out)[8], __nv_bfloat16)
{
    const __nv_bfloat162 *p = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(p[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void widen8(const uint4 &raw, float (&out)[8], __half)
{
    const __half2 *p = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(p[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}

// Segment of a row given an int32 prefix array (n_seg + 1 entries): largest s with pre[s] <= r.
__device__ __forceinline__ int find_segment(const int32_t *__restrict__ pre, int n_seg, int r)
{
    int lo = 0, hi = n_seg;            // invariant: pre[lo] <= r < pre[hi]
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (pre[mid] <= r) lo = mid; else hi = mid;
    }
    return lo;
}

// Order-preserving float -> uint32 key (bigger float <=> bigger key); -0.0 folds onto +0.0.
__device__ __forceinline__ uint32_t float_key(float f)
{
    if (f == 0.0f) f = 0.0f;
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

}  // namespace fm
