// Shared host/device helpers for the C-ABI library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/flaggems_b200.h"

// Thread-local text of the last error returned by an entry point.
void fg_set_error(const char* fmt, ...);

#define FG_REQUIRE(cond, code, ...)        \
    do {                                   \
        if (!(cond)) {                     \
            fg_set_error(__VA_ARGS__);     \
            return (code);                 \
        }                                  \
    } while (0)

#define FG_CUDA(call)                                                              \
    do {                                                                           \
        cudaError_t e__ = (call);                                                  \
        if (e__ != cudaSuccess) {                                                  \
            fg_set_error("%s failed: %s", #call, cudaGetErrorString(e__));         \
            return FG_ERR_CUDA;                                                    \
        }                                                                          \
    } while (0)

#define FG_LAUNCH_CHECK()                                                          \
    do {                                                                           \
        cudaError_t e__ = cudaGetLastError();                                      \
        if (e__ != cudaSuccess) {                                                  \
            fg_set_error("kernel launch failed: %s", cudaGetErrorString(e__));     \
            return FG_ERR_CUDA;                                                    \
        }                                                                          \
    } while (0)

// Device-side status word (0 = healthy).  Kernels with bounded waits record the
// first failure here; fg_device_status() reads and clears it.
unsigned int* fg_status_word_device_ptr();

static inline int64_t fg_cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

int fg_num_sms();

// Index of the current device clamped to [0, 63]: the key of every per-device cache in the library.
int fg_device_index();

// Adds n to the process-wide count of kernels launched by this library.
void fg_count_launch(int n);

#ifdef __CUDACC__
template <typename T> struct FgVec8;  // eight elements of T as raw words

__device__ __forceinline__ float fg_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float fg_to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float fg_to_float(float v) { return v; }

template <typename T> __device__ __forceinline__ T fg_from_float(float v);
template <> __device__ __forceinline__ __nv_bfloat16 fg_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half fg_from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float fg_from_float<float>(float v) { return v; }

// Load eight consecutive elements as floats; p must be 16-byte aligned for
// 16-bit types and 32-byte aligned for fp32.
template <typename T>
__device__ __forceinline__ void fg_load8(const T* p, float (&f)[8]) {
    if constexpr (sizeof(T) == 2) {
        uint4 raw = *reinterpret_cast<const uint4*>(p);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = fg_to_float(e[i]);
    } else {
        float4 a = reinterpret_cast<const float4*>(p)[0];
        float4 b = reinterpret_cast<const float4*>(p)[1];
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
        f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
}

// Eight 16-bit elements already in registers (one 16-byte load) as floats.
template <typename T>
__device__ __forceinline__ void fg_unpack8(const uint4& raw, float (&f)[8]) {
    static_assert(sizeof(T) == 2, "16-bit element types only");
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = fg_to_float(e[i]);
}

template <typename T>
__device__ __forceinline__ void fg_store8(T* p, const float (&f)[8]) {
    if constexpr (sizeof(T) == 2) {
        uint4 raw;
        T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = fg_from_float<T>(f[i]);
        *reinterpret_cast<uint4*>(p) = raw;
    } else {
        reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
}

// Eight floats -> eight e4m3 bytes (round to nearest even, saturate to +-448).
__device__ __forceinline__ uint2 fg_pack_e4m3x8(const float (&q)[8]) {
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q[4 * h + 0], q[4 * h + 1]), __NV_SATFINITE, __NV_E4M3);
        uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q[4 * h + 2], q[4 * h + 3]), __NV_SATFINITE, __NV_E4M3);
        w[h] = lo | (hi << 16);
    }
    return make_uint2(w[0], w[1]);
}
#endif
