// Shared device/host helpers of the mpsbnb_b200 library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mpsbnb_b200.h"

namespace mpsbnb {

// ------------------------------------------------------------------ host-side status plumbing
// Records the failing cudaError_t for mpsbnb_last_cuda_error(); returns MPSBNB_ERR_CUDA.
int record_cuda_error(cudaError_t e);
// Checks the launch that was just enqueued (cudaPeekAtLastError, no synchronisation).
int check_launch();

#define MPSBNB_CUDA_TRY(expr)                                         \
    do {                                                              \
        cudaError_t _e = (expr);                                      \
        if (_e != cudaSuccess) return ::mpsbnb::record_cuda_error(_e); \
    } while (0)

inline bool is_16bit(int dt) { return dt == MPSBNB_F16 || dt == MPSBNB_BF16; }
inline bool valid_dtype(int dt) { return dt >= MPSBNB_F16 && dt <= MPSBNB_F32; }
inline int dtype_bytes(int dt) { return dt == MPSBNB_F32 ? 4 : 2; }
inline bool is_pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// K rounded up to a multiple of the block size (plus one block if that is odd): the row
// length of the packed layout (mps_bitsandbytes/functional.py:219-221).
inline int64_t padded_k(int64_t K, int64_t bs) {
    int64_t kp = ((K + bs - 1) / bs) * bs;
    if (kp & 1) kp += bs;
    return kp;
}

int sm_count();

// ------------------------------------------------------------------ codebooks
// mps_bitsandbytes/functional.py:21-26 and :29-32 (FP4 index 8 is -0.0).
#define MPSBNB_NF4_TABLE                                                                    \
    {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,              \
     -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,             \
     0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f, \
     0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f}
#define MPSBNB_FP4_TABLE                                                     \
    {0.0f, 0.0625f, 0.125f, 0.25f, 0.375f, 0.5f, 0.75f, 1.0f, -0.0f, -0.0625f, \
     -0.125f, -0.25f, -0.375f, -0.5f, -0.75f, -1.0f}

static __device__ __constant__ const float kCode[2][16] = {MPSBNB_NF4_TABLE, MPSBNB_FP4_TABLE};

// ------------------------------------------------------------------ element conversion
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }

// round-to-nearest-even, as torch's .to(dtype)
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

// ------------------------------------------------------------------ int8 helpers shared by the 8-bit kernels
// `127.0 / scale` as torch evaluates it for a Python scalar over a tensor: reciprocal, then times 127
// (two roundings; decides round-half-even ties, mps_bitsandbytes/functional.py:518, 621, 852, 859, 920).
__device__ __forceinline__ float rdiv127(float s) { return __fmul_rn(__frcp_rn(s), 127.0f); }

__device__ __forceinline__ int8_t quant_i8(float x, float f) {
    float v = rintf(__fmul_rn(x, f));                       // torch.round: half to even
    return (int8_t)(int)fminf(fmaxf(v, -127.0f), 127.0f);
}

// CTA-wide max of non-negative values; every thread gets the result.
__device__ __forceinline__ float cta_max(float a, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    __syncthreads();                                        // red[] may still be read by a previous use
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
    __syncthreads();
    a = red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) a = fmaxf(a, red[w]);
    return a;
}

// q (exact in T) times a scale that is rounded to T FIRST, the product rounded to T: the form
// `q.to(dtype) * (scales / 127.0).to(dtype)` of mps_bitsandbytes/nn/embedding.py:269 and
// nn/outlier_aware.py:118-119.  The product of two 16-bit floats is exact in fp32, so one fp32 multiply and
// one rounding equal the multiply in T.
template <typename T> __device__ __forceinline__ T i8_times_rounded_scale(int8_t q, float s_over_127) {
    const float s = to_f32<T>(from_f32<T>(s_over_127));
    return from_f32<T>(__fmul_rn((float)q, s));
}

// Dispatch a callable templated on the element type.
#define MPSBNB_DISPATCH_DTYPE(dt, T, ...)                             \
    do {                                                              \
        if ((dt) == MPSBNB_F16) { using T = __half; __VA_ARGS__; }     \
        else if ((dt) == MPSBNB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else { using T = float; __VA_ARGS__; }                        \
    } while (0)

}  // namespace mpsbnb
