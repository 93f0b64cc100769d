// Outlier-aware INT8 linear (LLM.int8 mixed-precision decomposition), the forward of the reference's
// OutlierAwareLinear (mps_bitsandbytes/nn/outlier_aware.py:84-146):
//   y = deq(quantize_rowwise(x_main)) . deq(W_int8_main)^T  +  x_outlier . W_outlier^T  (+ bias)
// where "main" are the input features that are not outlier columns, both dequantisations use a scale
// rounded to the compute type first (`q.to(dtype) * (s / 127).to(dtype)`, :118-119, :138-139), and the
// outlier columns of x meet weights kept in 16 bits.
//
// The reference slices columns out of x and W and runs two matrix products.  Here both parts share ONE
// contraction over the full K: the operand built from x holds the re-quantised value in a main column and
// the untouched 16-bit value in an outlier column; the operand built from W holds the dequantised int8
// weight in a main column and the 16-bit outlier weight in an outlier column.  The tcgen05 GEMM then
// accumulates main and outlier products together in fp32 (the reference rounds the two partial results to
// 16 bits before adding them; the difference is far inside the 1e-2 matmul bound).  No gather, no second
// GEMM, no addition pass.  With no outlier columns this is the pure INT8 path (:112-121).
//
// Workspace (caller-supplied): slot[K] int32 (0 = main column, j + 1 = outlier j), x operand
// [M, ld8(K)], W operand [N, ld8(K)] in the compute type.
#include "ops.cuh"

namespace mpsbnb {

static inline int64_t o_ld8(int64_t k) { return (k + 7) / 8 * 8; }
static inline size_t o_align256(size_t b) { return (b + 255) / 256 * 256; }

__global__ void outlier_slot_kernel(const int64_t *__restrict__ idx, int64_t n_out, int64_t K, int *__restrict__ slot) {
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n_out) return;
    const int64_t k = idx[j];
    if (k >= 0 && k < K) slot[k] = (int)(j + 1);
}

// One CTA per row of x: row maximum over the main columns (clamped to 1e-8), then every main element is
// quantised to int8 and expanded again, outlier elements are passed through in the compute type.
// ZERO_OUT: outlier columns are written as zeros (the fused path multiplies them separately).
template <typename TX, typename T, bool ZERO_OUT = false>
__global__ void __launch_bounds__(256) outlier_x_kernel(const TX *__restrict__ x, int64_t M, int64_t K,
                                                        const int *__restrict__ slot, T *__restrict__ out, int64_t ld) {
    __shared__ float red[8];
    for (int64_t m = blockIdx.x; m < M; m += gridDim.x) {
        const TX *row = x + m * K;
        float a = 0.0f;
        for (int64_t k = threadIdx.x; k < K; k += blockDim.x)
            if (slot[k] == 0) a = fmaxf(a, fabsf(to_f32<TX>(row[k])));
        a = fmaxf(cta_max(a, red), 1e-8f);
        const float f = rdiv127(a);
        const float s127 = __fdiv_rn(a, 127.0f);
        for (int64_t k = threadIdx.x; k < K; k += blockDim.x) {
            const float v = to_f32<TX>(row[k]);
            out[m * ld + k] = slot[k] == 0 ? i8_times_rounded_scale<T>(quant_i8(v, f), s127) : (ZERO_OUT ? from_f32<T>(0.0f) : from_f32<T>(v));
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) outlier_w_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
                                                        const T *__restrict__ outlier_w, int64_t n_out, int64_t N,
                                                        int64_t K, const int *__restrict__ slot, T *__restrict__ out,
                                                        int64_t ld) {
    const int64_t total = N * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / K, k = i - n * K;
        const int s = slot[k];
        out[n * ld + k] = s == 0 ? i8_times_rounded_scale<T>(q[i], __fdiv_rn(__ldg(scales + n), 127.0f))
                                 : outlier_w[n * n_out + (s - 1)];
    }
}

// The same, 16 elements per thread (K % 16 == 0, 16-byte aligned rows): one 16-byte load of codes, four of
// the column map, two 16-byte stores.  Bound by HBM instead of by the per-element index arithmetic.
template <typename T>
__global__ void __launch_bounds__(256) outlier_w16_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
                                                          const T *__restrict__ outlier_w, int64_t n_out, int64_t N,
                                                          int64_t K, const int *__restrict__ slot, T *__restrict__ out,
                                                          int64_t ld) {
    const int64_t cpr = K / 16, total = N * cpr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t n, c;
        if (total < 0x7fffffffll) { const uint32_t n32 = (uint32_t)i / (uint32_t)cpr; n = n32; c = (uint32_t)i - n32 * (uint32_t)cpr; }
        else { n = i / cpr; c = i - n * cpr; }
        const uint4 w = __ldg(reinterpret_cast<const uint4 *>(q + n * K + c * 16));
        const int8_t *b = reinterpret_cast<const int8_t *>(&w);
        __align__(16) int sl[16];
#pragma unroll
        for (int v = 0; v < 4; ++v) reinterpret_cast<int4 *>(sl)[v] = __ldg(reinterpret_cast<const int4 *>(slot + c * 16) + v);
        const float s127 = __fdiv_rn(__ldg(scales + n), 127.0f);
        __align__(16) T vals[16];
#pragma unroll
        for (int e = 0; e < 16; ++e)
            vals[e] = sl[e] == 0 ? i8_times_rounded_scale<T>(b[e], s127) : outlier_w[n * n_out + (sl[e] - 1)];
        uint4 *dst = reinterpret_cast<uint4 *>(out + n * ld + c * 16);
        dst[0] = reinterpret_cast<const uint4 *>(vals)[0];
        dst[1] = reinterpret_cast<const uint4 *>(vals)[1];
    }
}

// y[m, n] += sum_j x[m, idx[j]] * outlier_w[n, j] (+ bias[n]): the 16-bit part of the decomposition, a few dozen
// columns wide.  One thread per output column n, 16 rows of x per CTA (their outlier values sit in shared memory).
template <typename TX, typename T, typename TY>
__global__ void __launch_bounds__(256) outlier_add_kernel(const TX *__restrict__ x, int64_t M, int64_t K,
                                                          const int64_t *__restrict__ idx, int n_out,
                                                          const T *__restrict__ ow, const T *__restrict__ bias, int64_t N,
                                                          TY *__restrict__ y) {
    extern __shared__ float xs[];                               // [16][n_out]
    const int64_t m0 = (int64_t)blockIdx.y * 16;
    const int rows = (int)(M - m0 < 16 ? M - m0 : 16);
    for (int i = threadIdx.x; i < rows * n_out; i += blockDim.x) {
        const int r = i / n_out, j = i - r * n_out;
        const int64_t k = idx[j];
        // the reference casts x to the compute type before the outlier product
        xs[i] = (k >= 0 && k < K) ? to_f32<T>(from_f32<T>(to_f32<TX>(x[(m0 + r) * K + k]))) : 0.0f;
    }
    __syncthreads();
    const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float acc[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) acc[r] = 0.0f;
    for (int j = 0; j < n_out; ++j) {
        const float w = to_f32<T>(ow[n * n_out + j]);
#pragma unroll
        for (int r = 0; r < 16; ++r) acc[r] = fmaf(xs[r * n_out + j], w, acc[r]);   // rows beyond `rows` read stale, unused values
    }
    const float b = bias != nullptr ? to_f32<T>(bias[n]) : 0.0f;
#pragma unroll
    for (int r = 0; r < 16; ++r)
        if (r < rows) {
            TY *p = y + (m0 + r) * N + n;
            *p = from_f32<TY>(to_f32<TY>(*p) + to_f32<T>(from_f32<T>(acc[r])) + b);
        }
}

static inline unsigned o_grid(int64_t items) {
    const int64_t ctas = (items + 255) / 256, cap = (int64_t)sm_count() * 16;
    return (unsigned)(ctas < 1 ? 1 : (ctas > cap ? cap : ctas));
}

}  // namespace mpsbnb

using namespace mpsbnb;

extern "C" size_t mpsbnb_outlier_linear_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return o_align256((size_t)K * 4) + o_align256((size_t)M * (size_t)o_ld8(K) * 2) + o_align256((size_t)N * (size_t)o_ld8(K) * 2);
}

extern "C" int mpsbnb_outlier_linear(const void *x, int x_dtype, int64_t M, const int8_t *W, const float *w_scales,
                                     const int64_t *outlier_idx, int64_t n_outliers, const void *outlier_w,
                                     int64_t N, int64_t K, const void *bias, int op_dtype, void *y, int y_dtype,
                                     void *workspace, size_t workspace_bytes, void *stream) {
    if (!valid_dtype(x_dtype) || !is_16bit(op_dtype) || !valid_dtype(y_dtype) || M < 0 || N < 0 || K <= 0 || n_outliers < 0)
        return MPSBNB_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return MPSBNB_OK;
    if (x == nullptr || W == nullptr || w_scales == nullptr || y == nullptr || workspace == nullptr) return MPSBNB_ERR_INVALID_ARG;
    if (n_outliers > 0 && (outlier_idx == nullptr || outlier_w == nullptr)) return MPSBNB_ERR_INVALID_ARG;
    if (workspace_bytes < mpsbnb_outlier_linear_workspace_bytes(M, N, K) || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return MPSBNB_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned char *ws = reinterpret_cast<unsigned char *>(workspace);
    int *slot = reinterpret_cast<int *>(ws);
    ws += o_align256((size_t)K * 4);
    void *xo = ws;
    ws += o_align256((size_t)M * (size_t)o_ld8(K) * 2);
    void *wo = ws;
    const int64_t ld = o_ld8(K);
    MPSBNB_CUDA_TRY(cudaMemsetAsync(slot, 0, (size_t)K * 4, st));
    if (n_outliers > 0) {
        outlier_slot_kernel<<<(unsigned)((n_outliers + 255) / 256), 256, 0, st>>>(outlier_idx, n_outliers, K, slot);
        int rc = check_launch();
        if (rc != MPSBNB_OK) return rc;
    }
    const bool vec16 = K % 16 == 0 && aligned16(W);             // slot and the operand live in the 256-byte aligned workspace
    const unsigned xgrid = (unsigned)(M < (int64_t)sm_count() * 8 ? M : (int64_t)sm_count() * 8);
    if (vec16 && n_outliers <= 512) {
        // Fused path: the int8 weight is never expanded in memory.  x operand = re-quantised main columns, zeros in the
        // outlier columns; main product by the fused dequantise-GEMM (row scale / 127 on the accumulator); then the
        // outlier columns' 16-bit product and the bias are added to y.
        if (op_dtype == MPSBNB_F16) {
            MPSBNB_DISPATCH_DTYPE(x_dtype, TX, (outlier_x_kernel<TX, __half, true><<<xgrid, 256, 0, st>>>((const TX *)x, M, K, slot, (__half *)xo, ld)));
        } else {
            MPSBNB_DISPATCH_DTYPE(x_dtype, TX, (outlier_x_kernel<TX, __nv_bfloat16, true><<<xgrid, 256, 0, st>>>((const TX *)x, M, K, slot, (__nv_bfloat16 *)xo, ld)));
        }
        int rc = check_launch();
        if (rc != MPSBNB_OK) return rc;
        const bool tail = n_outliers > 0 || bias != nullptr;
        rc = gemm_wq(1, xo, ld, op_dtype, M, W, K, nullptr, nullptr, w_scales, 1.0f / 127.0f, 0, N, K, 0, nullptr, y, y_dtype, st);
        if (rc != MPSBNB_OK || !tail) return rc;
        const dim3 grid((unsigned)((N + 255) / 256), (unsigned)((M + 15) / 16));
        const size_t smem = (size_t)16 * (size_t)(n_outliers > 0 ? n_outliers : 1) * sizeof(float);
#define MPSBNB_OUTLIER_ADD(TX, T, TY) outlier_add_kernel<TX, T, TY><<<grid, 256, smem, st>>>((const TX *)x, M, K, outlier_idx, (int)n_outliers, (const T *)outlier_w, (const T *)bias, N, (TY *)y)
        if (op_dtype == MPSBNB_F16) {
            MPSBNB_DISPATCH_DTYPE(x_dtype, TX, MPSBNB_DISPATCH_DTYPE(y_dtype, TY, MPSBNB_OUTLIER_ADD(TX, __half, TY)));
        } else {
            MPSBNB_DISPATCH_DTYPE(x_dtype, TX, MPSBNB_DISPATCH_DTYPE(y_dtype, TY, MPSBNB_OUTLIER_ADD(TX, __nv_bfloat16, TY)));
        }
#undef MPSBNB_OUTLIER_ADD
        return check_launch();
    }
    if (op_dtype == MPSBNB_F16) {
        MPSBNB_DISPATCH_DTYPE(x_dtype, TX, (outlier_x_kernel<TX, __half><<<xgrid, 256, 0, st>>>((const TX *)x, M, K, slot, (__half *)xo, ld)));
        if (vec16) outlier_w16_kernel<__half><<<o_grid(N * K / 16), 256, 0, st>>>(W, w_scales, (const __half *)outlier_w, n_outliers, N, K, slot, (__half *)wo, ld);
        else outlier_w_kernel<__half><<<o_grid(N * K), 256, 0, st>>>(W, w_scales, (const __half *)outlier_w, n_outliers, N, K, slot, (__half *)wo, ld);
    } else {
        MPSBNB_DISPATCH_DTYPE(x_dtype, TX, (outlier_x_kernel<TX, __nv_bfloat16><<<xgrid, 256, 0, st>>>((const TX *)x, M, K, slot, (__nv_bfloat16 *)xo, ld)));
        if (vec16) outlier_w16_kernel<__nv_bfloat16><<<o_grid(N * K / 16), 256, 0, st>>>(W, w_scales, (const __nv_bfloat16 *)outlier_w, n_outliers, N, K, slot, (__nv_bfloat16 *)wo, ld);
        else outlier_w_kernel<__nv_bfloat16><<<o_grid(N * K), 256, 0, st>>>(W, w_scales, (const __nv_bfloat16 *)outlier_w, n_outliers, N, K, slot, (__nv_bfloat16 *)wo, ld);
    }
    int rc = check_launch();
    if (rc != MPSBNB_OK) return rc;
    return gemm_16bit(xo, ld, wo, ld, op_dtype, M, N, K, nullptr, nullptr, bias, op_dtype, y, N, y_dtype, st);
}
