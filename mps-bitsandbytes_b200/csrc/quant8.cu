// 8-bit quantisers and dequantisers: row-wise int8, LLM.int8 row+column statistics,
// col+row int8, and row-scaled FP8 E4M3.  Bit-identical to the reference's CPU path
// (mps_bitsandbytes/functional.py:607-673, 814-932, 1086-1216).
//
// Two arithmetic details of the reference decide exact ties and are reproduced:
//  * `127.0 / scale` is computed by torch as scale.reciprocal() * 127.0 (two roundings);
//  * the FP8 exponent is floor(log2(x)) evaluated in fp32, which returns the NEXT integer
//    for the few floats just below a power of two (see fp8_exponent()).
#include "common.cuh"

namespace mpsbnb {

// ------------------------------------------------------------------ row statistics
// One CTA per row: max|x| over the row (NOT clamped).
template <typename T>
__global__ void __launch_bounds__(256) row_absmax_kernel(const T *__restrict__ x, int64_t rows, int64_t cols,
                                                         float *__restrict__ out, float floor_value) {
    __shared__ float red[8];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        float a = 0.0f;
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) a = fmaxf(a, fabsf(to_f32<T>(x[r * cols + c])));
        a = cta_max(a, red);
        if (threadIdx.x == 0) out[r] = fmaxf(a, floor_value);
    }
}

__global__ void fill_kernel(float *p, int64_t n, float v) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        p[i] = v;
}

// Column maxima: threads run along columns (coalesced), CTAs in y split the rows and
// merge with an integer atomicMax (valid because the values are non-negative floats).
// `out` must be pre-filled with the floor value (1e-8).
template <typename T>
__global__ void col_absmax_kernel(const T *__restrict__ x, int64_t rows, int64_t cols, float *__restrict__ out) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const int64_t per = (rows + gridDim.y - 1) / gridDim.y;
    const int64_t r0 = blockIdx.y * per, r1 = min(rows, r0 + per);
    float a = 0.0f;
    for (int64_t r = r0; r < r1; ++r) a = fmaxf(a, fabsf(to_f32<T>(x[r * cols + c])));
    atomicMax(reinterpret_cast<int *>(out) + c, __float_as_int(a));
}

// ------------------------------------------------------------------ int8 quantisers
// mode 0: f = 127/row[r]; mode 1: f = 127/col[c]; mode 2: f = 127/sqrt(row[r]*col[c])
template <typename T, int MODE>
__global__ void quantize_i8_kernel(const T *__restrict__ x, int64_t rows, int64_t cols,
                                   const float *__restrict__ row_s, const float *__restrict__ col_s,
                                   int8_t *__restrict__ q) {
    const int64_t total = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols, c = i - r * cols;
        float f;
        if (MODE == 0) f = rdiv127(__ldg(row_s + r));
        else if (MODE == 1) f = rdiv127(__ldg(col_s + c));
        else f = rdiv127(__fsqrt_rn(__fmul_rn(__ldg(row_s + r), __ldg(col_s + c))));
        q[i] = quant_i8(to_f32<T>(x[i]), f);
    }
}

// mode 0: q * (row[r]/127); mode 2: q * (sqrt(row[r]*col[c]) / 127)
template <typename T, int MODE>
__global__ void dequantize_i8_kernel(const int8_t *__restrict__ q, int64_t rows, int64_t cols,
                                     const float *__restrict__ row_s, const float *__restrict__ col_s,
                                     T *__restrict__ out, int64_t ld) {
    const int64_t total = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols, c = i - r * cols;
        float s = __ldg(row_s + r);
        if (MODE == 2) s = __fsqrt_rn(__fmul_rn(s, __ldg(col_s + c)));
        out[r * ld + c] = from_f32<T>(__fmul_rn((float)q[i], __fdiv_rn(s, 127.0f)));
    }
}

// ------------------------------------------------------------------ FP8 E4M3
// floor(log2(a)) as an fp32 log2 followed by floor gives it, for a normal float a > 0:
// with E = exponent(a) + 1 and k = number of floats between a and 2^E (inclusive of 2^E),
// a correctly rounded log2 returns E itself when k <= kmax(j), where 2^(j-24) is half
// the float spacing next to E on the side of log2(a): j = floor(log2(E-1)) for E >= 2,
// j = floor(log2|E|) for E < 0, and no rounding up for E in {0, 1}.
__device__ __forceinline__ int fp8_exponent(uint32_t bits) {
    const int e = (int)(bits >> 23) - 127;
    const int E = e + 1;
    const int k = 0x800000 - (int)(bits & 0x7FFFFFu);
    int j = -1;
    if (E >= 2) j = 31 - __clz(E - 1);
    else if (E < 0) j = 31 - __clz(-E);
    // floor((1 - 2^-(2^(j-24))) * 2^24) for j = 0..7
    const int kmax = j < 0 ? 0 : (j == 0 ? 0 : j == 1 ? 1 : j == 2 ? 2 : j == 3 ? 5 : j == 4 ? 11 : j == 5 ? 22 : j == 6 ? 44 : 88);
    return k <= kmax ? E : e;
}

// mps_bitsandbytes/functional.py:1106-1163 for one already-normalised, clamped value.
__device__ __forceinline__ uint8_t fp8_encode(float n) {
    if (n != n) return 0x7F;
    const uint32_t sign = n < 0.0f ? 0x80u : 0u;
    const float a = fminf(fabsf(n), 448.0f);
    const uint32_t bits = __float_as_uint(a);
    if ((bits >> 23) == 0) return (uint8_t)sign;            // zero, or far below 2^-7
    const int e = fp8_exponent(bits);
    const int biased = e + 7;
    if (biased <= 0) return (uint8_t)sign;                  // "subnormal" range flushes to signed zero
    if (biased >= 15) return (uint8_t)(sign | 0x77u);       // clamps to 240, not 448
    const float pow2 = __uint_as_float((uint32_t)(e + 127) << 23);
    const float mf = __fsub_rn(__fdiv_rn(a, pow2), 1.0f);
    float mb = __fadd_rn(__fmul_rn(mf, 8.0f), 0.5f);
    mb = fminf(fmaxf(mb, 0.0f), 7.0f);                      // no carry into the exponent
    return (uint8_t)(sign | ((uint32_t)biased << 3) | (uint32_t)mb);
}

__device__ __forceinline__ float fp8_decode(uint32_t c) {   // functional.py:1178-1216
    const uint32_t exp = (c >> 3) & 0xFu, man = c & 7u;
    float r;
    if (exp == 0) r = __fmul_rn((float)man * 0.125f, 0.015625f);
    else if (exp == 15 && man == 7) r = __int_as_float(0x7FC00000);
    else r = __fmul_rn(1.0f + (float)man * 0.125f, __uint_as_float((exp - 7 + 127) << 23));
    return (c & 0x80u) ? -r : r;
}

template <typename T>
__global__ void quantize_fp8_kernel(const T *__restrict__ x, int64_t rows, int64_t cols,
                                    const float *__restrict__ scales, uint8_t *__restrict__ codes) {
    const int64_t total = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const float s = __ldg(scales + i / cols);
        float n = __fdiv_rn(to_f32<T>(x[i]), s);
        n = fminf(fmaxf(n, -448.0f), 448.0f);               // NaN passes through both
        if (n != n) n = __int_as_float(0x7FC00000);
        codes[i] = fp8_encode(n);
    }
}

// scales = clamp(rowmax / 448, 1e-12)
__global__ void fp8_scales_kernel(float *__restrict__ s, int64_t rows) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += (int64_t)gridDim.x * blockDim.x)
        s[i] = fmaxf(__fdiv_rn(s[i], 448.0f), 1e-12f);
}

template <typename T>
__global__ void dequantize_fp8_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ scales,
                                      int64_t rows, int64_t cols, T *__restrict__ out, int64_t ld) {
    __shared__ float lut[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = fp8_decode(i);
    __syncthreads();
    const int64_t total = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x)
    {
            const int64_t r = i / cols;
            out[r * ld + (i - r * cols)] = from_f32<T>(__fmul_rn(lut[codes[i]], __ldg(scales + r)));
        }
}

// Operand expansion for the GEMM paths, 16 elements per thread: one 16-byte load, two 16-byte stores (fp32
// output: four).  Needs cols % 16 == 0, a 16-byte aligned source and destination and ld % 8 == 0.  The
// one-element kernels above spend their time on a 64-bit division per element; this one is bound by HBM.
// KIND 0: int8 * (row / 127); 2: int8 * (sqrt(row * col) / 127); 3: FP8 E4M3 code * row scale.
template <typename T, int KIND>
__global__ void __launch_bounds__(256) expand16_kernel(const uint8_t *__restrict__ src, int64_t rows, int64_t cols,
                                                       const float *__restrict__ row_s, const float *__restrict__ col_s,
                                                       T *__restrict__ out, int64_t ld) {
    __shared__ float lut[256];
    if (KIND == 3) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = fp8_decode(i);
        __syncthreads();
    }
    const int64_t cpr = cols / 16, total = rows * cpr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r, c;
        if (total < 0x7fffffffll) { const uint32_t r32 = (uint32_t)i / (uint32_t)cpr; r = r32; c = (uint32_t)i - r32 * (uint32_t)cpr; }
        else { r = i / cpr; c = i - r * cpr; }
        const uint4 w = __ldg(reinterpret_cast<const uint4 *>(src + r * cols + c * 16));
        const uint8_t *b = reinterpret_cast<const uint8_t *>(&w);
        const float rs = __ldg(row_s + r);
        __align__(16) T vals[16];
        if (KIND == 0) {
            const float f = __fdiv_rn(rs, 127.0f);
#pragma unroll
            for (int e = 0; e < 16; ++e) vals[e] = from_f32<T>(__fmul_rn((float)(int8_t)b[e], f));
        } else if (KIND == 2) {
            __align__(16) float cs[16];
#pragma unroll
            for (int v = 0; v < 4; ++v) reinterpret_cast<float4 *>(cs)[v] = __ldg(reinterpret_cast<const float4 *>(col_s + c * 16) + v);
#pragma unroll
            for (int e = 0; e < 16; ++e)
                vals[e] = from_f32<T>(__fmul_rn((float)(int8_t)b[e], __fdiv_rn(__fsqrt_rn(__fmul_rn(rs, cs[e])), 127.0f)));
        } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) vals[e] = from_f32<T>(__fmul_rn(lut[b[e]], rs));
        }
        uint4 *dst = reinterpret_cast<uint4 *>(out + r * ld + c * 16);
#pragma unroll
        for (int v = 0; v < (int)sizeof(T); ++v) dst[v] = reinterpret_cast<const uint4 *>(vals)[v];
    }
}

static inline bool expand16_ok(const void *src, int64_t cols, const void *out, int64_t ld, const void *col_s) {
    return cols % 16 == 0 && ld % 8 == 0 && aligned16(src) && aligned16(out) && (col_s == nullptr || aligned16(col_s));
}

static int grid_1d(int64_t n, int threads = 256) {
    int64_t g = (n + threads - 1) / threads;
    const int64_t cap = (int64_t)sm_count() * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

template <typename T>
static int launch_col_absmax(const T *x, int64_t rows, int64_t cols, float *out, cudaStream_t st) {
    fill_kernel<<<grid_1d(cols), 256, 0, st>>>(out, cols, 1e-8f);
    const int gx = (int)((cols + 255) / 256);
    int64_t gy = (int64_t)sm_count() * 4 / gx;
    if (gy < 1) gy = 1;
    if (gy > rows) gy = rows;
    col_absmax_kernel<T><<<dim3(gx, (unsigned)gy), 256, 0, st>>>(x, rows, cols, out);
    return check_launch();
}

// out[n, k] = float(B[k, n]) * (col_scales[n] / 127): the transposed, dequantised copy of a
// [K, N] int8 matrix with per-column scales (mps_bitsandbytes/functional.py:792).
template <typename T>
__global__ void dequantize_i8_transposed_kernel(const int8_t *__restrict__ B, const float *__restrict__ col_s,
                                                int64_t K, int64_t N, T *__restrict__ out, int64_t ld) {
    __shared__ int8_t tile[32][33];
    const int64_t k0 = (int64_t)blockIdx.y * 32, n0 = (int64_t)blockIdx.x * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int64_t k = k0 + j, n = n0 + threadIdx.x;
        tile[j][threadIdx.x] = (k < K && n < N) ? B[k * N + n] : (int8_t)0;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int64_t n = n0 + j, k = k0 + threadIdx.x;
        if (n < N && k < K)
            out[n * ld + k] = from_f32<T>(__fmul_rn((float)tile[threadIdx.x][j], __fdiv_rn(__ldg(col_s + n), 127.0f)));
    }
}

// The same through a 64 x 64 tile: 16-byte loads along n, 16-byte stores along k (16-bit output only).
// Needs N % 16 == 0, K % 8 == 0, B and out 16-byte aligned, ld % 8 == 0.
template <typename T>
__global__ void __launch_bounds__(256) dequantize_i8_transposed64_kernel(const int8_t *__restrict__ B, const float *__restrict__ col_s,
                                                                         int64_t K, int64_t N, T *__restrict__ out, int64_t ld) {
    static_assert(sizeof(T) == 2, "16-bit output");
    __shared__ __align__(16) int8_t tile[64][80];               // pitch 80: rows stay 16-byte aligned
    const int64_t k0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
    const int t = threadIdx.x;
    {
        const int kr = t >> 2, nc = (t & 3) * 16;               // 64 rows x 4 chunks of 16 columns
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (k0 + kr < K && n0 + nc < N) v = __ldg(reinterpret_cast<const uint4 *>(B + (k0 + kr) * N + n0 + nc));
        *reinterpret_cast<uint4 *>(&tile[kr][nc]) = v;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int id = t + 256 * j;                             // 64 columns x 8 chunks of 8 k
        const int nn = id >> 3, kc = (id & 7) * 8;
        const int64_t n = n0 + nn, k = k0 + kc;
        if (n < N && k < K) {
            const float f = __fdiv_rn(__ldg(col_s + n), 127.0f);
            __align__(16) T vals[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) vals[e] = from_f32<T>(__fmul_rn((float)tile[kc + e][nn], f));
            *reinterpret_cast<uint4 *>(out + n * ld + k) = *reinterpret_cast<const uint4 *>(vals);
        }
    }
}

template <typename T>
__global__ void copy_rows_kernel(const T *__restrict__ src, int64_t rows, int64_t cols, T *__restrict__ dst, int64_t ld) {
    const int64_t total = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols;
        dst[r * ld + (i - r * cols)] = src[i];
    }
}

int dequantize_i8_ld(const int8_t *q, int64_t rows, int64_t cols, const float *row_s, const float *col_s, void *out,
                     int64_t ld, int out_dtype, cudaStream_t st) {
    if (expand16_ok(q, cols, out, ld, col_s)) {
        const uint8_t *src = reinterpret_cast<const uint8_t *>(q);
        if (col_s == nullptr)
            MPSBNB_DISPATCH_DTYPE(out_dtype, T, (expand16_kernel<T, 0><<<grid_1d(rows * cols / 16), 256, 0, st>>>(src, rows, cols, row_s, nullptr, (T *)out, ld)));
        else
            MPSBNB_DISPATCH_DTYPE(out_dtype, T, (expand16_kernel<T, 2><<<grid_1d(rows * cols / 16), 256, 0, st>>>(src, rows, cols, row_s, col_s, (T *)out, ld)));
        return check_launch();
    }
    if (col_s == nullptr)
        MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize_i8_kernel<T, 0><<<grid_1d(rows * cols), 256, 0, st>>>(
                                                q, rows, cols, row_s, nullptr, (T *)out, ld)));
    else
        MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize_i8_kernel<T, 2><<<grid_1d(rows * cols), 256, 0, st>>>(
                                                q, rows, cols, row_s, col_s, (T *)out, ld)));
    return check_launch();
}

int dequantize_i8_transposed_ld(const int8_t *B, const float *col_s, int64_t K, int64_t N, void *out, int64_t ld,
                                int out_dtype, cudaStream_t st) {
    if (is_16bit(out_dtype) && N % 16 == 0 && K % 8 == 0 && ld % 8 == 0 && aligned16(B) && aligned16(out)) {
        const dim3 grid64((unsigned)((N + 63) / 64), (unsigned)((K + 63) / 64));
        if (out_dtype == MPSBNB_F16) dequantize_i8_transposed64_kernel<__half><<<grid64, 256, 0, st>>>(B, col_s, K, N, (__half *)out, ld);
        else dequantize_i8_transposed64_kernel<__nv_bfloat16><<<grid64, 256, 0, st>>>(B, col_s, K, N, (__nv_bfloat16 *)out, ld);
        return check_launch();
    }
    const dim3 grid((unsigned)((N + 31) / 32), (unsigned)((K + 31) / 32)), block(32, 8);
    MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize_i8_transposed_kernel<T><<<grid, block, 0, st>>>(B, col_s, K, N, (T *)out, ld)));
    return check_launch();
}

int dequantize_fp8_ld(const uint8_t *codes, const float *scales, int64_t rows, int64_t cols, void *out, int64_t ld,
                      int out_dtype, cudaStream_t st) {
    if (expand16_ok(codes, cols, out, ld, nullptr)) {
        MPSBNB_DISPATCH_DTYPE(out_dtype, T, (expand16_kernel<T, 3><<<grid_1d(rows * cols / 16), 256, 0, st>>>(codes, rows, cols, scales, nullptr, (T *)out, ld)));
        return check_launch();
    }
    MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize_fp8_kernel<T><<<grid_1d(rows * cols), 256, 0, st>>>(
                                            codes, scales, rows, cols, (T *)out, ld)));
    return check_launch();
}

int copy_rows_16bit_ld(const void *src, int64_t rows, int64_t cols, void *dst, int64_t ld, cudaStream_t st) {
    copy_rows_kernel<uint16_t><<<grid_1d(rows * cols), 256, 0, st>>>((const uint16_t *)src, rows, cols, (uint16_t *)dst, ld);
    return check_launch();
}

}  // namespace mpsbnb

using namespace mpsbnb;

extern "C" int mpsbnb_quantize_rowwise(const void *x, int x_dtype, int64_t rows, int64_t cols, int8_t *q,
                                       float *scales, void *stream) {
    if (!valid_dtype(x_dtype) || rows < 0 || cols < 0) return MPSBNB_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return MPSBNB_OK;
    if (x == nullptr || q == nullptr || scales == nullptr) return MPSBNB_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int g = (int)(rows < (int64_t)sm_count() * 16 ? rows : (int64_t)sm_count() * 16);
    MPSBNB_DISPATCH_DTYPE(x_dtype, T, (row_absmax_kernel<T><<<g, 256, 0, st>>>((const T *)x, rows, cols, scales, 1e-8f)));
    MPSBNB_DISPATCH_DTYPE(x_dtype, T, (quantize_i8_kernel<T, 0><<<grid_1d(rows * cols), 256, 0, st>>>(
                                          (const T *)x, rows, cols, scales, nullptr, q)));
    return check_launch();
}

extern "C" int mpsbnb_dequantize_rowwise(const int8_t *q, const float *scales, int64_t rows, int64_t cols,
                                         void *out, int out_dtype, void *stream) {
    if (!valid_dtype(out_dtype) || rows < 0 || cols < 0) return MPSBNB_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return MPSBNB_OK;
    if (q == nullptr || scales == nullptr || out == nullptr) return MPSBNB_ERR_INVALID_ARG;
    MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize_i8_kernel<T, 0><<<grid_1d(rows * cols), 256, 0, (cudaStream_t)stream>>>(
                                            q, rows, cols, scales, nullptr, (T *)out, cols)));
    return check_launch();
}

__global__ void dequant_absmax_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales, int64_t rows,
                                      int64_t nblk, int64_t ndq, int blocksize, float *__restrict__ out) {
    const int64_t total = rows * nblk;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / nblk, b = i - r * nblk;
        out[i] = __fmul_rn((float)q[i], scales[r * ndq + b / blocksize]);
    }
}

extern "C" int mpsbnb_dequant_absmax(const int8_t *q, const float *scales, int64_t rows, int64_t nblk, int64_t ndq,
                                     int blocksize, float *out, void *stream) {
    if (rows < 0 || nblk < 0 || blocksize <= 0) return MPSBNB_ERR_INVALID_ARG;
    if (rows == 0 || nblk == 0) return MPSBNB_OK;
    if (q == nullptr || scales == nullptr || out == nullptr || ndq < (nblk + blocksize - 1) / blocksize) return MPSBNB_ERR_INVALID_ARG;
    dequant_absmax_kernel<<<grid_1d(rows * nblk), 256, 0, (cudaStream_t)stream>>>(q, scales, rows, nblk, ndq, blocksize, out);
    return check_launch();
}

extern "C" int mpsbnb_double_quant(const void *A, int a_dtype, int64_t rows, int64_t cols,
                                   const float *row_stats_in, const float *col_stats_in, int8_t *out_row,
                                   int8_t *out_col, float *row_stats_out, float *col_stats_out, void *stream) {
    if (!valid_dtype(a_dtype) || rows < 0 || cols < 0) return MPSBNB_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return MPSBNB_OK;
    if (A == nullptr) return MPSBNB_ERR_INVALID_ARG;
    if ((row_stats_in == nullptr && row_stats_out == nullptr) || (col_stats_in == nullptr && col_stats_out == nullptr))
        return MPSBNB_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const float *rs = row_stats_in, *cs = col_stats_in;
    if (rs == nullptr) {
        const int g = (int)(rows < (int64_t)sm_count() * 16 ? rows : (int64_t)sm_count() * 16);
        MPSBNB_DISPATCH_DTYPE(a_dtype, T, (row_absmax_kernel<T><<<g, 256, 0, st>>>((const T *)A, rows, cols, row_stats_out, 1e-8f)));
        rs = row_stats_out;
    }
    if (cs == nullptr) {
        int rc = MPSBNB_OK;
        MPSBNB_DISPATCH_DTYPE(a_dtype, T, (rc = launch_col_absmax<T>((const T *)A, rows, cols, col_stats_out, st)));
        if (rc != MPSBNB_OK) return rc;
        cs = col_stats_out;
    }
    if (out_row != nullptr)
        MPSBNB_DISPATCH_DTYPE(a_dtype, T, (quantize_i8_kernel<T, 0><<<grid_1d(rows * cols), 256, 0, st>>>(
                                              (const T *)A, rows, cols, rs, cs, out_row)));
    if (out_col != nullptr)
        MPSBNB_DISPATCH_DTYPE(a_dtype, T, (quantize_i8_kernel<T, 1><<<grid_1d(rows * cols), 256, 0, st>>>(
                                              (const T *)A, rows, cols, rs, cs, out_col)));
    return check_launch();
}

extern "C" int mpsbnb_quantize_colrow(const void *W, int w_dtype, int64_t rows, int64_t cols, int8_t *q,
                                      float *row_absmax, float *col_absmax, void *stream) {
    if (!valid_dtype(w_dtype) || rows < 0 || cols < 0) return MPSBNB_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return MPSBNB_OK;
    if (W == nullptr || q == nullptr || row_absmax == nullptr || col_absmax == nullptr) return MPSBNB_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int g = (int)(rows < (int64_t)sm_count() * 16 ? rows : (int64_t)sm_count() * 16);
    MPSBNB_DISPATCH_DTYPE(w_dtype, T, (row_absmax_kernel<T><<<g, 256, 0, st>>>((const T *)W, rows, cols, row_absmax, 1e-8f)));
    int rc = MPSBNB_OK;
    MPSBNB_DISPATCH_DTYPE(w_dtype, T, (rc = launch_col_absmax<T>((const T *)W, rows, cols, col_absmax, st)));
    if (rc != MPSBNB_OK) return rc;
    MPSBNB_DISPATCH_DTYPE(w_dtype, T, (quantize_i8_kernel<T, 2><<<grid_1d(rows * cols), 256, 0, st>>>(
                                          (const T *)W, rows, cols, row_absmax, col_absmax, q)));
    return check_launch();
}

extern "C" int mpsbnb_dequantize_colrow(const int8_t *q, const float *row_scales, const float *col_scales,
                                        int64_t rows, int64_t cols, void *out, int out_dtype, void *stream) {
    if (!valid_dtype(out_dtype) || rows < 0 || cols < 0) return MPSBNB_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return MPSBNB_OK;
    if (q == nullptr || row_scales == nullptr || col_scales == nullptr || out == nullptr) return MPSBNB_ERR_INVALID_ARG;
    MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize_i8_kernel<T, 2><<<grid_1d(rows * cols), 256, 0, (cudaStream_t)stream>>>(
                                            q, rows, cols, row_scales, col_scales, (T *)out, cols)));
    return check_launch();
}

extern "C" int mpsbnb_quantize_fp8_e4m3(const void *x, int x_dtype, int64_t rows, int64_t cols, uint8_t *codes,
                                        float *scales, void *stream) {
    if (!valid_dtype(x_dtype) || rows < 0 || cols < 0) return MPSBNB_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return MPSBNB_OK;
    if (x == nullptr || codes == nullptr || scales == nullptr) return MPSBNB_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int g = (int)(rows < (int64_t)sm_count() * 16 ? rows : (int64_t)sm_count() * 16);
    MPSBNB_DISPATCH_DTYPE(x_dtype, T, (row_absmax_kernel<T><<<g, 256, 0, st>>>((const T *)x, rows, cols, scales, 0.0f)));
    fp8_scales_kernel<<<grid_1d(rows), 256, 0, st>>>(scales, rows);
    MPSBNB_DISPATCH_DTYPE(x_dtype, T, (quantize_fp8_kernel<T><<<grid_1d(rows * cols), 256, 0, st>>>(
                                          (const T *)x, rows, cols, scales, codes)));
    return check_launch();
}

extern "C" int mpsbnb_dequantize_fp8_e4m3(const uint8_t *codes, const float *scales, int64_t rows, int64_t cols,
                                          void *out, int out_dtype, void *stream) {
    if (!valid_dtype(out_dtype) || rows < 0 || cols < 0) return MPSBNB_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return MPSBNB_OK;
    if (codes == nullptr || scales == nullptr || out == nullptr) return MPSBNB_ERR_INVALID_ARG;
    MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize_fp8_kernel<T><<<grid_1d(rows * cols), 256, 0, (cudaStream_t)stream>>>(
                                            codes, scales, rows, cols, (T *)out, cols)));
    return check_launch();
}
