// Internal (non-ABI) entry points shared between translation units.
#pragma once
#include "common.cuh"

namespace mpsbnb {

int dequantize_4bit_ld(const uint8_t *packed, const void *absmax, const float *absmax2, int64_t rows, int64_t cols,
                       int blocksize, int quant_type, void *out, int64_t ld, int out_dtype, cudaStream_t st);
int dequantize_i8_ld(const int8_t *q, int64_t rows, int64_t cols, const float *row_s, const float *col_s, void *out,
                     int64_t ld, int out_dtype, cudaStream_t st);
int dequantize_i8_transposed_ld(const int8_t *B, const float *col_s, int64_t K, int64_t N, void *out, int64_t ld,
                                int out_dtype, cudaStream_t st);
int dequantize_fp8_ld(const uint8_t *codes, const float *scales, int64_t rows, int64_t cols, void *out, int64_t ld,
                      int out_dtype, cudaStream_t st);
int copy_rows_16bit_ld(const void *src, int64_t rows, int64_t cols, void *dst, int64_t ld, cudaStream_t st);
int gemm_16bit(const void *a, int64_t lda, const void *b, int64_t ldb, int ab_dtype, int64_t M, int64_t N, int64_t K,
               const float *row_scale, const float *col_scale, const void *bias, int bias_dtype, void *y, int64_t ldy,
               int y_dtype, cudaStream_t st);

// fused dequantise-GEMM (gemm_wq.cu): mode 0 = 4-bit packed, 1 = int8 rows, 2 = FP8 E4M3 rows
bool gemm_wq_supported(const void *x, int64_t ldx, const void *wq, int64_t row_bytes);
int gemm_wq(int mode, const void *x, int64_t ldx, int x_dtype, int64_t M, const void *wq, int64_t row_bytes,
            const void *absmax, const float *absmax2, const float *wscale, float wscale_mul, int wscale_sqrt, int64_t N,
            int64_t K, int quant_type, const void *bias, void *y, int y_dtype, cudaStream_t st);
int scale_cols_16bit(const void *x, int64_t M, int64_t K, int64_t ldx, const float *c, void *out, int64_t ldo, int dtype,
                     cudaStream_t st);
int wq_status_fetch(int *out, bool reset);

int gemv4_stream_single(const void *x, int x_dtype, int64_t M, const uint8_t *packed, const void *absmax,
                        const float *absmax2, int64_t N, int64_t K, int quant_type, const void *bias, void *y,
                        int y_dtype, cudaStream_t st);
int stream_status_fetch(int *out, bool reset);

// tensor-path decode kernel (gemv4_tc.cu)
int gemv4_tc_single(const void *x, int x_dtype, int64_t M, const uint8_t *packed, const void *absmax,
                    const float *absmax2, int64_t N, int64_t K, int quant_type, const void *bias, void *y,
                    int y_dtype, cudaStream_t st);
size_t tc_plan_bytes(const mpsbnb_linear4_desc *descs, int n_linears);
int tc_plan(const mpsbnb_linear4_desc *descs, int n_linears, int64_t M, int x_dtype, int y_dtype, int quant_type,
            void *plan_dev, size_t plan_bytes, mpsbnb_group_plan *plan_out, cudaStream_t st);
int tc_run(const mpsbnb_group_plan *plan, cudaStream_t st);
int tc_status_fetch(int *out, bool reset);
int xchg_status_fetch(int *out, bool reset);   // exchange.cu

}  // namespace mpsbnb
