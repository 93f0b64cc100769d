// Prefill-shape linear layers over quantised weights.  Default: the fused kernel of gemm_wq.cu
// (quantised bytes by TMA, expanded in shared memory, tcgen05 MMA) - no 16-bit copy of the weight
// exists anywhere.  Layouts the fused kernel cannot take (block size other than 64, row pitches
// that are not multiples of 16 bytes, the K x N int8 operand of matmul_int8) are expanded once into
// the caller's workspace in the operand type, as the reference's CPU path materialises the weight
// (mps_bitsandbytes/functional.py:756, 791-792, 800, 940), and multiplied by the plain tcgen05
// GEMM.  Matrices whose K is not a multiple of 8 get a padded leading dimension (TMA needs
// 16-byte row pitches); the pad is never read as data because the tensor map's extent stays K.
#include "ops.cuh"

namespace mpsbnb {

static inline int64_t ld8(int64_t k) { return (k + 7) / 8 * 8; }
static inline size_t align256(size_t b) { return (b + 255) / 256 * 256; }

// bytes for a [rows, ld8(K)] 16-bit matrix
static inline size_t mat_bytes(int64_t rows, int64_t K) { return align256((size_t)rows * (size_t)ld8(K) * 2); }

// x as a GEMM operand: the caller's buffer when its pitch and base suit TMA, else a padded copy.
static int stage_x(const void *x, int64_t M, int64_t K, unsigned char *&ws, const void *&xa, int64_t &lda,
                   cudaStream_t st) {
    if (K % 8 == 0 && aligned16(x)) { xa = x; lda = K; return MPSBNB_OK; }
    lda = ld8(K);
    int rc = copy_rows_16bit_ld(x, M, K, ws, lda, st);
    xa = ws;
    ws += mat_bytes(M, K);
    return rc;
}

}  // namespace mpsbnb

using namespace mpsbnb;

extern "C" size_t mpsbnb_gemm_4bit_workspace_bytes(int64_t M, int64_t N, int64_t K, int blocksize) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    // block size 64: the fused kernel needs room only for a re-pitched copy of x (used when K % 8 != 0 or x is
    // not 16-byte aligned); other block sizes expand the whole weight
    return (blocksize == 64 ? 0 : mat_bytes(N, K)) + mat_bytes(M, K);
}

extern "C" int mpsbnb_gemm_4bit(const void *x, int x_dtype, int64_t M, const uint8_t *packed, const void *absmax,
                                const float *absmax2, int64_t N, int64_t K, int blocksize, int quant_type,
                                const void *bias, void *y, int y_dtype, void *workspace, size_t workspace_bytes,
                                void *stream) {
    if (!is_16bit(x_dtype) || !valid_dtype(y_dtype)) return MPSBNB_ERR_INVALID_ARG;
    if (M < 0 || N < 0 || K <= 0) return K == 0 && M >= 0 && N >= 0 ? MPSBNB_ERR_UNSUPPORTED : MPSBNB_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return MPSBNB_OK;
    if (x == nullptr || packed == nullptr || absmax == nullptr || y == nullptr || workspace == nullptr)
        return MPSBNB_ERR_INVALID_ARG;
    if (workspace_bytes < mpsbnb_gemm_4bit_workspace_bytes(M, N, K, blocksize) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return MPSBNB_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned char *ws = reinterpret_cast<unsigned char *>(workspace);
    if (blocksize == 64) {
        if (!aligned16(packed)) return MPSBNB_ERR_UNSUPPORTED;       // TMA reads the packed rows
        const void *xa; int64_t lda;
        int rc = stage_x(x, M, K, ws, xa, lda, st);
        if (rc != MPSBNB_OK) return rc;
        return gemm_wq(0, xa, lda, x_dtype, M, packed, padded_k(K, 64) / 2, absmax, absmax2, nullptr, 1.0f, 0, N, K,
                       quant_type, bias, y, y_dtype, st);
    }
    void *w = ws;
    ws += mat_bytes(N, K);
    int rc = dequantize_4bit_ld(packed, absmax, absmax2, N, K, blocksize, quant_type, w, ld8(K), x_dtype, st);
    if (rc != MPSBNB_OK) return rc;
    const void *xa; int64_t lda;
    rc = stage_x(x, M, K, ws, xa, lda, st);
    if (rc != MPSBNB_OK) return rc;
    return gemm_16bit(xa, lda, w, ld8(K), x_dtype, M, N, K, nullptr, nullptr, bias, x_dtype, y, N, y_dtype, st);
}

extern "C" size_t mpsbnb_matmul_int8_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return mat_bytes(M, K) + mat_bytes(N, K);
}

extern "C" int mpsbnb_matmul_int8(const int8_t *A, const int8_t *B, const float *a_scales, const float *b_scales,
                                  int64_t M, int64_t N, int64_t K, void *y, int y_dtype, void *workspace,
                                  size_t workspace_bytes, void *stream) {
    if (!valid_dtype(y_dtype) || M < 0 || N < 0 || K <= 0) return MPSBNB_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return MPSBNB_OK;
    if (A == nullptr || B == nullptr || a_scales == nullptr || b_scales == nullptr || y == nullptr || workspace == nullptr)
        return MPSBNB_ERR_INVALID_ARG;
    if (workspace_bytes < mpsbnb_matmul_int8_workspace_bytes(M, N, K) || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return MPSBNB_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    // operands are dequantised to the output type as the reference does (fp32 output -> fp16 operands)
    const int op = y_dtype == MPSBNB_BF16 ? MPSBNB_BF16 : MPSBNB_F16;
    unsigned char *ws = reinterpret_cast<unsigned char *>(workspace);
    void *a = ws;
    void *bt = ws + mat_bytes(M, K);
    int rc = dequantize_i8_ld(A, M, K, a_scales, nullptr, a, ld8(K), op, st);
    if (rc != MPSBNB_OK) return rc;
    if (N % 16 == 0 && aligned16(B))
        // fused: B is brought in as it is stored (K x N), transposed and widened exactly inside the GEMM; its
        // column scale (and 1 / 127) multiplies the fp32 accumulator
        return gemm_wq(3, a, ld8(K), op, M, B, N, nullptr, nullptr, b_scales, 1.0f / 127.0f, 0, N, K, 0, nullptr, y, y_dtype, st);
    rc = dequantize_i8_transposed_ld(B, b_scales, K, N, bt, ld8(K), op, st);
    if (rc != MPSBNB_OK) return rc;
    return gemm_16bit(a, ld8(K), bt, ld8(K), op, M, N, K, nullptr, nullptr, nullptr, op, y, N, y_dtype, st);
}

extern "C" size_t mpsbnb_linear_int8_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return mat_bytes(N, K) + mat_bytes(M, K);
}

extern "C" int mpsbnb_linear_int8(const void *x, int x_dtype, int64_t M, const int8_t *W, const float *row_scales,
                                  const float *col_scales, int64_t N, int64_t K, const void *bias, void *y,
                                  int y_dtype, void *workspace, size_t workspace_bytes, void *stream) {
    if (!is_16bit(x_dtype) || !valid_dtype(y_dtype) || M < 0 || N < 0 || K <= 0) return MPSBNB_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return MPSBNB_OK;
    if (x == nullptr || W == nullptr || row_scales == nullptr || y == nullptr || workspace == nullptr)
        return MPSBNB_ERR_INVALID_ARG;
    if (workspace_bytes < mpsbnb_linear_int8_workspace_bytes(M, N, K) || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return MPSBNB_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned char *ws = reinterpret_cast<unsigned char *>(workspace);
    if (K % 16 == 0 && aligned16(W) && aligned16(x)) {
        // fused: int8 -> 16-bit exactly inside the GEMM; the row scale (and 1 / 127) multiplies the fp32
        // accumulator; the column half sqrt(c[k]) of a col+row scale is moved onto x
        const void *xa = x;
        if (col_scales != nullptr) {
            int rc = scale_cols_16bit(x, M, K, K, col_scales, ws, K, x_dtype, st);
            if (rc != MPSBNB_OK) return rc;
            xa = ws;
        }
        return gemm_wq(1, xa, K, x_dtype, M, W, K, nullptr, nullptr, row_scales, 1.0f / 127.0f, col_scales != nullptr ? 1 : 0,
                       N, K, 0, bias, y, y_dtype, st);
    }
    void *w = ws;
    ws += mat_bytes(N, K);
    int rc = dequantize_i8_ld(W, N, K, row_scales, col_scales, w, ld8(K), x_dtype, st);
    if (rc != MPSBNB_OK) return rc;
    const void *xa; int64_t lda;
    rc = stage_x(x, M, K, ws, xa, lda, st);
    if (rc != MPSBNB_OK) return rc;
    return gemm_16bit(xa, lda, w, ld8(K), x_dtype, M, N, K, nullptr, nullptr, bias, x_dtype, y, N, y_dtype, st);
}

extern "C" size_t mpsbnb_linear_fp8_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    return mpsbnb_linear_int8_workspace_bytes(M, N, K);
}

extern "C" int mpsbnb_linear_fp8_e4m3(const void *x, int x_dtype, int64_t M, const uint8_t *codes, const float *scales,
                                      int64_t N, int64_t K, const void *bias, void *y, int y_dtype, void *workspace,
                                      size_t workspace_bytes, void *stream) {
    if (!is_16bit(x_dtype) || !valid_dtype(y_dtype) || M < 0 || N < 0 || K <= 0) return MPSBNB_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return MPSBNB_OK;
    if (x == nullptr || codes == nullptr || scales == nullptr || y == nullptr || workspace == nullptr)
        return MPSBNB_ERR_INVALID_ARG;
    if (workspace_bytes < mpsbnb_linear_fp8_workspace_bytes(M, N, K) || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return MPSBNB_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned char *ws = reinterpret_cast<unsigned char *>(workspace);
    if (K % 16 == 0 && aligned16(codes) && aligned16(x))
        return gemm_wq(2, x, K, x_dtype, M, codes, K, nullptr, nullptr, scales, 1.0f, 0, N, K, 0, bias, y, y_dtype, st);
    void *w = ws;
    ws += mat_bytes(N, K);
    int rc = dequantize_fp8_ld(codes, scales, N, K, w, ld8(K), x_dtype, st);
    if (rc != MPSBNB_OK) return rc;
    const void *xa; int64_t lda;
    rc = stage_x(x, M, K, ws, xa, lda, st);
    if (rc != MPSBNB_OK) return rc;
    return gemm_16bit(xa, lda, w, ld8(K), x_dtype, M, N, K, nullptr, nullptr, bias, x_dtype, y, N, y_dtype, st);
}
