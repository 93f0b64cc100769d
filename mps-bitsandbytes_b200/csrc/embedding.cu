// Quantised embedding look-ups: gather rows of a 4-bit (NF4 / FP4, blockwise absmax) or an
// int8 (row-scaled) table and expand them in the same pass.  Stands for the reference's
// Embedding4bit / Embedding8bit forward (mps_bitsandbytes/nn/embedding.py:78-139, 244-275;
// Metal bindings _C.embedding_4bit_nf4 / _fp4 / embedding_8bit), with the arithmetic of its
// Python path, which is the one the CPU oracle follows:
//   4-bit: out = code[nibble] * absmax[row, k / blocksize] in fp32, rounded once to the output type
//          (functional.py:388-416 on a single row);
//   8-bit: out = T(q) * T(scale / 127)  — the scale is rounded to the output type FIRST
//          (embedding.py:269), unlike dequantize_rowwise.
// Rows equal to padding_idx come out as zeros (embedding.py:135-137, 271-273).  Indices outside
// [0, num_embeddings) also give zero rows: a kernel cannot raise, and it must not fault.
//
// Bound: HBM.  Per looked-up row D/2 + 4 D/blocksize bytes read and D * sizeof(T) written
// (4-bit); D + 4 read and D * sizeof(T) written (8-bit).
#include "common.cuh"

namespace mpsbnb {

__device__ __forceinline__ int64_t load_index(const void *idx, int idx64, int64_t t) {
    return idx64 ? reinterpret_cast<const int64_t *>(idx)[t] : (int64_t) reinterpret_cast<const int32_t *>(idx)[t];
}

// Fast path: D % 16 == 0, blocksize % 16 == 0, packed pitch % 8 == 0, out 16-byte aligned.
// One thread expands 8 packed bytes (16 codes, all of one block) of one looked-up row.
template <typename T>
__global__ void __launch_bounds__(256) embedding4_vec_kernel(const void *__restrict__ idx, int idx64, int64_t n_idx,
                                                             const uint8_t *__restrict__ packed, int64_t packed_ld,
                                                             const float *__restrict__ absmax, int64_t nb, int64_t V,
                                                             int64_t D, int blocksize, int qt, int64_t padding_idx,
                                                             T *__restrict__ out) {
    __shared__ float code[16];
    if (threadIdx.x < 16) code[threadIdx.x] = kCode[qt][threadIdx.x];
    __syncthreads();
    const int64_t chunks = D / 16;
    const int64_t total = n_idx * chunks;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t t, c;                                              // 32-bit division where the sizes allow it
        if (total < 0x7fffffffll) { const uint32_t t32 = (uint32_t)i / (uint32_t)chunks; t = t32; c = (uint32_t)i - t32 * (uint32_t)chunks; }
        else { t = i / chunks; c = i - t * chunks; }
        const int64_t row = load_index(idx, idx64, t);
        __align__(16) T vals[16];
        if (row < 0 || row >= V || row == padding_idx) {
#pragma unroll
            for (int e = 0; e < 16; ++e) vals[e] = from_f32<T>(0.0f);
        } else {
            const uint2 w = *reinterpret_cast<const uint2 *>(packed + row * packed_ld + c * 8);
            const float a = __ldg(absmax + row * nb + (c * 16) / blocksize);
            const uint32_t ww[2] = {w.x, w.y};
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const uint32_t nib = (ww[e >> 3] >> ((e & 7) * 4)) & 15u;     // low nibble = even k
                vals[e] = from_f32<T>(__fmul_rn(code[nib], a));
            }
        }
        uint4 *dst = reinterpret_cast<uint4 *>(out + t * D + c * 16);
        const uint4 *src = reinterpret_cast<const uint4 *>(vals);
#pragma unroll
        for (int v = 0; v < (int)(sizeof(T) * 16 / 16); ++v) __stcs(dst + v, src[v]);
    }
}

// General path: any even D, any block size, one element per thread.
template <typename T>
__global__ void __launch_bounds__(256) embedding4_kernel(const void *__restrict__ idx, int idx64, int64_t n_idx,
                                                         const uint8_t *__restrict__ packed, int64_t packed_ld,
                                                         const float *__restrict__ absmax, int64_t nb, int64_t V,
                                                         int64_t D, int blocksize, int qt, int64_t padding_idx,
                                                         T *__restrict__ out) {
    const int64_t total = n_idx * D;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / D, k = i - t * D;
        const int64_t row = load_index(idx, idx64, t);
        float v = 0.0f;
        if (row >= 0 && row < V && row != padding_idx) {
            const uint32_t b = packed[row * packed_ld + (k >> 1)];
            const uint32_t nib = (k & 1) ? (b >> 4) : (b & 15u);
            v = __fmul_rn(kCode[qt][nib], __ldg(absmax + row * nb + k / blocksize));
        }
        out[i] = from_f32<T>(v);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) embedding8_kernel(const void *__restrict__ idx, int idx64, int64_t n_idx,
                                                         const int8_t *__restrict__ q, const float *__restrict__ scales,
                                                         int64_t V, int64_t D, int64_t padding_idx, int vec,
                                                         T *__restrict__ out) {
    if (vec) {                                               // D % 16 == 0, q rows and out 16-byte aligned
        const int64_t chunks = D / 16, total = n_idx * chunks;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            int64_t t, c;
            if (total < 0x7fffffffll) { const uint32_t t32 = (uint32_t)i / (uint32_t)chunks; t = t32; c = (uint32_t)i - t32 * (uint32_t)chunks; }
            else { t = i / chunks; c = i - t * chunks; }
            const int64_t row = load_index(idx, idx64, t);
            __align__(16) T vals[16];
            if (row < 0 || row >= V || row == padding_idx) {
#pragma unroll
                for (int e = 0; e < 16; ++e) vals[e] = from_f32<T>(0.0f);
            } else {
                const uint4 w = *reinterpret_cast<const uint4 *>(q + row * D + c * 16);
                const float s = __fdiv_rn(__ldg(scales + row), 127.0f);
                const int8_t *b = reinterpret_cast<const int8_t *>(&w);
#pragma unroll
                for (int e = 0; e < 16; ++e) vals[e] = i8_times_rounded_scale<T>(b[e], s);
            }
            uint4 *dst = reinterpret_cast<uint4 *>(out + t * D + c * 16);
            const uint4 *src = reinterpret_cast<const uint4 *>(vals);
#pragma unroll
            for (int v = 0; v < (int)(sizeof(T) * 16 / 16); ++v) __stcs(dst + v, src[v]);
        }
        return;
    }
    const int64_t total = n_idx * D;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / D, k = i - t * D;
        const int64_t row = load_index(idx, idx64, t);
        T v = from_f32<T>(0.0f);
        if (row >= 0 && row < V && row != padding_idx) v = i8_times_rounded_scale<T>(q[row * D + k], __fdiv_rn(__ldg(scales + row), 127.0f));
        out[i] = v;
    }
}

static inline unsigned grid_for(int64_t work_items) {
    const int64_t ctas = (work_items + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;             // grid-stride beyond this
    return (unsigned)(ctas < 1 ? 1 : (ctas > cap ? cap : ctas));
}

}  // namespace mpsbnb

using namespace mpsbnb;

extern "C" int mpsbnb_embedding_4bit(const void *indices, int index_bytes, int64_t n_indices, const uint8_t *packed,
                                     int64_t packed_ld, const float *absmax, int64_t num_embeddings, int64_t dim,
                                     int blocksize, int quant_type, int64_t padding_idx, void *out, int out_dtype,
                                     void *stream) {
    if ((index_bytes != 4 && index_bytes != 8) || !valid_dtype(out_dtype) || (quant_type != MPSBNB_NF4 && quant_type != MPSBNB_FP4))
        return MPSBNB_ERR_INVALID_ARG;
    if (n_indices < 0 || num_embeddings < 0 || dim < 0 || (dim & 1) || blocksize <= 0 || packed_ld < dim / 2)
        return MPSBNB_ERR_INVALID_ARG;
    if (n_indices == 0 || dim == 0) return MPSBNB_OK;
    if (indices == nullptr || packed == nullptr || absmax == nullptr || out == nullptr) return MPSBNB_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t nb = (dim + blocksize - 1) / blocksize;
    const int idx64 = index_bytes == 8;
    const bool vec = dim % 16 == 0 && blocksize % 16 == 0 && packed_ld % 8 == 0 &&
                     (reinterpret_cast<uintptr_t>(packed) & 7) == 0 && aligned16(out);
    if (vec)
        MPSBNB_DISPATCH_DTYPE(out_dtype, T, (embedding4_vec_kernel<T><<<grid_for(n_indices * (dim / 16)), 256, 0, st>>>(
                                                indices, idx64, n_indices, packed, packed_ld, absmax, nb, num_embeddings,
                                                dim, blocksize, quant_type, padding_idx, (T *)out)));
    else
        MPSBNB_DISPATCH_DTYPE(out_dtype, T, (embedding4_kernel<T><<<grid_for(n_indices * dim), 256, 0, st>>>(
                                                indices, idx64, n_indices, packed, packed_ld, absmax, nb, num_embeddings,
                                                dim, blocksize, quant_type, padding_idx, (T *)out)));
    return check_launch();
}

extern "C" int mpsbnb_embedding_8bit(const void *indices, int index_bytes, int64_t n_indices, const int8_t *q,
                                     const float *scales, int64_t num_embeddings, int64_t dim, int64_t padding_idx,
                                     void *out, int out_dtype, void *stream) {
    if ((index_bytes != 4 && index_bytes != 8) || !valid_dtype(out_dtype)) return MPSBNB_ERR_INVALID_ARG;
    if (n_indices < 0 || num_embeddings < 0 || dim < 0) return MPSBNB_ERR_INVALID_ARG;
    if (n_indices == 0 || dim == 0) return MPSBNB_OK;
    if (indices == nullptr || q == nullptr || scales == nullptr || out == nullptr) return MPSBNB_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int vec = dim % 16 == 0 && aligned16(q) && aligned16(out);
    MPSBNB_DISPATCH_DTYPE(out_dtype, T, (embedding8_kernel<T><<<grid_for(vec ? n_indices * (dim / 16) : n_indices * dim), 256, 0, st>>>(
                                            indices, index_bytes == 8, n_indices, q, scales, num_embeddings, dim,
                                            padding_idx, vec, (T *)out)));
    return check_launch();
}
