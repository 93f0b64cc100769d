// Prefill-shape tensor-core GEMM for sm_100a:  y[M,N] = a[M,K] . b[N,K]^T  (+ epilogue),
// 16-bit operands (fp16 / bf16), fp32 accumulation in tensor memory.
//
// One persistent CTA per SM, warp-specialised, 192 threads:
//   warp 0   TMA producer: cp.async.bulk.tensor loads of a 128 x 64 tile of a and a BN x 64
//            tile of b (128-byte swizzle) into a 4-stage shared-memory ring;
//   warp 1   MMA issuer: one elected thread issues tcgen05.mma (128 x BN x 16, kind::f16) four
//            times per stage, then tcgen05.commit to hand the stage back to the producer;
//   warps 2-5 epilogue: tcgen05.ld the fp32 accumulator (TMEM lane = output row), apply
//            row/column scales and bias, round, and store.
// The accumulator is double-buffered in TMEM (2 x BN columns of the 512), so the epilogue of
// tile i overlaps the main loop of tile i+1.  Tiles are walked M-fastest so that CTAs running
// at the same time share the same b (weight) tile through L2.
// Every mbarrier wait is bounded: on time-out the role records a status word, raises a
// CTA-wide abort flag and all roles fall through to the common exit, which frees TMEM.
#include "common.cuh"
#include "ops.cuh"
#include "sm100.cuh"

namespace mpsbnb {

using namespace sm100;

constexpr int BM = 128, BK = 64, STAGES = 4;
constexpr int GEMM_THREADS = 192;

static __device__ int g_device_status = 0;            // 0 = ok; set by a kernel whose bounded wait ran out

struct GemmEpilogue {
    const float *row_scale;                    // nullptr or [M]
    const float *col_scale;                    // nullptr or [N]
    const void *bias;                          // nullptr or [N] in operand dtype
    void *y;                                   // [M, ldy]
    int64_t ldy;
    int y_dtype;
    int bias_dtype;
    int M, N, K;
};

template <int BN>
struct GemmSmem {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], then tmem slot + abort flag
    static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
};

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const GemmEpilogue ep, int fmt) {
    extern __shared__ unsigned char smem_raw[];
    using S = GemmSmem<BN>;
    // the swizzled operand tiles need 1024-byte alignment; the launch reserves the slack
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + S::BAR_OFFSET;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + S::BAR_OFFSET + (2 * STAGES + 4) * 8);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (ep.M + BM - 1) / BM, tiles_n = (ep.N + BN - 1) / BN;
    const int ntiles = tiles_m * tiles_n;
    const int kblocks = (ep.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 4); }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {                                           // the MMA warp owns the TMEM allocation
        tmem_alloc(smem_u32((const void *)tmem_slot), 2 * BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tensormap(&tm_a);
            prefetch_tensormap(&tm_b);
            int stage = 0; uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < ntiles && !*abort_flag; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) { atomicExch(&g_device_status, 101); *abort_flag = 1; break; }
                    const uint32_t a_dst = smem_base + stage * S::STAGE_BYTES;
                    mbar_arrive_expect_tx(full_bar(stage), S::STAGE_BYTES);
                    tma_load_2d(a_dst, &tm_a, full_bar(stage), kb * BK, m0);
                    tma_load_2d(a_dst + S::A_BYTES, &tm_b, full_bar(stage), kb * BK, n0);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(fmt, BM, BN);
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            for (int tile = blockIdx.x; tile < ntiles && !*abort_flag; tile += gridDim.x) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag)) { atomicExch(&g_device_status, 102); *abort_flag = 1; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                bool ok = true;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) { atomicExch(&g_device_status, 103); *abort_flag = 1; ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + stage * S::STAGE_BYTES;
                    const uint64_t da = umma_desc_k_sw128(a_addr), db = umma_desc_k_sw128(a_addr + S::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)            // 16 elements = 32 bytes = 2 descriptor units
                        umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, kb > 0 || k > 0);
                    umma_commit(empty_bar(stage));               // frees the stage once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(tfull_bar(acc));                     // accumulator complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;                                  // TMEM lane quarter this warp may read
        int acc = 0; uint32_t acc_phase = 0;
        for (int tile = blockIdx.x; tile < ntiles && !*abort_flag; tile += gridDim.x) {
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) { atomicExch(&g_device_status, 104); *abort_flag = 1; break; }
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const float rs = (ep.row_scale != nullptr && row < ep.M) ? __ldg(ep.row_scale + row) : 1.0f;
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= ep.N) break;                      // warp-uniform
                uint32_t v[32];
                tmem_ld_32x32(t_row + (uint32_t)c0, v);
                tmem_ld_wait();
                if (row < ep.M) {
                    float f[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int col = n0 + c0 + j;
                        float x = __uint_as_float(v[j]) * rs;
                        if (col < ep.N) {
                            if (ep.col_scale != nullptr) x *= __ldg(ep.col_scale + col);
                            if (ep.bias != nullptr)
                                x += ep.bias_dtype == MPSBNB_F16 ? __half2float(reinterpret_cast<const __half *>(ep.bias)[col])
                                   : ep.bias_dtype == MPSBNB_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(ep.bias)[col])
                                                                  : reinterpret_cast<const float *>(ep.bias)[col];
                        }
                        f[j] = x;
                    }
                    const int64_t off = (int64_t)row * ep.ldy + n0 + c0;
                    const bool full = n0 + c0 + 32 <= ep.N;
                    if (ep.y_dtype == MPSBNB_F32) {
                        float *dst = reinterpret_cast<float *>(ep.y) + off;
                        if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<float4 *>(dst)[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
                        } else {
                            for (int j = 0; j < 32; ++j) if (n0 + c0 + j < ep.N) dst[j] = f[j];
                        }
                    } else {
                        uint32_t h[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (ep.y_dtype == MPSBNB_F16) {
                                const __half2 t2 = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
                                h[j] = *reinterpret_cast<const uint32_t *>(&t2);
                            } else {
                                const __nv_bfloat162 t2 = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
                                h[j] = *reinterpret_cast<const uint32_t *>(&t2);
                            }
                        }
                        uint16_t *dst = reinterpret_cast<uint16_t *>(ep.y) + off;
                        if (full && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                reinterpret_cast<uint4 *>(dst)[j] = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (n0 + c0 + j < ep.N) dst[j] = (uint16_t)(h[j >> 1] >> (16 * (j & 1)));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }

    // common exit: every role arrives here (also after a time-out), then TMEM is released
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * BN);
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D map over a row-major [rows, cols] 16-bit matrix with leading dimension ld (elements):
// box = 64 columns (128 bytes) x box_rows, 128-byte swizzle, zero fill outside.
static int make_map_16bit(CUtensorMap *map, const void *base, int dtype, int64_t rows, int64_t cols, int64_t ld,
                          int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return MPSBNB_ERR_NO_DEVICE;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = fn(map, dtype == MPSBNB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                          const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MPSBNB_OK : MPSBNB_ERR_INVALID_ARG;
}

template <int BN>
static int launch_gemm(const CUtensorMap &ma, const CUtensorMap &mb, const GemmEpilogue &ep, int fmt, cudaStream_t st) {
    using S = GemmSmem<BN>;
    constexpr int smem = S::TOTAL + 1024;                      // slack for the 1024-byte alignment of the ring
    static bool configured[64] = {};
    int dev = 0;
    MPSBNB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        MPSBNB_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int tiles = ((ep.M + BM - 1) / BM) * ((ep.N + BN - 1) / BN);
    int grid = sm_count();
    if (grid > tiles) grid = tiles;
    gemm_tc_kernel<BN><<<grid, GEMM_THREADS, smem, st>>>(ma, mb, ep, fmt);
    return check_launch();
}

// y[M,N] = a[M,K] (ld lda) . b[N,K]^T (ld ldb); lda, ldb multiples of 8 elements, bases 16-byte aligned.
int gemm_16bit(const void *a, int64_t lda, const void *b, int64_t ldb, int ab_dtype, int64_t M, int64_t N, int64_t K,
               const float *row_scale, const float *col_scale, const void *bias, int bias_dtype, void *y, int64_t ldy,
               int y_dtype, cudaStream_t st) {
    if (!is_16bit(ab_dtype) || !valid_dtype(y_dtype)) return MPSBNB_ERR_INVALID_ARG;
    if (M <= 0 || N <= 0) return MPSBNB_OK;
    if (K <= 0) return MPSBNB_ERR_UNSUPPORTED;
    if ((lda % 8) || (ldb % 8) || !aligned16(a) || !aligned16(b)) return MPSBNB_ERR_UNSUPPORTED;
    if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return MPSBNB_ERR_TOO_LARGE;
    GemmEpilogue ep;
    ep.row_scale = row_scale; ep.col_scale = col_scale; ep.bias = bias; ep.y = y; ep.ldy = ldy;
    ep.y_dtype = y_dtype; ep.bias_dtype = bias_dtype; ep.M = (int)M; ep.N = (int)N; ep.K = (int)K;
    // BN = 256 unless that leaves most SMs idle
    const int64_t tiles256 = ((M + BM - 1) / BM) * ((N + 255) / 256);
    const bool use128 = tiles256 < sm_count() && N > 128;
    const int bn = use128 ? 128 : 256;
    CUtensorMap ma, mb;
    int rc = make_map_16bit(&ma, a, ab_dtype, M, K, lda, BM);
    if (rc != MPSBNB_OK) return rc;
    rc = make_map_16bit(&mb, b, ab_dtype, N, K, ldb, bn);
    if (rc != MPSBNB_OK) return rc;
    const int fmt = ab_dtype == MPSBNB_F16 ? 0 : 1;
    return use128 ? launch_gemm<128>(ma, mb, ep, fmt, st) : launch_gemm<256>(ma, mb, ep, fmt, st);
}

}  // namespace mpsbnb

using namespace mpsbnb;

extern "C" int mpsbnb_device_status(int *status_out, int reset) {
    if (status_out == nullptr) return MPSBNB_ERR_INVALID_ARG;
    MPSBNB_CUDA_TRY(cudaMemcpyFromSymbol(status_out, g_device_status, sizeof(int)));
    if (reset) {
        const int zero = 0;
        MPSBNB_CUDA_TRY(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    }
    int other = 0;
    const int rc = stream_status_fetch(&other, reset != 0);
    if (rc != MPSBNB_OK) return rc;
    if (*status_out == 0) *status_out = other;
    const int rc2 = tc_status_fetch(&other, reset != 0);
    if (rc2 != MPSBNB_OK) return rc2;
    if (*status_out == 0) *status_out = other;
    const int rc3 = xchg_status_fetch(&other, reset != 0);
    if (rc3 != MPSBNB_OK) return rc3;
    if (*status_out == 0) *status_out = other;
    const int rc4 = wq_status_fetch(&other, reset != 0);
    if (rc4 != MPSBNB_OK) return rc4;
    if (*status_out == 0) *status_out = other;
    return MPSBNB_OK;
}

extern "C" int mpsbnb_gemm_f16(const void *a, int64_t lda, const void *b, int64_t ldb, int ab_dtype, int64_t M,
                               int64_t N, int64_t K, const float *row_scale, const float *col_scale,
                               const void *bias, void *y, int y_dtype, void *stream) {
    if (a == nullptr || b == nullptr || y == nullptr) return (M <= 0 || N <= 0) ? MPSBNB_OK : MPSBNB_ERR_INVALID_ARG;
    return gemm_16bit(a, lda, b, ldb, ab_dtype, M, N, K, row_scale, col_scale, bias, ab_dtype, y, N, y_dtype,
                      (cudaStream_t)stream);
}
