// Blockwise 4-bit (NF4 / FP4) quantise + pack, dequantise, and the blockwise int8
// quantiser used for double quantisation of absmax.  All results are bit-identical to the
// reference's CPU path (mps_bitsandbytes/functional.py:163-600).
//
// Quantise, fast path (16-bit input, block size 32..256, K % 8 == 0): every thread owns 8
// consecutive elements (one 128-bit load), the bs/8 threads of a block reduce |x| with
// warp shuffles, and each thread emits 4 packed bytes (one 32-bit store).  The nearest
// code is found with 4 comparisons against decision thresholds instead of the reference's
// 16-way |v - code| search; the thresholds are the exact floats at which the rounded
// 16-way search changes its answer (ties included), and v = x / absmax is produced by a
// reciprocal, a multiply and two fused corrections.  Both shortcuts are proven equal to
// the reference arithmetic for every (x, absmax) pair of fp16 and of bf16 by
// oracle/oracle.c:o_prove_quantizer with block maxima in [1e-30, 1e30]; fp32 input and maxima
// outside that range use IEEE division.
#include "common.cuh"

namespace mpsbnb {

// Largest v for which code i (and not i+1) is the first minimiser of |v - code|:
// derived by oracle/oracle.c:o_nf4_thresholds, checked by tests/test_cpu_library.py.
#define NF4_T0 -0x1.b239b2p-1f
#define NF4_T1 -0x1.38a4e2p-1f
#define NF4_T2 -0x1.d709p-2f
#define NF4_T3 -0x1.5bd4eep-2f
#define NF4_T4 -0x1.e079dap-3f
#define NF4_T5 -0x1.1a7178p-3f
#define NF4_T6 -0x1.74f0e2p-5f
#define NF4_T7 0x1.45f5fep-5f
#define NF4_T8 0x1.ec90c4p-4f
#define NF4_T9 0x1.a0cfcp-3f
#define NF4_T10 0x1.2b05a8p-2f
#define NF4_T11 0x1.8ea7f2p-2f
#define NF4_T12 0x1.00da06p-1f
#define NF4_T13 0x1.491b5ep-1f
#define NF4_T14 0x1.b913b2p-1f
// FP4 works on |v|: magnitudes 0, 1/16, 1/8, 1/4, 3/8, 1/2, 3/4, 1; ties go to the smaller.
#define FP4_T0 0x1p-5f
#define FP4_T1 0x1.8p-4f
#define FP4_T2 0x1.8p-3f
#define FP4_T3 0x1.4p-2f
#define FP4_T4 0x1.cp-2f
#define FP4_T5 0x1.4p-1f
#define FP4_T6 0x1.cp-1f

__device__ __forceinline__ uint32_t nf4_code(float v) {
    uint32_t idx = v > NF4_T7 ? 8u : 0u;
    float t = idx ? NF4_T11 : NF4_T3;
    idx |= v > t ? 4u : 0u;
    t = (idx & 8u) ? ((idx & 4u) ? NF4_T13 : NF4_T9) : ((idx & 4u) ? NF4_T5 : NF4_T1);
    idx |= v > t ? 2u : 0u;
    const float ta = (idx & 2u) ? NF4_T2 : NF4_T0, tb = (idx & 2u) ? NF4_T6 : NF4_T4;
    const float tc = (idx & 2u) ? NF4_T10 : NF4_T8, td = (idx & 2u) ? NF4_T14 : NF4_T12;
    t = (idx & 8u) ? ((idx & 4u) ? td : tc) : ((idx & 4u) ? tb : ta);
    idx |= v > t ? 1u : 0u;
    return idx;
}

__device__ __forceinline__ uint32_t fp4_code(float v) {
    const float a = fabsf(v);
    uint32_t m = a > FP4_T3 ? 4u : 0u;
    float t = m ? FP4_T5 : FP4_T1;
    m |= a > t ? 2u : 0u;
    t = (m & 4u) ? ((m & 2u) ? FP4_T6 : FP4_T4) : ((m & 2u) ? FP4_T2 : FP4_T0);
    m |= a > t ? 1u : 0u;
    // negative values take codes 9..15; code 0 (+0.0) beats code 8 (-0.0) on the tie
    return (v < 0.0f && m != 0u) ? (m | 8u) : m;
}

template <int QT> __device__ __forceinline__ uint32_t code_of(float v) {
    return QT == MPSBNB_NF4 ? nf4_code(v) : fp4_code(v);
}

// NF4 search by buckets: [-1, 1] is cut into sixteen buckets of width 1/8; no bucket holds more than two of the
// fifteen thresholds, so the code is (thresholds below the bucket) + (v > first) + (v > second): one FMA, one
// conversion, one 8-byte shared load and two compares instead of four dependent compare-and-select levels.  The same
// thresholds decide, so the result is the binary search's; the bucket a value within rounding error of an edge lands
// in does not matter, because no threshold is closer than 1.7e-3 to an edge (oracle/oracle.c:o_prove_nf4_buckets
// checks every float).  tab[g] = the bucket's two thresholds (+inf where it has fewer).
#define NF4_INF __int_as_float(0x7f800000)
__device__ __forceinline__ void nf4_bucket_table_fill(float2 *tab, int g) {
    const float a[16] = {NF4_INF, NF4_T0, NF4_INF, NF4_T1, NF4_T2, NF4_T3, NF4_T4, NF4_T6, NF4_T7, NF4_T9, NF4_T10, NF4_T11, NF4_T12, NF4_T13, NF4_T14, NF4_INF};
    tab[g] = make_float2(a[g], g == 6 ? NF4_T5 : (g == 8 ? NF4_T8 : NF4_INF));
}
__device__ __forceinline__ uint32_t nf4_code_bucket(float v, const float2 *tab) {
    const int g = max(0, min(15, __float2int_rz(__fmaf_rn(v, 8.0f, 8.0f))));
    const float2 t = tab[g];
    // thresholds below bucket g, four bits each: 0 0 1 1 2 3 4 6 7 9 10 11 12 13 14 15
    const uint32_t base = (uint32_t)(0xFEDCBA9764321100ull >> (4 * g)) & 15u;
    return base + (v > t.x ? 1u : 0u) + (v > t.y ? 1u : 0u);
}
// The search of the streaming quantiser, for quotients in [-1, 1] (|x| <= absmax of its own block): 32 buckets of width
// 1/16, none of which holds more than one threshold; the bucket is the low six bits of fma_rz(v, 16, 2^23 + 16) =
// floor(16 v + 16) - no conversion, no clamp (32, reached by v = 1 only, carries bucket 31's entry) - and
// code = (thresholds below the bucket) + (v > the bucket's threshold, +inf if it has none).
// oracle/oracle.c:o_prove_nf4_buckets32_rz compares it with the threshold search on every float of [-1, 1].
// The table is replicated per lane - entry g of lane l at g * 256 + l * 8 bytes - so that a warp's 32 lookups are two
// conflict-free wavefronts whatever the values are (the shared-memory pipe, not arithmetic, bounds this kernel).
constexpr int NF4_B32_ENTRIES = 33;
constexpr int NF4_B32_BYTES = NF4_B32_ENTRIES * 256;
__device__ __forceinline__ void nf4_bucket32_fill(float2 *tab, int tid, int nthreads) {
    const float t[15] = {NF4_T0, NF4_T1, NF4_T2, NF4_T3, NF4_T4, NF4_T5, NF4_T6, NF4_T7, NF4_T8, NF4_T9, NF4_T10, NF4_T11, NF4_T12, NF4_T13, NF4_T14};
    for (int i = tid; i < NF4_B32_ENTRIES * 32; i += nthreads) {
        const int g = i >> 5, b = g < 32 ? g : 31;
        const float lo = -1.0f + (float)b * 0.0625f, hi = -1.0f + (float)(b + 1) * 0.0625f;   // exact
        int below = 0;
        float th = NF4_INF;
#pragma unroll
        for (int j = 0; j < 15; ++j) {
            if (t[j] < lo) ++below;
            else if (t[j] < hi) th = t[j];
        }
        tab[i] = make_float2(th, __int_as_float(below));
    }
}
__device__ __forceinline__ uint32_t nf4_code_bucket32(float v, uint32_t tab_lane) {   // tab_lane: shared address of the table + lane * 8
    const uint32_t bits = __float_as_uint(__fmaf_rz(v, 16.0f, 8388624.0f));
    float th; uint32_t base;
    // bits = 0x4B000000 + bucket: shifted left by 8 the constant part leaves the 32-bit word, so no mask is needed
    asm("ld.shared.v2.b32 {%0, %1}, [%2];" : "=f"(th), "=r"(base) : "r"(tab_lane + (bits << 8)));
    return base + (v > th ? 1u : 0u);
}
// FP4, same idea on the magnitude: 16 buckets of width 1/16 hold one of the seven thresholds at most; bucket = low five
// bits of fma_rz(|v|, 16, 2^23) = floor(16 |v|) (16, reached by |v| = 1 only, carries bucket 15's entry); the sign as in
// fp4_code.  oracle/oracle.c:o_prove_fp4_buckets16_rz checks every float of [-1, 1].  Entry g of lane l at g * 256 + l * 8.
constexpr int FP4_B16_ENTRIES = 17;
__device__ __forceinline__ void fp4_bucket16_fill(float2 *tab, int tid, int nthreads) {
    const float t[7] = {FP4_T0, FP4_T1, FP4_T2, FP4_T3, FP4_T4, FP4_T5, FP4_T6};
    for (int i = tid; i < FP4_B16_ENTRIES * 32; i += nthreads) {
        const int g = i >> 5, b = g < 16 ? g : 15;
        const float lo = (float)b * 0.0625f, hi = (float)(b + 1) * 0.0625f;   // exact
        int below = 0;
        float th = NF4_INF;
#pragma unroll
        for (int j = 0; j < 7; ++j) {
            if (t[j] < lo) ++below;
            else if (t[j] < hi) th = t[j];
        }
        tab[i] = make_float2(th, __int_as_float(below));
    }
}
__device__ __forceinline__ uint32_t fp4_code_bucket16(float v, uint32_t tab_lane) {
    const float a = fabsf(v);
    const uint32_t bits = __float_as_uint(__fmaf_rz(a, 16.0f, 8388608.0f));
    float th; uint32_t base;
    asm("ld.shared.v2.b32 {%0, %1}, [%2];" : "=f"(th), "=r"(base) : "r"(tab_lane + (bits << 8)));   // (as for NF4: no mask)
    const uint32_t m = base + (a > th ? 1u : 0u);
    return (v < 0.0f && m != 0u) ? (m | 8u) : m;                   // code 0 (+0.0) beats code 8 (-0.0) on the tie
}
template <int QT> __device__ __forceinline__ uint32_t code_unit(float v, uint32_t tab_lane) {
    return QT == MPSBNB_NF4 ? nf4_code_bucket32(v, tab_lane) : fp4_code_bucket16(v, tab_lane);
}
template <int QT> __device__ __forceinline__ uint32_t code_fast(float v, const float2 *tab) {
    return QT == MPSBNB_NF4 ? nf4_code_bucket(v, tab) : fp4_code(v);
}

// x / a rounded to nearest, a > 0.  EXACT16: x and a are fp16- or bf16-representable and
// 1e-30 <= a <= 1e30, where the 4-operation form is proven equal to IEEE division for
// the purpose of code selection.
template <bool EXACT16> __device__ __forceinline__ float block_div(float x, float a, float r) {
    if (EXACT16) {
        const float q = __fmul_rn(x, r);
        return __fmaf_rn(__fmaf_rn(-q, a, x), r, q);
    }
    return __fdiv_rn(x, a);
}

// ------------------------------------------------------------------------------------------
// Fast quantiser: 8 elements per thread, LPB = blocksize / 8 lanes per block.
// ------------------------------------------------------------------------------------------
template <typename T, int QT, int LPB>
__global__ void __launch_bounds__(256)
quantize4_fast_kernel(const T *__restrict__ A, int64_t rows, int64_t cols, int64_t chunks_per_row,
                      const float *__restrict__ absmax_in, uint8_t *__restrict__ packed,
                      float *__restrict__ absmax_out) {
    static_assert(sizeof(T) == 2, "fast path takes 16-bit input");
    __shared__ float2 nf4_tab[16];
    if (QT == MPSBNB_NF4) {
        if (threadIdx.x < 16) nf4_bucket_table_fill(nf4_tab, threadIdx.x);
        __syncthreads();
    }
    constexpr int U = 4;                                   // 16-byte loads in flight per thread: the kernel is a
                                                           // pure stream and needs ~100 KB in flight per SM
    const int64_t total = rows * chunks_per_row;           // multiple of LPB
    const int64_t nwarp_iters = (total + 31) / 32;
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const bool small = total < 0x7fffffffll && chunks_per_row < 0x7fffffffll;   // 32-bit index arithmetic
    for (int64_t wb = warp0; wb < nwarp_iters; wb += nwarps * U) {
        uint4 raw[U];
        int64_t cs[U], rowv[U], kcv[U];
        bool livev[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t wi = wb + (int64_t)u * nwarps;
            const int64_t c = wi * 32 + lane;
            const bool live = wi < nwarp_iters && c < total;
            int64_t row, kc;
            if (small) {
                const uint32_t c32 = live ? (uint32_t)c : 0u, cpr = (uint32_t)chunks_per_row;
                const uint32_t r32 = c32 / cpr;
                row = r32; kc = c32 - r32 * cpr;
            } else {
                row = live ? c / chunks_per_row : 0;
                kc = live ? c - row * chunks_per_row : 0;
            }
            cs[u] = c; rowv[u] = row; kcv[u] = kc; livev[u] = live;
            raw[u] = make_uint4(0u, 0u, 0u, 0u);           // zero padding beyond K
            if (live && kc * 8 < cols) raw[u] = __ldg(reinterpret_cast<const uint4 *>(A + row * cols + kc * 8));
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            // warp-uniform: the shuffles below need the whole warp
            if (wb + (int64_t)u * nwarps >= nwarp_iters) break;
            const bool live = livev[u];
            const int64_t row = rowv[u], kc = kcv[u];
            float x[8];
            {
                const T *h = reinterpret_cast<const T *>(&raw[u]);
#pragma unroll
                for (int j = 0; j < 8; ++j) x[j] = to_f32<T>(h[j]);
            }
            const int64_t blk = row * (chunks_per_row / LPB) + kc / LPB;
            float a;
            if (absmax_in != nullptr) {
                a = live ? absmax_in[blk] : 1.0f;
            } else {
                a = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) a = fmaxf(a, fabsf(x[j]));
#pragma unroll
                for (int o = 1; o < LPB; o <<= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
                a = fmaxf(a, 1e-8f);                           // clamp(min=1e-8)
                if (live && (lane & (LPB - 1)) == 0) absmax_out[blk] = a;
            }
            uint32_t word = 0;
            if (a > 1e-8f && a <= 1e30f && absmax_in == nullptr) {   // a is a 16-bit input's magnitude: covered by the proof
                                                                     // (a == 1e-8f is the clamp, not an input value: exact division)
                const float r = __frcp_rn(a);
#pragma unroll
                for (int j = 0; j < 8; ++j) word |= code_fast<QT>(block_div<true>(x[j], a, r), nf4_tab) << (4 * j);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) word |= code_fast<QT>(block_div<false>(x[j], a, 0.f), nf4_tab) << (4 * j);
            }
            if (live) reinterpret_cast<uint32_t *>(packed)[cs[u]] = word;   // byte j/2: low nibble = even k
        }
    }
}

// ------------------------------------------------------------------------------------------
// Streaming quantiser: the common case (16-bit input, block size 64, K a multiple of 64, maxima computed here).
// The fast kernel above loads, computes and stores in turn, so its loads are in flight only part of the time
// (measured 1.9 TB/s with exactly the algorithmic DRAM traffic: latency, not bytes or arithmetic).  Here every thread
// keeps NS - 1 asynchronous 16-byte copies into its own slots of a shared-memory ring in flight WHILE it computes:
// 80 bytes per thread, 120 KB per SM, whatever the arithmetic is doing.  A thread reads only what it copied
// itself, so the copy groups' own completion is the only synchronisation.  With K a multiple of 64 the matrix is one
// run of 8-element chunks: no row / column arithmetic, block = chunk / 8.
// ------------------------------------------------------------------------------------------
constexpr int QS_NS = 6;
__device__ __forceinline__ void qs_cp_async16(void *dst_shared, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src) : "memory");
}
template <typename T, int QT, typename IDX>                        // IDX: chunk counters in 32 bits where the matrix allows it
__global__ void __launch_bounds__(256, 6)
quantize4_stream_kernel(const T *__restrict__ A, IDX total, uint8_t *__restrict__ packed, float *__restrict__ absmax_out) {
    static_assert(sizeof(T) == 2, "16-bit input");
    __shared__ uint4 ring[QS_NS][256];
    __shared__ __align__(16) float2 nf4_tab[(QT == MPSBNB_NF4 ? NF4_B32_ENTRIES : FP4_B16_ENTRIES) * 32];
    const int tid = threadIdx.x, lane = tid & 31;
    if (QT == MPSBNB_NF4) nf4_bucket32_fill(nf4_tab, tid, 256);
    else fp4_bucket16_fill(nf4_tab, tid, 256);
    __syncthreads();
    const uint32_t tab_lane = (uint32_t)__cvta_generic_to_shared(nf4_tab) + (uint32_t)lane * 8u;
    const IDX stride = (IDX)gridDim.x * 256;
    IDX c_next = (IDX)blockIdx.x * 256 + (IDX)tid;                   // chunk of the next copy
#pragma unroll
    for (int s = 0; s < QS_NS - 1; ++s) {
        if (c_next < total) qs_cp_async16(&ring[s][tid], A + (size_t)c_next * 8);
        asm volatile("cp.async.commit_group;" ::: "memory");
        c_next += stride;
    }
    // total is a multiple of 8 and a warp's 32 chunks start at a multiple of 32: the eight lanes of a block are live
    // together; the loop condition is warp-uniform (first lane's chunk) because of the shuffles.  The ring's slots are
    // taken in turn by an unrolled inner loop, so slot numbers are constants.
    IDX c = (IDX)blockIdx.x * 256 + (IDX)tid;
    bool more = true;
    while (more) {
#pragma unroll
        for (int s = 0; s < QS_NS; ++s) {
            if (c - (IDX)lane >= total) { more = false; break; }
            asm volatile("cp.async.wait_group %0;" ::"n"(QS_NS - 2) : "memory");
            const bool live = c < total;
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (live) raw = ring[s][tid];
            // refill the slot read one iteration ago (its values have been consumed)
            if (c_next < total) qs_cp_async16(&ring[(s + QS_NS - 1) % QS_NS][tid], A + (size_t)c_next * 8);
            asm volatile("cp.async.commit_group;" ::: "memory");
            c_next += stride;
            float x[8];
            {
                const T *h = reinterpret_cast<const T *>(&raw);
#pragma unroll
                for (int j = 0; j < 8; ++j) x[j] = to_f32<T>(h[j]);
            }
            float a = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) a = fmaxf(a, fabsf(x[j]));
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
            a = fmaxf(a, 1e-8f);                                       // clamp(min=1e-8)
            if (live && (lane & 7) == 0) absmax_out[(size_t)(c >> 3)] = a;
            uint32_t word = 0;
            if (a > 1e-8f && a <= 1e30f) {                             // a 16-bit input's magnitude: the shortcut is proven exact
                const float r = __frcp_rn(a);
#pragma unroll
                for (int j = 0; j < 8; ++j) word += code_unit<QT>(block_div<true>(x[j], a, r), tab_lane) << (4 * j);   // nibbles do not overlap: + is |
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) word += code_unit<QT>(block_div<false>(x[j], a, 0.f), tab_lane) << (4 * j);
            }
            if (live) reinterpret_cast<uint32_t *>(packed)[(size_t)c] = word;   // byte j/2: low nibble = even k
            c += stride;
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
}

// ------------------------------------------------------------------------------------------
// General quantiser (any dtype, block size, K, alignment): block maxima with one warp per
// block, then one thread per packed byte.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void absmax_blocks_kernel(const T *__restrict__ A, int64_t rows, int64_t cols, int64_t bs,
                                     int64_t nb, float *__restrict__ absmax_out) {
    const int lane = threadIdx.x & 31;
    const int64_t nblk = rows * nb;
    const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    for (int64_t b = warp0; b < nblk; b += (int64_t)gridDim.x * (blockDim.x >> 5)) {
        const int64_t row = b / nb, k0 = (b - row * nb) * bs;
        float a = 0.0f;
        for (int64_t j = lane; j < bs; j += 32) {
            const int64_t k = k0 + j;
            if (k < cols) a = fmaxf(a, fabsf(to_f32<T>(A[row * cols + k])));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        if (lane == 0) absmax_out[b] = fmaxf(a, 1e-8f);
    }
}

template <typename T, int QT>
__global__ void quantize4_bytes_kernel(const T *__restrict__ A, int64_t rows, int64_t cols, int64_t bs,
                                       int64_t Kp, const float *__restrict__ absmax,
                                       uint8_t *__restrict__ packed) {
    const int64_t half = Kp / 2, total = rows * half, nb = Kp / bs;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / half, j = i - row * half;
        uint32_t byte = 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t k = 2 * j + h;
            const float x = k < cols ? to_f32<T>(A[row * cols + k]) : 0.0f;
            const float a = absmax[row * nb + k / bs];
            byte |= code_of<QT>(__fdiv_rn(x, a)) << (4 * h);
        }
        packed[i] = (uint8_t)byte;
    }
}

// ------------------------------------------------------------------------------------------
// Dequantise.  absmax of block i: fp32 absmax[i], or float(q[i]) * (absmax2[i/256] / 127)
// (mps_bitsandbytes/functional.py:592-593: divide first, then multiply).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_absmax(const void *absmax, const float *absmax2, int64_t i) {
    if (absmax2 == nullptr) return __ldg(reinterpret_cast<const float *>(absmax) + i);
    const float q = (float)__ldg(reinterpret_cast<const int8_t *>(absmax) + i);
    return __fmul_rn(q, __fdiv_rn(__ldg(absmax2 + (i >> 8)), 127.0f));
}

// 16 elements (8 packed bytes) per thread; needs cols % 16 == 0 and blocksize >= 16.
template <typename T, int QT>
__global__ void __launch_bounds__(256)
dequantize4_fast_kernel(const uint8_t *__restrict__ packed, const void *__restrict__ absmax,
                        const float *__restrict__ absmax2, int64_t rows, int64_t cols, int64_t Kp,
                        int bs_shift, T *__restrict__ out, int64_t ld) {
    __shared__ float lut[16];
    if (threadIdx.x < 16) lut[threadIdx.x] = kCode[QT][threadIdx.x];
    __syncthreads();
    const int64_t per_row = cols / 16, total = rows * per_row, nb = Kp >> bs_shift;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / per_row, k0 = (i - row * per_row) * 16;
        const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(packed + row * (Kp / 2) + k0 / 2));
        const float a = block_absmax(absmax, absmax2, row * nb + (k0 >> bs_shift));
        T vals[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t w = j < 4 ? raw.x : raw.y;
            const uint32_t byte = (w >> (8 * (j & 3))) & 0xFFu;
            vals[2 * j] = from_f32<T>(__fmul_rn(lut[byte & 15u], a));
            vals[2 * j + 1] = from_f32<T>(__fmul_rn(lut[byte >> 4], a));
        }
        T *dst = out + row * ld + k0;
        if (sizeof(T) == 2) {
            reinterpret_cast<uint4 *>(dst)[0] = reinterpret_cast<const uint4 *>(vals)[0];
            reinterpret_cast<uint4 *>(dst)[1] = reinterpret_cast<const uint4 *>(vals)[1];
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q)
                reinterpret_cast<uint4 *>(dst)[q] = reinterpret_cast<const uint4 *>(vals)[q];
        }
    }
}

// The same for a contiguous matrix whose rows are whole blocks (ld == cols, cols a multiple of the block size): the
// matrix is one run of 16-element chunks - no 64-bit division per chunk - and four chunks' loads are issued before the
// first is expanded (the kernel above waits on its single 8-byte load most of the time: 49 % issue, 48 % DRAM).
template <typename T, int QT>
__global__ void __launch_bounds__(256)
dequantize4_stream_kernel(const uint8_t *__restrict__ packed, const void *__restrict__ absmax,
                          const float *__restrict__ absmax2, int64_t total, int chunk_shift, T *__restrict__ out) {
    __shared__ float lut[16];
    if (threadIdx.x < 16) lut[threadIdx.x] = kCode[QT][threadIdx.x];
    __syncthreads();
    constexpr int U = 4;
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i0 = (int64_t)blockIdx.x * 256 + threadIdx.x; i0 < total; i0 += stride * U) {
        uint2 raw[U];
        float a[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            raw[u] = make_uint2(0u, 0u); a[u] = 0.0f;
            if (i < total) {
                raw[u] = __ldg(reinterpret_cast<const uint2 *>(packed) + i);
                a[u] = block_absmax(absmax, absmax2, i >> chunk_shift);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i >= total) break;
            T vals[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t w = j < 4 ? raw[u].x : raw[u].y;
                const uint32_t byte = (w >> (8 * (j & 3))) & 0xFFu;
                vals[2 * j] = from_f32<T>(__fmul_rn(lut[byte & 15u], a[u]));
                vals[2 * j + 1] = from_f32<T>(__fmul_rn(lut[byte >> 4], a[u]));
            }
            T *dst = out + i * 16;
#pragma unroll
            for (int q = 0; q < (int)(sizeof(T) * 16 / 16); ++q)
                __stcs(reinterpret_cast<uint4 *>(dst) + q, reinterpret_cast<const uint4 *>(vals)[q]);   // written once, not re-read here
        }
    }
}

template <typename T, int QT>
__global__ void dequantize4_elem_kernel(const uint8_t *__restrict__ packed, const void *__restrict__ absmax,
                                        const float *__restrict__ absmax2, int64_t rows, int64_t cols,
                                        int64_t Kp, int64_t bs, T *__restrict__ out, int64_t ld) {
    const int64_t total = rows * cols, nb = Kp / bs;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / cols, k = i - row * cols;
        const uint32_t byte = packed[row * (Kp / 2) + k / 2];
        const uint32_t idx = (k & 1) ? (byte >> 4) : (byte & 15u);
        out[row * ld + k] = from_f32<T>(__fmul_rn(kCode[QT][idx], block_absmax(absmax, absmax2, row * nb + k / bs)));
    }
}

// ------------------------------------------------------------------------------------------
// Blockwise int8 (mps_bitsandbytes/functional.py:469-600).  One CTA per block of `bs`
// values.  scale = 127.0 / absmax is evaluated as reciprocal * 127 — torch computes
// scalar / tensor as tensor.reciprocal() * scalar — which decides round-half-even ties.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
quantize_blockwise_kernel(const T *__restrict__ A, int64_t n, int64_t bs, const float *__restrict__ absmax_in,
                          int8_t *__restrict__ q, float *__restrict__ absmax_out) {
    __shared__ float red[8];
    __shared__ float s_scale;
    const int64_t nblk = (n + bs - 1) / bs;
    for (int64_t b = blockIdx.x; b < nblk; b += gridDim.x) {
        const int64_t i0 = b * bs;
        const int64_t len = min(bs, n - i0);
        float a;
        if (absmax_in != nullptr) {
            a = absmax_in[b];
        } else {
            a = 0.0f;
            for (int64_t j = threadIdx.x; j < len; j += blockDim.x) a = fmaxf(a, fabsf(to_f32<T>(A[i0 + j])));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
            __syncthreads();
            a = red[0];
            for (int w = 1; w < (int)(blockDim.x >> 5); ++w) a = fmaxf(a, red[w]);
            a = fmaxf(a, 1e-8f);
        }
        if (threadIdx.x == 0) {
            if (absmax_out != nullptr) absmax_out[b] = a;
            s_scale = __fmul_rn(__frcp_rn(a), 127.0f);
        }
        __syncthreads();
        const float scale = s_scale;
        for (int64_t j = threadIdx.x; j < len; j += blockDim.x) {
            float v = rintf(__fmul_rn(to_f32<T>(A[i0 + j]), scale));   // round half to even
            v = fminf(fmaxf(v, -127.0f), 127.0f);
            q[i0 + j] = (int8_t)(int)v;
        }
        __syncthreads();
    }
}

// Block size 256, fp32 input (the second level of double quantisation: one block maximum per 64 weights, millions of
// them): a WARP per block - eight values per lane, maxima by shuffles, no CTA barrier - instead of a CTA per block with
// three barriers each.  Same operations per element as above, so the same codes.
__global__ void __launch_bounds__(256)
quantize_blockwise256_f32_kernel(const float *__restrict__ A, int64_t n, const float *__restrict__ absmax_in,
                                 int8_t *__restrict__ q, float *__restrict__ absmax_out) {
    const int lane = threadIdx.x & 31;
    const int64_t nblk = (n + 255) / 256;
    const int64_t warp0 = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (int64_t)gridDim.x * 8;
    for (int64_t b = warp0; b < nblk; b += nwarps) {
        const int64_t i0 = b * 256 + lane * 8;
        float x[8];
        if (i0 + 8 <= n) {
            const float4 v0 = __ldg(reinterpret_cast<const float4 *>(A + i0)), v1 = __ldg(reinterpret_cast<const float4 *>(A + i0) + 1);
            x[0] = v0.x; x[1] = v0.y; x[2] = v0.z; x[3] = v0.w; x[4] = v1.x; x[5] = v1.y; x[6] = v1.z; x[7] = v1.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = i0 + e < n ? A[i0 + e] : 0.0f;
        }
        float a;
        if (absmax_in != nullptr) {
            a = absmax_in[b];
        } else {
            a = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; ++e) a = fmaxf(a, fabsf(x[e]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
            a = fmaxf(a, 1e-8f);
        }
        if (lane == 0 && absmax_out != nullptr) absmax_out[b] = a;
        const float scale = __fmul_rn(__frcp_rn(a), 127.0f);
        uint32_t w[2] = {0u, 0u};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float v = rintf(__fmul_rn(x[e], scale));               // round half to even
            v = fminf(fmaxf(v, -127.0f), 127.0f);
            w[e >> 2] |= ((uint32_t)(int)v & 0xFFu) << (8 * (e & 3));
        }
        if (i0 + 8 <= n) {
            *reinterpret_cast<uint2 *>(q + i0) = make_uint2(w[0], w[1]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (i0 + e < n) q[i0 + e] = (int8_t)((w[e >> 2] >> (8 * (e & 3))) & 0xFFu);
        }
    }
}

template <typename T>
__global__ void dequantize_blockwise_kernel(const int8_t *__restrict__ q, const float *__restrict__ absmax,
                                            int64_t n, int64_t bs, T *__restrict__ out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(__fmul_rn((float)q[i], __fdiv_rn(__ldg(absmax + i / bs), 127.0f)));
}

static int grid_for(int64_t work_items, int threads, int per_sm) {
    int64_t g = (work_items + threads - 1) / threads;
    const int64_t cap = (int64_t)sm_count() * per_sm;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

static int shift_of(int64_t v) {
    int s = 0;
    while ((1ll << s) < v) ++s;
    return s;
}

}  // namespace mpsbnb

using namespace mpsbnb;

extern "C" int mpsbnb_quantize_4bit(const void *A, int a_dtype, int64_t rows, int64_t cols, int blocksize,
                                    int quant_type, const float *absmax_in, uint8_t *packed,
                                    float *absmax_out, void *stream) {
    if (!valid_dtype(a_dtype) || (quant_type != MPSBNB_NF4 && quant_type != MPSBNB_FP4)) return MPSBNB_ERR_INVALID_ARG;
    if (rows < 0 || cols < 0 || !is_pow2(blocksize) || blocksize > 65536) return MPSBNB_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return MPSBNB_OK;
    if (A == nullptr || packed == nullptr || (absmax_in == nullptr && absmax_out == nullptr)) return MPSBNB_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t Kp = padded_k(cols, blocksize), nb = Kp / blocksize;
    const bool fast = is_16bit(a_dtype) && blocksize >= 32 && blocksize <= 256 && (cols % 8) == 0 &&
                      aligned16(A) && ((reinterpret_cast<uintptr_t>(packed) & 3) == 0);
    if (fast && blocksize == 64 && cols % 64 == 0 && absmax_in == nullptr) {
        const int64_t total = rows * (cols / 8);
        const int64_t want = (total + 255) / 256;
        const int grid = (int)(want < 6 * sm_count() ? want : 6 * sm_count());   // six CTAs per SM stay resident
#define LAUNCH_STREAM(T, QT)                                                                                             \
    do {                                                                                                                 \
        if (total < 0x7f000000ll)                                                                                        \
            quantize4_stream_kernel<T, QT, uint32_t><<<grid, 256, 0, st>>>((const T *)A, (uint32_t)total, packed, absmax_out); \
        else                                                                                                             \
            quantize4_stream_kernel<T, QT, int64_t><<<grid, 256, 0, st>>>((const T *)A, total, packed, absmax_out);      \
    } while (0)
        if (quant_type == MPSBNB_NF4) {
            if (a_dtype == MPSBNB_F16) LAUNCH_STREAM(__half, MPSBNB_NF4);
            else LAUNCH_STREAM(__nv_bfloat16, MPSBNB_NF4);
        } else {
            if (a_dtype == MPSBNB_F16) LAUNCH_STREAM(__half, MPSBNB_FP4);
            else LAUNCH_STREAM(__nv_bfloat16, MPSBNB_FP4);
        }
#undef LAUNCH_STREAM
        return check_launch();
    }
    if (fast) {
        const int64_t cpr = Kp / 8, total = rows * cpr;
        const int grid = grid_for((total + 31) / 32 * 32, 256, 16);
#define LAUNCH_FAST(T, QT, LPB)                                                                     \
    quantize4_fast_kernel<T, QT, LPB><<<grid, 256, 0, st>>>((const T *)A, rows, cols, cpr, absmax_in, \
                                                             packed, absmax_out)
#define LAUNCH_FAST_QT(T, LPB)                                                   \
    do {                                                                         \
        if (quant_type == MPSBNB_NF4) LAUNCH_FAST(T, MPSBNB_NF4, LPB);           \
        else LAUNCH_FAST(T, MPSBNB_FP4, LPB);                                    \
    } while (0)
#define LAUNCH_FAST_T(LPB)                                                       \
    do {                                                                         \
        if (a_dtype == MPSBNB_F16) LAUNCH_FAST_QT(__half, LPB);                  \
        else LAUNCH_FAST_QT(__nv_bfloat16, LPB);                                 \
    } while (0)
        switch (blocksize) {
            case 32: LAUNCH_FAST_T(4); break;
            case 64: LAUNCH_FAST_T(8); break;
            case 128: LAUNCH_FAST_T(16); break;
            default: LAUNCH_FAST_T(32); break;
        }
        return check_launch();
    }
    const float *am = absmax_in;
    if (am == nullptr) {
        const int grid = grid_for(rows * nb * 32, 256, 16);
        MPSBNB_DISPATCH_DTYPE(a_dtype, T, (absmax_blocks_kernel<T><<<grid, 256, 0, st>>>(
                                              (const T *)A, rows, cols, blocksize, nb, absmax_out)));
        int rc = check_launch();
        if (rc != MPSBNB_OK) return rc;
        am = absmax_out;
    }
    const int grid = grid_for(rows * (Kp / 2), 256, 16);
    if (quant_type == MPSBNB_NF4)
        MPSBNB_DISPATCH_DTYPE(a_dtype, T, (quantize4_bytes_kernel<T, MPSBNB_NF4><<<grid, 256, 0, st>>>(
                                              (const T *)A, rows, cols, blocksize, Kp, am, packed)));
    else
        MPSBNB_DISPATCH_DTYPE(a_dtype, T, (quantize4_bytes_kernel<T, MPSBNB_FP4><<<grid, 256, 0, st>>>(
                                              (const T *)A, rows, cols, blocksize, Kp, am, packed)));
    return check_launch();
}

namespace mpsbnb {
// Dequantise into a matrix with leading dimension ld (elements), ld >= cols.
int dequantize_4bit_ld(const uint8_t *packed, const void *absmax, const float *absmax2, int64_t rows, int64_t cols,
                       int blocksize, int quant_type, void *out, int64_t ld, int out_dtype, cudaStream_t st) {
    if (!valid_dtype(out_dtype) || (quant_type != MPSBNB_NF4 && quant_type != MPSBNB_FP4)) return MPSBNB_ERR_INVALID_ARG;
    if (rows < 0 || cols < 0 || ld < cols || !is_pow2(blocksize) || blocksize > 65536) return MPSBNB_ERR_INVALID_ARG;
    if (rows == 0 || cols == 0) return MPSBNB_OK;
    if (packed == nullptr || absmax == nullptr || out == nullptr) return MPSBNB_ERR_INVALID_ARG;
    const int64_t Kp = padded_k(cols, blocksize);
    const bool fast = blocksize >= 16 && (cols % 16) == 0 && aligned16(out) && (ld * dtype_bytes(out_dtype)) % 16 == 0 &&
                      ((reinterpret_cast<uintptr_t>(packed) & 7) == 0);
    if (fast && ld == cols && Kp == cols) {
        const int64_t total = rows * (cols / 16);
        const int64_t want = (total + 256 * 4 - 1) / (256 * 4);
        const int grid = (int)(want < 8 * sm_count() ? want : 8 * sm_count());
        const int csh = shift_of(blocksize) - 4;
        if (quant_type == MPSBNB_NF4)
            MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize4_stream_kernel<T, MPSBNB_NF4><<<grid, 256, 0, st>>>(
                                                    packed, absmax, absmax2, total, csh, (T *)out)));
        else
            MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize4_stream_kernel<T, MPSBNB_FP4><<<grid, 256, 0, st>>>(
                                                    packed, absmax, absmax2, total, csh, (T *)out)));
        return check_launch();
    }
    if (fast) {
        const int grid = grid_for(rows * (cols / 16), 256, 16);
        const int sh = shift_of(blocksize);
        if (quant_type == MPSBNB_NF4)
            MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize4_fast_kernel<T, MPSBNB_NF4><<<grid, 256, 0, st>>>(
                                                    packed, absmax, absmax2, rows, cols, Kp, sh, (T *)out, ld)));
        else
            MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize4_fast_kernel<T, MPSBNB_FP4><<<grid, 256, 0, st>>>(
                                                    packed, absmax, absmax2, rows, cols, Kp, sh, (T *)out, ld)));
        return check_launch();
    }
    const int grid = grid_for(rows * cols, 256, 16);
    if (quant_type == MPSBNB_NF4)
        MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize4_elem_kernel<T, MPSBNB_NF4><<<grid, 256, 0, st>>>(
                                                packed, absmax, absmax2, rows, cols, Kp, blocksize, (T *)out, ld)));
    else
        MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize4_elem_kernel<T, MPSBNB_FP4><<<grid, 256, 0, st>>>(
                                                packed, absmax, absmax2, rows, cols, Kp, blocksize, (T *)out, ld)));
    return check_launch();
}
}  // namespace mpsbnb

extern "C" int mpsbnb_dequantize_4bit(const uint8_t *packed, const void *absmax, const float *absmax2,
                                      int64_t rows, int64_t cols, int blocksize, int quant_type, void *out,
                                      int out_dtype, void *stream) {
    return dequantize_4bit_ld(packed, absmax, absmax2, rows, cols, blocksize, quant_type, out, cols, out_dtype,
                              (cudaStream_t)stream);
}

extern "C" int mpsbnb_quantize_blockwise(const void *A, int a_dtype, int64_t n, int blocksize,
                                         const float *absmax_in, int8_t *q, float *absmax_out, void *stream) {
    if (!valid_dtype(a_dtype) || n < 0 || blocksize <= 0 || blocksize > 65536) return MPSBNB_ERR_INVALID_ARG;
    if (n == 0) return MPSBNB_OK;
    if (A == nullptr || q == nullptr || (absmax_in == nullptr && absmax_out == nullptr)) return MPSBNB_ERR_INVALID_ARG;
    const int64_t nblk = (n + blocksize - 1) / blocksize;
    if (blocksize == 256 && a_dtype == MPSBNB_F32 && aligned16(A) && (reinterpret_cast<uintptr_t>(q) & 7) == 0) {
        int64_t g = (nblk + 7) / 8;
        const int64_t gcap = (int64_t)sm_count() * 8;
        if (g > gcap) g = gcap;
        quantize_blockwise256_f32_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>((const float *)A, n, absmax_in, q, absmax_out);
        return check_launch();
    }
    int64_t grid = nblk;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (grid > cap) grid = cap;
    MPSBNB_DISPATCH_DTYPE(a_dtype, T, (quantize_blockwise_kernel<T><<<(int)grid, 256, 0, (cudaStream_t)stream>>>(
                                          (const T *)A, n, blocksize, absmax_in, q, absmax_out)));
    return check_launch();
}

extern "C" int mpsbnb_dequantize_blockwise(const int8_t *q, const float *absmax, int64_t n, int blocksize,
                                           void *out, int out_dtype, void *stream) {
    if (!valid_dtype(out_dtype) || n < 0 || blocksize <= 0) return MPSBNB_ERR_INVALID_ARG;
    if (n == 0) return MPSBNB_OK;
    if (q == nullptr || absmax == nullptr || out == nullptr) return MPSBNB_ERR_INVALID_ARG;
    const int grid = grid_for(n, 256, 16);
    MPSBNB_DISPATCH_DTYPE(out_dtype, T, (dequantize_blockwise_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
                                            q, absmax, n, blocksize, (T *)out)));
    return check_launch();
}
