// Fused dequantise-GEMM for sm_100a:  y[m, n] = sum_k x[m, k] * W[n, k]  (* wscale[n]) (+ bias[n]),
// where W is never materialised in global memory: the quantised weight bytes are brought into shared
// memory by TMA, expanded to 16-bit values by eight "expander" warps straight into the 128-byte-swizzled
// K-major operand tile that tcgen05.mma reads, and multiplied on the tensor cores with fp32 accumulators
// in tensor memory.  Stands for mps_bitsandbytes/functional.py:680-773 (matmul_4bit), :796-807
// (matmul_fp8_e4m3), :935-945 (matmul_colrow) and nn/linear8bit.py:91-102 on prefill shapes; the
// reference's Metal analogues dequantise inside their K loops in the same way (mps_bitsandbytes.mm:567-696
// nf4_matmul_large, :203-305 int8_matmul_simd, :1101-1203 fp8_matmul_simd).
//
// Orientation: the WEIGHT is the MMA's A operand (128 weight rows = the 128 lanes of tensor memory) and
// x is the B operand (TM = 32 ... 256 rows of x = accumulator columns).  A 128 x TM tile therefore
// expands 128 x 64 weights per 64-wide K step whatever TM is - half of what a 128 (x) x 256 (weight)
// tile would need - and a small batch simply uses a narrow TM.  One persistent CTA per SM, 23 warps:
//   warp 0      TMA producer of x tiles (TM rows x 64 k, 128-byte swizzle) into the X ring (3 stages of 32 KB for
//               TM = 256 ... 16 stages of 4 KB for TM = 32: a stage is in flight for a whole TMA round trip);
//   warp 1      MMA issuer: per K step four tcgen05.mma (128 x TM x 16, kind::f16), then tcgen05.commit
//               hands the W and X stages back; owns the tensor-memory allocation (2 x TM columns: the
//               accumulator is double-buffered, so the epilogue of a tile overlaps the next tile);
//   warp 2      TMA producer of quantised weight chunks into the Q ring: 128 rows x 128 bytes (128-byte swizzle) =
//               256 k of 4-bit codes or 128 k of 8-bit codes, or 64 k-rows x 128 n-bytes of a K x N int8 operand;
//   warps 3-6   epilogue: tcgen05.ld (lane = weight row n, column = x row m), scale, bias, round, store;
//   warps 7-22  expanders, two groups of eight warps that take alternate K steps (each group alternates between two
//               of the four W stages, so it fills one while the tensor core reads the other).  Thread (r, h) turns
//               half a row (32 k) of a K step into 64 bytes of the W stage.
//               4-bit: byte -> (code[lo], code[hi]) by a 256-entry fp16-pair table replicated per lane in shared
//               memory, times the block's absmax (one packed fp16 multiply when the scale sits well inside the
//               fp16 range, else an fp32 product rounded once).
//               int8: exact conversion (the per-row scale is applied to the fp32 accumulator instead); a K x N
//               operand is transposed on the way (byte permutes in registers).
//               fp8 E4M3: exact hardware conversion (per-row scale in the epilogue as well).
// What bounds it (measured): for TM = 256 the tensor pipe and the L2 -> shared-memory traffic of the x tiles, as in
// the unfused GEMM; for narrow tiles the serial MMA-issuer thread (two waits, four MMAs, two commits per K step cost
// it about 900 cycles, of which the expanders' work is entirely hidden), i.e. about 1 TB/s of weight bytes.
// Every wait is bounded; a time-out records a status word and all roles leave through the common exit.
#include "common.cuh"
#include "ops.cuh"
#include "sm100.cuh"

#include <string.h>

namespace mpsbnb {

using namespace sm100;

constexpr int WQ_GROUPS = 2;                 // expander groups; group g takes the K steps kb = g (mod 2)
constexpr int WQ_GROUP_WARPS = 8;
// Warp schedulers take warps by (warp index mod 4).  The MMA issuer is warp 1, and its loop is the serial path of the
// kernel, so no expander warp may share its scheduler: expanders are the warps from 7 on whose index is not 1 mod 4; the
// warps in between (9, 13, 17, 21, 25) do nothing.
constexpr int WQ_FIRST_EXPANDER = 7;
constexpr int WQ_WARPS = 28;
constexpr int WQ_THREADS = WQ_WARPS * 32;
__host__ __device__ constexpr int wq_expander_index(int warp) {      // 0 .. 15, or -1
    return (warp < WQ_FIRST_EXPANDER || (warp & 3) == 1) ? -1 : warp - WQ_FIRST_EXPANDER - (warp >= 9 ? (warp - 9) / 4 + 1 : 0);
}
static_assert(wq_expander_index(7) == 0 && wq_expander_index(8) == 1 && wq_expander_index(10) == 2 && wq_expander_index(27) == 15 &&
              wq_expander_index(9) == -1 && wq_expander_index(25) == -1, "sixteen expander warps");
constexpr int WQ_ROWS = 128;                 // weight rows per tile (MMA M)
constexpr int WQ_BK = 64;                    // k per MMA stage
constexpr int WQ_WS = 4;                     // W stages (expanded operand tiles, 16 KB each)
constexpr int WQ_W_BYTES = WQ_ROWS * WQ_BK * 2;
constexpr int WQ_Q_BYTES = WQ_ROWS * 128;
constexpr int WQ_LUT_BYTES = 256 * 128;      // entry b of lane l at b * 128 + l * 4
static_assert(WQ_WS % WQ_GROUPS == 0 && WQ_WS > WQ_GROUPS, "a group alternates between WQ_WS / WQ_GROUPS stages of its own");

enum { WQ_4BIT = 0, WQ_INT8 = 1, WQ_FP8 = 2, WQ_INT8T = 3 };   // INT8T: int8 stored [K, N] (N contiguous), transposed on the fly

static __device__ int g_wq_status = 0;


struct WqArgs {
    const void *absmax;        // 4-bit: fp32 [N, nb] or int8 [N, nb] (absmax2 != nullptr)
    const float *absmax2;      // 4-bit double quantisation: fp32 [ceil(N nb / 256)]
    const float *wscale;       // 8-bit: fp32 [N] per-row scale applied to the accumulator (may be nullptr)
    float wscale_mul;          // ... times this constant (1 / 127 for int8)
    int wscale_sqrt;           // ... after a square root (col+row scaled int8: sqrt(r[n]); x carries sqrt(c[k]))
    const void *bias;          // [N] in the operand dtype, or nullptr
    void *y;                   // [M, N] in y_dtype
    int y_dtype, fmt;          // fmt: 0 = fp16 operands, 1 = bf16
    int M, N, K, nb;           // nb: absmax blocks per row (4-bit)
    int quant_type;
};

template <int TM> struct WqSmem {
    // x stages: a stage is in flight for a whole TMA round trip (about a microsecond), so a narrow tile, whose
    // K steps are short, needs many of them
    static constexpr int XS = TM >= 256 ? 3 : TM >= 128 ? 4 : TM >= 64 ? 8 : 16;
    // Q chunks (quantised bytes, 16 KB each): what is in flight from HBM.  A narrow x tile leaves room for a deep ring,
    // which the weight-streaming (small batch) case needs; a wide tile is bound by the tensor pipe and needs little.
    static constexpr int QS = TM >= 256 ? 2 : 4;
    static constexpr int X_BYTES = TM * 128;
    static constexpr int W_OFF = 0;
    static constexpr int X_OFF = WQ_WS * WQ_W_BYTES;
    static constexpr int Q_OFF = X_OFF + XS * X_BYTES;
    static constexpr int LUT_OFF = Q_OFF + QS * WQ_Q_BYTES;
    static constexpr int BAR_OFF = LUT_OFF + WQ_LUT_BYTES;
    // wfull[4] wempty[4] xfull[16] xempty[16] qfull[4] qempty[4] tfull[2] tempty[2], tmem slot, abort flag
    static constexpr int TOTAL = BAR_OFF + 52 * 8 + 16;
};

__device__ __forceinline__ uint4 wq_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void wq_sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// the table is written once in the prologue: the compiler may schedule these loads freely
__device__ __forceinline__ uint32_t wq_lut(uint32_t addr) { uint32_t v; asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr)); return v; }

// (code[lo], code[hi]) as an fp16 pair, each times s in fp32, rounded once to the operand type
template <int FMT> __device__ __forceinline__ uint32_t wq_scale_pair(uint32_t pair, float s) {
    const __half2 h = *reinterpret_cast<const __half2 *>(&pair);
    const float2 f = __half22float2(h);
    if (FMT == 0) {
        const __half2 o = __floats2half2_rn(f.x * s, f.y * s);
        return *reinterpret_cast<const uint32_t *>(&o);
    } else {
        const __nv_bfloat162 o = __floats2bfloat162_rn(f.x * s, f.y * s);
        return *reinterpret_cast<const uint32_t *>(&o);
    }
}

// four int8 (one word) -> two pairs of the operand type, exactly
template <int FMT> __device__ __forceinline__ void wq_i8x4(uint32_t w, uint32_t &lo, uint32_t &hi) {
    if (FMT == 0) {
        // (b ^ 0x80) is b + 128 as an unsigned byte; 0x6400 | u is the fp16 number 1024 + u; minus 1152 gives b
        const uint32_t u = w ^ 0x80808080u;
        const uint32_t p0 = __byte_perm(u, 0x64646464u, 0x4140), p1 = __byte_perm(u, 0x64646464u, 0x4342);
        const __half2 k = __floats2half2_rn(1152.0f, 1152.0f);
        const __half2 a = __hsub2(*reinterpret_cast<const __half2 *>(&p0), k), b = __hsub2(*reinterpret_cast<const __half2 *>(&p1), k);
        lo = *reinterpret_cast<const uint32_t *>(&a); hi = *reinterpret_cast<const uint32_t *>(&b);
    } else {
        // bf16 holds integers up to 256 exactly: 0x4300 | u is 128 + u for u < 128 only, so convert through fp32
        const int b0 = (int)(int8_t)(w & 0xFFu), b1 = (int)(int8_t)((w >> 8) & 0xFFu), b2 = (int)(int8_t)((w >> 16) & 0xFFu), b3 = (int)(int8_t)(w >> 24);
        const __nv_bfloat162 a = __floats2bfloat162_rn((float)b0, (float)b1), b = __floats2bfloat162_rn((float)b2, (float)b3);
        lo = *reinterpret_cast<const uint32_t *>(&a); hi = *reinterpret_cast<const uint32_t *>(&b);
    }
}

// four FP8 E4M3 codes -> two pairs of the operand type (every E4M3 value is exact in fp16 and in bf16)
template <int FMT> __device__ __forceinline__ void wq_f8x4(uint32_t w, uint32_t &lo, uint32_t &hi) {
    uint32_t h0, h1;
    asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}\n"
        : "=r"(h0), "=r"(h1) : "r"(w));
    if (FMT == 0) { lo = h0; hi = h1; }
    else {
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&h0)), f1 = __half22float2(*reinterpret_cast<const __half2 *>(&h1));
        const __nv_bfloat162 a = __floats2bfloat162_rn(f0.x, f0.y), b = __floats2bfloat162_rn(f1.x, f1.y);
        lo = *reinterpret_cast<const uint32_t *>(&a); hi = *reinterpret_cast<const uint32_t *>(&b);
    }
}

template <int TM, int MODE, int FMT>
__global__ void __launch_bounds__(WQ_THREADS, 1)
mpsbnb_gemm_wq_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_q, const WqArgs a) {
    extern __shared__ unsigned char smem_raw[];
    using S = WqSmem<TM>;
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sb = smem_u32(smem);
    const uint32_t bar = sb + S::BAR_OFF;
    auto wfull = [&](int s) { return bar + 8u * s; };
    auto wempty = [&](int s) { return bar + 8u * (4 + s); };
    auto xfull = [&](int s) { return bar + 8u * (8 + s); };
    auto xempty = [&](int s) { return bar + 8u * (24 + s); };
    auto qfull = [&](int s) { return bar + 8u * (40 + s); };
    auto qempty = [&](int s) { return bar + 8u * (44 + s); };
    auto tfull = [&](int b) { return bar + 8u * (48 + b); };
    auto tempty = [&](int b) { return bar + 8u * (50 + b); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + S::BAR_OFF + 52 * 8);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (a.M + TM - 1) / TM, tiles_n = (a.N + WQ_ROWS - 1) / WQ_ROWS;
    const int ntiles = tiles_m * tiles_n;
    const int kblocks = (a.K + WQ_BK - 1) / WQ_BK;
    // every role walks K in whole rounds of the W ring; steps beyond K see zero x (TMA fills) and cost nothing else
    const int kbp = (kblocks + WQ_WS - 1) / WQ_WS * WQ_WS;
    // MMA stages per quantised chunk: 128 bytes per weight row (256 4-bit or 128 8-bit codes), or, for the K x N int8
    // operand, one box of 64 k-rows x 128 n-bytes
    constexpr int SPQ = MODE == WQ_4BIT ? 4 : MODE == WQ_INT8T ? 1 : 2;
    constexpr int Q_TX = MODE == WQ_INT8T ? 64 * 128 : WQ_Q_BYTES;

    if (threadIdx.x == 0) {
        for (int s = 0; s < WQ_WS; ++s) { mbar_init(wfull(s), WQ_GROUP_WARPS); mbar_init(wempty(s), 1); }
        for (int s = 0; s < S::XS; ++s) { mbar_init(xfull(s), 1); mbar_init(xempty(s), 1); }
        for (int s = 0; s < S::QS; ++s) { mbar_init(qfull(s), 1); mbar_init(qempty(s), SPQ * WQ_GROUP_WARPS); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull(b), 1); mbar_init(tempty(b), 4); }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void *)tmem_slot), 2 * TM);
        tmem_relinquish();
    }
    if (MODE == WQ_4BIT && wq_expander_index(warp) >= 0 && wq_expander_index(warp) < 8) {
        // byte -> (code[low nibble], code[high nibble]) as an fp16 pair, one replica per lane
        const int w7 = wq_expander_index(warp);
        const float my_code = kCode[a.quant_type][lane & 15];
        const int byte = w7 * 32 + lane;
        const float lo = __shfl_sync(0xffffffffu, my_code, byte & 15);
        const float hi = __shfl_sync(0xffffffffu, my_code, byte >> 4);
        const __half2 pr = __floats2half2_rn(lo, hi);
        const uint32_t mine = *reinterpret_cast<const uint32_t *>(&pr);
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {
            const uint32_t v = __shfl_sync(0xffffffffu, mine, j);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(sb + (uint32_t)(S::LUT_OFF + (w7 * 32 + j) * 128 + lane * 4)), "r"(v) : "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ x tiles
        if (lane == 0) {
            prefetch_tensormap(&tm_x);
            int stage = 0; uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < ntiles && !*abort_flag; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * TM;
                for (int kb = 0; kb < kbp; ++kb) {
                    if (!mbar_wait(xempty(stage), phase ^ 1, abort_flag)) { atomicExch(&g_wq_status, 301); *abort_flag = 1; break; }
                    mbar_arrive_expect_tx(xfull(stage), S::X_BYTES);
                    tma_load_2d(sb + S::X_OFF + stage * S::X_BYTES, &tm_x, xfull(stage), kb * WQ_BK, m0);
                    if (++stage == S::XS) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------ quantised weight chunks
        if (lane == 0) {
            prefetch_tensormap(&tm_q);
            int slot = 0; uint32_t phase = 0;
            const int nchunks = kbp / SPQ;
            for (int tile = blockIdx.x; tile < ntiles && !*abort_flag; tile += gridDim.x) {
                const int n0 = (tile / tiles_m) * WQ_ROWS;
                for (int c = 0; c < nchunks; ++c) {
                    if (!mbar_wait(qempty(slot), phase ^ 1, abort_flag)) { atomicExch(&g_wq_status, 302); *abort_flag = 1; break; }
                    mbar_arrive_expect_tx(qfull(slot), Q_TX);
                    if (MODE == WQ_INT8T) tma_load_2d(sb + S::Q_OFF + slot * WQ_Q_BYTES, &tm_q, qfull(slot), n0, c * WQ_BK);
                    else tma_load_2d(sb + S::Q_OFF + slot * WQ_Q_BYTES, &tm_q, qfull(slot), c * 128, n0);
                    if (++slot == S::QS) { slot = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(a.fmt, WQ_ROWS, TM);
            int ws = 0; uint32_t wph = 0;
            int xs = 0; uint32_t xph = 0;
            int acc = 0; uint32_t acc_phase = 0;
            for (int tile = blockIdx.x; tile < ntiles && !*abort_flag; tile += gridDim.x) {
                if (!mbar_wait(tempty(acc), acc_phase ^ 1, abort_flag)) { atomicExch(&g_wq_status, 303); *abort_flag = 1; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * TM);
                bool ok = true;
                for (int kb = 0; kb < kbp; ++kb) {
                    if (!mbar_wait(wfull(ws), wph, abort_flag)) { atomicExch(&g_wq_status, 304); *abort_flag = 1; ok = false; break; }
                    if (!mbar_wait(xfull(xs), xph, abort_flag)) { atomicExch(&g_wq_status, 305); *abort_flag = 1; ok = false; break; }
                    tc_fence_after();
                    const uint64_t da = umma_desc_k_sw128(sb + S::W_OFF + ws * WQ_W_BYTES);
                    const uint64_t db = umma_desc_k_sw128(sb + S::X_OFF + xs * S::X_BYTES);
#pragma unroll
                    for (int k = 0; k < WQ_BK / 16; ++k)
                        umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, kb > 0 || k > 0);
                    umma_commit(wempty(ws));
                    umma_commit(xempty(xs));
                    if (++ws == WQ_WS) { ws = 0; wph ^= 1; }
                    if (++xs == S::XS) { xs = 0; xph ^= 1; }
                }
                if (!ok) break;
                umma_commit(tfull(acc));
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else if (warp < 7) {
        // ------------------------------------------------------------ epilogue (warps 3..6)
        const int q = warp & 3;                                  // the TMEM lane quarter this warp may read
        int acc = 0; uint32_t acc_phase = 0;
        for (int tile = blockIdx.x; tile < ntiles && !*abort_flag; tile += gridDim.x) {
            const int m0 = (tile % tiles_m) * TM, n0 = (tile / tiles_m) * WQ_ROWS;
            const int n = n0 + q * 32 + lane;
            const bool n_ok = n < a.N;
            float ws = 1.0f, bv = 0.0f;
            if (n_ok) {
                if (a.wscale != nullptr) {
                    const float s = __ldg(a.wscale + n);
                    ws = (a.wscale_sqrt ? sqrtf(s) : s) * a.wscale_mul;
                }
                if (a.bias != nullptr)
                    bv = a.fmt == 0 ? __half2float(reinterpret_cast<const __half *>(a.bias)[n])
                                    : __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(a.bias)[n]);
            }
            if (!mbar_wait(tfull(acc), acc_phase, abort_flag)) { atomicExch(&g_wq_status, 306); *abort_flag = 1; break; }
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * TM);
#pragma unroll 1
            for (int c0 = 0; c0 < TM; c0 += 32) {
                if (m0 + c0 >= a.M) break;                       // warp-uniform
                uint32_t v[32];
                tmem_ld_32x32(t_row + (uint32_t)c0, v);
                tmem_ld_wait();
                if (n_ok) {
                    const int mlim = a.M - (m0 + c0);
                    const int64_t o = (int64_t)(m0 + c0) * a.N + n;
                    if (a.y_dtype == MPSBNB_F16) {
                        __half *y = reinterpret_cast<__half *>(a.y) + o;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < mlim) y[(int64_t)j * a.N] = __float2half_rn(fmaf(__uint_as_float(v[j]), ws, bv));
                    } else if (a.y_dtype == MPSBNB_BF16) {
                        __nv_bfloat16 *y = reinterpret_cast<__nv_bfloat16 *>(a.y) + o;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < mlim) y[(int64_t)j * a.N] = __float2bfloat16_rn(fmaf(__uint_as_float(v[j]), ws, bv));
                    } else {
                        float *y = reinterpret_cast<float *>(a.y) + o;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < mlim) y[(int64_t)j * a.N] = fmaf(__uint_as_float(v[j]), ws, bv);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    } else if (wq_expander_index(warp) >= 0) {
        // ------------------------------------------------------------ expanders (sixteen of the warps 7..27)
        // Two groups of eight warps; group g expands the K steps kb = g, g + 2, ... of every tile, alternating between
        // two W stages of its own, so that it can fill one while the tensor core still reads the other.  Thread
        // (r, h) of a group owns half a weight row of the stage (32 k): 16 packed bytes in, 64 bytes out.
        const int ew = wq_expander_index(warp);
        const int grp = ew / WQ_GROUP_WARPS;
        // lanes 0-15 of a warp take the first half (h = 0) of sixteen consecutive rows, lanes 16-31 the second: eight
        // consecutive lanes then touch eight different 16-byte columns of the swizzled tiles (no bank conflicts)
        const int r = (ew % WQ_GROUP_WARPS) * 16 + (lane & 15), h = lane >> 4, sw = r & 7;
        const uint32_t lut_lane = sb + (uint32_t)S::LUT_OFF + (uint32_t)lane * 4u;
        int qc0 = 0, kb0 = 0;                                        // chunks / K steps of the tiles before this one
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok && !*abort_flag; tile += gridDim.x, qc0 += kbp / SPQ, kb0 += kbp) {
            const int n0 = (tile / tiles_m) * WQ_ROWS;
            const int n = n0 + r;
            const bool row_ok = n < a.N;
            auto scale_of = [&](int kb) -> float {               // 4-bit: the block's absmax as fp32
                if (MODE != WQ_4BIT || !row_ok || kb >= a.nb) return 0.0f;
                const int64_t i = (int64_t)n * a.nb + kb;
                if (a.absmax2 == nullptr) return __ldg(reinterpret_cast<const float *>(a.absmax) + i);
                // divide first, then multiply, as functional.py:592-593
                return __fmul_rn((float)__ldg(reinterpret_cast<const int8_t *>(a.absmax) + i), __fdiv_rn(__ldg(a.absmax2 + (i >> 8)), 127.0f));
            };
            // Block scales of a 256-k chunk (four blocks) come in one aligned load per row, fetched one chunk ahead and
            // converted when the chunk starts (rows of absmax whose length is not a multiple of 4 use scale_of per step).
            const bool vec = MODE == WQ_4BIT && (a.nb & 3) == 0;
            uint32_t rq = 0u; float4 rf = make_float4(0.f, 0.f, 0.f, 0.f); float ra2 = 0.0f;
            float sc4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            auto issue = [&](int c) {
                rq = 0u; rf = make_float4(0.f, 0.f, 0.f, 0.f); ra2 = 0.0f;
                if (!vec || !row_ok || 4 * c >= a.nb) return;
                const int64_t i = (int64_t)n * a.nb + 4 * c;
                if (a.absmax2 == nullptr) rf = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(a.absmax) + i));
                else { rq = __ldg(reinterpret_cast<const uint32_t *>(reinterpret_cast<const int8_t *>(a.absmax) + i)); ra2 = __ldg(a.absmax2 + (i >> 8)); }
            };
            auto convert = [&]() {
                if (a.absmax2 == nullptr) { sc4[0] = rf.x; sc4[1] = rf.y; sc4[2] = rf.z; sc4[3] = rf.w; }
                else {
                    const float f = __fdiv_rn(ra2, 127.0f);        // divide first, then multiply, as functional.py:592-593
#pragma unroll
                    for (int j = 0; j < 4; ++j) sc4[j] = __fmul_rn((float)(int)(int8_t)((rq >> (8 * j)) & 0xFFu), f);
                }
            };
            if (vec) issue(0);
            for (int kb = grp; kb < kbp; kb += WQ_GROUPS) {
                const int ks = kb % SPQ;
                const int qc = qc0 + kb / SPQ;
                const int qs = qc % S::QS;
                const int ws = kb % WQ_WS;                       // kbp is a multiple of WQ_WS: the ring position of step kb
                const uint32_t wvisit = (uint32_t)((kb0 + kb) / WQ_WS);
                const uint32_t wrow = sb + (uint32_t)(S::W_OFF + ws * WQ_W_BYTES + r * 128);
                float s_cur = 0.0f;
                if (MODE == WQ_4BIT) {
                    if (vec) {
                        if ((kb & 3) < WQ_GROUPS) { convert(); issue((kb >> 2) + 1); }   // my first step of this chunk
                        s_cur = (kb & 3) == 0 ? sc4[0] : (kb & 3) == 1 ? sc4[1] : (kb & 3) == 2 ? sc4[2] : sc4[3];
                    } else {
                        s_cur = scale_of(kb);
                    }
                }
                if (!mbar_wait(qfull(qs), (uint32_t)(qc / S::QS) & 1u, abort_flag)) { atomicExch(&g_wq_status, 307); *abort_flag = 1; ok = false; break; }
                if (!mbar_wait(wempty(ws), (wvisit & 1u) ^ 1u, abort_flag)) { atomicExch(&g_wq_status, 308); *abort_flag = 1; ok = false; break; }
                const uint32_t qrow = sb + (uint32_t)(S::Q_OFF + qs * WQ_Q_BYTES + r * 128);
                if (MODE == WQ_4BIT) {
                    // fp16 operands and a scale well inside the fp16 range: one packed multiply per pair; otherwise the
                    // product is formed in fp32 and rounded once
                    const bool fast = FMT == 0 && __all_sync(0xffffffffu, s_cur == 0.0f || (s_cur >= 0.001953125f && s_cur <= 32768.0f));
                    const __half2 s2 = __float2half2_rn(s_cur);
                    {
                        const uint4 v = wq_lds128(qrow + (uint32_t)((((ks << 1) | h) ^ sw) << 4));
                        const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t w = w4[j];
                            uint32_t p[4];
                            p[0] = wq_lut(lut_lane + __byte_perm(w, 0u, 0x4440) * 128u);
                            p[1] = wq_lut(lut_lane + __byte_perm(w, 0u, 0x4441) * 128u);
                            p[2] = wq_lut(lut_lane + __byte_perm(w, 0u, 0x4442) * 128u);
                            p[3] = wq_lut(lut_lane + __byte_perm(w, 0u, 0x4443) * 128u);
                            if (fast) {
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const __half2 o = __hmul2(*reinterpret_cast<const __half2 *>(&p[e]), s2);
                                    p[e] = *reinterpret_cast<const uint32_t *>(&o);
                                }
                            } else {
#pragma unroll
                                for (int e = 0; e < 4; ++e) p[e] = wq_scale_pair<FMT>(p[e], s_cur);
                            }
                            wq_sts128(wrow + (uint32_t)((((h << 2) | j) ^ sw) << 4), p[0], p[1], p[2], p[3]);
                        }
                    }
                } else if (MODE == WQ_INT8T) {
                    // The chunk is [64 k][128 n] bytes, unswizzled.  Thread (kg = warp of the group, lane) reads the
                    // words of n = 4 lane .. 4 lane + 3 for k = 8 kg .. 8 kg + 7 (a warp reads 128 consecutive bytes per
                    // k) and writes, for each of its four n, the eight k as one 16-byte column of W row n.  The four
                    // rows are written in a lane-dependent order so that eight consecutive lanes hit eight different columns.
                    const int kg = ew % WQ_GROUP_WARPS;
                    const uint32_t qb = sb + (uint32_t)(S::Q_OFF + qs * WQ_Q_BYTES + kg * 8 * 128 + lane * 4);
                    uint32_t wk[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(wk[i]) : "r"(qb + (uint32_t)(i * 128)) : "memory");
                    const uint32_t wtile = sb + (uint32_t)(S::W_OFF + ws * WQ_W_BYTES);
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const int j = (t + (lane >> 1)) & 3;
                        const int nn = 4 * lane + j;
                        uint32_t o[4];
                        if (FMT == 0) {
                            const uint32_t sel = 0x4400u + 0x1111u * (uint32_t)j;      // byte j of both words -> bytes 0 and 2
                            const __half2 k1152 = __floats2half2_rn(1152.0f, 1152.0f);
#pragma unroll
                            for (int pp = 0; pp < 4; ++pp) {
                                const uint32_t u = (__byte_perm(wk[2 * pp], wk[2 * pp + 1], sel) & 0x00FF00FFu) ^ 0x64806480u;
                                const __half2 v2 = __hsub2(*reinterpret_cast<const __half2 *>(&u), k1152);
                                o[pp] = *reinterpret_cast<const uint32_t *>(&v2);
                            }
                        } else {
#pragma unroll
                            for (int pp = 0; pp < 4; ++pp) {
                                const int b0 = (int)(int8_t)((wk[2 * pp] >> (8 * j)) & 0xFFu), b1 = (int)(int8_t)((wk[2 * pp + 1] >> (8 * j)) & 0xFFu);
                                const __nv_bfloat162 v2 = __floats2bfloat162_rn((float)b0, (float)b1);
                                o[pp] = *reinterpret_cast<const uint32_t *>(&v2);
                            }
                        }
                        wq_sts128(wtile + (uint32_t)(nn * 128 + ((kg ^ (nn & 7)) << 4)), o[0], o[1], o[2], o[3]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint4 v = wq_lds128(qrow + (uint32_t)((((ks << 2) | (h << 1) | j) ^ sw) << 4));
                        uint32_t o[8];
                        if (MODE == WQ_INT8) {
                            wq_i8x4<FMT>(v.x, o[0], o[1]); wq_i8x4<FMT>(v.y, o[2], o[3]); wq_i8x4<FMT>(v.z, o[4], o[5]); wq_i8x4<FMT>(v.w, o[6], o[7]);
                        } else {
                            wq_f8x4<FMT>(v.x, o[0], o[1]); wq_f8x4<FMT>(v.y, o[2], o[3]); wq_f8x4<FMT>(v.z, o[4], o[5]); wq_f8x4<FMT>(v.w, o[6], o[7]);
                        }
                        wq_sts128(wrow + (uint32_t)((((h << 2) | (j << 1)) ^ sw) << 4), o[0], o[1], o[2], o[3]);
                        wq_sts128(wrow + (uint32_t)((((h << 2) | (j << 1) | 1) ^ sw) << 4), o[4], o[5], o[6], o[7]);
                    }
                }
                fence_proxy_async_smem();                        // my stores before the tensor core's reads
                __syncwarp();
                if (lane == 0) { mbar_arrive(wfull(ws)); mbar_arrive(qempty(qs)); }   // every lane has read its bytes
            }
        }
    }

    // common exit: every role arrives here (also after a time-out), then TMEM is released
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * TM);
    }
}

// x'[m, k] = x[m, k] * sqrt(c[k]) in the operand type: the column half of the col+row scale sqrt(r[n] c[k])
// (mps_bitsandbytes/functional.py:896-945) moved from the weight onto the activations
template <typename T>
__global__ void scale_cols_kernel(const T *__restrict__ x, int64_t M, int64_t K, int64_t ldx, const float *__restrict__ c,
                                  T *__restrict__ out, int64_t ldo) {
    const int64_t total = M * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / K, k = i - m * K;
        out[m * ldo + k] = from_f32<T>(to_f32<T>(x[m * ldx + k]) * sqrtf(__ldg(c + k)));
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*WqEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static WqEncodeFn wq_encode_fn() {
    static WqEncodeFn fn = nullptr;
    if (fn == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<WqEncodeFn>(p);
    }
    return fn;
}

template <int TM, int MODE, int FMT>
static int wq_launch(const CUtensorMap &mx, const CUtensorMap &mq, const WqArgs &args, cudaStream_t st) {
    using S = WqSmem<TM>;
    constexpr int smem = S::TOTAL + 1024;                      // slack for the 1024-byte alignment of the rings
    static_assert(smem <= 227 * 1024, "shared memory of the fused GEMM exceeds the CTA limit");
    static bool configured[64] = {};
    int dev = 0;
    MPSBNB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        MPSBNB_CUDA_TRY(cudaFuncSetAttribute(mpsbnb_gemm_wq_kernel<TM, MODE, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int tiles = ((args.M + TM - 1) / TM) * ((args.N + WQ_ROWS - 1) / WQ_ROWS);
    int grid = sm_count();
    if (grid > tiles) grid = tiles;
    mpsbnb_gemm_wq_kernel<TM, MODE, FMT><<<grid, WQ_THREADS, smem, st>>>(mx, mq, args);
    return check_launch();
}

template <int MODE, int FMT>
static int wq_launch_tm(int tm, const CUtensorMap &mx, const CUtensorMap &mq, const WqArgs &args, cudaStream_t st) {
    switch (tm) {
        case 32: return wq_launch<32, MODE, FMT>(mx, mq, args, st);
        case 64: return wq_launch<64, MODE, FMT>(mx, mq, args, st);
        case 128: return wq_launch<128, MODE, FMT>(mx, mq, args, st);
        default: return wq_launch<256, MODE, FMT>(mx, mq, args, st);
    }
}

bool gemm_wq_supported(const void *x, int64_t ldx, const void *wq, int64_t row_bytes) {
    return aligned16(x) && ldx % 8 == 0 && aligned16(wq) && row_bytes % 16 == 0;
}

// mode: WQ_4BIT (wq = packed [N, row_bytes = Kp / 2]), WQ_INT8 / WQ_FP8 (wq = codes [N, row_bytes = K]),
// WQ_INT8T (wq = int8 [K, row_bytes = N]: the B operand of matmul_int8).
int gemm_wq(int mode, const void *x, int64_t ldx, int x_dtype, int64_t M, const void *wq, int64_t row_bytes,
            const void *absmax, const float *absmax2, const float *wscale, float wscale_mul, int wscale_sqrt, int64_t N,
            int64_t K, int quant_type, const void *bias, void *y, int y_dtype, cudaStream_t st) {
    if (!is_16bit(x_dtype) || !valid_dtype(y_dtype)) return MPSBNB_ERR_INVALID_ARG;
    if (M <= 0 || N <= 0) return MPSBNB_OK;
    if (K <= 0) return MPSBNB_ERR_UNSUPPORTED;
    if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return MPSBNB_ERR_TOO_LARGE;
    if (!gemm_wq_supported(x, ldx, wq, row_bytes)) return MPSBNB_ERR_UNSUPPORTED;
    WqEncodeFn fn = wq_encode_fn();
    if (fn == nullptr) return MPSBNB_ERR_NO_DEVICE;
    const int tm = M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    CUtensorMap mx, mq;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
        const cuuint32_t box[2] = {64u, (cuuint32_t)tm};
        const cuuint32_t estr[2] = {1u, 1u};
        if (fn(&mx, x_dtype == MPSBNB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
               const_cast<void *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return MPSBNB_ERR_INVALID_ARG;
    }
    if (mode == WQ_INT8T) {
        // B int8 [K, N]: box = 128 n-bytes x 64 k-rows, no swizzle (row_bytes = N)
        const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K};
        const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
        const cuuint32_t box[2] = {128u, (cuuint32_t)WQ_BK};
        const cuuint32_t estr[2] = {1u, 1u};
        if (fn(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(wq), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return MPSBNB_ERR_INVALID_ARG;
    } else {
        const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)N};
        const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
        const cuuint32_t box[2] = {128u, (cuuint32_t)WQ_ROWS};
        const cuuint32_t estr[2] = {1u, 1u};
        if (fn(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(wq), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return MPSBNB_ERR_INVALID_ARG;
    }
    WqArgs a;
    memset(&a, 0, sizeof(a));
    a.absmax = absmax; a.absmax2 = absmax2; a.wscale = wscale; a.wscale_mul = wscale_mul; a.wscale_sqrt = wscale_sqrt;
    a.bias = bias; a.y = y; a.y_dtype = y_dtype; a.fmt = x_dtype == MPSBNB_F16 ? 0 : 1;
    a.M = (int)M; a.N = (int)N; a.K = (int)K; a.nb = (int)(padded_k(K, 64) / 64); a.quant_type = quant_type;
    const bool f16 = x_dtype == MPSBNB_F16;
    if (mode == WQ_4BIT) return f16 ? wq_launch_tm<WQ_4BIT, 0>(tm, mx, mq, a, st) : wq_launch_tm<WQ_4BIT, 1>(tm, mx, mq, a, st);
    if (mode == WQ_INT8) return f16 ? wq_launch_tm<WQ_INT8, 0>(tm, mx, mq, a, st) : wq_launch_tm<WQ_INT8, 1>(tm, mx, mq, a, st);
    if (mode == WQ_FP8) return f16 ? wq_launch_tm<WQ_FP8, 0>(tm, mx, mq, a, st) : wq_launch_tm<WQ_FP8, 1>(tm, mx, mq, a, st);
    if (mode == WQ_INT8T) return f16 ? wq_launch_tm<WQ_INT8T, 0>(tm, mx, mq, a, st) : wq_launch_tm<WQ_INT8T, 1>(tm, mx, mq, a, st);
    return MPSBNB_ERR_INVALID_ARG;
}

int scale_cols_16bit(const void *x, int64_t M, int64_t K, int64_t ldx, const float *c, void *out, int64_t ldo, int dtype,
                     cudaStream_t st) {
    const int64_t total = M * K;
    const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dtype == MPSBNB_F16)
        scale_cols_kernel<__half><<<grid, 256, 0, st>>>((const __half *)x, M, K, ldx, c, (__half *)out, ldo);
    else
        scale_cols_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16 *)x, M, K, ldx, c, (__nv_bfloat16 *)out, ldo);
    return check_launch();
}

int wq_status_fetch(int *out, bool reset) {
    MPSBNB_CUDA_TRY(cudaMemcpyFromSymbol(out, g_wq_status, sizeof(int)));
    if (reset) {
        const int zero = 0;
        MPSBNB_CUDA_TRY(cudaMemcpyToSymbol(g_wq_status, &zero, sizeof(int)));
    }
    return MPSBNB_OK;
}

}  // namespace mpsbnb
