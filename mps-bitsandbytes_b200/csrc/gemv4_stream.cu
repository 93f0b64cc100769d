// Streaming decode GEMV for 4-bit weights (block size 64), batch M <= 8, one or many linears
// per launch:   y[m, n] = sum_k x[m, k] * code[W[n, k]] * absmax[n, k / 64]   (+ bias[n]).
// Stands for mps_bitsandbytes/functional.py:680-773 on decode shapes (the reference's Metal
// analogue is nf4_matmul_simd, mps_bitsandbytes.mm:440-560, launched once per linear).
//
// Bound: HBM.  Every packed byte crosses the memory system once.  One persistent CTA per SM
// with 22 warps:
//   warp 16  TMA producer.  Work is cut into units of 32 weight rows x a run of stages; a
//            stage is 32 rows x 1024 k = 16 KB of packed bytes, fetched as four
//            cp.async.bulk.tensor boxes (32 rows x 128 B, 128-byte swizzle) into a ring of
//            shared-memory slots.  The ring keeps 100+ KB in flight per SM regardless of what the
//            consumers are doing (register prefetch could not: it was the limiter before).
//   warps 17-20  loaders, taking stages in turn.  For its stage a loader writes, into the same
//            slot, the 32 x 16 block scales already expanded to fp32 (double-quantised absmax is
//            int8 * absmax2 / 127) and the 1024 x values of each batch row, so consumers never
//            touch global memory.  Four of them keep four stages' worth of loads in flight.
//   warps 0-15  consumers.  Warp (rt, kg) owns row tile rt (16 rows) and blocks 2 kg, 2 kg + 1
//            of every stage.  Per block: two 8-byte shared loads (rows g and g + 8 — the swizzle
//            and a row permutation make them bank-conflict free), 16 table lookups that turn a
//            packed byte into a pair of 16-bit codes (one byte-permute + one shared load each,
//            table replicated per lane), 4 mma.sync.m16n8k16 with the weights as the M side,
//            then one fp32 multiply-add per row with the block scale.
//   warp 21  reducer.  At the end of a unit every consumer warp drops its partial sums into a
//            double-buffered shared array and signals an mbarrier; the reducer adds the eight kg
//            partials of each row and stores them (or atomically adds them to an fp32
//            accumulator when K is split across units or several linears sum into one output).
//            Consumers never wait for each other, and producers run ahead into the next unit, so
//            the HBM stream does not pause at unit boundaries.
// All waits are bounded (see sm100.cuh); a time-out sets the device status word.
#include "common.cuh"
#include <cstdio>
#include <cstdlib>
#include "ops.cuh"
#include "sm100.cuh"

#include <stdlib.h>
#include <type_traits>
#include <string.h>

namespace mpsbnb {

using namespace sm100;

constexpr int SG_CONSUMERS = 16;
constexpr int SG_GROUPS = 4;                             // independent consumer groups (each takes every 4th stage)
constexpr int SG_GROUP_WARPS = SG_CONSUMERS / SG_GROUPS;
constexpr int SG_ITEMS = 8 / (SG_GROUP_WARPS / 2);       // block pairs a warp works through per stage
constexpr int SG_LOADERS = 4;                           // must equal SG_MAX_XS (see there)
constexpr int SG_THREADS = (SG_CONSUMERS + 1 + SG_LOADERS + 2) * 32;   // + TMA warp + reducer warp + closer warp
constexpr int SG_MAIL = 4;                               // mailbox entries between reducer and closer
constexpr int SG_ROWS = 32;                              // weight rows per unit
constexpr int SG_STAGE_BLOCKS = 16;                      // quantisation blocks (of 64 k) per stage
constexpr int SG_W_BYTES = SG_ROWS * SG_STAGE_BLOCKS * 32;   // 16384 packed bytes per stage
constexpr int SG_A_BYTES = SG_STAGE_BLOCKS * SG_ROWS * 4;    // 2048: fp32 scale [block][row]
constexpr int SG_XPITCH = 2048 + 64;                     // bytes between batch rows of x in a slot
constexpr int SG_RED_BYTES = SG_CONSUMERS * 8 * 20 * 4;  // [warp][m][16 rows + 4 pad] fp32
constexpr int SG_MAX_SLOTS = 8;
constexpr int SG_MAX_M = 8;

// status word of this translation unit (device code is not linked relocatably); read by
// stream_status_fetch() on behalf of mpsbnb_device_status()
static __device__ int g_stream_status = 0;
// the FIRST wait that gave up names the cause; the others give up because of it
__device__ __forceinline__ void sg_fail(int code) { atomicCAS(&g_stream_status, 0, code); }

#ifdef MPSBNB_TRACE
// Development aid (compiled in with -DMPSBNB_TRACE only): per segment, when CTA 0's first loader began and ended its
// wait for the segment's input flags, and when this GPU raised its own flag; nanoseconds of %globaltimer.
static __device__ unsigned long long g_trace[3 * 256];
__device__ __forceinline__ unsigned long long trace_now() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define MPSBNB_TRACE_SET(slot, seg) do { if ((seg) >= 0 && (seg) < 256) g_trace[(slot) * 256 + (seg)] = trace_now(); } while (0)
// cycles CTA 0's roles spend inside each kind of barrier wait (lane 0 of every warp adds its own), [15] = CTA 0's total
static __device__ unsigned long long g_wait[16];
static __device__ unsigned int g_fail[8];
#define SG_FAIL_DETAIL(a_, b_, c_, d_, e_) do { if (atomicCAS(&g_fail[0], 0u, 1u) == 0u) { g_fail[1] = blockIdx.x; g_fail[2] = (a_); g_fail[3] = (b_); g_fail[4] = (c_); g_fail[5] = (d_); g_fail[6] = (e_); } } while (0)
#define SG_TIMED(idx, expr) ([&]() { const long long t0_ = clock64(); const bool r_ = (expr); if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) atomicAdd(&g_wait[idx], (unsigned long long)(clock64() - t0_)); return r_; }())
#else
#define MPSBNB_TRACE_SET(slot, seg) do { } while (0)
#define SG_TIMED(idx, expr) (expr)
#define SG_FAIL_DETAIL(a_, b_, c_, d_, e_) do { } while (0)
#endif


struct StreamLinear {
    CUtensorMap map;          // packed weights as [N][row_bytes] bytes; box 128 B x 32 rows, 128-byte swizzle
    const void *x;            // activations [M, x_ld]; column index is taken modulo x_period
    const void *absmax;       // fp32 [N, nb], or int8 [N, nb] when absmax2 != nullptr
    const float *absmax2;     // fp32 [ceil(N nb / 256)] or nullptr
    const void *bias;         // [N] in the activation dtype, or nullptr
    void *y;                  // [M, N] in y_dtype; used when acc == nullptr
    float *acc;               // fp32 [M, N] atomicAdd target, or nullptr
    int64_t x_ld;
    int N, K, nb, nbv;        // nb: blocks per row in the layout; nbv: blocks that hold real k
    int x_period;             // x column = k mod x_period (x_period >= K: plain)
    int y_dtype;
    int x_vec_ok;             // 16-byte loads of x are legal
    int x_bulk_ok;            // every stage's x columns are one 16-byte-aligned contiguous run: TMA bulk copies
    int map3d;                // map is {128 B, N rows, row_bytes / 128}: one box {128, 32, 4} fetches a whole stage
    int segment;              // linears of segment g + 1 read what the closing step of segment g wrote
};

// nbv: copy of the linear's count of blocks that hold real k - what the consumer warps need of the linear, so that a
// unit switch costs them no dependent global load
struct __align__(16) StreamUnit { int lin, row0, s_begin, s_end, nbv, pad0, pad1, pad2; };

struct StreamArgs {
    const StreamLinear *lins; // device array, or nullptr: use `one`
    const StreamUnit *units;  // device array, or nullptr: unit u = rows [32 u, 32 u + 32) x all stages of `one`
    int nunits, M, quant_type;
    uint32_t zero;            // always 0; known only at run time (orders the slot release after the loads)
    const int *wait_flags;    // wait_n flags in this GPU's memory that the loaders wait for before the first read of x:
    const int *wait_step;     //   every flag >= (*wait_step) * wait_mul + wait_add  (peers raise them, see exchange.cu)
    int wait_n, wait_mul, wait_add, wait_seg_mul;
    int x_ll;                 // x of every linear is in tagged form: 8-byte entries {two 16-bit values, tag} (see the closer warp)
    mpsbnb_group_epilogue ep; // closing step by the last CTA (ep.acc == nullptr: none)
    uint32_t sleep_cons;      // ns a consumer warp sleeps between probes of a barrier that is not ready
    uint32_t sleep_other;     // same for the producer, loader and reducer warps
    StreamLinear one;
};

__device__ __forceinline__ void mma16816_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma16816_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename XT> __device__ __forceinline__ void mma_x(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma_x<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) { mma16816_f16(d, a0, a1, a2, a3, b0, b1); }
template <> __device__ __forceinline__ void mma_x<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) { mma16816_bf16(d, a0, a1, a2, a3, b0, b1); }

template <typename XT> __device__ __forceinline__ uint32_t pair_bits(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pair_bits<__half>(float lo, float hi) { const __half2 h = __floats2half2_rn(lo, hi); return *reinterpret_cast<const uint32_t *>(&h); }
template <> __device__ __forceinline__ uint32_t pair_bits<__nv_bfloat16>(float lo, float hi) { const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<const uint32_t *>(&h); }

// ---- shared-memory access by 32-bit shared address (no generic-pointer arithmetic in the hot loop)
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// A consumer warp's inner loop is written in PTX so that the instruction stream is what the design
// counts on.  Per stage a warp owns two quantisation blocks (16 weight rows x 64 k each).
//
// fetch_stage: four 8-byte shared loads bring the packed bytes of both blocks into registers
//   (w[0..1]: block 0 row g, w[2..3]: block 0 row g + 8, w[4..7]: block 1).  After it the weight
//   slot is no longer needed by this warp.
__device__ __forceinline__ void fetch_stage(uint32_t (&w)[8], uint32_t wa0, uint32_t wa1) {
    asm volatile(
        "ld.shared.v2.u32 {%0, %1}, [%8];\n\t"
        "ld.shared.v2.u32 {%2, %3}, [%8+1024];\n\t"
        "ld.shared.v2.u32 {%4, %5}, [%9];\n\t"
        "ld.shared.v2.u32 {%6, %7}, [%9+1024];\n\t"
        : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
        : "r"(wa0), "r"(wa1)
        : "memory");
}

// Sixteen (byte-permute, table load) pairs: packed bytes of rows g (wa, wb) and g + 8 (wc, wd) become
// the A fragments F0..F15 of four MMAs.  LW is the lane word of the table address.
#define MPSBNB_LUT16(F, WA, WB, WC, WD, LW)                                                    \
    "prmt.b32 ad, " WA ", " LW ", 0x7604;\n\t ld.shared.u32 " F "0, [ad];\n\t"                   \
    "prmt.b32 ad, " WC ", " LW ", 0x7604;\n\t ld.shared.u32 " F "1, [ad];\n\t"                   \
    "prmt.b32 ad, " WA ", " LW ", 0x7614;\n\t ld.shared.u32 " F "2, [ad];\n\t"                   \
    "prmt.b32 ad, " WC ", " LW ", 0x7614;\n\t ld.shared.u32 " F "3, [ad];\n\t"                   \
    "prmt.b32 ad, " WA ", " LW ", 0x7624;\n\t ld.shared.u32 " F "4, [ad];\n\t"                   \
    "prmt.b32 ad, " WC ", " LW ", 0x7624;\n\t ld.shared.u32 " F "5, [ad];\n\t"                   \
    "prmt.b32 ad, " WA ", " LW ", 0x7634;\n\t ld.shared.u32 " F "6, [ad];\n\t"                   \
    "prmt.b32 ad, " WC ", " LW ", 0x7634;\n\t ld.shared.u32 " F "7, [ad];\n\t"                   \
    "prmt.b32 ad, " WB ", " LW ", 0x7604;\n\t ld.shared.u32 " F "8, [ad];\n\t"                   \
    "prmt.b32 ad, " WD ", " LW ", 0x7604;\n\t ld.shared.u32 " F "9, [ad];\n\t"                   \
    "prmt.b32 ad, " WB ", " LW ", 0x7614;\n\t ld.shared.u32 " F "10, [ad];\n\t"                  \
    "prmt.b32 ad, " WD ", " LW ", 0x7614;\n\t ld.shared.u32 " F "11, [ad];\n\t"                  \
    "prmt.b32 ad, " WB ", " LW ", 0x7624;\n\t ld.shared.u32 " F "12, [ad];\n\t"                  \
    "prmt.b32 ad, " WD ", " LW ", 0x7624;\n\t ld.shared.u32 " F "13, [ad];\n\t"                  \
    "prmt.b32 ad, " WB ", " LW ", 0x7634;\n\t ld.shared.u32 " F "14, [ad];\n\t"                  \
    "prmt.b32 ad, " WD ", " LW ", 0x7634;\n\t ld.shared.u32 " F "15, [ad];\n\t"

#define MPSBNB_MMA(TYPE, D, A0, A1, A2, A3, B0, B1, C)                                         \
    "mma.sync.aligned.m16n8k16.row.col.f32." TYPE "." TYPE ".f32 {" D "0," D "1," D "2," D "3}, {" A0 "," A1 "," A2 "," A3 "}, {" B0 "," B1 "}, " C ";\n\t"

// compute_stage: both blocks of a stage.  x (16 values per block; lanes without a batch row read a
// zero area) and the four block scales come from the scale/x slot at xa0, xa1, aa0, aa1; the 32 table
// loads of both blocks are issued before the first MMA, the two MMA chains are interleaved, and eight
// FMAs apply the scales.  The weight registers were filled by fetch_stage one iteration earlier.
#define MPSBNB_STAGE_ASM(TYPE)                                                                              \
    asm volatile(                                                                                           \
        "{\n\t"                                                                                             \
        ".reg .b32 ad, x<8>, y<8>;\n\t"                                                                     \
        ".reg .b32 f<16>, g<16>;\n\t"                                                                       \
        ".reg .f32 m<4>, t<4>, u<4>, z;\n\t"                                                                \
        ".reg .pred px;\n\t"                                                                                \
        "setp.ne.u32 px, %17, 0;\n\t"                                                                       \
        "mov.b32 x0, 0;\n\t mov.b32 x1, 0;\n\t mov.b32 x2, 0;\n\t mov.b32 x3, 0;\n\t"                       \
        "mov.b32 x4, 0;\n\t mov.b32 x5, 0;\n\t mov.b32 x6, 0;\n\t mov.b32 x7, 0;\n\t"                       \
        "mov.b32 y0, 0;\n\t mov.b32 y1, 0;\n\t mov.b32 y2, 0;\n\t mov.b32 y3, 0;\n\t"                       \
        "mov.b32 y4, 0;\n\t mov.b32 y5, 0;\n\t mov.b32 y6, 0;\n\t mov.b32 y7, 0;\n\t"                       \
        "@px ld.shared.v4.u32 {x0, x1, x2, x3}, [%14];\n\t"                                                 \
        "@px ld.shared.v4.u32 {x4, x5, x6, x7}, [%14+16];\n\t"                                              \
        "@px ld.shared.v4.u32 {y0, y1, y2, y3}, [%15];\n\t"                                                 \
        "@px ld.shared.v4.u32 {y4, y5, y6, y7}, [%15+16];\n\t"                                              \
        "ld.shared.f32 m0, [%12];\n\t"                                                                      \
        "ld.shared.f32 m1, [%12+32];\n\t"                                                                   \
        "ld.shared.f32 m2, [%13];\n\t"                                                                      \
        "ld.shared.f32 m3, [%13+32];\n\t"                                                                   \
        "mov.f32 z, 0f00000000;\n\t"                                                                        \
        MPSBNB_LUT16("f", "%4", "%5", "%6", "%7", "%16")                                                    \
        MPSBNB_LUT16("g", "%8", "%9", "%10", "%11", "%16")                                                  \
        MPSBNB_MMA(TYPE, "t", "f0", "f1", "f2", "f3", "x0", "x1", "{z,z,z,z}")                              \
        MPSBNB_MMA(TYPE, "u", "g0", "g1", "g2", "g3", "y0", "y1", "{z,z,z,z}")                              \
        MPSBNB_MMA(TYPE, "t", "f4", "f5", "f6", "f7", "x2", "x3", "{t0,t1,t2,t3}")                          \
        MPSBNB_MMA(TYPE, "u", "g4", "g5", "g6", "g7", "y2", "y3", "{u0,u1,u2,u3}")                          \
        MPSBNB_MMA(TYPE, "t", "f8", "f9", "f10", "f11", "x4", "x5", "{t0,t1,t2,t3}")                        \
        MPSBNB_MMA(TYPE, "u", "g8", "g9", "g10", "g11", "y4", "y5", "{u0,u1,u2,u3}")                        \
        MPSBNB_MMA(TYPE, "t", "f12", "f13", "f14", "f15", "x6", "x7", "{t0,t1,t2,t3}")                      \
        MPSBNB_MMA(TYPE, "u", "g12", "g13", "g14", "g15", "y6", "y7", "{u0,u1,u2,u3}")                      \
        "fma.rn.f32 %0, m0, t0, %0;\n\t fma.rn.f32 %1, m0, t1, %1;\n\t"                                     \
        "fma.rn.f32 %2, m1, t2, %2;\n\t fma.rn.f32 %3, m1, t3, %3;\n\t"                                     \
        "fma.rn.f32 %0, m2, u0, %0;\n\t fma.rn.f32 %1, m2, u1, %1;\n\t"                                     \
        "fma.rn.f32 %2, m3, u2, %2;\n\t fma.rn.f32 %3, m3, u3, %3;\n\t"                                     \
        "}\n"                                                                                               \
        : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])                                            \
        : "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]),           \
          "r"(aa0), "r"(aa1), "r"(xa0), "r"(xa1), "r"(lw), "r"(hasx)                                        \
        : "memory")

// compute_block: one block only (the ragged last stage of a row whose K is not a multiple of 128)
#define MPSBNB_BLOCK_ASM(TYPE)                                                                              \
    asm volatile(                                                                                           \
        "{\n\t"                                                                                             \
        ".reg .b32 ad, x<8>;\n\t"                                                                           \
        ".reg .b32 f<16>;\n\t"                                                                              \
        ".reg .f32 m<2>, t<4>, z;\n\t"                                                                      \
        ".reg .pred px;\n\t"                                                                                \
        "setp.ne.u32 px, %11, 0;\n\t"                                                                       \
        "mov.b32 x0, 0;\n\t mov.b32 x1, 0;\n\t mov.b32 x2, 0;\n\t mov.b32 x3, 0;\n\t"                       \
        "mov.b32 x4, 0;\n\t mov.b32 x5, 0;\n\t mov.b32 x6, 0;\n\t mov.b32 x7, 0;\n\t"                       \
        "@px ld.shared.v4.u32 {x0, x1, x2, x3}, [%9];\n\t"                                                  \
        "@px ld.shared.v4.u32 {x4, x5, x6, x7}, [%9+16];\n\t"                                               \
        "ld.shared.f32 m0, [%8];\n\t"                                                                       \
        "ld.shared.f32 m1, [%8+32];\n\t"                                                                    \
        "mov.f32 z, 0f00000000;\n\t"                                                                        \
        MPSBNB_LUT16("f", "%4", "%5", "%6", "%7", "%10")                                                    \
        MPSBNB_MMA(TYPE, "t", "f0", "f1", "f2", "f3", "x0", "x1", "{z,z,z,z}")                              \
        MPSBNB_MMA(TYPE, "t", "f4", "f5", "f6", "f7", "x2", "x3", "{t0,t1,t2,t3}")                          \
        MPSBNB_MMA(TYPE, "t", "f8", "f9", "f10", "f11", "x4", "x5", "{t0,t1,t2,t3}")                        \
        MPSBNB_MMA(TYPE, "t", "f12", "f13", "f14", "f15", "x6", "x7", "{t0,t1,t2,t3}")                      \
        "fma.rn.f32 %0, m0, t0, %0;\n\t fma.rn.f32 %1, m0, t1, %1;\n\t"                                     \
        "fma.rn.f32 %2, m1, t2, %2;\n\t fma.rn.f32 %3, m1, t3, %3;\n\t"                                     \
        "}\n"                                                                                               \
        : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])                                            \
        : "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(aa0), "r"(xa0), "r"(lw), "r"(hasx)                \
        : "memory")

template <typename XT> struct StageOps;
template <> struct StageOps<__half> {
    static __device__ __forceinline__ void stage(float (&acc)[4], const uint32_t (&w)[8], uint32_t aa0, uint32_t aa1,
                                                 uint32_t xa0, uint32_t xa1, uint32_t lw, uint32_t hasx) { MPSBNB_STAGE_ASM("f16"); }
    static __device__ __forceinline__ void block(float (&acc)[4], const uint32_t (&w)[8], uint32_t aa0, uint32_t xa0,
                                                 uint32_t lw, uint32_t hasx) { MPSBNB_BLOCK_ASM("f16"); }
};
template <> struct StageOps<__nv_bfloat16> {
    static __device__ __forceinline__ void stage(float (&acc)[4], const uint32_t (&w)[8], uint32_t aa0, uint32_t aa1,
                                                 uint32_t xa0, uint32_t xa1, uint32_t lw, uint32_t hasx) { MPSBNB_STAGE_ASM("bf16"); }
    static __device__ __forceinline__ void block(float (&acc)[4], const uint32_t (&w)[8], uint32_t aa0, uint32_t xa0,
                                                 uint32_t lw, uint32_t hasx) { MPSBNB_BLOCK_ASM("bf16"); }
};

// ---- batch <= 2: plain dot products instead of tensor-core MMAs.
// With one or two batch rows an MMA spends 7/8 of its columns on padding and, worse, its issue cost sits on
// the critical path of the warp that also has to issue the table loads.  Here a LANE owns a weight ROW: it
// reads the 32 packed bytes of its row for one block, looks every byte up (same byte-permute + table load)
// and multiplies the two codes with the two x values by mixed-precision FMAs (fp16 x fp16 + fp32 -> fp32,
// exact products, fp32 accumulation).  x is the same for all lanes, so its loads are broadcasts.
constexpr int SG_DOT_MAX_M = 2;                          // array bound of the dot path (it can do two batch rows)
constexpr int SG_DOT_RUN_M = 1;                          // ... and the batch up to which it runs: at batch 2 the MMA path
                                                         // measured 11 % faster (3317 against 3003 GB/s on the 70B-shaped stack)
__device__ __forceinline__ uint4 lds128v(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t lds_u32v(uint32_t addr) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory"); return v; }
__device__ __forceinline__ float lds_f32v(uint32_t addr) { float v; asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory"); return v; }
// the table never changes after the prologue: the compiler may schedule this load freely
__device__ __forceinline__ uint32_t lut_pair(uint32_t addr) { uint32_t v; asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr)); return v; }
// acc += lo(w) * lo(x) + hi(w) * hi(x), both products exact, accumulated in fp32
template <typename XT> __device__ __forceinline__ void fma_pair(float &acc, uint32_t w, uint32_t x);
template <> __device__ __forceinline__ void fma_pair<__half>(float &acc, uint32_t w, uint32_t x) {
    asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\tmov.b32 {wl, wh}, %1;\n\tmov.b32 {xl, xh}, %2;\n\t"
        "fma.rn.f32.f16 %0, wl, xl, %0;\n\tfma.rn.f32.f16 %0, wh, xh, %0;\n\t}\n" : "+f"(acc) : "r"(w), "r"(x));
}
template <> __device__ __forceinline__ void fma_pair<__nv_bfloat16>(float &acc, uint32_t w, uint32_t x) {
    asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\tmov.b32 {wl, wh}, %1;\n\tmov.b32 {xl, xh}, %2;\n\t"
        "fma.rn.f32.bf16 %0, wl, xl, %0;\n\tfma.rn.f32.bf16 %0, wh, xh, %0;\n\t}\n" : "+f"(acc) : "r"(w), "r"(x));
}
// one block (64 k) of this lane's row against NM batch rows; w[0..7] = the row's 32 packed bytes
template <typename XT, int NM>
__device__ __forceinline__ void dot_block(float (&tot)[SG_DOT_MAX_M], const uint32_t (&w)[8], float scale, uint32_t xa, uint32_t lw) {
    float p[NM][4];
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e) p[m][e] = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint4 xv[NM];
#pragma unroll
        for (int m = 0; m < NM; ++m) xv[m] = lds128v(xa + (uint32_t)(m * SG_XPITCH + 16 * i));   // k = 8 i .. 8 i + 7, same for all lanes
        const uint32_t c0 = lut_pair(__byte_perm(w[i], lw, 0x7604));
        const uint32_t c1 = lut_pair(__byte_perm(w[i], lw, 0x7614));
        const uint32_t c2 = lut_pair(__byte_perm(w[i], lw, 0x7624));
        const uint32_t c3 = lut_pair(__byte_perm(w[i], lw, 0x7634));
#pragma unroll
        for (int m = 0; m < NM; ++m) {
            fma_pair<XT>(p[m][0], c0, xv[m].x);
            fma_pair<XT>(p[m][1], c1, xv[m].y);
            fma_pair<XT>(p[m][2], c2, xv[m].z);
            fma_pair<XT>(p[m][3], c3, xv[m].w);
        }
    }
#pragma unroll
    for (int m = 0; m < NM; ++m) tot[m] = fmaf(scale, (p[m][0] + p[m][1]) + (p[m][2] + p[m][3]), tot[m]);
}
__device__ __forceinline__ void fetch_row_block(uint32_t (&w)[8], uint32_t a0, uint32_t a1) {
    asm volatile(
        "ld.shared.v4.u32 {%0, %1, %2, %3}, [%8];\n\t"
        "ld.shared.v4.u32 {%4, %5, %6, %7}, [%9];\n\t"
        : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
        : "r"(a0), "r"(a1)
        : "memory");
}

// Shared-memory map, in ABSOLUTE shared-window addresses.  The code-pair table sits at exactly
// 128 KiB so that "table + byte * 256 + lane * 4" is one byte-permute of (weight word, lane word):
// byte 0 = lane * 4, byte 1 = the weight byte, byte 2 = 0x02 — no addition.  Below it: partial
// sums, barriers, the scale/x ring and most weight slots; above it (from 192 KiB) two more slots.
constexpr uint32_t SG_LUT_ABS = 131072u;
constexpr uint32_t SG_HIGH_ABS = 196608u;
constexpr int SG_SMEM_BYTES = 227 * 1024;
constexpr int SG_MAX_XS = 8;
// Stage i is filled by loader warp i % SG_LOADERS into scale/x slot i % SG_MAX_XS.  An mbarrier parity
// wait only distinguishes "this phase" from "the one before", so every waiter has to see EVERY phase
// of a barrier: all fills of one slot must come from the same warp, one after the other.  With as many
// the slot count a multiple of the loader count, the slot determines the loader.  (Two warps filling the same slot in
// different rounds could pass the same parity test early and arrive twice in one phase.)
// The ring has 8 slots for batch <= 2 and 4 above; both are multiples of the number of loaders, so
// slot i % nxs is always filled by warp (i % nxs) % SG_LOADERS.
static_assert(SG_MAX_XS % SG_LOADERS == 0 && 4 % SG_LOADERS == 0, "each scale/x slot must belong to exactly one loader warp");

struct SlotMap {
    uint32_t low0, high0;
    int nlow, nslots;
    __device__ __forceinline__ uint32_t addr(int slot) const {
        return slot < nlow ? low0 + (uint32_t)slot * SG_W_BYTES : high0 + (uint32_t)(slot - nlow) * SG_W_BYTES;
    }
};

template <typename XT>
__global__ void __launch_bounds__(SG_THREADS, 1) mpsbnb_decode4_stream_kernel(const __grid_constant__ StreamArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t s_base = smem_u32(smem);
    const uint32_t s_red = s_base;                                   // 2 x SG_RED_BYTES
    // full[8] empty[8] red_full[2] red_empty[2] xfull[8] xempty[8] (288 B), abort flag, 32 zero bytes at +320
    const uint32_t s_bar = s_base + 2 * SG_RED_BYTES;
    const uint32_t s_zero = s_bar + 320u;

    const int nxs = a.M <= 2 ? SG_MAX_XS : 4;                        // scale/x slots (released after the MMAs)
    const uint32_t xs_bytes = (uint32_t)(SG_A_BYTES + ((a.M * SG_XPITCH + 127) / 128) * 128);
    // mailbox reducer -> closer: full[4] empty[4] barriers at +352, the tile indices at +416
    auto mail_full = [&](int i) { return s_bar + 352u + 8u * i; };
    auto mail_empty = [&](int i) { return s_bar + 352u + 8u * (SG_MAIL + i); };
    const uint32_t s_mail = s_bar + 416u;
    const uint32_t s_xs = (s_bar + 512u + 127u) & ~127u;
    // tagged x, batch 1: a staging buffer per loader warp for one stage's entries (1024 columns = 512 entries of 8 bytes), filled by bulk copies
    const uint32_t s_stage = s_xs + (uint32_t)nxs * xs_bytes;
    const uint32_t stage_bytes = (a.x_ll && a.M == 1) ? (uint32_t)SG_LOADERS * 4096u : 0u;
    auto sfull_bar = [&](int i) { return s_bar + 448u + 8u * i; };
    SlotMap sm;
    sm.low0 = (s_stage + stage_bytes + 1023u) & ~1023u;
    sm.high0 = SG_HIGH_ABS;
    sm.nlow = (int)((SG_LUT_ABS - sm.low0) / SG_W_BYTES);
    {
        const int nhigh = (int)((s_base + (uint32_t)SG_SMEM_BYTES - SG_HIGH_ABS) / SG_W_BYTES);
        const int n = sm.nlow + nhigh;
        sm.nslots = n > SG_MAX_SLOTS ? SG_MAX_SLOTS : n;
        sm.nslots -= sm.nslots % SG_GROUPS;                          // every slot belongs to one consumer group
        if (sm.nlow > sm.nslots) sm.nlow = sm.nslots;
    }
    const int nslots = sm.nslots;
    unsigned char *p_generic0 = smem - s_base;                       // generic pointer of shared address 0
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(p_generic0 + s_bar + 8 * (2 * SG_MAX_SLOTS + 4 + 2 * SG_MAX_XS));
    auto full_bar = [&](int s) { return s_bar + 8u * s; };
    auto empty_bar = [&](int s) { return s_bar + 8u * (SG_MAX_SLOTS + s); };
    auto red_full = [&](int b) { return s_bar + 8u * (2 * SG_MAX_SLOTS + b); };
    auto red_empty = [&](int b) { return s_bar + 8u * (2 * SG_MAX_SLOTS + 2 + b); };
    auto xfull_bar = [&](int s) { return s_bar + 8u * (2 * SG_MAX_SLOTS + 4 + s); };
    auto xempty_bar = [&](int s) { return s_bar + 8u * (2 * SG_MAX_SLOTS + 4 + SG_MAX_XS + s); };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#ifdef MPSBNB_TRACE
    const long long trace_t0 = clock64();
#endif
    pdl_launch_dependents();

    if (tid == 0) {
        for (int s = 0; s < nslots; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), SG_GROUP_WARPS); }
        for (int b = 0; b < 2; ++b) { mbar_init(red_full(b), SG_CONSUMERS); mbar_init(red_empty(b), 1); }
        for (int i = 0; i < SG_MAIL; ++i) { mbar_init(mail_full(i), 1); mbar_init(mail_empty(i), 1); }
        for (int i = 0; i < SG_LOADERS; ++i) mbar_init(sfull_bar(i), 1);
        for (int s = 0; s < nxs; ++s) { mbar_init(xfull_bar(s), 1); mbar_init(xempty_bar(s), SG_GROUP_WARPS); }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp < 8) {
        // byte -> (code[low nibble], code[high nibble]) pairs, one replica per lane: entry b of lane l
        // at table + b * 256 + l * 4.  Warp w fills bytes 32 w .. 32 w + 31.
        const float my_code = kCode[a.quant_type][lane & 15];
        const int byte = warp * 32 + lane;
        const float lo = __shfl_sync(0xffffffffu, my_code, byte & 15);
        const float hi = __shfl_sync(0xffffffffu, my_code, byte >> 4);
        const uint32_t mine = pair_bits<XT>(lo, hi);
#pragma unroll 8
        for (int j = 0; j < 32; ++j)
            sts32(SG_LUT_ABS + (uint32_t)((warp * 32 + j) * 256 + lane * 4), __shfl_sync(0xffffffffu, mine, j));
    } else {
        // the scale/x ring starts as zeros (x columns beyond K are never written, and 0 * stale bits must
        // be 0), and so does the zero area that lanes without a batch row read their x from
        const int total = nxs * (int)xs_bytes;
        for (int o = (tid - 256) * 16; o < total; o += (SG_THREADS - 256) * 16) sts128(s_xs + o, make_uint4(0u, 0u, 0u, 0u));
        if (tid == 256) { sts128(s_zero, make_uint4(0u, 0u, 0u, 0u)); sts128(s_zero + 16, make_uint4(0u, 0u, 0u, 0u)); }
    }
    fence_proxy_async_smem();
    __syncthreads();

    auto unit_of = [&](int u) -> StreamUnit {
        if (a.units != nullptr) return a.units[u];
        StreamUnit un;
        un.lin = 0; un.row0 = u * SG_ROWS; un.s_begin = 0; un.s_end = (a.one.nb + SG_STAGE_BLOCKS - 1) / SG_STAGE_BLOCKS;
        un.nbv = a.one.nbv; un.pad0 = un.pad1 = un.pad2 = 0;
        return un;
    };
    auto lin_of = [&](int i) -> const StreamLinear * { return a.lins != nullptr ? a.lins + i : &a.one; };

    if (warp == SG_CONSUMERS) {
        // ------------------------------------------------------------ TMA producer: packed weights
        if (lane == 0) {
            // The only serial thread on the data path: per stage one barrier wait, one expect-tx and one
            // (3-D) tensor copy.  Weights never depend on the previous kernel in the stream, so this thread
            // does not wait for it; the loaders, which bring x, do.
            int u = blockIdx.x;
            int slot = 0; uint32_t ph = 0;
            while (u < a.nunits && !*abort_flag) {
                const StreamUnit un = unit_of(u);
                const StreamLinear *L = lin_of(un.lin);
                const CUtensorMap *map = &L->map;
                const bool m3 = L->map3d != 0;
                bool ok = true;
                for (int s = un.s_begin; s < un.s_end; ++s) {
                    if (!SG_TIMED(0, mbar_wait_sleep(empty_bar(slot), ph ^ 1u, abort_flag, a.sleep_other))) { sg_fail(201); *abort_flag = 1; ok = false; break; }
                    const uint32_t bar = full_bar(slot), dst = sm.addr(slot);
                    mbar_arrive_expect_tx(bar, SG_W_BYTES);
                    if (m3) {
                        tma_load_3d(dst, map, bar, 0, un.row0, s * 4);
                    } else {
#pragma unroll
                        for (int p = 0; p < 4; ++p) tma_load_2d(dst + p * 4096, map, bar, (s * 4 + p) * 128, un.row0);
                    }
                    if (++slot == nslots) { slot = 0; ph ^= 1u; }
                }
                if (!ok) break;
                u += gridDim.x;
            }
        }
    } else if (warp == SG_CONSUMERS + 1 + SG_LOADERS) {
        // ------------------------------------------------------------ reducer: sums the 8 kg partials of a unit
        // lane = tile row.  MMA row i of row tile rt is tile row 16 rt + rho(i & 7) + 8 (i >> 3).
        const int rr = lane & 15, v = rr & 7;
        const int i = ((v >> 1) + 4 * (v & 1)) + 8 * (rr >> 3);
        const int wrt = lane >> 4;
        pdl_grid_dependency_wait();                              // outputs may still be read by the previous kernel
        int uc = 0;
        // every unit that added into the accumulator is handed to the closer warp (mailbox: segment << 16 | tile), which
        // counts it, and, when it was the tile's last contribution, converts the tile, stores it into every rank's h
        // and re-arms the accumulator - the round trip of the count never holds this warp up
        int mail_i = 0; uint32_t mail_ph = 0;
        auto post = [&](int tile) {
            if (!mbar_wait_sleep(mail_empty(mail_i), mail_ph ^ 1u, abort_flag, a.sleep_other)) { sg_fail(208); *abort_flag = 1; return; }
            if (lane == 0) { sts32(s_mail + 4u * mail_i, (uint32_t)tile); mbar_arrive(mail_full(mail_i)); }
            __syncwarp();
            if (++mail_i == SG_MAIL) { mail_i = 0; mail_ph ^= 1u; }
        };
        for (int u = blockIdx.x; u < a.nunits && !*abort_flag; u += gridDim.x, ++uc) {
            const StreamUnit un = unit_of(u);
            const StreamLinear *L = lin_of(un.lin);
            // what this unit needs of its linear is fetched before the wait, so that the two dependent global loads
            // (unit, then linear) pass while the consumers are still working on the unit
            const int LN = L->N, Ldt = L->y_dtype, Lseg = L->segment;
            const void *Lbias = L->bias;
            float *Lacc = L->acc;
            void *Ly = L->y;
            const int buf = uc & 1;
            if (!SG_TIMED(1, mbar_wait_sleep(red_full(buf), (uint32_t)(uc >> 1) & 1u, abort_flag, a.sleep_other))) { sg_fail(204); *abort_flag = 1; break; }
            const float *red = reinterpret_cast<const float *>(p_generic0 + s_red + buf * SG_RED_BYTES);
            const int n = un.row0 + lane;
            for (int m = 0; m < a.M; ++m) {
                float sum = 0.0f;
                if (a.M <= SG_DOT_RUN_M) {
                    // dot-product path: [warp][m][row] partial sums of all 16 warps
#pragma unroll
                    for (int w16 = 0; w16 < SG_CONSUMERS; ++w16) sum += red[(w16 * SG_DOT_MAX_M + m) * 32 + lane];
                } else {
#pragma unroll
                    for (int k8 = 0; k8 < 8; ++k8) sum += red[((k8 * 2 + wrt) * 8 + m) * 20 + i];
                }
                if (n < LN) {
                    if (Lbias != nullptr && un.s_begin == 0) sum += to_f32<XT>(reinterpret_cast<const XT *>(Lbias)[n]);
                    const int64_t o = (int64_t)m * LN + n;
                    if (Lacc != nullptr) atomicAdd(Lacc + o, sum);
                    else if (Ldt == MPSBNB_F16) reinterpret_cast<__half *>(Ly)[o] = __float2half_rn(sum);
                    else if (Ldt == MPSBNB_BF16) reinterpret_cast<__nv_bfloat16 *>(Ly)[o] = __float2bfloat16_rn(sum);
                    else reinterpret_cast<float *>(Ly)[o] = sum;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(red_empty(buf));
            if (a.ep.tile_cnt != nullptr && Lacc != nullptr &&
                (Lacc == a.ep.acc || (a.ep.count_tiles == 2 && Lacc == a.ep.acc + (int64_t)a.M * a.ep.hs))) {   // (tagged: two copies)
                // streamed closing step: the closer warp counts this unit's contribution to its 32-row tile.  The mailbox
                // barrier (release / acquire inside the CTA) orders this warp's accumulator updates before the closer's
                // count, which is a release and an acquire at GPU scope.
                __syncwarp();
                post((Lseg << 16) | (un.row0 / SG_ROWS));
            }
        }
        if (a.ep.tile_cnt != nullptr && !*abort_flag) post(-1);    // tells the closer warp that nothing more will come
        __threadfence();                                         // my results before this CTA's arrival at the closing step
    } else if (warp == SG_CONSUMERS + 2 + SG_LOADERS) {
        // ------------------------------------------------------------ closer (streamed closing step only)
        if (a.ep.tile_cnt != nullptr) {
            XT *const *all_peers = reinterpret_cast<XT *const *>(a.ep.peer_h);
            const int nbuf = a.ep.nbuf > 1 ? a.ep.nbuf : 1;
            int mi = 0; uint32_t mph = 0;
            while (!*abort_flag) {
                if (!SG_TIMED(11, mbar_wait_sleep(mail_full(mi), mph, abort_flag, a.sleep_other))) { sg_fail(209); *abort_flag = 1; break; }
#ifdef MPSBNB_TRACE
                const long long tclose0 = clock64();
#endif
                const int word = (int)lds_u32v(s_mail + 4u * mi);
                __syncwarp();
                if (lane == 0) mbar_arrive(mail_empty(mi));
                if (++mi == SG_MAIL) { mi = 0; mph ^= 1u; }
                if (word < 0) break;
                const int seg = word >> 16, tile = word & 0xFFFF;
                {
                    int old = 0;
                    // counts 0 .. expect - 1 and wraps to 0 by itself: the count needs no re-arming store
                    // Tagged exchange: a unit of the next segment runs as soon as ITS columns of x carry the tag, possibly before
                    // this tile of this segment is closed - counts and accumulators exist twice, by segment parity (a tile
                    // of segment s + 1 cannot close before every tile of segment s has: two copies are enough).
                    const int par_cnt = a.ep.count_tiles == 2 ? (seg & 1) * ((a.ep.hs + SG_ROWS - 1) / SG_ROWS) : 0;
                    if (lane == 0)
                        asm volatile("atom.inc.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(a.ep.tile_cnt + par_cnt + tile), "r"(a.ep.tile_expect - 1) : "memory");
                    old = __shfl_sync(0xffffffffu, old, 0);
                    if (old != a.ep.tile_expect - 1) continue;       // not the tile's last contribution
                }
                if (a.ep.count_tiles == 2) {
                    // Tagged exchange: column pair (2 p, 2 p + 1) of h travels as ONE 8-byte store {two 16-bit values, tag}
                    // with tag = step * L + layer of the consumer, into every rank's buffer.  An aligned 8-byte store
                    // arrives whole, so a reader that sees the tag has the data: no fence, no count, no flag, and the
                    // accumulator is read and re-armed by one atomic exchange per element.
                    unsigned long long *const *peers_ll = reinterpret_cast<unsigned long long *const *>(a.ep.peer_h) +
                                                          (nbuf > 1 ? ((seg + 1) % nbuf) * a.ep.nranks : 0);
                    const uint32_t tag = (uint32_t)((*a.ep.step) * a.ep.mul + a.ep.add + seg);
                    const int c = tile * SG_ROWS + lane;
                    for (int m = 0; m < a.M; ++m) {
                        float v = 0.0f;
                        if (c < a.ep.hs) v = atomicExch(a.ep.acc + ((int64_t)(seg & 1) * a.M + m) * a.ep.hs + c, 0.0f);
                        const float vn = __shfl_down_sync(0xffffffffu, v, 1);
                        if ((lane & 1) == 0 && c < a.ep.hs) {
                            const unsigned long long w = ((unsigned long long)tag << 32) | pair_bits<XT>(a.ep.alpha * v, a.ep.alpha * vn);
                            const int64_t o = ((int64_t)m * a.ep.H + (int64_t)a.ep.rank * a.ep.hs + c) >> 1;
                            for (int r = 0; r < a.ep.nranks; ++r)
                                asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(peers_ll[r] + o), "l"(w) : "memory");
                        }
                    }
                    MPSBNB_TRACE_SET(2, seg + 1);
                    continue;
                }
                XT *const *peers = all_peers + (nbuf > 1 ? ((seg + 1) % nbuf) * a.ep.nranks : 0);
                const int n = tile * SG_ROWS + lane;
                if (n < a.ep.hs) {
                    for (int m = 0; m < a.M; ++m) {
                        float *pa = a.ep.acc + (int64_t)m * a.ep.hs + n;
                        const XT hv = from_f32<XT>(a.ep.alpha * __ldcg(pa));
                        *pa = 0.0f;
                        const int64_t o = (int64_t)m * a.ep.H + (int64_t)a.ep.rank * a.ep.hs + n;
                        for (int r = 0; r < a.ep.nranks; ++r) peers[r][o] = hv;
                    }
                }
                if (a.ep.count_tiles) {
                    // every closed tile adds 1 to this rank's count on every rank.  The addition is a release at system
                    // scope (the warp barrier makes it cover all lanes' stores) and needs no answer: no counter of this
                    // GPU, no second fence, no separate flag store on the path to the waiting ranks.
                    __syncwarp();
                    if (lane < a.ep.nranks)
                        asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(a.ep.peer_flags[lane] + a.ep.rank) : "memory");
                    MPSBNB_TRACE_SET(2, seg + 1);
                } else {
                (void)SG_TIMED(14, ((a.ep.nranks > 1 ? __threadfence_system() : __threadfence()), true));   // the stores before the count
                __syncwarp();
                int done = 0;
                if (lane == 0) done = atomicAdd(a.ep.counter, 1);
                done = __shfl_sync(0xffffffffu, done, 0);
                if (done == (a.ep.hs + SG_ROWS - 1) / SG_ROWS - 1) {
                    // every tile of this rank's shard has been stored (each store was fenced before its count)
                    if (a.ep.nranks > 1) __threadfence_system(); else __threadfence();
                    if (lane == 0) *a.ep.counter = 0;
                    if (lane == 0) MPSBNB_TRACE_SET(2, seg + 1);
                    if (a.ep.peer_flags != nullptr && lane < a.ep.nranks)
                        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.ep.peer_flags[lane] + a.ep.rank), "r"((*a.ep.step) * a.ep.mul + a.ep.add + seg) : "memory");
                }
                }
#ifdef MPSBNB_TRACE
                if (blockIdx.x == 0 && lane == 0) { atomicAdd(&g_wait[10], (unsigned long long)(clock64() - tclose0)); atomicAdd(&g_wait[12], 1ull); }
#endif
            }
        }
    } else if (warp > SG_CONSUMERS) {
        // ------------------------------------------------------------ loaders: block scales and x into the scale/x ring
        // SG_LOADERS warps take stages in turn; each reads the scales of its NEXT stage before it stores
        // the current one, so two rounds of global loads are in flight per warp.
        const int me = warp - SG_CONSUMERS - 1;
        pdl_grid_dependency_wait();                              // x is written by the previous kernel in the stream
        {
            auto read_scales = [&](const StreamLinear *L, int row0, int s, float (&sc)[16]) {
                const int n = row0 + lane;
                const int b0 = s * SG_STAGE_BLOCKS;
                const int64_t i0 = (int64_t)n * L->nb + b0;
                if (n >= L->N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) sc[j] = 0.0f;
                } else if (L->absmax2 == nullptr) {
                    const float *am = reinterpret_cast<const float *>(L->absmax);
                    if (b0 + 16 <= L->nb && (i0 & 3) == 0) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float4 v = __ldg(reinterpret_cast<const float4 *>(am + i0) + q);
                            sc[4 * q] = v.x; sc[4 * q + 1] = v.y; sc[4 * q + 2] = v.z; sc[4 * q + 3] = v.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) sc[j] = (b0 + j < L->nb) ? __ldg(am + i0 + j) : 0.0f;
                    }
                } else {
                    // int8 code * (second-level maximum / 127); 16 consecutive blocks see at most two maxima
                    const int8_t *aq = reinterpret_cast<const int8_t *>(L->absmax);
                    const int last = (b0 + 15 < L->nb ? b0 + 15 : L->nb - 1) - b0;
                    const float f0 = __fdiv_rn(__ldg(L->absmax2 + (i0 >> 8)), 127.0f);       // divide first, as functional.py:592-593
                    const float f1 = __fdiv_rn(__ldg(L->absmax2 + ((i0 + last) >> 8)), 127.0f);
                    const int split = (int)(((i0 >> 8) + 1) * 256 - i0);          // first j that uses f1
                    uint32_t raw[4];
                    if (b0 + 16 <= L->nb && (i0 & 3) == 0) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) raw[q] = __ldg(reinterpret_cast<const uint32_t *>(aq + i0) + q);
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            raw[q] = 0u;
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (b0 + 4 * q + e < L->nb) raw[q] |= (uint32_t)(uint8_t)__ldg(aq + i0 + 4 * q + e) << (8 * e);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int code = (int)(int8_t)((raw[j >> 2] >> (8 * (j & 3))) & 0xFFu);
                        sc[j] = (b0 + j < L->nb) ? (float)code * (j < split ? f0 : f1) : 0.0f;
                    }
                }
            };
            int u = blockIdx.x;
            StreamUnit un = {0, 0, 0, 0, 0, 0, 0, 0};
            const StreamLinear *L = nullptr;
            int s = 0, turn = 0, xslot = 0;  // turn: global stage index modulo SG_LOADERS
            uint32_t xph = 0;
            bool have = false;
            auto step = [&]() {                  // to the next stage of the global sequence
                ++s;
                if (++turn == SG_LOADERS) turn = 0;
                if (++xslot == nxs) { xslot = 0; xph ^= 1u; }
            };
            auto advance_to_mine = [&]() {       // positions the cursor on my next stage; returns false at the end
                for (;;) {
                    if (!have) {
                        if (u >= a.nunits) return false;
                        un = unit_of(u); L = lin_of(un.lin); s = un.s_begin; have = true;
                    }
                    if (s >= un.s_end) { have = false; u += gridDim.x; continue; }
                    if (turn == me) return true;
                    step();
                }
            };
            float cur[16];
            int ready_seg = -1;                  // segments whose input is known to be complete
            // tagged x: whether the stage under the cursor was requested into this warp's staging buffer (a bulk copy needs a
            // 16-byte aligned source and size - four columns per 16 bytes - in one run, and there is one buffer: batch 1)
            bool req = false;
            uint32_t sph = 0;                    // the phase the staging buffer completes next
            auto request_x = [&]() {
                req = false;
                if (stage_bytes == 0u) return;
                int xc = L->K - s * (SG_STAGE_BLOCKS * 64);
                xc = xc > SG_STAGE_BLOCKS * 64 ? SG_STAGE_BLOCKS * 64 : xc;
                const int col0 = (s * (SG_STAGE_BLOCKS * 64)) % L->x_period;
                if (xc <= 0 || (xc & 3) != 0 || (col0 & 3) != 0 || col0 + xc > L->x_period || (reinterpret_cast<uintptr_t>(L->x) & 15) != 0) return;
                req = true;
                if (lane == 0) {
                    mbar_arrive_expect_tx(sfull_bar(me), (uint32_t)(xc >> 1) * 8u);
                    bulk_load_1d(s_stage + (uint32_t)me * 4096u, reinterpret_cast<const unsigned long long *>(L->x) + (col0 >> 1), (uint32_t)(xc >> 1) * 8u, sfull_bar(me));
                }
            };
            bool more = advance_to_mine();
            if (more) { read_scales(L, un.row0, s, cur); if (a.x_ll) request_x(); }
            while (more && !*abort_flag) {
                const int my_x = xslot, my_s = s;
                const uint32_t my_ph = xph;
                const StreamLinear *my_L = L;
                const bool my_req = req;
                step();
                float nxt[16];
                more = advance_to_mine();
                if (more) read_scales(L, un.row0, s, nxt);
                if (!SG_TIMED(2, mbar_wait_sleep(xempty_bar(my_x), my_ph ^ 1u, abort_flag, a.sleep_other))) { sg_fail(202); *abort_flag = 1; break; }
                const uint32_t xb = s_xs + (uint32_t)my_x * xs_bytes;
                if (a.wait_n > 0 && my_L->segment > ready_seg) {
                    // x of this segment is written by closing steps: of the previous launch or segment, on this GPU and,
                    // in the N-sharded stack, on the others.  Wait (bounded) for their flags.
                    const int expect = (*a.wait_step) * a.wait_mul + a.wait_add + my_L->segment * a.wait_seg_mul;
                    bool arrived = true;
                    if (blockIdx.x == 0 && me == 0 && lane == 0) MPSBNB_TRACE_SET(0, my_L->segment);
                    if (lane < a.wait_n) {
                        const long long t0 = clock64();
                        for (;;) {
                            int v;
                            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(a.wait_flags + lane) : "memory");
                            if (v >= expect) break;
                            __nanosleep(64);
                            if (*abort_flag != 0 || clock64() - t0 > 2000000000ll) { arrived = false; break; }
                        }
                    }
                    arrived = __all_sync(0xffffffffu, arrived);
                    asm volatile("fence.proxy.async;" ::: "memory");      // x is then read by bulk copies (async proxy)
                    if (!arrived) { sg_fail(207); *abort_flag = 1; break; }
                    if (blockIdx.x == 0 && me == 0 && lane == 0) MPSBNB_TRACE_SET(1, my_L->segment);
                    ready_seg = my_L->segment;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) sts_f32(xb + (j * 32 + lane) * 4, cur[j]);
                int xcols = my_L->K - my_s * (SG_STAGE_BLOCKS * 64);
                xcols = xcols > SG_STAGE_BLOCKS * 64 ? SG_STAGE_BLOCKS * 64 : (xcols < 0 ? 0 : xcols);
                if (a.x_ll) {
                    // x in tagged form, written by closer warps here or on other GPUs: 8-byte entries {two values, tag}.  Seeing the
                    // expected tag IS having the data (an aligned 8-byte store arrives whole): no flag, fence or acquire is
                    // involved, an entry that does not carry the tag yet is read again (bounded).
                    const uint32_t expect = (uint32_t)((*a.wait_step) * a.wait_mul + a.wait_add + my_L->segment * a.wait_seg_mul);
                    const int k_base = my_s * (SG_STAGE_BLOCKS * 64);
                    const unsigned long long *x2 = reinterpret_cast<const unsigned long long *>(my_L->x);
                    bool ok = true;
                    if (my_req) {
                        // this stage's entries were requested into the warp's staging buffer when the previous one had been
                        // examined (a loader's stages lie SG_LOADERS apart: the round trip to L2 is long over)
                        const uint32_t sb = s_stage + (uint32_t)me * 4096u;
                        const int npairs = xcols >> 1;
                        const unsigned long long *src = x2 + (((my_s * (SG_STAGE_BLOCKS * 64)) % my_L->x_period) >> 1);
                        if (!SG_TIMED(13, mbar_wait_sleep(sfull_bar(me), sph, abort_flag, a.sleep_other))) { sg_fail(210); ok = false; }
                        sph ^= 1u;
                        long long t0 = 0;
                        // First pass: the staged copy.  If an entry there is late, the following passes read the entries where
                        // they lie with system-scope loads - NOT another bulk copy: a bulk copy is a weak read, and one that races
                        // with another GPU's store was seen to keep returning the old entry for good.
                        for (bool staged = true; ok; staged = false) {
                            bool good = true;
                            uint32_t bad_tag = 0u; int bad_c = -1;               // (trace builds report the first entry that is late)
                            // 16-byte chunks (two entries) c = lane + 32 j; four loads are issued before the first value is looked at
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                uint32_t r[4][4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const int c = lane + 32 * (4 * h + j);
                                    if (2 * c >= npairs) { r[j][1] = expect; r[j][3] = expect; r[j][0] = 0u; r[j][2] = 0u; }
                                    else if (staged)
                                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r[j][0]), "=r"(r[j][1]), "=r"(r[j][2]), "=r"(r[j][3]) : "r"(sb + (uint32_t)c * 16u));
                                    else {
                                        asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(r[j][0]), "=r"(r[j][1]) : "l"(src + 2 * c) : "memory");
                                        asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(r[j][2]), "=r"(r[j][3]) : "l"(src + 2 * c + 1) : "memory");
                                    }
                                }
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const int c = lane + 32 * (4 * h + j);
                                    good = good && r[j][1] == expect && r[j][3] == expect;
                                    if (bad_c < 0 && (r[j][1] != expect || r[j][3] != expect)) { bad_c = c; bad_tag = r[j][1] != expect ? r[j][1] : r[j][3]; }
                                    if (2 * c < npairs)                           // K is a multiple of 4 here: no column beyond it
                                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" :: "r"(xb + (uint32_t)SG_A_BYTES + (uint32_t)c * 8u), "r"(r[j][0]), "r"(r[j][2]) : "memory");
                                }
                            }
                            if (__all_sync(0xffffffffu, good)) break;
                            if (t0 == 0) t0 = clock64();
                            if (*abort_flag != 0 || clock64() - t0 > 2000000000ll) {
                                if (*abort_flag == 0 && bad_c >= 0) SG_FAIL_DETAIL(expect, bad_tag, (uint32_t)((my_L->segment << 16) | my_s), (uint32_t)bad_c, (uint32_t)*a.wait_step);
                                sg_fail(207); ok = false;
                            }
                        }
                    } else {
                        // a batch above 1, a stage that straddles the period, an odd offset: the entries are read where they lie
                        const int npairs = (xcols + 1) >> 1;
                        for (int m = 0; m < a.M; ++m)
                            for (int i = lane; i < npairs; i += 32) {
                                const unsigned long long *p = x2 + (int64_t)m * (my_L->x_ld >> 1) + (((k_base + 2 * i) % my_L->x_period) >> 1);
                                unsigned long long v;
                                const long long t0 = clock64();
                                for (;;) {
                                    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
                                    if ((uint32_t)(v >> 32) == expect) break;
                                    if (*abort_flag != 0 || clock64() - t0 > 2000000000ll) { ok = false; break; }
                                }
                                uint32_t d = (uint32_t)v;
                                if (2 * i + 1 >= xcols) d &= 0xFFFFu;             // odd K: the column beyond it stays zero
                                sts32(xb + SG_A_BYTES + m * SG_XPITCH + i * 4, d);
                            }
                        if (!__all_sync(0xffffffffu, ok)) sg_fail(207);
                    }
                    if (!__all_sync(0xffffffffu, ok)) { *abort_flag = 1; break; }
                    __syncwarp();                                                // the staging buffer is free again
                    if (more) request_x();                                       // the next stage of this warp
                    if (lane == 0) mbar_arrive(xfull_bar(my_x));
                } else if (my_L->x_bulk_ok) {
                    // x: one bulk copy per batch row, tracked by the slot's barrier (columns beyond K keep their zeros)
                    __syncwarp();
                    if (lane == 0) {
                        const uint32_t nb2 = (uint32_t)xcols * 2u;
                        mbar_arrive_expect_tx(xfull_bar(my_x), nb2 * (uint32_t)a.M);
                        const int col = (my_s * (SG_STAGE_BLOCKS * 64)) % my_L->x_period;
                        const unsigned char *src = reinterpret_cast<const unsigned char *>(my_L->x) + (int64_t)col * 2;
                        if (nb2 != 0u)
                            for (int m = 0; m < a.M; ++m)
                                bulk_load_1d(xb + SG_A_BYTES + m * SG_XPITCH, src + (int64_t)m * my_L->x_ld * 2, nb2, xfull_bar(my_x));
                    }
                } else {
                    // x: 1024 columns of every batch row by plain loads, zero beyond K
                    const XT *x = reinterpret_cast<const XT *>(my_L->x);
                    const int k_base = my_s * (SG_STAGE_BLOCKS * 64);
                    for (int m = 0; m < a.M; ++m) {
                        const XT *xr = x + (int64_t)m * my_L->x_ld;
#pragma unroll
                        for (int c4 = 0; c4 < 4; ++c4) {
                            const int k0 = k_base + (lane + 32 * c4) * 8;
                            uint16_t e[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                e[j] = (k0 + j < my_L->K) ? __ldcg(reinterpret_cast<const unsigned short *>(xr + (k0 + j) % my_L->x_period))
                                                          : (unsigned short)0;    // L2 only: x may have been written during this launch
                            sts128(xb + SG_A_BYTES + m * SG_XPITCH + (lane + 32 * c4) * 16,
                                   make_uint4(e[0] | ((uint32_t)e[1] << 16), e[2] | ((uint32_t)e[3] << 16),
                                              e[4] | ((uint32_t)e[5] << 16), e[6] | ((uint32_t)e[7] << 16)));
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(xfull_bar(my_x));
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) cur[j] = nxt[j];
            }
        }
    } else {
        // ------------------------------------------------------------ consumers
        // The 16 warps form SG_GROUPS independent groups; group q takes every SG_GROUPS-th stage of the
        // CTA's stage sequence, so the groups drift apart in time and one group's barrier waits are covered
        // by the table loads and MMAs of the others.  Inside a group of W = 16 / SG_GROUPS warps, warp j owns
        // row tile j & 1 and the block pairs kg = (j >> 1) + (W / 2) i, i = 0 .. SG_ITEMS - 1, of each stage:
        // while item i runs from one register set, the packed bytes of item i + 1 are on their way into the
        // other.  The weight slot is handed back when the last item's bytes are in registers, the scale/x
        // slot after the last MMA.
        const int g = lane >> 2, t = lane & 3;
        const int grp = warp / SG_GROUP_WARPS, j = warp % SG_GROUP_WARPS;
        const int rt = j & 1, kg0 = j >> 1;
        const int rho = ((2 * g) & 7) + (g >> 2);                // tile row of MMA row g (conflict-free permutation)
        const uint32_t lane_word = SG_LUT_ABS | ((uint32_t)lane * 4u);   // bytes 0, 2, 3 of every table address
        // offsets of item 0; item i adds SG_ITEM_W / SG_ITEM_X bytes
        uint32_t woff[2], xoff[2], aoff[2];
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const int blk = 2 * kg0 + b;
            const int box = blk >> 2, c = 2 * (blk & 3) + (t >> 1);
            const int r0 = 16 * rt + rho;
            woff[b] = (uint32_t)(box * 4096 + r0 * 128 + ((c ^ rho) << 4) + 8 * (t & 1));
            xoff[b] = (uint32_t)(SG_A_BYTES + g * SG_XPITCH + (blk * 64 + 16 * t) * 2);
            aoff[b] = (uint32_t)((blk * 32 + r0) * 4);
        }
        constexpr int KG_STEP = SG_GROUP_WARPS / 2;                  // block pairs between two items of a warp
        constexpr uint32_t ITEM_W = (uint32_t)(KG_STEP * 2 * 1024);   // 2 blocks = half a 4 KiB box
        constexpr uint32_t ITEM_X = (uint32_t)(KG_STEP * 2 * 64 * 2); // x bytes per block pair step
        constexpr uint32_t ITEM_A = (uint32_t)(KG_STEP * 2 * 32 * 4); // scale bytes per block pair step
        const bool dot = a.M <= SG_DOT_RUN_M;                     // lane = row, one block per item (see dot_block)
        if (dot) {
            woff[0] = (uint32_t)(lane * 128 + (((2 * j) ^ (lane & 7)) << 4));
            woff[1] = (uint32_t)(lane * 128 + (((2 * j + 1) ^ (lane & 7)) << 4));
            xoff[0] = (uint32_t)(SG_A_BYTES + j * 128);
            aoff[0] = (uint32_t)((j * 32 + lane) * 4);
        }
        static_assert(SG_GROUP_WARPS == 4 && SG_ITEMS == 4, "the dot path deals the 16 blocks of a stage to 4 warps, box by box");
        const uint32_t hasx = g < a.M ? 1u : 0u;
        uint32_t wA[8], wB[8];

        // The walk over this warp's stages, shared by the compute variants below.  stage_fn(s, nbv, sb, xb, ebar)
        // does one stage (and arrives on ebar, the weight slot's "empty" barrier, once its bytes are in
        // registers); it returns a word that depends on its last result.  flush_fn(rb) stores the unit's partial
        // sums into the reducer's buffer and clears them.  Only ONE variant runs in a launch, so only its code
        // is resident in the instruction caches.
        auto run_units = [&](auto &&stage_fn, auto &&flush_fn) {
            int slot = grp % nslots, xslot = grp % nxs;              // ring positions of my next stage
            uint32_t ph = (uint32_t)(grp / nslots) & 1u, xph = (uint32_t)(grp / nxs) & 1u;
            int nextq = grp;                                          // my next stage in the CTA's stage sequence
            int qb = 0, uc = 0;
            bool ok = true;
            StreamUnit un = {0, 0, 0, 0, 0, 0, 0, 0};
            int u = (int)blockIdx.x;
            if (u < a.nunits) un = unit_of(u);
            while (u < a.nunits && ok && !*abort_flag) {
                const int un_next = u + (int)gridDim.x;
                StreamUnit nx = {0, 0, 0, 0, 0, 0, 0, 0};
                if (un_next < a.nunits) nx = unit_of(un_next);        // in flight while this unit's stages run
                const int nbv = un.nbv;
                const int qe = qb + (un.s_end - un.s_begin);
#pragma unroll 1
                for (; nextq < qe; nextq += SG_GROUPS) {
                    const int s = un.s_begin + (nextq - qb);
                    if (!SG_TIMED(warp == 0 ? 3 : 6, mbar_wait_sleep(full_bar(slot), ph, abort_flag, a.sleep_cons))) { sg_fail(203); *abort_flag = 1; ok = false; break; }
                    if (!SG_TIMED(warp == 0 ? 4 : 7, mbar_wait_sleep(xfull_bar(xslot), xph, abort_flag, a.sleep_cons))) { sg_fail(206); *abort_flag = 1; ok = false; break; }
                    const uint32_t dep = stage_fn(s, nbv, sm.addr(slot), s_xs + (uint32_t)xslot * xs_bytes, empty_bar(slot));
                    __syncwarp();
                    if (lane == 0) mbar_arrive(xempty_bar(xslot) + (dep & a.zero));
                    slot += SG_GROUPS; if (slot >= nslots) { slot -= nslots; ph ^= 1u; }
                    xslot += SG_GROUPS; if (xslot >= nxs) { xslot -= nxs; xph ^= 1u; }
                }
                if (!ok) break;
                // hand the partial sums to the reducer warp (zeros if none of this unit's stages were mine); the
                // buffer of two units ago must have been drained
                const int buf = uc & 1;
                if (!SG_TIMED(warp == 0 ? 5 : 8, mbar_wait_sleep(red_empty(buf), ((uint32_t)(uc >> 1) & 1u) ^ 1u, abort_flag, a.sleep_cons))) { sg_fail(205); *abort_flag = 1; break; }
                flush_fn(s_red + (uint32_t)(buf * SG_RED_BYTES));
                __syncwarp();
                if (lane == 0) mbar_arrive(red_full(buf));
                ++uc;
                qb = qe; u = un_next; un = nx;
            }
        };
        // hands the weight slot back; `last` is a register filled by the slot's last load
        auto release_slot = [&](uint32_t ebar, uint32_t last) {
            const uint32_t dep = last & a.zero;
            __syncwarp();
            if (lane == 0) mbar_arrive(ebar + dep);
        };

        if (!dot) {
            // ---- batch 3 .. 8: tensor-core MMAs, two blocks x 16 rows per item
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            auto stage_mma = [&](int s, int nbv, uint32_t sb, uint32_t xb, uint32_t ebar) -> uint32_t {
                const int nv0 = nbv - (s * SG_STAGE_BLOCKS + 2 * kg0);   // real-k blocks from item 0's first block on
                fetch_stage(wA, sb + woff[0], sb + woff[1]);
#pragma unroll
                for (int i = 0; i < SG_ITEMS; ++i) {
                    uint32_t (&wc)[8] = (i & 1) ? wB : wA;
                    uint32_t (&wn)[8] = (i & 1) ? wA : wB;
                    if (i + 1 < SG_ITEMS) fetch_stage(wn, sb + woff[0] + (uint32_t)(i + 1) * ITEM_W, sb + woff[1] + (uint32_t)(i + 1) * ITEM_W);
                    if (i + 1 == SG_ITEMS) release_slot(ebar, wc[7]);     // the last item's bytes are needed now anyway
                    const int nvalid = nv0 - 2 * KG_STEP * i;
                    const uint32_t ao = xb + (uint32_t)i * ITEM_A, xo = xb + (uint32_t)i * ITEM_X;
                    if (nvalid >= 2) StageOps<XT>::stage(acc, wc, ao + aoff[0], ao + aoff[1], xo + xoff[0], xo + xoff[1], lane_word, hasx);
                    else if (nvalid == 1) StageOps<XT>::block(acc, wc, ao + aoff[0], xo + xoff[0], lane_word, hasx);
                }
                return __float_as_uint(acc[0]);
            };
            auto flush_mma = [&](uint32_t rb) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    sts_f32(rb + (uint32_t)(((warp * 8 + 2 * t + (c & 1)) * 20 + g + 8 * (c >> 1)) * 4), acc[c]);
                    acc[c] = 0.0f;
                }
            };
            run_units(stage_mma, flush_mma);
        } else {
            // ---- batch 1 and 2: dot products, one block x 32 rows per item, two items per loop trip
            float tot[SG_DOT_MAX_M] = {0.0f, 0.0f};
            auto flush_dot = [&](uint32_t rb) {
#pragma unroll
                for (int m = 0; m < SG_DOT_MAX_M; ++m) {
                    sts_f32(rb + (uint32_t)(((warp * SG_DOT_MAX_M + m) * 32 + lane) * 4), tot[m]);
                    tot[m] = 0.0f;
                }
            };
            auto stage_dot = [&](auto nm_tag, int s, int nbv, uint32_t sb, uint32_t xb, uint32_t ebar) -> uint32_t {
                constexpr int NM = decltype(nm_tag)::value;
                const int nvd = nbv - (s * SG_STAGE_BLOCKS + j);          // real-k blocks from my first block on, in steps of 4
                const uint32_t w0 = sb + woff[0], w1 = sb + woff[1];
                const uint32_t xx = xb + xoff[0];
                const uint32_t ab = xb + aoff[0];                     // my row's scale of block j + 4 i: fp32 [block][row]
                fetch_row_block(wA, w0, w1);
#pragma unroll 1
                for (int i = 0; i < SG_ITEMS; i += 2) {
                    fetch_row_block(wB, w0 + (uint32_t)(i + 1) * ITEM_W, w1 + (uint32_t)(i + 1) * ITEM_W);
                    if (nvd - 4 * i >= 1) dot_block<XT, NM>(tot, wA, lds_f32v(ab + (uint32_t)i * ITEM_A), xx + (uint32_t)i * ITEM_X, lane_word);
                    if (i + 2 < SG_ITEMS) fetch_row_block(wA, w0 + (uint32_t)(i + 2) * ITEM_W, w1 + (uint32_t)(i + 2) * ITEM_W);
                    else release_slot(ebar, wB[7]);
                    if (nvd - 4 * (i + 1) >= 1) dot_block<XT, NM>(tot, wB, lds_f32v(ab + (uint32_t)(i + 1) * ITEM_A), xx + (uint32_t)(i + 1) * ITEM_X, lane_word);
                }
                return __float_as_uint(tot[0]);
            };
            if (a.M == 1)
                run_units([&](int s, int nbv, uint32_t sb, uint32_t xb, uint32_t ebar) { return stage_dot(std::integral_constant<int, 1>{}, s, nbv, sb, xb, ebar); }, flush_dot);
            else
                run_units([&](int s, int nbv, uint32_t sb, uint32_t xb, uint32_t ebar) { return stage_dot(std::integral_constant<int, 2>{}, s, nbv, sb, xb, ebar); }, flush_dot);
        }
    }
    // After a time-out the roles leave early while copies may still be on their way into this CTA's
    // shared memory: give them a bounded moment to land before the CTA retires.
    __syncthreads();                                                 // every role of this CTA is done
#ifdef MPSBNB_TRACE
    if (blockIdx.x == 0 && tid == 0) atomicAdd(&g_wait[15], (unsigned long long)(clock64() - trace_t0));
#endif
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 400000ll) { }
        return;
    }
    if (a.ep.acc == nullptr || a.ep.tile_cnt != nullptr) return;
    // ---- closing step: the CTA that finishes last turns the accumulated o + down into the next layer's input
    volatile uint32_t *last_flag = abort_flag + 1;
    if (tid == 0) {
        __threadfence();
        *last_flag = atomicAdd(a.ep.counter, 1) == (int)gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (*last_flag == 0u) return;
    __threadfence();
    {
        const int total = a.ep.M * a.ep.hs;                          // hs is a multiple of 8
        XT *const *peers = reinterpret_cast<XT *const *>(a.ep.peer_h);
        for (int i = tid * 8; i < total; i += SG_THREADS * 8) {
            const int m = i / a.ep.hs, c = i - m * a.ep.hs;
            const float4 a0 = __ldcg(reinterpret_cast<const float4 *>(a.ep.acc + i));
            const float4 a1 = __ldcg(reinterpret_cast<const float4 *>(a.ep.acc + i + 4));
            *reinterpret_cast<float4 *>(a.ep.acc + i) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4 *>(a.ep.acc + i + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            const float al = a.ep.alpha;
            XT v[8] = {from_f32<XT>(al * a0.x), from_f32<XT>(al * a0.y), from_f32<XT>(al * a0.z), from_f32<XT>(al * a0.w),
                       from_f32<XT>(al * a1.x), from_f32<XT>(al * a1.y), from_f32<XT>(al * a1.z), from_f32<XT>(al * a1.w)};
            const uint4 bits = *reinterpret_cast<const uint4 *>(v);
            const int64_t o = (int64_t)m * a.ep.H + (int64_t)a.ep.rank * a.ep.hs + c;
            for (int r = 0; r < a.ep.nranks; ++r) *reinterpret_cast<uint4 *>(peers[r] + o) = bits;
        }
    }
    __threadfence_system();                                          // the stores before the flags
    __syncthreads();
    if (tid == 0) *a.ep.counter = 0;
    if (a.ep.peer_flags != nullptr && tid < a.ep.nranks)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.ep.peer_flags[tid] + a.ep.rank), "r"((*a.ep.step) * a.ep.mul + a.ep.add) : "memory");
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
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

struct HostLinear {
    const void *x; int64_t x_ld; int64_t x_period; const uint8_t *packed; const void *absmax; const float *absmax2;
    const void *bias; void *y; float *acc; int64_t N, K; int64_t segment;
};

static int fill_linear(StreamLinear &L, const HostLinear &h, int y_dtype) {
    if (h.N <= 0 || h.K <= 0 || h.N > 0x7fffffff || h.K > 0x7fffffff) return MPSBNB_ERR_INVALID_ARG;
    if (h.x == nullptr || h.packed == nullptr || h.absmax == nullptr || (h.y == nullptr && h.acc == nullptr)) return MPSBNB_ERR_INVALID_ARG;
    if (!aligned16(h.packed)) return MPSBNB_ERR_INVALID_ARG;
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return MPSBNB_ERR_NO_DEVICE;
    const int64_t Kp = padded_k(h.K, 64);
    const int64_t row_bytes = Kp / 2;
    CUresult cr = CUDA_ERROR_INVALID_VALUE;
    L.map3d = 0;
    if (row_bytes % 128 == 0) {
        // 3-D view {128 B, N rows, row_bytes / 128 parts}: a box {128, 32, 4} lands as [part][row][128 B],
        // the same shared-memory image as four 2-D boxes, with one instruction
        const cuuint64_t dims[3] = {128u, (cuuint64_t)h.N, (cuuint64_t)(row_bytes / 128)};
        const cuuint64_t strides[2] = {(cuuint64_t)row_bytes, 128u};
        const cuuint32_t box[3] = {128u, (cuuint32_t)SG_ROWS, 4u};
        const cuuint32_t estr[3] = {1u, 1u, 1u};
        cr = fn(&L.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t *>(h.packed), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        L.map3d = cr == CUDA_SUCCESS ? 1 : 0;
    }
    if (!L.map3d) {
        const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)h.N};
        const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
        const cuuint32_t box[2] = {128u, (cuuint32_t)SG_ROWS};
        const cuuint32_t estr[2] = {1u, 1u};
        cr = fn(&L.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(h.packed), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (cr != CUDA_SUCCESS) return MPSBNB_ERR_INVALID_ARG;
    L.x = h.x; L.absmax = h.absmax; L.absmax2 = h.absmax2; L.bias = h.bias; L.y = h.y; L.acc = h.acc;
    L.x_ld = h.x_ld;
    L.N = (int)h.N; L.K = (int)h.K; L.nb = (int)(Kp / 64); L.nbv = (int)((h.K + 63) / 64);
    L.segment = (int)h.segment;
    L.x_period = (int)(h.x_period > 0 ? h.x_period : h.K);
    L.y_dtype = y_dtype;
    L.x_vec_ok = (h.x_ld % 8 == 0) && (L.x_period % 8 == 0) && (h.K % 8 == 0) && aligned16(h.x);
    L.x_bulk_ok = L.x_vec_ok && (L.x_period >= L.K || L.x_period % (SG_STAGE_BLOCKS * 64) == 0);
    return MPSBNB_OK;
}

template <typename XT>
static int launch_stream(StreamArgs &args, cudaStream_t st, bool pdl = false, bool cooperative = false) {
    args.zero = 0u;
    args.sleep_cons = 32u; args.sleep_other = 200u;
    const int smem = SG_SMEM_BYTES;
    static int configured[64] = {};
    int dev = 0;
    MPSBNB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || configured[dev] < smem) {
        MPSBNB_CUDA_TRY(cudaFuncSetAttribute(mpsbnb_decode4_stream_kernel<XT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        if (dev >= 0 && dev < 64) configured[dev] = 227 * 1024;
    }
    int grid = sm_count();
    if (grid > args.nunits) grid = args.nunits;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(SG_THREADS); cfg.dynamicSmemBytes = (size_t)smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (cooperative) {
        // CTAs of one launch wait for each other's closing steps: all of them have to be resident
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
    } else {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
    }
    cfg.attrs = attr; cfg.numAttrs = (pdl || cooperative) ? 1 : 0;
    MPSBNB_CUDA_TRY(cudaLaunchKernelEx(&cfg, mpsbnb_decode4_stream_kernel<XT>, args));
    return check_launch();
}

int stream_status_fetch(int *out, bool reset) {
    MPSBNB_CUDA_TRY(cudaMemcpyFromSymbol(out, g_stream_status, sizeof(int)));
    if (reset) {
        const int zero = 0;
        MPSBNB_CUDA_TRY(cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int)));
    }
    return MPSBNB_OK;
}

#ifdef MPSBNB_TRACE
extern "C" int mpsbnb_debug_trace(unsigned long long *out768) {
    return cudaMemcpyFromSymbol(out768, g_trace, sizeof(unsigned long long) * 768) == cudaSuccess ? 0 : -3;
}
extern "C" int mpsbnb_debug_fail(unsigned int *out8) {
    if (cudaMemcpyFromSymbol(out8, g_fail, sizeof(unsigned int) * 8) != cudaSuccess) return -3;
    unsigned int z[8] = {0}; cudaMemcpyToSymbol(g_fail, z, sizeof(z));
    return 0;
}
extern "C" int mpsbnb_debug_waits(unsigned long long *out16, int reset) {
    if (cudaMemcpyFromSymbol(out16, g_wait, sizeof(unsigned long long) * 16) != cudaSuccess) return -3;
    if (reset) { unsigned long long z[16] = {0}; cudaMemcpyToSymbol(g_wait, z, sizeof(z)); }
    return 0;
}
#endif

// Single linear, M <= 8 (called from mpsbnb_gemv_4bit).
int gemv4_stream_single(const void *x, int x_dtype, int64_t M, const uint8_t *packed, const void *absmax,
                        const float *absmax2, int64_t N, int64_t K, int quant_type, const void *bias, void *y,
                        int y_dtype, cudaStream_t st) {
    StreamArgs args;
    memset(&args, 0, sizeof(args));
    args.lins = nullptr; args.units = nullptr;
    HostLinear h{x, K, K, packed, absmax, absmax2, bias, y, nullptr, N, K, 0};
    int rc = fill_linear(args.one, h, y_dtype);
    if (rc != MPSBNB_OK) return rc;
    args.nunits = (int)((N + SG_ROWS - 1) / SG_ROWS);
    args.M = (int)M; args.quant_type = quant_type;
    return x_dtype == MPSBNB_F16 ? launch_stream<__half>(args, st) : launch_stream<__nv_bfloat16>(args, st);
}

}  // namespace mpsbnb

using namespace mpsbnb;

// batch <= 8: this file's kernel; batch 9 .. 32: the tensor-memory kernel of gemv4_tc.cu
extern "C" int mpsbnb_gemv_4bit_group_max_m(void) { return 32; }

// ------------------------------------------------------------------------------------------
// grouped launches: a plan (device memory supplied by the caller) holds the linears and units
// ------------------------------------------------------------------------------------------
static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Stages per unit of a linear that adds into an accumulator (its K is cut so that the tiles of the layer boundary
// complete early and evenly): 8 when the accumulator has at least one 32-row tile per SM (one GPU holding a whole
// wide layer: fewer, longer units measured 3 % faster), else 4 (N-sharded: 8 was 12 % slower on an 8-way shard).
static int sg_chunk(const mpsbnb_linear4_desc *d, int n) {
    int64_t min_tiles = -1;
    for (int i = 0; i < n; ++i)
        if (d[i].acc != nullptr) {
            const int64_t t = (d[i].N + SG_ROWS - 1) / SG_ROWS;
            if (min_tiles < 0 || t < min_tiles) min_tiles = t;
        }
    return (min_tiles >= sm_count()) ? 8 : 4;
}
static int count_units(const mpsbnb_linear4_desc *d, int n, int chunk_stages) {
    int64_t total = 0;
    for (int i = 0; i < n; ++i) {
        const int64_t S = (padded_k(d[i].K, 64) / 64 + SG_STAGE_BLOCKS - 1) / SG_STAGE_BLOCKS;
        const int64_t chunks = d[i].acc != nullptr ? (S + chunk_stages - 1) / chunk_stages : 1;
        total += ((d[i].N + SG_ROWS - 1) / SG_ROWS) * chunks;
    }
    return total > 0x7fffffff ? -1 : (int)total;
}

extern "C" size_t mpsbnb_gemv_4bit_group_plan_bytes(const mpsbnb_linear4_desc *descs, int n_linears) {
    if (descs == nullptr || n_linears <= 0) return 0;
    const int nu = count_units(descs, n_linears, 4);            // the smaller chunk gives the larger plan
    if (nu < 0) return 0;
    const size_t mine = align_up(sizeof(StreamLinear) * (size_t)n_linears, 256) + align_up(sizeof(StreamUnit) * (size_t)nu, 256);
    const size_t other = tc_plan_bytes(descs, n_linears);
    return mine > other ? mine : other;
}

extern "C" int mpsbnb_gemv_4bit_group_plan(const mpsbnb_linear4_desc *descs, int n_linears, int64_t M, int x_dtype,
                                           int y_dtype, int quant_type, void *plan_dev, size_t plan_bytes,
                                           mpsbnb_group_plan *plan_out, void *stream) {
    if (descs == nullptr || n_linears <= 0 || plan_dev == nullptr || plan_out == nullptr) return MPSBNB_ERR_INVALID_ARG;
    if (!is_16bit(x_dtype) || !valid_dtype(y_dtype) || (quant_type != MPSBNB_NF4 && quant_type != MPSBNB_FP4)) return MPSBNB_ERR_INVALID_ARG;
    if (M <= 0 || M > 32) return MPSBNB_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(plan_dev) & 255) != 0) return MPSBNB_ERR_INVALID_ARG;
    if (M > SG_MAX_M)
        return tc_plan(descs, n_linears, M, x_dtype, y_dtype, quant_type, plan_dev, plan_bytes, plan_out, (cudaStream_t)stream);
    const int chunk = sg_chunk(descs, n_linears);
    const int nu = count_units(descs, n_linears, chunk);
    if (nu <= 0) return MPSBNB_ERR_INVALID_ARG;
    const size_t lin_bytes = align_up(sizeof(StreamLinear) * (size_t)n_linears, 256);
    const size_t need = lin_bytes + align_up(sizeof(StreamUnit) * (size_t)nu, 256);
    if (plan_bytes < need) return MPSBNB_ERR_WORKSPACE;
    unsigned char *host = (unsigned char *)malloc(need);
    if (host == nullptr) return MPSBNB_ERR_INVALID_ARG;
    memset(host, 0, need);
    StreamLinear *lins = reinterpret_cast<StreamLinear *>(host);
    StreamUnit *units = reinterpret_cast<StreamUnit *>(host + lin_bytes);
    int rc = MPSBNB_OK;
    int acc_parts = 0, n_segments = 1;
    for (int i = 0; i < n_linears && rc == MPSBNB_OK; ++i) {
        HostLinear h{descs[i].x, descs[i].x_ld, descs[i].x_period, descs[i].packed, descs[i].absmax, descs[i].absmax2,
                     descs[i].bias, descs[i].y, descs[i].acc, descs[i].N, descs[i].K, descs[i].segment};
        rc = fill_linear(lins[i], h, y_dtype);
    }
    if (rc == MPSBNB_OK) {
        // units: linears that add into an accumulator first (what depends on them can then be finished while
        // the rest of the launch still runs), within each class longest first so that the round-robin
        // remainder consists of the short ones
        int nu2 = 0;
        for (int i = 0; i < n_linears; ++i) {
            if (lins[i].segment < 0 || lins[i].segment >= 0x7fff) rc = MPSBNB_ERR_INVALID_ARG;
            else if (lins[i].segment + 1 > n_segments) n_segments = lins[i].segment + 1;
        }
        // contributions per accumulator tile: the same in every segment (the closing step counts to one number)
        for (int seg = 0; seg < n_segments && rc == MPSBNB_OK; ++seg) {
            int parts = 0;
            for (int i = 0; i < n_linears; ++i)
                if (lins[i].segment == seg && lins[i].acc != nullptr)
                    parts += ((lins[i].nb + SG_STAGE_BLOCKS - 1) / SG_STAGE_BLOCKS + chunk - 1) / chunk;
            if (seg == 0) acc_parts = parts;
            else if (parts != acc_parts) rc = MPSBNB_ERR_UNSUPPORTED;
        }
        for (int seg = 0; seg < n_segments; ++seg)
        for (int cls = 0; cls < 2; ++cls)
        for (int pass = chunk * 8; pass >= 1; --pass) {
            for (int i = 0; i < n_linears; ++i) {
                if (lins[i].segment != seg) continue;
                if ((lins[i].acc != nullptr) != (cls == 0)) continue;
                const int S = (lins[i].nb + SG_STAGE_BLOCKS - 1) / SG_STAGE_BLOCKS;
                const int step = lins[i].acc != nullptr ? chunk : S;
                for (int s0 = 0; s0 < S; s0 += step) {
                    const int s1 = s0 + step < S ? s0 + step : S;
                    const int len = s1 - s0 > chunk * 8 ? chunk * 8 : s1 - s0;
                    if (len != pass) continue;
                    for (int r0 = 0; r0 < lins[i].N; r0 += SG_ROWS) units[nu2++] = StreamUnit{i, r0, s0, s1, lins[i].nbv, 0, 0, 0};
                }
            }
        }
        if (rc == MPSBNB_OK && nu2 != nu) rc = MPSBNB_ERR_INVALID_ARG;
    }
    if (rc == MPSBNB_OK) {
        cudaStream_t st = (cudaStream_t)stream;
        cudaError_t e = cudaMemcpyAsync(plan_dev, host, need, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) rc = record_cuda_error(e);
    }
    free(host);
    if (rc != MPSBNB_OK) return rc;
    plan_out->dev = plan_dev;
    plan_out->units_offset = (int64_t)lin_bytes;
    plan_out->n_linears = n_linears;
    plan_out->n_units = nu;
    plan_out->M = (int)M;
    plan_out->x_dtype = x_dtype;
    plan_out->quant_type = quant_type;
    plan_out->flags = 0;
    plan_out->aux_offset = 0;
    plan_out->grid = 0;
    plan_out->impl = 0;
    plan_out->wait_flags = nullptr; plan_out->wait_step = nullptr;
    plan_out->wait_n = plan_out->wait_mul = plan_out->wait_add = 0;
    plan_out->acc_parts = acc_parts;
    plan_out->n_segments = n_segments; plan_out->wait_seg_mul = 0;
    memset(&plan_out->ep, 0, sizeof(plan_out->ep));
    return MPSBNB_OK;
}

extern "C" int mpsbnb_gemv_4bit_group_run(const mpsbnb_group_plan *plan, void *stream) {
    if (plan == nullptr || plan->dev == nullptr || plan->n_units <= 0) return MPSBNB_ERR_INVALID_ARG;
    if (plan->impl == 1) {
        if (plan->wait_n > 0 || plan->ep.acc != nullptr) return MPSBNB_ERR_UNSUPPORTED;   // both live in the default kernel
        return plan->grid > 0 ? tc_run(plan, (cudaStream_t)stream) : MPSBNB_ERR_INVALID_ARG;
    }
    StreamArgs args;
    memset(&args, 0, sizeof(args));
    args.lins = reinterpret_cast<const StreamLinear *>(plan->dev);
    args.units = reinterpret_cast<const StreamUnit *>(reinterpret_cast<const unsigned char *>(plan->dev) + plan->units_offset);
    args.nunits = plan->n_units; args.M = plan->M; args.quant_type = plan->quant_type;
    const bool tagged = plan->ep.acc != nullptr && plan->ep.count_tiles == 2;   // x and h travel in tagged form: no flags
    if (plan->wait_n > 0 || tagged) {
        if (plan->wait_step == nullptr || plan->wait_n > 32 || (plan->wait_n > 0 && plan->wait_flags == nullptr)) return MPSBNB_ERR_INVALID_ARG;
        args.wait_flags = plan->wait_flags; args.wait_step = plan->wait_step;
        args.wait_n = tagged ? 0 : plan->wait_n; args.wait_mul = plan->wait_mul; args.wait_add = plan->wait_add;
        args.wait_seg_mul = plan->wait_seg_mul > 0 ? plan->wait_seg_mul : 1;
    }
    if (plan->ep.acc != nullptr) {
        const mpsbnb_group_epilogue &e = plan->ep;
        if (e.peer_h == nullptr || e.counter == nullptr || e.M != plan->M || e.hs <= 0 || e.hs % 8 != 0 || e.nranks <= 0 ||
            e.nranks > 32 || e.rank < 0 || e.rank >= e.nranks || e.H < e.hs * e.nranks || ((e.peer_flags != nullptr || tagged) && e.step == nullptr) ||
            (tagged && (e.tile_cnt == nullptr || e.H % 2 != 0)) ||
            (e.tile_cnt != nullptr && (e.tile_expect <= 0 || e.tile_expect != plan->acc_parts)))
            return MPSBNB_ERR_INVALID_ARG;
        args.ep = e;
        args.x_ll = e.count_tiles == 2 ? 1 : 0;
    }
    const bool coop = plan->n_segments > 1;
    if (coop && (plan->ep.tile_cnt == nullptr || (!tagged && (plan->wait_n <= 0 || plan->ep.peer_flags == nullptr))))
        return MPSBNB_ERR_INVALID_ARG;                             // later segments need the streamed closing step and its flags or tags
    const bool pdl = (plan->flags & MPSBNB_GROUP_PDL) != 0 && !coop;
    return plan->x_dtype == MPSBNB_F16 ? launch_stream<__half>(args, (cudaStream_t)stream, pdl, coop)
                                       : launch_stream<__nv_bfloat16>(args, (cudaStream_t)stream, pdl, coop);
}
