// Decode-shape (M <= 32) 4-bit linear on the Blackwell tensor path: y[M,N] = x[M,K] . dequant(W)[N,K]^T.
//
// HBM-bound: the packed weights are read exactly once, by TMA, into a shared-memory ring; everything
// else is arranged so that the ring never waits.  One persistent CTA per SM, warp-specialised:
//
//   warp 16      TMA producer: one 16 KiB box (128 weight rows x 256 k, 128-byte swizzle) per stage.
//   warps 18-19  loaders: per stage the 128 x 4 block scales (fp32, or int8 * second-level absmax / 127)
//                and the 256 x values of every batch row, the latter written as the K-major, 128-byte
//                swizzled B tile [NB x 256] that tcgen05.mma reads (NB = 16 or 32 batch columns; rows >= M stay zero).
//   warps 0-15   expanders, in two groups of eight that take alternate stages (a warp passes the barriers once
//                per two stages; the groups overlap).  In a group, warp (h, r) owns weight rows 32 r .. 32 r + 31
//                and blocks 2 h, 2 h + 1 of the stage: a lane reads the 64 packed bytes of ITS row, turns every
//                byte into a (code, code) half2 with one byte-permute + one shared load (lane-replicated
//                256-entry table), multiplies by the block scale and stores the 2 x 64 fp16 weights with two
//                tcgen05.st into the A tile in tensor memory (TMEM lane = weight row, 2 k per 32-bit column).
//                No mma.sync, no fragment shuffles.
//   warp 17      one thread issues 16 tcgen05.mma (M = 128, N = NB, K = 16; A from TMEM, B = x from shared
//                memory) per stage into fp32 accumulators in TMEM and commits to mbarriers.
//   warps 20-23  epilogue: when a row tile's K range is finished, read the accumulator (tcgen05.ld), add the
//                bias, store y (or atomically add into an fp32 target).
//
// Work split: the stages of all row tiles of all linears of a launch form one sequence that is cut into
// equal contiguous ranges, one per CTA.  A row tile cut by a range boundary is finished by two CTAs: both
// add their partial sums into an fp32 workspace and the one that arrives last converts (a counter per
// tile quarter; nobody waits for anybody).
//
// Every wait is bounded (sm100.cuh); a time-out raises the CTA's abort flag, all roles leave their loops,
// and the CTA frees its tensor memory before it retires.
#include "common.cuh"
#include "ops.cuh"
#include "sm100.cuh"

#include <stdlib.h>
#include <string.h>

namespace mpsbnb {

using namespace sm100;

constexpr int TG_CONSUMERS = 16;
constexpr int TG_EGROUPS = 2;                              // expander groups (of TG_CONSUMERS / TG_EGROUPS warps) that alternate stages
constexpr int TG_GROUP_WARPS = TG_CONSUMERS / TG_EGROUPS;
constexpr int TG_WARP_PRODUCER = 16, TG_WARP_MMA = 17, TG_WARP_LOADER0 = 18, TG_LOADERS = 2, TG_WARP_EPI0 = 20;
constexpr int TG_THREADS = 24 * 32;
constexpr int TG_ROWS = 128;                               // weight rows per tile = UMMA M
constexpr int TG_STAGE_BLOCKS = 4;                         // quantisation blocks (64 k) per stage
constexpr int TG_STAGE_K = TG_STAGE_BLOCKS * 64;
constexpr int TG_W_BYTES = TG_ROWS * TG_STAGE_K / 2;       // 16384
constexpr int TG_A_BYTES = TG_STAGE_BLOCKS * TG_ROWS * 4;  // 2048: fp32 scale [row][block], or int8 codes [row] + fp32 maxima [row]
constexpr int TG_NXS = 4;                                  // scale/x slots (a multiple of TG_LOADERS: one loader per slot)
constexpr int TG_MAX_SLOTS = 9;
constexpr int TG_ABUFS = 3;                                // A tiles in tensor memory (128 columns each)
constexpr int TG_MAX_M = 32;                               // largest batch (the 32-column instance)
constexpr uint32_t TG_LUT_ABS = 131072u;                   // table at an absolute shared address: see expander
constexpr uint32_t TG_HIGH_ABS = TG_LUT_ABS + 65536u;      // entry b of lane l sits at b * 256 + l * 4: a 64 KiB span
constexpr int TG_SMEM_BYTES = 227 * 1024;
constexpr uint32_t TG_TMEM_COLS = 512, TG_D_COL0 = TG_ABUFS * 128;
// Consecutive K steps add into tg_dsplit(NB) different accumulators (step j -> accumulator j % split), which
// the epilogue sums.  (Measured: an MMA of this shape costs about 46 cycles whatever N <= 64 is and whether
// or not consecutive MMAs share an accumulator, so the split neither helps nor hurts; it keeps the fp32
// partial sums of a long K shorter.)
// (two accumulator buffers of NB * split columns each fit the 128 columns left beside the A tiles.)
__host__ __device__ constexpr int tg_dsplit(int nb) { return 64 / nb; }
static_assert(TG_NXS % TG_LOADERS == 0, "each scale/x slot must belong to exactly one loader warp");

static __device__ int g_tc_status = 0;

struct TcLinear {
    CUtensorMap map;          // packed weights as [N][row_bytes] bytes; box 128 B x 128 rows, 128-byte swizzle
    const void *x;            // activations [M, x_ld]; column index is taken modulo x_period
    const void *absmax;       // fp32 [N, nb], or int8 [N, nb] when absmax2 != nullptr
    const float *absmax2;     // fp32 [ceil(N nb / 256)] or nullptr
    const void *bias;         // [N] in the activation dtype, or nullptr
    void *y;                  // [M, N] in y_dtype; used when acc == nullptr
    float *acc;               // fp32 [M, N] atomicAdd target, or nullptr
    float *ws;                // fp32 [M, N], all zero between launches: partial sums of tiles cut between CTAs
    int *cnt;                 // [4 * tiles], all zero between launches: arrivals per tile quarter
    int64_t x_ld;
    int N, K, nb;             // nb: blocks per row in the layout
    int x_period;             // x column = k mod x_period (x_period >= K: plain)
    int y_dtype;
    int x_vec_ok;             // 16-byte loads of x are legal and never straddle K or the period
    int scale_async;          // every stage's scales of a row are one aligned, complete group of four: async copies
    int pad1;
};

struct __align__(16) TcPiece { int lin, row0, s_begin, s_end, parts, pad0, pad1, pad2; };   // parts: pieces of this tile (1 = whole)

struct TcArgs {
    const TcLinear *lins;     // device array, or nullptr: use `one`
    const TcPiece *pieces;    // device array, or nullptr: piece p = row tile p of `one`, whole K
    const int *cta_first;     // [grid + 1] first piece of every CTA (with `pieces`)
    int npieces, M, quant_type;
    uint32_t zero;            // always 0; known only at run time
    TcLinear one;
};

template <typename XT> __host__ __device__ constexpr int tg_fmt();            // tcgen05 operand format code
template <> __host__ __device__ constexpr int tg_fmt<__half>() { return 0; }
template <> __host__ __device__ constexpr int tg_fmt<__nv_bfloat16>() { return 1; }
template <typename XT> __device__ __forceinline__ uint32_t tg_pair_bits(float lo, float hi);
template <> __device__ __forceinline__ uint32_t tg_pair_bits<__half>(float lo, float hi) { const __half2 h = __floats2half2_rn(lo, hi); return *reinterpret_cast<const uint32_t *>(&h); }
template <> __device__ __forceinline__ uint32_t tg_pair_bits<__nv_bfloat16>(float lo, float hi) { const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<const uint32_t *>(&h); }
template <typename XT> __device__ __forceinline__ uint32_t tg_mul2(uint32_t a, uint32_t b);
template <> __device__ __forceinline__ uint32_t tg_mul2<__half>(uint32_t a, uint32_t b) { uint32_t d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
template <> __device__ __forceinline__ uint32_t tg_mul2<__nv_bfloat16>(uint32_t a, uint32_t b) { uint32_t d; asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }

__device__ __forceinline__ void tg_sts_f32(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void tg_sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ void tg_sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 tg_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t tg_lds_u32(uint32_t addr) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory"); return v; }
__device__ __forceinline__ float tg_lds_f32(uint32_t addr) { float v; asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory"); return v; }
// Ampere-style asynchronous copies global -> shared (4 or 16 bytes per thread); `bytes_valid` < 16 zero-fills.
__device__ __forceinline__ void tg_cp_async4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void tg_cp_async16(uint32_t dst, const void *src, uint32_t bytes_valid) {
    // .cg: L2 only.  x is rewritten between the layers of a stack while, with programmatic dependent launch, this SM's
    // L1 can still hold the lines the previous layer's kernel read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes_valid) : "memory");
}
// one arrival on `bar` once all asynchronous copies this thread has issued so far have landed
__device__ __forceinline__ void tg_cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// table load: the table never changes after the prologue, so the compiler may move this freely
__device__ __forceinline__ uint32_t tg_lut(uint32_t addr) { uint32_t v; asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr)); return v; }

struct TgSlots {
    uint32_t low0, high0;
    int nlow, nslots;
    __device__ __forceinline__ uint32_t addr(int slot) const {
        return slot < nlow ? low0 + (uint32_t)slot * TG_W_BYTES : high0 + (uint32_t)(slot - nlow) * TG_W_BYTES;
    }
};

template <typename XT, int NB>
__global__ void __launch_bounds__(TG_THREADS, 1) mpsbnb_decode4_tmem_kernel(const __grid_constant__ TcArgs a) {
    // NB = batch rows the x tile and the accumulators hold (the UMMA N): 16 or 32
    constexpr int X_BYTES = NB * TG_STAGE_K * 2;                     // four [NB x 64] atoms of NB * 128 bytes
    constexpr int XS_BYTES = X_BYTES + TG_A_BYTES;
    constexpr int DSPLIT = tg_dsplit(NB);
    constexpr uint32_t D_STRIDE = NB * DSPLIT;                       // columns per accumulator buffer
    static_assert(TG_D_COL0 + 2 * D_STRIDE <= TG_TMEM_COLS && TG_STAGE_K / 16 >= DSPLIT, "accumulators fit; the first stage initialises all");
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t s_base = smem_u32(smem);
    // barriers: full[9] empty[9] xfull[4] xempty[4] afull[3] aempty[3] dfull[2] dempty[2]; then the TMEM
    // address holder (+320) and the abort flag (+324)
    const uint32_t s_bar = s_base;
    auto full_bar = [&](int s) { return s_bar + 8u * s; };
    auto empty_bar = [&](int s) { return s_bar + 8u * (TG_MAX_SLOTS + s); };
    auto xfull_bar = [&](int s) { return s_bar + 8u * (2 * TG_MAX_SLOTS + s); };
    auto xempty_bar = [&](int s) { return s_bar + 8u * (2 * TG_MAX_SLOTS + TG_NXS + s); };
    auto afull_bar = [&](int s) { return s_bar + 8u * (2 * TG_MAX_SLOTS + 2 * TG_NXS + s); };
    auto aempty_bar = [&](int s) { return s_bar + 8u * (2 * TG_MAX_SLOTS + 2 * TG_NXS + TG_ABUFS + s); };
    auto dfull_bar = [&](int s) { return s_bar + 8u * (2 * TG_MAX_SLOTS + 2 * TG_NXS + 2 * TG_ABUFS + s); };
    auto dempty_bar = [&](int s) { return s_bar + 8u * (2 * TG_MAX_SLOTS + 2 * TG_NXS + 2 * TG_ABUFS + 2 + s); };
    static_assert(8 * (2 * TG_MAX_SLOTS + 2 * TG_NXS + 2 * TG_ABUFS + 4) <= 320, "barrier area");
    const uint32_t s_holder = s_bar + 320u;
    const uint32_t s_mode = s_bar + 336u;                             // per scale/x slot: 1 = raw int8 scales + second-level maxima

    const uint32_t s_xs = (s_bar + 512u + 1023u) & ~1023u;            // scale/x ring: [x tile 8 KiB][scales 2 KiB] per slot
    TgSlots sm;
    sm.low0 = s_xs + (uint32_t)(TG_NXS * XS_BYTES);
    sm.high0 = TG_HIGH_ABS;
    sm.nlow = (int)((TG_LUT_ABS - sm.low0) / TG_W_BYTES);
    {
        const int nhigh = (int)((s_base + (uint32_t)TG_SMEM_BYTES - TG_HIGH_ABS) / TG_W_BYTES);
        const int n = sm.nlow + nhigh;
        sm.nslots = n > TG_MAX_SLOTS ? TG_MAX_SLOTS : n;
        if (sm.nlow > sm.nslots) sm.nlow = sm.nslots;
    }
    const int nslots = sm.nslots;
    unsigned char *p_generic0 = smem - s_base;                       // generic pointer of shared address 0
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(p_generic0 + s_bar + 324u);
    volatile uint32_t *holder = reinterpret_cast<volatile uint32_t *>(p_generic0 + s_holder);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();

    if (tid == 0) {
        for (int s = 0; s < nslots; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), TG_GROUP_WARPS); }
        for (int s = 0; s < TG_NXS; ++s) { mbar_init(xfull_bar(s), 32); mbar_init(xempty_bar(s), TG_GROUP_WARPS + 1); }
        for (int s = 0; s < TG_ABUFS; ++s) { mbar_init(afull_bar(s), TG_GROUP_WARPS); mbar_init(aempty_bar(s), 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(dfull_bar(s), 1); mbar_init(dempty_bar(s), 4); }
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
        const uint32_t mine = tg_pair_bits<XT>(lo, hi);
#pragma unroll 8
        for (int j = 0; j < 32; ++j)
            tg_sts32(TG_LUT_ABS + (uint32_t)((warp * 32 + j) * 256 + lane * 4), __shfl_sync(0xffffffffu, mine, j));
    } else if (warp < 16) {
        // the scale/x ring starts as zeros: batch rows >= M of every x tile are never written
        const int total = TG_NXS * XS_BYTES;
        for (int o = (tid - 256) * 16; o < total; o += 256 * 16) tg_sts128(s_xs + o, make_uint4(0u, 0u, 0u, 0u));
    } else if (warp == TG_WARP_MMA) {
        tmem_alloc(s_holder, TG_TMEM_COLS);
        tmem_relinquish();
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *holder;

    int p_first, p_last, p_step;
    if (a.pieces != nullptr) { p_first = a.cta_first[blockIdx.x]; p_last = a.cta_first[blockIdx.x + 1]; p_step = 1; }
    else { p_first = (int)blockIdx.x; p_last = a.npieces; p_step = (int)gridDim.x; }
    auto piece_of = [&](int p) -> TcPiece {
        if (a.pieces != nullptr) return a.pieces[p];
        TcPiece q;
        q.lin = 0; q.row0 = p * TG_ROWS; q.s_begin = 0; q.s_end = (a.one.nb + TG_STAGE_BLOCKS - 1) / TG_STAGE_BLOCKS; q.parts = 1;
        q.pad0 = q.pad1 = q.pad2 = 0;
        return q;
    };
    auto lin_of = [&](int i) -> const TcLinear * { return a.lins != nullptr ? a.lins + i : &a.one; };
    constexpr uint32_t kSleepFast = 20u, kSleepSlow = 200u;

    if (warp == TG_WARP_PRODUCER) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int slot = 0; uint32_t ph = 0;
            bool ok = true;
            for (int p = p_first; p < p_last && ok && !*abort_flag; p += p_step) {
                const TcPiece pc = piece_of(p);
                const CUtensorMap *map = &lin_of(pc.lin)->map;
                for (int s = pc.s_begin; s < pc.s_end; ++s) {
                    if (!mbar_wait_sleep(empty_bar(slot), ph ^ 1u, abort_flag, kSleepSlow)) { atomicExch(&g_tc_status, 401); *abort_flag = 1; ok = false; break; }
                    mbar_arrive_expect_tx(full_bar(slot), TG_W_BYTES);
                    tma_load_2d(sm.addr(slot), map, full_bar(slot), s * 128, pc.row0);
                    if (++slot == nslots) { slot = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == TG_WARP_MMA) {
        // ------------------------------------------------------------ MMA issue
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(tg_fmt<XT>(), TG_ROWS, NB);
            int abuf = 0, xslot = 0, dcount = 0;
            uint32_t aph = 0, xph = 0;
            bool ok = true;
            for (int p = p_first; p < p_last && ok && !*abort_flag; p += p_step, ++dcount) {
                const TcPiece pc = piece_of(p);
                const int d = dcount & 1;
                if (!mbar_wait_sleep(dempty_bar(d), (((uint32_t)dcount >> 1) & 1u) ^ 1u, abort_flag, kSleepFast)) { atomicExch(&g_tc_status, 402); *abort_flag = 1; break; }
                const uint32_t tmem_d = tmem_base + TG_D_COL0 + D_STRIDE * (uint32_t)d;
                for (int s = pc.s_begin; s < pc.s_end; ++s) {
                    if (!mbar_wait_sleep(xfull_bar(xslot), xph, abort_flag, kSleepFast)) { atomicExch(&g_tc_status, 403); *abort_flag = 1; ok = false; break; }
                    if (!mbar_wait_sleep(afull_bar(abuf), aph, abort_flag, kSleepFast)) { atomicExch(&g_tc_status, 404); *abort_flag = 1; ok = false; break; }
                    tc_fence_after();
                    fence_proxy_async_smem();                            // the x tile was written through the generic proxy
                    const uint64_t xdesc = umma_desc_k_sw128(s_xs + (uint32_t)(xslot * XS_BYTES));
                    const uint32_t tmem_a = tmem_base + (uint32_t)(abuf * 128);
#pragma unroll
                    for (int j = 0; j < TG_STAGE_K / 16; ++j) {
                        // K step j: 8 columns of the A tile; 32 bytes further in the 128-byte row of atom j / 4
                        const uint64_t bd = xdesc + (uint64_t)((((j >> 2) * (NB * 128)) + (j & 3) * 32) >> 4);
                        umma_f16_tmem_a(tmem_d + (uint32_t)(NB * (j % DSPLIT)), tmem_a + (uint32_t)(8 * j), bd, idesc,
                                        s > pc.s_begin || j >= DSPLIT);
                    }
                    umma_commit(aempty_bar(abuf));
                    umma_commit(xempty_bar(xslot));
                    if (++abuf == TG_ABUFS) { abuf = 0; aph ^= 1u; }
                    if (++xslot == TG_NXS) { xslot = 0; xph ^= 1u; }
                }
                if (!ok) break;
                umma_commit(dfull_bar(d));
            }
        }
    } else if (warp >= TG_WARP_EPI0) {
        // ------------------------------------------------------------ epilogue: accumulator -> y
        const int e = warp - TG_WARP_EPI0;                               // TMEM lane quarter
        pdl_grid_dependency_wait();                                      // outputs may still be in use by the previous kernel
        int dcount = 0;
        for (int p = p_first; p < p_last && !*abort_flag; p += p_step, ++dcount) {
            const TcPiece pc = piece_of(p);
            const TcLinear *L = lin_of(pc.lin);
            const int LN = L->N, ydt = L->y_dtype;
            const void *bias = L->bias;
            float *acc = L->acc, *ws = L->ws;
            void *y = L->y;
            const int d = dcount & 1;
            if (!mbar_wait_sleep(dfull_bar(d), ((uint32_t)dcount >> 1) & 1u, abort_flag, kSleepSlow)) { atomicExch(&g_tc_status, 405); *abort_flag = 1; break; }
            tc_fence_after();
            float v[NB];
#pragma unroll
            for (int i = 0; i < NB; ++i) v[i] = 0.0f;
            {
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * e) << 16) + TG_D_COL0 + D_STRIDE * (uint32_t)d;
#pragma unroll
                for (int q = 0; q < DSPLIT; ++q) {
                    uint32_t part[NB];
#pragma unroll
                    for (int c = 0; c < NB / 8; ++c) {
                        uint32_t r8[8];
                        if (a.M > 8 * c) {
                            tmem_ld_32x8(taddr + (uint32_t)(NB * q + 8 * c), r8);
#pragma unroll
                            for (int i = 0; i < 8; ++i) part[8 * c + i] = r8[i];
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) part[8 * c + i] = 0u;
                        }
                    }
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < NB; ++i) v[i] += __uint_as_float(part[i]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(dempty_bar(d));
            const int n = pc.row0 + 32 * e + lane;
            const bool mine = n < LN;
            const float bv = (mine && bias != nullptr) ? to_f32<XT>(reinterpret_cast<const XT *>(bias)[n]) : 0.0f;
            auto store_y = [&](int m, float val) {
                const int64_t o = (int64_t)m * LN + n;
                if (ydt == MPSBNB_F16) reinterpret_cast<__half *>(y)[o] = __float2half_rn(val);
                else if (ydt == MPSBNB_BF16) reinterpret_cast<__nv_bfloat16 *>(y)[o] = __float2bfloat16_rn(val);
                else reinterpret_cast<float *>(y)[o] = val;
            };
            if (acc != nullptr) {
                if (mine)
#pragma unroll
                    for (int m = 0; m < NB; ++m) if (m < a.M) atomicAdd(acc + (int64_t)m * LN + n, v[m] + (pc.s_begin == 0 ? bv : 0.0f));
            } else if (pc.parts == 1) {
                if (mine)
#pragma unroll
                    for (int m = 0; m < NB; ++m) if (m < a.M) store_y(m, v[m] + bv);
            } else {
                if (mine)
#pragma unroll
                    for (int m = 0; m < NB; ++m) if (m < a.M) atomicAdd(ws + (int64_t)m * LN + n, v[m]);
                __threadfence();
                __syncwarp();
                int old = 0;
                int *cnt = L->cnt + (pc.row0 / TG_ROWS) * 4 + e;
                if (lane == 0) old = atomicAdd(cnt, 1);
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old == pc.parts - 1) {
                    // last piece of this tile quarter: every partial sum is in the workspace
                    __threadfence();
                    if (mine)
                        for (int m = 0; m < a.M; ++m) {
                            float *w = ws + (int64_t)m * LN + n;
                            const float total = __ldcg(w);
                            *w = 0.0f;
                            store_y(m, total + bv);
                        }
                    if (lane == 0) *cnt = 0;
                }
            }
        }
    } else if (warp >= TG_WARP_LOADER0) {
        // ------------------------------------------------------------ loaders: block scales and the x tile
        const int me = warp - TG_WARP_LOADER0;
        pdl_grid_dependency_wait();                                      // x is written by the previous kernel in the stream
        auto read_scales = [&](const TcLinear *L, int row0, int s, float (&sc)[16]) {
            const int b0 = s * TG_STAGE_BLOCKS;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int n = row0 + lane + 32 * i;
                const int64_t i0 = (int64_t)n * L->nb + b0;
                if (n >= L->N) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) sc[4 * i + j] = 0.0f;
                } else if (L->absmax2 == nullptr) {
                    const float *am = reinterpret_cast<const float *>(L->absmax);
                    if (b0 + 4 <= L->nb && (i0 & 3) == 0) {
                        const float4 v = __ldg(reinterpret_cast<const float4 *>(am + i0));
                        sc[4 * i] = v.x; sc[4 * i + 1] = v.y; sc[4 * i + 2] = v.z; sc[4 * i + 3] = v.w;
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) sc[4 * i + j] = (b0 + j < L->nb) ? __ldg(am + i0 + j) : 0.0f;
                    }
                } else {
                    // int8 code * (second-level maximum / 127), as the reference expands it
                    const int8_t *aq = reinterpret_cast<const int8_t *>(L->absmax);
                    if (b0 + 4 <= L->nb && (i0 & 3) == 0) {
                        const uint32_t raw = __ldg(reinterpret_cast<const uint32_t *>(aq + i0));
                        const float f = __fdiv_rn(__ldg(L->absmax2 + (i0 >> 8)), 127.0f);
#pragma unroll
                        for (int j = 0; j < 4; ++j) sc[4 * i + j] = (float)(int)(int8_t)((raw >> (8 * j)) & 0xFFu) * f;
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            sc[4 * i + j] = (b0 + j < L->nb)
                                ? (float)(int)__ldg(aq + i0 + j) * __fdiv_rn(__ldg(L->absmax2 + ((i0 + j) >> 8)), 127.0f) : 0.0f;
                    }
                }
            }
        };
        // my 16-byte chunk of the 256 x values of batch row m in stage s (zero beyond K)
        auto read_x = [&](const TcLinear *L, int s, int m) -> uint4 {
            const int k0 = s * TG_STAGE_K + lane * 8;
            const XT *xr = reinterpret_cast<const XT *>(L->x) + (int64_t)m * L->x_ld;
            if (L->x_vec_ok) {
                if (k0 >= L->K) return make_uint4(0u, 0u, 0u, 0u);
                // L2 only: with programmatic dependent launch this SM's L1 may still hold lines of x that the previous
                // layer's kernel read before the boundary kernel rewrote them
                return __ldcg(reinterpret_cast<const uint4 *>(xr + (k0 % L->x_period)));
            }
            uint16_t ev[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                ev[j] = (k0 + j < L->K) ? __ldcg(reinterpret_cast<const unsigned short *>(xr + (k0 + j) % L->x_period)) : (unsigned short)0;
            return make_uint4(ev[0] | ((uint32_t)ev[1] << 16), ev[2] | ((uint32_t)ev[3] << 16),
                              ev[4] | ((uint32_t)ev[5] << 16), ev[6] | ((uint32_t)ev[7] << 16));
        };
        // cursor over the CTA's stage sequence; `turn` = stage index modulo TG_LOADERS
        int p = p_first;
        TcPiece pc = {0, 0, 0, 0, 1, 0, 0, 0};
        const TcLinear *L = nullptr;
        int s = 0, turn = 0, xslot = 0;
        uint32_t xph = 0;
        bool have = false;
        auto step = [&]() {
            ++s;
            if (++turn == TG_LOADERS) turn = 0;
            if (++xslot == TG_NXS) { xslot = 0; xph ^= 1u; }
        };
        auto advance_to_mine = [&]() {
            for (;;) {
                if (!have) {
                    if (p >= p_last) return false;
                    pc = piece_of(p); L = lin_of(pc.lin); s = pc.s_begin; have = true;
                }
                if (s >= pc.s_end) { have = false; p += p_step; continue; }
                if (turn == me) return true;
                step();
            }
        };
        float cur[16];
        bool more = advance_to_mine();
        if (more && !L->scale_async) read_scales(L, pc.row0, s, cur);
        while (more && !*abort_flag) {
            const int my_x = xslot, my_s = s, my_row0 = pc.row0;
            const uint32_t my_ph = xph;
            const TcLinear *my_L = L;
            const bool my_async = my_L->scale_async != 0;
            step();
            float nxt[16];
            more = advance_to_mine();
            if (more && !L->scale_async) read_scales(L, pc.row0, s, nxt);
            if (!mbar_wait_sleep(xempty_bar(my_x), my_ph ^ 1u, abort_flag, kSleepSlow)) { atomicExch(&g_tc_status, 406); *abort_flag = 1; break; }
            const uint32_t xb = s_xs + (uint32_t)(my_x * XS_BYTES);
            const uint32_t ab = xb + X_BYTES;
            if (my_async) {
                // scales: nothing passes through registers, so this warp never waits for global memory and runs
                // as far ahead as the ring allows.  Row n gets its four codes (or floats) and its second-level maximum.
                const int b0 = my_s * TG_STAGE_BLOCKS;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = lane + 32 * i;
                    const int n = my_row0 + rr;
                    if (n < my_L->N) {
                        const int64_t i0 = (int64_t)n * my_L->nb + b0;
                        if (my_L->absmax2 != nullptr) {
                            tg_cp_async4(ab + (uint32_t)(rr * 4), reinterpret_cast<const int8_t *>(my_L->absmax) + i0);
                            tg_cp_async4(ab + 512u + (uint32_t)(rr * 4), my_L->absmax2 + (i0 >> 8));
                        } else {
                            tg_cp_async16(ab + (uint32_t)(rr * 16), reinterpret_cast<const float *>(my_L->absmax) + i0, 16u);
                        }
                    } else if (my_L->absmax2 != nullptr) {
                        tg_sts32(ab + (uint32_t)(rr * 4), 0u);
                        tg_sts_f32(ab + 512u + (uint32_t)(rr * 4), 0.0f);
                    } else {
                        tg_sts128(ab + (uint32_t)(rr * 16), make_uint4(0u, 0u, 0u, 0u));
                    }
                }
                if (lane == 0) tg_sts32(s_mode + 4u * my_x, my_L->absmax2 != nullptr ? 1u : 0u);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    tg_sts128(ab + (uint32_t)((lane + 32 * i) * 16),
                              make_uint4(__float_as_uint(cur[4 * i]), __float_as_uint(cur[4 * i + 1]), __float_as_uint(cur[4 * i + 2]), __float_as_uint(cur[4 * i + 3])));
                if (lane == 0) tg_sts32(s_mode + 4u * my_x, 0u);
            }
            // x tile: row m of atom (lane >> 3) (rows 8..15 are the second 8-row group, 1 KiB further), 16-byte chunk
            // (lane & 7) ^ (m & 7)  (128-byte swizzle)
            // Everything that does not depend on m is computed once: the asynchronous copies below are "memory"
            // operations to the compiler, so a load or the 64-bit modulo left inside the loop would be redone for
            // every batch row (that made the loaders the limit of the kernel from batch 8 up).
            {
                const int k0 = my_s * TG_STAGE_K + lane * 8;
                const bool vec = my_L->x_vec_ok != 0;
                const bool in = k0 < my_L->K;
                const int64_t ld = my_L->x_ld;
                const XT *src = reinterpret_cast<const XT *>(my_L->x) + (in && vec ? k0 % my_L->x_period : 0);
                const uint32_t nbytes = in ? 16u : 0u;
                const uint32_t dst0 = xb + (uint32_t)((lane >> 3) * (NB * 128));
                const int M = a.M;
                if (vec) {
#pragma unroll 4
                    for (int m = 0; m < M; ++m, src += ld)
                        tg_cp_async16(dst0 + (uint32_t)((m >> 3) * 1024 + (m & 7) * 128 + (((lane & 7) ^ (m & 7)) << 4)), src, nbytes);
                } else {
                    for (int m = 0; m < M; ++m)
                        tg_sts128(dst0 + (uint32_t)((m >> 3) * 1024 + (m & 7) * 128 + (((lane & 7) ^ (m & 7)) << 4)), read_x(my_L, my_s, m));
                }
            }
            fence_proxy_async_smem();
            tg_cp_async_arrive(xfull_bar(my_x));                         // 32 arrivals complete the slot
#pragma unroll
            for (int j = 0; j < 16; ++j) cur[j] = nxt[j];
        }
    } else {
        // ------------------------------------------------------------ expanders: packed bytes -> fp16 weights in TMEM
        // Two groups of eight warps; group g takes the stages q = g, g + 2, ... of the CTA's sequence, so a warp
        // goes through the barriers once per TWO stages and the groups overlap each other.  Inside a group warp
        // (h, r) owns weight rows 32 r .. 32 r + 31 and the blocks 2 h, 2 h + 1 of the stage.
        const int g = warp >> 3, h = (warp >> 2) & 1, r = warp & 3;
        const int row = 32 * r + lane;
        const uint32_t lane_word = TG_LUT_ABS | ((uint32_t)lane * 4u);   // bytes 0, 2, 3 of every table address
        const uint32_t tmem_mine = tmem_base + ((uint32_t)(32 * r) << 16) + (uint32_t)(64 * h);
        uint32_t woff[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) woff[c] = (uint32_t)(row * 128 + (((4 * h + c) ^ (row & 7)) << 4));
        // ring positions of stage q = g: every ring is entered at position g and advanced by TG_EGROUPS per stage
        int slot = g % nslots, xslot = g % TG_NXS, abuf = g % TG_ABUFS;
        uint32_t ph = (uint32_t)(g / nslots) & 1u, xph = (uint32_t)(g / TG_NXS) & 1u, aph = (uint32_t)(g / TG_ABUFS) & 1u;
        bool ok = true;
        int total = 0;                                                   // stages of this CTA
        for (int p = p_first; p < p_last; p += p_step) { const TcPiece pc = piece_of(p); total += pc.s_end - pc.s_begin; }
        for (int q = g; q < total && ok && !*abort_flag; q += TG_EGROUPS) {
            // the stage's packed bytes: this lane's 64 bytes, then the slot is free for the producer
            if (!mbar_wait_sleep(full_bar(slot), ph, abort_flag, kSleepFast)) { atomicExch(&g_tc_status, 407); *abort_flag = 1; ok = false; break; }
            const uint32_t sb = sm.addr(slot);
            uint4 w4[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) w4[c] = tg_lds128(sb + woff[c]);
            {
                const uint32_t dep = w4[3].w & a.zero;                   // the arrive cannot issue before the loads returned
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(slot) + dep);
            }
            if (!mbar_wait_sleep(xfull_bar(xslot), xph, abort_flag, kSleepFast)) { atomicExch(&g_tc_status, 408); *abort_flag = 1; ok = false; break; }
            const uint32_t ab = s_xs + (uint32_t)(xslot * XS_BYTES) + X_BYTES;
            const bool coded = tg_lds_u32(s_mode + 4u * xslot) != 0u;   // int8 codes [row] + second-level maximum [row], or fp32 [row][4]
            const uint32_t codes = coded ? tg_lds_u32(ab + (uint32_t)(row * 4)) : 0u;
            const float f2 = coded ? __fdiv_rn(tg_lds_f32(ab + 512u + (uint32_t)(row * 4)), 127.0f) : 0.0f;
#pragma unroll
            for (int bb = 0; bb < 2; ++bb) {
                const int blk = 2 * h + bb;
                const float scale = coded ? (float)(int)(int8_t)((codes >> (8 * blk)) & 0xFFu) * f2
                                          : tg_lds_f32(ab + (uint32_t)(row * 16 + blk * 4));
                const uint32_t s2 = tg_pair_bits<XT>(scale, scale);
                const uint32_t wv[8] = {w4[2 * bb].x, w4[2 * bb].y, w4[2 * bb].z, w4[2 * bb].w,
                                        w4[2 * bb + 1].x, w4[2 * bb + 1].y, w4[2 * bb + 1].z, w4[2 * bb + 1].w};
                uint32_t out[32];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    out[4 * i + 0] = tg_mul2<XT>(tg_lut(__byte_perm(wv[i], lane_word, 0x7604)), s2);
                    out[4 * i + 1] = tg_mul2<XT>(tg_lut(__byte_perm(wv[i], lane_word, 0x7614)), s2);
                    out[4 * i + 2] = tg_mul2<XT>(tg_lut(__byte_perm(wv[i], lane_word, 0x7624)), s2);
                    out[4 * i + 3] = tg_mul2<XT>(tg_lut(__byte_perm(wv[i], lane_word, 0x7634)), s2);
                }
                if (bb == 0) {
                    // the A tile is free once the MMAs that read it three stages ago have completed
                    if (!mbar_wait_sleep(aempty_bar(abuf), aph ^ 1u, abort_flag, kSleepFast)) { atomicExch(&g_tc_status, 409); *abort_flag = 1; ok = false; break; }
                    tc_fence_after();
                }
                tmem_st_32x32(tmem_mine + (uint32_t)(abuf * 128 + 32 * bb), out);
            }
            if (!ok) break;
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(afull_bar(abuf)); mbar_arrive(xempty_bar(xslot)); }
#pragma unroll
            for (int e = 0; e < TG_EGROUPS; ++e) {
                if (++slot == nslots) { slot = 0; ph ^= 1u; }
                if (++xslot == TG_NXS) { xslot = 0; xph ^= 1u; }
                if (++abuf == TG_ABUFS) { abuf = 0; aph ^= 1u; }
            }
        }
    }
    // After a time-out the roles leave early while copies or MMAs may still be in flight: give them a
    // bounded moment before the tensor memory is released and the CTA retires.
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 400000ll) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == TG_WARP_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TG_TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*TcEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static TcEncodeTiledFn tc_encode_tiled() {
    static TcEncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<TcEncodeTiledFn>(p);
    }
    return fn;
}

struct TcHostLinear {
    const void *x; int64_t x_ld; int64_t x_period; const uint8_t *packed; const void *absmax; const float *absmax2;
    const void *bias; void *y; float *acc; int64_t N, K;
};

static int tc_fill_linear(TcLinear &L, const TcHostLinear &h, int y_dtype) {
    if (h.N <= 0 || h.K <= 0 || h.N > 0x7fffffff || h.K > 0x7fffffff) return MPSBNB_ERR_INVALID_ARG;
    if (h.x == nullptr || h.packed == nullptr || h.absmax == nullptr || (h.y == nullptr && h.acc == nullptr)) return MPSBNB_ERR_INVALID_ARG;
    if (!aligned16(h.packed)) return MPSBNB_ERR_INVALID_ARG;
    TcEncodeTiledFn fn = tc_encode_tiled();
    if (fn == nullptr) return MPSBNB_ERR_NO_DEVICE;
    const int64_t Kp = padded_k(h.K, 64);
    const int64_t row_bytes = Kp / 2;
    const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)h.N};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {128u, (cuuint32_t)TG_ROWS};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult cr = fn(&L.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(h.packed), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return MPSBNB_ERR_INVALID_ARG;
    L.x = h.x; L.absmax = h.absmax; L.absmax2 = h.absmax2; L.bias = h.bias; L.y = h.y; L.acc = h.acc;
    L.ws = nullptr; L.cnt = nullptr;
    L.x_ld = h.x_ld;
    L.N = (int)h.N; L.K = (int)h.K; L.nb = (int)(Kp / 64);
    L.x_period = (int)(h.x_period > 0 ? h.x_period : h.K);
    L.y_dtype = y_dtype;
    L.x_vec_ok = (h.x_ld % 8 == 0) && (L.x_period % 8 == 0) && (h.K % 8 == 0) && aligned16(h.x);
    L.scale_async = (L.nb % 4 == 0) && ((reinterpret_cast<uintptr_t>(h.absmax) & 15) == 0) &&
                    (h.absmax2 == nullptr || (reinterpret_cast<uintptr_t>(h.absmax2) & 3) == 0);
    L.pad1 = 0;
    return MPSBNB_OK;
}

template <typename XT, int NB>
static int tc_launch_nb(TcArgs &args, int grid, cudaStream_t st, bool pdl) {
    args.zero = 0u;
    static int configured[64] = {};
    int dev = 0;
    MPSBNB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        MPSBNB_CUDA_TRY(cudaFuncSetAttribute(mpsbnb_decode4_tmem_kernel<XT, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, TG_SMEM_BYTES));
        if (dev >= 0 && dev < 64) configured[dev] = 1;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(TG_THREADS); cfg.dynamicSmemBytes = (size_t)TG_SMEM_BYTES; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    MPSBNB_CUDA_TRY(cudaLaunchKernelEx(&cfg, mpsbnb_decode4_tmem_kernel<XT, NB>, args));
    return check_launch();
}
// batch <= 16 runs the 16-column instance (half the x tile, more weight slots), 17 .. 32 the 32-column one
template <typename XT>
static int tc_launch(TcArgs &args, int grid, cudaStream_t st, bool pdl) {
    return args.M <= 16 ? tc_launch_nb<XT, 16>(args, grid, st, pdl) : tc_launch_nb<XT, 32>(args, grid, st, pdl);
}

int tc_status_fetch(int *out, bool reset) {
    MPSBNB_CUDA_TRY(cudaMemcpyFromSymbol(out, g_tc_status, sizeof(int)));
    if (reset) {
        const int zero = 0;
        MPSBNB_CUDA_TRY(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)));
    }
    return MPSBNB_OK;
}

// Single linear, M <= 8: whole row tiles, dealt round-robin to the CTAs (no workspace, so no tile is cut).
int gemv4_tc_single(const void *x, int x_dtype, int64_t M, const uint8_t *packed, const void *absmax,
                    const float *absmax2, int64_t N, int64_t K, int quant_type, const void *bias, void *y,
                    int y_dtype, cudaStream_t st) {
    TcArgs args;
    memset(&args, 0, sizeof(args));
    TcHostLinear h{x, K, K, packed, absmax, absmax2, bias, y, nullptr, N, K};
    int rc = tc_fill_linear(args.one, h, y_dtype);
    if (rc != MPSBNB_OK) return rc;
    args.npieces = (int)((N + TG_ROWS - 1) / TG_ROWS);
    args.M = (int)M; args.quant_type = quant_type;
    int grid = sm_count();
    if (grid > args.npieces) grid = args.npieces;
    return x_dtype == MPSBNB_F16 ? tc_launch<__half>(args, grid, st, false) : tc_launch<__nv_bfloat16>(args, grid, st, false);
}

// ---- grouped launches.  Plan memory (caller-allocated): [TcLinear x n][TcPiece x npieces][int x (grid + 1)]
// [per linear with a y output: fp32 workspace M_max x N, then 4 counters per tile], everything 256-byte aligned.
static inline size_t tc_align(size_t v, size_t a) { return (v + a - 1) / a * a; }
static inline int64_t tc_stages(int64_t K) { return (padded_k(K, 64) / 64 + TG_STAGE_BLOCKS - 1) / TG_STAGE_BLOCKS; }
static inline int64_t tc_tiles(int64_t N) { return (N + TG_ROWS - 1) / TG_ROWS; }

static int64_t tc_max_pieces(const mpsbnb_linear4_desc *d, int n, int grid) {
    int64_t tiles = 0;
    for (int i = 0; i < n; ++i) tiles += tc_tiles(d[i].N);
    return tiles + grid;                                       // every CTA boundary cuts at most one tile
}

size_t tc_plan_bytes(const mpsbnb_linear4_desc *descs, int n_linears) {
    const int grid = sm_count();
    if (grid <= 0) return 0;
    size_t need = tc_align(sizeof(TcLinear) * (size_t)n_linears, 256);
    need += tc_align(sizeof(TcPiece) * (size_t)tc_max_pieces(descs, n_linears, grid), 256);
    need += tc_align(sizeof(int) * (size_t)(grid + 1), 256);
    for (int i = 0; i < n_linears; ++i)
        if (descs[i].acc == nullptr)
            need += tc_align(sizeof(float) * (size_t)TG_MAX_M * (size_t)descs[i].N, 256) + tc_align(sizeof(int) * 4 * (size_t)tc_tiles(descs[i].N), 256);
    return need;
}

int tc_plan(const mpsbnb_linear4_desc *descs, int n_linears, int64_t M, int x_dtype, int y_dtype, int quant_type,
            void *plan_dev, size_t plan_bytes, mpsbnb_group_plan *plan_out, cudaStream_t st) {
    const int grid_max = sm_count();
    if (grid_max <= 0) return MPSBNB_ERR_NO_DEVICE;
    const size_t need = tc_plan_bytes(descs, n_linears);
    if (plan_bytes < need) return MPSBNB_ERR_WORKSPACE;
    const size_t lin_bytes = tc_align(sizeof(TcLinear) * (size_t)n_linears, 256);
    const size_t piece_bytes = tc_align(sizeof(TcPiece) * (size_t)tc_max_pieces(descs, n_linears, grid_max), 256);
    const size_t first_bytes = tc_align(sizeof(int) * (size_t)(grid_max + 1), 256);
    unsigned char *host = (unsigned char *)malloc(need);
    if (host == nullptr) return MPSBNB_ERR_INVALID_ARG;
    memset(host, 0, need);                                     // workspaces and counters start as zeros
    TcLinear *lins = reinterpret_cast<TcLinear *>(host);
    TcPiece *pieces = reinterpret_cast<TcPiece *>(host + lin_bytes);
    int *first = reinterpret_cast<int *>(host + lin_bytes + piece_bytes);
    int rc = MPSBNB_OK;
    size_t off = lin_bytes + piece_bytes + first_bytes;
    int64_t total = 0;
    for (int i = 0; i < n_linears && rc == MPSBNB_OK; ++i) {
        TcHostLinear h{descs[i].x, descs[i].x_ld, descs[i].x_period, descs[i].packed, descs[i].absmax, descs[i].absmax2,
                       descs[i].bias, descs[i].y, descs[i].acc, descs[i].N, descs[i].K};
        rc = tc_fill_linear(lins[i], h, y_dtype);
        if (rc != MPSBNB_OK) break;
        if (descs[i].acc == nullptr) {
            lins[i].ws = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(plan_dev) + off);
            off += tc_align(sizeof(float) * (size_t)TG_MAX_M * (size_t)descs[i].N, 256);
            lins[i].cnt = reinterpret_cast<int *>(reinterpret_cast<unsigned char *>(plan_dev) + off);
            off += tc_align(sizeof(int) * 4 * (size_t)tc_tiles(descs[i].N), 256);
        }
        total += tc_tiles(descs[i].N) * tc_stages(descs[i].K);
    }
    int npieces = 0, grid = 0;
    if (rc == MPSBNB_OK) {
        if (total <= 0 || total > 0x7fffffff) rc = MPSBNB_ERR_INVALID_ARG;
    }
    if (rc == MPSBNB_OK) {
        // the stage sequence (linear by linear, tile by tile) is cut into `grid` equal contiguous ranges
        grid = (int)(total < grid_max ? total : grid_max);
        int c = 0;                                             // CTA that owns the stage being placed
        int64_t q = 0;                                         // stages placed so far
        first[0] = 0;
        auto range_end = [&](int cta) { return (total * (int64_t)(cta + 1)) / grid; };
        for (int i = 0; i < n_linears; ++i) {
            const int S = (int)tc_stages(descs[i].K);
            for (int64_t t = 0; t < tc_tiles(descs[i].N); ++t) {
                int s = 0, parts = 0;
                const int first_piece = npieces;
                while (s < S) {
                    while (q >= range_end(c)) { ++c; first[c] = npieces; }
                    const int64_t room = range_end(c) - q;
                    const int len = (int)((int64_t)(S - s) < room ? (S - s) : room);
                    pieces[npieces++] = TcPiece{i, (int)(t * TG_ROWS), s, s + len, 0, 0, 0, 0};
                    s += len; q += len; ++parts;
                }
                for (int k = first_piece; k < npieces; ++k) pieces[k].parts = parts;
            }
        }
        while (c < grid) { ++c; first[c] = npieces; }
    }
    if (rc == MPSBNB_OK) {
        cudaError_t e = cudaMemcpyAsync(plan_dev, host, need, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) rc = record_cuda_error(e);
    }
    free(host);
    if (rc != MPSBNB_OK) return rc;
    plan_out->dev = plan_dev;
    plan_out->units_offset = (int64_t)lin_bytes;
    plan_out->n_linears = n_linears;
    plan_out->n_units = npieces;
    plan_out->M = (int)M;
    plan_out->x_dtype = x_dtype;
    plan_out->quant_type = quant_type;
    plan_out->flags = 0;
    plan_out->aux_offset = (int64_t)(lin_bytes + piece_bytes);
    plan_out->grid = grid;
    plan_out->impl = 1;
    plan_out->wait_flags = nullptr; plan_out->wait_step = nullptr;
    plan_out->wait_n = plan_out->wait_mul = plan_out->wait_add = plan_out->acc_parts = 0;
    plan_out->n_segments = 1; plan_out->wait_seg_mul = 0;
    memset(&plan_out->ep, 0, sizeof(plan_out->ep));
    return MPSBNB_OK;
}

int tc_run(const mpsbnb_group_plan *plan, cudaStream_t st) {
    TcArgs args;
    memset(&args, 0, sizeof(args));
    const unsigned char *base = reinterpret_cast<const unsigned char *>(plan->dev);
    args.lins = reinterpret_cast<const TcLinear *>(base);
    args.pieces = reinterpret_cast<const TcPiece *>(base + plan->units_offset);
    args.cta_first = reinterpret_cast<const int *>(base + plan->aux_offset);
    args.npieces = plan->n_units; args.M = plan->M; args.quant_type = plan->quant_type;
    const bool pdl = (plan->flags & MPSBNB_GROUP_PDL) != 0;
    return plan->x_dtype == MPSBNB_F16 ? tc_launch<__half>(args, plan->grid, st, pdl)
                                       : tc_launch<__nv_bfloat16>(args, plan->grid, st, pdl);
}

}  // namespace mpsbnb
