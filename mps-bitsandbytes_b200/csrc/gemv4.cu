// Decode-shape fused dequantise-GEMV for 4-bit (NF4 / FP4) weights, block size 64:
//     y[m, n] = sum_k x[m, k] * code[W[n, k]] * absmax[n, k / 64]  (+ bias[n]),  M <= 32.
// Stands for mps_bitsandbytes/functional.py:680-773 (matmul_4bit) on decode shapes and for
// the reference's Metal kernel nf4_matmul_simd (mps_bitsandbytes.mm:440-560).
//
// The kernel is bound by HBM: every packed byte is read exactly once, straight into
// registers, and never staged.  What it has to avoid is becoming bound by instruction issue
// or shared-memory bandwidth instead: at HBM speed one SM must expand ~50 weights per clock.
//   * One warp works on 16 weight rows x 64 k (one quantisation block per row) at a time.
//     Lane (g, t) (g = lane / 4, t = lane % 4) loads 8 bytes of row g and of row g + 8 —
//     the 16 consecutive k that start at 16 t — so a warp request covers whole 32-byte
//     sectors and the eight warps of a CTA together read 256 contiguous bytes of each row.
//   * A packed byte is expanded to two 16-bit values with ONE byte-permute and ONE
//     conflict-free shared-memory read: a table of 256 (lo, hi) pairs, replicated for each of
//     the 32 lanes (entry b of lane l lives at b * 256 + l * 4, so a lane always hits its own
//     bank).  The permute builds that address directly from the weight byte and the lane offset.
//   * The pairs are exactly the A fragments of mma.sync.m16n8k16 (weight rows are the M side
//     of the MMA, the batch is its N side), so the multiply-accumulate costs 1/8 instruction per
//     weight and M up to 8 is free.  The order of k inside an MMA is arbitrary as long as x
//     is fed in the same order; each lane feeds the 16 x values matching its own 16 weights.
//   * absmax is applied once per (row, block) to the fp32 partial sum of that block, not per
//     weight.  The matmul therefore differs from "dequantise to fp16, then GEMM" only by
//     fp16 roundings of the weights (the parity bound for matmuls is 1e-2 relative).
// tcgen05 is not used here: with M <= 32 the tensor pipe is idle either way, and operands of
// tcgen05.mma must sit in shared memory, which would add a store and a load per weight to
// the one resource (shared-memory bandwidth) that is already the tightest.
#include "common.cuh"
#include "ops.cuh"
#include "sm100.cuh"

#include <string.h>

namespace mpsbnb {

struct Gemv4Params {
    const void *x;           // [M, K]
    const uint8_t *packed;   // [N, row_bytes]
    const void *absmax;      // fp32 [N, nb] or int8 [N, nb]
    const float *absmax2;    // nullptr or fp32 [ceil(N*nb/256)]
    const void *bias;        // nullptr or [N] in x dtype
    void *y;                 // [M, N]
    int M, N, K;
    int nb;                  // blocks per row in the layout (Kp / 64)
    int64_t row_bytes;       // Kp / 2
    int y_dtype;
    int quant_type;
    int x_vec_ok;            // x rows 16-byte aligned (K % 8 == 0 and base aligned)
};

constexpr int kWarps = 8;
constexpr int kLutBytes = 65536;

__device__ __forceinline__ uint2 ldg_stream_v2(const uint8_t *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, __half) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, __nv_bfloat16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename XT> __device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// x[m, k0 .. k0+16) as 8 packed pairs; zero outside [0, K) and for m >= M.
template <typename XT>
__device__ __forceinline__ void load_x16(const XT *__restrict__ x, int m, int M, int64_t k0, int K, bool vec_ok,
                                         uint32_t (&out)[8]) {
    if (m >= M || k0 >= K) {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = 0u;
        return;
    }
    const XT *row = x + (int64_t)m * K;
    if (vec_ok && k0 + 16 <= K) {
        const uint4 a = __ldg(reinterpret_cast<const uint4 *>(row + k0));
        const uint4 b = __ldg(reinterpret_cast<const uint4 *>(row + k0 + 8));
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
        out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
        return;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t k = k0 + 2 * i;
        const uint16_t lo = k < K ? *reinterpret_cast<const uint16_t *>(row + k) : (uint16_t)0;
        const uint16_t hi = k + 1 < K ? *reinterpret_cast<const uint16_t *>(row + k + 1) : (uint16_t)0;
        out[i] = (uint32_t)lo | ((uint32_t)hi << 16);
    }
}

template <typename T> __device__ __forceinline__ void store_out(void *y, int y_dtype, int64_t i, float v) {
    if (y_dtype == MPSBNB_F16) reinterpret_cast<__half *>(y)[i] = __float2half_rn(v);
    else if (y_dtype == MPSBNB_BF16) reinterpret_cast<__nv_bfloat16 *>(y)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float *>(y)[i] = v;
}

// XT: x / MMA operand type.  MT: number of 8-wide batch tiles (M <= 8 MT).  R: 16-row tiles
// per CTA pass (the x fragments of a block are reused for all R tiles).
template <typename XT, int MT, int R>
__global__ void __launch_bounds__(kWarps * 32, 2) mpsbnb_decode4_direct_kernel(const Gemv4Params p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    constexpr int ROWS = 16 * R;
    constexpr int RED_STRIDE = ROWS + 4;                    // conflict-free accumulator dump
    float *red = reinterpret_cast<float *>(smem + kLutBytes);   // [kWarps][8 MT][RED_STRIDE]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // lane-replicated byte -> (code[lo nibble], code[hi nibble]) table.  Warp w fills bytes
    // 32 w .. 32 w + 31: lane l computes the pair of byte 32 w + l once, and in round j every lane
    // stores byte (32 w + j)'s pair into its own replica (consecutive lanes, consecutive banks).
    {
        const float my_code = kCode[p.quant_type][lane & 15];
        const int byte = warp * 32 + lane;
        const float lo = __shfl_sync(0xffffffffu, my_code, byte & 15);
        const float hi = __shfl_sync(0xffffffffu, my_code, byte >> 4);
        const uint32_t mine = pack_pair<XT>(lo, hi);
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {
            const uint32_t v = __shfl_sync(0xffffffffu, mine, j);
            *reinterpret_cast<uint32_t *>(smem + (warp * 32 + j) * 256 + lane * 4) = v;
        }
    }
    __syncthreads();

    const XT *x = reinterpret_cast<const XT *>(p.x);
    const uint32_t lane4 = (uint32_t)lane * 4u;
    const int nbv = (p.K + 63) >> 6;                        // blocks that hold real k
    const int ntiles = (p.N + ROWS - 1) / ROWS;
    const bool dq = p.absmax2 != nullptr;
    const float *am_f = reinterpret_cast<const float *>(p.absmax);
    const int8_t *am_q = reinterpret_cast<const int8_t *>(p.absmax);

    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int row0 = tile * ROWS;
        int64_t rown[2 * R];                                // clamped row index of slot r*2+h
#pragma unroll
        for (int s = 0; s < 2 * R; ++s) {
            int rr = row0 + 16 * (s >> 1) + 8 * (s & 1) + g;
            rown[s] = rr < p.N ? rr : p.N - 1;
        }
        float acc[R][MT][4];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[r][mt][c] = 0.0f;

        const int iters = nbv > warp ? (nbv - warp + kWarps - 1) / kWarps : 0;
        constexpr int P = 4;                                // weight prefetch depth (iterations)
        uint2 wq[P][2 * R];
        float aq[2][2 * R];
        uint32_t xq[2][MT][8];

        auto load_w = [&](int it, uint2 (&dst)[2 * R]) {
            const int64_t off = (int64_t)(warp + it * kWarps) * 32 + t * 8;
#pragma unroll
            for (int s = 0; s < 2 * R; ++s) dst[s] = ldg_stream_v2(p.packed + rown[s] * p.row_bytes + off);
        };
        auto load_ax = [&](int it, float (&a)[2 * R], uint32_t (&xv)[MT][8]) {
            const int b = warp + it * kWarps;
#pragma unroll
            for (int s = 0; s < 2 * R; ++s) {
                const int64_t i = rown[s] * p.nb + b;
                if (dq) a[s] = (float)__ldg(am_q + i) * (__ldg(p.absmax2 + (i >> 8)) * (1.0f / 127.0f));
                else a[s] = __ldg(am_f + i);
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                load_x16<XT>(x, 8 * mt + g, p.M, (int64_t)b * 64 + t * 16, p.K, p.x_vec_ok != 0, xv[mt]);
        };

#pragma unroll
        for (int pp = 0; pp < P; ++pp)
            if (pp < iters) load_w(pp, wq[pp]);
        if (iters > 0) load_ax(0, aq[0], xq[0]);

        for (int it0 = 0; it0 < iters; it0 += P) {
#pragma unroll
            for (int pp = 0; pp < P; ++pp) {
                const int it = it0 + pp;
                if (it < iters) {
                    uint2 w[2 * R];
#pragma unroll
                    for (int s = 0; s < 2 * R; ++s) w[s] = wq[pp][s];
                    if (it + P < iters) load_w(it + P, wq[pp]);
                    const int cur = pp & 1;                 // P is even, so parity of it == parity of pp
                    if (it + 1 < iters) load_ax(it + 1, aq[cur ^ 1], xq[cur ^ 1]);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        float tmp[MT][4];
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                            for (int c = 0; c < 4; ++c) tmp[mt][c] = 0.0f;
#pragma unroll
                        for (int s = 0; s < 4; ++s) {
                            // bytes 2s, 2s+1 of each 8-byte group: word s>>1, byte pair (s&1)*2
                            const uint32_t w0 = (s < 2) ? w[2 * r].x : w[2 * r].y;       // row g
                            const uint32_t w1 = (s < 2) ? w[2 * r + 1].x : w[2 * r + 1].y; // row g+8
                            const uint32_t selA = (s & 1) ? 0x7624u : 0x7604u;
                            const uint32_t selB = (s & 1) ? 0x7634u : 0x7614u;
                            const uint32_t a0 = *reinterpret_cast<const uint32_t *>(smem + __byte_perm(w0, lane4, selA));
                            const uint32_t a1 = *reinterpret_cast<const uint32_t *>(smem + __byte_perm(w1, lane4, selA));
                            const uint32_t a2 = *reinterpret_cast<const uint32_t *>(smem + __byte_perm(w0, lane4, selB));
                            const uint32_t a3 = *reinterpret_cast<const uint32_t *>(smem + __byte_perm(w1, lane4, selB));
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt)
                                mma16816(tmp[mt], a0, a1, a2, a3, xq[cur][mt][2 * s], xq[cur][mt][2 * s + 1], XT());
                        }
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            acc[r][mt][0] = fmaf(aq[cur][2 * r], tmp[mt][0], acc[r][mt][0]);
                            acc[r][mt][1] = fmaf(aq[cur][2 * r], tmp[mt][1], acc[r][mt][1]);
                            acc[r][mt][2] = fmaf(aq[cur][2 * r + 1], tmp[mt][2], acc[r][mt][2]);
                            acc[r][mt][3] = fmaf(aq[cur][2 * r + 1], tmp[mt][3], acc[r][mt][3]);
                        }
                    }
                }
            }
        }

        // cross-warp reduction: red[warp][m][row]
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int m = 8 * mt + 2 * t + (c & 1);
                    const int nl = 16 * r + g + 8 * (c >> 1);
                    red[(warp * 8 * MT + m) * RED_STRIDE + nl] = acc[r][mt][c];
                }
        __syncthreads();
        for (int o = tid; o < p.M * ROWS; o += kWarps * 32) {
            const int m = o / ROWS, nl = o - m * ROWS;
            const int n = row0 + nl;
            if (n < p.N) {
                float s = 0.0f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) s += red[(w * 8 * MT + m) * RED_STRIDE + nl];
                if (p.bias != nullptr) s += to_f32<XT>(reinterpret_cast<const XT *>(p.bias)[n]);
                store_out<XT>(p.y, p.y_dtype, (int64_t)m * p.N + n, s);
            }
        }
        __syncthreads();
    }
}

template <typename XT, int MT, int R>
static int launch_gemv4(const Gemv4Params &p, cudaStream_t st) {
    constexpr int ROWS = 16 * R;
    const size_t smem = kLutBytes + (size_t)kWarps * 8 * MT * (ROWS + 4) * sizeof(float);
    static bool configured[64] = {};                        // per device: the attribute lives in the context
    int dev = 0;
    MPSBNB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        MPSBNB_CUDA_TRY(cudaFuncSetAttribute(mpsbnb_decode4_direct_kernel<XT, MT, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int ntiles = (p.N + ROWS - 1) / ROWS;
    int grid = sm_count() * 2;
    if (grid > ntiles) grid = ntiles;
    mpsbnb_decode4_direct_kernel<XT, MT, R><<<grid, kWarps * 32, smem, st>>>(p);
    return check_launch();
}

template <typename XT>
static int dispatch_gemv4(const Gemv4Params &p, cudaStream_t st) {
    // few rows per CTA when N is small, so that every SM gets work
    const bool small_n = p.N < 32 * 2 * sm_count();
    if (p.M <= 8) return small_n ? launch_gemv4<XT, 1, 1>(p, st) : launch_gemv4<XT, 1, 2>(p, st);
    if (p.M <= 16) return small_n ? launch_gemv4<XT, 2, 1>(p, st) : launch_gemv4<XT, 2, 2>(p, st);
    if (p.M <= 24) return launch_gemv4<XT, 3, 1>(p, st);
    return launch_gemv4<XT, 4, 1>(p, st);
}

// Layer boundary of the synthetic decoder-layer stack: h[m, j] = alpha * (o[m, j] + d[m, j]),
// and e[m, j] = h[m, j mod H] for j < F (the F-wide input of the next layer's down projection).
template <typename T>
__global__ void stack_boundary_kernel(const T *__restrict__ o, const T *__restrict__ d, float alpha, int M, int H, int F,
                                      T *__restrict__ h, T *__restrict__ e) {
    const int64_t total = (int64_t)M * F;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / F), j = (int)(i - (int64_t)m * F);
        const int c = j % H;
        const T v = from_f32<T>(alpha * (to_f32<T>(o[(int64_t)m * H + c]) + to_f32<T>(d[(int64_t)m * H + c])));
        if (j < H) h[(int64_t)m * H + j] = v;
        if (e != nullptr) e[i] = v;
    }
}

// After an all-gather of per-rank shards G[r][m][c] (c < H / g): h[m, r * H/g + c] = G[r][m][c],
// and e[m, j] = h[m, j mod H].
template <typename T>
__global__ void stack_expand_kernel(const T *__restrict__ G, int g, int M, int H, int F, T *__restrict__ h,
                                    T *__restrict__ e) {
    const int Hs = H / g;
    const int64_t total = (int64_t)M * F;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / F), j = (int)(i - (int64_t)m * F);
        const int c = j % H;
        const T v = G[((int64_t)(c / Hs) * M + m) * Hs + (c % Hs)];
        if (j < H) h[(int64_t)m * H + j] = v;
        if (e != nullptr) e[i] = v;
    }
}

// h[i] = alpha * acc[i] (rounded to T), then acc[i] = 0: closes a layer whose o and down
// projections were accumulated into one fp32 matrix, and re-arms the accumulator.
template <typename T>
__global__ void stack_boundary_acc_kernel(float *__restrict__ acc, float alpha, int64_t n, T *__restrict__ h) {
    sm100::pdl_launch_dependents();
    sm100::pdl_grid_dependency_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        h[i] = from_f32<T>(alpha * acc[i]);
        acc[i] = 0.0f;
    }
}

}  // namespace mpsbnb

using namespace mpsbnb;

extern "C" int mpsbnb_stack_boundary_acc(float *acc, float alpha, int64_t n, void *h, int dtype, int flags,
                                         void *stream) {
    if (!is_16bit(dtype) || n < 0) return MPSBNB_ERR_INVALID_ARG;
    if (n == 0) return MPSBNB_OK;
    if (acc == nullptr || h == nullptr) return MPSBNB_ERR_INVALID_ARG;
    int64_t grid = (n + 255) / 256;
    if (grid > sm_count() * 8) grid = sm_count() * 8;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(256); cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = (flags & MPSBNB_GROUP_PDL) ? 1 : 0;
    if (dtype == MPSBNB_F16)
        MPSBNB_CUDA_TRY(cudaLaunchKernelEx(&cfg, stack_boundary_acc_kernel<__half>, acc, alpha, n, (__half *)h));
    else
        MPSBNB_CUDA_TRY(cudaLaunchKernelEx(&cfg, stack_boundary_acc_kernel<__nv_bfloat16>, acc, alpha, n, (__nv_bfloat16 *)h));
    return check_launch();
}

extern "C" int mpsbnb_stack_expand(const void *G, int dtype, int64_t nranks, int64_t M, int64_t H, int64_t F, void *h,
                                   void *e, void *stream) {
    if (!is_16bit(dtype) || M < 0 || H <= 0 || F < H || nranks <= 0 || H % nranks != 0) return MPSBNB_ERR_INVALID_ARG;
    if (M == 0) return MPSBNB_OK;
    if (G == nullptr || h == nullptr) return MPSBNB_ERR_INVALID_ARG;
    int64_t grid = (M * F + 255) / 256;
    if (grid > sm_count() * 8) grid = sm_count() * 8;
    stack_expand_kernel<uint16_t><<<(int)grid, 256, 0, (cudaStream_t)stream>>>(
        (const uint16_t *)G, (int)nranks, (int)M, (int)H, (int)F, (uint16_t *)h, (uint16_t *)e);
    return check_launch();
}

extern "C" int mpsbnb_stack_boundary(const void *o, const void *d, int dtype, float alpha, int64_t M, int64_t H,
                                     int64_t F, void *h, void *e, void *stream) {
    if (!is_16bit(dtype) || M < 0 || H <= 0 || F < H) return MPSBNB_ERR_INVALID_ARG;
    if (M == 0) return MPSBNB_OK;
    if (o == nullptr || d == nullptr || h == nullptr) return MPSBNB_ERR_INVALID_ARG;
    const int64_t total = M * F;
    int64_t grid = (total + 255) / 256;
    if (grid > sm_count() * 8) grid = sm_count() * 8;
    if (dtype == MPSBNB_F16)
        stack_boundary_kernel<__half><<<(int)grid, 256, 0, (cudaStream_t)stream>>>(
            (const __half *)o, (const __half *)d, alpha, (int)M, (int)H, (int)F, (__half *)h, (__half *)e);
    else
        stack_boundary_kernel<__nv_bfloat16><<<(int)grid, 256, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16 *)o, (const __nv_bfloat16 *)d, alpha, (int)M, (int)H, (int)F, (__nv_bfloat16 *)h,
            (__nv_bfloat16 *)e);
    return check_launch();
}

extern "C" int mpsbnb_gemv_4bit_max_m(void) { return 32; }

extern "C" int mpsbnb_gemv_4bit(const void *x, int x_dtype, int64_t M, const uint8_t *packed, const void *absmax,
                                const float *absmax2, int64_t N, int64_t K, int blocksize, int quant_type,
                                const void *bias, void *y, int y_dtype, void *stream) {
    if (!is_16bit(x_dtype) || !valid_dtype(y_dtype)) return MPSBNB_ERR_INVALID_ARG;
    if (quant_type != MPSBNB_NF4 && quant_type != MPSBNB_FP4) return MPSBNB_ERR_INVALID_ARG;
    if (M < 0 || N < 0 || K < 0) return MPSBNB_ERR_INVALID_ARG;
    if (blocksize != 64 || M > 32) return MPSBNB_ERR_UNSUPPORTED;
    if (N > 0x7fffffff || K > 0x7fffffff) return MPSBNB_ERR_TOO_LARGE;
    if (M == 0 || N == 0) return MPSBNB_OK;
    if (x == nullptr || packed == nullptr || absmax == nullptr || y == nullptr) return MPSBNB_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(packed) & 7) != 0) return MPSBNB_ERR_INVALID_ARG;
    Gemv4Params p;
    p.x = x; p.packed = packed; p.absmax = absmax; p.absmax2 = absmax2; p.bias = bias; p.y = y;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    const int64_t Kp = padded_k(K, 64);
    p.nb = (int)(Kp / 64);
    p.row_bytes = Kp / 2;
    p.y_dtype = y_dtype;
    p.quant_type = quant_type;
    p.x_vec_ok = (K % 8 == 0) && aligned16(x);
    if (K == 0) {                                           // empty contraction: y = bias
        p.K = 0;
    }
    cudaStream_t st = (cudaStream_t)stream;
    // batch 9 .. 32 takes the tensor-memory kernel (1.6 - 1.9 TB/s against 1.0 - 1.4 for the direct-load kernel below)
    if (M > 8 && M <= 32 && K > 0 && aligned16(packed))       // TMA ring + tcgen05
        return gemv4_tc_single(x, x_dtype, M, packed, absmax, absmax2, N, K, quant_type, bias, y, y_dtype, st);
    if (M <= 8 && K > 0 && aligned16(packed))                  // TMA ring + mma.sync
        return gemv4_stream_single(x, x_dtype, M, packed, absmax, absmax2, N, K, quant_type, bias, y, y_dtype, st);
    return x_dtype == MPSBNB_F16 ? dispatch_gemv4<__half>(p, st) : dispatch_gemv4<__nv_bfloat16>(p, st);
}
