// Layer-boundary exchange of the N-sharded layer stack without a collective library call.
//
// Every rank (one process per GPU) owns [M, H / g] columns of the next layer's input h.  Instead of
// "write shard -> NCCL all-gather -> re-lay", the boundary kernel converts its shard and STORES it
// straight into every rank's h buffer over NVLink (plain peer stores into memory opened with CUDA IPC),
// then raises a flag on every rank; the next layer's GEMV waits for the g flags before it reads x.
// Flags only grow: the boundary of (step s, layer l) writes s * L + l + 1, the GEMV of (step s, layer l)
// waits for >= s * L + l, so nothing is ever reset and a CUDA graph can replay the step (s lives in device
// memory and is advanced by mpsbnb_counter_add inside the graph).  h is double-buffered by layer parity:
// a rank can be at most one layer ahead of its slowest peer, so the buffer it stores into is never the
// one a peer is still reading.
//
// All waits are bounded (about a second); a wait that runs out records status 501 / 502 and returns,
// the context stays usable.  No multicast, no cluster-wide TMA: ordinary st.global to peer addresses.
#include "common.cuh"
#include "sm100.cuh"

#include <string.h>

namespace mpsbnb {

static __device__ int g_xchg_status = 0;

__device__ __forceinline__ int ld_acquire_sys(const int *p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int *p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Polls flags[lane] (lane < n) until it reaches `expect` or ~1 s has passed.  Whole-warp call.
__device__ __forceinline__ bool wait_flags_warp(const int *flags, int n, int expect, int lane) {
    bool ok = true;
    if (lane < n) {
        const long long t0 = clock64();
        while (ld_acquire_sys(flags + lane) < expect) {
            __nanosleep(64);
            if (clock64() - t0 > 2000000000ll) { ok = false; break; }
        }
    }
    return __all_sync(0xffffffffu, ok);
}

// One CTA.  h_shard = alpha * acc (rounded to T) goes to columns [rank * hs, (rank + 1) * hs) of every rank's
// h; acc is re-armed; then flag[rank] on every rank becomes (*step) * mul + add.
template <typename T>
__global__ void __launch_bounds__(1024, 1)
stack_boundary_push_kernel(float *__restrict__ acc, float alpha, int M, int hs, int H, int rank, int nranks,
                           T *const *__restrict__ peer_h, int *const *__restrict__ peer_flags, const int *step, int mul,
                           int add) {
    sm100::pdl_launch_dependents();
    sm100::pdl_grid_dependency_wait();                               // acc is complete when the GEMV grid has finished
    const int total = M * hs;                                        // hs is a multiple of 8
    for (int i = (int)threadIdx.x * 8; i < total; i += (int)blockDim.x * 8) {
        const int m = i / hs, c = i - m * hs;
        float4 a0 = *reinterpret_cast<const float4 *>(acc + i), a1 = *reinterpret_cast<const float4 *>(acc + i + 4);
        *reinterpret_cast<float4 *>(acc + i) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4 *>(acc + i + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
        T v[8] = {from_f32<T>(alpha * a0.x), from_f32<T>(alpha * a0.y), from_f32<T>(alpha * a0.z), from_f32<T>(alpha * a0.w),
                  from_f32<T>(alpha * a1.x), from_f32<T>(alpha * a1.y), from_f32<T>(alpha * a1.z), from_f32<T>(alpha * a1.w)};
        const uint4 bits = *reinterpret_cast<const uint4 *>(v);
        const int64_t o = (int64_t)m * H + (int64_t)rank * hs + c;
        for (int r = 0; r < nranks; ++r) *reinterpret_cast<uint4 *>(peer_h[r] + o) = bits;
    }
    __threadfence_system();                                          // my stores before anything that follows the barrier
    __syncthreads();
    if ((int)threadIdx.x < nranks) st_release_sys(peer_flags[threadIdx.x] + rank, (*step) * mul + add);
}

__global__ void flags_wait_kernel(const int *flags, int n, const int *step, int mul, int add) {
    sm100::pdl_launch_dependents();
    sm100::pdl_grid_dependency_wait();
    if (!wait_flags_warp(flags, n, (*step) * mul + add, (int)threadIdx.x) && threadIdx.x == 0) atomicExch(&g_xchg_status, 502);
}

__global__ void flags_push_kernel(int *const *peer_flags, int rank, int nranks, const int *step, int mul, int add) {
    sm100::pdl_launch_dependents();
    sm100::pdl_grid_dependency_wait();
    __threadfence_system();
    if ((int)threadIdx.x < nranks) st_release_sys(peer_flags[threadIdx.x] + rank, (*step) * mul + add);
}

// Tagged form of a 16-bit matrix [M, H]: entry p of row m = {columns 2 p and 2 p + 1, tag} in 8 bytes (see the closer
// warp of the decode kernel).  ll_write puts a plain matrix into that form with tag (*step) * mul + add.
__global__ void ll_write_kernel(const uint32_t *__restrict__ x, int64_t npairs, unsigned long long *__restrict__ dst,
                                const int *step, int mul, int add) {
    sm100::pdl_launch_dependents();
    sm100::pdl_grid_dependency_wait();
    const unsigned long long tag = (unsigned long long)(uint32_t)((*step) * mul + add) << 32;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < npairs; i += (int64_t)gridDim.x * blockDim.x)
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + i), "l"(tag | x[i]) : "memory");
}

// The reverse, for a matrix that other GPUs are still writing: every entry is read until it carries the expected tag
// (bounded: about a second, then status 502), then its two values are stored.
__global__ void ll_read_kernel(const unsigned long long *__restrict__ src, int64_t npairs, uint32_t *__restrict__ out,
                               const int *step, int mul, int add) {
    sm100::pdl_launch_dependents();
    sm100::pdl_grid_dependency_wait();
    const uint32_t expect = (uint32_t)((*step) * mul + add);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < npairs; i += (int64_t)gridDim.x * blockDim.x) {
        unsigned long long v;
        const long long t0 = clock64();
        for (;;) {
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(src + i) : "memory");
            if ((uint32_t)(v >> 32) == expect) break;
            if (clock64() - t0 > 2000000000ll) { atomicExch(&g_xchg_status, 502); break; }
        }
        out[i] = (uint32_t)v;
    }
}

__global__ void counter_add_kernel(int *ctr, int v) {
    sm100::pdl_launch_dependents();
    sm100::pdl_grid_dependency_wait();
    *ctr += v;
}

int xchg_status_fetch(int *out, bool reset) {
    MPSBNB_CUDA_TRY(cudaMemcpyFromSymbol(out, g_xchg_status, sizeof(int)));
    if (reset) {
        const int zero = 0;
        MPSBNB_CUDA_TRY(cudaMemcpyToSymbol(g_xchg_status, &zero, sizeof(int)));
    }
    return MPSBNB_OK;
}

static void pdl_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *attr, dim3 grid, dim3 block, cudaStream_t st, bool pdl) {
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid; cfg.blockDim = block; cfg.stream = st;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
}

}  // namespace mpsbnb

using namespace mpsbnb;

// ---- CUDA IPC plumbing (no allocation here: the caller's buffer is exported / a peer's buffer is mapped)
extern "C" int mpsbnb_ipc_export(const void *dev_ptr, void *handle64, int64_t *offset_out) {
    if (dev_ptr == nullptr || handle64 == nullptr || offset_out == nullptr) return MPSBNB_ERR_INVALID_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    // the handle names the whole allocation that contains dev_ptr; find its base
    typedef CUresult (*RangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);
    static RangeFn range = nullptr;
    if (range == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            return MPSBNB_ERR_NO_DEVICE;
        range = reinterpret_cast<RangeFn>(p);
    }
    CUdeviceptr base = 0;
    size_t size = 0;
    if (range(&base, &size, reinterpret_cast<CUdeviceptr>(dev_ptr)) != CUDA_SUCCESS) return MPSBNB_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    MPSBNB_CUDA_TRY(cudaIpcGetMemHandle(&h, reinterpret_cast<void *>(base)));
    memcpy(handle64, &h, 64);
    *offset_out = (int64_t)(reinterpret_cast<CUdeviceptr>(dev_ptr) - base);
    return MPSBNB_OK;
}

extern "C" int mpsbnb_ipc_open(const void *handle64, void **base_out) {
    if (handle64 == nullptr || base_out == nullptr) return MPSBNB_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    MPSBNB_CUDA_TRY(cudaIpcOpenMemHandle(base_out, h, cudaIpcMemLazyEnablePeerAccess));
    return MPSBNB_OK;
}

extern "C" int mpsbnb_ipc_close(void *base) {
    if (base == nullptr) return MPSBNB_OK;
    MPSBNB_CUDA_TRY(cudaIpcCloseMemHandle(base));
    return MPSBNB_OK;
}

extern "C" int mpsbnb_stack_boundary_push(float *acc, float alpha, int64_t M, int64_t hs, int64_t H, int rank, int nranks,
                                          void *const *peer_h, int *const *peer_flags, const int *step, int mul, int add,
                                          int dtype, int flags, void *stream) {
    if (!is_16bit(dtype) || M <= 0 || M > 64 || hs <= 0 || hs % 8 != 0 || H < hs * nranks || rank < 0 || rank >= nranks ||
        nranks > 32 || M * hs > (1 << 24))
        return MPSBNB_ERR_INVALID_ARG;
    if (acc == nullptr || peer_h == nullptr || peer_flags == nullptr || step == nullptr) return MPSBNB_ERR_INVALID_ARG;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    pdl_config(cfg, attr, dim3(1), dim3(1024), (cudaStream_t)stream, (flags & MPSBNB_GROUP_PDL) != 0);
    if (dtype == MPSBNB_F16)
        MPSBNB_CUDA_TRY(cudaLaunchKernelEx(&cfg, stack_boundary_push_kernel<__half>, acc, alpha, (int)M, (int)hs, (int)H, rank,
                                           nranks, (__half *const *)peer_h, peer_flags, step, mul, add));
    else
        MPSBNB_CUDA_TRY(cudaLaunchKernelEx(&cfg, stack_boundary_push_kernel<__nv_bfloat16>, acc, alpha, (int)M, (int)hs, (int)H,
                                           rank, nranks, (__nv_bfloat16 *const *)peer_h, peer_flags, step, mul, add));
    return check_launch();
}

extern "C" int mpsbnb_flags_wait(const int *flags, int n, const int *step, int mul, int add, int pdl, void *stream) {
    if (flags == nullptr || step == nullptr || n <= 0 || n > 32) return MPSBNB_ERR_INVALID_ARG;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    pdl_config(cfg, attr, dim3(1), dim3(32), (cudaStream_t)stream, pdl != 0);
    MPSBNB_CUDA_TRY(cudaLaunchKernelEx(&cfg, flags_wait_kernel, flags, n, step, mul, add));
    return check_launch();
}

extern "C" int mpsbnb_flags_push(int *const *peer_flags, int rank, int nranks, const int *step, int mul, int add, void *stream) {
    if (peer_flags == nullptr || step == nullptr || nranks <= 0 || nranks > 32 || rank < 0 || rank >= nranks) return MPSBNB_ERR_INVALID_ARG;
    flags_push_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(peer_flags, rank, nranks, step, mul, add);
    return check_launch();
}

extern "C" int mpsbnb_tagged_write(const void *x, int64_t M, int64_t H, void *tagged, const int *step, int mul, int add, void *stream) {
    if (x == nullptr || tagged == nullptr || step == nullptr || M <= 0 || H <= 0 || H % 2 != 0) return MPSBNB_ERR_INVALID_ARG;
    const int64_t n = M * H / 2;
    ll_write_kernel<<<(unsigned)((n + 255) / 256 < 296 ? (n + 255) / 256 : 296), 256, 0, (cudaStream_t)stream>>>(
        (const uint32_t *)x, n, (unsigned long long *)tagged, step, mul, add);
    return check_launch();
}

extern "C" int mpsbnb_tagged_read(const void *tagged, int64_t M, int64_t H, void *out, const int *step, int mul, int add, void *stream) {
    if (out == nullptr || tagged == nullptr || step == nullptr || M <= 0 || H <= 0 || H % 2 != 0) return MPSBNB_ERR_INVALID_ARG;
    const int64_t n = M * H / 2;
    ll_read_kernel<<<(unsigned)((n + 255) / 256 < 296 ? (n + 255) / 256 : 296), 256, 0, (cudaStream_t)stream>>>(
        (const unsigned long long *)tagged, n, (uint32_t *)out, step, mul, add);
    return check_launch();
}

extern "C" int mpsbnb_counter_add(int *counter, int value, void *stream) {
    if (counter == nullptr) return MPSBNB_ERR_INVALID_ARG;
    counter_add_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(counter, value);
    return check_launch();
}
