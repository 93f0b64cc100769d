// 4-bit GEMM that needs no memory from the caller: the expanded weight (and, when x has to be
// re-pitched, the copy of x) lives in a fixed array that is part of this library's device
// image, so the call neither allocates nor frees anything and needs no workspace argument.
//
// Who this is for: hosts that hand all device memory to their own arena at start-up (serving
// engines that pre-partition HBM into weights + KV cache, language bindings without an
// allocator of their own) and therefore cannot produce the workspace that mpsbnb_gemm_4bit
// asks for.  The price is a fixed size limit and one shared scratch per device.
//
// Rules of use:
//  * The first call on each device looks the array's address up (cudaGetSymbolAddress).  That
//    look-up is set-up work, not a stream operation: make the first call on a device before
//    any stream capture that will contain later calls.
//  * All calls on one device share the one array.  Calls enqueued on the same stream are
//    ordered and safe.  Calls on different streams (or from different threads on different
//    streams) that can overlap in time race on the scratch and give wrong results; order them
//    with events or use mpsbnb_gemm_4bit with separate workspaces.
//  * Nothing in the scratch has to start at zero: every byte a call reads it has written first.
//  * The looked-up address is cached per device for the life of the process.  cudaDeviceReset
//    destroys the context the address belongs to; a process that resets a device must call
//    mpsbnb_gemm_4bit_static_forget() afterwards, which drops the cache so that the next call
//    looks the address up again.
#include <atomic>

#include "ops.cuh"

namespace mpsbnb {

constexpr size_t STATIC_SCRATCH_BYTES = (size_t)32 << 20;      // 32 MiB: one 4096 x 4096 fp16 weight
constexpr int STATIC_MAX_DEVICES = 64;

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

// address of g_static_scratch on each device, looked up once per device
static std::atomic<unsigned char *> g_scratch_ptr[STATIC_MAX_DEVICES];

static inline int64_t pitch8(int64_t k) { return (k + 7) / 8 * 8; }
static inline size_t round256(size_t b) { return (b + 255) / 256 * 256; }
static inline size_t matrix_bytes(int64_t rows, int64_t K) { return round256((size_t)rows * (size_t)pitch8(K) * 2); }
static inline bool x_needs_copy(const void *x, int64_t K) { return K % 8 != 0 || !aligned16(x); }

static int scratch_for_current_device(unsigned char **out) {
    int dev = -1;
    MPSBNB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= STATIC_MAX_DEVICES) return MPSBNB_ERR_NO_DEVICE;
    unsigned char *p = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        // the symbol resolves to the copy that belongs to the device that is current right now;
        // two threads racing here store the same value
        MPSBNB_CUDA_TRY(cudaGetSymbolAddress((void **)&p, g_static_scratch));
        if (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 255) != 0) return MPSBNB_ERR_CUDA;
        g_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return MPSBNB_OK;
}

}  // namespace mpsbnb

using namespace mpsbnb;

extern "C" size_t mpsbnb_gemm_4bit_static_max_bytes(void) { return STATIC_SCRATCH_BYTES; }

extern "C" void mpsbnb_gemm_4bit_static_forget(void) {
    for (int d = 0; d < STATIC_MAX_DEVICES; ++d) g_scratch_ptr[d].store(nullptr, std::memory_order_release);
}

extern "C" size_t mpsbnb_gemm_4bit_static_bytes(const void *x, int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return (size_t)-1;   // beyond any scratch
    return matrix_bytes(N, K) + (x_needs_copy(x, K) ? matrix_bytes(M, K) : 0);
}

extern "C" int mpsbnb_gemm_4bit_static(const void *x, int x_dtype, int64_t M, const uint8_t *packed, const void *absmax,
                                       const float *absmax2, int64_t N, int64_t K, int blocksize, int quant_type,
                                       const void *bias, void *y, int y_dtype, void *stream) {
    if (!is_16bit(x_dtype) || !valid_dtype(y_dtype)) return MPSBNB_ERR_INVALID_ARG;
    if (M < 0 || N < 0 || K <= 0) return K == 0 && M >= 0 && N >= 0 ? MPSBNB_ERR_UNSUPPORTED : MPSBNB_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return MPSBNB_OK;
    if (x == nullptr || packed == nullptr || absmax == nullptr || y == nullptr) return MPSBNB_ERR_INVALID_ARG;
    // sizes beyond the fixed array are refused before anything is enqueued (and before any size arithmetic)
    if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return MPSBNB_ERR_TOO_LARGE;
    if (mpsbnb_gemm_4bit_static_bytes(x, M, N, K) > STATIC_SCRATCH_BYTES) return MPSBNB_ERR_TOO_LARGE;
    unsigned char *scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc != MPSBNB_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    void *w = scratch;
    const int64_t ldw = pitch8(K);
    rc = dequantize_4bit_ld(packed, absmax, absmax2, N, K, blocksize, quant_type, w, ldw, x_dtype, st);
    if (rc != MPSBNB_OK) return rc;
    const void *xa = x;
    int64_t lda = K;
    if (x_needs_copy(x, K)) {
        unsigned char *xs = scratch + matrix_bytes(N, K);
        lda = pitch8(K);
        rc = copy_rows_16bit_ld(x, M, K, xs, lda, st);
        if (rc != MPSBNB_OK) return rc;
        xa = xs;
    }
    return gemm_16bit(xa, lda, w, ldw, x_dtype, M, N, K, nullptr, nullptr, bias, x_dtype, y, N, y_dtype, st);
}
