// Shared declarations of the sm_100a kernel library: storage types, error reporting and the
// conventions of the exported C entry points.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and a CUDA stream,
// launches on that stream without synchronising, and returns 0 or a negative code; the
// message of the last failure on the calling thread is read with kestrel_last_error().
// Storage type codes: 0 = float32, 1 = bfloat16.  Sums, norms, softmax, rotation angles and
// the residual stream are float32 whatever the storage type.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// every exported entry point is declared in the package's one C header; a definition that
// differs from its declaration there does not compile
#include "../../include/kestrel.h"

int kestrel_fail(int code, const char *fmt, ...);
// multiprocessors of the current device (cost models and grids size themselves by it); a
// B200's 148 where no device can be asked, as when a cost model is called on a host without one
static inline int kestrel_sms() {
    int n = kestrel_sm_count();
    return n > 0 ? n : 148;
}
int kestrel_check_launch(const char *what);

#define KESTREL_REQUIRE(cond, ...)                       \
    do {                                                 \
        if (!(cond)) return kestrel_fail(-2, __VA_ARGS__); \
    } while (0)

// Programmatic dependent launch.  Every kernel of the library is launched with the attribute
// that lets it start while its predecessor on the stream is still draining, calls
// pdl_launch_dependents() first thing (so that its own successor may be scheduled as soon as
// all of its blocks are resident) and pdl_wait() before it touches global memory (which
// returns once the predecessor has completed and its writes are visible).  Because every
// kernel waits, completion is transitive along the stream.  What runs before the wait - barrier
// set-up, TMEM allocation, descriptor prefetch, index arithmetic - overlaps the predecessor's
// tail.  kestrel_set_pdl(0) switches the attribute off; the instructions are then no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

extern int g_kestrel_pdl;

template <typename... KArgs, typename... Args>
static inline cudaError_t kestrel_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_kestrel_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Dynamic shared memory to ask for so that the block scheduler spreads a grid of few, long-running
// CTAs evenly over the SMs.  A kernel launched as a programmatic dependent gets its CTAs placed
// while the predecessor's last blocks still hold most SMs: the scheduler fills the first SMs that
// free up with as many CTAs as fit, so a latency-bound scan of 128 small CTAs ends up three to an
// SM on a third of the chip and runs at half speed.  Asking for 1/n of an SM's shared memory, with
// n = ceil(ctas / SMs), caps every SM at the share an even spread gives it.  `need` is what the
// kernel uses; the result is never smaller.  (228 KB an SM, 1 KB of it reserved per resident CTA.)
#define KESTREL_SMEM_MAX_DYNAMIC (227 * 1024)
static inline size_t kestrel_spread_smem(long ctas, size_t need) {
    const long per_sm = (ctas + 147) / 148;
    if (per_sm > 32) return need;
    size_t want = ((size_t)(228 * 1024) / (size_t)per_sm - 1024) & ~(size_t)127;
    if (want > KESTREL_SMEM_MAX_DYNAMIC) want = KESTREL_SMEM_MAX_DYNAMIC;
    return want > need ? want : need;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum of a product's float32 slices at one element, in ascending slice order; the loads of eight
// (then four) slices are in flight at once (the adds keep their order, so the bits are those of a
// plain loop).
__device__ __forceinline__ float sum_slices(const float *__restrict__ p, int S, size_t slice_stride, size_t off) {
    float v = 0.f;
    int s = 0;
    for (; s + 8 <= S; s += 8) {
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = p[(size_t)(s + j) * slice_stride + off];
#pragma unroll
        for (int j = 0; j < 8; ++j) v += x[j];
    }
    for (; s + 4 <= S; s += 4) {
        const float a = p[(size_t)s * slice_stride + off], b = p[(size_t)(s + 1) * slice_stride + off];
        const float c = p[(size_t)(s + 2) * slice_stride + off], d = p[(size_t)(s + 3) * slice_stride + off];
        v += a; v += b; v += c; v += d;
    }
    const int rest = S - s;                           // up to three more: their loads in flight together as well
    if (rest == 3) {
        const float a = p[(size_t)s * slice_stride + off], b = p[(size_t)(s + 1) * slice_stride + off], c = p[(size_t)(s + 2) * slice_stride + off];
        v += a; v += b; v += c;
    } else if (rest == 2) {
        const float a = p[(size_t)s * slice_stride + off], b = p[(size_t)(s + 1) * slice_stride + off];
        v += a; v += b;
    } else if (rest == 1) {
        v += p[(size_t)s * slice_stride + off];
    }
    return v;
}
