// Shared helpers of the kernel modules: element types, loads that widen to float, the error
// convention of the C entry points.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and a stream, launches on
// that stream and returns 0 or a cudaError_t value; it never allocates and never synchronises.
// Element types of activations, weights and cache are chosen by an integer code so that one
// library serves the 32-bit and the bfloat16 engine.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define VOB_F32 0
#define VOB_BF16 1

#define VOB_EXPORT extern "C" __attribute__((visibility("default")))

// Status codes beyond cudaError_t (which stays below 1000).
#define VOB_ERR_BAD_ARG 2001       // a size or code the kernel refuses
#define VOB_ERR_UNSUPPORTED 2002   // a size outside what this kernel was built for

static inline int vob_launch_status() {
    cudaError_t e = cudaGetLastError();
    return (int)e;
}

// Programmatic dependent launch. Every kernel of this package calls pdl_launch_dependents() first
// thing (so the next kernel in the stream may start as soon as all blocks of this one have
// started) and pdl_wait() before it touches anything an earlier kernel wrote or still reads (the
// wait returns once every earlier grid has completed and its memory is visible). What a kernel
// does between the two (barrier set-up, tensor-memory allocation, prefetch of weights, which no
// kernel writes) overlaps the tail of its predecessors. Launches carry the attribute only while
// the switch below is on; without it both instructions do nothing.
// Optional timeline of a step (a debugging aid, compiled in only with -DVOB_TIMELINE, i.e. when the
// libraries are built with VOB_TIMELINE=1 in the environment, and off unless a buffer is set): block 0 of every
// kernel notes the global timer when it starts and when its wait returns; the wait of kernel n+1
// returns when kernel n has completed, so consecutive entries give each kernel's place in time.
// Layout: tl[0] = next free entry; entry e = {tag, start_ns, ready_ns} at tl[1 + 3e].
__device__ unsigned long long* g_vob_timeline = nullptr;
__device__ __forceinline__ unsigned long long vob_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait(int tag = 0) {
#ifdef VOB_TIMELINE
    unsigned long long* tl = g_vob_timeline;
    bool rec = tl && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    unsigned long long t0 = rec ? vob_now_ns() : 0;
#endif
    asm volatile("griddepcontrol.wait;" ::: "memory");
#ifdef VOB_TIMELINE
    if (rec) {
        unsigned long long e = atomicAdd(tl, 1ull);
        if (e < 4096) { tl[1 + 3 * e] = (unsigned long long)tag; tl[2 + 3 * e] = t0; tl[3 + 3 * e] = vob_now_ns(); }
    }
#endif
}

static int g_vob_pdl = 0;

template <typename... P, typename... A>
static inline int vob_launch(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_vob_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
    return e != cudaSuccess ? (int)e : vob_launch_status();
}

#define VOB_PDL_SWITCH(module)                                                              \
    VOB_EXPORT void vob_set_pdl_##module(int on) { g_vob_pdl = on; }                        \
    VOB_EXPORT int vob_set_timeline_##module(unsigned long long* buf) {                      \
        return (int)cudaMemcpyToSymbol(g_vob_timeline, &buf, sizeof(buf));                   \
    }

template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> {
    static constexpr int code = VOB_F32;
    __device__ static inline float load(const float* p) { return *p; }
    __device__ static inline void store(float* p, float v) { *p = v; }
};
template <> struct ElemTraits<__nv_bfloat16> {
    static constexpr int code = VOB_BF16;
    __device__ static inline float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    __device__ static inline void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

template <typename T> __device__ inline float ld_f(const T* p) { return ElemTraits<T>::load(p); }
template <typename T> __device__ inline void st_f(T* p, float v) { ElemTraits<T>::store(p, v); }

__device__ inline float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ inline float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Dispatch on an element code: the statement given uses the type ElemT.
#define VOB_DISPATCH_ELEM(code, ...)                                   \
    do {                                                               \
        if ((code) == VOB_F32) { using ElemT = float; __VA_ARGS__; }       \
        else if ((code) == VOB_BF16) { using ElemT = __nv_bfloat16; __VA_ARGS__; } \
        else return VOB_ERR_BAD_ARG;                                   \
    } while (0)
