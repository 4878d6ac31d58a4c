// Picking the next token from float32 logits [R, V]: greedy, or temperature sampling by the
// Gumbel-max rule, one pick per row, on the device.
//
//   temperature == 0:  first index of the maximum (strictly-greater comparison keeps the first,
//                      crates/engine/src/backend/cpu/mod.rs:370-388); a NaN anywhere in the row
//                      makes the row's pick -1, which the host turns into an error (:377-379).
//   temperature  > 0:  argmax_i(logit_i / temperature + g_i),  g_i = -log(-log(u_i)),
//                      u_i in (0,1) from a counter-based hash of (seed, generated index, i):
//                      a draw from softmax(logits / temperature) that depends on nothing but the
//                      request's own seed and progress (the reference samples greedily only;
//                      this rule is this engine's own).
// Two launches: `pick_partial` gives every (row, slice of the vocabulary) block a best
// (value, index) pair in scratch memory, `pick_final` reduces a row's pairs. The scratch is
// [R, splits] pairs supplied by the caller. Bound: memory (R * V * 4 bytes read once).
#include "common.cuh"
VOB_PDL_SWITCH(sampling)

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
    return x;
}

struct Best { float v; int i; };

__device__ __forceinline__ Best better(Best a, Best b) {
    // larger value wins; equal values: smaller index wins
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ Best block_best(Best b, Best* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
        b = better(b, other);
    }
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) sh[wid] = b;
    __syncthreads();
    if (wid == 0) {
        Best x = lane < (blockDim.x >> 5) ? sh[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other;
            other.v = __shfl_xor_sync(0xffffffffu, x.v, o);
            other.i = __shfl_xor_sync(0xffffffffu, x.i, o);
            x = better(x, other);
        }
        b = x;
    }
    return b;   // valid in thread 0
}

__global__ void __launch_bounds__(256)
pick_partial_kernel(const float* __restrict__ logits, long long ld, int V, const float* __restrict__ temperature,
                    const uint32_t* __restrict__ seeds, const int* __restrict__ steps, int splits,
                    float* __restrict__ part_val, int* __restrict__ part_idx, int* __restrict__ nan_flags) {
    pdl_launch_dependents();
    pdl_wait(9);
    __shared__ Best sh[32];
    int r = blockIdx.y, sp = blockIdx.x;
    int per = (V + splits - 1) / splits;
    int lo = sp * per, hi = min(V, lo + per);
    const float* row = logits + (size_t)r * ld;
    float tau = temperature ? temperature[r] : 0.f;
    uint32_t ctr = 0;
    if (tau > 0.f) {
        uint32_t key = mix32(seeds[2 * r] ^ mix32(seeds[2 * r + 1] + 0x85EBCA6Bu));
        ctr = mix32(key ^ mix32((uint32_t)steps[r] + 0x9E3779B9u));
    }
    Best b{-INFINITY, 0x7fffffff};
    bool saw_nan = false;
#pragma unroll 4
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float x = row[i];
        if (x != x) saw_nan = true;
        float v = x;
        if (tau > 0.f) {
            uint32_t h = mix32(ctr ^ (uint32_t)i);
            float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
            v = x / tau + (-logf(-logf(u)));
        }
        if (v > b.v) { b.v = v; b.i = i; }      // ascending i per thread: first maximum kept
    }
    if (saw_nan) atomicExch(nan_flags + r, 1);
    b = block_best(b, sh);
    if (threadIdx.x == 0) {
        part_val[(size_t)r * splits + sp] = b.v;
        part_idx[(size_t)r * splits + sp] = b.i;
    }
}

// `also_a`, `also_b` (either may be null): two more places the picked token of every row is written
// to, e.g. the next step's token rows and a host buffer the device can address, so that no copy has
// to follow the kernel.
__global__ void pick_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                  int splits, int V, int* __restrict__ nan_flags, int* __restrict__ out,
                                  int* also_a, int* also_b) {
    pdl_launch_dependents();
    pdl_wait(10);
    __shared__ Best sh[32];
    int r = blockIdx.x;
    Best b{-INFINITY, 0x7fffffff};
    for (int s = threadIdx.x; s < splits; s += blockDim.x)
        b = better(b, Best{part_val[(size_t)r * splits + s], part_idx[(size_t)r * splits + s]});
    b = block_best(b, sh);
    // all values -inf or NaN: fall back to index 0, as a scan that never finds a greater value does
    // A row that held a NaN yields -1 (the host turns it into an error) and its flag is cleared.
    if (threadIdx.x == 0) {
        int tok = (b.i >= 0 && b.i < V) ? b.i : 0;
        if (nan_flags[r]) { tok = -1; nan_flags[r] = 0; }
        out[r] = tok;
        if (also_a) also_a[r] = tok;
        if (also_b) also_b[r] = tok;
    }
}

// Scratch needed: R * splits floats and R * splits ints. `splits` is chosen by the caller
// (vob_pick_splits gives the default for a vocabulary size).
VOB_EXPORT int vob_pick_splits(int V) {
    // slices of 1,024 logits: four per thread, all loads of a thread in flight at once (with slices
    // of 4,096 a thread made sixteen dependent round trips: 10 us for 8 rows of 128,256)
    int s = (V + 1023) / 1024;
    return s < 1 ? 1 : (s > 256 ? 256 : s);
}

VOB_EXPORT int vob_pick_tokens_to(const float* logits, long long ld, int R, int V, const float* temperature,
                                  const uint32_t* seeds, const int* steps, int splits, float* part_val,
                                  int* part_idx, int* nan_flags, int* out, int* also_a, int* also_b, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || splits <= 0 || ld < V || R > 65535) return VOB_ERR_BAD_ARG;
    if (temperature && (!seeds || !steps)) return VOB_ERR_BAD_ARG;
    dim3 grid(splits, R);
    int e = vob_launch(pick_partial_kernel, grid, dim3(256), 0, stream, logits, ld, V, temperature, seeds, steps, splits,
                       part_val, part_idx, nan_flags);
    if (e) return e;
    return vob_launch(pick_final_kernel, dim3(R), dim3(64), 0, stream, (const float*)part_val, (const int*)part_idx, splits, V,
                      nan_flags, out, also_a, also_b);
}

VOB_EXPORT int vob_pick_tokens(const float* logits, long long ld, int R, int V, const float* temperature,
                               const uint32_t* seeds, const int* steps, int splits, float* part_val,
                               int* part_idx, int* nan_flags, int* out, cudaStream_t stream) {
    return vob_pick_tokens_to(logits, ld, R, V, temperature, seeds, steps, splits, part_val, part_idx, nan_flags, out, nullptr,
                              nullptr, stream);
}

// The second launch alone: the pairs come from elsewhere (the output head's own epilogue reduces
// each of its tiles to a pair: EPI_PICK in gemm_sm100.cu), `splits` of them per row.
VOB_EXPORT int vob_pick_final_to(const float* part_val, const int* part_idx, int R, int splits, int V, int* nan_flags, int* out,
                                 int* also_a, int* also_b, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || splits <= 0 || R > 65535) return VOB_ERR_BAD_ARG;
    // one pair per thread where that is possible: a thread that walks many pairs pays a memory round trip for each
    const int threads = splits > 512 ? 1024 : splits > 256 ? 512 : splits > 64 ? 256 : 64;
    return vob_launch(pick_final_kernel, dim3(R), dim3(threads), 0, stream, part_val, part_idx, splits, V, nan_flags, out, also_a,
                      also_b);
}

VOB_EXPORT int vob_pick_final(const float* part_val, const int* part_idx, int R, int splits, int V, int* nan_flags, int* out,
                              cudaStream_t stream) {
    return vob_pick_final_to(part_val, part_idx, R, splits, V, nan_flags, out, nullptr, nullptr, stream);
}

// The address under which the device reaches a page-locked host buffer (0 on success). A kernel may
// then write there directly; what it wrote is the host's to read once the kernel has completed.
VOB_EXPORT int vob_host_device_pointer(void* host, void** device) {
    if (!host || !device) return VOB_ERR_BAD_ARG;
    *device = nullptr;
    return (int)cudaHostGetDevicePointer(device, host, 0);
}

// ---------------------------------------------------------------------------------------------
// The same pick for callers that cannot allocate: scratch in a fixed device array of this
// library (see no_alloc.h for who needs this and the rules that come with it).
// ---------------------------------------------------------------------------------------------
#include "no_alloc.h"
#include <mutex>

static __device__ __align__(256) unsigned char vob_pick_static_scratch[VOB_PICK_STATIC_BYTES];

// Device address of the array on the current device. In host code the array's name is only a
// handle for the runtime, not an address a kernel could use; the address comes from
// cudaGetSymbolAddress, once per device, with that device current.
static int pick_static_scratch_address(unsigned char** ptr) {
    static std::mutex mu;
    static unsigned char* known[64] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return VOB_ERR_BAD_ARG;
    std::lock_guard<std::mutex> g(mu);
    if (!known[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, vob_pick_static_scratch);
        if (e != cudaSuccess) return (int)e;
        known[dev] = static_cast<unsigned char*>(p);
    }
    *ptr = known[dev];
    return 0;
}

int vob_pick_tokens_static(const float* logits, long long ld, int R, int V, const float* temperature,
                           const uint32_t* seeds, const int* steps, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (R > VOB_PICK_STATIC_MAX_ROWS) return VOB_ERR_STATIC_TOO_LARGE;
    if (V <= 0 || ld < V || !logits || !out) return VOB_ERR_BAD_ARG;
    if (temperature && (!seeds || !steps)) return VOB_ERR_BAD_ARG;
    int splits = vob_pick_splits(V);
    if (splits > VOB_PICK_STATIC_MAX_SPLITS) return VOB_ERR_STATIC_TOO_LARGE;
    unsigned char* base = nullptr;
    int rc = pick_static_scratch_address(&base);
    if (rc) return rc;
    float* part_val = reinterpret_cast<float*>(base);
    int* part_idx = reinterpret_cast<int*>(base + VOB_PICK_STATIC_MAX_ROWS * VOB_PICK_STATIC_MAX_SPLITS * 4);
    int* nan_flags = reinterpret_cast<int*>(base + VOB_PICK_STATIC_MAX_ROWS * VOB_PICK_STATIC_MAX_SPLITS * 8);
    // the array keeps what the last call left: the NaN marks must start at zero (a call that ran to
    // its end has put its own marks back; one that failed between its two launches has not)
    cudaError_t e = cudaMemsetAsync(nan_flags, 0, sizeof(int) * R, stream);
    if (e != cudaSuccess) return (int)e;
    return vob_pick_tokens(logits, ld, R, V, temperature, seeds, steps, splits, part_val, part_idx, nan_flags, out, stream);
}

// For the test of the rule above: sets the NaN marks of the first `rows` rows in the fixed array,
// as a call that failed between its two launches would leave them.
int vob_pick_static_test_leave_marks(int rows, cudaStream_t stream) {
    if (rows < 0 || rows > VOB_PICK_STATIC_MAX_ROWS) return VOB_ERR_BAD_ARG;
    unsigned char* base = nullptr;
    int rc = pick_static_scratch_address(&base);
    if (rc) return rc;
    int* nan_flags = reinterpret_cast<int*>(base + VOB_PICK_STATIC_MAX_ROWS * VOB_PICK_STATIC_MAX_SPLITS * 8);
    return (int)cudaMemsetAsync(nan_flags, 0x01, sizeof(int) * rows, stream);
}
