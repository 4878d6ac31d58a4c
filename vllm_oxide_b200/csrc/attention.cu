// Causal grouped-query attention over the paged cache, for portions of prompts and for single
// decoded tokens alike.
//
// Math per (row, head a), the row at position p of its request, kvh = a / (H / KV):
//   s_j = (q_a . K[j, kvh]) * scale         for keys j in [first, p],  first = max(0, p+1-window)
//   out_a = sum_j softmax(s)_j * V[j, kvh]   softmax in float32 (running max and sum)
// Causality is "visit keys 0..p only", with the step's own keys already in the cache; there is
// no mask tensor. Reference: crates/engine/src/backend/cpu/attention.rs:76-128 (two passes
// there, one pass with a running maximum here; same value up to rounding), called for prefill
// and decode alike (crates/engine/src/backend/cpu/mod.rs:310,337).
// Cache layout per layer: K and V are [num_pages][KV][page_size][hd]; key j of a request lives
// in page block_table[seq][j / page_size] at offset j % page_size.
#include "common.cuh"
VOB_PDL_SWITCH(attention)

// ---------------------------------------------------------------------------------------------
// General kernel: one warp per (row, head). Keys are visited in chunks of 32: each lane scores
// one key (its K row read in 16-byte pieces against q held in shared memory), the warp agrees
// on the running maximum, then the 32 weighted V rows are summed with lanes spread over the
// head's dimensions. Any head_dim that is a multiple of 8 up to 256, any H, KV, page size.
// Launch: ceil(T*H / 4) blocks of 128 threads; 4*hd floats of shared memory.
// Bound: L2/L1 bandwidth (every head of a group re-reads its K/V); this is the kernel of the
// 32-bit engine and the fallback of the bfloat16 engine for sizes its tuned kernels refuse.
// A row's result depends only on its own q and keys, never on the batch around it.
// ---------------------------------------------------------------------------------------------
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static inline void load(const float* p, float* o) {
        float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static inline void load(const __nv_bfloat16* p, float* o) {
        uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(h[i]);
            o[2 * i] = f.x; o[2 * i + 1] = f.y;
        }
    }
};

template <typename T>
__global__ void __launch_bounds__(128, 8)
paged_attention_warp_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                            const T* __restrict__ kcache, const T* __restrict__ vcache,
                            const int* __restrict__ block_tables, int max_pages,
                            const int* __restrict__ row_seq, const int* __restrict__ positions,
                            int T_rows, int H, int KV, int hd, int page_size, int window, float scale) {
    pdl_launch_dependents();
    pdl_wait(6);
    extern __shared__ float qs_all[];
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long w = (long long)blockIdx.x * 4 + warp;
    if (w >= (long long)T_rows * H) return;          // whole warp leaves together
    int row = (int)(w / H), head = (int)(w % H);
    int kvh = head / (H / KV);
    float* qs = qs_all + warp * hd;
    const T* qp = q + (size_t)row * q_stride + (size_t)head * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = ld_f(qp + d);
    __syncwarp();

    int pos = positions[row];
    if (pos < 0) {                                   // a padding row: no keys, zero output
        T* op0 = out + (size_t)row * out_stride + (size_t)head * hd;
        for (int d = lane; d < hd; d += 32) st_f(op0 + d, 0.f);
        return;
    }
    int seq = row_seq[row];
    const int* bt = block_tables + (size_t)seq * max_pages;
    int first = window > 0 ? max(0, pos + 1 - window) : 0;

    constexpr int VN = Vec16<T>::N;
    float m = -INFINITY, l = 0.f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;

    for (int c0 = first; c0 <= pos; c0 += 32) {
        int j = c0 + lane;
        bool valid = j <= pos;
        int slot_row = 0;          // row index of key j in the [.., hd] view of the layer's cache
        float s = -INFINITY;
        if (valid) {
            int page = bt[j / page_size];
            slot_row = (page * KV + kvh) * page_size + (j % page_size);
            const T* kp = kcache + (size_t)slot_row * hd;
            float dot = 0.f;
            for (int d = 0; d < hd; d += VN) {
                float kv[VN];
                Vec16<T>::load(kp + d, kv);
#pragma unroll
                for (int i = 0; i < VN; ++i) dot = fmaf(qs[d + i], kv[i], dot);
            }
            s = dot * scale;
        }
        float m_new = fmaxf(m, warp_max(s));
        float p = valid ? expf(s - m_new) : 0.f;
        float alpha = expf(m - m_new);               // 0 on the first chunk (m = -inf)
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= alpha;
        m = m_new;
        int nk = min(32, pos - c0 + 1);
        for (int jj = 0; jj < nk; ++jj) {
            float pj = __shfl_sync(0xffffffffu, p, jj);
            int sr = __shfl_sync(0xffffffffu, slot_row, jj);
            const T* vp = vcache + (size_t)sr * hd;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int d = 2 * lane + 64 * i;
                if (d < hd) {
                    acc[2 * i] = fmaf(pj, ld_f(vp + d), acc[2 * i]);
                    acc[2 * i + 1] = fmaf(pj, ld_f(vp + d + 1), acc[2 * i + 1]);
                }
            }
        }
    }
    float inv_l = 1.0f / l;
    T* op = out + (size_t)row * out_stride + (size_t)head * hd;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int d = 2 * lane + 64 * i;
        if (d < hd) {
            st_f(op + d, acc[2 * i] * inv_l);
            st_f(op + d + 1, acc[2 * i + 1] * inv_l);
        }
    }
}

VOB_EXPORT int vob_paged_attention(const void* q, long long q_stride, void* out, long long out_stride,
                                   const void* kcache, const void* vcache, int code,
                                   const int* block_tables, int max_pages, const int* row_seq,
                                   const int* positions, int T_rows, int H, int KV, int hd, int page_size,
                                   int window, float scale, cudaStream_t stream) {
    if (T_rows <= 0) return 0;
    if (H <= 0 || KV <= 0 || H % KV != 0 || page_size <= 0 || max_pages <= 0) return VOB_ERR_BAD_ARG;
    if (hd <= 0 || hd % 8 != 0 || hd > 256) return VOB_ERR_UNSUPPORTED;
    long long warps = (long long)T_rows * H;
    long long blocks = (warps + 3) / 4;
    if (blocks > 0x7fffffffLL) return VOB_ERR_UNSUPPORTED;
    size_t smem = 4 * (size_t)hd * sizeof(float);
    VOB_DISPATCH_ELEM(code, return vob_launch(paged_attention_warp_kernel<ElemT>, dim3((unsigned)blocks), dim3(128), smem, stream,
        (const ElemT*)q, q_stride, (ElemT*)out, out_stride, (const ElemT*)kcache, (const ElemT*)vcache, block_tables,
        max_pages, row_seq, positions, T_rows, H, KV, hd, page_size, window, scale));
    return 0;
}
