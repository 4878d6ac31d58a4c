// Memory-bound row kernels of a decoder step: embedding gather, residual add + RMSNorm,
// rotary positions + cache write, SwiGLU.
//
// Conventions: the residual stream is float32 in both engines; `act` tensors (inputs of the
// matrix products, q/k/v, the cache) are float32 or bfloat16 by an element code. All
// reductions, rotation angles and the activation are float32. One block works on one row, so a
// row's result does not depend on what else is in the batch.
#include "common.cuh"
VOB_PDL_SWITCH(elementwise)

// ---------------------------------------------------------------------------------------------
// Embedding gather: out[t, :] = table[tokens[t], :]   (float32 out)
// Reference op: crates/engine/src/backend/cpu/mod.rs:172-180.
// Launch: one block per token, 256 threads. Bound: memory (2 * h * 4 bytes per token).
// A token outside [0, vocab) writes zeros and raises *err_flag (the host checks ids first).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int h, int vocab, int* err_flag) {
    pdl_launch_dependents();
    pdl_wait(1);
    int t = blockIdx.x;
    int tok = tokens[t];
    bool ok = tok >= 0 && tok < vocab;
    if (!ok && threadIdx.x == 0 && err_flag) atomicExch(err_flag, 1);
    const T* src = table + (size_t)(ok ? tok : 0) * h;
    float* dst = out + (size_t)t * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) dst[i] = ok ? ld_f(src + i) : 0.f;
}

VOB_EXPORT int vob_embed(const void* table, int table_code, const int* tokens, float* out, int T, int h,
                         int vocab, int* err_flag, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (h <= 0 || vocab <= 0) return VOB_ERR_BAD_ARG;
    VOB_DISPATCH_ELEM(table_code, return vob_launch(embed_kernel<ElemT>, dim3(T), dim3(256), 0, stream, (const ElemT*)table, tokens, out, h, vocab, err_flag));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Embedding gather that also prepares the first norm's input in folded form (see EPI_RESID in
// gemm_sm100.cu): resid[t] = table[token]; xn[t] = bf16(resid * next_w); ssq[tile][t] = the sum of
// squares of resid over features tile*128 .. +127. One block of 128 threads per token and tile (a
// block per token that walked the tiles took one memory round trip per tile: 14 us for a width of
// 2,048); the order of every sum is fixed.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
embed_fold_kernel(const T* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ resid,
                  const float* __restrict__ next_w, __nv_bfloat16* __restrict__ xn, float* __restrict__ ssq, int ld_ssq, int h,
                  int vocab, int* err_flag) {
    pdl_launch_dependents();
    pdl_wait(1);
    __shared__ float red[4];
    const int t = blockIdx.x, tile = blockIdx.y;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < vocab;
    if (!ok && threadIdx.x == 0 && tile == 0 && err_flag) atomicExch(err_flag, 1);
    const T* src = table + (size_t)(ok ? tok : 0) * h;
    const int f = tile * 128 + threadIdx.x;
    float v = 0.f;
    if (f < h) {
        v = ok ? ld_f(src + f) : 0.f;
        resid[(size_t)t * h + f] = v;
        xn[(size_t)t * h + f] = __float2bfloat16_rn(v * next_w[f]);
    }
    float sq = warp_sum(v * v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x == 0) ssq[(size_t)tile * ld_ssq + t] = (red[0] + red[1]) + (red[2] + red[3]);
}

VOB_EXPORT int vob_embed_fold(const void* table, int table_code, const int* tokens, float* resid, const float* next_w, void* xn,
                              float* ssq, int ld_ssq, int T, int h, int vocab, int* err_flag, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (h <= 0 || vocab <= 0 || ld_ssq < T) return VOB_ERR_BAD_ARG;
    if ((h + 127) / 128 > 65535) return VOB_ERR_UNSUPPORTED;
    VOB_DISPATCH_ELEM(table_code, return vob_launch(embed_fold_kernel<ElemT>, dim3(T, (h + 127) / 128), dim3(128), 0, stream, (const ElemT*)table, tokens,
                                                    resid, next_w, (__nv_bfloat16*)xn, ssq, ld_ssq, h, vocab, err_flag));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Residual add + RMSNorm:
//   x = resid[src] (+ delta[src]);  if no row list: resid[src] = x  (the residual sum, float32)
//   out[r] = w * (x * 1/sqrt(mean(x^2) + eps))
// Reference ops: add (crates/engine/src/backend/cpu/mod.rs:351-358) followed by rmsnorm
// (:182-197); the weight multiplies last, as there. With a row list (`rows`, R entries) only
// those rows are normalised (gather_rows + rmsnorm, crates/engine/src/model.rs:335-342) and
// the residual is left untouched.
// Launch: one block per output row, 256 threads, h floats of shared memory; the row is read
// once. Sum of squares: per-thread strided partial sums, then a fixed tree, so a row's value is
// the same in every batch. Bound: memory.
// ---------------------------------------------------------------------------------------------
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                   const float* __restrict__ weight, const int* __restrict__ rows,
                                   TO* __restrict__ out, int h, float eps) {
    pdl_launch_dependents();
    pdl_wait(2);
    extern __shared__ float row[];
    __shared__ float red[32];
    int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    float* x = resid + (size_t)src * h;
    const TD* d = delta ? delta + (size_t)src * h : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        float v = x[i];
        if (d) {
            v += ld_f(d + i);
            if (!rows) x[i] = v;
        }
        row[i] = v;
        ss += v * v;
    }
    ss = warp_sum(ss);
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) red[wid] = ss;
    __syncthreads();
    if (wid == 0) {
        float v = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
        v = warp_sum(v);
        if (lane == 0) red[0] = v;
    }
    __syncthreads();
    float mean_square = red[0] / (float)h;
    float inv = 1.0f / sqrtf(mean_square + eps);
    TO* o = out + (size_t)r * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) st_f(o + i, weight[i] * (row[i] * inv));
}

// Fast path for rows whose width is a multiple of 4 and fits NV float4 per thread: every load of
// the row is issued before anything depends on one (a row of a small batch is latency-bound, not
// bandwidth-bound), the row stays in registers, and the sums take the same fixed order for every
// row. Same arithmetic as the kernel above.
template <typename TD> struct Load4;
template <> struct Load4<float> {
    __device__ static inline float4 ld(const float* p) { return *reinterpret_cast<const float4*>(p); }
};
template <> struct Load4<__nv_bfloat16> {
    __device__ static inline float4 ld(const __nv_bfloat16* p) {
        uint2 u = *reinterpret_cast<const uint2*>(p);
        float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
};
template <typename TO> struct Store4;
template <> struct Store4<float> {
    __device__ static inline void st(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Store4<__nv_bfloat16> {
    __device__ static inline void st(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&a);
        u.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

template <typename TD, typename TO, int NV>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ resid, const TD* __restrict__ delta, const float* __restrict__ weight,
                       const int* __restrict__ rows, TO* __restrict__ out, int h, float eps) {
    pdl_launch_dependents();
    pdl_wait(2);
    __shared__ float red[32];
    int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    float* x = resid + (size_t)src * h;
    const TD* d = delta ? delta + (size_t)src * h : nullptr;
    int nvec = h >> 2;
    float4 v[NV], dv[NV], w[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        int i = threadIdx.x + k * 256;
        if (i < nvec) {
            v[k] = *reinterpret_cast<const float4*>(x + 4 * i);
            dv[k] = d ? Load4<TD>::ld(d + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
            w[k] = *reinterpret_cast<const float4*>(weight + 4 * i);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        int i = threadIdx.x + k * 256;
        if (i < nvec) {
            v[k].x += dv[k].x; v[k].y += dv[k].y; v[k].z += dv[k].z; v[k].w += dv[k].w;
            if (d && !rows) *reinterpret_cast<float4*>(x + 4 * i) = v[k];
            ss += v[k].x * v[k].x; ss += v[k].y * v[k].y; ss += v[k].z * v[k].z; ss += v[k].w * v[k].w;
        }
    }
    ss = warp_sum(ss);
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) red[wid] = ss;
    __syncthreads();
    if (wid == 0) {
        float t = lane < 8 ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[0] = t;
    }
    __syncthreads();
    float inv = 1.0f / sqrtf(red[0] / (float)h + eps);
    TO* o = out + (size_t)r * h;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        int i = threadIdx.x + k * 256;
        if (i < nvec)
            Store4<TO>::st(o + 4 * i, make_float4(w[k].x * (v[k].x * inv), w[k].y * (v[k].y * inv),
                                                  w[k].z * (v[k].z * inv), w[k].w * (v[k].w * inv)));
    }
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* resid, const void* delta, const float* weight, const int* rows, void* out, int R,
                              int h, float eps, cudaStream_t stream) {
    bool aligned = (h % 4 == 0) && (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) % 16 == 0);
    int nv = (h / 4 + 255) / 256;
    if (aligned && nv <= 8) {
#define VEC(NV) return vob_launch(add_rmsnorm_vec_kernel<TD, TO, NV>, dim3(R), dim3(256), 0, stream, resid, (const TD*)delta, weight, rows, (TO*)out, h, eps)
        if (nv <= 1) VEC(1); else if (nv <= 2) VEC(2); else if (nv <= 4) VEC(4); else VEC(8);
#undef VEC
    }
    size_t smem = (size_t)h * sizeof(float);
    if (smem > 48 * 1024) return VOB_ERR_UNSUPPORTED;
    return vob_launch(add_rmsnorm_kernel<TD, TO>, dim3(R), dim3(256), smem, stream, resid, (const TD*)delta, weight, rows, (TO*)out, h, eps);
}

VOB_EXPORT int vob_add_rmsnorm(float* resid, const void* delta, int delta_code, const float* weight,
                               const int* rows, void* out, int out_code, int R, int h, float eps,
                               cudaStream_t stream) {
    if (R <= 0) return 0;
    if (h <= 0) return VOB_ERR_BAD_ARG;
    if (!delta) delta_code = VOB_F32;
    if (out_code == VOB_F32) {
        if (delta_code == VOB_F32) return launch_add_rmsnorm<float, float>(resid, delta, weight, rows, out, R, h, eps, stream);
        if (delta_code == VOB_BF16) return launch_add_rmsnorm<__nv_bfloat16, float>(resid, delta, weight, rows, out, R, h, eps, stream);
    } else if (out_code == VOB_BF16) {
        if (delta_code == VOB_F32) return launch_add_rmsnorm<float, __nv_bfloat16>(resid, delta, weight, rows, out, R, h, eps, stream);
        if (delta_code == VOB_BF16) return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, weight, rows, out, R, h, eps, stream);
    }
    return VOB_ERR_BAD_ARG;
}

// ---------------------------------------------------------------------------------------------
// Rotary positions on q and k, and the cache write of k and v, in one pass over a token's
// q/k/v rows:
//   theta_i = float(pos) * inv_freq[i]         (float32 product; cosf/sinf precise versions)
//   x1' = x1*cos - x2*sin ; x2' = x2*cos + x1*sin   with x1 = x[:hd/2], x2 = x[hd/2:] per head
//   K[page, kvh, off, :] = k'[kvh],  V[page, kvh, off, :] = v[kvh],  slot = page*page_size+off
// Reference ops: rope (crates/engine/src/backend/cpu/rope.rs:64-99) on q and k, then write_kv
// (crates/engine/src/backend/cpu/mod.rs:257-285), in that order before attention
// (crates/engine/src/model.rs:307-311). q is rotated in place. A page holds
// [kv_heads][page_size][head_dim], so one (page, head) is one contiguous tile.
// `slots` may be null (rotate only); a negative slot skips that token's write.
// `inv_freq` may be null (no rotation: the part has no position encoding).
// Launch: grid (tokens, ceil((H+KV)*hd/2 / 128)), one thread per (head, pair); each thread takes
// the sine and cosine of its own angle. Bound: memory.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
rope_kv_write_kernel(T* __restrict__ q, long long q_stride, T* __restrict__ k, long long k_stride,
                     const T* __restrict__ v, long long v_stride, const int* __restrict__ positions,
                     const int* __restrict__ slots, const float* __restrict__ inv_freq, T* __restrict__ kcache,
                     T* __restrict__ vcache, int H, int KV, int hd, int page_size) {
    // one thread per (head, pair i): heads 0..H-1 are q heads, H..H+KV-1 are k heads (with their v)
    pdl_launch_dependents();
    pdl_wait(4);
    int t = blockIdx.x;
    int half = hd >> 1;
    int e = blockIdx.y * blockDim.x + threadIdx.x;
    int nheads = H + (k ? KV : 0);
    if (e >= nheads * half) return;
    int head = e / half, i = e - head * half;
    float c = 1.f, s = 0.f;
    if (inv_freq) {
        float theta = (float)positions[t] * inv_freq[i];
        c = cosf(theta);
        s = sinf(theta);
    }
    if (head < H) {
        T* x = q + (size_t)t * q_stride + (size_t)head * hd;
        if (inv_freq) {
            float a = ld_f(x + i), b = ld_f(x + half + i);
            st_f(x + i, a * c - b * s);
            st_f(x + half + i, b * c + a * s);
        }
        return;
    }
    int kh = head - H;
    T* x = k + (size_t)t * k_stride + (size_t)kh * hd;
    float a = ld_f(x + i), b = ld_f(x + half + i);
    float ra = a, rb = b;
    if (inv_freq) {
        ra = a * c - b * s;
        rb = b * c + a * s;
        st_f(x + i, ra);
        st_f(x + half + i, rb);
    }
    int slot = slots ? slots[t] : -1;
    if (slot >= 0) {
        size_t page = (size_t)(slot / page_size);
        int off = slot % page_size;
        size_t base = ((page * KV + kh) * page_size + off) * (size_t)hd;
        const T* vr = v + (size_t)t * v_stride + (size_t)kh * hd;
        st_f(kcache + base + i, ra);
        st_f(kcache + base + half + i, rb);
        vcache[base + i] = vr[i];
        vcache[base + half + i] = vr[half + i];
    }
}

// The same for many tokens: one block per token, thread (pair i, head group): the sine and cosine
// of the pair's angle are taken once and reused for every head the thread walks over, instead
// of once per (head, pair).
template <typename T>
__global__ void __launch_bounds__(128)
rope_kv_write_token_kernel(T* __restrict__ q, long long q_stride, T* __restrict__ k, long long k_stride,
                           const T* __restrict__ v, long long v_stride, const int* __restrict__ positions,
                           const int* __restrict__ slots, const float* __restrict__ inv_freq, T* __restrict__ kcache,
                           T* __restrict__ vcache, int H, int KV, int hd, int page_size) {
    pdl_launch_dependents();
    pdl_wait(4);
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int groups = blockDim.x / half;          // head groups that work side by side
    const int i = threadIdx.x % half, hg = threadIdx.x / half;
    if (hg >= groups) return;
    float c = 1.f, s = 0.f;
    if (inv_freq) {
        float theta = (float)positions[t] * inv_freq[i];
        c = cosf(theta);
        s = sinf(theta);
    }
    if (inv_freq) {
        T* qr = q + (size_t)t * q_stride;
        for (int head = hg; head < H; head += groups) {
            T* x = qr + (size_t)head * hd;
            float a = ld_f(x + i), b = ld_f(x + half + i);
            st_f(x + i, a * c - b * s);
            st_f(x + half + i, b * c + a * s);
        }
    }
    if (!k) return;
    const int slot = slots ? slots[t] : -1;
    const size_t page = slot >= 0 ? (size_t)(slot / page_size) : 0;
    const int off = slot >= 0 ? slot % page_size : 0;
    for (int kh = hg; kh < KV; kh += groups) {
        T* x = k + (size_t)t * k_stride + (size_t)kh * hd;
        float a = ld_f(x + i), b = ld_f(x + half + i);
        float ra = a, rb = b;
        if (inv_freq) {
            ra = a * c - b * s;
            rb = b * c + a * s;
            st_f(x + i, ra);
            st_f(x + half + i, rb);
        }
        if (slot >= 0) {
            size_t base = ((page * KV + kh) * page_size + off) * (size_t)hd;
            const T* vr = v + (size_t)t * v_stride + (size_t)kh * hd;
            st_f(kcache + base + i, ra);
            st_f(kcache + base + half + i, rb);
            vcache[base + i] = vr[i];
            vcache[base + half + i] = vr[half + i];
        }
    }
}

// The same with 16-byte accesses, ROPE_TOK tokens per block: every thread takes 16-byte pieces of
// heads: it first requests all of its pieces (the first half of a head, the half that pairs with it
// and, for a k head, the pieces of v that go to the cache with it), so that a block has its whole
// traffic in flight at once; while they are on their way the tokens' sines and cosines go to shared
// memory once; then the pieces are rotated and stored. Needs 16-byte aligned rows.
constexpr int ROPE_TOK = 4;
constexpr int ROPE_THREADS = 256;
constexpr int ROPE_MAX_UNITS = 4;                  // pieces per thread handled in one go

template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_write_token_vec_kernel(T* __restrict__ q, long long q_stride, T* __restrict__ k, long long k_stride,
                               const T* __restrict__ v, long long v_stride, const int* __restrict__ positions,
                               const int* __restrict__ slots, const float* __restrict__ inv_freq, T* __restrict__ kcache,
                               T* __restrict__ vcache, int T_, int H, int KV, int hd, int page_size) {
    constexpr int E = 16 / sizeof(T);              // elements per 16 bytes
    pdl_launch_dependents();
    pdl_wait(4);
    extern __shared__ float s_cs[];                // [ROPE_TOK][half] cosines, then as many sines
    const int t0 = blockIdx.x * ROPE_TOK;
    const int ntok = min(ROPE_TOK, T_ - t0);
    const int half = hd >> 1;
    float* sc = s_cs;
    float* ss = s_cs + ROPE_TOK * half;
    const int chunks = half / E;                   // 16-byte pieces per half head
    const int heads = H + (k ? KV : 0);            // q heads, then k heads
    const int per_tok = heads * chunks;
    const int total = ntok * per_tok;
    uint4 ua[ROPE_MAX_UNITS], ub[ROPE_MAX_UNITS], va[ROPE_MAX_UNITS], vb[ROPE_MAX_UNITS];
    T* pa[ROPE_MAX_UNITS];
    long long cb[ROPE_MAX_UNITS];                  // where in the cache a piece of a k head (and of its v) goes; -1: nowhere
    // every piece a thread handles in one round is requested before anything is computed
    auto load_round = [&](int base) {
#pragma unroll
        for (int j = 0; j < ROPE_MAX_UNITS; ++j) {
            const int u = base + j * ROPE_THREADS + threadIdx.x;
            pa[j] = nullptr;
            cb[j] = -1;
            if (u < total) {
                const int tt = u / per_tok, r = u - tt * per_tok, head = r / chunks, ch = r - head * chunks;
                pa[j] = head < H ? q + (size_t)(t0 + tt) * q_stride + (size_t)head * hd + ch * E
                                 : k + (size_t)(t0 + tt) * k_stride + (size_t)(head - H) * hd + ch * E;
                ua[j] = *reinterpret_cast<const uint4*>(pa[j]);
                ub[j] = *reinterpret_cast<const uint4*>(pa[j] + half);
                if (head >= H) {
                    const int kh = head - H;
                    const int slot = slots ? slots[t0 + tt] : -1;
                    if (slot >= 0) {
                        cb[j] = (long long)(((((size_t)(slot / page_size)) * KV + kh) * page_size + slot % page_size) * (size_t)hd) + ch * E;
                        const T* vr = v + (size_t)(t0 + tt) * v_stride + (size_t)kh * hd + ch * E;
                        va[j] = *reinterpret_cast<const uint4*>(vr);
                        vb[j] = *reinterpret_cast<const uint4*>(vr + half);
                    }
                }
            }
        }
    };
    auto finish_round = [&](int base) {
#pragma unroll
        for (int j = 0; j < ROPE_MAX_UNITS; ++j) {
            const int u = base + j * ROPE_THREADS + threadIdx.x;
            if (u >= total) continue;
            const int tt = u / per_tok, r = u - tt * per_tok, head = r / chunks, ch = r - head * chunks;
            uint4 ra = ua[j], rb = ub[j];
            if (inv_freq) {
                const T* a = reinterpret_cast<const T*>(&ua[j]);
                const T* b = reinterpret_cast<const T*>(&ub[j]);
                T* oa = reinterpret_cast<T*>(&ra);
                T* ob = reinterpret_cast<T*>(&rb);
                const float* c = sc + tt * half + ch * E;
                const float* sn = ss + tt * half + ch * E;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const float x = ld_f(a + e), y = ld_f(b + e);
                    st_f(oa + e, x * c[e] - y * sn[e]);
                    st_f(ob + e, y * c[e] + x * sn[e]);
                }
                *reinterpret_cast<uint4*>(pa[j]) = ra;
                *reinterpret_cast<uint4*>(pa[j] + half) = rb;
            }
            if (cb[j] >= 0) {
                *reinterpret_cast<uint4*>(kcache + cb[j]) = ra;
                *reinterpret_cast<uint4*>(kcache + cb[j] + half) = rb;
                *reinterpret_cast<uint4*>(vcache + cb[j]) = va[j];
                *reinterpret_cast<uint4*>(vcache + cb[j] + half) = vb[j];
            }
        }
    };
    load_round(0);
    // the tokens' cosines and sines, while the first round's pieces are on their way
    for (int u = threadIdx.x; u < ntok * half; u += ROPE_THREADS) {
        const int tt = u / half, i = u - tt * half;
        float c = 1.f, s = 0.f;
        if (inv_freq) {
            float theta = (float)positions[t0 + tt] * inv_freq[i];
            c = cosf(theta);
            s = sinf(theta);
        }
        sc[u] = c;
        ss[u] = s;
    }
    __syncthreads();
    finish_round(0);
    for (int base = ROPE_THREADS * ROPE_MAX_UNITS; base < total; base += ROPE_THREADS * ROPE_MAX_UNITS) {
        load_round(base);
        finish_round(base);
    }
}

VOB_EXPORT int vob_rope_kv_write(void* q, long long q_stride, void* k, long long k_stride, const void* v,
                                 long long v_stride, const int* positions, const int* slots,
                                 const float* inv_freq, void* kcache, void* vcache, int code, int T, int H,
                                 int KV, int hd, int page_size, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || (hd & 1) || H <= 0 || KV < 0 || page_size <= 0) return VOB_ERR_BAD_ARG;
    if (k && slots && (!kcache || !vcache || !v)) return VOB_ERR_BAD_ARG;
    const int esz = code == VOB_BF16 ? 2 : 4;
    auto aligned = [&](const void* p, long long stride) { return !p || (((uintptr_t)p & 15) == 0 && (stride * esz) % 16 == 0); };
    if (T >= 64 && (hd / 2) % (16 / esz) == 0 && aligned(q, q_stride) && aligned(k, k_stride) && aligned(v, v_stride) &&
        aligned(kcache, hd) && aligned(vcache, hd)) {
        // many tokens, 16-byte aligned rows: sines and cosines once per token, 16-byte accesses
        VOB_DISPATCH_ELEM(code, return vob_launch(rope_kv_write_token_vec_kernel<ElemT>, dim3((T + ROPE_TOK - 1) / ROPE_TOK),
            dim3(ROPE_THREADS), (size_t)ROPE_TOK * hd * sizeof(float), stream, (ElemT*)q, q_stride, (ElemT*)k, k_stride,
            (const ElemT*)v, v_stride, positions, slots, inv_freq, (ElemT*)kcache, (ElemT*)vcache, T, H, KV, hd, page_size));
    }
    if (T >= 64 && hd / 2 <= 128) {
        // many tokens: a block per token, sines and cosines shared across heads
        VOB_DISPATCH_ELEM(code, return vob_launch(rope_kv_write_token_kernel<ElemT>, dim3(T), dim3(128), 0, stream,
            (ElemT*)q, q_stride, (ElemT*)k, k_stride, (const ElemT*)v, v_stride, positions, slots, inv_freq,
            (ElemT*)kcache, (ElemT*)vcache, H, KV, hd, page_size));
    }
    int pairs = (H + (k ? KV : 0)) * (hd / 2);
    dim3 grid(T, (pairs + 127) / 128);
    if (grid.y > 65535) return VOB_ERR_UNSUPPORTED;
    VOB_DISPATCH_ELEM(code, return vob_launch(rope_kv_write_kernel<ElemT>, grid, dim3(128), 0, stream,
        (ElemT*)q, q_stride, (ElemT*)k, k_stride, (const ElemT*)v, v_stride, positions, slots, inv_freq,
        (ElemT*)kcache, (ElemT*)vcache, H, KV, hd, page_size));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// SwiGLU: out[t, j] = gate / (1 + exp(-gate)) * up, gate = in[t, j], up = in[t, I + j]
// (divide, then multiply by up, as crates/engine/src/backend/cpu/mod.rs:341-349). The input is
// the output of one fused [gate; up] matrix product, row stride `in_stride` elements.
// Launch: grid (T, ceil(I/256)). Bound: memory.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out, int I) {
    pdl_launch_dependents();
    pdl_wait(5);
    int j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j >= I) return;
    const T* r = in + (size_t)blockIdx.x * in_stride;
    float g = ld_f(r + j), u = ld_f(r + I + j);
    st_f(out + (size_t)blockIdx.x * I + j, g / (1.0f + expf(-g)) * u);
}

// 16 bytes per load: 8 bfloat16 or 4 float per thread (I a multiple of that, rows 16-byte aligned).
template <typename T, int N>
__global__ void swiglu_vec_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out, int I) {
    pdl_launch_dependents();
    pdl_wait(5);
    int j = (blockIdx.y * blockDim.x + threadIdx.x) * N;
    if (j >= I) return;
    const T* r = in + (size_t)blockIdx.x * in_stride;
    uint4 gu = *reinterpret_cast<const uint4*>(r + j);
    uint4 uu = *reinterpret_cast<const uint4*>(r + I + j);
    const T* g = reinterpret_cast<const T*>(&gu);
    const T* u = reinterpret_cast<const T*>(&uu);
    uint4 ov;
    T* o = reinterpret_cast<T*>(&ov);
#pragma unroll
    for (int e = 0; e < N; ++e) {
        float gf = ld_f(g + e), uf = ld_f(u + e);
        st_f(o + e, gf / (1.0f + expf(-gf)) * uf);
    }
    *reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * I + j) = ov;
}

template <typename T>
static int launch_swiglu(const void* in, long long in_stride, void* out, int T_rows, int I, cudaStream_t stream) {
    constexpr int N = 16 / sizeof(T);
    bool vec = (I % N == 0) && (in_stride % N == 0) && (((uintptr_t)in | (uintptr_t)out) % 16 == 0);
    if (vec) {
        int per = 256 * N;
        if ((I + per - 1) / per > 65535) return VOB_ERR_UNSUPPORTED;
        dim3 grid(T_rows, (I + per - 1) / per);
        return vob_launch(swiglu_vec_kernel<T, N>, grid, dim3(256), 0, stream, (const T*)in, in_stride, (T*)out, I);
    } else {
        if ((I + 255) / 256 > 65535) return VOB_ERR_UNSUPPORTED;
        dim3 grid(T_rows, (I + 255) / 256);
        return vob_launch(swiglu_kernel<T>, grid, dim3(256), 0, stream, (const T*)in, in_stride, (T*)out, I);
    }
}

VOB_EXPORT int vob_swiglu(const void* in, long long in_stride, void* out, int code, int T, int I,
                          cudaStream_t stream) {
    if (T <= 0) return 0;
    if (I <= 0) return VOB_ERR_BAD_ARG;
    if (code == VOB_F32) return launch_swiglu<float>(in, in_stride, out, T, I, stream);
    if (code == VOB_BF16) return launch_swiglu<__nv_bfloat16>(in, in_stride, out, T, I, stream);
    return VOB_ERR_BAD_ARG;
}
