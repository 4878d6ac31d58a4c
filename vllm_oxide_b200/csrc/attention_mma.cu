// Tensor-core attention over the paged cache for the bfloat16 engine: one kernel for portions of
// prompts (and mixed batches), one for steps of single decoded tokens.
//
// Math (as csrc/attention.cu; reference crates/engine/src/backend/cpu/attention.rs:76-128):
//   s_j = (q . K_j) * scale over keys first..p, softmax in float32 with a running maximum,
//   out = sum_j softmax_j V_j. Q K^T and P V run on the tensor cores (mma.sync m16n8k16, bf16 in,
//   float32 accumulate); P is rounded to bfloat16 for the second product; everything between is
//   float32 (exp2 of scores pre-multiplied by scale * log2 e).
//
// Grouped-query packing: the G = H / KV query heads that share a kv head are stacked as rows, so a
// K/V tile is read once per kv head instead of once per head. Row rr of a request's row space is
// token rr / G (position context_len + rr / G) and head kvh * G + rr % G.
//
// K/V tiles of 64 keys are gathered page by page with 16-byte cp.async copies into padded shared
// memory (row stride head_dim + 8 elements keeps ldmatrix free of bank conflicts), double buffered.
// Keys outside [first, p] are never read from global memory (their pages may have been given
// back): their shared-memory rows are zero-filled and their scores masked to -inf.
//
// Kernels take head_dim 64 or 128, page sizes that divide 64, G <= 16 for the decode kernel;
// the launcher refuses anything else (the caller then uses the general kernel).
#include "common.cuh"
VOB_PDL_SWITCH(attention_mma)

namespace {

constexpr int BN = 64;        // keys per tile
constexpr int NTHREADS = 128;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special-function unit (two units in the last place: far inside what a bfloat16
// probability needs); -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Gather one tile of 64 keys (K and V of one kv head) into shared memory. Keys outside
// [lo, hi) are zero-filled and never touched in global memory. Page numbers come from `s_pages`,
// this block's copy of its request's block-table entries starting at logical page `page0` (a
// global lookup per key would put a dependent L2 round trip in front of every copy); page sizes
// are powers of two (they divide 64), so positions split into page and offset by shift and mask.
template <int HD>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* sK, __nv_bfloat16* sV, const __nv_bfloat16* __restrict__ kc,
                                             const __nv_bfloat16* __restrict__ vc, const int* s_pages, int page0, int kvh,
                                             int KV, int page_shift, int tile_start, int lo, int hi) {
    constexpr int LD = HD + 8;
    constexpr int CH = HD / 8;                 // 16-byte pieces per key
    constexpr int KEYS_PER_PASS = NTHREADS / CH;
    const int ch = threadIdx.x % CH;
    const int k0 = threadIdx.x / CH;
    const int page_size = 1 << page_shift;
#pragma unroll
    for (int key = k0; key < BN; key += KEYS_PER_PASS) {
        int j = tile_start + key;
        __nv_bfloat16* dk = sK + key * LD + ch * 8;
        __nv_bfloat16* dv = sV + key * LD + ch * 8;
        if (j >= lo && j < hi) {
            int page = s_pages[(j >> page_shift) - page0];
            size_t off = ((((size_t)page * KV + kvh) << page_shift) + (j & (page_size - 1))) * HD + ch * 8;
            cp_async16(dk, kc + off);
            cp_async16(dv, vc + off);
        } else {
            *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(dv) = make_uint4(0, 0, 0, 0);
        }
    }
}

// S (16 rows x 8*NB keys) += Q K^T for the n-blocks [nb0, nb0+NB) of the tile in sK.
template <int HD, int NB>
__device__ __forceinline__ void qk_tile(float (&s)[NB][4], const uint32_t (&qf)[HD / 16][4], const __nv_bfloat16* sK, int nb0) {
    constexpr int LD = HD + 8;
    int lane = threadIdx.x & 31;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int i = 0; i < 4; ++i) s[nb][i] = 0.f;
#pragma unroll
        for (int k2 = 0; k2 < HD / 32; ++k2) {
            uint32_t r[4];
            ldmatrix_x4(r, sK + ((nb0 + nb) * 8 + (lane & 7)) * LD + k2 * 32 + (lane >> 3) * 8);
            mma_bf16(s[nb], qf[2 * k2], r[0], r[1]);
            mma_bf16(s[nb], qf[2 * k2 + 1], r[2], r[3]);
        }
    }
}

// O (16 x HD) += P V for NK slices of 16 keys starting at key slice ks0 of the tile in sV.
template <int HD, int NK>
__device__ __forceinline__ void pv_tile(float (&o)[HD / 8][4], const uint32_t (&pa)[NK][4], const __nv_bfloat16* sV, int ks0) {
    constexpr int LD = HD + 8;
    int lane = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < NK; ++kk) {
#pragma unroll
        for (int n2 = 0; n2 < HD / 16; ++n2) {
            uint32_t r[4];
            ldmatrix_x4_trans(r, sV + ((ks0 + kk) * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + n2 * 16 + (lane >> 4) * 8);
            mma_bf16(o[2 * n2], pa[kk], r[0], r[1]);
            mma_bf16(o[2 * n2 + 1], pa[kk], r[2], r[3]);
        }
    }
}

// Mask, running maximum, exponentials; returns P as A-fragments. s holds NB n-blocks of 8 keys
// starting at key index key0; this thread's rows are r and r+8 with limits [lo, pos]. With MASK
// false the caller knows that every key of the tile is visible to every row of the warp.
template <int NB, int HDN, bool MASK>
__device__ __forceinline__ void softmax_step(float (&s)[NB][4], uint32_t (&pa)[NB / 2][4], float (&o)[HDN][4],
                                             float (&m)[2], float (&l)[2], int key0, const int (&lo)[2],
                                             const int (&pos)[2], float scale_log2) {
    int lane = threadIdx.x & 31;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int h = i >> 1;
            if (MASK) {
                int j = key0 + nb * 8 + (lane & 3) * 2 + (i & 1);
                if (!(j >= lo[h] && j <= pos[h])) s[nb][i] = -INFINITY;
            }
            mx[h] = fmaxf(mx[h], s[nb][i]);
        }
    }
    float alpha[2], msafe[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        float mn = fmaxf(m[h], mx[h] * scale_log2);   // scale > 0: the maximum of the scaled scores
        msafe[h] = mn == -INFINITY ? 0.f : mn;
        alpha[h] = fast_exp2(m[h] - msafe[h]);         // m = -inf: 0
        m[h] = mn;
        l[h] *= alpha[h];
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float p = fast_exp2(fmaf(s[nb][i], scale_log2, -msafe[i >> 1]));
            s[nb][i] = p;
            l[i >> 1] += p;                           // this thread's share; the quad is summed at the end
        }
    }
#pragma unroll
    for (int n = 0; n < HDN; ++n) {
        o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
        o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < NB / 2; ++kk) {
        pa[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    }
}

// ---------------------------------------------------------------------------------------------
// Portions of prompts and mixed batches. Grid (row tiles, requests, kv heads); a block of 4 warps
// owns 64 rows of one request's row space (16 rows per warp) and walks the key tiles that any of
// its rows can see. Blocks beyond a request's rows leave at once.
// Bound: tensor-core and exp throughput for long portions; for short ones the K/V reads.
// ---------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(NTHREADS)
attn_prefill_mma_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, __nv_bfloat16* __restrict__ out,
                        long long out_stride, const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                        const int* __restrict__ block_tables, int max_pages, const int* __restrict__ seq_starts,
                        const int* __restrict__ context_lens, int H, int KV, int page_shift, int window, float scale_log2) {
    constexpr int LD = HD + 8;
    constexpr int BM = 64;
    pdl_launch_dependents();
    pdl_wait(7);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sK0 = sQ + BM * LD;
    __nv_bfloat16* sV0 = sK0 + 2 * BN * LD;
    int* s_pages = reinterpret_cast<int*>(sV0 + 2 * BN * LD);            // [max_pages]

    const int G = H / KV;
    // Blocks are handed out in the order x, y, z: the kv head runs fastest and the row tile slowest,
    // later row tiles (which see more keys) first, so that over the whole grid the long blocks
    // start first and the short ones fill the gaps behind them.
    const int kvh = blockIdx.x, seq = blockIdx.y;
    const int row0 = seq_starts[seq];
    const int n_new = seq_starts[seq + 1] - row0;
    const int total_rows = n_new * G;
    const int tile_row0 = (gridDim.z - 1 - blockIdx.z) * BM;
    if (tile_row0 >= total_rows) return;
    const int ctx = context_lens[seq];
    const int* bt = block_tables + (size_t)seq * max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // rows of this block -> shared memory (zero for rows beyond the request)
    for (int c = threadIdx.x; c < BM * (HD / 8); c += NTHREADS) {
        int r = c / (HD / 8), ch = c - r * (HD / 8);
        int rr = tile_row0 + r;
        __nv_bfloat16* dst = sQ + r * LD + ch * 8;
        if (rr < total_rows) {
            int tok = rr / G, head = kvh * G + rr % G;
            cp_async16(dst, q + (size_t)(row0 + tok) * q_stride + (size_t)head * HD + ch * 8);
        } else {
            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
    // key range any row of the block reads
    const int last_rr = min(tile_row0 + BM, total_rows) - 1;
    const int hi = ctx + last_rr / G + 1;
    const int first_tok_pos = ctx + tile_row0 / G;
    const int lo_blk = window > 0 ? max(0, first_tok_pos + 1 - window) : 0;
    const int t_begin = lo_blk / BN, t_end = (hi + BN - 1) / BN;
    // this block's pages: logical pages [page0, page_end) of the request, one coalesced read
    const int page0 = lo_blk >> page_shift, page_end = ((hi - 1) >> page_shift) + 1;
    for (int i = threadIdx.x; i < page_end - page0; i += NTHREADS) s_pages[i] = bt[page0 + i];
    __syncthreads();

    load_kv_tile<HD>(sK0, sV0, kc, vc, s_pages, page0, kvh, KV, page_shift, t_begin * BN, lo_blk, hi);
    cp_async_commit();

    int pos[2], lo[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int rr = tile_row0 + warp * 16 + (lane >> 2) + h * 8;
        pos[h] = rr < total_rows ? ctx + rr / G : -1;
        lo[h] = window > 0 ? max(0, pos[h] + 1 - window) : 0;
    }
    // the warp's position range: tiles beyond its last position are skipped, tiles wholly inside
    // every row's [lo, pos] need no mask (rows beyond the request count as position -1: masked)
    int warp_last_pos = max(pos[0], pos[1]), warp_first_pos = min(pos[0], pos[1]), warp_max_lo = max(lo[0], lo[1]);
#pragma unroll
    for (int x = 4; x < 32; x <<= 1) {
        warp_last_pos = max(warp_last_pos, __shfl_xor_sync(0xffffffffu, warp_last_pos, x));
        warp_first_pos = min(warp_first_pos, __shfl_xor_sync(0xffffffffu, warp_first_pos, x));
        warp_max_lo = max(warp_max_lo, __shfl_xor_sync(0xffffffffu, warp_max_lo, x));
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
    uint32_t qf[HD / 16][4];

    for (int t = t_begin; t < t_end; ++t) {
        int buf = (t - t_begin) & 1;
        __nv_bfloat16* sK = sK0 + buf * BN * LD;
        __nv_bfloat16* sV = sV0 + buf * BN * LD;
        cp_async_wait<0>();
        __syncthreads();                       // tile t (and Q) visible; everyone is done with tile t-1
        if (t + 1 < t_end) {
            load_kv_tile<HD>(sK0 + (buf ^ 1) * BN * LD, sV0 + (buf ^ 1) * BN * LD, kc, vc, s_pages, page0, kvh, KV, page_shift,
                             (t + 1) * BN, lo_blk, hi);
            cp_async_commit();
        }
        if (t == t_begin) {
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk)
                ldmatrix_x4(qf[kk], sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk * 16 + (lane >> 4) * 8);
        }
        // a warp whose rows all lie before this tile's first key has nothing to do here
        if (t * BN <= warp_last_pos) {
            float s[8][4];
            qk_tile<HD, 8>(s, qf, sK, 0);
            uint32_t pa[4][4];
            // no masking where the whole tile lies inside [lo, pos] of every row of the warp
            if ((t + 1) * BN - 1 <= warp_first_pos && t * BN >= warp_max_lo)
                softmax_step<8, HD / 8, false>(s, pa, o, m, l, t * BN, lo, pos, scale_log2);
            else
                softmax_step<8, HD / 8, true>(s, pa, o, m, l, t * BN, lo, pos, scale_log2);
            pv_tile<HD, 4>(o, pa, sV, 0);
        }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int rr = tile_row0 + warp * 16 + (lane >> 2) + h * 8;
        if (rr >= total_rows) continue;
        int tok = rr / G, head = kvh * G + rr % G;
        float inv = 1.0f / l[h];
        __nv_bfloat16* op = out + (size_t)(row0 + tok) * out_stride + (size_t)head * HD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
            *reinterpret_cast<uint32_t*>(op + n * 8) = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
    }
}

constexpr int DEC_MIN_TILES = 3;            // measured on whole decode steps at batch 1: 8,192 keys 0.808 ms with 3, 0.838 with 2, 0.812 with 4
constexpr int DEC_MAX_SPLITS_WIDE = 64;

// The block of a request and kv head that arrives last adds the partials of all `splits` blocks
// up (merge through global memory). Everything is fetched with independent loads: first every
// partial's maxima and sums, from which each row's weights follow; then the values, a thread
// taking four neighbouring dims over one half of the partials, in rank order. `scratch` is the
// block's shared memory behind q; `out` points at the group's first head. Not inlined: the
// kernel's main path keeps its registers.
template <int HD>
__device__ __noinline__ void merge_partials(const float* __restrict__ all, int splits, int G, float* scratch,
                                            __nv_bfloat16* __restrict__ out) {
    constexpr int PART = 16 * HD + 32;
    float* ml = scratch;                                    // [splits][32]: 16 maxima, 16 sums
    float* fk = ml + DEC_MAX_SPLITS_WIDE * 32;              // [splits][16]: weight of partial k in row r
    float* hs = fk + DEC_MAX_SPLITS_WIDE * 16;              // [2][16 * HD]: the two halves' sums
    float* Lrow = hs + 2 * 16 * HD;                         // [16]
    static_assert(DEC_MAX_SPLITS_WIDE * 48 + 2 * 16 * HD + 16 <= 128 + 4 * 16 * HD + 16 * HD + 32, "merge scratch exceeds the combine area");
    for (int i = threadIdx.x; i < splits * 32; i += NTHREADS) ml[i] = __ldcg(all + (size_t)(i >> 5) * PART + 16 * HD + (i & 31));
    __syncthreads();
    if (threadIdx.x < G) {
        const int r = threadIdx.x;
        float M = -INFINITY;
        for (int k = 0; k < splits; ++k) M = fmaxf(M, ml[k * 32 + r]);
        const float Ms = M == -INFINITY ? 0.f : M;
        float L = 0.f;
        for (int k = 0; k < splits; ++k) {
            const float f = exp2f(ml[k * 32 + r] - Ms);
            fk[k * 16 + r] = f;
            L += f * ml[k * 32 + 16 + r];
        }
        Lrow[r] = L;
    }
    __syncthreads();
    const int items = G * HD / 4, k_half = splits / 2;
    for (int it = threadIdx.x; it < 2 * items; it += NTHREADS) {
        const int second = it >= items, e = (it - second * items) * 4, r = e / HD;
        const int k0 = second ? k_half : 0, k1 = second ? splits : k_half;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int k = k0; k < k1; ++k) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(all + (size_t)k * PART + e));
            const float f = fk[k * 16 + r];
            acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
        }
        *reinterpret_cast<float4*>(hs + second * 16 * HD + e) = acc;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < G * HD; e += NTHREADS) {
        const float L = Lrow[e / HD];
        out[e] = __float2bfloat16_rn(L > 0.f ? (hs[e] + hs[16 * HD + e]) / L : 0.f);
    }
}

// ---------------------------------------------------------------------------------------------
// Steps of single decoded tokens. Grid (requests, kv heads, splits): a block reads its share of
// the request's key tiles once for all G heads of the group; its 4 warps split every tile's 64
// keys (16 each) and combine through shared memory. The `splits` blocks of one (request, kv
// head) form a thread-block cluster: every block finishes a share of the outputs, and each sends
// the pieces of its unnormalised partial (running maximum, sum, weighted values) to the blocks
// that finish them, by stores into their shared memory (a region that nothing else uses, so a
// fast peer may write while the owner still works on its tiles); the cluster meets at a barrier
// once, and every block then adds up what it was sent in rank order (a fixed order, so the result
// does not depend on timing) and leaves: nobody reads a peer's memory, so nobody has to wait for
// the others to finish. K/V tiles go
// through a cp.async ring of three stages (two when the grid is so large that the smaller
// footprint lets one more block live on an SM). Bound: the K/V reads (memory).
//
// Few requests with long contexts would leave most SMs idle with 8 blocks each. For them the
// grid has up to 64 splits and no cluster (`partials` is given): a request uses as many of its
// blocks as it has tiles for (at least DEC_MIN_TILES each; the others leave at once), every
// block writes its partial to global memory and counts itself in, and the block that arrives
// last adds the partials up in rank order and puts the counter back to zero. Nobody waits.
// ---------------------------------------------------------------------------------------------

// Shared memory of a decode block: the K/V ring (used again for the combine of the four warps),
// then what the cluster's peers send, then the block's page list.
template <int HD, int DEC_STAGES> __host__ __device__ constexpr size_t decode_ring_bytes() {
    size_t ring = (size_t)(16 + 2 * DEC_STAGES * BN) * (HD + 8) * sizeof(__nv_bfloat16);
    size_t combine = 16 * (HD + 8) * sizeof(__nv_bfloat16) + (size_t)(128 + 4 * 16 * HD + 16 * HD + 32) * sizeof(float);
    return ((ring > combine ? ring : combine) + 15) / 16 * 16;
}
__host__ __device__ constexpr size_t decode_recv_bytes(int G, int HD) { return (size_t)(G * HD + 8 + 256) * sizeof(float); }

template <int HD, int DEC_STAGES>
__global__ void __launch_bounds__(NTHREADS)
attn_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, __nv_bfloat16* __restrict__ out,
                       long long out_stride, const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                       const int* __restrict__ block_tables, int max_pages, const int* __restrict__ positions,
                       int H, int KV, int page_shift, int window, float scale_log2, float* __restrict__ partials,
                       int* __restrict__ arrived) {
    constexpr int LD = HD + 8;
    constexpr int PART = 16 * HD + 32;                                          // floats of one block's partial
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int s_last;
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // 16 x LD
    __nv_bfloat16* sK0 = sQ + 16 * LD;                                          // DEC_STAGES x BN x LD
    __nv_bfloat16* sV0 = sK0 + DEC_STAGES * BN * LD;
    // what the peers of a cluster send this block: [splits][chunk] values, [8][16] maxima, [8][16] sums
    float* recv_val = reinterpret_cast<float*>(smem_raw + decode_ring_bytes<HD, DEC_STAGES>());
    float* recv_m = recv_val + (H / KV) * HD + 8;
    float* recv_l = recv_m + 128;
    // this block's pages (a launch without a cluster has no region for what peers send)
    int* s_pages = (!partials && gridDim.z > 1) ? reinterpret_cast<int*>(recv_l + 128) : reinterpret_cast<int*>(recv_val);

    // Positions and block tables were put on the device before this step's kernels began, and
    // every key but the newest was written by earlier steps: all of that may be read before the
    // wait, while the kernel in front (which writes the newest key and this step's q) still runs.
    const int G = H / KV;
    const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    int splits = gridDim.z;
    // every block of the cluster has started (and owns its shared memory) before anyone is sent
    // anything: arrive now, wait just before the first store to a peer
    if (!partials && splits > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    const int p = positions[seq];                 // one row per request: row index == request index
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* bt = block_tables + (size_t)seq * max_pages;
    const int hi = p + 1;
    const int lo_key = (p >= 0 && window > 0) ? max(0, p + 1 - window) : 0;
    const int t_first = lo_key / BN;
    const int n_tiles = p >= 0 ? (hi + BN - 1) / BN - t_first : 0;
    if (partials) {
        splits = max(1, min(splits, n_tiles / DEC_MIN_TILES));
        const int share = max(1, (n_tiles + splits - 1) / splits);
        splits = max(1, (n_tiles + share - 1) / share);      // no block without a tile
        if (split >= splits) return;                  // the whole block: this request has no tiles for it
    }
    const int per = (n_tiles + splits - 1) / splits;
    const int t_begin = t_first + split * per;
    const int t_end = min(t_first + n_tiles, t_begin + per);
    // this block's pages: those of its tiles, one coalesced read of the block table
    const int page0 = (t_begin * BN) >> page_shift;
    const int page_end = t_begin < t_end ? ((min(hi, t_end * BN) - 1) >> page_shift) + 1 : page0;
    for (int i = threadIdx.x; i < page_end - page0; i += NTHREADS) s_pages[i] = bt[page0 + i];
    __syncthreads();

    // prologue: the first DEC_STAGES - 1 tiles, one commit group each (empty groups keep the
    // count); tiles that end before the newest key go out before the wait, the rest after it
    int s_done = 0;
#pragma unroll
    for (int s = 0; s < DEC_STAGES - 1; ++s) {
        int t = t_begin + s;
        if (s_done == s && (t >= t_end || (t + 1) * BN <= p)) {
            if (t < t_end)
                load_kv_tile<HD>(sK0 + s * BN * LD, sV0 + s * BN * LD, kc, vc, s_pages, page0, kvh, KV, page_shift, t * BN, lo_key, hi);
            cp_async_commit();
            s_done = s + 1;
        }
    }
    pdl_wait(8);
    // q of this step: plain loads (it must be in shared memory before the first tile is used, and
    // it is too small to deserve a commit group of its own)
    for (int c = threadIdx.x; c < 16 * (HD / 8); c += NTHREADS) {
        int r = c / (HD / 8), ch = c - r * (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < G && p >= 0) v = *reinterpret_cast<const uint4*>(q + (size_t)seq * q_stride + (size_t)(kvh * G + r) * HD + ch * 8);
        *reinterpret_cast<uint4*>(sQ + r * LD + ch * 8) = v;
    }
#pragma unroll
    for (int s = 0; s < DEC_STAGES - 1; ++s) {
        if (s >= s_done) {
            int t = t_begin + s;
            if (t < t_end)
                load_kv_tile<HD>(sK0 + s * BN * LD, sV0 + s * BN * LD, kc, vc, s_pages, page0, kvh, KV, page_shift, t * BN, lo_key, hi);
            cp_async_commit();
        }
    }

    int pos[2], lo[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int r = (lane >> 2) + h * 8;
        pos[h] = r < G ? p : -1;
        lo[h] = lo_key;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
    uint32_t qf[HD / 16][4];

    for (int t = t_begin; t < t_end; ++t) {
        int buf = (t - t_begin) % DEC_STAGES;
        __nv_bfloat16* sK = sK0 + buf * BN * LD;
        __nv_bfloat16* sV = sV0 + buf * BN * LD;
        cp_async_wait<DEC_STAGES - 2>();        // tile t has landed (one newer group may be in flight)
        __syncthreads();                        // ... for every thread; and everyone is done with tile t-1
        {
            int tn = t + DEC_STAGES - 1;        // refill the buffer tile t-1 used
            int nb = (tn - t_begin) % DEC_STAGES;
            if (tn < t_end)
                load_kv_tile<HD>(sK0 + nb * BN * LD, sV0 + nb * BN * LD, kc, vc, s_pages, page0, kvh, KV, page_shift, tn * BN, lo_key, hi);
            cp_async_commit();
        }
        if (t == t_begin) {
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk)
                ldmatrix_x4(qf[kk], sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk * 16 + (lane >> 4) * 8);
        }
        float s[2][4];
        qk_tile<HD, 2>(s, qf, sK, warp * 2);                    // this warp's 16 keys of the tile
        uint32_t pa[1][4];
        softmax_step<2, HD / 8, true>(s, pa, o, m, l, t * BN + warp * 16, lo, pos, scale_log2);
        pv_tile<HD, 1>(o, pa, sV, warp);
    }
    cp_async_wait<0>();
    __syncthreads();                                            // K/V buffers are free: reuse them for the combine
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    float* cm = reinterpret_cast<float*>(sK0);                  // [4 warps][16 rows] max
    float* cl = cm + 64;                                        // [4][16] sum
    float* co = cl + 64;                                        // [4][16][HD]
    float* fin = co + 4 * 16 * HD;                              // this block's partial: [16][HD] values, [16] max, [16] sum
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int r = (lane >> 2) + h * 8;
        if ((lane & 3) == 0) { cm[warp * 16 + r] = m[h]; cl[warp * 16 + r] = l[h]; }
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            co[(warp * 16 + r) * HD + n * 8 + (lane & 3) * 2] = o[n][2 * h];
            co[(warp * 16 + r) * HD + n * 8 + (lane & 3) * 2 + 1] = o[n][2 * h + 1];
        }
    }
    __syncthreads();
    const bool push = splits > 1 && !partials;
    const int chunk = (G * HD + splits - 1) / splits;          // outputs each block of a cluster finishes
    if (push) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");       // the peers have started (they arrived at their start)
    for (int e = threadIdx.x; e < G * HD; e += NTHREADS) {
        int r = e / HD, d = e - r * HD;
        float M = fmaxf(fmaxf(cm[r], cm[16 + r]), fmaxf(cm[32 + r], cm[48 + r]));
        float Ms = M == -INFINITY ? 0.f : M;
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            float f = exp2f(cm[w * 16 + r] - Ms);
            acc += f * co[(w * 16 + r) * HD + d];
            L += f * cl[w * 16 + r];
        }
        if (splits == 1) {
            out[(size_t)seq * out_stride + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else if (push) {
            // to the block that finishes this output; the row's maximum and sum to every block
            const int owner = e / chunk;
            uint32_t dst;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(smem_u32(recv_val + split * chunk + (e - owner * chunk))), "r"(owner));
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst), "f"(acc) : "memory");
            if (d == 0) {
                for (int k = 0; k < splits; ++k) {
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(smem_u32(recv_m + split * 16 + r)), "r"(k));
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst), "f"(M) : "memory");
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst + 128 * 4), "f"(L) : "memory");
                }
            }
        } else {
            fin[r * HD + d] = acc;
            if (d == 0) { fin[16 * HD + r] = M; fin[16 * HD + 16 + r] = L; }
        }
    }
    if (splits > 1 && partials) {
        float* mine = partials + ((size_t)(seq * KV + kvh) * gridDim.z + split) * PART;
        __syncthreads();
        for (int e = threadIdx.x; e < G * HD; e += NTHREADS) mine[e] = fin[e];
        if (threadIdx.x < 32) mine[16 * HD + threadIdx.x] = fin[16 * HD + threadIdx.x];
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_last = atomicAdd(arrived + seq * KV + kvh, 1) == splits - 1;
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        merge_partials<HD>(partials + (size_t)(seq * KV + kvh) * gridDim.z * PART, splits, G, reinterpret_cast<float*>(sK0),
                           out + (size_t)seq * out_stride + (size_t)kvh * G * HD);
        if (threadIdx.x == 0) arrived[seq * KV + kvh] = 0;      // ready for the next launch
    } else if (splits > 1) {
        // what was sent is there once everyone has passed this barrier
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        const int total = G * HD;
        const int e0 = split * chunk, e1 = min(total, e0 + chunk);
        for (int e = e0 + threadIdx.x; e < e1; e += NTHREADS) {
            int r = e / HD, d = e - r * HD;
            float pm[8], pl[8], po[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                pm[k] = -INFINITY; pl[k] = 0.f; po[k] = 0.f;
                if (k < splits) { po[k] = recv_val[k * chunk + (e - e0)]; pm[k] = recv_m[k * 16 + r]; pl[k] = recv_l[k * 16 + r]; }
            }
            float M = -INFINITY;
#pragma unroll
            for (int k = 0; k < 8; ++k) M = fmaxf(M, pm[k]);
            float Ms = M == -INFINITY ? 0.f : M;
            float acc = 0.f, L = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) {                       // rank order; ranks beyond the last add zero
                float f = exp2f(pm[k] - Ms);
                acc += f * po[k];
                L += f * pl[k];
            }
            out[(size_t)seq * out_stride + (size_t)(kvh * G + r) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        }
        // nothing of this block is read by a peer: it may leave at once
    }
}

template <int HD> constexpr size_t prefill_smem() { return (size_t)(64 + 4 * BN) * (HD + 8) * sizeof(__nv_bfloat16); }
template <int HD, int DEC_STAGES> size_t decode_smem(int G, bool cluster) {
    return decode_ring_bytes<HD, DEC_STAGES>() + (cluster ? decode_recv_bytes(G, HD) : 0);
}

inline int log2_exact(int v) {
    int s = 0;
    while ((1 << s) < v) ++s;
    return s;
}

// Raise a kernel's dynamic shared-memory limit when a launch needs more than any before it.
template <typename Kern>
int ensure_smem(Kern kernel, size_t bytes, size_t* configured) {
    if (bytes > 227 * 1024) return VOB_ERR_UNSUPPORTED;
    if (bytes > *configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return (int)e;
        *configured = bytes;
    }
    return 0;
}

template <int HD>
int launch_prefill(const void* q, long long q_stride, void* out, long long out_stride, const void* kc, const void* vc,
                   const int* bt, int max_pages, const int* seq_starts, const int* context_lens, int S, int max_new,
                   int H, int KV, int page_size, int window, float scale, cudaStream_t stream) {
    static size_t configured = 0;
    size_t smem = prefill_smem<HD>() + (size_t)max_pages * sizeof(int);      // tiles + this request's page list
    int e = ensure_smem(attn_prefill_mma_kernel<HD>, smem, &configured);
    if (e) return e;
    int G = H / KV;
    const long long row_tiles = ((long long)max_new * G + 63) / 64;
    if (row_tiles > 65535) return VOB_ERR_UNSUPPORTED;
    dim3 grid(KV, S, (unsigned)row_tiles);
    return vob_launch(attn_prefill_mma_kernel<HD>, grid, dim3(NTHREADS), smem, stream,
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)kc,
        (const __nv_bfloat16*)vc, bt, max_pages, seq_starts, context_lens, H, KV, log2_exact(page_size), window,
        scale * 1.4426950408889634f);
}

template <int HD, int ST>
int launch_decode_st(const void* q, long long q_stride, void* out, long long out_stride, const void* kc, const void* vc,
                     const int* bt, int max_pages, const int* positions, int S, int H, int KV, int page_size, int window,
                     float scale, int splits, float* partials, int* arrived, cudaStream_t stream) {
    static size_t configured = 0;
    // a block's page list: its share of the tiles of the longest request the block table can hold
    // (a request with few tiles uses fewer blocks, but then the tiles are few)
    long long tiles_max = ((long long)max_pages * page_size + BN - 1) / BN;
    long long per_max = (tiles_max + splits - 1) / splits;
    if (partials && per_max < 2 * DEC_MIN_TILES) per_max = 2 * DEC_MIN_TILES;
    long long pages_cta = per_max * (BN / page_size) + 1;
    size_t smem = decode_smem<HD, ST>(H / KV, splits > 1 && !partials) + (size_t)pages_cta * sizeof(int);
    int e = ensure_smem(attn_decode_mma_kernel<HD, ST>, smem, &configured);
    if (e) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S, KV, splits);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = partials ? 1 : splits;      // the blocks that share one (request, kv head)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_vob_pdl ? 2 : 1;
    cudaError_t ce = cudaLaunchKernelEx(&cfg, attn_decode_mma_kernel<HD, ST>, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out,
                                        out_stride, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, bt, max_pages, positions,
                                        H, KV, log2_exact(page_size), window, scale * 1.4426950408889634f, partials, arrived);
    return ce != cudaSuccess ? (int)ce : vob_launch_status();
}

template <int HD>
int launch_decode(const void* q, long long q_stride, void* out, long long out_stride, const void* kc, const void* vc,
                  const int* bt, int max_pages, const int* positions, int S, int H, int KV, int page_size, int window,
                  float scale, int splits, float* partials, int* arrived, cudaStream_t stream) {
    static int num_sms = 0;
    if (!num_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (num_sms <= 0) num_sms = 148;
    }
    // three stages while every block of the grid can be resident at once with them; else two
    long long blocks = (long long)S * KV * splits;
    long long fit3 = (long long)num_sms * ((227 * 1024) / (long long)(decode_smem<HD, 3>(H / KV, splits > 1 && !partials) + 2048));
    if (blocks <= fit3)
        return launch_decode_st<HD, 3>(q, q_stride, out, out_stride, kc, vc, bt, max_pages, positions, S, H, KV, page_size,
                                       window, scale, splits, partials, arrived, stream);
    return launch_decode_st<HD, 2>(q, q_stride, out, out_stride, kc, vc, bt, max_pages, positions, S, H, KV, page_size,
                                   window, scale, splits, partials, arrived, stream);
}

bool sizes_ok(int H, int KV, int hd, int page_size) {
    return (hd == 64 || hd == 128) && KV > 0 && H % KV == 0 && page_size > 0 && BN % page_size == 0;
}

}  // namespace

// 1 if the tensor-core kernels take these sizes (decode additionally needs H / KV <= 16).
VOB_EXPORT int vob_attn_mma_supported(int H, int KV, int hd, int page_size, int decode) {
    if (!sizes_ok(H, KV, hd, page_size)) return 0;
    if (decode && H / KV > 16) return 0;
    return 1;
}

VOB_EXPORT int vob_attn_prefill_mma(const void* q, long long q_stride, void* out, long long out_stride, const void* kcache,
                                    const void* vcache, const int* block_tables, int max_pages, const int* seq_starts,
                                    const int* context_lens, int S, int max_new, int H, int KV, int hd, int page_size,
                                    int window, float scale, cudaStream_t stream) {
    if (S <= 0 || max_new <= 0) return 0;
    if (!sizes_ok(H, KV, hd, page_size)) return VOB_ERR_UNSUPPORTED;
    if (q_stride % 8 != 0 || out_stride % 2 != 0 || S > 65535 || KV > 65535) return VOB_ERR_BAD_ARG;
    if (hd == 64) return launch_prefill<64>(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, seq_starts,
                                           context_lens, S, max_new, H, KV, page_size, window, scale, stream);
    return launch_prefill<128>(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, seq_starts,
                               context_lens, S, max_new, H, KV, page_size, window, scale, stream);
}

// `splits` (1..8) blocks share each (request, kv head) as one cluster. With `partials` (float32
// [S * KV * splits * (16 * hd + 32)]) and `arrived` (int32 [S * KV], zero; left zero) up to 64 blocks
// share it without a cluster and merge through global memory.
VOB_EXPORT int vob_attn_decode_mma(const void* q, long long q_stride, void* out, long long out_stride, const void* kcache,
                                   const void* vcache, const int* block_tables, int max_pages, const int* positions, int S,
                                   int H, int KV, int hd, int page_size, int window, float scale, int splits,
                                   void* partials, int* arrived, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (!sizes_ok(H, KV, hd, page_size) || H / KV > 16) return VOB_ERR_UNSUPPORTED;
    if ((partials == nullptr) != (arrived == nullptr)) return VOB_ERR_BAD_ARG;
    if (q_stride % 8 != 0 || splits < 1 || splits > (partials ? DEC_MAX_SPLITS_WIDE : 8) || KV > 65535) return VOB_ERR_BAD_ARG;
    if (hd == 64) return launch_decode<64>(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, positions, S,
                                          H, KV, page_size, window, scale, splits, (float*)partials, arrived, stream);
    return launch_decode<128>(q, q_stride, out, out_stride, kcache, vcache, block_tables, max_pages, positions, S, H, KV,
                              page_size, window, scale, splits, (float*)partials, arrived, stream);
}
