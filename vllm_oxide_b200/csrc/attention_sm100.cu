// Attention for portions of prompts on the 5th-generation tensor cores (bfloat16 engine, head
// size 64 or 128): causal grouped-query attention over the paged cache.
//
// Math (as csrc/attention.cu; reference crates/engine/src/backend/cpu/attention.rs:76-128):
//   s_j = (q . K_j) * scale over keys 0..p, softmax in float32 with a running maximum,
//   out = sum_j softmax_j V_j. P is rounded to bfloat16 for the second product.
//
// One block = 128 rows of one (request, kv head): the G = H / KV query heads that share the kv
// head are stacked as rows (row rr = token rr / G, head kvh * G + rr % G), so a K/V tile is read
// once per kv head. Per tile of 64 keys:
//   S[128, 64] = Q K^T       tcgen05.mma, A = Q from tensor memory, B = the K tile (K-major) from
//                            shared memory, S in tensor memory
//   P = exp2(S * scale * log2 e - m)   128 threads, one row each: the row's 64 scores come to
//                                      registers with tcgen05.ld, P goes back over them as bfloat16
//                                      pairs (tcgen05.st)
//   O[128, 64] += P V        tcgen05.mma with A = P from tensor memory, B = the V tile exactly as
//                            it lies in the cache ([key][head_dim]: an MN-major operand)
// S has two buffers: the product for tile j+2 is issued right behind P V of tile j (tcgen05.mma
// of one thread run in issue order, and P lies over the first half of its S), so the rows find
// the next scores waiting. Q is copied to tensor memory once and is the A operand of every Q K^T
// from there. The running maximum only moves when a tile's maximum exceeds it by more than 2^8
// (the sums stay exact: the same reference is used for P, for the row sum and for O), so O in
// tensor memory is rescaled rarely, and only then do the rows wait for the previous P V.
//
// What bounds it (measured): a thread gets one tcgen05.mma or commit through in about 125 clocks
// whatever its size, and a tile of 64 keys costs ten of them (4 + 4 products of 32 clocks of
// tensor-core work each, two commits); two blocks per SM overlap their chains. Tried and
// measured slower: two threads per row (16 softmax warps per SM), exponentials shared with the
// FMA pipe by a cubic, separate issuing threads for the two products.
//
// Data movement: Q by one TMA box [tokens][G heads][64]; K and V page by page, one TMA box
// [page_size][64] per page straight from the page's place in the cache (a page of one kv head is
// contiguous), 128-byte swizzle, a ring of 4 tiles each. Page numbers come from the block table
// through shared memory. Pages past the request's last key are read as zeros (out-of-range
// coordinate); rows of the last V tile beyond the last key (stale values of a page's earlier
// user) are zeroed in shared memory before the product, so no value of another request can reach
// this one.
//
// Roles in a block of 192 threads: warp 0 issues TMA, warp 1 (one lane) issues tcgen05.mma and
// owns the tensor memory, warps 2-5 are the softmax rows. Two blocks fit one SM. Every mbarrier
// wait is bounded (see sm100.cuh); on expiry the block raises the error flag, frees its tensor
// memory and returns.
//
// Head size 128 is the same kernel with every operand tile in two 64-wide halves (two TMA boxes;
// Q K^T takes both halves of the head dimension in turn, P V fills all 128 columns of O with one
// instruction per 16 keys, the V tile's halves being one MN-major operand), O in 128 columns of
// tensor memory, Q read from shared memory (no room for it in tensor memory) and a ring of two K
// and two V tiles freed separately. A group
// size G that does not divide 128 leaves the last 128 mod G rows of a block unused.
//
// Takes head_dim 64 or 128, any G up to 128, page sizes 8..128 (powers of two), no window. The
// launcher refuses anything else and the caller uses another kernel.
#include "common.cuh"
VOB_PDL_SWITCH(attention_sm100)
#include "sm100.cuh"
#include <string>
#include <unordered_map>

namespace {
using namespace vob_sm100;

constexpr int BM = 128;            // rows (token, head) per block
constexpr int BN = 64;             // keys per tile
constexpr int NTHREADS = 192;
// K and V tiles in flight: four of 8 KB each at head size 64, two of 16 KB at 128 (two blocks per SM either way)
template <int HD> __host__ __device__ constexpr int stages() { return HD == 64 ? 4 : 2; }
constexpr int HALF_Q = BM * 128;   // bytes of a 64-wide half of the Q tile
constexpr int HALF_KV = BN * 128;  // bytes of a 64-wide half of a K or V tile

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD> __host__ __device__ constexpr size_t tile_bytes() { return (size_t)BN * HD * 2; }
template <int HD> constexpr size_t fixed_smem() { return 1024 + (size_t)BM * HD * 2 + 2 * stages<HD>() * tile_bytes<HD>() + 256; }

template <int HD>
__global__ void __launch_bounds__(NTHREADS, 2)
attn_prefill_sm100_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, long long out_stride,
                          const int* __restrict__ block_tables, int max_pages, const int* __restrict__ seq_starts,
                          const int* __restrict__ context_lens, int H, int KV, int page_shift, int num_pages,
                          float scale_log2, int* __restrict__ err_flag) {
    static_assert(HD == 64 || HD == 128, "rows of one or two 128-byte swizzle spans");
    constexpr int ST = stages<HD>();
    constexpr int NH = HD / 64;                    // 64-wide halves of the head dimension, each a tile of 128-byte rows
    constexpr bool Q_TMEM = HD == 64;              // Q as the A operand from tensor memory (there is room at head size 64)
    constexpr bool SPLIT_FREE = HD == 128;         // K stages are freed by Q K^T, V stages by P V (a ring of two needs that)
    pdl_launch_dependents();
    // The step's metadata was copied before the first kernel of the step started: readable now.
    const int G = H / KV;
    // Blocks are handed out in the order x, y, z: the kv head runs fastest and the row tile
    // slowest, later row tiles (which see more keys) first, so that over the whole grid the long
    // blocks start first and the short ones fill the gaps behind them.
    const int kvh = blockIdx.x, seq = blockIdx.y;
    const int row0 = seq_starts[seq];
    const int total_rows = (seq_starts[seq + 1] - row0) * G;
    const int tile_rows = (BM / G) * G;            // whole tokens only: BM when G divides it
    const int tile_row0 = (gridDim.z - 1 - blockIdx.z) * tile_rows;
    if (tile_row0 >= total_rows) return;
    const int ctx = context_lens[seq];

    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = base;
    unsigned char* sK = sQ + BM * HD * 2;
    unsigned char* sV = sK + ST * tile_bytes<HD>();
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + ST * tile_bytes<HD>());
    uint64_t* q_full = bars;                 // [1]
    uint64_t* k_full = bars + 1;             // [ST]
    uint64_t* v_full = k_full + ST;          // [ST]
    uint64_t* kv_free = v_full + ST;         // [ST] P V of the tile has completed: its V (and K) stage is free, O holds it
    uint64_t* k_free = kv_free + ST;         // [ST] Q K^T of the tile has completed (used when K stages are freed on their own)
    uint64_t* s_full = k_free + ST;          // [2] S of a tile is complete (one barrier per S buffer)
    uint64_t* p_ready = s_full + 2;          // [2] 128 rows have read S and written P over it
    uint64_t* q_ready = p_ready + 2;         // [1] Q has been copied to tensor memory
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(q_ready + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    int* s_pages = reinterpret_cast<int*>(bars) + 64;         // [page_end], behind 256 bytes of barriers

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int last_rr = min(tile_row0 + tile_rows, total_rows) - 1;
    const int hi = ctx + last_rr / G + 1;                     // keys any row of the block reads: [0, hi)
    const int first_tok_pos = ctx + tile_row0 / G;
    const int n_tiles = (hi + BN - 1) / BN;
    const int page_end = ((hi - 1) >> page_shift) + 1;
    constexpr int TMEM_COLS = 256;                            // S0 64 | S1 64 | O HD | Q 32 at head size 64 (P lies over the first half of its S)
    constexpr uint32_t COL_O = 2 * BN, COL_Q = 2 * BN + HD;
    static_assert(COL_O + HD + (Q_TMEM ? HD / 2 : 0) <= TMEM_COLS, "tensor memory layout");

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < ST; ++s) { mbar_init(k_full + s, 1); mbar_init(v_full + s, 1); mbar_init(kv_free + s, 1); mbar_init(k_free + s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(s_full + b, 1); mbar_init(p_ready + b, 128); }
        mbar_init(q_ready, 128);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    {
        const int* bt = block_tables + (size_t)seq * max_pages;
        for (int i = threadIdx.x; i < page_end; i += NTHREADS) s_pages[i] = bt[i];
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    pdl_wait(14);                                             // Q and this step's keys are written now

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        // a tile is BN keys: several whole pages, or a part of one large page
        const int page_size = 1 << page_shift;
        const int box_rows = min(page_size, BN);
        const int ppt = BN / box_rows;                        // boxes per tile
        const uint32_t box_bytes = (uint32_t)box_rows * 128;  // one 64-wide half of the box
        if (lane == 0) {
            mbar_expect_tx(q_full, (uint32_t)tile_rows * 128 * NH);
#pragma unroll
            for (int h = 0; h < NH; ++h)
                tma_load_3d(sQ + h * HALF_Q, &map_q, h * 64, kvh * G, row0 + tile_row0 / G, q_full);
        }
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j % ST;
            const uint32_t ph = (j / ST) & 1;
            const int key0 = j * BN + lane * box_rows;        // first key of this lane's box
            const int lp = key0 >> page_shift;
            const int phys = (lane < ppt && lp < page_end) ? s_pages[lp] : num_pages;       // past the end: zeros
            const int y = key0 & (page_size - 1);
            int ok = 1;
            if (lane == 0) {
                ok = mbar_wait(SPLIT_FREE ? k_free + s : kv_free + s, ph ^ 1, abort_flag, err_flag, 11) ? 1 : 0;
                if (ok) {
                    mbar_expect_tx(k_full + s, tile_bytes<HD>());
                    if (!SPLIT_FREE) mbar_expect_tx(v_full + s, tile_bytes<HD>());
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < ppt) {
#pragma unroll
                for (int h = 0; h < NH; ++h)
                    tma_load_4d(sK + s * tile_bytes<HD>() + h * HALF_KV + lane * box_bytes, &map_k, h * 64, y, kvh, phys, k_full + s);
            }
            if (SPLIT_FREE) {
                if (lane == 0) {
                    ok = mbar_wait(kv_free + s, ph ^ 1, abort_flag, err_flag, 12) ? 1 : 0;
                    if (ok) mbar_expect_tx(v_full + s, tile_bytes<HD>());
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
            }
            if (lane < ppt) {
#pragma unroll
                for (int h = 0; h < NH; ++h)
                    tma_load_4d(sV + s * tile_bytes<HD>() + h * HALF_KV + lane * box_bytes, &map_v, h * 64, y, kvh, phys, v_full + s);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16(BM, BN, false);
            constexpr uint32_t idesc_pv = umma_idesc_bf16(BM, 64, true);          // one 64-wide half of O at a time
            constexpr uint32_t idesc_pv_wide = umma_idesc_bf16(BM, HD, true);
            constexpr bool PV_WIDE = NH == 2;
            const uint32_t tO = tmem_base + COL_O;
            const uint32_t tQ = tmem_base + COL_Q;
            // S[j & 1] = Q K_j^T; tcgen05.mma of one thread run in issue order, so a product may be
            // issued as soon as what it overwrites has been handed over (p_ready of tile j - 2)
            auto issue_qk = [&](int j) -> bool {
                const int s = j % ST;
                if (!mbar_wait(k_full + s, (j / ST) & 1, abort_flag, err_flag, 14)) return false;
                tcgen05_fence_after();
                const uint32_t tS = tmem_base + (uint32_t)(j & 1) * BN;
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    const uint64_t kdesc = umma_desc_sw128(sK + s * tile_bytes<HD>() + h * HALF_KV);
                    const uint64_t qdesc = umma_desc_sw128(sQ + h * HALF_Q);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (Q_TMEM) umma_bf16_ts(tS, tQ + 8 * k, kdesc + 2 * k, idesc_qk, k > 0 ? 1u : 0u);
                        else umma_bf16(tS, qdesc + 2 * k, kdesc + 2 * k, idesc_qk, (h > 0 || k > 0) ? 1u : 0u);
                    }
                }
                if (SPLIT_FREE) umma_commit(k_free + s);
                umma_commit(s_full + (j & 1));
                return true;
            };
            bool ok = mbar_wait(Q_TMEM ? q_ready : q_full, 0, abort_flag, err_flag, 13);
            if (ok) { tcgen05_fence_after(); ok = issue_qk(0); }
            if (ok && n_tiles > 1) ok = issue_qk(1);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % ST;
                if (!mbar_wait(p_ready + (j & 1), (j >> 1) & 1, abort_flag, err_flag, 15)) break;       // S read, P written
                if (!mbar_wait(v_full + s, (j / ST) & 1, abort_flag, err_flag, 17)) break;
                tcgen05_fence_after();
                const uint32_t tP = tmem_base + (uint32_t)(j & 1) * BN;
                if (PV_WIDE) {
                    // all HD columns of O in one instruction per 16 keys: the V tile is an MN-major operand
                    // whose 64-wide halves lie HALF_KV bytes apart (the descriptor's leading byte offset)
                    const uint64_t vdesc = umma_desc_sw128(sV + s * tile_bytes<HD>(), HALF_KV);
#pragma unroll
                    for (int k = 0; k < BN / 16; ++k)
                        umma_bf16_ts(tO, tP + 8 * k, vdesc + (uint64_t)k * (2048 >> 4), idesc_pv_wide, (j > 0 || k > 0) ? 1u : 0u);
                } else {
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        const uint64_t vdesc = umma_desc_sw128(sV + s * tile_bytes<HD>() + h * HALF_KV);
#pragma unroll
                        for (int k = 0; k < BN / 16; ++k)      // 16 keys: 8 packed columns of P, 16 rows (2048 bytes) of V
                            umma_bf16_ts(tO + h * 64, tP + 8 * k, vdesc + (uint64_t)k * (2048 >> 4), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
                    }
                }
                umma_commit(kv_free + s);                   // V (and K) of the tile may be overwritten; O holds the tile
                if (j + 2 < n_tiles) ok = issue_qk(j + 2);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax rows
        const int quad = warp & 3;
        const int r = quad * 32 + lane;                       // row of the tile = lane of tensor memory
        const int rr = tile_row0 + r;
        const bool row_valid = r < tile_rows && rr < total_rows;
        const int pos = row_valid ? ctx + rr / G : -1;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        // tcgen05.ld / st are warp-wide: a warp gives up as a whole
        auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {
            return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, err_flag, code) ? 1 : 0) != 0;
        };
        // Q goes to tensor memory once: as the A operand of every Q K^T it is then read from there
        // and not from shared memory again (16 KB per tile of keys less for the tensor cores to
        // fetch). Row r of the swizzled tile: 16-byte chunk c lies at chunk position c ^ (r & 7).
        if (Q_TMEM) {
            if (wait_all(q_full, 0, 22)) {
                uint32_t qv[32];
                const uint4* qrow = reinterpret_cast<const uint4*>(sQ + (size_t)r * 128);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 x = qrow[c ^ (r & 7)];
                    qv[4 * c] = x.x; qv[4 * c + 1] = x.y; qv[4 * c + 2] = x.z; qv[4 * c + 3] = x.w;
                }
                tmem_st32(lane_addr + COL_Q, qv);
                tmem_wait_st();
                tcgen05_fence_before();
                mbar_arrive(q_ready);
            } else {
                ok = false;
            }
        }
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int kbase = j * BN;
            const uint32_t tS = lane_addr + (uint32_t)(j & 1) * BN;
            const bool masked_tile = kbase + BN - 1 > first_tok_pos;      // some row of the block does not see every key
            if (!wait_all(s_full + (j & 1), (j >> 1) & 1, 18)) { ok = false; break; }
            tcgen05_fence_after();
            uint32_t va[32], vb[32];
            tmem_ld32(tS, va);
            tmem_ld32(tS + 32, vb);
            tmem_wait_ld();
            if (masked_tile) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (kbase + i > pos) va[i] = 0xff800000u;             // -inf
                    if (kbase + 32 + i > pos) vb[i] = 0xff800000u;
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                mx0 = max3(mx0, __uint_as_float(va[i]), __uint_as_float(vb[i]));
                mx1 = max3(mx1, __uint_as_float(va[i + 1]), __uint_as_float(vb[i + 1]));
            }
            const float mx2 = fmaxf(mx0, mx1) * scale_log2;               // scale > 0: the maximum commutes
            const bool grow = mx2 > m_ref + 8.f;                          // also the first finite maximum
            const float m_new = grow ? mx2 : m_ref;
            const float alpha = grow ? fast_exp2(m_ref - m_new) : 1.f;    // m_ref = -inf: 0
            m_ref = m_new;
            l *= alpha;
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                // O may be touched once the previous tile's product has completed
                if (!wait_all(kv_free + (j - 1) % ST, ((j - 1) / ST) & 1, 19)) { ok = false; break; }
                tcgen05_fence_after();
#pragma unroll
                for (int c = 0; c < HD; c += 16) {
                    uint32_t v[16];
                    tmem_ld16(lane_addr + COL_O + c, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tmem_st16(lane_addr + COL_O + c, v);
                }
            }
            // two scores at a time: the packed float32 pair instructions of sm_100 halve the issue
            // slots of the scale-and-subtract and of the row sum
            const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(-m_use, -m_use);
            float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(va[i]), __uint_as_float(va[i + 1])), sc2, nm2);
                const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(vb[i]), __uint_as_float(vb[i + 1])), sc2, nm2);
                const float2 p0 = make_float2(fast_exp2(x0.x), fast_exp2(x0.y));        // -inf: 0
                const float2 p1 = make_float2(fast_exp2(x1.x), fast_exp2(x1.y));
                acc0 = __fadd2_rn(acc0, p0);
                acc1 = __fadd2_rn(acc1, p1);
                pk[i >> 1] = pack_bf16(p0.x, p0.y);
                pk[16 + (i >> 1)] = pack_bf16(p1.x, p1.y);
            }
            l += (acc0.x + acc0.y) + (acc1.x + acc1.y);
            tmem_st32(tS, pk);                                            // P over the first half of its S
            if (j == n_tiles - 1 && quad < 2 && kbase + quad * 32 + 31 >= hi) {
                // the last tile: V rows past the last key hold whatever the page held before
                const int s = j % ST;
                if (!wait_all(v_full + s, (j / ST) & 1, 20)) { ok = false; break; }
                if (kbase + r >= hi) {
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        uint4* row = reinterpret_cast<uint4*>(sV + s * tile_bytes<HD>() + h * HALF_KV + (size_t)r * 128);
#pragma unroll
                        for (int i = 0; i < 8; ++i) row[i] = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                }
                __syncwarp();
            }
            tmem_wait_st();
            tcgen05_fence_before();
            mbar_arrive(p_ready + (j & 1));
        }
        if (ok && wait_all(kv_free + (n_tiles - 1) % ST, ((n_tiles - 1) / ST) & 1, 21)) {
            tcgen05_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = out + (size_t)(row0 + rr / G) * out_stride + (size_t)(kvh * G + rr % G) * HD;
#pragma unroll
            for (int c = 0; c < HD; c += 16) {
                uint32_t v[16];
                tmem_ld16(lane_addr + COL_O + c, v);
                tmem_wait_ld();
                if (row_valid) {
                    uint4 a, b;
                    a.x = pack_bf16(__uint_as_float(v[0]) * inv, __uint_as_float(v[1]) * inv);
                    a.y = pack_bf16(__uint_as_float(v[2]) * inv, __uint_as_float(v[3]) * inv);
                    a.z = pack_bf16(__uint_as_float(v[4]) * inv, __uint_as_float(v[5]) * inv);
                    a.w = pack_bf16(__uint_as_float(v[6]) * inv, __uint_as_float(v[7]) * inv);
                    b.x = pack_bf16(__uint_as_float(v[8]) * inv, __uint_as_float(v[9]) * inv);
                    b.y = pack_bf16(__uint_as_float(v[10]) * inv, __uint_as_float(v[11]) * inv);
                    b.z = pack_bf16(__uint_as_float(v[12]) * inv, __uint_as_float(v[13]) * inv);
                    b.w = pack_bf16(__uint_as_float(v[14]) * inv, __uint_as_float(v[15]) * inv);
                    *reinterpret_cast<uint4*>(dst + c) = a;
                    *reinterpret_cast<uint4*>(dst + c + 8) = b;
                }
            }
        }
        tcgen05_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------ host side
// bfloat16 tensor maps with the 128-byte swizzle, cached by everything that defines them.
int make_map(CUtensorMap* out, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
             const cuuint32_t* box) {
    static std::mutex mu;
    static std::unordered_map<std::string, CUtensorMap> cache;
    std::string key(reinterpret_cast<const char*>(&ptr), sizeof(ptr));
    key.append(reinterpret_cast<const char*>(dims), rank * sizeof(cuuint64_t));
    key.append(reinterpret_cast<const char*>(strides_bytes), (rank - 1) * sizeof(cuuint64_t));
    key.append(reinterpret_cast<const char*>(box), rank * sizeof(cuuint32_t));
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return VOB_ERR_UNSUPPORTED;
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides_bytes, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return VOB_ERR_BAD_ARG;
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return 0;
}

inline int log2_exact(int v) {
    int s = 0;
    while ((1 << s) < v) ++s;
    return (1 << s) == v ? s : -1;
}

bool sizes_ok(int H, int KV, int hd, int page_size) {
    if ((hd != 64 && hd != 128) || KV <= 0 || H <= 0 || H % KV != 0) return false;
    int G = H / KV;
    if (G > BM) return false;
    if (page_size < 8 || page_size > 128 || log2_exact(page_size) < 0) return false;
    return true;
}

}  // namespace

VOB_EXPORT int vob_attn_prefill_sm100_supported(int H, int KV, int hd, int page_size, int max_pages) {
    if (!sizes_ok(H, KV, hd, page_size)) return 0;
    const size_t fixed = hd == 64 ? fixed_smem<64>() : fixed_smem<128>();
    return fixed + (size_t)max_pages * sizeof(int) <= 110 * 1024 ? 1 : 0;                  // two blocks per SM
}

// q [q_rows, H*hd] (row stride q_stride elements), out likewise; kcache / vcache [num_pages, KV,
// page_size, hd]; block_tables int32 [S, max_pages]; seq_starts int32 [S+1]; context_lens int32 [S];
// max_new = the longest portion of the step.
VOB_EXPORT int vob_attn_prefill_sm100(const void* q, long long q_rows, long long q_stride, void* out, long long out_stride,
                                      const void* kcache, const void* vcache, long long num_pages, const int* block_tables,
                                      int max_pages, const int* seq_starts, const int* context_lens, int S, int max_new, int H,
                                      int KV, int hd, int page_size, float scale, int* err_flag, cudaStream_t stream) {
    if (S <= 0 || max_new <= 0) return 0;
    if (!vob_attn_prefill_sm100_supported(H, KV, hd, page_size, max_pages)) return VOB_ERR_UNSUPPORTED;
    if (!(scale > 0.f) || q_rows <= 0 || num_pages <= 0 || num_pages > 0x7fffffff) return VOB_ERR_BAD_ARG;
    if (q_stride % 8 != 0 || out_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)kcache & 15) ||
        ((uintptr_t)vcache & 15) || S > 65535 || KV > 65535)
        return VOB_ERR_BAD_ARG;
    const int G = H / KV;
    CUtensorMap mq, mk, mv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)H, (cuuint64_t)q_rows};
        cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)q_stride * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(BM / G)};
        int e = make_map(&mq, q, 3, dims, strides, box);
        if (e) return e;
    }
    {
        cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)page_size, (cuuint64_t)KV, (cuuint64_t)num_pages};
        cuuint64_t strides[3] = {(cuuint64_t)hd * 2, (cuuint64_t)page_size * hd * 2, (cuuint64_t)KV * page_size * hd * 2};
        cuuint32_t box[4] = {64, (cuuint32_t)(page_size < BN ? page_size : BN), 1, 1};
        int e = make_map(&mk, kcache, 4, dims, strides, box);
        if (e) return e;
        e = make_map(&mv, vcache, 4, dims, strides, box);
        if (e) return e;
    }
    const long long tok_per_tile = BM / G;
    const long long row_tiles = ((long long)max_new + tok_per_tile - 1) / tok_per_tile;
    if (row_tiles > 65535) return VOB_ERR_UNSUPPORTED;
    dim3 grid(KV, S, (unsigned)row_tiles);
    if (hd == 64) {
        static size_t configured = 0;
        size_t smem = fixed_smem<64>() + (size_t)max_pages * sizeof(int);
        if (smem > configured) {
            cudaError_t e = cudaFuncSetAttribute(attn_prefill_sm100_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = smem;
        }
        return vob_launch(attn_prefill_sm100_kernel<64>, grid, dim3(NTHREADS), smem, stream, mq, mk, mv, (__nv_bfloat16*)out,
                          out_stride, block_tables, max_pages, seq_starts, context_lens, H, KV, log2_exact(page_size),
                          (int)num_pages, scale * 1.4426950408889634f, err_flag);
    }
    static size_t configured = 0;
    size_t smem = fixed_smem<128>() + (size_t)max_pages * sizeof(int);
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_sm100_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    return vob_launch(attn_prefill_sm100_kernel<128>, grid, dim3(NTHREADS), smem, stream, mq, mk, mv, (__nv_bfloat16*)out,
                      out_stride, block_tables, max_pages, seq_starts, context_lens, H, KV, log2_exact(page_size),
                      (int)num_pages, scale * 1.4426950408889634f, err_flag);
}
