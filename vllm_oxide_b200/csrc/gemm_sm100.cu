// bfloat16 matrix product on the 5th-generation tensor cores: C[T, N] = X[T, K] * W[N, K]^T.
// Reference op: crates/engine/src/backend/cpu/mod.rs:199-229 (x * W^T, W [out, in] row-major).
//
// Shape of the kernel. The weight matrix is the M operand of tcgen05.mma (128 weight rows per
// block), the tokens are the N operand (a tile of BT = 16 ... 256 tokens): D[128 features, BT
// tokens] accumulates in tensor memory in float32. Both operands are K-major, which is how W
// [N, K] and X [T, K] already lie in memory, so nothing is transposed. With the tokens on the N
// side one kernel serves a decode step of a few tokens (a weight-streaming, HBM-bound product:
// every weight byte is read exactly once, by TMA, through a multi-stage ring) and a prompt
// portion of thousands (tensor-bound).
//
// Roles inside a block of 192 threads: warp 0 (one elected lane) issues the TMA loads
// (cp.async.bulk.tensor, 128-byte swizzle, one mbarrier per stage), warp 1 allocates tensor
// memory and (one lane) issues tcgen05.mma, committing each stage back to the producer with
// tcgen05.commit; warps 2-5 read the accumulator with tcgen05.ld (each warp its own 32 lanes) and
// write C: lane = output feature, so one store instruction of a warp covers 32 consecutive
// features of one token. The kernel for few tokens has one more warp with a second issuing thread.
//
// Few tokens leave most SMs without a tile, so the K range can be split over blockIdx.z. The
// blocks of one tile form a thread-block cluster (up to 8): each leaves its float32 partial tile
// in its own shared memory, the cluster meets at a barrier, and every block then adds up a share
// of the tile's tokens, reading its peers' partials through distributed shared memory in rank
// order (a fixed order: the result does not depend on timing) and writes C. Nothing goes through
// global memory and nothing needs resetting between launches.
//
// Tiles of 16 tokens (decode steps of up to 16 requests) do the products another way. Measured on
// this GPU: a tcgen05.mma costs the tensor pipe some 160 clocks however few tokens it has (its A
// operand, 128 weight rows x 32 bytes, is fetched from shared memory at about 32 bytes a clock), so a
// stage of 64 k took 0.33 us of products whatever the token count, and the product phase of a block
// whose weights had all been prefetched was as long as its whole epilogue. For these tiles the four
// epilogue warps therefore do the products themselves: 32 weight rows each, fragments by ldmatrix
// straight from the TMA ring's swizzled tiles, mma.sync.m16n8k16 with float32 accumulators in
// registers (one 8-token half only when the step has at most 8 tokens); no tensor memory, no issuing
// threads, and the per-token scale's round trip to L2 hides behind the product loop. The rest of
// the kernel (TMA ring, cluster split of K, epilogues) is the same. A decode step at batch 1 / 8 / 16
// went from 0.750 / 0.858 / 1.002 to 0.733 / 0.848 / 0.966 ms. (Two or four accumulator sets to
// shorten the chain of dependent products cost registers, a second block no longer fitted the SM,
// and the step took 0.88 / 1.04 ms: dropped.)
//
// Every wait on an mbarrier is bounded (two seconds): on expiry the block raises the error flag,
// stops issuing work, frees its tensor memory and returns; the host turns the flag into an
// exception. No TMA load uses cluster multicast.
#include "common.cuh"
VOB_PDL_SWITCH(gemm_sm100)
#include "sm100.cuh"
#include <unordered_map>

namespace {
using namespace vob_sm100;

constexpr int BM = 128;           // weight rows (output features) per block
constexpr int BK = 64;            // K elements per stage: 128 bytes, one swizzle span
constexpr int UMMA_K = 16;
constexpr int NTHREADS = 192;
constexpr int ISSUERS = 2;          // MMA-issuing threads of the kernel for few tokens (warps 1, 6, 7, ...)
constexpr int NTHREADS_FEW = 192 + 32 * (ISSUERS - 1);
// kind::f16 instruction descriptor of this file's products: M = 128 weight rows, N = n tokens, both K-major.
__host__ __device__ constexpr uint32_t umma_idesc(int n) { return umma_idesc_bf16(BM, n, false); }

// For tiles of 16 tokens the products are done by mma.sync from the TMA ring (see the kernel's header
// comment below): 8 x 8 matrices of 16-bit elements from shared memory, four at a time, and the
// 16 x 8 x 16 product with float32 accumulators in registers.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
#ifdef VOB_FEW16_TCGEN05
constexpr bool FEW16_MMA_SYNC = false;
#else
constexpr bool FEW16_MMA_SYNC = true;
#endif

template <typename OutT> __device__ __forceinline__ void store_out(OutT* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// What the epilogue does with a finished element (token t, output feature f):
//   EPI_STORE   C[t, f] = value
//   EPI_SWIGLU  the block's 128 weight rows are 64 rows of the "gate" half and the same 64 rows of
//               the "up" half of a [2I, K] weight matrix (two TMA boxes into one operand tile):
//               C[t, f] = gate / (1 + exp(-gate)) * up (crates/engine/src/backend/cpu/mod.rs:341-349),
//               so the SwiGLU input never exists in memory
//   EPI_QKV     the weight matrix is [Wq; Wk; Wv]: q and k features are rotated by the rotary rule
//               (crates/engine/src/backend/cpu/rope.rs:87-99; angle float(pos) * inv_freq, precise
//               sinf/cosf), q goes to C, rotated k and v go straight to their cache slots
//               (crates/engine/src/backend/cpu/mod.rs:257-285): no separate rotary / cache-write pass
//   EPI_RESID   the product is a block's output (attention's or the feed-forward's): it is added to the
//               float32 residual (crates/engine/src/backend/cpu/mod.rs:351-358), and the input of the
//               NEXT norm is prepared in the same pass: x' = bf16(residual * next norm's weight) and,
//               per 128-feature tile and token, the sum of the residual's squares. The next product
//               multiplies its accumulator by 1 / sqrt(mean(residual^2) + eps), a per-token scalar
//               that commutes with the product, so the RMSNorm (:182-197) needs no kernel of its own.
//   EPI_PICK    the product is the output head and only the picked token is wanted: the block reduces
//               its 128 logits of every token to the best (value, index) pair, by the rule of
//               sampling.cu (greedy: first index of the maximum, crates/engine/src/backend/cpu/mod.rs:370-388;
//               temperature: logit / temperature + Gumbel noise from the row's seed), and writes one pair
//               per (token, tile); a row that holds a NaN is flagged. The logits never go to memory: the
//               pick's first pass over them, and its launch, are gone. No split of K.
enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_QKV = 2, EPI_RESID = 3, EPI_PICK = 4 };

// Everything an epilogue may need beyond C; a plain struct that the host fills (same layout in
// kernels.py). Unused members are null / 0.
struct EpiArgs {
    // EPI_QKV
    const int* positions;              // [T]
    const int* slots;                  // [T] cache slot of each token, -1: none
    const float* inv_freq;             // [hd / 2] or null (no rotation)
    __nv_bfloat16* kcache;             // [pages, KV, page_size, hd]
    __nv_bfloat16* vcache;
    // any mode: scale token t's accumulator by 1 / sqrt(sum_i ssq_in[i * ld_ssq + t] * inv_h + eps)
    const float* ssq_in;
    // EPI_RESID
    float* resid;                      // [T, N] float32, updated in place
    const float* next_w;               // [N] weight of the norm that follows
    __nv_bfloat16* xn_out;             // [T, N] bf16(residual * next_w)
    float* ssq_out;                    // [ceil(N / 128), ld_ssq] partial sums of squares
    long long ld_resid, ld_xn;
    int q_dim, kv_dim, hd, KV, page_size;
    int ssq_tiles, ld_ssq;
    float inv_h, eps;
    int pad_;
    // EPI_PICK
    const float* temperature;          // [T] or null (greedy)
    const uint32_t* seeds;             // [T][2]
    const int* steps;                  // [T] index of the generated token
    float* part_val;                   // [T][ld_part] best value of each tile
    int* part_idx;                     // [T][ld_part] its vocabulary index
    int* nan_flags;                    // [T] raised for a row that holds a NaN
    long long ld_part;
};
typedef EpiArgs QkvArgs;

__device__ __forceinline__ uint32_t mix32(uint32_t x) {          // the hash of sampling.cu
    x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
    return x;
}

template <int BT, int EPI> __host__ __device__ constexpr int stage_bytes() { return BM * BK * 2 + BT * BK * 2; }
template <int BT> __host__ __device__ constexpr int stage_bytes() { return stage_bytes<BT, EPI_STORE>(); }
// two accumulators of BT columns each (one per issuing thread) for few tokens
template <int BT, int EPI> __host__ __device__ constexpr int tmem_cols() { return ISSUERS * BT < 32 ? 32 : ISSUERS * BT; }
template <int BT> __host__ __device__ constexpr int tmem_cols() { return tmem_cols<BT, EPI_STORE>(); }

// 16 columns of this thread's lane, summed over the issuers' accumulators in a fixed order.
template <int BT> __device__ __forceinline__ void load_acc(uint32_t taddr, float* r) {
    uint32_t a[ISSUERS][16];
#pragma unroll
    for (int w = 0; w < ISSUERS; ++w) tmem_ld16(taddr + w * BT, a[w]);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        if (ISSUERS == 4) r[j] = (__uint_as_float(a[0][j]) + __uint_as_float(a[1][j])) + (__uint_as_float(a[2][j]) + __uint_as_float(a[3][j]));
        else if (ISSUERS == 2) r[j] = __uint_as_float(a[0][j]) + __uint_as_float(a[1][j]);
        else r[j] = __uint_as_float(a[0][j]);
    }
}

template <int BT, int STAGES, typename OutT, int EPI>
__global__ void __launch_bounds__(NTHREADS_FEW, 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, OutT* __restrict__ C,
                  long long ldc, int T, int N, int K, int kb_per_split, int* __restrict__ err_flag, int up_row0,
                  const QkvArgs qa, int test_extra_tx) {
    constexpr int SB = stage_bytes<BT, EPI>();
    constexpr int A_BYTES = BM * BK * 2;
    // Tiles of 16 tokens: the four epilogue warps do the products themselves with mma.sync, reading the
    // ring's tiles with ldmatrix; no tensor memory, no issuing threads (see the note above the kernel).
    constexpr bool MS = BT == 16 && FEW16_MMA_SYNC;
    constexpr int PRE = BT >= 64 ? 12 : (BT >= 32 ? 8 : 4);   // tokens per block whose rotation is worked out ahead
    pdl_launch_dependents();
    extern __shared__ unsigned char smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + STAGES * SB);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_bar = empty_bar + STAGES;
    uint64_t* done_bar = acc_bar + 1;              // under a split: every block of the cluster has read this block's partials
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(done_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    float* sc = reinterpret_cast<float*>(const_cast<int*>(abort_flag) + 2);       // BT floats: per-token scales
    float* s_tau = sc + 64;                                                        // EPI_PICK: per-token temperature,
    uint32_t* s_ctr = reinterpret_cast<uint32_t*>(s_tau + 64);                     // and the token's noise counter

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tile = blockIdx.x, n_tile = blockIdx.y, split = blockIdx.z, splits = gridDim.z;
    const int total_kb = (K + BK - 1) / BK;
    const int kb0 = split * kb_per_split;
    const int kb1 = min(total_kb, kb0 + kb_per_split);
    const int nkb = kb1 - kb0;                    // >= 1 by the launcher's choice of splits

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, MS ? 4 : ISSUERS); }
        mbar_init(acc_bar, ISSUERS);                     // both issuing threads commit to these
        mbar_init(done_bar, splits);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (!MS && warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(tmem_cols<BT, EPI>()) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = MS ? 0u : *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            // Weights are written by no kernel, so their loads start at once and overlap whatever
            // still runs before this kernel; the activations are loaded only after the wait.
            const int pre = nkb < STAGES ? nkb : STAGES;
            for (int i = 0; i < pre; ++i) {
                unsigned char* a = tiles + i * SB;
                // test_extra_tx is 0 except in the test of the give-up path: bytes that never arrive
                mbar_expect_tx(full_bar + i, SB + (i == 0 ? test_extra_tx : 0));
                if (EPI == EPI_SWIGLU) {
                    tma_load_2d(a, &map_w, (kb0 + i) * BK, m_tile * (BM / 2), full_bar + i);
                    tma_load_2d(a + (BM / 2) * BK * 2, &map_w, (kb0 + i) * BK, up_row0 + m_tile * (BM / 2), full_bar + i);
                } else {
                    tma_load_2d(a, &map_w, (kb0 + i) * BK, m_tile * BM, full_bar + i);
                }
            }
            pdl_wait(12);
            for (int i = 0; i < pre; ++i)
                tma_load_2d(tiles + i * SB + A_BYTES, &map_x, (kb0 + i) * BK, n_tile * BT, full_bar + i);
            for (int i = pre; i < nkb; ++i) {
                int s = i % STAGES;
                uint32_t ph = (i / STAGES) & 1;
                if (!mbar_wait(empty_bar + s, ph ^ 1, abort_flag, err_flag, 1)) break;
                unsigned char* a = tiles + s * SB;
                mbar_expect_tx(full_bar + s, SB);
                if (EPI == EPI_SWIGLU) {
                    tma_load_2d(a, &map_w, (kb0 + i) * BK, m_tile * (BM / 2), full_bar + s);
                    tma_load_2d(a + (BM / 2) * BK * 2, &map_w, (kb0 + i) * BK, up_row0 + m_tile * (BM / 2), full_bar + s);
                } else {
                    tma_load_2d(a, &map_w, (kb0 + i) * BK, m_tile * BM, full_bar + s);
                }
                tma_load_2d(a + A_BYTES, &map_x, (kb0 + i) * BK, n_tile * BT, full_bar + s);
            }
        }
    } else if (!MS && (warp == 1 || warp >= 6)) {
        // ISSUERS issuing threads. One thread gets a tcgen05.mma through about every 125 clocks
        // whatever its size, and an instruction of 128 x 16 x 16 consumes only 4 KB of weights: a
        // single issuer just about keeps pace with HBM, and its chain is what a block with few
        // k-blocks waits for. Each thread takes its share of every stage's K steps into an
        // accumulator of its own; the epilogue adds them in a fixed order. (Measured on a decode
        // step of 8 rows: two issuers +2.5 %, four +2.7 %.)
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BT);
            constexpr int KSTEPS = BK / UMMA_K / ISSUERS;
            const int w = warp >= 6 ? warp - 5 : 0;
            const uint32_t acc = tmem_base + (uint32_t)(w * BT);
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                int s = i % STAGES;
                uint32_t ph = (i / STAGES) & 1;
                ok = mbar_wait(full_bar + s, ph, abort_flag, err_flag, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char* a = tiles + s * SB;
                uint64_t adesc = umma_desc_sw128(a);
                uint64_t bdesc = umma_desc_sw128(a + A_BYTES);
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
                    // 16 K elements = 32 bytes = 2 units of the descriptor's start address
                    const int k = w * KSTEPS + kk;
                    umma_bf16(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(empty_bar + s);       // the stage is free once both threads' MMAs have read it
            }
            if (ok) umma_commit(acc_bar);         // the accumulator is complete
        }
    } else if (warp >= 2 && warp < 6) {
        // epilogue warps 2..5: warp w may touch tensor-memory lanes 32 * (w % 4) ... + 31
        const int quad = warp & 3;
        const int col = quad * 32 + lane;
        const int f = m_tile * BM + col;                       // this thread's output feature
        const int t0 = n_tile * BT;
        // The tokens this block finishes: its whole tile without a split, else every splits-th
        // token (number k is token tok_first + k * splits of the tile).
        const int tok_first = splits > 1 ? split : 0;
        const int tok_end = min(BT, T - t0);
        const int nk = tok_end > tok_first ? (tok_end - tok_first + splits - 1) / splits : 0;
        // Rotary positions: what this thread will need for the first tokens its block finishes
        // (cosine, sine, cache slot) depends only on data that was on the device before the step
        // began, so it is worked out now, while the weights stream, not after the accumulator is done.
        float pc[PRE], ps[PRE];
        int pslot[PRE];
        bool rot = false;
        float inv = 0.f;
        if (EPI == EPI_QKV) {
            const int hd = qa.hd, half = hd >> 1, i = f % hd;
            rot = qa.inv_freq && f < qa.q_dim + qa.kv_dim;
            inv = rot ? qa.inv_freq[i < half ? i : i - half] : 0.f;
#pragma unroll
            for (int k = 0; k < PRE; ++k) {
                pc[k] = 1.f; ps[k] = 0.f; pslot[k] = -1;
                if (k < nk) {
                    const int t = t0 + tok_first + k * splits;
                    const float theta = (float)qa.positions[t] * inv;
                    pc[k] = cosf(theta);
                    ps[k] = sinf(theta);
                    pslot[k] = qa.slots ? qa.slots[t] : -1;
                }
            }
        }
        pdl_wait();
        // per-token scale of the accumulator (the folded RMSNorm of this product's input): it comes
        // from kernels in front, so it is fetched after the wait, while the product itself runs
        // 128 threads = BT tokens x (128 / BT) lanes: lane l adds the tiles l, l + L, ... of its token,
        // then the lanes' sums are added pairwise in a fixed tree (one L2 round trip instead of one per
        // tile). The values are requested here; where this warp does the products itself they are
        // only added up behind the product loop, so that the round trip is hidden by it.
        constexpr int L = 128 / BT;
        const int tk = col / L, ln = col % L;
        float ssq_v[4] = {0.f, 0.f, 0.f, 0.f};
        float ssq_rest = 0.f;
        if (qa.ssq_in && t0 + tk < T) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (ln + u * L < qa.ssq_tiles) ssq_v[u] = qa.ssq_in[(size_t)(ln + u * L) * qa.ld_ssq + t0 + tk];
            for (int i = ln + 4 * L; i < qa.ssq_tiles; i += L) ssq_rest += qa.ssq_in[(size_t)i * qa.ld_ssq + t0 + tk];
        }
        float tau = 0.f;
        uint32_t ctr = 0;
        if (EPI == EPI_PICK && ln == 0) {
            const int t = t0 + tk;
            if (t < T && qa.temperature) tau = qa.temperature[t];
            if (tau > 0.f) {
                const uint32_t key = mix32(qa.seeds[2 * t] ^ mix32(qa.seeds[2 * t + 1] + 0x85EBCA6Bu));
                ctr = mix32(key ^ mix32((uint32_t)qa.steps[t] + 0x9E3779B9u));
            }
        }
        auto finish_scales = [&]() {
            float part = (((ssq_v[0] + ssq_v[1]) + ssq_v[2]) + ssq_v[3]) + ssq_rest;      // the order a walk over the tiles adds them in
#pragma unroll
            for (int o = L / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (ln == 0) sc[tk] = (qa.ssq_in && t0 + tk < T) ? 1.0f / sqrtf(part * qa.inv_h + qa.eps) : 1.f;
            if (EPI == EPI_PICK && ln == 0) { s_tau[tk] = tau; s_ctr[tk] = ctr; }
        };
        if (!MS) finish_scales();
        float next_w = 0.f;
        if (EPI == EPI_RESID) next_w = f < N ? qa.next_w[f] : 0.f;      // the next norm's weight of this feature
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // Shared memory over the operand stages (every product that read them has completed by the time
        // it is written): `tile` [BT][128] is this block's tile (a partial one under a split, which
        // peers read); `fin` [nk][128] the finished values of the tokens this block completes, in
        // which partners of a fused epilogue find each other; `red` [nk][4] sums of squares by warp.
        float* tile = reinterpret_cast<float*>(tiles);
        float* fin = splits > 1 ? tile + BT * BM : tile;
        float* red = fin + (splits > 1 ? (BT / 2) * BM : BT * BM);
        bool ok = true;
        if (MS) {
            // This warp's 32 weight rows of the tile against the 16 tokens, stage by stage: A fragments
            // (weights) and B fragments (tokens) by ldmatrix from the 128-byte-swizzled tiles (row r,
            // 16-byte piece c lies at piece c ^ (r & 7)), 16 mma.sync per stage and warp.
            float acc[2][2][4];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[mi][ni][e] = 0.f;
            const int mtx = lane >> 3, r8 = lane & 7;
            const int a_row = quad * 32 + r8 + ((mtx & 1) << 3), a_k = mtx >> 1;     // + 16 for the second 16 rows
            const int x_row = r8 + ((mtx >> 1) << 3), x_k = mtx & 1;
            const bool more_than_8 = T - t0 > 8;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(full_bar + s, (i / STAGES) & 1, abort_flag, err_flag, 2)) { ok = false; break; }
                const uint32_t a_base = smem_u32(tiles + s * SB), x_base = a_base + A_BYTES;
#pragma unroll
                for (int ks = 0; ks < BK / UMMA_K; ++ks) {
                    uint32_t b[4], a0[4], a1[4];
                    ldmatrix_x4(b, x_base + x_row * 128 + (((ks * 2 + x_k) ^ (x_row & 7)) << 4));
                    ldmatrix_x4(a0, a_base + a_row * 128 + (((ks * 2 + a_k) ^ (a_row & 7)) << 4));
                    ldmatrix_x4(a1, a_base + (a_row + 16) * 128 + (((ks * 2 + a_k) ^ (a_row & 7)) << 4));
                    mma_16816(acc[0][0], a0, b[0], b[1]);
                    mma_16816(acc[1][0], a1, b[0], b[1]);
                    if (more_than_8) {                                    // tokens 8..15 (the same in all threads)
                        mma_16816(acc[0][1], a0, b[2], b[3]);
                        mma_16816(acc[1][1], a1, b[2], b[3]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar + s);        // this warp has read the stage
            }
            ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
            finish_scales();
            // every warp is through with the stages (and the scales are written) before the tile is written over them
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (ok && !*abort_flag) {
                const int g = lane >> 2, t2 = (lane & 3) * 2;
#pragma unroll
                for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                    for (int ni = 0; ni < 2; ++ni) {
                        const int row = quad * 32 + mi * 16 + g, tok = ni * 8 + t2;
                        tile[tok * BM + row] = acc[mi][ni][0] * sc[tok];
                        tile[(tok + 1) * BM + row] = acc[mi][ni][1] * sc[tok + 1];
                        tile[tok * BM + row + 8] = acc[mi][ni][2] * sc[tok];
                        tile[(tok + 1) * BM + row + 8] = acc[mi][ni][3] * sc[tok + 1];
                    }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            ok = ok && !*abort_flag;
        } else {
            ok = mbar_wait(acc_bar, 0, abort_flag, err_flag, 3);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
        // 16 tokens of this thread's feature, scaled: from the tile in shared memory, or from tensor memory
        auto get16 = [&](int c, float* r) {
            if (MS) {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = tile[(c + j) * BM + col];
            } else {
                load_acc<BT>(taddr + c, r);
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] *= sc[c + j];
            }
        };
        if (ok && splits == 1 && EPI == EPI_STORE) {
#pragma unroll
            for (int c = 0; c < BT; c += 16) {
                float r[16];
                get16(c, r);
                if (f < N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (t0 + c + j < T) store_out<OutT>(C + (size_t)(t0 + c + j) * ldc + f, r[j]);
                }
            }
        } else if (ok && EPI == EPI_PICK) {
            // every warp reduces its 32 logits of a token to the best pair; the four pairs of a token
            // meet in shared memory (over the operand stages, which are free now)
            float* wv = reinterpret_cast<float*>(tiles) + (MS ? BT * BM : 0);   // [4][BT] (behind the tile where that is in use)
            int* wi = reinterpret_cast<int*>(wv + 4 * BT);                  // [4][BT]
            int* wn = wi + 4 * BT;                                          // [4][BT] a NaN was seen
#pragma unroll
            for (int c = 0; c < BT; c += 16) {
                if (t0 + c >= T) break;                                     // the same in all threads
                float r[16];
                get16(c, r);
                // sixteen tokens side by side: their five exchange steps are independent chains
                float bv[16];
                int bi[16];
                unsigned nan_bits = 0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float x = r[j];
                    const float tau = s_tau[c + j];
                    float v = x;
                    if (tau > 0.f) {
                        const uint32_t h = mix32(s_ctr[c + j] ^ (uint32_t)f);
                        const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
                        v = x / tau + (-logf(-logf(u)));
                    }
                    const bool take = f < N && v > -INFINITY;               // NaN and -inf never win, as in a scan by "greater than"
                    bv[j] = take ? v : -INFINITY;
                    bi[j] = take ? f : 0x7fffffff;
                    if (f < N && x != x) nan_bits |= 1u << j;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float ov = __shfl_xor_sync(0xffffffffu, bv[j], o);
                        const int oi = __shfl_xor_sync(0xffffffffu, bi[j], o);
                        if (ov > bv[j] || (ov == bv[j] && oi < bi[j])) { bv[j] = ov; bi[j] = oi; }      // larger value; equal: smaller index
                    }
                    nan_bits |= __shfl_xor_sync(0xffffffffu, nan_bits, o);
                }
                if (lane < 16) {                                            // lane j writes token c + j (every lane holds every result)
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (lane == j) { wv[quad * BT + c + j] = bv[j]; wi[quad * BT + c + j] = bi[j]; wn[quad * BT + c + j] = (nan_bits >> j) & 1; }
                    }
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (col < BT && t0 + col < T) {
                float bv = wv[col];
                int bi = wi[col], nn = wn[col];
#pragma unroll
                for (int w = 1; w < 4; ++w) {
                    const float ov = wv[w * BT + col];
                    const int oi = wi[w * BT + col];
                    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
                    nn |= wn[w * BT + col];
                }
                qa.part_val[(size_t)(t0 + col) * qa.ld_part + m_tile] = bv;
                qa.part_idx[(size_t)(t0 + col) * qa.ld_part + m_tile] = bi;
                if (nn) atomicExch(qa.nan_flags + t0 + col, 1);
            }
        } else if (ok && !MS) {
#pragma unroll
            for (int c = 0; c < BT; c += 16) {
                float r[16];
                get16(c, r);
#pragma unroll
                for (int j = 0; j < 16; ++j) tile[(c + j) * BM + col] = r[j];
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (splits > 1) {
            // every thread of every block of the cluster: partials are written, peers may read them
            __syncwarp();
            asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        } else {
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        // the same answer in all 128 threads (a wait that gave up has raised the block's flag)
        const bool go = !*abort_flag && !(splits == 1 && EPI == EPI_STORE) && EPI != EPI_PICK;
        if (go) {
            // Step one, all tokens at once (independent loads): under a split, add the peers'
            // partials up through distributed shared memory in rank order; a residual epilogue adds
            // the old residual. Only then do the tokens meet their partners, with no barrier per token.
            if (splits > 1) {
                uint32_t remote[8];
#pragma unroll
                for (int p = 0; p < 8; ++p)
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[p]) : "r"(smem_u32(tile + col)), "r"(p < splits ? p : 0));
#pragma unroll 2
                for (int k = 0; k < nk; ++k) {
                    const int j = tok_first + k * splits;
                    float part[8];
#pragma unroll
                    for (int p = 0; p < 8; ++p) {
                        part[p] = 0.f;
                        if (p < splits)
                            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(part[p]) : "r"(remote[p] + (uint32_t)(j * BM * 4)) : "memory");
                    }
                    float old = 0.f;
                    if (EPI == EPI_RESID && f < N) old = qa.resid[(size_t)(t0 + j) * qa.ld_resid + f];
                    float acc = 0.f;
#pragma unroll
                    for (int p = 0; p < 8; ++p) acc += part[p];       // rank order, zeros beyond the last rank
                    if (EPI == EPI_STORE) {
                        if (f < N) store_out<OutT>(C + (size_t)(t0 + j) * ldc + f, acc);
                    } else {
                        fin[k * BM + col] = old + acc;
                    }
                }
            } else if (EPI == EPI_RESID) {
#pragma unroll 4
                for (int k = 0; k < nk; ++k) {
                    const float old = f < N ? qa.resid[(size_t)(t0 + k) * qa.ld_resid + f] : 0.f;
                    fin[k * BM + col] = old + fin[k * BM + col];
                }
            }
        }
        if (splits > 1 || EPI == EPI_RESID) asm volatile("bar.sync 1, 128;" ::: "memory");
        if (splits > 1 && col < splits) {
            // this block has read what it needs of every peer's partials: tell each of them (a block
            // may leave, and free its shared memory, once all have said so; no second meeting)
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(done_bar)), "r"(col));
            asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
        }
        if (go) {
            if (EPI == EPI_SWIGLU) {
                // columns 0..63: gate of feature m_tile * 64 + col; columns 64..127: up of the same
                // features. The two halves of the threads take alternate tokens.
                const int c = col & (BM / 2 - 1);
                const int fo = m_tile * (BM / 2) + c;
                if (fo < N) {
                    for (int k = col / (BM / 2); k < nk; k += 2) {
                        const float g = fin[k * BM + c], u = fin[k * BM + c + BM / 2];
                        store_out<OutT>(C + (size_t)(t0 + tok_first + k * splits) * ldc + fo, g / (1.0f + expf(-g)) * u);
                    }
                }
            } else if (EPI == EPI_QKV) {
                const int hd = qa.hd, half = hd >> 1, i = f % hd;
                const bool is_q = f < qa.q_dim, is_k = !is_q && f < qa.q_dim + qa.kv_dim;
                const int pcol = i < half ? col + half : col - half;           // the rotation's partner
                const int g = is_q ? 0 : (is_k ? f - qa.q_dim : f - qa.q_dim - qa.kv_dim);
                const int kh = g / hd, d = g - kh * hd;
                auto finish = [&](int k, float c, float s_, int slot) {
                    const int t = t0 + tok_first + k * splits;
                    const float v = fin[k * BM + col];
                    float outv = v;
                    if (rot) {
                        const float partner = fin[k * BM + pcol];
                        outv = i < half ? v * c - partner * s_ : v * c + partner * s_;
                    }
                    if (is_q) {
                        store_out<OutT>(C + (size_t)t * ldc + f, outv);
                    } else if (slot >= 0) {
                        const size_t page = (size_t)(slot / qa.page_size);
                        const int off = slot % qa.page_size;
                        const size_t idx = ((page * qa.KV + kh) * qa.page_size + off) * (size_t)hd + d;
                        (is_k ? qa.kcache : qa.vcache)[idx] = __float2bfloat16_rn(outv);
                    }
                };
                if (f < N) {
#pragma unroll
                    for (int k = 0; k < PRE; ++k)
                        if (k < nk) finish(k, pc[k], ps[k], pslot[k]);
                    for (int k = PRE; k < nk; ++k) {
                        const int t = t0 + tok_first + k * splits;
                        float c = 1.f, s_ = 0.f;
                        if (rot) {
                            const float theta = (float)qa.positions[t] * inv;
                            c = cosf(theta);
                            s_ = sinf(theta);
                        }
                        finish(k, c, s_, is_q ? -1 : (qa.slots ? qa.slots[t] : -1));
                    }
                }
            } else if (EPI == EPI_RESID) {
                for (int k = 0; k < nk; ++k) {
                    const int t = t0 + tok_first + k * splits;
                    float sq = 0.f;
                    if (f < N) {
                        const float r_new = fin[k * BM + col];
                        qa.resid[(size_t)t * qa.ld_resid + f] = r_new;
                        qa.xn_out[(size_t)t * qa.ld_xn + f] = __float2bfloat16_rn(r_new * next_w);
                        sq = r_new * r_new;
                    }
                    sq = warp_sum(sq);
                    if (lane == 0) red[k * 4 + quad] = sq;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                for (int k = col; k < nk; k += 128)
                    qa.ssq_out[(size_t)m_tile * qa.ld_ssq + t0 + tok_first + k * splits] =
                        (red[k * 4] + red[k * 4 + 1]) + (red[k * 4 + 2] + red[k * 4 + 3]);
            }
        }
        // nobody leaves (and frees its shared memory) while a peer may still be reading it; by now
        // the peers' notices have usually come in
        if (splits > 1) {
            volatile int never = 0;          // this wait does not give up early: peers may be reading
            mbar_wait(done_bar, 0, &never, err_flag, 4);
        }
    }
    if (splits > 1 && (warp < 2 || warp >= 6)) {
        // the producer and MMA warps take part in the cluster's barrier as well
        __syncwarp();
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    __syncthreads();
    if (!MS && warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols<BT, EPI>()) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// Many tokens (prompt portions): a persistent form of the same kernel. One block per SM walks
// over output tiles (tile id -> weight-row block id / n_tiles, token block id % n_tiles, so the
// blocks running at one time share weight tiles and keep all of X in L2). The accumulator is
// double buffered in tensor memory (2 x BT columns): while the four epilogue warps drain one
// buffer to C, the MMA warp already fills the other, and the TMA ring runs ahead across tile
// boundaries; so the tensor cores never wait for an epilogue. Bound: tensor-core throughput.
// ------------------------------------------------------------------------------------------------

template <int BT, int STAGES, typename OutT>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_sm100_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                             OutT* __restrict__ C, long long ldc, int T, int N, int K, int* __restrict__ err_flag) {
    pdl_launch_dependents();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + STAGES * stage_bytes<BT>());
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;           // [2]
    uint64_t* acc_empty = acc_full + 2;                // [2]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_kb = (K + BK - 1) / BK;
    const int m_tiles = (N + BM - 1) / BM, n_tiles = (T + BT - 1) / BT;
    const int num_tiles = m_tiles * n_tiles;
    constexpr int ACC_COLS = 2 * BT;                   // 256 or 512 columns: a power of two

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(ACC_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_holder;
    pdl_wait(13);

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m_tile = tile / n_tiles, n_tile = tile % n_tiles;
                for (int kb = 0; kb < total_kb; ++kb, ++it) {
                    int s = it % STAGES;
                    uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty_bar + s, ph ^ 1, abort_flag, err_flag, 1)) { ok = false; break; }
                    unsigned char* a = tiles + s * stage_bytes<BT>();
                    mbar_expect_tx(full_bar + s, stage_bytes<BT>());
                    tma_load_2d(a, &map_w, kb * BK, m_tile * BM, full_bar + s);
                    tma_load_2d(a + BM * BK * 2, &map_x, kb * BK, n_tile * BT, full_bar + s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BT);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
                const uint32_t buf = local & 1, aph = (local >> 1) & 1;
                if (!mbar_wait(acc_empty + buf, aph ^ 1, abort_flag, err_flag, 2)) break;     // drained by the epilogue
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + buf * BT;
                for (int kb = 0; kb < total_kb; ++kb, ++it) {
                    int s = it % STAGES;
                    uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(full_bar + s, ph, abort_flag, err_flag, 2)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    unsigned char* a = tiles + s * stage_bytes<BT>();
                    uint64_t adesc = umma_desc_sw128(a);
                    uint64_t bdesc = umma_desc_sw128(a + BM * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty_bar + s);
                }
                if (ok) umma_commit(acc_full + buf);
            }
        }
    } else {
        const int quad = warp & 3;
        uint32_t local = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
            const int m_tile = tile / n_tiles, n_tile = tile % n_tiles;
            const uint32_t buf = local & 1, aph = (local >> 1) & 1;
            if (!mbar_wait(acc_full + buf, aph, abort_flag, err_flag, 3)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + buf * BT + ((uint32_t)(quad * 32) << 16);
            const int f = m_tile * BM + quad * 32 + lane;
            const int t0 = n_tile * BT;
#pragma unroll 2
            for (int c = 0; c < BT; c += 16) {
                uint32_t r[16];
                tmem_ld16(taddr + c, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (f < N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        int t = t0 + c + j;
                        if (t < T) store_out<OutT>(C + (size_t)t * ldc + f, __uint_as_float(r[j]));
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(acc_empty + buf);                   // 128 arrivals hand the buffer back to the MMA warp
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACC_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------ host side
struct MapKey {
    const void* ptr; long long rows, cols, ld; int box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h ^= std::hash<long long>()(k.rows * 1000003 + k.cols) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        h ^= std::hash<long long>()(k.ld * 131 + k.box_rows) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        return h;
    }
};

// A 2-D bfloat16 tensor [rows, cols] with row stride ld elements; boxes of [box_rows, 64] elements,
// 128-byte swizzle; rows and columns outside the tensor read as zero.
int make_map(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    MapKey key{ptr, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return VOB_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return VOB_ERR_BAD_ARG;
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return 0;
}

template <int BT, int STAGES, int EPI = EPI_STORE> constexpr size_t smem_bytes() {
    return (size_t)STAGES * stage_bytes<BT, EPI>() + 1024 + 1024;       // tiles + alignment slack + barriers and per-token scales
}

// Test hook (see vob_gemm_sm100_test_hooks): bytes by which the next launches over-declare what
// their first stage's barrier expects, so that the barrier never completes and the waits run out.
int g_test_extra_tx = 0;

template <int BT, int STAGES, typename OutT, int EPI>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* C, long long ldc, int T, int N, int K, int splits, int kb_per,
           int* err_flag, int up_row0, const QkvArgs& qa, cudaStream_t stream) {
    // Blocks of a cluster wait for one another, and tcgen05.alloc waits for columns: the blocks that
    // fit one SM by shared memory must all get their tensor memory, or two clusters could wait for
    // each other for ever.
    static_assert((227 * 1024 / smem_bytes<BT, STAGES, EPI>()) * tmem_cols<BT, EPI>() <= 512, "tensor memory oversubscribed");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_sm100_kernel<BT, STAGES, OutT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem_bytes<BT, STAGES, EPI>());
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    constexpr int FEATURES_PER_TILE = EPI == EPI_SWIGLU ? BM / 2 : BM;
    cfg.gridDim = dim3((N + FEATURES_PER_TILE - 1) / FEATURES_PER_TILE, (T + BT - 1) / BT, splits);
    cfg.blockDim = dim3(NTHREADS_FEW);
    cfg.dynamicSmemBytes = smem_bytes<BT, STAGES, EPI>();
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;            // the blocks that share one tile
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_vob_pdl ? 2 : 1;
    // the hook applies to a block on its own only (no cluster whose peers would wait for it)
    const int extra_tx = (splits == 1 && cfg.gridDim.x == 1 && cfg.gridDim.y == 1) ? g_test_extra_tx : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_sm100_kernel<BT, STAGES, OutT, EPI>, mw, mx, (OutT*)C, ldc, T, N, K, kb_per, err_flag,
                                       up_row0, qa, extra_tx);
    return e != cudaSuccess ? (int)e : vob_launch_status();
}

template <int BT, int STAGES, typename OutT>
int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mx, void* C, long long ldc, int T, int N, int K, int* err_flag,
                      cudaStream_t stream) {
    static bool configured = false;
    static int num_sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_sm100_persistent_kernel<BT, STAGES, OutT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<BT, STAGES>());
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (num_sms <= 0) num_sms = 148;
        configured = true;
    }
    int tiles = ((N + BM - 1) / BM) * ((T + BT - 1) / BT);
    int grid = tiles < num_sms ? tiles : num_sms;
    return vob_launch(gemm_sm100_persistent_kernel<BT, STAGES, OutT>, dim3(grid), dim3(NTHREADS), smem_bytes<BT, STAGES>(), stream,
                      mw, mx, (OutT*)C, ldc, T, N, K, err_flag);
}

// Stages of the ring for few tokens: as many as let two blocks share an SM (about 110 KB each).
// With one block per SM the next kernel's blocks (and their clusters, which need all their SMs
// free at one time) cannot move in beside this kernel's: its prefetch before the wait is lost and
// it runs in waves (measured at 32 rows: a QKV product of 8 us in block 0 took 19 us as a grid).
constexpr int few_stages(int bt) { return bt <= 16 ? 6 : bt <= 32 ? 5 : 4; }

int pick_bt(int T) { return T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256; }

}  // namespace

// For the test of the give-up path only. `extra_tx_bytes` > 0: launches of ONE block (one tile, no
// split) declare so many bytes more than their first stage's loads bring, so its barrier never
// completes; `wait_limit_ns` is the limit after which a wait gives up (the default is two seconds;
// 0 puts it back). The block then raises the error word, frees its tensor memory and returns:
// nothing faults and nothing hangs. Call with (0, 0) afterwards.
VOB_EXPORT int vob_gemm_sm100_test_hooks(int extra_tx_bytes, unsigned long long wait_limit_ns) {
    if (extra_tx_bytes < 0 || extra_tx_bytes > 1024) return VOB_ERR_BAD_ARG;
    unsigned long long limit = wait_limit_ns ? wait_limit_ns : WAIT_LIMIT_NS;
    cudaError_t e = cudaMemcpyToSymbol(g_wait_limit_ns, &limit, sizeof(limit));
    if (e != cudaSuccess) return (int)e;
    g_test_extra_tx = extra_tx_bytes;
    return 0;
}

// How many splits of K fill `num_sms` SMs for a product with few tokens (1 when the tiles alone do).
VOB_EXPORT int vob_gemm_sm100_pick_splits(int T, int N, int K, int num_sms) {
    int bt = pick_bt(T);
    int tiles = ((N + BM - 1) / BM) * ((T + bt - 1) / bt);
    int total_kb = (K + BK - 1) / BK;
    if (T > 64 || tiles * 2 > num_sms) return 1;
    int want = num_sms / tiles;
    if (want > 8) want = 8;                                           // the portable cluster size
    int max_splits = total_kb / 4 > 0 ? total_kb / 4 : 1;             // at least 4 k-blocks (256 of K) per split
    int s = want < max_splits ? want : max_splits;
    if (s < 1) s = 1;
    int per = (total_kb + s - 1) / s;
    return (total_kb + per - 1) / per;                                // every split gets at least one k-block
}

// C[T, N] (row stride ldc, bfloat16 or float32) = X[T, K] (row stride ldx) * W[N, K]^T (row stride ldw).
VOB_EXPORT int vob_gemm_sm100(const void* X, long long ldx, const void* W, long long ldw, void* C, long long ldc, int out_code,
                              int T, int N, int K, int splits, int* err_flag, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || ldx < K || ldw < K || ldc < N) return VOB_ERR_BAD_ARG;
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)X % 16) != 0 || ((uintptr_t)W % 16) != 0) return VOB_ERR_UNSUPPORTED;
    if (out_code != VOB_F32 && out_code != VOB_BF16) return VOB_ERR_BAD_ARG;
    int bt = pick_bt(T);
    if (bt == 256) {
        // 256-token tiles unless 128-token tiles fill the SMs in fewer token-columns of work
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        long long mt = (N + BM - 1) / BM;
        long long w256 = ((mt * ((T + 255) / 256) + sms - 1) / sms) * 256;
        long long w128 = ((mt * ((T + 127) / 128) + sms - 1) / sms) * 128;
        if (w128 < w256) bt = 128;
    }
    int total_kb = (K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > 8) splits = 8;
    if (splits > total_kb) splits = total_kb;
    int kb_per = (total_kb + splits - 1) / splits;
    splits = (total_kb + kb_per - 1) / kb_per;
    if ((T + bt - 1) / bt > 65535 || splits > 65535) return VOB_ERR_UNSUPPORTED;
    CUtensorMap mw, mx;
    int e = make_map(&mw, W, N, K, ldw, BM);
    if (e) return e;
    e = make_map(&mx, X, T, K, ldx, bt);
    if (e) return e;
#define GO(BT, ST)                                                                                                         \
    return out_code == VOB_F32                                                                                             \
               ? launch<BT, ST, float, EPI_STORE>(mw, mx, C, ldc, T, N, K, splits, kb_per, err_flag, 0, QkvArgs{}, stream)      \
               : launch<BT, ST, __nv_bfloat16, EPI_STORE>(mw, mx, C, ldc, T, N, K, splits, kb_per, err_flag, 0, QkvArgs{}, stream)
    switch (bt) {
        case 16: GO(16, few_stages(16));
        case 32: GO(32, few_stages(32));
        case 64: GO(64, few_stages(64));
        default: break;
    }
#undef GO
#define GOP(BT, ST)                                                                                                \
    return out_code == VOB_F32 ? launch_persistent<BT, ST, float>(mw, mx, C, ldc, T, N, K, err_flag, stream)          \
                               : launch_persistent<BT, ST, __nv_bfloat16>(mw, mx, C, ldc, T, N, K, err_flag, stream)
    if (bt == 128) { GOP(128, 6); }
    GOP(256, 4);
#undef GOP
}


// ------------------------------------------------------------------------------------------------ fused epilogues (few tokens)
namespace {
int fused_common(int T, int K, long long ldx, long long ldw, const void* X, const void* W, int* splits, int* kb_per) {
    if (T <= 0 || T > 64) return VOB_ERR_UNSUPPORTED;
    if (K <= 0 || ldx < K || ldw < K) return VOB_ERR_BAD_ARG;
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)X % 16) != 0 || ((uintptr_t)W % 16) != 0) return VOB_ERR_UNSUPPORTED;
    int total_kb = (K + BK - 1) / BK;
    if (*splits < 1) *splits = 1;
    if (*splits > 8) *splits = 8;
    if (*splits > total_kb) *splits = total_kb;
    *kb_per = (total_kb + *splits - 1) / *splits;
    *splits = (total_kb + *kb_per - 1) / *kb_per;
    return 0;
}
}  // namespace

// The general entry point for few tokens (T <= 64): any epilogue mode, with an optional per-token
// scale of the accumulator (`ea->ssq_in`, the folded RMSNorm of X). `mode` is one of EPI_*;
// `n_features` is the number of output features (for EPI_SWIGLU: I, with W of shape [2I, K]; for
// EPI_QKV: (H + 2 KV) * hd). `ea` is read on the host at launch time and passed by value.
VOB_EXPORT int vob_gemm_sm100_ex(const void* X, long long ldx, const void* W, long long ldw, void* C, long long ldc, int out_code,
                                 int T, int n_features, int K, int splits, int mode, const EpiArgs* ea, int* err_flag,
                                 cudaStream_t stream) {
    int kb_per = 0;
    int e = fused_common(T, K, ldx, ldw, X, W, &splits, &kb_per);
    if (e) return e;
    if (!ea || n_features <= 0) return VOB_ERR_BAD_ARG;
    if (ea->ssq_in && (ea->ssq_tiles <= 0 || ea->ld_ssq < T)) return VOB_ERR_BAD_ARG;
    if (mode == EPI_PICK) { splits = 1; kb_per = (K + BK - 1) / BK; }     // a tile's best pair is found by one block
    const int N = n_features;
    const long long w_rows = mode == EPI_SWIGLU ? 2LL * N : N;
    int bt = pick_bt(T);
    CUtensorMap mw, mx;
    e = make_map(&mw, W, w_rows, K, ldw, mode == EPI_SWIGLU ? BM / 2 : BM);
    if (e) return e;
    e = make_map(&mx, X, T, K, ldx, bt);
    if (e) return e;
#define GOX(BT_, OUT_, EPI_) return launch<BT_, few_stages(BT_), OUT_, EPI_>(mw, mx, C, ldc, T, N, K, splits, kb_per, err_flag, mode == EPI_SWIGLU ? N : 0, *ea, stream)
    switch (mode) {
        case EPI_STORE:
            if (ldc < N) return VOB_ERR_BAD_ARG;
            if (out_code == VOB_F32) { if (bt == 16) GOX(16, float, EPI_STORE); if (bt == 32) GOX(32, float, EPI_STORE); GOX(64, float, EPI_STORE); }
            if (out_code == VOB_BF16) { if (bt == 16) GOX(16, __nv_bfloat16, EPI_STORE); if (bt == 32) GOX(32, __nv_bfloat16, EPI_STORE); GOX(64, __nv_bfloat16, EPI_STORE); }
            return VOB_ERR_BAD_ARG;
        case EPI_SWIGLU:
            if (ldc < N || out_code != VOB_BF16) return VOB_ERR_BAD_ARG;
            if (bt == 16) GOX(16, __nv_bfloat16, EPI_SWIGLU);
            if (bt == 32) GOX(32, __nv_bfloat16, EPI_SWIGLU);
            GOX(64, __nv_bfloat16, EPI_SWIGLU);
        case EPI_QKV:
            if (out_code != VOB_BF16 || ea->hd <= 0 || (ea->hd & 1) || BM % ea->hd != 0 || ea->page_size <= 0 || !ea->positions ||
                !ea->kcache || !ea->vcache || ldc < ea->q_dim || N != ea->q_dim + 2 * ea->kv_dim)
                return VOB_ERR_BAD_ARG;
            if (bt == 16) GOX(16, __nv_bfloat16, EPI_QKV);
            if (bt == 32) GOX(32, __nv_bfloat16, EPI_QKV);
            GOX(64, __nv_bfloat16, EPI_QKV);
        case EPI_RESID:
            if (!ea->resid || !ea->next_w || !ea->xn_out || !ea->ssq_out || ea->ld_resid < N || ea->ld_xn < N || ea->ld_ssq < T)
                return VOB_ERR_BAD_ARG;
            if (bt == 16) GOX(16, __nv_bfloat16, EPI_RESID);
            if (bt == 32) GOX(32, __nv_bfloat16, EPI_RESID);
            GOX(64, __nv_bfloat16, EPI_RESID);
        case EPI_PICK:
            if (!ea->part_val || !ea->part_idx || !ea->nan_flags || ea->ld_part < (N + BM - 1) / BM || splits != 1 ||
                (ea->temperature && (!ea->seeds || !ea->steps)))
                return VOB_ERR_BAD_ARG;
            if (bt == 16) GOX(16, float, EPI_PICK);
            if (bt == 32) GOX(32, float, EPI_PICK);
            GOX(64, float, EPI_PICK);
        default:
            return VOB_ERR_BAD_ARG;
    }
#undef GOX
}

// C[T, I] = silu(X Wg^T) * (X Wu^T), W = [Wg; Wu] of shape [2I, K]; T <= 64.
VOB_EXPORT int vob_gemm_sm100_swiglu(const void* X, long long ldx, const void* W, long long ldw, void* C, long long ldc, int T,
                                     int I, int K, int splits, int* err_flag, cudaStream_t stream) {
    EpiArgs ea = {};
    return vob_gemm_sm100_ex(X, ldx, W, ldw, C, ldc, VOB_BF16, T, I, K, splits, EPI_SWIGLU, &ea, err_flag, stream);
}

// [q | k | v] = X [Wq; Wk; Wv]^T with rotary positions on q and k; q (rotated) -> Q[T, q_dim], rotated k
// and v -> their cache slots. T <= 64, 128 a multiple of head_dim.
VOB_EXPORT int vob_gemm_sm100_qkv(const void* X, long long ldx, const void* W, long long ldw, void* Q, long long ldq, int T, int K,
                                  int splits, int* err_flag, const int* positions, const int* slots, const float* inv_freq,
                                  void* kcache, void* vcache, int H, int KV, int hd, int page_size, cudaStream_t stream) {
    if (H <= 0 || KV <= 0 || hd <= 0 || (hd & 1) || BM % hd != 0 || page_size <= 0) return VOB_ERR_UNSUPPORTED;
    EpiArgs ea = {};
    ea.positions = positions; ea.slots = slots; ea.inv_freq = inv_freq;
    ea.kcache = (__nv_bfloat16*)kcache; ea.vcache = (__nv_bfloat16*)vcache;
    ea.q_dim = H * hd; ea.kv_dim = KV * hd; ea.hd = hd; ea.KV = KV; ea.page_size = page_size;
    return vob_gemm_sm100_ex(X, ldx, W, ldw, Q, ldq, VOB_BF16, T, (H + 2 * KV) * hd, K, splits, EPI_QKV, &ea, err_flag, stream);
}
