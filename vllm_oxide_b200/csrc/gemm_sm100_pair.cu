// bfloat16 matrix product for many tokens on pairs of SMs: C[T, N] = X[T, K] * W[N, K]^T.
// Reference op: crates/engine/src/backend/cpu/mod.rs:199-229 (x * W^T, W [out, in] row-major).
//
// Two blocks on neighbouring SMs (a cluster of two) share every tensor-core instruction
// (tcgen05.mma.cta_group::2): one instruction multiplies 256 weight rows by 256 tokens, each block
// holding its 128 weight rows (the A operand) and its 128 of the 256 tokens (half of the B
// operand) in its own shared memory, and each block's tensor memory receives its 128 weight rows
// of the result for all 256 tokens. Per byte of operand fetched from shared memory an SM does
// twice the work of a one-SM instruction, and one issued instruction (an issuing thread gets one
// through in about 125-170 clocks whatever its size) is worth 256 clocks of tensor-core time on
// each SM: that is what lifts this kernel over the one-SM persistent product.
//
// Roles in each block of 320 threads: warp 0 (one lane) issues its block's TMA loads, whose bytes
// are counted on the leader block's barrier (cp.async.bulk.tensor with .cta_group::2; no
// multicast); warp 1 owns the tensor memory and, in the leader block only, issues the products and
// commits them to both blocks' barriers (tcgen05.commit ... multicast::cluster); warps 2-9, two
// groups of four taking alternate rounds of 16 tokens, read their block's accumulator and write C
// (through shared memory, so that C is written in 16-byte pieces). The kernel is persistent: a pair walks over output tiles
// (256 weight rows x 256 tokens), the accumulator is double buffered (2 x 256 columns), the TMA
// ring runs ahead across tile boundaries.
//
// Every mbarrier wait is bounded (sm100.cuh); a block that gives up still meets its partner at the
// cluster barriers at the start and the end, so neither is left waiting.
#include "common.cuh"
VOB_PDL_SWITCH(gemm_sm100_pair)
#include "sm100.cuh"
#include <unordered_map>

namespace {
using namespace vob_sm100;

constexpr int BMH = 128;          // weight rows per block (256 per pair)
constexpr int BTH = 128;          // tokens per block (256 per pair)
constexpr int BK = 64;            // K elements per stage: 128 bytes, one swizzle span
constexpr int UMMA_K = 16;
constexpr int NTHREADS = 320;          // TMA warp, MMA warp, two epilogue groups of four warps
constexpr int EPI_GROUP_BYTES = 12288;  // per epilogue group: exchange and staging buffers
constexpr int STAGES = 6;
constexpr int STAGE_BYTES = (BMH + BTH) * BK * 2;            // 32 KB per block and stage
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;                  // a shared::cluster address with this mask is the pair's even block's

template <typename OutT> __device__ __forceinline__ void store_out(OutT* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A tile load whose bytes are counted on the barrier at the same offset in the pair's even block.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & PEER_MASK), "r"(x), "r"(y) : "memory");
}
// D[tmem of both blocks] (+)= A[smem of both blocks] * B[smem of both blocks]; issued by the even block.
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// All products issued so far by this thread complete -> one arrival on the barrier at this offset in both blocks.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
// One arrival on the barrier at this offset in the pair's even block.
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & PEER_MASK) : "memory");
}

// Epilogues. STORE: C[t, f] = acc. SWIGLU: the weight matrix is [Wg; Wu] ([2 * N, K]); a block's 128
// operand rows are 64 gate rows and the 64 up rows of the same features (two TMA boxes), so its
// accumulator holds both halves of 64 features and the epilogue writes C[t, f] = silu(gate) * up
// (crates/engine/src/backend/cpu/mod.rs:341-349; crates/engine/src/model.rs:325-331) without the
// gate / up activations ever going to memory. N counts output features in both modes.
enum { PAIR_STORE = 0, PAIR_SWIGLU = 1 };

template <typename OutT, int EPI>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_sm100_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                       OutT* __restrict__ C, long long ldc, int T, int N, int K, int wide, int* __restrict__ err_flag) {
    constexpr int FEATS = EPI == PAIR_SWIGLU ? BMH / 2 : BMH;        // output features per block and tile
    pdl_launch_dependents();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);      // [STAGES] used in the even block
    uint64_t* empty_bar = full_bar + STAGES;                                             // [STAGES] in both blocks
    uint64_t* acc_full = empty_bar + STAGES;                                             // [2] in both blocks
    uint64_t* acc_empty = acc_full + 2;                                                  // [2] used in the even block
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    // epilogue exchange, 8 KB, 16-byte aligned, behind 256 bytes of barriers: 2 x [16 tokens][128 features] bfloat16 or 2 x [8 tokens][2][64 features] float32
    float* xch = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(full_bar) + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();              // 0: the even block (issues the products), 1: its partner
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int total_kb = (K + BK - 1) / BK;
    const int m_tiles = (N + 2 * FEATS - 1) / (2 * FEATS), n_tiles = (T + 2 * BTH - 1) / (2 * BTH);
    const int num_tiles = m_tiles * n_tiles;
    constexpr int ACC_COLS = 512;                         // two accumulators of 256 token columns

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 512); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(ACC_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();                                   // both blocks' barriers exist before either signals the other's
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    pdl_wait(15);

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                const int m_tile = tile / n_tiles, n_tile = tile % n_tiles;
                for (int kb = 0; kb < total_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty_bar + s, ph ^ 1, abort_flag, err_flag, 31)) { ok = false; break; }
                    unsigned char* a = tiles + s * STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(full_bar + s, 2 * STAGE_BYTES);        // both blocks' bytes
                    if (EPI == PAIR_SWIGLU) {
                        const int f0 = (m_tile * 2 + (int)rank) * FEATS;
                        tma_load_2d_pair(a, &map_w, kb * BK, f0, full_bar + s);                             // 64 gate rows
                        tma_load_2d_pair(a + FEATS * BK * 2, &map_w, kb * BK, N + f0, full_bar + s);        // their up rows
                    } else {
                        tma_load_2d_pair(a, &map_w, kb * BK, m_tile * 2 * BMH + (int)rank * BMH, full_bar + s);
                    }
                    tma_load_2d_pair(a + BMH * BK * 2, &map_x, kb * BK, n_tile * 2 * BTH + (int)rank * BTH, full_bar + s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(2 * BMH, 2 * BTH, false);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
                const uint32_t buf = local & 1, aph = (local >> 1) & 1;
                if (!mbar_wait(acc_empty + buf, aph ^ 1, abort_flag, err_flag, 32)) break;      // drained by both blocks' epilogues
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * (2 * BTH);
                for (int kb = 0; kb < total_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(full_bar + s, ph, abort_flag, err_flag, 32)) { ok = false; break; }
                    tcgen05_fence_after();
                    unsigned char* a = tiles + s * STAGE_BYTES;
                    const uint64_t adesc = umma_desc_sw128(a);
                    const uint64_t bdesc = umma_desc_sw128(a + BMH * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(empty_bar + s);                  // the stage is free in both blocks
                }
                if (ok) umma_commit_pair(acc_full + buf);             // the accumulator is complete in both blocks
            }
        }
    } else {
        // Epilogue: two groups of four warps (a warp reaches the 32 lanes of tensor memory given by its
        // index modulo 4, so each group covers all 128); the groups take alternate rounds of 16 tokens.
        const int quad = warp & 3;
        const int grp = (warp - 2) >> 2;                          // 0 or 1
        const int row = quad * 32 + lane;                         // 0..127: lane of tensor memory
        unsigned char* xg = reinterpret_cast<unsigned char*>(xch) + grp * EPI_GROUP_BYTES;
        const uint32_t bar_id = 1 + grp;
        auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory"); };
        uint32_t local = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
            const int m_tile = tile / n_tiles, n_tile = tile % n_tiles;
            const uint32_t buf = local & 1, aph = (local >> 1) & 1;
            bool ok = mbar_wait(acc_full + buf, aph, abort_flag, err_flag, 33);
            {
                // the warps of a group meet at named barriers below: they give up together or not at all
                uint32_t all_ok;
                asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, %2, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                             : "=r"(all_ok) : "r"((uint32_t)ok), "r"(bar_id) : "memory");
                ok = all_ok != 0;
            }
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + buf * (2 * BTH) + ((uint32_t)(quad * 32) << 16);
            const int t0 = n_tile * 2 * BTH;
            if (EPI == PAIR_STORE && sizeof(OutT) == 2 && wide) {
                // 16 tokens at a time through shared memory, so that C is written in 16-byte pieces
                // along the features (a thread of the accumulator holds one feature of 16 tokens:
                // stored directly that would be 2-byte writes). Two buffers, one barrier per round.
                __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(xg);
                const int fbase = m_tile * 2 * BMH + (int)rank * BMH;
                for (int round = grp, n = 0; round < 2 * BTH / 16; round += 2, ++n) {
                    const int c = round * 16;
                    uint32_t r[16];
                    tmem_ld16(taddr + c, r);
                    tmem_wait_ld();
                    __nv_bfloat16* sb = stg + (n & 1) * (16 * BMH);
#pragma unroll
                    for (int j = 0; j < 16; ++j) sb[j * BMH + row] = __float2bfloat16_rn(__uint_as_float(r[j]));
                    group_sync();
#pragma unroll
                    for (int q = row; q < 16 * (BMH / 8); q += 128) {
                        const int tok = q / (BMH / 8), part = q % (BMH / 8);
                        const int t = t0 + c + tok, f0 = fbase + part * 8;
                        if (t < T && f0 < N)
                            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(C) + (size_t)t * ldc + f0) =
                                *reinterpret_cast<const uint4*>(sb + tok * BMH + part * 8);
                    }
                }
                group_sync();                                      // the buffers are free for the next tile
            } else if (EPI == PAIR_STORE) {
                const int f = m_tile * 2 * BMH + (int)rank * BMH + row;
                for (int round = grp; round < 2 * BTH / 16; round += 2) {
                    const int c = round * 16;
                    uint32_t r[16];
                    tmem_ld16(taddr + c, r);
                    tmem_wait_ld();
                    if (f < N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int t = t0 + c + j;
                            if (t < T) store_out<OutT>(C + (size_t)t * ldc + f, __uint_as_float(r[j]));
                        }
                    }
                }
            } else {
                // lanes 0..63 of the accumulator are gate, 64..127 the up values of the same features.
                // 16 tokens at a time the two halves swap what the other needs through shared memory:
                // the gate threads finish tokens 0..7 of the round, the up threads tokens 8..15, so all
                // threads share the activation's work. The results go to a staging tile and from there
                // to C in 16-byte pieces along the features (when C's rows allow it).
                const bool is_gate = row < FEATS;
                const int fl = row & (FEATS - 1);                 // feature within the block's 64
                const int fbase = (m_tile * 2 + (int)rank) * FEATS;
                float* xbuf = reinterpret_cast<float*>(xg);                                   // 2 x [8][2][64] float32
                __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(xg + 2 * 8 * 2 * FEATS * 4);   // 2 x [16][64] bfloat16
                for (int round = grp, n = 0; round < 2 * BTH / 16; round += 2, ++n) {
                    const int c = round * 16;
                    uint32_t r[16];
                    tmem_ld16(taddr + c, r);
                    tmem_wait_ld();
                    float* x = xbuf + (n & 1) * (8 * 2 * FEATS);
                    // gate threads hand over their tokens 8..15, up threads their tokens 0..7
#pragma unroll
                    for (int j = 0; j < 8; ++j) x[(j * 2 + (is_gate ? 0 : 1)) * FEATS + fl] = __uint_as_float(r[is_gate ? 8 + j : j]);
                    group_sync();
                    __nv_bfloat16* sb = stg + (n & 1) * (16 * FEATS);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int tok = is_gate ? j : 8 + j;
                        const float other = x[(j * 2 + (is_gate ? 1 : 0)) * FEATS + fl];
                        const float g = is_gate ? __uint_as_float(r[j]) : other;
                        const float u = is_gate ? other : __uint_as_float(r[8 + j]);
                        // silu(g) * u with the special-function unit's 2^x and reciprocal (a few units in
                        // the last place of float32, far inside the bfloat16 rounding of the result): the
                        // precise expf and division made this epilogue longer than the tile's products
                        // (measured: 133-187 us per call against 94 us for the products alone)
                        float e, rcp;
                        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-g * 1.4426950408889634f));
                        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp) : "f"(1.0f + e));
                        const float y = g * rcp * u;
                        if (wide) sb[tok * FEATS + fl] = __float2bfloat16_rn(y);
                        else if (t0 + c + tok < T && fbase + fl < N) store_out<OutT>(C + (size_t)(t0 + c + tok) * ldc + fbase + fl, y);
                    }
                    if (wide) {
                        group_sync();
                        const int tok = row / (FEATS / 8), part = row % (FEATS / 8);          // 16 tokens x 8 pieces = 128 threads
                        const int t = t0 + c + tok, f0 = fbase + part * 8;
                        if (t < T && f0 < N)
                            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(C) + (size_t)t * ldc + f0) =
                                *reinterpret_cast<const uint4*>(sb + tok * FEATS + part * 8);
                    }
                }
                group_sync();                                      // the buffers are free for the next tile
            }
            tcgen05_fence_before();
            mbar_arrive_leader(acc_empty + buf);            // 512 arrivals (both blocks) hand the buffer back
        }
        tcgen05_fence_before();
    }
    __syncthreads();
    cluster_sync_all();                                     // nobody leaves while its partner may still signal or read it
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACC_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------ host side
struct MapKey {
    const void* ptr; long long rows, cols, ld;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h ^= std::hash<long long>()(k.rows * 1000003 + k.cols) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        h ^= std::hash<long long>()(k.ld) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        return h;
    }
};

// A 2-D bfloat16 tensor [rows, cols] with row stride ld elements; boxes of [128, 64] elements,
// 128-byte swizzle; rows and columns outside the tensor read as zero.
int make_map(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    MapKey key{ptr, rows, cols, ld * 256 + box_rows};
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

constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024 + 256 + 2 * EPI_GROUP_BYTES;     // tiles, alignment slack, barriers, epilogue buffers

template <typename OutT, int EPI>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* C, long long ldc, int T, int N, int K, int* err_flag, cudaStream_t stream) {
    // 16-byte stores of C need aligned rows and a feature count that no piece of 8 straddles
    const int wide = (ldc % 8 == 0 && ((uintptr_t)C & 15) == 0 && N % 8 == 0) ? 1 : 0;
    static bool configured = false;
    static int num_sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_sm100_pair_kernel<OutT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (num_sms <= 0) num_sms = 148;
        configured = true;
    }
    constexpr int FEATS = EPI == PAIR_SWIGLU ? BMH / 2 : BMH;
    const long long tiles = (long long)((N + 2 * FEATS - 1) / (2 * FEATS)) * ((T + 2 * BTH - 1) / (2 * BTH));
    long long pairs = num_sms / 2;
    if (tiles < pairs) pairs = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_vob_pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_sm100_pair_kernel<OutT, EPI>, mw, mx, (OutT*)C, ldc, T, N, K, wide, err_flag);
    return e != cudaSuccess ? (int)e : vob_launch_status();
}

}  // namespace

// C[T, N] (row stride ldc, bfloat16 or float32) = X[T, K] (row stride ldx) * W[N, K]^T (row stride ldw).
VOB_EXPORT int vob_gemm_sm100_pair(const void* X, long long ldx, const void* W, long long ldw, void* C, long long ldc, int out_code,
                                   int T, int N, int K, int* err_flag, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || ldx < K || ldw < K || ldc < N) return VOB_ERR_BAD_ARG;
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)X % 16) != 0 || ((uintptr_t)W % 16) != 0) return VOB_ERR_UNSUPPORTED;
    if (out_code != VOB_F32 && out_code != VOB_BF16) return VOB_ERR_BAD_ARG;
    CUtensorMap mw, mx;
    int e = make_map(&mw, W, N, K, ldw, BMH);
    if (e) return e;
    e = make_map(&mx, X, T, K, ldx, BTH);
    if (e) return e;
    return out_code == VOB_F32 ? launch<float, PAIR_STORE>(mw, mx, C, ldc, T, N, K, err_flag, stream)
                               : launch<__nv_bfloat16, PAIR_STORE>(mw, mx, C, ldc, T, N, K, err_flag, stream);
}

// C[T, I] (bfloat16) = silu(X Wg^T) * (X Wu^T), W = [Wg; Wu] of shape [2I, K].
VOB_EXPORT int vob_gemm_sm100_pair_swiglu(const void* X, long long ldx, const void* W, long long ldw, void* C, long long ldc,
                                          int T, int I, int K, int* err_flag, cudaStream_t stream) {
    if (T <= 0 || I <= 0) return 0;
    if (K <= 0 || ldx < K || ldw < K || ldc < I) return VOB_ERR_BAD_ARG;
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)X % 16) != 0 || ((uintptr_t)W % 16) != 0) return VOB_ERR_UNSUPPORTED;
    CUtensorMap mw, mx;
    int e = make_map(&mw, W, 2LL * I, K, ldw, BMH / 2);         // boxes of 64 rows: half a block's operand from each half of W
    if (e) return e;
    e = make_map(&mx, X, T, K, ldx, BTH);
    if (e) return e;
    return launch<__nv_bfloat16, PAIR_SWIGLU>(mw, mx, C, ldc, T, I, K, err_flag, stream);
}
