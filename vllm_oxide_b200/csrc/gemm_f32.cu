// True 32-bit matrix product: C[M, N] = A[M, K] * W[N, K]^T, float32 in, float32 FMA, float32
// out. No tensor cores, no TF32, no split over K: each output element is one chain of FMAs over
// k = 0, 1, 2, ... in order, so its value does not depend on M, on the position of its row in
// the batch, or on what else runs. This is the matrix product of the 32-bit engine; it exists
// to show faults that bfloat16 rounding would hide, not to be fast.
// Reference op: crates/engine/src/backend/cpu/mod.rs:199-229 (x * W^T with W [out, in]).
// Launch: 64x64 output tile per block, 256 threads, 4x4 outputs per thread, K in slabs of 16
// through shared memory. Bound: CUDA-core FMA throughput. Any M, N, K >= 1; edges are guarded.
#include "common.cuh"
VOB_PDL_SWITCH(gemm_f32)

#define TM 64
#define TN 64
#define TK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, long long lda, const float* __restrict__ W, long long ldw,
                float* __restrict__ C, long long ldc, int M, int N, int K) {
    pdl_launch_dependents();
    pdl_wait(11);
    __shared__ float As[TK][TM + 4];
    __shared__ float Ws[TK][TN + 4];
    int tid = threadIdx.x;
    int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    int tx = tid & 15, ty = tid >> 4;          // outputs: rows ty*4.., cols tx*4..
    int lr = tid >> 2, lk = (tid & 3) * 4;     // loads: row lr of the tile, k offset lk..lk+3
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    bool vecA = ((lda & 3) == 0) && ((((uintptr_t)A) & 15) == 0);
    bool vecW = ((ldw & 3) == 0) && ((((uintptr_t)W) & 15) == 0);
    for (int k0 = 0; k0 < K; k0 += TK) {
        {
            int gm = m0 + lr, gk = k0 + lk;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (gm < M) {
                const float* p = A + (size_t)gm * lda + gk;
                if (vecA && gk + 3 < K) {
                    float4 f = *reinterpret_cast<const float4*>(p);
                    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) if (gk + i < K) v[i] = p[i];
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) As[lk + i][lr] = v[i];
        }
        {
            int gn = n0 + lr, gk = k0 + lk;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (gn < N) {
                const float* p = W + (size_t)gn * ldw + gk;
                if (vecW && gk + 3 < K) {
                    float4 f = *reinterpret_cast<const float4*>(p);
                    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) if (gk + i < K) v[i] = p[i];
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) Ws[lk + i][lr] = v[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
        }
    }
}

VOB_EXPORT int vob_gemm_f32(const float* A, long long lda, const float* W, long long ldw, float* C,
                            long long ldc, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return VOB_ERR_BAD_ARG;
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    if (grid.y > 65535) return VOB_ERR_UNSUPPORTED;
    return vob_launch(gemm_f32_kernel, grid, dim3(256), 0, stream, A, lda, W, ldw, C, ldc, M, N, K);
}
