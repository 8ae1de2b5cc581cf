// C[M, N] = A[M, K] @ W[N, K]^T in true float32 on the CUDA cores (FFMA only: no
// tensor cores, no TF32).  It is the matrix product of the 32-bit path, where the
// reference calls a library product with TF32 disabled (engine/engine.py:113-114,
// :341-350).  Every output element accumulates k = 0, 1, 2, ... in one accumulator, so a
// row's result does not depend on how many other rows the call has.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256) gemm_f32_kernel(float* __restrict__ C, const float* __restrict__ A,
                                                       const float* __restrict__ W, int M, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements per operand, 256 threads: 4 each; consecutive threads walk k.
        for (int e = tid; e < BM * BK; e += 256) {
            const int r = e / BK, c = e % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? A[(size_t)gm * K + gk] : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? W[(size_t)gn * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * N + gn] = acc[i][j];
        }
    }
}
}  // namespace

THN_API int thn_gemm_f32(float* C, const float* A, const float* W, int M, int N, int K, cudaStream_t stream) {
    THN_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return THN_OK;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    THN_UNSUPPORTED_IF(grid.y > 65535, "gemm_f32: %d rows exceed the grid limit", M);
    thn_launch(gemm_f32_kernel, grid, 256, 0, stream, C, A, W, M, N, K);
    return thn_launch_status("gemm_f32");
}

// ------------------------------------------------------------------ a few outputs per row, float32 out
//
// C[M, N] float32 = A[M, K] bfloat16 @ W[N, K]^T bfloat16 for a weight of few rows (a router, a
// gate of one number per token): the products that vendor libraries serve worst, since N is
// neither large nor a multiple of eight.  One warp per row of A: the row's 16-byte pieces stay in
// the L1 cache while the warp walks the outputs four at a time; every lane accumulates its
// pieces k = lane, lane + 32, ... in float32 and the lanes are summed by shuffles, so a row's
// result depends on nothing but K.  K is a multiple of eight and both operands are 16-byte
// aligned.
namespace {
constexpr int kSkinnyWarps = 8;

__device__ __forceinline__ float dot8(const uint4& a, const uint4& b, float acc) {
    const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* y = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 u = __bfloat1622float2(x[i]), v = __bfloat1622float2(y[i]);
        acc = fmaf(u.x, v.x, acc);
        acc = fmaf(u.y, v.y, acc);
    }
    return acc;
}

__global__ void __launch_bounds__(kSkinnyWarps * 32) linear_skinny_kernel(float* __restrict__ C,
                                                                          const __nv_bfloat16* __restrict__ A,
                                                                          const __nv_bfloat16* __restrict__ W, int M, int N,
                                                                          int vecs) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int m = blockIdx.x * kSkinnyWarps + (threadIdx.x >> 5);
    if (m >= M) return;
    const uint4* a = reinterpret_cast<const uint4*>(A) + (size_t)m * vecs;
    const uint4* w = reinterpret_cast<const uint4*>(W);
    for (int n0 = 0; n0 < N; n0 += 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const int live = min(4, N - n0);
        for (int i = lane; i < vecs; i += 32) {
            const uint4 av = a[i];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (j < live) acc[j] = dot8(av, __ldg(w + (size_t)(n0 + j) * vecs + i), acc[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float total = warp_sum(acc[j]);
            if (j < live && lane == 0) C[(size_t)m * N + n0 + j] = total;
        }
    }
}
}  // namespace

THN_API int thn_linear_skinny_supported(int N, int K) { return N >= 1 && N <= 64 && K >= 8 && K % 8 == 0; }

THN_API int thn_linear_skinny_bf16(float* C, const void* A, const void* W, int M, int N, int K, cudaStream_t stream) {
    THN_CHECK_ARG(M >= 0 && thn_linear_skinny_supported(N, K), "linear_skinny: bad sizes M=%d N=%d K=%d", M, N, K);
    THN_CHECK_ARG((((uintptr_t)A | (uintptr_t)W) & 15) == 0, "linear_skinny: operands must be 16-byte aligned (M=%d)", M);
    if (M == 0) return THN_OK;
    thn_launch(linear_skinny_kernel, (M + kSkinnyWarps - 1) / kSkinnyWarps, kSkinnyWarps * 32, 0, stream, C,
               (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, M, N, K / 8);
    return thn_launch_status("linear_skinny");
}
