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
// neither large nor a multiple of eight.  A block of eight warps takes ROWS rows of A and walks
// the outputs four at a time: a thread's 16-byte pieces k = t, t + 256, ... of the rows and of
// four weight rows are loaded side by side (one round trip to memory), multiplied in float32,
// summed over the warp by shuffles and over the warps in a fixed order.  A row's result depends on
// nothing but K, whatever ROWS is.  K is a multiple of eight and both operands are 16-byte aligned.
namespace {
constexpr int kSkinnyThreads = 256;

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

template <int ROWS>
__global__ void __launch_bounds__(kSkinnyThreads) linear_skinny_kernel(float* __restrict__ C,
                                                                       const __nv_bfloat16* __restrict__ A,
                                                                       const __nv_bfloat16* __restrict__ W, int M, int N,
                                                                       int vecs) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float part[kSkinnyThreads / 32][ROWS * 4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m0 = blockIdx.x * ROWS;
    const uint4* a = reinterpret_cast<const uint4*>(A);
    const uint4* w = reinterpret_cast<const uint4*>(W);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int n0 = 0; n0 < N; n0 += 4) {
        float acc[ROWS][4];
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[r][j] = 0.f;
        for (int i = threadIdx.x; i < vecs; i += kSkinnyThreads) {
            uint4 av[ROWS], wv[4];
#pragma unroll
            for (int r = 0; r < ROWS; ++r) av[r] = m0 + r < M ? a[(size_t)(m0 + r) * vecs + i] : zero;
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = n0 + j < N ? __ldg(w + (size_t)(n0 + j) * vecs + i) : zero;
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[r][j] = dot8(av[r], wv[j], acc[r][j]);
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float total = warp_sum(acc[r][j]);
                if (lane == 0) part[warp][r * 4 + j] = total;
            }
        __syncthreads();
        if (threadIdx.x < ROWS * 4) {
            const int r = threadIdx.x >> 2, j = threadIdx.x & 3;
            float total = 0.f;
#pragma unroll
            for (int k = 0; k < kSkinnyThreads / 32; ++k) total += part[k][threadIdx.x];
            if (m0 + r < M && n0 + j < N) C[(size_t)(m0 + r) * N + n0 + j] = total;
        }
        __syncthreads();
    }
}
}  // namespace

THN_API int thn_linear_skinny_supported(int N, int K) { return N >= 1 && N <= 64 && K >= 8 && K % 8 == 0; }

THN_API int thn_linear_skinny_bf16(float* C, const void* A, const void* W, int M, int N, int K, cudaStream_t stream) {
    THN_CHECK_ARG(M >= 0 && thn_linear_skinny_supported(N, K), "linear_skinny: bad sizes M=%d N=%d K=%d", M, N, K);
    THN_CHECK_ARG((((uintptr_t)A | (uintptr_t)W) & 15) == 0, "linear_skinny: operands must be 16-byte aligned (M=%d)", M);
    if (M == 0) return THN_OK;
    if (M >= 1024)      // enough rows to fill the SMs four at a time: the weight's rows are read a quarter as often
        thn_launch(linear_skinny_kernel<4>, (M + 3) / 4, kSkinnyThreads, 0, stream, C, (const __nv_bfloat16*)A,
                   (const __nv_bfloat16*)W, M, N, K / 8);
    else
        thn_launch(linear_skinny_kernel<1>, M, kSkinnyThreads, 0, stream, C, (const __nv_bfloat16*)A,
                   (const __nv_bfloat16*)W, M, N, K / 8);
    return thn_launch_status("linear_skinny");
}
