// Hyper-connections: a residual stream of s parallel copies per token, kept in float32.
//
// A sublayer f with the numbers a[s] (read), M[s][s] (mix, indexed [from][to]) and b[s] (write)
// does, for the streams X_0 .. X_(s-1) of a token,
//
//     u = sum_j a[j] X_j;   y = f(norm(u));   X'_i = sum_j M[j][i] X_j + b[i] y      (all i at once)
//
// hyper_norm is what stands between two sublayers, in one kernel: the write of the sublayer
// that has just produced y (its M and b), then the read of the next one (its a) and the RMS norm
// of what was read, u / sqrt(mean(u^2) + eps) * g with g one number or a vector:
//
//     write   X <- M^T X + b y          (absent at the start of the model)
//     read    n = norm(sum_j a[j] X_j)  (absent after the last sublayer if nothing reads)
//
// At the start of the model every stream is the embedding's row (start = 1: X is written from
// x0 [rows, width], not read).  With s = 1, M = [[1]], a = b = [1] this is the plain pre-norm
// residual x <- x + y, n = norm(x).  With a = ones it reads the sum of the streams, which is
// what the model's last norm sees.  float32 inside, one rounding at the store of n; one block per
// row, the row of u staged in shared memory, sums in an order that depends on the sizes only.
#include "common.cuh"

namespace {

constexpr int kMaxStreams = 16;
constexpr int kThreads = 256;

struct HyperNumbers {
    float mix[kMaxStreams * kMaxStreams];
    float write[kMaxStreams];
    float read[kMaxStreams];
};

template <typename T, int S>
__global__ void __launch_bounds__(kThreads) hyper_norm_kernel(
    T* __restrict__ n_out, float* __restrict__ X, const float* __restrict__ x0, const T* __restrict__ y,
    const float* __restrict__ mix, const float* __restrict__ write, const float* __restrict__ read,
    const float* __restrict__ gain, int gain_is_vector, float eps, int width, int n_streams) {
    pdl_launch_dependents();
    extern __shared__ float staged[];          // [width]: u
    __shared__ float scratch[33];
    __shared__ HyperNumbers numbers;
    const int s = S > 0 ? S : n_streams;
    // the numbers are weights: they may be read before the kernels ahead have finished
    for (int i = threadIdx.x; i < s * s; i += kThreads) numbers.mix[i] = mix ? mix[i] : 0.f;
    for (int i = threadIdx.x; i < s; i += kThreads) {
        numbers.write[i] = write ? write[i] : 0.f;
        numbers.read[i] = read ? read[i] : 0.f;
    }
    pdl_wait();
    __syncthreads();
    const size_t row = blockIdx.x;
    float* Xr = X + row * (size_t)s * width;
    const bool writes = y != nullptr;
    float ss = 0.f;
    for (int w = threadIdx.x; w < width; w += kThreads) {
        float x[S > 0 ? S : kMaxStreams];
#pragma unroll
        for (int j = 0; j < (S > 0 ? S : kMaxStreams); ++j)
            if (j < s) x[j] = x0 ? x0[row * width + w] : Xr[(size_t)j * width + w];
        float u = 0.f;
        if (writes) {
            const float yv = to_f32<T>(y[row * width + w]);
#pragma unroll
            for (int i = 0; i < (S > 0 ? S : kMaxStreams); ++i) {
                if (i >= s) break;
                float v = 0.f;
#pragma unroll
                for (int j = 0; j < (S > 0 ? S : kMaxStreams); ++j)
                    if (j < s) v += numbers.mix[j * s + i] * x[j];
                v += numbers.write[i] * yv;
                Xr[(size_t)i * width + w] = v;
                u += numbers.read[i] * v;
            }
        } else {
#pragma unroll
            for (int i = 0; i < (S > 0 ? S : kMaxStreams); ++i) {
                if (i >= s) break;
                if (x0) Xr[(size_t)i * width + w] = x[i];
                u += numbers.read[i] * x[i];
            }
        }
        staged[w] = u;
        ss += u * u;
    }
    if (n_out == nullptr) return;
    const float total = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(total / (float)width + eps);
    const float g0 = gain_is_vector ? 1.f : gain[0];
    for (int w = threadIdx.x; w < width; w += kThreads)
        n_out[row * width + w] = from_f32<T>(staged[w] * rstd * (gain_is_vector ? gain[w] : g0));
}

template <typename T>
int launch(void* n_out, float* X, const float* x0, const void* y, const float* mix, const float* write, const float* read,
           const float* gain, int gain_is_vector, float eps, int rows, int width, int s, cudaStream_t stream) {
    const size_t smem = (size_t)width * sizeof(float);
    THN_UNSUPPORTED_IF(smem > 200 * 1024, "hyper_norm: rows of %d do not fit shared memory", width);
#define THN_HYPER_LAUNCH(S)                                                                                              \
    do {                                                                                                                 \
        if (smem > 32 * 1024)                                                                                            \
            cudaFuncSetAttribute(hyper_norm_kernel<T, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        thn_launch(hyper_norm_kernel<T, S>, rows, kThreads, smem, stream, (T*)n_out, X, x0, (const T*)y, mix, write, read, \
                   gain, gain_is_vector, eps, width, s);                                                                 \
    } while (0)
    if (s == 1) THN_HYPER_LAUNCH(1);
    else if (s == 2) THN_HYPER_LAUNCH(2);
    else if (s == 4) THN_HYPER_LAUNCH(4);
    else THN_HYPER_LAUNCH(0);
#undef THN_HYPER_LAUNCH
    return thn_launch_status("hyper_norm");
}

}  // namespace

// X float32 [rows, streams, width], updated in place; x0 float32 [rows, width] (may be null): the
// row every stream starts as (X is then written, not read); y of the activation type
// [rows, width] (may be null: nothing is written back) with mix float32 [streams, streams]
// ([from][to]) and write float32 [streams]; read float32 [streams] and n_out of the activation
// type [rows, width] (both may be null: nothing is read) with gain float32 [1] or [width].
THN_API int thn_hyper_norm(void* n_out, float* X, const float* x0, const void* y, const float* mix, const float* write,
                           const float* read, const float* gain, int gain_is_vector, float eps, int rows, int width,
                           int streams, int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && width > 0 && X != nullptr, "hyper_norm: bad sizes rows=%d width=%d", rows, width);
    THN_UNSUPPORTED_IF(streams < 1 || streams > kMaxStreams, "hyper_norm: %d streams, at most %d", streams, kMaxStreams);
    THN_CHECK_ARG(y == nullptr || (mix != nullptr && write != nullptr), "hyper_norm: a write needs its mix and write numbers");
    THN_CHECK_ARG(y == nullptr || x0 == nullptr, "hyper_norm: the streams start before any sublayer writes");
    THN_CHECK_ARG((n_out == nullptr) == (read == nullptr), "hyper_norm: a read needs its numbers and its output");
    THN_CHECK_ARG(n_out == nullptr || (gain != nullptr && eps > 0.f), "hyper_norm: the norm needs a gain and eps > 0");
    THN_CHECK_ARG(n_out != nullptr || y != nullptr || x0 != nullptr, "hyper_norm: nothing to do");
    if (rows == 0) return THN_OK;
    if (dtype == THN_F32)
        return launch<float>(n_out, X, x0, y, mix, write, read, gain, gain_is_vector, eps, rows, width, streams, stream);
    if (dtype == THN_BF16)
        return launch<__nv_bfloat16>(n_out, X, x0, y, mix, write, read, gain, gain_is_vector, eps, rows, width, streams, stream);
    THN_CHECK_ARG(false, "hyper_norm: unknown dtype %d", dtype);
    return THN_OK;
}
