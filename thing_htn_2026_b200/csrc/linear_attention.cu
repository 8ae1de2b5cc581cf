// Linear attention with a decayed matrix state: per head a matrix S [key_dim, value_dim], zero at
// a sequence's start, and for every token
//
//     S <- diag(a_t) S + k_t v_t^T          o_t = S^T q_t * q_scale
//
// The decay a_t is one of
//   0  a constant per head (decay[head]); the same for every key channel and token;
//   1  a vector per token and head over the key channels, a = logistic(z)^(1 / tau) with
//      z = gate[row, head * key_dim + d] + gate_bias[head * key_dim + d] (float32), computed as
//      exp(-softplus(-z) / tau).
// q, k and v come from one projected row [q | k | v | ...] of the activation type; with
// silu_inputs they pass silu first.  Everything after the load is float32: the state, the decay
// with its softplus and exponential, the sums.
//
// A column of S (one entry of v and of o) evolves on its own.  It is held by 8 lanes of a warp,
// lane l keeping the key channels l, l + 8, ...; a token costs each lane its share of
// multiply-adds and the column three shuffles.  One block per (sequence, head, 16 columns) walks
// the sequence's tokens of the step in order, the next token's operands loaded while the
// current one is worked on.  A single-token step is the same kernel with one token.  A row's
// result depends on its sequence's own tokens only, in an order fixed by the sizes.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kLanes = 8;
constexpr int kColumns = 16;                  // columns of S per block
constexpr int kThreads = kLanes * kColumns;   // 128

// logistic(z)^(1 / tau) = exp(-softplus(-z) / tau), without overflow; in double on the 32-bit path
template <typename T> __device__ __forceinline__ float logistic_power(float z, float inv_tau) {
    const float log_logistic = z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
    return expf(log_logistic * inv_tau);
}
template <> __device__ __forceinline__ float logistic_power<float>(float z, float inv_tau) {
    const double x = (double)z;
    const double log_logistic = x >= 0.0 ? -log1p(exp(-x)) : x - log1p(exp(x));
    return (float)exp(log_logistic * (double)inv_tau);
}

template <typename T, int PER, int MODE, bool SILU>
__global__ void __launch_bounds__(kThreads) linear_attention_kernel(
    float* __restrict__ o, float* __restrict__ state, const T* __restrict__ proj, int proj_width, int q_offset,
    int k_offset, int v_offset, const float* __restrict__ decay, const float* __restrict__ gate, int gate_width,
    const float* __restrict__ gate_bias, float inv_tau, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
    int n_heads, int key_dim, int value_dim, float q_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.z, head = blockIdx.y;
    const int column = blockIdx.x * kColumns + threadIdx.x / kLanes;
    const int lane = threadIdx.x % kLanes;
    const bool live = column < value_dim;
    const int col = live ? column : value_dim - 1;     // idle columns mirror the last one and store nothing
    const int row0 = cu_seqlens[seq], row1 = cu_seqlens[seq + 1];
    const int slot = slots[seq];
    float* S = state + (((size_t)slot * n_heads + head) * value_dim + col) * key_dim;

    float s[PER], kc[PER], qc[PER], ac[MODE == 1 ? PER : 1], vc = 0.f;     // the current token's operands
    float kn[PER], qn[PER], an[MODE == 1 ? PER : 1], vn = 0.f;             // the next token's
    float bias[MODE == 1 ? PER : 1];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = lane + kLanes * i;
        s[i] = d < key_dim ? S[d] : 0.f;
        if (MODE == 1) bias[i] = d < key_dim && gate_bias ? gate_bias[head * key_dim + d] : 0.f;
    }
    const float constant = MODE == 0 ? decay[head] : 0.f;

#define THN_LA_LOAD(ROW, K_, Q_, A_, V_)                                                             \
    do {                                                                                             \
        const T* src = proj + (size_t)(ROW) * proj_width;                                            \
        _Pragma("unroll") for (int i = 0; i < PER; ++i) {                                            \
            const int d = lane + kLanes * i;                                                         \
            const bool in = d < key_dim;                                                             \
            K_[i] = in ? to_f32<T>(src[k_offset + head * key_dim + d]) : 0.f;                        \
            Q_[i] = in ? to_f32<T>(src[q_offset + head * key_dim + d]) : 0.f;                        \
            if (MODE == 1) A_[i] = in ? gate[(size_t)(ROW) * gate_width + head * key_dim + d] : 0.f; \
        }                                                                                            \
        V_ = to_f32<T>(src[v_offset + head * value_dim + col]);                                      \
    } while (0)

    if (row0 < row1) THN_LA_LOAD(row0, kc, qc, ac, vc);
    for (int row = row0; row < row1; ++row) {
        if (row + 1 < row1) THN_LA_LOAD(row + 1, kn, qn, an, vn);
        const float v = SILU ? silu_of<T>(vc) : vc;
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            float k = kc[i], q = qc[i];
            if (SILU) { k = silu_of<T>(k); q = silu_of<T>(q); }
            const float a = MODE == 0 ? constant : logistic_power<T>(ac[i] + bias[i], inv_tau);
            s[i] = a * s[i] + k * v;
            part += s[i] * q;
        }
#pragma unroll
        for (int off = kLanes / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
        if (lane == 0 && live) o[((size_t)row * n_heads + head) * value_dim + col] = part * q_scale;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            kc[i] = kn[i];
            qc[i] = qn[i];
            if (MODE == 1) ac[i] = an[i];
        }
        vc = vn;
    }
#undef THN_LA_LOAD
    if (live && row0 < row1) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + kLanes * i;
            if (d < key_dim) S[d] = s[i];
        }
    }
}

template <typename T, int PER>
void launch_per(float* o, float* state, const void* proj, int proj_width, int q_offset, int k_offset, int v_offset,
                const float* decay, const float* gate, int gate_width, const float* gate_bias, float inv_tau,
                const int* cu_seqlens, const int* slots, int n_seqs, int n_heads, int key_dim, int value_dim, float q_scale,
                int mode, int silu_inputs, cudaStream_t stream) {
    const dim3 grid((value_dim + kColumns - 1) / kColumns, n_heads, n_seqs);
#define THN_LA_LAUNCH(MODE, SILU)                                                                                       \
    thn_launch_ordered(linear_attention_kernel<T, PER, MODE, SILU>, grid, kThreads, 0, stream, o, state, (const T*)proj, \
                       proj_width, q_offset, k_offset, v_offset, decay, gate, gate_width, gate_bias, inv_tau, cu_seqlens, \
                       slots, n_heads, key_dim, value_dim, q_scale)
    if (mode == 0 && silu_inputs) THN_LA_LAUNCH(0, true);
    else if (mode == 0) THN_LA_LAUNCH(0, false);
    else if (silu_inputs) THN_LA_LAUNCH(1, true);
    else THN_LA_LAUNCH(1, false);
#undef THN_LA_LAUNCH
}

template <typename T>
int launch(float* o, float* state, const void* proj, int proj_width, int q_offset, int k_offset, int v_offset,
           const float* decay, const float* gate, int gate_width, const float* gate_bias, float inv_tau,
           const int* cu_seqlens, const int* slots, int n_seqs, int n_heads, int key_dim, int value_dim, float q_scale,
           int mode, int silu_inputs, cudaStream_t stream) {
    const int per = (key_dim + kLanes - 1) / kLanes;
#define THN_LA_PER(P)                                                                                                   \
    launch_per<T, P>(o, state, proj, proj_width, q_offset, k_offset, v_offset, decay, gate, gate_width, gate_bias, inv_tau, \
                     cu_seqlens, slots, n_seqs, n_heads, key_dim, value_dim, q_scale, mode, silu_inputs, stream)
    if (per <= 2) THN_LA_PER(2);
    else if (per <= 4) THN_LA_PER(4);
    else if (per <= 8) THN_LA_PER(8);
    else if (per <= 16) THN_LA_PER(16);
    else if (per <= 32) THN_LA_PER(32);
    else THN_LA_PER(64);
#undef THN_LA_PER
    return thn_launch_status("linear_attention");
}

}  // namespace

// o float32 [rows, heads, value_dim]; state float32 [slots, heads, value_dim, key_dim], read and
// updated; proj [rows, proj_width] of the activation type with q, k (heads * key_dim each) and v
// (heads * value_dim) from the given columns; mode 0: decay float32 [heads]; mode 1: gate float32
// [rows, gate_width] (the first heads * key_dim columns), gate_bias float32 [heads * key_dim] or
// null, tau > 0.  The tokens of sequence i are the rows [cu_seqlens[i], cu_seqlens[i + 1]).
THN_API int thn_linear_attention(float* o, float* state, const void* proj, int proj_width, int q_offset, int k_offset,
                                 int v_offset, const float* decay, const float* gate, int gate_width,
                                 const float* gate_bias, float tau, const int* cu_seqlens, const int* slots, int n_seqs,
                                 int n_heads, int key_dim, int value_dim, float q_scale, int mode, int silu_inputs,
                                 int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0 && n_heads > 0 && key_dim > 0 && value_dim > 0, "linear_attention: bad sizes");
    THN_UNSUPPORTED_IF(key_dim > 512, "linear_attention: keys of %d, at most 512", key_dim);
    THN_UNSUPPORTED_IF(n_heads > 65535 || n_seqs > 65535, "linear_attention: %d heads, %d sequences", n_heads, n_seqs);
    THN_CHECK_ARG(mode == 0 ? decay != nullptr : (mode == 1 && gate != nullptr && tau > 0.f && gate_width >= n_heads * key_dim),
                  "linear_attention: decay mode %d without its operands", mode);
    THN_CHECK_ARG(q_offset >= 0 && k_offset >= 0 && v_offset >= 0 && q_offset + n_heads * key_dim <= proj_width &&
                      k_offset + n_heads * key_dim <= proj_width && v_offset + n_heads * value_dim <= proj_width,
                  "linear_attention: q, k, v do not lie inside rows of %d", proj_width);
    if (n_seqs == 0) return THN_OK;
    const float inv_tau = mode == 1 ? 1.0f / tau : 0.f;
    if (dtype == THN_F32)
        return launch<float>(o, state, proj, proj_width, q_offset, k_offset, v_offset, decay, gate, gate_width, gate_bias,
                             inv_tau, cu_seqlens, slots, n_seqs, n_heads, key_dim, value_dim, q_scale, mode, silu_inputs, stream);
    if (dtype == THN_BF16)
        return launch<__nv_bfloat16>(o, state, proj, proj_width, q_offset, k_offset, v_offset, decay, gate, gate_width,
                                     gate_bias, inv_tau, cu_seqlens, slots, n_seqs, n_heads, key_dim, value_dim, q_scale,
                                     mode, silu_inputs, stream);
    THN_CHECK_ARG(false, "linear_attention: unknown dtype %d", dtype);
    return THN_OK;
}
