// The selective scan (Mamba): per channel c a state vector S[c, 0..N-1], zero at a sequence's
// start, and for every token
//
//     dt_c = softplus(dt_pre[c] + dt_bias[c])
//     S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n
//     y_c = (sum_n S[c, n] C_n + D_c x_c) * silu(z_c)
//
// with A < 0 a constant matrix, x the convolved input, B and C vectors of the token shared by
// all channels, z the token's gate.  Ahead of it a short causal convolution per channel with
// silu:  x_c[t] = silu(bias_c + sum_j w[c, j] raw_c[t - (taps - 1) + j]),  zeros before the
// sequence's start.
//
//   causal_conv   one thread per (row, channel).  A token's predecessors come from the step's own
//                 rows or, before the step's first row, from the ring: the last `taps` raw inputs
//                 of the sequence, position p at p mod taps.
//   conv_ring_update   after every reader of the ring has ended: the step's last raw inputs go in.
//   selective_scan     a channel's state is held by 8 lanes (entry n by lane n mod 8); one block
//                 per (sequence, 16 channels) walks the sequence's tokens of the step in order,
//                 the next token's operands loaded while the current one is worked on.
//
// float32 after the loads: the step size with its softplus, the decay with its exponential, the
// state, the sums, the gate.  The convolution is summed in float32 and rounded once after silu.
// With float32 activations the exponentials and logarithms are computed in double and rounded once
// (exp_of, silu_of, softplus_of in common.cuh).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kLanes = 8;
constexpr int kChannels = 16;
constexpr int kThreads = kLanes * kChannels;


template <typename T>
__global__ void causal_conv_kernel(T* __restrict__ out, const T* __restrict__ proj, int proj_width, int offset,
                                   const float* __restrict__ weight, const float* __restrict__ bias,
                                   const T* __restrict__ ring, const int* __restrict__ row_slot,
                                   const int* __restrict__ row_pos, const int* __restrict__ seq_lens, long long n,
                                   int channels, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const long long row = e / channels;
    const int c = (int)(e - row * channels);
    const int slot = row_slot[row], pos = row_pos[row];
    const int local = pos - seq_lens[slot];          // index of the row among its sequence's rows of this step
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;               // how many tokens before this one
        if (back > pos) continue;                    // before the sequence's start: zero
        float v;
        if (back <= local) v = to_f32<T>(proj[(size_t)(row - back) * proj_width + offset + c]);
        else v = to_f32<T>(ring[((size_t)slot * taps + (pos - back) % taps) * channels + c]);
        acc += weight[(size_t)c * taps + j] * v;
    }
    out[e] = from_f32<T>(silu_of<T>(acc));
}

template <typename T>
__global__ void conv_ring_update_kernel(T* __restrict__ ring, const T* __restrict__ proj, int proj_width, int offset,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                        const int* __restrict__ seq_lens, int channels, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.y;
    const int row0 = cu_seqlens[seq], row1 = cu_seqlens[seq + 1], slot = slots[seq];
    const int held = seq_lens[slot];
    const int first = max(row0, row1 - taps);
    const int total = (row1 - first) * channels;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int r = first + e / channels, c = e % channels;
        const int pos = held + (r - row0);
        ring[((size_t)slot * taps + pos % taps) * channels + c] = proj[(size_t)r * proj_width + offset + c];
    }
}

template <typename T, int PER>
__global__ void __launch_bounds__(kThreads) selective_scan_kernel(
    T* __restrict__ y, float* __restrict__ state, const T* __restrict__ x, const float* __restrict__ dt_pre,
    const float* __restrict__ dt_bias, const T* __restrict__ bc, int bc_width, const float* __restrict__ A,
    const float* __restrict__ D, const T* __restrict__ z, int z_stride, const int* __restrict__ cu_seqlens,
    const int* __restrict__ slots, int channels, int n_state) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.y;
    const int channel = blockIdx.x * kChannels + threadIdx.x / kLanes;
    const int lane = threadIdx.x % kLanes;
    const bool live = channel < channels;
    const int c = live ? channel : channels - 1;
    const int row0 = cu_seqlens[seq], row1 = cu_seqlens[seq + 1];
    const int slot = slots[seq];
    float* S = state + ((size_t)slot * channels + c) * n_state;

    float s[PER], a[PER], bc_[PER], cc[PER], bn[PER], cn[PER];     // B and C of the current and of the next token
    float dtc = 0.f, xc = 0.f, zc = 0.f, dtn = 0.f, xn = 0.f, zn = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int n = lane + kLanes * i;
        s[i] = n < n_state ? S[n] : 0.f;
        a[i] = n < n_state ? A[(size_t)c * n_state + n] : 0.f;
    }
    const float bias = dt_bias[c], skip = D[c];

#define THN_SCAN_LOAD(ROW, B_, C_, DT_, X_, Z_)                                                        \
    do {                                                                                               \
        _Pragma("unroll") for (int i = 0; i < PER; ++i) {                                              \
            const int n = lane + kLanes * i;                                                           \
            B_[i] = n < n_state ? to_f32<T>(bc[(size_t)(ROW) * bc_width + n]) : 0.f;                   \
            C_[i] = n < n_state ? to_f32<T>(bc[(size_t)(ROW) * bc_width + n_state + n]) : 0.f;         \
        }                                                                                              \
        DT_ = dt_pre[(size_t)(ROW) * channels + c];                                                    \
        X_ = to_f32<T>(x[(size_t)(ROW) * channels + c]);                                               \
        Z_ = to_f32<T>(z[(size_t)(ROW) * z_stride + c]);                                               \
    } while (0)

    if (row0 < row1) THN_SCAN_LOAD(row0, bc_, cc, dtc, xc, zc);
    for (int row = row0; row < row1; ++row) {
        if (row + 1 < row1) THN_SCAN_LOAD(row + 1, bn, cn, dtn, xn, zn);
        const float dt = softplus_of<T>(dtc + bias);
        const float xv = xc;
        const float dx = dt * xv;
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            s[i] = exp_of<T>(dt * a[i]) * s[i] + dx * bc_[i];
            part += s[i] * cc[i];
        }
#pragma unroll
        for (int off = kLanes / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
        if (lane == 0 && live)
            y[(size_t)row * channels + c] = from_f32<T>((part + skip * xv) * silu_of<T>(zc));
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            bc_[i] = bn[i];
            cc[i] = cn[i];
        }
        dtc = dtn; xc = xn; zc = zn;
    }
#undef THN_SCAN_LOAD
    if (live && row0 < row1) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int n = lane + kLanes * i;
            if (n < n_state) S[n] = s[i];
        }
    }
}

template <typename T>
int launch_scan(void* y, float* state, const void* x, const float* dt_pre, const float* dt_bias, const void* bc,
                int bc_width, const float* A, const float* D, const void* z, int z_stride, const int* cu_seqlens,
                const int* slots, int n_seqs, int channels, int n_state, cudaStream_t stream) {
    const dim3 grid((channels + kChannels - 1) / kChannels, n_seqs);
    const int per = (n_state + kLanes - 1) / kLanes;
#define THN_SCAN_LAUNCH(P)                                                                                              \
    thn_launch_ordered(selective_scan_kernel<T, P>, grid, kThreads, 0, stream, (T*)y, state, (const T*)x, dt_pre, dt_bias, \
                       (const T*)bc, bc_width, A, D, (const T*)z, z_stride, cu_seqlens, slots, channels, n_state)
    if (per <= 1) THN_SCAN_LAUNCH(1);
    else if (per <= 2) THN_SCAN_LAUNCH(2);
    else if (per <= 4) THN_SCAN_LAUNCH(4);
    else if (per <= 8) THN_SCAN_LAUNCH(8);
    else if (per <= 16) THN_SCAN_LAUNCH(16);
    else THN_SCAN_LAUNCH(32);
#undef THN_SCAN_LAUNCH
    return thn_launch_status("selective_scan");
}

}  // namespace

// out [rows, channels] of the activation type; the raw inputs are the columns [offset, offset +
// channels) of proj [rows, proj_width]; weight float32 [channels, taps] (the last tap is the
// current token's), bias float32 [channels] or null; ring [slots, taps, channels] of the
// activation type; seq_lens int32 [slots]: the tokens each slot held before the step.
THN_API int thn_causal_conv(void* out, const void* proj, int proj_width, int offset, const float* weight,
                            const float* bias, const void* ring, const int* row_slot, const int* row_pos,
                            const int* seq_lens, int n_rows, int channels, int taps, int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && channels > 0 && taps > 0 && offset >= 0 && offset + channels <= proj_width,
                  "causal_conv: bad sizes");
    const long long n = (long long)n_rows * channels;
    if (n == 0) return THN_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == THN_F32)
        thn_launch(causal_conv_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)proj, proj_width, offset,
                   weight, bias, (const float*)ring, row_slot, row_pos, seq_lens, n, channels, taps);
    else if (dtype == THN_BF16)
        thn_launch(causal_conv_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)proj, proj_width, offset, weight, bias, (const __nv_bfloat16*)ring, row_slot,
                   row_pos, seq_lens, n, channels, taps);
    else
        THN_CHECK_ARG(false, "causal_conv: unknown dtype %d", dtype);
    return thn_launch_status("causal_conv");
}

// The step's last raw inputs (at most taps per sequence) go into the ring, position p at p mod taps.
THN_API int thn_conv_ring_update(void* ring, const void* proj, int proj_width, int offset, const int* cu_seqlens,
                                 const int* slots, const int* seq_lens, int n_seqs, int channels, int taps, int dtype,
                                 cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0 && channels > 0 && taps > 0 && offset >= 0 && offset + channels <= proj_width,
                  "conv_ring_update: bad sizes");
    THN_UNSUPPORTED_IF(n_seqs > 65535, "conv_ring_update: %d sequences", n_seqs);
    if (n_seqs == 0) return THN_OK;
    const dim3 grid((unsigned)min((long long)(((long long)taps * channels + 255) / 256), 64ll), n_seqs);
    if (dtype == THN_F32)
        thn_launch(conv_ring_update_kernel<float>, grid, 256, 0, stream, (float*)ring, (const float*)proj, proj_width,
                   offset, cu_seqlens, slots, seq_lens, channels, taps);
    else if (dtype == THN_BF16)
        thn_launch(conv_ring_update_kernel<__nv_bfloat16>, grid, 256, 0, stream, (__nv_bfloat16*)ring,
                   (const __nv_bfloat16*)proj, proj_width, offset, cu_seqlens, slots, seq_lens, channels, taps);
    else
        THN_CHECK_ARG(false, "conv_ring_update: unknown dtype %d", dtype);
    return thn_launch_status("conv_ring_update");
}

// y, x [rows, channels] of the activation type; state float32 [slots, channels, n_state], read and
// updated; dt_pre float32 [rows, channels], dt_bias float32 [channels]; bc [rows, bc_width] of the
// activation type: B in the first n_state columns, C in the next; A float32 [channels, n_state]
// (negative); D float32 [channels]; z of the activation type, rows z_stride apart.
THN_API int thn_selective_scan(void* y, float* state, const void* x, const float* dt_pre, const float* dt_bias,
                               const void* bc, int bc_width, const float* A, const float* D, const void* z, int z_stride,
                               const int* cu_seqlens, const int* slots, int n_seqs, int channels, int n_state, int dtype,
                               cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0 && channels > 0 && n_state > 0 && bc_width >= 2 * n_state && z_stride >= channels,
                  "selective_scan: bad sizes");
    THN_UNSUPPORTED_IF(n_state > 256, "selective_scan: a state of %d per channel, at most 256", n_state);
    THN_UNSUPPORTED_IF(n_seqs > 65535, "selective_scan: %d sequences", n_seqs);
    if (n_seqs == 0) return THN_OK;
    if (dtype == THN_F32)
        return launch_scan<float>(y, state, x, dt_pre, dt_bias, bc, bc_width, A, D, z, z_stride, cu_seqlens, slots, n_seqs,
                                  channels, n_state, stream);
    if (dtype == THN_BF16)
        return launch_scan<__nv_bfloat16>(y, state, x, dt_pre, dt_bias, bc, bc_width, A, D, z, z_stride, cu_seqlens, slots,
                                          n_seqs, channels, n_state, stream);
    THN_CHECK_ARG(false, "selective_scan: unknown dtype %d", dtype);
    return THN_OK;
}
