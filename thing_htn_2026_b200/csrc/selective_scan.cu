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
//   selective_scan     a channel's state is held by 4 lanes (8 for states above 32; entry n by lane
//                 n mod lanes); one block per (sequence, 64 or 32 channels) walks the sequence's tokens of the step in order;
//                 the tokens come through shared memory, sixteen at a time in two buffers.
//
// float32 after the loads: the step size with its softplus, the decay with its exponential, the
// state, the sums, the gate.  The convolution is summed in float32 and rounded once after silu.
// With float32 activations the exponentials and logarithms are computed in double and rounded once
// (exp_of, silu_of, softplus_of in common.cuh).
#include <math.h>

#include "common.cuh"

namespace {



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

// The decay exp(dt * A).  With bfloat16 activations A is held times log2(e) and the exponential is
// the hardware's base-2 one (two ulp; four full ones a token are a third of the scan's instructions
// otherwise); on the 32-bit path it is computed in double and rounded once.
template <typename T> struct Decay {
    static __device__ __forceinline__ float hold(float a) { return a * 1.4426950408889634f; }
    static __device__ __forceinline__ float of(float dt, float held) { return exp2f(dt * held); }
};
template <> struct Decay<float> {
    static __device__ __forceinline__ float hold(float a) { return a; }
    static __device__ __forceinline__ float of(float dt, float held) { return exp_of<float>(dt * held); }
};

// LANES lanes hold a channel's state, PER entries each; NP = LANES * PER: the padded state size of a
// staged token's B and C.  A block of 256 threads takes 256 / LANES channels: 64 with four lanes
// (states up to 32), so that a token's step sizes, inputs and gates are runs of 128 to 256 bytes.
// A staged token is [B | C | dt of the block's channels | x | silu(z)]; FETCH values per thread
// and stage.  Every thread fetches its part of the next stage into registers, the block works
// through the current one, then the fetched values are transformed once per block (the step size
// with its bias and softplus, the gate with its silu) and stored for all lanes to read.
constexpr int kStage = 16;
constexpr int kScanThreads = 256;

// A value as it was loaded, untouched: turning it into a float is a use, and a use makes the thread
// wait for the load.  The stage's loads are all issued first and turned into floats when they are stored.
template <typename T> __device__ __forceinline__ uint32_t raw_load(const T* p);
template <> __device__ __forceinline__ uint32_t raw_load<float>(const float* p) { return *reinterpret_cast<const uint32_t*>(p); }
template <> __device__ __forceinline__ uint32_t raw_load<__nv_bfloat16>(const __nv_bfloat16* p) {
    return *reinterpret_cast<const unsigned short*>(p);
}
template <typename T> __device__ __forceinline__ float from_raw(uint32_t bits);
template <> __device__ __forceinline__ float from_raw<float>(uint32_t bits) { return __uint_as_float(bits); }
template <> __device__ __forceinline__ float from_raw<__nv_bfloat16>(uint32_t bits) { return __uint_as_float(bits << 16); }

template <typename T, int LANES, int PER, int FETCH>
__global__ void __launch_bounds__(kScanThreads) selective_scan_kernel(
    T* __restrict__ y, float* __restrict__ state, const T* __restrict__ x, const float* __restrict__ dt_pre,
    const float* __restrict__ dt_bias, const T* __restrict__ bc, int bc_width, const float* __restrict__ A,
    const float* __restrict__ D, const T* __restrict__ z, int z_stride, const int* __restrict__ cu_seqlens,
    const int* __restrict__ slots, int channels, int n_state) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int kLanes = LANES, kChannels = kScanThreads / LANES, kThreads = kScanThreads;
    constexpr int NP = kLanes * PER, ROW = 2 * NP + 3 * kChannels;
    __shared__ float stage_mem[2 * kStage * ROW];
    __shared__ float bias_mem[kChannels];
    const int seq = blockIdx.y;
    const int c0 = blockIdx.x * kChannels;
    const int group = threadIdx.x / kLanes, lane = threadIdx.x % kLanes;
    const int channel = c0 + group;
    const bool live = channel < channels;
    const int c = live ? channel : channels - 1;
    const int row0 = cu_seqlens[seq], row1 = cu_seqlens[seq + 1];
    const int slot = slots[seq];
    float* S = state + ((size_t)slot * channels + c) * n_state;

    float s[PER], a[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int n = lane + kLanes * i;
        s[i] = n < n_state ? S[n] : 0.f;
        a[i] = n < n_state ? Decay<T>::hold(A[(size_t)c * n_state + n]) : 0.f;
    }
    const float skip = D[c];
    if (threadIdx.x < kChannels) bias_mem[threadIdx.x] = dt_bias[min(c0 + (int)threadIdx.x, channels - 1)];

    uint32_t fetched[FETCH];
    auto fetch = [&](int first_row) {
#pragma unroll
        for (int j = 0; j < FETCH; ++j) {
            const int e = threadIdx.x + j * kThreads;
            const int t = e / ROW, k = e - t * ROW;
            const int row = first_row + t;
            uint32_t v = 0;
            if (row < row1) {
                if (k < 2 * NP) {
                    const int which = k / NP, n = k - which * NP;
                    if (n < n_state) v = raw_load<T>(bc + (size_t)row * bc_width + which * n_state + n);
                } else {
                    const int which = (k - 2 * NP) / kChannels, ch = min(c0 + (k - 2 * NP) % kChannels, channels - 1);
                    if (which == 0) v = raw_load<float>(dt_pre + (size_t)row * channels + ch);
                    else if (which == 1) v = raw_load<T>(x + (size_t)row * channels + ch);
                    else v = raw_load<T>(z + (size_t)row * z_stride + ch);
                }
            }
            fetched[j] = v;
        }
    };
    auto publish = [&](int buf, int n) {
        float* dst = stage_mem + buf * kStage * ROW;
#pragma unroll
        for (int j = 0; j < FETCH; ++j) {
            const int e = threadIdx.x + j * kThreads;
            if (e >= n * ROW) continue;          // what lies beyond the step's tokens is neither transformed nor read
            const int k = e % ROW;
            float v;
            if (k >= 2 * NP + 2 * kChannels) v = silu_of<T>(from_raw<T>(fetched[j]));
            else if (k >= 2 * NP + kChannels) v = from_raw<T>(fetched[j]);
            else if (k >= 2 * NP) v = softplus_of<T>(__uint_as_float(fetched[j]) + bias_mem[k - 2 * NP]);
            else v = from_raw<T>(fetched[j]);
            dst[e] = v;
        }
    };

    if (row1 - row0 == 1) {
        // a single token: straight from global memory, no stage and no barrier
        const float dt = softplus_of<T>(dt_pre[(size_t)row0 * channels + c] + dt_bias[c]);     // (bias_mem is not read here)
        const float xv = to_f32<T>(x[(size_t)row0 * channels + c]);
        const float dx = dt * xv;
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int n = lane + kLanes * i;
            const bool in = n < n_state;
            const float b = in ? to_f32<T>(bc[(size_t)row0 * bc_width + n]) : 0.f;
            const float cc = in ? to_f32<T>(bc[(size_t)row0 * bc_width + n_state + n]) : 0.f;
            s[i] = Decay<T>::of(dt, a[i]) * s[i] + dx * b;
            part += s[i] * cc;
            if (in && live) S[n] = s[i];
        }
#pragma unroll
        for (int off = kLanes / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
        if (lane == 0 && live)
            y[(size_t)row0 * channels + c] = from_f32<T>((part + skip * xv) * silu_of<T>(to_f32<T>(z[(size_t)row0 * z_stride + c])));
        return;
    }
    if (row0 < row1) fetch(row0);
    __syncthreads();                                   // the channels' biases are in place
    if (row0 < row1) publish(0, min(kStage, row1 - row0));
    __syncthreads();
    for (int first = row0, buf = 0; first < row1; first += kStage, buf ^= 1) {
        const bool more = first + kStage < row1;
        if (more) fetch(first + kStage);
        // the loads stay here, ahead of the stage's work: sunk to where their values are stored, each
        // would wait for memory in its turn
        asm volatile("" ::: "memory");
        const float* src = stage_mem + buf * kStage * ROW;
        const int n_tokens = min(kStage, row1 - first);
        // (unrolled: only the state's multiply-add links one token to the next; the loads, the
        // exponentials and the shuffles of several tokens then overlap)
#pragma unroll 4
        for (int t = 0; t < n_tokens; ++t) {
            const float* tok = src + t * ROW;
            const float dt = tok[2 * NP + group], xv = tok[2 * NP + kChannels + group];
            const float dx = dt * xv;
            float part = 0.f;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int n = lane + kLanes * i;
                s[i] = Decay<T>::of(dt, a[i]) * s[i] + dx * tok[n];
                part += s[i] * tok[NP + n];
            }
#pragma unroll
            for (int off = kLanes / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
            if (lane == 0 && live)
                y[(size_t)(first + t) * channels + c] = from_f32<T>((part + skip * xv) * tok[2 * NP + 2 * kChannels + group]);
        }
        if (more) publish(buf ^ 1, min(kStage, row1 - first - kStage));
        __syncthreads();
    }
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
#define THN_SCAN_LAUNCH(L, P)                                                                                           \
    thn_launch_ordered(selective_scan_kernel<T, L, P, (kStage * (2 * L * P + 3 * (kScanThreads / L)) + kScanThreads - 1) / kScanThreads>, \
                       dim3((channels + kScanThreads / L - 1) / (kScanThreads / L), n_seqs), kScanThreads, 0, stream, (T*)y, state, \
                       (const T*)x, dt_pre, dt_bias, (const T*)bc, bc_width, A, D, (const T*)z, z_stride, cu_seqlens, slots, \
                       channels, n_state)
    if (n_state <= 4) THN_SCAN_LAUNCH(4, 1);
    else if (n_state <= 8) THN_SCAN_LAUNCH(4, 2);
    else if (n_state <= 16) THN_SCAN_LAUNCH(4, 4);
    else if (n_state <= 32) THN_SCAN_LAUNCH(4, 8);
    else if (n_state <= 64) THN_SCAN_LAUNCH(8, 8);
    else THN_SCAN_LAUNCH(8, 16);
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
    THN_UNSUPPORTED_IF(n_state > 128, "selective_scan: a state of %d per channel, at most 128", n_state);
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
