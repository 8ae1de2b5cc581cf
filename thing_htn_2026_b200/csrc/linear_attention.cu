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
// Two kernels.  linear_attention_prepare does what is the same for every column, once per entry:
// silu of q, k and v where asked, the decay with its softplus and exponential, all to float32 rows
// [row][head][k | q | (decay) | v], the key parts filled up with zeros to a multiple of 32 and the
// values to a multiple of 16.  linear_attention_kernel is the recurrence.  A column of S (one entry
// of v and of o) evolves on its own.  It is held by 8 lanes of a warp, lane l keeping the key
// channels 4l .. 4l + 3, 32 + 4l .. (runs of four, for 16-byte accesses); a token costs each lane
// its share of multiply-adds and the column three shuffles.  One block per (sequence, head, 16
// columns) walks the sequence's tokens of the step in order.  The tokens come through shared
// memory, sixteen at a time (fewer for keys above 128) in two buffers: every thread fetches its
// 16-byte pieces of the next stage into registers, the block works through the current stage, and
// then the pieces are stored.  A single-token step is the same two kernels with one token.  A row's
// result depends on its sequence's own tokens only, in an order fixed by the sizes.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kLanes = 8;
constexpr int kColumns = 16;                  // columns of S per block
constexpr int kThreads = kLanes * kColumns;   // 128
// tokens per stage: fewer for long keys, so that a thread's share of a stage stays in registers
constexpr int stage_tokens(int per) { return per <= 16 ? 16 : per <= 32 ? 8 : 4; }

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

// prepared [rows][heads][parts * kp + vp] float32: k, q (and the decay) over kp entries each, then
// v over vp entries; entries beyond key_dim and value_dim are zero.
template <typename T>
__global__ void linear_attention_prepare_kernel(float* __restrict__ prepared, const T* __restrict__ proj, int proj_width,
                                                int q_offset, int k_offset, int v_offset, const float* __restrict__ gate,
                                                int gate_width, const float* __restrict__ gate_bias, float inv_tau,
                                                long long n, int n_heads, int key_dim, int value_dim, int kp, int vp,
                                                int parts, int silu_inputs) {
    pdl_launch_dependents();
    pdl_wait();
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const int per_head = parts * kp + vp;
    const long long unit = e / per_head;
    const int c = (int)(e - unit * per_head);
    const long long row = unit / n_heads;
    const int head = (int)(unit - row * n_heads);
    const T* src = proj + row * proj_width;
    float v = 0.f;
    if (c >= parts * kp) {
        const int d = c - parts * kp;
        if (d < value_dim) {
            v = to_f32<T>(src[v_offset + head * value_dim + d]);
            if (silu_inputs) v = silu_of<T>(v);
        }
    } else {
        const int part = c / kp, d = c - part * kp;
        if (d < key_dim) {
            if (part == 2) {
                v = logistic_power<T>(gate[row * gate_width + head * key_dim + d] + (gate_bias ? gate_bias[head * key_dim + d] : 0.f),
                                      inv_tau);
            } else {
                v = to_f32<T>(src[(part == 0 ? k_offset : q_offset) + head * key_dim + d]);
                if (silu_inputs) v = silu_of<T>(v);
            }
        }
    }
    prepared[e] = v;
}

// PER: key channels per lane (a multiple of 4); KP = 8 * PER: the padded key size.
// FETCH: 16-byte pieces per thread and stage, ceil(stage tokens * (parts * KP + 16) / 4 / 128).
template <int PER, int MODE, int FETCH>
__global__ void __launch_bounds__(kThreads) linear_attention_kernel(
    float* __restrict__ o, float* __restrict__ state, const float* __restrict__ prepared, int vp,
    const float* __restrict__ decay, const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int n_heads,
    int key_dim, int value_dim, float q_scale) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int KP = kLanes * PER, kStage = stage_tokens(PER);
    constexpr int PARTS = MODE == 1 ? 3 : 2;            // k, q (and the decay) per token
    constexpr int ROW = PARTS * KP + kColumns;          // floats of one staged token
    constexpr int PIECES = ROW / 4;
    extern __shared__ __align__(16) float stage_mem[];  // [2][kStage][ROW]
    const int seq = blockIdx.z, head = blockIdx.y;
    const int col0 = blockIdx.x * kColumns;
    const int column = col0 + threadIdx.x / kLanes;
    const int lane = threadIdx.x % kLanes;
    const bool live = column < value_dim;
    const int col = live ? column : value_dim - 1;     // idle columns mirror the last one and store nothing
    const int row0 = cu_seqlens[seq], row1 = cu_seqlens[seq + 1];
    const int slot = slots[seq];
    float* S = state + (((size_t)slot * n_heads + head) * value_dim + col) * key_dim;
    const size_t per_head = (size_t)PARTS * KP + vp;

    float s[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = (i / 4) * 32 + lane * 4 + (i & 3);
        s[i] = d < key_dim ? S[d] : 0.f;
    }
    const float constant = MODE == 0 ? decay[head] : 1.f;

    float4 fetched[FETCH];
    auto fetch = [&](int first_row) {
        const int n = min(kStage, row1 - first_row);
#pragma unroll
        for (int j = 0; j < FETCH; ++j) {
            const int piece = threadIdx.x + j * kThreads;
            const int t = piece / PIECES, c = (piece - t * PIECES) * 4;
            if (t < n) {
                const float* src = prepared + ((size_t)(first_row + t) * n_heads + head) * per_head;
                fetched[j] = *reinterpret_cast<const float4*>(c < PARTS * KP ? src + c : src + c + col0);
            }
        }
    };
    auto publish = [&](int buf, int n) {
        float* dst = stage_mem + (size_t)buf * kStage * ROW;
#pragma unroll
        for (int j = 0; j < FETCH; ++j) {
            const int piece = threadIdx.x + j * kThreads;
            if (piece / PIECES < n) *reinterpret_cast<float4*>(dst + piece * 4) = fetched[j];
        }
    };

    if (row0 < row1) {
        fetch(row0);
        publish(0, min(kStage, row1 - row0));
    }
    __syncthreads();
    const int v_at = PARTS * KP + threadIdx.x / kLanes;
    for (int first = row0, buf = 0; first < row1; first += kStage, buf ^= 1) {
        const bool more = first + kStage < row1;
        if (more) fetch(first + kStage);
        // the loads stay here, ahead of the stage's work: sunk to where their values are stored, each
        // would wait for memory in its turn
        asm volatile("" ::: "memory");
        const float* src = stage_mem + (size_t)buf * kStage * ROW;
        const int n = min(kStage, row1 - first);
        // (unrolled: only the state's multiply-adds link one token to the next; the loads and the
        // shuffles of two tokens then overlap)
#pragma unroll 2
        for (int t = 0; t < n; ++t) {
            const float* tok = src + t * ROW;
            const float v = tok[v_at];
            float part = 0.f;
#pragma unroll
            for (int i = 0; i < PER; i += 4) {
                const int d = (i / 4) * 32 + lane * 4;
                const float4 k = *reinterpret_cast<const float4*>(tok + d);
                const float4 q = *reinterpret_cast<const float4*>(tok + KP + d);
                float4 a = make_float4(constant, constant, constant, constant);
                if (MODE == 1) a = *reinterpret_cast<const float4*>(tok + 2 * KP + d);
                s[i] = a.x * s[i] + k.x * v;
                s[i + 1] = a.y * s[i + 1] + k.y * v;
                s[i + 2] = a.z * s[i + 2] + k.z * v;
                s[i + 3] = a.w * s[i + 3] + k.w * v;
                part += s[i] * q.x + s[i + 1] * q.y + s[i + 2] * q.z + s[i + 3] * q.w;
            }
#pragma unroll
            for (int off = kLanes / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
            if (lane == 0 && live) o[((size_t)(first + t) * n_heads + head) * value_dim + col] = part * q_scale;
        }
        if (more) publish(buf ^ 1, min(kStage, row1 - first - kStage));
        __syncthreads();
    }
    if (live && row0 < row1) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = (i / 4) * 32 + lane * 4 + (i & 3);
            if (d < key_dim) S[d] = s[i];
        }
    }
}

template <int PER, int MODE>
void launch_one(float* o, float* state, const float* prepared, int vp, const float* decay, const int* cu_seqlens,
                const int* slots, int n_seqs, int n_heads, int key_dim, int value_dim, float q_scale, cudaStream_t stream) {
    constexpr int KP = kLanes * PER, ROW = (MODE == 1 ? 3 : 2) * KP + kColumns, kStage = stage_tokens(PER);
    constexpr int FETCH = (kStage * ROW / 4 + kThreads - 1) / kThreads;
    const size_t smem = 2 * (size_t)kStage * ROW * sizeof(float);
    const dim3 grid((value_dim + kColumns - 1) / kColumns, n_heads, n_seqs);
    auto kernel = linear_attention_kernel<PER, MODE, FETCH>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    thn_launch_ordered(kernel, grid, kThreads, smem, stream, o, state, prepared, vp, decay, cu_seqlens, slots, n_heads, key_dim,
                       value_dim, q_scale);
}

template <typename T>
int launch(float* o, float* state, float* prepared, const void* proj, int proj_width, int q_offset, int k_offset, int v_offset,
           const float* decay, const float* gate, int gate_width, const float* gate_bias, float inv_tau,
           const int* cu_seqlens, const int* slots, int n_rows, int n_seqs, int n_heads, int key_dim, int value_dim,
           float q_scale, int mode, int silu_inputs, cudaStream_t stream) {
    const int per = (key_dim + 31) / 32 * 4;          // runs of four channels per lane
    const int per_t = per <= 4 ? 4 : per <= 8 ? 8 : per <= 16 ? 16 : per <= 32 ? 32 : 64;
    const int kp = kLanes * per_t, vp = (value_dim + kColumns - 1) / kColumns * kColumns, parts = mode == 1 ? 3 : 2;
    const long long n = (long long)n_rows * n_heads * (parts * kp + vp);
    thn_launch(linear_attention_prepare_kernel<T>, (unsigned)((n + 255) / 256), 256, 0, stream, prepared, (const T*)proj,
               proj_width, q_offset, k_offset, v_offset, gate, gate_width, gate_bias, inv_tau, n, n_heads, key_dim, value_dim, kp,
               vp, parts, silu_inputs);
#define THN_LA_PER(P)                                                                                                       \
    do {                                                                                                                    \
        if (mode == 0) launch_one<P, 0>(o, state, prepared, vp, decay, cu_seqlens, slots, n_seqs, n_heads, key_dim, value_dim, \
                                        q_scale, stream);                                                                   \
        else launch_one<P, 1>(o, state, prepared, vp, decay, cu_seqlens, slots, n_seqs, n_heads, key_dim, value_dim, q_scale, \
                              stream);                                                                                      \
    } while (0)
    if (per_t == 4) THN_LA_PER(4);
    else if (per_t == 8) THN_LA_PER(8);
    else if (per_t == 16) THN_LA_PER(16);
    else if (per_t == 32) THN_LA_PER(32);
    else THN_LA_PER(64);
#undef THN_LA_PER
    return thn_launch_status("linear_attention");
}

}  // namespace

// Floats of the scratch that thn_linear_attention needs for a step of n_rows rows.
THN_API long long thn_linear_attention_scratch_floats(int n_rows, int n_heads, int key_dim, int value_dim, int mode) {
    const int per = (key_dim + 31) / 32 * 4;
    const int per_t = per <= 4 ? 4 : per <= 8 ? 8 : per <= 16 ? 16 : per <= 32 ? 32 : 64;
    const long long kp = kLanes * per_t, vp = (value_dim + kColumns - 1) / kColumns * kColumns;
    return (long long)n_rows * n_heads * ((mode == 1 ? 3 : 2) * kp + vp);
}

// o float32 [rows, heads, value_dim]; state float32 [slots, heads, value_dim, key_dim], read and
// updated; proj [rows, proj_width] of the activation type with q, k (heads * key_dim each) and v
// (heads * value_dim) from the given columns; mode 0: decay float32 [heads]; mode 1: gate float32
// [rows, gate_width] (the first heads * key_dim columns), gate_bias float32 [heads * key_dim] or
// null, tau > 0.  The tokens of sequence i are the rows [cu_seqlens[i], cu_seqlens[i + 1]) of the
// step's n_rows rows.  scratch: float32, thn_linear_attention_scratch_floats(...) entries, 16-byte aligned.
THN_API int thn_linear_attention(float* o, float* state, float* scratch, const void* proj, int proj_width, int q_offset, int k_offset,
                                 int v_offset, const float* decay, const float* gate, int gate_width,
                                 const float* gate_bias, float tau, const int* cu_seqlens, const int* slots, int n_rows,
                                 int n_seqs, int n_heads, int key_dim, int value_dim, float q_scale, int mode, int silu_inputs,
                                 int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0 && n_heads > 0 && key_dim > 0 && value_dim > 0, "linear_attention: bad sizes");
    THN_UNSUPPORTED_IF(key_dim > 512, "linear_attention: keys of %d, at most 512", key_dim);
    THN_UNSUPPORTED_IF(n_heads > 65535 || n_seqs > 65535, "linear_attention: %d heads, %d sequences", n_heads, n_seqs);
    THN_CHECK_ARG(mode == 0 ? decay != nullptr : (mode == 1 && gate != nullptr && tau > 0.f && gate_width >= n_heads * key_dim),
                  "linear_attention: decay mode %d without its operands", mode);
    THN_CHECK_ARG(q_offset >= 0 && k_offset >= 0 && v_offset >= 0 && q_offset + n_heads * key_dim <= proj_width &&
                      k_offset + n_heads * key_dim <= proj_width && v_offset + n_heads * value_dim <= proj_width,
                  "linear_attention: q, k, v do not lie inside rows of %d", proj_width);
    THN_CHECK_ARG(scratch != nullptr && ((uintptr_t)scratch & 15) == 0 && n_rows >= 0, "linear_attention: scratch missing or unaligned");
    if (n_seqs == 0 || n_rows == 0) return THN_OK;
    const float inv_tau = mode == 1 ? 1.0f / tau : 0.f;
    if (dtype == THN_F32)
        return launch<float>(o, state, scratch, proj, proj_width, q_offset, k_offset, v_offset, decay, gate, gate_width, gate_bias,
                             inv_tau, cu_seqlens, slots, n_rows, n_seqs, n_heads, key_dim, value_dim, q_scale, mode, silu_inputs,
                             stream);
    if (dtype == THN_BF16)
        return launch<__nv_bfloat16>(o, state, scratch, proj, proj_width, q_offset, k_offset, v_offset, decay, gate, gate_width,
                                     gate_bias, inv_tau, cu_seqlens, slots, n_rows, n_seqs, n_heads, key_dim, value_dim, q_scale,
                                     mode, silu_inputs, stream);
    THN_CHECK_ARG(false, "linear_attention: unknown dtype %d", dtype);
    return THN_OK;
}
