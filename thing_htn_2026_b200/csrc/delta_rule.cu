// The gated delta rule: a recurrent token mixer whose state per head is a matrix S [dk, dv].
// For every token, with a unit key k, a scaled unit query q, a value v, a write strength b in
// (0, 1) and a decay g in (0, 1):
//
//     S <- g S;   u = b (v - S^T k);   S <- S + k u^T;   o = S^T q
//
// so the read-out sees the token's own write.  Every column of S (one entry of v, u and o)
// evolves on its own, which is what the kernels use: a column is held by 8 (or 32) lanes of a
// warp, a few values of the key axis each, in registers, for all the tokens a step brings.
//
// Steps of several tokens per sequence run three kernels: `prepare` (the short causal
// convolutions of q, k and v over time with their silu, the unit norms, b and g: one block per
// row), `recurrence` (one block per sequence, head and group of columns) and `ring update`
// (the convolution's window of raw inputs moves on, once nothing reads it any more).  Steps of
// one token per sequence run `decode`, which does all of it in one launch.  The state, the
// unit norms, b, g and all sums are float32; the projections come in the activation type.
//
// Per-sequence state.  S: float32 [slots, heads, dv, dk] (a column's dk values contiguous).
// The convolution's inputs: a ring [slots, taps, channels] of the activation type in which
// the raw projection of position p lies at p mod taps (channels: q, then k, then v).  A token
// reads its taps - 1 predecessors, from the step's own rows where they are part of the step
// and from the ring otherwise; positions before the sequence's start read as zero.
#include <math.h>

#include "common.cuh"

namespace {

// ------------------------------------------------------------------ prepare

struct DeltaShape {
    int n_heads, n_kv, dk, dv, taps;
    int proj_width;        // columns of a projected row: q | k | v | gate | b | a
    __host__ __device__ int qk_channels() const { return n_kv * dk; }
    __host__ __device__ int conv_channels() const { return 2 * n_kv * dk + n_heads * dv; }
    __host__ __device__ int gate_offset() const { return conv_channels(); }
    __host__ __device__ int b_offset() const { return conv_channels() + n_heads * dv; }
    __host__ __device__ int a_offset() const { return b_offset() + n_heads; }
};

// The convolution of channel c at the row of position pos, `back` = pos - (position of the
// sequence's first row in this step).
template <typename T>
__device__ __forceinline__ float conv_at(const T* __restrict__ proj_row, const T* __restrict__ ring_slot,
                                         const float* __restrict__ conv_w, const DeltaShape& s, int c, int pos, int back) {
    float acc = 0.f;
    const int C = s.conv_channels();
    for (int j = 0; j < s.taps; ++j) {
        const int d = s.taps - 1 - j;          // how many tokens back
        const int p = pos - d;
        if (p < 0) continue;
        const float x = d <= back ? to_f32<T>(proj_row[c - (long long)d * s.proj_width])
                                  : to_f32<T>(ring_slot[(size_t)(p % s.taps) * C + c]);
        acc = fmaf(conv_w[(size_t)c * s.taps + j], x, acc);
    }
    return acc;
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// The decay g = exp(-exp(a_log) softplus(a)).  A sequence's memory of a token far back is that
// token's write times the product of every g since, so an error of g that leans one way grows
// with the distance.  With float32 activations g is therefore computed in double and rounded
// once; with bfloat16 activations in float32.
template <typename T>
__device__ __forceinline__ float decay_of(float a_log, float a) {
    return expf(-expf(a_log) * softplus_f(a));
}
template <>
__device__ __forceinline__ float decay_of<float>(float a_log, float a) {
    const double z = (double)a;
    const double sp = z > 30.0 ? z : log1p(exp(z));
    return (float)exp(-exp((double)a_log) * sp);
}

template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(
    float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vc, float* __restrict__ beta,
    float* __restrict__ decay, const T* __restrict__ proj, const float* __restrict__ conv_w,
    const float* __restrict__ a_log, const float* __restrict__ dt_bias, const T* __restrict__ ring,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, const int* __restrict__ seq_lens, DeltaShape s,
    float unit_eps) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float act[];             // the row's convolved and activated q | k channels
    const int m = blockIdx.x;
    const int slot = row_slot[m], pos = row_pos[m];
    const int back = pos - seq_lens[slot];
    const int C = s.conv_channels(), QK = s.qk_channels();
    const T* row = proj + (size_t)m * s.proj_width;
    const T* ring_slot = ring + (size_t)slot * s.taps * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float y = silu_f(conv_at<T>(row, ring_slot, conv_w, s, c, pos, back));
        if (c < 2 * QK) act[c] = y;
        else vc[(size_t)m * (C - 2 * QK) + (c - 2 * QK)] = y;
    }
    for (int h = threadIdx.x; h < s.n_heads; h += blockDim.x) {
        const float b = to_f32<T>(row[s.b_offset() + h]);
        beta[(size_t)m * s.n_heads + h] = 1.0f / (1.0f + expf(-b));
        const float a = to_f32<T>(row[s.a_offset() + h]) + dt_bias[h];
        decay[(size_t)m * s.n_heads + h] = decay_of<T>(a_log[h], a);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int g = warp; g < 2 * s.n_kv; g += blockDim.x >> 5) {      // q groups, then k groups
        const float* x = act + g * s.dk;
        float ss = 0.f;
        for (int i = lane; i < s.dk; i += 32) ss += x[i] * x[i];
        ss = warp_sum(ss);
        const bool is_q = g < s.n_kv;
        const float r = (1.0f / sqrtf(ss + unit_eps)) * (is_q ? 1.0f / sqrtf((float)s.dk) : 1.0f);
        float* dst = is_q ? qn + ((size_t)m * s.n_kv + g) * s.dk : kn + ((size_t)m * s.n_kv + (g - s.n_kv)) * s.dk;
        for (int i = lane; i < s.dk; i += 32) dst[i] = x[i] * r;
    }
}

// ------------------------------------------------------------------ recurrence

constexpr int kLanesPerColumn = 8;
constexpr int kColumnsPerWarp = 32 / kLanesPerColumn;
constexpr int kRecurrenceWarps = 4;
constexpr int kColumnsPerBlock = kColumnsPerWarp * kRecurrenceWarps;

// Entry of the key axis that register r of lane l (of a column's 8 lanes) holds: with VEC 4 a
// lane holds runs of four consecutive entries (16-byte accesses), with VEC 1 every eighth.
template <int VEC>
__device__ __forceinline__ int key_index(int r, int l) {
    return VEC * (kLanesPerColumn * (r / VEC) + l) + (r % VEC);
}

template <typename A>
__device__ __forceinline__ A column_sum(A v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}

__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

constexpr int kTokensPerStage = 16;

// Entry of the key axis that register r of lane l (of a column's L lanes) holds.
template <int VEC, int L>
__device__ __forceinline__ int key_index_of(int r, int l) {
    return VEC * (L * (r / VEC) + l) + (r % VEC);
}

template <int L, typename A>
__device__ __forceinline__ A lanes_sum(A v) {
#pragma unroll
    for (int o = 1; o < L; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One block: one sequence of the step, one head, (32 / L) * W columns of its state, a column
// held by L lanes with R registers each (dk <= L R; entries beyond dk are zero and stay zero).
// L = 8 does the least work per column; L = 32 gives four times as many warps with a quarter
// of the registers each, for steps with so few columns that the schedulers would otherwise
// have one warp each and every latency of the token-by-token chain would show.
// The tokens' k, q, v, b and g come through shared memory, kTokensPerStage tokens at a time in
// two buffers filled by asynchronous copies, so that every warp of the block reads one copy
// and the next tokens travel while these are worked on; the read-outs of a stage are written
// together.  The sums over the key axis run in up to four partial sums (a shorter chain of
// dependent additions), in an order fixed by the lane layout.
// A: the type the state is carried in between the step's first and last token (the state in
// memory is float32 either way).  With double, the roundings of a long prompt's tokens do not
// add up: the true 32-bit path uses it, so that its result is the float32 rounding of the
// recurrence rather than a thousand roundings later.
template <int R, int VEC, int L, int W, typename A>
__global__ void __launch_bounds__(W * 32) delta_recurrence_kernel(
    float* __restrict__ o, float* __restrict__ state, const float* __restrict__ qn, const float* __restrict__ kn,
    const float* __restrict__ vc, const float* __restrict__ beta, const float* __restrict__ decay,
    const int* __restrict__ cu_seqlens, const int* __restrict__ slots, DeltaShape s) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int kThreads = W * 32, kTok = kTokensPerStage, kPad = L * R, kCols = (32 / L) * W;
    constexpr int kParts = R < 4 ? R : 4;
    // per buffer: k [kTok][kPad], q [kTok][kPad], v [kTok][kCols], b [kTok], g [kTok]; then o [kTok][kCols]
    extern __shared__ __align__(16) float stage_mem[];
    constexpr int kStageFloats = 2 * kTok * kPad + kTok * kCols + 2 * kTok;
    float* o_s = stage_mem + 2 * kStageFloats;
    const int seq = blockIdx.x, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane & (L - 1);
    const int col_in_block = warp * (32 / L) + lane / L;
    const int col0 = blockIdx.z * kCols, col = col0 + col_in_block;
    const bool live = col < s.dv;
    const int n_cols = min(kCols, s.dv - col0);
    const int g = head / (s.n_heads / s.n_kv);
    const int row0 = cu_seqlens[seq], row1 = cu_seqlens[seq + 1];
    float* S = state + (((size_t)slots[seq] * s.n_heads + head) * s.dv + (live ? col : 0)) * s.dk;
    const bool wide_k = s.dk % 4 == 0;
    const bool wide_v = n_cols == kCols && s.dv % 4 == 0 && kCols % 4 == 0;

    // the padding of the k and q rows stays zero for the whole kernel
    for (int i = threadIdx.x; i < 2 * kStageFloats; i += kThreads) stage_mem[i] = 0.f;
    __syncthreads();

    auto copy16 = [](float* dst, const float* src) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
    };
    auto copy4 = [](float* dst, const float* src) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
    };
    // every thread takes its share of the stage's copies
    auto issue = [&](int first_row, float* buf) {
        const int n = min(kTok, row1 - first_row);
        const int per_row = wide_k ? s.dk / 4 : s.dk;                 // copies per row of k or q
        for (int e = threadIdx.x; e < 2 * n * per_row; e += kThreads) {
            const int t2 = e / per_row, i = (e - t2 * per_row) * (wide_k ? 4 : 1);
            const int t = t2 >> 1, is_q = t2 & 1;
            const float* src = (is_q ? qn : kn) + ((size_t)(first_row + t) * s.n_kv + g) * s.dk + i;
            float* dst = buf + (is_q * kTok + t) * kPad + i;
            if (wide_k) copy16(dst, src); else copy4(dst, src);
        }
        float* v_s = buf + 2 * kTok * kPad;
        const int per_v = wide_v ? kCols / 4 : n_cols;
        for (int e = threadIdx.x; e < n * per_v; e += kThreads) {
            const int t = e / per_v, c = (e - t * per_v) * (wide_v ? 4 : 1);
            const float* src = vc + ((size_t)(first_row + t) * s.n_heads + head) * s.dv + col0 + c;
            if (wide_v) copy16(v_s + t * kCols + c, src); else copy4(v_s + t * kCols + c, src);
        }
        float* bg_s = v_s + kTok * kCols;
        for (int t = threadIdx.x; t < 2 * n; t += kThreads) {
            const int tt = t < n ? t : t - n;
            copy4(bg_s + (t < n ? 0 : kTok) + tt, (t < n ? beta : decay) + (size_t)(first_row + tt) * s.n_heads + head);
        }
        copy_async_commit();
    };

    A st[R];
#pragma unroll
    for (int r = 0; r < R; r += VEC) {
        const int i = key_index_of<VEC, L>(r, l);
        if (VEC == 4) {
            const float4 v = (live && i < s.dk) ? *reinterpret_cast<const float4*>(S + i) : make_float4(0, 0, 0, 0);
            st[r] = v.x; st[r + 1] = v.y; st[r + 2] = v.z; st[r + 3] = v.w;
        } else {
            st[r] = (live && i < s.dk) ? S[i] : 0.f;
        }
    }

    if (row0 < row1) issue(row0, stage_mem);
    int which = 0;
    for (int first = row0; first < row1; first += kTok, which ^= 1) {
        float* buf = stage_mem + which * kStageFloats;
        if (first + kTok < row1) issue(first + kTok, stage_mem + (which ^ 1) * kStageFloats);
        else copy_async_commit();
        copy_async_wait<1>();
        __syncthreads();
        const int n = min(kTok, row1 - first);
        const float* v_s = buf + 2 * kTok * kPad;
        const float* bg_s = v_s + kTok * kCols;
#pragma unroll 2
        for (int t = 0; t < n; ++t) {
            float kr[R], qr[R];
#pragma unroll
            for (int r = 0; r < R; r += VEC) {
                const int i = key_index_of<VEC, L>(r, l);    // < L R: inside the padded row
                if (VEC == 4) {
                    const float4 a = *reinterpret_cast<const float4*>(buf + t * kPad + i);
                    const float4 b = *reinterpret_cast<const float4*>(buf + (kTok + t) * kPad + i);
                    kr[r] = a.x; kr[r + 1] = a.y; kr[r + 2] = a.z; kr[r + 3] = a.w;
                    qr[r] = b.x; qr[r + 1] = b.y; qr[r + 2] = b.z; qr[r + 3] = b.w;
                } else {
                    kr[r] = buf[t * kPad + i];
                    qr[r] = buf[(kTok + t) * kPad + i];
                }
            }
            const A v = v_s[t * kCols + col_in_block], b = bg_s[t], gd = bg_s[kTok + t];
            A part[kParts];
#pragma unroll
            for (int i = 0; i < kParts; ++i) part[i] = 0;
#pragma unroll
            for (int r = 0; r < R; ++r) part[r % kParts] = fma(st[r], (A)kr[r], part[r % kParts]);
#pragma unroll
            for (int i = 1; i < kParts; ++i) part[0] += part[i];
            const A dot = lanes_sum<L>(part[0]);
            const A u = b * (v - gd * dot);
            A read[kParts];
#pragma unroll
            for (int i = 0; i < kParts; ++i) read[i] = 0;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                st[r] = fma((A)kr[r], u, gd * st[r]);
                read[r % kParts] = fma(st[r], (A)qr[r], read[r % kParts]);
            }
#pragma unroll
            for (int i = 1; i < kParts; ++i) read[0] += read[i];
            const A out = lanes_sum<L>(read[0]);
            if (l == 0) o_s[t * kCols + col_in_block] = (float)out;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < n * n_cols; e += kThreads) {
            const int t = e / n_cols, c = e % n_cols;
            o[((size_t)(first + t) * s.n_heads + head) * s.dv + col0 + c] = o_s[t * kCols + c];
        }
    }
    copy_async_wait<0>();
    if (live) {
#pragma unroll
        for (int r = 0; r < R; r += VEC) {
            const int i = key_index_of<VEC, L>(r, l);
            if (i >= s.dk) continue;
            if (VEC == 4)
                *reinterpret_cast<float4*>(S + i) = make_float4((float)st[r], (float)st[r + 1], (float)st[r + 2], (float)st[r + 3]);
            else
                S[i] = (float)st[r];
        }
    }
}

template <int R, int L, int W>
constexpr size_t recurrence_smem() {
    return sizeof(float) * (2 * (2 * kTokensPerStage * L * R + kTokensPerStage * (32 / L) * W + 2 * kTokensPerStage) +
                            kTokensPerStage * (32 / L) * W);
}

// After a step: the raw projections of the step's last taps - 1 positions go into the ring
// (position p at p mod taps).  One block per sequence.  Nothing reads the ring while this
// runs: the kernels of the step that read it have ended.
template <typename T>
__global__ void conv_ring_update_kernel(T* __restrict__ ring, const T* __restrict__ proj,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                        const int* __restrict__ seq_lens, DeltaShape s) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x;
    const int row0 = cu_seqlens[seq], n = cu_seqlens[seq + 1] - row0;
    const int slot = slots[seq], start = seq_lens[slot];
    const int C = s.conv_channels();
    const int keep = n < s.taps - 1 ? n : s.taps - 1;
    T* dst = ring + (size_t)slot * s.taps * C;
    for (int t = n - keep; t < n; ++t) {
        const int p = start + t;
        for (int c = threadIdx.x; c < C; c += blockDim.x)
            dst[(size_t)(p % s.taps) * C + c] = proj[(size_t)(row0 + t) * s.proj_width + c];
    }
}

// ------------------------------------------------------------------ one token per sequence

// The whole mixer step for one token of one sequence, between the projection and the output
// norm: one block per (sequence, head, kColumnsPerBlock columns).  The block convolves and
// normalises the q and k channels of its head's group (every block of the group does, the
// work is small), the v channels of its columns, updates its columns of the state and writes
// its part of the read-out.  The token's raw projection goes into the ring at pos mod taps,
// a place that no block reads in this step (the taps - 1 predecessors lie elsewhere); blocks
// of one group write the same q and k values there.
template <typename T, int R, int VEC>
__global__ void __launch_bounds__(kRecurrenceWarps * 32) delta_decode_kernel(
    float* __restrict__ o, float* __restrict__ state, T* __restrict__ ring, const T* __restrict__ proj,
    const float* __restrict__ conv_w, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, DeltaShape s, float unit_eps) {
    pdl_launch_dependents();
    extern __shared__ float sh[];              // k [dk], q [dk]
    __shared__ float sums[2][kRecurrenceWarps];
    const int m = blockIdx.x, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane & (kLanesPerColumn - 1);
    const int col = blockIdx.z * kColumnsPerBlock + warp * kColumnsPerWarp + lane / kLanesPerColumn;
    const bool live = col < s.dv;
    const int g = head / (s.n_heads / s.n_kv);
    const int C = s.conv_channels(), QK = s.qk_channels();
    pdl_wait();
    const int slot = row_slot[m], pos = row_pos[m];
    const T* row = proj + (size_t)m * s.proj_width;
    T* ring_slot = ring + (size_t)slot * s.taps * C;
    float* S = state + (((size_t)slot * s.n_heads + head) * s.dv + (live ? col : 0)) * s.dk;

    // state loads first: they are the step's traffic
    float st[R];
#pragma unroll
    for (int r = 0; r < R; r += VEC) {
        const int i = key_index<VEC>(r, l);
        if (VEC == 4) {
            const float4 v = (live && i < s.dk) ? *reinterpret_cast<const float4*>(S + i) : make_float4(0, 0, 0, 0);
            st[r] = v.x; st[r + 1] = v.y; st[r + 2] = v.z; st[r + 3] = v.w;
        } else {
            st[r] = (live && i < s.dk) ? S[i] : 0.f;
        }
    }
    // q and k of the group: convolution, silu, sums of squares
    float ss_k = 0.f, ss_q = 0.f;
    for (int i = threadIdx.x; i < 2 * s.dk; i += blockDim.x) {
        const bool is_q = i >= s.dk;
        const int c = (is_q ? 0 : QK) + g * s.dk + (is_q ? i - s.dk : i);
        const float y = silu_f(conv_at<T>(row, ring_slot, conv_w, s, c, pos, 0));
        sh[i] = y;
        if (is_q) ss_q += y * y; else ss_k += y * y;
        if (blockIdx.z == 0) ring_slot[(size_t)(pos % s.taps) * C + c] = row[c];
    }
    ss_k = warp_sum(ss_k);
    ss_q = warp_sum(ss_q);
    if (lane == 0) { sums[0][warp] = ss_k; sums[1][warp] = ss_q; }
    // v of this lane's column
    float v = 0.f;
    if (live) {
        const int c = 2 * QK + head * s.dv + col;
        v = silu_f(conv_at<T>(row, ring_slot, conv_w, s, c, pos, 0));
        if (l == 0) ring_slot[(size_t)(pos % s.taps) * C + c] = row[c];
    }
    const float b = 1.0f / (1.0f + expf(-to_f32<T>(row[s.b_offset() + head])));
    const float gd = decay_of<T>(a_log[head], to_f32<T>(row[s.a_offset() + head]) + dt_bias[head]);
    __syncthreads();
    float tk = 0.f, tq = 0.f;
#pragma unroll
    for (int w = 0; w < kRecurrenceWarps; ++w) { tk += sums[0][w]; tq += sums[1][w]; }
    const float rk = 1.0f / sqrtf(tk + unit_eps);
    const float rq = (1.0f / sqrtf(tq + unit_eps)) * (1.0f / sqrtf((float)s.dk));

    float kr[R], qr[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = key_index<VEC>(r, l);
        kr[r] = i < s.dk ? sh[i] * rk : 0.f;
        qr[r] = i < s.dk ? sh[s.dk + i] * rq : 0.f;
    }
    float dot = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) dot = fmaf(st[r], kr[r], dot);
    dot = column_sum(dot);
    const float u = b * (v - gd * dot);
    float read = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        st[r] = fmaf(kr[r], u, gd * st[r]);
        read = fmaf(st[r], qr[r], read);
    }
    read = column_sum(read);
    if (live) {
        if (l == 0) o[((size_t)m * s.n_heads + head) * s.dv + col] = read;
#pragma unroll
        for (int r = 0; r < R; r += VEC) {
            const int i = key_index<VEC>(r, l);
            if (i >= s.dk) continue;
            if (VEC == 4) *reinterpret_cast<float4*>(S + i) = make_float4(st[r], st[r + 1], st[r + 2], st[r + 3]);
            else S[i] = st[r];
        }
    }
}

int check_shape(const DeltaShape& s, const char* what) {
    THN_CHECK_ARG(s.n_heads > 0 && s.n_kv > 0 && s.dk > 0 && s.dv > 0 && s.taps > 0, "%s: bad sizes", what);
    THN_CHECK_ARG(s.n_heads % s.n_kv == 0, "%s: %d heads are not a multiple of %d key heads", what, s.n_heads, s.n_kv);
    THN_CHECK_ARG(s.proj_width >= s.a_offset() + s.n_heads, "%s: projected rows of %d are too short", what, s.proj_width);
    THN_UNSUPPORTED_IF(s.dk > 512, "%s: key size %d above 512", what, s.dk);
    return THN_OK;
}

// (Launched in plain stream order: see thn_launch_ordered.  1.46 against 0.73 ms for one
// 2,048-token prompt of 16 heads of 128 x 128 on B200.)
template <int R, int VEC, int L, int W>
void launch_recurrence(float* o, float* state, const float* qn, const float* kn, const float* vc, const float* beta,
                       const float* decay, const int* cu, const int* slots, int n_seqs, DeltaShape s, int carry_double,
                       cudaStream_t stream) {
    constexpr int kCols = (32 / L) * W;
    constexpr size_t smem = recurrence_smem<R, L, W>();
    dim3 grid(n_seqs, s.n_heads, (s.dv + kCols - 1) / kCols);
    if (carry_double) {
        if (smem > 32 * 1024)
            cudaFuncSetAttribute(delta_recurrence_kernel<R, VEC, L, W, double>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        thn_launch_ordered(delta_recurrence_kernel<R, VEC, L, W, double>, grid, W * 32, smem, stream, o, state, qn, kn, vc, beta,
                   decay, cu, slots, s);
    } else {
        if (smem > 32 * 1024)
            cudaFuncSetAttribute(delta_recurrence_kernel<R, VEC, L, W, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        thn_launch_ordered(delta_recurrence_kernel<R, VEC, L, W, float>, grid, W * 32, smem, stream, o, state, qn, kn, vc, beta,
                   decay, cu, slots, s);
    }
}

template <typename T, int R, int VEC>
void launch_decode(float* o, float* state, void* ring, const void* proj, const float* conv_w, const float* a_log,
                   const float* dt_bias, const int* row_slot, const int* row_pos, int n_rows, DeltaShape s,
                   float unit_eps, cudaStream_t stream) {
    dim3 grid(n_rows, s.n_heads, (s.dv + kColumnsPerBlock - 1) / kColumnsPerBlock);
    thn_launch(delta_decode_kernel<T, R, VEC>, grid, kRecurrenceWarps * 32, 2 * s.dk * sizeof(float), stream, o, state,
               (T*)ring, (const T*)proj, conv_w, a_log, dt_bias, row_slot, row_pos, s, unit_eps);
}

// Registers of state per lane for a key size, and whether 16-byte accesses fit.
#define THN_DELTA_DISPATCH(CALL)                                   \
    do {                                                           \
        const bool vec = s.dk % 4 == 0;                            \
        if (s.dk <= 32) { if (vec) CALL(4, 4); else CALL(4, 1); }          \
        else if (s.dk <= 64) { if (vec) CALL(8, 4); else CALL(8, 1); }     \
        else if (s.dk <= 128) { if (vec) CALL(16, 4); else CALL(16, 1); }  \
        else if (s.dk <= 256) { if (vec) CALL(32, 4); else CALL(32, 1); }  \
        else { if (vec) CALL(64, 4); else CALL(64, 1); }                   \
    } while (0)

}  // namespace

// proj [n_rows, proj_width] of the activation type (columns q | k | v | gate | b | a);
// conv_w float32 [channels, taps]; a_log, dt_bias float32 [heads]; ring as described above;
// seq_lens [slots]: tokens a sequence held before this step.  Outputs float32: qn, kn
// [n_rows, n_kv, dk], vc [n_rows, heads, dv], beta, decay [n_rows, heads].
THN_API int thn_delta_prepare(float* qn, float* kn, float* vc, float* beta, float* decay, const void* proj,
                              const float* conv_w, const float* a_log, const float* dt_bias, const void* ring,
                              const int* row_slot, const int* row_pos, const int* seq_lens, int n_rows, int n_heads,
                              int n_kv, int dk, int dv, int taps, int proj_width, float unit_eps, int dtype,
                              cudaStream_t stream) {
    DeltaShape s{n_heads, n_kv, dk, dv, taps, proj_width};
    if (int status = check_shape(s, "delta_prepare")) return status;
    if (n_rows <= 0) return THN_OK;
    const size_t smem = (size_t)2 * s.qk_channels() * sizeof(float);
    THN_UNSUPPORTED_IF(smem > 48 * 1024, "delta_prepare: %d key channels do not fit shared memory", 2 * s.qk_channels());
    if (dtype == THN_F32)
        thn_launch(delta_prepare_kernel<float>, n_rows, 128, smem, stream, qn, kn, vc, beta, decay, (const float*)proj,
                   conv_w, a_log, dt_bias, (const float*)ring, row_slot, row_pos, seq_lens, s, unit_eps);
    else if (dtype == THN_BF16)
        thn_launch(delta_prepare_kernel<__nv_bfloat16>, n_rows, 128, smem, stream, qn, kn, vc, beta, decay,
                   (const __nv_bfloat16*)proj, conv_w, a_log, dt_bias, (const __nv_bfloat16*)ring, row_slot, row_pos,
                   seq_lens, s, unit_eps);
    else
        THN_CHECK_ARG(false, "delta_prepare: unknown dtype %d", dtype);
    return thn_launch_status("delta_prepare");
}

// The recurrence over the rows of each of the step's sequences; o float32 [n_rows, heads, dv];
// state float32 [slots, heads, dv, dk], read and written.  carry_double: the state is carried
// in double between the step's first and last token.  lanes: 8 or 32 lanes per column of the
// state, or 0 to choose by the step's size (the result differs by rounding only).
THN_API int thn_delta_recurrence(float* o, float* state, const float* qn, const float* kn, const float* vc,
                                 const float* beta, const float* decay, const int* cu_seqlens, const int* slots,
                                 int n_seqs, int n_heads, int n_kv, int dk, int dv, int carry_double, int lanes,
                                 cudaStream_t stream) {
    DeltaShape s{n_heads, n_kv, dk, dv, 1, 1 << 30};
    if (int status = check_shape(s, "delta_recurrence")) return status;
    if (n_seqs <= 0) return THN_OK;
    THN_UNSUPPORTED_IF(n_heads > 65535, "delta_recurrence: %d heads exceed the grid limit", n_heads);
    // Eight lanes per column unless that leaves most SMs without a warp; then 32 lanes.  (One
    // 2,048-token prompt of 16 heads of 128 x 128, four warps per SM at 8 lanes: 0.65 ms against
    // 0.72 ms with 32 lanes, which execute twice the instructions.)
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    const long long warps_at_8 = (long long)n_seqs * n_heads * dv / 4;
    const bool narrow = lanes > 0 ? lanes == 8 : warps_at_8 >= (long long)(sms > 0 ? sms : 148) * 2;
    const bool vec = dk % 4 == 0;
#define CALL8(R, VEC) launch_recurrence<R, VEC, 8, 4>(o, state, qn, kn, vc, beta, decay, cu_seqlens, slots, n_seqs, s, carry_double, stream)
#define CALL32(R, VEC) launch_recurrence<R, VEC, 32, 8>(o, state, qn, kn, vc, beta, decay, cu_seqlens, slots, n_seqs, s, carry_double, stream)
    if (narrow) {
        THN_DELTA_DISPATCH(CALL8);
    } else if (dk <= 32) {
        CALL32(1, 1);
    } else if (dk <= 64) {
        CALL32(2, 1);
    } else if (dk <= 128) {
        if (vec) CALL32(4, 4); else CALL32(4, 1);
    } else if (dk <= 256) {
        if (vec) CALL32(8, 4); else CALL32(8, 1);
    } else {
        THN_DELTA_DISPATCH(CALL8);        // key sizes above 256: 8 lanes of 64 registers
    }
#undef CALL8
#undef CALL32
    return thn_launch_status("delta_recurrence");
}

THN_API int thn_delta_conv_ring_update(void* ring, const void* proj, const int* cu_seqlens, const int* slots,
                                       const int* seq_lens, int n_seqs, int n_heads, int n_kv, int dk, int dv, int taps,
                                       int proj_width, int dtype, cudaStream_t stream) {
    DeltaShape s{n_heads, n_kv, dk, dv, taps, proj_width};
    if (int status = check_shape(s, "delta_conv_ring_update")) return status;
    if (n_seqs <= 0 || taps <= 1) return THN_OK;
    if (dtype == THN_F32)
        thn_launch(conv_ring_update_kernel<float>, n_seqs, 256, 0, stream, (float*)ring, (const float*)proj, cu_seqlens,
                   slots, seq_lens, s);
    else if (dtype == THN_BF16)
        thn_launch(conv_ring_update_kernel<__nv_bfloat16>, n_seqs, 256, 0, stream, (__nv_bfloat16*)ring,
                   (const __nv_bfloat16*)proj, cu_seqlens, slots, seq_lens, s);
    else
        THN_CHECK_ARG(false, "delta_conv_ring_update: unknown dtype %d", dtype);
    return thn_launch_status("delta_conv_ring_update");
}

// One token per sequence: prepare, recurrence and ring update in one launch.
THN_API int thn_delta_decode(float* o, float* state, void* ring, const void* proj, const float* conv_w,
                             const float* a_log, const float* dt_bias, const int* row_slot, const int* row_pos,
                             int n_rows, int n_heads, int n_kv, int dk, int dv, int taps, int proj_width, float unit_eps,
                             int dtype, cudaStream_t stream) {
    DeltaShape s{n_heads, n_kv, dk, dv, taps, proj_width};
    if (int status = check_shape(s, "delta_decode")) return status;
    if (n_rows <= 0) return THN_OK;
    THN_UNSUPPORTED_IF(n_heads > 65535, "delta_decode: %d heads exceed the grid limit", n_heads);
    if (dtype == THN_F32) {
#define CALL(R, VEC) launch_decode<float, R, VEC>(o, state, ring, proj, conv_w, a_log, dt_bias, row_slot, row_pos, n_rows, s, unit_eps, stream)
        THN_DELTA_DISPATCH(CALL);
#undef CALL
    } else if (dtype == THN_BF16) {
#define CALL(R, VEC) launch_decode<__nv_bfloat16, R, VEC>(o, state, ring, proj, conv_w, a_log, dt_bias, row_slot, row_pos, n_rows, s, unit_eps, stream)
        THN_DELTA_DISPATCH(CALL);
#undef CALL
    } else {
        THN_CHECK_ARG(false, "delta_decode: unknown dtype %d", dtype);
    }
    return thn_launch_status("delta_decode");
}
