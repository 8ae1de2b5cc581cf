// Norms around a residual stream that is kept in float32 whatever the activation type is,
// with an optional norm of the branch output before it is added:
//
//     h <- h + m B(d + d2)   (d2, a second branch output, may be absent; m is 1 unless given)
//                      B(d) = d                                                  (post kind 0)
//                      B(d) = d / sqrt(mean(d^2) + eps_b) * (o_b + w_b)          (post kind 1, RMS)
//                      B(d) = (d - mean d) / sqrt(var d + eps_b) * (o_b + w_b) + b_b   (post kind 2, layer norm)
//     y  = N(h) with N of kind 1 or 2 as above (gain w, bias b), or
//     y  = h rounded to the activation type (kind 3: the stream itself is what a sublayer reads), or
//     no y (kind 0).
//
// An RMS norm of the stream (kind 1) may work in `groups` equal consecutive parts of the row,
// each divided by its own sqrt(mean(part^2) + eps) before the gain over the whole row.
//
// o_b and o are gain offsets: 0 for a gain stored as it multiplies, 1 for a gain stored around
// zero; a bias may be absent.  The variance is the mean of the squared deviations from the mean
// (two passes over the staged row).  Every sum, both square roots and the residual sum are
// float32; y is rounded once to the activation type T.  One block per row, the row staged in
// shared memory; the order of additions depends on the block size only, so a row's result does
// not depend on its batch.
#include <type_traits>

#include "common.cuh"

namespace {
constexpr int kThreads = 256;

struct NormArgs {
    const float* gain;
    const float* bias;
    float offset;
    float eps;
    int kind;     // 0 none, 1 RMS, 2 layer norm, 3 (output only) the stream as it is
    int groups;   // kind 1 as an output: equal consecutive parts with statistics of their own (1: the whole row)
};

// 1 / sqrt(mean(part^2) + eps) of each of `groups` equal parts of the staged row, into rstd[];
// a warp takes a part at a time, so the order of additions depends on the sizes only.
__device__ __forceinline__ void group_statistics(const float* row, int width, int groups, float eps, float* rstd) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, per = width / groups;
    for (int g = warp; g < groups; g += kThreads / 32) {
        float ss = 0.f;
        for (int i = lane; i < per; i += 32) ss += row[g * per + i] * row[g * per + i];
        ss = warp_sum(ss);
        if (lane == 0) rstd[g] = 1.0f / sqrtf(ss / (float)per + eps);
    }
    __syncthreads();
}

// (mean, 1 / sqrt(var + eps)) of the staged row for a norm of the given kind; mean is 0 for RMS.
__device__ __forceinline__ float2 row_statistics(const float* row, int width, int kind, float eps, float* scratch) {
    float mean = 0.f;
    if (kind == 2) {
        float s = 0.f;
        for (int i = threadIdx.x; i < width; i += kThreads) s += row[i];
        mean = block_sum(s, scratch) / (float)width;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += kThreads) {
        const float c = row[i] - mean;
        ss += c * c;
    }
    const float total = block_sum(ss, scratch);
    return make_float2(mean, 1.0f / sqrtf(total / (float)width + eps));
}

template <typename T>
__global__ void __launch_bounds__(kThreads) residual_norm_kernel(
    T* __restrict__ y, float* __restrict__ h, const T* __restrict__ d, const T* __restrict__ d2, float mult,
    NormArgs post, NormArgs out, int width, int h_is_new) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float row[];
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * width;
    if (d) {
        for (int i = threadIdx.x; i < width; i += kThreads)
            row[i] = d2 ? to_f32<T>(d[base + i]) + to_f32<T>(d2[base + i]) : to_f32<T>(d[base + i]);
        float2 st = make_float2(0.f, 1.f);
        if (post.kind) {
            __syncthreads();
            st = row_statistics(row, width, post.kind, post.eps, scratch);
        }
        for (int i = threadIdx.x; i < width; i += kThreads) {
            float v = row[i];
            if (post.kind) {
                v = (v - st.x) * st.y * (post.offset + post.gain[i]);
                if (post.bias) v += post.bias[i];
            }
            v *= mult;
            if (!h_is_new) v = h[base + i] + v;
            h[base + i] = v;
            row[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += kThreads) row[i] = h[base + i];
    }
    if (!out.kind) return;
    if (out.kind == 3) {
        for (int i = threadIdx.x; i < width; i += kThreads) y[base + i] = from_f32<T>(row[i]);
        return;
    }
    __syncthreads();
    if (out.kind == 1 && out.groups > 1) {
        float* rstd = row + width;
        group_statistics(row, width, out.groups, out.eps, rstd);
        const int per = width / out.groups;
        for (int i = threadIdx.x; i < width; i += kThreads) {
            float v = row[i] * rstd[i / per] * (out.offset + out.gain[i]);
            if (out.bias) v += out.bias[i];
            y[base + i] = from_f32<T>(v);
        }
        return;
    }
    const float2 st = row_statistics(row, width, out.kind, out.eps, scratch);
    for (int i = threadIdx.x; i < width; i += kThreads) {
        float v = (row[i] - st.x) * st.y * (out.offset + out.gain[i]);
        if (out.bias) v += out.bias[i];
        y[base + i] = from_f32<T>(v);
    }
}

// The same for bfloat16 activations, rows of a multiple of eight values and 16-byte aligned
// operands: every access to global memory moves eight values (16 bytes of bfloat16, two 16-byte
// pieces of float32).  The staged row, the statistics and every formula are those of the kernel
// above, so the two give the same bits.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(pairs[k]);
        v[2 * k] = f.x, v[2 * k + 1] = f.y;
    }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) pairs[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

__global__ void __launch_bounds__(kThreads) residual_norm_bf16x8_kernel(
    __nv_bfloat16* __restrict__ y, float* __restrict__ h, const __nv_bfloat16* __restrict__ d,
    const __nv_bfloat16* __restrict__ d2, float mult, NormArgs post, NormArgs out, int width, int h_is_new) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * width;
    float v[8], u[8];
    if (d) {
        if (post.kind) {
            for (int i = threadIdx.x * 8; i < width; i += kThreads * 8) {
                load8(d + base + i, v);
                if (d2) {
                    load8(d2 + base + i, u);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] += u[e];
                }
                store8(row + i, v);
            }
            __syncthreads();
        }
        float2 st = make_float2(0.f, 1.f);
        if (post.kind) st = row_statistics(row, width, post.kind, post.eps, scratch);
        for (int i = threadIdx.x * 8; i < width; i += kThreads * 8) {
            if (post.kind) {
                load8(row + i, v);
                load8(post.gain + i, u);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = (v[e] - st.x) * st.y * (post.offset + u[e]);
                if (post.bias) {
                    load8(post.bias + i, u);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] += u[e];
                }
            } else {
                load8(d + base + i, v);
                if (d2) {
                    load8(d2 + base + i, u);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] += u[e];
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] *= mult;
            if (!h_is_new) {
                load8(h + base + i, u);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = u[e] + v[e];
            }
            store8(h + base + i, v);
            store8(row + i, v);
        }
    } else {
        for (int i = threadIdx.x * 8; i < width; i += kThreads * 8) {
            load8(h + base + i, v);
            store8(row + i, v);
        }
    }
    if (!out.kind) return;
    if (out.kind == 3) {
        for (int i = threadIdx.x * 8; i < width; i += kThreads * 8) {
            load8(row + i, v);          // the thread's own pieces: no barrier needed
            store8(y + base + i, v);
        }
        return;
    }
    __syncthreads();
    const bool grouped = out.kind == 1 && out.groups > 1;
    float* rstd = row + width;
    float2 st = make_float2(0.f, 1.f);
    if (grouped) group_statistics(row, width, out.groups, out.eps, rstd);
    else st = row_statistics(row, width, out.kind, out.eps, scratch);
    const int per = width / out.groups;
    for (int i = threadIdx.x * 8; i < width; i += kThreads * 8) {
        load8(row + i, v);
        load8(out.gain + i, u);
#pragma unroll
        for (int e = 0; e < 8; ++e)
            v[e] = grouped ? v[e] * rstd[(i + e) / per] * (out.offset + u[e]) : (v[e] - st.x) * st.y * (out.offset + u[e]);
        if (out.bias) {
            load8(out.bias + i, u);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] += u[e];
        }
        store8(y + base + i, v);
    }
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

template <typename T>
int launch(void* y, float* h, const void* d, const void* d2, float mult, NormArgs post, NormArgs out, int rows, int width,
           int h_is_new, cudaStream_t stream) {
    const size_t smem = (size_t)(width + (out.groups > 1 ? out.groups : 0)) * sizeof(float);
    THN_UNSUPPORTED_IF(smem > 200 * 1024, "residual_norm: rows of %d values do not fit shared memory", width);
    if (std::is_same<T, __nv_bfloat16>::value && width % 8 == 0 && aligned16(y) && aligned16(h) && aligned16(d) &&
        aligned16(d2) && aligned16(post.gain) && aligned16(post.bias) && aligned16(out.gain) && aligned16(out.bias)) {
        if (smem > 32 * 1024)
            cudaFuncSetAttribute(residual_norm_bf16x8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        thn_launch(residual_norm_bf16x8_kernel, rows, kThreads, smem, stream, (__nv_bfloat16*)y, h, (const __nv_bfloat16*)d,
                   (const __nv_bfloat16*)d2, mult, post, out, width, h_is_new);
        return thn_launch_status("residual_norm");
    }
    if (smem > 32 * 1024)
        cudaFuncSetAttribute(residual_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    thn_launch(residual_norm_kernel<T>, rows, kThreads, smem, stream, (T*)y, h, (const T*)d, (const T*)d2, mult, post, out, width, h_is_new);
    return thn_launch_status("residual_norm");
}

// out[m, :] = d[m, :] / sqrt(mean(d[m, :]^2) + eps) * w * act(gate[m, :]) per group of `size`
// values: the read-out of a head of a recurrent mixer, normalised over the head, with one gain
// vector shared by the heads (w_stride 0) or one per head (w_stride = size) and a gate taken
// from `gate` (row stride gate_stride); act is silu (gate_kind 0) or the logistic function
// (gate_kind 1).  One warp per (row, head); float32 inside, rounded once.
template <typename T>
__global__ void gated_head_norm_kernel(T* __restrict__ out, const float* __restrict__ o, const T* __restrict__ gate,
                                       long long gate_stride, const float* __restrict__ w, float eps, long long n_units,
                                       int n_heads, int size, int w_stride, int gate_kind, long long out_stride,
                                       float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= n_units) return;
    const long long m = unit / n_heads;
    const int head = (int)(unit - m * n_heads);
    const float* src = o + unit * size;
    float ss = 0.f;
    for (int i = lane; i < size; i += 32) ss += src[i] * src[i];
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)size + eps);
    const T* g = gate + m * gate_stride + (long long)head * size;
    const float* wh = w + (size_t)head * w_stride;
    for (int i = lane; i < size; i += 32) {
        const float z = to_f32<T>(g[i]);
        const float logistic = 1.0f / (1.0f + expf(-z));
        out[m * out_stride + (long long)head * size + i] =
            from_f32<T>(src[i] * rstd * wh[i] * (gate_kind ? logistic : z * logistic) * scale);
    }
}
// One "head" that is a whole long row (one norm over all heads together): a block of 256 threads
// per row instead of a warp, four consecutive entries per thread where the sizes allow.  The
// order of additions depends on the size only.
template <typename T>
__global__ void __launch_bounds__(256) gated_row_norm_kernel(T* __restrict__ out, const float* __restrict__ o,
                                                             const T* __restrict__ gate, long long gate_stride,
                                                             const float* __restrict__ w, float eps, int size,
                                                             int gate_kind, long long out_stride, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const long long m = blockIdx.x;
    const float* src = o + m * size;
    const T* g = gate + m * gate_stride;
    T* dst = out + m * out_stride;
    const bool vec = size % 4 == 0 && (((uintptr_t)src | (uintptr_t)w) & 15) == 0;
    float ss = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 4; i < size; i += 1024) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < size; i += 256) ss += src[i] * src[i];
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)size + eps);
    auto gated = [&](float v, float gain, float z) {
        const float logistic = 1.0f / (1.0f + expf(-z));
        return v * rstd * gain * (gate_kind ? logistic : z * logistic) * scale;
    };
    if (vec) {
        for (int i = threadIdx.x * 4; i < size; i += 1024) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            const float4 gw = *reinterpret_cast<const float4*>(w + i);
            dst[i] = from_f32<T>(gated(v.x, gw.x, to_f32<T>(g[i])));
            dst[i + 1] = from_f32<T>(gated(v.y, gw.y, to_f32<T>(g[i + 1])));
            dst[i + 2] = from_f32<T>(gated(v.z, gw.z, to_f32<T>(g[i + 2])));
            dst[i + 3] = from_f32<T>(gated(v.w, gw.w, to_f32<T>(g[i + 3])));
        }
    } else {
        for (int i = threadIdx.x; i < size; i += 256) dst[i] = from_f32<T>(gated(src[i], w[i], to_f32<T>(g[i])));
    }
}

// The same with four consecutive entries per lane (16-byte loads of the read-out, 8-byte loads
// of the gate and stores), for sizes that are multiples of four and suitably aligned rows.
__global__ void gated_head_norm_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ o,
                                                const __nv_bfloat16* __restrict__ gate, long long gate_stride,
                                                const float* __restrict__ w, float eps, long long n_units, int n_heads,
                                                int size) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= n_units) return;
    const long long m = unit / n_heads;
    const int head = (int)(unit - m * n_heads);
    const float* src = o + unit * size;
    const __nv_bfloat16* g = gate + m * gate_stride + (long long)head * size;
    float4 first = make_float4(0, 0, 0, 0);          // the first chunk stays in registers (sizes up to 128: the only one)
    float ss = 0.f;
    for (int i = lane * 4; i < size; i += 128) {
        const float4 v = *reinterpret_cast<const float4*>(src + i);
        if (i < 128) first = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)size + eps);
    for (int i = lane * 4; i < size; i += 128) {
        const float4 v = i < 128 ? first : *reinterpret_cast<const float4*>(src + i);
        const float4 gw = *reinterpret_cast<const float4*>(w + i);
        const uint2 gz = *reinterpret_cast<const uint2*>(g + i);
        const float2 z0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gz.x));
        const float2 z1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gz.y));
        uint2 packed;
        *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(
            v.x * rstd * gw.x * (z0.x / (1.0f + expf(-z0.x))), v.y * rstd * gw.y * (z0.y / (1.0f + expf(-z0.y))));
        *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(
            v.z * rstd * gw.z * (z1.x / (1.0f + expf(-z1.x))), v.w * rstd * gw.w * (z1.y / (1.0f + expf(-z1.y))));
        *reinterpret_cast<uint2*>(out + unit * size + i) = packed;
    }
}
}  // namespace

// h float32 [rows, width], updated in place when d is given (h_is_new: h is not read, it
// becomes B(d)); d and y of the activation type; gains and biases float32 [width] (a bias may
// be null).  post_kind 0: d is added as it is; kind 0: no y is written; kind 3: y is h rounded.
// d2 (may be null): a second branch output, added to d before anything else; mult: the factor on
// what is added to h; groups (kind 1 only, a divisor of width): parts of the row with statistics
// of their own.
THN_API int thn_residual_norm(void* y, float* h, const void* d, const void* d2, float mult, const float* post_gain,
                              const float* post_bias, float post_offset, float post_eps, int post_kind, const float* gain,
                              const float* bias, float offset, float eps, int kind, int groups, int rows, int width,
                              int h_is_new, int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && width > 0, "residual_norm: bad sizes rows=%d width=%d", rows, width);
    THN_CHECK_ARG(d2 == nullptr || d != nullptr, "residual_norm: a second branch without a first");
    THN_CHECK_ARG(groups >= 1 && width % groups == 0 && (groups == 1 || kind == 1),
                  "residual_norm: %d groups over rows of %d (an RMS norm of the stream only)", groups, width);
    THN_CHECK_ARG(post_kind >= 0 && post_kind <= 2 && kind >= 0 && kind <= 3, "residual_norm: norm kinds %d, %d", post_kind,
                  kind);
    THN_CHECK_ARG(h != nullptr && (d != nullptr || kind != 0), "residual_norm: nothing to do");
    THN_CHECK_ARG(d != nullptr || !h_is_new, "residual_norm: a new residual stream needs a branch to start from");
    THN_CHECK_ARG(kind == 0 || y != nullptr, "residual_norm: an output norm without y");
    THN_CHECK_ARG(!(kind == 1 || kind == 2) || (gain != nullptr && eps > 0.f), "residual_norm: gain missing, or eps <= 0");
    THN_CHECK_ARG(post_kind == 0 || (post_gain != nullptr && post_eps > 0.f), "residual_norm: post gain missing, or eps <= 0");
    if (rows == 0) return THN_OK;
    const NormArgs post{post_gain, post_bias, post_offset, post_eps, d ? post_kind : 0, 1};
    const NormArgs out{gain, bias, offset, eps, kind, groups};
    if (dtype == THN_F32) return launch<float>(y, h, d, d2, mult, post, out, rows, width, h_is_new, stream);
    if (dtype == THN_BF16) return launch<__nv_bfloat16>(y, h, d, d2, mult, post, out, rows, width, h_is_new, stream);
    THN_CHECK_ARG(false, "residual_norm: unknown dtype %d", dtype);
    return THN_OK;
}

// o float32 [rows, n_heads, size]; gate of the activation type, row stride gate_stride
// elements; w float32 [size] (w_per_head 0) or [n_heads * size] (w_per_head 1); gate_kind 0: silu,
// 1: logistic; out of the activation type [rows, n_heads * size], its rows out_stride elements apart
// (0: n_heads * size); scale: a constant factor on the result.
THN_API int thn_gated_head_norm(void* out, const float* o, const void* gate, long long gate_stride, const float* w,
                                float eps, int rows, int n_heads, int size, int w_per_head, int gate_kind,
                                long long out_stride, float scale, int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && n_heads > 0 && size > 0 && eps > 0.f, "gated_head_norm: bad sizes");
    const long long units = (long long)rows * n_heads;
    if (units == 0) return THN_OK;
    const int warps = 4;
    const unsigned blocks = (unsigned)((units + warps - 1) / warps);
    const int w_stride = w_per_head ? size : 0;
    if (out_stride <= 0) out_stride = (long long)n_heads * size;
    THN_CHECK_ARG(out_stride >= (long long)n_heads * size, "gated_head_norm: output rows %lld apart are too short", out_stride);
    if (dtype == THN_BF16 && !w_per_head && gate_kind == 0 && size % 4 == 0 && gate_stride % 4 == 0 && scale == 1.0f &&
        out_stride == (long long)n_heads * size &&
        ((((uintptr_t)o | (uintptr_t)w) & 15) | (((uintptr_t)gate | (uintptr_t)out) & 7)) == 0) {
        thn_launch(gated_head_norm_bf16_vec_kernel, blocks, warps * 32, 0, stream, (__nv_bfloat16*)out, o,
                   (const __nv_bfloat16*)gate, gate_stride, w, eps, units, n_heads, size);
        return thn_launch_status("gated_head_norm");
    }
    if (n_heads == 1 && size >= 512 && (dtype == THN_F32 || dtype == THN_BF16)) {
        if (dtype == THN_F32)
            thn_launch(gated_row_norm_kernel<float>, rows, 256, 0, stream, (float*)out, o, (const float*)gate, gate_stride, w, eps,
                       size, gate_kind, out_stride, scale);
        else
            thn_launch(gated_row_norm_kernel<__nv_bfloat16>, rows, 256, 0, stream, (__nv_bfloat16*)out, o,
                       (const __nv_bfloat16*)gate, gate_stride, w, eps, size, gate_kind, out_stride, scale);
        return thn_launch_status("gated_head_norm");
    }
    if (dtype == THN_F32)
        thn_launch(gated_head_norm_kernel<float>, blocks, warps * 32, 0, stream, (float*)out, o, (const float*)gate,
                   gate_stride, w, eps, units, n_heads, size, w_stride, gate_kind, out_stride, scale);
    else if (dtype == THN_BF16)
        thn_launch(gated_head_norm_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream, (__nv_bfloat16*)out, o,
                   (const __nv_bfloat16*)gate, gate_stride, w, eps, units, n_heads, size, w_stride, gate_kind, out_stride,
                   scale);
    else
        THN_CHECK_ARG(false, "gated_head_norm: unknown dtype %d", dtype);
    return thn_launch_status("gated_head_norm");
}
