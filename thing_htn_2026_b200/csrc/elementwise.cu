// Row gather (embedding), RMSNorm with and without the residual add, SwiGLU, and the
// small kernels that turn a step's batch description into per-row indices.
//
// Formulas and rounding points: engine/kernels/torch_ref.py:47-58 (RMSNorm: the
// normalised value is rounded before the gain), :61-68 (residual add rounded once),
// :74-88 (silu rounded, product rounded).  Reductions are float32 with an order fixed
// by the block size, so a row's result does not depend on the batch it is in.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

static thread_local char g_error[512] = "";

void thn_set_error(const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, args);
    va_end(args);
}

int g_thn_pdl = 1;

// 0: plain launches; 1 (default): kernels may be scheduled while their predecessor drains.
THN_API void thn_set_pdl(int enabled) { g_thn_pdl = enabled ? 1 : 0; }

THN_API const char* thn_last_error() { return g_error; }
THN_API int thn_abi_version() { return 1; }

// ------------------------------------------------------------------ gather rows

template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ index,
                                   int width, int n_table_rows, int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    int row = index[m];
    if (row < 0 || row >= n_table_rows) {
        if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_TOKEN_RANGE);
        row = 0;
    }
    const T* src = table + (size_t)row * width;
    T* dst = out + (size_t)m * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

THN_API int thn_gather_rows(void* out, const void* table, const int* index, int n_rows, int width,
                            int n_table_rows, int dtype, int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && width > 0 && n_table_rows > 0, "gather_rows: bad sizes rows=%d width=%d table=%d",
                  n_rows, width, n_table_rows);
    if (n_rows == 0) return THN_OK;
    if (dtype == THN_F32)
        thn_launch(gather_rows_kernel<float>, n_rows, 256, 0, stream, (float*)out, (const float*)table, index, width,
                                                              n_table_rows, err);
    else if (dtype == THN_BF16)
        thn_launch(gather_rows_kernel<__nv_bfloat16>, n_rows, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)table, index, width, n_table_rows, err);
    else
        THN_CHECK_ARG(false, "gather_rows: unknown dtype %d", dtype);
    return thn_launch_status("gather_rows");
}

// out[m] = float(table[index[m]]) * scale in float32: token embeddings that start a residual
// stream kept in float32.  With freq (double [ceil(width / 2)]) and row_pos a sinusoidal
// position vector is added: entry 2i gets sin(p f_i), entry 2i + 1 cos(p f_i), p the row's
// position.  The angle and its sine are computed in double and rounded once, so that a far
// position is as exact as a near one.
template <typename T>
__global__ void gather_rows_scaled_kernel(float* __restrict__ out, const T* __restrict__ table,
                                          const int* __restrict__ index, int width, int n_table_rows, float scale,
                                          const int* __restrict__ row_pos, const double* __restrict__ freq,
                                          int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    int row = index[m];
    if (row < 0 || row >= n_table_rows) {
        if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_TOKEN_RANGE);
        row = 0;
    }
    const T* src = table + (size_t)row * width;
    float* dst = out + (size_t)m * width;
    if (freq == nullptr) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = to_f32<T>(src[i]) * scale;
        return;
    }
    const double p = (double)row_pos[m];
    for (int pair = threadIdx.x; 2 * pair < width; pair += blockDim.x) {
        double sn, cs;
        sincos(p * freq[pair], &sn, &cs);
        dst[2 * pair] = to_f32<T>(src[2 * pair]) * scale + (float)sn;
        if (2 * pair + 1 < width) dst[2 * pair + 1] = to_f32<T>(src[2 * pair + 1]) * scale + (float)cs;
    }
}

// row_pos and freq: both or neither.
THN_API int thn_gather_rows_scaled(float* out, const void* table, const int* index, int n_rows, int width,
                                   int n_table_rows, float scale, const int* row_pos, const double* freq, int dtype,
                                   int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && width > 0 && n_table_rows > 0, "gather_rows_scaled: bad sizes rows=%d width=%d table=%d",
                  n_rows, width, n_table_rows);
    THN_CHECK_ARG((row_pos == nullptr) == (freq == nullptr), "gather_rows_scaled: positions and frequencies go together");
    if (n_rows == 0) return THN_OK;
    if (dtype == THN_F32)
        thn_launch(gather_rows_scaled_kernel<float>, n_rows, 256, 0, stream, out, (const float*)table, index, width,
                   n_table_rows, scale, row_pos, freq, err);
    else if (dtype == THN_BF16)
        thn_launch(gather_rows_scaled_kernel<__nv_bfloat16>, n_rows, 256, 0, stream, out, (const __nv_bfloat16*)table, index,
                   width, n_table_rows, scale, row_pos, freq, err);
    else
        THN_CHECK_ARG(false, "gather_rows_scaled: unknown dtype %d", dtype);
    return thn_launch_status("gather_rows_scaled");
}

// x[i] *= scale in place, float32: a constant factor on logits.
__global__ void scale_f32_kernel(float* __restrict__ x, long long n, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) x[e] *= scale;
}

THN_API int thn_scale_f32(float* x, long long n, float scale, cudaStream_t stream) {
    THN_CHECK_ARG(n >= 0, "scale_f32: bad size");
    if (n == 0) return THN_OK;
    const long long want = (n + 255) / 256;
    thn_launch(scale_f32_kernel, (unsigned)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream, x, n, scale);
    return thn_launch_status("scale_f32");
}

// out[m, i] = a[m, i] * logistic(g[m, i]): an output gate on a mixer's concatenated heads.  The
// gate's rows are g_stride elements apart (it may be a slice of a wider projected row).
template <typename T>
__global__ void logistic_gate_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ g,
                                     long long g_stride, long long n, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const long long m = e / width;
    const float z = to_f32<T>(g[m * g_stride + (e - m * width)]);
    out[e] = from_f32<T>(to_f32<T>(a[e]) / (1.0f + expf(-z)));
}

// The same, eight bfloat16 entries per thread (16-byte accesses), one row per blockIdx.y.
__global__ void logistic_gate_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ a,
                                              const __nv_bfloat16* __restrict__ g, long long g_stride, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= width) return;
    const long long row = blockIdx.y;
    const uint4 ra = *reinterpret_cast<const uint4*>(a + row * width + c);
    const uint4 rg = *reinterpret_cast<const uint4*>(g + row * g_stride + c);
    const uint32_t ia[4] = {ra.x, ra.y, ra.z, ra.w}, ig[4] = {rg.x, rg.y, rg.z, rg.w};
    uint32_t res[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ia[i]));
        const float2 z = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ig[i]));
        const __nv_bfloat162 r = __floats2bfloat162_rn(x.x / (1.0f + expf(-z.x)), x.y / (1.0f + expf(-z.y)));
        res[i] = *reinterpret_cast<const uint32_t*>(&r);
    }
    *reinterpret_cast<uint4*>(out + row * width + c) = make_uint4(res[0], res[1], res[2], res[3]);
}

THN_API int thn_logistic_gate(void* out, const void* a, const void* g, long long g_stride, int n_rows, int width,
                              int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && width > 0 && g_stride >= width, "logistic_gate: bad sizes");
    const long long n = (long long)n_rows * width;
    if (n == 0) return THN_OK;
    if (dtype == THN_BF16 && width % 8 == 0 && g_stride % 8 == 0 && n_rows <= 65535 &&
        ((((uintptr_t)out) | ((uintptr_t)a) | ((uintptr_t)g)) & 15) == 0) {
        thn_launch(logistic_gate_bf16_vec_kernel, dim3((width / 8 + 127) / 128, n_rows), 128, 0, stream, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)a, (const __nv_bfloat16*)g, g_stride, width);
        return thn_launch_status("logistic_gate");
    }
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == THN_F32)
        thn_launch(logistic_gate_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)a, (const float*)g,
                   g_stride, n, width);
    else if (dtype == THN_BF16)
        thn_launch(logistic_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)a,
                   (const __nv_bfloat16*)g, g_stride, n, width);
    else
        THN_CHECK_ARG(false, "logistic_gate: unknown dtype %d", dtype);
    return thn_launch_status("logistic_gate");
}

// out[m, c] = turn_back(a[m, head, :])[d] * logistic(g[m, c]) * scale, c = head * size + d: the
// read-out of an attention whose values were turned by their positions before they were cached
// (csrc/qk_prepare.cu) is turned back by the row's own position, pair i by -pos * f_i (the tables
// hold cos and sin of +pos * f_i; layout 0: entry i pairs with i + rotary_dim / 2, 1: 2i with
// 2i + 1), then gated.  Without tables it is the gate alone.  float32 inside, one rounding; the
// output rows may be out_stride apart (a slice of a wider row).
template <typename T>
__global__ void rotate_gate_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ a,
                                   const T* __restrict__ g, long long g_stride, const float* __restrict__ cos_tab,
                                   const float* __restrict__ sin_tab, int table_len, int rotary_dim, int interleaved,
                                   const int* __restrict__ row_pos, long long n, int n_heads, int size, float scale,
                                   int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const int width = n_heads * size;
    const long long m = e / width;
    const int c = (int)(e - m * width), d = c % size;
    float v = to_f32<T>(a[e]);
    if (cos_tab != nullptr && d < rotary_dim) {
        const int pos = row_pos[m];
        if (pos >= table_len) {
            if (err) atomicOr(err, THN_ERR_POSITION_RANGE);
            return;
        }
        const int half = rotary_dim / 2;
        int i;
        long long partner;
        bool first;
        if (interleaved) {
            i = d >> 1; first = (d & 1) == 0; partner = first ? e + 1 : e - 1;
        } else {
            first = d < half; i = first ? d : d - half; partner = first ? e + half : e - half;
        }
        const float co = cos_tab[(size_t)pos * half + i], sn = sin_tab[(size_t)pos * half + i];
        const float other = to_f32<T>(a[partner]);
        v = first ? v * co + other * sn : v * co - other * sn;     // the turn by the negative angle
    }
    const float z = to_f32<T>(g[m * g_stride + c]);
    out[m * out_stride + c] = from_f32<T>(v / (1.0f + expf(-z)) * scale);
}

// The same for bfloat16 rows in the layout of halves, eight consecutive entries per thread (16-byte
// accesses): entries d .. d + 7 and their eight partners lie in one half each when half the
// rotated size is a multiple of eight.
__global__ void rotate_gate_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, long long out_stride,
                                            const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ g,
                                            long long g_stride, const float* __restrict__ cos_tab,
                                            const float* __restrict__ sin_tab, int table_len, int rotary_dim,
                                            const int* __restrict__ row_pos, int n_heads, int size, float scale,
                                            int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    const int width = n_heads * size;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= width) return;
    const long long m = blockIdx.y;
    const int d = c % size, half = rotary_dim / 2;
    const uint4 ra = *reinterpret_cast<const uint4*>(a + m * width + c);
    const uint4 rg = *reinterpret_cast<const uint4*>(g + m * g_stride + c);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&ra);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&rg);
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 x = __bfloat1622float2(a2[j]);
        v[2 * j] = x.x;
        v[2 * j + 1] = x.y;
    }
    if (cos_tab != nullptr && d < rotary_dim) {
        const int pos = row_pos[m];
        if (pos >= table_len) {
            if (err) atomicOr(err, THN_ERR_POSITION_RANGE);
            return;
        }
        const bool first = d < half;
        const int i = first ? d : d - half;
        const uint4 rp = *reinterpret_cast<const uint4*>(a + m * width + (first ? c + half : c - half));
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&rp);
        const float* co = cos_tab + (size_t)pos * half + i;
        const float* sn = sin_tab + (size_t)pos * half + i;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 other = __bfloat1622float2(p2[j]);
            v[2 * j] = first ? v[2 * j] * co[2 * j] + other.x * sn[2 * j] : v[2 * j] * co[2 * j] - other.x * sn[2 * j];
            v[2 * j + 1] = first ? v[2 * j + 1] * co[2 * j + 1] + other.y * sn[2 * j + 1]
                                 : v[2 * j + 1] * co[2 * j + 1] - other.y * sn[2 * j + 1];
        }
    }
    uint4 packed;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 z = __bfloat1622float2(g2[j]);
        ob[j] = __floats2bfloat162_rn(v[2 * j] / (1.0f + expf(-z.x)) * scale, v[2 * j + 1] / (1.0f + expf(-z.y)) * scale);
    }
    *reinterpret_cast<uint4*>(out + m * out_stride + c) = packed;
}

THN_API int thn_rotate_gate(void* out, long long out_stride, const void* a, const void* g, long long g_stride,
                            const float* cos_tab, const float* sin_tab, int table_len, int rotary_dim, int interleaved,
                            const int* row_pos, int n_rows, int n_heads, int size, float scale, int dtype, int* err,
                            cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && n_heads > 0 && size > 0 && g_stride >= (long long)n_heads * size &&
                      out_stride >= (long long)n_heads * size, "rotate_gate: bad sizes");
    THN_CHECK_ARG(cos_tab == nullptr || (sin_tab != nullptr && row_pos != nullptr && rotary_dim % 2 == 0 &&
                                         rotary_dim >= 0 && rotary_dim <= size),
                  "rotate_gate: the rotation needs tables, positions and an even size within %d", size);
    const long long n = (long long)n_rows * n_heads * size;
    if (n == 0) return THN_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    const bool turns = cos_tab != nullptr && rotary_dim > 0;
    if (dtype == THN_BF16 && size % 8 == 0 && out_stride % 8 == 0 && g_stride % 8 == 0 && n_rows <= 65535 &&
        (!turns || (!interleaved && (rotary_dim / 2) % 8 == 0)) &&
        ((((uintptr_t)out) | ((uintptr_t)a) | ((uintptr_t)g)) & 15) == 0) {
        const int width = n_heads * size;
        thn_launch(rotate_gate_bf16_vec_kernel, dim3((width / 8 + 127) / 128, n_rows), 128, 0, stream, (__nv_bfloat16*)out,
                   out_stride, (const __nv_bfloat16*)a, (const __nv_bfloat16*)g, g_stride, cos_tab, sin_tab, table_len,
                   turns ? rotary_dim : 0, row_pos, n_heads, size, scale, err);
        return thn_launch_status("rotate_gate");
    }
    if (dtype == THN_F32)
        thn_launch(rotate_gate_kernel<float>, blocks, 256, 0, stream, (float*)out, out_stride, (const float*)a,
                   (const float*)g, g_stride, cos_tab, sin_tab, table_len, rotary_dim, interleaved, row_pos, n, n_heads, size,
                   scale, err);
    else if (dtype == THN_BF16)
        thn_launch(rotate_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, out_stride,
                   (const __nv_bfloat16*)a, (const __nv_bfloat16*)g, g_stride, cos_tab, sin_tab, table_len, rotary_dim,
                   interleaved, row_pos, n, n_heads, size, scale, err);
    else
        THN_CHECK_ARG(false, "rotate_gate: unknown dtype %d", dtype);
    return thn_launch_status("rotate_gate");
}

// x[m, c] += bias[c] * scale in place (float32): the bias of a product of the 32-bit path.
__global__ void add_bias_f32_kernel(float* __restrict__ x, const float* __restrict__ bias, long long n, int width,
                                    float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e < n) x[e] += bias[e % width] * scale;
}

THN_API int thn_add_bias_f32(float* x, const float* bias, int n_rows, int width, float scale, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && width > 0, "add_bias: bad sizes");
    const long long n = (long long)n_rows * width;
    if (n == 0) return THN_OK;
    thn_launch(add_bias_f32_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, bias, n, width, scale);
    return thn_launch_status("add_bias");
}

// ------------------------------------------------------------------ RMSNorm

constexpr int kNormThreads = 256;
constexpr int kNormKeep = 16;   // values a thread keeps in registers between the two passes

// y = w * rnd(v * rstd), rstd = 1/sqrt(mean(v^2) + eps).  v = h, or with a branch output d:
// v = rnd(h + d), stored back to h first.  One block per row.
template <typename T, typename WT, bool ADD>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(T* __restrict__ y, T* __restrict__ h,
                                                               const T* __restrict__ d, const WT* __restrict__ w, int width,
                                                               float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * width;
    float keep[kNormKeep];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kNormKeep; ++j) {
        const int i = threadIdx.x + j * kNormThreads;
        float v = 0.f;
        if (i < width) {
            v = to_f32<T>(h[base + i]);
            if (ADD) {
                v = rnd<T>(v + to_f32<T>(d[base + i]));
                h[base + i] = from_f32<T>(v);
            }
        }
        keep[j] = v;
        ss += v * v;
    }
    for (int i = threadIdx.x + kNormKeep * kNormThreads; i < width; i += kNormThreads) {
        float v = to_f32<T>(h[base + i]);
        if (ADD) {
            v = rnd<T>(v + to_f32<T>(d[base + i]));
            h[base + i] = from_f32<T>(v);
        }
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
    for (int j = 0; j < kNormKeep; ++j) {
        const int i = threadIdx.x + j * kNormThreads;
        if (i < width) y[base + i] = from_f32<T>(to_f32<WT>(w[i]) * rnd<T>(keep[j] * rstd));
    }
    for (int i = threadIdx.x + kNormKeep * kNormThreads; i < width; i += kNormThreads) {
        const float v = to_f32<T>(h[base + i]);
        y[base + i] = from_f32<T>(to_f32<WT>(w[i]) * rnd<T>(v * rstd));
    }
}

// The common serving case, bfloat16 rows of up to 8192 values with width % 8 == 0: one
// 16-byte vector per thread, every load issued before the first use, same arithmetic and
// rounding as the kernel above.  blockDim depends on the width only.
template <typename WT, bool ADD>
__global__ void __launch_bounds__(1024) rmsnorm_bf16_vec_kernel(__nv_bfloat16* __restrict__ y,
                                                                __nv_bfloat16* __restrict__ h,
                                                                const __nv_bfloat16* __restrict__ d,
                                                                const WT* __restrict__ w, int width, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * width;
    const int i0 = threadIdx.x * 8;
    const bool live = i0 < width;
    uint4 hv = make_uint4(0, 0, 0, 0), dv = make_uint4(0, 0, 0, 0);
    float gain[8];
    if (live) {
        hv = *reinterpret_cast<const uint4*>(h + base + i0);
        if (ADD) dv = *reinterpret_cast<const uint4*>(d + base + i0);
        if (sizeof(WT) == 2) {
            const uint4 wv = *reinterpret_cast<const uint4*>(w + i0);
            const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(&wv);
#pragma unroll
            for (int j = 0; j < 8; ++j) gain[j] = __bfloat162float(wb[j]);
        } else {
            const float4 w0 = *reinterpret_cast<const float4*>(w + i0);
            const float4 w1 = *reinterpret_cast<const float4*>(w + i0 + 4);
            gain[0] = w0.x; gain[1] = w0.y; gain[2] = w0.z; gain[3] = w0.w;
            gain[4] = w1.x; gain[5] = w1.y; gain[6] = w1.z; gain[7] = w1.w;
        }
    }
    const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&hv);
    const __nv_bfloat16* db = reinterpret_cast<const __nv_bfloat16*>(&dv);
    float v[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        v[j] = __bfloat162float(hb[j]);
        if (ADD) v[j] = rnd<__nv_bfloat16>(v[j] + __bfloat162float(db[j]));
        ss += v[j] * v[j];
    }
    if (ADD && live) {
        uint4 out;
        __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&out);
#pragma unroll
        for (int j = 0; j < 8; ++j) ob[j] = __float2bfloat16_rn(v[j]);
        *reinterpret_cast<uint4*>(h + base + i0) = out;
    }
    const float total = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(total / (float)width + eps);
    if (live) {
        uint4 out;
        __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&out);
#pragma unroll
        for (int j = 0; j < 8; ++j) ob[j] = __float2bfloat16_rn(gain[j] * rnd<__nv_bfloat16>(v[j] * rstd));
        *reinterpret_cast<uint4*>(y + base + i0) = out;
    }
}

template <typename WT>
static bool launch_rmsnorm_vec(void* y, void* h, const void* d, const void* w, int rows,
                               int width, float eps, cudaStream_t stream) {
    if (width % 8 || width > 8192 || (((uintptr_t)y | (uintptr_t)h | (uintptr_t)d | (uintptr_t)w) & 15))
        return false;
    const int threads = ((width / 8 + 31) / 32) * 32;
    if (d)
        thn_launch(rmsnorm_bf16_vec_kernel<WT, true>, rows, threads, 0, stream, (__nv_bfloat16*)y, (__nv_bfloat16*)h, (const __nv_bfloat16*)d, (const WT*)w, width, eps);
    else
        thn_launch(rmsnorm_bf16_vec_kernel<WT, false>, rows, threads, 0, stream, (__nv_bfloat16*)y, (__nv_bfloat16*)h, nullptr, (const WT*)w, width, eps);
    return true;
}

template <typename T, typename WT>
static void launch_rmsnorm(void* y, void* h, const T* d, const void* w, int rows, int width, float eps,
                           cudaStream_t stream) {
    if (d)
        thn_launch(rmsnorm_kernel<T, WT, true>, rows, kNormThreads, 0, stream, (T*)y, (T*)h, d, (const WT*)w, width, eps);
    else
        thn_launch(rmsnorm_kernel<T, WT, false>, rows, kNormThreads, 0, stream, (T*)y, (T*)h, d, (const WT*)w, width, eps);
}

// y = RMSNorm(h).  With d (a tensor of h's type): h is updated in place to rnd(h + d) first.
THN_API int thn_rmsnorm(void* y, void* h, const void* d, const void* w, int rows, int width, float eps, int dtype,
                        int w_dtype, cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", rows, width);
    THN_CHECK_ARG(eps > 0.f, "rmsnorm: eps must be positive, got %g", (double)eps);
    if (rows == 0) return THN_OK;
    if (dtype == THN_F32 && w_dtype == THN_F32)
        launch_rmsnorm<float, float>(y, h, (const float*)d, w, rows, width, eps, stream);
    else if (dtype == THN_BF16 && w_dtype == THN_BF16 &&
             launch_rmsnorm_vec<__nv_bfloat16>(y, h, d, w, rows, width, eps, stream)) {
    } else if (dtype == THN_BF16 && w_dtype == THN_F32 && launch_rmsnorm_vec<float>(y, h, d, w, rows, width, eps, stream)) {
    } else if (dtype == THN_BF16 && w_dtype == THN_BF16)
        launch_rmsnorm<__nv_bfloat16, __nv_bfloat16>(y, h, (const __nv_bfloat16*)d, w, rows, width, eps, stream);
    else if (dtype == THN_BF16 && w_dtype == THN_F32)
        launch_rmsnorm<__nv_bfloat16, float>(y, h, (const __nv_bfloat16*)d, w, rows, width, eps, stream);
    else
        THN_CHECK_ARG(false, "rmsnorm: unsupported dtypes activation=%d gain=%d", dtype, w_dtype);
    return thn_launch_status("rmsnorm");
}

// ------------------------------------------------------------------ SwiGLU

// out[m, i] = rnd(rnd(g / (1 + exp(-g))) * u), g = gu[m, i], u = gu[m, inter + i].
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gu, long long total, int inter) {
    pdl_launch_dependents();
    pdl_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const long long m = e / inter;
        const int i = (int)(e - m * inter);
        const float g = to_f32<T>(gu[m * 2 * inter + i]);
        const float u = to_f32<T>(gu[m * 2 * inter + inter + i]);
        const float s = rnd<T>(g / (1.0f + expf(-g)));
        out[e] = from_f32<T>(s * u);
    }
}

// bfloat16 tensor input with inter % 8 == 0: eight values per thread, 16-byte accesses.
__global__ void swiglu_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu,
                                       long long total_vecs, int inter_vecs) {
    pdl_launch_dependents();
    pdl_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total_vecs; e += stride) {
        const long long m = e / inter_vecs;
        const int i = (int)(e - m * inter_vecs);
        const uint4 gv = *reinterpret_cast<const uint4*>(gu + (m * 2 * inter_vecs + i) * 8);
        const uint4 uv = *reinterpret_cast<const uint4*>(gu + (m * 2 * inter_vecs + inter_vecs + i) * 8);
        const __nv_bfloat16* gb = reinterpret_cast<const __nv_bfloat16*>(&gv);
        const __nv_bfloat16* ub = reinterpret_cast<const __nv_bfloat16*>(&uv);
        // silu in float32 with the fast exponential and reciprocal (a few float32 ulp, far below
        // the bfloat16 rounding that follows); the product of the two bfloat16 values with the
        // paired instruction, which rounds the exact product once as the reference's does.
        uint4 ov;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&ov);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(gb);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(ub);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]);
            const float s0 = __fdividef(g.x, 1.0f + __expf(-g.x)), s1 = __fdividef(g.y, 1.0f + __expf(-g.y));
            ob[j] = __hmul2(__floats2bfloat162_rn(s0, s1), u2[j]);
        }
        *reinterpret_cast<uint4*>(out + e * 8) = ov;
    }
}

// gu [rows, 2 * inter] (gate columns, then up columns) -> out [rows, inter].
THN_API int thn_swiglu(void* out, const void* gu, int rows, int inter, int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && inter > 0, "swiglu: bad sizes rows=%d inter=%d", rows, inter);
    const long long total = (long long)rows * inter;
    if (total == 0) return THN_OK;
    const int threads = 256;
    const long long want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == THN_BF16 && inter % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
        const long long vecs = total / 8;
        const long long want_vec = (vecs + threads - 1) / threads;
        thn_launch(swiglu_bf16_vec_kernel, (unsigned)(want_vec < 148 * 32 ? want_vec : 148 * 32), threads, 0, stream,
                   (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, vecs, inter / 8);
        return thn_launch_status("swiglu");
    }
    if (dtype == THN_F32)
        thn_launch(swiglu_kernel<float>, blocks, threads, 0, stream, (float*)out, (const float*)gu, total, inter);
    else if (dtype == THN_BF16)
        thn_launch(swiglu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)gu, total, inter);
    else
        THN_CHECK_ARG(false, "swiglu: unknown dtype %d", dtype);
    return thn_launch_status("swiglu");
}

// ------------------------------------------------------------------ clamped gated linear unit

// out[m, i] = g s(alpha g) (u + 1) with g = min(gu[m, i], limit), u = clamp(gu[m, inter + i], -limit, limit)
// and s the logistic function; float32 inside, rounded once.
template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ gu, long long total, int inter, float limit,
                                   float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const long long m = e / inter;
        const int i = (int)(e - m * inter);
        const float g = fminf(to_f32<T>(gu[m * 2 * inter + i]), limit);
        const float u = fminf(fmaxf(to_f32<T>(gu[m * 2 * inter + inter + i]), -limit), limit);
        out[e] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
    }
}

// bfloat16 with inter % 8 == 0: eight values per thread, 16-byte accesses, the same arithmetic.
__global__ void clamped_glu_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu,
                                            long long total_vecs, int inter_vecs, float limit, float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total_vecs; e += stride) {
        const long long m = e / inter_vecs;
        const int i = (int)(e - m * inter_vecs);
        const uint4 gv = *reinterpret_cast<const uint4*>(gu + (m * 2 * inter_vecs + i) * 8);
        const uint4 uv = *reinterpret_cast<const uint4*>(gu + (m * 2 * inter_vecs + inter_vecs + i) * 8);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 ov;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            const float g0 = fminf(g.x, limit), g1 = fminf(g.y, limit);
            const float u0 = fminf(fmaxf(u.x, -limit), limit), u1 = fminf(fmaxf(u.y, -limit), limit);
            ob[j] = __floats2bfloat162_rn(g0 / (1.0f + expf(-alpha * g0)) * (u0 + 1.0f),
                                          g1 / (1.0f + expf(-alpha * g1)) * (u1 + 1.0f));
        }
        *reinterpret_cast<uint4*>(out + e * 8) = ov;
    }
}

// gu [rows, 2 * inter] (gate columns, then up columns) -> out [rows, inter].
THN_API int thn_clamped_glu(void* out, const void* gu, int rows, int inter, float limit, float alpha, int dtype,
                            cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && inter > 0 && limit > 0.f, "clamped_glu: bad sizes rows=%d inter=%d limit=%g", rows, inter,
                  (double)limit);
    const long long total = (long long)rows * inter;
    if (total == 0) return THN_OK;
    const int threads = 256;
    const long long want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == THN_BF16 && inter % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
        const long long vecs = total / 8;
        const long long want_vec = (vecs + threads - 1) / threads;
        thn_launch(clamped_glu_bf16_vec_kernel, (unsigned)(want_vec < 148 * 32 ? want_vec : 148 * 32), threads, 0, stream,
                   (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, vecs, inter / 8, limit, alpha);
        return thn_launch_status("clamped_glu");
    }
    if (dtype == THN_F32)
        thn_launch(clamped_glu_kernel<float>, blocks, threads, 0, stream, (float*)out, (const float*)gu, total, inter,
                   limit, alpha);
    else if (dtype == THN_BF16)
        thn_launch(clamped_glu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)gu, total, inter, limit, alpha);
    else
        THN_CHECK_ARG(false, "clamped_glu: unknown dtype %d", dtype);
    return thn_launch_status("clamped_glu");
}

// out = a N(z) + b N(z^2) + c N(z^3) + e per row, powers taken entry by entry and
// N(v) = v / sqrt(mean(v^2) + eps) over the row; (a, b, c, e) = coef[0..3].  One block per row,
// the row staged in shared memory; the three sums of squares are float32 and their order depends
// on the block size only; one rounding at the store.
// Three sums over a block at once; every thread gets all three.  The order of additions depends
// only on blockDim.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float (*scratch)[33]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    c = warp_sum(c);
    if (lane == 0) {
        scratch[0][warp] = a;
        scratch[1][warp] = b;
        scratch[2][warp] = c;
    }
    __syncthreads();
    if (warp < 3) {
        const int n_warps = (blockDim.x + 31) >> 5;
        float t = lane < n_warps ? scratch[warp][lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[warp][32] = t;
    }
    __syncthreads();
    a = scratch[0][32];
    b = scratch[1][32];
    c = scratch[2][32];
}

template <typename T>
__global__ void __launch_bounds__(256) polynorm_kernel(T* __restrict__ out, const T* __restrict__ z,
                                                       const float* __restrict__ coef, int width, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float poly_row[];
    __shared__ float scratch[3][33];
    const size_t base = (size_t)blockIdx.x * width;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = to_f32<T>(z[base + i]);
        poly_row[i] = v;
        const float v2 = v * v;
        s1 += v2;
        s2 += v2 * v2;
        s3 += v2 * v2 * v2;
    }
    block_sum3(s1, s2, s3, scratch);
    const float n = (float)width;
    const float r1 = coef[0] / sqrtf(s1 / n + eps);
    const float r2 = coef[1] / sqrtf(s2 / n + eps);
    const float r3 = coef[2] / sqrtf(s3 / n + eps);
    const float shift = coef[3];
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = poly_row[i];
        out[base + i] = from_f32<T>(v * (r1 + v * (r2 + v * r3)) + shift);
    }
}

// The same for bfloat16 rows of a multiple of eight values at 16-byte aligned addresses: 16-byte
// accesses, the row staged as it was read.
template <int THREADS>
__global__ void __launch_bounds__(THREADS) polynorm_bf16x8_kernel(__nv_bfloat16* __restrict__ out,
                                                                  const __nv_bfloat16* __restrict__ z,
                                                                  const float* __restrict__ coef, int vecs, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ uint4 poly_vecs[];
    __shared__ float scratch[3][33];
    const uint4* src = reinterpret_cast<const uint4*>(z) + (size_t)blockIdx.x * vecs;
    uint4* dst = reinterpret_cast<uint4*>(out) + (size_t)blockIdx.x * vecs;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x; i < vecs; i += THREADS) {
        const uint4 raw = src[i];
        poly_vecs[i] = raw;
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 v = __bfloat1622float2(pairs[k]);
            const float a = v.x * v.x, b = v.y * v.y;
            s1 += a;
            s2 += a * a;
            s3 += a * a * a;
            s1 += b;
            s2 += b * b;
            s3 += b * b * b;
        }
    }
    block_sum3(s1, s2, s3, scratch);
    const float n = 8.f * (float)vecs;
    const float r1 = coef[0] / sqrtf(s1 / n + eps);
    const float r2 = coef[1] / sqrtf(s2 / n + eps);
    const float r3 = coef[2] / sqrtf(s3 / n + eps);
    const float shift = coef[3];
    for (int i = threadIdx.x; i < vecs; i += THREADS) {
        const uint4 raw = poly_vecs[i];
        const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
        uint4 res;
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 v = __bfloat1622float2(pairs[k]);
            o[k] = __floats2bfloat162_rn(v.x * (r1 + v.x * (r2 + v.x * r3)) + shift,
                                         v.y * (r1 + v.y * (r2 + v.y * r3)) + shift);
        }
        dst[i] = res;
    }
}

// z, out [rows, width] of the activation type; coef float32 [4].
THN_API int thn_polynorm(void* out, const void* z, const float* coef, int rows, int width, float eps, int dtype,
                         cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && width > 0 && eps > 0.f && coef != nullptr, "polynorm: bad sizes rows=%d width=%d", rows, width);
    if (rows == 0) return THN_OK;
    const size_t smem = (size_t)width * sizeof(float);
    THN_UNSUPPORTED_IF(smem > 200 * 1024, "polynorm: rows of %d values do not fit shared memory", width);
    if (dtype == THN_F32) {
        if (smem > 32 * 1024) cudaFuncSetAttribute(polynorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        thn_launch(polynorm_kernel<float>, rows, 256, smem, stream, (float*)out, (const float*)z, coef, width, eps);
    } else if (dtype == THN_BF16) {
        const bool aligned = width % 8 == 0 && ((uintptr_t)out | (uintptr_t)z) % 16 == 0;
        if (aligned && width >= 8192) {          // the choice depends on the row's size only
            const size_t staged = (size_t)width * sizeof(__nv_bfloat16);
            if (staged > 32 * 1024)
                cudaFuncSetAttribute(polynorm_bf16x8_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staged);
            thn_launch(polynorm_bf16x8_kernel<512>, rows, 512, staged, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)z,
                       coef, width / 8, eps);
        } else if (aligned) {
            thn_launch(polynorm_bf16x8_kernel<256>, rows, 256, (size_t)width * sizeof(__nv_bfloat16), stream,
                       (__nv_bfloat16*)out, (const __nv_bfloat16*)z, coef, width / 8, eps);
        } else {
            if (smem > 32 * 1024)
                cudaFuncSetAttribute(polynorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            thn_launch(polynorm_kernel<__nv_bfloat16>, rows, 256, smem, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)z,
                       coef, width, eps);
        }
    } else {
        THN_CHECK_ARG(false, "polynorm: unknown dtype %d", dtype);
    }
    return thn_launch_status("polynorm");
}

// ------------------------------------------------------------------ step bookkeeping

// Row m of a packed step belongs to sequence b with cu[b] <= m < cu[b+1]; its slot is
// slots[b] and its absolute position is seq_lens[slot] + (m - cu[b]).
__global__ void step_rows_kernel(int* __restrict__ row_slot, int* __restrict__ row_pos,
                                 const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                 const int* __restrict__ seq_lens, int n_seqs) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;
    if (b >= n_seqs) return;
    const int r0 = cu_seqlens[b], r1 = cu_seqlens[b + 1];
    const int slot = slots[b];
    const int start = seq_lens[slot];
    for (int r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
        row_slot[r] = slot;
        row_pos[r] = start + (r - r0);
    }
}

THN_API int thn_step_rows(int* row_slot, int* row_pos, const int* cu_seqlens, const int* slots, const int* seq_lens,
                          int n_seqs, cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0, "step_rows: bad batch %d", n_seqs);
    if (n_seqs == 0) return THN_OK;
    thn_launch(step_rows_kernel, n_seqs, 128, 0, stream, row_slot, row_pos, cu_seqlens, slots, seq_lens, n_seqs);
    return thn_launch_status("step_rows");
}

// seq_lens[slots[b]] += cu[b+1] - cu[b]: the step's tokens are now part of the sequences.
__global__ void advance_kernel(int* __restrict__ seq_lens, const int* __restrict__ slots,
                               const int* __restrict__ cu_seqlens, int n_seqs) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < n_seqs) seq_lens[slots[b]] += cu_seqlens[b + 1] - cu_seqlens[b];
}

THN_API int thn_advance(int* seq_lens, const int* slots, const int* cu_seqlens, int n_seqs, cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0, "advance: bad batch %d", n_seqs);
    if (n_seqs == 0) return THN_OK;
    thn_launch(advance_kernel, (n_seqs + 127) / 128, 128, 0, stream, seq_lens, slots, cu_seqlens, n_seqs);
    return thn_launch_status("advance");
}

// ------------------------------------------------------------------ rotary table

// cos/sin of angle = position * inv_freq[i], all float32 (engine/engine.py:238-247).
__global__ void rope_table_kernel(float* __restrict__ cos_out, float* __restrict__ sin_out,
                                  const float* __restrict__ inv_freq, int first, int n_positions, int half) {
    pdl_launch_dependents();
    pdl_wait();
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (long long)n_positions * half) return;
    const int p = (int)(e / half), i = (int)(e - (long long)p * half);
    const float angle = (float)(first + p) * inv_freq[i];
    cos_out[(size_t)(first + p) * half + i] = cosf(angle);
    sin_out[(size_t)(first + p) * half + i] = sinf(angle);
}

// Fills rows [first, first + n_positions) of tables [*, half].
THN_API int thn_rope_table(float* cos_out, float* sin_out, const float* inv_freq, int first, int n_positions,
                           int half, cudaStream_t stream) {
    THN_CHECK_ARG(first >= 0 && n_positions >= 0 && half > 0, "rope_table: bad sizes");
    const long long total = (long long)n_positions * half;
    if (total == 0) return THN_OK;
    thn_launch(rope_table_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, cos_out, sin_out, inv_freq, first,
                                                                           n_positions, half);
    return thn_launch_status("rope_table");
}

// ------------------------------------------------------------------ int32 scatter and gather

// dst[index[i]] = value[i]: block-table cells and per-sequence counters changed by the host.
__global__ void scatter_i32_kernel(int* __restrict__ dst, const long long* __restrict__ index,
                                   const int* __restrict__ value, int n, long long dst_size) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && index[i] >= 0 && index[i] < dst_size) dst[index[i]] = value[i];
}

THN_API int thn_scatter_i32(int* dst, const long long* index, const int* value, int n, long long dst_size,
                            cudaStream_t stream) {
    THN_CHECK_ARG(n >= 0 && dst_size >= 0, "scatter_i32: bad sizes");
    if (n == 0) return THN_OK;
    thn_launch(scatter_i32_kernel, (n + 127) / 128, 128, 0, stream, dst, index, value, n, dst_size);
    return thn_launch_status("scatter_i32");
}

// out[i] = src[index[i]]: the tokens that the sequences of a decode step feed next.
__global__ void gather_i32_kernel(int* __restrict__ out, const int* __restrict__ src, const int* __restrict__ index,
                                  int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = src[index[i]];
}

THN_API int thn_gather_i32(int* out, const int* src, const int* index, int n, cudaStream_t stream) {
    THN_CHECK_ARG(n >= 0, "gather_i32: bad size %d", n);
    if (n == 0) return THN_OK;
    thn_launch(gather_i32_kernel, (n + 127) / 128, 128, 0, stream, out, src, index, n);
    return thn_launch_status("gather_i32");
}
