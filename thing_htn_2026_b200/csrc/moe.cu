// Routing of a mixture of experts, and the experts' activation with the routing weights.
//
//   moe_route   per row: scores s = softmax(z) over all experts (scoring 0) or s = logistic(z),
//               each expert by itself (scoring 1); the experts form `groups` equal
//               groups of neighbours, a group's score is its largest s, and only experts of the
//               `keep` best groups can be chosen; the `top` allowed experts with the largest s
//               are chosen (the lower index wins a tie); a chosen expert's weight is s * scale,
//               not renormalised.  Writes the weights as a dense row [experts] (0 where not
//               chosen) and as lists chosen [top], chosen_weight [top].  float32 throughout.
//   routed_gelu the up-projections of all experts side by side, [experts * ff | shared_ff] per
//               row: out = gelu(u) * weight of the column's expert, and for the shared expert's
//               columns gelu(u) * logistic(gate logit of the row).  gelu is the exact one,
//               0.5 u (1 + erf(u / sqrt 2)).  An expert that was not chosen gets zeros, so one
//               down-projection over all columns gives the weighted sum of the chosen experts'
//               outputs plus the gated shared expert's.
//   routed_clamped_glu   experts of the form down(g * logistic(a g) * (u + 1)) with
//               g = min(gate(x'), limit), u = clamp(up(x'), -limit, limit), whose input is the
//               token times its routing weight, x' = w x.  The gate and up projections of all
//               experts and of the shared expert are one product over x; a projection is linear,
//               so the kernel multiplies the projected values by w (float32) before the clamps.
//               A row holds [gates of all columns | ups of all columns]; the columns are
//               [experts * ff | shared_ff].  The shared expert sees the token itself, has a limit
//               of its own, and its columns are multiplied by logistic(gate logit of the row).
//               With weight_output the routing weight multiplies the expert's activation instead
//               (the expert sees the token itself and its output is weighted).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kRouteWarps = 4;

struct Best {
    float value;
    int index;
};

__device__ __forceinline__ Best warp_best(Best b) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, b.value, o);
        const int i = __shfl_xor_sync(0xffffffffu, b.index, o);
        if (v > b.value || (v == b.value && i < b.index)) { b.value = v; b.index = i; }
    }
    return b;
}

__global__ void __launch_bounds__(kRouteWarps * 32) moe_route_kernel(
    float* __restrict__ dense, int* __restrict__ chosen, float* __restrict__ chosen_weight, const float* __restrict__ z,
    long long z_stride, int n_rows, int n_experts, int n_groups, int keep, int top, float scale, int scoring,
    int renormalise, float renorm_eps) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float shared[];     // per warp: scores [experts], group scores [groups]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * kRouteWarps + warp;
    if (row >= n_rows) return;
    float* s = shared + (size_t)warp * (n_experts + n_groups);
    float* group_score = s + n_experts;
    const float* zr = z + (size_t)row * z_stride;
    const int per = n_experts / n_groups;

    if (scoring == 1 && keep >= n_groups) {
        // Logistic scores of experts that are all eligible: the order of the scores is the order
        // of the logits, and the logits do not saturate, so the choice is made on them.
        for (int e = lane; e < n_experts; e += 32) {
            s[e] = zr[e];
            dense[(size_t)row * n_experts + e] = 0.f;
        }
        __syncwarp();
        for (int pick = 0; pick < top; ++pick) {
            Best b{-INFINITY, 0x7fffffff};
            for (int e = lane; e < n_experts; e += 32)
                if (s[e] > b.value || (s[e] == b.value && e < b.index)) { b.value = s[e]; b.index = e; }
            b = warp_best(b);
            __syncwarp();
            if (lane == 0) {
                if (b.index < n_experts) {
                    const float w = scale / (1.0f + expf(-b.value));
                    dense[(size_t)row * n_experts + b.index] = w;
                    chosen[(size_t)row * top + pick] = b.index;
                    chosen_weight[(size_t)row * top + pick] = w;
                    s[b.index] = -INFINITY;       // taken
                } else {                      // no logit compares (not a number): an index that exists, no weight
                    chosen[(size_t)row * top + pick] = pick;
                    chosen_weight[(size_t)row * top + pick] = 0.f;
                }
            }
            __syncwarp();
        }
        return;
    }
    if (scoring == 1) {
        for (int e = lane; e < n_experts; e += 32) {
            s[e] = 1.0f / (1.0f + expf(-zr[e]));
            dense[(size_t)row * n_experts + e] = 0.f;
        }
    } else {
        float mx = -INFINITY;
        for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, zr[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = expf(zr[e] - mx);
            s[e] = v;
            sum += v;
        }
        sum = warp_sum(sum);
        for (int e = lane; e < n_experts; e += 32) {
            s[e] = s[e] / sum;
            dense[(size_t)row * n_experts + e] = 0.f;
        }
    }
    __syncwarp();
    for (int g = lane; g < n_groups; g += 32) {
        float best = -1.f;
        for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, s[e]);
        group_score[g] = best;
    }
    __syncwarp();
    // the `keep` best groups stay as they are; the scores of the others are hidden behind a sign
    if (keep < n_groups) {
        for (int pick = 0; pick < keep; ++pick) {
            Best b{-1.f, 0x7fffffff};
            for (int g = lane; g < n_groups; g += 32)
                if (group_score[g] > b.value) { b.value = group_score[g]; b.index = g; }
            b = warp_best(b);
            __syncwarp();
            if (lane == 0) group_score[b.index] = -2.f;      // taken
            __syncwarp();
        }
        for (int e = lane; e < n_experts; e += 32)
            if (group_score[e / per] != -2.f) s[e] = -1.f - s[e];      // not allowed; the score is kept, negative
        __syncwarp();
    }
    for (int pick = 0; pick < top; ++pick) {
        Best b{-1.f, 0x7fffffff};
        for (int e = lane; e < n_experts; e += 32)
            if (s[e] > b.value) { b.value = s[e]; b.index = e; }
        b = warp_best(b);
        __syncwarp();
        if (lane == 0) {
            const float w = b.value * scale;
            dense[(size_t)row * n_experts + b.index] = w;
            chosen[(size_t)row * top + pick] = b.index;
            chosen_weight[(size_t)row * top + pick] = w;
            s[b.index] = -4.f;       // taken
        }
        __syncwarp();
    }
    if (renormalise && lane == 0) {
        // the chosen experts' weights divided by their sum (+ renorm_eps), summed in the order chosen
        float sum = 0.f;
        for (int pick = 0; pick < top; ++pick) sum += chosen_weight[(size_t)row * top + pick];
        const float r = scale / (sum / scale + renorm_eps);
        for (int pick = 0; pick < top; ++pick) {
            const float w = chosen_weight[(size_t)row * top + pick] / scale * r;
            chosen_weight[(size_t)row * top + pick] = w;
            dense[(size_t)row * n_experts + chosen[(size_t)row * top + pick]] = w;
        }
    }
}

__device__ __forceinline__ float gelu_exact(float u) { return 0.5f * u * (1.0f + erff(u * 0.70710678118654752f)); }

template <typename T>
__global__ void routed_gelu_kernel(T* __restrict__ out, const T* __restrict__ u, const float* __restrict__ dense,
                                   const float* __restrict__ shared_logit, long long logit_stride, long long n, int width,
                                   int n_experts, int ff) {
    pdl_launch_dependents();
    pdl_wait();
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const long long row = e / width;
    const int c = (int)(e - row * width);
    float w;
    if (c < n_experts * ff) {
        w = dense[row * n_experts + c / ff];
        if (w == 0.f) { out[e] = from_f32<T>(0.f); return; }
    } else {
        w = shared_logit ? 1.0f / (1.0f + expf(-shared_logit[row * logit_stride])) : 1.0f;
    }
    out[e] = from_f32<T>(gelu_exact(to_f32<T>(u[e])) * w);
}

// The same, eight bfloat16 columns per thread (16-byte accesses), one row per blockIdx.y: for
// sizes where no group of eight columns straddles two experts.  The columns of an expert that
// was not chosen are not read.
__global__ void routed_gelu_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ u,
                                            const float* __restrict__ dense, const float* __restrict__ shared_logit,
                                            long long logit_stride, int width, int n_experts, int ff) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= width) return;
    const long long row = blockIdx.y;
    float w;
    if (c < n_experts * ff) w = dense[row * n_experts + c / ff];
    else w = shared_logit ? 1.0f / (1.0f + expf(-shared_logit[row * logit_stride])) : 1.0f;
    uint4 packed = make_uint4(0, 0, 0, 0);
    if (w != 0.f) {
        const uint4 raw = *reinterpret_cast<const uint4*>(u + row * width + c);
        const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t res[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in[i]));
            const __nv_bfloat162 r = __floats2bfloat162_rn(gelu_exact(v.x) * w, gelu_exact(v.y) * w);
            res[i] = *reinterpret_cast<const uint32_t*>(&r);
        }
        packed = make_uint4(res[0], res[1], res[2], res[3]);
    }
    *reinterpret_cast<uint4*>(out + row * width + c) = packed;
}

// One thread per column of a row; see the head of the file.  A column of an expert that was not
// chosen (weight 0) is not read.
template <typename T>
__global__ void routed_clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ gu, const float* __restrict__ dense,
                                          const float* __restrict__ shared_logit, long long logit_stride, long long n,
                                          int width, int n_experts, int ff, float limit, float shared_limit, float alpha,
                                          int weight_output) {
    pdl_launch_dependents();
    pdl_wait();
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const long long row = e / width;
    const int c = (int)(e - row * width);
    float w = 1.0f, lim = shared_limit, after = 1.0f;
    if (c < n_experts * ff) {
        w = dense[row * n_experts + c / ff];
        lim = limit;
        if (w == 0.f) { out[e] = from_f32<T>(0.f); return; }
        if (weight_output) { after = w; w = 1.0f; }
    } else if (shared_logit) {
        after = 1.0f / (1.0f + expf(-shared_logit[row * logit_stride]));
    }
    const T* src = gu + row * 2 * width;
    const float g = fminf(w * to_f32<T>(src[c]), lim);
    const float u = fminf(fmaxf(w * to_f32<T>(src[width + c]), -lim), lim);
    out[e] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f) * after);
}

// The same, eight bfloat16 columns per thread (16-byte accesses), one row per blockIdx.y: for
// sizes where no group of eight columns straddles two experts.
__global__ void routed_clamped_glu_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu,
                                                   const float* __restrict__ dense, const float* __restrict__ shared_logit,
                                                   long long logit_stride, int width, int n_experts, int ff, float limit,
                                                   float shared_limit, float alpha, int weight_output) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= width) return;
    const long long row = blockIdx.y;
    float w = 1.0f, lim = shared_limit, after = 1.0f;
    if (c < n_experts * ff) {
        w = dense[row * n_experts + c / ff];
        lim = limit;
    } else if (shared_logit) {
        after = 1.0f / (1.0f + expf(-shared_logit[row * logit_stride]));
    }
    uint4 packed = make_uint4(0, 0, 0, 0);
    if (w != 0.f) {
        if (weight_output && c < n_experts * ff) { after = w; w = 1.0f; }
        const uint4 gv = *reinterpret_cast<const uint4*>(gu + row * 2 * width + c);
        const uint4 uv = *reinterpret_cast<const uint4*>(gu + row * 2 * width + width + c);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            const float g0 = fminf(w * g.x, lim), g1 = fminf(w * g.y, lim);
            const float u0 = fminf(fmaxf(w * u.x, -lim), lim), u1 = fminf(fmaxf(w * u.y, -lim), lim);
            ob[j] = __floats2bfloat162_rn(g0 / (1.0f + expf(-alpha * g0)) * (u0 + 1.0f) * after,
                                          g1 / (1.0f + expf(-alpha * g1)) * (u1 + 1.0f) * after);
        }
    }
    *reinterpret_cast<uint4*>(out + row * width + c) = packed;
}

}  // namespace

// z float32 [rows, >= experts] with rows z_stride apart; dense float32 [rows, experts]; chosen
// int32 and chosen_weight float32 [rows, top].
THN_API int thn_moe_route(float* dense, int* chosen, float* chosen_weight, const float* z, long long z_stride, int n_rows,
                          int n_experts, int n_groups, int keep, int top, float scale, int scoring, int renormalise,
                          float renorm_eps, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && n_experts > 0 && n_groups > 0 && n_experts % n_groups == 0,
                  "moe_route: %d experts in %d groups", n_experts, n_groups);
    THN_CHECK_ARG(scoring == 0 || scoring == 1, "moe_route: scoring %d (0: softmax, 1: logistic)", scoring);
    THN_CHECK_ARG(!renormalise || (scoring == 0 && scale != 0.f), "moe_route: weights are renormalised with softmax scores only");
    THN_CHECK_ARG(keep > 0 && keep <= n_groups && top > 0 && top <= keep * (n_experts / n_groups),
                  "moe_route: top %d of the experts of %d groups out of %d", top, keep, n_groups);
    THN_UNSUPPORTED_IF(n_experts > 4096, "moe_route: %d experts, at most 4096", n_experts);
    if (n_rows == 0) return THN_OK;
    const size_t smem = (size_t)kRouteWarps * (n_experts + n_groups) * sizeof(float);
    if (smem > 32 * 1024)
        cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    thn_launch(moe_route_kernel, (n_rows + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, smem, stream, dense, chosen,
               chosen_weight, z, z_stride, n_rows, n_experts, n_groups, keep, top, scale, scoring, renormalise, renorm_eps);
    return thn_launch_status("moe_route");
}

// u, out [rows, experts * ff + shared_ff] of the activation type; dense float32 [rows, experts];
// shared_logit: the rows' gate logits of the shared expert, logit_stride apart (null: no gate).
THN_API int thn_routed_gelu(void* out, const void* u, const float* dense, const float* shared_logit, long long logit_stride,
                            int n_rows, int n_experts, int ff, int shared_ff, int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && n_experts >= 0 && ff >= 0 && shared_ff >= 0 && n_experts * ff + shared_ff > 0,
                  "routed_gelu: bad sizes");
    const int width = n_experts * ff + shared_ff;
    const long long n = (long long)n_rows * width;
    if (n == 0) return THN_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == THN_BF16 && ff % 8 == 0 && width % 8 == 0 && n_rows <= 65535 &&
        ((((uintptr_t)out) | ((uintptr_t)u)) & 15) == 0) {
        thn_launch(routed_gelu_bf16_vec_kernel, dim3((width / 8 + 127) / 128, n_rows), 128, 0, stream, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)u, dense, shared_logit, logit_stride, width, n_experts, ff);
        return thn_launch_status("routed_gelu");
    }
    if (dtype == THN_F32)
        thn_launch(routed_gelu_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)u, dense, shared_logit,
                   logit_stride, n, width, n_experts, ff);
    else if (dtype == THN_BF16)
        thn_launch(routed_gelu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)u,
                   dense, shared_logit, logit_stride, n, width, n_experts, ff);
    else
        THN_CHECK_ARG(false, "routed_gelu: unknown dtype %d", dtype);
    return thn_launch_status("routed_gelu");
}

// gu [rows, 2 * (experts * ff + shared_ff)] of the activation type: the gates of all columns, then
// the ups; out [rows, experts * ff + shared_ff]; dense float32 [rows, experts]; shared_logit: the
// rows' gate logits of the shared expert, logit_stride apart (null: no gate).
THN_API int thn_routed_clamped_glu(void* out, const void* gu, const float* dense, const float* shared_logit,
                                   long long logit_stride, int n_rows, int n_experts, int ff, int shared_ff, float limit,
                                   float shared_limit, float alpha, int weight_output, int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && n_experts >= 0 && ff >= 0 && shared_ff >= 0 && n_experts * ff + shared_ff > 0,
                  "routed_clamped_glu: bad sizes");
    THN_CHECK_ARG((n_experts * ff == 0 || limit > 0.f) && (shared_ff == 0 || shared_limit > 0.f),
                  "routed_clamped_glu: limits must be positive");
    const int width = n_experts * ff + shared_ff;
    const long long n = (long long)n_rows * width;
    if (n == 0) return THN_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == THN_BF16 && ff % 8 == 0 && width % 8 == 0 && n_rows <= 65535 &&
        ((((uintptr_t)out) | ((uintptr_t)gu)) & 15) == 0) {
        thn_launch(routed_clamped_glu_bf16_vec_kernel, dim3((width / 8 + 127) / 128, n_rows), 128, 0, stream,
                   (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, dense, shared_logit, logit_stride, width, n_experts, ff,
                   limit, shared_limit, alpha, weight_output);
        return thn_launch_status("routed_clamped_glu");
    }
    if (dtype == THN_F32)
        thn_launch(routed_clamped_glu_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)gu, dense,
                   shared_logit, logit_stride, n, width, n_experts, ff, limit, shared_limit, alpha, weight_output);
    else if (dtype == THN_BF16)
        thn_launch(routed_clamped_glu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)gu, dense, shared_logit, logit_stride, n, width, n_experts, ff, limit, shared_limit,
                   alpha, weight_output);
    else
        THN_CHECK_ARG(false, "routed_clamped_glu: unknown dtype %d", dtype);
    return thn_launch_status("routed_clamped_glu");
}
