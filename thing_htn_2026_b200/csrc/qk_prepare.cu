// From a step's projected rows to queries and cache entries, for attention variants that the
// per-head kernel of rope_cache.cu does not cover.  One block per row; everything between
// the load and the one rounding at the store is float32.
//
//   norm scope   0: none.  1: RMS norm per head, gains [head_dim] shared by the heads.
//                2: RMS norm over the whole projection at once (all heads of q, all heads of
//                   k), gains [n_q * head_dim] and [n_kv * head_dim].
//   rotation     the first rotary_dim entries of every head, by the row's position; layout
//                0: entry i is paired with entry i + rotary_dim / 2 (rotate-half);
//                1: entry 2i is paired with entry 2i + 1 (interleaved).
//                The pair (a, b) with angle t becomes (a cos t - b sin t, b cos t + a sin t).
//   values       0: the row brings values of its own, [q | k | v] (a value may have a size of its
//                   own, value_dim);
//                1: the values are the keys as projected, before norm and rotation, [q | k].
//   value rotation   with tables of their own (v_rotary_dim entries of every value, in the layout of
//                the keys' rotation) the values of the row are turned by its position before they
//                go to the cache; a reader turns its output back by its own position.
#include "common.cuh"

namespace {

// Two sums over a block at once; every thread gets both.  The order of additions depends on
// the block size only.
template <int THREADS>
__device__ __forceinline__ float2 block_sum2(float a, float b, float* scratch /* >= 66 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) { scratch[warp] = a; scratch[32 + warp] = b; }
    __syncthreads();
    if (warp == 0) {
        float ta = lane < THREADS / 32 ? scratch[lane] : 0.f, tb = lane < THREADS / 32 ? scratch[32 + lane] : 0.f;
        ta = warp_sum(ta);
        tb = warp_sum(tb);
        if (lane == 0) { scratch[64] = ta; scratch[65] = tb; }
    }
    __syncthreads();
    return make_float2(scratch[64], scratch[65]);
}

template <typename T> struct Pair;
template <> struct Pair<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
    static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct Pair<__nv_bfloat16> {
    static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
    }
};

// One block of THREADS per row.  A thread takes pairs of adjacent entries (2j, 2j + 1): head
// sizes are even here (the launcher sends odd ones to the scalar kernel below), so a pair never
// straddles two heads, an interleaved rotation has both partners in one thread, and every
// access is 4 or 8 bytes wide.  Pass 1 stages the row in shared memory and sums the squares
// (and copies the values to the cache); pass 2 normalises, rotates and stores.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS) qk_prepare_kernel(
    T* __restrict__ q_out, const T* __restrict__ proj, int proj_width, const float* __restrict__ q_gain,
    const float* __restrict__ k_gain, int norm_scope, float gain_offset, float eps, const float* __restrict__ cos_tab,
    const float* __restrict__ sin_tab, int table_len, int rotary_dim, int interleaved, int values_are_keys,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, PagedKV kv, int n_q, int write_cache,
    int half_d_shift, const float* __restrict__ v_cos, const float* __restrict__ v_sin, int v_table_len, int v_rotary_dim,
    int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(8) float vals[];   // [(n_q + n_kv) * D] raw values; then [n_q + n_kv] scales per head
    __shared__ float scratch[66];
    const int m = blockIdx.x;
    const int D = kv.head_dim, half_d = D >> 1;
    const int nq = n_q * D, nk = kv.n_kv * D, total = nq + nk, n_heads = n_q + kv.n_kv;
    float* head_scale = vals + total;
    const T* src = proj + (size_t)m * proj_width;
    const int pos = row_pos[m];
    int page = -1;
    if (write_cache) {
        page = kv.block_table[(size_t)row_slot[m] * kv.bt_stride + pos / kv.page_size];
        if (page < 0) {
            if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
            write_cache = 0;
        }
    }
    const int in_page = pos % kv.page_size;
    auto head_of = [&](int pair) { return half_d_shift >= 0 ? pair >> half_d_shift : pair / half_d; };

    float ss_q = 0.f, ss_k = 0.f;
    for (int pair = threadIdx.x; pair < total / 2; pair += THREADS) {
        const int e = 2 * pair;
        const float2 v = Pair<T>::load(src + e);
        *reinterpret_cast<float2*>(vals + e) = v;
        const float sq = v.x * v.x + v.y * v.y;
        if (e < nq) ss_q += sq; else ss_k += sq;
        if (write_cache && (values_are_keys ? e >= nq : false)) {     // the keys as projected are the values
            const int kvh = head_of(pair) - n_q, d = e - nq - kvh * D;
            Pair<T>::store((T*)kv.base + kv_offset_sized(kv, page, 1, kvh, in_page) + d, v.x, v.y);
        }
    }
    if (write_cache && !values_are_keys) {
        const int DV = kv.value_dim > 0 ? kv.value_dim : D;
        const bool turn = v_cos != nullptr && v_rotary_dim > 0;
        if (turn && pos >= v_table_len) {
            if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_POSITION_RANGE);
        } else {
            const int v_half = v_rotary_dim / 2;
            for (int pair = threadIdx.x; pair < kv.n_kv * DV / 2; pair += THREADS) {
                const int e = 2 * pair, kvh = e / DV, d = e - kvh * DV;
                float2 v = Pair<T>::load(src + total + e);
                if (turn && d < v_rotary_dim) {
                    const float* c_row = v_cos + (size_t)pos * v_half;
                    const float* s_row = v_sin + (size_t)pos * v_half;
                    if (interleaved) {
                        const float c = c_row[d >> 1], sn = s_row[d >> 1];
                        v = make_float2(v.x * c - v.y * sn, v.y * c + v.x * sn);
                    } else {
                        // d and d + 1 lie in the same half (the launcher sends an odd half to the scalar kernel)
                        const bool first = d < v_half;
                        const int i = first ? d : d - v_half;
                        const float2 o = Pair<T>::load(src + total + (first ? e + v_half : e - v_half));
                        v = first ? make_float2(v.x * c_row[i] - o.x * s_row[i], v.y * c_row[i + 1] - o.y * s_row[i + 1])
                                  : make_float2(v.x * c_row[i] + o.x * s_row[i], v.y * c_row[i + 1] + o.y * s_row[i + 1]);
                    }
                }
                Pair<T>::store((T*)kv.base + kv_offset_sized(kv, page, 1, kvh, in_page) + d, v.x, v.y);
            }
        }
    }
    float rq = 1.f, rk = 1.f;
    if (norm_scope == 2) {
        const float2 t = block_sum2<THREADS>(ss_q, ss_k, scratch);
        rq = 1.0f / sqrtf(t.x / (float)nq + eps);
        rk = 1.0f / sqrtf(t.y / (float)nk + eps);
    } else {
        __syncthreads();
        if (norm_scope == 1) {
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            for (int head = warp; head < n_heads; head += THREADS / 32) {
                float ss = 0.f;
                for (int d = lane; d < D; d += 32) ss += vals[head * D + d] * vals[head * D + d];
                ss = warp_sum(ss);
                if (lane == 0) head_scale[head] = 1.0f / sqrtf(ss / (float)D + eps);
            }
            __syncthreads();
        }
    }
    const bool rotate = cos_tab != nullptr && rotary_dim > 0;
    if (rotate && pos >= table_len) {
        if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_POSITION_RANGE);
        return;
    }
    const int half = rotary_dim / 2;
    // the normalised value of entry e of the row (head, entry d of it)
    auto normed = [&](int e, int head, int d) {
        const bool is_q = e < nq;
        float v = vals[e];
        if (norm_scope == 2) v *= (is_q ? rq : rk) * (gain_offset + (is_q ? q_gain[e] : k_gain[e - nq]));
        else if (norm_scope == 1) v *= head_scale[head] * (gain_offset + (is_q ? q_gain[d] : k_gain[d]));
        return v;
    };
    for (int pair = threadIdx.x; pair < total / 2; pair += THREADS) {
        const int e = 2 * pair, head = head_of(pair), d = e - head * D;
        if (e >= nq && !write_cache) continue;
        float a = normed(e, head, d), b = normed(e + 1, head, d + 1);
        if (rotate && d < rotary_dim) {
            const float* c_row = cos_tab + (size_t)pos * half;
            const float* s_row = sin_tab + (size_t)pos * half;
            if (interleaved) {
                const float c = c_row[d >> 1], s = s_row[d >> 1];
                const float ra = a * c - b * s, rb = b * c + a * s;
                a = ra; b = rb;
            } else {
                // entries d and d + 1 are both in the first half or both in the second (half is whole
                // pairs only when rotary_dim / 2 is even; else the scalar kernel runs)
                const bool first = d < half;
                const int i = first ? d : d - half, other = first ? e + half : e - half;
                const float pa = normed(other, head, first ? d + half : d - half);
                const float pb = normed(other + 1, head, (first ? d + half : d - half) + 1);
                a = first ? a * c_row[i] - pa * s_row[i] : a * c_row[i] + pa * s_row[i];
                b = first ? b * c_row[i + 1] - pb * s_row[i + 1] : b * c_row[i + 1] + pb * s_row[i + 1];
            }
        }
        if (e < nq) Pair<T>::store(q_out + (size_t)m * nq + e, a, b);
        else Pair<T>::store((T*)kv.base + kv_offset_sized(kv, page, 0, head - n_q, in_page) + d, a, b);
    }
}

// Any sizes (odd head sizes, odd row widths, a rotation whose half is odd): one entry at a time.
template <typename T>
__global__ void __launch_bounds__(128) qk_prepare_scalar_kernel(
    T* __restrict__ q_out, const T* __restrict__ proj, int proj_width, const float* __restrict__ q_gain,
    const float* __restrict__ k_gain, int norm_scope, float gain_offset, float eps, const float* __restrict__ cos_tab,
    const float* __restrict__ sin_tab, int table_len, int rotary_dim, int interleaved, int values_are_keys,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, PagedKV kv, int n_q, int write_cache,
    const float* __restrict__ v_cos, const float* __restrict__ v_sin, int v_table_len, int v_rotary_dim,
    int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(8) float vals[];
    __shared__ float scratch[33];
    const int m = blockIdx.x;
    const int D = kv.head_dim;
    const int nq = n_q * D, nk = kv.n_kv * D, total = nq + nk;
    const T* src = proj + (size_t)m * proj_width;
    const int pos = row_pos[m];

    float ss_q = 0.f, ss_k = 0.f;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
        const float v = to_f32<T>(src[e]);
        vals[e] = v;
        if (e < nq) ss_q += v * v; else ss_k += v * v;
    }
    int page = -1;
    if (write_cache) {
        page = kv.block_table[(size_t)row_slot[m] * kv.bt_stride + pos / kv.page_size];
        if (page < 0) {
            if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
            write_cache = 0;
        }
    }
    const int in_page = pos % kv.page_size;
    if (write_cache) {
        const int DV = !values_are_keys && kv.value_dim > 0 ? kv.value_dim : D;
        const bool turn = !values_are_keys && v_cos != nullptr && v_rotary_dim > 0;
        if (turn && pos >= v_table_len) {
            if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_POSITION_RANGE);
            return;
        }
        const int v_half = v_rotary_dim / 2;
        for (int e = threadIdx.x; e < kv.n_kv * DV; e += blockDim.x) {
            const int kvh = e / DV, d = e - kvh * DV;
            T v = values_are_keys ? src[nq + e] : src[total + e];
            if (turn && d < v_rotary_dim) {
                int i, partner;
                bool first;
                if (interleaved) {
                    i = d >> 1; first = (d & 1) == 0; partner = first ? e + 1 : e - 1;
                } else {
                    first = d < v_half; i = first ? d : d - v_half; partner = first ? e + v_half : e - v_half;
                }
                const float c = v_cos[(size_t)pos * v_half + i], sn = v_sin[(size_t)pos * v_half + i];
                const float own = to_f32<T>(v), other = to_f32<T>(src[total + partner]);
                v = from_f32<T>(first ? own * c - other * sn : own * c + other * sn);
            }
            ((T*)kv.base)[kv_offset_sized(kv, page, 1, kvh, in_page) + d] = v;
        }
    }
    if (norm_scope == 2) {
        const float tq = block_sum(ss_q, scratch);
        const float tk = block_sum(ss_k, scratch);
        const float rq = 1.0f / sqrtf(tq / (float)nq + eps), rk = 1.0f / sqrtf(tk / (float)nk + eps);
        for (int e = threadIdx.x; e < total; e += blockDim.x)
            vals[e] = e < nq ? vals[e] * rq * (gain_offset + q_gain[e]) : vals[e] * rk * (gain_offset + k_gain[e - nq]);
    } else if (norm_scope == 1) {
        __syncthreads();
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        for (int head = warp; head < n_q + kv.n_kv; head += blockDim.x >> 5) {
            float ss = 0.f;
            for (int d = lane; d < D; d += 32) ss += vals[head * D + d] * vals[head * D + d];
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float)D + eps);
            const float* gain = head < n_q ? q_gain : k_gain;
            for (int d = lane; d < D; d += 32) vals[head * D + d] *= r * (gain_offset + gain[d]);
        }
    }
    __syncthreads();
    const bool rotate = cos_tab != nullptr && rotary_dim > 0;
    if (rotate && pos >= table_len) {
        if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_POSITION_RANGE);
        return;
    }
    const int half = rotary_dim / 2;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
        const int head = e / D, d = e - head * D;
        float out = vals[e];
        if (rotate && d < rotary_dim) {
            int i, partner;
            bool first;
            if (interleaved) {
                i = d >> 1; first = (d & 1) == 0; partner = first ? e + 1 : e - 1;
            } else {
                first = d < half; i = first ? d : d - half; partner = first ? e + half : e - half;
            }
            const float c = cos_tab[(size_t)pos * half + i], s = sin_tab[(size_t)pos * half + i];
            out = first ? out * c - vals[partner] * s : out * c + vals[partner] * s;
        }
        if (e < nq) {
            q_out[(size_t)m * nq + e] = from_f32<T>(out);
        } else if (write_cache) {
            const int kvh = head - n_q;
            ((T*)kv.base)[kv_offset_sized(kv, page, 0, kvh, in_page) + d] = from_f32<T>(out);
        }
    }
}

// No norm and no rotation: the projected row is only split, its queries to q_out, its keys and
// values to the cache.  A copy in pieces of 16 bytes, for sizes and addresses that keep every
// piece whole and aligned; the same bits as the kernels above produce.
template <typename T>
__global__ void __launch_bounds__(128) qk_split_kernel(
    T* __restrict__ q_out, const T* __restrict__ proj, int proj_width, int values_are_keys,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, PagedKV kv, int n_q, int write_cache,
    int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int V = 16 / (int)sizeof(T);
    const int m = blockIdx.x;
    const int D = kv.head_dim, DV = kv.value_dim > 0 ? kv.value_dim : D;
    const int nq = n_q * D, nk = kv.n_kv * D, nv = values_are_keys ? 0 : kv.n_kv * DV;
    const T* src = proj + (size_t)m * proj_width;
    const int pos = row_pos[m];
    int page = -1;
    if (write_cache) {
        page = kv.block_table[(size_t)row_slot[m] * kv.bt_stride + pos / kv.page_size];
        if (page < 0) {
            if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
            write_cache = 0;
        }
    }
    const int in_page = pos % kv.page_size;
    T* cache = (T*)kv.base;
    const int pieces = (write_cache ? nq + nk + nv : nq) / V;
    for (int piece = threadIdx.x; piece < pieces; piece += 128) {
        const int e = piece * V;
        const uint4 v = *reinterpret_cast<const uint4*>(src + e);
        if (e < nq) {
            *reinterpret_cast<uint4*>(q_out + (size_t)m * nq + e) = v;
        } else if (e < nq + nk) {
            const int kvh = (e - nq) / D, d = e - nq - kvh * D;
            *reinterpret_cast<uint4*>(cache + kv_offset_sized(kv, page, 0, kvh, in_page) + d) = v;
            if (values_are_keys) *reinterpret_cast<uint4*>(cache + kv_offset_sized(kv, page, 1, kvh, in_page) + d) = v;
        } else {
            const int kvh = (e - nq - nk) / DV, d = e - nq - nk - kvh * DV;
            *reinterpret_cast<uint4*>(cache + kv_offset_sized(kv, page, 1, kvh, in_page) + d) = v;
        }
    }
}

template <typename T>
int launch(void* q_out, const void* proj, int proj_width, const float* q_gain, const float* k_gain, int norm_scope,
           float gain_offset, float eps, const float* cos_tab, const float* sin_tab, int table_len, int rotary_dim,
           int interleaved, int values_are_keys, const int* row_slot, const int* row_pos, PagedKV kv, int n_rows,
           int n_q, int write_cache, const float* v_cos, const float* v_sin, int v_table_len, int v_rotary_dim, int* err,
           cudaStream_t stream) {
    const int D = kv.head_dim, n_heads = n_q + kv.n_kv;
    {
        constexpr int V = 16 / (int)sizeof(T);
        const int DV = kv.value_dim > 0 ? kv.value_dim : D;
        const bool rotates = cos_tab != nullptr && rotary_dim > 0;
        if (norm_scope == 0 && !rotates && !(v_cos != nullptr && v_rotary_dim > 0) && D % V == 0 && DV % V == 0 && proj_width % V == 0 &&
            (((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)kv.base) & 15) == 0) {
            thn_launch(qk_split_kernel<T>, n_rows, 128, 0, stream, (T*)q_out, (const T*)proj, proj_width, values_are_keys,
                       row_slot, row_pos, kv, n_q, write_cache, err);
            return thn_launch_status("qk_prepare");
        }
    }
    const size_t smem = ((size_t)n_heads * D + n_heads) * sizeof(float);
    THN_UNSUPPORTED_IF(smem > 200 * 1024, "qk_prepare: %d heads of %d do not fit shared memory", n_heads, D);
    // pairs of adjacent entries need even sizes everywhere and pair-aligned addresses
    const bool pairs = D % 2 == 0 && kv.value_dim % 2 == 0 && proj_width % 2 == 0 && (interleaved || (rotary_dim / 2) % 2 == 0) &&
                       (interleaved || v_cos == nullptr || (v_rotary_dim / 2) % 2 == 0) &&
                       (((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)kv.base) & (2 * sizeof(T) - 1)) == 0;
    if (!pairs) {
        if (smem > 32 * 1024)
            cudaFuncSetAttribute(qk_prepare_scalar_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        thn_launch(qk_prepare_scalar_kernel<T>, n_rows, 128, smem, stream, (T*)q_out, (const T*)proj, proj_width, q_gain,
                   k_gain, norm_scope, gain_offset, eps, cos_tab, sin_tab, table_len, rotary_dim, interleaved,
                   values_are_keys, row_slot, row_pos, kv, n_q, write_cache, v_cos, v_sin, v_table_len, v_rotary_dim, err);
        return thn_launch_status("qk_prepare");
    }
    int shift = -1;
    if (((D / 2) & (D / 2 - 1)) == 0) for (shift = 0; (1 << shift) < D / 2; ++shift) {}
    // few rows (single-token steps): the row's latency counts, 512 threads; many rows: 128 threads
    // and more blocks per SM, 256 for rows of 4,096 entries or more
#define THN_QK_LAUNCH(THREADS)                                                                                        \
    do {                                                                                                              \
        if (smem > 32 * 1024)                                                                                         \
            cudaFuncSetAttribute(qk_prepare_kernel<T, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        thn_launch(qk_prepare_kernel<T, THREADS>, n_rows, THREADS, smem, stream, (T*)q_out, (const T*)proj, proj_width, \
                   q_gain, k_gain, norm_scope, gain_offset, eps, cos_tab, sin_tab, table_len, rotary_dim, interleaved, \
                   values_are_keys, row_slot, row_pos, kv, n_q, write_cache, shift, v_cos, v_sin, v_table_len,         \
                   v_rotary_dim, err);                                                                                \
    } while (0)
    if (n_rows <= 64 && n_heads * D >= 2048) THN_QK_LAUNCH(512);
    else if (n_heads * D >= 4096) THN_QK_LAUNCH(256);
    else THN_QK_LAUNCH(128);
#undef THN_QK_LAUNCH
    return thn_launch_status("qk_prepare");
}
}  // namespace

THN_API int thn_qk_prepare(void* q_out, const void* proj, int proj_width, const float* q_gain, const float* k_gain,
                           int norm_scope, float gain_offset, float eps, const float* cos_tab, const float* sin_tab,
                           int table_len, int rotary_dim, int interleaved, int values_are_keys, const int* row_slot,
                           const int* row_pos, void* kv_base, const int* block_table, int bt_stride, int n_kv,
                           int page_size, int head_dim, int value_dim, int n_rows, int n_q, int write_cache,
                           const float* v_cos, const float* v_sin, int v_table_len, int v_rotary_dim, int dtype,
                           int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && n_q > 0 && n_kv > 0 && head_dim > 0 && page_size > 0, "qk_prepare: bad sizes");
    THN_CHECK_ARG(norm_scope >= 0 && norm_scope <= 2, "qk_prepare: norm scope %d", norm_scope);
    THN_CHECK_ARG(norm_scope == 0 || (q_gain && k_gain && eps > 0.f), "qk_prepare: a norm needs gains and eps");
    THN_CHECK_ARG(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
                  "qk_prepare: rotary_dim %d must be even and within the head size %d", rotary_dim, head_dim);
    if (value_dim <= 0) value_dim = head_dim;
    THN_CHECK_ARG(v_cos == nullptr || (v_sin != nullptr && !values_are_keys && v_rotary_dim >= 0 && v_rotary_dim % 2 == 0 &&
                                       v_rotary_dim <= value_dim),
                  "qk_prepare: a rotation of the values needs values of their own and an even size within %d", value_dim);
    THN_CHECK_ARG(!values_are_keys || value_dim == head_dim, "qk_prepare: values that are the keys have the keys' size");
    THN_CHECK_ARG(proj_width >= (n_q + n_kv) * head_dim + (values_are_keys ? 0 : n_kv * value_dim),
                  "qk_prepare: rows of %d are too short", proj_width);
    if (n_rows == 0) return THN_OK;
    PagedKV kv{kv_base, block_table, bt_stride, n_kv, page_size, head_dim, value_dim == head_dim ? 0 : value_dim};
    if (dtype == THN_F32)
        return launch<float>(q_out, proj, proj_width, q_gain, k_gain, norm_scope, gain_offset, eps, cos_tab, sin_tab,
                             table_len, rotary_dim, interleaved, values_are_keys, row_slot, row_pos, kv, n_rows, n_q,
                             write_cache, v_cos, v_sin, v_table_len, v_rotary_dim, err, stream);
    if (dtype == THN_BF16)
        return launch<__nv_bfloat16>(q_out, proj, proj_width, q_gain, k_gain, norm_scope, gain_offset, eps, cos_tab,
                                     sin_tab, table_len, rotary_dim, interleaved, values_are_keys, row_slot, row_pos, kv,
                                     n_rows, n_q, write_cache, v_cos, v_sin, v_table_len, v_rotary_dim, err, stream);
    THN_CHECK_ARG(false, "qk_prepare: unknown dtype %d", dtype);
    return THN_OK;
}
