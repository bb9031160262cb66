// Kernels around two kinds of attention layer that need more than a rotation and a split:
//
// LATENT attention.  A layer projects its input to queries (heads of d) and to ONE small latent c of
// r numbers per position; a head's keys and values are W_uk_h c and W_uv_h c.  Since
//     q_h . (W_uk_h c) = (W_uk_h^T q_h) . c        and        sum_j p_j W_uv_h c_j = W_uv_h (sum_j p_j c_j),
// the attention itself runs over the cached latents alone: every query head reads the same single
// record c as key AND as value, with queries W_uk_h^T q_h of r numbers, and the head's values are
// formed from the r numbers that come out.  The two per-head products are grouped products (a group
// a head) over rows laid out head by head, hence the transposes here.
//   latent_prepare    from the 32-bit projection row [q heads | latent]: c = x / sqrt(mean(x^2) + eps) * w
//                     over the latent, written as the step's key record of width D >= r (zero-filled)
//                     and, optionally, appended to the paged cache; the queries are written head by
//                     head, q_t[h][t][0..d).
//   heads_transpose   dst[b][a][0..wd) = src[a][b][0..n) (zero-filled beyond n), any of the two
//                     storage types on either side.
//
// DIFFERENTIAL attention.  Every head runs two softmax attentions ("maps") over the same values and
// joins them:  o = a1 - lambda a2;  o <- o / sqrt(mean(o^2) + eps) * mult;  o <- o * sigmoid(g_h),
// one gate logit a head.  The maps come as heads of their own (map 1 of all heads, then map 2).
//   diff_combine      out[t, h * dv + j] from ctx[t, h, j] and ctx[t, nh + h, j].
//
//   add_row           x[t, :] += delta[t, :] + row[:]   (a learned vector added to every token's
//                     stream, with whatever was still pending; 32-bit)
// Norms, the difference and the gate are 32-bit; only stores round to the activation dtype.
#include "common.cuh"

namespace {

struct LatentCommit {
    void* k_cache;            // null: no append
    void* v_cache;            // may equal k_cache (the values are the keys)
    const int* seq_end;
    const int* slots;
    const int* tables;
    int table_stride, ring, page_size, num_pages;
};

// four consecutive elements at once (the pointer is aligned to four elements)
__device__ __forceinline__ void ld4(const float* p, float* v) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x, v[1] = x.y, v[2] = x.z, v[3] = x.w;
}
__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float* v) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(x.x << 16), v[1] = __uint_as_float(x.x & 0xffff0000u);
    v[2] = __uint_as_float(x.y << 16), v[3] = __uint_as_float(x.y & 0xffff0000u);
}
__device__ __forceinline__ void st4(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float* v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 x;
    x.x = *reinterpret_cast<const unsigned*>(&a), x.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = x;
}

// One block a token.
template <typename OT>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ proj, int ld, const int* __restrict__ pos,
                      const int* __restrict__ seq_of_token, const float* __restrict__ w, float eps, int num_tokens,
                      int nh, int d, int r, int D, OT* __restrict__ q_t, OT* __restrict__ k_new,
                      const LatentCommit c, int* status, int vec4, int q_major) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    pdl_sync();
    const float* row = proj + (size_t)t * ld;
    const float* lat = row + (size_t)nh * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < r; i += blockDim.x) ss += lat[i] * lat[i];
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)r + eps);
    OT* cd = nullptr;
    OT* cv = nullptr;
    if (c.k_cache) {
        const int s = seq_of_token[t];
        const int p = pos[t];
        if (s >= 0 && !(c.ring > 0 && p < c.seq_end[s] - c.ring)) {
            const CachePos cp = cache_pos(p, c.ring, c.tables + (size_t)c.slots[s] * c.table_stride, c.page_size,
                                          c.num_pages, status);
            const size_t at = cache_index(cp, 0, 1, c.page_size, D);
            cd = (OT*)c.k_cache + at;
            if (c.v_cache && c.v_cache != c.k_cache) cv = (OT*)c.v_cache + at;
        }
    }
    OT* kd = k_new + (size_t)t * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float x = i < r ? lat[i] * inv * w[i] : 0.f;
        st_f(kd + i, x);
        if (cd) st_f(cd + i, x);
        if (cv) st_f(cv + i, x);
    }
    if (q_major) {       // the queries token by token, q[t][h][0..D), zero-filled beyond d
        OT* qd = q_t + (size_t)t * nh * D;
        if (vec4 && D % 4 == 0) {
            for (int i = threadIdx.x * 4; i < nh * D; i += blockDim.x * 4) {
                const int h = i / D, j = i % D;
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (j < d) ld4(row + (size_t)h * d + j, v);
                st4(qd + i, v);
            }
        } else {
            for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
                const int h = i / D, j = i % D;
                st_f(qd + i, j < d ? row[(size_t)h * d + j] : 0.f);
            }
        }
        return;
    }
    if (vec4) {          // d and the row pitch are multiples of four, both pointers aligned to four elements
        for (int i = threadIdx.x * 4; i < nh * d; i += blockDim.x * 4) {
            const int h = i / d, j = i % d;
            float v[4];
            ld4(row + i, v);
            st4(q_t + ((size_t)h * num_tokens + t) * d + j, v);
        }
        return;
    }
    for (int i = threadIdx.x; i < nh * d; i += blockDim.x) {
        const int h = i / d, j = i % d;
        st_f(q_t + ((size_t)h * num_tokens + t) * d + j, row[i]);
    }
}

__device__ __forceinline__ void ld2(const float* p, float* v) {
    const float2 x = *reinterpret_cast<const float2*>(p);
    v[0] = x.x, v[1] = x.y;
}
__device__ __forceinline__ void ld2(const __nv_bfloat16* p, float* v) {
    const unsigned x = *reinterpret_cast<const unsigned*>(p);
    v[0] = __uint_as_float(x << 16), v[1] = __uint_as_float(x & 0xffff0000u);
}
__device__ __forceinline__ void st2(float* p, const float* v) { *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]); }
__device__ __forceinline__ void st2(__nv_bfloat16* p, const float* v) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
}

// VEC = 4: n, wd and both pitches are multiples of four and both pointers aligned to four elements.
template <typename ST, typename DT, int VEC>
__global__ void heads_transpose_kernel(const ST* __restrict__ src, long long s_outer, long long s_inner, int A, int B,
                                       int n, int wd, DT* __restrict__ dst) {
    pdl_sync();
    const int wv = wd / VEC;
    const long long total = (long long)A * B * wv;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int j = (int)(i % wv) * VEC;
    const long long ba = i / wv;
    const int a = (int)(ba % A), b = (int)(ba / A);
    const ST* from = src + (size_t)a * s_outer + (size_t)b * s_inner + j;
    DT* to = dst + ba * wd + j;
    if (VEC == 4) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (j < n) ld4(from, v);
        st4(to, v);
    } else {
        st_f(to, j < n ? ld_f(from) : 0.f);
    }
}

// One warp a (token, head).  The head's difference stays in registers between the norm's sum and the
// store (dv <= 256: up to eight elements a lane); with an even dv (and 4-byte aligned rows) a lane
// takes two neighbouring elements a load.
template <typename T, int VEC>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const T* __restrict__ ctx, const float* __restrict__ gate, int gate_ld, long long pairs, int nh,
                    int dv, int D, float lambda, float eps, float mult, T* __restrict__ out) {
    pdl_sync();
    const long long w = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= pairs) return;
    const long long t = w / nh;
    const int h = (int)(w % nh);
    const T* a1 = ctx + ((size_t)t * 2 * nh + h) * D;
    const T* a2 = ctx + ((size_t)t * 2 * nh + nh + h) * D;
    constexpr int SLOTS = 256 / (32 * VEC);
    float o[SLOTS][VEC];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < SLOTS; i++) {
        const int j = (i * 32 + lane) * VEC;
#pragma unroll
        for (int e = 0; e < VEC; e++) o[i][e] = 0.f;
        if (j < dv) {
            if (VEC == 2) {
                float x[2], y[2];
                ld2(a1 + j, x), ld2(a2 + j, y);
                o[i][0] = x[0] - lambda * y[0], o[i][1] = x[1] - lambda * y[1];
            } else {
                o[i][0] = ld_f(a1 + j) - lambda * ld_f(a2 + j);
            }
        }
#pragma unroll
        for (int e = 0; e < VEC; e++) ss += o[i][e] * o[i][e];
    }
    ss = warp_sum(ss);
    float f = mult / sqrtf(ss / (float)dv + eps);
    if (gate) f *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_ld + h]));
    T* o_row = out + ((size_t)t * nh + h) * dv;
#pragma unroll
    for (int i = 0; i < SLOTS; i++) {
        const int j = (i * 32 + lane) * VEC;
        if (j < dv) {
            if (VEC == 2) {
                const float v[2] = {o[i][0] * f, o[i][1] * f};
                st2(o_row + j, v);
            } else {
                st_f(o_row + j, o[i][0] * f);
            }
        }
    }
}

__global__ void add_row_kernel(float* __restrict__ x, const float* __restrict__ delta, const float* __restrict__ row,
                               long long total, int width) {
    pdl_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float v = x[i];
    if (delta) v += delta[i];
    x[i] = v + row[i % width];
}

}  // namespace

// proj: [T, ld] 32-bit: nh * d query columns, then r latent columns.  q_t: [nh, T, d], or with q_major
// [T, nh, D] zero-filled beyond d (d <= D); k_new: [T, D].
MOE_API int moe_latent_prepare(const float* proj, int ld, const int* pos, const int* seq_of_token, const float* w,
                               float eps, int num_tokens, int nh, int d, int r, int D, void* q_t, void* k_new,
                               int out_dt, void* k_cache, void* v_cache, const int* seq_end, const int* slots,
                               const int* tables, int table_stride, int ring, int page_size, int num_pages,
                               int* status, int q_major, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (nh <= 0 || d <= 0 || r <= 0 || D < r || ld < nh * d + r || !proj || !w || !q_t || !k_new || (q_major && d > D))
        return (int)cudaErrorInvalidValue;
    if (k_cache && (!seq_end || !slots || !tables || !seq_of_token || !pos)) return (int)cudaErrorInvalidValue;
    const LatentCommit c{k_cache, v_cache, seq_end, slots, tables, table_stride, ring, page_size, num_pages};
    const int vec4 = d % 4 == 0 && ld % 4 == 0 && (uintptr_t)proj % 16 == 0 &&
                     (uintptr_t)q_t % (out_dt == DT_F32 ? 16 : 8) == 0;
    if (out_dt == DT_F32)
        return launch_pdl(latent_prepare_kernel<float>, num_tokens, 256, 0, stream, proj, ld, pos, seq_of_token, w, eps,
                          num_tokens, nh, d, r, D, (float*)q_t, (float*)k_new, c, status, vec4, q_major);
    return launch_pdl(latent_prepare_kernel<__nv_bfloat16>, num_tokens, 256, 0, stream, proj, ld, pos, seq_of_token, w,
                      eps, num_tokens, nh, d, r, D, (__nv_bfloat16*)q_t, (__nv_bfloat16*)k_new, c, status, vec4, q_major);
}

// src: element (a, b, j) at a * s_outer + b * s_inner + j, j < n; dst: dense [B, A, wd].
MOE_API int moe_heads_transpose(const void* src, int src_dt, long long s_outer, long long s_inner, int A, int B, int n,
                                int wd, void* dst, int dst_dt, cudaStream_t stream) {
    const long long total = (long long)A * B * wd;
    if (total <= 0) return 0;
    if (n < 0 || n > wd || !src || !dst) return (int)cudaErrorInvalidValue;
    const size_t se = src_dt == DT_F32 ? 4 : 2, de = dst_dt == DT_F32 ? 4 : 2;
    const bool vec = n % 4 == 0 && wd % 4 == 0 && s_outer % 4 == 0 && s_inner % 4 == 0 &&
                     (uintptr_t)src % (4 * se) == 0 && (uintptr_t)dst % (4 * de) == 0;
    const unsigned blocks = (unsigned)(((vec ? total / 4 : total) + 255) / 256);
#define TR(ST_, DT_)                                                                                                \
    return vec ? launch_pdl(heads_transpose_kernel<ST_, DT_, 4>, blocks, 256, 0, stream, (const ST_*)src, s_outer,      \
                            s_inner, A, B, n, wd, (DT_*)dst)                                                        \
               : launch_pdl(heads_transpose_kernel<ST_, DT_, 1>, blocks, 256, 0, stream, (const ST_*)src, s_outer,      \
                            s_inner, A, B, n, wd, (DT_*)dst)
    if (src_dt == DT_F32) {
        if (dst_dt == DT_F32) TR(float, float);
        TR(float, __nv_bfloat16);
    }
    if (dst_dt == DT_F32) TR(__nv_bfloat16, float);
    TR(__nv_bfloat16, __nv_bfloat16);
#undef TR
}

// ctx: [T, 2 nh, D] (map 1 of every head, then map 2); gate: first gate logit of token 0 (row pitch
// gate_ld, 32-bit) or null; out: [T, nh * dv].
MOE_API int moe_diff_combine(const void* ctx, const float* gate, int gate_ld, int num_tokens, int nh, int dv, int D,
                             float lambda, float eps, float mult, void* out, int dt, cudaStream_t stream) {
    const long long pairs = (long long)num_tokens * nh;
    if (pairs <= 0) return 0;
    if (dv <= 0 || D < dv || !ctx || !out) return (int)cudaErrorInvalidValue;
    if (dv > 256) return (int)cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)((pairs + 3) / 4);
    const size_t el = dt == DT_F32 ? 4 : 2;
    const bool vec = dv % 2 == 0 && D % 2 == 0 && (uintptr_t)ctx % (2 * el) == 0 && (uintptr_t)out % (2 * el) == 0;
#define DC(T_, V_)                                                                                                 \
    return launch_pdl(diff_combine_kernel<T_, V_>, blocks, 128, 0, stream, (const T_*)ctx, gate, gate_ld, pairs, nh, dv, \
                      D, lambda, eps, mult, (T_*)out)
    if (dt == DT_F32) {
        if (vec) DC(float, 2);
        DC(float, 1);
    }
    if (vec) DC(__nv_bfloat16, 2);
    DC(__nv_bfloat16, 1);
#undef DC
}

MOE_API int moe_add_row(float* x, const float* delta, const float* row, long long num_tokens, int width,
                        cudaStream_t stream) {
    const long long total = num_tokens * width;
    if (total <= 0) return 0;
    if (!x || !row) return (int)cudaErrorInvalidValue;
    return launch_pdl(add_row_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, x, delta, row, total, width);
}
