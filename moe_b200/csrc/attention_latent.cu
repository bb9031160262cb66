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

// One block a token.
template <typename OT>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ proj, int ld, const int* __restrict__ pos,
                      const int* __restrict__ seq_of_token, const float* __restrict__ w, float eps, int num_tokens,
                      int nh, int d, int r, int D, OT* __restrict__ q_t, OT* __restrict__ k_new,
                      const LatentCommit c, int* status) {
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
    for (int i = threadIdx.x; i < nh * d; i += blockDim.x) {
        const int h = i / d, j = i % d;
        st_f(q_t + ((size_t)h * num_tokens + t) * d + j, row[i]);
    }
}

template <typename ST, typename DT>
__global__ void heads_transpose_kernel(const ST* __restrict__ src, long long s_outer, long long s_inner, int A, int B,
                                       int n, int wd, DT* __restrict__ dst) {
    pdl_sync();
    const long long total = (long long)A * B * wd;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int j = (int)(i % wd);
    const long long ba = i / wd;
    const int a = (int)(ba % A), b = (int)(ba / A);
    st_f(dst + i, j < n ? ld_f(src + (size_t)a * s_outer + (size_t)b * s_inner + j) : 0.f);
}

// One warp a (token, head).
template <typename T>
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
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) {
        const float o = ld_f(a1 + j) - lambda * ld_f(a2 + j);
        ss += o * o;
    }
    ss = warp_sum(ss);
    float f = mult / sqrtf(ss / (float)dv + eps);
    if (gate) f *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_ld + h]));
    T* o_row = out + ((size_t)t * nh + h) * dv;
    for (int j = lane; j < dv; j += 32) st_f(o_row + j, (ld_f(a1 + j) - lambda * ld_f(a2 + j)) * f);
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

// proj: [T, ld] 32-bit: nh * d query columns, then r latent columns.  q_t: [nh, T, d]; k_new: [T, D].
MOE_API int moe_latent_prepare(const float* proj, int ld, const int* pos, const int* seq_of_token, const float* w,
                               float eps, int num_tokens, int nh, int d, int r, int D, void* q_t, void* k_new,
                               int out_dt, void* k_cache, void* v_cache, const int* seq_end, const int* slots,
                               const int* tables, int table_stride, int ring, int page_size, int num_pages,
                               int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (nh <= 0 || d <= 0 || r <= 0 || D < r || ld < nh * d + r || !proj || !w || !q_t || !k_new)
        return (int)cudaErrorInvalidValue;
    if (k_cache && (!seq_end || !slots || !tables || !seq_of_token || !pos)) return (int)cudaErrorInvalidValue;
    const LatentCommit c{k_cache, v_cache, seq_end, slots, tables, table_stride, ring, page_size, num_pages};
    if (out_dt == DT_F32)
        return launch_pdl(latent_prepare_kernel<float>, num_tokens, 256, 0, stream, proj, ld, pos, seq_of_token, w, eps,
                          num_tokens, nh, d, r, D, (float*)q_t, (float*)k_new, c, status);
    return launch_pdl(latent_prepare_kernel<__nv_bfloat16>, num_tokens, 256, 0, stream, proj, ld, pos, seq_of_token, w,
                      eps, num_tokens, nh, d, r, D, (__nv_bfloat16*)q_t, (__nv_bfloat16*)k_new, c, status);
}

// src: element (a, b, j) at a * s_outer + b * s_inner + j, j < n; dst: dense [B, A, wd].
MOE_API int moe_heads_transpose(const void* src, int src_dt, long long s_outer, long long s_inner, int A, int B, int n,
                                int wd, void* dst, int dst_dt, cudaStream_t stream) {
    const long long total = (long long)A * B * wd;
    if (total <= 0) return 0;
    if (n < 0 || n > wd || !src || !dst) return (int)cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)((total + 255) / 256);
#define TR(ST_, DT_)                                                                                              \
    return launch_pdl(heads_transpose_kernel<ST_, DT_>, blocks, 256, 0, stream, (const ST_*)src, s_outer, s_inner, A, B, \
                      n, wd, (DT_*)dst)
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
    const unsigned blocks = (unsigned)((pairs + 3) / 4);
    if (dt == DT_F32)
        return launch_pdl(diff_combine_kernel<float>, blocks, 128, 0, stream, (const float*)ctx, gate, gate_ld, pairs,
                          nh, dv, D, lambda, eps, mult, (float*)out);
    return launch_pdl(diff_combine_kernel<__nv_bfloat16>, blocks, 128, 0, stream, (const __nv_bfloat16*)ctx, gate,
                      gate_ld, pairs, nh, dv, D, lambda, eps, mult, (__nv_bfloat16*)out);
}

MOE_API int moe_add_row(float* x, const float* delta, const float* row, long long num_tokens, int width,
                        cudaStream_t stream) {
    const long long total = num_tokens * width;
    if (total <= 0) return 0;
    if (!x || !row) return (int)cudaErrorInvalidValue;
    return launch_pdl(add_row_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, x, delta, row, total, width);
}
