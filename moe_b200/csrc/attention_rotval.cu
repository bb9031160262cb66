// Between projection and attention, and between attention and output projection, for attention
// layers whose queries and keys are normed over the WHOLE projection and whose values carry a
// position of their own:
//
//   whole_prepare   from a token's 32-bit projection row [q heads | k heads | v heads]: an optional RMS
//                   norm over all query channels at once (x / sqrt(mean(x^2) + eps) * w, one weight a
//                   channel) and the same over all key channels; the rotation of the first `rot`
//                   dimensions of every query and key head (pairs (i, i + rot/2), angle pos * freq[i]);
//                   optionally the rotation of every value head over all its dv dimensions (pairs
//                   (m, m + dv/2), angle pos * vfreq[m]); the split into q, k and v records of the
//                   cache's width D >= max(d, dv), zero-filled; optionally the append to the paged cache.
//   unrotate_pack   out[t, h * dv + :] = the head's attention output turned back by the QUERY's position
//                   (pair m by -pos * vfreq[m]), which leaves every value turned by its distance to the
//                   query; the padding columns of the record are dropped.
// Norm, angles and rotations are 32-bit; only the stores round to the activation dtype.
#include "common.cuh"

namespace {

struct WholeCommit {
    void* k_cache;            // null: no append
    void* v_cache;
    const int* seq_end;
    const int* slots;
    const int* tables;
    int table_stride, ring, page_size, num_pages;
};

constexpr int WP_THREADS = 256;

template <typename OT>
__global__ void __launch_bounds__(WP_THREADS)
whole_prepare_kernel(const float* __restrict__ proj, int ld, const int* __restrict__ pos,
                     const int* __restrict__ seq_of_token, const float* __restrict__ q_norm,
                     const float* __restrict__ k_norm, float eps, const float* __restrict__ freq, int rot,
                     const float* __restrict__ vfreq, int nh, int nkv, int d, int dv, int D, OT* __restrict__ q,
                     OT* __restrict__ k, OT* __restrict__ v, long long ldq, long long ldkv, const WholeCommit c,
                     int* status) {
    extern __shared__ __align__(16) float wp_smem[];
    __shared__ float red[32];
    const int half = rot / 2, vhalf = vfreq ? dv / 2 : 0;
    float* ang = wp_smem;                 // cos[half], sin[half]
    float* vang = wp_smem + 2 * half;     // cos[vhalf], sin[vhalf]
    const int t = blockIdx.x;
    pdl_sync();
    const int p_int = pos[t];
    const float p = (float)p_int;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(p * freq[i], &sn, &cs);
        ang[i] = cs, ang[half + i] = sn;
    }
    for (int i = threadIdx.x; i < vhalf; i += blockDim.x) {
        float sn, cs;
        sincosf(p * vfreq[i], &sn, &cs);
        vang[i] = cs, vang[vhalf + i] = sn;
    }
    const float* row = proj + (size_t)t * ld;
    const int nq = nh * d, nk = nkv * d;
    float inv_q = 1.f, inv_k = 1.f;
    const int my_per = (nh + 2 * nkv + gridDim.y - 1) / gridDim.y;
    const bool has_q = blockIdx.y * my_per < nh;
    const bool has_k = blockIdx.y * my_per < nh + nkv && (blockIdx.y + 1) * my_per > nh;
    if (q_norm && has_q) {
        float ss = 0.f;
        for (int e = threadIdx.x; e < nq; e += blockDim.x) ss = fmaf(row[e], row[e], ss);
        inv_q = 1.0f / sqrtf(block_sum(ss, red) / (float)nq + eps);
    }
    if (k_norm && has_k) {
        float ss = 0.f;
        for (int e = threadIdx.x; e < nk; e += blockDim.x) ss = fmaf(row[nq + e], row[nq + e], ss);
        inv_k = 1.0f / sqrtf(block_sum(ss, red) / (float)nk + eps);
    }
    __syncthreads();
    bool append = false;
    CachePos cp;
    cp.page = 0, cp.off = 0;
    if (c.k_cache) {
        const int s = seq_of_token[t];
        if (s >= 0 && !(c.ring > 0 && p_int < c.seq_end[s] - c.ring)) {
            cp = cache_pos(p_int, c.ring, c.tables + (size_t)c.slots[s] * c.table_stride, c.page_size, c.num_pages,
                           status);
            append = true;
        }
    }
    // (few tokens: gridDim.y blocks share a token's head slots, each forming the sums of squares for itself)
    const int hs_count = nh + 2 * nkv;
    const int per = (hs_count + gridDim.y - 1) / gridDim.y;
    const int hs_lo = blockIdx.y * per, hs_hi = min(hs_count, hs_lo + per);
    for (int idx = hs_lo * D + threadIdx.x; idx < hs_hi * D; idx += blockDim.x) {
        const int hs = idx / D, e = idx % D;
        const bool is_q = hs < nh, is_k = !is_q && hs < nh + nkv;
        const int head = is_q ? hs : is_k ? hs - nh : hs - nh - nkv;
        float x = 0.f;
        if (is_q || is_k) {
            if (e < d) {
                const int c0 = (is_q ? 0 : nq) + head * d;          // the head's first channel in the row
                const float inv = is_q ? inv_q : inv_k;
                const float* nw = is_q ? q_norm : k_norm;
                const int wc = head * d;                            // ... and in the norm's weight
                auto val = [&](int i) { return nw ? row[c0 + i] * inv * nw[wc + i] : row[c0 + i]; };
                if (e < rot) {
                    const int i = e < half ? e : e - half;
                    const float a = val(i), b = val(i + half), cs = ang[i], sn = ang[half + i];
                    x = e < half ? rot_lo(a, b, cs, sn) : rot_hi(a, b, cs, sn);
                } else {
                    x = val(e);
                }
            }
        } else if (e < dv) {
            const float* src = row + nq + nk + head * dv;
            if (vhalf && e < 2 * vhalf) {
                const int i = e < vhalf ? e : e - vhalf;
                const float a = src[i], b = src[i + vhalf], cs = vang[i], sn = vang[vhalf + i];
                x = e < vhalf ? rot_lo(a, b, cs, sn) : rot_hi(a, b, cs, sn);
            } else {
                x = src[e];
            }
        }
        OT* dst = is_q ? q + (size_t)t * ldq + (size_t)head * D : (is_k ? k : v) + (size_t)t * ldkv + (size_t)head * D;
        st_f(dst + e, x);
        if (!is_q && append)
            st_f((OT*)(is_k ? c.k_cache : c.v_cache) + cache_index(cp, head, nkv, c.page_size, D) + e, x);
    }
}

// A block per token: the token's angles once in shared memory, then every pair of every head.
template <typename OT>
__global__ void __launch_bounds__(128)
unrotate_pack_kernel(const OT* __restrict__ ctx, const int* __restrict__ pos, const float* __restrict__ vfreq, int nh,
                     int dv, int D, OT* __restrict__ out) {
    extern __shared__ __align__(16) float up_smem[];
    const int t = blockIdx.x, vhalf = dv / 2;
    pdl_sync();
    const float p = (float)pos[t];
    for (int i = threadIdx.x; i < vhalf; i += blockDim.x) {
        float sn, cs;
        sincosf(p * vfreq[i], &sn, &cs);
        up_smem[i] = cs, up_smem[vhalf + i] = -sn;      // the turn back
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nh * vhalf; idx += blockDim.x) {
        const int h = idx / vhalf, m = idx % vhalf;
        const OT* src = ctx + ((size_t)t * nh + h) * D;
        OT* dst = out + ((size_t)t * nh + h) * dv;
        const float a = ld_f(src + m), b = ld_f(src + m + vhalf), cs = up_smem[m], sn = up_smem[vhalf + m];
        st_f(dst + m, rot_lo(a, b, cs, sn));
        st_f(dst + m + vhalf, rot_hi(a, b, cs, sn));
    }
    if (dv & 1)
        for (int h = threadIdx.x; h < nh; h += blockDim.x)
            st_f(out + ((size_t)t * nh + h) * dv + dv - 1, ld_f(ctx + ((size_t)t * nh + h) * D + dv - 1));
}

}  // namespace

// proj: [T, ld] 32-bit: q heads (nh * d), k heads (nkv * d), v heads (nkv * dv).  q_norm [nh * d], k_norm
// [nkv * d] or null (no norm); freq [rot / 2]; vfreq [dv / 2] or null (values are not rotated).
// q: [T, nh, D] with a token pitch of ldq elements; k, v: [T, nkv, D] with a token pitch of ldkv.
MOE_API int moe_whole_prepare(const float* proj, int ld, const int* pos, const int* seq_of_token, const float* q_norm,
                              const float* k_norm, float eps, const float* freq, int rot, const float* vfreq,
                              int num_tokens, int nh, int nkv, int d, int dv, int D, void* q, void* k, void* v,
                              long long ldq, long long ldkv, int out_dt, void* k_cache, void* v_cache,
                              const int* seq_end, const int* slots, const int* tables, int table_stride, int ring,
                              int page_size, int num_pages, int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1) || (rot > 0 && !freq) || d <= 0 || dv <= 0 || D < d || D < dv || !q || !k ||
        !v || ld < (nh + nkv) * d + nkv * dv || ldq < (long long)nh * D || ldkv < (long long)nkv * D)
        return (int)cudaErrorInvalidValue;
    if (k_cache && (!v_cache || !seq_end || !slots || !tables || !seq_of_token)) return (int)cudaErrorInvalidValue;
    const WholeCommit c{k_cache, v_cache, seq_end, slots, tables, table_stride, ring, page_size, num_pages};
    const size_t smem = (size_t)(rot + (vfreq ? (dv / 2) * 2 : 0) + 4) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    // from 128 tokens on the blocks fill the GPU anyway; fewer tokens are spread over more blocks
    const int hs_count = nh + 2 * nkv;
    const dim3 grid(num_tokens, num_tokens >= 128 ? 1 : min(hs_count, max(1, (hs_count + 3) / 4)));
    if (out_dt == DT_F32)
        return launch_pdl(whole_prepare_kernel<float>, grid, WP_THREADS, smem, stream, proj, ld, pos,
                          seq_of_token, q_norm, k_norm, eps, freq, rot, vfreq, nh, nkv, d, dv, D, (float*)q, (float*)k,
                          (float*)v, ldq, ldkv, c, status);
    return launch_pdl(whole_prepare_kernel<__nv_bfloat16>, grid, WP_THREADS, smem, stream, proj, ld, pos,
                      seq_of_token, q_norm, k_norm, eps, freq, rot, vfreq, nh, nkv, d, dv, D, (__nv_bfloat16*)q,
                      (__nv_bfloat16*)k, (__nv_bfloat16*)v, ldq, ldkv, c, status);
}

// ctx: [T, nh, D]; out: [T, nh * dv]; vfreq: [dv / 2].
MOE_API int moe_unrotate_pack(const void* ctx, const int* pos, const float* vfreq, int num_tokens, int nh, int dv,
                              int D, void* out, int dt, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (!ctx || !pos || !vfreq || !out || nh <= 0 || dv <= 0 || D < dv) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)((dv / 2) * 2 + 4) * sizeof(float);
    if (dt == DT_F32)
        return launch_pdl(unrotate_pack_kernel<float>, dim3(num_tokens), 128, smem, stream, (const float*)ctx, pos,
                          vfreq, nh, dv, D, (float*)out);
    return launch_pdl(unrotate_pack_kernel<__nv_bfloat16>, dim3(num_tokens), 128, smem, stream,
                      (const __nv_bfloat16*)ctx, pos, vfreq, nh, dv, D, (__nv_bfloat16*)out);
}
