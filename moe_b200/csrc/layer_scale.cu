// The residual sum of a layer whose two sublayers read the same normed input and whose outputs are
// scaled per channel before they join the stream, fused with the RMS norm that follows:
//
//   v = x[r] + a[r] * sa + b[r] * sb      (b and sb may be null: one sublayer)
//   if write_back: x[r] = v               (the 32-bit residual stream)
//   y = v / sqrt(mean(v^2) + eps) * w;  out32[i] = y;  out16[i] = bf16(y)
//   with w2: out32b[i] = v / sqrt(mean(v^2) + eps) * w2, a second norm of the same row (one statistic)
// b may still be the uncombined output of routed experts (ScaledCombine),
//   b[t] = sum_j w[t, j] * y[pos[t, j]] + shared[t],
// added up here in the order of moe_combine_kernel in moe.cu, which spares that launch and a pass.
//
// One block per output row i; source row r = rows ? rows[i] : i.  The row is held in shared memory
// so that the stream and both outputs are read once.  Sum and norm are 32-bit.
#include "common.cuh"

namespace {

// The second sublayer's output as routed experts left it (y null: b is a plain tensor).
struct ScaledCombine {
    const float* y;        // [pairs, hidden]
    const int* pos;        // [T, top_k], -1: no expert
    const float* w;        // [T, top_k]
    int top_k;
    const float* shared;   // [T, hidden] or null
};

__device__ __forceinline__ float combined(const ScaledCombine& cs, int r, int hidden, int j) {
    float acc = 0.f;
    for (int q = 0; q < cs.top_k; q++) {
        const int p = cs.pos[(size_t)r * cs.top_k + q];
        if (p >= 0) acc = fmaf(cs.w[(size_t)r * cs.top_k + q], cs.y[(size_t)p * hidden + j], acc);
    }
    if (cs.shared) acc += cs.shared[(size_t)r * hidden + j];
    return acc;
}

template <bool VEC>
__global__ void __launch_bounds__(512)
rmsnorm_scaled_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ sa,
                      const float* __restrict__ b, const float* __restrict__ sb, const float* __restrict__ w,
                      const int* __restrict__ rows, float* __restrict__ out32, __nv_bfloat16* __restrict__ out16,
                      int hidden, float eps, int write_back, int num_src_rows, int* status, const ScaledCombine cs,
                      const float* __restrict__ w2, float* __restrict__ out32b) {
    extern __shared__ __align__(16) float row[];
    __shared__ float red[32];
    const int i = blockIdx.x;
    pdl_sync();
    int r = rows ? rows[i] : i;
    if (r < 0 || r >= num_src_rows) {
        if (threadIdx.x == 0 && status) atomicOr(status, ST_BAD_ROW);
        r = 0;
    }
    float* xr = x + (size_t)r * hidden;
    const float* ar = a + (size_t)r * hidden;
    const float* br = b ? b + (size_t)r * hidden : nullptr;
    float ss = 0.f;
    if (VEC) {
        for (int j = threadIdx.x; j < hidden / 4; j += blockDim.x) {
            float4 v = reinterpret_cast<const float4*>(xr)[j];
            const float4 av = reinterpret_cast<const float4*>(ar)[j], as = reinterpret_cast<const float4*>(sa)[j];
            v.x = fmaf(av.x, as.x, v.x), v.y = fmaf(av.y, as.y, v.y), v.z = fmaf(av.z, as.z, v.z), v.w = fmaf(av.w, as.w, v.w);
            if (br || cs.y) {
                float4 bv;
                if (cs.y) {
                    bv = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int q = 0; q < cs.top_k; q++) {
                        const int p = cs.pos[(size_t)r * cs.top_k + q];
                        if (p >= 0) {
                            const float4 yv = *reinterpret_cast<const float4*>(cs.y + (size_t)p * hidden + 4 * j);
                            const float wq = cs.w[(size_t)r * cs.top_k + q];
                            bv.x = fmaf(wq, yv.x, bv.x), bv.y = fmaf(wq, yv.y, bv.y), bv.z = fmaf(wq, yv.z, bv.z), bv.w = fmaf(wq, yv.w, bv.w);
                        }
                    }
                    if (cs.shared) {
                        const float4 sv = *reinterpret_cast<const float4*>(cs.shared + (size_t)r * hidden + 4 * j);
                        bv.x += sv.x, bv.y += sv.y, bv.z += sv.z, bv.w += sv.w;
                    }
                } else {
                    bv = reinterpret_cast<const float4*>(br)[j];
                }
                const float4 bs = reinterpret_cast<const float4*>(sb)[j];
                v.x = fmaf(bv.x, bs.x, v.x), v.y = fmaf(bv.y, bs.y, v.y), v.z = fmaf(bv.z, bs.z, v.z), v.w = fmaf(bv.w, bs.w, v.w);
            }
            if (write_back) reinterpret_cast<float4*>(xr)[j] = v;
            reinterpret_cast<float4*>(row)[j] = v;
            ss += v.x * v.x, ss += v.y * v.y, ss += v.z * v.z, ss += v.w * v.w;
        }
    } else {
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
            float v = fmaf(ar[j], sa[j], xr[j]);
            if (cs.y) v = fmaf(combined(cs, r, hidden, j), sb[j], v);
            else if (br) v = fmaf(br[j], sb[j], v);
            if (write_back) xr[j] = v;
            row[j] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    if (VEC) {
        for (int j = threadIdx.x; j < hidden / 4; j += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(row)[j], g = reinterpret_cast<const float4*>(w)[j];
            const float4 y = make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
            if (out32) reinterpret_cast<float4*>(out32 + (size_t)i * hidden)[j] = y;
            if (out16) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
                uint2 u;
                u.x = *reinterpret_cast<unsigned*>(&lo), u.y = *reinterpret_cast<unsigned*>(&hi);
                reinterpret_cast<uint2*>(out16 + (size_t)i * hidden)[j] = u;
            }
            if (w2) {       // a second norm of the same row: the same statistic, another weight
                const float4 g2 = reinterpret_cast<const float4*>(w2)[j];
                reinterpret_cast<float4*>(out32b + (size_t)i * hidden)[j] =
                    make_float4(v.x * scale * g2.x, v.y * scale * g2.y, v.z * scale * g2.z, v.w * scale * g2.w);
            }
        }
        return;
    }
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        const float y = row[j] * scale * w[j];
        if (out32) out32[(size_t)i * hidden + j] = y;
        if (out16) out16[(size_t)i * hidden + j] = __float2bfloat16_rn(y);
        if (w2) out32b[(size_t)i * hidden + j] = row[j] * scale * w2[j];
    }
}

}  // namespace

MOE_API int moe_rmsnorm_scaled(float* x, const float* a, const float* sa, const float* b, const float* sb,
                               const float* w, const int* rows, float* out32, void* out16, int num_out_rows,
                               int num_src_rows, int hidden, float eps, int write_back, int* status,
                               const float* cy, const int* cpos, const float* cw, int top_k, const float* cshared,
                               const float* w2, float* out32b, cudaStream_t stream) {
    if (num_out_rows <= 0) return 0;
    if (!x || !a || !sa || !w || ((b || cy) && !sb) || (b && cy) || (cy && (!cpos || !cw || top_k <= 0)) || hidden <= 0 ||
        (w2 && !out32b))
        return (int)cudaErrorInvalidValue;
    const ScaledCombine cs{cy, cpos, cw, top_k, cshared};
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    auto al = [](const void* p, size_t n) { return ((uintptr_t)p % n) == 0; };
    const bool vec = hidden % 4 == 0 && al(x, 16) && al(a, 16) && al(sa, 16) && al(b, 16) && al(sb, 16) && al(w, 16) &&
                     al(out32, 16) && al(out16, 8) && al(cy, 16) && al(cshared, 16) && al(w2, 16) && al(out32b, 16);
    if (smem > 48 * 1024) {
        const cudaError_t e = vec ? cudaFuncSetAttribute(rmsnorm_scaled_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                  : cudaFuncSetAttribute(rmsnorm_scaled_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (vec)
        return launch_pdl(rmsnorm_scaled_kernel<true>, dim3(num_out_rows), threads, smem, stream, x, a, sa, b, sb, w, rows,
                          out32, (__nv_bfloat16*)out16, hidden, eps, write_back, num_src_rows, status, cs, w2, out32b);
    return launch_pdl(rmsnorm_scaled_kernel<false>, dim3(num_out_rows), threads, smem, stream, x, a, sa, b, sb, w, rows,
                      out32, (__nv_bfloat16*)out16, hidden, eps, write_back, num_src_rows, status, cs, w2, out32b);
}
