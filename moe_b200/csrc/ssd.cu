// The recurrence of a state-space mixer with a scalar decay per head (Mamba-2) and what follows it.
//
//   ssd_scan    per sequence and head h (group g = h / (heads / groups)), tokens in order, with
//                 dt = softplus(dt_raw + dt_bias[h]),  a = exp(-exp(A_log[h]) * dt):
//                 S <- a S + dt B_t x_t^T   (S: [N, dv], 32-bit, the sequence's state)
//                 y_t = S^T C_t + D[h] x_t
//               x, B and C are columns of one 32-bit buffer (the convolution's output), dt_raw a column
//               block of the input projection.
//   ssd_finish  y * silu(z), then an RMS norm over each of `norm_groups` equal parts of the row
//               (x / sqrt(mean(x^2) + eps) * w), rounded to the activation dtype.
// Everything is 32-bit arithmetic; the state never leaves 32 bits.
#include "common.cuh"

namespace {

constexpr int SSD_COLS = 32;      // value columns a block
constexpr int SSD_NP = 8;         // threads that share a column's N rows
constexpr int SSD_TOK = 16;       // tokens staged at a time

__device__ __forceinline__ float softplus32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// grid (ceil(dv / 32), heads, sequences), 256 threads: thread (col = tid / 8, kp = tid % 8) holds rows
// kp, kp + 8, ... of column col of S in registers.
template <int RPT>
__global__ void __launch_bounds__(SSD_COLS * SSD_NP)
ssd_scan_kernel(const float* __restrict__ xbc, long long ldx, const float* __restrict__ dt_raw, long long lddt,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ dskip,
                float* __restrict__ state, long long state_pitch, const int* __restrict__ cu_seqlens,
                const int* __restrict__ slots, int heads, int groups, int N, int dv, float* __restrict__ y) {
    extern __shared__ __align__(16) float ssd_smem[];   // per staged token: B[N], C[N], x[32], dt, a
    const int rowlen = 2 * N + SSD_COLS + 2;
    const int tid = threadIdx.x, kp = tid & (SSD_NP - 1), cl = tid / SSD_NP;
    const int h = blockIdx.y, s = blockIdx.z, g = h / (heads / groups);
    const int col = blockIdx.x * SSD_COLS + cl;
    pdl_sync();
    const int tok0 = cu_seqlens[s], cnt = cu_seqlens[s + 1] - tok0;
    if (cnt <= 0) return;
    const int inner = heads * dv;
    float* S = state + (size_t)slots[s] * state_pitch + (size_t)h * N * dv;
    float sreg[RPT];
#pragma unroll
    for (int m = 0; m < RPT; m++) {
        const int n = kp + m * SSD_NP;
        sreg[m] = (n < N && col < dv) ? S[(size_t)n * dv + col] : 0.f;
    }
    const float bias = dt_bias[h], rate = expf(a_log[h]), skip = dskip[h];
    for (int t0 = 0; t0 < cnt; t0 += SSD_TOK) {
        const int nt = min(SSD_TOK, cnt - t0);
        __syncthreads();
        for (int idx = tid; idx < nt * rowlen; idx += blockDim.x) {
            const int tt = idx / rowlen, e = idx % rowlen;
            const size_t r = (size_t)(tok0 + t0 + tt);
            float v;
            if (e < N)
                v = xbc[r * ldx + inner + (size_t)g * N + e];
            else if (e < 2 * N)
                v = xbc[r * ldx + inner + (size_t)groups * N + (size_t)g * N + (e - N)];
            else if (e < 2 * N + SSD_COLS) {
                const int c = blockIdx.x * SSD_COLS + (e - 2 * N);
                v = c < dv ? xbc[r * ldx + (size_t)h * dv + c] : 0.f;
            } else {
                const float dt = softplus32(dt_raw[r * lddt + h] + bias);
                v = e == 2 * N + SSD_COLS ? dt : expf(-rate * dt);
            }
            ssd_smem[idx] = v;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float* row = ssd_smem + (size_t)tt * rowlen;
            const float xv = row[2 * N + cl], dt = row[2 * N + SSD_COLS], a = row[2 * N + SSD_COLS + 1];
            const float dx = dt * xv;
            float acc = 0.f;
#pragma unroll
            for (int m = 0; m < RPT; m++) {
                const int n = kp + m * SSD_NP;
                if (n < N) {
                    sreg[m] = fmaf(a, sreg[m], row[n] * dx);
                    acc = fmaf(row[N + n], sreg[m], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (kp == 0 && col < dv) y[(size_t)(tok0 + t0 + tt) * inner + (size_t)h * dv + col] = fmaf(skip, xv, acc);
        }
    }
#pragma unroll
    for (int m = 0; m < RPT; m++) {
        const int n = kp + m * SSD_NP;
        if (n < N && col < dv) S[(size_t)n * dv + col] = sreg[m];
    }
}

// A block per (token, part of the row).
template <typename OT>
__global__ void __launch_bounds__(256)
ssd_finish_kernel(const float* __restrict__ y, const float* __restrict__ z, long long ldz,
                  const float* __restrict__ norm_w, float eps, const int* __restrict__ seq_of_token, int inner,
                  int part, OT* __restrict__ out) {
    __shared__ float red[32];
    pdl_sync();
    const int t = blockIdx.x, c0 = blockIdx.y * part;
    OT* o = out + (size_t)t * inner + c0;
    if (seq_of_token[t] < 0) {
        for (int e = threadIdx.x; e < part; e += blockDim.x) st_f(o + e, 0.f);
        return;
    }
    const float* yr = y + (size_t)t * inner + c0;
    const float* zr = z + (size_t)t * ldz + c0;
    float ss = 0.f;
    for (int e = threadIdx.x; e < part; e += blockDim.x) {
        const float gate = zr[e];
        const float v = yr[e] * (gate / (1.0f + expf(-gate)));
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)part + eps);
    for (int e = threadIdx.x; e < part; e += blockDim.x) {
        const float gate = zr[e];
        st_f(o + e, yr[e] * (gate / (1.0f + expf(-gate))) * inv * norm_w[c0 + e]);
    }
}

}  // namespace

// xbc: [T, ldx] 32-bit, columns [x: heads * dv | B: groups * N | C: groups * N]; dt_raw: [T, lddt], a column
// per head; dt_bias, a_log, dskip: [heads]; state: per slot heads * N * dv floats ([head][n][v]) from the
// pointer given, rows of state_pitch floats; y: [T, heads * dv] 32-bit (rows of no sequence are left alone).
MOE_API int moe_ssd_scan(const float* xbc, long long ldx, const float* dt_raw, long long lddt, const float* dt_bias,
                         const float* a_log, const float* dskip, float* state, long long state_pitch,
                         const int* cu_seqlens, const int* slots, int num_seqs, int heads, int groups, int N, int dv,
                         float* y, cudaStream_t stream) {
    if (num_seqs <= 0) return 0;
    if (!xbc || !dt_raw || !dt_bias || !a_log || !dskip || !state || !y || heads <= 0 || groups <= 0 || heads % groups ||
        N <= 0 || N > 256 || dv <= 0 || ldx < (long long)heads * dv + 2LL * groups * N || lddt < heads ||
        state_pitch < (long long)heads * N * dv || heads > 65535 || num_seqs > 65535)
        return (int)cudaErrorInvalidValue;
    const dim3 grid((dv + SSD_COLS - 1) / SSD_COLS, heads, num_seqs);
    const size_t smem = (size_t)SSD_TOK * (2 * N + SSD_COLS + 2) * sizeof(float);
#define SCAN(RPT_)                                                                                                  \
    return launch_pdl(ssd_scan_kernel<RPT_>, grid, dim3(SSD_COLS * SSD_NP), smem, stream, xbc, ldx, dt_raw, lddt,    \
                      dt_bias, a_log, dskip, state, state_pitch, cu_seqlens, slots, heads, groups, N, dv, y)
    if (N <= 32) SCAN(4);
    if (N <= 64) SCAN(8);
    if (N <= 128) SCAN(16);
    SCAN(32);
#undef SCAN
}

// y: [T, inner] 32-bit; z: the gate's columns of the input projection, row pitch ldz; norm_w: [inner];
// out: [T, inner] in out_dt.  inner must be a multiple of norm_groups.
MOE_API int moe_ssd_finish(const float* y, const float* z, long long ldz, const float* norm_w, float eps,
                           const int* seq_of_token, int num_tokens, int inner, int norm_groups, void* out, int out_dt,
                           cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (!y || !z || !norm_w || !out || !seq_of_token || inner <= 0 || norm_groups <= 0 || inner % norm_groups ||
        ldz < inner || norm_groups > 65535)
        return (int)cudaErrorInvalidValue;
    const dim3 grid(num_tokens, norm_groups);
    if (out_dt == DT_F32)
        return launch_pdl(ssd_finish_kernel<float>, grid, dim3(256), 0, stream, y, z, ldz, norm_w, eps, seq_of_token,
                          inner, inner / norm_groups, (float*)out);
    return launch_pdl(ssd_finish_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, y, z, ldz, norm_w, eps,
                      seq_of_token, inner, inner / norm_groups, (__nv_bfloat16*)out);
}
