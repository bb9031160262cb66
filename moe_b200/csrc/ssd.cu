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
//               Few, long sequences leave most SMs idle and the chain over the tokens long, so a sequence's
//               tokens may be cut into `segs` segments that run side by side (the decay is one number a
//               head and step, so a segment's effect on what follows is its own end state from a zero
//               start, E, and the product of its decays, A):
//                 phase 1  every segment but a sequence's last: E and A into a workspace, no outputs
//                 phase 2  every segment: its start state S <- A_q S + E_q over the segments q before it,
//                          begun from the sequence's state, then the recurrence with outputs; the last
//                          segment that holds tokens writes the state back
//               which changes the order of additions, nothing else.
// Everything is 32-bit arithmetic; the state never leaves 32 bits.
#include "common.cuh"

namespace {

constexpr int SSD_CPT = 4;        // value columns a thread
constexpr int SSD_CG = 16;        // column groups a block: 64 columns
constexpr int SSD_COLS = SSD_CPT * SSD_CG;

__device__ __forceinline__ float softplus32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// grid (ceil(dv / 64), heads, sequences), KP * 16 threads: thread (kp = tid % KP, cg = tid / KP) holds rows
// kp * RPT ... kp * RPT + RPT - 1 of four neighbouring columns of S in registers (KP * RPT >= N; rows beyond
// N stay zero).  A run of SSD_TOK tokens is staged in shared memory as [B | C | the block's columns of x |
// dt | decay] a token (SSD_TOK: tokens staged at a time), the next run's loads in flight while this one is
// worked on; within a run the chain over the tokens has no barrier.
struct SsdSegments {
    int segs;          // segments a sequence (1: none of this)
    int seg_len;       // tokens a segment (a multiple of the staged run)
    int phase;         // 0: the whole sequence in one go; 1, 2: see the head of this file
    float* ends;       // [sequence][segment][head][N][dv]: a segment's end state from a zero start
    float* decays;     // [sequence][segment][head]: the product of its decays
};

// PHASE (of SsdSegments) is known when compiled, so that the plain chain carries nothing of the other two.
template <int RPT, int KP, int SSD_TOK, int PHASE>
__global__ void __launch_bounds__(KP * SSD_CG)
ssd_scan_kernel(const float* __restrict__ xbc, long long ldx, const float* __restrict__ dt_raw, long long lddt,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ dskip,
                float* __restrict__ state, long long state_pitch, const int* __restrict__ cu_seqlens,
                const int* __restrict__ slots, int heads, int groups, int N, int dv, float* __restrict__ y,
                const SsdSegments sg) {
    constexpr int NP = RPT * KP, THREADS = KP * SSD_CG;
    constexpr int PER_TOK = 2 * NP + SSD_COLS + 2;
    constexpr int ROWLEN = (PER_TOK + 3) & ~3;
    constexpr int XPT = (PER_TOK + THREADS - 1) / THREADS;
    __shared__ __align__(16) float sm[SSD_TOK * ROWLEN];
    const int tid = threadIdx.x, kp = tid % KP, cg = tid / KP;
    const int h = blockIdx.y, s = blockIdx.z / sg.segs, seg = blockIdx.z % sg.segs, g = h / (heads / groups);
    const int c0 = blockIdx.x * SSD_COLS, col = c0 + cg * SSD_CPT;
    pdl_sync();
    const int seq_tok0 = cu_seqlens[s], seq_cnt = cu_seqlens[s + 1] - seq_tok0;
    // this block's tokens: the sequence's, or one segment of them
    const int tok0 = seq_tok0 + seg * sg.seg_len;
    const int cnt = sg.segs > 1 ? min(sg.seg_len, seq_cnt - seg * sg.seg_len) : seq_cnt;
    if (cnt <= 0) return;
    const bool last_seg = sg.segs == 1 || (seg + 1) * sg.seg_len >= seq_cnt;       // the last one that holds tokens
    if (PHASE == 1 && last_seg) return;                                         // nothing comes after it
    const int inner = heads * dv;
    float* S = state + (size_t)slots[s] * state_pitch + (size_t)h * N * dv;
    const size_t plane = (size_t)N * dv;
    float* ends = sg.ends ? sg.ends + ((size_t)s * sg.segs * heads + h) * plane : nullptr;      // + segment * heads * plane
    float* decays = sg.decays ? sg.decays + (size_t)s * sg.segs * heads + h : nullptr;           // + segment * heads
    const bool vec = (dv % 4 == 0) && (((uintptr_t)S) % 16 == 0) && (state_pitch % 4 == 0) && (((uintptr_t)sg.ends) % 16 == 0);
    float sreg[RPT][SSD_CPT];
#pragma unroll
    for (int m = 0; m < RPT; m++) {
        const int n = kp * RPT + m;
        if (PHASE != 1 && vec && n < N && col < dv) {
            const float4 t4 = *reinterpret_cast<const float4*>(S + (size_t)n * dv + col);
            sreg[m][0] = t4.x, sreg[m][1] = t4.y, sreg[m][2] = t4.z, sreg[m][3] = t4.w;
        } else {
#pragma unroll
            for (int c = 0; c < SSD_CPT; c++)
                sreg[m][c] = (PHASE != 1 && n < N && col + c < dv) ? S[(size_t)n * dv + col + c] : 0.f;
        }
    }
    if (PHASE == 2)       // the segments before this one, in order: S <- A_q S + E_q
        for (int q = 0; q < seg; q++) {
            const float aq = decays[(size_t)q * heads];
            const float* eq = ends + (size_t)q * heads * plane;
#pragma unroll
            for (int m = 0; m < RPT; m++) {
                const int n = kp * RPT + m;
#pragma unroll
                for (int c = 0; c < SSD_CPT; c++)
                    if (n < N && col + c < dv) sreg[m][c] = fmaf(aq, sreg[m][c], eq[(size_t)n * dv + col + c]);
            }
        }
    float decay_product = 1.f;
    const float bias = dt_bias[h], rate = expf(a_log[h]), skip = dskip[h];
    const size_t b_at = (size_t)inner + (size_t)g * N, c_at = (size_t)inner + (size_t)groups * N + (size_t)g * N;
    // What this thread brings into shared memory of every token: elements x = tid, tid + THREADS, ... of
    // [B | C | the block's columns of x | dt | decay]; where each comes from is worked out once.
    const float* src[XPT];
    long long pitch[XPT];
#pragma unroll
    for (int e = 0; e < XPT; e++) {
        const int x = tid + e * THREADS;
        src[e] = nullptr, pitch[e] = 0;
        if (x < NP) {
            if (x < N) src[e] = xbc + (size_t)tok0 * ldx + b_at + x, pitch[e] = ldx;
        } else if (x < 2 * NP) {
            if (x - NP < N) src[e] = xbc + (size_t)tok0 * ldx + c_at + (x - NP), pitch[e] = ldx;
        } else if (x < 2 * NP + SSD_COLS) {
            const int c = c0 + x - 2 * NP;
            if (c < dv) src[e] = xbc + (size_t)tok0 * ldx + (size_t)h * dv + c, pitch[e] = ldx;
        } else if (x < PER_TOK) {
            src[e] = dt_raw + (size_t)tok0 * lddt + h, pitch[e] = lddt;      // turned into dt or the decay when it is stored
        }
    }
    float ahead[SSD_TOK][XPT];
    auto fetch = [&](int t0) {
        const int nt = min(SSD_TOK, cnt - t0);
#pragma unroll
        for (int tt = 0; tt < SSD_TOK; tt++) {
            const long long r = t0 + min(tt, nt - 1);
#pragma unroll
            for (int e = 0; e < XPT; e++) ahead[tt][e] = src[e] ? src[e][r * pitch[e]] : 0.f;
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < cnt; t0 += SSD_TOK) {
        const int nt = min(SSD_TOK, cnt - t0);
        __syncthreads();                     // the run before is no longer read
#pragma unroll
        for (int tt = 0; tt < SSD_TOK; tt++)
#pragma unroll
            for (int e = 0; e < XPT; e++) {
                const int x = tid + e * THREADS;
                if (x < PER_TOK) {
                    float val = ahead[tt][e];
                    if (x >= 2 * NP + SSD_COLS) {
                        const float dt = softplus32(val + bias);
                        val = x == 2 * NP + SSD_COLS ? dt : expf(-rate * dt);
                    }
                    sm[tt * ROWLEN + x] = val;
                }
            }
        __syncthreads();
        if (t0 + SSD_TOK < cnt) fetch(t0 + SSD_TOK);
#pragma unroll 2
        for (int tt = 0; tt < nt; tt++) {
            const float* row = sm + tt * ROWLEN;
            const float4 x4 = *reinterpret_cast<const float4*>(row + 2 * NP + cg * SSD_CPT);
            const float dt = row[2 * NP + SSD_COLS], a = row[2 * NP + SSD_COLS + 1];
            const float xv[SSD_CPT] = {x4.x, x4.y, x4.z, x4.w};
            const float dx[SSD_CPT] = {dt * x4.x, dt * x4.y, dt * x4.z, dt * x4.w};
            if (PHASE == 1) {         // the end state and the decays' product alone
                decay_product *= a;
#pragma unroll
                for (int m = 0; m < RPT; m++) {
                    const float bm = row[kp * RPT + m];
#pragma unroll
                    for (int c = 0; c < SSD_CPT; c++) sreg[m][c] = fmaf(a, sreg[m][c], bm * dx[c]);
                }
                continue;
            }
            float acc[2][SSD_CPT] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};      // two chains a column
#pragma unroll
            for (int m0 = 0; m0 < RPT; m0 += 4) {
                const float4 b4 = *reinterpret_cast<const float4*>(row + kp * RPT + m0);
                const float4 c4 = *reinterpret_cast<const float4*>(row + NP + kp * RPT + m0);
                const float bi[4] = {b4.x, b4.y, b4.z, b4.w}, ci[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                for (int z = 0; z < 4; z++)
#pragma unroll
                    for (int c = 0; c < SSD_CPT; c++) {
                        sreg[m0 + z][c] = fmaf(a, sreg[m0 + z][c], bi[z] * dx[c]);
                        acc[z & 1][c] = fmaf(ci[z], sreg[m0 + z][c], acc[z & 1][c]);
                    }
            }
            // the KP threads of a column group add up their parts; on the way every thread drops the
            // columns another one carries on (4 shuffles instead of 12): lane bits 0 and 1 of kp say which
            // column's sum it ends with
            const bool b0 = (kp & 1) != 0, b1 = (kp & 2) != 0;
            float v0, v1;
            {
                const float p0 = acc[0][0] + acc[1][0], p1 = acc[0][1] + acc[1][1];
                const float p2 = acc[0][2] + acc[1][2], p3 = acc[0][3] + acc[1][3];
                v0 = (b0 ? p2 : p0) + __shfl_xor_sync(0xffffffffu, b0 ? p0 : p2, 1);
                v1 = (b0 ? p3 : p1) + __shfl_xor_sync(0xffffffffu, b0 ? p1 : p3, 1);
            }
            v0 = (b1 ? v1 : v0) + __shfl_xor_sync(0xffffffffu, b1 ? v0 : v1, 2);
#pragma unroll
            for (int off = 4; off < KP; off <<= 1) v0 += __shfl_xor_sync(0xffffffffu, v0, off);
            if (kp < 4) {
                const int c = (b0 ? 2 : 0) + (b1 ? 1 : 0);
                const float xc = b0 ? (b1 ? xv[3] : xv[2]) : (b1 ? xv[1] : xv[0]);
                if (col + c < dv) y[(size_t)(tok0 + t0 + tt) * inner + (size_t)h * dv + col + c] = fmaf(skip, xc, v0);
            }
        }
    }
    if (PHASE == 2 && !last_seg) return;          // only the sequence's last segment leaves the state behind
    if (PHASE == 1) {
        S = ends + (size_t)seg * heads * plane;
        if (tid == 0) decays[(size_t)seg * heads] = decay_product;
    }
#pragma unroll
    for (int m = 0; m < RPT; m++) {
        const int n = kp * RPT + m;
        if (n >= N) continue;
        if (vec && col < dv) {
            *reinterpret_cast<float4*>(S + (size_t)n * dv + col) = make_float4(sreg[m][0], sreg[m][1], sreg[m][2], sreg[m][3]);
        } else {
#pragma unroll
            for (int c = 0; c < SSD_CPT; c++)
                if (col + c < dv) S[(size_t)n * dv + col + c] = sreg[m][c];
        }
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
                         float* y, int segs, int seg_len, float* ends, float* decays, cudaStream_t stream) {
    if (num_seqs <= 0) return 0;
    if (!xbc || !dt_raw || !dt_bias || !a_log || !dskip || !state || !y || heads <= 0 || groups <= 0 || heads % groups ||
        N <= 0 || N > 512 || dv <= 0 || ldx < (long long)heads * dv + 2LL * groups * N || lddt < heads ||
        state_pitch < (long long)heads * N * dv || heads > 65535 || num_seqs > 65535)
        return (int)cudaErrorInvalidValue;
    if (segs < 1 || (segs > 1 && (!ends || !decays || seg_len <= 0 || seg_len % 16 || (long long)num_seqs * segs > 65535)))
        return (int)cudaErrorInvalidValue;
    const dim3 grid((dv + SSD_COLS - 1) / SSD_COLS, heads, num_seqs * segs);
    // one launch, or phase 1 and then phase 2 of the segmented form
    for (int phase = segs > 1 ? 1 : 0; phase <= (segs > 1 ? 2 : 0); phase++) {
        const SsdSegments sg{segs, seg_len, phase, ends, decays};
        int code;
#define SCAN_P(RPT_, KP_, TOK_, PH_)                                                                                    \
    code = launch_pdl(ssd_scan_kernel<RPT_, KP_, TOK_, PH_>, grid, dim3(KP_ * SSD_CG), 0, stream, xbc, ldx, dt_raw, lddt,    \
                      dt_bias, a_log, dskip, state, state_pitch, cu_seqlens, slots, heads, groups, N, dv, y, sg)
#define SCAN(RPT_, KP_, TOK_)                                                                                          \
    do {                                                                                                               \
        if (phase == 0) SCAN_P(RPT_, KP_, TOK_, 0);                                                                    \
        else if (phase == 1) SCAN_P(RPT_, KP_, TOK_, 1);                                                               \
        else SCAN_P(RPT_, KP_, TOK_, 2);                                                                               \
    } while (0)
        if (N <= 32) SCAN(4, 8, 16);
        else if (N <= 64) SCAN(8, 8, 16);
        else if (N <= 128) SCAN(16, 8, 16);
        else if (N <= 256) SCAN(16, 16, 16);
        else SCAN(32, 16, 8);
#undef SCAN
#undef SCAN_P
        if (code) return code;
    }
    return 0;
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
