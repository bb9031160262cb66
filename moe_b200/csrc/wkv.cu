// A recurrent mixer with a matrix-valued state per head and data-dependent decay (RWKV-style time
// mixing).  Three kernels around the projections:
//
//   wkv_shift_mix   every projection reads its own blend of the token's input n_t and the previous
//                   token's n_(t-1):  x_s = n_t + (n_(t-1) - n_t) * mu_s  for s of `streams` blends.
//                   The previous token of a step's first row is the sequence's state (zeros at
//                   position 0); the block of that row also stores the sequence's LAST row of the
//                   step as the new state (it alone reads the old one, element by element before it
//                   writes).  The last blend may go to a 32-bit buffer of its own (the decay's), or be
//                   turned into the decay in the same kernel (a narrow projection of up to 32).
//   wkv_decay       w_t[i] = exp(-exp(w0[i] + sum_q W2[i][q] tanh(low_t[q]))), low = W1 x_w being the
//                   decay's first, narrow projection: the second projection, its bias and both
//                   exponentials in one pass, 32-bit.
//   wkv_scan        per (sequence, head), tokens in order:
//                       o_t[j] = sum_i r_t[i] (S[i][j] + u[i] k_t[i] v_t[j])
//                       S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j]
//                   S lives in 32-bit floats in the sequence's state and is
//                   held in registers over the step: a block owns 64 value columns j of one head, a
//                   thread four neighbouring ones, eight lanes share them (a run of rows each),
//                   and the eight partial sums of o_t[j] are added by shuffles in a fixed order.  r, k,
//                   the decay and the block's columns of v pass through shared memory a few tokens
//                   at a time, the next run's loads in flight while a run is worked on.
//   wkv_finish      each head's o_t is divided by its root mean square (x / sqrt(mean(x^2) + eps)),
//                   multiplied by a weight per channel and by silu(gate projection), and rounded to
//                   the activation dtype for the output projection.
// Everything here is 32-bit arithmetic; only wkv_shift_mix and wkv_finish round their stores.
#include "common.cuh"

namespace {

constexpr int SCAN_KP = 8, SCAN_CPT = 4, SCAN_THREADS = 128, SCAN_BCOLS = SCAN_THREADS / SCAN_KP * SCAN_CPT;
// tokens of a run through shared memory: fewer for the largest heads, whose state fills the registers
__host__ __device__ constexpr int scan_tok(int rpt) { return rpt >= 32 ? 4 : 8; }

constexpr int FUSED_RANK = 32;       // widest narrow projection that the blends' kernel forms itself
struct DecayArgs {                   // the decay formed in the blends' kernel (w1 null: not)
    const float* w1;                 // [rank, width]
    const float* w2t;                // [rank, inner]
    const float* w0;                 // [inner]
    float* out;                      // [T, inner]
    int rank, inner;
};

// DECAY: the block also forms the token's decay: the last blend never leaves the registers; its narrow
// projection is added up per thread, then over the block; tanh; the second projection, a thread a channel.
template <typename OT, bool DECAY>
__global__ void __launch_bounds__(256)
wkv_shift_mix_kernel(const float* __restrict__ h, const float* __restrict__ mu, int streams, float* __restrict__ state,
                     long long state_pitch, const int* __restrict__ seq_of_token, const int* __restrict__ pos,
                     const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int num_tokens, int width,
                     OT* __restrict__ out, float* __restrict__ last32, const DecayArgs da) {
    __shared__ float part[8][FUSED_RANK];
    __shared__ float th[FUSED_RANK];
    pdl_sync();
    const int t = blockIdx.x;
    const int s = seq_of_token[t];
    const size_t plane = (size_t)num_tokens * width;
    const int planes = streams - ((last32 || DECAY) ? 1 : 0);        // blends that go to `out`
    if (s < 0) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            for (int m = 0; m < planes; m++) st_f(out + m * plane + (size_t)t * width + c, 0.f);
            if (last32) last32[(size_t)t * width + c] = 0.f;
        }
        return;
    }
    const int tok0 = cu_seqlens[s], last = cu_seqlens[s + 1] - 1;
    const bool first = t == tok0;
    float* st = state + (size_t)slots[s] * state_pitch;
    const bool from_zero = pos[t] == 0;
    float acc[DECAY ? FUSED_RANK : 1];
#pragma unroll
    for (int q = 0; q < (DECAY ? FUSED_RANK : 1); q++) acc[q] = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float x = h[(size_t)t * width + c];
        float prev;
        if (first) {
            prev = from_zero ? 0.f : st[c];
            st[c] = h[(size_t)last * width + c];
        } else {
            prev = h[(size_t)(t - 1) * width + c];
        }
        const float diff = prev - x;
        for (int m = 0; m < streams; m++) {
            const float y = fmaf(diff, mu[(size_t)m * width + c], x);
            if (m < planes) {
                st_f(out + m * plane + (size_t)t * width + c, y);
            } else if (DECAY) {
#pragma unroll
                for (int q = 0; q < FUSED_RANK; q++)
                    if (q < da.rank) acc[q] = fmaf(y, da.w1[(size_t)q * width + c], acc[q]);
            } else {
                last32[(size_t)t * width + c] = y;
            }
        }
    }
    if (!DECAY) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int q = 0; q < FUSED_RANK; q++)
        if (q < da.rank) {
            const float v = warp_sum(acc[q]);
            if (lane == 0) part[warp][q] = v;
        }
    __syncthreads();
    if (threadIdx.x < da.rank) {
        float v = 0.f;
        for (int w = 0; w < 8; w++) v += part[w][threadIdx.x];       // fixed order
        th[threadIdx.x] = tanhf(v);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < da.inner; c += blockDim.x) {
        float a = 0.f;
        for (int q = 0; q < da.rank; q++) a = fmaf(da.w2t[(size_t)q * da.inner + c], th[q], a);
        da.out[(size_t)t * da.inner + c] = expf(-expf(a + da.w0[c]));
    }
}

constexpr int MAX_RANK = 256, DECAY_TOK = 8;
// One block per DECAY_TOK tokens: their narrow rows through tanh into shared memory, then a thread a
// channel, which reads its column of the transposed second projection once for all the block's tokens
// (w2t: [rank, inner], so that neighbouring threads read neighbouring addresses).
__global__ void __launch_bounds__(256)
wkv_decay_kernel(const float* __restrict__ low, const float* __restrict__ w2t, const float* __restrict__ w0,
                 int num_tokens, int inner, int rank, float* __restrict__ out) {
    extern __shared__ float th[];            // [DECAY_TOK][rank]
    pdl_sync();
    const int t0 = blockIdx.x * DECAY_TOK, nt = min(DECAY_TOK, num_tokens - t0);
    for (int i = threadIdx.x; i < nt * rank; i += blockDim.x) th[i] = tanhf(low[(size_t)t0 * rank + i]);
    __syncthreads();
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < inner; c += gridDim.y * blockDim.x) {
        float acc[DECAY_TOK];
#pragma unroll
        for (int j = 0; j < DECAY_TOK; j++) acc[j] = 0.f;
        for (int q = 0; q < rank; q++) {
            const float w = w2t[(size_t)q * inner + c];
#pragma unroll
            for (int j = 0; j < DECAY_TOK; j++) acc[j] = fmaf(w, j < nt ? th[j * rank + q] : 0.f, acc[j]);
        }
        const float b0 = w0[c];
#pragma unroll
        for (int j = 0; j < DECAY_TOK; j++)
            if (j < nt) out[(size_t)(t0 + j) * inner + c] = expf(-expf(acc[j] + b0));
    }
}

// Few, long sequences leave most SMs idle and the chain over the tokens long, so a sequence's tokens may
// be cut into `segs` segments that run side by side.  The decay acts on a row of the state at a time, so a
// segment's effect on what follows is its own end state from a zero start, E [d][d], and the product of
// its decays per row, A [d]:
//   phase 1  every segment but a sequence's last: E and A into a workspace, no outputs
//   phase 2  every segment: its start state S <- diag(A_q) S + E_q over the segments q before it, begun
//            from the sequence's state, then the recurrence with outputs; the last segment that holds
//            tokens writes the state back
// which changes the order of additions, nothing else.
struct WkvSegments {
    int segs;          // segments a sequence (1: none of this)
    int seg_len;       // tokens a segment (a multiple of 8)
    int phase;         // 0: the whole sequence in one go; 1, 2: see above
    float* ends;       // [sequence][segment][head][d][d]
    float* decays;     // [sequence][segment][head][d]
};

// A thread owns CPT = 4 neighbouring value columns and the rows i = kp + 8 m of them; a warp covers 16
// columns, a block of four warps 64.  VEC: the state's rows are read and written 16 bytes at a time.
template <int RPT, bool VEC>
__global__ void __launch_bounds__(SCAN_THREADS)
wkv_scan_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                const float* __restrict__ w, long long ld, const float* __restrict__ u, float* __restrict__ state,
                long long state_pitch, const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int heads,
                int d, float* __restrict__ out, const WkvSegments sg) {
    constexpr int SCAN_TOK = scan_tok(RPT);
    extern __shared__ __align__(16) float scan_smem[];     // [SCAN_TOK][3 d + SCAN_BCOLS]: r, k, decay, v of the block's columns
    pdl_sync();
    const int seq = blockIdx.z / sg.segs, seg = blockIdx.z % sg.segs, head = blockIdx.y;
    const int seq_tok0 = cu_seqlens[seq], seq_cnt = cu_seqlens[seq + 1] - seq_tok0;
    // this block's tokens: the sequence's, or one segment of them
    const int tok0 = seq_tok0 + seg * sg.seg_len;
    const int cnt = sg.segs > 1 ? min(sg.seg_len, seq_cnt - seg * sg.seg_len) : seq_cnt;
    if (cnt <= 0) return;
    const bool last_seg = sg.segs == 1 || (seg + 1) * sg.seg_len >= seq_cnt;       // the last one that holds tokens
    if (sg.phase == 1 && last_seg) return;                                         // nothing comes after it
    const int kp = threadIdx.x % SCAN_KP, cg = threadIdx.x / SCAN_KP;      // row group, column group
    const int c0 = blockIdx.x * SCAN_BCOLS;                                // the block's first column
    const int col = c0 + cg * SCAN_CPT;                                    // this thread's first column
    const size_t hc = (size_t)head * d;
    const int rowlen = 3 * d + SCAN_BCOLS;
    float* S = state + (size_t)slots[seq] * state_pitch + hc * d;          // [d (i)][d (j)] of this head
    float sreg[RPT][SCAN_CPT], ureg[RPT];
    const size_t plane = (size_t)d * d;
    float* ends = sg.ends ? sg.ends + ((size_t)seq * sg.segs * heads + head) * plane : nullptr;      // + segment * heads * plane
    float* decays = sg.decays ? sg.decays + ((size_t)seq * sg.segs * heads + head) * d : nullptr;     // + segment * heads * d
#pragma unroll
    for (int m = 0; m < RPT; m++) {
        const int i = kp * RPT + m;
        ureg[m] = i < d ? u[hc + i] : 0.f;
        if (sg.phase == 1) {
#pragma unroll
            for (int c = 0; c < SCAN_CPT; c++) sreg[m][c] = 0.f;
        } else if (VEC && i < d && col < d) {
            const float4 t4 = *reinterpret_cast<const float4*>(S + (size_t)i * d + col);
            sreg[m][0] = t4.x, sreg[m][1] = t4.y, sreg[m][2] = t4.z, sreg[m][3] = t4.w;
        } else {
#pragma unroll
            for (int c = 0; c < SCAN_CPT; c++) sreg[m][c] = (i < d && col + c < d) ? S[(size_t)i * d + col + c] : 0.f;
        }
    }
    if (sg.phase == 2)       // the segments before this one, in order: S <- diag(A_q) S + E_q
        for (int q = 0; q < seg; q++) {
            const float* aq = decays + (size_t)q * heads * d;
            const float* eq = ends + (size_t)q * heads * plane;
#pragma unroll
            for (int m = 0; m < RPT; m++) {
                const int i = kp * RPT + m;
                if (i >= d) continue;
                const float ai = aq[i];
#pragma unroll
                for (int c = 0; c < SCAN_CPT; c++)
                    if (col + c < d) sreg[m][c] = fmaf(ai, sreg[m][c], eq[(size_t)i * d + col + c]);
            }
        }
    float wprod[RPT];        // phase 1: the product of this thread's rows' decays
#pragma unroll
    for (int m = 0; m < RPT; m++) wprod[m] = 1.f;
    // what a thread brings into shared memory for a run of SCAN_TOK tokens: of every token the elements
    // x = thread, thread + 128, ... of [r | k | decay | the block's columns of v] (no division anywhere),
    // asked for one run ahead, so that their latency passes while the run before is worked on
    constexpr int XPT = (3 * SCAN_KP * RPT + SCAN_BCOLS + SCAN_THREADS - 1) / SCAN_THREADS;
    const int per_tok = 3 * d + SCAN_BCOLS;
    float ahead[SCAN_TOK][XPT];
    auto fetch = [&](int t0) {
        const int nt = min(SCAN_TOK, cnt - t0);
#pragma unroll
        for (int tt = 0; tt < SCAN_TOK; tt++) {
            const size_t at = (size_t)(tok0 + t0 + min(tt, nt - 1)) * ld + hc;
#pragma unroll
            for (int e = 0; e < XPT; e++) {
                const int x = threadIdx.x + e * SCAN_THREADS;
                float val = 0.f;
                if (x < d) val = r[at + x];
                else if (x < 2 * d) val = k[at + x - d];
                else if (x < 3 * d) val = w[at + x - 2 * d];
                else if (x < per_tok && c0 + x - 3 * d < d) val = v[at + c0 + x - 3 * d];
                ahead[tt][e] = val;
            }
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < cnt; t0 += SCAN_TOK) {
        const int nt = min(SCAN_TOK, cnt - t0);
        __syncthreads();                     // the run before is no longer read
#pragma unroll
        for (int tt = 0; tt < SCAN_TOK; tt++)
#pragma unroll
            for (int e = 0; e < XPT; e++) {
                const int x = threadIdx.x + e * SCAN_THREADS;
                if (x < per_tok) scan_smem[(size_t)tt * rowlen + x] = ahead[tt][e];
            }
        __syncthreads();
        if (t0 + SCAN_TOK < cnt) fetch(t0 + SCAN_TOK);
#pragma unroll 2
        for (int tt = 0; tt < nt; tt++) {
            const float* row = scan_smem + (size_t)tt * rowlen;
            const float4 v4 = *reinterpret_cast<const float4*>(row + 3 * d + cg * SCAN_CPT);
            const float vj[SCAN_CPT] = {v4.x, v4.y, v4.z, v4.w};
            if (sg.phase == 1) {         // the end state and the decays' products alone
#pragma unroll
                for (int m = 0; m < RPT; m++) {
                    const int i = kp * RPT + m;
                    const float ki = i < d ? row[d + i] : 0.f, wi = i < d ? row[2 * d + i] : 0.f;
                    wprod[m] *= wi;
#pragma unroll
                    for (int c = 0; c < SCAN_CPT; c++) sreg[m][c] = fmaf(wi, sreg[m][c], ki * vj[c]);
                }
                continue;
            }
            float acc[SCAN_CPT] = {0.f, 0.f, 0.f, 0.f};
            // o[j] = sum_i r_i S[i][j] + v_j sum_i r_i u_i k_i: the bonus's sum is the same for every column
            float ruk = 0.f;
#pragma unroll
            for (int m0 = 0; m0 < RPT; m0 += 4) {
                const int i0 = kp * RPT + m0;
                float ri[4], ki[4], wi[4];
                if (VEC) {
                    if (i0 < d) {
                        const float4 a4 = *reinterpret_cast<const float4*>(row + i0);
                        const float4 b4 = *reinterpret_cast<const float4*>(row + d + i0);
                        const float4 c4 = *reinterpret_cast<const float4*>(row + 2 * d + i0);
                        ri[0] = a4.x, ri[1] = a4.y, ri[2] = a4.z, ri[3] = a4.w;
                        ki[0] = b4.x, ki[1] = b4.y, ki[2] = b4.z, ki[3] = b4.w;
                        wi[0] = c4.x, wi[1] = c4.y, wi[2] = c4.z, wi[3] = c4.w;
                    } else {
#pragma unroll
                        for (int z = 0; z < 4; z++) ri[z] = ki[z] = wi[z] = 0.f;
                    }
                } else {
#pragma unroll
                    for (int z = 0; z < 4; z++) {
                        const bool in = i0 + z < d;
                        ri[z] = in ? row[i0 + z] : 0.f, ki[z] = in ? row[d + i0 + z] : 0.f, wi[z] = in ? row[2 * d + i0 + z] : 0.f;
                    }
                }
#pragma unroll
                for (int z = 0; z < 4; z++) {
                    ruk = fmaf(ri[z] * ureg[m0 + z], ki[z], ruk);
#pragma unroll
                    for (int c = 0; c < SCAN_CPT; c++) {
                        acc[c] = fmaf(ri[z], sreg[m0 + z][c], acc[c]);
                        sreg[m0 + z][c] = fmaf(wi[z], sreg[m0 + z][c], ki[z] * vj[c]);
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < SCAN_CPT; c++) acc[c] = fmaf(vj[c], ruk, acc[c]);
#pragma unroll
            for (int c = 0; c < SCAN_CPT; c++) {
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 1);
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 2);
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 4);
            }
            if (kp == 0) {
                float* o = out + (size_t)(tok0 + t0 + tt) * ((size_t)heads * d) + hc + col;
#pragma unroll
                for (int c = 0; c < SCAN_CPT; c++)
                    if (col + c < d) o[c] = acc[c];
            }
        }
    }
    if (sg.phase == 2 && !last_seg) return;          // only the sequence's last segment leaves the state behind
    if (sg.phase == 1) {
        S = ends + (size_t)seg * heads * plane;
        if (cg == 0 && blockIdx.x == 0) {
#pragma unroll
            for (int m = 0; m < RPT; m++)
                if (kp * RPT + m < d) decays[(size_t)seg * heads * d + kp * RPT + m] = wprod[m];
        }
    }
#pragma unroll
    for (int m = 0; m < RPT; m++) {
        const int i = kp * RPT + m;
        if (i >= d) continue;
        if (VEC && col < d) {
            *reinterpret_cast<float4*>(S + (size_t)i * d + col) = make_float4(sreg[m][0], sreg[m][1], sreg[m][2], sreg[m][3]);
        } else {
#pragma unroll
            for (int c = 0; c < SCAN_CPT; c++)
                if (col + c < d) S[(size_t)i * d + col + c] = sreg[m][c];
        }
    }
}

// One warp per (token, head).
template <typename OT>
__global__ void __launch_bounds__(256)
wkv_finish_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long ldg,
                  const float* __restrict__ norm_w, float eps, const int* __restrict__ seq_of_token, int num_tokens,
                  int heads, int d, OT* __restrict__ out) {
    pdl_sync();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)num_tokens * heads) return;
    const int t = (int)(item / heads), head = (int)(item % heads);
    const size_t base = (size_t)t * heads * d + (size_t)head * d;
    if (seq_of_token[t] < 0) {
        for (int e = lane; e < d; e += 32) st_f(out + base + e, 0.f);
        return;
    }
    float ss = 0.f;
    for (int e = lane; e < d; e += 32) {
        const float x = o[base + e];
        ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int e = lane; e < d; e += 32) {
        const float g = gate[(size_t)t * ldg + (size_t)head * d + e];
        st_f(out + base + e, o[base + e] * inv * norm_w[(size_t)head * d + e] * (g / (1.0f + expf(-g))));
    }
}

}  // namespace

// h: [T, width] 32-bit; mu: [streams, width]; state: per slot `width` floats at the start of a row of
// state_pitch floats; out: [streams, T, width] in out_dt; last32 (may be null): [T, width] 32-bit, receives
// the last blend instead of out.  With w1 ([rank, width], rank <= 32), w2t ([rank, inner]) and w0 ([inner])
// the last blend is not stored at all: decay [T, inner] = exp(-exp(w0 + w2t^T tanh(w1 x))) is formed here.
MOE_API int moe_wkv_shift_mix(const float* h, const float* mu, int streams, float* state, long long state_pitch,
                              const int* seq_of_token, const int* pos, const int* cu_seqlens, const int* slots,
                              int num_tokens, int width, void* out, int out_dt, float* last32, const float* w1,
                              const float* w2t, const float* w0, int rank, int inner, float* decay, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (!h || !mu || !state || !out || streams <= 0 || width <= 0 || state_pitch < width) return (int)cudaErrorInvalidValue;
    if (w1 && (!w2t || !w0 || !decay || last32 || rank <= 0 || rank > FUSED_RANK || inner <= 0))
        return (int)cudaErrorInvalidValue;
    const DecayArgs da{w1, w2t, w0, decay, rank, inner};
#define MIX(OT_, D_)                                                                                                 \
    return launch_pdl(wkv_shift_mix_kernel<OT_, D_>, dim3(num_tokens), 256, 0, stream, h, mu, streams, state, state_pitch, \
                      seq_of_token, pos, cu_seqlens, slots, num_tokens, width, (OT_*)out, last32, da)
    if (out_dt == DT_F32) {
        if (w1) MIX(float, true);
        MIX(float, false);
    }
    if (w1) MIX(__nv_bfloat16, true);
    MIX(__nv_bfloat16, false);
#undef MIX
}

// low: [T, rank] 32-bit; w2t: [rank, inner] (the second projection, transposed); w0: [inner]; out: [T, inner]
// 32-bit, the decay.
MOE_API int moe_wkv_decay(const float* low, const float* w2t, const float* w0, int num_tokens, int inner, int rank,
                          float* out, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (!low || !w2t || !w0 || !out || inner <= 0 || rank <= 0 || rank > MAX_RANK) return (int)cudaErrorInvalidValue;
    return launch_pdl(wkv_decay_kernel, dim3((num_tokens + DECAY_TOK - 1) / DECAY_TOK, (inner + 255) / 256), 256,
                      (size_t)DECAY_TOK * rank * sizeof(float), stream, low, w2t, w0, num_tokens, inner, rank, out);
}

// r, k, v, w (the decay): [T, heads * d] 32-bit with a row pitch of ld floats; u: [heads, d];
// state: per slot heads * d * d floats ([head][i][j]) at the start of a row of state_pitch floats;
// out: [T, heads * d] 32-bit (rows of no sequence are left alone).
MOE_API int moe_wkv_scan(const float* r, const float* k, const float* v, const float* w, long long ld,
                         const float* u, float* state, long long state_pitch, const int* cu_seqlens, const int* slots,
                         int num_seqs, int heads, int d, float* out, int segs, int seg_len, float* ends, float* decays,
                         cudaStream_t stream) {
    if (num_seqs <= 0) return 0;
    if (!r || !k || !v || !w || !u || !state || !out || heads <= 0 || d <= 0 || d > 256 ||
        ld < (long long)heads * d || state_pitch < (long long)heads * d * d || heads > 65535 || num_seqs > 65535)
        return (int)cudaErrorInvalidValue;
    if (segs < 1 || (segs > 1 && (!ends || !decays || seg_len <= 0 || seg_len % 8 || (long long)num_seqs * segs > 65535)))
        return (int)cudaErrorInvalidValue;
    const dim3 grid((d + SCAN_BCOLS - 1) / SCAN_BCOLS, heads, num_seqs * segs);
    const size_t smem = (size_t)scan_tok(d > 128 ? 32 : 8) * (3 * d + SCAN_BCOLS) * sizeof(float);
    // rows of the state 16 bytes at a time where every row of every head starts on such a boundary
    const bool vec = d % 4 == 0 && state_pitch % 4 == 0 && ((uintptr_t)state % 16) == 0 && ((uintptr_t)ends % 16) == 0;
    // one launch, or phase 1 and then phase 2 of the segmented form
    for (int phase = segs > 1 ? 1 : 0; phase <= (segs > 1 ? 2 : 0); phase++) {
        const WkvSegments sg{segs, seg_len, phase, ends, decays};
        int code;
#define SCAN(RPT_)                                                                                                    \
    code = vec ? launch_pdl(wkv_scan_kernel<RPT_, true>, grid, SCAN_THREADS, smem, stream, r, k, v, w, ld, u, state,       \
                            state_pitch, cu_seqlens, slots, heads, d, out, sg)                                        \
               : launch_pdl(wkv_scan_kernel<RPT_, false>, grid, SCAN_THREADS, smem, stream, r, k, v, w, ld, u, state,      \
                            state_pitch, cu_seqlens, slots, heads, d, out, sg)
        if (d <= 32) SCAN(4);
        else if (d <= 64) SCAN(8);
        else if (d <= 128) SCAN(16);
        else SCAN(32);
#undef SCAN
        if (code) return code;
    }
    return 0;
}

// o: [T, heads * d] 32-bit; gate: the gate projection's output, 32-bit, row pitch ldg; norm_w: [heads * d];
// out: [T, heads * d] in out_dt.
MOE_API int moe_wkv_finish(const float* o, const float* gate, long long ldg, const float* norm_w, float eps,
                           const int* seq_of_token, int num_tokens, int heads, int d, void* out, int out_dt,
                           cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (!o || !gate || !norm_w || !out || heads <= 0 || d <= 0 || ldg < (long long)heads * d)
        return (int)cudaErrorInvalidValue;
    const long long items = (long long)num_tokens * heads;
    const unsigned blocks = (unsigned)((items + 7) / 8);
    if (out_dt == DT_F32)
        return launch_pdl(wkv_finish_kernel<float>, dim3(blocks), 256, 0, stream, o, gate, ldg, norm_w, eps,
                          seq_of_token, num_tokens, heads, d, (float*)out);
    return launch_pdl(wkv_finish_kernel<__nv_bfloat16>, dim3(blocks), 256, 0, stream, o, gate, ldg, norm_w, eps,
                      seq_of_token, num_tokens, heads, d, (__nv_bfloat16*)out);
}
