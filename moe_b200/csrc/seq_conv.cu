// Small kernels around a sublayer whose inputs depend on the tokens before it:
//
//   seq_conv        a causal convolution over time on every channel of a step's rows,
//                     y_t = act(sum_j w[j] * u_(t - taps + 1 + j) + bias) (+ u_t with `residual`),
//                   where rows before the step's first come from the sequence's state (the last
//                   taps - 1 rows it has seen, oldest first; zeros at a sequence's start).  In a step of
//                   one token a sequence (`shift`) the same thread also moves the state on; else
//                   conv_state_update (attention_conv.cu) does that afterwards, in a launch of its own,
//                   because blocks of this one still read the old state.
//   embed_pair      x = rmsnorm(embed[token] + pair[(previous * mul_prev + token * mul_cur) mod buckets]),
//                   row `buckets` of the pair table for a sequence's first token; the previous token of
//                   a step's first row is the sequence's state, which the block of that row then
//                   replaces by the step's last token (it is the state's only reader).
//   pair_norm_mean  out = (rmsnorm(a) * wa + rmsnorm(b) * wb) / 2, both norms over the model's width.
//   relu2           out = relu(in)^2 element by element, rounded to the activation dtype (where the
//                   tensor-core product's epilogue does not form it).
//   table_route     a token's experts are row `token id` of an integer table; each weighs 1 / top.
// All arithmetic is 32-bit; only stores into activation buffers round.
#include "common.cuh"

namespace {

constexpr int SC_MAX_TAPS = 16;
enum : int { SC_ACT_NONE = 0, SC_ACT_SILU = 1 };

struct ConvJob {
    const float* u;          // [T, ldu] the step's rows
    const float* w;          // [taps, channels]
    const float* bias;       // [channels] or null
    float* state;            // this job's first float in a slot's state row
    float* out32;            // [T, channels] or null
    __nv_bfloat16* out16;    // [T, channels] or null
    long long ldu;
};
struct ConvJobs {
    ConvJob j[2];
};

__device__ __forceinline__ void sc_store(float* o32, __nv_bfloat16* o16, size_t at, const float (&y)[4], int n) {
    if (n == 4) {
        if (o32) *reinterpret_cast<float4*>(o32 + at) = make_float4(y[0], y[1], y[2], y[3]);
        if (o16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
            uint2 u;
            u.x = *reinterpret_cast<unsigned*>(&lo), u.y = *reinterpret_cast<unsigned*>(&hi);
            *reinterpret_cast<uint2*>(o16 + at) = u;
        }
    } else {
        for (int e = 0; e < n; e++) {
            if (o32) o32[at + e] = y[e];
            if (o16) o16[at + e] = __float2bfloat16_rn(y[e]);
        }
    }
}

// grid (token, channel block, job).  VEC: a thread takes four neighbouring channels 16 bytes at a time;
// else one channel.  Nothing is kept in an array over the taps: a tap's input is used, moved one place
// down in the state where the step brings one row a sequence (`shift`: the place was read a tap ago), and
// forgotten.
template <bool VEC, int TAPS, int TOKB>
__global__ void __launch_bounds__(256)
seq_conv_kernel(const ConvJobs jobs, int taps_any, int channels, long long state_pitch,
                const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens,
                const int* __restrict__ slots, int num_tokens, int residual, int act, int shift) {
    constexpr int W = VEC ? 4 : 1;
    const int taps = TAPS > 0 ? TAPS : taps_any;      // (a number known when compiled: the taps' loads are all in flight at once)
    pdl_sync();
    const ConvJob& J = jobs.j[blockIdx.z];
    const int ch = (blockIdx.y * blockDim.x + threadIdx.x) * W;
    if (ch >= channels) return;
    // TOKB rows a block (many rows: fewer, longer blocks with more loads in flight a thread)
#pragma unroll
    for (int tt = 0; tt < TOKB; tt++) {
        const int t = blockIdx.x * TOKB + tt;
        if (t >= num_tokens) break;
        const int s = seq_of_token[t];
        const size_t oat = (size_t)t * channels + ch;
        float y[4] = {0.f, 0.f, 0.f, 0.f};
        if (s < 0) {          // a row of no sequence: something finite, no state touched
            sc_store(J.out32, J.out16, oat, y, W);
            continue;
        }
        const int li = t - cu_seqlens[s];                 // the row's place among the sequence's rows of this step
        float* st = taps > 1 ? J.state + (size_t)slots[s] * state_pitch : nullptr;
        if (J.bias) {
#pragma unroll
            for (int e = 0; e < W; e++) y[e] = J.bias[ch + e];
        }
        float own[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < taps; j++) {
            const int r = li - (taps - 1) + j;            // the row tap j reads, relative to the step's first
            const float* src = r >= 0 ? J.u + (size_t)(t - li + r) * J.ldu + ch : st + (size_t)(taps - 1 + r) * channels + ch;
            const float* wj = J.w + (size_t)j * channels + ch;
            if (VEC) {
                const float4 x4 = *reinterpret_cast<const float4*>(src), w4 = *reinterpret_cast<const float4*>(wj);
                own[0] = x4.x, own[1] = x4.y, own[2] = x4.z, own[3] = x4.w;
                y[0] = fmaf(w4.x, x4.x, y[0]), y[1] = fmaf(w4.y, x4.y, y[1]);
                y[2] = fmaf(w4.z, x4.z, y[2]), y[3] = fmaf(w4.w, x4.w, y[3]);
                if (shift && j >= 1) *reinterpret_cast<float4*>(st + (size_t)(j - 1) * channels + ch) = x4;
            } else {
                own[0] = *src;
                y[0] = fmaf(*wj, own[0], y[0]);
                if (shift && j >= 1) st[(size_t)(j - 1) * channels + ch] = own[0];
            }
        }
#pragma unroll
        for (int e = 0; e < W; e++) {
            if (act == SC_ACT_SILU) y[e] = y[e] / (1.0f + expf(-y[e]));
            if (residual) y[e] += own[e];
        }
        sc_store(J.out32, J.out16, oat, y, W);
    }
}

template <typename WT>
__global__ void __launch_bounds__(256)
embed_pair_kernel(const WT* __restrict__ table, const WT* __restrict__ pair, const float* __restrict__ norm_w,
                  float eps, const int* __restrict__ tokens, float* __restrict__ x, int hidden, int vocab, int buckets,
                  int mul_prev, int mul_cur, int* __restrict__ prev_state, const int* __restrict__ seq_of_token,
                  const int* __restrict__ pos, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                  const int* __restrict__ last_token, int* status) {
    extern __shared__ float ep_row[];
    __shared__ float red[32];
    pdl_sync();
    const int t = blockIdx.x;
    const int s = seq_of_token[t];
    float* out = x + (size_t)t * hidden;
    if (s < 0) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = 0.f;
        return;
    }
    auto token_at = [&](int r) {
        int tok = tokens[r];
        if (tok == -1 && last_token) tok = last_token[slots[s]];
        if (tok < 0 || tok >= vocab) {
            if (threadIdx.x == 0) atomicOr(status, ST_BAD_TOKEN);
            tok = 0;
        }
        return tok;
    };
    const int first = cu_seqlens[s], end = cu_seqlens[s + 1];
    const int tok = token_at(t);
    long long prow = buckets;
    if (pos[t] > 0) {
        const int prev = t > first ? token_at(t - 1) : prev_state[slots[s]];
        prow = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
    }
    __syncthreads();      // the state was read (by every thread of the block that needs it) before it changes
    if (t == first && threadIdx.x == 0) prev_state[slots[s]] = token_at(end - 1);
    const WT* a = table + (size_t)tok * hidden;
    const WT* b = pair + (size_t)prow * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = ld_f(a + i) + ld_f(b + i);
        ep_row[i] = v;
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = ep_row[i] * inv * norm_w[i];
}

__global__ void __launch_bounds__(256)
pair_norm_mean_kernel(const float* __restrict__ a, const float* __restrict__ wa, const float* __restrict__ b,
                      const float* __restrict__ wb, float eps, int hidden, float* __restrict__ out) {
    __shared__ float red[32];
    pdl_sync();
    const size_t base = (size_t)blockIdx.x * hidden;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float x = a[base + i], y = b[base + i];
        sa = fmaf(x, x, sa), sb = fmaf(y, y, sb);
    }
    const float ia = 1.0f / sqrtf(block_sum(sa, red) / (float)hidden + eps);
    const float ib = 1.0f / sqrtf(block_sum(sb, red) / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        out[base + i] = 0.5f * (a[base + i] * ia * wa[i] + b[base + i] * ib * wb[i]);
}

template <typename OT>
__global__ void relu2_kernel(const float* __restrict__ in, OT* __restrict__ out, long long n) {
    pdl_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = fmaxf(in[i], 0.f);
    st_f(out + i, v * v);
}

__global__ void table_route_kernel(const int* __restrict__ table, int width, const int* __restrict__ tokens,
                                   const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                   const int* __restrict__ last_token, int num_tokens, int vocab, int top,
                                   int num_experts, int* __restrict__ topk_idx, float* __restrict__ topk_w, int* status) {
    pdl_sync();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_tokens * top) return;
    const int t = i / top, j = i % top;
    const int s = seq_of_token ? seq_of_token[t] : 0;
    if (s < 0) {
        topk_idx[i] = -1, topk_w[i] = 0.f;
        return;
    }
    int tok = tokens[t];
    if (tok == -1 && last_token) tok = last_token[slots[s]];
    if (tok < 0 || tok >= vocab) {
        atomicOr(status, ST_BAD_TOKEN);
        tok = 0;
    }
    int e = table[(size_t)tok * width + j];
    if (e < 0 || e >= num_experts) {
        atomicOr(status, ST_BAD_EXPERT);
        e = 0;
    }
    topk_idx[i] = e;
    topk_w[i] = 1.0f / (float)top;
}

}  // namespace

// Up to two convolutions of one shape in a launch (`njobs`).  u*: [T, ldu*] 32-bit rows; w*: [taps, channels];
// bias*: [channels] or null; state*: [slots + 1, state_pitch] with (taps - 1) * channels floats used from the
// pointer given; out32* / out16*: [T, channels] or null.
MOE_API int moe_seq_conv(int njobs, const float* u0, long long ldu0, const float* w0, const float* bias0, float* state0,
                         float* out32_0, void* out16_0, const float* u1, long long ldu1, const float* w1,
                         const float* bias1, float* state1, float* out32_1, void* out16_1, int taps, int channels,
                         long long state_pitch, const int* seq_of_token, const int* pos, const int* cu_seqlens,
                         const int* slots, int num_tokens, int residual, int act, int shift, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (njobs < 1 || njobs > 2 || taps < 1 || taps > SC_MAX_TAPS || channels <= 0 || !u0 || !w0 || !seq_of_token ||
        !cu_seqlens || !slots || (taps > 1 && !state0) || ldu0 < channels)
        return (int)cudaErrorInvalidValue;
    if (njobs == 2 && (!u1 || !w1 || (taps > 1 && !state1) || ldu1 < channels)) return (int)cudaErrorInvalidValue;
    ConvJobs jobs;
    jobs.j[0] = ConvJob{u0, w0, bias0, state0, out32_0, (__nv_bfloat16*)out16_0, ldu0};
    jobs.j[1] = ConvJob{u1, w1, bias1, state1, out32_1, (__nv_bfloat16*)out16_1, ldu1};
    auto al = [](const void* p, size_t a) { return ((uintptr_t)p % a) == 0; };
    bool vec = channels % 4 == 0 && state_pitch % 4 == 0;
    for (int i = 0; i < njobs; i++) {
        const ConvJob& J = jobs.j[i];
        vec = vec && J.ldu % 4 == 0 && al(J.u, 16) && al(J.w, 16) && al(J.bias, 16) && al(J.state, 16) && al(J.out32, 16) &&
              al(J.out16, 8);
    }
    const int lanes = vec ? channels / 4 : channels;
    const int threads = lanes >= 256 ? 256 : ((lanes + 31) / 32) * 32;
    const int tokb = (vec && num_tokens >= 1024 && taps >= 2 && taps <= 4) ? 4 : 1;
    const dim3 grid((num_tokens + tokb - 1) / tokb, (lanes + threads - 1) / threads, njobs);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
#define CONV(VEC_, TAPS_, TOKB_)                                                                                            \
    return launch_pdl(seq_conv_kernel<VEC_, TAPS_, TOKB_>, grid, dim3(threads), 0, stream, jobs, taps, channels, state_pitch, \
                      seq_of_token, cu_seqlens, slots, num_tokens, residual, act, shift)
    if (vec && tokb == 4) {
        if (taps == 2) CONV(true, 2, 4);
        if (taps == 3) CONV(true, 3, 4);
        CONV(true, 4, 4);
    }
    if (vec) {
        if (taps == 2) CONV(true, 2, 1);
        if (taps == 3) CONV(true, 3, 1);
        if (taps == 4) CONV(true, 4, 1);
        CONV(true, 0, 1);
    }
    if (taps == 4) CONV(false, 4, 1);
    CONV(false, 0, 1);
#undef CONV
}

// table: [vocab, hidden], pair: [buckets + 1, hidden] in table_dt; norm_w: [hidden] 32-bit; x: [T, hidden] 32-bit;
// prev_state: [slots + 1] the token each sequence saw last.
MOE_API int moe_embed_pair(const void* table, const void* pair, int table_dt, const float* norm_w, float eps,
                           const int* tokens, float* x, int num_tokens, int hidden, int vocab, int buckets,
                           int mul_prev, int mul_cur, int* prev_state, const int* seq_of_token, const int* pos,
                           const int* cu_seqlens, const int* slots, const int* last_token, int* status,
                           cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (!table || !pair || !norm_w || !tokens || !x || !prev_state || !seq_of_token || !pos || !cu_seqlens || !slots ||
        buckets <= 0 || hidden <= 0 || (size_t)hidden * sizeof(float) > 48 * 1024)
        return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (table_dt == DT_F32)
        return launch_pdl(embed_pair_kernel<float>, dim3(num_tokens), 256, smem, stream, (const float*)table,
                          (const float*)pair, norm_w, eps, tokens, x, hidden, vocab, buckets, mul_prev, mul_cur,
                          prev_state, seq_of_token, pos, cu_seqlens, slots, last_token, status);
    return launch_pdl(embed_pair_kernel<__nv_bfloat16>, dim3(num_tokens), 256, smem, stream,
                      (const __nv_bfloat16*)table, (const __nv_bfloat16*)pair, norm_w, eps, tokens, x, hidden, vocab,
                      buckets, mul_prev, mul_cur, prev_state, seq_of_token, pos, cu_seqlens, slots, last_token, status);
}

MOE_API int moe_pair_norm_mean(const float* a, const float* wa, const float* b, const float* wb, float eps,
                               int num_tokens, int hidden, float* out, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (!a || !wa || !b || !wb || !out || hidden <= 0) return (int)cudaErrorInvalidValue;
    return launch_pdl(pair_norm_mean_kernel, dim3(num_tokens), 256, 0, stream, a, wa, b, wb, eps, hidden, out);
}

MOE_API int moe_relu2(const float* in, void* out, int out_dt, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dt == DT_F32) return launch_pdl(relu2_kernel<float>, dim3(blocks), 256, 0, stream, in, (float*)out, n);
    return launch_pdl(relu2_kernel<__nv_bfloat16>, dim3(blocks), 256, 0, stream, in, (__nv_bfloat16*)out, n);
}

// table: [vocab, width >= top] int32; topk_idx / topk_w: [T, top].
MOE_API int moe_table_route(const int* table, int width, const int* tokens, const int* seq_of_token, const int* slots,
                            const int* last_token, int num_tokens, int vocab, int top, int num_experts, int* topk_idx,
                            float* topk_w, int* status, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (!table || !tokens || !topk_idx || !topk_w || top <= 0 || width < top || (last_token && (!seq_of_token || !slots)))
        return (int)cudaErrorInvalidValue;
    const int n = num_tokens * top;
    return launch_pdl(table_route_kernel, dim3((n + 255) / 256), 256, 0, stream, table, width, tokens, seq_of_token,
                      slots, last_token, num_tokens, vocab, top, num_experts, topk_idx, topk_w, status);
}
