// Kernels of a selective state-space mixer (state-space duality form): a short causal convolution per
// channel with SiLU, and the recurrence
//     S_t = exp(-exp(A_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T ,   y_t = S_t^T C_t + D_h x_t
// per head h (S is N x P; B and C are shared by the heads of a group), with dt = softplus(raw + bias).
//
// Both carry state from step to step per request: the convolution its last taps - 1 inputs, the
// recurrence S.  A request's state lives in one row of a float32 state tensor (`state`, rows of
// `state_stride` floats): S as [heads][N][P] at offset 0, the convolution's inputs as
// [taps - 1][channels] (oldest first) at `conv_off`.  The tokens that a sequence brings to a step are
// contiguous rows [cu_seqlens[s], cu_seqlens[s + 1]); state_slots[s] < 0 marks a padding row, which
// reads and writes no state.  Decays, step sizes, the state and the sums are float32 whatever the
// storage type of the activations.
#include "common.cuh"

__device__ __forceinline__ float rv_load_any(const void* p, int dtype, size_t i) {
    return dtype == RV_DTYPE_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
// The bits of an element, unconverted (a load whose result nothing touches yet does not hold the warp up), and their value.
__device__ __forceinline__ uint32_t rv_load_raw(const void* p, int dtype, size_t i) {
    return dtype == RV_DTYPE_F32 ? ((const uint32_t*)p)[i] : (uint32_t)((const unsigned short*)p)[i];
}
__device__ __forceinline__ float rv_raw_value(uint32_t raw, int dtype) {
    return __uint_as_float(dtype == RV_DTYPE_F32 ? raw : raw << 16);
}
__device__ __forceinline__ void rv_store_any(void* p, int dtype, size_t i, float v) {
    if (dtype == RV_DTYPE_F32) ((float*)p)[i] = v;
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

#define RV_MAX_TAPS 16

// ------------------------------------------------------------------ causal convolution + SiLU
// out[t, c] = silu(bias[c] + sum_j w[c, j] * in(t - (taps - 1) + j, c)); inputs before the step's first token of the
// sequence come from the request's state (zeros at the start of a sequence: a fresh slot is zeroed).
// `in` is a slice of a wider row: column col0 .. col0 + channels of rows of `in_stride` elements.
__global__ void __launch_bounds__(256)
causal_conv_silu_kernel(const void* __restrict__ in, int in_dtype, int in_stride, int col0,
                        const void* __restrict__ w, const void* __restrict__ bias, int w_dtype,
                        const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ state_slots, const float* __restrict__ state, size_t state_stride,
                        size_t conv_off, void* __restrict__ out, int out_dtype, int n_tokens, int channels, int taps, int t0) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = t0 + blockIdx.y;
    if (c >= channels || t >= n_tokens) return;
    const int seq = token_seq[t];
    const int start = cu_seqlens[seq];
    const int i = t - start;
    const int slot = state_slots[seq];
    const float* hist = slot >= 0 ? state + (size_t)slot * state_stride + conv_off : nullptr;
    float acc = bias ? rv_load_param(bias, w_dtype, c) : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int idx = i - (taps - 1) + j;
        float v;
        if (idx >= 0) v = rv_load_any(in, in_dtype, (size_t)(start + idx) * in_stride + col0 + c);
        else v = hist ? hist[(size_t)(taps - 1 + idx) * channels + c] : 0.f;
        acc = fmaf(rv_load_param(w, w_dtype, c * taps + j), v, acc);
    }
    rv_store_any(out, out_dtype, (size_t)t * channels + c, acc / (1.0f + expf(-acc)));
}

// The same for up to four taps, RV_CONV_TOKENS consecutive tokens per thread: the last taps - 1 inputs stay in registers
// from token to token, so a token costs one load; where a new sequence begins inside the thread's run the registers
// are filled again from the rows before it or from the request's state.
#define RV_CONV_TOKENS 8
template <int TAPS>
__global__ void __launch_bounds__(256)
causal_conv_silu_run_kernel(const void* __restrict__ in, int in_dtype, int in_stride, int col0,
                            const void* __restrict__ w, const void* __restrict__ bias, int w_dtype,
                            const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ state_slots, const float* __restrict__ state, size_t state_stride,
                            size_t conv_off, void* __restrict__ out, int out_dtype, int n_tokens, int channels) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int t_begin = blockIdx.y * RV_CONV_TOKENS;
    const int t_end = t_begin + RV_CONV_TOKENS < n_tokens ? t_begin + RV_CONV_TOKENS : n_tokens;
    float wt[TAPS], win[TAPS > 1 ? TAPS - 1 : 1];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wt[j] = rv_load_param(w, w_dtype, c * TAPS + j);
    const float b = bias ? rv_load_param(bias, w_dtype, c) : 0.f;
    int seq_end = -1;
    for (int t = t_begin; t < t_end; ++t) {
        if (t >= seq_end) {                            // the thread's first token, or the first of another sequence
            const int seq = token_seq[t];
            const int start = cu_seqlens[seq];
            seq_end = cu_seqlens[seq + 1];
            const int slot = state_slots[seq];
            const float* hist = slot >= 0 ? state + (size_t)slot * state_stride + conv_off : nullptr;
#pragma unroll
            for (int k = 0; k < TAPS - 1; ++k) {
                const int idx = (t - start) - (TAPS - 1) + k;
                win[k] = idx >= 0 ? rv_load_any(in, in_dtype, (size_t)(start + idx) * in_stride + col0 + c)
                                  : (hist ? hist[(size_t)(TAPS - 1 + idx) * channels + c] : 0.f);
            }
        }
        const float v = rv_load_any(in, in_dtype, (size_t)t * in_stride + col0 + c);
        float acc = b;
#pragma unroll
        for (int k = 0; k < TAPS - 1; ++k) acc = fmaf(wt[k], win[k], acc);
        acc = fmaf(wt[TAPS - 1], v, acc);
#pragma unroll
        for (int k = 0; k + 1 < TAPS - 1; ++k) win[k] = win[k + 1];
        if (TAPS > 1) win[TAPS - 2] = v;
        rv_store_any(out, out_dtype, (size_t)t * channels + c, acc / (1.0f + expf(-acc)));
    }
}

// After the convolution of a step: the state becomes the last taps - 1 inputs of each sequence.
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const void* __restrict__ in, int in_dtype, int in_stride, int col0,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                         float* __restrict__ state, size_t state_stride, size_t conv_off, int channels, int taps) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.y;
    if (c >= channels) return;
    const int slot = state_slots[seq];
    if (slot < 0) return;
    const int start = cu_seqlens[seq], n = cu_seqlens[seq + 1] - start;
    float* hist = state + (size_t)slot * state_stride + conv_off;
    float keep[RV_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < RV_MAX_TAPS; ++k) {
        if (k < taps - 1) {
            const int idx = n - (taps - 1) + k;            // index among the step's tokens of this sequence
            keep[k] = idx >= 0 ? rv_load_any(in, in_dtype, (size_t)(start + idx) * in_stride + col0 + c)
                               : hist[(size_t)(k + n) * channels + c];
        }
    }
#pragma unroll
    for (int k = 0; k < RV_MAX_TAPS; ++k)
        if (k < taps - 1) hist[(size_t)k * channels + c] = keep[k];
}

RV_EXPORT int rv_causal_conv_silu(const void* in, int in_dtype, int in_stride, int col0, const void* w, const void* bias,
                                  int w_dtype, const int* token_seq, const int* cu_seqlens, const int* state_slots,
                                  float* state, long long state_stride, long long conv_off, void* out, int out_dtype,
                                  int n_tokens, int n_seqs, int channels, int taps, cudaStream_t stream) {
    if (n_tokens < 0 || n_seqs < 0 || channels <= 0 || taps < 1 || taps > RV_MAX_TAPS || col0 < 0 || in_stride < col0 + channels)
        return RV_ERR_BAD_SIZE;
    if ((in_dtype | w_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (n_tokens == 0 || n_seqs == 0) return RV_OK;
    if (n_tokens > 65535 * 8 || n_seqs > 65535) return RV_ERR_BAD_SIZE;
    const int threads = channels >= 256 ? 256 : 128;
    const int bx = (channels + threads - 1) / threads;
    if (taps <= 4) {
        const dim3 grid(bx, (n_tokens + RV_CONV_TOKENS - 1) / RV_CONV_TOKENS);
#define RV_CONV_LAUNCH(TAPS)                                                                                                          \
        RV_LAUNCH_ST = rv_launch(causal_conv_silu_run_kernel<TAPS>, dim3(grid), dim3(threads), 0, stream, in, in_dtype, in_stride, col0, w, \
                                 bias, w_dtype, token_seq, cu_seqlens, state_slots, (const float*)state, (size_t)state_stride,        \
                                 (size_t)conv_off, out, out_dtype, n_tokens, channels)
        if (taps == 1) RV_CONV_LAUNCH(1);
        else if (taps == 2) RV_CONV_LAUNCH(2);
        else if (taps == 3) RV_CONV_LAUNCH(3);
        else RV_CONV_LAUNCH(4);
#undef RV_CONV_LAUNCH
        if (RV_LAUNCH_ST != RV_OK) return rv_launch_status();
    } else
    for (int t0 = 0; t0 < n_tokens; t0 += 65535) {          // (gridDim.y is limited)
        const int nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
        RV_LAUNCH_ST = rv_launch(causal_conv_silu_kernel, dim3(bx, nt), dim3(threads), 0, stream,
                                 in, in_dtype, in_stride, col0, w, bias, w_dtype, token_seq, cu_seqlens, state_slots,
                                 (const float*)state, (size_t)state_stride, (size_t)conv_off, out, out_dtype,
                                 n_tokens, channels, taps, t0);
        if (RV_LAUNCH_ST != RV_OK) return rv_launch_status();
    }
    if (taps > 1)
        RV_LAUNCH_ST = rv_launch(conv_state_update_kernel, dim3(bx, n_seqs), dim3(threads), 0, stream, in, in_dtype, in_stride, col0,
                                 cu_seqlens, state_slots, state, (size_t)state_stride, (size_t)conv_off, channels, taps);
    return rv_launch_status();
}

// ------------------------------------------------------------------ the recurrence
// Grid (P / 32 column blocks, heads, sequences); 128 threads = 32 columns p x 4 slices of the state dimension: thread
// (p, s) keeps S[n][p] for the NPT consecutive n of its slice in registers, and the four slices of a column add their
// parts of y with shuffles.  The tokens of a sequence are walked in chunks of RV_SCAN_CHUNK: B, C, the decay and dt x of
// a chunk are staged in shared memory (as floats, a slice's part of a row padded by four so that the slices' 16-byte
// reads fall into different banks), then the chunk runs without a barrier per token.  Where the rows allow 16-byte
// loads (bfloat16, sizes that are multiples of 8) the next chunk is fetched into registers before the current one is
// computed, so that its way from memory is hidden behind the arithmetic.
#define RV_SCAN_CHUNK 16

template <int NPT, int NC>
__global__ void __launch_bounds__(128)
ssm_scan_kernel(const void* __restrict__ xbc, int x_dtype, int channels,           // [T, channels]: x | B | C after the convolution
                const void* __restrict__ dt_in, int dt_dtype, int dt_stride, int dt_col0,   // raw dt: column dt_col0 + h of rows of dt_stride
                const void* __restrict__ dt_bias, const void* __restrict__ a_log, const void* __restrict__ d_skip, int p_dtype,
                const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                float* __restrict__ state, size_t state_stride, float* __restrict__ y,
                int heads, int P, int N, int groups,
                int seg_tokens, int max_segs, float* __restrict__ seg_state, float* __restrict__ seg_decay, float* __restrict__ dcum) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    constexpr int NSL = 8;                            // slices of the state dimension
    constexpr int COLS = NC * 128 / NSL;              // columns p of a block
    constexpr int SEG = NPT + 4, TOK = NSL * SEG;     // floats of a slice's part, and of a token's B (or C)
    constexpr int PRE = NSL * NPT >= 32 ? NSL * NPT / 32 : 1;   // 16-byte pieces of a chunk's B and C per thread
    constexpr int XV = COLS / 8;                      // 16-byte pieces of a token's x
    extern __shared__ __align__(16) float sm[];
    float* sB = sm;                                   // [chunk][TOK]
    float* sC = sB + RV_SCAN_CHUNK * TOK;             // [chunk][TOK]
    float* sX = sC + RV_SCAN_CHUNK * TOK;             // [chunk][32]   x
    float* sY = sX + RV_SCAN_CHUNK * COLS;    // [chunk][32]
    float* sDec = sY + RV_SCAN_CHUNK * COLS;  // [chunk]       exp(-exp(A_log) dt)
    float* sDt = sDec + RV_SCAN_CHUNK;                // [chunk]
    const int tid = threadIdx.x;
    // With seg_tokens > 0 a sequence's tokens are cut into segments of that many and grid.z counts (sequence, segment):
    // segment 0 starts from the request's state, the others from zero; a sequence of several segments leaves each
    // segment's last state, the product of its decays and the running product at every token in scratch memory, from which
    // ssm_segment_carry_kernel and ssm_segment_correct_kernel put the pieces together.
    const int seq = blockIdx.z / max_segs, seg = blockIdx.z - seq * max_segs;
    const int h = blockIdx.y, p0 = blockIdx.x * COLS;
    const int seq_start = cu_seqlens[seq], seq_tok = cu_seqlens[seq + 1] - seq_start;
    const int n_segs = seg_tokens > 0 ? (seq_tok + seg_tokens - 1) / seg_tokens : 1;
    if (seg >= n_segs) return;
    const int start = seq_start + seg * seg_tokens;
    const int n_tok = seg_tokens > 0 ? (seq_tok - seg * seg_tokens < seg_tokens ? seq_tok - seg * seg_tokens : seg_tokens) : seq_tok;
    const int slot = state_slots[seq];
    const int inner = heads * P;
    const int lane_p = (tid / NSL) * NC, slice = tid % NSL;      // the thread's first column within the block
    const int p = p0 + lane_p;
    if (slot < 0) {                                    // a padding row: no state; its output is zero
        for (int i = tid; i < n_tok * COLS; i += blockDim.x) {
            const int tk = i / COLS, pp = p0 + (i - tk * COLS);
            if (pp < P) y[(size_t)(start + tk) * inner + h * P + pp] = 0.f;
        }
        return;
    }
    const int g = h / (heads / groups);
    const float A = -expf(rv_load_param(a_log, p_dtype, h));
    const float bias = rv_load_param(dt_bias, p_dtype, h);
    const float Dh = rv_load_param(d_skip, p_dtype, h);
    float* S = state + (size_t)slot * state_stride + (size_t)h * N * P;
    float s[NC][NPT];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int n = slice * NPT + i;
            s[c][i] = (seg == 0 && p + c < P && n < N) ? S[(size_t)n * P + p + c] : 0.f;
        }
    for (int i = tid; i < 2 * RV_SCAN_CHUNK * TOK; i += blockDim.x) sm[i] = 0.f;      // state indices beyond N stay zero
    const size_t b_col = (size_t)inner + (size_t)g * N, c_col = (size_t)inner + (size_t)groups * N + (size_t)g * N;
    const bool vec = x_dtype == RV_DTYPE_BF16 && !(N & 7) && !(inner & 7) && !((groups * N) & 7) && !(channels & 7) && !(P & 7) &&
                     (reinterpret_cast<uintptr_t>(xbc) & 15) == 0;
    const int vpr = N >> 3;                            // 16-byte pieces per row of B (or C)
    uint4 pre_bc[PRE];
    uint4 pre_x = make_uint4(0, 0, 0, 0);
    float pre_dt = 0.f;
    const __nv_bfloat16* xb = (const __nv_bfloat16*)xbc;

    auto fetch = [&](int t0) {                         // the chunk's rows into registers (vector path only)
        const int nt = n_tok - t0 < RV_SCAN_CHUNK ? n_tok - t0 : RV_SCAN_CHUNK;
#pragma unroll
        for (int j = 0; j < PRE; ++j) {
            const int v = tid + j * 128;
            if (v < nt * vpr * 2) {
                const int tk = v / (2 * vpr), r = v - tk * 2 * vpr;
                const int which = r >= vpr, k = r - which * vpr;
                pre_bc[j] = *reinterpret_cast<const uint4*>(xb + (size_t)(start + t0 + tk) * channels + (which ? c_col : b_col) + k * 8);
            }
        }
        if (tid < nt * XV) {
            const int tk = tid / XV, k = tid % XV;
            const int col = h * P + p0 + k * 8;
            pre_x = col + 8 <= channels ? *reinterpret_cast<const uint4*>(xb + (size_t)(start + t0 + tk) * channels + col) : make_uint4(0, 0, 0, 0);
        }
        if (tid >= 64 && tid < 64 + nt)
            pre_dt = rv_load_any(dt_in, dt_dtype, (size_t)(start + t0 + tid - 64) * dt_stride + dt_col0 + h);
    };
    auto stage = [&](int t0) {                         // registers -> shared memory, as floats
        const int nt = n_tok - t0 < RV_SCAN_CHUNK ? n_tok - t0 : RV_SCAN_CHUNK;
#pragma unroll
        for (int j = 0; j < PRE; ++j) {
            const int v = tid + j * 128;
            if (v < nt * vpr * 2) {
                const int tk = v / (2 * vpr), r = v - tk * 2 * vpr;
                const int which = r >= vpr, k = r - which * vpr;
                const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&pre_bc[j]);
                float* dst = (which ? sC : sB) + tk * TOK;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int n = k * 8 + q;
                    dst[(n / NPT) * SEG + (n % NPT)] = __bfloat162float(e[q]);
                }
            }
        }
        if (tid < nt * XV) {
            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&pre_x);
#pragma unroll
            for (int q = 0; q < 8; ++q) sX[(tid / XV) * COLS + (tid % XV) * 8 + q] = __bfloat162float(e[q]);
        }
        if (tid >= 64 && tid < 64 + nt) {
            const float raw = pre_dt + bias;
            const float dt = raw > 20.f ? raw : log1pf(expf(raw));
            sDt[tid - 64] = dt;
            sDec[tid - 64] = expf(A * dt);
        }
    };
    auto stage_plain = [&](int t0) {                   // any type and size: element by element, four loads in flight
        const int nt = n_tok - t0 < RV_SCAN_CHUNK ? n_tok - t0 : RV_SCAN_CHUNK;
        if (tid < nt) {
            const float raw = rv_load_any(dt_in, dt_dtype, (size_t)(start + t0 + tid) * dt_stride + dt_col0 + h) + bias;
            const float dt = raw > 20.f ? raw : log1pf(expf(raw));
            sDt[tid] = dt;
            sDec[tid] = expf(A * dt);
        }
#pragma unroll 4
        for (int i = tid; i < nt * N; i += 128) {
            const int tk = i / N, n = i - tk * N;
            const size_t rowb = (size_t)(start + t0 + tk) * channels;
            const int at = tk * TOK + (n / NPT) * SEG + (n % NPT);
            sB[at] = rv_load_any(xbc, x_dtype, rowb + b_col + n);
            sC[at] = rv_load_any(xbc, x_dtype, rowb + c_col + n);
        }
#pragma unroll 4
        for (int i = tid; i < nt * COLS; i += 128) {
            const int tk = i / COLS, pp = p0 + (i - tk * COLS);
            sX[i] = pp < P ? rv_load_any(xbc, x_dtype, (size_t)(start + t0 + tk) * channels + h * P + pp) : 0.f;
        }
    };

    float run = 1.f;                                   // product of the decays from the segment's first token on
    const bool keeps_run = n_segs > 1 && tid == 0 && blockIdx.x == 0;
    if (vec && n_tok > 0) fetch(0);
    for (int t0 = 0; t0 < n_tok; t0 += RV_SCAN_CHUNK) {
        const int nt = n_tok - t0 < RV_SCAN_CHUNK ? n_tok - t0 : RV_SCAN_CHUNK;
        __syncthreads();                               // the chunk before has been read (and its sY written out)
        if (vec) stage(t0); else stage_plain(t0);
        __syncthreads();
        if (vec && t0 + RV_SCAN_CHUNK < n_tok) fetch(t0 + RV_SCAN_CHUNK);
        auto token = [&](int tk) {
            const float dec = sDec[tk], dtv = sDt[tk];
            run *= dec;
            if (keeps_run) dcum[(size_t)(start + t0 + tk) * heads + h] = run;
            const float4* B4 = reinterpret_cast<const float4*>(sB + tk * TOK + slice * SEG);
            const float4* C4 = reinterpret_cast<const float4*>(sC + tk * TOK + slice * SEG);
            float xv[NC], dx[NC], acc[NC][4];
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                xv[c] = sX[tk * COLS + lane_p + c];
                dx[c] = dtv * xv[c];
                acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < NPT / 4; ++j) {
                const float4 b = B4[j], cc = C4[j];            // one read of B and C serves the thread's NC columns
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    s[c][4 * j] = fmaf(dec, s[c][4 * j], dx[c] * b.x);         acc[c][0] = fmaf(s[c][4 * j], cc.x, acc[c][0]);
                    s[c][4 * j + 1] = fmaf(dec, s[c][4 * j + 1], dx[c] * b.y); acc[c][1] = fmaf(s[c][4 * j + 1], cc.y, acc[c][1]);
                    s[c][4 * j + 2] = fmaf(dec, s[c][4 * j + 2], dx[c] * b.z); acc[c][2] = fmaf(s[c][4 * j + 2], cc.z, acc[c][2]);
                    s[c][4 * j + 3] = fmaf(dec, s[c][4 * j + 3], dx[c] * b.w); acc[c][3] = fmaf(s[c][4 * j + 3], cc.w, acc[c][3]);
                }
            }
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                float a = (acc[c][0] + acc[c][1]) + (acc[c][2] + acc[c][3]);
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                a += __shfl_xor_sync(0xffffffffu, a, 2);
                a += __shfl_xor_sync(0xffffffffu, a, 4);
                if (slice == 0) sY[tk * COLS + lane_p + c] = fmaf(Dh, xv[c], a);
            }
        };
        if (nt == RV_SCAN_CHUNK) {                      // a whole chunk: unrolled, so that a token's loads overlap the one before
#pragma unroll 4
            for (int tk = 0; tk < RV_SCAN_CHUNK; ++tk) token(tk);
        } else {
            for (int tk = 0; tk < nt; ++tk) token(tk);
        }
        __syncthreads();
        for (int i = tid; i < nt * COLS; i += blockDim.x) {
            const int tk = i / COLS, pp = p0 + (i - tk * COLS);
            if (pp < P) y[(size_t)(start + t0 + tk) * inner + h * P + pp] = sY[i];
        }
    }
    float* S_out = n_segs == 1 ? S : seg_state + ((size_t)blockIdx.z * heads + h) * N * P;
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int n = slice * NPT + i;
            if (p + c < P && n < N) S_out[(size_t)n * P + p + c] = s[c][i];
        }
    if (keeps_run) seg_decay[(size_t)blockIdx.z * heads + h] = run;
}

// A sequence of several segments: element by element, the state walks through the segments,
//     S_start(1) = what segment 0 left (it started from the request's state),  S_start(k + 1) = decay(k) S_start(k) + S_local(k),
// every S_local(k), k >= 1, in scratch is replaced by S_start(k), and the last value becomes the request's state.
__global__ void __launch_bounds__(256)
ssm_segment_carry_kernel(const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, float* __restrict__ state,
                         size_t state_stride, float* __restrict__ seg_state, const float* __restrict__ seg_decay, int heads,
                         int NP, int seg_tokens, int max_segs) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int h = blockIdx.y, seq = blockIdx.z;
    if (e >= NP) return;
    const int n_segs = (cu_seqlens[seq + 1] - cu_seqlens[seq] + seg_tokens - 1) / seg_tokens;
    const int slot = state_slots[seq];
    if (n_segs <= 1 || slot < 0) return;
    float* sp = state + (size_t)slot * state_stride + (size_t)h * NP + e;
    // segment 0 started from the request's state, so what it left is already the state at the start of segment 1
    float S = seg_state[(((size_t)seq * max_segs) * heads + h) * NP + e];
    for (int k = 1; k < n_segs; ++k) {
        const size_t idx = ((size_t)seq * max_segs + k) * heads + h;
        const float local = seg_state[idx * NP + e];
        seg_state[idx * NP + e] = S;
        S = fmaf(seg_decay[idx], S, local);
    }
    *sp = S;
}

// What the state at a segment's start adds to the outputs of its tokens (segments 1 and later; the scan ran them from zero):
//     y_t += (product of the decays from the segment's first token to t) * S_start^T C_t.
// Grid (P / 32, heads, sequences x segments); 128 threads = 32 columns x 4 groups of 4 tokens of a chunk of 16.
__global__ void __launch_bounds__(128)
ssm_segment_correct_kernel(const void* __restrict__ xbc, int x_dtype, int channels, const int* __restrict__ cu_seqlens,
                           const int* __restrict__ state_slots, const float* __restrict__ seg_state,
                           const float* __restrict__ dcum, float* __restrict__ y, int heads, int P, int N, int groups,
                           int seg_tokens, int max_segs) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ __align__(16) float sm[];
    float* sS = sm;                  // [N][32]  S_start of this head's 32 columns
    float* sCt = sm + N * 32;        // [N][16]  C of a chunk's tokens, transposed
    const int seq = blockIdx.z / max_segs, seg = blockIdx.z - seq * max_segs;
    const int h = blockIdx.y, p0 = blockIdx.x * 32;
    const int seq_start = cu_seqlens[seq], seq_tok = cu_seqlens[seq + 1] - seq_start;
    const int n_segs = (seq_tok + seg_tokens - 1) / seg_tokens;
    if (seg == 0 || seg >= n_segs || state_slots[seq] < 0) return;
    const int start = seq_start + seg * seg_tokens;
    const int n_tok = seq_tok - seg * seg_tokens < seg_tokens ? seq_tok - seg * seg_tokens : seg_tokens;
    const int inner = heads * P, g = h / (heads / groups);
    const size_t c_col = (size_t)inner + (size_t)groups * N + (size_t)g * N;
    const float* S0 = seg_state + ((size_t)blockIdx.z * heads + h) * N * P;
    const int tid = threadIdx.x, pl = tid & 31, tq = tid >> 5;
    for (int i = tid; i < N * 32; i += 128) {
        const int n = i >> 5, pp = p0 + (i & 31);
        sS[i] = pp < P ? S0[(size_t)n * P + pp] : 0.f;
    }
    for (int t0 = 0; t0 < n_tok; t0 += 16) {
        const int nt = n_tok - t0 < 16 ? n_tok - t0 : 16;
        __syncthreads();
#pragma unroll 4
        for (int i = tid; i < 16 * N; i += 128) {
            const int tk = i / N, n = i - tk * N;
            sCt[n * 16 + tk] = tk < nt ? rv_load_any(xbc, x_dtype, (size_t)(start + t0 + tk) * channels + c_col + n) : 0.f;
        }
        __syncthreads();
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 8
        for (int n = 0; n < N; ++n) {
            const float sv = sS[n * 32 + pl];
            const float4 c = *reinterpret_cast<const float4*>(sCt + n * 16 + tq * 4);
            a0 = fmaf(sv, c.x, a0); a1 = fmaf(sv, c.y, a1); a2 = fmaf(sv, c.z, a2); a3 = fmaf(sv, c.w, a3);
        }
        const float acc[4] = {a0, a1, a2, a3};
        if (p0 + pl < P)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int tk = tq * 4 + j;
                if (tk < nt) {
                    const size_t t = (size_t)(start + t0 + tk);
                    y[t * inner + h * P + p0 + pl] += dcum[t * heads + h] * acc[j];
                }
            }
    }
}

template <int NPT, int NC>
static int launch_scan(cudaStream_t stream, const void* xbc, int x_dtype, int channels, const void* dt_in, int dt_dtype,
                       int dt_stride, int dt_col0, const void* dt_bias, const void* a_log, const void* d_skip, int p_dtype,
                       const int* cu_seqlens, const int* state_slots, float* state, size_t state_stride, float* y, int n_seqs,
                       int heads, int P, int N, int groups, int seg_tokens, int max_segs, float* seg_state, float* seg_decay,
                       float* dcum) {
    constexpr int COLS = NC * 16;
    const dim3 grid((P + COLS - 1) / COLS, heads, n_seqs * max_segs);
    const size_t smem = sizeof(float) * ((size_t)2 * RV_SCAN_CHUNK * 8 * (NPT + 4) + 2 * RV_SCAN_CHUNK * COLS + 2 * RV_SCAN_CHUNK);
    static RvPerDevice configured;
    if (smem > 48 * 1024)
        if (int e = rv_configure_smem(configured, ssm_scan_kernel<NPT, NC>, (int)smem)) return e;
    return rv_launch(ssm_scan_kernel<NPT, NC>, grid, dim3(128), smem, stream, xbc, x_dtype, channels, dt_in, dt_dtype, dt_stride, dt_col0,
                     dt_bias, a_log, d_skip, p_dtype, cu_seqlens, state_slots, state, state_stride, y, heads, P, N, groups,
                     seg_tokens, max_segs, seg_state, seg_decay, dcum);
}

// `columns`: columns per thread, 1 or 2; 0 lets the launcher choose by the size of the grid.
// `seg_tokens` > 0 (a multiple of 16): sequences are cut into segments of that many tokens that run side by side
// (`max_segs` = the most segments of any sequence; scratch: seg_state [n_seqs * max_segs, heads, N, P], seg_decay
// [n_seqs * max_segs, heads], dcum [tokens, heads], all float), then two small kernels carry the state through the segments
// and add what each segment's starting state contributes to its outputs.  The results equal the one-pass walk up to
// float32 rounding.
RV_EXPORT int rv_ssm_scan(const void* xbc, int x_dtype, int channels, const void* dt_in, int dt_dtype, int dt_stride, int dt_col0,
                          const void* dt_bias, const void* a_log, const void* d_skip, int p_dtype, const int* cu_seqlens,
                          const int* state_slots, float* state, long long state_stride, float* y, int n_seqs, int heads, int P,
                          int N, int groups, int columns, int seg_tokens, int max_segs, float* seg_state, float* seg_decay,
                          float* dcum, cudaStream_t stream) {
    if (n_seqs < 0 || heads <= 0 || P <= 0 || N <= 0 || groups <= 0 || heads % groups) return RV_ERR_BAD_SIZE;
    if (channels < heads * P + 2 * groups * N || dt_stride < dt_col0 + heads || dt_col0 < 0) return RV_ERR_BAD_SIZE;
    if ((x_dtype | dt_dtype | p_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (columns < 0 || columns > 2) return RV_ERR_BAD_SIZE;
    if (N > 256 || heads > 65535 || n_seqs > 65535) return RV_ERR_UNSUPPORTED;
    if (n_seqs == 0) return RV_OK;
    if (seg_tokens < 0 || (seg_tokens & 15)) return RV_ERR_BAD_SIZE;
    if (seg_tokens == 0) max_segs = 1;
    else if (max_segs < 1 || !seg_state || !seg_decay || !dcum) return RV_ERR_BAD_SIZE;
    if ((long long)n_seqs * max_segs > 65535) return RV_ERR_UNSUPPORTED;
    // one column per thread (16 per block) only where blocks of 32 columns would leave half of the SMs without one, and for
    // the largest states (two columns of 32 state values each would not fit the registers)
    const bool narrow = columns ? columns == 1 : (N > 128 || 2LL * ((P + 31) / 32) * heads * n_seqs * max_segs <= (long long)rv_sm_count());
#define RV_SCAN_LAUNCH(NPT, NC)                                                                                                  \
    RV_LAUNCH_ST = launch_scan<NPT, NC>(stream, xbc, x_dtype, channels, dt_in, dt_dtype, dt_stride, dt_col0, dt_bias, a_log,     \
                                        d_skip, p_dtype, cu_seqlens, state_slots, state, (size_t)state_stride, y, n_seqs, heads, P, N, groups, \
                                        seg_tokens, max_segs, seg_state, seg_decay, dcum)
    if (narrow || N > 128) {
        if (N <= 32) RV_SCAN_LAUNCH(4, 1);
        else if (N <= 64) RV_SCAN_LAUNCH(8, 1);
        else if (N <= 128) RV_SCAN_LAUNCH(16, 1);
        else RV_SCAN_LAUNCH(32, 1);
    } else {
        if (N <= 32) RV_SCAN_LAUNCH(4, 2);
        else if (N <= 64) RV_SCAN_LAUNCH(8, 2);
        else RV_SCAN_LAUNCH(16, 2);
    }
#undef RV_SCAN_LAUNCH
    if (seg_tokens == 0 || max_segs == 1 || RV_LAUNCH_ST != RV_OK) return rv_launch_status();
    const int NP = N * P;
    RV_LAUNCH_ST = rv_launch(ssm_segment_carry_kernel, dim3((NP + 255) / 256, heads, n_seqs), dim3(256), 0, stream, cu_seqlens, state_slots,
                             state, (size_t)state_stride, seg_state, (const float*)seg_decay, heads, NP, seg_tokens, max_segs);
    if (RV_LAUNCH_ST != RV_OK) return rv_launch_status();
    RV_LAUNCH_ST = rv_launch(ssm_segment_correct_kernel, dim3((P + 31) / 32, heads, n_seqs * max_segs), dim3(128), (size_t)N * 48 * sizeof(float),
                             stream, xbc, x_dtype, channels, cu_seqlens, state_slots, (const float*)seg_state, (const float*)dcum, y, heads, P,
                             N, groups, seg_tokens, max_segs);
    return rv_launch_status();
}

// ------------------------------------------------------------------ the recurrence with one state row per channel
// The older form of the selective scan: every channel c has its own decays A[c, :] and its own step size,
//     S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n ,   y_c = sum_n S[c, n] C_n + D_c u_c ,   out_c = y_c silu(z_c)
// with dt_c = softplus(raw_c + bias_c); B and C are shared by all channels of a token.  S lives as [inner][N] at
// offset 0 of the request's state row.  A channel is served by `parts` neighbouring lanes with up to NS states
// each (partial sums meet by shuffles), a block by 128 threads; grid (channel blocks, sequences).  The tokens' B
// and C wait in shared memory in chunks of SCAN1_CHUNK tokens.
#define SCAN1_CHUNK 16
#define SCAN1_PRE 4          // per thread: (token, channel) pairs of a chunk that the prefetch holds, 128 / parts <= 8 * SCAN1_PRE
#define SCAN1_PRE_BC 8       // per thread: B | C entries of a chunk that the prefetch holds, 2 N <= 8 * SCAN1_PRE_BC

// Shared memory (floats): B | C of the chunk [SCAN1_CHUNK][2 N], then per token and channel of the block the step size
// [SCAN1_CHUNK][per_block] and the input [SCAN1_CHUNK][per_block] (which the walk overwrites with y).  Softplus, the loads
// of a chunk and the gate y silu(z) with its store are done by all threads side by side; only the recurrence itself
// walks token by token, out of shared memory, four tokens at a time: their decays and inputs are worked out first (they
// do not depend on the state), so that the chain from token to token is one multiply-add per state; the last one to
// three tokens of a sequence go one by one.
// PRE: the raw inputs of the next chunk are loaded into registers, unconverted, before the current one is walked.
template <int NS, bool PRE>
__global__ void __launch_bounds__(128)
selective_scan1_kernel(const void* __restrict__ u, int u_dtype, const float* __restrict__ dt_raw, const float* __restrict__ dt_bias,
                       const float* __restrict__ A, const float* __restrict__ bc, int bc_stride, int b_col0, int c_col0,
                       const float* __restrict__ d_skip, const void* __restrict__ z, int z_dtype, int z_stride, int z_col0,
                       const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, float* __restrict__ state,
                       size_t state_stride, void* __restrict__ out, int out_dtype, int inner, int N, int parts) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ float sBC[];                     // [SCAN1_CHUNK][2 N]
    const int seq = blockIdx.y;
    const int slot = state_slots[seq];
    if (slot < 0) return;
    const int start = cu_seqlens[seq], n_tok = cu_seqlens[seq + 1] - start;
    const int per_block = blockDim.x / parts;
    float* sDt = sBC + SCAN1_CHUNK * 2 * N;            // [SCAN1_CHUNK][per_block]
    float* sU = sDt + SCAN1_CHUNK * per_block;         // [SCAN1_CHUNK][per_block]
    const int c_first = blockIdx.x * per_block;
    const int cl = threadIdx.x / parts;
    const int c = c_first + cl;
    const int part = threadIdx.x % parts;
    const bool live = c < inner;
    const int n0 = part * NS;
    float S[NS], a[NS];
    float* srow = state + (size_t)slot * state_stride + (size_t)c * N;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const bool ok = live && n0 + i < N;
        S[i] = ok ? srow[n0 + i] : 0.f;
        a[i] = ok ? A[(size_t)c * N + n0 + i] : 0.f;
    }
    const float dsk = live ? d_skip[c] : 0.f;

    float p_dt[SCAN1_PRE], p_bias[SCAN1_PRE], p_bc[SCAN1_PRE_BC];
    uint32_t p_u[SCAN1_PRE], p_z[SCAN1_PRE];
    auto load_chunk = [&](int t0) {                    // PRE only
        const int nt = min(SCAN1_CHUNK, n_tok - t0);
#pragma unroll
        for (int y = 0; y < SCAN1_PRE; ++y) {
            const int i = threadIdx.x + 128 * y;
            const int tt = i / per_block, cc = c_first + (i - tt * per_block);
            p_dt[y] = 0.f; p_bias[y] = 0.f; p_u[y] = 0; p_z[y] = 0;
            if (tt < nt && cc < inner) {
                const size_t row = (size_t)(start + t0 + tt);
                p_dt[y] = dt_raw[row * inner + cc];
                p_bias[y] = dt_bias[cc];
                p_u[y] = rv_load_raw(u, u_dtype, row * inner + cc);
                p_z[y] = rv_load_raw(z, z_dtype, row * z_stride + z_col0 + cc);
            }
        }
#pragma unroll
        for (int y = 0; y < SCAN1_PRE_BC; ++y) {
            const int i = threadIdx.x + 128 * y;
            const int tt = i / (2 * N), j = i - tt * 2 * N;
            p_bc[y] = 0.f;
            if (tt < nt) p_bc[y] = bc[(size_t)(start + t0 + tt) * bc_stride + (j < N ? b_col0 + j : c_col0 + j - N)];
        }
    };
    const bool pre = PRE && n_tok > SCAN1_CHUNK;         // (a short portion, a decode step's single token: loaded when its turn comes)
    if (pre) load_chunk(0);
    for (int t0 = 0; t0 < n_tok; t0 += SCAN1_CHUNK) {
        const int nt = min(SCAN1_CHUNK, n_tok - t0);
        float zs[SCAN1_PRE];                               // PRE: silu(z) of this thread's (token, channel) pairs
        __syncthreads();
        if (pre) {
#pragma unroll
            for (int y = 0; y < SCAN1_PRE_BC; ++y) {
                const int i = threadIdx.x + 128 * y;
                if (i < SCAN1_CHUNK * 2 * N) sBC[i] = p_bc[y];
            }
#pragma unroll
            for (int y = 0; y < SCAN1_PRE; ++y) {
                const int i = threadIdx.x + 128 * y;
                if (i < SCAN1_CHUNK * per_block) {
                    const float raw = p_dt[y] + p_bias[y];
                    const bool real = i < nt * per_block;
                    sDt[i] = real ? (raw > 20.f ? raw : log1pf(expf(raw))) : 0.f;
                    sU[i] = rv_raw_value(p_u[y], u_dtype);
                    const float zv = rv_raw_value(p_z[y], z_dtype);
                    zs[y] = zv / (1.0f + expf(-zv));
                }
            }
        } else {
            for (int i = threadIdx.x; i < nt * 2 * N; i += blockDim.x) {
                const int tt = i / (2 * N), j = i - tt * 2 * N;
                sBC[i] = bc[(size_t)(start + t0 + tt) * bc_stride + (j < N ? b_col0 + j : c_col0 + j - N)];
            }
            for (int i = threadIdx.x; i < nt * per_block; i += blockDim.x) {
                const int tt = i / per_block, cc = c_first + (i - tt * per_block);
                float dt = 0.f, uv = 0.f;
                if (cc < inner) {
                    const size_t row = (size_t)(start + t0 + tt);
                    const float raw = dt_raw[row * inner + cc] + dt_bias[cc];
                    dt = raw > 20.f ? raw : log1pf(expf(raw));
                    uv = rv_load_any(u, u_dtype, row * inner + cc);
                }
                sDt[i] = dt;
                sU[i] = uv;
            }
        }
        __syncthreads();
        if (pre && t0 + SCAN1_CHUNK < n_tok) load_chunk(t0 + SCAN1_CHUNK);
        int tt0 = 0;
        for (; tt0 + 4 <= nt; tt0 += 4) {                   // (threads beyond the last channel walk along: the shuffles need every lane)
            float dec[4][NS], dub[4][NS], uv[4], acc[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const float dt = sDt[(tt0 + x) * per_block + cl];
                uv[x] = sU[(tt0 + x) * per_block + cl];
                const float du = dt * uv[x];
                const float* B = sBC + (tt0 + x) * 2 * N + n0;
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    const bool ok = n0 + i < N;
                    dec[x][i] = expf(dt * a[i]);
                    dub[x][i] = ok ? du * B[i] : 0.f;
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const float* C = sBC + (tt0 + x) * 2 * N + N + n0;
                acc[x] = 0.f;
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    S[i] = fmaf(dec[x][i], S[i], dub[x][i]);
                    acc[x] = fmaf(S[i], n0 + i < N ? C[i] : 0.f, acc[x]);
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                for (int o = 1; o < parts; o <<= 1) acc[x] += __shfl_xor_sync(0xffffffffu, acc[x], o);
                if (part == 0) sU[(tt0 + x) * per_block + cl] = fmaf(dsk, uv[x], acc[x]);
            }
        }
        for (int tt = tt0; tt < nt; ++tt) {                 // the last one to three tokens of a sequence (a decode step's only one)
            const float dt = sDt[tt * per_block + cl];
            const float uv = sU[tt * per_block + cl];
            const float du = dt * uv;
            const float* B = sBC + tt * 2 * N + n0;
            const float* C = B + N;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < NS; ++i) {
                if (n0 + i < N) {
                    S[i] = fmaf(expf(dt * a[i]), S[i], du * B[i]);
                    acc = fmaf(S[i], C[i], acc);
                }
            }
            for (int o = 1; o < parts; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (part == 0) sU[tt * per_block + cl] = fmaf(dsk, uv, acc);
        }
        __syncthreads();
        if (pre) {
#pragma unroll
            for (int y = 0; y < SCAN1_PRE; ++y) {
                const int i = threadIdx.x + 128 * y;
                const int tt = i / per_block, cc = c_first + (i - tt * per_block);
                if (i < nt * per_block && cc < inner) rv_store_any(out, out_dtype, (size_t)(start + t0 + tt) * inner + cc, sU[i] * zs[y]);
            }
        } else {
            for (int i = threadIdx.x; i < nt * per_block; i += blockDim.x) {
                const int tt = i / per_block, cc = c_first + (i - tt * per_block);
                if (cc < inner) {
                    const size_t row = (size_t)(start + t0 + tt);
                    const float zv = rv_load_any(z, z_dtype, row * z_stride + z_col0 + cc);
                    rv_store_any(out, out_dtype, row * inner + cc, sU[i] * (zv / (1.0f + expf(-zv))));
                }
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NS; ++i)
            if (n0 + i < N) srow[n0 + i] = S[i];
    }
}

RV_EXPORT int rv_selective_scan1(const void* u, int u_dtype, const float* dt_raw, const float* dt_bias, const float* A,
                                 const float* bc, int bc_stride, int b_col0, int c_col0, const float* d_skip, const void* z,
                                 int z_dtype, int z_stride, int z_col0, const int* cu_seqlens, const int* state_slots, float* state,
                                 long long state_stride, void* out, int out_dtype, int n_seqs, int inner, int N, cudaStream_t stream) {
    if (n_seqs < 0 || inner <= 0 || N <= 0 || N > 32 * 16 || n_seqs > 65535) return RV_ERR_BAD_SIZE;
    if (b_col0 < 0 || c_col0 < 0 || b_col0 + N > bc_stride || c_col0 + N > bc_stride || z_col0 < 0 || z_col0 + inner > z_stride ||
        state_stride < (long long)inner * N)
        return RV_ERR_BAD_SIZE;
    if ((u_dtype | z_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (n_seqs == 0) return RV_OK;
    // four states per lane where a warp's lanes can hold a channel's row so (neighbouring lanes then read neighbouring
    // 16 bytes of the state, and four times as many threads walk the tokens); sixteen per lane for longer rows
    const int ns = N <= 32 * 4 ? 4 : 16;
    int parts = 1;
    while (parts * ns < N) parts <<= 1;                // a power of two of at most 32 lanes of one warp
    const int per_block = 128 / parts;
    const size_t smem = (size_t)SCAN1_CHUNK * (2 * N + 2 * per_block) * sizeof(float);
    if (smem > 48 * 1024) return RV_ERR_UNSUPPORTED;
    const bool pre = per_block <= 8 * SCAN1_PRE && 2 * N <= 8 * SCAN1_PRE_BC;
    auto kernel = ns == 4 ? (pre ? selective_scan1_kernel<4, true> : selective_scan1_kernel<4, false>)
                          : (pre ? selective_scan1_kernel<16, true> : selective_scan1_kernel<16, false>);
    RV_LAUNCH_ST = rv_launch(kernel, dim3((inner + per_block - 1) / per_block, n_seqs), dim3(128), smem, stream, u, u_dtype, dt_raw,
                             dt_bias, A, bc, bc_stride, b_col0, c_col0, d_skip, z, z_dtype, z_stride, z_col0, cu_seqlens, state_slots,
                             state, (size_t)state_stride, out, out_dtype, inner, N, parts);
    return rv_launch_status();
}

// ------------------------------------------------------------------ the gated delta rule
// Per value head h, with S of size d x vd (d: key size, vd: value size) kept as [heads][d][vd] at offset 0 of the request's
// state row:
//     q <- q / sqrt(sum q^2 + unit_eps) d^(-1/2),   k <- k / sqrt(sum k^2 + unit_eps)          (q/k head h / (heads / qk_heads))
//     beta = sigmoid(b),   g = exp(-exp(A_log_h) softplus(a + dt_bias_h))
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// Every step of the rule acts on the columns of S one by one, so a column is one thread's work (no exchange between
// columns): a column's d entries live in the registers of `parts` lanes, NS each, whose partial sums
// meet by shuffles.  Grid (column blocks, heads, sequences), 128 threads.  The unit vectors q and k of DR_CHUNK tokens, and
// the tokens' g and beta, wait in shared memory; a lane's NS entries of a row start at a multiple of NS + 4 floats, so
// that the 16-byte reads of the `parts` lanes of a column fall on different banks.  Rows are zero beyond d.
#define DR_CHUNK 16
#define DR_PRE_Q 4          // q (and k) elements per lane and token that the prefetch holds: d <= 32 * DR_PRE_Q
#define DR_PRE_V 8          // values per thread and chunk that the prefetch holds: 128 / parts <= 8 * DR_PRE_V

// PRE: the raw inputs of the next chunk are loaded into registers before the current chunk is walked, so that their way
// from memory lies behind the walk; without it (wider keys, or more columns per block than the registers hold) a chunk
// is loaded when its turn comes.
// NS: entries of a column per lane (8, 16 or 32: a key of up to 4 NS entries lies in four lanes).
template <int NS, bool PRE>
__global__ void __launch_bounds__(128)
delta_rule_kernel(const void* __restrict__ qkv, int qkv_dtype, int qkv_stride, const float* __restrict__ proj, int proj_stride,
                  int b_col0, int a_col0, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, float* __restrict__ state,
                  size_t state_stride, float* __restrict__ out, int heads, int qk_heads, int d, int vd, int parts, float unit_eps) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ __align__(16) float dr_smem[];
    const int seq = blockIdx.z, h = blockIdx.y;
    const int slot = state_slots[seq];
    if (slot < 0) return;
    const int start = cu_seqlens[seq], n_tok = cu_seqlens[seq + 1] - start;
    const int row_floats = parts * (NS + 4);
    float* sQ = dr_smem;                                   // [DR_CHUNK][row_floats]
    float* sK = sQ + DR_CHUNK * row_floats;
    float* sG = sK + DR_CHUNK * row_floats;                // [DR_CHUNK]
    float* sBeta = sG + DR_CHUNK;
    float* sV = sBeta + DR_CHUNK;                          // [DR_CHUNK][128 / parts]: the chunk's values of the block's columns
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per_block = 128 / parts;
    // a warp holds 32 / parts neighbouring columns; the `parts` lanes of a column lie 32 / parts lanes apart, so that
    // neighbouring lanes read and write neighbouring floats of the state
    const int cpw = 32 / parts;
    const int colb = warp * cpw + lane % cpw;
    const int col = blockIdx.x * per_block + colb;
    const int part = lane / cpw;
    const bool live = col < vd;
    const int n0 = part * NS;
    const int kh = h / (heads / qk_heads);
    const int qk = qk_heads * d;
    const float q_scale = rsqrtf((float)d);
    float S[NS];
    float* srow = state + (size_t)slot * state_stride + (size_t)h * d * vd;
#pragma unroll
    for (int i = 0; i < NS; ++i) S[i] = (live && n0 + i < d) ? srow[(size_t)(n0 + i) * vd + col] : 0.f;
    for (int i = tid; i < 2 * DR_CHUNK * row_floats; i += 128) dr_smem[i] = 0.f;      // the padding stays zero from here on
    const float decay_rate = expf(a_log[h]), a_bias = dt_bias[h];

    uint32_t pq[DR_CHUNK / 4][DR_PRE_Q], pk[DR_CHUNK / 4][DR_PRE_Q], pv[DR_PRE_V];      // raw bits: converted when their chunk's turn comes
    float pb = 0.f, pa = 0.f;
    auto load_chunk = [&](int t0) {                       // PRE only: the chunk's raw q, k (a warp per token), v, b and a
        const int nt = min(DR_CHUNK, n_tok - t0);
#pragma unroll
        for (int x = 0; x < DR_CHUNK / 4; ++x) {
            const int tt = warp + 4 * x;
            const size_t row = (size_t)(start + t0 + tt) * qkv_stride + (size_t)kh * d;
#pragma unroll
            for (int y = 0; y < DR_PRE_Q; ++y) {
                const int e = lane + 32 * y;
                pq[x][y] = 0; pk[x][y] = 0;
                if (tt < nt && e < d) {
                    pq[x][y] = rv_load_raw(qkv, qkv_dtype, row + e);
                    pk[x][y] = rv_load_raw(qkv, qkv_dtype, row + qk + e);
                }
            }
        }
#pragma unroll
        for (int y = 0; y < DR_PRE_V; ++y) {
            const int i = tid + 128 * y;
            const int tt = i / per_block, cc = blockIdx.x * per_block + (i - tt * per_block);
            pv[y] = 0;
            if (tt < nt && cc < vd) pv[y] = rv_load_raw(qkv, qkv_dtype, (size_t)(start + t0 + tt) * qkv_stride + 2 * qk + (size_t)h * vd + cc);
        }
        if (tid < nt) {
            const size_t row = (size_t)(start + t0 + tid) * proj_stride;
            pb = proj[row + b_col0 + h];
            pa = proj[row + a_col0 + h];
        }
    };
    const bool pre = PRE && n_tok > DR_CHUNK;           // (a short portion, a decode step's single token: loaded when its turn comes)
    if (pre) load_chunk(0);
    for (int t0 = 0; t0 < n_tok; t0 += DR_CHUNK) {
        const int nt = min(DR_CHUNK, n_tok - t0);
        __syncthreads();
        if (pre) {
#pragma unroll
            for (int x = 0; x < DR_CHUNK / 4; ++x) {
                const int tt = warp + 4 * x;                                  // (a warp-uniform test)
                if (tt < nt) {
                    float sq = 0.f, sk = 0.f, fq[DR_PRE_Q], fk[DR_PRE_Q];
#pragma unroll
                    for (int y = 0; y < DR_PRE_Q; ++y) {
                        fq[y] = rv_raw_value(pq[x][y], qkv_dtype);
                        fk[y] = rv_raw_value(pk[x][y], qkv_dtype);
                        sq = fmaf(fq[y], fq[y], sq);
                        sk = fmaf(fk[y], fk[y], sk);
                    }
                    sq = rv_warp_sum(sq);
                    sk = rv_warp_sum(sk);
                    const float rq = q_scale / sqrtf(sq + unit_eps), rk = 1.0f / sqrtf(sk + unit_eps);
#pragma unroll
                    for (int y = 0; y < DR_PRE_Q; ++y) {
                        const int e = lane + 32 * y;
                        if (e < d) {
                            const int at = tt * row_floats + (e / NS) * (NS + 4) + (e % NS);
                            sQ[at] = fq[y] * rq;
                            sK[at] = fk[y] * rk;
                        }
                    }
                }
            }
#pragma unroll
            for (int y = 0; y < DR_PRE_V; ++y) {
                const int i = tid + 128 * y;
                if (i < DR_CHUNK * per_block) sV[i] = rv_raw_value(pv[y], qkv_dtype);       // (zero beyond the sequence)
            }
            if (tid < DR_CHUNK) {                          // beyond the sequence: beta 0 and decay 1 leave the state as it is
                const float a = pa + a_bias;
                const float sp = a > 20.f ? a : log1pf(expf(a));
                sBeta[tid] = tid < nt ? 1.0f / (1.0f + expf(-pb)) : 0.f;
                sG[tid] = tid < nt ? expf(-decay_rate * sp) : 1.f;
            }
        } else {
            for (int tt = warp; tt < nt; tt += 4) {                       // a warp per token: q and k of the head, made unit vectors
                const size_t row = (size_t)(start + t0 + tt) * qkv_stride;
                float sq = 0.f, sk = 0.f;
                for (int e = lane; e < d; e += 32) {
                    const float qv = rv_load_any(qkv, qkv_dtype, row + (size_t)kh * d + e);
                    const float kv = rv_load_any(qkv, qkv_dtype, row + qk + (size_t)kh * d + e);
                    const int at = tt * row_floats + (e / NS) * (NS + 4) + (e % NS);
                    sQ[at] = qv;
                    sK[at] = kv;
                    sq = fmaf(qv, qv, sq);
                    sk = fmaf(kv, kv, sk);
                }
                sq = rv_warp_sum(sq);
                sk = rv_warp_sum(sk);
                const float rq = q_scale / sqrtf(sq + unit_eps), rk = 1.0f / sqrtf(sk + unit_eps);
                for (int e = lane; e < d; e += 32) {                      // every lane rescales what it wrote itself
                    const int at = tt * row_floats + (e / NS) * (NS + 4) + (e % NS);
                    sQ[at] *= rq;
                    sK[at] *= rk;
                }
            }
            for (int i = tid; i < nt * per_block; i += 128) {
                const int tt = i / per_block, cc = blockIdx.x * per_block + (i - tt * per_block);
                sV[i] = cc < vd ? rv_load_any(qkv, qkv_dtype, (size_t)(start + t0 + tt) * qkv_stride + 2 * qk + (size_t)h * vd + cc) : 0.f;
            }
            if (tid < nt) {
                const size_t row = (size_t)(start + t0 + tid) * proj_stride;
                const float b = proj[row + b_col0 + h];
                const float a = proj[row + a_col0 + h] + a_bias;
                const float sp = a > 20.f ? a : log1pf(expf(a));
                sBeta[tid] = 1.0f / (1.0f + expf(-b));
                sG[tid] = expf(-decay_rate * sp);
            }
        }
        __syncthreads();
        if (pre && t0 + DR_CHUNK < n_tok) load_chunk(t0 + DR_CHUNK);
        // (threads beyond the last column walk along: the shuffles need every lane)
        auto step = [&](int tt) {
            const size_t trow = (size_t)(start + t0 + tt);
            const float4* K4 = reinterpret_cast<const float4*>(sK + tt * row_floats + part * (NS + 4));
            const float4* Q4 = reinterpret_cast<const float4*>(sQ + tt * row_floats + part * (NS + 4));
            const float vv = sV[tt * per_block + colb];
            float kreg[NS];
            float ac[4] = {0.f, 0.f, 0.f, 0.f};                // four sums side by side: the chain of a column is a quarter as long
#pragma unroll
            for (int i = 0; i < NS / 4; ++i) {
                const float4 k4 = K4[i];
                kreg[4 * i] = k4.x; kreg[4 * i + 1] = k4.y; kreg[4 * i + 2] = k4.z; kreg[4 * i + 3] = k4.w;
                ac[0] = fmaf(S[4 * i], k4.x, ac[0]); ac[1] = fmaf(S[4 * i + 1], k4.y, ac[1]);
                ac[2] = fmaf(S[4 * i + 2], k4.z, ac[2]); ac[3] = fmaf(S[4 * i + 3], k4.w, ac[3]);
            }
            float acc = (ac[0] + ac[1]) + (ac[2] + ac[3]);
            for (int o = cpw; o < 32; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            const float g = sG[tt];
            const float u = sBeta[tt] * (vv - g * acc);
            float ov4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < NS / 4; ++i) {
                const float4 q4 = Q4[i];
                S[4 * i] = fmaf(g, S[4 * i], kreg[4 * i] * u);             ov4[0] = fmaf(S[4 * i], q4.x, ov4[0]);
                S[4 * i + 1] = fmaf(g, S[4 * i + 1], kreg[4 * i + 1] * u); ov4[1] = fmaf(S[4 * i + 1], q4.y, ov4[1]);
                S[4 * i + 2] = fmaf(g, S[4 * i + 2], kreg[4 * i + 2] * u); ov4[2] = fmaf(S[4 * i + 2], q4.z, ov4[2]);
                S[4 * i + 3] = fmaf(g, S[4 * i + 3], kreg[4 * i + 3] * u); ov4[3] = fmaf(S[4 * i + 3], q4.w, ov4[3]);
            }
            float ov = (ov4[0] + ov4[1]) + (ov4[2] + ov4[3]);
            for (int o = cpw; o < 32; o <<= 1) ov += __shfl_xor_sync(0xffffffffu, ov, o);
            if (part == 0 && live && tt < nt) out[trow * heads * vd + (size_t)h * vd + col] = ov;
        };
        if (nt == DR_CHUNK) {                              // a whole chunk: neighbouring tokens may run into one another
#pragma unroll 4
            for (int tt = 0; tt < DR_CHUNK; ++tt) step(tt);
        } else {
            for (int tt = 0; tt < nt; ++tt) step(tt);
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NS; ++i)
            if (n0 + i < d) srow[(size_t)(n0 + i) * vd + col] = S[i];
    }
}

// qkv rows: [q: qk_heads x d | k: qk_heads x d | v: heads x vd] (after the convolution); the logits of beta and of the
// decay are float columns b_col0 .. and a_col0 .. of `proj`; out: float [tokens, heads x vd].
RV_EXPORT int rv_delta_rule(const void* qkv, int qkv_dtype, int qkv_stride, const float* proj, int proj_stride, int b_col0,
                            int a_col0, const float* a_log, const float* dt_bias, const int* cu_seqlens, const int* state_slots,
                            float* state, long long state_stride, float* out, int n_seqs, int heads, int qk_heads, int d, int vd,
                            float unit_eps, cudaStream_t stream) {
    if (n_seqs < 0 || heads <= 0 || qk_heads <= 0 || heads % qk_heads || d <= 0 || d > 32 * 32 || vd <= 0 || n_seqs > 65535 ||
        heads > 65535)
        return RV_ERR_BAD_SIZE;
    if (qkv_stride < 2 * qk_heads * d + heads * vd || b_col0 < 0 || a_col0 < 0 || b_col0 + heads > proj_stride ||
        a_col0 + heads > proj_stride || state_stride < (long long)heads * d * vd)
        return RV_ERR_BAD_SIZE;
    if (qkv_dtype & ~1) return RV_ERR_BAD_DTYPE;
    if (n_seqs == 0) return RV_OK;
    const int ns = d > 64 ? 32 : (d > 32 ? 16 : 8);    // four lanes per column up to a key size of 128
    int parts = 1;
    while (parts * ns < d) parts <<= 1;                // a power of two of at most 32 lanes of one warp
    const int per_block = 128 / parts;
    const size_t smem = sizeof(float) * (2 * (size_t)DR_CHUNK * parts * (ns + 4) + 2 * DR_CHUNK + (size_t)DR_CHUNK * per_block);
    if (smem > 48 * 1024) return RV_ERR_UNSUPPORTED;
    const bool pre = d <= 32 * DR_PRE_Q && per_block <= 8 * DR_PRE_V;
    auto kernel = ns == 32 ? (pre ? delta_rule_kernel<32, true> : delta_rule_kernel<32, false>)
                : ns == 16 ? (pre ? delta_rule_kernel<16, true> : delta_rule_kernel<16, false>)
                           : (pre ? delta_rule_kernel<8, true> : delta_rule_kernel<8, false>);
    RV_LAUNCH_ST = rv_launch(kernel, dim3((vd + per_block - 1) / per_block, heads, n_seqs), dim3(128), smem, stream, qkv,
                             qkv_dtype, qkv_stride, proj, proj_stride, b_col0, a_col0, a_log, dt_bias, cu_seqlens, state_slots, state,
                             (size_t)state_stride, out, heads, qk_heads, d, vd, parts, unit_eps);
    return rv_launch_status();
}
