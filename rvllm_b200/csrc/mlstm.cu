// The mLSTM matrix memory: per head a state S of d x (vd + 1) floats and a running maximum m, walked token by token.
//
//     q <- q d^(-1/2);   i = cap tanh((i' + bi) / cap);   f = logsigmoid(cap tanh((f' + bf) / cap))      (logarithms of the gates)
//     m_t = max(f + m_(t-1), i);   a = exp(f + m_(t-1) - m_t);   b = exp(i - m_t)
//     S_t = a S_(t-1) + b k [v | 1]^T;      raw_t = S_t^T q       (vd + 1 numbers: the numerators and, last, n_t . q)
//
// The normaliser n of the design is the memory of the constant value 1: column vd of S.  Every step acts on the columns
// of S one by one, so a column is the work of `parts` lanes with NS entries each (registers), whose partial sums meet by
// shuffles.  Grid (column blocks, heads, sequences), 128 threads.  q, k of ML_CHUNK tokens and the tokens' a and b wait in
// shared memory; a lane's NS entries of a row start at a multiple of NS + 4 floats, so that the 16-byte reads of the
// lanes of a column fall on different banks.  The gates of a chunk are formed side by side, one thread walks the maximum
// through the chunk (an add and a max a token), and the exponentials are again formed side by side; the next chunk's raw
// inputs wait in registers behind the walk.  State row of a request: [heads][d][vd + 1], then m [heads]; all float32.
//
//   mlstm_scan     raw [tokens, heads x (vd + 1)] and top [tokens, heads] (m_t) from the float32 projection
//   mlstm_output   o = raw / (max(|n . q|, exp(-m)) + den_eps);  o / sqrt(mean(o^2) + eps) per head, times a weight per
//                  element, times sigmoid of the gate columns; in the activations' type.  It also stores the m of a
//                  sequence's last token into the request's state row (the scan's column blocks all read the old one)
#include "common.cuh"

#define ML_CHUNK 16
#define ML_PRE_Q 4          // q (and k) elements per lane and token that the prefetch holds: d <= 32 * ML_PRE_Q
#define ML_PRE_V 8          // values per thread and chunk that the prefetch holds: 128 / parts <= 8 * ML_PRE_V

// PRE: the raw inputs of the next chunk are loaded into registers before the current chunk is walked, so that their way
// from memory lies behind the walk; without it (wider keys, or more columns per block than the registers hold) a chunk
// is loaded when its turn comes.
template <int NS, bool PRE>
__global__ void __launch_bounds__(128)
mlstm_scan_kernel(const float* __restrict__ proj, int stride, int i_col0, int f_col0, const float* __restrict__ i_bias,
                  const float* __restrict__ f_bias, const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                  float* __restrict__ state, size_t state_stride, float* __restrict__ raw, float* __restrict__ top, int heads, int d,
                  int vd, int parts, float cap) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ __align__(16) float ml_smem[];
    const int seq = blockIdx.z, h = blockIdx.y;
    const int slot = state_slots[seq];
    if (slot < 0) return;
    const int start = cu_seqlens[seq], n_tok = cu_seqlens[seq + 1] - start;
    const int row_floats = parts * (NS + 4);
    float* sQ = ml_smem;                                   // [ML_CHUNK][row_floats]
    float* sK = sQ + ML_CHUNK * row_floats;
    float* sA = sK + ML_CHUNK * row_floats;                // [ML_CHUNK] decay of the state
    float* sB = sA + ML_CHUNK;                             // [ML_CHUNK] weight of the new outer product
    float* sI = sB + ML_CHUNK;                             // [ML_CHUNK] log input gate
    float* sF = sI + ML_CHUNK;                             // [ML_CHUNK] log forget gate
    float* sM = sF + ML_CHUNK;                             // [ML_CHUNK + 1] the running maximum before and after each token
    float* sV = sM + ML_CHUNK + 4;                         // [ML_CHUNK][128 / parts]: the chunk's values of the block's columns
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per_block = 128 / parts;
    // a warp holds 32 / parts neighbouring columns; the `parts` lanes of a column lie 32 / parts lanes apart, so that
    // neighbouring lanes read and write neighbouring floats of the state
    const int cpw = 32 / parts;
    const int colb = warp * cpw + lane % cpw;
    const int col = blockIdx.x * per_block + colb;
    const int part = lane / cpw;
    const int width = vd + 1;                              // columns of a head's state: the values and the constant 1
    const bool live = col < width;
    const int n0 = part * NS;
    const int qk = heads * d;
    const float q_scale = rsqrtf((float)d);
    float S[NS];
    float* srow = state + (size_t)slot * state_stride + (size_t)h * d * width;
    const float* mrow = state + (size_t)slot * state_stride + (size_t)heads * d * width + h;
#pragma unroll
    for (int i = 0; i < NS; ++i) S[i] = (live && n0 + i < d) ? srow[(size_t)(n0 + i) * width + col] : 0.f;
    for (int i = tid; i < 2 * ML_CHUNK * row_floats; i += 128) ml_smem[i] = 0.f;      // the padding stays zero from here on
    float m = *mrow;                                       // (every thread reads it; thread 0 carries it)
    const float bi = i_bias[h], bf = f_bias[h];
    const float inv_cap = 1.0f / cap;
    float pq[ML_CHUNK / 4][ML_PRE_Q], pk[ML_CHUNK / 4][ML_PRE_Q], pv[ML_PRE_V];
    float pgi = 0.f, pgf = 0.f;
    auto load_chunk = [&](int t0) {                       // PRE only: the chunk's raw q, k (a warp per token), v and gate logits
        const int nt = min(ML_CHUNK, n_tok - t0);
#pragma unroll
        for (int x = 0; x < ML_CHUNK / 4; ++x) {
            const int tt = warp + 4 * x;
            const size_t row = (size_t)(start + t0 + tt) * stride + (size_t)h * d;
#pragma unroll
            for (int y = 0; y < ML_PRE_Q; ++y) {
                const int e = lane + 32 * y;
                pq[x][y] = 0.f; pk[x][y] = 0.f;
                if (tt < nt && e < d) {
                    pq[x][y] = proj[row + e];
                    pk[x][y] = proj[row + qk + e];
                }
            }
        }
#pragma unroll
        for (int y = 0; y < ML_PRE_V; ++y) {
            const int i = tid + 128 * y;
            const int tt = i / per_block, cc = blockIdx.x * per_block + (i - tt * per_block);
            pv[y] = 0.f;
            if (tt < nt && cc <= vd) pv[y] = cc < vd ? proj[(size_t)(start + t0 + tt) * stride + 2 * qk + (size_t)h * vd + cc] : 1.f;
        }
        if (tid < nt) {
            const size_t row = (size_t)(start + t0 + tid) * stride;
            pgi = proj[row + i_col0 + h];
            pgf = proj[row + f_col0 + h];
        }
    };
    auto gates = [&](float raw_i, float raw_f, int at) {
        const float gi = cap * tanhf((raw_i + bi) * inv_cap);
        const float x = cap * tanhf((raw_f + bf) * inv_cap);
        sI[at] = gi;
        sF[at] = x < 0.f ? x - log1pf(expf(x)) : -log1pf(expf(-x));          // log sigmoid
    };
    const bool pre = PRE && n_tok > ML_CHUNK;            // (a short portion, a decode step's single token: loaded when its turn comes)
    if (pre) load_chunk(0);
    for (int t0 = 0; t0 < n_tok; t0 += ML_CHUNK) {
        const int nt = min(ML_CHUNK, n_tok - t0);
        __syncthreads();
        if (pre) {
#pragma unroll
            for (int x = 0; x < ML_CHUNK / 4; ++x) {
                const int tt = warp + 4 * x;
#pragma unroll
                for (int y = 0; y < ML_PRE_Q; ++y) {
                    const int e = lane + 32 * y;
                    if (tt < nt && e < d) {
                        const int at = tt * row_floats + (e / NS) * (NS + 4) + (e % NS);
                        sQ[at] = pq[x][y] * q_scale;
                        sK[at] = pk[x][y];
                    }
                }
            }
#pragma unroll
            for (int y = 0; y < ML_PRE_V; ++y) {
                const int i = tid + 128 * y;
                if (i < ML_CHUNK * per_block) sV[i] = pv[y];
            }
            if (tid < nt) gates(pgi, pgf, tid);
        } else {
            if (tid < nt) {
                const size_t row = (size_t)(start + t0 + tid) * stride;
                gates(proj[row + i_col0 + h], proj[row + f_col0 + h], tid);
            }
            for (int tt = warp; tt < nt; tt += 4) {                                   // a warp per token: q and k of the head
                const size_t row = (size_t)(start + t0 + tt) * stride + (size_t)h * d;
                for (int e = lane; e < d; e += 32) {
                    const int at = tt * row_floats + (e / NS) * (NS + 4) + (e % NS);
                    sQ[at] = proj[row + e] * q_scale;
                    sK[at] = proj[row + qk + e];
                }
            }
            for (int i = tid; i < nt * per_block; i += 128) {
                const int tt = i / per_block, cc = blockIdx.x * per_block + (i - tt * per_block);
                sV[i] = cc < vd ? proj[(size_t)(start + t0 + tt) * stride + 2 * qk + (size_t)h * vd + cc] : (cc == vd ? 1.f : 0.f);
            }
        }
        __syncthreads();
        if (pre && t0 + ML_CHUNK < n_tok) load_chunk(t0 + ML_CHUNK);
        if (tid == 0) {                                    // the running maximum is a chain through the chunk: an add and a max a token
            sM[0] = m;
            for (int tt = 0; tt < nt; ++tt) {
                m = fmaxf(sF[tt] + m, sI[tt]);
                sM[tt + 1] = m;
            }
        }
        __syncthreads();
        if (tid < nt) {                                    // ... the exponentials side by side
            const float m_old = sM[tid], m_new = sM[tid + 1];
            sA[tid] = expf(sF[tid] + m_old - m_new);
            sB[tid] = expf(sI[tid] - m_new);
            if (blockIdx.x == 0) top[(size_t)(start + t0 + tid) * heads + h] = m_new;
        }
        __syncthreads();
        // (threads beyond the last column walk along: the shuffles need every lane)
        auto step = [&](int tt) {
            const size_t trow = (size_t)(start + t0 + tt);
            const float4* K4 = reinterpret_cast<const float4*>(sK + tt * row_floats + part * (NS + 4));
            const float4* Q4 = reinterpret_cast<const float4*>(sQ + tt * row_floats + part * (NS + 4));
            const float a = sA[tt];
            const float bu = sB[tt] * sV[tt * per_block + colb];
            float ov4[4] = {0.f, 0.f, 0.f, 0.f};                // four sums side by side: a quarter of the chain
#pragma unroll
            for (int i = 0; i < NS / 4; ++i) {
                const float4 k4 = K4[i], q4 = Q4[i];
                S[4 * i] = fmaf(a, S[4 * i], k4.x * bu);         ov4[0] = fmaf(S[4 * i], q4.x, ov4[0]);
                S[4 * i + 1] = fmaf(a, S[4 * i + 1], k4.y * bu); ov4[1] = fmaf(S[4 * i + 1], q4.y, ov4[1]);
                S[4 * i + 2] = fmaf(a, S[4 * i + 2], k4.z * bu); ov4[2] = fmaf(S[4 * i + 2], q4.z, ov4[2]);
                S[4 * i + 3] = fmaf(a, S[4 * i + 3], k4.w * bu); ov4[3] = fmaf(S[4 * i + 3], q4.w, ov4[3]);
            }
            float ov = (ov4[0] + ov4[1]) + (ov4[2] + ov4[3]);
            for (int o = cpw; o < 32; o <<= 1) ov += __shfl_xor_sync(0xffffffffu, ov, o);
            if (part == 0 && live) raw[trow * heads * width + (size_t)h * width + col] = ov;
        };
        if (nt == ML_CHUNK) {
#pragma unroll 4
            for (int tt = 0; tt < ML_CHUNK; ++tt) step(tt);
        } else {
            for (int tt = 0; tt < nt; ++tt) step(tt);
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NS; ++i)
            if (n0 + i < d) srow[(size_t)(n0 + i) * width + col] = S[i];
    }
    // (m is read by every column block of the head and so must not be written here: the output kernel, which runs after
    // all of them, stores the sequence's last m)
}

// proj rows: [q: heads x d | k: heads x d | v: heads x vd | ...]; the raw gate columns at i_col0 .. and f_col0 ..;
// raw: float [tokens, heads x (vd + 1)], top: float [tokens, heads].
RV_EXPORT int rv_mlstm_scan(const float* proj, int stride, int i_col0, int f_col0, const float* i_bias, const float* f_bias,
                            const int* cu_seqlens, const int* state_slots, float* state, long long state_stride, float* raw, float* top,
                            int n_seqs, int heads, int d, int vd, float cap, cudaStream_t stream) {
    if (n_seqs < 0 || heads <= 0 || d <= 0 || d > 32 * 32 || vd <= 0 || n_seqs > 65535 || heads > 65535 || !(cap > 0.f))
        return RV_ERR_BAD_SIZE;
    if (stride < 2 * heads * d + heads * vd || i_col0 < 0 || f_col0 < 0 || i_col0 + heads > stride || f_col0 + heads > stride ||
        state_stride < (long long)heads * d * (vd + 1) + heads)
        return RV_ERR_BAD_SIZE;
    if (n_seqs == 0) return RV_OK;
    const int ns = d > 64 ? 32 : (d > 32 ? 16 : 8);    // four lanes per column up to a key size of 128
    int parts = 1;
    while (parts * ns < d) parts <<= 1;                // a power of two of at most 32 lanes of one warp
    const int per_block = 128 / parts;
    const size_t smem = sizeof(float) * (2 * (size_t)ML_CHUNK * parts * (ns + 4) + 5 * ML_CHUNK + 4 + (size_t)ML_CHUNK * per_block);
    if (smem > 48 * 1024) return RV_ERR_UNSUPPORTED;
    const bool pre = d <= 32 * ML_PRE_Q && per_block <= 8 * ML_PRE_V;
    auto kernel = ns == 32 ? (pre ? mlstm_scan_kernel<32, true> : mlstm_scan_kernel<32, false>)
                : ns == 16 ? (pre ? mlstm_scan_kernel<16, true> : mlstm_scan_kernel<16, false>)
                           : (pre ? mlstm_scan_kernel<8, true> : mlstm_scan_kernel<8, false>);
    RV_LAUNCH_ST = rv_launch(kernel, dim3((vd + 1 + per_block - 1) / per_block, heads, n_seqs), dim3(128), smem, stream, proj, stride,
                             i_col0, f_col0, i_bias, f_bias, cu_seqlens, state_slots, state, (size_t)state_stride, raw, top, heads, d,
                             vd, parts, cap);
    return rv_launch_status();
}

// One warp per (token, head).
__global__ void __launch_bounds__(128)
mlstm_output_kernel(const float* __restrict__ raw, const float* __restrict__ top, const float* __restrict__ gamma,
                    const float* __restrict__ proj, int stride, int g_col0, void* __restrict__ out, int out_dtype, int n_tokens,
                    int heads, int vd, float eps, float den_eps, const int* __restrict__ token_seq,
                    const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, float* __restrict__ state,
                    size_t state_stride, size_t m_offset) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int lane = threadIdx.x & 31;
    const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (size_t)n_tokens * heads) return;
    const size_t t = item / heads;
    const int h = (int)(item - t * heads);
    const int seq = token_seq[t];
    const int slot = seq >= 0 ? state_slots[seq] : -1;
    if (slot < 0) return;                                  // a padding row: the scan left nothing for it
    if (lane == 0 && (int)t == cu_seqlens[seq + 1] - 1) state[(size_t)slot * state_stride + m_offset + h] = top[item];
    const float* r = raw + item * (vd + 1);
    const float inv = 1.0f / (fmaxf(fabsf(r[vd]), expf(-top[item])) + den_eps);
    float ss = 0.f;
    for (int c = lane; c < vd; c += 32) { const float o = r[c] * inv; ss = fmaf(o, o, ss); }
    ss = rv_warp_sum(ss);
    const float unit = inv / sqrtf(ss / (float)vd + eps);
    const float* z = proj + t * stride + g_col0 + (size_t)h * vd;
    const size_t o0 = t * heads * vd + (size_t)h * vd;
    for (int c = lane; c < vd; c += 32) {
        const float y = r[c] * unit * gamma[h * vd + c] / (1.0f + expf(-z[c]));
        if (out_dtype == RV_DTYPE_F32) ((float*)out)[o0 + c] = y;
        else ((__nv_bfloat16*)out)[o0 + c] = __float2bfloat16_rn(y);
    }
}

RV_EXPORT int rv_mlstm_output(const float* raw, const float* top, const float* gamma, const float* proj, int stride, int g_col0,
                              void* out, int out_dtype, int n_tokens, int heads, int d, int vd, float eps, float den_eps,
                              const int* token_seq, const int* cu_seqlens, const int* state_slots, float* state,
                              long long state_stride, cudaStream_t stream) {
    if (n_tokens < 0 || heads <= 0 || d <= 0 || vd <= 0 || g_col0 < 0 || g_col0 + heads * vd > stride) return RV_ERR_BAD_SIZE;
    if (state_stride < (long long)heads * d * (vd + 1) + heads) return RV_ERR_BAD_SIZE;
    if (out_dtype & ~1) return RV_ERR_BAD_DTYPE;
    if (n_tokens == 0) return RV_OK;
    const size_t items = (size_t)n_tokens * heads;
    RV_LAUNCH_ST = rv_launch(mlstm_output_kernel, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, raw, top, gamma, proj, stride,
                             g_col0, out, out_dtype, n_tokens, heads, vd, eps, den_eps, token_seq, cu_seqlens, state_slots, state,
                             (size_t)state_stride, (size_t)heads * d * (vd + 1));
    return rv_launch_status();
}
