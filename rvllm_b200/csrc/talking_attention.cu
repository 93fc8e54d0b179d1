// Attention whose softmax weights are mixed across the heads ("talking heads"), over the paged cache; keys and
// values may differ in width, a distance bias may be taken off the scores, and a query may be limited to the keys
// of its own block of `chunk` positions.
//
//   kv_prepare          rows [q | k | v] of the stacked product -> q in the activations' type, k and v into the
//                       token's cache slot; v is first divided by its root mean square per head (option)
//   talking_attention   s_h(i, j) = scale q_h(i) . k(j) - r1_h ln(1 + r2_h (i - j));  p_h = softmax_j s_h over the
//                       visible keys;  p'_h = sum_g talk[h, g] p_g;  o_h(i) = sum_j p'_h(i, j) v_{kv(h)}(j)
//
// A page of the cache holds the key rows of all its kv heads, [nkv][page_size][hd], and behind them the value rows,
// [nkv][page_size][vd] (with hd = vd this is the layout [2][nkv][page_size][hd] of the other attention kernels).
//
// The weights of ALL heads of a token have to be final before they can be mixed, so a token is one CTA's work:
// a first walk over the visible keys finds every head's maximum and denominator, a second one forms a tile of
// normalised weights for all heads in shared memory, mixes them with `talk`, and adds the tile's values to the
// outputs (which wait in shared memory).  Scores, weights, the bias and the mixing are float32 whatever the cache
// holds.  The q_len tokens a sequence brings to a step are the tail of its ctx_len cached tokens; ctx_len <= 0
// marks a padded row (zeros are written, no table is read).
#include "common.cuh"

#define TA_THREADS 256
#define TA_WARPS 8
#define TA_TILE 32

__device__ __forceinline__ float ta_load(const void* p, int dtype, size_t i) {
    return dtype == RV_DTYPE_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void ta_store(void* p, int dtype, size_t i, float v) {
    if (dtype == RV_DTYPE_F32) ((float*)p)[i] = v;
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

// ------------------------------------------------------------------ q, and k | v into the cache
// One CTA of 128 threads per token.
template <typename TC>
__global__ void __launch_bounds__(128)
kv_prepare_kernel(const void* __restrict__ proj, int p_dtype, int p_stride, const int* __restrict__ slot_mapping,
                  TC* __restrict__ cache, void* __restrict__ q_out, int q_dtype, int nh, int nkv, int hd, int vd, int page_size,
                  float eps, int norm_v, int write_kv) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int t = blockIdx.x;
    const size_t row = (size_t)t * p_stride;
    const int qw = nh * hd, kw = nkv * hd;
    for (int i = threadIdx.x; i < qw; i += blockDim.x) ta_store(q_out, q_dtype, (size_t)t * qw + i, ta_load(proj, p_dtype, row + i));
    if (!write_kv) return;
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    const size_t page_elems = (size_t)nkv * page_size * (hd + vd);
    TC* page = cache + (size_t)(slot / page_size) * page_elems;
    const int off = slot % page_size;
    for (int i = threadIdx.x; i < kw; i += blockDim.x) {
        const int g = i / hd, e = i - g * hd;
        page[((size_t)g * page_size + off) * hd + e] = rv_from_float<TC>(ta_load(proj, p_dtype, row + qw + i));
    }
    TC* vpage = page + (size_t)nkv * page_size * hd;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int g = warp; g < nkv; g += nwarps) {
        const size_t vb = row + qw + kw + (size_t)g * vd;
        float r = 1.0f;
        if (norm_v) {
            float ss = 0.f;
            for (int e = lane; e < vd; e += 32) {
                const float v = ta_load(proj, p_dtype, vb + e);
                ss = fmaf(v, v, ss);
            }
            ss = rv_warp_sum(ss);
            r = 1.0f / sqrtf(ss / (float)vd + eps);
        }
        for (int e = lane; e < vd; e += 32)
            vpage[((size_t)g * page_size + off) * vd + e] = rv_from_float<TC>(ta_load(proj, p_dtype, vb + e) * r);
    }
}

RV_EXPORT int rv_kv_prepare(const void* proj, int p_dtype, int p_stride, const int* slot_mapping, void* cache, int cache_dtype,
                            void* q_out, int q_dtype, int n_tokens, int nh, int nkv, int hd, int vd, int page_size, float eps,
                            int norm_v, int write_kv, cudaStream_t stream) {
    if (n_tokens < 0 || nh <= 0 || nkv <= 0 || hd <= 0 || vd <= 0 || page_size <= 0 || p_stride < nh * hd + nkv * (hd + vd))
        return RV_ERR_BAD_SIZE;
    if ((p_dtype | q_dtype | cache_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (n_tokens == 0) return RV_OK;
    if (cache_dtype == RV_DTYPE_F32)
        RV_LAUNCH_ST = rv_launch(kv_prepare_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, proj, p_dtype, p_stride, slot_mapping,
                                 (float*)cache, q_out, q_dtype, nh, nkv, hd, vd, page_size, eps, norm_v, write_kv);
    else
        RV_LAUNCH_ST = rv_launch(kv_prepare_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, stream, proj, p_dtype, p_stride,
                                 slot_mapping, (__nv_bfloat16*)cache, q_out, q_dtype, nh, nkv, hd, vd, page_size, eps, norm_v, write_kv);
    return rv_launch_status();
}

// ------------------------------------------------------------------ the attention itself
// q . k over hd elements; q waits in shared memory as float.  VEC: 16-byte reads of the key row.
template <typename T, bool VEC>
__device__ __forceinline__ float ta_dot(const T* __restrict__ kp, const float* __restrict__ qs, int hd) {
    float s = 0.f;
    if constexpr (VEC && sizeof(T) == 2) {
        for (int e = 0; e < hd; e += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(kp + e);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float4 qa = *reinterpret_cast<const float4*>(qs + e), qb = *reinterpret_cast<const float4*>(qs + e + 4);
            const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
            const float2 f2 = __bfloat1622float2(h2[2]), f3 = __bfloat1622float2(h2[3]);
            s = fmaf(f0.x, qa.x, s); s = fmaf(f0.y, qa.y, s); s = fmaf(f1.x, qa.z, s); s = fmaf(f1.y, qa.w, s);
            s = fmaf(f2.x, qb.x, s); s = fmaf(f2.y, qb.y, s); s = fmaf(f3.x, qb.z, s); s = fmaf(f3.y, qb.w, s);
        }
    } else if constexpr (VEC) {
        for (int e = 0; e < hd; e += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(kp + e);
            const float4 q4 = *reinterpret_cast<const float4*>(qs + e);
            s = fmaf(k4.x, q4.x, s); s = fmaf(k4.y, q4.y, s); s = fmaf(k4.z, q4.z, s); s = fmaf(k4.w, q4.w, s);
        }
    } else {
        for (int e = 0; e < hd; ++e) s = fmaf(rv_to_float(kp[e]), qs[e], s);
    }
    return s;
}

// The score of head h against the key at position j (one lane's work).
template <typename T, bool VEC>
__device__ __forceinline__ float ta_score(const T* __restrict__ cache, const int* __restrict__ table, size_t page_elems, int page_size,
                                          int hd, int kvh, int j, int pos, const float* __restrict__ qs, float scale, float r1, float r2,
                                          bool biased) {
    const int page = table[j / page_size];
    const T* kp = cache + (size_t)page * page_elems + ((size_t)kvh * page_size + (j % page_size)) * hd;
    float s = ta_dot<T, VEC>(kp, qs, hd) * scale;
    if (biased) s -= r1 * log1pf(r2 * (float)(pos - j));
    return s;
}

// Shared memory (floats): q [nh * hd] | O [nh * vd] | P [nh][TA_TILE] | P' [nh][TA_TILE] | talk [nh * nh] | m [nh] | 1/l [nh],
// and TA_TILE 64-bit offsets of the tile's value rows.
template <typename T, bool VEC>
__global__ void __launch_bounds__(TA_THREADS)
talking_attention_kernel(const T* __restrict__ q, const T* __restrict__ cache, const int* __restrict__ block_tables,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ ctx_lens, const int* __restrict__ token_seq,
                         T* __restrict__ out, int nh, int nkv, int hd, int vd, int page_size, int max_blocks, float scale,
                         const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ talk, int chunk) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ __align__(16) unsigned char ta_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t = blockIdx.x;
    const int seq = token_seq[t];
    const int ctx = seq >= 0 ? ctx_lens[seq] : 0;
    T* o = out + (size_t)t * nh * vd;
    if (ctx <= 0) {
        for (int i = tid; i < nh * vd; i += TA_THREADS) o[i] = rv_from_float<T>(0.f);
        return;
    }
    size_t* vrow = reinterpret_cast<size_t*>(ta_smem);
    float* qs = reinterpret_cast<float*>(ta_smem + TA_TILE * sizeof(size_t));
    float* Os = qs + (size_t)nh * hd;
    float* P = Os + (size_t)nh * vd;
    float* PM = talk ? P + nh * TA_TILE : P;
    float* talk_s = P + 2 * nh * TA_TILE;
    float* ms = talk_s + nh * nh;
    float* linv = ms + nh;

    const int q_start = cu_seqlens[seq];
    const int q_len = cu_seqlens[seq + 1] - q_start;
    const int pos = ctx - q_len + (t - q_start);
    const int lo = chunk > 0 ? (pos / chunk) * chunk : 0;
    const int rep = nh / nkv;
    const int* table = block_tables + (size_t)seq * max_blocks;
    const size_t page_elems = (size_t)nkv * page_size * (hd + vd);
    const size_t v_off = (size_t)nkv * page_size * hd;
    const bool biased = r1 != nullptr;

    for (int i = tid; i < nh * hd; i += TA_THREADS) qs[i] = rv_to_float(q[(size_t)t * nh * hd + i]);
    for (int i = tid; i < nh * vd; i += TA_THREADS) Os[i] = 0.f;
    if (talk)
        for (int i = tid; i < nh * nh; i += TA_THREADS) talk_s[i] = talk[i];
    __syncthreads();

    // every head's maximum and denominator: a warp per head, a lane per key, joined at the end
    for (int h = warp; h < nh; h += TA_WARPS) {
        const float a1 = biased ? r1[h] : 0.f, a2 = biased ? r2[h] : 0.f;
        float m = -INFINITY, l = 0.f;
        for (int j = lo + lane; j <= pos; j += 32) {
            const float s = ta_score<T, VEC>(cache, table, page_elems, page_size, hd, h / rep, j, pos, qs + (size_t)h * hd, scale, a1, a2, biased);
            const float m_new = fmaxf(m, s);
            l = l * expf(m - m_new) + expf(s - m_new);
            m = m_new;
        }
        const float M = rv_warp_max(m);
        l = rv_warp_sum(m == -INFINITY ? 0.f : l * expf(m - M));
        if (lane == 0) {
            ms[h] = M;
            linv[h] = 1.0f / l;
        }
    }
    __syncthreads();

    for (int j0 = lo; j0 <= pos; j0 += TA_TILE) {
        const int nk = min(TA_TILE, pos - j0 + 1);
        // the tile's normalised weights, head by head
        for (int h = warp; h < nh; h += TA_WARPS) {
            float p = 0.f;
            if (lane < nk) {
                const float a1 = biased ? r1[h] : 0.f, a2 = biased ? r2[h] : 0.f;
                const float s = ta_score<T, VEC>(cache, table, page_elems, page_size, hd, h / rep, j0 + lane, pos, qs + (size_t)h * hd, scale,
                                                 a1, a2, biased);
                p = expf(s - ms[h]) * linv[h];
            }
            P[h * TA_TILE + lane] = p;
        }
        if (tid < nk) {
            const int j = j0 + tid;
            vrow[tid] = (size_t)table[j / page_size] * page_elems + v_off + (size_t)(j % page_size) * vd;
        }
        __syncthreads();
        if (talk) {
            for (int i = tid; i < nh * TA_TILE; i += TA_THREADS) {
                const int h = i / TA_TILE, jj = i - h * TA_TILE;
                float a = 0.f;
                for (int g = 0; g < nh; ++g) a = fmaf(talk_s[h * nh + g], P[g * TA_TILE + jj], a);
                PM[i] = a;
            }
            __syncthreads();
        }
        // the tile's values, weighted: a thread per output element
        for (int i = tid; i < nh * vd; i += TA_THREADS) {
            const int h = i / vd, e = i - h * vd;
            const size_t head_off = (size_t)(h / rep) * page_size * vd + e;
            const float* pw = PM + h * TA_TILE;
            float acc = Os[i];
            for (int jj = 0; jj < nk; ++jj) acc = fmaf(pw[jj], rv_to_float(cache[vrow[jj] + head_off]), acc);
            Os[i] = acc;
        }
        __syncthreads();
    }
    for (int i = tid; i < nh * vd; i += TA_THREADS) o[i] = rv_from_float<T>(Os[i]);
}

static RvPerDevice g_ta_once[4];

template <typename T, bool VEC>
static int ta_launch(int which, const void* q, const void* cache, const int* block_tables, const int* cu_seqlens, const int* ctx_lens,
                     const int* token_seq, void* out, int n_tokens, int nh, int nkv, int hd, int vd, int page_size, int max_blocks,
                     float scale, const float* r1, const float* r2, const float* talk, int chunk, size_t smem, cudaStream_t stream) {
    const int st = rv_configure_smem(g_ta_once[which], talking_attention_kernel<T, VEC>, 200 * 1024);
    if (st != RV_OK) return st;
    RV_LAUNCH_ST = rv_launch(talking_attention_kernel<T, VEC>, dim3(n_tokens), dim3(TA_THREADS), smem, stream, (const T*)q, (const T*)cache,
                             block_tables, cu_seqlens, ctx_lens, token_seq, (T*)out, nh, nkv, hd, vd, page_size, max_blocks, scale, r1, r2,
                             talk, chunk);
    return rv_launch_status();
}

// q, cache and out share one type (`dtype`); r1 / r2 (both or neither), talk and chunk (<= 0: none) are options.
RV_EXPORT int rv_talking_attention(const void* q, const void* cache, const int* block_tables, const int* cu_seqlens,
                                   const int* ctx_lens, const int* token_seq, void* out, int n_tokens, int nh, int nkv, int hd, int vd,
                                   int page_size, int max_blocks, float scale, const float* r1, const float* r2, const float* talk,
                                   int chunk, int dtype, cudaStream_t stream) {
    if (n_tokens < 0 || nh <= 0 || nkv <= 0 || nh % nkv || hd <= 0 || vd <= 0 || page_size <= 0 || max_blocks <= 0) return RV_ERR_BAD_SIZE;
    if ((r1 == nullptr) != (r2 == nullptr)) return RV_ERR_BAD_SIZE;
    if (dtype & ~1) return RV_ERR_BAD_DTYPE;
    const size_t smem = TA_TILE * sizeof(size_t) +
                        sizeof(float) * ((size_t)nh * hd + (size_t)nh * vd + 2 * (size_t)nh * TA_TILE + (size_t)nh * nh + 2 * (size_t)nh);
    if (smem > 200 * 1024) return RV_ERR_UNSUPPORTED;
    if (n_tokens == 0) return RV_OK;
    const int el = dtype == RV_DTYPE_F32 ? 4 : 2;
    const bool vec = (hd * el) % 16 == 0 && (vd * el) % 16 == 0 && ((uintptr_t)cache % 16) == 0;
#define TA_GO(W, T, V) return ta_launch<T, V>(W, q, cache, block_tables, cu_seqlens, ctx_lens, token_seq, out, n_tokens, nh, nkv, hd, vd, \
                                              page_size, max_blocks, scale, r1, r2, talk, chunk, smem, stream)
    if (dtype == RV_DTYPE_F32) {
        if (vec) TA_GO(0, float, true);
        TA_GO(1, float, false);
    }
    if (vec) TA_GO(2, __nv_bfloat16, true);
    TA_GO(3, __nv_bfloat16, false);
#undef TA_GO
}

// ------------------------------------------------------------------ few tokens, many keys: the keys split over CTAs
// A step of single tokens gives the kernel above one CTA per sequence, which walks all its keys alone.  Here a
// token's visible keys are cut into `nsplit` ranges of `span` keys, and three launches do the work:
//   scores   CTA (token, range): every head's scores of the range into `S` [tokens][nh][nsplit * span] (float), and the
//            range's maximum and sum of exponentials per head into `stats` [tokens][nsplit][nh][2]
//   apply    CTA (token, range): joins the token's statistics, turns the range's scores into normalised weights, mixes
//            the heads and sums the range's values into `part` [tokens][nsplit][nh * vd] (float)
//   join     CTA per token: adds the parts in the order of the ranges
// The weights are linear in the values once every head's maximum and denominator are known, so the parts only add.
struct TaWhere {
    int ctx, pos, lo, k0, k1, nvalid;
    const int* table;
};

__device__ __forceinline__ TaWhere ta_where(const int* block_tables, const int* cu_seqlens, const int* ctx_lens, const int* token_seq, int t,
                                            int sp, int span, int chunk, int max_blocks) {
    TaWhere w;
    const int seq = token_seq[t];
    w.ctx = seq >= 0 ? ctx_lens[seq] : 0;
    w.pos = w.lo = w.k0 = w.k1 = w.nvalid = 0;
    w.table = nullptr;
    if (w.ctx <= 0) return w;
    const int q_start = cu_seqlens[seq];
    const int q_len = cu_seqlens[seq + 1] - q_start;
    w.pos = w.ctx - q_len + (t - q_start);
    w.lo = chunk > 0 ? (w.pos / chunk) * chunk : 0;
    w.k0 = w.lo + sp * span;
    w.k1 = min(w.k0 + span, w.pos + 1);
    w.nvalid = (w.pos - w.lo) / span + 1;
    w.table = block_tables + (size_t)seq * max_blocks;
    return w;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(TA_THREADS)
ta_split_scores_kernel(const T* __restrict__ q, const T* __restrict__ cache, const int* __restrict__ block_tables,
                       const int* __restrict__ cu_seqlens, const int* __restrict__ ctx_lens, const int* __restrict__ token_seq,
                       float* __restrict__ S, float* __restrict__ stats, int nh, int nkv, int hd, int vd, int page_size, int max_blocks,
                       float scale, const float* __restrict__ r1, const float* __restrict__ r2, int chunk, int span, int nsplit) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ __align__(16) unsigned char ta_smem[];
    float* qs = reinterpret_cast<float*>(ta_smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t = blockIdx.x, sp = blockIdx.y;
    const TaWhere w = ta_where(block_tables, cu_seqlens, ctx_lens, token_seq, t, sp, span, chunk, max_blocks);
    if (w.ctx <= 0 || w.k0 > w.pos) return;
    for (int i = tid; i < nh * hd; i += TA_THREADS) qs[i] = rv_to_float(q[(size_t)t * nh * hd + i]);
    const int rep = nh / nkv;
    const size_t page_elems = (size_t)nkv * page_size * (hd + vd);
    {   // the range's value rows are asked into L2 now: the next launch reads them while this one still works on the keys
        const int lines = (int)((vd * sizeof(T) + 127) / 128);
        const int total = (w.k1 - w.k0) * nkv * lines;
        for (int i = tid; i < total; i += TA_THREADS) {
            const int ln = i % lines, rest = i / lines;
            const int g = rest % nkv, j = w.k0 + rest / nkv;
            const T* vp = cache + (size_t)w.table[j / page_size] * page_elems + (size_t)nkv * page_size * hd +
                          ((size_t)g * page_size + (j % page_size)) * vd;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(vp) + ln * 128));
        }
    }
    __syncthreads();
    const bool biased = r1 != nullptr;
    const size_t stride = (size_t)nsplit * span;
    if constexpr (VEC && sizeof(T) == 2) {
        if (rep % 4 == 0) {
            // a warp per block of four heads of one key/value head, a lane per key: the key's row is read once, 16 bytes at a time
            for (int hb = warp; hb < nh / 4; hb += TA_WARPS) {
                const int h0 = hb * 4, kvh = h0 / rep;
                float m[4], l[4], a1[4], a2[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    m[x] = -INFINITY; l[x] = 0.f;
                    a1[x] = biased ? r1[h0 + x] : 0.f; a2[x] = biased ? r2[h0 + x] : 0.f;
                }
                for (int j = w.k0 + lane; j < w.k1; j += 32) {
                    const T* kp = cache + (size_t)w.table[j / page_size] * page_elems + ((size_t)kvh * page_size + (j % page_size)) * hd;
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    for (int e0 = 0; e0 < hd; e0 += 64) {               // eight 16-byte pieces of the row on their way at a time
                        uint4 raw4[8];
#pragma unroll
                        for (int y = 0; y < 8; ++y) raw4[y] = e0 + 8 * y < hd ? *reinterpret_cast<const uint4*>(kp + e0 + 8 * y) : make_uint4(0, 0, 0, 0);
#pragma unroll
                        for (int y = 0; y < 8; ++y) {
                            const int e = e0 + 8 * y;
                            if (e < hd) {
                                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw4[y]);
                                const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
                                const float2 f2 = __bfloat1622float2(h2[2]), f3 = __bfloat1622float2(h2[3]);
#pragma unroll
                                for (int x = 0; x < 4; ++x) {
                                    const float* qx = qs + (size_t)(h0 + x) * hd + e;
                                    const float4 qa = *reinterpret_cast<const float4*>(qx), qb = *reinterpret_cast<const float4*>(qx + 4);
                                    float sacc = acc[x];
                                    sacc = fmaf(f0.x, qa.x, sacc); sacc = fmaf(f0.y, qa.y, sacc); sacc = fmaf(f1.x, qa.z, sacc); sacc = fmaf(f1.y, qa.w, sacc);
                                    sacc = fmaf(f2.x, qb.x, sacc); sacc = fmaf(f2.y, qb.y, sacc); sacc = fmaf(f3.x, qb.z, sacc); sacc = fmaf(f3.y, qb.w, sacc);
                                    acc[x] = sacc;
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        float sc = acc[x] * scale;
                        if (biased) sc -= a1[x] * log1pf(a2[x] * (float)(w.pos - j));
                        S[((size_t)t * nh + h0 + x) * stride + (j - w.lo)] = sc;
                        const float m_new = fmaxf(m[x], sc);
                        l[x] = l[x] * expf(m[x] - m_new) + expf(sc - m_new);
                        m[x] = m_new;
                    }
                }
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float M = rv_warp_max(m[x]);
                    const float L = rv_warp_sum(m[x] == -INFINITY ? 0.f : l[x] * expf(m[x] - M));
                    if (lane == 0) {
                        float* st = stats + (((size_t)t * nsplit + sp) * nh + h0 + x) * 2;
                        st[0] = M;
                        st[1] = L;
                    }
                }
            }
            return;
        }
    }
    for (int h = warp; h < nh; h += TA_WARPS) {
        const float a1 = biased ? r1[h] : 0.f, a2 = biased ? r2[h] : 0.f;
        float* row = S + ((size_t)t * nh + h) * stride;
        float m = -INFINITY, l = 0.f;
        for (int j = w.k0 + lane; j < w.k1; j += 32) {
            const float s = ta_score<T, VEC>(cache, w.table, page_elems, page_size, hd, h / rep, j, w.pos, qs + (size_t)h * hd, scale, a1, a2, biased);
            row[j - w.lo] = s;
            const float m_new = fmaxf(m, s);
            l = l * expf(m - m_new) + expf(s - m_new);
            m = m_new;
        }
        const float M = rv_warp_max(m);
        l = rv_warp_sum(m == -INFINITY ? 0.f : l * expf(m - M));
        if (lane == 0) {
            float* st = stats + (((size_t)t * nsplit + sp) * nh + h) * 2;
            st[0] = M;
            st[1] = l;
        }
    }
}

// Shared memory: TA_TILE 64-bit offsets | O [nh * vd] | P [nh][TA_TILE] | P' [nh][TA_TILE] | talk [nh * nh] | m [nh] | 1/l [nh].
template <typename T, bool VEC>
__global__ void __launch_bounds__(TA_THREADS)
ta_split_apply_kernel(const T* __restrict__ cache, const int* __restrict__ block_tables, const int* __restrict__ cu_seqlens,
                      const int* __restrict__ ctx_lens, const int* __restrict__ token_seq, const float* __restrict__ S,
                      const float* __restrict__ stats, const float* __restrict__ talk, float* __restrict__ part, int nh, int nkv, int hd,
                      int vd, int page_size, int max_blocks, int chunk, int span, int nsplit) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ __align__(16) unsigned char ta_smem[];
    const int tid = threadIdx.x;
    const int t = blockIdx.x, sp = blockIdx.y;
    const TaWhere w = ta_where(block_tables, cu_seqlens, ctx_lens, token_seq, t, sp, span, chunk, max_blocks);
    if (w.ctx <= 0 || w.k0 > w.pos) return;
    size_t* vrow = reinterpret_cast<size_t*>(ta_smem);
    float* Os = reinterpret_cast<float*>(ta_smem + TA_TILE * sizeof(size_t));
    float* P = Os + (size_t)nh * vd;
    float* PM = talk ? P + nh * TA_TILE : P;
    float* talk_s = P + 2 * nh * TA_TILE;
    float* ms = talk_s + nh * nh;
    float* linv = ms + nh;
    const int rep = nh / nkv;
    const size_t page_elems = (size_t)nkv * page_size * (hd + vd);
    const size_t v_off = (size_t)nkv * page_size * hd;
    const size_t stride = (size_t)nsplit * span;

    for (int hb = 0; hb < nh; hb += TA_THREADS / 8) {        // eight lanes per head, each a share of the ranges
        const int h = hb + tid / 8, sub = tid & 7;
        float M = -INFINITY, L = 0.f;
        if (h < nh) {
            const float* st = stats + ((size_t)t * nsplit * nh + h) * 2;
            for (int s = sub; s < w.nvalid; s += 8) {
                const float2 ml = *reinterpret_cast<const float2*>(st + (size_t)s * nh * 2);
                const float m_new = fmaxf(M, ml.x);
                L = L * expf(M - m_new) + ml.y * expf(ml.x - m_new);
                M = m_new;
            }
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            const float M2 = __shfl_xor_sync(0xffffffffu, M, o), L2 = __shfl_xor_sync(0xffffffffu, L, o);
            const float m_new = fmaxf(M, M2);
            L = (M == -INFINITY ? 0.f : L * expf(M - m_new)) + (M2 == -INFINITY ? 0.f : L2 * expf(M2 - m_new));
            M = m_new;
        }
        if (h < nh && sub == 0) {
            ms[h] = M;
            linv[h] = 1.0f / L;
        }
    }
    for (int i = tid; i < nh * vd; i += TA_THREADS) Os[i] = 0.f;
    if (talk)
        for (int i = tid; i < nh * nh; i += TA_THREADS) talk_s[i] = talk[i];
    __syncthreads();

    constexpr int EV = VEC ? 16 / (int)sizeof(T) : 1;      // value elements per thread and key
    const int vblocks = vd / EV;
    const bool quads = VEC && sizeof(T) == 2 && rep % 4 == 0;
    for (int j0 = w.k0; j0 < w.k1; j0 += TA_TILE) {
        const int nk = min(TA_TILE, w.k1 - j0);
        for (int i = tid; i < nh * TA_TILE; i += TA_THREADS) {
            const int h = i / TA_TILE, jj = i - h * TA_TILE;
            P[i] = jj < nk ? expf(S[((size_t)t * nh + h) * stride + (j0 + jj - w.lo)] - ms[h]) * linv[h] : 0.f;
        }
        if (tid < nk) {
            const int j = j0 + tid;
            vrow[tid] = (size_t)w.table[j / page_size] * page_elems + v_off + (size_t)(j % page_size) * vd;
        }
        __syncthreads();
        if (talk) {
            for (int i = tid; i < nh * TA_TILE; i += TA_THREADS) {
                const int h = i / TA_TILE, jj = i - h * TA_TILE;
                float a = 0.f;
                for (int g = 0; g < nh; ++g) a = fmaf(talk_s[h * nh + g], P[g * TA_TILE + jj], a);
                PM[i] = a;
            }
            __syncthreads();
        }
        if (quads) {
            // four heads of one key/value head and four value elements per thread: every value of the tile is read once
            const int v4 = vd / 4;
            for (int i = tid; i < (nh / 4) * v4; i += TA_THREADS) {
                const int hb = i / v4, e = (i - hb * v4) * 4, h0 = hb * 4;
                const size_t head_off = (size_t)(h0 / rep) * page_size * vd + e;
                float acc[4][4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float4 o4 = *reinterpret_cast<const float4*>(Os + (h0 + x) * vd + e);
                    acc[x][0] = o4.x; acc[x][1] = o4.y; acc[x][2] = o4.z; acc[x][3] = o4.w;
                }
                for (int j8 = 0; j8 < nk; j8 += 8) {                // eight value pieces on their way at a time
                    uint2 raw8[8];
#pragma unroll
                    for (int y = 0; y < 8; ++y)
                        raw8[y] = j8 + y < nk ? *reinterpret_cast<const uint2*>(cache + vrow[j8 + y] + head_off) : make_uint2(0, 0);
#pragma unroll
                    for (int y = 0; y < 8; ++y) {
                        const int jj = j8 + y;                          // (beyond nk: the weights of the tile's tail are zero)
                        const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw8[y].x));
                        const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw8[y].y));
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
                            const float p = PM[(h0 + x) * TA_TILE + jj];
                            acc[x][0] = fmaf(p, fa.x, acc[x][0]); acc[x][1] = fmaf(p, fa.y, acc[x][1]);
                            acc[x][2] = fmaf(p, fb.x, acc[x][2]); acc[x][3] = fmaf(p, fb.y, acc[x][3]);
                        }
                    }
                }
#pragma unroll
                for (int x = 0; x < 4; ++x)
                    *reinterpret_cast<float4*>(Os + (h0 + x) * vd + e) = make_float4(acc[x][0], acc[x][1], acc[x][2], acc[x][3]);
            }
            __syncthreads();
            continue;
        }
        for (int i = tid; i < nh * vblocks; i += TA_THREADS) {
            const int h = i / vblocks, e = (i - h * vblocks) * EV;
            const size_t head_off = (size_t)(h / rep) * page_size * vd + e;
            const float* pw = PM + h * TA_TILE;
            float acc[EV];
#pragma unroll
            for (int x = 0; x < EV; ++x) acc[x] = Os[h * vd + e + x];
            for (int jj = 0; jj < nk; ++jj) {
                const float p = pw[jj];
                const T* vp = cache + vrow[jj] + head_off;
                if constexpr (VEC && sizeof(T) == 2) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(vp);
                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const float2 f = __bfloat1622float2(h2[x]);
                        acc[2 * x] = fmaf(p, f.x, acc[2 * x]);
                        acc[2 * x + 1] = fmaf(p, f.y, acc[2 * x + 1]);
                    }
                } else if constexpr (VEC) {
                    const float4 f = *reinterpret_cast<const float4*>(vp);
                    acc[0] = fmaf(p, f.x, acc[0]); acc[1] = fmaf(p, f.y, acc[1]);
                    acc[2] = fmaf(p, f.z, acc[2]); acc[3] = fmaf(p, f.w, acc[3]);
                } else {
                    acc[0] = fmaf(p, rv_to_float(vp[0]), acc[0]);
                }
            }
#pragma unroll
            for (int x = 0; x < EV; ++x) Os[h * vd + e + x] = acc[x];
        }
        __syncthreads();
    }
    float* o = part + ((size_t)t * nsplit + sp) * nh * vd;
    for (int i = tid; i < nh * vd; i += TA_THREADS) o[i] = Os[i];
}

template <typename T>
__global__ void __launch_bounds__(TA_THREADS)
ta_split_join_kernel(const float* __restrict__ part, const int* __restrict__ cu_seqlens, const int* __restrict__ ctx_lens,
                     const int* __restrict__ token_seq, T* __restrict__ out, int width, int chunk, int span, int nsplit) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int t = blockIdx.x;
    const TaWhere w = ta_where(nullptr, cu_seqlens, ctx_lens, token_seq, t, 0, span, chunk, 0);
    for (int i = blockIdx.y * TA_THREADS + threadIdx.x; i < width; i += gridDim.y * TA_THREADS) {
        float a = 0.f;
        for (int s = 0; s < w.nvalid; ++s) a += part[((size_t)t * nsplit + s) * width + i];
        out[(size_t)t * width + i] = rv_from_float<T>(a);
    }
}

static RvPerDevice g_ta_split_once[4];

template <typename T, bool VEC>
static int ta_split_launch(int which, const void* q, const void* cache, const int* block_tables, const int* cu_seqlens, const int* ctx_lens,
                           const int* token_seq, void* out, float* S, float* stats, float* part, int n_tokens, int nh, int nkv, int hd,
                           int vd, int page_size, int max_blocks, float scale, const float* r1, const float* r2, const float* talk, int chunk,
                           int span, int nsplit, size_t smem, cudaStream_t stream) {
    const int st = rv_configure_smem(g_ta_split_once[which], ta_split_apply_kernel<T, VEC>, 200 * 1024);
    if (st != RV_OK) return st;
    RV_LAUNCH_ST = rv_launch(ta_split_scores_kernel<T, VEC>, dim3(n_tokens, nsplit), dim3(TA_THREADS), sizeof(float) * (size_t)nh * hd, stream,
                             (const T*)q, (const T*)cache, block_tables, cu_seqlens, ctx_lens, token_seq, S, stats, nh, nkv, hd, vd, page_size,
                             max_blocks, scale, r1, r2, chunk, span, nsplit);
    if (rv_launch_status() != RV_OK) return rv_launch_status();
    RV_LAUNCH_ST = rv_launch(ta_split_apply_kernel<T, VEC>, dim3(n_tokens, nsplit), dim3(TA_THREADS), smem, stream, (const T*)cache,
                             block_tables, cu_seqlens, ctx_lens, token_seq, (const float*)S, (const float*)stats, talk, part, nh, nkv, hd, vd,
                             page_size, max_blocks, chunk, span, nsplit);
    if (rv_launch_status() != RV_OK) return rv_launch_status();
    RV_LAUNCH_ST = rv_launch(ta_split_join_kernel<T>, dim3(n_tokens, (nh * vd + TA_THREADS - 1) / TA_THREADS), dim3(TA_THREADS), 0, stream, (const float*)part, cu_seqlens, ctx_lens,
                             token_seq, (T*)out, nh * vd, chunk, span, nsplit);
    return rv_launch_status();
}

// Floats of scratch that rv_talking_attention_split needs behind `scratch`: S, then stats, then the parts.
RV_EXPORT long long rv_talking_attention_split_floats(int n_tokens, int nh, int vd, int span, int nsplit) {
    return (long long)n_tokens * nh * nsplit * span + (long long)n_tokens * nsplit * nh * 2 + (long long)n_tokens * nsplit * nh * vd;
}

// As rv_talking_attention, the visible keys of every token cut into `nsplit` ranges of `span` keys (nsplit * span covers
// the longest visible run of the step); `scratch` holds rv_talking_attention_split_floats floats.
RV_EXPORT int rv_talking_attention_split(const void* q, const void* cache, const int* block_tables, const int* cu_seqlens,
                                         const int* ctx_lens, const int* token_seq, void* out, float* scratch, int n_tokens, int nh, int nkv,
                                         int hd, int vd, int page_size, int max_blocks, float scale, const float* r1, const float* r2,
                                         const float* talk, int chunk, int span, int nsplit, int dtype, cudaStream_t stream) {
    if (n_tokens < 0 || nh <= 0 || nkv <= 0 || nh % nkv || hd <= 0 || vd <= 0 || page_size <= 0 || max_blocks <= 0 || span <= 0 || nsplit <= 0)
        return RV_ERR_BAD_SIZE;
    if ((r1 == nullptr) != (r2 == nullptr)) return RV_ERR_BAD_SIZE;
    if (dtype & ~1) return RV_ERR_BAD_DTYPE;
    const size_t smem = TA_TILE * sizeof(size_t) +
                        sizeof(float) * ((size_t)nh * vd + 2 * (size_t)nh * TA_TILE + (size_t)nh * nh + 2 * (size_t)nh);
    if (smem > 200 * 1024 || sizeof(float) * (size_t)nh * hd > 48 * 1024) return RV_ERR_UNSUPPORTED;
    if (n_tokens == 0) return RV_OK;
    float* S = scratch;
    float* stats = S + (size_t)n_tokens * nh * nsplit * span;
    float* part = stats + (size_t)n_tokens * nsplit * nh * 2;
    const int el = dtype == RV_DTYPE_F32 ? 4 : 2;
    const bool vec = (hd * el) % 16 == 0 && (vd * el) % 16 == 0 && ((uintptr_t)cache % 16) == 0;
#define TA_GO(W, T, V) return ta_split_launch<T, V>(W, q, cache, block_tables, cu_seqlens, ctx_lens, token_seq, out, S, stats, part, n_tokens, \
                                                    nh, nkv, hd, vd, page_size, max_blocks, scale, r1, r2, talk, chunk, span, nsplit, smem, stream)
    if (dtype == RV_DTYPE_F32) {
        if (vec) TA_GO(0, float, true);
        TA_GO(1, float, false);
    }
    if (vec) TA_GO(2, __nv_bfloat16, true);
    TA_GO(3, __nv_bfloat16, false);
#undef TA_GO
}
