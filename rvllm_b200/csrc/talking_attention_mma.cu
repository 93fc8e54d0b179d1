// Attention whose softmax weights are mixed across the heads, for prompt portions in bfloat16: the tensor-core build of
// talking_attention.cu (same cache layout, same arguments, same arithmetic: scores, softmax, distance bias and the
// mixing in float32; the two matrix products q k^T and p' v take bfloat16 operands and sum in float32).
//
// The weights of all heads of a token must be final before they are mixed, so a CTA owns ALL heads of a few tokens.
// The `rep` = nh / nkv query heads that share a key/value head are stacked with TOK = 16 / rep neighbouring tokens into
// the 16 rows of one mma tile (row = head-in-group * TOK + token), one warp per (token group, key/value head); a CTA has
// TG token groups, i.e. CT = TG * TOK tokens and TG * nkv warps.  Two walks over the visible keys, in tiles of TA_BN:
//   walk 1   s = scale q k^T - bias per warp -> every row's maximum and denominator (kept in registers)
//   walk 2   s again -> p = exp(s - m) / l into shared memory as float [nh][CT][TA_BN];  all threads mix the heads,
//            p'_h = sum_g talk[h, g] p_g, four heads x four keys per thread, and leave p' as bfloat16 in each warp's
//            A-operand tile;  O += p' v per warp.
// Key and value tiles of all key/value heads come by cp.async (16 bytes per copy, rows beyond the last visible key are
// zero-filled); the next key tile is requested as soon as the scores of this one are out, the next value tile after
// this tile's p' v, so both arrive behind the mixing.
#include "common.cuh"
#include <mma.h>

#define TA_BN 32
#define TA_MAX_WARPS 8

__device__ __forceinline__ void tm_ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void tm_ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void tm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void tm_cp16(void* smem, const void* gmem, bool real) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    const int n = real ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void tm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct TmArgs {
    const __nv_bfloat16* q;
    const __nv_bfloat16* cache;
    const int* block_tables;
    const int* cu_seqlens;
    const int* ctx_lens;
    __nv_bfloat16* out;
    const float* r1;
    const float* r2;
    const float* talk;
    int nh, nkv, hd, vd, page_size, max_blocks, chunk, tg;
    float scale;
};

// rows [row0, row0 + TA_BN) of one kind (keys: width hd at offset 0 of a page; values: width vd behind the keys) of all
// key/value heads into `dst` [nkv][TA_BN][width + 8]
__device__ __forceinline__ void tm_fetch(__nv_bfloat16* dst, const TmArgs& a, const int* table, int j0, int j_end, int width, size_t kind_off,
                                         int tid, int nthreads) {
    // two lanes per row (a pair copies one 32-byte sector per step): the row's place in the cache is worked out once
    const int chunks = width / 8, ld = width + 8;
    const int rows = a.nkv * TA_BN;
    const size_t page_elems = (size_t)a.nkv * a.page_size * (a.hd + a.vd);
    const int l2 = tid & 1;
    for (int rowi = tid >> 1; rowi < rows; rowi += nthreads >> 1) {
        const int jj = rowi % TA_BN, g = rowi / TA_BN;
        const int j = j0 + jj;
        const bool real = j <= j_end;
        const __nv_bfloat16* src = a.cache;
        if (real) {
            const int pg = j / a.page_size;
            src += (size_t)table[pg] * page_elems + kind_off + ((size_t)g * a.page_size + (j - pg * a.page_size)) * width + l2 * 8;
        }
        const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst + ((size_t)g * TA_BN + jj) * ld + l2 * 8);
        const int n = real ? 16 : 0, step = real ? 16 : 0;
        for (int c = l2; c < chunks; c += 2) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d + (c - l2) * 16), "l"(src + (c - l2) * (step / 2)), "r"(n) : "memory");
        }
    }
}

template <int HD, int VD>
__global__ void __launch_bounds__(TA_MAX_WARPS * 32)
talking_attention_mma_kernel(const TmArgs a) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ __align__(16) unsigned char tm_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
    const int nh = a.nh, nkv = a.nkv, hd = a.hd, vd = a.vd;
    const int rep = nh / nkv, TOK = 16 / rep, CT = a.tg * TOK;
    const int seq = blockIdx.y;
    const int q_start = a.cu_seqlens[seq];
    const int q_len = a.cu_seqlens[seq + 1] - q_start;
    const int tile0 = (gridDim.x - 1 - blockIdx.x) * CT;           // the long tiles first
    if (tile0 >= q_len) return;
    const int ctx = a.ctx_lens[seq];
    const int n_tok = min(CT, q_len - tile0);
    if (ctx <= 0) {
        for (int i = tid; i < n_tok * nh * vd; i += nthreads) a.out[(size_t)(q_start + tile0) * nh * vd + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int pos0 = ctx - q_len + tile0, pos_last = pos0 + n_tok - 1;
    const int lo_min = a.chunk > 0 ? (pos0 / a.chunk) * a.chunk : 0;
    const int* table = a.block_tables + (size_t)seq * a.max_blocks;

    const int ldk = hd + 8, ldv = vd + 8, ldp = TA_BN + 8;
    const int nh4 = (nh + 3) & ~3;
    __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(tm_smem);                       // [nkv][TA_BN][hd + 8]
    __nv_bfloat16* sV = sK + (size_t)nkv * TA_BN * ldk;                                    // [nkv][TA_BN][vd + 8]
    __nv_bfloat16* sPM = sV + (size_t)nkv * TA_BN * ldv;                                   // [warps][16][TA_BN + 8]
    float* sP = reinterpret_cast<float*>(sPM + (size_t)(nthreads / 32) * 16 * ldp);      // [nh][CT][TA_BN]
    float* sT = sP + (size_t)nh * CT * TA_BN;                                            // talk transposed [g][nh4]

    const int tgi = warp / nkv, g = warp % nkv;
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
    // this lane's two rows of the warp's tile: row r -> head g * rep + r / TOK, token tile0 + tgi * TOK + r % TOK
    int row_head[2], row_tok[2], row_pos[2], row_lo[2];
    float row_r1[2], row_r2[2];
    bool row_ok[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int r = r0 + 8 * x;
        row_head[x] = g * rep + r / TOK;
        row_tok[x] = tgi * TOK + r % TOK;
        row_ok[x] = row_tok[x] < n_tok;
        row_pos[x] = pos0 + row_tok[x];
        row_lo[x] = a.chunk > 0 ? (row_pos[x] / a.chunk) * a.chunk : 0;
        row_r1[x] = a.r1 ? a.r1[row_head[x]] : 0.f;
        row_r2[x] = a.r1 ? a.r2[row_head[x]] : 0.f;
    }
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int rr = x & 1, col = kk * 16 + c0 + (x >> 1) * 8;
            uint32_t v = 0;
            if (row_ok[rr] && col < hd)
                v = *reinterpret_cast<const uint32_t*>(a.q + ((size_t)(q_start + tile0 + row_tok[rr]) * nh + row_head[rr]) * hd + col);
            qf[kk][x] = v;
        }
    }
    if (a.talk)
        for (int i = tid; i < nh * nh4; i += nthreads) {
            const int gg = i / nh4, h = i - gg * nh4;
            sT[i] = h < nh ? a.talk[h * nh + gg] : 0.f;
        }

    const size_t my_k_off = (size_t)g * TA_BN * ldk;
    const __nv_bfloat16* myV = sV + (size_t)g * TA_BN * ldv;
    __nv_bfloat16* myPM = sPM + (size_t)warp * 16 * ldp;
    const size_t v_off = (size_t)nkv * a.page_size * hd;
    const int mi = lane >> 3, mr = lane & 7;

    // the scores of the warp's 16 rows against the tile's keys, bias taken off, hidden keys at -inf
    const int lo_max = a.chunk > 0 ? (pos_last / a.chunk) * a.chunk : 0;
    auto scores = [&](float (&s)[TA_BN / 8][4], int j0, const __nv_bfloat16* myK) {
        const bool open = n_tok == CT && j0 + TA_BN - 1 <= pos0 && j0 >= lo_max;      // every key of the tile is seen by every row
#pragma unroll
        for (int nt = 0; nt < TA_BN / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            if (kk * 16 < hd) {
#pragma unroll
                for (int np = 0; np < TA_BN / 16; ++np) {
                    uint32_t b0, b1, b2, b3;
                    tm_ldmatrix_x4(b0, b1, b2, b3, myK + (size_t)((np * 2 + (mi >> 1)) * 8 + mr) * ldk + kk * 16 + (mi & 1) * 8);
                    tm_mma(s[np * 2], qf[kk], b0, b1);
                    tm_mma(s[np * 2 + 1], qf[kk], b2, b3);
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < TA_BN / 8; ++nt) {
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int rr = x >> 1, j = j0 + nt * 8 + c0 + (x & 1);
                float v = s[nt][x] * a.scale;
                if (a.r1) v -= row_r1[rr] * __logf(1.0f + row_r2[rr] * (float)(row_pos[rr] - j));
                s[nt][x] = (open || (row_ok[rr] && j <= row_pos[rr] && j >= row_lo[rr])) ? v : -INFINITY;
            }
        }
    };

    // ---- walk 1: maxima and denominators
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    // (the value tile's place is free in this walk: where it is large enough the key tiles alternate between the two, and
    // the next tile is on its way while this one is used)
    const bool two = vd >= hd;
    tm_fetch(sK, a, table, lo_min, pos_last, hd, 0, tid, nthreads);
    tm_commit();
    int turn = 0;
    for (int j0 = lo_min; j0 <= pos_last; j0 += TA_BN, turn ^= 1) {
        const bool more = j0 + TA_BN <= pos_last;
        __nv_bfloat16* cur = (two && turn) ? sV : sK;
        if (two) {
            if (more) tm_fetch(turn ? sK : sV, a, table, j0 + TA_BN, pos_last, hd, 0, tid, nthreads);
            tm_commit();
            tm_wait<1>();
        } else {
            tm_wait<0>();
        }
        __syncthreads();
        float s[TA_BN / 8][4];
        scores(s, j0, cur + my_k_off);
        __syncthreads();
        if (!two) {
            if (more) tm_fetch(sK, a, table, j0 + TA_BN, pos_last, hd, 0, tid, nthreads);
            tm_commit();
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            float mx = m[rr];
#pragma unroll
            for (int nt = 0; nt < TA_BN / 8; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * rr], s[nt][2 * rr + 1]));
            if (mx > -INFINITY) {
                float sum = l[rr] * __expf(m[rr] - mx);
#pragma unroll
                for (int nt = 0; nt < TA_BN / 8; ++nt) sum += __expf(s[nt][2 * rr] - mx) + __expf(s[nt][2 * rr + 1] - mx);
                l[rr] = sum;
                m[rr] = mx;
            }
        }
    }
    float linv[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        float M = fmaxf(m[rr], __shfl_xor_sync(0xffffffffu, m[rr], 1));
        M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, 2));
        float L = m[rr] > -INFINITY ? l[rr] * __expf(m[rr] - M) : 0.f;
        L += __shfl_xor_sync(0xffffffffu, L, 1);
        L += __shfl_xor_sync(0xffffffffu, L, 2);
        m[rr] = M;
        linv[rr] = L > 0.f ? 1.0f / L : 0.f;
    }

    // ---- walk 2: weights, mixed, applied
    float o[VD / 8][4];
#pragma unroll
    for (int nt = 0; nt < VD / 8; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    tm_wait<0>();
    __syncthreads();
    tm_fetch(sK, a, table, lo_min, pos_last, hd, 0, tid, nthreads);
    tm_commit();
    tm_fetch(sV, a, table, lo_min, pos_last, vd, v_off, tid, nthreads);
    tm_commit();
    const int mix_items = CT * (TA_BN / 4) * (nh4 / 4);
    for (int j0 = lo_min; j0 <= pos_last; j0 += TA_BN) {
        const bool more = j0 + TA_BN <= pos_last;
        tm_wait<1>();                                   // the key tile (the value tile may still be on its way)
        __syncthreads();
        {
            float s[TA_BN / 8][4];
            scores(s, j0, sK + my_k_off);
#pragma unroll
            for (int nt = 0; nt < TA_BN / 8; ++nt) {
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const float p0 = row_ok[rr] ? __expf(s[nt][2 * rr] - m[rr]) * linv[rr] : 0.f;
                    const float p1 = row_ok[rr] ? __expf(s[nt][2 * rr + 1] - m[rr]) * linv[rr] : 0.f;
                    if (a.talk)
                        *reinterpret_cast<float2*>(sP + ((size_t)row_head[rr] * CT + row_tok[rr]) * TA_BN + nt * 8 + c0) = make_float2(p0, p1);
                    else
                        *reinterpret_cast<__nv_bfloat162*>(myPM + (size_t)(r0 + 8 * rr) * ldp + nt * 8 + c0) = __floats2bfloat162_rn(p0, p1);
                }
            }
        }
        __syncthreads();                                // all scores are out: the key tile is free
        if (more) tm_fetch(sK, a, table, j0 + TA_BN, pos_last, hd, 0, tid, nthreads);
        tm_commit();
        if (a.talk) {
            for (int it = tid; it < mix_items; it += nthreads) {
                const int jq = it % (TA_BN / 4), rest = it / (TA_BN / 4);
                const int tok = rest % CT, hb = rest / CT;
                float acc[4][4];
#pragma unroll
                for (int x = 0; x < 4; ++x) acc[x][0] = acc[x][1] = acc[x][2] = acc[x][3] = 0.f;
                const float* pp = sP + (size_t)tok * TA_BN + jq * 4;
                const float* tt = sT + hb * 4;
                for (int gg = 0; gg < nh; ++gg) {
                    const float4 p = *reinterpret_cast<const float4*>(pp + (size_t)gg * CT * TA_BN);
                    const float4 w = *reinterpret_cast<const float4*>(tt + (size_t)gg * nh4);
                    acc[0][0] = fmaf(w.x, p.x, acc[0][0]); acc[0][1] = fmaf(w.x, p.y, acc[0][1]); acc[0][2] = fmaf(w.x, p.z, acc[0][2]); acc[0][3] = fmaf(w.x, p.w, acc[0][3]);
                    acc[1][0] = fmaf(w.y, p.x, acc[1][0]); acc[1][1] = fmaf(w.y, p.y, acc[1][1]); acc[1][2] = fmaf(w.y, p.z, acc[1][2]); acc[1][3] = fmaf(w.y, p.w, acc[1][3]);
                    acc[2][0] = fmaf(w.z, p.x, acc[2][0]); acc[2][1] = fmaf(w.z, p.y, acc[2][1]); acc[2][2] = fmaf(w.z, p.z, acc[2][2]); acc[2][3] = fmaf(w.z, p.w, acc[2][3]);
                    acc[3][0] = fmaf(w.w, p.x, acc[3][0]); acc[3][1] = fmaf(w.w, p.y, acc[3][1]); acc[3][2] = fmaf(w.w, p.z, acc[3][2]); acc[3][3] = fmaf(w.w, p.w, acc[3][3]);
                }
                const bool tok_ok = tok < n_tok;
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const int h = hb * 4 + x;
                    if (h < nh) {
                        const int w_dst = (tok / TOK) * nkv + h / rep, row = (h % rep) * TOK + tok % TOK;
                        __nv_bfloat162 lo2 = __floats2bfloat162_rn(tok_ok ? acc[x][0] : 0.f, tok_ok ? acc[x][1] : 0.f);
                        __nv_bfloat162 hi2 = __floats2bfloat162_rn(tok_ok ? acc[x][2] : 0.f, tok_ok ? acc[x][3] : 0.f);
                        uint2 pk;
                        pk.x = *reinterpret_cast<uint32_t*>(&lo2);
                        pk.y = *reinterpret_cast<uint32_t*>(&hi2);
                        *reinterpret_cast<uint2*>(sPM + ((size_t)w_dst * 16 + row) * ldp + jq * 4) = pk;
                    }
                }
            }
        }
        if (more) tm_wait<1>(); else tm_wait<0>();      // the value tile (the next key tile may still be on its way)
        __syncthreads();
#pragma unroll
        for (int k2 = 0; k2 < TA_BN / 16; ++k2) {
            uint32_t pa[4];
            tm_ldmatrix_x4(pa[0], pa[1], pa[2], pa[3], myPM + (size_t)(mr + (mi & 1) * 8) * ldp + k2 * 16 + (mi >> 1) * 8);
#pragma unroll
            for (int np = 0; np < VD / 16; ++np) {
                if (np * 16 < vd) {
                    uint32_t b0, b1, b2, b3;
                    tm_ldmatrix_x4_trans(b0, b1, b2, b3, myV + (size_t)(k2 * 16 + (mi & 1) * 8 + mr) * ldv + (np * 2 + (mi >> 1)) * 8);
                    tm_mma(o[np * 2], pa, b0, b1);
                    tm_mma(o[np * 2 + 1], pa, b2, b3);
                }
            }
        }
        __syncthreads();                                // the value tile and the weights are free
        if (more) tm_fetch(sV, a, table, j0 + TA_BN, pos_last, vd, v_off, tid, nthreads);
        tm_commit();
    }
    tm_wait<0>();
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        if (!row_ok[rr]) continue;
        __nv_bfloat16* dst = a.out + ((size_t)(q_start + tile0 + row_tok[rr]) * nh + row_head[rr]) * vd;
#pragma unroll
        for (int nt = 0; nt < VD / 8; ++nt)
            if (nt * 8 < vd) *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8 + c0) = __floats2bfloat162_rn(o[nt][2 * rr], o[nt][2 * rr + 1]);
    }
}

static RvPerDevice g_tm_once[2];

// 1 if the sizes fit this build (the caller falls back to the plain kernel otherwise).
RV_EXPORT int rv_talking_attention_mma_fits(int nh, int nkv, int hd, int vd) {
    if (nh <= 0 || nkv <= 0 || nh % nkv) return 0;
    const int rep = nh / nkv;
    if (rep > 16 || (16 % rep) || nkv > TA_MAX_WARPS) return 0;
    if (hd % 16 || vd % 16 || hd > 128 || vd > 128 || hd < 16 || vd < 16) return 0;
    return 1;
}

RV_EXPORT int rv_talking_attention_mma(const void* q, const void* cache, const int* block_tables, const int* cu_seqlens, const int* ctx_lens,
                                       void* out, int n_seqs, int max_q_len, int nh, int nkv, int hd, int vd, int page_size, int max_blocks,
                                       float scale, const float* r1, const float* r2, const float* talk, int chunk, cudaStream_t stream) {
    if (!rv_talking_attention_mma_fits(nh, nkv, hd, vd)) return RV_ERR_UNSUPPORTED;
    if (n_seqs < 0 || max_q_len < 0 || page_size <= 0 || max_blocks <= 0 || n_seqs > 65535) return RV_ERR_BAD_SIZE;
    if ((r1 == nullptr) != (r2 == nullptr)) return RV_ERR_BAD_SIZE;
    if (((uintptr_t)cache | (uintptr_t)q | (uintptr_t)out) % 16) return RV_ERR_ALIGNMENT;
    if (n_seqs == 0 || max_q_len == 0) return RV_OK;
    const int rep = nh / nkv, TOK = 16 / rep;
    int tg = TA_MAX_WARPS / nkv;
    while (tg > 1 && (tg - 1) * TOK >= max_q_len) --tg;             // no token groups beyond the longest portion
    const int CT = tg * TOK, warps = tg * nkv, nh4 = (nh + 3) & ~3;
    const size_t smem = 2 * ((size_t)nkv * TA_BN * (hd + 8) + (size_t)nkv * TA_BN * (vd + 8) + (size_t)warps * 16 * (TA_BN + 8)) +
                        4 * ((size_t)nh * CT * TA_BN + (size_t)nh * nh4);
    if (smem > 220 * 1024) return RV_ERR_UNSUPPORTED;
    TmArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_tables, cu_seqlens, ctx_lens, (__nv_bfloat16*)out, r1, r2, talk,
             nh, nkv, hd, vd, page_size, max_blocks, chunk, tg, scale};
    const dim3 grid((max_q_len + CT - 1) / CT, n_seqs);
    if (hd <= 64 && vd <= 64) {
        const int st = rv_configure_smem(g_tm_once[0], talking_attention_mma_kernel<64, 64>, 220 * 1024);
        if (st != RV_OK) return st;
        RV_LAUNCH_ST = rv_launch(talking_attention_mma_kernel<64, 64>, grid, dim3(warps * 32), smem, stream, a);
    } else {
        const int st = rv_configure_smem(g_tm_once[1], talking_attention_mma_kernel<128, 128>, 220 * 1024);
        if (st != RV_OK) return st;
        RV_LAUNCH_ST = rv_launch(talking_attention_mma_kernel<128, 128>, grid, dim3(warps * 32), smem, stream, a);
    }
    return rv_launch_status();
}
