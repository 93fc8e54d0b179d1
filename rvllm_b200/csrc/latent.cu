// Row and small-product kernels of latent attention (one cached low-rank row per token, from which every head's
// keys and values are projected):
//
//   latent_prepare   rows [q: nh x (dq + dr) | c': R | r: dr | gate logits: nh] of a stacked projection.
//                    c = c' / sqrt(mean(c'^2) + eps) * w;  the leading `rot` elements of r and of every head's last dr
//                    query elements are turned in pairs (2i, 2i + 1) - with `halves`: (i, i + rot / 2) - by the angle of (position, i);
//                    [c | r] goes into the token's cache slot, the unrotated query parts into q_plain [T, nh, dq],
//                    the rotated ones into columns R .. R + dr of q_row [T, nh, R + dr] (whose leading R columns
//                    the absorbing product fills afterwards), sigmoid of the gate logits into a float array.
//   head_linear      out[t, h, :] = W[h] x[t, h, :] for W [nh, N, K]: the per-head products that move a head's key
//                    up-projection onto its query and apply its value up-projection to the attended latent.
//                    x and out are given with row and head strides (slices of wider rows).  bfloat16 operands with
//                    aligned rows run on the tensor cores (mma.sync), everything else as FFMA on the CUDA cores;
//                    float accumulation either way, in an order over K that does not depend on the number of rows.
//
// All arithmetic is float; storage is float or bfloat16 per argument.  Any sizes.
#include "common.cuh"

__device__ __forceinline__ float lt_load(const void* p, int dtype, size_t i) {
    return dtype == RV_DTYPE_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void lt_store(void* p, int dtype, size_t i, float v) {
    if (dtype == RV_DTYPE_F32) ((float*)p)[i] = v;
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

// One block per token.
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const void* __restrict__ proj, int in_dtype, int row_stride, const void* __restrict__ c_gamma, int gamma_dtype,
                      const int* __restrict__ positions, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                      int rot, int table_rows, const int* __restrict__ slot_mapping, void* __restrict__ cache,
                      void* __restrict__ q_plain, void* __restrict__ q_row, int out_dtype, float* __restrict__ gate_out,
                      int nh, int dq, int dr, int R, float eps, int write_kv, int halves) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const size_t row = (size_t)t * row_stride;
    const int qw = nh * (dq + dr), D = R + dr;
    const size_t c0 = row + qw;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) { const float v = lt_load(proj, in_dtype, c0 + i); ss = fmaf(v, v, ss); }
    ss = rv_block_sum(ss, scratch);
    const float rc = 1.0f / sqrtf(ss / (float)R + eps);
    int pos = positions[t];
    if (pos < 0) pos = 0;
    if (pos >= table_rows) pos = table_rows - 1;      // the host refuses such positions; never read outside
    const int half = rot >> 1;
    const float* cs = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* sn = sin_t ? sin_t + (size_t)pos * half : nullptr;
    const int slot = write_kv ? slot_mapping[t] : -1;
    if (slot >= 0) {
        const size_t d0 = (size_t)slot * D;                      // one plane, one kv head: a slot is a row
        for (int i = threadIdx.x; i < R; i += blockDim.x)
            lt_store(cache, out_dtype, d0 + i, lt_load(proj, in_dtype, c0 + i) * rc * rv_load_param(c_gamma, gamma_dtype, i));
        // the shared rotated key part: pairs below `rot`, the rest as projected
        for (int i = threadIdx.x; i < dr - half; i += blockDim.x) {
            if (i < half) {
                const int ia = halves ? i : 2 * i, ib = halves ? i + half : 2 * i + 1;         // the two elements of pair i
                const float a = lt_load(proj, in_dtype, c0 + R + ia), b = lt_load(proj, in_dtype, c0 + R + ib);
                const float c = cs[i], s = sn[i];
                lt_store(cache, out_dtype, d0 + R + ia, a * c - b * s);
                lt_store(cache, out_dtype, d0 + R + ib, b * c + a * s);
            } else {
                const int j = i + half;
                lt_store(cache, out_dtype, d0 + R + j, lt_load(proj, in_dtype, c0 + R + j));
            }
        }
    }
    // queries: per head dq plain elements, then dr rotated ones (dr - half items: a pair or a single element)
    const int per_head = dq + dr - half;
    for (int item = threadIdx.x; item < nh * per_head; item += blockDim.x) {
        const int h = item / per_head, i = item - h * per_head;
        const size_t src = row + (size_t)h * (dq + dr);
        if (i < dq) {
            lt_store(q_plain, out_dtype, ((size_t)t * nh + h) * dq + i, lt_load(proj, in_dtype, src + i));
            continue;
        }
        const int k = i - dq;
        const size_t dst = ((size_t)t * nh + h) * D + R;
        if (k < half) {
            const int ia = halves ? k : 2 * k, ib = halves ? k + half : 2 * k + 1;
            const float a = lt_load(proj, in_dtype, src + dq + ia), b = lt_load(proj, in_dtype, src + dq + ib);
            const float c = cs[k], s = sn[k];
            lt_store(q_row, out_dtype, dst + ia, a * c - b * s);
            lt_store(q_row, out_dtype, dst + ib, b * c + a * s);
        } else {
            const int j = k + half;
            lt_store(q_row, out_dtype, dst + j, lt_load(proj, in_dtype, src + dq + j));
        }
    }
    if (gate_out)
        for (int h = threadIdx.x; h < nh; h += blockDim.x) {
            const float g = lt_load(proj, in_dtype, row + qw + D + h);
            gate_out[(size_t)t * nh + h] = 1.0f / (1.0f + expf(-g));
        }
}

RV_EXPORT int rv_latent_prepare(const void* proj, int in_dtype, int row_stride, const void* c_gamma, int gamma_dtype,
                                const int* positions, const float* cos_t, const float* sin_t, int rot, int table_rows,
                                const int* slot_mapping, void* cache, void* q_plain, void* q_row, int out_dtype, float* gate_out,
                                int n_tokens, int nh, int dq, int dr, int R, float eps, int write_kv, int halves, cudaStream_t stream) {
    if (n_tokens < 0 || nh <= 0 || dq <= 0 || dr < 0 || R <= 0 || table_rows <= 0) return RV_ERR_BAD_SIZE;
    if (rot < 0 || rot > dr || (rot & 1)) return RV_ERR_BAD_SIZE;
    if (row_stride < nh * (dq + dr) + R + dr + (gate_out ? nh : 0)) return RV_ERR_BAD_SIZE;
    if ((in_dtype | gamma_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (n_tokens == 0) return RV_OK;
    if (!cos_t || !sin_t) rot = 0;
    RV_LAUNCH_ST = rv_launch(latent_prepare_kernel, dim3(n_tokens), dim3(256), 0, stream, proj, in_dtype, row_stride, c_gamma,
                             gamma_dtype, positions, cos_t, sin_t, rot, table_rows, slot_mapping, cache, q_plain, q_row, out_dtype,
                             gate_out, nh, dq, dr, R, eps, write_kv, halves);
    return rv_launch_status();
}

// ------------------------------------------------------------------ per-head products on the CUDA cores
#define HL_TM 32
#define HL_TN 32
#define HL_TK 32

// grid (n tiles, row tiles, heads); 256 threads, 2 x 2 outputs each
__global__ void __launch_bounds__(256)
head_linear_kernel(const void* __restrict__ x, int x_dtype, long long x_row, long long x_head,
                   const void* __restrict__ w, int w_dtype, void* __restrict__ out, int out_dtype, long long o_row, long long o_head,
                   int T, int N, int K) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ float xs[HL_TK][HL_TM + 1];
    __shared__ float ws[HL_TK][HL_TN + 1];
    const int h = blockIdx.z, m0 = blockIdx.y * HL_TM, n0 = blockIdx.x * HL_TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const size_t xb = (size_t)h * x_head, wb = (size_t)h * N * K, ob = (size_t)h * o_head;
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < K; k0 += HL_TK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = threadIdx.x + r * 256;
            const int rr = idx >> 5, col = idx & 31;
            const int k = k0 + col;
            xs[col][rr] = (m0 + rr < T && k < K) ? lt_load(x, x_dtype, xb + (size_t)(m0 + rr) * x_row + k) : 0.f;
            ws[col][rr] = (n0 + rr < N && k < K) ? lt_load(w, w_dtype, wb + (size_t)(n0 + rr) * K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HL_TK; ++k) {
            const float a0 = xs[k][ty * 2], a1 = xs[k][ty * 2 + 1], b0 = ws[k][tx * 2], b1 = ws[k][tx * 2 + 1];
            acc[0][0] = fmaf(a0, b0, acc[0][0]); acc[0][1] = fmaf(a0, b1, acc[0][1]);
            acc[1][0] = fmaf(a1, b0, acc[1][0]); acc[1][1] = fmaf(a1, b1, acc[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = m0 + ty * 2 + i;
        if (m >= T) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int n = n0 + tx * 2 + j;
            if (n < N) lt_store(out, out_dtype, ob + (size_t)m * o_row + n, acc[i][j]);
        }
    }
}

// ------------------------------------------------------------------ the same on the tensor cores (bfloat16 operands)
// 64 rows x 64 features per CTA of four warps (16 rows each), K in slices of 32 through padded shared-memory tiles,
// mma.sync m16n8k16 with float accumulators; needs K a multiple of 8 and 16-byte aligned rows of x and W.
__device__ __forceinline__ void hl_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void hl_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
#define HM_T 64
#define HM_K 32
#define HM_ROW (HM_K + 8)      // elements of a shared-memory row: 80 bytes, an odd multiple of 16

__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, long long x_row, long long x_head, const __nv_bfloat16* __restrict__ w,
                       void* __restrict__ out, int out_dtype, long long o_row, long long o_head, int T, int N, int K) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ __align__(16) __nv_bfloat16 xs[HM_T][HM_ROW];
    __shared__ __align__(16) __nv_bfloat16 ws[HM_T][HM_ROW];
    const int h = blockIdx.z, m0 = blockIdx.y * HM_T, n0 = blockIdx.x * HM_T;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const __nv_bfloat16* xb = x + (size_t)h * x_head;
    const __nv_bfloat16* wb = w + (size_t)h * N * K;
    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
    for (int k0 = 0; k0 < K; k0 += HM_K) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int idx = threadIdx.x + r * 128;
            const int row = idx >> 2, c = (idx & 3) * 8;
            uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
            if (k0 + c < K) {
                if (m0 + row < T) a = *reinterpret_cast<const uint4*>(xb + (size_t)(m0 + row) * x_row + k0 + c);
                if (n0 + row < N) b = *reinterpret_cast<const uint4*>(wb + (size_t)(n0 + row) * K + k0 + c);
            }
            *reinterpret_cast<uint4*>(&xs[row][c]) = a;
            *reinterpret_cast<uint4*>(&ws[row][c]) = b;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HM_K / 16; ++kk) {
            uint32_t a[4];
            hl_ldmatrix_x4(a, &xs[warp * 16 + (lane & 15)][kk * 16 + (lane >> 4) * 8]);
#pragma unroll
            for (int n2 = 0; n2 < 4; ++n2) {
                uint32_t b[4];
                hl_ldmatrix_x4(b, &ws[n2 * 16 + (lane >> 4) * 8 + (lane & 7)][kk * 16 + ((lane >> 3) & 1) * 8]);
                hl_mma(acc[2 * n2], a, b[0], b[1]);
                hl_mma(acc[2 * n2 + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    const int quad = lane >> 2, tq = lane & 3;
    const size_t ob = (size_t)h * o_head;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = m0 + warp * 16 + quad + 8 * i;
        if (m >= T) continue;
#pragma unroll
        for (int n8 = 0; n8 < 8; ++n8) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int n = n0 + n8 * 8 + tq * 2 + j;
                if (n < N) lt_store(out, out_dtype, ob + (size_t)m * o_row + n, acc[n8][2 * i + j]);
            }
        }
    }
}

RV_EXPORT int rv_head_linear(const void* x, int x_dtype, long long x_row, long long x_head, const void* w, int w_dtype,
                             void* out, int out_dtype, long long o_row, long long o_head, int T, int nh, int N, int K,
                             cudaStream_t stream) {
    if (T < 0 || nh <= 0 || N <= 0 || K <= 0 || nh > 65535) return RV_ERR_BAD_SIZE;
    if ((x_dtype | w_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (T == 0) return RV_OK;
    if (x_dtype == RV_DTYPE_BF16 && w_dtype == RV_DTYPE_BF16 && K % 8 == 0 && x_row % 8 == 0 && x_head % 8 == 0 &&
        reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 && (T + HM_T - 1) / HM_T <= 65535) {
        const dim3 g((N + HM_T - 1) / HM_T, (T + HM_T - 1) / HM_T, nh);
        RV_LAUNCH_ST = rv_launch(head_linear_mma_kernel, dim3(g), dim3(128), 0, stream, (const __nv_bfloat16*)x, x_row, x_head,
                                 (const __nv_bfloat16*)w, out, out_dtype, o_row, o_head, T, N, K);
        return rv_launch_status();
    }
    const dim3 grid((N + HL_TN - 1) / HL_TN, (T + HL_TM - 1) / HL_TM, nh);
    if (grid.y > 65535) return RV_ERR_BAD_SIZE;
    RV_LAUNCH_ST = rv_launch(head_linear_kernel, dim3(grid), dim3(256), 0, stream, x, x_dtype, x_row, x_head, w, w_dtype, out, out_dtype,
                             o_row, o_head, T, N, K);
    return rv_launch_status();
}
