// What stands between the stacked q/k/v product and the attention kernels for mixers whose queries and keys are
// rotated and then made unit-RMS vectors per head:
//
//   qk_unit_prepare   rows [q: nh x d | k: nkv x d | v: nkv x vd | gate logits: nh] of a float32 projection (k and v only
//                     where the layer has them).  The leading `rot` elements of every head of q and k turn by the angle
//                     of (position, pair): pairs (2i, 2i + 1), or (i, i + rot / 2) with `halves`; then the head is divided
//                     by sqrt(mean(x^2) + eps) over its d elements (no weight).  q goes to q_out [T, nh, P], k and v
//                     into the token's cache slot (planes 0 and 1 of [pages, 2, nkv, page, P]); P >= max(d, vd), and
//                     what lies beyond a head's d (or vd) elements is written as zeros.  sigmoid of the gate logits
//                     goes to a float array.  A token with slot -1 writes no key and no value.
//
// All arithmetic is float; the results are rounded once, when they are stored (float or bfloat16).
#include "common.cuh"

#define QP_WARPS 8
#define QP_MAX_DIM 256

__device__ __forceinline__ void qp_store(void* p, int dtype, size_t i, float v) {
    if (dtype == RV_DTYPE_F32) ((float*)p)[i] = v;
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

// One block per token; a warp takes one head of q, k or v at a time.  NJ: elements of a head slot per lane (P <= 32 NJ).
template <int NJ>
__global__ void __launch_bounds__(QP_WARPS * 32)
qk_unit_prepare_kernel(const float* __restrict__ proj, int row_stride, const int* __restrict__ positions,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot, int table_rows, int halves,
                       const int* __restrict__ slot_mapping, void* __restrict__ cache, void* __restrict__ q_out, int out_dtype,
                       float* __restrict__ gate_out, int nh, int nkv, int d, int vd, int P, int page_size, float eps, int write_kv) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ float buf[QP_WARPS][32 * NJ];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t row = (size_t)t * row_stride;
    int pos = positions[t];
    if (pos < 0) pos = 0;
    if (pos >= table_rows) pos = table_rows - 1;      // the host refuses such positions; never read outside
    const int half = rot >> 1;
    const float* cs = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* sn = sin_t ? sin_t + (size_t)pos * half : nullptr;
    const int slot = write_kv ? slot_mapping[t] : -1;
    const int items = nh + (write_kv ? 2 * nkv : 0);
    float* mine = buf[warp];
    for (int item = warp; item < items; item += QP_WARPS) {
        const int kind = item < nh ? 0 : (item < nh + nkv ? 1 : 2);          // q, k, v
        const int head = kind == 0 ? item : (kind == 1 ? item - nh : item - nh - nkv);
        if (kind != 0 && slot < 0) continue;                                  // (the same for the whole warp)
        const int n = kind == 2 ? vd : d;
        const size_t src = row + (kind == 0 ? (size_t)head * d
                                            : (kind == 1 ? (size_t)nh * d + (size_t)head * d
                                                         : (size_t)(nh + nkv) * d + (size_t)head * vd));
        for (int i = lane; i < n; i += 32) mine[i] = proj[src + i];
        __syncwarp();
        float vals[NJ];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int i = lane + 32 * j;
            float v = i < n ? mine[i] : 0.f;
            if (kind != 2 && i < rot) {
                if (halves) {
                    const bool first = i < half;
                    const int p = first ? i : i - half;
                    const float other = mine[first ? i + half : i - half];
                    v = first ? v * cs[p] - other * sn[p] : v * cs[p] + other * sn[p];
                } else {
                    const int p = i >> 1;
                    const float other = mine[i ^ 1];
                    v = (i & 1) ? v * cs[p] + other * sn[p] : v * cs[p] - other * sn[p];
                }
            }
            vals[j] = v;
            ss = fmaf(v, v, ss);
        }
        float r = 1.f;
        if (kind != 2) {
            ss = rv_warp_sum(ss);
            r = 1.0f / sqrtf(ss / (float)n + eps);
        }
        void* dst_base;
        size_t dst;
        if (kind == 0) {
            dst_base = q_out;
            dst = ((size_t)t * nh + head) * P;
        } else {
            dst_base = cache;
            const size_t page = (size_t)(slot / page_size), off = (size_t)(slot % page_size);
            dst = (((page * 2 + (kind == 2 ? 1 : 0)) * nkv + head) * page_size + off) * P;
        }
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int i = lane + 32 * j;
            if (i < P) qp_store(dst_base, out_dtype, dst + i, i < n ? vals[j] * r : 0.f);
        }
        __syncwarp();
    }
    if (gate_out) {
        const size_t g0 = row + (size_t)nh * d + (write_kv ? (size_t)nkv * (d + vd) : 0);
        for (int h = threadIdx.x; h < nh; h += blockDim.x)
            gate_out[(size_t)t * nh + h] = 1.0f / (1.0f + expf(-proj[g0 + h]));
    }
}

RV_EXPORT int rv_qk_unit_prepare(const float* proj, int row_stride, const int* positions, const float* cos_t, const float* sin_t,
                                 int rot, int table_rows, int halves, const int* slot_mapping, void* cache, void* q_out, int out_dtype,
                                 float* gate_out, int n_tokens, int nh, int nkv, int d, int vd, int P, int page_size, float eps,
                                 int write_kv, cudaStream_t stream) {
    if (n_tokens < 0 || nh <= 0 || nkv <= 0 || d <= 0 || vd <= 0 || P < d || P < vd || page_size <= 0 || table_rows <= 0)
        return RV_ERR_BAD_SIZE;
    if (P > QP_MAX_DIM) return RV_ERR_UNSUPPORTED;
    if (rot < 0 || rot > d || (rot & 1)) return RV_ERR_BAD_SIZE;
    if (row_stride < nh * d + (write_kv ? nkv * (d + vd) : 0) + (gate_out ? nh : 0)) return RV_ERR_BAD_SIZE;
    if (write_kv && (!slot_mapping || !cache)) return RV_ERR_BAD_SIZE;
    if (out_dtype & ~1) return RV_ERR_BAD_DTYPE;
    if (n_tokens == 0) return RV_OK;
    if (!cos_t || !sin_t) rot = 0;
    auto kernel = P <= 32 ? qk_unit_prepare_kernel<1> : (P <= 64 ? qk_unit_prepare_kernel<2> : (P <= 128 ? qk_unit_prepare_kernel<4>
                                                                                                              : qk_unit_prepare_kernel<8>));
    RV_LAUNCH_ST = rv_launch(kernel, dim3(n_tokens), dim3(QP_WARPS * 32), 0, stream, proj, row_stride, positions, cos_t,
                             sin_t, rot, table_rows, halves, slot_mapping, cache, q_out, out_dtype, gate_out, nh, nkv, d, vd, P,
                             page_size, eps, write_kv);
    return rv_launch_status();
}
