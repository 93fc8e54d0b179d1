// A mixture of experts whose choice per token is given (a table lookup by token id, a router's top-k): every token runs
// `top` experts and adds them, with one weight for all or one per (token, slot).  An expert is gated,
// down_e( silu(gate_e x) * up_e x ), or plain, down_e( relu(up_e x)^2 ).
//
// Layout: gate_up [experts, 2 ff, width] (an expert's gate rows, then its up rows; plain experts: up [experts, ff, width]),
// down [experts, width, ff], chosen [tokens, top] int32 expert numbers (numbers outside 0 .. experts-1 contribute
// nothing), weights float [tokens, top] or null.
//
//   moe_route_top act on a router's float32 logits: s = sigmoid(z); the choice is made among s + correction, within the best
//                 `keep` of `groups` equal groups of neighbouring experts (a group counts by the sum of its two largest
//                 corrected scores); chosen [tokens, top], weights = the chosen s over their sum (+ eps)
//   moe_gate_up   act[t * top + k, f] = silu(gate_e[f] . x_t) * (up_e[f] . x_t)  or  relu(up_e[f] . x_t)^2,  e = chosen[t, k]
//   moe_down      out[t, n] = (add[t, n]) + weight * sum_k weights[t, k] down_e(k)[n] . act[t * top + k]
//
// One CTA per (token, slot) and block of features keeps the token's vector in shared memory as float; a warp owns a
// feature at a time and its lanes walk the weight row (16-byte loads where rows are aligned).  The weights of an
// expert are read once per token that chose it: the kernels serve decoded tokens and short portions, where the step
// is bound by reading the chosen experts' weights; sums are float, in one order whatever the batch.
//
// Many tokens take another way, on the tensor cores: the (token, slot) pairs are sorted by expert into a buffer in
// which every expert's rows are padded to whole row tiles, and two grouped products (gemm_tcgen05.cu: row tile t is
// multiplied with the matrices of expert tile_group[t]) run over it.  The kernels here do the sorting and the sum:
//
//   moe_route     row_of[pair], src_of[row] and the products' work units (tile_group, tile_rows) from chosen (one CTA:
//                 counts, padded offsets, places)
//   moe_gather    xs[row] = x[src_of[row]], zeros in the padding
//   moe_combine   out[t] = (add[t]) + weight * sum_k weights[t, k] ys[row_of[t * top + k]]   (slots in their order: one sum per element)
#include "common.cuh"

// N rows of W against one vector at a time: the lanes walk all rows together, so N loads are in flight per lane and step
// (one row after the other left the memory idle between a row's reduction and the next row's first load).
template <typename T, int N>
__device__ __forceinline__ void moe_dot_rows(const T* const (&w)[N], const float* __restrict__ x, int n, int lane, float (&out)[N]) {
    float s[N];
#pragma unroll
    for (int r = 0; r < N; ++r) s[r] = 0.f;
    constexpr int V = 16 / sizeof(T);                      // elements of a 16-byte load
    bool aligned = (n % V) == 0;
#pragma unroll
    for (int r = 0; r < N; ++r) aligned = aligned && ((uintptr_t)w[r] & 15) == 0;
    if (aligned) {
        for (int i = lane * V; i < n; i += 32 * V) {
            uint4 v[N];
#pragma unroll
            for (int r = 0; r < N; ++r) v[r] = __ldg(reinterpret_cast<const uint4*>(w[r] + i));
#pragma unroll
            for (int r = 0; r < N; ++r) {
                if constexpr (sizeof(T) == 4) {
                    const float* f = reinterpret_cast<const float*>(&v[r]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) s[r] = fmaf(f[j], x[i + j], s[r]);
                } else {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[r]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __bfloat1622float2(h[j]);
                        s[r] = fmaf(f.x, x[i + 2 * j], s[r]);
                        s[r] = fmaf(f.y, x[i + 2 * j + 1], s[r]);
                    }
                }
            }
        }
    } else {
        for (int i = lane; i < n; i += 32)
#pragma unroll
            for (int r = 0; r < N; ++r) s[r] = fmaf(rv_to_float(w[r][i]), x[i], s[r]);
    }
#pragma unroll
    for (int r = 0; r < N; ++r) out[r] = rv_warp_sum(s[r]);
}

#define MOE_WARPS 8
#define MOE_FEATURES 32      // features of one CTA
#define MOE_PER_WARP (MOE_FEATURES / MOE_WARPS)

// grid (tokens * top, feature blocks).  GATED: an expert's first matrix holds gate rows and up rows, a CTA covers MOE_FEATURES
// features; plain: up rows only, a CTA covers twice as many (the same number of weight rows walked together).
template <typename T, bool GATED>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_gate_up_kernel(const T* __restrict__ x, const int* __restrict__ chosen, const T* __restrict__ gate_up, T* __restrict__ act,
                   int top, int experts, int ff, int width) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ float xs[];
    const int pair = blockIdx.x, t = pair / top;
    const int e = chosen[pair];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int FEATURES = GATED ? MOE_FEATURES : 2 * MOE_FEATURES;
    const int f0 = blockIdx.y * FEATURES;
    if (e < 0 || e >= experts) {
        for (int f = f0 + threadIdx.x; f < min(ff, f0 + FEATURES); f += blockDim.x) act[(size_t)pair * ff + f] = rv_from_float<T>(0.f);
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = rv_to_float(x[(size_t)t * width + i]);
    __syncthreads();
    if constexpr (!GATED) {
        const T* wu = gate_up + (size_t)e * ff * width;
        const T* rows[2 * MOE_PER_WARP];
#pragma unroll
        for (int j = 0; j < 2 * MOE_PER_WARP; ++j) rows[j] = wu + (size_t)min(ff - 1, f0 + warp + j * MOE_WARPS) * width;
        float r[2 * MOE_PER_WARP];
        moe_dot_rows<T, 2 * MOE_PER_WARP>(rows, xs, width, lane, r);
#pragma unroll
        for (int j = 0; j < 2 * MOE_PER_WARP; ++j) {
            const int f = f0 + warp + j * MOE_WARPS;
            const float v = fmaxf(r[j], 0.f);
            if (lane == 0 && f < ff) act[(size_t)pair * ff + f] = rv_from_float<T>(v * v);
        }
        return;
    }
    const T* wg = gate_up + (size_t)e * 2 * ff * width;
    const T* wu = wg + (size_t)ff * width;
    // a warp's features f0 + warp, + MOE_WARPS, ...: their gate and up rows are walked together (a feature beyond ff reads
    // the last row again and is not stored)
    const T* rows[2 * MOE_PER_WARP];
#pragma unroll
    for (int j = 0; j < MOE_PER_WARP; ++j) {
        const int f = min(ff - 1, f0 + warp + j * MOE_WARPS);
        rows[2 * j] = wg + (size_t)f * width;
        rows[2 * j + 1] = wu + (size_t)f * width;
    }
    float r[2 * MOE_PER_WARP];
    moe_dot_rows<T, 2 * MOE_PER_WARP>(rows, xs, width, lane, r);
#pragma unroll
    for (int j = 0; j < MOE_PER_WARP; ++j) {
        const int f = f0 + warp + j * MOE_WARPS;
        if (lane == 0 && f < ff) act[(size_t)pair * ff + f] = rv_from_float<T>(r[2 * j] / (1.0f + expf(-r[2 * j])) * r[2 * j + 1]);
    }
}

// grid (tokens, feature blocks)
template <typename T, typename TO>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_down_kernel(const T* __restrict__ act, const int* __restrict__ chosen, const T* __restrict__ down, const float* add,
                TO* out, int top, int experts, int ff, int width, float weight, const float* __restrict__ weights) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ float as[];                 // [top][ff]
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) as[i] = rv_to_float(act[(size_t)t * top * ff + i]);
    __syncthreads();
    const int n0 = blockIdx.y * MOE_FEATURES;
    float sum[MOE_PER_WARP];
#pragma unroll
    for (int j = 0; j < MOE_PER_WARP; ++j) sum[j] = 0.f;
    for (int k = 0; k < top; ++k) {                       // the slots in their order: one sum per element, whatever the batch
        const int e = chosen[t * top + k];
        if (e < 0 || e >= experts) continue;
        const T* rows[MOE_PER_WARP];
#pragma unroll
        for (int j = 0; j < MOE_PER_WARP; ++j) rows[j] = down + ((size_t)e * width + min(width - 1, n0 + warp + j * MOE_WARPS)) * ff;
        float r[MOE_PER_WARP];
        moe_dot_rows<T, MOE_PER_WARP>(rows, as + (size_t)k * ff, ff, lane, r);
        const float wk = weights ? weights[t * top + k] : 1.f;
#pragma unroll
        for (int j = 0; j < MOE_PER_WARP; ++j) sum[j] = fmaf(wk, r[j], sum[j]);
    }
#pragma unroll
    for (int j = 0; j < MOE_PER_WARP; ++j) {
        const int n = n0 + warp + j * MOE_WARPS;
        if (lane == 0 && n < width) {
            float v = sum[j] * weight;
            if (add) v += add[(size_t)t * width + n];
            out[(size_t)t * width + n] = rv_from_float<TO>(v);
        }
    }
}

static RvPerDevice g_once[8];

template <typename T>
static int moe_launch(const void* x, const int* chosen, const float* weights, const void* gate_up, const void* down, void* act,
                      const float* add, void* out, int out_f32, int tokens, int top, int experts, int ff, int width, float weight,
                      int gated, int slot, cudaStream_t stream) {
    const int smem_a = width * 4, smem_b = top * ff * 4;
    if (smem_a > 200 * 1024 || smem_b > 200 * 1024) return RV_ERR_UNSUPPORTED;
    int st;
    if (gated) {
        st = rv_configure_smem(g_once[slot], moe_gate_up_kernel<T, true>, 200 * 1024);
        if (st != RV_OK) return st;
        RV_LAUNCH_ST = rv_launch(moe_gate_up_kernel<T, true>, dim3(tokens * top, (ff + MOE_FEATURES - 1) / MOE_FEATURES), dim3(MOE_WARPS * 32),
                                 (size_t)smem_a, stream, (const T*)x, chosen, (const T*)gate_up, (T*)act, top, experts, ff, width);
    } else {
        st = rv_configure_smem(g_once[slot + 3], moe_gate_up_kernel<T, false>, 200 * 1024);
        if (st != RV_OK) return st;
        RV_LAUNCH_ST = rv_launch(moe_gate_up_kernel<T, false>, dim3(tokens * top, (ff + 2 * MOE_FEATURES - 1) / (2 * MOE_FEATURES)),
                                 dim3(MOE_WARPS * 32), (size_t)smem_a, stream, (const T*)x, chosen, (const T*)gate_up, (T*)act, top,
                                 experts, ff, width);
    }
    st = rv_launch_status();
    if (st != RV_OK) return st;
    const dim3 grid(tokens, (width + MOE_FEATURES - 1) / MOE_FEATURES);
    if (out_f32) {
        st = rv_configure_smem(g_once[slot + 1], moe_down_kernel<T, float>, 200 * 1024);
        if (st != RV_OK) return st;
        RV_LAUNCH_ST = rv_launch(moe_down_kernel<T, float>, dim3(grid), dim3(MOE_WARPS * 32), (size_t)smem_b, stream, (const T*)act,
                                 chosen, (const T*)down, add, (float*)out, top, experts, ff, width, weight, weights);
    } else {
        st = rv_configure_smem(g_once[slot + 2], moe_down_kernel<T, T>, 200 * 1024);
        if (st != RV_OK) return st;
        RV_LAUNCH_ST = rv_launch(moe_down_kernel<T, T>, dim3(grid), dim3(MOE_WARPS * 32), (size_t)smem_b, stream, (const T*)act,
                                 chosen, (const T*)down, add, (T*)out, top, experts, ff, width, weight, weights);
    }
    return rv_launch_status();
}

// x [tokens, width], act [tokens * top, ff] (scratch of the weights' type), add float [tokens, width] or null,
// weights float [tokens, top] or null, out [tokens, width] float (out_f32) or of the weights' type.  gated: 1 the experts'
// first matrix is [gate | up] with SiLU, 0 it is the up matrix with a squared relu.  Two launches.
RV_EXPORT int rv_moe_experts_ex(const void* x, const int* chosen, const float* weights, const void* gate_up, const void* down, void* act,
                                const float* add, void* out, int out_f32, int tokens, int top, int experts, int ff, int width,
                                float weight, int gated, int dtype, cudaStream_t stream) {
    if (tokens < 0 || top <= 0 || experts <= 0 || ff <= 0 || width <= 0) return RV_ERR_BAD_SIZE;
    if ((long long)tokens * top > 0x7fffffffLL || ff > 65535 * MOE_FEATURES || width > 65535 * MOE_FEATURES) return RV_ERR_BAD_SIZE;
    if (tokens == 0) return RV_OK;
    if (dtype == RV_DTYPE_F32)
        return moe_launch<float>(x, chosen, weights, gate_up, down, act, add, out, 1, tokens, top, experts, ff, width, weight, gated, 0, stream);
    if (dtype == RV_DTYPE_BF16)
        return moe_launch<__nv_bfloat16>(x, chosen, weights, gate_up, down, act, add, out, out_f32, tokens, top, experts, ff, width, weight,
                                         gated, 4, stream);
    return RV_ERR_BAD_DTYPE;
}

RV_EXPORT int rv_moe_experts(const void* x, const int* chosen, const void* gate_up, const void* down, void* act, const float* add,
                             void* out, int out_f32, int tokens, int top, int experts, int ff, int width, float weight,
                             int dtype, cudaStream_t stream) {
    return rv_moe_experts_ex(x, chosen, nullptr, gate_up, down, act, add, out, out_f32, tokens, top, experts, ff, width, weight, 1, dtype,
                             stream);
}

// ------------------------------------------------------------------ sorting pairs by expert for the grouped products
// One CTA.  Shared memory: counts[experts], offsets[experts], cursor[experts], first unit[experts].
// Rows: expert e gets ceil(count / block) blocks of `block` rows from offsets[e] on.  Work units of the grouped product:
// `ranks` blocks of one expert each (the CTAs of a tile); where an expert's blocks run out, the unit's last entries are -1.
// order_a / order_b: the work lists of the two products (nt_a / nt_b column tiles per unit), see GemmParams::tile_order.
__global__ void __launch_bounds__(1024)
moe_route_kernel(const int* __restrict__ chosen, int pairs, int top, int experts, int block, int max_rows, int ranks, int max_units,
                 int* __restrict__ row_of, int* __restrict__ src_of, int* __restrict__ tile_group, int* __restrict__ tile_rows,
                 int nt_a, int* __restrict__ order_a, int nt_b, int* __restrict__ order_b) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ int sm[];
    int* counts = sm;
    int* offsets = sm + experts;
    int* cursor = sm + 2 * experts;
    int* unit0 = sm + 3 * experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
    for (int r = threadIdx.x; r < max_rows; r += blockDim.x) src_of[r] = -1;
    for (int t = threadIdx.x; t < max_units; t += blockDim.x) tile_group[t] = -1;
    for (int t = threadIdx.x; t < max_units * ranks; t += blockDim.x) tile_rows[t] = -1;
    for (int t = threadIdx.x; t < max_units * nt_a; t += blockDim.x) order_a[t] = -1;
    for (int t = threadIdx.x; t < max_units * nt_b; t += blockDim.x) order_b[t] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = chosen[i];
        if (e >= 0 && e < experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, unit = 0;
        for (int e = 0; e < experts; ++e) {
            const int blocks = (counts[e] + block - 1) / block;
            offsets[e] = at;
            unit0[e] = unit;
            at += blocks * block;
            unit += (blocks + ranks - 1) / ranks;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const int blocks = (counts[e] + block - 1) / block;
        for (int b = 0; b < blocks; ++b) {
            const int unit = unit0[e] + b / ranks;
            if (unit >= max_units) break;
            tile_group[unit] = e;
            tile_rows[unit * ranks + b % ranks] = offsets[e] + b * block;
        }
        // the order of the two products' work: this expert's entries lie together, column tile by column tile, its units within
        const int units = min((blocks + ranks - 1) / ranks, max(0, max_units - unit0[e]));
        for (int i = 0; i < units * nt_a; ++i) order_a[unit0[e] * nt_a + i] = ((unit0[e] + i % units) << 16) | (i / units);
        for (int i = 0; i < units * nt_b; ++i) order_b[unit0[e] * nt_b + i] = ((unit0[e] + i % units) << 16) | (i / units);
    }
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = chosen[i];
        int row = -1;
        if (e >= 0 && e < experts) {
            row = offsets[e] + atomicAdd(&cursor[e], 1);
            if (row < max_rows) src_of[row] = i / top; else row = -1;
        }
        row_of[i] = row;
    }
}

// xs[row, :] = x[src_of[row], :] or zeros; 16-byte words (`words` per row)
__global__ void moe_gather_kernel(const uint4* __restrict__ x, const int* __restrict__ src_of, uint4* __restrict__ xs, int words,
                                  size_t total) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / words;
        const int src = src_of[row];
        xs[i] = src >= 0 ? x[(size_t)src * words + (i - row * words)] : make_uint4(0u, 0u, 0u, 0u);
    }
}

template <typename TO>
__global__ void moe_combine_kernel(const float* __restrict__ ys, const int* __restrict__ row_of, const float* add, TO* out,
                                   int top, int width, float weight, size_t total, const float* __restrict__ weights) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / width;
        const int n = (int)(i - t * width);
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const int row = row_of[t * top + k];
            if (row >= 0) s = fmaf(weights ? weights[t * top + k] : 1.f, ys[(size_t)row * width + n], s);
        }
        float v = s * weight;
        if (add) v += add[i];
        out[i] = rv_from_float<TO>(v);
    }
}

RV_EXPORT int rv_moe_route(const int* chosen, int pairs, int top, int experts, int block, int max_rows, int ranks, int max_units,
                           int* row_of, int* src_of, int* tile_group, int* tile_rows, int nt_a, int* order_a, int nt_b, int* order_b,
                           cudaStream_t stream) {
    if (pairs < 0 || top <= 0 || experts <= 0 || block <= 0 || max_rows <= 0 || ranks <= 0 || max_units <= 0) return RV_ERR_BAD_SIZE;
    if (nt_a <= 0 || nt_b <= 0 || nt_a > 65535 || nt_b > 65535 || max_units > 32767 || !order_a || !order_b) return RV_ERR_BAD_SIZE;
    if (experts > 4096) return RV_ERR_UNSUPPORTED;
    if ((long long)max_rows < (long long)pairs) return RV_ERR_BAD_SIZE;
    RV_LAUNCH_ST = rv_launch(moe_route_kernel, dim3(1), dim3(1024), (size_t)4 * experts * sizeof(int), stream, chosen, pairs, top, experts,
                             block, max_rows, ranks, max_units, row_of, src_of, tile_group, tile_rows, nt_a, order_a, nt_b, order_b);
    return rv_launch_status();
}

RV_EXPORT int rv_moe_gather(const void* x, const int* src_of, void* xs, int rows, int width_bytes, cudaStream_t stream) {
    if (rows < 0 || width_bytes <= 0 || width_bytes % 16) return RV_ERR_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(xs)) % 16) return RV_ERR_ALIGNMENT;
    if (rows == 0) return RV_OK;
    const size_t total = (size_t)rows * (width_bytes / 16);
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    RV_LAUNCH_ST = rv_launch(moe_gather_kernel, dim3(blocks), dim3(256), 0, stream, (const uint4*)x, src_of, (uint4*)xs, width_bytes / 16, total);
    return rv_launch_status();
}

RV_EXPORT int rv_moe_combine(const float* ys, const int* row_of, const float* add, void* out, int out_f32, int tokens, int top,
                             int width, float weight, const float* weights, cudaStream_t stream) {
    if (tokens < 0 || top <= 0 || width <= 0) return RV_ERR_BAD_SIZE;
    if (tokens == 0) return RV_OK;
    const size_t total = (size_t)tokens * width;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (out_f32)
        RV_LAUNCH_ST = rv_launch(moe_combine_kernel<float>, dim3(blocks), dim3(256), 0, stream, ys, row_of, add, (float*)out, top, width, weight, total, weights);
    else
        RV_LAUNCH_ST = rv_launch(moe_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, ys, row_of, add, (__nv_bfloat16*)out, top,
                                 width, weight, total, weights);
    return rv_launch_status();
}

// ------------------------------------------------------------------ the router's choice
// One warp per token.  Shared memory per warp: s[experts], c[experts], group scores[groups].
#define MR_WARPS 4

__device__ __forceinline__ void mr_argmax(const float* v, int n, int lane, float& best, int& at) {
    best = -INFINITY; at = 0x7fffffff;
    for (int i = lane; i < n; i += 32) {
        const float x = v[i];
        if (x > best || (x == best && i < at)) { best = x; at = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
}

__global__ void __launch_bounds__(MR_WARPS * 32)
moe_route_top_kernel(const float* __restrict__ logits, int stride, const float* __restrict__ correction, int* __restrict__ chosen,
                     float* __restrict__ weights, float* __restrict__ gate_out, int tokens, int experts, int top, int groups, int keep,
                     float weight_eps) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ float mr_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * MR_WARPS + warp;
    if (t >= tokens) return;
    float* s = mr_smem + (size_t)warp * (2 * experts + groups);
    float* c = s + experts;
    float* gs = c + experts;
    const float* z = logits + (size_t)t * stride;
    for (int e = lane; e < experts; e += 32) {
        const float v = 1.0f / (1.0f + expf(-z[e]));
        s[e] = v;
        c[e] = v + correction[e];
    }
    if (gate_out && lane == 0) gate_out[t] = 1.0f / (1.0f + expf(-z[experts]));
    __syncwarp();
    if (keep < groups) {
        const int per = experts / groups;
        for (int g = lane; g < groups; g += 32) {           // a group counts by its two largest corrected scores
            float a = -INFINITY, b = -INFINITY;
            for (int i = 0; i < per; ++i) {
                const float v = c[g * per + i];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            gs[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        for (int k = 0; k < keep; ++k) {                    // the kept groups are marked +inf, then the others are closed
            float best; int at;
            mr_argmax(gs, groups, lane, best, at);
            if (lane == 0) gs[at] = -INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < experts; e += 32)
            if (gs[e / per] != -INFINITY) c[e] = -INFINITY;  // (a kept group was set to -inf when it was taken)
        __syncwarp();
    }
    float sum = 0.f, mine = 0.f;
    for (int k = 0; k < top; ++k) {
        float best; int at;
        mr_argmax(c, experts, lane, best, at);
        if (at >= experts) at = 0;                           // (cannot happen: top <= the experts of the kept groups)
        const float w = s[at];
        sum += w;
        if (lane == k % 32 && k < 32) mine = w;
        if (lane == 0) {
            chosen[(size_t)t * top + k] = at;
            if (k >= 32) weights[(size_t)t * top + k] = w;    // (beyond a warp's lanes: scaled below through memory)
            c[at] = -INFINITY;
        }
        __syncwarp();
    }
    const float inv = 1.0f / (sum + weight_eps);
    if (lane < top && lane < 32) weights[(size_t)t * top + lane] = mine * inv;
    if (lane == 0)
        for (int k = 32; k < top; ++k) weights[(size_t)t * top + k] *= inv;
}

// logits float [tokens, stride]: the experts' logits and, with gate_out, one more column whose sigmoid goes to gate_out.
RV_EXPORT int rv_moe_route_top(const float* logits, int stride, const float* correction, int* chosen, float* weights, float* gate_out,
                               int tokens, int experts, int top, int groups, int keep, float weight_eps, cudaStream_t stream) {
    if (tokens < 0 || experts <= 0 || top <= 0 || top > experts || groups <= 0 || experts % groups || keep <= 0 || keep > groups)
        return RV_ERR_BAD_SIZE;
    if (stride < experts + (gate_out ? 1 : 0) || top > (experts / groups) * keep) return RV_ERR_BAD_SIZE;
    if (experts > 1024) return RV_ERR_UNSUPPORTED;
    if (tokens == 0) return RV_OK;
    const size_t smem = (size_t)MR_WARPS * (2 * experts + groups) * sizeof(float);
    RV_LAUNCH_ST = rv_launch(moe_route_top_kernel, dim3((tokens + MR_WARPS - 1) / MR_WARPS), dim3(MR_WARPS * 32), smem, stream, logits,
                             stride, correction, chosen, weights, gate_out, tokens, experts, top, groups, keep, weight_eps);
    return rv_launch_status();
}
