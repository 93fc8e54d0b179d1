// Row-wise kernels for pre-norm layers on a float32 residual stream, and small steps around their mixers:
//
//   scale_add_sinusoid    x <- x * s + pe(p): the embedded tokens, scaled, plus a sinusoidal position vector
//                         (pe[2i] = sin(p w_i), pe[2i+1] = cos(p w_i)); the angle is formed in double precision and
//                         brought into one turn before the float32 sine and cosine
//   stream_add_norm       x += y on the float32 stream (y optional), and a second result in the activations' type:
//                         the new x itself, or the new x under an RMSNorm (the input of the next sublayer)
//   gelu_mul_columns      gelu_tanh(g[t, c]) * e[t, col0 + c]: a gate times a slice of a wider row
//   column_slice          a contiguous copy of some columns of a matrix, in another type
//   scaled_sum            a <- sa * a + sb * b (float32), or a <- sb * b where a starts
//   act_mul_clamp         rows [gate | up] -> g sigmoid(alpha g) (u + 1), g = min(gate, L), u = clamp(up, -L, L)
//   head_norm_gate        per head: o / sqrt(mean(o^2) + eps) * w * silu(z), w shared by the heads
//
// All arithmetic is float (the angle: double); storage is float or bfloat16 per argument.  Any width.
#include "common.cuh"

__device__ __forceinline__ float so_load(const void* p, int dtype, size_t i) {
    return dtype == RV_DTYPE_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void so_store(void* p, int dtype, size_t i, float v) {
    if (dtype == RV_DTYPE_F32) ((float*)p)[i] = v;
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float so_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float so_gelu_tanh(float z) {
    const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.0f + tanhf(u));
}

// ------------------------------------------------------------------ scaled embeddings + position vector
// One thread per pair of columns (2i, 2i + 1).
__global__ void scale_add_sinusoid_kernel(const void* __restrict__ x, int x_dtype, const int* __restrict__ positions,
                                          const double* __restrict__ freq, float scale, float* __restrict__ out, int cols,
                                          int pairs, size_t total_pairs) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const double two_pi = 6.283185307179586476925286766559;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_pairs; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / pairs;
        const int pr = (int)(i - row * pairs);
        double a = (double)positions[row] * freq[pr];
        a -= two_pi * rint(a / two_pi);
        float s, c;
        sincosf((float)a, &s, &c);
        const size_t e = row * cols + 2 * pr;
        out[e] = fmaf(so_load(x, x_dtype, e), scale, s);
        if (2 * pr + 1 < cols) out[e + 1] = fmaf(so_load(x, x_dtype, e + 1), scale, c);
    }
}

RV_EXPORT int rv_scale_add_sinusoid(const void* x, int x_dtype, const int* positions, const double* freq, float scale, float* out,
                                    int rows, int cols, cudaStream_t stream) {
    if (rows < 0 || cols <= 0) return RV_ERR_BAD_SIZE;
    if (x_dtype & ~1) return RV_ERR_BAD_DTYPE;
    if (rows == 0) return RV_OK;
    const int pairs = (cols + 1) / 2;
    const size_t total = (size_t)rows * pairs;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    RV_LAUNCH_ST = rv_launch(scale_add_sinusoid_kernel, dim3(blocks), dim3(256), 0, stream, x, x_dtype, positions, freq, scale, out,
                             cols, pairs, total);
    return rv_launch_status();
}

// ------------------------------------------------------------------ stream += y, and the next sublayer's input
// One block per row.  gamma null: the second result is the new stream itself (rounded); rounded null: only the sum.
__global__ void __launch_bounds__(256)
stream_add_norm_kernel(float* __restrict__ x, const float* __restrict__ y, const void* __restrict__ gamma, int gamma_dtype,
                       void* __restrict__ rounded, int rounded_dtype, int cols, float eps) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * cols;
    float ss = 0.f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float v = x[base + i];
        if (y) {
            v += y[base + i];
            x[base + i] = v;
        }
        ss = fmaf(v, v, ss);
        if (rounded && !gamma) so_store(rounded, rounded_dtype, base + i, v);
    }
    if (!rounded || !gamma) return;
    ss = rv_block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)cols + eps);
    for (int i = threadIdx.x; i < cols; i += blockDim.x)     // every thread reads back what it wrote itself
        so_store(rounded, rounded_dtype, base + i, x[base + i] * r * rv_load_param(gamma, gamma_dtype, i));
}

RV_EXPORT int rv_stream_add_norm(float* x, const float* y, const void* gamma, int gamma_dtype, void* rounded, int rounded_dtype,
                                 int rows, int cols, float eps, cudaStream_t stream) {
    if (rows < 0 || cols <= 0) return RV_ERR_BAD_SIZE;
    if ((gamma_dtype | rounded_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (rows == 0 || (!y && !rounded)) return RV_OK;
    RV_LAUNCH_ST = rv_launch(stream_add_norm_kernel, dim3(rows), dim3(cols >= 1024 ? 256 : 128), 0, stream, x, y, gamma, gamma_dtype,
                             rounded, rounded_dtype, cols, eps);
    return rv_launch_status();
}

// ------------------------------------------------------------------ small element-wise steps
__global__ void gelu_mul_columns_kernel(const void* __restrict__ g, int g_dtype, const void* __restrict__ e, int e_dtype,
                                        int e_stride, int col0, void* __restrict__ out, int out_dtype, int cols, size_t total) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / cols, c = i - row * cols;
        so_store(out, out_dtype, i, so_gelu_tanh(so_load(g, g_dtype, i)) * so_load(e, e_dtype, row * e_stride + col0 + c));
    }
}

RV_EXPORT int rv_gelu_mul_columns(const void* g, int g_dtype, const void* e, int e_dtype, int e_stride, int col0, void* out,
                                  int out_dtype, int rows, int cols, cudaStream_t stream) {
    if (rows < 0 || cols <= 0 || col0 < 0 || col0 + cols > e_stride) return RV_ERR_BAD_SIZE;
    if ((g_dtype | e_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (rows == 0) return RV_OK;
    const size_t total = (size_t)rows * cols;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    RV_LAUNCH_ST = rv_launch(gelu_mul_columns_kernel, dim3(blocks), dim3(256), 0, stream, g, g_dtype, e, e_dtype, e_stride, col0, out,
                             out_dtype, cols, total);
    return rv_launch_status();
}

__global__ void column_slice_kernel(const void* __restrict__ x, int x_dtype, int x_stride, int col0, void* __restrict__ out,
                                    int out_dtype, int cols, size_t total) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / cols, c = i - row * cols;
        so_store(out, out_dtype, i, so_load(x, x_dtype, row * x_stride + col0 + c));
    }
}

RV_EXPORT int rv_column_slice(const void* x, int x_dtype, int x_stride, int col0, void* out, int out_dtype, int rows, int cols,
                              cudaStream_t stream) {
    if (rows < 0 || cols <= 0 || col0 < 0 || col0 + cols > x_stride) return RV_ERR_BAD_SIZE;
    if ((x_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (rows == 0) return RV_OK;
    const size_t total = (size_t)rows * cols;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    RV_LAUNCH_ST = rv_launch(column_slice_kernel, dim3(blocks), dim3(256), 0, stream, x, x_dtype, x_stride, col0, out, out_dtype, cols,
                             total);
    return rv_launch_status();
}

// out = sa * a + sb * b; a null: out = sb * b.  out may be a.
__global__ void scaled_sum_kernel(const float* a, float sa, const float* __restrict__ b, float sb, float* out, size_t total) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = a ? fmaf(sa, a[i], sb * b[i]) : sb * b[i];
}

RV_EXPORT int rv_scaled_sum(const float* a, float sa, const float* b, float sb, float* out, long long total, cudaStream_t stream) {
    if (total < 0) return RV_ERR_BAD_SIZE;
    if (total == 0) return RV_OK;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    RV_LAUNCH_ST = rv_launch(scaled_sum_kernel, dim3(blocks), dim3(256), 0, stream, a, sa, b, sb, out, (size_t)total);
    return rv_launch_status();
}

__global__ void act_mul_clamp_kernel(const void* __restrict__ gate_up, int in_dtype, void* __restrict__ out, int out_dtype,
                                     int inter, size_t total, float limit, float alpha) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / inter, c = i - row * inter;
        const float g = fminf(so_load(gate_up, in_dtype, row * 2 * inter + c), limit);
        const float u = fminf(fmaxf(so_load(gate_up, in_dtype, row * 2 * inter + inter + c), -limit), limit);
        so_store(out, out_dtype, i, g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
    }
}

RV_EXPORT int rv_act_mul_clamp(const void* gate_up, int in_dtype, void* out, int out_dtype, int rows, int inter, float limit,
                               float alpha, cudaStream_t stream) {
    if (rows < 0 || inter <= 0 || !(limit > 0.f)) return RV_ERR_BAD_SIZE;
    if ((in_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (rows == 0) return RV_OK;
    const size_t total = (size_t)rows * inter;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    RV_LAUNCH_ST = rv_launch(act_mul_clamp_kernel, dim3(blocks), dim3(256), 0, stream, gate_up, in_dtype, out, out_dtype, inter, total,
                             limit, alpha);
    return rv_launch_status();
}

// ------------------------------------------------------------------ per-head RMSNorm with a shared weight, then a SiLU gate
// One warp per (token, head); z is read from rows of `z_stride` elements at column z_col0.
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ o, const void* __restrict__ gamma, int gamma_dtype, const void* __restrict__ z,
                      int z_dtype, int z_stride, int z_col0, void* __restrict__ out, int out_dtype, int heads, int vd, float eps,
                      size_t total_heads) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int lane = threadIdx.x & 31;
    const size_t w = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= total_heads) return;
    const size_t t = w / heads;
    const int h = (int)(w - t * heads);
    const size_t ob = w * vd, zb = t * z_stride + z_col0 + (size_t)h * vd;
    float ss = 0.f;
    for (int i = lane; i < vd; i += 32) ss = fmaf(o[ob + i], o[ob + i], ss);
    ss = rv_warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)vd + eps);
    for (int i = lane; i < vd; i += 32)
        so_store(out, out_dtype, ob + i, o[ob + i] * r * rv_load_param(gamma, gamma_dtype, i) * so_silu(so_load(z, z_dtype, zb + i)));
}

RV_EXPORT int rv_head_norm_gate(const float* o, const void* gamma, int gamma_dtype, const void* z, int z_dtype, int z_stride,
                                int z_col0, void* out, int out_dtype, int rows, int heads, int vd, float eps, cudaStream_t stream) {
    if (rows < 0 || heads <= 0 || vd <= 0 || z_col0 < 0 || z_col0 + heads * vd > z_stride) return RV_ERR_BAD_SIZE;
    if ((gamma_dtype | z_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (rows == 0) return RV_OK;
    const size_t total = (size_t)rows * heads;
    RV_LAUNCH_ST = rv_launch(head_norm_gate_kernel, dim3((unsigned)((total + 7) / 8)), dim3(256), 0, stream, o, gamma, gamma_dtype, z,
                             z_dtype, z_stride, z_col0, out, out_dtype, heads, vd, eps, total);
    return rv_launch_status();
}
