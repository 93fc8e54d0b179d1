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
//   dynamic_tanh          tanh(alpha x) * w + b element by element (alpha: one number on the device)
//   residual_dynamic_tanh x += tanh(alpha y) * w + b on the float32 stream and, optionally, the same form of norm of the
//                         new x with a second (alpha, w, b), in the activations' type: the next sublayer's input
//   scale_rows            x * s as float32 (the start of a float32 stream from a table kept in 16 bits)
//   act_rows              relu(u)^2, optionally times one number per row, in the activations' type
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

// ------------------------------------------------------------------ Dynamic-Tanh norms
// Element-wise, four neighbouring columns per thread where the width allows 16-byte accesses of the float arrays.
__global__ void dynamic_tanh_kernel(const void* __restrict__ x, int x_dtype, const float* __restrict__ alpha, const float* __restrict__ w,
                                    const float* __restrict__ b, void* __restrict__ out, int out_dtype, int cols, size_t total) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const float a = alpha[0];
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % cols);
        so_store(out, out_dtype, i, fmaf(tanhf(a * so_load(x, x_dtype, i)), w[c], b[c]));
    }
}

// x and y float [rows, cols]; `next` (alpha2, w2, b2) optional.  vec: cols % 4 == 0 and 16-byte aligned float pointers.
template <bool VEC>
__global__ void residual_dynamic_tanh_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ alpha,
                                             const float* __restrict__ w, const float* __restrict__ b, const float* __restrict__ alpha2,
                                             const float* __restrict__ w2, const float* __restrict__ b2, void* __restrict__ out,
                                             int out_dtype, int cols, size_t total) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const float a = alpha[0], a2 = out ? alpha2[0] : 0.f;
    if constexpr (VEC) {
        const size_t quads = total / 4;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (size_t)gridDim.x * blockDim.x) {
            const int c = (int)((i * 4) % cols);
            float4 xv = reinterpret_cast<float4*>(x)[i];
            const float4 yv = reinterpret_cast<const float4*>(y)[i];
            const float4 wv = *reinterpret_cast<const float4*>(w + c), bv = *reinterpret_cast<const float4*>(b + c);
            xv.x += fmaf(tanhf(a * yv.x), wv.x, bv.x); xv.y += fmaf(tanhf(a * yv.y), wv.y, bv.y);
            xv.z += fmaf(tanhf(a * yv.z), wv.z, bv.z); xv.w += fmaf(tanhf(a * yv.w), wv.w, bv.w);
            reinterpret_cast<float4*>(x)[i] = xv;
            if (out) {
                const float4 w2v = *reinterpret_cast<const float4*>(w2 + c), b2v = *reinterpret_cast<const float4*>(b2 + c);
                const float o0 = fmaf(tanhf(a2 * xv.x), w2v.x, b2v.x), o1 = fmaf(tanhf(a2 * xv.y), w2v.y, b2v.y);
                const float o2 = fmaf(tanhf(a2 * xv.z), w2v.z, b2v.z), o3 = fmaf(tanhf(a2 * xv.w), w2v.w, b2v.w);
                if (out_dtype == RV_DTYPE_F32) {
                    reinterpret_cast<float4*>(out)[i] = make_float4(o0, o1, o2, o3);
                } else {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
                    uint2 pk;
                    pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
                    reinterpret_cast<uint2*>(out)[i] = pk;
                }
            }
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
            const int c = (int)(i % cols);
            const float v = x[i] + fmaf(tanhf(a * y[i]), w[c], b[c]);
            x[i] = v;
            if (out) so_store(out, out_dtype, i, fmaf(tanhf(a2 * v), w2[c], b2[c]));
        }
    }
}

static inline int so_blocks(size_t items) {
    const size_t want = (items + 255) / 256;
    return (int)(want < 148 * 16 ? (want ? want : 1) : 148 * 16);
}

RV_EXPORT int rv_dynamic_tanh(const void* x, int x_dtype, const float* alpha, const float* w, const float* b, void* out, int out_dtype,
                              int rows, int cols, cudaStream_t stream) {
    if (rows < 0 || cols <= 0) return RV_ERR_BAD_SIZE;
    if ((x_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (rows == 0) return RV_OK;
    const size_t total = (size_t)rows * cols;
    RV_LAUNCH_ST = rv_launch(dynamic_tanh_kernel, dim3(so_blocks(total)), dim3(256), 0, stream, x, x_dtype, alpha, w, b, out, out_dtype,
                             cols, total);
    return rv_launch_status();
}

RV_EXPORT int rv_residual_dynamic_tanh(float* x, const float* y, const float* alpha, const float* w, const float* b, const float* alpha2,
                                       const float* w2, const float* b2, void* out, int out_dtype, int rows, int cols,
                                       cudaStream_t stream) {
    if (rows < 0 || cols <= 0) return RV_ERR_BAD_SIZE;
    if (out_dtype & ~1) return RV_ERR_BAD_DTYPE;
    if (out && (!alpha2 || !w2 || !b2)) return RV_ERR_BAD_SIZE;
    if (rows == 0) return RV_OK;
    const size_t total = (size_t)rows * cols;
    uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w) |
                     reinterpret_cast<uintptr_t>(b);
    if (out) bits |= reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(w2) | reinterpret_cast<uintptr_t>(b2);
    if (cols % 4 == 0 && bits % 16 == 0)
        RV_LAUNCH_ST = rv_launch(residual_dynamic_tanh_kernel<true>, dim3(so_blocks(total / 4)), dim3(256), 0, stream, x, y, alpha, w, b,
                                 alpha2, w2, b2, out, out_dtype, cols, total);
    else
        RV_LAUNCH_ST = rv_launch(residual_dynamic_tanh_kernel<false>, dim3(so_blocks(total)), dim3(256), 0, stream, x, y, alpha, w, b,
                                 alpha2, w2, b2, out, out_dtype, cols, total);
    return rv_launch_status();
}

// ------------------------------------------------------------------ scaled rows, squared-relu rows
__global__ void scale_rows_kernel(const void* __restrict__ x, int x_dtype, float scale, float* __restrict__ out, size_t total) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = so_load(x, x_dtype, i) * scale;
}

__global__ void act_rows_kernel(const void* __restrict__ u, int u_dtype, const float* __restrict__ row_scale, void* __restrict__ out,
                                int out_dtype, int cols, size_t total) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(so_load(u, u_dtype, i), 0.f);
        so_store(out, out_dtype, i, row_scale ? v * v * row_scale[i / cols] : v * v);
    }
}

// float32 in, bfloat16 out, four neighbouring columns per thread (cols % 4 == 0, aligned pointers)
__global__ void act_rows_vec_kernel(const float4* __restrict__ u, const float* __restrict__ row_scale, uint2* __restrict__ out, int cols,
                                    size_t quads) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = u[i];
        const float s = row_scale ? row_scale[(i * 4) / cols] : 1.f;
        const float a = fmaxf(v.x, 0.f), b = fmaxf(v.y, 0.f), c = fmaxf(v.z, 0.f), d = fmaxf(v.w, 0.f);
        // (the same products in the same order as the general kernel: v * v, then the row's scale)
        __nv_bfloat162 lo = row_scale ? __floats2bfloat162_rn(a * a * s, b * b * s) : __floats2bfloat162_rn(a * a, b * b);
        __nv_bfloat162 hi = row_scale ? __floats2bfloat162_rn(c * c * s, d * d * s) : __floats2bfloat162_rn(c * c, d * d);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
        out[i] = pk;
    }
}

RV_EXPORT int rv_scale_rows(const void* x, int x_dtype, float scale, float* out, long long total, cudaStream_t stream) {
    if (total < 0) return RV_ERR_BAD_SIZE;
    if (x_dtype & ~1) return RV_ERR_BAD_DTYPE;
    if (total == 0) return RV_OK;
    RV_LAUNCH_ST = rv_launch(scale_rows_kernel, dim3(so_blocks((size_t)total)), dim3(256), 0, stream, x, x_dtype, scale, out, (size_t)total);
    return rv_launch_status();
}

// mode 0: relu(u)^2
RV_EXPORT int rv_act_rows(const void* u, int u_dtype, const float* row_scale, void* out, int out_dtype, int mode, int rows, int cols,
                          cudaStream_t stream) {
    if (rows < 0 || cols <= 0) return RV_ERR_BAD_SIZE;
    if ((u_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (mode != 0) return RV_ERR_UNSUPPORTED;
    if (rows == 0) return RV_OK;
    const size_t total = (size_t)rows * cols;
    if (u_dtype == RV_DTYPE_F32 && out_dtype == RV_DTYPE_BF16 && cols % 4 == 0 &&
        (reinterpret_cast<uintptr_t>(u) % 16) == 0 && (reinterpret_cast<uintptr_t>(out) % 8) == 0)
        RV_LAUNCH_ST = rv_launch(act_rows_vec_kernel, dim3(so_blocks(total / 4)), dim3(256), 0, stream, (const float4*)u, row_scale, (uint2*)out,
                                 cols, total / 4);
    else
        RV_LAUNCH_ST = rv_launch(act_rows_kernel, dim3(so_blocks(total)), dim3(256), 0, stream, u, u_dtype, row_scale, out, out_dtype, cols, total);
    return rv_launch_status();
}
