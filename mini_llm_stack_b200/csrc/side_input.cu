// A layer's input from a per-token side table, applied to the settled residual stream:
//
//   mls_settle_cast     x += delta (a tensor, the K-parts of a product, or nothing);
//                       out = x in the activation type (what the gate's product reads)
//   mls_gelu_gate_rows  out[t, c] = gelu_tanh(z[t, c]) * table[token[t], col0 + c] for c < n_real,
//                       0 for the other columns of the row (a row padded for the products)
//                       gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
//   mls_rms_scale       out[t] = y[t] / sqrt(mean(y[t]^2) + eps) * w   (float32; y a tensor or
//                       the K-parts of a product) -- a delta for the residual stream
//
// All sums and functions in float32; a row's sum of squares runs in thread-stride order and
// the block's fixed tree, so it does not depend on the batch.
#include "common.cuh"

namespace {
__device__ __forceinline__ float delta_at(const void* delta, int dtype, int n_parts, size_t stride,
                                          size_t i) {
    if (!delta) return 0.f;
    if (dtype == MLS_BF16) return __bfloat162float(((const __nv_bfloat16*)delta)[i]);
    float s = 0.f;
    for (int k = 0; k < n_parts; ++k) s += ((const float*)delta)[i + (size_t)k * stride];
    return s;
}

template <typename T>
__global__ void settle_cast_kernel(float* __restrict__ x, const void* __restrict__ delta,
                                   int delta_dtype, int n_parts, long long stride,
                                   T* __restrict__ out, size_t n) {
    chain_release();
    chain_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i];
        if (delta) {
            v += delta_at(delta, delta_dtype, n_parts, (size_t)stride, i);
            x[i] = v;
        }
        Elem<T>::store(out + i, v);
    }
}

template <typename T>
__global__ void gelu_gate_rows_kernel(const float* __restrict__ z, const void* __restrict__ table,
                                      int table_dtype, int table_width, int col0,
                                      const int* __restrict__ ids, int vocab, T* __restrict__ out,
                                      int n_tokens, int dim, int n_real, int* __restrict__ status) {
    chain_release();
    chain_wait();
    const size_t n = (size_t)n_tokens * dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / dim, c = i - t * dim;
        const int id = ids[t];
        if (id < 0 || id >= vocab || (int)c >= n_real) {
            if ((int)c < n_real && status) atomicOr(status, MLS_STATUS_BAD_TOKEN);
            Elem<T>::store(out + i, 0.f);
            continue;
        }
        const float v = z[i];
        const float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
        const float g = 0.5f * v * (1.0f + tanhf(inner));
        Elem<T>::store(out + i, g * load_as_float(table, (size_t)id * table_width + col0 + c,
                                                  table_dtype));
    }
}

__global__ void __launch_bounds__(256)
rms_scale_kernel(const void* __restrict__ y, int y_dtype, int n_parts, long long stride,
                 const float* __restrict__ w, float eps, float* __restrict__ out, int d) {
    chain_release();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * d;
    chain_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = delta_at(y, y_dtype, n_parts, (size_t)stride, base + i);
        out[base + i] = v;
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[base + i] = out[base + i] * inv * w[i];
}
}  // namespace

MLS_API int mls_settle_cast(float* x, const void* delta, int delta_dtype, int n_parts,
                            long long stride, void* out, int out_dtype, int n_tokens, int d,
                            cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const size_t n = (size_t)n_tokens * d;
    const size_t want = (n + 255) / 256;
    const int blocks = (int)(want < (size_t)(8 * sm_count()) ? want : 8 * sm_count());
    if (out_dtype == MLS_BF16)
        MLS_LAUNCH((settle_cast_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, x, delta,
                   delta_dtype, n_parts, stride, (__nv_bfloat16*)out, n);
    else
        MLS_LAUNCH((settle_cast_kernel<float>), dim3(blocks), dim3(256), 0, stream, x, delta,
                   delta_dtype, n_parts, stride, (float*)out, n);
    return launch_status();
}

MLS_API int mls_gelu_gate_rows(const float* z, const void* table, int table_dtype, int table_width,
                               int col0, const int* ids, int vocab, void* out, int out_dtype,
                               int n_tokens, int dim, int n_real, int* status,
                               cudaStream_t stream) {
    if (n_tokens <= 0 || dim <= 0) return 0;
    if (col0 < 0 || n_real > dim || col0 + n_real > table_width) return MLS_ERR_UNSUPPORTED;
    const size_t n = (size_t)n_tokens * dim;
    const size_t want = (n + 255) / 256;
    const int blocks = (int)(want < (size_t)(8 * sm_count()) ? want : 8 * sm_count());
    if (out_dtype == MLS_BF16)
        MLS_LAUNCH((gelu_gate_rows_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, z,
                   table, table_dtype, table_width, col0, ids, vocab, (__nv_bfloat16*)out, n_tokens,
                   dim, n_real, status);
    else
        MLS_LAUNCH((gelu_gate_rows_kernel<float>), dim3(blocks), dim3(256), 0, stream, z, table,
                   table_dtype, table_width, col0, ids, vocab, (float*)out, n_tokens, dim, n_real, status);
    return launch_status();
}

MLS_API int mls_rms_scale(const void* y, int y_dtype, int n_parts, long long stride, const float* w,
                          float eps, float* out, int n_tokens, int d, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    MLS_LAUNCH((rms_scale_kernel), dim3(n_tokens), dim3(256), 0, stream, y, y_dtype, n_parts,
               stride, w, eps, out, d);
    return launch_status();
}
