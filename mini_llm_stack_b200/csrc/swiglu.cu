// SwiGLU activation: out[t, i] = silu(gate[t, i]) * up[t, i] with
// silu(z) = z * sigmoid(z) (reference: train/model.py:135), computed in float32.
// gu: [T, 2*I], a row holds [gate | up].
#include "common.cuh"

namespace {
__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

// 16 bytes per thread and operand: I must be a multiple of 8 (bfloat16) or 4 (float32).
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu,
                                     __nv_bfloat16* __restrict__ out, int inter) {
    chain_release();
    chain_wait();
    const size_t t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;       // chunk of 8
    if (c * 8 >= inter) return;
    const __nv_bfloat16* row = gu + t * 2 * (size_t)inter;
    const uint4 g4 = *reinterpret_cast<const uint4*>(row + c * 8);
    const uint4 u4 = *reinterpret_cast<const uint4*>(row + inter + c * 8);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
        o2[e] = __floats2bfloat162_rn(silu_mul(g.x, u.x), silu_mul(g.y, u.y));
    }
    *reinterpret_cast<uint4*>(out + t * (size_t)inter + c * 8) = o4;
}

__global__ void swiglu_f32x4_kernel(const float* __restrict__ gu, float* __restrict__ out,
                                    int inter) {
    chain_release();
    chain_wait();
    const size_t t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;       // chunk of 4
    if (c * 4 >= inter) return;
    const float* row = gu + t * 2 * (size_t)inter;
    const float4 g = *reinterpret_cast<const float4*>(row + c * 4);
    const float4 u = *reinterpret_cast<const float4*>(row + inter + c * 4);
    float4 o;
    o.x = silu_mul(g.x, u.x);
    o.y = silu_mul(g.y, u.y);
    o.z = silu_mul(g.z, u.z);
    o.w = silu_mul(g.w, u.w);
    *reinterpret_cast<float4*>(out + t * (size_t)inter + c * 4) = o;
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter) {
    chain_release();
    chain_wait();
    const size_t t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const T* row = gu + t * 2 * (size_t)inter;
    Elem<T>::store(out + t * (size_t)inter + i,
                   silu_mul(Elem<T>::load(row + i), Elem<T>::load(row + inter + i)));
}

// The gated product with another gate: g' = min(g, limit), u' = clamp(u, -limit, limit),
// out = g' * sigmoid(alpha * g') * (u' + 1).  (limit <= 0: no clamping.)
__device__ __forceinline__ float clamped_glu(float g, float u, float alpha, float limit) {
    if (limit > 0.f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    return (g / (1.0f + expf(-alpha * g))) * (u + 1.0f);
}
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter,
                                   float alpha, float limit) {
    chain_release();
    chain_wait();
    const size_t t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const T* row = gu + t * 2 * (size_t)inter;
    Elem<T>::store(out + t * (size_t)inter + i,
                   clamped_glu(Elem<T>::load(row + i), Elem<T>::load(row + inter + i), alpha,
                               limit));
}

// Activations without a gate: out = act(in + bias), element by element (in place allowed when
// the types agree); `bias` [width] is optional and belongs to the columns of rows of `width`.
// kind 0: the square of relu.
template <typename TI, typename TO>
__global__ void unary_act_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n,
                                 int kind, const void* __restrict__ bias, int bias_dtype,
                                 int width) {
    chain_release();
    chain_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        float z = Elem<TI>::load(in + i);
        if (bias) z += load_as_float(bias, i % width, bias_dtype);
        z = fmaxf(z, 0.f);
        Elem<TO>::store(out + i, z * z);
    }
}

// x = cap * tanh(x / cap) on float32 values.
__global__ void softcap_f32_kernel(float* __restrict__ x, size_t n, float cap) {
    chain_release();
    chain_wait();
    const float inv = 1.0f / cap;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

__global__ void scale_f32_kernel(float* __restrict__ x, size_t n, float scale) {
    chain_release();
    chain_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        x[i] *= scale;
}
}  // namespace

// out[i] = relu(in[i] + bias[i % width])^2 (kind 0; other kinds are refused).  `in` is of type
// `in_dtype`, `out` of `dtype`; a float32 input with a bfloat16 output is the one mixed pair.
MLS_API int mls_unary_act(const void* in, int in_dtype, void* out, int dtype, long long n,
                          int kind, const void* bias, int bias_dtype, int width,
                          cudaStream_t stream) {
    if (n <= 0) return 0;
    if (kind != 0 || (bias && width <= 0)) return MLS_ERR_UNSUPPORTED;
    if (in_dtype != dtype && !(in_dtype == MLS_F32 && dtype == MLS_BF16)) return MLS_ERR_UNSUPPORTED;
    const long long want = (n + 255) / 256;
    const int blocks = (int)(want < 16LL * sm_count() ? want : 16LL * sm_count());
    if (dtype == MLS_BF16 && in_dtype == MLS_BF16)
        MLS_LAUNCH((unary_act_kernel<__nv_bfloat16, __nv_bfloat16>), dim3(blocks), dim3(256), 0,
                   stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, (size_t)n, kind, bias,
                   bias_dtype, width);
    else if (dtype == MLS_BF16)
        MLS_LAUNCH((unary_act_kernel<float, __nv_bfloat16>), dim3(blocks), dim3(256), 0, stream,
                   (const float*)in, (__nv_bfloat16*)out, (size_t)n, kind, bias, bias_dtype, width);
    else
        MLS_LAUNCH((unary_act_kernel<float, float>), dim3(blocks), dim3(256), 0, stream,
                   (const float*)in, (float*)out, (size_t)n, kind, bias, bias_dtype, width);
    return launch_status();
}

// x[i] = cap * tanh(x[i] / cap) on float32 values (capped logits).
MLS_API int mls_softcap_f32(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return MLS_ERR_UNSUPPORTED;
    const long long want = (n + 255) / 256;
    const int blocks = (int)(want < 16LL * sm_count() ? want : 16LL * sm_count());
    MLS_LAUNCH((softcap_f32_kernel), dim3(blocks), dim3(256), 0, stream, x, (size_t)n, cap);
    return launch_status();
}

// x[i] *= scale on float32 values (logits times a constant).
MLS_API int mls_scale_f32(float* x, long long n, float scale, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long want = (n + 255) / 256;
    const int blocks = (int)(want < 16LL * sm_count() ? want : 16LL * sm_count());
    MLS_LAUNCH((scale_f32_kernel), dim3(blocks), dim3(256), 0, stream, x, (size_t)n, scale);
    return launch_status();
}

// gu: [T, 2*I], a row holds [gate | up]; out[t, i] = clamped_glu(gate, up).
MLS_API int mls_clamped_glu(const void* gu, void* out, int dtype, int n_tokens, int inter,
                            float alpha, float limit, cudaStream_t stream) {
    if (n_tokens <= 0 || inter <= 0) return 0;
    const int threads = 256;
    dim3 grid((inter + threads - 1) / threads, n_tokens);
    if (dtype == MLS_BF16)
        MLS_LAUNCH((clamped_glu_kernel<__nv_bfloat16>), dim3(grid), dim3(threads), 0, stream,
                   (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, alpha, limit);
    else
        MLS_LAUNCH((clamped_glu_kernel<float>), dim3(grid), dim3(threads), 0, stream,
                   (const float*)gu, (float*)out, inter, alpha, limit);
    return launch_status();
}

MLS_API int mls_swiglu(const void* gu, void* out, int dtype, int n_tokens, int inter,
                       cudaStream_t stream) {
    if (n_tokens <= 0 || inter <= 0) return 0;
    const int threads = 256;
    if (dtype == MLS_BF16 && inter % 8 == 0) {
        dim3 grid((inter / 8 + threads - 1) / threads, n_tokens);
        MLS_LAUNCH((swiglu_bf16x8_kernel), dim3(grid), dim3(threads), 0, stream,
                   (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter);
    } else if (dtype == MLS_F32 && inter % 4 == 0) {
        dim3 grid((inter / 4 + threads - 1) / threads, n_tokens);
        MLS_LAUNCH((swiglu_f32x4_kernel), dim3(grid), dim3(threads), 0, stream, (const float*)gu,
                   (float*)out, inter);
    } else {
        dim3 grid((inter + threads - 1) / threads, n_tokens);
        if (dtype == MLS_BF16)
            MLS_LAUNCH((swiglu_kernel<__nv_bfloat16>), dim3(grid), dim3(threads), 0, stream,
                       (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter);
        else
            MLS_LAUNCH((swiglu_kernel<float>), dim3(grid), dim3(threads), 0, stream,
                       (const float*)gu, (float*)out, inter);
    }
    return launch_status();
}
