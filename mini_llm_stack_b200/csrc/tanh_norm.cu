// The norm without statistics: n(v) = tanh(alpha * v) * w + b, element by element, with a
// scalar alpha and vectors w, b.  Because nothing is reduced over the row, a block that puts
// such a norm behind a sublayer as well (x <- x + s * n_post(y), s a per-channel scale) needs
// no pass of its own for it: the kernel that adds the sublayer's output to the residual stream
// and applies the next norm does all of it while it reads the row once.
//
// mls_add_tanh_norm, for every output row i (source row t = rows ? rows[i] : i):
//   y = sum of the delta's parts at row t (+ delta_bias)        (delta may be absent)
//   if post_w:  y = (tanh(post_alpha * y) * post_w + post_b) * post_scale   (scale optional)
//   v = x[t] + y;  without `rows`, x[t] = v                     (x may be absent: v = y)
//   h[i] = tanh(alpha * v) * w + b                              (h may be absent)
//   y_out[i] = y                                                (y_out may be absent)
// Everything is float32 inside (tanhf, not an approximation), one rounding at the store of h.
#include "common.cuh"

namespace {
struct TanhNormArgs {
    float* x;                      // [T, d] float32 residual stream, or nullptr
    const void* delta;             // [parts][T, d], or nullptr
    int delta_dtype, n_parts;
    long long part_stride;
    const void* delta_bias;        // [d] or nullptr
    float post_alpha;
    const void* post_w;            // [d] or nullptr: no map on the delta
    const void* post_b;
    const void* post_scale;        // [d] or nullptr
    float alpha;
    const void* w;                 // [d]
    const void* b;
    int vec_dtype;                 // type of every vector above
    void* h;                       // [n_out, d] or nullptr
    int h_dtype;
    float* y_out;                  // [n_out, d] float32 or nullptr
    const int* rows;               // [n_out] or nullptr
    int n_out, d;
};

__device__ __forceinline__ float delta_at(const TanhNormArgs& a, size_t at) {
    float y = 0.f;
    if (a.delta) {
        if (a.delta_dtype == MLS_BF16) {
            y = __bfloat162float(((const __nv_bfloat16*)a.delta)[at]);
        } else {
            const float* p = (const float*)a.delta + at;
            for (int k = 0; k < a.n_parts; ++k) y += p[(size_t)k * a.part_stride];
        }
    }
    return y;
}

__global__ void __launch_bounds__(256) add_tanh_norm_kernel(const TanhNormArgs a) {
    chain_release();
    chain_wait();
    const size_t n = (size_t)a.n_out * a.d;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int i = (int)(idx / a.d), c = (int)(idx - (size_t)i * a.d);
        const int t = a.rows ? a.rows[i] : i;
        const size_t at = (size_t)t * a.d + c;
        float y = delta_at(a, at);
        if (a.delta_bias) y += load_as_float(a.delta_bias, c, a.vec_dtype);
        if (a.post_w) {
            y = tanhf(a.post_alpha * y) * load_as_float(a.post_w, c, a.vec_dtype) +
                load_as_float(a.post_b, c, a.vec_dtype);
            if (a.post_scale) y *= load_as_float(a.post_scale, c, a.vec_dtype);
        }
        float v = y;
        if (a.x) {
            v = a.x[at] + y;
            if (!a.rows) a.x[at] = v;
        }
        if (a.h)
            store_from_float(a.h, idx, a.h_dtype,
                             tanhf(a.alpha * v) * load_as_float(a.w, c, a.vec_dtype) +
                                 load_as_float(a.b, c, a.vec_dtype));
        if (a.y_out) a.y_out[idx] = y;
    }
}

// Four consecutive channels a thread (d a multiple of four): 16-byte loads of the stream and of
// float32 parts, 8-byte loads of bfloat16 rows and vectors.
__device__ __forceinline__ void load4(const void* base, size_t i, int dtype, float (&o)[4]) {
    if (dtype == MLS_BF16) {
        const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)base + i);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 lo = __bfloat1622float2(h2[0]), hi = __bfloat1622float2(h2[1]);
        o[0] = lo.x; o[1] = lo.y; o[2] = hi.x; o[3] = hi.y;
    } else {
        const float4 v = *reinterpret_cast<const float4*>((const float*)base + i);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
}

__global__ void __launch_bounds__(256) add_tanh_norm_kernel4(const TanhNormArgs a) {
    chain_release();
    // the vectors are written by no kernel of a step: they may be fetched before the wait
    const int d4 = a.d / 4;
    const size_t n = (size_t)a.n_out * d4;
    chain_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int i = (int)(idx / d4), c = (int)(idx - (size_t)i * d4) * 4;
        const int t = a.rows ? a.rows[i] : i;
        const size_t at = (size_t)t * a.d + c;
        float y[4] = {0.f, 0.f, 0.f, 0.f};
        if (a.delta) {
            if (a.delta_dtype == MLS_BF16) {
                load4(a.delta, at, MLS_BF16, y);
            } else {
                // four parts' loads under way at a time; the additions keep the parts' order
                int k = 0;
                for (; k + 4 <= a.n_parts; k += 4) {
                    float p[4][4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        load4(a.delta, (size_t)(k + j) * a.part_stride + at, MLS_F32, p[j]);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int e = 0; e < 4; ++e) y[e] += p[j][e];
                }
                for (; k < a.n_parts; ++k) {
                    float p[4];
                    load4(a.delta, (size_t)k * a.part_stride + at, MLS_F32, p);
#pragma unroll
                    for (int e = 0; e < 4; ++e) y[e] += p[e];
                }
            }
        }
        if (a.delta_bias) {
            float p[4];
            load4(a.delta_bias, c, a.vec_dtype, p);
#pragma unroll
            for (int e = 0; e < 4; ++e) y[e] += p[e];
        }
        if (a.post_w) {
            float pw[4], pb[4];
            load4(a.post_w, c, a.vec_dtype, pw);
            load4(a.post_b, c, a.vec_dtype, pb);
#pragma unroll
            for (int e = 0; e < 4; ++e) y[e] = tanhf(a.post_alpha * y[e]) * pw[e] + pb[e];
            if (a.post_scale) {
                float ps[4];
                load4(a.post_scale, c, a.vec_dtype, ps);
#pragma unroll
                for (int e = 0; e < 4; ++e) y[e] *= ps[e];
            }
        }
        float v[4] = {y[0], y[1], y[2], y[3]};
        if (a.x) {
            float xv[4];
            load4(a.x, at, MLS_F32, xv);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = xv[e] + y[e];
            if (!a.rows) *reinterpret_cast<float4*>(a.x + at) = make_float4(v[0], v[1], v[2], v[3]);
        }
        if (a.h) {
            float w[4], b[4], o[4];
            load4(a.w, c, a.vec_dtype, w);
            load4(a.b, c, a.vec_dtype, b);
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = tanhf(a.alpha * v[e]) * w[e] + b[e];
            const size_t out_at = (size_t)i * a.d + c;
            if (a.h_dtype == MLS_BF16) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]);
                __nv_bfloat162 hi = __floats2bfloat162_rn(o[2], o[3]);
                uint2 raw;
                raw.x = *reinterpret_cast<uint32_t*>(&lo);
                raw.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>((__nv_bfloat16*)a.h + out_at) = raw;
            } else {
                *reinterpret_cast<float4*>((float*)a.h + out_at) = make_float4(o[0], o[1], o[2], o[3]);
            }
        }
        if (a.y_out)
            *reinterpret_cast<float4*>(a.y_out + (size_t)i * a.d + c) = make_float4(y[0], y[1], y[2], y[3]);
    }
}
}  // namespace

MLS_API int mls_add_tanh_norm(float* x, const void* delta, int delta_dtype, int n_parts,
                              long long part_stride, const void* delta_bias, float post_alpha,
                              const void* post_w, const void* post_b, const void* post_scale,
                              float alpha, const void* w, const void* b, int vec_dtype, void* h,
                              int h_dtype, float* y_out, const int* rows, int n_out, int d,
                              cudaStream_t stream) {
    if (n_out <= 0 || d <= 0) return 0;
    if ((h && (!w || !b)) || (post_w && !post_b) || (delta && n_parts < 1)) return MLS_ERR_UNSUPPORTED;
    TanhNormArgs a;
    a.x = x; a.delta = delta; a.delta_dtype = delta_dtype; a.n_parts = n_parts;
    a.part_stride = part_stride; a.delta_bias = delta_bias; a.post_alpha = post_alpha;
    a.post_w = post_w; a.post_b = post_b; a.post_scale = post_scale; a.alpha = alpha; a.w = w;
    a.b = b; a.vec_dtype = vec_dtype; a.h = h; a.h_dtype = h_dtype; a.y_out = y_out; a.rows = rows;
    a.n_out = n_out; a.d = d;
    // four channels a thread only where every row and vector starts at a 16-byte address
    uintptr_t bits = 0;
    for (const void* p : {(const void*)x, delta, delta_bias, post_w, post_b, post_scale, w, b,
                          (const void*)h, (const void*)y_out})
        bits |= reinterpret_cast<uintptr_t>(p);
    const bool by4 = d % 4 == 0 && part_stride % 4 == 0 && bits % 16 == 0;
    const size_t n = (size_t)n_out * (by4 ? d / 4 : d);
    const size_t want = (n + 255) / 256;
    const int blocks = (int)(want < (size_t)(8 * sm_count()) ? want : 8 * sm_count());
    if (by4)
        MLS_LAUNCH((add_tanh_norm_kernel4), dim3(blocks), dim3(256), 0, stream, a);
    else
        MLS_LAUNCH((add_tanh_norm_kernel), dim3(blocks), dim3(256), 0, stream, a);
    return launch_status();
}
