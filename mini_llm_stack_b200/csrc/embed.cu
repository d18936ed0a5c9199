// Token embedding: x[t, :] = E[token[t], :], widened to the float32 residual
// stream, times a constant (1 in the reference, which has no scaling and no position
// term: train/model.py:224,239).  With frequencies (float64, one a pair of entries) a
// sinusoidal position vector is added: entry 2i gets sin(position * freq[i]), entry 2i + 1 the
// cosine of the same angle (the angle in float64, reduced to [-pi, pi] before the functions).
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ x, int d, int vocab, float scale, int* status,
                             const int* __restrict__ positions, const double* __restrict__ freq) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    bool bad = id < 0 || id >= vocab;
    if (bad) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLS_STATUS_BAD_TOKEN);
    }
    const T* row = table + (size_t)(bad ? 0 : id) * d;
    float* out = x + (size_t)t * d;
    if (!freq) {
        for (int i = threadIdx.x; i < d; i += blockDim.x)
            out[i] = bad ? 0.f : Elem<T>::load(row + i) * scale;
        return;
    }
    const int p = positions[t];
    for (int pair = threadIdx.x; 2 * pair < d; pair += blockDim.x) {
        float c, s;
        angle_cos_sin(p, freq[pair], c, s);
        const int i = 2 * pair;
        out[i] = bad ? 0.f : Elem<T>::load(row + i) * scale + s;
        if (i + 1 < d) out[i + 1] = bad ? 0.f : Elem<T>::load(row + i + 1) * scale + c;
    }
}

MLS_API int mls_embed(const int* ids, const void* table, int table_dtype, float* x,
                      int n_tokens, int d, int vocab, float scale, int* status,
                      const int* positions, const double* freq, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    int threads = d >= 1024 ? 256 : (d >= 256 ? 128 : 64);
    if (table_dtype == MLS_BF16)
        MLS_LAUNCH((embed_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(threads), 0, stream, ids,
                   (const __nv_bfloat16*)table, x, d, vocab, scale, status, positions, freq);
    else
        MLS_LAUNCH((embed_kernel<float>), dim3(n_tokens), dim3(threads), 0, stream, ids,
                   (const float*)table, x, d, vocab, scale, status, positions, freq);
    return launch_status();
}
