// Latent attention: the normalised latents of a step, and the per-head products that
// let attention run over the cached latent itself.
//
// A token caches one latent c [r] (r = latent size): every head's key is W_uk[h] c and
// its value W_uv[h] c.  Then  q_h . k_h = (W_uk[h]^T q_h) . c  and
// sum_j p_j v_hj = W_uv[h] (sum_j p_j c_j):  with the query taken into the latent space
// first and the result taken out of it afterwards, attention is multi-query attention
// with the latent as the single key AND value head, and the paged kernels run on the
// latent pool as it is.  Nothing but c is cached and no key or value is rebuilt.
//
// mls_latent_norm_store: down [T, rq + r] float32 (the two down projections side by
//   side).  cq[t] = unit_rms(down[t, :rq]) * wq  (skipped if rq == 0);
//   c = unit_rms(down[t, rq:]) * wkv goes to the pool at slot_map[t], zero-padded to
//   the pool's row width rp >= r; the rest of a page the request enters is cleared.
//   unit_rms(v) = v / sqrt(mean(v^2) + eps), float32 with one rounding at the store.
//
// mls_headwise_linear: out[t, h, n] = sum_k in[t, h, k] * W[h, n, k] for every head h
//   (W [H, N, K], K contiguous), rows and heads of in / out at given strides; float32
//   accumulation over k ascending, whatever T is: a token's result does not depend on
//   its batch.
//
// mls_latent_rope_prep: the variant whose heads carry, beside the part that meets the latent,
//   a rotated part that meets one rotated key part shared by all heads: the cached row is
//   [latent | rotated key part], a query row [W_uk^T q_plain | rotated q part], and the same
//   multi-query attention runs over rows of that width; its result's first r entries are the
//   weighted latent.  mls_sigmoid_gate: the heads' outputs times sigmoid(gate).
#include "common.cuh"
#include "page_tail.cuh"

namespace {
constexpr int LT_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(LT_THREADS)
latent_norm_store_kernel(const float* __restrict__ down, int rq, int r, int rp,
                         const void* __restrict__ wq, const void* __restrict__ wkv, int w_dtype,
                         float eps, T* __restrict__ cq, const int* __restrict__ slot_map,
                         T* __restrict__ pool, int block_size, int pool_slots, int* status) {
    chain_release();
    chain_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const float* row = down + (size_t)t * (rq + r);
    if (rq > 0) {
        float s = 0.f;
        for (int c = threadIdx.x; c < rq; c += LT_THREADS) s = fmaf(row[c], row[c], s);
        const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)rq + eps);
        for (int c = threadIdx.x; c < rq; c += LT_THREADS)
            Elem<T>::store(cq + (size_t)t * rq + c, row[c] * inv * load_as_float(wq, c, w_dtype));
    }
    const int slot = slot_map[t];
    const bool slot_ok = slot >= 0 && slot < pool_slots;
    if (!slot_ok && threadIdx.x == 0 && status) atomicOr(status, MLS_STATUS_BAD_SLOT);
    float s = 0.f;
    for (int c = threadIdx.x; c < r; c += LT_THREADS) s = fmaf(row[rq + c], row[rq + c], s);
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)r + eps);
    if (!slot_ok) return;
    T* dst = pool + (size_t)slot * rp;
    for (int c = threadIdx.x; c < rp; c += LT_THREADS)
        Elem<T>::store(dst + c, c < r ? row[rq + c] * inv * load_as_float(wkv, c, w_dtype) : 0.f);
    clear_page_tail<T>(page_tail_to_clear(slot_map, t, gridDim.x, slot, block_size), slot,
                       block_size, pool_slots / block_size, 1, rp, pool, pool);
}


// Values of a projection's row that may still lie in the parts of a cut along K.  The parts'
// loads go out B at a time (a lone block of a decode step would otherwise wait for one part
// after the other); the additions keep the parts' order.
template <int B, typename V, typename Ld, typename Add>
__device__ __forceinline__ void add_parts(V& v, int& k, int n, Ld ld, Add add) {
    for (; k + B <= n; k += B) {
        V w[B];
#pragma unroll
        for (int i = 0; i < B; ++i) w[i] = ld(k + i);
#pragma unroll
        for (int i = 0; i < B; ++i) add(v, w[i]);
    }
}
struct RowParts {
    const float* base;             // [n_parts][T, width]
    int n_parts;
    long long part_stride;
    int width;
    __device__ __forceinline__ float at(int t, int col) const {
        const float* p = base + (size_t)t * width + col;
        if (n_parts == 1) return *p;
        float v = 0.f;
        int k = 0;
        auto ld = [&](int i) { return p[(size_t)i * part_stride]; };
        auto add = [](float& a, float b) { a += b; };
        add_parts<8>(v, k, n_parts, ld, add);
        add_parts<4>(v, k, n_parts, ld, add);
        add_parts<1>(v, k, n_parts, ld, add);
        return v;
    }
};

// Entry i of a vector of n entries whose first `dims` turn, entry j with entry j + dims/2
// (j < dims/2), by the token's angle j, whose cosine is cs[j] and sine cs[dims/2 + j]; the
// others pass.  get(j) reads entry j.
template <typename Get>
__device__ __forceinline__ float rotated_entry(Get get, int i, int dims,
                                               const float* __restrict__ cs) {
    const int half = dims >> 1;
    if (i >= dims) return get(i);
    const int j = i < half ? i : i - half;
    const float c = cs[j], s = cs[half + j];
    const float u = get(j), v = get(j + half);
    return i < half ? u * c - v * s : v * c + u * s;
}

// Four neighbouring float32 entries of a projection row (summed over its parts), and four
// values stored side by side in the activations' type.
__device__ __forceinline__ float4 row_parts_at4(const RowParts& proj, int t, int col) {
    const float* p = proj.base + (size_t)t * proj.width + col;
    if (proj.n_parts == 1) return *reinterpret_cast<const float4*>(p);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    int k = 0;
    auto ld = [&](int i) {
        return *reinterpret_cast<const float4*>(p + (size_t)i * proj.part_stride);
    };
    auto add = [](float4& a, const float4& b) {
        a.x += b.x;
        a.y += b.y;
        a.z += b.z;
        a.w += b.w;
    };
    add_parts<8>(v, k, proj.n_parts, ld, add);
    add_parts<4>(v, k, proj.n_parts, ld, add);
    add_parts<1>(v, k, proj.n_parts, ld, add);
    return v;
}
__device__ __forceinline__ void store4(float* dst, float4 v) {
    *reinterpret_cast<float4*>(dst) = v;
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const unsigned*>(&lo);
    u.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(dst) = u;
}

// One block a token.  From the float32 projection row [q heads (e plain | g turned) ... |
// r + g down-projected entries]:
//   q_plain[t, h, :e]                    the plain part of every head, as it is
//   q_in[t, h * rp + r + i]              the turned part of every head, rotated (i < g);
//                                        q_in[t, h * rp + r + g ..] = 0 up to rp
//   pool[slot] = [unit_rms(down[:r]) * w | rotate(down[r : r + g]) | 0 ...]   (has_kv only)
// and the rest of a page the request enters is cleared.  The token's dims/2 angles are taken
// once (the product with the position and its reduction are float64) and kept in shared
// memory as cos | sin.  by4: every column offset and width is a multiple of four and the
// buffers start at 16-byte addresses, so the plain parts move four entries at a time.
// staged: the entries that are turned or normed (every head's g and the r + g of the down
// projection) are first brought into shared memory, all loads under way at once, and the
// rest of the kernel reads them there; without it (a row too long for shared memory) every
// entry is read where it is used.  kv4: the down-projected entries also move by fours.  The
// latent norm's weight waits there too, read before the wait on the kernel ahead.
template <typename T>
__global__ void __launch_bounds__(LT_THREADS)
latent_rope_prep_kernel(const RowParts proj, int q_col, int kv_col, int n_heads, int e, int g,
                        int r, int rp, int rot_dims, const double* __restrict__ freq,
                        const int* __restrict__ positions, const void* __restrict__ wkv,
                        int w_dtype, float eps, T* __restrict__ q_plain, T* __restrict__ q_in,
                        int q_in_width, int has_kv, const int* __restrict__ slot_map,
                        T* __restrict__ pool, int block_size, int pool_slots, int by4, int kv4,
                        int staged, int* status) {
    chain_release();
    extern __shared__ __align__(16) float cs[];      // [rot_dims]: cos | sin, then the staged entries
    float* sq = cs + ((rot_dims + 3) & ~3);          // [n_heads, g]
    float* skv = sq + n_heads * g;                   // [r + g]
    float* swn = skv + r + g;                        // [r]: the latent norm's weight
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int slot = has_kv ? slot_map[t] : -1;
    const int tail = has_kv ? page_tail_to_clear(slot_map, t, gridDim.x, slot, block_size) : 0;
    for (int j = threadIdx.x; j < (rot_dims >> 1); j += LT_THREADS)
        angle_cos_sin(pos, freq[j], cs[j], cs[(rot_dims >> 1) + j]);
    // weights are no result of the kernel before: they may be read ahead of the wait
    if (staged && has_kv)
        for (int c = threadIdx.x; c < r; c += LT_THREADS) swn[c] = load_as_float(wkv, c, w_dtype);
    chain_wait();
    const int hw = e + g;
    if (staged) {
        if (by4) {
            const int g4 = g >> 2;
#pragma unroll 4
            for (int u = threadIdx.x; u < n_heads * g4; u += LT_THREADS) {
                const int h = u / g4, i = (u - h * g4) << 2;
                store4(sq + h * g + i, row_parts_at4(proj, t, q_col + h * hw + e + i));
            }
        } else {
#pragma unroll 4
            for (int u = threadIdx.x; u < n_heads * g; u += LT_THREADS) {
                const int h = u / g, i = u - h * g;
                sq[u] = proj.at(t, q_col + h * hw + e + i);
            }
        }
        if (has_kv && kv4) {
#pragma unroll 2
            for (int c = threadIdx.x * 4; c < r + g; c += LT_THREADS * 4)
                store4(skv + c, row_parts_at4(proj, t, kv_col + c));
        } else if (has_kv) {
#pragma unroll 4
            for (int c = threadIdx.x; c < r + g; c += LT_THREADS) skv[c] = proj.at(t, kv_col + c);
        }
    }
    __shared__ float scratch[33];
    if (by4) {
        const int e4 = e >> 2;
#pragma unroll 2
        for (int u = threadIdx.x; u < n_heads * e4; u += LT_THREADS) {
            const int h = u / e4, i = (u - h * e4) << 2;
            store4(q_plain + (size_t)t * n_heads * e + h * e + i,
                   row_parts_at4(proj, t, q_col + h * hw + i));
        }
    } else {
        for (int u = threadIdx.x; u < n_heads * e; u += LT_THREADS) {
            const int h = u / e, i = u - h * e;
            Elem<T>::store(q_plain + (size_t)t * n_heads * e + u, proj.at(t, q_col + h * hw + i));
        }
    }
    __syncthreads();
    const int turned = rp - r;                       // g rotated entries, then zeros
    for (int u = threadIdx.x; u < n_heads * turned; u += LT_THREADS) {
        const int h = u / turned, i = u - h * turned;
        float v = 0.f;
        if (i < g)
            v = rotated_entry(
                [&](int j) { return staged ? sq[h * g + j] : proj.at(t, q_col + h * hw + e + j); },
                i, rot_dims, cs);
        Elem<T>::store(q_in + (size_t)t * q_in_width + (size_t)h * rp + r + i, v);
    }
    if (!has_kv) return;
    const bool slot_ok = slot >= 0 && slot < pool_slots;
    if (!slot_ok && threadIdx.x == 0 && status) atomicOr(status, MLS_STATUS_BAD_SLOT);
    auto down = [&](int c) { return staged ? skv[c] : proj.at(t, kv_col + c); };
    float s = 0.f;
    for (int c = threadIdx.x; c < r; c += LT_THREADS) {
        const float v = down(c);
        s = fmaf(v, v, s);
    }
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)r + eps);
    if (!slot_ok) return;
    T* dst = pool + (size_t)slot * rp;
    for (int c = threadIdx.x; c < rp; c += LT_THREADS) {
        float v = 0.f;
        if (c < r)
            v = down(c) * inv * (staged ? swn[c] : load_as_float(wkv, c, w_dtype));
        else if (c < r + g)
            v = rotated_entry([&](int j) { return down(r + j); }, c - r, rot_dims, cs);
        Elem<T>::store(dst + c, v);
    }
    clear_page_tail<T>(tail, slot, block_size, pool_slots / block_size, 1, rp, pool, pool);
}

// o[t, c] *= sigmoid(gate[t, gate_col + c]), the gate read from a float32 projection row.
// by4: four entries a thread where widths and offsets are multiples of four.
__device__ __forceinline__ float4 load4(const float* src) {
    return *reinterpret_cast<const float4*>(src);
}
__device__ __forceinline__ float4 load4(const __nv_bfloat16* src) {
    const uint2 u = *reinterpret_cast<const uint2*>(src);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* __restrict__ o, const RowParts proj, int gate_col, int n_tokens, int n,
                    int by4) {
    chain_release();
    chain_wait();
    if (by4) {
        const int n4 = n >> 2;
        const size_t total = (size_t)n_tokens * n4;
        for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
             idx += (size_t)gridDim.x * blockDim.x) {
            const int t = (int)(idx / n4), c = (int)(idx - (size_t)t * n4) << 2;
            const float4 z = row_parts_at4(proj, t, gate_col + c);
            T* at = o + (size_t)t * n + c;
            float4 v = load4(at);
            v.x = v.x / (1.0f + expf(-z.x));
            v.y = v.y / (1.0f + expf(-z.y));
            v.z = v.z / (1.0f + expf(-z.z));
            v.w = v.w / (1.0f + expf(-z.w));
            store4(at, v);
        }
        return;
    }
    const size_t total = (size_t)n_tokens * n;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / n), c = (int)(idx - (size_t)t * n);
        const float z = proj.at(t, gate_col + c);
        Elem<T>::store(o + idx, Elem<T>::load(o + idx) / (1.0f + expf(-z)));
    }
}

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads

template <typename T>
__global__ void __launch_bounds__(256)
headwise_linear_kernel(const T* __restrict__ in, long long in_row, long long in_head,
                       const T* __restrict__ W, T* __restrict__ out, long long out_row,
                       long long out_head, int M, int N, int K) {
    chain_release();
    chain_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x, head = blockIdx.z;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const T* A = in + (size_t)head * in_head;
    const T* Wh = W + (size_t)head * N * K;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + e][lrow] = (am < M && k < K) ? Elem<T>::load(A + (size_t)am * in_row + k) : 0.f;
            Ws[lk + e][lrow] = (wn < N && k < K) ? Elem<T>::load(Wh + (size_t)wn * K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
    T* O = out + (size_t)head * out_head;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) Elem<T>::store(O + (size_t)m * out_row + n, acc[i][j]);
        }
    }
}
}  // namespace

MLS_API int mls_latent_norm_store(const float* down, int n_tokens, int rq, int r, int rp,
                                  const void* wq, const void* wkv, int w_dtype, float eps,
                                  void* cq, int dtype, const int* slot_map, void* pool,
                                  int block_size, long long pool_slots, int* status,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (r <= 0 || rp < r || rq < 0 || block_size <= 0) return MLS_ERR_UNSUPPORTED;
    if (dtype == MLS_BF16)
        MLS_LAUNCH((latent_norm_store_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(LT_THREADS), 0,
                   stream, down, rq, r, rp, wq, wkv, w_dtype, eps, (__nv_bfloat16*)cq, slot_map,
                   (__nv_bfloat16*)pool, block_size, (int)pool_slots, status);
    else
        MLS_LAUNCH((latent_norm_store_kernel<float>), dim3(n_tokens), dim3(LT_THREADS), 0, stream,
                   down, rq, r, rp, wq, wkv, w_dtype, eps, (float*)cq, slot_map, (float*)pool,
                   block_size, (int)pool_slots, status);
    return launch_status();
}

MLS_API int mls_headwise_linear(const void* in, long long in_row, long long in_head,
                                const void* W, void* out, long long out_row, long long out_head,
                                int dtype, int n_tokens, int n_heads, int N, int K,
                                cudaStream_t stream) {
    if (n_tokens <= 0 || n_heads <= 0 || N <= 0) return 0;
    if (n_heads > 65535) return MLS_ERR_UNSUPPORTED;
    dim3 grid((N + BN - 1) / BN, (n_tokens + BM - 1) / BM, n_heads);
    if (dtype == MLS_BF16)
        MLS_LAUNCH((headwise_linear_kernel<__nv_bfloat16>), dim3(grid), dim3(256), 0, stream,
                   (const __nv_bfloat16*)in, in_row, in_head, (const __nv_bfloat16*)W,
                   (__nv_bfloat16*)out, out_row, out_head, n_tokens, N, K);
    else
        MLS_LAUNCH((headwise_linear_kernel<float>), dim3(grid), dim3(256), 0, stream,
                   (const float*)in, in_row, in_head, (const float*)W, (float*)out, out_row,
                   out_head, n_tokens, N, K);
    return launch_status();
}

MLS_API int mls_latent_rope_prep(const float* proj, int n_parts, long long part_stride,
                                 int proj_width, int q_col, int kv_col, int n_tokens, int n_heads,
                                 int e, int g, int r, int rp, int rot_dims, const double* freq,
                                 const int* positions, const void* wkv, int w_dtype, float eps,
                                 void* q_plain, void* q_in, int q_in_width, int dtype, int has_kv,
                                 const int* slot_map, void* pool, int block_size,
                                 long long pool_slots, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (r <= 0 || g < 0 || rp < r + g || e < 0 || n_heads <= 0 || n_parts < 1 || rot_dims < 0 ||
        rot_dims > g || (rot_dims & 1) || (rot_dims > 0 && !freq) || (has_kv && block_size <= 0))
        return MLS_ERR_UNSUPPORTED;
    const RowParts rows{proj, n_parts, part_stride, proj_width};
    // cos | sin, then (where they fit) every head's turned entries, the down projection's and
    // the latent norm's weight
    const size_t angles = ((size_t)rot_dims + 3) & ~(size_t)3;
    const size_t stage = (size_t)n_heads * g + (has_kv ? (size_t)2 * r + g : 0);
    const int staged = (angles + stage) * sizeof(float) <= 40 * 1024;
    const size_t smem = (angles + (staged ? stage : 0)) * sizeof(float);
    if (smem > 40 * 1024) return MLS_ERR_UNSUPPORTED;
    const int by4 = e % 4 == 0 && g % 4 == 0 && q_col % 4 == 0 && proj_width % 4 == 0 &&
                    part_stride % 4 == 0 && reinterpret_cast<uintptr_t>(proj) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(q_plain) % 16 == 0;
    const int kv4 = g % 4 == 0 && r % 4 == 0 && kv_col % 4 == 0 && (n_heads * g) % 4 == 0 &&
                    proj_width % 4 == 0 && part_stride % 4 == 0 &&
                    reinterpret_cast<uintptr_t>(proj) % 16 == 0;
    if (dtype == MLS_BF16)
        MLS_LAUNCH((latent_rope_prep_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(LT_THREADS), smem,
                   stream, rows, q_col, kv_col, n_heads, e, g, r, rp, rot_dims, freq, positions, wkv,
                   w_dtype, eps, (__nv_bfloat16*)q_plain, (__nv_bfloat16*)q_in, q_in_width, has_kv,
                   slot_map, (__nv_bfloat16*)pool, block_size, (int)pool_slots, by4, kv4, staged,
                   status);
    else
        MLS_LAUNCH((latent_rope_prep_kernel<float>), dim3(n_tokens), dim3(LT_THREADS), smem, stream,
                   rows, q_col, kv_col, n_heads, e, g, r, rp, rot_dims, freq, positions, wkv, w_dtype,
                   eps, (float*)q_plain, (float*)q_in, q_in_width, has_kv, slot_map, (float*)pool,
                   block_size, (int)pool_slots, by4, kv4, staged, status);
    return launch_status();
}

MLS_API int mls_sigmoid_gate(void* o, int dtype, const float* proj, int n_parts,
                             long long part_stride, int proj_width, int gate_col, int n_tokens,
                             int n, cudaStream_t stream) {
    if (n_tokens <= 0 || n <= 0) return 0;
    if (n_parts < 1) return MLS_ERR_UNSUPPORTED;
    const RowParts rows{proj, n_parts, part_stride, proj_width};
    const int by4 = n % 4 == 0 && gate_col % 4 == 0 && proj_width % 4 == 0 && part_stride % 4 == 0 &&
                    reinterpret_cast<uintptr_t>(proj) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(o) % 16 == 0;
    const size_t want = ((size_t)n_tokens * (by4 ? n / 4 : n) + 255) / 256;
    const int blocks = (int)(want < (size_t)(8 * sm_count()) ? want : 8 * sm_count());
    if (dtype == MLS_BF16)
        MLS_LAUNCH((sigmoid_gate_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream,
                   (__nv_bfloat16*)o, rows, gate_col, n_tokens, n, by4);
    else
        MLS_LAUNCH((sigmoid_gate_kernel<float>), dim3(blocks), dim3(256), 0, stream, (float*)o, rows,
                   gate_col, n_tokens, n, by4);
    return launch_status();
}
