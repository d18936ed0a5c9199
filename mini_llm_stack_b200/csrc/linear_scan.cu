// Linear recurrences over a matrix state per head, carried from token to token in a
// float32 state slot per request, and what surrounds them.
//
// Per head, with key size e and value size f, the state S is [e, f] and one token does
//
//   read first  (a bonus u on the current token, a decay per key channel and token):
//       o_j = sum_i a_i (S_ij + u_i k_i v_j);   S_ij <- w_i S_ij + k_i v_j
//   write first (one fixed decay a head):
//       S_ij <- g S_ij + k_i v_j;               o_j = sum_i a_i S_ij
//
// with a the "receptance" or query.  mls_linear_scan walks the tokens of every request of
// the step in order, from the state the slot holds, and leaves o [T, H*f] in float32; the
// state goes back to the slot.  A CTA owns 16 columns of one head's S for one request:
// thread (column, row group) keeps every eighth row of its column in registers, a warp holds
// four columns times eight row groups, and the sum over i is the thread's rows in order
// followed by three shuffles: the order never depends on the batch or on how the tokens
// were cut into steps.  Tokens are taken 16 or 32 at a time through shared memory, four of
// them side by side where only the state's own update has to wait for the token before.
//
//   mls_scan_finish      o / rms(o) per head (eps inside the root) * weight * silu(gate)
//   mls_scan_finish_row  o / rms(o) over a token's whole row of heads * weight * sigmoid(gate)
//                        * a constant, into rows that may be wider than the heads
//   mls_rotate_rows      rotation of the first `dims` entries of every head of q and k,
//                        entry i paired with i + dims/2, k then times a constant; float32 out
//   mls_decay_lowrank    w = exp(-exp(W2 tanh(lo) + w0)) from the low-rank pre-activation
//                        (W2 handed over transposed)
//
// State, decays, exponentials, angles' cosines and sines, norms and sums are float32 (the
// angles themselves float64: position * frequency); a, k, v come from the projections, with
// `act` = 1 through silu (z * sigmoid(z), float32) as they are loaded.
#include "common.cuh"

namespace {
constexpr int LS_COLS = 16;         // columns of S a CTA owns
constexpr int LS_GROUPS = 8;        // row groups: lanes that share a column
constexpr int LS_THREADS = LS_COLS * LS_GROUPS;
constexpr int LS_UNROLL = 4;        // tokens whose sums over the row groups run side by side

// Four consecutive entries of a row as floats (the index a multiple of four, the row's start
// aligned to 16 bytes).
__device__ __forceinline__ float4 load4(const void* base, int dtype, size_t i) {
    if (dtype == MLS_BF16) {
        const uint2 raw = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)base + i);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(lo.x, lo.y, hi.x, hi.y);
    }
    return *reinterpret_cast<const float4*>((const float*)base + i);
}

__device__ __forceinline__ float silu1(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float4 silu4(float4 v) {
    return make_float4(silu1(v.x), silu1(v.y), silu1(v.z), silu1(v.w));
}

// (Four CTAs an SM up to 16 rows a thread: 592 places, so that the 512 CTAs of 32 heads with
// 256 value columns are one round and not two.)
template <int RPT, bool TOK_DECAY>
__global__ void __launch_bounds__(LS_THREADS, RPT <= 16 ? 4 : 2)
linear_scan_kernel(const void* __restrict__ a_src, int a_dtype, int a_row, int a_off,
                   const void* __restrict__ k_src, int k_dtype, int k_row, int k_off,
                   const void* __restrict__ v_src, int v_dtype, int v_row, int v_off,
                   const float* __restrict__ decay_tok, int decay_row,
                   const float* __restrict__ decay_head,
                   const void* __restrict__ bonus, int bonus_dtype, int read_first,
                   const int* __restrict__ cu_q, const int* __restrict__ state_slot,
                   float* __restrict__ state, long long state_stride,
                   int n_heads, int e, int f, int tokens_a_pass, float* __restrict__ out, int act) {
    chain_release();
    chain_wait();
    const int r = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * LS_COLS;
    const int t0 = cu_q[r], n = cu_q[r + 1] - t0;
    if (n <= 0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int grp = lane & (LS_GROUPS - 1);               // row group: the low three lane bits
    const int my_col = warp * 4 + (lane >> 3);
    const int col = col0 + my_col;
    const bool col_ok = col < f;
    extern __shared__ float4 akw_s[];                     // [tokens][e]: (a, k, decay, -)
    float* v_s = reinterpret_cast<float*>(akw_s + (size_t)tokens_a_pass * e);   // [tokens][LS_COLS]

    float* S = state + (size_t)state_slot[r] * state_stride + (size_t)head * e * f;
    float s[RPT], ub[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int row = i * LS_GROUPS + grp;
        s[i] = (col_ok && row < e) ? S[(size_t)row * f + col] : 0.f;
        ub[i] = (bonus && row < e) ? load_as_float(bonus, (size_t)head * e + row, bonus_dtype) : 0.f;
    }
    const float g = TOK_DECAY ? 1.f : decay_head[head];
    // whether every row of a, k, v and the decays can be read four entries at a time
    const bool vec4 = ((e | f | a_row | a_off | k_row | k_off | v_row | v_off) & 3) == 0 &&
                      (!TOK_DECAY || (decay_row & 3) == 0);
    float* out_col = out + (size_t)head * f + col;
    const size_t out_row = (size_t)n_heads * f;

    for (int b0 = 0; b0 < n; b0 += tokens_a_pass) {
        const int nb = min(tokens_a_pass, n - b0);
        __syncthreads();
        if (vec4) {
            // four consecutive entries a load, two such units a thread under way at a time
            const int e4 = e >> 2, units = nb * e4;
            for (int u0 = threadIdx.x; u0 < units; u0 += 2 * LS_THREADS) {
                float4 av[2], kv[2], wv[2];
                int at[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int u = u0 + j * LS_THREADS;
                    at[j] = -1;
                    if (u < units) {
                        const int tt = u / e4, i = (u - tt * e4) << 2;
                        const size_t t = (size_t)(t0 + b0 + tt);
                        av[j] = load4(a_src, a_dtype, t * a_row + a_off + head * e + i);
                        kv[j] = load4(k_src, k_dtype, t * k_row + k_off + head * e + i);
                        if (act) {
                            av[j] = silu4(av[j]);
                            kv[j] = silu4(kv[j]);
                        }
                        wv[j] = TOK_DECAY ? *reinterpret_cast<const float4*>(
                                                decay_tok + t * decay_row + head * e + i)
                                          : make_float4(g, g, g, g);
                        at[j] = tt * e + i;
                    }
                }
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    if (at[j] >= 0) {
                        float4* dst = akw_s + at[j];
                        dst[0] = make_float4(av[j].x, kv[j].x, wv[j].x, 0.f);
                        dst[1] = make_float4(av[j].y, kv[j].y, wv[j].y, 0.f);
                        dst[2] = make_float4(av[j].z, kv[j].z, wv[j].z, 0.f);
                        dst[3] = make_float4(av[j].w, kv[j].w, wv[j].w, 0.f);
                    }
                }
            }
            for (int u = threadIdx.x; u < nb * (LS_COLS / 4); u += LS_THREADS) {
                const int tt = u / (LS_COLS / 4), j = (u - tt * (LS_COLS / 4)) << 2;
                const size_t t = (size_t)(t0 + b0 + tt);
                float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                if (col0 + j < f)                      // f is a multiple of four here
                    x = load4(v_src, v_dtype, t * v_row + v_off + head * f + col0 + j);
                if (act) x = silu4(x);
                *reinterpret_cast<float4*>(v_s + tt * LS_COLS + j) = x;
            }
        } else {
            for (int u = threadIdx.x; u < nb * e; u += LS_THREADS) {
                const int tt = u / e, i = u - tt * e;
                const size_t t = (size_t)(t0 + b0 + tt);
                float4 x;
                x.x = load_as_float(a_src, t * a_row + a_off + head * e + i, a_dtype);
                x.y = load_as_float(k_src, t * k_row + k_off + head * e + i, k_dtype);
                x.z = TOK_DECAY ? decay_tok[t * decay_row + head * e + i] : g;
                x.w = 0.f;
                if (act) {
                    x.x = silu1(x.x);
                    x.y = silu1(x.y);
                }
                akw_s[u] = x;
            }
            for (int u = threadIdx.x; u < nb * LS_COLS; u += LS_THREADS) {
                const int tt = u / LS_COLS, j = u - tt * LS_COLS;
                const size_t t = (size_t)(t0 + b0 + tt);
                const float x = col0 + j < f
                    ? load_as_float(v_src, t * v_row + v_off + head * f + col0 + j, v_dtype) : 0.f;
                v_s[u] = act ? silu1(x) : x;
            }
        }
        __syncthreads();
        // LS_UNROLL tokens at a time: their sums over the row groups (three shuffles each)
        // run side by side, only the state's own chain is sequential
        for (int tt0 = 0; tt0 < nb; tt0 += LS_UNROLL) {
            float acc[LS_UNROLL];
#pragma unroll
            for (int u = 0; u < LS_UNROLL; ++u) {
                acc[u] = 0.f;
                const int tt = tt0 + u;
                if (tt < nb) {
                    const float vj = v_s[tt * LS_COLS + my_col];
                    const float4* row = akw_s + (size_t)tt * e + grp;
                    if (read_first) {
#pragma unroll
                        for (int i = 0; i < RPT; ++i) {
                            if (i * LS_GROUPS + grp < e) {
                                const float4 x = row[i * LS_GROUPS];
                                acc[u] = fmaf(x.x, fmaf(ub[i] * x.y, vj, s[i]), acc[u]);
                                s[i] = fmaf(x.z, s[i], x.y * vj);
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < RPT; ++i) {
                            if (i * LS_GROUPS + grp < e) {
                                const float4 x = row[i * LS_GROUPS];
                                s[i] = fmaf(x.z, s[i], x.y * vj);
                                acc[u] = fmaf(x.x, s[i], acc[u]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < LS_UNROLL; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], 1);
#pragma unroll
            for (int u = 0; u < LS_UNROLL; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], 2);
#pragma unroll
            for (int u = 0; u < LS_UNROLL; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], 4);
            if (grp == 0 && col_ok) {
#pragma unroll
                for (int u = 0; u < LS_UNROLL; ++u)
                    if (tt0 + u < nb) out_col[(size_t)(t0 + b0 + tt0 + u) * out_row] = acc[u];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int row = i * LS_GROUPS + grp;
        if (col_ok && row < e) S[(size_t)row * f + col] = s[i];
    }
}

// One warp a (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
scan_finish_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_row,
                   int gate_off, const void* __restrict__ w, int w_dtype, float eps,
                   T* __restrict__ out, int n_tokens, int n_heads, int f) {
    chain_release();
    chain_wait();
    const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (unit >= (long long)n_tokens * n_heads) return;
    const int lane = threadIdx.x & 31;
    const int t = (int)(unit / n_heads), head = (int)(unit % n_heads);
    const float* row = o + (size_t)t * n_heads * f + (size_t)head * f;
    float ss = 0.f;
    for (int j = lane; j < f; j += 32) ss = fmaf(row[j], row[j], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)f + eps);
    for (int j = lane; j < f; j += 32) {
        const int c = head * f + j;
        const float z = Elem<T>::load(gate + (size_t)t * gate_row + gate_off + c);
        float v = row[j] * inv;
        if (w) v *= load_as_float(w, c, w_dtype);
        Elem<T>::store(out + (size_t)t * n_heads * f + c, v * (z / (1.0f + expf(-z))));
    }
}

// One block a token: the norm runs over the token's whole row of heads.
template <typename T>
__global__ void __launch_bounds__(256)
scan_finish_row_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_row,
                       int gate_off, const float* __restrict__ w, float eps, float out_scale,
                       T* __restrict__ out, long long out_row, int width) {
    chain_release();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    chain_wait();
    const float* row = o + (size_t)t * width;
    float ss = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) ss = fmaf(row[j], row[j], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float z = Elem<T>::load(gate + (size_t)t * gate_row + gate_off + j);
        float v = row[j] * inv;
        if (w) v *= w[j];
        Elem<T>::store(out + (size_t)t * out_row + j, v * (1.0f / (1.0f + expf(-z))) * out_scale);
    }
}

// One block a token; thread (head, i) rotates the pair (i, i + dims/2) of q and of k.
template <typename T>
__global__ void __launch_bounds__(256)
rotate_rows_kernel(const T* __restrict__ src, int src_row, int q_off, int k_off,
                   const int* __restrict__ positions, const double* __restrict__ freq, int dims,
                   float k_scale, float* __restrict__ out, int n_heads, int e) {
    chain_release();
    extern __shared__ float cs[];                        // [dims]: cos | sin
    const int t = blockIdx.x, half = dims / 2;
    chain_wait();
    const int p = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x)
        angle_cos_sin(p, freq[i], cs[i], cs[half + i]);
    __syncthreads();
    const int width = n_heads * e;
    for (int u = threadIdx.x; u < 2 * width; u += blockDim.x) {
        const int which = u / width, c = u - which * width, i = c % e;
        const T* row = src + (size_t)t * src_row + (which ? k_off : q_off);
        float v = Elem<T>::load(row + c);
        if (i < dims) {
            const bool low = i < half;
            const float m = Elem<T>::load(row + (low ? c + half : c - half));
            const float co = cs[low ? i : i - half], si = cs[half + (low ? i : i - half)];
            v = low ? __fsub_rn(__fmul_rn(v, co), __fmul_rn(m, si))
                    : __fadd_rn(__fmul_rn(v, co), __fmul_rn(m, si));
        }
        out[(size_t)t * 2 * width + u] = which ? v * k_scale : v;
    }
}

// lo (float32 [T, rank], before its tanh) -> w [T, channels].  A block takes DL_TOKENS tokens
// and 256 channels: tanh(lo) of its tokens lies in shared memory, a thread owns one channel
// and reads its column of W2 (handed over transposed, [rank, channels], so that a warp reads
// consecutive floats) once for all its tokens.  k ascending: a token's sum does not depend
// on its block.
constexpr int DL_TOKENS = 16;
__global__ void __launch_bounds__(256)
decay_lowrank_kernel(const float* __restrict__ lo, int rank, const float* __restrict__ w2t,
                     const void* __restrict__ w0, int w0_dtype, float* __restrict__ out,
                     int n_tokens, int channels) {
    chain_release();
    extern __shared__ float th[];                        // [DL_TOKENS][rank]
    const int t0 = blockIdx.y * DL_TOKENS, nt = min(DL_TOKENS, n_tokens - t0);
    const int c = blockIdx.x * 256 + threadIdx.x;
    chain_wait();
    for (int u = threadIdx.x; u < nt * rank; u += 256) th[u] = tanhf(lo[(size_t)t0 * rank + u]);
    __syncthreads();
    if (c >= channels) return;
    float z[DL_TOKENS];
#pragma unroll
    for (int tt = 0; tt < DL_TOKENS; ++tt) z[tt] = 0.f;
#pragma unroll 8
    for (int i = 0; i < rank; ++i) {                     // (eight loads under way; the sums stay in order)
        const float w = w2t[(size_t)i * channels + c];
#pragma unroll
        for (int tt = 0; tt < DL_TOKENS; ++tt)
            if (tt < nt) z[tt] = fmaf(w, th[tt * rank + i], z[tt]);
    }
    const float b = load_as_float(w0, c, w0_dtype);
#pragma unroll
    for (int tt = 0; tt < DL_TOKENS; ++tt)
        if (tt < nt) out[(size_t)(t0 + tt) * channels + c] = expf(-expf(z[tt] + b));
}

template <int RPT>
int launch_scan(dim3 grid, size_t smem, cudaStream_t stream, const void* a_src, int a_dtype,
                int a_row, int a_off, const void* k_src, int k_dtype, int k_row, int k_off,
                const void* v_src, int v_dtype, int v_row, int v_off, const float* decay_tok,
                int decay_row, const float* decay_head, const void* bonus, int bonus_dtype,
                int read_first, const int* cu_q, const int* state_slot, float* state,
                long long state_stride, int n_heads, int e, int f, int tokens_a_pass, float* out,
                int act) {
    auto kernel = decay_tok ? linear_scan_kernel<RPT, true> : linear_scan_kernel<RPT, false>;
    if (smem > 48 * 1024) {
        const int rc = (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem);
        if (rc) return rc;
    }
    MLS_LAUNCH(kernel, grid, dim3(LS_THREADS), smem, stream, a_src, a_dtype, a_row, a_off, k_src,
               k_dtype, k_row, k_off, v_src, v_dtype, v_row, v_off, decay_tok, decay_row,
               decay_head, bonus, bonus_dtype, read_first, cu_q, state_slot, state, state_stride,
               n_heads, e, f, tokens_a_pass, out, act);
    return launch_status();
}
}  // namespace

MLS_API int mls_linear_scan(const void* a_src, int a_dtype, int a_row, int a_off,
                            const void* k_src, int k_dtype, int k_row, int k_off,
                            const void* v_src, int v_dtype, int v_row, int v_off,
                            const float* decay_tok, int decay_row, const float* decay_head,
                            const void* bonus, int bonus_dtype, int read_first, const int* cu_q,
                            const int* state_slot, float* state, long long state_stride,
                            int n_requests, int n_heads, int e, int f, float* out, int act,
                            cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (e <= 0 || f <= 0 || e > 32 * LS_GROUPS || (!decay_tok == !decay_head))
        return MLS_ERR_UNSUPPORTED;
    const dim3 grid((f + LS_COLS - 1) / LS_COLS, n_heads, n_requests);
    const int tokens_a_pass = e <= 64 ? 32 : 16;
    const size_t smem = (size_t)tokens_a_pass * (e * sizeof(float4) + LS_COLS * sizeof(float));
    const int rpt = (e + LS_GROUPS - 1) / LS_GROUPS;
#define LS_GO(R)                                                                                 \
    return launch_scan<R>(grid, smem, stream, a_src, a_dtype, a_row, a_off, k_src, k_dtype, k_row, \
                          k_off, v_src, v_dtype, v_row, v_off, decay_tok, decay_row, decay_head,  \
                          bonus, bonus_dtype, read_first, cu_q, state_slot, state, state_stride,  \
                          n_heads, e, f, tokens_a_pass, out, act)
    if (rpt <= 2) LS_GO(2);
    if (rpt <= 4) LS_GO(4);
    if (rpt <= 8) LS_GO(8);
    if (rpt <= 16) LS_GO(16);
    LS_GO(32);
#undef LS_GO
}

MLS_API int mls_scan_finish(const float* o, const void* gate, int act_dtype, int gate_row,
                            int gate_off, const void* w, int w_dtype, float eps, void* out,
                            int n_tokens, int n_heads, int f, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const long long units = (long long)n_tokens * n_heads;
    const int blocks = (int)((units + 3) / 4);
    if (act_dtype == MLS_BF16)
        MLS_LAUNCH((scan_finish_kernel<__nv_bfloat16>), dim3(blocks), dim3(128), 0, stream, o,
                   (const __nv_bfloat16*)gate, gate_row, gate_off, w, w_dtype, eps,
                   (__nv_bfloat16*)out, n_tokens, n_heads, f);
    else
        MLS_LAUNCH((scan_finish_kernel<float>), dim3(blocks), dim3(128), 0, stream, o,
                   (const float*)gate, gate_row, gate_off, w, w_dtype, eps, (float*)out, n_tokens,
                   n_heads, f);
    return launch_status();
}

MLS_API int mls_scan_finish_row(const float* o, const void* gate, int act_dtype, int gate_row,
                                int gate_off, const float* w, float eps, float out_scale,
                                void* out, long long out_row, int n_tokens, int width,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (act_dtype == MLS_BF16)
        MLS_LAUNCH((scan_finish_row_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(256), 0, stream, o,
                   (const __nv_bfloat16*)gate, gate_row, gate_off, w, eps, out_scale,
                   (__nv_bfloat16*)out, out_row, width);
    else
        MLS_LAUNCH((scan_finish_row_kernel<float>), dim3(n_tokens), dim3(256), 0, stream, o,
                   (const float*)gate, gate_row, gate_off, w, eps, out_scale, (float*)out, out_row,
                   width);
    return launch_status();
}

MLS_API int mls_rotate_rows(const void* src, int src_dtype, int src_row, int q_off, int k_off,
                            const int* positions, const double* freq, int dims, float k_scale,
                            float* out, int n_tokens, int n_heads, int e, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dims < 0 || dims > e || (dims & 1) || (dims > 0 && !freq)) return MLS_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(dims > 0 ? dims : 1) * sizeof(float);
    if (smem > 48 * 1024) return MLS_ERR_UNSUPPORTED;
    if (src_dtype == MLS_BF16)
        MLS_LAUNCH((rotate_rows_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(256), smem, stream,
                   (const __nv_bfloat16*)src, src_row, q_off, k_off, positions, freq, dims,
                   k_scale, out, n_heads, e);
    else
        MLS_LAUNCH((rotate_rows_kernel<float>), dim3(n_tokens), dim3(256), smem, stream,
                   (const float*)src, src_row, q_off, k_off, positions, freq, dims, k_scale, out,
                   n_heads, e);
    return launch_status();
}

MLS_API int mls_decay_lowrank(const float* lo, int rank, const float* w2t, const void* w0,
                              int w0_dtype, float* out, int n_tokens, int channels,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const size_t smem = (size_t)DL_TOKENS * rank * sizeof(float);
    if (rank <= 0 || smem > 48 * 1024) return MLS_ERR_UNSUPPORTED;
    const dim3 grid((channels + 255) / 256, (n_tokens + DL_TOKENS - 1) / DL_TOKENS);
    MLS_LAUNCH((decay_lowrank_kernel), grid, dim3(256), smem, stream, lo, rank, w2t, w0, w0_dtype,
               out, n_tokens, channels);
    return launch_status();
}
