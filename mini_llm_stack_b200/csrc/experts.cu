// Routed experts: choose, sort, multiply expert by expert, add up.
//
// mls_route_topk: scores s = sigmoid(z), or softmax(z) over all outputs, of float32 router
//   logits z [T, E]; for every token the `top` largest scores (plus a per-output correction
//   that enters the choice only; the lowest index wins a tie) with the scores themselves as
//   weights (optionally divided by their sum + renorm_eps).  With n_groups > 1 the outputs form
//   n_groups equal groups of neighbours; a group's score is the sum of its two largest choice
//   scores, and only outputs of the keep_groups best groups (lowest index on a tie) can be
//   chosen.  A (token, choice) pair is a "slot": slot = t * top + j.  Outputs n_real .. E-1 stand for experts without weights that
//   return their input: they get no tiles, and mls_expert_combine adds weight * h for them.
// mls_route_sort: slots ordered by expert: order[p] = slot, offsets[E + 1], and the list
//   of row tiles (tile_expert, tile_row0) the products below walk.  One CTA.
// mls_expert_glu: y[p, :] = unit(Wg[e] a, Wu[e] a) with unit(g, u) = silu(g) * u or, with a
//   limit > 0, g' * sigmoid(alpha g') * (u' + 1), g' = min(g, limit), u' = clamp(u, +-limit);
//   a = weight[slot] * h[token]
//   (input scaling: the weight multiplies what enters the expert) or a = h[token]
//   (output scaling, applied by the down product instead).
// mls_expert_down: per_slot[slot, :] = Wd[e] y[p, :] (times the weight with output
//   scaling), float32.
// mls_expert_combine: delta[t] = sum_j per_slot[t * top + j] + shared[t], j ascending; with a
//   gate (float32, one number a token) the shared addend is multiplied by sigmoid(gate[t]).
//
// The products run with float32 accumulation over k ascending (bfloat16 rows of whole
// 16-byte pieces on the tensor cores, everything else on CUDA cores), one row
// tile of one expert a CTA; every row is computed by itself, so a token's result does
// not depend on the batch, on its place in the sorted order or on the other tokens of
// its expert.
#include "common.cuh"

namespace {
constexpr int BM = 32, BN = 64, BK = 32, TM = 2, TN = 4;   // 256 threads

constexpr int MAX_GROUPS = 256;

__global__ void route_topk_kernel(const float* __restrict__ logits, int logit_stride, int n_tokens,
                                  int n_experts, int top, int renorm, int softmax,
                                  const float* __restrict__ correction, float renorm_eps,
                                  int n_groups, int keep_groups,
                                  int* __restrict__ idx, float* __restrict__ weight) {
    chain_release();
    chain_wait();
    // one warp a token
    __shared__ float group_score[4][MAX_GROUPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n_tokens) return;
    const float* z = logits + (size_t)t * logit_stride;
    // softmax over all outputs: the largest logit and the sum of exponentials, both in the
    // order of the lanes' strides, so a token's scores do not depend on its batch
    float z_max = 0.f, inv_sum = 1.f;
    if (softmax) {
        z_max = -INFINITY;
        for (int e = lane; e < n_experts; e += 32) z_max = fmaxf(z_max, z[e]);
        z_max = warp_max(z_max);
        float sum = 0.f;
        for (int e = lane; e < n_experts; e += 32) sum += expf(z[e] - z_max);
        inv_sum = 1.0f / warp_sum(sum);
    }
    const int group_size = n_groups > 1 ? n_experts / n_groups : n_experts;
    if (n_groups > 1) {
        // a group's score: the sum of its two largest choice scores (one, if it has one member)
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;
            for (int e = g * group_size; e < (g + 1) * group_size; ++e) {
                const float s = softmax ? expf(z[e] - z_max) * inv_sum : 1.0f / (1.0f + expf(-z[e]));
                const float c = correction ? s + correction[e] : s;
                if (c > a) { b = a; a = c; } else if (c > b) { b = c; }
            }
            group_score[warp][g] = group_size > 1 ? a + b : a;
        }
        __syncwarp();
    }
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY, best_s = 0.f;
        int arg = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            bool taken = false;
            if (n_groups > 1) {
                // the group's rank: how many groups come before it
                const int g = e / group_size;
                const float mine = group_score[warp][g];
                int before = 0;
                for (int o = 0; o < n_groups; ++o) {
                    const float other = group_score[warp][o];
                    before += (other > mine || (other == mine && o < g)) ? 1 : 0;
                }
                taken = before >= keep_groups;
            }
            for (int p = 0; p < j; ++p) taken |= idx[(size_t)t * top + p] == e;
            const float s = softmax ? expf(z[e] - z_max) * inv_sum : 1.0f / (1.0f + expf(-z[e]));
            const float c = correction ? s + correction[e] : s;      // the choice's score
            if (!taken && (c > best || (c == best && e < arg))) {
                best = c;
                best_s = s;
                arg = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) {
                best = ob;
                best_s = os;
                arg = oa;
            }
        }
        if (arg >= n_experts) {                  // only scores that are not numbers were left
            arg = 0;
            best_s = 0.f;
        }
        if (lane == 0) {
            idx[(size_t)t * top + j] = arg;
            weight[(size_t)t * top + j] = best_s;
        }
        total += best_s;
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int j = 0; j < top; ++j) weight[(size_t)t * top + j] /= total + renorm_eps;
}

__global__ void __launch_bounds__(1024)
route_sort_kernel(const int* __restrict__ idx, int n_slots, int n_experts, int n_real,
                  int* __restrict__ order, int* __restrict__ offsets,
                  int* __restrict__ tile_expert, int* __restrict__ tile_row0, int max_tiles,
                  int* __restrict__ cursor /* [E] scratch */) {
    chain_release();
    chain_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) cursor[e] = 0;
    __syncthreads();
    for (int s = threadIdx.x; s < n_slots; s += blockDim.x) atomicAdd(&cursor[idx[s]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tile = 0;
        for (int e = 0; e < n_experts; ++e) {
            const int c = cursor[e];
            offsets[e] = at;
            // (an expert past n_real has no weights: its slots are settled where the sum is taken)
            for (int r = 0; r < c && e < n_real && tile < max_tiles; r += BM) {
                tile_expert[tile] = e;
                tile_row0[tile] = at + r;
                ++tile;
            }
            cursor[e] = at;
            at += c;
        }
        offsets[n_experts] = at;
        for (; tile < max_tiles; ++tile) tile_expert[tile] = -1;
    }
    __syncthreads();
    // which place a slot gets inside its expert is left to the atomics: every row is
    // computed by itself, so the values do not depend on it
    for (int s = threadIdx.x; s < n_slots; s += blockDim.x)
        order[atomicAdd(&cursor[idx[s]], 1)] = s;
}

// 16 bytes of a row as floats: eight bfloat16 or four float32.
template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            out[2 * e] = f.x;
            out[2 * e + 1] = f.y;
        }
    }
};

// Fill tile[k][row] (k < BK, row < ROWS) from rows of K-contiguous values: row r comes from
// src(r) (nullptr: zeros), scaled by scale(r).  16-byte loads where K allows them.
template <typename T, int ROWS, int PAD, typename Src>
__device__ __forceinline__ void fill_tile(float (*tile)[ROWS + PAD], int k0, int K, bool vec_ok,
                                          Src src) {
    constexpr int V = Vec<T>::N;
    if (vec_ok) {
        for (int u = threadIdx.x; u < ROWS * (BK / V); u += 256) {
            const int r = u / (BK / V), kv = (u - r * (BK / V)) * V;
            float scale = 1.f;
            const T* p = src(r, scale);
            float v[V];
            if (p && k0 + kv < K) {
                Vec<T>::load(p + k0 + kv, v);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) v[e] = 0.f;
            }
#pragma unroll
            for (int e = 0; e < V; ++e) tile[kv + e][r] = v[e] * scale;
        }
    } else {
        for (int u = threadIdx.x; u < ROWS * BK; u += 256) {
            const int r = u / BK, k = u - r * BK;
            float scale = 1.f;
            const T* p = src(r, scale);
            tile[k][r] = (p && k0 + k < K) ? Elem<T>::load(p + k0 + k) * scale : 0.f;
        }
    }
}

// The gated unit on the two products' float32 sums.
__device__ __forceinline__ float gated_unit(float g, float u, float alpha, float limit) {
    if (limit > 0.f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return (g / (1.0f + expf(-alpha * g))) * (u + 1.0f);
    }
    return (g / (1.0f + expf(-g))) * u;
}

// GLU: A row = h[slot / top] (* weight[slot] if scale), W = [gate rows | up rows] of
// expert e ([2F, K]), out y[p, n] = silu(gate) * up in T.
// !GLU: A row = y[p], W = Wd[e] ([N, K]), out per_slot[slot, n] float32 (* weight[slot]
// if scale).  A thread owns rows ty*TM.. and the columns tx, tx + 16, tx + 32, tx + 48.
template <typename T, bool GLU>
__global__ void __launch_bounds__(256)
expert_gemm_kernel(const T* __restrict__ A, const T* __restrict__ W, void* __restrict__ out,
                   const int* __restrict__ order, const int* __restrict__ offsets,
                   const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                   const float* __restrict__ weight, int top, int scale, int N, int K,
                   float alpha, float limit) {
    chain_release();
    chain_wait();
    const int e = tile_expert[blockIdx.y];
    if (e < 0) return;
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[BK][BN + 1];
    __shared__ float Us[GLU ? BK : 1][BN + 1];
    __shared__ int slot_s[BM];
    const int tid = threadIdx.x;
    const int p0 = tile_row0[blockIdx.y], p_end = offsets[e + 1];
    const int n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;                     // 16 x 16
    if (tid < BM) slot_s[tid] = p0 + tid < p_end ? order[p0 + tid] : -1;
    __syncthreads();
    const T* We = W + (size_t)e * (GLU ? 2 : 1) * N * K;
    const bool vec_ok = K % Vec<T>::N == 0 &&
                        (reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) % 16 == 0;
    float acc[TM][TN], acu[GLU ? TM : 1][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = 0.f;
            if (GLU) acu[i][j] = 0.f;
        }
    for (int k0 = 0; k0 < K; k0 += BK) {
        fill_tile<T, BM, 1>(As, k0, K, vec_ok, [&](int r, float& sc) -> const T* {
            const int slot = slot_s[r];
            if (slot < 0) return nullptr;
            if (GLU) {
                if (scale) sc = weight[slot];
                return A + (size_t)(slot / top) * K;
            }
            return A + (size_t)(p0 + r) * K;
        });
        fill_tile<T, BN, 1>(Ws, k0, K, vec_ok, [&](int r, float&) -> const T* {
            return n0 + r < N ? We + (size_t)(n0 + r) * K : nullptr;
        });
        if (GLU)
            fill_tile<T, BN, 1>(Us, k0, K, vec_ok, [&](int r, float&) -> const T* {
                return n0 + r < N ? We + (size_t)(N + n0 + r) * K : nullptr;
            });
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN], u[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                w[j] = Ws[kk][tx + 16 * j];
                if (GLU) u[j] = Us[kk][tx + 16 * j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
                    if (GLU) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = ty * TM + i;
        const int slot = slot_s[r];
        if (slot < 0) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n >= N) continue;
            if (GLU) {
                Elem<T>::store((T*)out + (size_t)(p0 + r) * N + n,
                               gated_unit(acc[i][j], acu[i][j], alpha, limit));
            } else {
                ((float*)out)[(size_t)slot * N + n] = scale ? acc[i][j] * weight[slot] : acc[i][j];
            }
        }
    }
}

// The same products for bfloat16 on the tensor cores (mma.sync m16n8k16, float32
// accumulators): a CTA takes up to four of the same tiles of 32 sorted rows x 64 output
// columns, its eight warps 32 x 32 each; operands go through shared memory in rows of 32 + 8 values, so that
// the fragment loads (one 32-bit word a lane) meet no bank twice.  Every output element is
// its own dot product over k ascending in steps of 16, whatever else is in the tile.  With
// input scaling the row is rounded to bfloat16 once more after the weight is applied.
constexpr int MK = 32, MKP = MK + 8;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A CTA walks RT consecutive entries of the tile list; entries of one expert that follow each
// other (a prompt gives an expert many rows) are taken together, up to RT * 32 = 128 rows
// against one load of every weight tile; rows that are not there are zeros.
// RT = 1 (few rows an expert: decoding) keeps one entry a CTA, so that as many CTAs as
// possible stream weights.
template <bool GLU, int RT>
__global__ void __launch_bounds__(256)
expert_mma_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                  void* __restrict__ out, const int* __restrict__ order,
                  const int* __restrict__ offsets, const int* __restrict__ tile_expert,
                  const int* __restrict__ tile_row0, int max_tiles,
                  const float* __restrict__ weight, int top, int scale, int N, int K,
                  float alpha, float limit) {
    chain_release();
    chain_wait();
    constexpr int MROWS = RT * BM;
    // RT 4: 4 x 2 warps of 32 rows x 32 columns; RT 1: 2 x 4 warps of 16 x 16
    constexpr int MF = RT == 4 ? 2 : 1, NF = RT == 4 ? 4 : 2, WARPS_N = RT == 4 ? 2 : 4;
    constexpr int LOADS = (MROWS * 4 + 255) / 256;            // 16-byte pieces of A a thread loads
    __shared__ __align__(16) __nv_bfloat16 As[MROWS][MKP];
    __shared__ __align__(16) __nv_bfloat16 Ws[BN][MKP];
    __shared__ __align__(16) __nv_bfloat16 Us[GLU ? BN : 1][MKP];
    __shared__ int slot_s[MROWS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BN;
    const int wm = warp / WARPS_N, wn = warp % WARPS_N;
    const int g = lane >> 2, c = (lane & 3) * 2;
    const int lrow = tid >> 2, lk = (tid & 3) * 8;            // who loads what: 16 bytes a thread
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const int t_end = min(max_tiles, (int)(blockIdx.y + 1) * RT);   // every output element is the same sum for either RT
    int t = blockIdx.y * RT;
    while (t < t_end) {
        const int e = tile_expert[t];
        if (e < 0) break;                                     // the list's unused tail
        int run = 1;
        while (t + run < t_end && tile_expert[t + run] == e) ++run;
        const int p0 = tile_row0[t], p_end = offsets[e + 1];
        t += run;
        __syncthreads();                                      // the last run's slot_s is read no more
        if (tid < MROWS) slot_s[tid] = (tid < run * BM && p0 + tid < p_end) ? order[p0 + tid] : -1;
        __syncthreads();
        const __nv_bfloat16* We = W + (size_t)e * (GLU ? 2 : 1) * N * K;
        float acc[MF][NF][4], acu[GLU ? MF : 1][NF][4];
#pragma unroll
        for (int i = 0; i < MF; ++i)
#pragma unroll
            for (int j = 0; j < NF; ++j)
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    acc[i][j][x] = 0.f;
                    if (GLU) acu[i][j][x] = 0.f;
                }
        const __nv_bfloat16* a_src[LOADS];
        float a_scale[LOADS];
#pragma unroll
        for (int h2 = 0; h2 < LOADS; ++h2) {
            const int r = lrow + 64 * h2;
            const int slot = r < MROWS ? slot_s[r] : -1;
            a_src[h2] = nullptr;
            a_scale[h2] = 1.f;
            if (slot >= 0) {
                if (GLU) {
                    a_src[h2] = A + (size_t)(slot / top) * K;
                    if (scale) a_scale[h2] = weight[slot];
                } else {
                    a_src[h2] = A + (size_t)(p0 + r) * K;
                }
            }
        }
        const bool w_ok = n0 + lrow < N;
        const __nv_bfloat16* w_src = We + (size_t)(n0 + lrow) * K;
        const __nv_bfloat16* u_src = We + (size_t)(N + n0 + lrow) * K;
        for (int k0 = 0; k0 < K; k0 += MK) {
            const bool k_ok = k0 + lk < K;
#pragma unroll
            for (int h2 = 0; h2 < LOADS; ++h2) {
                if (lrow + 64 * h2 >= MROWS) continue;
                uint4 v = (a_src[h2] && k_ok) ? *reinterpret_cast<const uint4*>(a_src[h2] + k0 + lk) : zero;
                if (GLU && scale && a_src[h2]) {
                    __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const float2 f2 = __bfloat1622float2(p2[x]);
                        p2[x] = __floats2bfloat162_rn(f2.x * a_scale[h2], f2.y * a_scale[h2]);
                    }
                }
                *reinterpret_cast<uint4*>(&As[lrow + 64 * h2][lk]) = v;
            }
            *reinterpret_cast<uint4*>(&Ws[lrow][lk]) =
                (w_ok && k_ok) ? *reinterpret_cast<const uint4*>(w_src + k0 + lk) : zero;
            if (GLU)
                *reinterpret_cast<uint4*>(&Us[lrow][lk]) =
                    (w_ok && k_ok) ? *reinterpret_cast<const uint4*>(u_src + k0 + lk) : zero;
            __syncthreads();
            if (16 * MF * wm < run * BM) {                    // a warp whose rows are not there idles
#pragma unroll
                for (int kk = 0; kk < MK; kk += 16) {
                    uint32_t a[MF][4];
#pragma unroll
                    for (int mf = 0; mf < MF; ++mf) {
                        const int r = 16 * MF * wm + 16 * mf + g;
                        a[mf][0] = *reinterpret_cast<const uint32_t*>(&As[r][kk + c]);
                        a[mf][1] = *reinterpret_cast<const uint32_t*>(&As[r + 8][kk + c]);
                        a[mf][2] = *reinterpret_cast<const uint32_t*>(&As[r][kk + c + 8]);
                        a[mf][3] = *reinterpret_cast<const uint32_t*>(&As[r + 8][kk + c + 8]);
                    }
#pragma unroll
                    for (int nf = 0; nf < NF; ++nf) {
                        const int n = 8 * NF * wn + 8 * nf + g;
                        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&Ws[n][kk + c]);
                        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&Ws[n][kk + c + 8]);
#pragma unroll
                        for (int mf = 0; mf < MF; ++mf) mma_bf16(acc[mf][nf], a[mf], b0, b1);
                        if (GLU) {
                            const uint32_t u0 = *reinterpret_cast<const uint32_t*>(&Us[n][kk + c]);
                            const uint32_t u1 = *reinterpret_cast<const uint32_t*>(&Us[n][kk + c + 8]);
#pragma unroll
                            for (int mf = 0; mf < MF; ++mf) mma_bf16(acu[mf][nf], a[mf], u0, u1);
                        }
                    }
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int mf = 0; mf < MF; ++mf)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = 16 * MF * wm + 16 * mf + g + 8 * half;
                const int slot = slot_s[r];
                if (slot < 0) continue;
#pragma unroll
                for (int nf = 0; nf < NF; ++nf)
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const int n = n0 + 8 * NF * wn + 8 * nf + c + x;
                        if (n >= N) continue;
                        const float v = acc[mf][nf][2 * half + x];
                        if (GLU)
                            ((__nv_bfloat16*)out)[(size_t)(p0 + r) * N + n] = __float2bfloat16_rn(
                                gated_unit(v, acu[mf][nf][2 * half + x], alpha, limit));
                        else
                            ((float*)out)[(size_t)slot * N + n] = scale ? v * weight[slot] : v;
                    }
            }
    }
}

// bfloat16 rows of whole 16-byte pieces at 16-byte addresses: the tensor-core kernel's.
static inline bool takes_mma(int dtype, const void* a, const void* w, int K) {
    return dtype == MLS_BF16 && K % 8 == 0 &&
           (reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) % 16 == 0;
}

template <typename T>
__global__ void expert_combine_kernel(const float* __restrict__ per_slot, int top,
                                      const void* __restrict__ shared, int shared_dtype,
                                      const int* __restrict__ idx, const float* __restrict__ weight,
                                      int n_real, const T* __restrict__ h,
                                      const float* __restrict__ gate, int gate_stride,
                                      T* __restrict__ delta, size_t n, int d) {
    chain_release();
    chain_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / d, c = i - t * d;
        float s = 0.f;
        for (int j = 0; j < top; ++j) {
            // a choice past the experts that have weights returns its input, times its weight
            if (idx && idx[t * top + j] >= n_real)
                s += weight[t * top + j] * Elem<T>::load(h + i);
            else
                s += per_slot[(t * top + j) * d + c];
        }
        if (shared) {
            const float v = load_as_float(shared, i, shared_dtype);
            s += gate ? v / (1.0f + expf(-gate[t * gate_stride])) : v;
        }
        Elem<T>::store(delta + i, s);
    }
}
}  // namespace

MLS_API int mls_expert_tile_rows() { return BM; }

MLS_API int mls_route_topk(const float* logits, int logit_stride, int n_tokens, int n_experts,
                           int top, int renorm, int softmax, const float* correction,
                           float renorm_eps, int n_groups, int keep_groups, int* idx,
                           float* weight, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top <= 0 || top > n_experts) return MLS_ERR_UNSUPPORTED;
    if (n_groups > 1 && (n_groups > MAX_GROUPS || n_experts % n_groups || keep_groups < 1 ||
                         keep_groups > n_groups || top > keep_groups * (n_experts / n_groups)))
        return MLS_ERR_UNSUPPORTED;
    MLS_LAUNCH((route_topk_kernel), dim3((n_tokens + 3) / 4), dim3(128), 0, stream, logits,
               logit_stride, n_tokens, n_experts, top, renorm, softmax, correction, renorm_eps,
               n_groups, keep_groups, idx, weight);
    return launch_status();
}

MLS_API int mls_route_sort(const int* idx, int n_slots, int n_experts, int n_real, int* order,
                           int* offsets,
                           int* tile_expert, int* tile_row0, int max_tiles, int* cursor,
                           cudaStream_t stream) {
    if (n_slots <= 0) return 0;
    MLS_LAUNCH((route_sort_kernel), dim3(1), dim3(1024), 0, stream, idx, n_slots, n_experts,
               n_real, order, offsets, tile_expert, tile_row0, max_tiles, cursor);
    return launch_status();
}

MLS_API int mls_expert_glu(const void* h, const void* w_gate_up, void* y, int dtype,
                           const int* order, const int* offsets, const int* tile_expert,
                           const int* tile_row0, int max_tiles, const float* weight, int top,
                           int scale_in, int F, int K, int many_rows, float alpha, float limit,
                           cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    dim3 grid((F + BN - 1) / BN, max_tiles);
    if (takes_mma(dtype, h, w_gate_up, K) && many_rows)
        MLS_LAUNCH((expert_mma_kernel<true, 4>), dim3(grid.x, (max_tiles + 3) / 4), dim3(256), 0,
                   stream, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w_gate_up, y, order, offsets,
                   tile_expert, tile_row0, max_tiles, weight, top, scale_in, F, K, alpha, limit);
    else if (takes_mma(dtype, h, w_gate_up, K))
        MLS_LAUNCH((expert_mma_kernel<true, 1>), dim3(grid), dim3(256), 0, stream,
                   (const __nv_bfloat16*)h, (const __nv_bfloat16*)w_gate_up, y, order, offsets,
                   tile_expert, tile_row0, max_tiles, weight, top, scale_in, F, K, alpha, limit);
    else if (dtype == MLS_BF16)
        MLS_LAUNCH((expert_gemm_kernel<__nv_bfloat16, true>), dim3(grid), dim3(256), 0, stream,
                   (const __nv_bfloat16*)h, (const __nv_bfloat16*)w_gate_up, y, order, offsets,
                   tile_expert, tile_row0, weight, top, scale_in, F, K, alpha, limit);
    else
        MLS_LAUNCH((expert_gemm_kernel<float, true>), dim3(grid), dim3(256), 0, stream,
                   (const float*)h, (const float*)w_gate_up, y, order, offsets, tile_expert,
                   tile_row0, weight, top, scale_in, F, K, alpha, limit);
    return launch_status();
}

MLS_API int mls_expert_down(const void* y, const void* w_down, float* per_slot, int dtype,
                            const int* order, const int* offsets, const int* tile_expert,
                            const int* tile_row0, int max_tiles, const float* weight, int top,
                            int scale_out, int D, int F, int many_rows, cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    dim3 grid((D + BN - 1) / BN, max_tiles);
    if (takes_mma(dtype, y, w_down, F) && many_rows)
        MLS_LAUNCH((expert_mma_kernel<false, 4>), dim3(grid.x, (max_tiles + 3) / 4), dim3(256), 0,
                   stream, (const __nv_bfloat16*)y, (const __nv_bfloat16*)w_down, (void*)per_slot,
                   order, offsets, tile_expert, tile_row0, max_tiles, weight, top, scale_out, D, F, 0.f, 0.f);
    else if (takes_mma(dtype, y, w_down, F))
        MLS_LAUNCH((expert_mma_kernel<false, 1>), dim3(grid), dim3(256), 0, stream,
                   (const __nv_bfloat16*)y, (const __nv_bfloat16*)w_down, (void*)per_slot, order,
                   offsets, tile_expert, tile_row0, max_tiles, weight, top, scale_out, D, F, 0.f, 0.f);
    else if (dtype == MLS_BF16)
        MLS_LAUNCH((expert_gemm_kernel<__nv_bfloat16, false>), dim3(grid), dim3(256), 0, stream,
                   (const __nv_bfloat16*)y, (const __nv_bfloat16*)w_down, (void*)per_slot, order,
                   offsets, tile_expert, tile_row0, weight, top, scale_out, D, F, 0.f, 0.f);
    else
        MLS_LAUNCH((expert_gemm_kernel<float, false>), dim3(grid), dim3(256), 0, stream,
                   (const float*)y, (const float*)w_down, (void*)per_slot, order, offsets,
                   tile_expert, tile_row0, weight, top, scale_out, D, F, 0.f, 0.f);
    return launch_status();
}

MLS_API int mls_expert_combine(const float* per_slot, int top, const void* shared,
                               int shared_dtype, const int* idx, const float* weight, int n_real,
                               const void* h, const float* gate, int gate_stride, void* delta,
                               int dtype, int n_tokens, int d, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const size_t n = (size_t)n_tokens * d;
    const size_t want = (n + 255) / 256;
    const int blocks = (int)(want < (size_t)(8 * sm_count()) ? want : 8 * sm_count());
    if (dtype == MLS_BF16)
        MLS_LAUNCH((expert_combine_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream,
                   per_slot, top, shared, shared_dtype, idx, weight, n_real, (const __nv_bfloat16*)h,
                   gate, gate_stride, (__nv_bfloat16*)delta, n, d);
    else
        MLS_LAUNCH((expert_combine_kernel<float>), dim3(blocks), dim3(256), 0, stream, per_slot,
                   top, shared, shared_dtype, idx, weight, n_real, (const float*)h, gate, gate_stride,
                   (float*)delta, n, d);
    return launch_status();
}
