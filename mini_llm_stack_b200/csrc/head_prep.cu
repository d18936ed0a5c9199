// Preparation of grouped-query attention without rotation: from the float32 projection row
// [.. q heads (e each) .. k heads (e each) .. v heads (f each) ..] of every token of a step
//
//   q_h <- (q_h + b_q) ;  k_g <- (k_g + b_k) ;  v_g <- (v_g + b_v) * v_scale      biases optional
//   q_h <- q_h / sqrt(mean(q_h^2) + eps) * w_q, k_g likewise with w_k           per head, optional;
//                                                                  the weights [e] serve all heads
//   q_h <- q_h * (1 + coef * ln(floor((p + 1) / every) + 1))      the query's temperature at
//                                                                  position p, optional
//
// q goes to the row the attention kernels read ([T, q_width], head h at h * hd), k and v into
// the pages at the step's slots.  Heads are hd wide in both places: the entries past e (past
// f for the values) are zeros, which changes no score and leaves zeros in the outputs' extra
// entries.  The rest of a page that a request enters in this step is cleared.
//
// One block a token, one warp a head at a time; sums of squares in float32 in lane-stride
// order and five shuffles, so a token's values depend on nothing else in the batch.
#include "common.cuh"
#include "page_tail.cuh"

namespace {
constexpr int HP_THREADS = 128;      // a block of a prompt's token
constexpr int HP_MAX_THREADS = 512;  // few tokens: up to a warp a head, so that no warp takes many in turn

template <typename T>
__global__ void __launch_bounds__(HP_MAX_THREADS)
head_prep_kernel(const float* __restrict__ proj, int proj_width, int q_col, int k_col, int v_col,
                 const float* __restrict__ b_q, const float* __restrict__ b_k,
                 const float* __restrict__ b_v, const float* __restrict__ w_q,
                 const float* __restrict__ w_k, float eps, float temp_coef, int temp_every,
                 float v_scale, const int* __restrict__ positions,
                 const int* __restrict__ slot_map, T* __restrict__ q_out, int q_width,
                 T* __restrict__ k_pool, T* __restrict__ v_pool, int block_size, int n_pages,
                 int n_tokens, int n_heads, int n_kv, int e, int f, int hd, int writes,
                 int* __restrict__ status) {
    chain_release();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    int slot = -1, rest = 0;
    if (writes) {
        slot = slot_map[t];
        if (slot < 0 || slot >= n_pages * block_size) {
            if (threadIdx.x == 0 && status) atomicOr(status, MLS_STATUS_BAD_SLOT);
            slot = -1;
        } else {
            rest = page_tail_to_clear(slot_map, t, n_tokens, slot, block_size);
        }
    }
    float temp = 1.f;
    if (temp_every > 0)
        temp = 1.0f + temp_coef * logf((float)((positions[t] + 1) / temp_every + 1));
    chain_wait();
    const float* row = proj + (size_t)t * proj_width;
    const int units = n_heads + (writes ? 2 * n_kv : 0);
    for (int u = warp; u < units; u += n_warps) {
        // which head this is, where it comes from and where it goes
        const int kind = u < n_heads ? 0 : (u < n_heads + n_kv ? 1 : 2);
        const int head = kind == 0 ? u : (kind == 1 ? u - n_heads : u - n_heads - n_kv);
        const int width = kind == 2 ? f : e;
        const float* src = row + (kind == 0 ? q_col : kind == 1 ? k_col : v_col) + (size_t)head * width;
        const float* bias = kind == 0 ? b_q : kind == 1 ? b_k : b_v;
        if (bias) bias += (size_t)head * width;
        const float* w = kind == 0 ? w_q : kind == 1 ? w_k : nullptr;
        T* dst;
        if (kind == 0) {
            dst = q_out + (size_t)t * q_width + (size_t)head * hd;
        } else {
            if (slot < 0) continue;
            const int page = slot / block_size, off = slot - page * block_size;
            dst = (kind == 1 ? k_pool : v_pool) +
                  (((size_t)head * n_pages + page) * block_size + off) * hd;
        }
        float mul = kind == 0 ? temp : (kind == 2 ? v_scale : 1.f);
        if (w) {
            float ss = 0.f;
            for (int i = lane; i < width; i += 32) {
                const float x = src[i] + (bias ? bias[i] : 0.f);
                ss = fmaf(x, x, ss);
            }
            mul *= 1.0f / sqrtf(warp_sum(ss) / (float)width + eps);
        }
        for (int i = lane; i < hd; i += 32) {
            float x = 0.f;
            if (i < width) {
                x = (src[i] + (bias ? bias[i] : 0.f)) * mul;
                if (w) x *= w[i];
            }
            Elem<T>::store(dst + i, x);
        }
    }
    if (writes && slot >= 0) {
        __syncthreads();
        clear_page_tail<T>(rest, slot, block_size, n_pages, n_kv, hd, k_pool, v_pool);
    }
}
}  // namespace

MLS_API int mls_head_prep_store(const float* proj, int proj_width, int q_col, int k_col, int v_col,
                                const float* b_q, const float* b_k, const float* b_v,
                                const float* w_q, const float* w_k, float eps, float temp_coef,
                                int temp_every, float v_scale, const int* positions,
                                const int* slot_map, void* q_out, int q_width, int dtype,
                                void* k_pool, void* v_pool, int block_size, int n_pages,
                                int n_tokens, int n_heads, int n_kv, int e, int f, int hd,
                                int writes, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (e <= 0 || f <= 0 || hd < e || hd < f || n_heads <= 0 || n_kv <= 0) return MLS_ERR_UNSUPPORTED;
    const int units = n_heads + (writes ? 2 * n_kv : 0);
    const int threads = n_tokens > 64 ? HP_THREADS
        : (32 * units < HP_THREADS ? HP_THREADS : (32 * units > HP_MAX_THREADS ? HP_MAX_THREADS : 32 * units));
    if (dtype == MLS_BF16)
        MLS_LAUNCH((head_prep_kernel<__nv_bfloat16>), dim3(n_tokens), dim3(threads), 0, stream,
                   proj, proj_width, q_col, k_col, v_col, b_q, b_k, b_v, w_q, w_k, eps, temp_coef,
                   temp_every, v_scale, positions, slot_map, (__nv_bfloat16*)q_out, q_width,
                   (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, block_size, n_pages, n_tokens,
                   n_heads, n_kv, e, f, hd, writes, status);
    else
        MLS_LAUNCH((head_prep_kernel<float>), dim3(n_tokens), dim3(threads), 0, stream, proj,
                   proj_width, q_col, k_col, v_col, b_q, b_k, b_v, w_q, w_k, eps, temp_coef,
                   temp_every, v_scale, positions, slot_map, (float*)q_out, q_width,
                   (float*)k_pool, (float*)v_pool, block_size, n_pages, n_tokens, n_heads, n_kv,
                   e, f, hd, writes, status);
    return launch_status();
}
