// True 32-bit matrix product for the float32 path: out[M, N] = A[M, K] * W[N, K]^T.
// A may be held in bfloat16 (a router's input in a 16-bit run): its values are widened as
// they are loaded, the arithmetic is the same.
//
// Plain FFMA on CUDA cores: no tensor cores, no TF32, no reduced-precision mode.
// Each output element is accumulated over k = 0 .. K-1 in that order, whatever M
// and N are, so a token's result does not depend on the batch it is computed in.
// Both operands are K-contiguous (the reference's nn.Linear layout [out, in],
// train/model.py:79-82,130-132).
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const void* __restrict__ A, int a_dtype, const float* __restrict__ W,
                float* __restrict__ out, int M, int N, int K, int ldo) {
    chain_release();
    chain_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // each thread loads 4 elements of each tile: row = tid / 4 (0..63), k = (tid % 4) * 4 ..
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + e][lrow] = (am < M && k < K) ? load_as_float(A, (size_t)am * K + k, a_dtype) : 0.f;
            Ws[lk + e][lrow] = (wn < N && k < K) ? W[(size_t)wn * K + k] : 0.f;
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
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) out[(size_t)m * ldo + n] = acc[i][j];
        }
    }
}

// Few output columns (a router's or a gate's scores: N <= SKINNY_N): the tile kernel above
// would leave all but a few SMs idle and walk K in steps of 16 behind two barriers each.
// Here a block holds SK_ROWS rows of A in shared memory, each of its eight warps owns COLS
// neighbouring output columns and its lanes walk K four entries at a time with a stride of
// 128 (one entry at a time with a stride of 32 where rows of K entries are not whole 16-byte
// chunks); the 32 partial sums are added by a fixed tree.  The order of the additions
// depends on K alone (never on M, on COLS or on the row's place in its block), and which
// kernel runs depends on N alone, so a token's result still does not depend on its batch:
// many rows take COLS = 4 (four products for every value read from shared memory), few rows
// COLS = 1 (four times the blocks), with the same bits.
constexpr int SKINNY_N = 256, SK_ROWS = 8, SK_KC = 1024;

template <int COLS>
__global__ void __launch_bounds__(256)
gemm_f32_skinny_kernel(const void* __restrict__ A, int a_dtype, const float* __restrict__ W,
                       float* __restrict__ out, int M, int N, int K, int by4) {
    chain_release();
    chain_wait();
    __shared__ __align__(16) float As[SK_ROWS][SK_KC];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * SK_ROWS;
    const int n0 = (blockIdx.y * 8 + warp) * COLS;
    float acc[COLS][SK_ROWS];
#pragma unroll
    for (int c = 0; c < COLS; ++c)
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r) acc[c][r] = 0.f;
    for (int k0 = 0; k0 < K; k0 += SK_KC) {
        const int kc = min(SK_KC, K - k0);
        __syncthreads();
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r)
            for (int k = threadIdx.x; k < kc; k += 256)
                As[r][k] = m0 + r < M ? load_as_float(A, (size_t)(m0 + r) * K + k0 + k, a_dtype) : 0.f;
        __syncthreads();
        if (n0 >= N) continue;
        if (by4) {
            // several rounds' loads of W under way at a time: the sums keep their order
#pragma unroll 4
            for (int k = lane * 4; k < kc; k += 128) {
                float4 a[SK_ROWS];
#pragma unroll
                for (int r = 0; r < SK_ROWS; ++r) a[r] = *reinterpret_cast<const float4*>(&As[r][k]);
#pragma unroll
                for (int c = 0; c < COLS; ++c) {
                    if (n0 + c >= N) break;
                    const float4 w = *reinterpret_cast<const float4*>(W + (size_t)(n0 + c) * K + k0 + k);
#pragma unroll
                    for (int r = 0; r < SK_ROWS; ++r) {
                        float s = acc[c][r];
                        s = fmaf(a[r].x, w.x, s);
                        s = fmaf(a[r].y, w.y, s);
                        s = fmaf(a[r].z, w.z, s);
                        acc[c][r] = fmaf(a[r].w, w.w, s);
                    }
                }
            }
        } else {
            for (int k = lane; k < kc; k += 32) {
#pragma unroll
                for (int c = 0; c < COLS; ++c) {
                    if (n0 + c >= N) break;
                    const float w = W[(size_t)(n0 + c) * K + k0 + k];
#pragma unroll
                    for (int r = 0; r < SK_ROWS; ++r) acc[c][r] = fmaf(As[r][k], w, acc[c][r]);
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < COLS; ++c)
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r) {
            const float s = warp_sum(acc[c][r]);
            if (lane == 0 && n0 + c < N && m0 + r < M) out[(size_t)(m0 + r) * N + n0 + c] = s;
        }
}
}  // namespace

MLS_API int mls_gemm_f32(const void* A, int a_dtype, const float* W, float* out, int M, int N,
                         int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (a_dtype != MLS_F32 && a_dtype != MLS_BF16) return MLS_ERR_UNSUPPORTED;
    if (N <= SKINNY_N) {
        // four entries of K at a time where every row of W starts at a 16-byte address
        const int by4 = K % 4 == 0 && reinterpret_cast<uintptr_t>(W) % 16 == 0;
        const int rows = (M + SK_ROWS - 1) / SK_ROWS;
        if (M >= 64)
            MLS_LAUNCH((gemm_f32_skinny_kernel<4>), dim3(rows, (N + 31) / 32), dim3(256), 0, stream,
                       A, a_dtype, W, out, M, N, K, by4);
        else
            MLS_LAUNCH((gemm_f32_skinny_kernel<1>), dim3(rows, (N + 7) / 8), dim3(256), 0, stream,
                       A, a_dtype, W, out, M, N, K, by4);
        return launch_status();
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    MLS_LAUNCH((gemm_f32_kernel), dim3(grid), dim3(256), 0, stream, A, a_dtype, W, out, M, N, K, N);
    return launch_status();
}
