// True 32-bit matrix product for the float32 path: out[M, N] = A[M, K] * W[N, K]^T.
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
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ out,
                int M, int N, int K, int ldo) {
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
            As[lk + e][lrow] = (am < M && k < K) ? A[(size_t)am * K + k] : 0.f;
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
// Here a block holds SK_ROWS rows of A in shared memory, each of its eight warps owns one of
// eight output columns (blockIdx.y names the eight) and its lanes walk K with a stride of 32;
// the 32 partial sums are added by a fixed tree.  The order of the additions depends on K alone (never on M or on
// the row's place in its block), and which kernel runs depends on N alone, so a token's
// result still does not depend on its batch.
constexpr int SKINNY_N = 64, SK_ROWS = 8, SK_KC = 1024;

__global__ void __launch_bounds__(256)
gemm_f32_skinny_kernel(const float* __restrict__ A, const float* __restrict__ W,
                       float* __restrict__ out, int M, int N, int K) {
    chain_release();
    chain_wait();
    __shared__ float As[SK_ROWS][SK_KC];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * SK_ROWS;
    {
        const int n = blockIdx.y * 8 + warp;
        float acc[SK_ROWS];
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r) acc[r] = 0.f;
        for (int k0 = 0; k0 < K; k0 += SK_KC) {
            const int kc = min(SK_KC, K - k0);
            __syncthreads();
            for (int i = threadIdx.x; i < SK_ROWS * kc; i += 256) {
                const int r = i / kc, k = i - r * kc;
                As[r][k] = m0 + r < M ? A[(size_t)(m0 + r) * K + k0 + k] : 0.f;
            }
            __syncthreads();
            if (n < N) {
                const float* wr = W + (size_t)n * K + k0;
                for (int k = lane; k < kc; k += 32) {
                    const float w = wr[k];
#pragma unroll
                    for (int r = 0; r < SK_ROWS; ++r) acc[r] = fmaf(As[r][k], w, acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r) {
            const float s = warp_sum(acc[r]);
            if (lane == 0 && n < N && m0 + r < M) out[(size_t)(m0 + r) * N + n] = s;
        }
    }
}
}  // namespace

MLS_API int mls_gemm_f32(const float* A, const float* W, float* out, int M, int N, int K,
                         cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (N <= SKINNY_N) {
        MLS_LAUNCH((gemm_f32_skinny_kernel), dim3((M + SK_ROWS - 1) / SK_ROWS, (N + 7) / 8),
                   dim3(256), 0, stream, A, W, out, M, N, K);
        return launch_status();
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    MLS_LAUNCH((gemm_f32_kernel), dim3(grid), dim3(256), 0, stream, A, W, out, M, N, K, N);
    return launch_status();
}
