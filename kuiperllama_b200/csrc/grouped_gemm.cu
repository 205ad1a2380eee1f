// Many small matrix products in one launch: C_g = A_g W_g^T for groups g that each have weights of
// their own, [N, K] row-major as everywhere in this package.  Two ways to say which rows belong to
// which group:
//
//   * batched (tile_group == null): every group takes all M rows; group g reads the columns of A that
//     start at g * a_gs and writes the columns of C that start at g * c_gs.  This is a per-head
//     projection ([tokens, heads, k] x [heads, n, k]) or a block-diagonal matrix.
//   * routed (tile_group given): the rows are positions of a list that is sorted by group and padded
//     so that every tile of BM rows lies in one group; tile_group[tile] names it (-1: no rows) and
//     a_rows[position] the row of A to read (-1: padding; null: the position itself).  This is a
//     mixture of experts: the list holds (token, choice) pairs.
//
// Epilogues: plain, or a gated activation over weights that hold N gate rows followed by N up rows:
//     g = min(gate, limit), u = clamp(up, -limit, limit) (no clamp when limit <= 0),
//     y = g * sigmoid(alpha * g) * (u + shift).
// Arithmetic is 32-bit FMA for both dtypes; every output is one thread's sum in ascending k, so a row's
// result does not depend on which other rows share its tile.  ExiledOfCode/KuiperLLama has single
// products alone (matmul_kernel.cu:6-54).
#include "common.cuh"

namespace kl {

constexpr int GG_BN = 64, GG_BK = 16, GG_THREADS = 256;
enum : int { GG_PLAIN = 0, GG_GATED = 1 };

template <typename TI, typename TO, int BM, int EPI>
__global__ void __launch_bounds__(GG_THREADS)
grouped_gemm_kernel(const TI* __restrict__ A, long long lda, long long a_gs, const int* __restrict__ a_rows,
                    const TI* __restrict__ W, long long w_gs, TO* __restrict__ C, long long ldc, long long c_gs,
                    const int* __restrict__ tile_group, int M, int N, int K, float limit, float alpha, float shift) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int RM = BM / 16;                                   // rows per thread
    __shared__ float As[GG_BK][BM + 4];
    __shared__ float Ws[EPI == GG_GATED ? 2 : 1][GG_BK][GG_BN + 4];
    __shared__ int src[BM];
    const int g = tile_group ? tile_group[blockIdx.y] : (int)blockIdx.z;
    if (g < 0) return;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * GG_BN;
    for (int i = threadIdx.x; i < BM; i += GG_THREADS) {
        const int m = m0 + i;
        src[i] = m < M ? (a_rows ? a_rows[m] : m) : -1;
    }
    __syncthreads();
    const TI* Ag = A + (size_t)g * a_gs;
    const TI* Wg = W + (size_t)g * w_gs;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[EPI == GG_GATED ? 2 : 1][RM][4];
#pragma unroll
    for (int z = 0; z < (EPI == GG_GATED ? 2 : 1); ++z)
#pragma unroll
        for (int i = 0; i < RM; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[z][i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GG_BK) {
        for (int e = threadIdx.x; e < BM * GG_BK; e += GG_THREADS) {
            const int row = e / GG_BK, kk = e % GG_BK, gk = k0 + kk;
            const int s = src[row];
            As[kk][row] = (s >= 0 && gk < K) ? to_f32(Ag[(size_t)s * lda + gk]) : 0.f;
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = threadIdx.x + r * GG_THREADS;
            const int row = e / GG_BK, kk = e % GG_BK, gn = n0 + row, gk = k0 + kk;
            const bool ok = gn < N && gk < K;
            Ws[0][kk][row] = ok ? to_f32(Wg[(size_t)gn * K + gk]) : 0.f;
            if (EPI == GG_GATED) Ws[1][kk][row] = ok ? to_f32(Wg[(size_t)(N + gn) * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            float a[RM];
#pragma unroll
            for (int i = 0; i < RM; ++i) a[i] = As[kk][ty * RM + i];
#pragma unroll
            for (int z = 0; z < (EPI == GG_GATED ? 2 : 1); ++z) {
                float b[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Ws[z][kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < RM; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[z][i][j] = fmaf(a[i], b[j], acc[z][i][j]);
            }
        }
        __syncthreads();
    }
    TO* Cg = C + (size_t)g * c_gs;
#pragma unroll
    for (int i = 0; i < RM; ++i) {
        const int row = ty * RM + i;
        if (src[row] < 0) continue;
        TO* crow = Cg + (size_t)(m0 + row) * ldc;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float y = acc[0][i][j];
            if (EPI == GG_GATED) {
                float gt = y, up = acc[1][i][j];
                if (limit > 0.f) { gt = fminf(gt, limit); up = fminf(fmaxf(up, -limit), limit); }
                y = gt / (1.0f + expf(-alpha * gt)) * (up + shift);
            }
            crow[gn] = from_f32<TO>(y);
        }
    }
}

}  // namespace kl

using namespace kl;

// groups: the number of groups of a batched call (ignored for a routed one, whose tile_group has
// `tiles` entries).  gated: 0 plain (W_g is [N, K]), 1 gated activation (W_g is [2 N, K]).
KL_API int kl_grouped_gemm(const void* A, long long lda, long long a_gs, const int* a_rows, const void* W, long long w_gs,
                           void* C, long long ldc, long long c_gs, const int* tile_group, int tiles, int tile_rows, int groups,
                           int M, int N, int K, int gated, float limit, float alpha, float shift, int in_dtype, int out_dtype,
                           cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KL_OK;
    if (K <= 0 || (tile_rows != 16 && tile_rows != 64)) return KL_ERR_BAD_SIZE;
    const int my = tile_group ? tiles : (M + tile_rows - 1) / tile_rows;
    const int gz = tile_group ? 1 : groups;
    if (my <= 0 || gz <= 0) return KL_OK;
    if (my > 65535 || gz > 65535) return KL_ERR_BAD_SIZE;
    const dim3 grid((N + GG_BN - 1) / GG_BN, my, gz);
#define KL_GG(TI, TO, BM, EPI)                                                                                              \
    launch_kernel(grouped_gemm_kernel<TI, TO, BM, EPI>, grid, GG_THREADS, 0, stream, (const TI*)A, lda, a_gs, a_rows,         \
                  (const TI*)W, w_gs, (TO*)C, ldc, c_gs, tile_group, M, N, K, limit, alpha, shift)
#define KL_GG_BY(TI, TO)                                                                                                    \
    do {                                                                                                                    \
        if (tile_rows == 16) { if (gated) KL_GG(TI, TO, 16, GG_GATED); else KL_GG(TI, TO, 16, GG_PLAIN); }                  \
        else { if (gated) KL_GG(TI, TO, 64, GG_GATED); else KL_GG(TI, TO, 64, GG_PLAIN); }                                  \
    } while (0)
    if (in_dtype == KL_F32 && out_dtype == KL_F32) KL_GG_BY(float, float);
    else if (in_dtype == KL_BF16 && out_dtype == KL_BF16) KL_GG_BY(bf16, bf16);
    else if (in_dtype == KL_BF16 && out_dtype == KL_F32) KL_GG_BY(bf16, float);
    else return KL_ERR_BAD_DTYPE;
#undef KL_GG_BY
#undef KL_GG
    KL_LAUNCH_CHECK();
    return KL_OK;
}
