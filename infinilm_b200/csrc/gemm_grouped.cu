// Matrix products over groups, C_g = A_g W_g^T with W_g [N,K] row-major, in two forms that share one kernel:
//   ragged:  the rows of A stand sorted by group, group g owning the places group_off[g] .. group_off[g+1]-1 (the
//            experts of a routed feed-forward); the row of A at a place may be named by a gather list (`a_rows`), the
//            row of C is the place. Tiles are dealt out over a bound on their number (places / BM + groups), the surplus leaves.
//   batched: every group has all M rows, and group g reads A, W and writes C at a fixed element offset g * stride
//            (one product per head over column ranges of shared rows).
// Epilogues: plain; GLU - W_g holds N gate rows and then N up rows, C = silu(gate) * up; gated - C is multiplied by
// sigmoid(G[m, g * gate_gs + n]). Products accumulate in f32 in the order of K whatever the tile, one accumulator per
// output element, so a row's result does not depend on what else is in the batch. float32 runs on the FP32 pipes
// (FFMA); bfloat16 inputs are widened to f32 in shared memory (exact) and run the same loop.
#include "common.cuh"

template <typename TA, bool GLU>
__global__ void __launch_bounds__(256) gemm_grouped_kernel(const TA* A, int lda, long long a_gs, const int* __restrict__ a_rows,
                                                           const TA* __restrict__ W, int ldw, long long w_gs, TA* __restrict__ C, int ldc,
                                                           long long c_gs, const int* __restrict__ group_off, int n_groups, int M, int N,
                                                           int K, const TA* gate, int ld_gate, long long gate_gs) {
    constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[GLU ? 2 : 1][BK][BN + 4];
    __shared__ int sh_g, sh_r0, sh_r1;
    const int tid = threadIdx.x;
    il_pdl_begin();
    int g, r0, r1;
    if (group_off) {
        if (tid == 0) {
            int tile = blockIdx.y, gg = 0, a = 0, b = 0;
            for (; gg < n_groups; ++gg) {
                a = group_off[gg];
                b = group_off[gg + 1];
                const int nt = (b - a + BM - 1) / BM;
                if (tile < nt) break;
                tile -= nt;
            }
            sh_g = gg;
            sh_r0 = a + tile * BM;
            sh_r1 = b;
        }
        __syncthreads();
        g = sh_g, r0 = sh_r0, r1 = sh_r1;
        if (g >= n_groups) return;
    } else {
        g = blockIdx.z, r0 = blockIdx.y * BM, r1 = M;
    }
    const int n0 = blockIdx.x * BN;
    const TA* Ag = A + (size_t)g * a_gs;
    const TA* Wg = W + (size_t)g * w_gs;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    float acc[TM][TN], acc2[GLU ? TM : 1][GLU ? TN : 1];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = 0.f;
            if (GLU) acc2[i][j] = 0.f;
        }
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int idx = tid; idx < BM * BK; idx += 256) {
            const int r = idx / BK, k = idx - r * BK;
            const int p = r0 + r, gk = k0 + k;
            float v = 0.f;
            if (p < r1 && gk < K) v = il_to_f(Ag[(size_t)(a_rows ? a_rows[p] : p) * lda + gk]);
            As[k][r] = v;
        }
        for (int idx = tid; idx < BN * BK; idx += 256) {
            const int r = idx / BK, k = idx - r * BK;
            const int gn = n0 + r, gk = k0 + k;
            const bool in = gn < N && gk < K;
            Ws[0][k][r] = in ? il_to_f(Wg[(size_t)gn * ldw + gk]) : 0.f;
            if (GLU) Ws[1][k][r] = in ? il_to_f(Wg[(size_t)(N + gn) * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN], b2[GLU ? TN : 1];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                b[j] = Ws[0][k][tx * TN + j];
                if (GLU) b2[j] = Ws[1][k][tx * TN + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (GLU) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
    TA* Cg = C + (size_t)g * c_gs;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int p = r0 + ty * TM + i;
        if (p >= r1) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (GLU) {
                // the gate and up products are rounded to the activation type first, as two separate products would be
                const float gt = il_to_f(il_from_f<TA>(v)), up = il_to_f(il_from_f<TA>(acc2[i][j]));
                v = gt / (1.f + expf(-gt)) * up;
            }
            if (gate) {
                const float gt = il_to_f(gate[(size_t)p * ld_gate + (size_t)g * gate_gs + gn]);
                v = il_to_f(il_from_f<TA>(v)) / (1.f + expf(-gt));
            }
            Cg[(size_t)p * ldc + gn] = il_from_f<TA>(v);
        }
    }
}

// The largest number of row tiles a ragged product of `M` places over `n_groups` groups can have.
IL_EXPORT int il_gemm_grouped_max_tiles(int M, int n_groups) { return (M + 63) / 64 + n_groups; }

IL_EXPORT int il_gemm_grouped(const void* A, int act_kind, int lda, long long a_gs, const int* a_rows, const void* W, int ldw, long long w_gs,
                              void* C, int ldc, long long c_gs, const int* group_off, int n_groups, int M, int N, int K, int glu,
                              const void* gate, int ld_gate, long long gate_gs, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || n_groups <= 0) return IL_OK;
    if (K <= 0 || (glu && gate)) return IL_BAD_ARG;
    dim3 grid((N + 63) / 64, group_off ? il_gemm_grouped_max_tiles(M, n_groups) : (M + 63) / 64, group_off ? 1 : n_groups);
    if (grid.y > 65535 || grid.z > 65535) return IL_UNSUPPORTED;
#define GG_LAUNCH(TA, G)                                                                                                                 \
    IL_LAUNCH((gemm_grouped_kernel<TA, G>), grid, 256, 0, stream, (const TA*)A, lda, a_gs, a_rows, (const TA*)W, ldw, w_gs, (TA*)C, ldc, \
              c_gs, group_off, n_groups, M, N, K, (const TA*)gate, ld_gate, gate_gs)
    if (act_kind == IL_F32) {
        if (glu) GG_LAUNCH(float, true); else GG_LAUNCH(float, false);
    } else if (act_kind == IL_BF16) {
        if (glu) GG_LAUNCH(__nv_bfloat16, true); else GG_LAUNCH(__nv_bfloat16, false);
    } else
        return IL_BAD_ARG;
#undef GG_LAUNCH
    IL_LAUNCH_CHECK();
    return IL_OK;
}
