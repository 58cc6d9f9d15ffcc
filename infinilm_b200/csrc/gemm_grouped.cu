// Matrix products over groups, C_g = A_g W_g^T with W_g [N,K] row-major, in two forms that share one kernel:
//   ragged:  the rows of A stand sorted by group, group g owning the places group_off[g] .. group_off[g+1]-1 (the
//            experts of a routed feed-forward); the row of A at a place may be named by a gather list (`a_rows`), the
//            row of C is the place. Tiles are dealt out over a bound on their number (places / BM + groups), the surplus leaves.
//   batched: every group has all M rows, and group g reads A, W and writes C at a fixed element offset g * stride
//            (one product per head over column ranges of shared rows).
// Epilogues: plain; GLU - W_g holds N gate rows and then N up rows, C = silu(gate) * up; gated - C is multiplied by
// sigmoid(G[m, g * gate_gs + n]). Products accumulate in f32 in the order of K whatever the tile, one accumulator per
// output element, so a row's result does not depend on what else is in the batch. float32 runs on the FP32 pipes
// (FFMA); bfloat16 runs on the tensor cores (mma.sync m16n8k16, operands staged by cp.async in a three-stage ring: a
// block streams a tile of 64 weight rows over all of K once, against up to 32 rows of its group, which is what a decode
// step's few rows per expert need - the weights of the experts that were chosen are read once, at the rate the memory
// gives); bfloat16 operands that are not 16-byte aligned are widened to f32 in shared memory (exact) and run the FFMA loop.
#include "common.cuh"

// ---- bfloat16 on the tensor cores ---------------------------------------------------------------------------------
namespace ggm {
constexpr int BN = 64, BK = 64, STAGES = 3, ROW = BK * 2 + 16;      // a tile row: 64 bfloat16 and 16 bytes of padding (ldmatrix bank spread)
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src)); }
__device__ __forceinline__ void zero16(uint32_t dst) { asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(dst), "r"(0u)); }
__device__ __forceinline__ void commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <int BM, bool GLU> constexpr int smem_bytes() { return STAGES * (BM + (GLU ? 2 : 1) * BN) * ROW; }
}  // namespace ggm

template <int BM, bool GLU>
__global__ void __launch_bounds__(128) gemm_grouped_mma_kernel(const __nv_bfloat16* A, int lda, long long a_gs, const int* __restrict__ a_rows,
                                                               const __nv_bfloat16* __restrict__ W, int ldw, long long w_gs,
                                                               __nv_bfloat16* __restrict__ C, int ldc, long long c_gs,
                                                               const int* __restrict__ group_off, int n_groups, int M, int N, int K,
                                                               const __nv_bfloat16* gate, int ld_gate, long long gate_gs, const float* row_scale) {
    using namespace ggm;
    constexpr int MT = BM / 16, NW = GLU ? 2 : 1;
    constexpr int A_BYTES = BM * ROW, W_BYTES = BN * ROW, STAGE_BYTES = A_BYTES + NW * W_BYTES;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int sh_g, sh_r0, sh_r1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int g, r0, r1;
    if (group_off) {                              // (the groups' ranges come from the sort kernel before this one)
        il_pdl_begin();
        if (tid == 0) {
            int tile = blockIdx.y, gg = 0, a = 0, b = 0;
            for (; gg < n_groups; ++gg) {
                a = group_off[gg];
                b = group_off[gg + 1];
                const int nt = (b - a + BM - 1) / BM;
                if (tile < nt) break;
                tile -= nt;
            }
            sh_g = gg, sh_r0 = a + tile * BM, sh_r1 = b;
        }
        __syncthreads();
        g = sh_g, r0 = sh_r0, r1 = sh_r1;
        if (g >= n_groups) return;
    } else {
        g = blockIdx.z, r0 = blockIdx.y * BM, r1 = M;
        il_pdl_begin();
    }
    const int n0 = blockIdx.x * BN;
    const __nv_bfloat16* Ag = A + (size_t)g * a_gs;
    const __nv_bfloat16* Wg = W + (size_t)g * w_gs;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);

    // what this thread copies per stage: chunks of 16 bytes, chunk c of row r at tile + r * ROW + c * 16
    constexpr int A_CH = BM * 8 / 128, W_CH = NW * BN * 8 / 128;
    const __nv_bfloat16* a_src[A_CH];
    const __nv_bfloat16* w_src[W_CH];
#pragma unroll
    for (int i = 0; i < A_CH; ++i) {
        const int ch = tid + i * 128, r = ch >> 3, p = r0 + r;
        a_src[i] = p < r1 ? Ag + (size_t)(a_rows ? a_rows[p] : p) * lda + (ch & 7) * 8 : nullptr;
    }
#pragma unroll
    for (int i = 0; i < W_CH; ++i) {
        const int ch = tid + i * 128, r = ch >> 3, half = r / BN, gn = n0 + (r - half * BN);
        w_src[i] = gn < N ? Wg + (size_t)(half * N + gn) * ldw + (ch & 7) * 8 : nullptr;
    }
    const int n_kb = (K + BK - 1) / BK;
    auto issue = [&](int kb) {
        if (kb < n_kb) {
            const uint32_t st = sbase + (kb % STAGES) * STAGE_BYTES;
            const int k0 = kb * BK;
#pragma unroll
            for (int i = 0; i < A_CH; ++i) {
                const int ch = tid + i * 128;
                const uint32_t dst = st + (ch >> 3) * ROW + (ch & 7) * 16;
                if (a_src[i] && k0 + (ch & 7) * 8 < K) cp16(dst, a_src[i] + k0); else zero16(dst);
            }
#pragma unroll
            for (int i = 0; i < W_CH; ++i) {
                const int ch = tid + i * 128;
                const uint32_t dst = st + A_BYTES + (ch >> 3) * ROW + (ch & 7) * 16;
                if (w_src[i] && k0 + (ch & 7) * 8 < K) cp16(dst, w_src[i] + k0); else zero16(dst);
            }
        }
        commit();
    };
    float acc[MT][2][4], acc2[GLU ? MT : 1][2][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                acc[i][j][k] = 0.f;
                if (GLU) acc2[i][j][k] = 0.f;
            }
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) issue(s);
    const int mat = lane >> 3, rr = lane & 7;
    const uint32_t a_off = ((mat & 1) * 8 + rr) * ROW + (mat >> 1) * 16;                       // A fragment: rows (mat&1)*8.., k (mat>>1)*8..
    const uint32_t b_off = A_BYTES + (warp * 16 + (mat >> 1) * 8 + rr) * ROW + (mat & 1) * 16; // B fragment: weight rows (mat>>1)*8.., k (mat&1)*8..
    for (int kb = 0; kb < n_kb; ++kb) {
        wait<STAGES - 2>();
        __syncthreads();                          // stage kb has landed for everyone, and everyone is done with stage kb - 1
        issue(kb + STAGES - 1);
        const uint32_t st = sbase + (kb % STAGES) * STAGE_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            uint32_t b[4], b2[4];
            ldsm4(b[0], b[1], b[2], b[3], st + b_off + kk * 32);
            if (GLU) ldsm4(b2[0], b2[1], b2[2], b2[3], st + b_off + W_BYTES + kk * 32);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t a[4];
                ldsm4(a[0], a[1], a[2], a[3], st + a_off + mt * 16 * ROW + kk * 32);
                mma(acc[mt][0], a, b[0], b[1]);
                mma(acc[mt][1], a, b[2], b[3]);
                if (GLU) {
                    mma(acc2[mt][0], a, b2[0], b2[1]);
                    mma(acc2[mt][1], a, b2[2], b2[3]);
                }
            }
        }
    }
    wait<0>();
    il_pdl_tail();
    __nv_bfloat16* Cg = C + (size_t)g * c_gs;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int p = r0 + mt * 16 + (lane >> 2) + 8 * h;
            if (p >= r1) continue;
            // a factor per source row (the rstd of a norm that the rows of A have not been divided by yet)
            const float rs = row_scale ? row_scale[a_rows ? a_rows[p] : p] : 1.f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                float out2[2];
                const int gn0 = n0 + warp * 16 + nt * 8 + (lane & 3) * 2;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int gn = gn0 + c;
                    float v = acc[mt][nt][2 * h + c] * rs;
                    if (gn < N) {
                        if (GLU) {
                            const float gt = __bfloat162float(__float2bfloat16_rn(v)), up = __bfloat162float(__float2bfloat16_rn(acc2[mt][nt][2 * h + c] * rs));
                            v = gt / (1.f + expf(-gt)) * up;
                        }
                        if (gate) {
                            const float gt = __bfloat162float(gate[(size_t)p * ld_gate + (size_t)g * gate_gs + gn]);
                            v = __bfloat162float(__float2bfloat16_rn(v)) / (1.f + expf(-gt));
                        }
                    }
                    out2[c] = v;
                }
                __nv_bfloat16* dst = Cg + (size_t)p * ldc + gn0;
                if (gn0 + 1 < N && !((uintptr_t)dst & 3)) {       // a pair of neighbouring columns in one 4-byte store
                    *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(out2[0], out2[1]);
                } else {
                    if (gn0 < N) dst[0] = __float2bfloat16_rn(out2[0]);
                    if (gn0 + 1 < N) dst[1] = __float2bfloat16_rn(out2[1]);
                }
            }
        }
}

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

template <int BM, bool GLU>
static int launch_mma(const void* A, int lda, long long a_gs, const int* a_rows, const void* W, int ldw, long long w_gs, void* C, int ldc,
                      long long c_gs, const int* group_off, int n_groups, int M, int N, int K, const void* gate, int ld_gate, long long gate_gs,
                      const float* row_scale, cudaStream_t stream) {
    constexpr int smem = ggm::smem_bytes<BM, GLU>();
    static bool attr_set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_grouped_mma_kernel<BM, GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return 1000 + (int)e;
        attr_set[dev] = true;
    }
    dim3 grid((N + ggm::BN - 1) / ggm::BN, group_off ? (M + BM - 1) / BM + n_groups : (M + BM - 1) / BM, group_off ? 1 : n_groups);
    if (grid.y > 65535 || grid.z > 65535) return IL_UNSUPPORTED;
    IL_LAUNCH((gemm_grouped_mma_kernel<BM, GLU>), grid, 128, smem, stream, (const __nv_bfloat16*)A, lda, a_gs, a_rows, (const __nv_bfloat16*)W, ldw,
              w_gs, (__nv_bfloat16*)C, ldc, c_gs, group_off, n_groups, M, N, K, (const __nv_bfloat16*)gate, ld_gate, gate_gs, row_scale);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

IL_EXPORT int il_gemm_grouped(const void* A, int act_kind, int lda, long long a_gs, const int* a_rows, const void* W, int ldw, long long w_gs,
                              void* C, int ldc, long long c_gs, const int* group_off, int n_groups, int M, int N, int K, int glu,
                              const void* gate, int ld_gate, long long gate_gs, const float* row_scale, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || n_groups <= 0) return IL_OK;
    if (K <= 0 || (glu && gate)) return IL_BAD_ARG;
    if (act_kind == IL_BF16 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && a_gs % 8 == 0 && w_gs % 8 == 0 && !((uintptr_t)A & 15) &&
        !((uintptr_t)W & 15)) {
        // rows of 16-byte chunks: the tensor-core kernel. Few rows a group (a decode step): tiles of 32 rows; else 64.
        const bool few = group_off ? M <= 32 * n_groups : M <= 32;
        if (glu)
            return few ? launch_mma<32, true>(A, lda, a_gs, a_rows, W, ldw, w_gs, C, ldc, c_gs, group_off, n_groups, M, N, K, gate, ld_gate, gate_gs, row_scale, stream)
                       : launch_mma<64, true>(A, lda, a_gs, a_rows, W, ldw, w_gs, C, ldc, c_gs, group_off, n_groups, M, N, K, gate, ld_gate, gate_gs, row_scale, stream);
        return few ? launch_mma<32, false>(A, lda, a_gs, a_rows, W, ldw, w_gs, C, ldc, c_gs, group_off, n_groups, M, N, K, gate, ld_gate, gate_gs, row_scale, stream)
                   : launch_mma<64, false>(A, lda, a_gs, a_rows, W, ldw, w_gs, C, ldc, c_gs, group_off, n_groups, M, N, K, gate, ld_gate, gate_gs, row_scale, stream);
    }
    if (row_scale) return IL_UNSUPPORTED;         // a factor per row: the tensor-core kernel's epilogue only
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
