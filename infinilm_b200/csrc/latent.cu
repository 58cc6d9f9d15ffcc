// The latent rows of a latent-attention mixer after their joint down-projection: per token, segment A of the projected
// row (the query latent) and segment B (the key/value latent) are each divided by their root mean square
// (x / sqrt(mean(x^2) + eps), f32) and multiplied by a weight vector. A goes to a row buffer for the query's
// up-projection; B - the only thing the mixer keeps of a token - is written to the token's slot of the paged cache,
// into the K plane and the V plane alike (the attention kernels read keys and values from the two planes; here they are
// the same vectors), and optionally to a row buffer.
// Cache layout of one layer: [page][0=K,1=V][kv head = 1][slot in page][width of B].
#include "common.cuh"

template <typename TA>
__global__ void latent_norm_store_kernel(const TA* proj, int row_stride, int off_a, int n_a, int off_b, int n_b,
                                         const void* __restrict__ w_a, const void* __restrict__ w_b, int w_kind, float eps,
                                         TA* __restrict__ out_a, TA* __restrict__ out_b, const int* __restrict__ tok_pos,
                                         const int* __restrict__ tok_entry, const int* __restrict__ block_table, int bt_stride,
                                         TA* __restrict__ cache, int page_size) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    TA* kdst = nullptr;
    size_t plane = 0;
    if (cache) {
        const int page = block_table[(size_t)tok_entry[t] * bt_stride + pos / page_size];
        if (page >= 0) {                          // the host reserves every page a step touches; never write elsewhere
            plane = (size_t)page_size * n_b;
            kdst = cache + (size_t)page * 2 * plane + (size_t)(pos % page_size) * n_b;
        }
    }
    il_pdl_begin();
    const TA* row = proj + (size_t)t * row_stride;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < n_a; i += blockDim.x) {
        const float x = il_to_f(row[off_a + i]);
        sa += x * x;
    }
    for (int i = threadIdx.x; i < n_b; i += blockDim.x) {
        const float x = il_to_f(row[off_b + i]);
        sb += x * x;
    }
    sa = il_block_sum(sa, red);
    sb = il_block_sum(sb, red);
    const float ra = n_a > 0 ? rsqrtf(sa / (float)n_a + eps) : 0.f, rb = rsqrtf(sb / (float)n_b + eps);
    for (int i = threadIdx.x; i < n_a; i += blockDim.x)
        out_a[(size_t)t * n_a + i] = il_from_f<TA>(il_to_f(row[off_a + i]) * ra * il_load_any(w_a, w_kind, i));
    for (int i = threadIdx.x; i < n_b; i += blockDim.x) {
        const TA v = il_from_f<TA>(il_to_f(row[off_b + i]) * rb * il_load_any(w_b, w_kind, i));
        if (out_b) out_b[(size_t)t * n_b + i] = v;
        if (kdst) {
            kdst[i] = v;
            kdst[plane + i] = v;
        }
    }
}

IL_EXPORT int il_latent_norm_store(const void* proj, int act_kind, int row_stride, int off_a, int n_a, int off_b, int n_b, const void* w_a,
                                   const void* w_b, int w_kind, float eps, void* out_a, void* out_b, const int* tok_pos,
                                   const int* tok_entry, const int* block_table, int bt_stride, void* cache, int page_size, int T,
                                   cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (n_b <= 0 || n_a < 0 || page_size <= 0 || (n_a > 0 && !out_a)) return IL_BAD_ARG;
    const int threads = (n_a + n_b) >= 1024 ? 256 : 128;
    if (act_kind == IL_F32)
        IL_LAUNCH(latent_norm_store_kernel<float>, T, threads, 0, stream, (const float*)proj, row_stride, off_a, n_a, off_b, n_b, w_a, w_b,
                  w_kind, eps, (float*)out_a, (float*)out_b, tok_pos, tok_entry, block_table, bt_stride, (float*)cache, page_size);
    else if (act_kind == IL_BF16)
        IL_LAUNCH(latent_norm_store_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)proj, row_stride, off_a, n_a, off_b,
                  n_b, w_a, w_b, w_kind, eps, (__nv_bfloat16*)out_a, (__nv_bfloat16*)out_b, tok_pos, tok_entry, block_table, bt_stride,
                  (__nv_bfloat16*)cache, page_size);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// y[t, c] *= sigmoid(g[t, c]) for rows of `n` columns (y contiguous, g with a row stride): the heads' gate where the product
// before it was the library's and has no epilogue of ours.
template <typename TA>
__global__ void sigmoid_gate_kernel(TA* y, const TA* g, int ldg, int n, long long total) {
    il_pdl_begin();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / n;
        const int c = (int)(i - t * n);
        const float gt = il_to_f(g[(size_t)t * ldg + c]);
        y[i] = il_from_f<TA>(il_to_f(y[i]) / (1.f + expf(-gt)));
    }
}

IL_EXPORT int il_sigmoid_gate(void* y, int act_kind, const void* g, int ldg, int T, int n, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return IL_OK;
    const long long total = (long long)T * n;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    if (act_kind == IL_F32)
        IL_LAUNCH(sigmoid_gate_kernel<float>, blocks, 256, 0, stream, (float*)y, (const float*)g, ldg, n, total);
    else if (act_kind == IL_BF16)
        IL_LAUNCH(sigmoid_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)y, (const __nv_bfloat16*)g, ldg, n, total);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
