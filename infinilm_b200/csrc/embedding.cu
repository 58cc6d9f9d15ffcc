// Token embedding: gathers table rows, multiplies by the embedding scale in f32 and writes the
// f32 residual stream. With round_bf16 the product is rounded to bfloat16 first, which is the
// value a table pre-scaled in bfloat16 would hold.
#include "common.cuh"

template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table, float scale,
                             float* __restrict__ out, int H, int V, int round_bf16) {
    il_pdl_begin();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {  // the host rejects such ids before launch; never read out of range
        for (int h = threadIdx.x; h < H; h += blockDim.x) o[h] = __int_as_float(0x7fc00000);
        return;
    }
    const TW* row = table + (size_t)id * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float v = il_to_f(row[h]) * scale;
        if (round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
        o[h] = v;
    }
}

IL_EXPORT int il_embed(const int* ids, const void* table, int table_kind, float scale, float* out,
                       int T, int H, int V, int round_bf16, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (H <= 0 || V <= 0) return IL_BAD_ARG;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_kind == IL_F32)
        IL_LAUNCH(embed_kernel<float>, T, threads, 0, stream, ids, (const float*)table, scale, out, H, V, round_bf16);
    else if (table_kind == IL_BF16)
        IL_LAUNCH(embed_kernel<__nv_bfloat16>, T, threads, 0, stream, ids, (const __nv_bfloat16*)table, scale, out, H, V, round_bf16);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// token_ids[rows[i]] = src[src_idx[i]]: puts tokens that were sampled on the device (and not read by the host yet)
// into the next step's token list. Out-of-vocabulary values are caught by the gather above.
__global__ void patch_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ rows, const int* __restrict__ src_idx,
                                    const int* __restrict__ src, int n) {
    il_pdl_begin();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) token_ids[rows[i]] = src[src_idx[i]];
}

IL_EXPORT int il_patch_tokens(int* token_ids, const int* rows, const int* src_idx, const int* src, int n, cudaStream_t stream) {
    if (n <= 0) return IL_OK;
    IL_LAUNCH(patch_tokens_kernel, (n + 127) / 128, 128, 0, stream, token_ids, rows, src_idx, src, n);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// Token embedding with two additions, all summed in f32: a row of a second table chosen by a hash of (previous token,
// token) - the table's last row for a sequence's first token - and a sinusoidal position vector (entry 2i the sine,
// entry 2i+1 the cosine of pos * inv_freq[i]). Either addition is left out when its pointer is null.
// The previous token of an entry's first token comes from a per-request state word (`prev_state[slot]` holds token + 1,
// 0: none); the block of that first token reads it and then writes the entry's last token there, so the read of an entry
// always comes before its write, and no other block touches the slot.
template <typename TW>
__global__ void embed_pair_pos_kernel(const int* __restrict__ ids, const int* __restrict__ tok_pos, const int* __restrict__ tok_entry,
                                      const int* __restrict__ entry_qstart, const TW* __restrict__ table, float scale,
                                      const TW* __restrict__ pair_table, int buckets, long long mul_prev, long long mul_cur,
                                      int* prev_state, const int* __restrict__ read_slots, const int* __restrict__ write_slots,
                                      const float* __restrict__ inv_freq, float* __restrict__ out, int H, int V) {
    il_pdl_begin();
    __shared__ int sh_prev;
    const int t = blockIdx.x;
    const int id = ids[t], pos = tok_pos[t];
    float* o = out + (size_t)t * H;
    if (threadIdx.x == 0) {
        const int e = tok_entry[t], first = entry_qstart[e];
        int prev = -1;
        if (t == first) {
            if (prev_state) {
                prev = prev_state[read_slots[e]] - 1;
                if (write_slots) prev_state[write_slots[e]] = ids[entry_qstart[e + 1] - 1] + 1;
            }
        } else {
            prev = ids[t - 1];
        }
        sh_prev = pos == 0 ? -1 : prev;
    }
    __syncthreads();
    if (id < 0 || id >= V) {  // the host rejects such ids before launch; never read out of range
        for (int h = threadIdx.x; h < H; h += blockDim.x) o[h] = __int_as_float(0x7fc00000);
        return;
    }
    const TW* row = table + (size_t)id * H;
    const TW* pair = nullptr;
    if (pair_table) {
        const int prev = sh_prev;
        const long long r = (prev < 0 || prev >= V) ? (long long)buckets : ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
        pair = pair_table + (size_t)r * H;
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float v = il_to_f(row[h]) * scale;
        if (pair) v += il_to_f(pair[h]);
        if (inv_freq) {
            const float ang = (float)pos * inv_freq[h >> 1];
            v += (h & 1) ? cosf(ang) : sinf(ang);
        }
        o[h] = v;
    }
}

IL_EXPORT int il_embed_pair_pos(const int* ids, const int* tok_pos, const int* tok_entry, const int* entry_qstart, const void* table,
                                int table_kind, float scale, const void* pair_table, int buckets, long long mul_prev, long long mul_cur,
                                int* prev_state, const int* read_slots, const int* write_slots, const float* inv_freq, float* out,
                                int T, int H, int V, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (H <= 0 || V <= 0 || (pair_table && buckets <= 0) || (prev_state && !read_slots)) return IL_BAD_ARG;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_kind == IL_F32)
        IL_LAUNCH(embed_pair_pos_kernel<float>, T, threads, 0, stream, ids, tok_pos, tok_entry, entry_qstart, (const float*)table, scale,
                  (const float*)pair_table, buckets, mul_prev, mul_cur, prev_state, read_slots, write_slots, inv_freq, out, H, V);
    else if (table_kind == IL_BF16)
        IL_LAUNCH(embed_pair_pos_kernel<__nv_bfloat16>, T, threads, 0, stream, ids, tok_pos, tok_entry, entry_qstart,
                  (const __nv_bfloat16*)table, scale, (const __nv_bfloat16*)pair_table, buckets, mul_prev, mul_cur, prev_state, read_slots,
                  write_slots, inv_freq, out, H, V);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
