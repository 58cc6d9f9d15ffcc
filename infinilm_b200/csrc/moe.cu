// Routing of a mixture-of-experts feed-forward, all on the device so that a step never waits for the host:
//   route:   per token, router logits z = W_r h + b in f32, the `top` largest chosen (ties: the lower expert), their
//            weights the softmax over the chosen logits alone; one warp a token, a fixed order of sums, so a token's
//            routing does not depend on what else is in the batch.
//   sort:    the (token, choice) slots ordered by expert: where each expert's rows start (`group_off`), the sorted place
//            of every slot (`pos_of_slot`) and the token whose row stands at every place (`row_of_pos`). One block.
//   combine: out[t] = sum over the token's choices, in the order of the choices, of weight * expert output row
//            (+ a row that is added for every token: the shared expert), summed in f32.
#include "common.cuh"

#define MOE_MAX_TOP 32

template <typename TA>
__global__ void __launch_bounds__(128) moe_route_kernel(const TA* x, int ldx, const TA* __restrict__ w, const void* __restrict__ bias, int b_kind,
                                                        int* __restrict__ idx, float* __restrict__ wt, int T, int H, int E, int top) {
    extern __shared__ float zs[];                 // [warps][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    il_pdl_begin();
    if (t >= T) return;
    float* z = zs + (size_t)warp * E;
    const TA* row = x + (size_t)t * ldx;
    for (int e = 0; e < E; ++e) {
        const TA* wr = w + (size_t)e * H;
        float s = 0.f;
        for (int h = lane; h < H; h += 32) s = fmaf(il_to_f(row[h]), il_to_f(wr[h]), s);
        s = il_warp_sum(s);
        if (lane == 0) z[e] = s + (bias ? il_load_any(bias, b_kind, e) : 0.f);
    }
    __syncwarp();
    float chosen_v[MOE_MAX_TOP];
    float vmax = 0.f, den = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > bv || (v == bv && e < bi)) bv = v, bi = e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
        }
        if (bi >= E) bi = 0;                      // every logit NaN: still a valid expert
        if (k == 0) vmax = bv;
        const float p = expf(bv - vmax);
        den += p;
        chosen_v[k] = p;
        if (lane == 0) {
            idx[(size_t)t * top + k] = bi;
            z[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0)
        for (int k = 0; k < top; ++k) wt[(size_t)t * top + k] = chosen_v[k] / den;
}

__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ idx, int n_slots, int top, int E, int* __restrict__ group_off,
                                                        int* __restrict__ pos_of_slot, int* __restrict__ row_of_pos) {
    extern __shared__ int sh[];                   // [E] counts, then [E] cursors
    int* cnt = sh;
    int* cur = sh + E;
    il_pdl_begin();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_slots; i += blockDim.x) {
        const int e = idx[i];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int a = 0;
        for (int e = 0; e < E; ++e) {
            group_off[e] = a;
            cur[e] = a;
            a += cnt[e];
        }
        group_off[E] = a;
    }
    __syncthreads();
    // the order of the rows inside an expert's range is whatever the atomics give: a row's result does not depend on it
    for (int i = threadIdx.x; i < n_slots; i += blockDim.x) {
        const int e = idx[i];
        if (e >= 0 && e < E) {
            const int p = atomicAdd(&cur[e], 1);
            pos_of_slot[i] = p;
            row_of_pos[p] = i / top;
        }
    }
}

template <typename TA>
__global__ void moe_combine_kernel(const TA* y, const int* pos_of_slot, const float* wt, const TA* shared_rows, TA* __restrict__ out,
                                   int H, int top) {
    const int t = blockIdx.x;
    il_pdl_begin();
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k)
            s = fmaf(wt[(size_t)t * top + k], il_to_f(y[(size_t)pos_of_slot[(size_t)t * top + k] * H + h]), s);
        if (shared_rows) s += il_to_f(shared_rows[(size_t)t * H + h]);
        out[(size_t)t * H + h] = il_from_f<TA>(s);
    }
}

IL_EXPORT int il_moe_route(const void* x, int act_kind, int ldx, const void* w, const void* bias, int b_kind, int* idx, float* wt, int T,
                           int H, int E, int top, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (H <= 0 || E <= 0 || top <= 0 || top > E || top > MOE_MAX_TOP) return IL_BAD_ARG;
    const int warps = 4;
    const size_t smem = (size_t)warps * E * sizeof(float);
    if (smem > 48 * 1024) return IL_UNSUPPORTED;
    if (act_kind == IL_F32)
        IL_LAUNCH(moe_route_kernel<float>, (T + warps - 1) / warps, warps * 32, smem, stream, (const float*)x, ldx, (const float*)w, bias, b_kind,
                  idx, wt, T, H, E, top);
    else if (act_kind == IL_BF16)
        IL_LAUNCH(moe_route_kernel<__nv_bfloat16>, (T + warps - 1) / warps, warps * 32, smem, stream, (const __nv_bfloat16*)x, ldx,
                  (const __nv_bfloat16*)w, bias, b_kind, idx, wt, T, H, E, top);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

IL_EXPORT int il_moe_sort(const int* idx, int n_slots, int top, int E, int* group_off, int* pos_of_slot, int* row_of_pos, cudaStream_t stream) {
    if (E <= 0 || top <= 0 || n_slots < 0) return IL_BAD_ARG;
    const size_t smem = (size_t)2 * E * sizeof(int);
    if (smem > 48 * 1024) return IL_UNSUPPORTED;
    IL_LAUNCH(moe_sort_kernel, 1, 1024, smem, stream, idx, n_slots, top, E, group_off, pos_of_slot, row_of_pos);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

IL_EXPORT int il_moe_combine(const void* y, int act_kind, const int* pos_of_slot, const float* wt, const void* shared_rows, void* out, int T,
                             int H, int top, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (H <= 0 || top <= 0) return IL_BAD_ARG;
    const int threads = H >= 1024 ? 256 : 128;
    if (act_kind == IL_F32)
        IL_LAUNCH(moe_combine_kernel<float>, T, threads, 0, stream, (const float*)y, pos_of_slot, wt, (const float*)shared_rows, (float*)out, H, top);
    else if (act_kind == IL_BF16)
        IL_LAUNCH(moe_combine_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)y, pos_of_slot, wt,
                  (const __nv_bfloat16*)shared_rows, (__nv_bfloat16*)out, H, top);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
