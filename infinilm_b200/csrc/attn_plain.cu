// Plain attention over the paged cache: one warp per (token, query head), keys visited one by
// one with an online softmax in f32. It takes any mix of prompt portions and single decoded
// tokens, any head size up to 1024, any number of heads and groups, and an optional window.
// It is the attention of the 32-bit path and the reference beside the fast bfloat16 kernels.
// With `sink` (one f32 number per query head) the softmax's denominator also holds exp(sink[head]): a key without a
// value whose score is the number itself, not multiplied by `scale`.
//
// The query of token t is at absolute position p = tok_pos[t] of its request and sees cache
// positions max(0, p - window + 1) .. p (window <= 0: all). Query head j reads kv head j / (nh / nkv).
// With `dist_bias` (f32 [dist_far + 1][heads]) the scaled score of a key n positions back gets dist_bias[min(n, dist_far)][head]
// added: a learned bias by distance that is constant from dist_far on.
#include "common.cuh"

// A lane holds head_dim / 32 elements of the query and of the output: 8 (head_dim <= 256) or 32 (<= 1024).
template <typename TA, int AP_MAX_PER_LANE>
__global__ void attn_plain_kernel(const TA* __restrict__ qkv, int row_stride, TA* __restrict__ out,
                                  const TA* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
                                  const int* __restrict__ tok_pos, const int* __restrict__ tok_entry, int page_size,
                                  int nh, int nkv, int hd, float scale, int window, const float* __restrict__ sink,
                                  const float* __restrict__ dist_bias, int dist_far) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.y * (blockDim.x >> 5) + warp;
    const int t = blockIdx.x;
    if (j >= nh) return;
    const int g = j / (nh / nkv);
    const int pos = tok_pos[t];
    const int* bt = block_table + (size_t)tok_entry[t] * bt_stride;
    const int lo = il_mask_lo(pos, window);

    float q[AP_MAX_PER_LANE], acc[AP_MAX_PER_LANE];
    const TA* qrow = qkv + (size_t)t * row_stride + (size_t)j * hd;
#pragma unroll
    for (int r = 0; r < AP_MAX_PER_LANE; ++r) {
        const int d = lane + 32 * r;
        q[r] = d < hd ? il_to_f(qrow[d]) : 0.f;
        acc[r] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const size_t page_elems = (size_t)2 * nkv * page_size * hd;
    for (int kp = lo; kp <= pos; ++kp) {
        const int page = bt[kp / page_size];
        const TA* krow = cache + (size_t)page * page_elems + ((size_t)g * page_size + kp % page_size) * hd;
        const TA* vrow = krow + (size_t)nkv * page_size * hd;
        float dot = 0.f;
#pragma unroll
        for (int r = 0; r < AP_MAX_PER_LANE; ++r) {
            const int d = lane + 32 * r;
            if (d < hd) dot += q[r] * il_to_f(krow[d]);
        }
        dot = il_warp_sum(dot) * scale;
        if (dist_bias) dot += dist_bias[(size_t)min(pos - kp, dist_far) * nh + j];
        const float mn = fmaxf(m, dot);
        const float corr = expf(m - mn);  // exp(-inf) = 0 on the first key
        const float p = expf(dot - mn);
        l = l * corr + p;
#pragma unroll
        for (int r = 0; r < AP_MAX_PER_LANE; ++r) {
            const int d = lane + 32 * r;
            if (d < hd) acc[r] = acc[r] * corr + p * il_to_f(vrow[d]);
        }
        m = mn;
    }
    TA* orow = out + (size_t)t * nh * hd + (size_t)j * hd;
    if (sink) l += expf(sink[j] - m);             // (+inf when the sink towers over every score: the row is then zero)
    const float inv = 1.f / l;
#pragma unroll
    for (int r = 0; r < AP_MAX_PER_LANE; ++r) {
        const int d = lane + 32 * r;
        if (d < hd) orow[d] = il_from_f<TA>(acc[r] * inv);
    }
}

IL_EXPORT int il_attn_plain(const void* qkv, int act_kind, int row_stride, void* out, const void* cache,
                            const int* block_table, int bt_stride, const int* tok_pos, const int* tok_entry,
                            int page_size, int T, int nh, int nkv, int hd, float scale, int window,
                            const float* sink, const float* dist_bias, int dist_far, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (dist_bias && dist_far < 0) return IL_BAD_ARG;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || page_size <= 0) return IL_BAD_ARG;
    if (hd > 1024) return IL_UNSUPPORTED;
    const int warps = 4;
    dim3 grid(T, (nh + warps - 1) / warps);
#define AP_LAUNCH(TA, N)                                                                                                                \
    attn_plain_kernel<TA, N><<<grid, warps * 32, 0, stream>>>((const TA*)qkv, row_stride, (TA*)out, (const TA*)cache, block_table, bt_stride, \
                                                              tok_pos, tok_entry, page_size, nh, nkv, hd, scale, window, sink, dist_bias, dist_far)
    if (act_kind == IL_F32) {
        if (hd <= 256) AP_LAUNCH(float, 8); else AP_LAUNCH(float, 32);
    } else if (act_kind == IL_BF16) {
        if (hd <= 256) AP_LAUNCH(__nv_bfloat16, 8); else AP_LAUNCH(__nv_bfloat16, 32);
    } else
        return IL_BAD_ARG;
#undef AP_LAUNCH
    IL_LAUNCH_CHECK();
    return IL_OK;
}
