// Routing of a mixture-of-experts feed-forward, all on the device so that a step never waits for the host:
//   route:   per token, router logits z = W_r h + b in f32, the `top` largest chosen (ties: the lower expert), their
//            weights the softmax over the chosen logits alone; a fixed order of sums, so a token's routing does not
//            depend on what else is in the batch.
//   sort:    the (token, choice) slots ordered by expert: where each expert's rows start (`group_off`), the sorted place
//            of every slot (`pos_of_slot`) and the token whose row stands at every place (`row_of_pos`). One block.
//   combine: out[t] = sum over the token's choices, in the order of the choices, of weight * expert output row
//            (+ a row that is added for every token: the shared expert), summed in f32.
#include "common.cuh"

#define MOE_MAX_TOP 32

// Eight f32 values of a row from 16 bytes of bfloat16, or from two 16-byte loads of float32.
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void ld8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}

// One warp picks the `top` largest of a token's E logits in shared memory (overwritten), the lower expert winning a
// tie, and writes the experts and their weights. Two rules:
//   rule 0: the largest logits are chosen; the weights are the softmax over the chosen logits alone.
//   rule 1: scores s = softmax of the logits over all E; the largest s + corr are chosen (`corr`: one number per expert, or
//           null); the weights are the chosen experts' s over their sum (+ 1e-20), times out_scale.
__device__ __forceinline__ void moe_pick(float* z, int E, int top, int* __restrict__ idx, float* __restrict__ wt, int lane, int rule = 0,
                                         const void* __restrict__ corr = nullptr, int c_kind = 0, float out_scale = 1.f) {
    float chosen_v[MOE_MAX_TOP];
    float vmax = 0.f, den = 0.f;
    if (rule == 1) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        mx = il_warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) sum += expf(z[e] - mx);
        sum = il_warp_sum(sum);
        for (int e = lane; e < E; e += 32) z[e] = expf(z[e] - mx) / sum;      // the scores; a chosen one is marked by -1
        __syncwarp();
        for (int k = 0; k < top; ++k) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                if (z[e] < 0.f) continue;
                const float v = z[e] + (corr ? il_load_any(corr, c_kind, e) : 0.f);
                if (v > bv || (v == bv && e < bi)) bv = v, bi = e;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
            }
            if (bi >= E) bi = 0;                  // every score NaN: still a valid expert
            const float sb = z[bi];
            chosen_v[k] = sb;
            den += sb;
            __syncwarp();
            if (lane == 0) {
                idx[k] = bi;
                z[bi] = -1.f;
            }
            __syncwarp();
        }
        if (lane == 0)
            for (int k = 0; k < top; ++k) wt[k] = chosen_v[k] / (den + 1e-20f) * out_scale;
        return;
    }
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
            idx[k] = bi;
            z[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0)
        for (int k = 0; k < top; ++k) wt[k] = chosen_v[k] / den;
}

// A block routes TOK tokens: their rows stand in shared memory as f32; the block's warps deal the experts out among
// themselves (32 warps where a block has one token, a decode step: the kernel is then a few round trips to memory per warp), a warp reading an expert's weight row once (16 bytes a lane and step) for all TOK tokens; a lane sums its
// chunks in the order of the row and the warp adds the lanes' sums in a fixed tree, so a token's logits are the same
// whatever TOK is and whatever else is in the batch. Then one warp per token picks the `top` largest.
template <typename TA, int TOK, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) moe_route_kernel(const TA* x, int ldx, const TA* __restrict__ w, const void* __restrict__ bias, int b_kind,
                                                        int* __restrict__ idx, float* __restrict__ wt, int T, int H, int E, int top, int vec,
                                                        const float* sumsq, int n_partial, float inv_h, float eps, float* __restrict__ rstd_out) {
    extern __shared__ __align__(16) float sm[];   // [TOK][H] rows, then [TOK][E] logits
    __shared__ float rstd_s[TOK];
    float* xs = sm;
    float* zs = sm + (size_t)TOK * H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * TOK;
    if (TOK == 1) {
        // A decode step: a handful of blocks, each a chain of round trips to memory. The router's weights do not come from
        // the kernel before: the blocks ask for their lines (128 bytes a thread, dealt out over the grid) to be brought
        // into L2 while that kernel still runs.
        const char* wb = reinterpret_cast<const char*>(w);
        const size_t bytes = (size_t)E * H * sizeof(TA);
        for (size_t off = ((size_t)blockIdx.x * (WARPS * 32) + threadIdx.x) * 128; off < bytes; off += (size_t)gridDim.x * (WARPS * 32) * 128)
            asm volatile("prefetch.global.L2 [%0];\n" ::"l"(wb + off));
    }
    il_pdl_begin();
    // Rows whose RMSNorm is not finished (x = residual * norm weight, `sumsq` the sums of the residual's squares per row
    // and block of columns, left by the product before): the row is multiplied by rstd = rsqrt(sum / H + eps) here, in
    // f32, and rstd is left in `rstd_out` for the products that read the same rows.
    if (warp < TOK) {
        float r = 1.f;
        if (sumsq && t0 + warp < T) {
            float sq = 0.f;
            for (int k = lane; k < n_partial; k += 32) sq += sumsq[(size_t)(t0 + warp) * n_partial + k];
            r = rsqrtf(il_warp_sum(sq) * inv_h + eps);
            if (lane == 0 && rstd_out) rstd_out[t0 + warp] = r;
        }
        if (lane == 0) rstd_s[warp] = r;
    }
    __syncthreads();
    // Vector path: a lane multiplies 8 consecutive columns at a time; the row is kept as two halves, columns 8j..8j+3 of
    // every chunk j in the first and 8j+4..8j+7 in the second, so that the lanes of a warp read consecutive 16-byte pieces
    // of a half (8 consecutive floats a lane would put lanes 0 and 4 on the same banks).
    for (int i = threadIdx.x; i < TOK * H; i += WARPS * 32) {
        const int tk = i / H, h = i - tk * H;
        const int at = vec ? ((h >> 3) << 2) + (h & 3) + ((h >> 2) & 1) * (H >> 1) : h;
        xs[tk * H + at] = t0 + tk < T ? il_to_f(x[(size_t)(t0 + tk) * ldx + h]) * rstd_s[tk] : 0.f;
    }
    __syncthreads();
    for (int e = warp; e < E; e += WARPS) {
        const TA* wr = w + (size_t)e * H;
        float s[TOK];
#pragma unroll
        for (int tk = 0; tk < TOK; ++tk) s[tk] = 0.f;
        if (vec) {
            // four 16-byte loads of the weight row in flight at a time: with one, a decode step's few blocks spend the
            // kernel waiting for memory one load after the other
            for (int h0 = lane * 8; h0 < H; h0 += 1024) {
                float wv[4][8];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int h = h0 + u * 256;
                    if (h < H) ld8(wr + h, wv[u]);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int h = h0 + u * 256;
                    if (h >= H) break;
#pragma unroll
                    for (int tk = 0; tk < TOK; ++tk) {
                        const float4 a = *reinterpret_cast<const float4*>(xs + tk * H + (h >> 1)),
                                     b = *reinterpret_cast<const float4*>(xs + tk * H + (H >> 1) + (h >> 1));
                        float acc = s[tk];
                        acc = fmaf(a.x, wv[u][0], acc), acc = fmaf(a.y, wv[u][1], acc), acc = fmaf(a.z, wv[u][2], acc), acc = fmaf(a.w, wv[u][3], acc);
                        acc = fmaf(b.x, wv[u][4], acc), acc = fmaf(b.y, wv[u][5], acc), acc = fmaf(b.z, wv[u][6], acc), acc = fmaf(b.w, wv[u][7], acc);
                        s[tk] = acc;
                    }
                }
            }
        } else {
            for (int h = lane; h < H; h += 32) {
                const float wv = il_to_f(wr[h]);
#pragma unroll
                for (int tk = 0; tk < TOK; ++tk) s[tk] = fmaf(xs[tk * H + h], wv, s[tk]);
            }
        }
        const float be = bias ? il_load_any(bias, b_kind, e) : 0.f;
#pragma unroll
        for (int tk = 0; tk < TOK; ++tk) {
            const float v = il_warp_sum(s[tk]);
            if (lane == 0) zs[tk * E + e] = v + be;
        }
    }
    __syncthreads();
    if (warp >= TOK || t0 + warp >= T) return;
    moe_pick(zs + (size_t)warp * E, E, top, idx + (size_t)(t0 + warp) * top, wt + (size_t)(t0 + warp) * top, lane);
}

// The choice alone, for logits that a matrix product has written already (z [T, ldz] f32, the bias still to be added):
// a warp a token, its row of logits in shared memory.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) moe_select_kernel(const float* __restrict__ z, int ldz, const void* __restrict__ bias, int b_kind,
                                                               int* __restrict__ idx, float* __restrict__ wt, int T, int E, int top, int rule,
                                                               float out_scale) {
    extern __shared__ __align__(16) float sm[];   // [WARPS][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * WARPS + warp;
    il_pdl_begin();
    if (t >= T) return;
    float* zs = sm + (size_t)warp * E;
    // (rule 1: the bias is no part of the logits; it joins the scores where the experts are chosen)
    for (int e = lane; e < E; e += 32) zs[e] = z[(size_t)t * ldz + e] + ((bias && rule == 0) ? il_load_any(bias, b_kind, e) : 0.f);
    __syncwarp();
    moe_pick(zs, E, top, idx + (size_t)t * top, wt + (size_t)t * top, lane, rule, bias, b_kind, out_scale);
}

// The body of the sort, by one whole block; `sh`: 2 * E ints of shared memory. (idx is not declared __restrict__: the
// fused kernel below reads what its own warps have just written.)
__device__ __forceinline__ void moe_sort_body(int* sh, const int* idx, int n_slots, int top, int E, int* __restrict__ group_off,
                                              int* __restrict__ pos_of_slot, int* __restrict__ row_of_pos) {
    int* cnt = sh;
    int* cur = sh + E;
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

__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* idx, int n_slots, int top, int E, int* __restrict__ group_off,
                                                        int* __restrict__ pos_of_slot, int* __restrict__ row_of_pos) {
    extern __shared__ int sh[];                   // [E] counts, then [E] cursors
    il_pdl_begin();
    moe_sort_body(sh, idx, n_slots, top, E, group_off, pos_of_slot, row_of_pos);
}

// ---- the router of a decode step (a few bfloat16 rows) as two short kernels --------------------------------------------
// One block a token, as moe_route_kernel does it, is a chain of round trips to memory on a handful of SMs: sums of
// squares, the row, then the weight rows of each of a warp's experts in turn, then the choice. Here a warp owns one
// (token, expert) pair: it asks for its weight row before it waits for the kernel before (the weights do not come from
// it), then reads the row's columns it needs straight from memory, so the logits are one round trip deep; a second kernel
// of one block chooses for every token (a warp a token) and sorts the slots. Sums in a fixed order: a token's logits do
// not depend on what else is in the batch.
constexpr int ML_WARPS = 8, ML_CH = 8;            // a lane holds ML_CH chunks of 8 columns: 2,048 columns a pass
__global__ void __launch_bounds__(ML_WARPS * 32) moe_logits_kernel(const __nv_bfloat16* x, int ldx, const __nv_bfloat16* __restrict__ w,
                                                                   const void* __restrict__ bias, int b_kind, float* __restrict__ z, int T, int H, int E,
                                                                   const float* sumsq, int n_partial, float inv_h, float eps, float* __restrict__ rstd_out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * ML_WARPS + warp, t = blockIdx.y;
    const __nv_bfloat16* wr = w + (size_t)(e < E ? e : 0) * H;
    uint4 wv[ML_CH];
#pragma unroll
    for (int u = 0; u < ML_CH; ++u) {
        const int h = lane * 8 + u * 256;
        wv[u] = h < H ? *reinterpret_cast<const uint4*>(wr + h) : make_uint4(0u, 0u, 0u, 0u);
    }
    il_pdl_begin();
    float rstd = 1.f;
    if (sumsq) {
        float sq = 0.f;
        for (int k = lane; k < n_partial; k += 32) sq += sumsq[(size_t)t * n_partial + k];
        rstd = rsqrtf(il_warp_sum(sq) * inv_h + eps);
        if (e == 0 && lane == 0 && rstd_out) rstd_out[t] = rstd;
    }
    if (e >= E) return;
    const __nv_bfloat16* xr = x + (size_t)t * ldx;
    float acc = 0.f;
    for (int base = 0; base < H; base += 256 * ML_CH) {
        uint4 xv[ML_CH];
#pragma unroll
        for (int u = 0; u < ML_CH; ++u) {
            const int h = base + lane * 8 + u * 256;
            if (base > 0) wv[u] = h < H ? *reinterpret_cast<const uint4*>(wr + h) : make_uint4(0u, 0u, 0u, 0u);
            xv[u] = h < H ? *reinterpret_cast<const uint4*>(xr + h) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < ML_CH; ++u) {
            const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&xv[u]);
            const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&wv[u]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 fa = __bfloat1622float2(a[i]), fb = __bfloat1622float2(b[i]);
                acc = fmaf(fa.x, fb.x, acc);
                acc = fmaf(fa.y, fb.y, acc);
            }
        }
    }
    acc = il_warp_sum(acc);
    if (lane == 0) z[(size_t)t * E + e] = acc * rstd + (bias ? il_load_any(bias, b_kind, e) : 0.f);
}

// Chooses for every token (a warp a token, in turns) from logits z [T, E], then sorts the slots: one block.
__global__ void __launch_bounds__(1024) moe_select_sort_kernel(const float* z, int ldz, int* idx, float* __restrict__ wt, int T, int E, int top,
                                                               int* __restrict__ group_off, int* __restrict__ pos_of_slot, int* __restrict__ row_of_pos,
                                                               int rule, const void* __restrict__ corr, int c_kind, float out_scale) {
    extern __shared__ __align__(16) float sm[];   // [32][E] logits of the warps' tokens, then 2 * E ints for the sort
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    il_pdl_begin();
    float* zs = sm + (size_t)warp * E;
    for (int t = warp; t < T; t += 32) {
        for (int e = lane; e < E; e += 32) zs[e] = z[(size_t)t * ldz + e];
        __syncwarp();
        moe_pick(zs, E, top, idx + (size_t)t * top, wt + (size_t)t * top, lane, rule, corr, c_kind, out_scale);
        __syncwarp();
    }
    __syncthreads();                              // the choices, written to memory by this block's warps, are read below
    moe_sort_body(reinterpret_cast<int*>(sm + (size_t)32 * E), idx, T * top, top, E, group_off, pos_of_slot, row_of_pos);
}

__device__ __forceinline__ float4 ld4c(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4c(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4c(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4c(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a), u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

// One block a token; a thread sums four neighbouring columns (H a multiple of 4: `vec`), the token's rows one after the
// other in the order of its choices, so the sum does not depend on the number of threads or on the batch.
// Experts without weights ("identity": the experts from n_real on, whose places in the sorted order start at
// group_off[n_real]) return their input: such a choice adds weight * x[t] (`x` [T, ldx], the rows the experts read).
// `sgate` (or null): one f32 number per token (stride ld_sg) whose sigmoid multiplies the shared row.
template <typename TA>
__global__ void moe_combine_kernel(const TA* y, const int* pos_of_slot, const float* wt, const TA* shared_rows, TA* __restrict__ out,
                                   int H, int top, int vec, const int* group_off, int n_real, const TA* x, int ldx, const float* sgate,
                                   int ld_sg) {
    __shared__ int sp[MOE_MAX_TOP];
    __shared__ float sw[MOE_MAX_TOP];
    const int t = blockIdx.x;
    il_pdl_begin();
    if (threadIdx.x < top) {                      // the token's places and weights once, not once per column
        const int p = pos_of_slot[(size_t)t * top + threadIdx.x];
        sp[threadIdx.x] = (group_off && p >= group_off[n_real]) ? -1 : p;       // -1: the input row itself
        sw[threadIdx.x] = wt[(size_t)t * top + threadIdx.x];
    }
    __syncthreads();
    const float sg = (shared_rows && sgate) ? 1.f / (1.f + expf(-sgate[(size_t)t * ld_sg])) : 1.f;
    if (vec) {
        for (int h = threadIdx.x * 4; h < H; h += blockDim.x * 4) {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < top; ++k) {
                const float4 v = sp[k] >= 0 ? ld4c(y + (size_t)sp[k] * H + h) : ld4c(x + (size_t)t * ldx + h);
                const float w = sw[k];
                s.x = fmaf(w, v.x, s.x), s.y = fmaf(w, v.y, s.y), s.z = fmaf(w, v.z, s.z), s.w = fmaf(w, v.w, s.w);
            }
            if (shared_rows) {
                const float4 v = ld4c(shared_rows + (size_t)t * H + h);
                s.x = fmaf(sg, v.x, s.x), s.y = fmaf(sg, v.y, s.y), s.z = fmaf(sg, v.z, s.z), s.w = fmaf(sg, v.w, s.w);
            }
            st4c(out + (size_t)t * H + h, s);
        }
        return;
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) s = fmaf(sw[k], il_to_f(sp[k] >= 0 ? y[(size_t)sp[k] * H + h] : x[(size_t)t * ldx + h]), s);
        if (shared_rows) s = fmaf(sg, il_to_f(shared_rows[(size_t)t * H + h]), s);
        out[(size_t)t * H + h] = il_from_f<TA>(s);
    }
}

// The combine as the last step of a branch of a few bfloat16 rows: the token's sum, rounded to bfloat16 as the branch is
// when it is passed on, goes into the float32 residual (resid += bscale * branch), and what the next RMSNorm needs is
// left for the product that follows: xw = resid * norm weight (bfloat16) and, per block of 16 columns, the sum of the
// residual's squares (sumsq [T][n_partial]). Four columns a thread: four neighbouring lanes own a block of 16.
__global__ void moe_combine_resid_kernel(const __nv_bfloat16* y, const int* pos_of_slot, const float* wt, const __nv_bfloat16* shared_rows, int H, int top,
                                         float* resid, float bscale, const void* __restrict__ norm_w, int nw_kind, __nv_bfloat16* __restrict__ xw,
                                         float* __restrict__ sumsq, int n_partial) {
    __shared__ int sp[MOE_MAX_TOP];
    __shared__ float sw[MOE_MAX_TOP];
    const int t = blockIdx.x;
    il_pdl_begin();
    if (threadIdx.x < top) {
        sp[threadIdx.x] = pos_of_slot[(size_t)t * top + threadIdx.x];
        sw[threadIdx.x] = wt[(size_t)t * top + threadIdx.x];
    }
    __syncthreads();
    for (int base = 0; base < H; base += blockDim.x * 4) {
        const int h = base + threadIdx.x * 4;
        float sq = 0.f;
        if (h < H) {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < top; ++k) {
                const float4 v = ld4c(y + (size_t)sp[k] * H + h);
                const float w = sw[k];
                s.x = fmaf(w, v.x, s.x), s.y = fmaf(w, v.y, s.y), s.z = fmaf(w, v.z, s.z), s.w = fmaf(w, v.w, s.w);
            }
            if (shared_rows) {
                const float4 v = ld4c(shared_rows + (size_t)t * H + h);
                s.x += v.x, s.y += v.y, s.z += v.z, s.w += v.w;
            }
            float4 r = *reinterpret_cast<const float4*>(resid + (size_t)t * H + h);
            r.x = fmaf(bscale, __bfloat162float(__float2bfloat16_rn(s.x)), r.x);
            r.y = fmaf(bscale, __bfloat162float(__float2bfloat16_rn(s.y)), r.y);
            r.z = fmaf(bscale, __bfloat162float(__float2bfloat16_rn(s.z)), r.z);
            r.w = fmaf(bscale, __bfloat162float(__float2bfloat16_rn(s.w)), r.w);
            *reinterpret_cast<float4*>(resid + (size_t)t * H + h) = r;
            st4c(xw + (size_t)t * H + h, make_float4(r.x * il_load_any(norm_w, nw_kind, h), r.y * il_load_any(norm_w, nw_kind, h + 1),
                                                     r.z * il_load_any(norm_w, nw_kind, h + 2), r.w * il_load_any(norm_w, nw_kind, h + 3)));
            sq = (r.x * r.x + r.y * r.y) + (r.z * r.z + r.w * r.w);
        }
        sq += __shfl_xor_sync(0xffffffffu, sq, 1);
        sq += __shfl_xor_sync(0xffffffffu, sq, 2);
        if (h < H && (threadIdx.x & 3) == 0) sumsq[(size_t)t * n_partial + (h >> 4)] = sq;
    }
}

// out[p] = x[rows[p]]: the rows of the tokens in the order of the sorted slots, for a product that wants them contiguous.
template <typename TA>
__global__ void gather_rows_kernel(const TA* x, int ldx, const int* rows, TA* __restrict__ out, int H) {
    const int p = blockIdx.x;
    il_pdl_begin();
    const TA* src = x + (size_t)rows[p] * ldx;
    TA* dst = out + (size_t)p * H;
    if ((H * sizeof(TA)) % 16 == 0 && (ldx * sizeof(TA)) % 16 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)out & 15)) {
        const int n = H * sizeof(TA) / 16;
        for (int i = threadIdx.x; i < n; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
    }
}

// The combine of a few bfloat16 rows with the residual add and the next norm's inputs (see moe_combine_resid_kernel).
// H a multiple of 4, sumsq [T][ceil(H / 16)].
IL_EXPORT int il_moe_combine_resid(const void* y, const int* pos_of_slot, const float* wt, const void* shared_rows, int T, int H, int top, float* resid,
                                   float bscale, const void* norm_w, int nw_kind, void* xw, float* sumsq, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (H <= 0 || top <= 0 || top > MOE_MAX_TOP || !resid || !norm_w || !xw || !sumsq) return IL_BAD_ARG;
    if (H % 4 || ((uintptr_t)y & 15) || ((uintptr_t)shared_rows & 15) || ((uintptr_t)resid & 15) || ((uintptr_t)xw & 7)) return IL_UNSUPPORTED;
    const int threads = H >= 2048 ? 512 : H >= 1024 ? 256 : 128;
    IL_LAUNCH(moe_combine_resid_kernel, T, threads, 0, stream, (const __nv_bfloat16*)y, pos_of_slot, wt, (const __nv_bfloat16*)shared_rows, H, top, resid,
              bscale, norm_w, nw_kind, (__nv_bfloat16*)xw, sumsq, (H + 15) / 16);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

IL_EXPORT int il_gather_rows(const void* x, int act_kind, int ldx, const int* rows, void* out, int n_rows, int H, cudaStream_t stream) {
    if (n_rows <= 0) return IL_OK;
    if (H <= 0) return IL_BAD_ARG;
    if (act_kind == IL_F32)
        IL_LAUNCH(gather_rows_kernel<float>, n_rows, 128, 0, stream, (const float*)x, ldx, rows, (float*)out, H);
    else if (act_kind == IL_BF16)
        IL_LAUNCH(gather_rows_kernel<__nv_bfloat16>, n_rows, 128, 0, stream, (const __nv_bfloat16*)x, ldx, rows, (__nv_bfloat16*)out, H);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

template <typename TA, int TOK, int WARPS>
static int launch_route(const void* x, int ldx, const void* w, const void* bias, int b_kind, int* idx, float* wt, int T, int H, int E, int top,
                        int vec, const float* sumsq, int n_partial, float eps, float* rstd_out, cudaStream_t stream) {
    const size_t smem = ((size_t)TOK * H + (size_t)TOK * E) * sizeof(float);
    if (smem > 200 * 1024) return IL_UNSUPPORTED;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(moe_route_kernel<TA, TOK, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return 1000 + (int)e;
    }
    IL_LAUNCH((moe_route_kernel<TA, TOK, WARPS>), (T + TOK - 1) / TOK, WARPS * 32, smem, stream, (const TA*)x, ldx, (const TA*)w, bias, b_kind, idx, wt, T, H, E,
              top, vec, sumsq, n_partial, 1.f / (float)H, eps, rstd_out);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// sumsq (or null): [T][n_partial] sums of squares of the rows' residual; x is then residual * norm weight, the router
// finishes the norm itself and leaves rstd [T] in rstd_out (if given).
IL_EXPORT int il_moe_route(const void* x, int act_kind, int ldx, const void* w, const void* bias, int b_kind, int* idx, float* wt, int T,
                           int H, int E, int top, const float* sumsq, int n_partial, float eps, float* rstd_out, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (H <= 0 || E <= 0 || top <= 0 || top > E || top > MOE_MAX_TOP || (sumsq && n_partial <= 0)) return IL_BAD_ARG;
    const int vec = (H % 8 == 0 && !((uintptr_t)w & 15)) ? 1 : 0;
    // few tokens (a decode step): a block a token, so that the experts' rows are read by as many SMs as there are tokens;
    // many: four tokens a block share each read
    const bool four = T > 128 && ((size_t)4 * (H + E) * sizeof(float)) <= 160 * 1024;
    if (act_kind == IL_F32)
        return four ? launch_route<float, 4, 8>(x, ldx, w, bias, b_kind, idx, wt, T, H, E, top, vec, sumsq, n_partial, eps, rstd_out, stream)
                    : launch_route<float, 1, 32>(x, ldx, w, bias, b_kind, idx, wt, T, H, E, top, vec, sumsq, n_partial, eps, rstd_out, stream);
    if (act_kind == IL_BF16)
        return four ? launch_route<__nv_bfloat16, 4, 8>(x, ldx, w, bias, b_kind, idx, wt, T, H, E, top, vec, sumsq, n_partial, eps, rstd_out, stream)
                    : launch_route<__nv_bfloat16, 1, 32>(x, ldx, w, bias, b_kind, idx, wt, T, H, E, top, vec, sumsq, n_partial, eps, rstd_out, stream);
    return IL_BAD_ARG;
}

// rule 0: the `top` largest of z + bias, weights their softmax. rule 1: scores softmax(z) over all E, the largest score + bias
// chosen, weights the chosen scores over their sum, times out_scale (see moe_pick).
IL_EXPORT int il_moe_select(const float* z, int ldz, const void* bias, int b_kind, int* idx, float* wt, int T, int E, int top, int rule,
                            float out_scale, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (E <= 0 || top <= 0 || top > E || top > MOE_MAX_TOP || ldz < E || (rule != 0 && rule != 1)) return IL_BAD_ARG;
    constexpr int WARPS = 8;
    const size_t smem = (size_t)WARPS * E * sizeof(float);
    if (smem > 200 * 1024) return IL_UNSUPPORTED;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(moe_select_kernel<WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return 1000 + (int)e;
    }
    IL_LAUNCH(moe_select_kernel<WARPS>, (T + WARPS - 1) / WARPS, WARPS * 32, smem, stream, z, ldz, bias, b_kind, idx, wt, T, E, top, rule, out_scale);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// Router and sort of a few bfloat16 rows (a decode step): logits z [T, E + extra] (scratch), then the choice and the sort in one
// block. IL_UNSUPPORTED where the rows are not whole 16-byte chunks or the experts' logits do not fit a block's memory.
// `extra`: rows of `w` behind the E experts' whose products are written to z as further columns and take no part in the
// choice (a gate that is a function of the same rows). rule, out_scale: see il_moe_select.
IL_EXPORT int il_moe_route_sort_small(const void* x, int ldx, const void* w, const void* bias, int b_kind, float* z, int* idx, float* wt, int T, int H,
                                      int E, int top, const float* sumsq, int n_partial, float eps, float* rstd_out, int* group_off,
                                      int* pos_of_slot, int* row_of_pos, int extra, int rule, float out_scale, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (H <= 0 || E <= 0 || top <= 0 || top > E || top > MOE_MAX_TOP || (sumsq && n_partial <= 0) || extra < 0 || (rule != 0 && rule != 1) ||
        (extra > 0 && bias && rule == 0))
        return IL_BAD_ARG;
    const size_t smem = (size_t)32 * E * sizeof(float) + (size_t)2 * E * sizeof(int);
    if (H % 8 || ldx % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || smem > 200 * 1024 || T > 65535) return IL_UNSUPPORTED;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(moe_select_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return 1000 + (int)e;
    }
    const int EZ = E + extra;                     // the logits kernel knows no experts: it writes one column per row of w
    IL_LAUNCH(moe_logits_kernel, dim3((EZ + ML_WARPS - 1) / ML_WARPS, T), ML_WARPS * 32, 0, stream, (const __nv_bfloat16*)x, ldx,
              (const __nv_bfloat16*)w, rule == 0 ? bias : (const void*)nullptr, b_kind, z, T, H, EZ, sumsq, n_partial, 1.f / (float)H, eps, rstd_out);
    IL_LAUNCH(moe_select_sort_kernel, 1, 1024, smem, stream, (const float*)z, EZ, idx, wt, T, E, top, group_off, pos_of_slot, row_of_pos, rule,
              rule == 1 ? bias : (const void*)nullptr, b_kind, out_scale);
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
                             int H, int top, const int* group_off, int n_real, const void* x, int ldx, const float* sgate, int ld_sg,
                             cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (H <= 0 || top <= 0 || (group_off && (!x || n_real < 0 || ldx < H))) return IL_BAD_ARG;
    const int vec = (H % 4 == 0 && !((uintptr_t)y & 15) && !((uintptr_t)out & 15) && !((uintptr_t)shared_rows & 15) &&
                     (!group_off || (ldx % 4 == 0 && !((uintptr_t)x & 15)))) ? 1 : 0;
    const int threads = vec ? (H >= 2048 ? 512 : H >= 1024 ? 256 : 128) : (H >= 1024 ? 256 : 128);
    if (act_kind == IL_F32)
        IL_LAUNCH(moe_combine_kernel<float>, T, threads, 0, stream, (const float*)y, pos_of_slot, wt, (const float*)shared_rows, (float*)out, H, top, vec,
                  group_off, n_real, (const float*)x, ldx, sgate, ld_sg);
    else if (act_kind == IL_BF16)
        IL_LAUNCH(moe_combine_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)y, pos_of_slot, wt,
                  (const __nv_bfloat16*)shared_rows, (__nv_bfloat16*)out, H, top, vec, group_off, n_real, (const __nv_bfloat16*)x, ldx, sgate, ld_sg);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
