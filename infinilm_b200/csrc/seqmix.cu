// Sequence mixers that carry a fixed-size state per request instead of (or beside) cached keys: a short causal
// convolution over time with its last inputs as state, two linear recurrences over a matrix state per head (a decayed
// outer-product sum, and the gated delta rule), a norm over groups of columns with a gate, a gate per head, and a soft cap.
//
// A step's rows are the tokens of its entries one after the other (entry e: rows qstart[e] .. qstart[e+1]-1); an entry
// reads its state from slot read_slots[e] (slot 0 holds zeros: a request's first step) and leaves it in write_slots[e].
// Every recurrence runs token by token in the order of the sequence, in float32, so what a token gets does not depend on
// how the sequence was cut into steps or on what else is in the batch.
#include "common.cuh"

__device__ __forceinline__ float sm_silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sm_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float sm_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// SiLU by the fast exponential and division (relative error near 2^-21): the one the recurrences apply to their inputs,
// in the kernel or as a pass of its own, so that a token's state does not depend on which of the two ran.
__device__ __forceinline__ float sm_silu_fast(float z) { return __fdividef(z, 1.f + __expf(-z)); }

#define SM_MAX_TAPS 16

// ---- short convolution ----------------------------------------------------------------------------------------------
// y[t, ch] = act( sum_j w[ch, j] * u[t - (taps-1) + j, ch] ), u before the step's first row from the state (its row i is
// the input (taps-1-i) tokens before the step's first), zeros before the sequence's start (the zero slot).
// Channels are read as segments of seg_in columns and written as segments of seg_out >= seg_in columns, the rest zero
// (heads padded to a common size). One thread per (row, output column).
template <typename TI, typename TO>
__global__ void short_conv_kernel(const TI* __restrict__ x, int ldx, int x_off, const float* __restrict__ w, int taps,
                                  float* state, size_t slot_stride, int st_off, int st_ld,
                                  const int* __restrict__ read_slots, const int* __restrict__ write_slots, const int* __restrict__ tok_entry,
                                  const int* __restrict__ qstart, TO* __restrict__ out, int ldo, int out_off, int n_seg, int seg_in,
                                  int n_seg2, int seg_in2, int seg_out, int act, int T) {
    // columns: n_seg segments of seg_in channels, then n_seg2 of seg_in2, every segment written seg_out wide.
    // blockIdx.y walks the tokens, the block's threads consecutive columns.
    const int cols = (n_seg + n_seg2) * seg_out;
    const int oc = blockIdx.x * blockDim.x + threadIdx.x;
    if (oc >= cols) return;
    const int seg = oc / seg_out, within = oc - seg * seg_out;
    const bool second = seg >= n_seg;
    const int width = second ? seg_in2 : seg_in;
    const int ch = second ? n_seg * seg_in + (seg - n_seg) * seg_in2 + within : seg * seg_in + within;
    float wt[SM_MAX_TAPS];
    if (within < width)
        for (int j = 0; j < taps; ++j) wt[j] = w[(size_t)ch * taps + j];
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        TO* o = out + (size_t)t * ldo + out_off + oc;
        if (within >= width) {
            *o = il_from_f<TO>(0.f);
            continue;
        }
        const int e = tok_entry[t];
        const int first = qstart[e], local = t - first;
        const bool alone = write_slots && qstart[e + 1] - first == 1;     // the entry's only token: this thread also moves the state on
        float* st = state + (size_t)read_slots[e] * slot_stride + st_off + ch;
        float acc = 0.f, keep[SM_MAX_TAPS];
        for (int j = 0; j < taps; ++j) {
            const int s = local - (taps - 1) + j;
            const float u = s >= 0 ? il_to_f(x[(size_t)(t - local + s) * ldx + x_off + ch]) : st[(size_t)(taps - 1 + s) * st_ld];
            acc = fmaf(wt[j], u, acc);
            keep[j] = u;
        }
        *o = il_from_f<TO>(act == 1 ? sm_silu(acc) : acc);
        if (alone) {                              // nobody else reads this entry's state for this channel: safe in place
            float* wr = state + (size_t)write_slots[e] * slot_stride + st_off + ch;
            for (int j = 1; j < taps; ++j) wr[(size_t)(j - 1) * st_ld] = keep[j];
        }
    }
}

// The same with the taps known at compile time and a thread walking TT consecutive tokens of its column: the last
// taps-1 inputs ride along in registers (rows of an entry are consecutive, so the row before a token is its predecessor
// whenever it has one in this step), each input is read once, nothing lives in local memory.
template <typename TI, typename TO, int TAPS, int TT>
__global__ void short_conv_tile_kernel(const TI* __restrict__ x, int ldx, int x_off, const float* __restrict__ w,
                                       float* state, size_t slot_stride, int st_off, int st_ld,
                                       const int* __restrict__ read_slots, const int* __restrict__ write_slots, const int* __restrict__ tok_entry,
                                       const int* __restrict__ qstart, TO* __restrict__ out, int ldo, int out_off, int n_seg, int seg_in,
                                       int n_seg2, int seg_in2, int seg_out, int act, int T) {
    const int cols = (n_seg + n_seg2) * seg_out;
    const int oc = blockIdx.x * blockDim.x + threadIdx.x;
    if (oc >= cols) return;
    const int seg = oc / seg_out, within = oc - seg * seg_out;
    const bool second = seg >= n_seg;
    const int width = second ? seg_in2 : seg_in;
    const int t0 = blockIdx.y * TT;
    if (within >= width) {
        for (int i = 0; i < TT && t0 + i < T; ++i) out[(size_t)(t0 + i) * ldo + out_off + oc] = il_from_f<TO>(0.f);
        return;
    }
    const int ch = second ? n_seg * seg_in + (seg - n_seg) * seg_in2 + within : seg * seg_in + within;
    float wt[TAPS], win[TAPS > 1 ? TAPS - 1 : 1];         // win[j]: the input j + 1 rows back
#pragma unroll
    for (int j = 0; j < TAPS; ++j) wt[j] = w[(size_t)ch * TAPS + j];
#pragma unroll
    for (int j = 0; j < TAPS - 1; ++j) win[j] = t0 - 1 - j >= 0 ? il_to_f(x[(size_t)(t0 - 1 - j) * ldx + x_off + ch]) : 0.f;
#pragma unroll
    for (int i = 0; i < TT; ++i) {
        const int t = t0 + i;
        if (t < T) {
            const float cur = il_to_f(x[(size_t)t * ldx + x_off + ch]);
            const int e = tok_entry[t];
            const int first = qstart[e], local = t - first;
            const float* st = state + (size_t)read_slots[e] * slot_stride + st_off + ch;
            float u[TAPS];                        // u[j]: the input j tokens back in the sequence
            u[0] = cur;
#pragma unroll
            for (int j = 1; j < TAPS; ++j) u[j] = local - j >= 0 ? win[j - 1] : st[(size_t)(TAPS - 1 + local - j) * st_ld];
            float acc = 0.f;
#pragma unroll
            for (int j = TAPS - 1; j >= 0; --j) acc = fmaf(wt[TAPS - 1 - j], u[j], acc);      // oldest first, as the plain kernel sums
            out[(size_t)t * ldo + out_off + oc] = il_from_f<TO>(act == 1 ? sm_silu(acc) : acc);
            if (write_slots && qstart[e + 1] - first == 1) {       // the entry's only token: this thread also moves the state on
                float* wr = state + (size_t)write_slots[e] * slot_stride + st_off + ch;
#pragma unroll
                for (int j = 0; j < TAPS - 1; ++j) wr[(size_t)(TAPS - 2 - j) * st_ld] = u[j];
            }
#pragma unroll
            for (int j = TAPS - 2; j > 0; --j) win[j] = win[j - 1];
            if (TAPS > 1) win[0] = cur;
        }
    }
}

// The state after the step: the last taps-1 inputs of each entry (older ones from the state it had). One thread per
// (entry, channel) reads all it needs before it writes, so an entry may read and write the same slot.
template <typename TI>
__global__ void short_conv_state_kernel(const TI* __restrict__ x, int ldx, int x_off, int C, int taps, float* state,
                                        size_t slot_stride, int st_off, int st_ld, const int* __restrict__ read_slots,
                                        const int* __restrict__ write_slots, const int* __restrict__ qstart, int E, int e0) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= E * C) return;
    const int e = e0 + idx / C, ch = idx % C;
    const int q0 = qstart[e], n = qstart[e + 1] - q0;
    if (n <= 0) return;
    const float* rd = state + (size_t)read_slots[e] * slot_stride + st_off + ch;
    float keep[SM_MAX_TAPS];
    for (int i = 0; i < taps - 1; ++i) {
        const int s = n - (taps - 1) + i;
        keep[i] = s >= 0 ? il_to_f(x[(size_t)(q0 + s) * ldx + x_off + ch]) : rd[(size_t)(taps - 1 + s) * st_ld];
    }
    float* wr = state + (size_t)write_slots[e] * slot_stride + st_off + ch;
    for (int i = 0; i < taps - 1; ++i) wr[(size_t)i * st_ld] = keep[i];
}

static inline int sm_grid(size_t total, int threads) {
    size_t g = (total + threads - 1) / threads;
    return (int)(g > 148 * 32 ? 148 * 32 : (g < 1 ? 1 : g));
}

// write_slots (may be null): entries that bring a single token get their state moved on by this kernel; the others (and
// all of them, without write_slots) by il_short_conv_state.
IL_EXPORT int il_short_conv(const void* x, int x_kind, int ldx, int x_off, const float* w, int taps, float* state,
                            long long slot_stride, int st_off, int st_ld, const int* read_slots, const int* write_slots, const int* tok_entry,
                            const int* qstart, void* out, int out_kind, int ldo, int out_off, int n_seg, int seg_in, int n_seg2, int seg_in2,
                            int seg_out, int act, int T, cudaStream_t stream) {
    if (T <= 0 || n_seg <= 0) return IL_OK;
    if (taps < 1 || taps > SM_MAX_TAPS || seg_in <= 0 || seg_out < seg_in || n_seg2 < 0 || (n_seg2 > 0 && (seg_in2 <= 0 || seg_out < seg_in2)))
        return IL_BAD_ARG;
    const int cols_all = (n_seg + n_seg2) * seg_out;
    if (taps <= 8) {                              // the usual few taps: the tiled form
        constexpr int TT = 8;
        const dim3 tgrid((cols_all + 127) / 128, (T + TT - 1) / TT);
#define SC_TILE(TI_, TO_, TAPS_)                                                                                              \
        short_conv_tile_kernel<TI_, TO_, TAPS_, TT><<<tgrid, 128, 0, stream>>>((const TI_*)x, ldx, x_off, w, state, (size_t)slot_stride, st_off, \
            st_ld, read_slots, write_slots, tok_entry, qstart, (TO_*)out, ldo, out_off, n_seg, seg_in, n_seg2, seg_in2, seg_out, act, T)
#define SC_TAPS(TI_, TO_)                                                                                  \
        switch (taps) {                                                                                    \
            case 1: SC_TILE(TI_, TO_, 1); break; case 2: SC_TILE(TI_, TO_, 2); break;                      \
            case 3: SC_TILE(TI_, TO_, 3); break; case 4: SC_TILE(TI_, TO_, 4); break;                      \
            case 5: SC_TILE(TI_, TO_, 5); break; case 6: SC_TILE(TI_, TO_, 6); break;                      \
            case 7: SC_TILE(TI_, TO_, 7); break; default: SC_TILE(TI_, TO_, 8); break;                     \
        }
        if (x_kind == IL_F32 && out_kind == IL_F32) { SC_TAPS(float, float) }
        else if (x_kind == IL_BF16 && out_kind == IL_F32) { SC_TAPS(__nv_bfloat16, float) }
        else if (x_kind == IL_BF16 && out_kind == IL_BF16) { SC_TAPS(__nv_bfloat16, __nv_bfloat16) }
        else return IL_BAD_ARG;
        IL_LAUNCH_CHECK();
        return IL_OK;
    }
    const dim3 grid((cols_all + 255) / 256, T < 32768 ? T : 32768);
#define SC_ARGS ldx, x_off, w, taps, state, (size_t)slot_stride, st_off, st_ld, read_slots, write_slots, tok_entry, qstart
#define SC_TAIL ldo, out_off, n_seg, seg_in, n_seg2, seg_in2, seg_out, act, T
    if (x_kind == IL_F32 && out_kind == IL_F32)
        short_conv_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)x, SC_ARGS, (float*)out, SC_TAIL);
    else if (x_kind == IL_BF16 && out_kind == IL_F32)
        short_conv_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, SC_ARGS, (float*)out, SC_TAIL);
    else if (x_kind == IL_BF16 && out_kind == IL_BF16)
        short_conv_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, SC_ARGS, (__nv_bfloat16*)out, SC_TAIL);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// Entries e0 .. e0 + E - 1.
IL_EXPORT int il_short_conv_state(const void* x, int x_kind, int ldx, int x_off, int C, int taps, float* state, long long slot_stride,
                                  int st_off, int st_ld, const int* read_slots, const int* write_slots, const int* qstart, int E, int e0,
                                  cudaStream_t stream) {
    if (E <= 0 || C <= 0 || taps <= 1) return IL_OK;
    if (taps > SM_MAX_TAPS || e0 < 0) return IL_BAD_ARG;
    const int grid = (E * C + 255) / 256;
    if (x_kind == IL_F32)
        short_conv_state_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, ldx, x_off, C, taps, state, (size_t)slot_stride, st_off, st_ld,
                                                                 read_slots, write_slots, qstart, E, e0);
    else if (x_kind == IL_BF16)
        short_conv_state_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, x_off, C, taps, state, (size_t)slot_stride,
                                                                         st_off, st_ld, read_slots, write_slots, qstart, E, e0);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- preparing the gated delta rule's inputs -------------------------------------------------------------------------
// q and k heads (float32, in place) become unit vectors: x / sqrt(sum x^2 + unit_eps), q also times q_scale; and per value
// head beta = sigmoid(b), g = exp(-exp(A_log) * softplus(a + dt_bias)), both float32 [T, H]. One warp per (row, q/k head),
// then the same warps over the value heads.
__global__ void delta_prep_kernel(float* qk, int ld, int q_off, int k_off, int G, int dim, float q_scale, float unit_eps,
                                  const float* __restrict__ ab, int ld_ab, int b_off, int a_off, const float* __restrict__ A_log,
                                  const float* __restrict__ dt_bias, float* __restrict__ beta, float* __restrict__ gdec, int H, int T) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int per_row = 2 * G;
    if (warp >= T * per_row) return;
    const int t = warp / per_row, j = warp - t * per_row;
    const bool is_q = j < G;
    float* v = qk + (size_t)t * ld + (is_q ? q_off + j * dim : k_off + (j - G) * dim);
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss += v[d] * v[d];
    ss = il_warp_sum(ss);
    const float r = (1.f / sqrtf(ss + unit_eps)) * (is_q ? q_scale : 1.f);
    for (int d = lane; d < dim; d += 32) v[d] *= r;
    if (j == 0)
        for (int h = lane; h < H; h += 32) {
            beta[(size_t)t * H + h] = sm_sigmoid(ab[(size_t)t * ld_ab + b_off + h]);
            gdec[(size_t)t * H + h] = expf(-expf(A_log[h]) * sm_softplus(ab[(size_t)t * ld_ab + a_off + h] + dt_bias[h]));
        }
}

IL_EXPORT int il_delta_prep(float* qk, int ld, int q_off, int k_off, int G, int dim, float q_scale, float unit_eps, const float* ab,
                            int ld_ab, int b_off, int a_off, const float* A_log, const float* dt_bias, float* beta, float* gdec, int H,
                            int T, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (G <= 0 || dim <= 0 || H <= 0) return IL_BAD_ARG;
    const size_t warps = (size_t)T * 2 * G;
    delta_prep_kernel<<<(int)((warps * 32 + 255) / 256), 256, 0, stream>>>(qk, ld, q_off, k_off, G, dim, q_scale, unit_eps, ab, ld_ab, b_off,
                                                                        a_off, A_log, dt_bias, beta, gdec, H, T);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- recurrences over a matrix state --------------------------------------------------------------------------------
// State S [dim, vdim] per (request, head), float32, stored column by column ([vdim][dim]: the dim entries that one output
// column needs lie together). A block owns `blockDim.x` columns of one head of one entry, one column a
// thread, the column in shared memory (column c of row d at s[d * (ncol + 1) + c]: no bank is shared). Tokens in order:
//   MODE 0 (decayed sum):  S = decay_h S + k v^T;                               o = S^T q
//   MODE 1 (delta rule):   S = g_t S;  u = beta_t (v - S^T k);  S = S + k u^T;   o = S^T q
//   MODE 3 (gated sum):    S = g_t S + beta_t k [v, 1]^T;                        o = S^T q   - per-token decay and input
//                          weight; the state has one column more than v (vdim counts it), fed by the constant 1: it gathers
//                          the weighted keys alone (the normaliser of a matrix memory), and the output's last column is its
//                          product with q. v heads are vdim - 1 wide, the output's vdim.
//   MODE 4 (channel decay): o = (S + diag(u_h) k v^T)^T q;  then  S = diag(w_t) S + k v^T   - a decay per token, head and key
//                          channel (w: float32 rows of H * dim, row stride ld_g, passed as `gdec`), and a bonus u (float32
//                          [H, dim], passed as `decay`) that lets the token's own k v^T into its read-out without entering
//                          the state: the read-out comes BEFORE the state moves on.
// q and k of SM_CHUNK tokens are staged in shared memory at a time. `in_act` 1: silu on q, k, v as they are read.
// q/k head of value head h: h / (H / G). This form takes every size; key sizes up to 256 run the register form below
// (`generic` 0), which gives the same sums in another order.
#define SM_CHUNK 8
template <int MODE>
__global__ void matrix_state_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int ld_q,
                                         int ld_k, int ld_v, int H, int G, int dim, int vdim, int in_act,
                                         const float* __restrict__ decay, const float* __restrict__ beta, const float* __restrict__ gdec,
                                         float* state, size_t slot_stride, const int* __restrict__ read_slots,
                                         const int* __restrict__ write_slots, const int* __restrict__ qstart, float* __restrict__ out,
                                         int ldo, int e0, int ld_g) {
    extern __shared__ float sm[];
    const int ncol = blockDim.x;
    const int ncs = ncol + 1;
    float* S = sm;                                // [dim][ncol + 1]
    float* qs = sm + (size_t)dim * ncs;           // [SM_CHUNK][dim]
    float* ks = qs + SM_CHUNK * dim;              // [SM_CHUNK][dim]
    const int e = e0 + blockIdx.x, h = blockIdx.y, c = blockIdx.z * ncol + threadIdx.x;
    const int q0 = qstart[e], n = qstart[e + 1] - q0;
    if (n <= 0) return;
    const int hq = h / (H / G);
    const bool live = c < vdim;
    const int c0 = blockIdx.z * ncol;
    const float* rd = state + (size_t)read_slots[e] * slot_stride + (size_t)h * dim * vdim;
    for (int i = threadIdx.x; i < ncol * dim; i += ncol) {
        const int cc = i / dim, d = i - cc * dim;
        S[d * ncs + cc] = c0 + cc < vdim ? rd[(size_t)(c0 + cc) * dim + d] : 0.f;
    }
    __syncthreads();
    const float dec = MODE == 0 ? decay[h] : 0.f;
    for (int t0 = 0; t0 < n; t0 += SM_CHUNK) {
        const int nt = min(SM_CHUNK, n - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * dim; i += ncol) {
            const int tt = i / dim, d = i - tt * dim;
            const size_t row = (size_t)(q0 + t0 + tt);
            float a = q[row * ld_q + hq * dim + d], b = k[row * ld_k + hq * dim + d];
            if (in_act) a = sm_silu_fast(a), b = sm_silu_fast(b);
            qs[i] = a, ks[i] = b;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const size_t row = (size_t)(q0 + t0 + tt);
            float vc = MODE == 3 ? (c < vdim - 1 ? v[row * ld_v + h * (vdim - 1) + c] : c == vdim - 1 ? 1.f : 0.f)
                                 : live ? v[row * ld_v + h * vdim + c] : 0.f;
            if (in_act) vc = sm_silu_fast(vc);
            const float* qq = qs + tt * dim;
            const float* kk = ks + tt * dim;
            float o = 0.f;
            if (MODE == 0) {
                for (int d = 0; d < dim; ++d) {
                    const float s = fmaf(dec, S[d * ncs + threadIdx.x], kk[d] * vc);
                    S[d * ncs + threadIdx.x] = s;
                    o = fmaf(s, qq[d], o);
                }
            } else if (MODE == 3) {
                const float g = gdec[row * H + h], u = beta[row * H + h] * vc;
                for (int d = 0; d < dim; ++d) {
                    const float s = fmaf(g, S[d * ncs + threadIdx.x], kk[d] * u);
                    S[d * ncs + threadIdx.x] = s;
                    o = fmaf(s, qq[d], o);
                }
            } else if (MODE == 4) {
                const float* ww = gdec + row * ld_g + (size_t)h * dim;
                const float* uu = decay + (size_t)h * dim;
                for (int d = 0; d < dim; ++d) {
                    const float kv = kk[d] * vc, s = S[d * ncs + threadIdx.x];
                    o = fmaf(qq[d], fmaf(uu[d], kv, s), o);
                    S[d * ncs + threadIdx.x] = fmaf(ww[d], s, kv);
                }
            } else {
                const float g = gdec[row * H + h], bt = beta[row * H + h];
                float sk = 0.f;
                for (int d = 0; d < dim; ++d) {
                    const float s = g * S[d * ncs + threadIdx.x];
                    S[d * ncs + threadIdx.x] = s;
                    sk = fmaf(s, kk[d], sk);
                }
                const float u = bt * (vc - sk);
                for (int d = 0; d < dim; ++d) {
                    const float s = fmaf(kk[d], u, S[d * ncs + threadIdx.x]);
                    S[d * ncs + threadIdx.x] = s;
                    o = fmaf(s, qq[d], o);
                }
            }
            if (live) out[row * ldo + h * vdim + c] = o;
        }
    }
    __syncthreads();
    float* wr = state + (size_t)write_slots[e] * slot_stride + (size_t)h * dim * vdim;
    for (int i = threadIdx.x; i < ncol * dim; i += ncol) {
        const int cc = i / dim, d = i - cc * dim;
        if (c0 + cc < vdim) wr[(size_t)(c0 + cc) * dim + d] = S[d * ncs + cc];
    }
}

// The same recurrences with the state in registers. A column of S is shared by `split` neighbouring lanes, each holding
// DPT of its rows (rows beyond dim are padding: their q and k are staged as zeros, so they stay zero); the dot products
// S^T k and S^T q are finished by xor-shuffles among those lanes. A block is 128 threads = 128 / split columns of one head
// of one entry. q, k, v (and the delta rule's g and beta) of SR_CHUNK tokens (8; 1 in the form for entries that bring a single
// token, which then needs few registers and many blocks fit an SM) are staged in shared memory; the next
// chunk's values are loaded into registers while the current chunk is computed, so the token loop waits for no global
// load. Per token the critical path is one multiply, one dot product of DPT terms, log2(split) shuffles and one update.
#define SR_THREADS 128
template <int MODE, int DPT, int SR_CHUNK, int SR_MAX_SPLIT>
__global__ void __launch_bounds__(SR_THREADS) matrix_state_scan_reg_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int ld_q, int ld_k, int ld_v, int H, int G,
    int dim, int vdim, int in_act, const float* __restrict__ decay, const float* __restrict__ beta, const float* __restrict__ gdec,
    float* state, size_t slot_stride, const int* __restrict__ read_slots, const int* __restrict__ write_slots,
    const int* __restrict__ qstart, float* __restrict__ out, int ldo, int log_split, int e0, int n_ent, int seg_len, float* seg_state,
    int ld_g) {
    extern __shared__ float sm[];
    constexpr int LOG_DPT = DPT == 8 ? 3 : DPT == 16 ? 4 : 5;
    constexpr int SEG = DPT + 4;                  // a lane's DPT values of q (or k) and 4 floats of padding: the lanes of a column then
                                                  // read their 16-byte pieces from different banks
    const int split = 1 << log_split, dimp = DPT << log_split;
    const int cpb = SR_THREADS >> log_split, log_cpb = 7 - log_split;
    const int row_f = SEG << log_split;           // floats of a staged token's q (or k)
    float* qs = sm;                               // [SR_CHUNK][split][SEG]
    float* ks = qs + SR_CHUNK * row_f;            // [SR_CHUNK][split][SEG]
    float* vs = ks + SR_CHUNK * row_f;            // [SR_CHUNK][cpb]
    float* gb = vs + SR_CHUNK * cpb;              // [2][SR_CHUNK]: g, beta
    float* wsm = gb + ((2 * SR_CHUNK + 3) & ~3);  // MODE 4: [SR_CHUNK][split][SEG], the decays of the key channels, laid out as k
    const int h = blockIdx.y, tid = threadIdx.x;
    const int part = tid & (split - 1), col_l = tid >> log_split, c = blockIdx.z * cpb + col_l;
    // Which tokens this block walks. Plain form (seg_len 0): entry e0 + blockIdx.x, all of it. Segmented form (the decayed
    // sum of long portions): blockIdx.x counts segments of seg_len tokens, entry after entry; segment p of an entry starts
    // from nothing (p > 0) and leaves what it gathered in seg_state, and a second pass (MODE 2) adds what the state at the
    // segment's start contributes: S is linear in its start, o_t += decay^(t - t0 + 1) S_start^T q_t.
    int e = e0 + blockIdx.x, q0, n, p = 0, n_seg = 1, first_tile = 0;
    if (seg_len > 0) {
        int tile = blockIdx.x;
        for (e = e0;; ++e) {
            if (e >= e0 + n_ent) return;          // a surplus block (the grid is a bound)
            const int a = qstart[e], cnt = (qstart[e + 1] - a + seg_len - 1) / seg_len;
            if (tile < cnt) {
                p = tile, n_seg = cnt, first_tile = blockIdx.x - tile;
                break;
            }
            tile -= cnt;
        }
        const int a = qstart[e], len = qstart[e + 1] - a;
        q0 = a + p * seg_len;
        n = min(seg_len, len - p * seg_len);
        if (MODE == 2 && p == 0) return;          // the first segment started from the request's own state: nothing to add
    } else {
        q0 = qstart[e];
        n = qstart[e + 1] - q0;
    }
    if (n <= 0) return;
    const int hq = h / (H / G);
    const bool live = c < vdim;
    const int d0 = part * DPT;
    float S[DPT];
    const float dec = (MODE == 0 || MODE == 2) ? decay[h] : 0.f;
    auto load_cols = [&](const float* src, float* dst) {      // this lane's DPT rows of column c from a [vdim][dim] matrix
        if (live && (dim & 3) == 0) {             // a column's rows lie together: 16 bytes a load (dim a multiple of 4 keeps them aligned)
#pragma unroll
            for (int i = 0; i < DPT; i += 4) {
                const float4 x = d0 + i < dim ? *reinterpret_cast<const float4*>(src + (size_t)c * dim + d0 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                dst[i] = x.x, dst[i + 1] = x.y, dst[i + 2] = x.z, dst[i + 3] = x.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < DPT; ++i) dst[i] = (live && d0 + i < dim) ? src[(size_t)c * dim + d0 + i] : 0.f;
        }
    };
    auto store_cols = [&](float* dst, const float* src) {
        if (!live) return;
        if ((dim & 3) == 0) {
#pragma unroll
            for (int i = 0; i < DPT; i += 4)
                if (d0 + i < dim) *reinterpret_cast<float4*>(dst + (size_t)c * dim + d0 + i) = make_float4(src[i], src[i + 1], src[i + 2], src[i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < DPT; ++i)
                if (d0 + i < dim) dst[(size_t)c * dim + d0 + i] = src[i];
        }
    };
    const size_t head_f = (size_t)dim * vdim;     // floats of one head's state
    if (MODE == 2) {
        // the state at this segment's start: what the segments before it gathered, each decayed over those behind it
        const float dseg = powf(dec, (float)seg_len);
        load_cols(seg_state + ((size_t)first_tile * H + h) * head_f, S);
        for (int j = 1; j < p; ++j) {
            float L[DPT];
            load_cols(seg_state + ((size_t)(first_tile + j) * H + h) * head_f, L);
#pragma unroll
            for (int i = 0; i < DPT; ++i) S[i] = fmaf(dseg, S[i], L[i]);
        }
        if (p == n_seg - 1) {                     // the last segment also leaves the request's state: its start decayed over it, plus its own
            float L[DPT];
            load_cols(seg_state + ((size_t)(first_tile + p) * H + h) * head_f, L);
            const float dn = powf(dec, (float)n);
#pragma unroll
            for (int i = 0; i < DPT; ++i) L[i] = fmaf(dn, S[i], L[i]);
            store_cols(state + (size_t)write_slots[e] * slot_stride + (size_t)h * head_f, L);
        }
    } else if (p == 0) {
        load_cols(state + (size_t)read_slots[e] * slot_stride + (size_t)h * head_f, S);
    } else {
#pragma unroll
        for (int i = 0; i < DPT; ++i) S[i] = 0.f;
    }
    // Staging: a token's values are fetched by TPT = 128 / SR_CHUNK neighbouring threads, thread l of them taking entries
    // l, l + TPT, ...: one base address a chunk, then constant strides, in global and in shared memory alike.
    constexpr int TPT = SR_THREADS / SR_CHUNK;
    constexpr int NQ = (DPT * SR_MAX_SPLIT + TPT - 1) / TPT;       // q (and k) values per thread at the widest split
    constexpr int NV = (SR_THREADS + TPT - 1) / TPT;               // v values per thread at split 1
    static_assert(TPT >= DPT, "a staging thread's entries must fall into whole lane segments");
    float qr[NQ], kr[NQ], vr[NV], gr = 0.f, wr_[MODE == 4 ? NQ : 1];
    float U[MODE == 4 ? DPT : 1];                 // MODE 4: the bonus of this lane's key channels
    if (MODE == 4) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) U[i] = d0 + i < dim ? decay[(size_t)h * dim + d0 + i] : 0.f;
    }
    const int s_tt = tid / TPT, s_l = tid % TPT;
    const int s_at = s_tt * row_f + (s_l >> LOG_DPT) * SEG + (s_l & (DPT - 1));   // + j * (TPT >> LOG_DPT) * SEG

    auto fetch = [&](int t0) {                    // the chunk's values into registers (zeros beyond the entry's end and in padding)
        const bool tok = t0 + s_tt < n;
        const size_t row = (size_t)(q0 + t0 + s_tt);
        const float* qp = q + row * ld_q + hq * dim + s_l;
        const float* kp = k + row * ld_k + hq * dim + s_l;
#pragma unroll
        for (int j = 0; j < NQ; ++j) {
            const bool ok = tok && s_l + j * TPT < dim;
            qr[j] = ok ? qp[j * TPT] : 0.f;
            kr[j] = (MODE != 2 && ok) ? kp[j * TPT] : 0.f;
            if (MODE == 4) wr_[j] = ok ? gdec[row * ld_g + (size_t)h * dim + s_l + j * TPT] : 0.f;
        }
        if (MODE == 3) {                          // v heads are vdim - 1 wide; the state's last column is fed by the constant 1
            const float* vp = v + row * ld_v + h * (vdim - 1) + blockIdx.z * cpb + s_l;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int cc = blockIdx.z * cpb + s_l + j * TPT;
                vr[j] = (tok && s_l + j * TPT < cpb) ? (cc < vdim - 1 ? vp[j * TPT] : cc == vdim - 1 ? 1.f : 0.f) : 0.f;
            }
        } else if (MODE != 2) {
            const float* vp = v + row * ld_v + h * vdim + blockIdx.z * cpb + s_l;
#pragma unroll
            for (int j = 0; j < NV; ++j)
                vr[j] = (tok && s_l + j * TPT < cpb && blockIdx.z * cpb + s_l + j * TPT < vdim) ? vp[j * TPT] : 0.f;
        }
        if ((MODE == 1 || MODE == 3) && tid < 2 * SR_CHUNK) {
            const int tt = tid & (SR_CHUNK - 1);
            gr = t0 + tt < n ? (tid < SR_CHUNK ? gdec : beta)[(size_t)(q0 + t0 + tt) * H + h] : 0.f;
        }
    };
    auto stage = [&]() {                          // registers to shared memory, the activation applied once per value
#pragma unroll
        for (int j = 0; j < NQ; ++j)
            if (s_l + j * TPT < dimp) {
                qs[s_at + j * (TPT >> LOG_DPT) * SEG] = in_act ? sm_silu_fast(qr[j]) : qr[j];
                if (MODE != 2) ks[s_at + j * (TPT >> LOG_DPT) * SEG] = in_act ? sm_silu_fast(kr[j]) : kr[j];
                if (MODE == 4) wsm[s_at + j * (TPT >> LOG_DPT) * SEG] = wr_[j];
            }
        if (MODE != 2) {
#pragma unroll
            for (int j = 0; j < NV; ++j)
                if (s_l + j * TPT < cpb) vs[(s_tt << log_cpb) + s_l + j * TPT] = in_act ? sm_silu_fast(vr[j]) : vr[j];
        }
        if ((MODE == 1 || MODE == 3) && tid < 2 * SR_CHUNK) gb[tid] = gr;
    };

    fetch(0);
    stage();
    __syncthreads();
    // The tokens of a chunk are unrolled (a token beyond the entry's end is skipped by a predicate), so that the loads of
    // a later token's q and k are issued while an earlier token's products run; and a token's output is only summed over
    // the lanes of its column when the chunk is done: its shuffles then wait for one another's results, not the tokens.
    for (int t0 = 0; t0 < n; t0 += SR_CHUNK) {
        const int nt = min(SR_CHUNK, n - t0);
        if (t0 + SR_CHUNK < n) fetch(t0 + SR_CHUNK);
        float oacc[SR_CHUNK], oold[MODE == 2 ? SR_CHUNK : 1];
        if (MODE == 2 && live && part == 0) {     // what the first pass wrote, asked for before the products
#pragma unroll
            for (int tt = 0; tt < SR_CHUNK; ++tt) oold[tt] = tt < nt ? out[(size_t)(q0 + t0 + tt) * ldo + h * vdim + c] : 0.f;
        }
#pragma unroll
        for (int tt = 0; tt < SR_CHUNK; ++tt) {
            oacc[tt] = 0.f;
            if (tt < nt) {
                const float4* qq = reinterpret_cast<const float4*>(qs + tt * row_f + part * SEG);
                const float4* kk = reinterpret_cast<const float4*>(ks + tt * row_f + part * SEG);
                const float vc = MODE != 2 ? vs[(tt << log_cpb) + col_l] : 0.f;
                float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
                if (MODE == 2) {
#pragma unroll
                    for (int i = 0; i < DPT / 4; ++i) {
                        const float4 q4 = qq[i];
                        o0 = fmaf(S[4 * i], q4.x, o0), o1 = fmaf(S[4 * i + 1], q4.y, o1);
                        o2 = fmaf(S[4 * i + 2], q4.z, o2), o3 = fmaf(S[4 * i + 3], q4.w, o3);
                    }
                } else if (MODE == 0) {
#pragma unroll
                    for (int i = 0; i < DPT / 4; ++i) {
                        const float4 k4 = kk[i], q4 = qq[i];
                        S[4 * i] = fmaf(dec, S[4 * i], k4.x * vc);
                        S[4 * i + 1] = fmaf(dec, S[4 * i + 1], k4.y * vc);
                        S[4 * i + 2] = fmaf(dec, S[4 * i + 2], k4.z * vc);
                        S[4 * i + 3] = fmaf(dec, S[4 * i + 3], k4.w * vc);
                        o0 = fmaf(S[4 * i], q4.x, o0), o1 = fmaf(S[4 * i + 1], q4.y, o1);
                        o2 = fmaf(S[4 * i + 2], q4.z, o2), o3 = fmaf(S[4 * i + 3], q4.w, o3);
                    }
                } else if (MODE == 4) {
                    // the read-out first (the state before this token, plus the token's own k v^T weighted by the bonus), then
                    // the state moves on under this token's decays
                    const float4* ww = reinterpret_cast<const float4*>(wsm + tt * row_f + part * SEG);
#pragma unroll
                    for (int i = 0; i < DPT / 4; ++i) {
                        const float4 k4 = kk[i], q4 = qq[i], w4 = ww[i];
                        const float a0 = k4.x * vc, a1 = k4.y * vc, a2 = k4.z * vc, a3 = k4.w * vc;
                        o0 = fmaf(q4.x, fmaf(U[4 * i], a0, S[4 * i]), o0), o1 = fmaf(q4.y, fmaf(U[4 * i + 1], a1, S[4 * i + 1]), o1);
                        o2 = fmaf(q4.z, fmaf(U[4 * i + 2], a2, S[4 * i + 2]), o2), o3 = fmaf(q4.w, fmaf(U[4 * i + 3], a3, S[4 * i + 3]), o3);
                        S[4 * i] = fmaf(w4.x, S[4 * i], a0), S[4 * i + 1] = fmaf(w4.y, S[4 * i + 1], a1);
                        S[4 * i + 2] = fmaf(w4.z, S[4 * i + 2], a2), S[4 * i + 3] = fmaf(w4.w, S[4 * i + 3], a3);
                    }
                } else if (MODE == 3) {
                    const float g = gb[tt], u = gb[SR_CHUNK + tt] * vc;
#pragma unroll
                    for (int i = 0; i < DPT / 4; ++i) {
                        const float4 k4 = kk[i], q4 = qq[i];
                        S[4 * i] = fmaf(g, S[4 * i], k4.x * u);
                        S[4 * i + 1] = fmaf(g, S[4 * i + 1], k4.y * u);
                        S[4 * i + 2] = fmaf(g, S[4 * i + 2], k4.z * u);
                        S[4 * i + 3] = fmaf(g, S[4 * i + 3], k4.w * u);
                        o0 = fmaf(S[4 * i], q4.x, o0), o1 = fmaf(S[4 * i + 1], q4.y, o1);
                        o2 = fmaf(S[4 * i + 2], q4.z, o2), o3 = fmaf(S[4 * i + 3], q4.w, o3);
                    }
                } else {
                    // g scales the whole state, so S^T k of the scaled state is g times that of the old one, and the
                    // scaling joins the update as one fused multiply-add: S = g S + k u
                    const float g = gb[tt], bt = gb[SR_CHUNK + tt];
                    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                    for (int i = 0; i < DPT / 4; ++i) {
                        const float4 k4 = kk[i];
                        s0 = fmaf(S[4 * i], k4.x, s0), s1 = fmaf(S[4 * i + 1], k4.y, s1);
                        s2 = fmaf(S[4 * i + 2], k4.z, s2), s3 = fmaf(S[4 * i + 3], k4.w, s3);
                    }
                    float sk = (s0 + s1) + (s2 + s3);
#pragma unroll
                    for (int m = SR_MAX_SPLIT / 2; m > 0; m >>= 1)
                        if (m < split) sk += __shfl_xor_sync(0xffffffffu, sk, m);
                    const float u = bt * (vc - g * sk);
#pragma unroll
                    for (int i = 0; i < DPT / 4; ++i) {
                        const float4 k4 = kk[i], q4 = qq[i];
                        S[4 * i] = fmaf(g, S[4 * i], k4.x * u);
                        S[4 * i + 1] = fmaf(g, S[4 * i + 1], k4.y * u);
                        S[4 * i + 2] = fmaf(g, S[4 * i + 2], k4.z * u);
                        S[4 * i + 3] = fmaf(g, S[4 * i + 3], k4.w * u);
                        o0 = fmaf(S[4 * i], q4.x, o0), o1 = fmaf(S[4 * i + 1], q4.y, o1);
                        o2 = fmaf(S[4 * i + 2], q4.z, o2), o3 = fmaf(S[4 * i + 3], q4.w, o3);
                    }
                }
                oacc[tt] = (o0 + o1) + (o2 + o3);
            }
        }
#pragma unroll
        for (int m = SR_MAX_SPLIT / 2; m > 0; m >>= 1)
            if (m < split) {
#pragma unroll
                for (int tt = 0; tt < SR_CHUNK; ++tt) oacc[tt] += __shfl_xor_sync(0xffffffffu, oacc[tt], m);
            }
        if (live && part == 0) {
            if (MODE == 2) {                      // token i of the segment sees its start through i + 1 decays
                float pw = powf(dec, (float)(t0 + 1));
#pragma unroll
                for (int tt = 0; tt < SR_CHUNK; ++tt) {
                    if (tt < nt) out[(size_t)(q0 + t0 + tt) * ldo + h * vdim + c] = fmaf(pw, oacc[tt], oold[tt]);
                    pw *= dec;
                }
            } else {
#pragma unroll
                for (int tt = 0; tt < SR_CHUNK; ++tt)
                    if (tt < nt) out[(size_t)(q0 + t0 + tt) * ldo + h * vdim + c] = oacc[tt];
            }
        }
        __syncthreads();                          // everyone has read this chunk
        if (t0 + SR_CHUNK < n) stage();
        __syncthreads();
    }
    if (MODE != 2) {
        // what this block gathered: the request's state, or - a segment of several - its share for the second pass
        if (n_seg == 1) store_cols(state + (size_t)write_slots[e] * slot_stride + (size_t)h * head_f, S);
        else store_cols(seg_state + ((size_t)blockIdx.x * H + h) * head_f, S);
    }
}

template <int MODE, int DPT, int CH, int MS>
static void sr_launch(dim3 grid, size_t smem, cudaStream_t stream, const float* q, const float* k, const float* v, int ld_q, int ld_k, int ld_v,
                      int H, int G, int dim, int vdim, int in_act, const float* decay, const float* beta, const float* gdec, float* state,
                      size_t slot_stride, const int* read_slots, const int* write_slots, const int* qstart, float* out, int ldo, int log_split,
                      int e0, int n_ent, int seg_len, float* seg_state, int ld_g) {
    matrix_state_scan_reg_kernel<MODE, DPT, CH, MS><<<grid, SR_THREADS, smem, stream>>>(q, k, v, ld_q, ld_k, ld_v, H, G, dim, vdim, in_act, decay, beta,
                                                                                    gdec, state, slot_stride, read_slots, write_slots, qstart, out,
                                                                                    ldo, log_split, e0, n_ent, seg_len, seg_state, ld_g);
}

// In place: x[t, c] = silu(x[t, c]) for the first `cols` columns of float32 rows (the recurrences' inputs, as a pass of its own).
__global__ void silu_cols_kernel(float* x, int ld, int cols, int T) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        float* p = x + (size_t)t * ld + c;
        *p = sm_silu_fast(*p);
    }
}

IL_EXPORT int il_silu_cols(float* x, int ld, int cols, int T, cudaStream_t stream) {
    if (T <= 0 || cols <= 0) return IL_OK;
    silu_cols_kernel<<<dim3((cols + 255) / 256, T < 32768 ? T : 32768), 256, 0, stream>>>(x, ld, cols, T);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

IL_EXPORT int il_matrix_state_scan(int mode, const float* q, const float* k, const float* v, int ld_q, int ld_k, int ld_v, int H, int G,
                                   int dim, int vdim, int in_act, const float* decay, const float* beta, const float* gdec, float* state,
                                   long long slot_stride, const int* read_slots, const int* write_slots, const int* qstart, int E,
                                   float* out, int ldo, int generic, int e0, int single, int seg_len, int n_tiles, float* seg_state,
                                   int ld_g, cudaStream_t stream) {
    // mode 4: `gdec` holds the decays per token and key channel (float32 rows of H * dim, row stride ld_g), `decay` the bonus
    // [H, dim]; G = H.
    if (E <= 0) return IL_OK;
    if (e0 < 0) return IL_BAD_ARG;
    // seg_len > 0 (decayed sum, register form only): the entries' tokens in segments of seg_len, n_tiles of them at most
    // (a bound is enough), seg_state float32 [n_tiles, H, vdim, dim] scratch; two passes.
    if (seg_len > 0 && (mode != 0 || generic || single || dim > 256 || n_tiles <= 0 || !seg_state || seg_len % 8)) return IL_BAD_ARG;
    if (H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || (mode != 0 && mode != 1 && mode != 3 && mode != 4)) return IL_BAD_ARG;
    if (mode == 3 && (vdim < 2 || in_act)) return IL_BAD_ARG;
    if (mode == 4 ? (!decay || !gdec || G != H || in_act || ld_g < H * dim) : mode == 0 ? !decay : (!beta || !gdec)) return IL_BAD_ARG;
    if (dim <= 256 && !generic) {
        // Rows of a column per lane (8 or 16) and lanes per column (a power of two up to 16) that cover dim. Few blocks (one
        // long prompt) of the decayed sum take the narrower lanes: twice the warps, each with half the products per token
        // (measured at 16 heads of 128 x 128 over 2,048 tokens: 945 -> 695 us); the delta rule, whose sum over the lanes
        // stands between a token's two updates, loses by the longer shuffle chain (648 -> 771 us) and keeps 16.
        int dpt = dim <= 32 ? 8 : 16;
        if ((mode == 0 || mode == 4) && dim > 32 && dim <= 128) {       // (the channel decay, like the decayed sum, has no sum over the lanes between a token's updates)
            const int cols16 = SR_THREADS / ((dim + 15) / 16 <= 1 ? 1 : (dim <= 32 ? 2 : dim <= 64 ? 4 : 8));
            if ((long long)(seg_len > 0 ? n_tiles : E) * H * ((vdim + cols16 - 1) / cols16) <= 148) dpt = 8;     // at most one block an SM otherwise
        }
        int log_split = 0;
        while ((dpt << log_split) < dim) ++log_split;
        const int cpb = SR_THREADS >> log_split;
        const int ch = single ? 1 : 8;
        const size_t smem_r = ((size_t)ch * ((mode == 4 ? 3 : 2) * ((dpt + 4) << log_split) + cpb) + ((2 * ch + 3) & ~3)) * sizeof(float);
        const dim3 grid_r(seg_len > 0 ? n_tiles : E, H, (vdim + cpb - 1) / cpb);
#define SR_ARGS grid_r, smem_r, stream, q, k, v, ld_q, ld_k, ld_v, H, G, dim, vdim, in_act, decay, beta, gdec, state, (size_t)slot_stride, \
                read_slots, write_slots, qstart, out, ldo, log_split, e0, E, seg_len, seg_state, ld_g
        // (the widest split a variant is built for sizes its staging registers: 8 lanes up to dim = 8 DPT, 16 beyond)
#define SR_PICK(MODE_, DPT_)                                                                                     \
        do {                                                                                                     \
            if (log_split <= 3) { if (single) sr_launch<MODE_, DPT_, 1, 8>(SR_ARGS); else sr_launch<MODE_, DPT_, 8, 8>(SR_ARGS); } \
            else { if (single) sr_launch<MODE_, DPT_, 1, 16>(SR_ARGS); else sr_launch<MODE_, DPT_, 8, 16>(SR_ARGS); }               \
        } while (0)
        if (mode == 0) {
            if (dpt == 8) SR_PICK(0, 8); else SR_PICK(0, 16);
            if (seg_len > 0) {                    // the second pass: what each segment's start contributes
                IL_LAUNCH_CHECK();
                if (log_split <= 3) { if (dpt == 8) sr_launch<2, 8, 8, 8>(SR_ARGS); else sr_launch<2, 16, 8, 8>(SR_ARGS); }
                else { if (dpt == 8) sr_launch<2, 8, 8, 16>(SR_ARGS); else sr_launch<2, 16, 8, 16>(SR_ARGS); }
            }
        } else if (mode == 1) {
            if (dpt == 8) SR_PICK(1, 8); else SR_PICK(1, 16);
        } else if (mode == 4) {
            if (dpt == 8) SR_PICK(4, 8); else SR_PICK(4, 16);
        } else {
            if (dpt == 8) SR_PICK(3, 8); else SR_PICK(3, 16);
        }
        IL_LAUNCH_CHECK();
        return IL_OK;
    }
    int ncol = vdim >= 128 ? 128 : vdim > 32 ? 64 : 32;
    size_t smem = ((size_t)dim * (ncol + 1) + 2 * SM_CHUNK * dim) * sizeof(float);
    while (smem > 200 * 1024 && ncol > 32) {
        ncol >>= 1;
        smem = ((size_t)dim * (ncol + 1) + 2 * SM_CHUNK * dim) * sizeof(float);
    }
    if (smem > 200 * 1024) return IL_UNSUPPORTED;
    const dim3 grid(E, H, (vdim + ncol - 1) / ncol);
    if (mode == 4) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(matrix_state_scan_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        matrix_state_scan_kernel<4><<<grid, ncol, smem, stream>>>(q, k, v, ld_q, ld_k, ld_v, H, G, dim, vdim, in_act, decay, beta, gdec, state,
                                                                  (size_t)slot_stride, read_slots, write_slots, qstart, out, ldo, e0, ld_g);
    } else if (mode == 3) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(matrix_state_scan_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        matrix_state_scan_kernel<3><<<grid, ncol, smem, stream>>>(q, k, v, ld_q, ld_k, ld_v, H, G, dim, vdim, in_act, decay, beta, gdec, state,
                                                                  (size_t)slot_stride, read_slots, write_slots, qstart, out, ldo, e0, ld_g);
    } else if (mode == 0) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(matrix_state_scan_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        matrix_state_scan_kernel<0><<<grid, ncol, smem, stream>>>(q, k, v, ld_q, ld_k, ld_v, H, G, dim, vdim, in_act, decay, beta, gdec, state,
                                                                  (size_t)slot_stride, read_slots, write_slots, qstart, out, ldo, e0, ld_g);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(matrix_state_scan_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        matrix_state_scan_kernel<1><<<grid, ncol, smem, stream>>>(q, k, v, ld_q, ld_k, ld_v, H, G, dim, vdim, in_act, decay, beta, gdec, state,
                                                                  (size_t)slot_stride, read_slots, write_slots, qstart, out, ldo, e0, ld_g);
    }
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- a norm over groups of columns, times a gate -----------------------------------------------------------------------
// out[t, j] = x[t, j] / sqrt(mean over j's group of x^2 + eps) * w[j % n_w] * act(gate[t, j]); groups of `group` columns;
// act 0: sigmoid, 1: silu. x float32, the gate float32 or bfloat16, out float32 or bfloat16. One block per (row, group).
// With `den_floor` (float32 [T, groups]) a group of x is group + 1 columns wide, its last column the read-out's normaliser:
// the group is first divided by max(|x_scale * that column|, den_floor[t, g]) + den_eps (and multiplied by x_scale) - the
// output of a matrix memory whose numerator and normaliser were read with the same unscaled query.
template <typename TG, typename TO>
__global__ void group_norm_gate_kernel(const float* __restrict__ x, int ldx, const void* __restrict__ w, int w_kind, int n_w, float eps,
                                       const TG* __restrict__ gate, int ldg, int g_off, int act, TO* __restrict__ out, int ldo, int group,
                                       const float* __restrict__ den_floor, float x_scale, float den_eps) {
    __shared__ float red[32];
    const int t = blockIdx.x, j0 = blockIdx.y * group;
    const float* xr = x + (size_t)t * ldx + (den_floor ? blockIdx.y * (group + 1) : j0);
    float pre = 1.f;
    if (den_floor) pre = x_scale / (fmaxf(fabsf(x_scale * xr[group]), den_floor[(size_t)t * gridDim.y + blockIdx.y]) + den_eps);
    float ss = 0.f;
    for (int j = threadIdx.x; j < group; j += blockDim.x) ss += (xr[j] * pre) * (xr[j] * pre);
    ss = il_block_sum(ss, red);
    const float r = pre * (1.f / sqrtf(ss / (float)group + eps));
    for (int j = threadIdx.x; j < group; j += blockDim.x) {
        const float z = il_to_f(gate[(size_t)t * ldg + g_off + j0 + j]);
        const float a = act == 0 ? sm_sigmoid(z) : sm_silu(z);
        out[(size_t)t * ldo + j0 + j] = il_from_f<TO>(xr[j] * r * il_load_any(w, w_kind, (j0 + j) % n_w) * a);
    }
}

static int group_norm_gate_launch(const float* x, int ldx, const void* w, int w_kind, int n_w, float eps, const void* gate, int gate_kind,
                                  int ldg, int g_off, int act, void* out, int out_kind, int ldo, int group, int n_groups, int T,
                                  const float* den_floor, float x_scale, float den_eps, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (group <= 0 || n_groups <= 0 || n_w <= 0) return IL_BAD_ARG;
    // (a group of thousands of columns is one block: many threads, two to four columns each, keep its two passes short)
    const int threads = group >= 2048 ? 1024 : group >= 1024 ? 512 : group >= 256 ? 256 : group >= 128 ? 128 : 64;
    const dim3 grid(T, n_groups);
#define GN_ARGS x, ldx, w, w_kind, n_w, eps
    if (gate_kind == IL_F32 && out_kind == IL_F32)
        group_norm_gate_kernel<float, float><<<grid, threads, 0, stream>>>(GN_ARGS, (const float*)gate, ldg, g_off, act, (float*)out, ldo, group, den_floor, x_scale, den_eps);
    else if (gate_kind == IL_F32 && out_kind == IL_BF16)
        group_norm_gate_kernel<float, __nv_bfloat16><<<grid, threads, 0, stream>>>(GN_ARGS, (const float*)gate, ldg, g_off, act, (__nv_bfloat16*)out, ldo, group, den_floor, x_scale, den_eps);
    else if (gate_kind == IL_BF16 && out_kind == IL_BF16)
        group_norm_gate_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, threads, 0, stream>>>(GN_ARGS, (const __nv_bfloat16*)gate, ldg, g_off, act, (__nv_bfloat16*)out, ldo, group, den_floor, x_scale, den_eps);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

IL_EXPORT int il_group_norm_gate(const float* x, int ldx, const void* w, int w_kind, int n_w, float eps, const void* gate, int gate_kind,
                                 int ldg, int g_off, int act, void* out, int out_kind, int ldo, int group, int n_groups, int T,
                                 cudaStream_t stream) {
    return group_norm_gate_launch(x, ldx, w, w_kind, n_w, eps, gate, gate_kind, ldg, g_off, act, out, out_kind, ldo, group, n_groups, T,
                                  nullptr, 1.f, 0.f, stream);
}

// x [T, groups * (group + 1)]: every group followed by its normaliser column (see the kernel).
IL_EXPORT int il_group_norm_gate_den(const float* x, int ldx, const void* w, int w_kind, int n_w, float eps, const void* gate, int gate_kind,
                                     int ldg, int g_off, int act, void* out, int out_kind, int ldo, int group, int n_groups, int T,
                                     const float* den_floor, float x_scale, float den_eps, cudaStream_t stream) {
    if (!den_floor) return IL_BAD_ARG;
    return group_norm_gate_launch(x, ldx, w, w_kind, n_w, eps, gate, gate_kind, ldg, g_off, act, out, out_kind, ldo, group, n_groups, T,
                                  den_floor, x_scale, den_eps, stream);
}

// ---- log-space gates with a running maximum ------------------------------------------------------------------------------
// A matrix memory with exponential gates keeps its sums scaled by exp(-m), m the running maximum of the log weights:
//   i_t = cap tanh(zi_t / cap),  f_t = logsigmoid(cap tanh(zf_t / cap))          (cap <= 0: zi, logsigmoid(zf) as they are)
//   m_t = max(f_t + m_(t-1), i_t);  decay_t = exp(f_t + m_(t-1) - m_t);  inw_t = exp(i_t - m_t);  floor_t = exp(-m_t)
// m is part of the request's state (float32 [slots, heads]; the zero slot gives m = 0). zi, zf: float32 columns of z, one per
// head. One block per (entry, head): the transcendental parts are done by all threads for a chunk of tokens at a time, the chain
// of maxima by one thread in the order of the sequence (an add and a max a token), so a token's gates do not depend on
// how the sequence was cut into steps.
// (SG_TOK tokens at a time: 512 where the entries bring long portions - the loads' and the exponentials' latency is paid once a
// chunk -, 128 where they bring few tokens.)
__device__ __forceinline__ float sm_logsigmoid(float x) { return x >= 0.f ? -log1pf(expf(-x)) : x - log1pf(expf(x)); }
template <int SG_TOK>
__global__ void __launch_bounds__(SG_TOK) stabilized_gates_kernel(const float* z, int ldz, int i_off, int f_off, float cap, float* mstate,
                                                                  int slot_stride, const int* __restrict__ read_slots,
                                                                  const int* __restrict__ write_slots, const int* __restrict__ qstart,
                                                                  float* __restrict__ decay, float* __restrict__ inw,
                                                                  float* __restrict__ floor_, int H, int e0) {
    __shared__ __align__(16) float si[SG_TOK], sf[SG_TOK], sm_[SG_TOK];    // sm_[i]: the maximum after token i of the chunk
    __shared__ float m_start;                     // the maximum before the chunk's first token
    const int e = e0 + blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int q0 = qstart[e], n = qstart[e + 1] - q0;
    if (n <= 0) return;
    if (tid == 0) m_start = mstate[(size_t)read_slots[e] * slot_stride + h];
    for (int t0 = 0; t0 < n; t0 += SG_TOK) {
        const int nt = min(SG_TOK, n - t0);
        float il = 0.f, fl = 0.f;
        if (tid < nt) {
            const size_t row = (size_t)(q0 + t0 + tid);
            const float zi = z[row * ldz + i_off + h], zf = z[row * ldz + f_off + h];
            il = cap > 0.f ? cap * tanhf(zi / cap) : zi;
            fl = sm_logsigmoid(cap > 0.f ? cap * tanhf(zf / cap) : zf);
            si[tid] = il, sf[tid] = fl;
        }
        __syncthreads();
        if (tid == 0) {                           // four tokens a turn, 16 bytes a load and a store: the chain itself is an add and a max a token
            float m = m_start;
            int i = 0;
            for (; i + 4 <= nt; i += 4) {
                const float4 f4 = *reinterpret_cast<const float4*>(sf + i), i4 = *reinterpret_cast<const float4*>(si + i);
                float4 o;
                o.x = fmaxf(f4.x + m, i4.x), o.y = fmaxf(f4.y + o.x, i4.y), o.z = fmaxf(f4.z + o.y, i4.z), o.w = fmaxf(f4.w + o.z, i4.w);
                *reinterpret_cast<float4*>(sm_ + i) = o;
                m = o.w;
            }
            for (; i < nt; ++i) {
                m = fmaxf(sf[i] + m, si[i]);
                sm_[i] = m;
            }
        }
        __syncthreads();
        if (tid < nt) {
            const size_t o = (size_t)(q0 + t0 + tid) * H + h;
            const float mp = tid == 0 ? m_start : sm_[tid - 1], m = sm_[tid];
            decay[o] = expf(fl + mp - m);
            inw[o] = expf(il - m);
            floor_[o] = expf(-m);
        }
        __syncthreads();
        if (tid == 0) m_start = sm_[nt - 1];
    }
    __syncthreads();
    if (tid == 0) mstate[(size_t)write_slots[e] * slot_stride + h] = m_start;
}

IL_EXPORT int il_stabilized_gates(const float* z, int ldz, int i_off, int f_off, float cap, float* mstate, int slot_stride, const int* read_slots,
                                  const int* write_slots, const int* qstart, float* decay, float* inw, float* floor_, int H, int E, int e0,
                                  int T, cudaStream_t stream) {
    if (E <= 0) return IL_OK;
    if (H <= 0 || e0 < 0 || slot_stride < H) return IL_BAD_ARG;
    if (T >= 256 * E)                             // (T: the rows of the step; only their average per entry is used)
        stabilized_gates_kernel<512><<<dim3(E, H), 512, 0, stream>>>(z, ldz, i_off, f_off, cap, mstate, slot_stride, read_slots, write_slots,
                                                                     qstart, decay, inw, floor_, H, e0);
    else
        stabilized_gates_kernel<128><<<dim3(E, H), 128, 0, stream>>>(z, ldz, i_off, f_off, cap, mstate, slot_stride, read_slots, write_slots,
                                                                     qstart, decay, inw, floor_, H, e0);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- one gate per head --------------------------------------------------------------------------------------------------
// out[t, h * vdim + c] = y[t, h * hd + c] * sigmoid(gate[t, g_off + h]) for c < vdim <= hd (heads that were padded to hd
// columns come out packed). Without a gate only the packing is done.
template <typename TA>
__global__ void head_gate_kernel(const TA* __restrict__ y, int ldy, int hd, const TA* __restrict__ gate, int ldg, int g_off,
                                 TA* __restrict__ out, int ldo, int nh, int vdim, int T) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;      // output column; blockIdx.y walks the tokens
    if (j >= nh * vdim) return;
    const int h = j / vdim, c = j - h * vdim;
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        const float s = gate ? sm_sigmoid(il_to_f(gate[(size_t)t * ldg + g_off + h])) : 1.f;
        out[(size_t)t * ldo + j] = il_from_f<TA>(il_to_f(y[(size_t)t * ldy + h * hd + c]) * s);
    }
}

IL_EXPORT int il_head_gate(const void* y, int kind, int ldy, int hd, const void* gate, int ldg, int g_off, void* out, int ldo, int nh,
                           int vdim, int T, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (nh <= 0 || vdim <= 0 || vdim > hd) return IL_BAD_ARG;
    const dim3 grid((nh * vdim + 255) / 256, T < 32768 ? T : 32768);
    if (kind == IL_F32)
        head_gate_kernel<float><<<grid, 256, 0, stream>>>((const float*)y, ldy, hd, (const float*)gate, ldg, g_off, (float*)out, ldo, nh, vdim, T);
    else if (kind == IL_BF16)
        head_gate_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)y, ldy, hd, (const __nv_bfloat16*)gate, ldg, g_off,
                                                                  (__nv_bfloat16*)out, ldo, nh, vdim, T);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- a weighted sum of two branches: out = sa * a + sb * b, summed in float32 ------------------------------------------------
template <typename TA>
__global__ void scaled_sum_kernel(const TA* __restrict__ a, float sa, const TA* __restrict__ b, float sb, TA* __restrict__ out, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
        out[idx] = il_from_f<TA>(fmaf(sa, il_to_f(a[idx]), sb * il_to_f(b[idx])));
}

IL_EXPORT int il_scaled_sum(const void* a, float sa, const void* b, float sb, void* out, int kind, long long total, cudaStream_t stream) {
    if (total <= 0) return IL_OK;
    const int grid = sm_grid((size_t)total, 256);
    if (kind == IL_F32)
        scaled_sum_kernel<float><<<grid, 256, 0, stream>>>((const float*)a, sa, (const float*)b, sb, (float*)out, (size_t)total);
    else if (kind == IL_BF16)
        scaled_sum_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)a, sa, (const __nv_bfloat16*)b, sb, (__nv_bfloat16*)out, (size_t)total);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- soft cap: y = cap * tanh(y / cap), float32 in place ------------------------------------------------------------------
__global__ void softcap_kernel(float* y, float cap, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
        y[idx] = cap * tanhf(y[idx] / cap);
}

IL_EXPORT int il_softcap(float* y, float cap, long long total, cudaStream_t stream) {
    if (total <= 0) return IL_OK;
    if (!(cap > 0.f)) return IL_BAD_ARG;
    softcap_kernel<<<sm_grid((size_t)total, 256), 256, 0, stream>>>(y, cap, (size_t)total);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- a token's input blended with its predecessor's ------------------------------------------------------------------------
// out[t, m * W + c] = h[t, c] + (h[t - 1, c] - h[t, c]) * mu[m, c] for m < n_mix: every projection of a mixer reads its own blend
// of the token's row and the row before it in the sequence. The row before a step's first token comes from the request's
// state (float32 [W]; the zero slot for a sequence's first token), which then receives the entry's last row. Only the thread
// of an entry's first token touches the state of its column - it reads before it writes - so an entry may read and write one
// slot. Blends are computed in f32 and written in the rows' dtype. One thread per (token, column).
template <typename TA>
__global__ void token_shift_mix_kernel(const TA* __restrict__ h, int ldh, const float* __restrict__ mu, int n_mix, float* state,
                                       size_t slot_stride, const int* __restrict__ read_slots, const int* __restrict__ write_slots,
                                       const int* __restrict__ tok_entry, const int* __restrict__ qstart, TA* __restrict__ out, int ldo,
                                       int W, int T) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        const int e = tok_entry[t];
        const int first = qstart[e];
        const float cur = il_to_f(h[(size_t)t * ldh + c]);
        float prev;
        if (t == first) {
            prev = state[(size_t)read_slots[e] * slot_stride + c];
            if (write_slots) state[(size_t)write_slots[e] * slot_stride + c] = il_to_f(h[(size_t)(qstart[e + 1] - 1) * ldh + c]);
        } else {
            prev = il_to_f(h[(size_t)(t - 1) * ldh + c]);
        }
        const float d = prev - cur;
        for (int m = 0; m < n_mix; ++m) out[(size_t)t * ldo + (size_t)m * W + c] = il_from_f<TA>(fmaf(d, mu[(size_t)m * W + c], cur));
    }
}

// Four neighbouring columns a thread (W a multiple of 4, rows on 16-byte borders): 8- or 16-byte loads and stores.
__device__ __forceinline__ float4 ts_ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ts_ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void ts_st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void ts_st4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&a);
    u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}
template <typename TA>
__global__ void token_shift_mix4_kernel(const TA* __restrict__ h, int ldh, const float* __restrict__ mu, int n_mix, float* state,
                                        size_t slot_stride, const int* __restrict__ read_slots, const int* __restrict__ write_slots,
                                        const int* __restrict__ tok_entry, const int* __restrict__ qstart, TA* __restrict__ out, int ldo,
                                        int W, int T) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= W) return;
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        const int e = tok_entry[t];
        const int first = qstart[e];
        const float4 cur = ts_ld4(h + (size_t)t * ldh + c);
        float4 prev;
        if (t == first) {
            prev = ts_ld4(state + (size_t)read_slots[e] * slot_stride + c);
            if (write_slots) ts_st4(state + (size_t)write_slots[e] * slot_stride + c, ts_ld4(h + (size_t)(qstart[e + 1] - 1) * ldh + c));
        } else {
            prev = ts_ld4(h + (size_t)(t - 1) * ldh + c);
        }
        const float4 d = make_float4(prev.x - cur.x, prev.y - cur.y, prev.z - cur.z, prev.w - cur.w);
        for (int m = 0; m < n_mix; ++m) {
            const float4 u = ts_ld4(mu + (size_t)m * W + c);
            ts_st4(out + (size_t)t * ldo + (size_t)m * W + c, make_float4(fmaf(d.x, u.x, cur.x), fmaf(d.y, u.y, cur.y), fmaf(d.z, u.z, cur.z), fmaf(d.w, u.w, cur.w)));
        }
    }
}

IL_EXPORT int il_token_shift_mix(const void* h, int kind, int ldh, const float* mu, int n_mix, float* state, long long slot_stride,
                                 const int* read_slots, const int* write_slots, const int* tok_entry, const int* qstart, void* out, int ldo,
                                 int W, int T, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (W <= 0 || n_mix <= 0 || ldo < n_mix * W || slot_stride < W) return IL_BAD_ARG;
    if (kind != IL_F32 && kind != IL_BF16) return IL_BAD_ARG;
    if (((W | ldh | ldo | (int)(slot_stride & 3)) & 3) == 0 && (((uintptr_t)h | (uintptr_t)mu | (uintptr_t)state | (uintptr_t)out) & 15) == 0) {
        const int threads = W >= 512 ? 128 : 64;
        const dim3 grid4((W / 4 + threads - 1) / threads, T < 32768 ? T : 32768);
        if (kind == IL_F32)
            token_shift_mix4_kernel<float><<<grid4, threads, 0, stream>>>((const float*)h, ldh, mu, n_mix, state, (size_t)slot_stride, read_slots,
                                                                          write_slots, tok_entry, qstart, (float*)out, ldo, W, T);
        else
            token_shift_mix4_kernel<__nv_bfloat16><<<grid4, threads, 0, stream>>>((const __nv_bfloat16*)h, ldh, mu, n_mix, state, (size_t)slot_stride,
                                                                                  read_slots, write_slots, tok_entry, qstart, (__nv_bfloat16*)out, ldo, W, T);
        IL_LAUNCH_CHECK();
        return IL_OK;
    }
    const dim3 grid((W + 127) / 128, T < 32768 ? T : 32768);
    if (kind == IL_F32)
        token_shift_mix_kernel<float><<<grid, 128, 0, stream>>>((const float*)h, ldh, mu, n_mix, state, (size_t)slot_stride, read_slots, write_slots,
                                                                tok_entry, qstart, (float*)out, ldo, W, T);
    else
        token_shift_mix_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)h, ldh, mu, n_mix, state, (size_t)slot_stride, read_slots,
                                                                        write_slots, tok_entry, qstart, (__nv_bfloat16*)out, ldo, W, T);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- a decay from its pre-activation: w = exp(-exp(z + w0)), float32 in place (z [T, ld], the first `cols` columns; w0 [cols]) ----
__global__ void double_exp_decay_kernel(float* z, int ld, const float* __restrict__ w0, int cols, int T) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const float b = w0 ? w0[c] : 0.f;
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        float* p = z + (size_t)t * ld + c;
        *p = expf(-expf(*p + b));
    }
}

IL_EXPORT int il_double_exp_decay(float* z, int ld, const float* w0, int cols, int T, cudaStream_t stream) {
    if (T <= 0 || cols <= 0) return IL_OK;
    double_exp_decay_kernel<<<dim3((cols + 255) / 256, T < 32768 ? T : 32768), 256, 0, stream>>>(z, ld, w0, cols, T);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- out = tanh(x), float32 rows in, rows of the compute dtype out (the inner activation of a low-rank projection) ----------
template <typename TO>
__global__ void tanh_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
        out[idx] = il_from_f<TO>(tanhf(x[idx]));
}

IL_EXPORT int il_tanh_rows(const float* x, void* out, int out_kind, long long total, cudaStream_t stream) {
    if (total <= 0) return IL_OK;
    const int grid = sm_grid((size_t)total, 256);
    if (out_kind == IL_F32) tanh_rows_kernel<float><<<grid, 256, 0, stream>>>(x, (float*)out, (size_t)total);
    else if (out_kind == IL_BF16) tanh_rows_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(x, (__nv_bfloat16*)out, (size_t)total);
    else return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
