// What stands between an attention mixer's projection and its attention when queries and keys are normed per head and
// positions do not rotate anything: per token and head
//   q_h <- q_h / sqrt(mean(q_h^2) + eps) * w_q * temp(pos)        temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)  (or 1)
//   k_g <- k_g / sqrt(mean(k_g^2) + eps) * w_k                     -> the token's slot of the cache, K plane
//   v_g                                                            -> the V plane: the value columns, or the key columns as
//                                                                     projected, before the norm (a mixer whose values are its keys)
// all in f32; w_q and w_k are one vector each, shared by the heads. Heads are laid out at hd >= key size, value size: the
// surplus columns are written as zeros (a zero column adds nothing to a score). A mixer that reads another layer's cache
// gives no key columns (k_off < 0): only its queries are normed.
// Cache layout of one layer: [page][0=K,1=V][kv head][slot in page][hd]. One warp per (token, head).
#include "common.cuh"

// four neighbouring values at a time (16 bytes of f32, 8 of bfloat16)
__device__ __forceinline__ float4 qn_ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 qn_ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void qn_st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void qn_st4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&a);
    u.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ float4 qn_w4(const void* w, int kind, int d) {
    return make_float4(il_load_any(w, kind, d), il_load_any(w, kind, d + 1), il_load_any(w, kind, d + 2), il_load_any(w, kind, d + 3));
}

// The form for sizes and offsets that are multiples of 4 (rows, segments and heads then start on 8- or 16-byte borders): the
// lanes hold 4 neighbouring columns instead of every 32nd (the sum of squares is gathered in another order). VEC 1 is the form for
// every size.
template <typename TA, int VEC>
__global__ void qk_norm_store_kernel(const TA* proj, int ld, int q_off, int k_off, int v_off, int nh, int nkv, int dk, int dv, int hd,
                                     const void* __restrict__ wq, const void* __restrict__ wk, int w_kind, float eps, float t_coef,
                                     int t_every, TA* __restrict__ q_out, const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_entry, const int* __restrict__ block_table, int bt_stride,
                                     TA* __restrict__ cache, int page_size, int T) {
    const int jobs = nh + (k_off >= 0 ? 2 * nkv : 0);
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)T * jobs) return;
    const int t = (int)(wid / jobs), j = (int)(wid - (long long)t * jobs);
    const int pos = tok_pos[t];
    il_pdl_wait();
    const TA* row = proj + (size_t)t * ld;
    if (j < nh) {                                 // a query head
        const TA* x = row + q_off + (size_t)j * dk;
        TA* o = q_out + ((size_t)t * nh + j) * hd;
        float ss = 0.f;
        if (VEC == 4) {
            for (int d = 4 * lane; d < dk; d += 128) {
                const float4 a = qn_ld4(x + d);
                ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            }
        } else {
            for (int d = lane; d < dk; d += 32) {
                const float a = il_to_f(x[d]);
                ss += a * a;
            }
        }
        ss = il_warp_sum(ss);
        float r = 1.f / sqrtf(ss / (float)dk + eps);
        if (t_every > 0) r *= 1.f + t_coef * logf((float)((pos + 1) / t_every) + 1.f);
        if (VEC == 4) {
            for (int d = 4 * lane; d < hd; d += 128) {
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                if (d < dk) {
                    const float4 w = qn_w4(wq, w_kind, d);
                    a = qn_ld4(x + d);
                    a.x *= r * w.x, a.y *= r * w.y, a.z *= r * w.z, a.w *= r * w.w;
                }
                qn_st4(o + d, a);
            }
        } else {
            for (int d = lane; d < hd; d += 32) o[d] = il_from_f<TA>(d < dk ? il_to_f(x[d]) * r * il_load_any(wq, w_kind, d) : 0.f);
        }
        return;
    }
    if (!cache) return;
    const int page = block_table[(size_t)tok_entry[t] * bt_stride + pos / page_size];
    if (page < 0) return;                         // the host reserves every page a step touches; never write elsewhere
    const bool is_k = j < nh + nkv;
    const int g = is_k ? j - nh : j - nh - nkv;
    TA* dst = cache + (((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + g) * (size_t)page_size * hd + (size_t)(pos % page_size) * hd;
    if (is_k) {
        const TA* x = row + k_off + (size_t)g * dk;
        float ss = 0.f;
        if (VEC == 4) {
            for (int d = 4 * lane; d < dk; d += 128) {
                const float4 a = qn_ld4(x + d);
                ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            }
        } else {
            for (int d = lane; d < dk; d += 32) {
                const float a = il_to_f(x[d]);
                ss += a * a;
            }
        }
        ss = il_warp_sum(ss);
        const float r = 1.f / sqrtf(ss / (float)dk + eps);
        if (VEC == 4) {
            for (int d = 4 * lane; d < hd; d += 128) {
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                if (d < dk) {
                    const float4 w = qn_w4(wk, w_kind, d);
                    a = qn_ld4(x + d);
                    a.x *= r * w.x, a.y *= r * w.y, a.z *= r * w.z, a.w *= r * w.w;
                }
                qn_st4(dst + d, a);
            }
        } else {
            for (int d = lane; d < hd; d += 32) dst[d] = il_from_f<TA>(d < dk ? il_to_f(x[d]) * r * il_load_any(wk, w_kind, d) : 0.f);
        }
    } else {
        const TA* x = row + v_off + (size_t)g * dv;
        if (VEC == 4) {
            for (int d = 4 * lane; d < hd; d += 128) qn_st4(dst + d, d < dv ? qn_ld4(x + d) : make_float4(0.f, 0.f, 0.f, 0.f));
        } else {
            for (int d = lane; d < hd; d += 32) dst[d] = d < dv ? x[d] : il_from_f<TA>(0.f);
        }
    }
}

IL_EXPORT int il_qk_norm_store(const void* proj, int act_kind, int ld, int q_off, int k_off, int v_off, int nh, int nkv, int dk, int dv, int hd,
                               const void* wq, const void* wk, int w_kind, float eps, float t_coef, int t_every, void* q_out,
                               const int* tok_pos, const int* tok_entry, const int* block_table, int bt_stride, void* cache, int page_size,
                               int T, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (nh <= 0 || nkv <= 0 || dk <= 0 || dv <= 0 || hd < dk || hd < dv || page_size <= 0 || !wq || (k_off >= 0 && !wk)) return IL_BAD_ARG;
    const long long warps = (long long)T * (nh + (k_off >= 0 ? 2 * nkv : 0));
    const long long blocks = (warps + 3) / 4;
    if (blocks > 0x7fffffffLL) return IL_UNSUPPORTED;
    if (act_kind != IL_F32 && act_kind != IL_BF16) return IL_BAD_ARG;
    const bool vec = ((ld | q_off | v_off | dk | dv | hd) & 3) == 0 && (k_off < 0 || (k_off & 3) == 0) &&
                     (((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)cache) & 15) == 0;
#define QN_GO(TA, VEC)                                                                                                                  \
    IL_LAUNCH((qk_norm_store_kernel<TA, VEC>), (int)blocks, 128, 0, stream, (const TA*)proj, ld, q_off, k_off, v_off, nh, nkv, dk, dv, hd, wq, wk, \
              w_kind, eps, t_coef, t_every, (TA*)q_out, tok_pos, tok_entry, block_table, bt_stride, (TA*)cache, page_size, T)
    if (act_kind == IL_F32) {
        if (vec) QN_GO(float, 4); else QN_GO(float, 1);
    } else {
        if (vec) QN_GO(__nv_bfloat16, 4); else QN_GO(__nv_bfloat16, 1);
    }
#undef QN_GO
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// out[t, h * dv + c] = y[t, h * hd + c] * sigmoid(gate[t, g_off + h * dv + c]) for c < dv <= hd: a gate per output column,
// and heads that were laid out at hd columns come out packed. Without a gate only the packing is done.
template <typename TA>
__global__ void gate_pack_kernel(const TA* y, int hd, const TA* gate, int ldg, int g_off, TA* __restrict__ out, int nh, int dv, int T) {
    il_pdl_wait();
    const int n = nh * dv;
    const long long total = (long long)T * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / n;
        const int jc = (int)(i - t * n), h = jc / dv, c = jc - h * dv;
        float v = il_to_f(y[((size_t)t * nh + h) * hd + c]);
        if (gate) v = v / (1.f + expf(-il_to_f(gate[(size_t)t * ldg + g_off + jc])));
        out[i] = il_from_f<TA>(v);
    }
}

template <typename TA>
__global__ void gate_pack4_kernel(const TA* y, int hd, const TA* gate, int ldg, int g_off, TA* __restrict__ out, int nh, int dv, int T) {
    il_pdl_wait();
    const int n4 = (nh * dv) >> 2;
    const long long total = (long long)T * n4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / n4;
        const int jc = (int)(i - t * n4) << 2, h = jc / dv, c = jc - h * dv;
        float4 v = qn_ld4(y + ((size_t)t * nh + h) * hd + c);
        if (gate) {
            const float4 z = qn_ld4(gate + (size_t)t * ldg + g_off + jc);
            v.x = v.x / (1.f + expf(-z.x)), v.y = v.y / (1.f + expf(-z.y)), v.z = v.z / (1.f + expf(-z.z)), v.w = v.w / (1.f + expf(-z.w));
        }
        qn_st4(out + (size_t)t * nh * dv + jc, v);
    }
}

IL_EXPORT int il_gate_pack(const void* y, int act_kind, int hd, const void* gate, int ldg, int g_off, void* out, int nh, int dv, int T,
                           cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (nh <= 0 || dv <= 0 || dv > hd) return IL_BAD_ARG;
    if (act_kind != IL_F32 && act_kind != IL_BF16) return IL_BAD_ARG;
    if (((hd | dv | ldg | g_off) & 3) == 0 && (((uintptr_t)y | (uintptr_t)gate | (uintptr_t)out) & 15) == 0) {
        const long long g4 = ((long long)T * nh * dv / 4 + 255) / 256;
        const int blocks4 = (int)(g4 > 148 * 16 ? 148 * 16 : g4);
        if (act_kind == IL_F32)
            IL_LAUNCH(gate_pack4_kernel<float>, blocks4, 256, 0, stream, (const float*)y, hd, (const float*)gate, ldg, g_off, (float*)out, nh, dv, T);
        else
            IL_LAUNCH(gate_pack4_kernel<__nv_bfloat16>, blocks4, 256, 0, stream, (const __nv_bfloat16*)y, hd, (const __nv_bfloat16*)gate, ldg,
                      g_off, (__nv_bfloat16*)out, nh, dv, T);
        IL_LAUNCH_CHECK();
        return IL_OK;
    }
    const long long g = ((long long)T * nh * dv + 255) / 256;
    const int blocks = (int)(g > 148 * 16 ? 148 * 16 : g);
    if (act_kind == IL_F32)
        IL_LAUNCH(gate_pack_kernel<float>, blocks, 256, 0, stream, (const float*)y, hd, (const float*)gate, ldg, g_off, (float*)out, nh, dv, T);
    else if (act_kind == IL_BF16)
        IL_LAUNCH(gate_pack_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)y, hd, (const __nv_bfloat16*)gate, ldg, g_off,
                  (__nv_bfloat16*)out, nh, dv, T);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- queries and keys normed over the whole projection, then rotated ---------------------------------------------------
// Per token: the nh * dk query columns are divided by THEIR root mean square, all heads together, and multiplied by a
// weight of that many entries; the nkv * dk key columns likewise. Then, of every head, the first `rot` dimensions turn by
// angle = pos * inv_freq[i], dimension i paired with i + rot / 2 ((u, v) -> (u cos - v sin, v cos + u sin)); the others
// pass. Queries go to q_out [T, nh * hd], keys to the K plane of the token's cache slot, values to the V plane, heads laid
// out at hd columns with the surplus zero. k_off < 0: no keys or values (the mixer reads another layer's cache).
// Sums of squares, angles and the rotation are f32. One block per token.
#define QR_MAX_ROT 1024
template <typename TA>
__global__ void qk_rows_norm_rope_store_kernel(const TA* proj, int ld, int q_off, int k_off, int v_off, int nh, int nkv, int dk, int dv, int hd,
                                               const void* __restrict__ wq, const void* __restrict__ wk, int w_kind, float eps, int rot,
                                               const float* __restrict__ inv_freq, TA* __restrict__ q_out,
                                               const int* __restrict__ tok_pos, const int* __restrict__ tok_entry,
                                               const int* __restrict__ block_table, int bt_stride, TA* __restrict__ cache, int page_size) {
    __shared__ float red[32];
    __shared__ float s_cos[QR_MAX_ROT / 2], s_sin[QR_MAX_ROT / 2];      // the token's angles, once for all its heads
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const bool has_k = k_off >= 0;
    int page = -1;
    if (has_k && cache) page = block_table[(size_t)tok_entry[t] * bt_stride + pos / page_size];
    for (int i = threadIdx.x; i < (rot >> 1); i += blockDim.x) sincosf((float)pos * inv_freq[i], &s_sin[i], &s_cos[i]);
    il_pdl_wait();
    const TA* row = proj + (size_t)t * ld;
    const int nq = nh * dk, nk = nkv * dk, half = rot >> 1;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
        const float x = il_to_f(row[q_off + i]);
        sq += x * x;
    }
    if (has_k)
        for (int i = threadIdx.x; i < nk; i += blockDim.x) {
            const float x = il_to_f(row[k_off + i]);
            sk += x * x;
        }
    sq = il_block_sum(sq, red);
    sk = il_block_sum(sk, red);
    const float rq = 1.f / sqrtf(sq / (float)nq + eps), rk = has_k ? 1.f / sqrtf(sk / (float)nk + eps) : 0.f;
    // element d of head j of a normed and weighted projection, rotated
    auto turned = [&](const TA* x, const void* w, float r, int j, int d) -> float {
        const int c = j * dk + d;
        const float a = il_to_f(x[c]) * r * il_load_any(w, w_kind, c);
        if (d >= rot) return a;
        const bool low = d < half;
        const int c2 = low ? c + half : c - half;
        const float b = il_to_f(x[c2]) * r * il_load_any(w, w_kind, c2);
        const float s = s_sin[low ? d : d - half], co = s_cos[low ? d : d - half];
        return low ? a * co - b * s : a * co + b * s;
    };
    for (int idx = threadIdx.x; idx < nh * hd; idx += blockDim.x) {
        const int j = idx / hd, d = idx - j * hd;
        q_out[(size_t)t * nh * hd + idx] = il_from_f<TA>(d < dk ? turned(row + q_off, wq, rq, j, d) : 0.f);
    }
    if (page < 0) return;                         // no keys of its own, or no slot (the host reserves every page a step touches)
    const size_t plane = (size_t)nkv * page_size * hd;
    TA* kdst = cache + (size_t)page * 2 * plane + (size_t)(pos % page_size) * hd;
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
        const int g = idx / hd, d = idx - g * hd;
        const size_t at = (size_t)g * page_size * hd + d;
        kdst[at] = il_from_f<TA>(d < dk ? turned(row + k_off, wk, rk, g, d) : 0.f);
        kdst[plane + at] = d < dv ? row[v_off + g * dv + d] : il_from_f<TA>(0.f);
    }
}

IL_EXPORT int il_qk_rows_norm_rope_store(const void* proj, int act_kind, int ld, int q_off, int k_off, int v_off, int nh, int nkv, int dk, int dv,
                                         int hd, const void* wq, const void* wk, int w_kind, float eps, int rot, const float* inv_freq,
                                         void* q_out, const int* tok_pos, const int* tok_entry, const int* block_table, int bt_stride,
                                         void* cache, int page_size, int T, cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (nh <= 0 || nkv <= 0 || dk <= 0 || dv <= 0 || hd < dk || hd < dv || page_size <= 0 || !wq || (k_off >= 0 && !wk)) return IL_BAD_ARG;
    if (rot < 0 || (rot & 1) || rot > dk || (rot > 0 && !inv_freq)) return IL_BAD_ARG;
    if (rot > QR_MAX_ROT) return IL_UNSUPPORTED;
    const int work = nh * hd;
    const int threads = work >= 2048 ? 512 : work >= 512 ? 256 : 128;
    if (act_kind == IL_F32)
        IL_LAUNCH(qk_rows_norm_rope_store_kernel<float>, T, threads, 0, stream, (const float*)proj, ld, q_off, k_off, v_off, nh, nkv, dk, dv, hd, wq,
                  wk, w_kind, eps, rot, inv_freq, (float*)q_out, tok_pos, tok_entry, block_table, bt_stride, (float*)cache, page_size);
    else if (act_kind == IL_BF16)
        IL_LAUNCH(qk_rows_norm_rope_store_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)proj, ld, q_off, k_off, v_off, nh, nkv,
                  dk, dv, hd, wq, wk, w_kind, eps, rot, inv_freq, (__nv_bfloat16*)q_out, tok_pos, tok_entry, block_table, bt_stride,
                  (__nv_bfloat16*)cache, page_size);
    else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}
