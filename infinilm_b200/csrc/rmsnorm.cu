// Residual add fused with RMSNorm.
//   x = resid[r] + branch_scale * branch[r] + vec   (branch may be absent; vec too: f32, one vector added to every row, or -
//                                                    vec_stride = H - a row of its own for every row of resid)
//   resid[r] = x                              (kept in f32; skipped when a row list is given)
//   out[i]  = x / sqrt(mean(x^2) + eps) * w
// Sum of squares, rsqrt and the scaling are f32; one block per row with a fixed thread count,
// so a row's result does not depend on what else is in the batch.
#include "common.cuh"

template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TA* __restrict__ branch, float bscale,
                                   const void* __restrict__ w, int w_kind, float eps, TA* __restrict__ out,
                                   const int* __restrict__ rows, int H, const float* __restrict__ vec, int vec_stride) {
    extern __shared__ float xs[];
    __shared__ float red[32];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* rr = resid + (size_t)r * H;
    const TA* br = branch ? branch + (size_t)r * H : nullptr;
    if (vec) vec += (size_t)r * vec_stride;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float x = rr[h];
        if (br) x += bscale * il_to_f(br[h]);
        if (vec) x += vec[h];
        xs[h] = x;
        ss += x * x;
        if (!rows && (br || vec)) rr[h] = x;
    }
    ss = il_block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)i * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x)
        o[h] = il_from_f<TA>(xs[h] * rstd * il_load_any(w, w_kind, h));
}

// The same with 4 elements per thread and access: 16-byte loads of the residual, 8- or 16-byte loads of
// the branch and the weight, all of a thread's loads issued before the first use.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename TA, int MAXV>
__global__ void __launch_bounds__(256) add_rmsnorm_vec_kernel(float* resid, const TA* branch, float bscale,
                                                              const void* __restrict__ w, int w_kind, float eps, TA* __restrict__ out,
                                                              const int* __restrict__ rows, int H, const float* __restrict__ vec, int vec_stride) {
    __shared__ float red[32];
    const int i = blockIdx.x;
    const int nv = H >> 2;                        // float4 groups in a row
    // the norm's weights and the row index do not come from the kernel before this one: read while it still runs
    float4 wv[MAXV];
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int v = threadIdx.x + k * 256;
        wv[k] = v < nv ? (w_kind == IL_F32 ? ld4((const float*)w + 4 * v) : ld4((const __nv_bfloat16*)w + 4 * v)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int r = rows ? rows[i] : i;
    il_pdl_wait();
    float* rr = resid + (size_t)r * H;
    const TA* br = branch ? branch + (size_t)r * H : nullptr;
    float4 x[MAXV];
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int v = threadIdx.x + k * 256;
        x[k] = v < nv ? ld4(rr + 4 * v) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (br) {
        float4 b[MAXV];
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int v = threadIdx.x + k * 256;
            b[k] = v < nv ? ld4(br + 4 * v) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            x[k].x += bscale * b[k].x;
            x[k].y += bscale * b[k].y;
            x[k].z += bscale * b[k].z;
            x[k].w += bscale * b[k].w;
        }
    }
    if (vec) {
        vec += (size_t)r * vec_stride;
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int v = threadIdx.x + k * 256;
            const float4 a = v < nv ? ld4(vec + 4 * v) : make_float4(0.f, 0.f, 0.f, 0.f);
            x[k].x += a.x, x[k].y += a.y, x[k].z += a.z, x[k].w += a.w;
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) ss += x[k].x * x[k].x + x[k].y * x[k].y + x[k].z * x[k].z + x[k].w * x[k].w;
    if (!rows && (br || vec)) {
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int v = threadIdx.x + k * 256;
            if (v < nv) st4(rr + 4 * v, x[k]);
        }
    }
    ss = il_block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)i * H;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int v = threadIdx.x + k * 256;
        if (v < nv) st4(o + 4 * v, make_float4(x[k].x * rstd * wv[k].x, x[k].y * rstd * wv[k].y, x[k].z * rstd * wv[k].z, x[k].w * rstd * wv[k].w));
    }
}

template <typename TA>
static int launch_vec(float* resid, const void* branch, float bscale, const void* w, int w_kind, float eps, void* out,
                      const int* rows, int n_rows, int H, const float* vec, int vec_stride, cudaStream_t stream) {
    const int nv = H >> 2;
    if (nv <= 256 * 2)
        IL_LAUNCH((add_rmsnorm_vec_kernel<TA, 2>), n_rows, 256, 0, stream, resid, (const TA*)branch, bscale, w, w_kind, eps, (TA*)out, rows, H, vec, vec_stride);
    else if (nv <= 256 * 4)
        IL_LAUNCH((add_rmsnorm_vec_kernel<TA, 4>), n_rows, 256, 0, stream, resid, (const TA*)branch, bscale, w, w_kind, eps, (TA*)out, rows, H, vec, vec_stride);
    else
        IL_LAUNCH((add_rmsnorm_vec_kernel<TA, 8>), n_rows, 256, 0, stream, resid, (const TA*)branch, bscale, w, w_kind, eps, (TA*)out, rows, H, vec, vec_stride);
    return 0;
}

IL_EXPORT int il_add_rmsnorm(float* resid, const void* branch, float bscale, const void* w, int w_kind,
                             float eps, void* out, int act_kind, const int* rows, int n_rows, int H,
                             const float* vec, int vec_stride, cudaStream_t stream) {
    if (n_rows <= 0) return IL_OK;
    if (H <= 0) return IL_BAD_ARG;
    if (H % 4 == 0 && H <= 256 * 8 * 4 && (act_kind == IL_F32 || act_kind == IL_BF16)) {
        if (act_kind == IL_F32) launch_vec<float>(resid, branch, bscale, w, w_kind, eps, out, rows, n_rows, H, vec, vec_stride, stream);
        else launch_vec<__nv_bfloat16>(resid, branch, bscale, w, w_kind, eps, out, rows, n_rows, H, vec, vec_stride, stream);
        IL_LAUNCH_CHECK();
        return IL_OK;
    }
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return IL_UNSUPPORTED;
    const int threads = 256;
    if (act_kind == IL_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_rmsnorm_kernel<float><<<n_rows, threads, smem, stream>>>(resid, (const float*)branch, bscale, w, w_kind, eps, (float*)out, rows, H, vec, vec_stride);
    } else if (act_kind == IL_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, smem, stream>>>(resid, (const __nv_bfloat16*)branch, bscale, w, w_kind, eps, (__nv_bfloat16*)out, rows, H, vec, vec_stride);
    } else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- the norm on the branch, then the residual add -------------------------------------------------------------------
//   resid[r] += scale * branch[r] / sqrt(mean(branch[r]^2) + eps) * w        (f32)
//   copy[r]   = resid[r] in the activations' type (optional: what the next sublayer reads)
// The block layout of a model whose sublayers read the residual stream itself and whose norms sit on the sublayers'
// outputs. One block per row with a fixed thread count; the branch row waits in shared memory as f32 between the two passes.
template <typename TA>
__global__ void __launch_bounds__(256) norm_add_kernel(float* resid, const TA* branch, float scale, const void* __restrict__ w, int w_kind,
                                                       float eps, TA* copy, int H) {
    extern __shared__ float bs[];
    __shared__ float red[32];
    const int r = blockIdx.x;
    il_pdl_wait();
    const TA* br = branch + (size_t)r * H;
    float* rr = resid + (size_t)r * H;
    float ss = 0.f;
    if ((H & 3) == 0) {
        for (int v = threadIdx.x; v < (H >> 2); v += blockDim.x) {
            const float4 b = ld4(br + 4 * v);
            st4(bs + 4 * v, b);
            ss += b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
        }
    } else {
        for (int h = threadIdx.x; h < H; h += blockDim.x) {
            const float b = il_to_f(br[h]);
            bs[h] = b;
            ss += b * b;
        }
    }
    ss = il_block_sum(ss, red);
    const float k = scale * (1.f / sqrtf(ss / (float)H + eps));
    if ((H & 3) == 0) {
        for (int v = threadIdx.x; v < (H >> 2); v += blockDim.x) {
            const float4 b = ld4(bs + 4 * v);
            const float4 wv = w_kind == IL_F32 ? ld4((const float*)w + 4 * v) : ld4((const __nv_bfloat16*)w + 4 * v);
            float4 x = ld4(rr + 4 * v);
            x.x = fmaf(k * b.x, wv.x, x.x), x.y = fmaf(k * b.y, wv.y, x.y), x.z = fmaf(k * b.z, wv.z, x.z), x.w = fmaf(k * b.w, wv.w, x.w);
            st4(rr + 4 * v, x);
            if (copy) st4(copy + (size_t)r * H + 4 * v, x);
        }
    } else {
        for (int h = threadIdx.x; h < H; h += blockDim.x) {
            const float x = fmaf(k * bs[h], il_load_any(w, w_kind, h), rr[h]);
            rr[h] = x;
            if (copy) copy[(size_t)r * H + h] = il_from_f<TA>(x);
        }
    }
}

// rows of f32 copied into the activations' type (the first sublayer's input, where no norm_add ran before it)
template <typename TA>
__global__ void cast_rows_kernel(const float* x, TA* out, size_t total) {
    il_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) out[i] = il_from_f<TA>(x[i]);
}

IL_EXPORT int il_norm_add(float* resid, const void* branch, float scale, const void* w, int w_kind, float eps, void* copy, int act_kind,
                          int n_rows, int H, cudaStream_t stream) {
    if (n_rows <= 0) return IL_OK;
    if (H <= 0 || !branch) return IL_BAD_ARG;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return IL_UNSUPPORTED;
    if (act_kind == IL_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(norm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        IL_LAUNCH(norm_add_kernel<float>, n_rows, 256, smem, stream, resid, (const float*)branch, scale, w, w_kind, eps, (float*)copy, H);
    } else if (act_kind == IL_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(norm_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        IL_LAUNCH(norm_add_kernel<__nv_bfloat16>, n_rows, 256, smem, stream, resid, (const __nv_bfloat16*)branch, scale, w, w_kind, eps,
                  (__nv_bfloat16*)copy, H);
    } else
        return IL_BAD_ARG;
    IL_LAUNCH_CHECK();
    return IL_OK;
}

IL_EXPORT int il_cast_rows(const float* x, void* out, int out_kind, long long total, cudaStream_t stream) {
    if (total <= 0) return IL_OK;
    if (out_kind != IL_BF16) return IL_BAD_ARG;
    const long long g = (total + 255) / 256;
    IL_LAUNCH(cast_rows_kernel<__nv_bfloat16>, (int)(g > 148 * 16 ? 148 * 16 : g), 256, 0, stream, x, (__nv_bfloat16*)out, (size_t)total);
    IL_LAUNCH_CHECK();
    return IL_OK;
}

// ---- several copies of the residual stream ("hyper-connections") ---------------------------------------------------------------
// A model may keep S copies x_1 .. x_S of the residual stream (streams [T, S, H], f32). A sublayer reads u = sum_s in[s] x_s
// through a norm, and its output y goes back as x_t <- sum_s mix[s, t] x_s + out[t] y, every new copy from the old ones.
// One kernel does what lies between two sublayers, for one row a block:
//   init (or null):   x_s = init[r] for every s           (the copies start as the embedding's output)
//   y (or null):      the write-back of the sublayer before, with mix [S, S] (from, to) and out [S]
//   in_next (or null): u = sum_t in_next[t] x_t, normed = u / sqrt(mean(u^2) + eps) * w   -> normed[r] (the next sublayer's input)
//   sum_out (or null): sum_out[r] = sum_t x_t              (the stream as one row: what the model's last norm reads)
// Everything is f32 but y (read) and normed (written), which have the compute dtype. S <= HC_MAX_STREAMS.
// Dynamic shared memory: H floats (u between its two passes).
#define HC_MAX_STREAMS 16
// (MAXS: the copies a thread holds in registers, 4, 8 or 16 - the smallest that takes S)
template <typename TA, int MAXS>
__global__ void hyper_step_kernel(float* streams, const float* init, const TA* y, const float* __restrict__ mix,
                                  const float* __restrict__ out_w, const float* __restrict__ in_next, const void* __restrict__ w, int w_kind,
                                  float eps, TA* __restrict__ normed, float* __restrict__ sum_out, int S, int H) {
    extern __shared__ float us[];
    __shared__ float red[32];
    __shared__ float s_mix[HC_MAX_STREAMS * HC_MAX_STREAMS], s_out[HC_MAX_STREAMS], s_in[HC_MAX_STREAMS];
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < S * S && y; i += blockDim.x) s_mix[i] = mix[i];
    if (threadIdx.x < S) {
        if (y) s_out[threadIdx.x] = out_w[threadIdx.x];
        if (in_next) s_in[threadIdx.x] = in_next[threadIdx.x];
    }
    il_pdl_wait();
    __syncthreads();
    float* xr = streams + (size_t)r * S * H;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float x[MAXS], xn[MAXS];
#pragma unroll
        for (int s = 0; s < MAXS; ++s)
            if (s < S) x[s] = init ? init[(size_t)r * H + h] : xr[(size_t)s * H + h];
        if (y) {
            const float yv = il_to_f(y[(size_t)r * H + h]);
#pragma unroll
            for (int t = 0; t < MAXS; ++t)
                if (t < S) {
                    float a = 0.f;
#pragma unroll
                    for (int s = 0; s < MAXS; ++s)
                        if (s < S) a = fmaf(s_mix[s * S + t], x[s], a);
                    xn[t] = fmaf(s_out[t], yv, a);
                }
        } else {
#pragma unroll
            for (int t = 0; t < MAXS; ++t)
                if (t < S) xn[t] = x[t];
        }
        if (y || init) {
#pragma unroll
            for (int t = 0; t < MAXS; ++t)
                if (t < S) xr[(size_t)t * H + h] = xn[t];
        }
        if (sum_out) {
            float a = 0.f;
#pragma unroll
            for (int t = 0; t < MAXS; ++t)
                if (t < S) a += xn[t];
            sum_out[(size_t)r * H + h] = a;
        }
        if (in_next) {
            float u = 0.f;
#pragma unroll
            for (int t = 0; t < MAXS; ++t)
                if (t < S) u = fmaf(s_in[t], xn[t], u);
            us[h] = u;
            ss += u * u;
        }
    }
    if (!in_next) return;
    ss = il_block_sum(ss, red);
    const float rstd = 1.f / sqrtf(ss / (float)H + eps);
    for (int h = threadIdx.x; h < H; h += blockDim.x)
        normed[(size_t)r * H + h] = il_from_f<TA>(us[h] * rstd * il_load_any(w, w_kind, h));
}

// The same with four neighbouring columns a thread (H a multiple of 4, rows on 16-byte borders): 16-byte loads of the copies,
// all of a thread's loads issued before the first use. Every column's sums run in the scalar kernel's order.
template <typename TA, int MAXS>
__global__ void __launch_bounds__(256) hyper_step_vec_kernel(float* streams, const float* init, const TA* y, const float* __restrict__ mix,
                                                             const float* __restrict__ out_w, const float* __restrict__ in_next,
                                                             const void* __restrict__ w, int w_kind, float eps, TA* __restrict__ normed,
                                                             float* __restrict__ sum_out, int S, int H) {
    extern __shared__ __align__(16) float us[];
    __shared__ float red[32];
    __shared__ float s_mix[MAXS * MAXS], s_out[MAXS], s_in[MAXS];
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < S * S && y; i += blockDim.x) s_mix[i] = mix[i];
    if (threadIdx.x < S) {
        if (y) s_out[threadIdx.x] = out_w[threadIdx.x];
        if (in_next) s_in[threadIdx.x] = in_next[threadIdx.x];
    }
    il_pdl_wait();
    __syncthreads();
    float* xr = streams + (size_t)r * S * H;
    const int nv = H >> 2;
    float ss = 0.f;
    for (int v = threadIdx.x; v < nv; v += blockDim.x) {
        const int h = 4 * v;
        float4 x[MAXS], xn[MAXS];
        if (init) {
            const float4 e = ld4(init + (size_t)r * H + h);
#pragma unroll
            for (int s = 0; s < MAXS; ++s) x[s] = e;
        } else {
#pragma unroll
            for (int s = 0; s < MAXS; ++s)
                if (s < S) x[s] = ld4(xr + (size_t)s * H + h);
        }
        if (y) {
            const float4 yv = ld4(y + (size_t)r * H + h);
#pragma unroll
            for (int t = 0; t < MAXS; ++t)
                if (t < S) {
                    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int s = 0; s < MAXS; ++s)
                        if (s < S) {
                            const float m = s_mix[s * S + t];
                            a.x = fmaf(m, x[s].x, a.x), a.y = fmaf(m, x[s].y, a.y), a.z = fmaf(m, x[s].z, a.z), a.w = fmaf(m, x[s].w, a.w);
                        }
                    const float o = s_out[t];
                    xn[t] = make_float4(fmaf(o, yv.x, a.x), fmaf(o, yv.y, a.y), fmaf(o, yv.z, a.z), fmaf(o, yv.w, a.w));
                }
        } else {
#pragma unroll
            for (int t = 0; t < MAXS; ++t) xn[t] = x[t];
        }
        if (y || init) {
#pragma unroll
            for (int t = 0; t < MAXS; ++t)
                if (t < S) st4(xr + (size_t)t * H + h, xn[t]);
        }
        if (sum_out) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int t = 0; t < MAXS; ++t)
                if (t < S) a.x += xn[t].x, a.y += xn[t].y, a.z += xn[t].z, a.w += xn[t].w;
            st4(sum_out + (size_t)r * H + h, a);
        }
        if (in_next) {
            float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int t = 0; t < MAXS; ++t)
                if (t < S) {
                    const float m = s_in[t];
                    u.x = fmaf(m, xn[t].x, u.x), u.y = fmaf(m, xn[t].y, u.y), u.z = fmaf(m, xn[t].z, u.z), u.w = fmaf(m, xn[t].w, u.w);
                }
            *reinterpret_cast<float4*>(us + h) = u;
            ss += (u.x * u.x + u.y * u.y) + (u.z * u.z + u.w * u.w);
        }
    }
    if (!in_next) return;
    ss = il_block_sum(ss, red);
    const float rstd = 1.f / sqrtf(ss / (float)H + eps);
    for (int v = threadIdx.x; v < nv; v += blockDim.x) {
        const int h = 4 * v;
        const float4 u = *reinterpret_cast<const float4*>(us + h);
        const float4 wv = w_kind == IL_F32 ? ld4((const float*)w + h) : ld4((const __nv_bfloat16*)w + h);
        st4(normed + (size_t)r * H + h, make_float4(u.x * rstd * wv.x, u.y * rstd * wv.y, u.z * rstd * wv.z, u.w * rstd * wv.w));
    }
}

IL_EXPORT int il_hyper_step(float* streams, const float* init, const void* y, int act_kind, const float* mix, const float* out_w,
                            const float* in_next, const void* w, int w_kind, float eps, void* normed, float* sum_out, int S, int H, int T,
                            cudaStream_t stream) {
    if (T <= 0) return IL_OK;
    if (S <= 0 || S > HC_MAX_STREAMS || H <= 0 || (y && (!mix || !out_w)) || (in_next && (!w || !normed))) return IL_BAD_ARG;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return IL_UNSUPPORTED;
    const int threads = H >= 4096 ? 512 : H >= 1024 ? 256 : 128;
    // four columns a thread where rows are whole 16-byte pieces (and the copies fit the registers)
    const bool vec = (H & 3) == 0 && S <= 8 &&
                     (((uintptr_t)streams | (uintptr_t)init | (uintptr_t)y | (uintptr_t)w | (uintptr_t)normed | (uintptr_t)sum_out) & 15) == 0;
    const int vthreads = H >= 1024 ? 256 : H >= 512 ? 128 : 64;
#define HC_GO(TA, MAXS)                                                                                                                  \
    do {                                                                                                                                 \
        if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_step_kernel<TA, MAXS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        IL_LAUNCH((hyper_step_kernel<TA, MAXS>), T, threads, smem, stream, streams, init, (const TA*)y, mix, out_w, in_next, w, w_kind, eps, \
                  (TA*)normed, sum_out, S, H);                                                                                           \
    } while (0)
#define HC_GOV(TA, MAXS)                                                                                                                     \
    do {                                                                                                                                     \
        if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_step_vec_kernel<TA, MAXS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        IL_LAUNCH((hyper_step_vec_kernel<TA, MAXS>), T, vthreads, smem, stream, streams, init, (const TA*)y, mix, out_w, in_next, w, w_kind, \
                  eps, (TA*)normed, sum_out, S, H);                                                                                          \
    } while (0)
#define HC_PICK(TA)                                          \
    do {                                                     \
        if (vec && S <= 2) HC_GOV(TA, 2);                    \
        else if (vec && S <= 4) HC_GOV(TA, 4);               \
        else if (vec) HC_GOV(TA, 8);                         \
        else if (S <= 4) HC_GO(TA, 4);                       \
        else if (S <= 8) HC_GO(TA, 8);                       \
        else HC_GO(TA, 16);                                  \
    } while (0)
    if (act_kind == IL_F32) HC_PICK(float);
    else if (act_kind == IL_BF16) HC_PICK(__nv_bfloat16);
    else return IL_BAD_ARG;
#undef HC_PICK
#undef HC_GOV
#undef HC_GO
    IL_LAUNCH_CHECK();
    return IL_OK;
}
