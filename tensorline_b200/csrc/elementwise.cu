// Embedding gather, residual-add + RMSNorm, SwiGLU activation.
//
// Each kernel has a plain reference in tests/plain/qwen2_plain.py.  Formulas:
//   embedding   x[t,:] = E[ids[t],:]                       (tensorline/paged.py:240)
//   add+RMSNorm x += alpha r;  h = cast(x * rsqrt(mean(x^2)+eps)) * w   (tensorline/fused.py:19-32;
//               the cast to the activation type comes before the weight multiply, fused.py:32; with
//               `cast_first` 0 the norm is float to the end and only h is rounded; alpha = 1 is the plain sum)
//   SwiGLU      m = silu(g) * u,  silu(z) = z / (1 + e^-z), from the fused gate|up product
// The residual stream x is float in both engines, so the residual sum is a 32-bit sum.
#include "common.cuh"

// 1 if this library was compiled as the checking build (-DTL_CHECK=1).
TL_EXPORT int tl_check_build() { return TL_CHECKING; }

// ------------------------------------------------------------------ embedding
template <typename TW>
__global__ void embed_kernel(float* __restrict__ x, const TW* __restrict__ table,
                             const int* __restrict__ ids, int H, float scale) {
    const int t = blockIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    const TW* row = table + (size_t)ids[t] * H;
    float* out = x + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = to_f<TW>(row[i]) * scale;      // * 1.0f is exact
}

TL_EXPORT int tl_embed(void* x, const void* table, int table_dtype, const int* ids, int T, int H, float scale,
                       cudaStream_t stream) {
    if (T <= 0) return 0;
    if (table_dtype == TL_F32)
        launch_after_wait(embed_kernel<float>, dim3(T), dim3(256), 0, stream, (float*)x, (const float*)table, ids, H, scale);
    else
        launch_after_wait(embed_kernel<bf16>, dim3(T), dim3(256), 0, stream, (float*)x, (const bf16*)table, ids, H, scale);
    return tl_launch_status();
}

// ------------------------------------------------------------------ residual add + RMSNorm
// One block per output row.  rows == nullptr: row i of x; else row rows[i] (x is then only
// read, as for the final norm on the rows that want logits).
template <typename TA, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TA* __restrict__ r,
                                   const TW* __restrict__ w, TA* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps, int write_x, float alpha,
                                   int cast_first) {
    __shared__ float red[33];
    const int i = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[i] : i) * H;
    float* xr = x + src;
    const TA* rr = r ? r + src : nullptr;
    TA* o = out + (size_t)i * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = xr[c];
        if (rr) {
            v = fmaf(alpha, to_f<TA>(rr[c]), v);
            if (write_x) xr[c] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = xr[c];
        if (rr && !write_x) v = fmaf(alpha, to_f<TA>(rr[c]), v);
        const float n = cast_first ? to_f<TA>(from_f<TA>(v * rstd)) : v * rstd;      // cast first, then the weight
        o[c] = from_f<TA>(n * to_f<TW>(w[c]));
    }
}

// The fast path: H a multiple of 4, each thread keeps its NV chunks of 4 values in registers, so
// every load of the row is in flight at once and x, r are read exactly once.  Same arithmetic.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[4]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<uint32_t*>(&a); t.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = t;
    }
};

// `partial` (instead of r): the addend is still in pieces, [splits][rows of x][H] float, as a split-K product
// leaves them; they are summed in split order and rounded to the activation type first, which is what a
// separate reduction pass would have handed over as r.
template <typename TA, typename TW, int NV, bool PIECES>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ x, const TA* __restrict__ r,
                                       const TW* __restrict__ w, TA* __restrict__ out,
                                       const int* __restrict__ rows, int H, float eps, int write_x,
                                       const float* __restrict__ partial, int splits, size_t plane, float alpha,
                                       int cast_first) {
    __shared__ float red[33];
    const int i = blockIdx.x, nvec = H >> 2;
    float v[NV][4], wv[NV][4];
    // The weights are nobody's output.  A launch of few rows (a decode step) reads them before the wait for the
    // kernel in front, so only the row itself is fetched after it; a launch of many rows keeps all its loads
    // together behind the wait (the wait would otherwise stand between two memory latencies in every block).
    const bool early = gridDim.x <= 128;
    if (early) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nvec) Vec4<TW>::load(w + 4 * c, wv[k]);
        }
    }
    grid_dependency_wait();
    grid_dependency_trigger();
    const size_t src = (size_t)(rows ? rows[i] : i) * H;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < nvec) {
            Vec4<float>::load(x + src + 4 * c, v[k]);
            if (!early) Vec4<TW>::load(w + 4 * c, wv[k]);
        }
    }
    if (PIECES) {                                        // an instantiation of its own: the plain one keeps its registers
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nvec) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                for (int sp = 0; sp < splits; ++sp) {
                    float pv[4];
                    Vec4<float>::load(partial + sp * plane + src + 4 * c, pv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[e] += pv[e];
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) v[k][e] = fmaf(alpha, to_f<TA>(from_f<TA>(acc[e])), v[k][e]);
                if (write_x) Vec4<float>::store(x + src + 4 * c, v[k]);
            }
        }
    } else if (r) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nvec) {
                float rv[4];
                Vec4<TA>::load(r + src + 4 * c, rv);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[k][e] = fmaf(alpha, rv[e], v[k][e]);
                if (write_x) Vec4<float>::store(x + src + 4 * c, v[k]);
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
        if (threadIdx.x + k * blockDim.x < nvec)
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(v[k][e], v[k][e], ss);
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < nvec) {
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = (cast_first ? to_f<TA>(from_f<TA>(v[k][e] * rstd)) : v[k][e] * rstd) * wv[k][e];
            Vec4<TA>::store(out + (size_t)i * H + 4 * c, o);
        }
    }
}

template <typename TA, typename TW>
static int launch_add_rmsnorm(void* x, const void* r, const void* w, void* out, const int* rows, int R, int H,
                              float eps, int write_x, const float* partial, int splits, size_t plane, float alpha,
                              int cast_first, cudaStream_t stream) {
    const int nvec = H >> 2;
    const bool vec = (H & 3) == 0 && nvec <= 8192 &&
                     ((((uintptr_t)x | (uintptr_t)r | (uintptr_t)w | (uintptr_t)out | (uintptr_t)partial) & 15) == 0);
    if (partial && !vec) return 1;                       // pieces only on the vector path; the caller sums them first
#define VLAUNCH(NV) { int th = ((nvec + NV - 1) / NV + 31) / 32 * 32; \
        if (partial) launch_after_wait(add_rmsnorm_vec_kernel<TA, TW, NV, true>, dim3(R), dim3(th), 0, stream, (float*)x, (const TA*)r, (const TW*)w, (TA*)out, rows, H, eps, write_x, partial, splits, plane, alpha, cast_first); \
        else launch_after_wait(add_rmsnorm_vec_kernel<TA, TW, NV, false>, dim3(R), dim3(th), 0, stream, (float*)x, (const TA*)r, (const TW*)w, (TA*)out, rows, H, eps, write_x, partial, splits, plane, alpha, cast_first); }
    if (!vec) add_rmsnorm_kernel<TA, TW><<<R, 256, 0, stream>>>((float*)x, (const TA*)r, (const TW*)w, (TA*)out, rows, H, eps, write_x, alpha, cast_first);
    else if (nvec <= 1024) VLAUNCH(1)
    else if (nvec <= 2048) VLAUNCH(2)
    else if (nvec <= 4096) VLAUNCH(4)
    else VLAUNCH(8)
#undef VLAUNCH
    return 0;
}

TL_EXPORT int tl_add_rmsnorm(void* x, const void* r, const void* w, int w_dtype, void* out, int act_dtype,
                             const int* rows, int R, int H, float eps, int write_x, const float* partial, int splits,
                             long long plane, float alpha, int cast_first, cudaStream_t stream) {
    if (R <= 0) return 0;
    int e;
    if (act_dtype == TL_F32) {
        if (w_dtype == TL_F32) e = launch_add_rmsnorm<float, float>(x, r, w, out, rows, R, H, eps, write_x, partial, splits, (size_t)plane, alpha, cast_first, stream);
        else e = launch_add_rmsnorm<float, bf16>(x, r, w, out, rows, R, H, eps, write_x, partial, splits, (size_t)plane, alpha, cast_first, stream);
    } else {
        if (w_dtype == TL_F32) e = launch_add_rmsnorm<bf16, float>(x, r, w, out, rows, R, H, eps, write_x, partial, splits, (size_t)plane, alpha, cast_first, stream);
        else e = launch_add_rmsnorm<bf16, bf16>(x, r, w, out, rows, R, H, eps, write_x, partial, splits, (size_t)plane, alpha, cast_first, stream);
    }
    return e ? e : tl_launch_status();
}

// ------------------------------------------------------------------ SwiGLU activation
// gu is [T, 2*I], out [T, I].  Gate and up columns alternate in blocks of `blk` columns: out column c has its
// gate at (c / blk) * 2 blk + c % blk and its up value blk columns further.  blk = I is the plain layout
// (gate in [0, I), up in [I, 2I)); blk = 64 is what a product against interleaved weight rows leaves.
// `act` picks the gate's function: TL_ACT_SILU, or TL_ACT_GELU_TANH (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))).
template <typename TA>
__global__ void silu_mul_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int I, int blk, size_t total, int act,
                                float limit, float alpha) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int c = (int)(idx - t * I);
        const int gc = (c / blk) * 2 * blk + c % blk;
        const float g = to_f<TA>(gu[t * 2 * I + gc]);
        const float u = to_f<TA>(gu[t * 2 * I + gc + blk]);
        if (act == TL_ACT_GELU_TANH) out[idx] = from_f<TA>(tl_gelu_tanh(g) * u);
        else if (act == TL_ACT_SWISH_CLAMPED)
            out[idx] = from_f<TA>(sizeof(TA) == 4 ? tl_swish_clamped(g, u, limit, alpha) : tl_swish_clamped_bf16(g, u, limit, alpha));
        else if constexpr (sizeof(TA) == 4) out[idx] = (g / (1.0f + expf(-g))) * u;     // the 32-bit engine: exact division
        else                           out[idx] = from_f<TA>(tl_silu_mul(g, u));
    }
}

// 8 values (16 bytes of bfloat16) per thread and chunk: requires I % 8 == 0 and blk % 8 == 0.  grid (column
// groups, tokens): no division per element; with many tokens a thread takes two chunks a block's width apart,
// so four 16-byte loads are in flight before the first is used; with few it takes one, for more blocks.
template <int CHUNKS, int ACT>
__global__ void __launch_bounds__(256) silu_mul_vec8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I, int blk,
                                                            float limit, float alpha) {
    const size_t t = blockIdx.y;
    const int c0 = (blockIdx.x * 256 * CHUNKS + threadIdx.x) * 8;
    grid_dependency_wait();
    grid_dependency_trigger();
    const bf16* row = gu + t * 2 * (size_t)I;
    uint4 gv[CHUNKS], uv[CHUNKS];
    int cs[CHUNKS];
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) cs[k] = c0 + k * 256 * 8;
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
        if (cs[k] < I) {
            const int gc = (cs[k] / blk) * 2 * blk + cs[k] % blk;
            gv[k] = *reinterpret_cast<const uint4*>(row + gc);
            uv[k] = *reinterpret_cast<const uint4*>(row + gc + blk);
        }
    }
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
        if (cs[k] >= I) continue;
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv[k]);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv[k]);
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float g0 = __low2float(g2[e]), g1 = __high2float(g2[e]);
            const float u0 = __low2float(u2[e]), u1 = __high2float(u2[e]);
            if (ACT == TL_ACT_GELU_TANH) o2[e] = __floats2bfloat162_rn(tl_gelu_tanh(g0) * u0, tl_gelu_tanh(g1) * u1);
            else if (ACT == TL_ACT_SWISH_CLAMPED)
                o2[e] = __floats2bfloat162_rn(tl_swish_clamped_bf16(g0, u0, limit, alpha), tl_swish_clamped_bf16(g1, u1, limit, alpha));
            else o2[e] = __floats2bfloat162_rn(tl_silu_mul(g0, u0), tl_silu_mul(g1, u1));
        }
        *reinterpret_cast<uint4*>(out + t * I + cs[k]) = ov;
    }
}

TL_EXPORT int tl_silu_mul(const void* gu, void* out, int act_dtype, int T, int I, int blk, int act, float limit, float alpha,
                          cudaStream_t stream) {
    const size_t total = (size_t)T * I;
    if (total == 0) return 0;
    if (blk <= 0 || I % blk || (act != TL_ACT_SILU && act != TL_ACT_GELU_TANH && act != TL_ACT_SWISH_CLAMPED)) return 1;
    const int threads = 256;
    if (act_dtype == TL_BF16 && (I & 7) == 0 && (blk & 7) == 0 && T <= 65535 && ((((uintptr_t)gu | (uintptr_t)out) & 15) == 0)) {
#define SMV(CH, A) launch_after_wait(silu_mul_vec8_kernel<CH, A>, dim3((unsigned)((I / 8 + 256 * CH - 1) / (256 * CH)), (unsigned)T), dim3(threads), 0, stream, \
                                 (const bf16*)gu, (bf16*)out, I, blk, limit, alpha)
        if (act == TL_ACT_SWISH_CLAMPED) return T >= 256 ? SMV(2, TL_ACT_SWISH_CLAMPED) : SMV(1, TL_ACT_SWISH_CLAMPED);
        if (act == TL_ACT_GELU_TANH) return T >= 256 ? SMV(2, TL_ACT_GELU_TANH) : SMV(1, TL_ACT_GELU_TANH);
        return T >= 256 ? SMV(2, TL_ACT_SILU) : SMV(1, TL_ACT_SILU);
#undef SMV
    }
    const size_t cap = (size_t)tl_num_sms() * 16;
    const int blocks = (int)((total + threads - 1) / threads < cap ? (total + threads - 1) / threads : cap);
    if (act_dtype == TL_F32)
        silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, I, blk, total, act, limit, alpha);
    else
        silu_mul_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, I, blk, total, act, limit, alpha);
    return tl_launch_status();
}

// ------------------------------------------------------------------ a sub-block's own norm, the residual sum, the next norm
// For blocks that normalise a sub-block's output before it joins the residual stream:
//   x += a / rms(a) * w_post  (+ extra, a row vector added once);   h = x / rms(x) * w_pre
// all in float, one block a row.  `a` null: no addend (only extra and the norm); `out` null: no norm (only the sum);
// `rows`: as above, x is then left alone.  Nothing is rounded before h.
template <typename TA, typename TW>
__global__ void __launch_bounds__(256) post_norm_add_norm_kernel(float* __restrict__ x, const TA* __restrict__ a, const TW* __restrict__ w_post,
                                                                 const float* __restrict__ extra, const TW* __restrict__ w_pre,
                                                                 TA* __restrict__ out, const int* __restrict__ rows, int H, float eps,
                                                                 int write_x) {
    __shared__ float red[33];
    const int i = blockIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    const size_t src = (size_t)(rows ? rows[i] : i) * H;
    float* xr = x + src;
    float ra = 0.f;
    if (a) {
        float sa = 0.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) { const float v = to_f<TA>(a[src + c]); sa = fmaf(v, v, sa); }
        sa = block_sum(sa, red);
        ra = 1.0f / sqrtf(sa / (float)H + eps);
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = xr[c];
        if (a) v += to_f<TA>(a[src + c]) * ra * to_f<TW>(w_post[c]);
        if (extra) v += extra[c];
        if (write_x) xr[c] = v;
        ss = fmaf(v, v, ss);
    }
    if (!out) return;
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = xr[c];
        if (!write_x) {                                  // the same chain of operations as above
            if (a) v += to_f<TA>(a[src + c]) * ra * to_f<TW>(w_post[c]);
            if (extra) v += extra[c];
        }
        out[(size_t)i * H + c] = from_f<TA>(v * rstd * to_f<TW>(w_pre[c]));
    }
}

// The fast path: H a multiple of 4; a thread keeps its NV chunks of 4 values of x and a in registers, so every load of the
// row is in flight at once and x, a are read exactly once.  A launch of few rows (a decode step) reads the weights, which
// are nobody's output, before the wait for the kernel in front.
template <typename TA, typename TW, int NV>
__global__ void post_norm_add_norm_vec_kernel(float* __restrict__ x, const TA* __restrict__ a, const TW* __restrict__ w_post,
                                              const float* __restrict__ extra, const TW* __restrict__ w_pre, TA* __restrict__ out,
                                              const int* __restrict__ rows, int H, float eps, int write_x) {
    __shared__ float red[33];
    const int i = blockIdx.x, nvec = H >> 2;
    float v[NV][4], av[NV][4], wv[NV][4];
    const bool early = gridDim.x <= 128;
    if (early && a) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nvec) Vec4<TW>::load(w_post + 4 * c, wv[k]);
        }
    }
    grid_dependency_wait();
    grid_dependency_trigger();
    const size_t src = (size_t)(rows ? rows[i] : i) * H;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < nvec) {
            Vec4<float>::load(x + src + 4 * c, v[k]);
            if (a) {
                Vec4<TA>::load(a + src + 4 * c, av[k]);
                if (!early) Vec4<TW>::load(w_post + 4 * c, wv[k]);
            }
        }
    }
    if (a) {
        float sa = 0.f;
#pragma unroll
        for (int k = 0; k < NV; ++k)
            if (threadIdx.x + k * blockDim.x < nvec)
#pragma unroll
                for (int e = 0; e < 4; ++e) sa = fmaf(av[k][e], av[k][e], sa);
        sa = block_sum(sa, red);
        const float ra = 1.0f / sqrtf(sa / (float)H + eps);
#pragma unroll
        for (int k = 0; k < NV; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) v[k][e] += av[k][e] * ra * wv[k][e];
    }
    if (extra) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nvec) {
                float ev[4];
                Vec4<float>::load(extra + 4 * c, ev);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[k][e] += ev[e];
            }
        }
    }
    if (write_x && (a || extra)) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nvec) Vec4<float>::store(x + src + 4 * c, v[k]);
        }
    }
    if (!out) return;
#pragma unroll
    for (int k = 0; k < NV; ++k) {                           // the second norm's weights: the first one's are done with
        const int c = threadIdx.x + k * blockDim.x;
        if (c < nvec) Vec4<TW>::load(w_pre + 4 * c, wv[k]);
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
        if (threadIdx.x + k * blockDim.x < nvec)
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(v[k][e], v[k][e], ss);
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < nvec) {
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = v[k][e] * rstd * wv[k][e];
            Vec4<TA>::store(out + (size_t)i * H + 4 * c, o);
        }
    }
}

template <typename TA, typename TW>
static int launch_post_norm(void* x, const void* a, const void* w_post, const float* extra, const void* w_pre, void* out,
                            const int* rows, int R, int H, float eps, int write_x, cudaStream_t stream) {
    const int nvec = H >> 2;
    const bool vec = (H & 3) == 0 && nvec <= 4096 &&
                     ((((uintptr_t)x | (uintptr_t)a | (uintptr_t)w_post | (uintptr_t)w_pre | (uintptr_t)out | (uintptr_t)extra) & 15) == 0);
#define PNV(NV) { int th = ((nvec + NV - 1) / NV + 31) / 32 * 32; \
        return launch_after_wait(post_norm_add_norm_vec_kernel<TA, TW, NV>, dim3(R), dim3(th), 0, stream, (float*)x, (const TA*)a, \
                                 (const TW*)w_post, extra, (const TW*)w_pre, (TA*)out, rows, H, eps, write_x); }
    if (vec) {
        if (nvec <= 1024) PNV(1)
        else if (nvec <= 2048) PNV(2)
        else PNV(4)
    }
#undef PNV
    return launch_after_wait(post_norm_add_norm_kernel<TA, TW>, dim3(R), dim3(256), 0, stream, (float*)x, (const TA*)a,
                             (const TW*)w_post, extra, (const TW*)w_pre, (TA*)out, rows, H, eps, write_x);
}

TL_EXPORT int tl_post_norm_add_norm(void* x, const void* a, const void* w_post, const float* extra, const void* w_pre, int w_dtype,
                                    void* out, int act_dtype, const int* rows, int R, int H, float eps, int write_x,
                                    cudaStream_t stream) {
    if (R <= 0) return 0;
    int e;
    if (act_dtype == TL_F32) {
        e = w_dtype == TL_F32 ? launch_post_norm<float, float>(x, a, w_post, extra, w_pre, out, rows, R, H, eps, write_x, stream)
                              : launch_post_norm<float, bf16>(x, a, w_post, extra, w_pre, out, rows, R, H, eps, write_x, stream);
    } else {
        e = w_dtype == TL_F32 ? launch_post_norm<bf16, float>(x, a, w_post, extra, w_pre, out, rows, R, H, eps, write_x, stream)
                              : launch_post_norm<bf16, bf16>(x, a, w_post, extra, w_pre, out, rows, R, H, eps, write_x, stream);
    }
    return e ? e : tl_launch_status();
}


// ------------------------------------------------------------------ the residual sum and two norms of one stream
// For blocks whose two sub-blocks read the same stream (x += mixer(norm1(x)) + feed_forward(norm2(x))):
//   x += a + b   (either may be null; the two are added first, then to x);   h1 = x / rms(x) * w1;   h2 = x / rms(x) * w2
// all in float, one block a row, one set of statistics for both norms; only h1 and h2 are rounded.  `h2` null: one norm.
// `rows`: only those rows are produced and x is left alone.
template <typename TA, typename TW>
__global__ void __launch_bounds__(256) add_rmsnorm_pair_kernel(float* __restrict__ x, const TA* __restrict__ a, const TA* __restrict__ b,
                                                               const TW* __restrict__ w1, const TW* __restrict__ w2, TA* __restrict__ h1,
                                                               TA* __restrict__ h2, const int* __restrict__ rows, int H, float eps) {
    __shared__ float red[33];
    const int i = blockIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    const size_t src = (size_t)(rows ? rows[i] : i) * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = x[src + c];
        if (a) {
            const float add = b ? to_f<TA>(a[src + c]) + to_f<TA>(b[src + c]) : to_f<TA>(a[src + c]);
            v += add;
            if (!rows) x[src + c] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = x[src + c];                            // its own write of the first pass, or the untouched row
        if (a && rows) v += b ? to_f<TA>(a[src + c]) + to_f<TA>(b[src + c]) : to_f<TA>(a[src + c]);
        const float n = v * rstd;
        h1[(size_t)i * H + c] = from_f<TA>(n * to_f<TW>(w1[c]));
        if (h2) h2[(size_t)i * H + c] = from_f<TA>(n * to_f<TW>(w2[c]));
    }
}

// The fast path, as for the single norm: H a multiple of 4, a thread keeps its NV chunks of 4 values in registers, every load
// of the row is in flight at once, x, a and b are read once.  Few rows (a decode step): the weights, nobody's output, are read
// before the wait for the kernel in front.  Same arithmetic as above but for the order of the sum of squares.
template <typename TA, typename TW, int NV>
__global__ void add_rmsnorm_pair_vec_kernel(float* __restrict__ x, const TA* __restrict__ a, const TA* __restrict__ b,
                                            const TW* __restrict__ w1, const TW* __restrict__ w2, TA* __restrict__ h1,
                                            TA* __restrict__ h2, const int* __restrict__ rows, int H, float eps) {
    __shared__ float red[33];
    const int i = blockIdx.x, nvec = H >> 2;
    float v[NV][4], wa[NV][4], wb[NV][4];
    const bool early = gridDim.x <= 128 && NV <= 2;
    if (early) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nvec) {
                Vec4<TW>::load(w1 + 4 * c, wa[k]);
                if (h2) Vec4<TW>::load(w2 + 4 * c, wb[k]);
            }
        }
    }
    grid_dependency_wait();
    grid_dependency_trigger();
    const size_t src = (size_t)(rows ? rows[i] : i) * H;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < nvec) Vec4<float>::load(x + src + 4 * c, v[k]);
    }
    if (a) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nvec) {
                float av[4], bv[4] = {0.f, 0.f, 0.f, 0.f};
                Vec4<TA>::load(a + src + 4 * c, av);
                if (b) Vec4<TA>::load(b + src + 4 * c, bv);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[k][e] += b ? av[e] + bv[e] : av[e];
                if (!rows) Vec4<float>::store(x + src + 4 * c, v[k]);
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
        if (threadIdx.x + k * blockDim.x < nvec)
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(v[k][e], v[k][e], ss);
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < nvec) {
            if (!early) {
                Vec4<TW>::load(w1 + 4 * c, wa[k]);
                if (h2) Vec4<TW>::load(w2 + 4 * c, wb[k]);
            }
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = v[k][e] * rstd * wa[k][e];
            Vec4<TA>::store(h1 + (size_t)i * H + 4 * c, o);
            if (h2) {
#pragma unroll
                for (int e = 0; e < 4; ++e) o[e] = v[k][e] * rstd * wb[k][e];
                Vec4<TA>::store(h2 + (size_t)i * H + 4 * c, o);
            }
        }
    }
}

template <typename TA, typename TW>
static void launch_add_rmsnorm_pair(float* x, const void* a, const void* b, const void* w1, const void* w2, void* h1, void* h2,
                                    const int* rows, int R, int H, float eps, cudaStream_t stream) {
    const int nvec = H >> 2;
    const bool vec = (H & 3) == 0 && nvec <= 8192 &&
                     ((((uintptr_t)x | (uintptr_t)a | (uintptr_t)b | (uintptr_t)w1 | (uintptr_t)w2 | (uintptr_t)h1 | (uintptr_t)h2) & 15) == 0);
#define PLAUNCH(NV) launch_after_wait(add_rmsnorm_pair_vec_kernel<TA, TW, NV>, dim3(R), dim3(((nvec + NV - 1) / NV + 31) / 32 * 32), 0, stream, \
        x, (const TA*)a, (const TA*)b, (const TW*)w1, (const TW*)w2, (TA*)h1, (TA*)h2, rows, H, eps)
    if (!vec) launch_after_wait(add_rmsnorm_pair_kernel<TA, TW>, dim3(R), dim3(256), 0, stream, x, (const TA*)a, (const TA*)b,
                                (const TW*)w1, (const TW*)w2, (TA*)h1, (TA*)h2, rows, H, eps);
    else if (nvec <= 1024) PLAUNCH(1);
    else if (nvec <= 2048) PLAUNCH(2);
    else if (nvec <= 4096) PLAUNCH(4);
    else PLAUNCH(8);
#undef PLAUNCH
}

TL_EXPORT int tl_add_rmsnorm_pair(float* x, const void* a, const void* b, const void* w1, const void* w2, int w_dtype, void* h1,
                                  void* h2, int act_dtype, const int* rows, int R, int H, float eps, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (b && !a) return 1;
#define ARP(TA, TW) launch_add_rmsnorm_pair<TA, TW>(x, a, b, w1, w2, h1, h2, rows, R, H, eps, stream)
    if (act_dtype == TL_F32) { if (w_dtype == TL_F32) ARP(float, float); else ARP(float, bf16); }
    else { if (w_dtype == TL_F32) ARP(bf16, float); else ARP(bf16, bf16); }
#undef ARP
    return tl_launch_status();
}

// ------------------------------------------------------------------ a sigmoid gate per (token, head) on attention's output
// o[t, h, :] *= sigmoid(gate[t, h]); gate float [T, nq].
template <typename TA>
__global__ void head_gate_kernel(TA* __restrict__ o, const float* __restrict__ gate, int d, size_t total) {
    grid_dependency_wait();
    grid_dependency_trigger();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const float g = 1.0f / (1.0f + expf(-gate[idx / d]));
        o[idx] = from_f<TA>(to_f<TA>(o[idx]) * g);
    }
}

// sixteen bytes a thread (eight bfloat16 or four floats of one head: d is a multiple of that many, o is 16-byte aligned)
template <typename TA>
__global__ void head_gate_vec_kernel(TA* __restrict__ o, const float* __restrict__ gate, int vecs_per_head, size_t vecs) {
    constexpr int N = 16 / sizeof(TA);
    grid_dependency_wait();
    grid_dependency_trigger();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < vecs; idx += (size_t)gridDim.x * blockDim.x) {
        const float g = 1.0f / (1.0f + expf(-gate[idx / vecs_per_head]));
        uint4 raw = reinterpret_cast<const uint4*>(o)[idx];
        TA* e = reinterpret_cast<TA*>(&raw);
#pragma unroll
        for (int k = 0; k < N; ++k) e[k] = from_f<TA>(to_f<TA>(e[k]) * g);
        reinterpret_cast<uint4*>(o)[idx] = raw;
    }
}

TL_EXPORT int tl_head_gate(void* o, int act_dtype, const float* gate, int T, int nq, int d, cudaStream_t stream) {
    const size_t total = (size_t)T * nq * d;
    if (total == 0) return 0;
    const size_t cap = (size_t)tl_num_sms() * 16;
    const int per = act_dtype == TL_F32 ? 4 : 8;
    if (d % per == 0 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
        const size_t vecs = total / per;
        const unsigned vb = (unsigned)((vecs + 255) / 256 < cap ? (vecs + 255) / 256 : cap);
        if (act_dtype == TL_F32) launch_after_wait(head_gate_vec_kernel<float>, dim3(vb), dim3(256), 0, stream, (float*)o, gate, d / per, vecs);
        else launch_after_wait(head_gate_vec_kernel<bf16>, dim3(vb), dim3(256), 0, stream, (bf16*)o, gate, d / per, vecs);
        return tl_launch_status();
    }
    const unsigned blocks = (unsigned)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
    if (act_dtype == TL_F32) launch_after_wait(head_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)o, gate, d, total);
    else launch_after_wait(head_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)o, gate, d, total);
    return tl_launch_status();
}
