// A residual stream kept as several copies (hyper-connections), an embedding with a hashed table of token pairs, a cap
// on the logits and a sigmoid gate, all float arithmetic.
//
//   embedding   e[t] = E[id_t] * scale + P[(prev_t * mul_prev + id_t * mul_cur) mod buckets]; a request's first token has no
//               previous one and takes row `buckets` of P.  `prev_t` is the token in front of t in the step, or, for the first
//               row of a request's portion, the request's last token of the step before (an int a request slot).  e is
//               written `copies` times side by side: the S streams start equal.
//   streams     x [T, S, W].  One kernel per sublayer boundary does, per token and column,
//                   y      = alpha a + beta b                       the sublayer's output (two addends of a mixer pair)
//                   x_r'   = sum_s mix[s, r] x_s + out[r] y         every stream from the old ones
//                   u      = sum_r read[r] x_r'                     what the next sublayer reads (read null: the plain sum)
//                   h      = u / sqrt(mean(u^2) + eps) * w          rounded once to the activation type
//               with every part optional: no update (the first sublayer of a model), no norm (u alone is wanted), picked
//               rows (x is then left alone).  The order of the sums is fixed: s = 0 .. S - 1, then r = 0 .. S - 1.
//   cap         z <- cap tanh(z / cap) over the logits, in place
//   gate        y[t, c] = o[t, c] * sigmoid(g[t, c]), g float with a row stride of its own
#include "common.cuh"

constexpr int STREAMS_MAX = 16;

template <typename TW>
__global__ void __launch_bounds__(256) embed_streams_kernel(float* __restrict__ x, const TW* __restrict__ table, const int* __restrict__ ids,
                                                            int H, float scale, int copies, const TW* __restrict__ pairs, int buckets,
                                                            int mul_prev, int mul_cur, const int* __restrict__ pos,
                                                            const int* __restrict__ req_slot, const int* __restrict__ last_token) {
    const int t = blockIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    const int id = ids[t];
    const TW* row = table + (size_t)id * H;
    const TW* prow = nullptr;
    if (pairs) {
        long long r = buckets;
        if (pos[t] > 0) {
            const int slot = req_slot[t];
            const long long prev = (t > 0 && req_slot[t - 1] == slot) ? ids[t - 1] : last_token[slot];
            r = (prev * (long long)mul_prev + (long long)id * (long long)mul_cur) % (long long)buckets;
            if (r < 0) r += buckets;
        }
        prow = pairs + (size_t)r * H;
    }
    float* out = x + (size_t)t * H * copies;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = to_f<TW>(row[i]) * scale;
        if (prow) v += to_f<TW>(prow[i]);
        for (int c = 0; c < copies; ++c) out[(size_t)c * H + i] = v;
    }
}

TL_EXPORT int tl_embed_streams(float* x, const void* table, int table_dtype, const int* ids, int T, int H, float scale, int copies,
                               const void* pairs, int buckets, int mul_prev, int mul_cur, const int* pos, const int* req_slot,
                               const int* last_token, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (copies < 1 || (pairs && (buckets < 1 || !pos || !req_slot || !last_token))) return 1;
    if (table_dtype == TL_F32)
        launch_after_wait(embed_streams_kernel<float>, dim3(T), dim3(256), 0, stream, x, (const float*)table, ids, H, scale, copies,
                          (const float*)pairs, buckets, mul_prev, mul_cur, pos, req_slot, last_token);
    else
        launch_after_wait(embed_streams_kernel<bf16>, dim3(T), dim3(256), 0, stream, x, (const bf16*)table, ids, H, scale, copies,
                          (const bf16*)pairs, buckets, mul_prev, mul_cur, pos, req_slot, last_token);
    return tl_launch_status();
}

// last_token[slots[b]] = the last id of request b's rows in this step (q_start [B + 1]).  A launch of its own behind the
// embedding: the first row of a portion reads what the last row of the portion before left.
__global__ void remember_last_kernel(const int* __restrict__ ids, const int* __restrict__ q_start, const int* __restrict__ slots, int B,
                                     int* __restrict__ last_token) {
    grid_dependency_wait();
    grid_dependency_trigger();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B && q_start[b + 1] > q_start[b]) last_token[slots[b]] = ids[q_start[b + 1] - 1];
}

TL_EXPORT int tl_remember_last(const int* ids, const int* q_start, const int* slots, int B, int* last_token, cudaStream_t stream) {
    if (B <= 0) return 0;
    launch_after_wait(remember_last_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, ids, q_start, slots, B, last_token);
    return tl_launch_status();
}

// One block a row.  Shared memory: mix [S * S], out [S], read [S], then u [W].
template <typename TA, typename TW>
__global__ void __launch_bounds__(256) stream_step_kernel(float* __restrict__ x, int S, int W, const TA* __restrict__ a, float alpha,
                                                          const TA* __restrict__ b, float beta, const float* __restrict__ mix,
                                                          const float* __restrict__ out, const float* __restrict__ read,
                                                          const TW* __restrict__ w, float eps, TA* __restrict__ h,
                                                          float* __restrict__ u_out, const int* __restrict__ rows, int write_x) {
    extern __shared__ float sm[];
    __shared__ float red[33];
    float* s_mix = sm;
    float* s_out = sm + S * S;
    float* s_read = s_out + S;
    float* u = s_read + S;
    const int i = blockIdx.x;
    for (int k = threadIdx.x; k < S * S; k += blockDim.x) s_mix[k] = mix ? mix[k] : 0.f;
    for (int k = threadIdx.x; k < S; k += blockDim.x) { s_out[k] = out ? out[k] : 0.f; s_read[k] = read ? read[k] : 1.0f; }
    grid_dependency_wait();
    grid_dependency_trigger();
    __syncthreads();
    const size_t t = rows ? (size_t)rows[i] : (size_t)i;
    float* xr = x + t * (size_t)S * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float old[STREAMS_MAX];
#pragma unroll
        for (int s = 0; s < STREAMS_MAX; ++s) if (s < S) old[s] = xr[(size_t)s * W + c];
        float acc = 0.f;
        if (mix) {
            float y = 0.f;
            if (a) y = alpha * to_f<TA>(a[t * W + c]);
            if (b) y = fmaf(beta, to_f<TA>(b[t * W + c]), y);
#pragma unroll
            for (int r = 0; r < STREAMS_MAX; ++r) {
                if (r < S) {
                    float v = 0.f;
#pragma unroll
                    for (int s = 0; s < STREAMS_MAX; ++s) if (s < S) v = fmaf(s_mix[s * S + r], old[s], v);
                    v = fmaf(s_out[r], y, v);
                    if (write_x) xr[(size_t)r * W + c] = v;
                    acc = fmaf(s_read[r], v, acc);
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < STREAMS_MAX; ++r) if (r < S) acc = fmaf(s_read[r], old[r], acc);
        }
        u[c] = acc;
        ss = fmaf(acc, acc, ss);
    }
    if (u_out) for (int c = threadIdx.x; c < W; c += blockDim.x) u_out[(size_t)i * W + c] = u[c];
    if (!h) return;
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) h[(size_t)i * W + c] = from_f<TA>(u[c] * rstd * to_f<TW>(w[c]));
}

// Four columns a thread (W % 4 == 0, every pointer aligned for it), as many threads as the row has such groups (up to 1,024):
// a row of up to 4,096 columns is one pass with all of a thread's loads in flight together.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    return make_float4(__low2float(h[0]), __high2float(h[0]), __low2float(h[1]), __high2float(h[1]));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(bf16* p, float4 v) {
    uint2 o;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
    h[0] = __floats2bfloat162_rn(v.x, v.y); h[1] = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = o;
}
__device__ __forceinline__ float4 fma4(float k, float4 v, float4 acc) {
    return make_float4(fmaf(k, v.x, acc.x), fmaf(k, v.y, acc.y), fmaf(k, v.z, acc.z), fmaf(k, v.w, acc.w));
}

// SM: the most copies this instance takes (a thread keeps SM x 4 old values in registers); MAXT: its largest block.
template <typename TA, typename TW, int SM, int MAXT>
__global__ void __launch_bounds__(MAXT) stream_step_vec_kernel(float* __restrict__ x, int S, int W, const TA* __restrict__ a, float alpha,
                                                               const TA* __restrict__ b, float beta, const float* __restrict__ mix,
                                                               const float* __restrict__ out, const float* __restrict__ read,
                                                               const TW* __restrict__ w, float eps, TA* __restrict__ h,
                                                               float* __restrict__ u_out, const int* __restrict__ rows, int write_x) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[33];
    float* u = sm;                                         // [W], then mix [S * S], out [S], read [S]
    float* s_mix = sm + W;
    float* s_out = s_mix + S * S;
    float* s_read = s_out + S;
    const int i = blockIdx.x;
    for (int k = threadIdx.x; k < S * S; k += blockDim.x) s_mix[k] = mix ? mix[k] : 0.f;
    for (int k = threadIdx.x; k < S; k += blockDim.x) { s_out[k] = out ? out[k] : 0.f; s_read[k] = read ? read[k] : 1.0f; }
    grid_dependency_wait();
    grid_dependency_trigger();
    __syncthreads();
    const size_t t = rows ? (size_t)rows[i] : (size_t)i;
    float* xr = x + t * (size_t)S * W;
    float ss = 0.f;
    for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
        float4 old[SM];
#pragma unroll
        for (int s = 0; s < SM; ++s) if (s < S) old[s] = ld4(xr + (size_t)s * W + c);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (mix) {
            float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
            if (a) { const float4 av = ld4(a + t * W + c); y = make_float4(alpha * av.x, alpha * av.y, alpha * av.z, alpha * av.w); }
            if (b) y = fma4(beta, ld4(b + t * W + c), y);
#pragma unroll
            for (int r = 0; r < SM; ++r) {
                if (r < S) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int s = 0; s < SM; ++s) if (s < S) v = fma4(s_mix[s * S + r], old[s], v);
                    v = fma4(s_out[r], y, v);
                    if (write_x) st4(xr + (size_t)r * W + c, v);
                    acc = fma4(s_read[r], v, acc);
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < SM; ++r) if (r < S) acc = fma4(s_read[r], old[r], acc);
        }
        st4(u + c, acc);
        ss = fmaf(acc.x, acc.x, ss); ss = fmaf(acc.y, acc.y, ss); ss = fmaf(acc.z, acc.z, ss); ss = fmaf(acc.w, acc.w, ss);
    }
    if (u_out) for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) st4(u_out + (size_t)i * W + c, ld4(u + c));
    if (!h) return;
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
        const float4 uv = ld4(u + c), wv = ld4(w + c);
        st4(h + (size_t)i * W + c, make_float4(uv.x * rstd * wv.x, uv.y * rstd * wv.y, uv.z * rstd * wv.z, uv.w * rstd * wv.w));
    }
}

TL_EXPORT int tl_stream_step(float* x, int S, int W, const void* a, float alpha, const void* b, float beta, int act_dtype,
                             const float* mix, const float* out, const float* read, const void* w, int w_dtype, float eps, void* h,
                             float* u_out, const int* rows, int R, int write_x, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (S < 1 || S > STREAMS_MAX || (mix == nullptr) != (out == nullptr) || (h && !w)) return 1;
    const size_t smem = ((size_t)S * S + 2 * S + W) * sizeof(float);
    if (smem > 200 * 1024) return 1;
    if (rows) write_x = 0;
    const uintptr_t all = (uintptr_t)x | (uintptr_t)a | (uintptr_t)b | (uintptr_t)w | (uintptr_t)h | (uintptr_t)u_out;
    if (W % 4 == 0 && (all & 15) == 0) {                   // (bfloat16 rows of W % 4 == 0 columns keep the alignment of their base)
        const int groups = W / 4, most = S <= 4 ? 1024 : S <= 8 ? 512 : 256;
        const int threads = groups >= most ? most : groups <= 64 ? 64 : ((groups + 31) / 32) * 32;
#define SV3(TA, TW, SM, MAXT) do { \
        if (smem > 48 * 1024) cudaFuncSetAttribute(stream_step_vec_kernel<TA, TW, SM, MAXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_after_wait(stream_step_vec_kernel<TA, TW, SM, MAXT>, dim3(R), dim3(threads), smem, stream, x, S, W, (const TA*)a, alpha, (const TA*)b, beta, \
                          mix, out, read, (const TW*)w, eps, (TA*)h, u_out, rows, write_x); } while (0)
#define SV(TA, TW) do { if (S <= 4) SV3(TA, TW, 4, 1024); else if (S <= 8) SV3(TA, TW, 8, 512); else SV3(TA, TW, 16, 256); } while (0)
        if (act_dtype == TL_F32) { if (w_dtype == TL_F32) SV(float, float); else SV(float, bf16); }
        else { if (w_dtype == TL_F32) SV(bf16, float); else SV(bf16, bf16); }
#undef SV
#undef SV3
        return tl_launch_status();
    }
#define SS(TA, TW) do { \
        if (smem > 48 * 1024) cudaFuncSetAttribute(stream_step_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_after_wait(stream_step_kernel<TA, TW>, dim3(R), dim3(256), smem, stream, x, S, W, (const TA*)a, alpha, (const TA*)b, beta, \
                          mix, out, read, (const TW*)w, eps, (TA*)h, u_out, rows, write_x); } while (0)
    if (act_dtype == TL_F32) { if (w_dtype == TL_F32) SS(float, float); else SS(float, bf16); }
    else { if (w_dtype == TL_F32) SS(bf16, float); else SS(bf16, bf16); }
#undef SS
    return tl_launch_status();
}

__global__ void softcap_kernel(float* __restrict__ z, size_t n, float cap) {
    grid_dependency_wait();
    grid_dependency_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) z[i] = cap * tanhf(z[i] / cap);
}

TL_EXPORT int tl_softcap(float* z, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return 1;
    launch_after_wait(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, z, (size_t)n, cap);
    return tl_launch_status();
}

template <typename TA>
__global__ void sigmoid_gate_kernel(const TA* __restrict__ o, const float* __restrict__ g, int ldg, TA* __restrict__ y, int N, size_t total) {
    grid_dependency_wait();
    grid_dependency_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / N, c = i - t * N;
    y[i] = from_f<TA>(to_f<TA>(o[i]) / (1.0f + expf(-g[t * ldg + c])));
}

TL_EXPORT int tl_sigmoid_gate(const void* o, const float* g, int ldg, void* y, int T, int N, int act_dtype, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    const size_t total = (size_t)T * N;
    const dim3 grid((unsigned)((total + 255) / 256));
    if (act_dtype == TL_F32) launch_after_wait(sigmoid_gate_kernel<float>, grid, dim3(256), 0, stream, (const float*)o, g, ldg, (float*)y, N, total);
    else launch_after_wait(sigmoid_gate_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)o, g, ldg, (bf16*)y, N, total);
    return tl_launch_status();
}
