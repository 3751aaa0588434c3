// The recurrent block with a real-gated linear recurrent unit: the short causal convolution in front of it and the scan.
//
//   causal_conv   u[t, c] = cb[c] + sum_k w[c, k] * x[t - (taps - 1) + k, c],  x = proj[:, off + c] + xb[c]; positions before
//                 the step come from the request's state slot (its last taps - 1 inputs, zero for a new request), which a
//                 second kernel then brings up to date
//   rglru_scan    per (request, channel), tokens in order:
//                 r = sigmoid(zr + br), i = sigmoid(zi + bi), log a = -sharpness * r * softplus(lam), a = exp(log a)
//                 S <- a S + sqrt(1 - a^2) * i * u;   out = S * gelu_tanh(ypre + yb)
// Every value is float; only `out` is rounded to the activation type.  sqrt(1 - a^2) is taken as sqrt(-expm1(2 log a)),
// which keeps its relative accuracy where a is close to one.  A channel's chain of operations does not depend on what else
// the step holds; steps shorter than two chunks (see below) walk their tokens in order, so that the state after a token is
// the same float however such steps were cut.
#include "common.cuh"

constexpr int CONV_TOKENS = 16;                          // tokens a block of the convolution walks

__global__ void __launch_bounds__(128) causal_conv_kernel(const float* __restrict__ proj, int ldp, int off, const float* __restrict__ xb,
                                                          const float* __restrict__ w, const float* __restrict__ cb, int taps,
                                                          const float* __restrict__ state, size_t slot_stride,
                                                          const int* __restrict__ q_start, const int* __restrict__ slots,
                                                          float* __restrict__ u, int W) {
    const int b = blockIdx.z, c = blockIdx.x * blockDim.x + threadIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    const int first = q_start[b], end = q_start[b + 1];
    const int t0 = first + blockIdx.y * CONV_TOKENS, t1 = min(end, t0 + CONV_TOKENS);
    if (c >= W || t0 >= t1) return;
    const float bias_in = xb ? xb[off + c] : 0.f, bias_out = cb ? cb[c] : 0.f;
    const float* old = taps > 1 ? state + (size_t)slots[b] * slot_stride : nullptr;
    for (int t = t0; t < t1; ++t) {
        float acc = bias_out;
        for (int k = 0; k < taps; ++k) {
            const int j = t - (taps - 1) + k;            // the row of the step this tap reads, or one before the step
            const float x = j >= first ? proj[(size_t)j * ldp + off + c] + bias_in : old[(size_t)(taps - 1 + j - first) * W + c];
            acc = fmaf(w[(size_t)c * taps + k], x, acc);
        }
        u[(size_t)t * W + c] = acc;
    }
}

// the request's last taps - 1 inputs after the step: rows of the step where it has enough, else the old ones moved up
__global__ void __launch_bounds__(128) conv_state_kernel(const float* __restrict__ proj, int ldp, int off, const float* __restrict__ xb,
                                                         int taps, float* __restrict__ state, size_t slot_stride,
                                                         const int* __restrict__ q_start, const int* __restrict__ slots, int W) {
    const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    if (c >= W) return;
    const int first = q_start[b], n = q_start[b + 1] - first;
    if (n <= 0) return;
    float* st = state + (size_t)slots[b] * slot_stride;
    const float bias_in = xb ? xb[off + c] : 0.f;
    for (int j = 0; j < taps - 1; ++j) {                 // new row j is the input n - (taps - 1) + j rows after the step's start
        const int r = n - (taps - 1) + j;
        st[(size_t)j * W + c] = r >= 0 ? proj[(size_t)(first + r) * ldp + off + c] + bias_in : st[(size_t)(j + n) * W + c];
    }
}

TL_EXPORT int tl_causal_conv(const float* proj, int ldp, int off, const float* xb, const float* w, const float* cb, int taps,
                             float* state, long long slot_stride, const int* q_start, const int* slots, float* u, int B,
                             int max_q_len, int W, cudaStream_t stream) {
    if (B <= 0 || max_q_len <= 0) return 0;
    if (taps < 1 || (taps > 1 && !state) || B > 65535) return 1;
    const dim3 grid((W + 127) / 128, (max_q_len + CONV_TOKENS - 1) / CONV_TOKENS, B);
    if (grid.y > 65535) return 1;
    int e = launch_after_wait(causal_conv_kernel, grid, dim3(128), 0, stream, proj, ldp, off, xb, w, cb, taps, (const float*)state,
                              (size_t)slot_stride, q_start, slots, u, W);
    if (e || taps == 1) return e;
    return launch_after_wait(conv_state_kernel, dim3((W + 127) / 128, B), dim3(128), 0, stream, proj, ldp, off, xb, taps, state,
                             (size_t)slot_stride, q_start, slots, W);
}

// A float as three bfloat16 numbers whose sum is the float to within one part in 2^24, so that a product with bfloat16 weights
// on the tensor cores (float accumulators) is as exact as one in float: x [T, W] -> parts [blocks, T, 3, bw], the leading parts
// of a block's bw channels, then the middle ones, then the last.
__global__ void __launch_bounds__(256) split3_kernel(const float* __restrict__ x, bf16* __restrict__ parts, int T, int W, int bw) {
    grid_dependency_wait();
    grid_dependency_trigger();
    const size_t total = (size_t)T * W;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / W), c = (int)(idx - (size_t)t * W);
        const int blk = c / bw, j = c - blk * bw;
        const float v = x[idx];
        const bf16 hi = __float2bfloat16_rn(v);
        const float r1 = v - __bfloat162float(hi);
        const bf16 mid = __float2bfloat16_rn(r1);
        const bf16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
        bf16* p = parts + ((size_t)blk * T + t) * 3 * bw + j;
        p[0] = hi;
        p[bw] = mid;
        p[2 * bw] = lo;
    }
}

// the same, eight channels of one block a thread (bw a multiple of 8, both pointers 16-byte aligned)
__global__ void __launch_bounds__(256) split3_vec_kernel(const float* __restrict__ x, bf16* __restrict__ parts, int T, int W, int bw) {
    grid_dependency_wait();
    grid_dependency_trigger();
    const size_t total = (size_t)T * W / 8;
    const int row = W / 8;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / row), c = (int)(idx - (size_t)t * row) * 8;
        const int blk = c / bw, j = c - blk * bw;
        const float4 a = reinterpret_cast<const float4*>(x)[2 * idx], b = reinterpret_cast<const float4*>(x)[2 * idx + 1];
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint4 out[3];
        bf16* hi = reinterpret_cast<bf16*>(&out[0]);
        bf16* mid = reinterpret_cast<bf16*>(&out[1]);
        bf16* lo = reinterpret_cast<bf16*>(&out[2]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            hi[k] = __float2bfloat16_rn(v[k]);
            const float r1 = v[k] - __bfloat162float(hi[k]);
            mid[k] = __float2bfloat16_rn(r1);
            lo[k] = __float2bfloat16_rn(r1 - __bfloat162float(mid[k]));
        }
        bf16* p = parts + ((size_t)blk * T + t) * 3 * bw + j;
        *reinterpret_cast<uint4*>(p) = out[0];
        *reinterpret_cast<uint4*>(p + bw) = out[1];
        *reinterpret_cast<uint4*>(p + 2 * bw) = out[2];
    }
}

TL_EXPORT int tl_split3(const float* x, void* parts, int T, int W, int blocks, cudaStream_t stream) {
    if (T <= 0 || W <= 0) return 0;
    if (blocks < 1 || W % blocks) return 1;
    const int bw = W / blocks;
    if (bw % 8 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(parts)) & 15) == 0) {
        const size_t vecs = (size_t)T * W / 8;
        const int grid = (int)min((size_t)tl_num_sms() * 8, (vecs + 255) / 256);
        return launch_after_wait(split3_vec_kernel, dim3(grid), dim3(256), 0, stream, x, (bf16*)parts, T, W, bw);
    }
    const size_t total = (size_t)T * W;
    const int grid = (int)min((size_t)tl_num_sms() * 8, (total + 255) / 256);
    return launch_after_wait(split3_kernel, dim3(grid), dim3(256), 0, stream, x, (bf16*)parts, T, W, bw);
}

constexpr int RG_CHUNK = 32;                             // tokens of a chunk of a long step (see rglru_chunk_kernel)

__device__ __forceinline__ float rg_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// gates: token t's pre-activations of block b start at gates[b * gsb + t * gst], the r ones then the i ones, without their biases
// (gb [blocks, 2 bw]); [T, blocks * 2 bw] is gsb = 2 bw, gst = 2 W, and [blocks, T, 2 bw] is gsb = T * 2 bw, gst = 2 bw;
// u [T, W]; ypre = proj[:, yoff + c] + yb[yoff + c]; state [slots, W].
template <typename TA, int UNROLL, bool CHUNKED>
__global__ void rglru_scan_kernel(const float* __restrict__ gates, const float* __restrict__ gb, const float* __restrict__ u,
                                  const float* __restrict__ proj, int ldp, int yoff, const float* __restrict__ yb,
                                  const float* __restrict__ lam, float* __restrict__ state, const int* __restrict__ q_start,
                                  const int* __restrict__ slots, TA* __restrict__ out, int W, int bw, float sharpness,
                                  const float* __restrict__ summary, int chunks, size_t gsb, size_t gst) {
    const int b = CHUNKED ? blockIdx.z : blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int blk = c / bw, j = c - blk * bw;
    const int gr = blk * 2 * bw + j, gi = gr + bw;       // in the biases; a token's pre-activations lie gst floats apart, a block's gsb
    gates += (size_t)blk * gsb + j;
    const float l = lam[c];
    const float coef = -sharpness * (l > 20.f ? l : log1pf(expf(l)));          // softplus, exact where exp would overflow
    const float br = gb[gr], bi = gb[gi], by = yb ? yb[yoff + c] : 0.f;
    grid_dependency_wait();
    grid_dependency_trigger();
    int first = q_start[b], end = q_start[b + 1];
    float* sp = nullptr;
    float S;
    if (CHUNKED) {                                       // this chunk's tokens, from the state the carry kernel left for it
        first += blockIdx.y * RG_CHUNK;
        end = min(end, first + RG_CHUNK);
        if (first >= end) return;
        S = summary[(((size_t)b * chunks + blockIdx.y) * 2 + 1) * W + c];
    } else {
        if (first >= end) return;
        sp = state + (size_t)slots[b] * W + c;
        S = *sp;
    }
    int t = first;
    for (; t + UNROLL <= end; t += UNROLL) {
        float zr[UNROLL], zi[UNROLL], uv[UNROLL], yv[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {               // every load of the group is in flight before the first is used
            zr[k] = gates[(size_t)(t + k) * gst];
            zi[k] = gates[(size_t)(t + k) * gst + bw];
            uv[k] = u[(size_t)(t + k) * W + c];
            yv[k] = proj[(size_t)(t + k) * ldp + yoff + c];
        }
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            const float loga = coef * rg_sigmoid(zr[k] + br);
            const float a = expf(loga), in = sqrtf(-expm1f(2.0f * loga)) * (rg_sigmoid(zi[k] + bi) * uv[k]);
            S = fmaf(a, S, in);
            out[(size_t)(t + k) * W + c] = from_f<TA>(S * tl_gelu_tanh(yv[k] + by));
        }
    }
    for (; t < end; ++t) {
        const float loga = coef * rg_sigmoid(gates[(size_t)t * gst] + br);
        const float a = expf(loga), in = sqrtf(-expm1f(2.0f * loga)) * (rg_sigmoid(gates[(size_t)t * gst + bw] + bi) * u[(size_t)t * W + c]);
        S = fmaf(a, S, in);
        out[(size_t)t * W + c] = from_f<TA>(S * tl_gelu_tanh(proj[(size_t)t * ldp + yoff + c] + by));
    }
    if (!CHUNKED) *sp = S;
}


// Long steps are cut into chunks of RG_CHUNK tokens that run side by side, since the recurrence is linear in S:
//   rglru_chunk_kernel   per (request, chunk, channel): the product P of the chunk's decays and the state L the chunk reaches
//                        from zero, into summary[b][chunk][0 | 1][c]
//   rglru_carry_kernel   per (request, channel), chunks in order from the slot's state: the state a chunk starts from takes
//                        L's place in the summary, S <- P S + L, and the last S goes back to the slot
//   rglru_scan_kernel    with CHUNKED: every chunk walks its tokens from the state it starts from, as a short step would
// Within a chunk the chain of operations is that of the unchunked kernel; only the state a chunk starts from is summed
// in another order, which differs from the token-by-token value by roundings of float.

__global__ void __launch_bounds__(128) rglru_chunk_kernel(const float* __restrict__ gates, const float* __restrict__ gb,
                                                          const float* __restrict__ u, const float* __restrict__ lam,
                                                          const int* __restrict__ q_start, float* __restrict__ summary, int chunks,
                                                          int W, int bw, float sharpness, size_t gsb, size_t gst) {
    const int b = blockIdx.z, k = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int blk = c / bw, j = c - blk * bw;
    const int gr = blk * 2 * bw + j, gi = gr + bw;       // in the biases; a token's pre-activations lie gst floats apart, a block's gsb
    gates += (size_t)blk * gsb + j;
    const float l = lam[c];
    const float coef = -sharpness * (l > 20.f ? l : log1pf(expf(l)));
    const float br = gb[gr], bi = gb[gi];
    grid_dependency_wait();
    grid_dependency_trigger();
    const int first = q_start[b], end = q_start[b + 1];
    const int t0 = first + k * RG_CHUNK, t1 = min(end, t0 + RG_CHUNK);
    if (t0 >= t1) return;
    float P = 1.f, S = 0.f;
    int t = t0;
    for (; t + 8 <= t1; t += 8) {
        float zr[8], zi[8], uv[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            zr[q] = gates[(size_t)(t + q) * gst];
            zi[q] = gates[(size_t)(t + q) * gst + bw];
            uv[q] = u[(size_t)(t + q) * W + c];
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float loga = coef * rg_sigmoid(zr[q] + br);
            const float a = expf(loga), in = sqrtf(-expm1f(2.0f * loga)) * (rg_sigmoid(zi[q] + bi) * uv[q]);
            S = fmaf(a, S, in);
            P *= a;
        }
    }
    for (; t < t1; ++t) {
        const float loga = coef * rg_sigmoid(gates[(size_t)t * gst] + br);
        const float a = expf(loga), in = sqrtf(-expm1f(2.0f * loga)) * (rg_sigmoid(gates[(size_t)t * gst + bw] + bi) * u[(size_t)t * W + c]);
        S = fmaf(a, S, in);
        P *= a;
    }
    float* sm = summary + ((size_t)b * chunks + k) * 2 * W;
    sm[c] = P;
    sm[W + c] = S;
}

__global__ void __launch_bounds__(128) rglru_carry_kernel(float* __restrict__ summary, int chunks, float* __restrict__ state,
                                                          const int* __restrict__ q_start, const int* __restrict__ slots, int W) {
    const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    if (c >= W) return;
    const int n = q_start[b + 1] - q_start[b];
    if (n <= 0) return;
    const int used = (n + RG_CHUNK - 1) / RG_CHUNK;
    float* sp = state + (size_t)slots[b] * W + c;
    float* sm = summary + (size_t)b * chunks * 2 * W + c;
    float S = *sp;
    int k = 0;
    for (; k + 8 <= used; k += 8) {
        float P[8], L[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            P[q] = sm[(size_t)(k + q) * 2 * W];
            L[q] = sm[(size_t)(k + q) * 2 * W + W];
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            sm[(size_t)(k + q) * 2 * W + W] = S;
            S = fmaf(P[q], S, L[q]);
        }
    }
    for (; k < used; ++k) {
        const float P = sm[(size_t)k * 2 * W], L = sm[(size_t)k * 2 * W + W];
        sm[(size_t)k * 2 * W + W] = S;
        S = fmaf(P, S, L);
    }
    *sp = S;
}

TL_EXPORT int tl_rglru_chunk() { return RG_CHUNK; }

// summary: float [B, chunks, 2, W] with chunks >= ceil(max_q_len / RG_CHUNK) for the chunked form, or null: tokens in order.
TL_EXPORT int tl_rglru_scan(const float* gates, const float* gb, const float* u, const float* proj, int ldp, int yoff, const float* yb,
                            const float* lam, float* state, const int* q_start, const int* slots, void* out, int act_dtype, int B,
                            int W, int blocks, float sharpness, int max_q_len, float* summary, int chunks, long long gate_block_stride,
                            long long gate_token_stride, cudaStream_t stream) {
    if (B <= 0 || max_q_len <= 0) return 0;
    const size_t gsb = (size_t)gate_block_stride, gst = (size_t)gate_token_stride;
    if (blocks < 1 || W % blocks || B > 65535) return 1;
    if (summary) {
        if (chunks < (max_q_len + RG_CHUNK - 1) / RG_CHUNK || chunks > 65535) return 1;
        const dim3 grid((W + 127) / 128, chunks, B);
        int e = launch_after_wait(rglru_chunk_kernel, grid, dim3(128), 0, stream, gates, gb, u, lam, q_start, summary, chunks, W,
                                  W / blocks, sharpness, gsb, gst);
        if (e) return e;
        e = launch_after_wait(rglru_carry_kernel, dim3((W + 127) / 128, B), dim3(128), 0, stream, summary, chunks, state, q_start, slots, W);
        if (e) return e;
#define RC(TA) launch_after_wait(rglru_scan_kernel<TA, 8, true>, grid, dim3(128), 0, stream, gates, gb, u, proj, ldp, yoff, yb, lam, state, \
                                 q_start, slots, (TA*)out, W, W / blocks, sharpness, (const float*)summary, chunks, gsb, gst)
        return act_dtype == TL_F32 ? RC(float) : RC(bf16);
#undef RC
    }
    // few (request, channel) pairs: small blocks, so that the chains spread over all SMs
    const long long pairs = (long long)B * W;
    const int threads = pairs >= 2LL * 128 * tl_num_sms() ? 128 : pairs >= 2LL * 64 * tl_num_sms() ? 64 : 32;
    const dim3 grid((W + threads - 1) / threads, B);
#define RS(TA, U) launch_after_wait(rglru_scan_kernel<TA, U, false>, grid, dim3(threads), 0, stream, gates, gb, u, proj, ldp, yoff, yb, lam, \
                                    state, q_start, slots, (TA*)out, W, W / blocks, sharpness, (const float*)nullptr, 0, gsb, gst)
    if (act_dtype == TL_F32) return max_q_len >= 8 ? RS(float, 8) : RS(float, 1);
    return max_q_len >= 8 ? RS(bf16, 8) : RS(bf16, 1);
#undef RS
}
