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
// the step holds or on how the tokens were cut into steps: the state after a token is the same float either way.
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

__device__ __forceinline__ float rg_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// gates [T, blocks * 2 bw]: per block the r pre-activations then the i pre-activations (without their biases gb, laid out alike);
// u [T, W]; ypre = proj[:, yoff + c] + yb[yoff + c]; state [slots, W].
template <typename TA, int UNROLL>
__global__ void rglru_scan_kernel(const float* __restrict__ gates, const float* __restrict__ gb, const float* __restrict__ u,
                                  const float* __restrict__ proj, int ldp, int yoff, const float* __restrict__ yb,
                                  const float* __restrict__ lam, float* __restrict__ state, const int* __restrict__ q_start,
                                  const int* __restrict__ slots, TA* __restrict__ out, int W, int bw, float sharpness) {
    const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int blk = c / bw, j = c - blk * bw;
    const int gr = blk * 2 * bw + j, gi = gr + bw;
    const float l = lam[c];
    const float coef = -sharpness * (l > 20.f ? l : log1pf(expf(l)));          // softplus, exact where exp would overflow
    const float br = gb[gr], bi = gb[gi], by = yb ? yb[yoff + c] : 0.f;
    grid_dependency_wait();
    grid_dependency_trigger();
    const int first = q_start[b], end = q_start[b + 1];
    if (first >= end) return;
    float* sp = state + (size_t)slots[b] * W + c;
    float S = *sp;
    int t = first;
    for (; t + UNROLL <= end; t += UNROLL) {
        float zr[UNROLL], zi[UNROLL], uv[UNROLL], yv[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {               // every load of the group is in flight before the first is used
            zr[k] = gates[(size_t)(t + k) * 2 * W + gr];
            zi[k] = gates[(size_t)(t + k) * 2 * W + gi];
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
        const float loga = coef * rg_sigmoid(gates[(size_t)t * 2 * W + gr] + br);
        const float a = expf(loga), in = sqrtf(-expm1f(2.0f * loga)) * (rg_sigmoid(gates[(size_t)t * 2 * W + gi] + bi) * u[(size_t)t * W + c]);
        S = fmaf(a, S, in);
        out[(size_t)t * W + c] = from_f<TA>(S * tl_gelu_tanh(proj[(size_t)t * ldp + yoff + c] + by));
    }
    *sp = S;
}

TL_EXPORT int tl_rglru_scan(const float* gates, const float* gb, const float* u, const float* proj, int ldp, int yoff, const float* yb,
                            const float* lam, float* state, const int* q_start, const int* slots, void* out, int act_dtype, int B,
                            int W, int blocks, float sharpness, int max_q_len, cudaStream_t stream) {
    if (B <= 0 || max_q_len <= 0) return 0;
    if (blocks < 1 || W % blocks || B > 65535) return 1;
    // few (request, channel) pairs: small blocks, so that the chains spread over all SMs
    const long long pairs = (long long)B * W;
    const int threads = pairs >= 2LL * 128 * tl_num_sms() ? 128 : pairs >= 2LL * 64 * tl_num_sms() ? 64 : 32;
    const dim3 grid((W + threads - 1) / threads, B);
#define RS(TA, U) launch_after_wait(rglru_scan_kernel<TA, U>, grid, dim3(threads), 0, stream, gates, gb, u, proj, ldp, yoff, yb, lam, state, \
                                    q_start, slots, (TA*)out, W, W / blocks, sharpness)
    if (act_dtype == TL_F32) return max_q_len >= 8 ? RS(float, 8) : RS(float, 1);
    return max_q_len >= 8 ? RS(bf16, 8) : RS(bf16, 1);
#undef RS
}
