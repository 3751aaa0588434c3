// Routed feed-forward (mixture of experts): router, choice of experts, and the experts' two products.
//
//   z = h Wr^T + br                         float, whatever the engine's activation type (small_proj)
//   chosen = the `top` largest z, lowest index first on a tie; weights = softmax over the chosen z only
//   y = sum_j weight_j * Wdown[e_j] act(Wup[e_j] h),   act(u) = relu(u)^2
// Options, all arguments: the weights as the sigmoid of each chosen logit instead of the softmax over the chosen
// (`mode`); gated experts, Wdown (act(Wgate x) * Wup x) with gate and up rows stacked [2F, K] (`gated`, `act`); the weight
// on the expert's input instead of its output, x = weight * h (`in_scale`; the output sum is then unweighted); and one
// more addend a token, gate_t * extra[t] with gate_t = sigmoid of a column of the router's product (a shared expert).
//
// Two routes for the experts' products.  Steps of few tokens (decoding): every (token, chosen expert) pair streams its
// expert's rows (moe_up), and every token sums its experts' down products in the order they were chosen (moe_down):
// one pass over the weights the step needs, no sorting, nothing on the host, so the step can sit in a CUDA graph.
// Steps of many tokens: the pairs are sorted by expert on the device (moe_sort), the tokens' rows gathered in that
// order (every expert's run in a buffer of `cap` rows of its own, so that one batched product serves all experts), two
// dense products run on them, and moe_combine sums each token's rows by weight.
// Every output element is one fixed chain of additions, so a token's result does not depend on the step's other tokens.
#include "common.cuh"

// dot product of a weight row with a float vector in shared memory, lanes striding; every lane gets the sum
template <typename TW> __device__ __forceinline__ float warp_dot(const TW* __restrict__ w, const float* __restrict__ x, int K, int lane);
template <> __device__ __forceinline__ float warp_dot<float>(const float* __restrict__ w, const float* __restrict__ x, int K, int lane) {
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(w[k], x[k], acc);
    return warp_sum(acc);
}
template <> __device__ __forceinline__ float warp_dot<bf16>(const bf16* __restrict__ w, const float* __restrict__ x, int K, int lane) {
    float acc = 0.f;
    if ((K & 7) == 0 && (((uintptr_t)w) & 15) == 0) {
        for (int k = lane * 8; k < K; k += 256) {
            const uint4 v = *reinterpret_cast<const uint4*>(w + k);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc = fmaf(__low2float(p[e]), x[k + 2 * e], acc);
                acc = fmaf(__high2float(p[e]), x[k + 2 * e + 1], acc);
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(__bfloat162float(w[k]), x[k], acc);
    }
    return warp_sum(acc);
}

// Four rows (`rows` of them real, a row `ld` elements after the other) against the same vector: the loads of all four are
// issued before the first product, so a warp keeps four times as many bytes in flight.  A row's sum is the chain of
// warp_dot, whichever rows share the call.
template <typename TW> __device__ __forceinline__ void warp_dot4(const TW* __restrict__ w, int ld, int rows, const float* __restrict__ x,
                                                                 int K, int lane, float (&out)[4]);
template <> __device__ __forceinline__ void warp_dot4<float>(const float* __restrict__ w, int ld, int rows, const float* __restrict__ x,
                                                             int K, int lane, float (&out)[4]) {
#pragma unroll
    for (int r = 0; r < 4; ++r) out[r] = r < rows ? warp_dot<float>(w + (size_t)r * ld, x, K, lane) : 0.f;
}
template <> __device__ __forceinline__ void warp_dot4<bf16>(const bf16* __restrict__ w, int ld, int rows, const float* __restrict__ x,
                                                            int K, int lane, float (&out)[4]) {
    if ((K & 7) || (ld & 7) || (((uintptr_t)w) & 15)) {
#pragma unroll
        for (int r = 0; r < 4; ++r) out[r] = r < rows ? warp_dot<bf16>(w + (size_t)r * ld, x, K, lane) : 0.f;
        return;
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int k = lane * 8; k < K; k += 256) {
        uint4 v[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) v[r] = r < rows ? *reinterpret_cast<const uint4*>(w + (size_t)r * ld + k) : make_uint4(0, 0, 0, 0);
        const float4 x0 = *reinterpret_cast<const float4*>(x + k), x1 = *reinterpret_cast<const float4*>(x + k + 4);
        const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[r]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[r] = fmaf(__low2float(p[e]), xv[2 * e], acc[r]);
                acc[r] = fmaf(__high2float(p[e]), xv[2 * e + 1], acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) out[r] = warp_sum(acc[r]);
}

// ------------------------------------------------------------------ small projection in float
// out[t, n] = bias[n] + sum_k h[t, k] w[n, k]: for outputs that must be 32-bit whatever the engine (router logits,
// gate pre-activations of a recurrence).  One block per token; the token's row sits in shared memory as float.
template <typename TA, typename TW>
__global__ void __launch_bounds__(128) small_proj_kernel(const TA* __restrict__ h, int ldh, const TW* __restrict__ w,
                                                         const TW* __restrict__ bias, float* __restrict__ out, int ldo, int N, int K) {
    extern __shared__ __align__(16) float xs[];
    const int t = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    grid_dependency_wait();                              // launched as a dependent: nothing of another kernel is touched before this
    grid_dependency_trigger();
    for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_f<TA>(h[(size_t)t * ldh + k]);
    __syncthreads();
    for (int n = (blockIdx.y * 4 + wid) * 4; n < N; n += gridDim.y * 16) {      // four outputs a warp, their loads in flight together
        float v[4];
        const int rows = min(4, N - n);
        warp_dot4<TW>(w + (size_t)n * K, K, rows, xs, K, lane, v);
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (lane == 0 && r < rows) out[(size_t)t * ldo + n + r] = v[r] + (bias ? to_f<TW>(bias[n + r]) : 0.f);
    }
}

TL_EXPORT int tl_small_proj(const void* h, int act_dtype, int ldh, const void* w, const void* bias, int w_dtype, float* out,
                            int ldo, int T, int N, int K, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    const size_t smem = (size_t)K * sizeof(float);
    if (smem > 48 * 1024) return 1;
    // few tokens: the outputs of a token are dealt out to several blocks, so that a step of one token still fills SMs
    const dim3 grid(T, T >= 512 ? 1 : min((N + 15) / 16, 64));
#define SP(TA, TW) launch_after_wait(small_proj_kernel<TA, TW>, grid, dim3(128), smem, stream, (const TA*)h, ldh, (const TW*)w, (const TW*)bias, out, ldo, N, K)
    if (act_dtype == TL_F32) { if (w_dtype == TL_F32) SP(float, float); else SP(float, bf16); }
    else { if (w_dtype == TL_F32) SP(bf16, float); else SP(bf16, bf16); }
#undef SP
    return tl_launch_status();
}

// ------------------------------------------------------------------ choice of experts
// One warp per token.  `top` rounds of a warp-wide arg-max (largest value, lowest index on a tie); the weights are
// the softmax over the chosen logits.  E <= 1024, top <= 32.
__global__ void __launch_bounds__(128) topk_softmax_kernel(const float* __restrict__ z, int ldz, int E, int top, int* __restrict__ idx,
                                                           float* __restrict__ wts, int T, int mode) {
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    grid_dependency_wait();                              // launched as a dependent: nothing of another kernel is touched before this
    grid_dependency_trigger();
    if (t >= T) return;
    const float* row = z + (size_t)t * ldz;
    unsigned taken = 0;                                  // bit c: my element lane + 32 c is chosen
    float mine = 0.f, first = 0.f, sum = 0.f;            // lane j keeps the j-th chosen logit
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY; int bi = 0x7fffffff;
        for (int c = 0, e = lane; e < E; ++c, e += 32) {
            const float v = row[e];
            if (!((taken >> c) & 1u) && (v > best || (v == best && e < bi) || bi == 0x7fffffff)) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
        }
        if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
        if (j == 0) first = best;
        const float p = mode ? 1.0f / (1.0f + expf(-best)) : expf(best - first);
        sum += p;
        if (lane == j) mine = p;
        if (lane == 0) idx[(size_t)t * top + j] = bi;
    }
    if (lane < top) wts[(size_t)t * top + lane] = mode ? mine : mine / sum;
}

TL_EXPORT int tl_topk_softmax(const float* z, int ldz, int E, int top, int* idx, float* wts, int T, int mode, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E > 1024 || top > 32 || top > E || top < 1) return 1;
    launch_after_wait(topk_softmax_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, z, ldz, E, top, idx, wts, T, mode);
    return tl_launch_status();
}

// ------------------------------------------------------------------ choice of experts among groups
// One warp per token.  s = sigmoid(z); the choice scores are c = s + correction.  The experts form `groups` equal groups
// of neighbours; a group's score is the sum of its `gtop` largest c; the `keep` groups with the largest scores stay, the
// experts of the others cannot be chosen (their c may be anything, also negative).  `top` rounds of a warp-wide arg-max
// over c among the experts that stay (largest value, lowest index on a tie); the weights are the chosen experts' s divided
// by their sum (+ 1e-20), times `scale`.  E <= 1024, top <= 32.  Shared memory: c [E], s [E], the groups' scores [groups].
__global__ void __launch_bounds__(32) route_groups_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ correction,
                                                          int E, int top, int groups, int keep, int gtop, float scale,
                                                          int* __restrict__ idx, float* __restrict__ wts, int softmax) {
    extern __shared__ float sm[];
    float* c = sm;
    float* s = sm + E;
    float* gs = sm + 2 * E;
    const int t = blockIdx.x, lane = threadIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    const float* row = z + (size_t)t * ldz;
    float top_z = -INFINITY, total = 0.f;                // softmax: the scores are the shares of all entries' exponentials
    if (softmax) {
        for (int e = lane; e < E; e += 32) top_z = fmaxf(top_z, row[e]);
        top_z = warp_max(top_z);
        for (int e = lane; e < E; e += 32) total += expf(row[e] - top_z);
        total = warp_sum(total);
    }
    for (int e = lane; e < E; e += 32) {
        const float sv = softmax ? expf(row[e] - top_z) / total : 1.0f / (1.0f + expf(-row[e]));
        s[e] = sv;
        c[e] = sv + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    const int per = E / groups;
    // a group's score: the sum of its gtop largest choice scores (all of them, if it has fewer), taken largest first
    // (every group kept: nothing to judge, all of them are marked as kept right away)
    if (keep == groups) {
        for (int g = lane; g < groups; g += 32) gs[g] = INFINITY;
        __syncwarp();
    } else
    for (int g = lane; g < groups; g += 32) {
        const float* cg = c + g * per;
        float sum = 0.f, last = INFINITY; int last_i = -1;
        for (int r = 0; r < gtop && r < per; ++r) {
            float best = -INFINITY; int bi = -1;
            for (int i = 0; i < per; ++i) {
                const float v = cg[i];
                const bool below = v < last || (v == last && i > last_i);      // not one of those already taken
                if (below && (bi < 0 || v > best)) { best = v; bi = i; }
            }
            sum += best; last = best; last_i = bi;
        }
        gs[g] = sum;
    }
    __syncwarp();
    // the groups that stay: `keep` rounds of an arg-max over the groups' scores (lowest index on a tie); a group that was
    // picked is marked by a score of +inf, which no sum of sigmoids and corrections reaches
    for (int r = 0; r < (keep == groups ? 0 : keep); ++r) {
        float best = -INFINITY; int bi = 0x7fffffff;
        for (int g = lane; g < groups; g += 32) {
            const float v = gs[g];
            if (v != INFINITY && (bi == 0x7fffffff || v > best)) { best = v; bi = g; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
        }
        if (lane == 0 && bi != 0x7fffffff) gs[bi] = INFINITY;
        __syncwarp();
    }
    unsigned taken = 0;                                  // bit k: my element lane + 32 k is chosen
    float mine = 0.f, sum = 0.f;                         // lane j keeps the j-th chosen expert's s
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY; int bi = 0x7fffffff;
        for (int k = 0, e = lane; e < E; ++k, e += 32) {
            if (((taken >> k) & 1u) || gs[e / per] != INFINITY) continue;
            const float v = c[e];
            if (bi == 0x7fffffff || v > best) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;                    // fewer experts stay than `top` asks for (the launcher refuses that)
        if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
        const float p = s[bi];
        sum += p;
        if (lane == j) mine = p;
        if (lane == 0) idx[(size_t)t * top + j] = bi;
    }
    if (lane < top) wts[(size_t)t * top + lane] = mine / (sum + 1e-20f) * scale;
}

TL_EXPORT int tl_route_groups(const float* z, int ldz, const float* correction, int E, int top, int groups, int keep, int gtop, int softmax,
                              float scale, int* idx, float* wts, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E > 1024 || top > 32 || top < 1 || groups < 1 || E % groups || keep < 1 || keep > groups || gtop < 1 ||
        top > keep * (E / groups)) return 1;
    const size_t smem = ((size_t)2 * E + groups) * sizeof(float);
    launch_after_wait(route_groups_kernel, dim3(T), dim3(32), smem, stream, z, ldz, correction, E, top, groups, keep, gtop, scale, idx, wts, softmax);
    return tl_launch_status();
}

// ------------------------------------------------------------------ experts, few tokens
constexpr int MOE_ROWS = 16;                             // output rows a block of moe_up (4 a warp, their loads in flight together)
constexpr int MOE_DOWN_ROWS = 4;                         // output rows a block of moe_down (a warp an expert)

// a[pair, f] = act(s Wup[e][f, :] . h[t, :]), pair = t * top + j, e = idx[pair], s = in_scale ? in_scale[pair] : 1;
// gated: a[pair, f] = act(s Wgu[e][f, :] . h[t, :]) * (s Wgu[e][F + f, :] . h[t, :]) with an expert's matrix [2F, K].
template <typename TA, typename TW>
__global__ void __launch_bounds__(128) moe_up_kernel(const TA* __restrict__ h, const TW* __restrict__ w_up, const int* __restrict__ idx,
                                                     TA* __restrict__ a, int K, int F, int top, int gated, int act,
                                                     const float* __restrict__ in_scale, float limit, float alpha, int n_real) {
    extern __shared__ __align__(16) float xs[];
    const int pair = blockIdx.x, t = pair / top, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    grid_dependency_wait();                              // launched as a dependent: nothing of another kernel is touched before this
    grid_dependency_trigger();
    const int e = idx[pair];
    if (e >= n_real) return;                             // an identity entry: its output is the token's row itself (moe_down)
    for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_f<TA>(h[(size_t)t * K + k]);
    __syncthreads();
    const TW* w = w_up + (size_t)e * F * K * (gated ? 2 : 1);
    const float sc = in_scale ? in_scale[pair] : 1.0f;
    const int f0 = blockIdx.y * MOE_ROWS + wid * (MOE_ROWS / 4), f1 = min(F, f0 + MOE_ROWS / 4);    // a warp's four rows
    for (int f = f0; f < f1; f += 4) {                   // four rows at a time: their loads are in flight together
        float u[4], g[4];
        warp_dot4<TW>(w + (size_t)f * K, K, min(4, f1 - f), xs, K, lane, u);
        if (gated) {
#pragma unroll
            for (int r = 0; r < 4; ++r) g[r] = u[r];
            warp_dot4<TW>(w + (size_t)(F + f) * K, K, min(4, f1 - f), xs, K, lane, u);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (lane == 0 && f + r < f1)
                a[(size_t)pair * F + f + r] = from_f<TA>(gated ? tl_act_pair(sc * g[r], sc * u[r], act, limit, alpha) : tl_act(sc * u[r], act));
    }
}

// y[t, n] = sum_j wts[t, j] * (Wdown[e_j][n, :] . a[t * top + j, :]), j in the order chosen.  A block has four rows n of one
// token; its warps take the chosen experts in turn (warp w: j = w, w + 4, ...), each with its expert's inner row in shared
// memory of its own, and leave their four products in red[j]; then one thread a row adds them up in the order chosen.
template <typename TA, typename TW>
__global__ void __launch_bounds__(128) moe_down_kernel(const TA* __restrict__ a, const TW* __restrict__ w_down, const int* __restrict__ idx,
                                                       const float* __restrict__ wts, TA* __restrict__ y, int F, int N, int top,
                                                       const TA* __restrict__ extra, const float* __restrict__ extra_gate, int ldg,
                                                       int n_real, const TA* __restrict__ same) {
    extern __shared__ __align__(16) float xs[];          // [4 warps][F], then red [top][4]
    float* red = xs + 4 * (size_t)F;
    const int t = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int n0 = blockIdx.y * MOE_DOWN_ROWS, rows = min(MOE_DOWN_ROWS, N - n0);
    float* mine = xs + (size_t)wid * F;
    grid_dependency_wait();                              // launched as a dependent: nothing of another kernel is touched before this
    grid_dependency_trigger();
    for (int j = wid; j < top; j += 4) {
        const int e = idx[(size_t)t * top + j];
        if (e >= n_real) {                               // an identity entry: the token's own row (`same` [T, N]) stands for the product
            if (lane < 4) red[j * 4 + lane] = lane < rows ? to_f<TA>(same[(size_t)t * N + n0 + lane]) : 0.f;
            continue;
        }
        __syncwarp();
        for (int k = lane; k < F; k += 32) mine[k] = to_f<TA>(a[((size_t)t * top + j) * F + k]);
        __syncwarp();
        float v[4];
        warp_dot4<TW>(w_down + ((size_t)e * N + n0) * F, F, rows, mine, F, lane, v);
        const float mv = lane == 0 ? v[0] : lane == 1 ? v[1] : lane == 2 ? v[2] : v[3];
        if (lane < 4) red[j * 4 + lane] = mv;
    }
    __syncthreads();
    if (threadIdx.x < rows) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j) acc = wts ? fmaf(wts[(size_t)t * top + j], red[j * 4 + threadIdx.x], acc) : acc + red[j * 4 + threadIdx.x];
        if (extra) {
            const float gt = extra_gate ? 1.0f / (1.0f + expf(-extra_gate[(size_t)t * ldg])) : 1.0f;
            acc = fmaf(gt, to_f<TA>(extra[(size_t)t * N + n0 + threadIdx.x]), acc);
        }
        y[(size_t)t * N + n0 + threadIdx.x] = from_f<TA>(acc);
    }
}

TL_EXPORT int tl_moe_up(const void* h, int act_dtype, const void* w_up, int w_dtype, const int* idx, void* a, int P, int K,
                        int F, int top, int gated, int act, const float* in_scale, float limit, float alpha, int n_real,
                        cudaStream_t stream) {
    if (P <= 0) return 0;
    if (act == TL_ACT_SWISH_CLAMPED && !gated) return 1;
    const size_t smem = (size_t)K * sizeof(float);
    if (smem > 48 * 1024) return 1;
    const dim3 grid(P, (F + MOE_ROWS - 1) / MOE_ROWS);
    if (grid.y > 65535) return 1;
#define MU(TA, TW) launch_after_wait(moe_up_kernel<TA, TW>, grid, dim3(128), smem, stream, (const TA*)h, (const TW*)w_up, idx, (TA*)a, K, F, top, gated, act, in_scale, limit, alpha, n_real)
    if (act_dtype == TL_F32) { if (w_dtype == TL_F32) MU(float, float); else MU(float, bf16); }
    else { if (w_dtype == TL_F32) MU(bf16, float); else MU(bf16, bf16); }
#undef MU
    return tl_launch_status();
}

TL_EXPORT int tl_moe_down(const void* a, int act_dtype, const void* w_down, int w_dtype, const int* idx, const float* wts,
                          void* y, int T, int F, int N, int top, const void* extra, const float* extra_gate, int ldg,
                          int n_real, const void* same, cudaStream_t stream) {
    if (T <= 0) return 0;
    const size_t smem = ((size_t)4 * F + (size_t)top * 4) * sizeof(float);
    if (smem > 48 * 1024) return 1;
    const dim3 grid(T, (N + MOE_DOWN_ROWS - 1) / MOE_DOWN_ROWS);
    if (grid.y > 65535) return 1;
#define MD(TA, TW) launch_after_wait(moe_down_kernel<TA, TW>, grid, dim3(128), smem, stream, (const TA*)a, (const TW*)w_down, idx, wts, (TA*)y, F, N, top, (const TA*)extra, extra_gate, ldg, n_real, (const TA*)same)
    if (act_dtype == TL_F32) { if (w_dtype == TL_F32) MD(float, float); else MD(float, bf16); }
    else { if (w_dtype == TL_F32) MD(bf16, float); else MD(bf16, bf16); }
#undef MD
    return tl_launch_status();
}

// ------------------------------------------------------------------ experts, many tokens
// Counting sort of the P = T * top pairs by expert, one block: offsets[e] .. offsets[e + 1] is expert e's run of
// sorted places; place_of[pair] is where the pair went, pair_at[place] the pair there.  The order inside a run is
// the order of the pairs (a thread takes a contiguous range of pairs and the ranges are placed in thread order), so
// the same step sorts the same way every time.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ idx, int P, int E, int* __restrict__ offsets,
                                                        int* __restrict__ place_of, int* __restrict__ pair_at) {
    extern __shared__ int cnt[];                         // [E][blockDim.x + 1] would be too much: counts per (expert, warp)
    const int nw = blockDim.x >> 5, wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int* base = cnt + E * nw;                            // [E + 1]
    for (int i = threadIdx.x; i < E * nw; i += blockDim.x) cnt[i] = 0;
    __syncthreads();
    const int per = (P + nw - 1) / nw, lo = wid * per, hi = min(P, lo + per);      // a warp's contiguous range of pairs
    for (int p = lo + lane; p < hi; p += 32) atomicAdd(&cnt[idx[p] * nw + wid], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            base[e] = run;
            for (int w = 0; w < nw; ++w) { const int c = cnt[e * nw + w]; cnt[e * nw + w] = run; run += c; }
        }
        base[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = base[e];
    // inside a warp's range: pairs in order, 32 at a time, ranked by a ballot per expert value
    for (int p0 = lo; p0 < hi; p0 += 32) {
        const int p = p0 + lane;
        const int e = p < hi ? idx[p] : -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(same & ((1u << lane) - 1u));
        int start = 0;
        if (e >= 0) start = cnt[e * nw + wid];
        __syncwarp();
        if (e >= 0) {
            const int place = start + rank;
            place_of[p] = place;
            pair_at[place] = p;
            if (rank == __popc(same) - 1) cnt[e * nw + wid] = start + rank + 1;
        }
        __syncwarp();
    }
}

TL_EXPORT int tl_moe_sort(const int* idx, int P, int E, int* offsets, int* place_of, int* pair_at, cudaStream_t stream) {
    if (P <= 0) return 0;
    const size_t smem = ((size_t)E * 32 + E + 1) * sizeof(int);
    if (smem > 48 * 1024) return 1;
    moe_sort_kernel<<<1, 1024, smem, stream>>>(idx, P, E, offsets, place_of, pair_at);
    return tl_launch_status();
}

// Where a sorted place lies in the experts' row buffer.  cap = 0: the runs lie one behind the other (row = place);
// cap > 0: every expert has `cap` rows of its own (row = expert * cap + place - offsets[expert]), so that one batched
// product serves all experts; rows beyond an expert's run stay as the caller filled them.
__device__ __forceinline__ size_t moe_row(int place, int expert, const int* __restrict__ offsets, int cap) {
    return cap ? (size_t)expert * cap + (place - offsets[expert]) : (size_t)place;
}

// rows[row of place, :] = h[pair_at[place] / top, :].  cap = 0: a block a sorted place.  cap > 0: a block a row of the
// experts' buffer, (expert, r): the r-th place of the expert's run, or zeros behind the run's end.
template <typename TA>
__global__ void moe_gather_kernel(const TA* __restrict__ h, const int* __restrict__ pair_at, const int* __restrict__ offsets, int cap,
                                  TA* __restrict__ rows, int K, int top, const float* __restrict__ scale) {
    int place = blockIdx.x;
    if (cap) {
        const int e = blockIdx.x / cap, r = blockIdx.x - e * cap;
        place = offsets[e] + r < offsets[e + 1] ? offsets[e] + r : -1;
    }
    TA* dst = rows + (size_t)blockIdx.x * K;
    const TA* src = place >= 0 ? h + (size_t)(pair_at[place] / top) * K : nullptr;
    if (scale && src) {                                  // rows = scale[pair] * h: the weight on the expert's input
        const float sc = scale[pair_at[place]];
        for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = from_f<TA>(sc * to_f<TA>(src[k]));
        return;
    }
    const bool wide = ((size_t)K * sizeof(TA)) % 16 == 0 && ((((uintptr_t)h) | ((uintptr_t)rows)) & 15) == 0;
    if (wide) {
        const int n16 = (int)((size_t)K * sizeof(TA) / 16);
        for (int k = threadIdx.x; k < n16; k += blockDim.x)
            reinterpret_cast<uint4*>(dst)[k] = src ? reinterpret_cast<const uint4*>(src)[k] : make_uint4(0, 0, 0, 0);
    } else {
        for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = src ? src[k] : from_f<TA>(0.f);
    }
}

TL_EXPORT int tl_moe_gather(const void* h, int act_dtype, const int* pair_at, const int* idx, const int* offsets, int cap,
                            void* rows, int P, int E, int K, int top, const float* scale, cudaStream_t stream) {
    (void)idx;
    const long long blocks = cap ? (long long)E * cap : P;
    if (blocks <= 0) return 0;
    if (blocks > 2147483647LL) return 1;
    if (act_dtype == TL_F32) moe_gather_kernel<float><<<(unsigned)blocks, 128, 0, stream>>>((const float*)h, pair_at, offsets, cap, (float*)rows, K, top, scale);
    else moe_gather_kernel<bf16><<<(unsigned)blocks, 128, 0, stream>>>((const bf16*)h, pair_at, offsets, cap, (bf16*)rows, K, top, scale);
    return tl_launch_status();
}

// u = relu(u)^2 in place
template <typename TA>
__global__ void relu_square_kernel(TA* __restrict__ u, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f<TA>(u[i]), 0.f);
        u[i] = from_f<TA>(v * v);
    }
}
// bfloat16, eight values (16 bytes) a thread and step; n8 = n / 8
__global__ void relu_square_vec8_kernel(uint4* __restrict__ u, size_t n8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        uint4 v = u[i];
        __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float a = fmaxf(__low2float(p[e]), 0.f), b = fmaxf(__high2float(p[e]), 0.f);
            p[e] = __floats2bfloat162_rn(a * a, b * b);
        }
        u[i] = v;
    }
}

TL_EXPORT int tl_relu_square(void* u, int act_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (act_dtype == TL_BF16 && n % 8 == 0 && (((uintptr_t)u) & 15) == 0) {
        const long long n8 = n / 8;
        const int vblocks = (int)((n8 + 255) / 256 < (long long)tl_num_sms() * 32 ? (n8 + 255) / 256 : (long long)tl_num_sms() * 32);
        relu_square_vec8_kernel<<<vblocks, 256, 0, stream>>>((uint4*)u, (size_t)n8);
        return tl_launch_status();
    }
    const int blocks = (int)((n + 255) / 256 < (long long)tl_num_sms() * 16 ? (n + 255) / 256 : (long long)tl_num_sms() * 16);
    if (act_dtype == TL_F32) relu_square_kernel<float><<<blocks, 256, 0, stream>>>((float*)u, (size_t)n);
    else relu_square_kernel<bf16><<<blocks, 256, 0, stream>>>((bf16*)u, (size_t)n);
    return tl_launch_status();
}

// y[t, :] = sum_j wts[t, j] * rows[row of place_of[t * top + j], :], j in the order chosen
template <typename TA>
__global__ void moe_combine_kernel(const TA* __restrict__ rows, const int* __restrict__ place_of, const int* __restrict__ idx,
                                   const int* __restrict__ offsets, int cap, const float* __restrict__ wts,
                                   TA* __restrict__ y, int N, int top, const TA* __restrict__ extra,
                                   const float* __restrict__ extra_gate, int ldg) {
    const int t = blockIdx.x;
    const float gt = !extra ? 0.f : extra_gate ? 1.0f / (1.0f + expf(-extra_gate[(size_t)t * ldg])) : 1.0f;
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j) {
            const size_t pair = (size_t)t * top + j;
            const float v = to_f<TA>(rows[moe_row(place_of[pair], idx[pair], offsets, cap) * N + n]);
            acc = wts ? fmaf(wts[pair], v, acc) : acc + v;
        }
        if (extra) acc = fmaf(gt, to_f<TA>(extra[(size_t)t * N + n]), acc);
        y[(size_t)t * N + n] = from_f<TA>(acc);
    }
}

TL_EXPORT int tl_moe_combine(const void* rows, int act_dtype, const int* place_of, const int* idx, const int* offsets, int cap,
                             const float* wts, void* y, int T, int N, int top, const void* extra, const float* extra_gate, int ldg,
                             cudaStream_t stream) {
    if (T <= 0) return 0;
    if (act_dtype == TL_F32) moe_combine_kernel<float><<<T, 256, 0, stream>>>((const float*)rows, place_of, idx, offsets, cap, wts, (float*)y, N, top, (const float*)extra, extra_gate, ldg);
    else moe_combine_kernel<bf16><<<T, 256, 0, stream>>>((const bf16*)rows, place_of, idx, offsets, cap, wts, (bf16*)y, N, top, (const bf16*)extra, extra_gate, ldg);
    return tl_launch_status();
}
