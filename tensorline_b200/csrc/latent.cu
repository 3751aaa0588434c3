// Attention through a latent: what a token leaves in the cache is one vector c (the normalised down-projection, `rank`
// numbers) and one rotated key part r (`dr` numbers) shared by all heads; a head's key is Wuk_h c and its value Wuv_h c.
// The scores and outputs are computed in the latent's own space, which is the same sums in another order:
//     q_h . (Wuk_h c) = (Wuk_h^T q_h) . c,          sum_j p_j Wuv_h c_j = Wuv_h (sum_j p_j c_j)
// so the cache is read by the ordinary paged attention kernels as ONE key/value head of size rank + dr whose value is the
// key itself (the output's first `rank` columns are sum_j p_j c_j).  Kernels here:
//   latent_prep     per token: the query latent's RMS norm; c's RMS norm; r rotated by position; [c | r | 0] into the page
//   latent_qrot     per (token, head): the rotated query part into the wide query row [Wuk_h^T q_h | rot(q_r) | 0]
//   head_matmul     y[t, h, :] = x[t, h, :] W[h]  with W[h] stored [K, N]: both changes of space above
// Norm statistics, angles and every sum are float.
#include "common.cuh"

// rotation of one pair of the first `rot` of n values at position p (pair i is (i, i + rot/2), or with `interleaved`
// (2i, 2i + 1)); values past rot pass through
__device__ __forceinline__ void turn_pair(float a, float b, int p, float f, float& ra, float& rb) {
    float s, c;
    sincosf(__fmul_rn((float)p, f), &s, &c);
    ra = __fmul_rn(a, c) - __fmul_rn(b, s);
    rb = __fmul_rn(b, c) + __fmul_rn(a, s);
}

// down: float rows `ld` apart, each [qr + rank + dr ...] (query latent, key/value latent, shared key part, then whatever else
// rode in the same product).  cq: [T, qr]; the page row: d wide.
template <typename TA, typename TW>
__global__ void __launch_bounds__(256) latent_prep_kernel(const float* __restrict__ down, int ld, int qr, int rank, int dr, const TW* __restrict__ wq,
                                                          const TW* __restrict__ wkv, float eps, const float* __restrict__ inv_freq, int rot,
                                                          const int* __restrict__ pos, const int* __restrict__ req_slot,
                                                          const int* __restrict__ table, int max_pages, int page_size,
                                                          TA* __restrict__ cq, TA* __restrict__ k_pages, int d, int write_kv, int interleaved,
                                                          const TlLimits L) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    const float* row = down + (size_t)t * ld;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < qr; i += blockDim.x) sq = fmaf(row[i], row[i], sq);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) sk = fmaf(row[qr + i], row[qr + i], sk);
    if (qr > 0) sq = block_sum(sq, red);                 // qr 0: the queries come from a projection of their own, no latent
    sk = block_sum(sk, red);
    const float rq = qr > 0 ? 1.0f / sqrtf(sq / (float)qr + eps) : 0.f, rk = 1.0f / sqrtf(sk / (float)rank + eps);
    for (int i = threadIdx.x; i < qr; i += blockDim.x) cq[(size_t)t * qr + i] = from_f<TA>(row[i] * rq * to_f<TW>(wq[i]));
    if (!write_kv) return;
    const int p = pos[t];
    const int slot = tl_checked(req_slot[t], L.table_rows, L, TL_K_ROPE);
    const int page = tl_checked(table[(size_t)slot * max_pages + tl_checked(p / page_size, max_pages, L, TL_K_ROPE)],
                                L.total_pages, L, TL_K_ROPE);
    TA* dst = k_pages + ((size_t)page * page_size + (p % page_size)) * d;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f<TA>(row[qr + i] * rk * to_f<TW>(wkv[i]));
    const float* r = row + qr + rank;
    const int rhalf = rot >> 1;
    for (int i = threadIdx.x; i < rhalf; i += blockDim.x) {
        float a, b;
        const int e1 = interleaved ? 2 * i : i, e2 = interleaved ? 2 * i + 1 : i + rhalf;
        turn_pair(r[e1], r[e2], p, inv_freq[i], a, b);
        dst[rank + e1] = from_f<TA>(a); dst[rank + e2] = from_f<TA>(b);
    }
    for (int i = rot + threadIdx.x; i < dr; i += blockDim.x) dst[rank + i] = from_f<TA>(r[i]);
    for (int i = rank + dr + threadIdx.x; i < d; i += blockDim.x) dst[i] = from_f<TA>(0.f);
}

TL_EXPORT int tl_latent_prep(const float* down, int ld, int qr, int rank, int dr, const void* wq, const void* wkv, int w_dtype, float eps,
                             const float* inv_freq, int rot, const int* pos, const int* req_slot, const int* table, int max_pages,
                             int page_size, void* cq, void* k_pages, int act_dtype, int d, int write_kv, int T, int interleaved,
                             int table_rows, int total_pages, int* fault, cudaStream_t stream) {
    if (T <= 0) return 0;
    if ((rot & 1) || rot > dr || rank + dr > d || ld < qr + rank + dr) return 1;
    const TlLimits L{table_rows, total_pages, fault};
#define LP(TA, TW) launch_after_wait(latent_prep_kernel<TA, TW>, dim3(T), dim3(256), 0, stream, down, ld, qr, rank, dr, (const TW*)wq, (const TW*)wkv, \
        eps, inv_freq, rot, pos, req_slot, table, max_pages, page_size, (TA*)cq, (TA*)k_pages, d, write_kv, interleaved, L)
    if (act_dtype == TL_F32) { if (w_dtype == TL_F32) LP(float, float); else LP(float, bf16); }
    else { if (w_dtype == TL_F32) LP(bf16, float); else LP(bf16, bf16); }
#undef LP
    return tl_launch_status();
}

// q: [T, H, dk + dr] (plain part, then the part to rotate); qa: [T, H, d]: columns [rank, rank + dr) get the rotated part,
// columns from rank + dr on zeros.
template <typename TA>
__global__ void latent_qrot_kernel(const TA* __restrict__ q, int dk, int dr, const float* __restrict__ inv_freq, int rot,
                                   const int* __restrict__ pos, TA* __restrict__ qa, int rank, int d, int H, int interleaved) {
    const int t = blockIdx.x, h = blockIdx.y;
    grid_dependency_wait();
    grid_dependency_trigger();
    const TA* src = q + ((size_t)t * H + h) * (dk + dr) + dk;
    TA* dst = qa + ((size_t)t * H + h) * d + rank;
    const int p = pos[t], rhalf = rot >> 1;
    for (int i = threadIdx.x; i < rhalf; i += blockDim.x) {
        float a, b;
        const int e1 = interleaved ? 2 * i : i, e2 = interleaved ? 2 * i + 1 : i + rhalf;
        turn_pair(to_f<TA>(src[e1]), to_f<TA>(src[e2]), p, inv_freq[i], a, b);
        dst[e1] = from_f<TA>(a); dst[e2] = from_f<TA>(b);
    }
    for (int i = rot + threadIdx.x; i < dr; i += blockDim.x) dst[i] = src[i];
    for (int i = dr + threadIdx.x; i < d - rank; i += blockDim.x) dst[i] = from_f<TA>(0.f);
}

TL_EXPORT int tl_latent_qrot(const void* q, int dk, int dr, const float* inv_freq, int rot, const int* pos, void* qa, int rank, int d,
                             int H, int T, int act_dtype, int interleaved, cudaStream_t stream) {
    if (T <= 0 || H <= 0) return 0;
    if ((rot & 1) || rot > dr || rank + dr > d || H > 65535) return 1;
    if (act_dtype == TL_F32) launch_after_wait(latent_qrot_kernel<float>, dim3(T, H), dim3(64), 0, stream, (const float*)q, dk, dr, inv_freq, rot, pos, (float*)qa, rank, d, H, interleaved);
    else launch_after_wait(latent_qrot_kernel<bf16>, dim3(T, H), dim3(64), 0, stream, (const bf16*)q, dk, dr, inv_freq, rot, pos, (bf16*)qa, rank, d, H, interleaved);
    return tl_launch_status();
}

// y[t, h, n] = sum_k x[t, h, k] w[h, k, n];  x rows `ldx` apart, heads `hx` apart (y: ldy, hy).  grid (token tiles, heads,
// column tiles of 32); a block is 32 columns x 4 quarters of k: a thread sums its quarter of k in order for HM_T tokens (their x
// rows sit in shared memory as float, a weight is loaded once for HM_T sums, eight weights' loads are in flight at a time), and
// the four quarters are added in order.  Every output is one fixed chain of additions: a row's result does not depend on the
// step's other rows or on how many there are.
constexpr int HM_T = 8;
template <typename TA, typename TW>
__global__ void __launch_bounds__(128) head_matmul_kernel(const TA* __restrict__ x, int ldx, int hx, const TW* __restrict__ w,
                                                          TA* __restrict__ y, int ldy, int hy, int T, int K, int N) {
    extern __shared__ float xs[];                        // [HM_T][K], then the quarters' sums [4][HM_T][32]
    float* part = xs + HM_T * K;
    const int col = threadIdx.x & 31, quarter = threadIdx.x >> 5;
    const int t0 = blockIdx.x * HM_T, h = blockIdx.y, n = blockIdx.z * 32 + col;
    grid_dependency_wait();
    grid_dependency_trigger();
    const int nt = min(HM_T, T - t0);
    for (int i = threadIdx.x; i < nt * K; i += blockDim.x) {
        const int t = i / K, k = i - t * K;
        xs[i] = to_f<TA>(x[(size_t)(t0 + t) * ldx + (size_t)h * hx + k]);
    }
    __syncthreads();
    float acc[HM_T];
#pragma unroll
    for (int t = 0; t < HM_T; ++t) acc[t] = 0.f;
    const int per = (K + 3) / 4, k1 = min(K, (quarter + 1) * per);
    int k = quarter * per;
    if (n < N) {
        const TW* wh = w + (size_t)h * K * N + n;
        for (; k + 8 <= k1; k += 8) {
            TW w8[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) w8[u] = wh[(size_t)(k + u) * N];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float wv = to_f<TW>(w8[u]);
#pragma unroll
                for (int t = 0; t < HM_T; ++t) if (t < nt) acc[t] = fmaf(xs[t * K + k + u], wv, acc[t]);
            }
        }
        for (; k < k1; ++k) {
            const float wv = to_f<TW>(wh[(size_t)k * N]);
#pragma unroll
            for (int t = 0; t < HM_T; ++t) if (t < nt) acc[t] = fmaf(xs[t * K + k], wv, acc[t]);
        }
    }
#pragma unroll
    for (int t = 0; t < HM_T; ++t) part[(quarter * HM_T + t) * 32 + col] = acc[t];
    __syncthreads();
    if (quarter == 0 && n < N) {
#pragma unroll
        for (int t = 0; t < HM_T; ++t) {
            if (t < nt) {
                const float v = ((part[t * 32 + col] + part[(HM_T + t) * 32 + col]) + part[(2 * HM_T + t) * 32 + col]) +
                                part[(3 * HM_T + t) * 32 + col];
                y[(size_t)(t0 + t) * ldy + (size_t)h * hy + n] = from_f<TA>(v);
            }
        }
    }
}

TL_EXPORT int tl_head_matmul(const void* x, int ldx, int hx, const void* w, int w_dtype, void* y, int ldy, int hy, int T, int H, int K,
                             int N, int act_dtype, cudaStream_t stream) {
    if (T <= 0 || H <= 0 || N <= 0) return 0;
    const size_t smem = ((size_t)HM_T * K + 4 * HM_T * 32) * sizeof(float);
    if (smem > 48 * 1024 || H > 65535 || (N + 31) / 32 > 65535) return 1;
    const dim3 grid((T + HM_T - 1) / HM_T, H, (N + 31) / 32);
#define HM(TA, TW) launch_after_wait(head_matmul_kernel<TA, TW>, grid, dim3(128), smem, stream, (const TA*)x, ldx, hx, (const TW*)w, (TA*)y, ldy, hy, T, K, N)
    if (act_dtype == TL_F32) { if (w_dtype == TL_F32) HM(float, float); else HM(float, bf16); }
    else { if (w_dtype == TL_F32) HM(bf16, float); else HM(bf16, bf16); }
#undef HM
    return tl_launch_status();
}
