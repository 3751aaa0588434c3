// Paged causal grouped-query attention, one warp per (token, query head).
//
// This is the exact-order kernel: the true 32-bit engine uses it for prompts and for decoding,
// and the tests use it (in bfloat16 too) as the on-device reference of the tensor-core kernels.
// A query at position p of a request reads the keys at positions lo..p of that request from the
// cache pages, lo = 0 or p - window + 1 (tensorline/paged.py:237; tensorline/paged_attn.py:43).
// s = (q . k) * scale, softmax over keys in float, o = P V (tensorline/paged_attn.py:46-57).
// `sink` (float per query head, may be null): the denominator also holds exp(sink[h]), a term with no
// key and no value that is not scaled and counts once.
// `keep_first` (with a window): the keys at positions below it are read as well, however far the window has moved.
// `gate` (float [T, nq], may be null): the finished row is multiplied by sigmoid(gate[t, h]).
// `chunk` (> 0, instead of a window): the sequence is cut into chunks of that many positions counted from position 0, and
// a query reads the keys of its own chunk only: lo = (p / chunk) * chunk.
// `slopes` (float per query head, may be null): a key's score loses slopes[h] * (p - j), its distance from the query.
//
// Keys are taken in tiles of 32 aligned to absolute position 0, each lane owning one key of the
// tile, with a running maximum and sum.  The order of every addition depends only on the
// query's position and the window, never on how the step was cut or batched, so the result for
// a position is bit-identical under every schedule.
#include "common.cuh"

#define ATT_MAX_D 512

template <typename TA>
__global__ void attn_tokenwise_kernel(const TA* __restrict__ q, int q_stride, TA* __restrict__ out,
                                      const TA* __restrict__ k_pages, const TA* __restrict__ v_pages,
                                      const int* __restrict__ table, int max_pages, int page_size,
                                      const int* __restrict__ pos, const int* __restrict__ req_slot,
                                      int nq, int nkv, int d, int window, float scale,
                                      const float* __restrict__ sink, int keep_first, const float* __restrict__ gate,
                                      int chunk, const float* __restrict__ slopes, const TlLimits L) {
    __shared__ float qs[ATT_MAX_D];
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    const int kh = h / (nq / nkv);
    const int p = pos[t];
    const int lo = chunk > 0 ? (p / chunk) * chunk : (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const float slope = slopes ? slopes[h] : 0.f;
    const int* tab = table + (size_t)tl_checked(req_slot[t], L.table_rows, L, TL_K_TOKENWISE) * max_pages;
    const TA* qrow = q + (size_t)t * q_stride + (size_t)h * d;
    for (int e = lane; e < d; e += 32) qs[e] = to_f<TA>(qrow[e]);
    __syncwarp();

    constexpr int MAXC = ATT_MAX_D / 32;
    float acc[MAXC];
#pragma unroll
    for (int c = 0; c < MAXC; ++c) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;

    // tiles of 32 keys from position 0 on; those that lie wholly between the kept first keys and the window are skipped
    const int kept = min(keep_first, lo);                // keys [0, kept) and [lo, p]
    for (int j0 = 0; j0 <= p; j0 += 32) {
        if (j0 >= kept && j0 + 32 <= lo) { j0 = (lo / 32) * 32 - 32; continue; }
        const int j = j0 + lane;
        const bool valid = (j >= lo || j < kept) && (j <= p);
        size_t row = 0;
        float s = -INFINITY;
        if (valid) {
            const int page = tl_checked(tab[tl_checked(j / page_size, max_pages, L, TL_K_TOKENWISE)], L.total_pages, L, TL_K_TOKENWISE);
            row = (((size_t)page * nkv + kh) * page_size + (j % page_size)) * d;
            const TA* kr = k_pages + row;
            float dot = 0.f;
            for (int e = 0; e < d; ++e) dot = fmaf(qs[e], to_f<TA>(kr[e]), dot);
            s = dot * scale;
            if (slopes) s -= slope * (float)(p - j);
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = expf(m - m_new);            // 0 on the first tile (m = -inf)
        const float pj = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(pj);
#pragma unroll
        for (int c = 0; c < MAXC; ++c) acc[c] *= alpha;
        const int n_here = min(32, p - j0 + 1);
        for (int jj = 0; jj < n_here; ++jj) {
            const float pb = __shfl_sync(0xffffffffu, pj, jj);
            const unsigned long long rb = __shfl_sync(0xffffffffu, (unsigned long long)row, jj);
            if (pb != 0.f) {                             // uniform over the warp
                const TA* vr = v_pages + rb;
#pragma unroll
                for (int c = 0; c < MAXC; ++c) {
                    const int e = lane + 32 * c;
                    if (e < d) acc[c] = fmaf(pb, to_f<TA>(vr[e]), acc[c]);
                }
            }
        }
        m = m_new;
    }
    if (sink) {                                          // one more term of the denominator: no key, no value
        const float m_new = fmaxf(m, sink[h]);
        const float alpha = expf(m - m_new);
        l = l * alpha + expf(sink[h] - m_new);
#pragma unroll
        for (int c = 0; c < MAXC; ++c) acc[c] *= alpha;
    }
    TA* orow = out + ((size_t)t * nq + h) * d;
    float inv = 1.0f / l;
    if (gate) inv *= 1.0f / (1.0f + expf(-gate[(size_t)t * nq + h]));
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
        const int e = lane + 32 * c;
        if (e < d) orow[e] = from_f<TA>(acc[c] * inv);
    }
}

TL_EXPORT int tl_attn_tokenwise(const void* q, int q_stride, void* out, int act_dtype,
                                const void* k_pages, const void* v_pages, const int* table, int max_pages,
                                int page_size, const int* pos, const int* req_slot, int T, int nq, int nkv,
                                int d, int window, float scale, const float* sink, int keep_first, const float* gate,
                                int chunk, const float* slopes, int table_rows, int total_pages, int* fault, cudaStream_t stream) {
    const TlLimits L{table_rows, total_pages, fault};
    if (T <= 0) return 0;
    if (d > ATT_MAX_D || nq % nkv || (chunk > 0 && window > 0) || chunk < 0) return 1;
    dim3 grid(T, nq);
    if (act_dtype == TL_F32)
        attn_tokenwise_kernel<float><<<grid, 32, 0, stream>>>((const float*)q, q_stride, (float*)out,
            (const float*)k_pages, (const float*)v_pages, table, max_pages, page_size, pos, req_slot,
            nq, nkv, d, window, scale, sink, window > 0 ? keep_first : 0, gate, chunk, slopes, L);
    else
        attn_tokenwise_kernel<bf16><<<grid, 32, 0, stream>>>((const bf16*)q, q_stride, (bf16*)out,
            (const bf16*)k_pages, (const bf16*)v_pages, table, max_pages, page_size, pos, req_slot,
            nq, nkv, d, window, scale, sink, window > 0 ? keep_first : 0, gate, chunk, slopes, L);
    return tl_launch_status();
}
