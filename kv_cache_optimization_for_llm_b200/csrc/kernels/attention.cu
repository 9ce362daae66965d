// Attention over the paged cache, general form: any mix of query runs (a prompt
// portion, a single decoded token) against the keys of their own requests.
//
// One block per (query token, query head); its four warps take the keys in chunks
// of 32 consecutive positions, chunk c going to warp c % 4.  The chunking follows
// absolute key positions, so the sums a query sees are the same however its
// request was cut into steps, whatever else is in the batch and wherever its
// pages lie.  Scores, softmax and the weighted sum of values are float32.
//
// Upstream computes the same thing in two kernels, one over a packed prompt
// (base/src/kernels.cu:361-466) and one over the cache for a single token
// (paged_attention/src/kernels.cu:150-219): score = (q.k)/sqrt(d), keys j <= pos,
// kv head = q head / (nq/nkv), online softmax.  `window` > 0 keeps only keys
// j > pos - window (upstream has none).
#include "common.cuh"

#include <math_constants.h>

constexpr int kMaxHeadDim = 256;
constexpr int kWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
paged_attention_generic_kernel(const T* __restrict__ q_base, int q_row_stride,
                               const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                               const int* __restrict__ block_table, int max_pages, int page_size,
                               int num_pages, const int* __restrict__ positions,
                               const int* __restrict__ token_req, T* __restrict__ out, int nq, int nkv,
                               int d, float scale, int window, int* status) {
  __shared__ float q_s[kMaxHeadDim];
  __shared__ float acc_s[kWarps][kMaxHeadDim];
  __shared__ float m_s[kWarps], l_s[kWarps];

  const int t = blockIdx.x;
  const int h = blockIdx.y;
  const int hk = h / (nq / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[t];
  const int* table = block_table + (size_t)token_req[t] * max_pages;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;

  const T* q = q_base + (size_t)t * q_row_stride + (size_t)h * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) q_s[i] = to_f32(q[i]);
  __syncthreads();

  float m = -CUDART_INF_F, l = 0.f;
  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int r = 0; r < kMaxHeadDim / 32; ++r) acc[r] = 0.f;

  for (int c = lo / 32 + ((warp - lo / 32) % kWarps + kWarps) % kWarps; c * 32 <= pos; c += kWarps) {
    const int j = c * 32 + lane;
    const bool valid = j >= lo && j <= pos;
    long long off = -1;
    float s = -CUDART_INF_F;
    if (valid) {
      const int lp = j / page_size;
      const int page = lp < max_pages ? table[lp] : -1;
      if (page < 0 || page >= num_pages) {
        atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
      } else {
        off = (((long long)page * nkv + hk) * page_size + (j % page_size)) * d;
        const T* k = k_pages + off;
        float dot = 0.f;
        for (int i = 0; i < d; ++i) dot = fmaf(q_s[i], to_f32(k[i]), dot);
        s = dot * scale;
      }
    }
    const float cm = warp_max(s);
    if (cm == -CUDART_INF_F) continue;  // nothing readable in this chunk (only after an error)
    const float m_new = fmaxf(m, cm);
    const float corr = (m == -CUDART_INF_F) ? 0.f : expf(m - m_new);
    const float p = (off >= 0) ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int r = 0; r < kMaxHeadDim / 32; ++r) acc[r] *= corr;
    const int n_in_chunk = min(32, pos - c * 32 + 1);
    for (int jj = 0; jj < n_in_chunk; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long oj = __shfl_sync(0xffffffffu, off, jj);
      if (oj < 0) continue;
      const T* v = v_pages + oj;
#pragma unroll
      for (int r = 0; r < kMaxHeadDim / 32; ++r) {
        const int i = r * 32 + lane;
        if (i < d) acc[r] = fmaf(pj, to_f32(v[i]), acc[r]);
      }
    }
    m = m_new;
  }

  if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
  for (int r = 0; r < kMaxHeadDim / 32; ++r) {
    const int i = r * 32 + lane;
    if (i < d) acc_s[warp][i] = acc[r];
  }
  __syncthreads();
  if (warp == 0) {
    float M = m_s[0];
    for (int w = 1; w < kWarps; ++w) M = fmaxf(M, m_s[w]);
    float L = 0.f, f[kWarps];
    for (int w = 0; w < kWarps; ++w) {
      f[w] = (m_s[w] == -CUDART_INF_F) ? 0.f : expf(m_s[w] - M);
      L += l_s[w] * f[w];
    }
    T* o = out + ((size_t)t * nq + h) * d;
    for (int i = lane; i < d; i += 32) {
      float a = 0.f;
      for (int w = 0; w < kWarps; ++w) a += acc_s[w][i] * f[w];
      o[i] = from_f32<T>(L > 0.f ? a / L : 0.f);
    }
  }
}

// q points at the first query head of token 0; consecutive tokens are q_row_stride
// elements apart (the fused q|k|v row).  out is [T, nq*d], dense.
// Refuses: d > 256, odd d, nq not a multiple of nkv.
KVB_EXPORT int kvb_paged_attention_generic(const void* q, int q_row_stride, const void* k_pages,
                                           const void* v_pages, const int* block_table, int max_pages,
                                           int page_size, int num_pages, const int* positions,
                                           const int* token_req, void* out, int T_, int nq, int nkv,
                                           int d, float scale, int window, int dtype, int* status,
                                           cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (d > kMaxHeadDim || d < 2 || (d & 1) || nkv < 1 || nq % nkv) return KVB_ERR_BAD_SIZE;
  dim3 grid(T_, nq);
  KVB_DISPATCH_DTYPE(dtype, T, (paged_attention_generic_kernel<T><<<grid, kWarps * 32, 0, stream>>>(
                                   (const T*)q, q_row_stride, (const T*)k_pages, (const T*)v_pages,
                                   block_table, max_pages, page_size, num_pages, positions, token_req,
                                   (T*)out, nq, nkv, d, scale, window, status)));
  return kvb_launch_result();
}
