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

  pdl_trigger();
  pdl_wait();
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
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(paged_attention_generic_kernel<T>, grid, dim3(kWarps * 32), 0, stream,
                                            (const T*)q, q_row_stride, (const T*)k_pages, (const T*)v_pages,
                                            block_table, max_pages, page_size, num_pages, positions, token_req,
                                            (T*)out, nq, nkv, d, scale, window, status)));
  return kvb_launch_result();
}

// ===========================================================================
// Decode attention: every request brings one query token.  Split over the keys.
//
// Block (kv head, request, key block b) takes the keys [b*KB, (b+1)*KB) of its
// request and all `group` query heads that share the kv head, so each key and
// value is read from memory once for the group (upstream reads them once per query
// head: paged_attention/src/kernels.cu:150-219).  A thread owns one key for the
// scores (its K row against the group's queries, which sit pre-scaled in shared
// memory), the block agrees on max and sum per head, then each warp folds its 32
// values into the output dims its lanes own.  The block writes an unnormalised
// partial (o, m, l) to scratch; `decode_attention_combine_kernel` merges the key
// blocks of a (request, head) in ascending order.  Key blocks are cut at absolute
// positions with a size fixed by the engine, so a token's sums do not depend on
// the batch it runs in.
// ===========================================================================

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};

constexpr int kDecThreads = 128;  // 4 warps, 128 keys per pass

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

// Grid (kv head, request, slot): slot z takes the key blocks z, z + gridDim.z, ... of its
// request, so no block of an absent key range is ever launched and the grid does not
// depend on the contexts' lengths.  The partial result of key block b lands in
// part_*[..., b], whoever computed it.
template <typename T, int D, int GMAX>
__global__ void __launch_bounds__(kDecThreads, 5)
decode_attention_split_kernel(const T* __restrict__ q_base, int q_row_stride, const T* __restrict__ k_pages,
                              const T* __restrict__ v_pages, const int* __restrict__ block_table,
                              int max_pages, int page_size, int num_pages, const int* __restrict__ q_start,
                              const int* __restrict__ ctx_len, float* __restrict__ part_o,
                              float* __restrict__ part_ml, int nq, int nkv, int G, float scale, int window,
                              int KB, int NB, int* status) {
  constexpr int DPL = D / 32;                    // output dims per lane
  constexpr int CPK = D * (int)sizeof(T) / 16;   // 16-byte chunks per value row
  __shared__ __align__(16) float q_s[GMAX][D];
  __shared__ float red_s[4][GMAX];
  extern __shared__ __align__(16) unsigned char dec_smem[];
  T (*v_s)[32][D] = reinterpret_cast<T (*)[32][D]>(dec_smem);  // each warp stages the values of its 32 keys

  pdl_trigger();
  pdl_wait();
  const int hk = blockIdx.x, r = blockIdx.y;
  const int pos = ctx_len[r] - 1;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if ((int)blockIdx.z * KB > pos) return;
  const int* table = block_table + (size_t)r * max_pages;

  const T* q = q_base + (size_t)q_start[r] * q_row_stride + (size_t)hk * G * D;
  for (int i = tid; i < G * D; i += kDecThreads) q_s[i / D][i % D] = to_f32(q[i]) * scale;
  __syncthreads();

  for (int b = blockIdx.z; b * KB <= pos && b < NB; b += gridDim.z) {
    const int k0 = b * KB;
    if (k0 + KB <= lo) continue;  // the window has passed this block; combine skips it too
    float m_run[GMAX], l_run[GMAX], acc[GMAX][DPL];
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
      m_run[g] = -CUDART_INF_F; l_run[g] = 0.f;
#pragma unroll
      for (int e = 0; e < DPL; ++e) acc[g][e] = 0.f;
    }
    const int k_end = min(k0 + KB, pos + 1);
    for (int base = k0; base < k_end; base += kDecThreads) {
      const int j = base + tid;
      const bool valid = j < k_end && j >= lo;
      long long off = -1;
      if (valid) {
        const int lp = j / page_size;
        const int page = lp < max_pages ? table[lp] : -1;
        if (page < 0 || page >= num_pages) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
        else off = (((long long)page * nkv + hk) * page_size + (j % page_size)) * D;
      }
      // the values of this warp's keys start their way to shared memory now and
      // arrive while the scores are computed
#pragma unroll
      for (int i = 0; i < CPK; ++i) {
        const int c = i * 32 + lane;
        const int key = c / CPK, part = c % CPK;
        const long long oj = __shfl_sync(0xffffffffu, off, key);
        if (oj >= 0)
          cp_async_16(reinterpret_cast<char*>(&v_s[warp][key][0]) + part * 16,
                      reinterpret_cast<const char*>(v_pages + oj) + part * 16);
      }
      float s[GMAX];
#pragma unroll
      for (int g = 0; g < GMAX; ++g) s[g] = -CUDART_INF_F;
      if (off >= 0) {
        const T* k = k_pages + off;
#pragma unroll
        for (int g = 0; g < GMAX; ++g) s[g] = 0.f;
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
          float kf[8];
          Vec8<T>::load(k + c * 8, kf);
#pragma unroll
          for (int g = 0; g < GMAX; ++g) {
            if (g < G) {
              const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][c * 8]);
              const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][c * 8 + 4]);
              float t = s[g];
              t = fmaf(qa.x, kf[0], t); t = fmaf(qa.y, kf[1], t); t = fmaf(qa.z, kf[2], t); t = fmaf(qa.w, kf[3], t);
              t = fmaf(qb.x, kf[4], t); t = fmaf(qb.y, kf[5], t); t = fmaf(qb.z, kf[6], t); t = fmaf(qb.w, kf[7], t);
              s[g] = t;
            }
          }
        }
      }
      // block-wide max per head
#pragma unroll
      for (int g = 0; g < GMAX; ++g) {
        const float wm = warp_max(g < G ? s[g] : -CUDART_INF_F);
        if (lane == 0) red_s[warp][g] = wm;
      }
      __syncthreads();
      float p[GMAX], corr[GMAX];
#pragma unroll
      for (int g = 0; g < GMAX; ++g) {
        const float bm = fmaxf(fmaxf(red_s[0][g], red_s[1][g]), fmaxf(red_s[2][g], red_s[3][g]));
        const float m_new = fmaxf(m_run[g], bm);
        corr[g] = (m_run[g] == -CUDART_INF_F) ? 0.f : __expf(m_run[g] - m_new);
        p[g] = (off >= 0 && g < G) ? __expf(s[g] - m_new) : 0.f;
        m_run[g] = m_new;
      }
      __syncthreads();
#pragma unroll
      for (int g = 0; g < GMAX; ++g) {
        const float ws = warp_sum(p[g]);
        if (lane == 0) red_s[warp][g] = ws;
      }
      __syncthreads();
#pragma unroll
      for (int g = 0; g < GMAX; ++g) {
        l_run[g] = l_run[g] * corr[g] + ((red_s[0][g] + red_s[1][g]) + (red_s[2][g] + red_s[3][g]));
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[g][e] *= corr[g];
      }
      // fold the staged values of this warp's 32 keys into the dims its lanes own
      cp_async_wait_all();
      __syncwarp();
      const int n_here = min(32, k_end - (base + warp * 32));
      for (int jj = 0; jj < n_here; ++jj) {
        const long long oj = __shfl_sync(0xffffffffu, off, jj);
        float pj[GMAX];
#pragma unroll
        for (int g = 0; g < GMAX; ++g) pj[g] = __shfl_sync(0xffffffffu, p[g], jj);
        if (oj < 0) continue;
        float vf[DPL];
        const T* v = &v_s[warp][jj][lane * DPL];
        if constexpr (sizeof(T) == 2 && DPL == 2) {
          const unsigned w = *reinterpret_cast<const unsigned*>(v);
          vf[0] = __uint_as_float(w << 16); vf[1] = __uint_as_float(w & 0xffff0000u);
        } else if constexpr (sizeof(T) == 2 && DPL == 4) {
          const uint2 w = *reinterpret_cast<const uint2*>(v);
          vf[0] = __uint_as_float(w.x << 16); vf[1] = __uint_as_float(w.x & 0xffff0000u);
          vf[2] = __uint_as_float(w.y << 16); vf[3] = __uint_as_float(w.y & 0xffff0000u);
        } else {
#pragma unroll
          for (int e = 0; e < DPL; ++e) vf[e] = to_f32(v[e]);
        }
#pragma unroll
        for (int g = 0; g < GMAX; ++g)
          if (g < G)
#pragma unroll
            for (int e = 0; e < DPL; ++e) acc[g][e] = fmaf(pj[g], vf[e], acc[g][e]);
      }
      __syncthreads();  // red_s and v_s are rewritten by the next pass
    }
    // sum the four warps' partial outputs in a fixed order, through shared memory
    float* red = reinterpret_cast<float*>(dec_smem);  // the value stage is free again and large enough
    static_assert(sizeof(T) * 32 >= sizeof(float) * GMAX, "the value stage must hold the warps' partial outputs");
#pragma unroll
    for (int g = 0; g < GMAX; ++g)
      if (g < G)
#pragma unroll
        for (int e = 0; e < DPL; ++e) red[(warp * GMAX + g) * D + lane * DPL + e] = acc[g][e];
    __syncthreads();
    for (int i = tid; i < G * D; i += kDecThreads) {
      const int g = i / D, dd = i % D;
      const float o = (red[(0 * GMAX + g) * D + dd] + red[(1 * GMAX + g) * D + dd]) +
                      (red[(2 * GMAX + g) * D + dd] + red[(3 * GMAX + g) * D + dd]);
      part_o[(((size_t)r * nq + hk * G + g) * NB + b) * D + dd] = o;
    }
    if (tid < G) {
      float mm = 0.f, ll = 0.f;  // m_run and l_run are equal in every thread
#pragma unroll
      for (int g = 0; g < GMAX; ++g) if (g == tid) { mm = m_run[g]; ll = l_run[g]; }
      float* ml = part_ml + (((size_t)r * nq + hk * G + tid) * NB + b) * 2;
      ml[0] = mm; ml[1] = ll;
    }
    __syncthreads();  // red (v_s) is staged into again by the next key block
  }
}

// ---------------------------------------------------------------------------
// The whole attention of a decode step in one launch: rotary encoding of the query
// and the new key, the write of the new key and value into their page, the split
// attention over the key blocks, and the merge of the key blocks' partials.
//
// Block (kv head, request, slot) as above.  Every block rotates its own copy of the
// group's queries (kept in float32).  The block that owns the key block holding the
// token's own position rotates the new key, stores key and value into the cache, and
// then reads them back like any other key.  After its last key block a block adds one
// to the counter of its (request, kv head); the block that brings the counter to the
// number of participating blocks merges all partials in ascending key-block order and
// writes the output, then clears the counter.  Nobody waits for anybody.
// qkv rows stay as the projection wrote them (unrotated).
// ---------------------------------------------------------------------------
template <typename T, int D, int GMAX>
__global__ void __launch_bounds__(kDecThreads, 4)
decode_attention_fused_kernel(const T* __restrict__ qkv, int q_row_stride, T* __restrict__ k_pages,
                              T* __restrict__ v_pages, int write_kv, const int* __restrict__ block_table,
                              int max_pages, int page_size, int num_pages, const int* __restrict__ q_start,
                              const int* __restrict__ ctx_len, const float* __restrict__ cos_t,
                              const float* __restrict__ sin_t, int table_len, int rot, T* __restrict__ out,
                              float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters,
                              int nq, int nkv, int G, float scale, int window, int KB, int NB, int* status,
                              unsigned long long* trace) {
  constexpr int DPL = D / 32;
  constexpr int CPK = D * (int)sizeof(T) / 16;   // 16-byte chunks per key or value row
  constexpr int EPC = 16 / (int)sizeof(T);       // elements per chunk
  __shared__ __align__(16) float q_s[GMAX][D];
  __shared__ float red_s[4][GMAX];
  __shared__ int last_s;
  extern __shared__ __align__(16) unsigned char dec_smem[];
  T (*k_s)[32][D] = reinterpret_cast<T (*)[32][D]>(dec_smem);                                  // [4][32][D]
  T (*v_s)[32][D] = reinterpret_cast<T (*)[32][D]>(dec_smem + (size_t)4 * 32 * D * sizeof(T)); // [4][32][D]
  // optional profiling: nanosecond stamps of this block's phases, [blocks, 8]
  auto stamp = [&](int slot) {
    if (trace && threadIdx.x == 0) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      trace[(((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + slot] = t;
    }
  };
  stamp(0);
  pdl_trigger();
  // Lengths, block tables and the keys and values of earlier tokens were all written
  // before the kernel in front of this one started, so they may be read at once.
  const int hk = blockIdx.x, r = blockIdx.y;
  const int pos = ctx_len[r] - 1;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (pos < 0 || pos / KB >= NB || (cos_t != nullptr && pos >= table_len)) {
    pdl_wait();
    if (tid == 0 && blockIdx.z == 0) atomicCAS(status, 0, KVB_STATUS_BAD_POSITION);
    return;
  }
  if ((int)blockIdx.z * KB > pos) return;   // no key block for this slot; it is not counted either
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int* table = block_table + (size_t)r * max_pages;
  const int half = rot >> 1;
  const bool rotary = cos_t != nullptr && rot > 0;

  // Requests the keys and values of the 128 positions from `base` on into shared memory;
  // the token's own position is left out when this step writes it (it is filled in below).
  // Returns this thread's own key's offset, -1 if it has none to read.
  auto request_tile = [&](int base, int k_end, bool skip_pos) -> long long {
    const int j = base + tid;
    long long off = -1;
    if (j < k_end && j >= lo && !(skip_pos && j == pos)) {
      const int lp = j / page_size;
      const int page = lp < max_pages ? table[lp] : -1;
      if (page < 0 || page >= num_pages) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
      else off = (((long long)page * nkv + hk) * page_size + (j % page_size)) * D;
    }
#pragma unroll
    for (int i = 0; i < CPK; ++i) {
      const int c = i * 32 + lane;
      const int key = c / CPK, part = c % CPK;
      const long long oj = __shfl_sync(0xffffffffu, off, key);
      if (oj >= 0) {
        cp_async_16(reinterpret_cast<char*>(&k_s[warp][key][0]) + part * 16,
                    reinterpret_cast<const char*>(k_pages + oj) + part * 16);
        cp_async_16(reinterpret_cast<char*>(&v_s[warp][key][0]) + part * 16,
                    reinterpret_cast<const char*>(v_pages + oj) + part * 16);
      }
    }
    return off;
  };

  const int b_first = blockIdx.z;
  const int k_end_first = min(b_first * KB + KB, pos + 1);
  long long off = -1;
  const bool first_has_keys = b_first * KB + KB > lo;
  // A layer that reads another layer's cache finds the key and value of the token's own position
  // there: the owning layer wrote them earlier in this same step, several launches back.  Only the
  // wait below orders this kernel behind all of those, so a first tile that holds that position
  // is asked for after it.
  const bool own_key_from_this_step = !write_kv && pos >= b_first * KB && pos < b_first * KB + kDecThreads;
  if (first_has_keys && !own_key_from_this_step) off = request_tile(b_first * KB, k_end_first, write_kv != 0);

  pdl_wait();
  stamp(1);   // the kernel before this one has finished: its q, k, v rows may be read
  if (first_has_keys && own_key_from_this_step) off = request_tile(b_first * KB, k_end_first, false);
  const T* row = qkv + (size_t)q_start[r] * q_row_stride;
  // the group's queries, rotated (pairs (j, j + rot/2) of the first rot dims), scaled
  for (int i = tid; i < G * D; i += kDecThreads) {
    const int g = i / D, dd = i % D;
    const T* qh = row + (size_t)(hk * G + g) * D;
    float val;
    if (rotary && dd < rot) {
      const int j = dd < half ? dd : dd - half;
      const float c = cos_t[(size_t)pos * half + j], sn = sin_t[(size_t)pos * half + j];
      const float x1 = to_f32(qh[j]), x2 = to_f32(qh[j + half]);
      val = dd < half ? x1 * c - x2 * sn : x1 * sn + x2 * c;
    } else {
      val = to_f32(qh[dd]);
    }
    q_s[g][dd] = val * scale;
  }
  // The new key and value: the block that owns the key block of `pos` rotates the key,
  // stores both in the cache, and puts them into its shared-memory tile itself.
  const int b_star = pos / KB;
  const bool owner = write_kv && (b_star % (int)gridDim.z) == (int)blockIdx.z;
  // `pos` lies in the tile that was requested above: its key and value are put there directly
  const bool place_direct = owner && b_star == b_first && (pos - b_star * KB) < kDecThreads;
  bool own_ok = false;
  if (owner) {
    const int lp = pos / page_size;
    const int page = lp < max_pages ? table[lp] : -1;
    if (page < 0 || page >= num_pages) {
      if (tid == 0) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
    } else {
      own_ok = true;
      const size_t dst = (((size_t)page * nkv + hk) * page_size + (pos % page_size)) * D;
      const T* kh = row + (size_t)(nq + hk) * D;
      const T* vh = row + (size_t)(nq + nkv + hk) * D;
      const int slot = (pos - b_star * KB) % kDecThreads;  // place of `pos` inside its 128-key pass
      for (int dd = tid; dd < D; dd += kDecThreads) {
        float val;
        if (rotary && dd < rot) {
          const int j = dd < half ? dd : dd - half;
          const float c = cos_t[(size_t)pos * half + j], sn = sin_t[(size_t)pos * half + j];
          const float x1 = to_f32(kh[j]), x2 = to_f32(kh[j + half]);
          val = dd < half ? x1 * c - x2 * sn : x1 * sn + x2 * c;
        } else {
          val = to_f32(kh[dd]);
        }
        const T kr = from_f32<T>(val);
        k_pages[dst + dd] = kr;
        v_pages[dst + dd] = vh[dd];
        if (place_direct) { k_s[slot >> 5][slot & 31][dd] = kr; v_s[slot >> 5][slot & 31][dd] = vh[dd]; }
      }
      if (!place_direct) __threadfence();  // it will be fetched from L2 by a later pass of this block
    }
  }
  __syncthreads();
  stamp(2);   // queries rotated, new key/value stored

  for (int b = b_first; b * KB <= pos && b < NB; b += gridDim.z) {
    const int k0 = b * KB;
    if (k0 + KB <= lo) continue;
    float m_run[GMAX], l_run[GMAX], acc[GMAX][DPL];
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
      m_run[g] = -CUDART_INF_F; l_run[g] = 0.f;
#pragma unroll
      for (int e = 0; e < DPL; ++e) acc[g][e] = 0.f;
    }
    const int k_end = min(k0 + KB, pos + 1);
    for (int base = k0; base < k_end; base += kDecThreads) {
      const bool prefetched = (b == b_first && base == k0);
      // Later tiles are requested here; by now the new key, if it falls into one of them,
      // is in the cache and is read like any other.
      if (!prefetched) off = request_tile(base, k_end, false);
      const int j_mine = base + tid;
      bool have = off >= 0;
      if (prefetched && place_direct && own_ok && j_mine == pos) have = true;   // the key this block placed itself
      cp_async_wait_all();
      __syncwarp();
      float s[GMAX];
#pragma unroll
      for (int g = 0; g < GMAX; ++g) s[g] = have ? 0.f : -CUDART_INF_F;
      if (have) {
        const T* k = &k_s[warp][lane][0];
#pragma unroll
        for (int c = 0; c < CPK; ++c) {
          const int cc = (c + lane) % CPK;                // each lane starts at another chunk: no bank conflicts
          float kf[8];
          if constexpr (sizeof(T) == 2) {
            Vec8<T>::load(k + cc * 8, kf);
#pragma unroll
            for (int g = 0; g < GMAX; ++g) {
              if (g < G) {
                const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][cc * 8]);
                const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][cc * 8 + 4]);
                float t = s[g];
                t = fmaf(qa.x, kf[0], t); t = fmaf(qa.y, kf[1], t); t = fmaf(qa.z, kf[2], t); t = fmaf(qa.w, kf[3], t);
                t = fmaf(qb.x, kf[4], t); t = fmaf(qb.y, kf[5], t); t = fmaf(qb.z, kf[6], t); t = fmaf(qb.w, kf[7], t);
                s[g] = t;
              }
            }
          } else {
            const float4 ka = *reinterpret_cast<const float4*>(k + cc * EPC);
#pragma unroll
            for (int g = 0; g < GMAX; ++g) {
              if (g < G) {
                const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][cc * EPC]);
                float t = s[g];
                t = fmaf(qa.x, to_f32(ka.x), t); t = fmaf(qa.y, to_f32(ka.y), t);
                t = fmaf(qa.z, to_f32(ka.z), t); t = fmaf(qa.w, to_f32(ka.w), t);
                s[g] = t;
              }
            }
          }
        }
      }
#pragma unroll
      for (int g = 0; g < GMAX; ++g) {
        const float wm = warp_max(g < G ? s[g] : -CUDART_INF_F);
        if (lane == 0) red_s[warp][g] = wm;
      }
      __syncthreads();
      float p[GMAX], corr[GMAX];
#pragma unroll
      for (int g = 0; g < GMAX; ++g) {
        const float bm = fmaxf(fmaxf(red_s[0][g], red_s[1][g]), fmaxf(red_s[2][g], red_s[3][g]));
        const float m_new = fmaxf(m_run[g], bm);
        corr[g] = (m_run[g] == -CUDART_INF_F) ? 0.f : __expf(m_run[g] - m_new);
        p[g] = (have && g < G) ? __expf(s[g] - m_new) : 0.f;
        m_run[g] = m_new;
      }
      __syncthreads();
#pragma unroll
      for (int g = 0; g < GMAX; ++g) {
        const float ws = warp_sum(p[g]);
        if (lane == 0) red_s[warp][g] = ws;
      }
      __syncthreads();
#pragma unroll
      for (int g = 0; g < GMAX; ++g) {
        l_run[g] = l_run[g] * corr[g] + ((red_s[0][g] + red_s[1][g]) + (red_s[2][g] + red_s[3][g]));
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[g][e] *= corr[g];
      }
      const int n_here = min(32, k_end - (base + warp * 32));
      const unsigned have_mask = __ballot_sync(0xffffffffu, have);
      for (int jj = 0; jj < n_here; ++jj) {
        float pj[GMAX];
#pragma unroll
        for (int g = 0; g < GMAX; ++g) pj[g] = __shfl_sync(0xffffffffu, p[g], jj);
        if (!((have_mask >> jj) & 1u)) continue;
        float vf[DPL];
        const T* v = &v_s[warp][jj][lane * DPL];
        if constexpr (sizeof(T) == 2 && DPL == 2) {
          const unsigned w = *reinterpret_cast<const unsigned*>(v);
          vf[0] = __uint_as_float(w << 16); vf[1] = __uint_as_float(w & 0xffff0000u);
        } else if constexpr (sizeof(T) == 2 && DPL == 4) {
          const uint2 w = *reinterpret_cast<const uint2*>(v);
          vf[0] = __uint_as_float(w.x << 16); vf[1] = __uint_as_float(w.x & 0xffff0000u);
          vf[2] = __uint_as_float(w.y << 16); vf[3] = __uint_as_float(w.y & 0xffff0000u);
        } else {
#pragma unroll
          for (int e = 0; e < DPL; ++e) vf[e] = to_f32(v[e]);
        }
#pragma unroll
        for (int g = 0; g < GMAX; ++g)
          if (g < G)
#pragma unroll
            for (int e = 0; e < DPL; ++e) acc[g][e] = fmaf(pj[g], vf[e], acc[g][e]);
      }
      __syncthreads();   // red_s and the tiles are rewritten by the next pass
    }
    float* red = reinterpret_cast<float*>(dec_smem);
    static_assert(sizeof(T) * 32 >= sizeof(float) * GMAX, "the tiles must hold the warps' partial outputs");
#pragma unroll
    for (int g = 0; g < GMAX; ++g)
      if (g < G)
#pragma unroll
        for (int e = 0; e < DPL; ++e) red[(warp * GMAX + g) * D + lane * DPL + e] = acc[g][e];
    __syncthreads();
    for (int i = tid; i < G * D; i += kDecThreads) {
      const int g = i / D, dd = i % D;
      const float o = (red[(0 * GMAX + g) * D + dd] + red[(1 * GMAX + g) * D + dd]) +
                      (red[(2 * GMAX + g) * D + dd] + red[(3 * GMAX + g) * D + dd]);
      part_o[(((size_t)r * nq + hk * G + g) * NB + b) * D + dd] = o;
    }
    if (tid < G) {
      float mm = 0.f, ll = 0.f;
#pragma unroll
      for (int g = 0; g < GMAX; ++g) if (g == tid) { mm = m_run[g]; ll = l_run[g]; }
      float* ml = part_ml + (((size_t)r * nq + hk * G + tid) * NB + b) * 2;
      ml[0] = mm; ml[1] = ll;
    }
    __syncthreads();
  }
  stamp(3);   // key blocks done

  // ---- who is last merges
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int expected = min((int)gridDim.z, pos / KB + 1);
    const int old = atomicAdd(&counters[r * nkv + hk], 1);
    last_s = (old == expected - 1);
    if (last_s) counters[r * nkv + hk] = 0;   // ready for the next launch
  }
  __syncthreads();
  stamp(4);   // counted
  if (!last_s) return;
  __threadfence();
  // (max, sum) of every head and key block first, all requested at once; then the outputs
  const int b0 = lo / KB, b1 = pos / KB, nbk = b1 - b0 + 1;
  float* ml_s = reinterpret_cast<float*>(dec_smem);            // [G][nbk][2], nbk <= 64
  for (int i = tid; i < G * nbk * 2; i += kDecThreads) {
    const int g = i / (nbk * 2), rest = i % (nbk * 2);
    ml_s[i] = __ldcg(part_ml + ((size_t)r * nq + hk * G + g) * NB * 2 + (size_t)b0 * 2 + rest);
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += kDecThreads) {
    const int g = i / D, dd = i % D;
    const float* mlg = ml_s + (size_t)g * nbk * 2;
    const float* po = part_o + (((size_t)r * nq + hk * G + g) * NB + b0) * D + dd;
    float M = -CUDART_INF_F;
    for (int b = 0; b < nbk; ++b) M = fmaxf(M, mlg[2 * b]);
    float L = 0.f, a = 0.f;
    for (int bb = 0; bb < nbk; bb += 8) {
      float x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) x[u] = (bb + u < nbk) ? __ldcg(po + (size_t)(bb + u) * D) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (bb + u < nbk) {
          const float f = __expf(mlg[2 * (bb + u)] - M);
          L += mlg[2 * (bb + u) + 1] * f;
          a += x[u] * f;
        }
      }
    }
    out[((size_t)q_start[r] * nq + hk * G + g) * D + dd] = from_f32<T>(L > 0.f ? a / L : 0.f);
  }
  stamp(5);   // merged
}

template <typename T, int D>
__global__ void decode_attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                                                T* __restrict__ out, int nq, int window, int KB, int NB,
                                                int* status) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int pos = ctx_len[r] - 1;
  if (pos < 0 || pos / KB >= NB) {  // a context beyond the key blocks the scratch was sized for
    if (threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_BAD_POSITION);
    return;
  }
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int b0 = lo / KB, b1 = pos / KB;  // blocks that hold keys
  const float* ml = part_ml + ((size_t)r * nq + h) * NB * 2;
  const float* po = part_o + ((size_t)r * nq + h) * NB * D;
  float M = -CUDART_INF_F;
  for (int b = b0; b <= b1; ++b) M = fmaxf(M, ml[2 * b]);
  float L = 0.f;
  for (int b = b0; b <= b1; ++b) L += ml[2 * b + 1] * __expf(ml[2 * b] - M);
  T* o = out + ((size_t)q_start[r] * nq + h) * D;
  for (int dd = threadIdx.x; dd < D; dd += blockDim.x) {
    float a = 0.f;
    for (int b = b0; b <= b1; ++b) a += po[(size_t)b * D + dd] * __expf(ml[2 * b] - M);
    o[dd] = from_f32<T>(L > 0.f ? a / L : 0.f);
  }
}

template <typename T, int D, int GMAX>
static int launch_decode(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                         const int* block_table, int max_pages, int page_size, int num_pages, const int* q_start,
                         const int* ctx_len, void* out, float* part_o, float* part_ml, int R, int nq, int nkv,
                         float scale, int window, int KB, int NB, int* status, cudaStream_t stream) {
  // about four blocks per SM in total, never more slots than key blocks
  int slots = (4 * kvb_sm_count() + nkv * R - 1) / (nkv * R);
  slots = slots < 1 ? 1 : (slots > NB ? NB : slots);
  dim3 grid(nkv, R, slots);
  const size_t smem = (size_t)4 * 32 * D * sizeof(T);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_split_kernel<T, D, GMAX>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  kvb_launch(decode_attention_split_kernel<T, D, GMAX>, grid, dim3(kDecThreads), smem, stream, (const T*)q,
             q_row_stride, (const T*)k_pages, (const T*)v_pages, block_table, max_pages, page_size, num_pages,
             q_start, ctx_len, part_o, part_ml, nq, nkv, nq / nkv, scale, window, KB, NB, status);
  kvb_launch(decode_attention_combine_kernel<T, D>, dim3(R, nq), dim3(D >= 64 ? 64 : 32), 0, stream,
             (const float*)part_o, (const float*)part_ml, q_start, ctx_len, (T*)out, nq, window, KB, NB, status);
  return kvb_launch_result();
}

// Returns 1 when (d, group) has a split kernel: d in {32, 64, 128}, group <= 8.
KVB_EXPORT int kvb_decode_attention_supported(int d, int group) {
  return (d == 32 || d == 64 || d == 128) && group >= 1 && group <= 8;
}

// One query token per request: token row q_start[r], position ctx_len[r]-1.
// Scratch: part_o [R, nq, NB, d] and part_ml [R, nq, NB, 2] float32, NB = key blocks
// of KB keys (KB a multiple of 128) covering the longest context the caller allows.
// Two launches.  Refuses what kvb_decode_attention_supported refuses, and R or NB > 65535.
KVB_EXPORT int kvb_decode_attention(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                    const int* block_table, int max_pages, int page_size, int num_pages,
                                    const int* q_start, const int* ctx_len, void* out, float* part_o,
                                    float* part_ml, int R, int nq, int nkv, int d, float scale, int window,
                                    int KB, int NB, int dtype, int* status, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (nkv < 1 || nq % nkv || !kvb_decode_attention_supported(d, nq / nkv) || KB % kDecThreads || NB < 1 ||
      R > 65535 || NB > 65535)
    return KVB_ERR_BAD_SIZE;
  const int G = nq / nkv;
#define KVB_DEC(T, D, GM)                                                                                  \
  return launch_decode<T, D, GM>(q, q_row_stride, k_pages, v_pages, block_table, max_pages, page_size,    \
                                 num_pages, q_start, ctx_len, out, part_o, part_ml, R, nq, nkv, scale,    \
                                 window, KB, NB, status, stream)
#define KVB_DEC_D(T, D) do { if (G <= 2) KVB_DEC(T, D, 2); else if (G <= 4) KVB_DEC(T, D, 4); else KVB_DEC(T, D, 8); } while (0)
#define KVB_DEC_T(T) do { if (d == 32) KVB_DEC_D(T, 32); else if (d == 64) KVB_DEC_D(T, 64); else KVB_DEC_D(T, 128); } while (0)
  if (dtype == KVB_BF16) KVB_DEC_T(__nv_bfloat16);
  if (dtype == KVB_F32) KVB_DEC_T(float);
  return KVB_ERR_BAD_DTYPE;
}

// ===========================================================================
// The same decode attention for callers that cannot allocate: the scratch between
// the split and the combine launch is a static device array of this library.
// Declared and documented in decode_attention_noalloc.h.
// ===========================================================================
#include "decode_attention_noalloc.h"

#include <mutex>

static __device__ __align__(256) float g_decode_noalloc_scratch[KVB_DECODE_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};  // device address of the array, per device ordinal

// In host code `g_decode_noalloc_scratch` is only a handle for the runtime, not an
// address a kernel could use; the device address has to be asked for, once per
// device, with that device current.
int noalloc_scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return KVB_ERR_SCRATCH_SETUP;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return KVB_ERR_SCRATCH_SETUP;
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

KVB_EXPORT unsigned long long kvb_decode_attention_noalloc_scratch_needed(int R, int nq, int NB, int d) {
  if (R < 0 || nq < 0 || NB < 0 || d < 0) return ~0ull;
  return (unsigned long long)R * nq * NB * (unsigned long long)(d + 2);
}

KVB_EXPORT const char* kvb_decode_attention_noalloc_error(int code) {
  switch (code) {
    case 0: return "ok";
    case KVB_ERR_BAD_DTYPE: return "unsupported dtype (0 = float32, 1 = bfloat16)";
    case KVB_ERR_BAD_SIZE:
      return "a size the decode kernel refuses (head size must be 32, 64 or 128, group size 1..8, KB a multiple of 128)";
    case KVB_ERR_SCRATCH_TOO_SMALL:
      return "R * nq * NB * (d + 2) exceeds the 4 Mi floats of built-in scratch; use kvb_decode_attention with "
             "caller-provided scratch, or fewer requests / key blocks per call";
    case KVB_ERR_SCRATCH_SETUP: return "the built-in scratch could not be located on the current device";
    default: return code > 0 ? "a CUDA runtime error (the code is a cudaError_t)" : "unknown error code";
  }
}

KVB_EXPORT int kvb_decode_attention_noalloc(const void* q, int q_row_stride, const void* k_pages,
                                            const void* v_pages, const int* block_table, int max_pages,
                                            int page_size, int num_pages, const int* q_start,
                                            const int* ctx_len, void* out, int R, int nq, int nkv, int d,
                                            float scale, int window, int KB, int NB, int dtype, int* status,
                                            cudaStream_t stream) {
  if (R <= 0) return 0;
  if (nq < 1 || NB < 1 || d < 1) return KVB_ERR_BAD_SIZE;
  const unsigned long long need = kvb_decode_attention_noalloc_scratch_needed(R, nq, NB, d);
  if (need > (unsigned long long)KVB_DECODE_NOALLOC_SCRATCH_FLOATS) return KVB_ERR_SCRATCH_TOO_SMALL;
  float* scratch = nullptr;
  const int rc = noalloc_scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // Partial outputs first, then the (max, sum) pairs.  The array itself is aligned to 256 bytes;
  // the second offset, R * nq * NB * d floats, is a multiple of 16 bytes because the split kernel
  // takes head sizes 32, 64 and 128 only (any other d is refused by kvb_decode_attention below
  // before anything is launched), so d floats are always a multiple of 128 bytes.
  float* part_o = scratch;
  float* part_ml = scratch + (size_t)R * nq * NB * d;
  return kvb_decode_attention(q, q_row_stride, k_pages, v_pages, block_table, max_pages, page_size, num_pages,
                              q_start, ctx_len, out, part_o, part_ml, R, nq, nkv, d, scale, window, KB, NB,
                              dtype, status, stream);
}


template <typename T, int D, int GMAX>
static int launch_decode_fused(const void* qkv, int q_row_stride, void* k_pages, void* v_pages, int write_kv,
                               const int* block_table, int max_pages, int page_size, int num_pages,
                               const int* q_start, const int* ctx_len, const float* cos_t, const float* sin_t,
                               int table_len, int rot, void* out, float* part_o, float* part_ml, int* counters,
                               int R, int nq, int nkv, float scale, int window, int KB, int NB, int* status,
                               unsigned long long* trace, cudaStream_t stream) {
  int slots = (4 * kvb_sm_count() + nkv * R - 1) / (nkv * R);
  slots = slots < 1 ? 1 : (slots > NB ? NB : slots);
  dim3 grid(nkv, R, slots);
  const size_t smem = (size_t)2 * 4 * 32 * D * sizeof(T);   // a key tile and a value tile of 128 positions
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_fused_kernel<T, D, GMAX>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  kvb_launch(decode_attention_fused_kernel<T, D, GMAX>, grid, dim3(kDecThreads), smem, stream, (const T*)qkv,
             q_row_stride, (T*)k_pages, (T*)v_pages, write_kv, block_table, max_pages, page_size, num_pages,
             q_start, ctx_len, cos_t, sin_t, table_len, rot, (T*)out, part_o, part_ml, counters, nq, nkv, nq / nkv,
             scale, window, KB, NB, status, trace);
  return kvb_launch_result();
}

// The attention of a decode step in one launch (see decode_attention_fused_kernel).
// qkv: [T, (nq + 2 nkv) d] as the projection wrote it; request r's token is row q_start[r]
// at position ctx_len[r]-1.  write_kv = 0: the layer reads another layer's cache and
// writes nothing.  cos_t/sin_t: [table_len, rot/2] or nullptr for no rotation.
// Scratch: part_o [R, nq, NB, d], part_ml [R, nq, NB, 2] float32; counters [R * nkv] int32,
// zero on entry, left zero.  trace: nullptr, or [blocks, 8] uint64 phase stamps (profiling).
// Same size rules as kvb_decode_attention.
KVB_EXPORT int kvb_decode_attention_fused(const void* qkv, int q_row_stride, void* k_pages, void* v_pages,
                                          int write_kv, const int* block_table, int max_pages, int page_size,
                                          int num_pages, const int* q_start, const int* ctx_len,
                                          const float* cos_t, const float* sin_t, int table_len, int rot, void* out,
                                          float* part_o, float* part_ml, int* counters, int R, int nq, int nkv,
                                          int d, float scale, int window, int KB, int NB, int dtype, int* status,
                                          unsigned long long* trace, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (nkv < 1 || nq % nkv || !kvb_decode_attention_supported(d, nq / nkv) || KB % kDecThreads || NB < 1 ||
      R > 65535 || (rot & 1) || rot > d)
    return KVB_ERR_BAD_SIZE;
  const int G = nq / nkv;
#define KVB_DECF(T, D, GM)                                                                                   \
  return launch_decode_fused<T, D, GM>(qkv, q_row_stride, k_pages, v_pages, write_kv, block_table, max_pages, \
                                       page_size, num_pages, q_start, ctx_len, cos_t, sin_t, table_len, rot,  \
                                       out, part_o, part_ml, counters, R, nq, nkv, scale, window, KB, NB,     \
                                       status, trace, stream)
#define KVB_DECF_D(T, D) do { if (G <= 2) KVB_DECF(T, D, 2); else if (G <= 4) KVB_DECF(T, D, 4); else KVB_DECF(T, D, 8); } while (0)
#define KVB_DECF_T(T) do { if (d == 32) KVB_DECF_D(T, 32); else if (d == 64) KVB_DECF_D(T, 64); else KVB_DECF_D(T, 128); } while (0)
  if (dtype == KVB_BF16) KVB_DECF_T(__nv_bfloat16);
  if (dtype == KVB_F32) KVB_DECF_T(float);
  return KVB_ERR_BAD_DTYPE;
}
