// Tensor-core attention over the paged cache for bfloat16 steps that carry runs of
// query tokens (prompt portions, alone or beside single decode tokens).
//
// A block owns a tile of 64 query rows: `tokens_per_tile` consecutive tokens of one
// request times the (padded) group of query heads that share one key/value head, so a
// key/value tile is fetched once for the whole group.  It walks the request's keys in
// tiles of 64, from the first key any of its rows may read to the last: pages are
// gathered through the block table with 16-byte cp.async copies into swizzled shared
// memory, two tiles in flight; scores and the weighted sum of values run on
// mma.sync m16n8k16 (bfloat16 in, float32 accumulate); the softmax is the running
// max/sum form in float32 (upstream's recurrence, base/src/kernels.cu:436-453, on its
// packed-prompt kernel base/src/kernels.cu:361-466, which reads the step's own keys and
// therefore cannot continue a prompt; this one reads the cache).
// Causal limit per row: key <= position of the row's token; with a window also
// key > position - window.
#include "common.cuh"

#include <math_constants.h>

namespace {

constexpr int BN = 64;   // keys per tile
// Query rows per block: 16 per warp.  Eight warps (128 rows) when the step has enough
// query tiles to fill the GPU with them, four warps (64 rows) otherwise.

__device__ __forceinline__ void cp_async_16_zfill(void* smem_dst, const void* gmem_src, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;  // src-size 0: the 16 bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a [rows][D] bfloat16 tile whose
// chunks are XOR-swizzled with the row, so that the 8 rows of an 8x8 matrix fall into
// 8 different bank groups.
template <int D> __device__ __forceinline__ int swz(int row, int chunk) {
  return row * (D * 2) + ((chunk ^ (row & 7)) << 4);
}

struct TileDesc { int req, t0, n_tok, pad; };

template <int D, int NW>
__global__ void __launch_bounds__(NW * 32, (D == 64 ? 16 : 8) / NW)
paged_flash_attention_kernel(const __nv_bfloat16* __restrict__ q_base, int q_row_stride,
                             const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                             const int* __restrict__ block_table, int max_pages, int page_shift, int num_pages,
                             const int* __restrict__ positions, const TileDesc* __restrict__ tiles,
                             __nv_bfloat16* __restrict__ out, int nq, int nkv, int G, int gp_shift,
                             float scale_log2, int window, int* status) {
  constexpr int BM = NW * 16;       // query rows of this block
  constexpr int kThreads = NW * 32;
  constexpr int CPK = D / 8;        // 16-byte chunks per row
  constexpr int KSTEPS = D / 16;    // k-steps of the score product
  constexpr int DT = D / 8;         // n-tiles of the output
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                         // [BM][D]
  unsigned char* k_s = q_s + BM * D * 2;             // [2][BN][D]
  unsigned char* v_s = k_s + 2 * BN * D * 2;         // [2][BN][D]
  int* row_pos = reinterpret_cast<int*>(v_s + 2 * BN * D * 2);  // [BM] position of each row's token, -1 if none

  pdl_trigger();
  pdl_wait();
  const TileDesc tile = tiles[blockIdx.x];
  const int hk = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gp = 1 << gp_shift;
  const int page_mask = (1 << page_shift) - 1;
  const int* table = block_table + (size_t)tile.req * max_pages;

  if (tid < BM) {
    const int ti = tid >> gp_shift, hi = tid & (gp - 1);
    row_pos[tid] = (ti < tile.n_tok && hi < G) ? positions[tile.t0 + ti] : -1;
  }
  const int pos_first = positions[tile.t0];
  const int pos_last = positions[tile.t0 + tile.n_tok - 1];
  const int k_hi = pos_last + 1;                                    // keys [.., k_hi) are read
  const int k_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int first_tile = k_lo / BN, last_tile = (k_hi - 1) / BN;

  // ---- loaders ------------------------------------------------------------------
  auto load_q = [&]() {
#pragma unroll
    for (int i = 0; i < BM * CPK / kThreads; ++i) {
      const int c = i * kThreads + tid;
      const int row = c / CPK, part = c % CPK;
      const int ti = row >> gp_shift, hi = row & (gp - 1);
      const bool ok = ti < tile.n_tok && hi < G;
      const __nv_bfloat16* src = q_base + (size_t)(tile.t0 + (ok ? ti : 0)) * q_row_stride +
                                 (size_t)(hk * G + (ok ? hi : 0)) * D + part * 8;
      cp_async_16_zfill(q_s + swz<D>(row, part), src, ok);
    }
  };
  // A key's row is copied by kThreads / BN threads, so that its page is looked up once per
  // thread and tile.
  auto load_kv = [&](int t, int buf) {
    constexpr int TPK = kThreads / BN;          // threads per key
    constexpr int CPT = CPK / TPK;              // chunks per thread
    unsigned char* kd = k_s + buf * BN * D * 2;
    unsigned char* vd = v_s + buf * BN * D * 2;
    const int key = tid / TPK, part0 = (tid % TPK) * CPT;
    const int j = t * BN + key;
    bool ok = j < k_hi && j >= k_lo;
    size_t off = 0;
    if (ok) {
      const int lp = j >> page_shift;
      const int page = lp < max_pages ? __ldg(table + lp) : -1;
      if (page < 0 || page >= num_pages) {
        atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
        ok = false;
      } else {
        off = ((((size_t)page * nkv + hk) << page_shift) + (j & page_mask)) * D;
      }
    }
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      const int part = part0 + i;
      cp_async_16_zfill(kd + swz<D>(key, part), k_pages + off + part * 8, ok);
      cp_async_16_zfill(vd + swz<D>(key, part), v_pages + off + part * 8, ok);
    }
  };

  load_q();
  load_kv(first_tile, 0);
  cp_async_commit();

  // ---- per-thread state: rows r0 = warp*16 + lane/4 and r0 + 8 ---------------------
  float o[DT][4];
#pragma unroll
  for (int n = 0; n < DT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};
  unsigned qf[KSTEPS][4];
  const int r0 = warp * 16 + (lane >> 2);
  int pos_r[2], lo_r[2];

  for (int t = first_tile; t <= last_tile; ++t) {
    const int buf = (t - first_tile) & 1;
    if (t < last_tile) {
      load_kv(t + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (t == first_tile) {
      // query fragments stay in registers for the whole walk
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk)
        ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3],
                    q_s + swz<D>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));
      pos_r[0] = row_pos[r0]; pos_r[1] = row_pos[r0 + 8];
      lo_r[0] = window > 0 ? max(0, pos_r[0] - window + 1) : 0;
      lo_r[1] = window > 0 ? max(0, pos_r[1] - window + 1) : 0;
    }
    const unsigned char* kt = k_s + buf * BN * D * 2;
    const unsigned char* vt = v_s + buf * BN * D * 2;

    // S = Q K^T : 16 rows x 64 keys per warp
    float s[BN / 8][4];
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        unsigned b0, b1, b2, b3;
        // lanes 0-7: keys np*16+l, chunk 2kk | 8-15: same keys, chunk 2kk+1 | 16-23: keys +8, chunk 2kk | 24-31: keys +8, chunk 2kk+1
        const int key = np * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int chunk = kk * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(b0, b1, b2, b3, kt + swz<D>(key, chunk));
        mma_bf16(s[2 * np], qf[kk], b0, b1);
        mma_bf16(s[2 * np + 1], qf[kk], b2, b3);
      }
    }
    // mask and running softmax; scores are kept in units of log2 (scale * log2 e folded in).
    // A tile that lies wholly at or below every row's position and wholly inside every row's
    // window needs no per-element test; the tiles on the diagonal and at the window's edge do.
    const int kbase = t * BN + ((lane & 3) << 1);
    float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
    const bool full = (t * BN + BN - 1 <= min(pos_r[0], pos_r[1])) && (t * BN >= max(lo_r[0], lo_r[1])) &&
                      pos_r[0] >= 0 && pos_r[1] >= 0;
    if (__all_sync(0xffffffffu, full)) {
#pragma unroll
      for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[n][e] *= scale_log2;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = kbase + n * 8 + (e & 1);
          const int rr = e >> 1;
          const bool ok = j <= pos_r[rr] && j >= lo_r[rr];
          s[n][e] = ok ? s[n][e] * scale_log2 : -CUDART_INF_F;
          mx[rr] = fmaxf(mx[rr], s[n][e]);
        }
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
      const float m_new = fmaxf(m_run[rr], mx[rr]);
      m_use[rr] = (m_new == -CUDART_INF_F) ? 0.f : m_new;   // a row with no key yet: keep everything at zero
      corr[rr] = (m_run[rr] == -CUDART_INF_F) ? 0.f : exp2f(m_run[rr] - m_use[rr]);
      m_run[rr] = m_new;
      l_run[rr] *= corr[rr];
    }
#pragma unroll
    for (int n = 0; n < DT; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
    unsigned pf[BN / 16][4];
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
      const float p0 = exp2f(s[n][0] - m_use[0]), p1 = exp2f(s[n][1] - m_use[0]);
      const float p2 = exp2f(s[n][2] - m_use[1]), p3 = exp2f(s[n][3] - m_use[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      // the accumulator layout of two neighbouring score tiles is the A layout of one k-step
      pf[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
      for (int dp = 0; dp < DT / 2; ++dp) {
        unsigned b0, b1, b2, b3;
        // lanes 0-7: keys kk*16+l, chunk 2dp | 8-15: keys +8, chunk 2dp | 16-23: keys kk*16+l, chunk 2dp+1 | 24-31: keys +8, chunk 2dp+1
        const int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int chunk = dp * 2 + (lane >> 4);
        ldmatrix_x4_trans(b0, b1, b2, b3, vt + swz<D>(key, chunk));
        mma_bf16(o[2 * dp], pf[kk], b0, b1);
        mma_bf16(o[2 * dp + 1], pf[kk], b2, b3);
      }
    }
    __syncthreads();  // the buffer just read is filled again by the next iteration's prefetch
  }

  // ---- normalise and store ---------------------------------------------------------
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
    l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = r0 + rr * 8;
    const int ti = row >> gp_shift, hi = row & (gp - 1);
    if (ti >= tile.n_tok || hi >= G) continue;
    const float inv = l_run[rr] > 0.f ? 1.0f / l_run[rr] : 0.f;
    __nv_bfloat16* dst = out + ((size_t)(tile.t0 + ti) * nq + hk * G + hi) * D + ((lane & 3) << 1);
#pragma unroll
    for (int n = 0; n < DT; ++n)
      *reinterpret_cast<unsigned*>(dst + n * 8) = pack_bf16(o[n][rr * 2] * inv, o[n][rr * 2 + 1] * inv);
  }
}

template <int D, int NW>
int launch(const void* q, int q_row_stride, const void* k_pages, const void* v_pages, const int* block_table,
           int max_pages, int page_shift, int num_pages, const int* positions, const void* tiles, int num_tiles,
           void* out, int nq, int nkv, int G, int gp_shift, float scale, int window, int* status,
           cudaStream_t stream) {
  constexpr int BM = NW * 16;
  const size_t smem = (size_t)BM * D * 2 + 4 * (size_t)BN * D * 2 + BM * sizeof(int);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(paged_flash_attention_kernel<D, NW>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(num_tiles, nkv);
  kvb_launch(paged_flash_attention_kernel<D, NW>, grid, dim3(NW * 32), smem, stream, (const __nv_bfloat16*)q,
             q_row_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, max_pages,
             page_shift, num_pages, positions, (const TileDesc*)tiles, (__nv_bfloat16*)out, nq, nkv, G, gp_shift,
             scale * 1.4426950408889634f, window, status);
  return kvb_launch_result();
}

int log2_exact(int x) {
  int s = 0;
  while ((1 << s) < x) ++s;
  return (1 << s) == x ? s : -1;
}

}  // namespace

// 1 when the tensor-core kernel takes these sizes: head size 64 or 128, a group of at
// most 64 query heads per key/value head, a page size that is a power of two.
KVB_EXPORT int kvb_flash_attention_supported(int d, int group, int page_size) {
  return (d == 64 || d == 128) && group >= 1 && group <= 64 && log2_exact(page_size) >= 0;
}

// Query tokens per tile for a group size: rows / the group padded to a power of two, with
// rows = 128 (`wide` != 0) or 64.
KVB_EXPORT int kvb_flash_attention_tokens_per_tile(int group, int wide) {
  int gp = 1;
  while (gp < group) gp <<= 1;
  const int nt = (wide ? 128 : 64) / gp;
  return nt < 1 ? 1 : nt;
}

// tiles: num_tiles x {request row, first token row, tokens (<= tokens_per_tile(group, wide)), 0},
// int32.  The tokens of a tile are consecutive tokens of one request, positions ascending.
// wide: the tiles were cut for 128 query rows per block, else for 64.
// bfloat16 only.  out is [T, nq*d].
KVB_EXPORT int kvb_paged_flash_attention(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                         const int* block_table, int max_pages, int page_size, int num_pages,
                                         const int* positions, const void* tiles, int num_tiles, int wide, void* out,
                                         int nq, int nkv, int d, float scale, int window, int* status,
                                         cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (nkv < 1 || nq % nkv) return KVB_ERR_BAD_SIZE;
  const int G = nq / nkv;
  if (!kvb_flash_attention_supported(d, G, page_size) || nkv > 65535) return KVB_ERR_BAD_SIZE;
  int gp_shift = 0;
  while ((1 << gp_shift) < G) ++gp_shift;
  const int page_shift = log2_exact(page_size);
  if (wide && (128 >> gp_shift) < 1) return KVB_ERR_BAD_SIZE;
#define KVB_FA(D, NW)                                                                                           \
  return launch<D, NW>(q, q_row_stride, k_pages, v_pages, block_table, max_pages, page_shift, num_pages, positions, \
                       tiles, num_tiles, out, nq, nkv, G, gp_shift, scale, window, status, stream)
  if (d == 64) { if (wide) KVB_FA(64, 8); KVB_FA(64, 4); }
  if (wide) KVB_FA(128, 8);
  KVB_FA(128, 4);
}
