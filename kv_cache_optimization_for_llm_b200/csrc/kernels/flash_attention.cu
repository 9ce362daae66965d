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
#include "page_maps.cuh"

#include <cuda.h>
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
  // the last tiles of a request read the most keys: they start first, so that the grid's
  // last blocks to start are short ones
  const TileDesc tile = tiles[gridDim.x - 1 - blockIdx.x];
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

// ---------------------------------------------------------------------------------------------
// The same attention on the 5th-generation tensor cores, for tiles of 128 query rows and head
// size 64.  A block of 256 threads owns one query tile; threads r and r + 128 share row r:
// each takes half of a tile's keys in the softmax and half of the output dims.  Per tile of
// 128 keys:
//   S = Q K^T     one thread issues tcgen05.mma (M 128, N 128, K 16 x 4) from shared memory
//                 into tensor memory; keys and values were gathered through the block table by
//                 16-byte cp.async copies, in the 128-byte-swizzled layout the tensor cores read
//   softmax       every thread reads its half row of S from tensor memory (tcgen05.ld), masks
//                 (only where a warp's rows meet the diagonal or the window's edge), keeps the
//                 running max and sum in float32, and writes its probabilities in bfloat16 to
//                 shared memory, again in the swizzled K-major layout
//   P V           tcgen05.mma (M 128, N 64, K 16 x 4); V is read as the MN-major operand, so
//                 the same [key][dim] tile serves
//   O += P V      accumulates in tensor memory; the rows are rescaled there only when the running
//                 maximum has grown by more than a threshold since the last time.
// The next tile's scores are started as soon as every thread has read this tile's out of
// tensor memory, so they run under this tile's exponentials; keys and values are requested
// one tile ahead; P V of a tile runs under the next tile's softmax.  A block holds 128
// columns of tensor memory and 80 registers per thread, so that three blocks share an SM and
// fill each other's gaps (two blocks with double-buffered scores measured 10 % slower).
// mbarrier waits are bounded: a wait that runs out records
// KVB_STATUS_WAIT_TIMEOUT and the block frees its tensor memory and returns.
namespace tc5 {

constexpr unsigned kSpinLimit = 20u * 1000u * 1000u;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ bool mbar_try_wait(void* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity) {   // false: the limit ran out
  for (unsigned i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tmem_alloc(void* holder, unsigned cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                          unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// 32 consecutive columns of this thread's lane of tensor memory
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float* v) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 64 consecutive columns of this thread's lane of tensor memory: two loads of 32, one wait
__device__ __forceinline__ void tmem_ld32x2(unsigned taddr, float* v) {
  unsigned r[64];
#pragma unroll
  for (int h = 0; h < 2; ++h)
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[32 * h + 0]), "=r"(r[32 * h + 1]), "=r"(r[32 * h + 2]), "=r"(r[32 * h + 3]), "=r"(r[32 * h + 4]),
          "=r"(r[32 * h + 5]), "=r"(r[32 * h + 6]), "=r"(r[32 * h + 7]), "=r"(r[32 * h + 8]), "=r"(r[32 * h + 9]),
          "=r"(r[32 * h + 10]), "=r"(r[32 * h + 11]), "=r"(r[32 * h + 12]), "=r"(r[32 * h + 13]), "=r"(r[32 * h + 14]),
          "=r"(r[32 * h + 15]), "=r"(r[32 * h + 16]), "=r"(r[32 * h + 17]), "=r"(r[32 * h + 18]), "=r"(r[32 * h + 19]),
          "=r"(r[32 * h + 20]), "=r"(r[32 * h + 21]), "=r"(r[32 * h + 22]), "=r"(r[32 * h + 23]), "=r"(r[32 * h + 24]),
          "=r"(r[32 * h + 25]), "=r"(r[32 * h + 26]), "=r"(r[32 * h + 27]), "=r"(r[32 * h + 28]), "=r"(r[32 * h + 29]),
          "=r"(r[32 * h + 30]), "=r"(r[32 * h + 31])
        : "r"(taddr + 32 * h));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// 32 consecutive columns of this thread's lane of tensor memory, written
__device__ __forceinline__ void tmem_st32(unsigned taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 16 consecutive columns of this thread's lane of tensor memory, read and written
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float* v) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st16(unsigned taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle, rows of 128 bytes, groups of 8 rows 1024
// bytes apart, base aligned to 1024 bytes.  The same image is a K-major operand (rows are
// M or N, the 64 elements of a row run along K) or, with the major bit of the instruction
// descriptor set, an MN-major one (rows run along K, the 64 elements of a row along N).
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned addr) {
  return (unsigned long long)((addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

constexpr int BM = 128, BNK = 64, D = 64;
constexpr int kThreads = 256;                // two threads per query row: each takes half of the keys of a tile
constexpr int kQBytes = BM * D * 2;          // [128 rows][64] bfloat16
constexpr int kKVBytes = BNK * D * 2;        // [64 keys][64]
constexpr int kPBytes = BM * BNK * 2;        // [128 rows][64 keys]
constexpr unsigned kTmemCols = 128;          // S: columns 0..63, the output: columns 64..127

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two float32 operations in one instruction (sm_100: fma.rn.f32x2, add.rn.f32x2; each half is the
// IEEE operation of the scalar form) and the maximum of three.  The softmax threads are bound by
// the instructions they issue, not by any one pipe: these halve the multiply-adds and the sums.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)),
        "l"(reinterpret_cast<unsigned long long&>(c)));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__global__ void __launch_bounds__(kThreads, 3)
paged_flash_attention_tc_kernel(const __nv_bfloat16* __restrict__ q_base, int q_row_stride,
                                const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                                const int* __restrict__ block_table, int max_pages, int page_shift, int num_pages,
                                const int* __restrict__ positions, const TileDesc* __restrict__ tiles,
                                __nv_bfloat16* __restrict__ out, int nq, int nkv, int G, int gp_shift,
                                float scale_log2, int window, int* status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* q_s = base;                       // [128 rows][64]
  unsigned char* k_s = q_s + kQBytes;              // [2][64 keys][64]
  unsigned char* v_s = k_s + 2 * kKVBytes;         // [2][64 keys][64]
  unsigned char* p_s = v_s + 2 * kKVBytes;         // [128 rows][64 keys]
  float* mx_s = reinterpret_cast<float*>(p_s + kPBytes);   // [2][128] the halves' row maxima of a tile
  unsigned long long* bar_s = reinterpret_cast<unsigned long long*>(mx_s + 2 * BM);   // [2]: one per S buffer
  unsigned long long* bar_o = bar_s + 2;
  unsigned* tmem_holder = reinterpret_cast<unsigned*>(bar_o + 1);
  int* abort_flag = reinterpret_cast<int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int r = tid & (BM - 1);      // this thread's query row (= its lane of tensor memory)
  const int h = tid >> 7;            // which half of a tile's keys, and of the output dims, it takes
  if (tid == 0) {
    mbar_init(&bar_s[0], 1);
    mbar_init(&bar_s[1], 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(tmem_holder, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = *tmem_holder;
  // only now may the kernel behind this one start: its resident, waiting blocks must not be
  // able to take tensor memory that a block of this grid still needs
  pdl_trigger();
  pdl_wait();

  // the last tiles of a request read the most keys: they start first, so that the grid's
  // last blocks to start are short ones
  const TileDesc tile = tiles[gridDim.x - 1 - blockIdx.x];
  const int hk = blockIdx.y;
  const int gp = 1 << gp_shift;
  const int page_mask = (1 << page_shift) - 1;
  const int* table = block_table + (size_t)tile.req * max_pages;
  const int ti = r >> gp_shift, hi = r & (gp - 1);
  const bool row_ok = ti < tile.n_tok && hi < G;
  const int pos = row_ok ? positions[tile.t0 + ti] : -1;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int pos_first = positions[tile.t0];
  const int pos_last = positions[tile.t0 + tile.n_tok - 1];
  const int k_hi = pos_last + 1;
  const int k_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int first_tile = k_lo / BNK, last_tile = (k_hi - 1) / BNK;
  const int n_tiles = last_tile - first_tile + 1;

  // Loaders.  Query: thread (r, h) brings the 16-byte pieces 4h..4h+3 of row r.  Keys and
  // values: thread j brings pieces 2 (j mod 4), +1 of key j / 4 of a tile; a key's page is
  // looked up when the tile is requested (the tile is not needed before the next tile's turn).
  {
    const __nv_bfloat16* src = q_base + (size_t)(tile.t0 + (row_ok ? ti : 0)) * q_row_stride +
                               (size_t)(hk * G + (row_ok ? hi : 0)) * D;
#pragma unroll
    for (int i = 0; i < 4; ++i) cp_async_16_zfill(q_s + swz<D>(r, 4 * h + i), src + (4 * h + i) * 8, row_ok);
  }
  const int lkey = tid >> 2, lpart = (tid & 3) * 2;
  auto load_tile = [&](int i, unsigned char* dst, const __nv_bfloat16* pages) {   // i-th tile of this block
    const int j = (first_tile + i) * BNK + lkey;
    bool ok = i < n_tiles && j < k_hi && j >= k_lo;
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
    cp_async_16_zfill(dst + swz<D>(lkey, lpart), pages + off + lpart * 8, ok);
    cp_async_16_zfill(dst + swz<D>(lkey, lpart + 1), pages + off + (lpart + 1) * 8, ok);
  };
  // Every thread commits the same groups in the same order, requests or not:
  //   prologue: [Q, K0] [K1] [V0];  tile i: [K(i+2)] after S(i) has been read, [V(i+1)] after P V(i-1) has been.
  load_tile(0, k_s, k_pages);
  cp_async_commit();
  load_tile(1, k_s + kKVBytes, k_pages);
  cp_async_commit();
  load_tile(0, v_s, v_pages);
  cp_async_commit();

  // instruction descriptors: float32 accumulator, bfloat16 operands, N >> 3 at bit 17, M >> 4 at bit 24
  const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BNK >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
  const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) /* B is MN-major */ |
                           ((unsigned)(D >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
  const unsigned lane_base = tmem + ((unsigned)((warp & 3) * 32) << 16);
  const unsigned o_cols = lane_base + 64 + 32 * h;     // this thread's 32 output dims
  const unsigned long long qd = smem_desc_sw128(smem_u32(q_s));
  auto issue_s = [&](int i) {   // S(i) = Q K(i)^T, keys from buffer i mod 2   (one thread)
    const unsigned long long kd = smem_desc_sw128(smem_u32(k_s + (i & 1) * kKVBytes));
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) umma_bf16(tmem, qd + 2 * kk, kd + 2 * kk, idesc_s, kk > 0 ? 1u : 0u);
    umma_commit(&bar_s[0]);
  };

  // The output accumulates in tensor memory over the tiles.  Probabilities are taken against a
  // reference maximum m_ref that follows the running maximum only when that has grown by more
  // than kRescale (in log2 units): any reference gives the same softmax as long as nothing
  // overflows (probabilities stay below 2^kRescale), and the rows of the output then need
  // rescaling (read, multiply, write back) only a few times per sequence.
  constexpr float kRescale = 8.0f;
  float m_ref = -CUDART_INF_F, l_run = 0.f;   // l_run: the sum over this thread's half of the keys
  bool failed = false;

  // S(0) is started here; S(i+1) as soon as every thread has read S(i) out of tensor memory,
  // so that it runs under tile i's exponentials.
  cp_async_wait<2>();                      // Q and K0
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  if (tid == 0) { tc_fence_after(); issue_s(0); }

  for (int i = 0; i < n_tiles; ++i) {
    const int t = first_tile + i;
    // ---- S(i): this thread's 32 scores, kept in registers
    if (!failed && !mbar_wait(&bar_s[0], (unsigned)i & 1u)) { failed = true; *abort_flag = 1; }
    tc_fence_after();
    float v[32];
    tmem_ld32(lane_base + 32 * h, v);
    load_tile(i + 2, k_s + (i & 1) * kKVBytes, k_pages);   // K(i) has been read: its buffer takes K(i+2)
    cp_async_commit();

    const int kb = t * BNK + 32 * h;       // first key of this thread's half
    const bool full = pos >= 0 && t * BNK + BNK - 1 <= pos && t * BNK >= lo;
    const bool plain = __all_sync(0xffffffffu, full);   // no key of the tile is masked for any row of the warp
    float mx = -CUDART_INF_F;
    if (plain) {
#pragma unroll
      for (int j = 0; j < 32; ++j) mx = fmaxf(mx, v[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int key = kb + j;
        if (!(key <= pos && key >= lo)) v[j] = -CUDART_INF_F;
        mx = fmaxf(mx, v[j]);
      }
    }
    mx_s[h * BM + r] = mx * scale_log2;    // the scale is positive: the maximum commutes with it
    cp_async_wait<2>();                    // K(i+1) is here (newer: V(i), or V(i) and ... see the group list above)
    fence_async_smem();
    tc_fence_before();
    __syncthreads();                       // everybody has read S(i): the next tile's scores may overwrite it
    if (*abort_flag) { failed = true; break; }
    if (tid == 0 && i + 1 < n_tiles) { tc_fence_after(); issue_s(i + 1); }
    const float m_new = fmaxf(m_ref, fmaxf(mx_s[r], mx_s[BM + r]));
    const bool grow = m_new > m_ref + kRescale;     // also: the row's first key (m_ref is -inf)

    // ---- P V(i-1), which ran while this tile's scores were read, has to be over before the
    // output may be rescaled and before P is written again
    if (i > 0) {
      if (!failed && !mbar_wait(bar_o, (unsigned)(i - 1) & 1u)) { failed = true; *abort_flag = 1; }
      tc_fence_after();
    }
    load_tile(i + 1, v_s + ((i + 1) & 1) * kKVBytes, v_pages);   // V(i-1) has been read: its buffer takes V(i+1)
    cp_async_commit();
    if (__any_sync(0xffffffffu, grow)) {
      const float corr = !grow ? 1.0f : (m_ref == -CUDART_INF_F ? 0.f : ex2(m_ref - m_new));
      if (i > 0) {                                  // before the first product the output holds nothing yet
        float ov[32];
        tmem_ld32(o_cols, ov);
#pragma unroll
        for (int j = 0; j < 32; ++j) ov[j] *= corr;
        tmem_st32(o_cols, ov);
      }
      l_run *= corr;
      if (grow) m_ref = m_new;
    }
    const float m_use = (m_ref == -CUDART_INF_F) ? 0.f : m_ref;   // a row with no key yet: everything stays zero

    // ---- P(i): probabilities of this thread's 32 keys, bfloat16, pieces 4h..4h+3 of row r
    unsigned pk[16];
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      // a masked score is -inf: its probability comes out as zero
      const float p0 = ex2(fmaf(v[j], scale_log2, -m_use)), p1 = ex2(fmaf(v[j + 1], scale_log2, -m_use));
      l_run += p0 + p1;
      pk[j >> 1] = pack_bf16(p0, p1);
    }
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4)
      *reinterpret_cast<uint4*>(p_s + swz<D>(r, 4 * h + q4)) =
          make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);

    // ---- P V(i) is started and left to run
    cp_async_wait<2>();                    // V(i) is here (newer: K(i+2), V(i+1))
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) { failed = true; break; }
    if (tid == 0) {
      tc_fence_after();
      const unsigned long long pd = smem_desc_sw128(smem_u32(p_s));
      const unsigned long long vd = smem_desc_sw128(smem_u32(v_s + (i & 1) * kKVBytes));
#pragma unroll
      for (int kk = 0; kk < BNK / 16; ++kk)   // 16 keys per step: 32 bytes along a row of P, 16 rows of V
        umma_bf16(tmem + 64, pd + 2 * kk, vd + 128 * kk, idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
      umma_commit(bar_o);
    }
  }
  float o[D / 2];
#pragma unroll
  for (int j = 0; j < D / 2; ++j) o[j] = 0.f;
  if (!failed && n_tiles > 0) {
    if (!mbar_wait(bar_o, (unsigned)(n_tiles - 1) & 1u)) { failed = true; *abort_flag = 1; }
    tc_fence_after();
    tmem_ld32(o_cols, o);
  }
  cp_async_wait<0>();
  __syncthreads();
  if (*abort_flag) failed = true;

  if (failed) {
    if (tid == 0) atomicCAS(status, 0, KVB_STATUS_WAIT_TIMEOUT);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let products that may still run finish
  } else {
    // the row's sum is the sum of its two halves
    mx_s[h * BM + r] = l_run;
    __syncthreads();
    const float l = mx_s[r] + mx_s[BM + r];
    if (row_ok) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = out + ((size_t)(tile.t0 + ti) * nq + hk * G + hi) * D + 32 * h;
#pragma unroll
      for (int j = 0; j < D / 2; j += 8)
        *reinterpret_cast<uint4*>(dst + j) =
            make_uint4(pack_bf16(o[j] * inv, o[j + 1] * inv), pack_bf16(o[j + 2] * inv, o[j + 3] * inv),
                       pack_bf16(o[j + 4] * inv, o[j + 5] * inv), pack_bf16(o[j + 6] * inv, o[j + 7] * inv));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

int launch(const void* q, int q_row_stride, const void* k_pages, const void* v_pages, const int* block_table,
           int max_pages, int page_shift, int num_pages, const int* positions, const void* tiles, int num_tiles,
           void* out, int nq, int nkv, int G, int gp_shift, float scale, int window, int* status,
           cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)kQBytes + 4 * (size_t)kKVBytes + kPBytes + 2 * BM * 4 + 64;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(paged_flash_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid(num_tiles, nkv);
  kvb_launch(paged_flash_attention_tc_kernel, grid, dim3(kThreads), smem, stream, (const __nv_bfloat16*)q, q_row_stride,
             (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, max_pages, page_shift,
             num_pages, positions, (const TileDesc*)tiles, (__nv_bfloat16*)out, nq, nkv, G, gp_shift,
             scale * 1.4426950408889634f, window, status);
  return kvb_launch_result();
}


// ---------------------------------------------------------------- the same, with roles
// Warp-specialised form (224 threads, two blocks per SM):
//   warp 0        the loader: finds the pages of a 64-key tile through the block table and
//                 requests them as TMA boxes (cp.async.bulk.tensor, 128-byte swizzle) into rings
//                 of three key and three value stages; the copies count their bytes on the
//                 stage's mbarrier, so nobody waits on the loader itself;
//   warps 1, 2    one thread each issues tcgen05.mma: warp 1 the scores S(i) = Q K(i)^T into the
//                 score buffer that the softmax warps have read already (two tiles ahead),
//                 warp 2 the products O += P(i) V(i) as soon as the probabilities of tile i are
//                 in shared memory; tcgen05.commit hands stages and buffers back;
//   warps 3..6    the softmax: a thread owns one query row (its lane of tensor memory) and all
//                 64 keys of a tile, so the row's maximum and sum need no exchange; scores out
//                 of tensor memory in halves of 32, mask on the diagonal and at the window's
//                 edge only, probabilities in bfloat16 to one of two swizzled buffers, the
//                 output rescaled in tensor memory only when the running maximum has grown by
//                 2^8.
// Tensor memory: scores in columns 0..63 and 64..127 (double-buffered), the output from 128 on;
// 256 columns per block, two blocks per SM at both head sizes (at 128 with two key stages, one
// value stage and one buffer of probabilities: 96 KB of shared memory).  The roles meet on mbarriers only; every wait is
// bounded and gives up early when another role has given up.  Needs pages of at least 8 rows
// (a TMA box of 8 x 64 bfloat16 is the smallest that the 128-byte swizzle repeats over) and
// 16-byte aligned page pools.
constexpr int kWsThreads = 224;
constexpr int kStages = 3;
constexpr unsigned kWsTmemCols = 256;

struct WsBars {
  unsigned long long q_full, k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  unsigned long long s_full[2], s_free[2], p_full[2], o_done[2];
};

__device__ __forceinline__ void mbar_arrive(void* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// Bounded wait that also ends when another role of the block has given up.  false: gave up.
__device__ __forceinline__ bool mbar_test_wait(void* bar, unsigned parity) {   // a look, no suspension
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool wait_or_abort(void* bar, unsigned parity, volatile int* abort_flag) {
  if (mbar_test_wait(bar, parity)) return true;
  for (unsigned i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// DH: the head size, 64 or 128.  Operands wider than 64 elements lie in shared memory as sub-tiles of
// 64 columns side by side (a row of the 128-byte swizzle holds 64 bfloat16): Q, K and V have DH / 64
// of them.  The scores take DH / 16 products of 16 along the head, the output DH / 64 times 4
// products of 64 columns each; tensor memory holds the output in columns 128 .. 128 + DH.
template <int DH>
__global__ void __launch_bounds__(kWsThreads, 2)
paged_flash_attention_ws_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                int box_rows, const __nv_bfloat16* __restrict__ q_base, int q_row_stride,
                                const int* __restrict__ block_table, int max_pages, int page_shift, int num_pages,
                                const int* __restrict__ positions, const TileDesc* __restrict__ tiles,
                                __nv_bfloat16* __restrict__ out, int nq, int nkv, int G, int gp_shift,
                                float scale_log2, int window, int* status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kSub = DH / 64;                        // sub-tiles of 64 columns in Q, K and V
  constexpr int kQSub = BM * 128, kKVSub = BNK * 128;  // bytes of one sub-tile: rows x 128 bytes
  constexpr int kQB = kSub * kQSub, kKVB = kSub * kKVSub;
  // Stages of keys and of values and buffers of probabilities: 3, 3 and 2 at head size 64; 2, 1 and 1
  // at head size 128, where a block then takes 96 KB and two of them fit an SM (eight softmax warps
  // instead of four).  One value stage is enough: V(i) is requested when P V(i - 1) is over, at the
  // start of the softmax of tile i, and is needed at its end.
  constexpr int kKSt = DH == 64 ? 3 : 2, kVSt = DH == 64 ? 3 : 1, kPB = DH == 64 ? 2 : 1;
  unsigned char* q_s = base;                           // [DH/64][128 rows][64]
  unsigned char* k_s = q_s + kQB;                      // [kKSt][DH/64][64 keys][64]
  unsigned char* v_s = k_s + kKSt * kKVB;              // [kVSt][DH/64][64 keys][64]
  unsigned char* p_s = v_s + kVSt * kKVB;              // [kPB][128 rows][64 keys]
  WsBars* bars = reinterpret_cast<WsBars*>(p_s + kPB * kPBytes);
  unsigned* tmem_holder = reinterpret_cast<unsigned*>(bars + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(&bars->q_full, 4);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->k_full[s], 1); mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1); mbar_init(&bars->v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->s_full[b], 1); mbar_init(&bars->s_free[b], 4);
      mbar_init(&bars->p_full[b], 4); mbar_init(&bars->o_done[b], 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(tmem_holder, kWsTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = *tmem_holder;
  // only now may the kernel behind this one start: its resident, waiting blocks must not be
  // able to take tensor memory that a block of this grid still needs
  pdl_trigger();
  pdl_wait();

  // Blocks start in the order of their linear index.  The last tiles of a request read the most
  // keys: they come first, for every key/value head, so that the blocks that start last are
  // short ones.
  const int lin = blockIdx.y * gridDim.x + blockIdx.x;
  const TileDesc tile = tiles[gridDim.x - 1 - lin / nkv];
  const int hk = lin % nkv;
  const int gp = 1 << gp_shift;
  const int page_mask = (1 << page_shift) - 1;
  const int* table = block_table + (size_t)tile.req * max_pages;
  const int pos_first = positions[tile.t0];
  const int pos_last = positions[tile.t0 + tile.n_tok - 1];
  const int k_hi = pos_last + 1;
  const int k_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int first_tile = k_lo / BNK, last_tile = (k_hi - 1) / BNK;
  const int n_tiles = last_tile - first_tile + 1;
  bool failed = false;

  if (warp == 0) {
    // ---------------------------------------------------------------- loader
    // A tile of 64 keys is 64 / box_rows boxes of the tensor map over the pages
    // ([pages x kv heads x page_size rows][64]; box_rows = min(page size, 64)), each found
    // through the block table and copied by TMA with the 128-byte swizzle the products read;
    // the copies count their bytes on the tile's barrier.  Lane 0 waits and issues; the warp
    // reads the block table 32 boxes at a time, one entry per lane, and hands lane 0 the pages
    // by shuffle, so that no copy waits for a load of its own.  A box that no row may see and
    // that has no page is requested beyond the end of the map, where TMA delivers zeros.  Keys
    // run two tiles ahead of values: a key stage is free again when the scores of its tile are
    // done, a value stage only when the tile's P V is.
    const int total_rows = (num_pages * nkv) << page_shift;
    const int n_box = BNK / box_rows;                 // 1, 2, 4 or 8: a tile never straddles 32 boxes
    const int first_box = first_tile * n_box;
    auto pages_of = [&](int chunk) -> int {           // this lane's entry of boxes 32 chunk .. 32 chunk + 31 of the block
      const int lp = (int)(((long long)(first_box + chunk * 32 + lane) * box_rows) >> page_shift);
      return lp < max_pages ? __ldg(table + lp) : -1;
    };
    auto request = [&](int i, int pg, unsigned char* dst, const CUtensorMap* map, void* bar) {
      if (lane == 0) mbar_expect_tx(bar, kKVB);
      __syncwarp();                                              // the bytes are expected before any copy can report
      const int page = __shfl_sync(0xffffffffu, pg, (i * n_box + lane) & 31);
      if (lane < n_box) {                                        // lane c requests box c of the tile
        const int kj = (first_tile + i) * BNK + lane * box_rows;
        int row = total_rows;                                    // zeros
        if (page >= 0 && page < num_pages) {
          row = (((page * nkv) + hk) << page_shift) + (kj & page_mask);
        } else if (kj < k_hi && kj + box_rows > k_lo) {
          atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);        // keys that a row reads
        }
#pragma unroll
        for (int sub = 0; sub < kSub; ++sub)                     // columns 64 sub .. 64 sub + 63 of the box's rows
          tma_load_2d(dst + sub * kKVSub + lane * box_rows * 128, map, 64 * sub, row, bar);
      }
    };
    int pg_k = -1, pg_v = -1, chunk_k = -1, chunk_v = -1;
    for (int it = 0; it < n_tiles + 2; ++it) {
      const int kt = it, vt = it - 2;
      if (kt < n_tiles) {
        const int chunk = (kt * n_box) >> 5;
        if (chunk != chunk_k) { pg_k = pages_of(chunk); chunk_k = chunk; }
        if (lane == 0 && kt >= kKSt &&
            !wait_or_abort(&bars->k_empty[kt % kKSt], (unsigned)(kt / kKSt - 1) & 1u, abort_flag))
          failed = true;
        failed = __shfl_sync(0xffffffffu, (int)failed, 0) != 0;
        if (failed) break;
        request(kt, pg_k, k_s + (kt % kKSt) * kKVB, &map_k, &bars->k_full[kt % kKSt]);
      }
      if (vt >= 0) {
        const int chunk = (vt * n_box) >> 5;
        if (chunk != chunk_v) { pg_v = pages_of(chunk); chunk_v = chunk; }
        if (lane == 0 && vt >= kVSt &&
            !wait_or_abort(&bars->v_empty[vt % kVSt], (unsigned)(vt / kVSt - 1) & 1u, abort_flag))
          failed = true;
        failed = __shfl_sync(0xffffffffu, (int)failed, 0) != 0;
        if (failed) break;
        request(vt, pg_v, v_s + (vt % kVSt) * kKVB, &map_v, &bars->v_full[vt % kVSt]);
      }
    }
  } else if (warp <= 2) {
    // ---------------------------------------------------------------- tcgen05.mma issuers
    // Two threads, so that neither product waits behind the other's barriers: lane 0 issues the
    // scores, lane 1 the P V products (in order: the output accumulates).
    const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BNK >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
    const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) /* B is MN-major */ |
                             ((unsigned)(64 >> 3) << 17) | ((unsigned)(BM >> 4) << 24);   // 64 output columns at a time
    if (warp == 1 && lane == 0) {
      if (!wait_or_abort(&bars->q_full, 0, abort_flag)) failed = true;
      for (int i = 0; i < n_tiles && !failed; ++i) {
        // S(i) = Q K(i)^T into score buffer i mod 2, which the softmax has read (tile i - 2)
        if (!wait_or_abort(&bars->k_full[i % kKSt], (unsigned)(i / kKSt) & 1u, abort_flag)) { failed = true; break; }
        if (i >= 2 && !wait_or_abort(&bars->s_free[i & 1], (unsigned)((i - 2) >> 1) & 1u, abort_flag)) { failed = true; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {   // 16 of the head per step: sub-tile kk / 4, 32 bytes further along its rows
          const unsigned long long qd = smem_desc_sw128(smem_u32(q_s + (kk >> 2) * kQSub));
          const unsigned long long kd = smem_desc_sw128(smem_u32(k_s + (i % kKSt) * kKVB + (kk >> 2) * kKVSub));
          umma_bf16(tmem + 64 * (i & 1), qd + 2 * (kk & 3), kd + 2 * (kk & 3), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->k_empty[i % kKSt]);
        umma_commit(&bars->s_full[i & 1]);
      }
    } else if (warp == 2 && lane == 0) {
      for (int j = 0; j < n_tiles && !failed; ++j) {
        // O += P(j) V(j)
        if (!wait_or_abort(&bars->p_full[j % kPB], (unsigned)(j / kPB) & 1u, abort_flag)) { failed = true; break; }
        if (!wait_or_abort(&bars->v_full[j % kVSt], (unsigned)(j / kVSt) & 1u, abort_flag)) { failed = true; break; }
        tc_fence_after();
        const unsigned long long pd = smem_desc_sw128(smem_u32(p_s + (j % kPB) * kPBytes));
#pragma unroll
        for (int sub = 0; sub < kSub; ++sub) {    // output columns 64 sub .. 64 sub + 63 from V's sub-tile
          const unsigned long long vd = smem_desc_sw128(smem_u32(v_s + (j % kVSt) * kKVB + sub * kKVSub));
#pragma unroll
          for (int kk = 0; kk < BNK / 16; ++kk)   // 16 keys per step: 32 bytes along a row of P, 16 rows of V
            umma_bf16(tmem + 128 + 64 * sub, pd + 2 * kk, vd + 128 * kk, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bars->v_empty[j % kVSt]);
        umma_commit(&bars->o_done[j & 1]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax
    const int quarter = warp & 3;                   // the lanes of tensor memory this warp may read
    const int r = quarter * 32 + lane;              // query row
    const int ti = r >> gp_shift, hi = r & (gp - 1);
    const bool row_ok = ti < tile.n_tok && hi < G;
    const int pos = row_ok ? positions[tile.t0 + ti] : -1;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    {
      const __nv_bfloat16* src = q_base + (size_t)(tile.t0 + (row_ok ? ti : 0)) * q_row_stride +
                                 (size_t)(hk * G + (row_ok ? hi : 0)) * DH;
#pragma unroll
      for (int i = 0; i < DH / 8; ++i) cp_async_16_zfill(q_s + (i >> 3) * kQSub + swz<64>(r, i & 7), src + i * 8, row_ok);
      cp_async_commit();
      cp_async_wait<0>();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->q_full);
    }
    const unsigned lane_base = tmem + ((unsigned)(quarter * 32) << 16);
    const unsigned o_cols = lane_base + 128;
    constexpr float kRescale = 8.0f;
    float m_ref = -CUDART_INF_F, l_run = 0.f;
    for (int i = 0; i < n_tiles; ++i) {
      const int b = i & 1;
      const int t = first_tile + i;
      if (!wait_or_abort(&bars->s_full[b], (unsigned)(i >> 1) & 1u, abort_flag)) { failed = true; break; }
      tc_fence_after();
      // The row's 64 scores are read once, both halves requested before either is waited for, and
      // stay in registers through the maximum and the probabilities (106 + 32 registers: two blocks
      // per SM still fit).
      const int kb = t * BNK;
      const bool full = pos >= 0 && kb + BNK - 1 <= pos && kb >= lo;
      const bool plain = __all_sync(0xffffffffu, full);
      float v[64];
      tmem_ld32x2(lane_base + 64 * b, v);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->s_free[b]);    // this warp has read its rows of S(i)
      if (!plain) {
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const int key = kb + j;
          if (!(key <= pos && key >= lo)) v[j] = -CUDART_INF_F;
        }
      }
      float m8[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) m8[c] = max3(v[c], v[8 + c], v[16 + c]);
#pragma unroll
      for (int j = 24; j < 56; j += 16) {
#pragma unroll
        for (int c = 0; c < 8; ++c) m8[c] = max3(m8[c], v[j + c], v[j + 8 + c]);
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) m8[c] = fmaxf(m8[c], v[56 + c]);
      const float mx = max3(max3(m8[0], m8[1], m8[2]), max3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7]));
      const float m_new = fmaxf(m_ref, mx * scale_log2);   // the scale is positive: the maximum commutes with it
      const bool grow = m_new > m_ref + kRescale;          // also: the row's first key (m_ref is -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float corr = !grow ? 1.0f : (m_ref == -CUDART_INF_F ? 0.f : ex2(m_ref - m_new));
        if (i > 0) {
          // every product into the output so far has to be over; P V(i) is not issued before this
          // thread's probabilities of tile i are written
          if (!wait_or_abort(&bars->o_done[(i - 1) & 1], (unsigned)((i - 1) >> 1) & 1u, abort_flag)) { failed = true; break; }
          tc_fence_after();
#pragma unroll
          for (int part = 0; part < DH / 16; ++part) {
            float ov[16];
            tmem_ld16(o_cols + 16 * part, ov);
#pragma unroll
            for (int j = 0; j < 16; ++j) ov[j] *= corr;
            tmem_st16(o_cols + 16 * part, ov);
          }
        }
        l_run *= corr;
        if (grow) m_ref = m_new;
      }
      const float m_use = (m_ref == -CUDART_INF_F) ? 0.f : m_ref;   // a row with no key yet: everything stays zero
      // the buffer of P(i) was read by P V(i - kPB)
      if (i >= kPB && !wait_or_abort(&bars->o_done[(i - kPB) & 1], (unsigned)((i - kPB) >> 1) & 1u, abort_flag)) { failed = true; break; }
      unsigned char* pb = p_s + (i % kPB) * kPBytes;
      float2 l2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};   // the tile's sum in four chains, added up in a fixed order
      const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(-m_use, -m_use);
#pragma unroll
      for (int q8 = 0; q8 < 8; ++q8) {       // piece q8 of row r of P: keys 8 q8 .. 8 q8 + 7
        unsigned pk[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // a masked score is -inf: its probability comes out as zero
          const float2 t = ffma2(make_float2(v[8 * q8 + 2 * j], v[8 * q8 + 2 * j + 1]), sc2, nm2);
          const float2 pr = make_float2(ex2(t.x), ex2(t.y));
          l2[j & 1] = fadd2(l2[j & 1], pr);
          pk[j] = pack_bf16(pr.x, pr.y);
        }
        *reinterpret_cast<uint4*>(pb + swz<64>(r, q8)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l_run += (l2[0].x + l2[0].y) + (l2[1].x + l2[1].y);
      fence_async_smem();
      tc_fence_before();     // orders the rescaled output before the product that the arrival lets go
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[i % kPB]);
    }
    if (!failed) {
      if (!wait_or_abort(&bars->o_done[(n_tiles - 1) & 1], (unsigned)((n_tiles - 1) >> 1) & 1u, abort_flag)) failed = true;
    }
    if (!failed) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      __nv_bfloat16* dst = out + ((size_t)(tile.t0 + ti) * nq + hk * G + hi) * DH;
#pragma unroll
      for (int half = 0; half < DH / 32; ++half) {
        float o[32];
        tmem_ld32(o_cols + 32 * half, o);
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8)
            *reinterpret_cast<uint4*>(dst + 32 * half + j) =
                make_uint4(pack_bf16(o[j] * inv, o[j + 1] * inv), pack_bf16(o[j + 2] * inv, o[j + 3] * inv),
                           pack_bf16(o[j + 4] * inv, o[j + 5] * inv), pack_bf16(o[j + 6] * inv, o[j + 7] * inv));
        }
      }
    }
  }
  if (failed) *abort_flag = 1;
  cp_async_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) atomicCAS(status, 0, KVB_STATUS_WAIT_TIMEOUT);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let products that may still run finish
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem, kWsTmemCols);
}

using kvb_page_maps::pages_map;

template <int DH>
int launch_ws(const void* q, int q_row_stride, const void* k_pages, const void* v_pages, const int* block_table,
              int max_pages, int page_shift, int num_pages, const int* positions, const void* tiles, int num_tiles,
              void* out, int nq, int nkv, int G, int gp_shift, float scale, int window, int* status,
              cudaStream_t stream) {
  const int page_size = 1 << page_shift;
  const int box_rows = page_size < BNK ? page_size : BNK;
  const long long rows = (long long)num_pages * nkv * page_size;
  if (rows >= (1ll << 31)) return KVB_ERR_BAD_SIZE;
  CUtensorMap mk, mv;
  int e = pages_map(&mk, k_pages, rows, box_rows, DH);
  if (e) return e;
  e = pages_map(&mv, v_pages, rows, box_rows, DH);
  if (e) return e;
  constexpr int kKSt = DH == 64 ? 3 : 2, kVSt = DH == 64 ? 3 : 1, kPB = DH == 64 ? 2 : 1;   // as in the kernel
  const size_t smem = 1024 + (size_t)BM * DH * 2 + (kKSt + kVSt) * (size_t)BNK * DH * 2 + kPB * kPBytes + sizeof(WsBars) + 64;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t ce = cudaFuncSetAttribute(paged_flash_attention_ws_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    // two blocks per SM need the largest shared-memory configuration
    ce = cudaFuncSetAttribute(paged_flash_attention_ws_kernel<DH>, cudaFuncAttributePreferredSharedMemoryCarveout,
                              (int)cudaSharedmemCarveoutMaxShared);
    if (ce != cudaSuccess) return (int)ce;
    attr_set = true;
  }
  dim3 grid(num_tiles, nkv);
  kvb_launch(paged_flash_attention_ws_kernel<DH>, grid, dim3(kWsThreads), smem, stream, mk, mv, box_rows,
             (const __nv_bfloat16*)q, q_row_stride, block_table, max_pages, page_shift,
             num_pages, positions, (const TileDesc*)tiles, (__nv_bfloat16*)out, nq, nkv, G, gp_shift,
             scale * 1.4426950408889634f, window, status);
  return kvb_launch_result();
}

}  // namespace tc5

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
// wide: 0: the tiles were cut for 64 query rows per block; 1: for 128; 2: for 128, and the
// kernel is the tcgen05 form (head size 64 only); 3: for 128, the tcgen05 form with roles
// (head size 64 or 128, pages of at least 8 rows, page pools aligned to 16 bytes).
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
  if (wide == 3) {   // tcgen05 form with roles
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (q_row_stride & 7) || page_size < 8 ||
        (reinterpret_cast<uintptr_t>(k_pages) & 15) || (reinterpret_cast<uintptr_t>(v_pages) & 15))
      return KVB_ERR_BAD_SIZE;
    if (d == 64)
      return tc5::launch_ws<64>(q, q_row_stride, k_pages, v_pages, block_table, max_pages, page_shift, num_pages,
                                positions, tiles, num_tiles, out, nq, nkv, G, gp_shift, scale, window, status, stream);
    return tc5::launch_ws<128>(q, q_row_stride, k_pages, v_pages, block_table, max_pages, page_shift, num_pages,
                               positions, tiles, num_tiles, out, nq, nkv, G, gp_shift, scale, window, status, stream);
  }
  if (wide == 2) {   // tcgen05 form
    if (d != 64 || (reinterpret_cast<uintptr_t>(q) & 15) || (q_row_stride & 7)) return KVB_ERR_BAD_SIZE;
    return tc5::launch(q, q_row_stride, k_pages, v_pages, block_table, max_pages, page_shift, num_pages, positions,
                       tiles, num_tiles, out, nq, nkv, G, gp_shift, scale, window, status, stream);
  }
#define KVB_FA(D, NW)                                                                                           \
  return launch<D, NW>(q, q_row_stride, k_pages, v_pages, block_table, max_pages, page_shift, num_pages, positions, \
                       tiles, num_tiles, out, nq, nkv, G, gp_shift, scale, window, status, stream)
  if (d == 64) { if (wide) KVB_FA(64, 8); KVB_FA(64, 4); }
  if (wide) KVB_FA(128, 8);
  KVB_FA(128, 4);
}
