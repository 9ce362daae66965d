// bfloat16 linear layers on the 5th-generation tensor cores:  C[M,N] = X[M,K] . W[N,K]^T
// (upstream: cublasGemmEx with bfloat16 operands and float32 accumulation,
// base/src/engine.cu:643-671).
//
// Skinny form, for steps with few rows (decode): the weight matrix is the streamed
// operand.  A block takes 128 output features (rows of W) and a slice of K; the
// weights arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle) in tiles of
// 128 x 64, the step's rows X as tiles of MP x 64 (MP = M padded to 16..256, rows
// beyond M read as zeros), through a ring of shared-memory stages guarded by
// mbarriers.  One thread issues tcgen05.mma (kind::f16, M=128, N=MP, K=16) with the
// accumulator D[feature, row] in tensor memory; tcgen05.commit hands each stage back
// to the TMA thread.  The four warps then read the accumulator with tcgen05.ld (warp
// w owns features 32w..32w+31) and store C[row, feature].
// When N gives too few blocks to pull the whole memory system, K is split over the
// blocks of a thread-block cluster (gridDim.y = cluster size).  Groups of four consecutive
// rows have an owner block (group g: block g mod S); block s sends its float32 partials of a
// group, four rows of a feature in one 16-byte st.async, to slot s in the shared memory of
// the owner (distributed shared memory), which counts the bytes on an mbarrier; an owner
// goes on as soon as the partials of its own rows are there (it does not wait for the whole
// cluster) and adds up the slots in block order, so the sum has one fixed order.  The
// cluster meets once, at the start, while the first weights are already on their way, so
// that no block writes to a peer whose barrier is not set up.  No scratch in global
// memory, no counters.
// The weights do not depend on the step's data: a block requests its first ring of
// weight tiles before it waits for the kernel in front of it (programmatic dependent
// launch), so that the first tiles are under way while that kernel finishes.
// Every wait on an mbarrier is bounded; a wait that runs out records
// KVB_STATUS_WAIT_TIMEOUT, and the block frees its tensor memory and returns.
#include "common.cuh"

#include <cuda.h>

#include <mutex>
#include <unordered_map>

namespace {

constexpr int TILE_N = 128;  // output features per block = UMMA M
constexpr int TILE_K = 64;   // one 128-byte swizzle row of bfloat16
constexpr int kThreads = 128;
constexpr unsigned kSpinLimit = 20u * 1000u * 1000u;

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// Bounded wait.  false: the limit ran out.
__device__ __forceinline__ bool mbar_wait_limited(void* bar, unsigned parity, unsigned limit) {
  for (unsigned i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity) { return mbar_wait_limited(bar, parity, kSpinLimit); }
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// The same with an L2 eviction policy: weights are read once per step and should not push the
// step's small, re-read tensors (rows, residual, partial sums) out of the L2 cache.
__device__ __forceinline__ unsigned long long l2_policy_evict_first() {
  unsigned long long pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* map, int x, int y, void* bar,
                                                 unsigned long long policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(smem_u32(dst)), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy) : "memory");
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

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Stores four floats (16 bytes, 16-byte aligned) at the place in block `rank`'s shared memory
// that `my_smem_ptr` names in ours and counts their bytes on that block's mbarrier `my_bar`
// (asynchronous: the store is complete for the receiver when its barrier says so).
__device__ __forceinline__ void st_async_peer_f32x4(void* my_smem_ptr, void* my_bar, unsigned rank, float a, float b,
                                                    float c, float d) {
  unsigned remote, remote_bar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(my_smem_ptr)), "r"(rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(smem_u32(my_bar)), "r"(rank));
  asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(remote), "r"(__float_as_uint(a)), "r"(__float_as_uint(b)), "r"(__float_as_uint(c)),
                 "r"(__float_as_uint(d)), "r"(remote_bar) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of
// 128 bytes, groups of 8 rows 1024 bytes apart, tile base aligned to 1024 bytes.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned addr) {
  return (unsigned long long)((addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// What happens to the finished sums:
//   EPI_STORE     C[m, n] = sum
//   EPI_SWIGLU    the weight rows come in blocks of 128: 64 gate features, then the 64 up
//                 features of the same indices; out[m, 64 t + j] = silu(gate) * up
//                 (upstream: a kernel of its own after the product, base/src/kernels.cu:45-52)
//   EPI_RESIDUAL  resid[m, n] += sum, in float32 and in place (every element has one owner);
//                 xb[m, n] = bfloat16(new resid[m, n]), the rows of the product that reads the
//                 residual next; and sumsq[m, tile] = the sum of the squares of the new
//                 resid[m, n] over the tile's 128 features, added up in a fixed order.
// Row scale (x_sumsq != nullptr), with any epilogue but EPI_RESIDUAL: the finished sum of
// row m is multiplied by rsqrt(sum_p x_sumsq[m, p] / K + eps) first.  With the RMSNorm's
// weight multiplied into the columns of W beforehand, a product over the bare residual
// rows (xb) scaled so is the product over the normalised rows:
//   sum_k (r[m,k] * rstd[m] * g[k]) * W[n,k]  =  rstd[m] * sum_k r[m,k] * (g[k] * W[n,k]),
// so the add and the norm between two products need no kernel of their own (upstream: two
// kernels, base/src/kernels.cu:10-43), and nothing of them lies on the path between the
// end of one product and the first multiplication of the next: the partial sums are
// read by the two warps that have no other work while the products run.
// (Two other forms were tried and measured slower than the separate add+norm kernel:
// adding and normalising in the block that finishes last, whose serial tail costs more
// than the launch it saves, and normalising the float32 rows while loading them, which
// puts two to three microseconds of loads in front of the first multiplication.)
enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_RESIDUAL = 2 };

struct Params {
  int M, N, K, MP;            // MP: rows padded to the UMMA N extent
  int k_tiles, splits;        // k tiles in all, blocks along K
  int stages;
  int accs;                   // issuing warps, each with an accumulator of its own in tensor memory (1 or 2)
  int red_bytes;              // shared memory set aside for the partials that peers send (splits > 1)
  int out_f32;                // 1: C is float32, 0: bfloat16
  void* out;                  // [M, N]; EPI_SWIGLU: [M, N/2]
  int epilogue;               // EPI_*
  int fin_bytes;              // shared memory for the rows' final sums (EPI_SWIGLU)
  float* resid;               // EPI_RESIDUAL: [M, ld_resid] float32, updated in place
  int ld_resid;
  __nv_bfloat16* xb_out;      // EPI_RESIDUAL: [M, N] bfloat16 copy of the new residual rows
  float* sumsq_out;           // EPI_RESIDUAL: [M, tiles along N]
  const float* x_sumsq;       // row scale: [M, x_parts] partial sums of squares of the rows' source, or nullptr
  int x_parts;
  float eps;
  int* status;
  unsigned long long* trace;  // optional [blocks, 8] nanosecond stamps of the phases of each block (profiling)
};

__device__ __forceinline__ void stamp(const Params& p, int slot) {
  if (p.trace) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.trace[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 8 + slot] = t;
  }
}

template <int kUnused = 0>
__global__ void __launch_bounds__(kThreads, 2)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const Params p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // carve: stages x (W tile, X tile), then barriers
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int a_bytes = TILE_N * TILE_K * 2;
  const int b_bytes = p.MP * TILE_K * 2;
  unsigned char* a_s = base;
  unsigned char* b_s = base + (size_t)p.stages * a_bytes;
  float* red = reinterpret_cast<float*>(b_s + (size_t)p.stages * b_bytes);  // never part of the stage ring:
  // peers write here while this block may still be multiplying
  float* fin = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(red) + p.red_bytes);   // [rows][128]
  unsigned long long* full = reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(fin) + p.fin_bytes);
  unsigned long long* empty = full + p.stages;
  unsigned long long* accum = empty + p.stages;
  unsigned long long* red_bar = accum + 1;       // counts the bytes of the partials that peers send
  unsigned* tmem_holder = reinterpret_cast<unsigned*>(red_bar + 1);
  int* flags = reinterpret_cast<int*>(tmem_holder + 1);  // [0]: abort, [1]: this block reduces the splits
  float* rstd = reinterpret_cast<float*>(flags + 2);     // [64] row scale

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) stamp(p, 0);   // block started
  const int n0 = blockIdx.x * TILE_N;
  const int per = (p.k_tiles + p.splits - 1) / p.splits;
  const int kt0 = blockIdx.y * per;
  const int kt1 = min(p.k_tiles, kt0 + per);
  const int my_tiles = max(0, kt1 - kt0);
  // One thread issues a 128 x rows x 16 product about every 110 cycles however few the rows (measured:
  // 439 cycles per tile of four; two threads of different warps issuing side by side reach one per
  // 42 cycles between them), while 16 KB of weights per tile arrive faster than that when the block
  // has an SM to itself.  So two warps issue, tile about, each into an accumulator of its own; the
  // epilogue adds the two up.
  const unsigned acc_stride = p.MP < 32 ? 32u : (unsigned)p.MP;
  const unsigned tmem_cols = acc_stride * (unsigned)p.accs;

  // Which rows' final sums this block holds.  K not split: all.  K split: groups of four
  // consecutive rows go round the blocks, group g to block g mod splits, so that a sender hands
  // over four rows of a feature in one 16-byte store (measured faster than single rows spread
  // over all blocks, at every number of rows).
  const int S = p.splits, y = (int)blockIdx.y;
  const int groups_all = (p.M + 3) >> 2;
  const int groups_own = (S > 1 && groups_all > y) ? (groups_all - 1 - y) / S + 1 : 0;
  // own rows are numbered j = 0 .. own_slots-1 (the last group may reach beyond M)
  const int own_slots = S == 1 ? p.M : 4 * groups_own;
  auto own_row = [&](int j) -> int { return S == 1 ? j : 4 * (y + (j >> 2) * S) + (j & 3); };
  const unsigned red_expect = (unsigned)(groups_own * S * TILE_N * 16);
  const int first = min(p.stages, my_tiles);
  const unsigned long long w_policy = l2_policy_evict_first();
  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(accum, (unsigned)p.accs);
    mbar_init(red_bar, 1);
    flags[0] = 0; flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // every block of the cluster sends 128 floats for each of this block's rows
    if (S > 1) mbar_expect_tx(red_bar, red_expect);
    // The weights do not depend on the kernel before this one: the first round of weight
    // tiles is requested at once, before anything else.
    for (int i = 0; i < first; ++i) {
      mbar_expect_tx(&full[i], a_bytes + b_bytes);
      tma_load_2d_hint(a_s + (size_t)i * a_bytes, &map_w, (kt0 + i) * TILE_K, n0, &full[i], w_policy);
    }
    stamp(p, 1);                 // first round of weight tiles requested
  }
  if (warp == 1) tmem_alloc(tmem_holder, tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_d = *tmem_holder;
  // From here on peers may write into this block's shared memory: every block's barrier is set up.
  if (p.splits > 1) cluster_sync_all();
  // The kernel behind this one may start only now that this block holds its tensor memory:
  // blocks of that kernel which wait, resident, for this grid to finish must not be able to
  // take the columns that a block of this grid still needs.
  pdl_trigger();

  if (warp == 0 && lane == 0) {
    // ---- TMA producer.  The rows are requested only after the kernel before this one has
    // finished.
    pdl_wait();
    stamp(p, 2);                 // the kernel before this one has finished
    for (int i = 0; i < first; ++i)
      tma_load_2d(b_s + (size_t)i * b_bytes, &map_x, (kt0 + i) * TILE_K, 0, &full[i]);
    for (int i = first; i < my_tiles; ++i) {
      const int s = i % p.stages;
      const unsigned phase = (i / p.stages) & 1;
      if (!mbar_wait(&empty[s], phase ^ 1)) { atomicExch(&flags[0], 1); break; }
      mbar_expect_tx(&full[s], a_bytes + b_bytes);
      tma_load_2d_hint(a_s + (size_t)s * a_bytes, &map_w, (kt0 + i) * TILE_K, n0, &full[s], w_policy);
      tma_load_2d(b_s + (size_t)s * b_bytes, &map_x, (kt0 + i) * TILE_K, 0, &full[s]);
    }
  } else if ((warp == 1 || (warp == 2 && p.accs == 2)) && lane == 0) {
    // ---- MMA issuers: warp 1 takes the even tiles, warp 2 (when there are two) the odd ones
    const int w = warp - 1;
    const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(p.MP >> 3) << 17) | ((unsigned)(TILE_N >> 4) << 24);
    const unsigned acc = tmem_d + (unsigned)w * acc_stride;
    bool ok = true;
    for (int i = w; i < my_tiles && ok; i += p.accs) {
      const int s = i % p.stages;
      const unsigned phase = (i / p.stages) & 1;
      if (!mbar_wait(&full[s], phase)) { atomicExch(&flags[0], 1); ok = false; break; }
      if (i == 0) stamp(p, 3);   // first tile arrived
      const unsigned long long ad = smem_desc_sw128(smem_u32(a_s + (size_t)s * a_bytes));
      const unsigned long long bd = smem_desc_sw128(smem_u32(b_s + (size_t)s * b_bytes));
#pragma unroll
      for (int k = 0; k < TILE_K / 16; ++k)  // 32 bytes further along K per step: +2 in the address field
        umma_bf16(acc, ad + 2 * k, bd + 2 * k, idesc, (i > w || k > 0) ? 1u : 0u);
      umma_commit(&empty[s]);   // the stage is free once these products have read it
    }
    if (w == 0) stamp(p, 4);    // last product issued
    // everything this warp issued has landed in tensor memory (a warp without a tile just arrives)
    if (my_tiles > w) umma_commit(accum); else mbar_arrive(accum);
  }
  __syncwarp();

  // ---- epilogue: all four warps (the accumulator depends on rows loaded after pdl_wait;
  // the explicit wait also covers blocks that had no k tile)
  pdl_wait();
  // The residual values that the block's first group of rows is added to ([4][128] in shared
  // memory): warp 3 fetches them now, while the products run and the memory system is quiet.  Once
  // the accumulator is complete the blocks of the kernel behind this one are streaming their
  // weights, and a load that starts then waits behind them (measured: 1.5 us instead of 0.5).
  float* resid_s = fin + own_slots * 4;
  const bool resid_staged = p.epilogue == EPI_RESIDUAL && S > 1 && groups_own > 0;
  float rv[16];
  if (resid_staged && warp == 3) {
    const int m0 = own_row(0);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int nn = n0 + q * 32 + lane;
        rv[k * 4 + q] = (m0 + k < p.M && nn < p.N) ? p.resid[(size_t)(m0 + k) * p.ld_resid + nn] : 0.f;
      }
    }
  }
  if (p.x_sumsq && warp == 3) {
    // Row scale: warp 3 has nothing else to do while the products run.  A thread takes a row (two
    // beyond 32 rows) and adds up its parts in their order.
    for (int r = lane; r < p.M; r += 32) {
      float ss = 0.f;
      const float* src = p.x_sumsq + (size_t)r * p.x_parts;
      int q = 0;
      for (; q + 4 <= p.x_parts; q += 4) {        // four loads in flight, added in order
        const float a0 = src[q], a1 = src[q + 1], a2 = src[q + 2], a3 = src[q + 3];
        ss = (((ss + a0) + a1) + a2) + a3;
      }
      for (; q < p.x_parts; ++q) ss += src[q];
      rstd[r] = rsqrtf(ss / (float)p.K + p.eps);
    }
  }
  if (resid_staged && warp == 3) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#pragma unroll
      for (int q = 0; q < 4; ++q) resid_s[k * TILE_N + q * 32 + lane] = rv[k * 4 + q];
    }
  }
  if (p.epilogue == EPI_RESIDUAL && n0 + tid < p.N) {
    // the residual values of further groups of rows: towards L1 while the products run
    for (int j = (S > 1 ? 4 : 0); j < own_slots; ++j) {
      const int m = own_row(j);
      if (m < p.M) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.resid + (size_t)m * p.ld_resid + n0 + tid));
    }
  }
  bool good = true;
  if (my_tiles > 0) good = mbar_wait(accum, 0);
  if (!good) atomicExch(&flags[0], 1);
  tc_fence_after();
  __syncthreads();
  const bool aborted = flags[0] != 0;
  if (aborted && tid == 0) atomicCAS(p.status, 0, KVB_STATUS_WAIT_TIMEOUT);
  if (tid == 0) stamp(p, 5);   // accumulator complete

  // 16 rows (columns c .. c+15 of this thread's feature) of the finished sums: the issuing warps' accumulators added up
  auto load_sums = [&](int c, float* v) {
    tmem_ld16(tmem_d + ((unsigned)(warp * 32) << 16) + c, v);
    if (p.accs == 2 && my_tiles > 1) {
      float w1[16];
      tmem_ld16(tmem_d + ((unsigned)(warp * 32) << 16) + acc_stride + c, w1);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] += w1[i];
    }
  };
  const int n = n0 + warp * 32 + lane;           // the feature this thread holds
  // What this block does with the final sum of (row m, its j-th own row, this thread's feature).
  const bool scaled = p.x_sumsq != nullptr;
  auto emit = [&](int m, int j, float val) {
    if (scaled) val *= rstd[m];
    if (p.epilogue == EPI_SWIGLU) {
      fin[j * TILE_N + tid] = val;
    } else if (p.epilogue == EPI_RESIDUAL) {
      float nv = 0.f;
      if (n < p.N) {
        float* r = p.resid + (size_t)m * p.ld_resid + n;
        nv = *r + val;
        *r = nv;
        p.xb_out[(size_t)m * p.N + n] = __float2bfloat16_rn(nv);
      }
      float sq = nv * nv;                           // lanes in a fixed tree, then the four warps in order
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (lane == 0) fin[j * 4 + warp] = sq;
    } else if (n < p.N) {
      if (p.out_f32) {
        reinterpret_cast<float*>(p.out)[(size_t)m * p.N + n] = val;
      } else {
        reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(val);
      }
    }
  };
  if (S > 1 || !aborted) {
    if (S == 1) {
      for (int c = 0; c < p.MP && c < p.M; c += 16) {
        float v[16];
        if (my_tiles > 0) load_sums(c, v);
        else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (c + i < p.M) emit(c + i, c + i, v[i]);
      }
    } else {
      // Send this block's partials to the rows' owners, slot blockIdx.y there.  A block that gave
      // up sends zeros, so that the byte counts of its peers still come out.
      for (int c = 0; c < p.MP && c < p.M; c += 16) {
        float v[16];
        if (my_tiles > 0 && !aborted) load_sums(c, v);
        else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0.f;
        }
        // rows c+4k .. c+4k+3 are group c/4 + k: red4[(group / S) * S + slot][feature] in block group mod S
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int g4 = (c >> 2) + k;
          if (g4 < groups_all)
            st_async_peer_f32x4(reinterpret_cast<float4*>(red) + ((g4 / S) * S + y) * TILE_N + tid, red_bar,
                                (unsigned)(g4 % S), v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
        }
      }
    }
  }
  bool red_ok = true;
  if (S > 1) {
    // The partials of this block's rows: complete when the barrier has counted all their bytes.
    // Nobody leaves before that, so no block writes into the memory of a peer that is gone.
    if (own_slots > 0) red_ok = mbar_wait(red_bar, 0);
    red_ok = __syncthreads_and(red_ok) != 0;        // one answer for the whole block
    if (!red_ok && tid == 0) atomicCAS(p.status, 0, KVB_STATUS_WAIT_TIMEOUT);
    if (tid == 0) stamp(p, 7);   // this block's partials are here
    if (!aborted && red_ok) {
      {
        for (int gi = 0; gi < groups_own; ++gi) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          const float4* slots = reinterpret_cast<const float4*>(red) + (size_t)gi * S * TILE_N + tid;
          for (int s0 = 0; s0 < S; s0 += 8) {       // the blocks' partials in block order, eight loads at a time
            float4 part[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              part[i] = s0 + i < S ? slots[(s0 + i) * TILE_N] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (s0 + i < S) { acc.x += part[i].x; acc.y += part[i].y; acc.z += part[i].z; acc.w += part[i].w; }
            }
          }
          const int m0 = own_row(4 * gi);
          if (p.epilogue == EPI_RESIDUAL) {
            // the group's four rows side by side, so that their loads and their reductions overlap
            float a4[4] = {acc.x, acc.y, acc.z, acc.w}, nv[4], sq[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              nv[k] = 0.f;
              if (m0 + k < p.M && n < p.N)
                nv[k] = (gi == 0 ? resid_s[k * TILE_N + tid] : p.resid[(size_t)(m0 + k) * p.ld_resid + n]) +
                        (scaled ? a4[k] * rstd[m0 + k] : a4[k]);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (m0 + k < p.M && n < p.N) {
                p.resid[(size_t)(m0 + k) * p.ld_resid + n] = nv[k];
                p.xb_out[(size_t)(m0 + k) * p.N + n] = __float2bfloat16_rn(nv[k]);
              }
              sq[k] = nv[k] * nv[k];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
              for (int k = 0; k < 4; ++k) sq[k] += __shfl_xor_sync(0xffffffffu, sq[k], o);
            }
            if (lane == 0) {
#pragma unroll
              for (int k = 0; k < 4; ++k) fin[(4 * gi + k) * 4 + warp] = sq[k];
            }
          } else {
            if (m0 < p.M) emit(m0, 4 * gi, acc.x);
            if (m0 + 1 < p.M) emit(m0 + 1, 4 * gi + 1, acc.y);
            if (m0 + 2 < p.M) emit(m0 + 2, 4 * gi + 2, acc.z);
            if (m0 + 3 < p.M) emit(m0 + 3, 4 * gi + 3, acc.w);
          }
        }
      }
    }
  }
  if (p.epilogue == EPI_SWIGLU && !aborted && red_ok) {
    // gate and up of one feature sit 64 threads apart: pair them through shared memory
    __syncthreads();
    // 64 columns per row; the block's threads take (row, column) pairs in turn
    const int c = tid & (TILE_N / 2 - 1);
    const int col = blockIdx.x * (TILE_N / 2) + c;
    if (col < p.N / 2) {
      // four rows at a time, side by side: with four warps on the SM a single chain of
      // exponential, division and store would run at its latency, not at its throughput
      constexpr int kStep = kThreads / (TILE_N / 2);
      for (int j0 = tid >> 6; j0 < own_slots; j0 += 4 * kStep) {
        float g[4], u[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j = j0 + i * kStep;
          const bool in = j < own_slots;
          g[i] = in ? fin[j * TILE_N + c] : 0.f;
          u[i] = in ? fin[j * TILE_N + TILE_N / 2 + c] : 0.f;
        }
        float a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = g[i] * (1.0f / (1.0f + expf(-g[i]))) * u[i];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j = j0 + i * kStep;
          if (j < own_slots) {
            const int m = own_row(j);
            if (m < p.M) reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * (p.N / 2) + col] = __float2bfloat16_rn(a[i]);
          }
        }
      }
    }
  }
  if (p.epilogue == EPI_RESIDUAL && !aborted && red_ok) {
    __syncthreads();
    if (tid < own_slots) {                          // thread j finishes the block's j-th own row
      const int m = own_row(tid);
      if (m < p.M)
        p.sumsq_out[(size_t)m * gridDim.x + blockIdx.x] =
            ((fin[tid * 4] + fin[tid * 4 + 1]) + fin[tid * 4 + 2]) + fin[tid * 4 + 3];
    }
  }
  if (aborted) {
    // give copies that may still be in flight time to land before the block ends
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  if (tid == 0) stamp(p, 6);   // result stored
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_d, tmem_cols);
}

// One warp waits, with a limit of `polls`, on a barrier that nothing ever completes, and
// reports what the product kernel reports when one of its waits runs out.
__global__ void wait_selftest_kernel(unsigned polls, int* status) {
  __shared__ unsigned long long bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  if (!mbar_wait_limited(&bar, 0, polls) && threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// A [rows, K] bfloat16 row-major matrix as a 2-D tensor map with boxes of box_rows x 64.
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return KVB_ERR_BAD_SIZE;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

struct MapKey {
  const void* ptr; int rows, K, ld, box;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && K == o.K && ld == o.ld && box == o.box; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (size_t)k.rows * 1315423911u ^ (size_t)k.K * 2654435761u ^ (size_t)k.box;
  }
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;  // weights keep their address: encode once

int cached_map(CUtensorMap* out, const void* ptr, int rows, int K, int ld, int box) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  MapKey key{ptr, rows, K, ld, box};
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    CUtensorMap m;
    const int rc = make_map(&m, ptr, rows, K, ld, box);
    if (rc) return rc;
    if (g_maps.size() > 4096) g_maps.clear();
    it = g_maps.emplace(key, m).first;
  }
  *out = it->second;
  return 0;
}

}  // namespace

// How the skinny kernel would cut a problem: blocks along K (= cluster size) and tiles
// along N.  Returns 0 if it takes the sizes (M <= 256, K a multiple of 8),
// KVB_ERR_BAD_SIZE otherwise.
KVB_EXPORT int kvb_gemm_skinny_plan(int M, int N, int K, int* splits, int* n_tiles) {
  if (M < 1 || M > 256 || N < 1 || K < 8 || (K & 7)) return KVB_ERR_BAD_SIZE;
  const int tiles = (N + TILE_N - 1) / TILE_N;
  const int k_tiles = (K + TILE_K - 1) / TILE_K;
  // Two blocks fit an SM.  A grid that fills both places of every SM leaves none for the blocks of the
  // kernel behind it, which then start (and request their first weights) only when this grid ends;
  // measured at three model sizes, one and a half blocks per SM is the better target, except where it
  // would leave K unsplit although two blocks per tile still fit (then: two).
  int s = (3 * kvb_sm_count() / 2) / tiles;
  if (s < 2 && 2 * tiles <= 2 * kvb_sm_count()) s = 2;
  if (s > k_tiles / 2) s = k_tiles / 2;      // at least two k tiles per block
  if (s > 8) s = 8;                          // the largest portable cluster (clusters of 16 were measured: they
                                             // do not all fit at once, and the second wave costs more than they gain)
  if (s < 1) s = 1;
  while (s > 1 && (k_tiles + s - 1) / s * (s - 1) >= k_tiles) --s;  // no block without work
  *splits = s;
  *n_tiles = tiles;
  return 0;
}

namespace {

struct Extras {
  // row scale
  const float* x_sumsq = nullptr; int x_parts = 0; float eps = 0.f;
  // EPI_RESIDUAL
  float* resid = nullptr; int ld_resid = 0; __nv_bfloat16* xb_out = nullptr; float* sumsq_out = nullptr;
};

int gemm_skinny_launch(const void* x, int ldx, const void* w, int ldw, void* out, int out_f32, int M, int N, int K,
                       int x_is_static, int epilogue, const Extras& ex, int* status, unsigned long long* trace,
                       cudaStream_t stream) {
  int splits, tiles;
  const int rc = kvb_gemm_skinny_plan(M, N, K, &splits, &tiles);
  if (rc) return rc;
  if ((ldx & 7) || (ldw & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return KVB_ERR_ALIGN;
  int MP = 16;
  while (MP < M) MP <<= 1;
  Params p;
  p.M = M; p.N = N; p.K = K; p.MP = MP;
  p.k_tiles = (K + TILE_K - 1) / TILE_K;
  p.splits = splits;
  p.accs = 2;                       // two issuing warps: 2 x max(32, MP) columns, at most all 512 (256 rows, one block per SM)
  p.out_f32 = out_f32; p.out = out; p.status = status; p.trace = trace;
  if (epilogue < EPI_STORE || epilogue > EPI_RESIDUAL) return KVB_ERR_BAD_SIZE;
  if (epilogue != EPI_STORE && (M > 64 || out_f32)) return KVB_ERR_BAD_SIZE;
  if (epilogue == EPI_SWIGLU && (N % TILE_N)) return KVB_ERR_BAD_SIZE;
  if (epilogue == EPI_RESIDUAL && (!ex.resid || !ex.sumsq_out || !ex.xb_out || ex.ld_resid < N || ex.x_sumsq))
    return KVB_ERR_BAD_SIZE;
  if (ex.x_sumsq && (M > 64 || ex.x_parts < 1)) return KVB_ERR_BAD_SIZE;
  p.epilogue = epilogue;
  p.resid = ex.resid; p.ld_resid = ex.ld_resid; p.xb_out = ex.xb_out; p.sumsq_out = ex.sumsq_out;
  p.x_sumsq = ex.x_sumsq; p.x_parts = ex.x_parts; p.eps = ex.eps;
  const int stage_bytes = TILE_N * TILE_K * 2 + MP * TILE_K * 2;
  // two blocks per SM while the stages stay deep enough, one block otherwise
  const int budget = MP <= 64 ? 108 * 1024 : 200 * 1024;
  // Room for the partials of this block's rows from every block of the cluster, and for the
  // finished sums that an epilogue passes between threads (one slot per own row; see the kernel
  // for which rows a block owns).
  auto own_slots = [&](int s) {
    if (s == 1) return M;
    return 4 * ((((M + 3) >> 2) + s - 1) / s);
  };
  auto fin_bytes = [&](int s) {
    return epilogue == EPI_SWIGLU ? own_slots(s) * TILE_N * 4 : epilogue == EPI_RESIDUAL ? own_slots(s) * 4 * 4 + (s > 1 ? 4 * TILE_N * 4 : 0) : 0;
  };
  int red_bytes = splits > 1 ? own_slots(splits) * splits * TILE_N * 4 : 0;
  if (red_bytes + fin_bytes(splits) > budget - 2 * stage_bytes) { splits = 1; red_bytes = 0; }   // no room: one block does all of K
  p.fin_bytes = fin_bytes(splits);
  if (p.fin_bytes > budget - 2 * stage_bytes) return KVB_ERR_BAD_SIZE;
  p.splits = splits;
  p.red_bytes = red_bytes;
  int stages = (budget - red_bytes - p.fin_bytes) / stage_bytes;
  if (stages > 8) stages = 8;
  const int per = (p.k_tiles + splits - 1) / splits;
  if (stages > per) stages = per;
  if (stages < 2) stages = 2;
  // Two issuing warps take the tiles in turn.  A stage must always be read by the same warp, tile
  // after tile in order: a wait on a stage's barrier tells a phase only from the one before it, and a
  // warp that ran two uses of a stage ahead of the other would take the old phase for the new one.
  // With an even number of stages tile i and stage i mod stages have the same parity.
  if (p.accs == 2) stages &= ~1;
  p.stages = stages;
  const size_t smem = 1024 + (size_t)stages * stage_bytes + red_bytes + p.fin_bytes + (2 * stages + 2) * 8 + 16 + 256;
  CUtensorMap mw, mx;
  int e = cached_map(&mw, w, N, K, ldw, TILE_N);
  if (e) return e;
  // The rows' map is kept like the weights': the key names address, shape and box, so an entry can
  // only ever describe the memory it is looked up for, and a step's tensors lie at the same places
  // step after step (the flag is kept in the interface; encoding a map costs microseconds per launch).
  (void)x_is_static;
  e = cached_map(&mx, x, M, K, ldx, MP);
  if (e) return e;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t ce = cudaFuncSetAttribute(gemm_skinny_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024);  // the kernel also has a little static shared memory
    if (ce != cudaSuccess) return (int)ce;
    ce = cudaFuncSetAttribute(gemm_skinny_kernel<0>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (ce != cudaSuccess) return (int)ce;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, splits, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = splits;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = kvb_pdl_enabled() ? 2 : 1;
  cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<0>, mw, mx, p);
  if (le != cudaSuccess) return (int)le;
  return kvb_launch_result();
}

}  // namespace

// C[M,N] = X[M,K] . W[N,K]^T, bfloat16 operands (ldx, ldw in elements, multiples of 8),
// C bfloat16 (out_f32 = 0) or float32, dense [M,N].  x_is_static: the activation's
// address is stable (a captured graph); no longer needed, since the rows' tensor map is
// kept by address and shape like the weights'.  trace: nullptr, or [blocks, 8] uint64 for the phase stamps of every
// block (profiling only).
// epilogue (see EPI_*): 0 store; 1 SwiGLU on row-interleaved weights, out is bfloat16
// [M, N/2], N a multiple of 128, M <= 64.
// Uses no memory beyond its operands.
KVB_EXPORT int kvb_gemm_skinny(const void* x, int ldx, const void* w, int ldw, void* out, int out_f32, int M, int N,
                               int K, int x_is_static, int epilogue, int* status, unsigned long long* trace,
                               cudaStream_t stream) {
  if (epilogue == EPI_RESIDUAL) return KVB_ERR_BAD_SIZE;
  return gemm_skinny_launch(x, ldx, w, ldw, out, out_f32, M, N, K, x_is_static, epilogue, Extras(), status, trace,
                            stream);
}

// The same product with the residual stream's add and RMSNorm folded around it, M <= 64.
//  - x_sumsq != nullptr (row scale): row m of the result is multiplied by
//    rsqrt(sum_p x_sumsq[m, p] / K + eps) before the epilogue (0 or 1) sees it; x holds the
//    bare residual rows in bfloat16 and W has the norm's weight multiplied into its columns.
//  - epilogue 2 (EPI_RESIDUAL): resid[M, ld_resid] += X . W^T in place, xb_out[M, N] gets the
//    new rows in bfloat16 and sumsq_out[M, ceil(N/128)] their partial sums of squares; out unused.
KVB_EXPORT int kvb_gemm_skinny_fused(const void* x, int ldx, const void* w, int ldw, void* out, int M, int N, int K,
                                     int x_is_static, int epilogue, const float* x_sumsq, int x_parts, float eps,
                                     float* resid, int ld_resid, void* xb_out, float* sumsq_out, int* status,
                                     unsigned long long* trace, cudaStream_t stream) {
  Extras ex;
  ex.x_sumsq = x_sumsq; ex.x_parts = x_parts; ex.eps = eps;
  ex.resid = resid; ex.ld_resid = ld_resid; ex.xb_out = reinterpret_cast<__nv_bfloat16*>(xb_out);
  ex.sumsq_out = sumsq_out;
  return gemm_skinny_launch(x, ldx, w, ldw, out, 0, M, N, K, x_is_static, epilogue, ex, status, trace, stream);
}

// Runs the bounded wait of this file's kernels against a barrier that is never completed: after
// `polls` polls the kernel gives up, records KVB_STATUS_WAIT_TIMEOUT in *status and returns; the
// context stays usable.  For tests of the give-up path.
KVB_EXPORT int kvb_wait_selftest(unsigned polls, int* status, cudaStream_t stream) {
  wait_selftest_kernel<<<1, 32, 0, stream>>>(polls, status);
  return kvb_launch_result();
}
