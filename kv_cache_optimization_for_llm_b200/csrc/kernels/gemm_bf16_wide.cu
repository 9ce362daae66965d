// bfloat16 linear layers for steps with many rows (prompt portions) on the 5th-generation
// tensor cores:  C[M,N] = X[M,K] . W[N,K]^T, float32 accumulation
// (upstream: cublasGemmEx with bfloat16 operands and float32 accumulation,
// base/src/engine.cu:643-671; its SiLU(gate)*up is a kernel of its own after two products,
// base/src/kernels.cu:45-52, here it is the epilogue of one product over gate|up).
//
// Persistent kernel, one block per SM, 192 or 320 threads in three roles that meet on mbarriers only:
//   warp 0       one thread requests the operand tiles by TMA (cp.async.bulk.tensor, 128-byte
//                swizzle): 128 rows of X and BN rows of W, 64 elements of K each, into a ring of
//                shared-memory stages;
//   warp 1       one thread issues tcgen05.mma (kind::f16, M = 128, N = BN, K = 16), four per
//                stage, into one of two accumulators in tensor memory (lane = row of X, column
//                = feature); tcgen05.commit hands a stage back to the loader and a finished
//                accumulator to the epilogue;
//   warps 2..5   the epilogue: a thread owns one row of the tile (its lane of tensor memory),
//                reads 32 columns at a time with tcgen05.ld and stores them; the other
//                accumulator is being filled meanwhile.
// What bounds a single block is the operand traffic of its SM, not the tensor pipe: a tile of
// 128 x 256 writes 48 KB into shared memory per 64 of K and reads as much for the products, and
// the pipe is busy 57 % of the time.  Tiles of 256 x 256 (two accumulators of 128 rows over the
// same tile of W, warps 6..9 the epilogue of the second) need a third less per product, but fill
// the tensor memory, so that their epilogue does not overlap with the next tile.  The form on
// pairs of SMs further down halves the traffic per SM and keeps the overlap; it is the one
// that large problems get.
// Tiles go round the blocks in a fixed order, rows of X fastest, so that the blocks that run
// together share a few tiles of W in L2.  Rows and features beyond M and N and the end of K
// are read as zeros by TMA and never stored.
// Every wait on an mbarrier is bounded; a role whose wait runs out tells the others, the
// block records KVB_STATUS_WAIT_TIMEOUT, frees its tensor memory and returns.
#include "common.cuh"

#include <cuda.h>

#include <mutex>
#include <unordered_map>

namespace {

constexpr int BM = 128;      // rows of X per tile = UMMA M
constexpr int BK = 64;       // one 128-byte swizzle row of bfloat16
constexpr unsigned kSpinLimit = 20u * 1000u * 1000u;
constexpr int kMaxStages = 8;

// What happens to the finished sums (the same three as for steps of few rows, gemm_bf16.cu):
//   EPI_STORE     C[m, n] = sum
//   EPI_SWIGLU    the rows of W come in blocks of 128: 64 gate features, then the 64 up features of
//                 the same indices; out[m, 64 t + j] = silu(gate) * up
//   EPI_RESIDUAL  resid[m, n] += sum, in float32 and in place (every element has one owner);
//                 xb[m, n] = bfloat16(new resid[m, n]), the rows that the next product reads;
//                 sumsq[m, tile] = the sum of the squares of the new resid[m, n] over the tile's
//                 256 features, added up in the order of the features.
// Row scale (x_sumsq != nullptr, not with EPI_RESIDUAL): the finished sum of row m is multiplied
// by rsqrt(sum_p x_sumsq[m, p] / K + eps) first.  With the RMSNorm's weight multiplied into the
// columns of W beforehand, the product over the bare residual rows, scaled so, is the product
// over the normalised rows, and the add and the norm between two products (upstream: two
// kernels, base/src/kernels.cu:10-43) need no kernel of their own.
enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_RESIDUAL = 2 };

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
// Bounded wait that also ends when another role of the block has given up.  false: gave up.
__device__ __forceinline__ bool wait_or_abort(void* bar, unsigned parity, volatile int* abort_flag) {
  for (unsigned i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
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
// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of
// 128 bytes, groups of 8 rows 1024 bytes apart, tile base aligned to 1024 bytes.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned addr) {
  return (unsigned long long)((addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// 16 bfloat16 (one 32-byte sector) in one store
__device__ __forceinline__ void st_global_32(void* p, const unsigned* w) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
               "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}
__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&h);
}

struct Params {
  int M, N, K;
  int m_tiles, n_tiles, k_tiles, stages;
  __nv_bfloat16* out;
  int ldo;          // elements between rows of out
  int store32;      // rows of out start on 32-byte boundaries and N is a multiple of 16: whole sectors per store
  const float* x_sumsq;   // row scale: [M, x_parts] partial sums of squares of the rows' source, or nullptr
  int x_parts;
  float eps;
  float* resid;           // EPI_RESIDUAL: [M, ld_resid] float32, updated in place
  int ld_resid;
  __nv_bfloat16* xb_out;  // EPI_RESIDUAL: [M, N] bfloat16 copy of the new residual rows
  float* sumsq_out;       // EPI_RESIDUAL: [M, n_tiles]
  int* status;
  unsigned long long* trace;   // nullptr, or [64][8] uint64: phase stamps of the first pair's first 64 stages (profiling)
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define KVB_STAMP(slot) do { if (p.trace && pair == 0 && it < 64) p.trace[it * 8 + (slot)] = globaltimer_ns(); } while (0)

struct Bars {
  unsigned long long full[kMaxStages], empty[kMaxStages], acc_full[2], acc_empty[2];
};

// g / (1 + e^-g) with the hardware's exponential and reciprocal (a few units in the last place of
// float32, far below the bfloat16 rounding that follows): the activation of a tile's last round
// is not hidden under products.
__device__ __forceinline__ float silu_fast(float g) { return g * __fdividef(1.0f, 1.0f + __expf(-g)); }

// The epilogue of one row: BN finished sums of row m, features n0.., out of this thread's lane of
// tensor memory (columns `cols`..), 32 at a time.  Every lane of the warp takes part in the
// reads, whatever its row.
template <int BN, int EPI>
__device__ __forceinline__ void epilogue_rows(const Params& p, unsigned cols, int m, int n0) {
  float rstd = 1.0f;
  if (EPI != EPI_RESIDUAL && p.x_sumsq != nullptr && m < p.M) {
    const float* src = p.x_sumsq + (size_t)m * p.x_parts;
    float ss = 0.f;
    for (int i = 0; i < p.x_parts; ++i) ss += src[i];      // one fixed order
    rstd = rsqrtf(ss / (float)p.K + p.eps);
  }
  if (EPI == EPI_RESIDUAL) {
    // this thread's row of the residual, BN features from n0: 128 bytes of float32 per 32 features
    float* res = p.resid + (size_t)m * p.ld_resid + n0;
    __nv_bfloat16* xb = p.xb_out + (size_t)m * p.N + n0;
    float ss = 0.f;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      float v[32];
      tmem_ld32(cols + c, v);     // every lane of the warp takes part, whatever its row
      if (m < p.M) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (n0 + c + j < p.N) {   // N is a multiple of 8
            const float4 r0 = *reinterpret_cast<const float4*>(res + c + j);
            const float4 r1 = *reinterpret_cast<const float4*>(res + c + j + 4);
            const float4 a0 = make_float4(r0.x + v[j], r0.y + v[j + 1], r0.z + v[j + 2], r0.w + v[j + 3]);
            const float4 a1 = make_float4(r1.x + v[j + 4], r1.y + v[j + 5], r1.z + v[j + 6], r1.w + v[j + 7]);
            *reinterpret_cast<float4*>(res + c + j) = a0;
            *reinterpret_cast<float4*>(res + c + j + 4) = a1;
            *reinterpret_cast<uint4*>(xb + c + j) = make_uint4(pack_bf16(a0.x, a0.y), pack_bf16(a0.z, a0.w),
                                                              pack_bf16(a1.x, a1.y), pack_bf16(a1.z, a1.w));
            ss += a0.x * a0.x; ss += a0.y * a0.y; ss += a0.z * a0.z; ss += a0.w * a0.w;
            ss += a1.x * a1.x; ss += a1.y * a1.y; ss += a1.z * a1.z; ss += a1.w * a1.w;
          }
        }
      }
    }
    if (m < p.M) p.sumsq_out[(size_t)m * p.n_tiles + n0 / BN] = ss;
  } else if (EPI == EPI_STORE) {
    __nv_bfloat16* dst = p.out + (size_t)m * p.ldo + n0;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      float v[32];
      tmem_ld32(cols + c, v);     // every lane of the warp takes part, whatever its row
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= rstd;
      if (m < p.M) {
        if (p.store32) {
#pragma unroll
          for (int j = 0; j < 32; j += 16) {
            if (n0 + c + j < p.N) {
              unsigned pk[8];
#pragma unroll
              for (int q = 0; q < 8; ++q) pk[q] = pack_bf16(v[j + 2 * q], v[j + 2 * q + 1]);
              st_global_32(dst + c + j, pk);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (n0 + c + j < p.N)   // N is a multiple of 8
              *reinterpret_cast<uint4*>(dst + c + j) =
                  make_uint4(pack_bf16(v[j], v[j + 1]), pack_bf16(v[j + 2], v[j + 3]),
                             pack_bf16(v[j + 4], v[j + 5]), pack_bf16(v[j + 6], v[j + 7]));
          }
        }
      }
    }
  } else {
    // features in blocks of 128: 64 gate features, then the 64 up features of the same indices
    __nv_bfloat16* dst = p.out + (size_t)m * p.ldo + n0 / 2;
#pragma unroll 1
    for (int c = 0; c < BN; c += 128) {
#pragma unroll 1
      for (int h = 0; h < 64; h += 32) {
        float g[32], u[32];
        tmem_ld32(cols + c + h, g);
        tmem_ld32(cols + c + 64 + h, u);
        if (m < p.M && n0 + c < p.N) {   // N is a multiple of 128
#pragma unroll
          for (int j = 0; j < 32; j += 16) {
            unsigned pk[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float g0 = g[j + 2 * q] * rstd, g1 = g[j + 2 * q + 1] * rstd;
              pk[q] = pack_bf16(silu_fast(g0) * (u[j + 2 * q] * rstd), silu_fast(g1) * (u[j + 2 * q + 1] * rstd));
            }
            if (p.store32) {
              st_global_32(dst + c / 2 + h + j, pk);
            } else {
              *reinterpret_cast<uint4*>(dst + c / 2 + h + j) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              *reinterpret_cast<uint4*>(dst + c / 2 + h + j + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
          }
        }
      }
    }
  }
}

// MT: accumulators of 128 rows per tile (1 or 2; with 2 a tile has 256 rows of X, the second
// product of every step reads the same tile of W, and the block has eight epilogue warps).
// Two tiles' accumulators fit the 512 columns of tensor memory unless MT * BN = 512: then the
// products of the next tile wait for the epilogue of this one.
template <int MT, int BN, int EPI>
__global__ void __launch_bounds__(64 + 128 * MT, 1)
gemm_wide_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const Params p) {
  constexpr unsigned kStageBytes = (MT * BM + BN) * BK * 2;
  constexpr int NBUF = MT * BN * 2 <= 512 ? 2 : 1;
  constexpr unsigned kTmemCols = NBUF * MT * BN;   // a power of two >= 32
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bars = reinterpret_cast<Bars*>(base + (size_t)p.stages * kStageBytes);
  unsigned* tmem_holder = reinterpret_cast<unsigned*>(bars + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&bars->acc_full[a], 1); mbar_init(&bars->acc_empty[a], 4 * MT); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_holder, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = *tmem_holder;
  // the kernel behind this one may start only now: its resident, waiting blocks must not be
  // able to take tensor memory that a block of this grid still needs
  pdl_trigger();
  pdl_wait();

  const int total = p.m_tiles * p.n_tiles;
  bool failed = false;

  if (warp == 0) {
    // ---------------------------------------------------------------- loader
    if (lane == 0) {
      int it = 0;   // stages filled so far, over all tiles
      for (int tile = blockIdx.x; tile < total && !failed; tile += gridDim.x) {
        const int m0 = (tile % p.m_tiles) * (MT * BM), n0 = (tile / p.m_tiles) * BN;
        for (int k = 0; k < p.k_tiles; ++k, ++it) {
          const int s = it % p.stages;
          if (it >= p.stages && !wait_or_abort(&bars->empty[s], (unsigned)(it / p.stages - 1) & 1u, abort_flag)) {
            failed = true;
            break;
          }
          unsigned char* a_s = base + (size_t)s * kStageBytes;
          mbar_expect_tx(&bars->full[s], kStageBytes);
          tma_load_2d(a_s, &map_x, k * BK, m0, &bars->full[s]);
          tma_load_2d(a_s + MT * BM * BK * 2, &map_w, k * BK, n0, &bars->full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- tcgen05.mma issuer
    if (lane == 0) {
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
      int it = 0, n_local = 0;
      for (int tile = blockIdx.x; tile < total && !failed; tile += gridDim.x, ++n_local) {
        const int acc = n_local % NBUF;
        // the epilogue has read this accumulator's last contents (tile n_local - NBUF)
        if (n_local >= NBUF && !wait_or_abort(&bars->acc_empty[acc], (unsigned)(n_local / NBUF - 1) & 1u, abort_flag)) {
          failed = true;
          break;
        }
        tc_fence_after();
        const unsigned d = tmem + (unsigned)(acc * MT * BN);
        for (int k = 0; k < p.k_tiles; ++k, ++it) {
          const int s = it % p.stages;
          if (!wait_or_abort(&bars->full[s], (unsigned)(it / p.stages) & 1u, abort_flag)) { failed = true; break; }
          tc_fence_after();
          const unsigned a_addr = smem_u32(base + (size_t)s * kStageBytes);
          const unsigned long long bd = smem_desc_sw128(a_addr + MT * BM * BK * 2);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
#pragma unroll
            for (int t = 0; t < MT; ++t)   // the second 128 rows of X meet the same tile of W
              umma_bf16(d + t * BN, smem_desc_sw128(a_addr + t * BM * BK * 2) + 2 * kk, bd + 2 * kk, idesc,
                        (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&bars->empty[s]);
        }
        if (!failed) umma_commit(&bars->acc_full[acc]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;                 // the lanes of tensor memory this warp may read
    const int half = (warp - 2) >> 2;             // which of the tile's accumulators
    const int r = half * BM + quarter * 32 + lane;   // row of the tile
    const unsigned lane_base = tmem + ((unsigned)(quarter * 32) << 16);
    int n_local = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++n_local) {
      const int acc = n_local % NBUF;
      const int m = (tile % p.m_tiles) * (MT * BM) + r, n0 = (tile / p.m_tiles) * BN;
      if (!wait_or_abort(&bars->acc_full[acc], (unsigned)(n_local / NBUF) & 1u, abort_flag)) { failed = true; break; }
      tc_fence_after();
      const unsigned cols = lane_base + (unsigned)((acc * MT + half) * BN);
      epilogue_rows<BN, EPI>(p, cols, m, n0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
    }
  }
  if (failed) *abort_flag = 1;
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) atomicCAS(p.status, 0, KVB_STATUS_WAIT_TIMEOUT);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let copies and products that may still run finish
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// ------------------------------------------------------------------ the same on pairs of SMs
// Two blocks of a cluster share a tile of 256 rows of X and 256 features (tcgen05 with
// cta_group::2): each block loads its 128 rows of X and its 128 of the 256 rows of W, 32 KB per
// 64 of K instead of 48, and holds the accumulator of its own rows (128 lanes x 256 columns, two
// of them).  The tensor cores of both SMs read both halves of W, so each SM's shared memory
// delivers a half of what a tile of its own would ask of it; that is what bounds the single form.
// Measured on a B200 (2048 rows): 0.35 us per 64 of K and pair, the tensor pipe of both SMs busy
// throughout; gate|up with its SiLU * up 95 us against 108 us single and 117 us for the library
// product followed by the activation kernel (97 us for the library product alone).
//   warp 0       of either block loads the block's own operands;
//   warp 1       of the first block (the leader) issues the products for both and hands stages
//                and accumulators back to both blocks (tcgen05.commit with multicast); warp 1 of
//                the second block tells the leader when the second block's operands of a stage
//                have arrived;
//   warps 2..5   of either block: the epilogue of the block's own rows; a finished read is
//                reported to the leader's barrier.
__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The same without release semantics: for a thread that only passes on what a barrier of its own
// block told it (the arrival of tiles by TMA).  An arrival with release semantics waits for the
// thread's earlier memory operations to be visible in the whole cluster, and a thread that makes
// one per stage then passes on a stage a microsecond.
__device__ __forceinline__ void mbar_arrive_remote_relaxed(void* my_bar, unsigned rank) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(my_bar)), "r"(rank));
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// Arrives on the barrier that `my_bar` names, in block `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(void* my_bar, unsigned rank) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(my_bar)), "r"(rank));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(void* holder, unsigned cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(unsigned taddr, unsigned cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc,
                                               unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once the products issued so far are complete, on the barrier at this place in both blocks.
__device__ __forceinline__ void umma_commit_pair(void* bar) {
  const unsigned short mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

// PBN: features per tile (each block loads a half of these rows of W).  Only 256 is built: tiles
// of 192 features, which would cut 3072 features into rounds of three quarters the length, took
// 0.69 us per stage against 0.35 us for 256 when they were measured.
constexpr int pair_stages(int pbn) { return pbn == 256 ? 6 : 7; }

template <int PBN, int EPI>
__global__ void __launch_bounds__(192, 1)
gemm_wide_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const Params p) {
  constexpr unsigned kHalfBytes = BM * BK * 2;           // 128 rows of 128 bytes
  constexpr unsigned kStageBytes = kHalfBytes + (PBN / 2) * BK * 2;   // this block's rows of X and of W
  constexpr unsigned kTmemCols = 512;                    // two accumulators, 256 columns apart
  constexpr int kPairStages = pair_stages(PBN);
  constexpr int kPairBN = PBN;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bars = reinterpret_cast<Bars*>(base + (size_t)kPairStages * kStageBytes);
  unsigned* tmem_holder = reinterpret_cast<unsigned*>(bars + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const unsigned rank = cluster_rank();
  const bool leader = rank == 0;
  if (tid == 0) {
    // the leader's `full` waits for its own bytes and for the second block's word
    for (int s = 0; s < kPairStages; ++s) { mbar_init(&bars->full[s], leader ? 2 : 1); mbar_init(&bars->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&bars->acc_full[a], 1); mbar_init(&bars->acc_empty[a], 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(tmem_holder, kTmemCols);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // no block signals a barrier of its peer before that barrier is set up
  tc_fence_after();
  const unsigned tmem = *tmem_holder;
  pdl_trigger();
  pdl_wait();

  const int total = p.m_tiles * p.n_tiles;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  bool failed = false;

  if (warp == 0) {
    // ---------------------------------------------------------------- loader (both blocks)
    if (lane == 0) {
      int it = 0;
      for (int tile = pair; tile < total && !failed; tile += pairs) {
        const int m0 = (tile % p.m_tiles) * (2 * BM) + (int)rank * BM;
        const int n0 = (tile / p.m_tiles) * kPairBN + (int)rank * (kPairBN / 2);
        for (int k = 0; k < p.k_tiles; ++k, ++it) {
          const int s = it % kPairStages;
          if (leader) KVB_STAMP(3);
          if (it >= kPairStages && !wait_or_abort(&bars->empty[s], (unsigned)(it / kPairStages - 1) & 1u, abort_flag)) {
            failed = true;
            break;
          }
          unsigned char* a_s = base + (size_t)s * kStageBytes;
          mbar_expect_tx(&bars->full[s], kStageBytes);
          tma_load_2d(a_s, &map_x, k * BK, m0, &bars->full[s]);
          tma_load_2d(a_s + kHalfBytes, &map_w, k * BK, n0, &bars->full[s]);
          KVB_STAMP(leader ? 4 : 6);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------------------------------------------------------- tcgen05.mma issuer (leader)
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(kPairBN >> 3) << 17) | ((unsigned)((2 * BM) >> 4) << 24);
      int it = 0, n_local = 0;
      for (int tile = pair; tile < total && !failed; tile += pairs, ++n_local) {
        const int acc = n_local & 1;
        if (n_local >= 2 && !wait_or_abort(&bars->acc_empty[acc], (unsigned)((n_local >> 1) - 1) & 1u, abort_flag)) {
          failed = true;
          break;
        }
        tc_fence_after();
        const unsigned d = tmem + (unsigned)(acc * 256);
        for (int k = 0; k < p.k_tiles; ++k, ++it) {
          const int s = it % kPairStages;
          KVB_STAMP(0);
          if (!wait_or_abort(&bars->full[s], (unsigned)(it / kPairStages) & 1u, abort_flag)) { failed = true; break; }
          KVB_STAMP(1);
          tc_fence_after();
          const unsigned a_addr = smem_u32(base + (size_t)s * kStageBytes);
          const unsigned long long ad = smem_desc_sw128(a_addr), bd = smem_desc_sw128(a_addr + kHalfBytes);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) umma_bf16_pair(d, ad + 2 * kk, bd + 2 * kk, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          umma_commit_pair(&bars->empty[s]);
          KVB_STAMP(2);
        }
        if (!failed) umma_commit_pair(&bars->acc_full[acc]);
      }
    } else if (lane == 0) {
      // ---------------------------------------------------------------- the second block's word
      int it = 0;
      for (int tile = pair; tile < total && !failed; tile += pairs) {
        for (int k = 0; k < p.k_tiles; ++k, ++it) {
          const int s = it % kPairStages;
          if (!wait_or_abort(&bars->full[s], (unsigned)(it / kPairStages) & 1u, abort_flag)) { failed = true; break; }
          KVB_STAMP(5);
          mbar_arrive_remote_relaxed(&bars->full[s], 0);
          KVB_STAMP(7);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both blocks)
    const int quarter = warp & 3;
    const int r = (int)rank * BM + quarter * 32 + lane;      // row of the pair's tile
    const unsigned lane_base = tmem + ((unsigned)(quarter * 32) << 16);
    int n_local = 0;
    for (int tile = pair; tile < total; tile += pairs, ++n_local) {
      const int acc = n_local & 1;
      const int m = (tile % p.m_tiles) * (2 * BM) + r, n0 = (tile / p.m_tiles) * kPairBN;
      if (!wait_or_abort(&bars->acc_full[acc], (unsigned)(n_local >> 1) & 1u, abort_flag)) { failed = true; break; }
      tc_fence_after();
      const unsigned cols = lane_base + (unsigned)(acc * 256);
      epilogue_rows<PBN, EPI>(p, cols, m, n0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(&bars->acc_empty[acc], 0);
    }
  }
  if (failed) *abort_flag = 1;
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) atomicCAS(p.status, 0, KVB_STATUS_WAIT_TIMEOUT);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  cluster_sync_all();     // neither block leaves while the other may still signal its barriers or read its tiles
  if (warp == 1) tmem_dealloc_pair(tmem, kTmemCols);
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

// A [rows, K] bfloat16 row-major matrix as a 2-D tensor map with boxes of box_rows x 64 and the
// 128-byte swizzle; what lies outside the matrix reads as zeros.
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return KVB_ERR_BAD_SIZE;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
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

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1)
      n = kvb_sm_count();
  }
  return n;
}

template <int MT, int BN, int EPI>
int launch_wide(const CUtensorMap& mx, const CUtensorMap& mw, Params p, cudaStream_t stream) {
  const size_t stage_bytes = (size_t)(MT * BM + BN) * BK * 2;
  int stages = (int)((220 * 1024 - 1024 - sizeof(Bars) - 64) / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p.stages = stages;
  const size_t smem = 1024 + stages * stage_bytes + sizeof(Bars) + 64;
  static bool attr_set = false;   // one per instantiation
  if (!attr_set) {
    cudaError_t ce = cudaFuncSetAttribute(gemm_wide_kernel<MT, BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    attr_set = true;
  }
  const int total = p.m_tiles * p.n_tiles;
  const int blocks = total < sm_count() ? total : sm_count();
  kvb_launch(gemm_wide_kernel<MT, BN, EPI>, dim3(blocks), dim3(64 + 128 * MT), smem, stream, mx, mw, p);
  return kvb_launch_result();
}

// The pairs are persistent: there must be no more of them than the GPU holds at a time (fewer
// than SMs / 2 where a group of SMs that can host a cluster has an odd number of them free), or
// the ones left over would run after the others, each with a full share of tiles.
unsigned long long* g_trace = nullptr;   // set by kvb_gemm_wide_trace

template <int PBN, int EPI>
int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, Params p, cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)pair_stages(PBN) * (BM + PBN / 2) * BK * 2 + sizeof(Bars) + 64;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static int max_pairs = 0;
  if (!max_pairs) {
    cudaError_t ce = cudaFuncSetAttribute(gemm_wide_pair_kernel<PBN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    cfg.gridDim = dim3(2 * (sm_count() / 2), 1, 1);
    cfg.numAttrs = 1;
    int n = 0;
    ce = cudaOccupancyMaxActiveClusters(&n, gemm_wide_pair_kernel<PBN, EPI>, &cfg);
    if (ce != cudaSuccess) return (int)ce;
    if (n < 1) return KVB_ERR_BAD_SIZE;
    max_pairs = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  const int total = p.m_tiles * p.n_tiles;
  const int pairs = total < max_pairs ? total : max_pairs;
  p.stages = pair_stages(PBN);
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.numAttrs = kvb_pdl_enabled() ? 2 : 1;
  cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_wide_pair_kernel<PBN, EPI>, mx, mw, p);
  if (le != cudaSuccess) return (int)le;
  return kvb_launch_result();
}

}  // namespace

// The tile that kvb_gemm_wide takes for a problem when the caller leaves the choice to it:
// rows of X (128 or 256), features (64, 128 or 256), and whether two blocks share it.  The one
// with the least rounds of tiles over the SMs (over the pairs of SMs), each round weighted by the
// time a tile of that shape takes per 64 of K (measured on a B200, microseconds: a single block
// is bound by the operand bytes it takes in per product, a pair by the tensor pipe).
KVB_EXPORT int kvb_gemm_wide_tile(int M, int N, int epilogue, int* rows, int* cols, int* pair) {
  const int sms = sm_count();
  double best_cost = 0;
  *rows = 0;
  for (int form = 0; form < 5; ++form) {
    const int bm = form >= 3 ? 256 : 128, bn = form == 0 ? 64 : form == 1 ? 128 : 256, pr = form == 4;
    if (epilogue == EPI_SWIGLU && bn == 64) continue;
    if (epilogue == EPI_RESIDUAL && form != 2 && form != 4) continue;
    const double per_tile = form == 0 ? 0.40 : form == 1 ? 0.41 : form == 2 ? 0.45
                          : form == 3 ? (epilogue == EPI_SWIGLU ? 0.95 : 0.83) : 0.36;
    const int tiles = ((M + bm - 1) / bm) * ((N + bn - 1) / bn);
    const int slots = pr ? sms / 2 : sms;
    const double cost = (double)((tiles + slots - 1) / slots) * per_tile;
    if (!*rows || cost < best_cost) { *rows = bm; *cols = bn; *pair = pr; best_cost = cost; }
  }
  return 0;
}

namespace {

struct Extras {
  // row scale
  const float* x_sumsq = nullptr; int x_parts = 0; float eps = 0.f;
  // EPI_RESIDUAL
  float* resid = nullptr; int ld_resid = 0; __nv_bfloat16* xb_out = nullptr; float* sumsq_out = nullptr;
};

int gemm_wide_launch(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                     int epilogue, int bm, int bn, int pair, const Extras& ex, int* status, cudaStream_t stream) {
  if (M < 1 || N < 1) return 0;
  if (K < 8 || (K & 7) || epilogue < EPI_STORE || epilogue > EPI_RESIDUAL) return KVB_ERR_BAD_SIZE;
  if (epilogue == EPI_SWIGLU ? (N & 127) : (N & 7)) return KVB_ERR_BAD_SIZE;
  if ((ldx & 7) || (ldw & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return KVB_ERR_ALIGN;
  if (epilogue == EPI_RESIDUAL) {
    if (!ex.resid || !ex.xb_out || !ex.sumsq_out || ex.x_sumsq || ex.ld_resid < N) return KVB_ERR_BAD_SIZE;
    if ((ex.ld_resid & 3) || (reinterpret_cast<uintptr_t>(ex.resid) & 15) || (reinterpret_cast<uintptr_t>(ex.xb_out) & 15))
      return KVB_ERR_ALIGN;
  } else {
    if ((ldo & 7) || (reinterpret_cast<uintptr_t>(out) & 15)) return KVB_ERR_ALIGN;
    if (ex.x_sumsq && ex.x_parts < 1) return KVB_ERR_BAD_SIZE;
  }
  if (bm == 0 && bn == 0) kvb_gemm_wide_tile(M, N, epilogue, &bm, &bn, &pair);
  if (pair) {
    if (bm != 256 || bn != 256) return KVB_ERR_BAD_SIZE;
  } else {
    if (bn != 64 && bn != 128 && bn != 256) return KVB_ERR_BAD_SIZE;
    if (bm != 128 && !(bm == 256 && bn == 256)) return KVB_ERR_BAD_SIZE;
    if (bn == 64 && epilogue == EPI_SWIGLU) return KVB_ERR_BAD_SIZE;
    if (epilogue == EPI_RESIDUAL && !(bm == 128 && bn == 256)) return KVB_ERR_BAD_SIZE;
  }
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.m_tiles = (M + bm - 1) / bm;
  p.n_tiles = (N + bn - 1) / bn;
  p.k_tiles = (K + BK - 1) / BK;
  p.stages = 0;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.store32 = (ldo % 16 == 0) && (reinterpret_cast<uintptr_t>(out) % 32 == 0) && (N % 16 == 0);
  p.x_sumsq = ex.x_sumsq; p.x_parts = ex.x_parts; p.eps = ex.eps;
  p.resid = ex.resid; p.ld_resid = ex.ld_resid; p.xb_out = ex.xb_out; p.sumsq_out = ex.sumsq_out;
  p.status = status;
  p.trace = g_trace;
  CUtensorMap mx, mw;
  int e = make_map(&mx, x, M, K, ldx, pair ? BM : bm);
  if (e) return e;
  e = cached_map(&mw, w, N, K, ldw, pair ? bn / 2 : bn);
  if (e) return e;
  if (pair) {
    if (epilogue == EPI_STORE) return launch_pair<256, EPI_STORE>(mx, mw, p, stream);
    if (epilogue == EPI_SWIGLU) return launch_pair<256, EPI_SWIGLU>(mx, mw, p, stream);
    return launch_pair<256, EPI_RESIDUAL>(mx, mw, p, stream);
  }
  if (epilogue == EPI_RESIDUAL) return launch_wide<1, 256, EPI_RESIDUAL>(mx, mw, p, stream);
  if (epilogue == EPI_STORE) {
    if (bm == 256) return launch_wide<2, 256, EPI_STORE>(mx, mw, p, stream);
    if (bn == 64) return launch_wide<1, 64, EPI_STORE>(mx, mw, p, stream);
    if (bn == 128) return launch_wide<1, 128, EPI_STORE>(mx, mw, p, stream);
    return launch_wide<1, 256, EPI_STORE>(mx, mw, p, stream);
  }
  if (bm == 256) return launch_wide<2, 256, EPI_SWIGLU>(mx, mw, p, stream);
  if (bn == 128) return launch_wide<1, 128, EPI_SWIGLU>(mx, mw, p, stream);
  return launch_wide<1, 256, EPI_SWIGLU>(mx, mw, p, stream);
}

}  // namespace

// C = X[M,K] . W[N,K]^T, bfloat16, float32 accumulation.  ldx, ldw, ldo in elements; x, w and
// out aligned to 16 bytes, ldx, ldw, ldo and K multiples of 8.
// epilogue 0: out[M, N] = C, N a multiple of 8.
// epilogue 1: the rows of W come in blocks of 128, 64 gate features and then the 64 up features
//             of the same indices; out[M, N/2], out[m, 64 t + j] = silu(gate) * up; N a multiple
//             of 128.
// bm x bn: the tile, 128 x 64 (epilogue 0 only), 128 x 128, 128 x 256 or 256 x 256, or 0, 0 for
// the choice of kvb_gemm_wide_tile.  pair != 0 (with 256 x 256 only): the tile is shared by the
// two blocks of a cluster (cta_group::2).  Uses no memory beyond its operands.
KVB_EXPORT int kvb_gemm_wide(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                             int epilogue, int bm, int bn, int pair, int* status, cudaStream_t stream) {
  if (epilogue == EPI_RESIDUAL) return KVB_ERR_BAD_SIZE;
  return gemm_wide_launch(x, ldx, w, ldw, out, ldo, M, N, K, epilogue, bm, bn, pair, Extras(), status, stream);
}

// The same product with the residual stream's add and RMSNorm folded around it.
//  - x_sumsq != nullptr (row scale): row m of the result is multiplied by
//    rsqrt(sum_p x_sumsq[m, p] / K + eps) before the epilogue (0 or 1) sees it; x holds the
//    bare residual rows in bfloat16 and W has the norm's weight multiplied into its columns.
//  - epilogue 2 (EPI_RESIDUAL): resid[M, ld_resid] += X . W^T in place (float32, 16-byte aligned
//    rows), xb_out[M, N] gets the new rows in bfloat16 and sumsq_out[M, ceil(N/256)] their partial
//    sums of squares; out unused; tiles of 128 x 256, or 256 x 256 on pairs.
KVB_EXPORT int kvb_gemm_wide_fused(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N,
                                   int K, int epilogue, int bm, int bn, int pair, const float* x_sumsq, int x_parts,
                                   float eps, float* resid, int ld_resid, void* xb_out, float* sumsq_out, int* status,
                                   cudaStream_t stream) {
  Extras ex;
  ex.x_sumsq = x_sumsq; ex.x_parts = x_parts; ex.eps = eps;
  ex.resid = resid; ex.ld_resid = ld_resid; ex.xb_out = reinterpret_cast<__nv_bfloat16*>(xb_out);
  ex.sumsq_out = sumsq_out;
  return gemm_wide_launch(x, ldx, w, ldw, out, ldo, M, N, K, epilogue, bm, bn, pair, ex, status, stream);
}

// Profiling: the kernels of pairs write the phase stamps (globaltimer, ns) of the first pair's
// first 64 stages to buf [64][8] (device memory): 0 the issuer starts to wait for the stage,
// 1 has it, 2 has issued its products; 3 the leader's loader starts to wait for the stage to be
// free, 4 has requested its tiles; 5 the second block's tiles are there, 7 the leader has been
// told; 6 the second block's loader has requested them.  nullptr switches the stamps off.
KVB_EXPORT void kvb_gemm_wide_trace(unsigned long long* buf) { g_trace = buf; }
