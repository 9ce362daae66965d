// The attention of a bfloat16 decode step in one launch, on tensor cores.
//
// Every request brings one query token.  The 128-key tiles of a request's context fall into
// C classes (tile t belongs to class t mod C; C is 4, 8 or 16 by the token's own position,
// never by the batch: more classes for longer contexts, up to the kernel's capacity, which
// the caller chooses from the longest context it allows).  A class is one running softmax over
// its tiles; the C class results are merged in class order.  So the sums of a token are
// cut at absolute positions and added in one fixed order, whatever else is in the batch.
// A cluster of S blocks (a power of two up to the capacity; the launcher takes a smaller S
// for a larger batch) serves one (request, key/value head): block z walks the classes z,
// z + S, ... below C one after the other (a block beyond C has nothing to do).  S changes
// who computes a class, not what is computed.  The rows of the tensor-core tile are the query
// heads that share the key/value head (padded to 16), so keys and values are fetched
// once for the whole group (upstream fetches them once per query head:
// paged_attention/src/kernels.cu:150-219).
//
// Per block: the keys and values of its first two tiles are requested (head size 64: cp.async, 16-byte
// chunks gathered through the block table; head size 128: whole pages by TMA through a tensor map over
// the layer's pages; either way into two swizzled shared-memory stages) before
// the block waits for the projection kernel in front of it; then the group's queries are
// rotated (rotary encoding, float32) and the block that owns the tile of the token's
// own position rotates the new key, stores key and value in the cache and, when that
// tile is one of the two under way, in its stage by hand (a later tile fetches them from
// the cache).  While a tile is multiplied the tile after the next is requested.  Each warp walks its own 32-key slice of every tile of the block: it multiplies
// the queries with the keys (mma.sync m16n8k16, float32 accumulate), keeps a running
// max and sum per head and a running output, and multiplies the probabilities with its
// 32 values; no block-wide barrier inside the walk.  The four warps' partials are
// merged in warp order, and each block sends one partial
// (output, max, sum per head) into the shared memory of block 0 of its cluster
// (distributed shared memory); after the cluster's hardware barrier block 0 merges the
// S partials in block order and writes the output.  No scratch in global memory,
// no counters, no spinning.
#include "common.cuh"
#include "page_maps.cuh"

#include <cuda.h>
#include <math_constants.h>

#include <cstdint>
#include <cstdlib>

namespace {

constexpr int kThreads = 128;
constexpr int kTile = 128;     // keys per tile (32 per warp)
constexpr unsigned kSpinLimit = 20u * 1000u * 1000u;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
// Bounded wait that also ends at once when the block has given up somewhere else.  false: gave up.
__device__ __forceinline__ bool mbar_wait_or_abort(void* bar, unsigned parity, volatile int* abort_flag,
                                                   unsigned limit = kSpinLimit) {
  for (unsigned i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
// One box of a tensor map (x: column, y: row of its first element) into shared memory; the bytes are counted on bar.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"((unsigned long long)map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// Orders what this thread did to shared memory by ordinary loads and stores before copies by TMA that follow.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 16 bytes into shared memory; `valid` false: zeros are written and nothing is read.
__device__ __forceinline__ void cp_async_16_zfill(void* smem_dst, const void* gmem_src, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(n) : "memory");
}
// 2^x by the special-function unit alone (exp2f wraps the same instruction in a rescaling for
// results below 2^-126, which a probability does not need).  ex2(-inf) = 0.
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
// Waits until at most N of this thread's committed groups are still under way.
template <int N> __device__ __forceinline__ void cp_async_wait_but() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
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
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_peer_f32(void* my_smem_ptr, unsigned rank, float v) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote) : "r"((unsigned)__cvta_generic_to_shared(my_smem_ptr)), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
// Byte offset of 16-byte chunk `chunk` of row `row` in a warp's slice of a tile, 32 rows of D bfloat16:
// sub-tiles of 64 columns side by side (one at head size 64, two at 128), each [32 rows][128 bytes] with
// the chunks of a row XOR-swizzled with the row, so that the 8 rows of an 8x8 matrix hit 8 bank groups.
// This is the 128-byte swizzle of TMA for a sub-tile that starts on a 1024-byte boundary.
template <int D> __device__ __forceinline__ int swz(int row, int chunk) {
  return (chunk >> 3) * (32 * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// How many classes the tiles of a token at position pos fall into: 4 below 2048, 8 below 8192,
// 16 beyond (32 tiles of 128 keys per class at most up to 65536 positions).
__host__ __device__ __forceinline__ int classes_at(int pos) { return pos < 2048 ? 4 : (pos < 8192 ? 8 : 16); }

// GP: the group of query heads padded to 4, 8 or 16 (rows that are kept).  kClasses: classes
// of tiles per (request, kv head); gridDim.z = cluster size = blocks that share them.  kStages: tiles in shared memory at a time, 2 when the whole grid
// is resident at once anyway (small batches: the second tile is under way before the
// projection has finished), 1 when more blocks per SM matter more (large batches).  The
// order of the sums is the same for both.
// kTma: keys and values come page by page (boxes of min(page size, 32) rows) through tensor maps over the
// layer's pages, counted on one mbarrier per stage and warp; needs pages of at least 8 rows.  Otherwise
// 16 bytes at a time by cp.async (any page size).  The launcher takes TMA at head size 128, where it measured
// faster, and cp.async at head size 64, where the boxes of a page are 2 KB and it did not.
template <int D, int GP, int kClasses, int kStages, bool kTma>
__global__ void __launch_bounds__(kThreads, D == 64 ? 4 : 2)   // four blocks per SM at head size 64: 128 registers
decode_attention_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const __nv_bfloat16* __restrict__ qkv, int q_row_stride,
                            __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages, int write_kv,
                            const int* __restrict__ block_table, int max_pages, int page_shift, int num_pages,
                            const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_len, int rot,
                            __nv_bfloat16* __restrict__ out, int nq, int nkv, int G, float scale_log2, int window,
                            int* status, unsigned long long* trace) {
  constexpr int CPK = D / 8;      // 16-byte chunks per row
  constexpr int KSTEPS = D / 16;
  constexpr int DT = D / 8;       // n-tiles of the output
  constexpr int PW = D + 2;       // floats per head in a partial: output dims, max, sum
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // (the swizzle of TMA follows the address: the stages start on a 1024-byte boundary)
  unsigned char* smem = kTma ? reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023))
                             : smem_raw;
  constexpr int kTileBytes = 4 * 32 * D * 2;                   // keys (or values) of one tile
  constexpr int kSub = D / 64;                                 // sub-tiles of 64 columns
  unsigned char* k_s = smem;                                   // [kStages][4][32][D] bf16, swizzled
  unsigned char* v_s = k_s + kStages * kTileBytes;             // [kStages][4][32][D]
  float* q_s = reinterpret_cast<float*>(v_s + kStages * kTileBytes); // [GP][D] rotated, scaled queries
  float* run = q_s + GP * D;                                   // [GP][PW] this block's partial so far
  float* recv = run + GP * PW;                                 // [kClasses][GP][PW], used in block 0 only
  float* wpart = recv + kClasses * GP * PW;                    // [4][GP][PW] the four warps' partials of a class
  // kTma only:
  unsigned long long* full_b = reinterpret_cast<unsigned long long*>(wpart + 4 * GP * PW);   // [kStages][4] bytes of a slice
  __nv_bfloat16* newkv_s = reinterpret_cast<__nv_bfloat16*>(full_b + kStages * 4);           // [2][D] the new key and value
  int* abort_flag = reinterpret_cast<int*>(newkv_s + 2 * D);                                 // a wait ran out

  pdl_trigger();
  const int hk = blockIdx.x, r = blockIdx.y, z = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // profiling only: nanosecond stamps of this block's phases, [blocks][8]
  auto stamp = [&](int slot) {
    if (trace && tid == 0) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      trace[(((size_t)r * gridDim.x + hk) * gridDim.z + z) * 8 + slot] = now;
    }
  };
  stamp(0);   // block started
  const int page_mask = (1 << page_shift) - 1;
  const int pos = ctx_len[r] - 1;   // lengths and block tables were written before the step's kernels started
  const bool bad = pos < 0 || (cos_t != nullptr && pos >= table_len);
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int* table = block_table + (size_t)r * max_pages;
  const int half = rot >> 1;
  const bool rotary = cos_t != nullptr && rot > 0;
  const int n_tiles = bad ? 0 : pos / kTile + 1;
  const int t_first = lo / kTile;               // tiles below it hold no key the window keeps
  const int t_star = bad ? -1 : pos / kTile;    // the tile of the token's own position
  // Classes of tiles for this token: a function of its own position only (and of the kernel's
  // capacity kClasses, which the launcher takes from the longest context of the step).
  const int C = min(kClasses, classes_at(pos));

  for (int i = tid; i < GP * PW; i += kThreads) run[i] = ((i % PW) == D) ? -CUDART_INF_F : 0.f;

  // Requests this warp's 32 keys and values of tile t into a stage and returns the mask of this warp's
  // keys that are there.  In two steps, so that the look-up in the block table (a load whose answer the
  // addresses wait for) can be started a tile's worth of work before the requests go out.
  //
  // By cp.async, key by key: `skip_pos` leaves the token's own position out (it is placed by hand); keys
  // that are absent (beyond the context, outside the window) are filled with zeros, so that a probability
  // of zero times whatever lay there before cannot turn into NaN.
  // By TMA, page by page: a slice of 32 keys is 32 / box_rows boxes, lane c looks up and requests box c;
  // a box without a key in reach, or without a page, is requested beyond the end of the map, where TMA
  // delivers zeros.  Rows of a box that hold no key in reach (the page's rows beyond the context, or in
  // front of the window) arrive as they lie in the cache: their scores are masked, and their values
  // are set to zero once the slice is there.  The row of the token's own position is overwritten then too.
  const int box_shift = page_shift < 5 ? page_shift : 5;     // kTma: rows per box = min(page size, 32)
  const int n_box = 32 >> box_shift;
  const int total_rows = (num_pages * nkv) << page_shift;    // kTma: the first row beyond the map
  // Step one: where this lane's key (cp.async: an offset in elements; -1: absent, zero-fill; -2: placed by
  // hand, leave alone) or this lane's box (TMA: a row of the map) of tile t lies.
  auto locate_key = [&](int t, bool skip_pos) -> long long {
    if constexpr (kTma) {
      int row = total_rows;
      const int kj = t * kTile + warp * 32 + (lane << box_shift);
      if (lane < n_box && kj <= pos && kj + (1 << box_shift) > lo) {
        const int lp = kj >> page_shift;
        const int page = lp < max_pages ? table[lp] : -1;
        if (page < 0 || page >= num_pages) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
        else row = (((page * nkv) + hk) << page_shift) + (kj & page_mask);
      }
      return row;
    } else {
      const int j = t * kTile + warp * 32 + lane;
      long long off = -1;
      if (skip_pos && j == pos) off = -2;
      else if (j <= pos && j >= lo) {
        const int lp = j >> page_shift;
        const int page = lp < max_pages ? table[lp] : -1;
        if (page < 0 || page >= num_pages) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
        else off = ((((long long)page * nkv + hk) << page_shift) + (j & page_mask)) * D;
      }
      return off;
    }
  };
  // Step two: the requests.
  auto request_located = [&](int t, int stage, long long off) -> unsigned {
    unsigned char* kd = k_s + stage * kTileBytes + warp * 32 * D * 2;
    unsigned char* vd = v_s + stage * kTileBytes + warp * 32 * D * 2;
    if constexpr (kTma) {
      const int row = (int)off;
      const int j = t * kTile + warp * 32 + lane;
      const int box_row = __shfl_sync(0xffffffffu, row, lane >> box_shift);
      const unsigned there = __ballot_sync(0xffffffffu, j <= pos && j >= lo && box_row != total_rows);
      if (there != 0u) {
        // what this warp read from or wrote to the slice by hand comes before the copies that overwrite it
        fence_proxy_async_smem();
        __syncwarp();
        unsigned long long* bar = full_b + stage * 4 + warp;
        if (lane == 0) mbar_expect_tx(bar, 2u * 32u * D * 2u);
        __syncwarp();                                          // the bytes are expected before any copy can report
        if (lane < n_box) {
          const int at = (lane << box_shift) * 128;
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub) {
            tma_load_2d(kd + sub * (32 * 128) + at, &map_k, 64 * sub, row, bar);
            tma_load_2d(vd + sub * (32 * 128) + at, &map_v, 64 * sub, row, bar);
          }
        }
      }
      return there;
    } else {
#pragma unroll
      for (int i = 0; i < CPK; ++i) {
        const int c = i * 32 + lane;
        const int key = c / CPK, part = c % CPK;
        const long long oj = __shfl_sync(0xffffffffu, off, key);
        if (oj != -2) {
          const long long src = oj >= 0 ? oj + part * 8 : 0;
          cp_async_16_zfill(kd + swz<D>(key, part), k_pages + src, oj >= 0);
          cp_async_16_zfill(vd + swz<D>(key, part), v_pages + src, oj >= 0);
        }
      }
      return __ballot_sync(0xffffffffu, off >= 0);
    }
  };
  auto request_tile = [&](int t, int stage, bool skip_pos) -> unsigned {
    return request_located(t, stage, locate_key(t, skip_pos));
  };

  // The first tiles of this block's first class: on their way before the projection kernel
  // has finished.  Every thread commits one group per stage at the start of a class and one
  // per tile walked, requests or not, so that "all but the newest group(s)" always means
  // "the tile that is multiplied next".
  const int S = (int)gridDim.z;
  int my_first = z;                              // first tile of the class that is being walked
  while (my_first < t_first) my_first += C;
  int n_mine = (z < C && my_first < n_tiles) ? (n_tiles - 1 - my_first) / C + 1 : 0;   // a block beyond the classes has no tile
  unsigned have[kStages];                        // per stage: which of this warp's 32 keys are there
#pragma unroll
  for (int s = 0; s < kStages; ++s) have[s] = 0u;
  // (the stage of a tile is known only at run time; these keep the masks in registers all the same)
  auto have_of = [&](int stage) -> unsigned {
    unsigned h = have[0];
#pragma unroll
    for (int s = 1; s < kStages; ++s) h = stage == s ? have[s] : h;
    return h;
  };
  auto set_have = [&](int stage, unsigned h) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) have[s] = stage == s ? h : have[s];
  };
  auto request_first_tiles = [&](bool skip_pos) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      have[s] = n_mine > s ? request_tile(my_first + s * C, s, skip_pos) : 0u;
      if constexpr (!kTma) cp_async_commit();
    }
  };
  unsigned parity = 0u;                          // kTma: bit s is the phase that stage s's barrier completes next
  if constexpr (kTma) {
    if (tid == 0) {
      for (int i = 0; i < kStages * 4; ++i) mbar_init(full_b + i, 1);
      *abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
  }
  // A layer that reads another layer's cache finds the key and value of the token's own
  // position there: the owning layer's attention wrote them earlier in this same step, several
  // launches back.  The wait below orders this kernel behind all of those, a read in front of
  // it does not; so a block whose first tiles hold that position asks for them after the wait.
  const bool own_key_from_this_step = !bad && !write_kv && t_star >= my_first && (t_star - my_first) % C == 0 &&
                                      (t_star - my_first) / C < kStages;
  if (!own_key_from_this_step) request_first_tiles(write_kv != 0);

  // The new key and value are stored by the block that owns their tile; where they go does
  // not depend on the projection in front, so the page is looked up before the wait.
  const int c_star = bad ? 0 : t_star % C;                  // the class of the new key's tile
  const bool owner = !bad && write_kv && (t_star >= t_first) && (c_star % S == z);
  int own_page = -1;
  if (owner) {
    const int lp = pos >> page_shift;
    own_page = lp < max_pages ? table[lp] : -1;
    if (own_page < 0 || own_page >= num_pages) {
      if (tid == 0) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
      own_page = -1;
    }
  }
  const bool own_t = own_page >= 0 && tid < D;              // this thread carries dim `tid` of the new key and value

  // The rotation's angle depends on the position only, and a thread meets one dim of the head in
  // all its work (the block's threads are a multiple of the head size): fetched before the wait.
  static_assert(kThreads % D == 0, "a thread must keep its dim of the head");
  const size_t q_row = (size_t)q_start[r];       // the host wrote it, like the lengths: no need to wait for it
  float rot_c = 1.f, rot_s = 0.f;
  if (!bad && rotary && (tid % D) < rot) {
    const int dd = tid % D, j = dd < half ? dd : dd - half;
    rot_c = cos_t[(size_t)pos * half + j];
    rot_s = sin_t[(size_t)pos * half + j];
  }

  pdl_wait();
  stamp(1);   // the projection in front has finished
  if (own_key_from_this_step) request_first_tiles(false);
  const __nv_bfloat16* row = qkv + q_row * q_row_stride;
  // the owner's loads go out first, so that they are under way while the queries are rotated
  float nk1 = 0.f, nk2 = 0.f;
  const float nc = rot_c, ns = rot_s;
  __nv_bfloat16 nv = __float2bfloat16_rn(0.f);
  if (own_t) {
    const __nv_bfloat16* kh = row + (size_t)(nq + hk) * D;
    const int dd = tid;
    if (rotary && dd < rot) {
      const int j = dd < half ? dd : dd - half;
      nk1 = to_f32(kh[j]);
      nk2 = to_f32(kh[j + half]);
    } else {
      nk1 = to_f32(kh[dd]);
    }
    nv = row[(size_t)(nq + nkv + hk) * D + dd];
  }
  if (!bad) {
    // the group's queries, rotated (pairs (j, j + rot/2) of the first rot dims), scaled, float32
    for (int i = tid; i < GP * D; i += kThreads) {
      const int g = i / D, dd = i % D;
      float val = 0.f;
      if (g < G) {
        const __nv_bfloat16* qh = row + (size_t)(hk * G + g) * D;
        if (rotary && dd < rot) {
          const int j = dd < half ? dd : dd - half;
          const float c = rot_c, sn = rot_s;
          const float x1 = to_f32(qh[j]), x2 = to_f32(qh[j + half]);
          val = dd < half ? x1 * c - x2 * sn : x1 * sn + x2 * c;
        } else {
          val = to_f32(qh[dd]);
        }
      }
      q_s[i] = val * scale_log2;
    }
    // the new key and value
    if (owner && own_page >= 0) {
      {
        const size_t dst = ((((size_t)own_page * nkv + hk) << page_shift) + (pos & page_mask)) * D;
        const int star_i = (t_star - my_first) / C;   // which tile of its class it is
        const bool direct = c_star == z && star_i < kStages;   // its tile is one of those already requested
        const int slot = pos - t_star * kTile;          // 0..127: warp slot>>5, key slot&31
        if (own_t) {
          const int dd = tid;
          const float val = (rotary && dd < rot) ? (dd < half ? nk1 * nc - nk2 * ns : nk1 * ns + nk2 * nc) : nk1;
          const __nv_bfloat16 kr = __float2bfloat16_rn(val);
          k_pages[dst + dd] = kr;
          v_pages[dst + dd] = nv;
          if constexpr (kTma) {
            // kept for the warp that walks the slice of this position: it overwrites the row of the
            // slice with them once the slice has arrived (the page may have been fetched before this store)
            newkv_s[dd] = kr;
            newkv_s[D + dd] = nv;
          } else if (direct) {
            const int key = slot & 31;
            const int off_b = star_i * kTileBytes + (slot >> 5) * 32 * D * 2 + swz<D>(key, dd >> 3) + (dd & 7) * 2;
            *reinterpret_cast<__nv_bfloat16*>(k_s + off_b) = kr;
            *reinterpret_cast<__nv_bfloat16*>(v_s + off_b) = nv;
          }
        }
        if constexpr (!kTma) {
          if (direct) {
            if (warp == (slot >> 5)) set_have(star_i, have_of(star_i) | (1u << (slot & 31)));
          }
          else __threadfence();   // a later tile of this block fetches it from L2
        }
      }
    }
  }
  __syncthreads();
  stamp(2);   // queries rotated, new key and value stored

  // query fragments (A operand, rows = heads): row lane/4 and lane/4 + 8, bfloat16
  unsigned qf[KSTEPS][4];
  {
    const int r0 = lane >> 2, c0 = (lane & 3) << 1;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int c = kk * 16 + c0;
      qf[kk][0] = r0 < GP ? pack_bf16(q_s[r0 * D + c], q_s[r0 * D + c + 1]) : 0u;
      qf[kk][1] = r0 + 8 < GP ? pack_bf16(q_s[(r0 + 8) * D + c], q_s[(r0 + 8) * D + c + 1]) : 0u;
      qf[kk][2] = r0 < GP ? pack_bf16(q_s[r0 * D + c + 8], q_s[r0 * D + c + 9]) : 0u;
      qf[kk][3] = r0 + 8 < GP ? pack_bf16(q_s[(r0 + 8) * D + c + 8], q_s[(r0 + 8) * D + c + 9]) : 0u;
    }
  }

  // Class after class.  Each warp walks its 32-key slices of the class's tiles on its own, with
  // a running max and sum per head (rows lane/4 and lane/4 + 8) and a running output in
  // registers; the slices of a warp are private to it, so the walk needs no block-wide barrier.
  for (int cls = z; cls < C; cls += S) {
  if (cls != z) {
    // the new key, if in this class, is in the cache by now
    my_first = cls;
    while (my_first < t_first) my_first += C;
    n_mine = my_first < n_tiles ? (n_tiles - 1 - my_first) / C + 1 : 0;
    request_first_tiles(false);
  }
  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};
  float o[DT][4];
#pragma unroll
  for (int n = 0; n < DT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  for (int i = 0; i < n_mine; ++i) {
    const int stage = i % kStages;
    const unsigned char* kt = k_s + stage * kTileBytes + warp * 32 * D * 2;
    const unsigned char* vt = v_s + stage * kTileBytes + warp * 32 * D * 2;
    const unsigned hv = have_of(stage);
    // where the tile lies that takes this one's place in the ring: looked up now, asked for after the products
    const bool more = i + kStages < n_mine;
    const long long next_off = more ? locate_key(my_first + (i + kStages) * C, false) : -1;
    bool arrived = true;
    if constexpr (kTma) {
      if (hv != 0u) {
        arrived = mbar_wait_or_abort(full_b + stage * 4 + warp, (parity >> stage) & 1u, abort_flag);
        arrived = __all_sync(0xffffffffu, arrived);
        parity ^= 1u << stage;
        if (arrived) {
          unsigned char* vw = v_s + stage * kTileBytes + warp * 32 * D * 2;
          if (hv != 0xffffffffu && !((hv >> lane) & 1u)) {
            // this lane's key is not in reach: whatever the page holds in its row must not meet a probability of zero
#pragma unroll
            for (int c = 0; c < CPK; ++c) *reinterpret_cast<uint4*>(vw + swz<D>(lane, c)) = make_uint4(0u, 0u, 0u, 0u);
          }
          const int t_now = my_first + i * C;
          if (owner && own_page >= 0 && t_now == t_star && warp == ((pos - t_star * kTile) >> 5) && lane < 2 * CPK) {
            // the new key and value, as this block stored them: lanes 0 .. CPK-1 a chunk of the key each, the next CPK of the value
            const int key = (pos - t_star * kTile) & 31, c = lane % CPK;
            unsigned char* dstw = (lane < CPK ? k_s : v_s) + stage * kTileBytes + warp * 32 * D * 2 + swz<D>(key, c);
            *reinterpret_cast<uint4*>(dstw) = *reinterpret_cast<const uint4*>(newkv_s + (lane < CPK ? 0 : D) + c * 8);
          }
        } else if (lane == 0) {
          atomicCAS(status, 0, KVB_STATUS_WAIT_TIMEOUT);
        }
      }
    } else {
      cp_async_wait_but<kStages - 1>();
    }
    __syncwarp();
    if (hv != 0u && arrived) {
      float s[4][4];
#pragma unroll
      for (int n = 0; n < 4; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          unsigned b0, b1, b2, b3;
          const int key = np * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int chunk = kk * 2 + ((lane >> 3) & 1);
          ldmatrix_x4(b0, b1, b2, b3, kt + swz<D>(key, chunk));
          mma_bf16(s[2 * np], qf[kk], b0, b1);
          mma_bf16(s[2 * np + 1], qf[kk], b2, b3);
        }
      }
      float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
      if (hv != 0xffffffffu) {        // a slice at the context's end or at the window's edge
#pragma unroll
        for (int n = 0; n < 4; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = n * 8 + ((lane & 3) << 1) + (e & 1);
            if (!((hv >> key) & 1u)) s[n][e] = -CUDART_INF_F;
          }
        }
      }
#pragma unroll
      for (int n = 0; n < 4; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
      }
      float corr[2], m_use[2];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
        mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
        const float m_new = fmaxf(m_run[rr], mx[rr]);       // finite: the slice holds at least one key
        m_use[rr] = m_new;
        corr[rr] = m_run[rr] == -CUDART_INF_F ? 0.f : ex2(m_run[rr] - m_new);
        m_run[rr] = m_new;
        l_run[rr] *= corr[rr];
      }
      if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {    // a maximum has grown somewhere in the warp
#pragma unroll
        for (int n = 0; n < DT; ++n) { o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1]; }
      }
      unsigned pf[2][4];
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const float p0 = ex2(s[n][0] - m_use[0]), p1 = ex2(s[n][1] - m_use[0]);
        const float p2 = ex2(s[n][2] - m_use[1]), p3 = ex2(s[n][3] - m_use[1]);
        l_run[0] += p0 + p1;     // each lane keeps the sum of its own columns; the four lanes of a row
        l_run[1] += p2 + p3;     // are added up after the walk
        pf[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p0, p1);
        pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
        for (int dp = 0; dp < DT / 2; ++dp) {
          unsigned b0, b1, b2, b3;
          const int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int chunk = dp * 2 + (lane >> 4);
          ldmatrix_x4_trans(b0, b1, b2, b3, vt + swz<D>(key, chunk));
          mma_bf16(o[2 * dp], pf[kk], b0, b1);
          mma_bf16(o[2 * dp + 1], pf[kk], b2, b3);
        }
      }
    }
    __syncwarp();   // the slice is read; the next request may overwrite it
    if (more && arrived) set_have(stage, request_located(my_first + (i + kStages) * C, stage, next_off));
    else if (more) set_have(stage, 0u);   // (cp.async: the new key, if in that tile, is in the cache by now)
    if constexpr (!kTma) cp_async_commit();
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
    l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
  }
  if (cls == z) stamp(3);   // first class walked
  {
    const int r0 = lane >> 2, c0 = (lane & 3) << 1;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int rowi = r0 + rr * 8;
      if (rowi < GP) {
        float* dst = wpart + ((size_t)warp * GP + rowi) * PW;
#pragma unroll
        for (int n = 0; n < DT; ++n) { dst[n * 8 + c0] = o[n][rr * 2]; dst[n * 8 + c0 + 1] = o[n][rr * 2 + 1]; }
        if ((lane & 3) == 0) { dst[D] = m_run[rr]; dst[D + 1] = l_run[rr]; }
      }
    }
  }
  __syncthreads();
  // the four warps' partials, merged in warp order, are this block's partial
  for (int i = tid; i < GP * PW; i += kThreads) {
    const int g = i / PW, dd = i % PW;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, wpart[((size_t)w * GP + g) * PW + D]);
    float a = 0.f;
    if (dd == D) a = M;
    else if (M != -CUDART_INF_F) {
      const int col = dd == D + 1 ? D + 1 : dd;   // the sum merges like an output dim
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = wpart[((size_t)w * GP + g) * PW + D];
        if (mw != -CUDART_INF_F) a += wpart[((size_t)w * GP + g) * PW + col] * exp2f(mw - M);
      }
    }
    run[i] = a;
  }
  __syncthreads();

  // ---- the class's partial goes to block 0 of the cluster
  for (int i = tid; i < GP * PW; i += kThreads) st_peer_f32(recv + (size_t)cls * GP * PW + i, 0u, run[i]);
  }   // classes
  stamp(4);   // the block's partials are complete
  if constexpr (kTma) {
    // a wait ran out: copies may still be on their way into this block's shared memory
    if (*abort_flag) { for (int i = 0; i < 2000; ++i) __nanosleep(1000); }
  }
  // ---- block 0 merges the classes in class order
  cluster_sync_all();
  stamp(5);   // the cluster has met
  if (z != 0 || bad) {
    if (bad && z == 0 && tid == 0) atomicCAS(status, 0, KVB_STATUS_BAD_POSITION);
    return;
  }
  for (int i = tid; i < G * D; i += kThreads) {
    const int g = i / D, dd = i % D;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int c = 0; c < C; ++c) M = fmaxf(M, recv[((size_t)c * GP + g) * PW + D]);
    float L = 0.f, a = 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const float mc = recv[((size_t)c * GP + g) * PW + D];
      if (mc != -CUDART_INF_F) {
        const float f = exp2f(mc - M);
        L += recv[((size_t)c * GP + g) * PW + D + 1] * f;
        a += recv[((size_t)c * GP + g) * PW + dd] * f;
      }
    }
    out[(q_row * nq + hk * G + g) * D + dd] = __float2bfloat16_rn(L > 0.f ? a / L : 0.f);
  }
  stamp(6);   // output stored
}

// Two warps wait, with a limit of `polls`, on barriers that nothing ever completes: the first to run out
// raises the block's flag, the other sees the flag and leaves at once; the first reports what the attention
// kernel reports when a slice does not arrive.  flags_out[0]: the flag afterwards, [1]: polls the second warp made.
__global__ void decode_wait_selftest_kernel(unsigned polls, int* status, int* flags_out) {
  __shared__ unsigned long long bars[2];
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  // warp 1 gets a limit that it could not reach in the test's time: it must leave through the flag
  const bool ok = mbar_wait_or_abort(&bars[warp], 0, &abort_flag, warp == 0 ? polls : kSpinLimit);
  if (!ok && warp == 0 && (threadIdx.x & 31) == 0) atomicCAS(status, 0, KVB_STATUS_WAIT_TIMEOUT);
  __syncthreads();
  if (threadIdx.x == 0) flags_out[0] = abort_flag;
  if (threadIdx.x == 32) flags_out[1] = ok ? 1 : 0;
}

int log2_exact(int x) {
  int s = 0;
  while ((1 << s) < x) ++s;
  return (1 << s) == x ? s : -1;
}

template <int D, int GP, int kClasses, int kStages, bool kTma>
constexpr size_t smem_bytes() {
  constexpr int PW = D + 2;
  return (size_t)kStages * 2 * 4 * 32 * D * 2 + (size_t)GP * D * 4 + (size_t)GP * PW * 4 +
         (size_t)kClasses * GP * PW * 4 + (size_t)4 * GP * PW * 4 +
         (kTma ? 1024 + (size_t)kStages * 4 * 8 + 2 * D * 2 + 16 : 0);   // alignment, barriers, new key and value, flag
}

// How many clusters of `blocks_per_cluster` blocks of this form the GPU holds at once (0: the query failed).
template <int D, int GP, int kClasses, int kStages, bool kTma>
int clusters_at_once(int blocks_per_cluster) {
  static int answer[17] = {};      // by cluster size; 0: not asked yet, -1: the query failed
  if (answer[blocks_per_cluster] == 0) {
    constexpr size_t smem = smem_bytes<D, GP, kClasses, kStages, kTma>();
    auto* fn = decode_attention_mma_kernel<D, GP, kClasses, kStages, kTma>;
    int n = -1;
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess &&
        cudaFuncSetAttribute(fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(1, 1, blocks_per_cluster);
      cfg.blockDim = dim3(kThreads, 1, 1);
      cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = blocks_per_cluster;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int got = 0;
      if (cudaOccupancyMaxActiveClusters(&got, fn, &cfg) == cudaSuccess) n = got;
      else (void)cudaGetLastError();
    } else {
      (void)cudaGetLastError();
    }
    answer[blocks_per_cluster] = n > 0 ? n : -1;
  }
  return answer[blocks_per_cluster] > 0 ? answer[blocks_per_cluster] : 0;
}

template <int D, int GP, int kClasses, int kStages, bool kTma>
int launch(const CUtensorMap& map_k, const CUtensorMap& map_v, const void* qkv, int q_row_stride, void* k_pages, void* v_pages, int write_kv, const int* block_table,
           int max_pages, int page_shift, int num_pages, const int* q_start, const int* ctx_len, const float* cos_t,
           const float* sin_t, int table_len, int rot, void* out, int R, int nq, int nkv, float scale, int window,
           int blocks_per_cluster, int* status, unsigned long long* trace, cudaStream_t stream) {
  const size_t smem = smem_bytes<D, GP, kClasses, kStages, kTma>();
  static bool attr_set = false;
  if (!attr_set) {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(decode_attention_mma_kernel<D, GP, kClasses, kStages, kTma>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    if (kClasses > 8) {   // clusters of 16 are beyond the portable size
      cudaError_t e = cudaFuncSetAttribute(decode_attention_mma_kernel<D, GP, kClasses, kStages, kTma>,
                                           cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (e != cudaSuccess) return (int)e;
    }
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nkv, R, blocks_per_cluster);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = blocks_per_cluster;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = kvb_pdl_enabled() ? 2 : 1;
  cudaError_t le = cudaLaunchKernelEx(
      &cfg, decode_attention_mma_kernel<D, GP, kClasses, kStages, kTma>, map_k, map_v, (const __nv_bfloat16*)qkv, q_row_stride, (__nv_bfloat16*)k_pages,
      (__nv_bfloat16*)v_pages, write_kv, block_table, max_pages, page_shift, num_pages, q_start, ctx_len, cos_t, sin_t,
      table_len, rot, (__nv_bfloat16*)out, nq, nkv, nq / nkv, scale * 1.4426950408889634f, window, status, trace);
  if (le != cudaSuccess) return (int)le;
  return kvb_launch_result();
}

}  // namespace

// 1 when the kernel takes these sizes: head size 64 or 128, a group of at most 16 query
// heads per key/value head, a page size that is a power of two.
KVB_EXPORT int kvb_decode_attention_mma_supported(int d, int group, int page_size) {
  return (d == 64 || d == 128) && group >= 1 && group <= 16 && log2_exact(page_size) >= 0;
}

// qkv: [T, (nq + 2 nkv) d] bfloat16 as the projection wrote it; request r's token is row
// q_start[r] at position ctx_len[r]-1.  write_kv = 0: the layer reads another layer's
// cache and writes nothing.  cos_t/sin_t: [table_len, rot/2] or nullptr.  out: [T, nq d].
// max_ctx: the longest context of the step (a hint from the host, 0: unknown): it decides how
// many classes the kernel has room for and how many blocks share a (request, kv head), not
// the sums, which are cut by each token's own position.
// trace: nullptr, or [R * nkv * cluster, 8] uint64 for the phase stamps of every block (profiling only).
// Uses no memory beyond its operands.  R <= 65535.
KVB_EXPORT int kvb_decode_attention_mma(const void* qkv, int q_row_stride, void* k_pages, void* v_pages, int write_kv,
                                        const int* block_table, int max_pages, int page_size, int num_pages,
                                        const int* q_start, const int* ctx_len, const float* cos_t,
                                        const float* sin_t, int table_len, int rot, void* out, int R, int nq, int nkv,
                                        int d, float scale, int window, int max_ctx, int* status,
                                        unsigned long long* trace, cudaStream_t stream) {
  if (R <= 0) return 0;
  // the kernel is built for as many classes as the longest context of the step needs
  // (head size 128: 8 at most, for the shared memory the partials take)
  int cluster = max_ctx > 0 ? classes_at(max_ctx - 1) : 16;
  if (d != 64 && cluster > 8) cluster = 8;
  if (nkv < 1 || nq % nkv || !kvb_decode_attention_mma_supported(d, nq / nkv, page_size) || R > 65535 || (rot & 1) ||
      rot > d || nkv > 65535)
    return KVB_ERR_BAD_SIZE;
  const int G = nq / nkv;
  const int ps = log2_exact(page_size);
  // blocks per cluster: as many as there are classes while the grid stays small, fewer for
  // larger batches (every block then walks several classes and pays its fixed cost once)
  int S = cluster;
  // (an SM holds four blocks of head size 64 with one stage, two of head size 128: no second wave)
  while (S > 1 && (long long)R * nkv * S > (d == 64 ? 4 : 2) * kvb_sm_count()) S >>= 1;
  // Whole pages by TMA at head size 128 where the pages allow it (at least 8 rows, so that a box fills whole
  // rows of the swizzle pattern; addresses that a tensor map takes); key by key otherwise, at head size 128
  // then in the one-stage form only.  At head size 64 TMA measured level or slower (batch 8 at 4096 tokens
  // 18.3 against 16.3 us) and is not built.  KVB200_DECODE_TMA=0 switches it off (tests, comparisons).
  static const bool tma_off = [] { const char* e = getenv("KVB200_DECODE_TMA"); return e && e[0] == '0'; }();
  const long long rows = (long long)num_pages * nkv * page_size;
  const bool tma = !tma_off && d == 128 && page_size >= 8 && rows < (1ll << 31) - 64 &&
                   reinterpret_cast<uintptr_t>(k_pages) % 16 == 0 && reinterpret_cast<uintptr_t>(v_pages) % 16 == 0;
  CUtensorMap mk = {}, mv = {};
  if (tma) {
    const int box_rows = page_size < 32 ? page_size : 32;
    int e = kvb_page_maps::pages_map(&mk, k_pages, rows, box_rows, d);
    if (e) return e;
    e = kvb_page_maps::pages_map(&mv, v_pages, rows, box_rows, d);
    if (e) return e;
  }
  // Clusters that do not all run at once cost a second round, which doubles the time when the clusters are
  // few (a GPU holds fewer clusters of 16 than 148 / 16 times the blocks per SM: a cluster stays inside one
  // GPC).  So, for few clusters: half the blocks per cluster if that lets all run at once; and two stages only
  // if all clusters run at once with them (they need twice the shared memory).  Clusters of 8 and 16 with two
  // stages measured well only with one block per SM (head size 64, 64 000 tokens: two requests 97 us with two
  // stages, 61 us with one; four requests 130 to 150 us against 111 us), small clusters also with two.
#define KVB_DM_ARGS mk, mv, qkv, q_row_stride, k_pages, v_pages, write_kv, block_table, max_pages, ps, num_pages, q_start, \
                    ctx_len, cos_t, sin_t, table_len, rot, out, R, nq, nkv, scale, window, S, status, trace, stream
#define KVB_FITS(D, GP, CL, ST, TMA, SS) (clusters_at_once<D, GP, CL, ST, TMA>(SS) >= R * nkv)
#define KVB_PICK(D, GP, CL, TMA)                                                                          \
  do {                                                                                                    \
    if (cluster == CL) {                                                                                  \
      if (R * nkv <= 32 && S > 1 && !KVB_FITS(D, GP, CL, 1, TMA, S) && KVB_FITS(D, GP, CL, 1, TMA, S >> 1)) S >>= 1; \
      if ((long long)R * nkv * S <= (long long)((D == 64 && S < 8) ? 2 : 1) * kvb_sm_count() &&           \
          (S == 1 || KVB_FITS(D, GP, CL, 2, TMA, S)))                                                     \
        return launch<D, GP, CL, 2, TMA>(KVB_DM_ARGS);                                                    \
      return launch<D, GP, CL, 1, TMA>(KVB_DM_ARGS);                                                      \
    }                                                                                                     \
  } while (0)
#define KVB_DM64(GP) do { KVB_PICK(64, GP, 16, false); KVB_PICK(64, GP, 4, false); KVB_PICK(64, GP, 8, false); } while (0)
#define KVB_DM128(GP)                                                                                     \
  do {                                                                                                    \
    if (tma) { KVB_PICK(128, GP, 4, true); KVB_PICK(128, GP, 8, true); }                                  \
    if (cluster == 4) return launch<128, GP, 4, 1, false>(KVB_DM_ARGS);                                   \
    return launch<128, GP, 8, 1, false>(KVB_DM_ARGS);                                                     \
  } while (0)
  if (d == 64) { if (G <= 4) KVB_DM64(4); if (G <= 8) KVB_DM64(8); KVB_DM64(16); }
  if (G <= 4) KVB_DM128(4);
  if (G <= 8) KVB_DM128(8);
  KVB_DM128(16);
}

// Runs the bounded wait of this file's kernel against barriers that are never completed (see the kernel above);
// the context stays usable.  For tests of the give-up path.
KVB_EXPORT int kvb_decode_wait_selftest(unsigned polls, int* status, int* flags_out, cudaStream_t stream) {
  decode_wait_selftest_kernel<<<1, 64, 0, stream>>>(polls, status, flags_out);
  return kvb_launch_result();
}
