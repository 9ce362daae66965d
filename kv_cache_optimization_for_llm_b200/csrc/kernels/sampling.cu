// Token selection from float32 logits: greedy, or temperature sampling by inverse
// CDF with a counter-based uniform draw, both with an optional repetition penalty.
//
// One block per row does what upstream spreads over five kernels
// (argmaxPartial / argmaxFinalize / rowMax / expSumPartial / sampleFinalize,
// base/src/kernels.cu:515-835):
//   greedy:       the largest logit, the lower index winning a tie (:489-496);
//   temperature:  p ~ exp((l - max) / T); u = counter_uniform(seed, key, pos) (:638-649);
//                 the token is the first whose inclusive prefix sum exceeds u * total,
//                 the last token if rounding lets none exceed it (:733-835);
//   penalty:      a token the request already produced has its logit divided by the
//                 penalty when positive, multiplied when negative (:504-513).
// The draw depends on (seed, key, pos) only, so it is the same however requests are
// batched and after a request was dropped and recomputed.
#include "common.cuh"

#include <math_constants.h>

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ float counter_uniform(unsigned seed, unsigned key, unsigned pos) {
  unsigned long long z = ((unsigned long long)key << 32) ^ (unsigned long long)pos;
  z ^= (unsigned long long)seed * 0x9E3779B97F4A7C15ULL;
  z += 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);  // 24 bits: always below 1
}

__device__ __forceinline__ float penalised(const float* row, const unsigned char* mask, float pen, int i) {
  const float l = row[i];
  if (mask != nullptr && mask[i]) return l > 0.f ? l / pen : l * pen;
  return l;
}

__device__ __forceinline__ void better(float& bv, int& bi, float v, int i) {
  if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const unsigned* __restrict__ seed, const unsigned* __restrict__ key,
              const unsigned* __restrict__ pos, const float* __restrict__ penalty,
              unsigned char* __restrict__ mask_base, const int* __restrict__ slots,
              int* __restrict__ out_ids, const int* __restrict__ status_in, int status_at) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ float s_scan[kSampleThreads];
  __shared__ int s_owner;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* l = logits + (size_t)row * V;
  const float pen = penalty ? penalty[row] : 1.0f;
  unsigned char* mask = (mask_base != nullptr && pen != 1.0f) ? mask_base + (size_t)slots[row] * V : nullptr;

  // pass 1: maximum and its lowest index.  Without a penalty the row is read 16 bytes at a
  // time (the bulk of it; the ragged ends one by one).
  float bv = -CUDART_INF_F;
  int bi = 0x7fffffff;
  if (mask == nullptr) {
    const int head = (int)((16 - (reinterpret_cast<uintptr_t>(l) & 15)) & 15) / 4;   // floats before alignment
    const int lead = head < V ? head : V;
    const int groups = (V - lead) / 4;
    const float4* l4 = reinterpret_cast<const float4*>(l + lead);
    for (int g = tid; g < groups; g += kSampleThreads) {
      const float4 v = l4[g];
      const int i = lead + 4 * g;
      better(bv, bi, v.x, i); better(bv, bi, v.y, i + 1); better(bv, bi, v.z, i + 2); better(bv, bi, v.w, i + 3);
    }
    for (int i = tid; i < lead; i += kSampleThreads) better(bv, bi, l[i], i);
    for (int i = lead + 4 * groups + tid; i < V; i += kSampleThreads) better(bv, bi, l[i], i);
  } else {
    for (int i = tid; i < V; i += kSampleThreads) better(bv, bi, penalised(l, mask, pen, i), i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    better(bv, bi, ov, oi);
  }
  if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = s_val[lane]; bi = s_idx[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      better(bv, bi, ov, oi);
    }
    if (lane == 0) { s_val[0] = bv; s_idx[0] = bi; }
  }
  __syncthreads();
  const float row_max = s_val[0];
  int chosen = s_idx[0];
  const float T = temperature ? temperature[row] : 0.f;

  if (T > 0.f) {
    // pass 2: every thread owns a contiguous span; sums of the spans are scanned in
    // thread order, then the owner of the target walks its span.
    const float inv_t = 1.0f / T;
    const int span = (V + kSampleThreads - 1) / kSampleThreads;
    const int a = tid * span, b = min(V, a + span);
    float mine = 0.f;
    for (int i = a; i < b; ++i) mine += expf((penalised(l, mask, pen, i) - row_max) * inv_t);
    s_scan[tid] = mine;
    __syncthreads();
    // inclusive scan, Hillis-Steele: a fixed order of additions for a given V
    for (int o = 1; o < kSampleThreads; o <<= 1) {
      const float add = tid >= o ? s_scan[tid - o] : 0.f;
      __syncthreads();
      s_scan[tid] += add;
      __syncthreads();
    }
    const float total = s_scan[kSampleThreads - 1];
    const float target = counter_uniform(seed[row], key[row], pos[row]) * total;
    if (tid == 0) s_owner = -1;
    __syncthreads();
    const float before = tid ? s_scan[tid - 1] : 0.f;
    if (a < b && before <= target && target < s_scan[tid]) s_owner = tid;  // at most one thread
    __syncthreads();
    if (s_owner < 0) {
      chosen = V - 1;  // rounding left the target at or above the total
    } else if (tid == s_owner) {
      float acc = before;
      int pick = b - 1;
      for (int i = a; i < b; ++i) {
        acc += expf((penalised(l, mask, pen, i) - row_max) * inv_t);
        if (target < acc) { pick = i; break; }
      }
      s_idx[1] = pick;
    }
    __syncthreads();
    if (s_owner >= 0) chosen = s_idx[1];
  }
  if (tid == 0) {
    if (row == 0 && status_in) out_ids[status_at] = *status_in;   // the kernels' error word rides along
    out_ids[row] = chosen;
    if (mask != nullptr) mask[chosen] = 1;  // the new token counts as seen from now on
  }
}

// logits [R, V] float32.  temperature/seed/key/pos/penalty are per-row arrays;
// temperature == nullptr means greedy for all rows, penalty == nullptr means none.
// mask_base is [num_slots, V] bytes (1 = the request already produced this token),
// indexed through slots[row]; it may be nullptr when no row uses a penalty.
// status_in != nullptr: *status_in (the device word that kernels report errors into) is
// copied to out_ids[status_at], so that one transfer brings the tokens and the word.
KVB_EXPORT int kvb_sample(const float* logits, int R, int V, const float* temperature, const unsigned* seed,
                          const unsigned* key, const unsigned* pos, const float* penalty,
                          unsigned char* mask_base, const int* slots, int* out_ids, const int* status_in,
                          int status_at, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V < 1) return KVB_ERR_BAD_SIZE;
  sample_kernel<<<R, kSampleThreads, 0, stream>>>(logits, V, temperature, seed, key, pos, penalty, mask_base,
                                                  slots, out_ids, status_in, status_at);
  return kvb_launch_result();
}

// mask[slot, :] = 0, then mask[slot, tokens[i]] = 1: rebuilds a request's record of
// produced tokens when it is admitted again (upstream: markTokenListKernel,
// paged_attention/src/kernels.cu:254-262, after a cudaMemset of the row).
__global__ void reset_mask_kernel(unsigned char* mask_row, int V, const int* tokens, int n, int phase) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (phase == 0) {
    if (i < V) mask_row[i] = 0;
  } else if (i < n) {
    const int t = tokens[i];
    if (t >= 0 && t < V) mask_row[t] = 1;
  }
}

KVB_EXPORT int kvb_reset_mask(unsigned char* mask_base, int slot, int V, const int* tokens, int n,
                              cudaStream_t stream) {
  unsigned char* row = mask_base + (size_t)slot * V;
  reset_mask_kernel<<<(V + 255) / 256, 256, 0, stream>>>(row, V, tokens, 0, 0);
  if (n > 0) reset_mask_kernel<<<(n + 255) / 256, 256, 0, stream>>>(row, V, tokens, n, 1);
  return kvb_launch_result();
}
