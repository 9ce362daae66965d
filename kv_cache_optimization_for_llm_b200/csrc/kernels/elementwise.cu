// Row-wise kernels of the decoder: embedding gather, residual-add + RMSNorm,
// SiLU-multiply, and rotary encoding fused with the write of keys and values
// into cache pages.  Each takes float32 or bfloat16 activations; statistics,
// rotation and the residual sum are float32 in both.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// residual[t, :] = table[ids[t], :]   (upstream: base/src/kernels.cu:279-287)
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ resid, int H, int V, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_BAD_TOKEN);
    for (int i = threadIdx.x; i < H; i += blockDim.x) resid[(size_t)t * H + i] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) resid[(size_t)t * H + i] = to_f32(row[i]);
}

KVB_EXPORT int kvb_embed_gather(const void* table, int dtype, const int* ids, float* resid, int T_,
                                int H, int V, int* status, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(embed_gather_kernel<T>, dim3(T_), dim3(threads), 0, stream,
                                            (const T*)table, ids, resid, H, V, status)));
  return kvb_launch_result();
}

// ---------------------------------------------------------------- add + RMSNorm
// v = resid[row] (+ delta[row]);  resid[row] = v (when delta is given and rows is null);
// out[b] = v / sqrt(mean(v^2) + eps) * w          (upstream: base/src/kernels.cu:10-43)
// The row is kept in shared memory between the two passes.  Sums run in a fixed
// order that depends on H and the block size only, never on the batch.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const float* __restrict__ w, T* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps) {
  extern __shared__ float row_cache[];
  __shared__ float warp_part[32];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  const size_t src = (size_t)(rows ? rows[b] : b) * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = resid[src + i];
    if (delta) {
      v += to_f32(delta[src + i]);
      if (!rows) resid[src + i] = v;
    }
    row_cache[i] = v;
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? warp_part[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) warp_part[0] = 1.0f / sqrtf(v / (float)H + eps);
  }
  __syncthreads();
  const float inv = warp_part[0];
  T* o = out + (size_t)b * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<T>(row_cache[i] * inv * w[i]);
}

KVB_EXPORT int kvb_add_rmsnorm(float* resid, const void* delta, const float* w, void* out,
                               const int* rows, int n_out_rows, int H, float eps, int dtype,
                               cudaStream_t stream) {
  if (n_out_rows <= 0) return 0;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return KVB_ERR_BAD_SIZE;  // widths above 51200 are refused
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  KVB_DISPATCH_DTYPE(dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    kvb_launch(add_rmsnorm_kernel<T>, dim3(n_out_rows), dim3(threads), smem, stream, resid, (const T*)delta, w,
               (T*)out, rows, H, eps);
  });
  return kvb_launch_result();
}

// ---------------------------------------------------------------- SiLU * up
// out[t, i] = g * (1 / (1 + exp(-g))) * u with g = gu[t, i], u = gu[t, I + i]
// (upstream: base/src/kernels.cu:45-52)
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_f32(gu[t * 2 * I + i]);
    const float u = to_f32(gu[t * 2 * I + I + i]);
    out[idx] = from_f32<T>(g * (1.0f / (1.0f + expf(-g))) * u);
  }
}

KVB_EXPORT int kvb_silu_mul(const void* gu, void* out, int T_, int I, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  const size_t total = (size_t)T_ * I;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads
                                                                      : 148 * 16);
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(silu_mul_kernel<T>, dim3(blocks), dim3(threads), 0, stream, (const T*)gu,
                                            (T*)out, I, total)));
  return kvb_launch_result();
}

// ---------------------------------------------------------------- rotary + cache write
// qkv is [T, (nq + 2*nkv) * d]: q heads, then k heads, then v heads.  For token t at
// position p: q and k heads are rotated by the rotate-half rule on the first `rot`
// dims, pairs (j, j + rot/2):  x[j] = x1*c - x2*s ; x[j+rot/2] = x1*s + x2*c with
// c,s = cos,sin[p, j]  (upstream: base/src/kernels.cu:289-319).  q is rewritten in
// place; k (rotated) and v go to the page that holds position p of the token's
// request: pages[page, head, p % page_size, :]  (upstream: paged_attention/src/kernels.cu:335-360).
// k_pages == nullptr: the layer reads another layer's cache, only q is rotated.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ token_req,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                     int table_len, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     const int* __restrict__ block_table, int max_pages, int page_size,
                                     int num_pages, int nq, int nkv, int d, int rot, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rot >> 1;
  const bool rotary = cos_t != nullptr && rot > 0;
  if (rotary && (pos < 0 || pos >= table_len)) {
    if (threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_BAD_POSITION);
    return;
  }
  T* row = qkv + (size_t)t * (nq + 2 * nkv) * d;
  size_t dst = 0;
  bool write = k_pages != nullptr;
  if (write) {
    const int lp = pos / page_size;
    const int page = (lp < max_pages) ? block_table[(size_t)token_req[t] * max_pages + lp] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
      write = false;
    } else {
      dst = ((size_t)page * nkv * page_size + (pos % page_size)) * d;  // + head * page_size * d
    }
  }
  const int halfd = d >> 1;  // work items per head: one per pair of the head's dims
  const int n_rot_heads = nq + nkv;
  for (int w = threadIdx.x; w < (nq + 2 * nkv) * halfd; w += blockDim.x) {
    const int head = w / halfd;
    const int j = w - head * halfd;
    T* x = row + (size_t)head * d;
    if (head < n_rot_heads) {
      // Pair (j, j + half) inside the rotary part; dims beyond it pass through.
      float a, b;
      int ia, ib;
      if (rotary && j < half) {
        ia = j; ib = j + half;
        const float x1 = to_f32(x[ia]), x2 = to_f32(x[ib]);
        const float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
        a = x1 * c - x2 * s;
        b = x1 * s + x2 * c;
      } else {
        // the 2*(halfd - half) pass-through dims, two per work item
        const int k = rotary ? j - half : j;
        ia = (rotary ? rot : 0) + 2 * k; ib = ia + 1;
        a = to_f32(x[ia]); b = to_f32(x[ib]);
      }
      if (head < nq) {
        x[ia] = from_f32<T>(a);
        x[ib] = from_f32<T>(b);
      } else if (write) {
        T* kd = k_pages + dst + (size_t)(head - nq) * page_size * d;
        kd[ia] = from_f32<T>(a);
        kd[ib] = from_f32<T>(b);
      }
    } else if (write) {
      T* vd = v_pages + dst + (size_t)(head - nq - nkv) * page_size * d;
      vd[2 * j] = x[2 * j];
      vd[2 * j + 1] = x[2 * j + 1];
    }
  }
}

KVB_EXPORT int kvb_rope_kv_write(void* qkv, const int* positions, const int* token_req,
                                 const float* cos_t, const float* sin_t, int table_len,
                                 void* k_pages, void* v_pages, const int* block_table, int max_pages,
                                 int page_size, int num_pages, int T_, int nq, int nkv, int d, int rot,
                                 int dtype, int* status, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (d % 2 || rot % 2 || rot > d) return KVB_ERR_BAD_SIZE;
  const int work = (nq + 2 * nkv) * (d / 2);
  const int threads = work >= 1024 ? 256 : 128;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(rope_kv_write_kernel<T>, dim3(T_), dim3(threads), 0, stream, (T*)qkv,
                                            positions, token_req, cos_t, sin_t, table_len, (T*)k_pages,
                                            (T*)v_pages, block_table, max_pages, page_size, num_pages, nq, nkv, d,
                                            rot, status)));
  return kvb_launch_result();
}
