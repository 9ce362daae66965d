// Row-wise kernels of the decoder: embedding gather, residual-add + RMSNorm,
// SiLU-multiply, and rotary encoding fused with the write of keys and values
// into cache pages.  Each takes float32 or bfloat16 activations; statistics,
// rotation and the residual sum are float32 in both.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// residual[t, :] = table[ids[t], :]   (upstream: base/src/kernels.cu:279-287)
// An id below zero names a token that the sampling kernel of the step before left on the
// device: -(1 + r) stands for sampled[r] (n_sampled entries), so that a step can be
// launched before the host has seen the tokens it starts from.
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    const int* __restrict__ sampled, int n_sampled,
                                    float* __restrict__ resid, int H, int V, int* status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && sampled && -(id + 1) < n_sampled) id = sampled[-(id + 1)];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_BAD_TOKEN);
    for (int i = threadIdx.x; i < H; i += blockDim.x) resid[(size_t)t * H + i] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) resid[(size_t)t * H + i] = to_f32(row[i]);
}

KVB_EXPORT int kvb_embed_gather(const void* table, int dtype, const int* ids, const int* sampled, int n_sampled,
                                float* resid, int T_, int H, int V, int* status, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(embed_gather_kernel<T>, dim3(T_), dim3(threads), 0, stream,
                                            (const T*)table, ids, sampled, n_sampled, resid, H, V, status)));
  return kvb_launch_result();
}

// ---------------------------------------------------------------- add + RMSNorm
// v = resid[row] (+ delta[row]);  resid[row] = v (when delta is given and rows is null);
// out[b] = v / sqrt(mean(v^2) + eps) * w          (upstream: base/src/kernels.cu:10-43)
// Each thread keeps its share of the row in registers between the two passes (up to
// kNormVec*4 elements per thread, 16-byte accesses).  Sums run in a fixed order that
// depends on H and the block size only, never on the batch.
constexpr int kNormThreads = 256;
constexpr int kNormVec = 8;   // float4 groups per thread: rows up to 256*8*4 = 8192 wide stay in registers

template <typename T> struct Pack4;
template <> struct Pack4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Pack4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                       __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&a);
    u.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

__device__ __forceinline__ float block_sum(float v, float* warp_part) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  const int nw = blockDim.x >> 5;
  for (int i = 0; i < nw; ++i) t += warp_part[i];   // every thread adds the warps' sums in the same order
  return t;
}

template <typename T>
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ w,
                       T* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
  __shared__ float warp_part[32];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x;
  const size_t src = (size_t)(rows ? rows[b] : b) * H;
  const int groups = H >> 2;
  float4 v[kNormVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNormVec; ++i) {
    const int g = i * kNormThreads + threadIdx.x;
    if (g < groups) {
      float4 x = *reinterpret_cast<const float4*>(resid + src + 4 * g);
      if (delta) {
        const float4 d = Pack4<T>::load(delta + src + 4 * g);
        x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w;
        if (!rows) *reinterpret_cast<float4*>(resid + src + 4 * g) = x;
      }
      v[i] = x;
      ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, warp_part) / (float)H + eps);
  T* o = out + (size_t)b * H;
#pragma unroll
  for (int i = 0; i < kNormVec; ++i) {
    const int g = i * kNormThreads + threadIdx.x;
    if (g < groups) {
      const float4 ww = w ? *reinterpret_cast<const float4*>(w + 4 * g) : make_float4(1.f, 1.f, 1.f, 1.f);
      Pack4<T>::store(o + 4 * g, make_float4(v[i].x * inv * ww.x, v[i].y * inv * ww.y, v[i].z * inv * ww.z,
                                             v[i].w * inv * ww.w));
    }
  }
}

// General form: any H, the row is kept in shared memory between the two passes.
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
  const float inv = 1.0f / sqrtf(block_sum(ss, warp_part) / (float)H + eps);
  T* o = out + (size_t)b * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<T>(row_cache[i] * inv * (w ? w[i] : 1.0f));
}

KVB_EXPORT int kvb_add_rmsnorm(float* resid, const void* delta, const float* w, void* out,
                               const int* rows, int n_out_rows, int H, float eps, int dtype,
                               cudaStream_t stream) {
  if (n_out_rows <= 0) return 0;
  if (H % 4 == 0 && H <= kNormThreads * kNormVec * 4) {
    KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(add_rmsnorm_vec_kernel<T>, dim3(n_out_rows), dim3(kNormThreads), 0,
                                              stream, resid, (const T*)delta, w, (T*)out, rows, H, eps)));
    return kvb_launch_result();
  }
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
// out[t, i] = g * (1 / (1 + exp(-g))) * u  (upstream: base/src/kernels.cu:45-52).
// A row of gu holds gate and up in blocks of BL: [gate 0..BL) | up 0..BL) | gate BL..2BL) | ...],
// so g = gu[t, (i / BL) * 2 BL + i % BL] and u = BL further.  BL = I is the plain [gate | up] row.
// Four elements per thread when BL % 4 == 0.
__device__ __forceinline__ float silu_mul_one(float g, float u) { return g * (1.0f / (1.0f + expf(-g))) * u; }

template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int BL, size_t groups) {
  pdl_trigger();
  pdl_wait();
  const int gpr = I >> 2;  // groups of four per row
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < groups;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / gpr;
    const int i = (int)(idx - t * gpr) << 2;
    const size_t at = t * 2 * I + (size_t)(i / BL) * 2 * BL + (i % BL);
    const float4 g = Pack4<T>::load(gu + at);
    const float4 u = Pack4<T>::load(gu + at + BL);
    Pack4<T>::store(out + t * I + i, make_float4(silu_mul_one(g.x, u.x), silu_mul_one(g.y, u.y),
                                                 silu_mul_one(g.z, u.z), silu_mul_one(g.w, u.w)));
  }
}

// bfloat16 with blocks that are multiples of 8: eight elements per thread, 16-byte accesses.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I,
                                       int BL, size_t groups) {
  pdl_trigger();
  pdl_wait();
  const int gpr = I >> 3;  // groups of eight per row
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < groups;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / gpr;
    const int i = (int)(idx - t * gpr) << 3;
    const size_t at = t * 2 * I + (size_t)(i / BL) * 2 * BL + (i % BL);
    const uint4 g = *reinterpret_cast<const uint4*>(gu + at);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + at + BL);
    const unsigned gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    unsigned ow[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float a = silu_mul_one(__uint_as_float(gw[k] << 16), __uint_as_float(uw[k] << 16));
      const float b = silu_mul_one(__uint_as_float(gw[k] & 0xffff0000u), __uint_as_float(uw[k] & 0xffff0000u));
      __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
      ow[k] = *reinterpret_cast<unsigned*>(&v);
    }
    *reinterpret_cast<uint4*>(out + t * I + i) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int BL, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const size_t at = t * 2 * I + (size_t)(i / BL) * 2 * BL + (i % BL);
    out[idx] = from_f32<T>(silu_mul_one(to_f32(gu[at]), to_f32(gu[at + BL])));
  }
}

KVB_EXPORT int kvb_silu_mul(const void* gu, void* out, int T_, int I, int BL, int dtype, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (BL < 1 || I % BL) return KVB_ERR_BAD_SIZE;
  const int threads = 256;
  if (dtype == KVB_BF16 && BL % 8 == 0 && (reinterpret_cast<uintptr_t>(gu) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const size_t work8 = (size_t)T_ * (I / 8);
    const size_t want8 = (work8 + threads - 1) / threads;
    const int blocks8 = (int)(want8 < (size_t)kvb_sm_count() * 32 ? want8 : (size_t)kvb_sm_count() * 32);
    kvb_launch(silu_mul_bf16x8_kernel, dim3(blocks8), dim3(threads), 0, stream, (const __nv_bfloat16*)gu,
               (__nv_bfloat16*)out, I, BL, work8);
    return kvb_launch_result();
  }
  const bool vec = (BL % 4 == 0);
  const size_t work = vec ? (size_t)T_ * (I / 4) : (size_t)T_ * I;
  size_t want = (work + threads - 1) / threads;
  const int blocks = (int)(want < (size_t)kvb_sm_count() * 32 ? want : (size_t)kvb_sm_count() * 32);
  if (vec) {
    KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(silu_mul_vec_kernel<T>, dim3(blocks), dim3(threads), 0, stream,
                                              (const T*)gu, (T*)out, I, BL, work)));
  } else {
    KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(silu_mul_kernel<T>, dim3(blocks), dim3(threads), 0, stream,
                                              (const T*)gu, (T*)out, I, BL, work)));
  }
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

// The same for the common case of a full rotary dimension (rot == d): 16 bytes per
// access.  A work item is VEC consecutive dims j..j+VEC-1 of a head's lower half together
// with the matching dims of the upper half (q and k heads), or VEC dims of a v head.
template <typename T> struct Vec16;
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* f) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<unsigned*>(&v);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                         const int* __restrict__ token_req, const float* __restrict__ cos_t,
                                         const float* __restrict__ sin_t, int table_len, T* __restrict__ k_pages,
                                         T* __restrict__ v_pages, const int* __restrict__ block_table,
                                         int max_pages, int page_size, int num_pages, int nq, int nkv, int d,
                                         int* status) {
  constexpr int VEC = Vec16<T>::N;
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = d >> 1;
  if (pos < 0 || pos >= table_len) {
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
      dst = ((size_t)page * nkv * page_size + (pos % page_size)) * d;
    }
  }
  const int per_rot = half / VEC;            // items per rotated head
  const int per_v = d / VEC;                 // items per v head
  const int n_rot = (nq + nkv) * per_rot;
  const int n_items = n_rot + nkv * per_v;
  const float* cr = cos_t + (size_t)pos * half;
  const float* sr = sin_t + (size_t)pos * half;
  for (int w = threadIdx.x; w < n_items; w += blockDim.x) {
    if (w < n_rot) {
      const int head = w / per_rot, j = (w - head * per_rot) * VEC;
      T* x = row + (size_t)head * d;
      float x1[VEC], x2[VEC], a[VEC], b[VEC];
      Vec16<T>::load(x + j, x1);
      Vec16<T>::load(x + j + half, x2);
      // the angles of these VEC pairs, four at a time (j is a multiple of VEC, VEC of 4; the tables' rows
      // start on 16 bytes when half is a multiple of 4, which the launcher checks)
      float cs[VEC], sn[VEC];
#pragma unroll
      for (int e = 0; e < VEC; e += 4) {
        *reinterpret_cast<float4*>(cs + e) = *reinterpret_cast<const float4*>(cr + j + e);
        *reinterpret_cast<float4*>(sn + e) = *reinterpret_cast<const float4*>(sr + j + e);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        a[e] = x1[e] * cs[e] - x2[e] * sn[e];
        b[e] = x1[e] * sn[e] + x2[e] * cs[e];
      }
      if (head < nq) {
        Vec16<T>::store(x + j, a);
        Vec16<T>::store(x + j + half, b);
      } else if (write) {
        T* kd = k_pages + dst + (size_t)(head - nq) * page_size * d;
        Vec16<T>::store(kd + j, a);
        Vec16<T>::store(kd + j + half, b);
      }
    } else if (write) {
      const int wv = w - n_rot;
      const int head = wv / per_v, j = (wv - head * per_v) * VEC;
      const uint4 val = *reinterpret_cast<const uint4*>(row + (size_t)(nq + nkv + head) * d + j);
      *reinterpret_cast<uint4*>(v_pages + dst + (size_t)head * page_size * d + j) = val;
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
  const int esz = dtype == KVB_F32 ? 4 : 2;
  if (cos_t != nullptr && rot == d && (d / 2) % (16 / esz) == 0 && dtype <= KVB_BF16 &&
      ((reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t)) & 15) == 0) {
    const int items = (nq + nkv) * (d / 2) / (16 / esz) + nkv * d / (16 / esz);
    const int th = items >= 192 ? 256 : (items >= 96 ? 128 : 64);
    KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(rope_kv_write_vec_kernel<T>, dim3(T_), dim3(th), 0, stream, (T*)qkv,
                                              positions, token_req, cos_t, sin_t, table_len, (T*)k_pages,
                                              (T*)v_pages, block_table, max_pages, page_size, num_pages, nq, nkv, d,
                                              status)));
    return kvb_launch_result();
  }
  const int work = (nq + 2 * nkv) * (d / 2);
  const int threads = work >= 1024 ? 256 : 128;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(rope_kv_write_kernel<T>, dim3(T_), dim3(threads), 0, stream, (T*)qkv,
                                            positions, token_req, cos_t, sin_t, table_len, (T*)k_pages,
                                            (T*)v_pages, block_table, max_pages, page_size, num_pages, nq, nkv, d,
                                            rot, status)));
  return kvb_launch_result();
}
