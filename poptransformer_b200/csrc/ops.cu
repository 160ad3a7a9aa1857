// Small decode-path ops: Int4ToHalf, NormCE, RMSNorm(+residual), SoftmaxV3, dense KVCache / KVCachePipeline,
// top-k, BeamSearch, FP8 cast / reference FP8 matmul, RWKV WKV, embedding, loop carry.  All are HBM- or
// latency-bound elementwise / row-reduction kernels; each follows the reference arithmetic rounding by rounding.
#include <cfloat>

#include "common.cuh"

namespace pt {

// ------------------------------------------------------------------------------------------ Int4ToHalf
// axis 1: w int8 [n, m] -> out fp16 [2m, n].  32x32 byte tile through shared memory so that both the byte reads
// (along m) and the fp16 writes (along n) are coalesced.
__global__ void int4_to_half_axis1_kernel(const int8_t *__restrict__ w, const __half *__restrict__ scale, int n, int m, int group,
                                          __half *__restrict__ out) {
  __shared__ int8_t tile[32][33];
  const int j0 = blockIdx.x * 32, i0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int i = i0 + r, j = j0 + threadIdx.x;
    tile[r][threadIdx.x] = (i < n && j < m) ? w[(size_t)i * m + j] : (int8_t)0;
  }
  __syncthreads();
  const int ngroups = group > 0 ? (2 * m) / group : 1;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int j = j0 + r, i = i0 + threadIdx.x;
    if (i < n && j < m) {
      const int8_t b = tile[threadIdx.x][r];
      const int hi = b >> 4;                       // arithmetic shift of the signed byte
      const int lo = ((int8_t)(b << 4)) >> 4;
      const __half s = group > 0 ? scale[(size_t)i * ngroups + (2 * j) / group] : scale[i];
      out[(size_t)(2 * j) * n + i] = h_mul(__int2half_rn(hi), s);
      out[(size_t)(2 * j + 1) * n + i] = h_mul(__int2half_rn(lo), s);
    }
  }
}
// axis 0: w [n, m], scale [m] -> out [2n, m]: out[2i, j] = high * s[j], out[2i+1, j] = low * s[j]
__global__ void int4_to_half_axis0_kernel(const int8_t *__restrict__ w, const __half *__restrict__ scale, int n, int m,
                                          __half *__restrict__ out) {
  const size_t total = (size_t)n * m;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t i = idx / m, j = idx - i * m;
    const int8_t b = w[idx];
    const __half s = scale[j];
    out[(2 * i) * m + j] = h_mul(__int2half_rn(b >> 4), s);
    out[(2 * i + 1) * m + j] = h_mul(__int2half_rn(((int8_t)(b << 4)) >> 4), s);
  }
}

// ------------------------------------------------------------------------------------------ norms
// One block per row.  single_row selects GetInPlaceNorm's arithmetic (fp32 mean, no clamp, rsqrt) over
// normInfKernel's (fp16-rounded mean inside the variance, clamp at 0, 1/sqrt).
__global__ void norm_ce_kernel(const __half *__restrict__ x, const __half *__restrict__ gamma, const __half *__restrict__ beta,
                               int dim, float eps, int single_row, __half *__restrict__ out) {
  __shared__ float red[32];
  const __half *xr = x + (size_t)blockIdx.x * dim;
  float s = 0.f, sq = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = __half2float(xr[i]);
    s += v;
    sq += v * v;
  }
  s = block_sum(s, red);
  sq = block_sum(sq, red);
  const float inv_n = 1.0f / (float)dim;
  __half m, r;
  if (single_row) {
    const float mean = s * inv_n;
    const float var = sq * inv_n - mean * mean + eps;
    m = __float2half_rn(mean);
    r = __float2half_rn(1.0f / sqrtf(var));
  } else {
    m = __float2half_rn(s * inv_n);
    const float mf = __half2float(m);
    float var = sq * inv_n - mf * mf;
    var = fmaxf(var, 0.f) + eps;
    r = __float2half_rn(1.0f / sqrtf(var));
  }
  for (int i = threadIdx.x; i < dim; i += blockDim.x)
    out[(size_t)blockIdx.x * dim + i] = h_add(h_mul(h_mul(h_sub(xr[i], m), r), gamma[i]), beta[i]);
}

// norm_ce_kernel with the row kept in registers between the statistics and the normalisation: one pass over memory with 16-byte
// accesses (dim a multiple of 8, below 8192 as the op requires).  Same arithmetic, statistics summed per thread over 8-element
// units instead of single elements.
__global__ void norm_ce_vec_kernel(const __half *__restrict__ x, const __half *__restrict__ gamma, const __half *__restrict__ beta,
                                   int dim, float eps, int single_row, __half *__restrict__ out) {
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * dim;
  const int units = dim / 8;
  constexpr int MAXQ = 4;
  uint4 v[MAXQ];
  float s = 0.f, sq = 0.f;
#pragma unroll
  for (int q = 0; q < MAXQ; ++q) {
    const int u = threadIdx.x + q * blockDim.x;
    if (u < units) {
      v[q] = __ldcg(reinterpret_cast<const uint4 *>(x + base) + u);
      const __half2 *h2 = reinterpret_cast<const __half2 *>(&v[q]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h2[j]);
        s += f.x + f.y;
        sq += f.x * f.x + f.y * f.y;
      }
    }
  }
  s = block_sum(s, red);
  sq = block_sum(sq, red);
  const float inv_n = 1.0f / (float)dim;
  __half m, r;
  if (single_row) {
    const float mean = s * inv_n;
    const float var = sq * inv_n - mean * mean + eps;
    m = __float2half_rn(mean);
    r = __float2half_rn(1.0f / sqrtf(var));
  } else {
    m = __float2half_rn(s * inv_n);
    const float mf = __half2float(m);
    float var = sq * inv_n - mf * mf;
    var = fmaxf(var, 0.f) + eps;
    r = __float2half_rn(1.0f / sqrtf(var));
  }
#pragma unroll
  for (int q = 0; q < MAXQ; ++q) {
    const int u = threadIdx.x + q * blockDim.x;
    if (u < units) {
      const uint4 gv = __ldg(reinterpret_cast<const uint4 *>(gamma) + u), bv = __ldg(reinterpret_cast<const uint4 *>(beta) + u);
      __half *h = reinterpret_cast<__half *>(&v[q]);
      const __half *gh = reinterpret_cast<const __half *>(&gv), *bh = reinterpret_cast<const __half *>(&bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) h[j] = h_add(h_mul(h_mul(h_sub(h[j], m), r), gh[j]), bh[j]);
      reinterpret_cast<uint4 *>(out + base)[u] = v[q];
    }
  }
}

// The row stays in registers between the statistics and the scaling: one pass over memory, 16-byte accesses (dim a multiple of 8,
// at most 8 * 8 * 256).  The scalar two-pass kernel below took 15 us for 16 rows of 4096, all of it load latency.
__global__ void rms_norm_vec_kernel(const __half *__restrict__ x, const __half *__restrict__ residual, const __half *__restrict__ gamma,
                                    int dim, float eps, __half *__restrict__ out, __half *__restrict__ sum_out) {
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * dim;
  const int units = dim / 8;
  constexpr int MAXQ = 8;
  uint4 v[MAXQ];
  float sq = 0.f;
#pragma unroll
  for (int q = 0; q < MAXQ; ++q) {
    const int u = threadIdx.x + q * blockDim.x;
    if (u < units) {
      v[q] = __ldcg(reinterpret_cast<const uint4 *>(x + base) + u);
      if (residual) {
        const uint4 rv = __ldcg(reinterpret_cast<const uint4 *>(residual + base) + u);
        __half *h = reinterpret_cast<__half *>(&v[q]);
        const __half *rh = reinterpret_cast<const __half *>(&rv);
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = h_add(h[j], rh[j]);
        reinterpret_cast<uint4 *>(sum_out + base)[u] = v[q];
      }
      const __half2 *h2 = reinterpret_cast<const __half2 *>(&v[q]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h2[j]);
        sq += f.x * f.x + f.y * f.y;
      }
    }
  }
  sq = block_sum(sq, red);
  const __half r = __float2half_rn(1.0f / sqrtf(sq / (float)dim + eps));
#pragma unroll
  for (int q = 0; q < MAXQ; ++q) {
    const int u = threadIdx.x + q * blockDim.x;
    if (u < units) {
      const uint4 gv = __ldg(reinterpret_cast<const uint4 *>(gamma) + u);
      __half *h = reinterpret_cast<__half *>(&v[q]);
      const __half *gh = reinterpret_cast<const __half *>(&gv);
#pragma unroll
      for (int j = 0; j < 8; ++j) h[j] = h_mul(h_mul(h[j], r), gh[j]);
      reinterpret_cast<uint4 *>(out + base)[u] = v[q];
    }
  }
}

__global__ void rms_norm_kernel(const __half *__restrict__ x, const __half *__restrict__ residual, const __half *__restrict__ gamma,
                                int dim, float eps, __half *__restrict__ out, __half *__restrict__ sum_out) {
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * dim;
  float sq = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    __half v = x[base + i];
    if (residual) {
      v = h_add(v, residual[base + i]);
      sum_out[base + i] = v;
    }
    const float f = __half2float(v);
    sq += f * f;
  }
  sq = block_sum(sq, red);
  const __half r = __float2half_rn(1.0f / sqrtf(sq / (float)dim + eps));
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const __half v = residual ? sum_out[base + i] : x[base + i];
    out[base + i] = h_mul(h_mul(v, r), gamma[i]);
  }
}

// ------------------------------------------------------------------------------------------ SoftmaxV3
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }

// exp in the input dtype, sum in fp32, reciprocal cast to the input dtype, multiply in the input dtype.
template <typename T>
__global__ void softmax_kernel(const T *__restrict__ x, int dim, int stable, T *__restrict__ out) {
  __shared__ float red[32];
  const T *xr = x + (size_t)blockIdx.x * dim;
  T *orow = out + (size_t)blockIdx.x * dim;
  float mx = 0.f;
  if (stable) {
    mx = -FLT_MAX;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) mx = fmaxf(mx, to_f(xr[i]));
    mx = block_max(mx, red);
  }
  float s = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = to_f(xr[i]);
    if (stable) v = to_f(from_f<T>(v - mx));
    const T e = from_f<T>(expf(v));
    orow[i] = e;
    s += to_f(e);
  }
  s = block_sum(s, red);
  const T inv = from_f<T>(1.0f / s);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) orow[i] = from_f<T>(to_f(orow[i]) * to_f(inv));
}

// ------------------------------------------------------------------------------------------ dense KVCache ops
// scratch <- (step == 0 ? 0 : cache)
__global__ void kv_clone_kernel(const int *step_dev, const uint16_t *__restrict__ cache, uint16_t *__restrict__ scratch, size_t total) {
  const bool zero = (*step_dev == 0);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    scratch[i] = zero ? (uint16_t)0 : cache[i];
}
// cache[o, l, i] <- l < step_len ? kv_new[o, l, i] : scratch[o, l - step_len, i]
__global__ void kv_shift_kernel(const uint16_t *__restrict__ kv_new, const uint16_t *__restrict__ scratch, uint16_t *__restrict__ cache,
                                size_t outer, int max_len, int step_len, size_t inner) {
  const size_t total = outer * max_len * inner;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t i = idx % inner;
    const size_t l = (idx / inner) % max_len;
    const size_t o = idx / (inner * max_len);
    cache[idx] = l < (size_t)step_len ? kv_new[(o * step_len + l) * inner + i] : scratch[(o * max_len + (l - step_len)) * inner + i];
  }
}
// KVCachePipeline: zero every cache at step 0; out <- shifted insert into cache[step % max_bps]
__global__ void kv_pipe_shift_kernel(const int *step_dev, const uint16_t *__restrict__ kv_new, const uint16_t *__restrict__ caches,
                                     uint16_t *__restrict__ out, int max_bps, size_t outer, int max_len, int step_len, size_t inner) {
  const int step = *step_dev;
  const size_t per = outer * max_len * inner;
  const uint16_t *sel = caches + (size_t)(step % max_bps) * per;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < per; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t i = idx % inner;
    const size_t l = (idx / inner) % max_len;
    const size_t o = idx / (inner * max_len);
    uint16_t v;
    if (l < (size_t)step_len) v = kv_new[(o * step_len + l) * inner + i];
    else v = step == 0 ? (uint16_t)0 : sel[(o * max_len + (l - step_len)) * inner + i];
    out[idx] = v;
  }
}
__global__ void kv_pipe_commit_kernel(const int *step_dev, const uint16_t *__restrict__ out, uint16_t *__restrict__ caches, int max_bps,
                                      size_t per) {
  const int step = *step_dev;
  const int sel = step % max_bps;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < per * max_bps; idx += (size_t)gridDim.x * blockDim.x) {
    const int c = idx / per;
    const size_t r = idx - (size_t)c * per;
    if (c == sel) caches[idx] = out[r];
    else if (step == 0) caches[idx] = 0;
  }
}

// ---- the same ops with 8-bit storage (`fp8` attribute, kv_cache.cpp:43-75, 100-104, 183-185; kv_cache_pipeline.cpp:386-388, 437-439):
// the update is cast to E4M3 before the insert, the cache lives as bytes and the op returns it cast back to fp16.  One thread per
// (outer, inner) column walks the sequence from its far end, so the shift happens in place and needs no clone.
__device__ __forceinline__ uint8_t kv_to_e4m3(__half v, float inv_scale) {
  return (uint8_t)__nv_cvt_float_to_fp8(__half2float(v) * inv_scale, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ __half kv_from_e4m3(uint8_t b, float scale) {
  return __float2half_rn(__half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3))) * scale);
}
// caches: [n_caches][outer][max_len][inner] bytes.  Cache `sel` (step % n_caches) takes the insert and is decoded into `out`;
// at step 0 every cache starts from zeros.
__global__ void kv_fp8_kernel(const int *step_dev, const __half *__restrict__ kv_new, uint8_t *__restrict__ caches, __half *__restrict__ out,
                              float scale, int n_caches, size_t outer, int max_len, int step_len, size_t inner) {
  const int step = *step_dev;
  const int sel = step % n_caches;
  const size_t cols = outer * inner, per = outer * (size_t)max_len * inner;
  const float inv_scale = 1.0f / scale;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < cols * n_caches; idx += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(idx / cols);
    const size_t col = idx - (size_t)c * cols, o = col / inner, i = col - o * inner;
    uint8_t *cache = caches + (size_t)c * per + o * (size_t)max_len * inner + i;
    if (c != sel) {
      if (step == 0)
        for (int l = 0; l < max_len; ++l) cache[(size_t)l * inner] = 0;
      continue;
    }
    __half *dst = out + o * (size_t)max_len * inner + i;
    for (int l = max_len - 1; l >= step_len; --l) {
      const uint8_t b = step == 0 ? (uint8_t)0 : cache[(size_t)(l - step_len) * inner];
      cache[(size_t)l * inner] = b;
      dst[(size_t)l * inner] = kv_from_e4m3(b, scale);
    }
    for (int l = 0; l < step_len && l < max_len; ++l) {
      const uint8_t b = kv_to_e4m3(kv_new[(o * step_len + l) * inner + i], inv_scale);
      cache[(size_t)l * inner] = b;
      dst[(size_t)l * inner] = kv_from_e4m3(b, scale);
    }
  }
}

// ------------------------------------------------------------------------------------------ top-k
// One block per row, k <= 32: k rounds of arg-max with the already chosen indices masked out.  The key orders
// by value descending, then by index ascending, so ties resolve to the lowest index.
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// zero_sub: exact-zero inputs are read as -10000 (the TP LM head's vocabulary-padding rule); id_offset is added to
// the reported indices (rank * vocab_per_rank).
template <typename T>
__global__ void topk_kernel(const T *__restrict__ x, int dim, int k, T *__restrict__ vals, int *__restrict__ ids, int zero_sub = 0,
                            int id_offset = 0) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int chosen[32];
  const T *xr = x + (size_t)blockIdx.x * dim;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int bi = INT_MAX;
    if (r == 0) {
      // first round (the only one of the greedy head): nothing is masked yet, so eight loads of a thread can be in flight together
      // (one dependent 2-byte load per trip made this kernel 29 us for 50257 logits)
      constexpr int U = 8;
      for (int i0 = threadIdx.x; i0 < dim; i0 += U * blockDim.x) {
        float v[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
          const int i = i0 + j * blockDim.x;
          v[j] = i < dim ? to_f(xr[i]) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
          const int i = i0 + j * blockDim.x;
          if (i < dim) {
            float w = v[j];
            if (zero_sub && w == 0.f) w = -10000.f;
            if (better(w, i, bv, bi) || bi == INT_MAX) { bv = w; bi = i; }
          }
        }
      }
    } else {
      for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        bool skip = false;
        for (int c = 0; c < r; ++c) skip |= (chosen[c] == i);
        if (skip) continue;
        float v = to_f(xr[i]);
        if (zero_sub && v == 0.f) v = -10000.f;
        if (better(v, i, bv, bi) || bi == INT_MAX) { bv = v; bi = i; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != INT_MAX && (bi == INT_MAX || better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float fv = sv[0];
      int fi = si[0];
      for (int w = 1; w < nw; ++w)
        if (si[w] != INT_MAX && (fi == INT_MAX || better(sv[w], si[w], fv, fi))) { fv = sv[w]; fi = si[w]; }
      chosen[r] = fi;
      vals[(size_t)blockIdx.x * k + r] = from_f<T>(fv);
      ids[(size_t)blockIdx.x * k + r] = fi + id_offset;
    }
    __syncthreads();
  }
}

// TP LM-head merge: gathered (value, id) pairs [tp, rows]; the first maximum over ranks wins (aiOnnx.argmax).
__global__ void tp_pick_kernel(const __half *__restrict__ vals, const int *__restrict__ ids, int tp, int rows, int *__restrict__ out) {
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
    float bv = __half2float(vals[r]);
    int bi = ids[r];
    for (int t = 1; t < tp; ++t) {
      const float v = __half2float(vals[(size_t)t * rows + r]);
      if (v > bv) { bv = v; bi = ids[(size_t)t * rows + r]; }
    }
    out[r] = bi;
  }
}

// ------------------------------------------------------------------------------------------ BeamSearch
// After the per-beam top-k (val/idx [b, beam, beam]) one block per batch row finishes the step.
template <typename T>
__global__ void beam_finish_kernel(const T *__restrict__ val, const int *__restrict__ idx, const int *__restrict__ hyp_in,
                                   int *__restrict__ hyp_out, T *__restrict__ prob, const int *step_dev, int beam, int max_len,
                                   int *__restrict__ next_id, int *__restrict__ gbest, int *__restrict__ parent) {
  __shared__ float cand[32 * 32];
  __shared__ int gsel[32];
  const int b = blockIdx.x, step = *step_dev, bb = beam * beam;
  const T *v = val + (size_t)b * bb;
  const int *id = idx + (size_t)b * bb;
  if (step == 0) {
    for (int k = threadIdx.x; k < beam; k += blockDim.x) {
      next_id[b * beam + k] = id[k];
      gbest[b * beam + k] = id[k];
      prob[b * beam + k] = v[k];
      if (parent) parent[b * beam + k] = b * beam;  // every slot continues the (identical) first hypothesis
    }
    for (int i = threadIdx.x; i < max_len * beam; i += blockDim.x) {
      const int t = i / beam, k = i - t * beam;
      hyp_out[(size_t)b * max_len * beam + i] = (t == 0) ? id[k] : hyp_in[(size_t)b * max_len * beam + i];
    }
    return;
  }
  // cand[i*beam + j] = T(val[i][j] + prob[i])
  for (int i = threadIdx.x; i < bb; i += blockDim.x) cand[i] = to_f(from_f<T>(to_f(v[i]) + to_f(prob[b * beam + i / beam])));
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int r = 0; r < beam; ++r) {
      float bv = -INFINITY;
      int bi = -1;
      for (int i = 0; i < bb; ++i) {
        bool used = false;
        for (int c = 0; c < r; ++c) used |= (gsel[c] == i);
        if (!used && (bi < 0 || cand[i] > bv)) { bv = cand[i]; bi = i; }
      }
      gsel[r] = bi;
    }
  }
  __syncthreads();
  for (int k = threadIdx.x; k < beam; k += blockDim.x) {
    const int gsl = gsel[k];
    next_id[b * beam + k] = id[gsl];
    gbest[b * beam + k] = gsl;
    if (parent) parent[b * beam + k] = b * beam + gsl / beam;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < max_len * beam; i += blockDim.x) {
    const int t = i / beam, k = i - t * beam;
    const int gsl = gsel[k];
    hyp_out[(size_t)b * max_len * beam + i] = (t == step) ? id[gsl] : hyp_in[((size_t)b * max_len + t) * beam + gsl / beam];
  }
  __syncthreads();
  for (int k = threadIdx.x; k < beam; k += blockDim.x) prob[b * beam + k] = from_f<T>(cand[gsel[k]]);
}
__global__ void copy_i32_kernel(const int *__restrict__ src, int *__restrict__ dst, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
}

// ------------------------------------------------------------------------------------------ FP8
__global__ void cast_fp8_kernel(const __half *__restrict__ x, float inv_scale, size_t n, uint8_t *__restrict__ out) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = __nv_cvt_float_to_fp8(__half2float(x[i]) * inv_scale, __NV_SATFINITE, __NV_E4M3);
}

// Reference-layout FP8 matmul for arbitrary m: out[i, j] = fp16(sum_k a[i,k] b[j,k] * scale).  32x32 output tile per
// block, k staged through shared memory in slices of 64.  (The decode path uses the streaming linear kernel; this
// entry keeps the op surface complete.)
__global__ void fp8_matmul_kernel(const uint8_t *__restrict__ a, const uint8_t *__restrict__ b, float scale, int m, int n, int k,
                                  __half *__restrict__ out) {
  __shared__ float as[32][65], bs[32][65];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int i0 = blockIdx.y * 32, j0 = blockIdx.x * 32;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < k; k0 += 64) {
    for (int e = threadIdx.x; e < 32 * 64; e += 256) {
      const int r = e >> 6, c = e & 63;
      const int kk = k0 + c;
      float av = 0.f, bv = 0.f;
      if (kk < k) {
        if (i0 + r < m) av = __half2float(__half(__nv_cvt_fp8_to_halfraw(a[(size_t)(i0 + r) * k + kk], __NV_E4M3)));
        if (j0 + r < n) bv = __half2float(__half(__nv_cvt_fp8_to_halfraw(b[(size_t)(j0 + r) * k + kk], __NV_E4M3)));
      }
      as[r][c] = av;
      bs[r][c] = bv;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = ty + 8 * q;
      float s = acc[q];
      for (int c = 0; c < 64; ++c) s += as[r][c] * bs[tx][c];
      acc[q] = s;
    }
    __syncthreads();
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int i = i0 + ty + 8 * q, j = j0 + tx;
    if (i < m && j < n) out[(size_t)i * n + j] = __float2half_rn(acc[q] * scale);
  }
}

// ------------------------------------------------------------------------------------------ RWKV WKV
__global__ void wkv_kernel(const __half *__restrict__ k, const __half *__restrict__ v, const float *__restrict__ tf,
                           const float *__restrict__ td, float *__restrict__ num, float *__restrict__ den, float *__restrict__ mx,
                           int b, int c, __half *__restrict__ out) {
  const size_t total = (size_t)b * c;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int ch = i % c;
    const float kk = __half2float(k[i]), vv = __half2float(v[i]);
    const float n0 = num[i], d0 = den[i], m0 = mx[i];
    const float ww = kk + tf[ch];
    const float p = fmaxf(m0, ww);
    float e1 = expf(m0 - p), e2 = expf(ww - p);
    out[i] = __float2half_rn((e1 * n0 + e2 * vv) / (e1 * d0 + e2));
    const float ww2 = m0 - expf(td[ch]);
    const float p2 = fmaxf(ww2, kk);
    e1 = expf(ww2 - p2);
    e2 = expf(kk - p2);
    num[i] = e1 * n0 + e2 * vv;
    den[i] = e1 * d0 + e2;
    mx[i] = p2;
  }
}

// RWKV token-shift gates (poptransformer/models/rwkv/attention.py:59-64, ffn.py:40-45): out_x = fp16(fp16(h * w_x) + fp16(fp16(1 - w_x) * s)) for up to
// three mixing vectors, then the state takes the current hidden vector.
__global__ void rwkv_mix_kernel(const __half *__restrict__ hidden, __half *__restrict__ state, const __half *__restrict__ wa,
                                const __half *__restrict__ wb, const __half *__restrict__ wc, __half *__restrict__ oa, __half *__restrict__ ob,
                                __half *__restrict__ oc, int rows, int dim) {
  const size_t total = (size_t)rows * dim;
  const __half one = __float2half_rn(1.0f);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int ch = i % dim;
    const __half h = hidden[i], s = state[i];
    oa[i] = h_add(h_mul(h, wa[ch]), h_mul(h_sub(one, wa[ch]), s));
    if (ob) ob[i] = h_add(h_mul(h, wb[ch]), h_mul(h_sub(one, wb[ch]), s));
    if (oc) oc[i] = h_add(h_mul(h, wc[ch]), h_mul(h_sub(one, wc[ch]), s));
    state[i] = h;
  }
}
// RWKV element-wise steps: 0: out = fp16(sigmoid(a)) * b   (receptance gate, attention.py:76,103; ffn.py:57-58)
//                          1: out = relu(a)^2              (ffn.py:53-54)
//                          2: out = a / 2                  (rescale_every, rwkv/model.py:115-116)
__global__ void rwkv_act_kernel(int mode, const __half *__restrict__ a, const __half *__restrict__ b, __half *__restrict__ out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const __half x = a[i];
    if (mode == 0) {
      const __half sg = __float2half_rn(1.0f / (1.0f + expf(-__half2float(x))));
      out[i] = h_mul(sg, b[i]);
    } else if (mode == 1) {
      const __half r = __hgt(x, __float2half_rn(0.f)) ? x : __float2half_rn(0.f);
      out[i] = h_mul(r, r);
    } else {
      out[i] = h_mul(x, __float2half_rn(0.5f));
    }
  }
}

// ------------------------------------------------------------------------------------------ loop carry
__global__ void embedding_kernel(const uint4 *__restrict__ table, const int *__restrict__ ids, int ids_stride, const int *step_dev,
                                 int dim8, int vocab, uint4 *__restrict__ out) {
  const int b = blockIdx.x;
  const int step = step_dev ? min(max(*step_dev, 0), ids_stride - 1) : 0;  // a step past the container reads its last column
  int id = ids[(size_t)b * ids_stride + step];
  id = min(max(id, 0), vocab - 1);
  for (int i = threadIdx.x; i < dim8; i += blockDim.x) out[(size_t)b * dim8 + i] = table[(size_t)id * dim8 + i];
}
__global__ void step_containers_kernel(int *ids, int batch, int max_len, int *step_dev, const int *next_ids, int pad_id, int eos_id,
                                       int *stop_mask, int *done_flag) {
  __shared__ int s_running;
  if (done_flag) {
    if (*done_flag) return;   // uniform: every thread reads the same word
    if (threadIdx.x == 0) s_running = 0;
    __syncthreads();
    // keep_going = sum(stop_mask) < batch on the mask BEFORE this iteration's update (models/base_model.py:348-352)
    for (int b = threadIdx.x; b < batch; b += blockDim.x)
      if (!stop_mask[b]) atomicAdd(&s_running, 1);
    __syncthreads();
  }
  const int nxt = *step_dev + 1;
  for (int b = threadIdx.x; b < batch; b += blockDim.x) {
    if (nxt < max_len) {
      const int cur = ids[(size_t)b * max_len + nxt];
      const int upd = (cur == pad_id) ? next_ids[b] : cur;
      ids[(size_t)b * max_len + nxt] = upd;
      if (stop_mask) stop_mask[b] |= (upd == eos_id) ? 1 : 0;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *step_dev = nxt;
    if (done_flag && s_running == 0) *done_flag = 1;
  }
}
__global__ void add_f16_kernel(const __half *__restrict__ a, const __half *__restrict__ b, size_t n, __half *__restrict__ out) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = h_add(a[i], b[i]);
}

// SwiGLU on the output of a fused gate|up linear whose rows are [gate features | up features]: out = fp16(up * swish(gate)).
__global__ void swiglu_kernel(const __half *__restrict__ gu, int rows, int f, __half *__restrict__ out, int out_ld) {
  const size_t total = (size_t)rows * f;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t b = i / f, j = i - b * f;
    out[b * out_ld + j] = h_mul(gu[b * 2 * f + f + j], swish_h(gu[b * 2 * f + j]));
  }
}

// RMSNorm (reference fp16 roundings) followed by the E4M3 cast of an FP8 linear's input: one block per row, the row read once
// into registers (dim <= 8 * 8 * 256), bytes out.
__global__ void rms_norm_fp8_kernel(const __half *__restrict__ x, const __half *__restrict__ gamma, int dim, float eps, float inv_scale,
                                    uint8_t *__restrict__ out) {
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * dim;
  const int units = dim / 8;
  constexpr int MAXQ = 8;
  uint4 v[MAXQ];
  float sq = 0.f;
#pragma unroll
  for (int q = 0; q < MAXQ; ++q) {
    const int u = threadIdx.x + q * blockDim.x;
    if (u < units) {
      v[q] = __ldcg(reinterpret_cast<const uint4 *>(x + base) + u);
      const __half2 *h = reinterpret_cast<const __half2 *>(&v[q]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        sq += f.x * f.x + f.y * f.y;
      }
    }
  }
  sq = block_sum(sq, red);
  const __half r = __float2half_rn(1.0f / sqrtf(sq / (float)dim + eps));
#pragma unroll
  for (int q = 0; q < MAXQ; ++q) {
    const int u = threadIdx.x + q * blockDim.x;
    if (u < units) {
      const uint4 gv = __ldg(reinterpret_cast<const uint4 *>(gamma) + u);
      const __half *h = reinterpret_cast<const __half *>(&v[q]), *gh = reinterpret_cast<const __half *>(&gv);
      uint32_t b[2] = {0u, 0u};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const __half e = h_mul(h_mul(h[j], r), gh[j]);
        b[j >> 2] |= (uint32_t)__nv_cvt_float_to_fp8(__half2float(e) * inv_scale, __NV_SATFINITE, __NV_E4M3) << (8 * (j & 3));
      }
      *reinterpret_cast<uint2 *>(out + base + (size_t)u * 8) = make_uint2(b[0], b[1]);
    }
  }
}
// SwiGLU of [gate features | up features] rows, cast to E4M3 for the FP8 linear that follows.
__global__ void swiglu_fp8_kernel(const __half *__restrict__ gu, int rows, int f, float inv_scale, uint8_t *__restrict__ out, int out_ld) {
  const size_t total = (size_t)rows * f;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t b = i / f, j = i - b * f;
    const __half y = h_mul(gu[b * 2 * f + f + j], swish_h(gu[b * 2 * f + j]));
    out[b * out_ld + j] = (uint8_t)__nv_cvt_float_to_fp8(__half2float(y) * inv_scale, __NV_SATFINITE, __NV_E4M3);
  }
}

static inline int grid_for(size_t n, int block = 256) {
  size_t g = (n + block - 1) / block;
  const size_t cap = (size_t)sm_count() * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace pt

using namespace pt;

extern "C" int pt_int4_to_half(const void *w, const void *scale, int n, int m, int axis, int group, void *out, void *stream) {
  PT_REQUIRE(w && scale && out, "pt_int4_to_half: null pointer argument");
  PT_REQUIRE(n > 0 && m > 0, "pt_int4_to_half: bad shape [%d, %d]", n, m);
  PT_REQUIRE(axis == 0 || axis == 1, "pt_int4_to_half: axis must be 0 or 1, got %d", axis);
  cudaStream_t st = as_stream(stream);
  if (axis == 1) {
    PT_REQUIRE(group == 0 || (group % 2 == 0 && (2 * m) % group == 0), "pt_int4_to_half: group=%d must be even and divide %d", group, 2 * m);
    dim3 grid(ceil_div(m, 32), ceil_div(n, 32)), block(32, 8);
    int4_to_half_axis1_kernel<<<grid, block, 0, st>>>((const int8_t *)w, (const __half *)scale, n, m, group, (__half *)out);
  } else {
    PT_REQUIRE(group == 0, "pt_int4_to_half: group scales are only defined for axis 1");
    int4_to_half_axis0_kernel<<<grid_for((size_t)n * m), 256, 0, st>>>((const int8_t *)w, (const __half *)scale, n, m, (__half *)out);
  }
  PT_LAUNCH_CHECK("pt_int4_to_half");
  return PT_OK;
}

extern "C" int pt_norm_ce(const void *x, const void *gamma, const void *beta, int rows, int dim, float eps, void *out, void *stream) {
  PT_REQUIRE(x && gamma && beta && out, "pt_norm_ce: null pointer argument");
  PT_REQUIRE(rows > 0 && dim > 0, "pt_norm_ce: bad shape [%d, %d]", rows, dim);
  PT_REQUIRE((dim & 3) == 0, "our normCEOp require 4x a last dim, and current is: %d", dim);
  PT_REQUIRE(dim < 8192, "normalize_ce, last_dim_size should be <= 8192, and current is: %d", dim);
  if (dim % 8 == 0 && (((uintptr_t)x | (uintptr_t)out | (uintptr_t)gamma | (uintptr_t)beta) & 15) == 0)
    norm_ce_vec_kernel<<<rows, 256, 0, as_stream(stream)>>>((const __half *)x, (const __half *)gamma, (const __half *)beta, dim, eps,
                                                           rows == 1 ? 1 : 0, (__half *)out);
  else
    norm_ce_kernel<<<rows, 256, 0, as_stream(stream)>>>((const __half *)x, (const __half *)gamma, (const __half *)beta, dim, eps,
                                                       rows == 1 ? 1 : 0, (__half *)out);
  PT_LAUNCH_CHECK("pt_norm_ce");
  return PT_OK;
}

extern "C" int pt_rms_norm(const void *x, const void *residual, const void *gamma, int rows, int dim, float eps, void *out, void *sum_out,
                           void *stream) {
  PT_REQUIRE(x && gamma && out, "pt_rms_norm: null pointer argument");
  PT_REQUIRE(rows > 0 && dim > 0, "pt_rms_norm: bad shape [%d, %d]", rows, dim);
  PT_REQUIRE(!residual || sum_out, "pt_rms_norm: residual given without sum_out");
  const bool vec = dim % 8 == 0 && dim <= 8 * 8 * 256 && (((uintptr_t)x | (uintptr_t)out | (uintptr_t)gamma | (uintptr_t)residual | (uintptr_t)sum_out) & 15) == 0;
  if (vec)
    rms_norm_vec_kernel<<<rows, 256, 0, as_stream(stream)>>>((const __half *)x, (const __half *)residual, (const __half *)gamma, dim, eps,
                                                            (__half *)out, (__half *)sum_out);
  else
    rms_norm_kernel<<<rows, 256, 0, as_stream(stream)>>>((const __half *)x, (const __half *)residual, (const __half *)gamma, dim, eps,
                                                        (__half *)out, (__half *)sum_out);
  PT_LAUNCH_CHECK("pt_rms_norm");
  return PT_OK;
}

extern "C" int pt_softmax(const void *x, int rows, int dim, int stable_mode, int dtype, void *out, void *stream) {
  PT_REQUIRE(x && out, "pt_softmax: null pointer argument");
  PT_REQUIRE(rows > 0 && dim > 0, "pt_softmax: bad shape [%d, %d]", rows, dim);
  PT_REQUIRE(dtype == 0 || dtype == 1, "pt_softmax: dtype must be 0 (fp16) or 1 (fp32)");
  if (dtype == 0) softmax_kernel<__half><<<rows, 256, 0, as_stream(stream)>>>((const __half *)x, dim, stable_mode, (__half *)out);
  else softmax_kernel<float><<<rows, 256, 0, as_stream(stream)>>>((const float *)x, dim, stable_mode, (float *)out);
  PT_LAUNCH_CHECK("pt_softmax");
  return PT_OK;
}

extern "C" int pt_kv_cache(const int32_t *step_dev, const void *kv_new, void *cache, void *scratch, int64_t outer, int max_len,
                           int step_len, int64_t inner, void *stream) {
  PT_REQUIRE(step_dev && kv_new && cache && scratch, "pt_kv_cache: null pointer argument");
  PT_REQUIRE(outer > 0 && inner > 0 && max_len > 0 && step_len > 0 && step_len <= max_len, "pt_kv_cache: bad shape outer=%lld max_len=%d step_len=%d inner=%lld",
             (long long)outer, max_len, step_len, (long long)inner);
  const size_t total = (size_t)outer * max_len * inner;
  cudaStream_t st = as_stream(stream);
  kv_clone_kernel<<<grid_for(total), 256, 0, st>>>(step_dev, (const uint16_t *)cache, (uint16_t *)scratch, total);
  PT_LAUNCH_CHECK("pt_kv_cache(clone)");
  kv_shift_kernel<<<grid_for(total), 256, 0, st>>>((const uint16_t *)kv_new, (const uint16_t *)scratch, (uint16_t *)cache, (size_t)outer,
                                                  max_len, step_len, (size_t)inner);
  PT_LAUNCH_CHECK("pt_kv_cache(shift)");
  return PT_OK;
}

extern "C" int pt_kv_cache_pipeline(const int32_t *step_dev, const void *kv_new, void *caches, void *out, int max_bps, int64_t outer,
                                    int max_len, int step_len, int64_t inner, void *stream) {
  PT_REQUIRE(step_dev && kv_new && caches && out, "pt_kv_cache_pipeline: null pointer argument");
  PT_REQUIRE(max_bps > 0 && outer > 0 && inner > 0 && max_len > 0 && step_len > 0 && step_len <= max_len, "pt_kv_cache_pipeline: bad shape");
  const size_t per = (size_t)outer * max_len * inner;
  cudaStream_t st = as_stream(stream);
  kv_pipe_shift_kernel<<<grid_for(per), 256, 0, st>>>(step_dev, (const uint16_t *)kv_new, (const uint16_t *)caches, (uint16_t *)out, max_bps,
                                                     (size_t)outer, max_len, step_len, (size_t)inner);
  PT_LAUNCH_CHECK("pt_kv_cache_pipeline(shift)");
  kv_pipe_commit_kernel<<<grid_for(per * max_bps), 256, 0, st>>>(step_dev, (const uint16_t *)out, (uint16_t *)caches, max_bps, per);
  PT_LAUNCH_CHECK("pt_kv_cache_pipeline(commit)");
  return PT_OK;
}

extern "C" int pt_kv_cache_fp8(const int32_t *step_dev, const void *kv_new, void *cache, void *out, float scale, int64_t outer, int max_len,
                               int step_len, int64_t inner, void *stream) {
  PT_REQUIRE(step_dev && kv_new && cache && out, "pt_kv_cache_fp8: null pointer argument");
  PT_REQUIRE(outer > 0 && inner > 0 && max_len > 0 && step_len > 0 && step_len <= max_len, "pt_kv_cache_fp8: bad shape");
  PT_REQUIRE(scale > 0.f, "pt_kv_cache_fp8: scale must be > 0");
  kv_fp8_kernel<<<grid_for((size_t)(outer * inner)), 256, 0, as_stream(stream)>>>(step_dev, (const __half *)kv_new, (uint8_t *)cache, (__half *)out, scale,
                                                                                    1, (size_t)outer, max_len, step_len, (size_t)inner);
  PT_LAUNCH_CHECK("pt_kv_cache_fp8");
  return PT_OK;
}

extern "C" int pt_kv_cache_pipeline_fp8(const int32_t *step_dev, const void *kv_new, void *caches, void *out, float scale, int max_bps,
                                        int64_t outer, int max_len, int step_len, int64_t inner, void *stream) {
  PT_REQUIRE(step_dev && kv_new && caches && out, "pt_kv_cache_pipeline_fp8: null pointer argument");
  PT_REQUIRE(max_bps > 0 && outer > 0 && inner > 0 && max_len > 0 && step_len > 0 && step_len <= max_len, "pt_kv_cache_pipeline_fp8: bad shape");
  PT_REQUIRE(scale > 0.f, "pt_kv_cache_pipeline_fp8: scale must be > 0");
  kv_fp8_kernel<<<grid_for((size_t)(outer * inner * max_bps)), 256, 0, as_stream(stream)>>>(
      step_dev, (const __half *)kv_new, (uint8_t *)caches, (__half *)out, scale, max_bps, (size_t)outer, max_len, step_len, (size_t)inner);
  PT_LAUNCH_CHECK("pt_kv_cache_pipeline_fp8");
  return PT_OK;
}

extern "C" int pt_topk(const void *x, int rows, int dim, int k, int dtype, void *vals, int32_t *ids, void *stream) {
  PT_REQUIRE(x && vals && ids, "pt_topk: null pointer argument");
  PT_REQUIRE(rows > 0 && dim > 0 && k >= 1 && k <= 32 && k <= dim, "pt_topk: bad shape rows=%d dim=%d k=%d (k <= 32)", rows, dim, k);
  PT_REQUIRE(dtype == 0 || dtype == 1, "pt_topk: dtype must be 0 (fp16) or 1 (fp32)");
  const int threads = dim >= 8192 ? 1024 : 256;
  if (dtype == 0) topk_kernel<__half><<<rows, threads, 0, as_stream(stream)>>>((const __half *)x, dim, k, (__half *)vals, ids);
  else topk_kernel<float><<<rows, threads, 0, as_stream(stream)>>>((const float *)x, dim, k, (float *)vals, ids);
  PT_LAUNCH_CHECK("pt_topk");
  return PT_OK;
}

extern "C" int pt_lm_head_local_topk(const void *logits, int rows, int dim, int id_offset, void *vals, int32_t *ids, void *stream) {
  PT_REQUIRE(logits && vals && ids, "pt_lm_head_local_topk: null pointer argument");
  PT_REQUIRE(rows > 0 && dim > 0, "pt_lm_head_local_topk: bad shape rows=%d dim=%d", rows, dim);
  const int threads = dim >= 8192 ? 1024 : 256;
  topk_kernel<__half><<<rows, threads, 0, as_stream(stream)>>>((const __half *)logits, dim, 1, (__half *)vals, ids, 1, id_offset);
  PT_LAUNCH_CHECK("pt_lm_head_local_topk");
  return PT_OK;
}

extern "C" int pt_lm_head_tp_pick(const void *vals, const int32_t *ids, int tp, int rows, int32_t *next_ids, void *stream) {
  PT_REQUIRE(vals && ids && next_ids && tp > 0 && rows > 0, "pt_lm_head_tp_pick: bad arguments");
  tp_pick_kernel<<<1, 128, 0, as_stream(stream)>>>((const __half *)vals, ids, tp, rows, next_ids);
  PT_LAUNCH_CHECK("pt_lm_head_tp_pick");
  return PT_OK;
}

extern "C" size_t pt_beam_search_workspace_bytes(int b, int beam, int max_len) {
  // hypothesis snapshot + per-beam top-k ids + per-beam top-k values (fp32-sized slots)
  return ((size_t)b * max_len * beam + 2 * (size_t)b * beam * beam) * sizeof(int32_t);
}

extern "C" int pt_beam_search(const void *logits, int32_t *hyp, void *prob, const int32_t *step_dev, int b, int beam, int vocab, int max_len,
                              int dtype, int32_t *next_id, int32_t *global_best_id, int32_t *parent, void *workspace,
                              size_t workspace_bytes, void *stream) {
  PT_REQUIRE(logits && hyp && prob && step_dev && next_id && global_best_id && workspace, "pt_beam_search: null pointer argument");
  PT_REQUIRE(b > 0 && beam >= 1 && beam <= 32 && beam <= vocab && max_len > 0, "pt_beam_search: bad shape b=%d beam=%d vocab=%d", b, beam, vocab);
  PT_REQUIRE(dtype == 0 || dtype == 1, "pt_beam_search: dtype must be 0 (fp16) or 1 (fp32)");
  const size_t need = pt_beam_search_workspace_bytes(b, beam, max_len);
  PT_REQUIRE(workspace_bytes >= need, "pt_beam_search: workspace needs %zu bytes, got %zu", need, workspace_bytes);
  int *hyp_tmp = (int *)workspace;
  int *tk_ids = hyp_tmp + (size_t)b * max_len * beam;
  void *tk_vals = tk_ids + (size_t)b * beam * beam;
  cudaStream_t st = as_stream(stream);
  const int threads = vocab >= 8192 ? 1024 : 256;
  if (dtype == 0) topk_kernel<__half><<<b * beam, threads, 0, st>>>((const __half *)logits, vocab, beam, (__half *)tk_vals, tk_ids);
  else topk_kernel<float><<<b * beam, threads, 0, st>>>((const float *)logits, vocab, beam, (float *)tk_vals, tk_ids);
  PT_LAUNCH_CHECK("pt_beam_search(topk)");
  const size_t nh = (size_t)b * max_len * beam;
  copy_i32_kernel<<<grid_for(nh), 256, 0, st>>>(hyp, hyp_tmp, nh);
  PT_LAUNCH_CHECK("pt_beam_search(copy)");
  if (dtype == 0)
    beam_finish_kernel<__half><<<b, 128, 0, st>>>((const __half *)tk_vals, tk_ids, hyp_tmp, hyp, (__half *)prob, step_dev, beam, max_len, next_id,
                                                 global_best_id, parent);
  else
    beam_finish_kernel<float><<<b, 128, 0, st>>>((const float *)tk_vals, tk_ids, hyp_tmp, hyp, (float *)prob, step_dev, beam, max_len, next_id,
                                                global_best_id, parent);
  PT_LAUNCH_CHECK("pt_beam_search(finish)");
  return PT_OK;
}

extern "C" int pt_cast_fp8(const void *x, float scale, int64_t n, void *out, void *stream) {
  PT_REQUIRE(x && out && n > 0, "pt_cast_fp8: bad arguments");
  PT_REQUIRE(scale > 0.f, "pt_cast_fp8: scale must be > 0");
  cast_fp8_kernel<<<grid_for((size_t)n), 256, 0, as_stream(stream)>>>((const __half *)x, 1.0f / scale, (size_t)n, (uint8_t *)out);
  PT_LAUNCH_CHECK("pt_cast_fp8");
  return PT_OK;
}

extern "C" int pt_fp8_matmul(const void *a, const void *b, float scale_a, float scale_b, int m, int n, int k, void *out, void *stream) {
  PT_REQUIRE(a && b && out, "pt_fp8_matmul: null pointer argument");
  PT_REQUIRE(m > 0 && n > 0 && k > 0, "pt_fp8_matmul: bad shape m=%d n=%d k=%d", m, n, k);
  if (k % 128 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)b & 15) == 0) {
    // the tcgen05 GEMM (one k-slice: this entry point has no workspace argument)
    pt_gemm_args g{};
    g.wfmt = PT_W_FP8; g.m = m; g.n_out = n; g.k_in = k; g.epilogue = PT_EPI_STORE; g.ksplit = 1;
    g.x = a; g.w = b; g.x_scale = scale_a; g.w_scale = scale_b; g.out = out;
    return pt_gemm(&g, stream);
  }
  // shapes the tensor-core kernel does not take (k not a multiple of 128): scalar tiles
  dim3 grid(ceil_div(n, 32), ceil_div(m, 32));
  fp8_matmul_kernel<<<grid, 256, 0, as_stream(stream)>>>((const uint8_t *)a, (const uint8_t *)b, scale_a * scale_b, m, n, k, (__half *)out);
  PT_LAUNCH_CHECK("pt_fp8_matmul");
  return PT_OK;
}

extern "C" int pt_wkv(const void *k, const void *v, const float *time_first, const float *time_decay, float *num, float *den,
                      float *max_state, int b, int c, void *out, void *stream) {
  PT_REQUIRE(k && v && time_first && time_decay && num && den && max_state && out, "pt_wkv: null pointer argument");
  PT_REQUIRE(b > 0 && c > 0, "pt_wkv: bad shape [%d, %d]", b, c);
  wkv_kernel<<<grid_for((size_t)b * c), 256, 0, as_stream(stream)>>>((const __half *)k, (const __half *)v, time_first, time_decay, num, den,
                                                                     max_state, b, c, (__half *)out);
  PT_LAUNCH_CHECK("pt_wkv");
  return PT_OK;
}

extern "C" int pt_rwkv_mix(const void *hidden, void *state, const void *mix_a, const void *mix_b, const void *mix_c, void *out_a, void *out_b,
                           void *out_c, int rows, int dim, void *stream) {
  PT_REQUIRE(hidden && state && mix_a && out_a && (!out_b || mix_b) && (!out_c || mix_c), "pt_rwkv_mix: null pointer argument");
  PT_REQUIRE(rows > 0 && dim > 0, "pt_rwkv_mix: bad shape [%d, %d]", rows, dim);
  rwkv_mix_kernel<<<grid_for((size_t)rows * dim), 256, 0, as_stream(stream)>>>((const __half *)hidden, (__half *)state, (const __half *)mix_a,
                                                                              (const __half *)mix_b, (const __half *)mix_c, (__half *)out_a,
                                                                              (__half *)out_b, (__half *)out_c, rows, dim);
  PT_LAUNCH_CHECK("pt_rwkv_mix");
  return PT_OK;
}

extern "C" int pt_rwkv_act(int mode, const void *a, const void *b, void *out, int64_t n, void *stream) {
  PT_REQUIRE(a && out && n > 0 && mode >= 0 && mode <= 2 && (mode != 0 || b), "pt_rwkv_act: bad arguments (mode %d)", mode);
  rwkv_act_kernel<<<grid_for((size_t)n), 256, 0, as_stream(stream)>>>(mode, (const __half *)a, (const __half *)b, (__half *)out, (size_t)n);
  PT_LAUNCH_CHECK("pt_rwkv_act");
  return PT_OK;
}

extern "C" int pt_embedding(const void *table, const int32_t *ids, int ids_stride, const int32_t *step_dev, int batch, int dim, int vocab,
                            void *out, void *stream) {
  PT_REQUIRE(table && ids && out, "pt_embedding: null pointer argument");
  PT_REQUIRE(batch > 0 && dim > 0 && dim % 8 == 0 && vocab > 0, "pt_embedding: bad shape batch=%d dim=%d (dim %% 8 == 0)", batch, dim);
  embedding_kernel<<<batch, 128, 0, as_stream(stream)>>>((const uint4 *)table, ids, ids_stride, step_dev, dim / 8, vocab, (uint4 *)out);
  PT_LAUNCH_CHECK("pt_embedding");
  return PT_OK;
}

extern "C" int pt_step_containers(int32_t *ids, int batch, int max_len, int32_t *step_dev, const int32_t *next_ids, int pad_id, int eos_id,
                                  int32_t *stop_mask, void *stream) {
  PT_REQUIRE(ids && step_dev && next_ids, "pt_step_containers: null pointer argument");
  PT_REQUIRE(batch > 0 && max_len > 0, "pt_step_containers: bad shape");
  step_containers_kernel<<<1, 128, 0, as_stream(stream)>>>(ids, batch, max_len, step_dev, next_ids, pad_id, eos_id, stop_mask, nullptr);
  PT_LAUNCH_CHECK("pt_step_containers");
  return PT_OK;
}

extern "C" int pt_step_containers_early_stop(int32_t *ids, int batch, int max_len, int32_t *step_dev, const int32_t *next_ids, int pad_id,
                                             int eos_id, int32_t *stop_mask, int32_t *done_flag, void *stream) {
  PT_REQUIRE(ids && step_dev && next_ids && stop_mask && done_flag, "pt_step_containers_early_stop: null pointer argument");
  PT_REQUIRE(batch > 0 && max_len > 0, "pt_step_containers_early_stop: bad shape");
  step_containers_kernel<<<1, 128, 0, as_stream(stream)>>>(ids, batch, max_len, step_dev, next_ids, pad_id, eos_id, stop_mask, done_flag);
  PT_LAUNCH_CHECK("pt_step_containers_early_stop");
  return PT_OK;
}

extern "C" int pt_swiglu(const void *gate_up, int rows, int f, void *out, int out_ld, void *stream) {
  PT_REQUIRE(gate_up && out && rows > 0 && f > 0, "pt_swiglu: bad arguments");
  swiglu_kernel<<<grid_for((size_t)rows * f), 256, 0, as_stream(stream)>>>((const __half *)gate_up, rows, f, (__half *)out, out_ld > 0 ? out_ld : f);
  PT_LAUNCH_CHECK("pt_swiglu");
  return PT_OK;
}

extern "C" int pt_rms_norm_fp8(const void *x, const void *gamma, int rows, int dim, float eps, float act_scale, void *out, void *stream) {
  PT_REQUIRE(x && gamma && out, "pt_rms_norm_fp8: null pointer argument");
  PT_REQUIRE(rows > 0 && dim > 0 && dim % 8 == 0 && dim <= 8 * 8 * 256, "pt_rms_norm_fp8: bad shape [%d, %d] (dim a multiple of 8, at most 16384)", rows, dim);
  PT_REQUIRE(act_scale > 0.f, "pt_rms_norm_fp8: act_scale must be > 0");
  rms_norm_fp8_kernel<<<rows, 256, 0, as_stream(stream)>>>((const __half *)x, (const __half *)gamma, dim, eps, 1.0f / act_scale, (uint8_t *)out);
  PT_LAUNCH_CHECK("pt_rms_norm_fp8");
  return PT_OK;
}

extern "C" int pt_swiglu_fp8(const void *gate_up, int rows, int f, float act_scale, void *out, int out_ld, void *stream) {
  PT_REQUIRE(gate_up && out && rows > 0 && f > 0, "pt_swiglu_fp8: bad arguments");
  PT_REQUIRE(act_scale > 0.f, "pt_swiglu_fp8: act_scale must be > 0");
  swiglu_fp8_kernel<<<grid_for((size_t)rows * f), 256, 0, as_stream(stream)>>>((const __half *)gate_up, rows, f, 1.0f / act_scale, (uint8_t *)out,
                                                                                 out_ld > 0 ? out_ld : f);
  PT_LAUNCH_CHECK("pt_swiglu_fp8");
  return PT_OK;
}

extern "C" int pt_add_f16(const void *a, const void *b, int64_t n, void *out, void *stream) {
  PT_REQUIRE(a && b && out && n > 0, "pt_add_f16: bad arguments");
  add_f16_kernel<<<grid_for((size_t)n), 256, 0, as_stream(stream)>>>((const __half *)a, (const __half *)b, (size_t)n, (__half *)out);
  PT_LAUNCH_CHECK("pt_add_f16");
  return PT_OK;
}
