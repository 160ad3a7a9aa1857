// Streaming skinny matmul for decode-sized batches: y[b, n] = sum_k x[b, k] * W[n, k].
//
// One kernel template serves INT4 (fused dequant), FP16 and FP8-E4M3 weights.  The weights are
// streamed from HBM exactly once: every warp owns one 16-row tile and pulls its (contiguous) stream of
// 1 KB chunk tiles into a private shared-memory ring with 16-byte asynchronous copies (cp.async, two
// fully coalesced 512-byte warp requests per tile), so several kilobytes per warp are in flight without
// holding them in registers.  (Measured on B200: for these 1 KB tiles the per-warp cp.async ring streams
// at the rate of plain 128-bit loads, whereas a ring of 1 KB cp.async.bulk copies per warp was 1.5-2.5x
// slower, so the TMA engine is left to the attention kernel's larger tiles.)  The multiply runs on the
// tensor cores with mma.m16n8k16 (fp16 x fp16 products are exact, accumulation in fp32); the CUDA cores
// only turn nibbles into fp16.  The activations (at most 32 rows) sit in shared memory.
// The kernel is HBM-bound: algorithmic bytes = packed weights + scales, read once.
//
// Packed layout (built once by pt_linear_repack): tile[row_tile][chunk], each tile
//     64 x 16 B : unit [half h][lane] = 16 bytes of row (g + 8h) for lane (g = lane/4, tig = lane%4)
//   (+ 2 x 16 B : the 16 fp16 group scales of the tile's rows, [g][h], INT4 only)
//   chunk = the k-range covered by 4 lanes x 16 bytes of one row (INT4: 128 k, FP8: 64 k, FP16: 32 k),
//   so lane (g, tig) finds its A-fragments for the chunk's mma instructions at fixed offsets of the tile,
//   and the tiles of one row tile are contiguous in k order.
//
// INT4 arithmetic.  A 32-bit word holds 8 consecutive k as offset-binary nibbles u = q + 8, nibble i /
// i+4 holding k = 2i / 2i+1.  (w & 0x000F000F) | 0x64006400 is the fp16 pair (1024 + u, 1024 + u) and
// (w & 0x00F000F0) | 0x54005400 is the pair (64 + u, 64 + u), so one shift and four LOP3 turn a word
// into the four fragment registers of two mma instructions.  The constant offsets (1032 and 72 on top
// of q) are removed after the chunk's mma using per-chunk sums of x that the block computes once
// while staging x:  sum_k q_k x_k = sum_k h_k x_k - 1032 * sum_{k in A} x_k - 72 * sum_{k in B} x_k,
// and the group scale multiplies the fp32 chunk sum.  The reference instead rounds q * scale to fp16
// before its matmul (Int4ToHalf); the difference is at most 2^-12 relative per weight, far inside the
// logit tolerance, and pt_int4_to_half remains the bit-exact form of that op.
#include <algorithm>

#include "tile_math.cuh"

namespace pt {

constexpr int kWarps = 8;  // warps per block = row tiles per block
constexpr int kThreads = kWarps * 32;
// Ring depth per warp.  (Measured on B200 at 16 and 32 batch rows: 8 stages are slower than 4, the doubled ring costs more
// in resident blocks than the deeper prefetch gains.)
constexpr int kRingStages = 4;

struct LinearParams {
  const unsigned char *w;
  const __half *x, *gamma, *beta, *bias, *residual;
  __half *out;
  float *partial;
  int *counters, *error_flag;
  int B, N, K, n_rt, nchunks, chunks_per_split, ksplit, pro, epi, xs_stride, out_ld, pdl;
  float eps, inv_act_scale, out_scale;
};

// ------------------------------------------------------------------------------------------ device helpers
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// ------------------------------------------------------------------------------------------
// Grid: (ceil(row_tiles / 8), ksplit).  Block: 8 warps; warp w owns row tile blockIdx.x * 8 + w and the block's
// k-slice.  Dynamic shared memory: [activations, B rows, swizzled per chunk][INT4 offset corrections]
// [ring: 8 warps x kStages tiles].
template <int WFMT, int NB, int kStages>
__global__ void __launch_bounds__(kThreads) linear_kernel(const LinearParams p) {
  constexpr int UNITS = WTraits<WFMT>::kUnits;
  constexpr int CHUNK_K = WTraits<WFMT>::kChunkK;
  constexpr int TILE = WTraits<WFMT>::kTileBytes;
  constexpr int CHUNK_X_BYTES = CHUNK_K * 2;  // fp16 activations per chunk
  constexpr int BP = 8 * NB;                  // padded batch

  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tig = lane & 3;
  const int rt = blockIdx.x * kWarps + warp, ks = blockIdx.y;
  const bool active = rt < p.n_rt;
  const int c_begin = ks * p.chunks_per_split;
  const int c_end = min(p.nchunks, c_begin + p.chunks_per_split);
  const int nslice = c_end - c_begin;

  unsigned char *xs = smem;
  const size_t xs_bytes = ((size_t)p.B * p.xs_stride + 127) / 128 * 128;
  float *corr = reinterpret_cast<float *>(smem + xs_bytes);  // [slice chunks][BP] (INT4 only)
  const size_t corr_bytes = WFMT == PT_W_INT4 ? ((size_t)p.chunks_per_split * BP * sizeof(float) + 127) / 128 * 128 : 0;
  unsigned char *ring = smem + xs_bytes + corr_bytes + (size_t)warp * kStages * TILE;
  __shared__ float s_stat[32], s_mean[32];
  __shared__ float s_part[32 * kWarps], s_part1[32 * kWarps];
  __shared__ int s_last;

  // ---- start streaming this warp's tiles before anything else (they do not depend on the previous kernel)
  const unsigned char *wsrc = p.w + ((size_t)(active ? rt : 0) * p.nchunks + c_begin) * TILE + lane * 16;
  const uint32_t ring_lane = smem_addr(ring) + lane * 16;
  auto issue = [&](int i) {   // tile i of the slice -> stage i % kStages; always commits so that group counting stays uniform
    if (active && i < nslice) {
      const uint32_t d = ring_lane + (i % kStages) * TILE;
      const unsigned char *src = wsrc + (size_t)i * TILE;
      cp_async16(d, src);
      cp_async16(d + 512, src + 512);
      if (TILE > 1024 && lane < (TILE - 1024) / 16) cp_async16(d + 1024, src + 1024);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue(s);
  if (p.pdl) {
    // let the next kernel of the stream start its own weight prefetch, then wait for the producer of x
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }

  // ---- prologue: stage (and optionally normalise / quantise) the activation slice
  const int slice_units = nslice * 4 * UNITS;  // 16-byte units per batch row
  const bool norm_ce = p.pro == PT_PRO_NORMCE;   // LayerNorm with the NormCE arithmetic instead of RMSNorm
  const bool do_norm = (p.pro == PT_PRO_RMSNORM || p.pro == PT_PRO_RMSNORM_CAST_FP8 || norm_ce);
  const bool do_cast = (p.pro == PT_PRO_CAST_FP8 || p.pro == PT_PRO_RMSNORM_CAST_FP8);
  // Activations come from the previous kernel of the stream: read them through L2 (ld.cg) so that a line another
  // block of this SM cached earlier can never be served stale when kernels overlap.  The slice this block stages is
  // requested first (kept in registers when it is small), so the statistics pass adds no second round trip.
  constexpr int PRE = 4;
  const int total_units = p.B * slice_units;
  const bool fits = total_units <= PRE * kThreads;
  auto unit_src = [&](int i) {
    const int b = i / slice_units, u = i - b * slice_units;
    return reinterpret_cast<const uint4 *>(p.x + (size_t)b * p.K + (size_t)c_begin * CHUNK_K + (size_t)u * 8);
  };
  uint4 pre[PRE];
  if (fits) {
#pragma unroll
    for (int q = 0; q < PRE; ++q)
      if (tid + q * kThreads < total_units) pre[q] = __ldcg(unit_src(tid + q * kThreads));
  }
  if (do_norm) {
    // r_b = fp16(1 / sqrt(mean(x^2) + eps)) over the whole row (all chunks, not only this slice).  The 8 warps are spread over
    // the rows: with 8 or more rows warp w takes rows w, w + 8, ...; with fewer rows each row gets 8 / B warps that sum
    // interleaved parts of it.  Lane order, shuffle tree and the order of the parts are fixed: deterministic.
    const int units = p.K / 8;
    const int wpr = p.B >= kWarps ? 1 : kWarps / p.B;           // warps per row
    const int part = warp % wpr;
    for (int b = warp / wpr; b < p.B; b += kWarps / wpr) {
      float ss = 0.f, s1 = 0.f;
      const uint4 *xr = reinterpret_cast<const uint4 *>(p.x + (size_t)b * p.K);
      for (int i0 = part * 32 + lane; i0 < units; i0 += 4 * 32 * wpr) {
        uint4 v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] = (i0 + q * 32 * wpr < units) ? __ldcg(xr + i0 + q * 32 * wpr) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const __half2 *h = reinterpret_cast<const __half2 *>(&v[q]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __half22float2(h[j]);
            ss += f.x * f.x + f.y * f.y;
            s1 += f.x + f.y;
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (norm_ce) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      }
      if (lane == 0) {
        s_part[b * kWarps + part] = ss;
        s_part1[b * kWarps + part] = s1;
      }
    }
    __syncthreads();
    if (tid < p.B) {
      float ss = 0.f, s1 = 0.f;
      for (int q = 0; q < wpr; ++q) {
        ss += s_part[tid * kWarps + q];
        s1 += s_part1[tid * kWarps + q];
      }
      if (norm_ce) {
        // one row: GetInPlaceNorm's arithmetic (fp32 mean inside the variance, no clamp); several rows: normInfKernel's (the
        // fp16-rounded mean inside the variance, clamped at zero) -- custom_ops/NormCECodelets.cpp:65-112, NormCE.S:243-427
        const float inv_n = 1.0f / (float)p.K;
        if (p.B == 1) {
          const float mean = s1 * inv_n;
          s_mean[tid] = __half2float(__float2half_rn(mean));
          s_stat[tid] = __half2float(__float2half_rn(1.0f / sqrtf(ss * inv_n - mean * mean + p.eps)));
        } else {
          const float mf = __half2float(__float2half_rn(s1 * inv_n));
          s_mean[tid] = mf;
          s_stat[tid] = __half2float(__float2half_rn(1.0f / sqrtf(fmaxf(ss * inv_n - mf * mf, 0.f) + p.eps)));
        }
      } else {
        s_stat[tid] = __half2float(__float2half_rn(1.0f / sqrtf(ss / (float)p.K + p.eps)));
      }
    }
    __syncthreads();
  }
  auto stage_unit = [&](int i, uint4 v) {
    const int b = i / slice_units, u = i - b * slice_units;
    const int cl = u / (4 * UNITS), r = u - cl * (4 * UNITS);
    const int t4 = r / UNITS, w = r - t4 * UNITS;
    if (do_norm || do_cast) {
      const size_t k = (size_t)c_begin * CHUNK_K + (size_t)u * 8;
      __half *h = reinterpret_cast<__half *>(&v);
      const __half rb = do_norm ? __float2half_rn(s_stat[b]) : __half(0);
      const __half mb = norm_ce ? __float2half_rn(s_mean[b]) : __half(0);
      uint4 gv = do_norm ? __ldg(reinterpret_cast<const uint4 *>(p.gamma + k)) : make_uint4(0, 0, 0, 0);
      uint4 bv = norm_ce ? __ldg(reinterpret_cast<const uint4 *>(p.beta + k)) : make_uint4(0, 0, 0, 0);
      const __half *gh = reinterpret_cast<const __half *>(&gv), *bh = reinterpret_cast<const __half *>(&bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        __half e = h[j];
        if (norm_ce) e = h_add(h_mul(h_mul(h_sub(e, mb), rb), gh[j]), bh[j]);
        else if (do_norm) e = h_mul(h_mul(e, rb), gh[j]);
        if (do_cast) e = e4m3_round_h(__half2float(e) * p.inv_act_scale);
        h[j] = e;
      }
    }
    *reinterpret_cast<uint4 *>(xs + (size_t)b * p.xs_stride + cl * CHUNK_X_BYTES + w * 64 + t4 * 16) = v;
  };
  if (fits) {
#pragma unroll
    for (int q = 0; q < PRE; ++q)
      if (tid + q * kThreads < total_units) stage_unit(tid + q * kThreads, pre[q]);
  } else if constexpr (NB == 1) {
    for (int i = tid; i < total_units; i += kThreads) stage_unit(i, __ldcg(unit_src(i)));
  } else {
    for (int i0 = tid; i0 < total_units; i0 += PRE * kThreads) {   // PRE loads in flight per thread
      uint4 v[PRE];
#pragma unroll
      for (int q = 0; q < PRE; ++q)
        if (i0 + q * kThreads < total_units) v[q] = __ldcg(unit_src(i0 + q * kThreads));
#pragma unroll
      for (int q = 0; q < PRE; ++q)
        if (i0 + q * kThreads < total_units) stage_unit(i0 + q * kThreads, v[q]);
    }
  }
  __syncthreads();
  if constexpr (WFMT == PT_W_INT4) {
    // corr[chunk][b] = 1032 * sum of x over the k with offset 1032 + 72 * sum over the k with offset 72.
    // Four lanes (one per tig) share a (b, chunk); fixed order, so the result is deterministic.
    for (int i = tid; i < BP * nslice * 4; i += kThreads) {
      const int t4 = i & 3, b = (i >> 2) % BP, cl = i / (4 * BP);
      float sa = 0.f, sb = 0.f;
      if (b < p.B) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const uint4 v = *reinterpret_cast<const uint4 *>(xs + (size_t)b * p.xs_stride + cl * CHUNK_X_BYTES + w * 64 + t4 * 16);
          const float2 p0 = __half22float2(*reinterpret_cast<const __half2 *>(&v.x));
          const float2 p1 = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
          const float2 p2 = __half22float2(*reinterpret_cast<const __half2 *>(&v.z));
          const float2 p3 = __half22float2(*reinterpret_cast<const __half2 *>(&v.w));
          sa += (p0.x + p0.y) + (p2.x + p2.y);
          sb += (p1.x + p1.y) + (p3.x + p3.y);
        }
      }
      sa += __shfl_xor_sync(0xffffffffu, sa, 1);
      sb += __shfl_xor_sync(0xffffffffu, sb, 1);
      sa += __shfl_xor_sync(0xffffffffu, sa, 2);
      sb += __shfl_xor_sync(0xffffffffu, sb, 2);
      if (t4 == 0) corr[cl * BP + b] = kOffA * sa + kOffB * sb;
    }
    __syncthreads();
  }

  // ---- main loop over this warp's chunk tiles
  float acc[NB][4];
#pragma unroll
  for (int t = 0; t < NB; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;
  if (active) {
    const unsigned char *xbase = xs + tig * 16;
    for (int i = 0; i < nslice; ++i) {
      cp_async_wait<kStages - 2>();   // this lane's copies of tile i have landed
      __syncwarp();                   // ... and so have the other lanes'
      const unsigned char *tile = ring + (i % kStages) * TILE;
      const uint4 va = *reinterpret_cast<const uint4 *>(tile + lane * 16);
      const uint4 vb = *reinterpret_cast<const uint4 *>(tile + 512 + lane * 16);
      float2 sf = make_float2(1.f, 1.f);
      if constexpr (WFMT == PT_W_INT4) sf = __half22float2(*reinterpret_cast<const __half2 *>(tile + 1024 + g * 4));
      __syncwarp();                   // every lane holds its part of the tile in registers: the stage may be refilled
      issue(i + kStages - 1);
      float c[NB][4];
#pragma unroll
      for (int t = 0; t < NB; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) c[t][j] = 0.f;
      const unsigned char *xc = xbase + (size_t)i * CHUNK_X_BYTES;
#pragma unroll
      for (int u = 0; u < UNITS; ++u) {
        uint32_t fa[4], fb[4];
        expand8<WFMT>(va, u, fa);
        expand8<WFMT>(vb, u, fb);
#pragma unroll
        for (int t = 0; t < NB; ++t) {
          const int brow = g + 8 * t;
          uint4 xv = make_uint4(0, 0, 0, 0);
          if (brow < p.B) xv = *reinterpret_cast<const uint4 *>(xc + (size_t)brow * p.xs_stride + u * 64);
          if constexpr (WFMT == PT_W_INT4) {
            mma16816(c[t], fa[0], fb[0], fa[1], fb[1], xv.x, xv.y);
            mma16816(c[t], fa[2], fb[2], fa[3], fb[3], xv.z, xv.w);
          } else {
            mma16816(acc[t], fa[0], fb[0], fa[1], fb[1], xv.x, xv.y);
            mma16816(acc[t], fa[2], fb[2], fa[3], fb[3], xv.z, xv.w);
          }
        }
      }
      if constexpr (WFMT == PT_W_INT4) {
#pragma unroll
        for (int t = 0; t < NB; ++t) {
          const float2 co = *reinterpret_cast<const float2 *>(corr + i * BP + t * 8 + 2 * tig);
          acc[t][0] += sf.x * (c[t][0] - co.x);
          acc[t][1] += sf.x * (c[t][1] - co.y);
          acc[t][2] += sf.y * (c[t][2] - co.x);
          acc[t][3] += sf.y * (c[t][3] - co.y);
        }
      }
    }
  }
  cp_async_wait<0>();

  // ---- split-k: partials to the workspace; the last block of this row group sums them in split order
  const int npad = p.n_rt * 16;
  if (p.ksplit > 1) {
    if (active) {
#pragma unroll
      for (int t = 0; t < NB; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int bcol = t * 8 + 2 * tig + (j & 1), row = g + 8 * (j >> 1);
          if (bcol < p.B) p.partial[((size_t)ks * p.B + bcol) * npad + rt * 16 + row] = acc[t][j];
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(p.counters + blockIdx.x, 1) == p.ksplit - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) p.counters[blockIdx.x] = 0;  // ready for the next launch on this stream
    if (active) {
      // Sum in split order (deterministic).  The loads of two splits (2 x 4 NB values) are issued together, so the reduction
      // costs ksplit / 2 trips to L2 instead of one per (value, split).
#pragma unroll
      for (int t = 0; t < NB; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;
      const float *base = p.partial + (size_t)rt * 16 + g;
      for (int s0 = 0; s0 < p.ksplit; s0 += 2) {
        float a0[NB][4], a1[NB][4];
        const bool two = s0 + 1 < p.ksplit;
#pragma unroll
        for (int t = 0; t < NB; ++t)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int bcol = t * 8 + 2 * tig + (j & 1), row8 = 8 * (j >> 1);
            const bool ok = bcol < p.B;
            a0[t][j] = ok ? __ldcg(base + ((size_t)s0 * p.B + bcol) * npad + row8) : 0.f;
            a1[t][j] = (ok && two) ? __ldcg(base + ((size_t)(s0 + 1) * p.B + bcol) * npad + row8) : 0.f;
          }
#pragma unroll
        for (int t = 0; t < NB; ++t)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[t][j] += a0[t][j];
            if (two) acc[t][j] += a1[t][j];
          }
      }
    }
  }
  if (!active) return;

  // ---- epilogue straight from the accumulator registers: lane (g, tig) holds rows g, g+8 x batch columns 2tig, 2tig+1
#pragma unroll
  for (int t = 0; t < NB; ++t) {
#pragma unroll
    for (int jb = 0; jb < 2; ++jb) {
      const int b = t * 8 + 2 * tig + jb;
      if (b >= p.B) continue;
      const float lo = acc[t][jb] * p.out_scale, hi = acc[t][2 + jb] * p.out_scale;  // rows g and g + 8
      if (p.epi == PT_EPI_SWIGLU) {
        const int n = rt * 8 + g;  // rows 0..7 of the tile are gate rows, 8..15 the matching up rows
        if (n < p.N / 2) p.out[(size_t)b * p.out_ld + n] = h_mul(__float2half_rn(hi), swish_h(__float2half_rn(lo)));
        continue;
      }
#pragma unroll
      for (int hr = 0; hr < 2; ++hr) {
        const int n = rt * 16 + g + 8 * hr;
        if (n >= p.N) continue;
        __half y = __float2half_rn(hr ? hi : lo);
        const size_t o = (size_t)b * p.N + n;
        switch (p.epi) {
          case PT_EPI_RESIDUAL: y = h_add(__ldcg(p.residual + o), y); break;
          case PT_EPI_BIAS: y = h_add(y, p.bias[n]); break;
          case PT_EPI_BIAS_GELU: y = gelu_h(h_add(y, p.bias[n])); break;
          case PT_EPI_BIAS_RESIDUAL: y = h_add(__ldcg(p.residual + o), h_add(y, p.bias[n])); break;
          default: break;
        }
        p.out[(size_t)b * p.out_ld + n] = y;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// One-time re-layout of W[n_out, k] (k contiguous) into the tile order above.
__global__ void repack_kernel(const uint4 *__restrict__ src, const __half *__restrict__ scale, uint4 *__restrict__ dst, int wfmt, int n_out,
                              int units_per_row, int nchunks, int n_rt, int interleave, int ngroups, int group_chunks) {
  const int tile_u = wfmt == PT_W_INT4 ? 66 : 64;  // 16-byte units per tile
  const size_t total = (size_t)n_rt * nchunks * tile_u;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int e = i % tile_u;
    const size_t tc = i / tile_u;
    const int c = tc % nchunks, rt = tc / nchunks;
    auto src_row = [&](int h, int g) {
      int row;
      if (interleave) {
        const int f = rt * 8 + g;
        row = (f < n_out / 2) ? (h ? n_out / 2 + f : f) : -1;
      } else {
        row = rt * 16 + h * 8 + g;
        if (row >= n_out) row = -1;
      }
      return row;
    };
    if (e >= 64) {  // the tile's 16 scales as fp16 [g][h]; units 64 and 65 hold g = 0..3 and 4..7
      __half sc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int g = (e - 64) * 4 + j / 2, h = j & 1;
        const int row = src_row(h, g);
        sc[j] = row >= 0 ? scale[(size_t)row * ngroups + c / group_chunks] : __half(0);
      }
      dst[i] = *reinterpret_cast<uint4 *>(sc);
      continue;
    }
    const int lane = e & 31, h = e >> 5;
    const int g = lane >> 2, tig = lane & 3;
    const int row = src_row(h, g);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row >= 0) v = src[(size_t)row * units_per_row + c * 4 + tig];
    if (wfmt == PT_W_INT4) {
      uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        // source bytes j = 0..3: high nibble = k 2j, low nibble = k 2j+1 (two's complement);
        // destination nibble j <- high ^ 8, nibble j+4 <- low ^ 8 (offset-binary).
        uint32_t o = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t byte = (wd[w] >> (8 * j)) & 0xFFu;
          o |= (((byte >> 4) ^ 8u) & 0xFu) << (4 * j);
          o |= ((byte ^ 8u) & 0xFu) << (4 * (j + 4));
        }
        wd[w] = (row >= 0) ? o : 0x88888888u;
      }
      v = make_uint4(wd[0], wd[1], wd[2], wd[3]);
    }
    dst[i] = v;
  }
}

template <int WFMT, int NB, int ST> static int launch_linear(const LinearParams &p, size_t smem, cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    PT_CUDA(cudaFuncSetAttribute(linear_kernel<WFMT, NB, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ceil_div(p.n_rt, kWarps), p.ksplit);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, linear_kernel<WFMT, NB, ST>, p);
  if (e != cudaSuccess) return pt::set_error(PT_ERR_CUDA, "pt_linear: %s", cudaGetErrorString(e));
  PT_LAUNCH_CHECK("pt_linear");
  return PT_OK;
}

template <int WFMT> static int dispatch_nb(const LinearParams &p, size_t smem, cudaStream_t st) {
  if (p.B <= 8) return launch_linear<WFMT, 1, kRingStages>(p, smem, st);
  if (p.B <= 16) return launch_linear<WFMT, 2, kRingStages>(p, smem, st);
  return launch_linear<WFMT, 4, kRingStages>(p, smem, st);
}

}  // namespace pt

using namespace pt;

extern "C" size_t pt_linear_packed_bytes(int wfmt, int n_out, int k_in) {
  const int n_rt = ceil_div(n_out, 16);
  return (size_t)n_rt * (k_in / chunk_k(wfmt)) * tile_bytes(wfmt);
}

// Split-k workspace layout: [arrival counters, kCounterBytes][partial sums].  The counter region has ONE size for every shape,
// so that linears of different widths can share a workspace: a narrow linear's partial sums never land where a wide one
// expects zeroed counters.  One counter per group of 8 row tiles: 2048 counters cover n_out up to 262144.
constexpr size_t kCounterBytes = 8192;
constexpr int kMaxCounters = (int)(kCounterBytes / sizeof(int));

extern "C" size_t pt_linear_workspace_bytes(int batch, int n_out, int max_ksplit) {
  const size_t npad = (size_t)ceil_div(n_out, 16) * 16;
  return kCounterBytes + (size_t)max_ksplit * batch * npad * sizeof(float);
}

namespace {
// The k-split of a linear launch and the shared memory it needs; one rule for pt_linear and pt_linear_static_scratch.
// About 24 warps per SM in total (one warp per (row tile, k-slice)); at least 8 chunks (8 KB of weights) per warp for
// FP16 / FP8 so that the fixed cost of a warp (prologue, split-k reduction) stays small, 4 chunks for INT4, whose tiles carry
// four times the math (both measured on B200 over the decode shapes of the supported models); and an activation slice that
// fits shared memory next to the rings.
struct SplitPlan { int ksplit, chunks_per_split; size_t smem; bool fits; };
SplitPlan plan_split(int wfmt, int batch, int n_out, int k_in, int ksplit_req) {
  const int ck = chunk_k(wfmt), n_rt = ceil_div(n_out, 16), nchunks = k_in / ck;
  const int nb = batch <= 8 ? 1 : (batch <= 16 ? 2 : 4);
  int ksplit = ksplit_req;
  if (ksplit <= 0) {
    const int want_warps = sm_count() * 24;
    ksplit = std::max(1, want_warps / n_rt);
    ksplit = std::max(1, std::min(ksplit, nchunks / (wfmt == PT_W_INT4 ? 4 : 8)));
  }
  ksplit = std::max(1, std::min(ksplit, nchunks));
  const size_t ring_bytes = (size_t)kWarps * kRingStages * tile_bytes(wfmt);
  const size_t smem_budget = 200 * 1024;
  auto smem_bytes = [&](int ksp) {
    const int cps = ceil_div(nchunks, ksp);
    const size_t slice = (size_t)cps * ck * 2;
    // row stride = 64 (mod 128) keeps the 8 batch rows of a quad on distinct banks
    const size_t xs = ((size_t)batch * (slice | 64) + 127) / 128 * 128;
    const size_t corr = wfmt == PT_W_INT4 ? ((size_t)cps * 8 * nb * sizeof(float) + 127) / 128 * 128 : 0;
    return xs + corr + ring_bytes;
  };
  while (smem_bytes(ksplit) > smem_budget && ksplit < nchunks) ++ksplit;
  SplitPlan pl;
  pl.fits = smem_bytes(ksplit) <= smem_budget;
  pl.chunks_per_split = ceil_div(nchunks, ksplit);
  pl.ksplit = ceil_div(nchunks, pl.chunks_per_split);  // no empty splits
  pl.smem = smem_bytes(pl.ksplit);
  return pl;
}
}  // namespace

extern "C" int pt_linear_repack(int wfmt, const void *w, const void *scale, int n_out, int k_in, int group, int interleave_rows,
                                void *packed_w, void *stream) {
  PT_REQUIRE(wfmt == PT_W_INT4 || wfmt == PT_W_FP16 || wfmt == PT_W_FP8, "pt_linear_repack: unknown weight format %d", wfmt);
  PT_REQUIRE(n_out > 0 && k_in > 0 && k_in % chunk_k(wfmt) == 0, "pt_linear_repack: k_in=%d must be a positive multiple of %d", k_in,
             chunk_k(wfmt));
  PT_REQUIRE(!interleave_rows || n_out % 16 == 0, "pt_linear_repack: interleaved (gate|up) layout needs n_out %% 16 == 0, got %d", n_out);
  PT_REQUIRE(w && packed_w, "pt_linear_repack: null weight pointer");
  int ngroups = 0, group_chunks = 1;
  if (wfmt == PT_W_INT4) {
    PT_REQUIRE(group > 0 && group % 128 == 0 && k_in % group == 0, "pt_linear_repack: INT4 group=%d must be a multiple of 128 dividing k_in=%d",
               group, k_in);
    PT_REQUIRE(scale, "pt_linear_repack: INT4 needs scales");
    ngroups = k_in / group;
    group_chunks = group / 128;
  }
  const int n_rt = ceil_div(n_out, 16);
  const int units_per_row = row_bytes(wfmt, k_in) / 16;
  const int nchunks = units_per_row / 4;
  repack_kernel<<<sm_count() * 8, 256, 0, as_stream(stream)>>>((const uint4 *)w, (const __half *)scale, (uint4 *)packed_w, wfmt, n_out, units_per_row,
                                                       nchunks, n_rt, interleave_rows, ngroups, group_chunks);
  PT_LAUNCH_CHECK("pt_linear_repack");
  return PT_OK;
}

extern "C" int pt_linear(const pt_linear_args *a, void *stream) {
  PT_REQUIRE(a, "pt_linear: null args");
  PT_REQUIRE(a->wfmt == PT_W_INT4 || a->wfmt == PT_W_FP16 || a->wfmt == PT_W_FP8, "pt_linear: unknown weight format %d", a->wfmt);
  PT_REQUIRE(a->batch >= 1 && a->batch <= 32, "pt_linear: batch=%d outside 1..32 (larger batches use the GEMM path)", a->batch);
  const int ck = chunk_k(a->wfmt);
  PT_REQUIRE(a->n_out > 0 && a->k_in > 0 && a->k_in % ck == 0, "pt_linear: k_in=%d must be a positive multiple of %d", a->k_in, ck);
  PT_REQUIRE(a->x && a->packed_w && a->out, "pt_linear: null x / packed_w / out");
  PT_REQUIRE(a->prologue >= PT_PRO_NONE && a->prologue <= PT_PRO_NORMCE, "pt_linear: bad prologue %d", a->prologue);
  PT_REQUIRE(a->epilogue >= PT_EPI_STORE && a->epilogue <= PT_EPI_BIAS_RESIDUAL, "pt_linear: bad epilogue %d", a->epilogue);
  const bool norm = a->prologue == PT_PRO_RMSNORM || a->prologue == PT_PRO_RMSNORM_CAST_FP8 || a->prologue == PT_PRO_NORMCE;
  PT_REQUIRE(a->prologue != PT_PRO_NORMCE || a->norm_beta, "pt_linear: NormCE prologue needs norm_beta");
  const bool cast = a->prologue == PT_PRO_CAST_FP8 || a->prologue == PT_PRO_RMSNORM_CAST_FP8;
  PT_REQUIRE(!norm || a->norm_gamma, "pt_linear: RMSNorm prologue needs norm_gamma");
  PT_REQUIRE(!cast || a->act_scale > 0.f, "pt_linear: FP8 activation cast needs act_scale > 0");
  if (a->epilogue == PT_EPI_RESIDUAL || a->epilogue == PT_EPI_BIAS_RESIDUAL) PT_REQUIRE(a->residual, "pt_linear: residual epilogue needs residual");
  if (a->epilogue >= PT_EPI_BIAS) PT_REQUIRE(a->bias, "pt_linear: bias epilogue needs bias");
  if (a->epilogue == PT_EPI_SWIGLU) PT_REQUIRE(a->n_out % 16 == 0, "pt_linear: SwiGLU epilogue needs n_out %% 16 == 0, got %d", a->n_out);
  if (a->wfmt == PT_W_INT4)
    PT_REQUIRE(a->group > 0 && a->group % 128 == 0 && a->k_in % a->group == 0, "pt_linear: INT4 group=%d must be a multiple of 128 dividing k_in=%d",
               a->group, a->k_in);

  LinearParams p{};
  p.w = (const unsigned char *)a->packed_w;
  p.x = (const __half *)a->x;
  p.gamma = (const __half *)a->norm_gamma;
  p.beta = (const __half *)a->norm_beta;
  p.bias = (const __half *)a->bias;
  p.residual = (const __half *)a->residual;
  p.out = (__half *)a->out;
  p.error_flag = a->error_flag;
  p.pdl = a->pdl ? 1 : 0;
  p.B = a->batch; p.N = a->n_out; p.K = a->k_in;
  p.out_ld = a->out_ld > 0 ? a->out_ld : (a->epilogue == PT_EPI_SWIGLU ? a->n_out / 2 : a->n_out);
  p.n_rt = ceil_div(a->n_out, 16);
  p.nchunks = a->k_in / ck;
  p.pro = a->prologue; p.epi = a->epilogue;
  p.eps = a->norm_eps;
  p.inv_act_scale = cast ? 1.0f / a->act_scale : 1.0f;
  p.out_scale = 1.0f;
  if (a->wfmt == PT_W_FP8) p.out_scale = (a->w_scale > 0.f ? a->w_scale : 1.0f) * (cast ? a->act_scale : 1.0f);

  const SplitPlan plan = plan_split(a->wfmt, a->batch, a->n_out, a->k_in, a->ksplit);
  PT_REQUIRE(plan.fits, "pt_linear: activation slice does not fit shared memory (batch=%d k=%d)", a->batch, a->k_in);
  p.chunks_per_split = plan.chunks_per_split;
  p.ksplit = plan.ksplit;
  p.xs_stride = (int)(((size_t)p.chunks_per_split * ck * 2) | 64);
  if (p.ksplit > 1) {
    const size_t need = pt_linear_workspace_bytes(a->batch, a->n_out, p.ksplit);
    PT_REQUIRE(a->workspace && a->workspace_bytes >= need, "pt_linear: split-k=%d needs %zu workspace bytes, got %zu", p.ksplit, need,
               a->workspace_bytes);
    PT_REQUIRE(ceil_div(p.n_rt, kWarps) <= kMaxCounters, "pt_linear: n_out=%d exceeds the %d arrival counters of a split-k workspace", a->n_out,
               kMaxCounters);
    p.counters = (int *)a->workspace;
    p.partial = (float *)((char *)a->workspace + kCounterBytes);
  }
  const size_t smem = plan.smem;
  cudaStream_t st = as_stream(stream);
  switch (a->wfmt) {
    case PT_W_INT4: return dispatch_nb<PT_W_INT4>(p, smem, st);
    case PT_W_FP16: return dispatch_nb<PT_W_FP16>(p, smem, st);
    default: return dispatch_nb<PT_W_FP8>(p, smem, st);
  }
}

// ------------------------------------------------------------------------------------------ no-allocation variant
// Split-k scratch that lives in the library image: 4 MiB per GPU that loads the library, held until the process exits.
namespace {
constexpr size_t kStaticWsBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_linear_static_ws[kStaticWsBytes];
}  // namespace

// pt_linear for callers that have no way to obtain device scratch memory (see include/pt_b200.h).
// The name g_linear_static_ws is only a host-side handle here; the device address is fetched once per device with
// cudaGetSymbolAddress (with that device current) and cached.
extern "C" int pt_linear_static_scratch(const pt_linear_args *a, void *stream) {
  PT_REQUIRE(a, "pt_linear_static_scratch: null args");
  int dev = -1;
  PT_CUDA(cudaGetDevice(&dev));
  PT_REQUIRE(dev >= 0 && dev < 64, "pt_linear_static_scratch: device ordinal %d outside 0..63", dev);
  static void *ws_of_device[64] = {};
  if (!ws_of_device[dev]) {  // first call on this device: resolve the array's device address
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_linear_static_ws);
    if (e != cudaSuccess || !ptr) return pt::set_error(PT_ERR_CUDA, "pt_linear_static_scratch: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    ws_of_device[dev] = ptr;
  }
  const int ck = chunk_k(a->wfmt == PT_W_INT4 || a->wfmt == PT_W_FP16 || a->wfmt == PT_W_FP8 ? a->wfmt : PT_W_FP16);
  PT_REQUIRE(a->batch >= 1 && a->n_out > 0 && a->k_in > 0 && a->k_in % ck == 0, "pt_linear_static_scratch: bad shape batch=%d n_out=%d k_in=%d",
             a->batch, a->n_out, a->k_in);
  PT_REQUIRE(a->batch <= 32, "pt_linear_static_scratch: batch=%d outside 1..32", a->batch);
  // The split pt_linear will settle on (one rule, shared with it), so that the scratch need is known before the launch.
  const SplitPlan plan = plan_split(a->wfmt, a->batch, a->n_out, a->k_in, a->ksplit);
  PT_REQUIRE(plan.fits, "pt_linear_static_scratch: activation slice does not fit shared memory (batch=%d k=%d)", a->batch, a->k_in);
  const size_t need = plan.ksplit > 1 ? pt_linear_workspace_bytes(a->batch, a->n_out, plan.ksplit) : 0;
  PT_REQUIRE(need <= kStaticWsBytes,
             "pt_linear_static_scratch: batch=%d n_out=%d k-split=%d needs %zu bytes of scratch, the built-in scratch holds %zu; use pt_linear "
             "with a caller-provided workspace",
             a->batch, a->n_out, plan.ksplit, need, (size_t)kStaticWsBytes);
  pt_linear_args b = *a;
  b.ksplit = plan.ksplit;
  b.workspace = ws_of_device[dev];
  b.workspace_bytes = kStaticWsBytes;
  if (plan.ksplit > 1) {
    // The array keeps whatever the previous call left; the arrival counters at its start must be zero.
    PT_CUDA(cudaMemsetAsync(ws_of_device[dev], 0, kCounterBytes, as_stream(stream)));
  }
  return pt_linear(&b, stream);
}
