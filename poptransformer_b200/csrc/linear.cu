// Streaming skinny matmul for decode-sized batches: y[b, n] = sum_k x[b, k] * W[n, k].
//
// One kernel template serves INT4 (fused dequant), FP16 and FP8-E4M3 weights.  The weights are
// streamed from HBM exactly once with fully coalesced 128-bit loads (each warp instruction reads
// 512 contiguous bytes of a pre-tiled layout), dequantised in registers to the same fp16 values the
// reference's Int4ToHalf produces (integer * fp16 scale, one fp16 rounding), and multiplied on the
// tensor cores with mma.m16n8k16 (fp16 x fp16 products are exact, accumulation in fp32) so that the
// CUDA cores only pay for the dequant; the activations (at most 32 rows) sit in shared memory.
// The kernel is HBM-bound: algorithmic bytes = packed weights + scales, read once.
//
// Tile order ("packed" layout, built once by pt_linear_repack):
//   w_packed[row_tile][chunk][half][lane] : one 16-byte unit each
//     row_tile = 16 output rows, lane = (g = lane/4, tig = lane%4), half h selects row g (+8),
//     chunk    = the k-range covered by 4 lanes x 16 bytes of one row
//                (INT4: 128 k, FP8: 64 k, FP16: 32 k),
//   so lane (g, tig) of a warp receives, per chunk, 16 bytes of row g and 16 bytes of row g+8, which
//   are exactly its A-fragments for the chunk's mma instructions.  INT4 words are re-ordered so that
//   nibble i / i+4 of a 32-bit word hold k = 2i / 2i+1 (offset-binary), which lets one LOP3 produce a
//   half2 of two consecutive k.
//   scales_packed[row_tile][group][g][h] fp16 (INT4 only).
#include <algorithm>

#include "common.cuh"

namespace pt {

template <int WFMT> struct WTraits;
template <> struct WTraits<PT_W_INT4> { static constexpr int kChunkK = 128, kUnits = 4; };
template <> struct WTraits<PT_W_FP8> { static constexpr int kChunkK = 64, kUnits = 2; };
template <> struct WTraits<PT_W_FP16> { static constexpr int kChunkK = 32, kUnits = 1; };

static inline int chunk_k(int wfmt) { return wfmt == PT_W_INT4 ? 128 : (wfmt == PT_W_FP8 ? 64 : 32); }
static inline int row_bytes(int wfmt, int k) { return wfmt == PT_W_INT4 ? k / 2 : (wfmt == PT_W_FP8 ? k : 2 * k); }

struct LinearParams {
  const uint4 *w;
  const __half2 *scales;
  const __half *x, *gamma, *bias, *residual;
  __half *out;
  float *partial;
  int *counters;
  int B, N, K, n_rt, nchunks, ngroups, group_chunks, chunks_per_split, ksplit, pro, epi, xs_stride, out_ld;
  float eps, inv_act_scale, out_scale;
};

// ------------------------------------------------------------------------------------------
// device helpers
__device__ __forceinline__ uint64_t make_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
// Weights are read once per token and never fit in L2 next to the activations: stream them past L1
// and mark them first to leave L2.
__device__ __forceinline__ uint4 ldg_stream(const uint4 *p, uint64_t pol) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(pol));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Offset-binary nibbles i and i+4 of `word` -> half2 (q_lo * s, q_hi * s), q = nibble - 8.
// (word >> 4i) & 0x000F000F | 0x64006400 is the fp16 pair (1024 + u_lo, 1024 + u_hi); subtracting 1032
// gives the exact signed integer, and the multiply rounds once like the reference's fp16 product.
template <int I> __device__ __forceinline__ uint32_t deq_i4(uint32_t word, __half2 s2) {
  uint32_t t = ((word >> (4 * I)) & 0x000F000Fu) | 0x64006400u;
  __half2 h = __hsub2(*reinterpret_cast<__half2 *>(&t), __half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408)));
  h = __hmul2(h, s2);
  return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t cvt_e4m3x2(uint32_t two_bytes) {
  __half2_raw r = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(two_bytes & 0xFFFFu), __NV_E4M3);
  return (uint32_t)r.x | ((uint32_t)r.y << 16);
}

// Expand one lane's 16 bytes of one row into A-fragment registers: frag[u][0..3] are the half2
// pairs (k0,k1) (k2,k3) (k4,k5) (k6,k7) of the lane's u-th group of 8 consecutive k.
template <int WFMT>
__device__ __forceinline__ void expand(uint4 v, __half2 s2, uint32_t (&frag)[WTraits<WFMT>::kUnits][4]) {
  if constexpr (WFMT == PT_W_INT4) {
    const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      frag[u][0] = deq_i4<0>(wd[u], s2);
      frag[u][1] = deq_i4<1>(wd[u], s2);
      frag[u][2] = deq_i4<2>(wd[u], s2);
      frag[u][3] = deq_i4<3>(wd[u], s2);
    }
  } else if constexpr (WFMT == PT_W_FP8) {
    const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      frag[u][0] = cvt_e4m3x2(wd[2 * u]);
      frag[u][1] = cvt_e4m3x2(wd[2 * u] >> 16);
      frag[u][2] = cvt_e4m3x2(wd[2 * u + 1]);
      frag[u][3] = cvt_e4m3x2(wd[2 * u + 1] >> 16);
    }
  } else {
    frag[0][0] = v.x; frag[0][1] = v.y; frag[0][2] = v.z; frag[0][3] = v.w;
  }
}

// ------------------------------------------------------------------------------------------
// Grid: (row_tiles, ksplit).  Block: 256 threads = 8 warps; warp w owns chunks w, w+8, ... of the
// block's k-slice.  Dynamic shared memory: activations (B rows, swizzled per chunk) then the 8-warp
// reduction buffer.
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

template <int WFMT, int NB, int U>
__global__ void __launch_bounds__(kThreads) linear_kernel(const LinearParams p) {
  constexpr int UNITS = WTraits<WFMT>::kUnits;
  constexpr int CHUNK_K = WTraits<WFMT>::kChunkK;
  constexpr int CHUNK_X_BYTES = CHUNK_K * 2;  // fp16 activations per chunk

  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char *xs = smem;
  float *red = reinterpret_cast<float *>(smem + (size_t)p.B * p.xs_stride);
  __shared__ float s_stat[32];
  __shared__ int s_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tig = lane & 3;
  const int rt = blockIdx.x, ks = blockIdx.y;
  const int c_begin = ks * p.chunks_per_split;
  const int c_end = min(p.nchunks, c_begin + p.chunks_per_split);

  const uint64_t pol = make_evict_first_policy();
  const uint4 *wrow = p.w + (size_t)rt * p.nchunks * 64;
  const __half2 *srow = p.scales + (size_t)rt * p.ngroups * 8 + g;

  // ---- first weight batch goes in flight before anything else
  uint4 wa[U], wb[U];
  __half2 sc[U];
  auto load_batch = [&](int c0, uint4 (&a)[U], uint4 (&b)[U], __half2 (&s)[U]) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = c0 + u * kWarps;
      if (c < c_end) {
        a[u] = ldg_stream(wrow + (size_t)c * 64 + lane, pol);
        b[u] = ldg_stream(wrow + (size_t)c * 64 + 32 + lane, pol);
        if constexpr (WFMT == PT_W_INT4) s[u] = __ldg(srow + (size_t)(c / p.group_chunks) * 8);
      }
    }
  };
  int c0 = c_begin + warp;
  load_batch(c0, wa, wb, sc);

  // ---- prologue: stage (and optionally normalise / quantise) the activation slice
  const int slice_units = (c_end - c_begin) * 4 * UNITS;  // 16-byte units per batch row
  const bool do_norm = (p.pro == PT_PRO_RMSNORM || p.pro == PT_PRO_RMSNORM_CAST_FP8);
  const bool do_cast = (p.pro == PT_PRO_CAST_FP8 || p.pro == PT_PRO_RMSNORM_CAST_FP8);
  if (do_norm) {
    // r_b = fp16(1 / sqrt(mean(x^2) + eps)) over the whole row (all chunks, not only this slice)
    for (int b = 0; b < p.B; ++b) {
      float ss = 0.f;
      const uint4 *xr = reinterpret_cast<const uint4 *>(p.x + (size_t)b * p.K);
      for (int i = tid; i < p.K / 8; i += kThreads) {
        uint4 v = __ldg(xr + i);
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __half22float2(h[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
      ss = block_sum(ss, red);
      if (tid == 0) s_stat[b] = __half2float(__float2half_rn(1.0f / sqrtf(ss / (float)p.K + p.eps)));
    }
    __syncthreads();
  }
  for (int i = tid; i < p.B * slice_units; i += kThreads) {
    const int b = i / slice_units, u = i - b * slice_units;
    const int cl = u / (4 * UNITS), r = u - cl * (4 * UNITS);
    const int t4 = r / UNITS, w = r - t4 * UNITS;
    const size_t k = (size_t)c_begin * CHUNK_K + (size_t)u * 8;
    uint4 v = __ldg(reinterpret_cast<const uint4 *>(p.x + (size_t)b * p.K + k));
    if (do_norm || do_cast) {
      __half *h = reinterpret_cast<__half *>(&v);
      const __half rb = do_norm ? __float2half_rn(s_stat[b]) : __half(0);
      uint4 gv = do_norm ? __ldg(reinterpret_cast<const uint4 *>(p.gamma + k)) : make_uint4(0, 0, 0, 0);
      const __half *gh = reinterpret_cast<const __half *>(&gv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        __half e = h[j];
        if (do_norm) e = h_mul(h_mul(e, rb), gh[j]);
        if (do_cast) e = e4m3_round_h(__half2float(e) * p.inv_act_scale);
        h[j] = e;
      }
    }
    *reinterpret_cast<uint4 *>(xs + (size_t)b * p.xs_stride + cl * CHUNK_X_BYTES + w * 64 + t4 * 16) = v;
  }
  __syncthreads();

  // ---- main loop: register double buffering, U chunks per batch
  float acc[NB][4];
#pragma unroll
  for (int t = 0; t < NB; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;

  auto compute_batch = [&](int cbase, const uint4 (&a)[U], const uint4 (&b)[U], const __half2 (&s)[U]) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = cbase + u * kWarps;
      if (c < c_end) {
        uint32_t fa[UNITS][4], fb[UNITS][4];
        __half2 sa2 = __half2(), sb2 = __half2();
        if constexpr (WFMT == PT_W_INT4) {
          sa2 = __half2(s[u].x, s[u].x);
          sb2 = __half2(s[u].y, s[u].y);
        }
        expand<WFMT>(a[u], sa2, fa);
        expand<WFMT>(b[u], sb2, fb);
        const unsigned char *xc = xs + (size_t)(c - c_begin) * CHUNK_X_BYTES + tig * 16;
#pragma unroll
        for (int w = 0; w < UNITS; ++w) {
#pragma unroll
          for (int t = 0; t < NB; ++t) {
            const int brow = g + 8 * t;
            uint4 xv = make_uint4(0, 0, 0, 0);
            if (brow < p.B) xv = *reinterpret_cast<const uint4 *>(xc + (size_t)brow * p.xs_stride + w * 64);
            mma16816(acc[t], fa[w][0], fb[w][0], fa[w][1], fb[w][1], xv.x, xv.y);
            mma16816(acc[t], fa[w][2], fb[w][2], fa[w][3], fb[w][3], xv.z, xv.w);
          }
        }
      }
    }
  };

  while (true) {
    const int cn = c0 + kWarps * U;
    const bool has_next = cn < c_end;
    uint4 na[U], nbv[U];
    __half2 ns[U];
    if (has_next) load_batch(cn, na, nbv, ns);
    compute_batch(c0, wa, wb, sc);
    if (!has_next) break;
#pragma unroll
    for (int u = 0; u < U; ++u) { wa[u] = na[u]; wb[u] = nbv[u]; sc[u] = ns[u]; }
    c0 = cn;
  }

  // ---- reduce the 8 warps' partial tiles in a fixed order
#pragma unroll
  for (int t = 0; t < NB; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) red[(warp * NB * 4 + t * 4 + j) * 32 + lane] = acc[t][j];
  __syncthreads();

  float val = 0.f;
  int row = 0, bcol = 0;
  const bool owner = tid < NB * 128;
  if (owner) {
    const int t = tid >> 7, j = (tid >> 5) & 3, ln = tid & 31;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) val += red[(w * NB * 4 + t * 4 + j) * 32 + ln];
    row = (ln >> 2) + 8 * (j >> 1);
    bcol = t * 8 + 2 * (ln & 3) + (j & 1);
  }
  const int npad = p.n_rt * 16;
  if (p.ksplit > 1) {
    if (owner && bcol < p.B) p.partial[((size_t)ks * p.B + bcol) * npad + rt * 16 + row] = val;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(p.counters + rt, 1) == p.ksplit - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (owner && bcol < p.B) {
      val = 0.f;
      for (int s = 0; s < p.ksplit; ++s) val += __ldcg(p.partial + ((size_t)s * p.B + bcol) * npad + rt * 16 + row);
    }
    if (tid == 0) p.counters[rt] = 0;  // ready for the next launch on this stream
  }
  __syncthreads();  // all reads of `red` done; reuse it as fin[row][batch]
  float *fin = red;
  if (owner) fin[row * (8 * NB) + bcol] = val * p.out_scale;
  __syncthreads();

  // ---- epilogue
  if (p.epi == PT_EPI_SWIGLU) {
    const int half_n = p.N / 2;
    for (int e = tid; e < 8 * p.B; e += kThreads) {
      const int f = e & 7, b = e >> 3;
      const int n = rt * 8 + f;
      if (n < half_n) {
        const __half gate = __float2half_rn(fin[f * (8 * NB) + b]);
        const __half up = __float2half_rn(fin[(f + 8) * (8 * NB) + b]);
        p.out[(size_t)b * p.out_ld + n] = h_mul(up, swish_h(gate));
      }
    }
    return;
  }
  for (int e = tid; e < 16 * p.B; e += kThreads) {
    const int r = e & 15, b = e >> 4;
    const int n = rt * 16 + r;
    if (n >= p.N) continue;
    __half y = __float2half_rn(fin[r * (8 * NB) + b]);
    const size_t o = (size_t)b * p.N + n;
    switch (p.epi) {
      case PT_EPI_RESIDUAL: y = h_add(p.residual[o], y); break;
      case PT_EPI_BIAS: y = h_add(y, p.bias[n]); break;
      case PT_EPI_BIAS_GELU: y = gelu_h(h_add(y, p.bias[n])); break;
      case PT_EPI_BIAS_RESIDUAL: y = h_add(p.residual[o], h_add(y, p.bias[n])); break;
      default: break;
    }
    p.out[(size_t)b * p.out_ld + n] = y;
  }
}

// ------------------------------------------------------------------------------------------
// One-time re-layout of W[n_out, k] (k contiguous) into the tile order above.
__global__ void repack_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, int wfmt, int n_out,
                              int units_per_row, int nchunks, int n_rt, int interleave) {
  const size_t total = (size_t)n_rt * nchunks * 64;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int lane = i & 31, h = (i >> 5) & 1;
    const size_t tc = i >> 6;
    const int c = tc % nchunks, rt = tc / nchunks;
    const int g = lane >> 2, tig = lane & 3;
    int row;
    if (interleave) {
      const int f = rt * 8 + g;
      row = (f < n_out / 2) ? (h ? n_out / 2 + f : f) : -1;
    } else {
      row = rt * 16 + h * 8 + g;
      if (row >= n_out) row = -1;
    }
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

__global__ void repack_scale_kernel(const __half *__restrict__ src, __half *__restrict__ dst, int n_out, int ngroups,
                                    int n_rt, int interleave) {
  const size_t total = (size_t)n_rt * ngroups * 16;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int h = i & 1, g = (i >> 1) & 7;
    const size_t tg = i >> 4;
    const int gi = tg % ngroups, rt = tg / ngroups;
    int row;
    if (interleave) {
      const int f = rt * 8 + g;
      row = (f < n_out / 2) ? (h ? n_out / 2 + f : f) : -1;
    } else {
      row = rt * 16 + h * 8 + g;
      if (row >= n_out) row = -1;
    }
    dst[i] = row >= 0 ? src[(size_t)row * ngroups + gi] : __half(0);
  }
}

template <int WFMT, int NB, int U> static int launch_linear(const LinearParams &p, size_t smem, cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    PT_CUDA(cudaFuncSetAttribute(linear_kernel<WFMT, NB, U>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_set = true;
  }
  dim3 grid(p.n_rt, p.ksplit);
  linear_kernel<WFMT, NB, U><<<grid, kThreads, smem, st>>>(p);
  PT_LAUNCH_CHECK("pt_linear");
  return PT_OK;
}

template <int WFMT> static int dispatch_nb(const LinearParams &p, size_t smem, cudaStream_t st) {
  if (p.B <= 8) return launch_linear<WFMT, 1, 2>(p, smem, st);
  if (p.B <= 16) return launch_linear<WFMT, 2, 2>(p, smem, st);
  return launch_linear<WFMT, 4, 1>(p, smem, st);
}

}  // namespace pt

using namespace pt;

extern "C" size_t pt_linear_packed_bytes(int wfmt, int n_out, int k_in) {
  const int n_rt = ceil_div(n_out, 16);
  return (size_t)n_rt * 16 * row_bytes(wfmt, k_in);
}

extern "C" size_t pt_linear_packed_scale_bytes(int wfmt, int n_out, int k_in, int group) {
  if (wfmt != PT_W_INT4 || group <= 0) return 0;
  return (size_t)ceil_div(n_out, 16) * 16 * (k_in / group) * sizeof(__half);
}

extern "C" size_t pt_linear_workspace_bytes(int batch, int n_out, int max_ksplit) {
  const size_t npad = (size_t)ceil_div(n_out, 16) * 16;
  // counters (one int per row tile, rounded up to 256 B) followed by the split-k partials
  const size_t counters = ((npad / 16) * sizeof(int) + 255) / 256 * 256;
  return counters + (size_t)max_ksplit * batch * npad * sizeof(float);
}

extern "C" int pt_linear_repack(int wfmt, const void *w, const void *scale, int n_out, int k_in, int group,
                                int interleave_rows, void *packed_w, void *packed_scale, void *stream) {
  PT_REQUIRE(wfmt == PT_W_INT4 || wfmt == PT_W_FP16 || wfmt == PT_W_FP8, "pt_linear_repack: unknown weight format %d", wfmt);
  PT_REQUIRE(n_out > 0 && k_in > 0 && k_in % chunk_k(wfmt) == 0, "pt_linear_repack: k_in=%d must be a positive multiple of %d",
             k_in, chunk_k(wfmt));
  PT_REQUIRE(!interleave_rows || n_out % 16 == 0, "pt_linear_repack: interleaved (gate|up) layout needs n_out %% 16 == 0, got %d", n_out);
  PT_REQUIRE(w && packed_w, "pt_linear_repack: null weight pointer");
  const int n_rt = ceil_div(n_out, 16);
  const int units_per_row = row_bytes(wfmt, k_in) / 16;
  const int nchunks = units_per_row / 4;
  cudaStream_t st = as_stream(stream);
  repack_kernel<<<148 * 8, 256, 0, st>>>((const uint4 *)w, (uint4 *)packed_w, wfmt, n_out, units_per_row, nchunks, n_rt,
                                         interleave_rows);
  PT_LAUNCH_CHECK("pt_linear_repack");
  if (wfmt == PT_W_INT4) {
    PT_REQUIRE(group > 0 && group % 128 == 0 && k_in % group == 0,
               "pt_linear_repack: INT4 group=%d must be a multiple of 128 dividing k_in=%d", group, k_in);
    PT_REQUIRE(scale && packed_scale, "pt_linear_repack: INT4 needs scales");
    repack_scale_kernel<<<148 * 2, 256, 0, st>>>((const __half *)scale, (__half *)packed_scale, n_out, k_in / group, n_rt,
                                                 interleave_rows);
    PT_LAUNCH_CHECK("pt_linear_repack(scales)");
  }
  return PT_OK;
}

extern "C" int pt_linear(const pt_linear_args *a, void *stream) {
  PT_REQUIRE(a, "pt_linear: null args");
  PT_REQUIRE(a->wfmt == PT_W_INT4 || a->wfmt == PT_W_FP16 || a->wfmt == PT_W_FP8, "pt_linear: unknown weight format %d", a->wfmt);
  PT_REQUIRE(a->batch >= 1 && a->batch <= 32, "pt_linear: batch=%d outside 1..32 (larger batches use the GEMM path)", a->batch);
  const int ck = chunk_k(a->wfmt);
  PT_REQUIRE(a->n_out > 0 && a->k_in > 0 && a->k_in % ck == 0, "pt_linear: k_in=%d must be a positive multiple of %d", a->k_in, ck);
  PT_REQUIRE(a->x && a->packed_w && a->out, "pt_linear: null x / packed_w / out");
  PT_REQUIRE(a->prologue >= PT_PRO_NONE && a->prologue <= PT_PRO_RMSNORM_CAST_FP8, "pt_linear: bad prologue %d", a->prologue);
  PT_REQUIRE(a->epilogue >= PT_EPI_STORE && a->epilogue <= PT_EPI_BIAS_RESIDUAL, "pt_linear: bad epilogue %d", a->epilogue);
  const bool norm = a->prologue == PT_PRO_RMSNORM || a->prologue == PT_PRO_RMSNORM_CAST_FP8;
  const bool cast = a->prologue == PT_PRO_CAST_FP8 || a->prologue == PT_PRO_RMSNORM_CAST_FP8;
  PT_REQUIRE(!norm || a->norm_gamma, "pt_linear: RMSNorm prologue needs norm_gamma");
  PT_REQUIRE(!cast || a->act_scale > 0.f, "pt_linear: FP8 activation cast needs act_scale > 0");
  if (a->epilogue == PT_EPI_RESIDUAL || a->epilogue == PT_EPI_BIAS_RESIDUAL) PT_REQUIRE(a->residual, "pt_linear: residual epilogue needs residual");
  if (a->epilogue >= PT_EPI_BIAS) PT_REQUIRE(a->bias, "pt_linear: bias epilogue needs bias");
  if (a->epilogue == PT_EPI_SWIGLU) PT_REQUIRE(a->n_out % 16 == 0, "pt_linear: SwiGLU epilogue needs n_out %% 16 == 0, got %d", a->n_out);

  LinearParams p{};
  p.w = (const uint4 *)a->packed_w;
  p.scales = (const __half2 *)a->packed_scale;
  p.x = (const __half *)a->x;
  p.gamma = (const __half *)a->norm_gamma;
  p.bias = (const __half *)a->bias;
  p.residual = (const __half *)a->residual;
  p.out = (__half *)a->out;
  p.B = a->batch; p.N = a->n_out; p.K = a->k_in;
  p.out_ld = a->out_ld > 0 ? a->out_ld : (a->epilogue == PT_EPI_SWIGLU ? a->n_out / 2 : a->n_out);
  p.n_rt = ceil_div(a->n_out, 16);
  p.nchunks = a->k_in / ck;
  p.pro = a->prologue; p.epi = a->epilogue;
  p.eps = a->norm_eps;
  p.inv_act_scale = cast ? 1.0f / a->act_scale : 1.0f;
  p.out_scale = 1.0f;
  if (a->wfmt == PT_W_FP8) p.out_scale = (a->w_scale > 0.f ? a->w_scale : 1.0f) * (cast ? a->act_scale : 1.0f);
  if (a->wfmt == PT_W_INT4) {
    PT_REQUIRE(a->group > 0 && a->group % 128 == 0 && a->k_in % a->group == 0,
               "pt_linear: INT4 group=%d must be a multiple of 128 dividing k_in=%d", a->group, a->k_in);
    PT_REQUIRE(a->packed_scale, "pt_linear: INT4 needs packed_scale");
    p.ngroups = a->k_in / a->group;
    p.group_chunks = a->group / 128;
  } else {
    p.ngroups = 0; p.group_chunks = 1;
  }

  // k-split: enough blocks to fill the machine, but at least kWarps chunks per block, and an activation slice
  // that fits shared memory.
  int ksplit = a->ksplit;
  if (ksplit <= 0) {
    ksplit = 1;
    const int want_blocks = 148 * 4;
    if (p.n_rt < want_blocks) ksplit = ceil_div(want_blocks, p.n_rt);
    ksplit = std::max(1, std::min(ksplit, p.nchunks / kWarps));
  }
  ksplit = std::min(ksplit, p.nchunks);
  const size_t smem_budget = 160 * 1024;
  auto xs_bytes = [&](int ksp) {
    const int cps = ceil_div(p.nchunks, ksp);
    const size_t slice = (size_t)cps * ck * 2;
    return (size_t)a->batch * (slice | 64);  // stride = 64 (mod 128) keeps the 8 batch rows of a quad on distinct banks
  };
  while (xs_bytes(ksplit) > smem_budget && ksplit < p.nchunks) ++ksplit;
  PT_REQUIRE(xs_bytes(ksplit) <= smem_budget, "pt_linear: activation slice does not fit shared memory (batch=%d k=%d)", a->batch, a->k_in);
  p.ksplit = ksplit;
  p.chunks_per_split = ceil_div(p.nchunks, ksplit);
  p.ksplit = ceil_div(p.nchunks, p.chunks_per_split);  // no empty splits
  p.xs_stride = (int)(((size_t)p.chunks_per_split * ck * 2) | 64);
  if (p.ksplit > 1) {
    const size_t need = pt_linear_workspace_bytes(a->batch, a->n_out, p.ksplit);
    PT_REQUIRE(a->workspace && a->workspace_bytes >= need, "pt_linear: split-k=%d needs %zu workspace bytes, got %zu", p.ksplit, need,
               a->workspace_bytes);
    const size_t counters = ((size_t)p.n_rt * sizeof(int) + 255) / 256 * 256;
    p.counters = (int *)a->workspace;
    p.partial = (float *)((char *)a->workspace + counters);
  }
  const int nb = a->batch <= 8 ? 1 : (a->batch <= 16 ? 2 : 4);
  const size_t smem = (size_t)p.B * p.xs_stride + (size_t)kWarps * nb * 4 * 32 * sizeof(float);
  cudaStream_t st = as_stream(stream);
  switch (a->wfmt) {
    case PT_W_INT4: return dispatch_nb<PT_W_INT4>(p, smem, st);
    case PT_W_FP16: return dispatch_nb<PT_W_FP16>(p, smem, st);
    default: return dispatch_nb<PT_W_FP8>(p, smem, st);
  }
}
