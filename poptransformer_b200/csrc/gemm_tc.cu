// Block-cooperative tensor-core GEMMs for 16 or more activation rows (batched decode, prefill):
//     Y[m, n] = sum_k X[m, k] * W[n, k]          W row-major with k contiguous, like every weight of the reference
//
//   * FP8:  W and X are OCP E4M3 bytes with per-tensor scales (the reference's FP8MatMul, custom_ops/matmul_fp8.cpp:885-1091,
//           in the E4M3 form): tcgen05.mma kind::f8f6f4, fp32 accumulation in tensor memory, scales applied in the epilogue.
//   * INT4: W is packed nibbles with fp16 group scales (utils/param_handler/precision_strategy.py:24-42,56-60).  A transform
//           warpgroup turns every staged tile into fp16(q) * scale - one fp16 rounding per weight, exactly the reference's
//           Int4ToHalf (custom_ops/int4_to_half_codelets.cpp:18-38) - in the shared-memory layout the tensor core reads;
//           tcgen05.mma kind::f16 multiplies it with the fp16 activations, fp32 accumulation.
//
// The weights are the big operand, so they take the 128-row M side of the instruction and the activation rows the N side
// (16 .. 256 columns): the kernel computes Y^T tiles, D[128 weight rows, mb activation rows] in tensor memory.
// One CTA per (128 weight rows, k-slice): warp 0 feeds a ring of shared-memory stages with TMA (cp.async.bulk.tensor, this GPU's
// memory only, no multicast), one thread of warp 1 issues the MMAs and hands stages back with tcgen05.commit, warps 2-5 convert
// (INT4) and run the epilogue (tcgen05.ld, scale, fp16, coalesced stores along n).  k-slices of one tile meet in a workspace and
// the last CTA to arrive sums them in slice order (deterministic).  Every wait is bounded: on a time-out the CTA raises the
// error flag, skips its remaining waits and still frees its tensor memory.
#include <cuda.h>

#include <algorithm>

#include "tile_math.cuh"

namespace pt {
namespace tc {

constexpr int BM = 128;            // weight rows per CTA
constexpr int BKB = 128;           // bytes of k per stage and operand row (one 128-byte swizzle atom)
constexpr int THREADS = 192;       // warp 0: TMA, warp 1: MMA + tensor-memory allocation, warps 2-5: transform + epilogue
constexpr int WAIT_LIMIT = 1 << 22;

struct GemmParams {
  int M, N, K;
  int mb;                 // activation rows per CTA (multiple of 16, at most 256)
  int int4;               // 1: INT4 weights (A tile produced by the transform warps), 0: FP8
  int group;              // INT4 scale group along k
  int kb_per_split, n_kb; // k blocks (of 128 bytes of operand row) per k-slice / in total
  int ksplit, stages;
  int epilogue;           // PT_EPI_STORE or PT_EPI_RESIDUAL
  float out_scale;
  const __half *scales;   // INT4: [N][K / group]
  const __half *residual;
  __half *out;
  int out_ld;
  float *partial;         // [ksplit][M][N] (ksplit > 1)
  int *counters;          // [n tiles * m tiles]
  int *error_flag;
};

// ------------------------------------------------------------------------------------------ PTX
__device__ __forceinline__ uint32_t sa(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
// Bounded wait; gives up at once when the CTA has already recorded a failure.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  for (int it = 0; it < WAIT_LIMIT; ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 1000;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    if (ok) return true;
    if (*abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst), "l"(map),
               "r"(bar), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem desc] * B[smem desc]
template <bool F8>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (F8)
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
                 "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
                 : "memory");
  else
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
                 "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
                 : "memory");
}
// The mbarrier gets one arrival once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                 "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the 128-byte swizzle (the layout
// TMA writes with CU_TENSOR_MAP_SWIZZLE_128B and the transform warps reproduce): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major operands)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                    // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                    // 128-byte swizzle
  return d;
}
// Instruction descriptor: fp32 accumulator, both operands K-major, M = 128, N = n.
__host__ __device__ inline uint32_t instr_desc(bool f8, int n) {
  uint32_t d = 0;
  d |= 1u << 4;                 // D format: fp32
  d |= 0u << 7;                 // A format: E4M3 (f8f6f4) / F16 (f16)
  d |= 0u << 10;                // B format: the same
  d |= (uint32_t)(n >> 3) << 17;
  d |= (uint32_t)(BM >> 4) << 24;
  (void)f8;
  return d;
}

struct SharedCtl {
  uint64_t full[8], ready[8], empty[8], accum;
  uint32_t tmem_base;
  volatile int abort;
  int last;
};

// Dynamic shared memory: [stage][A tile 16 KB | B tile mb * 128 B (| INT4: packed A tile 4 KB)], every tile 1024-byte aligned.
template <bool INT4>
__global__ void __launch_bounds__(THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                                             const GemmParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ SharedCtl ctl;
  unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BM, m0 = blockIdx.z * p.mb, ks = blockIdx.y;
  const int kb0 = ks * p.kb_per_split, kb1 = min(p.n_kb, kb0 + p.kb_per_split);
  const int n_it = kb1 - kb0;
  const uint32_t a_bytes = BM * BKB, b_bytes = (uint32_t)p.mb * BKB, raw_bytes = INT4 ? BM * 32u : 0u;
  const uint32_t stage_bytes = a_bytes + ((b_bytes + 1023u) & ~1023u) + ((raw_bytes + 1023u) & ~1023u);
  const uint32_t smem_s = sa(smem);
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < p.mb) tmem_cols <<= 1;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(sa(&ctl.full[s]), 1);
      mbar_init(sa(&ctl.ready[s]), 4);   // one arrival per transform warp
      mbar_init(sa(&ctl.empty[s]), 1);
    }
    mbar_init(sa(&ctl.accum), 1);
    ctl.abort = 0;
    ctl.last = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(sa(&ctl.tmem_base), tmem_cols);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = ctl.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int it = 0; it < n_it; ++it) {
        const int s = it % p.stages;
        if (it >= p.stages && !mbar_wait(sa(&ctl.empty[s]), ((it / p.stages) - 1) & 1, &ctl.abort)) {
          if (!ctl.abort && p.error_flag) atomicCAS(p.error_flag, 0, 21);
          ctl.abort = 1;
        }
        if (ctl.abort) break;
        const uint32_t st = smem_s + s * stage_bytes, fb = sa(&ctl.full[s]);
        const int kb = kb0 + it;
        mbar_expect_tx(fb, (INT4 ? raw_bytes : a_bytes) + b_bytes);
        if (INT4) {
          tma_load_2d(st + a_bytes + ((b_bytes + 1023u) & ~1023u), &map_w, kb * 32, n0, fb);   // 64 k of packed nibbles = 32 bytes per row
          tma_load_2d(st + a_bytes, &map_x, kb * 64, m0, fb);                                  // 64 fp16 activations per row
        } else {
          tma_load_2d(st, &map_w, kb * BKB, n0, fb);
          tma_load_2d(st + a_bytes, &map_x, kb * BKB, m0, fb);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(!INT4, p.mb);
      for (int it = 0; it < n_it; ++it) {
        const int s = it % p.stages;
        const uint32_t bar = INT4 ? sa(&ctl.ready[s]) : sa(&ctl.full[s]);
        if (!mbar_wait(bar, (it / p.stages) & 1, &ctl.abort)) {
          if (!ctl.abort && p.error_flag) atomicCAS(p.error_flag, 0, 22);
          ctl.abort = 1;
        }
        if (ctl.abort) break;
        fence_after();
        const uint32_t st = smem_s + s * stage_bytes;
        const uint64_t adesc = smem_desc_sw128(st), bdesc = smem_desc_sw128(st + a_bytes);
#pragma unroll
        for (int j = 0; j < 4; ++j)   // four MMAs of 32 bytes of k each; inside the swizzle atom the start address moves by 32 bytes
          umma<!INT4>(tmem, adesc + (uint64_t)(j * 2), bdesc + (uint64_t)(j * 2), idesc, (it > 0 || j > 0) ? 1u : 0u);
        umma_commit(sa(&ctl.empty[s]));
      }
      umma_commit(sa(&ctl.accum));   // fires when every MMA above has completed (at once if none was issued)
    }
  } else {
    // ------------------------------------------------ transform (INT4) + epilogue: warps 2-5, tensor-memory lane quarter warp % 4
    const int q = warp & 3;
    const int row = q * 32 + lane;            // row of the 128-row tile this thread owns
    if (INT4) {
      const int n = n0 + row;
      const int ngroups = p.K / p.group;
      for (int it = 0; it < n_it; ++it) {
        const int s = it % p.stages;
        if (!mbar_wait(sa(&ctl.full[s]), (it / p.stages) & 1, &ctl.abort)) {
          if (!ctl.abort && p.error_flag) atomicCAS(p.error_flag, 0, 23);
          ctl.abort = 1;
        }
        if (ctl.abort) break;
        const int kb = kb0 + it;
        unsigned char *st = smem + (size_t)s * stage_bytes;
        const uint4 *raw = reinterpret_cast<const uint4 *>(st + a_bytes + ((b_bytes + 1023u) & ~1023u) + row * 32);
        const uint4 w0 = raw[0], w1 = raw[1];
        const __half sc = (n < p.N) ? __ldg(p.scales + (size_t)n * ngroups + (kb * 64) / p.group) : __half(0);
        const __half2 s2 = __half2half2(sc);
        const __half2 offA = __float2half2_rn(1032.0f), offB = __float2half2_rn(72.0f);
        unsigned char *arow = st + (row >> 3) * 1024 + (row & 7) * 128;
        const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          // word c holds k = 8c .. 8c+7 as offset-binary nibbles u = q + 8: bits [0,4) k0, [16,20) k1, [4,8) k2, [20,24) k3, and the
          // same again one byte up for k4..k7.  (1024 + u) and (64 + u) are exact in fp16; subtracting the offsets is exact; the
          // product with the scale is the one fp16 rounding of the reference's Int4ToHalf.
          const uint32_t w = words[c], w8 = w >> 8;
          __half2 h[4];
          *reinterpret_cast<uint32_t *>(&h[0]) = (w & 0x000F000Fu) | 0x64006400u;
          *reinterpret_cast<uint32_t *>(&h[1]) = (w & 0x00F000F0u) | 0x54005400u;
          *reinterpret_cast<uint32_t *>(&h[2]) = (w8 & 0x000F000Fu) | 0x64006400u;
          *reinterpret_cast<uint32_t *>(&h[3]) = (w8 & 0x00F000F0u) | 0x54005400u;
          h[0] = __hmul2(__hsub2(h[0], offA), s2);
          h[1] = __hmul2(__hsub2(h[1], offB), s2);
          h[2] = __hmul2(__hsub2(h[2], offA), s2);
          h[3] = __hmul2(__hsub2(h[3], offB), s2);
          *reinterpret_cast<uint4 *>(arow + ((c ^ (row & 7)) << 4)) = *reinterpret_cast<const uint4 *>(h);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(sa(&ctl.ready[s]));
      }
    }
    // ---- epilogue
    if (!mbar_wait(sa(&ctl.accum), 0, &ctl.abort)) {
      if (!ctl.abort && p.error_flag) atomicCAS(p.error_flag, 0, 24);
      ctl.abort = 1;
    }
    fence_after();
    const int n = n0 + row;
    if (!ctl.abort && n_it > 0) {
      for (int c0 = 0; c0 < p.mb; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c0 + j;
            if (m >= p.M) break;
            const float acc = __uint_as_float(v[j]);
            if (p.ksplit > 1) {
              p.partial[((size_t)ks * p.M + m) * p.N + n] = acc;
            } else {
              __half y = __float2half_rn(acc * p.out_scale);
              if (p.epilogue == PT_EPI_RESIDUAL) y = h_add(__ldcg(p.residual + (size_t)m * p.N + n), y);
              p.out[(size_t)m * p.out_ld + n] = y;
            }
          }
        }
      }
    }
    fence_before();
  }

  // ---- k-slices of this tile meet: the last CTA to arrive sums them in slice order
  if (p.ksplit > 1) {
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int tile = blockIdx.z * gridDim.x + blockIdx.x;
      ctl.last = (atomicAdd(p.counters + tile, 1) == p.ksplit - 1);
      if (ctl.last) p.counters[tile] = 0;   // ready for the next launch on this stream
    }
    __syncthreads();
    if (ctl.last && !ctl.abort) {
      __threadfence();
      const int rows = min(p.mb, p.M - m0);
      for (int i = tid; i < rows * BM; i += THREADS) {
        const int m = m0 + i / BM, n = n0 + (i % BM);
        if (n >= p.N) continue;
        float acc = 0.f;
        for (int s = 0; s < p.ksplit; ++s) acc += __ldcg(p.partial + ((size_t)s * p.M + m) * p.N + n);
        __half y = __float2half_rn(acc * p.out_scale);
        if (p.epilogue == PT_EPI_RESIDUAL) y = h_add(__ldcg(p.residual + (size_t)m * p.N + n), y);
        p.out[(size_t)m * p.out_ld + n] = y;
      }
    }
  }
  __syncthreads();
  fence_after();
  if (warp == 1) tmem_dealloc(tmem, tmem_cols);
}

// Reference int4 checkpoint rows (int8 [n, k/2]: byte j = k 2j in the high nibble, k 2j+1 in the low, two's complement) -> words
// of eight offset-binary nibbles in the order the transform warps split with two masks: bits [0,4) k0, [16,20) k1, [4,8) k2,
// [20,24) k3, [8,12) k4, [24,28) k5, [12,16) k6, [28,32) k7.  Row-major, k contiguous, so TMA tiles it directly.
__global__ void int4_gemm_repack_kernel(const uint8_t *__restrict__ src, uint32_t *__restrict__ dst, size_t n_words) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t b = reinterpret_cast<const uint32_t *>(src)[i];   // four bytes = k 0..7 of this word
    uint32_t o = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t byte = (b >> (8 * j)) & 0xFFu;
      const uint32_t even = ((byte >> 4) ^ 8u) & 0xFu, odd = (byte ^ 8u) & 0xFu;   // k = 2j, 2j + 1
      // pair j -> positions: j = 0: (0, 16), 1: (4, 20), 2: (8, 24), 3: (12, 28)
      o |= even << (4 * j);
      o |= odd << (16 + 4 * j);
    }
    dst[i] = o;
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// 2-D row-major byte/fp16 matrix [rows][row_bytes]: box = box_bytes x box_rows.
static int make_map(CUtensorMap *map, const void *base, CUtensorMapDataType dt, int elem_bytes, uint64_t row_elems, uint64_t rows, uint32_t box_elems,
                    uint32_t box_rows, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return pt::set_error(PT_ERR_CUDA, "pt_gemm: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {row_elems, rows};
  const cuuint64_t strides[1] = {row_elems * (uint64_t)elem_bytes};
  const cuuint32_t box[2] = {box_elems, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return pt::set_error(PT_ERR_CUDA, "pt_gemm: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return PT_OK;
}

}  // namespace tc
}  // namespace pt

using namespace pt;

extern "C" size_t pt_gemm_int4_packed_bytes(int n_out, int k_in) { return (size_t)n_out * (k_in / 2); }

extern "C" int pt_gemm_int4_repack(const void *w, int n_out, int k_in, void *packed, void *stream) {
  PT_REQUIRE(w && packed && w != packed, "pt_gemm_int4_repack: needs distinct source and destination buffers");
  PT_REQUIRE(n_out > 0 && k_in > 0 && k_in % 128 == 0, "pt_gemm_int4_repack: k_in=%d must be a positive multiple of 128", k_in);
  const size_t n_words = (size_t)n_out * (k_in / 8);
  tc::int4_gemm_repack_kernel<<<sm_count() * 8, 256, 0, as_stream(stream)>>>((const uint8_t *)w, (uint32_t *)packed, n_words);
  PT_LAUNCH_CHECK("pt_gemm_int4_repack");
  return PT_OK;
}

extern "C" size_t pt_gemm_workspace_bytes(int m, int n_out, int max_ksplit) {
  const size_t tiles = (size_t)ceil_div(n_out, tc::BM) * (size_t)ceil_div(m, 16);
  return ((tiles * sizeof(int) + 255) / 256) * 256 + (size_t)max_ksplit * m * n_out * sizeof(float);
}

extern "C" int pt_gemm(const pt_gemm_args *a, void *stream) {
  PT_REQUIRE(a, "pt_gemm: null args");
  PT_REQUIRE(a->wfmt == PT_W_INT4 || a->wfmt == PT_W_FP8, "pt_gemm: weight format %d (INT4 or FP8)", a->wfmt);
  const bool int4 = a->wfmt == PT_W_INT4;
  PT_REQUIRE(a->m >= 1 && a->n_out >= 1 && a->k_in >= 128 && a->k_in % 128 == 0, "pt_gemm: bad shape m=%d n_out=%d k_in=%d (k_in a multiple of 128)",
             a->m, a->n_out, a->k_in);
  PT_REQUIRE(a->x && a->w && a->out, "pt_gemm: null x / w / out");
  PT_REQUIRE(((uintptr_t)a->x & 15) == 0 && ((uintptr_t)a->w & 15) == 0, "pt_gemm: x and w must be 16-byte aligned");
  PT_REQUIRE(a->epilogue == PT_EPI_STORE || a->epilogue == PT_EPI_RESIDUAL, "pt_gemm: epilogue %d (store or residual)", a->epilogue);
  PT_REQUIRE(a->epilogue != PT_EPI_RESIDUAL || a->residual, "pt_gemm: residual epilogue needs residual");
  if (int4)
    PT_REQUIRE(a->scales && a->group >= 128 && a->group % 128 == 0 && a->k_in % a->group == 0,
               "pt_gemm: INT4 needs scales and a group (%d) that is a multiple of 128 dividing k_in=%d", a->group, a->k_in);

  tc::GemmParams p{};
  p.M = a->m; p.N = a->n_out; p.K = a->k_in;
  p.int4 = int4 ? 1 : 0;
  p.group = int4 ? a->group : 0;
  p.mb = std::min(256, ceil_div(a->m, 16) * 16);
  const int m_tiles = ceil_div(a->m, p.mb);
  const int n_tiles = ceil_div(a->n_out, tc::BM);
  p.n_kb = int4 ? a->k_in / 64 : a->k_in / 128;
  // k-slices: fill the GPU when there are few tiles, but keep at least 8 k-blocks per CTA
  int ksplit = a->ksplit;
  if (ksplit <= 0) {
    ksplit = std::max(1, sm_count() / (n_tiles * m_tiles));
    ksplit = std::max(1, std::min(ksplit, p.n_kb / 8));
  }
  ksplit = std::max(1, std::min(ksplit, p.n_kb));
  p.kb_per_split = ceil_div(p.n_kb, ksplit);
  p.ksplit = ceil_div(p.n_kb, p.kb_per_split);
  p.epilogue = a->epilogue;
  p.out_scale = int4 ? 1.0f : (a->x_scale > 0.f ? a->x_scale : 1.0f) * (a->w_scale > 0.f ? a->w_scale : 1.0f);
  p.scales = (const __half *)a->scales;
  p.residual = (const __half *)a->residual;
  p.out = (__half *)a->out;
  p.out_ld = a->out_ld > 0 ? a->out_ld : a->n_out;
  p.error_flag = a->error_flag;
  if (p.ksplit > 1) {
    const size_t need = pt_gemm_workspace_bytes(a->m, a->n_out, p.ksplit);
    PT_REQUIRE(a->workspace && a->workspace_bytes >= need, "pt_gemm: %d k-slices need %zu workspace bytes, got %zu", p.ksplit, need, a->workspace_bytes);
    const size_t tiles = (size_t)ceil_div(a->n_out, tc::BM) * (size_t)ceil_div(a->m, 16);
    p.counters = (int *)a->workspace;
    p.partial = (float *)((char *)a->workspace + ((tiles * sizeof(int) + 255) / 256) * 256);
  }

  const uint32_t a_bytes = tc::BM * tc::BKB, b_bytes = (uint32_t)p.mb * tc::BKB, raw_bytes = int4 ? tc::BM * 32u : 0u;
  const uint32_t stage_bytes = a_bytes + ((b_bytes + 1023u) & ~1023u) + ((raw_bytes + 1023u) & ~1023u);
  p.stages = (int)std::min<uint32_t>(8, (200u * 1024u) / stage_bytes);
  PT_REQUIRE(p.stages >= 2, "pt_gemm: tile does not fit shared memory");
  const size_t smem = (size_t)p.stages * stage_bytes + 1024;

  CUtensorMap map_w, map_x;
  if (int4) {
    if (int rc = tc::make_map(&map_w, a->w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a->k_in / 2, (uint64_t)a->n_out, 32, tc::BM, CU_TENSOR_MAP_SWIZZLE_NONE)) return rc;
    if (int rc = tc::make_map(&map_x, a->x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)a->k_in, (uint64_t)a->m, 64, (uint32_t)p.mb, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  } else {
    if (int rc = tc::make_map(&map_w, a->w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a->k_in, (uint64_t)a->n_out, 128, tc::BM, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    if (int rc = tc::make_map(&map_x, a->x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a->k_in, (uint64_t)a->m, 128, (uint32_t)p.mb, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  }
  static bool attr_set = false;
  if (!attr_set) {
    PT_CUDA(cudaFuncSetAttribute(tc::gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    PT_CUDA(cudaFuncSetAttribute(tc::gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_set = true;
  }
  dim3 grid(n_tiles, p.ksplit, m_tiles);
  if (int4)
    tc::gemm_tc_kernel<true><<<grid, tc::THREADS, smem, as_stream(stream)>>>(map_w, map_x, p);
  else
    tc::gemm_tc_kernel<false><<<grid, tc::THREADS, smem, as_stream(stream)>>>(map_w, map_x, p);
  PT_LAUNCH_CHECK("pt_gemm");
  return PT_OK;
}
