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
// One CTA per (128 weight rows, k-slice).  Weights of a model are tiled once at load time (pt_gemm_repack) so that the tile of
// every stage is one contiguous run in global memory, already in the shared-memory image the tensor core wants: the producer
// fetches it with a single bulk copy (measured on B200: a 2-D TMA box of 128 strided rows costs about 0.65 us per box whatever
// the row width, which caps an SM near 25 GB/s; contiguous bulk copies stream at the HBM rate).  The activations (few rows) and
// the row-major weights of the plain FP8MatMul op come through tiled TMA (cp.async.bulk.tensor; this GPU's memory only, no
// multicast).  One thread issues the MMAs and hands stages back with tcgen05.commit; the other warps convert (INT4: a deep ring
// of raw nibble tiles feeds a short ring of fp16 operand tiles) and run the epilogue (tcgen05.ld, scale, fp16, coalesced stores
// along n).  k-slices of one tile meet in a workspace and the last CTA to arrive sums them in slice order (deterministic).
// Every wait is bounded: on a time-out the CTA raises the error flag, skips its remaining waits and still frees its tensor
// memory.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "tile_math.cuh"

namespace pt {
namespace tc {

constexpr int BM = 128;            // weight rows per CTA
constexpr int BKB = 128;           // bytes of k per stage and operand row (one 128-byte swizzle atom)
constexpr int THREADS_F8 = 192;    // warp 0: producer, warp 1: MMA + tensor-memory allocation, warps 2-5: epilogue
constexpr int THREADS_I4 = 352;    // warp 0: raw-tile producer, warp 1: MMA, warps 2-9: transform + epilogue, warp 10: activation producer
constexpr int A_TILE = BM * BKB;   // 16 KB: 128 rows x 128 bytes of k, 128-byte swizzle
constexpr int RAW_TILE = BM * 32;  // 4 KB: 128 rows x 64 k of packed nibbles
constexpr int WAIT_LIMIT = 1 << 22;
#ifndef PT_TC_HINT
#define PT_TC_HINT 1000   // suspend-time hint (ns) of the barrier waits; negative: plain polling with test_wait
#endif

struct GemmParams {
  int M, N, K;
  int mb;                 // activation rows per CTA (multiple of 16, at most 256)
  int int4;               // 1: INT4 weights (A tile produced by the transform warps), 0: FP8
  int group;              // INT4 scale group along k
  int kb_per_split, n_kb; // k blocks (of 128 bytes of operand row) per k-slice / in total
  int ksplit, stages, raw_stages;
  int w_tiled;            // weights tiled by pt_gemm_repack (one contiguous tile per stage) instead of row-major
  int epilogue;           // PT_EPI_STORE, PT_EPI_RESIDUAL or PT_EPI_BIAS
  float out_scale;
  const unsigned char *w; // tiled weights (w_tiled)
  const __half *scales;   // INT4: [N][K / group]
  const __half *residual;
  const __half *bias;
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
#if PT_TC_HINT < 0
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
#else
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity), "r"((uint32_t)PT_TC_HINT)
                 : "memory");
#endif
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
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
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
  uint64_t raw_full[24], raw_empty[24];
  uint32_t tmem_base;
  volatile int abort;
  int last;
};

// What every role does when one of its waits runs out.
__device__ __forceinline__ void give_up(SharedCtl &ctl, int *error_flag, int code) {
  if (!ctl.abort && error_flag) atomicCAS(error_flag, 0, code);
  ctl.abort = 1;
}

// Epilogue of the warps that own the tile's rows (tensor-memory lane quarter warp % 4): `part` of `parts` warps share a quarter
// and take alternate 16-column chunks.
__device__ __forceinline__ void epilogue(const GemmParams &p, uint32_t tmem, int q, int lane, int part, int parts, int n0, int m0, int ks) {
  const int n = n0 + q * 32 + lane;
  for (int c0 = part * 16; c0 < p.mb; c0 += 16 * parts) {
    uint32_t v[16];
    float sum[16];
    tmem_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
    for (int j = 0; j < 16; ++j) sum[j] = __uint_as_float(v[j]);
    if (n < p.N) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int m = m0 + c0 + j;
        if (m >= p.M) break;
        const float acc = sum[j];
        if (p.ksplit > 1) {
          p.partial[((size_t)ks * p.M + m) * p.N + n] = acc;
        } else {
          __half y = __float2half_rn(acc * p.out_scale);
          if (p.epilogue == PT_EPI_RESIDUAL) y = h_add(__ldcg(p.residual + (size_t)m * p.N + n), y);
          else if (p.epilogue == PT_EPI_BIAS) y = h_add(y, p.bias[n]);
          p.out[(size_t)m * p.out_ld + n] = y;
        }
      }
    }
  }
}

// k-slices of this tile meet: the last CTA to arrive sums them in slice order.
__device__ __forceinline__ void reduce_slices(const GemmParams &p, SharedCtl &ctl, int n0, int m0, int threads) {
  const int tid = threadIdx.x;
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
    // every thread sums the slices of one output element at a time, all slices' loads in flight together (at most 8 per batch)
    const int rows = min(p.mb, p.M - m0);
    for (int i = tid; i < rows * BM; i += threads) {
      const int m = m0 + i / BM, n = n0 + (i % BM);
      if (n >= p.N) continue;
      float acc = 0.f;
      for (int s0 = 0; s0 < p.ksplit; s0 += 8) {
        float part[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) part[j] = (s0 + j < p.ksplit) ? __ldcg(p.partial + ((size_t)(s0 + j) * p.M + m) * p.N + n) : 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += part[j];
      }
      __half y = __float2half_rn(acc * p.out_scale);
      if (p.epilogue == PT_EPI_RESIDUAL) y = h_add(__ldcg(p.residual + (size_t)m * p.N + n), y);
      else if (p.epilogue == PT_EPI_BIAS) y = h_add(y, p.bias[n]);
      p.out[(size_t)m * p.out_ld + n] = y;
    }
  }
}

// ------------------------------------------------------------------------------------------ FP8
// Dynamic shared memory: [stage][A tile 16 KB | B tile mb * 128 B], every tile 1024-byte aligned.
__global__ void __launch_bounds__(THREADS_F8, 1) gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                                                 const GemmParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ SharedCtl ctl;
  unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BM, m0 = blockIdx.z * p.mb, ks = blockIdx.y;
  const int kb0 = ks * p.kb_per_split, kb1 = min(p.n_kb, kb0 + p.kb_per_split);
  const int n_it = kb1 - kb0;
  const uint32_t b_bytes = (uint32_t)p.mb * BKB;
  const uint32_t stage_bytes = A_TILE + ((b_bytes + 1023u) & ~1023u);
  const uint32_t smem_s = sa(smem);
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < p.mb) tmem_cols <<= 1;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(sa(&ctl.full[s]), 1);
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
    if (lane == 0) {
      // (ring positions and parities are carried as counters: this thread's instruction count per stage is what limits a CTA)
      const unsigned char *wt = p.w + ((size_t)blockIdx.x * p.n_kb + kb0) * A_TILE;
      const uint32_t tx = A_TILE + b_bytes, full0 = sa(&ctl.full[0]), empty0 = sa(&ctl.empty[0]);
      const bool tiled = p.w_tiled != 0;
      int s = 0, kx = kb0 * BKB;
      uint32_t par = 1;   // parity of the `empty` phase that must have completed before slot s is refilled (none in the first round)
      bool first_round = true;
      for (int it = 0; it < n_it; ++it) {
        if (!first_round && !mbar_wait(empty0 + s * 8, par, &ctl.abort)) give_up(ctl, p.error_flag, 21);
        if (ctl.abort) break;
        const uint32_t st = smem_s + s * stage_bytes, fb = full0 + s * 8;
        mbar_expect_tx(fb, tx);
        if (tiled) bulk_g2s(st, wt, A_TILE, fb);
        else tma_load_2d(st, &map_w, kx, n0, fb);
        tma_load_2d(st + A_TILE, &map_x, kx, m0, fb);
        wt += A_TILE;
        kx += BKB;
        if (++s == p.stages) { s = 0; par ^= 1u; first_round = false; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // One thread issues every MMA of the CTA, so its loop is kept to a few dozen instructions per stage: descriptors are one
      // 64-bit add away from the stage-0 descriptors (the start-address field counts 16-byte units), ring position and parity
      // are counters.  (Measured: with divisions and descriptor rebuilds in this loop a stage took 0.6 us whatever its size.)
      const uint32_t idesc = instr_desc(true, p.mb);
      const uint64_t adesc0 = smem_desc_sw128(smem_s), bdesc0 = smem_desc_sw128(smem_s + A_TILE);
      const uint32_t full0 = sa(&ctl.full[0]), empty0 = sa(&ctl.empty[0]), stage16 = stage_bytes >> 4;
      int s = 0;
      uint32_t par = 0, acc = 0;
      for (int it = 0; it < n_it; ++it) {
        if (!mbar_wait(full0 + s * 8, par, &ctl.abort)) give_up(ctl, p.error_flag, 22);
        if (ctl.abort) break;
        fence_after();
        const uint64_t adesc = adesc0 + (uint64_t)(s * stage16), bdesc = bdesc0 + (uint64_t)(s * stage16);
        umma<true>(tmem, adesc, bdesc, idesc, acc);   // four MMAs of 32 bytes of k each; inside the swizzle atom the start address moves by 32 bytes
        umma<true>(tmem, adesc + 2, bdesc + 2, idesc, 1u);
        umma<true>(tmem, adesc + 4, bdesc + 4, idesc, 1u);
        umma<true>(tmem, adesc + 6, bdesc + 6, idesc, 1u);
        umma_commit(empty0 + s * 8);
        acc = 1u;
        if (++s == p.stages) { s = 0; par ^= 1u; }
      }
      umma_commit(sa(&ctl.accum));   // fires when every MMA above has completed
    }
  } else {
    if (!mbar_wait(sa(&ctl.accum), 0, &ctl.abort)) give_up(ctl, p.error_flag, 24);
    fence_after();
    if (!ctl.abort && n_it > 0) epilogue(p, tmem, warp & 3, lane, 0, 1, n0, m0, ks);
    fence_before();
  }
  if (p.ksplit > 1) reduce_slices(p, ctl, n0, m0, THREADS_F8);
  __syncthreads();
  fence_after();
  if (warp == 1) tmem_dealloc(tmem, tmem_cols);
}

// ------------------------------------------------------------------------------------------ INT4
// Dynamic shared memory: [operand stage][A tile 16 KB | B tile mb * 128 B] then [raw stage][4 KB of packed nibbles].
// The raw ring is deep (it is what keeps HBM busy: up to 24 x 4 KB in flight per SM), the operand ring short.
__global__ void __launch_bounds__(THREADS_I4, 1) gemm_int4_kernel(const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ SharedCtl ctl;
  unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BM, m0 = blockIdx.z * p.mb, ks = blockIdx.y;
  const int kb0 = ks * p.kb_per_split, kb1 = min(p.n_kb, kb0 + p.kb_per_split);
  const int n_it = kb1 - kb0;
  const int S = p.stages, R = p.raw_stages;
  const uint32_t b_bytes = (uint32_t)p.mb * BKB;
  const uint32_t stage_bytes = A_TILE + ((b_bytes + 1023u) & ~1023u);
  unsigned char *raw_ring = smem + (size_t)S * stage_bytes;
  const uint32_t smem_s = sa(smem);
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < p.mb) tmem_cols <<= 1;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(sa(&ctl.full[s]), 1);    // the activation tile of the stage has landed
      mbar_init(sa(&ctl.ready[s]), 8);   // one arrival per transform warp: the fp16 weight tile is written
      mbar_init(sa(&ctl.empty[s]), 1);   // the MMAs that read the stage have completed
    }
    for (int r = 0; r < R; ++r) {
      mbar_init(sa(&ctl.raw_full[r]), 1);
      mbar_init(sa(&ctl.raw_empty[r]), 8);
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
    // ---- raw nibble tiles: one contiguous 4 KB bulk copy per k block
    if (lane == 0) {
      const unsigned char *wt = p.w + ((size_t)blockIdx.x * p.n_kb + kb0) * RAW_TILE;
      const uint32_t raw0 = sa(raw_ring), full0 = sa(&ctl.raw_full[0]), empty0 = sa(&ctl.raw_empty[0]);
      int r = 0;
      uint32_t par = 1;
      bool first_round = true;
      for (int it = 0; it < n_it; ++it) {
        if (!first_round && !mbar_wait(empty0 + r * 8, par, &ctl.abort)) give_up(ctl, p.error_flag, 21);
        if (ctl.abort) break;
        const uint32_t fb = full0 + r * 8;
        mbar_expect_tx(fb, RAW_TILE);
        bulk_g2s(raw0 + r * RAW_TILE, wt, RAW_TILE, fb);
        wt += RAW_TILE;
        if (++r == R) { r = 0; par ^= 1u; first_round = false; }
      }
    }
  } else if (warp == 10) {
    // ---- activation tiles (64 fp16 of k per row)
    if (lane == 0) {
      const uint32_t full0 = sa(&ctl.full[0]), empty0 = sa(&ctl.empty[0]);
      int s = 0, kx = kb0 * 64;
      uint32_t par = 1;
      bool first_round = true;
      for (int it = 0; it < n_it; ++it) {
        if (!first_round && !mbar_wait(empty0 + s * 8, par, &ctl.abort)) give_up(ctl, p.error_flag, 25);
        if (ctl.abort) break;
        const uint32_t fb = full0 + s * 8;
        mbar_expect_tx(fb, b_bytes);
        tma_load_2d(smem_s + s * stage_bytes + A_TILE, &map_x, kx, m0, fb);
        kx += 64;
        if (++s == S) { s = 0; par ^= 1u; first_round = false; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = instr_desc(false, p.mb);
      const uint64_t adesc0 = smem_desc_sw128(smem_s), bdesc0 = smem_desc_sw128(smem_s + A_TILE);
      const uint32_t ready0 = sa(&ctl.ready[0]), full0 = sa(&ctl.full[0]), empty0 = sa(&ctl.empty[0]), stage16 = stage_bytes >> 4;
      int s = 0;
      uint32_t par = 0, acc = 0;
      for (int it = 0; it < n_it; ++it) {
        if (!mbar_wait(ready0 + s * 8, par, &ctl.abort) || !mbar_wait(full0 + s * 8, par, &ctl.abort)) give_up(ctl, p.error_flag, 22);
        if (ctl.abort) break;
        fence_after();
        const uint64_t adesc = adesc0 + (uint64_t)(s * stage16), bdesc = bdesc0 + (uint64_t)(s * stage16);
        umma<false>(tmem, adesc, bdesc, idesc, acc);   // four MMAs of 16 k (32 bytes) each
        umma<false>(tmem, adesc + 2, bdesc + 2, idesc, 1u);
        umma<false>(tmem, adesc + 4, bdesc + 4, idesc, 1u);
        umma<false>(tmem, adesc + 6, bdesc + 6, idesc, 1u);
        umma_commit(empty0 + s * 8);
        acc = 1u;
        if (++s == S) { s = 0; par ^= 1u; }
      }
      umma_commit(sa(&ctl.accum));
    }
  } else {
    // ---- transform + epilogue: warps 2-9.  A warp reads tensor-memory lanes [32 (warp % 4), +32), so thread (warp, lane) owns row
    // 32 (warp % 4) + lane of the tile; the two warps of a row share its k (transform) and its activation columns (epilogue).
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    const int n = n0 + row;
    const int ngroups = p.K / p.group;
    const __half *srow = p.scales + (size_t)min(n, p.N - 1) * ngroups;
    __half sc_next = (n_it > 0) ? __ldg(srow + (kb0 * 64) / p.group) : __half(0);
    const __half2 offA = __float2half2_rn(1032.0f), offB = __float2half2_rn(72.0f);
    const uint32_t raw_full0 = sa(&ctl.raw_full[0]), raw_empty0 = sa(&ctl.raw_empty[0]), empty0 = sa(&ctl.empty[0]), ready0 = sa(&ctl.ready[0]);
    const unsigned char *raw_mine = raw_ring + row * 32 + half * 16;
    unsigned char *arow0 = smem + (row >> 3) * 1024 + (row & 7) * 128;
    // scale index of a k block: blocks of 64 k, groups of p.group k -> the index moves on every (group / 64) blocks
    const int blocks_per_group = p.group / 64;
    int gidx = (kb0 * 64) / p.group, gleft = blocks_per_group - (kb0 % blocks_per_group);
    int r = 0, s = 0;
    uint32_t rpar = 0, spar = 1;
    bool first_round = true;
    for (int it = 0; it < n_it; ++it) {
      const __half2 s2 = __half2half2(sc_next);
      if (--gleft == 0) { ++gidx; gleft = blocks_per_group; }
      if (it + 1 < n_it) sc_next = __ldg(srow + gidx);   // next block's scale: its latency hides behind this block
      if (!mbar_wait(raw_full0 + r * 8, rpar, &ctl.abort)) give_up(ctl, p.error_flag, 23);
      if (ctl.abort) break;
      const uint4 w4 = *reinterpret_cast<const uint4 *>(raw_mine + (size_t)r * RAW_TILE);
      const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
      __syncwarp();
      if (lane == 0) mbar_arrive(raw_empty0 + r * 8);   // the nibbles are in registers: the raw stage may be refilled
      if (!first_round && !mbar_wait(empty0 + s * 8, spar, &ctl.abort)) give_up(ctl, p.error_flag, 26);
      if (ctl.abort) break;
      unsigned char *arow = arow0 + (size_t)s * stage_bytes;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        // a word holds eight consecutive k as offset-binary nibbles u = q + 8: bits [0,4) k0, [16,20) k1, [4,8) k2, [20,24) k3, and the
        // same again one byte up for k4..k7.  (1024 + u) and (64 + u) are exact in fp16; subtracting the offsets is exact; the
        // product with the scale is the one fp16 rounding of the reference's Int4ToHalf.
        const int c = half * 4 + c4;
        const uint32_t w = words[c4], w8 = w >> 8;
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
      if (lane == 0) mbar_arrive(ready0 + s * 8);
      if (++r == R) { r = 0; rpar ^= 1u; }
      if (++s == S) { s = 0; spar ^= 1u; first_round = false; }
    }
    if (!mbar_wait(sa(&ctl.accum), 0, &ctl.abort)) give_up(ctl, p.error_flag, 24);
    fence_after();
    if (!ctl.abort && n_it > 0) epilogue(p, tmem, q, lane, half, 2, n0, m0, ks);
    fence_before();
  }
  if (p.ksplit > 1) reduce_slices(p, ctl, n0, m0, THREADS_I4);
  __syncthreads();
  fence_after();
  if (warp == 1) tmem_dealloc(tmem, tmem_cols);
}

// ------------------------------------------------------------------------------------------ load-time tiling
// FP8 bytes W[n, k] (k contiguous) -> tiles [n tile][k block of 128]: 16 KB each, the image of a 128 x 128-byte tile under the
// 128-byte swizzle (row r at (r / 8) * 1024 + (r % 8) * 128, its 16-byte chunk c at position c ^ (r % 8)); rows beyond n are zero.
__global__ void fp8_tile_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, int n, int k, int n_kb, size_t n_units) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_units; i += (size_t)gridDim.x * blockDim.x) {
    const int u = (int)(i % 1024);            // 16-byte unit inside the tile
    const size_t tile = i / 1024;
    const int kb = (int)(tile % n_kb), nt = (int)(tile / n_kb);
    const int grp = u >> 6, r8 = (u >> 3) & 7, pc = u & 7;   // destination: 8-row group, row in it, physical chunk
    const int row = nt * BM + grp * 8 + r8, c = pc ^ r8;
    dst[i] = row < n ? src[((size_t)row * k + (size_t)kb * 128) / 16 + c] : make_uint4(0, 0, 0, 0);
  }
}
// Reference int4 rows (int8 [n, k/2]: byte j = k 2j in the high nibble, k 2j+1 in the low, two's complement) -> tiles
// [n tile][k block of 64]: 4 KB each, [128 rows][32 bytes]; a word holds eight consecutive k as offset-binary nibbles in the order
// the transform warps split with two masks: bits [0,4) k0, [16,20) k1, [4,8) k2, [20,24) k3, [8,12) k4, [24,28) k5, [12,16) k6,
// [28,32) k7.  Rows beyond n hold q = 0.
__global__ void int4_tile_kernel(const uint32_t *__restrict__ src, uint32_t *__restrict__ dst, int n, int k, int n_kb, size_t n_words) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_words; i += (size_t)gridDim.x * blockDim.x) {
    const int wi = (int)(i % 1024);           // word inside the tile: row * 8 + word of the row
    const size_t tile = i / 1024;
    const int kb = (int)(tile % n_kb), nt = (int)(tile / n_kb);
    const int row = nt * BM + (wi >> 3), w = wi & 7;
    uint32_t o = 0x88888888u;
    if (row < n) {
      const uint32_t b = src[((size_t)row * (k / 2) + (size_t)kb * 32) / 4 + w];   // four bytes = k 0..7 of this word
      o = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t byte = (b >> (8 * j)) & 0xFFu;
        const uint32_t even = ((byte >> 4) ^ 8u) & 0xFu, odd = (byte ^ 8u) & 0xFu;   // k = 2j, 2j + 1
        o |= even << (4 * j);
        o |= odd << (16 + 4 * j);
      }
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

extern "C" size_t pt_gemm_packed_bytes(int wfmt, int n_out, int k_in) {
  const size_t rows = (size_t)ceil_div(n_out, tc::BM) * tc::BM;
  return wfmt == PT_W_INT4 ? rows * (size_t)(k_in / 2) : rows * (size_t)k_in;
}

extern "C" int pt_gemm_repack(int wfmt, const void *w, int n_out, int k_in, void *packed, void *stream) {
  PT_REQUIRE(wfmt == PT_W_INT4 || wfmt == PT_W_FP8, "pt_gemm_repack: weight format %d (INT4 or FP8)", wfmt);
  PT_REQUIRE(w && packed && w != packed, "pt_gemm_repack: needs distinct source and destination buffers");
  PT_REQUIRE(((uintptr_t)w & 15) == 0 && ((uintptr_t)packed & 15) == 0, "pt_gemm_repack: buffers must be 16-byte aligned");
  PT_REQUIRE(n_out > 0 && k_in > 0 && k_in % 128 == 0, "pt_gemm_repack: k_in=%d must be a positive multiple of 128", k_in);
  const int n_tiles = ceil_div(n_out, tc::BM);
  if (wfmt == PT_W_INT4) {
    const int n_kb = k_in / 64;
    const size_t n_words = (size_t)n_tiles * n_kb * 1024;
    tc::int4_tile_kernel<<<sm_count() * 8, 256, 0, as_stream(stream)>>>((const uint32_t *)w, (uint32_t *)packed, n_out, k_in, n_kb, n_words);
  } else {
    const int n_kb = k_in / 128;
    const size_t n_units = (size_t)n_tiles * n_kb * 1024;
    tc::fp8_tile_kernel<<<sm_count() * 8, 256, 0, as_stream(stream)>>>((const uint4 *)w, (uint4 *)packed, n_out, k_in, n_kb, n_units);
  }
  PT_LAUNCH_CHECK("pt_gemm_repack");
  return PT_OK;
}

// k-slice workspace layout: [arrival counters, kGemmCounterBytes][partial sums].  The counter region has ONE size for every
// shape, so that GEMMs of different widths can share a workspace: with a shape-dependent offset the partial sums of a narrow
// GEMM (o_proj) would land where a wide one (q|k|v) expects zeroed counters.  16384 counters: one per (128-row weight tile,
// block of activation rows); a shape with more tiles than that runs without k-slices when the split is automatic.
constexpr size_t kGemmCounterBytes = 65536;
constexpr size_t kGemmMaxCounters = kGemmCounterBytes / sizeof(int);

extern "C" size_t pt_gemm_workspace_bytes(int m, int n_out, int max_ksplit) {
  return kGemmCounterBytes + (size_t)max_ksplit * m * n_out * sizeof(float);
}

extern "C" int pt_gemm(const pt_gemm_args *a, void *stream) {
  PT_REQUIRE(a, "pt_gemm: null args");
  PT_REQUIRE(a->wfmt == PT_W_INT4 || a->wfmt == PT_W_FP8, "pt_gemm: weight format %d (INT4 or FP8)", a->wfmt);
  const bool int4 = a->wfmt == PT_W_INT4;
  PT_REQUIRE(a->m >= 1 && a->n_out >= 1 && a->k_in >= 128 && a->k_in % 128 == 0, "pt_gemm: bad shape m=%d n_out=%d k_in=%d (k_in a multiple of 128)",
             a->m, a->n_out, a->k_in);
  PT_REQUIRE(a->x && a->w && a->out, "pt_gemm: null x / w / out");
  PT_REQUIRE(((uintptr_t)a->x & 15) == 0 && ((uintptr_t)a->w & 15) == 0, "pt_gemm: x and w must be 16-byte aligned");
  PT_REQUIRE(a->epilogue == PT_EPI_STORE || a->epilogue == PT_EPI_RESIDUAL || a->epilogue == PT_EPI_BIAS, "pt_gemm: epilogue %d (store, residual or bias)",
             a->epilogue);
  PT_REQUIRE(a->epilogue != PT_EPI_RESIDUAL || a->residual, "pt_gemm: residual epilogue needs residual");
  PT_REQUIRE(a->epilogue != PT_EPI_BIAS || a->bias, "pt_gemm: bias epilogue needs bias");
  PT_REQUIRE(!int4 || a->w_tiled, "pt_gemm: INT4 weights must be tiled with pt_gemm_repack");
  if (int4)
    PT_REQUIRE(a->scales && a->group >= 128 && a->group % 128 == 0 && a->k_in % a->group == 0,
               "pt_gemm: INT4 needs scales and a group (%d) that is a multiple of 128 dividing k_in=%d", a->group, a->k_in);

  tc::GemmParams p{};
  p.M = a->m; p.N = a->n_out; p.K = a->k_in;
  p.int4 = int4 ? 1 : 0;
  p.group = int4 ? a->group : 0;
  p.w_tiled = a->w_tiled ? 1 : 0;
  p.w = (const unsigned char *)a->w;
  p.mb = std::min(256, ceil_div(a->m, 16) * 16);
  const int m_tiles = ceil_div(a->m, p.mb);
  const int n_tiles = ceil_div(a->n_out, tc::BM);
  p.n_kb = int4 ? a->k_in / 64 : a->k_in / 128;
  // k-slices: fill the GPU when there are few tiles, but keep at least PT_TC_MIN_KB k-blocks per CTA
#ifndef PT_TC_MIN_KB
#define PT_TC_MIN_KB 8
#endif
  int ksplit = a->ksplit;
  if (ksplit <= 0) {
    ksplit = std::max(1, (p.mb <= 64 ? 2 : 1) * sm_count() / (n_tiles * m_tiles));   // two CTAs fit an SM up to 64 activation rows
    ksplit = std::max(1, std::min(ksplit, p.n_kb / PT_TC_MIN_KB));
    ksplit = std::min(ksplit, 8);                                           // what pt_gemm_workspace_bytes is usually asked for ...
    while (ksplit > 1 && pt_gemm_workspace_bytes(a->m, a->n_out, ksplit) > a->workspace_bytes) --ksplit;   // ... and never more than the caller's workspace holds
    if ((size_t)n_tiles * m_tiles > kGemmMaxCounters) ksplit = 1;
  }
  ksplit = std::max(1, std::min(ksplit, p.n_kb));
  p.kb_per_split = ceil_div(p.n_kb, ksplit);
  p.ksplit = ceil_div(p.n_kb, p.kb_per_split);
  p.epilogue = a->epilogue;
  p.out_scale = int4 ? 1.0f : (a->x_scale > 0.f ? a->x_scale : 1.0f) * (a->w_scale > 0.f ? a->w_scale : 1.0f);
  p.scales = (const __half *)a->scales;
  p.residual = (const __half *)a->residual;
  p.bias = (const __half *)a->bias;
  p.out = (__half *)a->out;
  p.out_ld = a->out_ld > 0 ? a->out_ld : a->n_out;
  p.error_flag = a->error_flag;
  if (p.ksplit > 1) {
    const size_t need = pt_gemm_workspace_bytes(a->m, a->n_out, p.ksplit);
    PT_REQUIRE(a->workspace && a->workspace_bytes >= need, "pt_gemm: %d k-slices need %zu workspace bytes, got %zu", p.ksplit, need, a->workspace_bytes);
    PT_REQUIRE((size_t)n_tiles * m_tiles <= kGemmMaxCounters, "pt_gemm: %d x %d tiles exceed the %zu arrival counters of a k-slice workspace", n_tiles,
               m_tiles, kGemmMaxCounters);
    p.counters = (int *)a->workspace;
    p.partial = (float *)((char *)a->workspace + kGemmCounterBytes);
  }

  const uint32_t b_bytes = (uint32_t)p.mb * tc::BKB;
  const uint32_t stage_bytes = tc::A_TILE + ((b_bytes + 1023u) & ~1023u);
  // Up to 64 activation rows a stage is small, and what limits the kernel is the one thread per CTA that issues the MMAs (about
  // 75 cycles per tcgen05.mma whatever its N): two CTAs per SM (half the shared memory each) issue side by side.  Measured on
  // B200, FP8 65024 x 4096 at 8 / 32 rows: 63 / 66 us with one CTA per SM, 45 / 47 us with two.
#ifndef PT_TC_BUDGET_SMALL_KB
#define PT_TC_BUDGET_SMALL_KB 100
#endif
  const bool small = p.mb <= 64;
  const uint32_t budget = (small ? PT_TC_BUDGET_SMALL_KB : 200) * 1024u;
  size_t smem;
  if (int4) {
    p.stages = (int)std::min<uint32_t>(4, (budget - 8 * tc::RAW_TILE) / stage_bytes);
    PT_REQUIRE(p.stages >= 2, "pt_gemm: tile does not fit shared memory");
    p.raw_stages = (int)std::min<uint32_t>(24, (budget - p.stages * stage_bytes) / tc::RAW_TILE);
    smem = (size_t)p.stages * stage_bytes + (size_t)p.raw_stages * tc::RAW_TILE + 1024;
  } else {
    p.stages = (int)std::min<uint32_t>(8, budget / stage_bytes);
    PT_REQUIRE(p.stages >= 2, "pt_gemm: tile does not fit shared memory");
    smem = (size_t)p.stages * stage_bytes + 1024;
  }

  CUtensorMap map_w, map_x;
  memset(&map_w, 0, sizeof(map_w));
  if (int4) {
    if (int rc = tc::make_map(&map_x, a->x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)a->k_in, (uint64_t)a->m, 64, (uint32_t)p.mb, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  } else {
    if (!p.w_tiled)
      if (int rc = tc::make_map(&map_w, a->w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a->k_in, (uint64_t)a->n_out, 128, tc::BM, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    if (int rc = tc::make_map(&map_x, a->x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a->k_in, (uint64_t)a->m, 128, (uint32_t)p.mb, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  }
  static bool attr_set = false;
  if (!attr_set) {
    PT_CUDA(cudaFuncSetAttribute(tc::gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    PT_CUDA(cudaFuncSetAttribute(tc::gemm_int4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_set = true;
  }
  dim3 grid(n_tiles, p.ksplit, m_tiles);
  if (int4)
    tc::gemm_int4_kernel<<<grid, tc::THREADS_I4, smem, as_stream(stream)>>>(map_x, p);
  else
    tc::gemm_fp8_kernel<<<grid, tc::THREADS_F8, smem, as_stream(stream)>>>(map_w, map_x, p);
  PT_LAUNCH_CHECK("pt_gemm");
  return PT_OK;
}
