// Persistent decode-step kernel for the Llama architecture (INT4 transformer linears, fp16 LM head, batch <= 2).
//
// One block per SM, launched cooperatively, executes a whole loop iteration of the reference's decode graph
// (poptransformer/models/llama2/model.py:162-197 and models/base_model.py:313-355): embedding, 32 x
// [RMSNorm + QKV, RoPE + KV append + attention, o_proj + residual, RMSNorm + gate|up + SwiGLU, down_proj + residual],
// final RMSNorm + LM head + arg-max, and the loop-carry update.
//
// Why one kernel: at batch 1 a layer streams ~110 MB in ~17 us, so per-kernel launch, prologue and tail
// latencies (several microseconds each, five kernels per layer) cost more than the data movement.  Here
//   * warp 16 is a producer: it walks this SM's share of every weight matrix of the whole step, in order, and
//     keeps a ring of 16.5 KB shared-memory stages full with 1-D bulk async copies (TMA engine, one mbarrier
//     per stage).  Weights do not depend on activations, so the producer runs ahead across the grid-wide
//     barriers and HBM stays busy while the consumers wait for each other;
//   * warps 0-15 are consumers: consumer w takes tile w of every stage (a stage = 16 consecutive [row tile][chunk]
//     tiles of the packed layout of linear.cu), does the same nibble -> fp16 -> mma arithmetic as the streaming
//     linear kernel, and the 16 partial sums of a row tile meet in shared memory in warp order (deterministic);
//   * K/V pages travel through the same ring; the attention arithmetic is that of attention.cu;
//   * phases are separated by a grid barrier (one atomic per block, bounded spin, error flag on time-out).
// Every SM owns whole row tiles: rows [s * n_rt / G, (s + 1) * n_rt / G).
#include <algorithm>

#include "tile_math.cuh"

namespace pt {
namespace mk {

#ifndef PT_MK_WARPS
#define PT_MK_WARPS 16
#endif
constexpr int NCW = PT_MK_WARPS;        // consumer warps
constexpr int NCT = NCW * 32;           // consumer threads
constexpr int THREADS = NCT + 32;       // + the producer warp
constexpr int NGRP = NCW / 4;           // 4-warp attention groups
constexpr int TILE_I4 = 1056, TILE_F16 = 1024;
constexpr int STAGE_TILES = NCW;                  // one tile per consumer warp per stage
constexpr int STAGE_BYTES = ((STAGE_TILES * TILE_I4 + 127) / 128 * 128) > 33792 ? ((STAGE_TILES * TILE_I4 + 127) / 128 * 128) : 33792;
constexpr int V_OFFSET = 16896;                   // a K page and a V page (2 x 16 KB) share one attention stage
constexpr int MAXU = 8;                           // attention units handled per SM per pass
constexpr int BMAX = 2;
constexpr int H = 128, PAGE = 64;
constexpr int SPIN_LIMIT = 1 << 22;

struct Params {
  int B, d, n_head, ffn, vocab, n_layer, max_len, max_pages, ns, xs_stride, pad_id, eos_id, debug;
  float eps;
  __half score_scale;
  const pt_llama_layer *layers;
  const __half *norm, *emb, *sin_t, *cos_t;
  const unsigned char *head;
  int *ids, *step, *stop_mask, *next_ids;
  const int *page_table;
  __half *x, *qkv, *attn, *act, *logits;
  float *ws_o;        // [B, n_head, max_pages, H]
  float2 *ws_ml;      // [B, n_head, max_pages]
  int *attn_counters; // [B, n_head]
  float *cand_val;    // [B, grid]
  int *cand_idx;
  unsigned *barrier;  // [0], [1]: counters used by alternate launches; [2]: which one the next launch uses
  int *error_flag;
  unsigned long long *trace;  // optional: [grid][n_layer][12] global-timer stamps of the phase boundaries
};

// ------------------------------------------------------------------------------------------ small helpers
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
               "r"(bar)
               : "memory");
}
// Bounded wait.  Each try_wait carries a suspend-time hint, so a waiting warp sleeps in hardware instead of burning issue
// slots that the working warps (and the producer) need.  The wait gives up early when the block has already recorded a
// failure, so that after an error every loop of the kernel still runs its normal trip count (all named barriers stay
// matched) but finishes quickly.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const volatile int *abort_flag) {
  for (int it = 0; it < (1 << 18); ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity), "r"(2000u)
                 : "memory");
    if (ok) return true;
    if ((it & 7) == 7 && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NCT) : "memory"); }

struct Shared {           // fixed-size part, placed after the ring / activations
  float red[NCW][2][32][4];  // per warp: partial sums of the first / last row tile of its tile range
  float corr[96][8];      // [chunk][batch column], up to 96 chunks of 128 k
  __half qs[MAXU][H], newk[MAXU][H], newv[MAXU][H];
  float ps[NGRP][PAGE];   // one row per 4-warp attention group
  float ml[NGRP][2];
  int last[MAXU];
  float stat[BMAX];
  float wred[32];
  float bestv[32][BMAX];
  int besti[32][BMAX];
  volatile int abort;
  uint64_t full[16], empty[16];
};

struct Ctx {
  const Params &p;
  unsigned char *ring, *xs;
  Shared *sh;
  int sm, G, step;
  unsigned *bar_ctr;
  unsigned bar_target;
  uint32_t gs;  // global stage counter (same sequence in producer and consumers)
  unsigned long long *tr;  // optional fine-grained stamps of the current layer
};

// Grid barrier over all blocks (consumer threads only).  Bounded: on time-out the error flag is set and the block
// stops doing work (every later wait is bounded too), so the kernel always terminates.
__device__ void grid_sync(Ctx &c) {
  const int tid = threadIdx.x;
  c.bar_target += c.G;
  consumer_sync();
  if (tid == 0) {
    __threadfence();
    atomicAdd(c.bar_ctr, 1u);
    bool ok = false;
    for (int it = 0; it < SPIN_LIMIT; ++it) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(c.bar_ctr) : "memory");
      if (v >= c.bar_target) { ok = true; break; }
      if (c.sh->abort) break;
    }
    if (!ok) {
      c.sh->abort = 1;
      if (c.p.error_flag) atomicExch(c.p.error_flag, 3);
    }
  }
  consumer_sync();
}

__device__ __forceinline__ float consumer_sum(Ctx &c, float v) {  // sum over the 512 consumer threads, fixed order
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  consumer_sync();
  if (lane == 0) c.sh->wred[warp] = v;
  consumer_sync();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < NCW; ++i) t += c.sh->wred[i];
  return t;
}

// RMSNorm weights of the next phase, requested before the grid barrier so that their (HBM) latency hides behind it.
struct Gamma { uint4 v[3]; };
__device__ __forceinline__ Gamma load_gamma(const __half *gamma, int K) {
  Gamma g;
#pragma unroll
  for (int q = 0; q < 3; ++q)
    g.v[q] = (gamma && (int)threadIdx.x + q * NCT < K / 8) ? __ldg(reinterpret_cast<const uint4 *>(gamma) + threadIdx.x + q * NCT) : make_uint4(0, 0, 0, 0);
  return g;
}

// Stage activations src[B, K] (global, written by other SMs: read through L2) into shared memory for the next linear phase.
// INT4 phases use the per-chunk swizzle of linear.cu ([chunk][w][tig] 16-byte units) and produce the offset corrections;
// the fp16 phase (LM head) keeps the natural order.  gamma != nullptr applies RMSNorm first (weights in `gm`).
template <bool INT4>
__device__ void stage_x(Ctx &c, const __half *src, int K, const __half *gamma, const Gamma &gm) {
  const Params &p = c.p;
  const int tid = threadIdx.x;
  const int units = K / 8;
  for (int b = 0; b < p.B; ++b) {
    uint4 v[3];
    const uint4 *xr = reinterpret_cast<const uint4 *>(src + (size_t)b * K);
#pragma unroll
    for (int q = 0; q < 3; ++q) v[q] = (tid + q * NCT < units) ? __ldcg(xr + tid + q * NCT) : make_uint4(0, 0, 0, 0);
    __half rb = __half(0);
    if (c.tr && tid == 0 && b == 0) { c.tr[13] = gtime(); c.tr[14] = (unsigned long long)(v[0].x); c.tr[14] = gtime(); }
    if (gamma) {
      float ss = 0.f;
#pragma unroll
      for (int q = 0; q < 3; ++q) {
        const __half2 *h = reinterpret_cast<const __half2 *>(&v[q]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __half22float2(h[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
      ss = consumer_sum(c, ss);
      rb = __float2half_rn(1.0f / sqrtf(ss / (float)K + p.eps));
      if (c.tr && tid == 0 && b == 0) c.tr[15] = gtime();
    }
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const int u = tid + q * NCT;
      const bool valid = u < units;
      __half *h = reinterpret_cast<__half *>(&v[q]);
      if (gamma && valid) {
        const __half *gh = reinterpret_cast<const __half *>(&gm.v[q]);
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = h_mul(h_mul(h[j], rb), gh[j]);
      }
      if (INT4) {
        // units of one 128-k chunk are 16 consecutive u, i.e. 16 consecutive lanes
        float sa = 0.f, sb = 0.f;
        if (valid) {
          sa = (__half2float(h[0]) + __half2float(h[1])) + (__half2float(h[4]) + __half2float(h[5]));
          sb = (__half2float(h[2]) + __half2float(h[3])) + (__half2float(h[6]) + __half2float(h[7]));
        }
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) {
          sa += __shfl_xor_sync(0xffffffffu, sa, o);
          sb += __shfl_xor_sync(0xffffffffu, sb, o);
        }
        if (valid) {
          const int chunk = u >> 4, r = u & 15, t4 = r >> 2, w = r & 3;
          *reinterpret_cast<uint4 *>(c.xs + (size_t)b * p.xs_stride + chunk * 256 + w * 64 + t4 * 16) = v[q];
          if (r == 0) c.sh->corr[chunk][b] = kOffA * sa + kOffB * sb;
        }
      } else if (valid) {
        *reinterpret_cast<uint4 *>(c.xs + (size_t)b * p.xs_stride + u * 16) = v[q];
      }
    }
  }
  consumer_sync();
}

// Epilogue kinds of the linear phases
enum { EPI_QKV = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_HEAD = 3 };

struct Best { float v[BMAX]; int i[BMAX]; };

// How the T tiles of an SM's share of a matrix (its row tiles, [row tile][chunk] order) are dealt to the consumer warps:
// warp w owns the contiguous range [start(w), start(w) + len(w)), ranges differ by at most one tile.
struct Split {
  int base, rem;
  __device__ __forceinline__ Split(int T) : base(T / NCW), rem(T % NCW) {}
  __device__ __forceinline__ int len(int w) const { return base + (w < rem ? 1 : 0); }
  __device__ __forceinline__ int start(int w) const { return w * base + min(w, rem); }
  __device__ __forceinline__ int owner(int q) const {  // warp whose range holds tile q
    const int big = rem * (base + 1);
    if (q < big) return q / (base + 1);
    return base > 0 ? rem + (q - big) / base : NCW - 1;
  }
  __device__ __forceinline__ int stages() const { return base + (rem ? 1 : 0); }
};

template <int EPI>
__device__ __forceinline__ void tile_epilogue(const Params &p, const float (&v)[4], int rt, int lane, __half *out, int N, Best *best) {
  const int g = lane >> 2, tig = lane & 3;
  if (tig != 0) return;  // batch columns 0 and 1 live in the tig == 0 lanes
#pragma unroll
  for (int jb = 0; jb < 2; ++jb) {
    const int b = jb;
    if (b >= p.B) continue;
    const float lo = v[jb], hi = v[2 + jb];  // rows g and g + 8
    if (EPI == EPI_SWIGLU) {
      const int n = rt * 8 + g;
      if (n < N / 2) out[(size_t)b * (N / 2) + n] = h_mul(__float2half_rn(hi), swish_h(__float2half_rn(lo)));
    } else {
#pragma unroll
      for (int hr = 0; hr < 2; ++hr) {
        const int n = rt * 16 + g + 8 * hr;
        if (n >= N) continue;
        __half y = __float2half_rn(hr ? hi : lo);
        if (EPI == EPI_RESID) y = h_add(__ldcg(out + (size_t)b * N + n), y);
        if (EPI == EPI_HEAD) {
          const float f = __half2float(y);
          if (f > best->v[b] || (f == best->v[b] && n < best->i[b])) { best->v[b] = f; best->i[b] = n; }
          if (out) out[(size_t)b * N + n] = y;
        } else {
          out[(size_t)b * N + n] = y;
        }
      }
    }
  }
}

// One linear phase over this SM's row tiles [r0, r1) of a matrix with `nchunks` tiles per row tile.  The SM's tiles arrive
// in "stream order": stage j holds tile start(w) + j of every warp w that still has one (see pt_llama_stream_permute), so
// each warp accumulates a contiguous run of chunks in registers and there is no synchronisation inside the phase.  Row
// tiles that are split between warps are summed after one barrier, in warp order (deterministic).
template <int WFMT, int EPI>
__device__ void linear_phase(Ctx &c, int n_rt, int nchunks, __half *out, int N, Best *best) {
  constexpr int TILE = WTraits<WFMT>::kTileBytes;
  constexpr int UNITS = WTraits<WFMT>::kUnits;
  constexpr int CHUNK_X_BYTES = WTraits<WFMT>::kChunkK * 2;
  const Params &p = c.p;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tig = lane & 3;
  const int r0 = (int)((long long)c.sm * n_rt / c.G), r1 = (int)((long long)(c.sm + 1) * n_rt / c.G);
  const int m = r1 - r0, total = m * nchunks;
  const Split sp(total);
  const int len = sp.len(warp), start = sp.start(warp), nstages = sp.stages();
  const int first_rt = start / nchunks;
  int rt = first_rt, ch = start - first_rt * nchunks;
  const int ch_first = ch;  // chunk at which this warp enters its first row tile
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t ring_s = smem_addr(c.ring) + warp * TILE + lane * 16;
  const uint32_t xs_s = smem_addr(c.xs) + tig * 16 + g * p.xs_stride;
  const uint32_t corr_s = smem_addr(&c.sh->corr[0][0]) + 8 * tig;

  auto store_partial = [&](int slot) {
    *reinterpret_cast<float4 *>(&c.sh->red[warp][slot][lane][0]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  };

  // Software pipeline: the tile of stage j + 1 is pulled into registers (and its stage released to the producer) before
  // the tile of stage j is multiplied, so the registers act as one more ring stage and refills start earlier.
  uint4 va = make_uint4(0, 0, 0, 0), vb = va, na = va, nb = va;
  float2 sf = make_float2(1.f, 1.f), nsf = sf;
  auto fetch = [&](int j, uint4 &a4, uint4 &b4, float2 &s2) {  // stage j of this phase (global stage c.gs) -> registers
    const int slot = c.gs % p.ns;
    const bool got = mbar_wait(smem_addr(&c.sh->full[slot]), (c.gs / p.ns) & 1, &c.sh->abort);
    if (!got) {
      c.sh->abort = 1;
      if (lane == 0 && p.error_flag) atomicExch(p.error_flag, 4);
    }
    if (j < len && got) {
      const uint32_t t_s = ring_s + slot * STAGE_BYTES;
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a4.x), "=r"(a4.y), "=r"(a4.z), "=r"(a4.w) : "r"(t_s));
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b4.x), "=r"(b4.y), "=r"(b4.z), "=r"(b4.w) : "r"(t_s + 512));
      if (WFMT == PT_W_INT4) {
        uint32_t sraw;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sraw) : "r"(t_s - lane * 16 + 1024 + g * 4));
        s2 = __half22float2(*reinterpret_cast<__half2 *>(&sraw));
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_addr(&c.sh->empty[slot]));  // this warp's tile is in registers
    ++c.gs;
  };
  if (nstages > 0) fetch(0, va, vb, sf);
  for (int j = 0; j < nstages; ++j) {
    if (j + 1 < nstages) fetch(j + 1, na, nb, nsf);
    if (j < len && !(p.debug & 1)) {
      float cc[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t x_s = xs_s + ch * CHUNK_X_BYTES;
#pragma unroll
      for (int u = 0; u < UNITS; ++u) {
        uint32_t fa[4], fb[4];
        expand8<WFMT>(va, u, fa);
        expand8<WFMT>(vb, u, fb);
        uint4 xv = make_uint4(0, 0, 0, 0);
        if (g < p.B) asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(xv.x), "=r"(xv.y), "=r"(xv.z), "=r"(xv.w) : "r"(x_s + u * 64));
        mma16816(cc, fa[0], fb[0], fa[1], fb[1], xv.x, xv.y);
        mma16816(cc, fa[2], fb[2], fa[3], fb[3], xv.z, xv.w);
      }
      if (WFMT == PT_W_INT4) {
        float2 co;
        asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(co.x), "=f"(co.y) : "r"(corr_s + ch * 32));
        acc[0] += sf.x * (cc[0] - co.x);
        acc[1] += sf.x * (cc[1] - co.y);
        acc[2] += sf.y * (cc[2] - co.x);
        acc[3] += sf.y * (cc[3] - co.y);
      } else {
        acc[0] += cc[0]; acc[1] += cc[1]; acc[2] += cc[2]; acc[3] += cc[3];
      }
      if (++ch == nchunks) {  // this warp reached the end of row tile rt
        if (rt == first_rt && ch_first != 0) store_partial(0);                  // entered it midway: another warp holds the beginning
        else tile_epilogue<EPI>(p, acc, r0 + rt, lane, out, N, best);           // had all of it
        ch = 0;
        ++rt;
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      }
    }
    va = na; vb = nb; sf = nsf;
  }
  if (len > 0 && ch != 0) store_partial(rt == first_rt ? 0 : 1);  // the range ended inside a row tile
  consumer_sync();
  // ---- row tiles shared by several warps: warp (r % NCW) sums the pieces in warp order
  for (int r = warp; r < m; r += NCW) {
    const int q0 = r * nchunks, q1 = q0 + nchunks - 1;
    const int w_lo = sp.owner(q0), w_hi = sp.owner(q1);
    if (w_lo == w_hi) continue;  // one warp had the whole row tile and already wrote it
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int w = w_lo; w <= w_hi; ++w) {
      const int s_w = (sp.start(w) / nchunks == r) ? 0 : 1;  // r is the first row tile of w's range, or its last
      const float4 t = *reinterpret_cast<const float4 *>(&c.sh->red[w][s_w][lane][0]);
      v[0] += t.x; v[1] += t.y; v[2] += t.z; v[3] += t.w;
    }
    tile_epilogue<EPI>(p, v, r0 + r, lane, out, N, best);
  }
}

// RoPE (rotate_half form) on one head vector in global memory -> dst (shared), reference fp16 roundings.
__device__ __forceinline__ void rope_pair(const __half *x, const __half *sin_r, const __half *cos_r, int i, __half *dst) {
  const __half a = __ldcg(x + i), b = __ldcg(x + i + H / 2), s = sin_r[i], co = cos_r[i];
  dst[i] = h_add(h_mul(a, co), h_mul(__hneg(b), s));
  dst[i + H / 2] = h_add(h_mul(b, co), h_mul(a, s));
}
__device__ __forceinline__ void group_sync(int grp) { asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory"); }

// Attention phase.  Units (b, head, page) are dealt round-robin to the SMs (unit u -> SM u % G); the producer has queued
// one stage per unit that has cached tokens (K page at offset 0, V page at V_OFFSET).  The consumer warps form NGRP
// groups of four warps; group q handles this SM's units q, q + NGRP, ... on its own (scores with 8 lanes per token, softmax
// statistics by warp shuffles, P.V with one thread per channel), so units of an SM run concurrently.
__device__ void attention_phase(Ctx &c, const pt_llama_layer &L) {
  const Params &p = c.p;
  Shared *sh = c.sh;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gt = tid & 127;
  const int grp = (warp >> 2) < NGRP ? (warp >> 2) : -1;  // warps beyond the last full group only release stages
  const int step = c.step, n_active = step / PAGE + 1;
  const int n_units = p.B * p.n_head * n_active;
  const int row_elems = 3 * p.d;
  const __half *sin_r = p.sin_t + (size_t)step * (H / 2), *cos_r = p.cos_t + (size_t)step * (H / 2);
  for (int u0 = c.sm; u0 < n_units; u0 += MAXU * c.G) {
    const int nu = min(MAXU, (n_units - u0 + c.G - 1) / c.G);  // units of this pass: u0 + k G
    // ---- q (and the new token's k, v) of every unit in one go: one L2 round trip for the whole pass
    {
      const int k = tid >> 6, i = tid & 63;
      if (k < nu) {
        const int u = u0 + k * c.G;
        const int pg = u % n_active, head = (u / n_active) % p.n_head, b = u / (n_active * p.n_head);
        const __half *qrow = p.qkv + (size_t)b * row_elems;
        rope_pair(qrow + (size_t)head * H, sin_r, cos_r, i, sh->qs[k]);
        if (pg == n_active - 1) {
          rope_pair(qrow + p.d + (size_t)head * H, sin_r, cos_r, i, sh->newk[k]);
          sh->newv[k][i] = __ldcg(qrow + 2 * p.d + (size_t)head * H + i);
          sh->newv[k][i + 64] = __ldcg(qrow + 2 * p.d + (size_t)head * H + i + 64);
        }
      }
    }
    consumer_sync();
    // stage index of each unit of the pass (units without cached tokens have none)
    uint32_t gs_unit[MAXU];
    {
      uint32_t g0 = c.gs;
      for (int k = 0; k < nu; ++k) {
        const int u = u0 + k * c.G;
        const int pg = u % n_active;
        const int n_valid = min(PAGE, step + 1 - pg * PAGE);
        const int n_load = (pg == n_active - 1) ? n_valid - 1 : n_valid;
        gs_unit[k] = g0;
        if (n_load > 0) ++g0;
      }
      c.gs = g0;
    }
    for (int k = 0; k < nu; ++k) {
      const int u = u0 + k * c.G;
      const int pg = u % n_active, head = (u / n_active) % p.n_head, b = u / (n_active * p.n_head);
      const int n_valid = min(PAGE, step + 1 - pg * PAGE);
      const bool owner = (pg == n_active - 1);
      const int n_load = owner ? n_valid - 1 : n_valid;
      const int slot = gs_unit[k] % p.ns;
      if ((k % NGRP) != grp) {  // not this group's unit: release the stage at once
        if (n_load > 0 && lane == 0) {
          // the arrival only counts once the stage is full, so wait for it first (keeps phases aligned)
          mbar_wait(smem_addr(&sh->full[slot]), (gs_unit[k] / p.ns) & 1, &sh->abort);
          mbar_arrive(smem_addr(&sh->empty[slot]));
        }
        continue;
      }
      const __half *Ks = nullptr, *Vs = nullptr;
      if (n_load > 0) {
        if (!mbar_wait(smem_addr(&sh->full[slot]), (gs_unit[k] / p.ns) & 1, &sh->abort)) {
          sh->abort = 1;
          if (lane == 0 && p.error_flag) atomicExch(p.error_flag, 5);
        }
        Ks = reinterpret_cast<const __half *>(c.ring + (size_t)slot * STAGE_BYTES);
        Vs = reinterpret_cast<const __half *>(c.ring + (size_t)slot * STAGE_BYTES + V_OFFSET);
      }
      if (owner && !sh->abort) {  // append the new token to the pool
        const int phys = p.page_table[(size_t)b * p.max_pages + pg];
        __half *gK = (__half *)L.pool + (((size_t)phys * 2 + 0) * p.n_head + head) * PAGE * H + (size_t)(n_valid - 1) * H;
        __half *gV = (__half *)L.pool + (((size_t)phys * 2 + 1) * p.n_head + head) * PAGE * H + (size_t)(n_valid - 1) * H;
        gK[gt] = sh->newk[k][gt];
        gV[gt] = sh->newv[k][gt];
      }
      // scores: 8 lanes per cached token, 16 tokens per pass of the 128-thread group
      float *ps = sh->ps[grp];
      {
        const int sub = lane & 7;
        for (int tb = 0; tb < n_valid; tb += 16) {
          const int t = tb + (gt >> 3);
          float sc = 0.f;
          if (t < n_valid && !sh->abort) {
            const __half *kr = (t < n_load) ? Ks + (size_t)t * H : sh->newk[k];
#pragma unroll
            for (int v = 0; v < 2; ++v) {
              const uint4 kq = *reinterpret_cast<const uint4 *>(kr + v * 64 + sub * 8);
              const uint4 qq = *reinterpret_cast<const uint4 *>(sh->qs[k] + v * 64 + sub * 8);
              const __half2 *kh = reinterpret_cast<const __half2 *>(&kq), *qh = reinterpret_cast<const __half2 *>(&qq);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 a = __half22float2(kh[j]), q2 = __half22float2(qh[j]);
                sc += a.x * q2.x + a.y * q2.y;
              }
            }
          }
          sc += __shfl_xor_sync(0xffffffffu, sc, 1);
          sc += __shfl_xor_sync(0xffffffffu, sc, 2);
          sc += __shfl_xor_sync(0xffffffffu, sc, 4);
          if (sub == 0 && t < n_valid) ps[t] = __half2float(h_mul(__float2half_rn(sc), p.score_scale));
        }
      }
      group_sync(grp);
      if ((warp & 3) == 0) {  // softmax statistics of the page (fp32, like the reference's cast before SoftmaxV3)
        float m = -INFINITY;
        for (int t = lane; t < n_valid; t += 32) m = fmaxf(m, ps[t]);
        m = warp_max(m);
        float l = 0.f;
        for (int t = lane; t < n_valid; t += 32) {
          const float e = expf(ps[t] - m);
          ps[t] = e;
          l += e;
        }
        l = warp_sum(l);
        if (lane == 0) { sh->ml[grp][0] = m; sh->ml[grp][1] = l; }
      }
      group_sync(grp);
      {  // P.V: one thread per channel
        float o = 0.f;
        if (!sh->abort)
          for (int t = 0; t < n_valid; ++t) {
            const __half vv = (t < n_load) ? Vs[(size_t)t * H + gt] : sh->newv[k][gt];
            o += ps[t] * __half2float(vv);
          }
        const size_t hd = (size_t)b * p.n_head + head;
        p.ws_o[(hd * p.max_pages + pg) * H + gt] = o;
        if (gt == 0) p.ws_ml[hd * p.max_pages + pg] = make_float2(sh->ml[grp][0], sh->ml[grp][1]);
      }
      group_sync(grp);  // the group is done with the stage and with ps / ml
      if (n_load > 0 && lane == 0) mbar_arrive(smem_addr(&sh->empty[slot]));
    }
    // ---- last page of a (sequence, head) to arrive combines that head in page order
    __threadfence();
    consumer_sync();
    if (tid < nu) {
      const int u = u0 + tid * c.G;
      const int head = (u / n_active) % p.n_head, b = u / (n_active * p.n_head);
      sh->last[tid] = (atomicAdd(p.attn_counters + (size_t)b * p.n_head + head, 1) == n_active - 1);
    }
    consumer_sync();
    for (int k = grp; k >= 0 && k < nu; k += NGRP) {
      if (!sh->last[k]) continue;
      const int u = u0 + k * c.G;
      const int head = (u / n_active) % p.n_head, b = u / (n_active * p.n_head);
      const size_t hd = (size_t)b * p.n_head + head;
      __threadfence();
      if (gt == 0) p.attn_counters[hd] = 0;
      float M = -INFINITY;
      for (int i = 0; i < n_active; ++i) M = fmaxf(M, __ldcg(&p.ws_ml[hd * p.max_pages + i]).x);
      float Lsum = 0.f, o = 0.f;
      for (int i = 0; i < n_active; ++i) {
        const float2 v = __ldcg(&p.ws_ml[hd * p.max_pages + i]);
        const float w = expf(v.x - M);
        Lsum += v.y * w;
        o += __ldcg(&p.ws_o[(hd * p.max_pages + i) * H + gt]) * w;
      }
      p.attn[(size_t)b * p.d + (size_t)head * H + gt] = __float2half_rn(o / Lsum);
    }
    consumer_sync();
  }
}

// ------------------------------------------------------------------------------------------ producer
struct Producer {
  const Params &p;
  Shared *sh;
  int sm, G;
  int slot;            // ring slot of the next stage
  uint32_t parity;     // parity to wait for on that slot's `empty` barrier
  bool first_round;    // slots have not been used yet: nothing to wait for
  uint32_t ring_s, full_s, empty_s;  // shared-memory addresses
  bool ok;
  // The loop below competes with the consumer warps for issue slots, so it is kept to a handful of instructions per stage:
  // no divisions, all addresses incremental.  One stage: `bytes` from src at offset 0 and, for attention stages, `bytes2`
  // from src2 at V_OFFSET.
  __device__ __forceinline__ void push(const void *src, uint32_t bytes, const void *src2, uint32_t bytes2) {
    if (!first_round && !mbar_wait(empty_s + slot * 8, parity, &sh->abort)) {
      if (ok && p.error_flag) atomicExch(p.error_flag, 6);
      ok = false;
      sh->abort = 1;
    }
    if (ok) {
      const uint32_t fb = full_s + slot * 8, dst = ring_s + slot * STAGE_BYTES;
      mbar_expect_tx(fb, bytes + bytes2);
      bulk_g2s(dst, src, bytes, fb);
      if (bytes2) bulk_g2s(dst + V_OFFSET, src2, bytes2, fb);
    }
    if (++slot == p.ns) {
      slot = 0;
      if (first_round) first_round = false;
      else parity ^= 1u;
    }
  }
  __device__ __forceinline__ void push_matrix(const unsigned char *w, int n_rt, int nchunks, int tile) {
    const int r0 = (int)((long long)sm * n_rt / G), r1 = (int)((long long)(sm + 1) * n_rt / G);
    int left = (r1 - r0) * nchunks * tile;                 // bytes of this SM's share
    const unsigned char *src = w + (size_t)r0 * nchunks * tile;
    const int stage = STAGE_TILES * tile;
    // stream order: full stages of NCW tiles, then one short stage with the T % NCW warps that have one more tile
    for (; left > 0 && ok; left -= stage, src += stage) push(src, (uint32_t)min(stage, left), nullptr, 0);
  }
  __device__ void push_attention(const pt_llama_layer &L, int step) {
    const int n_active = step / PAGE + 1;
    const int n_units = p.B * p.n_head * n_active;
    for (int u = sm; u < n_units && ok; u += G) {
      const int pg = u % n_active, head = (u / n_active) % p.n_head, b = u / (n_active * p.n_head);
      const int n_valid = min(PAGE, step + 1 - pg * PAGE);
      const int n_load = (pg == n_active - 1) ? n_valid - 1 : n_valid;
      if (n_load <= 0) continue;
      const int phys = p.page_table[(size_t)b * p.max_pages + pg];
      const __half *gK = (const __half *)L.pool + (((size_t)phys * 2 + 0) * p.n_head + head) * PAGE * H;
      const __half *gV = (const __half *)L.pool + (((size_t)phys * 2 + 1) * p.n_head + head) * PAGE * H;
      push(gK, (uint32_t)n_load * H * 2, gV, (uint32_t)n_load * H * 2);
    }
  }
};

__global__ void __launch_bounds__(THREADS, 1) llama_step_kernel(const Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char *ring = smem;
  unsigned char *xs = smem + (size_t)p.ns * STAGE_BYTES;
  Shared *sh = reinterpret_cast<Shared *>(xs + (((size_t)BMAX * p.xs_stride + 127) / 128) * 128);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int step = *p.step;

  if (tid == 0) {
    for (int s = 0; s < p.ns; ++s) {
      mbar_init(smem_addr(&sh->full[s]), 1);
      mbar_init(smem_addr(&sh->empty[s]), NCW);
    }
    sh->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int n_rt_qkv = 3 * p.d / 16, n_rt_o = p.d / 16, n_rt_gu = 2 * p.ffn / 16, n_rt_head = (p.vocab + 15) / 16;
  const int nc_d = p.d / 128, nc_f = p.ffn / 128, nc_head = p.d / 32;

  if (warp == NCW) {
    // ---------------- producer: one lane walks the whole step's weight / KV stream of this SM
    if (lane == 0) {
      Producer pr{p, sh, (int)blockIdx.x, (int)gridDim.x, 0, 0u, true, smem_addr(ring), smem_addr(&sh->full[0]), smem_addr(&sh->empty[0]), true};
      for (int l = 0; l < p.n_layer; ++l) {
        const pt_llama_layer &L = p.layers[l];
        pr.push_matrix((const unsigned char *)L.qkv, n_rt_qkv, nc_d, TILE_I4);
        pr.push_attention(L, step);
        pr.push_matrix((const unsigned char *)L.o, n_rt_o, nc_d, TILE_I4);
        pr.push_matrix((const unsigned char *)L.gu, n_rt_gu, nc_d, TILE_I4);
        pr.push_matrix((const unsigned char *)L.down, n_rt_o, nc_f, TILE_I4);
      }
      pr.push_matrix(p.head, n_rt_head, nc_head, TILE_F16);
    }
    return;
  }

  // ---------------- consumers
  // Two barrier counters are used by alternate launches: word [2] says which one is this launch's (it is zero: the
  // previous launch cleared it when it finished); the last block clears the other one at the very end.
  const unsigned which = __ldcg(p.barrier + 2) & 1u;
  Ctx c{p, ring, xs, sh, (int)blockIdx.x, (int)gridDim.x, step, p.barrier + which, 0u, 0u, nullptr};

  // embedding: every SM gathers the rows itself (no barrier needed); the copy in global memory serves the residual adds
  for (int i = tid; i < p.B * (p.d / 8); i += NCT) {
    const int b = i / (p.d / 8), u = i - b * (p.d / 8);
    int id = p.ids[(size_t)b * p.max_len + step];
    id = min(max(id, 0), p.vocab - 1);
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p.emb + (size_t)id * p.d) + u);
    if ((u % c.G) == c.sm) reinterpret_cast<uint4 *>(p.x + (size_t)b * p.d)[u] = v;
  }
  Gamma g1 = load_gamma((const __half *)p.layers[0].ln1, p.d);
  const Gamma gnone = load_gamma(nullptr, 0);
  grid_sync(c);

  unsigned long long *tr = p.trace ? p.trace + ((size_t)blockIdx.x * p.n_layer) * 16 : nullptr;
#define PT_STAMP(k) do { if (tr && tid == 0) tr[l * 16 + (k)] = gtime(); } while (0)
  for (int l = 0; l < p.n_layer; ++l) {
    const pt_llama_layer &L = p.layers[l];
    PT_STAMP(0);
    c.tr = tr ? tr + l * 16 : nullptr;
    stage_x<true>(c, p.x, p.d, (const __half *)L.ln1, g1);
    c.tr = nullptr;
    PT_STAMP(1);
    linear_phase<PT_W_INT4, EPI_QKV>(c, n_rt_qkv, nc_d, p.qkv, 3 * p.d, nullptr);
    PT_STAMP(2);
    grid_sync(c);
    PT_STAMP(3);
    attention_phase(c, L);
    PT_STAMP(4);
    grid_sync(c);
    PT_STAMP(5);
    stage_x<true>(c, p.attn, p.d, nullptr, gnone);
    linear_phase<PT_W_INT4, EPI_RESID>(c, n_rt_o, nc_d, p.x, p.d, nullptr);
    PT_STAMP(6);
    const Gamma g2 = load_gamma((const __half *)L.ln2, p.d);
    grid_sync(c);
    PT_STAMP(7);
    stage_x<true>(c, p.x, p.d, (const __half *)L.ln2, g2);
    PT_STAMP(8);
    linear_phase<PT_W_INT4, EPI_SWIGLU>(c, n_rt_gu, nc_d, p.act, 2 * p.ffn, nullptr);
    PT_STAMP(9);
    grid_sync(c);
    PT_STAMP(10);
    stage_x<true>(c, p.act, p.ffn, nullptr, gnone);
    linear_phase<PT_W_INT4, EPI_RESID>(c, n_rt_o, nc_f, p.x, p.d, nullptr);
    PT_STAMP(11);
    g1 = load_gamma(l + 1 < p.n_layer ? (const __half *)p.layers[l + 1].ln1 : p.norm, p.d);
    grid_sync(c);
    PT_STAMP(12);
  }
#undef PT_STAMP

  // final norm + LM head + arg-max (lowest index wins ties)
  Best best;
#pragma unroll
  for (int b = 0; b < BMAX; ++b) { best.v[b] = -INFINITY; best.i[b] = 0x7fffffff; }
  stage_x<false>(c, p.x, p.d, p.norm, g1);
  linear_phase<PT_W_FP16, EPI_HEAD>(c, n_rt_head, nc_head, p.logits, p.vocab, &best);
  for (int b = 0; b < p.B; ++b) {
    float v = best.v[b];
    int i = best.i[b];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, i, o);
      if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
    if (lane == 0) { sh->bestv[warp][b] = v; sh->besti[warp][b] = i; }
  }
  consumer_sync();
  if (tid < p.B) {
    float v = sh->bestv[0][tid];
    int i = sh->besti[0][tid];
    for (int w = 1; w < NCW; ++w) {
      const float ov = sh->bestv[w][tid];
      const int oi = sh->besti[w][tid];
      if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
    p.cand_val[(size_t)tid * c.G + c.sm] = v;
    p.cand_idx[(size_t)tid * c.G + c.sm] = i;
  }
  grid_sync(c);
  if (blockIdx.x == 0 && warp == 0 && !sh->abort) {
    // merge the per-SM candidates, then the loop carry (step_containers / step_loop_cond)
    for (int b = 0; b < p.B; ++b) {
      float v = -INFINITY;
      int i = 0x7fffffff;
      for (int s = lane; s < c.G; s += 32) {
        const float ov = __ldcg(p.cand_val + (size_t)b * c.G + s);
        const int oi = __ldcg(p.cand_idx + (size_t)b * c.G + s);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
      }
      if (lane == 0) {
        p.next_ids[b] = i;
        const int nxt = step + 1;
        if (nxt < p.max_len) {
          const int cur = p.ids[(size_t)b * p.max_len + nxt];
          const int upd = (cur == p.pad_id) ? i : cur;
          p.ids[(size_t)b * p.max_len + nxt] = upd;
          if (p.stop_mask) p.stop_mask[b] |= (upd == p.eos_id) ? 1 : 0;
        }
      }
    }
    __syncwarp();
    if (lane == 0) *p.step = step + 1;
  }
  if (blockIdx.x == 0 && tid == 0) {  // every block has passed the last barrier of this launch
    p.barrier[which ^ 1u] = 0;
    p.barrier[2] = which ^ 1u;
  }
}

// Re-orders the tiles of a packed matrix ([row tile][chunk] order) inside every SM's share into stream order: the tile that
// consumer warp w processes at its j-th step sits at position j * NCW + w of the share.
__global__ void stream_permute_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, int n_rt, int nchunks, int tile_u, int G) {
  for (int sm = blockIdx.y; sm < G; sm += gridDim.y) {
    const int r0 = (int)((long long)sm * n_rt / G), r1 = (int)((long long)(sm + 1) * n_rt / G);
    const int T = (r1 - r0) * nchunks;
    const Split sp(T);
    const size_t seg = (size_t)r0 * nchunks * tile_u;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < (size_t)T * tile_u; i += (size_t)gridDim.x * blockDim.x) {
      const int d = (int)(i / tile_u), e = (int)(i - (size_t)d * tile_u);
      int j, w;
      if (d < sp.base * NCW) { j = d / NCW; w = d - j * NCW; }
      else { j = sp.base; w = d - sp.base * NCW; }
      const int q = sp.start(w) + j;
      dst[seg + (size_t)d * tile_u + e] = src[seg + (size_t)q * tile_u + e];
    }
  }
}

}  // namespace mk
}  // namespace pt

using namespace pt;

static int mk_sm_count(int *out) {
  static int n_sm = 0;
  if (n_sm == 0) {
    int dev = 0;
    PT_CUDA(cudaGetDevice(&dev));
    PT_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
  }
  *out = n_sm;
  return PT_OK;
}

extern "C" int pt_llama_stream_permute(int wfmt, const void *packed, void *out, int n_out, int k_in, void *stream) {
  PT_REQUIRE(packed && out && packed != out, "pt_llama_stream_permute: needs distinct source and destination buffers");
  PT_REQUIRE(wfmt == PT_W_INT4 || wfmt == PT_W_FP16, "pt_llama_stream_permute: weight format %d not used by the persistent kernel", wfmt);
  PT_REQUIRE(n_out > 0 && k_in > 0 && k_in % chunk_k(wfmt) == 0, "pt_llama_stream_permute: bad shape [%d, %d]", n_out, k_in);
  int n_sm = 0;
  if (int rc = mk_sm_count(&n_sm)) return rc;
  mk::stream_permute_kernel<<<dim3(32, n_sm), 256, 0, as_stream(stream)>>>((const uint4 *)packed, (uint4 *)out, ceil_div(n_out, 16), k_in / chunk_k(wfmt),
                                                                            tile_bytes(wfmt) / 16, n_sm);
  PT_LAUNCH_CHECK("pt_llama_stream_permute");
  return PT_OK;
}

extern "C" size_t pt_llama_step_workspace_bytes(int batch, int n_head, int head_dim, int max_pages) {
  const size_t heads = (size_t)batch * n_head;
  auto al = [](size_t v) { return (v + 255) / 256 * 256; };
  // barrier counters | attention counters | (max, sum) | partial outputs | arg-max candidates (value, index) for up to 256 SMs
  return 256 + al(heads * sizeof(int)) + al(heads * max_pages * sizeof(float2)) + al(heads * max_pages * head_dim * sizeof(float)) +
         2 * al((size_t)batch * 256 * sizeof(float));
}

extern "C" int pt_llama_decode_step(const pt_llama_step_args *a, void *stream) {
  PT_REQUIRE(a, "pt_llama_decode_step: null args");
  PT_REQUIRE(a->batch >= 1 && a->batch <= mk::BMAX, "pt_llama_decode_step: batch=%d outside 1..%d (larger batches use the per-op kernels)", a->batch,
             mk::BMAX);
  PT_REQUIRE(a->head_dim == mk::H && a->page_size == mk::PAGE, "pt_llama_decode_step: needs head_dim=%d and page_size=%d", mk::H, mk::PAGE);
  PT_REQUIRE(a->d_model % 128 == 0 && a->ffn % 128 == 0 && a->d_model == a->n_head * a->head_dim && a->d_model <= 96 * 128 && a->ffn <= 96 * 128,
             "pt_llama_decode_step: d_model=%d ffn=%d must be multiples of 128 (at most 12288) with d_model = n_head * head_dim", a->d_model, a->ffn);
  PT_REQUIRE((2 * a->ffn) % 16 == 0 && a->vocab > 0 && a->n_layer > 0 && a->max_len > 0 && a->max_pages * mk::PAGE >= a->max_len,
             "pt_llama_decode_step: bad shape");
  PT_REQUIRE(a->layers && a->norm && a->head && a->emb && a->ids && a->step_dev && a->page_table && a->rope_sin && a->rope_cos && a->x && a->qkv &&
                 a->attn && a->act && a->next_ids && a->workspace,
             "pt_llama_decode_step: null pointer argument");
  const size_t need = pt_llama_step_workspace_bytes(a->batch, a->n_head, a->head_dim, a->max_pages);
  PT_REQUIRE(a->workspace_bytes >= need, "pt_llama_decode_step: workspace needs %zu bytes, got %zu", need, a->workspace_bytes);

  int n_sm = 0;
  if (int rc = mk_sm_count(&n_sm)) return rc;
  static size_t smem_max = 0;
  if (smem_max == 0) {
    int dev = 0, v = 0;
    PT_CUDA(cudaGetDevice(&dev));
    PT_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    PT_CUDA(cudaFuncSetAttribute(mk::llama_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, v));
    smem_max = (size_t)v;
  }
  PT_REQUIRE(n_sm <= 256, "pt_llama_decode_step: %d SMs exceed the candidate buffer", n_sm);

  mk::Params p{};
  p.B = a->batch; p.d = a->d_model; p.n_head = a->n_head; p.ffn = a->ffn; p.vocab = a->vocab; p.n_layer = a->n_layer;
  p.max_len = a->max_len; p.max_pages = a->max_pages; p.pad_id = a->pad_id; p.eos_id = a->eos_id;
  p.eps = a->norm_eps;
  p.score_scale = __float2half_rn(a->score_scale);
  p.layers = a->layers; p.norm = (const __half *)a->norm; p.emb = (const __half *)a->emb;
  p.sin_t = (const __half *)a->rope_sin; p.cos_t = (const __half *)a->rope_cos; p.head = (const unsigned char *)a->head;
  p.ids = a->ids; p.step = a->step_dev; p.stop_mask = a->stop_mask; p.next_ids = a->next_ids; p.page_table = a->page_table;
  p.x = (__half *)a->x; p.qkv = (__half *)a->qkv; p.attn = (__half *)a->attn; p.act = (__half *)a->act; p.logits = (__half *)a->logits;
  p.error_flag = a->error_flag;
  p.trace = (unsigned long long *)a->trace;
  p.debug = a->debug;
  auto al = [](size_t v) { return (v + 255) / 256 * 256; };
  const size_t heads = (size_t)a->batch * a->n_head;
  char *ws = (char *)a->workspace;
  p.barrier = (unsigned *)ws; ws += 256;
  p.attn_counters = (int *)ws; ws += al(heads * sizeof(int));
  p.ws_ml = (float2 *)ws; ws += al(heads * a->max_pages * sizeof(float2));
  p.ws_o = (float *)ws; ws += al(heads * a->max_pages * a->head_dim * sizeof(float));
  p.cand_val = (float *)ws; ws += al((size_t)a->batch * 256 * sizeof(float));
  p.cand_idx = (int *)ws;

  const int kmax = std::max(a->d_model, a->ffn);
  p.xs_stride = (kmax * 2) | 64;
  const size_t fixed = (((size_t)mk::BMAX * p.xs_stride + 127) / 128) * 128 + sizeof(mk::Shared) + 128;
  PT_REQUIRE(smem_max > fixed + 3 * (size_t)mk::STAGE_BYTES, "pt_llama_decode_step: shared memory too small");
  p.ns = (int)std::min<size_t>(16, (smem_max - fixed) / mk::STAGE_BYTES);
  const size_t smem = (size_t)p.ns * mk::STAGE_BYTES + fixed;

  void *kargs[] = {(void *)&p};
  cudaError_t e = cudaLaunchCooperativeKernel((const void *)mk::llama_step_kernel, dim3(n_sm), dim3(mk::THREADS), kargs, smem, as_stream(stream));
  if (e != cudaSuccess) return pt::set_error(PT_ERR_CUDA, "pt_llama_decode_step: %s", cudaGetErrorString(e));
  PT_LAUNCH_CHECK("pt_llama_decode_step");
  return PT_OK;
}
