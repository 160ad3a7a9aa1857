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

constexpr int NCW = 16;                 // consumer warps
constexpr int NCT = NCW * 32;           // consumer threads
constexpr int THREADS = NCT + 32;       // + the producer warp
constexpr int TILE_I4 = 1056, TILE_F16 = 1024;
constexpr int STAGE_BYTES = NCW * TILE_I4;  // 16896
constexpr int BMAX = 2;
constexpr int H = 128, PAGE = 64;
constexpr int SPIN_LIMIT = 1 << 22;

struct Params {
  int B, d, n_head, ffn, vocab, n_layer, max_len, max_pages, ns, xs_stride, pad_id, eos_id;
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
// Bounded wait; gives up at once when the block has already recorded a failure, so that after an error every loop of the
// kernel still runs its normal trip count (all named barriers stay matched) but finishes quickly.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const volatile int *abort_flag) {
  for (int it = 0; it < SPIN_LIMIT; ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    if (ok) return true;
    if (*abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NCT) : "memory"); }

struct Shared {           // fixed-size part, placed after the ring / activations
  float red[2][NCW][32][4];
  float corr[96][8];      // [chunk][batch column], up to 96 chunks of 128 k
  __half qs[H], newk[H], newv[H];
  float ps[PAGE + 1];
  float o4[4][H];
  float stat[BMAX];
  float wred[NCW];
  float bestv[NCW][BMAX];
  int besti[NCW][BMAX];
  float ml[2];
  volatile int abort;
  int last;
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

// Stage activations src[B, K] (global, written by other SMs: read through L2) into shared memory for the next linear phase.
// INT4 phases use the per-chunk swizzle of linear.cu ([chunk][w][tig] 16-byte units) and produce the offset corrections;
// the fp16 phase (LM head) keeps the natural order.  gamma != nullptr applies RMSNorm first.
template <bool INT4>
__device__ void stage_x(Ctx &c, const __half *src, int K, const __half *gamma) {
  const Params &p = c.p;
  const int tid = threadIdx.x;
  const int units = K / 8;
  for (int b = 0; b < p.B; ++b) {
    uint4 v[3];
    const uint4 *xr = reinterpret_cast<const uint4 *>(src + (size_t)b * K);
#pragma unroll
    for (int q = 0; q < 3; ++q) v[q] = (tid + q * NCT < units) ? __ldcg(xr + tid + q * NCT) : make_uint4(0, 0, 0, 0);
    __half rb = __half(0);
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
    }
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const int u = tid + q * NCT;
      const bool valid = u < units;
      __half *h = reinterpret_cast<__half *>(&v[q]);
      if (gamma && valid) {
        const uint4 gv = __ldg(reinterpret_cast<const uint4 *>(gamma) + u);
        const __half *gh = reinterpret_cast<const __half *>(&gv);
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

// One linear phase over this SM's row tiles [r0, r1) of a matrix with `nchunks` tiles per row tile.
template <int WFMT, int EPI>
__device__ void linear_phase(Ctx &c, int n_rt, int nchunks, __half *out, int N, Best *best) {
  constexpr int TILE = WTraits<WFMT>::kTileBytes;
  constexpr int UNITS = WTraits<WFMT>::kUnits;
  constexpr int CHUNK_X_BYTES = WTraits<WFMT>::kChunkK * 2;
  const Params &p = c.p;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tig = lane & 3;
  const int r0 = (int)((long long)c.sm * n_rt / c.G), r1 = (int)((long long)(c.sm + 1) * n_rt / c.G);
  const int total = (r1 - r0) * nchunks;
  int cur = 0, buf = 0;  // row tile (local index) whose partial sums `acc` holds
  float acc[4] = {0.f, 0.f, 0.f, 0.f};

  auto flush = [&](int rt_l) {
    float4 *slot = reinterpret_cast<float4 *>(&c.sh->red[buf][warp][lane][0]);
    *slot = make_float4(acc[0], acc[1], acc[2], acc[3]);
    consumer_sync();
    if (warp == (rt_l & (NCW - 1))) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w = 0; w < NCW; ++w) {
        const float4 t = *reinterpret_cast<const float4 *>(&c.sh->red[buf][w][lane][0]);
        v[0] += t.x; v[1] += t.y; v[2] += t.z; v[3] += t.w;
      }
      const int rt = r0 + rt_l;
      if (tig == 0) {  // batch columns 0 and 1 live in the tig == 0 lanes
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
    }
    buf ^= 1;
  };

  for (int t0 = 0; t0 < total; t0 += NCW, ++c.gs) {
    const int t = t0 + warp;
    const int slot = c.gs % p.ns;
    const bool got = mbar_wait(smem_addr(&c.sh->full[slot]), (c.gs / p.ns) & 1, &c.sh->abort);
    if (!got) {
      c.sh->abort = 1;
      if (lane == 0 && p.error_flag) atomicExch(p.error_flag, 4);
    }
    uint4 va = make_uint4(0, 0, 0, 0), vb = va;
    float2 sf = make_float2(1.f, 1.f);
    const bool have = t < total;
    if (have && got) {
      const unsigned char *tile = c.ring + (size_t)slot * STAGE_BYTES + (size_t)warp * TILE;
      va = *reinterpret_cast<const uint4 *>(tile + lane * 16);
      vb = *reinterpret_cast<const uint4 *>(tile + 512 + lane * 16);
      if (WFMT == PT_W_INT4) sf = __half22float2(*reinterpret_cast<const __half2 *>(tile + 1024 + g * 4));
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_addr(&c.sh->empty[slot]));  // this warp's tile is in registers
    if (!have) continue;
    const int rt_l = t / nchunks, ch = t - rt_l * nchunks;
    while (cur < rt_l) {  // every warp flushes every row tile exactly once, in order (zeros if it had no tile of it)
      flush(cur);
      ++cur;
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
    }
    float cc[4] = {0.f, 0.f, 0.f, 0.f};
    const unsigned char *xc = c.xs + (size_t)ch * CHUNK_X_BYTES + tig * 16;
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
      uint32_t fa[4], fb[4];
      expand8<WFMT>(va, u, fa);
      expand8<WFMT>(vb, u, fb);
      uint4 xv = make_uint4(0, 0, 0, 0);
      if (g < p.B) xv = *reinterpret_cast<const uint4 *>(xc + (size_t)g * p.xs_stride + u * 64);
      if (WFMT == PT_W_INT4) {
        mma16816(cc, fa[0], fb[0], fa[1], fb[1], xv.x, xv.y);
        mma16816(cc, fa[2], fb[2], fa[3], fb[3], xv.z, xv.w);
      } else {
        mma16816(acc, fa[0], fb[0], fa[1], fb[1], xv.x, xv.y);
        mma16816(acc, fa[2], fb[2], fa[3], fb[3], xv.z, xv.w);
      }
    }
    if (WFMT == PT_W_INT4) {
      const float2 co = *reinterpret_cast<const float2 *>(&c.sh->corr[ch][2 * tig]);
      acc[0] += sf.x * (cc[0] - co.x);
      acc[1] += sf.x * (cc[1] - co.y);
      acc[2] += sf.y * (cc[2] - co.x);
      acc[3] += sf.y * (cc[3] - co.y);
    }
  }
  while (cur < r1 - r0) {
    flush(cur);
    ++cur;
    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
  }
}

// RoPE (rotate_half form) on one head vector in global memory -> dst (shared), reference fp16 roundings.
__device__ __forceinline__ void rope_pair(const __half *x, const __half *sin_r, const __half *cos_r, int i, __half *dst) {
  const __half a = __ldcg(x + i), b = __ldcg(x + i + H / 2), s = sin_r[i], co = cos_r[i];
  dst[i] = h_add(h_mul(a, co), h_mul(__hneg(b), s));
  dst[i + H / 2] = h_add(h_mul(b, co), h_mul(a, s));
}

// Attention phase: units (b, head, page) are dealt round-robin to the SMs; the producer has queued K and V tiles.
__device__ void attention_phase(Ctx &c, const pt_llama_layer &L) {
  const Params &p = c.p;
  Shared *sh = c.sh;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int step = c.step, n_active = step / PAGE + 1;
  const int n_units = p.B * p.n_head * n_active;
  const int row_elems = 3 * p.d;
  const __half *sin_r = p.sin_t + (size_t)step * (H / 2), *cos_r = p.cos_t + (size_t)step * (H / 2);
  for (int u = c.sm; u < n_units; u += c.G) {
    const int pg = u % n_active, head = (u / n_active) % p.n_head, b = u / (n_active * p.n_head);
    const int n_valid = min(PAGE, step + 1 - pg * PAGE);
    const bool owner = (pg == n_active - 1);
    const int n_load = owner ? n_valid - 1 : n_valid;
    const __half *qrow = p.qkv + (size_t)b * row_elems;
    if (tid < H / 2) rope_pair(qrow + (size_t)head * H, sin_r, cos_r, tid, sh->qs);
    if (owner) {
      if (tid >= 64 && tid < 64 + H / 2) rope_pair(qrow + p.d + (size_t)head * H, sin_r, cos_r, tid - 64, sh->newk);
      if (tid >= 128 && tid < 128 + H) sh->newv[tid - 128] = __ldcg(qrow + 2 * p.d + (size_t)head * H + tid - 128);
    }
    const __half *Ks = nullptr, *Vs = nullptr;
    int slotK = 0, slotV = 0;
    if (n_load > 0) {
      slotK = c.gs % p.ns;
      const bool g1 = mbar_wait(smem_addr(&sh->full[slotK]), (c.gs / p.ns) & 1, &sh->abort);
      ++c.gs;
      slotV = c.gs % p.ns;
      const bool g2 = mbar_wait(smem_addr(&sh->full[slotV]), (c.gs / p.ns) & 1, &sh->abort);
      ++c.gs;
      if (!(g1 && g2)) {
        sh->abort = 1;
        if (lane == 0 && p.error_flag) atomicExch(p.error_flag, 5);
      }
      Ks = reinterpret_cast<const __half *>(c.ring + (size_t)slotK * STAGE_BYTES);
      Vs = reinterpret_cast<const __half *>(c.ring + (size_t)slotV * STAGE_BYTES);
    }
    consumer_sync();  // q (and the new k, v) staged
    if (owner && !sh->abort) {  // append the new token to the pool
      const int phys = p.page_table[(size_t)b * p.max_pages + pg];
      __half *gK = (__half *)L.pool + (((size_t)phys * 2 + 0) * p.n_head + head) * PAGE * H + (size_t)(n_valid - 1) * H;
      __half *gV = (__half *)L.pool + (((size_t)phys * 2 + 1) * p.n_head + head) * PAGE * H + (size_t)(n_valid - 1) * H;
      if (tid < H) gK[tid] = sh->newk[tid];
      else if (tid < 2 * H) gV[tid - H] = sh->newv[tid - H];
    }
    // scores: 8 lanes per cached token, all 64 tokens of the page in one pass
    {
      const int sub = lane & 7, t = tid >> 3;
      float s = 0.f;
      if (t < n_valid && !sh->abort) {
        const __half *kr = (t < n_load) ? Ks + (size_t)t * H : sh->newk;
#pragma unroll
        for (int v = 0; v < 2; ++v) {
          const uint4 kq = *reinterpret_cast<const uint4 *>(kr + v * 64 + sub * 8);
          const uint4 qq = *reinterpret_cast<const uint4 *>(sh->qs + v * 64 + sub * 8);
          const __half2 *kh = reinterpret_cast<const __half2 *>(&kq), *qh = reinterpret_cast<const __half2 *>(&qq);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 a = __half22float2(kh[j]), q2 = __half22float2(qh[j]);
            s += a.x * q2.x + a.y * q2.y;
          }
        }
      }
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (sub == 0 && t < n_valid) sh->ps[t] = __half2float(h_mul(__float2half_rn(s), p.score_scale));
    }
    consumer_sync();
    if (warp == 0) {  // softmax statistics of the page (fp32, like the reference's cast before SoftmaxV3)
      float m = -INFINITY;
      for (int t = lane; t < n_valid; t += 32) m = fmaxf(m, sh->ps[t]);
      m = warp_max(m);
      float l = 0.f;
      for (int t = lane; t < n_valid; t += 32) {
        const float e = expf(sh->ps[t] - m);
        sh->ps[t] = e;
        l += e;
      }
      l = warp_sum(l);
      if (lane == 0) { sh->ml[0] = m; sh->ml[1] = l; }
    }
    consumer_sync();
    {  // P.V: 4 token quarters x 128 channels
      const int q4 = tid >> 7, j = tid & 127;
      float o = 0.f;
      if (!sh->abort)
        for (int t = q4; t < n_valid; t += 4) {
          const __half vv = (t < n_load) ? Vs[(size_t)t * H + j] : sh->newv[j];
          o += sh->ps[t] * __half2float(vv);
        }
      sh->o4[q4][j] = o;
    }
    consumer_sync();
    if (n_load > 0 && lane == 0) {  // the K and V stages may be refilled
      mbar_arrive(smem_addr(&sh->empty[slotK]));
      mbar_arrive(smem_addr(&sh->empty[slotV]));
    }
    const size_t hd = (size_t)b * p.n_head + head;
    if (tid < H) p.ws_o[(hd * p.max_pages + pg) * H + tid] = (sh->o4[0][tid] + sh->o4[1][tid]) + (sh->o4[2][tid] + sh->o4[3][tid]);
    if (tid == 0) p.ws_ml[hd * p.max_pages + pg] = make_float2(sh->ml[0], sh->ml[1]);
    __threadfence();
    consumer_sync();
    if (tid == 0) sh->last = (atomicAdd(p.attn_counters + hd, 1) == n_active - 1);
    consumer_sync();
    if (sh->last) {  // last page of this (sequence, head) to arrive: combine in page order
      __threadfence();
      if (tid == 0) p.attn_counters[hd] = 0;
      if (tid < H) {
        float M = -INFINITY;
        for (int i = 0; i < n_active; ++i) M = fmaxf(M, __ldcg(&p.ws_ml[hd * p.max_pages + i]).x);
        float Lsum = 0.f, o = 0.f;
        for (int i = 0; i < n_active; ++i) {
          const float2 v = __ldcg(&p.ws_ml[hd * p.max_pages + i]);
          const float w = expf(v.x - M);
          Lsum += v.y * w;
          o += __ldcg(&p.ws_o[(hd * p.max_pages + i) * H + tid]) * w;
        }
        p.attn[(size_t)b * p.d + (size_t)head * H + tid] = __float2half_rn(o / Lsum);
      }
    }
    consumer_sync();
  }
}

// ------------------------------------------------------------------------------------------ producer
struct Producer {
  const Params &p;
  Shared *sh;
  unsigned char *ring;
  int sm, G;
  uint32_t gs;
  bool ok;
  __device__ void push(const void *src, uint32_t bytes) {
    if (!ok) return;
    const int slot = gs % p.ns;
    const uint32_t use = gs / p.ns;
    if (use > 0 && !mbar_wait(smem_addr(&sh->empty[slot]), (use - 1) & 1, &sh->abort)) {
      ok = false;
      sh->abort = 1;
      if (p.error_flag) atomicExch(p.error_flag, 6);
      return;
    }
    mbar_expect_tx(smem_addr(&sh->full[slot]), bytes);
    bulk_g2s(smem_addr(ring + (size_t)slot * STAGE_BYTES), src, bytes, smem_addr(&sh->full[slot]));
    ++gs;
  }
  __device__ void push_matrix(const unsigned char *w, int n_rt, int nchunks, int tile) {
    const int r0 = (int)((long long)sm * n_rt / G), r1 = (int)((long long)(sm + 1) * n_rt / G);
    const int total = (r1 - r0) * nchunks;
    const unsigned char *base = w + (size_t)r0 * nchunks * tile;
    for (int t = 0; t < total && ok; t += NCW) push(base + (size_t)t * tile, (uint32_t)min(NCW, total - t) * tile);
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
      push(gK, (uint32_t)n_load * H * 2);
      push(gV, (uint32_t)n_load * H * 2);
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
      Producer pr{p, sh, ring, (int)blockIdx.x, (int)gridDim.x, 0u, true};
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
  Ctx c{p, ring, xs, sh, (int)blockIdx.x, (int)gridDim.x, step, p.barrier + which, 0u, 0u};

  // embedding: every SM gathers the rows itself (no barrier needed); the copy in global memory serves the residual adds
  for (int i = tid; i < p.B * (p.d / 8); i += NCT) {
    const int b = i / (p.d / 8), u = i - b * (p.d / 8);
    int id = p.ids[(size_t)b * p.max_len + step];
    id = min(max(id, 0), p.vocab - 1);
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p.emb + (size_t)id * p.d) + u);
    if ((u % c.G) == c.sm) reinterpret_cast<uint4 *>(p.x + (size_t)b * p.d)[u] = v;
  }
  grid_sync(c);

  for (int l = 0; l < p.n_layer; ++l) {
    const pt_llama_layer &L = p.layers[l];
    stage_x<true>(c, p.x, p.d, (const __half *)L.ln1);
    linear_phase<PT_W_INT4, EPI_QKV>(c, n_rt_qkv, nc_d, p.qkv, 3 * p.d, nullptr);
    grid_sync(c);
    attention_phase(c, L);
    grid_sync(c);
    stage_x<true>(c, p.attn, p.d, nullptr);
    linear_phase<PT_W_INT4, EPI_RESID>(c, n_rt_o, nc_d, p.x, p.d, nullptr);
    grid_sync(c);
    stage_x<true>(c, p.x, p.d, (const __half *)L.ln2);
    linear_phase<PT_W_INT4, EPI_SWIGLU>(c, n_rt_gu, nc_d, p.act, 2 * p.ffn, nullptr);
    grid_sync(c);
    stage_x<true>(c, p.act, p.ffn, nullptr);
    linear_phase<PT_W_INT4, EPI_RESID>(c, n_rt_o, nc_f, p.x, p.d, nullptr);
    grid_sync(c);
  }

  // final norm + LM head + arg-max (lowest index wins ties)
  Best best;
#pragma unroll
  for (int b = 0; b < BMAX; ++b) { best.v[b] = -INFINITY; best.i[b] = 0x7fffffff; }
  stage_x<false>(c, p.x, p.d, p.norm);
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

}  // namespace mk
}  // namespace pt

using namespace pt;

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

  static int n_sm = 0;
  static size_t smem_max = 0;
  if (n_sm == 0) {
    int dev = 0;
    PT_CUDA(cudaGetDevice(&dev));
    cudaDeviceProp prop;
    PT_CUDA(cudaGetDeviceProperties(&prop, dev));
    n_sm = prop.multiProcessorCount;
    smem_max = prop.sharedMemPerBlockOptin;
    PT_CUDA(cudaFuncSetAttribute(mk::llama_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max));
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
