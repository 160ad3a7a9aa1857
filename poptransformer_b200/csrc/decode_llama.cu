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
//     keeps a ring of 33 KB shared-memory stages full with 1-D bulk async copies (TMA engine, one mbarrier
//     per stage).  Weights do not depend on activations, so the producer runs ahead across the phase
//     boundaries and HBM stays busy while the consumers wait for each other's activations;
//   * warps 0-15 are consumers: consumer w takes tiles w and 16 + w of every stage (a stage = 32 tiles of the packed
//     layout of linear.cu, re-ordered so that each warp walks a contiguous run of [row tile][chunk] tiles).  INT4 tiles are
//     multiplied on the integer tensor-core path: the nibbles of a packed word become two u8 operands with one AND each,
//     the activations are 16-bit block fixed point split into two s8 columns, and the s32 sums are scaled once per
//     128-k group; sums of a row tile that several warps share meet in shared memory in warp order (deterministic);
//   * K/V pages travel through the same ring; the attention arithmetic is that of attention.cu;
//   * there is no grid-wide barrier between phases: activations travel through global memory as 32-bit tagged words
//     (fp16 value + 16-bit phase tag), every SM publishes one progress word per phase, one warp per SM polls the
//     progress words and the data words validate themselves when they are loaded.  Every wait is bounded and raises the
//     error flag when it runs out.  One grid barrier remains, before the arg-max merge at the end of the step.
// Every SM owns whole row tiles: rows [s * n_rt / G, (s + 1) * n_rt / G).
#include <algorithm>

#include "tile_math.cuh"

// This file is compiled twice: as itself, and included by decode_llama_short.cu with PT_MK_SHORT_VARIANT defined, which builds
// the same kernel in namespace mk_short with the short poll limit and only a launcher around it.
#ifdef PT_MK_SHORT_VARIANT
#define PT_MK_NS mk_short
#define PT_MK_POLL_LIMIT kShortPollLimit
#else
#define PT_MK_NS mk
#endif

namespace pt {
namespace PT_MK_NS {

#ifndef PT_MK_WARPS
#define PT_MK_WARPS 16
#endif
constexpr int NCW = PT_MK_WARPS;        // consumer warps
constexpr int NCT = NCW * 32;           // consumer threads
constexpr int THREADS = NCT + 32;       // + the producer warp
constexpr int NGRP = NCW / 4;           // 4-warp attention groups
constexpr int TILE_I4 = 1056, TILE_F16 = 1024;
constexpr int STAGE_TILES = 2 * NCW;              // two tiles per consumer warp per stage
constexpr int STAGE_BYTES = ((STAGE_TILES * TILE_I4 + 127) / 128 * 128) > 33792 ? ((STAGE_TILES * TILE_I4 + 127) / 128 * 128) : 33792;
constexpr int V_OFFSET = 16896;                   // a K page and a V page (2 x 16 KB) share one attention stage
constexpr int MAXU = NCT / 64;                    // attention units handled per SM per pass (64 threads fetch q / k / v of one)
constexpr int BMAX = 2;
constexpr int H = 128, PAGE = 64;
static_assert(NCT % 64 == 0 || NCT % 32 == 0, "consumer threads come in whole warps");

struct Params {
  int B, d, n_head, ffn, vocab, n_layer, max_len, max_pages, ns, xs_stride, pad_id, eos_id, debug;
  // Tensor parallelism: d is the full hidden size; n_head, ffn and vocab are this rank's shares.  dq = n_head * H is the
  // width of the rank's q / k / v / attention vectors (the k range of its o_proj slice); the rank's MLP activations are
  // ffn_valid values at offset ffn_off inside a window of ffn columns (a multiple of 128; the weights outside are zero).
  int tp, rank, dq, ffn_off, ffn_valid, vocab_off, emb_rows;  // emb_rows: rows of the (replicated) embedding table
  uint32_t *peer_part[8];   // every rank's partial-sum buffer [2 (o_proj, down_proj)][tp][B][d], tagged words
  uint32_t *peer_flag[8];   // every rank's progress words [tp][256]
  uint2 *peer_cand[8];      // every rank's arg-max candidates [tp][BMAX][2] {value bits | index, sequence number}
  float eps;
  __half score_scale;
  const pt_llama_layer *layers;
  const __half *norm, *emb, *sin_t, *cos_t;
  const unsigned char *head;
  int *ids, *step, *stop_mask, *next_ids, *done_flag;
  const int *page_table;
  uint32_t *xw, *qkvw, *attnw, *actw;  // activations as tagged words; xw holds two copies [2][B][d] when tp > 1
  __half *logits;
  uint2 *ws_o;        // [B, n_head, max_pages, H] partial attention outputs as {fp32 bits, tag}
  uint2 *ws_ml;       // [B, n_head, max_pages, 2] page max and sum, same format
  float *cand_val;    // [B, grid]
  int *cand_idx;
  unsigned *barrier;  // [0], [1]: counters used by alternate launches; [2]: which one the next launch uses; [3]: launch count
  uint32_t *flag_sm;  // [256] sequence number of the last linear phase (or embedding) that SM s has finished writing
  uint2 *flag_ssq;    // [BMAX][256] {sum of squares of the x rows SM s wrote for batch row b (fp32 bits), sequence number}: written by the
                      // phases that produce x (embedding, o_proj, down_proj) just before flag_sm, so that whoever waits for x gets the
                      // RMSNorm statistics with the very loads that tell it x is complete
  uint32_t *flag_head;  // [B, n_head] sequence number of the last attention output written for that head
  int *error_flag;
  unsigned long long *trace;  // optional: [grid][n_layer][32] global-timer stamps of the phase boundaries
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
__constant__ uint32_t c_wait_hint = 2000u;  // suspend-time hint (ns) of the mbarrier waits
// Trip limit of every polling loop on global memory (progress words, tagged words, arrival counters); one trip is one L2 or
// NVLink round trip, so the default gives a waiter about two seconds before it gives up and raises the error flag.
constexpr int kDefaultPollLimit = 1 << 21;
constexpr int kShortPollLimit = 1 << 12;   // the short-wait build of the kernel (pt_llama_step_args.wait_limit != 0): a few milliseconds
// The limit is a compile-time constant of each kernel instantiation: a run-time bound costs the polling loops a register, and
// this kernel has none to spare (measured: 2 % of the step).
#ifndef PT_MK_POLL_LIMIT
#define PT_MK_POLL_LIMIT kDefaultPollLimit
#endif
constexpr int POLL_LIMIT = PT_MK_POLL_LIMIT;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const volatile int *abort_flag) {
  {  // the usual case inside a phase: the stage has landed, and a plain test costs less than a wait with a suspend hint (1.3 % of the step)
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    if (ok) return true;
  }
  const uint32_t hint = c_wait_hint;
  for (int it = 0; it < (1 << 18); ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity), "r"(hint)
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
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
// ---- Tagged words.  Activations that one SM produces and all SMs consume (x, qkv, attention output, MLP activations)
// travel through global memory as 32-bit words: fp16 value in the low half, the 16-bit tag of the producing phase in the
// high half.  A 32-bit store is indivisible, so a consumer that finds the expected tag also has the value: it polls the
// data itself and no grid-wide barrier (one atomic round trip, one polling round trip, then the load) separates the
// phases.  Tags grow with every phase and launch (period 32768 phases), every word is rewritten at least once per launch,
// so a stale word never carries the expected tag.  Re-use of a buffer is safe without barriers because the writer of the
// next value has (through the chain of phases in between) waited for data that every reader produced after reading.
__device__ __forceinline__ uint4 ld_words(const uint32_t *p) {
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_word(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// 64-bit variant for fp32 partial results: {value bits, tag}
__device__ __forceinline__ uint2 ld_tagged(const uint2 *p) {
  uint2 v;
  asm volatile("ld.relaxed.gpu.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_tagged(uint2 *p, uint32_t bits, uint32_t tag) {
  asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(bits), "r"(tag) : "memory");
}
__device__ __forceinline__ bool poll_tagged(const uint2 *p, uint32_t tag, uint32_t &bits, const volatile int *abort_flag) {
  for (int it = 0; it < POLL_LIMIT; ++it) {
    const uint2 v = ld_tagged(p);
    if (v.y == tag) { bits = v.x; return true; }
    if ((it & 63) == 63 && *abort_flag) break;
  }
  bits = 0;
  return false;
}
// Stores to another GPU's memory (or to this GPU's copy of a buffer that peers also write): system scope.
__device__ __forceinline__ void st_sys(uint32_t *p, uint32_t v) { asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void st_sys2(uint2 *p, uint32_t a, uint32_t b) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_sys2(const uint2 *p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_add_sys(uint32_t *p, uint32_t v) { asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void st_flag(uint32_t *p, uint32_t v) { asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void st_word(uint32_t *p, uint32_t tag, __half v) { *p = (tag << 16) | (uint32_t)__half_as_ushort(v); }
// Eight consecutive tagged words -> eight fp16 values (as a uint4).  Bounded: on time-out returns false.
__device__ __forceinline__ bool poll8(const uint32_t *p, uint32_t tag, uint4 &out, const volatile int *abort_flag) {
  for (int it = 0; it < POLL_LIMIT; ++it) {
    const uint4 a = ld_words(p), b = ld_words(p + 4);
    const uint32_t all = a.x & a.y & a.z & a.w & b.x & b.y & b.z & b.w, any = a.x | a.y | a.z | a.w | b.x | b.y | b.z | b.w;
    if ((all >> 16) == tag && (any >> 16) == tag) {
      out = make_uint4(__byte_perm(a.x, a.y, 0x5410), __byte_perm(a.z, a.w, 0x5410), __byte_perm(b.x, b.y, 0x5410), __byte_perm(b.z, b.w, 0x5410));
      return true;
    }
    if ((it & 63) == 63 && *abort_flag) break;
  }
  out = make_uint4(0, 0, 0, 0);
  return false;
}
__device__ __forceinline__ bool poll1(const uint32_t *p, uint32_t tag, __half &out, const volatile int *abort_flag) {
  for (int it = 0; it < POLL_LIMIT; ++it) {
    const uint32_t w = ld_word(p);
    if ((w >> 16) == tag) { out = __ushort_as_half((unsigned short)(w & 0xFFFFu)); return true; }
    if ((it & 63) == 63 && *abort_flag) break;
  }
  out = __half(0);
  return false;
}
// Warp 0 waits until every one of rows x cols progress words (row stride 256) has reached sequence number `want` (producers
// may already be one phase further).  This keeps the polling traffic to one warp per SM; the data words still carry tags, so
// a word whose store lags behind its producer's progress word is caught when it is loaded.
__device__ __forceinline__ bool wait_flags(const uint32_t *flags, int rows, int cols, uint32_t want, const volatile int *abort_flag) {
  const int lane = threadIdx.x & 31;
  for (int it = 0; it < POLL_LIMIT; ++it) {
    bool ok = true;
    for (int r = 0; r < rows; ++r) {
      // all of a lane's words (cols <= 256: up to eight) are requested before the first is looked at: one round trip per row
      uint32_t f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = (lane + 32 * j < cols) ? ld_word(flags + r * 256 + lane + 32 * j) : want;
#pragma unroll
      for (int j = 0; j < 8; ++j) ok &= (int)(f[j] - want) >= 0;
    }
    if (__all_sync(0xffffffffu, ok)) return true;
    if ((it & 63) == 63 && *abort_flag) break;
  }
  return false;
}
// The same wait on the entries {partial sum of squares, sequence number} that the producers of x publish (one entry per SM and
// batch row): when every entry carries `want`, the loads that proved it also hold the RMSNorm statistics.  Lane l sums entries
// l, l + 32, ... in that order, then the lanes meet in a fixed shuffle tree: the same bits on every SM and in every run.
// rb[b] <- 1 / sqrt(sum / K + eps) rounded to fp16 (layers/rms_layer_norm.py:26-36).
__device__ __forceinline__ bool wait_flags_ssq(const uint2 *flags, int B, int cols, uint32_t want, int K, float eps, float *rb,
                                               const volatile int *abort_flag) {
  const int lane = threadIdx.x & 31;
  for (int it = 0; it < POLL_LIMIT; ++it) {
    bool ok = true;
    float part[BMAX];
#pragma unroll
    for (int b = 0; b < BMAX; ++b) {
      part[b] = 0.f;
      if (b < B) {
        uint2 e[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) e[j] = (lane + 32 * j < cols) ? ld_tagged(flags + b * 256 + lane + 32 * j) : make_uint2(0u, want);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ok &= e[j].y == want;
          part[b] += __uint_as_float(e[j].x);
        }
      }
    }
    if (__all_sync(0xffffffffu, ok)) {
#pragma unroll
      for (int b = 0; b < BMAX; ++b)
        if (b < B) {
          const float ss = warp_sum(part[b]);
          if (lane == 0) rb[b] = __half2float(__float2half_rn(1.0f / sqrtf(ss / (float)K + eps)));
        }
      return true;
    }
    if ((it & 63) == 63 && *abort_flag) break;
  }
  return false;
}
// Tensor parallelism: one arrival counter per source rank (row stride 256 words), incremented once by every SM of that rank when
// its partial sums of a row-parallel linear are pushed.  Lane r looks at rank r's counter: one round trip per poll.
__device__ __forceinline__ bool wait_counters(const uint32_t *counters, int rows, uint32_t want, const volatile int *abort_flag) {
  const int lane = threadIdx.x & 31;
  for (int it = 0; it < POLL_LIMIT; ++it) {
    const bool ok = lane >= rows || (int)(ld_word(counters + lane * 256) - want) >= 0;
    if (__all_sync(0xffffffffu, ok)) return true;
    if ((it & 63) == 63 && *abort_flag) break;
  }
  return false;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NCT) : "memory"); }

// Operands of the running linear phase that only the (rare) row-tile epilogues need.  They live in shared memory rather than
// in registers, which the multiplication loop needs for itself.
struct PhaseInfo {
  uint32_t *outw;   // tagged-word output (phases between layers)
  __half *logits;   // fp16 output of the LM head (optional)
  uint32_t tag, out_seq;
  int epi, N, r0;
  int out_ld, out_off;  // MLP activations: row stride and offset of the first feature inside the k window of down_proj
  int push;         // 1: the rows are partial sums of a row-parallel linear, pushed into slot `push_slot` of every rank's buffer
  size_t push_slot; // word offset of this rank's slot for this linear in a rank's partial-sum buffer
};

// How one matrix is shared out: to this SM (row tiles [r0, r0 + m)) and, inside the SM, to the consumer warps (warp w owns the
// contiguous tile range [start(w), start(w) + len(w)) in [row tile][chunk] order, ranges differ by at most one tile).  Worked
// out once per launch, so that no phase starts with divisions.
constexpr int GEO_RT = 16;  // local row tiles with a precomputed owner range (more: computed on the fly)
struct Geo {
  int r0, m, base, rem;
  short first_rt[NCW];     // local row tile in which warp w's range starts ...
  short ch0[NCW];          // ... and the chunk inside it
  unsigned char w_lo[GEO_RT], w_hi[GEO_RT];  // first / last warp holding a part of local row tile r
};
enum { MAT_QKV = 0, MAT_O = 1, MAT_GU = 2, MAT_DOWN = 3, MAT_HEAD = 4 };

struct Shared {           // fixed-size part, placed after the ring / activations (128-byte aligned)
  alignas(16) float red[NCW][2][32][2];  // per warp: partial sums of the first / last row tile of its tile range
  int4 corr[96][BMAX];    // [chunk][batch]: C-fragment initialiser {-8 sum(t1), -8 sum(t2)} x 2 rows, up to 96 chunks of 128 k
  float xscale[96][BMAX]; // [chunk][batch]: activation scale of the chunk / 16
  uint4 zeros[2];         // what lanes without a batch column read as their B operand / C initialiser
  alignas(16) __half qs[MAXU][H], newk[MAXU][H], newv[MAXU][H];
  float ps[NGRP][PAGE];   // one row per 4-warp attention group
  float pw[NCW][PAGE];    // softmax weights of the page, one private copy per warp
  float ml[NGRP][2];
  int phys[MAXU];         // physical page of each unit of the attention pass (for the append of the new token)
  float stat[BMAX];       // RMSNorm factor of each batch row for the staging in progress
  float wssq[NCW][BMAX];  // per warp: sum of squares of the x values its epilogues wrote
  float wred[32];
  float bestv[32][BMAX];
  int besti[32][BMAX];
  volatile int abort;
  uint64_t full[16], empty[16];
  PhaseInfo phase;
  Geo geo[5];             // this SM's share of q|k|v, o, gate|up, down and the LM head (filled once per launch)
};

struct Ctx {
  const Params &p;
  unsigned char *ring, *xs;
  Shared *sh;
  int sm, G, step;
  unsigned *bar_ctr;
  unsigned bar_target;
  uint32_t slot, par;  // ring slot and mbarrier parity of the next stage (same sequence in producer and consumers)
  uint32_t tag0;       // tag of phase 0 of this launch
  __device__ __forceinline__ uint32_t tag(int phase) const { return ((tag0 + (uint32_t)phase) & 0x7FFFu) | 0x8000u; }
  __device__ __forceinline__ uint32_t seq(int phase) const { return tag0 + (uint32_t)phase + 1u; }  // never 0 in the first launches
  uint32_t push0;      // row-parallel linears pushed by every SM before this launch (tp > 1)
  // arrivals expected once the o_proj (which = 0) / down_proj (which = 1) of layer l has been pushed by all G SMs of a rank
  __device__ __forceinline__ uint32_t arrivals(int l, int which) const { return (push0 + 2u * (uint32_t)l + (uint32_t)which + 1u) * (uint32_t)G; }
  __device__ __forceinline__ void advance() {
    if (++slot == (uint32_t)p.ns) { slot = 0; par ^= 1u; }
  }
  unsigned long long *tr;  // optional fine-grained stamps of the current layer
};

// Grid barrier over all blocks (consumer threads only).  Bounded: on time-out the error flag is set and the block
// stops doing work (every later wait is bounded too), so the kernel always terminates.
__device__ __forceinline__ void grid_sync(Ctx &c) {
  const int tid = threadIdx.x;
  c.bar_target += c.G;
  consumer_sync();
  if (tid == 0) {
    __threadfence();
    atomicAdd(c.bar_ctr, 1u);
    bool ok = false;
    for (int it = 0, lim = 2 * POLL_LIMIT; it < lim; ++it) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(c.bar_ctr) : "memory");
      if (v >= c.bar_target) { ok = true; break; }
      if (c.sh->abort) break;
    }
    if (!ok) {
      c.sh->abort = 1;
      if (c.p.error_flag) atomicCAS(c.p.error_flag, 0, 3);
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

// RMSNorm weights of a phase, requested before the wait for its input so that their latency hides behind it.
struct Gamma { uint4 v[3]; };
__device__ __forceinline__ Gamma load_gamma(const __half *gamma, int K) {
  Gamma g;
#pragma unroll
  for (int q = 0; q < 3; ++q)
    g.v[q] = (gamma && (int)threadIdx.x + q * NCT < K / 8) ? __ldg(reinterpret_cast<const uint4 *>(gamma) + threadIdx.x + q * NCT) : make_uint4(0, 0, 0, 0);
  return g;
}

// Stage activations src[B, K] (global, written by other SMs: read through L2) into shared memory for the next linear phase.
// gamma != nullptr applies RMSNorm first (weights in `gm`), with the reference's fp16 roundings.
//
// INT4 phases multiply on the integer tensor-core path (u8 x s8 -> s32), so the fp16 activations of every 128-k chunk are
// turned into 16-bit block fixed point here: T = round(x * 32000 / max|x| of the chunk), split into two signed bytes
// T = 256 t1 + t2.  t1 and t2 become two columns of the mma's B operand (batch b -> columns 2b and 2b + 1), stored in the
// order in which a lane needs them: [chunk][column][tig][32 bytes].  The quantisation step is 2^-5 of an fp16 ulp of the
// chunk's largest element, so the product differs from the exact fp16 x int4 dot product by far less than the final fp16
// rounding.  The weights stay offset-binary nibbles u = q + 8; sum(q T) = sum(u T) - 8 sum(T) and the second term goes
// into the accumulator's initial value (corr).  The fp16 phase (LM head) keeps x as fp16 in natural order.
// Tensor parallelism: v (eight fp16 values of x) += fp16(sum over ranks, in rank order, of the ranks' fp16 partial sums), so that
// every rank computes the same words.
__device__ __forceinline__ bool add_partial_sums(const uint32_t *parts, int n_parts, uint32_t part_tag, int B, int b, int K, int u, uint4 &v,
                                              const volatile int *abort_flag) {
  bool got = true;
  float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int r0 = 0; r0 < n_parts; r0 += 2) {  // two ranks' words in flight together
    uint4 pa[2], pb[2];
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (r0 + i < n_parts) {
        const uint32_t *w = parts + ((size_t)(r0 + i) * B + b) * K + (size_t)u * 8;
        pa[i] = ld_words(w);
        pb[i] = ld_words(w + 4);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (r0 + i < n_parts) {
        const uint32_t all = pa[i].x & pa[i].y & pa[i].z & pa[i].w & pb[i].x & pb[i].y & pb[i].z & pb[i].w;
        const uint32_t any = pa[i].x | pa[i].y | pa[i].z | pa[i].w | pb[i].x | pb[i].y | pb[i].z | pb[i].w;
        uint4 pv = make_uint4(__byte_perm(pa[i].x, pa[i].y, 0x5410), __byte_perm(pa[i].z, pa[i].w, 0x5410), __byte_perm(pb[i].x, pb[i].y, 0x5410),
                              __byte_perm(pb[i].z, pb[i].w, 0x5410));
        if ((all >> 16) != part_tag || (any >> 16) != part_tag)  // not there yet: wait for this rank's words
          got &= poll8(parts + ((size_t)(r0 + i) * B + b) * K + (size_t)u * 8, part_tag, pv, abort_flag);
        const __half2 *ph = reinterpret_cast<const __half2 *>(&pv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t2 = __half22float2(ph[j]);
          f[2 * j] += t2.x;
          f[2 * j + 1] += t2.y;
        }
      }
  }
  __half *h = reinterpret_cast<__half *>(&v);
#pragma unroll
  for (int j = 0; j < 8; ++j) h[j] = h_add(h[j], __float2half_rn(f[j]));
  return got;
}

// Where a staging step takes its input from.
struct StageSrc {
  const uint32_t *x;        // tagged words [B][K]
  uint32_t x_tag;
  const uint32_t *flags;    // progress words to wait for first: rows x cols (row stride 256), sequence number `want`;
                            // cols == 0: one arrival counter per row instead, `want` arrivals
  int flag_rows, flag_cols;
  uint32_t want;
  const uint2 *ssq_flags;   // non-null: wait on the {sum of squares, sequence} entries of the x producers instead (rows = batch)
  // tensor parallelism: the input is x + the sum over ranks of the partial sums of a row-parallel linear
  const uint32_t *parts;    // [n_parts][B][K] tagged words (nullptr: no partial sums)
  int n_parts;
  uint32_t part_tag;
  uint32_t *x_out;          // where the sum is stored (units u with u % G == sm), tagged x_out_tag; nullptr: nowhere
  uint32_t x_out_tag;
  int lo_unit, hi_unit;     // 8-element units outside [lo_unit, hi_unit) are zero and are not loaded (window of a k slice)
};

template <bool INT4, bool TP>
__device__ __forceinline__ void stage_x(Ctx &c, const StageSrc &src, int K, const __half *gamma, int trace_slot = 0) {
  const Params &p = c.p;
  const int tid = threadIdx.x;
  const int units = K / 8;
  const uint32_t tag = src.x_tag;
  Gamma gm;
  if (!TP) gm = load_gamma(gamma, K);  // requested before the wait, used after it
  unsigned long long *ts = (c.tr && trace_slot && tid == 0) ? c.tr + trace_slot : nullptr;
  if (ts) ts[0] = gtime();
#ifdef PT_MK_TRACE_WAITS
  long long sq[6];
  auto sclk = []() { long long t; asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)); return t; };
  sq[0] = sclk();
  sq[1] = sq[2] = sq[3] = sq[4] = sq[0];
#endif
  // First attempt at this thread's words of batch row 0 right away: an SM that arrives after all producers are done then
  // has its data one round trip earlier.  Words that are not there yet are fetched again after the wait.
  uint4 v[3];
  unsigned have = 0;
#pragma unroll
  for (int q = 0; q < 3; ++q) {
    v[q] = make_uint4(0, 0, 0, 0);
    const int u = tid + q * NCT;
    if (u < units && u >= src.lo_unit && u < src.hi_unit) {
      const uint32_t *w = src.x + (size_t)u * 8;
      const uint4 a = ld_words(w), b4 = ld_words(w + 4);
      const uint32_t all = a.x & a.y & a.z & a.w & b4.x & b4.y & b4.z & b4.w, any = a.x | a.y | a.z | a.w | b4.x | b4.y | b4.z | b4.w;
      if ((all >> 16) == tag && (any >> 16) == tag) {
        v[q] = make_uint4(__byte_perm(a.x, a.y, 0x5410), __byte_perm(a.z, a.w, 0x5410), __byte_perm(b4.x, b4.y, 0x5410), __byte_perm(b4.z, b4.w, 0x5410));
        have |= 1u << q;
      }
    }
  }
  if (tid < 32 && !(src.ssq_flags ? wait_flags_ssq(src.ssq_flags, p.B, src.flag_cols, src.want, K, p.eps, c.sh->stat, &c.sh->abort)
                    : src.flag_cols == 0 ? wait_counters(src.flags, src.flag_rows, src.want, &c.sh->abort)
                                         : wait_flags(src.flags, src.flag_rows, src.flag_cols, src.want, &c.sh->abort))) {
    c.sh->abort = 1;
    if (p.error_flag) atomicCAS(p.error_flag, 0, 10);
  }
  consumer_sync();
  if (ts) ts[1] = gtime();
#ifdef PT_MK_TRACE_WAITS
  sq[1] = sclk();
#endif
  for (int b = 0; b < p.B; ++b) {
    bool got = true;
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const int u = tid + q * NCT;
      if (u >= units || u < src.lo_unit || u >= src.hi_unit) { v[q] = make_uint4(0, 0, 0, 0); continue; }
      if (!(b == 0 && (have >> q & 1))) got &= poll8(src.x + (size_t)b * K + (size_t)u * 8, tag, v[q], &c.sh->abort);
      if (TP && src.n_parts > 0) {
        got &= add_partial_sums(src.parts, src.n_parts, src.part_tag, p.B, b, K, u, v[q], &c.sh->abort);
        if (src.x_out && (u % c.G) == c.sm) {
          const uint32_t *hw = reinterpret_cast<const uint32_t *>(&v[q]);
          const uint32_t t = src.x_out_tag << 16;
          uint32_t *dst = src.x_out + (size_t)b * K + (size_t)u * 8;
          reinterpret_cast<uint4 *>(dst)[0] = make_uint4(t | (hw[0] & 0xFFFFu), t | (hw[0] >> 16), t | (hw[1] & 0xFFFFu), t | (hw[1] >> 16));
          reinterpret_cast<uint4 *>(dst)[1] = make_uint4(t | (hw[2] & 0xFFFFu), t | (hw[2] >> 16), t | (hw[3] & 0xFFFFu), t | (hw[3] >> 16));
        }
      }
    }
    if (!got) {
      c.sh->abort = 1;
      if (p.error_flag) atomicCAS(p.error_flag, 0, 7);
    }
    if (ts && b == 0) ts[2] = gtime();
#ifdef PT_MK_TRACE_WAITS
    if (b == 0) asm volatile("{\n\t.reg .u32 z;\n\tadd.u32 z, %1, %2;\n\tand.b32 z, z, 0;\n\tmov.u64 %0, %%clock64;\n\t}" : "=l"(sq[2]) : "r"(v[0].x), "r"(v[0].w));
#endif
    __half rb = __half(0);
    if (TP) gm = load_gamma(gamma, K);  // tp > 1: requested only now (registers), its latency hides behind the reduction below
    if (gamma && src.ssq_flags) {
      rb = __float2half_rn(c.sh->stat[b]);   // from the producers' statistics, written by warp 0 before the barrier above
    } else if (gamma) {
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
#ifdef PT_MK_TRACE_WAITS
    if (b == 0) asm volatile("{\n\t.reg .u32 z;\n\tadd.u32 z, %1, %1;\n\tand.b32 z, z, 0;\n\tmov.u64 %0, %%clock64;\n\t}" : "=l"(sq[3]) : "r"((uint32_t)__half_as_ushort(rb)));
#endif
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      if (q * NCT >= units) break;  // uniform: nothing left for any thread
      const int u = tid + q * NCT;
      const bool valid = u < units;
      __half *h = reinterpret_cast<__half *>(&v[q]);
      if (gamma && valid) {
        const __half *gh = reinterpret_cast<const __half *>(&gm.v[q]);
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = h_mul(h_mul(h[j], rb), gh[j]);
      }
      if (INT4) {
        // the 16 units of one 128-k chunk are 16 consecutive u, i.e. one half-warp (invalid units hold zeros)
        const uint32_t *hw = reinterpret_cast<const uint32_t *>(&v[q]);
        __half2 mx = __hmax2(__hmax2(u32_as_h2(hw[0] & 0x7FFF7FFFu), u32_as_h2(hw[1] & 0x7FFF7FFFu)),
                             __hmax2(u32_as_h2(hw[2] & 0x7FFF7FFFu), u32_as_h2(hw[3] & 0x7FFF7FFFu)));
        // non-negative fp16 bit patterns order like integers: one integer max-reduction over the half-warp
        const unsigned half_mask = (threadIdx.x & 16) ? 0xFFFF0000u : 0x0000FFFFu;
        const uint32_t mbits = __reduce_max_sync(half_mask, max(h2_as_u32(mx) & 0xFFFFu, h2_as_u32(mx) >> 16));
        const float amax = __half2float(__ushort_as_half((unsigned short)mbits));
        const float inv = amax > 0.f ? __fdividef(32000.0f, amax) : 0.f;
        // U = T + 128 as 16-bit halves of four registers: t1 = high byte of U, t2 = low byte of U xor 0x80
        uint32_t U[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(u32_as_h2(hw[j]));
          const int lo = __float2int_rn(fmaf(f.x, inv, 128.0f)), hi = __float2int_rn(fmaf(f.y, inv, 128.0f));
          U[j] = __byte_perm((uint32_t)lo, (uint32_t)hi, 0x5410);
        }
        // bytes in the order of the packed weight word: k offsets (0,4,1,5) sit in the low nibbles of its bytes 0..3 and
        // (2,6,3,7) in the high nibbles
        const uint32_t t1a = __byte_perm(U[0], U[2], 0x7351), t1b = __byte_perm(U[1], U[3], 0x7351);
        const uint32_t t2a = __byte_perm(U[0], U[2], 0x6240) ^ 0x80808080u, t2b = __byte_perm(U[1], U[3], 0x6240) ^ 0x80808080u;
        int s12 = __dp4a((int)t1a, 0x01010101, __dp4a((int)t1b, 0x01010101, 0)) * 65536 + __dp4a((int)t2a, 0x01010101, __dp4a((int)t2b, 0x01010101, 0));
        s12 = __reduce_add_sync(half_mask, s12);
        if (valid) {
          // words (0,1) of a lane feed its first mma pair, words (2,3) the second; see linear_phase
          const int chunk = u >> 4, r = u & 15, tk = r >> 2, w = r & 3;
          unsigned char *base = c.xs + (size_t)chunk * (p.B * 256) + (size_t)b * 256 + tk * 32 + ((w >> 1) * 4 + (w & 1)) * 4;
          *reinterpret_cast<uint32_t *>(base) = t1a;            // column 2b (t1): low-nibble operand
          *reinterpret_cast<uint32_t *>(base + 8) = t1b;        //                  high-nibble operand
          *reinterpret_cast<uint32_t *>(base + 128) = t2a;      // column 2b + 1 (t2)
          *reinterpret_cast<uint32_t *>(base + 136) = t2b;
          if (r == 0) {
            const int s2 = (int)(short)(s12 & 0xFFFF), s1 = (s12 - s2) >> 16;
            c.sh->corr[chunk][b] = make_int4(-8 * s1, -8 * s2, -8 * s1, -8 * s2);
            c.sh->xscale[chunk][b] = amax * (1.0f / (32000.0f * 16.0f));
          }
        }
      } else if (valid) {
        *reinterpret_cast<uint4 *>(c.xs + (size_t)b * p.xs_stride + u * 16) = v[q];
      }
    }
  }
#ifdef PT_MK_TRACE_WAITS
  sq[4] = sclk();
#endif
  consumer_sync();
#ifdef PT_MK_TRACE_WAITS
  sq[5] = sclk();
  if (c.tr && tid == 0)
    for (int q = 0; q < 5; ++q) atomicAdd(c.tr + 48 + q, (unsigned long long)(sq[q + 1] - sq[q]));
#endif
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

// Finished sums of row tile `rt` of this SM: lane (g, tig) with tig < B holds batch tig, rows g (lo) and g + 8 (hi) of the tile.
// Phases between layers write tagged words; the LM head keeps its arg-max and optionally writes fp16 logits.
template <bool HEAD, bool TP>
__device__ __forceinline__ void tile_epilogue(const Params &p, const volatile PhaseInfo *pi, float lo, float hi, int rt, int lane, Best *best,
                                              float &ssq, const uint32_t *pre = nullptr) {
  const int g = lane >> 2, b = lane & 3;
  if (b >= p.B) return;
  const int epi = pi->epi, N = pi->N;
  const uint32_t tag = pi->tag;
  uint32_t *outw = pi->outw;
  rt += pi->r0;
  if (!HEAD && epi == EPI_SWIGLU) {  // rows g / g + 8 are the gate / up feature rt * 8 + g
    const int n = rt * 8 + g;
    if (n < N / 2) st_word(outw + (size_t)b * pi->out_ld + pi->out_off + n, tag, h_mul(__float2half_rn(hi), swish_h(__float2half_rn(lo))));
    return;
  }
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    const int n = rt * 16 + g + 8 * hr;
    if (n >= N) continue;
    __half y = __float2half_rn(hr ? hi : lo);
    if (HEAD) {
      float f = __half2float(y);
      if (TP && f == 0.f) f = -10000.0f;  // the tensor-parallel LM head reads exact zeros as -10000 (layers/lm_head.py:86-88)
      const int id = TP ? n + p.vocab_off : n;
      if (f > best->v[b] || (f == best->v[b] && id < best->i[b])) { best->v[b] = f; best->i[b] = id; }
      __half *logits = pi->logits;
      if (logits) logits[(size_t)b * N + n] = y;
    } else if (TP && pi->push) {
      // partial sum of a row-parallel linear: one copy into this rank's slot on every rank (the sum and the residual add
      // happen in the next staging step, on every rank alike)
      const uint32_t word = (tag << 16) | (uint32_t)__half_as_ushort(y);
      const size_t at = pi->push_slot + (size_t)b * N + n;
      for (int r = 0; r < p.tp; ++r) st_sys(p.peer_part[r] + at, word);
    } else {
      uint32_t *w = outw + (size_t)b * N + n;
      // the residual is the value this SM wrote to the same word one or two phases ago (or the embedding, which the first
      // staging of this launch has already seen complete)
      if (epi == EPI_RESID) {
        y = h_add(__ushort_as_half((unsigned short)((pre ? pre[hr] : ld_word(w)) & 0xFFFFu)), y);
        const float yf = __half2float(y);
        ssq = fmaf(yf, yf, ssq);   // this lane's share of sum(x^2) of its batch row, for the RMSNorm of the next staging
      }
      st_word(w, tag, y);
    }
  }
}

__device__ __forceinline__ void imma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma0(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {  // d = a b
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// d = a b + {c0, c1, c0, c1}: both rows of the lane start from the same per-column initialiser
__device__ __forceinline__ void imma_c(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, int c0, int c1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
}

// One tile in registers: the lane's 16 bytes of rows g (a) and g + 8 (b), and the two rows' group scales (INT4).
struct TileRegs { uint4 a, b; uint32_t s; };

// One linear phase over this SM's row tiles [r0, r1) of a matrix with `nchunks` tiles per row tile.  The SM's tiles arrive
// in "stream order": stage j holds tile start(w) + j of every warp w that still has one (see pt_llama_stream_permute), so
// each warp accumulates a contiguous run of chunks in registers and there is no synchronisation inside the phase.  Row
// tiles that are split between warps are summed after one barrier, in warp order (deterministic).
// The loop body is what bounds the kernel once the stream flows, so it is kept to the instructions that the arithmetic
// needs: two AND per packed word and one integer mma per 512 weights (INT4), operands and accumulator initialisers that
// arrive from shared memory in fragment order, ring positions advanced without divisions.
#ifdef PT_MK_TRACE_WAITS
constexpr bool NOMATH = true;   // diagnostics build: bit 0 of `debug` skips the tile math, waits are timed
constexpr int TRS = 64;         // trace slots per (SM, layer)
#else
constexpr bool NOMATH = false;
constexpr int TRS = 32;
#endif
template <int WFMT, bool TP>
__device__ __forceinline__ void linear_phase(Ctx &c, int mat, int nchunks, Best *best) {
  constexpr int TILE = WTraits<WFMT>::kTileBytes;
  constexpr bool I4 = (WFMT == PT_W_INT4);
  const Params &p = c.p;
  const volatile PhaseInfo *pi = &c.sh->phase;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tig = lane & 3;
#ifdef PT_MK_TRACE_WAITS
  long long pq[6];
  auto pclk = []() { long long t; asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)); return t; };
  pq[0] = pclk();
#endif
  const Geo &geo = c.sh->geo[mat];
  const int r0 = geo.r0, m = geo.m;
  Split sp(0);
  sp.base = geo.base;
  sp.rem = geo.rem;
  const int len = sp.len(warp), nstages = sp.stages();
  const int first_rt = geo.first_rt[warp];
  int rt = first_rt, ch = geo.ch0[warp];
  const bool enters_midway = ch != 0;  // another warp holds the beginning of this warp's first row tile
  float acc0 = 0.f, acc1 = 0.f;
  float ssq = 0.f;   // sum of squares of the x values this lane's epilogues write (residual phases)
  const uint32_t ring_s = smem_addr(c.ring) + warp * TILE + lane * 16;
  const uint32_t full_s = smem_addr(&c.sh->full[0]), empty_s = smem_addr(&c.sh->empty[0]);
  // Per-lane operand addresses: base + chunk * stride, with stride 0 and the zero block for lanes that carry no batch column
  // (every lane loads unconditionally: a conditional load would turn the operand registers into values that live across
  // the loop iterations, and this loop has no registers to spare).
  uint32_t x_s, x_cs, corr_s, corr_cs, xsc_s;
  {
    const uint32_t zero_s = smem_addr(&c.sh->zeros[0]);
    if (I4) {
      const bool has = g < 2 * p.B;
      x_s = has ? smem_addr(c.xs) + g * 128 + tig * 32 : zero_s;
      x_cs = has ? p.B * 256 : 0;
      corr_s = tig < p.B ? smem_addr(&c.sh->corr[0][tig]) : zero_s;
      corr_cs = tig < p.B ? (uint32_t)sizeof(int4) * BMAX : 0;
      xsc_s = smem_addr(&c.sh->xscale[0][tig < p.B ? tig : 0]);
    } else {
      const bool has = !(g & 1) && (g >> 1) < p.B;   // batch b sits in column 2b, so that lane tig = b ends up with its sums
      x_s = has ? smem_addr(c.xs) + (g >> 1) * p.xs_stride + tig * 16 : zero_s;
      x_cs = has ? 64 : 0;
      corr_s = corr_cs = xsc_s = 0;
    }
  }

  // Residual words of the row tile whose sum this warp will finish after the loop (row tiles shared by several warps, the usual
  // case of the residual phases): requested now, so that their round trip is not at the end of the phase.
  uint32_t pre[2] = {0u, 0u};
  bool has_pre = false;
  if (I4 && pi->epi == EPI_RESID && !(TP && pi->push) && warp < m && tig < p.B) {
    const uint32_t *w = pi->outw + (size_t)tig * pi->N + (size_t)(r0 + warp) * 16 + g;
    pre[0] = ld_word(w);
    pre[1] = ld_word(w + 8);
    has_pre = true;
  }
  auto store_partial = [&](int slot) { *reinterpret_cast<float2 *>(&c.sh->red[warp][slot][lane][0]) = make_float2(acc0, acc1); };
  auto load_tile = [&](uint32_t t_s, TileRegs &t) {
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(t.a.x), "=r"(t.a.y), "=r"(t.a.z), "=r"(t.a.w) : "r"(t_s));
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(t.b.x), "=r"(t.b.y), "=r"(t.b.z), "=r"(t.b.w) : "r"(t_s + 512));
    if (I4) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(t.s) : "r"(t_s - lane * 16 + 1024 + g * 4));
  };
  // End of a tile: the chunk counter moves on; at the end of a row tile its sum is finished (or parked, when another warp
  // holds the row tile's beginning).
  auto next_chunk = [&]() {
    if (++ch == nchunks) {  // this warp reached the end of row tile rt
      if (rt == first_rt && enters_midway) store_partial(0);
      else tile_epilogue<!I4, TP>(p, pi, acc0, acc1, rt, lane, best, ssq);  // had all of it
      ch = 0;
      ++rt;
      acc0 = acc1 = 0.f;
    }
  };
  constexpr uint32_t LO = 0x0F0F0F0Fu, HI = 0xF0F0F0F0u;
  // value x 16 = 4096 lo(t1) + 16 lo(t2) + 256 hi(t1) + hi(t2); |.| < 2^31 for |t1| <= 125 (see stage_x)
  auto fold = [&](const int (&lo)[4], const int (&hi)[4], uint32_t s, float xs) {
    const int v0 = ((lo[0] << 8) + lo[1]) * 16 + (hi[0] << 8) + hi[1];
    const int v1 = ((lo[2] << 8) + lo[3]) * 16 + (hi[2] << 8) + hi[3];
    const float2 sf = __half22float2(u32_as_h2(s));
    acc0 = fmaf(sf.x * xs, (float)v0, acc0);
    acc1 = fmaf(sf.y * xs, (float)v1, acc1);
  };
  // The activation-side operands of one tile: the chunk's two 16-byte B-operand pieces, the accumulator initialiser
  // {-8 sum(t1), -8 sum(t2)} and the chunk's scale.  They do not depend on the weight stream, so they are requested BEFORE the
  // wait for the stage and their latency hides behind it.
  struct XOps { uint4 x0, x1; int c0, c1; float xs; };
  auto load_xops = [&](int chunk, XOps &o) {
    const uint32_t xaddr = x_s + chunk * x_cs;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(o.x0.x), "=r"(o.x0.y), "=r"(o.x0.z), "=r"(o.x0.w) : "r"(xaddr));
    if (I4) {
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(o.x1.x), "=r"(o.x1.y), "=r"(o.x1.z), "=r"(o.x1.w) : "r"(xaddr + 16));
      asm volatile("ld.shared.v2.s32 {%0,%1}, [%2];" : "=r"(o.c0), "=r"(o.c1) : "r"(corr_s + chunk * corr_cs));
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(o.xs) : "r"(xsc_s + chunk * (uint32_t)(sizeof(float) * BMAX)));
    }
  };
  // One tile (the last of an odd-length range, and the fp16 tiles of the LM head).
  auto compute = [&](const TileRegs &t, const XOps &o) {
    if (NOMATH && (p.debug & 1)) return;
    if (I4) {
      int lo[4], hi[4];
      imma0(hi, t.a.x & HI, t.b.x & HI, t.a.y & HI, t.b.y & HI, o.x0.z, o.x0.w);
      imma_c(lo, t.a.x & LO, t.b.x & LO, t.a.y & LO, t.b.y & LO, o.x0.x, o.x0.y, o.c0, o.c1);
      imma(hi, t.a.z & HI, t.b.z & HI, t.a.w & HI, t.b.w & HI, o.x1.z, o.x1.w);
      imma(lo, t.a.z & LO, t.b.z & LO, t.a.w & LO, t.b.w & LO, o.x1.x, o.x1.y);
      fold(lo, hi, t.s, o.xs);
    } else {
      float cc[4] = {acc0, 0.f, acc1, 0.f};
      mma16816(cc, t.a.x, t.b.x, t.a.y, t.b.y, o.x0.x, o.x0.y);
      mma16816(cc, t.a.z, t.b.z, t.a.w, t.b.w, o.x0.z, o.x0.w);
      acc0 = cc[0];
      acc1 = cc[2];
    }
    next_chunk();
  };
#ifdef PT_MK_TRACE_WAITS
  pq[1] = pclk();
  // diagnostics build: SM-cycle accounting of the loop of one sample warp, per matrix (wait for the stage / operand loads + math)
  const int dw = (warp == 5 && mat < 4) ? mat : -1;
  unsigned long long *dslot = (c.tr && dw >= 0 && lane == 0) ? c.tr + 32 + 4 * dw : nullptr;
  auto clk = []() { long long t; asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)); return t; };
#endif
  // Stage j / 2 of this phase holds tiles j and j + 1 of this warp's range.  The first tile is multiplied while the second is on
  // its way to the registers; the stage is handed back to the producer as soon as the second tile's loads are issued.
  // (Measured on B200: multiplying the two tiles as interleaved mma chains, or requesting the activation operands before the
  // wait, is 7-10 % slower per step than this plain order, with or without register spills.)
  for (int j = 0; j < nstages; j += 2) {
    const bool first = j < len, second = j + 1 < len;
    XOps oa, ob;
#ifdef PT_MK_TRACE_WAITS
    const unsigned long long t_w = (c.tr && tid == 0) ? gtime() : 0ull;
    const long long c0 = clk();
#endif
    const bool got = mbar_wait(full_s + c.slot * 8, c.par, &c.sh->abort);
#ifdef PT_MK_TRACE_WAITS
    if (c.tr && tid == 0) c.tr[23] += gtime() - t_w;   // time this phase's consumer spent waiting for the weight stream
    const long long c1 = clk();
#endif
    if (!got) {
      c.sh->abort = 1;
      if (lane == 0 && p.error_flag) atomicCAS(p.error_flag, 0, 4);
    }
    const uint32_t t_s = ring_s + c.slot * STAGE_BYTES;
    TileRegs ta, tb;
    if (first && got) {
      load_tile(t_s, ta);
      load_xops(ch, oa);
      compute(ta, oa);
    }
    if (second && got) load_tile(t_s + NCW * TILE, tb);
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_s + c.slot * 8);
    c.advance();
    if (second && got) {
      load_xops(ch, ob);
      compute(tb, ob);
    }
#ifdef PT_MK_TRACE_WAITS
    long long c3;
    asm volatile("{\n\t.reg .u32 z;\n\tadd.u32 z, %1, %2;\n\tand.b32 z, z, 0;\n\tmov.u64 %0, %%clock64;\n\t}" : "=l"(c3) : "r"(__float_as_uint(acc0)), "r"(__float_as_uint(acc1)));
    if (dslot) {
      atomicAdd(dslot + 0, (unsigned long long)(c1 - c0));
      atomicAdd(dslot + 2, (unsigned long long)(c3 - c1));
      atomicAdd(dslot + 3, 1ull);
    }
#endif
  }
#ifdef PT_MK_TRACE_WAITS
  pq[2] = pclk();
#endif
  if (len > 0 && ch != 0) store_partial(rt == first_rt ? 0 : 1);  // the range ended inside a row tile
  consumer_sync();
#ifdef PT_MK_TRACE_WAITS
  pq[3] = pclk();
#endif
  // ---- row tiles shared by several warps: warp (r % NCW) sums the pieces in warp order
  for (int r = warp; r < m; r += NCW) {
    int w_lo, w_hi;
    if (r < GEO_RT) {
      w_lo = geo.w_lo[r];
      w_hi = geo.w_hi[r];
    } else {
      const int q0 = r * nchunks;
      w_lo = sp.owner(q0);
      w_hi = sp.owner(q0 + nchunks - 1);
    }
    if (w_lo == w_hi) continue;  // one warp had the whole row tile and already wrote it
    float v0 = 0.f, v1 = 0.f;
    for (int w = w_lo; w <= w_hi; ++w) {
      const int s_w = (geo.first_rt[w] == r) ? 0 : 1;  // r is the first row tile of w's range, or its last
      const float2 t = *reinterpret_cast<const float2 *>(&c.sh->red[w][s_w][lane][0]);
      v0 += t.x;
      v1 += t.y;
    }
    tile_epilogue<!I4, TP>(p, pi, v0, v1, r, lane, best, ssq, (has_pre && r == warp) ? pre : nullptr);
  }
#ifdef PT_MK_TRACE_WAITS
  pq[4] = pclk();
#endif
  const bool makes_x = I4 && pi->epi == EPI_RESID && !(TP && pi->push);
  if (makes_x) {  // lanes (g, tig) of a warp hold batch row tig: sum over g, lanes 0 .. B-1 keep the warp's sums
    float v = ssq;
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 16);
    if (lane < p.B) c.sh->wssq[warp][lane] = v;
  }
  if (pi->out_seq) {  // tell the other SMs (of every rank, for pushed partial sums) that this SM's rows of the phase are written
    consumer_sync();
    if (TP && pi->push) {
      if (tid < p.tp) red_add_sys(p.peer_flag[tid] + p.rank * 256, 1u);
    } else if (tid == 0) {
      if (makes_x)
        for (int b = 0; b < p.B; ++b) {
          float t = 0.f;
#pragma unroll
          for (int w = 0; w < NCW; ++w) t += c.sh->wssq[w][b];
          st_tagged(p.flag_ssq + b * 256 + c.sm, __float_as_uint(t), pi->out_seq);
        }
      st_flag(p.flag_sm + c.sm, pi->out_seq);
    }
  }
#ifdef PT_MK_TRACE_WAITS
  pq[5] = pclk();
  if (c.tr && tid == 0)
    for (int q = 0; q < 5; ++q) atomicAdd(c.tr + 56 + q, (unsigned long long)(pq[q + 1] - pq[q]));
#endif
}

// RoPE (rotate_half form) on elements i and i + H/2 of one head vector -> dst (shared), reference fp16 roundings.
__device__ __forceinline__ void rope_pair(__half a, __half b, __half s, __half co, int i, __half *dst) {
  dst[i] = h_add(h_mul(a, co), h_mul(__hneg(b), s));
  dst[i + H / 2] = h_add(h_mul(b, co), h_mul(a, s));
}
__device__ __forceinline__ void group_sync(int grp) { asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory"); }

// Attention phase.  Units (b, head, page) are dealt round-robin to the SMs (unit u -> SM u % G); the producer has queued
// one stage per unit that has cached tokens (K page at offset 0, V page at V_OFFSET).  The consumer warps form NGRP
// groups of four warps; group q handles this SM's units q, q + NGRP, ... on its own (scores with 8 lanes per token, softmax
// statistics by warp shuffles, P.V with one thread per channel), so units of an SM run concurrently.
__device__ __forceinline__ void attention_phase(Ctx &c, const pt_llama_layer &L, uint32_t qkv_tag, uint32_t attn_tag, uint32_t attn_seq) {
  const Params &p = c.p;
  Shared *sh = c.sh;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gt = tid & 127;
  const int grp = (warp >> 2) < NGRP ? (warp >> 2) : -1;  // warps beyond the last full group only release stages
  const int step = c.step, n_active = step / PAGE + 1;
  const int n_units = p.B * p.n_head * n_active;
  const int row_elems = 3 * p.dq;
  const __half *sin_r = p.sin_t + (size_t)step * (H / 2), *cos_r = p.cos_t + (size_t)step * (H / 2);
  for (int u0 = c.sm; u0 < n_units; u0 += MAXU * c.G) {
    const int nu = min(MAXU, (n_units - u0 + c.G - 1) / c.G);  // units of this pass: u0 + k G
    if (tid < nu) {  // page-table entries of the pass, requested now so that their latency hides behind the poll below
      const int u = u0 + tid * c.G;
      sh->phys[tid] = p.page_table[(size_t)(u / (n_active * p.n_head)) * p.max_pages + u % n_active];
    }
    // ---- q (and the new token's k, v) of every unit in one go.  The words carry the tag of this layer's QKV phase; all six
    // loads of a thread are in flight together, so once the producing SMs are done this costs one L2 round trip.
    {
      const int k = tid >> 6, i = tid & 63;
      if (k < nu) {
        const int u = u0 + k * c.G;
        const int pg = u % n_active, head = (u / n_active) % p.n_head, b = u / (n_active * p.n_head);
        const bool owner = (pg == n_active - 1);
        const uint32_t *qw = p.qkvw + (size_t)b * row_elems + (size_t)head * H + i;
        const __half rs = sin_r[i], rc = cos_r[i];  // requested before the poll: their latency hides behind it
        uint32_t w[6];
        bool got = false;
        for (int it = 0; it < POLL_LIMIT && !got; ++it) {
          w[0] = ld_word(qw);
          w[1] = ld_word(qw + H / 2);
          w[2] = owner ? ld_word(qw + p.dq) : w[0];
          w[3] = owner ? ld_word(qw + p.dq + H / 2) : w[0];
          w[4] = owner ? ld_word(qw + 2 * p.dq) : w[0];
          w[5] = owner ? ld_word(qw + 2 * p.dq + H / 2) : w[0];
          const uint32_t all = w[0] & w[1] & w[2] & w[3] & w[4] & w[5], any = w[0] | w[1] | w[2] | w[3] | w[4] | w[5];
          got = (all >> 16) == qkv_tag && (any >> 16) == qkv_tag;
          if ((it & 63) == 63 && sh->abort) break;
        }
        if (!got) {
          sh->abort = 1;
          if (p.error_flag) atomicCAS(p.error_flag, 0, 8);
        }
        auto val = [&](int j) { return __ushort_as_half((unsigned short)(w[j] & 0xFFFFu)); };
        rope_pair(val(0), val(1), rs, rc, i, sh->qs[k]);
        if (owner) {
          rope_pair(val(2), val(3), rs, rc, i, sh->newk[k]);
          sh->newv[k][i] = val(4);
          sh->newv[k][i + 64] = val(5);
        }
      }
    }
    consumer_sync();
    if (c.tr && tid == 0 && u0 == c.sm) c.tr[13] = gtime();
    // The units of the pass one after the other, each with all consumer warps (an SM has two or three units at the sizes
    // this kernel is for, and a unit is a chain of short steps, so width beats concurrency).
    for (int k = 0; k < nu; ++k) {
      const int u = u0 + k * c.G;
      const int pg = u % n_active, head = (u / n_active) % p.n_head, b = u / (n_active * p.n_head);
      const int n_valid = min(PAGE, step + 1 - pg * PAGE);
      const bool owner = (pg == n_active - 1);
      const int n_load = owner ? n_valid - 1 : n_valid;  // tokens that come from the pool (units without any have no stage)
      const uint32_t slot = c.slot;
      const __half *Ks = nullptr, *Vs = nullptr;
      if (n_load > 0) {
        if (!mbar_wait(smem_addr(&sh->full[slot]), c.par, &sh->abort)) {
          sh->abort = 1;
          if (lane == 0 && p.error_flag) atomicCAS(p.error_flag, 0, 5);
        }
        if (c.tr && tid == 0 && k == 0) c.tr[15] = gtime();
        Ks = reinterpret_cast<const __half *>(c.ring + (size_t)slot * STAGE_BYTES);
        Vs = reinterpret_cast<const __half *>(c.ring + (size_t)slot * STAGE_BYTES + V_OFFSET);
        c.advance();
      }
      if (owner && tid < H && !sh->abort) {  // append the new token to the pool
        const int phys = sh->phys[k];
        __half *gK = (__half *)L.pool + (((size_t)phys * 2 + 0) * p.n_head + head) * PAGE * H + (size_t)(n_valid - 1) * H;
        __half *gV = (__half *)L.pool + (((size_t)phys * 2 + 1) * p.n_head + head) * PAGE * H + (size_t)(n_valid - 1) * H;
        gK[tid] = sh->newk[k][tid];
        gV[tid] = sh->newv[k][tid];
      }
      // scores: 8 lanes per cached token, all 64 tokens of the page at once
      float *ps = sh->ps[0];
#pragma unroll
      for (int tb = 0; tb < PAGE; tb += NCT / 8) {   // one pass with 16 consumer warps
        const int sub = lane & 7, t = tb + (tid >> 3);
        float sc0 = 0.f, sc1 = 0.f;
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
              sc0 = fmaf(a.x, q2.x, sc0);
              sc1 = fmaf(a.y, q2.y, sc1);
            }
          }
        }
        float sc = sc0 + sc1;
        sc += __shfl_xor_sync(0xffffffffu, sc, 1);
        sc += __shfl_xor_sync(0xffffffffu, sc, 2);
        sc += __shfl_xor_sync(0xffffffffu, sc, 4);
        if (sub == 0 && t < n_valid) ps[t] = __half2float(h_mul(__float2half_rn(sc), p.score_scale));
      }
      consumer_sync();
      if (c.tr && tid == 0 && k == 0) c.tr[16] = gtime();
      // softmax statistics of the page (fp32, like the reference's cast before SoftmaxV3): every warp works them out for
      // itself (same values), which saves a barrier and a single-warp section
      float *pw = sh->pw[warp];
      float m, l;
      {
        const float s0 = lane < n_valid ? ps[lane] : -INFINITY, s1 = lane + 32 < n_valid ? ps[lane + 32] : -INFINITY;
        m = warp_max(fmaxf(s0, s1));
        const float e0 = lane < n_valid ? expf(s0 - m) : 0.f, e1 = lane + 32 < n_valid ? expf(s1 - m) : 0.f;
        pw[lane] = e0;
        pw[lane + 32] = e1;
        l = warp_sum(e0 + e1);
      }
      __syncwarp();
      if (c.tr && tid == 0 && k == 0) c.tr[17] = gtime();
      // P.V: warp w takes tokens w, w + 16, ...; lane takes channels 4 lane .. 4 lane + 3; the 16 partial sums meet in shared
      // memory in warp order
      float *part = reinterpret_cast<float *>(&sh->red[0][0][0][0]);  // [NCW][H]; red is idle during attention
      {
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        if (!sh->abort) {
#pragma unroll
          for (int j = 0; j < (PAGE + NCW - 1) / NCW; ++j) {
            const int t = warp + NCW * j;
            if (t < n_valid) {
              const uint2 raw = *reinterpret_cast<const uint2 *>((t < n_load ? Vs + (size_t)t * H : sh->newv[k]) + 4 * lane);
              const float2 v01 = __half22float2(u32_as_h2(raw.x)), v23 = __half22float2(u32_as_h2(raw.y));
              const float e = pw[t];
              o[0] += e * v01.x; o[1] += e * v01.y; o[2] += e * v23.x; o[3] += e * v23.y;
            }
          }
        }
        *reinterpret_cast<float4 *>(part + warp * H + 4 * lane) = make_float4(o[0], o[1], o[2], o[3]);
      }
      consumer_sync();  // everyone is done with the stage
      if (c.tr && tid == 0 && k == 0) c.tr[18] = gtime();
      if (n_load > 0 && lane == 0) mbar_arrive(smem_addr(&sh->empty[slot]));
      if (tid < H) {  // publish this page's partial result as tagged words; the unit of the head's last page collects them (below)
        const size_t hd = (size_t)b * p.n_head + head;
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < NCW; ++w) o += part[w * H + tid];
        st_tagged(&p.ws_o[(hd * p.max_pages + pg) * H + tid], __float_as_uint(o), attn_tag);
        if (tid == 0) {
          st_tagged(&p.ws_ml[(hd * p.max_pages + pg) * 2 + 0], __float_as_uint(m), attn_tag);
          st_tagged(&p.ws_ml[(hd * p.max_pages + pg) * 2 + 1], __float_as_uint(l), attn_tag);
        }
      }
      consumer_sync();  // part / ps are reused by the next unit
      if (c.tr && tid == 0 && k == 0) c.tr[19] = gtime();
    }
    if (c.tr && tid == 0 && u0 == c.sm) c.tr[14] = gtime();
    consumer_sync();
  }
  // ---- combine: the SM that had the last page of a (sequence, head) sums that head's pages in page order.  This comes
  // after all of the SM's own pages, so producing a partial result never waits for a combine (no circular waits between SMs).
  {
    int idx = 0;
    for (int u = c.sm; u < n_units; u += c.G) {
      const int pg = u % n_active, head = (u / n_active) % p.n_head, b = u / (n_active * p.n_head);
      if (pg != n_active - 1) continue;
      if ((idx++ % NGRP) != grp) continue;
      const size_t hd = (size_t)b * p.n_head + head;
      const int tq = warp & 3;
      float *wts = sh->ps[grp];  // [0, 32): w_i = exp(m_i - M), [32, 64): l_i w_i of up to 32 pages at a time
      bool got = true;
      if (tq == 0) {  // pass 1: M = max over pages
        float M = -INFINITY;
        for (int i0 = 0; i0 < n_active; i0 += 32) {
          float v = -INFINITY;
          if (i0 + lane < n_active) {
            uint32_t bits;
            got &= poll_tagged(&p.ws_ml[(hd * p.max_pages + i0 + lane) * 2 + 0], attn_tag, bits, &sh->abort);
            v = __uint_as_float(bits);
          }
          M = fmaxf(M, warp_max(v));
        }
        if (lane == 0) sh->ml[grp][0] = M;
      }
      group_sync(grp);
      const float M = sh->ml[grp][0];
      float Lsum = 0.f, o = 0.f;
      constexpr int CB = 6;  // pages whose partial outputs are fetched together
      for (int i0 = 0; i0 < n_active; i0 += 32) {
        if (i0) group_sync(grp);
        if (tq == 0 && i0 + lane < n_active) {
          uint32_t mb, lb;   // already seen complete in pass 1 (same lane, same page); the two loads go out together
          const uint2 a0 = ld_tagged(&p.ws_ml[(hd * p.max_pages + i0 + lane) * 2 + 0]), a1 = ld_tagged(&p.ws_ml[(hd * p.max_pages + i0 + lane) * 2 + 1]);
          mb = a0.x;
          lb = a1.x;
          if (a0.y != attn_tag) got &= poll_tagged(&p.ws_ml[(hd * p.max_pages + i0 + lane) * 2 + 0], attn_tag, mb, &sh->abort);
          if (a1.y != attn_tag) got &= poll_tagged(&p.ws_ml[(hd * p.max_pages + i0 + lane) * 2 + 1], attn_tag, lb, &sh->abort);
          const float w = expf(__uint_as_float(mb) - M);
          wts[lane] = w;
          wts[32 + lane] = __uint_as_float(lb) * w;
        }
        group_sync(grp);
        const int n_here = min(32, n_active - i0);
        for (int j0 = 0; j0 < n_here; j0 += CB) {
          uint32_t ov[CB];
          bool all = false;
          for (int it = 0; it < POLL_LIMIT && !all; ++it) {
            all = true;
#pragma unroll
            for (int j = 0; j < CB; ++j)
              if (j0 + j < n_here) {
                const uint2 w2 = ld_tagged(&p.ws_o[(hd * p.max_pages + i0 + j0 + j) * H + gt]);
                ov[j] = w2.x;
                all &= (w2.y == attn_tag);
              }
            if ((it & 63) == 63 && sh->abort) break;
          }
          got &= all;
#pragma unroll
          for (int j = 0; j < CB; ++j)
            if (j0 + j < n_here) {
              Lsum += wts[32 + j0 + j];
              o += __uint_as_float(ov[j]) * wts[j0 + j];
            }
        }
      }
      if (!got) {
        sh->abort = 1;
        if (p.error_flag) atomicCAS(p.error_flag, 0, 9);
      }
      st_word(p.attnw + (size_t)b * p.dq + (size_t)head * H + gt, attn_tag, __float2half_rn(o / Lsum));
      group_sync(grp);  // ps / ml may be reused by the group's next combine; the head's words are all issued
      if (gt == 0) st_flag(p.flag_head + hd, attn_seq);
    }
  }
  consumer_sync();
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
  unsigned long long *tr;  // optional stamps of the layer being pushed: [27] += time blocked on a full ring, [31] = layer pushed
  // The loop below competes with the consumer warps for issue slots, so it is kept to a handful of instructions per stage:
  // no divisions, all addresses incremental.  One stage: `bytes` from src at offset 0 and, for attention stages, `bytes2`
  // from src2 at V_OFFSET.
  __device__ __forceinline__ void push(const void *src, uint32_t bytes, const void *src2, uint32_t bytes2) {
#ifdef PT_MK_TRACE_WAITS
    const unsigned long long t_w = tr ? gtime() : 0ull;
#endif
    if (!first_round && !mbar_wait(empty_s + slot * 8, parity, &sh->abort)) {
      if (ok && p.error_flag) atomicCAS(p.error_flag, 0, 6);
      ok = false;
      sh->abort = 1;
    }
#ifdef PT_MK_TRACE_WAITS
    if (tr) tr[27] += gtime() - t_w;
#endif
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
    for (int u0 = sm; u0 < n_units && ok; u0 += MAXU * G) {
      // the page-table entries of a pass first (independent loads, one round trip), then the copies
      int phys[MAXU];
#pragma unroll
      for (int k = 0; k < MAXU; ++k) {
        const int u = u0 + k * G;
        phys[k] = u < n_units ? p.page_table[(size_t)(u / (n_active * p.n_head)) * p.max_pages + u % n_active] : 0;
      }
#pragma unroll
      for (int k = 0; k < MAXU; ++k) {
        const int u = u0 + k * G;
        if (u < n_units && ok) {
          const int pg = u % n_active, head = (u / n_active) % p.n_head;
          const int n_valid = min(PAGE, step + 1 - pg * PAGE);
          const int n_load = (pg == n_active - 1) ? n_valid - 1 : n_valid;
          if (n_load > 0) {
            const __half *gK = (const __half *)L.pool + (((size_t)phys[k] * 2 + 0) * p.n_head + head) * PAGE * H;
            const __half *gV = (const __half *)L.pool + (((size_t)phys[k] * 2 + 1) * p.n_head + head) * PAGE * H;
            push(gK, (uint32_t)n_load * H * 2, gV, (uint32_t)n_load * H * 2);
          }
        }
      }
    }
  }
};
template <bool TP>
__global__ void __launch_bounds__(THREADS, 1) llama_step_kernel(const Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char *ring = smem;
  unsigned char *xs = smem + (size_t)p.ns * STAGE_BYTES;
  Shared *sh = reinterpret_cast<Shared *>(xs + (((size_t)p.B * p.xs_stride + 127) / 128) * 128);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int step = *p.step;
  // Every block takes the same decision here: the words it depends on are only written at the very end of a launch.
  if (p.done_flag && __ldcg(p.done_flag)) return;  // early stop: every sequence had produced its eos id before the previous step
  if (step < 0 || step >= p.max_len) {             // no position left in the id container / RoPE tables / page table
    if (tid == 0 && p.error_flag) atomicCAS(p.error_flag, 0, 12);
    return;
  }

  if (tid == 0) {
    for (int s = 0; s < p.ns; ++s) {
      mbar_init(smem_addr(&sh->full[s]), 1);
      mbar_init(smem_addr(&sh->empty[s]), NCW);
    }
    sh->abort = 0;
    sh->zeros[0] = sh->zeros[1] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int n_rt_qkv = 3 * p.dq / 16, n_rt_o = p.d / 16, n_rt_gu = 2 * p.ffn_valid / 16, n_rt_head = (p.vocab + 15) / 16;
  const int nc_d = p.d / 128, nc_q = p.dq / 128, nc_f = p.ffn / 128, nc_head = p.d / 32;

  if (warp == NCW) {
    // ---------------- producer: one lane walks the whole step's weight / KV stream of this SM
    if (lane == 0) {
      Producer pr{p, sh, (int)blockIdx.x, (int)gridDim.x, 0, 0u, true, smem_addr(ring), smem_addr(&sh->full[0]), smem_addr(&sh->empty[0]), true, nullptr};
      for (int l = 0; l < p.n_layer; ++l) {
        const pt_llama_layer &L = p.layers[l];
#ifdef PT_MK_TRACE_WAITS
        if (p.trace) {
          if (pr.tr) pr.tr[31] = gtime();
          pr.tr = p.trace + ((size_t)blockIdx.x * p.n_layer + l) * TRS;
          pr.tr[27] = 0ull;
        }
#endif
        pr.push_matrix((const unsigned char *)L.qkv, n_rt_qkv, nc_d, TILE_I4);
        pr.push_attention(L, step);
        pr.push_matrix((const unsigned char *)L.o, n_rt_o, nc_q, TILE_I4);
        pr.push_matrix((const unsigned char *)L.gu, n_rt_gu, nc_d, TILE_I4);
        pr.push_matrix((const unsigned char *)L.down, n_rt_o, nc_f, TILE_I4);
      }
#ifdef PT_MK_TRACE_WAITS
      if (pr.tr) pr.tr[31] = gtime();
      pr.tr = nullptr;
#endif
      pr.push_matrix(p.head, n_rt_head, nc_head, TILE_F16);
    }
    return;
  }
  // ---------------- consumers
  // Two barrier counters are used by alternate launches: word [2] says which one is this launch's (it is zero: the
  // previous launch cleared it when it finished); the last block clears the other one at the very end.
  const unsigned which = __ldcg(p.barrier + 2) & 1u;
  // Word [3] counts launches; it numbers the tags of this launch (block 0 advances it after the final barrier).
  const int n_phases = 5 * p.n_layer + 1;  // phase 0: embedding; layer l: 1 + 5 l + {0 qkv, 1 attention, 2 o, 3 gate|up, 4 down}
  const uint32_t launches = __ldcg(p.barrier + 3);
  Ctx c{p, ring, xs, sh, (int)blockIdx.x, (int)gridDim.x, step, p.barrier + which, 0u, 0u, 0u, launches * (uint32_t)n_phases,
        launches * 2u * (uint32_t)p.n_layer, nullptr};

  // this SM's share of every matrix and the warps' tile ranges inside it
  {
    const int n_rt_of[5] = {n_rt_qkv, n_rt_o, n_rt_gu, n_rt_o, n_rt_head};
    const int nch_of[5] = {nc_d, nc_q, nc_d, nc_f, nc_head};
    if (tid < 5) {
      Geo &gq = sh->geo[tid];
      const int a0 = (int)((long long)blockIdx.x * n_rt_of[tid] / (int)gridDim.x), a1 = (int)((long long)(blockIdx.x + 1) * n_rt_of[tid] / (int)gridDim.x);
      const Split sq((a1 - a0) * nch_of[tid]);
      gq.r0 = a0; gq.m = a1 - a0; gq.base = sq.base; gq.rem = sq.rem;
    }
    consumer_sync();
    if (tid < 5 * NCW) {
      const int k = tid / NCW, w = tid - k * NCW;
      Geo &gq = sh->geo[k];
      Split sq(0);
      sq.base = gq.base; sq.rem = gq.rem;
      const int st = sq.start(w), fr = st / nch_of[k];
      gq.first_rt[w] = (short)fr;
      gq.ch0[w] = (short)(st - fr * nch_of[k]);
    } else if (tid >= 128 && tid < 128 + 5 * GEO_RT) {
      const int k = (tid - 128) / GEO_RT, r = (tid - 128) - k * GEO_RT;
      Geo &gq = sh->geo[k];
      if (r < gq.m) {
        Split sq(0);
        sq.base = gq.base; sq.rem = gq.rem;
        gq.w_lo[r] = (unsigned char)sq.owner(r * nch_of[k]);
        gq.w_hi[r] = (unsigned char)sq.owner(r * nch_of[k] + nch_of[k] - 1);
      }
    }
  }
  // embedding: the SMs share the gather; the copy in global memory feeds the first staging and the residual adds
  {
    float esq[BMAX];
#pragma unroll
    for (int b = 0; b < BMAX; ++b) esq[b] = 0.f;
    for (int i = tid; i < p.B * (p.d / 8); i += NCT) {
      const int b = i / (p.d / 8), u = i - b * (p.d / 8);
      if ((u % c.G) != c.sm) continue;
      int id = p.ids[(size_t)b * p.max_len + step];
      id = min(max(id, 0), p.emb_rows - 1);
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p.emb + (size_t)id * p.d) + u);
      const uint32_t hw[4] = {v.x, v.y, v.z, v.w}, t = c.tag(0) << 16;
      uint32_t *dst = p.xw + (size_t)b * p.d + (size_t)u * 8;
      reinterpret_cast<uint4 *>(dst)[0] = make_uint4(t | (hw[0] & 0xFFFFu), t | (hw[0] >> 16), t | (hw[1] & 0xFFFFu), t | (hw[1] >> 16));
      reinterpret_cast<uint4 *>(dst)[1] = make_uint4(t | (hw[2] & 0xFFFFu), t | (hw[2] >> 16), t | (hw[3] & 0xFFFFu), t | (hw[3] >> 16));
      float q = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(u32_as_h2(hw[j]));
        q += f.x * f.x + f.y * f.y;
      }
#pragma unroll
      for (int bb = 0; bb < BMAX; ++bb)
        if (bb == b) esq[bb] += q;
    }
    {  // this SM's share of sum(x^2) per batch row, published with the progress word (see Params::flag_ssq); the first staging
       // of the launch uses it on every rank (layer 0 has no partial sums to add)
#pragma unroll
      for (int b = 0; b < BMAX; ++b) {
        const float t = (b < p.B) ? consumer_sum(c, esq[b]) : 0.f;
        if (b < p.B && tid == 0) st_tagged(p.flag_ssq + b * 256 + c.sm, __float_as_uint(t), c.seq(0));
      }
    }
  }
  consumer_sync();
  if (tid == 0) st_flag(p.flag_sm + c.sm, c.seq(0));

  // The four linear phases of a layer run through one copy of the staging and multiplication code (a loop with a table of
  // operands), which keeps the kernel small enough for the instruction cache and lets the compiler inline everything.
  unsigned long long *tr = p.trace ? p.trace + ((size_t)blockIdx.x * p.n_layer) * TRS : nullptr;
#define PT_STAMP(k) do { if (tr && tid == 0) tr[l * TRS + (k)] = gtime(); } while (0)
  int xcur = 0;  // which copy of x is current (tp > 1)
  for (int l = 0; l < p.n_layer; ++l) {
    const pt_llama_layer &L = p.layers[l];
    const int ph0 = 1 + 5 * l;
    PT_STAMP(0);
#ifdef PT_MK_TRACE_WAITS
    if (tr && tid == 0) tr[l * TRS + 23] = 0ull;
#endif
    for (int ph = 0; ph < 4; ++ph) {
      // x lives in xw[cur] (two copies alternate when tp > 1, where every staging that follows a row-parallel linear forms
      // x + sum of the ranks' partial sums and stores it into the other copy)
      const bool tpar = TP;
      const size_t xsz = (size_t)p.B * p.d, psz = (size_t)p.tp * p.B * p.d;
      StageSrc src{};
      const __half *gamma;
      uint32_t *out;
      int K, epi, n_rt, N, out_phase, push = 0, out_ld = 0, out_off = 0;
      src.flags = p.flag_sm; src.flag_rows = 1; src.flag_cols = c.G;
      src.lo_unit = 0; src.hi_unit = 1 << 30;
      if (ph == 0) {
        // input: the embedding (layer 0), or x + the down_proj partial sums of the previous layer
        gamma = (const __half *)L.ln1; K = p.d; epi = EPI_QKV; n_rt = n_rt_qkv; out = p.qkvw; N = 3 * p.dq; out_phase = ph0;
        if (tpar && l > 0) {
          src.x = p.xw + xcur * xsz; src.x_tag = c.tag(ph0 - 2);   // written by the staging before gate|up of the previous layer
          src.parts = p.peer_part[p.rank] + psz; src.n_parts = p.tp; src.part_tag = c.tag(ph0 - 1);
          src.flags = p.peer_flag[p.rank]; src.flag_rows = p.tp; src.flag_cols = 0; src.want = c.arrivals(l - 1, 1);
          src.x_out = p.xw + (xcur ^ 1) * xsz; src.x_out_tag = c.tag(ph0);
        } else {
          src.x = p.xw + xcur * xsz; src.x_tag = c.tag(ph0 - 1); src.want = c.seq(ph0 - 1);
          src.ssq_flags = p.flag_ssq;   // written by the embedding / the previous layer's down_proj
        }
      } else if (ph == 1) {
        src.x = p.attnw; src.x_tag = c.tag(ph0 + 1); src.flags = p.flag_head; src.flag_cols = p.B * p.n_head; src.want = c.seq(ph0 + 1);
        gamma = nullptr; K = p.dq; epi = EPI_RESID; n_rt = n_rt_o; out = p.xw + xcur * xsz; N = p.d; out_phase = ph0 + 2;
        push = tpar;
      } else if (ph == 2) {
        gamma = (const __half *)L.ln2; K = p.d; epi = EPI_SWIGLU; n_rt = n_rt_gu; out = p.actw; N = 2 * p.ffn_valid; out_phase = ph0 + 3;
        out_ld = p.ffn; out_off = p.ffn_off;
        if (tpar) {
          src.x = p.xw + xcur * xsz; src.x_tag = (l == 0) ? c.tag(0) : c.tag(ph0);  // the embedding, or this layer's phase-0 staging
          src.parts = p.peer_part[p.rank]; src.n_parts = p.tp; src.part_tag = c.tag(ph0 + 2);
          src.flags = p.peer_flag[p.rank]; src.flag_rows = p.tp; src.flag_cols = 0; src.want = c.arrivals(l, 0);
          src.x_out = p.xw + (xcur ^ 1) * xsz; src.x_out_tag = c.tag(ph0 + 3);
        } else {
          src.x = p.xw; src.x_tag = c.tag(ph0 + 2); src.want = c.seq(ph0 + 2);
          src.ssq_flags = p.flag_ssq;   // written by this layer's o_proj
        }
      } else {
        src.x = p.actw; src.x_tag = c.tag(ph0 + 3); src.want = c.seq(ph0 + 3);
        src.lo_unit = p.ffn_off / 8; src.hi_unit = (p.ffn_off + p.ffn_valid) / 8;
        gamma = nullptr; K = p.ffn; epi = EPI_RESID; n_rt = n_rt_o; out = p.xw + xcur * xsz; N = p.d; out_phase = ph0 + 4;
        push = tpar;
      }
      if (tid == 0) {
        PhaseInfo *w = &sh->phase;
        w->outw = out; w->logits = nullptr; w->tag = c.tag(out_phase); w->out_seq = c.seq(out_phase);
        w->epi = epi; w->N = N; w->r0 = sh->geo[ph].r0;
        w->out_ld = out_ld; w->out_off = out_off;
        w->push = push; w->push_slot = (size_t)(ph == 3 ? 1 : 0) * psz + (size_t)p.rank * xsz;
      }
      c.tr = tr ? tr + l * TRS : nullptr;
      stage_x<true, TP>(c, src, K, gamma, ph == 0 ? 20 : (ph == 3 ? 24 : (ph == 2 ? 28 : 0)));
      if (src.x_out) xcur ^= 1;
      PT_STAMP(ph == 0 ? 1 : (ph == 1 ? 5 : (ph == 2 ? 8 : 10)));
      linear_phase<PT_W_INT4, TP>(c, ph, K / 128, nullptr);
      PT_STAMP(ph == 0 ? 2 : (ph == 1 ? 6 : (ph == 2 ? 9 : 11)));
      if (ph == 1) PT_STAMP(7);
      if (ph == 0) {
        PT_STAMP(3);
        attention_phase(c, L, c.tag(ph0), c.tag(ph0 + 1), c.seq(ph0 + 1));
        c.tr = nullptr;
        PT_STAMP(4);
      }
    }
    PT_STAMP(12);
  }
#undef PT_STAMP

  // final norm + LM head + arg-max (lowest index wins ties)
  Best best;
#pragma unroll
  for (int b = 0; b < BMAX; ++b) { best.v[b] = -INFINITY; best.i[b] = 0x7fffffff; }
  if (tid == 0) {
    PhaseInfo *w = &sh->phase;
    w->outw = nullptr; w->logits = p.logits; w->tag = 0u; w->out_seq = 0u;
    w->epi = EPI_HEAD; w->N = p.vocab; w->r0 = sh->geo[MAT_HEAD].r0;
    w->out_ld = 0; w->out_off = 0; w->push = 0; w->push_slot = 0;
  }
  {
    const int last = 5 * p.n_layer;  // the last down_proj phase
    StageSrc src{};
    src.x = p.xw + (size_t)xcur * p.B * p.d;
    src.lo_unit = 0; src.hi_unit = 1 << 30;
    if (TP) {
      src.x_tag = c.tag(last - 1);   // staging before gate|up of the last layer
      src.parts = p.peer_part[p.rank] + (size_t)p.tp * p.B * p.d; src.n_parts = p.tp; src.part_tag = c.tag(last);
      src.flags = p.peer_flag[p.rank]; src.flag_rows = p.tp; src.flag_cols = 0; src.want = c.arrivals(p.n_layer - 1, 1);
    } else {
      src.x_tag = c.tag(last);
      src.flags = p.flag_sm; src.flag_rows = 1; src.flag_cols = c.G; src.want = c.seq(last);
      src.ssq_flags = p.flag_ssq;
    }
    stage_x<false, TP>(c, src, p.d, p.norm);
  }
  linear_phase<PT_W_FP16, TP>(c, MAT_HEAD, nc_head, &best);
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
    if (p.done_flag && p.stop_mask && lane == 0) {
      // keep_going = sum(stop_mask) < batch, taken on the mask as it was BEFORE this iteration's update (base_model.py:348-352)
      int stopped = 0;
      for (int b = 0; b < p.B; ++b) stopped += p.stop_mask[b] ? 1 : 0;
      if (stopped == p.B) *p.done_flag = 1;
    }
    __syncwarp();
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
      if (TP) {
        // vocabulary-parallel head (layers/lm_head.py:75-116): every rank sends its best (value, id) to every rank, and each
        // takes the first maximum in rank order, so all ranks append the same id
        const uint32_t sq = c.seq(5 * p.n_layer + 1);
        if (lane < p.tp) {
          uint2 *dst = p.peer_cand[lane] + ((size_t)p.rank * BMAX + b) * 2;
          st_sys2(dst, __float_as_uint(v), sq);
          st_sys2(dst + 1, (uint32_t)i, sq);
        }
        float rv = -INFINITY;
        int ri = 0x7fffffff;
        if (lane < p.tp) {
          const uint2 *srcc = p.peer_cand[p.rank] + ((size_t)lane * BMAX + b) * 2;
          bool got = false;
          for (int it = 0; it < POLL_LIMIT && !got; ++it) {
            const uint2 a0 = ld_sys2(srcc), a1 = ld_sys2(srcc + 1);
            if (a0.y == sq && a1.y == sq) { rv = __uint_as_float(a0.x); ri = (int)a1.x; got = true; }
            if ((it & 63) == 63 && sh->abort) break;
          }
          if (!got) {
            sh->abort = 1;
            if (p.error_flag) atomicCAS(p.error_flag, 0, 11);
          }
        }
        v = rv;
        i = ri;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, o);
          const int oi = __shfl_xor_sync(0xffffffffu, i, o);
          if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
        }
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
    p.barrier[3] = __ldcg(p.barrier + 3) + 1u;
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

}  // namespace PT_MK_NS
}  // namespace pt

#ifdef PT_MK_SHORT_VARIANT
namespace pt {
// Launches the short-wait build of the kernel.  `params` points to a Params of the default build (same layout).
int mk_short_launch(bool tp, const void *params, int n_sm, size_t smem, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    int dev = 0, v = 0;
    PT_CUDA(cudaGetDevice(&dev));
    PT_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    PT_CUDA(cudaFuncSetAttribute(mk_short::llama_step_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, v));
    PT_CUDA(cudaFuncSetAttribute(mk_short::llama_step_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, v));
    attr_set = true;
  }
  void *kargs[] = {const_cast<void *>(params)};
  const void *kernel = tp ? (const void *)mk_short::llama_step_kernel<true> : (const void *)mk_short::llama_step_kernel<false>;
  cudaError_t e = cudaLaunchCooperativeKernel(kernel, dim3(n_sm), dim3(mk_short::THREADS), kargs, smem, stream);
  if (e != cudaSuccess) return pt::set_error(PT_ERR_CUDA, "pt_llama_decode_step: %s", cudaGetErrorString(e));
  return PT_OK;
}
}  // namespace pt
#else
namespace pt {
int mk_short_launch(bool tp, const void *params, int n_sm, size_t smem, cudaStream_t stream);
}
using namespace pt;

extern "C" int pt_llama_stream_permute(int wfmt, const void *packed, void *out, int n_out, int k_in, void *stream) {
  PT_REQUIRE(packed && out && packed != out, "pt_llama_stream_permute: needs distinct source and destination buffers");
  PT_REQUIRE(wfmt == PT_W_INT4 || wfmt == PT_W_FP16, "pt_llama_stream_permute: weight format %d not used by the persistent kernel", wfmt);
  PT_REQUIRE(n_out > 0 && k_in > 0 && k_in % chunk_k(wfmt) == 0, "pt_llama_stream_permute: bad shape [%d, %d]", n_out, k_in);
  const int n_sm = pt::sm_count();
  mk::stream_permute_kernel<<<dim3(32, n_sm), 256, 0, as_stream(stream)>>>((const uint4 *)packed, (uint4 *)out, ceil_div(n_out, 16), k_in / chunk_k(wfmt),
                                                                            tile_bytes(wfmt) / 16, n_sm);
  PT_LAUNCH_CHECK("pt_llama_stream_permute");
  return PT_OK;
}

extern "C" size_t pt_llama_step_workspace_bytes(int batch, int n_head, int head_dim, int max_pages) {
  const size_t heads = (size_t)batch * n_head;
  auto al = [](size_t v) { return (v + 255) / 256 * 256; };
  // barrier words | per-SM progress words | per-SM x statistics | per-head progress words | page (max, sum) | partial outputs (both as 8-byte tagged words) | arg-max candidates (value, index) for up to 256 SMs
  return 256 + 1024 + (size_t)mk::BMAX * 256 * sizeof(uint2) + al(heads * sizeof(uint32_t)) + al(heads * max_pages * 2 * sizeof(uint2)) + al(heads * max_pages * head_dim * sizeof(uint2)) + 2 * al((size_t)batch * 256 * sizeof(float));
}

extern "C" size_t pt_llama_tp_buffer_bytes(int batch, int d_model, int tp_size) {
  return (size_t)2 * tp_size * batch * d_model * sizeof(uint32_t) + (size_t)tp_size * 256 * sizeof(uint32_t) + (size_t)tp_size * mk::BMAX * 2 * sizeof(uint2);
}

extern "C" int pt_llama_decode_step(const pt_llama_step_args *a, void *stream) {
  PT_REQUIRE(a, "pt_llama_decode_step: null args");
  PT_REQUIRE(a->batch >= 1 && a->batch <= mk::BMAX, "pt_llama_decode_step: batch=%d outside 1..%d (larger batches use the per-op kernels)", a->batch,
             mk::BMAX);
  PT_REQUIRE(a->head_dim == mk::H && a->page_size == mk::PAGE, "pt_llama_decode_step: needs head_dim=%d and page_size=%d", mk::H, mk::PAGE);
  const int tp = a->tp_size > 1 ? a->tp_size : 1;
  PT_REQUIRE(tp <= 8 && a->tp_rank >= 0 && a->tp_rank < tp, "pt_llama_decode_step: tp_size=%d tp_rank=%d (at most 8 ranks)", a->tp_size, a->tp_rank);
  PT_REQUIRE(a->d_model % 128 == 0 && a->ffn % 128 == 0 && a->d_model == a->n_head * a->head_dim * tp && a->d_model <= 96 * 128 && a->ffn <= 96 * 128,
             "pt_llama_decode_step: d_model=%d ffn=%d must be multiples of 128 (at most 12288) with d_model = tp * n_head * head_dim", a->d_model, a->ffn);
  const int ffn_off = tp > 1 ? a->ffn_offset : 0, ffn_valid = tp > 1 ? a->ffn_valid : a->ffn;
  PT_REQUIRE(ffn_off >= 0 && ffn_valid > 0 && ffn_off % 8 == 0 && ffn_valid % 8 == 0 && ffn_off + ffn_valid <= a->ffn,
             "pt_llama_decode_step: MLP slice [%d, %d) must be a multiple-of-8 range inside the window of %d columns", ffn_off, ffn_off + ffn_valid, a->ffn);
  if (tp > 1)
    for (int r = 0; r < tp; ++r) PT_REQUIRE(a->tp_buffers[r], "pt_llama_decode_step: tp_buffers[%d] is null", r);
  PT_REQUIRE((2 * a->ffn) % 16 == 0 && a->vocab > 0 && a->n_layer > 0 && a->max_len > 0 && a->max_pages * mk::PAGE >= a->max_len,
             "pt_llama_decode_step: bad shape");
  PT_REQUIRE(a->layers && a->norm && a->head && a->emb && a->ids && a->step_dev && a->page_table && a->rope_sin && a->rope_cos && a->x && a->qkv &&
                 a->attn && a->act && a->next_ids && a->workspace,
             "pt_llama_decode_step: null pointer argument");
  const size_t need = pt_llama_step_workspace_bytes(a->batch, a->n_head, a->head_dim, a->max_pages);
  PT_REQUIRE(a->workspace_bytes >= need, "pt_llama_decode_step: workspace needs %zu bytes, got %zu", need, a->workspace_bytes);

  const int n_sm = pt::sm_count();
  static size_t smem_max = 0;
  if (smem_max == 0) {
    int dev = 0, v = 0;
    PT_CUDA(cudaGetDevice(&dev));
    PT_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    PT_CUDA(cudaFuncSetAttribute(mk::llama_step_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, v));
    PT_CUDA(cudaFuncSetAttribute(mk::llama_step_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, v));
    smem_max = (size_t)v;
  }
  PT_REQUIRE(n_sm <= 256, "pt_llama_decode_step: %d SMs exceed the candidate buffer", n_sm);

  mk::Params p{};
  p.B = a->batch; p.d = a->d_model; p.n_head = a->n_head; p.ffn = a->ffn; p.vocab = a->vocab; p.n_layer = a->n_layer;
  p.tp = tp; p.rank = tp > 1 ? a->tp_rank : 0; p.dq = a->n_head * a->head_dim; p.ffn_off = ffn_off; p.ffn_valid = ffn_valid;
  p.vocab_off = tp > 1 ? a->vocab_offset : 0;
  p.emb_rows = tp > 1 ? a->emb_rows : a->vocab;
  PT_REQUIRE(p.emb_rows > 0, "pt_llama_decode_step: emb_rows=%d", p.emb_rows);
  for (int r = 0; r < tp && tp > 1; ++r) {
    // exchange buffer of rank r: partial sums [2][tp][B][d] | progress words [tp][256] | arg-max candidates [tp][BMAX][2]
    char *base = (char *)a->tp_buffers[r];
    const size_t part_bytes = (size_t)2 * tp * a->batch * a->d_model * sizeof(uint32_t);
    p.peer_part[r] = (uint32_t *)base;
    p.peer_flag[r] = (uint32_t *)(base + part_bytes);
    p.peer_cand[r] = (uint2 *)(base + part_bytes + (size_t)tp * 256 * sizeof(uint32_t));
  }
  p.max_len = a->max_len; p.max_pages = a->max_pages; p.pad_id = a->pad_id; p.eos_id = a->eos_id;
  p.eps = a->norm_eps;
  p.score_scale = __float2half_rn(a->score_scale);
  p.layers = a->layers; p.norm = (const __half *)a->norm; p.emb = (const __half *)a->emb;
  p.sin_t = (const __half *)a->rope_sin; p.cos_t = (const __half *)a->rope_cos; p.head = (const unsigned char *)a->head;
  p.ids = a->ids; p.step = a->step_dev; p.stop_mask = a->stop_mask; p.next_ids = a->next_ids; p.page_table = a->page_table;
  p.done_flag = a->done_flag;
  PT_REQUIRE(!a->done_flag || a->stop_mask, "pt_llama_decode_step: done_flag needs stop_mask");
  p.xw = (uint32_t *)a->x; p.qkvw = (uint32_t *)a->qkv; p.attnw = (uint32_t *)a->attn; p.actw = (uint32_t *)a->act; p.logits = (__half *)a->logits;
  p.error_flag = a->error_flag;
  p.trace = (unsigned long long *)a->trace;
  p.debug = a->debug;
  auto al = [](size_t v) { return (v + 255) / 256 * 256; };
  const size_t heads = (size_t)a->batch * a->n_head;
  char *ws = (char *)a->workspace;
  p.barrier = (unsigned *)ws; ws += 256;
  p.flag_sm = (uint32_t *)ws; ws += 1024;
  p.flag_ssq = (uint2 *)ws; ws += (size_t)mk::BMAX * 256 * sizeof(uint2);
  p.flag_head = (uint32_t *)ws; ws += al(heads * sizeof(uint32_t));
  p.ws_ml = (uint2 *)ws; ws += al(heads * a->max_pages * 2 * sizeof(uint2));
  p.ws_o = (uint2 *)ws; ws += al(heads * a->max_pages * a->head_dim * sizeof(uint2));
  p.cand_val = (float *)ws; ws += al((size_t)a->batch * 256 * sizeof(float));
  p.cand_idx = (int *)ws;

  const int kmax = std::max(a->d_model, a->ffn);
  p.xs_stride = (kmax * 2) | 64;
  const size_t fixed = (((size_t)p.B * p.xs_stride + 127) / 128) * 128 + sizeof(mk::Shared) + 128;
  PT_REQUIRE(smem_max > fixed + 3 * (size_t)mk::STAGE_BYTES, "pt_llama_decode_step: shared memory too small");
  p.ns = (int)std::min<size_t>(16, (smem_max - fixed) / mk::STAGE_BYTES);
  const size_t smem = (size_t)p.ns * mk::STAGE_BYTES + fixed;

  {
    // per device: what the constants currently hold (stream-ordered updates; launches on other streams of the same device
    // that overlap a change may see either value)
    static uint32_t hint_set[64];
    int dev = 0;
    PT_CUDA(cudaGetDevice(&dev));
    PT_REQUIRE(dev >= 0 && dev < 64, "pt_llama_decode_step: device ordinal %d outside 0..63", dev);
    const uint32_t want = ((uint32_t)a->debug >> 16) ? ((uint32_t)a->debug >> 16) : 2000u;
    if (want != (hint_set[dev] ? hint_set[dev] : 2000u)) {
      PT_CUDA(cudaMemcpyToSymbolAsync(mk::c_wait_hint, &want, sizeof(want), 0, cudaMemcpyHostToDevice, as_stream(stream)));
      hint_set[dev] = want;
    }
  }
  PT_REQUIRE(a->wait_limit >= 0, "pt_llama_decode_step: wait_limit=%d", a->wait_limit);
  if (a->wait_limit > 0) {  // the short-wait build (its limit is a compile-time constant, like the default build's)
    if (int rc = mk_short_launch(tp > 1, &p, n_sm, smem, as_stream(stream))) return rc;
    pt::count_launch();
    return PT_OK;
  }
  void *kargs[] = {(void *)&p};
  const void *kernel = tp > 1 ? (const void *)mk::llama_step_kernel<true> : (const void *)mk::llama_step_kernel<false>;
  cudaError_t e = cudaLaunchCooperativeKernel(kernel, dim3(n_sm), dim3(mk::THREADS), kargs, smem, as_stream(stream));
  if (e != cudaSuccess) return pt::set_error(PT_ERR_CUDA, "pt_llama_decode_step: %s", cudaGetErrorString(e));
  PT_LAUNCH_CHECK("pt_llama_decode_step");
  return PT_OK;
}
#endif  // PT_MK_SHORT_VARIANT
