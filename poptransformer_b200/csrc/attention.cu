// Paged KV cache: append of the new token fused with split flash-decode attention.
//
// One block handles one page (page_size cached tokens) of one (sequence, kv-head): its K and V tiles are
// contiguous in the pool, so each is fetched with a single 1-D bulk async copy (TMA engine,
// cp.async.bulk + mbarrier) while the threads apply RoPE to q (and to the new k).  The block that owns the
// page holding position `step` writes the new k/v into the pool and into its shared-memory tile, so the
// append costs no extra pass over the cache.  Scores use 8 lanes per cached token with warp-shuffle
// reductions, the softmax statistics are warp-shuffle reductions, and P.V is one thread per output
// channel.  Every block leaves (max, sum, partial output) in the workspace; the last block to arrive for
// a (sequence, kv-head) combines the pages in a fixed order, which keeps the result deterministic.
//
// HBM-bound: algorithmic bytes = 2 * (step + 1) * head_dim * 2 per (sequence, kv-head), read once.
#include "common.cuh"

namespace pt {

struct AttnParams {
  int B, n_head, n_kv, qpk, qsplit, H, page, max_pages, max_len, rope_mode, softmax_mode, rot_half, out_ld, pdl;
  __half scale_h;
  int use_scale;
  const int *step;
  const __half *qkv, *sin_t, *cos_t;
  __half *pool;
  const int *page_table;
  __half *out;
  float *ws_o;     // [B, n_head, max_pages, H]
  float2 *ws_ml;   // [B, n_head, max_pages]
  int *counters;   // [B, n_kv, qsplit]
  int *error_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Bounded wait: returns false if the phase did not complete within the iteration limit.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t phase) {
  for (int it = 0; it < (1 << 22); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(phase)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// RoPE on one head vector x[H] (global, fp16) -> dst[H] (fp16), with the reference's fp16 roundings.
// Llama (rotate_half): y_j = fp16(fp16(x_j c_j) + fp16(-x_{j+H/2} s_j)), y_{j+H/2} = fp16(fp16(x_{j+H/2} c_j) + fp16(x_j s_j)).
// ChatGLM2: only the first H/2 channels rotate, as interleaved pairs (2i, 2i+1) with angle i:
//   y_{2i} = fp16(fp16(x_{2i} c_i) - fp16(x_{2i+1} s_i)), y_{2i+1} = fp16(fp16(x_{2i+1} c_i) + fp16(x_{2i} s_i)).
__device__ __forceinline__ void rope_pair(const AttnParams &p, const __half *x, const __half *sin_r, const __half *cos_r, int i,
                                          __half *dst) {
  if (p.rope_mode == PT_ROPE_LLAMA) {
    const int h2 = p.H / 2;
    const __half a = x[i], b = x[i + h2], s = sin_r[i], c = cos_r[i];
    dst[i] = h_add(h_mul(a, c), h_mul(__hneg(b), s));
    dst[i + h2] = h_add(h_mul(b, c), h_mul(a, s));
  } else if (p.rope_mode == PT_ROPE_CHATGLM2) {
    const int nrot = p.H / 4;  // rotated pairs
    if (i < nrot) {
      const __half a = x[2 * i], b = x[2 * i + 1], s = sin_r[i], c = cos_r[i];
      dst[2 * i] = h_sub(h_mul(a, c), h_mul(b, s));
      dst[2 * i + 1] = h_add(h_mul(b, c), h_mul(a, s));
    } else {
      dst[2 * i] = x[2 * i];
      dst[2 * i + 1] = x[2 * i + 1];
    }
  } else {
    dst[2 * i] = x[2 * i];
    dst[2 * i + 1] = x[2 * i + 1];
  }
}

constexpr int kAttnThreads = 128;

template <int H>
__global__ void __launch_bounds__(kAttnThreads) kv_append_attn_kernel(const AttnParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int PAGE = p.page;
  __half *Ks = reinterpret_cast<__half *>(smem);
  __half *Vs = Ks + (size_t)PAGE * H;
  const int nq_s = p.qpk / p.qsplit;                       // q heads handled by this block
  __half *qs = Vs + (size_t)PAGE * H;                      // [nq][H]
  float *ps = reinterpret_cast<float *>(qs + (size_t)nq_s * H);  // [nq][PAGE]
  float *ml = ps + (size_t)nq_s * PAGE;                    // [nq][2]
  __shared__ __align__(8) uint64_t bar;
  __shared__ int s_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // With many q heads per kv head (multi-query attention) the heads of a group are shared out over `qsplit` blocks: each
  // re-reads the group's K/V page (through L2) and handles nq of the group's heads, which shortens both the per-page work
  // and the serial combine of the last block.
  const int pg = blockIdx.x, kvh = blockIdx.y / p.qsplit, qpart = blockIdx.y - kvh * p.qsplit, b = blockIdx.z;
  const int nq = p.qpk / p.qsplit, q_lo = qpart * nq;   // this block's heads of the group: q_lo .. q_lo + nq - 1
  if (p.pdl) {
    // let the next kernel start prefetching its weights; everything this kernel reads was produced upstream
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  const int step = *p.step;
  if (step < 0 || step >= p.max_len) {  // no page / no RoPE row for this position: report it and leave the counters untouched
    if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 12);
    return;
  }
  const int n_active = step / PAGE + 1;
  if (pg >= n_active) return;
  const int n_valid = min(PAGE, step + 1 - pg * PAGE);
  const bool owner = (pg == n_active - 1);
  const int n_load = owner ? n_valid - 1 : n_valid;  // the newest token is not in the pool yet

  const int phys = p.page_table[(size_t)b * p.max_pages + pg];
  __half *gK = p.pool + (((size_t)phys * 2 + 0) * p.n_kv + kvh) * PAGE * H;
  __half *gV = p.pool + (((size_t)phys * 2 + 1) * p.n_kv + kvh) * PAGE * H;

  if (tid == 0) {
    mbar_init(&bar, 1);
    if (n_load > 0) {
      const uint32_t bytes = (uint32_t)n_load * H * sizeof(__half);
      mbar_expect_tx(&bar, 2 * bytes);
      bulk_g2s(Ks, gK, bytes, &bar);
      bulk_g2s(Vs, gV, bytes, &bar);
    }
  }

  // ---- RoPE on the group's q heads (and on the new k) while the tiles are in flight
  const int row_elems = (p.n_head + 2 * p.n_kv) * H;
  const __half *qrow = p.qkv + (size_t)b * row_elems;
  const __half *sin_r = p.sin_t + (size_t)step * p.rot_half;
  const __half *cos_r = p.cos_t + (size_t)step * p.rot_half;
  for (int i = tid; i < nq * (H / 2); i += kAttnThreads) {
    const int qh = i / (H / 2), j = i - qh * (H / 2);
    rope_pair(p, qrow + (size_t)(kvh * p.qpk + q_lo + qh) * H, sin_r, cos_r, j, qs + (size_t)qh * H);
  }
  if (owner) {
    const int slot = n_valid - 1;
    const __half *knew = qrow + (size_t)(p.n_head + kvh) * H;
    const __half *vnew = qrow + (size_t)(p.n_head + p.n_kv + kvh) * H;
    for (int j = tid; j < H / 2; j += kAttnThreads) rope_pair(p, knew, sin_r, cos_r, j, Ks + (size_t)slot * H);
    for (int j = tid; j < H; j += kAttnThreads) Vs[(size_t)slot * H + j] = vnew[j];
    __syncthreads();
    if (qpart == 0) {   // one block of the group appends to the pool; the others only need the new token in their tile
      for (int j = tid; j < H; j += kAttnThreads) {
        gK[(size_t)slot * H + j] = Ks[(size_t)slot * H + j];
        gV[(size_t)slot * H + j] = Vs[(size_t)slot * H + j];
      }
    }
  }
  __syncthreads();  // barrier initialised, q staged
  if (n_load > 0 && !mbar_wait(&bar, 0)) {
    if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 1);
    return;  // bounded wait gave up: report, do not hang
  }

  // ---- scores: 8 lanes per cached token
  {
    constexpr int EPL = H / 8;  // elements per lane: vector v of a lane covers channels v*64 + sub*8 .. +8,
                                // so the 8 lanes of a token read 128 contiguous bytes (no bank conflicts)
    const int sub = lane & 7, tgrp = tid >> 3;  // 16 token groups per pass
    for (int t0 = 0; t0 < n_valid; t0 += kAttnThreads / 8) {
      const int t = t0 + tgrp;
      float kf[EPL];
      if (t < n_valid) {
#pragma unroll
        for (int v = 0; v < EPL / 8; ++v) {
          uint4 raw = *reinterpret_cast<const uint4 *>(Ks + (size_t)t * H + v * 64 + sub * 8);
          const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __half22float2(h[j]);
            kf[v * 8 + 2 * j] = f.x;
            kf[v * 8 + 2 * j + 1] = f.y;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < EPL; ++j) kf[j] = 0.f;
      }
      for (int qh = 0; qh < nq; ++qh) {
        float s = 0.f;
#pragma unroll
        for (int v = 0; v < EPL / 8; ++v) {
          uint4 raw = *reinterpret_cast<const uint4 *>(qs + (size_t)qh * H + v * 64 + sub * 8);
          const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __half22float2(h[j]);
            s += kf[v * 8 + 2 * j] * f.x;
            s += kf[v * 8 + 2 * j + 1] * f.y;
          }
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (sub == 0 && t < n_valid) {
          __half s16 = __float2half_rn(s);               // fp16 matmul output
          if (p.use_scale) s16 = h_mul(s16, p.scale_h);  // ops.mul by fp16(1/sqrt(H))
          ps[(size_t)qh * PAGE + t] = __half2float(s16);
        }
      }
    }
  }
  __syncthreads();

  // ---- per-head softmax statistics (one warp per q head, warp-shuffle reductions)
  for (int qh = warp; qh < nq; qh += kAttnThreads / 32) {
    float *pr = ps + (size_t)qh * PAGE;
    float m = -INFINITY;
    if (p.softmax_mode == PT_SOFTMAX_F32) {
      for (int t = lane; t < n_valid; t += 32) m = fmaxf(m, pr[t]);
      m = warp_max(m);
    } else {
      m = 0.f;  // the reference exponentiates fp16 scores without subtracting the maximum
    }
    float l = 0.f;
    for (int t = lane; t < n_valid; t += 32) {
      float e = expf(pr[t] - m);
      if (p.softmax_mode == PT_SOFTMAX_F16) e = __half2float(__float2half_rn(e));
      pr[t] = e;
      l += e;
    }
    l = warp_sum(l);
    if (lane == 0) { ml[2 * qh] = m; ml[2 * qh + 1] = l; }
  }
  __syncthreads();

  // ---- P.V: one thread per output channel, V element reused across the group's q heads
  const size_t head0 = (size_t)b * p.n_head + (size_t)kvh * p.qpk + q_lo;
  if (tid < H) {
    for (int q0 = 0; q0 < nq; q0 += 4) {
      float o[4] = {0.f, 0.f, 0.f, 0.f};
      const int n4 = min(4, nq - q0);
      for (int t = 0; t < n_valid; ++t) {
        const float v = __half2float(Vs[(size_t)t * H + tid]);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (k < n4) o[k] += ps[(size_t)(q0 + k) * PAGE + t] * v;
      }
      for (int k = 0; k < n4; ++k) p.ws_o[((head0 + q0 + k) * p.max_pages + pg) * H + tid] = o[k];
    }
  }
  if (tid < nq) p.ws_ml[(head0 + tid) * p.max_pages + pg] = make_float2(ml[2 * tid], ml[2 * tid + 1]);
  for (int qh = tid + kAttnThreads; qh < nq; qh += kAttnThreads)
    p.ws_ml[(head0 + qh) * p.max_pages + pg] = make_float2(ml[2 * qh], ml[2 * qh + 1]);

  // ---- last block to arrive for this (sequence, kv-head) combines the pages in page order
  __threadfence();
  __syncthreads();
  int *ctr = p.counters + ((size_t)b * p.n_kv + kvh) * p.qsplit + qpart;
  if (tid == 0) s_last = (atomicAdd(ctr, 1) == n_active - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (tid == 0) *ctr = 0;
  // The K tile is no longer needed: its shared memory takes the pages' (max, sum) pairs, then their weights.  All loads of a
  // stage are issued before the first is used, so the combine costs a handful of L2 round trips whatever the number of pages
  // and heads (a loop of dependent-looking loads per head and page made it the longest part of the kernel at 17 pages).
  float *cw = reinterpret_cast<float *>(Ks);           // [nq][n_active] weights exp(m_i - M)
  float *cl = cw + (size_t)nq * n_active;              // [nq][n_active] page sums, then cl[qh * n_active] = L of the head
  // (worth its two extra barriers from about sixteen (head, page) pairs on: measured 1 % slower than the plain loop at 1 head x 6 pages)
  const bool staged = nq * n_active >= 16 && (size_t)2 * nq * n_active * sizeof(float) <= (size_t)PAGE * H * sizeof(__half);
  if (staged) {
    for (int idx = tid; idx < nq * n_active; idx += kAttnThreads) {
      const int qh = idx / n_active, i = idx - qh * n_active;
      const float2 v = __ldcg(&p.ws_ml[(head0 + qh) * p.max_pages + i]);
      cw[idx] = v.x;
      cl[idx] = v.y;
    }
    __syncthreads();
    for (int qh = warp; qh < nq; qh += kAttnThreads / 32) {
      float *w = cw + (size_t)qh * n_active, *l = cl + (size_t)qh * n_active;
      float M = -INFINITY;
      for (int i = lane; i < n_active; i += 32) M = fmaxf(M, w[i]);
      M = warp_max(M);
      for (int i = lane; i < n_active; i += 32) w[i] = expf(w[i] - M);
      __syncwarp();
      if (lane == 0) {   // the head's sum in page order, like the outputs below
        float L = 0.f;
        for (int i = 0; i < n_active; ++i) L += l[i] * w[i];
        l[0] = L;
      }
    }
    __syncthreads();
    if (tid < H) {
      constexpr int PB = 8;   // pages in flight per head; two heads at a time
      for (int q0 = 0; q0 < nq; q0 += 2) {
        const bool two = q0 + 1 < nq;
        float o0 = 0.f, o1 = 0.f;
        const float *w0 = cw + (size_t)q0 * n_active, *w1 = cw + (size_t)(two ? q0 + 1 : q0) * n_active;
        const float *src0 = p.ws_o + ((head0 + q0) * p.max_pages) * H + tid, *src1 = src0 + (two ? (size_t)p.max_pages * H : 0);
        for (int i0 = 0; i0 < n_active; i0 += PB) {
          float v0[PB], v1[PB];
#pragma unroll
          for (int j = 0; j < PB; ++j) {
            const bool in = i0 + j < n_active;
            v0[j] = in ? __ldcg(src0 + (size_t)(i0 + j) * H) : 0.f;
            v1[j] = (in && two) ? __ldcg(src1 + (size_t)(i0 + j) * H) : 0.f;
          }
#pragma unroll
          for (int j = 0; j < PB; ++j)
            if (i0 + j < n_active) {
              o0 += v0[j] * w0[i0 + j];
              o1 += v1[j] * w1[i0 + j];
            }
        }
        __half *dst = p.out + (size_t)b * p.out_ld + ((size_t)kvh * p.qpk + q_lo + q0) * H + tid;
        dst[0] = __float2half_rn(o0 / cl[(size_t)q0 * n_active]);
        if (two) dst[H] = __float2half_rn(o1 / cl[(size_t)(q0 + 1) * n_active]);
      }
    }
    return;
  }
  if (tid < H) {   // more pages than the tile holds statistics for: the plain loop
    for (int qh = 0; qh < nq; ++qh) {
      const size_t hd = head0 + qh;
      float M = -INFINITY;
      for (int i = 0; i < n_active; ++i) M = fmaxf(M, __ldcg(&p.ws_ml[hd * p.max_pages + i]).x);
      float L = 0.f, o = 0.f;
      for (int i = 0; i < n_active; ++i) {
        const float2 v = __ldcg(&p.ws_ml[hd * p.max_pages + i]);
        const float w = expf(v.x - M);
        L += v.y * w;
        o += __ldcg(&p.ws_o[(hd * p.max_pages + i) * H + tid]) * w;
      }
      p.out[(size_t)b * p.out_ld + ((size_t)kvh * p.qpk + q_lo + qh) * H + tid] = __float2half_rn(o / L);
    }
  }
}

// dense[kv][b][h][l][:] = l <= step ? token (step - l) of the paged cache : 0
__global__ void kv_export_kernel(const __half *pool, const int *page_table, const int *step_dev, int B, int n_kv, int H, int page,
                                 int max_pages, int max_len, __half *dense) {
  const int step = *step_dev;
  const size_t total = (size_t)2 * B * n_kv * max_len * (H / 8);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i;
    const int u = r % (H / 8); r /= (H / 8);
    const int l = r % max_len; r /= max_len;
    const int h = r % n_kv; r /= n_kv;
    const int b = r % B; r /= B;
    const int kv = (int)r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (l <= step) {
      const int t = step - l;
      const int phys = page_table[(size_t)b * max_pages + t / page];
      v = *reinterpret_cast<const uint4 *>(pool + ((((size_t)phys * 2 + kv) * n_kv + h) * page + t % page) * H + u * 8);
    }
    reinterpret_cast<uint4 *>(dense)[i] = v;
  }
}

// Copies the page being filled (slots 0 .. step % page) of row parent[r] into row r's spare page.
__global__ void kv_reorder_pages_kernel(__half *pool, const int *page_table, const int *spare, const int *parent, const int *step_dev,
                                        int n_kv, int H, int page, int max_pages) {
  const int r = blockIdx.x, step = *step_dev;
  const int pg = step / page, n_slots = step % page + 1;
  const int src = page_table[(size_t)parent[r] * max_pages + pg], dst = spare[r];
  const size_t page_elems = (size_t)2 * n_kv * page * H;
  const uint4 *s4 = reinterpret_cast<const uint4 *>(pool + (size_t)src * page_elems);
  uint4 *d4 = reinterpret_cast<uint4 *>(pool + (size_t)dst * page_elems);
  const int row_u = H / 8;                       // 16-byte units per token
  const int total = 2 * n_kv * n_slots * row_u;  // only the filled slots of each (k|v, head) tile
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < total; i += gridDim.y * blockDim.x) {
    const int u = i % row_u, t = (i / row_u) % n_slots, hk = i / (row_u * n_slots);
    const size_t off = ((size_t)hk * page + t) * row_u + u;
    d4[off] = s4[off];
  }
}
// new_table[r][p < pg] = old[parent[r]][p]; new_table[r][pg] = spare[r]; spare[r] = old[r][pg]; later pages stay.
__global__ void kv_reorder_table_kernel(int *table, const int *old, int *spare, const int *parent, const int *step_dev, int rows,
                                        int page, int max_pages) {
  const int pg = *step_dev / page;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * max_pages; i += gridDim.x * blockDim.x) {
    const int r = i / max_pages, p = i - r * max_pages;
    if (p < pg) table[i] = old[(size_t)parent[r] * max_pages + p];
    else if (p == pg) {
      table[i] = spare[r];
      spare[r] = old[i];
    }
  }
}

}  // namespace pt

using namespace pt;

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

extern "C" size_t pt_attn_workspace_bytes(int batch, int n_head, int head_dim, int max_pages) {
  const size_t heads = (size_t)batch * n_head;
  return align256(heads * sizeof(int)) + align256(heads * max_pages * sizeof(float2)) + heads * max_pages * head_dim * sizeof(float);
}

extern "C" int pt_kv_append_attn(const pt_attn_args *a, void *stream) {
  PT_REQUIRE(a, "pt_kv_append_attn: null args");
  PT_REQUIRE(a->batch > 0 && a->n_head > 0 && a->n_kv > 0 && a->n_head % a->n_kv == 0,
             "pt_kv_append_attn: n_head=%d must be a positive multiple of n_kv=%d", a->n_head, a->n_kv);
  PT_REQUIRE(a->head_dim == 64 || a->head_dim == 128, "pt_kv_append_attn: head_dim=%d (supported: 64, 128)", a->head_dim);
  PT_REQUIRE(a->page_size >= 8 && a->page_size <= 128 && a->page_size % 8 == 0, "pt_kv_append_attn: page_size=%d must be a multiple of 8 in 8..128",
             a->page_size);
  PT_REQUIRE(a->max_pages > 0, "pt_kv_append_attn: max_pages=%d", a->max_pages);
  PT_REQUIRE(a->rope_mode >= PT_ROPE_NONE && a->rope_mode <= PT_ROPE_CHATGLM2, "pt_kv_append_attn: bad rope_mode %d", a->rope_mode);
  PT_REQUIRE(a->softmax_mode == PT_SOFTMAX_F32 || a->softmax_mode == PT_SOFTMAX_F16, "pt_kv_append_attn: bad softmax_mode %d", a->softmax_mode);
  PT_REQUIRE(a->step_dev && a->qkv && a->pool && a->page_table && a->out && a->workspace, "pt_kv_append_attn: null pointer argument");
  PT_REQUIRE(a->rope_mode == PT_ROPE_NONE || (a->rope_sin && a->rope_cos), "pt_kv_append_attn: RoPE needs sin/cos tables");
  const size_t need = pt_attn_workspace_bytes(a->batch, a->n_head, a->head_dim, a->max_pages);
  PT_REQUIRE(a->workspace_bytes >= need, "pt_kv_append_attn: workspace needs %zu bytes, got %zu", need, a->workspace_bytes);

  AttnParams p{};
  p.B = a->batch; p.n_head = a->n_head; p.n_kv = a->n_kv; p.qpk = a->n_head / a->n_kv; p.H = a->head_dim;
  p.qsplit = (p.qpk > 4 && p.qpk % 4 == 0) ? p.qpk / 4 : 1;   // four q heads per block for multi-query groups
  p.page = a->page_size; p.max_pages = a->max_pages; p.rope_mode = a->rope_mode; p.softmax_mode = a->softmax_mode;
  p.rot_half = a->rope_mode == PT_ROPE_CHATGLM2 ? a->head_dim / 4 : a->head_dim / 2;
  p.out_ld = a->out_ld > 0 ? a->out_ld : a->n_head * a->head_dim;
  p.use_scale = a->score_scale != 1.0f;
  p.scale_h = __float2half_rn(a->score_scale);
  p.step = a->step_dev;
  p.qkv = (const __half *)a->qkv; p.sin_t = (const __half *)a->rope_sin; p.cos_t = (const __half *)a->rope_cos;
  p.pool = (__half *)a->pool; p.page_table = a->page_table; p.out = (__half *)a->out;
  const size_t heads = (size_t)a->batch * a->n_head;
  char *ws = (char *)a->workspace;
  p.counters = (int *)ws; ws += align256(heads * sizeof(int));
  p.ws_ml = (float2 *)ws; ws += align256(heads * a->max_pages * sizeof(float2));
  p.ws_o = (float *)ws;
  p.error_flag = a->error_flag;
  p.pdl = a->pdl ? 1 : 0;
  PT_REQUIRE(a->max_len >= 0 && a->max_len <= a->page_size * a->max_pages, "pt_kv_append_attn: max_len=%d exceeds the %d positions of the page table",
             a->max_len, a->page_size * a->max_pages);
  p.max_len = a->max_len > 0 ? a->max_len : a->page_size * a->max_pages;

  const int nq = p.qpk / p.qsplit;
  const size_t smem = (size_t)2 * p.page * p.H * sizeof(__half) + (size_t)nq * p.H * sizeof(__half) +
                      (size_t)nq * p.page * sizeof(float) + (size_t)nq * 2 * sizeof(float);
  PT_REQUIRE(smem <= 200 * 1024, "pt_kv_append_attn: tile needs %zu bytes of shared memory", smem);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a->max_pages, a->n_kv * p.qsplit, a->batch);
  cfg.blockDim = dim3(kAttnThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  cudaError_t le;
  if (p.H == 128) {
    static bool set128 = false;
    if (!set128) { PT_CUDA(cudaFuncSetAttribute(kv_append_attn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); set128 = true; }
    le = cudaLaunchKernelEx(&cfg, kv_append_attn_kernel<128>, p);
  } else {
    static bool set64 = false;
    if (!set64) { PT_CUDA(cudaFuncSetAttribute(kv_append_attn_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); set64 = true; }
    le = cudaLaunchKernelEx(&cfg, kv_append_attn_kernel<64>, p);
  }
  if (le != cudaSuccess) return pt::set_error(PT_ERR_CUDA, "pt_kv_append_attn: %s", cudaGetErrorString(le));
  PT_LAUNCH_CHECK("pt_kv_append_attn");
  return PT_OK;
}

extern "C" int pt_kv_export(const void *pool, const int32_t *page_table, const int32_t *step_dev, int batch, int n_kv, int head_dim,
                            int page_size, int max_pages, int max_len, void *dense_out, void *stream) {
  PT_REQUIRE(pool && page_table && step_dev && dense_out, "pt_kv_export: null pointer argument");
  PT_REQUIRE(head_dim % 8 == 0 && max_len <= page_size * max_pages, "pt_kv_export: max_len=%d exceeds page capacity %d", max_len,
             page_size * max_pages);
  kv_export_kernel<<<sm_count() * 4, 256, 0, as_stream(stream)>>>((const __half *)pool, page_table, step_dev, batch, n_kv, head_dim, page_size,
                                                          max_pages, max_len, (__half *)dense_out);
  PT_LAUNCH_CHECK("pt_kv_export");
  return PT_OK;
}

extern "C" int pt_kv_reorder_pages(void *pool, const int32_t *page_table, const int32_t *spare_pages, const int32_t *parent,
                                   const int32_t *step_dev, int rows, int n_kv, int head_dim, int page_size, int max_pages, void *stream) {
  PT_REQUIRE(pool && page_table && spare_pages && parent && step_dev, "pt_kv_reorder_pages: null pointer argument");
  PT_REQUIRE(rows > 0 && n_kv > 0 && head_dim % 8 == 0 && page_size > 0 && max_pages > 0, "pt_kv_reorder_pages: bad shape");
  dim3 grid(rows, 8);
  kv_reorder_pages_kernel<<<grid, 256, 0, as_stream(stream)>>>((__half *)pool, page_table, spare_pages, parent, step_dev, n_kv, head_dim,
                                                              page_size, max_pages);
  PT_LAUNCH_CHECK("pt_kv_reorder_pages");
  return PT_OK;
}

extern "C" int pt_kv_reorder_table(int32_t *page_table, int32_t *table_tmp, int32_t *spare_pages, const int32_t *parent,
                                   const int32_t *step_dev, int rows, int page_size, int max_pages, void *stream) {
  PT_REQUIRE(page_table && table_tmp && spare_pages && parent && step_dev, "pt_kv_reorder_table: null pointer argument");
  PT_REQUIRE(rows > 0 && page_size > 0 && max_pages > 0, "pt_kv_reorder_table: bad shape");
  cudaStream_t st = as_stream(stream);
  PT_CUDA(cudaMemcpyAsync(table_tmp, page_table, (size_t)rows * max_pages * sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
  kv_reorder_table_kernel<<<ceil_div(rows * max_pages, 256), 256, 0, st>>>(page_table, table_tmp, spare_pages, parent, step_dev, rows,
                                                                          page_size, max_pages);
  PT_LAUNCH_CHECK("pt_kv_reorder_table");
  return PT_OK;
}
