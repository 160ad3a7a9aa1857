// Paged KV cache: append of the new token fused with split flash-decode attention.
//
// One block handles one page (page_size cached tokens) of one (sequence, kv-head): its K and V tiles are contiguous in the
// pool.  The block that owns the page holding position `step` writes the new k/v into the pool and takes them from shared
// memory itself, so the append costs no extra pass over the cache.  Scores and P.V run on the tensor cores (see the kernel),
// the softmax statistics are warp-shuffle reductions.  Every block leaves (max, sum, partial output) in the workspace; the
// last block to arrive for a (sequence, kv-head) combines the pages in a fixed order, which keeps the result deterministic.
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
  uint8_t *out8;   // optional: the same output cast to E4M3 with inv_out_scale (the input of an FP8 linear), [B, n_head * H]
  float inv_out_scale;
  float *ws_o;     // [B, n_head, max_pages, H]
  float2 *ws_ml;   // [B, n_head, max_pages]
  int *counters;   // [B, n_kv, qsplit]
  int *error_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

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
constexpr int NQ_MAX = 8;   // q heads of one kv head per block: the n side of an m16n8 tensor-core tile (larger groups take several blocks)

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f2h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// One block = one page of one (sequence, kv head, part of the group's q heads).  Both products run on the tensor cores
// (mma.sync m16n8k16, fp32 accumulation of exact fp16 products):
//   scores^T [keys x heads] = K [keys x H] . q^T: warp w takes keys 16 w .. 16 w + 15 of each 64-key pass.  Its K rows go from
//     global memory STRAIGHT into the A fragments: a lane loads 16 bytes = channels 32 pp + 8 tig .. + 7 of its two key rows,
//     which serve two k-steps whose k order is a permutation of the channels (a dot product does not care, and q, the B operand,
//     is read from shared memory with the same permutation: the same 16 bytes of the head's row).  No shared-memory tile, no
//     bank conflicts, no barrier wait for K.
//   out [heads x H] += P [heads x keys] . V [keys x H]: P comes from the softmax weights in shared memory (rows = heads, padded
//     to 16 with zeros), V is staged in shared memory with padded rows and read through ldmatrix.trans; warp w owns H / 4 channels.
// The new token's key / value are staged in shared memory by the block that owns the last page and appended to the pool by one
// block per kv head.
template <int H>
__global__ void __launch_bounds__(kAttnThreads, 5) kv_append_attn_kernel(const AttnParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int VLD = H + 8;                               // V rows padded: ldmatrix reads 8 rows in 8 different bank groups
  constexpr int QLD = H + 32;                              // q rows: two heads read in one shared-memory phase sit 16 banks apart
  const int PAGE = p.page, KP = (PAGE + 15) & ~15;         // keys padded to whole 16-key steps
  const int PSLD = KP + 8;                                 // row stride of the score / weight rows
  __half *Vs = reinterpret_cast<__half *>(smem);           // [KP][VLD]
  __half *qs = Vs + (size_t)KP * VLD;                      // [NQ_MAX][QLD], rows >= nq are zero
  __half *newk = qs + (size_t)NQ_MAX * QLD;                // [H]: the new token's rotated key (owner block)
  float *ps = reinterpret_cast<float *>(newk + H);         // [NQ_MAX][PSLD]
  float *ml = ps + (size_t)NQ_MAX * PSLD;                  // [NQ_MAX][2]
  __shared__ int s_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tig = lane & 3;
  // With many q heads per kv head (multi-query attention) the heads of a group are shared out over `qsplit` blocks: each
  // re-reads the group's K/V page (through L2) and handles nq of the group's heads.
  const int pg = blockIdx.x, kvh = blockIdx.y / p.qsplit, qpart = blockIdx.y - kvh * p.qsplit, b = blockIdx.z;
  const int nq = p.qpk / p.qsplit, q_lo = qpart * nq;   // this block's heads of the group: q_lo .. q_lo + nq - 1
  if (p.pdl) {
    // let the next kernel start prefetching its weights; everything this kernel reads was produced upstream
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  // the page-table entry does not depend on the step: both loads go out together (one round trip less before the K / V loads)
  const int phys = p.page_table[(size_t)b * p.max_pages + pg];
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
  const int slot = n_valid - 1;                      // owner: where the new token goes

  __half *gK = p.pool + (((size_t)phys * 2 + 0) * p.n_kv + kvh) * PAGE * H;
  __half *gV = p.pool + (((size_t)phys * 2 + 1) * p.n_kv + kvh) * PAGE * H;

  // ---- this warp's K rows of the first 64-key pass, requested before anything else (keys 16 warp + g and + 8)
  uint4 kf[2][H / 32];
  auto load_k = [&](int kbase) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int key = kbase + g + 8 * r;
#pragma unroll
      for (int pp = 0; pp < H / 32; ++pp)
        kf[r][pp] = key < n_load ? __ldcg(reinterpret_cast<const uint4 *>(gK + (size_t)key * H + pp * 32 + tig * 8)) : make_uint4(0, 0, 0, 0);
    }
  };
  load_k(warp * 16);
  const int row_elems = (p.n_head + 2 * p.n_kv) * H;
  const __half *qrow = p.qkv + (size_t)b * row_elems;
  // ---- V page -> shared memory as asynchronous 16-byte copies (no registers, in flight together with the K loads above)
  const __half *vnew = qrow + (size_t)(p.n_head + p.n_kv + kvh) * H;
  for (int e = tid; e < KP * (H / 8); e += kAttnThreads) {
    const int r = e / (H / 8), c8 = e - r * (H / 8);
    __half *dst = Vs + (size_t)r * VLD + c8 * 8;
    if (r < n_load) {
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(gV + (size_t)r * H + c8 * 8) : "memory");
    } else {   // rows beyond the valid tokens multiply weights of zero: keep them finite; the new token's row comes from qkv
      uint4 v = make_uint4(0, 0, 0, 0);
      if (owner && r == slot) v = *reinterpret_cast<const uint4 *>(vnew + c8 * 8);
      *reinterpret_cast<uint4 *>(dst) = v;
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");

  // ---- RoPE on the block's q heads (and on the new k)
  const __half *sin_r = p.sin_t + (size_t)step * p.rot_half;
  const __half *cos_r = p.cos_t + (size_t)step * p.rot_half;
  for (int i = tid; i < (NQ_MAX - nq) * (H / 2); i += kAttnThreads) {   // unused head rows of the B operand: zeros
    const int qh = nq + i / (H / 2), j = i - (qh - nq) * (H / 2);
    reinterpret_cast<uint32_t *>(qs + (size_t)qh * QLD)[j] = 0u;
  }
  for (int i = tid; i < nq * (H / 2); i += kAttnThreads) {
    const int qh = i / (H / 2), j = i - qh * (H / 2);
    rope_pair(p, qrow + (size_t)(kvh * p.qpk + q_lo + qh) * H, sin_r, cos_r, j, qs + (size_t)qh * QLD);
  }
  if (owner) {
    const __half *knew = qrow + (size_t)(p.n_head + kvh) * H;
    for (int j = tid; j < H / 2; j += kAttnThreads) rope_pair(p, knew, sin_r, cos_r, j, newk);
  }
  for (int i = tid; i < NQ_MAX * PSLD; i += kAttnThreads) ps[i] = 0.f;   // weights of padded keys and unused heads
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncthreads();
  if (owner && qpart == 0) {   // one block of the group appends to the pool
    for (int j = tid; j < H; j += kAttnThreads) {
      gK[(size_t)slot * H + j] = newk[j];
      gV[(size_t)slot * H + j] = Vs[(size_t)slot * VLD + j];
    }
  }

  // ---- scores: keys 16 warp .. + 15 of every 64-key pass against the block's heads
  for (int kbase = warp * 16; kbase < n_valid; kbase += 64) {
    if (kbase != warp * 16) load_k(kbase);
    if (owner) {   // the new token's key row comes from shared memory
#pragma unroll
      for (int r = 0; r < 2; ++r)
        if (kbase + g + 8 * r == slot) {
#pragma unroll
          for (int pp = 0; pp < H / 32; ++pp) kf[r][pp] = *reinterpret_cast<const uint4 *>(newk + pp * 32 + tig * 8);
        }
    }
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int pp = 0; pp < H / 32; ++pp) {
      const uint4 qv = *reinterpret_cast<const uint4 *>(qs + (size_t)g * QLD + pp * 32 + tig * 8);
      mma_f16(sc, kf[0][pp].x, kf[1][pp].x, kf[0][pp].y, kf[1][pp].y, qv.x, qv.y);
      mma_f16(sc, kf[0][pp].z, kf[1][pp].z, kf[0][pp].w, kf[1][pp].w, qv.z, qv.w);
    }
    // lane (g, tig): keys kbase + g (sc[0], sc[1]) and kbase + g + 8 (sc[2], sc[3]) against heads 2 tig and 2 tig + 1
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = kbase + g + 8 * (e >> 1), qh = 2 * tig + (e & 1);
      if (key < n_valid && qh < nq) {
        __half s16 = __float2half_rn(sc[e]);           // fp16 matmul output
        if (p.use_scale) s16 = h_mul(s16, p.scale_h);  // ops.mul by fp16(1/sqrt(H))
        ps[(size_t)qh * PSLD + key] = __half2float(s16);
      }
    }
  }
  __syncthreads();

  // ---- per-head softmax statistics (one warp per q head, warp-shuffle reductions)
  for (int qh = warp; qh < nq; qh += kAttnThreads / 32) {
    float *pr = ps + (size_t)qh * PSLD;
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

  // ---- P.V: warp w owns channels [w H/4, (w + 1) H/4); rows of the A operand = heads (8 .. 15 are zero)
  const size_t head0 = (size_t)b * p.n_head + (size_t)kvh * p.qpk + q_lo;
  {
    constexpr int NT = H / 32;                 // 8-channel tiles per warp
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    const float *pr = ps + (size_t)g * PSLD + 2 * tig;      // g < NQ_MAX: rows of unused heads are zero
    const uint32_t v_lane = smem_u32(Vs + (size_t)(lane & 15) * VLD + warp * (H / 4) + (lane >> 4) * 8);
    for (int k2 = 0; k2 * 16 < n_valid; ++k2) {
      // The weights are rounded to fp16 for the tensor core; they are at most 1 (max-subtracted mode) or fp16 values already
      // (the reference's fp16 softmax mode), so this costs at most 2^-11 relative per weight.
      const float2 p0 = *reinterpret_cast<const float2 *>(pr + k2 * 16), p1 = *reinterpret_cast<const float2 *>(pr + k2 * 16 + 8);
      const uint32_t a0 = pack_f2h2(p0.x, p0.y), a2 = pack_f2h2(p1.x, p1.y);
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(v_lane + (uint32_t)(k2 * 16 * VLD + j * 8) * 2u, b0, b1, b2, b3);
        mma_f16(o[j], a0, 0u, a2, 0u, b0, b1);
        if (j + 1 < NT) mma_f16(o[j + 1], a0, 0u, a2, 0u, b2, b3);
      }
    }
    if (g < nq) {
#pragma unroll
      for (int j = 0; j < NT; ++j)
        *reinterpret_cast<float2 *>(&p.ws_o[((head0 + g) * p.max_pages + pg) * H + warp * (H / 4) + j * 8 + 2 * tig]) = make_float2(o[j][0], o[j][1]);
    }
  }
  if (tid < nq) p.ws_ml[(head0 + tid) * p.max_pages + pg] = make_float2(ml[2 * tid], ml[2 * tid + 1]);

  // ---- last block to arrive for this (sequence, kv-head) combines the pages in page order
  __threadfence();
  __syncthreads();
  int *ctr = p.counters + ((size_t)b * p.n_kv + kvh) * p.qsplit + qpart;
  if (tid == 0) s_last = (atomicAdd(ctr, 1) == n_active - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (tid == 0) *ctr = 0;
  // The V tile is no longer needed: its shared memory takes the pages' (max, sum) pairs, then their weights.  All loads of a
  // stage are issued before the first is used, so the combine costs a handful of L2 round trips whatever the number of pages
  // and heads (a loop of dependent-looking loads per head and page made it the longest part of the kernel at 17 pages).
  float *cw = reinterpret_cast<float *>(Vs);           // [nq][n_active] weights exp(m_i - M)
  float *cl = cw + (size_t)nq * n_active;              // [nq][n_active] page sums, then cl[qh * n_active] = L of the head
  // (worth its two extra barriers from about sixteen (head, page) pairs on: measured 1 % slower than the plain loop at 1 head x 6 pages)
  const bool staged = nq * n_active >= 16 && (size_t)2 * nq * n_active * sizeof(float) <= (size_t)KP * VLD * sizeof(__half);
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
        const __half y0 = __float2half_rn(o0 / cl[(size_t)q0 * n_active]);
        dst[0] = y0;
        uint8_t *dst8 = p.out8 ? p.out8 + (size_t)b * p.n_head * H + ((size_t)kvh * p.qpk + q_lo + q0) * H + tid : nullptr;
        if (dst8) dst8[0] = (uint8_t)__nv_cvt_float_to_fp8(__half2float(y0) * p.inv_out_scale, __NV_SATFINITE, __NV_E4M3);
        if (two) {
          const __half y1 = __float2half_rn(o1 / cl[(size_t)(q0 + 1) * n_active]);
          dst[H] = y1;
          if (dst8) dst8[H] = (uint8_t)__nv_cvt_float_to_fp8(__half2float(y1) * p.inv_out_scale, __NV_SATFINITE, __NV_E4M3);
        }
      }
    }
    return;
  }
  if (tid < H) {   // few pages and heads: the plain loop
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
      const __half y = __float2half_rn(o / L);
      p.out[(size_t)b * p.out_ld + ((size_t)kvh * p.qpk + q_lo + qh) * H + tid] = y;
      if (p.out8)
        p.out8[(size_t)b * p.n_head * H + ((size_t)kvh * p.qpk + q_lo + qh) * H + tid] =
            (uint8_t)__nv_cvt_float_to_fp8(__half2float(y) * p.inv_out_scale, __NV_SATFINITE, __NV_E4M3);
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
  {  // at most NQ_MAX q heads per block (the n side of the tensor-core tile): larger groups are shared out over several blocks
    int nq_blk = p.qpk;
    if (p.qpk > NQ_MAX)
      for (nq_blk = NQ_MAX; p.qpk % nq_blk; --nq_blk) {}
    p.qsplit = p.qpk / nq_blk;
  }
  p.page = a->page_size; p.max_pages = a->max_pages; p.rope_mode = a->rope_mode; p.softmax_mode = a->softmax_mode;
  p.rot_half = a->rope_mode == PT_ROPE_CHATGLM2 ? a->head_dim / 4 : a->head_dim / 2;
  p.out_ld = a->out_ld > 0 ? a->out_ld : a->n_head * a->head_dim;
  p.use_scale = a->score_scale != 1.0f;
  p.scale_h = __float2half_rn(a->score_scale);
  p.step = a->step_dev;
  p.qkv = (const __half *)a->qkv; p.sin_t = (const __half *)a->rope_sin; p.cos_t = (const __half *)a->rope_cos;
  p.pool = (__half *)a->pool; p.page_table = a->page_table; p.out = (__half *)a->out;
  p.out8 = (uint8_t *)a->out_fp8;
  PT_REQUIRE(!a->out_fp8 || a->out_fp8_scale > 0.f, "pt_kv_append_attn: out_fp8 needs out_fp8_scale > 0");
  p.inv_out_scale = a->out_fp8 ? 1.0f / a->out_fp8_scale : 0.f;
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
  (void)nq;
  const int kp = (p.page + 15) & ~15;
  const size_t smem = ((size_t)kp * (p.H + 8) + (size_t)NQ_MAX * (p.H + 32) + p.H) * sizeof(__half) +
                      ((size_t)NQ_MAX * (kp + 8) + (size_t)NQ_MAX * 2) * sizeof(float);
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
