// Prompt ingestion ("prefill") attention for the Llama architecture: all tokens of a prompt in one pass instead of one decode
// step per token.  The reference's two-stage models process the prompt with sequence_length = prompt length
// (poptransformer/models/base_model.py:358-494); its attention for sequence_length != 1 is the same chain as for decode with a
// causal mask and a softmax WITH max subtraction (llama2/attention.py:97-114: stable_mode = seq_len != 1).
//
//   prefill_rope_kv_kernel : RoPE (llama2/attention.py:28-56, same fp16 roundings as the decode kernels) on q and k of every
//                            prompt token; k and v go to their slots of the paged cache, q is rotated in place.
//   prefill_attn_kernel    : one block per (sequence, head, 64 query tokens), 16 queries per warp; keys come page by page (64
//                            tokens, contiguous 16 KB for K and for V) from the paged cache, which now also holds the prompt's
//                            own keys; Q K^T and P V run on the tensor cores (mma.sync m16n8k16, fp32 accumulation); scores are
//                            rounded like the reference's fp16 matmul output and scaled in fp16, softmax statistics are fp32
//                            and online (running max / sum per query), probabilities are fp16 like the reference's.
// The linears around it run on the tcgen05 GEMM.
#include "tile_math.cuh"

namespace pt {
namespace pf {

constexpr int H = 128, PAGE = 64, BQ = 64, THREADS = 128, KPAD = 136;   // K / V rows padded to 136 halfs: fragment loads hit 32 different banks

struct Params {
  int B, P, start, n_head, max_pages;
  const __half *sin_t, *cos_t;
  __half *qkv;              // [B * P, 3 * n_head * H], row b * P + t
  __half *pool;
  const int *page_table;    // [B, max_pages]
  __half *out;              // [B * P, n_head * H]
  __half scale_h;
};

// x rows of the prompt tokens (row b * n_tokens + t <- table[ids[b, start + t]]) and the stop mask the token-by-token loop would
// have built over them: its step s marks a sequence whose id at position s + 1 is the eos id (models/base_model.py:313-346).
__global__ void prefill_embed_kernel(const uint4 *__restrict__ table, const int *__restrict__ ids, int ids_stride, int n_tokens, int start, int dim8,
                                     int vocab, int eos_id, int *stop_mask, uint4 *__restrict__ out) {
  const int row = blockIdx.x, b = row / n_tokens, t = row - b * n_tokens;
  int id = ids[(size_t)b * ids_stride + start + t];
  id = min(max(id, 0), vocab - 1);
  for (int i = threadIdx.x; i < dim8; i += blockDim.x) out[(size_t)row * dim8 + i] = table[(size_t)id * dim8 + i];
  if (threadIdx.x == 0 && stop_mask && start + t + 1 < ids_stride && ids[(size_t)b * ids_stride + start + t + 1] == eos_id) atomicOr(stop_mask + b, 1);
}

__global__ void __launch_bounds__(64) prefill_rope_kv_kernel(const Params p) {
  const int row = blockIdx.x, head = blockIdx.y, i = threadIdx.x;     // i: pair (i, i + 64)
  const int b = row / p.P, t = row - b * p.P, pos = p.start + t;
  const int dq = p.n_head * H;
  __half *q = p.qkv + (size_t)row * 3 * dq + (size_t)head * H, *k = q + dq, *v = k + dq;
  const __half s = p.sin_t[(size_t)pos * (H / 2) + i], c = p.cos_t[(size_t)pos * (H / 2) + i];
  const __half q1 = q[i], q2 = q[i + 64], k1 = k[i], k2 = k[i + 64];
  q[i] = h_add(h_mul(q1, c), h_mul(__hneg(q2), s));
  q[i + 64] = h_add(h_mul(q2, c), h_mul(q1, s));
  const int phys = p.page_table[(size_t)b * p.max_pages + pos / PAGE], slot = pos % PAGE;
  __half *gK = p.pool + (((size_t)phys * 2 + 0) * p.n_head + head) * PAGE * H + (size_t)slot * H;
  __half *gV = p.pool + (((size_t)phys * 2 + 1) * p.n_head + head) * PAGE * H + (size_t)slot * H;
  gK[i] = h_add(h_mul(k1, c), h_mul(__hneg(k2), s));
  gK[i + 64] = h_add(h_mul(k2, c), h_mul(k1, s));
  gV[i] = v[i];
  gV[i + 64] = v[i + 64];
}

// ldmatrix of four 8x8 b16 matrices, transposed on the way: from a row-major [key][channel] tile this yields the B fragments
// (k = key, n = channel) of two adjacent channel tiles for one 16-key step.
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// One block per (sequence, head, 64 query tokens): warp w owns queries 16 w .. 16 w + 15 of the tile, their q fragments stay in
// registers.  Per page of 64 keys: S = Q K^T as 8 x 8 m16n8k16 tensor-core steps per warp (fp32 sums of exact fp16 products,
// rounded to fp16 and scaled in fp16 like the reference's matmul output times its fp16 constant), causal mask, online softmax
// (running max / sum per query, fp32), the probabilities rounded to fp16 (the reference's softmax output is fp16) and used as
// the A operand of O += P V (4 x 16 steps), fp32 accumulators.
__global__ void __launch_bounds__(THREADS) prefill_attn_kernel(const Params p) {
  __shared__ __align__(16) __half Ks[PAGE][KPAD];
  __shared__ __align__(16) __half Vs[PAGE][KPAD];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tig = lane & 3;
  const int t0 = blockIdx.x * BQ, head = blockIdx.y, b = blockIdx.z;
  const int dq = p.n_head * H;
  const int q0 = t0 + warp * 16 + g, q1 = q0 + 8;                     // this lane's two query tokens (rows g and g + 8 of the warp's tile)
  const bool ok0 = q0 < p.P, ok1 = q1 < p.P;
  const int pos0 = p.start + q0, pos1 = p.start + q1;
  // Q fragments (already rotated by prefill_rope_kv_kernel): a0 / a2 = row g, a1 / a3 = row g + 8, channels 16 kk + 2 tig (+8)
  uint32_t qa[H / 16][4];
  {
    const __half *r0 = p.qkv + (size_t)(b * p.P + (ok0 ? q0 : 0)) * 3 * dq + (size_t)head * H + 2 * tig;
    const __half *r1 = p.qkv + (size_t)(b * p.P + (ok1 ? q1 : 0)) * 3 * dq + (size_t)head * H + 2 * tig;
#pragma unroll
    for (int kk = 0; kk < H / 16; ++kk) {
      qa[kk][0] = ok0 ? *reinterpret_cast<const uint32_t *>(r0 + kk * 16) : 0u;
      qa[kk][1] = ok1 ? *reinterpret_cast<const uint32_t *>(r1 + kk * 16) : 0u;
      qa[kk][2] = ok0 ? *reinterpret_cast<const uint32_t *>(r0 + kk * 16 + 8) : 0u;
      qa[kk][3] = ok1 ? *reinterpret_cast<const uint32_t *>(r1 + kk * 16 + 8) : 0u;
    }
  }
  float o[H / 8][4];
#pragma unroll
  for (int j = 0; j < H / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int last_pos = p.start + min(p.P, t0 + BQ) - 1;               // newest key any query of the tile may see
  const int warp_last = p.start + min(p.P, t0 + warp * 16 + 16) - 1;  // ... and any query of this warp
  for (int pg = 0; pg * PAGE <= last_pos; ++pg) {
    __syncthreads();                                                 // previous tiles consumed
    const int phys = p.page_table[(size_t)b * p.max_pages + pg];
    const __half *gK = p.pool + (((size_t)phys * 2 + 0) * p.n_head + head) * PAGE * H;
    const __half *gV = p.pool + (((size_t)phys * 2 + 1) * p.n_head + head) * PAGE * H;
    for (int e = tid; e < PAGE * (H / 8); e += THREADS) {
      const int r = e / (H / 8), c8 = e - r * (H / 8);
      *reinterpret_cast<uint4 *>(&Ks[r][c8 * 8]) = *reinterpret_cast<const uint4 *>(gK + (size_t)r * H + c8 * 8);
      *reinterpret_cast<uint4 *>(&Vs[r][c8 * 8]) = *reinterpret_cast<const uint4 *>(gV + (size_t)r * H + c8 * 8);
    }
    __syncthreads();
    if (pg * PAGE > warp_last) continue;                             // nothing of this page is visible to this warp's queries (uniform per warp)
    // ---- scores of the warp's 16 queries against the page's 64 keys
    float sc[PAGE / 8][4];
#pragma unroll
    for (int j = 0; j < PAGE / 8; ++j) {
      sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
      const __half *kr = &Ks[j * 8 + g][2 * tig];
#pragma unroll
      for (int kk = 0; kk < H / 16; ++kk)
        mma16816(sc[j], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], *reinterpret_cast<const uint32_t *>(kr + kk * 16),
                 *reinterpret_cast<const uint32_t *>(kr + kk * 16 + 8));
    }
    float m_tile[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < PAGE / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kpos = pg * PAGE + j * 8 + 2 * tig + (e & 1);
        const bool vis = (e < 2) ? (ok0 && kpos <= pos0) : (ok1 && kpos <= pos1);
        const float v = vis ? __half2float(h_mul(__float2half_rn(sc[j][e]), p.scale_h)) : -INFINITY;
        sc[j][e] = v;
        m_tile[e >> 1] = fmaxf(m_tile[e >> 1], v);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      m_tile[r] = fmaxf(m_tile[r], __shfl_xor_sync(0xffffffffu, m_tile[r], 1));
      m_tile[r] = fmaxf(m_tile[r], __shfl_xor_sync(0xffffffffu, m_tile[r], 2));
      const float m_new = fmaxf(m_run[r], m_tile[r]);
      corr[r] = (m_new == -INFINITY) ? 1.f : expf(m_run[r] - m_new);    // exp(-inf) = 0 the first time
      m_run[r] = m_new;
    }
    float l_tile[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < PAGE / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // the probability as the reference holds it: fp16; the row sum adds the rounded values, like the division would see them
        const float pe = (sc[j][e] == -INFINITY) ? 0.f : __half2float(__float2half_rn(expf(sc[j][e] - m_run[e >> 1])));
        sc[j][e] = pe;
        l_tile[e >> 1] += pe;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_tile[r] += __shfl_xor_sync(0xffffffffu, l_tile[r], 1);
      l_tile[r] += __shfl_xor_sync(0xffffffffu, l_tile[r], 2);
      l_run[r] = l_run[r] * corr[r] + l_tile[r];
    }
#pragma unroll
    for (int j = 0; j < H / 8; ++j) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0];
      o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }
    // ---- O += P V: the score accumulators of two adjacent key tiles are the A fragment of one 16-key step
    const uint32_t v_lane = smem_addr(&Vs[lane & 15][(lane >> 4) * 8]);
#pragma unroll
    for (int k2 = 0; k2 < PAGE / 16; ++k2) {
      const uint32_t a0 = pack_h2(sc[2 * k2][0], sc[2 * k2][1]), a1 = pack_h2(sc[2 * k2][2], sc[2 * k2][3]);
      const uint32_t a2 = pack_h2(sc[2 * k2 + 1][0], sc[2 * k2 + 1][1]), a3 = pack_h2(sc[2 * k2 + 1][2], sc[2 * k2 + 1][3]);
#pragma unroll
      for (int jn = 0; jn < H / 8; jn += 2) {
        uint32_t b0, b1, b2, b3;   // keys 16 k2 .. +15: channels 8 jn .. +7 (b0, b1) and 8 jn + 8 .. +15 (b2, b3)
        ldmatrix_x4_trans(v_lane + (uint32_t)(k2 * 16 * KPAD + jn * 8) * 2u, b0, b1, b2, b3);
        mma16816(o[jn], a0, a1, a2, a3, b0, b1);
        mma16816(o[jn + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  const float inv0 = ok0 ? 1.0f / l_run[0] : 0.f, inv1 = ok1 ? 1.0f / l_run[1] : 0.f;
  __half *d0 = p.out + (size_t)(b * p.P + (ok0 ? q0 : 0)) * dq + (size_t)head * H + 2 * tig;
  __half *d1 = p.out + (size_t)(b * p.P + (ok1 ? q1 : 0)) * dq + (size_t)head * H + 2 * tig;
#pragma unroll
  for (int j = 0; j < H / 8; ++j) {
    if (ok0) *reinterpret_cast<uint32_t *>(d0 + j * 8) = pack_h2(o[j][0] * inv0, o[j][1] * inv0);
    if (ok1) *reinterpret_cast<uint32_t *>(d1 + j * 8) = pack_h2(o[j][2] * inv1, o[j][3] * inv1);
  }
}

}  // namespace pf
}  // namespace pt

using namespace pt;

extern "C" int pt_prefill_embed(const void *table, const int32_t *ids, int ids_stride, int batch, int n_tokens, int start, int dim, int vocab, int eos_id,
                                int32_t *stop_mask, void *out, void *stream) {
  PT_REQUIRE(table && ids && out, "pt_prefill_embed: null pointer argument");
  PT_REQUIRE(batch > 0 && n_tokens > 0 && start >= 0 && start + n_tokens <= ids_stride && dim > 0 && dim % 8 == 0 && vocab > 0,
             "pt_prefill_embed: bad shape batch=%d n_tokens=%d start=%d ids_stride=%d dim=%d", batch, n_tokens, start, ids_stride, dim);
  pf::prefill_embed_kernel<<<batch * n_tokens, 128, 0, as_stream(stream)>>>((const uint4 *)table, ids, ids_stride, n_tokens, start, dim / 8, vocab, eos_id,
                                                                            stop_mask, (uint4 *)out);
  PT_LAUNCH_CHECK("pt_prefill_embed");
  return PT_OK;
}

extern "C" int pt_prefill_attn(const pt_prefill_attn_args *a, void *stream) {
  PT_REQUIRE(a, "pt_prefill_attn: null args");
  PT_REQUIRE(a->batch > 0 && a->n_tokens > 0 && a->n_head > 0 && a->start >= 0, "pt_prefill_attn: bad shape batch=%d n_tokens=%d n_head=%d start=%d",
             a->batch, a->n_tokens, a->n_head, a->start);
  PT_REQUIRE(a->head_dim == pf::H && a->page_size == pf::PAGE, "pt_prefill_attn: needs head_dim=%d and page_size=%d", pf::H, pf::PAGE);
  PT_REQUIRE(a->start + a->n_tokens <= a->max_len && a->max_len <= a->page_size * a->max_pages,
             "pt_prefill_attn: positions %d..%d exceed max_len=%d (page table: %d positions)", a->start, a->start + a->n_tokens - 1, a->max_len,
             a->page_size * a->max_pages);
  PT_REQUIRE(a->qkv && a->rope_sin && a->rope_cos && a->pool && a->page_table && a->out, "pt_prefill_attn: null pointer argument");
  pf::Params p{};
  p.B = a->batch; p.P = a->n_tokens; p.start = a->start; p.n_head = a->n_head; p.max_pages = a->max_pages;
  p.sin_t = (const __half *)a->rope_sin; p.cos_t = (const __half *)a->rope_cos;
  p.qkv = (__half *)a->qkv; p.pool = (__half *)a->pool; p.page_table = a->page_table; p.out = (__half *)a->out;
  p.scale_h = __float2half_rn(a->score_scale);
  pf::prefill_rope_kv_kernel<<<dim3(a->batch * a->n_tokens, a->n_head), 64, 0, as_stream(stream)>>>(p);
  PT_LAUNCH_CHECK("pt_prefill_attn");
  pf::prefill_attn_kernel<<<dim3(ceil_div(a->n_tokens, pf::BQ), a->n_head, a->batch), pf::THREADS, 0, as_stream(stream)>>>(p);
  PT_LAUNCH_CHECK("pt_prefill_attn");
  return PT_OK;
}
