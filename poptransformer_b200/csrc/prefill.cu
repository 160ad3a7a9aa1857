// Prompt ingestion ("prefill") attention for the Llama architecture: all tokens of a prompt in one pass instead of one decode
// step per token.  The reference's two-stage models process the prompt with sequence_length = prompt length
// (poptransformer/models/base_model.py:358-494); its attention for sequence_length != 1 is the same chain as for decode with a
// causal mask and a softmax WITH max subtraction (llama2/attention.py:97-114: stable_mode = seq_len != 1).
//
//   prefill_rope_kv_kernel : RoPE (llama2/attention.py:28-56, same fp16 roundings as the decode kernels) on q and k of every
//                            prompt token; k and v go to their slots of the paged cache, q is rotated in place.
//   prefill_attn_kernel    : one block per (sequence, head, 16 query tokens); keys come page by page (64 tokens, contiguous
//                            16 KB for K and for V) from the paged cache, which now also holds the prompt's own keys; scores
//                            are rounded like the reference's fp16 matmul output and scaled in fp16, softmax statistics are
//                            fp32 and online (running max / sum per query), P.V accumulates in fp32.
// Compute-bound on the CUDA cores (2 x 128 FMA per (query, key)); the linears around it run on the tcgen05 GEMM.
#include "tile_math.cuh"

namespace pt {
namespace pf {

constexpr int H = 128, PAGE = 64, QT = 16, THREADS = 128, KPAD = 136;   // key rows padded to 136 halfs: 8 lanes read 8 different rows

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

__global__ void __launch_bounds__(THREADS) prefill_attn_kernel(const Params p) {
  __shared__ __align__(16) __half Qs[QT][H];
  __shared__ __align__(16) __half Ks[PAGE][KPAD];
  __shared__ __align__(16) __half Vs[PAGE][H];
  __shared__ float Ps[QT][PAGE + 1];
  const int tid = threadIdx.x, qi = tid >> 3, l8 = tid & 7;           // 16 queries x 8 lanes
  const int t0 = blockIdx.x * QT, head = blockIdx.y, b = blockIdx.z;
  const int dq = p.n_head * H;
  const int qt = t0 + qi;                                            // this thread's query token (may be beyond the prompt)
  const bool q_ok = qt < p.P;
  const int qpos = p.start + qt;
  for (int e = tid; e < QT * (H / 8); e += THREADS) {                // Q tile (already rotated)
    const int r = e / (H / 8), c8 = e - r * (H / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t0 + r < p.P) v = *reinterpret_cast<const uint4 *>(p.qkv + (size_t)(b * p.P + t0 + r) * 3 * dq + (size_t)head * H + c8 * 8);
    *reinterpret_cast<uint4 *>(&Qs[r][c8 * 8]) = v;
  }
  float m_run = -INFINITY, l_run = 0.f, acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.f;
  const int last_pos = p.start + min(p.P, t0 + QT) - 1;               // newest key any query of the tile may see
  for (int pg = 0; pg * PAGE <= last_pos; ++pg) {
    __syncthreads();                                                 // previous tile consumed (and Q staged)
    const int phys = p.page_table[(size_t)b * p.max_pages + pg];
    const __half *gK = p.pool + (((size_t)phys * 2 + 0) * p.n_head + head) * PAGE * H;
    const __half *gV = p.pool + (((size_t)phys * 2 + 1) * p.n_head + head) * PAGE * H;
    for (int e = tid; e < PAGE * (H / 8); e += THREADS) {
      const int r = e / (H / 8), c8 = e - r * (H / 8);
      *reinterpret_cast<uint4 *>(&Ks[r][c8 * 8]) = *reinterpret_cast<const uint4 *>(gK + (size_t)r * H + c8 * 8);
      *reinterpret_cast<uint4 *>(&Vs[r][c8 * 8]) = *reinterpret_cast<const uint4 *>(gV + (size_t)r * H + c8 * 8);
    }
    __syncthreads();
    // scores of this thread's query against keys l8, l8 + 8, ...: fp32 dot, rounded to fp16, scaled in fp16 (the reference's fp16
    // matmul output times its fp16 constant), causal mask
    float s[8], m_tile = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int kr = l8 + 8 * j, kpos = pg * PAGE + kr;
      float d = 0.f;
#pragma unroll 4
      for (int c8 = 0; c8 < H / 8; ++c8) {
        const uint4 kq = *reinterpret_cast<const uint4 *>(&Ks[kr][c8 * 8]);
        const uint4 qq = *reinterpret_cast<const uint4 *>(&Qs[qi][c8 * 8]);
        const __half2 *kh = reinterpret_cast<const __half2 *>(&kq), *qh = reinterpret_cast<const __half2 *>(&qq);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float2 a = __half22float2(kh[u]), q2 = __half22float2(qh[u]);
          d = fmaf(a.x, q2.x, d);
          d = fmaf(a.y, q2.y, d);
        }
      }
      s[j] = (q_ok && kpos <= qpos) ? __half2float(h_mul(__float2half_rn(d), p.scale_h)) : -INFINITY;
      m_tile = fmaxf(m_tile, s[j]);
    }
    m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
    m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
    m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 4));
    const float m_new = fmaxf(m_run, m_tile);
    const float corr = (m_new == -INFINITY) ? 1.f : expf(m_run - m_new);   // exp(-inf) = 0 the first time
    float l_tile = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float e = (s[j] == -INFINITY) ? 0.f : expf(s[j] - m_new);
      Ps[qi][l8 + 8 * j] = e;
      l_tile += e;
    }
    l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 1);
    l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 2);
    l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 4);
    l_run = l_run * corr + l_tile;
    m_run = m_new;
    __syncwarp();                                                    // the 8 lanes of a query sit in one warp: Ps[qi] is complete
    // P.V: this thread owns channels [16 l8, 16 l8 + 16) of its query
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] *= corr;
    for (int kr = 0; kr < PAGE; ++kr) {
      const float e = Ps[qi][kr];
      const uint4 v0 = *reinterpret_cast<const uint4 *>(&Vs[kr][l8 * 16]), v1 = *reinterpret_cast<const uint4 *>(&Vs[kr][l8 * 16 + 8]);
      const __half2 *h0 = reinterpret_cast<const __half2 *>(&v0), *h1 = reinterpret_cast<const __half2 *>(&v1);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 a = __half22float2(h0[u]), c2 = __half22float2(h1[u]);
        acc[2 * u] = fmaf(e, a.x, acc[2 * u]);
        acc[2 * u + 1] = fmaf(e, a.y, acc[2 * u + 1]);
        acc[8 + 2 * u] = fmaf(e, c2.x, acc[8 + 2 * u]);
        acc[8 + 2 * u + 1] = fmaf(e, c2.y, acc[8 + 2 * u + 1]);
      }
    }
  }
  if (q_ok) {
    const float inv = 1.0f / l_run;
    __half o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j] = __float2half_rn(acc[j] * inv);
    __half *dst = p.out + (size_t)(b * p.P + qt) * dq + (size_t)head * H + l8 * 16;
    *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(&o[0]);
    *reinterpret_cast<uint4 *>(dst + 8) = *reinterpret_cast<const uint4 *>(&o[8]);
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
  pf::prefill_attn_kernel<<<dim3(ceil_div(a->n_tokens, pf::QT), a->n_head, a->batch), pf::THREADS, 0, as_stream(stream)>>>(p);
  PT_LAUNCH_CHECK("pt_prefill_attn");
  return PT_OK;
}
