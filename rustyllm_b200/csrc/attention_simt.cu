// Attention of the step's query tokens over the paged key/value cache, on the CUDA
// cores, for any head size up to 1,024 (steps of 2), any number of heads and groups,
// float or bf16 storage.  Serves prefill and decode alike: a query token at
// position p attends to cached positions [max(0, p + 1 - window), p] of its own
// sequence (with `chunk` > 0 instead: to [p - p % chunk, p], the positions of its own
// block of `chunk` positions counted from the sequence's start), which the rope/cache-write
// kernel has filled before this runs.
//
// Formulas (SimonWaldherr/RustyLLM): query head h uses KV head g = h / (H/G)
// (src/model.rs:6034-6198); score_t = (q_h . K[t, g]) / sqrt(head_dim); streaming
// softmax with running (max, denominator, output) in 32-bit (src/model.rs:5807-5869);
// causality by loop bound, window start max(0, pos + 1 - W) (src/model.rs:7239-7243).
//
// One CTA of eight warps per (token, query head).  Keys are taken 32 at a time in position
// order, chunk c of a token's keys by warp c % 8; within a chunk every key's row is read by
// the whole warp (lane l holds dimensions l, l + 32, ...: consecutive lanes, consecutive
// addresses, for keys and values alike) and its score is the warp's sum of the lanes'
// partial products.  At the end the warps' (max, denominator, output) are merged in the order
// of the warps.  Chunks, their warps and every order of summation depend on the token's
// position and the window alone, so the result for a position does not depend on the batch
// or on how the tokens were split into steps - bit for bit.
#include <math.h>

#include "common.cuh"

#define ATT_WARPS 8
#define ATT_MAX_HD 1024        // rows of 256 elements and less run the kernel with 8 elements a lane, wider ones with 32

template <typename T, int NE>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ k_pool,
                      const T* __restrict__ v_pool, const int* __restrict__ page_table, int max_pages,
                      const int* __restrict__ slot_of_token, const int* __restrict__ positions,
                      T* __restrict__ out, int ldo, int H, int G, int hd, int vd, float scale, int window,
                      int sink, const T* __restrict__ gate, int ldg, float softcap, int keep_first, int chunk, int ldv,
                      int gate_per_head) {
  __shared__ float s_acc[ATT_WARPS][NE * 32];
  __shared__ float s_max[ATT_WARPS], s_sum[ATT_WARPS];
  const int m = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = h / (H / G);
  const int pos = positions[m];
  const int slot = slot_of_token[m];
  const int* pages = page_table + (size_t)slot * max_pages;
  const T* qrow = q + (size_t)m * ldq + (size_t)h * hd;
  float qv[NE];                       // this lane's dimensions of the query, scaled
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    const int d = lane + 32 * e;
    qv[e] = d < hd ? rl_ld(qrow + d) * scale : 0.f;
  }

  const int start = chunk > 0 ? pos - pos % chunk : (window > 0 && pos + 1 - window > 0) ? pos + 1 - window : 0;
  // kept first tokens: positions [0, nfirst) in front of the window are seen as well.  The keys are walked
  // as one run of `total` places: place v is position v for v < nfirst and start + (v - nfirst) behind.
  const int nfirst = min(keep_first, start);
  const int total = nfirst + pos - start + 1;
  const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
  float acc[NE];
#pragma unroll
  for (int e = 0; e < NE; ++e) acc[e] = 0.f;
  float run_max = -INFINITY, run_sum = 0.f;
  // a value row is `ldv` elements long (its first vd are the value): ldv = vd for a pool of values of its own,
  // ldv = hd where the values are the front part of the key rows and v_pool is the key pool
  const size_t head_off = (size_t)g * RL_PAGE * hd, v_head_off = (size_t)g * RL_PAGE * ldv;
  const size_t page_stride = (size_t)G * RL_PAGE * hd, v_page_stride = (size_t)G * RL_PAGE * ldv;

  for (int v0 = 32 * warp; v0 < total; v0 += 32 * ATT_WARPS) {
    const int n = min(32, total - v0);
    float s = -INFINITY;              // lane j: the score of the key at place v0 + j
    for (int j = 0; j < n; ++j) {
      const int tj = v0 + j < nfirst ? v0 + j : start + (v0 + j - nfirst);
      const T* krow = k_pool + (size_t)pages[tj / RL_PAGE] * page_stride + head_off + (size_t)(tj % RL_PAGE) * hd;
      float part = 0.f;
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        const int d = lane + 32 * e;
        if (d < hd) part = fmaf(qv[e], rl_ld(krow + d), part);
      }
      const float sj = rl_warp_sum(part);
      if (lane == j) s = sj;
    }
    if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);      // tanh(-inf) = -1 on lanes without a key: masked below
    if (lane >= n) s = -INFINITY;
    const float new_max = fmaxf(run_max, rl_warp_max(s));   // finite: the chunk's first key is valid
    const float corr = expf(run_max - new_max);              // exp(-inf) = 0 on the warp's first chunk
    const float p = (lane < n) ? expf(s - new_max) : 0.f;
    run_sum = run_sum * corr + rl_warp_sum(p);
    run_max = new_max;
#pragma unroll
    for (int e = 0; e < NE; ++e) acc[e] *= corr;
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int tj = v0 + j < nfirst ? v0 + j : start + (v0 + j - nfirst);
      const T* vrow = v_pool + (size_t)pages[tj / RL_PAGE] * v_page_stride + v_head_off + (size_t)(tj % RL_PAGE) * ldv;
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        const int d = lane + 32 * e;
        if (d < vd) acc[e] = fmaf(pj, rl_ld(vrow + d), acc[e]);
      }
    }
  }
  // ---- the warps' results, merged in the order of the warps (warp 0 always holds keys) ----
  if (lane == 0) { s_max[warp] = run_max; s_sum[warp] = run_sum; }
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    const int d = lane + 32 * e;
    if (d < vd) s_acc[warp][d] = acc[e];
  }
  __syncthreads();
  // sink: one more term in the denominator with score 0 and no value, p_j = e^{s_j} / (1 + sum e^{s_t})
  float M = sink ? 0.f : -INFINITY;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, s_max[w]);
  float wgt[ATT_WARPS], L = sink ? expf(-M) : 0.f;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) {
    wgt[w] = s_max[w] > -INFINITY ? expf(s_max[w] - M) : 0.f;
    L += s_sum[w] * wgt[w];
  }
  const float inv = 1.0f / L;
  T* orow = out + (size_t)m * ldo + (size_t)h * vd;
  for (int d = threadIdx.x; d < vd; d += ATT_WARPS * 32) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) o += s_acc[w][d] * wgt[w];
    o *= inv;
    if (gate)       // output gate, in 32-bit: a number for every output element, or one for the head
      o *= 1.0f / (1.0f + expf(-rl_ld(gate + (size_t)m * ldg + (gate_per_head ? (size_t)h : (size_t)h * vd + d))));
    rl_st(orow + d, o);
  }
}

// q: [M, ldq] with head h at columns [h*hd, (h+1)*hd); out: [M, ldo] with head h at columns
// [h*vd, (h+1)*vd).  k_pool: [num_pages, G, RL_PAGE, hd], v_pool: [num_pages, G, RL_PAGE, vd]
// (value heads may be narrower or wider than key heads: the reference keeps value_dim apart
// from head_dim, src/model.rs:33, 67-69), both in the same dtype as q.
//
// sink != 0: the softmax has one more term in its denominator, of score 0 and without a value.
// gate (may be null): [M, ldg], same dtype; head h's output is multiplied element by element with
// sigmoid(gate[m, h*vd + i]) before it is stored.
//
// softcap > 0: every score s (scale included) becomes softcap * tanh(s / softcap).  keep_first > 0 (with a window):
// a query also sees positions [0, keep_first) that the window has left behind.
//
// chunk > 0 (instead of a window): a query at position p sees positions [p - p % chunk, p].  value_stride: elements
// from one value row to the next (0: value_dim); with value_stride = head_dim and v_pool = k_pool the values are the
// first value_dim elements of the key rows.  gate_per_head != 0: gate is [M, ldg] with one number a head.
extern "C" int rl_attention_simt_shaped(const void* q, int ldq, const void* k_pool, const void* v_pool,
                                        int dtype, const int* page_table, int max_pages,
                                        const int* slot_of_token, const int* positions, void* out, int ldo,
                                        int num_tokens, int num_heads, int num_kv_heads, int head_dim, int value_dim,
                                        float scale, int window, int sink, const void* gate, int ldg, float softcap,
                                        int keep_first, int chunk, int value_stride, int gate_per_head, cudaStream_t stream) {
  RL_REQUIRE(chunk >= 0 && !(chunk > 0 && window > 0), "rl_attention_simt: a chunked mask and a window exclude one another");
  RL_REQUIRE(value_stride == 0 || value_stride >= value_dim, "rl_attention_simt: value rows %d apart are shorter than a value (%d)",
             value_stride, value_dim);
  const int ldv = value_stride ? value_stride : value_dim;
  RL_REQUIRE(softcap >= 0.f && keep_first >= 0, "rl_attention_simt: negative soft cap or number of kept first tokens");
  RL_REQUIRE(gate == nullptr || ldg >= (gate_per_head ? num_heads : num_heads * value_dim), "rl_attention_simt: the gate's row stride is too small");
  RL_REQUIRE(num_tokens >= 0 && num_heads > 0 && num_kv_heads > 0, "rl_attention_simt: bad sizes");
  RL_REQUIRE(num_heads % num_kv_heads == 0, "rl_attention_simt: %d heads are no multiple of %d KV heads",
             num_heads, num_kv_heads);
  RL_REQUIRE(head_dim > 0 && head_dim <= ATT_MAX_HD && head_dim % 2 == 0,
             "rl_attention_simt: head_dim %d must be even and <= %d", head_dim, ATT_MAX_HD);
  RL_REQUIRE(value_dim > 0 && value_dim <= ATT_MAX_HD, "rl_attention_simt: value_dim %d must lie in (0, %d]", value_dim, ATT_MAX_HD);
  RL_REQUIRE(ldq >= num_heads * head_dim && ldo >= num_heads * value_dim, "rl_attention_simt: row strides too small");
  RL_REQUIRE(window >= 0, "rl_attention_simt: negative window");
  if (num_tokens == 0) return RL_OK;
  dim3 grid(num_tokens, num_heads);
  const bool wide = head_dim > 256 || value_dim > 256;
#define RL_ATT_SIMT_LAUNCH(T, NE)                                                                                         \
  attention_simt_kernel<T, NE><<<grid, ATT_WARPS * 32, 0, stream>>>(                                                      \
      (const T*)q, ldq, (const T*)k_pool, (const T*)v_pool, page_table, max_pages, slot_of_token, positions, (T*)out, ldo, \
      num_heads, num_kv_heads, head_dim, value_dim, scale, window, sink, (const T*)gate, ldg, softcap, keep_first, chunk,  \
      ldv, gate_per_head)
  if (dtype == RL_F32) {
    if (wide) RL_ATT_SIMT_LAUNCH(float, 32); else RL_ATT_SIMT_LAUNCH(float, 8);
  } else if (dtype == RL_BF16) {
    if (wide) RL_ATT_SIMT_LAUNCH(__nv_bfloat16, 32); else RL_ATT_SIMT_LAUNCH(__nv_bfloat16, 8);
  } else {
    RL_REQUIRE(false, "rl_attention_simt: unknown dtype %d", dtype);
  }
#undef RL_ATT_SIMT_LAUNCH
  RL_LAUNCH_CHECK("rl_attention_simt");
  return RL_OK;
}

extern "C" int rl_attention_simt_masked(const void* q, int ldq, const void* k_pool, const void* v_pool,
                                        int dtype, const int* page_table, int max_pages,
                                        const int* slot_of_token, const int* positions, void* out, int ldo,
                                        int num_tokens, int num_heads, int num_kv_heads, int head_dim, int value_dim,
                                        float scale, int window, int sink, const void* gate, int ldg, float softcap,
                                        int keep_first, cudaStream_t stream) {
  return rl_attention_simt_shaped(q, ldq, k_pool, v_pool, dtype, page_table, max_pages, slot_of_token, positions, out, ldo,
                                  num_tokens, num_heads, num_kv_heads, head_dim, value_dim, scale, window, sink, gate, ldg, softcap,
                                  keep_first, 0, 0, 0, stream);
}

extern "C" int rl_attention_simt_gated(const void* q, int ldq, const void* k_pool, const void* v_pool,
                                       int dtype, const int* page_table, int max_pages,
                                       const int* slot_of_token, const int* positions, void* out, int ldo,
                                       int num_tokens, int num_heads, int num_kv_heads, int head_dim, int value_dim,
                                       float scale, int window, int sink, const void* gate, int ldg, cudaStream_t stream) {
  return rl_attention_simt_masked(q, ldq, k_pool, v_pool, dtype, page_table, max_pages, slot_of_token, positions, out, ldo,
                                  num_tokens, num_heads, num_kv_heads, head_dim, value_dim, scale, window, sink, gate, ldg, 0.f, 0,
                                  stream);
}

extern "C" int rl_attention_simt(const void* q, int ldq, const void* k_pool, const void* v_pool,
                                 int dtype, const int* page_table, int max_pages,
                                 const int* slot_of_token, const int* positions, void* out, int ldo,
                                 int num_tokens, int num_heads, int num_kv_heads, int head_dim, int value_dim,
                                 float scale, int window, cudaStream_t stream) {
  return rl_attention_simt_gated(q, ldq, k_pool, v_pool, dtype, page_table, max_pages, slot_of_token, positions, out, ldo,
                                 num_tokens, num_heads, num_kv_heads, head_dim, value_dim, scale, window, 0, nullptr, 0, stream);
}
