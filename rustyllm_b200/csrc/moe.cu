// Mixture of experts on the CUDA cores: router, and the chosen experts' gated feed-forward
// per (token, choice).  Float or bf16 storage, 32-bit accumulation.
//
//   router : z = Wr h + b (32-bit), the `top` largest logits chosen (ties: the lower index),
//            weights = softmax over the chosen logits only
//   expert : y_e = Wdown_e (silu(Wgate_e h) * (Wup_e h))
//   output : residual += sum_c weight_c * y_{e_c}     (choices in the order of falling logits)
//
// Every token is computed by itself, its sums in an order that its own sizes fix, so a token's
// result does not depend on the batch.  Weights: gate_up [E, 2, F, d] (an expert's gate rows,
// then its up rows), down [E, d, F].
#include <math.h>

#include "common.cuh"

#define MOE_THREADS 256
#define MOE_MAX_TOP 32

// 8 consecutive elements of a row times 8 of the input, for rows whose length is a multiple of 8 (bf16: one
// 16-byte load a lane, so a warp's load instruction covers 512 consecutive bytes of the weight row)
__device__ __forceinline__ float moe_dot8(const __nv_bfloat16* w, const float* xs) {
  const uint4 v = *reinterpret_cast<const uint4*>(w);
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
  float acc = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(p[k]);
    acc = fmaf(xs[2 * k], f.x, acc);
    acc = fmaf(xs[2 * k + 1], f.y, acc);
  }
  return acc;
}
__device__ __forceinline__ float moe_dot8(const float* w, const float* xs) {
  float acc = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) acc = fmaf(xs[k], w[k], acc);
  return acc;
}

// ------------------------------------------------------------------ router
// The logits of block m's token into s_logit[E] (s_x [d] is scratch): warp w takes experts w, w + 8, ...
template <typename T>
__device__ __forceinline__ void moe_logits(const T* __restrict__ x, int ldx, const T* __restrict__ wr, const float* __restrict__ bias,
                                           int d, int E, float* s_logit, float* s_x) {
  const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* xr = x + (size_t)m * ldx;
  for (int i = threadIdx.x; i < d; i += MOE_THREADS) s_x[i] = rl_ld(xr + i);
  __syncthreads();
  const bool vec = d % 8 == 0 && ((uintptr_t)wr & 15) == 0;
  for (int e = warp; e < E; e += MOE_THREADS / 32) {
    const T* w = wr + (size_t)e * d;
    float part = 0.f;
    if (vec) {
      for (int i = 8 * lane; i < d; i += 256) part += moe_dot8(w + i, s_x + i);
    } else {
      for (int i = lane; i < d; i += 32) part = fmaf(s_x[i], rl_ld(w + i), part);
    }
    part = rl_warp_sum(part);
    if (lane == 0) s_logit[e] = part + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
}

// One block a token; then warp 0 selects.
template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_route_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ wr, const float* __restrict__ bias,
                 int d, int E, int top, int* __restrict__ ids, float* __restrict__ weights) {
  extern __shared__ float s_logit[];     // [E], then the token's input [d]
  float* s_x = s_logit + ((E + 3) & ~3);
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  moe_logits(x, ldx, wr, bias, d, E, s_logit, s_x);
  if (warp != 0) return;
  float chosen = 0.f, first = 0.f, denom = 0.f;      // lane c keeps choice c's logit
  int chosen_id = 0;
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float z = s_logit[e];
      if (z > best) { best = z; at = e; }            // ascending e: the lower index wins a tie
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = 0;                    // all logits NaN or -inf: still a valid index
    if (c == 0) first = best;
    if (lane == c) { chosen = best; chosen_id = at; }
    __syncwarp();
    if (lane == 0) s_logit[at] = -INFINITY;
    __syncwarp();
  }
  const float e_c = lane < top ? expf(chosen - first) : 0.f;
  denom = rl_warp_sum(e_c);
  if (lane < top) {
    ids[(size_t)m * top + lane] = chosen_id;
    weights[(size_t)m * top + lane] = e_c / denom;
  }
}

// The selection alone, from logits a matrix product has made (many tokens: the router is then one product
// [M, d] x [d, E] with the bias in its epilogue, and this kernel - a warp a token - picks and weighs).
__global__ void __launch_bounds__(MOE_THREADS)
moe_select_kernel(const float* __restrict__ logits, int M, int E, int top, int* __restrict__ ids, float* __restrict__ weights) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * (MOE_THREADS / 32) + warp;
  if (m >= M) return;
  const float* z = logits + (size_t)m * E;
  float chosen = 0.f, first = 0.f;
  int chosen_id = 0;
  unsigned taken_lo = 0;                 // experts this lane has given away already, for E <= 1024: bit j = expert lane + 32 j
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane, j = 0; e < E; e += 32, ++j) {
      if (taken_lo >> j & 1u) continue;
      const float v = z[e];
      if (v > best) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = 0;
    if (c == 0) first = best;
    if (lane == c) { chosen = best; chosen_id = at; }
    if ((at & 31) == lane) taken_lo |= 1u << (at >> 5);
  }
  const float e_c = lane < top ? expf(chosen - first) : 0.f;
  const float denom = rl_warp_sum(e_c);
  if (lane < top) {
    ids[(size_t)m * top + lane] = chosen_id;
    weights[(size_t)m * top + lane] = e_c / denom;
  }
}

extern "C" int rl_moe_select(const float* logits, int num_tokens, int num_experts, int top, int* ids, float* weights,
                             cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && num_experts > 0 && num_experts <= 1024, "rl_moe_select: bad sizes M=%d E=%d (at most 1,024 experts)", num_tokens, num_experts);
  RL_REQUIRE(top > 0 && top <= num_experts && top <= MOE_MAX_TOP, "rl_moe_select: top %d must lie in [1, min(%d, %d)]", top, num_experts, MOE_MAX_TOP);
  if (num_tokens == 0) return RL_OK;
  const int per = MOE_THREADS / 32;
  rl_launch_pdl(moe_select_kernel, (num_tokens + per - 1) / per, MOE_THREADS, 0, stream, logits, num_tokens, num_experts, top, ids, weights);
  RL_LAUNCH_CHECK("rl_moe_select");
  return RL_OK;
}

extern "C" int rl_moe_route(const void* x, int ldx, const void* router, const float* bias, int dtype, int num_tokens,
                            int hidden, int num_experts, int top, int* ids, float* weights, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && hidden > 0 && num_experts > 0, "rl_moe_route: bad sizes M=%d d=%d E=%d", num_tokens, hidden, num_experts);
  RL_REQUIRE(top > 0 && top <= num_experts && top <= MOE_MAX_TOP, "rl_moe_route: top %d must lie in [1, min(%d, %d)]", top, num_experts, MOE_MAX_TOP);
  RL_REQUIRE(num_experts <= 8192, "rl_moe_route: at most 8192 experts");
  if (num_tokens == 0) return RL_OK;
  RL_REQUIRE(hidden + num_experts <= 11000, "rl_moe_route: hidden size plus experts above 11,000");
  const size_t smem = (size_t)(((num_experts + 3) & ~3) + hidden) * sizeof(float);
  if (dtype == RL_F32)
    rl_launch_pdl(moe_route_kernel<float>, num_tokens, MOE_THREADS, smem, stream, (const float*)x, ldx, (const float*)router, bias,
                  hidden, num_experts, top, ids, weights);
  else if (dtype == RL_BF16)
    rl_launch_pdl(moe_route_kernel<__nv_bfloat16>, num_tokens, MOE_THREADS, smem, stream, (const __nv_bfloat16*)x, ldx,
                  (const __nv_bfloat16*)router, bias, hidden, num_experts, top, ids, weights);
  else
    RL_REQUIRE(false, "rl_moe_route: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_moe_route");
  return RL_OK;
}

// ------------------------------------------------------------------ router with sigmoid scores
// scores s = sigmoid(z); an expert is chosen by s + correction[e] ("choice score"), weighed by s itself (not
// renormalised).  Experts form `groups` equal groups of neighbours; a group's score is the sum of its two
// largest choice scores (of its one, in groups of one); only experts of the `keep` best groups can be chosen.
// Ties go to the lower index.  One warp: s_score [E] holds the logits on entry, s_choice [E] and s_group
// [2 * groups] are scratch.
// Variants, each an argument: `softmax_all` - the scores are the softmax of the logits over all experts instead of
// their sigmoids; `group_top` - a group's score is the sum of its `group_top` largest choice scores (2 above; 1: its
// largest); `renorm` - the weights are the chosen scores divided by their sum (+ 1e-20).
__device__ __forceinline__ void moe_pick_sigmoid(float* s_score, float* s_choice, float* s_group, const float* __restrict__ correction,
                                                 int E, int top, int groups, int keep, int lane, int* __restrict__ ids,
                                                 float* __restrict__ weights, int softmax_all = 0, int group_top = 2, int renorm = 0) {
  if (softmax_all) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s_score[e]);
    mx = rl_warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float p = expf(s_score[e] - mx);
      s_score[e] = p;
      sum += p;
    }
    sum = rl_warp_sum(sum);
    for (int e = lane; e < E; e += 32) {
      const float sc = s_score[e] / sum;
      s_score[e] = sc;
      s_choice[e] = sc + (correction ? correction[e] : 0.f);
    }
  } else {
    for (int e = lane; e < E; e += 32) {
      const float sc = 1.0f / (1.0f + expf(-s_score[e]));
      s_score[e] = sc;
      s_choice[e] = sc + (correction ? correction[e] : 0.f);
    }
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int size = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float t1 = -INFINITY, t2 = -INFINITY;
      for (int e = g * size; e < (g + 1) * size; ++e) {
        const float v = s_choice[e];
        if (v > t1) { t2 = t1; t1 = v; }
        else if (v > t2) t2 = v;
      }
      s_group[g] = (size > 1 && group_top > 1) ? t1 + t2 : t1;
      s_group[groups + g] = 0.f;           // 1: the group is kept
    }
    __syncwarp();
    for (int c = 0; c < keep; ++c) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = s_group[g];
        if (s_group[groups + g] == 0.f && (v > best || at == 0x7fffffff)) { best = v; at = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
      }
      __syncwarp();
      if (lane == 0 && at != 0x7fffffff) s_group[groups + at] = 1.f;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (s_group[groups + e / size] == 0.f) s_choice[e] = -INFINITY;
    __syncwarp();
  }
  float chosen_w = 0.f;
  int chosen_id = 0;
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float z = s_choice[e];
      if (z > best) { best = z; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = 0;
    if (lane == c) { chosen_id = at; chosen_w = s_score[at]; }
    __syncwarp();
    if (lane == 0) s_choice[at] = -INFINITY;
    __syncwarp();
  }
  if (renorm) {
    const float total = rl_warp_sum(lane < top ? chosen_w : 0.f);
    chosen_w = chosen_w / (total + 1e-20f);
  }
  if (lane < top) {
    ids[lane] = chosen_id;
    weights[lane] = chosen_w;
  }
}

template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_route_sigmoid_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ wr, const float* __restrict__ correction,
                         int d, int E, int top, int groups, int keep, int* __restrict__ ids, float* __restrict__ weights, int softmax_all,
                         int group_top, int renorm) {
  extern __shared__ float s_logit[];     // scores [E], choice scores [E], groups [2 * groups], then the token's input [d]
  const int Ep = (E + 3) & ~3;
  float* s_x = s_logit + 4 * Ep;
  rl_pdl_trigger();
  rl_pdl_wait();
  moe_logits(x, ldx, wr, (const float*)nullptr, d, E, s_logit, s_x);
  if (threadIdx.x >= 32) return;
  const size_t m = blockIdx.x;
  moe_pick_sigmoid(s_logit, s_logit + Ep, s_logit + 2 * Ep, correction, E, top, groups, keep, threadIdx.x, ids + m * top, weights + m * top,
                   softmax_all, group_top, renorm);
}

// from logits a matrix product has made: one warp a token
__global__ void __launch_bounds__(32)
moe_select_sigmoid_kernel(const float* __restrict__ logits, int E, int top, const float* __restrict__ correction, int groups, int keep,
                          int* __restrict__ ids, float* __restrict__ weights, int softmax_all, int group_top, int renorm) {
  extern __shared__ float s_logit[];
  const int Ep = (E + 3) & ~3;
  rl_pdl_trigger();
  rl_pdl_wait();
  const size_t m = blockIdx.x;
  for (int e = threadIdx.x; e < E; e += 32) s_logit[e] = logits[m * E + e];
  __syncwarp();
  moe_pick_sigmoid(s_logit, s_logit + Ep, s_logit + 2 * Ep, correction, E, top, groups, keep, threadIdx.x, ids + m * top, weights + m * top,
                   softmax_all, group_top, renorm);
}

static int moe_sigmoid_args(const char* who, int num_experts, int top, int groups, int keep) {
  RL_REQUIRE(num_experts > 0 && num_experts <= 1024, "%s: %d experts (at most 1,024)", who, num_experts);
  RL_REQUIRE(top > 0 && top <= num_experts && top <= MOE_MAX_TOP, "%s: top %d must lie in [1, min(%d, %d)]", who, top, num_experts, MOE_MAX_TOP);
  RL_REQUIRE(groups >= 1 && num_experts % groups == 0 && keep >= 1 && keep <= groups, "%s: %d groups (keep %d) do not divide %d experts", who,
             groups, keep, num_experts);
  RL_REQUIRE(keep * (num_experts / groups) >= top, "%s: the %d kept groups hold fewer than top = %d experts", who, keep, top);
  return RL_OK;
}

// rl_moe_select_scored / rl_moe_route_scored: the routers above with the variants as arguments (softmax_all,
// group_top 1 or 2, renorm; see moe_pick_sigmoid); the *_sigmoid entry points are (0, 2, 0).
extern "C" int rl_moe_select_scored(const float* logits, int num_tokens, int num_experts, int top, const float* correction, int groups,
                                    int keep, int softmax_all, int group_top, int renorm, int* ids, float* weights, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && (group_top == 1 || group_top == 2), "rl_moe_select_scored: bad sizes or group_top %d", group_top);
  if (const int rc = moe_sigmoid_args("rl_moe_select_sigmoid", num_experts, top, groups, keep)) return rc;
  if (num_tokens == 0) return RL_OK;
  const size_t smem = (size_t)4 * ((num_experts + 3) & ~3) * sizeof(float);
  rl_launch_pdl(moe_select_sigmoid_kernel, num_tokens, 32, smem, stream, logits, num_experts, top, correction, groups, keep, ids, weights,
                softmax_all, group_top, renorm);
  RL_LAUNCH_CHECK("rl_moe_select_sigmoid");
  return RL_OK;
}

extern "C" int rl_moe_select_sigmoid(const float* logits, int num_tokens, int num_experts, int top, const float* correction, int groups,
                                     int keep, int* ids, float* weights, cudaStream_t stream) {
  return rl_moe_select_scored(logits, num_tokens, num_experts, top, correction, groups, keep, 0, 2, 0, ids, weights, stream);
}

extern "C" int rl_moe_route_scored(const void* x, int ldx, const void* router, const float* correction, int dtype, int num_tokens,
                                   int hidden, int num_experts, int top, int groups, int keep, int softmax_all, int group_top, int renorm,
                                   int* ids, float* weights, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && hidden > 0 && (group_top == 1 || group_top == 2), "rl_moe_route_sigmoid: bad sizes M=%d d=%d", num_tokens, hidden);
  if (const int rc = moe_sigmoid_args("rl_moe_route_sigmoid", num_experts, top, groups, keep)) return rc;
  if (num_tokens == 0) return RL_OK;
  RL_REQUIRE(hidden + 4 * num_experts <= 11000, "rl_moe_route_sigmoid: hidden size plus four times the experts above 11,000");
  const size_t smem = (size_t)(4 * ((num_experts + 3) & ~3) + hidden) * sizeof(float);
  if (dtype == RL_F32)
    rl_launch_pdl(moe_route_sigmoid_kernel<float>, num_tokens, MOE_THREADS, smem, stream, (const float*)x, ldx, (const float*)router,
                  correction, hidden, num_experts, top, groups, keep, ids, weights, softmax_all, group_top, renorm);
  else if (dtype == RL_BF16)
    rl_launch_pdl(moe_route_sigmoid_kernel<__nv_bfloat16>, num_tokens, MOE_THREADS, smem, stream, (const __nv_bfloat16*)x, ldx,
                  (const __nv_bfloat16*)router, correction, hidden, num_experts, top, groups, keep, ids, weights, softmax_all, group_top, renorm);
  else
    RL_REQUIRE(false, "rl_moe_route_sigmoid: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_moe_route_sigmoid");
  return RL_OK;
}

extern "C" int rl_moe_route_sigmoid(const void* x, int ldx, const void* router, const float* correction, int dtype, int num_tokens,
                                    int hidden, int num_experts, int top, int groups, int keep, int* ids, float* weights,
                                    cudaStream_t stream) {
  return rl_moe_route_scored(x, ldx, router, correction, dtype, num_tokens, hidden, num_experts, top, groups, keep, 0, 2, 0, ids, weights,
                             stream);
}

// ------------------------------------------------------------------ gate and up of the chosen experts
// grid (row blocks of F, M * top); the token's input in shared memory; a warp a row of the expert.
// interleaved: an expert's rows are (gate_0, up_0, gate_1, up_1, ...) instead of all gate rows, then all up rows
template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_gate_up_kernel(const T* __restrict__ x, int ldx, const T* __restrict__ wgu, const int* __restrict__ ids,
                   int d, int F, int top, T* __restrict__ h, int interleaved) {
  extern __shared__ float s_x[];          // [d]
  rl_pdl_trigger();
  rl_pdl_wait();
  const int pair = blockIdx.y, m = pair / top;
  const int e = ids[pair];
  const T* xr = x + (size_t)m * ldx;
  for (int i = threadIdx.x; i < d; i += MOE_THREADS) s_x[i] = rl_ld(xr + i);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (MOE_THREADS / 32) + warp;
  if (r >= F) return;
  const T* wg = wgu + ((size_t)e * 2 * F + (interleaved ? 2 * r : r)) * d;
  const T* wu = wg + (size_t)(interleaved ? 1 : F) * d;
  float g = 0.f, u = 0.f;
  if (d % 8 == 0 && ((uintptr_t)wgu & 15) == 0) {
    for (int i = 8 * lane; i < d; i += 256) {
      g += moe_dot8(wg + i, s_x + i);
      u += moe_dot8(wu + i, s_x + i);
    }
  } else {
    for (int i = lane; i < d; i += 32) {
      const float xv = s_x[i];
      g = fmaf(xv, rl_ld(wg + i), g);
      u = fmaf(xv, rl_ld(wu + i), u);
    }
  }
  g = rl_warp_sum(g);
  u = rl_warp_sum(u);
  if (lane == 0) rl_st(h + (size_t)pair * F + r, g / (1.0f + expf(-g)) * u);
}

// ------------------------------------------------------------------ down of the chosen experts, weighted, into the residual
// grid (row blocks of d, M); a warp an output element; choices summed in their order.
template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_down_kernel(const T* __restrict__ h, const T* __restrict__ wd, const int* __restrict__ ids,
                const float* __restrict__ weights, int d, int F, int top, float* __restrict__ residual) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (MOE_THREADS / 32) + warp;
  if (r >= d) return;
  float y = 0.f;
  for (int c = 0; c < top; ++c) {
    const int e = ids[(size_t)m * top + c];
    const T* w = wd + ((size_t)e * d + r) * F;
    const T* hr = h + ((size_t)m * top + c) * F;
    float part = 0.f;
    if (F % 8 == 0 && ((uintptr_t)wd & 15) == 0 && ((uintptr_t)h & 15) == 0) {
      for (int i = 8 * lane; i < F; i += 256) {
        float hs[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) hs[k] = rl_ld(hr + i + k);
        part += moe_dot8(w + i, hs);
      }
    } else {
      for (int i = lane; i < F; i += 32) part = fmaf(rl_ld(hr + i), rl_ld(w + i), part);
    }
    part = rl_warp_sum(part);
    y = fmaf(weights[(size_t)m * top + c], part, y);
  }
  if (lane == 0) residual[(size_t)m * d + r] += y;
}

// x [M, ldx]; gate_up [E, 2, F, d], or with `interleaved` [E, F, 2, d] (gate_r, up_r in turn); down [E, d, F]; ids, weights [M, top] (from rl_moe_route);
// h [M * top, F] scratch in the same dtype; residual [M, d] float, added into.
extern "C" int rl_moe_experts(const void* x, int ldx, const void* gate_up, const void* down, int dtype, const int* ids,
                              const float* weights, int num_tokens, int hidden, int expert_ff, int num_experts, int top,
                              int interleaved, void* h, float* residual, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && hidden > 0 && expert_ff > 0 && num_experts > 0 && top > 0,
             "rl_moe_experts: bad sizes M=%d d=%d F=%d E=%d top=%d", num_tokens, hidden, expert_ff, num_experts, top);
  RL_REQUIRE((long long)num_tokens * top <= 65535LL * 1024, "rl_moe_experts: too many (token, choice) pairs for one launch");
  RL_REQUIRE(hidden <= 48 * 1024 / 4, "rl_moe_experts: hidden size %d above %d", hidden, 48 * 1024 / 4);
  if (num_tokens == 0) return RL_OK;
  const int per = MOE_THREADS / 32;
  // grid.y is limited to 65535: pairs beyond that run as further launches
  for (long long p0 = 0; p0 < (long long)num_tokens * top; p0 += 65535LL / top * top) {
    const long long n = ((long long)num_tokens * top - p0) < 65535LL / top * top ? ((long long)num_tokens * top - p0) : 65535LL / top * top;
    const int m0 = (int)(p0 / top), mt = (int)(n / top);
    dim3 g1((expert_ff + per - 1) / per, (unsigned)n), g2((hidden + per - 1) / per, (unsigned)mt);
    const size_t smem = (size_t)hidden * sizeof(float);
    if (dtype == RL_F32) {
      rl_launch_pdl(moe_gate_up_kernel<float>, g1, MOE_THREADS, smem, stream, (const float*)x + (size_t)m0 * ldx, ldx, (const float*)gate_up,
                    ids + p0, hidden, expert_ff, top, (float*)h + (size_t)p0 * expert_ff, interleaved);
      rl_launch_pdl(moe_down_kernel<float>, g2, MOE_THREADS, 0, stream, (const float*)h + (size_t)p0 * expert_ff, (const float*)down,
                    ids + p0, weights + p0, hidden, expert_ff, top, residual + (size_t)m0 * hidden);
    } else if (dtype == RL_BF16) {
      rl_launch_pdl(moe_gate_up_kernel<__nv_bfloat16>, g1, MOE_THREADS, smem, stream, (const __nv_bfloat16*)x + (size_t)m0 * ldx, ldx,
                    (const __nv_bfloat16*)gate_up, ids + p0, hidden, expert_ff, top, (__nv_bfloat16*)h + (size_t)p0 * expert_ff, interleaved);
      rl_launch_pdl(moe_down_kernel<__nv_bfloat16>, g2, MOE_THREADS, 0, stream, (const __nv_bfloat16*)h + (size_t)p0 * expert_ff,
                    (const __nv_bfloat16*)down, ids + p0, weights + p0, hidden, expert_ff, top, residual + (size_t)m0 * hidden);
    } else {
      RL_REQUIRE(false, "rl_moe_experts: unknown dtype %d", dtype);
    }
    RL_LAUNCH_CHECK("rl_moe_experts");
  }
  return RL_OK;
}

// ------------------------------------------------------------------ the tensor-core way: rows ordered by expert
// For many tokens the chosen experts run as grouped matrix products (rl_gemm_tc_grouped): the (token, choice)
// pairs are put in the order of their experts, every expert's rows padded to whole token tiles of `bt` rows, so
// that a tile meets one expert's matrix.
//   plan   : row[p] = the pair's row; tile_group[t] = the expert of tile t, or -1 for a tile that holds no pair
//   gather : xs[row[p], :] = x[p / top, :]
//   (grouped products: gate and up with the activation in the epilogue, then down, into y [rows, d] float)
//   combine: residual[m, :] += sum_c weights[m, c] * y[row[m * top + c], :]   (choices in their order)
// Which row a pair gets within its expert depends on timing; no result does: a row of a product depends on that
// row alone, and the combination walks a token's choices in their order.

// One block.  counts in shared memory; pairs are ranked within their expert by an atomic counter.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int pairs, int E, int bt, int max_tiles, int* __restrict__ row,
                int* __restrict__ tile_group) {
  extern __shared__ int s_plan[];          // [E] counts, then [E] first rows
  int* s_count = s_plan;
  int* s_first = s_plan + E;
  rl_pdl_trigger();
  rl_pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_count[e] = 0;
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) tile_group[t] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) row[p] = atomicAdd(&s_count[ids[p]], 1);   // rank within the expert
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      s_first[e] = at;
      at += (s_count[e] + bt - 1) / bt * bt;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int t0 = s_first[e] / bt, nt = (s_count[e] + bt - 1) / bt;
    for (int t = 0; t < nt; ++t)
      if (t0 + t < max_tiles) tile_group[t0 + t] = e;
  }
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) row[p] += s_first[ids[p]];
}

__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ row, int top, int d,
                                  __nv_bfloat16* __restrict__ xs) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int p = blockIdx.x;
  const __nv_bfloat16* src = x + (size_t)(p / top) * ldx;
  __nv_bfloat16* dst = xs + (size_t)row[p] * d;
  for (int i = threadIdx.x; i < d / 8; i += blockDim.x)          // d is a multiple of 8, rows 16-byte aligned
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ row, const float* __restrict__ weights,
                                   int top, int d, float* __restrict__ residual) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  // d is a multiple of 4 and all rows are 16-byte aligned: four columns a thread, the choices' rows read side by side
  for (int i = 4 * threadIdx.x; i < d; i += 4 * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = 0; c < top; ++c) {
      const float w = weights[(size_t)m * top + c];
      const float4 v = __ldcs(reinterpret_cast<const float4*>(y + (size_t)row[(size_t)m * top + c] * d + i));
      acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
    }
    float4* r = reinterpret_cast<float4*>(residual + (size_t)m * d + i);
    float4 o = *r;
    o.x += acc.x; o.y += acc.y; o.z += acc.z; o.w += acc.w;
    *r = o;
  }
}

// Rows the ordered layout can need for `pairs` pairs over E experts at a token tile of bt: every expert's rows
// rounded up to whole tiles.
extern "C" long long rl_moe_sorted_rows(long long pairs, int num_experts, int bt) {
  const long long used = pairs < num_experts ? pairs : num_experts;       // experts that can hold a pair
  return (pairs + used * (bt - 1)) / bt * bt;
}

extern "C" int rl_moe_plan(const int* ids, int pairs, int num_experts, int bt, int max_tiles, int* row, int* tile_group,
                           cudaStream_t stream) {
  RL_REQUIRE(pairs > 0 && num_experts > 0 && num_experts <= 4096 && bt > 0 && max_tiles > 0, "rl_moe_plan: bad sizes");
  rl_launch_pdl(moe_plan_kernel, 1, 1024, (size_t)2 * num_experts * sizeof(int), stream, ids, pairs, num_experts, bt, max_tiles, row, tile_group);
  RL_LAUNCH_CHECK("rl_moe_plan");
  return RL_OK;
}

extern "C" int rl_moe_gather(const void* x, int ldx, const int* row, int pairs, int top, int hidden, void* xs, cudaStream_t stream) {
  RL_REQUIRE(pairs > 0 && top > 0 && hidden % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)xs & 15) == 0,
             "rl_moe_gather: rows must be 16-byte aligned and a multiple of 8 long");
  rl_launch_pdl(moe_gather_kernel, pairs, 128, 0, stream, (const __nv_bfloat16*)x, ldx, row, top, hidden, (__nv_bfloat16*)xs);
  RL_LAUNCH_CHECK("rl_moe_gather");
  return RL_OK;
}

extern "C" int rl_moe_combine(const float* y, const int* row, const float* weights, int num_tokens, int top, int hidden,
                              float* residual, cudaStream_t stream) {
  RL_REQUIRE(num_tokens > 0 && top > 0 && hidden > 0 && hidden % 4 == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)residual & 15) == 0,
             "rl_moe_combine: bad sizes (the hidden size must be a multiple of 4, the rows 16-byte aligned)");
  rl_launch_pdl(moe_combine_kernel, num_tokens, hidden >= 2048 ? 256 : 128, 0, stream, y, row, weights, top, hidden, residual);
  RL_LAUNCH_CHECK("rl_moe_combine");
  return RL_OK;
}
