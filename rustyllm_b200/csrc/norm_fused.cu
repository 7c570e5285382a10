// Norms on a sublayer's output, fused with what stands around them.  All arithmetic is 32-bit.
//
// rl_norm_add     x += m * rms_norm(s0 * y0 + s1 * y1) * w  (a layer that norms what its sublayer returns
//                 before it joins the stream; two terms for two mixers side by side; m: a constant of the
//                 model on every normed sublayer output); optionally the new x is also left as bf16 for the
//                 next sublayer's first product
// rl_gated_norm   the output of a recurrent mixer: y * act(gate), an RMS norm in `groups` equal parts, times w
//                 ("gate first"), or the norm of y over the row times w, then times act(gate) ("gate last")
// rl_gelu_gate    out = gelu_tanh(t) * table[token, col0 : col0 + n]    (a learned vector per token and layer
//                 gating a small projection of the stream)
#include <math.h>

#include "common.cuh"

#define NF_THREADS 256

__device__ __forceinline__ float nf_block_sum(float v, float* s_part) {
  v = rl_warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                       // s_part may still be read from an earlier call
  if (lane == 0) s_part[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < NF_THREADS / 32; ++w) t += s_part[w];
  return t;
}

__global__ void __launch_bounds__(NF_THREADS)
norm_add_kernel(float* __restrict__ x, const float* __restrict__ y0, float s0, const float* __restrict__ y1, float s1,
                const float* __restrict__ w, float eps, float out_scale, int d, __nv_bfloat16* __restrict__ x_bf16) {
  __shared__ float s_part[NF_THREADS / 32];
  rl_pdl_trigger();
  rl_pdl_wait();
  const size_t row = (size_t)blockIdx.x * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += NF_THREADS) {
    const float v = y1 ? fmaf(s1, y1[row + i], s0 * y0[row + i]) : s0 * y0[row + i];
    ss = fmaf(v, v, ss);
  }
  const float r = 1.0f / sqrtf(nf_block_sum(ss, s_part) / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += NF_THREADS) {
    const float v = y1 ? fmaf(s1, y1[row + i], s0 * y0[row + i]) : s0 * y0[row + i];
    const float nx = x[row + i] + out_scale * (v * r * w[i]);
    x[row + i] = nx;
    if (x_bf16) x_bf16[row + i] = __float2bfloat16_rn(nx);
  }
}

__device__ __forceinline__ float nf_act(float z, int act) {
  const float s = 1.0f / (1.0f + expf(-z));
  return act == 0 ? z * s : s;           // 0: silu, 1: sigmoid
}

template <typename T>
__global__ void __launch_bounds__(NF_THREADS)
gated_norm_kernel(const float* __restrict__ y, int ldy, const T* __restrict__ gate, int ldg, int act, int gate_first,
                  const float* __restrict__ w, float eps, int n, T* __restrict__ out, int ldo) {
  __shared__ float s_part[NF_THREADS / 32];
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x, c0 = blockIdx.y * n;     // group blockIdx.y of the row: columns [c0, c0 + n)
  const float* yr = y + (size_t)m * ldy + c0;
  const T* gr = gate + (size_t)m * ldg + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += NF_THREADS) {
    const float v = gate_first ? yr[i] * nf_act(rl_ld(gr + i), act) : yr[i];
    ss = fmaf(v, v, ss);
  }
  const float r = 1.0f / sqrtf(nf_block_sum(ss, s_part) / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += NF_THREADS) {
    const float g = nf_act(rl_ld(gr + i), act);
    const float v = gate_first ? yr[i] * g * r * w[c0 + i] : yr[i] * r * w[c0 + i] * g;
    rl_st(out + (size_t)m * ldo + c0 + i, v);
  }
}

// The same for groups of up to 1,024 values in steps of many tokens: a warp a (token, group), eight a block, no
// barrier; the second pass finds the group in L1.
template <typename T>
__global__ void __launch_bounds__(NF_THREADS)
gated_norm_warp_kernel(const float* __restrict__ y, int ldy, const T* __restrict__ gate, int ldg, int act, int gate_first,
                       const float* __restrict__ w, float eps, int n, int groups, long long rows, T* __restrict__ out, int ldo) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const long long row = (long long)blockIdx.x * (NF_THREADS / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long m = row / groups;
  const int c0 = (int)(row % groups) * n;
  const float* yr = y + (size_t)m * ldy + c0;
  const T* gr = gate + (size_t)m * ldg + c0;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) {
    const float v = gate_first ? yr[i] * nf_act(rl_ld(gr + i), act) : yr[i];
    ss = fmaf(v, v, ss);
  }
  const float r = 1.0f / sqrtf(rl_warp_sum(ss) / (float)n + eps);
  for (int i = lane; i < n; i += 32) {
    const float g = nf_act(rl_ld(gr + i), act);
    const float v = gate_first ? yr[i] * g * r * w[c0 + i] : yr[i] * r * w[c0 + i] * g;
    rl_st(out + (size_t)m * ldo + c0 + i, v);
  }
}

template <typename T>
__global__ void __launch_bounds__(NF_THREADS)
gelu_gate_kernel(const T* __restrict__ t, int ldt, const int* __restrict__ tokens, const T* __restrict__ table, int ld_table,
                 int col0, int n, T* __restrict__ out, int ldo, long long total) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const long long idx = (long long)blockIdx.x * NF_THREADS + threadIdx.x;
  if (idx >= total) return;
  const int m = (int)(idx / n), i = (int)(idx % n);
  const float z = rl_ld(t + (size_t)m * ldt + i);
  const float g = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  rl_st(out + (size_t)m * ldo + i, g * rl_ld(table + (size_t)tokens[m] * ld_table + col0 + i));
}

extern "C" int rl_norm_add(float* x, const float* y0, float s0, const float* y1, float s1, const float* weight, float eps,
                           float out_scale, int num_tokens, int width, void* x_bf16, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && width > 0 && y0 != nullptr && weight != nullptr, "rl_norm_add: bad arguments");
  if (num_tokens == 0) return RL_OK;
  rl_launch_pdl(norm_add_kernel, num_tokens, NF_THREADS, 0, stream, x, y0, s0, y1, s1, weight, eps, out_scale, width, (__nv_bfloat16*)x_bf16);
  RL_LAUNCH_CHECK("rl_norm_add");
  return RL_OK;
}

// y float [M, ldy], gate [M, ldg] and out [M, ldo] in `dtype`, weight float [groups * n]; act 0 silu, 1 sigmoid.
extern "C" int rl_gated_norm(const float* y, int ldy, const void* gate, int ldg, int dtype, int act, int gate_first,
                             const float* weight, float eps, int num_tokens, int groups, int n, void* out, int ldo,
                             cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && groups > 0 && groups <= 65535 && n > 0, "rl_gated_norm: bad sizes");
  RL_REQUIRE(ldy >= groups * n && ldg >= groups * n && ldo >= groups * n, "rl_gated_norm: row strides too small");
  RL_REQUIRE((act == 0 || act == 1) && (gate_first == 0 || gate_first == 1), "rl_gated_norm: unknown option");
  if (num_tokens == 0) return RL_OK;
  const dim3 grid(num_tokens, groups);
  const long long rows = (long long)num_tokens * groups;
  if (n <= 1024 && rows >= 4096) {          // many small groups: a warp each
    const unsigned blocks = (unsigned)((rows + NF_THREADS / 32 - 1) / (NF_THREADS / 32));
    if (dtype == RL_F32)
      rl_launch_pdl(gated_norm_warp_kernel<float>, blocks, NF_THREADS, 0, stream, y, ldy, (const float*)gate, ldg, act, gate_first, weight,
                    eps, n, groups, rows, (float*)out, ldo);
    else if (dtype == RL_BF16)
      rl_launch_pdl(gated_norm_warp_kernel<__nv_bfloat16>, blocks, NF_THREADS, 0, stream, y, ldy, (const __nv_bfloat16*)gate, ldg, act,
                    gate_first, weight, eps, n, groups, rows, (__nv_bfloat16*)out, ldo);
    else
      RL_REQUIRE(false, "rl_gated_norm: unknown dtype %d", dtype);
    RL_LAUNCH_CHECK("rl_gated_norm");
    return RL_OK;
  }
  if (dtype == RL_F32)
    rl_launch_pdl(gated_norm_kernel<float>, grid, NF_THREADS, 0, stream, y, ldy, (const float*)gate, ldg, act, gate_first, weight, eps,
                  n, (float*)out, ldo);
  else if (dtype == RL_BF16)
    rl_launch_pdl(gated_norm_kernel<__nv_bfloat16>, grid, NF_THREADS, 0, stream, y, ldy, (const __nv_bfloat16*)gate, ldg, act,
                  gate_first, weight, eps, n, (__nv_bfloat16*)out, ldo);
  else
    RL_REQUIRE(false, "rl_gated_norm: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_gated_norm");
  return RL_OK;
}

extern "C" int rl_gelu_gate(const void* t, int ldt, const int* tokens, const void* table, int ld_table, int col0, int n,
                            int dtype, void* out, int ldo, int num_tokens, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && n > 0 && col0 >= 0 && col0 + n <= ld_table && ldt >= n && ldo >= n, "rl_gelu_gate: bad sizes");
  if (num_tokens == 0) return RL_OK;
  const long long total = (long long)num_tokens * n;
  const unsigned blocks = (unsigned)((total + NF_THREADS - 1) / NF_THREADS);
  if (dtype == RL_F32)
    rl_launch_pdl(gelu_gate_kernel<float>, blocks, NF_THREADS, 0, stream, (const float*)t, ldt, tokens, (const float*)table, ld_table,
                  col0, n, (float*)out, ldo, total);
  else if (dtype == RL_BF16)
    rl_launch_pdl(gelu_gate_kernel<__nv_bfloat16>, blocks, NF_THREADS, 0, stream, (const __nv_bfloat16*)t, ldt, tokens,
                  (const __nv_bfloat16*)table, ld_table, col0, n, (__nv_bfloat16*)out, ldo, total);
  else
    RL_REQUIRE(false, "rl_gelu_gate: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_gelu_gate");
  return RL_OK;
}
