// Small kernels around a mixer that reads, beside a token's input h_t, the previous token's h_{t-1}:
//
// rl_token_shift_mix  n blends of the two, m_s = h_t + (h_{t-1} - h_t) * mu_s  (s = 0 .. n-1, mu_s a vector), in
//                     32-bit, stored in the compute dtype as [n, rows >= M, d].  The previous token's input is the row in
//                     front where that row belongs to the same sequence, the sequence's state (float [d] a slot,
//                     the last input it was fed) where the step's first token of a sequence continues one under
//                     way, and zero at position 0.  The block of a sequence's first token of the step, the only
//                     reader of the old state, also leaves the sequence's last input of the step there: one
//                     kernel, no race, any cut of a sequence into steps.
// rl_tanh_cast        out = tanh(x), x float, out in the compute dtype
// rl_scaled_add       x += s0 * y0 + s1 * y1          (float; two mixers side by side with constant factors)
// rl_row_gate_add     x[m, :] += sigmoid(h[m, :] . g) * y[m, :]   (a sublayer that joins the stream through one
//                     learned gate a token)
// rl_scale            y *= s                           (float, in place)
#include <math.h>

#include "common.cuh"

#define TS_THREADS 256
#define TS_MAX_MIX 8

// V consecutive elements a thread (V * sizeof(T) = 16 bytes where the rows allow it, else 1); blockIdx.y walks the row
// in pieces of TS_THREADS * V elements, so that a step of few tokens still fills the machine.
template <typename T, int V>
__global__ void __launch_bounds__(TS_THREADS)
token_shift_mix_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ mu, int n_mix, const int* __restrict__ positions,
                       const int* __restrict__ slot_of_token, const int* __restrict__ cu_seqlens, int num_seqs,
                       float* __restrict__ state, long long state_stride, T* __restrict__ out, int M, int d, long long blend_rows) {
  __shared__ int s_first, s_last;
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const int slot = slot_of_token[m];
  if (threadIdx.x == 0) {
    const bool first = m == 0 || slot_of_token[m - 1] != slot;
    int last = -1;
    if (first) {                       // the sequence b with cu_seqlens[b] == m
      int lo = 0, hi = num_seqs - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (cu_seqlens[mid] <= m) lo = mid; else hi = mid - 1;
      }
      last = cu_seqlens[lo + 1] - 1;
    }
    s_first = first ? 1 : 0;
    s_last = last;
  }
  __syncthreads();
  const bool first = s_first != 0;
  const bool fresh = positions[m] == 0;
  const int i = (blockIdx.y * TS_THREADS + threadIdx.x) * V;
  if (i >= d) return;
  const T* cur = h + (size_t)m * ldh + i;
  float* st = state + (size_t)slot * state_stride + i;
  struct alignas(V * sizeof(T)) Pack { T e[V]; };
  float c[V], p[V];
  {
    const Pack pk = *reinterpret_cast<const Pack*>(cur);
#pragma unroll
    for (int k = 0; k < V; ++k) c[k] = rl_ld(&pk.e[k]);
  }
  if (!first) {                        // the row in front belongs to the same sequence
    const Pack pk = *reinterpret_cast<const Pack*>(cur - ldh);
#pragma unroll
    for (int k = 0; k < V; ++k) p[k] = rl_ld(&pk.e[k]);
  } else {
    // this thread alone reads and writes its elements of the state: the old value first, then the sequence's last
    // input of the step
#pragma unroll
    for (int k = 0; k < V; ++k) p[k] = fresh ? 0.f : st[k];
    const Pack pk = *reinterpret_cast<const Pack*>(h + (size_t)s_last * ldh + i);
#pragma unroll
    for (int k = 0; k < V; ++k) st[k] = rl_ld(&pk.e[k]);
  }
  for (int s = 0; s < n_mix; ++s) {
    Pack o;
#pragma unroll
    for (int k = 0; k < V; ++k) rl_st(&o.e[k], fmaf(p[k] - c[k], mu[(size_t)s * d + i + k], c[k]));
    *reinterpret_cast<Pack*>(out + ((size_t)s * blend_rows + m) * d + i) = o;
  }
}

template <typename T>
__global__ void __launch_bounds__(TS_THREADS)
tanh_cast_kernel(const float* __restrict__ x, T* __restrict__ out, size_t n) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const size_t i = (size_t)blockIdx.x * TS_THREADS + threadIdx.x;
  if (i < n) rl_st(out + i, tanhf(x[i]));
}

__global__ void __launch_bounds__(TS_THREADS)
scaled_add_kernel(float* __restrict__ x, const float* __restrict__ y0, float s0, const float* __restrict__ y1, float s1, size_t n4) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const size_t i = (size_t)blockIdx.x * TS_THREADS + threadIdx.x;
  if (i >= n4) return;
  float4 a = reinterpret_cast<float4*>(x)[i];
  const float4 b = reinterpret_cast<const float4*>(y0)[i];
  a.x = fmaf(s0, b.x, a.x); a.y = fmaf(s0, b.y, a.y); a.z = fmaf(s0, b.z, a.z); a.w = fmaf(s0, b.w, a.w);
  if (y1) {
    const float4 c = reinterpret_cast<const float4*>(y1)[i];
    a.x = fmaf(s1, c.x, a.x); a.y = fmaf(s1, c.y, a.y); a.z = fmaf(s1, c.z, a.z); a.w = fmaf(s1, c.w, a.w);
  }
  reinterpret_cast<float4*>(x)[i] = a;
}

__global__ void __launch_bounds__(TS_THREADS)
scaled_add_tail_kernel(float* __restrict__ x, const float* __restrict__ y0, float s0, const float* __restrict__ y1, float s1, size_t from,
                       size_t n) {
  const size_t i = from + (size_t)blockIdx.x * TS_THREADS + threadIdx.x;
  if (i < n) x[i] = fmaf(s0, y0[i], x[i]) + (y1 ? s1 * y1[i] : 0.f);
}

template <typename T>
__global__ void __launch_bounds__(TS_THREADS)
row_gate_add_kernel(float* __restrict__ x, const float* __restrict__ y, const T* __restrict__ h, int ldh, const T* __restrict__ g, int d) {
  __shared__ float s_part[TS_THREADS / 32];
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const T* hr = h + (size_t)m * ldh;
  float dot = 0.f;
  for (int i = threadIdx.x; i < d; i += TS_THREADS) dot = fmaf(rl_ld(hr + i), rl_ld(g + i), dot);
  dot = rl_warp_sum(dot);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = dot;
  __syncthreads();
  float z = 0.f;
#pragma unroll
  for (int w = 0; w < TS_THREADS / 32; ++w) z += s_part[w];
  const float gate = 1.0f / (1.0f + expf(-z));
  const size_t row = (size_t)m * d;
  for (int i = threadIdx.x; i < d; i += TS_THREADS) x[row + i] = fmaf(gate, y[row + i], x[row + i]);
}

__global__ void __launch_bounds__(TS_THREADS)
scale_kernel(float* __restrict__ y, size_t n, float s) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const size_t i = (size_t)blockIdx.x * TS_THREADS + threadIdx.x;
  if (i < n) y[i] *= s;
}

// h [M, ldh] and out [n_mix, blend_rows, d] in `dtype` (blend_rows >= M: every blend's rows may be padded, e.g. to whole
// tiles of a product that reads them; rows beyond M are not written); mu float [n_mix, d]; state float, [d] of slot s at state + s * state_stride.
extern "C" int rl_token_shift_mix(const void* h, int ldh, int dtype, const float* mu, int n_mix, const int* positions,
                                  const int* slot_of_token, const int* cu_seqlens, int num_seqs, float* state, long long state_stride,
                                  void* out, int blend_rows, int num_tokens, int width, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && width > 0 && ldh >= width && num_seqs >= 0 && blend_rows >= num_tokens, "rl_token_shift_mix: bad sizes");
  RL_REQUIRE(n_mix > 0 && n_mix <= TS_MAX_MIX, "rl_token_shift_mix: %d blends outside [1, %d]", n_mix, TS_MAX_MIX);
  RL_REQUIRE(state != nullptr && state_stride >= width, "rl_token_shift_mix: no state, or its rows are shorter than %d", width);
  if (num_tokens == 0) return RL_OK;
  RL_REQUIRE(num_seqs > 0, "rl_token_shift_mix: tokens without a sequence");
  const int esz = dtype == RL_F32 ? 4 : 2, vec = 16 / esz;
  const bool wide = width % vec == 0 && ldh % vec == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)out & 15) == 0;
  const dim3 grid(num_tokens, (width + TS_THREADS * (wide ? vec : 1) - 1) / (TS_THREADS * (wide ? vec : 1)));
#define TS_GO(T, V)                                                                                                                   \
  rl_launch_pdl(token_shift_mix_kernel<T, V>, grid, TS_THREADS, 0, stream, (const T*)h, ldh, mu, n_mix, positions, slot_of_token, cu_seqlens, \
                num_seqs, state, state_stride, (T*)out, num_tokens, width, (long long)blend_rows)
  if (dtype == RL_F32) {
    if (wide) TS_GO(float, 4); else TS_GO(float, 1);
  } else if (dtype == RL_BF16) {
    if (wide) TS_GO(__nv_bfloat16, 8); else TS_GO(__nv_bfloat16, 1);
  } else {
    RL_REQUIRE(false, "rl_token_shift_mix: unknown dtype %d", dtype);
  }
#undef TS_GO
  RL_LAUNCH_CHECK("rl_token_shift_mix");
  return RL_OK;
}

extern "C" int rl_tanh_cast(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
  RL_REQUIRE(n >= 0, "rl_tanh_cast: bad size");
  if (n == 0) return RL_OK;
  const unsigned blocks = (unsigned)((n + TS_THREADS - 1) / TS_THREADS);
  if (out_dtype == RL_F32) rl_launch_pdl(tanh_cast_kernel<float>, blocks, TS_THREADS, 0, stream, x, (float*)out, (size_t)n);
  else if (out_dtype == RL_BF16) rl_launch_pdl(tanh_cast_kernel<__nv_bfloat16>, blocks, TS_THREADS, 0, stream, x, (__nv_bfloat16*)out, (size_t)n);
  else RL_REQUIRE(false, "rl_tanh_cast: unknown dtype %d", out_dtype);
  RL_LAUNCH_CHECK("rl_tanh_cast");
  return RL_OK;
}

extern "C" int rl_scaled_add(float* x, const float* y0, float s0, const float* y1, float s1, long long n, cudaStream_t stream) {
  RL_REQUIRE(n >= 0 && y0 != nullptr, "rl_scaled_add: bad arguments");
  if (n == 0) return RL_OK;
  const bool vec = (((uintptr_t)x | (uintptr_t)y0 | (uintptr_t)y1) & 15) == 0;
  const size_t n4 = vec ? (size_t)n / 4 : 0;
  if (n4) rl_launch_pdl(scaled_add_kernel, (unsigned)((n4 + TS_THREADS - 1) / TS_THREADS), TS_THREADS, 0, stream, x, y0, s0, y1, s1, n4);
  if (4 * n4 < (size_t)n) {
    const size_t left = (size_t)n - 4 * n4;
    scaled_add_tail_kernel<<<(unsigned)((left + TS_THREADS - 1) / TS_THREADS), TS_THREADS, 0, stream>>>(x, y0, s0, y1, s1, 4 * n4, (size_t)n);
  }
  RL_LAUNCH_CHECK("rl_scaled_add");
  return RL_OK;
}

// x, y float [M, d]; h [M, ldh] and g [d] in `dtype`.
extern "C" int rl_row_gate_add(float* x, const float* y, const void* h, int ldh, const void* g, int dtype, int num_tokens, int width,
                               cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && width > 0 && ldh >= width, "rl_row_gate_add: bad sizes");
  if (num_tokens == 0) return RL_OK;
  if (dtype == RL_F32)
    rl_launch_pdl(row_gate_add_kernel<float>, num_tokens, TS_THREADS, 0, stream, x, y, (const float*)h, ldh, (const float*)g, width);
  else if (dtype == RL_BF16)
    rl_launch_pdl(row_gate_add_kernel<__nv_bfloat16>, num_tokens, TS_THREADS, 0, stream, x, y, (const __nv_bfloat16*)h, ldh,
                  (const __nv_bfloat16*)g, width);
  else
    RL_REQUIRE(false, "rl_row_gate_add: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_row_gate_add");
  return RL_OK;
}

extern "C" int rl_scale(float* y, long long n, float s, cudaStream_t stream) {
  RL_REQUIRE(n >= 0, "rl_scale: bad size");
  if (n == 0) return RL_OK;
  rl_launch_pdl(scale_kernel, (unsigned)((n + TS_THREADS - 1) / TS_THREADS), TS_THREADS, 0, stream, y, (size_t)n, s);
  RL_LAUNCH_CHECK("rl_scale");
  return RL_OK;
}
