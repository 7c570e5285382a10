// Layer norm with a weight and no bias, in 32-bit:  y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w.
//
// The variance is the mean of the squared deviations from the mean (two passes over a row that stays in
// registers, so nothing cancels).  A layer whose two sublayers both read norms of the same stream needs the
// row's mean and variance once: the kernel takes a second weight and a second output and writes both
// normed rows from one read of x.
#include <math.h>

#include "common.cuh"

#define LN_THREADS 256

__device__ __forceinline__ float ln_block_sum(float v, float* s_part) {
  v = rl_warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                       // s_part may still be read from an earlier call
  if (lane == 0) s_part[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < LN_THREADS / 32; ++w) t += s_part[w];
  return t;
}

// any width: the row is read three times (the second and third time from L1)
template <typename TO>
__global__ void __launch_bounds__(LN_THREADS)
layer_norm_kernel(const float* __restrict__ x, const float* __restrict__ w0, TO* __restrict__ out0, const float* __restrict__ w1,
                  TO* __restrict__ out1, const int* __restrict__ rows, int d, float eps) {
  __shared__ float s_part[LN_THREADS / 32];
  rl_pdl_trigger();
  rl_pdl_wait();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * d;
  float s = 0.f;
  for (int i = threadIdx.x; i < d; i += LN_THREADS) s += xr[i];
  const float mean = ln_block_sum(s, s_part) / (float)d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += LN_THREADS) {
    const float c = xr[i] - mean;
    ss = fmaf(c, c, ss);
  }
  const float inv = 1.0f / sqrtf(ln_block_sum(ss, s_part) / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += LN_THREADS) {
    const float c = (xr[i] - mean) * inv;
    rl_st(out0 + (size_t)r * d + i, c * w0[i]);
    if (out1) rl_st(out1 + (size_t)r * d + i, c * w1[i]);
  }
}

// rows of up to LN_THREADS * 4 * MAXV floats, a multiple of 4 long, 16-byte aligned: one read of the row
template <typename TO, int MAXV>
__global__ void __launch_bounds__(LN_THREADS)
layer_norm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w0, TO* __restrict__ out0, const float* __restrict__ w1,
                      TO* __restrict__ out1, const int* __restrict__ rows, int d, float eps) {
  __shared__ float s_part[LN_THREADS / 32];
  rl_pdl_trigger();
  rl_pdl_wait();
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
  const int nv = d / 4;
  float4 v[MAXV];
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * LN_THREADS;
    v[k] = i < nv ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
  }
  const float mean = ln_block_sum(s, s_part) / (float)d;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * LN_THREADS;
    if (i < nv) {
      v[k].x -= mean; v[k].y -= mean; v[k].z -= mean; v[k].w -= mean;
      ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss);
      ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
    }
  }
  const float inv = 1.0f / sqrtf(ln_block_sum(ss, s_part) / (float)d + eps);
  auto store = [&](TO* o, const float4* w4, int i, const float4& c) {
    const float4 g = w4[i];
    const float a = c.x * inv * g.x, b = c.y * inv * g.y, e = c.z * inv * g.z, f = c.w * inv * g.w;
    if constexpr (sizeof(TO) == 2) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(e, f);
      *reinterpret_cast<uint2*>(o + 4 * i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    } else {
      *reinterpret_cast<float4*>(o + 4 * i) = make_float4(a, b, e, f);
    }
  };
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * LN_THREADS;
    if (i < nv) {
      store(out0 + (size_t)r * d, reinterpret_cast<const float4*>(w0), i, v[k]);
      if (out1) store(out1 + (size_t)r * d, reinterpret_cast<const float4*>(w1), i, v[k]);
    }
  }
}

template <typename TO>
static void layer_norm_launch(const float* x, const float* w0, void* out0, const float* w1, void* out1, const int* rows, int num_rows,
                              int d, float eps, cudaStream_t stream) {
  const bool vec = d % 4 == 0 && d <= LN_THREADS * 4 * 8 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w0 & 15) == 0 &&
                   ((uintptr_t)out0 & 15) == 0 && ((uintptr_t)w1 & 15) == 0 && ((uintptr_t)out1 & 15) == 0;
  if (vec && d <= LN_THREADS * 4 * 2)
    rl_launch_pdl(layer_norm_vec_kernel<TO, 2>, num_rows, LN_THREADS, 0, stream, x, w0, (TO*)out0, w1, (TO*)out1, rows, d, eps);
  else if (vec)
    rl_launch_pdl(layer_norm_vec_kernel<TO, 8>, num_rows, LN_THREADS, 0, stream, x, w0, (TO*)out0, w1, (TO*)out1, rows, d, eps);
  else
    rl_launch_pdl(layer_norm_kernel<TO>, num_rows, LN_THREADS, 0, stream, x, w0, (TO*)out0, w1, (TO*)out1, rows, d, eps);
}

// out0[r, :] = layer_norm(x[rows ? rows[r] : r, :]) * weight0 and, where out1 is given, out1[r, :] = the same row's
// norm times weight1, for r in [0, num_rows).  x and the weights float; the outputs in out_dtype.
extern "C" int rl_layer_norm(const float* x, const float* weight0, void* out0, const float* weight1, void* out1, int out_dtype,
                             const int* rows, int num_rows, int hidden, float eps, cudaStream_t stream) {
  RL_REQUIRE(num_rows >= 0 && hidden > 0, "rl_layer_norm: bad sizes rows=%d d=%d", num_rows, hidden);
  RL_REQUIRE(eps > 0.f, "rl_layer_norm: eps must be > 0, got %g", (double)eps);
  RL_REQUIRE(weight0 != nullptr && out0 != nullptr && (weight1 == nullptr) == (out1 == nullptr),
             "rl_layer_norm: a weight without an output, or the other way round");
  if (num_rows == 0) return RL_OK;
  if (out_dtype == RL_F32)
    layer_norm_launch<float>(x, weight0, out0, weight1, out1, rows, num_rows, hidden, eps, stream);
  else if (out_dtype == RL_BF16)
    layer_norm_launch<__nv_bfloat16>(x, weight0, out0, weight1, out1, rows, num_rows, hidden, eps, stream);
  else
    RL_REQUIRE(false, "rl_layer_norm: unknown output dtype %d", out_dtype);
  RL_LAUNCH_CHECK("rl_layer_norm");
  return RL_OK;
}
