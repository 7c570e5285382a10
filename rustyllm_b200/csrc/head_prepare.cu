// What stands between a layer's first projections and its attention, for heads that are turned first and
// brought to unit size afterwards, and for attention through a latent.  All arithmetic is 32-bit (angles from
// float(position) * inv_freq with the accurate sincosf; sums of squares; 1 / sqrtf), one rounding at the store.
//
// rl_qk_rotate_unit   u holds H query heads and G key heads as projected.  Each head: the first `rot` dimensions
//                     turn by the token's position (neighbouring pairs (2i, 2i + 1) or split pairs (i, i + rot/2)),
//                     then - unit_norm - the whole head is divided by its root mean square (no weight).  Queries
//                     go to q_out, keys to their page.  value_from_key: the key head as it was projected (before
//                     the turn and the norm) is also the value and goes to the value pool's page.
// rl_latent_prepare   u holds [query latent (q_rank) | key/value latent (kv_rank) | shared rotary key (rd)].  The
//                     query latent is RMS-normed with a weight into cq; the key/value latent is RMS-normed with a
//                     weight, the rotary part turned, and [latent | rotary key] written as the token's one key row
//                     of kv_rank + rd elements (the values are its first kv_rank elements).
// rl_latent_query     the rotary parts of the query heads ([plain (hd) | rotary (rd)] a head) are turned and written
//                     behind the kv_rank columns of each head of the latent query buffer [M, H, kv_rank + rd]
//                     (whose first kv_rank columns a product with the keys' up-projection fills).
#include <math.h>

#include "common.cuh"

#define HP_WARPS 4
#define HP_MAX_W 256
#define HP_THREADS 256

template <typename T>
__global__ void __launch_bounds__(HP_WARPS * 32)
qk_rotate_unit_kernel(const T* __restrict__ u, int ldu, T* __restrict__ q_out, int ldq, const int* __restrict__ positions,
                      const int* __restrict__ slot_of_token, const int* __restrict__ page_table, int max_pages,
                      const float* __restrict__ inv_freq, int rot, int interleaved, int unit_norm, float eps, int H, int G, int hd,
                      int value_from_key, T* __restrict__ k_pool, T* __restrict__ v_pool) {
  constexpr int NE = HP_MAX_W / 32;
  __shared__ float s_val[HP_WARPS][HP_MAX_W];
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hs = blockIdx.y * HP_WARPS + warp;          // head: queries first, then keys
  if (hs >= H + G) return;
  const bool is_q = hs < H;
  const int pos = positions[m];
  const T* src = u + (size_t)m * ldu + (size_t)hs * hd;
  float val[NE];
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    const int i = lane + 32 * e;
    val[e] = i < hd ? rl_ld(src + i) : 0.f;
    if (i < hd) s_val[warp][i] = val[e];
  }
  T* kdst = nullptr;
  if (!is_q && k_pool != nullptr) {
    const int slot = slot_of_token[m];
    const int page = page_table[(size_t)slot * max_pages + pos / RL_PAGE];
    const size_t row = (((size_t)page * G + (hs - H)) * RL_PAGE + pos % RL_PAGE) * hd;
    kdst = k_pool + row;
    if (value_from_key) {
      T* vdst = v_pool + row;
#pragma unroll
      for (int e = 0; e < NE; ++e) {
        const int i = lane + 32 * e;
        if (i < hd) rl_st(vdst + i, val[e]);
      }
    }
  }
  __syncwarp();
  if (rot > 0) {
    const int half = rot / 2;
#pragma unroll
    for (int e = 0; e < NE; ++e) {
      const int i = lane + 32 * e;
      if (i < rot) {
        // first: this element is the pair's (u); else its (v).  (u, v) -> (u c - v s, v c + u s)
        const bool first = interleaved ? (i & 1) == 0 : i < half;
        const int pair = interleaved ? i >> 1 : (first ? i : i - half);
        const int partner = interleaved ? i ^ 1 : (first ? i + half : i - half);
        const float other = s_val[warp][partner];
        float sn, cs;
        sincosf((float)pos * inv_freq[pair], &sn, &cs);
        val[e] = first ? val[e] * cs - other * sn : val[e] * cs + other * sn;
      }
    }
  }
  if (unit_norm) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < NE; ++e) ss = fmaf(val[e], val[e], ss);     // elements beyond hd are 0
    const float r = 1.0f / sqrtf(rl_warp_sum(ss) / (float)hd + eps);
#pragma unroll
    for (int e = 0; e < NE; ++e) val[e] *= r;
  }
  T* dst = is_q ? q_out + (size_t)m * ldq + (size_t)hs * hd : kdst;
  if (dst == nullptr) return;
#pragma unroll
  for (int e = 0; e < NE; ++e) {
    const int i = lane + 32 * e;
    if (i < hd) rl_st(dst + i, val[e]);
  }
}

// The same for neighbouring pairs (2i, 2i + 1) with even widths and strides: a lane owns whole pairs (elements
// 2 lane + 64 e and the next), so a pair is one load and one store of twice the width, its partner needs no shared
// memory, and an angle's sine and cosine are computed once a pair.
__device__ __forceinline__ float2 hp_ld2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 hp_ld2(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ void hp_st2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void hp_st2(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }

template <typename T>
__global__ void __launch_bounds__(HP_WARPS * 32)
qk_rotate_unit_pairs_kernel(const T* __restrict__ u, int ldu, T* __restrict__ q_out, int ldq, const int* __restrict__ positions,
                            const int* __restrict__ slot_of_token, const int* __restrict__ page_table, int max_pages,
                            const float* __restrict__ inv_freq, int rot, int unit_norm, float eps, int H, int G, int hd,
                            int value_from_key, T* __restrict__ k_pool, T* __restrict__ v_pool) {
  constexpr int NP = HP_MAX_W / 64;
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hs = blockIdx.y * HP_WARPS + warp;          // head: queries first, then keys
  if (hs >= H + G) return;
  const bool is_q = hs < H;
  const int pos = positions[m];
  const T* src = u + (size_t)m * ldu + (size_t)hs * hd;
  float a[NP], b[NP];
#pragma unroll
  for (int e = 0; e < NP; ++e) {
    const int i = 2 * lane + 64 * e;
    const float2 v = i < hd ? hp_ld2(src + i) : make_float2(0.f, 0.f);
    a[e] = v.x; b[e] = v.y;
  }
  T* kdst = nullptr;
  if (!is_q && k_pool != nullptr) {
    const int slot = slot_of_token[m];
    const int page = page_table[(size_t)slot * max_pages + pos / RL_PAGE];
    const size_t row = (((size_t)page * G + (hs - H)) * RL_PAGE + pos % RL_PAGE) * hd;
    kdst = k_pool + row;
    if (value_from_key) {
      T* vdst = v_pool + row;
#pragma unroll
      for (int e = 0; e < NP; ++e) {
        const int i = 2 * lane + 64 * e;
        if (i < hd) hp_st2(vdst + i, a[e], b[e]);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < NP; ++e) {
    const int i = 2 * lane + 64 * e;
    if (i < rot) {
      float sn, cs;
      sincosf((float)pos * inv_freq[i >> 1], &sn, &cs);
      const float x = a[e], y = b[e];
      a[e] = x * cs - y * sn;
      b[e] = y * cs + x * sn;
    }
  }
  if (unit_norm) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < NP; ++e) ss = fmaf(b[e], b[e], fmaf(a[e], a[e], ss));     // elements beyond hd are 0
    const float r = 1.0f / sqrtf(rl_warp_sum(ss) / (float)hd + eps);
#pragma unroll
    for (int e = 0; e < NP; ++e) { a[e] *= r; b[e] *= r; }
  }
  T* dst = is_q ? q_out + (size_t)m * ldq + (size_t)hs * hd : kdst;
  if (dst == nullptr) return;
#pragma unroll
  for (int e = 0; e < NP; ++e) {
    const int i = 2 * lane + 64 * e;
    if (i < hd) hp_st2(dst + i, a[e], b[e]);
  }
}

// u [M, ldu]: columns [0, H*hd) the query heads, [H*hd, (H+G)*hd) the key heads.  q_out [M, ldq] (may be u itself:
// a head is read whole before it is written).  k_pool, v_pool: [pages, G, RL_PAGE, hd]; k_pool null: nothing is
// cached.  v_pool is needed (and written) only with value_from_key.
extern "C" int rl_qk_rotate_unit(const void* u, int ldu, void* q_out, int ldq, int dtype, const int* positions,
                                 const int* slot_of_token, const int* page_table, int max_pages, const float* inv_freq,
                                 int rotary_dim, int interleaved, int unit_norm, float eps, int num_tokens, int num_heads,
                                 int num_kv_heads, int head_dim, int value_from_key, void* k_pool, void* v_pool,
                                 cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && num_heads > 0 && num_kv_heads > 0, "rl_qk_rotate_unit: bad sizes");
  RL_REQUIRE(head_dim > 0 && head_dim <= HP_MAX_W, "rl_qk_rotate_unit: head width %d outside (0, %d]", head_dim, HP_MAX_W);
  RL_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
             "rl_qk_rotate_unit: rotary width %d must be even and <= %d", rotary_dim, head_dim);
  RL_REQUIRE(ldu >= (num_heads + num_kv_heads) * head_dim && ldq >= num_heads * head_dim, "rl_qk_rotate_unit: row strides too small");
  RL_REQUIRE(k_pool == nullptr || !value_from_key || v_pool != nullptr, "rl_qk_rotate_unit: values from keys need a value pool");
  if (num_tokens == 0) return RL_OK;
  const dim3 grid(num_tokens, (num_heads + num_kv_heads + HP_WARPS - 1) / HP_WARPS);
  // neighbouring pairs (or no rotation at all) on even sizes and addresses of whole pairs: a pair a load
  const uintptr_t two = dtype == RL_F32 ? 8 : 4;
  const bool pairs = (interleaved || rotary_dim == 0) && head_dim % 2 == 0 && ldu % 2 == 0 && ldq % 2 == 0 &&
                     (uintptr_t)u % two == 0 && (uintptr_t)q_out % two == 0 && (uintptr_t)k_pool % two == 0 && (uintptr_t)v_pool % two == 0;
  if (pairs && dtype == RL_F32)
    rl_launch_pdl(qk_rotate_unit_pairs_kernel<float>, grid, HP_WARPS * 32, 0, stream, (const float*)u, ldu, (float*)q_out, ldq, positions,
                  slot_of_token, page_table, max_pages, inv_freq, rotary_dim, unit_norm, eps, num_heads, num_kv_heads,
                  head_dim, value_from_key, (float*)k_pool, (float*)v_pool);
  else if (pairs && dtype == RL_BF16)
    rl_launch_pdl(qk_rotate_unit_pairs_kernel<__nv_bfloat16>, grid, HP_WARPS * 32, 0, stream, (const __nv_bfloat16*)u, ldu,
                  (__nv_bfloat16*)q_out, ldq, positions, slot_of_token, page_table, max_pages, inv_freq, rotary_dim,
                  unit_norm, eps, num_heads, num_kv_heads, head_dim, value_from_key, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool);
  else if (dtype == RL_F32)
    rl_launch_pdl(qk_rotate_unit_kernel<float>, grid, HP_WARPS * 32, 0, stream, (const float*)u, ldu, (float*)q_out, ldq, positions,
                  slot_of_token, page_table, max_pages, inv_freq, rotary_dim, interleaved, unit_norm, eps, num_heads, num_kv_heads,
                  head_dim, value_from_key, (float*)k_pool, (float*)v_pool);
  else if (dtype == RL_BF16)
    rl_launch_pdl(qk_rotate_unit_kernel<__nv_bfloat16>, grid, HP_WARPS * 32, 0, stream, (const __nv_bfloat16*)u, ldu,
                  (__nv_bfloat16*)q_out, ldq, positions, slot_of_token, page_table, max_pages, inv_freq, rotary_dim, interleaved,
                  unit_norm, eps, num_heads, num_kv_heads, head_dim, value_from_key, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool);
  else
    RL_REQUIRE(false, "rl_qk_rotate_unit: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_qk_rotate_unit");
  return RL_OK;
}

// ------------------------------------------------------------------ attention through a latent
__device__ __forceinline__ float hp_block_sum(float v, float* s_part) {
  v = rl_warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) s_part[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < HP_THREADS / 32; ++w) t += s_part[w];
  return t;
}

// the element i of a rotary part of width rd whose first `rot` dimensions turn: (u, v) -> (u c - v s, v c + u s)
template <typename T>
__device__ __forceinline__ float hp_turned(const T* part, int i, int rot, int interleaved, int pos, const float* inv_freq) {
  const float mine = rl_ld(part + i);
  if (i >= rot) return mine;
  const int half = rot / 2;
  const bool first = interleaved ? (i & 1) == 0 : i < half;
  const int pair = interleaved ? i >> 1 : (first ? i : i - half);
  const int partner = interleaved ? i ^ 1 : (first ? i + half : i - half);
  const float other = rl_ld(part + partner);
  float sn, cs;
  sincosf((float)pos * inv_freq[pair], &sn, &cs);
  return first ? mine * cs - other * sn : mine * cs + other * sn;
}

template <typename T>
__global__ void __launch_bounds__(HP_THREADS)
latent_prepare_kernel(const T* __restrict__ u, int ldu, int q_rank, int kv_rank, int rd, const float* __restrict__ q_w,
                      const float* __restrict__ kv_w, float eps, T* __restrict__ cq, int ldc, const int* __restrict__ positions,
                      const int* __restrict__ slot_of_token, const int* __restrict__ page_table, int max_pages,
                      const float* __restrict__ inv_freq, int rot, int interleaved, T* __restrict__ k_pool) {
  __shared__ float s_part[HP_THREADS / 32];
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const T* row = u + (size_t)m * ldu;
  const int pos = positions[m];
  if (q_rank > 0) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += HP_THREADS) {
      const float v = rl_ld(row + i);
      ss = fmaf(v, v, ss);
    }
    const float r = 1.0f / sqrtf(hp_block_sum(ss, s_part) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += HP_THREADS) rl_st(cq + (size_t)m * ldc + i, rl_ld(row + i) * r * q_w[i]);
  }
  const T* c = row + q_rank;
  float ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += HP_THREADS) {
    const float v = rl_ld(c + i);
    ss = fmaf(v, v, ss);
  }
  const float r = 1.0f / sqrtf(hp_block_sum(ss, s_part) / (float)kv_rank + eps);
  if (k_pool == nullptr) return;
  const int slot = slot_of_token[m];
  const int page = page_table[(size_t)slot * max_pages + pos / RL_PAGE];
  T* dst = k_pool + ((size_t)page * RL_PAGE + pos % RL_PAGE) * (kv_rank + rd);
  for (int i = threadIdx.x; i < kv_rank; i += HP_THREADS) rl_st(dst + i, rl_ld(c + i) * r * kv_w[i]);
  for (int i = threadIdx.x; i < rd; i += HP_THREADS) rl_st(dst + kv_rank + i, hp_turned(c + kv_rank, i, rot, interleaved, pos, inv_freq));
}

// The same with a thread owning neighbouring pairs (all widths, strides and offsets even; rotation of neighbours
// or none): accesses of twice the width, one sine and cosine a pair.
template <typename T>
__global__ void __launch_bounds__(HP_THREADS)
latent_prepare_pairs_kernel(const T* __restrict__ u, int ldu, int q_rank, int kv_rank, int rd, const float* __restrict__ q_w,
                            const float* __restrict__ kv_w, float eps, T* __restrict__ cq, int ldc, const int* __restrict__ positions,
                            const int* __restrict__ slot_of_token, const int* __restrict__ page_table, int max_pages,
                            const float* __restrict__ inv_freq, int rot, T* __restrict__ k_pool) {
  __shared__ float s_part[HP_THREADS / 32];
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const T* row = u + (size_t)m * ldu;
  const int pos = positions[m];
  if (q_rank > 0) {
    float ss = 0.f;
    for (int i = 2 * threadIdx.x; i < q_rank; i += 2 * HP_THREADS) {
      const float2 v = hp_ld2(row + i);
      ss = fmaf(v.y, v.y, fmaf(v.x, v.x, ss));
    }
    const float r = 1.0f / sqrtf(hp_block_sum(ss, s_part) / (float)q_rank + eps);
    for (int i = 2 * threadIdx.x; i < q_rank; i += 2 * HP_THREADS) {
      const float2 v = hp_ld2(row + i);
      hp_st2(cq + (size_t)m * ldc + i, v.x * r * q_w[i], v.y * r * q_w[i + 1]);
    }
  }
  const T* c = row + q_rank;
  float ss = 0.f;
  for (int i = 2 * threadIdx.x; i < kv_rank; i += 2 * HP_THREADS) {
    const float2 v = hp_ld2(c + i);
    ss = fmaf(v.y, v.y, fmaf(v.x, v.x, ss));
  }
  const float r = 1.0f / sqrtf(hp_block_sum(ss, s_part) / (float)kv_rank + eps);
  if (k_pool == nullptr) return;
  const int slot = slot_of_token[m];
  const int page = page_table[(size_t)slot * max_pages + pos / RL_PAGE];
  T* dst = k_pool + ((size_t)page * RL_PAGE + pos % RL_PAGE) * (kv_rank + rd);
  for (int i = 2 * threadIdx.x; i < kv_rank; i += 2 * HP_THREADS) {
    const float2 v = hp_ld2(c + i);
    hp_st2(dst + i, v.x * r * kv_w[i], v.y * r * kv_w[i + 1]);
  }
  for (int i = 2 * threadIdx.x; i < rd; i += 2 * HP_THREADS) {
    float2 v = hp_ld2(c + kv_rank + i);
    if (i < rot) {
      float sn, cs;
      sincosf((float)pos * inv_freq[i >> 1], &sn, &cs);
      v = make_float2(v.x * cs - v.y * sn, v.y * cs + v.x * sn);
    }
    hp_st2(dst + kv_rank + i, v.x, v.y);
  }
}

// u [M, ldu] with columns [0, q_rank) | [q_rank, q_rank + kv_rank) | [.., + rd); q_w float [q_rank], kv_w float [kv_rank];
// cq [M, ldc]; k_pool [pages, 1, RL_PAGE, kv_rank + rd] (null: nothing is cached).  q_rank 0: no query latent.
extern "C" int rl_latent_prepare(const void* u, int ldu, int dtype, int q_rank, int kv_rank, int rot_dim, const float* q_w,
                                 const float* kv_w, float eps, void* cq, int ldc, const int* positions, const int* slot_of_token,
                                 const int* page_table, int max_pages, const float* inv_freq, int rotary_dim, int interleaved,
                                 int num_tokens, void* k_pool, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && q_rank >= 0 && kv_rank > 0 && rot_dim >= 0, "rl_latent_prepare: bad sizes");
  RL_REQUIRE(rotary_dim >= 0 && rotary_dim <= rot_dim && rotary_dim % 2 == 0, "rl_latent_prepare: rotary width %d must be even and <= %d",
             rotary_dim, rot_dim);
  RL_REQUIRE(ldu >= q_rank + kv_rank + rot_dim && (q_rank == 0 || ldc >= q_rank), "rl_latent_prepare: row strides too small");
  RL_REQUIRE(kv_w != nullptr && (q_rank == 0 || (q_w != nullptr && cq != nullptr)), "rl_latent_prepare: a norm weight or the output is missing");
  if (num_tokens == 0) return RL_OK;
  const uintptr_t two = dtype == RL_F32 ? 8 : 4;
  const bool pairs = (interleaved || rotary_dim == 0) && q_rank % 2 == 0 && kv_rank % 2 == 0 && rot_dim % 2 == 0 && ldu % 2 == 0 &&
                     ldc % 2 == 0 && (uintptr_t)u % two == 0 && (uintptr_t)cq % two == 0 && (uintptr_t)k_pool % two == 0;
  if (pairs && dtype == RL_F32)
    rl_launch_pdl(latent_prepare_pairs_kernel<float>, num_tokens, HP_THREADS, 0, stream, (const float*)u, ldu, q_rank, kv_rank, rot_dim,
                  q_w, kv_w, eps, (float*)cq, ldc, positions, slot_of_token, page_table, max_pages, inv_freq, rotary_dim, (float*)k_pool);
  else if (pairs && dtype == RL_BF16)
    rl_launch_pdl(latent_prepare_pairs_kernel<__nv_bfloat16>, num_tokens, HP_THREADS, 0, stream, (const __nv_bfloat16*)u, ldu, q_rank,
                  kv_rank, rot_dim, q_w, kv_w, eps, (__nv_bfloat16*)cq, ldc, positions, slot_of_token, page_table, max_pages, inv_freq,
                  rotary_dim, (__nv_bfloat16*)k_pool);
  else if (dtype == RL_F32)
    rl_launch_pdl(latent_prepare_kernel<float>, num_tokens, HP_THREADS, 0, stream, (const float*)u, ldu, q_rank, kv_rank, rot_dim, q_w,
                  kv_w, eps, (float*)cq, ldc, positions, slot_of_token, page_table, max_pages, inv_freq, rotary_dim, interleaved,
                  (float*)k_pool);
  else if (dtype == RL_BF16)
    rl_launch_pdl(latent_prepare_kernel<__nv_bfloat16>, num_tokens, HP_THREADS, 0, stream, (const __nv_bfloat16*)u, ldu, q_rank, kv_rank,
                  rot_dim, q_w, kv_w, eps, (__nv_bfloat16*)cq, ldc, positions, slot_of_token, page_table, max_pages, inv_freq,
                  rotary_dim, interleaved, (__nv_bfloat16*)k_pool);
  else
    RL_REQUIRE(false, "rl_latent_prepare: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_latent_prepare");
  return RL_OK;
}

template <typename T>
__global__ void __launch_bounds__(HP_THREADS)
latent_query_kernel(const T* __restrict__ q, int ldq, int H, int hd, int rd, const int* __restrict__ positions,
                    const float* __restrict__ inv_freq, int rot, int interleaved, T* __restrict__ out, int ldo, int lat) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const int pos = positions[m];
  for (int e = threadIdx.x; e < H * rd; e += HP_THREADS) {
    const int h = e / rd, i = e % rd;
    const T* part = q + (size_t)m * ldq + (size_t)h * (hd + rd) + hd;
    rl_st(out + (size_t)m * ldo + (size_t)h * (lat + rd) + lat + i, hp_turned(part, i, rot, interleaved, pos, inv_freq));
  }
}

template <typename T>
__global__ void __launch_bounds__(HP_THREADS)
latent_query_pairs_kernel(const T* __restrict__ q, int ldq, int H, int hd, int rd, const int* __restrict__ positions,
                          const float* __restrict__ inv_freq, int rot, T* __restrict__ out, int ldo, int lat) {
  rl_pdl_trigger();
  rl_pdl_wait();
  const int m = blockIdx.x;
  const int pos = positions[m];
  const int half = rd >> 1;
  for (int e = threadIdx.x; e < H * half; e += HP_THREADS) {
    const int h = e / half, i = 2 * (e % half);
    float2 v = hp_ld2(q + (size_t)m * ldq + (size_t)h * (hd + rd) + hd + i);
    if (i < rot) {
      float sn, cs;
      sincosf((float)pos * inv_freq[i >> 1], &sn, &cs);
      v = make_float2(v.x * cs - v.y * sn, v.y * cs + v.x * sn);
    }
    hp_st2(out + (size_t)m * ldo + (size_t)h * (lat + rd) + lat + i, v.x, v.y);
  }
}

// q [M, ldq]: H heads of [hd | rd]; out [M, ldo]: H heads of [lat | rd], of which this fills the rd columns.
extern "C" int rl_latent_query(const void* q, int ldq, int dtype, int num_heads, int head_dim, int rot_dim, const int* positions,
                               const float* inv_freq, int rotary_dim, int interleaved, void* out, int ldo, int latent_dim,
                               int num_tokens, cudaStream_t stream) {
  RL_REQUIRE(num_tokens >= 0 && num_heads > 0 && head_dim > 0 && rot_dim >= 0 && latent_dim > 0, "rl_latent_query: bad sizes");
  RL_REQUIRE(rotary_dim >= 0 && rotary_dim <= rot_dim && rotary_dim % 2 == 0, "rl_latent_query: rotary width %d must be even and <= %d",
             rotary_dim, rot_dim);
  RL_REQUIRE(ldq >= num_heads * (head_dim + rot_dim) && ldo >= num_heads * (latent_dim + rot_dim), "rl_latent_query: row strides too small");
  if (num_tokens == 0 || rot_dim == 0) return RL_OK;
  const uintptr_t two = dtype == RL_F32 ? 8 : 4;
  const bool pairs = (interleaved || rotary_dim == 0) && head_dim % 2 == 0 && rot_dim % 2 == 0 && latent_dim % 2 == 0 && ldq % 2 == 0 &&
                     ldo % 2 == 0 && (uintptr_t)q % two == 0 && (uintptr_t)out % two == 0;
  if (pairs && dtype == RL_F32)
    rl_launch_pdl(latent_query_pairs_kernel<float>, num_tokens, HP_THREADS, 0, stream, (const float*)q, ldq, num_heads, head_dim, rot_dim,
                  positions, inv_freq, rotary_dim, (float*)out, ldo, latent_dim);
  else if (pairs && dtype == RL_BF16)
    rl_launch_pdl(latent_query_pairs_kernel<__nv_bfloat16>, num_tokens, HP_THREADS, 0, stream, (const __nv_bfloat16*)q, ldq, num_heads,
                  head_dim, rot_dim, positions, inv_freq, rotary_dim, (__nv_bfloat16*)out, ldo, latent_dim);
  else if (dtype == RL_F32)
    rl_launch_pdl(latent_query_kernel<float>, num_tokens, HP_THREADS, 0, stream, (const float*)q, ldq, num_heads, head_dim, rot_dim,
                  positions, inv_freq, rotary_dim, interleaved, (float*)out, ldo, latent_dim);
  else if (dtype == RL_BF16)
    rl_launch_pdl(latent_query_kernel<__nv_bfloat16>, num_tokens, HP_THREADS, 0, stream, (const __nv_bfloat16*)q, ldq, num_heads,
                  head_dim, rot_dim, positions, inv_freq, rotary_dim, interleaved, (__nv_bfloat16*)out, ldo, latent_dim);
  else
    RL_REQUIRE(false, "rl_latent_query: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_latent_query");
  return RL_OK;
}

// ------------------------------------------------------------------ a product a head, few tokens
// out[m, a * out_head + n] = sum_k W[a][n][k] * x[m, a * x_head + k]: every head a has a matrix [N, K] of its own
// and its own K columns of x (H small products as one launch; with few tokens they only stream the weights).
// A block: 8 output columns of one head (a warp each) for 16 tokens, whose K inputs wait in shared memory as float.
#define HL_TOKENS 16
template <typename T>
__global__ void __launch_bounds__(256)
heads_linear_kernel(const T* __restrict__ x, int ldx, int x_head, const T* __restrict__ w, T* __restrict__ out, int ldo,
                    int out_head, int M, int N, int K) {
  extern __shared__ float hl_x[];          // [HL_TOKENS][K]
  const int a = blockIdx.y, m0 = blockIdx.z * HL_TOKENS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < HL_TOKENS * K; i += 256) {
    const int m = i / K, k = i - m * K;
    hl_x[i] = m0 + m < M ? rl_ld(x + (size_t)(m0 + m) * ldx + (size_t)a * x_head + k) : 0.f;
  }
  __syncthreads();
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const T* wrow = w + ((size_t)a * N + n) * K;
  float acc[HL_TOKENS];
#pragma unroll
  for (int m = 0; m < HL_TOKENS; ++m) acc[m] = 0.f;
  for (int k = lane; k < K; k += 32) {
    const float wv = rl_ld(wrow + k);
#pragma unroll
    for (int m = 0; m < HL_TOKENS; ++m) acc[m] = fmaf(wv, hl_x[m * K + k], acc[m]);
  }
  float mine = 0.f;
#pragma unroll
  for (int m = 0; m < HL_TOKENS; ++m) {
    const float v = rl_warp_sum(acc[m]);
    if (lane == m) mine = v;
  }
  if (lane < HL_TOKENS && m0 + lane < M) rl_st(out + (size_t)(m0 + lane) * ldo + (size_t)a * out_head + n, mine);
}

// x: [M, ldx] with head a's K inputs at columns [a * x_head, a * x_head + K); w: [H, N, K] contiguous; out: [M, ldo]
// with head a's N outputs at columns [a * out_head, a * out_head + N); all of one dtype, sums in 32-bit.
extern "C" int rl_heads_linear(const void* x, int ldx, int x_head, const void* w, void* out, int ldo, int out_head, int dtype,
                               int M, int H, int N, int K, cudaStream_t stream) {
  RL_REQUIRE(M >= 0 && H > 0 && N > 0 && K > 0 && H <= 65535, "rl_heads_linear: bad sizes");
  RL_REQUIRE(ldx >= (H - 1) * x_head + K && ldo >= (H - 1) * out_head + N && x_head >= 0 && out_head >= N,
             "rl_heads_linear: row strides too small for the heads");
  const size_t smem = (size_t)HL_TOKENS * K * sizeof(float);
  RL_REQUIRE(smem <= 48 * 1024, "rl_heads_linear: %d inputs a head exceed the %d this kernel holds", K, 48 * 1024 / (HL_TOKENS * 4));
  if (M == 0) return RL_OK;
  const dim3 grid((N + 7) / 8, H, (M + HL_TOKENS - 1) / HL_TOKENS);
  RL_REQUIRE(grid.z <= 65535, "rl_heads_linear: too many tokens (%d) for this kernel", M);
  if (dtype == RL_F32)
    heads_linear_kernel<float><<<grid, 256, smem, stream>>>((const float*)x, ldx, x_head, (const float*)w, (float*)out, ldo, out_head, M, N, K);
  else if (dtype == RL_BF16)
    heads_linear_kernel<__nv_bfloat16><<<grid, 256, smem, stream>>>((const __nv_bfloat16*)x, ldx, x_head, (const __nv_bfloat16*)w,
                                                                   (__nv_bfloat16*)out, ldo, out_head, M, N, K);
  else
    RL_REQUIRE(false, "rl_heads_linear: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_heads_linear");
  return RL_OK;
}
