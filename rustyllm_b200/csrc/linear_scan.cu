// Linear recurrences with a matrix state per head, carried from step to step:
//
//   S_t = a_t S_{t-1} + b_t k_t v_t^T          (S: dk x dv, float, zero for a fresh sequence)
//   o_t = S_t^T q_t (+ skip_h v_t)
//
// mode 0: a_t = decay[h], b_t = 1 (linear attention with a fixed decay a head);
// mode 1: dt = softplus(dt_raw[t, h] + dt_bias[h]), a_t = exp(-exp(rate[h]) dt), b_t = dt (a selective
//         state space: q = C, k = B, v = x, skip = D).
// mode 2: a decay a key channel and token, and a bonus for the current token that does not enter the state:
//           o_t = (S_{t-1} + diag(u_h) k_t v_t^T)^T q_t,   S_t = diag(w_t) S_{t-1} + k_t v_t^T,
//         w_t = exp(-exp(wlog[t, h, :])) from the float logarithms `wlog` (the decay is never stored in fewer bits),
//         u float [H, dk].  (Template parameter CH; the other two modes are CH = false.)
// Query and key heads may be shared by `hpg` consecutive heads (head h reads group h / hpg).  With act = 1
// q, k and v pass through silu as they are loaded.  Everything behind the loads is 32-bit.
//
// A block owns 8 or 16 columns of one head's state of one sequence and walks the sequence's tokens of
// the step in order; R neighbouring lanes share a column (each holds NPT consecutive rows) and add their
// parts of q . S[:, col] by shuffles.  Tokens are staged 16 (8 in the shape for single-token steps) at a time in shared memory.  The walk is
// one dependent multiply-add a state element and token; everything else (the loads of q and k from shared
// memory, the dot product, the shuffles) is latency to hide, so R grows with dk (8, 16, 32: a block of 128,
// 256 or 512 threads, at most 8 state elements a thread): more warps an SM, fewer instructions a thread.
// The order of every sum is fixed by the sizes alone, so a position's output does not depend on how the
// sequence was cut into steps or on the batch.  State layout per slot: [H, dv, dk].
#include <math.h>

#include "common.cuh"

#define SCAN_MAX_DK 256

// silu at the load: accurate in a 32-bit run; with the fast exponential and division in a bfloat16 run, whose
// projections carry 8 bits
__device__ __forceinline__ float scan_silu(float z, float) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float scan_silu(float z, __nv_bfloat16) { return __fdividef(z, 1.0f + __expf(-z)); }

template <typename T, int NPT, int R, int SCAN_COLS, int SCAN_TILE, bool CH>
__global__ void __launch_bounds__(R * SCAN_COLS)
linear_scan_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ k, int ldk, const T* __restrict__ v, int ldv,
                   const T* __restrict__ dt_raw, int lddt, const float* __restrict__ dt_bias, const float* __restrict__ rate,
                   const float* __restrict__ skip, int mode, int act, const int* __restrict__ cu_seqlens,
                   const int* __restrict__ seq_slots, float* __restrict__ state, long long state_stride,
                   float* __restrict__ out, int ldo, int H, int hpg, int dk, int dv, const float* __restrict__ wlog, int ldw,
                   const float* __restrict__ bonus) {
  constexpr int DKP = NPT * R;                  // dk rounded up to what the lanes of a column hold: a power of two
  constexpr int THREADS = R * SCAN_COLS;
  // Two shapes.  Many tokens a sequence (NPT <= 8): a lane holds NPT consecutive rows (16-byte loads from shared
  // memory in the walk) and the next tile's q, k, v and step sizes are fetched into registers while this
  // tile is walked, so that no load from global memory is waited for.  Few tokens (NPT > 8, 8 lanes a column): a
  // lane holds rows r, r + 8, ... (the state's loads and stores are whole lines), staged directly.
  constexpr bool LONG = NPT <= 8;
  static_assert(!LONG || (R * SCAN_COLS >= SCAN_TILE * SCAN_COLS && (NPT % 4 == 0 || NPT == 2)), "the long shape stages a tile's values one a thread");
  // rows beyond dk are staged as zeros, so the walk needs no bounds: their state stays zero
  __shared__ __align__(16) float s_q[SCAN_TILE][DKP], s_k[SCAN_TILE][DKP];
  __shared__ float s_v[SCAN_TILE][SCAN_COLS], s_bv[SCAN_TILE][SCAN_COLS], s_a[SCAN_TILE];
  __shared__ __align__(16) float s_w[CH ? SCAN_TILE : 1][CH ? DKP : 4];      // the tokens' decays a key channel
  rl_pdl_trigger();
  rl_pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, r = tid % R, c = tid / R;
  const int col = blockIdx.z * SCAN_COLS + c;
  const bool live = col < dv;
  const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1];
  auto row_of = [&](int i) { return LONG ? NPT * r + i : r + R * i; };
  float* st = state + (size_t)seq_slots[b] * state_stride + ((size_t)h * dv + (live ? col : 0)) * dk;
  float S[NPT], U[CH ? NPT : 1];
#pragma unroll
  for (int i = 0; i < NPT; ++i) S[i] = (live && row_of(i) < dk) ? st[row_of(i)] : 0.f;
  if constexpr (CH) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) U[i] = row_of(i) < dk ? bonus[(size_t)h * dk + row_of(i)] : 0.f;
  }
  const int qk0 = (h / hpg) * dk;
  const float skip_h = skip ? skip[h] : 0.f;
  const float rate_h = CH ? 0.f : rate[h], bias_h = (!CH && mode) ? dt_bias[h] : 0.f;
  const float neg_rate = (!CH && mode) ? -expf(rate_h) : 0.f;

  // what a thread stages of a tile: QI elements of q and of k (element idx = tid + j * THREADS of the tile's
  // [SCAN_TILE, DKP]), one of v (threads below SCAN_TILE * SCAN_COLS) with its token's raw step size
  constexpr int VT = SCAN_TILE * SCAN_COLS;
  constexpr int QI = LONG ? SCAN_TILE * DKP / THREADS : 1;
  static_assert(!LONG || QI * THREADS == SCAN_TILE * DKP, "a tile's q and k are dealt evenly to the threads");
  float fq[QI], fk[QI], fw[CH ? QI : 1], fv = 0.f, fdt = 0.f;
  auto fetch = [&](int t0, int nt) {            // raw values of the tile at t0 into registers (zeros outside)
#pragma unroll
    for (int j = 0; j < QI; ++j) {
      const int idx = tid + j * THREADS, tt = idx / DKP, n = idx % DKP;
      const bool in = tt < nt && n < dk;
      fq[j] = in ? rl_ld(q + (size_t)(t0 + tt) * ldq + qk0 + n) : 0.f;
      fk[j] = in ? rl_ld(k + (size_t)(t0 + tt) * ldk + qk0 + n) : 0.f;
      if constexpr (CH) fw[j] = in ? wlog[(size_t)(t0 + tt) * ldw + (size_t)h * dk + n] : 0.f;
    }
    if (THREADS >= VT ? tid < VT : true) {
      const int tt = tid / SCAN_COLS, cc = blockIdx.z * SCAN_COLS + tid % SCAN_COLS;
      fv = (tt < nt && cc < dv) ? rl_ld(v + (size_t)(t0 + tt) * ldv + (size_t)h * dv + cc) : 0.f;
      fdt = (!CH && mode && tt < nt) ? rl_ld(dt_raw + (size_t)(t0 + tt) * lddt + h) : 0.f;
    }
  };
  auto step_size = [&](float raw) { const float z = raw + bias_h; return z > 20.0f ? z : log1pf(expf(z)); };
  auto commit = [&]() {                         // the fetched values, activated, into shared memory
#pragma unroll
    for (int j = 0; j < QI; ++j) {
      const int idx = tid + j * THREADS, tt = idx / DKP, n = idx % DKP;
      float qv = fq[j], kv = fk[j];
      if (act && n < dk) { qv = scan_silu(qv, T()); kv = scan_silu(kv, T()); }
      s_q[tt][n] = qv;
      s_k[tt][n] = kv;
      if constexpr (CH) s_w[tt][n] = n < dk ? expf(-expf(fw[j])) : 0.f;
    }
    if (tid < VT) {
      const int tt = tid / SCAN_COLS;
      const float vv = act ? scan_silu(fv, T()) : fv;
      const float dt = (!CH && mode) ? step_size(fdt) : 1.0f;
      s_v[tt][tid % SCAN_COLS] = vv;
      s_bv[tt][tid % SCAN_COLS] = dt * vv;
      if (tid % SCAN_COLS == 0) s_a[tt] = (!CH && mode) ? expf(neg_rate * dt) : rate_h;
    }
  };
  if (LONG && lo < hi) fetch(lo, min(SCAN_TILE, hi - lo));
  for (int t0 = lo; t0 < hi; t0 += SCAN_TILE) {
    const int nt = min(SCAN_TILE, hi - t0);
    __syncthreads();
    if (LONG) {
      commit();
    } else {
      // few tokens: straight from global memory (THREADS < VT here, so loops)
      for (int idx = tid; idx < nt * DKP; idx += THREADS) {
        const int tt = idx / DKP, n = idx % DKP;
        float qv = 0.f, kv = 0.f;
        if (n < dk) {
          qv = rl_ld(q + (size_t)(t0 + tt) * ldq + qk0 + n);
          kv = rl_ld(k + (size_t)(t0 + tt) * ldk + qk0 + n);
          if (act) { qv = scan_silu(qv, T()); kv = scan_silu(kv, T()); }
        }
        s_q[tt][n] = qv;
        s_k[tt][n] = kv;
        if constexpr (CH) s_w[tt][n] = n < dk ? expf(-expf(wlog[(size_t)(t0 + tt) * ldw + (size_t)h * dk + n])) : 0.f;
      }
      for (int idx = tid; idx < nt * SCAN_COLS; idx += THREADS) {
        const int tt = idx / SCAN_COLS, cc = blockIdx.z * SCAN_COLS + idx % SCAN_COLS;
        float vv = cc < dv ? rl_ld(v + (size_t)(t0 + tt) * ldv + (size_t)h * dv + cc) : 0.f;
        if (act) vv = scan_silu(vv, T());
        const float dt = (!CH && mode) ? step_size(rl_ld(dt_raw + (size_t)(t0 + tt) * lddt + h)) : 1.0f;
        s_v[tt][idx % SCAN_COLS] = vv;
        s_bv[tt][idx % SCAN_COLS] = dt * vv;
        if (idx % SCAN_COLS == 0) s_a[tt] = (!CH && mode) ? expf(neg_rate * dt) : rate_h;
      }
    }
    __syncthreads();
    if (LONG && t0 + SCAN_TILE < hi) fetch(t0 + SCAN_TILE, min(SCAN_TILE, hi - t0 - SCAN_TILE));   // in flight during the walk
    // the walk itself: loads from shared memory and multiply-adds only; every token's part of q . S[:, col]
    // stays in a register, and the lanes' parts are added afterwards, sixteen independent chains of shuffles
    float part[SCAN_TILE];
#pragma unroll
    for (int tt = 0; tt < SCAN_TILE; ++tt) {
      part[tt] = 0.f;
      if (tt < nt) {
        const float a = s_a[tt], bv = s_bv[tt][c];
        if constexpr (LONG && NPT == 2) {
          // two rows a lane (32 lanes a column of 64 rows): twice the warps of the four-row shape for one more shuffle
          const float2 kk = *reinterpret_cast<const float2*>(&s_k[tt][2 * r]), qq = *reinterpret_cast<const float2*>(&s_q[tt][2 * r]);
          if constexpr (CH) {
            const float2 ww = *reinterpret_cast<const float2*>(&s_w[tt][2 * r]);
            const float p0 = bv * kk.x, p1 = bv * kk.y;
            part[tt] = fmaf(fmaf(U[0], p0, S[0]), qq.x, part[tt]);
            part[tt] = fmaf(fmaf(U[1], p1, S[1]), qq.y, part[tt]);
            S[0] = fmaf(ww.x, S[0], p0);
            S[1] = fmaf(ww.y, S[1], p1);
          } else {
            S[0] = fmaf(a, S[0], bv * kk.x);
            S[1] = fmaf(a, S[1], bv * kk.y);
            part[tt] = fmaf(S[0], qq.x, part[tt]);
            part[tt] = fmaf(S[1], qq.y, part[tt]);
          }
        } else if (LONG) {
          const float4* k4 = reinterpret_cast<const float4*>(&s_k[tt][NPT * r]);
          const float4* q4 = reinterpret_cast<const float4*>(&s_q[tt][NPT * r]);
#pragma unroll
          for (int i = 0; i < NPT / 4; ++i) {
            const float4 kk = k4[i], qq = q4[i];
            if constexpr (CH) {
              // the output reads the state before this token enters it, plus the bonus on the token's own product
              const float4 ww = reinterpret_cast<const float4*>(&s_w[tt][NPT * r])[i];
              const float p0 = bv * kk.x, p1 = bv * kk.y, p2 = bv * kk.z, p3 = bv * kk.w;
              part[tt] = fmaf(fmaf(U[4 * i], p0, S[4 * i]), qq.x, part[tt]);
              part[tt] = fmaf(fmaf(U[4 * i + 1], p1, S[4 * i + 1]), qq.y, part[tt]);
              part[tt] = fmaf(fmaf(U[4 * i + 2], p2, S[4 * i + 2]), qq.z, part[tt]);
              part[tt] = fmaf(fmaf(U[4 * i + 3], p3, S[4 * i + 3]), qq.w, part[tt]);
              S[4 * i] = fmaf(ww.x, S[4 * i], p0);
              S[4 * i + 1] = fmaf(ww.y, S[4 * i + 1], p1);
              S[4 * i + 2] = fmaf(ww.z, S[4 * i + 2], p2);
              S[4 * i + 3] = fmaf(ww.w, S[4 * i + 3], p3);
              continue;
            }
            S[4 * i] = fmaf(a, S[4 * i], bv * kk.x);
            S[4 * i + 1] = fmaf(a, S[4 * i + 1], bv * kk.y);
            S[4 * i + 2] = fmaf(a, S[4 * i + 2], bv * kk.z);
            S[4 * i + 3] = fmaf(a, S[4 * i + 3], bv * kk.w);
            part[tt] = fmaf(S[4 * i], qq.x, part[tt]);
            part[tt] = fmaf(S[4 * i + 1], qq.y, part[tt]);
            part[tt] = fmaf(S[4 * i + 2], qq.z, part[tt]);
            part[tt] = fmaf(S[4 * i + 3], qq.w, part[tt]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < NPT; ++i) {
            if constexpr (CH) {
              const float p = bv * s_k[tt][r + R * i];
              part[tt] = fmaf(fmaf(U[i], p, S[i]), s_q[tt][r + R * i], part[tt]);
              S[i] = fmaf(s_w[tt][r + R * i], S[i], p);
              continue;
            }
            S[i] = fmaf(a, S[i], bv * s_k[tt][r + R * i]);
            part[tt] = fmaf(S[i], s_q[tt][r + R * i], part[tt]);
          }
        }
      }
    }
#pragma unroll
    for (int tt = 0; tt < SCAN_TILE; ++tt) {
      if (tt < nt) {
        float p = part[tt];
#pragma unroll
        for (int o = 1; o < R; o <<= 1) p += __shfl_xor_sync(0xffffffffu, p, o);
        if (r == 0 && live) out[(size_t)(t0 + tt) * ldo + (size_t)h * dv + col] = p + skip_h * s_v[tt][c];
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i)
      if (row_of(i) < dk) st[row_of(i)] = S[i];
  }
}

template <typename T, bool CH = false>
static int scan_launch(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const void* dt_raw, int lddt,
                       const float* dt_bias, const float* rate, const float* skip, int mode, int act, const int* cu_seqlens,
                       const int* seq_slots, int num_seqs, float* state, long long state_stride, float* out, int ldo, int H,
                        int hpg, int dk, int dv, int wide, cudaStream_t stream, const float* wlog = nullptr, int ldw = 0,
                       const float* bonus = nullptr) {
#define SCAN_GO(NPT, R, COLS)                                                                                                      \
  rl_launch_pdl(linear_scan_kernel<T, NPT, R, COLS, (NPT > 8 || (CH && NPT * R > 128) ? 8 : 16), CH>, dim3(num_seqs, H, (dv + COLS - 1) / COLS), R * COLS, 0, stream, (const T*)q, ldq, \
                (const T*)k, ldk, (const T*)v, ldv, (const T*)dt_raw, lddt, dt_bias, rate, skip, mode, act, cu_seqlens, seq_slots,      \
                state, state_stride, out, ldo, H, hpg, dk, dv, wlog, ldw, bonus)
  // tokens a tile: 8 in the shape for single-token steps (64 registers a thread and half the shared memory: 35.7
  // against 39.7 us at 64 sequences), 16 in long steps (8: 759 against 575 us, a barrier pair every 8 tokens)
  // columns of the state a block: 16 in single-token steps (fewer, larger blocks: 0.52 against 0.43 of the copy
  // bandwidth at 64 sequences), 8 in long steps (two blocks an SM whose phases overlap: 575 against 655 us for
  // 2,048 tokens of 16 heads of 128 x 128)
  if (!wide) {                      // few tokens a sequence: the state's traffic is the work; 8 lanes a column
    if (dk <= 128) SCAN_GO(16, 8, 16);
    else SCAN_GO(32, 8, 16);
  } else if (dk <= 64) {
    if constexpr (CH) SCAN_GO(2, 32, 16);
    else SCAN_GO(4, 16, 8);
  }
  else if (dk <= 128) SCAN_GO(4, 32, 8);
  else SCAN_GO(8, 32, 8);
#undef SCAN_GO
  return 0;
}

// q, k: [M, ld] with group g at columns [g * dk, (g + 1) * dk); v: [M, ldv] with head h at [h * dv, (h + 1) * dv);
// dt_raw [M, lddt] (mode 1; same dtype); dt_bias, rate, skip: float [H] (skip may be null; rate is the decay itself
// in mode 0 and the logarithm of the decay rate in mode 1).  state: float, this recurrence's [H, dv, dk] of slot s
// at state + s * state_stride.  out: float [M, ldo].  wide != 0: the launch shape for many tokens a sequence (more
// lanes a column of the state); 0: for few (single-token steps).  The two differ in the order of a dot product's sum.
extern "C" int rl_linear_scan(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const void* dt_raw,
                              int lddt, int dtype, const float* dt_bias, const float* rate, const float* skip, int mode, int act,
                              const int* cu_seqlens, const int* seq_slots, int num_seqs, float* state, long long state_stride,
                              float* out, int ldo, int num_heads, int heads_per_group, int dk, int dv, int wide,
                              cudaStream_t stream) {
  RL_REQUIRE(num_seqs >= 0 && num_heads > 0 && heads_per_group > 0 && num_heads % heads_per_group == 0, "rl_linear_scan: bad sizes");
  RL_REQUIRE(dk > 0 && dk <= SCAN_MAX_DK && dv > 0, "rl_linear_scan: dk %d outside (0, %d] or dv %d", dk, SCAN_MAX_DK, dv);
  RL_REQUIRE(mode == 0 || (mode == 1 && dt_raw != nullptr && dt_bias != nullptr), "rl_linear_scan: mode %d, or no step sizes", mode);
  RL_REQUIRE(rate != nullptr && state != nullptr, "rl_linear_scan: no decay or no state");
  RL_REQUIRE(num_heads <= 65535, "rl_linear_scan: more than 65,535 heads");
  if (num_seqs == 0) return RL_OK;
  if (dtype == RL_F32)
    scan_launch<float>(q, ldq, k, ldk, v, ldv, dt_raw, lddt, dt_bias, rate, skip, mode, act, cu_seqlens, seq_slots, num_seqs, state,
                       state_stride, out, ldo, num_heads, heads_per_group, dk, dv, wide, stream);
  else if (dtype == RL_BF16)
    scan_launch<__nv_bfloat16>(q, ldq, k, ldk, v, ldv, dt_raw, lddt, dt_bias, rate, skip, mode, act, cu_seqlens, seq_slots, num_seqs,
                               state, state_stride, out, ldo, num_heads, heads_per_group, dk, dv, wide, stream);
  else
    RL_REQUIRE(false, "rl_linear_scan: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_linear_scan");
  return RL_OK;
}

// The recurrence with a decay a key channel and a bonus for the current token (mode 2 above).  q, k [M, ld] with
// head h at columns [h * dk, (h + 1) * dk); v [M, ldv] with head h at [h * dv, (h + 1) * dv); wlog float [M, ldw]
// with head h at [h * dk, (h + 1) * dk): the decay of key channel n at token t is exp(-exp(wlog[t, h * dk + n]));
// bonus float [H, dk].  State, output and `wide` as in rl_linear_scan.
extern "C" int rl_channel_decay_scan(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, int dtype,
                                     const float* wlog, int ldw, const float* bonus, const int* cu_seqlens, const int* seq_slots,
                                     int num_seqs, float* state, long long state_stride, float* out, int ldo, int num_heads, int dk,
                                     int dv, int wide, cudaStream_t stream) {
  RL_REQUIRE(num_seqs >= 0 && num_heads > 0 && num_heads <= 65535, "rl_channel_decay_scan: bad sizes");
  RL_REQUIRE(dk > 0 && dk <= SCAN_MAX_DK && dv > 0, "rl_channel_decay_scan: dk %d outside (0, %d] or dv %d", dk, SCAN_MAX_DK, dv);
  RL_REQUIRE(wlog != nullptr && bonus != nullptr && state != nullptr && ldw >= num_heads * dk, "rl_channel_decay_scan: no decays, bonus or state");
  if (num_seqs == 0) return RL_OK;
  if (dtype == RL_F32)
    scan_launch<float, true>(q, ldq, k, ldk, v, ldv, nullptr, 0, nullptr, nullptr, nullptr, 0, 0, cu_seqlens, seq_slots, num_seqs, state,
                             state_stride, out, ldo, num_heads, 1, dk, dv, wide, stream, wlog, ldw, bonus);
  else if (dtype == RL_BF16)
    scan_launch<__nv_bfloat16, true>(q, ldq, k, ldk, v, ldv, nullptr, 0, nullptr, nullptr, nullptr, 0, 0, cu_seqlens, seq_slots, num_seqs,
                                     state, state_stride, out, ldo, num_heads, 1, dk, dv, wide, stream, wlog, ldw, bonus);
  else
    RL_REQUIRE(false, "rl_channel_decay_scan: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK("rl_channel_decay_scan");
  return RL_OK;
}
