// Attention of many query heads over ONE cached row a position whose front part is also the value
// (attention through a latent: the row is [latent | rotary key part], the value is the latent), on
// the tensor cores, for prompt portions and single tokens alike.
//
//   s_ij = (q_i . row_j) * scale over all DK elements,  j <= i,  i - j < window (if window > 0)
//   o_i  = sigmoid(gate_i) * sum_j softmax_j(s_ij) row_j[0 .. DV)        (gate: one number a token and head)
//
// The rows of a tile are (token, head) pairs of one sequence: HG = min(H, 16) heads of TOK = 16 / HG
// consecutive tokens (more than 16 heads: groups of 16 along grid y).  All of them read the same keys,
// so a block of 64 keys (one page) is brought into shared memory once a tile and serves both products:
//   1. warp w: S[16 x 16] = Q[16 x DK] . K[16w .. 16w + 16)^T   (mma.sync m16n8k16, Q and K by ldmatrix)
//      scaled into the exp2 domain, masked, to shared memory
//   2. warp w: rows 4w .. 4w + 3: running maximum and sum, P = exp2(S - max) as bf16 to shared memory
//   3. warp w: O[16 x its quarter of DV] = O * corr + P[16 x 64] . K[64 x its columns]  (values by
//      ldmatrix.trans from the same key block)
// A block of the prompt form holds MT = 2 such tiles (consecutive tokens), four warps each, over the same key
// blocks (half the key traffic a token, twice the warps a multiprocessor) where shared memory has room for both.
// Key blocks are double-buffered with cp.async.  What a row sums, and in which order, depends on its
// position, the window and the page borders alone - not on the batch or on how a prompt was cut.
#include <math.h>
#include <stdint.h>

#include "common.cuh"

#define SK_WARPS 4
#define SK_ROWS 16
#define SK_KEYS RL_PAGE      // keys a block: one page

__device__ __forceinline__ void sk_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void sk_cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void sk_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void sk_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void sk_ldm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void sk_ldm4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Shared memory: MT query tiles [16][DK + 8] bf16, two key blocks [64][DK + 8] bf16 (8 elements of padding
// make a row an odd number of 16-byte pieces: ldmatrix without bank conflicts), the scores [16][64 + 4]
// float, the weights [16][64 + 8] bf16, and a row's correction factor [16], each once a tile.
struct SkLayout {
  int ldk;              // elements from row to row of the query tile and the key blocks
  uint32_t q_off, k_off, s_off, p_off, c_off, bytes;
};
__host__ __device__ inline SkLayout sk_layout(int DK, int MT) {
  SkLayout L;
  L.ldk = DK + 8;
  L.q_off = 0;
  L.k_off = L.q_off + MT * SK_ROWS * L.ldk * 2;
  L.s_off = L.k_off + 2 * SK_KEYS * L.ldk * 2;
  L.p_off = L.s_off + MT * SK_ROWS * (SK_KEYS + 4) * 4;
  L.c_off = L.p_off + MT * SK_ROWS * (SK_KEYS + 8) * 2;
  L.bytes = L.c_off + MT * SK_ROWS * 4;
  return L;
}
// tiles a block of the prompt form: two where both fit shared memory
static inline int sk_prompt_tiles(int DK) { return sk_layout(DK, 2).bytes <= 227u * 1024u ? 2 : 1; }

// NTW: output n-tiles (8 columns each) a warp owns; 4 * NTW * 8 >= DV.  MT: tiles a block (SK_WARPS warps each).
template <int NTW, int MT>
__global__ void __launch_bounds__(MT * SK_WARPS * 32)
attention_shared_key_kernel(const __nv_bfloat16* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ k_pool,
                            const int* __restrict__ page_table, int max_pages, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ seq_slots, const int* __restrict__ kv_lens, int num_seqs,
                            int one_token_each, __nv_bfloat16* __restrict__ out, int ldo,
                            const __nv_bfloat16* __restrict__ gate, int ldg, int H, int DK, int DV, float scale_log2e,
                            int window, int splits, float* __restrict__ part, int head_tiles) {
  extern __shared__ __align__(128) uint8_t sk_smem[];
  __shared__ int s_where[2];
  const SkLayout L = sk_layout(DK, MT);
  const int ldk = L.ldk;
  const int mt = MT > 1 ? (int)(threadIdx.x >> 5) / SK_WARPS : 0;      // this warp's tile
  const int warp = (threadIdx.x >> 5) % SK_WARPS, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int HG = H < 16 ? H : 16;              // heads a tile
  const int TOK = SK_ROWS / HG;                // tokens a tile
  // ---- which sequence, which tile of its tokens ----
  if (one_token_each) {
    if (threadIdx.x == 0) { s_where[0] = blockIdx.x; s_where[1] = 0; }
  } else if (threadIdx.x == 0) {
    int x = blockIdx.x, b = 0;
    for (; b < num_seqs; ++b) {
      const int n = (cu_seqlens[b + 1] - cu_seqlens[b] + MT * TOK - 1) / (MT * TOK);
      if (x < n) break;
      x -= n;
    }
    s_where[0] = b; s_where[1] = x;
  }
  __syncthreads();
  const int b = s_where[0];
  if (b >= num_seqs) return;                   // the grid is sized exactly; defensive
  const int row0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - row0, kv_len = kv_lens[b];
  const int start_pos = kv_len - q_len;
  // a block's tiles lie along the tokens (prompts) or, with head_tiles, along the head groups of the same tokens
  const int tok_tiles = head_tiles ? 1 : MT;
  const int blk_tok0 = s_where[1] * tok_tiles * TOK;                  // the block's first token
  const int blk_toks = min(tok_tiles * TOK, q_len - blk_tok0);
  const int tok0 = blk_tok0 + (head_tiles ? 0 : mt) * TOK;             // this tile's
  const int toks_here = max(0, min(TOK, q_len - tok0));
  const int head0 = (head_tiles ? (int)blockIdx.y * MT + mt : (int)blockIdx.y) * 16;
  const int* pages = page_table + (size_t)seq_slots[b] * max_pages;
  const uint32_t smem = (uint32_t)__cvta_generic_to_shared(sk_smem);
  float* s_s = reinterpret_cast<float*>(sk_smem + L.s_off) + mt * SK_ROWS * (SK_KEYS + 4);
  __nv_bfloat16* s_p = reinterpret_cast<__nv_bfloat16*>(sk_smem + L.p_off) + mt * SK_ROWS * (SK_KEYS + 8);
  float* s_c = reinterpret_cast<float*>(sk_smem + L.c_off) + mt * SK_ROWS;
  const uint32_t q_tile = L.q_off + (uint32_t)(mt * SK_ROWS * ldk * 2);
  const uint32_t p_tile = L.p_off + (uint32_t)(mt * SK_ROWS * (SK_KEYS + 8) * 2);

  // the key blocks any row of the block sees (a tile whose rows see none of a block adds zeros there)
  const int pos_first = start_pos + tok0;
  const int blk_first = start_pos + blk_tok0, blk_last = blk_first + blk_toks - 1;
  const int first_key = window > 0 ? max(0, blk_first + 1 - window) : 0;
  int kb_begin = first_key / SK_KEYS, kb_end = blk_last / SK_KEYS + 1;
  // single tokens with few sequences: the key blocks of a sequence in `splits` runs along grid z, each run's
  // unnormalised sums, maximum and denominator to `part` (float [16][DV + 2] a block) for the combining kernel
  float* my_part = nullptr;
  if (splits > 1) {
    if (head0 < H)                             // (a tile behind the last head group has no rows and no place)
      my_part = part + (((size_t)blockIdx.x * ((H + 15) / 16) + head0 / 16) * splits + blockIdx.z) * SK_ROWS * (DV + 2);
    const int per = (kb_end - kb_begin + splits - 1) / splits;
    kb_begin += (int)blockIdx.z * per;
    kb_end = min(kb_end, kb_begin + per);
    if (kb_begin >= kb_end) {                  // nothing left for this run: it counts as weight zero
      if (my_part != nullptr && warp == 0 && lane < SK_ROWS) { my_part[lane * (DV + 2) + DV] = -INFINITY; my_part[lane * (DV + 2) + DV + 1] = 0.f; }
      return;
    }
  }
  const int pieces_row = DK >> 3;              // 16-byte pieces a row

  // ---- the query tile: row r = (token r / HG, head head0 + r % HG); rows without a token or head are zero ----
  for (int i = threadIdx.x; i < MT * SK_ROWS * pieces_row; i += MT * SK_WARPS * 32) {
    const int r = i / pieces_row, ch = i % pieces_row;               // rows of all tiles: tile r / 16
    const int rl = r % SK_ROWS, tile = r / SK_ROWS;
    const int tok = (head_tiles ? 0 : tile * TOK) + rl / HG;
    const int head = (head_tiles ? (int)blockIdx.y * MT + tile : (int)blockIdx.y) * 16 + rl % HG;
    const uint32_t dst = smem + L.q_off + (uint32_t)(r * ldk * 2 + ch * 16);
    if (rl / HG < TOK && tok < blk_toks && head < H) sk_cp16(dst, q + (size_t)(row0 + blk_tok0 + tok) * ldq + (size_t)head * DK + ch * 8);
    else *reinterpret_cast<uint4*>(sk_smem + L.q_off + r * ldk * 2 + ch * 16) = make_uint4(0u, 0u, 0u, 0u);
  }
  auto issue = [&](int kb, int buf) {
    const __nv_bfloat16* src = k_pool + (size_t)pages[kb] * SK_KEYS * DK;
    const uint32_t dst = smem + L.k_off + (uint32_t)(buf * SK_KEYS * ldk * 2);
    for (int i = threadIdx.x; i < SK_KEYS * pieces_row; i += MT * SK_WARPS * 32) {
      const int row = i / pieces_row, ch = i % pieces_row;
      sk_cp16(dst + (uint32_t)(row * ldk * 2 + ch * 16), src + (size_t)i * 8);
    }
  };
  issue(kb_begin, 0);
  sk_commit();

  float acc[NTW][4];
#pragma unroll
  for (int j = 0; j < NTW; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  // softmax state of row 4 * warp + lane / 8 (the same in its 8 lanes)
  float m_run = -INFINITY, l_run = 0.f;
  const int r8 = lane & 7, mat = lane >> 3;
  // this lane's two rows of the score and output fragments
  const int tok_lo = g / HG, tok_hi = (g + 8) / HG;
  const bool valid_lo = tok_lo < toks_here && head0 + g % HG < H, valid_hi = tok_hi < toks_here && head0 + (g + 8) % HG < H;
  const int pos_lo = pos_first + tok_lo, pos_hi = pos_first + tok_hi;
  const int nt_total = DV >> 3;

  for (int kb = kb_begin; kb < kb_end; ++kb) {
    const int buf = (kb - kb_begin) & 1;
    sk_wait<0>();
    __syncthreads();                           // block kb (and the queries) have landed; everyone is done with block kb - 1
    if (kb + 1 < kb_end) { issue(kb + 1, buf ^ 1); sk_commit(); }
    const uint32_t kbase = smem + L.k_off + (uint32_t)(buf * SK_KEYS * ldk * 2);
    // ---- 1. scores of this warp's 16 keys ----
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const uint32_t qa = smem + q_tile + (uint32_t)(((r8 + 8 * (mat & 1)) * ldk + 8 * (mat >> 1)) * 2);
      const uint32_t ka = kbase + (uint32_t)(((16 * warp + r8 + 8 * (mat >> 1)) * ldk + 8 * (mat & 1)) * 2);
      for (int ks = 0; ks < DK; ks += 16) {
        uint32_t a[4], bb[4];
        sk_ldm4(a, qa + ks * 2);
        sk_ldm4(bb, ka + ks * 2);
        sk_mma(s[0], a[0], a[1], a[2], a[3], bb[0], bb[1]);
        sk_mma(s[1], a[0], a[1], a[2], a[3], bb[2], bb[3]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int col = 16 * warp + 8 * nt + 2 * t;
      const int key = kb * SK_KEYS + col;
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int k = key + (e & 1), pos = e < 2 ? pos_lo : pos_hi;
        const bool ok = (e < 2 ? valid_lo : valid_hi) && k <= pos && (window <= 0 || k > pos - window);
        v[e] = ok ? s[nt][e] * scale_log2e : -INFINITY;
      }
      *reinterpret_cast<float2*>(&s_s[g * (SK_KEYS + 4) + col]) = make_float2(v[0], v[1]);
      *reinterpret_cast<float2*>(&s_s[(g + 8) * (SK_KEYS + 4) + col]) = make_float2(v[2], v[3]);
    }
    __syncthreads();
    // ---- 2. rows 4 * warp .. + 3: eight lanes a row, eight scores a lane ----
    {
      const int row = 4 * warp + (lane >> 3), sub = lane & 7;
      const float4 x0 = *reinterpret_cast<const float4*>(&s_s[row * (SK_KEYS + 4) + 8 * sub]);
      const float4 x1 = *reinterpret_cast<const float4*>(&s_s[row * (SK_KEYS + 4) + 8 * sub + 4]);
      float mx = fmaxf(fmaxf(fmaxf(x0.x, x0.y), fmaxf(x0.z, x0.w)), fmaxf(fmaxf(x1.x, x1.y), fmaxf(x1.z, x1.w)));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      const float m_new = fmaxf(m_run, mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;        // a row that has seen nothing yet
      const float corr = exp2f(m_run - m_use);
      const float p0 = exp2f(x0.x - m_use), p1 = exp2f(x0.y - m_use), p2 = exp2f(x0.z - m_use), p3 = exp2f(x0.w - m_use);
      const float p4 = exp2f(x1.x - m_use), p5 = exp2f(x1.y - m_use), p6 = exp2f(x1.z - m_use), p7 = exp2f(x1.w - m_use);
      float sum = ((p0 + p1) + (p2 + p3)) + ((p4 + p5) + (p6 + p7));
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      l_run = l_run * corr + sum;
      m_run = m_new;
      __nv_bfloat162 h0 = __floats2bfloat162_rn(p0, p1), h1 = __floats2bfloat162_rn(p2, p3);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(p4, p5), h3 = __floats2bfloat162_rn(p6, p7);
      uint4 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
      pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
      *reinterpret_cast<uint4*>(&s_p[row * (SK_KEYS + 8) + 8 * sub]) = pk;
      if (sub == 0) s_c[row] = corr;
    }
    __syncthreads();
    // ---- 3. this warp's columns of the output ----
    {
      const float c_lo = s_c[g], c_hi = s_c[g + 8];
#pragma unroll
      for (int j = 0; j < NTW; ++j) { acc[j][0] *= c_lo; acc[j][1] *= c_lo; acc[j][2] *= c_hi; acc[j][3] *= c_hi; }
      const uint32_t pa = smem + p_tile + (uint32_t)(((r8 + 8 * (mat & 1)) * (SK_KEYS + 8) + 8 * (mat >> 1)) * 2);
#pragma unroll
      for (int kk = 0; kk < SK_KEYS / 16; ++kk) {
        uint32_t a[4];
        sk_ldm4(a, pa + kk * 32);
        const uint32_t va = kbase + (uint32_t)(((16 * kk + r8 + 8 * (mat & 1)) * ldk + 8 * (mat >> 1)) * 2);
#pragma unroll
        for (int jp = 0; jp < NTW / 2; ++jp) {
          const int nt = warp * NTW + 2 * jp;
          if (nt < nt_total) {                 // warp-uniform
            uint32_t bb[4];
            sk_ldm4_trans(bb, va + nt * 16);
            sk_mma(acc[2 * jp], a[0], a[1], a[2], a[3], bb[0], bb[1]);
            sk_mma(acc[2 * jp + 1], a[0], a[1], a[2], a[3], bb[2], bb[3]);
          }
        }
      }
    }
  }
  if (splits > 1) {
    if (my_part == nullptr) return;
    if ((lane & 7) == 0) {
      float* pr = my_part + (4 * warp + (lane >> 3)) * (DV + 2) + DV;
      pr[0] = m_run; pr[1] = l_run;
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (!(half ? valid_hi : valid_lo)) continue;
      float* pr = my_part + (g + 8 * half) * (DV + 2);
#pragma unroll
      for (int j = 0; j < NTW; ++j) {
        const int nt = warp * NTW + j;
        if (nt < nt_total) *reinterpret_cast<float2*>(pr + 8 * nt + 2 * t) = make_float2(acc[j][2 * half], acc[j][2 * half + 1]);
      }
    }
    return;
  }
  // ---- the rows' sums to everyone; normalise, gate, store ----
  __syncthreads();
  if ((lane & 7) == 0) s_c[4 * warp + (lane >> 3)] = l_run;
  __syncthreads();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = g + 8 * half;
    if (!(half ? valid_hi : valid_lo)) continue;
    const int tok = r / HG, head = head0 + r % HG;
    const size_t m = (size_t)(row0 + tok0 + tok);
    const float l = s_c[r];
    float f = l > 0.f ? 1.0f / l : 0.f;
    if (gate) f *= 1.0f / (1.0f + expf(-__bfloat162float(gate[m * ldg + head])));
    __nv_bfloat16* orow = out + m * ldo + (size_t)head * DV;
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      const int nt = warp * NTW + j;
      if (nt < nt_total)
        *reinterpret_cast<__nv_bfloat162*>(orow + 8 * nt + 2 * t) = __floats2bfloat162_rn(acc[j][2 * half] * f, acc[j][2 * half + 1] * f);
    }
  }
}

// The runs of a sequence's single token joined: out = gate * sum_z w_z acc_z / sum_z w_z l_z with w_z = 2^(m_z - max m).
// grid (sequences, head groups, heads a group); always in the order of z, so a row's sum does not depend on timing.
__global__ void __launch_bounds__(128)
attention_shared_key_combine_kernel(const float* __restrict__ part, int splits, const int* __restrict__ cu_seqlens,
                                    __nv_bfloat16* __restrict__ out, int ldo, const __nv_bfloat16* __restrict__ gate, int ldg,
                                    int H, int DV) {
  const int r = blockIdx.z, head = blockIdx.y * 16 + r;
  if (head >= H) return;
  const float* base = part + ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * splits * SK_ROWS * (DV + 2) + (size_t)r * (DV + 2);
  const size_t run = (size_t)SK_ROWS * (DV + 2);
  float m = -INFINITY;
  for (int z = 0; z < splits; ++z) m = fmaxf(m, base[z * run + DV]);
  float w[8], l = 0.f;
#pragma unroll
  for (int z = 0; z < 8; ++z) {
    w[z] = (z < splits && m != -INFINITY) ? exp2f(base[z * run + DV] - m) : 0.f;
    if (z < splits) l += w[z] * base[z * run + DV + 1];
  }
  const size_t row = (size_t)cu_seqlens[blockIdx.x];
  float f = l > 0.f ? 1.0f / l : 0.f;
  if (gate) f *= 1.0f / (1.0f + expf(-__bfloat162float(gate[row * ldg + head])));
  for (int c = threadIdx.x; c < DV; c += 128) {
    float o = 0.f;
#pragma unroll
    for (int z = 0; z < 8; ++z)
      if (w[z] > 0.f) o += w[z] * base[z * run + c];
    out[row * ldo + (size_t)head * DV + c] = __float2bfloat16_rn(o * f);
  }
}

// Blocks along the heads (grid y) for this shape: a block takes 16 heads, or 32 as two tiles for single tokens.
extern "C" int rl_attention_shared_key_head_blocks(int num_heads, int key_dim, int one_token_each) {
  if (num_heads <= 0 || key_dim <= 0) return 0;
  const int groups = (num_heads + 15) / 16;
  return one_token_each && groups >= 2 && sk_prompt_tiles(key_dim) == 2 ? (groups + 1) / 2 : groups;
}

// 1 if the kernel takes this shape: rows of key_dim elements (a multiple of 16) whose first value_dim (a multiple of
// 8, at most 512) are the value, and a key block pair that fits shared memory.
extern "C" int rl_attention_shared_key_supported(int num_heads, int key_dim, int value_dim) {
  if (num_heads <= 0 || key_dim <= 0 || key_dim % 16 != 0 || value_dim <= 0 || value_dim % 8 != 0) return 0;
  if (value_dim > key_dim || value_dim > 512) return 0;
  return sk_layout(key_dim, 1).bytes <= 227u * 1024u ? 1 : 0;
}

// Tokens a block of the kernel takes: its tiles (one for single tokens, sk_prompt_tiles for prompts) times the
// tokens a tile.
extern "C" int rl_attention_shared_key_block_tokens(int num_heads, int key_dim, int one_token_each) {
  if (num_heads <= 0 || key_dim <= 0) return 0;
  const int per_tile = SK_ROWS / (num_heads < 16 ? num_heads : 16);
  return one_token_each ? per_tile : per_tile * sk_prompt_tiles(key_dim);
}

// q: [M, ldq] bf16, head h at columns [h * key_dim, (h + 1) * key_dim), the step's tokens packed by sequence
// (cu_seqlens: [B + 1] offsets; kv_lens[b]: the sequence's length after this step).  k_pool: [pages, 1, RL_PAGE,
// key_dim] bf16.  out: [M, ldo] bf16, head h at columns [h * value_dim, ...).  gate (may be null): bf16 [M, ldg], one
// number a head.  num_tiles = the blocks: sum over sequences of ceil(tokens / rl_attention_shared_key_block_tokens).  one_token_each != 0: every sequence brings one token (num_tiles = num_seqs).
// window > 0: a query at position i sees positions j with 0 <= i - j < window; 0: all j <= i.
// splits > 1 (single tokens only): a sequence's key blocks in that many runs, joined by a second kernel; part: float
// workspace of num_seqs * head groups * splits * 16 * (value_dim + 2).
extern "C" int rl_attention_shared_key(const void* q, int ldq, const void* k_pool, const int* page_table, int max_pages,
                                       const int* cu_seqlens, const int* seq_slots, const int* kv_lens, int num_seqs,
                                       int num_tiles, int one_token_each, void* out, int ldo, const void* gate, int ldg,
                                       int num_heads, int key_dim, int value_dim, float scale, int window,
                                       int splits, float* part, cudaStream_t stream) {
  RL_REQUIRE(rl_attention_shared_key_supported(num_heads, key_dim, value_dim),
             "rl_attention_shared_key: unsupported shape (heads %d, key rows of %d, values of %d): key rows must be a multiple "
             "of 16, values a multiple of 8 and at most 512", num_heads, key_dim, value_dim);
  RL_REQUIRE(num_seqs >= 0 && num_tiles >= 0 && window >= 0, "rl_attention_shared_key: bad sizes");
  RL_REQUIRE(ldq >= num_heads * key_dim && ldq % 8 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)k_pool & 15) == 0,
             "rl_attention_shared_key: q and the pool must be 16-byte aligned, q's row stride a multiple of 8 that holds all heads");
  RL_REQUIRE(ldo >= num_heads * value_dim && ldo % 2 == 0 && ((uintptr_t)out & 3) == 0,
             "rl_attention_shared_key: the output's row stride is too small or odd, or the output is misaligned");
  RL_REQUIRE(gate == nullptr || ldg >= num_heads, "rl_attention_shared_key: the gate's row stride is too small");
  RL_REQUIRE(!one_token_each || num_tiles == num_seqs, "rl_attention_shared_key: one token a sequence means a tile a sequence");
  RL_REQUIRE(splits >= 1 && splits <= 8 && (splits == 1 || (one_token_each && part != nullptr)),
             "rl_attention_shared_key: 1 to 8 runs a sequence, more than one only for single tokens and with a workspace");
  if (num_seqs == 0 || num_tiles == 0) return RL_OK;
  const int groups = (num_heads + 15) / 16;
  RL_REQUIRE(groups <= 65535, "rl_attention_shared_key: too many heads");
  // single tokens of more than 16 heads: the two tiles of a block are two head groups of the token
  const int head_tiles = one_token_each && groups >= 2 && sk_prompt_tiles(key_dim) == 2;
  const int MT = one_token_each && !head_tiles ? 1 : sk_prompt_tiles(key_dim);
  const SkLayout L = sk_layout(key_dim, MT);
  const dim3 grid(num_tiles, head_tiles ? (groups + 1) / 2 : groups, splits), block(MT * SK_WARPS * 32);
  const float sl2 = scale * 1.4426950408889634f;
#define RL_SK_LAUNCH(NTW)                                                                                                   \
  do {                                                                                                                      \
    if (MT == 2) RL_SK_LAUNCH_MT(NTW, 2);                                                                                   \
    else RL_SK_LAUNCH_MT(NTW, 1);                                                                                           \
  } while (0)
#define RL_SK_LAUNCH_MT(NTW, MTV)                                                                                           \
  do {                                                                                                                      \
    static int reserved = 0;                                                                                                \
    if ((int)L.bytes > reserved) {                                                                                          \
      cudaError_t e = cudaFuncSetAttribute(attention_shared_key_kernel<NTW, MTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)L.bytes);                                                                   \
      RL_REQUIRE(e == cudaSuccess, "rl_attention_shared_key: cannot reserve %u bytes of shared memory: %s", L.bytes,        \
                 cudaGetErrorString(e));                                                                                    \
      reserved = (int)L.bytes;                                                                                              \
    }                                                                                                                       \
    attention_shared_key_kernel<NTW, MTV><<<grid, block, L.bytes, stream>>>(                                                     \
        (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)k_pool, page_table, max_pages, cu_seqlens, seq_slots, kv_lens,  \
        num_seqs, one_token_each, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)gate, ldg, num_heads, key_dim, value_dim, \
        sl2, window, splits, part, head_tiles);                                                                             \
  } while (0)
  if (value_dim <= 64) RL_SK_LAUNCH(2);
  else if (value_dim <= 128) RL_SK_LAUNCH(4);
  else if (value_dim <= 256) RL_SK_LAUNCH(8);
  else RL_SK_LAUNCH(16);
#undef RL_SK_LAUNCH
#undef RL_SK_LAUNCH_MT
  if (splits > 1) {
    const int hg = num_heads < 16 ? num_heads : 16;
    attention_shared_key_combine_kernel<<<dim3(num_seqs, groups, hg), 128, 0, stream>>>(
        part, splits, cu_seqlens, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)gate, ldg, num_heads, value_dim);
  }
  RL_LAUNCH_CHECK("rl_attention_shared_key");
  return RL_OK;
}
