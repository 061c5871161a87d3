// The general attention (attention_general.cu) in bfloat16 on tensor cores, for prompts and for decode steps.
//
// A CTA of four warps owns one work item: up to RG groups of 16 query rows that share their keys (consecutive new
// tokens of a sequence x the heads of one key/value group, for one score map) and one contiguous range of that
// sequence's keys.  Keys are visited in tiles of 64 (one page); the groups go through every phase of a tile together
// and share its key and value fragments.  Per tile:
//   scores   warp w computes the 16 x 16 block of rows x keys 16w..16w+15: mma.sync.m16n8k16 over the key
//            dimension, Q fragments from shared memory, K fragments straight from the cache rows (a dot product
//            may visit the dimension in any order as long as Q and K agree: lane t of a row takes the 8
//            contiguous values 8t..8t+7 of every 32, as attention_mma.cu does);
//   softmax  scale, query factor, tanh cap and mask in float32; the row maximum of the tile goes through shared
//            memory; every warp rescales by the same running maximum and keeps the sum of its own keys;
//   values   the probabilities are float32; the tensor core takes bfloat16, so each is split into a high and a low
//            bfloat16 part (p = hi + lo to 16 bits of mantissa) that go through shared memory, and warp w adds
//            hi V + lo V for the chunks of 32 value dimensions c = w, w + 4, ...  (V fragments straight from the
//            cache rows, transposed by movmatrix as in attention_mma.cu).
// Keys and values come from the paged cache, or (`dense`) from two plain matrices that hold, from row seq_start[s]
// on, the keys and values of sequence s by position (a mixer that forms its heads' keys and values for a whole
// prompt; the matrices have 64 readable rows beyond the last sequence's).
// With one key range and one map the normalised result is written directly.  Otherwise every item leaves its
// unnormalised value sum, its maximum and its denominator in scratch, and the finishing kernel merges the
// ranges in order and combines the maps (see attention_general.cu for the formulas).
#include <math.h>

#include "attention_general.h"
#include "common.cuh"
#include "mma_common.cuh"

#define GM_WARPS 4
#define GM_TILE 64
#define GM_PSTRIDE 72          // bf16 per row of the probability tiles: 64 keys + 8 of padding (no bank conflicts)

// this kernel is launched the ordinary way: it starts when the kernels before it have ended, so plain loads (which
// may be served by L1) see what they wrote
__device__ __forceinline__ uint4 gm_ldg16(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// the same instruction as mma16816, left to the compiler to schedule among its neighbours (its only effect is its result)
__device__ __forceinline__ void gm_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// A 16 x 16 block of bfloat16 from shared memory as the A operand of m16n8k16: lane l gives the address of row
// l % 16, columns 8 (l / 16) .. + 7 of the block.
__device__ __forceinline__ void gm_ldmatrix4(uint32_t (&a)[4], const void* lane_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
               : "r"((uint32_t)__cvta_generic_to_shared(lane_row)) : "memory");
}

__host__ __device__ __forceinline__ int gm_q_stride(int D) {       // bytes per row of Q in shared memory: = 64 mod 128
  int s = ((D * 2 + 15) / 16) * 16;
  while (s % 128 != 64) s += 16;
  return s;
}

template <int CPW, int RG>
__global__ void __launch_bounds__(GM_WARPS * 32)
attention_general_mma_kernel(const GeneralAttention P) {
  extern __shared__ __align__(16) unsigned char gm_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int D = P.qk_dim, Dv = P.v_dim;
  const int qstride = gm_q_stride(D);
  unsigned char* q_s = gm_smem;                                                  // [RG][16][qstride bytes]
  bf16* p_hi = reinterpret_cast<bf16*>(gm_smem + RG * 16 * qstride);             // [RG][16][GM_PSTRIDE]
  bf16* p_lo = p_hi + RG * 16 * GM_PSTRIDE;
  float* max_s = reinterpret_cast<float*>(p_lo + RG * 16 * GM_PSTRIDE);          // [RG][GM_WARPS][16]
  float* sum_s = max_s + RG * GM_WARPS * 16;                                     // [GM_WARPS][16]

  const int rows_per_token = P.group < 16 ? P.group : 16;
  const int head_groups = (P.group + 15) / 16;
  const int n_kv = P.n_heads / P.group;
  int item = blockIdx.x;
  const int split = item % P.n_splits; item /= P.n_splits;
  const int map = item % P.maps; item /= P.maps;
  const int hg = item % head_groups; item /= head_groups;
  const int kv = item % n_kv; item /= n_kv;
  const int qb = item;
  const int seq = P.qb_seq ? P.qb_seq[qb] : P.token_seq[qb];
  if (seq < 0) return;                                                           // padding
  const int tok0 = P.qb_tok0 ? P.qb_tok0[qb] : qb;
  const int ntok = P.qb_ntok ? P.qb_ntok[qb] : 1;
  const int tpg = P.tokens_per_block;                                            // tokens of one group of 16 rows

  // the two rows of this lane in every group of 16 rows: r = g and g + 8;  row -> (token of the group, head)
  int row_tok[RG][2], row_head[2], row_pos[RG][2];
  bool row_ok[RG][2];
  float row_factor[RG][2];
#pragma unroll
  for (int e = 0; e < 2; e++) {
    const int r = g + 8 * e;
    const int tr = r / rows_per_token, hr = r % rows_per_token;
    const int hq = hg * 16 + hr;
    row_head[e] = kv * P.group + (hq < P.group ? hq : 0);
#pragma unroll
    for (int rg = 0; rg < RG; rg++) {
      const int tk = rg * tpg + tr;
      row_ok[rg][e] = tr < tpg && tk < ntok && hq < P.group;
      row_tok[rg][e] = tok0 + (row_ok[rg][e] ? tk : 0);
      row_pos[rg][e] = P.token_pos[row_tok[rg][e]];
      float temp = 1.f;
      if (P.temp_coef != 0.f) temp = 1.f + P.temp_coef * logf((float)((row_pos[rg][e] + 1) / P.temp_every) + 1.f);
      row_factor[rg][e] = P.scale * temp;
    }
  }
  const int first_pos = P.token_pos[tok0];
  const int last_pos = first_pos + ntok - 1;
  const int lo_block = (P.window > 0 && first_pos - P.window + 1 > 0) ? first_pos - P.window + 1 : 0;
  const int k_begin = split * P.chunk;
  const int k_end = min((split + 1) * P.chunk, last_pos + 1);
  // tiles wholly in front of the window of the block's first row hold nothing any row sees, unless they hold kept
  // first keys (positions below keep_first stay visible through a window)
  const int lo_tile = (lo_block / GM_TILE) * GM_TILE;
  const int keep = P.window > 0 ? P.keep_first : 0;
  const bool dense = P.dense != 0;
  const int* bt = dense ? nullptr : P.block_table + (size_t)seq * P.bt_stride;
  const size_t seq_row0 = dense ? (size_t)P.seq_start[seq] : 0;

  // Q rows of this item into shared memory (16 bytes per thread and turn; rows that do not exist are zero)
  {
    const int pieces = D / 8;
    for (int i = threadIdx.x; i < RG * 16 * pieces; i += blockDim.x) {
      const int r = i / pieces, c = i - r * pieces;
      const int rg = r / 16, rr = r % 16;
      const int tr = rr / rows_per_token, hr = rr % rows_per_token;
      const int hq = hg * 16 + hr, tk = rg * tpg + tr;
      const bool ok = tr < tpg && tk < ntok && hq < P.group;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (ok)
        v = ld_fresh((const uint4*)((const bf16*)P.q + (size_t)(tok0 + tk) * P.ldq +
                                    ((size_t)(kv * P.group + hq) * P.maps + map) * D + 8 * c));
      *reinterpret_cast<uint4*>(q_s + (size_t)r * qstride + 16 * c) = v;
    }
  }
  __syncthreads();

  const size_t k_page = (size_t)P.n_k_heads * P.page_tokens * D;
  const size_t k_head = (size_t)(kv * P.maps + map) * P.page_tokens * D;
  const bf16* v_base = P.v_in_k ? (const bf16*)P.k_cache : (const bf16*)P.v_cache;
  const int v_row = dense ? P.ldv : (P.v_in_k ? D : Dv);
  const int k_row = dense ? P.ldk : D;
  const size_t v_page = P.v_in_k ? k_page : (size_t)P.n_v_heads * P.page_tokens * Dv;
  const size_t v_head = P.v_in_k ? (size_t)(kv * P.maps) * P.page_tokens * D : (size_t)kv * P.page_tokens * Dv;
  const int n_kc = (D + 31) / 32;                 // chunks of the key dimension
  const int n_vc = (Dv + 31) / 32;                // chunks of the value dimension

  float o[RG][CPW * 4][4];
  float m_run[RG][2], l_run[RG][2];
#pragma unroll
  for (int rg = 0; rg < RG; rg++) {
#pragma unroll
    for (int i = 0; i < CPW * 4; i++) { o[rg][i][0] = o[rg][i][1] = o[rg][i][2] = o[rg][i][3] = 0.f; }
    m_run[rg][0] = m_run[rg][1] = -INFINITY;
    l_run[rg][0] = l_run[rg][1] = 0.f;
  }
  const uint4 zero4 = make_uint4(0, 0, 0, 0);

  for (int key0 = (k_begin / GM_TILE) * GM_TILE; key0 < k_end; key0 += GM_TILE) {
    if (key0 < lo_tile && key0 >= keep) {          // on to the window's first tile (the same for every thread)
      key0 = lo_tile - GM_TILE;
      continue;
    }
    const int kw = key0 + 16 * warp;
    const bf16* kr;
    const bf16* vr;
    if (dense) {                                   // key j of the sequence is row seq_row0 + j of the matrices
      kr = (const bf16*)P.k_cache + (seq_row0 + kw) * k_row + (size_t)(kv * P.maps + map) * D;
      vr = (const bf16*)P.v_cache + (seq_row0 + key0) * v_row + (size_t)kv * Dv;
    } else {
      const int page = bt[key0 / P.page_tokens];
      const int in_page = key0 % P.page_tokens;
      kr = (const bf16*)P.k_cache + (size_t)page * k_page + k_head + (size_t)(in_page + 16 * warp) * D;
      vr = v_base + (size_t)page * v_page + v_head + (size_t)in_page * v_row;
    }
    // ---- scores of keys key0 + 16 warp + [0, 16), for every group of rows: the key fragments are loaded once
    float s[RG][2][4];
#pragma unroll
    for (int rg = 0; rg < RG; rg++)
#pragma unroll
      for (int i = 0; i < 2; i++) { s[rg][i][0] = s[rg][i][1] = s[rg][i][2] = s[rg][i][3] = 0.f; }
    const bool any = kw < k_end && kw + 15 >= k_begin;
    if (any) {
      for (int c0 = 0; c0 < n_kc; c0 += 4) {            // four chunks' loads in flight together
        uint4 ka[4], kb[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int d = 32 * (c0 + u) + 8 * t;
          const bool d_ok = d < D;
          ka[u] = d_ok ? gm_ldg16(kr + (size_t)g * k_row + d) : zero4;
          kb[u] = d_ok ? gm_ldg16(kr + (size_t)(g + 8) * k_row + d) : zero4;
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int d = 32 * (c0 + u) + 8 * t;
          if (32 * (c0 + u) >= D) break;
          const bool d_ok = d < D;
#pragma unroll
          for (int rg = 0; rg < RG; rg++) {
            const unsigned char* qg = q_s + (size_t)rg * 16 * qstride;
            const uint4 qa = d_ok ? *reinterpret_cast<const uint4*>(qg + (size_t)g * qstride + 2 * d) : zero4;
            const uint4 qc = d_ok ? *reinterpret_cast<const uint4*>(qg + (size_t)(g + 8) * qstride + 2 * d) : zero4;
            gm_mma(s[rg][0], qa.x, qc.x, qa.y, qc.y, ka[u].x, ka[u].y);
            gm_mma(s[rg][1], qa.x, qc.x, qa.y, qc.y, kb[u].x, kb[u].y);
            gm_mma(s[rg][0], qa.z, qc.z, qa.w, qc.w, ka[u].z, ka[u].w);
            gm_mma(s[rg][1], qa.z, qc.z, qa.w, qc.w, kb[u].z, kb[u].w);
          }
        }
      }
    }
    // a tile every row of the CTA sees whole (all of it at or before the first row's position, inside the item's
    // range, no window) needs no mask: rows that do not exist carry zeros and are never written
    const bool whole_tile = P.window == 0 && key0 + GM_TILE - 1 <= first_pos && key0 >= k_begin && key0 + GM_TILE <= k_end;
#pragma unroll
    for (int rg = 0; rg < RG; rg++) {
      float bm[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 2; i++) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int e = j >> 1;
          float v = s[rg][i][j] * row_factor[rg][e];
          if (P.softcap > 0.f) v = P.softcap * tanhf(v / P.softcap);
          if (!whole_tile) {
            const int key = kw + 8 * i + 2 * t + (j & 1);
            const int pos = row_pos[rg][e];
            const int lo = (P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
            const bool ok = any && row_ok[rg][e] && key <= pos && (key >= lo || key < keep) && key < k_end && key >= k_begin;
            v = ok ? v : -INFINITY;
          }
          s[rg][i][j] = v;
          bm[e] = fmaxf(bm[e], v);
        }
      }
#pragma unroll
      for (int e = 0; e < 2; e++) {
        bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 1));
        bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 2));
        if (t == 0) max_s[(rg * GM_WARPS + warp) * 16 + g + 8 * e] = bm[e];
      }
    }
    __syncthreads();
    float corr[RG][2];
#pragma unroll
    for (int rg = 0; rg < RG; rg++) {
      float m_use[2];
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int r = rg * GM_WARPS * 16 + g + 8 * e;
        const float tile_max = fmaxf(fmaxf(max_s[r], max_s[16 + r]), fmaxf(max_s[32 + r], max_s[48 + r]));
        const float m_new = fmaxf(m_run[rg][e], tile_max);
        m_use[e] = (m_new == -INFINITY) ? 0.f : m_new;      // a row with no key yet: exponents of -inf give 0
        corr[rg][e] = __expf(m_run[rg][e] - m_use[e]);      // first keys: exp(-inf) = 0
        m_run[rg][e] = m_new;
      }
      float psum[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 2; i++) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const float p0 = __expf(s[rg][i][2 * e] - m_use[e]), p1 = __expf(s[rg][i][2 * e + 1] - m_use[e]);
          psum[e] += p0 + p1;
          const __nv_bfloat162 hi = __floats2bfloat162_rn(p0, p1);
          const __nv_bfloat162 lo = __floats2bfloat162_rn(p0 - __bfloat162float(hi.x), p1 - __bfloat162float(hi.y));
          const int at = (rg * 16 + g + 8 * e) * GM_PSTRIDE + 16 * warp + 8 * i + 2 * t;
          *reinterpret_cast<__nv_bfloat162*>(p_hi + at) = hi;
          *reinterpret_cast<__nv_bfloat162*>(p_lo + at) = lo;
        }
      }
#pragma unroll
      for (int e = 0; e < 2; e++) l_run[rg][e] = l_run[rg][e] * corr[rg][e] + psum[e];
    }
    __syncthreads();
    // ---- values: chunks of 32 dimensions c = warp, warp + 4, ...; the value fragments are loaded and transposed
    // once for all groups of rows
#pragma unroll
    for (int rg = 0; rg < RG; rg++)
#pragma unroll
      for (int i = 0; i < CPW * 4; i++) {
        o[rg][i][0] *= corr[rg][0]; o[rg][i][1] *= corr[rg][0]; o[rg][i][2] *= corr[rg][1]; o[rg][i][3] *= corr[rg][1];
      }
    const int blocks = min(GM_TILE, k_end - key0 + 15) / 16;          // blocks of 16 keys that hold a key
#pragma unroll
    for (int cc = 0; cc < CPW; cc++) {
      const int c = warp + GM_WARPS * cc;
      const int d = 32 * c + 8 * t;
      if (c >= n_vc) break;
      // all of the tile's loads of this chunk first, so that their latencies overlap
      uint4 va[GM_TILE / 16], vb[GM_TILE / 16];
#pragma unroll
      for (int kb = 0; kb < GM_TILE / 16; kb++) {
        const bool ok = kb < blocks && d < Dv;
        va[kb] = ok ? gm_ldg16(vr + (size_t)(16 * kb + g) * v_row + d) : zero4;
        vb[kb] = ok ? gm_ldg16(vr + (size_t)(16 * kb + 8 + g) * v_row + d) : zero4;
      }
#pragma unroll
      for (int kb = 0; kb < GM_TILE / 16; kb++) {
        if (kb >= blocks) break;
        uint32_t b0[4], b1[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
          b0[i] = transpose8x8(reg_of(va[kb], i));
          b1[i] = transpose8x8(reg_of(vb[kb], i));
        }
#pragma unroll
        for (int rg = 0; rg < RG; rg++) {
          uint32_t hi[4], lo[4];
          const int a_at = (rg * 16 + (lane & 15)) * GM_PSTRIDE + 16 * kb + 8 * (lane >> 4);
          gm_ldmatrix4(hi, p_hi + a_at);
          gm_ldmatrix4(lo, p_lo + a_at);
#pragma unroll
          for (int i = 0; i < 4; i++) gm_mma(o[rg][4 * cc + i], hi[0], hi[1], hi[2], hi[3], b0[i], b1[i]);
#pragma unroll
          for (int i = 0; i < 4; i++) gm_mma(o[rg][4 * cc + i], lo[0], lo[1], lo[2], lo[3], b0[i], b1[i]);
        }
      }
    }
    __syncthreads();                               // the tiles of probabilities and the maxima are written again
  }

  const bool direct = P.n_splits == 1 && P.combine == 0;
#pragma unroll
  for (int rg = 0; rg < RG; rg++) {
    if (rg > 0 && rg * tpg >= ntok) break;
    // denominators: across the four lanes of a row, then across the warps
    float l_all[2];
#pragma unroll
    for (int e = 0; e < 2; e++) {
      float l = l_run[rg][e];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (t == 0) sum_s[warp * 16 + g + 8 * e] = l;
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const int r = g + 8 * e;
      l_all[e] = (sum_s[r] + sum_s[16 + r]) + (sum_s[32 + r] + sum_s[48 + r]);
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 2; e++) {
      if (!row_ok[rg][e]) continue;
      if (direct) {
        if (P.sink) l_all[e] += expf(P.sink[row_head[e]] - m_run[rg][e]);
        const float inv = 1.0f / l_all[e];
        bf16* op = (bf16*)P.out + (size_t)row_tok[rg][e] * P.ldo + (size_t)row_head[e] * Dv;
#pragma unroll
        for (int cc = 0; cc < CPW; cc++) {
          const int d = 32 * (warp + GM_WARPS * cc) + 8 * t;
          if (d >= Dv) continue;
          uint4 v;
          v.x = pack_bf16(o[rg][4 * cc + 0][2 * e] * inv, o[rg][4 * cc + 0][2 * e + 1] * inv);
          v.y = pack_bf16(o[rg][4 * cc + 1][2 * e] * inv, o[rg][4 * cc + 1][2 * e + 1] * inv);
          v.z = pack_bf16(o[rg][4 * cc + 2][2 * e] * inv, o[rg][4 * cc + 2][2 * e + 1] * inv);
          v.w = pack_bf16(o[rg][4 * cc + 3][2 * e] * inv, o[rg][4 * cc + 3][2 * e + 1] * inv);
          *reinterpret_cast<uint4*>(op + d) = v;
        }
      } else {
        const size_t slot = (((size_t)row_tok[rg][e] * P.n_heads + row_head[e]) * P.maps + map) * P.n_splits + split;
        float* po = P.part_o + slot * Dv;
#pragma unroll
        for (int cc = 0; cc < CPW; cc++) {
          const int d = 32 * (warp + GM_WARPS * cc) + 8 * t;
          if (d >= Dv) continue;
          *reinterpret_cast<float4*>(po + d) = make_float4(o[rg][4 * cc + 0][2 * e], o[rg][4 * cc + 0][2 * e + 1],
                                                           o[rg][4 * cc + 1][2 * e], o[rg][4 * cc + 1][2 * e + 1]);
          *reinterpret_cast<float4*>(po + d + 4) = make_float4(o[rg][4 * cc + 2][2 * e], o[rg][4 * cc + 2][2 * e + 1],
                                                               o[rg][4 * cc + 3][2 * e], o[rg][4 * cc + 3][2 * e + 1]);
        }
        if (warp == 0 && t == 0) {
          P.part_ml[slot * 2] = m_run[rg][e];
          P.part_ml[slot * 2 + 1] = l_all[e];
        }
      }
    }
  }
}

// Merge the key ranges of every (token, head, map) in range order, then combine the maps; one block per
// (token, head), one thread per value dimension.  A range that held no key of a row left maximum -inf and sum 0
// and drops out.
#define GM_MAX_SPLITS 64
template <int MAPS>
__global__ void __launch_bounds__(128) attention_general_finish_kernel(const GeneralAttention P) {
  __shared__ float weight[MAPS][GM_MAX_SPLITS];
  __shared__ float scratch[33];
  const int item = blockIdx.x;
  const int tok = item / P.n_heads, h = item - tok * P.n_heads;
  if (P.token_seq[tok] < 0) return;
  const int Dv = P.v_dim, S = P.n_splits;
  if (threadIdx.x < MAPS) {
    const int m = threadIdx.x;
    const float* ml = P.part_ml + ((size_t)item * MAPS + m) * S * 2;
    float mx = -INFINITY;
    for (int s = 0; s < S; s++) mx = fmaxf(mx, ml[2 * s]);
    float l = 0.f;
    for (int s = 0; s < S; s++) {
      const float w = ml[2 * s] == -INFINITY ? 0.f : expf(ml[2 * s] - mx);
      weight[m][s] = w;
      l += ml[2 * s + 1] * w;
    }
    if (P.sink) l += expf(P.sink[h] - mx);
    const float inv = 1.0f / l;
    for (int s = 0; s < S; s++) weight[m][s] *= inv;
  }
  __syncthreads();
  bf16* op = (bf16*)P.out + (size_t)tok * P.ldo + (size_t)h * Dv;
  float o[4], ss = 0.f;                              // v_dim <= 512: at most four dimensions per thread
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int d = threadIdx.x + 128 * i;
    o[i] = 0.f;
    if (d >= Dv) continue;
    float a[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      const float* po = P.part_o + ((size_t)item * MAPS + m) * S * Dv + d;
      float acc = 0.f;
#pragma unroll 4
      for (int s = 0; s < S; s++) acc = fmaf(po[(size_t)s * Dv], weight[m][s], acc);
      a[m] = acc;
    }
    if (MAPS == 1) {
      op[d] = __float2bfloat16_rn(a[0]);
    } else {
      o[i] = a[0] - P.lambda * a[MAPS - 1];
      ss = fmaf(o[i], o[i], ss);
    }
  }
  if (MAPS == 1) return;
  ss = block_sum(ss, scratch);
  float mul = P.out_scale / sqrtf(ss / (float)Dv + P.eps);
  if (P.gate_col >= 0) {
    const float z = ld_fresh((const bf16*)P.q + (size_t)tok * P.ldq + P.gate_col + h);
    mul *= 1.0f / (1.0f + expf(-z));
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int d = threadIdx.x + 128 * i;
    if (d < Dv) op[d] = __float2bfloat16_rn(o[i] * mul);
  }
}

STRATUM_EXPORT long long stratum_attention_general_mma_smem(int qk_dim, int row_groups) {
  return 16LL * row_groups * gm_q_stride(qk_dim) + 2LL * row_groups * 16 * GM_PSTRIDE * sizeof(bf16) +
         (row_groups + 1LL) * GM_WARPS * 16 * sizeof(float);
}

// Groups of 16 rows a CTA takes for a value size (prompts): what the host cuts its query blocks by.  Two groups share
// every key and value fragment (and its transposition) of a tile.  Measured on prompts of 2,048 tokens, four layers:
// values of 512 (keys of 576, four chunks of values a warp) 5.02 ms with two groups against 5.38 with one; values of
// 256 (keys of 288, two chunks a warp) 1.83 against 1.75; values of 64 to 128 (one chunk a warp: heads of ordinary
// sizes) 2.36 against 2.41 ms a prompt step and 4.94 against 5.31.  So: one group where a warp holds two chunks,
// else two.  STRATUM_GENERAL_ATTENTION_ROW_GROUPS=1|2 forces either (measurements).
STRATUM_EXPORT int stratum_attention_general_mma_row_groups(int v_dim) {
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("STRATUM_GENERAL_ATTENTION_ROW_GROUPS");
    forced = e ? atoi(e) : 0;
  }
  if (forced == 1 || forced == 2) return forced;
  const int cpw = ((v_dim + 31) / 32 + GM_WARPS - 1) / GM_WARPS;
  return cpw == 2 ? 1 : 2;
}

// q, the caches and out bfloat16.  `reserved` in the parameters: groups of 16 rows per query block (0 or 1: one;
// else what stratum_attention_general_mma_row_groups gives).  Needs qk_dim % 8 == 0, v_dim % 8 == 0 (v_dim % 32 == 0 when results go through
// scratch is not needed: rows of scratch are v_dim floats and v_dim % 8 == 0 keeps them 16-byte aligned), rows of
// q and out 16-byte aligned, pages of 64 tokens.
STRATUM_EXPORT int stratum_attention_general_mma(const GeneralAttention* params, cudaStream_t stream) {
  const GeneralAttention& P = *params;
  if (P.n_tokens <= 0 || P.n_qblocks <= 0) return 0;
  const int bad = general_attention_check(P);
  if (bad) return bad;
  if (P.dense && (P.v_in_k || !P.seq_start || P.ldk % 8 != 0 || P.ldv % 8 != 0 ||
                  P.ldk < P.n_k_heads * P.qk_dim || P.ldv < P.n_v_heads * P.v_dim))
    return STRATUM_ERR_SHAPE;
  if (P.qk_dim % 8 != 0 || P.v_dim % 8 != 0 || P.ldq % 8 != 0 || P.ldo % 8 != 0 || P.page_tokens != GM_TILE)
    return STRATUM_ERR_SHAPE;
  if ((((uintptr_t)P.q | (uintptr_t)P.out | (uintptr_t)P.k_cache | (uintptr_t)P.v_cache) & 15) != 0)
    return STRATUM_ERR_ALIGN;
  if (P.n_splits < 1 || P.n_splits > GM_MAX_SPLITS || P.v_dim > 512 || P.chunk < GM_TILE || P.chunk % GM_TILE != 0 || P.tokens_per_block < 1) return STRATUM_ERR_SHAPE;
  const bool direct = P.n_splits == 1 && P.combine == 0;
  if (!direct && (!P.part_o || !P.part_ml)) return STRATUM_ERR_SHAPE;
  const int n_vc = (P.v_dim + 31) / 32;
  const int cpw = (n_vc + GM_WARPS - 1) / GM_WARPS;
  // groups of 16 rows per CTA: as many as the accumulators leave registers for (prompts; decode steps have one)
  const int rg = P.reserved <= 1 ? 1 : P.reserved;
  if (rg > 2) return STRATUM_ERR_SHAPE;
  const size_t smem = (size_t)stratum_attention_general_mma_smem(P.qk_dim, rg);
  if (smem > 200 * 1024) return STRATUM_ERR_LIMIT;
  const int head_groups = (P.group + 15) / 16;
  const long long items = (long long)P.n_qblocks * (P.n_heads / P.group) * head_groups * P.maps * P.n_splits;
  if (items > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  void (*kern)(const GeneralAttention) = nullptr;
  if (cpw <= 1) kern = rg == 1 ? attention_general_mma_kernel<1, 1> : attention_general_mma_kernel<1, 2>;
  else if (cpw <= 2) kern = rg == 1 ? attention_general_mma_kernel<2, 1> : attention_general_mma_kernel<2, 2>;
  else if (cpw <= 4) kern = rg == 1 ? attention_general_mma_kernel<4, 1> : attention_general_mma_kernel<4, 2>;
  else return STRATUM_ERR_LIMIT;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  kern<<<(unsigned)items, GM_WARPS * 32, smem, stream>>>(P);
  int st = launch_status();
  if (st || direct) return st;
  const long long rows = (long long)P.n_tokens * P.n_heads;
  if (rows > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  if (P.maps == 1) attention_general_finish_kernel<1><<<(unsigned)rows, 128, 0, stream>>>(P);
  else attention_general_finish_kernel<2><<<(unsigned)rows, 128, 0, stream>>>(P);
  return launch_status();
}
