// Between the query/key(/value) projection and attention, for mixers whose queries and keys are RMS-normalised
// before they are rotated.
//
// Per token, from the float32 sums of the projection (row = [q: n_heads * dim | k: n_kv * dim | v: n_kv * v_dim]):
//   values   v_dim = 0: the key columns as projected; else the value columns; rounded once to the cache's dtype and
//            appended to the value cache;
//   q, k     divided by a root mean square (eps inside the root) and multiplied by a gain: of the whole stretch (all
//            heads together) with a gain per column, or (per_head) of every head by itself with one gain of `dim`
//            values for all heads; then in every head the first 2 * rot_pairs dimensions are turned by the angle
//            pos * inv_freq[i] (float32), (u, v) -> ((u cos - v sin) m, (v cos + u sin) m) with m the magnitude:
//            pairs (2i, 2i + 1), or (half) pairs (i, i + rot_pairs);
//   q goes to q_out [tokens][ldq] in the compute dtype, k is appended to the key cache.
// Everything between the projection's sums and the rounding of the results is float32.  Tokens of no sequence
// (sequence index -1) write nothing to the caches.  One block per token; the block's shape is fixed, so a row's sums
// do not depend on the step.
#include <math.h>

#include "common.cuh"

struct QKNormRope {
  const float* proj;        // [tokens][ld]
  const int* token_pos;
  const int* token_seq;
  const int* block_table;   // [seqs][bt_stride]
  const float* q_gain;      // [n_heads * dim]
  const float* k_gain;      // [n_kv * dim]
  const float* inv_freq;    // [rot_pairs]
  void* q_out;              // [tokens][ldq]
  void* k_cache;            // [pages][n_kv][page_tokens][dim]
  void* v_cache;            // the same shape, or [pages][n_kv][page_tokens][v_dim]
  int ld, ldq, bt_stride, n_tokens;
  int n_heads, n_kv, dim, rot_pairs;
  int page_tokens, write_cache;
  float eps, magnitude;
  int v_dim, per_head, half, reserved;
};

#define QK_THREADS 256

// the value of column c (of a stretch that begins at column c0 of the row) after norm and rotation
__device__ __forceinline__ float qk_turned(const QKNormRope& P, const float* row, int c0, int c, int d, float mul,
                                           const float* gain, int pos) {
  const int g = P.per_head ? d : c;
  float v = ld_fresh(row + c0 + c) * mul * gain[g];
  const int rp = P.rot_pairs;
  if (d < 2 * rp) {
    int mate, pair;
    bool second;
    if (P.half) { second = d >= rp; mate = second ? c - rp : c + rp; pair = second ? d - rp : d; }
    else { second = d & 1; mate = second ? c - 1 : c + 1; pair = d >> 1; }
    const float w = ld_fresh(row + c0 + mate) * mul * gain[P.per_head ? d + (mate - c) : mate];
    float sn, cs;
    sincosf((float)pos * P.inv_freq[pair], &sn, &cs);
    v = (second ? v * cs + w * sn : v * cs - w * sn) * P.magnitude;
  }
  return v;
}

template <typename T>
__global__ void __launch_bounds__(QK_THREADS) qk_norm_rope_kernel(const QKNormRope P) {
  __shared__ float scratch[33];
  extern __shared__ float head_mul[];                // per_head: 1 / rms of every query head, then of every key head
  pdl_trigger();
  pdl_wait();                                        // the projection is the work of the kernel before: ld_fresh
  const int t = blockIdx.x;
  const float* row = P.proj + (size_t)t * P.ld;
  const int D = P.dim, nq = P.n_heads * D, nk = P.n_kv * D;
  float sq = 0.f, sk = 0.f;
  if (P.per_head) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int h = warp; h < P.n_heads + P.n_kv; h += QK_THREADS / 32) {     // a head's sum: one warp, one order
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) {
        const float v = ld_fresh(row + (size_t)h * D + d);
        ss = fmaf(v, v, ss);
      }
      ss = warp_sum(ss);
      if (lane == 0) head_mul[h] = 1.0f / sqrtf(ss / (float)D + P.eps);
    }
    __syncthreads();
  } else {
    float ssq = 0.f, ssk = 0.f;
    for (int c = threadIdx.x; c < nq; c += QK_THREADS) {
      const float v = ld_fresh(row + c);
      ssq = fmaf(v, v, ssq);
    }
    for (int c = threadIdx.x; c < nk; c += QK_THREADS) {
      const float v = ld_fresh(row + nq + c);
      ssk = fmaf(v, v, ssk);
    }
    ssq = block_sum(ssq, scratch);
    ssk = block_sum(ssk, scratch);
    sq = 1.0f / sqrtf(ssq / (float)nq + P.eps);
    sk = 1.0f / sqrtf(ssk / (float)nk + P.eps);
  }
  const int pos = P.token_pos[t], seq = P.token_seq[t];

  T* qo = (T*)P.q_out + (size_t)t * P.ldq;
  for (int c = threadIdx.x; c < nq; c += QK_THREADS) {
    const int h = c / D, d = c - h * D;
    qo[c] = from_float<T>(qk_turned(P, row, 0, c, d, P.per_head ? head_mul[h] : sq, P.q_gain, pos));
  }
  if (!P.write_cache || seq < 0) return;
  const int page = P.block_table[(size_t)seq * P.bt_stride + pos / P.page_tokens];
  if (page < 0) return;
  const int in_page = pos % P.page_tokens;
  for (int c = threadIdx.x; c < nk; c += QK_THREADS) {
    const int h = c / D, d = c - h * D;
    const size_t at = (((size_t)page * P.n_kv + h) * P.page_tokens + in_page) * D + d;
    if (P.v_dim == 0) ((T*)P.v_cache)[at] = from_float<T>(ld_fresh(row + nq + c));
    ((T*)P.k_cache)[at] =
        from_float<T>(qk_turned(P, row, nq, c, d, P.per_head ? head_mul[P.n_heads + h] : sk, P.k_gain, pos));
  }
  const int V = P.v_dim;
  for (int c = threadIdx.x; c < P.n_kv * V; c += QK_THREADS) {
    const int h = c / V, d = c - h * V;
    const size_t at = (((size_t)page * P.n_kv + h) * P.page_tokens + in_page) * V + d;
    ((T*)P.v_cache)[at] = from_float<T>(ld_fresh(row + nq + nk + c));
  }
}

STRATUM_EXPORT int stratum_qk_norm_rope(const QKNormRope* params, int dtype, cudaStream_t stream) {
  const QKNormRope& P = *params;
  if (P.n_tokens <= 0) return 0;
  if (P.n_heads < 1 || P.n_kv < 1 || P.dim < 1 || P.rot_pairs < 0 || 2 * P.rot_pairs > P.dim || P.page_tokens < 1)
    return STRATUM_ERR_SHAPE;
  if (P.v_dim < 0 || P.ld < (P.n_heads + P.n_kv) * P.dim + P.n_kv * P.v_dim || P.ldq < P.n_heads * P.dim)
    return STRATUM_ERR_SHAPE;
  const size_t smem = P.per_head ? (size_t)(P.n_heads + P.n_kv) * sizeof(float) : 0;
  if (smem > 40 * 1024) return STRATUM_ERR_LIMIT;
  if (dtype == STRATUM_DT_F32) launch_pdl(qk_norm_rope_kernel<float>, P.n_tokens, QK_THREADS, smem, stream, P);
  else if (dtype == STRATUM_DT_BF16) launch_pdl(qk_norm_rope_kernel<bf16>, P.n_tokens, QK_THREADS, smem, stream, P);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}
