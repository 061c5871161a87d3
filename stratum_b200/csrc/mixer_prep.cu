// Between a mixer's fused projection and its attention: rotate, normalise, and append to the paged cache.
//
// x [tokens][ld] holds, per token, what one matrix product made: query heads, key heads and value heads, each
// kind a run of equal heads from its own column on.  For every token of a sequence (index >= 0) at position p:
//   query head j   the dimensions [q_rot_off, q_rot_off + 2 R) are rotated in place; or, where q_out is given, the
//                  dimensions from q_rot_off to the head's end go (the first 2 R of them rotated) to
//                  q_out[token][j * q_out_step + q_out_off ...], and x keeps what it had;
//   key head j     the first k_norm_n dimensions become u / sqrt(mean(u^2) + eps) * gain (k_norm_n = 0: as they are),
//                  the dimensions [k_rot_off, k_rot_off + 2 R) are rotated, and the head goes to the token's row of
//                  the key cache [pages][n_k][page_tokens][k_dim];
//                  with k_out the same numbers also go to row t of that matrix (rows of tokens of no sequence: zeros);
//   value head j   goes to the value cache [pages][n_v][page_tokens][v_dim]  (n_v = 0: the mixer keeps no values).
// Rotation: pair (i, i + R), i < R (or, with `interleaved`, the neighbours (2i, 2i + 1)), angle a = (float)p *
// inv_freq[i]:  (u, v) -> (u cos a - v sin a, v cos a + u sin a).
//
// gate_heads: a[t][j * block + i] *= sigmoid(g[t][j]): every head's stretch of a row times the head's gate, whose
// pre-activation is a column of a projection.
// Everything is evaluated in float32 and rounded once to the storage type.  One block per token; the order of
// every sum depends on the row alone.
#include <math.h>

#include "common.cuh"

struct MixerPrep {
  void* x;
  const int* token_pos;
  const int* token_seq;
  const int* block_table;
  const float* inv_freq;      // [rot_pairs]
  const float* k_norm_gain;   // [k_norm_n]
  void* k_cache;
  void* v_cache;
  void* q_out;
  void* k_out;
  int ld, bt_stride, n_tokens, rot_pairs;
  int n_q, q_dim, q_col, q_rot_off;
  int n_k, k_dim, k_col, k_rot_off, k_norm_n;
  int n_v, v_dim, v_col;
  int page_tokens, write_cache;
  float eps;
  int q_out_ld, q_out_step, q_out_off;
  int k_out_ld, interleaved;
};

template <typename T>
__global__ void __launch_bounds__(128) mixer_prep_kernel(const MixerPrep P) {
  extern __shared__ float2 mp_cs[];                 // [rot_pairs] (cos, sin)
  __shared__ float scratch[33];
  pdl_trigger();
  const int t = blockIdx.x;
  const int seq = P.token_seq[t];
  if (seq < 0) {                                    // a padding token
    pdl_wait();
    if (P.k_out) {
      T* ko = (T*)P.k_out + (size_t)t * P.k_out_ld;
      for (int d = threadIdx.x; d < P.n_k * P.k_dim; d += blockDim.x) ko[d] = from_float<T>(0.f);
    }
    return;
  }
  const int pos = P.token_pos[t];
  const int R = P.rot_pairs;
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * P.inv_freq[i], &s, &c);
    mp_cs[i] = make_float2(c, s);
  }
  size_t row = 0;
  if (P.write_cache) row = (size_t)P.block_table[(size_t)seq * P.bt_stride + pos / P.page_tokens];
  const int in_page = pos % P.page_tokens;
  T* x = (T*)P.x + (size_t)t * P.ld;
  __syncthreads();
  pdl_wait();
  // queries: rotate in place, or into q_out together with what follows the rotated dimensions
  const int tail = P.q_out ? P.q_dim - P.q_rot_off - 2 * R : 0;
  T* qo = P.q_out ? (T*)P.q_out + (size_t)t * P.q_out_ld + P.q_out_off : nullptr;
  for (int it = threadIdx.x; it < P.n_q * (R + tail); it += blockDim.x) {
    const int j = it / (R + tail), i = it - j * (R + tail);
    T* u = x + P.q_col + (size_t)j * P.q_dim + P.q_rot_off;
    T* w = qo ? qo + (size_t)j * P.q_out_step : u;
    if (i < R) {
      const int ia = P.interleaved ? 2 * i : i, ib = P.interleaved ? 2 * i + 1 : i + R;
      const float a = ld_fresh(u + ia), b = ld_fresh(u + ib);
      const float2 f = mp_cs[i];
      w[ia] = from_float<T>(a * f.x - b * f.y);
      w[ib] = from_float<T>(b * f.x + a * f.y);
    } else {
      w[i + R] = from_float<T>(ld_fresh(u + i + R));
    }
  }
  if (!P.write_cache) return;
  for (int j = 0; j < P.n_k; j++) {
    const T* k = x + P.k_col + (size_t)j * P.k_dim;
    T* dst = (T*)P.k_cache + ((row * P.n_k + j) * P.page_tokens + in_page) * (size_t)P.k_dim;
    float mul = 1.f;
    if (P.k_norm_n > 0) {
      float ss = 0.f;
      for (int d = threadIdx.x; d < P.k_norm_n; d += blockDim.x) {
        const float v = ld_fresh(k + d);
        ss = fmaf(v, v, ss);
      }
      ss = block_sum(ss, scratch);
      mul = 1.0f / sqrtf(ss / (float)P.k_norm_n + P.eps);
    }
    for (int d = threadIdx.x; d < P.k_dim; d += blockDim.x) {
      float v = ld_fresh(k + d);
      if (d < P.k_norm_n) {
        v = v * mul * P.k_norm_gain[d];
      } else if (d >= P.k_rot_off && d < P.k_rot_off + 2 * R) {
        const int i = d - P.k_rot_off;
        if (P.interleaved) {
          const float2 f = mp_cs[i >> 1];
          const float other = ld_fresh(k + d + ((i & 1) ? -1 : 1));
          v = (i & 1) ? v * f.x + other * f.y : v * f.x - other * f.y;
        } else if (i < R) {
          const float2 f = mp_cs[i];
          v = v * f.x - ld_fresh(k + d + R) * f.y;
        } else {
          const float2 f = mp_cs[i - R];
          v = v * f.x + ld_fresh(k + d - R) * f.y;
        }
      }
      dst[d] = from_float<T>(v);
      if (P.k_out) ((T*)P.k_out)[(size_t)t * P.k_out_ld + (size_t)j * P.k_dim + d] = from_float<T>(v);
    }
  }
  for (int it = threadIdx.x; it < P.n_v * P.v_dim; it += blockDim.x) {
    const int j = it / P.v_dim, d = it - j * P.v_dim;
    T* dst = (T*)P.v_cache + ((row * P.n_v + j) * P.page_tokens + in_page) * (size_t)P.v_dim;
    dst[d] = from_float<T>(ld_fresh(x + P.v_col + it));
  }
}

template <typename T>
__global__ void gate_heads_kernel(T* a, int lda, const T* g, int ldg, int n_heads, int block, size_t total) {
  pdl_trigger();
  pdl_wait();                                        // a and g are the work of kernels before this one: ld_fresh
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int width = n_heads * block;
  const size_t t = i / width;
  const int c = (int)(i - t * width);
  const float z = ld_fresh((const T*)g + t * ldg + c / block);
  T* p = a + t * lda + c;
  *p = from_float<T>(ld_fresh((const T*)p) / (1.0f + expf(-z)));
}

STRATUM_EXPORT int stratum_gate_heads(void* a, int lda, const void* g, int ldg, int n_rows, int n_heads, int block,
                                      int dtype, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * n_heads * block;
  if (total == 0) return 0;
  if (n_heads < 1 || block < 1 || lda < n_heads * block || ldg < n_heads) return STRATUM_ERR_SHAPE;
  const size_t blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffULL) return STRATUM_ERR_LIMIT;
  if (dtype == STRATUM_DT_F32)
    launch_pdl(gate_heads_kernel<float>, (unsigned)blocks, 256, 0, stream, (float*)a, lda, (const float*)g, ldg,
               n_heads, block, total);
  else if (dtype == STRATUM_DT_BF16)
    launch_pdl(gate_heads_kernel<bf16>, (unsigned)blocks, 256, 0, stream, (bf16*)a, lda, (const bf16*)g, ldg, n_heads,
               block, total);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}

STRATUM_EXPORT int stratum_mixer_prep(const MixerPrep* params, int dtype, cudaStream_t stream) {
  const MixerPrep& P = *params;
  if (P.n_tokens <= 0) return 0;
  if (P.rot_pairs < 0 || P.n_q < 0 || P.n_k < 0 || P.n_v < 0 || P.page_tokens < 1) return STRATUM_ERR_SHAPE;
  if (P.rot_pairs > 0 && (!P.inv_freq || P.q_rot_off + 2 * P.rot_pairs > P.q_dim ||
                          (P.n_k > 0 && P.k_rot_off + 2 * P.rot_pairs > P.k_dim)))
    return STRATUM_ERR_SHAPE;
  if (P.k_norm_n > 0 && (!P.k_norm_gain || P.k_norm_n > P.k_rot_off || P.k_norm_n > P.k_dim)) return STRATUM_ERR_SHAPE;
  if (P.write_cache && ((P.n_k > 0 && !P.k_cache) || (P.n_v > 0 && !P.v_cache) || !P.block_table))
    return STRATUM_ERR_SHAPE;
  const size_t smem = (size_t)P.rot_pairs * sizeof(float2);
  if (smem > 40 * 1024) return STRATUM_ERR_LIMIT;
  if (dtype == STRATUM_DT_F32) return launch_pdl(mixer_prep_kernel<float>, P.n_tokens, 128, smem, stream, P);
  if (dtype == STRATUM_DT_BF16) return launch_pdl(mixer_prep_kernel<bf16>, P.n_tokens, 128, smem, stream, P);
  return STRATUM_ERR_DTYPE;
}
