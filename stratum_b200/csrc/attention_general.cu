// Causal attention over the paged cache for mixers whose heads do not look like grouped-query attention's:
// keys and values of different sizes, values that are a stretch of the key rows themselves, several score maps
// per head over one set of values, scores squashed by a tanh, a query factor that grows with the position,
// and an epilogue that combines the maps.  One warp per (token, head); CUDA cores, float32 throughout.  It is the
// kernel of the true 32-bit path for prompts and decoding alike and the bfloat16 path's fallback for the shapes
// its tensor-core kernel (attention_general_mma.cu) refuses.
//
// For head h of a token at position p in sequence s, and map m < maps:
//   key head   kh = (h / group) * maps + m          value head  vh = h / group
//   score_t    = (q[h][m] . K_t[kh]) * scale * temp(p),  temp(p) = 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)
//   score_t   <- softcap * tanh(score_t / softcap)       (softcap > 0)
//   a_m        = sum_t softmax_t(score) V_t[vh]           over the keys t in [lo, p], lo = 0 or p - window + 1,
//                                                         and with a window also the keys t < keep_first
// Values: rows of the value cache, or (v_in_k) the first v_dim values of the key rows of head (h / group) * maps.
// sink: where given, exp(sink[h]) is one more term of every softmax's denominator (it has no key and no value).
// combine 0 (maps = 1): out[h] = a_0.
// combine 1 (maps = 2): o = a_0 - lambda * a_1;  o <- o / sqrt(mean(o^2) + eps) * out_scale;
//                       o <- o * sigmoid(gate[h]) where a gate column is given (gate: q's rows, column gate_col + h).
//
// Keys are visited in chunks of 32 whose boundaries are multiples of 32 from position 0, and the running maximum,
// denominator and output are updated once per chunk in key order.  So the result at a position does not depend
// on how the tokens were cut into steps, on the other sequences of the step, or on which pages hold the keys.
#include <math.h>

#include "attention_general.h"
#include "common.cuh"

#define AG_WARPS 4

template <typename T, int MAPS, int VCH>
__global__ void __launch_bounds__(AG_WARPS * 32)
attention_general_kernel(const GeneralAttention P) {
  extern __shared__ float ag_q[];                   // [warps][MAPS][qk_dim]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * AG_WARPS + warp;
  if (item >= (long long)P.n_tokens * P.n_heads) return;
  const int t = (int)(item / P.n_heads), h = (int)(item - (long long)t * P.n_heads);
  const int seq = P.token_seq[t];
  if (seq < 0) return;                              // padding token
  const int pos = P.token_pos[t];
  const int D = P.qk_dim, Dv = P.v_dim;
  const T* q = (const T*)P.q + (size_t)t * P.ldq + (size_t)h * MAPS * D;
  float* qs = ag_q + (size_t)warp * MAPS * D;
  for (int d = lane; d < MAPS * D; d += 32) qs[d] = to_float(q[d]);
  __syncwarp();

  float temp = 1.f;
  if (P.temp_coef != 0.f) temp = 1.f + P.temp_coef * logf((float)((pos + 1) / P.temp_every) + 1.f);
  const float factor = P.scale * temp;
  const int lo = (P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
  // chunks are visited in key order: those that hold kept first keys, then those from the window's first key on
  const int first_win = (lo / 32) * 32;
  const int kept_end = min(P.window > 0 ? P.keep_first : 0, lo);
  const int* bt = P.block_table + (size_t)seq * P.bt_stride;
  const int kv = h / P.group;
  const size_t k_page = (size_t)P.n_k_heads * P.page_tokens * D;
  const T* vbase = P.v_in_k ? (const T*)P.k_cache : (const T*)P.v_cache;
  const int v_row = P.v_in_k ? D : Dv;
  const size_t v_page = P.v_in_k ? k_page : (size_t)P.n_v_heads * P.page_tokens * Dv;
  const size_t v_head = P.v_in_k ? (size_t)kv * MAPS * P.page_tokens * D : (size_t)kv * P.page_tokens * Dv;

  float m_run[MAPS], l_run[MAPS], acc[MAPS][VCH];
#pragma unroll
  for (int m = 0; m < MAPS; m++) {
    m_run[m] = -INFINITY;
    l_run[m] = 0.f;
#pragma unroll
    for (int i = 0; i < VCH; i++) acc[m][i] = 0.f;
  }

  for (int base = 0; base <= pos; base += 32) {
    if (base >= kept_end && base < first_win) {      // nothing between the kept keys and the window is seen
      base = first_win - 32;
      continue;
    }
    const int key = base + lane;
    const bool valid = (key >= lo || key < kept_end) && key <= pos;
    const int page = bt[base / P.page_tokens];      // page_tokens is a multiple of 32: one page per chunk
    const int in_page = base % P.page_tokens;
    const T* vr = vbase + (size_t)page * v_page + v_head + (size_t)in_page * v_row;
    const int n_here = min(32, pos - base + 1);
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      float s = -INFINITY;
      if (valid) {
        const T* kr = (const T*)P.k_cache + (size_t)page * k_page +
                      ((size_t)(kv * MAPS + m) * P.page_tokens + in_page + lane) * D;
        const float* qm = qs + m * D;
        float dot = 0.f;
        for (int d = 0; d < D; d++) dot = fmaf(qm[d], to_float(kr[d]), dot);
        s = dot * factor;
        if (P.softcap > 0.f) s = P.softcap * tanhf(s / P.softcap);
      }
      const float m_new = fmaxf(m_run[m], warp_max(s));   // finite: every chunk visited holds a valid key
      const float corr = expf(m_run[m] - m_new);          // exp(-inf) = 0 on the first chunk
      const float p = valid ? expf(s - m_new) : 0.f;
      float chunk_sum = 0.f;
#pragma unroll
      for (int j = 0; j < 32; j++) chunk_sum += __shfl_sync(0xffffffffu, p, j);
      l_run[m] = l_run[m] * corr + chunk_sum;
#pragma unroll
      for (int i = 0; i < VCH; i++) acc[m][i] *= corr;
      for (int j = 0; j < n_here; j++) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
        for (int i = 0; i < VCH; i++) {
          const int d = lane + 32 * i;
          if (d < Dv) acc[m][i] = fmaf(pj, to_float(vr[(size_t)j * v_row + d]), acc[m][i]);
        }
      }
      m_run[m] = m_new;
    }
  }

  if (P.sink) {
#pragma unroll
    for (int m = 0; m < MAPS; m++) l_run[m] += expf(P.sink[h] - m_run[m]);
  }
  T* op = (T*)P.out + (size_t)t * P.ldo + (size_t)h * Dv;
  if (MAPS == 1 || P.combine == 0) {
    const float inv = 1.0f / l_run[0];
#pragma unroll
    for (int i = 0; i < VCH; i++) {
      const int d = lane + 32 * i;
      if (d < Dv) op[d] = from_float<T>(acc[0][i] * inv);
    }
    return;
  }
  const float inv0 = 1.0f / l_run[0], inv1 = 1.0f / l_run[MAPS - 1];
  float o[VCH], ss = 0.f;
#pragma unroll
  for (int i = 0; i < VCH; i++) {
    const int d = lane + 32 * i;
    o[i] = d < Dv ? acc[0][i] * inv0 - P.lambda * (acc[MAPS - 1][i] * inv1) : 0.f;
    ss = fmaf(o[i], o[i], ss);
  }
  ss = warp_sum(ss);
  float mul = P.out_scale / sqrtf(ss / (float)Dv + P.eps);
  if (P.gate_col >= 0) {
    const float z = to_float(((const T*)P.q)[(size_t)t * P.ldq + P.gate_col + h]);
    mul *= 1.0f / (1.0f + expf(-z));
  }
#pragma unroll
  for (int i = 0; i < VCH; i++) {
    const int d = lane + 32 * i;
    if (d < Dv) op[d] = from_float<T>(o[i] * mul);
  }
}

template <typename T, int MAPS>
static int launch_general(const GeneralAttention& P, cudaStream_t stream) {
  const long long items = (long long)P.n_tokens * P.n_heads;
  const long long blocks = (items + AG_WARPS - 1) / AG_WARPS;
  if (blocks > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  const size_t smem = (size_t)AG_WARPS * MAPS * P.qk_dim * sizeof(float);
  if (smem > 48 * 1024) return STRATUM_ERR_LIMIT;
  const int vch = (P.v_dim + 31) / 32;
#define AG_LAUNCH(V)                                                                                          \
  attention_general_kernel<T, MAPS, V><<<(unsigned)blocks, AG_WARPS * 32, smem, stream>>>(P)
  if (vch <= 2) AG_LAUNCH(2);
  else if (vch <= 4) AG_LAUNCH(4);
  else if (vch <= 8) AG_LAUNCH(8);
  else if (vch <= 16) AG_LAUNCH(16);
  else if (vch <= 32) AG_LAUNCH(32);
  else return STRATUM_ERR_LIMIT;
#undef AG_LAUNCH
  return launch_status();
}

STRATUM_EXPORT int stratum_attention_general(const GeneralAttention* params, int dtype, cudaStream_t stream) {
  const GeneralAttention& P = *params;
  if (P.n_tokens <= 0) return 0;
  const int bad = general_attention_check(P);
  if (bad) return bad;
  if (dtype == STRATUM_DT_F32)
    return P.maps == 1 ? launch_general<float, 1>(P, stream) : launch_general<float, 2>(P, stream);
  if (dtype == STRATUM_DT_BF16)
    return P.maps == 1 ? launch_general<bf16, 1>(P, stream) : launch_general<bf16, 2>(P, stream);
  return STRATUM_ERR_DTYPE;
}
