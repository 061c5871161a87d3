// What the general attention kernels are told (mirrored field by field by kernels.py: pointers first, then
// 4-byte fields).  See attention_general.cu for the meaning of every field.
#pragma once
#include "common.cuh"

struct GeneralAttention {
  const void* q;            // [tokens][ldq]: head h, map m at column (h * maps + m) * qk_dim
  const void* k_cache;      // [pages][n_k_heads][page_tokens][qk_dim]
  const void* v_cache;      // [pages][n_v_heads][page_tokens][v_dim], unused when v_in_k
  void* out;                // [tokens][ldo]: head h at column h * v_dim
  const int* token_pos;     // [tokens]
  const int* token_seq;     // [tokens]: index of the token's sequence in the step, -1 = padding
  const int* block_table;   // [seqs][bt_stride]
  const int* qb_seq;        // query blocks (tensor-core prompt kernel): sequence, first row, tokens
  const int* qb_tok0;
  const int* qb_ntok;
  float* part_o;            // scratch of the key splits (tensor-core decode kernel)
  float* part_ml;
  const int* seq_start;     // dense keys (tensor-core kernel): first row of every sequence of the step
  const float* sink;        // [n_heads] or null: exp(sink[h]) joins the softmax's denominator (no key, no value, not scaled)
  int ldq, ldo, bt_stride, n_tokens;
  int n_heads, group, maps;
  int qk_dim, v_dim, n_k_heads, n_v_heads, v_in_k;
  int page_tokens, window, combine, gate_col;
  int temp_every, n_qblocks, tokens_per_block, n_splits, chunk, reserved;
  int dense, ldk, ldv;      // dense: keys and values are rows of plain matrices (see attention_general_mma.cu)
  int keep_first;           // with a window: keys at positions below this stay visible to every later row
  float scale, softcap, temp_coef, lambda, out_scale, eps;
};

static inline int general_attention_check(const GeneralAttention& P) {
  if (P.n_heads < 1 || P.group < 1 || P.n_heads % P.group != 0 || P.page_tokens % 32 != 0) return STRATUM_ERR_SHAPE;
  if (P.maps < 1 || P.maps > 2 || P.qk_dim < 1 || P.v_dim < 1) return STRATUM_ERR_LIMIT;
  if (P.n_k_heads != (P.n_heads / P.group) * P.maps) return STRATUM_ERR_SHAPE;
  if (P.v_in_k ? P.v_dim > P.qk_dim : P.n_v_heads != P.n_heads / P.group) return STRATUM_ERR_SHAPE;
  if (P.combine == 0 ? P.maps != 1 : (P.combine != 1 || P.maps != 2)) return STRATUM_ERR_SHAPE;
  if (P.temp_coef != 0.f && P.temp_every < 1) return STRATUM_ERR_SHAPE;
  if (P.window < 0 || P.keep_first < 0) return STRATUM_ERR_SHAPE;
  if (P.ldq < P.n_heads * P.maps * P.qk_dim || P.ldo < P.n_heads * P.v_dim) return STRATUM_ERR_SHAPE;
  return 0;
}
