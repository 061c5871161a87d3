// Gated linear attention: a recurrent mixer whose state is one matrix S [dim][vdim] per head, in float32, with a decay
// per key channel.
//
// Per token, from the float32 sums of the fused input projection (row = [q | k | v | g | a]: n_heads * dim twice,
// n_heads * vdim twice, then `rank` values of the decay's inner projection):
//   cast      the `rank` values a go, rounded to the compute dtype, to a matrix of their own: the operand of the decay's
//             second projection z = W_a2 a + b, which is a matrix product like any other (float32 sums);
//   decay     alpha = sigmoid(z)^(1/tau) = exp(log_sigmoid(z) / tau), in place, the logarithm taken without forming
//             sigmoid(z);
//   recur     per head, token after token:  S <- diag(alpha) S + k v^T;  o = S^T q * dim^(-1/2)
//             (the decay acts on the rows of S, which belong to key channels; o sees the token's own write).
//   finish    o / sqrt(mean_vdim(o^2) + eps) * gain * silu(g), rounded to the compute dtype for the output product.
// All of it is float32 whatever the compute dtype.
//
// The recurrence is sequential in the tokens of a sequence and independent across sequences, heads and columns of S:
// a block owns (sequence, head, a tile of columns), a lane 16 rows of one column, so a column's read-out is split over
// neighbouring lanes and added by shuffles in a fixed order; the tokens' k, q, alpha and v come through a double
// buffer in shared memory that the next tokens fill (cp.async) while the current ones are worked on.  Nothing depends
// on how a sequence's tokens are cut into steps or on the other sequences of a step.
#include <math.h>

#include "common.cuh"

struct Gla {
  const float* proj;        // [tokens][ld]
  void* inner;              // [tokens][ld_inner], the compute dtype: the decay's inner projection (cast)
  const float* reserved_p;
  const float* gain;        // [vdim]
  float* alpha;             // [tokens][n_heads * dim]: z when `decay` begins, alpha when it ends
  float* o_raw;             // [tokens][n_heads * vdim]
  void* out;                // [tokens][ldo] compute dtype
  float* state;             // [slots][state_stride]: S^T [n_heads][vdim][dim]
  const int* token_seq;
  const int* seq_start;     // [seqs + 1]
  const int* seq_slot;      // [seqs]
  int ld, ldo, n_tokens, n_seqs;
  int n_heads, dim, vdim, rank;
  int state_stride, write_state, ld_inner, reserved_i;
  float eps, inv_tau, q_scale, reserved;
};

__device__ __forceinline__ float gla_silu(float z) { return z / (1.0f + expf(-z)); }

// ---------------------------------------------------------------- cast and decay: elementwise
template <typename T>
__global__ void __launch_bounds__(256) gla_cast_kernel(const Gla P) {
  pdl_trigger();
  pdl_wait();                                        // the projection is the work of the kernel before: ld_fresh
  const size_t n = (size_t)P.n_tokens * P.rank;
  const size_t first = 2 * (size_t)P.n_heads * P.dim + 2 * (size_t)P.n_heads * P.vdim;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / P.rank, r = i - t * P.rank;
    ((T*)P.inner)[t * P.ld_inner + r] = from_float<T>(ld_fresh(P.proj + t * P.ld + first + r));
  }
}

__global__ void __launch_bounds__(256) gla_decay_kernel(const Gla P) {
  pdl_trigger();
  pdl_wait();                                        // z is the work of the kernel before: ld_fresh
  const size_t n = (size_t)P.n_tokens * P.n_heads * P.dim;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float z = ld_fresh(P.alpha + i);
    const float ls = z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));      // log sigmoid(z)
    P.alpha[i] = expf(ls * P.inv_tau);
  }
}

// ---------------------------------------------------------------- the recurrence
#define GLA_THREADS 128
#define GLA_ROWS 16           // rows of a column of S that a lane holds
#define GLA_MAX_CHUNK 16      // tokens staged in shared memory at a time, at most

__device__ __forceinline__ void gla_copy4(float* dst_shared, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void gla_copy16(float* dst_shared, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void gla_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void gla_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// The state of a head lies in memory column by column (S^T: [vdim][dim]), so the rows a lane holds are contiguous and
// neighbouring lanes read neighbouring stretches.  A column is spread over L lanes of 16 rows each (dim <= 16 L).
template <int L>
__global__ void __launch_bounds__(GLA_THREADS) gla_recur_kernel(const Gla P) {
  constexpr int ROWS = GLA_ROWS;
  constexpr int COLS = GLA_THREADS / L;
  constexpr int PITCH = 20;                          // floats between two lanes' stretches: float4 reads of eight
  constexpr int KQ = L * PITCH;                      // neighbouring lanes fall on different banks
  constexpr int FIT = 1280 / KQ;
  constexpr int CHUNK = FIT < 2 ? 2 : (FIT > GLA_MAX_CHUNK ? GLA_MAX_CHUNK : FIT);
  __shared__ __align__(16) float kqa_s[2][CHUNK][3][KQ];      // k, q, alpha of the staged tokens
  __shared__ float v_s[2][CHUNK][COLS];
  const int seq = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
  const int r0 = P.seq_start[seq], r1 = P.seq_start[seq + 1];
  if (r0 >= r1) return;
  const int D = P.dim, V = P.vdim, HD = P.n_heads * D, HV = P.n_heads * V;
  const int part = threadIdx.x % L, col = threadIdx.x / L;
  const int j = tile * COLS + col;
  const bool live = j < V;
  if (P.token_seq[r0] < 0) {                         // rows of no sequence: nothing is kept, the output is zero
    if (part == 0 && live)
      for (int r = r0; r < r1; r++) P.o_raw[(size_t)r * HV + (size_t)h * V + j] = 0.f;
    return;
  }
  float* Sg = P.state + (size_t)P.seq_slot[seq] * P.state_stride + ((size_t)h * V + (live ? j : 0)) * D + part * ROWS;
  const bool vec = D % 4 == 0 && (P.state_stride % 4) == 0 && (((uintptr_t)P.state) & 15) == 0;
  float2 S[ROWS / 2];
#pragma unroll
  for (int i = 0; i < ROWS; i += 4) {
    const int d = part * ROWS + i;
    if (live && vec && d + 3 < D) {
      const float4 v4 = *reinterpret_cast<const float4*>(Sg + i);
      S[i / 2] = make_float2(v4.x, v4.y); S[i / 2 + 1] = make_float2(v4.z, v4.w);
    } else {
      float e[4];
#pragma unroll
      for (int u = 0; u < 4; u++) e[u] = (live && d + u < D) ? Sg[i + u] : 0.f;
      S[i / 2] = make_float2(e[0], e[1]); S[i / 2 + 1] = make_float2(e[2], e[3]);
    }
  }
  if (D != ROWS * L) {       // the dimensions beyond dim in the staging buffers stay zero: nothing below writes them
    for (int i = threadIdx.x; i < 2 * CHUNK * 3 * KQ; i += GLA_THREADS) (&kqa_s[0][0][0][0])[i] = 0.f;
    __syncthreads();
  }

  const bool vec_in = D % 4 == 0 && P.ld % 4 == 0 && ((((uintptr_t)P.proj) | ((uintptr_t)P.alpha)) & 15) == 0;
  auto stage = [&](int buf, int c0) {                // ask for the tokens c0 .. of this sequence
    const int n_here = min(CHUNK, r1 - c0);
    for (int tok = 0; tok < n_here; tok++) {
      const float* row = P.proj + (size_t)(c0 + tok) * P.ld + (size_t)h * D;
      const float* al = P.alpha + (size_t)(c0 + tok) * HD + (size_t)h * D;
      if (vec_in) {
        for (int d = 4 * threadIdx.x; d < 3 * D; d += 4 * GLA_THREADS) {         // k, then q, then alpha
          const int which = d / D, dd = d - which * D;
          const float* src = which == 0 ? row + HD + dd : (which == 1 ? row + dd : al + dd);
          gla_copy16(&kqa_s[buf][tok][which][(dd / ROWS) * PITCH + dd % ROWS], src);
        }
      } else {
        for (int d = threadIdx.x; d < 3 * D; d += GLA_THREADS) {
          const int which = d / D, dd = d - which * D;
          const float* src = which == 0 ? row + HD + dd : (which == 1 ? row + dd : al + dd);
          gla_copy4(&kqa_s[buf][tok][which][(dd / ROWS) * PITCH + dd % ROWS], src);
        }
      }
    }
    for (int i = threadIdx.x; i < n_here * COLS; i += GLA_THREADS) {
      const int tok = i / COLS, cc = i - tok * COLS, jj = tile * COLS + cc;
      if (jj < V) gla_copy4(&v_s[buf][tok][cc], P.proj + (size_t)(c0 + tok) * P.ld + 2 * (size_t)HD + (size_t)h * V + jj);
    }
    gla_commit();
  };

  stage(0, r0);
  int buf = 0;
  for (int c0 = r0; c0 < r1; c0 += CHUNK, buf ^= 1) {
    gla_wait_all();
    __syncthreads();                                 // this chunk has landed, and the other buffer is free again
    if (c0 + CHUNK < r1) stage(buf ^ 1, c0 + CHUNK);
    const int n_here = min(CHUNK, r1 - c0);
    float* o_row = P.o_raw + (size_t)c0 * HV + (size_t)h * V + (live ? j : 0);
#pragma unroll 2
    for (int tok = 0; tok < n_here; tok++, o_row += HV) {
      const float4* kk = reinterpret_cast<const float4*>(&kqa_s[buf][tok][0][part * PITCH]);
      const float4* qq = reinterpret_cast<const float4*>(&kqa_s[buf][tok][1][part * PITCH]);
      const float4* aa = reinterpret_cast<const float4*>(&kqa_s[buf][tok][2][part * PITCH]);
      const float vj = v_s[buf][tok][col];
      const float2 vv = make_float2(vj, vj);
      float2 acc0 = make_float2(0.f, 0.f), acc1 = acc0;
#pragma unroll
      for (int i = 0; i < ROWS / 4; i++) {
        const float4 k4 = kk[i], q4 = qq[i], a4 = aa[i];
        S[2 * i] = __ffma2_rn(make_float2(k4.x, k4.y), vv, __fmul2_rn(make_float2(a4.x, a4.y), S[2 * i]));
        S[2 * i + 1] = __ffma2_rn(make_float2(k4.z, k4.w), vv, __fmul2_rn(make_float2(a4.z, a4.w), S[2 * i + 1]));
        acc0 = __ffma2_rn(S[2 * i], make_float2(q4.x, q4.y), acc0);
        acc1 = __ffma2_rn(S[2 * i + 1], make_float2(q4.z, q4.w), acc1);
      }
      const float2 acc = __fadd2_rn(acc0, acc1);
      float o = acc.x + acc.y;
#pragma unroll
      for (int s = 1; s < L; s <<= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
      if (part == 0 && live) *o_row = o * P.q_scale;
    }
  }
  if (P.write_state && live) {
#pragma unroll
    for (int i = 0; i < ROWS; i += 4) {
      const int d = part * ROWS + i;
      const float e[4] = {S[i / 2].x, S[i / 2].y, S[i / 2 + 1].x, S[i / 2 + 1].y};
      if (vec && d + 3 < D) {
        *reinterpret_cast<float4*>(Sg + i) = make_float4(e[0], e[1], e[2], e[3]);
      } else {
#pragma unroll
        for (int u = 0; u < 4; u++)
          if (d + u < D) Sg[i + u] = e[u];
      }
    }
  }
}

// ---------------------------------------------------------------- finish: one warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(128) gla_finish_kernel(const Gla P) {
  const int lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();                // o_raw and the projection are the work of kernels before this one: ld_fresh
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long long)P.n_tokens * P.n_heads) return;
  const int t = (int)(item / P.n_heads), h = (int)(item - (long long)t * P.n_heads);
  const int V = P.vdim, HD = P.n_heads * P.dim, HV = P.n_heads * V;
  const float* o = P.o_raw + (size_t)t * HV + (size_t)h * V;
  const float* g = P.proj + (size_t)t * P.ld + 2 * (size_t)HD + HV + (size_t)h * V;
  T* out = (T*)P.out + (size_t)t * P.ldo + (size_t)h * V;
  float ss = 0.f;
  for (int d = lane; d < V; d += 32) {
    const float x = ld_fresh(o + d);
    ss = fmaf(x, x, ss);
  }
  ss = warp_sum(ss);
  const float mul = 1.0f / sqrtf(ss / (float)V + P.eps);
  for (int d = lane; d < V; d += 32)
    out[d] = from_float<T>(ld_fresh(o + d) * mul * P.gain[d] * gla_silu(ld_fresh(g + d)));
}

static int gla_check(const Gla& P) {
  if (P.n_heads < 1 || P.dim < 1 || P.vdim < 1 || P.rank < 1) return STRATUM_ERR_SHAPE;
  if (P.ld < 2 * P.n_heads * P.dim + 2 * P.n_heads * P.vdim + P.rank || P.ldo < P.n_heads * P.vdim)
    return STRATUM_ERR_SHAPE;
  if (P.state_stride < P.n_heads * P.dim * P.vdim) return STRATUM_ERR_SHAPE;
  if (P.dim > 32 * GLA_ROWS) return STRATUM_ERR_LIMIT;
  if (P.n_heads > 65535 || P.n_seqs > 65535) return STRATUM_ERR_LIMIT;
  return 0;
}

static unsigned gla_blocks(size_t n) {
  const size_t blocks = (n + 255) / 256;
  return (unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks);
}

// The decay's inner projection as a matrix of the compute dtype (one launch).
STRATUM_EXPORT int stratum_gla_cast(const Gla* params, int dtype, cudaStream_t stream) {
  const Gla& P = *params;
  if (P.n_tokens <= 0) return 0;
  const int bad = gla_check(P);
  if (bad) return bad;
  if (!P.inner || P.ld_inner < P.rank) return STRATUM_ERR_SHAPE;
  const unsigned blocks = gla_blocks((size_t)P.n_tokens * P.rank);
  if (dtype == STRATUM_DT_F32) launch_pdl(gla_cast_kernel<float>, blocks, 256, 0, stream, P);
  else if (dtype == STRATUM_DT_BF16) launch_pdl(gla_cast_kernel<bf16>, blocks, 256, 0, stream, P);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}

template <int L>
static void gla_recur_launch(const Gla& P, cudaStream_t stream) {
  const int cols = GLA_THREADS / L;
  const dim3 grid((P.vdim + cols - 1) / cols, P.n_heads, P.n_seqs);
  gla_recur_kernel<L><<<grid, GLA_THREADS, 0, stream>>>(P);
}

// The rest of a step, one launch each: which = 0 the decays from z (in place), 1 the recurrence, 2 finish.  dtype:
// the compute dtype of `out`.
STRATUM_EXPORT int stratum_gla(const Gla* params, int which, int dtype, cudaStream_t stream) {
  const Gla& P = *params;
  if (P.n_tokens <= 0 || P.n_seqs <= 0) return 0;
  const int bad = gla_check(P);
  if (bad) return bad;
  if (dtype != STRATUM_DT_F32 && dtype != STRATUM_DT_BF16) return STRATUM_ERR_DTYPE;
  if (which == 0) {
    launch_pdl(gla_decay_kernel, gla_blocks((size_t)P.n_tokens * P.n_heads * P.dim), 256, 0, stream, P);
    return launch_status();
  }
  if (which == 1) {
    int L = 1;
    while (GLA_ROWS * L < P.dim) L <<= 1;
    switch (L) {
      case 1: gla_recur_launch<1>(P, stream); break;
      case 2: gla_recur_launch<2>(P, stream); break;
      case 4: gla_recur_launch<4>(P, stream); break;
      case 8: gla_recur_launch<8>(P, stream); break;
      case 16: gla_recur_launch<16>(P, stream); break;
      default: gla_recur_launch<32>(P, stream); break;
    }
    return launch_status();
  }
  if (which != 2) return STRATUM_ERR_SHAPE;
  const long long items = (long long)P.n_tokens * P.n_heads;
  const long long blocks = (items + 3) / 4;
  if (blocks > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  if (dtype == STRATUM_DT_F32) launch_pdl(gla_finish_kernel<float>, (unsigned)blocks, 128, 0, stream, P);
  else launch_pdl(gla_finish_kernel<bf16>, (unsigned)blocks, 128, 0, stream, P);
  return launch_status();
}
