// A selective state-space mixer (the scalar-decay form): per head one matrix S [n_state][vdim] in float32.
//
// Per token, from the float32 sums of the fused input projection (row = [z | x | B | C | dt]: inner = n_heads * vdim,
// inner, n_groups * n_state, n_groups * n_state, n_heads):
//   prep      x, B and C (the `channels` = inner + 2 n_groups n_state columns from column inner on) pass a short causal
//             convolution over time with a bias (taps per channel, the last tap is the current token's; the taps - 1
//             inputs before a step's first token come from the sequence's state, zeros before the sequence's start) and
//             silu;  dt <- softplus(dt + dt_bias), not clamped;  decay = exp(-exp(A_log) dt).
//   recur     per head h (its B and C are those of group h / (n_heads / n_groups)), token after token:
//             S <- decay S + dt B x^T;   y = S^T C + D x.   The convolution's tail is moved on as well.
//   finish    y <- y silu(z); the row is cut into `norm_groups` equal parts, each divided by its own root mean square
//             (eps inside the root); times the gain; rounded to the compute dtype for the output product.
// All of it is float32 whatever the compute dtype.
//
// Every entry of S follows a recurrence of its own, so the work is independent across sequences, heads, columns and
// rows of S and sequential only in time.  A block owns (sequence, head, a tile of columns), a thread a few rows of a
// few columns; a column's read-out is added over neighbouring lanes by shuffles in a fixed order.  The tokens' B, C, x,
// dt and decay come through a double buffer in shared memory (cp.async).  Nothing depends on how a sequence's
// tokens are cut into steps, nor on the other sequences of a step.
#include <math.h>

#include "common.cuh"

struct SsmScan {
  const float* proj;        // [tokens][ld]
  const float* conv_w;      // [channels][taps]
  const float* conv_b;      // [channels]
  const float* a_log;       // [n_heads]
  const float* dt_bias;     // [n_heads]
  const float* d_skip;      // [n_heads]
  const float* gain;        // [inner]
  float* act;               // [tokens][lda]: x | B | C after prep, then dt [n_heads], decay [n_heads]
  float* y_raw;             // [tokens][inner]
  void* out;                // [tokens][ldo] compute dtype
  float* state;             // [slots][state_stride]: S^T [n_heads][vdim][n_state], then the tail [taps - 1][channels]
  const int* token_pos;
  const int* token_seq;
  const int* seq_start;     // [seqs + 1]
  const int* seq_slot;      // [seqs]
  int ld, lda, ldo, n_tokens, n_seqs;
  int n_heads, vdim, n_state, n_groups, taps, norm_groups;
  int state_stride, write_state;
  float eps;
};

__device__ __forceinline__ float ss_silu(float z) { return z / (1.0f + expf(-z)); }

// ---------------------------------------------------------------- prep: a block per (token, stretch of channels)
#define SS_PREP_THREADS 256
__global__ void __launch_bounds__(SS_PREP_THREADS) ssm_prep_kernel(const SsmScan P) {
  pdl_trigger();
  pdl_wait();                // the projection and the state are the work of kernels before this one: ld_fresh
  const int t = blockIdx.x;
  const int inner = P.n_heads * P.vdim, C = inner + 2 * P.n_groups * P.n_state;
  const int item = blockIdx.y * SS_PREP_THREADS + threadIdx.x;      // a channel, or behind the channels a head
  if (item >= C + P.n_heads) return;
  float* out = P.act + (size_t)t * P.lda;
  if (item >= C) {
    const int h = item - C;
    const float z = ld_fresh(P.proj + (size_t)t * P.ld + inner + C + h) + P.dt_bias[h];
    const float dt = z > 20.f ? z : log1pf(expf(z));
    out[C + h] = dt;
    out[C + P.n_heads + h] = expf(-expf(P.a_log[h]) * dt);
    return;
  }
  const int c = item;
  const int seq = P.token_seq[t], pos = P.token_pos[t];
  int in_step = 0;           // tokens of this sequence that the step brought before this one
  const float* tail = nullptr;
  if (seq >= 0) {
    in_step = t - P.seq_start[seq];
    tail = P.state + (size_t)P.seq_slot[seq] * P.state_stride + (size_t)inner * P.n_state;
  }
  const int n = P.taps;
  const float* w = P.conv_w + (size_t)c * n;
  float acc = P.conv_b[c];
  for (int i = n - 1; i >= 0; i--) {                 // oldest input first: one fixed order
    float x = 0.f;
    if (i <= in_step) x = ld_fresh(P.proj + (size_t)(t - i) * P.ld + inner + c);
    else if (tail && pos - i >= 0) x = ld_fresh(tail + (size_t)(n - 1 - (i - in_step)) * C + c);
    acc = fmaf(w[n - 1 - i], x, acc);
  }
  out[c] = ss_silu(acc);
}

// ---------------------------------------------------------------- the recurrence
#define SS_THREADS 128
#define SS_HELD 16            // entries of S that a lane holds: R rows of Q columns
#define SS_MAX_CHUNK 8        // tokens staged in shared memory at a time, at most

__device__ __forceinline__ void ss_copy4(float* dst_shared, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void ss_copy16(float* dst_shared, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void ss_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void ss_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// The state of a head lies in memory column by column (S^T: [vdim][n_state]), so the rows a thread holds are
// contiguous.  A thread holds R rows of Q neighbouring columns (R Q = SS_HELD), and a group of L lanes covers the
// rows of its Q columns (n_state <= R L).  A 16-byte load from shared memory costs a quarter-warp one pass however
// many of its lanes share an address, so few rows per lane make every pass carry distinct words of B and C, and one
// load serves Q columns.  Per token a lane only leaves the Q partial read-outs of its rows in shared memory; when a
// chunk of tokens is through, the block adds them, a thread per (token, column), over the lanes in their order, with
// the skip term.  So the loop over tokens has no exchange between lanes, and its only chain is the state's own.
template <int L, int R>
__global__ void __launch_bounds__(SS_THREADS) ssm_recur_kernel(const SsmScan P) {
  constexpr int Q = SS_HELD / R;
  constexpr int COLS = SS_THREADS / L * Q;
  constexpr int PITCH = R == 4 ? 4 : R + 4;          // floats between two lanes' stretches of B and C: 16-byte
  constexpr int BC = L * PITCH;                      // aligned, and a quarter-warp's loads fall on distinct banks
  constexpr int WIDEST = BC > COLS ? BC : COLS;
  constexpr int FIT = 1024 / WIDEST;
  constexpr int CHUNK = FIT < 4 ? 4 : (FIT > SS_MAX_CHUNK ? SS_MAX_CHUNK : (FIT & ~3));
  constexpr int GROUPS = SS_THREADS / L;
  constexpr int PART_PITCH = (L + 1) * Q;            // floats between two groups' partial read-outs: banks spread
  __shared__ __align__(16) float bc_s[2][CHUNK][2][BC];
  __shared__ __align__(16) float x_s[2][CHUNK][COLS];
  __shared__ __align__(8) float dd_s[2][CHUNK][2];   // dt, decay
  __shared__ __align__(16) float part_s[CHUNK][GROUPS][PART_PITCH];
  pdl_trigger();             // (launched the ordinary way itself: it starts when prep is done)
  const int seq = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
  const int r0 = P.seq_start[seq], r1 = P.seq_start[seq + 1];
  if (r0 >= r1) return;
  const int N = P.n_state, V = P.vdim, inner = P.n_heads * V, GN = P.n_groups * N, C = inner + 2 * GN;
  const int part = threadIdx.x % L, grp = threadIdx.x / L;
  const int j0 = tile * COLS + grp * Q;              // the first of this lane's columns
  if (P.token_seq[r0] < 0) {                         // rows of no sequence: nothing is kept, the output is zero
    if (part == 0)
      for (int r = r0; r < r1; r++)
        for (int q = 0; q < Q; q++)
          if (j0 + q < V) P.y_raw[(size_t)r * inner + (size_t)h * V + j0 + q] = 0.f;
    return;
  }
  float* slot = P.state + (size_t)P.seq_slot[seq] * P.state_stride;

  // the convolution's tail moves on by this step's tokens: the blocks of a sequence share the channels, a thread
  // takes a channel through time in order, so that an entry is read before it is overwritten
  if (P.write_state && P.taps > 1) {
    float* tail = slot + (size_t)inner * N;
    const int keep = P.taps - 1, n_new = r1 - r0;
    const int n_blocks = gridDim.x * gridDim.y, me = blockIdx.y * gridDim.x + blockIdx.x;
    const int per = (C + n_blocks - 1) / n_blocks;
    const int c_end = min(C, (me + 1) * per);
    for (int c = me * per + threadIdx.x; c < c_end; c += SS_THREADS)
      for (int i = 0; i < keep; i++) {
        const int back = keep - i;                   // this entry is the input `back` tokens before the next one
        tail[(size_t)i * C + c] = back <= n_new ? P.proj[(size_t)(r1 - back) * P.ld + inner + c]
                                                : tail[(size_t)(i + n_new) * C + c];
      }
  }

  const int g = h / (P.n_heads / P.n_groups);
  const float d_skip = P.d_skip[h];
  float* Sg = slot + ((size_t)h * V + j0) * N + part * R;              // column q of this lane: + q N
  const bool vec = N % 4 == 0 && (P.state_stride % 4) == 0 && (((uintptr_t)P.state) & 15) == 0;
  float2 S[Q][R / 2];
#pragma unroll
  for (int q = 0; q < Q; q++) {
    const bool live = j0 + q < V;
#pragma unroll
    for (int i = 0; i < R; i += 4) {
      const int d = part * R + i;
      if (live && vec && d + 3 < N) {
        const float4 v4 = *reinterpret_cast<const float4*>(Sg + (size_t)q * N + i);
        S[q][i / 2] = make_float2(v4.x, v4.y); S[q][i / 2 + 1] = make_float2(v4.z, v4.w);
      } else {
        float e[4];
#pragma unroll
        for (int u = 0; u < 4; u++) e[u] = (live && d + u < N) ? Sg[(size_t)q * N + i + u] : 0.f;
        S[q][i / 2] = make_float2(e[0], e[1]); S[q][i / 2 + 1] = make_float2(e[2], e[3]);
      }
    }
  }
  // rows beyond n_state and columns beyond vdim stay zero in the staging buffers: nothing below writes them
  if (N != R * L || (tile + 1) * COLS > V) {
    for (int i = threadIdx.x; i < 2 * CHUNK * 2 * BC; i += SS_THREADS) (&bc_s[0][0][0][0])[i] = 0.f;
    for (int i = threadIdx.x; i < 2 * CHUNK * COLS; i += SS_THREADS) (&x_s[0][0][0])[i] = 0.f;
    __syncthreads();
  }

  const bool vec_act = N % 4 == 0 && P.lda % 4 == 0 && inner % 4 == 0 && (((uintptr_t)P.act) & 15) == 0;
  auto stage = [&](int buf, int c0) {                // ask for the tokens c0 .. of this sequence
    const int n_here = min(CHUNK, r1 - c0);
    for (int tok = 0; tok < n_here; tok++) {
      const float* a = P.act + (size_t)(c0 + tok) * P.lda + inner + (size_t)g * N;
      if (vec_act) {
        for (int d = 4 * threadIdx.x; d < 2 * N; d += 4 * SS_THREADS) {          // B, then C
          const int which = d >= N, dd = d - which * N;
          ss_copy16(&bc_s[buf][tok][which][(dd / R) * PITCH + dd % R], a + which * GN + dd);
        }
      } else {
        for (int d = threadIdx.x; d < 2 * N; d += SS_THREADS) {
          const int which = d >= N, dd = d - which * N;
          ss_copy4(&bc_s[buf][tok][which][(dd / R) * PITCH + dd % R], a + which * GN + dd);
        }
      }
    }
    for (int i = threadIdx.x; i < n_here * COLS; i += SS_THREADS) {
      const int tok = i / COLS, cc = i - tok * COLS, jj = tile * COLS + cc;
      if (jj < V) ss_copy4(&x_s[buf][tok][cc], P.act + (size_t)(c0 + tok) * P.lda + (size_t)h * V + jj);
    }
    if (threadIdx.x < n_here * 2) {
      const int tok = threadIdx.x >> 1, which = threadIdx.x & 1;                 // 0 = dt, 1 = decay
      ss_copy4(&dd_s[buf][tok][which], P.act + (size_t)(c0 + tok) * P.lda + C + which * P.n_heads + h);
    }
    ss_commit();
  };

  stage(0, r0);
  int buf = 0;
  for (int c0 = r0; c0 < r1; c0 += CHUNK, buf ^= 1) {
    ss_wait_all();
    __syncthreads();                                 // this chunk has landed, and the other buffer is free again
    if (c0 + CHUNK < r1) stage(buf ^ 1, c0 + CHUNK);
    const int n_here = min(CHUNK, r1 - c0);
    auto token = [&](int tok) {                      // one token of the chunk: the state moves on, partials out
      const float4* bb = reinterpret_cast<const float4*>(&bc_s[buf][tok][0][part * PITCH]);
      const float4* cc = reinterpret_cast<const float4*>(&bc_s[buf][tok][1][part * PITCH]);
      float4 b4[R / 4], c4[R / 4];
#pragma unroll
      for (int i = 0; i < R / 4; i++) { b4[i] = bb[i]; c4[i] = cc[i]; }
      const float2 dd = *reinterpret_cast<const float2*>(&dd_s[buf][tok][0]);
      const float2 dk = make_float2(dd.y, dd.y);
      float xq[Q], y[Q];
      if constexpr (Q == 4) {
        const float4 x4 = *reinterpret_cast<const float4*>(&x_s[buf][tok][grp * Q]);
        xq[0] = x4.x; xq[1] = x4.y; xq[2] = x4.z; xq[3] = x4.w;
      } else if constexpr (Q == 2) {
        const float2 x2 = *reinterpret_cast<const float2*>(&x_s[buf][tok][grp * Q]);
        xq[0] = x2.x; xq[1] = x2.y;
      } else {
        xq[0] = x_s[buf][tok][grp];
      }
#pragma unroll
      for (int q = 0; q < Q; q++) {
        const float dtx = dd.x * xq[q];
        const float2 uu = make_float2(dtx, dtx);
        float2 a0 = make_float2(0.f, 0.f), a1 = a0;
#pragma unroll
        for (int i = 0; i < R / 4; i++) {
          S[q][2 * i] = __ffma2_rn(make_float2(b4[i].x, b4[i].y), uu, __fmul2_rn(dk, S[q][2 * i]));
          S[q][2 * i + 1] = __ffma2_rn(make_float2(b4[i].z, b4[i].w), uu, __fmul2_rn(dk, S[q][2 * i + 1]));
          a0 = __ffma2_rn(S[q][2 * i], make_float2(c4[i].x, c4[i].y), a0);
          a1 = __ffma2_rn(S[q][2 * i + 1], make_float2(c4[i].z, c4[i].w), a1);
        }
        const float2 s2 = __fadd2_rn(a0, a1);
        y[q] = s2.x + s2.y;
      }
      float* mine = &part_s[tok][grp][part * Q];
      if constexpr (Q == 4) *reinterpret_cast<float4*>(mine) = make_float4(y[0], y[1], y[2], y[3]);
      else if constexpr (Q == 2) *reinterpret_cast<float2*>(mine) = make_float2(y[0], y[1]);
      else *mine = y[0];
    };
    if (n_here == CHUNK) {                           // a whole chunk: the tokens' loads and sums interleave
#pragma unroll
      for (int tok = 0; tok < CHUNK; tok++) token(tok);
    } else {
      for (int tok = 0; tok < n_here; tok++) token(tok);
    }
    __syncthreads();                                 // the chunk's partial read-outs are all there
    for (int o = threadIdx.x; o < n_here * COLS; o += SS_THREADS) {
      const int tok = o / COLS, c = o - tok * COLS;
      const float* p = &part_s[tok][c / Q][c % Q];
      float y = 0.f;
#pragma unroll
      for (int l = 0; l < L; l++) y += p[l * Q];
      if (tile * COLS + c < V)
        P.y_raw[(size_t)(c0 + tok) * inner + (size_t)h * V + tile * COLS + c] = fmaf(d_skip, x_s[buf][tok][c], y);
    }
  }
  if (P.write_state) {
#pragma unroll
    for (int q = 0; q < Q; q++) {
      if (j0 + q >= V) continue;
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        const int d = part * R + i;
        const float e[4] = {S[q][i / 2].x, S[q][i / 2].y, S[q][i / 2 + 1].x, S[q][i / 2 + 1].y};
        if (vec && d + 3 < N) {
          *reinterpret_cast<float4*>(Sg + (size_t)q * N + i) = make_float4(e[0], e[1], e[2], e[3]);
        } else {
#pragma unroll
          for (int u = 0; u < 4; u++)
            if (d + u < N) Sg[(size_t)q * N + i + u] = e[u];
        }
      }
    }
  }
}

// ---------------------------------------------------------------- finish: a block per (token, part of the row)
// The sum of squares is added in an order that the part's size alone fixes: a thread over its strided entries, a
// warp by shuffles, the warps one after another.
#define SS_FIN_THREADS 128
template <typename T>
__global__ void __launch_bounds__(SS_FIN_THREADS) ssm_finish_kernel(const SsmScan P) {
  __shared__ float warp_ss[SS_FIN_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_trigger();
  pdl_wait();                // y_raw and the projection are the work of kernels before this one: ld_fresh
  const long long item = blockIdx.x;
  const int t = (int)(item / P.norm_groups), part = (int)(item - (long long)t * P.norm_groups);
  const int inner = P.n_heads * P.vdim, size = inner / P.norm_groups;
  const float* y = P.y_raw + (size_t)t * inner + (size_t)part * size;
  const float* z = P.proj + (size_t)t * P.ld + (size_t)part * size;
  const float* gain = P.gain + (size_t)part * size;
  T* out = (T*)P.out + (size_t)t * P.ldo + (size_t)part * size;
  constexpr int KEEP = 4;    // entries a thread keeps between the two passes (parts of up to 512 are read once)
  float kept[KEEP];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < KEEP; i++) {
    const int d = threadIdx.x + i * SS_FIN_THREADS;
    kept[i] = d < size ? ld_fresh(y + d) * ss_silu(ld_fresh(z + d)) : 0.f;
    ss = fmaf(kept[i], kept[i], ss);
  }
  for (int d = threadIdx.x + KEEP * SS_FIN_THREADS; d < size; d += SS_FIN_THREADS) {
    const float v = ld_fresh(y + d) * ss_silu(ld_fresh(z + d));
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if (lane == 0) warp_ss[warp] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < SS_FIN_THREADS / 32; i++) total += warp_ss[i];
  const float mul = 1.0f / sqrtf(total / (float)size + P.eps);
#pragma unroll
  for (int i = 0; i < KEEP; i++) {
    const int d = threadIdx.x + i * SS_FIN_THREADS;
    if (d < size) out[d] = from_float<T>(kept[i] * mul * gain[d]);
  }
  for (int d = threadIdx.x + KEEP * SS_FIN_THREADS; d < size; d += SS_FIN_THREADS)
    out[d] = from_float<T>(ld_fresh(y + d) * ss_silu(ld_fresh(z + d)) * mul * gain[d]);
}

static int ssm_check(const SsmScan& P) {
  if (P.n_heads < 1 || P.n_groups < 1 || P.n_heads % P.n_groups != 0 || P.vdim < 1 || P.n_state < 1 || P.taps < 1)
    return STRATUM_ERR_SHAPE;
  const int inner = P.n_heads * P.vdim, C = inner + 2 * P.n_groups * P.n_state;
  if (P.norm_groups < 1 || inner % P.norm_groups != 0) return STRATUM_ERR_SHAPE;
  if (P.ld < inner + C + P.n_heads || P.lda < C + 2 * P.n_heads || P.ldo < inner) return STRATUM_ERR_SHAPE;
  if ((long long)P.state_stride < (long long)inner * P.n_state + (long long)(P.taps - 1) * C) return STRATUM_ERR_SHAPE;
  if (P.n_state > 32 * SS_HELD) return STRATUM_ERR_LIMIT;
  if (P.n_heads > 65535 || P.n_seqs > 65535) return STRATUM_ERR_LIMIT;
  return 0;
}

template <int L, int R>
static void ssm_recur_launch(const SsmScan& P, cudaStream_t stream) {
  const int cols = SS_THREADS / L * (SS_HELD / R);
  const dim3 grid((P.vdim + cols - 1) / cols, P.n_heads, P.n_seqs);
  ssm_recur_kernel<L, R><<<grid, SS_THREADS, 0, stream>>>(P);
}

// Everything of a step: prep, recurrence, finish (three launches).  out_dtype: the compute dtype of `out`.
STRATUM_EXPORT int stratum_ssm_scan(const SsmScan* params, int out_dtype, cudaStream_t stream) {
  const SsmScan& P = *params;
  if (P.n_tokens <= 0 || P.n_seqs <= 0) return 0;
  const int bad = ssm_check(P);
  if (bad) return bad;
  {
    const int inner = P.n_heads * P.vdim, items = inner + 2 * P.n_groups * P.n_state + P.n_heads;
    launch_pdl(ssm_prep_kernel, dim3(P.n_tokens, (items + SS_PREP_THREADS - 1) / SS_PREP_THREADS), SS_PREP_THREADS, 0,
               stream, P);
  }
  int st = launch_status();
  if (st) return st;
  // few rows per lane while a warp still covers the rows: 4 up to 128 rows, 8 up to 256, 16 beyond
  if (P.n_state > 256) ssm_recur_launch<32, 16>(P, stream);
  else if (P.n_state > 128) ssm_recur_launch<32, 8>(P, stream);
  else {
    int L = 1;
    while (4 * L < P.n_state) L <<= 1;
    switch (L) {
      case 1: ssm_recur_launch<1, 4>(P, stream); break;
      case 2: ssm_recur_launch<2, 4>(P, stream); break;
      case 4: ssm_recur_launch<4, 4>(P, stream); break;
      case 8: ssm_recur_launch<8, 4>(P, stream); break;
      case 16: ssm_recur_launch<16, 4>(P, stream); break;
      default: ssm_recur_launch<32, 4>(P, stream); break;
    }
  }
  st = launch_status();
  if (st) return st;
  const long long blocks = (long long)P.n_tokens * P.norm_groups;
  if (blocks > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  if (out_dtype == STRATUM_DT_F32) launch_pdl(ssm_finish_kernel<float>, (unsigned)blocks, SS_FIN_THREADS, 0, stream, P);
  else if (out_dtype == STRATUM_DT_BF16) launch_pdl(ssm_finish_kernel<bf16>, (unsigned)blocks, SS_FIN_THREADS, 0, stream, P);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}
