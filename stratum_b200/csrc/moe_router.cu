// Routing of a mixture of experts, in float32, and the weighting of the experts' activations.
//
// route: per token, z = W_r h (h in the compute dtype, W_r and the sums float32); s = sigmoid(z); the choice score of
//   expert e is c_e = s_e + correction_e.  The experts form `n_groups` equal groups of neighbours; a group's score is
//   the sum of its two largest c (of its only c when a group is one expert); only the `keep` best groups stay (the
//   others' c count as -inf).  The `top` experts with the largest c are chosen (among equals the lowest index), and
//   their weights are s_e / (sum of the chosen s + 1e-20) * scale.  Written: the chosen experts and their weights
//   [tokens][top], and the same as a row of n_experts weights with zeros for the others.
//   One block per token; a sum's order depends on the row's length alone.
//   Variants, all parameters: score = 1 takes s = softmax(z) over all experts in sigmoid's place; renorm = 0 leaves
//   the chosen scores as they are (weight s_e * scale); correction may be absent; with w_gate (one more row of
//   `width` weights) the token's sigmoid(w_gate . h) is written behind the experts' weights, dense[t][n_experts]:
//   the gate of a shared expert; with `bias` the logits are z = W_r h + bias.  (Softmax scores divided by the sum of
//   the chosen ones are the softmax over the chosen logits alone.)
// scale_column_blocks: a[t][e * block + j] *= w[t][e] for e < n_blocks (columns beyond n_blocks * block are left
//   alone): the activations of every expert, side by side in one row, times the token's weight for that expert, so
//   that one product with the experts' stacked down matrices sums the weighted expert outputs.
// group / gather / combine: the other way to run the experts, for steps of many tokens: the (token, choice) pairs are
//   put in the order of their experts (within an expert in the order of the tokens: a stable counting sort, one block
//   per expert), the tokens' rows are gathered in that order, every expert runs on its own stretch of rows, and each
//   token adds up its experts' outputs times its weights, in the order of its choices.
#include <math.h>

#include "common.cuh"

struct MoeRoute {
  const void* x;            // [tokens][ldx]
  const float* w_router;    // [n_experts][width]
  const float* correction;  // [n_experts]
  float* dense;             // [tokens][ldd] weights, zeros for experts not chosen
  int* chosen;              // [tokens][top]
  float* weights;           // [tokens][top]
  int ldx, ldd, n_tokens, width;
  int n_experts, top, n_groups, keep;
  float scale, reserved;
  const float* w_gate;      // [width] or null
  int score, renorm;        // score: 0 sigmoid, 1 softmax over all experts;  renorm: weights divided by their sum
  const float* bias;        // [n_experts] or null: added to the logits z before anything else
};

#define MR_WARPS 8

// one block per token: the warps share the experts' dot products (warp w takes experts w, w + 8, ...; a lane's partial
// sum runs over its elements in order, four at a time where the rows are aligned), then warp 0 chooses
template <typename T>
__global__ void __launch_bounds__(MR_WARPS * 32) moe_route_kernel(const MoeRoute P) {
  extern __shared__ float mr_s[];                    // s [E], c [E], group score [n_groups]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();                                        // x is the work of a kernel before this one: ld_fresh
  const int t = blockIdx.x;
  const int E = P.n_experts, G = P.n_groups, per = E / G;
  float* s = mr_s;
  float* c = s + E;
  float* gs = c + E;
  const T* x = (const T*)P.x + (size_t)t * P.ldx;
  const bool vec = P.width % 4 == 0 && (((uintptr_t)x | (uintptr_t)P.w_router | (uintptr_t)P.w_gate) & 15) == 0 &&
                   (P.ldx * sizeof(T)) % 16 == 0;
  const int n_rows = E + (P.w_gate ? 1 : 0);         // the gate of a shared expert is one more row
  for (int e = warp; e < n_rows; e += MR_WARPS) {
    const float* w = e < E ? P.w_router + (size_t)e * P.width : P.w_gate;
    float acc = 0.f;
    if (vec) {
      // four stretches of four elements in flight per lane, each with a sum of its own; the sums are added in one
      // fixed order, which depends on the row's length alone
      auto x4 = [&](int i, float& x0, float& x1, float& x2, float& x3) {
        if constexpr (sizeof(T) == 4) {
          const float4 xv = ld_fresh(reinterpret_cast<const float4*>(x + i));
          x0 = xv.x; x1 = xv.y; x2 = xv.z; x3 = xv.w;
        } else {
          const uint2 xv = __ldcg(reinterpret_cast<const uint2*>(x + i));
          const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&xv.x);
          const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&xv.y);
          x0 = __low2float(lo); x1 = __high2float(lo); x2 = __low2float(hi); x3 = __high2float(hi);
        }
      };
      float part[4] = {0.f, 0.f, 0.f, 0.f};
      for (int i0 = lane * 4; i0 < P.width; i0 += 512) {
        float4 wv[4];
        float xs[4][4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int i = i0 + 128 * u;
          wv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          xs[u][0] = xs[u][1] = xs[u][2] = xs[u][3] = 0.f;
          if (i < P.width) {
            wv[u] = *reinterpret_cast<const float4*>(w + i);
            x4(i, xs[u][0], xs[u][1], xs[u][2], xs[u][3]);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
          part[u] = fmaf(xs[u][0], wv[u].x, part[u]); part[u] = fmaf(xs[u][1], wv[u].y, part[u]);
          part[u] = fmaf(xs[u][2], wv[u].z, part[u]); part[u] = fmaf(xs[u][3], wv[u].w, part[u]);
        }
      }
      acc = (part[0] + part[1]) + (part[2] + part[3]);
    } else {
      for (int i = lane; i < P.width; i += 32) acc = fmaf(ld_fresh(x + i), w[i], acc);
    }
    acc = warp_sum(acc);
    if (P.bias && e < E) acc += P.bias[e];
    if (lane == 0) {
      const float sg = 1.0f / (1.0f + expf(-acc));
      if (e == E) {
        P.dense[(size_t)t * P.ldd + E] = sg;
      } else if (P.score == 1) {
        s[e] = acc;                                  // the logit; the softmax follows once all are there
      } else {
        s[e] = sg;
        c[e] = sg + (P.correction ? P.correction[e] : 0.f);
      }
    }
  }
  __syncthreads();
  if (warp != 0) return;
  if (P.score == 1) {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, s[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float v = expf(s[e] - m);
      s[e] = v;
      sum += v;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) {
      const float v = s[e] / sum;
      s[e] = v;
      c[e] = v + (P.correction ? P.correction[e] : 0.f);
    }
    __syncwarp();
  }
  // group scores, then all but the `keep` best groups are closed
  for (int g = lane; g < G; g += 32) {
    float a = -INFINITY, b = -INFINITY;              // the two largest
    for (int i = 0; i < per; i++) {
      const float v = c[g * per + i];
      if (v > a) { b = a; a = v; } else if (v > b) b = v;
    }
    gs[g] = per > 1 ? a + b : a;
  }
  __syncwarp();
  if (P.keep < G) {
    for (int g = lane; g < G; g += 32) {
      int better = 0;                                // groups ahead of g: a larger score, or the same and a lower index
      for (int o = 0; o < G; o++) better += (gs[o] > gs[g]) || (gs[o] == gs[g] && o < g);
      if (better >= P.keep)
        for (int i = 0; i < per; i++) c[g * per + i] = -INFINITY;
    }
    __syncwarp();
  }
  float* dense = P.dense + (size_t)t * P.ldd;
  for (int e = lane; e < E; e += 32) dense[e] = 0.f;
  __syncwarp();
  float total = 0.f;
  for (int k = 0; k < P.top; k++) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (c[e] > best) { best = c[e]; at = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = 0;                    // fewer open experts than `top` (refused by the host)
    total += s[at];
    if (lane == 0) {
      P.chosen[(size_t)t * P.top + k] = at;
      c[at] = -INFINITY;
    }
    __syncwarp();
  }
  const float mul = P.renorm ? P.scale / (total + 1e-20f) : P.scale;
  for (int k = lane; k < P.top; k += 32) {
    const int e = P.chosen[(size_t)t * P.top + k];
    const float w = s[e] * mul;
    P.weights[(size_t)t * P.top + k] = w;
    dense[e] = w;
  }
}

STRATUM_EXPORT int stratum_moe_route(const MoeRoute* params, int dtype, cudaStream_t stream) {
  const MoeRoute& P = *params;
  if (P.n_tokens <= 0) return 0;
  if (P.n_experts < 1 || P.n_groups < 1 || P.n_experts % P.n_groups != 0 || P.keep < 1 || P.keep > P.n_groups ||
      P.top < 1 || P.top > (P.n_experts / P.n_groups) * P.keep || P.ldd < P.n_experts + (P.w_gate ? 1 : 0) ||
      P.ldx < P.width)
    return STRATUM_ERR_SHAPE;
  const size_t smem = (size_t)(2 * P.n_experts + P.n_groups) * sizeof(float);
  if (smem > 48 * 1024) return STRATUM_ERR_LIMIT;
  const int blocks = P.n_tokens;
  if (dtype == STRATUM_DT_F32) launch_pdl(moe_route_kernel<float>, blocks, MR_WARPS * 32, smem, stream, P);
  else if (dtype == STRATUM_DT_BF16) launch_pdl(moe_route_kernel<bf16>, blocks, MR_WARPS * 32, smem, stream, P);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}

// a thread takes eight neighbouring columns of one row (they lie in one expert's stretch when `block` is a multiple
// of eight; otherwise, and for rows that are not 16-byte aligned, column by column)
template <typename T>
__global__ void scale_column_blocks_kernel(T* a, int lda, const float* w, int ldw, int n_rows, int block, int n_blocks,
                                           int vec) {
  pdl_trigger();
  pdl_wait();                                        // a and w are the work of kernels before this one: ld_fresh
  const int cols = block * n_blocks;
  const int per_row = (cols + 7) / 8;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n_rows * per_row) return;
  const int r = (int)(i / per_row), c0 = (int)(i - (long long)r * per_row) * 8;
  T* p = a + (size_t)r * lda + c0;
  const float* wr = w + (size_t)r * ldw;
  if (vec && c0 + 8 <= cols) {
    const float f = ld_fresh(wr + c0 / block);
    if constexpr (sizeof(T) == 2) {
      uint4 v = ld_fresh(reinterpret_cast<const uint4*>(p));
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int u = 0; u < 4; u++) h[u] = __floats2bfloat162_rn(__low2float(h[u]) * f, __high2float(h[u]) * f);
      *reinterpret_cast<uint4*>(p) = v;
    } else {
      float4* q = reinterpret_cast<float4*>(p);
      float4 x = ld_fresh(q), y = ld_fresh(q + 1);
      q[0] = make_float4(x.x * f, x.y * f, x.z * f, x.w * f);
      q[1] = make_float4(y.x * f, y.y * f, y.z * f, y.w * f);
    }
    return;
  }
  for (int c = c0; c < min(c0 + 8, cols); c++)
    p[c - c0] = from_float<T>(ld_fresh((const T*)p + (c - c0)) * ld_fresh(wr + c / block));
}

STRATUM_EXPORT int stratum_scale_column_blocks(void* a, int dtype, int lda, const float* w, int ldw, int n_rows,
                                               int block, int n_blocks, cudaStream_t stream) {
  if (n_rows <= 0 || n_blocks <= 0) return 0;
  if (block < 1 || lda < block * n_blocks || ldw < n_blocks) return STRATUM_ERR_SHAPE;
  const long long n = (long long)n_rows * ((block * n_blocks + 7) / 8);
  const long long blocks = (n + 255) / 256;
  if (blocks > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  const int elem = dtype == STRATUM_DT_F32 ? 4 : 2;
  const int vec = block % 8 == 0 && ((size_t)lda * elem) % 16 == 0 && ((uintptr_t)a & 15) == 0;
  if (dtype == STRATUM_DT_F32)
    launch_pdl(scale_column_blocks_kernel<float>, (unsigned)blocks, 256, 0, stream, (float*)a, lda, w, ldw, n_rows,
               block, n_blocks, vec);
  else if (dtype == STRATUM_DT_BF16)
    launch_pdl(scale_column_blocks_kernel<bf16>, (unsigned)blocks, 256, 0, stream, (bf16*)a, lda, w, ldw, n_rows, block,
               n_blocks, vec);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}

// ---------------------------------------------------------------- grouping the (token, choice) pairs by expert
#define MG_THREADS 256

__global__ void __launch_bounds__(MG_THREADS) moe_count_kernel(const int* __restrict__ chosen, int n, int* counts) {
  __shared__ float scratch[33];
  const int e = blockIdx.x;
  float c = 0.f;                                       // exact in float32 up to 2^24 pairs
  for (int i = threadIdx.x; i < n; i += MG_THREADS) c += chosen[i] == e ? 1.f : 0.f;
  c = block_sum(c, scratch);
  if (threadIdx.x == 0) counts[e] = (int)c;
}

// order[r] = the pair (token * top + choice) that stands at place r; where[pair] = its place.
__global__ void __launch_bounds__(MG_THREADS) moe_place_kernel(const int* __restrict__ chosen, int n,
                                                               const int* __restrict__ counts, int* order, int* where) {
  __shared__ int warp_n[MG_THREADS / 32];
  __shared__ int base_s;
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    int off = 0;
    for (int o = 0; o < e; o++) off += counts[o];
    base_s = off;
  }
  __syncthreads();
  int base = base_s;
  for (int i0 = 0; i0 < n; i0 += MG_THREADS) {
    const int i = i0 + threadIdx.x;
    const bool mine = i < n && chosen[i] == e;
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) warp_n[warp] = __popc(m);
    __syncthreads();
    int before = 0, total = 0;
    for (int w = 0; w < MG_THREADS / 32; w++) {
      if (w < warp) before += warp_n[w];
      total += warp_n[w];
    }
    if (mine) {
      const int r = base + before + __popc(m & ((1u << lane) - 1u));
      order[r] = i;
      where[i] = r;
    }
    base += total;
    __syncthreads();
  }
}

STRATUM_EXPORT int stratum_moe_group(const int* chosen, int n_pairs, int n_experts, int* counts, int* order, int* where,
                                     cudaStream_t stream) {
  if (n_pairs <= 0 || n_experts <= 0) return 0;
  if (n_pairs > (1 << 24)) return STRATUM_ERR_LIMIT;
  moe_count_kernel<<<n_experts, MG_THREADS, 0, stream>>>(chosen, n_pairs, counts);
  int st = launch_status();
  if (st) return st;
  moe_place_kernel<<<n_experts, MG_THREADS, 0, stream>>>(chosen, n_pairs, counts, order, where);
  return launch_status();
}

// out[r] = x[order[r] / top]: the rows of the tokens in the order of their experts.
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, int ldx, const int* __restrict__ order, int top, T* out,
                                   int width) {
  const int r = blockIdx.x;
  const T* src = x + (size_t)(order[r] / top) * ldx;
  T* dst = out + (size_t)r * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

STRATUM_EXPORT int stratum_gather_rows(const void* x, int dtype, int ldx, const int* order, int top, void* out, int n_rows,
                                       int width, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (top < 1 || width < 1 || ldx < width) return STRATUM_ERR_SHAPE;
  if (dtype == STRATUM_DT_F32)
    gather_rows_kernel<float><<<n_rows, 256, 0, stream>>>((const float*)x, ldx, order, top, (float*)out, width);
  else if (dtype == STRATUM_DT_BF16)
    gather_rows_kernel<bf16><<<n_rows, 256, 0, stream>>>((const bf16*)x, ldx, order, top, (bf16*)out, width);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}

// y[t] (+)= sum_k weights[t][k] * outs[where[t * top + k]], float32, the choices in their order.
__global__ void moe_combine_kernel(const float* __restrict__ outs, const int* __restrict__ where,
                                   const float* __restrict__ weights, float* y, int top, int width, int accumulate) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float acc = accumulate ? y[(size_t)t * width + i] : 0.f;
    for (int k = 0; k < top; k++)
      acc = fmaf(weights[(size_t)t * top + k], outs[(size_t)where[(size_t)t * top + k] * width + i], acc);
    y[(size_t)t * width + i] = acc;
  }
}

STRATUM_EXPORT int stratum_moe_combine(const float* outs, const int* where, const float* weights, float* y, int n_tokens,
                                       int top, int width, int accumulate, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (top < 1 || width < 1) return STRATUM_ERR_SHAPE;
  moe_combine_kernel<<<n_tokens, 256, 0, stream>>>(outs, where, weights, y, top, width, accumulate);
  return launch_status();
}
