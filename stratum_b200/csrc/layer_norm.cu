// Layer norm with a weight and no bias, on the float32 residual stream:
//   LN(v) = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * gain.
//
//   layernorm                 out[r] = LN(x[rows[r]] or x[r]), float32 in, compute dtype out (the norm in front of a
//                             sublayer, or the model's last norm on the wanted rows).
//   layernorm_into_residual   x[r] (+)= LN(y[r]) (the norm behind a sublayer; its gain may carry the layer's residual
//                             factor), and, where asked, next_out[r] = LN'(x[r]) of the new row with a second gain: the
//                             norm in front of the next sublayer, taken while the row is still in shared memory, so
//                             that the stream is read and written once between two sublayers.
//
// One block per row, the row held in shared memory; mean first, then the squared deviations from it.  The block's
// shape follows from the row's length alone, so every sum has one order whatever the step's size.
#include "common.cuh"

template <bool VEC>
__device__ __forceinline__ void ln_load(const float* src, float* row, int hidden) {
  if (VEC) {
    for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x)
      reinterpret_cast<float4*>(row)[i] = ld_fresh(reinterpret_cast<const float4*>(src) + i);
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) row[i] = ld_fresh(src + i);
  }
}

// Sum over the block with one barrier: the warps' sums go to `slots` (32 floats that nothing else uses in this
// launch), and every thread adds them in the warps' order.
__device__ __forceinline__ float ln_block_sum(float v, float* slots) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) slots[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < n_warps; w++) t += slots[w];
  return t;
}

// (mean, 1 / sqrt(var + eps)) of the row in shared memory; every thread gets both.  scratch: 64 floats of its own.
template <bool VEC>
__device__ __forceinline__ float2 ln_stats(const float* row, int hidden, float eps, float* scratch) {
  float s = 0.f;
  if (VEC) {
    for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x) {
      const float4 v = reinterpret_cast<const float4*>(row)[i];
      s += (v.x + v.y) + (v.z + v.w);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) s += row[i];
  }
  const float mean = ln_block_sum(s, scratch) / (float)hidden;
  float q = 0.f;
  if (VEC) {
    for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x) {
      const float4 v = reinterpret_cast<const float4*>(row)[i];
      const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
      q += fmaf(a, a, b * b) + fmaf(c, c, d * d);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float d = row[i] - mean;
      q = fmaf(d, d, q);
    }
  }
  const float var = ln_block_sum(q, scratch + 32) / (float)hidden;
  return make_float2(mean, 1.0f / sqrtf(var + eps));
}

// (v - mean) * rstd * gain for four neighbours
__device__ __forceinline__ float4 ln_apply(float4 v, float2 st, float4 g) {
  return make_float4((v.x - st.x) * st.y * g.x, (v.y - st.x) * st.y * g.y, (v.z - st.x) * st.y * g.z,
                     (v.w - st.x) * st.y * g.w);
}
__device__ __forceinline__ void ln_store4(float* o, float4 v) { *reinterpret_cast<float4*>(o) = v; }
__device__ __forceinline__ void ln_store4(bf16* o, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const unsigned*>(&lo);
  u.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(o) = u;
}

template <typename T, bool VEC>
__global__ void layernorm_kernel(const float* x, const float* __restrict__ gain, const int* __restrict__ rows, T* out,
                                 int hidden, float eps) {
  extern __shared__ __align__(16) float ln_row[];
  __shared__ float scratch[128];
  pdl_trigger();
  const int r = blockIdx.x;
  pdl_wait();                                        // x (and rows) are the work of kernels before this one
  const int src = rows ? __ldcg(rows + r) : r;
  ln_load<VEC>(x + (size_t)src * hidden, ln_row, hidden);
  __syncthreads();
  const float2 st = ln_stats<VEC>(ln_row, hidden, eps, scratch);
  T* o = out + (size_t)r * hidden;
  if (VEC) {
    for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x)
      ln_store4(o + 4 * i, ln_apply(reinterpret_cast<const float4*>(ln_row)[i], st,
                                    __ldg(reinterpret_cast<const float4*>(gain) + i)));
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<T>((ln_row[i] - st.x) * st.y * gain[i]);
  }
}

#define LN_AHEAD 4
template <typename T, bool VEC>
__global__ void layernorm_into_residual_kernel(const float* y, const float* __restrict__ gain, float* x,
                                               const float* __restrict__ next_gain, T* next_out, int hidden, float eps,
                                               float next_eps, int accumulate) {
  extern __shared__ __align__(16) float ln_row[];
  __shared__ float scratch[128];
  pdl_trigger();
  pdl_wait();
  const size_t at = (size_t)blockIdx.x * hidden;
  float* xr = x + at;
  // the stream's row is asked for together with y's, so that one wait on memory covers both (rows of up to
  // LN_AHEAD x 4 x blockDim numbers; longer ones read it where they need it)
  float4 ahead[LN_AHEAD];
  const bool early = VEC && accumulate && hidden / 4 <= LN_AHEAD * (int)blockDim.x;
  if (early) {
#pragma unroll
    for (int k = 0; k < LN_AHEAD; k++) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < hidden / 4) ahead[k] = ld_fresh(reinterpret_cast<const float4*>(xr) + i);
    }
  }
  ln_load<VEC>(y + at, ln_row, hidden);
  __syncthreads();
  const float2 st = ln_stats<VEC>(ln_row, hidden, eps, scratch);
  if (VEC && early) {                                            // a thread rewrites the entries it reads
#pragma unroll
    for (int k = 0; k < LN_AHEAD; k++) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < hidden / 4) {
        float4 v = ln_apply(reinterpret_cast<const float4*>(ln_row)[i], st,
                            __ldg(reinterpret_cast<const float4*>(gain) + i));
        v.x += ahead[k].x; v.y += ahead[k].y; v.z += ahead[k].z; v.w += ahead[k].w;
        reinterpret_cast<float4*>(xr)[i] = v;
        reinterpret_cast<float4*>(ln_row)[i] = v;
      }
    }
  } else if (VEC) {
    for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x) {
      float4 v = ln_apply(reinterpret_cast<const float4*>(ln_row)[i], st,
                          __ldg(reinterpret_cast<const float4*>(gain) + i));
      if (accumulate) {
        const float4 was = ld_fresh(reinterpret_cast<const float4*>(xr) + i);
        v.x += was.x; v.y += was.y; v.z += was.z; v.w += was.w;
      }
      reinterpret_cast<float4*>(xr)[i] = v;
      reinterpret_cast<float4*>(ln_row)[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = (ln_row[i] - st.x) * st.y * gain[i];
      if (accumulate) v += ld_fresh(xr + i);
      xr[i] = v;
      ln_row[i] = v;
    }
  }
  if (next_out == nullptr) return;
  __syncthreads();
  const float2 nx = ln_stats<VEC>(ln_row, hidden, next_eps, scratch + 64);
  T* o = next_out + at;
  if (VEC) {
    for (int i = threadIdx.x; i < hidden / 4; i += blockDim.x)
      ln_store4(o + 4 * i, ln_apply(reinterpret_cast<const float4*>(ln_row)[i], nx,
                                    __ldg(reinterpret_cast<const float4*>(next_gain) + i)));
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      o[i] = from_float<T>((ln_row[i] - nx.x) * nx.y * next_gain[i]);
  }
}

// four vector loads a thread where the row allows it: more blocks an SM, at different points of their way
static inline int ln_threads(int hidden) { return hidden > 4096 ? 512 : (hidden > 2048 ? 256 : 128); }

template <typename KernelT>
static int ln_shared(KernelT kernel, size_t bytes) {
  if (bytes > 200 * 1024) return STRATUM_ERR_LIMIT;
  if (bytes > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

template <typename T>
static int launch_layernorm(const float* x, const float* gain, const int* rows, T* out, int n_rows, int hidden,
                            float eps, cudaStream_t stream) {
  const size_t bytes = (size_t)hidden * sizeof(float);
  const bool vec = hidden % 4 == 0 && ((((uintptr_t)x) | ((uintptr_t)gain) | ((uintptr_t)out)) & 15) == 0;
  auto kernel = vec ? layernorm_kernel<T, true> : layernorm_kernel<T, false>;
  const int bad = ln_shared(kernel, bytes);
  if (bad) return bad;
  launch_pdl(kernel, n_rows, ln_threads(hidden), bytes, stream, x, gain, rows, out, hidden, eps);
  return launch_status();
}

STRATUM_EXPORT int stratum_layernorm(const float* x, const float* gain, const int* rows, void* out, int out_dtype,
                                     int n_rows, int hidden, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden < 1) return STRATUM_ERR_SHAPE;
  if (out_dtype == STRATUM_DT_F32) return launch_layernorm<float>(x, gain, rows, (float*)out, n_rows, hidden, eps, stream);
  if (out_dtype == STRATUM_DT_BF16) return launch_layernorm<bf16>(x, gain, rows, (bf16*)out, n_rows, hidden, eps, stream);
  return STRATUM_ERR_DTYPE;
}

template <typename T>
static int launch_into(const float* y, const float* gain, float* x, const float* next_gain, T* next_out, int n_rows,
                       int hidden, float eps, float next_eps, int accumulate, cudaStream_t stream) {
  const size_t bytes = (size_t)hidden * sizeof(float);
  const bool vec = hidden % 4 == 0 &&
                   ((((uintptr_t)y) | ((uintptr_t)gain) | ((uintptr_t)x) | ((uintptr_t)next_gain) | ((uintptr_t)next_out)) & 15) == 0;
  auto kernel = vec ? layernorm_into_residual_kernel<T, true> : layernorm_into_residual_kernel<T, false>;
  const int bad = ln_shared(kernel, bytes);
  if (bad) return bad;
  launch_pdl(kernel, n_rows, ln_threads(hidden), bytes, stream, y, gain, x, next_gain, next_out, hidden, eps, next_eps,
             accumulate);
  return launch_status();
}

// next_out may be null (then next_gain and next_dtype are not looked at).
STRATUM_EXPORT int stratum_layernorm_into_residual(const float* y, const float* gain, float* x, const float* next_gain,
                                                   void* next_out, int next_dtype, int n_rows, int hidden, float eps,
                                                   float next_eps, int accumulate, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (hidden < 1) return STRATUM_ERR_SHAPE;
  if (next_out != nullptr && next_gain == nullptr) return STRATUM_ERR_SHAPE;
  if (next_out == nullptr || next_dtype == STRATUM_DT_F32)
    return launch_into<float>(y, gain, x, next_gain, (float*)next_out, n_rows, hidden, eps, next_eps, accumulate, stream);
  if (next_dtype == STRATUM_DT_BF16)
    return launch_into<bf16>(y, gain, x, next_gain, (bf16*)next_out, n_rows, hidden, eps, next_eps, accumulate, stream);
  return STRATUM_ERR_DTYPE;
}

// out[r][col0 + i] = x[r][i], rounded to out's type: the rows of a float32 matrix laid into a stretch of columns of
// a wider one (the operand of a product over several streams side by side).
template <typename T>
__global__ void pack_columns_kernel(const float* x, T* out, int width, int ldo, int col0, size_t total) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / width;
  const int c = (int)(i - r * width);
  out[r * ldo + col0 + c] = from_float<T>(ld_fresh(x + i));
}

STRATUM_EXPORT int stratum_pack_columns(const float* x, void* out, int out_dtype, int n_rows, int width, int ldo,
                                        int col0, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * width;
  if (total == 0) return 0;
  if (col0 < 0 || ldo < col0 + width) return STRATUM_ERR_SHAPE;
  const size_t blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffULL) return STRATUM_ERR_LIMIT;
  if (out_dtype == STRATUM_DT_F32)
    launch_pdl(pack_columns_kernel<float>, (unsigned)blocks, 256, 0, stream, x, (float*)out, width, ldo, col0, total);
  else if (out_dtype == STRATUM_DT_BF16)
    launch_pdl(pack_columns_kernel<bf16>, (unsigned)blocks, 256, 0, stream, x, (bf16*)out, width, ldo, col0, total);
  else return STRATUM_ERR_DTYPE;
  return launch_status();
}
