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

// (mean, 1 / sqrt(var + eps)) of the row in shared memory; every thread gets both
__device__ __forceinline__ float2 ln_stats(const float* row, int hidden, float eps, float* scratch) {
  float s = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) s += row[i];
  const float mean = block_sum(s, scratch) / (float)hidden;
  float q = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float d = row[i] - mean;
    q = fmaf(d, d, q);
  }
  const float var = block_sum(q, scratch) / (float)hidden;
  return make_float2(mean, 1.0f / sqrtf(var + eps));
}

template <typename T, bool VEC>
__global__ void layernorm_kernel(const float* x, const float* __restrict__ gain, const int* __restrict__ rows, T* out,
                                 int hidden, float eps) {
  extern __shared__ __align__(16) float ln_row[];
  __shared__ float scratch[33];
  pdl_trigger();
  const int r = blockIdx.x;
  pdl_wait();                                        // x (and rows) are the work of kernels before this one
  const int src = rows ? __ldcg(rows + r) : r;
  ln_load<VEC>(x + (size_t)src * hidden, ln_row, hidden);
  __syncthreads();
  const float2 st = ln_stats(ln_row, hidden, eps, scratch);
  T* o = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<T>((ln_row[i] - st.x) * st.y * gain[i]);
}

template <typename T, bool VEC>
__global__ void layernorm_into_residual_kernel(const float* y, const float* __restrict__ gain, float* x,
                                               const float* __restrict__ next_gain, T* next_out, int hidden, float eps,
                                               float next_eps, int accumulate) {
  extern __shared__ __align__(16) float ln_row[];
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t at = (size_t)blockIdx.x * hidden;
  ln_load<VEC>(y + at, ln_row, hidden);
  __syncthreads();
  const float2 st = ln_stats(ln_row, hidden, eps, scratch);
  float* xr = x + at;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {      // a thread rewrites the entries it reads
    float v = (ln_row[i] - st.x) * st.y * gain[i];
    if (accumulate) v += ld_fresh(xr + i);
    xr[i] = v;
    ln_row[i] = v;
  }
  if (next_out == nullptr) return;
  __syncthreads();
  const float2 nx = ln_stats(ln_row, hidden, next_eps, scratch);
  T* o = next_out + at;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_float<T>((ln_row[i] - nx.x) * nx.y * next_gain[i]);
}

static inline int ln_threads(int hidden) { return hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128); }

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
  const bool vec = hidden % 4 == 0 && (((uintptr_t)x) & 15) == 0;
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
  const bool vec = hidden % 4 == 0 && (((uintptr_t)y) & 15) == 0;
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
