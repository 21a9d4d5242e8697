// RMSNorm and embedding gather (HBM-bound; 128-bit loads, warp-shuffle reductions).
#include "common.cuh"

// y[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps) * w, statistics and scaling in fp32, one rounding
// (torch.nn.RMSNorm arithmetic; reference selection flash_stu/layers/stu_layer.py:17-36).
template <typename T, bool VECTOR>
__global__ void __launch_bounds__(128) rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                      T* __restrict__ y, int d, long long x_rstride,
                                                      long long y_rstride, float eps) {
  constexpr int V = Elem<T>::VEC;
  const T* xr = x + (size_t)blockIdx.x * x_rstride;
  T* yr = y + (size_t)blockIdx.x * y_rstride;
  // launched with the programmatic attribute: the CTAs are resident while the kernel before them drains, and the
  // kernel after this one may bring its weights in meanwhile
  pdl_trigger();
  pdl_wait();
  float ss = 0.f;
  if (VECTOR) {
    for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
      float v[V];
      load_vec(xr + i, v);
#pragma unroll
      for (int j = 0; j < V; j++) ss += v[j] * v[j];
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      float v = Elem<T>::to_f(xr[i]);
      ss += v * v;
    }
  }
  __shared__ float red[4];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = red[0] + red[1] + red[2] + red[3];
  float r = rsqrtf(tot / (float)d + eps);
  if (VECTOR) {
    for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
      float v[V], g[V];
      load_vec(xr + i, v);
      load_vec(w + i, g);
#pragma unroll
      for (int j = 0; j < V; j++) v[j] = v[j] * r * g[j];
      store_vec(yr + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x)
      yr[i] = Elem<T>::from_f(Elem<T>::to_f(xr[i]) * r * Elem<T>::to_f(w[i]));
  }
}

template <typename T>
static int launch_rmsnorm(const void* x, const void* w, void* y, int rows, int d, long long xs, long long ys,
                          float eps, cudaStream_t st) {
  constexpr int V = Elem<T>::VEC;
  bool vec = (d % V == 0) && (xs % V == 0) && (ys % V == 0) && aligned16(x) && aligned16(w) && aligned16(y);
  cudaError_t e;
  if (vec)
    e = launch_maybe_overlapped(rmsnorm_kernel<T, true>, dim3(rows), dim3(128), 0, st, true, (const T*)x, (const T*)w,
                                (T*)y, d, xs, ys, eps);
  else
    e = launch_maybe_overlapped(rmsnorm_kernel<T, false>, dim3(rows), dim3(128), 0, st, true, (const T*)x,
                                (const T*)w, (T*)y, d, xs, ys, eps);
  if (e != cudaSuccess) return (int)e;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

extern "C" int stu_rmsnorm(const void* x, const void* w, void* y, int rows, int d, long long x_row_stride,
                           long long y_row_stride, float eps, int dtype, void* stream) {
  if (!x || !w || !y) return STU_ERR_NULL;
  if (rows < 0 || d <= 0) return STU_ERR_SHAPE;
  if (rows == 0) return STU_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == STU_F32) return launch_rmsnorm<float>(x, w, y, rows, d, x_row_stride, y_row_stride, eps, st);
  if (dtype == STU_BF16) return launch_rmsnorm<bf16>(x, w, y, rows, d, x_row_stride, y_row_stride, eps, st);
  return STU_ERR_DTYPE;
}

// x[r,:] = table[ids[r],:]  (nn.Embedding lookup, reference flash_stu/model.py:152).  Ids outside
// [0, vocab) write a zero row and raise the status word instead of reading out of bounds.
template <typename T>
__global__ void __launch_bounds__(128) embed_kernel(const long long* __restrict__ ids, const T* __restrict__ table,
                                                    T* __restrict__ out, int d, int vocab, int* status) {
  long long id = ids[blockIdx.x];
  bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && status) atomicExch(status, 1);
  const T* src = table + (size_t)(ok ? id : 0) * d;
  T* dst = out + (size_t)blockIdx.x * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = ok ? src[i] : Elem<T>::from_f(0.f);
}

extern "C" int stu_embed(const long long* ids, const void* table, void* out, int rows, int d, int vocab,
                         int* status, int dtype, void* stream) {
  if (!ids || !table || !out) return STU_ERR_NULL;
  if (rows < 0 || d <= 0 || vocab <= 0) return STU_ERR_SHAPE;
  if (rows == 0) return STU_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == STU_F32)
    embed_kernel<float><<<rows, 128, 0, st>>>(ids, (const float*)table, (float*)out, d, vocab, status);
  else if (dtype == STU_BF16)
    embed_kernel<bf16><<<rows, 128, 0, st>>>(ids, (const bf16*)table, (bf16*)out, d, vocab, status);
  else
    return STU_ERR_DTYPE;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// y[r, c] = act(y[r, c] + bias[c]) in place, one rounding after the bias and one after the activation (the reference's
// nn.Linear bias followed by an activation module: mini_stu/stu.py:171-211 post-MLP; the SiLU between the STU
// sandwich projections, flash_stu/layers/stu_layer.py:52,84).  act: 0 none, 1 ReLU, 2 GELU (erf), 3 tanh, 4 SiLU.
template <typename T>
__global__ void __launch_bounds__(256) bias_act_kernel(T* __restrict__ y, const T* __restrict__ bias, long long rows,
                                                       int cols, long long y_rstride, int act) {
  const long long total = rows * cols;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long r = i / cols;
    const int c = (int)(i - r * cols);
    T* p = y + r * y_rstride + c;
    float v = Elem<T>::to_f(*p);
    if (bias) v = round_to<T>(v + Elem<T>::to_f(bias[c]));
    switch (act) {
      case 1: v = fmaxf(v, 0.f); break;
      case 2: v = 0.5f * v * (1.f + erff(v * 0.70710678118654752f)); break;
      case 3: v = tanhf(v); break;
      case 4: v = v / (1.f + expf(-v)); break;
      default: break;
    }
    *p = Elem<T>::from_f(v);
  }
}

extern "C" int stu_bias_act(void* y, const void* bias, long long rows, int cols, long long y_row_stride, int act,
                            int dtype, void* stream) {
  if (!y) return STU_ERR_NULL;
  if (rows < 0 || cols <= 0 || act < 0 || act > 4) return STU_ERR_SHAPE;
  if (rows == 0) return STU_OK;
  const long long total = rows * cols;
  const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == STU_F32)
    bias_act_kernel<float><<<grid, 256, 0, st>>>((float*)y, (const float*)bias, rows, cols, y_row_stride, act);
  else if (dtype == STU_BF16)
    bias_act_kernel<bf16><<<grid, 256, 0, st>>>((bf16*)y, (const bf16*)bias, rows, cols, y_row_stride, act);
  else
    return STU_ERR_DTYPE;
  STU_CHECK_LAUNCH();
  return STU_OK;
}
