// Distilled-LDS variant of the STU (mini_stu/stu_lds.py:213-394; recurrence form mini_stu/lds.py:95-101):
//   h_t = A (.) h_{t-1} + B (.) x[b,t,i]   (one D-dimensional diagonal state per scalar channel (b,i), h_{-1} = 0)
//   U[b,t,f,i] = sum_n h_t[n] C[n,f]        (F = 48 features)
//   y[b,t,o]   = sum_{f,i} U[b,t,f,i] M[f,i,o]
// The modes nearly cancel in h @ C (|C| ~ 280 for outputs of order 1, |A| up to 0.99997): an fp32 state already
// costs ~1e-3 relative error on the features, so the state is kept and contracted in float64 (A, B are float64
// buffers in the reference too).  The work is tiny (D FMAs per channel per token); only the final contraction
// with M runs in the model dtype.
// Prefill outputs come from the equivalent causal convolution with the impulse responses
// G[j,f] = sum_n C[n,f] B[n] A[n]^j (built in float64 on the host), which goes through the full-variant
// Toeplitz GEMMs; the kernels here provide (1) the state at the end of a prefill, for the decode that follows,
// and (2) the recurrent decode step.
#include "common.cuh"

constexpr int LDS_MAXD = 256;  // state dimension limit (8 modes per lane)
constexpr int LDS_MAXF = 64;   // feature limit

// State after the T cached inputs of every channel: one warp per (b,i), lanes own modes lane, lane+32, ...
// The inputs are read from the parity-split history (time-major per channel).
template <typename T>
__global__ void __launch_bounds__(256) lds_final_state_kernel(const T* __restrict__ hist, double* __restrict__ h,
                                                              const double* __restrict__ A,
                                                              const double* __restrict__ Bv, int rows, int Lh, int Tn,
                                                              int D) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  double a[8], bb[8], st[8];
#pragma unroll
  for (int m = 0; m < 8; m++) {
    const int n = lane + 32 * m;
    a[m] = n < D ? A[n] : 0.0;
    bb[m] = n < D ? Bv[n] : 0.0;
    st[m] = 0.0;
  }
  const T* r0 = hist + (size_t)row * 2 * Lh;  // parity 0 run, parity 1 run follows at +Lh
  for (int t0 = 0; t0 < Tn; t0 += 64) {
    // lanes fetch 64 consecutive times (32 per parity) and broadcast them in order
    const int s = (t0 >> 1) + lane;
    const float xe = (2 * s < Tn) ? Elem<T>::to_f(r0[s]) : 0.f;
    const float xo = (2 * s + 1 < Tn) ? Elem<T>::to_f(r0[Lh + s]) : 0.f;
    const int lim = min(64, Tn - t0);
    for (int j = 0; j < lim; j++) {
      const double xv = (double)__shfl_sync(0xffffffffu, (j & 1) ? xo : xe, j >> 1);
#pragma unroll
      for (int m = 0; m < 8; m++) st[m] = fma(a[m], st[m], bb[m] * xv);
    }
  }
#pragma unroll
  for (int m = 0; m < 8; m++) {
    const int n = lane + 32 * m;
    if (n < D) h[(size_t)row * D + n] = st[m];
  }
}

// One recurrent step: h <- A (.) h + B (.) x_t, then U[b][f*d + i] = round(sum_n h[n] C[n,f]).
// One warp per (b,i).  The state update is spread over the lanes by mode (lane, lane+32, ...); for the contraction
// the warp puts its new state into shared memory and the lanes switch to features: lane f walks the D modes with
// the state as a broadcast read and C[n][f] as a conflict-free row read, so no cross-lane reduction is needed.
template <typename T>
__global__ void __launch_bounds__(256) lds_decode_kernel(const T* __restrict__ x, long long x_rstride,
                                                         double* __restrict__ h, const double* __restrict__ A,
                                                         const double* __restrict__ Bv, const T* __restrict__ C,
                                                         T* __restrict__ U, int B, int d, int D, int F) {
  extern __shared__ __align__(16) unsigned char lds_smem[];
  double* st_s = reinterpret_cast<double*>(lds_smem);            // [8 warps][D]
  float* Cs = reinterpret_cast<float*>(st_s + 8 * D);            // [D][F]
  for (int e = threadIdx.x; e < D * F; e += 256) Cs[e] = Elem<T>::to_f(C[e]);
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool rok = row < B * d;
  const int b = rok ? row / d : 0, i = rok ? row - b * d : 0;
  if (rok) {
    const double xv = (double)Elem<T>::to_f(x[(size_t)b * x_rstride + i]);
    for (int n = lane; n < D; n += 32) {
      const double v = fma(A[n], h[(size_t)row * D + n], Bv[n] * xv);
      h[(size_t)row * D + n] = v;
      st_s[warp * D + n] = v;
    }
  }
  __syncthreads();
  if (rok) {
    const double* sw = st_s + warp * D;
    for (int f = lane; f < F; f += 32) {
      double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
      int n = 0;
      for (; n + 4 <= D; n += 4) {
        a0 = fma(sw[n], (double)Cs[n * F + f], a0);
        a1 = fma(sw[n + 1], (double)Cs[(n + 1) * F + f], a1);
        a2 = fma(sw[n + 2], (double)Cs[(n + 2) * F + f], a2);
        a3 = fma(sw[n + 3], (double)Cs[(n + 3) * F + f], a3);
      }
      for (; n < D; n++) a0 = fma(sw[n], (double)Cs[n * F + f], a0);
      U[(size_t)b * F * d + (size_t)f * d + i] = Elem<T>::from_f((float)((a0 + a1) + (a2 + a3)));
    }
  }
}

// hist: [B*d][2][Lh] holding the Tn inputs of every channel; h: [B*d][D] float64 (overwritten); A, Bv: [D] float64.
extern "C" int stu_lds_final_state(const void* hist, double* h, const double* A, const double* Bv, int B, int d, int Lh,
                                   int Tn, int D, int dtype, void* stream) {
  if (!hist || !h || !A || !Bv) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || Lh <= 0 || Tn < 0 || Tn > 2 * Lh || D <= 0 || D > LDS_MAXD) return STU_ERR_SHAPE;
  const int rows = B * d;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == STU_F32)
    lds_final_state_kernel<float><<<(rows + 7) / 8, 256, 0, st>>>((const float*)hist, h, A, Bv, rows, Lh, Tn, D);
  else if (dtype == STU_BF16)
    lds_final_state_kernel<bf16><<<(rows + 7) / 8, 256, 0, st>>>((const bf16*)hist, h, A, Bv, rows, Lh, Tn, D);
  else
    return STU_ERR_DTYPE;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// x: [B, d] new inputs; h: [B*d][D] float64 state (updated in place); C: [D][F] model dtype; U: [B][F*d] features in
// the order the contraction with M[f,i,o] (flattened [F*d, d_out]) expects.
extern "C" int stu_lds_decode_features(const void* x, long long x_row_stride, double* h, const double* A,
                                       const double* Bv, const void* C, void* U, int B, int d, int D, int F, int dtype,
                                       void* stream) {
  if (!x || !h || !A || !Bv || !C || !U) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || D <= 0 || D > LDS_MAXD || F <= 0 || F > LDS_MAXF) return STU_ERR_SHAPE;
  const int rows = B * d;
  const size_t smem = (size_t)D * F * sizeof(float) + (size_t)8 * D * sizeof(double);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (dtype == STU_F32) {
    e = cudaFuncSetAttribute(lds_decode_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    lds_decode_kernel<float><<<(rows + 7) / 8, 256, smem, st>>>((const float*)x, x_row_stride, h, A, Bv,
                                                                (const float*)C, (float*)U, B, d, D, F);
  } else if (dtype == STU_BF16) {
    e = cudaFuncSetAttribute(lds_decode_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    lds_decode_kernel<bf16><<<(rows + 7) / 8, 256, smem, st>>>((const bf16*)x, x_row_stride, h, A, Bv, (const bf16*)C,
                                                               (bf16*)U, B, d, D, F);
  } else {
    return STU_ERR_DTYPE;
  }
  STU_CHECK_LAUNCH();
  return STU_OK;
}
