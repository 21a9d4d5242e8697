// Distilled-LDS variant of the STU (mini_stu/stu_lds.py:213-394; recurrence form mini_stu/lds.py:95-101):
//   h_t = A (.) h_{t-1} + B (.) x[b,t,i]   (one D-dimensional diagonal state per scalar channel (b,i), h_{-1} = 0)
//   U[b,t,f,i] = sum_n h_t[n] C[n,f]        (F = 48 features)
//   y[b,t,o]   = sum_{f,i} U[b,t,f,i] M[f,i,o]
// The modes nearly cancel in h @ C (|C| ~ 280 for outputs of order 1, |A| up to 0.99997): an fp32 state already
// costs ~1e-3 relative error on the features, so the state is kept and contracted in float64 (A, B are float64
// buffers in the reference too).  The work is tiny (D FMAs per channel per token); only the final contraction
// with M runs in the model dtype.
// Prefill is a chunked scan (chunks of Ck positions).  Inside a chunk starting at position t0 the features are
//   U[t0+tau, f] = sum_{sigma<=tau} G_f[tau-sigma] x[t0+sigma]  +  sum_n C[n,f] A_n^(tau+1) h_{t0-1}[n]
// the first term a causal Toeplitz product with the impulse responses G_f[j] = sum_n C[n,f] B[n] A[n]^j (benign,
// model dtype), the second the free response of the state carried into the chunk.  Evaluated mode by mode the carry
// term cancels to 1e-4 of its terms; it is evaluated instead in a rotated, balanced basis z = (V^T h) / sqrt(lambda)
// (V, lambda: leading eigenpairs of the reachability Gramian P[n,m] = B_n B_m / (1 - A_n A_m), float64 on the host),
// in which z and the rotated output map Q[(tau,f),k] are O(1) and nothing cancels, so both terms become ONE
// tensor-core GEMM per chunk column:  U[(tau,f), (chunk, channel)] = W[(tau,f), :] . Z[(chunk, channel), :]  with
// Z = [z_hi | z_lo | z_hi | x_chunk] and W = [Q_hi | Q_hi | Q_lo | Toeplitz(G)] (bf16 hi/lo split of the carry part;
// fp32 models keep [z | x] and [Q | Toeplitz]).  lds_chunk_scan_kernel below runs the exact float64 recurrence over
// the whole sequence (D FMAs per position and channel: cheap), writes Z at every chunk start and the final state;
// the GEMM scatters its tile straight into the [tokens, F*d] operand of the contraction with M.
// The other kernels here provide the state at the end of a prefill from a parity-split history and the recurrent
// decode step.
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
// Over the B*d channels the contraction is a [rows x D] . [D x F] product in float64: it runs on the float64 tensor
// path (mma.sync m8n8k4), a warp owning 8 consecutive channels.  Lane (r = lane / 4, c = lane % 4) updates the modes
// 4s + c of channel r - exactly the element of the A fragment it has to supply for K step s - so the new state goes
// from the update straight into the MMA without passing through shared memory; C sits in shared memory as float64
// with a row pitch of F + 4 (the four rows of a B fragment then fall on distinct banks).  One K step: 32 bytes of
// state per channel read and written (whole sectors), 6 MMAs for 48 features.  (The first form of this kernel gave a
// warp one channel and its lanes the features: 2 * D float64 FMAs per lane, each with a shared-memory read of C and a
// float -> double conversion; the 12-layer stack spent most of its token step there.)
constexpr int LDS_NTF = LDS_MAXF / 8;   // n-tiles of 8 features

__device__ __forceinline__ void dmma_884(double& c0, double& c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c0), "+d"(c1)
               : "d"(a), "d"(b));
}

template <typename T>
__global__ void __launch_bounds__(256) lds_decode_kernel(const T* __restrict__ x, long long x_rstride,
                                                         double* __restrict__ h, const double* __restrict__ A,
                                                         const double* __restrict__ Bv, const T* __restrict__ C,
                                                         T* __restrict__ U, int B, int d, int D, int F) {
  extern __shared__ __align__(16) unsigned char lds_smem[];
  const int Dp = (D + 3) & ~3, Fp = 8 * ((F + 7) / 8) + 4;
  double* Cs = reinterpret_cast<double*>(lds_smem);   // [Dp][Fp], zero outside [D][F]
  double* As = Cs + (size_t)Dp * Fp;                  // [Dp]
  double* Bs = As + Dp;                               // [Dp]
  for (int e = threadIdx.x; e < Dp * Fp; e += 256) {
    const int n = e / Fp, f = e - n * Fp;
    Cs[e] = (n < D && f < F) ? (double)Elem<T>::to_f(C[n * F + f]) : 0.0;
  }
  for (int n = threadIdx.x; n < Dp; n += 256) {
    As[n] = n < D ? A[n] : 0.0;
    Bs[n] = n < D ? Bv[n] : 0.0;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int rows = B * d;
  const int row = (blockIdx.x * 8 + warp) * 8 + r;
  const bool rok = row < rows;
  const int b = rok ? row / d : 0, i = rok ? row - b * d : 0;
  const double xv = rok ? (double)Elem<T>::to_f(x[(size_t)b * x_rstride + i]) : 0.0;
  double* hr = h + (size_t)(rok ? row : 0) * D;
  const int ntf = (F + 7) >> 3;
  double acc[LDS_NTF][2];
#pragma unroll
  for (int j = 0; j < LDS_NTF; j++) acc[j][0] = acc[j][1] = 0.0;
  // 16 K steps at a time: all their state loads go out before the first is used (64 bytes x 16 in flight per lane)
  for (int kc = 0; kc < Dp; kc += 64) {
    double hv[16];
#pragma unroll
    for (int u = 0; u < 16; u++) {
      const int n = kc + 4 * u + c;
      hv[u] = (rok && n < D) ? hr[n] : 0.0;
    }
#pragma unroll
    for (int u = 0; u < 16; u++) {
      const int n = kc + 4 * u + c;
      if (kc + 4 * u < Dp) {   // warp-uniform
        double v = 0.0;
        if (rok && n < D) {
          v = fma(As[n], hv[u], Bs[n] * xv);
          hr[n] = v;
        }
        const double* crow = Cs + (size_t)n * Fp + r;   // B fragment: C[4s + c][8j + r]
#pragma unroll
        for (int j = 0; j < LDS_NTF; j++)
          if (j < ntf) dmma_884(acc[j][0], acc[j][1], v, crow[8 * j]);
      }
    }
  }
  // accumulator: channel r, features 8j + 2c and 8j + 2c + 1
  if (rok) {
#pragma unroll
    for (int j = 0; j < LDS_NTF; j++) {
#pragma unroll
      for (int q = 0; q < 2; q++) {
        const int f = 8 * j + 2 * c + q;
        if (j < ntf && f < F) U[(size_t)b * F * d + (size_t)f * d + i] = Elem<T>::from_f((float)acc[j][q]);
      }
    }
  }
}

// Chunked scan: one CTA = 32 consecutive channels of one sequence (lane = channel), warp w owns modes
// w*MPW .. w*MPW+MPW-1 of all 32 (state, A and B in registers, float64).  Per chunk: (1) the state carried into the
// chunk is rotated, z_k = sum_n Vs[n][k] h[n] (Vs = V / sqrt(lambda), float64; every warp takes R/8 of the k through
// a shared-memory copy of the state) and written as the leading columns of Z; (2) the chunk's inputs are staged in
// shared memory, copied into the trailing Ck columns of Z (the Toeplitz operand) and (3) pushed through the
// recurrence h = fma(A, h, B*x) position by position - the same expression, in the same order, as
// lds_final_state_kernel, so the final state is bit-identical to that kernel's.
// Z: [B][nchunks][d][KZ] in the model dtype, KZ = 3*R + Ck (bf16: z_hi | z_lo | z_hi | x) or R + Ck (fp32: z | x).
// UNITB: every B[n] == 1 (the distilled checkpoint's case): B*x is x, so the multiplication is dropped and the
// result stays bit-identical to the general expression.
template <typename T, int MPW, bool UNITB>
__global__ void __launch_bounds__(256, UNITB ? 2 : 1) lds_chunk_scan_kernel(const T* __restrict__ x, long long x_bstride,
                                                             long long x_tstride, const double* __restrict__ A,
                                                             const double* __restrict__ Bv,
                                                             const double* __restrict__ Vs, T* __restrict__ Z,
                                                             double* __restrict__ hfin, int d, int Tn, int D, int R,
                                                             int Ck, int KZ) {
  extern __shared__ __align__(16) unsigned char scan_smem[];
  double* hs = reinterpret_cast<double*>(scan_smem);               // [D][33] state copy for the rotation
  T* xs = reinterpret_cast<T*>(hs + (size_t)D * 33);               // [Ck][32] inputs of the chunk
  constexpr bool SPLIT = (sizeof(T) == 2);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nblk = (d + 31) >> 5;
  const int b = blockIdx.x / nblk, i0 = (blockIdx.x - b * nblk) << 5;
  const int ch = i0 + lane;
  const bool chok = ch < d;
  const int nchunks = (Tn + Ck - 1) / Ck;
  double a[MPW], bb[UNITB ? 1 : MPW], h[MPW];
#pragma unroll
  for (int m = 0; m < MPW; m++) {
    const int n = warp * MPW + m;
    a[m] = n < D ? A[n] : 0.0;
    if (!UNITB) bb[m] = n < D ? Bv[n] : 0.0;
    h[m] = 0.0;
  }
  for (int c = 0; c < nchunks; c++) {
    const int t0 = c * Ck;
    T* zrow = Z + ((size_t)((size_t)b * nchunks + c) * d + (chok ? ch : 0)) * KZ;
    // ---- (1) rotate the carried state
#pragma unroll
    for (int m = 0; m < MPW; m++) {
      const int n = warp * MPW + m;
      if (n < D) hs[n * 33 + lane] = h[m];
    }
    __syncthreads();
    // this warp's coordinates k0 .. k0+7 (groups of eight; R % 8 == 0): one pass over the modes with eight
    // independent accumulators, the state value of a mode read once and the eight rotation entries as 16-byte
    // warp-uniform loads
    for (int k0 = warp * 8; k0 < R; k0 += 64) {
      double z[8];
#pragma unroll
      for (int j = 0; j < 8; j++) z[j] = 0.0;
#pragma unroll 2
      for (int n = 0; n < D; n++) {
        const double hv = hs[n * 33 + lane];
        const double2* vr = reinterpret_cast<const double2*>(Vs + (size_t)n * R + k0);
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const double2 v2 = __ldg(vr + j);
          z[2 * j] = fma(v2.x, hv, z[2 * j]);
          z[2 * j + 1] = fma(v2.y, hv, z[2 * j + 1]);
        }
      }
      if (chok) {
        float zf[8];
#pragma unroll
        for (int j = 0; j < 8; j++) zf[j] = (float)z[j];
        if (SPLIT) {   // eight consecutive coordinates: one 16-byte store per copy
          store_vec(zrow + k0, zf);           // rounds to the high parts
          store_vec(zrow + 2 * R + k0, zf);
#pragma unroll
          for (int j = 0; j < 8; j++) zf[j] -= round_to<T>(zf[j]);
          store_vec(zrow + R + k0, zf);       // low parts
        } else {
          store_vec(zrow + k0, zf);
          store_vec(zrow + k0 + 4, zf + 4);
        }
      }
    }
    // ---- (2) stage the chunk's inputs (zero past the end of the sequence) and copy them into Z
    const int zoff = SPLIT ? 3 * R : R;
    for (int e = threadIdx.x; e < Ck * 32; e += 256) {
      const int sg = e >> 5, cc = e & 31;
      const int t = t0 + sg;
      xs[e] = (t < Tn && i0 + cc < d) ? x[(size_t)b * x_bstride + (size_t)t * x_tstride + i0 + cc]
                                      : Elem<T>::from_f(0.f);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < Ck * 32; e += 256) {   // consecutive threads write consecutive positions of a row
      const int cc = e / Ck, sg = e - cc * Ck;
      if (i0 + cc < d)
        Z[((size_t)((size_t)b * nchunks + c) * d + i0 + cc) * KZ + zoff + sg] = xs[sg * 32 + cc];
    }
    // ---- (3) the recurrence over the chunk
    const int lim = min(Ck, Tn - t0);
#pragma unroll 4
    for (int sg = 0; sg < lim; sg++) {
      const double xv = (double)Elem<T>::to_f(xs[sg * 32 + lane]);
#pragma unroll
      for (int m = 0; m < MPW; m++) h[m] = UNITB ? fma(a[m], h[m], xv) : fma(a[m], h[m], bb[m] * xv);
    }
    __syncthreads();   // xs and hs are rewritten by the next chunk
  }
  if (chok) {
#pragma unroll
    for (int m = 0; m < MPW; m++) {
      const int n = warp * MPW + m;
      if (n < D) hfin[((size_t)b * d + ch) * D + n] = h[m];
    }
  }
}

// x: [B, Tn, d] (element strides x_bstride / x_tstride, channels contiguous); A, Bv: [D] float64; Vs: [D][R] float64
// (rotation with the balancing scale folded in); Z: [B][ceil(Tn/Ck)][d][KZ] model dtype, KZ = 3R+Ck (bf16) or R+Ck
// (fp32); hfin: [B*d][D] float64 = the state after the Tn inputs (what stu_lds_final_state computes).
// Replaces the scan of mini_stu/stu_lds.py:17-99,181-200,280-338 (lds_scan_kernel / affine_scan_with_fixed_a /
// FixedDiagonalLDS.forward) together with the GEMM the caller runs on Z.
extern "C" int stu_lds_chunk_scan(const void* x, long long x_bstride, long long x_tstride, const double* A,
                                  const double* Bv, const double* Vs, void* Z, double* hfin, int B, int d, int Tn,
                                  int D, int R, int Ck, int dtype, void* stream) {
  // bit 0x1000 of dtype: the caller has checked that every B[n] is exactly 1
  const bool unit_b = (dtype & 0x1000) != 0;
  dtype &= ~0x1000;
  if (!x || !A || !Bv || !Vs || !Z || !hfin) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || Tn <= 0 || D <= 0 || D > LDS_MAXD || R <= 0 || R > D || Ck <= 0 || Ck % 8 || R % 8)
    return STU_ERR_SHAPE;
  if (dtype != STU_F32 && dtype != STU_BF16) return STU_ERR_DTYPE;
  const int KZ = (dtype == STU_BF16 ? 3 * R : R) + Ck;
  const size_t elem = dtype == STU_BF16 ? 2 : 4;
  const size_t smem = (size_t)D * 33 * sizeof(double) + (size_t)Ck * 32 * elem;
  if (smem > 200 * 1024) return STU_ERR_UNSUPPORTED;
  const int grid = B * ((d + 31) / 32);
  cudaStream_t st = (cudaStream_t)stream;
  const int mpw = (D + 7) / 8;
#define LDS_SCAN_LAUNCH(TT, MPW_, UB_)                                                                             \
  do {                                                                                                             \
    cudaError_t e_ = cudaFuncSetAttribute(lds_chunk_scan_kernel<TT, MPW_, UB_>,                                    \
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                 \
    if (e_ != cudaSuccess) return (int)e_;                                                                         \
    lds_chunk_scan_kernel<TT, MPW_, UB_><<<grid, 256, smem, st>>>((const TT*)x, x_bstride, x_tstride, A, Bv, Vs,   \
                                                                  (TT*)Z, hfin, d, Tn, D, R, Ck, KZ);              \
  } while (0)
  if (dtype == STU_BF16) {
    if (mpw <= 20 && unit_b) LDS_SCAN_LAUNCH(bf16, 20, true);
    else if (mpw <= 20) LDS_SCAN_LAUNCH(bf16, 20, false);
    else LDS_SCAN_LAUNCH(bf16, 32, false);
  } else {
    if (mpw <= 20 && unit_b) LDS_SCAN_LAUNCH(float, 20, true);
    else if (mpw <= 20) LDS_SCAN_LAUNCH(float, 20, false);
    else LDS_SCAN_LAUNCH(float, 32, false);
  }
#undef LDS_SCAN_LAUNCH
  STU_CHECK_LAUNCH();
  return STU_OK;
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
  const int Dp = (D + 3) & ~3, Fp = 8 * ((F + 7) / 8) + 4;
  const size_t smem = ((size_t)Dp * Fp + 2 * (size_t)Dp) * sizeof(double);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (dtype == STU_F32) {
    e = cudaFuncSetAttribute(lds_decode_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    lds_decode_kernel<float><<<(rows + 63) / 64, 256, smem, st>>>((const float*)x, x_row_stride, h, A, Bv,
                                                                (const float*)C, (float*)U, B, d, D, F);
  } else if (dtype == STU_BF16) {
    e = cudaFuncSetAttribute(lds_decode_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    lds_decode_kernel<bf16><<<(rows + 63) / 64, 256, smem, st>>>((const bf16*)x, x_row_stride, h, A, Bv, (const bf16*)C,
                                                               (bf16*)U, B, d, D, F);
  } else {
    return STU_ERR_DTYPE;
  }
  STU_CHECK_LAUNCH();
  return STU_OK;
}
