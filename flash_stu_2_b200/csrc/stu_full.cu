// STU spectral convolution, full variant (flash_stu/modules/stu.py:100-118; MiniSTU mini_stu/stu.py:240-269):
//   U+-[b,t,k,i] = sum_j (+-1)^j phi[j,k] x[b,t-j,i]      (rounded to the model dtype)
//   y[b,t,o]     = sum_{k,i} U+[b,t,k,i] M_phi_plus[k,i,o] + U-[b,t,k,i] M_phi_minus[k,i,o]
// Here the K filters are shared by all channels, so the convolutions are real GEMMs.  With the history of the
// layer input kept parity-split and time-major per channel ([B][d][2][Lh], as for the approx variant):
//   E_k[(b,i,p)][m] = sum_s phi[2(m-s),   k] * H[(b,i,p)][s]          even taps, same parity
//   Q_k[(b,i,p)][m] = sum_s phi[2(m-s)+1-2p... see toeplitz_kernel     odd taps, other parity
//   U+ = E + Q,  U- = E - Q
// i.e. per filter three products of history rows with lower-triangular Toeplitz matrices built on the fly
// (toeplitz_kernel), run by the tcgen05 GEMM with its causal k-block skip, then combine_kernel writes
// U+- token-major [B*T][2*K*d] for the contraction GEMM with [M_phi_plus; M_phi_minus].
#include "common.cuh"

// x[b, t - t0, c] (token-major, t in [t0, t_end)) -> hist[b][c][t&1][t>>1]; 64 times x 8V channels per CTA.
template <typename T>
__global__ void __launch_bounds__(256) to_history_kernel(const T* __restrict__ x, long long x_bstride,
                                                         long long x_tstride, T* __restrict__ hist, int d, int Lh,
                                                         int t0, int t_end) {
  constexpr int V = Elem<T>::VEC;
  constexpr int TC = 8 * V;
  constexpr int TT = 64;
  __shared__ T tile[TT][TC + 2];
  const int b = blockIdx.z, c0 = blockIdx.y * TC, tb = t0 + blockIdx.x * TT;
  for (int item = threadIdx.x; item < TT * 8; item += 256) {
    const int tl = item >> 3, cg = item & 7;
    const int t = tb + tl, c = c0 + cg * V;
    float v[V];
#pragma unroll
    for (int j = 0; j < V; j++) v[j] = 0.f;
    if (t < t_end) {
      const T* px = x + (size_t)b * x_bstride + (size_t)(t - t0) * x_tstride + c;
      if (c + V <= d && ((reinterpret_cast<uintptr_t>(px) & 15u) == 0)) {
        load_vec(px, v);
      } else {
        for (int j = 0; j < V && c + j < d; j++) v[j] = Elem<T>::to_f(px[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < V; j++) tile[tl][cg * V + j] = Elem<T>::from_f(v[j]);
  }
  __syncthreads();
  for (int item = threadIdx.x; item < TC * TT; item += 256) {
    const int c = item / TT, tl = item % TT;
    const int t = tb + tl;
    if (c0 + c < d && t < t_end) hist[hist_off(b, c0 + c, t, d, Lh)] = tile[tl][c];
  }
}

extern "C" int stu_to_history(const void* x, long long x_bstride, long long x_tstride, void* hist, int B, int d, int Lh,
                              int t0, int t_end, int dtype, void* stream) {
  if (!x || !hist) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || Lh <= 0 || t0 < 0 || t_end <= t0 || t_end > 2 * Lh) return STU_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int tc = (dtype == STU_F32) ? 32 : 64;
  dim3 grid((t_end - t0 + 63) / 64, (d + tc - 1) / tc, B);
  if (dtype == STU_F32)
    to_history_kernel<float><<<grid, 256, 0, st>>>((const float*)x, x_bstride, x_tstride, (float*)hist, d, Lh, t0,
                                                   t_end);
  else if (dtype == STU_BF16)
    to_history_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)x, x_bstride, x_tstride, (bf16*)hist, d, Lh, t0,
                                                  t_end);
  else
    return STU_ERR_DTYPE;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// Lower-triangular Toeplitz matrices of one filter column f[0..L) (row stride f_stride), S x S each, row
// pitch ld:
//   kind 0 (even taps, same parity)      Tz[m][s] = f[2(m-s)]        m >= s
//   kind 1 (odd taps, outputs of parity 1 from inputs of parity 0)   Tz[m][s] = f[2(m-s)+1]   m >= s
//   kind 2 (odd taps, outputs of parity 0 from inputs of parity 1)   Tz[m][s] = f[2(m-s)-1]   m >  s
// (time t = 2m+p reads input time t-j = 2s+p'; the tap index j follows.)  Entries past L and above the
// diagonal are zero.
template <typename T>
__global__ void toeplitz_kernel(const T* __restrict__ f, long long f_stride, int L, T* __restrict__ out, int S,
                                long long ld) {
  const int kind = blockIdx.z;
  T* o = out + (size_t)kind * S * ld;
  const int m = blockIdx.y;
  for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < S; s += gridDim.x * blockDim.x) {
    int j = 2 * (m - s) + (kind == 0 ? 0 : (kind == 1 ? 1 : -1));
    T v = Elem<T>::from_f(0.f);
    if (m >= s && j >= 0 && j < L) v = f[(size_t)j * f_stride];
    o[(size_t)m * ld + s] = v;
  }
}

extern "C" int stu_toeplitz(const void* f, long long f_stride, int L, void* out, int S, long long ld, int dtype,
                            void* stream) {
  if (!f || !out) return STU_ERR_NULL;
  if (L <= 0 || S <= 0 || ld < S) return STU_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((S + 255) / 256 < 16 ? (S + 255) / 256 : 16, S, 3);
  if (dtype == STU_F32)
    toeplitz_kernel<float><<<grid, 256, 0, st>>>((const float*)f, f_stride, L, (float*)out, S, ld);
  else if (dtype == STU_BF16)
    toeplitz_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)f, f_stride, L, (bf16*)out, S, ld);
  else
    return STU_ERR_DTYPE;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// U[(b, t - t0)][sign*K*d + k*d + i] = round(E[(b,i,p)][m] +- Q[(b,i,p)][m]),  t = 2m + p in [t0, t_end).
// E and Q are [B*d*2][ldE] with rows in history order (b, i, p) and the time index m along the row.
// One CTA transposes 64 time indices x 8V channels of one (b, p) through shared memory so that both the
// reads (along m) and the writes (along i) are 16-byte vectors.
template <typename T>
__global__ void __launch_bounds__(256) combine_kernel(const T* __restrict__ E, const T* __restrict__ Q, long long ldE,
                                                      T* __restrict__ U, long long ldU, int d, int K, int k,
                                                      int both_signs, int Tn, int t0, int t_end) {
  constexpr int V = Elem<T>::VEC;
  constexpr int TC = 8 * V;
  constexpr int TS = 64;
  constexpr int SROW = (sizeof(T) == 2) ? 66 : 65;
  __shared__ __align__(16) T te[TC][SROW];
  __shared__ __align__(16) T tq[TC][SROW];
  const int bp = blockIdx.z, b = bp >> 1, p = bp & 1;
  const int c0 = blockIdx.y * TC;
  const int m_first = (t0 - p + 1) >> 1;           // first output index of this parity
  const int mb = (m_first - m_first % V) + blockIdx.x * TS;
  constexpr int NV = TS / V;
  for (int item = threadIdx.x; item < TC * NV; item += 256) {
    const int c = item / NV, v = item % NV;
    const int m = mb + v * V;
    float e[V], q[V];
#pragma unroll
    for (int j = 0; j < V; j++) e[j] = q[j] = 0.f;
    if (c0 + c < d && m + V <= ldE) {
      const size_t off = ((size_t)((size_t)b * d + c0 + c) * 2 + p) * ldE + m;
      load_vec(E + off, e);
      load_vec(Q + off, q);
    }
#pragma unroll
    for (int j = 0; j < V; j++) {
      te[c][v * V + j] = Elem<T>::from_f(e[j]);
      tq[c][v * V + j] = Elem<T>::from_f(q[j]);
    }
  }
  __syncthreads();
  for (int item = threadIdx.x; item < TS * 8; item += 256) {
    const int ml = item >> 3, cg = item & 7;
    const int m = mb + ml, t = 2 * m + p, c = c0 + cg * V;
    if (t >= t0 && t < t_end && c < d) {
      float up[V], um[V];
#pragma unroll
      for (int j = 0; j < V; j++) {
        const float e = Elem<T>::to_f(te[cg * V + j][ml]), q = Elem<T>::to_f(tq[cg * V + j][ml]);
        up[j] = e + q;
        um[j] = e - q;
      }
      T* row = U + ((size_t)b * Tn + (t - t0)) * ldU;
      T* pp = row + (size_t)k * d + c;
      T* pm = row + (size_t)(K + k) * d + c;
      if (c + V <= d && ((reinterpret_cast<uintptr_t>(pp) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(pm) & 15u) == 0)) {
        store_vec(pp, up);
        if (both_signs) store_vec(pm, um);
      } else {
        for (int j = 0; j < V && c + j < d; j++) {
          pp[j] = Elem<T>::from_f(up[j]);
          if (both_signs) pm[j] = Elem<T>::from_f(um[j]);
        }
      }
    }
  }
}

extern "C" int stu_full_combine(const void* E, const void* Q, long long ldE, void* U, long long ldU, int B, int d,
                                int K, int k, int both_signs, int t0, int t_end, int dtype, void* stream) {
  if (!E || !Q || !U) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || K <= 0 || k < 0 || k >= K || t0 < 0 || t_end <= t0 || 2 * ldE < t_end) return STU_ERR_SHAPE;
  if (ldE % 8 || !aligned16(E) || !aligned16(Q)) return STU_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  const int tc = (dtype == STU_F32) ? 32 : 64;
  const int v = (dtype == STU_F32) ? 4 : 8;
  const int m_first = t0 >> 1;  // smallest first index over the two parities
  const int m_last = (t_end + 1) >> 1;
  const int span = m_last - (m_first - m_first % v);
  dim3 grid((span + 63) / 64 + 1, (d + tc - 1) / tc, 2 * B);
  const int Tn = t_end - t0;
  if (dtype == STU_F32)
    combine_kernel<float><<<grid, 256, 0, st>>>((const float*)E, (const float*)Q, ldE, (float*)U, ldU, d, K, k,
                                                both_signs, Tn, t0, t_end);
  else if (dtype == STU_BF16)
    combine_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)E, (const bf16*)Q, ldE, (bf16*)U, ldU, d, K, k,
                                               both_signs, Tn, t0, t_end);
  else
    return STU_ERR_DTYPE;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// ------------------------------------------------------------------------------------------------
// Cached decode of the full variant.  One step at time t = pos[2b] (uniform over the batch: this path
// takes the position of sequence 0) is
//   G[(b,i,p')][0..K)   = sum_s H[(b,i,p')][s] * PhiT[k][s]        (even-tap columns)
//   G[(b,i,p')][K..2K)  = sum_s H[(b,i,p')][s] * PhiT[K+k][s]      (odd-tap columns)
// one tensor-core GEMM over ALL history rows against the 2K x Lh matrix PhiT of time-reversed taps that
// full_decode_prepare_kernel rebuilds every step from the device-side position:
//   PhiT[k][s]   = phi[2(sn-s), k]                       s <= sn            (sn = t>>1, p = t&1)
//   PhiT[K+k][s] = phi[2(sn-s)+1, k]  if p == 1 (s <= sn) | phi[2(sn-s)-1, k] if p == 0 (s < sn)
// Rows of parity p use the even columns (E), rows of parity 1-p the odd ones (Q);
// full_decode_combine_kernel forms U+- = E +- Q as the [B][2*K*d] operand of the contraction with
// [M_phi_plus; M_phi_minus] and advances the positions.  The same kernel first appends the new input.
template <typename T>
__global__ void __launch_bounds__(256) full_decode_prepare_kernel(const T* __restrict__ x, long long x_rstride,
                                                                  T* __restrict__ hist, const T* __restrict__ phi,
                                                                  const int* __restrict__ pos, T* __restrict__ PhiT,
                                                                  int B, int d, int K, int L, int Lh,
                                                                  int* __restrict__ status) {
  const int t = pos[0];
  if (t < 0 || t >= 2 * Lh || t >= L) {
    if (blockIdx.x == 0 && threadIdx.x == 0 && status) atomicExch(status, 2);
    return;
  }
  const int p = t & 1, sn = t >> 1;
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, gsz = (size_t)gridDim.x * blockDim.x;
  // append x_t
  for (size_t e = gid; e < (size_t)B * d; e += gsz) {
    const int b = (int)(e / d), c = (int)(e % d);
    hist[hist_off(b, c, t, d, Lh)] = x[(size_t)b * x_rstride + c];
  }
  // reversed taps
  for (size_t e = gid; e < (size_t)2 * K * Lh; e += gsz) {
    const int s = (int)(e % Lh), r = (int)(e / Lh);
    const int k = r % K, odd = r / K;
    int j = 2 * (sn - s);
    if (odd) j += p ? 1 : -1;
    T v = Elem<T>::from_f(0.f);
    if (s <= sn && j >= 0 && j < L) v = phi[(size_t)j * K + k];
    PhiT[e] = v;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) full_decode_combine_kernel(const T* __restrict__ G, long long ldG,
                                                                  int* __restrict__ pos, T* __restrict__ U, int B,
                                                                  int d, int K, int both_signs, int Lh) {
  const int t = pos[0];
  if (t >= 0 && t < 2 * Lh) {
    const int p = t & 1;
    const size_t total = (size_t)B * K * d;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
      const int i = (int)(e % d), k = (int)((e / d) % K), b = (int)(e / ((size_t)d * K));
      const size_t rowE = ((size_t)b * d + i) * 2 + p, rowQ = ((size_t)b * d + i) * 2 + (1 - p);
      const float ev = Elem<T>::to_f(G[rowE * ldG + k]), qv = Elem<T>::to_f(G[rowQ * ldG + K + k]);
      T* row = U + (size_t)b * (both_signs ? 2 : 1) * K * d;
      row[(size_t)k * d + i] = Elem<T>::from_f(ev + qv);
      if (both_signs) row[(size_t)(K + k) * d + i] = Elem<T>::from_f(ev - qv);
    }
  }
}

__global__ void advance_pos_kernel(int* pos, int B, int inc, int limit) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) {
    const int t = pos[2 * b];
    if (t >= 0 && t + inc <= limit) pos[2 * b] = t + inc;
  }
}

extern "C" int stu_full_decode_prepare(const void* x, long long x_row_stride, void* hist, const void* phi,
                                       const int* pos, void* PhiT, int B, int d, int K, int L, int Lh, int* status,
                                       int dtype, void* stream) {
  if (!x || !hist || !phi || !pos || !PhiT) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || K <= 0 || L <= 0 || Lh <= 0) return STU_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = 592;
  if (dtype == STU_F32)
    full_decode_prepare_kernel<float><<<grid, 256, 0, st>>>((const float*)x, x_row_stride, (float*)hist,
                                                            (const float*)phi, pos, (float*)PhiT, B, d, K, L, Lh,
                                                            status);
  else if (dtype == STU_BF16)
    full_decode_prepare_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)x, x_row_stride, (bf16*)hist,
                                                           (const bf16*)phi, pos, (bf16*)PhiT, B, d, K, L, Lh, status);
  else
    return STU_ERR_DTYPE;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// G: [B*d*2][ldG] with 2K columns from the GEMM above; U: [B][2*K*d] (or [B][K*d] with both_signs=0).
// advance != 0 moves every position forward by one afterwards (a second tiny launch).
extern "C" int stu_full_decode_combine(const void* G, long long ldG, int* pos, void* U, int B, int d, int K,
                                       int both_signs, int Lh, int advance, int dtype, void* stream) {
  if (!G || !pos || !U) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || K <= 0 || ldG < 2 * K) return STU_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = 296;
  if (dtype == STU_F32)
    full_decode_combine_kernel<float><<<grid, 256, 0, st>>>((const float*)G, ldG, pos, (float*)U, B, d, K,
                                                            both_signs, Lh);
  else if (dtype == STU_BF16)
    full_decode_combine_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)G, ldG, pos, (bf16*)U, B, d, K, both_signs,
                                                           Lh);
  else
    return STU_ERR_DTYPE;
  STU_CHECK_LAUNCH();
  if (advance) {
    advance_pos_kernel<<<(B + 127) / 128, 128, 0, st>>>(pos, B, 1, 2 * Lh);
    STU_CHECK_LAUNCH();
  }
  return STU_OK;
}
