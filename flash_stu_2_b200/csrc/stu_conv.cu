// STU spectral convolution, approx variant (project, then depthwise causal convolution).
//
// Reference semantics (flash_stu/modules/stu.py:85-98,120 + flash_stu/utils/stu_utils.py:208-228):
//   xp = x @ M_inputs ; fp = phi @ M_filters ; y = conv(xp, fp) + sgn * conv(sgn * xp, fp)
// The two branches share one filter, so the odd taps cancel:  y[t] = 2 * sum_{j even} fp[j] * xp[t-j].
// An even-tap convolution never mixes time parities, which is why the projected history is kept
// parity-split and time-major per channel ([B][d][2][Lh], see hist_off): for one (sequence, channel,
// parity) both the prefill convolution and the decode dot product walk one contiguous run.
//
// Kernels here:
//   taps_even_kernel     fp[L][d] -> taps[d][Lh] (even taps, channel-major)
//   conv_simt_kernel     fp32-accurate CUDA-core convolution (fp32 models, any Lh that fits smem)
//   conv_mma_kernel      bf16: lower-triangular Toeplitz product on mma.sync tensor cores, the
//                        Toeplitz fragments read straight from two shifted copies of the reversed taps
//   transpose_add_kernel x[b,t,c] += yT[b][c][t&1][t>>1]   (residual add, back to token-major)
//   stu_decode_kernel    one fused decode step: RMSNorm + M_inputs row + history append + tap dot +
//                        residual, one warp per (sequence, channel)
#include <stdlib.h>

#include "common.cuh"

// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void taps_even_kernel(const T* __restrict__ fp, T* __restrict__ taps, int L, int d, int Lh) {
  __shared__ T tile[32][33];
  int j0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int j = j0 + r, c = c0 + threadIdx.x;
    tile[r][threadIdx.x] = (2 * j < L && c < d) ? fp[(size_t)(2 * j) * d + c] : Elem<T>::from_f(0.f);
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int c = c0 + r, j = j0 + threadIdx.x;
    if (c < d && j < Lh) taps[(size_t)c * Lh + j] = tile[threadIdx.x][r];
  }
}

extern "C" int stu_taps_even(const void* fp, void* taps, int L, int d, int Lh, int dtype, void* stream) {
  if (!fp || !taps) return STU_ERR_NULL;
  if (L <= 0 || d <= 0 || Lh < (L + 1) / 2) return STU_ERR_SHAPE;
  dim3 grid((Lh + 31) / 32, (d + 31) / 32), block(32, 8);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == STU_F32)
    taps_even_kernel<float><<<grid, block, 0, st>>>((const float*)fp, (float*)taps, L, d, Lh);
  else if (dtype == STU_BF16)
    taps_even_kernel<bf16><<<grid, block, 0, st>>>((const bf16*)fp, (bf16*)taps, L, d, Lh);
  else
    return STU_ERR_DTYPE;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// Number of history elements of parity p among times [0, t_end), and first/last output index.
__host__ __device__ __forceinline__ int parity_count(int t_end, int p) { return (t_end - p + 1) >> 1; }

// ------------------------------------------------------------------------------------------------
// CUDA-core convolution.  grid (d, 2B); one (sequence, channel, parity) row per CTA.  Each thread owns
// four consecutive outputs and slides a 7-tap register window; taps and history are staged in
// shared memory as fp32 with three leading zeros so that the causal boundary needs no branch.
template <typename T>
__global__ void __launch_bounds__(256) conv_simt_kernel(const T* __restrict__ hist, const T* __restrict__ taps,
                                                        T* __restrict__ yT, int d, int Lh, int Lhy, int t0, int t_end) {
  extern __shared__ __align__(16) float sm[];
  const int c = blockIdx.x, row = blockIdx.y, b = row >> 1, p = row & 1;
  const int cnt = parity_count(t_end, p);  // valid inputs / end of outputs
  const int m_lo = parity_count(t0, p);    // first output of this call
  if (cnt <= m_lo) return;
  const int n4 = (cnt + 3) & ~3;
  float* g = sm;            // g[i] = taps[i-3] (i>=3) else 0, length n4+4
  float* h = sm + n4 + 4;   // h[i] = hist[i] (i<cnt) else 0, length n4
  const size_t rbase = ((size_t)((size_t)b * d + c) * 2 + p) * Lh;
  for (int i = threadIdx.x; i < n4 + 4; i += 256)
    g[i] = (i >= 3 && i - 3 < cnt) ? Elem<T>::to_f(taps[(size_t)c * Lh + (i - 3)]) : 0.f;
  for (int i = threadIdx.x; i < n4; i += 256) h[i] = (i < cnt) ? Elem<T>::to_f(hist[rbase + i]) : 0.f;
  __syncthreads();
  const int mstart = m_lo & ~3;
  for (int m0 = mstart + 4 * threadIdx.x; m0 < cnt; m0 += 1024) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    // window w[i] = g[(m0 - s) + i], i = 0..6, for the block of four inputs s..s+3:
    // acc[r] += h[s+u] * g[m0 + r - (s+u) + 3] = h[s+u] * w[r - u + 3]
    for (int s = 0; s <= m0; s += 4) {
      float4 h4 = *reinterpret_cast<const float4*>(h + s);
      float4 wa = *reinterpret_cast<const float4*>(g + (m0 - s));
      float4 wb = *reinterpret_cast<const float4*>(g + (m0 - s) + 4);
      float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
      float hv[4] = {h4.x, h4.y, h4.z, h4.w};
#pragma unroll
      for (int u = 0; u < 4; u++)
#pragma unroll
        for (int r = 0; r < 4; r++) acc[r] = fmaf(hv[u], w[r - u + 3], acc[r]);
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
      int m = m0 + r;
      if (m >= m_lo && m < cnt)
        yT[((size_t)((size_t)b * d + c) * 2 + p) * Lhy + m] = Elem<T>::from_f(2.f * acc[r]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Tensor-core convolution (bf16).  For one channel the even-tap convolution of all 2B parity rows is
//   Y^T[m][n] = sum_s Tz[m][s] * H^T[s][n],   Tz[m][s] = g[m-s] (0 above the diagonal),
// a lower-triangular Toeplitz product.  mma.sync m16n8k16 takes A = a 16x16 Toeplitz tile, whose
// fragment registers are pairs (g[x], g[x-1]); these are read as single 32-bit words from two
// copies of the *reversed* taps in shared memory (one shifted by one element so that either
// alignment is a word), so no Toeplitz matrix is ever materialised.  A tile depends only on
// (m-tile - k-tile), so a warp that owns four consecutive m-tiles keeps a sliding window of 15
// words and fetches two new words per k-step.  B = 16 consecutive inputs x 8 parity rows from a
// staged history chunk.
constexpr int CM_SB = 512;     // outputs per CTA step (8 warps x 64)
constexpr int CM_KC = 512;     // inputs staged per step
constexpr int CM_HLD = CM_KC + 8;  // history row stride (elements): 260 words == 4 mod 32 banks
constexpr int CM_RW = 528;     // words per reversed-tap copy (1024 + slack elements)

__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(256) conv_mma_kernel(const bf16* __restrict__ hist, const bf16* __restrict__ taps,
                                                       bf16* __restrict__ yT, int B, int d, int Lh, int Lhy,
                                                       int t0, int t_end) {
  __shared__ __align__(16) bf16 Hs[16 * CM_HLD];
  __shared__ __align__(16) uint32_t Rev[2][CM_RW];  // [0]: words (R[2w],R[2w+1]); [1]: (R[2w+1],R[2w+2])
  const int c = blockIdx.x, row0 = blockIdx.y * 16, nrows = 2 * B;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gi = lane >> 2, q = lane & 3;
  const int cnt_max = parity_count(t_end, 0);  // parity 0 holds the larger count
  const int mlo_min = parity_count(t0, 1);     // smallest first output index over parities
  const unsigned short* tg = reinterpret_cast<const unsigned short*>(taps + (size_t)c * Lh);

  for (int M0 = (mlo_min / CM_SB) * CM_SB; M0 < cnt_max; M0 += CM_SB) {
    // A superblock's cost grows with its index (causal: K0 <= M0).  The superblocks of a channel are dealt to two
    // CTAs (blockIdx.z) as {0,3,4,7,...} and {1,2,5,6,...}, which have equal cost, so that the grid is twice as
    // fine and its last wave half as long.
    const int sbi = M0 / CM_SB;
    if ((int)(((sbi & 3) == 1) || ((sbi & 3) == 2)) != (int)blockIdx.z) continue;
    float acc[4][2][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 2; j++)
#pragma unroll
        for (int r = 0; r < 4; r++) acc[i][j][r] = 0.f;

    for (int K0 = 0; K0 <= M0; K0 += CM_KC) {
      __syncthreads();  // previous step's readers are done
      // ---- stage 16 history rows x CM_KC inputs (zero beyond each row's valid count / row range)
      for (int v = tid; v < 16 * (CM_KC / 8); v += 256) {
        int n = v / (CM_KC / 8), s8 = (v % (CM_KC / 8)) * 8;
        int rg = row0 + n;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (rg < nrows) {
          int b = rg >> 1, p = rg & 1;
          int cnt = parity_count(t_end, p);
          int s = K0 + s8;
          const bf16* src = hist + ((size_t)((size_t)b * d + c) * 2 + p) * Lh + s;
          if (s + 8 <= cnt) {
            val = *reinterpret_cast<const uint4*>(src);
          } else if (s < cnt) {
            unsigned short e[8];
#pragma unroll
            for (int u = 0; u < 8; u++) e[u] = (s + u < cnt) ? reinterpret_cast<const unsigned short*>(src)[u] : 0;
            val = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
          }
        }
        *reinterpret_cast<uint4*>(Hs + n * CM_HLD + s8) = val;
      }
      // ---- stage reversed taps: R[y] = g[Gtop - y], Gtop = M0 - K0 + 511, zero outside [0, cnt_max)
      const int Gtop = M0 - K0 + (CM_SB - 1);
      for (int w = tid; w < CM_RW; w += 256) {
        unsigned short e[3];
#pragma unroll
        for (int u = 0; u < 3; u++) {
          int gidx = Gtop - (2 * w + u);
          e[u] = (gidx >= 0 && gidx < cnt_max) ? tg[gidx] : (unsigned short)0;
        }
        Rev[0][w] = e[0] | ((uint32_t)e[1] << 16);
        Rev[1][w] = e[1] | ((uint32_t)e[2] << 16);
      }
      __syncthreads();

      // ---- this warp: outputs M0 + 64*warp .. +63 (four m-tiles), k-tiles of the chunk up to the diagonal
      const int mw = M0 + 64 * warp;
      int kt_end = CM_KC / 16;
      if (K0 == M0) kt_end = min(kt_end, 4 * warp + 4);
      if (mw >= cnt_max) kt_end = 0;
      // y index of word P(j') = ybase + 8 j' ; ybase = Gtop - (M0 - K0 + 64 warp) - gi + 2q
      const int ybase = (CM_SB - 1) - 64 * warp - gi + 2 * q;
      const uint32_t* Rsel = Rev[ybase & 1];
      const int wbase = ybase >> 1;
      // window P[i] = P(2*kt0 - 7 + i), i = 0..14, for the 4 k-steps kt0..kt0+3
      uint32_t P[15];
#pragma unroll
      for (int i = 0; i < 15; i++) P[i] = 0;
      for (int kt0 = 0; kt0 < kt_end; kt0 += 4) {
        if (kt0 == 0) {
#pragma unroll
          for (int i = 0; i < 15; i++) {
            int w = wbase + 4 * (-7 + i);
            P[i] = (w >= 0) ? Rsel[w] : 0u;  // w < 0 only for taps beyond this warp's diagonal (zero by causality)
          }
        } else {
#pragma unroll
          for (int i = 0; i < 7; i++) P[i] = P[i + 8];
#pragma unroll
          for (int i = 7; i < 15; i++) P[i] = Rsel[wbase + 4 * (2 * kt0 - 7 + i)];
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int kt = kt0 + u;
          if (kt < kt_end) {
            uint32_t b[2][2];
#pragma unroll
            for (int j = 0; j < 2; j++) {
              const uint32_t* hp = reinterpret_cast<const uint32_t*>(Hs + (8 * j + gi) * CM_HLD) + 8 * kt + q;
              b[j][0] = hp[0];
              b[j][1] = hp[4];
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
              // fragment F(kt - i): a0a1 = P(2(kt-i)), a2a3 = P(2(kt-i)-1), a4a5 = P(2(kt-i)+1), a6a7 = a0a1
              const int base = 2 * (u - i) + 7;  // index of P(2(kt-i)) inside the window
              uint32_t a01 = P[base], a23 = P[base - 1], a45 = P[base + 1];
#pragma unroll
              for (int j = 0; j < 2; j++) mma_bf16(acc[i][j], a01, a23, a45, a01, b[j][0], b[j][1]);
            }
          }
        }
      }
    }
    // ---- write this superblock: yT row (b,c,p), index m, value round(2*acc)
    const int mw = M0 + 64 * warp;
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 2; j++)
#pragma unroll
        for (int r = 0; r < 4; r++) {
          int m = mw + 16 * i + gi + ((r >> 1) << 3);
          int rg = row0 + 8 * j + 2 * q + (r & 1);
          if (rg < nrows) {
            int b = rg >> 1, p = rg & 1;
            if (m >= parity_count(t0, p) && m < parity_count(t_end, p))
              yT[((size_t)((size_t)b * d + c) * 2 + p) * Lhy + m] = __float2bfloat16_rn(2.f * acc[i][j][r]);
          }
        }
  }
}

// ------------------------------------------------------------------------------------------------
// x[b, t - t0, c] = round(x + yT[b][c][t&1][t>>1]) for t in [t0, t_end).  One CTA moves 128 times x 8*V
// channels: 16-byte loads along time from the two parity rows of each channel into a padded shared
// tile, then 16-byte read-modify-writes along channels of the token-major residual stream.
template <typename T>
__global__ void __launch_bounds__(256) transpose_add_kernel(T* __restrict__ x, long long x_bstride,
                                                            long long x_tstride, const T* __restrict__ yT, int d,
                                                            int Lh, int t0, int t_end) {
  constexpr int V = Elem<T>::VEC;           // elements per 16 bytes
  constexpr int TC = 8 * V;                 // channels per CTA (64 bf16 / 32 fp32)
  constexpr int TS = 64;                    // time indices per parity per CTA
  constexpr int SROW = (sizeof(T) == 2) ? 66 : 65;  // row pitch in elements: odd number of 32-bit words
  __shared__ __align__(16) T tile[2][TC][SROW];
  // tile origin: the first time is rounded down to a multiple of 2V so that sb is a multiple of V and the
  // 16-byte loads along a parity row stay aligned for any t0
  const int b = blockIdx.z, c0 = blockIdx.y * TC, tb = (t0 - t0 % (2 * V)) + blockIdx.x * (2 * TS);
  const int sb = tb >> 1;
  constexpr int NV = TS / V;
  for (int item = threadIdx.x; item < 2 * TC * NV; item += 256) {
    const int p = item / (TC * NV), c = (item / NV) % TC, v = item % NV;
    const int s = sb + v * V;
    float val[V];
#pragma unroll
    for (int j = 0; j < V; j++) val[j] = 0.f;
    if (c0 + c < d && s + V <= Lh) load_vec(yT + ((size_t)((size_t)b * d + c0 + c) * 2 + p) * Lh + s, val);
#pragma unroll
    for (int j = 0; j < V; j++) tile[p][c][v * V + j] = Elem<T>::from_f(val[j]);
  }
  __syncthreads();
  for (int item = threadIdx.x; item < 2 * TS * 8; item += 256) {
    const int tl = item >> 3, cg = item & 7;
    const int t = tb + tl, c = c0 + cg * V;
    if (t >= t0 && t < t_end && c < d) {
      T* px = x + (size_t)b * x_bstride + (size_t)(t - t0) * x_tstride + c;
      const int p = tl & 1, si = tl >> 1;
      if (c + V <= d && ((reinterpret_cast<uintptr_t>(px) & 15u) == 0)) {
        float xv[V];
        load_vec(px, xv);
#pragma unroll
        for (int j = 0; j < V; j++) xv[j] += Elem<T>::to_f(tile[p][cg * V + j][si]);
        store_vec(px, xv);
      } else {
        for (int j = 0; j < V && c + j < d; j++)
          px[j] = Elem<T>::from_f(Elem<T>::to_f(px[j]) + Elem<T>::to_f(tile[p][cg * V + j][si]));
      }
    }
  }
}

// Residual add of a finished convolution: x[b, t - t0, :] += yT[b][:][t&1][t>>1] for t in [t0, t_end).
int launch_transpose_add(void* x, long long x_bstride, long long x_tstride, const void* yT, int B, int d, int y_Lh,
                         int t0, int t_end, int dtype, cudaStream_t st) {
  const int v2 = (dtype == STU_F32) ? 8 : 16;  // 2V: the kernel aligns its first tile to this
  int tb = t0 - t0 % v2;
  const int tc = (dtype == STU_F32) ? 32 : 64;
  dim3 g2((t_end - tb + 127) / 128, (d + tc - 1) / tc, B);
  if (dtype == STU_F32)
    transpose_add_kernel<float><<<g2, 256, 0, st>>>((float*)x, x_bstride, x_tstride, (const float*)yT, d, y_Lh, t0,
                                                    t_end);
  else
    transpose_add_kernel<bf16><<<g2, 256, 0, st>>>((bf16*)x, x_bstride, x_tstride, (const bf16*)yT, d, y_Lh, t0,
                                                   t_end);
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// Prefill convolution entry point: hist holds projected inputs for times [0, t_end); computes the
// convolution outputs for times [t0, t_end) into yT (same layout as hist, y_Lh elements per parity row) and adds them to x
// ([B, t_end - t0, d] with the given strides).  use_tensor_cores selects conv_mma_kernel (bf16).
extern "C" int stu_conv_prefill_approx(const void* hist, const void* taps, void* yT, void* x, long long x_bstride,
                                       long long x_tstride, int B, int d, int Lh, int y_Lh, int t0, int t_end,
                                       int dtype, int use_tensor_cores, void* stream) {
  if (!hist || !taps || !yT || !x) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || Lh <= 0 || t0 < 0 || t_end <= t0 || t_end > 2 * Lh || t_end > 2 * y_Lh)
    return STU_ERR_SHAPE;
  if (dtype != STU_F32 && dtype != STU_BF16) return STU_ERR_DTYPE;
  // the residual add reads yT with 16-byte loads along a parity row: the base and the row pitch must keep every
  // row start on a 16-byte boundary (y_Lh a multiple of 8 for bf16, of 4 for fp32)
  if (!aligned16(yT) || y_Lh % (dtype == STU_F32 ? 4 : 8)) return STU_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  if (use_tensor_cores) {
    if (dtype != STU_BF16) return STU_ERR_DTYPE;
    if (Lh % 8 || !aligned16(hist) || (((uintptr_t)taps) & 1u)) return STU_ERR_ALIGN;
    dim3 grid(d, (2 * B + 15) / 16, 2);
    conv_mma_kernel<<<grid, 256, 0, st>>>((const bf16*)hist, (const bf16*)taps, (bf16*)yT, B, d, Lh, y_Lh, t0, t_end);
  } else {
    int cnt = parity_count(t_end, 0);
    int n4 = (cnt + 3) & ~3;
    size_t smem = (size_t)(2 * n4 + 4) * sizeof(float);
    if (smem > 200 * 1024) return STU_ERR_UNSUPPORTED;
    dim3 grid(d, 2 * B);
    if (dtype == STU_F32) {
      cudaError_t e = cudaFuncSetAttribute(conv_simt_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem);
      if (e != cudaSuccess) return (int)e;
      conv_simt_kernel<float><<<grid, 256, smem, st>>>((const float*)hist, (const float*)taps, (float*)yT, d, Lh, y_Lh,
                                                       t0, t_end);
    } else if (dtype == STU_BF16) {
      cudaError_t e = cudaFuncSetAttribute(conv_simt_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem);
      if (e != cudaSuccess) return (int)e;
      conv_simt_kernel<bf16><<<grid, 256, smem, st>>>((const bf16*)hist, (const bf16*)taps, (bf16*)yT, d, Lh, y_Lh, t0,
                                                      t_end);
    } else {
      return STU_ERR_DTYPE;
    }
  }
  STU_CHECK_LAUNCH();
  return launch_transpose_add(x, x_bstride, x_tstride, yT, B, d, y_Lh, t0, t_end, dtype, st);
}

// ------------------------------------------------------------------------------------------------
// Fused decode step of one approx STU layer.  grid (d, ceil(B/8)); warp w of a CTA serves sequence
// b = 8*blockIdx.y + w for channel c = blockIdx.x:
//   xn   = rmsnorm(x[b,:]) * norm_w                        (rounded to T, as the reference's norm output)
//   xp   = round(xn . MinT[c,:])                           (row c of M_inputs^T)
//   hist[b][c][t&1][t>>1] = xp
//   y    = round(2 * sum_{j'<=t>>1} taps[c][j'] * hist[b][c][t&1][(t>>1)-j'])
//   out[b,c] = round(x[b,c] + y)
// with t = pos[2*b].  The taps are staged reversed in shared memory so that both operands of the
// dot product are ascending 128-bit vectors.  The last CTA to finish advances every pos[2*b] by one
// (pos[1] is the arrival counter), so a captured graph can be replayed without host-side arguments.
__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void unpack_vec(const uint4& v, float (&out)[8], bf16) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void unpack_vec(const uint4& v, float (&out)[4], float) {
  out[0] = __uint_as_float(v.x); out[1] = __uint_as_float(v.y);
  out[2] = __uint_as_float(v.z); out[3] = __uint_as_float(v.w);
}

// The kernel is latency-bound unless many loads are in flight, so the order of work is: read the
// positions, issue the first DEC_U 16-byte history loads of the warp's run and the CTA's tap loads,
// then do the RMSNorm / projection (whose own loads overlap the ones in flight), then reverse the taps
// into shared memory, then consume.
constexpr int DEC_U = 8;

template <typename T>
__global__ void __launch_bounds__(256) stu_decode_kernel(const T* __restrict__ x, long long x_rstride,
                                                         const T* __restrict__ norm_w, const T* __restrict__ MinT,
                                                         T* __restrict__ hist, const T* __restrict__ taps,
                                                         int* __restrict__ pos, T* __restrict__ out,
                                                         long long out_rstride, int B, int d, int Lh, float eps,
                                                         int* __restrict__ status) {
  constexpr int V = Elem<T>::VEC;
  extern __shared__ __align__(16) unsigned char smraw[];
  T* tr = reinterpret_cast<T*>(smraw);  // tr[i] = taps[c][smax - i], i = 0..smax, zero padded to a vector
  const int c = blockIdx.x, b0 = blockIdx.y * 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = b0 + warp;
  const bool active = b < B;
  // positions of the (up to eight) sequences of this CTA; every thread derives smax without a barrier
  int smax = 0, t = 0;
  bool bad = false;
#pragma unroll
  for (int w = 0; w < 8; w++) {
    if (b0 + w < B) {
      int tw = pos[2 * (b0 + w)];
      bool badw = (tw < 0 || tw >= 2 * Lh);
      if (badw) tw = 0;
      smax = max(smax, tw >> 1);
      if (w == warp) { t = tw; bad = badw; }
    }
  }
  if (bad && lane == 0 && status) atomicExch(status, 2);
  const int p = t & 1, s = t >> 1;
  const bool run = active && !bad;
  T* hrow = hist + ((size_t)((size_t)(run ? b : 0) * d + c) * 2 + p) * Lh;
  const int sh = smax - s;                 // offset of this row into the reversed taps
  const bool fast = run && (sh % V) == 0;  // uniform positions: vector path
  const int svec = (s / V) * V;
  // ---- 1. history prefetch (first DEC_U vectors per lane)
  uint4 hraw[DEC_U];
#pragma unroll
  for (int u = 0; u < DEC_U; u++) {
    const int i = (u * 32 + lane) * V;
    hraw[u] = (fast && i < svec) ? ldg_nc_v4(hrow + i) : make_uint4(0, 0, 0, 0);
  }
  // ---- 2. tap loads (forward order, reversed when written to shared memory below)
  const int ntaps = smax + 1;
  const int nvec = (ntaps + V - 1) / V;  // Lh % V == 0, so a partial last vector stays inside the row
  const T* trow = taps + (size_t)c * Lh;
  uint4 traw[2];
#pragma unroll
  for (int u = 0; u < 2; u++) {
    const int v = threadIdx.x + u * 256;
    traw[u] = (v < nvec) ? ldg_nc_v4(trow + v * V) : make_uint4(0, 0, 0, 0);
  }
  // ---- 3. RMSNorm statistic of row b and the projection onto channel c
  float xp = 0.f, xc = 0.f;
  if (run) {
    const T* xr = x + (size_t)b * x_rstride;
    float ss = 0.f;
    for (int k = lane * V; k < d; k += 32 * V) {
      float v[V];
      load_vec(xr + k, v);
#pragma unroll
      for (int j = 0; j < V; j++) ss += v[j] * v[j];
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)d + eps);
    const T* mrow = MinT + (size_t)c * d;
    float dot = 0.f;
    for (int k = lane * V; k < d; k += 32 * V) {
      float v[V], g[V], m[V];
      load_vec(xr + k, v);
      load_vec(norm_w + k, g);
      load_vec(mrow + k, m);
#pragma unroll
      for (int j = 0; j < V; j++) dot = fmaf(round_to<T>(v[j] * r * g[j]), m[j], dot);
    }
    dot = warp_sum(dot);
    xp = round_to<T>(dot);
    xc = Elem<T>::to_f(xr[c]);
    if (lane == 0) hrow[s] = Elem<T>::from_f(xp);
  }
  // ---- 4. reversed taps into shared memory
  const int ntr = nvec * V;
#pragma unroll
  for (int u = 0; u < 2; u++) {
    const int v = threadIdx.x + u * 256;
    if (v < nvec) {
      float tv[V];
      unpack_vec(traw[u], tv, T());
#pragma unroll
      for (int j = 0; j < V; j++) {
        const int tap = v * V + j;            // tap index; destination smax - tap (>= 0 only for real taps)
        if (tap <= smax) tr[smax - tap] = Elem<T>::from_f(tv[j]);
      }
    }
  }
  for (int v = threadIdx.x + 512; v < nvec; v += 256) {  // rows longer than 512 vectors (Lh > 4096 for bf16)
    float tv[V];
    load_vec(trow + v * V, tv);
#pragma unroll
    for (int j = 0; j < V; j++) {
      const int tap = v * V + j;
      if (tap <= smax) tr[smax - tap] = Elem<T>::from_f(tv[j]);
    }
  }
  for (int i = ntaps + threadIdx.x; i < ntr; i += 256) tr[i] = Elem<T>::from_f(0.f);
  __syncthreads();
  // ---- 5. tap dot product over the stored history [0, s); the new element pairs with tap 0 = tr[smax]
  if (run) {
    float acc0 = 0.f, acc1 = 0.f;
    if (fast) {
#pragma unroll
      for (int u = 0; u < DEC_U; u++) {
        const int i = (u * 32 + lane) * V;
        if (i < svec) {
          float hv[V], tv[V];
          unpack_vec(hraw[u], hv, T());
          load_vec(tr + sh + i, tv);
#pragma unroll
          for (int j = 0; j < V; j += 2) {
            acc0 = fmaf(hv[j], tv[j], acc0);
            acc1 = fmaf(hv[j + 1], tv[j + 1], acc1);
          }
        }
      }
      for (int base = DEC_U * 32 * V; base < svec; base += DEC_U * 32 * V) {
        uint4 raw[DEC_U];
#pragma unroll
        for (int u = 0; u < DEC_U; u++) {
          const int i = base + (u * 32 + lane) * V;
          raw[u] = (i < svec) ? ldg_nc_v4(hrow + i) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < DEC_U; u++) {
          const int i = base + (u * 32 + lane) * V;
          if (i < svec) {
            float hv[V], tv[V];
            unpack_vec(raw[u], hv, T());
            load_vec(tr + sh + i, tv);
#pragma unroll
            for (int j = 0; j < V; j += 2) {
              acc0 = fmaf(hv[j], tv[j], acc0);
              acc1 = fmaf(hv[j + 1], tv[j + 1], acc1);
            }
          }
        }
      }
    } else {
      for (int i = lane; i < svec; i += 32) acc0 = fmaf(Elem<T>::to_f(hrow[i]), Elem<T>::to_f(tr[sh + i]), acc0);
    }
    for (int i = svec + lane; i < s; i += 32) acc1 = fmaf(Elem<T>::to_f(hrow[i]), Elem<T>::to_f(tr[sh + i]), acc1);
    float acc = warp_sum(acc0 + acc1);
    if (lane == 0) {
      acc = fmaf(xp, Elem<T>::to_f(tr[smax]), acc);
      const float y = round_to<T>(2.f * acc);
      out[(size_t)b * out_rstride + c] = Elem<T>::from_f(xc + y);
    }
  }
  // ---- arrival counter: the last CTA advances the positions
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    int total = gridDim.x * gridDim.y;
    int old = atomicAdd(&pos[1], 1);
    if (old == total - 1) {
      pos[1] = 0;
      for (int i = 0; i < B; i++) {
        int tv = pos[2 * i];
        if (tv >= 0 && tv < 2 * Lh) pos[2 * i] = tv + 1;
      }
      __threadfence();
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Tensor-core form of the fused decode step (bf16).  The CUDA-core kernel above spends ~26 instructions per 16
// bytes of history (unpack, convert, FMA) and is issue-bound.  Here one warp owns one (sequence, channel) and
// streams that row's history and the channel's reversed taps as whole 512-byte runs (16 bytes per lane per
// instruction, full cache lines).  The dot product of a 256-element run is taken on the tensor cores as the
// DIAGONAL of a 16x16 product: the lane's four history words are the A fragment of mma.sync m16n8k16 (any
// fixed assignment of memory positions to (row, k) slots will do, as long as the taps use the same one), the
// taps words 0/2 and 1/3 are the B fragments of the two n-tiles, and sum_r D[r][r] is the dot product.  That is
// two MMAs per 16-byte load, with the access pattern of the CUDA-core kernel (one contiguous run per warp).
// The taps come from a table stored reversed and in all eight 16-byte alignments (taps8[e][c][Lh+8],
// taps8[e][c][u] = tap[Lh-1-(u+e)]), so the tap operand is an aligned 16-byte load at every position.
// The eight warps of a CTA are the (up to) eight sequences of one channel.  When they all stand at the same
// position (the usual case in batched generation) the channel's reversed tap row is copied once into shared
// memory and every warp takes its B fragments from there: the taps then cross the L2-to-SM fabric once per CTA
// instead of once per warp, which halves the kernel's load traffic, and the registers that held tap words hold
// history words instead (eight 512-byte runs in flight per warp).  With ragged positions every warp streams
// its own alignment of the table from global memory (four runs of history and four of taps in flight).
constexpr int DD_U = 8;  // uint4 registers per lane for data in flight

__device__ __forceinline__ uint4 lds_v4(const bf16* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"((uint32_t)__cvta_generic_to_shared(p)));
  return v;
}

// Masked A fragment of the last, partial run: elements [i0, i0 + 8) of which the first `keep` are history.
__device__ __forceinline__ void mask_tail(uint32_t (&a)[4], const uint4& raw, int keep) {
  a[0] = raw.x; a[1] = raw.y; a[2] = raw.z; a[3] = raw.w;
  if (keep < 8) {
#pragma unroll
    for (int jj = 0; jj < 4; jj++) {
      if (2 * jj + 1 >= keep) a[jj] = (2 * jj < keep) ? (a[jj] & 0x0000ffffu) : 0u;
    }
  }
}

// diagonal of the two accumulator tiles: D0[g][g] sits in lane (g, q = g/2) register g&1; D1[g+8][g] in the same
// lane, register 2+(g&1)
__device__ __forceinline__ float diag_part(const float (&acc0)[4], const float (&acc1)[4], int lane) {
  const int g = lane >> 2, q = lane & 3;
  return (q == (g >> 1)) ? ((g & 1) ? (acc0[1] + acc1[3]) : (acc0[0] + acc1[2])) : 0.f;
}

// Ragged positions: the warp streams its own alignment of the tap table from global memory (four runs of
// history and four of taps in flight).  Kept out of line so that its registers do not add to the common path.
__device__ __noinline__ float ragged_tap_dot(const bf16* __restrict__ hrow, const bf16* __restrict__ trow, int s,
                                             int lane) {
  constexpr int RU = 4;
  const int nfull = s >> 8;
  float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
  uint4 hv[RU], tv[RU];
  for (int j0 = 0; j0 < nfull; j0 += RU) {
#pragma unroll
    for (int u = 0; u < RU; u++) {
      if (j0 + u < nfull) {
        hv[u] = ldg_nc_v4(hrow + ((j0 + u) << 8) + 8 * lane);
        tv[u] = ldg_nc_v4(trow + ((j0 + u) << 8) + 8 * lane);
      }
    }
#pragma unroll
    for (int u = 0; u < RU; u++) {
      if (j0 + u < nfull) {  // warp-uniform
        mma_bf16(acc0, hv[u].x, hv[u].y, hv[u].z, hv[u].w, tv[u].x, tv[u].z);
        mma_bf16(acc1, hv[u].x, hv[u].y, hv[u].z, hv[u].w, tv[u].y, tv[u].w);
      }
    }
  }
  if (s & 255) {
    const int i0 = (nfull << 8) + 8 * lane;
    const int keep = s - i0;
    uint32_t a[4] = {0u, 0u, 0u, 0u};
    uint4 tt = make_uint4(0, 0, 0, 0);
    if (keep > 0) {
      mask_tail(a, ldg_nc_v4(hrow + i0), keep);
      tt = ldg_nc_v4(trow + i0);
    }
    mma_bf16(acc0, a[0], a[1], a[2], a[3], tt.x, tt.z);
    mma_bf16(acc1, a[0], a[1], a[2], a[3], tt.y, tt.w);
  }
  return diag_part(acc0, acc1, lane);
}

__global__ void __launch_bounds__(256, 4) stu_decode_diag_kernel(const bf16* __restrict__ x, long long x_rstride,
                                                              const bf16* __restrict__ norm_w,
                                                              const bf16* __restrict__ MinT, bf16* __restrict__ hist,
                                                              const bf16* __restrict__ taps8, int* __restrict__ pos,
                                                              bf16* __restrict__ out, long long out_rstride, int B,
                                                              int d, int Lh, float eps, int* __restrict__ status,
                                                              int pdl) {
  extern __shared__ __align__(16) unsigned char dd_smem[];
  bf16* s_tap = reinterpret_cast<bf16*>(dd_smem);  // [Lh + 8] reversed taps of this channel (uniform positions)
  __shared__ int s_t[8];
  if (pdl & STU_FLAG_EARLY_TRIGGER) pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5;
  const int c = blockIdx.x, b = blockIdx.y * 8 + warp;
  const int lane = threadIdx.x & 31;
  const int LP = Lh + 8;
  const bool inb = b < B;
  const int t = inb ? pos[2 * b] : -1;
  const bool run = inb && t >= 0 && t < 2 * Lh;
  if (inb && !run && lane == 0 && status) atomicExch(status, 2);
  if (lane == 0) s_t[warp] = run ? t : -1;
  const int p = t & 1, s = run ? (t >> 1) : 0;
  bf16* hrow = hist + ((size_t)((size_t)(inb ? b : 0) * d + c) * 2 + p) * Lh;
  // own alignment of the tap table (ragged positions): trow[i] = tap[s - i], 16-byte aligned
  auto tap_row = [&]() {
    const int o = Lh - 1 - s, e = o & 7;
    return taps8 + ((size_t)e * d + c) * LP + (o - e);
  };
  const int nfull = s >> 8;  // complete 256-element runs before s
  __syncthreads();
  // uniform: every sequence of this CTA that runs stands at the same position
  int tu = -1;
  bool uniform = true;
#pragma unroll
  for (int w = 0; w < 8; w++) {
    const int tw = s_t[w];
    if (tw >= 0) {
      if (tu < 0) tu = tw;
      else if (tw != tu) uniform = false;
    }
  }
  uint4 hv[DD_U];
  if (uniform) {
    if (run) {  // first half of the first round now, second half after the projection (register budget)
#pragma unroll
      for (int u = 0; u < DD_U / 2; u++)
        if (u < nfull) hv[u] = ldg_nc_v4(hrow + (u << 8) + 8 * lane);
    }
    if (tu >= 0) {  // all threads copy the tap row of position tu: elements [0, roundup8(su))
      const int su = tu >> 1;
      const int ou = Lh - 1 - su, eu = ou & 7;
      const bf16* tr = taps8 + ((size_t)eu * d + c) * LP + (ou - eu);
      const int nv = (su + 7) >> 3;
      for (int i = threadIdx.x; i < nv; i += 256) *reinterpret_cast<uint4*>(s_tap + 8 * i) = ldg_nc_v4(tr + 8 * i);
    }
  }
  // ---- RMSNorm statistic of row b and the projection onto channel c (overlaps the loads above)
  float xp = 0.f;
  const bf16* xr = x + (size_t)(inb ? b : 0) * x_rstride;
  if (run) {
    float ss = 0.f;
    for (int k = lane * 8; k < d; k += 256) {
      float v[8];
      load_vec(xr + k, v);
#pragma unroll
      for (int j = 0; j < 8; j++) ss += v[j] * v[j];
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)d + eps);
    const bf16* mrow = MinT + (size_t)c * d;
    float dot = 0.f;
    for (int k = lane * 8; k < d; k += 256) {
      float v[8], gw[8], m[8];
      load_vec(xr + k, v);
      load_vec(norm_w + k, gw);
      load_vec(mrow + k, m);
#pragma unroll
      for (int j = 0; j < 8; j++) dot = fmaf(round_to<bf16>(v[j] * r * gw[j]), m[j], dot);
    }
    dot = warp_sum(dot);
    xp = round_to<bf16>(dot);
    if (lane == 0) hrow[s] = __float2bfloat16_rn(xp);
    if (uniform) {
#pragma unroll
      for (int u = DD_U / 2; u < DD_U; u++)
        if (u < nfull) hv[u] = ldg_nc_v4(hrow + (u << 8) + 8 * lane);
    }
  }
  __syncthreads();  // the tap row is in shared memory
  if (run) {
    // ---- tap dot product over the stored history [0, s)
    float part;
    if (uniform) {
      float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
      for (int j0 = 0; j0 < nfull; j0 += DD_U) {
        if (j0) {
#pragma unroll
          for (int u = 0; u < DD_U; u++)
            if (j0 + u < nfull) hv[u] = ldg_nc_v4(hrow + ((j0 + u) << 8) + 8 * lane);
        }
#pragma unroll
        for (int u = 0; u < DD_U; u++) {
          if (j0 + u < nfull) {  // warp-uniform
            const uint4 tv = lds_v4(s_tap + ((j0 + u) << 8) + 8 * lane);
            mma_bf16(acc0, hv[u].x, hv[u].y, hv[u].z, hv[u].w, tv.x, tv.z);
            mma_bf16(acc1, hv[u].x, hv[u].y, hv[u].z, hv[u].w, tv.y, tv.w);
          }
        }
      }
      if (s & 255) {  // last, partial run: elements [256*nfull, s)
        const int i0 = (nfull << 8) + 8 * lane;
        const int keep = s - i0;
        uint32_t a[4] = {0u, 0u, 0u, 0u};
        uint4 tt = make_uint4(0, 0, 0, 0);
        if (keep > 0) {
          mask_tail(a, ldg_nc_v4(hrow + i0), keep);
          tt = lds_v4(s_tap + i0);
        }
        mma_bf16(acc0, a[0], a[1], a[2], a[3], tt.x, tt.z);
        mma_bf16(acc1, a[0], a[1], a[2], a[3], tt.y, tt.w);
      }
      part = diag_part(acc0, acc1, lane);
    } else {
      part = ragged_tap_dot(hrow, tap_row(), s, lane);
    }
    part = warp_sum(part);
    if (lane == 0) {
      const float tap0 = __bfloat162float(taps8[(size_t)c * LP + (Lh - 1)]);
      const float y = round_to<bf16>(2.f * fmaf(xp, tap0, part));
      out[(size_t)b * out_rstride + c] = __float2bfloat16_rn(__bfloat162float(xr[c]) + y);
    }
  }
  // ---- arrival counter: the last CTA advances the positions
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int total = gridDim.x * gridDim.y;
    if (atomicAdd(&pos[1], 1) == total - 1) {
      pos[1] = 0;
      for (int i = 0; i < B; i++) {
        const int tv2 = pos[2 * i];
        if (tv2 >= 0 && tv2 < 2 * Lh) pos[2 * i] = tv2 + 1;
      }
      __threadfence();
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Decode step for a batch whose sequences all stand at the same position (batched generation).
//
// The warp-per-(sequence, channel) kernel above is bound by instruction issue, not by memory: every warp
// recomputes the RMSNorm statistic and the normalised row and takes one row of M_inputs^T through scalar FMAs
// (~700 of its ~900 instructions), while a plain streaming read of the same history runs at 5.2 TB/s.  Here a
// CTA owns 8 channels x 8 sequences and both contractions are real MMAs with the sequences as rows:
//   projection  xp[b][c] = sum_k xn[b][k] MinT[c][k]   rows b, columns = the 8 channels, K split over the 32 warps
//   taps        y[b]     = sum_i hist[b][c][i] tap_c[s-i]   rows b, every column the tap vector of channel c
// Warp w streams channel (w & 7) for all eight sequences over the time slice (w >> 3) of four: a lane's 16-byte
// load is 8 consecutive history values of sequence g = lane / 4, and the k-order inside a 32-value chunk is
// permuted identically for history and taps, so no shuffles are needed.  The eight tap rows are staged once per
// CTA in shared memory (reversed, at the alignment of the common position).
// d is the width of the layer input (rows of x, rows of M_inputs^T); dch the number of channels this launch owns
// (history, taps, output columns): equal for a whole layer, dch = d/g for a tensor-parallel channel shard.
constexpr int R8_U = 8;        // 16-byte history loads a lane keeps in flight
// NW warps per CTA = 8 channels x NW/8 time slices.  One CTA of 32 warps per SM when the grid is small (one wave);
// 16-warp CTAs, two per SM, when there are several waves of CTAs, so that one CTA's prologue (statistics,
// projection, tap staging) overlaps the other's streaming.

__device__ __forceinline__ void mma_rows8(float (&c)[4], const uint4& a, const uint4& b) {
  // rows 8..15 of the A tile are zero (a1 = a3 = 0)
  mma_bf16(c, a.x, 0u, a.y, 0u, b.x, b.y);
  mma_bf16(c, a.z, 0u, a.w, 0u, b.z, b.w);
}

template <int NW>
__global__ void __launch_bounds__(NW * 32, 32 / NW)
    stu_decode_rows8_kernel(const bf16* __restrict__ x, long long x_rstride, const bf16* __restrict__ norm_w,
                            const bf16* __restrict__ MinT, bf16* __restrict__ hist, const bf16* __restrict__ taps8,
                            int* __restrict__ pos, bf16* __restrict__ out, long long out_rstride, int B, int d, int dch,
                            int add_resid, int Lh,
                            float eps, int* __restrict__ status, int pdl) {
  extern __shared__ __align__(16) unsigned char dd_smem[];
  bf16* s_tap = reinterpret_cast<bf16*>(dd_smem);  // [8][Lh + 8]
  constexpr int R8_WARPS = NW, R8_SLICES = NW / 8;
  __shared__ float s_r[8];
  __shared__ float s_red[R8_WARPS][64];
  __shared__ float s_xp[64];
  __shared__ float s_part[R8_SLICES][64];
  if (pdl & STU_FLAG_EARLY_TRIGGER) pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q = lane & 3;
  const int LP = Lh + 8;
  const int c0 = blockIdx.x * 8, b0 = blockIdx.y * 8;
  const int nb = min(8, B - b0);
  // ---- common position of the CTA's sequences
  const int t = pos[2 * b0];
  int bad = (t < 0 || t >= 2 * Lh) ? 1 : 0;
  if (tid < nb && pos[2 * (b0 + tid)] != t) bad = 2;
  bad = __syncthreads_or(bad);
  if (bad) {
    // 2: position outside the cache; 6: the caller promised one common position and the batch is ragged
    if (tid == 0 && status) atomicExch(status, (t < 0 || t >= 2 * Lh) ? 2 : 6);
  } else {
    const int p = t & 1, s = t >> 1;
    const int ch = warp & 7, slice = warp >> 3;
    const int nch = (s + 31) >> 5;  // 32-value chunks of history, the last one partial
    const bool rowok = g < nb;
    const bf16* hrow = hist + ((size_t)((size_t)(b0 + (rowok ? g : 0)) * dch + c0 + ch) * 2 + p) * Lh;
    uint4 hv[R8_U];
    auto issue = [&](int sc) {  // super-chunk sc = R8_U consecutive chunks
#pragma unroll
      for (int u = 0; u < R8_U; u++) {
        const int i0 = ((sc * R8_U + u) << 5) + q * 8;
        hv[u] = (rowok && i0 < s) ? ldg_nc_v4(hrow + i0) : make_uint4(0, 0, 0, 0);
      }
    };
    issue(slice);
    {  // the eight tap rows: elements [0, roundup8(s)) of trow_c[i] = tap_c[s - i]
      const int o = Lh - 1 - s, e = o & 7;
      const int nv = (s + 7) >> 3;
      const bf16* tbase = taps8 + ((size_t)e * dch + c0) * LP + (o - e);
      for (int idx = tid; idx < 8 * nv; idx += R8_WARPS * 32) {
        const int cc = idx / nv, i = idx - cc * nv;
        *reinterpret_cast<uint4*>(s_tap + (size_t)cc * LP + 8 * i) = ldg_nc_v4(tbase + (size_t)cc * LP + 8 * i);
      }
    }
    // ---- RMSNorm statistics of the eight rows
    if (warp < 8) {
      float r = 0.f;
      if (warp < nb) {
        const bf16* xr = x + (size_t)(b0 + warp) * x_rstride;
        float ss = 0.f;
        for (int k = lane * 8; k < d; k += 256) {
          float v[8];
          load_vec(xr + k, v);
#pragma unroll
          for (int j = 0; j < 8; j++) ss += v[j] * v[j];
        }
        ss = warp_sum(ss);
        r = rsqrtf(ss / (float)d + eps);
      }
      if (lane == 0) s_r[warp] = r;
    }
    __syncthreads();
    // ---- projection: rows = sequences, columns = the CTA's channels, K chunks dealt round-robin to the warps
    {
      float accp[4] = {0.f, 0.f, 0.f, 0.f};
      const bf16* xr = x + (size_t)(b0 + (rowok ? g : 0)) * x_rstride;
      const bf16* mrow = MinT + (size_t)(c0 + g) * d;
      const float rg = s_r[g];
      for (int kc = warp; kc < ((d + 31) >> 5); kc += R8_WARPS) {  // warp-uniform trip count
        const int k = (kc << 5) + q * 8;
        const bool kok = (k + 8) <= d;
        uint4 xa = make_uint4(0, 0, 0, 0), wv = make_uint4(0, 0, 0, 0);
        if (kok) {
          wv = *reinterpret_cast<const uint4*>(mrow + k);
          if (rowok) xa = norm_pack(*reinterpret_cast<const uint4*>(xr + k), rg, *reinterpret_cast<const uint4*>(norm_w + k));
        }
        mma_rows8(accp, xa, wv);
      }
      // accp[0], accp[1] = (sequence g, channels 2q, 2q+1)
      s_red[warp][g * 8 + 2 * q] = accp[0];
      s_red[warp][g * 8 + 2 * q + 1] = accp[1];
    }
    __syncthreads();
    if (tid < 64) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < R8_WARPS; w++) sum += s_red[w][tid];
      const float xp = round_to<bf16>(sum);
      s_xp[tid] = xp;
      const int bb = tid >> 3, cc = tid & 7;
      if (bb < nb) hist[((size_t)((size_t)(b0 + bb) * dch + c0 + cc) * 2 + p) * Lh + s] = __float2bfloat16_rn(xp);
    }
    // ---- taps over the stored history [0, s): super-chunks dealt round-robin to the four time slices
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bf16* tp = s_tap + (size_t)ch * LP;
    for (int sc = slice; sc * R8_U < nch; sc += R8_SLICES) {
      if (sc != slice) issue(sc);
#pragma unroll
      for (int u = 0; u < R8_U; u++) {
        if (sc * R8_U + u < nch) {  // warp-uniform: every lane reaches the MMAs
          const int i0 = ((sc * R8_U + u) << 5) + q * 8;
          const int keep = s - i0;  // values of this lane's vector that are history (the rest is masked)
          uint4 tv = make_uint4(0, 0, 0, 0);
          uint32_t a[4] = {0u, 0u, 0u, 0u};
          if (keep > 0) {
            tv = lds_v4(tp + i0);
            mask_tail(a, hv[u], keep);
          }
          mma_rows8(acc, make_uint4(a[0], a[1], a[2], a[3]), tv);
        }
      }
    }
    if (q == 0) s_part[slice][g * 8 + ch] = acc[0];  // every column of the tile holds the same dot product
    __syncthreads();
    if (tid < 64) {
      const int bb = tid >> 3, cc = tid & 7;
      if (bb < nb) {
        float part = 0.f;
#pragma unroll
        for (int sl = 0; sl < R8_SLICES; sl++) part += s_part[sl][tid];
        const float tap0 = __bfloat162float(taps8[(size_t)(c0 + cc) * LP + (Lh - 1)]);
        const float y = round_to<bf16>(2.f * fmaf(s_xp[tid], tap0, part));
        // add_resid: the layer's residual (input width == channel count); a channel shard returns y alone
        const float xin = add_resid ? __bfloat162float(x[(size_t)(b0 + bb) * x_rstride + c0 + cc]) : 0.f;
        out[(size_t)(b0 + bb) * out_rstride + c0 + cc] = __float2bfloat16_rn(xin + y);
      }
    }
  }
  // ---- arrival counter: the last CTA advances the positions
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int total = gridDim.x * gridDim.y;
    if (atomicAdd(&pos[1], 1) == total - 1) {
      pos[1] = 0;
      for (int i = 0; i < B; i++) {
        const int tv2 = pos[2 * i];
        if (tv2 >= 0 && tv2 < 2 * Lh) pos[2 * i] = tv2 + 1;
      }
      __threadfence();
    }
  }
}

// taps8[e][c][u] = taps[c][Lh-1-(u+e)] for u + e < Lh, else 0; row pitch Lh + 8.
__global__ void taps_rev8_kernel(const bf16* __restrict__ taps, bf16* __restrict__ taps8, int d, int Lh) {
  const int LP = Lh + 8;
  const size_t total = (size_t)8 * d * LP;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int u = (int)(idx % LP);
    const int c = (int)((idx / LP) % d);
    const int e = (int)(idx / ((size_t)LP * d));
    const int j = Lh - 1 - (u + e);
    taps8[idx] = (j >= 0) ? taps[(size_t)c * Lh + j] : __float2bfloat16_rn(0.f);
  }
}

extern "C" int stu_taps_rev8(const void* taps, void* taps8, int d, int Lh, int dtype, void* stream) {
  if (!taps || !taps8) return STU_ERR_NULL;
  if (d <= 0 || Lh <= 0 || Lh % 8) return STU_ERR_SHAPE;
  if (dtype != STU_BF16) return STU_ERR_DTYPE;
  taps_rev8_kernel<<<1024, 256, 0, (cudaStream_t)stream>>>((const bf16*)taps, (bf16*)taps8, d, Lh);
  STU_CHECK_LAUNCH();
  return STU_OK;
}

static int launch_rows8(const void* x, long long x_row_stride, const void* norm_w, const void* MinT, void* hist,
                        const void* taps8, int* pos, void* out, long long out_row_stride, int B, int d, int dch,
                        int add_resid, int Lh, float eps, int* status, int pdl, cudaStream_t st) {
  if (x_row_stride % 8 || !aligned16(x) || !aligned16(MinT) || !aligned16(hist) || !aligned16(norm_w) ||
      !aligned16(taps8))
    return STU_ERR_ALIGN;
  const size_t dsm = (size_t)8 * (Lh + 8) * sizeof(bf16);
  dim3 gd(dch / 8, (B + 7) / 8);
  const bool two_per_sm = (size_t)gd.x * gd.y > 160 && 2 * (dsm + 8 * 1024) <= (size_t)220 * 1024;
  cudaError_t ae = two_per_sm ? cudaFuncSetAttribute(stu_decode_rows8_kernel<16>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsm)
                              : cudaFuncSetAttribute(stu_decode_rows8_kernel<32>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsm);
  if (ae != cudaSuccess) return (int)ae;
  cudaError_t le =
      two_per_sm ? launch_maybe_overlapped(stu_decode_rows8_kernel<16>, gd, dim3(16 * 32), dsm, st,
                                           (pdl & STU_FLAG_OVERLAP) != 0, (const bf16*)x, x_row_stride,
                                           (const bf16*)norm_w, (const bf16*)MinT, (bf16*)hist, (const bf16*)taps8, pos,
                                           (bf16*)out, out_row_stride, B, d, dch, add_resid, Lh, eps, status, pdl)
                 : launch_maybe_overlapped(stu_decode_rows8_kernel<32>, gd, dim3(32 * 32), dsm, st,
                                           (pdl & STU_FLAG_OVERLAP) != 0, (const bf16*)x, x_row_stride,
                                           (const bf16*)norm_w, (const bf16*)MinT, (bf16*)hist, (const bf16*)taps8, pos,
                                           (bf16*)out, out_row_stride, B, d, dch, add_resid, Lh, eps, status, pdl);
  if (le != cudaSuccess) return (int)le;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// Channel shard of the fused decode step (tensor parallelism): x [B, d_in] is the full layer input, MinT
// [d_ch][d_in], hist [B][d_ch][2][Lh], taps8 [8][d_ch][Lh+8] and out [B, d_ch] belong to the d_ch channels of this
// rank; with add_residual = 0 out receives the STU output alone (the caller all-gathers the shards and adds them to
// the residual stream).  bf16, common position (checked on the device, status 6), d_ch % 8 == 0.
extern "C" int stu_decode_approx_shard(const void* x, long long x_row_stride, const void* norm_w, const void* MinT,
                                       void* hist, const void* taps8, int* pos, void* out, long long out_row_stride,
                                       int B, int d_in, int d_ch, int Lh, float eps, int add_residual, int* status,
                                       int dtype, void* stream) {
  if (!x || !norm_w || !MinT || !hist || !taps8 || !pos || !out) return STU_ERR_NULL;
  if (B <= 0 || d_in <= 0 || d_ch <= 0 || Lh <= 0 || d_in % 8 || d_ch % 8 || Lh % 8) return STU_ERR_SHAPE;
  if (add_residual && d_in != d_ch) return STU_ERR_SHAPE;
  const int pdl = dtype & (STU_FLAG_OVERLAP | STU_FLAG_EARLY_TRIGGER);
  dtype &= ~(STU_FLAG_OVERLAP | STU_FLAG_EARLY_TRIGGER | STU_FLAG_UNIFORM_POS);
  if (dtype != STU_BF16) return STU_ERR_DTYPE;
  if ((size_t)8 * (Lh + 8) * sizeof(bf16) > (size_t)180 * 1024) return STU_ERR_UNSUPPORTED;
  return launch_rows8(x, x_row_stride, norm_w, MinT, hist, taps8, pos, out, out_row_stride, B, d_in, d_ch,
                      add_residual, Lh, eps, status, pdl, (cudaStream_t)stream);
}

extern "C" int stu_decode_approx(const void* x, long long x_row_stride, const void* norm_w, const void* MinT,
                                 void* hist, const void* taps, const void* taps8, int* pos, void* out,
                                 long long out_row_stride, int B, int d, int Lh, float eps, int* status, int dtype,
                                 void* stream) {
  if (!x || !norm_w || !MinT || !hist || !taps || !pos || !out) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || Lh <= 0) return STU_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int pdl = dtype & (STU_FLAG_OVERLAP | STU_FLAG_EARLY_TRIGGER);  // honoured by the tensor-core kernels
  const bool uniform = (dtype & STU_FLAG_UNIFORM_POS) != 0;
  dtype &= ~(STU_FLAG_OVERLAP | STU_FLAG_EARLY_TRIGGER | STU_FLAG_UNIFORM_POS);
  if (taps8 && dtype == STU_BF16 && uniform && d % 8 == 0 && Lh % 8 == 0 &&
      (size_t)8 * (Lh + 8) * sizeof(bf16) <= (size_t)180 * 1024) {
    // common position promised by the caller: 8 channels x 8 sequences per CTA, both contractions as MMAs
    return launch_rows8(x, x_row_stride, norm_w, MinT, hist, taps8, pos, out, out_row_stride, B, d, d, 1, Lh, eps,
                        status, pdl, st);
  }
  if (taps8 && dtype == STU_BF16) {
    // tensor-core kernel: needs the reversed 8-alignment tap table
    if (d % 8 || Lh % 8 || x_row_stride % 8 || !aligned16(x) || !aligned16(MinT) || !aligned16(hist) ||
        !aligned16(norm_w) || !aligned16(taps8))
      return STU_ERR_ALIGN;
    dim3 gd(d, (B + 7) / 8);
    const size_t dsm = (size_t)(Lh + 8) * sizeof(bf16);
    if (dsm > 48 * 1024) {
      if (dsm > 200 * 1024) return STU_ERR_UNSUPPORTED;
      cudaError_t ae = cudaFuncSetAttribute(stu_decode_diag_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)dsm);
      if (ae != cudaSuccess) return (int)ae;
    }
    cudaError_t le = launch_maybe_overlapped(stu_decode_diag_kernel, gd, dim3(256), dsm, st,
                                             (pdl & STU_FLAG_OVERLAP) != 0, (const bf16*)x, x_row_stride,
                                             (const bf16*)norm_w, (const bf16*)MinT, (bf16*)hist,
                                             (const bf16*)taps8, pos, (bf16*)out, out_row_stride, B, d, Lh, eps,
                                             status, pdl);
    if (le != cudaSuccess) return (int)le;
    STU_CHECK_LAUNCH();
    return STU_OK;
  }
  dim3 grid(d, (B + 7) / 8);
  if (dtype == STU_F32) {
    if (d % 4 || Lh % 4 || x_row_stride % 4 || !aligned16(x) || !aligned16(MinT) || !aligned16(hist) ||
        !aligned16(norm_w))
      return STU_ERR_ALIGN;
    size_t smem = (size_t)(Lh + 4) * sizeof(float);
    if (smem > 200 * 1024) return STU_ERR_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(stu_decode_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    stu_decode_kernel<float><<<grid, 256, smem, st>>>((const float*)x, x_row_stride, (const float*)norm_w,
                                                      (const float*)MinT, (float*)hist, (const float*)taps, pos,
                                                      (float*)out, out_row_stride, B, d, Lh, eps, status);
  } else if (dtype == STU_BF16) {
    if (d % 8 || Lh % 8 || x_row_stride % 8 || !aligned16(x) || !aligned16(MinT) || !aligned16(hist) ||
        !aligned16(norm_w))
      return STU_ERR_ALIGN;
    size_t smem = (size_t)(Lh + 8) * sizeof(bf16);
    if (smem > 200 * 1024) return STU_ERR_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(stu_decode_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    stu_decode_kernel<bf16><<<grid, 256, smem, st>>>((const bf16*)x, x_row_stride, (const bf16*)norm_w,
                                                     (const bf16*)MinT, (bf16*)hist, (const bf16*)taps, pos,
                                                     (bf16*)out, out_row_stride, B, d, Lh, eps, status);
  } else {
    return STU_ERR_DTYPE;
  }
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// ------------------------------------------------------------------------------------------------
// Prefill convolution for callers that cannot allocate device memory.
//
// stu_conv_prefill_approx needs a scratch buffer (yT) that the caller normally allocates.  Some hosts
// cannot do that at the point where they call in: a serving process that handed the whole HBM to its
// own arena at start-up (so a later cudaMalloc fails), or a steady-state loop that runs under a
// "no allocation" rule because cudaMalloc/cudaFree synchronise the device and stall every stream.
// For them the scratch lives in the library image itself: a fixed 32 MiB array in device global
// memory that every GPU holding a context with this library loaded keeps until the process exits.
//
// Host code must not hand the array's name to a kernel: on the host the symbol is only a stand-in, and
// a kernel given it would fault or quietly use unrelated memory.  The device address is fetched with
// cudaGetSymbolAddress once per device, with that device current, and cached.
constexpr size_t STATIC_SCRATCH_BYTES = (size_t)32 << 20;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

#define STU_ERR_SCRATCH_TOO_SMALL (-7)

#include <mutex>
static std::mutex g_static_scratch_mutex;
static void* g_static_scratch_ptr[STU_MAX_DEVICES] = {nullptr};

// Same computation and arguments as stu_conv_prefill_approx, minus yT / y_Lh.
//   * Limit: B * d * 2 * roundup8(ceil(t_end / 2)) elements of the dtype must fit in 32 MiB
//     (e.g. bf16: B*d*t_end <= 16 Mi elements); larger calls return -7 before anything is launched.
//   * The first call on each device looks up the array's device address (no allocation, but a
//     runtime call that is not a kernel launch): make that first call outside any stream capture.
//   * All calls on a device share the one array.  Nothing in it has to start at zero (the convolution
//     writes every element the residual add reads), so it is never cleared and simply keeps the last
//     call's values; two calls that overlap in time on the same GPU (different streams) race on it.
//   * No cudaMalloc / cudaFree / allocating library routine is called on any path.
extern "C" int stu_conv_prefill_approx_static(const void* hist, const void* taps, void* x, long long x_bstride,
                                              long long x_tstride, int B, int d, int Lh, int t0, int t_end,
                                              int dtype, int use_tensor_cores, void* stream) {
  if (!hist || !taps || !x) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || Lh <= 0 || t0 < 0 || t_end <= t0 || t_end > 2 * Lh) return STU_ERR_SHAPE;
  if (dtype != STU_F32 && dtype != STU_BF16) return STU_ERR_DTYPE;
  const int y_Lh = (((t_end + 1) / 2) + 7) / 8 * 8;
  const size_t elem = dtype == STU_F32 ? 4 : 2;
  const size_t need = (size_t)B * (size_t)d * 2 * (size_t)y_Lh * elem;
  if (need > STATIC_SCRATCH_BYTES) return STU_ERR_SCRATCH_TOO_SMALL;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= STU_MAX_DEVICES) return STU_ERR_UNSUPPORTED;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_ptr[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess) return (int)e;
      g_static_scratch_ptr[dev] = p;
    }
    scratch = g_static_scratch_ptr[dev];
  }
  return stu_conv_prefill_approx(hist, taps, scratch, x, x_bstride, x_tstride, B, d, Lh, y_Lh, t0, t_end, dtype,
                                 use_tensor_cores, stream);
}
