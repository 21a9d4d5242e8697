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
// x[b, t - t0, c] = round(x + yT[b][c][t&1][t>>1]) for t in [t0, t_end); 64 times x 32 channels per CTA.
template <typename T>
__global__ void __launch_bounds__(256) transpose_add_kernel(T* __restrict__ x, long long x_bstride,
                                                            long long x_tstride, const T* __restrict__ yT, int d,
                                                            int Lh, int t0, int t_end) {
  __shared__ float tile[32][65];
  const int b = blockIdx.z, c0 = blockIdx.y * 32, tb = (t0 & ~1) + blockIdx.x * 64;  // tb even
  // read: for channel row r, 32 elements of each parity
  for (int e = threadIdx.x; e < 32 * 64; e += 256) {
    int r = e >> 6, i = e & 63, p = i >> 5, s = (tb >> 1) + (i & 31);
    int c = c0 + r, t = 2 * s + p;
    float v = 0.f;
    if (c < d && t >= t0 && t < t_end) v = Elem<T>::to_f(yT[((size_t)((size_t)b * d + c) * 2 + p) * Lh + s]);
    tile[r][2 * (i & 31) + p] = v;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 64 * 32; e += 256) {
    int tt = e >> 5, r = e & 31;
    int t = tb + tt, c = c0 + r;
    if (c < d && t >= t0 && t < t_end) {
      T* px = x + (size_t)b * x_bstride + (size_t)(t - t0) * x_tstride + c;
      *px = Elem<T>::from_f(Elem<T>::to_f(*px) + tile[r][tt]);
    }
  }
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
  cudaStream_t st = (cudaStream_t)stream;
  if (use_tensor_cores) {
    if (dtype != STU_BF16) return STU_ERR_DTYPE;
    if (Lh % 8 || !aligned16(hist)) return STU_ERR_ALIGN;
    dim3 grid(d, (2 * B + 15) / 16);
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
  int tb = t0 & ~1;
  dim3 g2((t_end - tb + 63) / 64, (d + 31) / 32, B);
  if (dtype == STU_F32)
    transpose_add_kernel<float><<<g2, 256, 0, st>>>((float*)x, x_bstride, x_tstride, (const float*)yT, d, y_Lh, t0,
                                                    t_end);
  else
    transpose_add_kernel<bf16><<<g2, 256, 0, st>>>((bf16*)x, x_bstride, x_tstride, (const bf16*)yT, d, y_Lh, t0,
                                                   t_end);
  STU_CHECK_LAUNCH();
  return STU_OK;
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
  __shared__ int s_smax;
  const int c = blockIdx.x, b0 = blockIdx.y * 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = b0 + warp;
  const bool active = b < B;
  int t = active ? pos[2 * b] : 0;
  bool bad = active && (t < 0 || t >= 2 * Lh);
  if (bad) {
    if (lane == 0 && status) atomicExch(status, 2);
    t = 0;
  }
  const int p = t & 1, s = t >> 1;
  if (threadIdx.x == 0) s_smax = 0;
  __syncthreads();
  if (lane == 0 && active) atomicMax(&s_smax, s);
  __syncthreads();
  const int smax = s_smax;
  const int ntr = (smax + 1 + V - 1) / V * V;
  for (int i = threadIdx.x; i < ntr; i += 256)
    tr[i] = (i <= smax) ? taps[(size_t)c * Lh + (smax - i)] : Elem<T>::from_f(0.f);
  __syncthreads();

  if (active && !bad) {
    // --- RMSNorm statistic of row b, then the projection onto channel c
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
    const float xp = round_to<T>(dot);
    T* hrow = hist + ((size_t)((size_t)b * d + c) * 2 + p) * Lh;
    if (lane == 0) hrow[s] = Elem<T>::from_f(xp);
    // --- tap dot product over the stored history [0, s); the new element pairs with tap 0 = tr[smax]
    const int sh = smax - s;  // this row's offset into the reversed taps (0 when positions are uniform)
    float acc0 = 0.f, acc1 = 0.f;
    const int svec = (s / V) * V;
    if ((sh % V) == 0) {
      for (int i = lane * V; i < svec; i += 32 * V) {
        float hv[V], tv[V];
        load_vec(hrow + i, hv);
        load_vec(tr + sh + i, tv);
#pragma unroll
        for (int j = 0; j < V; j += 2) {
          acc0 = fmaf(hv[j], tv[j], acc0);
          acc1 = fmaf(hv[j + 1], tv[j + 1], acc1);
        }
      }
    } else {
      for (int i = lane; i < svec; i += 32) acc0 = fmaf(Elem<T>::to_f(hrow[i]), Elem<T>::to_f(tr[sh + i]), acc0);
    }
    for (int i = svec + lane; i < s; i += 32) acc1 = fmaf(Elem<T>::to_f(hrow[i]), Elem<T>::to_f(tr[sh + i]), acc1);
    float acc = warp_sum(acc0 + acc1);
    if (lane == 0) {
      acc = fmaf(xp, Elem<T>::to_f(tr[smax]), acc);
      float y = round_to<T>(2.f * acc);
      out[(size_t)b * out_rstride + c] = Elem<T>::from_f(Elem<T>::to_f(xr[c]) + y);
    }
  }
  // --- arrival counter: the last CTA advances the positions
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

extern "C" int stu_decode_approx(const void* x, long long x_row_stride, const void* norm_w, const void* MinT,
                                 void* hist, const void* taps, int* pos, void* out, long long out_row_stride,
                                 int B, int d, int Lh, float eps, int* status, int dtype, void* stream) {
  if (!x || !norm_w || !MinT || !hist || !taps || !pos || !out) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || Lh <= 0) return STU_ERR_SHAPE;
  if (B < 1) return STU_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
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
static void* g_static_scratch_ptr[64] = {nullptr};

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
  if (dev < 0 || dev >= 64) return STU_ERR_UNSUPPORTED;
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
