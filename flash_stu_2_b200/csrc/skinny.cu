// Decode-time linear layers: M <= 64 activation rows against an [N,K] weight.  The step is bound by
// streaming the weight from HBM once, so the kernel is organised around 128-bit weight loads with
// all eight warps of a CTA splitting K for eight output features; the handful of activation rows
// sit in shared memory (optionally RMS-normalised on the way in).  bf16 uses mma.sync m16n8k16
// with fp32 accumulation (at 8..64 rows CUDA-core FMA throughput would cap the kernel below the HBM
// rate); fp32 models use fp32 FMAs.
#include "common.cuh"
#include "epilogue.cuh"

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int SK_PAD = 32;  // activation row padding (elements) that spreads rows over distinct banks

// Stage x[M,K] (bf16) into shared memory rows of K+SK_PAD elements; rows M..MT*16-1 are zero.
// With NORM each row is replaced by rmsnorm(x)*w rounded to bf16 (the tensor the reference feeds
// its nn.Linear).
template <bool NORM>
__device__ void stage_rows_bf16(bf16* xs, const bf16* __restrict__ x, long long lda, int M, int MT, int K,
                                const bf16* __restrict__ nw, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int ld = K + SK_PAD;
  for (int m = warp; m < MT * 16; m += nwarps) {
    bf16* dst = xs + (size_t)m * ld;
    if (m >= M) {
      for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
      continue;
    }
    const bf16* src = x + (size_t)m * lda;
    if (!NORM) {
      for (int k = lane * 8; k < K; k += 256)
        *reinterpret_cast<uint4*>(dst + k) = *reinterpret_cast<const uint4*>(src + k);
    } else {
      float ss = 0.f;
      for (int k = lane * 8; k < K; k += 256) {
        float v[8];
        load_vec(src + k, v);
#pragma unroll
        for (int j = 0; j < 8; j++) ss += v[j] * v[j];
      }
      ss = warp_sum(ss);
      float r = rsqrtf(ss / (float)K + eps);
      for (int k = lane * 8; k < K; k += 256) {
        float v[8], g[8];
        load_vec(src + k, v);
        load_vec(nw + k, g);
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = v[j] * r * g[j];
        store_vec(dst + k, v);
      }
    }
  }
}

template <int EPI, int MT, bool NORM>
__global__ void __launch_bounds__(256) skinny_bf16_kernel(const bf16* __restrict__ x, long long lda,
                                                          const bf16* __restrict__ W, long long ldb,
                                                          const bf16* __restrict__ W2, int M, int N, int K,
                                                          EpiArgs<bf16> ep, const bf16* __restrict__ nw, float eps) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  const int ld = K + SK_PAD;
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)MT * 16 * ld * sizeof(bf16));
  constexpr bool DUAL = (EPI == EPI_GELU_MUL);
  constexpr int NACC = DUAL ? 2 : 1;

  stage_rows_bf16<NORM>(xs, x, lda, M, MT, K, nw, eps);
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const int n0 = blockIdx.x * 8;
  const int n = n0 + g;
  const bool nvalid = n < N;
  const bf16* wrow = W + (size_t)(nvalid ? n : 0) * ldb;
  const bf16* wrow2 = DUAL ? (W2 + (size_t)(nvalid ? n : 0) * ldb) : nullptr;

  float acc[NACC][MT][4];
#pragma unroll
  for (int a = 0; a < NACC; a++)
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
      for (int i = 0; i < 4; i++) acc[a][t][i] = 0.f;

  const int nchunks = (K + 31) >> 5;
  constexpr int U = 4;
  for (int c0 = warp; c0 < nchunks; c0 += 8 * U) {
    uint4 wv[U], wv2[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      int k = ((c0 + 8 * u) << 5) + q * 8;
      bool ok = nvalid && (c0 + 8 * u) < nchunks && (k + 8) <= K;
      wv[u] = ok ? ldg_stream(wrow + k) : make_uint4(0, 0, 0, 0);
      if (DUAL) wv2[u] = ok ? ldg_stream(wrow2 + k) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      int k = ((c0 + 8 * u) << 5) + q * 8;
      if ((c0 + 8 * u) >= nchunks) break;
      bool kok = (k + 8) <= K;
#pragma unroll
      for (int t = 0; t < MT; t++) {
        uint4 xa = make_uint4(0, 0, 0, 0), xb = make_uint4(0, 0, 0, 0);
        if (kok) {
          xa = *reinterpret_cast<const uint4*>(xs + (size_t)(t * 16 + g) * ld + k);
          xb = *reinterpret_cast<const uint4*>(xs + (size_t)(t * 16 + g + 8) * ld + k);
        }
        mma_bf16_16816(acc[0][t], xa.x, xb.x, xa.y, xb.y, wv[u].x, wv[u].y);
        mma_bf16_16816(acc[0][t], xa.z, xb.z, xa.w, xb.w, wv[u].z, wv[u].w);
        if (DUAL) {
          mma_bf16_16816(acc[1][t], xa.x, xb.x, xa.y, xb.y, wv2[u].x, wv2[u].y);
          mma_bf16_16816(acc[1][t], xa.z, xb.z, xa.w, xb.w, wv2[u].z, wv2[u].w);
        }
      }
    }
  }
  // cross-warp (split-K) reduction: red[a][warp][t][i][lane]
#pragma unroll
  for (int a = 0; a < NACC; a++)
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
      for (int i = 0; i < 4; i++) red[(((a * 8 + warp) * MT + t) * 4 + i) * 32 + lane] = acc[a][t][i];
  __syncthreads();
  // element (row, col) of m-tile t lives in lane (row%8)*4 + col/2, register (row/8)*2 + col%2
  for (int e = threadIdx.x; e < MT * 128; e += 256) {
    int t = e >> 7, r = (e >> 3) & 15, cidx = e & 7;
    int src_lane = (r & 7) * 4 + (cidx >> 1), reg = (r >> 3) * 2 + (cidx & 1);
    float s = 0.f, s2 = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) {
      s += red[(((0 * 8 + w) * MT + t) * 4 + reg) * 32 + src_lane];
      if (DUAL) s2 += red[(((1 * 8 + w) * MT + t) * 4 + reg) * 32 + src_lane];
    }
    int m = t * 16 + r, nn = n0 + cidx;
    if (m < M && nn < N) epilogue_store<bf16, EPI>(ep, m, nn, s, s2);
  }
}

// fp32 models: one warp per output feature, lanes split K with 128-bit loads, up to 8 rows per pass.
template <int EPI>
__global__ void __launch_bounds__(256) skinny_f32_kernel(const float* __restrict__ x, long long lda,
                                                         const float* __restrict__ W, long long ldb,
                                                         const float* __restrict__ W2, int M, int N, int K,
                                                         EpiArgs<float> ep) {
  constexpr bool DUAL = (EPI == EPI_GELU_MUL);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const float* wr = W + (size_t)n * ldb;
  const float* wr2 = DUAL ? W2 + (size_t)n * ldb : nullptr;
  for (int m0 = 0; m0 < M; m0 += 8) {
    float acc[8] = {}, acc2[8] = {};
    for (int k = lane * 4; k < K; k += 128) {
      float4 w4 = *reinterpret_cast<const float4*>(wr + k);
      float4 v4 = DUAL ? *reinterpret_cast<const float4*>(wr2 + k) : make_float4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        if (m0 + i < M) {
          float4 a = *reinterpret_cast<const float4*>(x + (size_t)(m0 + i) * lda + k);
          acc[i] += a.x * w4.x + a.y * w4.y + a.z * w4.z + a.w * w4.w;
          if (DUAL) acc2[i] += a.x * v4.x + a.y * v4.y + a.z * v4.z + a.w * v4.w;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
      float s = warp_sum(acc[i]);
      float s2 = DUAL ? warp_sum(acc2[i]) : 0.f;
      if (lane == 0 && m0 + i < M) epilogue_store<float, EPI>(ep, m0 + i, n, s, s2);
    }
  }
}

static size_t skinny_smem_bytes(int MT, int K, bool dual) {
  return (size_t)MT * 16 * (K + SK_PAD) * sizeof(bf16) + (size_t)(dual ? 2 : 1) * 8 * MT * 4 * 32 * sizeof(float);
}

bool skinny_supported(const void* A, long long lda, const void* B, long long ldb, long long skb, const void* B2,
                      int M, int N, int K, int epi, int dtype) {
  if (M < 1 || M > 64 || skb != 1 || epi == EPI_HIST) return false;
  if (dtype == STU_BF16) {
    if (K % 8 || lda % 8 || ldb % 8 || !aligned16(A) || !aligned16(B) || (B2 && !aligned16(B2))) return false;
    int MT = (M + 15) / 16;
    return skinny_smem_bytes(MT, K, epi == EPI_GELU_MUL) <= 200 * 1024;
  }
  if (dtype == STU_F32)
    return !(K % 4 || lda % 4 || ldb % 4 || !aligned16(A) || !aligned16(B) || (B2 && !aligned16(B2)));
  return false;
}

template <int EPI, int MT>
static int launch_skinny_bf16(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M,
                              int N, int K, const EpiArgs<bf16>& ep, const void* nw, float eps, cudaStream_t st) {
  size_t smem = skinny_smem_bytes(MT, K, EPI == EPI_GELU_MUL);
  dim3 grid((N + 7) / 8);
  cudaError_t e;
  if (nw) {
    auto k = skinny_bf16_kernel<EPI, MT, true>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    k<<<grid, 256, smem, st>>>((const bf16*)A, lda, (const bf16*)B, ldb, (const bf16*)B2, M, N, K, ep,
                               (const bf16*)nw, eps);
  } else {
    auto k = skinny_bf16_kernel<EPI, MT, false>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    k<<<grid, 256, smem, st>>>((const bf16*)A, lda, (const bf16*)B, ldb, (const bf16*)B2, M, N, K, ep, nullptr,
                               eps);
  }
  STU_CHECK_LAUNCH();
  return STU_OK;
}

template <int EPI>
static int launch_skinny_bf16_mt(int MT, const void* A, long long lda, const void* B, long long ldb, const void* B2,
                                 int M, int N, int K, const EpiArgs<bf16>& ep, const void* nw, float eps,
                                 cudaStream_t st) {
  switch (MT) {
    case 1: return launch_skinny_bf16<EPI, 1>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, st);
    case 2: return launch_skinny_bf16<EPI, 2>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, st);
    case 3: return launch_skinny_bf16<EPI, 3>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, st);
    case 4: return launch_skinny_bf16<EPI, 4>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, st);
  }
  return STU_ERR_SHAPE;
}

int skinny_dispatch(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N, int K,
                    int epi, const EpiArgsAny& ep, const void* norm_w, float eps, int dtype, cudaStream_t st) {
  if (dtype == STU_BF16) {
    int MT = (M + 15) / 16;
    EpiArgs<bf16> e = ep.as<bf16>();
    switch (epi) {
      case EPI_STORE: return launch_skinny_bf16_mt<EPI_STORE>(MT, A, lda, B, ldb, B2, M, N, K, e, norm_w, eps, st);
      case EPI_RESID: return launch_skinny_bf16_mt<EPI_RESID>(MT, A, lda, B, ldb, B2, M, N, K, e, norm_w, eps, st);
      case EPI_GELU_MUL:
        return launch_skinny_bf16_mt<EPI_GELU_MUL>(MT, A, lda, B, ldb, B2, M, N, K, e, norm_w, eps, st);
    }
    return STU_ERR_UNSUPPORTED;
  }
  if (dtype == STU_F32) {
    if (norm_w) return STU_ERR_UNSUPPORTED;
    EpiArgs<float> e = ep.as<float>();
    dim3 grid((N + 7) / 8);
    switch (epi) {
      case EPI_STORE:
        skinny_f32_kernel<EPI_STORE><<<grid, 256, 0, st>>>((const float*)A, lda, (const float*)B, ldb, nullptr, M, N,
                                                           K, e);
        break;
      case EPI_RESID:
        skinny_f32_kernel<EPI_RESID><<<grid, 256, 0, st>>>((const float*)A, lda, (const float*)B, ldb, nullptr, M, N,
                                                           K, e);
        break;
      case EPI_GELU_MUL:
        skinny_f32_kernel<EPI_GELU_MUL><<<grid, 256, 0, st>>>((const float*)A, lda, (const float*)B, ldb,
                                                              (const float*)B2, M, N, K, e);
        break;
      default: return STU_ERR_UNSUPPORTED;
    }
    STU_CHECK_LAUNCH();
    return STU_OK;
  }
  return STU_ERR_DTYPE;
}
