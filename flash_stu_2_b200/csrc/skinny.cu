// Decode-time linear layers: M <= 64 activation rows against an [N,K] weight.  The step is bound by
// streaming the weight from HBM once, so the kernel is organised around 128-bit weight loads with
// the warps of a CTA splitting K for eight output features; the activation rows are L2-resident and are
// loaded straight into MMA fragments (optionally RMS-normalised on the way in).  bf16 uses mma.sync m16n8k16
// with fp32 accumulation (at 8..64 rows CUDA-core FMA throughput would cap the kernel below the HBM
// rate); fp32 models use fp32 FMAs.
#include <cooperative_groups.h>

#include "common.cuh"
#include "epilogue.cuh"

namespace cg = cooperative_groups;

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

// One CTA = eight output features; its NW warps split K in interleaved 32-element chunks.  Every lane
// loads 16 bytes of its weight row and 16 bytes of its activation row(s) per chunk straight from global
// memory (the activations are L2-resident) and feeds them to mma.sync with the k-order permuted so that
// no shuffle or shared-memory staging is needed.  All loads of a round (U chunks) are issued before any
// is used; with NORM the row statistics are computed while they are in flight.
//   MT   16-row activation tiles (M <= 16*MT);  LOW8: M <= 8, the upper half-tile is implicit zeros
//   KSPLIT > 1: the CTAs of a thread-block cluster (1 x KSPLIT x 1) split K between them; the partial tiles meet in
//   the shared memory of the cluster's first CTA (distributed shared memory), which runs the epilogue.  Used when N
//   alone gives too few CTAs to pull the weight through every SM (narrow outputs with long rows: down projections).
template <int EPI, int MT, bool LOW8, bool NORM, int U, int NW, int KSPLIT = 1>
__global__ void __launch_bounds__(NW * 32) skinny_bf16_kernel(const bf16* __restrict__ x, long long lda,
                                                              const bf16* __restrict__ W, long long ldb,
                                                              const bf16* __restrict__ W2, int M, int N, int K,
                                                              EpiArgs<bf16> ep, const bf16* __restrict__ nw,
                                                              float eps, int pdl) {
  constexpr bool DUAL = (EPI == EPI_GELU_MUL);
  constexpr int NACC = DUAL ? 2 : 1;
  constexpr int NH = LOW8 ? 1 : 2;  // activation half-tiles (rows g and g+8) per m-tile
  __shared__ float s_r[MT * 16];
  __shared__ float red[NACC * NW * MT * 4 * 32];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const int n0 = blockIdx.x * 8;
  const int n = n0 + g;
  const bool nvalid = n < N;
  const bf16* wrow = W + (size_t)(nvalid ? n : 0) * ldb;
  const bf16* wrow2 = DUAL ? (W2 + (size_t)(nvalid ? n : 0) * ldb) : nullptr;
  const int nchunks_all = (K + 31) >> 5;
  // this CTA's share of the K chunks
  const int per = (nchunks_all + KSPLIT - 1) / KSPLIT;
  const int c_begin = KSPLIT > 1 ? (int)blockIdx.y * per : 0;
  const int nchunks = KSPLIT > 1 ? min(nchunks_all, c_begin + per) : nchunks_all;

  uint4 wv[U], wv2[DUAL ? U : 1], xv[U][MT][NH], nwv[NORM ? U : 1];
  // constants of a round (weights, norm weights) and its activations are issued separately: in an overlapped
  // launch the constants are fetched while the kernel that produces the activations is still running
  auto issue_w = [&](int c0) {
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int ch = c0 + NW * u;
      const int k = (ch << 5) + q * 8;
      const bool kok = ch < nchunks && (k + 8) <= K;
      wv[u] = (kok && nvalid) ? ldg_stream(wrow + k) : make_uint4(0, 0, 0, 0);
      if (DUAL) wv2[u] = (kok && nvalid) ? ldg_stream(wrow2 + k) : make_uint4(0, 0, 0, 0);
      if (NORM) nwv[u] = kok ? *reinterpret_cast<const uint4*>(nw + k) : make_uint4(0, 0, 0, 0);
    }
  };
  auto issue_x = [&](int c0) {
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int ch = c0 + NW * u;
      const int k = (ch << 5) + q * 8;
      const bool kok = ch < nchunks && (k + 8) <= K;
#pragma unroll
      for (int t = 0; t < MT; t++)
#pragma unroll
        for (int h = 0; h < NH; h++) {
          const int m = t * 16 + h * 8 + g;
          xv[u][t][h] = (kok && m < M) ? *reinterpret_cast<const uint4*>(x + (size_t)m * lda + k)
                                       : make_uint4(0, 0, 0, 0);
        }
    }
  };
  if (pdl & STU_FLAG_EARLY_TRIGGER) pdl_trigger();
  issue_w(c_begin + warp);
  pdl_wait();
  if (!(pdl & STU_FLAG_EARLY_TRIGGER)) pdl_trigger();
  issue_x(c_begin + warp);

  if (NORM) {
    for (int m = warp; m < MT * 16; m += NW) {
      float r = 0.f;
      if (m < M) {
        const bf16* src = x + (size_t)m * lda;
        float ss = 0.f;
        for (int k = lane * 8; k < K; k += 256) {
          float v[8];
          load_vec(src + k, v);
#pragma unroll
          for (int j = 0; j < 8; j++) ss += v[j] * v[j];
        }
        ss = warp_sum(ss);
        r = rsqrtf(ss / (float)K + eps);
      }
      if (lane == 0) s_r[m] = r;
    }
    __syncthreads();
  }

  float acc[NACC][MT][4];
#pragma unroll
  for (int a = 0; a < NACC; a++)
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
      for (int i = 0; i < 4; i++) acc[a][t][i] = 0.f;

  for (int c0 = c_begin + warp; c0 < nchunks; c0 += NW * U) {
    if (c0 != c_begin + warp) {
      issue_w(c0);
      issue_x(c0);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int ch = c0 + NW * u;
      // ch is the same for the whole warp: mma.sync must be reached by all 32 lanes, so a lane whose k falls
      // past the end of a partial chunk takes part with zero operands (its loads above were predicated off)
      if (ch < nchunks) {
#pragma unroll
        for (int t = 0; t < MT; t++) {
          uint4 xa = xv[u][t][0];
          uint4 xb = LOW8 ? make_uint4(0, 0, 0, 0) : xv[u][t][NH - 1];
          if (NORM) {  // zero activations (k past the row end) stay zero
            xa = norm_pack(xa, s_r[t * 16 + g], nwv[u]);
            if (!LOW8) xb = norm_pack(xb, s_r[t * 16 + 8 + g], nwv[u]);
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
  }
  // cross-warp (split-K) reduction: red[a][warp][t][i][lane]
#pragma unroll
  for (int a = 0; a < NACC; a++)
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
      for (int i = 0; i < 4; i++) red[(((a * NW + warp) * MT + t) * 4 + i) * 32 + lane] = acc[a][t][i];
  __syncthreads();
  // element (row, col) of m-tile t lives in lane (row%8)*4 + col/2, register (row/8)*2 + col%2
  auto tile_sum = [&](int e, float& s, float& s2) {
    const int t = e >> 7, r = (e >> 3) & 15, cidx = e & 7;
    const int src_lane = (r & 7) * 4 + (cidx >> 1), reg = (r >> 3) * 2 + (cidx & 1);
    s = 0.f;
    s2 = 0.f;
#pragma unroll
    for (int w = 0; w < NW; w++) {
      s += red[(((0 * NW + w) * MT + t) * 4 + reg) * 32 + src_lane];
      if (DUAL) s2 += red[(((1 * NW + w) * MT + t) * 4 + reg) * 32 + src_lane];
    }
  };
  if constexpr (KSPLIT == 1) {
    for (int e = threadIdx.x; e < MT * 128; e += NW * 32) {
      float s, s2;
      tile_sum(e, s, s2);
      const int m = (e >> 7) * 16 + ((e >> 3) & 15), nn = n0 + (e & 7);
      if (m < M && nn < N) epilogue_store<bf16, EPI>(ep, m, nn, s, s2);
    }
  } else {
    static_assert(KSPLIT == 1 || !DUAL, "the cluster split is used for single-weight epilogues");
    __shared__ float part[MT * 128];
    cg::cluster_group cluster = cg::this_cluster();
    for (int e = threadIdx.x; e < MT * 128; e += NW * 32) {
      float s, s2;
      tile_sum(e, s, s2);
      part[e] = s;
    }
    cluster.sync();  // every CTA's partial tile is complete and visible cluster-wide
    if (cluster.block_rank() == 0) {
      for (int e = threadIdx.x; e < MT * 128; e += NW * 32) {
        float s = part[e];
#pragma unroll
        for (int rk = 1; rk < KSPLIT; rk++) s += *cluster.map_shared_rank(&part[e], rk);
        const int m = (e >> 7) * 16 + ((e >> 3) & 15), nn = n0 + (e & 7);
        if (m < M && nn < N) epilogue_store<bf16, EPI>(ep, m, nn, s, 0.f);
      }
    }
    cluster.sync();  // the other CTAs' shared memory stays alive until the first one has read it
  }
  if (EPI == EPI_STORE && ep.peer) {   // the rows went to the inboxes of the tensor-parallel ranks: signal them
    __syncthreads();
    if (threadIdx.x == 0) peer_signal_when_last(ep.peer, gridDim.x * gridDim.y);
  }
}

// fp32 models: SPLIT warps per output feature (8 / SPLIT features per CTA), lanes and warps split K with 128-bit
// loads, up to 8 rows per pass.  SPLIT > 1 keeps the grid large when N is small (a 512-wide down projection
// would otherwise be 64 CTAs streaming 12 MB of weights).
template <int EPI, int SPLIT>
__global__ void __launch_bounds__(256) skinny_f32_kernel(const float* __restrict__ x, long long lda,
                                                         const float* __restrict__ W, long long ldb,
                                                         const float* __restrict__ W2, int M, int N, int K,
                                                         EpiArgs<float> ep) {
  constexpr bool DUAL = (EPI == EPI_GELU_MUL);
  constexpr int FPC = 8 / SPLIT;
  __shared__ float red[DUAL ? 2 : 1][8][8];  // [acc][warp][row]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int feat = warp / SPLIT, part = warp % SPLIT;
  const int n = blockIdx.x * FPC + feat;
  const bool nok = n < N;
  const float* wr = W + (size_t)(nok ? n : 0) * ldb;
  const float* wr2 = DUAL ? W2 + (size_t)(nok ? n : 0) * ldb : nullptr;
  for (int m0 = 0; m0 < M; m0 += 8) {
    float acc[8] = {}, acc2[8] = {};
    if (nok) {
      for (int k = (part * 32 + lane) * 4; k < K; k += 128 * SPLIT) {
        const float4 w4 = *reinterpret_cast<const float4*>(wr + k);
        const float4 v4 = DUAL ? *reinterpret_cast<const float4*>(wr2 + k) : make_float4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          if (m0 + i < M) {
            const float4 a = *reinterpret_cast<const float4*>(x + (size_t)(m0 + i) * lda + k);
            acc[i] += a.x * w4.x + a.y * w4.y + a.z * w4.z + a.w * w4.w;
            if (DUAL) acc2[i] += a.x * v4.x + a.y * v4.y + a.z * v4.z + a.w * v4.w;
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
      acc[i] = warp_sum(acc[i]);
      if (DUAL) acc2[i] = warp_sum(acc2[i]);
    }
    if (SPLIT == 1) {
#pragma unroll
      for (int i = 0; i < 8; i++)
        if (lane == 0 && nok && m0 + i < M) epilogue_store<float, EPI>(ep, m0 + i, n, acc[i], acc2[i]);
    } else {
      __syncthreads();  // the previous pass has read red
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          red[0][warp][i] = acc[i];
          if (DUAL) red[DUAL ? 1 : 0][warp][i] = acc2[i];
        }
      }
      __syncthreads();
      if (part == 0 && lane < 8 && nok && m0 + lane < M) {
        float s = 0.f, s2 = 0.f;
#pragma unroll
        for (int pp = 0; pp < SPLIT; pp++) {
          s += red[0][feat * SPLIT + pp][lane];
          if (DUAL) s2 += red[DUAL ? 1 : 0][feat * SPLIT + pp][lane];
        }
        epilogue_store<float, EPI>(ep, m0 + lane, n, s, s2);
      }
    }
  }
}

template <int EPI>
static void launch_skinny_f32(const float* A, long long lda, const float* B, long long ldb, const float* B2, int M, int N,
                              int K, const EpiArgs<float>& e, cudaStream_t st) {
  // enough CTAs for about four per SM
  const int want = 592;
  if (N / 8 >= want || K < 1024) {
    skinny_f32_kernel<EPI, 1><<<(N + 7) / 8, 256, 0, st>>>(A, lda, B, ldb, B2, M, N, K, e);
  } else if (N / 4 >= want || K < 2048) {
    skinny_f32_kernel<EPI, 2><<<(N + 3) / 4, 256, 0, st>>>(A, lda, B, ldb, B2, M, N, K, e);
  } else if (N / 2 >= want || K < 4096) {
    skinny_f32_kernel<EPI, 4><<<(N + 1) / 2, 256, 0, st>>>(A, lda, B, ldb, B2, M, N, K, e);
  } else {
    skinny_f32_kernel<EPI, 8><<<N, 256, 0, st>>>(A, lda, B, ldb, B2, M, N, K, e);
  }
}

bool skinny_supported(const void* A, long long lda, const void* B, long long ldb, long long skb, const void* B2,
                      int M, int N, int K, int epi, int dtype) {
  if (M < 1 || M > 64 || skb != 1 || epi == EPI_HIST || epi == EPI_BLOCKCOL) return false;
  if (dtype == STU_BF16)
    return !(K % 8 || lda % 8 || ldb % 8 || !aligned16(A) || !aligned16(B) || (B2 && !aligned16(B2)));
  if (dtype == STU_F32)
    return !(K % 4 || lda % 4 || ldb % 4 || !aligned16(A) || !aligned16(B) || (B2 && !aligned16(B2)));
  return false;
}

// STU_B200_DISABLE_CLUSTER_SPLIT=1 keeps every decode linear on the single-CTA K loop.
static bool cluster_split_enabled() {
  static const bool off = getenv("STU_B200_DISABLE_CLUSTER_SPLIT") != nullptr;
  return !off;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_cluster_y(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, bool overlap,
                                           int cluster_y, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 1;
  at[0].val.clusterDim.y = cluster_y;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (overlap && pdl_enabled()) ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

template <int EPI, int MT, bool LOW8, int U, int NW, int KSPLIT = 1>
static int launch_skinny_cfg(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N,
                             int K, const EpiArgs<bf16>& ep, const void* nw, float eps, int pdl, cudaStream_t st) {
  dim3 grid((N + 7) / 8, KSPLIT);
  const bool ov = (pdl & STU_FLAG_OVERLAP) != 0;
  cudaError_t e;
  if constexpr (KSPLIT > 1) {
    e = launch_cluster_y(skinny_bf16_kernel<EPI, MT, LOW8, false, U, NW, KSPLIT>, grid, dim3(NW * 32), st, ov, KSPLIT,
                         (const bf16*)A, lda, (const bf16*)B, ldb, (const bf16*)B2, M, N, K, ep, (const bf16*)nullptr,
                         eps, pdl);
  } else if (nw)
    e = launch_maybe_overlapped(skinny_bf16_kernel<EPI, MT, LOW8, true, U, NW>, grid, dim3(NW * 32), 0, st, ov,
                                (const bf16*)A, lda, (const bf16*)B, ldb, (const bf16*)B2, M, N, K, ep,
                                (const bf16*)nw, eps, pdl);
  else
    e = launch_maybe_overlapped(skinny_bf16_kernel<EPI, MT, LOW8, false, U, NW>, grid, dim3(NW * 32), 0, st, ov,
                                (const bf16*)A, lda, (const bf16*)B, ldb, (const bf16*)B2, M, N, K, ep,
                                (const bf16*)nullptr, eps, pdl);
  if (e != cudaSuccess) return (int)e;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// Register budget: a round keeps U weight vectors (2U for gate/up) and U*MT*(1 or 2) activation vectors
// per lane.  Long K rows use 16 warps so that one or two rounds cover the row.
template <int EPI, int MT, bool LOW8>
static int launch_skinny_shape(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M,
                               int N, int K, const EpiArgs<bf16>& ep, const void* nw, float eps, int pdl, cudaStream_t st) {
  constexpr bool light = (EPI != EPI_GELU_MUL) && (MT == 1);  // few registers per chunk: deeper rounds fit
  const int chunks = (K + 31) / 32;
  const int per8 = (chunks + 7) / 8;
  if constexpr (EPI != EPI_GELU_MUL && MT <= 2) {
    // narrow output, long rows: too few CTAs for the machine unless K is split across a cluster
    if (!nw && cluster_split_enabled() && (N + 7) / 8 <= 96 && chunks >= 128) {  // measured: pays for N <= 768
      if (MT == 1 && chunks > 128)   // more than 32 chunks per CTA: deeper rounds (one m-tile leaves the registers)
        return launch_skinny_cfg<EPI, MT, LOW8, 8, 8, 4>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
      return launch_skinny_cfg<EPI, MT, LOW8, 4, 8, 4>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
    }
  }
  if constexpr (light) {
    if (per8 <= 4) return launch_skinny_cfg<EPI, MT, LOW8, 4, 8>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
    if (per8 <= 8) return launch_skinny_cfg<EPI, MT, LOW8, 8, 8>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
    return launch_skinny_cfg<EPI, MT, LOW8, 8, 16>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
  } else if constexpr (MT <= 2) {
    return launch_skinny_cfg<EPI, MT, LOW8, 4, 8>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
  } else {
    return launch_skinny_cfg<EPI, MT, LOW8, 2, 8>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
  }
}

template <int EPI>
static int launch_skinny_bf16_mt(int MT, const void* A, long long lda, const void* B, long long ldb, const void* B2,
                                 int M, int N, int K, const EpiArgs<bf16>& ep, const void* nw, float eps, int pdl,
                                 cudaStream_t st) {
  if (M <= 8) return launch_skinny_shape<EPI, 1, true>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
  switch (MT) {
    case 1: return launch_skinny_shape<EPI, 1, false>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
    case 2: return launch_skinny_shape<EPI, 2, false>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
    case 3: return launch_skinny_shape<EPI, 3, false>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
    case 4: return launch_skinny_shape<EPI, 4, false>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, pdl, st);
  }
  return STU_ERR_SHAPE;
}

bool skinny_stage_takes(int M, int N, int K, int epi, bool norm);
int skinny_stage_dispatch(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N,
                          int K, int epi, const EpiArgs<bf16>& ep, const void* nw, float eps, int pdl, cudaStream_t st);
bool skinny_umma_takes(int M, int N, int K, int epi, bool norm, bool peer);
int skinny_umma_dispatch(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N,
                         int K, int epi, const EpiArgs<bf16>& ep, int pdl, cudaStream_t st);
bool skinny_wide_takes(int M, int N, int K, int epi, bool norm);
int skinny_wide_dispatch(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K, int epi,
                         const EpiArgs<bf16>& ep, const void* nw, float eps, cudaStream_t st);

int skinny_dispatch(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N, int K,
                    int epi, const EpiArgsAny& ep, const void* norm_w, float eps, int dtype, int pdl, cudaStream_t st) {
  if (dtype == STU_BF16) {
    int MT = (M + 15) / 16;
    EpiArgs<bf16> e = ep.as<bf16>();
    if (skinny_umma_takes(M, N, K, epi, norm_w != nullptr, e.peer != nullptr))
      return skinny_umma_dispatch(A, lda, B, ldb, B2, M, N, K, epi, e, pdl, st);
    if (skinny_stage_takes(M, N, K, epi, norm_w != nullptr))
      return skinny_stage_dispatch(A, lda, B, ldb, B2, M, N, K, epi, e, norm_w, eps, pdl, st);
    if (!B2 && skinny_wide_takes(M, N, K, epi, norm_w != nullptr))
      return skinny_wide_dispatch(A, lda, B, ldb, M, N, K, epi, e, norm_w, eps, st);
    switch (epi) {
      case EPI_STORE: return launch_skinny_bf16_mt<EPI_STORE>(MT, A, lda, B, ldb, B2, M, N, K, e, norm_w, eps, pdl, st);
      case EPI_RESID: return launch_skinny_bf16_mt<EPI_RESID>(MT, A, lda, B, ldb, B2, M, N, K, e, norm_w, eps, pdl, st);
      case EPI_GELU_MUL:
        return launch_skinny_bf16_mt<EPI_GELU_MUL>(MT, A, lda, B, ldb, B2, M, N, K, e, norm_w, eps, pdl, st);
    }
    return STU_ERR_UNSUPPORTED;
  }
  if (dtype == STU_F32) {
    if (norm_w) return STU_ERR_UNSUPPORTED;
    EpiArgs<float> e = ep.as<float>();
    switch (epi) {
      case EPI_STORE:
        launch_skinny_f32<EPI_STORE>((const float*)A, lda, (const float*)B, ldb, nullptr, M, N, K, e, st);
        break;
      case EPI_RESID:
        launch_skinny_f32<EPI_RESID>((const float*)A, lda, (const float*)B, ldb, nullptr, M, N, K, e, st);
        break;
      case EPI_GELU_MUL:
        launch_skinny_f32<EPI_GELU_MUL>((const float*)A, lda, (const float*)B, ldb, (const float*)B2, M, N, K, e, st);
        break;
      default: return STU_ERR_UNSUPPORTED;
    }
    STU_CHECK_LAUNCH();
    return STU_OK;
  }
  return STU_ERR_DTYPE;
}
