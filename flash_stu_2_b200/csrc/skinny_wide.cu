// Decode-time linear layers for 17..64 activation rows (bf16): y = x[M,K] @ W[N,K]^T with the store / residual
// epilogues.  The 8-features-per-CTA kernel of skinny.cu re-reads all M activation rows in every CTA; at M = 32 that
// is four bytes of activations from L2 for every byte of weights from HBM, and the L2 traffic, not the weight stream,
// sets the time.  Here a CTA owns 32 output features (four n-tiles per warp, the activation fragments reused across
// them), so activations and weights weigh the same, and the K range is split over the CTAs of a thread-block cluster
// (partial tiles meet in the first CTA's shared memory) to keep enough CTAs in flight for the weight stream.
// Fragment scheme as in skinny.cu: every lane loads 16 bytes of its activation rows and of its weight rows per
// 32-element chunk straight from global memory and feeds them to mma.sync m16n8k16 with the k-order permuted
// identically on both operands.
#include <cooperative_groups.h>
#include <stdlib.h>

#include "common.cuh"
#include "epilogue.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int NT = 4;   // n-tiles (8 features each) per CTA
constexpr int NW = 8;   // warps, splitting K in interleaved chunks

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NORM: x is RMS-normalised with the weight nw on the way in (statistics over the whole row in every CTA, the
// normalised values rounded to bf16 as the reference's norm output is).
template <int EPI, int MT, int KSPLIT, bool NORM>
__global__ void __launch_bounds__(NW * 32) skinny_wide_kernel(const bf16* __restrict__ x, long long lda,
                                                              const bf16* __restrict__ W, long long ldb, int M, int N,
                                                              int K, EpiArgs<bf16> ep, const bf16* __restrict__ nw,
                                                              float eps) {
  constexpr int U = (MT <= 2) ? 2 : 1;   // chunks in flight per warp
  extern __shared__ float sm[];
  float* red = sm;                              // [NT][NW][MT][4][32]
  float* part = sm + NT * NW * MT * 128;        // [NT][MT][128], cluster partial (KSPLIT > 1)
  __shared__ float s_r[MT * 16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const int n0 = blockIdx.x * (8 * NT);
  const bf16* wrow[NT];
  bool nvalid[NT];
#pragma unroll
  for (int j = 0; j < NT; j++) {
    const int n = n0 + 8 * j + g;
    nvalid[j] = n < N;
    wrow[j] = W + (size_t)(nvalid[j] ? n : 0) * ldb;
  }
  const int nchunks_all = (K + 31) >> 5;
  const int per = (nchunks_all + KSPLIT - 1) / KSPLIT;
  const int c_begin = KSPLIT > 1 ? (int)blockIdx.y * per : 0;
  const int c_end = KSPLIT > 1 ? min(nchunks_all, c_begin + per) : nchunks_all;

  // The weights are nobody's output: the CTA asks for its whole slice (32 rows x its K range) towards L2 at once,
  // and, launched with the programmatic attribute, does so while the kernel before it is still running.  Everything
  // after the wait may read what that kernel wrote.
  {
    const int kb = c_begin << 5, ke = min(K, c_end << 5);
    const int lines = (ke - kb + 63) >> 6;   // 128-byte lines per weight row
    for (int i = threadIdx.x; i < 8 * NT * lines; i += NW * 32) {
      const int r = i / lines, l = i - r * lines;
      if (n0 + r < N) asm volatile("prefetch.global.L2 [%0];" ::"l"(W + (size_t)(n0 + r) * ldb + kb + l * 64));
    }
  }
  pdl_trigger();
  pdl_wait();

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

  float acc[NT][MT][4];
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
      for (int i = 0; i < 4; i++) acc[j][t][i] = 0.f;

  for (int c0 = c_begin + warp; c0 < c_end; c0 += NW * U) {
    uint4 wv[U][NT], xv[U][MT][2], nwv[NORM ? U : 1];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int ch = c0 + NW * u;
      const int k = (ch << 5) + q * 8;
      const bool kok = ch < c_end && (k + 8) <= K;
#pragma unroll
      for (int j = 0; j < NT; j++)
        wv[u][j] = (kok && nvalid[j]) ? ldg_stream(wrow[j] + k) : make_uint4(0, 0, 0, 0);
      if (NORM) nwv[u] = kok ? *reinterpret_cast<const uint4*>(nw + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int t = 0; t < MT; t++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int m = t * 16 + h * 8 + g;
          xv[u][t][h] = (kok && m < M) ? *reinterpret_cast<const uint4*>(x + (size_t)m * lda + k)
                                       : make_uint4(0, 0, 0, 0);
        }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      if (c0 + NW * u < c_end) {   // warp-uniform: mma.sync needs all 32 lanes
#pragma unroll
        for (int t = 0; t < MT; t++) {
          uint4 xa = xv[u][t][0], xb = xv[u][t][1];
          if (NORM) {   // zero activations (rows past M, k past the row end) stay zero
            xa = norm_pack(xa, s_r[t * 16 + g], nwv[u]);
            xb = norm_pack(xb, s_r[t * 16 + 8 + g], nwv[u]);
          }
#pragma unroll
          for (int j = 0; j < NT; j++) {
            mma_16816(acc[j][t], xa.x, xb.x, xa.y, xb.y, wv[u][j].x, wv[u][j].y);
            mma_16816(acc[j][t], xa.z, xb.z, xa.w, xb.w, wv[u][j].z, wv[u][j].w);
          }
        }
      }
    }
  }
  // ---- the warps' partial tiles meet in shared memory
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
      for (int i = 0; i < 4; i++) red[(((j * NW + warp) * MT + t) * 4 + i) * 32 + lane] = acc[j][t][i];
  __syncthreads();
  // element (row, col) of m-tile t, n-tile j lives in lane (row%8)*4 + col/2, register (row/8)*2 + col%2
  auto tile_sum = [&](int e) {
    const int j = e / (MT * 128), rem = e % (MT * 128);
    const int t = rem >> 7, r = (rem >> 3) & 15, cidx = rem & 7;
    const int src_lane = (r & 7) * 4 + (cidx >> 1), reg = (r >> 3) * 2 + (cidx & 1);
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < NW; w++) s += red[(((j * NW + w) * MT + t) * 4 + reg) * 32 + src_lane];
    return s;
  };
  auto store = [&](int e, float s) {
    const int j = e / (MT * 128), rem = e % (MT * 128);
    const int m = (rem >> 7) * 16 + ((rem >> 3) & 15), nn = n0 + 8 * j + (rem & 7);
    if (m < M && nn < N) epilogue_store<bf16, EPI>(ep, m, nn, s, 0.f);
  };
  if constexpr (KSPLIT == 1) {
    for (int e = threadIdx.x; e < NT * MT * 128; e += NW * 32) store(e, tile_sum(e));
  } else {
    cg::cluster_group cluster = cg::this_cluster();
    for (int e = threadIdx.x; e < NT * MT * 128; e += NW * 32) part[e] = tile_sum(e);
    cluster.sync();   // every CTA's partial tile is complete and visible cluster-wide
    if (cluster.block_rank() == 0) {
      for (int e = threadIdx.x; e < NT * MT * 128; e += NW * 32) {
        float s = part[e];
#pragma unroll
        for (int rk = 1; rk < KSPLIT; rk++) s += *cluster.map_shared_rank(&part[e], rk);
        store(e, s);
      }
    }
    cluster.sync();   // the other CTAs' shared memory stays alive until the first one has read it
  }
  if (EPI == EPI_STORE && ep.peer) {   // the rows went to the inboxes of the tensor-parallel ranks: signal them
    __syncthreads();
    if (threadIdx.x == 0) peer_signal_when_last(ep.peer, gridDim.x * gridDim.y);
  }
}

template <int EPI, int MT, int KSPLIT, bool NORM>
int launch_wide_n(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K,
                  const EpiArgs<bf16>& ep, const void* nw, float eps, cudaStream_t st) {
  const size_t smem = (size_t)(NT * NW * MT * 128 + (KSPLIT > 1 ? NT * MT * 128 : 0)) * sizeof(float);
  auto kern = skinny_wide_kernel<EPI, MT, KSPLIT, NORM>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((N + 8 * NT - 1) / (8 * NT), KSPLIT);
  cfg.blockDim = dim3(NW * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 1;
  at[0].val.clusterDim.y = KSPLIT;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  e = cudaLaunchKernelEx(&cfg, kern, (const bf16*)A, lda, (const bf16*)B, ldb, M, N, K, ep, (const bf16*)nw, eps);
  if (e != cudaSuccess) return (int)e;
  STU_CHECK_LAUNCH();
  return STU_OK;
}
template <int EPI, int MT, int KSPLIT>
int launch_wide(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K,
                const EpiArgs<bf16>& ep, const void* nw, float eps, cudaStream_t st) {
  if (nw) return launch_wide_n<EPI, MT, KSPLIT, true>(A, lda, B, ldb, M, N, K, ep, nw, eps, st);
  return launch_wide_n<EPI, MT, KSPLIT, false>(A, lda, B, ldb, M, N, K, ep, nw, eps, st);
}

template <int EPI, int MT>
int launch_wide_split(int ks, const void* A, long long lda, const void* B, long long ldb, int M, int N, int K,
                      const EpiArgs<bf16>& ep, const void* nw, float eps, cudaStream_t st) {
  switch (ks) {
    case 1: return launch_wide<EPI, MT, 1>(A, lda, B, ldb, M, N, K, ep, nw, eps, st);
    case 2: return launch_wide<EPI, MT, 2>(A, lda, B, ldb, M, N, K, ep, nw, eps, st);
    default: return launch_wide<EPI, MT, 4>(A, lda, B, ldb, M, N, K, ep, nw, eps, st);
  }
}

template <int EPI>
int launch_wide_mt(int ks, const void* A, long long lda, const void* B, long long ldb, int M, int N, int K,
                   const EpiArgs<bf16>& ep, const void* nw, float eps, cudaStream_t st) {
  switch ((M + 15) / 16) {
    case 1: return launch_wide_split<EPI, 1>(ks, A, lda, B, ldb, M, N, K, ep, nw, eps, st);
    case 2: return launch_wide_split<EPI, 2>(ks, A, lda, B, ldb, M, N, K, ep, nw, eps, st);
    case 3: return launch_wide_split<EPI, 3>(ks, A, lda, B, ldb, M, N, K, ep, nw, eps, st);
    case 4: return launch_wide_split<EPI, 4>(ks, A, lda, B, ldb, M, N, K, ep, nw, eps, st);
  }
  return STU_ERR_SHAPE;
}

}  // namespace

int device_sm_count();

// 17..64 rows, store / residual epilogue.  STU_B200_DISABLE_WIDE_SKINNY=1 keeps the 8-feature kernel.
bool skinny_wide_takes(int M, int N, int K, int epi, bool norm) {
  static const bool off = getenv("STU_B200_DISABLE_WIDE_SKINNY") != nullptr;
  // (asked only for shapes the tcgen05 kernel of gemm_tc.cu does not take: fused norm, peer stores, odd strides)
  (void)norm;
  return !off && M > 16 && M <= 64 && (epi == EPI_STORE || epi == EPI_RESID) && N >= 8 * NT && K >= 256;
}

int skinny_wide_dispatch(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K, int epi,
                         const EpiArgs<bf16>& ep, const void* nw, float eps, cudaStream_t st) {
  // split K over a cluster until there is about one CTA per SM, as long as every warp keeps at least one chunk
  const int ctas = (N + 8 * NT - 1) / (8 * NT), chunks = (K + 31) / 32, sms = device_sm_count();
  int ks = 1;
  while (ks < 4 && ctas * ks < sms && chunks / (2 * ks) >= NW) ks *= 2;
  if (epi == EPI_STORE) return launch_wide_mt<EPI_STORE>(ks, A, lda, B, ldb, M, N, K, ep, nw, eps, st);
  return launch_wide_mt<EPI_RESID>(ks, A, lda, B, ldb, M, N, K, ep, nw, eps, st);
}
