// Decode-time linear layers for 17..32 activation rows (bf16), all three epilogues (store, residual, GELU(gate)*up).
//
// The kernels of skinny.cu / skinny_wide.cu fetch activations and weights into registers a few chunks at a time, so
// a CTA pays one memory round trip per round of chunks; at these sizes (a few MB of weights per launch) the launches
// are 2-3 dependent round trips long and never reach the weight stream's rate.  Here every load of a CTA is in
// flight at once: the activation rows of the CTA's K range come into shared memory by one bulk copy per row
// (cp.async.bulk, mbarrier), and the 16 warps issue the register loads of ALL their weight chunks before the first is
// used.  A CTA owns 32 weight rows (32 output features, or 16 gate + 16 up rows); the K range is split over a
// thread-block cluster (at most 48 chunks of 32 per CTA), the partial tiles meet in the first CTA's shared memory.
// MMA fragments as in skinny.cu (k-order permuted identically on both operands); the activation rows sit at a pitch
// of K_c + 32 elements, which puts the eight lanes of a quarter warp (two rows x four 16-byte chunks) on distinct banks.
#include <cooperative_groups.h>
#include <stdlib.h>

#include "common.cuh"
#include "epilogue.cuh"
#include "tma.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int NT = 4;        // n-tiles of 8 weight rows per CTA
constexpr int NW = 16;       // warps: chunk c of the CTA goes to warp c % 16
constexpr int MAXC = 48;     // chunks (of 32 k) per CTA: three per warp, all loaded at once
constexpr int U = MAXC / NW;

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 lds128(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(tma::smem_u32(p)));
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

// nw != NULL (KSPLIT == 1 only: the CTA holds whole rows): the staged rows are RMS-normalised in shared memory
// before the MMAs, x * rsqrt(mean(x^2) + eps) * nw rounded to bf16 as the reference's norm output is.
template <int EPI, int MT, int KSPLIT>
__global__ void __launch_bounds__(NW * 32, 1) skinny_stage_kernel(const bf16* __restrict__ x, long long lda,
                                                                  const bf16* __restrict__ W, long long ldb,
                                                                  const bf16* __restrict__ W2, int M, int N, int K,
                                                                  EpiArgs<bf16> ep, const bf16* __restrict__ nw,
                                                                  float eps, int early_weights) {
  constexpr bool DUAL = (EPI == EPI_GELU_MUL);
  constexpr int NF = DUAL ? 16 : 32;   // output features per CTA
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ uint64_t s_bar;
  __shared__ int s_abort;
  __shared__ float part[NT * MT * 128];   // cluster partial (KSPLIT > 1)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const int n0 = blockIdx.x * NF;
  const int nchunks_all = K >> 5;   // K % 32 == 0
  const int per = (nchunks_all + KSPLIT - 1) / KSPLIT;
  const int c_begin = (int)blockIdx.y * per;
  const int c_end = min(nchunks_all, c_begin + per);
  const int nch = max(0, c_end - c_begin);
  const int pitch = per * 32 + 32;   // elements
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);

  // ---- weights first: every chunk of this warp at once.  early_weights is the caller's promise that the kernel
  // before this one in the stream does not write them; the loads then go out while that kernel is still running
  // (programmatic launch), otherwise they wait for it like everything else.
  const bf16* wrow[NT];
  bool nvalid[NT];
#pragma unroll
  for (int j = 0; j < NT; j++) {
    const int n = DUAL ? n0 + 8 * (j & 1) + g : n0 + 8 * j + g;
    nvalid[j] = n < N;
    wrow[j] = ((DUAL && j >= 2) ? W2 : W) + (size_t)(nvalid[j] ? n : 0) * ldb;
  }
  pdl_trigger();
  if (!early_weights) pdl_wait();
  uint4 wv[U][NT];
#pragma unroll
  for (int u = 0; u < U; u++) {
    const int ch = c_begin + warp + NW * u;
#pragma unroll
    for (int j = 0; j < NT; j++)
      wv[u][j] = (ch < c_end && nvalid[j]) ? ldg_stream(wrow[j] + (ch << 5) + q * 8) : make_uint4(0, 0, 0, 0);
  }
  // ---- activations: one bulk copy per row, rows past M zero-filled by the threads.  With the programmatic launch
  // attribute everything above ran while the preceding kernel was still draining.
  if (threadIdx.x == 0) {
    tma::mbar_init(&s_bar, 1);
    s_abort = 0;
    tma::fence_barrier_init();
  }
  for (int i = threadIdx.x; i < (MT * 16 - M) * (nch * 4); i += NW * 32) {   // 16-byte vectors of the rows M..
    const int r = M + i / (nch * 4), v = i % (nch * 4);
    *reinterpret_cast<uint4*>(xs + (size_t)r * pitch + v * 8) = make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  if (early_weights) pdl_wait();   // the activations are the output of the kernel before this one
  if (threadIdx.x == 0 && nch > 0) {
    tma::mbar_expect_tx(&s_bar, (uint32_t)M * nch * 64);
    for (int m = 0; m < M; m++)
      tma::bulk_load(xs + (size_t)m * pitch, x + (size_t)m * lda + c_begin * 32, nch * 64, &s_bar);
  }
  float acc[NT][MT][4];
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
      for (int i = 0; i < 4; i++) acc[j][t][i] = 0.f;

  bool ok = true;
  if (nch > 0) ok = tma::mbar_wait_bounded(&s_bar, 0, &s_abort);
  ok = __all_sync(0xffffffffu, ok);
  if (KSPLIT == 1 && nw) {
    // fused RMSNorm: warp w normalises rows w, w + 16, ... in place (a row is 16-byte vectors of 8 values)
    const int nvec = K >> 3;
    for (int m = warp; m < M; m += NW) {
      bf16* xr = xs + (size_t)m * pitch;
      float ss = 0.f;
      for (int v = lane; v < nvec; v += 32) {
        float f[8];
        load_vec(xr + v * 8, f);
#pragma unroll
        for (int j = 0; j < 8; j++) ss += f[j] * f[j];
      }
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)K + eps);
      for (int v = lane; v < nvec; v += 32) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr + v * 8);
        *reinterpret_cast<uint4*>(xr + v * 8) = norm_pack(raw, r, *reinterpret_cast<const uint4*>(nw + v * 8));
      }
    }
    __syncthreads();
  }
  if (ok) {
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int cl = warp + NW * u;   // chunk inside the CTA's range
      if (cl < nch) {                 // warp-uniform
#pragma unroll
        for (int t = 0; t < MT; t++) {
          const uint4 xa = lds128(xs + (size_t)(t * 16 + g) * pitch + cl * 32 + q * 8);
          const uint4 xb = lds128(xs + (size_t)(t * 16 + 8 + g) * pitch + cl * 32 + q * 8);
#pragma unroll
          for (int j = 0; j < NT; j++) {
            mma_16816(acc[j][t], xa.x, xb.x, xa.y, xb.y, wv[u][j].x, wv[u][j].y);
            mma_16816(acc[j][t], xa.z, xb.z, xa.w, xb.w, wv[u][j].z, wv[u][j].w);
          }
        }
      }
    }
  }
  // ---- the warps' partial tiles meet in shared memory (the activation rows are no longer needed)
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem_raw);   // [NT][NW][MT][4][32]
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
  // outputs: single weight: n-tile j = features n0 + 8j..; gate/up: tiles 0,1 gate and 2,3 up of features n0 + 8(j&1)..
  constexpr int OUT_T = DUAL ? 2 : NT;
  auto finish = [&](auto get) {
    for (int e = threadIdx.x; e < OUT_T * MT * 128; e += NW * 32) {
      const int j = e / (MT * 128), rem = e % (MT * 128);
      const int m = (rem >> 7) * 16 + ((rem >> 3) & 15), nn = n0 + 8 * j + (rem & 7);
      if (m < M && nn < N) epilogue_store<bf16, EPI>(ep, m, nn, get(e), DUAL ? get(e + 2 * MT * 128) : 0.f);
    }
  };
  if constexpr (KSPLIT == 1) {
    finish([&](int e) { return tile_sum(e); });
  } else {
    cg::cluster_group cluster = cg::this_cluster();
    for (int e = threadIdx.x; e < NT * MT * 128; e += NW * 32) part[e] = tile_sum(e);
    cluster.sync();   // every CTA's partial tile is complete and visible cluster-wide
    if (cluster.block_rank() == 0) {
      finish([&](int e) {
        float s = part[e];
#pragma unroll
        for (int rk = 1; rk < KSPLIT; rk++) s += *cluster.map_shared_rank(&part[e], rk);
        return s;
      });
    }
    cluster.sync();   // the other CTAs' shared memory stays alive until the first one has read it
  }
  if (EPI == EPI_STORE && ep.peer) {   // the rows went to the inboxes of the tensor-parallel ranks: signal them
    __syncthreads();
    if (threadIdx.x == 0) peer_signal_when_last(ep.peer, gridDim.x * gridDim.y);
  }
}

template <int EPI, int MT, int KSPLIT>
int launch_stage(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N, int K,
                 const EpiArgs<bf16>& ep, const void* nw, float eps, int early, cudaStream_t st) {
  constexpr int NF = (EPI == EPI_GELU_MUL) ? 16 : 32;
  const int per = ((K >> 5) + KSPLIT - 1) / KSPLIT;
  const size_t xs_bytes = (size_t)MT * 16 * (per * 32 + 32) * sizeof(bf16);
  const size_t red_bytes = (size_t)NT * NW * MT * 128 * sizeof(float);
  const size_t smem = xs_bytes > red_bytes ? xs_bytes : red_bytes;
  auto kern = skinny_stage_kernel<EPI, MT, KSPLIT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((N + NF - 1) / NF, KSPLIT);
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
  e = cudaLaunchKernelEx(&cfg, kern, (const bf16*)A, lda, (const bf16*)B, ldb, (const bf16*)B2, M, N, K, ep,
                         (const bf16*)nw, eps, early);
  if (e != cudaSuccess) return (int)e;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

template <int EPI, int MT>
int launch_stage_split(int ks, const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N,
                       int K, const EpiArgs<bf16>& ep, const void* nw, float eps, int early, cudaStream_t st) {
  switch (ks) {
    case 1: return launch_stage<EPI, MT, 1>(A, lda, B, ldb, B2, M, N, K, ep, nw, eps, early, st);
    case 2: return launch_stage<EPI, MT, 2>(A, lda, B, ldb, B2, M, N, K, ep, nullptr, eps, early, st);
    case 4: return launch_stage<EPI, MT, 4>(A, lda, B, ldb, B2, M, N, K, ep, nullptr, eps, early, st);
    case 8: return launch_stage<EPI, MT, 8>(A, lda, B, ldb, B2, M, N, K, ep, nullptr, eps, early, st);
  }
  return STU_ERR_UNSUPPORTED;
}

}  // namespace

// 17..32 rows, K a multiple of 32 and at most 8 x 48 chunks, no fused norm.  Measured on a B200 at 32 rows (weights
// from HBM): gate/up 6144 x 1536: 16.3 us (tcgen05 GEMM 17.8, 8-feature kernel 25.5); store / residual shapes are
// NOT faster than the 32-feature register-streaming kernel (down 6144 -> 1536: 14.6 against 11.4 us: one CTA per SM
// and two waves cost what its three load rounds cost), so only the gate/up epilogue is routed here unless
// STU_B200_STAGE_SKINNY=all.  STU_B200_DISABLE_STAGE_SKINNY=1 switches the kernel off.
bool skinny_stage_takes(int M, int N, int K, int epi, bool norm) {
  static const bool off = getenv("STU_B200_DISABLE_STAGE_SKINNY") != nullptr;
  static const bool all = getenv("STU_B200_STAGE_SKINNY") != nullptr;
  const bool epi_ok = epi == EPI_GELU_MUL || (all && (epi == EPI_STORE || epi == EPI_RESID));
  // a fused norm needs whole rows in one CTA: K within 48 chunks (no split over a cluster)
  if (norm && (K >> 5) > MAXC) return false;
  return !off && M > 16 && M <= 32 && K % 32 == 0 && K >= 256 && (K >> 5) <= 8 * MAXC && N >= 32 && epi_ok;
}

int skinny_stage_dispatch(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N,
                          int K, int epi, const EpiArgs<bf16>& ep, const void* nw, float eps, int pdl,
                          cudaStream_t st) {
  const int early = (pdl & STU_FLAG_OVERLAP) ? 1 : 0;
  int ks = 1;
  while (ks < 8 && ((K >> 5) + ks - 1) / ks > MAXC) ks *= 2;
  // short K: split further while that still leaves every warp a chunk and the grid is below one CTA per SM
  const int ctas = (N + (epi == EPI_GELU_MUL ? 16 : 32) - 1) / (epi == EPI_GELU_MUL ? 16 : 32);
  while (!nw && ks < 8 && ctas * ks < 148 && (K >> 5) / (2 * ks) >= NW) ks *= 2;
  switch (epi) {
    case EPI_STORE: return launch_stage_split<EPI_STORE, 2>(ks, A, lda, B, ldb, B2, M, N, K, ep, nw, eps, early, st);
    case EPI_RESID: return launch_stage_split<EPI_RESID, 2>(ks, A, lda, B, ldb, B2, M, N, K, ep, nw, eps, early, st);
    case EPI_GELU_MUL: return launch_stage_split<EPI_GELU_MUL, 2>(ks, A, lda, B, ldb, B2, M, N, K, ep, nw, eps, early, st);
  }
  return STU_ERR_UNSUPPORTED;
}
