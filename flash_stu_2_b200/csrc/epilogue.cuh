// GEMM epilogues shared by the CUDA-core, mma.sync and tcgen05 linear kernels.  Each one reproduces
// the rounding points of the reference's tensor-by-tensor evaluation in the model dtype.
#pragma once
#include "common.cuh"
#include "peer.cuh"

enum {
  EPI_STORE = 0,     // y = acc
  EPI_RESID = 1,     // y = resid + round(acc)            x.add_(h), flash_stu/layers/stu_layer.py:93,96
  EPI_GELU_MUL = 2,  // y = round(gelu_tanh(round(acc))) * round(acc2)   flash_stu/modules/swiglu.py:22-28
  EPI_HIST = 3,      // scatter acc into the parity-split channel-major history [B][N][2][Lh]
  EPI_BLOCKCOL = 5,  // y[m*ldy + (n / Tseq) * ld2 + (n % Tseq)] = acc: columns come in blocks of Tseq, every block ld2
                     // elements after the last (the distilled-LDS features: rows (tau, f), columns (chunk, channel),
                     // written straight into the [tokens, F*d] operand of the contraction with M)
};
// OR-ed into the epilogue code: W is lower triangular (W[n][k] = 0 for k > n); kernels may skip those blocks
#define EPI_FLAG_CAUSAL 0x100

template <typename T> struct EpiArgs {
  T* y;
  long long ldy;
  const T* resid;
  long long ldr;
  // EPI_HIST: row m of the GEMM is token (m / T) * .. + (m % T) of a [B,T] batch starting at time t0
  int Tseq, t0, Lh;
  long long ld2;  // EPI_BLOCKCOL: distance between column blocks
  const PeerDest* peer;  // EPI_STORE only, may be NULL: the rows go to every rank's inbox (row stride ldy) instead of y
};

struct EpiArgsAny {
  void* y;
  long long ldy;
  const void* resid;
  long long ldr;
  int Tseq, t0, Lh;
  long long ld2 = 0;
  const PeerDest* peer = nullptr;
  template <typename U> EpiArgs<U> as() const {
    EpiArgs<U> e;
    e.y = (U*)y; e.ldy = ldy; e.resid = (const U*)resid; e.ldr = ldr; e.Tseq = Tseq; e.t0 = t0; e.Lh = Lh;
    e.ld2 = ld2;
    e.peer = peer;
    return e;
  }
};

template <typename T, int EPI>
__device__ __forceinline__ void epilogue_store(const EpiArgs<T>& ep, int m, int n, float acc, float acc2) {
  if (EPI == EPI_STORE) {
    if (sizeof(T) == 2 && ep.peer) {
      const bf16 v = __float2bfloat16_rn(acc);
      for (int p = 0; p < ep.peer->n; p++) ep.peer->dest[p][(size_t)m * ep.ldy + n] = v;
    } else {
      ep.y[(size_t)m * ep.ldy + n] = Elem<T>::from_f(acc);
    }
  } else if (EPI == EPI_RESID) {
    float r = Elem<T>::to_f(ep.resid[(size_t)m * ep.ldr + n]);
    ep.y[(size_t)m * ep.ldy + n] = Elem<T>::from_f(r + round_to<T>(acc));
  } else if (EPI == EPI_GELU_MUL) {
    float g = round_to<T>(gelu_tanh(round_to<T>(acc)));
    ep.y[(size_t)m * ep.ldy + n] = Elem<T>::from_f(g * round_to<T>(acc2));
  } else if (EPI == EPI_BLOCKCOL) {
    ep.y[(size_t)m * ep.ldy + (size_t)(n / ep.Tseq) * ep.ld2 + (n % ep.Tseq)] = Elem<T>::from_f(acc);
  } else {  // EPI_HIST; ldy carries the channel count
    int b = m / ep.Tseq, t = ep.t0 + (m - b * ep.Tseq);
    ep.y[hist_off(b, n, t, (int)ep.ldy, ep.Lh)] = Elem<T>::from_f(acc);
  }
}

// host-side dispatchers implemented in the kernel files
int gemm_simt_dispatch(const void* A, long long lda, const void* B, long long ldb, long long skb, const void* B2,
                       int M, int N, int K, int epi, const EpiArgsAny& ep, int dtype, cudaStream_t st);
int gemm_tc_dispatch(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N,
                     int K, int epi, int causal, const EpiArgsAny& ep, cudaStream_t st);
bool gemm_tc_supported(const void* A, long long lda, const void* B, long long ldb, long long skb, const void* B2,
                       int M, int N, int K, int epi, const EpiArgsAny& ep, int dtype);
int skinny_dispatch(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N, int K,
                    int epi, const EpiArgsAny& ep, const void* norm_w, float eps, int dtype, int pdl, cudaStream_t st);
bool skinny_supported(const void* A, long long lda, const void* B, long long ldb, long long skb, const void* B2,
                      int M, int N, int K, int epi, int dtype);
