// C-ABI entry points that dispatch between the linear-layer kernels (see include/stu_b200.h).
#include <stdlib.h>

#include "common.cuh"
#include "epilogue.cuh"

extern "C" int stu_b200_version(void) { return 100; }

enum { BACKEND_AUTO = 0, BACKEND_SIMT = 1, BACKEND_TCGEN05 = 2, BACKEND_SKINNY = 3 };

// y = epilogue(x[M,K] @ W[N,K]^T).  element (n,k) of W at W[n*w_row_stride + k*w_k_stride].
//   epilogue 0: y = acc                  1: y = resid + round(acc)
//            2: y = round(gelu_tanh(round(x@W^T))) * round(x@W2^T)
//            +0x100: W is lower triangular (zero for k > n); the tcgen05 path skips those k-blocks
//            3: scatter into the parity-split history (y = hist base, hist_T tokens per sequence
//               starting at time hist_t0, N channels, hist_Lh elements per parity row)
//            5: y[m*y_row_stride + (n / hist_T) * resid_row_stride + (n % hist_T)] = acc  (columns in blocks of hist_T,
//               blocks resid_row_stride elements apart; resid itself is not read)
// norm_w != NULL asks for x to be RMS-normalised (eps) on the way in; only the decode (skinny) path
// fuses this, other shapes return STU_ERR_UNSUPPORTED so that the caller normalises separately.
static int g_pdl = -1;   // -1: not decided yet (environment), 0 off, 1 on
bool pdl_enabled() {
  if (g_pdl < 0) g_pdl = getenv("STU_B200_DISABLE_PDL") ? 0 : 1;
  return g_pdl != 0;
}
// Programmatic (overlapped) launches of the decode kernels on or off for the launches that follow; returns the
// previous setting.  A captured CUDA graph keeps the setting it was captured with.
extern "C" int stu_set_programmatic_launch(int on) {
  const int prev = pdl_enabled() ? 1 : 0;
  g_pdl = on ? 1 : 0;
  return prev;
}

bool skinny_umma_takes(int M, int N, int K, int epi, bool norm, bool peer);   // gemm_tc.cu

// Small-M shapes for which the tcgen05 GEMM beats the weight-streaming kernel.
static bool prefers_tensor_gemm(int M, int N) { return (M >= 32 && N >= 5120) || (M >= 16 && N >= 32768); }

extern "C" int stu_linear(const void* x, long long x_row_stride, const void* W, long long w_row_stride,
                          long long w_k_stride, const void* W2, const void* resid, long long resid_row_stride,
                          void* y, long long y_row_stride, int M, int N, int K, int epilogue, int hist_T,
                          int hist_t0, int hist_Lh, const void* norm_w, float eps, int dtype, int backend,
                          void* stream) {
  if (!x || !W || !y) return STU_ERR_NULL;
  if (M < 0 || N <= 0 || K <= 0) return STU_ERR_SHAPE;
  if (M == 0) return STU_OK;
  const int causal = (epilogue & EPI_FLAG_CAUSAL) ? 1 : 0;
  const int pdl = epilogue & (STU_FLAG_OVERLAP | STU_FLAG_EARLY_TRIGGER);  // honoured by the skinny kernels only
  epilogue &= ~(EPI_FLAG_CAUSAL | STU_FLAG_OVERLAP | STU_FLAG_EARLY_TRIGGER);
  if ((epilogue < EPI_STORE || epilogue > EPI_HIST) && epilogue != EPI_BLOCKCOL) return STU_ERR_UNSUPPORTED;
  // EPI_BLOCKCOL: hist_T = columns per block, resid_row_stride = distance between blocks (elements); resid unused
  if (epilogue == EPI_BLOCKCOL && (hist_T <= 0 || resid_row_stride <= 0)) return STU_ERR_SHAPE;
  if (epilogue == EPI_GELU_MUL && !W2) return STU_ERR_NULL;
  if (epilogue == EPI_RESID && !resid) return STU_ERR_NULL;
  if (epilogue == EPI_HIST && (hist_T <= 0 || hist_Lh <= 0 || hist_t0 < 0 || (M % hist_T) != 0 ||
                               hist_t0 + hist_T > 2 * hist_Lh))
    return STU_ERR_SHAPE;
  if (dtype != STU_F32 && dtype != STU_BF16) return STU_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  EpiArgsAny ep;
  ep.y = y;
  ep.ldy = (epilogue == EPI_HIST) ? (long long)N : y_row_stride;
  ep.resid = resid;
  ep.ldr = resid_row_stride;
  ep.Tseq = hist_T;
  ep.t0 = hist_t0;
  ep.Lh = hist_Lh;
  ep.ld2 = (epilogue == EPI_BLOCKCOL) ? resid_row_stride : 0;

  bool sk_ok = skinny_supported(x, x_row_stride, W, w_row_stride, w_k_stride, W2, M, N, K, epilogue, dtype);
  if (norm_w) {
    if (!sk_ok || dtype != STU_BF16 || (backend != BACKEND_AUTO && backend != BACKEND_SKINNY))
      return STU_ERR_UNSUPPORTED;
    return skinny_dispatch(x, x_row_stride, W, w_row_stride, W2, M, N, K, epilogue, ep, norm_w, eps, dtype, pdl, st);
  }
  bool tc_ok = gemm_tc_supported(x, x_row_stride, W, w_row_stride, w_k_stride, W2, M, N, K, epilogue, ep, dtype);
  if (backend == BACKEND_AUTO) {
    // 17..64 rows: the weight-streaming kernel's time grows with M, the tcgen05 GEMM's does not but it needs enough
    // 128-wide column tiles to fill the machine (measured cross-over on a B200, weights from HBM)
    // (gate/up at up to 32 rows stays on the weight-streaming side: its staged kernel keeps every SM pulling, while
    // 32 rows are a quarter of one 128-row tile for the tensor-core GEMM)
    // (17..64 rows stay on the weight-streaming side whatever N: there the weights are the tensor core's 128-row
    // operand; LM head 32 x 200064 x 1536: 103.5 against 111.3 us)
    if (sk_ok && tc_ok && prefers_tensor_gemm(M, N) && !skinny_umma_takes(M, N, K, epilogue, false, false))
      sk_ok = false;
    backend = sk_ok ? BACKEND_SKINNY : (tc_ok ? BACKEND_TCGEN05 : BACKEND_SIMT);
  }
  switch (backend) {
    case BACKEND_SKINNY:
      if (!sk_ok) return STU_ERR_UNSUPPORTED;
      return skinny_dispatch(x, x_row_stride, W, w_row_stride, W2, M, N, K, epilogue, ep, nullptr, eps, dtype, pdl, st);
    case BACKEND_TCGEN05:
      if (!tc_ok) return STU_ERR_UNSUPPORTED;
      return gemm_tc_dispatch(x, x_row_stride, W, w_row_stride, W2, M, N, K, epilogue, causal, ep, st);
    case BACKEND_SIMT:
      return gemm_simt_dispatch(x, x_row_stride, W, w_row_stride, w_k_stride, W2, M, N, K, epilogue, ep, dtype, st);
  }
  return STU_ERR_UNSUPPORTED;
}

// y = x[M,K] @ W[N,K]^T for M <= 64 rows (bf16) with the exchange fused in: the rows are stored into every rank's inbox
// (exchange descriptor `peer_dest`, device memory) with row stride dest_row_stride, and the ranks are signalled when the
// last CTA has stored.  Weight-streaming kernel only.
extern "C" int stu_linear_push(const void* x, long long x_row_stride, const void* W, long long w_row_stride, int M,
                               int N, int K, const void* peer_dest, long long dest_row_stride, int dtype,
                               void* stream) {
  if (!x || !W || !peer_dest) return STU_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0) return STU_ERR_SHAPE;
  if (dtype != STU_BF16) return STU_ERR_DTYPE;
  if (!skinny_supported(x, x_row_stride, W, w_row_stride, 1, nullptr, M, N, K, EPI_STORE, dtype))
    return STU_ERR_UNSUPPORTED;
  EpiArgsAny ep;
  ep.y = nullptr;
  ep.ldy = dest_row_stride;
  ep.resid = nullptr;
  ep.ldr = 0;
  ep.Tseq = ep.t0 = ep.Lh = 0;
  ep.peer = (const PeerDest*)peer_dest;
  return skinny_dispatch(x, x_row_stride, W, w_row_stride, nullptr, M, N, K, EPI_STORE, ep, nullptr, 0.f, dtype, 0,
                         (cudaStream_t)stream);
}

// 1 when stu_linear would fuse the RMSNorm for this shape (decode path), else 0.
extern "C" int stu_linear_can_fuse_norm(int M, int N, int K, int epilogue, int dtype) {
  if (dtype != STU_BF16 || M < 1 || M > 64 || K % 8 || epilogue == EPI_HIST) return 0;
  if (prefers_tensor_gemm(M, N)) return 0;   // a separate norm kernel + the tcgen05 GEMM is faster there
  // 17..64 rows: every CTA would recompute the statistics of all rows (the 32-feature kernel from L2, the staged
  // gate/up kernel from its shared-memory copy); a separate norm kernel measured faster both times (24-layer model,
  // B = 32: 2.17 against 2.27 ms per token step, and 2.19 against 2.30 ms).  The kernels accept norm_w all the same.
  // (a fused norm inside the tcgen05 token-step kernel measured slower as well: 2.12-2.25 against 1.71-1.85 ms)
  if (M > 16) return 0;
  return 1;
}
