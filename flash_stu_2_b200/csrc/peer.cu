// Peer memory for the tensor-parallel token loop (see peer.cuh) and the kernel on the receiving side.
//
// The reference is single-GPU; these entry points have no counterpart there.  They replace the all-gather after the
// STU sub-layer and the all-reduce after the MLP / attention sub-layers of a channel- and column-sharded model
// (the sub-layers themselves: flash_stu/layers/stu_layer.py:78-98, flash_stu/layers/attention_layer.py) for the one
// new token of a cached decode step, where the messages are a few KB and the cost of a collective is its latency.
#include <string.h>

#include "common.cuh"
#include "peer.cuh"

#define STATUS_PEER_WAIT 10

extern "C" int stu_peer_dest_bytes(void) { return (int)sizeof(PeerDest); }

// A dedicated device allocation (zero-filled) whose inter-process handle maps exactly it.
extern "C" int stu_peer_alloc(void** ptr, long long bytes) {
  if (!ptr || bytes <= 0) return STU_ERR_SHAPE;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) { cudaFree(p); return (int)e; }
  *ptr = p;
  return STU_OK;
}
extern "C" int stu_peer_free(void* ptr) { return ptr ? (int)cudaFree(ptr) : STU_OK; }
extern "C" int stu_peer_export(void* ptr, void* handle64) {
  if (!ptr || !handle64) return STU_ERR_NULL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  return (int)cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle64, ptr);
}
extern "C" int stu_peer_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return STU_ERR_NULL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int stu_peer_close(void* ptr) { return ptr ? (int)cudaIpcCloseMemHandle(ptr) : STU_OK; }
// Host <-> peer-buffer copies for setting up the exchange descriptors and for tests (synchronous).
extern "C" int stu_peer_write(void* dst, const void* host_src, long long bytes) {
  if (!dst || !host_src || bytes <= 0) return STU_ERR_NULL;
  return (int)cudaMemcpy(dst, host_src, (size_t)bytes, cudaMemcpyHostToDevice);
}
extern "C" int stu_peer_read(void* host_dst, const void* src, long long bytes) {
  if (!host_dst || !src || bytes <= 0) return STU_ERR_NULL;
  return (int)cudaMemcpy(host_dst, src, (size_t)bytes, cudaMemcpyDeviceToHost);
}

namespace {

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// One CTA per row.  Waits until every sender's flag has reached the local epoch of the exchange (set by this rank's
// own producing kernel, which ran before this one in the stream), then
//   x[row] = round(x[row] + round(sum over slots of inbox[slot][row]))        (the sum in fp32)
// and, with norm_w, xn[row] = round(x[row] * rsqrt(mean(x[row]^2) + eps) * norm_w), the RMSNorm of the next sub-layer.
// The wait is bounded: after wait_ns the CTA reports status 10 and returns without touching x.
template <int VPT>
__global__ void __launch_bounds__(256) peer_combine_kernel(bf16* __restrict__ x, long long x_rs,
                                                           const bf16* __restrict__ inbox, long long slot_stride,
                                                           long long in_rs, int slots, const unsigned* flags, int n,
                                                           const unsigned* epoch, const bf16* __restrict__ norm_w,
                                                           bf16* __restrict__ xn, long long xn_rs, float eps, int d,
                                                           int* status, unsigned long long wait_ns) {
  __shared__ int s_ok;
  __shared__ float s_red[8];
  const int row = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (tid < n) {
    const unsigned target = *epoch;
    bool ok = false;
    uint64_t start = 0;
    for (unsigned it = 0; it < (1u << 26); ++it) {
      if ((int)(ld_acquire_sys(flags + tid) - target) >= 0) { ok = true; break; }
      if ((it & 63u) == 63u) {
        const uint64_t now = global_ns();
        if (start == 0) start = now;
        else if (now - start > wait_ns) break;
      }
    }
    if (!ok) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) {
    if (tid == 0 && status) atomicExch(status, STATUS_PEER_WAIT);
    return;
  }
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    const int c = (tid + 256 * k) * 8;
    if (c < d) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < slots; s++) {
        float t[8];
        load_vec(inbox + (size_t)s * slot_stride + (size_t)row * in_rs + c, t);
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] += t[j];
      }
      float xv[8];
      load_vec(x + (size_t)row * x_rs + c, xv);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        v[k][j] = round_to<bf16>(xv[j] + round_to<bf16>(acc[j]));
        ss += v[k][j] * v[k][j];
      }
      store_vec(x + (size_t)row * x_rs + c, v[k]);
    }
  }
  if (!norm_w) return;
  ss = warp_sum(ss);
  if ((tid & 31) == 0) s_red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; w++) tot += s_red[w];
  const float r = rsqrtf(tot / (float)d + eps);
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    const int c = (tid + 256 * k) * 8;
    if (c < d) {
      float w[8], o[8];
      load_vec(norm_w + c, w);
#pragma unroll
      for (int j = 0; j < 8; j++) o[j] = v[k][j] * r * w[j];
      store_vec(xn + (size_t)row * xn_rs + c, o);
    }
  }
}

// Push + wait + combine of one exchange in ONE launch, one CTA per row of the token batch:
//   1. the CTA copies this rank's contribution of its row (`cols` values: the rank's channel slice for an all-gather,
//      a full-width partial sum for an all-reduce) into EVERY rank's inbox with 16-byte stores (whole lines over
//      NVLink), then raises this sender's counter of the row on every rank (one system-scope release);
//   2. it waits (bounded) until the counters of all other senders of the row have reached the row's own epoch;
//   3. x[row] = round(x[row] + round(sum of the inbox blocks' rows)), optionally followed by the next RMSNorm.
// Rows are independent: no grid-wide step, and a row's exchange starts as soon as its CTA runs.
template <int VPT>
__global__ void __launch_bounds__(256) peer_exchange_kernel(const PeerXchg* __restrict__ xd, bf16* __restrict__ x,
                                                            long long x_rs, const bf16* __restrict__ src,
                                                            long long src_rs, int cols, int gather, long long slot_stride,
                                                            int rows, const bf16* __restrict__ norm_w,
                                                            bf16* __restrict__ xn, long long xn_rs, float eps, int d,
                                                            int* status, unsigned long long wait_ns) {
  __shared__ int s_ok;
  __shared__ float s_red[8];
  const int row = blockIdx.x, tid = threadIdx.x;
  const int n = xd->n, rank = xd->rank;
  const unsigned target = xd->epoch[row] + 1u;
  if (tid == 0) s_ok = 1;
  // ---- 1. this rank's row into every inbox
  {
    const size_t off = (gather ? (size_t)rank * cols : (size_t)rank * slot_stride) + (size_t)row * d;
    for (int c = tid * 8; c < cols; c += 256 * 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)row * src_rs + c);
      for (int p = 0; p < n; p++) *reinterpret_cast<uint4*>(xd->inbox[p] + off + c) = v;
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    for (int p = 0; p < n; p++)
      if (p != rank)
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(xd->flag[p] + (size_t)rank * rows + row) : "memory");
  }
  // ---- 2. the other senders of this row
  if (tid < n && tid != rank) {
    const unsigned* f = xd->flag[rank] + (size_t)tid * rows + row;
    bool ok = false;
    uint64_t start = 0;
    for (unsigned it = 0; it < (1u << 26); ++it) {
      if ((int)(ld_acquire_sys(f) - target) >= 0) { ok = true; break; }
      if ((it & 63u) == 63u) {
        const uint64_t now = global_ns();
        if (start == 0) start = now;
        else if (now - start > wait_ns) break;
      }
    }
    if (!ok) s_ok = 0;
  }
  __syncthreads();
  if (tid == 0) xd->epoch[row] = target;   // sent once more, whether or not the others arrived
  if (!s_ok) {
    if (tid == 0 && status) atomicExch(status, STATUS_PEER_WAIT);
    return;
  }
  // ---- 3. combine
  const bf16* inbox = xd->inbox[rank];
  const int slots = gather ? 1 : n;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    const int c = (tid + 256 * k) * 8;
    if (c < d) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < slots; s++) {
        float t[8];
        load_vec(inbox + (size_t)s * slot_stride + (size_t)row * d + c, t);
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] += t[j];
      }
      float xv[8];
      load_vec(x + (size_t)row * x_rs + c, xv);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        v[k][j] = round_to<bf16>(xv[j] + round_to<bf16>(acc[j]));
        ss += v[k][j] * v[k][j];
      }
      store_vec(x + (size_t)row * x_rs + c, v[k]);
    }
  }
  if (!norm_w) return;
  ss = warp_sum(ss);
  if ((tid & 31) == 0) s_red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; w++) tot += s_red[w];
  const float r = rsqrtf(tot / (float)d + eps);
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    const int c = (tid + 256 * k) * 8;
    if (c < d) {
      float w[8], o[8];
      load_vec(norm_w + c, w);
#pragma unroll
      for (int j = 0; j < 8; j++) o[j] = v[k][j] * r * w[j];
      store_vec(xn + (size_t)row * xn_rs + c, o);
    }
  }
}

}  // namespace

extern "C" int stu_peer_xchg_bytes(void) { return (int)sizeof(PeerXchg); }

// One exchange of the token step in one launch (see peer_exchange_kernel).  xchg = the exchange's PeerXchg record in
// this rank's device memory; src [rows, cols] = this rank's contribution (gather != 0: its cols = d / n channels of every
// row; gather == 0: a full-width partial sum, cols = d); the inbox blocks are slot_stride elements apart.
extern "C" int stu_peer_exchange(const void* xchg, void* x, long long x_row_stride, const void* src,
                                 long long src_row_stride, int cols, int gather, long long slot_stride,
                                 const void* norm_w, void* xn, long long xn_row_stride, float eps, int rows, int d,
                                 int* status, int wait_ms, int dtype, void* stream) {
  if (!xchg || !x || !src || (norm_w && !xn)) return STU_ERR_NULL;
  if (dtype != STU_BF16) return STU_ERR_DTYPE;
  if (rows <= 0 || d <= 0 || d % 8 || d > 16384 || cols <= 0 || cols % 8 || cols > d) return STU_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(src) || (norm_w && (!aligned16(norm_w) || !aligned16(xn))) || x_row_stride % 8 ||
      src_row_stride % 8 || slot_stride % 8 || (norm_w && xn_row_stride % 8))
    return STU_ERR_ALIGN;
  const unsigned long long wait_ns = (unsigned long long)(wait_ms > 0 ? wait_ms : 2000) * 1000000ull;
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH_XCHG(V)                                                                                              \
  peer_exchange_kernel<V><<<rows, 256, 0, st>>>((const PeerXchg*)xchg, (bf16*)x, x_row_stride, (const bf16*)src,   \
                                                 src_row_stride, cols, gather, slot_stride, rows,                   \
                                                 (const bf16*)norm_w, (bf16*)xn, xn_row_stride, eps, d, status,     \
                                                 wait_ns)
  if (d <= 2048) LAUNCH_XCHG(1);
  else if (d <= 4096) LAUNCH_XCHG(2);
  else if (d <= 8192) LAUNCH_XCHG(4);
  else LAUNCH_XCHG(8);
#undef LAUNCH_XCHG
  STU_CHECK_LAUNCH();
  return STU_OK;
}

// Receiving side of one exchange: see peer_combine_kernel.  inbox = this rank's inbox region of the exchange
// ([slots] blocks slot_stride elements apart, rows in_row_stride apart), flags = this rank's n arrival counters of the
// exchange, epoch = this rank's own send counter of the exchange.  bf16, d % 8 == 0, d <= 16384, rows >= 1.
extern "C" int stu_peer_combine(void* x, long long x_row_stride, const void* inbox, long long slot_stride,
                                long long in_row_stride, int slots, const void* flags, int n_ranks, const void* epoch,
                                const void* norm_w, void* xn, long long xn_row_stride, float eps, int rows, int d,
                                int* status, int wait_ms, int dtype, void* stream) {
  if (!x || !inbox || !flags || !epoch || (norm_w && !xn)) return STU_ERR_NULL;
  if (dtype != STU_BF16) return STU_ERR_DTYPE;
  if (rows <= 0 || d <= 0 || d % 8 || d > 16384 || slots <= 0 || n_ranks <= 0 || n_ranks > STU_MAX_PEERS)
    return STU_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(inbox) || (norm_w && (!aligned16(norm_w) || !aligned16(xn))) || x_row_stride % 8 ||
      slot_stride % 8 || in_row_stride % 8 || (norm_w && xn_row_stride % 8))
    return STU_ERR_ALIGN;
  const unsigned long long wait_ns = (unsigned long long)(wait_ms > 0 ? wait_ms : 2000) * 1000000ull;
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH_COMBINE(V)                                                                                          \
  peer_combine_kernel<V><<<rows, 256, 0, st>>>((bf16*)x, x_row_stride, (const bf16*)inbox, slot_stride,          \
                                                in_row_stride, slots, (const unsigned*)flags, n_ranks,             \
                                                (const unsigned*)epoch, (const bf16*)norm_w, (bf16*)xn,            \
                                                xn_row_stride, eps, d, status, wait_ns)
  if (d <= 2048) LAUNCH_COMBINE(1);
  else if (d <= 4096) LAUNCH_COMBINE(2);
  else if (d <= 8192) LAUNCH_COMBINE(4);
  else LAUNCH_COMBINE(8);
#undef LAUNCH_COMBINE
  STU_CHECK_LAUNCH();
  return STU_OK;
}
