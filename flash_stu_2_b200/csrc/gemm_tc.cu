// Prefill linear layers on the 5th-generation tensor cores: D[M,N] = A[M,K] . B[N,K]^T in bf16 with
// fp32 accumulators held in tensor memory (TMEM).
//
// One CTA computes 128 x 128 or 128 x 256 output tiles.  Warp 0 is the TMA producer (cp.async.bulk.tensor, 128-byte
// swizzled 128x64 / 256x64 operand tiles into a ring of shared-memory stages), warp 1 allocates TMEM and
// issues tcgen05.mma from one thread, warps 2..5 drain the accumulator with tcgen05.ld and run the
// fused epilogue (store / residual add / tanh-GELU gate * up / transposed scatter into the projected
// history).  The kernel is persistent (one CTA per SM walks the tile list) and the accumulator is
// double-buffered in TMEM, so one tile's epilogue overlaps the next tile's main loop.  Every load is a plain
// single-CTA TMA load of this GPU's own memory.
//
// Every wait on an mbarrier is bounded: on expiry the waiter raises the status word, the CTA drains
// its outstanding bulk copies (bounded as well), frees its TMEM and returns.
#include <cooperative_groups.h>
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "epilogue.cuh"

int device_sm_count();   // SM count of the current device (cached per device)

namespace cg = cooperative_groups;

namespace {

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr uint32_t WAIT_LIMIT = 1u << 22;
enum { EPI_HIST_T = 4 };  // internal: rows = channels, columns = tokens (operands swapped by the host)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after WAIT_LIMIT polls or wait_ns of wall time (two seconds unless a test shortened it),
// whichever comes first.
// Returns false when the limit ran out or another role already gave up.
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned long long wait_ns) {
  uint64_t start = 0;
  for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u) {
      if (*abort_flag) return false;
      uint64_t now = global_ns();
      if (start == 0) start = now;
      else if (now - start > wait_ns) break;
    }
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major bf16 tile stored as rows of 128 bytes with the
// 128-byte swizzle (what the tensor maps below produce): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                 // leading byte offset (unused for swizzled K-major), encoded >> 4
  d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                 // descriptor version for this architecture
  d |= (uint64_t)2 << 61;                 // 128-byte swizzle
  return d;
}
// Instruction descriptor: D fp32, A/B bf16, both K-major, M = 128, N = the tile width (128 or 256).
template <int BN_>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  constexpr uint32_t IDESC =
      (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN_ >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
      "%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// tanh-GELU with the hardware tanh approximation (relative error ~2^-11, below the bf16 rounding that follows)
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(inner));
  return 0.5f * x * (1.0f + t);
}

// With `causal` the B operand is lower triangular (B[n][k] = 0 for k > n, the Toeplitz matrices of the STU
// full variant): k-blocks that lie entirely above the diagonal of the tile's last column are skipped.
__device__ __forceinline__ int tile_kb(int num_kb, int n0, int causal, int bn) {
  if (!causal) return num_kb;
  const int need = (n0 + bn + BK - 1) / BK;
  return need < num_kb ? need : num_kb;
}

// Persistent kernel: CTA i handles tiles i, i + gridDim.x, ...  The accumulator is double-buffered in TMEM
// (2 x TN columns, or 2 x 256 for the two accumulators of the gate/up epilogue), so the MMA warp starts the next
// tile while the epilogue warps drain the previous one.  TN = 256 (128 x 256 tiles) moves a third less operand
// data per flop through shared memory than 128 x 128 and is used when the problem has enough wide tiles.
template <int EPI, int STAGES, int TN = 128>
__global__ void __launch_bounds__(192, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA,
                                                         const __grid_constant__ CUtensorMap tmB,
                                                         const __grid_constant__ CUtensorMap tmB2, int M, int N,
                                                         int K, int tiles_m, int tiles_n, int m_fast,
                                                         int causal, EpiArgs<bf16> ep, int* status,
                                                         int drop_first_copy, unsigned long long wait_ns) {
  constexpr bool DUAL = (EPI == EPI_GELU_MUL);
  static_assert(!DUAL || TN == 128, "the two-accumulator epilogue uses 128-wide tiles");
  constexpr int BN = TN;                       // shadows the file-level default inside the kernel
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES * (DUAL ? 2 : 1);
  constexpr uint32_t ACC_COLS = DUAL ? 256 : (uint32_t)BN;
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* issued_ctr = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));
  int* consumed_ctr = issued_ctr + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128);
    }
    *abort_flag = 0;
    *issued_ctr = 0;
    *consumed_ctr = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer
      int g = 0;  // k-blocks issued so far (ring position)
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const int tm = m_fast ? (tile % tiles_m) : (tile / tiles_n);
        const int tn = m_fast ? (tile / tiles_m) : (tile % tiles_n);
        const int m0 = tm * BM, n0 = tn * BN;
        const int kb_end = tile_kb(num_kb, n0, causal, BN);
        for (int kb = 0; kb < kb_end; kb++, g++) {
          const int s = g % STAGES;
          const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, wait_ns)) { ok = false; break; }
          unsigned char* sa = smem + s * STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          // drop_first_copy (failure-detection test only): the first stage's copies are never issued, so its
          // barrier never completes and the consumer's bounded wait has to run out
          if (!(drop_first_copy && g == 0)) {
            tma_load_2d(sa, &tmA, &full_bar[s], kb * BK, m0);
            tma_load_2d(sa + A_BYTES, &tmB, &full_bar[s], kb * BK, n0);
            if (DUAL) tma_load_2d(sa + A_BYTES + B_BYTES, &tmB2, &full_bar[s], kb * BK, n0);
            *issued_ctr = g + 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer
      int g = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, it++) {
        const int buf = it & 1;
        const uint32_t acc_addr = tmem_base + (uint32_t)buf * ACC_COLS;
        const int tn_ = m_fast ? (tile / tiles_m) : (tile % tiles_n);
        const int kb_end = tile_kb(num_kb, tn_ * BN, causal, BN);
        if (!mbar_wait(&tmem_empty[buf], (((uint32_t)it >> 1) & 1u) ^ 1u, abort_flag, wait_ns)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int kb = 0; kb < kb_end; kb++, g++) {
          const int s = g % STAGES;
          const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, wait_ns)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + A_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; kk++) {
            // advancing 16 bf16 = 32 bytes along K inside the swizzled row: +2 in the (>>4) address field
            // gate/up: the two 128-row weight tiles lie back to back in the stage and form one 256-row B operand,
            // so one N = 256 instruction fills both accumulators (columns 0..127 gate, 128..255 up) and the A tile
            // is read from shared memory once instead of twice
            if (DUAL)
              umma<256>(acc_addr, da + 2 * kk, db + 2 * kk, (kb | kk) ? 1u : 0u);
            else
              umma<BN>(acc_addr, da + 2 * kk, db + 2 * kk, (kb | kk) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);  // arrives when the MMAs above have finished reading this stage
          *consumed_ctr = g + 1;
        }
        if (ok) umma_commit(&tmem_full[buf]);
      }
    }
  } else {
    // ---------------- epilogue warps: TMEM lane quarter = warp % 4
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, it++) {
      const int tm = m_fast ? (tile % tiles_m) : (tile / tiles_n);
      const int tn = m_fast ? (tile / tiles_m) : (tile % tiles_n);
      const int m0 = tm * BM, n0 = tn * BN;
      const int m = m0 + row;
      const int buf = it & 1;
      const uint32_t acc_addr = tmem_base + (uint32_t)buf * ACC_COLS;
      bool ok = mbar_wait(&tmem_full[buf], ((uint32_t)it >> 1) & 1u, abort_flag, wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int cch = 0; cch < BN / 32; cch++) {
        uint32_t r[32], r2[32];
        const uint32_t taddr = acc_addr + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(cch * 32);
        tmem_ld32(taddr, r);
        if (DUAL) tmem_ld32(taddr + BN, r2);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int nb = n0 + cch * 32;
        if (m < M && nb < N) {
          if (EPI == EPI_HIST_T) {
            // row m = channel, columns = tokens nb..nb+31 of the flattened [B, T] batch
            const int d = (int)ep.ldy;
            const bool fast = (ep.Tseq % 32 == 0) && (ep.t0 % 16 == 0) && (nb + 32 <= N) && (ep.Lh % 8 == 0);
            if (fast) {
              const int b = nb / ep.Tseq, t = ep.t0 + (nb - b * ep.Tseq);  // t % 16 == 0
              float ev[16], od[16];
#pragma unroll
              for (int j = 0; j < 16; j++) {
                ev[j] = __uint_as_float(r[2 * j]);
                od[j] = __uint_as_float(r[2 * j + 1]);
              }
              bf16* pe = ep.y + ((size_t)((size_t)b * d + m) * 2 + 0) * ep.Lh + (t >> 1);
              bf16* po = ep.y + ((size_t)((size_t)b * d + m) * 2 + 1) * ep.Lh + (t >> 1);
              store_vec(pe, ev);
              store_vec(pe + 8, ev + 8);
              store_vec(po, od);
              store_vec(po + 8, od + 8);
            } else {
              for (int j = 0; j < 32; j++) {
                int n = nb + j;
                if (n < N) {
                  int b = n / ep.Tseq, t = ep.t0 + (n - b * ep.Tseq);
                  ep.y[hist_off(b, m, t, d, ep.Lh)] = __float2bfloat16_rn(__uint_as_float(r[j]));
                }
              }
            }
          } else {
            bf16* yrow = ep.y + (size_t)m * ep.ldy + nb;
            if (EPI == EPI_BLOCKCOL)   // columns in blocks of Tseq, ld2 elements apart
              yrow = ep.y + (size_t)m * ep.ldy + (size_t)(nb / ep.Tseq) * ep.ld2 + (nb % ep.Tseq);
            const bf16* rrow = (EPI == EPI_RESID) ? ep.resid + (size_t)m * ep.ldr + nb : nullptr;
            const bool vec = (nb + 32 <= N) && (EPI != EPI_BLOCKCOL || ep.Tseq % 32 == 0);
#pragma unroll
            for (int v8 = 0; v8 < 4; v8++) {
              float o[8];
              if (EPI == EPI_RESID) {
                float rs[8];
                if (vec) {
                  load_vec(rrow + v8 * 8, rs);
                } else {
#pragma unroll
                  for (int j = 0; j < 8; j++) rs[j] = (nb + v8 * 8 + j < N) ? __bfloat162float(rrow[v8 * 8 + j]) : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 8; j++) o[j] = rs[j] + round_to<bf16>(__uint_as_float(r[v8 * 8 + j]));
              } else if (EPI == EPI_GELU_MUL) {
#pragma unroll
                for (int j = 0; j < 8; j++) {
                  float gte = round_to<bf16>(gelu_tanh_fast(round_to<bf16>(__uint_as_float(r[v8 * 8 + j]))));
                  o[j] = gte * round_to<bf16>(__uint_as_float(r2[v8 * 8 + j]));
                }
              } else {
#pragma unroll
                for (int j = 0; j < 8; j++) o[j] = __uint_as_float(r[v8 * 8 + j]);
              }
              if (vec) {
                store_vec(yrow + v8 * 8, o);
              } else if (EPI == EPI_BLOCKCOL) {
#pragma unroll
                for (int j = 0; j < 8; j++) {
                  const int n = nb + v8 * 8 + j;
                  if (n < N)
                    ep.y[(size_t)m * ep.ldy + (size_t)(n / ep.Tseq) * ep.ld2 + (n % ep.Tseq)] = __float2bfloat16_rn(o[j]);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 8; j++)
                  if (nb + v8 * 8 + j < N) yrow[v8 * 8 + j] = __float2bfloat16_rn(o[j]);
              }
            }
          }
        }
      }
      // this thread's TMEM reads of the buffer are complete (wait::ld above): hand it back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&tmem_empty[buf]);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (*abort_flag) {
    // A wait ran out.  Report it, then let copies that were issued but never consumed land (bounded)
    // before shared memory is released.
    if (threadIdx.x == 0) {
      if (status) atomicExch(status, 3);
      const int issued = *issued_ctr, consumed = *consumed_ctr;
      const uint64_t drain_start = global_ns();
      for (int g = consumed; g < issued; g++) {
        const int s = g % STAGES;
        const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
        for (uint32_t w = 0; w < WAIT_LIMIT; ++w) {
          if (mbar_try_wait(&full_bar[s], ph)) break;
          if ((w & 255u) == 255u && global_ns() - drain_start > wait_ns) break;
        }
      }
    }
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

// ---------------------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// 2-D map over a row-major bf16 matrix [rows, cols] with row stride ld (elements); box 64 x box_rows, 128B swizzle.
// A map depends on nothing but these arguments, so the encoded maps are kept in a small per-thread table keyed by
// them (a token step asks for the same few dozen maps over and over; an entry never goes stale, it is just an address
// and a shape).
struct MapKey {
  const void* base;
  long long rows, cols, ld;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int MAP_SLOTS = 1024;   // direct-mapped
int make_map_uncached(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows);
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows = BM) {
  static thread_local MapSlot* table = nullptr;
  if (!table) table = new MapSlot[MAP_SLOTS]();
  const MapKey key{base, rows, cols, ld, box_rows};
  unsigned long long h = (unsigned long long)(uintptr_t)base * 0x9E3779B97F4A7C15ull;
  h ^= (unsigned long long)rows * 0xC2B2AE3D27D4EB4Full + (unsigned long long)cols * 0x165667B19E3779F9ull +
       (unsigned long long)ld * 0x27D4EB2F165667C5ull + (unsigned long long)box_rows;
  MapSlot& slot = table[(h >> 20) % MAP_SLOTS];
  if (slot.used && slot.key == key) {
    *map = slot.map;
    return STU_OK;
  }
  const int rc = make_map_uncached(map, base, rows, cols, ld, box_rows);
  if (rc == STU_OK) {
    slot.key = key;
    slot.map = *map;
    slot.used = true;
  }
  return rc;
}
int make_map_uncached(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return STU_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? STU_OK : STU_ERR_UNSUPPORTED;
}

// Failure-detection test hooks (stu_test_inject_wait_expiry): drop the first operand copy of the next launch, and the
// wall-time bound of every mbarrier wait.
int g_drop_first_copy = 0;
unsigned long long g_wait_ns = 2000000000ull;

template <int EPI, int STAGES, int TN = 128>
int launch_tc(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& b2, int M, int N, int K, int m_fast,
              int causal, const EpiArgs<bf16>& ep, int* status, cudaStream_t st) {
  constexpr bool DUAL = (EPI == EPI_GELU_MUL);
  constexpr int BN = TN;
  constexpr int STAGE_BYTES = A_BYTES + BN * BK * 2 * (DUAL ? 2 : 1);
  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024 + 256;
  auto k = gemm_tc_kernel<EPI, STAGES, TN>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int sm_count = device_sm_count();
  const int tiles = tiles_m * tiles_n;
  const int grid = tiles < sm_count ? tiles : sm_count;  // one persistent CTA per SM
  const int drop = g_drop_first_copy;
  g_drop_first_copy = 0;   // the injected fault applies to one launch
  k<<<grid, 192, smem, st>>>(a, b, b2, M, N, K, tiles_m, tiles_n, m_fast, causal, ep, status, drop, g_wait_ns);
  STU_CHECK_LAUNCH();
  return STU_OK;
}


// ------------------------------------------------------------------------------------------------
// Token-step linear layers for 9..64 activation rows on the tensor cores, operands swapped: the WEIGHTS are the
// 128-row operand (a tile = 128 output features, or 64 gate + 64 up rows of the same 64 features), the activation rows
// the 16-, 32- or 64-column one, so every weight byte passes through shared memory exactly once and goes straight into
// tcgen05.mma (M = 128, N = 32, K = 16); nothing is staged through registers and there is no cross-warp reduction.
// The K range is split over the CTAs of a thread-block cluster (up to 16; grid = tiles x KSPLIT, about one to two CTAs per SM,
// 80 KB of operands in flight each); every CTA drains its 128 x 32 fp32 accumulator from tensor memory into its own
// shared memory (token-major, conflict-free), the cluster synchronises, and every CTA sums the partial tiles of its
// share of the tokens in a fixed order through distributed shared memory and runs their epilogue (coalesced along
// the features).
// Launched with the programmatic attribute: the successor is released once tensor memory has been allocated (a
// co-resident successor that allocated first could otherwise block this kernel's allocation while waiting for it);
// with early_weights (the caller's promise that the preceding kernel does not write the weights) the weight tiles of
// the first stages are requested before griddepcontrol.wait, the activation tiles after it.

// SU_BN: activation rows per tile, 16, 32 or 64 (the N of the MMA, the accumulator's columns).  nstages: ring depth,
// chosen by the host: shallow (two CTAs per SM) for grids of more CTAs than SMs, deep below that.
// (A fused RMSNorm - the drain warps normalising the rows into swizzled shared-memory tiles while the weight stream
// runs, bit-identical to the norm kernel - was built and measured: the 24-layer token step went from 1.71-1.85 ms
// to 2.12-2.25 ms, the MMAs waiting for 32 rows of statistics that a separate, overlapped norm kernel has long
// finished.  Callers keep the separate norm kernel.)
constexpr int SU_MAXST = 10;
template <int EPI, int KSPLIT, int SU_BN>
__global__ void __launch_bounds__(192, 1)
    skinny_umma_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmW2,
                       const __grid_constant__ CUtensorMap tmX, int M, int N, int K, EpiArgs<bf16> ep, int* status,
                       int early_weights, unsigned long long wait_ns, int nstages) {
  constexpr bool DUAL = (EPI == EPI_GELU_MUL);
  constexpr int NF = DUAL ? 64 : 128;   // output features per tile
  constexpr int SU_B_BYTES = SU_BN * BK * 2;
  constexpr int PART_BYTES = SU_BN * BM * 4;
  constexpr int stage_bytes = A_BYTES + SU_B_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * NF;
  const int num_kb = (K + BK - 1) / BK;
  const int per = (num_kb + KSPLIT - 1) / KSPLIT;
  const int kb0 = (int)blockIdx.y * per;
  const int nkb = max(0, min(num_kb, kb0 + per) - kb0);
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  // ring | partial tile | barriers
  float* part = reinterpret_cast<float*>(smem + nstages * stage_bytes);   // [SU_BN tokens][128 rows]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + nstages * stage_bytes + PART_BYTES);
  uint64_t* empty_bar = full_bar + SU_MAXST;
  uint64_t* tmem_full = empty_bar + SU_MAXST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* issued_ctr = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));
  int* consumed_ctr = issued_ctr + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < nstages; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full, 1);
    *abort_flag = 0;
    *issued_ctr = 0;
    *consumed_ctr = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(SU_BN < 32 ? 32 : SU_BN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();   // only now: this CTA holds its tensor memory

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer
      auto load_w = [&](int s, int kb) {
        unsigned char* sa = smem + s * stage_bytes;
        if (DUAL) {   // 64 gate rows, then the 64 up rows of the same features
          tma_load_2d(sa, &tmW, &full_bar[s], kb * BK, n0);
          tma_load_2d(sa + A_BYTES / 2, &tmW2, &full_bar[s], kb * BK, n0);
        } else {
          tma_load_2d(sa, &tmW, &full_bar[s], kb * BK, n0);
        }
      };
      auto load_x = [&](int s, int kb) {
        tma_load_2d(smem + s * stage_bytes + A_BYTES, &tmX, &full_bar[s], kb * BK, 0);
      };
      const int pre = early_weights ? min(nstages, nkb) : 0;
      for (int g = 0; g < pre; g++) {
        mbar_expect_tx(&full_bar[g], stage_bytes);
        load_w(g, kb0 + g);
        *issued_ctr = g + 1;
      }
      pdl_wait();   // the activations are the output of the kernel before this one
      for (int g = 0; g < pre; g++) load_x(g, kb0 + g);
      for (int g = pre; g < nkb; g++) {
        const int s = g % nstages;
        const uint32_t ph = (uint32_t)(g / nstages) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, wait_ns)) break;
        mbar_expect_tx(&full_bar[s], stage_bytes);
        load_w(s, kb0 + g);
        load_x(s, kb0 + g);
        *issued_ctr = g + 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer
      bool ok = true;
      for (int g = 0; ok && g < nkb; g++) {
        const int s = g % nstages;
        const uint32_t ph = (uint32_t)(g / nstages) & 1u;
        if (!mbar_wait(&full_bar[s], ph, abort_flag, wait_ns)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = smem_u32(smem + s * stage_bytes);
        const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + A_BYTES);
#pragma unroll
        for (int kk = 0; kk < BK / 16; kk++) umma<SU_BN>(tmem_base, da + 2 * kk, db + 2 * kk, (g | kk) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
        *consumed_ctr = g + 1;
      }
      if (ok && nkb > 0) umma_commit(tmem_full);
    }
  } else {
    // ---------------- accumulator drain: TMEM lane quarter = warp % 4, one weight row per thread
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    bool ok = true;
    if (nkb > 0) {
      ok = mbar_wait(tmem_full, 0, abort_flag, wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
#pragma unroll
    for (int h = 0; h < (SU_BN + 31) / 32; h++) {   // 16 rows: 32 columns are allocated, the upper 16 unused
      uint32_t r[32];
#pragma unroll
      for (int c = 0; c < 32; c++) r[c] = 0u;
      if (nkb > 0 && ok) {
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(h * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
#pragma unroll
      for (int c = 0; c < (SU_BN < 32 ? SU_BN : 32); c++) part[(h * 32 + c) * BM + row] = __uint_as_float(r[c]);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  // ---- the partial tiles of the cluster meet (the role branches left the warps of the producer and of the MMA
  // issuer diverged: they reconverge before the aligned cluster barrier)
  __syncwarp();
  __syncthreads();
  cg::cluster_group cluster = cg::this_cluster();
  if constexpr (KSPLIT > 1) cluster.sync();
  {
    // every CTA of the cluster sums and stores the tokens rank, rank + KSPLIT, ... of the tile (fixed order of the
    // partial tiles, whoever sums them)
    pdl_wait();   // returns at once (the producer waited before the first activation copy)
    const int rank = KSPLIT > 1 ? (int)cluster.block_rank() : 0;
    const float* parts[KSPLIT];
#pragma unroll
    for (int rk = 0; rk < KSPLIT; rk++) parts[rk] = KSPLIT > 1 ? cluster.map_shared_rank(part, rk) : part;
    auto sum_at = [&](int idx) {
      float v = parts[0][idx];
#pragma unroll
      for (int rk = 1; rk < KSPLIT; rk++) v += parts[rk][idx];
      return v;
    };
    if (!*abort_flag) {
      for (int e = threadIdx.x; e < ((SU_BN + KSPLIT - 1) / KSPLIT) * NF; e += 192) {
        const int mi = e / NF, f = e - mi * NF, m = rank + mi * KSPLIT, n = n0 + f;
        if (m < M && m < SU_BN && n < N)
          epilogue_store<bf16, EPI>(ep, m, n, sum_at(m * BM + f), DUAL ? sum_at(m * BM + 64 + f) : 0.f);
      }
    }
  }
  if constexpr (KSPLIT > 1) cluster.sync(); else __syncthreads();   // the other CTAs' partial tiles stay alive until read
  if (*abort_flag) {
    if (threadIdx.x == 0) {
      if (status) atomicExch(status, 3);
      const int issued = *issued_ctr, consumed = *consumed_ctr;
      const uint64_t drain_start = global_ns();
      for (int g = consumed; g < issued; g++) {
        const int s = g % nstages;
        const uint32_t ph = (uint32_t)(g / nstages) & 1u;
        for (uint32_t w = 0; w < WAIT_LIMIT; ++w) {
          if (mbar_try_wait(&full_bar[s], ph)) break;
          if ((w & 255u) == 255u && global_ns() - drain_start > wait_ns) break;
        }
      }
    }
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(SU_BN < 32 ? 32 : SU_BN));
  }
}

// Shared memory of one CTA: ring, partial tile, barriers and bookkeeping, alignment slack.
template <int SU_BN>
size_t su_smem_bytes(int nstages) {
  return (size_t)nstages * (A_BYTES + SU_BN * BK * 2) + (size_t)SU_BN * BM * 4 + (2 * SU_MAXST + 1) * 8 + 64 + 1024;
}

template <int EPI, int KSPLIT, int SU_BN>
int launch_skinny_umma(const CUtensorMap& w, const CUtensorMap& w2, const CUtensorMap& x, int M, int N, int K,
                       const EpiArgs<bf16>& ep, int early, int* status, cudaStream_t st) {
  constexpr int NF = (EPI == EPI_GELU_MUL) ? 64 : 128;
  const int tiles = (N + NF - 1) / NF;
  // ring depth: deep (about 160 KB of weights in flight, one CTA per SM) for grids that leave a third of the SMs
  // empty anyway, else as deep as lets two CTAs share an SM
  bool deep = 3 * tiles * KSPLIT <= 2 * device_sm_count();
  if (const char* sv = getenv("STU_B200_UMMA_STAGES")) deep = atoi(sv) == 8;   // tuning aid
  const size_t two_per_sm = (233472 / 2) - 1024;   // per-SM shared memory, per-CTA reservation
  int nstages = deep ? (SU_BN == 16 ? 10 : (SU_BN == 32 ? 8 : 6)) : 2;
  if (!deep)
    while (nstages < SU_MAXST && su_smem_bytes<SU_BN>(nstages + 1) <= two_per_sm) nstages++;
  while (nstages > 2 && su_smem_bytes<SU_BN>(nstages) > 227 * 1024) nstages--;
  if (su_smem_bytes<SU_BN>(nstages) > 227 * 1024) return STU_ERR_UNSUPPORTED;
  if (!deep && nstages > 5) nstages = 5;
  const size_t smem = su_smem_bytes<SU_BN>(nstages);
  auto kern = skinny_umma_kernel<EPI, KSPLIT, SU_BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  if (KSPLIT > 8) {   // clusters of 16 CTAs are outside the portable range
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return (int)e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, KSPLIT);
  cfg.blockDim = dim3(192);
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
  cfg.numAttrs = 1;
  if (KSPLIT > 8) {   // can the GPU co-schedule a cluster of this size and footprint at all?  (the caller falls back)
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters < 1) {
      (void)cudaGetLastError();
      return STU_ERR_UNSUPPORTED;
    }
  }
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  e = cudaLaunchKernelEx(&cfg, kern, w, w2, x, M, N, K, ep, status, early, g_wait_ns, nstages);
  if (e != cudaSuccess) return (int)e;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

template <int EPI, int KSPLIT>
int launch_skinny_umma_bn(const CUtensorMap& w, const CUtensorMap& w2, const CUtensorMap& x, int M, int N, int K,
                          const EpiArgs<bf16>& ep, int early, int* status, cudaStream_t st) {
  if (M <= 16) return launch_skinny_umma<EPI, KSPLIT, 16>(w, w2, x, M, N, K, ep, early, status, st);
  if (M <= 32) return launch_skinny_umma<EPI, KSPLIT, 32>(w, w2, x, M, N, K, ep, early, status, st);
  return launch_skinny_umma<EPI, KSPLIT, 64>(w, w2, x, M, N, K, ep, early, status, st);
}

template <int EPI>
int launch_skinny_umma_split(int ks, const CUtensorMap& w, const CUtensorMap& w2, const CUtensorMap& x, int M, int N,
                             int K, const EpiArgs<bf16>& ep, int early, int* status,
                             cudaStream_t st) {
  switch (ks) {
    case 1: return launch_skinny_umma_bn<EPI, 1>(w, w2, x, M, N, K, ep, early, status, st);
    case 2: return launch_skinny_umma_bn<EPI, 2>(w, w2, x, M, N, K, ep, early, status, st);
    case 4: return launch_skinny_umma_bn<EPI, 4>(w, w2, x, M, N, K, ep, early, status, st);
    case 16: {
      const int rc = launch_skinny_umma_bn<EPI, 16>(w, w2, x, M, N, K, ep, early, status, st);
      if (rc != STU_ERR_UNSUPPORTED) return rc;   // no room for clusters of 16 on this GPU: clusters of 8
    }
      [[fallthrough]];
    default: return launch_skinny_umma_bn<EPI, 8>(w, w2, x, M, N, K, ep, early, status, st);
  }
}

}  // namespace

// Per-device state of the library: the status word the host wrapper registered for the device that was current at
// the time (a kernel must never be handed a word that lives on another GPU) and that device's SM count.
static int* g_status_words[STU_MAX_DEVICES] = {nullptr};
static int g_sm_counts[STU_MAX_DEVICES] = {0};

static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= STU_MAX_DEVICES) return 0;
  return dev;
}

int device_sm_count() {
  const int dev = current_device();
  int n = g_sm_counts[dev];
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_counts[dev] = n;
  }
  return n;
}

static int* device_status_word() { return g_status_words[current_device()]; }

// Test hook for the failure-detection path: the next tcgen05 GEMM launch of this process never issues the copies of
// its first pipeline stage, and every bounded wait gives up after wait_ms milliseconds (0 restores the default of
// two seconds without arming a fault).  The kernel then reports status 3, drains what it did issue, frees its tensor
// memory and returns; nothing faults and the context stays usable.
extern "C" int stu_test_inject_wait_expiry(int wait_ms) {
  if (wait_ms < 0 || wait_ms > 10000) return STU_ERR_SHAPE;
  if (wait_ms == 0) {
    g_drop_first_copy = 0;
    g_wait_ns = 2000000000ull;
  } else {
    g_drop_first_copy = 1;
    g_wait_ns = (unsigned long long)wait_ms * 1000000ull;
  }
  return STU_OK;
}

extern "C" int stu_set_status_word(int* device_status) {
  g_status_words[current_device()] = device_status;
  return STU_OK;
}

bool gemm_tc_supported(const void* A, long long lda, const void* B, long long ldb, long long skb, const void* B2,
                       int M, int N, int K, int epi, const EpiArgsAny& ep, int dtype) {
  if (dtype != STU_BF16 || skb != 1) return false;
  static const bool disabled = getenv("STU_B200_DISABLE_TCGEN05") != nullptr;  // debugging aid: CUDA-core GEMM instead
  if (disabled) return false;
  if (lda % 8 || ldb % 8 || K % 8 || !aligned16(A) || !aligned16(B) || (B2 && !aligned16(B2))) return false;
  if (M < 1 || N < 1 || K < 8) return false;
  if (epi == EPI_HIST) return aligned16(ep.y) && get_encode_fn() != nullptr;
  if (ep.ldy % 8 || !aligned16(ep.y)) return false;
  if (epi == EPI_BLOCKCOL && (ep.ld2 % 8 || ep.Tseq % 8 || ep.Tseq <= 0)) return false;
  if (epi == EPI_RESID && (ep.ldr % 8 || !aligned16(ep.resid))) return false;
  return get_encode_fn() != nullptr;
}

// 128 x 256 tiles when the output has at least two waves of them (rows x cols of the GEMM as the kernel sees it).
// STU_B200_TILE_N=128 forces the square tiles.
static bool wide_tiles(long long rows, long long cols) {
  static const char* env = getenv("STU_B200_TILE_N");
  if (env && atoi(env) == 128) return false;
  return cols >= 512 && ((rows + BM - 1) / BM) * ((cols + 255) / 256) >= 2 * 148;
}

int gemm_tc_dispatch(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N,
                     int K, int epi, int causal, const EpiArgsAny& epa, cudaStream_t st) {
  CUtensorMap ma, mb, mb2;
  EpiArgs<bf16> ep = epa.as<bf16>();
  int rc;
  if (epi == EPI_HIST) {
    // swap operands: rows = channels (the weight), columns = tokens, so that each epilogue thread owns
    // one channel row of the history and writes whole 16-byte runs per parity
    const bool wide = wide_tiles(N, M);
    if ((rc = make_map(&ma, B, N, K, ldb)) != STU_OK) return rc;
    if ((rc = make_map(&mb, A, M, K, lda, wide ? 256 : BM)) != STU_OK) return rc;
    ep.ldy = N;  // channel count
    if (wide) return launch_tc<EPI_HIST_T, 4, 256>(ma, mb, mb, N, M, K, /*m_fast=*/1, 0, ep, device_status_word(), st);
    return launch_tc<EPI_HIST_T, 6>(ma, mb, mb, N, M, K, /*m_fast=*/1, 0, ep, device_status_word(), st);
  }
  const bool wide = epi != EPI_GELU_MUL && wide_tiles(M, N);
  if ((rc = make_map(&ma, A, M, K, lda)) != STU_OK) return rc;
  if ((rc = make_map(&mb, B, N, K, ldb, wide ? 256 : BM)) != STU_OK) return rc;
  mb2 = mb;
  if (epi == EPI_GELU_MUL && (rc = make_map(&mb2, B2, N, K, ldb)) != STU_OK) return rc;
  if (wide) {
    switch (epi) {
      case EPI_STORE: return launch_tc<EPI_STORE, 4, 256>(ma, mb, mb2, M, N, K, 0, causal, ep, device_status_word(), st);
      case EPI_RESID: return launch_tc<EPI_RESID, 4, 256>(ma, mb, mb2, M, N, K, 0, causal, ep, device_status_word(), st);
      case EPI_BLOCKCOL:
        return launch_tc<EPI_BLOCKCOL, 4, 256>(ma, mb, mb2, M, N, K, 0, causal, ep, device_status_word(), st);
    }
  }
  switch (epi) {
    case EPI_STORE: return launch_tc<EPI_STORE, 6>(ma, mb, mb2, M, N, K, 0, causal, ep, device_status_word(), st);
    case EPI_RESID: return launch_tc<EPI_RESID, 6>(ma, mb, mb2, M, N, K, 0, causal, ep, device_status_word(), st);
    case EPI_GELU_MUL: return launch_tc<EPI_GELU_MUL, 4>(ma, mb, mb2, M, N, K, 0, 0, ep, device_status_word(), st);
    case EPI_BLOCKCOL: return launch_tc<EPI_BLOCKCOL, 6>(ma, mb, mb2, M, N, K, 0, causal, ep, device_status_word(), st);
  }
  return STU_ERR_UNSUPPORTED;
}

// Token-step linears of 9..64 rows on the tensor cores with swapped operands (skinny_umma_kernel).
// STU_B200_DISABLE_UMMA_SKINNY=1 keeps them on the mma.sync weight-streaming kernels.
bool skinny_umma_takes(int M, int N, int K, int epi, bool norm, bool peer) {
  static const bool off = getenv("STU_B200_DISABLE_UMMA_SKINNY") != nullptr;
  if (off || peer || norm) return false;
  if (epi != EPI_STORE && epi != EPI_RESID && epi != EPI_GELU_MUL) return false;
  // up to 8 rows the 8-feature mma.sync kernel is faster (8 x 4096 x 1024 gate/up 6.0 against 6.3 us, down 4.5 against
  // 5.8 us); from 9 rows on this kernel is (16 rows: gate/up 6144 x 1536 14.2 -> 10.1 us, down 12.6 -> 7.9 us)
  static const int min_rows = getenv("STU_B200_UMMA_MIN_ROWS") ? atoi(getenv("STU_B200_UMMA_MIN_ROWS")) : 9;   // tuning aid
  return M >= min_rows && M <= 64 && K % 8 == 0 && K >= 128 && N >= 64;
}

int skinny_umma_dispatch(const void* A, long long lda, const void* B, long long ldb, const void* B2, int M, int N,
                         int K, int epi, const EpiArgs<bf16>& ep, int pdl, cudaStream_t st) {
  const bool dual = epi == EPI_GELU_MUL;
  CUtensorMap mw, mw2, mx;
  int rc = make_map(&mw, B, N, K, ldb, dual ? 64 : 128);
  if (rc != STU_OK) return rc;
  rc = make_map(&mw2, dual ? B2 : B, N, K, ldb, dual ? 64 : 128);
  if (rc != STU_OK) return rc;
  rc = make_map(&mx, A, M, K, lda, M <= 16 ? 16 : (M <= 32 ? 32 : 64));
  if (rc != STU_OK) return rc;
  // split K over a cluster until there is about one CTA per SM, every CTA keeping at least two 64-element blocks
  // (six for the step from 8 to 16 CTAs per cluster: down 1536 x 6144 at 32 rows 8.4 -> 7.8 us, the 16 x 1024 x 49152
  // contraction of the distilled-LDS features 31.9 -> 21.8 us, but c_proj 1536 x 1536 5.2 -> 5.6 us)
  const int tiles = (N + (dual ? 64 : 128) - 1) / (dual ? 64 : 128), num_kb = (K + BK - 1) / BK;
  const int sms = device_sm_count();
  int ks = 1;
  while (ks < 16 && tiles * ks < sms - sms / 8 && num_kb / (2 * ks) >= (ks >= 8 ? 6 : 2)) ks *= 2;
  if (const char* kv = getenv("STU_B200_UMMA_KS")) ks = atoi(kv);   // tuning aid
  const int early = (pdl & STU_FLAG_OVERLAP) ? 1 : 0;
  int* status = device_status_word();
  switch (epi) {
    case EPI_STORE: return launch_skinny_umma_split<EPI_STORE>(ks, mw, mw2, mx, M, N, K, ep, early, status, st);
    case EPI_RESID: return launch_skinny_umma_split<EPI_RESID>(ks, mw, mw2, mx, M, N, K, ep, early, status, st);
    case EPI_GELU_MUL:
      return launch_skinny_umma_split<EPI_GELU_MUL>(ks, mw, mw2, mx, M, N, K, ep, early, status, st);
  }
  return STU_ERR_UNSUPPORTED;
}
