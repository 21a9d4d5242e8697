// Prefill convolution of the approx STU variant on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory, the history brought in by cp.async.bulk.tensor).
//
// Reference semantics (flash_stu/modules/stu.py:85-98,120 + flash_stu/utils/stu_utils.py:208-228): per channel c the
// folded even-tap convolution of the 2B parity rows of the projected history,
//   Y[m][n] = sum_{s<=m} g_c[m-s] * H[n][s],          n = (sequence, parity), m, s = position inside the parity,
// is a lower-triangular Toeplitz product with only 2B columns.  A 128-wide instruction over 16 columns would leave
// the tensor pipe at a sixth of its rate, so the product is regrouped by the block distance delta = mb - sb between
// the 128-position output block mb and input block sb: every (mb, sb) pair with the same delta multiplies by the
// SAME 128 x 128 Toeplitz block T_delta[i][j] = g[128 delta + i - j], so the pairs are stacked along the instruction's
// N dimension:
//   D[i][(mb, n)] += T_delta[i][:] . H[n][128 (mb - delta) + :]        for all mb >= delta at once.
// With the history of one channel resident in shared memory as rows (sb, n), the B operand of shift delta is that
// array itself read from row 0, and the accumulator columns start at 16 delta: one instruction stream per delta, N up
// to 256.
//
// No Toeplitz block is ever materialised.  In the un-swizzled K-major operand layout a tile is a grid of 8 x 8
// "core matrices" of 128 contiguous bytes, addressed as start + (row group) * SBO + (column group) * LBO.  With the
// row groups of a block taken in descending order (row group q' holds outputs 120 - 8 q' .. 127 - 8 q'), core matrix
// (q', kc) of T_delta holds g[128 delta + 120 - 8 (q' + kc) + r - w] and so depends on V = q' + kc - 16 delta alone.
// One table CM[V][r][w] = g[120 - 8 V + r - w] (34 KB for 16 block distances, zeros where the tap index is
// negative: the causal part of the diagonal block included) therefore serves EVERY block distance through the operand
// descriptor alone: start = &CM[2 kk - 16 delta], SBO = LBO = 128 bytes.  Four generator warps fill the table from
// the reversed tap table (stu_taps_rev8: its eight alignments make every 16-byte row an aligned load).
//
// The accumulator of one unit (a channel, 16 parity rows, a superblock of 16 output blocks = 2048 positions) is 256
// columns of tensor memory; the two halves of tensor memory alternate between units, so one unit's epilogue runs
// under the next unit's MMAs.  A unit runs one phase per (history chunk of 16 blocks, sign of the block distance);
// a phase's operands - the 64 KB chunk and the 34 KB table of its block distances - form one of two shared-memory
// stages, filled a phase ahead of the MMAs.
//
// Roles (one persistent CTA per SM, 320 threads):
//   warp 0      producer: history chunks (2 x 32 KB tensor copies, 128-byte swizzle)
//   warp 1      allocates tensor memory, issues the MMAs from one thread, commits to the barriers
//   warps 2-5   epilogue: tcgen05.ld the accumulator, round 2*acc to bf16, turn 32 x 32 pieces round through a
//               staging tile and store 64-byte runs to yT (history layout)
//   warps 6-9   generators: the core-matrix table (asynchronous 16-byte copies); zero the history tail past each
//               row's valid count
// Every load is a plain single-CTA copy of this GPU's own memory.  Every wait is bounded: on expiry the CTA raises
// status 9, lets issued copies land (bounded), frees its tensor memory and returns.
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "tma.cuh"

int device_sm_count();
int launch_transpose_add(void* x, long long x_bstride, long long x_tstride, const void* yT, int B, int d, int y_Lh,
                         int t0, int t_end, int dtype, cudaStream_t st);

namespace {

constexpr int SUP = 16;                       // 128-position blocks per unit (256 accumulator columns / 16 rows)
constexpr int PLANE_BYTES = SUP * 16 * 128;   // 16 blocks x 16 rows x 64 positions
constexpr int HIST_BYTES = 2 * PLANE_BYTES;
constexpr int TAB_ENTRIES = 16 * SUP + 15;
constexpr int TAB_BYTES = (TAB_ENTRIES * 128 + 1023) / 1024 * 1024;
constexpr int STAGE_BYTES = HIST_BYTES + TAB_BYTES;
constexpr int STG_OFF = 2 * STAGE_BYTES;      // epilogue staging: 4 warps x 32 rows x 80 bytes
constexpr int STG_BYTES = 4 * 32 * 80;
constexpr int CTL_OFF = STG_OFF + STG_BYTES;
constexpr int SMEM_BYTES = CTL_OFF + 256 + 1024;
constexpr int ACC_COLS = 16 * SUP;
constexpr int STATUS_CONV_WAIT = 9;

struct Ctl {
  uint64_t hist_full[2], ready[2], stage_empty[2], tmem_full[2], tmem_empty[2];
  uint32_t tmem_slot;
  int abort_flag, issued_h, consumed_h;
};
static_assert(sizeof(Ctl) <= 256, "control block");

struct Geom {
  int B, d, Lh, y_Lh, t0, t_end;
  int nrg;        // groups of 8 sequences (16 parity rows)
  int nb_total;   // 128-position blocks that hold outputs
  int msb_first;  // first superblock with outputs of this call
  int n_sup;      // superblocks processed
};

__device__ __forceinline__ int parity_count(int t_end, int p) { return (t_end - p + 1) >> 1; }

// A unit (channel, row group, superblock msb of 16 output blocks) runs 2 msb + 1 phases.  Phase ph < 2 msb works on
// history chunk ssb = ph / 2 (16 input blocks) and covers the block distances dl = mb - sb (local to the two
// superblocks) 0 .. nb_m-1 (even ph) or -15 .. -1 (odd ph); the last phase is the chunk on the diagonal, dl >= 0
// only.  The first phase of a unit starts with dl = 0, which touches every accumulator column, so its first
// instruction overwrites instead of accumulating.
struct Phase {
  int ssb, dl_lo, ndl;
};
__device__ __forceinline__ Phase phase_of(int ph, int msb, int nb_m) {
  Phase p;
  if (ph == 2 * msb) {
    p.ssb = msb; p.dl_lo = 0; p.ndl = nb_m;
  } else {
    p.ssb = ph >> 1;
    p.dl_lo = (ph & 1) ? -(SUP - 1) : 0;
    p.ndl = (ph & 1) ? (SUP - 1) : nb_m;
  }
  return p;
}

// operand descriptors: B = history rows, K-major with the 128-byte swizzle of the tensor copies; A = core-matrix
// table, K-major without swizzle, 128 bytes between core matrices in either direction
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;            // leading byte offset: unused for swizzled K-major operands
  d |= (uint64_t)(1024 >> 4) << 32;  // 8-row groups are 1024 bytes apart
  d |= (uint64_t)1 << 46;            // descriptor version of this architecture
  d |= (uint64_t)2 << 61;            // 128-byte swizzle
  return d;
}
__device__ __forceinline__ uint64_t make_desc_table(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)(128 >> 4) << 16;   // next core matrix along K
  d |= (uint64_t)(128 >> 4) << 32;   // next core matrix along M
  d |= (uint64_t)1 << 46;
  return d;                          // layout field 0: no swizzle
}
__device__ __forceinline__ uint32_t idesc_n(int n) {   // D fp32, A/B bf16 K-major, M = 128, N = n
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tma::smem_u32(bar))
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
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// A CTA walks channel tasks (channel, row group) blockIdx.x, blockIdx.x + gridDim.x, ...; inside a task the
// superblocks run from the one with the most history down, so that the chunks they share are still in L2.
#define FOR_EACH_UNIT(task, msb, c, rg)                                     \
  for (int task = blockIdx.x; task < g.d * g.nrg; task += gridDim.x)        \
    for (int msb = g.msb_first + g.n_sup - 1, c = task / g.nrg, rg = task % g.nrg; msb >= g.msb_first; msb--)

#define TL_STAMP(ucnt, slot) \
  do { if (tl && blockIdx.x == 0 && (ucnt) < 8) tl[(ucnt) * 16 + (slot)] = tma::global_ns(); } while (0)

__global__ void __launch_bounds__(320, 1) conv_umma_kernel(const __grid_constant__ CUtensorMap tmH,
                                                           const bf16* __restrict__ taps8, bf16* __restrict__ yT,
                                                           Geom g, int* status, unsigned long long wait_ns,
                                                           unsigned long long* tl) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + CTL_OFF);
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; s++) {
      tma::mbar_init(&ctl->hist_full[s], 1);
      tma::mbar_init(&ctl->ready[s], 128);
      tma::mbar_init(&ctl->stage_empty[s], 1);
      tma::mbar_init(&ctl->tmem_full[s], 1);
      tma::mbar_init(&ctl->tmem_empty[s], 128);
    }
    ctl->abort_flag = 0;
    ctl->issued_h = ctl->consumed_h = 0;
    tma::fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(tma::smem_u32(&ctl->tmem_slot)));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = ctl->tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ producer: the history chunk of each phase
      int pc = 0;
      bool ok = true;
      FOR_EACH_UNIT(task, msb, c, rg) {
        if (!ok) break;
        for (int ph = 0; ph <= 2 * msb; ph++, pc++) {
          const int ssb = (ph == 2 * msb) ? msb : (ph >> 1);
          const int s = pc & 1;
          if (!tma::mbar_wait_bounded(&ctl->stage_empty[s], ((uint32_t)(pc >> 1) & 1u) ^ 1u, abort_flag, wait_ns)) { ok = false; break; }
          unsigned char* dst = smem + s * STAGE_BYTES;
          tma::mbar_expect_tx(&ctl->hist_full[s], HIST_BYTES);
          tma::load_5d(dst, &tmH, &ctl->hist_full[s], 0, 0, 8 * rg, SUP * ssb, c);
          tma::load_5d(dst + PLANE_BYTES, &tmH, &ctl->hist_full[s], 64, 0, 8 * rg, SUP * ssb, c);
          ctl->issued_h = pc + 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      int pc = 0, uc = 0;
      bool ok = true;
      FOR_EACH_UNIT(task, msb, c, rg) {
        if (!ok) break;
        (void)c; (void)rg;
        const int nb_m = min(SUP, g.nb_total - SUP * msb);
        const int buf = uc & 1;
        if (!tma::mbar_wait_bounded(&ctl->tmem_empty[buf], ((uint32_t)(uc >> 1) & 1u) ^ 1u, abort_flag, wait_ns)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        TL_STAMP(uc, 0);
        for (int ph = 0; ph <= 2 * msb; ph++, pc++) {
          const Phase P = phase_of(ph, msb, nb_m);
          const int s = pc & 1;
          if (!tma::mbar_wait_bounded(&ctl->ready[s], (uint32_t)(pc >> 1) & 1u, abort_flag, wait_ns)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (ph == 0) TL_STAMP(uc, 1);
          const uint32_t hist_s = tma::smem_u32(smem + s * STAGE_BYTES), tab_s = hist_s + HIST_BYTES;
          for (int st = 0; st < P.ndl; st++) {
            const int dl = P.dl_lo + st;
            const int mb_lo = max(0, dl), mb_hi = min(nb_m, SUP + dl);
            if (mb_hi <= mb_lo) continue;
            const uint32_t dcol = tmem_base + (uint32_t)(buf * ACC_COLS + 16 * mb_lo);
            const uint32_t idesc = idesc_n(16 * (mb_hi - mb_lo));
            // table entry of core matrix (q' = 0, kc = 0) of this distance: the table starts at the largest distance
            const uint64_t da0 = make_desc_table(tab_s + 16 * (P.ndl - 1 - st) * 128);
            const uint64_t db0 = make_desc_sw128(hist_s + (mb_lo - dl) * 2048);
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
              const uint32_t acc = (ph == 0 && st == 0 && kk == 0) ? 0u : 1u;
              umma(dcol, da0 + (uint64_t)(2 * kk * 128 >> 4),
                   db0 + (uint64_t)(((kk >> 2) * PLANE_BYTES + (kk & 3) * 32) >> 4), idesc, acc);
            }
          }
          umma_commit(&ctl->stage_empty[s]);
          ctl->consumed_h = pc + 1;
        }
        if (!ok) break;
        TL_STAMP(uc, 2);
        umma_commit(&ctl->tmem_full[buf]);
        uc++;
      }
    }
  } else if (warp < 6) {
    // -------------------------------------------------------------------- epilogue (TMEM lane quarter = warp % 4)
    // A lane holds one output position of 32 columns (two blocks x 16 parity rows).  Each 32 x 32 piece is turned
    // round through a staging tile of the warp, so that four lanes then write the 64 bytes (32 positions) of one
    // parity row.
    const int quarter = warp & 3;
    const int pos = 24 - 8 * (lane >> 3) + (lane & 7);   // rank of this lane's position among the warp's 32
    const int i_min = 96 - 32 * quarter;                 // first position (inside a block) of the warp's 32
    unsigned char* stg = smem + STG_OFF + (warp - 2) * (32 * 80);
    const int cnt0 = parity_count(g.t_end, 0), cnt1 = parity_count(g.t_end, 1);
    const int lo0 = parity_count(g.t0, 0), lo1 = parity_count(g.t0, 1);
    int uc = 0;
    bool ok = true;
    FOR_EACH_UNIT(task, msb, c, rg) {
      if (!ok) break;
      const int nb_m = min(SUP, g.nb_total - SUP * msb);
      const int buf = uc & 1;
      ok = tma::mbar_wait_bounded(&ctl->tmem_full[buf], (uint32_t)(uc >> 1) & 1u, abort_flag, wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (threadIdx.x == 64) TL_STAMP(uc, 3);
#pragma unroll 1
      for (int cch = 0; cch < ((nb_m + 1) >> 1); cch++) {   // 32 columns = two blocks
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * ACC_COLS + cch * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; j++)
          *reinterpret_cast<bf16*>(stg + j * 80 + pos * 2) = __float2bfloat16_rn(2.f * __uint_as_float(r[j]));
        __syncwarp();
        // four lanes write the 64 bytes of one column (one parity row, 32 positions), eight columns per store
#pragma unroll
        for (int v = 0; v < 4; v++) {
          const int col = 8 * v + (lane >> 2), q4 = lane & 3;
          const int mbl = 2 * cch + (col >> 4), n = col & 15, p = n & 1;
          const int b = 8 * rg + (n >> 1);
          const int m = (SUP * msb + mbl) * 128 + i_min + 8 * q4;
          const int lo = p ? lo1 : lo0, hi = p ? cnt1 : cnt0;
          if (mbl < nb_m && b < g.B) {
            const uint4 val = *reinterpret_cast<const uint4*>(stg + col * 80 + q4 * 16);
            bf16* dst = yT + ((size_t)((size_t)b * g.d + c) * 2 + p) * g.y_Lh + m;
            if (m >= lo && m + 8 <= hi) {
              *reinterpret_cast<uint4*>(dst) = val;
            } else if (m + 8 > lo && m < hi) {
              const unsigned short* e = reinterpret_cast<const unsigned short*>(&val);
#pragma unroll
              for (int w = 0; w < 8; w++)
                if (m + w >= lo && m + w < hi) reinterpret_cast<unsigned short*>(dst)[w] = e[w];
            }
          }
        }
        __syncwarp();
      }
      if (threadIdx.x == 64) TL_STAMP(uc, 4);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      tma::mbar_arrive(&ctl->tmem_empty[buf]);
      uc++;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  } else {
    // -------------------------------------------------------------------- generators
    const int gt = threadIdx.x - 192;
    const int cnt0 = parity_count(g.t_end, 0), cnt1 = parity_count(g.t_end, 1);
    const size_t pitch = (size_t)g.Lh + 8;
    int pc = 0;
    bool ok = true;
    FOR_EACH_UNIT(task, msb, c, rg) {
      if (!ok) break;
      (void)rg;
      const int nb_m = min(SUP, g.nb_total - SUP * msb);
      for (int ph = 0; ph <= 2 * msb; ph++, pc++) {
        const Phase P = phase_of(ph, msb, nb_m);
        const int s = pc & 1;
        unsigned char* stage = smem + s * STAGE_BYTES;
        ok = tma::mbar_wait_bounded(&ctl->stage_empty[s], ((uint32_t)(pc >> 1) & 1u) ^ 1u, abort_flag, wait_ns);
        if (!ok) break;
        if (gt == 0) TL_STAMP(pc, 5);
        // ---- core-matrix table of this phase: entry e <-> V = v_lo + e, row r: CM[V][r][w] = g[120 - 8 V + r - w];
        //      every row is an asynchronous 16-byte copy global -> shared, all in flight at once
        {
          const int d_hi = SUP * (msb - P.ssb) + P.dl_lo + P.ndl - 1;   // largest block distance of the phase
          const int v_lo = -16 * d_hi, rows = (16 * P.ndl + 15) * 8;
          for (int it = gt; it < rows; it += 128) {
            const int r = it & 7, V = v_lo + (it >> 3);
            const int uo = g.Lh - 128 + 8 * V;   // start inside row 7 - r of the reversed table (multiple of 8)
            // V >= 16: every tap index of the row is negative (above the diagonal).  A row that straddles tap 0 runs
            // into the table's own zero padding; one that would start before the table only has taps past the filter.
            if (V < 16 && uo >= 0)
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(tma::smem_u32(stage + HIST_BYTES + it * 16)),
                           "l"(taps8 + ((size_t)(7 - r) * g.d + c) * pitch + uo) : "memory");
            else
              *reinterpret_cast<uint4*>(stage + HIST_BYTES + it * 16) = make_uint4(0, 0, 0, 0);
          }
          asm volatile("cp.async.commit_group;" ::: "memory");
        }
        // ---- the history chunk: zero what lies past each row's valid count (stale cache contents must not meet the
        //      zero part of a Toeplitz block as 0 x NaN)
        ok = tma::mbar_wait_bounded(&ctl->hist_full[s], (uint32_t)(pc >> 1) & 1u, abort_flag, wait_ns);
        if (!ok) break;
        if (gt == 0) TL_STAMP(pc, 6);
        {
          const int base = SUP * 128 * P.ssb;
          const int lim = min(g.nb_total * 128, base + SUP * 128);
          if (lim > cnt1) {
            for (int el = gt; el < 16 * 129; el += 128) {
              const int n = el / 129, off = el % 129, p = n & 1;
              const int sx = max(p ? cnt1 : cnt0, base) + off;
              if (sx < lim) {
                const int sl = sx - base, rr = (sl >> 7) * 16 + n, kq = sl & 127, k = kq & 63;
                unsigned char* ptr = stage + (kq >> 6) * PLANE_BYTES + (rr >> 3) * 1024 + (rr & 7) * 128 +
                                     (((k >> 3) ^ (rr & 7)) << 4) + (k & 7) * 2;
                *reinterpret_cast<unsigned short*>(ptr) = 0;
              }
            }
          }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        fence_proxy_async();
        if (gt == 0) TL_STAMP(pc, 7);
        tma::mbar_arrive(&ctl->ready[s]);
      }
    }
  }
  __syncthreads();
  if (*abort_flag) {
    // A wait ran out.  Report it and let the copies that were issued but never consumed land before the shared
    // memory is released (bounded).
    if (threadIdx.x == 0) {
      if (status) atomicExch(status, STATUS_CONV_WAIT);
      const uint64_t t_start = tma::global_ns();
      for (int pc = ctl->consumed_h; pc < ctl->issued_h; pc++)
        for (uint32_t w = 0; w < (1u << 22); ++w) {
          if (tma::mbar_try_wait(&ctl->hist_full[pc & 1], (uint32_t)(pc >> 1) & 1u)) break;
          if ((w & 255u) == 255u && tma::global_ns() - t_start > wait_ns) break;
        }
    }
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base));
  }
}

}  // namespace

// Profiling aid: while a device buffer of 128 64-bit words is registered, CTA 0 of every launch writes nanosecond
// stamps (%globaltimer) of its first 8 units / phases into it, 16 words each: 0 accumulator free, 1 first operands
// ready, 2 last MMA issued, 3 accumulator complete, 4 epilogue done (indexed by unit); 5 stage free, 6 history chunk
// landed, 7 stage ready (indexed by phase).  NULL switches it off.
static unsigned long long* g_timeline = nullptr;
extern "C" int stu_conv_prefill_set_timeline(void* device_words) {
  g_timeline = (unsigned long long*)device_words;
  return STU_OK;
}

extern "C" int stu_conv_prefill_approx_tc5(const void* hist, const void* taps8, void* yT, void* x, long long x_bstride,
                                           long long x_tstride, int B, int d, int Lh, int y_Lh, int t0, int t_end,
                                           int* status, int dtype, void* stream) {
  if (!hist || !taps8 || !yT || !x) return STU_ERR_NULL;
  if (B <= 0 || d <= 0 || Lh <= 0 || t0 < 0 || t_end <= t0 || t_end > 2 * Lh || t_end > 2 * y_Lh) return STU_ERR_SHAPE;
  if (dtype != STU_BF16) return STU_ERR_DTYPE;
  if (!aligned16(yT) || y_Lh % 8 || !aligned16(hist) || !aligned16(taps8)) return STU_ERR_ALIGN;
  if (Lh % 128) return STU_ERR_UNSUPPORTED;   // the history is tiled in 128-position blocks

  Geom g;
  g.B = B; g.d = d; g.Lh = Lh; g.y_Lh = y_Lh; g.t0 = t0; g.t_end = t_end;
  g.nrg = (B + 7) / 8;
  const int cnt_max = (t_end + 1) >> 1, mlo_min = t0 >> 1;   // parity 0 has the most inputs, parity 1 the first output
  g.nb_total = (cnt_max + 127) / 128;
  g.msb_first = mlo_min / (SUP * 128);
  g.n_sup = (g.nb_total + SUP - 1) / SUP - g.msb_first;
  if (g.n_sup <= 0) return STU_ERR_SHAPE;

  CUtensorMap tmH;
  {
    // history [B][d][2][Lh] seen as (position inside a 128-block, parity, sequence, block, channel)
    cuuint64_t dims[5] = {128, 2, (cuuint64_t)B, (cuuint64_t)(Lh / 128), (cuuint64_t)d};
    cuuint64_t str[4] = {(cuuint64_t)Lh * 2, (cuuint64_t)d * 2 * Lh * 2, 256, (cuuint64_t)2 * Lh * 2};
    cuuint32_t box[5] = {64, 2, 8, SUP, 1};
    int rc = tma::encode_bf16(&tmH, hist, 5, dims, str, box, true);
    if (rc != STU_OK) return rc;
  }
  cudaError_t e = cudaFuncSetAttribute(conv_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return (int)e;
  cudaStream_t st = (cudaStream_t)stream;
  const int units = d * g.nrg;   // channel tasks; each runs its superblocks
  const int sms = device_sm_count();
  conv_umma_kernel<<<units < sms ? units : sms, 320, SMEM_BYTES, st>>>(tmH, (const bf16*)taps8, (bf16*)yT, g,
                                                                      status, 2000000000ull,
                                                                      g_timeline);
  STU_CHECK_LAUNCH();
  return launch_transpose_add(x, x_bstride, x_tstride, yT, B, d, y_Lh, t0, t_end, dtype, st);
}
