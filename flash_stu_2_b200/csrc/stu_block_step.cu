// One cached token step of a whole approx STU layer -- x += STU(norm(x)); x += MLP(norm(x)) for one new position of
// up to 8 sequences that stand at one common position -- as ONE persistent kernel (bf16, d <= 1024, I <= 4096).
// Reference semantics: flash_stu/layers/stu_layer.py:78-97 with flash_stu/modules/stu.py:85-98,120 and
// flash_stu/modules/swiglu.py:22-29 evaluated for the new position only (the reference keeps no STU cache).
//
// Launched kernel by kernel, a token step is a chain: history stream -> projection/combine -> gate|up -> down, and the
// stream (three quarters of the bytes) cannot overlap the MLP of the same step because the MLP needs every output
// channel of the STU.  The stream of the NEXT position, however, needs nothing this step produces: position t+1 reads
// the other time parity of the projected history, all of it written at steps <= t-1.  So this kernel pipelines across
// launches.  At position t, one CTA per SM runs four groups of warps side by side:
//   * producer (1 warp) + streaming consumers (8 warps): the partial sums sum_{i<s'} hist[.][i] tap[s'-i] of position
//     t+1, exactly as in stu_decode_pipe_kernel (units of 8 sequences x 8 channels x 256 positions through a 3-stage
//     bulk-copy ring, diagonal-of-an-MMA dot products), written to a workspace buffer for the next launch;
//   * compute group (8 warps): phase 1, RMS statistics and projection of the new token for the CTA's row, history
//     append, combine with the partial sums the PREVIOUS launch left for position t, write the STU sub-layer output
//     `mid` (every operand of the phase is requested before the first is used: one memory round trip); after a
//     grid-wide barrier (all rows of `mid` written) phase 2, the gate|up products of this CTA's share of the hidden
//     features (units of 8 features, K split over the warps, MMAs with the sequences as rows, tanh-GELU * up); after a
//     second grid-wide barrier phase 3, its 8 output channels of the down projection plus residual;
//   * MLP weight producer (1 warp): the CTA's gate|up and down weight rows as bulk copies of whole rows
//     (cp.async.bulk, 2 KB / 8 KB each) into a 96 KB shared-memory region, started at kernel entry, so that the
//     compute group never waits for a weight from HBM and the weights arrive as long contiguous bursts.
// The step then costs max(stream of 74 MB + 25 MB of MLP weights at HBM speed, the latency chain of the other three
// groups) instead of their sum.  A first step after a prefill has no partial sums waiting: mode 1 of the same kernel
// streams the CURRENT position into the workspace (nothing else), then the normal launch follows.
//
// Grid-wide barriers are monotonic arrival counters in the workspace; the launch is cooperative (all CTAs resident).
// Every wait (mbarrier or grid barrier) is bounded: on expiry the CTA raises status 7, stops, lets its outstanding
// copies land (bounded) and returns; the other CTAs' waits then run out the same way.
#include "common.cuh"
#include "tma.cuh"

int device_sm_count();  // gemm_tc.cu

namespace {

constexpr int SEG = 256;
constexpr int STAGES = 3;
constexpr int HIST_BYTES = 64 * SEG * 2;
constexpr int TAP_BYTES = 8 * SEG * 2;
constexpr int STAGE_BYTES = HIST_BYTES + TAP_BYTES;
constexpr int MLP_SLOT = 32 * 1024;      // one gate|up unit: 8 gate rows + 8 up rows of d <= 1024 values
constexpr int MLP_SLOTS = 3;
constexpr int MLP_BYTES = MLP_SLOTS * MLP_SLOT;   // shared-memory region the MLP weights pass through
constexpr int W_PROD = 8, W_WPROD = 9, W_COMP = 10;
constexpr int NTHREADS = 18 * 32;        // 8 streaming warps, 2 producer warps, 8 compute warps

__device__ __forceinline__ void comp_bar() { asm volatile("bar.sync 2, 256;" ::: "memory"); }

__device__ __forceinline__ uint4 lds128(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(tma::smem_u32(p)));
  return v;
}
// L2 loads of data another CTA of this launch wrote (L1 is not coherent across SMs)
__device__ __forceinline__ uint4 ldcg128(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_stream128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ int ld_relaxed(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_rows8(float (&c)[4], const uint4& a, const uint4& b) {
  mma16816(c, a.x, 0u, a.y, 0u, b.x, b.y);
  mma16816(c, a.z, 0u, a.w, 0u, b.z, b.w);
}
__device__ __forceinline__ uint4 keep_first(const uint4& v, int keep) {
  uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; j++)
    if (2 * j + 1 >= keep) w[j] = (2 * j < keep) ? (w[j] & 0x0000ffffu) : 0u;
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Grid barrier: a monotonic arrival counter in global memory.  Every CTA reads the launch epoch before it arrives
// anywhere; the barrier of launch e is passed once the counter has reached (e + 1) * G (compared as a wrapping
// difference).  The epoch is advanced once per launch by the CTA that advances the positions.
__device__ __forceinline__ void grid_arrive(int* counter) {
  __threadfence();
  atomicAdd(counter, 1);
}
__device__ __forceinline__ bool grid_wait(const int* counter, int target, volatile int* abort_flag) {
  uint64_t start = 0;
  for (uint32_t it = 0; it < (1u << 24); ++it) {
    if (ld_acquire(counter) - target >= 0) return true;
    if ((it & 63u) == 63u) {
      if (*abort_flag) return false;
      const uint64_t now = tma::global_ns();
      if (start == 0) start = now;
      else if (now - start > 2000000000ull) break;
    }
  }
  *abort_flag = 1;
  return false;
}

struct StepParams {
  const bf16* x;            // [B][d] layer input (residual stream); may alias out
  long long x_rstride;
  const bf16* stu_norm_w;
  const bf16* MinT;         // [d][d] rows = output channels
  bf16* hist;               // [B][d][2][Lh]
  const bf16* taps8;        // [8][d][Lh+8]
  int* pos;                 // [B][2]
  const bf16* mlp_norm_w;
  const bf16* Wg;           // [I][d]
  const bf16* Wu;           // [I][d]
  const bf16* Wd;           // [d][I]
  bf16* out;                // [B][d]
  long long out_rstride;
  int B, d, I, Lh;
  float eps_stu, eps_mlp;
  float* part;              // [2][rows][64] partial sums of position (index & 1)
  int* ws_pos;              // [2] the position each partial-sum buffer holds
  int* bar;                 // [3] launch epoch, arrival counters of the two grid barriers
  bf16* mid;                // [8][d]  STU sub-layer output of this step
  bf16* hbuf;               // [8][I]  MLP hidden activations of this step
  int* status;
  int mode;                 // 0: token step; 1: only stream the partial sums of the CURRENT position
  unsigned long long* tl;   // optional timeline of CTA 0 (16 globaltimer stamps in the workspace), else null
};

// timeline slots: 0 start, 1 positions read, 2 projection group done, 3 MLP group past barrier 1, 4 gate|up done,
// 5 MLP group past barrier 2, 6 down projection done, 7 stream done (consumer warp 0), 8 end of CTA
__device__ __forceinline__ void stamp(const StepParams& P, int slot) {
  if (P.tl && blockIdx.x == 0) P.tl[slot] = tma::global_ns();
}

__global__ void __launch_bounds__(NTHREADS, 1)
    stu_block_step_kernel(const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmT,
                          const StepParams P) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* wsm = smem + STAGES * STAGE_BYTES;                         // MLP weight region (MLP_BYTES)
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(wsm + MLP_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* wfull = empty_bar + STAGES;     // [3] a gate|up unit has landed in its slot
  uint64_t* wempty = wfull + MLP_SLOTS;     // [3] the compute group has finished with the slot
  uint64_t* dfull = wempty + MLP_SLOTS;     // [1] the down-projection unit has landed (slots 1 and 2)
  uint64_t* go_bar = dfull + 1;             // [1] the compute group's phase-1 operands have landed: start the stream
  __shared__ int s_abort, s_issued, s_ok;
  __shared__ float s_r[8];
  __shared__ float s_red[8][2][64];
  volatile int* abort_flag = &s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q = lane & 3;
  const int G = gridDim.x, cta = blockIdx.x;
  const int B = P.B, d = P.d, I = P.I, Lh = P.Lh;
  const int LP = Lh + 8;
  const int rows = d >> 3;   // B <= 8: one group of sequences
  const int nGu = (I >> 3) > cta ? ((I >> 3) - cta + G - 1) / G : 0;   // gate|up units of this CTA: cta, cta+G, ...
  const bool hasD = cta < (d >> 3);                                    // down-projection unit of this CTA

  if (tid == 0) {
    stamp(P, 0);
    for (int i = 0; i < STAGES; i++) {
      tma::mbar_init(&full_bar[i], 1);
      tma::mbar_init(&empty_bar[i], 8);
    }
    for (int i = 0; i < MLP_SLOTS; i++) {
      tma::mbar_init(&wfull[i], 1);
      tma::mbar_init(&wempty[i], 1);
    }
    tma::mbar_init(dfull, 1);
    tma::mbar_init(go_bar, 1);
    s_abort = 0;
    s_issued = 0;
    s_ok = 1;
    tma::fence_barrier_init();
  }
  // launch epoch, read before this CTA arrives at the position counter (whose last arrival advances it)
  const int epoch = ld_relaxed(&P.bar[0]);
  const int target = (epoch + 1) * (int)gridDim.x;
  const int t = P.pos[0];
  int bad = (t < 0 || t >= 2 * Lh) ? 1 : 0;
  for (int b = tid; b < B; b += NTHREADS)
    if (P.pos[2 * b] != t) bad = 2;
  if (P.mode == 0 && !bad && P.ws_pos[t & 1] != t) bad = 3;   // no partial sums waiting for this position
  bad = __syncthreads_or(bad);
  if (tid == 0) stamp(P, 1);
  // stream target: the next position (token step) or the current one (cold start)
  const int ts = t + (P.mode == 0 ? 1 : 0);
  if (warp == 0) {   // arrival counter of the grid: the last CTA to have read the positions advances them
    int last = 0;
    if (lane == 0) last = (atomicAdd(&P.pos[1], 1) == G - 1) ? 1 : 0;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      if (!bad) {
        if (P.mode == 0)
          for (int i = lane; i < B; i += 32) P.pos[2 * i] = t + 1;
        if (lane == 0) P.ws_pos[ts & 1] = ts;
      }
      if (lane == 0) {
        P.pos[1] = 0;
        if (!bad && P.mode == 0) atomicAdd(&P.bar[0], 1);   // next launch's epoch
      }
    }
  }
  if (bad) {
    // 2: position outside the cache; 6: ragged batch; 8: the workspace holds no partial sums for this position
    if (tid == 0 && cta == 0 && P.status) atomicExch(P.status, bad == 1 ? 2 : (bad == 2 ? 6 : 8));
  } else {
    const int p = t & 1, s = t >> 1;
    const int ps = ts & 1, ss = ts >> 1;
    const int nsl = (ts < 2 * Lh) ? (ss + SEG - 1) / SEG : 0;
    float* part_out = P.part + (size_t)(ts & 1) * rows * 64;
    const float* part_in = P.part + (size_t)(t & 1) * rows * 64;

    if (warp == W_PROD) {
      // ------------------------------------------------------------------ history producer
      if (lane == 0) {
        const int o = Lh - 1 - ss, e = o & 7, xo = o - e;
        const uint64_t once = tma::policy_evict_first();   // the history is read once per step: do not let it push the
        const uint64_t keep = tma::policy_evict_last();    // weights and taps (re-read every step) out of L2
        int n = 0;
        // the stream has slack, the projection does not: let the compute group's operands go first
        bool ok = P.mode != 0 || tma::mbar_wait_bounded(go_bar, 0u, abort_flag);
        for (int r = cta; ok && r < rows; r += G) {
          for (int sl = 0; sl < nsl; sl++, n++) {
            const int st = n % STAGES;
            if (!tma::mbar_wait_bounded(&empty_bar[st], (((uint32_t)(n / STAGES)) & 1u) ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            unsigned char* dst = smem + st * STAGE_BYTES;
            tma::mbar_expect_tx(&full_bar[st], STAGE_BYTES);
            tma::load_4d_hint(dst, &tmH, &full_bar[st], sl * SEG, ps, r * 8, 0, once);
            tma::load_3d_hint(dst + HIST_BYTES, &tmT, &full_bar[st], xo + sl * SEG, r * 8, e, keep);
            s_issued = n + 1;
          }
        }
      }
    } else if (warp == W_WPROD) {
      // ------------------------------------------------------------------ MLP weight producer (token step only)
      // gate|up unit j goes to slot (nGu-1-j) % 3 (rows n0..n0+7 of the gate weight, then of the up weight, each row
      // one bulk copy), so the last unit always sits in slot 0 and the down-projection unit (8 rows of I values, two
      // slots) can land in slots 1 and 2 while that last unit is still being used
      if (lane == 0 && P.mode == 0) {
        const uint32_t row_bytes = (uint32_t)d * 2;
        const uint64_t keep = tma::policy_evict_last();
        bool ok = true;
        for (int j = 0; ok && j < nGu; j++) {
          const int slot = (nGu - 1 - j) % MLP_SLOTS, n0 = (cta + j * G) * 8;
          if (!tma::mbar_wait_bounded(&wempty[slot], (((uint32_t)(j / MLP_SLOTS)) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          unsigned char* dst = wsm + slot * MLP_SLOT;
          tma::mbar_expect_tx(&wfull[slot], 16 * row_bytes);
          for (int rr = 0; rr < 8; rr++) {
            tma::bulk_load_hint(dst + rr * row_bytes, P.Wg + (size_t)(n0 + rr) * d, row_bytes, &wfull[slot], keep);
            tma::bulk_load_hint(dst + (8 + rr) * row_bytes, P.Wu + (size_t)(n0 + rr) * d, row_bytes, &wfull[slot], keep);
          }
        }
        if (ok && hasD) {
          // slots 1 and 2 free of their last gate|up unit (slot s is used by units j with (nGu-1-j) % 3 == s)
          for (int sl = 1; ok && sl <= 2; sl++) {
            const int uses = nGu > sl ? (nGu - 1 - sl) / MLP_SLOTS + 1 : 0;
            ok = tma::mbar_wait_bounded(&wempty[sl], (((uint32_t)uses) & 1u) ^ 1u, abort_flag);
          }
          if (ok) {
            const uint32_t drow = (uint32_t)I * 2;
            tma::mbar_expect_tx(dfull, 8 * drow);
            for (int rr = 0; rr < 8; rr++)
              tma::bulk_load_hint(wsm + MLP_SLOT + rr * drow, P.Wd + (size_t)(cta * 8 + rr) * I, drow, dfull, keep);
          }
        }
      }
    } else if (warp < 8) {
      // ------------------------------------------------------------------ streaming consumers (warp = channel)
      const int ch = warp;
      int n = 0;
      for (int r = cta; r < rows; r += G) {
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
        for (int sl = 0; sl < nsl; sl++, n++) {
          const int st = n % STAGES;
          const bool ok = __all_sync(0xffffffffu,
                                     tma::mbar_wait_bounded(&full_bar[st], ((uint32_t)(n / STAGES)) & 1u, abort_flag));
          if (ok) {
            const bf16* H = reinterpret_cast<const bf16*>(smem + st * STAGE_BYTES) + (size_t)(g * 8 + ch) * SEG;
            const bf16* T = reinterpret_cast<const bf16*>(smem + st * STAGE_BYTES + HIST_BYTES) + (size_t)ch * SEG;
            const bool tail = (sl == nsl - 1);
#pragma unroll
            for (int win = 0; win < SEG / 64; win++) {
#pragma unroll
              for (int pass = 0; pass < 2; pass++) {
                const int koff = win * 64 + ((q + 4 * ((g & 1) ^ pass)) << 3);
                uint4 a = lds128(H + koff);
                const uint4 b = lds128(T + koff);
                if (tail) {
                  const int keep = ss - (sl * SEG + koff);
                  if (keep <= 0) a = make_uint4(0, 0, 0, 0);
                  else if (keep < 8) a = keep_first(a, keep);
                }
                mma_rows8(acc[win], a, b);
              }
            }
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(&empty_bar[st]);
          }
        }
        if (q == (g >> 1)) {   // D[g][g] sits in lane (g, q = g/2), register g&1
          const float even = (acc[0][0] + acc[1][0]) + (acc[2][0] + acc[3][0]);
          const float odd = (acc[0][1] + acc[1][1]) + (acc[2][1] + acc[3][1]);
          __stcg(part_out + (size_t)r * 64 + g * 8 + ch, (g & 1) ? odd : even);
        }
      }
      if (tid == 0) stamp(P, 7);
    } else if (P.mode == 0) {
      // ------------------------------------------------------------------ compute group (warps 10..17)
      const int cw = warp - W_COMP, ct = tid - W_COMP * 32;
      const int nb = min(8, B);
      const bool rowok = g < nb;
      const int nchunks = (d + 31) >> 5;
      // ---- phase 1: projection of the new token, history append, combine with the waiting partial sums -> mid
      for (int r = cta; r < rows; r += G) {
        const int c0 = r * 8;
        // every operand is requested before the first is used: one memory round trip for the whole phase
        uint4 sx[4], wv[4], xr4[4], nw4[4];
        const bf16* xs = P.x + (size_t)(cw < nb ? cw : 0) * P.x_rstride;    // statistics: warp cw takes sequence cw
        const bf16* xg = P.x + (size_t)(rowok ? g : 0) * P.x_rstride;       // projection: lane row g
        const bf16* mrow = P.MinT + (size_t)(c0 + g) * d;
        float sq = 0.f;
        for (int k0 = 0; k0 < d; k0 += 1024) {   // statistics in rounds of 1024 values
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const int kk = k0 + lane * 8 + 256 * j;
            sx[j] = (kk + 8 <= d) ? *reinterpret_cast<const uint4*>(xs + kk) : make_uint4(0, 0, 0, 0);
          }
          if (k0 == 0) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const int kk = ((cw + 8 * j) << 5) + q * 8;
              const bool kok = (cw + 8 * j) < nchunks && kk + 8 <= d;
              wv[j] = kok ? ldg_stream128(mrow + kk) : make_uint4(0, 0, 0, 0);
              xr4[j] = (kok && rowok) ? *reinterpret_cast<const uint4*>(xg + kk) : make_uint4(0, 0, 0, 0);
              nw4[j] = kok ? *reinterpret_cast<const uint4*>(P.stu_norm_w + kk) : make_uint4(0, 0, 0, 0);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const uint32_t w[4] = {sx[j].x, sx[j].y, sx[j].z, sx[j].w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xffff0000u);
              sq += lo * lo + hi * hi;
            }
          }
        }
        float tap0 = 0.f, res = 0.f, pin = 0.f;
        const int bb = ct >> 3, cc = ct & 7;
        if (ct < 64 && bb < nb) {
          tap0 = __bfloat162float(P.taps8[(size_t)(c0 + cc) * LP + (Lh - 1)]);
          res = __bfloat162float(P.x[(size_t)bb * P.x_rstride + c0 + cc]);
          pin = __ldcg(part_in + (size_t)r * 64 + ct);
        }
        sq = warp_sum(sq);
        if (lane == 0) s_r[cw] = (cw < nb) ? rsqrtf(sq / (float)d + P.eps_stu) : 0.f;
        comp_bar();
        if (ct == 0 && r == cta) tma::mbar_arrive(go_bar);   // statistics done: the operands are here
        {
          float accp[4] = {0.f, 0.f, 0.f, 0.f};
          const float rg = s_r[g];
#pragma unroll
          for (int j = 0; j < 4; j++) mma_rows8(accp, rowok ? norm_pack(xr4[j], rg, nw4[j]) : make_uint4(0, 0, 0, 0), wv[j]);
          for (int kc0 = cw + 32; kc0 < nchunks; kc0 += 32) {   // layers wider than 1024: further rounds
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const int kk = ((kc0 + 8 * j) << 5) + q * 8;
              if ((kc0 + 8 * j) < nchunks && kk + 8 <= d) {
                const uint4 w2 = ldg_stream128(mrow + kk);
                const uint4 x2 = rowok ? norm_pack(*reinterpret_cast<const uint4*>(xg + kk), rg,
                                                   *reinterpret_cast<const uint4*>(P.stu_norm_w + kk))
                                       : make_uint4(0, 0, 0, 0);
                mma_rows8(accp, x2, w2);
              } else {
                mma_rows8(accp, make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0));
              }
            }
          }
          s_red[cw][0][g * 8 + 2 * q] = accp[0];
          s_red[cw][0][g * 8 + 2 * q + 1] = accp[1];
        }
        comp_bar();
        if (ct < 64 && bb < nb) {
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < 8; w++) sum += s_red[w][0][ct];
          const float xp = round_to<bf16>(sum);
          P.hist[((size_t)((size_t)bb * d + c0 + cc) * 2 + p) * Lh + s] = __float2bfloat16_rn(xp);
          const float y = round_to<bf16>(2.f * (pin + xp * tap0));
          P.mid[(size_t)bb * d + c0 + cc] = __float2bfloat16_rn(res + y);
        }
        comp_bar();
      }
      if (ct == 0 && cta >= rows) tma::mbar_arrive(go_bar);   // no row here: nothing to wait for
      if (ct == 0) {
        stamp(P, 2);
        grid_arrive(&P.bar[1]);                                        // this CTA's rows of mid are written
        s_ok = grid_wait(&P.bar[1], target, abort_flag) ? 1 : 0;       // ... and so are everybody else's
        stamp(P, 3);
      }
      comp_bar();
      bool ok = s_ok != 0;
      uint4 xa[4];   // normalised rows of mid as MMA A fragments, kept for all gate|up units (d <= 1024)
      if (ok) {
        {  // RMS statistics of mid: warp cw takes sequence cw
          float sq = 0.f;
          if (cw < nb) {
            const bf16* mr = P.mid + (size_t)cw * d;
            for (int kk = lane * 8; kk < d; kk += 256) {
              const uint4 raw = ldcg128(mr + kk);
              const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int i = 0; i < 4; i++) {
                const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xffff0000u);
                sq += lo * lo + hi * hi;
              }
            }
          }
          const bf16* mrow2 = P.mid + (size_t)(rowok ? g : 0) * d;
#pragma unroll
          for (int j = 0; j < 4; j++) {   // raw fragments requested in the same round trip as the statistics
            const int kk = ((cw + 8 * j) << 5) + q * 8;
            xa[j] = ((cw + 8 * j) < nchunks && kk + 8 <= d && rowok) ? ldcg128(mrow2 + kk) : make_uint4(0, 0, 0, 0);
          }
          sq = warp_sum(sq);
          if (lane == 0) s_r[cw] = (cw < nb) ? rsqrtf(sq / (float)d + P.eps_mlp) : 0.f;
        }
        comp_bar();
        {
          const float rg = s_r[g];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const int kk = ((cw + 8 * j) << 5) + q * 8;
            if ((cw + 8 * j) < nchunks && kk + 8 <= d && rowok)
              xa[j] = norm_pack(xa[j], rg, *reinterpret_cast<const uint4*>(P.mlp_norm_w + kk));
          }
        }
        // ---- phase 2: gate | up units from the shared-memory slots
        for (int j = 0; j < nGu; j++) {
          const int slot = (nGu - 1 - j) % MLP_SLOTS, n0 = (cta + j * G) * 8;
          const bool okw = __all_sync(0xffffffffu, tma::mbar_wait_bounded(&wfull[slot], ((uint32_t)(j / MLP_SLOTS)) & 1u,
                                                                         abort_flag));
          float ag[4] = {0.f, 0.f, 0.f, 0.f}, au[4] = {0.f, 0.f, 0.f, 0.f};
          if (okw) {
            const bf16* gsm = reinterpret_cast<const bf16*>(wsm + slot * MLP_SLOT) + (size_t)g * d;
            const bf16* usm = gsm + (size_t)8 * d;
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
              const int kk = ((cw + 8 * jj) << 5) + q * 8;
              if ((cw + 8 * jj) < nchunks && kk + 8 <= d) {
                mma_rows8(ag, xa[jj], lds128(gsm + kk));
                mma_rows8(au, xa[jj], lds128(usm + kk));
              }
            }
          }
          s_red[cw][0][g * 8 + 2 * q] = ag[0];
          s_red[cw][0][g * 8 + 2 * q + 1] = ag[1];
          s_red[cw][1][g * 8 + 2 * q] = au[0];
          s_red[cw][1][g * 8 + 2 * q + 1] = au[1];
          comp_bar();   // every warp has read the slot and written its partial products
          if (ct == 0) tma::mbar_arrive(&wempty[slot]);
          if (ct < 64) {
            float sg = 0.f, su = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) {
              sg += s_red[w][0][ct];
              su += s_red[w][1][ct];
            }
            const int bb = ct >> 3, cc = ct & 7;
            if (bb < nb) {
              const float gte = round_to<bf16>(gelu_tanh(round_to<bf16>(sg)));
              P.hbuf[(size_t)bb * I + n0 + cc] = __float2bfloat16_rn(gte * round_to<bf16>(su));
            }
          }
          comp_bar();
        }
        if (ct == 0) {
          stamp(P, 4);
          grid_arrive(&P.bar[2]);                                     // this CTA's hidden features are written
          s_ok = grid_wait(&P.bar[2], target, abort_flag) ? 1 : 0;
          stamp(P, 5);
        }
        comp_bar();
        ok = s_ok != 0;
      }
      if (ok && hasD) {
        // ---- phase 3: down projection + residual for output channels cta*8 .. cta*8+7
        const int n0 = cta * 8;
        const bf16* hrow = P.hbuf + (size_t)(rowok ? g : 0) * I;
        const int nch2 = (I + 31) >> 5;
        const bool okd = __all_sync(0xffffffffu, tma::mbar_wait_bounded(dfull, 0u, abort_flag));
        float ad[4] = {0.f, 0.f, 0.f, 0.f};
        if (okd) {
          const bf16* dsm = reinterpret_cast<const bf16*>(wsm + MLP_SLOT) + (size_t)g * I;
          for (int kc0 = cw; kc0 < nch2; kc0 += 64) {   // rounds of eight chunks per warp
            uint4 ha[8];
#pragma unroll
            for (int jj = 0; jj < 8; jj++) {
              const int kk = ((kc0 + 8 * jj) << 5) + q * 8;
              ha[jj] = ((kc0 + 8 * jj) < nch2 && kk + 8 <= I && rowok) ? ldcg128(hrow + kk) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int jj = 0; jj < 8; jj++) {
              const int kk = ((kc0 + 8 * jj) << 5) + q * 8;
              if ((kc0 + 8 * jj) < nch2 && kk + 8 <= I) mma_rows8(ad, ha[jj], lds128(dsm + kk));
            }
          }
        }
        s_red[cw][0][g * 8 + 2 * q] = ad[0];
        s_red[cw][0][g * 8 + 2 * q + 1] = ad[1];
        comp_bar();
        if (ct < 64) {
          float sd = 0.f;
#pragma unroll
          for (int w = 0; w < 8; w++) sd += s_red[w][0][ct];
          const int bb = ct >> 3, cc = ct & 7;
          if (bb < nb) {
            const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(P.mid) + (size_t)bb * d + n0 + cc);
            const float res = __uint_as_float((uint32_t)raw << 16);
            P.out[(size_t)bb * P.out_rstride + n0 + cc] = __float2bfloat16_rn(res + round_to<bf16>(sd));
          }
        }
        if (ct == 0) stamp(P, 6);
      }
    }
  }
  // ---- end of the CTA: failure report
  __syncthreads();
  if (tid == 0) stamp(P, 8);
  if (s_abort) {
    if (tid == 0 && P.status) atomicExch(P.status, 7);
    if (tid == 0) {
      const int issued = s_issued;
      for (int n = issued > STAGES ? issued - STAGES : 0; n < issued; n++) {
        int dummy = 0;
        tma::mbar_wait_bounded(&full_bar[n % STAGES], ((uint32_t)(n / STAGES)) & 1u, &dummy);
      }
      // weight copies in flight: their barriers complete once the bytes have landed
      int dummy = 0;
      for (int i = 0; i < MLP_SLOTS; i++) tma::mbar_wait_bounded(&wfull[i], 0u, &dummy, 20000000ull, 1u << 16);
    }
    __syncthreads();
  }
}

long long ws_bytes(int d, int I) {
  const long long rows = d / 8;
  return 256 + 2 * rows * 64 * 4 + (long long)8 * d * 2 + (long long)8 * I * 2;
}

}  // namespace

// Workspace of stu_block_decode_step for a layer of width d with I hidden MLP features: 256 bytes of control words
// (positions of the two partial-sum buffers, two grid barriers), the two partial-sum buffers, `mid` and the hidden
// activations.  Zero it once: an all-zero workspace is the correct state for position 0.
extern "C" long long stu_block_step_workspace_bytes(int d, int I) {
  if (d <= 0 || I <= 0 || d % 8) return 0;
  return ws_bytes(d, I);
}

// One cached token step of a whole approx STU layer for up to 8 sequences at one common position (bf16):
//   mid = x + STU(rmsnorm(x) * stu_norm_w);  out = mid + down(gelu_tanh(gate(n)) * up(n)), n = rmsnorm(mid) * mlp_norm_w
// mode 0 needs the partial sums of the current position in the workspace (left there by the previous mode-0 launch, by
// a mode-1 launch, or trivially for position 0 of a zeroed workspace; status 8 otherwise); it leaves those of the next
// position and advances pos.  mode 1 only computes the partial sums of the current position (cold start after a
// prefill).  out may alias x.  d % 8 == 0, I % 8 == 0, Lh % 8 == 0, B <= 8, workspace 256-byte aligned.
extern "C" int stu_block_decode_step(const void* x, long long x_row_stride, const void* stu_norm_w, const void* MinT,
                                     void* hist, const void* taps8, int* pos, const void* mlp_norm_w, const void* Wg,
                                     const void* Wu, const void* Wd, void* out, long long out_row_stride, int B, int d,
                                     int I, int Lh, float eps_stu, float eps_mlp, void* workspace,
                                     long long workspace_bytes, int mode, int* status, int dtype, void* stream) {
  if (!x || !stu_norm_w || !MinT || !hist || !taps8 || !pos || !mlp_norm_w || !Wg || !Wu || !Wd || !out || !workspace)
    return STU_ERR_NULL;
  const bool timeline = (mode & 0x10) != 0;   // record CTA 0's globaltimer stamps at byte 128 of the workspace
  mode &= ~0x10;
  if (B <= 0 || B > 8 || d <= 0 || I <= 0 || Lh <= 0 || d % 8 || I % 8 || Lh % 8 || (mode != 0 && mode != 1))
    return STU_ERR_SHAPE;
  if (dtype != STU_BF16) return STU_ERR_DTYPE;
  if (x_row_stride % 8 || out_row_stride % 8 || !aligned16(x) || !aligned16(MinT) || !aligned16(hist) ||
      !aligned16(stu_norm_w) || !aligned16(taps8) || !aligned16(mlp_norm_w) || !aligned16(Wg) || !aligned16(Wu) ||
      !aligned16(Wd) || !aligned16(out) || (((uintptr_t)workspace) & 255u))
    return STU_ERR_ALIGN;
  if (workspace_bytes < ws_bytes(d, I)) return STU_ERR_SHAPE;

  CUtensorMap tmH, tmT;
  {
    const cuuint64_t dims[4] = {(cuuint64_t)Lh, 2, (cuuint64_t)d, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)Lh * 2, (cuuint64_t)Lh * 4, (cuuint64_t)d * Lh * 4};
    const cuuint32_t box[4] = {SEG, 1, 8, 8};
    int rc = tma::encode_bf16(&tmH, hist, 4, dims, strides, box);
    if (rc != STU_OK) return rc;
  }
  {
    const cuuint64_t LP = (cuuint64_t)Lh + 8;
    const cuuint64_t dims[3] = {LP, (cuuint64_t)d, 8};
    const cuuint64_t strides[2] = {LP * 2, (cuuint64_t)d * LP * 2};
    const cuuint32_t box[3] = {SEG, 8, 1};
    int rc = tma::encode_bf16(&tmT, taps8, 3, dims, strides, box);
    if (rc != STU_OK) return rc;
  }
  StepParams P;
  P.x = (const bf16*)x;
  P.x_rstride = x_row_stride;
  P.stu_norm_w = (const bf16*)stu_norm_w;
  P.MinT = (const bf16*)MinT;
  P.hist = (bf16*)hist;
  P.taps8 = (const bf16*)taps8;
  P.pos = pos;
  P.mlp_norm_w = (const bf16*)mlp_norm_w;
  P.Wg = (const bf16*)Wg;
  P.Wu = (const bf16*)Wu;
  P.Wd = (const bf16*)Wd;
  P.out = (bf16*)out;
  P.out_rstride = out_row_stride;
  P.B = B;
  P.d = d;
  P.I = I;
  P.Lh = Lh;
  P.eps_stu = eps_stu;
  P.eps_mlp = eps_mlp;
  unsigned char* ws = (unsigned char*)workspace;
  P.ws_pos = (int*)ws;            // [2]
  P.bar = (int*)ws + 4;           // [3]
  const long long rows = d / 8;
  P.part = (float*)(ws + 256);
  P.mid = (bf16*)(ws + 256 + 2 * rows * 64 * 4);
  P.hbuf = P.mid + (size_t)8 * d;
  P.status = status;
  P.mode = mode;
  P.tl = timeline ? (unsigned long long*)(ws + 128) : nullptr;

  // the MLP weights pass through three 32 KB slots of shared memory: a gate|up unit (16 rows of d) must fit one, the
  // down-projection unit (8 rows of I) two
  if ((long long)32 * d > MLP_SLOT || (long long)16 * I > 2 * MLP_SLOT) return STU_ERR_UNSUPPORTED;
  const size_t smem = (size_t)STAGES * STAGE_BYTES + MLP_BYTES + (2 * STAGES + 2 * MLP_SLOTS + 2) * sizeof(uint64_t) + 1024;
  cudaError_t e =
      cudaFuncSetAttribute(stu_block_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, stu_block_step_kernel, NTHREADS, smem);
  if (e != cudaSuccess) return (int)e;
  if (per_sm < 1) return STU_ERR_UNSUPPORTED;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(device_sm_count());
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;   // the grid barriers need every CTA resident
  at[0].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, stu_block_step_kernel, tmH, tmT, P);
  if (e != cudaSuccess) return (int)e;
  STU_CHECK_LAUNCH();
  return STU_OK;
}
