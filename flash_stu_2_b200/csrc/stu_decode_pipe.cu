// Fused decode step of an approx STU layer for a batch that stands at one common position, as a persistent
// bulk-copy pipeline (bf16).  Same arithmetic as stu_decode_rows8_kernel (stu_conv.cu):
//   xn  = rmsnorm(x[b,:]) * norm_w ; xp = round(xn . MinT[c,:]) ; hist[b][c][t&1][t>>1] = xp
//   y   = round(2 * (sum_{i<s} hist[b][c][p][i] * tap_c[s-i] + xp * tap_c[0]))   (s = t>>1, p = t&1)
//   out[b,c] = round(x[b,c] + y)            (flash_stu/modules/stu.py:85-98,120 evaluated for the one new position)
//
// The step is bound by streaming one parity run of the projected history of every (sequence, channel) from HBM, so
// the kernel is organised around keeping as many bytes in flight as an SM can hold, and around keeping everything
// that is not streaming off the streaming warps' critical path:
//   * a ROW is 8 sequences x 8 channels; CTA i of the persistent grid (one CTA per SM) owns rows i, i + grid, ...;
//     a row's history is cut into UNITS of 256 positions (32 KB) plus the matching 8 x 256 reversed taps (4 KB); a
//     unit is fetched by two bulk tensor copies (cp.async.bulk.tensor 4-D / 3-D, zero fill outside the tensors)
//     into one stage of a 4-stage shared-memory ring, completion on an mbarrier: up to 144 KB in flight per SM
//     (the rest of the SM's shared memory is left to the CTAs of an overlapped neighbouring kernel);
//   * warp 8 is the producer (one thread issues the copies as stages free up, running ahead across rows);
//   * warps 0..7 are the streaming consumers, warp w owning channel w of the row: the dot products of its 8 sequences
//     are the diagonal of an mma.sync m16n8k16 product (history as A, taps as B; the k-order is permuted per row so
//     that the 16-byte shared-memory reads of a quarter warp hit 32 distinct banks; four independent accumulators);
//   * warps 9..12 are the projection group: for each row they compute the RMS statistics and the projection of the
//     new token (K split over the four warps, MMAs with the sequences as rows), append xp to the history, and, once
//     the consumers hand over the row's 64 partial sums through shared memory, write the outputs.  The consumers
//     never wait for them (two hand-over slots), so the projection of a row runs under the stream of that row.
// No cross-CTA reduction, no workspace: a row is summed inside one CTA, slices in order.
// In an overlapped (programmatic) launch only the projection group waits for the preceding kernel: history, taps and
// positions were written by this layer's previous step, which has completed by the time this kernel can start.
//
// Every mbarrier wait is bounded; on expiry the CTA raises status 7, lets its outstanding copies land (bounded) and
// returns.
#include "common.cuh"
#include "tma.cuh"
#include "peer.cuh"

int device_sm_count();  // gemm_tc.cu

namespace {

constexpr int SEG = 256;                       // history positions per unit
constexpr int STAGES = 4;   // 144 KB of the SM's shared memory: CTAs of a neighbouring kernel still fit beside this one
constexpr int HIST_BYTES = 64 * SEG * 2;       // 8 sequences x 8 channels x SEG bf16
constexpr int TAP_BYTES = 8 * SEG * 2;
constexpr int STAGE_BYTES = HIST_BYTES + TAP_BYTES;

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__device__ __forceinline__ uint4 lds128(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(tma::smem_u32(p)));
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
// rows 8..15 of the A tile are zero
__device__ __forceinline__ void mma_rows8(float (&c)[4], const uint4& a, const uint4& b) {
  mma16816(c, a.x, 0u, a.y, 0u, b.x, b.y);
  mma16816(c, a.z, 0u, a.w, 0u, b.z, b.w);
}
// keep the first `keep` (1..7) of the eight bf16 values of a vector
__device__ __forceinline__ uint4 keep_first(const uint4& v, int keep) {
  uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; j++)
    if (2 * j + 1 >= keep) w[j] = (2 * j < keep) ? (w[j] & 0x0000ffffu) : 0u;
  return make_uint4(w[0], w[1], w[2], w[3]);
}

struct Params {
  const bf16* x;
  long long x_rstride;
  const bf16* norm_w;
  const bf16* MinT;
  bf16* hist;
  const bf16* taps8;
  int* pos;
  bf16* out;
  long long out_rstride;
  int B, d, dch, add_resid, Lh;
  float eps;
  int* status;
  int pdl;
  const PeerDest* peer;   // tensor parallelism: the output rows go to every rank's inbox instead of `out`
  const bf16* xp_in;      // when set: the projected input of the new token, computed by the caller for the whole batch
  long long xp_rstride;   //           (rows of d_ch values); norm_w, MinT and the projection warps' MMAs are not used
};

constexpr int NTHREADS = 13 * 32;   // 8 consumer warps, 1 producer warp, 4 projection warps

__device__ __forceinline__ void group_bar() { asm volatile("bar.sync 2, 128;" ::: "memory"); }   // projection group

__global__ void __launch_bounds__(NTHREADS, 1)
    stu_decode_pipe_kernel(const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmT,
                           const Params P) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* part_full = empty_bar + STAGES;   // [2] consumers -> projection group: the row's partial sums are in s_part
  uint64_t* part_free = part_full + 2;        // [2] projection group -> consumers: the slot may be overwritten
  __shared__ int s_abort, s_issued;
  __shared__ float s_part[2][64];
  __shared__ float s_r[8];
  __shared__ float s_red[4][64];
  volatile int* abort_flag = &s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q = lane & 3;
  const int G = gridDim.x, cta = blockIdx.x;
  const int B = P.B, d = P.d, dch = P.dch, Lh = P.Lh;
  const int LP = Lh + 8;
  const int nbg = (B + 7) >> 3, ncg = dch >> 3, rows = nbg * ncg;

  if (tid == 0) {
    for (int i = 0; i < STAGES; i++) {
      tma::mbar_init(&full_bar[i], 1);
      tma::mbar_init(&empty_bar[i], 8);
    }
    for (int i = 0; i < 2; i++) {
      tma::mbar_init(&part_full[i], 8);
      tma::mbar_init(&part_free[i], 1);
    }
    s_abort = 0;
    s_issued = 0;
    tma::fence_barrier_init();
  }
  if (P.pdl & STU_FLAG_EARLY_TRIGGER) pdl_trigger();
  // ---- common position (written by this layer's previous step, not by the kernel an overlapped launch follows)
  const int t = P.pos[0];
  int bad = (t < 0 || t >= 2 * Lh) ? 1 : 0;
  for (int b = tid; b < B; b += NTHREADS)
    if (P.pos[2 * b] != t) bad = 2;
  bad = __syncthreads_or(bad);   // also publishes the barrier initialisation
  // ---- arrival counter of the grid: every thread of this CTA has read the positions, so it may say so now; the last
  // CTA to arrive advances them while the stream runs (nothing else in this launch reads them again), which keeps
  // the round trip of the counter and the update off the end of the kernel
  if (warp == 0) {
    int last = 0;
    if (lane == 0) last = (atomicAdd(&P.pos[1], 1) == G - 1) ? 1 : 0;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      if (!bad) {
        for (int i = lane; i < B; i += 32) {
          const int tv = P.pos[2 * i];
          if (tv >= 0 && tv < 2 * Lh) P.pos[2 * i] = tv + 1;
        }
      }
      if (lane == 0) P.pos[1] = 0;
    }
  }
  if (bad) {
    // 2: position outside the cache; 6: the caller promised one common position and the batch is ragged
    if (tid == 0 && cta == 0 && P.status) atomicExch(P.status, (t < 0 || t >= 2 * Lh) ? 2 : 6);
  } else {
    const int p = t & 1, s = t >> 1;
    const int nsl = (s + SEG - 1) / SEG;

    if (warp == 8) {
      // ------------------------------------------------------------------ producer
      if (lane == 0) {
        const int o = Lh - 1 - s, e = o & 7, xo = o - e;   // reversed tap row of position s at its 16-byte alignment
        int n = 0;
        bool ok = true;
        for (int r = cta; ok && r < rows; r += G) {
          const int bg = r / ncg, cg = r - bg * ncg;
          for (int sl = 0; sl < nsl; sl++, n++) {
            const int st = n % STAGES;
            if (!tma::mbar_wait_bounded(&empty_bar[st], (((uint32_t)(n / STAGES)) & 1u) ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            unsigned char* dst = smem + st * STAGE_BYTES;
            tma::mbar_expect_tx(&full_bar[st], STAGE_BYTES);
            tma::load_4d(dst, &tmH, &full_bar[st], sl * SEG, p, cg * 8, bg * 8);
            tma::load_3d(dst + HIST_BYTES, &tmT, &full_bar[st], xo + sl * SEG, cg * 8, e);
            s_issued = n + 1;
          }
        }
      }
    } else if (warp < 8) {
      // ------------------------------------------------------------------ streaming consumers (warp = channel)
      const int ch = warp;
      int n = 0, k = 0;
      for (int r = cta; r < rows; r += G, k++) {
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
        for (int sl = 0; sl < nsl; sl++, n++) {
          const int st = n % STAGES;
          // every lane waits (acquires the copied bytes); the vote keeps the warp converged for the MMAs
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
                // row g takes the chunks of its 64-value window in the order that keeps the eight lanes of a
                // quarter warp (two rows x four chunks) on distinct banks; taps use the same order, only D[g][g] is read
                const int koff = win * 64 + ((q + 4 * ((g & 1) ^ pass)) << 3);
                uint4 a = lds128(H + koff);
                const uint4 b = lds128(T + koff);
                if (tail) {
                  const int keep = s - (sl * SEG + koff);   // values of this vector that are stored history
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
        // hand the row's 64 partial sums to the projection group (slot k & 1)
        const int slot = k & 1;
        const bool okf = __all_sync(0xffffffffu, tma::mbar_wait_bounded(&part_free[slot], (((uint32_t)(k >> 1)) & 1u) ^ 1u,
                                                                       abort_flag));
        if (okf) {
          // D[g][g] sits in lane (g, q = g/2), register g&1
          if (q == (g >> 1)) {
            const float even = (acc[0][0] + acc[1][0]) + (acc[2][0] + acc[3][0]);
            const float odd = (acc[0][1] + acc[1][1]) + (acc[2][1] + acc[3][1]);
            s_part[slot][g * 8 + ch] = (g & 1) ? odd : even;
          }
          __syncwarp();
          if (lane == 0) tma::mbar_arrive(&part_full[slot]);
        }
      }
    } else {
      // ------------------------------------------------------------------ projection group (warps 9..12)
      const int gw = warp - 9, gt = tid - 9 * 32;   // warp / thread index inside the group
      bool waited = false;
      int k = 0;
      for (int r = cta; r < rows; r += G, k++) {
        if (!waited) {
          pdl_wait();   // x is written by the preceding kernel
          if (!(P.pdl & STU_FLAG_EARLY_TRIGGER)) pdl_trigger();
          waited = true;
        }
        const int bg = r / ncg, cg = r - bg * ncg;
        const int b0 = bg * 8, c0 = cg * 8;
        const int nb = min(8, B - b0);
        // RMS statistics: warp gw takes sequences gw and gw + 4
        if (!P.xp_in) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int bb = gw + 4 * h;
          float rr = 0.f;
          if (bb < nb) {
            const bf16* xr = P.x + (size_t)(b0 + bb) * P.x_rstride;
            float ss = 0.f;
            for (int kk = lane * 8; kk < d; kk += 256) {
              float v[8];
              load_vec(xr + kk, v);
#pragma unroll
              for (int j = 0; j < 8; j++) ss += v[j] * v[j];
            }
            ss = warp_sum(ss);
            rr = rsqrtf(ss / (float)d + P.eps);
          }
          if (lane == 0) s_r[bb] = rr;
        }
        group_bar();
        {
          float accp[4] = {0.f, 0.f, 0.f, 0.f};
          const bool rowok = g < nb;
          const bf16* xr = P.x + (size_t)(b0 + (rowok ? g : 0)) * P.x_rstride;
          const bf16* mrow = P.MinT + (size_t)(c0 + g) * d;
          const float rg = s_r[g];
          for (int kc = gw; kc < ((d + 31) >> 5); kc += 4) {   // warp-uniform trip count
            const int kk = (kc << 5) + q * 8;
            uint4 xa = make_uint4(0, 0, 0, 0), wv = make_uint4(0, 0, 0, 0);
            if (kk + 8 <= d) {
              wv = *reinterpret_cast<const uint4*>(mrow + kk);
              if (rowok)
                xa = norm_pack(*reinterpret_cast<const uint4*>(xr + kk), rg,
                               *reinterpret_cast<const uint4*>(P.norm_w + kk));
            }
            mma_rows8(accp, xa, wv);
          }
          s_red[gw][g * 8 + 2 * q] = accp[0];   // (sequence g, channels 2q, 2q+1)
          s_red[gw][g * 8 + 2 * q + 1] = accp[1];
        }
        group_bar();
        }   // !P.xp_in
        float term = 0.f, res = 0.f;
        const int bb = gt >> 3, cc = gt & 7;   // threads 0..63 of the group: (sequence, channel)
        if (gt < 64 && bb < nb) {
          const float xp = P.xp_in ? __bfloat162float(P.xp_in[(size_t)(b0 + bb) * P.xp_rstride + c0 + cc])
                                   : round_to<bf16>((s_red[0][gt] + s_red[1][gt]) + (s_red[2][gt] + s_red[3][gt]));
          P.hist[((size_t)((size_t)(b0 + bb) * dch + c0 + cc) * 2 + p) * Lh + s] = __float2bfloat16_rn(xp);
          term = xp * __bfloat162float(P.taps8[(size_t)(c0 + cc) * LP + (Lh - 1)]);
          if (P.add_resid) res = __bfloat162float(P.x[(size_t)(b0 + bb) * P.x_rstride + c0 + cc]);
        }
        // the row's partial sums from the streaming warps
        const int slot = k & 1;
        const bool okp = tma::mbar_wait_bounded(&part_full[slot], ((uint32_t)(k >> 1)) & 1u, abort_flag);
        if (okp && gt < 64 && bb < nb) {
          const float y = round_to<bf16>(2.f * (s_part[slot][gt] + term));
          const bf16 v = __float2bfloat16_rn(res + y);
          const size_t o = (size_t)(b0 + bb) * P.out_rstride + c0 + cc;
          if (P.peer) {
            for (int pr = 0; pr < P.peer->n; pr++) P.peer->dest[pr][o] = v;
          } else {
            P.out[o] = v;
          }
        }
        group_bar();   // s_part[slot] read by all, s_red free for the next row
        if (gt == 0) tma::mbar_arrive(&part_free[slot]);
      }
    }
  }
  // ---- end of the CTA: tell the other ranks (when the last CTA gets here), failure report
  __syncthreads();
  if (tid == 0 && P.peer) peer_signal_when_last(P.peer, (unsigned)G);
  if (s_abort) {
    if (tid == 0 && P.status) atomicExch(P.status, 7);
    if (tid == 0) {   // copies that were issued but never consumed must land before shared memory is released
      const int issued = s_issued;
      for (int n = issued > STAGES ? issued - STAGES : 0; n < issued; n++) {
        int dummy = 0;
        tma::mbar_wait_bounded(&full_bar[n % STAGES], ((uint32_t)(n / STAGES)) & 1u, &dummy);
      }
    }
    __syncthreads();
  }
}

}  // namespace

// The fused decode step as a bulk-copy pipeline.  Arguments as stu_decode_approx_shard (d_in = d_ch and
// add_residual = 1 for a whole layer).  bf16, d_in % 8 == 0, d_ch % 8 == 0, Lh % 8 == 0, every sequence at the same
// position (checked on the device: status 6).
static int launch_pipe(const void* x, long long x_row_stride, const void* norm_w, const void* MinT, void* hist,
                       const void* taps8, int* pos, void* out, long long out_row_stride, int B, int d_in, int d_ch,
                       int Lh, float eps, int add_residual, int* status, int dtype, void* stream,
                       const PeerDest* peer, const void* xp_in = nullptr, long long xp_row_stride = 0) {
  if (xp_in) {   // projection done by the caller: x is only the residual, norm_w / MinT are not read
    if ((add_residual && !x) || !hist || !taps8 || !pos || (!out && !peer)) return STU_ERR_NULL;
    if (!x) x = xp_in;
    norm_w = MinT = xp_in;
  }
  if (!x || !norm_w || !MinT || !hist || !taps8 || !pos || (!out && !peer)) return STU_ERR_NULL;
  if (B <= 0 || d_in <= 0 || d_ch <= 0 || Lh <= 0 || d_in % 8 || d_ch % 8 || Lh % 8) return STU_ERR_SHAPE;
  if (add_residual && d_in != d_ch) return STU_ERR_SHAPE;
  const int pdl = dtype & (STU_FLAG_OVERLAP | STU_FLAG_EARLY_TRIGGER);
  dtype &= ~(STU_FLAG_OVERLAP | STU_FLAG_EARLY_TRIGGER | STU_FLAG_UNIFORM_POS);
  if (dtype != STU_BF16) return STU_ERR_DTYPE;
  if (x_row_stride % 8 || !aligned16(x) || !aligned16(MinT) || !aligned16(hist) || !aligned16(norm_w) ||
      !aligned16(taps8))
    return STU_ERR_ALIGN;

  CUtensorMap tmH, tmT;
  {
    const cuuint64_t dims[4] = {(cuuint64_t)Lh, 2, (cuuint64_t)d_ch, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)Lh * 2, (cuuint64_t)Lh * 4, (cuuint64_t)d_ch * Lh * 4};
    const cuuint32_t box[4] = {SEG, 1, 8, 8};
    int rc = tma::encode_bf16(&tmH, hist, 4, dims, strides, box);
    if (rc != STU_OK) return rc;
  }
  {
    const cuuint64_t LP = (cuuint64_t)Lh + 8;
    const cuuint64_t dims[3] = {LP, (cuuint64_t)d_ch, 8};
    const cuuint64_t strides[2] = {LP * 2, (cuuint64_t)d_ch * LP * 2};
    const cuuint32_t box[3] = {SEG, 8, 1};
    int rc = tma::encode_bf16(&tmT, taps8, 3, dims, strides, box);
    if (rc != STU_OK) return rc;
  }
  Params P;
  P.x = (const bf16*)x;
  P.x_rstride = x_row_stride;
  P.norm_w = (const bf16*)norm_w;
  P.MinT = (const bf16*)MinT;
  P.hist = (bf16*)hist;
  P.taps8 = (const bf16*)taps8;
  P.pos = pos;
  P.out = (bf16*)out;
  P.out_rstride = out_row_stride;
  P.B = B;
  P.d = d_in;
  P.dch = d_ch;
  P.add_resid = add_residual;
  P.Lh = Lh;
  P.eps = eps;
  P.status = status;
  P.pdl = pdl;
  P.peer = peer;
  P.xp_in = (const bf16*)xp_in;
  P.xp_rstride = xp_row_stride;

  const size_t smem = (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * sizeof(uint64_t) + 1024;
  cudaError_t e = cudaFuncSetAttribute(stu_decode_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const long long rows = (long long)((B + 7) / 8) * (d_ch / 8);
  const int sms = device_sm_count();
  const int grid = (int)(rows < sms ? rows : sms);
  e = launch_maybe_overlapped(stu_decode_pipe_kernel, dim3(grid), dim3(NTHREADS), smem, (cudaStream_t)stream,
                              (pdl & STU_FLAG_OVERLAP) != 0, tmH, tmT, P);
  if (e != cudaSuccess) return (int)e;
  STU_CHECK_LAUNCH();
  return STU_OK;
}

extern "C" int stu_decode_approx_pipelined(const void* x, long long x_row_stride, const void* norm_w, const void* MinT,
                                           void* hist, const void* taps8, int* pos, void* out,
                                           long long out_row_stride, int B, int d_in, int d_ch, int Lh, float eps,
                                           int add_residual, int* status, int dtype, void* stream) {
  return launch_pipe(x, x_row_stride, norm_w, MinT, hist, taps8, pos, out, out_row_stride, B, d_in, d_ch, Lh, eps,
                     add_residual, status, dtype, stream, nullptr);
}

// The channel shard of the decode step with its all-gather fused in: the d_ch outputs of every sequence are stored
// straight into every rank's inbox (exchange descriptor `peer_dest`, device memory, see stu_peer_exchange_init) and
// the ranks are signalled when the last CTA has stored.
extern "C" int stu_decode_approx_push(const void* x, long long x_row_stride, const void* norm_w, const void* MinT,
                                      void* hist, const void* taps8, int* pos, const void* peer_dest,
                                      long long dest_row_stride, int B, int d_in, int d_ch, int Lh, float eps,
                                      int* status, int dtype, void* stream) {
  if (!peer_dest) return STU_ERR_NULL;
  return launch_pipe(x, x_row_stride, norm_w, MinT, hist, taps8, pos, nullptr, dest_row_stride, B, d_in, d_ch, Lh, eps,
                     0, status, dtype, stream, (const PeerDest*)peer_dest);
}

// The decode step for a caller that has computed the projected input of the new token itself, as one GEMM over the
// whole batch: xp [B, d_ch] = (rmsnorm(x) * norm_w) @ M_inputs (flash_stu/modules/stu.py:87), rounded to bf16.  The
// kernel appends xp to hist, streams the history against the taps, advances pos and writes
// out = (add_residual ? x : 0) + round(2 * taps . hist).  For batches of more than 8 sequences, where the per-row
// projection inside stu_decode_approx_pipelined (48 KB of operands per 8 x 8 outputs) costs more than the row's stream.
extern "C" int stu_decode_approx_projected(const void* x, long long x_row_stride, const void* xp,
                                           long long xp_row_stride, void* hist, const void* taps8, int* pos, void* out,
                                           long long out_row_stride, int B, int d_ch, int Lh, int add_residual,
                                           int* status, int dtype, void* stream) {
  if (!xp) return STU_ERR_NULL;
  if (xp_row_stride % 8 || !aligned16(xp)) return STU_ERR_ALIGN;
  return launch_pipe(x, x_row_stride, nullptr, nullptr, hist, taps8, pos, out, out_row_stride, B, d_ch, d_ch, Lh, 0.f,
                     add_residual, status, dtype, stream, nullptr, xp, xp_row_stride);
}
