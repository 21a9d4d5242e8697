// Sliding-window attention prefill on the 5th-generation tensor cores (bf16, head dimension 128, sequences that
// start at position 0: every key of the call lies in the call's own qkv activations).
//
// Reference semantics (flash_stu/modules/attention.py:72-101 + the documented flash_attn_func contract): per head,
// query i sees keys j in [i - w, i]; score = softcap * tanh(q.k * scale / softcap) - slope_h * (i - j); softmax; @ V.
//
// One CTA = 128 queries of one head of one sequence; key tiles of 64.  Per tile
//   S = Q K^T        tcgen05.mma, M = 128 queries, N = 64 keys, K = 128 dims; Q (two 64-wide k-blocks) and the key tile
//                    come by cp.async.bulk.tensor with the 128-byte swizzle; S lands in tensor memory (two buffers)
//   softmax          four warps, one query row per thread: tcgen05.ld of the row's 64 scores, soft cap (hardware
//                    tanh), ALiBi, window / causal mask, exponentials in the exp2 domain against a LAZY reference
//                    maximum (moved only when the row maximum outgrows it by 2^8, then the O row in tensor memory is
//                    rescaled with tcgen05.ld/st); P is rounded to bf16 and stored swizzled into shared memory
//   O += P V         tcgen05.mma, M = 128 queries, N = 128 dims, K = 64 keys, accumulating in tensor memory; the value
//                    operand is a tile of V^T (keys contiguous), which a transpose kernel writes beforehand
// O never leaves tensor memory until the last tile.  Warps: 0 producer (tensor copies), 1 MMA issuer, 2-5 softmax.
// 96 KB of shared memory and 256 columns of tensor memory per CTA: two CTAs share an SM, one computes its softmax
// while the other's MMAs run.  Every load is a plain single-CTA copy of this GPU's own memory; every wait is bounded
// (status 11: a wait ran out or a sequence was not at position 0).
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "tma.cuh"

int launch_kv_ring_write_bf16(const void* qkv, void* k_ring, void* v_ring, int* pos, int B, int Tn, int d, int W,
                              cudaStream_t st);

namespace {

constexpr int BM = 128, BN = 64, HD = 128;
constexpr int Q_OFF = 0;                      // 2 k-blocks x [128 rows][64 dims]
constexpr int K_OFF = 32768;                  // 2 stages x 2 k-blocks x [64 keys][64 dims]
constexpr int V_OFF = K_OFF + 2 * 16384;      // [128 dims][64 keys]
constexpr int P_OFF = V_OFF + 16384;          // [128 queries][64 keys]
constexpr int SMEM_BYTES = P_OFF + 16384 + 1024;
constexpr int STATUS_SWA = 11;
constexpr float LOG2E = 1.4426950408889634f;

struct Ctl {
  uint64_t q_full, k_full[2], k_empty[2], v_full, s_full[2], p_full, pv_done;
  uint32_t tmem_slot;
  int abort_flag;
};

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {   // K-major, 128-byte swizzle, 8-row groups 1 KB apart
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {   // ex2.approx: exact 0 for -inf
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Vt[b][h][c][t] = v of token t, head h, dim c; the pad t in [Tn, Tp) is written as zeros (a masked key's value is
// multiplied by P = 0, which stale NaN bits would turn into NaN)
__global__ void __launch_bounds__(256) v_transpose_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ vt, int Tn,
                                                          int Tp, int H) {
  __shared__ bf16 tile[64][HD + 2];
  const int b = blockIdx.z, h = blockIdx.y, t0 = blockIdx.x * 64;
  const int d = H * HD;
  for (int e = threadIdx.x; e < 64 * (HD / 8); e += 256) {
    const int r = e / (HD / 8), c8 = e % (HD / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t0 + r < Tn) v = *reinterpret_cast<const uint4*>(qkv + ((size_t)b * Tn + t0 + r) * 3 * d + 2 * d + h * HD + c8 * 8);
    const unsigned short* pv = reinterpret_cast<const unsigned short*>(&v);
#pragma unroll
    for (int j = 0; j < 8; j++) reinterpret_cast<unsigned short&>(tile[r][c8 * 8 + j]) = pv[j];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < HD * 8; e += 256) {
    const int c = e >> 3, t8 = (e & 7) * 8;
    unsigned short o[8];
#pragma unroll
    for (int j = 0; j < 8; j++) o[j] = reinterpret_cast<const unsigned short&>(tile[t8 + j][c]);
    if (t0 + t8 < Tp)
      *reinterpret_cast<uint4*>(vt + ((size_t)(b * H + h) * HD + c) * Tp + t0 + t8) =
          make_uint4(o[0] | (o[1] << 16), o[2] | (o[3] << 16), o[4] | (o[5] << 16), o[6] | (o[7] << 16));
  }
}

__global__ void __launch_bounds__(192, 2) swa_umma_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                       const __grid_constant__ CUtensorMap tmK,
                                                       const __grid_constant__ CUtensorMap tmV,
                                                       const int* __restrict__ pos, const float* __restrict__ slopes,
                                                       bf16* __restrict__ out, int Tn, int H, int window, float scale,
                                                       float softcap, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ Ctl ctl;
  volatile int* abort_flag = &ctl.abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BM;
  const int d = H * HD;
  const int i_last = min(q0 + BM, Tn) - 1;
  const int j_lo = max(0, q0 - window) & ~7;       // first key of the first tile (a multiple of 8: V^T copies)
  const int nt = (i_last - j_lo) / BN + 1;         // key tiles
  const bool fresh = pos[2 * b] == 0;

  if (threadIdx.x == 0) {
    tma::mbar_init(&ctl.q_full, 1);
    for (int s = 0; s < 2; s++) {
      tma::mbar_init(&ctl.k_full[s], 1);
      tma::mbar_init(&ctl.k_empty[s], 1);
      tma::mbar_init(&ctl.s_full[s], 1);
    }
    tma::mbar_init(&ctl.v_full, 1);
    tma::mbar_init(&ctl.p_full, 128);
    tma::mbar_init(&ctl.pv_done, 1);
    ctl.abort_flag = fresh ? 0 : 1;
    tma::fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(tma::smem_u32(&ctl.tmem_slot)));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = ctl.tmem_slot;
  const uint32_t tm_s = tmem_base, tm_o = tmem_base + 128;   // S buffers at columns 0 and 64, O at 128..255

  if (!fresh) {
    // not a prefill from position 0: nothing is computed (the caller takes the general kernel for such calls)
  } else if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ producer
      tma::mbar_expect_tx(&ctl.q_full, 32768);
      tma::load_3d(smem + Q_OFF, &tmQ, &ctl.q_full, h * HD, q0, b);
      tma::load_3d(smem + Q_OFF + 16384, &tmQ, &ctl.q_full, h * HD + 64, q0, b);
      auto load_k = [&](int t) {
        const int s = t & 1;
        if (!tma::mbar_wait_bounded(&ctl.k_empty[s], ((uint32_t)(t >> 1) & 1u) ^ 1u, abort_flag)) return false;
        unsigned char* dst = smem + K_OFF + s * 16384;
        tma::mbar_expect_tx(&ctl.k_full[s], 16384);
        tma::load_3d(dst, &tmK, &ctl.k_full[s], d + h * HD, j_lo + t * BN, b);
        tma::load_3d(dst + 8192, &tmK, &ctl.k_full[s], d + h * HD + 64, j_lo + t * BN, b);
        return true;
      };
      auto load_v = [&](int t) {
        if (t > 0 && !tma::mbar_wait_bounded(&ctl.pv_done, (uint32_t)(t - 1) & 1u, abort_flag)) return false;
        tma::mbar_expect_tx(&ctl.v_full, 16384);
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            ::"r"(tma::smem_u32(smem + V_OFF)), "l"(&tmV), "r"(tma::smem_u32(&ctl.v_full)), "r"(j_lo + t * BN),
              "r"((b * H + h) * HD)
            : "memory");
        return true;
      };
      bool ok = load_k(0) && load_v(0);
      if (ok && nt > 1) ok = load_k(1);
      for (int t = 1; ok && t < nt; t++) {
        ok = load_v(t);
        if (ok && t + 1 < nt) ok = load_k(t + 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      const uint32_t q_s = tma::smem_u32(smem + Q_OFF), k_s = tma::smem_u32(smem + K_OFF),
                     v_s = tma::smem_u32(smem + V_OFF), p_s = tma::smem_u32(smem + P_OFF);
      const uint32_t id_s = idesc_n(BN), id_o = idesc_n(HD);
      auto issue_s = [&](int t) {
        const int s = t & 1;
        if (!tma::mbar_wait_bounded(&ctl.k_full[s], (uint32_t)(t >> 1) & 1u, abort_flag)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kb = 0; kb < 2; kb++)
#pragma unroll
          for (int kk = 0; kk < 4; kk++)
            umma(tm_s + s * BN, make_desc(q_s + kb * 16384) + 2 * kk, make_desc(k_s + s * 16384 + kb * 8192) + 2 * kk,
                 id_s, (kb | kk) ? 1u : 0u);
        umma_commit(&ctl.s_full[s]);
        umma_commit(&ctl.k_empty[s]);
        return true;
      };
      bool ok = tma::mbar_wait_bounded(&ctl.q_full, 0, abort_flag);
      if (ok) ok = issue_s(0);
      if (ok && nt > 1) ok = issue_s(1);
      for (int t = 0; ok && t < nt; t++) {
        if (!tma::mbar_wait_bounded(&ctl.p_full, (uint32_t)t & 1u, abort_flag)) { ok = false; break; }
        if (!tma::mbar_wait_bounded(&ctl.v_full, (uint32_t)t & 1u, abort_flag)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < 4; kk++)
          umma(tm_o, make_desc(p_s) + 2 * kk, make_desc(v_s) + 2 * kk, id_o, (t | kk) ? 1u : 0u);
        umma_commit(&ctl.pv_done);
        if (t + 2 < nt) ok = issue_s(t + 2);   // its S buffer was read before p_full(t), its K stage freed by S(t)
      }
    }
  } else {
    // -------------------------------------------------------------------- softmax warps (TMEM lane quarter = warp % 4)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;       // query row of this thread
    const int i = q0 + row;                    // absolute position (the sequence starts at 0)
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float c2 = slopes[h] * LOG2E;
    const float base_i = -c2 * (float)i;
    const float k0 = softcap > 0.f ? scale / softcap : 0.f;
    const float k1 = softcap > 0.f ? softcap * LOG2E : scale * LOG2E;
    unsigned char* prow = smem + P_OFF + (row >> 3) * 1024 + (row & 7) * 128;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int t = 0; t < nt; t++) {
      const int jt = j_lo + t * BN;
      ok = tma::mbar_wait_bounded(&ctl.s_full[t & 1], (uint32_t)(t >> 1) & 1u, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t sr[64];
      tmem_ld32(tm_s + lane_base + (t & 1) * BN, sr);
      tmem_ld32(tm_s + lane_base + (t & 1) * BN + 32, sr + 32);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      // soft cap, ALiBi, mask; exp2 domain.  Constants folded so that a score costs one multiply, the hardware tanh
      // and two fused multiply-adds: score2 = tanh(s * k0) * k1 + (c2 * j + base_i), with k0 = scale / softcap,
      // k1 = softcap * log2(e), c2 = slope * log2(e), base_i = -c2 * i
      const bool interior = (jt + BN - 1 <= q0) && (jt >= q0 + BM - 1 - window) && (q0 + BM - 1 <= i_last);
      const float base_t = fmaf(c2, (float)jt, base_i);
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; c++) {
        float sc;
        if (softcap > 0.f) {   // hardware tanh: relative error 2^-11, below the bf16 rounding of P
          float th;
          asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(__uint_as_float(sr[c]) * k0));
          sc = fmaf(th, k1, fmaf(c2, (float)c, base_t));
        } else {
          sc = fmaf(__uint_as_float(sr[c]), k1, fmaf(c2, (float)c, base_t));
        }
        if (!interior) {
          const int j = jt + c;
          const bool valid = (j <= i) && (j >= i - window) && (i <= i_last);
          sc = valid ? sc : -INFINITY;
        }
        sr[c] = __float_as_uint(sc);
        mx = fmaxf(mx, sc);
      }
      // lazy reference maximum: moved (and the O row rescaled) only when some row of the warp outgrows it by 2^8
      const bool grow = (mx > m_ref + 8.f) || (m_ref == -INFINITY && mx > -INFINITY);
      float corr = 1.f;
      const bool rescale = __any_sync(0xffffffffu, grow);
      if (rescale) {
        const float m_new = fmaxf(m_ref, mx);
        corr = (m_new == -INFINITY) ? 1.f : fast_exp2(m_ref - m_new);   // 0 for a row that had no key yet
        m_ref = m_new;
        l *= corr;
      }
      const float msafe = (m_ref == -INFINITY) ? 0.f : m_ref;
      uint32_t pk[32];
      float psum = 0.f;
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = fast_exp2(__uint_as_float(sr[c]) - msafe), p1 = fast_exp2(__uint_as_float(sr[c + 1]) - msafe);
        psum += p0 + p1;
        pk[c >> 1] = pack_bf16(p0, p1);
      }
      l += psum;
      // the previous tile's P V product has read P and finished accumulating into O
      if (t > 0) {
        ok = tma::mbar_wait_bounded(&ctl.pv_done, (uint32_t)(t - 1) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (rescale) {
#pragma unroll 1
          for (int cc = 0; cc < 4; cc++) {
            uint32_t o[32];
            tmem_ld32(tm_o + lane_base + cc * 32, o);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int e = 0; e < 32; e++) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
            tmem_st32(tm_o + lane_base + cc * 32, o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
#pragma unroll
      for (int ch = 0; ch < 8; ch++)
        *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) =
            make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      tma::mbar_arrive(&ctl.p_full);
    }
    if (ok) {
      ok = tma::mbar_wait_bounded(&ctl.pv_done, (uint32_t)(nt - 1) & 1u, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      bf16* orow = out + ((size_t)b * Tn + i) * d + h * HD;
#pragma unroll 1
      for (int cc = 0; cc < 4; cc++) {
        uint32_t o[32];
        tmem_ld32(tm_o + lane_base + cc * 32, o);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (i <= i_last) {
#pragma unroll
          for (int v8 = 0; v8 < 4; v8++) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; e++) f[e] = __uint_as_float(o[v8 * 8 + e]) * inv_l;
            store_vec(orow + cc * 32 + v8 * 8, f);
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0 && status) atomicExch(status, STATUS_SWA);
  // (on a wait that ran out, copies already issued still land in this CTA's shared memory: the CTA keeps it for a
  // moment longer than any copy takes)
  if (*abort_flag && fresh && threadIdx.x == 0) {
    const uint64_t t_start = tma::global_ns();
    while (tma::global_ns() - t_start < 200000ull) {}   // 0.2 ms: any copy in flight has long landed
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem_base));
  }
}

int encode_sw128(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                 const cuuint32_t* box) {
  return tma::encode_bf16(map, base, rank, dims, strides, box, true);
}

}  // namespace

extern "C" long long stu_swa_prefill_scratch_elems(int B, int Tn, int H, int hd) {
  if (B <= 0 || Tn <= 0 || H <= 0 || hd != HD) return -1;
  return (long long)B * H * HD * ((Tn + 63) / 64 * 64);
}

// Attention of a prefill that starts at position 0 (bf16, head dimension 128) on the tcgen05 tensor cores; the
// sequences' keys and values then go into the rings and the positions advance by Tn, as stu_swa_forward does.
// vt_scratch: stu_swa_prefill_scratch_elems() bf16 elements, 16-byte aligned (V transposed per head).
extern "C" int stu_swa_prefill_tc5(const void* qkv, void* vt_scratch, void* k_ring, void* v_ring, int* pos,
                                   const float* slopes, void* out, int B, int Tn, int H, int hd, int W, int window,
                                   float softcap, int update_cache, int* status, int dtype, void* stream) {
  if (!qkv || !vt_scratch || !pos || !slopes || !out || (update_cache && (!k_ring || !v_ring))) return STU_ERR_NULL;
  if (dtype != STU_BF16) return STU_ERR_DTYPE;
  if (hd != HD) return STU_ERR_UNSUPPORTED;
  if (B <= 0 || Tn <= 0 || H <= 0 || window < 0 || (update_cache && W < window + 1)) return STU_ERR_SHAPE;
  if (!aligned16(qkv) || !aligned16(vt_scratch) || !aligned16(out)) return STU_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  const int d = H * HD, Tp = (Tn + 63) / 64 * 64;
  v_transpose_kernel<<<dim3(Tp / 64, H, B), 256, 0, st>>>((const bf16*)qkv, (bf16*)vt_scratch, Tn, Tp, H);
  STU_CHECK_LAUNCH();
  CUtensorMap tmQ, tmK, tmV;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)3 * d, (cuuint64_t)Tn, (cuuint64_t)B};
    const cuuint64_t str[2] = {(cuuint64_t)3 * d * 2, (cuuint64_t)Tn * 3 * d * 2};
    const cuuint32_t boxq[3] = {64, BM, 1}, boxk[3] = {64, BN, 1};
    int rc = encode_sw128(&tmQ, qkv, 3, dims, str, boxq);
    if (rc != STU_OK) return rc;
    rc = encode_sw128(&tmK, qkv, 3, dims, str, boxk);
    if (rc != STU_OK) return rc;
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)Tp, (cuuint64_t)B * H * HD};
    const cuuint64_t str[1] = {(cuuint64_t)Tp * 2};
    const cuuint32_t box[2] = {BN, HD};
    int rc = encode_sw128(&tmV, vt_scratch, 2, dims, str, box);
    if (rc != STU_OK) return rc;
  }
  cudaError_t e = cudaFuncSetAttribute(swa_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return (int)e;
  const float scale = 1.0f / sqrtf((float)HD);
  swa_umma_kernel<<<dim3((Tn + BM - 1) / BM, H, B), 192, SMEM_BYTES, st>>>(tmQ, tmK, tmV, pos, slopes, (bf16*)out, Tn,
                                                                           H, window, scale, softcap, status);
  STU_CHECK_LAUNCH();
  if (update_cache) return launch_kv_ring_write_bf16(qkv, k_ring, v_ring, pos, B, Tn, d, W, st);
  return STU_OK;
}
