// Sliding-window attention with ALiBi and tanh soft-capping over a ring-buffer KV cache.
//
// Reference semantics (flash_stu/modules/attention.py:72-101 calling flash_attn_func with causal=True,
// window_size=(w,0), alibi_slopes, softcap): query at absolute position i attends keys j in [i-w, i];
//   score = softcap * tanh(q.k * scale / softcap) - slope_h * (i - j);  out = softmax(score) . V
// The reference keeps every past (k,v) by torch.cat; only the last w+1 can be attended, so the cache
// here is a ring of W = w+1 slots per sequence ([B][W][H*hd]); token t lives in slot t % W.
//
// swa_attend_kernel: one CTA per (32-query tile, head, sequence); eight warps, four queries per warp.
// Key/value tiles of 32 keys are staged in shared memory as fp32 (keys transposed), lane = key for
// the score pass, lane = output dims for the P.V pass, online softmax per query.  Keys at positions
// >= t0 (this call's tokens) come from the qkv activations, older ones from the ring.
// kv_ring_write_kernel then stores this call's last W tokens into the ring and advances the positions.
#include "common.cuh"

constexpr int AT_QT = 32;   // queries per CTA
constexpr int AT_KT = 32;   // keys per tile
constexpr int AT_MAXHD = 128;

template <typename T>
__global__ void __launch_bounds__(256) swa_attend_kernel(const T* __restrict__ qkv, const T* __restrict__ k_ring,
                                                         const T* __restrict__ v_ring, const int* __restrict__ pos,
                                                         const float* __restrict__ slopes, T* __restrict__ out,
                                                         int Tn, int H, int hd, int W, int window, float scale,
                                                         float softcap) {
  extern __shared__ __align__(16) float at_smem[];
  const int hdp_ = (hd + 31) & ~31;
  float (*Qs)[AT_QT] = reinterpret_cast<float (*)[AT_QT]>(at_smem);                          // [dim][query]
  float (*Kt)[AT_KT + 1] = reinterpret_cast<float (*)[AT_KT + 1]>(at_smem + hdp_ * AT_QT);     // [dim][key]
  float* Vs = at_smem + hdp_ * AT_QT + hdp_ * (AT_KT + 1);                                    // [key][hdp]
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * AT_QT;
  const int d = H * hd;
  const int t0 = pos[2 * b];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hdp = (hd + 31) & ~31;
  const int dpl = hdp >> 5;  // dims per lane in the P.V pass (<= 4)
  // stage the query tile, pre-scaled
  for (int e = threadIdx.x; e < AT_QT * hdp; e += 256) {
    int qi = e / hdp, dd = e % hdp;
    int tq = q0 + qi;
    float v = 0.f;
    if (tq < Tn && dd < hd) v = Elem<T>::to_f(qkv[((size_t)b * Tn + tq) * 3 * d + h * hd + dd]) * scale;
    Qs[dd][qi] = v;
  }
  float mrun[4], lrun[4], acc[4][4];
#pragma unroll
  for (int u = 0; u < 4; u++) {
    mrun[u] = -INFINITY;
    lrun[u] = 0.f;
#pragma unroll
    for (int e = 0; e < 4; e++) acc[u][e] = 0.f;
  }
  const float slope = slopes[h];
  const int i_first = t0 + q0, i_last = t0 + min(q0 + AT_QT, Tn) - 1;  // absolute query positions of the tile
  const int j_lo = max(0, i_first - window), j_hi = i_last;
  for (int jt = j_lo; jt <= j_hi; jt += AT_KT) {
    __syncthreads();
    // stage keys jt..jt+31
    for (int e = threadIdx.x; e < AT_KT * hdp; e += 256) {
      int kj = e / hdp, dd = e % hdp;
      int j = jt + kj;
      float kv = 0.f, vv = 0.f;
      if (j <= j_hi && dd < hd) {
        if (j >= t0) {
          const T* base = qkv + ((size_t)b * Tn + (j - t0)) * 3 * d + h * hd + dd;
          kv = Elem<T>::to_f(base[d]);
          vv = Elem<T>::to_f(base[2 * d]);
        } else {
          size_t off = ((size_t)b * W + (j % W)) * d + h * hd + dd;
          kv = Elem<T>::to_f(k_ring[off]);
          vv = Elem<T>::to_f(v_ring[off]);
        }
      }
      Kt[dd][kj] = kv;
      Vs[kj * hdp + dd] = vv;
    }
    __syncthreads();
    // scores: lane = key, four queries per warp
    const int j = jt + lane;
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    for (int dd = 0; dd < hd; dd++) {
      float kv = Kt[dd][lane];
      float4 q4 = *reinterpret_cast<const float4*>(&Qs[dd][warp * 4]);
      s[0] = fmaf(q4.x, kv, s[0]);
      s[1] = fmaf(q4.y, kv, s[1]);
      s[2] = fmaf(q4.z, kv, s[2]);
      s[3] = fmaf(q4.w, kv, s[3]);
    }
    float pr[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int tq = q0 + warp * 4 + u, i = t0 + tq;
      const bool valid = (tq < Tn) && (j <= i) && (j >= i - window) && (j <= j_hi);
      float sc = s[u];
      if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
      sc -= slope * (float)(i - j);
      sc = valid ? sc : -INFINITY;
      const float mnew = fmaxf(mrun[u], warp_max(sc));
      const float corr = (mnew == -INFINITY) ? 1.f : __expf(mrun[u] - mnew);
      const float p = valid ? __expf(sc - mnew) : 0.f;
      lrun[u] = lrun[u] * corr + warp_sum(p);
      mrun[u] = mnew;
      pr[u] = p;
#pragma unroll
      for (int e = 0; e < 4; e++) acc[u][e] *= corr;
    }
    // P.V: lane owns dims lane + 32*e
    for (int kj = 0; kj < AT_KT; kj++) {
      float pv[4];
#pragma unroll
      for (int u = 0; u < 4; u++) pv[u] = __shfl_sync(0xffffffffu, pr[u], kj);
#pragma unroll
      for (int e = 0; e < 4; e++) {
        if (e < dpl) {
          const float vv = Vs[kj * hdp + lane + 32 * e];
#pragma unroll
          for (int u = 0; u < 4; u++) acc[u][e] = fmaf(pv[u], vv, acc[u][e]);
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < 4; u++) {
    const int tq = q0 + warp * 4 + u;
    if (tq < Tn) {
      const float inv = lrun[u] > 0.f ? 1.f / lrun[u] : 0.f;
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int dd = lane + 32 * e;
        if (e < dpl && dd < hd) out[((size_t)b * Tn + tq) * d + h * hd + dd] = Elem<T>::from_f(acc[u][e] * inv);
      }
    }
  }
}

// Store the last min(Tn, W) tokens of this call into the ring; the last CTA advances pos by Tn.
template <typename T>
__global__ void __launch_bounds__(256) kv_ring_write_kernel(const T* __restrict__ qkv, T* __restrict__ k_ring,
                                                            T* __restrict__ v_ring, int* __restrict__ pos, int B,
                                                            int Tn, int d, int W) {
  const int b = blockIdx.y;
  const int t0 = pos[2 * b];
  const int first = max(0, Tn - W);
  const int tq = first + blockIdx.x;
  if (tq < Tn) {
    const int slot = (t0 + tq) % W;
    const T* src = qkv + ((size_t)b * Tn + tq) * 3 * d;
    T* kd = k_ring + ((size_t)b * W + slot) * d;
    T* vd = v_ring + ((size_t)b * W + slot) * d;
    for (int e = threadIdx.x; e < d; e += 256) {
      kd[e] = src[d + e];
      vd[e] = src[2 * d + e];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int total = gridDim.x * gridDim.y;
    if (atomicAdd(&pos[1], 1) == total - 1) {
      pos[1] = 0;
      for (int i = 0; i < B; i++) pos[2 * i] += Tn;
      __threadfence();
    }
  }
}

// ------------------------------------------------------------------------------------------------
// One new token per sequence (cached decode): memory-bound, one CTA per (head, sequence).
// A key (or value) row of one head is hd elements = LPK lanes x 16 bytes, so a warp-wide load fetches 32/LPK
// keys; each group of LPK lanes keeps its own online-softmax state (running maximum, sum, weighted values of
// its 16-byte slice) over the keys it meets, with only the LPK-lane dot-product reduction per key, and the
// 8 * 32/LPK groups of the CTA are merged once at the end through shared memory.  The new token's key and
// value come from the qkv activations; the CTA then stores them into ring slot t % W for its head (no one reads
// that slot in this launch: it held key t-W, outside the window), and the last CTA advances the positions.
constexpr int DEC_U = 4;  // warp-wide key copies (and as many value copies) per round; two rounds in flight
constexpr int DEC_RING_BYTES = 2 * DEC_U * 2 * 256 * 16;

template <typename T> struct Vec16 {
  uint4 raw;
  __device__ __forceinline__ void unpack(float* f) const;
};
template <> __device__ __forceinline__ void Vec16<float>::unpack(float* f) const {
  f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
}
template <> __device__ __forceinline__ void Vec16<bf16>::unpack(float* f) const {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <typename T, int LPK>
__global__ void __launch_bounds__(256) swa_decode_kernel(const T* __restrict__ qkv, T* __restrict__ k_ring,
                                                         T* __restrict__ v_ring, int* __restrict__ pos,
                                                         const float* __restrict__ slopes, T* __restrict__ out, int B,
                                                         int H, int W, int window, float scale, float softcap,
                                                         int update_cache) {
  constexpr int VPL = 16 / sizeof(T);   // values per lane
  constexpr int HD = LPK * VPL;         // head dimension
  constexpr int KPW = 32 / LPK;         // keys per warp-wide load
  constexpr int NG = 8 * KPW;           // softmax groups per CTA
  __shared__ float s_m[NG], s_l[NG];
  __shared__ float s_acc[NG][HD];
  const int h = blockIdx.x, b = blockIdx.y;
  const int d = H * HD;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPK, grp = lane / LPK;
  pdl_trigger();   // launched with the programmatic attribute: resident while the qkv projection drains
  pdl_wait();
  const int t0 = pos[2 * b];
  if (update_cache) {
    // Every CTA has read its position before it arrives here; the last one to arrive moves all positions on.  Doing
    // this first (instead of after the output is stored) takes the fence, the atomic and the serial update off the
    // end of the kernel, where nothing could hide them.
    __syncthreads();
    if (threadIdx.x == 0) {
      const int total = gridDim.x * gridDim.y;
      if (atomicAdd(&pos[1], 1) == total - 1) {
        pos[1] = 0;
        for (int i = 0; i < B; i++) pos[2 * i] += 1;
      }
    }
  }
  const T* cur = qkv + (size_t)b * 3 * d + h * HD;   // q | k | v of the new token, this head
  float qv[VPL];
  {
    Vec16<T> q;
    q.raw = *reinterpret_cast<const uint4*>(cur + sub * VPL);
    q.unpack(qv);
#pragma unroll
    for (int e = 0; e < VPL; e++) qv[e] *= scale;
  }
  const float slope = slopes[h];
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const int j_lo = max(0, t0 - window);
  const int nkeys = t0 - j_lo + 1;  // the new token included
  float m = -INFINITY, l = 0.f, acc[VPL];
#pragma unroll
  for (int e = 0; e < VPL; e++) acc[e] = 0.f;
  const size_t ring_b = (size_t)b * W;
  // Keys and values travel global -> shared memory by 16-byte asynchronous copies, two rounds of DEC_U keys (and
  // values) in flight per thread: every thread copies into slots of its own and reads them back itself, so the ring
  // needs no barrier, and the bytes in flight are bounded by shared memory (64 KB per CTA), not by registers.
  extern __shared__ uint4 dec_ring[];   // [2 stages][DEC_U][key | value][256 threads]
  const int first = warp * KPW;
  const int niter = first < nkeys ? (nkeys - first + 8 * KPW * DEC_U - 1) / (8 * KPW * DEC_U) : 0;   // warp-uniform
  auto issue = [&](int it, int stage) {
    if (it < niter) {
#pragma unroll
      for (int u = 0; u < DEC_U; u++) {
        const int kk = first + it * 8 * KPW * DEC_U + u * 8 * KPW + grp;
        const bool ok = kk < nkeys;
        const int j = j_lo + kk;
        const T *ks, *vs;
        if (ok && j == t0) {   // the new token's key and value come from the qkv activations
          ks = cur + d + sub * VPL;
          vs = cur + 2 * d + sub * VPL;
        } else {
          const size_t off = (ring_b + (size_t)(ok ? j % W : 0)) * d + h * HD + sub * VPL;
          ks = k_ring + off;
          vs = v_ring + off;
        }
        const unsigned nbytes = ok ? 16u : 0u;   // 0: the slot is filled with zeros
        const unsigned kd = (unsigned)__cvta_generic_to_shared(&dec_ring[((stage * DEC_U + u) * 2 + 0) * 256 + threadIdx.x]);
        const unsigned vd = (unsigned)__cvta_generic_to_shared(&dec_ring[((stage * DEC_U + u) * 2 + 1) * 256 + threadIdx.x]);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kd), "l"(ks), "r"(nbytes) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vd), "l"(vs), "r"(nbytes) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");   // one group per call, empty past the end
  };
  issue(0, 0);
  issue(1, 1);
  for (int it = 0; it < niter; it++) {  // warp-uniform
    const int base = first + it * 8 * KPW * DEC_U;
    const int stage = it & 1;
    asm volatile("cp.async.wait_group 1;" ::: "memory");   // round `it` has landed, round it + 1 may be in flight
    Vec16<T> kr[DEC_U], vr[DEC_U];
#pragma unroll
    for (int u = 0; u < DEC_U; u++) {
      kr[u].raw = dec_ring[((stage * DEC_U + u) * 2 + 0) * 256 + threadIdx.x];
      vr[u].raw = dec_ring[((stage * DEC_U + u) * 2 + 1) * 256 + threadIdx.x];
    }
    issue(it + 2, stage);   // refill the slots just read
    // scores of the DEC_U keys of this group first, then ONE rescale of the running sums for all of them
    float sc[DEC_U];
#pragma unroll
    for (int u = 0; u < DEC_U; u++) {
      const int kk = base + u * 8 * KPW + grp;
      float kf[VPL];
      kr[u].unpack(kf);
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < VPL; e++) dot = fmaf(qv[e], kf[e], dot);
#pragma unroll
      for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (softcap > 0.f) {
        // bf16: hardware tanh, relative error 2^-11, below the bf16 rounding of the output (as in the prefill kernel)
        float th;
        if (sizeof(T) == 2) asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(dot * inv_cap));
        else th = tanhf(dot * inv_cap);
        dot = softcap * th;
      }
      sc[u] = (kk < nkeys) ? dot - slope * (float)(nkeys - 1 - kk) : -INFINITY;   // ALiBi: i - j
    }
    float mnew = m;
#pragma unroll
    for (int u = 0; u < DEC_U; u++) mnew = fmaxf(mnew, sc[u]);
    if (mnew > -INFINITY) {
      const float corr = __expf(m - mnew);   // 0 while the group has seen no key yet
      l *= corr;
#pragma unroll
      for (int e = 0; e < VPL; e++) acc[e] *= corr;
#pragma unroll
      for (int u = 0; u < DEC_U; u++) {
        const float pw = __expf(sc[u] - mnew);   // 0 for a key past the end
        float vf[VPL];
        vr[u].unpack(vf);
        l += pw;
#pragma unroll
        for (int e = 0; e < VPL; e++) acc[e] = fmaf(pw, vf[e], acc[e]);
      }
      m = mnew;
    }
  }
  const int gidx = warp * KPW + grp;
  if (sub == 0) {
    s_m[gidx] = m;
    s_l[gidx] = l;
  }
#pragma unroll
  for (int e = 0; e < VPL; e++) s_acc[gidx][sub * VPL + e] = acc[e];
  if (update_cache) {  // this head's slice of the new key and value
    const size_t slot = (ring_b + (size_t)(t0 % W)) * d + h * HD;
    if (threadIdx.x < LPK)
      *reinterpret_cast<uint4*>(k_ring + slot + threadIdx.x * VPL) =
          *reinterpret_cast<const uint4*>(cur + d + threadIdx.x * VPL);
    else if (threadIdx.x < 2 * LPK)
      *reinterpret_cast<uint4*>(v_ring + slot + (threadIdx.x - LPK) * VPL) =
          *reinterpret_cast<const uint4*>(cur + 2 * d + (threadIdx.x - LPK) * VPL);
  }
  __syncthreads();
  if (threadIdx.x < HD) {
    float M = -INFINITY;
#pragma unroll
    for (int g2 = 0; g2 < NG; g2++) M = fmaxf(M, s_m[g2]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int g2 = 0; g2 < NG; g2++) {
      const float mg = s_m[g2];
      if (mg > -INFINITY) {
        const float w = __expf(mg - M);
        num = fmaf(s_acc[g2][threadIdx.x], w, num);
        den = fmaf(s_l[g2], w, den);
      }
    }
    out[(size_t)b * d + h * HD + threadIdx.x] = Elem<T>::from_f(num / den);
  }
}

template <typename T>
static bool launch_swa_decode(const void* qkv, void* k_ring, void* v_ring, int* pos, const float* slopes, void* out,
                              int B, int H, int hd, int W, int window, float scale, float softcap, int update_cache,
                              cudaStream_t st) {
  constexpr int VPL = 16 / sizeof(T);
  if (hd % VPL || !aligned16(qkv) || !aligned16(k_ring) || !aligned16(v_ring) || !aligned16(out)) return false;
  dim3 grid(H, B);
#define STU_SWA_DEC(LPK_)                                                                                        \
  cudaFuncSetAttribute(swa_decode_kernel<T, LPK_>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_RING_BYTES);    \
  launch_maybe_overlapped(swa_decode_kernel<T, LPK_>, grid, dim3(256), DEC_RING_BYTES, st, true, (const T*)qkv,     \
                          (T*)k_ring, (T*)v_ring, pos, slopes, (T*)out, B, H, W, window, scale, softcap,            \
                          update_cache)
  switch (hd / VPL) {
    case 4: STU_SWA_DEC(4); return true;
    case 8: STU_SWA_DEC(8); return true;
    case 16: STU_SWA_DEC(16); return true;
    case 32: STU_SWA_DEC(32); return true;
  }
#undef STU_SWA_DEC
  return false;
}

// ------------------------------------------------------------------------------------------------
// Prefill (many new tokens), bf16, head dimension 64 or 128: tensor-core kernel in the flash-attention form.
// One CTA = 64 queries of one head of one sequence, four warps of 16 query rows.  Per 64-key tile:
//   S = Q K^T (mma.sync m16n8k16, Q fragments resident in registers, K through ldmatrix from a swizzled tile),
//   soft-capping, ALiBi, window/causal mask, online softmax in the exp2 domain, P repacked from the accumulator
//   layout straight into A fragments, O += P V (V through ldmatrix.trans).
// Only the key tiles that intersect [i - w, i] for some query of the CTA are visited (17-18 tiles for w = 1024
// instead of T/64).  Keys of this call come from the qkv activations, older ones from the ring.
constexpr int FA_BM = 64, FA_BN = 64;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16_zfill(void* smem_ptr, const void* gptr, bool valid) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a), "l"(gptr), "r"(n) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int HD>
__global__ void __launch_bounds__(128) swa_flash_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ k_ring,
                                                        const bf16* __restrict__ v_ring, const int* __restrict__ pos,
                                                        const float* __restrict__ slopes, bf16* __restrict__ out,
                                                        int Tn, int H, int W, int window, float scale, float softcap) {
  constexpr int CH = HD / 8;          // 16-byte chunks per row
  constexpr int KS = HD / 16;         // k-steps of the score product
  extern __shared__ __align__(128) unsigned char fa_smem[];
  bf16* Qs = reinterpret_cast<bf16*>(fa_smem);             // [64][HD], chunk index XOR (row & 7)
  bf16* KV = Qs + FA_BM * HD;                              // two stages of [K tile][V tile]
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * FA_BM;
  const int d = H * HD;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, q = lane & 3;
  const int t0 = pos[2 * b];
  auto sw = [](int row, int chunk) { return row * CH + (chunk ^ (row & 7)); };  // in 16-byte units

  // ---- stage Q (rows beyond Tn are zero)
  for (int idx = tid; idx < FA_BM * CH; idx += 128) {
    const int row = idx / CH, c = idx - row * CH;
    const int tq = q0 + row;
    const bf16* src = qkv + ((size_t)b * Tn + (tq < Tn ? tq : 0)) * 3 * d + h * HD + c * 8;
    cp_async16_zfill(Qs + sw(row, c) * 8, src, tq < Tn);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ks++) {
    const int row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
    ldmatrix_x4(qf[ks], Qs + sw(row, ks * 2 + (lane >> 4)) * 8);
  }

  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; n++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[n][e] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};   // rows g and g+8, exp2 domain
  const float slope = slopes[h];
  const float LOG2E = 1.4426950408889634f;
  const int i_first = t0 + q0, i_last = t0 + min(q0 + FA_BM, Tn) - 1;
  const int j_lo = max(0, i_first - window), j_hi = i_last;
  const int irow0 = t0 + q0 + warp * 16 + g;   // absolute position of row g (row g+8: +8)

  auto load_tile = [&](int jt, int stage) {
    bf16* Kd = KV + (size_t)stage * 2 * FA_BN * HD;
    bf16* Vd = Kd + FA_BN * HD;
    for (int idx = tid; idx < FA_BN * CH; idx += 128) {
      const int row = idx / CH, c = idx - row * CH;
      const int j = jt + row;
      const bool ok = j <= j_hi;
      const bf16 *ksrc, *vsrc;
      if (ok && j >= t0) {
        ksrc = qkv + ((size_t)b * Tn + (j - t0)) * 3 * d + d + h * HD + c * 8;
        vsrc = ksrc + d;
      } else {
        const size_t off = ((size_t)b * W + (size_t)((ok ? j : 0) % W)) * d + h * HD + c * 8;
        ksrc = k_ring + off;
        vsrc = v_ring + off;
      }
      cp_async16_zfill(Kd + sw(row, c) * 8, ksrc, ok);
      cp_async16_zfill(Vd + sw(row, c) * 8, vsrc, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // two-stage pipeline: the next key tile is in flight while the current one is multiplied
  load_tile(j_lo, 0);
  int stage = 0;
  for (int jt = j_lo; jt <= j_hi; jt += FA_BN, stage ^= 1) {
    if (jt + FA_BN <= j_hi) {
      load_tile(jt + FA_BN, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const bf16* Ks = KV + (size_t)stage * 2 * FA_BN * HD;
    const bf16* Vs = Ks + FA_BN * HD;

    // ---- S = Q K^T : 16 rows x 64 keys per warp
    float sacc[FA_BN / 8][4];
#pragma unroll
    for (int n = 0; n < FA_BN / 8; n++)
#pragma unroll
      for (int e = 0; e < 4; e++) sacc[n][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
#pragma unroll
      for (int np = 0; np < FA_BN / 16; np++) {   // two key n-tiles per ldmatrix.x4
        uint32_t kf[4];
        const int krow = np * 16 + (lane & 7) + 8 * (lane >> 4);
        ldmatrix_x4(kf, Ks + sw(krow, ks * 2 + ((lane >> 3) & 1)) * 8);
        mma_16816(sacc[2 * np], qf[ks], kf[0], kf[1]);
        mma_16816(sacc[2 * np + 1], qf[ks], kf[2], kf[3]);
      }
    }
    // ---- soft-capping, ALiBi, mask, online softmax (exp2 domain)
    float mnew[2] = {mrow[0], mrow[1]};
    // interior tile: every (query, key) pair of this warp's 16 rows x 64 keys lies inside the window (warp-uniform)
    const int iw0 = t0 + q0 + warp * 16;
    const bool interior = (jt + FA_BN - 1 <= iw0) && (jt >= iw0 + 15 - window) && (jt + FA_BN - 1 <= j_hi) &&
                          (iw0 + 15 <= i_last);
    const float cap2 = 2.f / softcap;
#pragma unroll
    for (int n = 0; n < FA_BN / 8; n++) {
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int r = e >> 1;                           // 0: row g, 1: row g+8
        const int i = irow0 + 8 * r;
        const int j = jt + n * 8 + 2 * q + (e & 1);
        float sc = sacc[n][e] * scale;
        if (softcap > 0.f) {   // softcap * tanh(sc / softcap); tanh.approx: relative error 2^-11, below P's bf16 rounding
          float th;
          asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(sc * 0.5f * cap2));
          sc = softcap * th;
        }
        sc = (sc - slope * (float)(i - j)) * LOG2E;
        if (!interior) {
          const bool valid = (j <= i) && (j >= i - window) && (j <= j_hi) && (i <= i_last);
          sc = valid ? sc : -INFINITY;
        }
        sacc[n][e] = sc;
        mnew[r] = fmaxf(mnew[r], sc);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mnew[r] = fmaxf(mnew[r], __shfl_xor_sync(0xffffffffu, mnew[r], 1));
      mnew[r] = fmaxf(mnew[r], __shfl_xor_sync(0xffffffffu, mnew[r], 2));
    }
    float corr[2], msafe[2], psum[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; r++) {
      msafe[r] = (mnew[r] == -INFINITY) ? 0.f : mnew[r];   // a row with no key yet keeps exp2(-inf) = 0 everywhere
      corr[r] = exp2f(mrow[r] - msafe[r]);
      mrow[r] = mnew[r];
    }
    uint32_t pf[FA_BN / 16][4];
#pragma unroll
    for (int n = 0; n < FA_BN / 8; n++) {
      const float p0 = exp2f(sacc[n][0] - msafe[0]), p1 = exp2f(sacc[n][1] - msafe[0]);
      const float p2 = exp2f(sacc[n][2] - msafe[1]), p3 = exp2f(sacc[n][3] - msafe[1]);
      psum[0] += p0 + p1;
      psum[1] += p2 + p3;
      // accumulator layout of two adjacent key n-tiles = A fragment of one k16 step
      pf[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int r = 0; r < 2; r++) lrow[r] = lrow[r] * corr[r] + psum[r];   // per-lane partial sums, reduced at the end
#pragma unroll
    for (int n = 0; n < HD / 8; n++) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < FA_BN / 16; kk++) {
#pragma unroll
      for (int np = 0; np < HD / 16; np++) {      // two dim n-tiles per ldmatrix.x4.trans
        uint32_t vf[4];
        const int vrow = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        ldmatrix_x4_trans(vf, Vs + sw(vrow, np * 2 + (lane >> 4)) * 8);
        mma_16816(o[2 * np], pf[kk], vf[0], vf[1]);
        mma_16816(o[2 * np + 1], pf[kk], vf[2], vf[3]);
      }
    }
    __syncthreads();   // this stage is refilled by the load issued at the top of the next iteration
  }
  // ---- normalise and store
#pragma unroll
  for (int r = 0; r < 2; r++) {
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; r++) {
    const int tq = q0 + warp * 16 + g + 8 * r;
    if (tq < Tn) {
      const float inv = lrow[r] > 0.f ? 1.f / lrow[r] : 0.f;
      bf16* dst = out + ((size_t)b * Tn + tq) * d + h * HD + 2 * q;
#pragma unroll
      for (int n = 0; n < HD / 8; n++)
        *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
    }
  }
}

// qkv: [B, Tn, 3d] activations of this call (c_attn output); rings: [B, W, d]; pos: [B,2] int32 device
// (column 0 = tokens already cached, column 1 of row 0 = arrival counter, must be 0); out: [B, Tn, d].
// ring write + position advance after a prefill whose attention ran elsewhere (attention_umma.cu)
int launch_kv_ring_write_bf16(const void* qkv, void* k_ring, void* v_ring, int* pos, int B, int Tn, int d, int W,
                              cudaStream_t st) {
  dim3 g2(Tn < W ? Tn : W, B);
  kv_ring_write_kernel<bf16><<<g2, 256, 0, st>>>((const bf16*)qkv, (bf16*)k_ring, (bf16*)v_ring, pos, B, Tn, d, W);
  STU_CHECK_LAUNCH();
  return STU_OK;
}

extern "C" int stu_swa_forward(const void* qkv, void* k_ring, void* v_ring, int* pos, const float* slopes, void* out,
                               int B, int Tn, int H, int hd, int W, int window, float softcap, int update_cache,
                               int dtype, void* stream) {
  if (!qkv || !k_ring || !v_ring || !pos || !slopes || !out) return STU_ERR_NULL;
  if (B <= 0 || Tn <= 0 || H <= 0 || hd <= 0 || hd > AT_MAXHD || W <= 0 || window < 0 || W < window + 1)
    return STU_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const float scale = 1.0f / sqrtf((float)hd);
  if (Tn == 1) {  // cached decode: the memory-bound kernel (also stores the new key/value and advances pos)
    bool done = false;
    if (dtype == STU_F32)
      done = launch_swa_decode<float>(qkv, k_ring, v_ring, pos, slopes, out, B, H, hd, W, window, scale, softcap,
                                      update_cache, st);
    else if (dtype == STU_BF16)
      done = launch_swa_decode<bf16>(qkv, k_ring, v_ring, pos, slopes, out, B, H, hd, W, window, scale, softcap,
                                     update_cache, st);
    else
      return STU_ERR_DTYPE;
    if (done) {
      STU_CHECK_LAUNCH();
      return STU_OK;
    }
  }
  dim3 grid((Tn + AT_QT - 1) / AT_QT, H, B);
  dim3 g2(Tn < W ? Tn : W, B);
  const int hdp = (hd + 31) & ~31;
  const size_t smem = (size_t)(hdp * AT_QT + hdp * (AT_KT + 1) + AT_KT * hdp) * sizeof(float);
  cudaError_t ea = cudaFuncSetAttribute(swa_attend_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  if (ea == cudaSuccess)
    ea = cudaFuncSetAttribute(swa_attend_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  if (ea != cudaSuccess) return (int)ea;
  if (dtype == STU_F32) {
    swa_attend_kernel<float><<<grid, 256, smem, st>>>((const float*)qkv, (const float*)k_ring, (const float*)v_ring, pos,
                                                   slopes, (float*)out, Tn, H, hd, W, window, scale, softcap);
    STU_CHECK_LAUNCH();
    if (update_cache)
      kv_ring_write_kernel<float><<<g2, 256, 0, st>>>((const float*)qkv, (float*)k_ring, (float*)v_ring, pos, B, Tn,
                                                      H * hd, W);
  } else if (dtype == STU_BF16) {
    const bool flash_ok = (hd == 64 || hd == 128) && aligned16(qkv) && aligned16(k_ring) && aligned16(v_ring) &&
                          aligned16(out);
    if (flash_ok) {
      dim3 fg((Tn + FA_BM - 1) / FA_BM, H, B);
      const size_t fsm = (size_t)(FA_BM + 4 * FA_BN) * hd * sizeof(bf16);
      if (hd == 128) {
        ea = cudaFuncSetAttribute(swa_flash_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fsm);
        if (ea != cudaSuccess) return (int)ea;
        swa_flash_kernel<128><<<fg, 128, fsm, st>>>((const bf16*)qkv, (const bf16*)k_ring, (const bf16*)v_ring, pos,
                                                    slopes, (bf16*)out, Tn, H, W, window, scale, softcap);
      } else {
        ea = cudaFuncSetAttribute(swa_flash_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fsm);
        if (ea != cudaSuccess) return (int)ea;
        swa_flash_kernel<64><<<fg, 128, fsm, st>>>((const bf16*)qkv, (const bf16*)k_ring, (const bf16*)v_ring, pos,
                                                   slopes, (bf16*)out, Tn, H, W, window, scale, softcap);
      }
    } else
    swa_attend_kernel<bf16><<<grid, 256, smem, st>>>((const bf16*)qkv, (const bf16*)k_ring, (const bf16*)v_ring, pos,
                                                  slopes, (bf16*)out, Tn, H, hd, W, window, scale, softcap);
    STU_CHECK_LAUNCH();
    if (update_cache)
      kv_ring_write_kernel<bf16><<<g2, 256, 0, st>>>((const bf16*)qkv, (bf16*)k_ring, (bf16*)v_ring, pos, B, Tn,
                                                     H * hd, W);
  } else {
    return STU_ERR_DTYPE;
  }
  STU_CHECK_LAUNCH();
  return STU_OK;
}
