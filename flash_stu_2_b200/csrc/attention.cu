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

// qkv: [B, Tn, 3d] activations of this call (c_attn output); rings: [B, W, d]; pos: [B,2] int32 device
// (column 0 = tokens already cached, column 1 of row 0 = arrival counter, must be 0); out: [B, Tn, d].
extern "C" int stu_swa_forward(const void* qkv, void* k_ring, void* v_ring, int* pos, const float* slopes, void* out,
                               int B, int Tn, int H, int hd, int W, int window, float softcap, int update_cache,
                               int dtype, void* stream) {
  if (!qkv || !k_ring || !v_ring || !pos || !slopes || !out) return STU_ERR_NULL;
  if (B <= 0 || Tn <= 0 || H <= 0 || hd <= 0 || hd > AT_MAXHD || W <= 0 || window < 0 || W < window + 1)
    return STU_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const float scale = 1.0f / sqrtf((float)hd);
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
