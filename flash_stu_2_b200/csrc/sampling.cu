// Next-token selection from the last-position logits (reference flash_stu/model.py:268-299):
//   z = clamp(logits / temperature, -1e4, 1e4)  (division rounded to the logits dtype)
//   top-k: keep z >= k-th largest (ties kept); top-p: sort kept descending (ties by index), drop an
//   entry when the probability mass ranked before it exceeds top_p; then argmax (greedy) or a draw.
// The reference draws with torch.multinomial; here one uniform u in [0,1) per sequence selects the
// first kept vocabulary index whose running sum of exp(z - max) (vocabulary order) exceeds u * total,
// which is reproducible across devices.
// One CTA of 1024 threads per sequence.  The scaled logits of the row are computed once, in the argmax pass, and kept
// as order-preserving 32-bit keys in shared memory when the vocabulary fits (<= 52 k entries), so the later passes
// neither re-read the logits nor repeat the division.  top-k uses a 4-pass radix select over those keys;
// when top-k is given the (<= 1024) survivors are gathered, bitonic-sorted in shared memory and the
// nucleus cut and the draw are made on that list, otherwise the draw scans the whole vocabulary.
#include <stdlib.h>

#include "common.cuh"

constexpr int SP_T = 1024;
constexpr int SP_CAND = 1024;

__device__ __forceinline__ uint32_t ord_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {   // inverse of ord_key
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
constexpr int SP_CACHE_MAX = 50 * 1024 + 512;   // vocabulary entries whose keys fit beside the other shared arrays
constexpr int SP_SUBH = 16;                     // radix histograms per CTA (one per pair of warps), two 16-bit bins per word

template <typename T> __device__ __forceinline__ float scaled_logit(const T* row, int i, float temperature) {
  float z = round_to<T>(__fdiv_rn(Elem<T>::to_f(row[i]), temperature));
  return fminf(fmaxf(z, -1e4f), 1e4f);
}

template <typename T>
__global__ void __launch_bounds__(SP_T) sample_kernel(const T* __restrict__ logits, long long ld, int V,
                                                      float temperature, int top_k, float top_p, int do_sample,
                                                      const float* __restrict__ uniforms, long long* __restrict__ out,
                                                      long long out_stride, int* __restrict__ status, int cache,
                                                      int variant) {
  extern __shared__ uint32_t s_key[];   // [V] when cache
  __shared__ unsigned int s_sub[SP_SUBH][128];
  __shared__ float s_val[SP_CAND];
  __shared__ int s_idx[SP_CAND];
  __shared__ unsigned int s_hist[256];
  __shared__ float s_red[32];
  __shared__ int s_redi[32];
  __shared__ unsigned int s_prefix, s_need, s_count;
  __shared__ int s_choice;
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* row = logits + (size_t)b * ld;

  // ---- argmax (lowest index among ties); also the fallback result
  float best = -INFINITY;
  int besti = V;
  int saw_nan = 0;
  for (int i = tid; i < V; i += SP_T) {
    float z = scaled_logit(row, i, temperature);
    saw_nan |= isnan(Elem<T>::to_f(row[i])) ? 1 : 0;   // (the clamp inside scaled_logit would hide it)
    if (cache) s_key[i] = ord_key(z);
    if (z > best || (z == best && i < besti)) { best = z; besti = i; }
  }
  saw_nan = __syncthreads_or(saw_nan);
  // scaled logit of entry i for the later passes
  auto zval = [&](int i) { return cache ? key_value(s_key[i]) : scaled_logit(row, i, temperature); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
  }
  if (lane == 0) { s_red[warp] = best; s_redi[warp] = besti; }
  __syncthreads();
  if (warp == 0) {
    best = s_red[lane]; besti = s_redi[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
    }
    if (lane == 0) { s_red[0] = best; s_redi[0] = besti; }
  }
  __syncthreads();
  const float zmax = s_red[0];
  const int imax = s_redi[0];
  if (!do_sample) {
    if (tid == 0) out[(size_t)b * out_stride] = imax < V ? imax : 0;
    return;
  }
  const float u = uniforms[b];
  if (saw_nan) {
    // a NaN logit makes the reference's softmax NaN everywhere and it falls back to a uniformly random token
    // (flash_stu/model.py:293-296); here the row's uniform picks it
    if (tid == 0) out[(size_t)b * out_stride] = min(V - 1, (int)(u * (float)V));
    return;
  }

  // ---- radix select: key of the need-th largest scaled logit (4 passes of 8 bits); all threads call it
  auto select_kth = [&](unsigned need_total) -> unsigned {
    if (tid == 0) { s_prefix = 0; s_need = need_total; }
    for (int pass = 0; pass < 4; pass++) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) s_hist[tid] = 0;
      for (int i = tid; i < SP_SUBH * 128; i += SP_T) (&s_sub[0][0])[i] = 0;
      __syncthreads();
      const unsigned prefix = s_prefix;
      const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      // logits share their sign and exponent bytes, so almost every key of a pass lands in one or two bins.  Each
      // pair of warps counts into a histogram of its own (16-bit counters, two per word: a row has fewer than
      // 65536 entries), which are summed afterwards; with one shared histogram the 32 warps queue on one counter.
      unsigned int* sub = s_sub[warp >> 1];
      for (int base = 0; base < V; base += SP_T) {
        const int i = base + tid;
        unsigned bin = 0xffffffffu;
        if (i < V) {
          const unsigned key = cache ? s_key[i] : ord_key(scaled_logit(row, i, temperature));
          if ((key & mask) == prefix) bin = (key >> shift) & 255u;
        }
        if (variant == 0) {
          const unsigned peers = __match_any_sync(0xffffffffu, bin);
          if (bin != 0xffffffffu && lane == __ffs(peers) - 1) atomicAdd(&s_hist[bin], (unsigned)__popc(peers));
        } else if (variant == 1) {
          if (bin != 0xffffffffu) atomicAdd(&sub[bin >> 1], 1u << (16 * (bin & 1)));
        } else {
          const unsigned peers = __match_any_sync(0xffffffffu, bin);
          if (bin != 0xffffffffu && lane == __ffs(peers) - 1)
            atomicAdd(&sub[bin >> 1], (unsigned)__popc(peers) << (16 * (bin & 1)));
        }
      }
      __syncthreads();
      if (variant != 0 && tid < 256) {
        unsigned c = 0;
#pragma unroll
        for (int h = 0; h < SP_SUBH; h++) c += (s_sub[h][tid >> 1] >> (16 * (tid & 1))) & 0xffffu;
        s_hist[tid] = c;
      }
      __syncthreads();
      // the bin that holds the need-th largest key: 8 bins per lane of warp 0, suffix sums across the lanes
      if (warp == 0) {
        const unsigned need = s_need;
        unsigned t = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) t += s_hist[8 * lane + j];
        unsigned S = t;   // bins of this lane and of all higher lanes
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const unsigned n = __shfl_down_sync(0xffffffffu, S, o);
          if (lane + o < 32) S += n;
        }
        const unsigned reach = __ballot_sync(0xffffffffu, S >= need);
        const int owner = reach ? 31 - __clz(reach) : 0;   // highest lane whose suffix reaches the need (else bin 0)
        if (lane == owner) {
          unsigned cum = S - t;
          int bin = 8 * lane + 7;
          for (; bin > 8 * lane; bin--) {
            if (cum + s_hist[bin] >= need) break;
            cum += s_hist[bin];
          }
          // (the lowest bin of the owner's range takes what is left, as bin 0 does in a sequential scan)
          s_need = need - cum;
          s_prefix = prefix | ((unsigned)bin << shift);
        }
      }
      __syncthreads();
    }
    const unsigned r = s_prefix;
    __syncthreads();
    return r;
  };
  unsigned floor_from_list = 0;   // set when the candidate list overflows (ties): the full-vocabulary path takes over
  if (top_k > 0 && top_k <= SP_CAND && top_k < V) {
    const unsigned kth_key = select_kth((unsigned)top_k);
    // ---- gather survivors (key >= kth_key)
    if (tid == 0) s_count = 0;
    __syncthreads();
    for (int i = tid; i < V; i += SP_T) {
      float z = zval(i);
      if (ord_key(z) >= kth_key) {
        unsigned slot = atomicAdd(&s_count, 1u);
        if (slot < SP_CAND) { s_val[slot] = z; s_idx[slot] = i; }
      }
    }
    __syncthreads();
    const int C = (int)s_count;
    if (C > SP_CAND && !cache) {  // more ties than the candidate list holds: report and return the argmax
      if (tid == 0) {
        if (status) atomicExch(status, 4);
        out[(size_t)b * out_stride] = imax;
      }
      return;
    }
    if (C > SP_CAND) {
      floor_from_list = kth_key;   // (a key of a finite logit is never 0)
    } else {
    if (tid >= C) { s_val[tid] = -INFINITY; s_idx[tid] = 0x7fffffff; }
    __syncthreads();
    int SN = 2;   // sort width: the power of two that holds the C survivors (the padding sorts to the end)
    while (SN < C) SN <<= 1;
    // ---- bitonic sort by (value descending, index ascending)
    for (int k = 2; k <= SN; k <<= 1)
      for (int j = k >> 1; j > 0; j >>= 1) {
        int ixj = tid ^ j;
        if (ixj > tid && ixj < SN) {
          float va = s_val[tid], vb = s_val[ixj];
          int ia = s_idx[tid], ib = s_idx[ixj];
          bool a_first = (va > vb) || (va == vb && ia < ib);  // a ranks before b
          bool up = ((tid & k) == 0);
          if (up ? !a_first : a_first) {
            s_val[tid] = vb; s_val[ixj] = va; s_idx[tid] = ib; s_idx[ixj] = ia;
          }
        }
        __syncthreads();
      }
    // ---- nucleus cut and draw (sequential over <= 1024 entries, fp32, deterministic)
    if (tid == 0) {
      int keep = C;
      if (top_p > 0.f && top_p < 1.f) {
        float tot = 0.f;
        for (int r = 0; r < C; r++) tot += __expf(s_val[r] - zmax);
        float cum = 0.f;
        keep = 0;
        for (int r = 0; r < C; r++) {
          if (r > 0 && cum > top_p) break;
          keep = r + 1;
          cum += __expf(s_val[r] - zmax) / tot;
        }
      }
      s_choice = keep;
    }
    __syncthreads();
    const int keep = s_choice;
    // re-sort the kept entries by index ascending for the vocabulary-order running sum
    if (tid >= keep) s_idx[tid] = 0x7fffffff;
    __syncthreads();
    for (int k = 2; k <= SN; k <<= 1)
      for (int j = k >> 1; j > 0; j >>= 1) {
        int ixj = tid ^ j;
        if (ixj > tid && ixj < SN) {
          int ia = s_idx[tid], ib = s_idx[ixj];
          bool up = ((tid & k) == 0);
          if (up ? (ia > ib) : (ia < ib)) {
            float va = s_val[tid];
            s_val[tid] = s_val[ixj]; s_val[ixj] = va; s_idx[tid] = ib; s_idx[ixj] = ia;
          }
        }
        __syncthreads();
      }
    if (tid == 0) {
      float tot = 0.f;
      for (int r = 0; r < keep; r++) tot += __expf(s_val[r] - zmax);
      const float target = u * tot;
      float cum = 0.f;
      int choice = s_idx[keep - 1];
      for (int r = 0; r < keep; r++) {
        cum += __expf(s_val[r] - zmax);
        if (cum > target) { choice = s_idx[r]; break; }
      }
      out[(size_t)b * out_stride] = choice;
    }
    return;
    }   // candidate list
  }
  // ---- full-vocabulary filters: nucleus without top-k, or a top-k wider than the candidate list (with or without a
  //      nucleus cut inside it).  Needs the row's keys in shared memory.
  const bool big_k = (top_k > SP_CAND && top_k < V) || floor_from_list != 0;
  const bool nucleus = top_p > 0.f && top_p < 1.f;
  unsigned keep_key = 0;          // entries with a key above this are kept ...
  unsigned tie_key = 0xffffffffu; // ... and, of the entries equal to tie_key, the first tie_keep in vocabulary order
  unsigned tie_keep = 0;
  bool filtered = false;
  if (big_k || nucleus) {
    if (!cache) {   // the vocabulary does not fit in shared memory
      if (tid == 0) {
        if (status) atomicExch(status, nucleus ? 5 : 4);
        out[(size_t)b * out_stride] = imax;
      }
      return;
    }
    filtered = true;
    unsigned floor_key = 0;   // top-k: keys below this are out (ties with the k-th are kept, as in the reference)
    if (big_k) floor_key = floor_from_list ? floor_from_list : select_kth((unsigned)top_k);
    if (!nucleus) {
      keep_key = floor_key > 0 ? floor_key - 1 : 0;
      if (floor_key == 0) filtered = false;
    } else {
      // Probability mass as 40-bit fixed point of exp(z - zmax): integer sums do not depend on the order of the
      // additions, so the cut is reproducible.  Sorted by (value descending, index ascending) an entry is kept while
      // the mass ranked before it is <= top_p * total (flash_stu/model.py:284-291): find the key v* at which the mass
      // from the top first exceeds that bound (4 passes of 8 bits over mass histograms); keys above v* are kept, of
      // the entries equal to v* the first floor((bound - mass above) / mass of one) + 1 in vocabulary order.
      unsigned long long* mh = reinterpret_cast<unsigned long long*>(&s_sub[0][0]);   // [4][256]
      auto mass_of = [&](unsigned key) {
        return (unsigned long long)(__expf(key_value(key) - zmax) * 1099511627776.f);   // 2^40
      };
      __shared__ unsigned long long s_total, s_bound, s_above;
      if (tid == 0) s_total = 0;
      __syncthreads();
      {
        unsigned long long part = 0;
        for (int i = tid; i < V; i += SP_T)
          if (s_key[i] >= floor_key) part += mass_of(s_key[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) atomicAdd(&s_total, part);
      }
      __syncthreads();
      if (tid == 0) {
        s_bound = (unsigned long long)((double)top_p * (double)s_total);
        s_above = 0;
        s_prefix = 0;
      }
      __syncthreads();
      for (int pass = 0; pass < 4; pass++) {
        const int shift = 24 - 8 * pass;
        for (int i = tid; i < 4 * 256; i += SP_T) mh[i] = 0;
        __syncthreads();
        const unsigned prefix = s_prefix;
        const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        unsigned long long* sub = mh + (warp >> 3) * 256;
        for (int i = tid; i < V; i += SP_T) {
          const unsigned key = s_key[i];
          if (key >= floor_key && (key & mask) == prefix) atomicAdd(&sub[(key >> shift) & 255u], mass_of(key));
        }
        __syncthreads();
        if (tid == 0) {
          // from the top bin down: the first bin whose mass pushes the running sum over the bound holds v*
          unsigned long long cum = s_above;
          const unsigned long long bound = s_bound;
          int bin = 255;
          for (; bin > 0; bin--) {
            const unsigned long long hb = mh[bin] + mh[256 + bin] + mh[512 + bin] + mh[768 + bin];
            if (cum + hb > bound) break;
            cum += hb;
          }
          s_above = cum;
          s_prefix = prefix | ((unsigned)bin << shift);
        }
        __syncthreads();
      }
      tie_key = s_prefix;
      if (tie_key < floor_key) tie_key = floor_key;   // the bound was never exceeded: everything above the floor stays
      keep_key = tie_key;
      const unsigned long long one = mass_of(tie_key);
      const unsigned long long room = s_bound >= s_above ? s_bound - s_above : 0;
      tie_keep = one ? (unsigned)min((unsigned long long)V, room / one + 1ull) : (unsigned)V;
      __syncthreads();
    }
  }
  // entry i survives the filters: above the cut, or one of the first tie_keep entries equal to the cut key (their
  // rank among the ties in vocabulary order is supplied by the caller)
  auto kept = [&](unsigned key, unsigned tie_rank) {
    return !filtered || key > keep_key || (key == tie_key && tie_rank < tie_keep);
  };

  // ---- plain temperature sampling over the whole vocabulary: chunked running sum in index order
  const int chunk = (V + SP_T - 1) / SP_T;
  const int lo = tid * chunk, hi = min(V, lo + chunk);
  // ties with the cut key before this thread's chunk (vocabulary order): exclusive scan of the per-thread counts
  unsigned tie_base = 0;
  if (filtered && tie_key != 0xffffffffu) {
    unsigned mine = 0;
    for (int i = lo; i < hi; i++) mine += (s_key[i] == tie_key);
    unsigned incl_t = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned n = __shfl_up_sync(0xffffffffu, incl_t, o);
      if (lane >= o) incl_t += n;
    }
    if (lane == 31) s_redi[warp] = (int)incl_t;
    __syncthreads();
    unsigned before = 0;
    for (int w = 0; w < warp; w++) before += (unsigned)s_redi[w];
    tie_base = before + incl_t - mine;
    __syncthreads();
  }
  float part = 0.f;
  {
    unsigned tr = tie_base;
    for (int i = lo; i < hi; i++) {
      const unsigned key = filtered ? s_key[i] : 0u;
      if (kept(key, tr)) part += __expf(zval(i) - zmax);
      if (filtered && key == tie_key) tr++;
    }
  }
  // block exclusive scan of the 1024 partial sums
  float incl = part;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    float n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) s_red[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    float w = s_red[lane], wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += n;
    }
    s_red[lane] = wi - w;  // exclusive prefix of warp totals
    if (lane == 31) s_hist[0] = __float_as_uint(wi);
  }
  if (tid == 0) s_choice = 0x7fffffff;
  __syncthreads();
  const float tot = __uint_as_float(s_hist[0]);
  const float target = u * tot;
  const float excl = s_red[warp] + incl - part;
  if (lo < hi && part > 0.f && excl <= target && target < excl + part) {
    float cum = excl;
    int choice = -1;
    unsigned tr = tie_base;
    for (int i = lo; i < hi; i++) {
      const unsigned key = filtered ? s_key[i] : 0u;
      if (kept(key, tr)) {
        choice = i;   // the last kept entry of the chunk takes what rounding leaves over
        cum += __expf(zval(i) - zmax);
        if (cum > target) break;
      }
      if (filtered && key == tie_key) tr++;
    }
    if (choice >= 0) atomicMin(&s_choice, choice);
  }
  __syncthreads();
  if (tid == 0) out[(size_t)b * out_stride] = (s_choice == 0x7fffffff) ? imax : s_choice;
}

// logits [B, V] (row stride ld); uniforms [B] fp32 on the device (read only when do_sample);
// out[b * out_stride] receives the token id (int64).  top_k <= 0 and top_p outside (0,1) disable the filters.
extern "C" int stu_sample(const void* logits, long long ld, int B, int V, float temperature, int top_k, float top_p,
                          int do_sample, const float* uniforms, long long* out, long long out_stride, int* status,
                          int dtype, void* stream) {
  if (!logits || !out) return STU_ERR_NULL;
  if (do_sample && !uniforms) return STU_ERR_NULL;
  if (B <= 0 || V <= 0 || !(temperature > 0.f)) return STU_ERR_SHAPE;
  if (top_k > SP_CAND && top_k < V && V > SP_CACHE_MAX) return STU_ERR_UNSUPPORTED;   // needs the row in shared memory
  cudaStream_t st = (cudaStream_t)stream;
  // greedy selection makes one pass only: nothing to keep
  const int cache = (do_sample && V <= SP_CACHE_MAX) ? 1 : 0;
  static const int variant = getenv("STU_SAMPLE_VARIANT") ? atoi(getenv("STU_SAMPLE_VARIANT")) : 2;
  const size_t smem = cache ? (size_t)V * sizeof(uint32_t) : 0;
  if (dtype == STU_F32) {
    if (cache) {
      cudaError_t e = cudaFuncSetAttribute(sample_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SP_CACHE_MAX * (int)sizeof(uint32_t));
      if (e != cudaSuccess) return (int)e;
    }
    sample_kernel<float><<<B, SP_T, smem, st>>>((const float*)logits, ld, V, temperature, top_k, top_p, do_sample,
                                                uniforms, out, out_stride, status, cache, (V < 65536) ? variant : 0);
  } else if (dtype == STU_BF16) {
    if (cache) {
      cudaError_t e = cudaFuncSetAttribute(sample_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SP_CACHE_MAX * (int)sizeof(uint32_t));
      if (e != cudaSuccess) return (int)e;
    }
    sample_kernel<bf16><<<B, SP_T, smem, st>>>((const bf16*)logits, ld, V, temperature, top_k, top_p, do_sample,
                                               uniforms, out, out_stride, status, cache, (V < 65536) ? variant : 0);
  } else {
    return STU_ERR_DTYPE;
  }
  STU_CHECK_LAUNCH();
  return STU_OK;
}
