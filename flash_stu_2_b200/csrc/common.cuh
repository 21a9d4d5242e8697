// Shared helpers for the sm_100a kernels behind the C-ABI in include/stu_b200.h.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define STU_OK 0
#define STU_ERR_DTYPE (-1)
#define STU_ERR_SHAPE (-2)
#define STU_ERR_ALIGN (-3)
#define STU_ERR_UNSUPPORTED (-4)
#define STU_ERR_NULL (-5)
#define STU_ERR_DEVICE_STATUS (-6)

#define STU_F32 0
#define STU_BF16 1

typedef __nv_bfloat16 bf16;

#define STU_CHECK_LAUNCH()                        \
  do {                                            \
    cudaError_t e__ = cudaGetLastError();         \
    if (e__ != cudaSuccess) return (int)e__;      \
  } while (0)

template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int VEC = 4;  // elements per 16-byte vector
  __device__ static __forceinline__ float to_f(float v) { return v; }
  __device__ static __forceinline__ float from_f(float v) { return v; }
};
template <> struct Elem<bf16> {
  static constexpr int VEC = 8;
  __device__ static __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
  __device__ static __forceinline__ bf16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// Round an fp32 value to the storage type and back: the rounding points of the reference's
// bf16 tensors are reproduced by calling this wherever the reference materialises a tensor.
template <typename T> __device__ __forceinline__ float round_to(float v) {
  return Elem<T>::to_f(Elem<T>::from_f(v));
}

// 16-byte vector load of VEC elements converted to fp32.
__device__ __forceinline__ void load_vec(const float* p, float* out) {
  float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void load_vec(const bf16* p, float* out) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void store_vec(float* p, const float* in) {
  *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
}
__device__ __forceinline__ void store_vec(bf16* p, const float* in) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    __nv_bfloat162 h = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// tanh-approximated GELU exactly as torch.nn.functional.gelu(approximate="tanh") states it.
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f;  // sqrt(2/pi)
  const float k1 = 0.044715f;
  float inner = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.0f + tanhf(inner));
}

// Offset (in elements) of the projected-history element of sequence b, channel c, time t.
// Layout [B][d][2][Lh]: time-major inside each parity so that the even-tap convolution of one
// channel reads a single contiguous run per parity.
__host__ __device__ __forceinline__ size_t hist_off(int b, int c, int t, int d, int Lh) {
  return ((size_t)((size_t)b * d + c) * 2 + (t & 1)) * Lh + (t >> 1);
}

static inline bool aligned16(const void* p) { return (((uintptr_t)p) & 15u) == 0; }
