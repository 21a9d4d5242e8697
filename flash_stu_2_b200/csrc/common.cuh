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

#define STU_MAX_DEVICES 64  // per-device tables (status word, SM count, static scratch address)

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

// ---- programmatic dependent launch (overlap of a kernel's constant-data prefetch with its predecessor) ----
// Flags OR-ed into the epilogue code of stu_linear and into the dtype code of stu_decode_approx:
//   STU_FLAG_OVERLAP        the launch carries the programmatic-stream-serialization attribute: its CTAs may start
//                           while the preceding kernel of the stream is still running; everything the kernel
//                           reads before griddepcontrol.wait must be data that kernel does not write
//   STU_FLAG_EARLY_TRIGGER  the kernel lets its own successor start as soon as all its CTAs are resident
//                           (otherwise: right after its own wait, i.e. once its predecessor has completed)
// Both instructions are no-ops in a launch without programmatic neighbours.
#define STU_FLAG_OVERLAP 0x200
#define STU_FLAG_EARLY_TRIGGER 0x400
// stu_decode_approx only: the caller promises that every sequence of the batch stands at the same position (the
// kernel checks and reports status 6 otherwise); selects the kernel that shares the taps between sequences.
#define STU_FLAG_UNIFORM_POS 0x800
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// STU_B200_DISABLE_PDL=1 turns every launch back into a plain stream-ordered one.
bool pdl_enabled();

// Launch with or without the programmatic attribute.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_maybe_overlapped(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                                  cudaStream_t st, bool overlap, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (overlap && pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
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

// Normalise eight activation values the way the reference's RMSNorm output tensor holds them
// (x * r * w rounded to bf16) and pack them as four bf16x2 words.
__device__ __forceinline__ uint4 norm_pack(const uint4& raw, float r, const uint4& nraw) {
  float xv[8], wv[8];
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  const uint32_t n[4] = {nraw.x, nraw.y, nraw.z, nraw.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    xv[2 * i] = __uint_as_float(w[i] << 16);
    xv[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    wv[2 * i] = __uint_as_float(n[i] << 16);
    wv[2 * i + 1] = __uint_as_float(n[i] & 0xffff0000u);
  }
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    __nv_bfloat162 h = __floats2bfloat162_rn(xv[2 * i] * r * wv[2 * i], xv[2 * i + 1] * r * wv[2 * i + 1]);
    o[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

