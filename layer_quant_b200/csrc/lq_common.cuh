// Shared host/device helpers of the layer_quant_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/layer_quant_b200.h"

#define LQ_EXPORT extern "C" __attribute__((visibility("default")))

namespace lq {

// ---- host-side error reporting ---------------------------------------------------------------
char* last_error_buffer();  // thread-local, 512 bytes (defined in lq_api.cu)

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define LQ_CHECK_ARG(cond, ...)                                  \
  do {                                                           \
    if (!(cond)) return ::lq::fail(LQ_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

#define LQ_CHECK_CUDA(expr)                                                                    \
  do {                                                                                         \
    cudaError_t e__ = (expr);                                                                  \
    if (e__ != cudaSuccess)                                                                    \
      return ::lq::fail(LQ_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));         \
  } while (0)

inline bool valid_dtype(int dt) { return dt == LQ_BF16 || dt == LQ_F16 || dt == LQ_F32; }
inline int dtype_bytes(int dt) { return dt == LQ_F32 ? 4 : 2; }

int sm_count();  // multiprocessors of the current device (cached per device; lq_api.cu)

// ---- device helpers --------------------------------------------------------------------------
__device__ __forceinline__ float load_as_float(const void* p, int64_t i, int dt) {
  if (dt == LQ_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  if (dt == LQ_F16) return __half2float(static_cast<const __half*>(p)[i]);
  return static_cast<const float*>(p)[i];
}

__device__ __forceinline__ void store_from_float(void* p, int64_t i, int dt, float v) {
  if (dt == LQ_BF16)
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else if (dt == LQ_F16)
    static_cast<__half*>(p)[i] = __float2half_rn(v);
  else
    static_cast<float*>(p)[i] = v;
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// Philox4x32-10 (Salmon et al. 2011), the generator behind Triton's tl.rand.
struct Philox4 {
  uint32_t w0, w1, w2, w3;
};

__device__ __forceinline__ Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                                 uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t pb = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    const uint64_t pa = static_cast<uint64_t>(0xD2511F53u) * c0;
    const uint32_t n0 = static_cast<uint32_t>(pb >> 32) ^ c1 ^ k0;
    const uint32_t n2 = static_cast<uint32_t>(pa >> 32) ^ c3 ^ k1;
    c1 = static_cast<uint32_t>(pb);
    c3 = static_cast<uint32_t>(pa);
    c0 = n0;
    c2 = n2;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return Philox4{c0, c1, c2, c3};
}

// Same generator with the ten round keys precomputed (k0 + r * 0x9E3779B9, k1 + r * 0xBB67AE85 at
// rk[2r], rk[2r + 1]); when rk lives in kernel parameters the keys cost no instruction.
struct PhiloxKeys {
  uint32_t rk[20];
};

inline PhiloxKeys make_philox_keys(uint64_t seed) {
  PhiloxKeys k;
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    k.rk[2 * r] = k0;
    k.rk[2 * r + 1] = k1;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return k;
}

__device__ __forceinline__ Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, const PhiloxKeys& keys) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t pb = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    const uint64_t pa = static_cast<uint64_t>(0xD2511F53u) * c0;
    const uint32_t n0 = static_cast<uint32_t>(pb >> 32) ^ c1 ^ keys.rk[2 * r];
    const uint32_t n2 = static_cast<uint32_t>(pa >> 32) ^ c3 ^ keys.rk[2 * r + 1];
    c1 = static_cast<uint32_t>(pb);
    c3 = static_cast<uint32_t>(pa);
    c0 = n0;
    c2 = n2;
  }
  return Philox4{c0, c1, c2, c3};
}

// Word -> uniform float in [0, 1) exactly as tl.rand does it: reinterpret as int32, fold the
// negative half with x -> -x - 1, convert (round to nearest) and scale by fp32(4.6566127342e-10).
__device__ __forceinline__ float word_to_uniform(uint32_t w) {
  int x = static_cast<int>(w);
  x = x < 0 ? ~x : x;
  return __int2float_rn(x) * 4.6566127342e-10f;
}

}  // namespace lq
