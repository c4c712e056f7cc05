// Operand access shared by the selective-state update kernels (MX-held and dense state): the
// reference's softplus and the 16-column slices of B / C.
#pragma once

#include "lq_common.cuh"

namespace lq {

// softplus as the reference's kernels compute it (mamba_state_8b_kernel.py:28-30)
__device__ __forceinline__ float softplus_ref(float x) { return x <= 20.0f ? logf(1.0f + expf(x)) : x; }

// 16 consecutive B or C values of (batch b, group grp) starting at column n0, as floats.  Contiguous
// 16-bit operands take two 128-bit loads; anything else goes value by value.
__device__ __forceinline__ void load_bc16(const void* base, const int64_t (&st)[3], int dtype, int b, int grp, int n0, float (&v)[16]) {
  const int64_t off = b * st[0] + grp * st[1] + n0 * st[2];
  if (dtype != LQ_F32 && st[2] == 1 && ((reinterpret_cast<uintptr_t>(base) + 2 * off) & 15) == 0) {
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + off);
    const uint4 lo = __ldg(src), hi = __ldg(src + 1);
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (dtype == LQ_BF16) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = load_as_float(base, off + i * st[2], dtype);
  }
}

}  // namespace lq
