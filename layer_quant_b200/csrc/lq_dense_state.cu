// Unquantised baselines of the Mamba2 decode step: the selective-state update on a dense
// (bf16 / f16 / f32) state and the depthwise causal-convolution update before it.  sm_100a.
//
// Both are plain HBM streaming kernels: the state update reads and writes every state value once
// (4 bytes per value for a 16-bit state), so the only design question is bytes in flight.  One CTA
// owns `hpc` consecutive heads of one (batch, B/C group) as the MX kernel does and a lane owns one
// 16-value block of a row.  Aligned states go through a ring of cp.async stages in shared memory in
// which every thread copies exactly the bytes it will itself consume, so the ring needs no barrier,
// only cp.async.wait_group: seven passes (28 KB) per CTA are in flight while one is computed.
// States that are not 16-byte aligned take the register path (four rows' loads issued before use).
#include <algorithm>
#include <cmath>

#include "lq_ssm_operands.cuh"

namespace lq {

constexpr int kDenseThreads = 128;
constexpr int kDenseRowsInFlight = 4;

struct DenseDerived {
  int32_t lpr_log2;       // lanes per row = dstate / 16 (a power of two)
  int32_t dt_uniform;     // dt and dt_bias do not depend on the row (dim) index
  int32_t a_scalar;       // A depends on the head only
  int32_t heads_per_cta;
  int32_t vector_ok;      // rows start on 16-byte boundaries
};

// 16 consecutive state values -> floats
template <int DT>
__device__ __forceinline__ void dense_load16(const void* base, int64_t off, bool vec, float (&v)[16]) {
  if (DT == LQ_F32) {
    const float* p = static_cast<const float*>(base) + off;
    if (vec) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 f = reinterpret_cast<const float4*>(p)[i];
        v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = p[i];
    }
  } else {
    const uint16_t* p = static_cast<const uint16_t*>(base) + off;
    uint32_t w[8];
    if (vec) {
      const uint4 lo = reinterpret_cast<const uint4*>(p)[0], hi = reinterpret_cast<const uint4*>(p)[1];
      w[0] = lo.x; w[1] = lo.y; w[2] = lo.z; w[3] = lo.w; w[4] = hi.x; w[5] = hi.y; w[6] = hi.z; w[7] = hi.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = static_cast<uint32_t>(p[2 * i]) | (static_cast<uint32_t>(p[2 * i + 1]) << 16);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (DT == LQ_BF16) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
      }
    }
  }
}

template <int DT>
__device__ __forceinline__ void dense_store16(void* base, int64_t off, bool vec, const float (&v)[16]) {
  if (DT == LQ_F32) {
    float* p = static_cast<float*>(base) + off;
    if (vec) {
#pragma unroll
      for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) p[i] = v[i];
    }
  } else {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (DT == LQ_BF16) {
        const __nv_bfloat162 r = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&r);
      } else {
        const __half2 r = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&r);
      }
    }
    uint16_t* p = static_cast<uint16_t*>(base) + off;
    if (vec) {
      reinterpret_cast<uint4*>(p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<uint4*>(p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        p[2 * i] = static_cast<uint16_t>(w[i]);
        p[2 * i + 1] = static_cast<uint16_t>(w[i] >> 16);
      }
    }
  }
}

// h' = h * dA + (B * dt) * x on 16 values and their share of <h', C>, two values per packed fp32x2 instruction (sm_100);
// dB = B * dt rounded, dB * x rounded, one fused multiply-add: the association of the Triton kernel this restates
__device__ __forceinline__ float dense_update_readout16(float (&hv)[16], const float (&Bv)[16], const float (&Cv)[16], float dA,
                                                        float dt, float x) {
  const float2 dA2 = make_float2(dA, dA), dt2 = make_float2(dt, dt), x2 = make_float2(x, x);
  float2 ya = make_float2(0.0f, 0.0f), yb = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    const float2 h0 = __ffma2_rn(make_float2(hv[i], hv[i + 1]), dA2, __fmul2_rn(__fmul2_rn(make_float2(Bv[i], Bv[i + 1]), dt2), x2));
    const float2 h1 = __ffma2_rn(make_float2(hv[i + 2], hv[i + 3]), dA2, __fmul2_rn(__fmul2_rn(make_float2(Bv[i + 2], Bv[i + 3]), dt2), x2));
    hv[i] = h0.x; hv[i + 1] = h0.y; hv[i + 2] = h1.x; hv[i + 3] = h1.y;
    ya = __ffma2_rn(h0, make_float2(Cv[i], Cv[i + 1]), ya);
    yb = __ffma2_rn(h1, make_float2(Cv[i + 2], Cv[i + 3]), yb);
  }
  return (ya.x + ya.y) + (yb.x + yb.y);
}

// h' = h exp(A dt) + (B dt) x on one 16-value block, and the block's share of <h', C>
struct DenseRowCtx {
  const lq_dense_update_args* a;
  const DenseDerived* d;
  int b, n0;
};
__device__ __forceinline__ float dense_row_update(const DenseRowCtx& c, float (&hv)[16], const float (&Bv)[16], const float (&Cv)[16],
                                                  int h, int p, float xv, float dt_h, float dA_h) {
  const lq_dense_update_args& a = *c.a;
  if (c.d->dt_uniform && c.d->a_scalar) {
#pragma unroll
    for (int i = 0; i < 16; ++i) hv[i] = fmaf(hv[i], dA_h, __fmul_rn(__fmul_rn(Bv[i], dt_h), xv));
  } else {
    float dt = dt_h;
    if (!c.d->dt_uniform) {
      dt = load_as_float(a.dt, c.b * a.dt_stride[0] + h * a.dt_stride[1] + p * a.dt_stride[2], a.dt_dtype);
      if (a.dt_bias) dt += load_as_float(a.dt_bias, h * a.dt_bias_stride[0] + p * a.dt_bias_stride[1], a.dt_bias_dtype);
      if (a.dt_softplus) dt = softplus_ref(dt);
    }
    if (c.d->a_scalar) {
      const float dA = expf(load_as_float(a.A, h * a.A_stride[0], a.A_dtype) * dt);
#pragma unroll
      for (int i = 0; i < 16; ++i) hv[i] = fmaf(hv[i], dA, __fmul_rn(__fmul_rn(Bv[i], dt), xv));
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float Ai = load_as_float(a.A, h * a.A_stride[0] + p * a.A_stride[1] + (c.n0 + i) * a.A_stride[2], a.A_dtype);
        hv[i] = fmaf(hv[i], expf(Ai * dt), __fmul_rn(__fmul_rn(Bv[i], dt), xv));
      }
    }
  }
  float y0 = 0.0f, y1 = 0.0f, y2 = 0.0f, y3 = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    y0 = fmaf(hv[i], Cv[i], y0);
    y1 = fmaf(hv[i + 1], Cv[i + 1], y1);
    y2 = fmaf(hv[i + 2], Cv[i + 2], y2);
    y3 = fmaf(hv[i + 3], Cv[i + 3], y3);
  }
  return (y0 + y1) + (y2 + y3);
}

// gridDim.x = batch * (heads / hpc)
template <int DT>
__global__ void __launch_bounds__(kDenseThreads, 4) dense_state_update_kernel(const lq_dense_update_args a, const DenseDerived d) {
  extern __shared__ float smem_dense[];  // x of the CTA's rows, <h', C> of the rows, per-head dt and exp(A dt)
  const int H = a.heads, P = a.dim;
  const int hpc = d.heads_per_cta;
  float* sx = smem_dense;
  float* sy = sx + hpc * P;
  float* sdt = sy + hpc * P;
  float* sdA = sdt + hpc;
  const int chunks = H / hpc;
  const int b = blockIdx.x / chunks;
  const int h0 = (blockIdx.x - b * chunks) * hpc;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int blk = lane & ((1 << d.lpr_log2) - 1);
  const int rsub = lane >> d.lpr_log2;
  const int rows_per_warp = 32 >> d.lpr_log2;
  const int rows_per_pass = rows_per_warp * (kDenseThreads / 32);
  const int n0 = blk * 16;
  const int grp = h0 / (H / a.ngroups);
  const bool vec = d.vector_ok != 0;

  auto row_dt = [&](int h, int p) {
    float dt = load_as_float(a.dt, b * a.dt_stride[0] + h * a.dt_stride[1] + p * a.dt_stride[2], a.dt_dtype);
    if (a.dt_bias) dt += load_as_float(a.dt_bias, h * a.dt_bias_stride[0] + p * a.dt_bias_stride[1], a.dt_bias_dtype);
    if (a.dt_softplus) dt = softplus_ref(dt);
    return dt;
  };
  for (int i = threadIdx.x; i < hpc * P; i += kDenseThreads) {
    const int hh = i / P, p = i - hh * P;
    sx[i] = load_as_float(a.x, b * a.x_stride[0] + (h0 + hh) * a.x_stride[1] + p * a.x_stride[2], a.x_dtype);
  }
  if (d.dt_uniform && threadIdx.x < hpc) {
    const float dt = row_dt(h0 + threadIdx.x, 0);
    sdt[threadIdx.x] = dt;
    sdA[threadIdx.x] = d.a_scalar ? expf(load_as_float(a.A, (h0 + threadIdx.x) * a.A_stride[0], a.A_dtype) * dt) : 0.0f;
  }
  float Bv[16], Cv[16];
  load_bc16(a.B, a.B_stride, a.B_dtype, b, grp, n0, Bv);
  load_bc16(a.C, a.C_stride, a.C_dtype, b, grp, n0, Cv);
  const DenseRowCtx rc{&a, &d, b, n0};
  __syncthreads();

#pragma unroll 1
  for (int hh = 0; hh < hpc; ++hh) {
    const int h = h0 + hh;
    const float dt_h = d.dt_uniform ? sdt[hh] : 0.0f;
    const float dA_h = sdA[hh];
    const int64_t base = b * a.state_stride[0] + h * a.state_stride[1] + n0;
    const float* sxh = sx + hh * P;
    float* syh = sy + hh * P;
#pragma unroll 1
    for (int pw = warp * rows_per_warp; pw < P; pw += rows_per_pass * kDenseRowsInFlight) {  // uniform over the warp
      const int p0 = pw + rsub;
      float hv[kDenseRowsInFlight][16];
#pragma unroll
      for (int u = 0; u < kDenseRowsInFlight; ++u) {
        const int p = p0 + u * rows_per_pass;
        if (p < P) dense_load16<DT>(a.state, base + p * a.state_stride[2], vec, hv[u]);
      }
#pragma unroll
      for (int u = 0; u < kDenseRowsInFlight; ++u) {
        const int p = p0 + u * rows_per_pass;
        const bool active = p < P;  // uniform over the lanes of a row
        float y = 0.0f;
        if (active) {
          y = dense_row_update(rc, hv[u], Bv, Cv, h, p, sxh[p], dt_h, dA_h);
          dense_store16<DT>(a.state, base + p * a.state_stride[2], vec, hv[u]);
        }
        for (int o = (1 << d.lpr_log2) >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xFFFFFFFFu, y, o);
        if (active && blk == 0) syh[p] = y;
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < hpc * P; i += kDenseThreads) {
    const int hh = i / P, p = i - hh * P, h = h0 + hh;
    float y = sy[i];
    if (a.D) y += sx[i] * load_as_float(a.D, h * a.D_stride[0] + p * a.D_stride[1], a.D_dtype);
    if (a.z) {
      const float z = load_as_float(a.z, b * a.z_stride[0] + h * a.z_stride[1] + p * a.z_stride[2], a.z_dtype);
      y *= z / (1.0f + expf(-z));
    }
    store_from_float(a.out, b * a.out_stride[0] + h * a.out_stride[1] + p * a.out_stride[2], a.out_dtype, y);
  }
}

// The aligned path.  Shared memory: a ring of kRingBytes, then the x / y / dt staging.  A stage holds one
// pass of the CTA; inside it every warp has its own 32 * CH 16-byte chunks (CH = chunks per 16-value
// block: 2 for a 16-bit state, 4 for fp32), in the order they have in the warp's rows.  Lane l copies
// chunks l, 32 + l, ... (contiguous 512 B per instruction, whole sectors) and consumes the CH chunks of
// its own block, so a warp synchronises with itself only (cp.async.wait_group + __syncwarp); results
// go back through the same chunks to leave with contiguous 16-byte stores.  Chunk c is kept at
// position c ^ ((c >> 3) & 3), which makes both access patterns free of bank conflicts.
constexpr int kRingBytes = 32 * 1024;

__device__ __forceinline__ void dense_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t dense_swz(uint32_t c) { return c ^ ((c >> 3) & 3u); }

// LPR_T: lanes per row when known at compile time (8 for dstate 128), 0 = taken from the arguments.
// SIMPLE: dt / dt_bias / A per head only and dim a multiple of the rows of a pass (every Mamba2 decode step):
// no row guards, no per-row operand reloads.
template <int DT, int LPR_T, bool SIMPLE>
__global__ void __launch_bounds__(kDenseThreads, 4) dense_state_update_ring_kernel(const lq_dense_update_args a, const DenseDerived d) {
  constexpr int ESZ = DT == LQ_F32 ? 4 : 2;
  constexpr int CH = ESZ;                                        // 16 * ESZ / 16
  constexpr int STAGES = kRingBytes / (CH * kDenseThreads * 16);  // 8 or 4
  constexpr uint32_t kStageBytes = CH * kDenseThreads * 16;
  extern __shared__ __align__(16) uint8_t smem_ring[];
  float* sx = reinterpret_cast<float*>(smem_ring + kRingBytes);
  const int H = a.heads, P = a.dim;
  const int hpc = d.heads_per_cta;
  float* sy = sx + hpc * P;
  float* sdt = sy + hpc * P;
  float* sdA = sdt + hpc;
  const int chunks = H / hpc;
  const int b = blockIdx.x / chunks;
  const int h0 = (blockIdx.x - b * chunks) * hpc;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lpr_log2 = LPR_T ? (LPR_T == 8 ? 3 : 0) : d.lpr_log2;
  static_assert(LPR_T == 0 || LPR_T == 8, "specialised for dstate 128 only");
  const int blk = lane & ((1 << lpr_log2) - 1);
  const int rsub = lane >> lpr_log2;
  const int rows_per_warp = 32 >> lpr_log2;
  const int rows_per_pass = rows_per_warp * (kDenseThreads / 32);
  const int n0 = blk * 16;
  const int grp = h0 / (H / a.ngroups);
  const int prow = warp * rows_per_warp + rsub;          // this thread's row inside a pass
  const int pph = (P + rows_per_pass - 1) / rows_per_pass;  // passes per head
  const int npass = hpc * pph;
  // byte steps of a row: to the next pass of a head, and from a head's last pass to the next head's first
  const int64_t pass_step = static_cast<int64_t>(rows_per_pass) * a.state_stride[2] * ESZ;
  const int64_t head_step = a.state_stride[1] * ESZ - (pph - 1) * pass_step;
  uint8_t* const warp_first = static_cast<uint8_t*>(a.state) +
                              (b * a.state_stride[0] + h0 * a.state_stride[1] + warp * rows_per_warp * a.state_stride[2]) * ESZ;
  // the chunks this lane moves: chunk c = 32 k + lane of the warp's rows -> row c / chunks-per-row, column chunk c % ...
  const int cpr_log2 = lpr_log2 + (CH == 2 ? 1 : 2);
  int64_t mv_off[CH];
  int mv_row[CH];
  uint32_t mv_smem[CH];
#pragma unroll
  for (int k = 0; k < CH; ++k) {
    const uint32_t c = 32 * k + lane;
    mv_row[k] = warp * rows_per_warp + static_cast<int>(c >> cpr_log2);
    mv_off[k] = static_cast<int64_t>(c >> cpr_log2) * a.state_stride[2] * ESZ + (c & ((1u << cpr_log2) - 1)) * 16;
    mv_smem[k] = warp * (32 * CH * 16) + dense_swz(c) * 16;
  }
  uint32_t own_smem[CH];  // the chunks of this lane's own block
#pragma unroll
  for (int k = 0; k < CH; ++k) own_smem[k] = warp * (32 * CH * 16) + dense_swz(lane * CH + k) * 16;
  const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(smem_ring));

  // producer cursor: pass `ip` of the CTA = pass `ipp` of its head, whose first row is `irow0`
  const uint8_t* iptr = warp_first;
  int ip = 0, ipp = 0, irow0 = 0;
  auto issue = [&]() {
    if (ip < npass) {
      const uint32_t dst = ring + (ip & (STAGES - 1)) * kStageBytes;
#pragma unroll
      for (int k = 0; k < CH; ++k)
        if (SIMPLE || irow0 + mv_row[k] < P) dense_cp_async16(dst + mv_smem[k], iptr + mv_off[k]);
      ++ip;
      if (++ipp == pph) {
        ipp = 0;
        irow0 = 0;
        iptr += head_step;
      } else {
        irow0 += rows_per_pass;
        iptr += pass_step;
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) issue();

  for (int i = threadIdx.x; i < hpc * P; i += kDenseThreads) {
    const int hh = i / P, p = i - hh * P;
    sx[i] = load_as_float(a.x, b * a.x_stride[0] + (h0 + hh) * a.x_stride[1] + p * a.x_stride[2], a.x_dtype);
  }
  if (d.dt_uniform && threadIdx.x < hpc) {
    const int h = h0 + threadIdx.x;
    float dt = load_as_float(a.dt, b * a.dt_stride[0] + h * a.dt_stride[1], a.dt_dtype);
    if (a.dt_bias) dt += load_as_float(a.dt_bias, h * a.dt_bias_stride[0], a.dt_bias_dtype);
    if (a.dt_softplus) dt = softplus_ref(dt);
    sdt[threadIdx.x] = dt;
    sdA[threadIdx.x] = d.a_scalar ? expf(load_as_float(a.A, h * a.A_stride[0], a.A_dtype) * dt) : 0.0f;
  }
  float Bv[16], Cv[16];
  load_bc16(a.B, a.B_stride, a.B_dtype, b, grp, n0, Bv);
  load_bc16(a.C, a.C_stride, a.C_dtype, b, grp, n0, Cv);
  const DenseRowCtx rc{&a, &d, b, n0};
  __syncthreads();

  // consumer cursor
  uint8_t* cptr = warp_first;
  int chh = 0, cpp = 0, crow0 = 0;
  float dt_h = d.dt_uniform ? sdt[0] : 0.0f, dA_h = sdA[0];
#pragma unroll 1
  for (int i = 0; i < npass; ++i) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");  // this lane's copies of pass i have landed
    __syncwarp();                                                           // ... and so have the other lanes'
    uint8_t* stage = smem_ring + (i & (STAGES - 1)) * kStageBytes;
    const int crow = crow0 + prow;
    const bool active = SIMPLE || crow < P;
    float hv[16];
    if (active) {
      if (DT == LQ_F32) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float4 f = *reinterpret_cast<const float4*>(stage + own_smem[k]);
          hv[4 * k] = f.x; hv[4 * k + 1] = f.y; hv[4 * k + 2] = f.z; hv[4 * k + 3] = f.w;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const uint4 q = *reinterpret_cast<const uint4*>(stage + own_smem[k]);
          const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (DT == LQ_BF16) {
              hv[8 * k + 2 * j] = __uint_as_float(w[j] << 16);
              hv[8 * k + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
            } else {
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
              hv[8 * k + 2 * j] = f.x;
              hv[8 * k + 2 * j + 1] = f.y;
            }
          }
        }
      }
    }
    issue();  // into the stage of pass i - 1, which the warp left before the __syncwarp above
    float y = 0.0f;
    const int srow = chh * P + crow;
    if (active) {
      if (SIMPLE) {
        y = dense_update_readout16(hv, Bv, Cv, dA_h, dt_h, sx[srow]);
      } else {
        y = dense_row_update(rc, hv, Bv, Cv, h0 + chh, crow, sx[srow], dt_h, dA_h);
      }
      // the rounded block back into its chunks
      if (DT == LQ_F32) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          *reinterpret_cast<float4*>(stage + own_smem[k]) = make_float4(hv[4 * k], hv[4 * k + 1], hv[4 * k + 2], hv[4 * k + 3]);
      } else {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (DT == LQ_BF16) {
              const __nv_bfloat162 r = __floats2bfloat162_rn(hv[8 * k + 2 * j], hv[8 * k + 2 * j + 1]);
              w[j] = *reinterpret_cast<const uint32_t*>(&r);
            } else {
              const __half2 r = __floats2half2_rn(hv[8 * k + 2 * j], hv[8 * k + 2 * j + 1]);
              w[j] = *reinterpret_cast<const uint32_t*>(&r);
            }
          }
          *reinterpret_cast<uint4*>(stage + own_smem[k]) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < CH; ++k)
      if (SIMPLE || crow0 + mv_row[k] < P)
        *reinterpret_cast<uint4*>(cptr + mv_off[k]) = *reinterpret_cast<const uint4*>(stage + mv_smem[k]);
    if (LPR_T == 8) {
      y += __shfl_xor_sync(0xFFFFFFFFu, y, 4);
      y += __shfl_xor_sync(0xFFFFFFFFu, y, 2);
      y += __shfl_xor_sync(0xFFFFFFFFu, y, 1);
    } else {
      for (int o = (1 << lpr_log2) >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xFFFFFFFFu, y, o);
    }
    if (active && blk == 0) sy[srow] = y;
    if (++cpp == pph) {
      cpp = 0;
      crow0 = 0;
      cptr += head_step;
      ++chh;
      if (chh < hpc) {
        dt_h = d.dt_uniform ? sdt[chh] : 0.0f;
        dA_h = sdA[chh];
      }
    } else {
      crow0 += rows_per_pass;
      cptr += pass_step;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < hpc * P; i += kDenseThreads) {
    const int hh = i / P, p = i - hh * P, h = h0 + hh;
    float y = sy[i];
    if (a.D) y += sx[i] * load_as_float(a.D, h * a.D_stride[0] + p * a.D_stride[1], a.D_dtype);
    if (a.z) {
      const float z = load_as_float(a.z, b * a.z_stride[0] + h * a.z_stride[1] + p * a.z_stride[2], a.z_dtype);
      y *= z / (1.0f + expf(-z));
    }
    store_from_float(a.out, b * a.out_stride[0] + h * a.out_stride[1] + p * a.out_stride[2], a.out_dtype, y);
  }
}

// One thread per (batch, channel); W is small (4 for Nemotron-H), the window is a handful of registers.
__global__ void __launch_bounds__(256) causal_conv1d_update_kernel(const lq_conv1d_update_args a) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(a.batch) * a.channels) return;
  const int b = static_cast<int>(idx / a.channels), c = static_cast<int>(idx - static_cast<int64_t>(b) * a.channels);
  const int W = a.width;
  const int64_t sbase = b * a.state_stride[0] + c * a.state_stride[1];
  float win[8];
#pragma unroll
  for (int w = 0; w < 8; ++w)
    if (w + 1 < W) win[w] = load_as_float(a.conv_state, sbase + (w + 1) * a.state_stride[2], a.state_dtype);
  const float xv = load_as_float(a.x, b * a.x_stride[0] + c * a.x_stride[1], a.x_dtype);
  float acc = a.bias ? load_as_float(a.bias, c * a.bias_stride[0], a.bias_dtype) : 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    if (w < W) {
      const float v = (w + 1 < W) ? win[w] : xv;
      store_from_float(a.conv_state, sbase + w * a.state_stride[2], a.state_dtype, v);
      acc = fmaf(v, load_as_float(a.weight, c * a.weight_stride[0] + w * a.weight_stride[1], a.weight_dtype), acc);
    }
  }
  if (a.silu) acc = acc / (1.0f + expf(-acc));
  store_from_float(a.out, b * a.out_stride[0] + c * a.out_stride[1], a.out_dtype, acc);
}

}  // namespace lq

using namespace lq;

static bool valid_dt(int32_t d) { return d == LQ_BF16 || d == LQ_F16 || d == LQ_F32; }

LQ_EXPORT int lq_dense_state_update(const lq_dense_update_args* args, void* cuda_stream) {
  LQ_CHECK_ARG(args != nullptr, "lq_dense_state_update: null args");
  const lq_dense_update_args& a = *args;
  LQ_CHECK_ARG(a.state && a.x && a.dt && a.A && a.B && a.C && a.out, "lq_dense_state_update: null state/x/dt/A/B/C/out");
  LQ_CHECK_ARG(a.batch >= 0 && a.heads > 0 && a.dim > 0 && a.dstate > 0, "lq_dense_state_update: bad shape [%d,%d,%d,%d]", a.batch,
               a.heads, a.dim, a.dstate);
  LQ_CHECK_ARG(valid_dt(a.state_dtype) && valid_dt(a.x_dtype) && valid_dt(a.dt_dtype) && valid_dt(a.A_dtype) && valid_dt(a.B_dtype) &&
                   valid_dt(a.C_dtype) && valid_dt(a.out_dtype) && (!a.D || valid_dt(a.D_dtype)) && (!a.z || valid_dt(a.z_dtype)) &&
                   (!a.dt_bias || valid_dt(a.dt_bias_dtype)),
               "lq_dense_state_update: bad dtype code");
  LQ_CHECK_ARG(a.ngroups > 0 && a.heads % a.ngroups == 0, "lq_dense_state_update: heads=%d not a multiple of ngroups=%d", a.heads,
               a.ngroups);
  LQ_CHECK_ARG(a.state_stride[3] == 1, "lq_dense_state_update: the state's last dimension must be contiguous");
  const int nblk = a.dstate / 16;
  if (a.dstate % 16 != 0 || nblk > 32 || (nblk & (nblk - 1)) != 0)
    return fail(LQ_ERR_UNSUPPORTED, "lq_dense_state_update: dstate=%d (supported: 16, 32, 64, 128, 256, 512)", a.dstate);
  if (a.batch == 0) return LQ_OK;
  DenseDerived d;
  d.lpr_log2 = 0;
  while ((1 << d.lpr_log2) < nblk) ++d.lpr_log2;
  d.dt_uniform = a.dt_stride[2] == 0 && (!a.dt_bias || a.dt_bias_stride[1] == 0);
  d.a_scalar = a.A_stride[1] == 0 && a.A_stride[2] == 0;
  const size_t esz = a.state_dtype == LQ_F32 ? 4 : 2;
  d.vector_ok = reinterpret_cast<uintptr_t>(a.state) % 16 == 0 && (a.state_stride[0] * esz) % 16 == 0 &&
                (a.state_stride[1] * esz) % 16 == 0 && (a.state_stride[2] * esz) % 16 == 0;
  // heads per CTA: as many of one B/C group as keep the grid at two waves or more of resident CTAs
  const int heads_per_group = a.heads / a.ngroups;
  int dev = 0, sms = 0;
  LQ_CHECK_CUDA(cudaGetDevice(&dev));
  LQ_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  // heads per CTA (all of one B/C group): the divisor that best fills whole waves of resident CTAs while
  // keeping the CTA's set-up (about six passes' worth) small against its passes
  const int rows_per_pass = (32 >> d.lpr_log2) * (kDenseThreads / 32);
  const int pph = (a.dim + rows_per_pass - 1) / rows_per_pass;
  const double resident = 4.0 * sms;
  int hpc = 1;
  double best = -1.0;
  for (int c = 1; c <= heads_per_group; c *= 2) {
    if (heads_per_group % c != 0 || static_cast<size_t>(c) * (2 * a.dim + 2) * sizeof(float) > 16 * 1024) break;
    const double waves = static_cast<double>(a.batch) * (a.heads / c) / resident;
    const double score = waves / std::ceil(waves) * (c * pph) / (c * pph + 6.0);
    if (score > best) {
      best = score;
      hpc = c;
    }
  }
  d.heads_per_cta = hpc;
  const size_t smem = static_cast<size_t>(hpc) * (2 * a.dim + 2) * sizeof(float);
  if (smem > 48 * 1024) return fail(LQ_ERR_UNSUPPORTED, "lq_dense_state_update: dim=%d too large", a.dim);
  const int64_t grid = static_cast<int64_t>(a.batch) * (a.heads / hpc);
  LQ_CHECK_ARG(grid <= 0x7FFFFFFFLL, "lq_dense_state_update: batch * heads too large");
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const unsigned g = static_cast<unsigned>(grid);
  if (d.vector_ok) {
    const size_t rsmem = kRingBytes + smem;
    const bool simple = d.dt_uniform && d.a_scalar && a.dim % rows_per_pass == 0;
#define LQ_DENSE_RING(DT_)                                                                                              \
  do {                                                                                                                  \
    if (nblk == 8 && simple) {                                                                                          \
      LQ_CHECK_CUDA(cudaFuncSetAttribute(dense_state_update_ring_kernel<DT_, 8, true>,                                  \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(rsmem)));        \
      dense_state_update_ring_kernel<DT_, 8, true><<<g, kDenseThreads, rsmem, st>>>(a, d);                              \
    } else {                                                                                                            \
      LQ_CHECK_CUDA(cudaFuncSetAttribute(dense_state_update_ring_kernel<DT_, 0, false>,                                 \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(rsmem)));        \
      dense_state_update_ring_kernel<DT_, 0, false><<<g, kDenseThreads, rsmem, st>>>(a, d);                             \
    }                                                                                                                   \
  } while (0)
    switch (a.state_dtype) {
      case LQ_BF16: LQ_DENSE_RING(LQ_BF16); break;
      case LQ_F16: LQ_DENSE_RING(LQ_F16); break;
      default: LQ_DENSE_RING(LQ_F32); break;
    }
#undef LQ_DENSE_RING
  } else {
    switch (a.state_dtype) {
      case LQ_BF16: dense_state_update_kernel<LQ_BF16><<<g, kDenseThreads, smem, st>>>(a, d); break;
      case LQ_F16: dense_state_update_kernel<LQ_F16><<<g, kDenseThreads, smem, st>>>(a, d); break;
      default: dense_state_update_kernel<LQ_F32><<<g, kDenseThreads, smem, st>>>(a, d); break;
    }
  }
  LQ_CHECK_CUDA(cudaGetLastError());
  return LQ_OK;
}

LQ_EXPORT int lq_causal_conv1d_update(const lq_conv1d_update_args* args, void* cuda_stream) {
  LQ_CHECK_ARG(args != nullptr, "lq_causal_conv1d_update: null args");
  const lq_conv1d_update_args& a = *args;
  LQ_CHECK_ARG(a.conv_state && a.x && a.weight && a.out, "lq_causal_conv1d_update: null conv_state/x/weight/out");
  LQ_CHECK_ARG(a.batch >= 0 && a.channels > 0, "lq_causal_conv1d_update: bad shape [%d,%d]", a.batch, a.channels);
  LQ_CHECK_ARG(a.width >= 1 && a.width <= 8, "lq_causal_conv1d_update: width=%d outside [1, 8]", a.width);
  LQ_CHECK_ARG(valid_dt(a.state_dtype) && valid_dt(a.x_dtype) && valid_dt(a.weight_dtype) && valid_dt(a.out_dtype) &&
                   (!a.bias || valid_dt(a.bias_dtype)),
               "lq_causal_conv1d_update: bad dtype code");
  if (a.batch == 0) return LQ_OK;
  const int64_t total = static_cast<int64_t>(a.batch) * a.channels;
  const int64_t grid = (total + 255) / 256;
  LQ_CHECK_ARG(grid <= 0x7FFFFFFFLL, "lq_causal_conv1d_update: batch * channels too large");
  causal_conv1d_update_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(a);
  LQ_CHECK_CUDA(cudaGetLastError());
  return LQ_OK;
}
