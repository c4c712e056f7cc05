// Unquantised baselines of the Mamba2 decode step: the selective-state update on a dense
// (bf16 / f16 / f32) state and the depthwise causal-convolution update before it.  sm_100a.
//
// Both are plain HBM streaming kernels: the state update reads and writes every state value once
// (4 bytes per value for a 16-bit state), so the only design question is bytes in flight.  One CTA
// owns `hpc` consecutive heads of one (batch, B/C group) as the MX kernel does; a lane owns one
// 16-value block of FOUR rows per iteration and issues all of their loads (8 x 16 B for a 16-bit
// state) before the first use, which with four resident CTAs keeps about 64 KB per SM in flight.
#include <algorithm>

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
  const bool hoisted = d.dt_uniform && d.a_scalar;
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
          const float xv = sxh[p];
          if (hoisted) {
            const float dtx = dt_h * xv;
#pragma unroll
            for (int i = 0; i < 16; ++i) hv[u][i] = hv[u][i] * dA_h + Bv[i] * dtx;
          } else {
            const float dt = d.dt_uniform ? dt_h : row_dt(h, p);
            const float dtx = dt * xv;
            if (d.a_scalar) {
              const float dA = expf(load_as_float(a.A, h * a.A_stride[0], a.A_dtype) * dt);
#pragma unroll
              for (int i = 0; i < 16; ++i) hv[u][i] = hv[u][i] * dA + Bv[i] * dtx;
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float Ai = load_as_float(a.A, h * a.A_stride[0] + p * a.A_stride[1] + (n0 + i) * a.A_stride[2], a.A_dtype);
                hv[u][i] = hv[u][i] * expf(Ai * dt) + Bv[i] * dtx;
              }
            }
          }
          float y0 = 0.0f, y1 = 0.0f, y2 = 0.0f, y3 = 0.0f;
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            y0 = fmaf(hv[u][i], Cv[i], y0);
            y1 = fmaf(hv[u][i + 1], Cv[i + 1], y1);
            y2 = fmaf(hv[u][i + 2], Cv[i + 2], y2);
            y3 = fmaf(hv[u][i + 3], Cv[i + 3], y3);
          }
          y = (y0 + y1) + (y2 + y3);
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
  int hpc = 1;
  while (hpc * 2 <= heads_per_group && heads_per_group % (hpc * 2) == 0 &&
         static_cast<int64_t>(a.batch) * (a.heads / (hpc * 2)) >= 8LL * sms &&
         static_cast<size_t>(hpc * 2) * (2 * a.dim + 2) * sizeof(float) <= 48 * 1024)
    hpc *= 2;
  d.heads_per_cta = hpc;
  const size_t smem = static_cast<size_t>(hpc) * (2 * a.dim + 2) * sizeof(float);
  if (smem > 48 * 1024) return fail(LQ_ERR_UNSUPPORTED, "lq_dense_state_update: dim=%d too large", a.dim);
  const int64_t grid = static_cast<int64_t>(a.batch) * (a.heads / hpc);
  LQ_CHECK_ARG(grid <= 0x7FFFFFFFLL, "lq_dense_state_update: batch * heads too large");
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  switch (a.state_dtype) {
    case LQ_BF16: dense_state_update_kernel<LQ_BF16><<<static_cast<unsigned>(grid), kDenseThreads, smem, st>>>(a, d); break;
    case LQ_F16: dense_state_update_kernel<LQ_F16><<<static_cast<unsigned>(grid), kDenseThreads, smem, st>>>(a, d); break;
    default: dense_state_update_kernel<LQ_F32><<<static_cast<unsigned>(grid), kDenseThreads, smem, st>>>(a, d); break;
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
