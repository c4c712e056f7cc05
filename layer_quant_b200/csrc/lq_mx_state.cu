// Mamba2 selective-state update on an MX8 / MX4-held recurrent state, fused in one pass, plus the
// stand-alone MX codec kernels.  sm_100a.
//
// Work decomposition of the fused kernel: one CTA per (batch, head); inside it one lane owns one
// 16-value block of a row (so block maximum, pair maxima, exponent and micro-exponent bits never
// leave the thread), dstate/16 neighbouring lanes own one row, and the <h', C> read-out is a
// shuffle reduction over those lanes.  B and C of the head's group stay in registers for all
// `dim` rows.  Each lane moves 16 B of mantissas per row with one 128-bit load and one 128-bit
// store; the next row's loads are issued before the current row is computed.
//
// The kernel is bound by instruction issue, not by HBM, on B200: at 18 bytes per block read and
// written the memory system could deliver one value every ~12 issue slots per SM sub-partition,
// and decode + update + read-out + exponent + rounding + random bits need more than that.
#include <algorithm>
#include <cstdlib>

#include "lq_mx_codec.cuh"
#include "lq_ssm_operands.cuh"

namespace lq {

constexpr int kUpdateThreads = 128;
// the slab kernel runs two warps per CTA, eight CTAs per SM: the same sixteen warps per SM as four CTAs of four warps
// (the register file allows no more), cut into slabs half as large
constexpr int kFastThreads = 64;
constexpr int kFastCtasPerSm = 8;

// ---- block load / store in either storage layout -----------------------------------------------
struct MxRaw {
  uint4 q;        // 16 mantissa bytes (8 for packed MX4: x, y)
  uint32_t e;     // shared exponent byte
  uint32_t mic;   // micro-exponent bits, bit i = pair i
};

template <int BITS, int LAYOUT>
struct MxBlockIO {
  static constexpr bool kNibbles = (BITS == 4 && LAYOUT == LQ_MX_LAYOUT_PACKED);
  static constexpr int kQBytes = kNibbles ? 8 : 16;

  static constexpr int kMicroBytes = (LAYOUT == LQ_MX_LAYOUT_PACKED) ? 1 : 8;

  // One block through plain pointers (dense states: the caller does the address arithmetic once).  The state
  // is streamed: loads go to L2 only, which also keeps them coherent with a predecessor's stores when the
  // kernel was scheduled before that predecessor finished.
  __device__ __forceinline__ static MxRaw load_ptr(const uint8_t* q, const uint8_t* e, const uint8_t* m) {
    MxRaw r;
    if (kNibbles) {
      const uint2 v = __ldcg(reinterpret_cast<const uint2*>(q));
      r.q = make_uint4(v.x, v.y, 0u, 0u);
    } else {
      r.q = __ldcg(reinterpret_cast<const uint4*>(q));
    }
    r.e = __ldcg(e);
    if (LAYOUT == LQ_MX_LAYOUT_PACKED) {
      r.mic = __ldcg(m);
    } else {
      const uint2 mm = __ldcg(reinterpret_cast<const uint2*>(m));
      r.mic = (((mm.x & 0x01010101u) * 0x10204080u) >> 28) | ((((mm.y & 0x01010101u) * 0x10204080u) >> 28) << 4);
    }
    return r;
  }

  __device__ __forceinline__ static void store_ptr(uint8_t* q, uint8_t* e, uint8_t* m, const uint32_t (&codes)[4], uint32_t ev,
                                                   uint32_t mic) {
    if (kNibbles) {
      uint32_t lo, hi;
      mx4_bytes_to_nibbles(codes, lo, hi);
      *reinterpret_cast<uint2*>(q) = make_uint2(lo, hi);
    } else {
      *reinterpret_cast<uint4*>(q) = make_uint4(codes[0], codes[1], codes[2], codes[3]);
    }
    *e = static_cast<uint8_t>(ev);
    if (LAYOUT == LQ_MX_LAYOUT_PACKED) {
      *m = static_cast<uint8_t>(mic);
    } else {
      const uint32_t lo = ((mic & 0xFu) * 0x00204081u) & 0x01010101u;
      const uint32_t hi = (((mic >> 4) & 0xFu) * 0x00204081u) & 0x01010101u;
      *reinterpret_cast<uint2*>(m) = make_uint2(lo, hi);
    }
  }

  __device__ __forceinline__ static MxRaw load(const lq_mx_state& s, int64_t qrow, int64_t erow, int64_t mrow, int blk) {
    MxRaw r;
    const uint8_t* q = static_cast<const uint8_t*>(s.q_state) + qrow + blk * kQBytes;
    if (kNibbles) {
      const uint2 v = *reinterpret_cast<const uint2*>(q);
      r.q = make_uint4(v.x, v.y, 0u, 0u);
    } else {
      r.q = *reinterpret_cast<const uint4*>(q);
    }
    r.e = s.shared_exp[erow + blk];
    if (LAYOUT == LQ_MX_LAYOUT_PACKED) {
      r.mic = s.micro_exp[mrow + blk];
    } else {
      const uint2 m = *reinterpret_cast<const uint2*>(s.micro_exp + mrow + blk * 8);
      r.mic = (((m.x & 0x01010101u) * 0x10204080u) >> 28) | ((((m.y & 0x01010101u) * 0x10204080u) >> 28) << 4);
    }
    return r;
  }

  __device__ __forceinline__ static void codes_of(const MxRaw& r, uint32_t (&codes)[4]) {
    if (kNibbles) {
      mx4_nibbles_to_bytes(r.q.x, r.q.y, codes);
    } else {
      codes[0] = r.q.x; codes[1] = r.q.y; codes[2] = r.q.z; codes[3] = r.q.w;
    }
  }

  __device__ __forceinline__ static void store(const lq_mx_state& s, int64_t qrow, int64_t erow, int64_t mrow, int blk,
                                               const uint32_t (&codes)[4], uint32_t e, uint32_t mic) {
    uint8_t* q = static_cast<uint8_t*>(s.q_state) + qrow + blk * kQBytes;
    if (kNibbles) {
      uint32_t lo, hi;
      mx4_bytes_to_nibbles(codes, lo, hi);
      *reinterpret_cast<uint2*>(q) = make_uint2(lo, hi);
    } else {
      *reinterpret_cast<uint4*>(q) = make_uint4(codes[0], codes[1], codes[2], codes[3]);
    }
    s.shared_exp[erow + blk] = static_cast<uint8_t>(e);
    if (LAYOUT == LQ_MX_LAYOUT_PACKED) {
      s.micro_exp[mrow + blk] = static_cast<uint8_t>(mic);
    } else {
      const uint32_t lo = ((mic & 0xFu) * 0x00204081u) & 0x01010101u;
      const uint32_t hi = (((mic >> 4) & 0xFu) * 0x00204081u) & 0x01010101u;
      *reinterpret_cast<uint2*>(s.micro_exp + mrow + blk * 8) = make_uint2(lo, hi);
    }
  }
};

// Rounding state that is the same for every block a thread handles.  `numel` = values in the whole
// state: the reference advances its Philox offset by it every step.
struct MxRoundBase {
  uint32_t wrap32, step, layer;
  uint64_t offset;
  const uint32_t* words;
};

__device__ __forceinline__ MxRoundBase make_round_base(const lq_rounding& r, uint64_t numel) {
  MxRoundBase b;
  const uint64_t extra = r.step_counter ? __ldcg(reinterpret_cast<const unsigned long long*>(r.step_counter)) : 0ull;
  b.offset = r.rng_offset + extra * numel;
  b.wrap32 = b.offset < (1ull << 32) ? 1u : 0u;
  b.step = static_cast<uint32_t>(r.step + extra);
  b.layer = r.layer;
  b.words = r.words;
  return b;
}

// Context of the block whose first value has linear index `lin` (a multiple of 16).
template <int MODE>
__device__ __forceinline__ MxRoundCtx round_ctx_at(const MxRoundBase& b, uint64_t lin) {
  MxRoundCtx c;
  c.wrap32 = b.wrap32;
  c.counter = (MODE == LQ_ROUND_PHILOX_LAYERED) ? (lin >> 4) : (MODE == LQ_ROUND_PHILOX_LAYERED4) ? (lin >> 2) : (b.offset + lin);
  c.step = b.step;
  c.layer = b.layer;
  c.words = (MODE == LQ_ROUND_SUPPLIED || MODE == LQ_ROUND_SUPPLIED_FIXED) ? b.words + lin : nullptr;
  return c;
}

struct MxUpdateDerived {
  int32_t nblk;        // dstate / 16
  int32_t lpr_log2;    // lanes per row = 1 << lpr_log2 >= nblk
  int32_t dt_uniform;  // dt and dt_bias do not depend on the row (dim) index
  int32_t a_scalar;    // A depends on the head only
  int32_t heads_per_cta;  // consecutive heads of one B/C group handled by one CTA
  PhiloxKeys keys;        // round keys of rounding.seed
  uint64_t units_total;   // fast path: batch * heads * dim / rows per pass (< 2^31)
  // fast path: the slab of a CTA without a division.  units_per_cta / units_rem: CTA c owns units_per_cta units, the
  // first units_rem CTAs one more.  FastDiv: floor(n / d) for n < 2^31 as (mulhi(n, magic) + n) >> shift.
  uint32_t units_per_cta, units_rem;
  struct FastDiv { uint32_t magic, shift; } div_units_per_head, div_heads, div_dim, div_heads_per_group;
};

__device__ __forceinline__ uint32_t fast_div(uint32_t n, const MxUpdateDerived::FastDiv& f) { return (__umulhi(n, f.magic) + n) >> f.shift; }

// One CTA = `hpc` consecutive heads of one (batch, B/C group): B and C are fetched once and stay in
// registers for hpc * dim rows.  gridDim.x = batch * (heads / hpc).
template <int BITS, int LAYOUT, int MODE>
__global__ void __launch_bounds__(kUpdateThreads, 4) mx_state_update_kernel(const lq_mx_update_args a, const MxUpdateDerived d) {
  using IO = MxBlockIO<BITS, LAYOUT>;
  extern __shared__ float smem_xy[];  // x of the CTA's rows, <h', C> of the rows, per-head dt and exp(A dt)
  const lq_mx_state& s = a.state;
  const int H = s.heads, P = s.dim, N = s.dstate;
  const int hpc = d.heads_per_cta;
  float* sx = smem_xy;
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
  const int rows_per_pass = rows_per_warp * (kUpdateThreads / 32);
  const bool blk_ok = blk < d.nblk;
  const int n0 = blk * 16;
  const int grp = h0 / (H / a.ngroups);  // the same for every head of the CTA
  const unsigned int* cut = mx_exp_cut_table<BITS>();

  auto row_dt = [&](int h, int p) {
    float dt = load_as_float(a.dt, b * a.dt_stride[0] + h * a.dt_stride[1] + p * a.dt_stride[2], a.dt_dtype);
    if (a.dt_bias) dt += load_as_float(a.dt_bias, h * a.dt_bias_stride[0] + p * a.dt_bias_stride[1], a.dt_bias_dtype);
    if (a.dt_softplus) dt = softplus_ref(dt);
    return dt;
  };
  for (int i = threadIdx.x; i < hpc * P; i += kUpdateThreads) {
    const int hh = i / P, p = i - hh * P;
    sx[i] = load_as_float(a.x, b * a.x_stride[0] + (h0 + hh) * a.x_stride[1] + p * a.x_stride[2], a.x_dtype);
  }
  if (d.dt_uniform && threadIdx.x < hpc) {
    const float dt = row_dt(h0 + threadIdx.x, 0);
    sdt[threadIdx.x] = dt;
    sdA[threadIdx.x] = d.a_scalar ? expf(load_as_float(a.A, (h0 + threadIdx.x) * a.A_stride[0], a.A_dtype) * dt) : 0.0f;
  }

  // B and C of the group, this lane's 16 columns
  float Bv[16], Cv[16];
  if (blk_ok) {
    load_bc16(a.B, a.B_stride, a.B_dtype, b, grp, n0, Bv);
    load_bc16(a.C, a.C_stride, a.C_dtype, b, grp, n0, Cv);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) Bv[i] = Cv[i] = 0.0f;
  }
  const bool hoisted = d.dt_uniform && d.a_scalar;
  const MxRoundBase rb = make_round_base(a.rounding, static_cast<uint64_t>(s.batch) * H * P * N);
  __syncthreads();

#pragma unroll 1
  for (int hh = 0; hh < hpc; ++hh) {
    const int h = h0 + hh;
    const float dt_h = d.dt_uniform ? sdt[hh] : 0.0f;
    const float dA_h = sdA[hh];
    const uint64_t lin_head = (static_cast<uint64_t>(b) * H + h) * P * static_cast<uint64_t>(N) + n0;
    const int64_t qbase = b * s.q_stride[0] + h * s.q_stride[1];
    const int64_t ebase = b * s.exp_stride[0] + h * s.exp_stride[1];
    const int64_t mbase = b * s.micro_stride[0] + h * s.micro_stride[1];
    const float* sxh = sx + hh * P;
    float* syh = sy + hh * P;

    int p0 = warp * rows_per_warp;
    MxRaw cur = {make_uint4(0, 0, 0, 0), 127u, 0u};
    if (blk_ok && p0 + rsub < P)
      cur = IO::load(s, qbase + (p0 + rsub) * s.q_stride[2], ebase + (p0 + rsub) * s.exp_stride[2],
                     mbase + (p0 + rsub) * s.micro_stride[2], blk);
#pragma unroll 1
    for (; p0 < P; p0 += rows_per_pass) {
      const int p = p0 + rsub;
      const bool active = blk_ok && p < P;
      // issue the next row's loads before working on this one
      const int pn = p + rows_per_pass;
      MxRaw nxt = {make_uint4(0, 0, 0, 0), 127u, 0u};
      if (blk_ok && pn < P)
        nxt = IO::load(s, qbase + pn * s.q_stride[2], ebase + pn * s.exp_stride[2], mbase + pn * s.micro_stride[2], blk);

      float y = 0.0f;
      if (active) {
        uint32_t codes[4];
        IO::codes_of(cur, codes);
        float hv[16];
        mx_decode_block(codes, cur.e, cur.mic, hv);
        const float xv = sxh[p];
        if (hoisted) {
          y = mx_update_readout16(hv, Bv, Cv, dA_h, dt_h, xv);  // h' = h exp(A dt) + (B dt) x
        } else {
          const float dt = d.dt_uniform ? dt_h : row_dt(h, p);
          if (d.a_scalar) {
            y = mx_update_readout16(hv, Bv, Cv, expf(load_as_float(a.A, h * a.A_stride[0], a.A_dtype) * dt), dt, xv);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float Ai = load_as_float(a.A, h * a.A_stride[0] + p * a.A_stride[1] + (n0 + i) * a.A_stride[2], a.A_dtype);
              hv[i] = fmaf(hv[i], expf(Ai * dt), __fmul_rn(__fmul_rn(Bv[i], dt), xv));
            }
            float y0 = 0.0f, y1 = 0.0f, y2 = 0.0f, y3 = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
              y0 = fmaf(hv[i], Cv[i], y0);
              y1 = fmaf(hv[i + 1], Cv[i + 1], y1);
              y2 = fmaf(hv[i + 2], Cv[i + 2], y2);
              y3 = fmaf(hv[i + 3], Cv[i + 3], y3);
            }
            y = (y0 + y1) + (y2 + y3);
          }
        }
        const uint64_t lin = lin_head + static_cast<uint64_t>(static_cast<uint32_t>(p) * static_cast<uint32_t>(N));
        if (a.h_out) {
          float4* dst = reinterpret_cast<float4*>(a.h_out + lin);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = make_float4(hv[4 * i], hv[4 * i + 1], hv[4 * i + 2], hv[4 * i + 3]);
        }
        const MxRoundCtx ctx = round_ctx_at<MODE>(rb, lin);
        uint32_t e_new, mic_new;
        mx_encode_block<BITS, MODE>(hv, cut, ctx, d.keys, codes, e_new, mic_new);
        IO::store(s, qbase + p * s.q_stride[2], ebase + p * s.exp_stride[2], mbase + p * s.micro_stride[2], blk, codes, e_new,
                  mic_new);
      }
      // y = <h', C> over the row: reduce across the lanes that share it
      for (int o = (1 << d.lpr_log2) >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xFFFFFFFFu, y, o);
      if (active && blk == 0) syh[p] = y;
      cur = nxt;
    }
  }
  __syncthreads();
  // y = <h', C> + D x (* z), stored for all the CTA's rows at once
  for (int i = threadIdx.x; i < hpc * P; i += kUpdateThreads) {
    const int hh = i / P, p = i - hh * P, h = h0 + hh;
    float y = sy[i];
    if (a.D) y += sx[i] * load_as_float(a.D, h * a.D_stride[0] + p * a.D_stride[1], a.D_dtype);
    if (a.z) y *= load_as_float(a.z, b * a.z_stride[0] + h * a.z_stride[1] + p * a.z_stride[2], a.z_dtype);
    store_from_float(a.out, b * a.out_stride[0] + h * a.out_stride[1] + p * a.out_stride[2], a.out_dtype, y);
  }
}

// Fast path of the fused update: the shape every Mamba2 decode step has.  Requirements (checked
// on the host): dense state tensors, dt / dt_bias / A per head only, dstate / 16 a power of two,
// dim a multiple of the rows one CTA pass covers, no h_out, fewer than 2^31 units.
//
// Work is cut into units of `rows_per_pass` consecutive rows (one pass of the CTA's two warps).
// Units are numbered in memory order and dealt out contiguously, U / G to each of the G CTAs and one
// more to the first U mod G: a contiguous
// slab of the state, balanced to within one unit whatever the batch, and the grid is one wave of
// resident CTAs whenever the slab's x / y staging fits in shared memory.  Every lane is always
// active, the three state pointers move by a constant per pass (also across head boundaries), and
// B / C are reloaded only when the slab crosses into another (batch, B/C group).
// NBLK_T = dstate / 16 when known at compile time (8 for Nemotron-H: all lane and address arithmetic
// folds to constants and the read-out reduction unrolls), 0 = taken from the arguments.
template <int BITS, int LAYOUT, int MODE, int NBLK_T>
__global__ void __launch_bounds__(kFastThreads, kFastCtasPerSm) mx_state_update_fast_kernel(const lq_mx_update_args a, const MxUpdateDerived d) {
  using IO = MxBlockIO<BITS, LAYOUT>;
  extern __shared__ float smem_xy[];
  const lq_mx_state& s = a.state;
  const int H = s.heads, P = s.dim;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nblk = NBLK_T ? NBLK_T : d.nblk;
  const int lpr_log2 = NBLK_T == 8 ? 3 : d.lpr_log2;
  const int dstate = NBLK_T ? NBLK_T * 16 : s.dstate;
  const int blk = lane & (nblk - 1);
  const int rsub = lane >> lpr_log2;
  const int rows_per_warp = 32 >> lpr_log2;
  const int rows_per_pass = rows_per_warp * (kFastThreads / 32);
  const int units_per_head = P / rows_per_pass;
  const int heads_per_group = H / a.ngroups;
  const int n0 = blk * 16;
  const unsigned int* cut = mx_exp_cut_table<BITS>();

  // this CTA's slab: units [u0, u1), rows [R0, R1) of the [batch * heads * dim] row space; the first units_rem CTAs
  // take one unit more than the others
  const uint32_t u0 = blockIdx.x * d.units_per_cta + min(blockIdx.x, d.units_rem);
  const int n_units = static_cast<int>(d.units_per_cta + (blockIdx.x < d.units_rem ? 1u : 0u));
  const uint32_t u1 = u0 + n_units;
  // let the next kernel in the stream be scheduled behind this one (no effect without the launch attribute)
  asm volatile("griddepcontrol.launch_dependents;");
  if (n_units == 0) return;
  const uint64_t R0 = static_cast<uint64_t>(u0) * rows_per_pass;
  const int n_rows = n_units * rows_per_pass;
  const uint32_t bh_first = fast_div(u0, d.div_units_per_head);  // first (batch * heads + head) index touched
  const int n_heads = static_cast<int>(fast_div(u1 - 1, d.div_units_per_head) - bh_first) + 1;
  float* sx = smem_xy;        // x of the slab's rows
  // read-out of the slab's rows: one partial sum per 16-value block when a row spans eight lanes (added up when
  // the slab's y is written, in the order a butterfly over the eight lanes would add them), else the row's sum
  float* sy = sx + n_rows;
  float* sdt = sy + n_rows * (NBLK_T == 8 ? 8 : 1);   // per touched head
  float* sdA = sdt + n_heads;

  // (batch, head, row) of the slab's first row, once per CTA
  const int unit_in_head0 = static_cast<int>(u0 - bh_first * static_cast<uint32_t>(units_per_head));
  const int p_first = unit_in_head0 * rows_per_pass;
  const int b_first = static_cast<int>(fast_div(bh_first, d.div_heads));
  const int h_first = static_cast<int>(bh_first - static_cast<uint32_t>(b_first) * static_cast<uint32_t>(H));
  auto row_coords = [&](int i, int& b, int& h, int& p) {
    const uint32_t pi = static_cast<uint32_t>(p_first + i);
    const uint32_t hq = fast_div(pi, d.div_dim);
    p = static_cast<int>(pi - hq * static_cast<uint32_t>(P));
    const uint32_t hh = static_cast<uint32_t>(h_first) + hq;
    const uint32_t bq = fast_div(hh, d.div_heads);
    b = b_first + static_cast<int>(bq);
    h = static_cast<int>(hh - bq * static_cast<uint32_t>(H));
  };
  const uint32_t q_row = nblk * IO::kQBytes, m_row = nblk * IO::kMicroBytes, e_row = nblk;
  const uint32_t r_first = warp * rows_per_warp + rsub;
  // this lane's block of its first row; every pass moves all three pointers by a constant
  uint8_t* qptr = static_cast<uint8_t*>(s.q_state) + (R0 + r_first) * q_row + blk * IO::kQBytes;
  uint8_t* eptr = s.shared_exp + (R0 + r_first) * e_row + blk;
  uint8_t* mptr = s.micro_exp + (R0 + r_first) * m_row + blk * IO::kMicroBytes;
  // linear index of the block's first value, kept pre-shifted to the Philox counter in the layered modes (block index /
  // quad index), so that the loop carries the counter itself
  constexpr int kCtrShift = MODE == LQ_ROUND_PHILOX_LAYERED ? 4 : (MODE == LQ_ROUND_PHILOX_LAYERED4 ? 2 : 0);
  uint64_t lin = ((R0 + r_first) * dstate + n0) >> kCtrShift;
  uint32_t row = r_first;
  const uint32_t dq = rows_per_pass * q_row, de = rows_per_pass * e_row, dm = rows_per_pass * m_row,
                 dl = (rows_per_pass * dstate) >> kCtrShift;
  // everything above is arithmetic on the arguments; from here on memory the predecessor may have written is read
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // the first row's block travels while the operands below are staged
  MxRaw cur = IO::load_ptr(qptr, eptr, mptr);

  for (int i = threadIdx.x; i < n_rows; i += kFastThreads) {
    int b, h, p;
    row_coords(i, b, h, p);
    sx[i] = load_as_float(a.x, b * a.x_stride[0] + h * a.x_stride[1] + p * a.x_stride[2], a.x_dtype);
  }
  for (int i = threadIdx.x; i < n_heads; i += kFastThreads) {
    const unsigned hh = static_cast<unsigned>(h_first + i);
    const int h = static_cast<int>(hh % static_cast<unsigned>(H)), b = b_first + static_cast<int>(hh / static_cast<unsigned>(H));
    float dt = load_as_float(a.dt, b * a.dt_stride[0] + h * a.dt_stride[1], a.dt_dtype);
    if (a.dt_bias) dt += load_as_float(a.dt_bias, h * a.dt_bias_stride[0], a.dt_bias_dtype);
    if (a.dt_softplus) dt = softplus_ref(dt);
    sdt[i] = dt;
    sdA[i] = expf(load_as_float(a.A, h * a.A_stride[0], a.A_dtype) * dt);
  }
  // position of the first unit: head index inside the slab, unit inside the head, head inside its group
  int head_i = 0;
  int unit_in_head = unit_in_head0;
  int b_cur = b_first;
  int g_cur = static_cast<int>(fast_div(static_cast<uint32_t>(h_first), d.div_heads_per_group));  // B / C group of the current head ...
  int h_in_group = h_first - g_cur * heads_per_group;    // ... and the head's place in it: advanced without divisions
  float Bv[16], Cv[16];
  load_bc16(a.B, a.B_stride, a.B_dtype, b_cur, g_cur, n0, Bv);
  load_bc16(a.C, a.C_stride, a.C_dtype, b_cur, g_cur, n0, Cv);
  const MxRoundBase rb = make_round_base(a.rounding, static_cast<uint64_t>(s.batch) * H * P * dstate);

  __syncthreads();

  int u = 0;
#pragma unroll 1
  while (u < n_units) {
    // units of one head
    const float dt_h = sdt[head_i], dA_h = sdA[head_i];
    const int u_head_end = min(n_units, u + units_per_head - unit_in_head);
#pragma unroll 1
    for (; u < u_head_end; ++u) {
      uint8_t* const qn = qptr + dq;
      uint8_t* const en = eptr + de;
      uint8_t* const mn = mptr + dm;
      MxRaw nxt = cur;
      if (u + 1 < n_units) nxt = IO::load_ptr(qn, en, mn);

      uint32_t codes[4];
      IO::codes_of(cur, codes);
      float hv[16];
      mx_decode_block(codes, cur.e, cur.mic, hv);
      float y = mx_update_readout16(hv, Bv, Cv, dA_h, dt_h, sx[row]);  // h' = h exp(A dt) + (B dt) x

      MxRoundCtx ctx = round_ctx_at<MODE>(rb, lin << kCtrShift);
      if (kCtrShift) ctx.counter = lin;
      uint32_t e_new, mic_new;
      mx_encode_block<BITS, MODE>(hv, cut, ctx, d.keys, codes, e_new, mic_new);
      IO::store_ptr(qptr, eptr, mptr, codes, e_new, mic_new);

      if (NBLK_T == 8) {
        sy[row * 8 + blk] = y;
      } else {
        for (int o = nblk >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xFFFFFFFFu, y, o);
        if (blk == 0) sy[row] = y;
      }
      cur = nxt;
      qptr = qn; eptr = en; mptr = mn;
      lin += dl;
      row += rows_per_pass;
    }
    // the next unit, if any, starts another head; B / C change only with the (batch, group)
    unit_in_head = 0;
    ++head_i;
    if (u < n_units && ++h_in_group == heads_per_group) {
      h_in_group = 0;
      if (++g_cur == a.ngroups) {
        g_cur = 0;
        ++b_cur;
      }
      load_bc16(a.B, a.B_stride, a.B_dtype, b_cur, g_cur, n0, Bv);
      load_bc16(a.C, a.C_stride, a.C_dtype, b_cur, g_cur, n0, Cv);
    }
  }
  __syncthreads();
  // y = <h', C> + D x (* z), stored for the whole slab at once
  for (int i = threadIdx.x; i < n_rows; i += kFastThreads) {
    int b, h, p;
    row_coords(i, b, h, p);
    float y;
    if (NBLK_T == 8) {
      const float4 p0 = *reinterpret_cast<const float4*>(sy + i * 8), p1 = *reinterpret_cast<const float4*>(sy + i * 8 + 4);
      y = ((p0.x + p1.x) + (p0.z + p1.z)) + ((p0.y + p1.y) + (p0.w + p1.w));  // the butterfly's order
    } else {
      y = sy[i];
    }
    if (a.D) y += sx[i] * load_as_float(a.D, h * a.D_stride[0] + p * a.D_stride[1], a.D_dtype);
    if (a.z) y *= load_as_float(a.z, b * a.z_stride[0] + h * a.z_stride[1] + p * a.z_stride[2], a.z_dtype);
    store_from_float(a.out, b * a.out_stride[0] + h * a.out_stride[1] + p * a.out_stride[2], a.out_dtype, y);
  }
}

// ---- stand-alone codec kernels: one thread per 16-value block ----------------------------------
template <int BITS, int LAYOUT, int MODE>
__global__ void mx_quantize_kernel(const lq_mx_state s, const void* __restrict__ src, int src_dtype, int64_t src_row_stride,
                                   const lq_rounding rnd, const PhiloxKeys keys, int64_t total_blocks) {
  using IO = MxBlockIO<BITS, LAYOUT>;
  const int nblk = s.dstate / 16;
  const unsigned int* cut = mx_exp_cut_table<BITS>();
  const MxRoundBase rb = make_round_base(rnd, static_cast<uint64_t>(s.batch) * s.heads * s.dim * s.dstate);
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < total_blocks;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = t / nblk;
    const int blk = static_cast<int>(t - row * nblk);
    const int p = static_cast<int>(row % s.dim);
    const int64_t bh = row / s.dim;
    const int h = static_cast<int>(bh % s.heads);
    const int64_t b = bh / s.heads;
    float hv[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) hv[i] = load_as_float(src, row * src_row_stride + blk * 16 + i, src_dtype);
    const uint64_t lin = static_cast<uint64_t>(row) * s.dstate + blk * 16;
    const MxRoundCtx ctx = round_ctx_at<MODE>(rb, lin);
    uint32_t codes[4], e, mic;
    mx_encode_block<BITS, MODE>(hv, cut, ctx, keys, codes, e, mic);
    IO::store(s, b * s.q_stride[0] + h * s.q_stride[1] + p * s.q_stride[2],
              b * s.exp_stride[0] + h * s.exp_stride[1] + p * s.exp_stride[2],
              b * s.micro_stride[0] + h * s.micro_stride[1] + p * s.micro_stride[2], blk, codes, e, mic);
  }
}

template <int BITS, int LAYOUT>
__global__ void mx_dequantize_kernel(const lq_mx_state s, float* __restrict__ dst, int64_t dst_row_stride, int64_t total_blocks) {
  using IO = MxBlockIO<BITS, LAYOUT>;
  const int nblk = s.dstate / 16;
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < total_blocks;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = t / nblk;
    const int blk = static_cast<int>(t - row * nblk);
    const int p = static_cast<int>(row % s.dim);
    const int64_t bh = row / s.dim;
    const int h = static_cast<int>(bh % s.heads);
    const int64_t b = bh / s.heads;
    const MxRaw r = IO::load(s, b * s.q_stride[0] + h * s.q_stride[1] + p * s.q_stride[2],
                             b * s.exp_stride[0] + h * s.exp_stride[1] + p * s.exp_stride[2],
                             b * s.micro_stride[0] + h * s.micro_stride[1] + p * s.micro_stride[2], blk);
    uint32_t codes[4];
    IO::codes_of(r, codes);
    float hv[16];
    mx_decode_block(codes, r.e, r.mic, hv);
#pragma unroll
    for (int i = 0; i < 16; ++i) dst[row * dst_row_stride + blk * 16 + i] = hv[i];
  }
}

template <int BITS, int SRC_LAYOUT, int DST_LAYOUT>
__global__ void mx_convert_kernel(const lq_mx_state src, const lq_mx_state dst, int64_t total_blocks) {
  using IOS = MxBlockIO<BITS, SRC_LAYOUT>;
  using IOD = MxBlockIO<BITS, DST_LAYOUT>;
  const int nblk = src.dstate / 16;
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < total_blocks;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = t / nblk;
    const int blk = static_cast<int>(t - row * nblk);
    const int p = static_cast<int>(row % src.dim);
    const int64_t bh = row / src.dim;
    const int h = static_cast<int>(bh % src.heads);
    const int64_t b = bh / src.heads;
    const MxRaw r = IOS::load(src, b * src.q_stride[0] + h * src.q_stride[1] + p * src.q_stride[2],
                              b * src.exp_stride[0] + h * src.exp_stride[1] + p * src.exp_stride[2],
                              b * src.micro_stride[0] + h * src.micro_stride[1] + p * src.micro_stride[2], blk);
    uint32_t codes[4];
    IOS::codes_of(r, codes);
    IOD::store(dst, b * dst.q_stride[0] + h * dst.q_stride[1] + p * dst.q_stride[2],
               b * dst.exp_stride[0] + h * dst.exp_stride[1] + p * dst.exp_stride[2],
               b * dst.micro_stride[0] + h * dst.micro_stride[1] + p * dst.micro_stride[2], blk, codes, r.e, r.mic);
  }
}

__global__ void counter_add_kernel(unsigned long long* counter, unsigned long long inc) { *counter += inc; }

// ---- host side --------------------------------------------------------------------------------
static int validate_state(const lq_mx_state& s, const char* who) {
  LQ_CHECK_ARG(s.q_state && s.shared_exp && s.micro_exp, "%s: null state pointer", who);
  LQ_CHECK_ARG(s.format_bits == 8 || s.format_bits == 4, "%s: Only MX8 and MX4 state quantization are supported, got format_bits=%d",
               who, s.format_bits);
  LQ_CHECK_ARG(s.layout == LQ_MX_LAYOUT_REFERENCE || s.layout == LQ_MX_LAYOUT_PACKED, "%s: unknown layout %d", who, s.layout);
  LQ_CHECK_ARG(s.batch > 0 && s.heads > 0 && s.dim > 0 && s.dstate > 0, "%s: empty state [%d,%d,%d,%d]", who, s.batch,
               s.heads, s.dim, s.dstate);
  LQ_CHECK_ARG(s.dstate % 16 == 0, "%s: MX%d state dim must be divisible by 16, got %d", who, s.format_bits, s.dstate);
  LQ_CHECK_ARG(static_cast<int64_t>(s.batch) * s.heads < (1ll << 31), "%s: batch*heads too large", who);
  const bool nib = s.format_bits == 4 && s.layout == LQ_MX_LAYOUT_PACKED;
  const int qalign = nib ? 8 : 16;
  LQ_CHECK_ARG(reinterpret_cast<uintptr_t>(s.q_state) % qalign == 0, "%s: q_state must be %d-byte aligned", who, qalign);
  for (int i = 0; i < 3; ++i)
    LQ_CHECK_ARG(s.q_stride[i] % qalign == 0, "%s: q_state strides must be multiples of %d bytes", who, qalign);
  if (s.layout == LQ_MX_LAYOUT_REFERENCE) {
    LQ_CHECK_ARG(reinterpret_cast<uintptr_t>(s.micro_exp) % 8 == 0, "%s: micro_exp must be 8-byte aligned", who);
    for (int i = 0; i < 3; ++i) LQ_CHECK_ARG(s.micro_stride[i] % 8 == 0, "%s: micro_exp strides must be multiples of 8", who);
  }
  return LQ_OK;
}

static int validate_rounding(const lq_rounding& r, const char* who) {
  LQ_CHECK_ARG(r.mode >= LQ_ROUND_HALF_UP && r.mode <= LQ_ROUND_PHILOX_LAYERED4, "%s: unknown rounding mode %d", who, r.mode);
  if (r.mode == LQ_ROUND_SUPPLIED || r.mode == LQ_ROUND_SUPPLIED_FIXED) {
    LQ_CHECK_ARG(r.words != nullptr, "%s: rounding mode %d needs words", who, r.mode);
    LQ_CHECK_ARG(reinterpret_cast<uintptr_t>(r.words) % 16 == 0, "%s: rounding words must be 16-byte aligned", who);
  }
  LQ_CHECK_ARG(reinterpret_cast<uintptr_t>(r.step_counter) % 8 == 0, "%s: step_counter must be 8-byte aligned", who);
  return LQ_OK;
}

template <int BITS, int LAYOUT>
static bool fast_update_applies(const lq_mx_update_args& a, const MxUpdateDerived& d) {
  using IO = MxBlockIO<BITS, LAYOUT>;
  const lq_mx_state& s = a.state;
  const int64_t q_row = static_cast<int64_t>(d.nblk) * IO::kQBytes, m_row = static_cast<int64_t>(d.nblk) * IO::kMicroBytes;
  const int rows_per_pass = (32 >> d.lpr_log2) * (kFastThreads / 32);
  const bool dense = s.q_stride[2] == q_row && s.q_stride[1] == q_row * s.dim && s.q_stride[0] == q_row * s.dim * s.heads &&
                     s.exp_stride[2] == d.nblk && s.exp_stride[1] == static_cast<int64_t>(d.nblk) * s.dim &&
                     s.exp_stride[0] == static_cast<int64_t>(d.nblk) * s.dim * s.heads && s.micro_stride[2] == m_row &&
                     s.micro_stride[1] == m_row * s.dim && s.micro_stride[0] == m_row * s.dim * s.heads;
  // fewer than 2^31 units keep the kernel's index arithmetic in 32 bits and its multiply-high divisions exact
  const uint64_t units = static_cast<uint64_t>(s.batch) * s.heads * (s.dim / rows_per_pass);
  return dense && d.dt_uniform && d.a_scalar && a.h_out == nullptr && (1 << d.lpr_log2) == d.nblk &&
         s.dim % rows_per_pass == 0 && units < (1ull << 31);
}

template <int BITS, int LAYOUT>
static void launch_update_mode(const lq_mx_update_args& a, const MxUpdateDerived& d, cudaStream_t st) {
  if (fast_update_applies<BITS, LAYOUT>(a, d)) {
    // One wave of resident CTAs (8 per SM) when a CTA's slab stays within kMaxUnitsPerCta units
    // (its x / y staging in shared memory: 36 bytes per row, 18 KB per CTA at most); more waves of equally sized
    // slabs otherwise.
    uint64_t kMaxUnitsPerCta = 64;
    if (const char* env = getenv("LQ_MX_MAX_UNITS")) kMaxUnitsPerCta = std::min(80, std::max(1, atoi(env)));  // tuning aid; 80 units stay under 48 KB
    const int rows_per_pass = (32 >> d.lpr_log2) * (kFastThreads / 32);
    MxUpdateDerived dd = d;
    dd.units_total = static_cast<uint64_t>(a.state.batch) * a.state.heads * (a.state.dim / rows_per_pass);
    const uint64_t wave = static_cast<uint64_t>(kFastCtasPerSm) * sm_count();
    uint64_t ctas = std::min<uint64_t>(dd.units_total, wave);
    if (dd.units_total > ctas * kMaxUnitsPerCta) {
      ctas = (dd.units_total + kMaxUnitsPerCta - 1) / kMaxUnitsPerCta;
      ctas = (ctas + wave - 1) / wave * wave;
    }
    dd.units_per_cta = static_cast<uint32_t>(dd.units_total / ctas);
    dd.units_rem = static_cast<uint32_t>(dd.units_total % ctas);
    auto fast_div_of = [](uint32_t dv) {
      MxUpdateDerived::FastDiv f;
      f.shift = 0;
      while ((1ull << f.shift) < dv) ++f.shift;  // ceil(log2 dv)
      f.magic = static_cast<uint32_t>(((1ull << (32 + f.shift)) + dv - 1) / dv - (1ull << 32));
      return f;
    };
    dd.div_units_per_head = fast_div_of(static_cast<uint32_t>(a.state.dim / rows_per_pass));
    dd.div_heads = fast_div_of(static_cast<uint32_t>(a.state.heads));
    dd.div_dim = fast_div_of(static_cast<uint32_t>(a.state.dim));
    dd.div_heads_per_group = fast_div_of(static_cast<uint32_t>(a.state.heads / a.ngroups));
    const uint64_t max_units = (dd.units_total + ctas - 1) / ctas;
    const uint64_t max_heads = max_units / (a.state.dim / rows_per_pass) + 2;
    const dim3 grid(static_cast<unsigned>(ctas)), block(kFastThreads);
    const size_t smem = sizeof(float) * ((d.nblk == 8 ? 9 : 2) * max_units * rows_per_pass + 2 * max_heads);
    const MxUpdateDerived& d = dd;
    // Programmatic dependent launch: the kernel may be scheduled while its predecessor in the stream is still
    // running (its CTAs take the slots the predecessor's CTAs leave); it touches no global memory before its
    // griddepcontrol.wait, which returns once the predecessor has completed and its writes are visible.
    static const bool pdl = [] {
      const char* env = getenv("LQ_MX_PDL");
      return env == nullptr || atoi(env) != 0;
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
#define LQ_FAST_LAUNCH(MODE_)                                                                         \
  do {                                                                                               \
    if (d.nblk == 8) cudaLaunchKernelEx(&cfg, mx_state_update_fast_kernel<BITS, LAYOUT, MODE_, 8>, a, d); \
    else cudaLaunchKernelEx(&cfg, mx_state_update_fast_kernel<BITS, LAYOUT, MODE_, 0>, a, d);         \
  } while (0)
    switch (a.rounding.mode) {
      case LQ_ROUND_HALF_UP: LQ_FAST_LAUNCH(LQ_ROUND_HALF_UP); break;
      case LQ_ROUND_HALF_EVEN: LQ_FAST_LAUNCH(LQ_ROUND_HALF_EVEN); break;
      case LQ_ROUND_PHILOX_REF: LQ_FAST_LAUNCH(LQ_ROUND_PHILOX_REF); break;
      case LQ_ROUND_SUPPLIED: LQ_FAST_LAUNCH(LQ_ROUND_SUPPLIED); break;
      case LQ_ROUND_PHILOX_LAYERED: LQ_FAST_LAUNCH(LQ_ROUND_PHILOX_LAYERED); break;
      case LQ_ROUND_PHILOX_LAYERED4: LQ_FAST_LAUNCH(LQ_ROUND_PHILOX_LAYERED4); break;
      default: LQ_FAST_LAUNCH(LQ_ROUND_SUPPLIED_FIXED); break;
    }
#undef LQ_FAST_LAUNCH
    return;
  }
  const dim3 grid(a.state.batch * (a.state.heads / d.heads_per_cta)), block(kUpdateThreads);
  const size_t smem = sizeof(float) * (2 * static_cast<size_t>(d.heads_per_cta) * a.state.dim + 2 * d.heads_per_cta);
  switch (a.rounding.mode) {
    case LQ_ROUND_HALF_UP: mx_state_update_kernel<BITS, LAYOUT, LQ_ROUND_HALF_UP><<<grid, block, smem, st>>>(a, d); break;
    case LQ_ROUND_HALF_EVEN: mx_state_update_kernel<BITS, LAYOUT, LQ_ROUND_HALF_EVEN><<<grid, block, smem, st>>>(a, d); break;
    case LQ_ROUND_PHILOX_REF: mx_state_update_kernel<BITS, LAYOUT, LQ_ROUND_PHILOX_REF><<<grid, block, smem, st>>>(a, d); break;
    case LQ_ROUND_SUPPLIED: mx_state_update_kernel<BITS, LAYOUT, LQ_ROUND_SUPPLIED><<<grid, block, smem, st>>>(a, d); break;
    case LQ_ROUND_PHILOX_LAYERED: mx_state_update_kernel<BITS, LAYOUT, LQ_ROUND_PHILOX_LAYERED><<<grid, block, smem, st>>>(a, d); break;
    case LQ_ROUND_PHILOX_LAYERED4: mx_state_update_kernel<BITS, LAYOUT, LQ_ROUND_PHILOX_LAYERED4><<<grid, block, smem, st>>>(a, d); break;
    default: mx_state_update_kernel<BITS, LAYOUT, LQ_ROUND_SUPPLIED_FIXED><<<grid, block, smem, st>>>(a, d); break;
  }
}

template <int BITS, int LAYOUT>
static void launch_quantize_mode(const lq_mx_state& s, const void* src, int dt, int64_t stride, const lq_rounding& r,
                                 int64_t total, cudaStream_t st) {
  const int block = 128;
  const int grid = static_cast<int>(std::min<int64_t>((total + block - 1) / block, 1 << 20));
  const PhiloxKeys keys = make_philox_keys(r.seed);
  switch (r.mode) {
    case LQ_ROUND_HALF_UP: mx_quantize_kernel<BITS, LAYOUT, LQ_ROUND_HALF_UP><<<grid, block, 0, st>>>(s, src, dt, stride, r, keys, total); break;
    case LQ_ROUND_HALF_EVEN: mx_quantize_kernel<BITS, LAYOUT, LQ_ROUND_HALF_EVEN><<<grid, block, 0, st>>>(s, src, dt, stride, r, keys, total); break;
    case LQ_ROUND_PHILOX_REF: mx_quantize_kernel<BITS, LAYOUT, LQ_ROUND_PHILOX_REF><<<grid, block, 0, st>>>(s, src, dt, stride, r, keys, total); break;
    case LQ_ROUND_SUPPLIED: mx_quantize_kernel<BITS, LAYOUT, LQ_ROUND_SUPPLIED><<<grid, block, 0, st>>>(s, src, dt, stride, r, keys, total); break;
    case LQ_ROUND_PHILOX_LAYERED: mx_quantize_kernel<BITS, LAYOUT, LQ_ROUND_PHILOX_LAYERED><<<grid, block, 0, st>>>(s, src, dt, stride, r, keys, total); break;
    case LQ_ROUND_PHILOX_LAYERED4: mx_quantize_kernel<BITS, LAYOUT, LQ_ROUND_PHILOX_LAYERED4><<<grid, block, 0, st>>>(s, src, dt, stride, r, keys, total); break;
    default: mx_quantize_kernel<BITS, LAYOUT, LQ_ROUND_SUPPLIED_FIXED><<<grid, block, 0, st>>>(s, src, dt, stride, r, keys, total); break;
  }
}

#define LQ_DISPATCH_BITS_LAYOUT(bits, layout, CALL)                                   \
  do {                                                                                \
    if ((bits) == 8 && (layout) == LQ_MX_LAYOUT_REFERENCE) { CALL(8, LQ_MX_LAYOUT_REFERENCE); } \
    else if ((bits) == 8) { CALL(8, LQ_MX_LAYOUT_PACKED); }                           \
    else if ((layout) == LQ_MX_LAYOUT_REFERENCE) { CALL(4, LQ_MX_LAYOUT_REFERENCE); } \
    else { CALL(4, LQ_MX_LAYOUT_PACKED); }                                            \
  } while (0)

}  // namespace lq

using namespace lq;

LQ_EXPORT int lq_mx_state_update(const lq_mx_update_args* args, void* cuda_stream) {
  LQ_CHECK_ARG(args != nullptr, "lq_mx_state_update: null args");
  const lq_mx_update_args& a = *args;
  if (int rc = validate_state(a.state, "lq_mx_state_update")) return rc;
  if (int rc = validate_rounding(a.rounding, "lq_mx_state_update")) return rc;
  LQ_CHECK_ARG(a.x && a.dt && a.A && a.B && a.C && a.out, "lq_mx_state_update: null operand");
  LQ_CHECK_ARG(valid_dtype(a.x_dtype) && valid_dtype(a.dt_dtype) && valid_dtype(a.A_dtype) && valid_dtype(a.B_dtype) &&
                   valid_dtype(a.C_dtype) && valid_dtype(a.out_dtype),
               "lq_mx_state_update: bad dtype");
  LQ_CHECK_ARG(!a.dt_bias || valid_dtype(a.dt_bias_dtype), "lq_mx_state_update: bad dt_bias dtype");
  LQ_CHECK_ARG(!a.D || valid_dtype(a.D_dtype), "lq_mx_state_update: bad D dtype");
  LQ_CHECK_ARG(!a.z || valid_dtype(a.z_dtype), "lq_mx_state_update: bad z dtype");
  LQ_CHECK_ARG(a.ngroups > 0 && a.state.heads % a.ngroups == 0, "lq_mx_state_update: heads=%d not divisible by ngroups=%d",
               a.state.heads, a.ngroups);
  MxUpdateDerived d;
  d.nblk = a.state.dstate / 16;
  if (d.nblk > 32) return fail(LQ_ERR_UNSUPPORTED, "lq_mx_state_update: dstate=%d > 512 is not implemented", a.state.dstate);
  if (a.state.dim > 4096) return fail(LQ_ERR_UNSUPPORTED, "lq_mx_state_update: dim=%d > 4096 is not implemented", a.state.dim);
  d.lpr_log2 = 0;
  while ((1 << d.lpr_log2) < d.nblk) ++d.lpr_log2;
  d.dt_uniform = (a.dt_stride[2] == 0 && (!a.dt_bias || a.dt_bias_stride[1] == 0)) ? 1 : 0;
  d.a_scalar = (a.A_stride[1] == 0 && a.A_stride[2] == 0) ? 1 : 0;
  d.keys = make_philox_keys(a.rounding.seed);
  {
    // Heads per CTA: as many heads of one B/C group as keeps the grid at >= 4 CTAs per SM (B and C
    // are then fetched, and dt / exp(A dt) evaluated, once for all of them), and shared memory small.
    const int per_group = a.state.heads / a.ngroups;
    const int64_t want_ctas = 4ll * sm_count();
    int hpc = per_group;
    while (hpc > 1 && (static_cast<int64_t>(a.state.batch) * (a.state.heads / hpc) < want_ctas || hpc * a.state.dim > 4096 ||
                       per_group % hpc != 0))
      --hpc;
    d.heads_per_cta = hpc;
  }
  if (a.h_out) LQ_CHECK_ARG(reinterpret_cast<uintptr_t>(a.h_out) % 16 == 0, "lq_mx_state_update: h_out must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
#define LQ_CALL(B_, L_) launch_update_mode<B_, L_>(a, d, st)
  LQ_DISPATCH_BITS_LAYOUT(a.state.format_bits, a.state.layout, LQ_CALL);
#undef LQ_CALL
  LQ_CHECK_CUDA(cudaGetLastError());
  return LQ_OK;
}

LQ_EXPORT int lq_mx_quantize(const lq_mx_state* state, const void* src, int32_t src_dtype, int64_t src_row_stride,
                              const lq_rounding* rounding, void* cuda_stream) {
  LQ_CHECK_ARG(state && src && rounding, "lq_mx_quantize: null argument");
  if (int rc = validate_state(*state, "lq_mx_quantize")) return rc;
  if (int rc = validate_rounding(*rounding, "lq_mx_quantize")) return rc;
  LQ_CHECK_ARG(valid_dtype(src_dtype), "lq_mx_quantize: bad dtype");
  LQ_CHECK_ARG(src_row_stride >= state->dstate, "lq_mx_quantize: src_row_stride=%lld < dstate", (long long)src_row_stride);
  const int64_t total = static_cast<int64_t>(state->batch) * state->heads * state->dim * (state->dstate / 16);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
#define LQ_CALL(B_, L_) launch_quantize_mode<B_, L_>(*state, src, src_dtype, src_row_stride, *rounding, total, st)
  LQ_DISPATCH_BITS_LAYOUT(state->format_bits, state->layout, LQ_CALL);
#undef LQ_CALL
  LQ_CHECK_CUDA(cudaGetLastError());
  return LQ_OK;
}

LQ_EXPORT int lq_counter_add(uint64_t* counter, uint64_t inc, void* cuda_stream) {
  LQ_CHECK_ARG(counter != nullptr && reinterpret_cast<uintptr_t>(counter) % 8 == 0, "lq_counter_add: counter must be an 8-byte aligned device pointer");
  counter_add_kernel<<<1, 1, 0, static_cast<cudaStream_t>(cuda_stream)>>>(reinterpret_cast<unsigned long long*>(counter), inc);
  LQ_CHECK_CUDA(cudaGetLastError());
  return LQ_OK;
}

LQ_EXPORT int lq_mx_dequantize(const lq_mx_state* state, float* dst, int64_t dst_row_stride, void* cuda_stream) {
  LQ_CHECK_ARG(state && dst, "lq_mx_dequantize: null argument");
  if (int rc = validate_state(*state, "lq_mx_dequantize")) return rc;
  LQ_CHECK_ARG(dst_row_stride >= state->dstate, "lq_mx_dequantize: dst_row_stride < dstate");
  const int64_t total = static_cast<int64_t>(state->batch) * state->heads * state->dim * (state->dstate / 16);
  const int block = 128;
  const int grid = static_cast<int>(std::min<int64_t>((total + block - 1) / block, 1 << 20));
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
#define LQ_CALL(B_, L_) mx_dequantize_kernel<B_, L_><<<grid, block, 0, st>>>(*state, dst, dst_row_stride, total)
  LQ_DISPATCH_BITS_LAYOUT(state->format_bits, state->layout, LQ_CALL);
#undef LQ_CALL
  LQ_CHECK_CUDA(cudaGetLastError());
  return LQ_OK;
}

LQ_EXPORT int lq_mx_convert_layout(const lq_mx_state* src, const lq_mx_state* dst, void* cuda_stream) {
  LQ_CHECK_ARG(src && dst, "lq_mx_convert_layout: null argument");
  if (int rc = validate_state(*src, "lq_mx_convert_layout(src)")) return rc;
  if (int rc = validate_state(*dst, "lq_mx_convert_layout(dst)")) return rc;
  LQ_CHECK_ARG(src->format_bits == dst->format_bits && src->batch == dst->batch && src->heads == dst->heads &&
                   src->dim == dst->dim && src->dstate == dst->dstate,
               "lq_mx_convert_layout: source and destination differ in shape or format");
  const int64_t total = static_cast<int64_t>(src->batch) * src->heads * src->dim * (src->dstate / 16);
  const int block = 128;
  const int grid = static_cast<int>(std::min<int64_t>((total + block - 1) / block, 1 << 20));
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const int bits = src->format_bits;
#define LQ_CONV(B_, S_, D_) mx_convert_kernel<B_, S_, D_><<<grid, block, 0, st>>>(*src, *dst, total)
  if (bits == 8) {
    if (src->layout == LQ_MX_LAYOUT_REFERENCE && dst->layout == LQ_MX_LAYOUT_PACKED) LQ_CONV(8, LQ_MX_LAYOUT_REFERENCE, LQ_MX_LAYOUT_PACKED);
    else if (src->layout == LQ_MX_LAYOUT_PACKED && dst->layout == LQ_MX_LAYOUT_REFERENCE) LQ_CONV(8, LQ_MX_LAYOUT_PACKED, LQ_MX_LAYOUT_REFERENCE);
    else if (src->layout == LQ_MX_LAYOUT_PACKED) LQ_CONV(8, LQ_MX_LAYOUT_PACKED, LQ_MX_LAYOUT_PACKED);
    else LQ_CONV(8, LQ_MX_LAYOUT_REFERENCE, LQ_MX_LAYOUT_REFERENCE);
  } else {
    if (src->layout == LQ_MX_LAYOUT_REFERENCE && dst->layout == LQ_MX_LAYOUT_PACKED) LQ_CONV(4, LQ_MX_LAYOUT_REFERENCE, LQ_MX_LAYOUT_PACKED);
    else if (src->layout == LQ_MX_LAYOUT_PACKED && dst->layout == LQ_MX_LAYOUT_REFERENCE) LQ_CONV(4, LQ_MX_LAYOUT_PACKED, LQ_MX_LAYOUT_REFERENCE);
    else if (src->layout == LQ_MX_LAYOUT_PACKED) LQ_CONV(4, LQ_MX_LAYOUT_PACKED, LQ_MX_LAYOUT_PACKED);
    else LQ_CONV(4, LQ_MX_LAYOUT_REFERENCE, LQ_MX_LAYOUT_REFERENCE);
  }
#undef LQ_CONV
  LQ_CHECK_CUDA(cudaGetLastError());
  return LQ_OK;
}
