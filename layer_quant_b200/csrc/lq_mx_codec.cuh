// Device-side MX8 / MX4 block codec: 16 values -> one biased exponent byte, 8 micro-exponent
// bits, 16 signed mantissas.  Bit-exact restatement of the reference's in-kernel requantiser
// (hybrid_quant/mamba_state_8b_kernel.py:168-203, :463-484, :511-534) and of its torch initial
// quantiser (:559-568), with IEEE fp32 division and a correctly rounded log2 as the canonical
// float semantics.  The exponent needs neither a division nor a logarithm here: it is a table
// look-up on the exponent field of the block maximum plus one mantissa compare (lq_exp_table.h).
//
// Instruction budget.  On B200 the integer / logic / compare / min-max / byte-permute pipe issues
// at half the rate of the FMA pipe, and at HBM speed an MX8 value may cost about 6 such
// instructions and 12 issue slots in total.  The code below therefore keeps work on the FMA pipe
// wherever the result is bit-identical: scale selection, micro-exponent bits and int -> byte
// conversion are done with exact float arithmetic and magic constants instead of selects, shifts
// and conversions; bytes are gathered with one byte-permute per value.
#pragma once

#include "lq_common.cuh"

#define LQ_EXP_TABLE_QUALIFIER static __device__ const
#include "lq_exp_table.h"

namespace lq {

template <int BITS>
__device__ __forceinline__ const unsigned int* mx_exp_cut_table() {
  return BITS == 8 ? LQ_MX8_EXP_CUT : LQ_MX4_EXP_CUT;
}

template <int BITS>
struct MxFormat {
  static constexpr float kMax = BITS == 8 ? 63.0f : 7.0f;
  static constexpr int kShift = BITS == 8 ? 6 : 3;  // floor(log2(2 * kMax))
};

// 2^(e - 127 + micro) for stored bytes e in [0, 255], micro in {0, 1} (reference: tl.exp2 at :132).
__device__ __forceinline__ float mx_decode_scale(uint32_t e, uint32_t micro) {
  const uint32_t s = e + micro;
  return __uint_as_float(s == 0 ? 0x00400000u : (s > 255u ? 255u : s) << 23);
}

// Rounding context of one 16-value block.
struct MxRoundCtx {
  uint64_t counter;      // PHILOX_REF: counter of value 0 of the block; PHILOX_LAYERED: index of the block; PHILOX_LAYERED4: of its first quad
  uint32_t wrap32;       // PHILOX_REF: counters are taken modulo 2^32 with a zero high word
  uint32_t step, layer;  // PHILOX_LAYERED
  const uint32_t* words; // SUPPLIED / SUPPLIED_FIXED: 16 words of this block
};

// 1.0f if a > b else 0.0f, as one FSET.
__device__ __forceinline__ float set_gt(float a, float b) {
  float r;
  asm("set.gt.f32.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// Byte 1 of four words -> one word (byte k from word k): three byte-permutes.
__device__ __forceinline__ uint32_t gather_byte1(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  const uint32_t ab = __byte_perm(a, b, 0x0051);  // [a.1, b.1, a.0, a.0]
  const uint32_t cd = __byte_perm(c, d, 0x0051);
  return __byte_perm(ab, cd, 0x5410);             // [ab.0, ab.1, cd.0, cd.1]
}

constexpr float kByteMagic = 49152.0f;  // 1.5 * 2^15: ulp 2^-8, mantissa bits 8..15 = integer part mod 256

// Encodes h[0..15].  codes[w] holds values 4w..4w+3 as int8 lanes; micro_bits bit i = pair i.
//
// Two rounding rules:
//  * reference rule (HALF_UP, HALF_EVEN, PHILOX_REF, SUPPLIED, PHILOX_LAYERED4): a = min(|h| / scale, M), level from
//    floor(a + .5) / rint(a) / floor(a) + (u < a - floor(a)), sign restored afterwards -- the
//    reference's expressions, evaluated with the same fp32 operations;
//  * fixed-point rule (PHILOX_LAYERED, SUPPLIED_FIXED): t = fl32(h / scale + 49152 + r8 / 256) in one
//    FMA, q = floor(t) - 49152, i.e. stochastic rounding with an 8-bit uniform draw r8; q (two's
//    complement) is byte 1 of t's bit pattern.  No clamp is needed: |h| / scale never exceeds
//    M + 2^-9 (the few-ulp overshoot of the rounded log2 is orders of magnitude smaller).
template <int BITS, int MODE>
__device__ __forceinline__ void mx_encode_block(const float (&h)[16], const unsigned int* __restrict__ cut_table,
                                                const MxRoundCtx& ctx, const PhiloxKeys& keys, uint32_t (&codes)[4],
                                                uint32_t& exp_byte, uint32_t& micro_bits) {
  constexpr float M = MxFormat<BITS>::kMax;
  constexpr bool kFixed = (MODE == LQ_ROUND_PHILOX_LAYERED || MODE == LQ_ROUND_SUPPLIED_FIXED);
  float pa[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) pa[j] = fmaxf(fabsf(h[2 * j]), fabsf(h[2 * j + 1]));
  const float amax = fmaxf(fmaxf(fmaxf(pa[0], pa[1]), fmaxf(pa[2], pa[3])), fmaxf(fmaxf(pa[4], pa[5]), fmaxf(pa[6], pa[7])));
  // biased = clamp(ceil(log2(max(amax / 2M, 1e-30))) + 127, 1, 254): always in [28, 252]
  const uint32_t abits = __float_as_uint(amax);
  const uint32_t field = abits >> 23;
  int biased = static_cast<int>(field) - MxFormat<BITS>::kShift + ((abits & 0x7FFFFFu) > __ldg(cut_table + field) ? 1 : 0);
  biased = biased < 28 ? 28 : biased;
  exp_byte = static_cast<uint32_t>(biased);
  // amax == 0 makes the reference use base 1.0; every mantissa is 0 with either base.
  const float thresh = M * __uint_as_float(static_cast<uint32_t>(biased) << 23);       // M * base, exact
  const float inv0 = __uint_as_float(static_cast<uint32_t>(254 - biased) << 23);        // 1 / base
  const float neg_half_inv0 = -0.5f * inv0;

  uint32_t rnd[16];  // SUPPLIED*: one word per value
  if (MODE == LQ_ROUND_SUPPLIED || MODE == LQ_ROUND_SUPPLIED_FIXED) {
    const uint4* w4 = reinterpret_cast<const uint4*>(ctx.words);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = __ldg(w4 + i);
      rnd[4 * i] = v.x; rnd[4 * i + 1] = v.y; rnd[4 * i + 2] = v.z; rnd[4 * i + 3] = v.w;
    }
  }
  if (MODE == LQ_ROUND_PHILOX_LAYERED4) {  // one Philox block per four values, value i of a quad takes word i
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
      const uint64_t c = ctx.counter + qd;
      const Philox4 r = philox4x32_10(static_cast<uint32_t>(c), static_cast<uint32_t>(c >> 32), ctx.step, ctx.layer, keys);
      rnd[4 * qd] = r.w0; rnd[4 * qd + 1] = r.w1; rnd[4 * qd + 2] = r.w2; rnd[4 * qd + 3] = r.w3;
    }
  }
  uint32_t pw[4] = {0u, 0u, 0u, 0u};  // PHILOX_LAYERED: 16 random bytes, value i = byte i & 3 of word i >> 2
  if (MODE == LQ_ROUND_PHILOX_LAYERED) {
    const Philox4 r = philox4x32_10(static_cast<uint32_t>(ctx.counter), static_cast<uint32_t>(ctx.counter >> 32), ctx.step,
                                    ctx.layer, keys);
    pw[0] = r.w0; pw[1] = r.w1; pw[2] = r.w2; pw[3] = r.w3;
  }

  float macc = 0.0f;  // sum of 2^j over pairs with the micro-exponent set (exact)
  uint32_t tb[16];    // bit patterns whose byte 1 is the code
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float micf = set_gt(pa[j], thresh);
    const float inv = fmaf(micf, neg_half_inv0, inv0);  // 1 / (base * 2^micro), exact
    macc = fmaf(micf, static_cast<float>(1 << j), macc);
    if (kFixed) {  // the pair shares 1 / scale: one packed fp32x2 FMA for both values
      float cf[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int i = 2 * j + k;
        const uint32_t c = (MODE == LQ_ROUND_SUPPLIED_FIXED) ? (0x47400000u | (rnd[i] & 0xFFu))
                                                             : __byte_perm(pw[i >> 2], 0x47400000u, 0x7650 + (i & 3));
        cf[k] = __uint_as_float(c);
      }
      const float2 t2 = __ffma2_rn(make_float2(h[2 * j], h[2 * j + 1]), make_float2(inv, inv), make_float2(cf[0], cf[1]));
      tb[2 * j] = __float_as_uint(t2.x);
      tb[2 * j + 1] = __float_as_uint(t2.y);
      continue;
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = 2 * j + k;
      float t;
      {
        const float a = fminf(fabsf(h[i]) * inv, M);
        float lvl;
        if (MODE == LQ_ROUND_HALF_UP) {
          lvl = floorf(a + 0.5f);
        } else if (MODE == LQ_ROUND_HALF_EVEN) {
          lvl = rintf(a);
        } else {
          uint32_t w;
          if (MODE == LQ_ROUND_SUPPLIED || MODE == LQ_ROUND_PHILOX_LAYERED4) {
            w = rnd[i];
          } else {  // the reference's stream: one Philox block per value, word 0
            const uint64_t c = ctx.counter + i;
            w = philox4x32_10(static_cast<uint32_t>(c), ctx.wrap32 ? 0u : static_cast<uint32_t>(c >> 32), 0u, 0u, keys).w0;
          }
          const float fl = floorf(a);
          lvl = fl + set_gt(a - fl, word_to_uniform(w));  // (u < a - fl) ? 1 : 0
        }
        lvl = fminf(lvl, M);
        t = copysignf(lvl, h[i]) + kByteMagic;  // exact; byte 1 = two's complement of the signed level
      }
      tb[i] = __float_as_uint(t);
    }
  }
#pragma unroll
  for (int w = 0; w < 4; ++w) codes[w] = gather_byte1(tb[4 * w], tb[4 * w + 1], tb[4 * w + 2], tb[4 * w + 3]);
  micro_bits = __float_as_uint(macc + 8388608.0f) & 0xFFu;
}

// h' = h * dA + (B * dt) * x on 16 values and the block's share of <h', C>, with packed fp32x2 instructions
// (sm_100: two IEEE fp32 results per instruction, same rounding per component as the scalar forms).
// Association as in the reference kernel (mamba_state_8b_kernel.py:158, dB = B * dt, then state * dA + dB * x):
// dB rounded, t = dB * x rounded, then fma(h, dA, t), which is what a compiler that contracts the reference's
// expression produces; the read-out keeps four partial sums over i mod 4, added as (y0 + y1) + (y2 + y3).
__device__ __forceinline__ float mx_update_readout16(float (&hv)[16], const float (&Bv)[16], const float (&Cv)[16], float dA,
                                                     float dt, float x) {
  const float2 dA2 = make_float2(dA, dA), dt2 = make_float2(dt, dt), x2 = make_float2(x, x);
  float2 ya = make_float2(0.0f, 0.0f), yb = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    const float2 t0 = __fmul2_rn(__fmul2_rn(make_float2(Bv[i], Bv[i + 1]), dt2), x2);
    const float2 t1 = __fmul2_rn(__fmul2_rn(make_float2(Bv[i + 2], Bv[i + 3]), dt2), x2);
    const float2 h0 = __ffma2_rn(make_float2(hv[i], hv[i + 1]), dA2, t0);
    const float2 h1 = __ffma2_rn(make_float2(hv[i + 2], hv[i + 3]), dA2, t1);
    hv[i] = h0.x; hv[i + 1] = h0.y; hv[i + 2] = h1.x; hv[i + 3] = h1.y;
    ya = __ffma2_rn(h0, make_float2(Cv[i], Cv[i + 1]), ya);
    yb = __ffma2_rn(h1, make_float2(Cv[i + 2], Cv[i + 3]), yb);
  }
  return (ya.x + ya.y) + (yb.x + yb.y);
}

// int8 lanes of `codes` times 2^(e - 127 + micro of the pair) -> fp32 (reference :132).
// Fast path (stored exponent in [1, 229], everything the codec itself writes is in [28, 252] and
// states of realistic magnitude stay far below 229): byte -> float by one byte-permute into the
// mantissa of 2^15 (value 32768 + 128 + q), then ONE exact FMA per value: (32896 + q) * s - 32896 * s.
// The per-pair scale is built on the FMA pipe from the micro bit: bits(s) = e << 23 + micro << 23.
__device__ __forceinline__ void mx_decode_block(const uint32_t (&codes)[4], uint32_t e, uint32_t micro_bits, float (&h)[16]) {
  if (__all_sync(__activemask(), e - 1u <= 228u)) {  // one uniform branch per warp; the exact path below takes every e
    const uint32_t ebits = e << 23;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = __uint_as_float((micro_bits & (1u << j)) * (1u << (23 - j)) + ebits);
      const float cs = -32896.0f * s;
      float f[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int i = 2 * j + k;
        const uint32_t biased = codes[i >> 2] ^ 0x80808080u;  // q + 128 as unsigned bytes
        f[k] = __uint_as_float(__byte_perm(biased, 0x47000000u, 0x7604 | ((i & 3) << 4)));  // 32768 + 128 + q
      }
      // the pair shares its scale: one packed fp32x2 FMA (sm_100) instead of two scalar ones
      const float2 r = __ffma2_rn(make_float2(f[0], f[1]), make_float2(s, s), make_float2(cs, cs));
      h[2 * j] = r.x;
      h[2 * j + 1] = r.y;
    }
  } else {  // exponents no quantiser emits: plain, overflow-safe form
    const float s0 = mx_decode_scale(e, 0), s1 = mx_decode_scale(e, 1);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int q = static_cast<int>(static_cast<int8_t>((codes[i >> 2] >> (8 * (i & 3))) & 0xFFu));
      h[i] = static_cast<float>(q) * (((micro_bits >> (i >> 1)) & 1u) ? s1 : s0);
    }
  }
}

// Storage helpers -----------------------------------------------------------------------------
// Expands 16 two's-complement nibbles (value 2j low, 2j+1 high) to int8 lanes.
__device__ __forceinline__ void mx4_nibbles_to_bytes(uint32_t lo, uint32_t hi, uint32_t (&codes)[4]) {
  const uint32_t src[2] = {lo, hi};
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    // even values sit in the low nibbles of the 4 bytes, odd values in the high nibbles
    const uint32_t ev = src[s] & 0x0F0F0F0Fu, od = (src[s] >> 4) & 0x0F0F0F0Fu;
    // interleave: result word 0 = values 0..3 = [ev.0, od.0, ev.1, od.1], word 1 = [ev.2, od.2, ev.3, od.3]
    uint32_t w0 = __byte_perm(ev, od, 0x5140), w1 = __byte_perm(ev, od, 0x7362);
    // sign-extend each byte from bit 3
    w0 |= (w0 & 0x08080808u) * 0x1Eu;
    w1 |= (w1 & 0x08080808u) * 0x1Eu;
    codes[2 * s] = w0;
    codes[2 * s + 1] = w1;
  }
}

__device__ __forceinline__ void mx4_bytes_to_nibbles(const uint32_t (&codes)[4], uint32_t& lo, uint32_t& hi) {
  uint32_t out[2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const uint32_t w0 = codes[2 * s] & 0x0F0F0F0Fu, w1 = codes[2 * s + 1] & 0x0F0F0F0Fu;
    const uint32_t ev = __byte_perm(w0, w1, 0x6420);  // values 0, 2, 4, 6
    const uint32_t od = __byte_perm(w0, w1, 0x7531);  // values 1, 3, 5, 7
    out[s] = ev | (od << 4);
  }
  lo = out[0];
  hi = out[1];
}

}  // namespace lq
