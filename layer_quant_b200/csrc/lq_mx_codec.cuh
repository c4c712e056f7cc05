// Device-side MX8 / MX4 block codec: 16 values -> one biased exponent byte, 8 micro-exponent
// bits, 16 signed mantissas.  Bit-exact restatement of the reference's in-kernel requantiser
// (hybrid_quant/mamba_state_8b_kernel.py:168-203, :463-484, :511-534) and of its torch initial
// quantiser (:559-568), with IEEE fp32 division and a correctly rounded log2 as the canonical
// float semantics.  The exponent needs neither a division nor a logarithm here: it is a table
// look-up on the exponent field of the block maximum plus one mantissa compare (lq_exp_table.h).
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
  uint32_t k0, k1;      // Philox key
  uint64_t counter;     // PHILOX_REF: counter of value 0 of the block; PHILOX_LAYERED: index of its first 8-group
  uint32_t wrap32;      // PHILOX_REF: counters are taken modulo 2^32 with a zero high word
  uint32_t step, layer; // PHILOX_LAYERED
  const uint32_t* words; // SUPPLIED*: 16 words of this block
};

// Encodes h[0..15].  codes[w] holds values 4w..4w+3 as int8 lanes; micro_bits bit i = pair i.
template <int BITS, int MODE>
__device__ __forceinline__ void mx_encode_block(const float (&h)[16], const unsigned int* __restrict__ cut_table,
                                                const MxRoundCtx& ctx, uint32_t (&codes)[4], uint32_t& exp_byte,
                                                uint32_t& micro_bits) {
  constexpr float M = MxFormat<BITS>::kMax;
  float pair_amax[8];
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    pair_amax[j] = fmaxf(fabsf(h[2 * j]), fabsf(h[2 * j + 1]));
    amax = fmaxf(amax, pair_amax[j]);
  }
  // biased = clamp(ceil(log2(max(amax / 2M, 1e-30))) + 127, 1, 254): always in [28, 252]
  const uint32_t abits = __float_as_uint(amax);
  const uint32_t field = abits >> 23;
  int biased = static_cast<int>(field) - MxFormat<BITS>::kShift + ((abits & 0x7FFFFFu) > __ldg(cut_table + field) ? 1 : 0);
  biased = biased < 28 ? 28 : biased;
  exp_byte = static_cast<uint32_t>(biased);
  // amax == 0 makes the reference use base 1.0; every mantissa is 0 with either base.
  const float base = __uint_as_float(static_cast<uint32_t>(biased) << 23);
  const float thresh = M * base;  // exact
  const float inv0 = __uint_as_float(static_cast<uint32_t>(254 - biased) << 23);  // 1 / base
  const float inv1 = __uint_as_float(static_cast<uint32_t>(253 - biased) << 23);  // 1 / (2 base)

  uint32_t supplied[16];
  if (MODE == LQ_ROUND_SUPPLIED || MODE == LQ_ROUND_SUPPLIED16) {
    const uint4* w4 = reinterpret_cast<const uint4*>(ctx.words);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = __ldg(w4 + i);
      supplied[4 * i] = v.x; supplied[4 * i + 1] = v.y; supplied[4 * i + 2] = v.z; supplied[4 * i + 3] = v.w;
    }
  }
  uint32_t r16[16];
  if (MODE == LQ_ROUND_PHILOX_LAYERED) {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const uint64_t idx = ctx.counter + g;
      const Philox4 r = philox4x32_10(static_cast<uint32_t>(idx), static_cast<uint32_t>(idx >> 32), ctx.step, ctx.layer,
                                      ctx.k0, ctx.k1);
      const uint32_t w[4] = {r.w0, r.w1, r.w2, r.w3};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        r16[8 * g + 2 * j] = w[j] & 0xFFFFu;
        r16[8 * g + 2 * j + 1] = w[j] >> 16;
      }
    }
  }

  micro_bits = 0;
  codes[0] = codes[1] = codes[2] = codes[3] = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const bool mic = pair_amax[i >> 1] > thresh;
    if ((i & 1) == 0) micro_bits |= (mic ? 1u : 0u) << (i >> 1);
    const float inv = mic ? inv1 : inv0;
    int q;
    if (MODE == LQ_ROUND_PHILOX_LAYERED || MODE == LQ_ROUND_SUPPLIED16) {
      // 16.16 fixed point of v/scale + 64 sits in the mantissa of a float in [128, 256)
      float t = fmaf(h[i], inv, 192.0f);
      t = fminf(fmaxf(t, 192.0f - M), 192.0f + M);
      const uint32_t r = (MODE == LQ_ROUND_SUPPLIED16) ? (supplied[i] & 0xFFFFu) : r16[i];
      q = static_cast<int>(((__float_as_uint(t) + r) >> 16) & 0xFFu) - 64;
    } else {
      const float a = fminf(fabsf(h[i]) * inv, M);
      float lvl;
      if (MODE == LQ_ROUND_HALF_UP) {
        lvl = floorf(a + 0.5f);
      } else if (MODE == LQ_ROUND_HALF_EVEN) {
        lvl = rintf(a);
      } else {
        uint32_t w;
        if (MODE == LQ_ROUND_SUPPLIED) {
          w = supplied[i];
        } else {  // the reference's stream: one Philox block per value, word 0
          const uint64_t c = ctx.counter + i;
          w = philox4x32_10(static_cast<uint32_t>(c), ctx.wrap32 ? 0u : static_cast<uint32_t>(c >> 32), 0u, 0u, ctx.k0,
                            ctx.k1).w0;
        }
        const float fl = floorf(a);
        lvl = fl + ((word_to_uniform(w) < a - fl) ? 1.0f : 0.0f);
      }
      lvl = fminf(lvl, M);
      q = static_cast<int>(lvl);
      q = h[i] < 0.0f ? -q : q;
    }
    codes[i >> 2] |= (static_cast<uint32_t>(q) & 0xFFu) << (8 * (i & 3));
  }
}

// int8 lanes of `codes` times `scale` (per pair) -> fp32, using the 2^23 magic-number conversion.
__device__ __forceinline__ void mx_decode_block(const uint32_t (&codes)[4], uint32_t e, uint32_t micro_bits, float (&h)[16]) {
  const float s0 = mx_decode_scale(e, 0), s1 = mx_decode_scale(e, 1);
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const uint32_t biased = codes[w] ^ 0x80808080u;  // q + 128 as unsigned bytes
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = 4 * w + k;
      const float f = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7650 + k)) - 8388736.0f;  // exact q
      h[i] = f * (((micro_bits >> (i >> 1)) & 1u) ? s1 : s0);
    }
  }
}

// Storage helpers -----------------------------------------------------------------------------
// Expands 16 two's-complement nibbles (value 2j low, 2j+1 high) to int8 lanes.
__device__ __forceinline__ void mx4_nibbles_to_bytes(uint32_t lo, uint32_t hi, uint32_t (&codes)[4]) {
  const uint32_t src[2] = {lo, hi};
#pragma unroll
  for (int s = 0; s < 2; ++s) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const uint32_t x = (src[s] >> (16 * half)) & 0xFFFFu;  // 4 nibbles
      // spread nibble k to byte k, then sign-extend each byte from bit 3
      uint32_t b = (x & 0xFu) | ((x & 0xF0u) << 4) | ((x & 0xF00u) << 8) | ((x & 0xF000u) << 12);
      b |= ((b & 0x08080808u) * 0x1Eu) & 0xF0F0F0F0u;
      codes[2 * s + half] = b;
    }
  }
}

__device__ __forceinline__ void mx4_bytes_to_nibbles(const uint32_t (&codes)[4], uint32_t& lo, uint32_t& hi) {
  uint32_t out[2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    uint32_t acc = 0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const uint32_t b = codes[2 * s + half] & 0x0F0F0F0Fu;
      const uint32_t x = (b & 0xFu) | ((b >> 4) & 0xF0u) | ((b >> 8) & 0xF00u) | ((b >> 12) & 0xF000u);
      acc |= x << (16 * half);
    }
    out[s] = acc;
  }
  lo = out[0];
  hi = out[1];
}

}  // namespace lq
