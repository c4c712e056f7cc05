// Packed signed-INT4 KV cache: append (quantise + pack) and q_len = 1 GQA decode attention with a
// split over the context (flash-decoding).  sm_100a.
//
// Decode kernel: one CTA per (split, kv head, batch).  A producer warp streams 64-token tiles of
// the packed K / V codes and their fp32 group scales from HBM into a 4-stage shared-memory ring
// with bulk asynchronous copies (cp.async.bulk, completion on an mbarrier; rows of one (batch,
// kv head) are contiguous, so a tile is four plain 1-D copies).  Eight consumer warps read the
// ring: 8 lanes share one token, each lane owning 16 of the 128 head dimensions for ALL query
// heads of the GQA group, so a K/V byte is fetched once per group instead of once per query head.
// Nibbles become floats with one byte-permute each (0x4300'0000 | n+8 << 16 = 136 + n); the
// constant 136 is removed algebraically (a per-lane -136 * sum(q) start value on the K side, a
// -136 * sum(p) correction on the V side).  Every 8-lane group runs its own online softmax
// (running max, sum and output), rescaling only when its max grows; groups, warps and finally
// splits are merged with the usual (max, sum, output) rule.  The CTA that arrives last at a
// per-(batch, kv head) ticket counter merges the splits, so no second launch and no waiting.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "lq_common.cuh"

namespace lq {

__device__ int g_int4_device_status = 0;

int int4_read_device_status(int32_t* status) {
  int v = 0;
  LQ_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_int4_device_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    LQ_CHECK_CUDA(cudaMemcpyToSymbol(g_int4_device_status, &zero, sizeof(int)));
  }
  *status = v;
  return LQ_OK;
}

constexpr int kHeadDim = 128;
constexpr int kTile = 64;           // tokens per ring stage
constexpr int kStages = 4;
constexpr int kConsumerWarps = 8;
constexpr int kDecodeThreads = kConsumerWarps * 32;  // thread 0 doubles as the copy producer
constexpr int kTokPerWarp = kTile / kConsumerWarps;  // 8 tokens = 2 passes of 4
constexpr uint32_t kWaitLimit = 1u << 22;            // polls before a wait gives up

// ---- mbarrier / bulk-copy wrappers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after kWaitLimit polls, records it in the device status word and in the
// CTA's abort flag so that every warp leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  atomicOr(&g_int4_device_status, 1);
  return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ---- INT4 row codec ---------------------------------------------------------------------------------
// scale = max(absmax / 7, 1e-8); code = clamp(rni(x / scale), -8, 7)   (int4_8b_attention.py:75-85)
__device__ __forceinline__ float int4_scale(float absmax) { return fmaxf(__fdiv_rn(absmax, 7.0f), 1.0e-8f); }
__device__ __forceinline__ uint32_t int4_code(float x, float scale) {
  int q = __float2int_rn(__fdiv_rn(x, scale));
  q = max(-8, min(7, q));
  return static_cast<uint32_t>(q) & 15u;
}

struct AppendParams {
  lq_int4_cache c;
  const void* k; const void* v;
  int64_t ks[4]; int64_t vs[4];
  int dtype; int q_len;
  const int64_t* positions;
};

// One thread per 8 consecutive values (one packed 32-bit word); the gs/8 threads of a group are
// neighbours in a warp and share the absmax by shuffles.  Requires gs/8 a power of two <= 32.
__global__ void int4_append_kernel(const AppendParams p, int64_t total_chunks, int lanes_per_group_log2) {
  const int D = p.c.head_dim, gs = p.c.group_size;
  const int chunks_per_row = D / 8;
  const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const bool live = t < total_chunks;
  const int64_t tt = live ? t : total_chunks - 1;  // clamp so that every lane takes part in the shuffles
  int64_t row = tt / chunks_per_row;
  const int chunk = static_cast<int>(tt - row * chunks_per_row);
  const int which = static_cast<int>(row & 1);  // 0 = K, 1 = V
  row >>= 1;
  const int tok = static_cast<int>(row % p.q_len);
  const int64_t bh = row / p.q_len;
  const int h = static_cast<int>(bh % p.c.kv_heads);
  const int64_t b = bh / p.c.kv_heads;
  const void* src = which ? p.v : p.k;
  const int64_t* ss = which ? p.vs : p.ks;
  const int64_t base = b * ss[0] + h * ss[1] + tok * ss[2];
  float x[8];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    x[i] = load_as_float(src, base + (chunk * 8 + i) * ss[3], p.dtype);
    amax = fmaxf(amax, fabsf(x[i]));
  }
  for (int o = (1 << lanes_per_group_log2) >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  const float scale = int4_scale(amax);
  uint32_t word = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) word |= int4_code(x[i], scale) << (4 * i);
  if (!live) return;
  const int64_t pos = p.positions[tok];
  uint8_t* packed = which ? p.c.v_packed : p.c.k_packed;
  const int64_t* ps = which ? p.c.vp_stride : p.c.kp_stride;
  uint8_t* dst = packed + b * ps[0] + h * ps[1] + pos * ps[2];
  if (ps[3] == 1 && (reinterpret_cast<uintptr_t>(dst + chunk * 4) & 3) == 0) {
    *reinterpret_cast<uint32_t*>(dst + chunk * 4) = word;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[(chunk * 4 + i) * ps[3]] = static_cast<uint8_t>(word >> (8 * i));
  }
  if (((chunk * 8) % gs) == 0) {
    float* sc = which ? p.c.v_scale : p.c.k_scale;
    const int64_t* sst = which ? p.c.vs_stride : p.c.ks_stride;
    sc[b * sst[0] + h * sst[1] + pos * sst[2] + (chunk * 8 / gs) * sst[3]] = scale;
  }
}

// Any even group size: one thread per group.
__global__ void int4_append_generic_kernel(const AppendParams p, int64_t total_groups) {
  const int D = p.c.head_dim, gs = p.c.group_size;
  const int groups = D / gs;
  const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (t >= total_groups) return;
  int64_t row = t / groups;
  const int g = static_cast<int>(t - row * groups);
  const int which = static_cast<int>(row & 1);
  row >>= 1;
  const int tok = static_cast<int>(row % p.q_len);
  const int64_t bh = row / p.q_len;
  const int h = static_cast<int>(bh % p.c.kv_heads);
  const int64_t b = bh / p.c.kv_heads;
  const void* src = which ? p.v : p.k;
  const int64_t* ss = which ? p.vs : p.ks;
  const int64_t base = b * ss[0] + h * ss[1] + tok * ss[2];
  float amax = 0.0f;
  for (int i = 0; i < gs; ++i) amax = fmaxf(amax, fabsf(load_as_float(src, base + (g * gs + i) * ss[3], p.dtype)));
  const float scale = int4_scale(amax);
  const int64_t pos = p.positions[tok];
  uint8_t* packed = which ? p.c.v_packed : p.c.k_packed;
  const int64_t* ps = which ? p.c.vp_stride : p.c.kp_stride;
  uint8_t* dst = packed + b * ps[0] + h * ps[1] + pos * ps[2];
  for (int i = 0; i < gs; i += 2) {
    const uint32_t lo = int4_code(load_as_float(src, base + (g * gs + i) * ss[3], p.dtype), scale);
    const uint32_t hi = int4_code(load_as_float(src, base + (g * gs + i + 1) * ss[3], p.dtype), scale);
    dst[((g * gs + i) / 2) * ps[3]] = static_cast<uint8_t>(lo | (hi << 4));
  }
  float* sc = which ? p.c.v_scale : p.c.k_scale;
  const int64_t* sst = which ? p.c.vs_stride : p.c.ks_stride;
  sc[b * sst[0] + h * sst[1] + pos * sst[2] + g * sst[3]] = scale;
}

// ---- decode attention -------------------------------------------------------------------------------
struct DecodeParams {
  lq_int4_decode_args a;
  int32_t splits;          // >= 1
  int32_t tiles_per_split;
  int32_t ctx_len;         // tokens read from the cache ring: seq_len, minus the fused new token
  int32_t* counters;       // [B * Hkv] tickets (workspace)
  float* part_ml;          // [B * Hq * splits * 2]
  float* part_acc;         // [B * Hq * splits * 128]
  // causal prefill over the quantised cache (tensor-pipe kernel with QB > 0 only)
  int32_t q_len = 1;       // query positions per sequence
  int32_t nqb = 1;         // query blocks per sequence = ceil(q_len / QB)
  int32_t first_len = 0;   // tokens the first query position sees (its own included)
  int64_t q_stride_t = 0, out_stride_t = 0;
};

// The lengths a launch works with.  Without a device counter they are the host's; with one the
// sequence length is read when the kernel runs (a recorded launch follows a growing context) and the
// tiles are dealt evenly to the launch's fixed number of splits.  A counter outside [1, capacity] is
// clamped and recorded in the device status word (bit 1).
struct RunLengths {
  int seq_len, ctx_len, tiles_per_split;
};
__device__ __forceinline__ RunLengths run_lengths(const DecodeParams& p) {
  RunLengths r{p.a.seq_len, p.ctx_len, p.tiles_per_split};
  if (p.a.seq_len_counter != nullptr) {
    const unsigned long long v = *p.a.seq_len_counter;
    const unsigned long long cap = static_cast<unsigned long long>(p.a.cache.capacity);
    if (v < 1ull || v > cap) atomicOr(&g_int4_device_status, 2);
    r.seq_len = static_cast<int>(v < 1ull ? 1ull : (v > cap ? cap : v));
    r.ctx_len = r.seq_len - (p.a.k_new != nullptr ? 1 : 0);
    const int ntiles = max(1, (r.ctx_len + kTile - 1) / kTile);
    r.tiles_per_split = (ntiles + p.splits - 1) / p.splits;
  }
  return r;
}

template <int GS>
struct StageLayout {
  static constexpr int kGroups = kHeadDim / GS;
  static constexpr int kCodeBytes = kTile * (kHeadDim / 2);    // 4096
  static constexpr int kScaleBytes = kTile * kGroups * 4;
  static constexpr int kKc = 0;
  static constexpr int kVc = kCodeBytes;
  static constexpr int kKs = 2 * kCodeBytes;
  static constexpr int kVs = 2 * kCodeBytes + kScaleBytes;
  static constexpr int kBytes = 2 * kCodeBytes + 2 * kScaleBytes;
  // the row appended in this step: K codes, V codes, K scales, V scales
  static constexpr int kNewRowBytes = 2 * (kHeadDim / 2) + 2 * 16 * 4;
};

// Running maxima start at kNegBig instead of -inf: exp2(kNegBig - m) is 0 for any finite m, and no
// inf - inf can appear.  A stream that saw no unmasked token keeps (kNegBig, 0, 0).
constexpr float kNegBig = -1.0e30f;
// The running maximum is only raised when a score exceeds it by more than this (log2 units), so
// probabilities stay below 2^8 and the output rescale is rare and taken by the whole warp at once.
constexpr float kRescaleSlack = 8.0f;

// 16 nibbles (two 32-bit words) -> 16 floats 136 + n
__device__ __forceinline__ void unpack16(uint2 c, float (&f)[16]) {
  const uint32_t w[2] = {c.x ^ 0x88888888u, c.y ^ 0x88888888u};
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const uint32_t lo = w[j] & 0x0F0F0F0Fu, hi = (w[j] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      f[8 * j + 2 * k] = __uint_as_float(__byte_perm(lo, 0x43000000u, 0x7044 | (k << 8)));
      f[8 * j + 2 * k + 1] = __uint_as_float(__byte_perm(hi, 0x43000000u, 0x7044 | (k << 8)));
    }
  }
}

template <int R, int GS, bool HAS_MASK>
__global__ void __launch_bounds__(kDecodeThreads, 1) int4_decode_kernel(const DecodeParams p) {
  using L = StageLayout<GS>;
  constexpr int G = L::kGroups;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ int s_abort;
  __shared__ int s_is_last;
  __shared__ float s_m[kConsumerWarps][R], s_l[kConsumerWarps][R];

  const lq_int4_decode_args& a = p.a;
  const lq_int4_cache& c = a.cache;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane & 7, tg = lane >> 3;  // 16-dim slice, token slot inside the warp
  const bool fused_new = a.k_new != nullptr;
  uint8_t* newrow = smem + kStages * L::kBytes;

  const RunLengths rl = run_lengths(p);
  const int ntiles = (rl.ctx_len + kTile - 1) / kTile;
  const int tile_begin = split * rl.tiles_per_split;
  const int tile_end = min(ntiles, tile_begin + rl.tiles_per_split);
  const int my_tiles = max(0, tile_end - tile_begin);
  const bool do_new = fused_new && split == p.splits - 1;

  if (threadIdx.x == 0) {
    s_abort = 0;
    s_is_last = 0;
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], kConsumerWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }

  // Fused append: warp 0 quantises the new K row, warp 1 the new V row (4 values per lane), write
  // them to the cache (row seq_len - 1) and keep a copy in shared memory for this step.
  if (do_new && warp < 2) {
    const void* src = warp == 0 ? a.k_new : a.v_new;
    const int64_t* ss = warp == 0 ? a.k_new_stride : a.v_new_stride;
    float x[4];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[i] = load_as_float(src, b * ss[0] + kvh * ss[1] + (lane * 4 + i) * ss[2], a.dtype);
      amax = fmaxf(amax, fabsf(x[i]));
    }
#pragma unroll
    for (int o = GS / 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    const float scale = int4_scale(amax);
    uint32_t half = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) half |= int4_code(x[i], scale) << (4 * i);
    const int pos = rl.seq_len - 1;
    uint8_t* gcodes = (warp == 0 ? c.k_packed : c.v_packed) +
                      (warp == 0 ? b * c.kp_stride[0] + kvh * c.kp_stride[1] + pos * c.kp_stride[2]
                                 : b * c.vp_stride[0] + kvh * c.vp_stride[1] + pos * c.vp_stride[2]);
    reinterpret_cast<uint16_t*>(gcodes)[lane] = static_cast<uint16_t>(half);
    reinterpret_cast<uint16_t*>(newrow + warp * (kHeadDim / 2))[lane] = static_cast<uint16_t>(half);
    if ((lane * 4) % GS == 0) {
      float* gs_ = (warp == 0 ? c.k_scale : c.v_scale) +
                   (warp == 0 ? b * c.ks_stride[0] + kvh * c.ks_stride[1] + pos * c.ks_stride[2]
                              : b * c.vs_stride[0] + kvh * c.vs_stride[1] + pos * c.vs_stride[2]);
      gs_[lane * 4 / GS] = scale;
      reinterpret_cast<float*>(newrow + kHeadDim + warp * 64)[lane * 4 / GS] = scale;
    }
  }
  __syncthreads();

  // per-lane state: the GQA group's queries (pre-scaled by log2(e)/sqrt(D)), running softmax
  float qf[R][16], qcorr[R];
  float m_run[R], l_run[R], psum[R];
  float acc[R][16];
  const float scale_sm = 1.4426950408889634f / sqrtf(static_cast<float>(kHeadDim));
  {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float s = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        qf[r][i] = load_as_float(a.q, b * a.q_stride[0] + (kvh * R + r) * a.q_stride[1] + (sub * 16 + i) * a.q_stride[2],
                                 a.dtype) * scale_sm;
        s += qf[r][i];
        acc[r][i] = 0.0f;
      }
      qcorr[r] = -136.0f * s;
      m_run[r] = kNegBig;
      l_run[r] = 0.0f;
      psum[r] = 0.0f;
    }
  }

  // One token for this lane's 8-lane group: scores for the R heads, online softmax, P.V.
  auto process_token = [&](bool valid, uint2 kc, uint2 vc, float ksc, float vsc, float bias) {
    float f[16];
    unpack16(kc, f);
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float s0 = qcorr[r], s1 = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        s0 = fmaf(qf[r][i], f[i], s0);
        s1 = fmaf(qf[r][i + 1], f[i + 1], s1);
      }
      s[r] = (s0 + s1) * ksc;
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
#pragma unroll
      for (int r = 0; r < R; ++r) s[r] += __shfl_xor_sync(0xFFFFFFFFu, s[r], o);
    }
    if (!valid) return;
    unpack16(vc, f);
    bool grow = false;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (HAS_MASK) s[r] += bias;
      grow |= s[r] > m_run[r] + kRescaleSlack;
    }
    if (grow) {  // rare: raise the running maxima and rescale the running sums
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float m_new = fmaxf(m_run[r], s[r]);
        const float alpha = exp2f(m_run[r] - m_new);
        l_run[r] *= alpha;
        psum[r] *= alpha;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[r][i] *= alpha;
        m_run[r] = m_new;
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float pr = exp2f(s[r] - m_run[r]);
      l_run[r] += pr;
      const float pv = pr * vsc;
      psum[r] += pv;
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[r][i] = fmaf(pv, f[i], acc[r][i]);
    }
  };

  const int64_t kp_base = b * c.kp_stride[0] + kvh * c.kp_stride[1];
  const int64_t vp_base = b * c.vp_stride[0] + kvh * c.vp_stride[1];
  const int64_t ks_base = b * c.ks_stride[0] + kvh * c.ks_stride[1];
  const int64_t vs_base = b * c.vs_stride[0] + kvh * c.vs_stride[1];

  // Thread 0 is also the copy producer: it fills the ring ahead of the consumers and, after its warp
  // has finished a tile, refills that stage as soon as every warp has released it.
  auto issue_tile = [&](int it) {
    const int st = it % kStages;
    const int tok0 = (tile_begin + it) * kTile;
    const int rows = min(kTile, rl.ctx_len - tok0);
    const uint32_t code_bytes = rows * (kHeadDim / 2);
    const uint32_t scale_bytes = rows * G * 4;
    const uint32_t scale_bulk = scale_bytes & ~15u;
    uint8_t* stage = smem + st * L::kBytes;
    const float* ks_src = c.k_scale + ks_base + static_cast<int64_t>(tok0) * G;
    const float* vs_src = c.v_scale + vs_base + static_cast<int64_t>(tok0) * G;
    // a ragged last tile can leave < 16 bytes of scales that a bulk copy cannot carry
    for (uint32_t o = scale_bulk; o < scale_bytes; o += 4) {
      *reinterpret_cast<float*>(stage + L::kKs + o) = ks_src[o / 4];
      *reinterpret_cast<float*>(stage + L::kVs + o) = vs_src[o / 4];
    }
    mbar_arrive_expect_tx(&bar_full[st], 2 * code_bytes + 2 * scale_bulk);
    bulk_copy_g2s(stage + L::kKc, c.k_packed + kp_base + static_cast<int64_t>(tok0) * (kHeadDim / 2), code_bytes, &bar_full[st]);
    bulk_copy_g2s(stage + L::kVc, c.v_packed + vp_base + static_cast<int64_t>(tok0) * (kHeadDim / 2), code_bytes, &bar_full[st]);
    if (scale_bulk) {
      bulk_copy_g2s(stage + L::kKs, ks_src, scale_bulk, &bar_full[st]);
      bulk_copy_g2s(stage + L::kVs, vs_src, scale_bulk, &bar_full[st]);
    }
  };
  int issued = 0, consumed = 0;  // meaningful in thread 0
  if (threadIdx.x == 0) {
    for (; issued < min(kStages, my_tiles); ++issued) issue_tile(issued);
  }
  {
    for (int it = 0; it < my_tiles; ++it) {
      const int st = it % kStages;
      if (!mbar_wait(&bar_full[st], (it / kStages) & 1, &s_abort)) break;
      consumed = it + 1;
      const uint8_t* stage = smem + st * L::kBytes;
      const int tok0 = (tile_begin + it) * kTile;
      const int rows = min(kTile, rl.ctx_len - tok0);
      uint2 kc[2], vc[2];
      float ksc[2], vsc[2], bias[2];
      int tl[2];
#pragma unroll
      for (int ps = 0; ps < 2; ++ps) {
        tl[ps] = warp * kTokPerWarp + ps * 4 + tg;
        const int t = min(tl[ps], rows - 1);  // ragged tile: stay inside what was copied
        kc[ps] = *reinterpret_cast<const uint2*>(stage + L::kKc + t * 64 + sub * 8);
        vc[ps] = *reinterpret_cast<const uint2*>(stage + L::kVc + t * 64 + sub * 8);
        ksc[ps] = *reinterpret_cast<const float*>(stage + L::kKs + (t * G + (sub * 16) / GS) * 4);
        vsc[ps] = *reinterpret_cast<const float*>(stage + L::kVs + (t * G + (sub * 16) / GS) * 4);
        bias[ps] = 0.0f;
        if (HAS_MASK) {
          const int n = tok0 + t;
          bias[ps] = n < a.mask_k_len ? a.mask[b * a.mask_stride_b + n * a.mask_stride_k] : -INFINITY;
        }
      }
#pragma unroll
      for (int ps = 0; ps < 2; ++ps) process_token(tl[ps] < rows, kc[ps], vc[ps], ksc[ps], vsc[ps], bias[ps]);
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_empty[st]);
      if (threadIdx.x == 0 && issued < my_tiles) {
        if (!mbar_wait(&bar_empty[st], (it / kStages) & 1, &s_abort)) break;
        issue_tile(issued);
        ++issued;
      }
    }
    // after an abort, let copies still in flight land before the CTA's shared memory goes away
    if (threadIdx.x == 0 && s_abort) {
      for (int it = consumed; it < issued; ++it) {
        const int st = it % kStages;
        for (uint32_t i = 0; i < kWaitLimit && !mbar_try_wait(&bar_full[st], (it / kStages) & 1); ++i) {
        }
      }
    }
    if (do_new) {  // the row appended in this step, read back from shared memory by one 8-lane group
      const uint2 kc = *reinterpret_cast<const uint2*>(newrow + sub * 8);
      const uint2 vc = *reinterpret_cast<const uint2*>(newrow + 64 + sub * 8);
      const float ksc = reinterpret_cast<const float*>(newrow + kHeadDim)[(sub * 16) / GS];
      const float vsc = reinterpret_cast<const float*>(newrow + kHeadDim + 64)[(sub * 16) / GS];
      float bias = 0.0f;
      if (HAS_MASK) {
        const int n = rl.seq_len - 1;
        bias = n < a.mask_k_len ? a.mask[b * a.mask_stride_b + n * a.mask_stride_k] : -INFINITY;
      }
      process_token(warp == 0 && tg == 0, kc, vc, ksc, vsc, bias);
    }
    // remove the +136 offset of the unpacked V values, then merge the warp's four token slots
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[r][i] = fmaf(-136.0f, psum[r], acc[r][i]);
    }
#pragma unroll
    for (int o = 8; o < 32; o <<= 1) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float m_o = __shfl_xor_sync(0xFFFFFFFFu, m_run[r], o);
        const float l_o = __shfl_xor_sync(0xFFFFFFFFu, l_run[r], o);
        const float m_n = fmaxf(m_run[r], m_o);
        const float fa = exp2f(m_run[r] - m_n), fb = exp2f(m_o - m_n);
        l_run[r] = l_run[r] * fa + l_o * fb;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a_o = __shfl_xor_sync(0xFFFFFFFFu, acc[r][i], o);
          acc[r][i] = acc[r][i] * fa + a_o * fb;
        }
        m_run[r] = m_n;
      }
    }
  }
  __syncthreads();  // every bulk copy has been consumed (or drained): the ring can be reused
  float* s_acc = reinterpret_cast<float*>(smem);  // [warps][R][128]
  if (tg == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float4* dst = reinterpret_cast<float4*>(s_acc + (warp * R + r) * kHeadDim + sub * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[i] = make_float4(acc[r][4 * i], acc[r][4 * i + 1], acc[r][4 * i + 2], acc[r][4 * i + 3]);
      if (sub == 0) {
        s_m[warp][r] = m_run[r];
        s_l[warp][r] = l_run[r];
      }
    }
  }
  __syncthreads();

  // merge the warps: thread -> (head r, dim d)
  const int hq0 = kvh * R;
  for (int o = threadIdx.x; o < R * kHeadDim; o += kDecodeThreads) {
    const int r = o / kHeadDim, d = o - r * kHeadDim;
    float M = kNegBig;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, s_m[w][r]);
    float Lsum = 0.0f, O = 0.0f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) {
      const float fct = exp2f(s_m[w][r] - M);
      Lsum = fmaf(s_l[w][r], fct, Lsum);
      O = fmaf(s_acc[(w * R + r) * kHeadDim + d], fct, O);
    }
    if (p.splits == 1) {
      store_from_float(a.out, b * a.out_stride[0] + (hq0 + r) * a.out_stride[1] + d * a.out_stride[2], a.dtype, O / Lsum);
    } else {
      const int64_t slot = (static_cast<int64_t>(b) * a.q_heads + hq0 + r) * p.splits + split;
      p.part_acc[slot * kHeadDim + d] = O;
      if (d == 0) {
        p.part_ml[slot * 2] = M;
        p.part_ml[slot * 2 + 1] = Lsum;
      }
    }
  }
  if (p.splits == 1) return;

  // Ticket: the CTA that completes the set merges the splits.  No CTA waits for another.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&p.counters[b * c.kv_heads + kvh], 1);
    s_is_last = (ticket == p.splits - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_is_last) return;
  __threadfence();
  for (int o = threadIdx.x; o < R * kHeadDim; o += kDecodeThreads) {
    const int r = o / kHeadDim, d = o - r * kHeadDim;
    const int64_t slot0 = (static_cast<int64_t>(b) * a.q_heads + hq0 + r) * p.splits;
    float M = kNegBig;
    for (int s = 0; s < p.splits; ++s) M = fmaxf(M, __ldcg(p.part_ml + (slot0 + s) * 2));
    float Lsum = 0.0f, O = 0.0f;
    for (int s = 0; s < p.splits; ++s) {
      const float fct = exp2f(__ldcg(p.part_ml + (slot0 + s) * 2) - M);
      Lsum = fmaf(__ldcg(p.part_ml + (slot0 + s) * 2 + 1), fct, Lsum);
      O = fmaf(__ldcg(p.part_acc + (slot0 + s) * kHeadDim + d), fct, O);
    }
    store_from_float(a.out, b * a.out_stride[0] + (hq0 + r) * a.out_stride[1] + d * a.out_stride[2], a.dtype, O / Lsum);
  }
  if (threadIdx.x == 0) p.counters[b * c.kv_heads + kvh] = 0;  // ready for the next launch
}

}  // namespace lq

#include "lq_int4_mma.cuh"

namespace lq {

// ---- host side ------------------------------------------------------------------------------------
static int validate_cache(const lq_int4_cache& c, const char* who) {
  LQ_CHECK_ARG(c.k_packed && c.v_packed && c.k_scale && c.v_scale, "%s: null cache pointer", who);
  LQ_CHECK_ARG(c.batch > 0 && c.kv_heads > 0 && c.capacity > 0 && c.head_dim > 0, "%s: empty cache", who);
  LQ_CHECK_ARG(c.group_size > 0 && c.head_dim % c.group_size == 0, "%s: head_dim=%d must be divisible by group_size=%d", who,
               c.head_dim, c.group_size);
  LQ_CHECK_ARG(c.group_size % 2 == 0, "%s: group_size=%d must be even for INT4 packing", who, c.group_size);
  return LQ_OK;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Workspace layout: a FIXED region of ticket counters first (one int32 per (batch, kv head), zero
// between launches), then the per-split partial results.  The counter region does not move with
// the problem size, so a buffer reused for a larger problem never finds stale partial results
// where it expects zeroed tickets.
constexpr size_t kMaxTickets = 65536;
constexpr size_t kTicketBytes = kMaxTickets * sizeof(int32_t);

// Split count from a cost model fitted to measurements on B200 (times in units of one 64-token tile
// on one SM, about 0.38 us): an SM works through its CTAs' tiles at the same rate whether one or three
// CTAs are resident, every CTA adds about five tiles' worth of set-up and merge, a lone CTA per SM
// cannot hide its set-up behind a neighbour, and every split adds a little merge traffic.
static int pick_splits(int batch, int kv_heads, int ctx_len) {
  const int ntiles = std::max(1, (ctx_len + kTile - 1) / kTile);
  const int sms = sm_count();
  const int64_t base = static_cast<int64_t>(batch) * kv_heads;
  int best = 1;
  double best_cost = 1.0e300;
  const int max_splits = std::min(ntiles, 128);
  for (int s = 1; s <= max_splits; ++s) {
    const int tps = (ntiles + s - 1) / s;
    if ((ntiles + tps - 1) / tps != s) continue;  // would leave empty splits
    const int64_t per_sm = (base * s + sms - 1) / sms;  // CTAs on the busiest SM
    const double cost = static_cast<double>(per_sm) * (tps + 5.3) + (per_sm == 1 ? 10.5 : 0.0) + 0.05 * s;
    if (cost < best_cost * 0.999) {  // ties go to fewer splits
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

// Raises a kernel's dynamic shared-memory limit once per device and process instead of on every launch (the
// attribute belongs to the function on a device; each expansion site has its own record, one bit per device).
#define LQ_SET_SMEM_ONCE(KERNEL_, BYTES_)                                                                          \
  do {                                                                                                              \
    static std::atomic<unsigned long long> lq_done_{0ull};                                                          \
    int lq_dev_ = 0;                                                                                                \
    LQ_CHECK_CUDA(cudaGetDevice(&lq_dev_));                                                                         \
    const unsigned long long lq_bit_ = 1ull << (lq_dev_ & 63);                                                      \
    if (lq_dev_ > 63 || !(lq_done_.load(std::memory_order_acquire) & lq_bit_)) {                                    \
      LQ_CHECK_CUDA(cudaFuncSetAttribute(KERNEL_, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(BYTES_)));     \
      lq_done_.fetch_or(lq_bit_, std::memory_order_release);                                                        \
    }                                                                                                               \
  } while (0)

template <int R, int GS>
static int launch_decode(const DecodeParams& p, cudaStream_t st) {
  using L = StageLayout<GS>;
  const size_t smem = kStages * L::kBytes + L::kNewRowBytes;
  const dim3 grid(p.splits, p.a.cache.kv_heads, p.a.cache.batch), block(kDecodeThreads);
  if (p.a.mask) {
    LQ_SET_SMEM_ONCE((int4_decode_kernel<R, GS, true>), smem);
    int4_decode_kernel<R, GS, true><<<grid, block, smem, st>>>(p);
  } else {
    LQ_SET_SMEM_ONCE((int4_decode_kernel<R, GS, false>), smem);
    int4_decode_kernel<R, GS, false><<<grid, block, smem, st>>>(p);
  }
  LQ_CHECK_CUDA(cudaGetLastError());
  return LQ_OK;
}

template <int R, int GS>
static int launch_decode_mma(const DecodeParams& p, cudaStream_t st) {
  using L = mma::TileLayout<GS>;
  const size_t smem = mma::kStagesM * L::kStage + L::kNewBytes;
  const dim3 grid(p.splits, p.a.cache.kv_heads, p.a.cache.batch), block(mma::kThreadsM);
#define LQ_MMA_LAUNCH(MASK_, SPLIT_)                                                                                \
  do {                                                                                                              \
    LQ_SET_SMEM_ONCE((mma::int4_decode_mma_kernel<R, GS, MASK_, SPLIT_>), smem);                                    \
    mma::int4_decode_mma_kernel<R, GS, MASK_, SPLIT_><<<grid, block, smem, st>>>(p);                                \
  } while (0)
  const bool qsplit = p.a.dtype != LQ_BF16;
  if (p.a.mask) {
    if (qsplit) LQ_MMA_LAUNCH(true, true); else LQ_MMA_LAUNCH(true, false);
  } else {
    if (qsplit) LQ_MMA_LAUNCH(false, true); else LQ_MMA_LAUNCH(false, false);
  }
#undef LQ_MMA_LAUNCH
  LQ_CHECK_CUDA(cudaGetLastError());
  return LQ_OK;
}

// The tensor-pipe kernel covers group sizes 32 / 64 / 128 (a 16-byte chunk of a row never straddles
// two groups); group size 16 stays on the CUDA-core kernel.  LQ_INT4_KERNEL=cuda_core forces the
// latter (A/B measurements).
static bool use_mma_kernel(int gs) {
  static const bool forced_off = [] {
    const char* e = getenv("LQ_INT4_KERNEL");
    return e != nullptr && strcmp(e, "cuda_core") == 0;
  }();
  return !forced_off && (gs == 32 || gs == 64 || gs == 128);
}

template <int R>
static int launch_decode_gs(const DecodeParams& p, cudaStream_t st) {
  if (use_mma_kernel(p.a.cache.group_size)) {
    switch (p.a.cache.group_size) {
      case 32: return launch_decode_mma<R, 32>(p, st);
      case 64: return launch_decode_mma<R, 64>(p, st);
      default: return launch_decode_mma<R, 128>(p, st);
    }
  }
  switch (p.a.cache.group_size) {
    case 16: return launch_decode<R, 16>(p, st);
    case 32: return launch_decode<R, 32>(p, st);
    case 64: return launch_decode<R, 64>(p, st);
    case 128: return launch_decode<R, 128>(p, st);
    default: return fail(LQ_ERR_UNSUPPORTED, "lq_int4_decode_attn: group_size=%d (supported: 16, 32, 64, 128)", p.a.cache.group_size);
  }
}

}  // namespace lq

using namespace lq;

LQ_EXPORT int lq_int4_kv_append(const lq_int4_cache* cache, const void* k, const int64_t k_stride[4], const void* v,
                                 const int64_t v_stride[4], int32_t dtype, const int64_t* positions, int32_t q_len,
                                 void* cuda_stream) {
  LQ_CHECK_ARG(cache && k && v && k_stride && v_stride && positions, "lq_int4_kv_append: null argument");
  if (int rc = validate_cache(*cache, "lq_int4_kv_append")) return rc;
  LQ_CHECK_ARG(valid_dtype(dtype), "lq_int4_kv_append: bad dtype");
  LQ_CHECK_ARG(q_len > 0, "lq_int4_kv_append: q_len=%d", q_len);
  AppendParams p;
  p.c = *cache; p.k = k; p.v = v; p.dtype = dtype; p.q_len = q_len; p.positions = positions;
  for (int i = 0; i < 4; ++i) { p.ks[i] = k_stride[i]; p.vs[i] = v_stride[i]; }
  const int64_t rows = static_cast<int64_t>(cache->batch) * cache->kv_heads * q_len * 2;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const int gs = cache->group_size, D = cache->head_dim;
  int lanes = gs / 8, lg = 0;
  while ((1 << lg) < lanes) ++lg;
  const bool fast = (gs % 8 == 0) && (D % 8 == 0) && ((1 << lg) == lanes) && lanes <= 32;
  const int block = 256;
  if (fast) {
    const int64_t total = rows * (D / 8);
    const int64_t grid = (total + block - 1) / block;
    LQ_CHECK_ARG(grid < (1ll << 31), "lq_int4_kv_append: too many rows");
    int4_append_kernel<<<static_cast<unsigned>(grid), block, 0, st>>>(p, total, lg);
  } else {
    const int64_t total = rows * (D / gs);
    const int64_t grid = (total + block - 1) / block;
    LQ_CHECK_ARG(grid < (1ll << 31), "lq_int4_kv_append: too many rows");
    int4_append_generic_kernel<<<static_cast<unsigned>(grid), block, 0, st>>>(p, total);
  }
  LQ_CHECK_CUDA(cudaGetLastError());
  return LQ_OK;
}

LQ_EXPORT size_t lq_int4_decode_workspace_bytes(int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                                                 int32_t max_splits) {
  if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || max_splits <= 0) return 0;
  const size_t ml = align_up(static_cast<size_t>(batch) * q_heads * max_splits * 2 * sizeof(float), 256);
  const size_t acc = static_cast<size_t>(batch) * q_heads * max_splits * head_dim * sizeof(float);
  return kTicketBytes + ml + acc;
}

LQ_EXPORT int32_t lq_int4_decode_auto_splits(int32_t batch, int32_t kv_heads, int32_t seq_len) {
  if (batch <= 0 || kv_heads <= 0 || seq_len <= 0) return 1;
  return pick_splits(batch, kv_heads, seq_len);
}

LQ_EXPORT int lq_int4_decode_attn(const lq_int4_decode_args* args, void* cuda_stream) {
  LQ_CHECK_ARG(args != nullptr, "lq_int4_decode_attn: null args");
  const lq_int4_decode_args& a = *args;
  const lq_int4_cache& c = a.cache;
  if (int rc = validate_cache(c, "lq_int4_decode_attn")) return rc;
  LQ_CHECK_ARG(a.q && a.out, "lq_int4_decode_attn: null q/out");
  LQ_CHECK_ARG(valid_dtype(a.dtype), "lq_int4_decode_attn: bad dtype");
  LQ_CHECK_ARG(a.seq_len >= 1 && a.seq_len <= c.capacity, "lq_int4_decode_attn: seq_len=%d outside [1, capacity=%d]", a.seq_len,
               c.capacity);
  LQ_CHECK_ARG(a.q_heads > 0 && a.q_heads % c.kv_heads == 0, "lq_int4_decode_attn: q_heads=%d not a multiple of kv_heads=%d",
               a.q_heads, c.kv_heads);
  LQ_CHECK_ARG((a.k_new == nullptr) == (a.v_new == nullptr), "lq_int4_decode_attn: k_new and v_new go together");
  if (c.head_dim != kHeadDim) return fail(LQ_ERR_UNSUPPORTED, "lq_int4_decode_attn: head_dim=%d (supported: 128)", c.head_dim);
  const int G = c.head_dim / c.group_size;
  // the tile copies need token-contiguous rows inside one (batch, kv head)
  LQ_CHECK_ARG(c.kp_stride[3] == 1 && c.vp_stride[3] == 1 && c.kp_stride[2] == c.head_dim / 2 && c.vp_stride[2] == c.head_dim / 2,
               "lq_int4_decode_attn: packed K/V rows must be contiguous (token stride %d, byte stride 1)", c.head_dim / 2);
  LQ_CHECK_ARG(c.ks_stride[3] == 1 && c.vs_stride[3] == 1 && c.ks_stride[2] == G && c.vs_stride[2] == G,
               "lq_int4_decode_attn: scale rows must be contiguous (token stride %d)", G);
  LQ_CHECK_ARG(reinterpret_cast<uintptr_t>(c.k_packed) % 16 == 0 && reinterpret_cast<uintptr_t>(c.v_packed) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(c.k_scale) % 16 == 0 && reinterpret_cast<uintptr_t>(c.v_scale) % 16 == 0,
               "lq_int4_decode_attn: cache tensors must be 16-byte aligned");
  LQ_CHECK_ARG(c.kp_stride[0] % 16 == 0 && c.kp_stride[1] % 16 == 0 && c.vp_stride[0] % 16 == 0 && c.vp_stride[1] % 16 == 0,
               "lq_int4_decode_attn: packed batch/head strides must be multiples of 16 bytes");
  LQ_CHECK_ARG(c.ks_stride[0] % 4 == 0 && c.ks_stride[1] % 4 == 0 && c.vs_stride[0] % 4 == 0 && c.vs_stride[1] % 4 == 0,
               "lq_int4_decode_attn: scale batch/head strides must be multiples of 4 elements");
  if (a.mask) LQ_CHECK_ARG(a.mask_k_len >= 0, "lq_int4_decode_attn: mask_k_len=%d", a.mask_k_len);

  DecodeParams p;
  p.a = a;
  p.ctx_len = a.seq_len - (a.k_new ? 1 : 0);
  const int ntiles = std::max(1, (p.ctx_len + kTile - 1) / kTile);
  int splits = a.splits > 0 ? a.splits : pick_splits(c.batch, c.kv_heads, std::max(p.ctx_len, 1));
  splits = std::max(1, std::min(std::min(splits, ntiles), mma::kMaxSplitsM));  // the merge holds one factor per split in shared memory
  int tps = (ntiles + splits - 1) / splits;
  splits = (ntiles + tps - 1) / tps;  // no empty splits
  p.splits = splits;
  p.tiles_per_split = tps;
  p.counters = nullptr; p.part_ml = nullptr; p.part_acc = nullptr;
  if (splits > 1) {
    const size_t need = lq_int4_decode_workspace_bytes(c.batch, a.q_heads, c.kv_heads, c.head_dim, splits);
    if (!a.workspace || a.workspace_bytes < need)
      return fail(LQ_ERR_WORKSPACE, "lq_int4_decode_attn: %d splits need %zu workspace bytes, got %zu", splits, need,
                  a.workspace ? a.workspace_bytes : (size_t)0);
    LQ_CHECK_ARG(reinterpret_cast<uintptr_t>(a.workspace) % 256 == 0, "lq_int4_decode_attn: workspace must be 256-byte aligned");
    uint8_t* w = static_cast<uint8_t*>(a.workspace);
    if (static_cast<size_t>(c.batch) * c.kv_heads > kMaxTickets)
      return fail(LQ_ERR_UNSUPPORTED, "lq_int4_decode_attn: batch * kv_heads = %lld exceeds %zu with more than one split",
                  (long long)c.batch * c.kv_heads, kMaxTickets);
    const size_t counters = kTicketBytes;
    const size_t ml = align_up(static_cast<size_t>(c.batch) * a.q_heads * splits * 2 * sizeof(float), 256);
    p.counters = reinterpret_cast<int32_t*>(w);
    p.part_ml = reinterpret_cast<float*>(w + counters);
    p.part_acc = reinterpret_cast<float*>(w + counters + ml);
  }
  LQ_CHECK_ARG(c.batch <= 65535 && c.kv_heads <= 65535, "lq_int4_decode_attn: batch and kv_heads must be <= 65535");
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  switch (a.q_heads / c.kv_heads) {
    case 1: return launch_decode_gs<1>(p, st);
    case 2: return launch_decode_gs<2>(p, st);
    case 4: return launch_decode_gs<4>(p, st);
    case 8: return launch_decode_gs<8>(p, st);
    default:
      return fail(LQ_ERR_UNSUPPORTED, "lq_int4_decode_attn: %d query heads per kv head (supported: 1, 2, 4, 8)", a.q_heads / c.kv_heads);
  }
}

// ---- causal prefill over the quantised cache ---------------------------------------------------------
template <int R, int GS>
static int launch_prefill_mma(const DecodeParams& p, cudaStream_t st) {
  using L = mma::TileLayout<GS>;
  constexpr int QB = 8 / R;  // query positions per CTA: R * QB = 8 head columns
  const size_t smem = mma::kStagesM * L::kStage + L::kNewBytes;
  const dim3 grid(static_cast<unsigned>(p.a.cache.batch) * p.nqb, p.a.cache.kv_heads, 1), block(mma::kThreadsM);
#define LQ_PREFILL_LAUNCH(SPLIT_)                                                                                   \
  do {                                                                                                              \
    LQ_SET_SMEM_ONCE((mma::int4_decode_mma_kernel<R, GS, false, SPLIT_, QB>), smem);                                \
    mma::int4_decode_mma_kernel<R, GS, false, SPLIT_, QB><<<grid, block, smem, st>>>(p);                            \
  } while (0)
  if (p.a.dtype != LQ_BF16) LQ_PREFILL_LAUNCH(true); else LQ_PREFILL_LAUNCH(false);
#undef LQ_PREFILL_LAUNCH
  LQ_CHECK_CUDA(cudaGetLastError());
  return LQ_OK;
}

template <int R>
static int launch_prefill_gs(const DecodeParams& p, cudaStream_t st) {
  switch (p.a.cache.group_size) {
    case 32: return launch_prefill_mma<R, 32>(p, st);
    case 64: return launch_prefill_mma<R, 64>(p, st);
    case 128: return launch_prefill_mma<R, 128>(p, st);
    default:
      return fail(LQ_ERR_UNSUPPORTED, "lq_int4_prefill_attn: group_size=%d (supported: 32, 64, 128)", p.a.cache.group_size);
  }
}

LQ_EXPORT int lq_int4_prefill_attn(const lq_int4_prefill_args* args, void* cuda_stream) {
  LQ_CHECK_ARG(args != nullptr, "lq_int4_prefill_attn: null args");
  const lq_int4_prefill_args& a = *args;
  const lq_int4_cache& c = a.cache;
  if (int rc = validate_cache(c, "lq_int4_prefill_attn")) return rc;
  LQ_CHECK_ARG(a.q && a.out, "lq_int4_prefill_attn: null q/out");
  LQ_CHECK_ARG(valid_dtype(a.dtype), "lq_int4_prefill_attn: bad dtype");
  LQ_CHECK_ARG(a.q_len >= 1 && a.first_len >= 1 && static_cast<int64_t>(a.first_len) + a.q_len - 1 <= c.capacity,
               "lq_int4_prefill_attn: first_len=%d, q_len=%d outside the cache (capacity %d)", a.first_len, a.q_len, c.capacity);
  LQ_CHECK_ARG(a.q_heads > 0 && a.q_heads % c.kv_heads == 0, "lq_int4_prefill_attn: q_heads=%d not a multiple of kv_heads=%d",
               a.q_heads, c.kv_heads);
  if (c.head_dim != kHeadDim) return fail(LQ_ERR_UNSUPPORTED, "lq_int4_prefill_attn: head_dim=%d (supported: 128)", c.head_dim);
  const int G = c.head_dim / c.group_size;
  LQ_CHECK_ARG(c.kp_stride[3] == 1 && c.vp_stride[3] == 1 && c.kp_stride[2] == c.head_dim / 2 && c.vp_stride[2] == c.head_dim / 2,
               "lq_int4_prefill_attn: packed K/V rows must be contiguous (token stride %d, byte stride 1)", c.head_dim / 2);
  LQ_CHECK_ARG(c.ks_stride[3] == 1 && c.vs_stride[3] == 1 && c.ks_stride[2] == G && c.vs_stride[2] == G,
               "lq_int4_prefill_attn: scale rows must be contiguous (token stride %d)", G);
  LQ_CHECK_ARG(reinterpret_cast<uintptr_t>(c.k_packed) % 16 == 0 && reinterpret_cast<uintptr_t>(c.v_packed) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(c.k_scale) % 16 == 0 && reinterpret_cast<uintptr_t>(c.v_scale) % 16 == 0,
               "lq_int4_prefill_attn: cache tensors must be 16-byte aligned");
  LQ_CHECK_ARG(c.kp_stride[0] % 16 == 0 && c.kp_stride[1] % 16 == 0 && c.vp_stride[0] % 16 == 0 && c.vp_stride[1] % 16 == 0,
               "lq_int4_prefill_attn: packed batch/head strides must be multiples of 16 bytes");
  LQ_CHECK_ARG(c.ks_stride[0] % 4 == 0 && c.ks_stride[1] % 4 == 0 && c.vs_stride[0] % 4 == 0 && c.vs_stride[1] % 4 == 0,
               "lq_int4_prefill_attn: scale batch/head strides must be multiples of 4 elements");
  const int ratio = a.q_heads / c.kv_heads;
  if (ratio != 1 && ratio != 2 && ratio != 4 && ratio != 8)
    return fail(LQ_ERR_UNSUPPORTED, "lq_int4_prefill_attn: %d query heads per kv head (supported: 1, 2, 4, 8)", ratio);
  DecodeParams p;
  p.a = lq_int4_decode_args{};
  p.a.cache = c;
  p.a.q = a.q;
  p.a.q_stride[0] = a.q_stride[0]; p.a.q_stride[1] = a.q_stride[1]; p.a.q_stride[2] = a.q_stride[3];
  p.a.out = a.out;
  p.a.out_stride[0] = a.out_stride[0]; p.a.out_stride[1] = a.out_stride[1]; p.a.out_stride[2] = a.out_stride[3];
  p.a.dtype = a.dtype;
  p.a.q_heads = a.q_heads;
  p.a.seq_len = a.first_len + a.q_len - 1;
  p.ctx_len = p.a.seq_len;
  p.splits = 1;
  p.tiles_per_split = (p.ctx_len + kTile - 1) / kTile;
  p.counters = nullptr; p.part_ml = nullptr; p.part_acc = nullptr;
  p.q_len = a.q_len;
  p.first_len = a.first_len;
  p.q_stride_t = a.q_stride[2];
  p.out_stride_t = a.out_stride[2];
  const int qb = (8 / ratio) * mma::kWarpsM;  // query positions per CTA: 8 / ratio per warp
  p.nqb = (a.q_len + qb - 1) / qb;
  LQ_CHECK_ARG(static_cast<int64_t>(c.batch) * p.nqb <= 0x7FFFFFFFLL && c.kv_heads <= 65535,
               "lq_int4_prefill_attn: batch * query blocks or kv_heads too large for one launch");
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  switch (ratio) {
    case 1: return launch_prefill_gs<1>(p, st);
    case 2: return launch_prefill_gs<2>(p, st);
    case 4: return launch_prefill_gs<4>(p, st);
    default: return launch_prefill_gs<8>(p, st);
  }
}

// ---- decode attention with built-in scratch --------------------------------------------------------
// Scratch for lq_int4_decode_attn_static: lives in the library image, so every GPU that loads the
// library holds these bytes until the process exits.  Layout = the ordinary workspace layout (ticket
// region first), sized for LQ_INT4_STATIC_MAX_SLOTS partial results of 128 dimensions.
namespace lq {
constexpr size_t kStaticScratchBytes =
    kTicketBytes + LQ_INT4_STATIC_MAX_SLOTS * 2 * sizeof(float) + LQ_INT4_STATIC_MAX_SLOTS * kHeadDim * sizeof(float);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// The array's name is only a host-side handle; the device address has to be asked for, per device.  Several host
// threads may make the first call on a device at once: each looks the address up and publishes the same value.
static int static_scratch_address(void** out) {
  static std::atomic<void*> cached[64];
  int dev = 0;
  LQ_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(LQ_ERR_UNSUPPORTED, "lq_int4_decode_attn_static: device index %d out of range", dev);
  void* p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    LQ_CHECK_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    if (p == nullptr) return fail(LQ_ERR_CUDA, "lq_int4_decode_attn_static: no device address for the built-in scratch");
    cached[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return LQ_OK;
}
}  // namespace lq

LQ_EXPORT size_t lq_int4_static_scratch_bytes(void) { return lq::kStaticScratchBytes; }

LQ_EXPORT int lq_int4_decode_attn_static(const lq_int4_decode_args* args, void* cuda_stream) {
  LQ_CHECK_ARG(args != nullptr, "lq_int4_decode_attn_static: null args");
  lq_int4_decode_args a = *args;
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  const lq_int4_cache& c = a.cache;
  LQ_CHECK_ARG(c.batch > 0 && c.kv_heads > 0 && a.q_heads > 0 && a.seq_len >= 1, "lq_int4_decode_attn_static: empty problem");
  const int64_t per_split = static_cast<int64_t>(c.batch) * a.q_heads;
  const int64_t max_splits = static_cast<int64_t>(LQ_INT4_STATIC_MAX_SLOTS) / per_split;
  int splits = a.splits;
  const int ctx_len = std::max(a.seq_len - (a.k_new ? 1 : 0), 1);
  if (splits <= 0) {  // library's choice, kept inside what the built-in scratch can hold
    splits = pick_splits(c.batch, c.kv_heads, ctx_len);
    if (splits > max_splits) splits = static_cast<int>(std::max<int64_t>(max_splits, 1));
  } else {
    // an explicit count is used as lq_int4_decode_attn would use it: never more splits than 64-token tiles, nor than 128
    splits = std::min(splits, std::min((ctx_len + kTile - 1) / kTile, 128));
  }
  if (splits > 1 && splits > max_splits) {
    return fail(LQ_ERR_WORKSPACE,
                "lq_int4_decode_attn_static: batch %d x %d query heads x %d splits = %lld partial results exceed the built-in "
                "scratch (%d); use fewer splits or lq_int4_decode_attn with a caller-provided workspace",
                c.batch, a.q_heads, splits, (long long)(per_split * splits), LQ_INT4_STATIC_MAX_SLOTS);
  }
  if (splits > 1 && static_cast<size_t>(c.batch) * c.kv_heads > kMaxTickets)
    return fail(LQ_ERR_WORKSPACE, "lq_int4_decode_attn_static: batch x kv heads = %lld exceeds %zu tickets",
                (long long)c.batch * c.kv_heads, kMaxTickets);
  a.splits = splits;
  a.workspace = scratch;
  a.workspace_bytes = kStaticScratchBytes;
  if (splits > 1) {
    // every call shares the array and finds what the last call left: tickets must start at zero
    LQ_CHECK_CUDA(cudaMemsetAsync(scratch, 0, static_cast<size_t>(c.batch) * c.kv_heads * sizeof(int32_t),
                                  static_cast<cudaStream_t>(cuda_stream)));
  }
  return lq_int4_decode_attn(&a, cuda_stream);
}
