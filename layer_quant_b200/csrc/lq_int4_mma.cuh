// q_len = 1 GQA decode attention over the packed INT4 KV cache on the tensor pipe.
//
// Per kv head the step is a small GEMM pair, S = Q K^T ([R x 128] . [128 x T]) and O = P V
// ([R x T] . [T x 128]) with R = query heads per kv head (4 for Nemotron-H).  On CUDA cores that is
// 4 FMAs per loaded nibble plus the unpack -- about four times the instruction issue a B200 SM can
// spend per byte at HBM speed.  Here the multiply-accumulates go to mma.sync (m16n8k16, bf16 inputs,
// fp32 accumulation): signed nibbles are exact in bf16 and q is bf16 already, so products are exact,
// and what is left for the CUDA cores is unpacking (about one instruction per nibble pair), the
// scales and the softmax.
//
// Layout of one 16-token step of a warp:
//   S:  M = heads (rows 0..R-1 of the 16), N = 8 tokens, K = 16 head dims.  A 16-byte chunk of a K
//       row (32 nibbles) is one quantisation group at group size 32, so every k-step lies inside one
//       group and each chunk gets its own accumulator; scales are applied to the accumulators in
//       fp32.  K nibbles reach the B fragment through ldmatrix (8 token rows x 16 bytes); the k
//       order inside a chunk is permuted, the same permutation is baked into the Q fragments.
//   O:  M = heads, N = 8 head dims, K = 16 tokens.  A = P * v_scale of the chunk, split into
//       bf16 hi (rows 0..7) + lo (rows 8..15) so that P keeps 16 bits of mantissa; the two halves
//       of the fp32 accumulator are added at the end.  V nibbles reach the B fragment through
//       ldmatrix.trans, which hands each thread the same 4 dims of two consecutive tokens.
// Tiles of 64 tokens are staged with 16-byte cp.async copies into a 4-stage ring; the 16-byte
// chunks of a row are XOR-swizzled by (row >> 1) & 3 so that ldmatrix reads without bank conflicts.
#pragma once

#include <type_traits>

#include "lq_common.cuh"

namespace lq {
namespace mma {

constexpr int kD = 128;
constexpr int kTileTok = 64;
constexpr int kStagesM = 4;
constexpr int kWarpsM = 4;
constexpr int kThreadsM = kWarpsM * 32;
constexpr float kNegBigM = -1.0e30f;
constexpr float kSlackM = 8.0f;
constexpr int kMaxSplitsM = 128;  // the merge keeps one factor per (head, split) in shared memory

__device__ __forceinline__ uint32_t s2u(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async16_full(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 2^x by the special-function unit alone (denormal results flush to zero, which is what a softmax wants)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two two's-complement nibbles n (bits 0..3 and 16..19 of x) -> bf16x2 {136 + n, 136 + n} in one LOP3:
// with M = 0x000F000F and K = 0x43084308 the result is (x ^ K) where M is set and K elsewhere, i.e. the
// nibble with its top bit flipped (n + 8) under the bf16 pattern of 128.
__device__ __forceinline__ uint32_t nib_pair_biased(uint32_t x) {
  uint32_t v;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(v) : "r"(x), "r"(0x000F000Fu), "r"(0x43084308u));
  return v;
}
// ... -> bf16x2 {n, n}, exact
__device__ __forceinline__ uint32_t nib_pair_to_bf16x2(uint32_t x) {
  const uint32_t v = nib_pair_biased(x);
  const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v), __float2bfloat162_rn(136.0f));
  return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&r);
}

// byte offset of 16-byte chunk c of row r in a swizzled [rows][64 B] tile
// D = A B + C with C in registers of its own: an accumulator starts from values that stay where they are
__device__ __forceinline__ void mma_bf16_from(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1, float c0, float c1, float c2, float c3) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}

// 8x8 matrix of 16-bit elements held one row per lane group (lane 4 r + c holds row r, columns 2c, 2c+1),
// transposed across the warp
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t c) { return r * 64u + ((c ^ ((r >> 1) & 3u)) << 4); }

// G consecutive fp32 scales of one token from shared memory (one vector load)
template <int G>
__device__ __forceinline__ void load_scales(const uint8_t* p, float (&sc)[G]) {
  if constexpr (G == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    sc[0] = v.x; sc[1] = v.y; sc[2] = v.z; sc[3] = v.w;
  } else if constexpr (G == 2) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    sc[0] = v.x; sc[1] = v.y;
  } else {
    static_assert(G == 1, "group sizes 32, 64 and 128 only");
    sc[0] = *reinterpret_cast<const float*>(p);
  }
}

template <int GS>
struct TileLayout {
  static constexpr int kG = kD / GS;                      // scale groups per row
  static constexpr int kCodeBytes = kTileTok * 64;         // 4096
  static constexpr int kScaleBytes = kTileTok * kG * 4;
  static constexpr int kKc = 0, kVc = kCodeBytes, kKs = 2 * kCodeBytes, kVs = 2 * kCodeBytes + kScaleBytes;
  static constexpr int kStage = 2 * kCodeBytes + 2 * kScaleBytes;
  // the row appended in this step, as a 16-row tile of its own (row 0 real, the rest masked)
  static constexpr int kNewKc = 0, kNewVc = 16 * 64, kNewKs = 2 * 16 * 64, kNewVs = 2 * 16 * 64 + 16 * kG * 4;
  static constexpr int kNewBytes = 2 * 16 * 64 + 2 * 16 * kG * 4;
};


// One CTA (4 warps) per (split, kv head, batch); warp w owns tokens [16 w, 16 w + 16) of every
// 64-token tile.  DecodeParams, int4_scale and int4_code come from lq_int4_kv.cu.
// QSPLIT: the query is not bf16 (fp16 / fp32 callers): it enters the tensor pipe as bf16 hi (rows 0..7)
// + bf16 lo (rows 8..15, otherwise idle), 16 bits of mantissa in all.
// QB: 0 = decode (one query token per sequence).  QB >= 1 = causal prefill over the quantised cache: every
// WARP of the CTA serves QB consecutive query positions of one (batch, kv head) -- 4 QB positions per CTA --
// each (query, head) pair being one head column with its own causal limit (R * QB <= 8 columns); a warp
// walks all 64 tokens of every staged tile its positions may see, so a tile is fetched once for 4 QB
// positions and nothing is merged between warps.  One split, no mask, no fused append.
template <int R, int GS, bool HAS_MASK, bool QSPLIT, int QB = 0>
__global__ void __launch_bounds__(kThreadsM, (R * (QB > 0 ? QB : 1) <= 4 && !QSPLIT) ? 3 : 2)
    int4_decode_mma_kernel(const DecodeParams p) {
  constexpr bool PREFILL = QB > 0;
  constexpr int RV = R * (PREFILL ? QB : 1);  // head columns in use
  static_assert(RV <= 8 && !(PREFILL && HAS_MASK), "at most eight head columns; prefill takes no mask");
  using L = TileLayout<GS>;
  constexpr int G = L::kG;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_is_last;
  __shared__ float s_m[kWarpsM][8], s_l[kWarpsM][8];

  const lq_int4_decode_args& a = p.a;
  const lq_int4_cache& c = a.cache;
  const int split = PREFILL ? 0 : blockIdx.x, kvh = blockIdx.y;
  const int b = PREFILL ? static_cast<int>(blockIdx.x) / p.nqb : blockIdx.z;
  const int cta_q_first = PREFILL ? (static_cast<int>(blockIdx.x) - b * p.nqb) * (QB * kWarpsM) : 0;  // first position of the CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;  // mma fragment coordinates: row / column group
  const int q_first = PREFILL ? cta_q_first + warp * QB : 0;  // first query position of this warp
  // Head columns.  Both products put the heads on the n side (8 columns).  Up to four query heads per kv
  // head: columns 4..7 repeat columns 0..3, so that the O^T product can take the bf16 hi part of
  // P * v_scale from columns 0..3 and the lo part from columns 4..7 of ONE n-tile.  Eight heads: columns
  // are heads, hi and lo parts go to two n-tiles.  In the Q^T fragments (B operand) column n = g; in the
  // accumulators a lane owns columns 2t and 2t + 1.
  constexpr bool DUP = RV <= 4;
  constexpr int NT = DUP ? 1 : 2;
  const int hrow = DUP ? (g & 3) : g;
  const bool is_lo = DUP && t >= 2;
  const uint32_t lo_mul = is_lo ? 65536u : 0u, lo_mask = is_lo ? 0xFFFF0000u : 0u;
  const bool fused_new = !PREFILL && a.k_new != nullptr;
  uint8_t* newtile = smem + kStagesM * L::kStage;

  RunLengths rl = run_lengths(p);
  if (PREFILL) {  // the CTA reads up to its last query's own position
    rl.seq_len = p.first_len + min(cta_q_first + QB * kWarpsM - 1, p.q_len - 1);
    rl.ctx_len = rl.seq_len;
    rl.tiles_per_split = (rl.ctx_len + kTileTok - 1) / kTileTok;
  }
  const int ntiles = (rl.ctx_len + kTileTok - 1) / kTileTok;
  const int tile_begin = split * rl.tiles_per_split;
  const int tile_end = min(ntiles, tile_begin + rl.tiles_per_split);
  const int my_tiles = max(0, tile_end - tile_begin);
  const bool do_new = fused_new && split == p.splits - 1;
  if (threadIdx.x == 0) s_is_last = 0;

  const int64_t kp_base = b * c.kp_stride[0] + kvh * c.kp_stride[1];
  const int64_t vp_base = b * c.vp_stride[0] + kvh * c.vp_stride[1];
  const int64_t ks_base = b * c.ks_stride[0] + kvh * c.ks_stride[1];
  const int64_t vs_base = b * c.vs_stride[0] + kvh * c.vs_stride[1];

  // ---- staging: every thread copies the same four code chunks and (at most) one scale chunk of every tile:
  // rows r0 and r0 + 32, chunk ch, of K and of V (the swizzle of rows r and r + 32 is the same) ---------
  const uint32_t r0 = threadIdx.x >> 2, ch = threadIdx.x & 3;
  const uint32_t code_src_off = r0 * 64 + ch * 16;
  const uint32_t code_dst_off = swz(r0, ch);
  constexpr int kScaleChunks = L::kScaleBytes / 16;          // per tensor
  const bool has_scale_chunk = threadIdx.x < 2 * kScaleChunks;
  const int scale_which = threadIdx.x >= kScaleChunks;       // 0: K scales, 1: V scales
  const int scale_off = (scale_which ? threadIdx.x - kScaleChunks : threadIdx.x) * 16;
  const uint8_t* const k_rows = c.k_packed + kp_base;
  const uint8_t* const v_rows = c.v_packed + vp_base;
  const uint8_t* const scale_rows = reinterpret_cast<const uint8_t*>(scale_which ? c.v_scale + vs_base : c.k_scale + ks_base);
  const uint32_t smem_base = s2u(smem);
  // Tiles are issued in order, so a full tile costs five copies from running pointers; the last, partial tile of the
  // context takes the general form with per-row byte counts (rows past the end are zero-filled).
  const uint8_t* k_src = k_rows + static_cast<int64_t>(tile_begin) * (kTileTok * 64) + code_src_off;
  const uint8_t* v_src = v_rows + static_cast<int64_t>(tile_begin) * (kTileTok * 64) + code_src_off;
  const uint8_t* s_src = scale_rows + static_cast<int64_t>(tile_begin) * (kTileTok * G * 4) + scale_off;
  auto issue_tile = [&](int it) {
    const uint32_t stage = smem_base + (it % kStagesM) * L::kStage;
    const int tok0 = (tile_begin + it) * kTileTok;
    if (tok0 + kTileTok <= rl.ctx_len) {
      cp_async16_full(stage + L::kKc + code_dst_off, k_src);
      cp_async16_full(stage + L::kKc + code_dst_off + 2048, k_src + 2048);
      cp_async16_full(stage + L::kVc + code_dst_off, v_src);
      cp_async16_full(stage + L::kVc + code_dst_off + 2048, v_src + 2048);
      if (has_scale_chunk) cp_async16_full(stage + (scale_which ? L::kVs : L::kKs) + scale_off, s_src);
    } else {
      const int rows = rl.ctx_len - tok0;
      const uint32_t ok0 = static_cast<int>(r0) < rows ? 16u : 0u, ok1 = static_cast<int>(r0) + 32 < rows ? 16u : 0u;
      const int64_t back = -static_cast<int64_t>(code_src_off);  // rows past the end copy nothing, from the tile's first byte
      cp_async16(stage + L::kKc + code_dst_off, k_src + (ok0 ? 0 : back), ok0);
      cp_async16(stage + L::kKc + code_dst_off + 2048, k_src + (ok1 ? 2048 : back), ok1);
      cp_async16(stage + L::kVc + code_dst_off, v_src + (ok0 ? 0 : back), ok0);
      cp_async16(stage + L::kVc + code_dst_off + 2048, v_src + (ok1 ? 2048 : back), ok1);
      if (has_scale_chunk) {
        const int left = rows * G * 4 - scale_off;
        const uint32_t nbytes = left >= 16 ? 16u : (left > 0 ? static_cast<uint32_t>(left) : 0u);
        cp_async16(stage + (scale_which ? L::kVs : L::kKs) + scale_off, s_src - (nbytes ? 0 : scale_off), nbytes);
      }
    }
    k_src += kTileTok * 64;
    v_src += kTileTok * 64;
    s_src += kTileTok * G * 4;
  };

  // start the ring now: the first tiles travel while the new row is quantised and the Q fragments are built
  for (int it = 0; it < kStagesM - 1; ++it) {
    if (it < my_tiles) issue_tile(it);
    cp_async_commit();
  }

  // the new row's values are fetched now and quantised after the Q fragments, so that the two sets of
  // loads are in flight together
  float xnew[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (do_new && warp < 2) {
    const void* src = warp == 0 ? a.k_new : a.v_new;
    const int64_t* ss = warp == 0 ? a.k_new_stride : a.v_new_stride;
#pragma unroll
    for (int i = 0; i < 4; ++i) xnew[i] = load_as_float(src, b * ss[0] + kvh * ss[1] + (lane * 4 + i) * ss[2], a.dtype);
  }
  if (do_new) {
    for (int i = threadIdx.x; i < L::kNewBytes / 16; i += kThreadsM) reinterpret_cast<uint4*>(newtile)[i] = make_uint4(0, 0, 0, 0);
  }

  // ---- Q fragments (A operand of S), in the k order the K unpack produces ------------------------------
  // chunk i, k-step s (0: nibbles 0,4,1,5; 1: nibbles 2,6,3,7 of this thread's 8-nibble word)
  // The K side feeds 136 + n to the tensor pipe and starts each chunk's accumulator at -136 * sum(q over
  // the chunk) instead (two mma per accumulator, so no long cancellation); qoff[i] is that start value
  // for head g, the sum taken over the bf16 values the fragments actually hold.
  uint32_t qa[4][2][2];
  uint32_t ql[QSPLIT ? 4 : 1][2][2];  // lo halves (QSPLIT only)
  float qoff[4], qoff_lo[QSPLIT ? 4 : 1];
  auto bf_lo = [](uint32_t v) { return __uint_as_float(v << 16); };
  auto bf_hi = [](uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); };
  // this lane's query row; a bf16 query whose head dims are contiguous and 16-byte aligned arrives as one 128-bit load per
  // chunk (the lane's eight dims 32 i + 8 t .. + 7), anything else as scalar loads
  const bool q_row_valid = hrow < RV && (!PREFILL || q_first + hrow / R < p.q_len);
  const int64_t q_row_base = b * a.q_stride[0] + (kvh * R + hrow % R) * a.q_stride[1] +
                             (PREFILL ? (q_first + hrow / R) * p.q_stride_t : 0);
  const bool q_vec = !QSPLIT && a.dtype == LQ_BF16 && a.q_stride[2] == 1 &&
                     ((reinterpret_cast<uintptr_t>(a.q) | (static_cast<uint64_t>(a.q_stride[0]) * 2) |
                       (static_cast<uint64_t>(a.q_stride[1]) * 2) | (PREFILL ? static_cast<uint64_t>(p.q_stride_t) * 2 : 0)) & 15) == 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float qs = 0.0f, qs_lo = 0.0f;
    uint4 qw = make_uint4(0u, 0u, 0u, 0u);  // dims 8t .. 8t+7 of chunk i as bf16 pairs (vector path)
    if (q_vec && q_row_valid)
      qw = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.q) + q_row_base + 32 * i + 8 * t));
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int d0 = 32 * i + 8 * t + 2 * s;
      uint32_t pa, pb;
      float q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
      if (q_vec) {  // (dim d0, d0 + 4) and (d0 + 1, d0 + 5) out of the eight loaded values
        const uint32_t wl = s == 0 ? qw.x : qw.y, wh = s == 0 ? qw.z : qw.w;
        pa = __byte_perm(wl, wh, 0x5410);
        pb = __byte_perm(wl, wh, 0x7632);
      } else {
        if (q_row_valid) {
          q0 = load_as_float(a.q, q_row_base + (d0 + 0) * a.q_stride[2], a.dtype);
          q1 = load_as_float(a.q, q_row_base + (d0 + 4) * a.q_stride[2], a.dtype);
          q2 = load_as_float(a.q, q_row_base + (d0 + 1) * a.q_stride[2], a.dtype);
          q3 = load_as_float(a.q, q_row_base + (d0 + 5) * a.q_stride[2], a.dtype);
        }
        pa = pack_bf16x2(q0, q1);
        pb = pack_bf16x2(q2, q3);
      }
      qa[i][s][0] = pa;  // a0: row g, k = 2t, 2t+1
      qa[i][s][1] = pb;  // a2: row g, k = 2t+8, 2t+9
      qs += (bf_lo(pa) + bf_hi(pa)) + (bf_lo(pb) + bf_hi(pb));  // of the values the fragments hold
      if (QSPLIT) {
        const uint32_t la = pack_bf16x2(q0 - bf_lo(pa), q1 - bf_hi(pa)), lb = pack_bf16x2(q2 - bf_lo(pb), q3 - bf_hi(pb));
        ql[i][s][0] = la;  // a1: row g + 8
        ql[i][s][1] = lb;  // a3
        qs_lo += (bf_lo(la) + bf_hi(la)) + (bf_lo(lb) + bf_hi(lb));
      }
    }
    qs += __shfl_xor_sync(0xFFFFFFFFu, qs, 1);  // the chunk's 32 dims live in the four lanes of row g
    qs += __shfl_xor_sync(0xFFFFFFFFu, qs, 2);
    qoff[i] = -136.0f * qs;
    if (QSPLIT) {
      qs_lo += __shfl_xor_sync(0xFFFFFFFFu, qs_lo, 1);
      qs_lo += __shfl_xor_sync(0xFFFFFFFFu, qs_lo, 2);
      qoff_lo[i] = -136.0f * qs_lo;
    }
  }
  // accumulator start values of this lane's two columns (the sums live in the lanes of row g = column)
  float qstart[4][2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float v = QSPLIT ? qoff[i] + qoff_lo[QSPLIT ? i : 0] : qoff[i];
    qstart[i][0] = __shfl_sync(0xFFFFFFFFu, v, 8 * t);      // lane (g = 2t, t = 0)
    qstart[i][1] = __shfl_sync(0xFFFFFFFFu, v, 8 * t + 4);  // lane (g = 2t + 1, t = 0)
  }
  // ---- fused append: quantise the new K / V row, write it to the cache and into a 16-row tile -------
  __syncthreads();  // the tile of the new row is zeroed
  if (do_new && warp < 2) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(xnew[i]));
#pragma unroll
    for (int o = GS / 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    const float scale = int4_scale(amax);
    uint32_t half = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) half |= int4_code(xnew[i], scale) << (4 * i);
    const int pos = rl.seq_len - 1;
    uint8_t* gcodes = (warp == 0 ? c.k_packed + kp_base + static_cast<int64_t>(pos) * c.kp_stride[2]
                                 : c.v_packed + vp_base + static_cast<int64_t>(pos) * c.vp_stride[2]);
    reinterpret_cast<uint16_t*>(gcodes)[lane] = static_cast<uint16_t>(half);
    reinterpret_cast<uint16_t*>(newtile + (warp == 0 ? L::kNewKc : L::kNewVc))[lane] = static_cast<uint16_t>(half);  // row 0: no swizzle
    if ((lane * 4) % GS == 0) {
      float* gsc = (warp == 0 ? c.k_scale + ks_base + static_cast<int64_t>(pos) * c.ks_stride[2]
                              : c.v_scale + vs_base + static_cast<int64_t>(pos) * c.vs_stride[2]);
      gsc[lane * 4 / GS] = scale;
      reinterpret_cast<float*>(newtile + (warp == 0 ? L::kNewKs : L::kNewVs))[lane * 4 / GS] = scale;
    }
  }

  const float scale_sm = 1.4426950408889634f / sqrtf(static_cast<float>(kD));

  // O^T accumulators: m-tile (chunk i, half sp) has row g = dim 32 i + 4 g + 2 sp and row g + 8 = that
  // dim + 1; columns 2t, 2t+1 are heads (DUP: head c & 3, hi part for c < 4, lo part for c >= 4).
  float oacc[4][2][NT][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int sp = 0; sp < 2; ++sp)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[i][sp][nt][e] = 0.0f;
  const int col_head0 = DUP ? ((2 * t) & 3) : 2 * t;  // head column of accumulator column 2t (column 2t+1: the next one)
  // prefill: the tokens a column may see, [0, its query's position]
  int col_limit[2] = {0x7FFFFFFF, 0x7FFFFFFF};
  int warp_limit = 0x7FFFFFFF;  // tokens this warp's positions may see at all (0: the warp has no position)
  if (PREFILL) {
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) col_limit[cc] = p.first_len + min(q_first + (col_head0 + cc) / R, p.q_len - 1);
    warp_limit = q_first < p.q_len ? p.first_len + min(q_first + QB - 1, p.q_len - 1) : 0;
  }
  float m_run[2] = {kNegBigM, kNegBigM}, l_run[2] = {0.0f, 0.0f};  // this lane's two columns (l: this lane's share)

  // Per-thread offsets inside a tile for this warp's 16 rows (row0 = 16 * warp; 0 for the new-row tile):
  // ldmatrix row addresses for K (two 8-token halves) and V (two chunk pairs), and the scale rows of
  // the two tokens this thread owns in the S^T fragments (rows g and g + 8).
  auto make_offsets = [&](int row0, uint32_t (&koff)[2], uint32_t (&voff)[2], uint32_t (&soff)[2]) {
#pragma unroll
    for (int j = 0; j < 2; ++j) koff[j] = swz(row0 + 8 * j + (lane & 7), lane >> 3);
    const int mtx = lane >> 3;
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) voff[cp] = swz(row0 + 8 * (mtx & 1) + (lane & 7), 2 * cp + (mtx >> 1));
#pragma unroll
    for (int r = 0; r < 2; ++r) soff[r] = (row0 + g + 8 * r) * G * 4;
  };
  uint32_t koff[2], voff[2], soff[2];
  make_offsets(PREFILL ? 0 : 16 * warp, koff, voff, soff);

  // One 16-token step of this warp.  kc / vc / ksc / vsc: shared-memory addresses of the tile's parts.
  // FULL: all 16 rows hold tokens (no validity selects); otherwise the first `valid` rows do, and the
  // rest were zero-filled by the staging copies (codes 0, scales 0), so they only need masking in S.
  auto step16 = [&](auto full_tag, uint32_t kc, uint32_t vc, const uint8_t* ksc, const uint8_t* vsc, const uint32_t (&ko)[2],
                    const uint32_t (&vo)[2], const uint32_t (&so)[2], int valid, int tok_first) {
    constexpr bool FULL = decltype(full_tag)::value;
    // S^T = K Q^T: M = the 16 tokens (rows g and g + 8), N = head columns, K = 16 dims per mma; the unpacked
    // codes are the A operand, the Q^T fragments stay in registers.  One accumulator per 16-byte chunk.
    float sacc[4][4];
    {
      uint32_t kr0[4], kr1[4];
      ldmatrix_x4(kr0, kc + ko[0]);
      ldmatrix_x4(kr1, kc + ko[1]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t w0 = kr0[i], w1 = kr1[i];
        mma_bf16_from(sacc[i], nib_pair_biased(w0), nib_pair_biased(w1), nib_pair_biased(w0 >> 4), nib_pair_biased(w1 >> 4),
                      qa[i][0][0], qa[i][0][1], qstart[i][0], qstart[i][1], qstart[i][0], qstart[i][1]);
        if (QSPLIT)
          mma_bf16(sacc[i], nib_pair_biased(w0), nib_pair_biased(w1), nib_pair_biased(w0 >> 4), nib_pair_biased(w1 >> 4),
                   ql[QSPLIT ? i : 0][0][0], ql[QSPLIT ? i : 0][0][1]);
        mma_bf16(sacc[i], nib_pair_biased(w0 >> 8), nib_pair_biased(w1 >> 8), nib_pair_biased(w0 >> 12), nib_pair_biased(w1 >> 12),
                 qa[i][1][0], qa[i][1][1]);
        if (QSPLIT)
          mma_bf16(sacc[i], nib_pair_biased(w0 >> 8), nib_pair_biased(w1 >> 8), nib_pair_biased(w0 >> 12),
                   nib_pair_biased(w1 >> 12), ql[QSPLIT ? i : 0][1][0], ql[QSPLIT ? i : 0][1][1]);
      }
    }
    // scores of tokens g (r = 0) and g + 8 (r = 1) for this lane's two columns
    float sv[2][2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float sc[G];
      load_scales(ksc + so[r], sc);
      const int rr = g + 8 * r;
      float bias = 0.0f;
      if (HAS_MASK) {
        const int n = tok_first + rr;
        bias = ((FULL || rr < valid) && n < a.mask_k_len) ? a.mask[b * a.mask_stride_b + n * a.mask_stride_k] : -INFINITY;
      }
      // both columns of the token at once: packed fp32x2 FMA / MUL (sm_100), same rounding per component
      float2 sum2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float k = sc[(32 * i) / GS];
        sum2 = __ffma2_rn(make_float2(k, k), make_float2(sacc[i][2 * r], sacc[i][2 * r + 1]), sum2);
      }
      sum2 = __fmul2_rn(sum2, make_float2(scale_sm, scale_sm));
      const float sums[2] = {sum2.x, sum2.y};
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        float sum = sums[cc];
        if (HAS_MASK) sum += bias;
        sv[r][cc] = ((FULL || rr < valid) && (!PREFILL || tok_first + rr < col_limit[cc])) ? sum : -INFINITY;
      }
    }
    // online softmax per column; the running max of a column is shared by the eight lanes that hold it.
    // Columns without a head (zero Q) run along harmlessly and are never read.
    const float smax0 = fmaxf(sv[0][0], sv[1][0]), smax1 = fmaxf(sv[0][1], sv[1][1]);
    if (__any_sync(0xFFFFFFFFu, smax0 > m_run[0] + kSlackM || smax1 > m_run[1] + kSlackM)) {
      float rm0 = smax0, rm1 = smax1;
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        rm0 = fmaxf(rm0, __shfl_xor_sync(0xFFFFFFFFu, rm0, o));
        rm1 = fmaxf(rm1, __shfl_xor_sync(0xFFFFFFFFu, rm1, o));
      }
      const float n0 = fmaxf(m_run[0], rm0), n1 = fmaxf(m_run[1], rm1);
      const float alpha0 = fast_exp2(m_run[0] - n0), alpha1 = fast_exp2(m_run[1] - n1);
      l_run[0] *= alpha0;
      l_run[1] *= alpha1;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int sp = 0; sp < 2; ++sp)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            oacc[i][sp][nt][0] *= alpha0;
            oacc[i][sp][nt][1] *= alpha1;
            oacc[i][sp][nt][2] *= alpha0;
            oacc[i][sp][nt][3] *= alpha1;
          }
      m_run[0] = n0;
      m_run[1] = n1;
    }
    float pv[2][2];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        pv[r][cc] = fast_exp2(sv[r][cc] - m_run[cc]);  // 0 for masked / padded tokens
        l_run[cc] += pv[r][cc];
      }
    // B operand of O^T: (P * v_scale)^T per scale group, k = the tokens 2t, 2t+1 (+8), n = column g.  What
    // this lane has is the other way round (token g / g + 8, columns 2t, 2t+1), so each packed pair goes
    // through movmatrix.  A lane of columns 0..3 keeps the bf16 rounding of the product, a lane of
    // columns 4..7 the bf16 rounding of what that left over (one formula: the part taken off is masked
    // to zero on the hi lanes).
    uint32_t pb[G][2][NT];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float vs[G];
      load_scales(vsc + so[r], vs);
#pragma unroll
      for (int q = 0; q < G; ++q) {
        const float2 pp = __fmul2_rn(make_float2(pv[r][0], pv[r][1]), make_float2(vs[q], vs[q]));
        const uint32_t hi = pack_bf16x2(pp.x, pp.y);
        if (DUP) {
          const float2 lo = __ffma2_rn(make_float2(__uint_as_float(hi * lo_mul), __uint_as_float(hi & lo_mask)), make_float2(-1.0f, -1.0f), pp);
          pb[q][r][0] = movmatrix_trans(pack_bf16x2(lo.x, lo.y));
        } else {
          const float2 lo = __ffma2_rn(make_float2(__uint_as_float(hi << 16), __uint_as_float(hi & 0xFFFF0000u)), make_float2(-1.0f, -1.0f), pp);
          pb[q][r][0] = movmatrix_trans(hi);
          pb[q][r][NT - 1] = movmatrix_trans(pack_bf16x2(lo.x, lo.y));
        }
      }
    }
    // O^T += V^T (P * v_scale)^T, chunk by chunk: the unpacked codes are the A operand
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) {
      uint32_t vr[4];
      ldmatrix_x4_trans(vr, vc + vo[cp]);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = 2 * cp + h;
        const int q = (32 * i) / GS;
        const uint32_t w0 = vr[2 * h], w1 = vr[2 * h + 1];
#pragma unroll
        for (int sp = 0; sp < 2; ++sp) {
          const uint32_t a0 = nib_pair_to_bf16x2(w0 >> (8 * sp)), a1 = nib_pair_to_bf16x2(w0 >> (8 * sp + 4));
          const uint32_t a2 = nib_pair_to_bf16x2(w1 >> (8 * sp)), a3 = nib_pair_to_bf16x2(w1 >> (8 * sp + 4));
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma_bf16(oacc[i][sp][nt], a0, a1, a2, a3, pb[q][0][nt], pb[q][1][nt]);
        }
      }
    }
  };

  // ---- main loop: 4-stage cp.async ring (its first stages were started before the prologue) --------
  for (int it = 0; it < my_tiles; ++it) {
    cp_async_wait<kStagesM - 2>();
    __syncthreads();  // tile `it` has landed for everyone; everyone is done with tile it - 1
    if (it + kStagesM - 1 < my_tiles) issue_tile(it + kStagesM - 1);
    cp_async_commit();
    const uint8_t* stage = smem + (it % kStagesM) * L::kStage;
    const int tok0 = (tile_begin + it) * kTileTok;
    const int rows = min(kTileTok, rl.ctx_len - tok0);
    const uint32_t sb = s2u(stage);
    if (PREFILL) {
#pragma unroll 1
      for (int blk = 0; blk < kTileTok / 16; ++blk) {  // the warp's own positions over the whole tile
        const int r16 = 16 * blk;
        if (r16 >= rows || tok0 + r16 >= warp_limit) break;
        const uint32_t cb = blk * (16 * 64);
        const int sbo = blk * (16 * G * 4);
        if (rows - r16 >= 16)
          step16(std::true_type{}, sb + L::kKc + cb, sb + L::kVc + cb, stage + L::kKs + sbo, stage + L::kVs + sbo, koff, voff, soff,
                 16, tok0 + r16);
        else
          step16(std::false_type{}, sb + L::kKc + cb, sb + L::kVc + cb, stage + L::kKs + sbo, stage + L::kVs + sbo, koff, voff,
                 soff, rows - r16, tok0 + r16);
      }
      continue;
    }
    const int row0 = 16 * warp;
    if (rows - row0 >= 16)
      step16(std::true_type{}, sb + L::kKc, sb + L::kVc, stage + L::kKs, stage + L::kVs, koff, voff, soff, 16, tok0 + row0);
    else if (row0 < rows)
      step16(std::false_type{}, sb + L::kKc, sb + L::kVc, stage + L::kKs, stage + L::kVs, koff, voff, soff, rows - row0,
             tok0 + row0);
  }
  cp_async_wait<0>();
  __syncthreads();
  if (do_new && warp == 0) {
    uint32_t ko0[2], vo0[2], so0[2];
    make_offsets(0, ko0, vo0, so0);
    const uint32_t nb = s2u(newtile);
    step16(std::false_type{}, nb + L::kNewKc, nb + L::kNewVc, newtile + L::kNewKs, newtile + L::kNewVs, ko0, vo0, so0, 1,
           rl.seq_len - 1);
  }

  // ---- merge the warps -------------------------------------------------------------------------------------
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {  // a column's denominator: over the eight lanes (token rows) that share it
    l_run[0] += __shfl_xor_sync(0xFFFFFFFFu, l_run[0], o);
    l_run[1] += __shfl_xor_sync(0xFFFFFFFFu, l_run[1], o);
  }
  float* s_acc = reinterpret_cast<float*>(smem);  // [warps][R][128], reuses the ring
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int sp = 0; sp < 2; ++sp)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v;
        if (DUP) {
          v = oacc[i][sp][0][e];
          v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);  // hi columns (t < 2) + lo columns (t >= 2) of the same heads
        } else {
          v = oacc[i][sp][0][e] + oacc[i][sp][NT - 1][e];
        }
        const int head = col_head0 + (e & 1);
        const int dim = 32 * i + 4 * g + 2 * sp + (e >> 1);
        if ((!DUP || t < 2) && head < RV) s_acc[(warp * RV + head) * kD + dim] = v;
      }
  if (g == 0 && (!DUP || t < 2)) {
#pragma unroll
    for (int cc = 0; cc < 2; ++cc)
      if (col_head0 + cc < RV) {
        s_m[warp][col_head0 + cc] = m_run[cc];
        s_l[warp][col_head0 + cc] = l_run[cc];
      }
  }
  __syncthreads();
  const int hq0 = kvh * R;
  for (int o = threadIdx.x; o < RV * kD; o += kThreadsM) {
    const int r = o / kD, d = o - r * kD;
    float M = kNegBigM;
#pragma unroll
    for (int w = 0; w < kWarpsM; ++w) M = fmaxf(M, s_m[w][r]);
    float Lsum = 0.0f, O = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarpsM; ++w) {
      const float fct = exp2f(s_m[w][r] - M);
      Lsum = fmaf(s_l[w][r], fct, Lsum);
      O = fmaf(s_acc[(w * RV + r) * kD + d], fct, O);
    }
    if (PREFILL) {
      // every warp holds complete results for its own positions: nothing to merge
#pragma unroll
      for (int w = 0; w < kWarpsM; ++w) {
        const int qi = cta_q_first + w * QB + r / R;
        if (qi < p.q_len)
          store_from_float(a.out, b * a.out_stride[0] + (hq0 + r % R) * a.out_stride[1] + qi * p.out_stride_t + d * a.out_stride[2],
                           a.dtype, s_acc[(w * RV + r) * kD + d] / s_l[w][r]);
      }
    } else if (p.splits == 1) {
      store_from_float(a.out, b * a.out_stride[0] + (hq0 + r) * a.out_stride[1] + d * a.out_stride[2], a.dtype, O / Lsum);
    } else {
      const int64_t slot = (static_cast<int64_t>(b) * a.q_heads + hq0 + r) * p.splits + split;
      p.part_acc[slot * kD + d] = O;
      if (d == 0) {
        p.part_ml[slot * 2] = M;
        p.part_ml[slot * 2 + 1] = Lsum;
      }
    }
  }
  if (PREFILL || p.splits == 1) return;

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
  // (1) one warp per head: the maximum over the splits, each split's factor (to shared memory) and the
  // denominator; (2) one thread per output: the weighted sum, its loads independent of one another.
  float* s_f = reinterpret_cast<float*>(smem);  // [R][kMaxSplitsM], reuses the ring
  float* s_den = s_f + R * kMaxSplitsM;         // [R]
  for (int r = warp; r < R; r += kWarpsM) {
    const float* ml = p.part_ml + (static_cast<int64_t>(b) * a.q_heads + hq0 + r) * p.splits * 2;
    float M = kNegBigM;
    for (int s = lane; s < p.splits; s += 32) M = fmaxf(M, __ldcg(ml + 2 * s));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
    float den = 0.0f;
    for (int s = lane; s < p.splits; s += 32) {
      const float fct = exp2f(__ldcg(ml + 2 * s) - M);
      s_f[r * kMaxSplitsM + s] = fct;
      den = fmaf(__ldcg(ml + 2 * s + 1), fct, den);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xFFFFFFFFu, den, o);
    if (lane == 0) s_den[r] = den;
  }
  __syncthreads();
  // four outputs per thread: the splits' partial results arrive as independent 128-bit loads, eight in flight per thread
  for (int o = threadIdx.x; o < R * (kD / 4); o += kThreadsM) {
    const int r = o / (kD / 4), d = (o - r * (kD / 4)) * 4;
    const float4* acc = reinterpret_cast<const float4*>(p.part_acc + (static_cast<int64_t>(b) * a.q_heads + hq0 + r) * p.splits * kD + d);
    float4 O = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
    for (int s = 0; s < p.splits; ++s) {
      const float4 v = __ldcg(acc + static_cast<int64_t>(s) * (kD / 4));
      const float f = s_f[r * kMaxSplitsM + s];
      O.x = fmaf(v.x, f, O.x); O.y = fmaf(v.y, f, O.y); O.z = fmaf(v.z, f, O.z); O.w = fmaf(v.w, f, O.w);
    }
    const float den = s_den[r];
    const int64_t ob = b * a.out_stride[0] + (hq0 + r) * a.out_stride[1] + d * a.out_stride[2];
    store_from_float(a.out, ob, a.dtype, O.x / den);
    store_from_float(a.out, ob + a.out_stride[2], a.dtype, O.y / den);
    store_from_float(a.out, ob + 2 * a.out_stride[2], a.dtype, O.z / den);
    store_from_float(a.out, ob + 3 * a.out_stride[2], a.dtype, O.w / den);
  }
  if (threadIdx.x == 0) p.counters[b * c.kv_heads + kvh] = 0;  // ready for the next launch
}

}  // namespace mma
}  // namespace lq
