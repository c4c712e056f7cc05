/*
 * layer_quant_b200 -- C ABI of the B200 (sm_100a) kernels behind the two Nemotron-H decode hot
 * paths of phcool/Layer_Quant: q_len = 1 GQA attention over a packed INT4 KV cache, and the
 * Mamba2 selective-state update on a recurrent state held in MX8 / MX4 blocks.
 *
 * Conventions
 *   - Every pointer named "device" memory is a raw CUDA device pointer owned by the caller.
 *   - Strides are in ELEMENTS of the tensor they describe.
 *   - Every entry point returns LQ_OK (0) or a negative LQ_ERR_* code, never throws, launches on
 *     the given stream and does not synchronise.  lq_last_error_string() describes the last
 *     failure seen by the calling thread.
 *   - No entry point allocates device memory; scratch ("workspace") is passed in.
 *
 * Each declaration cites the piece of the reference (file:line inside phcool/Layer_Quant) whose
 * job it takes over.  The reference's own boundary is Python (Triton launches); these are the
 * functions a ctypes / cffi / pybind stub binds instead of those launches.
 */
#ifndef LAYER_QUANT_B200_H
#define LAYER_QUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LQ_ABI_VERSION 1

/* status codes */
#define LQ_OK 0
#define LQ_ERR_INVALID_ARGUMENT (-1) /* bad shape / stride / alignment / null pointer            */
#define LQ_ERR_UNSUPPORTED (-2)      /* valid request outside what the sm_100a kernels implement  */
#define LQ_ERR_CUDA (-3)             /* a CUDA runtime call failed (message has the CUDA text)    */
#define LQ_ERR_WORKSPACE (-4)        /* workspace missing or too small                            */
#define LQ_ERR_DEVICE_STATUS (-5)    /* a kernel recorded a bounded-wait time-out                 */

/* element types of floating-point operands */
#define LQ_BF16 0
#define LQ_F16 1
#define LQ_F32 2

/* ------------------------------------------------------------------------------------------ */
/* MX8 / MX4 recurrent state                                                                  */
/* ------------------------------------------------------------------------------------------ */

/* Storage layouts of a state of shape [batch, heads, dim, dstate] (dstate % 16 == 0).
 *   REFERENCE  the tensors of MambaStateKernelCache (mamba_state_8b_kernel.py:19-25):
 *              q int8 [B,H,P,N] (MX4 too, one byte per mantissa), shared_exp u8 [B,H,P,N/16],
 *              micro_exp u8 [B,H,P,N/2] holding 0/1 per pair.  25 bytes per 16-value block.
 *   PACKED     q int8 [B,H,P,N] for MX8, u8 [B,H,P,N/2] two's-complement nibbles for MX4 (value
 *              2j in the low nibble); shared_exp u8 [B,H,P,N/16]; micro_exp u8 [B,H,P,N/16] with
 *              bit i of byte g = pair i of block g.  18 (MX8) / 10 (MX4) bytes per block.      */
#define LQ_MX_LAYOUT_REFERENCE 0
#define LQ_MX_LAYOUT_PACKED 1

/* Rounding of |v| / scale to a mantissa.
 *   HALF_UP         floor(a + 0.5)                      in-kernel deterministic mode (:201,:482,:532)
 *   HALF_EVEN       rint(a)                             torch initial quantiser (:568)
 *   PHILOX_REF      floor(a) + (u < a - floor(a)), u = tl.rand(seed, rng_offset + linear index):
 *                   the reference's stream, one Philox4x32-10 block per value (:196-199,:659)
 *   SUPPLIED        same rule, u derived from caller-supplied 32-bit words (one per value)
 *   PHILOX_LAYERED  library stream keyed on (seed, layer, step, block index): one Philox4x32-10
 *                   block (counter = block index lo/hi, step, layer) per 16-value MX block, value i
 *                   takes byte i & 3 of word i >> 2 as an 8-bit uniform draw r8; fixed-point rule
 *                   q = floor(fl32(v/scale + 49152 + r8/256)) - 49152.  No reference counterpart.
 *   SUPPLIED_FIXED  the fixed-point rule with r8 = low 8 bits of caller-supplied words
 *   PHILOX_LAYERED4 the reference's rule, floor(a) + (u < a - floor(a)) with u mapped from a 32-bit word as
 *                   tl.rand maps it, on the library's keying: one Philox4x32-10 block (counter = quad index
 *                   lo/hi, step, layer) per FOUR values, value i of a quad takes word i.  It separates the two
 *                   things PHILOX_LAYERED changes at once: this mode changes only where the numbers come from
 *                   (all four words, a layer term), PHILOX_LAYERED also the rounding rule.                    */
#define LQ_ROUND_HALF_UP 0
#define LQ_ROUND_HALF_EVEN 1
#define LQ_ROUND_PHILOX_REF 2
#define LQ_ROUND_SUPPLIED 3
#define LQ_ROUND_PHILOX_LAYERED 4
#define LQ_ROUND_SUPPLIED_FIXED 5
#define LQ_ROUND_PHILOX_LAYERED4 6

typedef struct lq_mx_state {
  void* q_state;         /* device; see layouts above                                           */
  uint8_t* shared_exp;   /* device                                                               */
  uint8_t* micro_exp;    /* device                                                               */
  int64_t q_stride[3];     /* batch, head, dim strides; innermost (dstate) stride must be 1      */
  int64_t exp_stride[3];   /* same for shared_exp                                                */
  int64_t micro_stride[3]; /* same for micro_exp                                                 */
  int32_t batch, heads, dim, dstate;
  int32_t format_bits;   /* 8 or 4                                                               */
  int32_t layout;        /* LQ_MX_LAYOUT_*                                                       */
} lq_mx_state;

typedef struct lq_rounding {
  int32_t mode;          /* LQ_ROUND_*                                                           */
  uint32_t layer;        /* PHILOX_LAYERED / PHILOX_LAYERED4 only                                */
  uint64_t seed;         /* Philox key (low word k0, high word k1)                               */
  uint64_t step;         /* PHILOX_LAYERED(4): counter word; PHILOX_REF: unused (see rng_offset) */
  uint64_t rng_offset;   /* PHILOX_REF: RNG_OFFSET = step * numel of the reference (:659, :716)  */
  const uint32_t* words; /* SUPPLIED / SUPPLIED_FIXED: device, one word per value, [B,H,P,N]   */
  const uint64_t* step_counter; /* optional device counter read when the kernel runs: its value is
                            added to `step`, and value * numel(state) to `rng_offset`, so that a
                            launch recorded once (CUDA graph) draws fresh numbers on every replay;
                            advance it with lq_counter_add                                        */
} lq_rounding;

/* One decode step of the Mamba2 selective-state update on an MX-held state, fused:
 * dequantise, dt = softplus(dt + dt_bias), h' = h * exp(A dt) + (B dt) x, y = <h', C> + D x (* z),
 * requantise h' in place.
 * Replaces mx_state_selective_update (mamba_state_8b_kernel.py:601-721) and the kernels it
 * launches: _state_update_requant_mx8_row_kernel (:33-222) for MX8, _state_update_mx8_kernel
 * (:225-443) + _requantize_mx4_kernel (:494-544) for MX4 (no fp32 temporary here).            */
typedef struct lq_mx_update_args {
  lq_mx_state state;
  const void* x;       int64_t x_stride[3];       int32_t x_dtype;   /* [B,H,P]                   */
  const void* dt;      int64_t dt_stride[3];      int32_t dt_dtype;  /* [B,H,P] (stride 0 allowed) */
  const void* dt_bias; int64_t dt_bias_stride[2]; int32_t dt_bias_dtype; /* [H,P] or NULL         */
  const void* A;       int64_t A_stride[3];       int32_t A_dtype;   /* [H,P,N] (stride 0 allowed) */
  const void* B;       int64_t B_stride[3];       int32_t B_dtype;   /* [B,G,N]                   */
  const void* C;       int64_t C_stride[3];       int32_t C_dtype;   /* [B,G,N]                   */
  const void* D;       int64_t D_stride[2];       int32_t D_dtype;   /* [H,P] or NULL             */
  const void* z;       int64_t z_stride[3];       int32_t z_dtype;   /* [B,H,P] or NULL           */
  void* out;           int64_t out_stride[3];     int32_t out_dtype; /* [B,H,P]                   */
  int32_t ngroups;     /* G; heads % G == 0, group = head / (heads / G)                          */
  int32_t dt_softplus; /* 0 / 1                                                                  */
  lq_rounding rounding;
  float* h_out;        /* optional device fp32 [B,H,P,N] dense: the updated state before
                          requantisation (what the reference's MX4 path keeps in tmp_state)      */
} lq_mx_update_args;

int lq_mx_state_update(const lq_mx_update_args* args, void* cuda_stream);

/* Stand-alone codec on a dense fp32 / bf16 / f16 source [rows, dstate] viewed through `state`
 * with batch = heads = 1, dim = rows.
 * Replaces _quantize_initial_state_mx (mamba_state_8b_kernel.py:547-572; HALF_EVEN) and the
 * unused-but-canonical _requantize_mx8_kernel / _requantize_mx4_kernel (:446-544).            */
int lq_mx_quantize(const lq_mx_state* state, const void* src, int32_t src_dtype, int64_t src_row_stride,
                   const lq_rounding* rounding, void* cuda_stream);

/* q * 2^(shared_exp - 127 + micro) -> dense fp32 [rows, dstate] (mamba_state_8b_kernel.py:132). */
int lq_mx_dequantize(const lq_mx_state* state, float* dst, int64_t dst_row_stride, void* cuda_stream);

/* *counter += inc on the stream (one thread); pairs with lq_rounding.step_counter. */
int lq_counter_add(uint64_t* counter, uint64_t inc, void* cuda_stream);

/* Convert between the two storage layouts (same format_bits and shape in both). */
int lq_mx_convert_layout(const lq_mx_state* src, const lq_mx_state* dst, void* cuda_stream);

/* ------------------------------------------------------------------------------------------ */
/* Packed INT4 KV cache                                                                       */
/* ------------------------------------------------------------------------------------------ */

/* One layer's cache, the tensors of Int4KVLayerCache (int4_8b_attention.py:12-18, :423-436):
 * k_packed / v_packed u8 [B, Hkv, capacity, D/2], byte j = code[2j] & 15 | (code[2j+1] & 15) << 4,
 * k_scale / v_scale fp32 [B, Hkv, capacity, D/group_size].                                     */
typedef struct lq_int4_cache {
  uint8_t* k_packed; uint8_t* v_packed; float* k_scale; float* v_scale; /* device                */
  int64_t kp_stride[4]; int64_t vp_stride[4]; int64_t ks_stride[4]; int64_t vs_stride[4];
  int32_t batch, kv_heads, capacity, head_dim, group_size;
} lq_int4_cache;

/* Quantise q_len new K and V rows per (batch, kv head) and scatter them to rows positions[t].
 * k, v: [B, Hkv, q_len, D] with arbitrary strides; positions: device int64 [q_len].
 * Replaces _pack_kv_into_cache / _pack_int4_kv_kernel (int4_8b_attention.py:32-111, :477-515),
 * both launches in one.                                                                        */
int lq_int4_kv_append(const lq_int4_cache* cache, const void* k, const int64_t k_stride[4], const void* v,
                      const int64_t v_stride[4], int32_t dtype, const int64_t* positions, int32_t q_len,
                      void* cuda_stream);

/* q_len = 1 GQA attention over rows [0, seq_len) of the cache, split over the context.
 * q: [B, Hq, D] (stride of the length-1 query axis is irrelevant); mask: optional device fp32
 * additive bias, element (b, n) at mask[b * mask_stride_b + n * mask_stride_k], tokens
 * n >= mask_k_len are masked out; the bias is added to scores already scaled by
 * log2(e)/sqrt(D) (one unit = a factor of two).  out: [B, Hq, D] in `dtype`.
 * splits = 0 lets the library choose; workspace (see lq_int4_decode_workspace_bytes) is needed
 * whenever more than one split is used and must start zeroed once (the kernel restores the
 * zero state of the part it uses as counters before it finishes).
 * Replaces _decode_attention / _int4_decode_attention_kernel (int4_8b_attention.py:254-402,
 * :518-566).                                                                                   */
typedef struct lq_int4_decode_args {
  lq_int4_cache cache;
  const void* q; int64_t q_stride[3]; /* batch, head, d */
  void* out;     int64_t out_stride[3];
  int32_t dtype;        /* of q and out                                                         */
  int32_t q_heads;
  int32_t seq_len;
  const float* mask; int64_t mask_stride_b; int64_t mask_stride_k; int32_t mask_k_len;
  int32_t splits;       /* 0: the library picks; otherwise used as given, capped at the tile count and at 128 */
  void* workspace; size_t workspace_bytes;
  /* Fused append (optional): when k_new != NULL the row seq_len - 1 of every (batch, kv head) is
   * quantised from k_new / v_new [B, Hkv, D] inside the attention kernel, written to the cache
   * and used for this step, i.e. lq_int4_kv_append(q_len = 1) followed by the attention.       */
  const void* k_new; int64_t k_new_stride[3];
  const void* v_new; int64_t v_new_stride[3];
  /* Optional device counter holding the sequence length.  When set, the kernel reads the length
   * when it RUNS, so one recorded launch (CUDA graph) serves every step of a growing context
   * (advance it with lq_counter_add); `seq_len` above then only sizes the launch (split count):
   * pass the current length or the longest the recording will see.  The number of splits is fixed
   * at launch and the tiles are dealt evenly to them on the device.  A counter outside
   * [1, capacity] is clamped and sets bit 1 of lq_device_status.  No reference counterpart: the
   * reference reads the length on the host each step (int4_8b_attention.py:667).               */
  const uint64_t* seq_len_counter;
} lq_int4_decode_args;

int lq_int4_decode_attn(const lq_int4_decode_args* args, void* cuda_stream);

/* Bytes of zero-initialised scratch lq_int4_decode_attn needs for up to max_splits splits: a fixed
 * 256 KiB of ticket counters (kept zero by the kernel) followed by the per-split partial results.
 * A buffer may be reused for any problem it is large enough for.                               */
size_t lq_int4_decode_workspace_bytes(int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                                      int32_t max_splits);
/* The split count the library would pick for this problem on the current device (>= 1). */
int32_t lq_int4_decode_auto_splits(int32_t batch, int32_t kv_heads, int32_t seq_len);

/* Causal attention of q_len consecutive query positions over the packed cache, which already holds
 * their own K / V rows (lq_int4_kv_append first): query i of a sequence attends rows
 * [0, first_len + i).  This is what the reference's _int4_prefill_attention_kernel computes
 * (int4_8b_attention.py:114-251, first_len = 1: a prompt from position 0), a kernel the reference
 * defines but never calls; its live prefill path attends the un-quantised K / V (:693-714).
 * first_len > 1 serves chunked prefill behind an existing context.  Group sizes 32 / 64 / 128.  */
typedef struct lq_int4_prefill_args {
  lq_int4_cache cache;
  const void* q; int64_t q_stride[4];   /* [B, Hq, Tq, D]: batch, head, position, d */
  void* out;     int64_t out_stride[4]; /* [B, Hq, Tq, D]                            */
  int32_t dtype;        /* of q and out */
  int32_t q_heads;
  int32_t q_len;
  int32_t first_len;    /* rows the first query position sees, its own included (>= 1) */
} lq_int4_prefill_args;

int lq_int4_prefill_attn(const lq_int4_prefill_args* args, void* cuda_stream);

/* lq_int4_decode_attn for callers that cannot hand over scratch memory of their own: a process
 * whose memory pool has already taken all of the device memory (a cudaMalloc would fail), or a
 * latency-critical thread that must not take the device-wide lock an allocation takes.  Same
 * arguments and results as lq_int4_decode_attn, except that args->workspace / workspace_bytes are
 * ignored: the split-merge scratch is an array built into the library image
 * (lq_int4_static_scratch_bytes() bytes, about 4.4 MB, held by every GPU that loads the library
 * until the process exits).  This entry point has no counterpart in the reference.
 *   - Limit: batch * q_heads * splits <= LQ_INT4_STATIC_MAX_SLOTS.  With splits = 0 the library
 *     picks a split count inside the limit; an explicit splits is first capped like
 *     lq_int4_decode_attn caps it (at the number of 64-token tiles and at 128) and refused with
 *     LQ_ERR_WORKSPACE if it is still beyond the limit.  One split needs no scratch and is
 *     always accepted.
 *   - It allocates nothing (no cudaMalloc / cudaFree / allocating library call).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *     with that device current); make that first call before any stream capture begins.  The
 *     array gets its device memory when the CUDA runtime loads the library's code onto that
 *     device, which with lazy loading happens at that first call (or at the first launch of any
 *     kernel of this library): make it before a memory pool takes what is left of the device
 *     memory, or the load itself fails.
 *   - All calls on a device share the one array, which still holds the previous call's contents;
 *     the ticket counters are cleared on the stream before each launch.  Two calls that may overlap
 *     on the GPU (different streams) race on it: serialise them, or use lq_int4_decode_attn with
 *     one workspace per stream.                                                                 */
#define LQ_INT4_STATIC_MAX_SLOTS 8192
int lq_int4_decode_attn_static(const lq_int4_decode_args* args, void* cuda_stream);
size_t lq_int4_static_scratch_bytes(void);

/* ------------------------------------------------------------------------------------------ */
/* Library                                                                                    */
/* ------------------------------------------------------------------------------------------ */
int lq_abi_version(void);
/* ---- Unquantised baselines: the step before the hot path and the state format it is compared with ----
 *
 * The reference takes both from third-party packages that are not part of its tree: the patched
 * global `selective_state_update` it falls back to (mamba_state_8b_kernel.py:743-761) is
 * mamba_ssm.ops.triton.selective_state_update, and the conv step before it is
 * causal_conv1d.causal_conv1d_update.  These two entry points restate their published behaviour. */

/* One decode step of the selective-state update on a dense state [B,H,P,N] (bf16 / f16 / f32, N
 * contiguous), in place, fp32 math: dt = softplus(dt + dt_bias), h' = h exp(A dt) + (B dt) x stored
 * rounded to the state's type, y = <h', C> + D x taken from the fp32 h'; with z the read-out is gated
 * as that package does it, y * z * sigmoid(z) (lq_mx_state_update multiplies by z alone, as the
 * reference's MX kernels do, mamba_state_8b_kernel.py:163-165).  Operands as in lq_mx_update_args. */
typedef struct lq_dense_update_args {
  void* state;         int64_t state_stride[4];   int32_t state_dtype; /* [B,H,P,N]               */
  int32_t batch, heads, dim, dstate;
  const void* x;       int64_t x_stride[3];       int32_t x_dtype;
  const void* dt;      int64_t dt_stride[3];      int32_t dt_dtype;
  const void* dt_bias; int64_t dt_bias_stride[2]; int32_t dt_bias_dtype;
  const void* A;       int64_t A_stride[3];       int32_t A_dtype;
  const void* B;       int64_t B_stride[3];       int32_t B_dtype;
  const void* C;       int64_t C_stride[3];       int32_t C_dtype;
  const void* D;       int64_t D_stride[2];       int32_t D_dtype;
  const void* z;       int64_t z_stride[3];       int32_t z_dtype;
  void* out;           int64_t out_stride[3];     int32_t out_dtype;
  int32_t ngroups;
  int32_t dt_softplus;
} lq_dense_update_args;

int lq_dense_state_update(const lq_dense_update_args* args, void* cuda_stream);

/* One decode step of the depthwise causal convolution: every channel's window conv_state[b,c,:]
 * moves one place to the left, x[b,c] enters at the end, out[b,c] = sum_w window[w] weight[c,w]
 * (+ bias[c]), through SiLU when `silu` is set.  fp32 math, the window stored back in its type. */
typedef struct lq_conv1d_update_args {
  void* conv_state;   int64_t state_stride[3]; int32_t state_dtype;  /* [B,C,W], W <= 8           */
  const void* x;      int64_t x_stride[2];     int32_t x_dtype;      /* [B,C]                     */
  const void* weight; int64_t weight_stride[2]; int32_t weight_dtype; /* [C,W]                    */
  const void* bias;   int64_t bias_stride[1];  int32_t bias_dtype;   /* [C] or NULL               */
  void* out;          int64_t out_stride[2];   int32_t out_dtype;    /* [B,C]                     */
  int32_t batch, channels, width;
  int32_t silu;
} lq_conv1d_update_args;

int lq_causal_conv1d_update(const lq_conv1d_update_args* args, void* cuda_stream);

/* sizeof of an ABI struct as the library was compiled: 0 lq_mx_state, 1 lq_rounding,
 * 2 lq_mx_update_args, 3 lq_int4_cache, 4 lq_int4_decode_args, 5 lq_dense_update_args,
 * 6 lq_conv1d_update_args, 7 lq_int4_prefill_args; -1 otherwise. */
int lq_abi_sizeof(int which);
const char* lq_last_error_string(void);
/* Reads (and clears) the device-side status word of the current device: 0, or a bit set: bit 0 a
 * bounded wait of a kernel ran out, bit 1 a seq_len_counter held a length outside [1, capacity]
 * (the kernel clamped it).  Synchronises the device. */
int lq_device_status(int32_t* status);

#ifdef __cplusplus
}
#endif
#endif /* LAYER_QUANT_B200_H */
