/*
 * C ABI of libovc.so: FP8 ExpCast forward attention for NVIDIA B200 (sm_100a).
 *
 * The reference project (open-vc-attn 0.3.0) is pure Python and has no FFI of its
 * own; its device work is reached through Python functions that JIT-compile
 * Triton and CuTe-DSL kernels.  Each entry point below replaces one of those
 * device stages and is what a Python/ctypes (or any other FFI) binding of the
 * path would call.  Citations are paths inside the reference project.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless stated otherwise; the caller owns
 *     all memory.  No entry point allocates, frees or synchronises.  The entry
 *     points that replace a stage of the reference stay capturable in a CUDA
 *     graph, as that stage is (tested through the Python layer).
 *   - Work is enqueued on `stream` (a cudaStream_t passed as void*) of the
 *     device that is current in the calling thread.
 *   - `dtype`: OVC_F16 or OVC_BF16, the element type of the 16-bit inputs.
 *   - FP8 means E4M3 (float8_e4m3fn), one byte per element.
 *   - Return value: OVC_OK (0) or a negative OVC_ERR_* code.  Nothing throws.
 *     ovc_error_string() maps a code to text; ovc_last_cuda_error() returns the
 *     cudaError_t / CUresult seen by the failing call, if any.
 *   - Tensors are dense row-major with the shapes given; D is always 128.
 */
#ifndef OVC_H
#define OVC_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OVC_F16 0
#define OVC_BF16 1

#define OVC_OK 0
#define OVC_ERR_ARGUMENT (-1)    /* null pointer, bad size, bad alignment, unknown dtype */
#define OVC_ERR_CUDA (-2)        /* a CUDA runtime call failed; see ovc_last_cuda_error() */
#define OVC_ERR_DRIVER (-3)      /* tensor-map creation failed */
#define OVC_ERR_UNSUPPORTED (-4) /* device is not sm_100 */
#define OVC_ERR_TOO_LARGE (-5)   /* a size exceeds what the library's built-in scratch memory can hold */

/* Bits of the device status word written by ovc_attention (0 = clean run). */
/* flags of ovc_attention_ex */
#define OVC_ATTN_CAUSAL 1     /* bottom-right aligned causal mask */
#define OVC_ATTN_V_UNPACKED 2 /* v is [B,Sk,H,128] FP8 (the layout of the quantisers' output), not the packed one */

#define OVC_STATUS_WAIT_EXPIRED 1u /* a bounded barrier wait gave up; the output rows of that launch hold NaN */

int ovc_version(void);
const char* ovc_error_string(int code);
int ovc_last_cuda_error(void);

/*
 * Per-(batch, head, 128-token block) FP8 quantisation of Q or K.
 * Replaces _per_block_quant_kernel / fp8_quantize_per_block_triton
 * (src/open_vc_attn/quantization.py:153-220).
 *   x        [B,S,H,128] f16/bf16
 *   codes    [B,S,H,128] fp8
 *   descale  [B,H,descale_stride] f32, first ceil(S/128) entries of each row written;
 *            when descale_stride > ceil(S/128) the entry at ceil(S/128) is set to 1.0
 *            (the even-count padding of src/open_vc_attn/preparation.py:47-49).
 */
int ovc_quantize_per_block(const void* x, int dtype, int64_t B, int64_t S, int64_t H, void* codes,
                           float* descale, int64_t descale_stride, void* stream);

/*
 * Per-(batch, head) max |v|.  Replaces the zero fill plus _per_head_amax_kernel
 * (src/open_vc_attn/quantization.py:22-53,121-134).  amax [B,H] f32 is reset and then reduced into.
 */
int ovc_head_amax(const void* v, int dtype, int64_t B, int64_t S, int64_t H, float* amax, void* stream);

/*
 * V cast with the per-(batch, head) scale 448/max(amax,1e-12); descale = max(amax,1e-12)/448.
 * Replaces _per_head_scale_cast_kernel and the host division
 * (src/open_vc_attn/quantization.py:56-93,144).
 *   codes [B,S,H,128] fp8, descale [B,H] f32.
 */
int ovc_quantize_per_head(const void* v, int dtype, int64_t B, int64_t S, int64_t H, const float* amax,
                          void* codes, float* descale, void* stream);

/*
 * Fused preparation of one sequence for the packed path.  Replaces prepare_fp8_fused's three
 * launches _quantize_qk, _per_head_amax_kernel, _cast_pack_v (src/open_vc_attn/preparation.py:83-162).
 *   q,k,v      [S,H,128] f16/bf16
 *   q8,k8      [S,H,128] fp8
 *   v_packed   [H,128,S_pad] fp8, S_pad = ceil(S/128)*128; columns S..S_pad-1 are written as zero
 *   q_descale  [H,q_blocks] f32, q_blocks = ceil(S/128) rounded up to even (padding entry = 1.0)
 *   k_descale  [H,ceil(S/128)] f32
 *   v_descale  [H] f32
 *   amax_ws    [H] f32 scratch (holds the per-head max |v| afterwards)
 */
int ovc_prepare_fused(const void* q, const void* k, const void* v, int dtype, int64_t S, int64_t H,
                      void* q8, void* k8, void* v_packed, float* q_descale, float* k_descale,
                      float* v_descale, float* amax_ws, void* stream);

/*
 * ovc_prepare_fused without the caller-provided scratch buffer.  (No counterpart in the reference; it
 * exists for this library's callers only.)
 *
 * Some hosts of this code cannot hand over even a few bytes of extra device memory per call: an
 * inference server whose memory pool was sized up front and already owns the whole GPU, a plugin that
 * is given input and output buffers and nothing else, or any caller that must not reach cudaMalloc on
 * its hot path.  For them the per-head max |v| scratch lives inside the library, in a fixed array of
 * OVC_STATIC_MAX_HEADS (4096) floats that every GPU loading libovc.so holds until the process ends.
 * The call allocates and frees nothing, on the device or through any library.
 *
 *   - H > 4096 is refused with OVC_ERR_TOO_LARGE; all other arguments as for ovc_prepare_fused.
 *   - The first call on each device looks up the array's device address (with that device current).
 *     Make that first call ahead of any stream capture.
 *   - All calls on a device share the one array.  Each call resets the entries it uses before
 *     accumulating, so back-to-back calls on one stream are independent; calls whose kernels overlap
 *     on the GPU (different streams, no ordering) race on it and must not be issued.
 *   - Results are bit-identical to ovc_prepare_fused.
 */
int ovc_prepare_fused_static(const void* q, const void* k, const void* v, int dtype, int64_t S, int64_t H,
                             void* q8, void* k8, void* v_packed, float* q_descale, float* k_descale,
                             float* v_descale, void* stream);

/*
 * FP8 byte transpose into the packed V layout.  Replaces transpose_v / pack_v
 * (src/open_vc_attn/_kernels/blackwell/flash_attn/cute/v_layout.py:8-49).
 *   codes [B,S,H,128] fp8 -> packed [B,H,128,S_pad] fp8 with a zero tail.
 */
int ovc_pack_v(const void* codes, int64_t B, int64_t S, int64_t H, void* packed, void* stream);

/*
 * q[i] = a[i] / b[i] with the division instruction the preparation kernels use (div.full.f32: the
 * dividend times the hardware's approximate reciprocal, which is what Triton emits for the `/` in
 * src/open_vc_attn/quantization.py:183-184, preparation.py:43-46,79 and v_repair.py:69-70,111).
 * For callers and tests that need the exact scales on the host; a, b, q: n floats in device memory.
 */
int ovc_div_full(const float* a, const float* b, float* q, int64_t n, void* stream);

/*
 * V cast plus per-token squared rounding residual.  Replaces _v_quant_score_kernel
 * (src/open_vc_attn/v_repair.py:52-76).
 *   v [S,H,128] f16/bf16, amax [H] f32 -> codes [S,H,128] fp8, score [H,S] f32.
 */
int ovc_repair_score(const void* v, int dtype, int64_t S, int64_t H, const float* amax, void* codes,
                     float* score, void* stream);

/*
 * Builds the repair prefix.  Replaces _repair_rows_kernel (src/open_vc_attn/v_repair.py:79-113).
 *   k_all,v_all [rows+S,H,128] fp8: rows [rows, rows+S) hold the original codes on entry; rows
 *               [0, rows) are written (key copies; V residual codes, zero for pad rows >= selected)
 *   v_src       [S,H,128] f16/bf16 original V
 *   k_descale   [H,k_blocks] f32, v_descale [H] f32
 *   index       [H,selected] int32 source token of each repair row
 *   repair_kd   [H,rows] f32 out: the source token's K descale
 */
int ovc_repair_rows(void* k_all, void* v_all, const void* v_src, int dtype, const float* k_descale,
                    const float* v_descale, const int32_t* index, float* repair_kd, int64_t selected,
                    int64_t rows, int64_t S, int64_t H, int64_t k_blocks, void* stream);

/*
 * FP8 ExpCast forward attention.  Replaces the compiled FlashAttentionForwardSm100 kernel behind
 * _flash_attn_fwd (src/open_vc_attn/_kernels/blackwell/flash_attn/cute/interface.py:110-179,
 * cute/flash_fwd_sm100.py:1438) for non-causal MHA, D = 128, with per-block Q/K and per-head V descales.
 *   q8          [B,Sq,H,128] fp8
 *   k8          [B,Sk,H,128] fp8 (Sk includes the repair prefix when repair_rows > 0)
 *   v_packed    [B,H,128,Sk_pad] fp8, Sk_pad = ceil(Sk/128)*128
 *   q_descale   [B,H,q_blocks] f32 with q_blocks >= ceil(Sq/128)
 *   k_descale   [B,H,ceil(Sk/128)] f32
 *   v_descale   [B,H] f32
 *   repair_kd   [H,repair_rows] f32 or NULL; repair_rows is a multiple of 128, < Sk, and needs B == 1
 *   out         [B,Sq,H,128] bf16
 *   softmax_scale   > 0 and finite
 *   mid_window_blocks  >= 0: start the key scan that many 128-key blocks right of the diagonal;
 *                      -1: plain right-to-left scan
 *   status      two uint32 in device memory, or NULL.  Every wait inside the kernel is bounded (about
 *               0.2 s).  A CTA whose wait expires ORs OVC_STATUS_* bits into both words, fills the output
 *               rows it owns with NaN (-inf in lse) and exits; CTAs of the same launch that start
 *               afterwards do the same without computing.  status[0] is this launch's word: the entry
 *               point clears it (stream-ordered) before the launch, so an expiry never leaks into later
 *               calls.  status[1] is sticky: the library only ever sets bits in it, the caller reads and
 *               clears it when it wants to know whether any launch since the last look gave up.
 */
int ovc_attention(const void* q8, const void* k8, const void* v_packed, const float* q_descale,
                  int64_t q_blocks, const float* k_descale, const float* v_descale, const float* repair_kd,
                  int64_t repair_rows, void* out, int64_t B, int64_t Sq, int64_t Sk, int64_t H,
                  float softmax_scale, int mid_window_blocks, uint32_t* status, void* stream);

/*
 * Measurement aid: runs the attention kernel's score conversion alone (tcgen05.ld of 128 scores, row max,
 * ExpCast codes, tcgen05.st) in `ctas` CTAs of 8 conversion warps, `tiles` key tiles each, on scores held in
 * tensor memory.  Timed by the caller, ctas * 256 * 128 * tiles scores per launch give the rate the CUDA cores
 * sustain without exp instructions: the denominator of the MUFU-free ExpCast roofline.  `sink`: one uint32 in
 * device memory (never written in practice).  No counterpart in the reference.
 */
int ovc_bench_conversion(uint32_t* sink, int64_t ctas, int64_t tiles, void* stream);

/*
 * Runs the kernels' bounded barrier wait on its own: one 64-thread CTA waits at most `limit_cycles` clock
 * ticks on a barrier that cannot complete, then sets OVC_STATUS_WAIT_EXPIRED in status[0] and status[1] (the
 * two words ovc_attention takes) and adds the number of threads that gave up to *gave_up (device memory).  No tensor-core work or copy is in flight, the
 * context stays usable.  For tests of the failure path; has no counterpart in the reference, whose waits are
 * unbounded (cute/blackwell_helpers.py:538-545).
 */
int ovc_selftest_wait(uint32_t* status, int64_t limit_cycles, uint32_t* gave_up, void* stream);

/*
 * Copies `heads` consecutive heads of a [S, src_heads, bytes_per_head] tensor into a
 * [S, dst_heads, bytes_per_head] tensor (one strided 2-D copy on `stream`), host to device when
 * to_device is non-zero, else device to host; the host side should be pinned memory for the copy to be
 * asynchronous.  Has no counterpart in the reference, whose callers keep Q, K, V on the device: it lets a
 * caller with host-resident tensors stream head groups through the GPU (heads are independent on this path),
 * overlapping the copies with the kernels of the previous group.
 */
int ovc_copy_head_slice(void* dst, int64_t dst_heads, int64_t dst_first, const void* src, int64_t src_heads,
                        int64_t src_first, int64_t heads, int64_t S, int64_t bytes_per_head, int to_device, void* stream);

/*
 * ovc_attention with the two options of _flash_attn_fwd that the default call does not use
 * (cute/interface.py:122,139-143):
 *   lse     [B,H,Sq] f32 or NULL: log-sum-exp of the scaled scores of every query row,
 *           (m * sigma + log2(l) - 8) * ln 2 with m the row maximum of the descaled scores,
 *           sigma = softmax_scale * log2(e) * q_descale and l the denominator; -inf for a row whose l is 0 or NaN
 *           (cute/flash_fwd_sm100.py:4437-4475).
 *   flags   OVC_ATTN_CAUSAL: key column c is visible to query row r iff c < r + 1 + Sk - Sq
 *           (cute/mask.py:186-199); tiles wholly above the diagonal are skipped.  Needs mid_window_blocks = -1 and
 *           no repair prefix.
 *           OVC_ATTN_V_UNPACKED: `v_packed` points to V codes in the [B,Sk,H,128] layout instead, which the
 *           kernel reads as the MN-major operand of P V (cute/flash_fwd_sm100.py:726-729,767-770: the reference's
 *           general path does the same), so no packing pass is needed; not with a repair prefix.
 */
int ovc_attention_ex(const void* q8, const void* k8, const void* v_packed, const float* q_descale,
                     int64_t q_blocks, const float* k_descale, const float* v_descale, const float* repair_kd,
                     int64_t repair_rows, void* out, float* lse, int flags, int64_t B, int64_t Sq, int64_t Sk,
                     int64_t H, float softmax_scale, int mid_window_blocks, uint32_t* status, void* stream);

/* ---- VC-Attention baseline: V-Smooth preparation and the mean-restoring attention variant ----
 *
 * Replaces the Triton kernels and launches of src/open_vc_attn/_kernels/blackwell/v_smooth.py and the
 * v_smooth=True specialisation of the attention kernel (cute/flash_fwd_sm100.py:140, 3895-3901,
 * 4111-4262).  One sequence; Q, K, V bf16 [S,H,128] read in place (no head-major copy).
 */

/*
 * labels[h][s] = argmin_k (|c_k|^2 - 2 v_s.c_k), first index on ties (_assign_values, v_smooth.py:10-39).
 *   v [S,H,128] bf16, centers [H,K,128] bf16, labels [H,S] int32 out; 1 <= K <= min(128, S).
 * The products are BF16 x BF16 -> FP32 tensor-core MMAs, as in the reference; the accumulation order of
 * such a product is not specified on either side, so near-tied tokens may be labelled differently.
 */
int ovc_vs_assign(const void* v, const void* centers, int32_t* labels, int64_t S, int64_t H, int64_t K, void* stream);

/*
 * Per-cluster float32 sums [H,K,128] and counts [H,K] of V rows; both outputs are cleared first
 * (_accumulate_centers, v_smooth.py:42-73, with the torch.zeros of :262-267).
 */
int ovc_vs_accumulate(const void* v, const int32_t* labels, float* sums, float* counts, int64_t S, int64_t H, int64_t K,
                      void* stream);

/* centers = count > 0 ? bf16(sum / count) : centers   (the torch.where of v_smooth.py:281-285). */
int ovc_vs_update_centers(const float* sums, const float* counts, void* centers, int64_t H, int64_t K, void* stream);

/*
 * Block means of V in group order and the per-channel maximum of |v - mean| (_block_stats, v_smooth.py:76-94).
 *   permutation [H,S] int64; means [H,ceil(S/128),128] f32 out; amax [H,128] f32 out (cleared first).
 * A channel's sum over a block is taken in float32 in a fixed order: rows g + 16 i in ascending i into
 * sixteen partial sums, then the partial sums in ascending g; rows past the end of the sequence count as 0.
 */
int ovc_vs_block_stats(const void* v, const int64_t* permutation, float* means, float* amax, int64_t S, int64_t H,
                       void* stream);

/*
 * Permuted FP8 K, FP8 V residual codes, block means in code units and channel scales
 * (_block_write, v_smooth.py:97-134).
 *   k_out, codes [S,H,128] fp8; means_out [ceil(S/128),H,128] f32 (BF16-rounded values); scale [H,128] f32.
 */
int ovc_vs_block_write(const void* k, const void* v, const int64_t* permutation, const float* means, const float* amax,
                       void* k_out, void* codes, float* means_out, float* scale, int64_t S, int64_t H, void* stream);

/*
 * Unscaled saturating cast of f16/bf16 to FP8 (q.to(float8_e4m3fn) in v_smooth.py:161; values beyond the
 * FP8 range saturate to +-448 here, where torch's cast gives NaN).  elements is a multiple of 8.
 */
int ovc_cast_e4m3(const void* x, int dtype, void* out, int64_t elements, void* stream);

/*
 * ExpCast attention with V-Smooth restoration: as ovc_attention with B = 1, no descales and no repair
 * prefix, and out = (P~ V_codes + sum over key blocks (row sum of P~ in the block) * means[block]) * scale
 * / (row sum of P~).
 *   v_packed      [H,128,Sk_pad] fp8 residual codes (ovc_pack_v of the codes)
 *   unit_descale  f32, at least H * ceil(max(Sq,Sk)/128) values, all 1.0
 *   means         [ceil(Sk/128),H,128] f32; channel_scale [H,128] f32
 *   workspace     device scratch of ovc_attention_vsmooth_workspace(Sk, H) bytes, 16-byte aligned; the call
 *                 fills it (the means as BF16 high and low parts in the layout its tensor-core products read)
 *                 and it may be reused or freed once the stream has passed the call
 * The restoration runs on the tensor core as in the reference (cute/flash_fwd_sm100.py:4482-4526): the masses
 * of sixteen key blocks at a time times their means, masses and means each split into two BF16 terms.
 */
int64_t ovc_attention_vsmooth_workspace(int64_t Sk, int64_t H);
int ovc_attention_vsmooth(const void* q8, const void* k8, const void* v_packed, const float* unit_descale,
                          const float* means, const float* channel_scale, void* workspace, void* out, int64_t Sq,
                          int64_t Sk, int64_t H, float softmax_scale, int mid_window_blocks, uint32_t* status,
                          void* stream);

#ifdef __cplusplus
}
#endif
#endif /* OVC_H */
