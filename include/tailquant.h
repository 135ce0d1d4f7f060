/* tailquant.h -- C ABI of libtailquant.so: the split W4A4 + tail linear on B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (`cudaStream_t` passed as void*; NULL = the legacy default stream), enqueues its work on
 * that stream and returns immediately.  Return value: 0 on success, a negative TQ_ERR_*
 * code otherwise (tq_error_string() gives text, tq_last_cuda_error() the CUDA runtime
 * message of the last failed launch on the calling thread).  No entry point allocates
 * device memory: the caller owns every buffer, as in the reference's extensions
 * ("all pre-allocated, written in place").
 *
 * "Reference" citations name files of Smilesky18/tailquant-kernel by their path in that
 * project.
 */
#ifndef TAILQUANT_H_
#define TAILQUANT_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TQ_OK 0
#define TQ_ERR_BAD_ARG (-1)       /* null pointer, non-positive size, R >= K, ...             */
#define TQ_ERR_UNSUPPORTED (-2)   /* K / rotation kind / R outside the compiled set          */
#define TQ_ERR_MISALIGNED (-3)    /* a pointer that must be 16-byte aligned is not           */
#define TQ_ERR_CUDA (-4)          /* a CUDA runtime / driver call failed                     */
#define TQ_ERR_DEVICE_STATUS (-5) /* a bounded device-side wait ran out (see tq_gemm_status) */
#define TQ_ERR_TOO_LARGE (-6)     /* beyond a stated maximum (no-allocation entry point)     */

/* Rotation applied to the last dimension before quantisation. */
#define TQ_HAD_NONE 0     /* input is already rotated                                       */
#define TQ_HAD_WHT 1      /* K = 2^n, 512..8192 : normalised Walsh-Hadamard                 */
#define TQ_HAD_KRON12 2   /* K = 12*2^n (6144, 12288): (H12 (x) H_2^n)/sqrt(K), H12 = Paley */
#define TQ_HAD_BLOCK128 3 /* K % 2048 == 0 (e.g. 14336): block-diagonal H128/sqrt(128)      */

/* Entries per (row, 64-wide half of a K slice) held by the tail records (a record is 48 bytes: three 128-bit
 * loads); longer runs are completed from the sorted lists. */
#define TQ_TAIL_REC_CAP 12

/* 16-bit float formats of activation inputs / outputs. */
#define TQ_BF16 0
#define TQ_FP16 1

int tq_version(void);
const char* tq_error_string(int code);
const char* tq_last_cuda_error(void);

/* ---------------------------------------------------------------------------------------
 * Prologue: rotation + per-token INT4 quantisation + top-R tail split, one kernel.
 *
 * Replaces, in the reference: the online rotation `RealPolicyLinear._rotate` (call sites
 * tools/bench_hadamard_three_schemes_quarot_dense_sharedqkv_inplace_fusedtopr_v43.py:482),
 * the select+pack kernels tools/fused_topr_pack_ext_v55.py:32-151 and
 * tools/fused_threshold_topr_pack_ext_v57.py:48-269, and for R == 0 the pure per-token
 * pack `pack_a_full_s4` (call site ...fusedtopr_v43.py:260).
 *
 *   x            [M,K] bf16, row-major, 16-byte aligned
 *   had_kind     TQ_HAD_*
 *   R            tail entries per row, 0 <= R < K (0 = pure per-token INT4)
 *   descending_rank  1-based rank (in |x| descending order, ties by lowest index) whose
 *                magnitude sets the body scale; R+1 = absmax of the body
 *   a_pack       [M,K/2] u8 : element 2i -> low nibble, 2i+1 -> high nibble; tail positions 0
 *                (may be NULL when a_q8 is given)
 *   a_q8         [M,K] i8 : the same codes, one per byte, the even elements of every 8-group
 *                first and then the odd ones -- the operand format of tq_split_gemm_mma (may be NULL)
 *   body_scale   [M] f32 = max(|x|_(rank), eps) / 7
 *   top_scale    [M] f32 = max(|x|_max, eps) / 7                     (may be NULL)
 *   tail_idx16   [M,tail_ld] u16 ascending channel indices, R per row (tail mode T16; may be NULL)
 *   tail_val     [M,tail_ld] bf16 rotated values at those indices    (T16; may be NULL)
 *   tail_ld      row pitch (elements) of tail_idx16 / tail_val, >= R; idx32 / top_q are dense [M,R]
 *   tail_ptr     [M,ptr_ld] u16, ptr_ld >= K/128 + 1: tail_ptr[m][j] = number of tail entries of row m
 *                with index < 128 j (run boundaries for tq_split_gemm_mma; K % 128 == 0; may be NULL)
 *   tail_rec     [2 ceil(M/256)][K/64][128][TQ_TAIL_REC_CAP] u32: the same entries regrouped per 128-row
 *                tile and 64-wide half of a K slice, one record of TQ_TAIL_REC_CAP consecutive words per row (the
 *                first min(count, TQ_TAIL_REC_CAP) entries of that half, ascending; the other words are not
 *                written) -- what tq_split_gemm_mma reads, three 128-bit loads per row and half.  Entry = bf16
 *                bits << 16 | p, where p = ((((index & 63) >> 3) ^ (m & 7)) << 3) | (index & 7) is half the byte
 *                offset of the value in its 128-byte row of the 128-byte-swizzled operand tile (may be NULL)
 *   tail_cnt     [2 ceil(M/256)][K/64][128] u16 entries per (row, half slice) (with tail_rec); the rows that
 *                pad M to a multiple of 256 are written as 0 (both arrays cover them: the CTA-pair GEMM
 *                works on 256-row tiles and does not check rows)
 *   tail_dense   [M,K] bf16: the rotated row with every element outside the tail set to zero, written when
 *                R > 0 -- tq_split_gemm_mma loads 32 x 64 blocks of it as operand rows where a row has more
 *                than TQ_TAIL_REC_CAP entries in a half slice (block-diagonal rotations with outlier channels
 *                concentrate the tail in a few 128-blocks); may be NULL
 *   idx32        [M,R] i32 the same indices                          (T4; may be NULL)
 *   top_q        [M,R] i8  clamp(rint(x / top_scale), -8, 7)         (T4; may be NULL)
 *   x_rot        [M,K] bf16 rotated activations                      (debug / weight prep; may be NULL)
 */
int tq_split_prologue(const void* x, int M, int K, int had_kind, int R, int descending_rank, float eps,
                      uint8_t* a_pack, int8_t* a_q8, float* body_scale, float* top_scale,
                      uint16_t* tail_idx16, void* tail_val, int tail_ld, uint16_t* tail_ptr, int ptr_ld,
                      uint32_t* tail_rec, uint16_t* tail_cnt, void* tail_dense, int32_t* idx32, int8_t* top_q,
                      void* x_rot, void* stream);

/* The same prologue with an RMSNorm fused in front of the rotation (the reference runs the norm as a separate
 * PyTorch module before the linear: tools/bench_layer_async_schedule_v22.py:237,249 -- `layer.input_layernorm`,
 * `layer.post_attention_layernorm`; x is the un-normalised hidden state, gamma the [K] bf16 norm weight):
 *   x_n[m,k] = bf16( bf16( x[m,k] / sqrt(mean_k(x[m,:]^2) + rms_eps) ) * gamma[k] ),
 * the squares summed in fp32 in a fixed order (K = 4096, 12288, 14336: thread t of K/64 adds its 64 consecutive
 * elements in index order; other K: thread t of 256 adds 16-element chunks t, t + 256, ...; then a butterfly over the
 * 32 threads of a warp and the warp sums in order), then everything as in tq_split_prologue on x_n.  No [M,K] normalised tensor is
 * written.  (T4 outputs idx32 / top_q are not offered here.) */
int tq_split_prologue_rmsnorm(const void* x, const void* gamma, float rms_eps, int M, int K, int had_kind, int R,
                              int descending_rank, float eps, uint8_t* a_pack, int8_t* a_q8, float* body_scale,
                              float* top_scale, uint16_t* tail_idx16, void* tail_val, int tail_ld,
                              uint16_t* tail_ptr, int ptr_ld, uint32_t* tail_rec, uint16_t* tail_cnt,
                              void* tail_dense, void* x_rot, void* stream);

/* Reference-signature select+pack on an already rotated matrix (T4 outputs):
 * fused_topr_pack(A, R, descending_rank, A_pack, body_scale, top_scale, top_q, idx, eps)
 *   tools/fused_topr_pack_ext_v55.py:112-121
 * threshold_topr_pack(<same>)
 *   tools/fused_threshold_topr_pack_ext_v57.py:236-245
 * Both names map here; indices are written in ascending order. `dtype` is TQ_BF16, or TQ_FP16 (the reference's
 * input type: the same select on the 15-bit magnitude of the half, tools/fused_threshold_topr_pack_ext_v57.py:32-35)
 * for K = 4096 and 12288, the widths the reference builds (same file :258-259). */
int tq_topr_pack(const void* A, int dtype, int M, int K, int R, int descending_rank,
                 uint8_t* A_pack, float* body_scale, float* top_scale, int8_t* top_q, int32_t* idx,
                 float eps, void* stream);

/* ---------------------------------------------------------------------------------------
 * Offline weight preparation.  Replaces the external `pack_weight_colmajor_s4` /
 * `pack_weight_rowmajor_s4_from_scale` (call sites
 * tools/bench_v61_dense_sparse_matrix_breakdown_v1.py:124-131), the RTN scale
 * tools/bench_multimodel_all_layers_policy_fastqf_v29.py:245-247 and the offline rotation
 * tools/bench_real_split_fullstack_rtn_ppl_v1.py:92-110.
 *
 *   w        [N,K] bf16 (nn.Linear.weight layout)
 *   b_col    [N,K/2] u8  INT4 codes, K-contiguous per output channel
 *   w_scale  [N] f32 = max(amax|w_rot| / 7, eps)
 *   w_rot    [N,K] bf16 rotated weight (may be NULL when w_t is NULL)
 *   b_row    [K,N/2] u8  INT4 codes, low nibble = even n          (T4 tail; may be NULL)
 *   w_t      [K,N] bf16 rotated weight, input-channel major: row k is what a tail entry with
 *            index k multiplies                                   (T16 tail; may be NULL)
 */
int tq_prepare_weight(const void* w, int N, int K, int had_kind, float eps,
                      uint8_t* b_col, float* w_scale, void* w_rot, uint8_t* b_row, void* w_t,
                      void* stream);

/* ---------------------------------------------------------------------------------------
 * Dense INT4 x INT4 GEMM on tcgen05 (kind::i8, int32 accumulators in tensor memory).
 * K % 128 == 0; a_pack and b_col 16-byte aligned.
 *
 * tq_int4_matmul replaces `qext.matmul(A_pack[M,K/2], B_col[N,K/2]) -> int32 [M,N]`
 * (call site tools/bench_hadamard_three_schemes_quarot_dense_sharedqkv_inplace_fusedtopr_v43.py:235-239)
 * and `main_ext.cutlass_s4_gemm` (tools/bench_standalone_int4_vs_torch_gemm_v12.py:149-157).
 * split_k > 1 splits the reduction over that many CTAs per tile and accumulates with int32
 * atomics: C must then be zero on entry (the small-M decode path).
 */
int tq_int4_matmul(const uint8_t* a_pack, const uint8_t* b_col, int32_t* C, int M, int N, int K,
                   int split_k, void* stream);

/* GEMM with the dequant fused into its epilogue; replaces the reference's GEMM followed by
 * `scale_i32_to_fp16` (call sites ...fusedtopr_v43.py:262,283) and its fused-epilogue
 * prototypes tools/quarot_split_fused_epilogue_ext_v1.py:283-432:
 *   out[m,n] = bf16( (float(acc) * body_scale[m]) * w_scale[n] + tail[m,n] + bias[n] )
 * `tail` ([M,N] f32, the result of tq_tail_gather) and `bias` ([N] f32) may be NULL. */
int tq_split_gemm_fused(const uint8_t* a_pack, const float* body_scale, const uint8_t* b_col,
                        const float* w_scale, const float* tail, const float* bias, void* out_bf16,
                        int M, int N, int K, void* stream);

/* The same linear in ONE kernel with the tail on the tensor cores: the dense part runs on tcgen05
 * kind::i8, the tail as a bf16 MMA (fp32 accumulation in tensor memory) over the zero-filled tail
 * matrix that the kernel builds in shared memory from the (index, value) lists.  The INT4 codes,
 * indices and int32 accumulators are the same bits as on the other path; the tail sum is an fp32
 * tensor-core accumulation instead of the fixed-order fma chain of tq_tail_gather, so the bf16 output
 * can differ from that path in the last bit.  Has the role of the reference's fused-epilogue
 * prototypes (tools/quarot_split_fused_epilogue_ext_v1.py:283-432).
 *   a_q8      [M,K] i8 from tq_split_prologue       w_rot  [N,K] bf16 from tq_prepare_weight (R > 0)
 *   tail_ptr, tail_rec, tail_cnt  from tq_split_prologue (R > 0)
 *   tail_dense  optional [M,K] bf16 from tq_split_prologue: with it, the 32-row blocks of a half slice in which a
 *               row has more than TQ_TAIL_REC_CAP entries are loaded from it by TMA (CTA-pair kernel); without
 *               it those rows are completed from tail_idx16 / tail_val.  Same results either way.
 *   dbg_acc   optional [M,N] i32: accumulators      dbg_tail  optional [M,N] f32: tail sums */
int tq_split_gemm_mma(const int8_t* a_q8, const float* body_scale, const uint8_t* b_col,
                      const float* w_scale, const void* w_rot, const uint16_t* tail_idx16,
                      const void* tail_val, int tail_ld, const uint16_t* tail_ptr, int ptr_ld,
                      const uint32_t* tail_rec, const uint16_t* tail_cnt, const void* tail_dense, int R,
                      const float* bias, void* out_bf16,
                      int32_t* dbg_acc, float* dbg_tail, int M, int N, int K, void* stream);

/* The same linear for a fused gate_up projection whose weight rows are INTERLEAVED (row 2i = gate_i, row 2i+1 =
 * up_i; N = 2 I): the epilogue applies SwiGLU to each channel pair and writes out [M, N/2] bf16,
 *   out[m,i] = bf16( bf16(silu(g)) * u ),  g = bf16(y[m,2i]), u = bf16(y[m,2i+1]),  silu(g) = g / (1 + exp(-g)),
 * i.e. what a bf16 framework computes from the two linears' bf16 outputs -- the reference does this step in
 * PyTorch (tools/bench_prefill_bf16_romeoquarotdense_split_total_v61_sharedprepare.py:214).  No [M, N]
 * intermediate is written. */
int tq_split_gemm_mma_swiglu(const int8_t* a_q8, const float* body_scale, const uint8_t* b_col,
                             const float* w_scale, const void* w_rot, const uint16_t* tail_idx16,
                             const void* tail_val, int tail_ld, const uint16_t* tail_ptr, int ptr_ld,
                             const uint32_t* tail_rec, const uint16_t* tail_cnt, const void* tail_dense, int R,
                             const float* bias, void* out_bf16, int M, int N, int K, void* stream);

/* tq_split_gemm_mma has two kernels: one CTA per 128 x 256 tile, and CTA pairs on 256 x 256 tiles
 * (tcgen05 cta_group::2; each CTA loads half of the weight tiles).  mode -1 (default) chooses by shape (pairs
 * without a tail or when there are more than 74 one-CTA tiles), 0 / 1 force one of them.  A tuning knob without
 * a reference counterpart. */
int tq_set_gemm_pair_mode(int mode);

/* The prologue has two kernels with identical outputs: one specialised for K = 4096, 12288 and 14336 (a thread per
 * 64 contiguous elements, the row staged by one TMA load) and a general one for every other built width.  mode -1
 * (default) uses the specialised kernel where it applies, 0 forces the general one.  A comparison switch without a
 * reference counterpart. */
int tq_set_prologue_mode(int mode);

/* Finisher of the split-K path: out = bf16((float(C)*body_scale[m])*w_scale[n] + tail + bias). */
int tq_dequant_finish(const int32_t* C, const float* body_scale, const float* w_scale,
                      const float* tail, const float* bias, void* out_bf16, int M, int N, void* stream);

/* ---------------------------------------------------------------------------------------
 * Sparse tail correction, tail mode T16 (bf16 values, 16-bit indices, bf16 weight rows):
 *   tail[m,n] = sum_r  tail_val[m,r] * w_t[tail_idx16[m,r], n]
 * evaluated as one fp32 fused-multiply-add chain per output in ascending index order.
 * Replaces `sparse_top_add_rowmajor_quad_shared` (call sites ...fusedtopr_v43.py:287-295)
 * and tools/sparse_correction_add_ext_v1.py:64-123 for the bf16-tail mode.
 * `tail` is [M,N] f32, fully written by this call.  N % 8 == 0, K <= 65536.
 */
int tq_tail_gather(const uint16_t* tail_idx16, const void* tail_val, const void* w_t,
                   float* tail, int M, int N, int K, int R, int tail_ld, void* stream);

/* Small-M (decode) variants, M <= 64.  The reference has no separate small-M path (its decode bench runs
 * the prefill kernels at M = 16/64/256: tools/bench_qwen3_decode_split_romeo_quarot_v33.py:36,97-108).
 * tq_int4_gemv_splitk: C [M,N] i32 = exact INT4 x INT4 product, weights streamed once at HBM speed, the
 *   reduction split over `split_k` CTAs per 64 output channels (split_k < 1 picks it); C is zeroed by the call.
 *   The activations come either packed (a_pack) or as the prologue's INT8 operand (a_q8): exactly one is given.
 * tq_tail_gather_small: the tail sums, reading only the M*R weight rows they need; per output eight
 *   interleaved fp32 fma chains (entry r on chain r mod 8) combined as ((c0+c1)+(c2+c3))+((c4+c5)+(c6+c7)). */
int tq_int4_gemv_splitk(const uint8_t* a_pack, const int8_t* a_q8, const uint8_t* b_col, int32_t* C, int M,
                        int N, int K, int split_k, void* stream);
/* The same product with the K ranges kept apart: partials [splits, M, N] i32, slab s = the sum over K range s,
 * every element written by plain stores (no zeroing, no atomics: one launch).  `splits` must be the count
 * tq_int4_gemv_plan(M, N, K, a_is_int8) returns (> 0; negative = error code).
 * tq_dequant_finish_partials adds the slabs (exactly) and finishes like tq_dequant_finish; act = 1 applies the
 * SwiGLU of tq_split_gemm_mma_swiglu (out [M, N/2]). */
int tq_int4_gemv_plan(int M, int N, int K, int a_is_int8);
/* 8-channel tiles that a warp of the GEMV multiplies with one activation fragment: -1 (default) = 1 up to 16 rows, 4
 * beyond (packed activations), or 1 / 2 / 4 for every call with more than 16 rows.  tq_int4_gemv_plan follows it.
 * A comparison switch without a reference counterpart. */
int tq_set_gemv_channel_tiles(int tiles);
int tq_int4_gemv_partials(const uint8_t* a_pack, const int8_t* a_q8, const uint8_t* b_col, int32_t* partials,
                          int M, int N, int K, int splits, void* stream);
int tq_dequant_finish_partials(const int32_t* partials, int splits, const float* body_scale, const float* w_scale,
                               const float* tail, const float* bias, void* out_bf16, int M, int N, int act,
                               void* stream);
int tq_tail_gather_small(const uint16_t* tail_idx16, const void* tail_val, const void* w_t, float* tail,
                         int M, int N, int K, int R, int tail_ld, void* stream);

/* ---------------------------------------------------------------------------------------
 * Reference-compatible tail mode T4 (INT4 tail codes against the INT4 weight rows).
 *
 * tq_scale_sparse_epilogue: scale_sparse_epilogue_quad|oct(C, body_scale, top_q, idx,
 *   B_row_pack, top_scale, w_scale, out, K)   tools/fused_sparse_epilogue_ext_v58.py:123-169
 *   out[m,n] = f16( float(C)*bs[m]*ws[n] + float(sum_r tq*qw[idx,n])*ts[m]*ws[n] )
 * tq_sparse_correction_add: sparse_correction_add_{bf16,fp16}_oct(out, top_q, idx, B_row_pack,
 *   top_scale, w_scale)                        tools/sparse_correction_add_ext_v1.py:175-224
 *   out[m,n] = f16( float(out[m,n]) + float(sum)*ts[m]*ws[n] ),  w_scale f32 or bf16
 * tq_sparse_top_write: sparse_{i32,u16}_c{4,8,16}_b{128,256}(...) write-only variants
 *                                              tools/split_sparse_idx16_ext_v1.py:50-109
 * tq_idx_i32_to_u16: idx_i32_to_u16            tools/split_sparse_idx16_ext_v1.py:31-48
 * `out_dtype` is TQ_BF16 or TQ_FP16; `idx_u16` selects 16-bit indices. */
int tq_scale_sparse_epilogue(const int32_t* C, const float* body_scale, const int8_t* top_q,
                             const int32_t* idx, const uint8_t* b_row, const float* top_scale,
                             const float* w_scale, void* out, int out_dtype, int M, int N, int K, int R,
                             void* stream);
int tq_sparse_correction_add(void* out, int out_dtype, const int8_t* top_q, const int32_t* idx,
                             const uint8_t* b_row, const float* top_scale, const void* w_scale,
                             int w_scale_bf16, int M, int N, int K, int R, void* stream);
int tq_sparse_top_write(void* out, int out_dtype, const int8_t* top_q, const void* idx, int idx_u16,
                        const uint8_t* b_row, const float* top_scale, const float* w_scale,
                        int M, int N, int K, int R, void* stream);
int tq_idx_i32_to_u16(const int32_t* idx, uint16_t* out, long long n, void* stream);

/* Split-K linear for callers that cannot allocate device memory: the same computation as
 * tq_int4_matmul(split_k) followed by tq_dequant_finish,
 *   out[m,n] = bf16((float(sum_k qa qw) * body_scale[m]) * w_scale[n] + tail[m,n] + bias[n]),
 * but the int32 accumulators between the two passes live in a fixed 4 MiB array inside the library instead of
 * a caller-supplied buffer (M * N <= TQ_NOALLOC_MAX_ELEMS, else TQ_ERR_TOO_LARGE).  `tail` and `bias` may be
 * NULL.  This entry point has no counterpart in the reference: it exists for hosts whose device memory is
 * entirely owned by their own pool, or that must not call cudaMalloc/cudaFree in their decode loop.
 * The array is shared by all calls on a device (the used part is zeroed at the start of each call), so calls
 * whose GPU work overlaps race; its device address is looked up on the first call on each device, which
 * should therefore be made once at start-up, before any stream capture begins. */
#define TQ_NOALLOC_MAX_ELEMS (1 << 20)
int tq_int4_linear_splitk_noalloc(const uint8_t* a_pack, const float* body_scale, const uint8_t* b_col,
                                  const float* w_scale, const float* tail, const float* bias, void* out_bf16,
                                  int M, int N, int K, int split_k, void* stream);

/* Status word of the GEMM launches on the current device since the previous call: 0, or a code naming the
 * pipeline wait that ran out of its time budget (the kernel then drains and returns instead of spinning; its
 * output is not valid).  Synchronises the device, returns TQ_ERR_DEVICE_STATUS when the word is non-zero and
 * clears it, so poll it at a synchronisation point after the launches whose result matters. */
int tq_gemm_status(unsigned int* status);

#ifdef __cplusplus
}
#endif
#endif /* TAILQUANT_H_ */
