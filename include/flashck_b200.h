/*
 * flashck_b200 -- C ABI of the B200-native attention path (libflashck_b200.so).
 *
 * Each entry point replaces one `extern "C"` function that FlashCK's generated
 * `generated_kernel.so` exports and that `Kernel::KernelLauncher` binds with
 * `dylib::get_function` (core/utils/dylib_utils.h:76-91).  Names and argument order
 * follow the reference; three things differ and are the same for every function:
 *   - `std::array<int64_t,2> window_size` is not expressible in C, so it is passed
 *     as two scalars `window_left, window_right` (-1 = unbounded);
 *   - `hipStream_t` becomes `void* stream` (a cudaStream_t);
 *   - the reference bakes the element type into each generated instance; here it is
 *     a trailing `int dtype` (3 = float16, 4 = bfloat16, the values of
 *     flashck::DataType, core/utils/dtype.h:16-28), and functions return an int
 *     status (0 = ok) instead of printing to stderr and returning void
 *     (core/module/kernels/attention_kernels/fmha_common_jinja.h:5-12).
 * Where the reference passes `nullptr` for the LSE (fmha_fwd/fmha_fwd_jinja.h:317),
 * a trailing optional `lse_ptr` receives it.
 *
 * All data pointers are device pointers; the caller owns every buffer, including
 * the split-KV workspaces, and the callee never allocates.  Calls are asynchronous
 * enqueues on `stream` and re-entrant.  Layouts are BSHD: Q [b,sq,hq,d],
 * K [b,sk,hkv,d], V [b,sk,hkv,dv], O [b,sq,hq,dv]; group (varlen) mode packs the
 * sequences along the token axis ([total,h,d]) with int64 `seqstart` arrays [b+1].
 * LSE is fp32: [b,hq,sq] in batch mode, [hq,total_q] in group mode.
 * mask_type: 0 none, 1 top-left, 2 bottom-right, 3 generic (treated as top-left
 * coordinates); causal = window (-1, 0).   scale == 0 means 1/sqrt(hdim_q).
 */
#ifndef FLASHCK_B200_H_
#define FLASHCK_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* exported with default visibility, like FC_EXPORT in the reference
 * (attention_kernels/fmha_common_jinja.h:14-17) */
#if defined(__GNUC__)
#define FLASHCK_API __attribute__((visibility("default")))
#else
#define FLASHCK_API
#endif

#define FLASHCK_DTYPE_FLOAT8 1   /* E4M3 (OCP, finite only) -- FmhaFwdFp8 and FmhaFwd */
#define FLASHCK_DTYPE_BFLOAT8 2  /* E5M2 */
#define FLASHCK_DTYPE_FLOAT16 3
#define FLASHCK_DTYPE_BFLOAT16 4
#define FLASHCK_DTYPE_FLOAT32 7 /* only as the output type of FmhaFwdSplitKVCombineStrided */

/* status codes */
#define FLASHCK_OK 0
#define FLASHCK_ERR_INVALID_ARGUMENT 1   /* null pointer, bad shape, hq % hkv != 0 ... */
#define FLASHCK_ERR_UNSUPPORTED 2        /* no kernel instance for this problem */
#define FLASHCK_ERR_CUDA 3               /* a CUDA runtime / driver call failed */
#define FLASHCK_ERR_DEVICE_TIMEOUT 4     /* a bounded device-side wait ran out */

/* Bits of the device status word (FlashckDeviceStatus).  The low 29 bits are set by bounded device-side waits that
 * ran out (each kernel role has its own code); the two bits below report work that a kernel refused to do. */
#define FLASHCK_STATUS_TIMEOUT_MASK 0x1fffffff
#define FLASHCK_STATUS_WORKLIST_OVERFLOW 0x20000000 /* an on-chip work list was too small: the launch did nothing */
#define FLASHCK_STATUS_APPEND_OVERFLOW 0x40000000   /* FmhaFwdAppendKV skipped tokens that did not fit the cache */

/* Human-readable text of the last error raised on the calling thread. */
FLASHCK_API const char* FlashckGetLastError(void);
/* Library version string. */
FLASHCK_API const char* FlashckVersion(void);
/* Reads and clears the device-side status word of the current device into *status_out (0 = nothing to report).
 * Synchronises the device.  Returns FLASHCK_ERR_DEVICE_TIMEOUT when a bounded wait ran out, FLASHCK_ERR_UNSUPPORTED
 * when a kernel skipped work (one of the two bits above), FLASHCK_OK when the word was 0. */
FLASHCK_API int FlashckDeviceStatus(int* status_out);

/*
 * FmhaFwd -- dense or varlen forward attention.
 * Replaces `FmhaFwd` (signature: core/module/kernels/attention_kernels/fmha_fwd/fmha_fwd_jinja.h:124-147;
 * declaration fmha_fwd/fmha_fwd_call.h:34-53; launcher fmha_fwd/fmha_fwd_kernel.cc:79-107).
 * Batch mode: the three seq pointers are NULL.  Group mode: q_seq_start / k_seq_start are int64 [batch+1]
 * device arrays; k_seq_len_ptr (int64 [batch], optional) overrides the key length of each sequence.
 * bias_buf_ptr: NULL, or a bias read the way the instance parameters `bias_enum` (1 elementwise, 2 alibi) and
 * `bias_rank_info` of family 0 say (the reference fixes both per compiled instance); see FmhaFwdBias.
 */
FLASHCK_API int FmhaFwd(void* q_buf_ptr, void* k_buf_ptr, void* v_buf_ptr, void* bias_buf_ptr, void* o_buf_ptr,
            int64_t* q_seq_start_ptr, int64_t* k_seq_start_ptr, int64_t* k_seq_len_ptr, int64_t batch,
            int64_t q_seq_len, int64_t kv_seq_len, int64_t q_num_heads, int64_t kv_num_heads, int64_t qk_head_dim,
            int64_t v_head_dim, int64_t q_max_seq_len, float scale, int64_t window_left, int64_t window_right,
            uint32_t mask_type, void* stream, void* lse_ptr, int dtype);

/*
 * FmhaFwdBias -- FmhaFwd with the instance properties the reference compiles in as call arguments
 * (core/profiling/attention/fmha_fwd/fmha_fwd_problem.h:59-81 `bias_enum`, `bias_rank_info`, `has_logits_soft_cap`;
 * bias strides attention_kernels/fmha_fwd/fmha_fwd_jinja.h:199-233,270-293; enum core/profiling/attention/
 * fmha_library.h:121-164).  bias_enum 1: bias_buf_ptr holds element-dtype values, bias_rank_info 0 = [1,1,sq,sk],
 * 1 = [1,hq,sq,sk], 2 = [b,hq,sq,sk] (group mode: sq and sk are the packed totals q_seq_len / kv_seq_len and a
 * sequence's block starts at its first packed row and key); contiguous K/V of the stated lengths only.
 * bias_enum 2 (alibi): bias_buf_ptr holds fp32 slopes, bias_rank_info 0 = [1,hq], 1 = [b,hq]; the score of query i
 * and key j gets -slope * |i + sk - sq - j| added.  logits_soft_cap > 0: score = cap * tanh(score / cap), applied to
 * the scaled score before the bias.  These calls run on the general (mma.sync) instance.
 */
FLASHCK_API int FmhaFwdBias(void* q_buf_ptr, void* k_buf_ptr, void* v_buf_ptr, void* bias_buf_ptr, void* o_buf_ptr,
            int64_t* q_seq_start_ptr, int64_t* k_seq_start_ptr, int64_t* k_seq_len_ptr, int64_t batch,
            int64_t q_seq_len, int64_t kv_seq_len, int64_t q_num_heads, int64_t kv_num_heads, int64_t qk_head_dim,
            int64_t v_head_dim, int64_t q_max_seq_len, float scale, int64_t window_left, int64_t window_right,
            uint32_t mask_type, void* stream, void* lse_ptr, int dtype, int bias_enum, int bias_rank_info,
            float logits_soft_cap);

/*
 * FmhaFwdFp8 -- forward attention on 8-bit operands with static quantisation scales: the reference's
 * FmhaFwdTypeConfig<fp8_t> / <bf8_t> (attention_kernels/fmha_common_jinja.h:157-187: Q, K, V, P and O are 8-bit floats,
 * S, softmax, O accumulator and LSE fp32) with the kernel arguments scale_s, scale_p, scale_o
 * (attention_kernels/fmha_fwd/fmha_fwd_jinja.h:93,326-328) as call arguments.  dtype: 1 = E4M3 (FLOAT8), 2 = E5M2
 * (BFLOAT8), the OCP formats; conversions round to nearest even and saturate.  Per row:
 *     S = scale_s * Q K^T;  p = exp(S - max);  l = sum p;  P8 = round8(scale_p * p);  O = scale_o * (P8 V) / l
 * so scale_s carries the softmax scale and the de-quantisation of Q and K (0 means 1/sqrt(hdim_q)), scale_p the stretch
 * of the probabilities over the 8-bit range, scale_o = (V de-quantisation) / (scale_p * O quantisation).
 * o_dtype: the type O is stored in -- 1 or 2 (one byte per element) or 3 / 4 (fp16 / bf16).  Batch mode or group mode
 * (q_seq_start / k_seq_start int64 [batch+1]) on contiguous K/V; hdim 64 or 128.
 * FmhaFwd called with dtype 1 or 2 is FmhaFwdFp8 with scale_s = scale, scale_p = scale_o = 1 and o_dtype = dtype (the
 * constants the reference passes, fmha_fwd_jinja.h:326-328).
 */
FLASHCK_API int FmhaFwdFp8(void* q_buf_ptr, void* k_buf_ptr, void* v_buf_ptr, void* o_buf_ptr, int64_t* q_seq_start_ptr,
               int64_t* k_seq_start_ptr, int64_t batch, int64_t q_seq_len, int64_t kv_seq_len, int64_t q_num_heads,
               int64_t kv_num_heads, int64_t qk_head_dim, int64_t v_head_dim, int64_t q_max_seq_len, float scale_s,
               float scale_p, float scale_o, int64_t window_left, int64_t window_right, uint32_t mask_type, void* stream,
               void* lse_ptr, int dtype, int o_dtype);

/*
 * FmhaFwdBatchPrefill -- varlen prefill whose K/V sit behind an SGLang-style page table.
 * The reference emits this family (core/profiling/attention/fmha_fwd_batch_prefill/
 * fmha_fwd_batch_prefill_codegen.cc:93-162, problem ..._problem.h:20-99 `num_total_pages`) but its glue
 * files (attention_kernels/fmha_fwd_batch_prefill/...) are empty, so the argument list is defined here:
 * Q [total_q,hq,d] with q_seq_start int64 [batch+1] and q_seq_len = total_q; K/V pools [num_total_pages,page,hkv,d|dv];
 * kv_indptr int32 [batch+1], kv_page_indices int32 [kv_indptr[batch]], kv_last_page_len int32 [batch].
 * bias_buf_ptr: NULL, or fp32 ALiBi slopes ([1,hq] / [batch,hq] by `bias_rank_info`) while the instance parameter
 * `bias_enum` of family 0 is 2; any other bias is refused (this holds for FmhaFwdPagedKVPrefill and FmhaFwdSplitKV too).
 */
FLASHCK_API int FmhaFwdBatchPrefill(void* q_buf_ptr, void* k_buf_ptr, void* v_buf_ptr, void* bias_buf_ptr, void* o_buf_ptr,
                        int64_t* q_seq_start_ptr, void* kv_indptr, void* kv_page_indices, void* kv_last_page_len,
                        int64_t batch, int64_t q_seq_len, int64_t q_num_heads, int64_t kv_num_heads,
                        int64_t qk_head_dim, int64_t v_head_dim, int64_t q_max_seq_len, int64_t num_total_pages,
                        int64_t paged_block_size, float scale, int64_t window_left, int64_t window_right,
                        uint32_t mask_type, void* stream, void* lse_ptr, int dtype);

/*
 * FmhaFwdPagedKVPrefill -- prefill reading K/V through a block table (same page layout as FmhaFwdSplitKV).
 * Family emitted at core/profiling/attention/fmha_fwd_paged_kv_prefill/fmha_fwd_paged_kv_prefill_codegen.cc:85-144;
 * glue files empty in the reference, argument list modelled on FmhaFwdSplitKV without the split workspaces.
 * k_seq_len_ptr: int32 [batch]; block_table: int32 [batch, max_num_page_blocks / batch].
 */
FLASHCK_API int FmhaFwdPagedKVPrefill(void* q_buf_ptr, void* k_buf_ptr, void* v_buf_ptr, void* bias_buf_ptr, void* o_buf_ptr,
                          int64_t* q_seq_start_ptr, void* k_seq_len_ptr, void* block_table_buf_ptr,
                          int64_t* cache_batch_idx_buf_ptr, int64_t batch, int64_t q_seq_len, int64_t q_num_heads,
                          int64_t kv_num_heads, int64_t qk_head_dim, int64_t v_head_dim, int64_t q_max_seq_len,
                          int64_t max_num_page_blocks, int64_t paged_block_size, float scale, int64_t window_left,
                          int64_t window_right, uint32_t mask_type, void* stream, void* lse_ptr, int dtype);

/*
 * FmhaFwdSplitKV -- per-split partial attention over contiguous or paged K/V.
 * Replaces `FmhaFwdSplitKV` (signature: attention_kernels/fmha_fwd_split_kv/fmha_fwd_split_kv_jinja.h:155-184;
 * launcher fmha_fwd_split_kv/fmha_fwd_split_kv_kernel.cc:90-123).
 * Writes o_acc fp32 [b,hq,num_splits,sq,dv] (normalised within the split) and lse_acc fp32 [b,hq,num_splits,sq]
 * (fmha_fwd_split_kv_jinja.h:543-547; group mode: b = 1, sq = total_q).  A split that received no keys gets
 * lse_acc = -inf.  lse_acc may be NULL only when num_splits == 1.
 * Paged: K/V pools [max_num_page_blocks, page, hkv, d|dv] (:512-519), block_table int32
 * [batch, max_num_page_blocks / batch] (:318,550), k_seq_len_ptr int32 [batch] (required when paged).  The pools'
 * tensor maps end after max_num_page_blocks pages (a page id beyond that reads as zeros); pools of another size go
 * through FmhaFwdSplitKVEx.
 * How the key range of a sequence is cut into splits is internal (balanced over the SMs); only
 * "at most num_splits splits per sequence" is guaranteed.
 */
FLASHCK_API int FmhaFwdSplitKV(void* q_buf_ptr, void* k_buf_ptr, void* v_buf_ptr, void* bias_buf_ptr, void* lse_acc_buf_ptr,
                   void* o_acc_buf_ptr, int64_t* q_seq_start_ptr, int64_t* kv_seq_start_ptr, void* k_seq_len_ptr,
                   void* block_table_buf_ptr, int64_t* cache_batch_idx_buf_ptr, int64_t batch, int64_t q_seq_len,
                   int64_t kv_seq_len, int64_t q_num_heads, int64_t kv_num_heads, int64_t qk_head_dim,
                   int64_t v_head_dim, int64_t q_max_seq_len, int64_t num_splits, int64_t max_num_page_blocks,
                   int64_t paged_block_size, float scale, int64_t window_left, int64_t window_right,
                   uint32_t mask_type, void* stream, int dtype);

/*
 * FmhaFwdBatchPrefillEx / FmhaFwdPagedKVPrefillEx / FmhaFwdSplitKVEx -- the three paged entry points with what the
 * reference compiles into an instance, or implies, stated per call (the relation of FmhaFwdBias to FmhaFwd):
 *   bias_enum, bias_rank_info   how bias_buf_ptr is read: 0 = ignored, 2 = fp32 ALiBi slopes ([1,hq] for rank 0,
 *                               [batch,hq] for rank 1; core/profiling/attention/fmha_library.h:121-164).  No
 *                               process-wide instance parameter is consulted, so concurrent callers cannot disturb each
 *                               other.
 *   num_pool_pages              pages the K/V pools really hold.  The reference sizes its pools to max_num_page_blocks
 *                               (= batch * pages_per_sequence, fmha_fwd_split_kv_jinja.h:512-519), which the plain
 *                               symbols assume; a serving pool is shared by more sequences than one call sees.  The
 *                               pools' tensor maps end at this extent: a page id at or beyond it reads as zeros.
 *                               FmhaFwdSplitKVEx on a contiguous cache with cache_batch_idx: rows of the cache (0 = unknown).
 * All other arguments are those of the plain symbols.
 */
FLASHCK_API int FmhaFwdBatchPrefillEx(void* q_buf_ptr, void* k_buf_ptr, void* v_buf_ptr, void* bias_buf_ptr, void* o_buf_ptr,
                          int64_t* q_seq_start_ptr, void* kv_indptr, void* kv_page_indices, void* kv_last_page_len,
                          int64_t batch, int64_t q_seq_len, int64_t q_num_heads, int64_t kv_num_heads,
                          int64_t qk_head_dim, int64_t v_head_dim, int64_t q_max_seq_len, int64_t num_total_pages,
                          int64_t paged_block_size, float scale, int64_t window_left, int64_t window_right,
                          uint32_t mask_type, void* stream, void* lse_ptr, int dtype, int bias_enum, int bias_rank_info);
FLASHCK_API int FmhaFwdPagedKVPrefillEx(void* q_buf_ptr, void* k_buf_ptr, void* v_buf_ptr, void* bias_buf_ptr, void* o_buf_ptr,
                            int64_t* q_seq_start_ptr, void* k_seq_len_ptr, void* block_table_buf_ptr,
                            int64_t* cache_batch_idx_buf_ptr, int64_t batch, int64_t q_seq_len, int64_t q_num_heads,
                            int64_t kv_num_heads, int64_t qk_head_dim, int64_t v_head_dim, int64_t q_max_seq_len,
                            int64_t max_num_page_blocks, int64_t paged_block_size, float scale, int64_t window_left,
                            int64_t window_right, uint32_t mask_type, void* stream, void* lse_ptr, int dtype,
                            int bias_enum, int bias_rank_info, int64_t num_pool_pages);
FLASHCK_API int FmhaFwdSplitKVEx(void* q_buf_ptr, void* k_buf_ptr, void* v_buf_ptr, void* bias_buf_ptr, void* lse_acc_buf_ptr,
                     void* o_acc_buf_ptr, int64_t* q_seq_start_ptr, int64_t* kv_seq_start_ptr, void* k_seq_len_ptr,
                     void* block_table_buf_ptr, int64_t* cache_batch_idx_buf_ptr, int64_t batch, int64_t q_seq_len,
                     int64_t kv_seq_len, int64_t q_num_heads, int64_t kv_num_heads, int64_t qk_head_dim,
                     int64_t v_head_dim, int64_t q_max_seq_len, int64_t num_splits, int64_t max_num_page_blocks,
                     int64_t paged_block_size, float scale, int64_t window_left, int64_t window_right,
                     uint32_t mask_type, void* stream, int dtype, int bias_enum, int bias_rank_info,
                     int64_t num_pool_pages);

/*
 * FmhaFwdSplitKVCombine -- LSE-weighted merge of the split partials into O (and LSE).
 * Replaces `FmhaFwdSplitKVCombine` (signature: attention_kernels/fmha_fwd_split_kv_combine/
 * fmha_fwd_split_kv_combine_jinja.h:78-92; declaration ..._combine_call.h:26-36).  The reference's code
 * generator names the symbol `FmhaSplitKVCombine` (..._combine_kernel.cc:16); both names are exported.
 */
FLASHCK_API int FmhaFwdSplitKVCombine(void* lse_acc_buf_ptr, void* o_acc_buf_ptr, void* o_buf_ptr, int64_t* q_seq_start_ptr,
                          int64_t batch, int64_t q_seq_len, int64_t q_num_heads, int64_t v_head_dim,
                          int64_t q_max_seq_len, int64_t num_splits, void* stream, void* lse_ptr, int dtype);
FLASHCK_API int FmhaSplitKVCombine(void* lse_acc_buf_ptr, void* o_acc_buf_ptr, void* o_buf_ptr, int64_t* q_seq_start_ptr,
                       int64_t batch, int64_t q_seq_len, int64_t q_num_heads, int64_t v_head_dim,
                       int64_t q_max_seq_len, int64_t num_splits, void* stream, void* lse_ptr, int dtype);

/*
 * FmhaFwdSplitKVCombineStrided -- the same LSE-weighted merge with explicit strides and an optional fp32 result.
 * The reference is single-GPU and has no counterpart; its combine kernel takes exactly these strides as kernel
 * arguments (MakeKargs, fmha_fwd_split_kv_combine_jinja.h:176-215), the C symbol just fixes them.  Used when the
 * KV sequence of one request is sharded over several GPUs: every rank merges its local splits into fp32
 * (out_dtype = 7), the ranks all-gather those partials, and one more merge over the gathered [rank][...] buffer
 * (num_splits = world size) gives O.  lse_strides / o_acc_strides: 4 int64 each, in elements, for
 * (batch, head, split, row); hdim is contiguous and o_acc strides must be multiples of 4.
 * Output o is [batch, rows, hq, dv] in out_dtype, lse (optional) fp32 [batch, hq, rows].
 */
FLASHCK_API int FmhaFwdSplitKVCombineStrided(void* lse_acc_buf_ptr, void* o_acc_buf_ptr, void* o_buf_ptr, void* lse_ptr,
                                             int64_t batch, int64_t rows, int64_t q_num_heads, int64_t v_head_dim,
                                             int64_t num_splits, const int64_t* lse_strides,
                                             const int64_t* o_acc_strides, int out_dtype, void* stream);

/*
 * FmhaFwdSplitKVShardedCombine -- for a KV sequence sharded over the GPUs of one node: the merge of this rank's splits,
 * the exchange of the per-rank fp32 partials (O_r, LSE_r) over NVLink and the merge over the ranks, in one kernel.
 * The reference is single-GPU and has no counterpart; the arithmetic is its combine's
 * (fmha_fwd_split_kv_combine_jinja.h:125-140) applied twice.  Every rank of the group calls it once per decode step,
 * after its FmhaFwdSplitKV, with
 *   lse_acc / o_acc      this rank's split workspaces in the reference layout ([b,hq,S,rows], [b,hq,S,rows,dv] fp32),
 *   o / lse              the results ([b,rows,hq,dv] in out_dtype, fp32 [b,hq,rows] or NULL), identical on every rank,
 *   exchange_bufs        `world` device pointers: the exchange buffer of every rank as mapped into this process (its
 *                        own from FlashckPeerBufferCreate, the others from FlashckPeerBufferOpen), each of
 *                        FlashckShardExchangeBytes(...) bytes, zeroed once before the first call and used for this
 *                        purpose only (same sizes on every call).
 * The pointer arguments are host arrays indexed by LOCAL rank: a process that owns one GPU passes local_ranks = 1 and
 * first_rank = its rank.  local_ranks > 1 plays several ranks of the group in one (cooperative) launch on one GPU, all
 * buffers local -- the form the single-GPU tests use.  Partials travel as plain stores to peer memory with a flag in
 * every 8 bytes; the waits for them are bounded (about a second), after which the row is left unwritten and
 * FlashckDeviceStatus reports FLASHCK_ERR_DEVICE_TIMEOUT.  Every rank must make the same sequence of calls.
 */
FLASHCK_API int64_t FlashckShardExchangeBytes(int64_t batch, int64_t rows, int64_t q_num_heads, int64_t v_head_dim, int world);
FLASHCK_API int FmhaFwdSplitKVShardedCombine(void* const* lse_acc_ptrs, void* const* o_acc_ptrs, void* const* o_ptrs,
                                 void* const* lse_ptrs, void* const* exchange_bufs, int first_rank, int local_ranks,
                                 int world, int64_t batch, int64_t rows, int64_t q_num_heads, int64_t v_head_dim,
                                 int64_t num_splits, int out_dtype, void* stream);
/* Exchange buffers.  Create: cudaMalloc + zero fill + a 64-byte handle another process of the node can open (CUDA IPC).
 * These four are set-up calls (they allocate, map and synchronise); nothing on the per-step path does. */
FLASHCK_API int FlashckPeerBufferCreate(int64_t bytes, void** ptr_out, void* handle_out64);
FLASHCK_API int FlashckPeerBufferOpen(const void* handle64, void** ptr_out);
FLASHCK_API int FlashckPeerBufferClose(void* ptr);
FLASHCK_API int FlashckPeerBufferFree(void* ptr);

/*
 * FmhaFwdAppendKV -- rotary embedding of Q and the new keys, and the K/V cache write.
 * The reference names the kind (core/profiling/attention/fmha_library.h:19,41), the rotary modes
 * (fmha_library.h:195-219: 0 none, 1 interleaved, 2 half-rotated) and the table generator
 * (attention_kernels/fmha_common_jinja.h:192-227) but has no source for the function; the argument list is
 * defined here in the reference's style.
 *   q: [b,sq,hq,d] or group mode [total_q,hq,d] (q_seq_start), rotated IN PLACE at positions
 *      seqlen_k[b] + n_new[b] - sq[b] + i.
 *   knew/vnew: [b,n,hkv,d|dv] or group mode [total_new,hkv,*] (knew_seq_start int64 [b+1]).
 *   k/v cache: paged pool [pages,page,hkv,*] + block_table int32 [b, max_num_page_blocks/b], or contiguous
 *      [b_cache, kv_seq_len, hkv, *] when block_table is NULL.  New token j lands at seqlen_k[b] + j.
 *   k_seq_len_ptr: int32 [b], cached length BEFORE the append (not updated by the call).  A new token that does not
 *      fit its sequence's cache (position >= pages_per_sequence * page, or >= kv_seq_len of a contiguous cache, or a
 *      negative block-table entry) is skipped and FLASHCK_STATUS_APPEND_OVERFLOW is set in the device status word.
 *   rotary_cos/sin: [positions, rotary_dim/2] in the element dtype, indexed by absolute position.
 * Cache contents are bit-exact against the CPU statement of the same arithmetic: fp32 products and sums,
 * each rounded separately (no FMA), round-to-nearest-even narrowing.
 */
FLASHCK_API int FmhaFwdAppendKV(void* q_buf_ptr, void* k_buf_ptr, void* knew_buf_ptr, void* v_buf_ptr, void* vnew_buf_ptr,
                    void* k_seq_len_ptr, int64_t* q_seq_start_ptr, int64_t* knew_seq_start_ptr,
                    void* rotary_cos_ptr, void* rotary_sin_ptr, void* block_table_buf_ptr,
                    int64_t* cache_batch_idx_buf_ptr, int64_t batch, int64_t q_seq_len, int64_t kv_seq_len,
                    int64_t knew_seq_len, int64_t q_num_heads, int64_t kv_num_heads, int64_t qk_head_dim,
                    int64_t v_head_dim, int64_t rotary_dim, int rope_type, int64_t max_num_page_blocks,
                    int64_t paged_block_size, void* stream, int dtype);

/*
 * FmhaFwdSplitKVStatic -- split-KV attention and combine in one call, for callers that cannot allocate.
 * This entry point has no counterpart in the reference.  It exists for callers that may not call cudaMalloc
 * (a serving loop with a fixed memory plan, code that must stay inside a framework allocator, threads barred
 * from the allocator's locks): instead of caller-owned lse_acc / o_acc workspaces it uses a 16 MiB array that
 * the library keeps in device memory on every GPU that loads it.  Arguments are those of FmhaFwdSplitKV with
 * the two workspaces replaced by the final outputs o (element dtype, [b,sq,hq,dv]) and lse (fp32, optional).
 *   - The workspaces of the call, (b*hq*num_splits*sq) * (dv + 1) floats, must fit 16 MiB; otherwise the call
 *     returns FLASHCK_ERR_UNSUPPORTED and the error text gives both sizes.
 *   - All calls on a device share the array and it keeps the previous call's contents (none of it has to be
 *     zero).  Calls that overlap on the GPU race on it: run them one after another.
 *   - The first call on each device looks up the array's device address; make that call before any stream
 *     capture.  No call allocates or frees device memory.
 */
FLASHCK_API int FmhaFwdSplitKVStatic(void* q_buf_ptr, void* k_buf_ptr, void* v_buf_ptr, void* o_buf_ptr, void* lse_ptr,
                                     int64_t* q_seq_start_ptr, int64_t* kv_seq_start_ptr, void* k_seq_len_ptr,
                                     void* block_table_buf_ptr, int64_t* cache_batch_idx_buf_ptr, int64_t batch,
                                     int64_t q_seq_len, int64_t kv_seq_len, int64_t q_num_heads, int64_t kv_num_heads,
                                     int64_t qk_head_dim, int64_t v_head_dim, int64_t q_max_seq_len,
                                     int64_t num_splits, int64_t max_num_page_blocks, int64_t paged_block_size,
                                     float scale, int64_t window_left, int64_t window_right, uint32_t mask_type,
                                     void* stream, int dtype);

/*
 * Instance selection (the reference picks a tile instance per problem through its tuner,
 * core/profiling/attention/fmha_fwd/fmha_fwd_emitter.cc:325-466).  `family`: 0 fmha_fwd, 2 fmha_fwd_split_kv
 * (FmhaKind values, fmha_library.h:17-25).  Keys, all process-wide integers:
 *   family 0 -- "use_sm100" (1: the tcgen05 instances serve what they can, 0: everything on the general instance),
 *     "use_sm100_hdim64", "use_sm100_fp8", "use_sm100_bias" (1: hdim 64 / 8-bit operands / elementwise bias tensors on
 *     their tcgen05 instances, 0: on the general one), "exp_mode" (0: fp32 exponentials on the exp2 unit; 1: packed
 *     f16x2; 11, 12, 13: 1, 2 or 3 of every 8 column pairs on an FMA-pipe polynomial), "rescale_log2_x100" (lag of the
 *     running max for exp_mode 1), "poly8" (read-only view of the polynomial share), "bias_enum" / "bias_rank_info"
 *     (meaning of the bias pointer of the reference-shaped FmhaFwd symbol), "log_fallback" (1: a call that leaves the
 *     tcgen05 instances says why on stderr), "last_instance" (read-only: 1 if the last forward call ran on a tcgen05
 *     instance);
 *   family 2 -- "stages" (0 = as many as fit), "ctas_per_sm_x100", "heads_per_cta", "row_tiles" (decode kernel tiling; 0 =
 *     chosen per call), "use_sm100_splitkv" (1: calls with more than 16 query rows per kv head run on the tcgen05 split
 *     modes), "exp_mode_splitkv", "split_item_cost", "split_min_piece_tiles" (work cut of the split modes);
 *   any family -- "use_pdl" (1: the kernels of a decode step and the prefill kernel are launched as programmatic
 *     dependents of the kernel before them in the stream, see csrc/common.cuh).
 * Unknown keys return FLASHCK_ERR_INVALID_ARGUMENT.  Set before launching; not thread-safe against launches.
 */
FLASHCK_API int FlashckSetInstanceParam(int family, const char* key, int64_t value);
FLASHCK_API int FlashckGetInstanceParam(int family, const char* key, int64_t* value_out);

#ifdef __cplusplus
}
#endif
#endif /* FLASHCK_B200_H_ */
