// Host-side launch interfaces of the flashck_b200 kernels (one per .cu file).
#pragma once

#include "common.cuh"

namespace fck {

// ---- split-KV combine (combine.cu) ------------------------------------------------------------
struct CombineParams {
    const float* lse_acc;  // [bs, hq, S, rows]
    const float* o_acc;    // [bs, hq, S, rows, dv]
    void* o;               // [bs, rows, hq, dv] in dtype
    float* lse;            // [bs, hq, rows] or nullptr
    int64_t bs, rows, hq, dv, num_splits;
    int dtype;              // output element type: 3 float16, 4 bfloat16, 7 float32
    bool strided;           // use the strides below instead of the reference layout
    int64_t lse_strides[4]; // lse_acc strides in elements: batch, head, split, row
    int64_t o_strides[4];   // o_acc strides in elements: batch, head, split, row (hdim is contiguous)
};
int launch_combine(const CombineParams& p, cudaStream_t stream);

// ---- append-KV (appendkv.cu) --------------------------------------------------------------------
struct AppendKVParams {
    void* q;
    void* k_cache;
    const void* knew;
    void* v_cache;
    const void* vnew;
    const int32_t* seqlen_k;
    const int64_t* seqstart_q;     // group mode or nullptr
    const int64_t* seqstart_knew;  // group mode or nullptr
    const void* rotary_cos;
    const void* rotary_sin;
    const int32_t* block_table;  // nullptr => contiguous cache
    const int64_t* cache_batch_idx;
    int64_t batch, seqlen_q, seqlen_k_cap, seqlen_knew;  // group mode: seqlen_q / seqlen_knew are totals
    int64_t hq, hkv, d, dv, rotary_dim, bt_stride, page;
    int rope_type;
    int dtype;
};
int launch_appendkv(const AppendKVParams& p, cudaStream_t stream);

// ---- split-KV decode over contiguous / paged K,V (splitkv_decode.cu) -----------------------------
struct SplitKVParams {
    const void* q;
    const void* k;
    const void* v;
    float* o_acc;
    float* lse_acc;  // may be nullptr when num_splits == 1
    const int64_t* seqstart_q;
    const int64_t* seqstart_k;
    const int32_t* seqlen_k;
    const int32_t* block_table;
    const int64_t* cache_batch_idx;
    int64_t batch, seqlen_q, seqlen_k_cap, hq, hkv, d, dv, max_seqlen_q, num_splits;
    int64_t total_q;    // rows of the q token axis (batch mode: seqlen_q; group mode: seqstart_q[batch])
    int64_t num_pages;  // paged: pool pages; contiguous: batch rows of the cache (or 0 if unknown)
    int64_t bt_stride, page;
    float scale;
    int mask_type;
    int64_t wl, wr;
    int dtype;
    // ALiBi (bias_enum 2 of the reference's schema): fp32 slopes [1,hq] (rank 0) or [batch,hq] (rank 1), or nullptr;
    // the score of query i and key j gets -slope * |i + sk - sq - j| added
    const float* alibi_slopes;
    int alibi_rank;
};
int launch_splitkv_decode(const SplitKVParams& p, cudaStream_t stream);
// instance parameters (see FlashckSetInstanceParam): "stages", "ctas_per_sm_x100" ...
int splitkv_set_param(const char* key, int64_t value);
int splitkv_get_param(const char* key, int64_t* value);

// ---- generic forward / prefill (fmha_fwd_generic.cu): mma.sync tiles, any mask, varlen, paged ----
struct FwdParams {
    const void* q;
    const void* k;
    const void* v;
    void* o;
    float* lse;  // may be nullptr
    const int64_t* seqstart_q;
    const int64_t* seqstart_k;
    const int64_t* seqlen_k64;   // FmhaFwd: int64 per-batch key lengths (optional)
    const int32_t* seqlen_k32;   // paged prefill: int32 per-batch key lengths
    const int32_t* block_table;  // [batch, bt_stride] page ids, or nullptr
    const int32_t* kv_indptr;    // SGLang-style page table (batch prefill) or nullptr
    const int32_t* kv_page_indices;
    const int32_t* kv_last_page_len;
    const int64_t* cache_batch_idx;
    int64_t batch, seqlen_q, seqlen_k, hq, hkv, d, dv, max_seqlen_q;
    int64_t total_q;
    int64_t bt_stride, page;
    int64_t num_pages;  // paged: token-slot pages in the K/V pools (0 if unknown)
    float scale;
    int mask_type;
    int64_t wl, wr;
    int dtype;
    // Additions to the scaled scores before the mask (attention_kernels/fmha_fwd/fmha_fwd_jinja.h:76,98-112,199-233):
    // bias_type 1: `bias` holds element-dtype values, rank 0 = [1,1,sq,sk], 1 = [1,hq,sq,sk], 2 = [b,hq,sq,sk] (group
    // mode: sq, sk are the packed totals and a sequence's block starts at its first packed row and key);
    // bias_type 2 (ALiBi): `bias` holds fp32 slopes, rank 0 = [1,hq], 1 = [b,hq]; score += -slope * |i + sk - sq - j|.
    // logits_soft_cap > 0: score = cap * tanh(score / cap) on the scaled score, before the bias.
    const void* bias;
    int bias_type, bias_rank;
    float logits_soft_cap;
    // 8-bit element types (dtype 1 / 2): static-quantisation scales of P and O, and the type O is stored in
    float scale_p = 1.f, scale_o = 1.f;
    int out_dtype = 0;
};
int launch_fwd_generic(const FwdParams& p, cudaStream_t stream);

// ---- tcgen05 prefill (fmha_fwd_sm100.cu): hdim 128, contiguous or paged K/V ------------------------------
bool fwd_sm100_supported(const FwdParams& p);
int launch_fwd_sm100(const FwdParams& p, cudaStream_t stream);
// the same kernel as a split-KV backend for several query rows per kv head (partials into the caller's workspaces)
bool splitkv_sm100_supported(const SplitKVParams& p);
int launch_splitkv_sm100(const SplitKVParams& p, cudaStream_t stream);
int fwd_set_param(const char* key, int64_t value);
int fwd_get_param(const char* key, int64_t* value);

}  // namespace fck
