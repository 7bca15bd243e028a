// flashck/fmha/fmha_fwd.h -- C++ operator API of the attention path (header only, over the C ABI).
//
// The reference reserves this header (include/flashck/fmha/fmha_fwd.h is an empty file) and shows the intended
// shape with its norm operators: `namespace flashck::naive { template<class T> T* <op>_fwd(T* device ptrs, dims,
// params) }`, throwing on failure (include/flashck/norm/layer_norm.h:30-77).  The parameter set follows
// `AttentionLayer<T>` (core/module/layers/attention_layers/attention_layer.h:13-33): mode, head counts, head
// dims, scale, window, mask, and the optional seqstart / seqlen arrays of group mode.  Unlike the norm operators
// the output buffer is caller-provided (the reference returns a pointer into its graph-owned pool).
// T is `_Float16`/`__half` (DataType::FLOAT16) or `unsigned short`/`__nv_bfloat16` (DataType::BFLOAT16), as in
// `template class AttentionLayer<ushort>; template class AttentionLayer<_Float16>;` (attention_layer.cc:67-68).
#pragma once

#include <array>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <type_traits>

#include "../../flashck_b200.h"

namespace flashck {

enum class FmhaOperationMode : int { Batch = 0, Group = 1 };
// values of core/profiling/attention/fmha_library.h:81-87, :121-126, :195-200
enum class GenericAttentionMaskEnum : int { NO_MASK = 0, MASK_FROM_TOP_LEFT = 1, MASK_FROM_BOTTOM_RIGHT = 2, MASK_GENERIC = 3 };
enum class BiasEnum : int { NO_BIAS = 0, ELEMENTWISE_BIAS = 1, ALIBI = 2 };
enum class RopeEnum : int { NONE = 0, INTERLEAVED = 1, HALF_ROTATED = 2 };

namespace detail {
template <typename T>
constexpr int dtype_code() {
    static_assert(sizeof(T) == 2, "attention supports 16-bit element types only");
    // 16-bit integer carriers mean bfloat16 (the reference uses `ushort` for bf16); everything else is float16
    return std::is_integral<T>::value ? FLASHCK_DTYPE_BFLOAT16 : FLASHCK_DTYPE_FLOAT16;
}
inline void check(int rc, const char* what) {
    if (rc != FLASHCK_OK) throw std::runtime_error(std::string(what) + " failed: " + FlashckGetLastError());
}
}  // namespace detail

// Tag type for callers whose bf16 type is not an integer carrier (e.g. __nv_bfloat16): pass dtype explicitly.
struct Bf16Tag {};

namespace naive {

// Dense (batch mode) or varlen (group mode: seqstart_q / seqstart_k non-null) forward attention.  Returns `o`.
template <typename T>
T* fmha_fwd(T* q, T* k, T* v, T* o, float* lse, int64_t* seqstart_q, int64_t* seqstart_k, int64_t* seqlen_k,
            int64_t batch, int64_t seqlen_q, int64_t seqlen_k_max, int64_t q_num_heads, int64_t kv_num_heads,
            int64_t qk_head_dim, int64_t v_head_dim, int64_t max_seqlen_q, float scale = 0.f,
            std::array<int64_t, 2> window_size = {-1, -1},
            GenericAttentionMaskEnum mask = GenericAttentionMaskEnum::NO_MASK, void* stream = nullptr,
            int dtype = detail::dtype_code<T>()) {
    detail::check(FmhaFwd(q, k, v, nullptr, o, seqstart_q, seqstart_k, seqlen_k, batch, seqlen_q, seqlen_k_max,
                          q_num_heads, kv_num_heads, qk_head_dim, v_head_dim, max_seqlen_q, scale, window_size[0],
                          window_size[1], static_cast<uint32_t>(mask), stream, lse, dtype),
                  "fmha_fwd");
    return o;
}

// The same with the score additions of the reference's instance schema: `bias` is an elementwise bias in T
// (bias_rank_info 0 = [1,1,sq,sk], 1 = [1,hq,sq,sk], 2 = [b,hq,sq,sk]) or fp32 ALiBi slopes (0 = [1,hq], 1 = [b,hq]),
// as `bias_enum` says; logits_soft_cap > 0 caps the scaled scores first.  Returns `o`.
template <typename T>
T* fmha_fwd_bias(T* q, T* k, T* v, const void* bias, BiasEnum bias_enum, int bias_rank_info, float logits_soft_cap, T* o,
                 float* lse, int64_t* seqstart_q, int64_t* seqstart_k, int64_t* seqlen_k, int64_t batch, int64_t seqlen_q,
                 int64_t seqlen_k_max, int64_t q_num_heads, int64_t kv_num_heads, int64_t qk_head_dim, int64_t v_head_dim,
                 int64_t max_seqlen_q, float scale = 0.f, std::array<int64_t, 2> window_size = {-1, -1},
                 GenericAttentionMaskEnum mask = GenericAttentionMaskEnum::NO_MASK, void* stream = nullptr,
                 int dtype = detail::dtype_code<T>()) {
    detail::check(FmhaFwdBias(q, k, v, const_cast<void*>(bias), o, seqstart_q, seqstart_k, seqlen_k, batch, seqlen_q,
                              seqlen_k_max, q_num_heads, kv_num_heads, qk_head_dim, v_head_dim, max_seqlen_q, scale,
                              window_size[0], window_size[1], static_cast<uint32_t>(mask), stream, lse, dtype,
                              static_cast<int>(bias_enum), bias_rank_info, logits_soft_cap),
                  "fmha_fwd_bias");
    return o;
}

// Varlen (group mode) forward attention on packed tokens: q [total_q, hq, d], k / v [total_k, hkv, d|dv], seqstart_*
// int64 [batch + 1].  The name the reference's test suite gives the operation (tests/pytorch/fmha/
// test_fmha_fwd_var_len.py); same C symbol as fmha_fwd.  Returns `o`.
template <typename T>
T* fmha_fwd_varlen(T* q, T* k, T* v, T* o, float* lse, int64_t* seqstart_q, int64_t* seqstart_k, int64_t batch,
                   int64_t total_q, int64_t total_k, int64_t q_num_heads, int64_t kv_num_heads, int64_t qk_head_dim,
                   int64_t v_head_dim, int64_t max_seqlen_q, float scale = 0.f, std::array<int64_t, 2> window_size = {-1, -1},
                   GenericAttentionMaskEnum mask = GenericAttentionMaskEnum::NO_MASK, void* stream = nullptr,
                   int dtype = detail::dtype_code<T>()) {
    if (seqstart_q == nullptr || seqstart_k == nullptr) throw std::runtime_error("fmha_fwd_varlen: seqstart arrays are required");
    return fmha_fwd<T>(q, k, v, o, lse, seqstart_q, seqstart_k, nullptr, batch, total_q, total_k, q_num_heads, kv_num_heads,
                       qk_head_dim, v_head_dim, max_seqlen_q, scale, window_size, mask, stream, dtype);
}

// Varlen prefill over an SGLang-style page table (fmha_fwd_batch_prefill): K/V pools [num_total_pages, page, hkv, d|dv],
// kv_indptr int32 [batch + 1], kv_page_indices int32, kv_last_page_len int32 [batch]; `alibi_slopes` (fp32, rank 0 =
// [1,hq], 1 = [batch,hq]) or nullptr.  Returns `o`.
template <typename T>
T* fmha_batch_prefill(T* q, T* k_pool, T* v_pool, T* o, float* lse, int64_t* seqstart_q, int32_t* kv_indptr,
                      int32_t* kv_page_indices, int32_t* kv_last_page_len, int64_t batch, int64_t total_q,
                      int64_t q_num_heads, int64_t kv_num_heads, int64_t qk_head_dim, int64_t v_head_dim,
                      int64_t max_seqlen_q, int64_t num_total_pages, int64_t page_block_size, float scale = 0.f,
                      std::array<int64_t, 2> window_size = {-1, 0},
                      GenericAttentionMaskEnum mask = GenericAttentionMaskEnum::MASK_FROM_BOTTOM_RIGHT,
                      const float* alibi_slopes = nullptr, int alibi_rank = 0, void* stream = nullptr,
                      int dtype = detail::dtype_code<T>()) {
    detail::check(FmhaFwdBatchPrefillEx(q, k_pool, v_pool, const_cast<float*>(alibi_slopes), o, seqstart_q, kv_indptr,
                                        kv_page_indices, kv_last_page_len, batch, total_q, q_num_heads, kv_num_heads,
                                        qk_head_dim, v_head_dim, max_seqlen_q, num_total_pages, page_block_size, scale,
                                        window_size[0], window_size[1], static_cast<uint32_t>(mask), stream, lse, dtype,
                                        alibi_slopes ? 2 : 0, alibi_rank),
                  "fmha_batch_prefill");
    return o;
}

// Prefill reading K/V through a block table (fmha_fwd_paged_kv_prefill): pools [num_pool_pages, page, hkv, d|dv],
// block_table int32 [batch, pages_per_seq], seqlen_k int32 [batch]; q in batch mode or packed with seqstart_q.
// Returns `o`.
template <typename T>
T* fmha_fwd_paged_kv_prefill(T* q, T* k_pool, T* v_pool, T* o, float* lse, int64_t* seqstart_q, int32_t* seqlen_k,
                             int32_t* block_table, int64_t* cache_batch_idx, int64_t batch, int64_t seqlen_q,
                             int64_t q_num_heads, int64_t kv_num_heads, int64_t qk_head_dim, int64_t v_head_dim,
                             int64_t max_seqlen_q, int64_t pages_per_seq, int64_t num_pool_pages, int64_t page_block_size,
                             float scale = 0.f, std::array<int64_t, 2> window_size = {-1, 0},
                             GenericAttentionMaskEnum mask = GenericAttentionMaskEnum::MASK_FROM_BOTTOM_RIGHT,
                             const float* alibi_slopes = nullptr, int alibi_rank = 0, void* stream = nullptr,
                             int dtype = detail::dtype_code<T>()) {
    detail::check(FmhaFwdPagedKVPrefillEx(q, k_pool, v_pool, const_cast<float*>(alibi_slopes), o, seqstart_q, seqlen_k,
                                          block_table, cache_batch_idx, batch, seqlen_q, q_num_heads, kv_num_heads,
                                          qk_head_dim, v_head_dim, max_seqlen_q, batch * pages_per_seq, page_block_size,
                                          scale, window_size[0], window_size[1], static_cast<uint32_t>(mask), stream, lse,
                                          dtype, alibi_slopes ? 2 : 0, alibi_rank, num_pool_pages),
                  "fmha_fwd_paged_kv_prefill");
    return o;
}

// Split-KV attention over a contiguous or paged cache followed by the combine.  Workspaces are caller-owned:
// lse_acc [b,hq,num_splits,sq], o_acc [b,hq,num_splits,sq,dv] fp32.  Returns `o`.
template <typename T>
T* fmha_fwd_splitkv(T* q, T* k_cache, T* v_cache, T* o, float* lse, float* lse_acc, float* o_acc, int64_t* seqstart_q,
                    int64_t* seqstart_k, int32_t* seqlen_k, int32_t* block_table, int64_t* cache_batch_idx,
                    int64_t batch, int64_t seqlen_q, int64_t seqlen_k_max, int64_t q_num_heads, int64_t kv_num_heads,
                    int64_t qk_head_dim, int64_t v_head_dim, int64_t max_seqlen_q, int64_t num_splits,
                    int64_t max_num_page_blocks, int64_t page_block_size, float scale = 0.f,
                    std::array<int64_t, 2> window_size = {-1, -1},
                    GenericAttentionMaskEnum mask = GenericAttentionMaskEnum::NO_MASK, void* stream = nullptr,
                    int dtype = detail::dtype_code<T>(), int64_t num_pool_pages = 0) {
    // num_pool_pages: pages the pools really hold (0 = max_num_page_blocks, the reference's pool size)
    detail::check(FmhaFwdSplitKVEx(q, k_cache, v_cache, nullptr, lse_acc, o_acc, seqstart_q, seqstart_k, seqlen_k,
                                   block_table, cache_batch_idx, batch, seqlen_q, seqlen_k_max, q_num_heads, kv_num_heads,
                                   qk_head_dim, v_head_dim, max_seqlen_q, num_splits, max_num_page_blocks, page_block_size,
                                   scale, window_size[0], window_size[1], static_cast<uint32_t>(mask), stream, dtype, 0, 0,
                                   num_pool_pages > 0 ? num_pool_pages : max_num_page_blocks),
                  "fmha_fwd_splitkv");
    detail::check(FmhaFwdSplitKVCombine(lse_acc, o_acc, o, seqstart_q, batch, seqlen_q, q_num_heads, v_head_dim,
                                        max_seqlen_q, num_splits, stream, lse, dtype),
                  "fmha_fwd_splitkv_combine");
    return o;
}

// RoPE on q (in place) and the new keys, then the K/V cache write.  Returns `q`.
template <typename T>
T* fmha_fwd_appendkv(T* q, T* k_cache, T* knew, T* v_cache, T* vnew, int32_t* seqlen_k, int64_t* seqstart_q,
                     int64_t* seqstart_knew, T* rotary_cos, T* rotary_sin, int32_t* block_table,
                     int64_t* cache_batch_idx, int64_t batch, int64_t seqlen_q, int64_t seqlen_k_capacity,
                     int64_t seqlen_knew, int64_t q_num_heads, int64_t kv_num_heads, int64_t qk_head_dim,
                     int64_t v_head_dim, int64_t rotary_dim, RopeEnum rope, int64_t max_num_page_blocks,
                     int64_t page_block_size, void* stream = nullptr, int dtype = detail::dtype_code<T>()) {
    detail::check(FmhaFwdAppendKV(q, k_cache, knew, v_cache, vnew, seqlen_k, seqstart_q, seqstart_knew, rotary_cos,
                                  rotary_sin, block_table, cache_batch_idx, batch, seqlen_q, seqlen_k_capacity,
                                  seqlen_knew, q_num_heads, kv_num_heads, qk_head_dim, v_head_dim, rotary_dim,
                                  static_cast<int>(rope), max_num_page_blocks, page_block_size, stream, dtype),
                  "fmha_fwd_appendkv");
    return q;
}

}  // namespace naive

// Layer facade with the reference's constructor and call parameters (attention_layer.h:13-33), over raw device
// pointers instead of graph `Variable*`s: the graph runtime is outside the attention path.
template <typename T>
class AttentionLayer {
public:
    AttentionLayer(FmhaOperationMode mode, int64_t q_num_heads, int64_t kv_num_heads, int64_t qk_head_dim,
                   int64_t v_head_dim, float scale = 1.0f, BiasEnum bias_enum = BiasEnum::NO_BIAS,
                   std::array<int64_t, 2> window_size = {-1, -1},
                   GenericAttentionMaskEnum mask_enum = GenericAttentionMaskEnum::NO_MASK)
        : mode_(mode), q_num_heads_(q_num_heads), kv_num_heads_(kv_num_heads), qk_head_dim_(qk_head_dim),
          v_head_dim_(v_head_dim), scale_(scale), bias_enum_(bias_enum), window_size_(window_size),
          mask_enum_(mask_enum) {
        if (mode != FmhaOperationMode::Batch && mode != FmhaOperationMode::Group)
            throw std::runtime_error("fmha only supports Batch && group mode");
    }

    // q [batch, q_seq_len, q_num_heads, qk_head_dim] (group mode: packed [total_q, ...] with q_seq_len = total_q);
    // seqstart_q / seqstart_k [batch+1] and seqlen_k [batch] only in group mode.  `bias` is read as the layer's
    // bias_enum says: ELEMENTWISE_BIAS -> values of type T, bias_rank_info 0 = [1,1,sq,sk], 1 = [1,hq,sq,sk],
    // 2 = [b,hq,sq,sk]; ALIBI -> fp32 slopes, 0 = [1,hq], 1 = [b,hq].  `out` receives O; returns it.
    T* operator()(T* q, T* k, T* v, T* out, int64_t batch, int64_t q_seq_len, int64_t kv_seq_len, int64_t max_seqlen_q,
                  const void* bias = nullptr, int64_t* seqstart_q = nullptr, int64_t* seqstart_k = nullptr,
                  int64_t* seqlen_k = nullptr, float* lse = nullptr, void* stream = nullptr, int bias_rank_info = 0,
                  float logits_soft_cap = 0.f, int dtype = detail::dtype_code<T>()) const {
        if ((bias != nullptr) != (bias_enum_ != BiasEnum::NO_BIAS))
            throw std::runtime_error("AttentionLayer: a bias buffer goes with a bias_enum other than NO_BIAS, and only with one");
        const bool group = mode_ == FmhaOperationMode::Group;
        return naive::fmha_fwd_bias<T>(q, k, v, bias, bias_enum_, bias_rank_info, logits_soft_cap, out, lse,
                                       group ? seqstart_q : nullptr, group ? seqstart_k : nullptr, group ? seqlen_k : nullptr,
                                       batch, q_seq_len, kv_seq_len, q_num_heads_, kv_num_heads_, qk_head_dim_, v_head_dim_,
                                       max_seqlen_q, scale_, window_size_, mask_enum_, stream, dtype);
    }

    FmhaOperationMode mode_;
    int64_t q_num_heads_, kv_num_heads_, qk_head_dim_, v_head_dim_;
    float scale_;
    BiasEnum bias_enum_;
    std::array<int64_t, 2> window_size_;
    GenericAttentionMaskEnum mask_enum_;
};

}  // namespace flashck
