// Compiled PyTorch binding `flash_ck` of the attention path.
//
// Mirrors the reference's binding layer: a pybind11 torch extension named `flash_ck` (core/pybind/CMakeLists.txt:14-15,
// core/pybind/pybind.cc:13-58) whose functions take at::Tensor, validate with TORCH_CHECK (-> Python RuntimeError),
// dispatch on the element type to the C++ operator API `flashck::naive::<op><T>` with the reference's carrier types
// (`_Float16` for fp16, `ushort` for bf16; core/pybind/norm/layer_norm.h:10-74) and return at::Tensor; the enums of
// core/pybind/pybind_helper.h:3-29 plus the attention ones; and the flag API of pybind.cc:21-45.  The operator API in
// turn is a header over the C ABI of libflashck_b200.so, so a call here runs:  Python -> this module ->
// include/flashck/fmha/fmha_fwd.h -> extern "C" symbol -> CUDA kernel on the current torch stream.
// Outputs are allocated by torch (the caller's allocator); the library itself allocates nothing.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <optional>
#include <tuple>

#include "flashck/fmha/fmha_fwd.h"

namespace py = pybind11;

namespace flashck {
namespace pytorch {

using OptTensor = std::optional<at::Tensor>;
typedef unsigned short ushort_t;  // the reference's carrier type for bfloat16

namespace {

void check_cuda(const at::Tensor& t, const char* name) {
    TORCH_CHECK(t.defined(), name, " is undefined");
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
void check_elem(const at::Tensor& t, const char* name, at::ScalarType want) {
    check_cuda(t, name);
    TORCH_CHECK(t.scalar_type() == want, name, " must have dtype ", want, ", got ", t.scalar_type());
}
at::ScalarType elem_type(const at::Tensor& q) {
    TORCH_CHECK(q.scalar_type() == at::kHalf || q.scalar_type() == at::kBFloat16,
                "attention supports float16 and bfloat16, got ", q.scalar_type());
    return q.scalar_type();
}
template <typename T>
T* ptr(const at::Tensor& t) { return reinterpret_cast<T*>(t.data_ptr()); }
template <typename T>
T* ptr(const OptTensor& t) { return t.has_value() ? reinterpret_cast<T*>(t->data_ptr()) : nullptr; }
void* stream() { return (void*)at::cuda::getCurrentCUDAStream().stream(); }

// (mask_type, left, right): causal = bottom-right aligned window (-1, 0); an explicit mask_type wins
std::tuple<GenericAttentionMaskEnum, int64_t, int64_t> resolve_mask(bool causal, int64_t wl, int64_t wr, int64_t mask_type) {
    if (mask_type >= 0) {
        TORCH_CHECK(mask_type <= 3, "mask_type must be 0..3");
        return {static_cast<GenericAttentionMaskEnum>(mask_type), wl, causal ? 0 : wr};
    }
    if (causal) return {GenericAttentionMaskEnum::MASK_FROM_BOTTOM_RIGHT, wl, 0};
    if (wl >= 0 || wr >= 0) return {GenericAttentionMaskEnum::MASK_FROM_BOTTOM_RIGHT, wl, wr};
    return {GenericAttentionMaskEnum::NO_MASK, -1, -1};
}

// Runs `fn.template operator()<T>()` with T = _Float16 or ushort by the tensor's element type.
#define FC_DISPATCH_ELEM(TYPE, ...)                                  \
    do {                                                             \
        if ((TYPE) == at::kHalf) { using T = _Float16; __VA_ARGS__; } \
        else { using T = ushort_t; __VA_ARGS__; }                    \
    } while (0)

}  // namespace

// Dense forward attention.  q [b,sq,hq,d], k [b,sk,hkv,d], v [b,sk,hkv,dv] -> (o [b,sq,hq,dv], lse [b,hq,sq] fp32).
// bias: [1|b, 1|hq, sq, sk] in q's dtype; alibi_slopes: fp32 [1|b, hq]; logits_soft_cap > 0 caps the scaled scores.
std::tuple<at::Tensor, at::Tensor> fmha_fwd(at::Tensor q, at::Tensor k, at::Tensor v, double scale, bool causal,
                                            int64_t window_left, int64_t window_right, int64_t mask_type, OptTensor bias,
                                            OptTensor alibi_slopes, double logits_soft_cap) {
    const auto et = elem_type(q);
    check_elem(q, "q", et); check_elem(k, "k", et); check_elem(v, "v", et);
    TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q, k, v must be [batch, seqlen, heads, hdim]");
    const int64_t b = q.size(0), sq = q.size(1), hq = q.size(2), d = q.size(3);
    const int64_t sk = k.size(1), hkv = k.size(2), dv = v.size(3);
    TORCH_CHECK(k.size(0) == b && v.size(0) == b && v.size(1) == sk && v.size(2) == hkv && k.size(3) == d,
                "inconsistent shapes q", q.sizes(), " k", k.sizes(), " v", v.sizes());
    TORCH_CHECK(!(bias.has_value() && alibi_slopes.has_value()), "bias and alibi_slopes are mutually exclusive");
    BiasEnum be = BiasEnum::NO_BIAS;
    int rank = 0;
    const void* bias_ptr = nullptr;
    if (bias.has_value()) {
        check_elem(*bias, "bias", et);
        TORCH_CHECK(bias->dim() == 4 && bias->size(2) == sq && bias->size(3) == sk && (bias->size(0) == 1 || bias->size(0) == b) &&
                        (bias->size(1) == 1 || bias->size(1) == hq) && (bias->size(0) == 1 || bias->size(1) == hq),
                    "bias must be [1|b, 1|hq, sq, sk] with a full head axis under a batch axis, got ", bias->sizes());
        be = BiasEnum::ELEMENTWISE_BIAS;
        rank = (bias->size(0) == 1 && bias->size(1) == 1) ? 0 : (bias->size(0) == 1 ? 1 : 2);
        bias_ptr = bias->data_ptr();
    } else if (alibi_slopes.has_value()) {
        check_elem(*alibi_slopes, "alibi_slopes", at::kFloat);
        TORCH_CHECK(alibi_slopes->dim() == 2 && alibi_slopes->size(1) == hq && (alibi_slopes->size(0) == 1 || alibi_slopes->size(0) == b),
                    "alibi_slopes must be fp32 [1|b, hq], got ", alibi_slopes->sizes());
        be = BiasEnum::ALIBI;
        rank = alibi_slopes->size(0) == 1 ? 0 : 1;
        bias_ptr = alibi_slopes->data_ptr();
    }
    auto [mask, wl, wr] = resolve_mask(causal, window_left, window_right, mask_type);
    c10::cuda::CUDAGuard guard(q.device());
    at::Tensor o = at::empty({b, sq, hq, dv}, q.options());
    at::Tensor lse = at::empty({b, hq, sq}, q.options().dtype(at::kFloat));
    FC_DISPATCH_ELEM(et, naive::fmha_fwd_bias<T>(ptr<T>(q), ptr<T>(k), ptr<T>(v), bias_ptr, be, rank, (float)logits_soft_cap,
                                                 ptr<T>(o), ptr<float>(lse), nullptr, nullptr, nullptr, b, sq, sk, hq, hkv, d,
                                                 dv, sq, (float)scale, {wl, wr}, mask, stream(),
                                                 et == at::kHalf ? FLASHCK_DTYPE_FLOAT16 : FLASHCK_DTYPE_BFLOAT16));
    return {o, lse};
}

// Varlen forward attention on packed tokens.  q [total_q,hq,d], k/v [total_k,hkv,*], cu_seqlens int64 [b+1]
// -> (o [total_q,hq,dv], lse [hq,total_q]).
std::tuple<at::Tensor, at::Tensor> fmha_fwd_varlen(at::Tensor q, at::Tensor k, at::Tensor v, at::Tensor cu_seqlens_q,
                                                   at::Tensor cu_seqlens_k, int64_t max_seqlen_q, double scale, bool causal,
                                                   int64_t window_left, int64_t window_right, int64_t mask_type) {
    const auto et = elem_type(q);
    check_elem(q, "q", et); check_elem(k, "k", et); check_elem(v, "v", et);
    check_elem(cu_seqlens_q, "cu_seqlens_q", at::kLong); check_elem(cu_seqlens_k, "cu_seqlens_k", at::kLong);
    TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "q, k, v must be packed [total_tokens, heads, hdim]");
    TORCH_CHECK(cu_seqlens_q.numel() == cu_seqlens_k.numel() && cu_seqlens_q.numel() >= 2,
                "cu_seqlens_q and cu_seqlens_k must both have batch + 1 entries");
    const int64_t batch = cu_seqlens_q.numel() - 1, total_q = q.size(0), hq = q.size(1), d = q.size(2);
    const int64_t total_k = k.size(0), hkv = k.size(1), dv = v.size(2);
    TORCH_CHECK(k.size(2) == d && v.size(0) == total_k && v.size(1) == hkv, "inconsistent shapes q", q.sizes(), " k", k.sizes(),
                " v", v.sizes());
    auto [mask, wl, wr] = resolve_mask(causal, window_left, window_right, mask_type);
    c10::cuda::CUDAGuard guard(q.device());
    at::Tensor o = at::empty({total_q, hq, dv}, q.options());
    at::Tensor lse = at::empty({hq, total_q}, q.options().dtype(at::kFloat));
    FC_DISPATCH_ELEM(et, naive::fmha_fwd_varlen<T>(ptr<T>(q), ptr<T>(k), ptr<T>(v), ptr<T>(o), ptr<float>(lse),
                                                   ptr<int64_t>(cu_seqlens_q), ptr<int64_t>(cu_seqlens_k), batch, total_q,
                                                   total_k, hq, hkv, d, dv, max_seqlen_q, (float)scale, {wl, wr}, mask, stream(),
                                                   et == at::kHalf ? FLASHCK_DTYPE_FLOAT16 : FLASHCK_DTYPE_BFLOAT16));
    return {o, lse};
}

// Varlen prefill over an SGLang-style page table.  Pools [pages, page, hkv, d|dv]; kv_indptr int32 [b+1],
// kv_page_indices int32, kv_last_page_len int32 [b].
std::tuple<at::Tensor, at::Tensor> fmha_batch_prefill(at::Tensor q, at::Tensor k_pool, at::Tensor v_pool, at::Tensor cu_seqlens_q,
                                                      at::Tensor kv_indptr, at::Tensor kv_page_indices,
                                                      at::Tensor kv_last_page_len, int64_t max_seqlen_q, double scale,
                                                      bool causal, int64_t window_left, int64_t window_right,
                                                      int64_t mask_type) {
    const auto et = elem_type(q);
    check_elem(q, "q", et); check_elem(k_pool, "k_pool", et); check_elem(v_pool, "v_pool", et);
    check_elem(cu_seqlens_q, "cu_seqlens_q", at::kLong);
    check_elem(kv_indptr, "kv_indptr", at::kInt); check_elem(kv_page_indices, "kv_page_indices", at::kInt);
    check_elem(kv_last_page_len, "kv_last_page_len", at::kInt);
    TORCH_CHECK(q.dim() == 3 && k_pool.dim() == 4 && v_pool.dim() == 4, "q must be [total_q, hq, d]; pools [pages, page, hkv, hdim]");
    const int64_t batch = cu_seqlens_q.numel() - 1, total_q = q.size(0), hq = q.size(1), d = q.size(2);
    TORCH_CHECK(batch >= 1 && kv_indptr.numel() == batch + 1 && kv_last_page_len.numel() == batch,
                "kv_indptr must have batch + 1 entries and kv_last_page_len batch entries");
    const int64_t pages = k_pool.size(0), page = k_pool.size(1), hkv = k_pool.size(2), dv = v_pool.size(3);
    TORCH_CHECK(k_pool.size(3) == d && v_pool.size(0) == pages && v_pool.size(1) == page && v_pool.size(2) == hkv,
                "inconsistent pool shapes k", k_pool.sizes(), " v", v_pool.sizes());
    auto [mask, wl, wr] = resolve_mask(causal, window_left, window_right, mask_type);
    c10::cuda::CUDAGuard guard(q.device());
    at::Tensor o = at::empty({total_q, hq, dv}, q.options());
    at::Tensor lse = at::empty({hq, total_q}, q.options().dtype(at::kFloat));
    FC_DISPATCH_ELEM(et, naive::fmha_batch_prefill<T>(ptr<T>(q), ptr<T>(k_pool), ptr<T>(v_pool), ptr<T>(o), ptr<float>(lse),
                                                      ptr<int64_t>(cu_seqlens_q), ptr<int32_t>(kv_indptr),
                                                      ptr<int32_t>(kv_page_indices), ptr<int32_t>(kv_last_page_len), batch,
                                                      total_q, hq, hkv, d, dv, max_seqlen_q, pages, page, (float)scale, {wl, wr},
                                                      mask, nullptr, 0, stream(),
                                                      et == at::kHalf ? FLASHCK_DTYPE_FLOAT16 : FLASHCK_DTYPE_BFLOAT16));
    return {o, lse};
}

// Prefill through a block table.  q [b,sq,hq,d] (or packed [total_q,hq,d] with cu_seqlens_q); block_table int32
// [b, pages_per_seq]; seqlen_k int32 [b].
std::tuple<at::Tensor, at::Tensor> fmha_fwd_paged_kv_prefill(at::Tensor q, at::Tensor k_pool, at::Tensor v_pool,
                                                             at::Tensor block_table, at::Tensor seqlen_k, OptTensor cu_seqlens_q,
                                                             int64_t max_seqlen_q, double scale, bool causal,
                                                             int64_t window_left, int64_t window_right, int64_t mask_type) {
    const auto et = elem_type(q);
    check_elem(q, "q", et); check_elem(k_pool, "k_pool", et); check_elem(v_pool, "v_pool", et);
    check_elem(block_table, "block_table", at::kInt); check_elem(seqlen_k, "seqlen_k", at::kInt);
    TORCH_CHECK(k_pool.dim() == 4 && v_pool.dim() == 4 && block_table.dim() == 2, "pools [pages, page, hkv, hdim]; block_table [b, pages_per_seq]");
    const bool group = cu_seqlens_q.has_value();
    const int64_t batch = block_table.size(0);
    int64_t shape_sq, max_sq, hq, d;
    std::vector<int64_t> o_shape, lse_shape;
    const int64_t dv = v_pool.size(3);
    if (group) {
        check_elem(*cu_seqlens_q, "cu_seqlens_q", at::kLong);
        TORCH_CHECK(q.dim() == 3 && cu_seqlens_q->numel() == batch + 1, "packed q must be [total_q, hq, d] with batch + 1 offsets");
        shape_sq = q.size(0); hq = q.size(1); d = q.size(2);
        max_sq = max_seqlen_q > 0 ? max_seqlen_q : shape_sq;
        o_shape = {shape_sq, hq, dv}; lse_shape = {hq, shape_sq};
    } else {
        TORCH_CHECK(q.dim() == 4 && q.size(0) == batch, "q must be [b, sq, hq, d] with one row of block_table per sequence");
        shape_sq = q.size(1); hq = q.size(2); d = q.size(3);
        max_sq = shape_sq;
        o_shape = {batch, shape_sq, hq, dv}; lse_shape = {batch, hq, shape_sq};
    }
    TORCH_CHECK(seqlen_k.numel() == batch && k_pool.size(3) == d, "seqlen_k must have batch entries; k_pool hdim must match q");
    auto [mask, wl, wr] = resolve_mask(causal, window_left, window_right, mask_type);
    c10::cuda::CUDAGuard guard(q.device());
    at::Tensor o = at::empty(o_shape, q.options());
    at::Tensor lse = at::empty(lse_shape, q.options().dtype(at::kFloat));
    FC_DISPATCH_ELEM(et, naive::fmha_fwd_paged_kv_prefill<T>(
                             ptr<T>(q), ptr<T>(k_pool), ptr<T>(v_pool), ptr<T>(o), ptr<float>(lse), ptr<int64_t>(cu_seqlens_q),
                             ptr<int32_t>(seqlen_k), ptr<int32_t>(block_table), nullptr, batch, shape_sq, hq, k_pool.size(2), d, dv,
                             max_sq, block_table.size(1), k_pool.size(0), k_pool.size(1), (float)scale, {wl, wr}, mask, nullptr, 0,
                             stream(), et == at::kHalf ? FLASHCK_DTYPE_FLOAT16 : FLASHCK_DTYPE_BFLOAT16));
    return {o, lse};
}

// Split-KV attention (decode) over a paged or contiguous cache, followed by the combine.  Workspaces come from torch.
std::tuple<at::Tensor, at::Tensor> fmha_fwd_splitkv(at::Tensor q, at::Tensor k_cache, at::Tensor v_cache, OptTensor seqlen_k,
                                                    OptTensor block_table, int64_t num_splits, double scale, bool causal) {
    const auto et = elem_type(q);
    check_elem(q, "q", et); check_elem(k_cache, "k_cache", et); check_elem(v_cache, "v_cache", et);
    TORCH_CHECK(q.dim() == 4 && k_cache.dim() == 4 && v_cache.dim() == 4, "q [b,sq,hq,d]; caches [pages|b, page|sk, hkv, hdim]");
    const int64_t b = q.size(0), sq = q.size(1), hq = q.size(2), d = q.size(3);
    const int64_t hkv = k_cache.size(2), dv = v_cache.size(3);
    TORCH_CHECK(k_cache.size(3) == d, "k_cache hdim differs from q");
    const bool paged = block_table.has_value();
    if (seqlen_k.has_value()) check_elem(*seqlen_k, "seqlen_k", at::kInt);
    int64_t max_pages = 0, page = 0, sk = 0;
    if (paged) {
        check_elem(*block_table, "block_table", at::kInt);
        TORCH_CHECK(seqlen_k.has_value(), "paged K/V needs seqlen_k");
        TORCH_CHECK(block_table->dim() == 2 && block_table->size(0) == b, "block_table must be [b, pages_per_seq]");
        page = k_cache.size(1);
        max_pages = b * block_table->size(1);
    } else {
        TORCH_CHECK(k_cache.size(0) == b, "a contiguous cache must have one row per sequence");
        sk = k_cache.size(1);
    }
    if (num_splits <= 0) num_splits = std::max<int64_t>(2, std::min<int64_t>(128, (2 * 148 + b - 1) / b + 1));
    auto [mask, wl, wr] = resolve_mask(causal, -1, -1, -1);
    c10::cuda::CUDAGuard guard(q.device());
    const auto f32 = q.options().dtype(at::kFloat);
    at::Tensor lse_acc = at::empty({b, hq, num_splits, sq}, f32), o_acc = at::empty({b, hq, num_splits, sq, dv}, f32);
    at::Tensor o = at::empty({b, sq, hq, dv}, q.options()), lse = at::empty({b, hq, sq}, f32);
    FC_DISPATCH_ELEM(et, naive::fmha_fwd_splitkv<T>(ptr<T>(q), ptr<T>(k_cache), ptr<T>(v_cache), ptr<T>(o), ptr<float>(lse),
                                                    ptr<float>(lse_acc), ptr<float>(o_acc), nullptr, nullptr, ptr<int32_t>(seqlen_k),
                                                    ptr<int32_t>(block_table), nullptr, b, sq, sk, hq, hkv, d, dv, sq, num_splits,
                                                    max_pages, page, (float)scale, {wl, wr}, mask, stream(),
                                                    et == at::kHalf ? FLASHCK_DTYPE_FLOAT16 : FLASHCK_DTYPE_BFLOAT16,
                                                    paged ? k_cache.size(0) : 0));
    return {o, lse};
}

// RoPE on q (in place) and on the new keys, then the K/V cache write (paged through block_table, or contiguous).
// Batch mode tensors: q [b,sq,hq,d], knew [b,n,hkv,d], vnew [b,n,hkv,dv]; seqlen_k int32 [b] = cached length before.
at::Tensor fmha_fwd_appendkv(at::Tensor q, at::Tensor k_cache, at::Tensor v_cache, at::Tensor knew, at::Tensor vnew,
                             at::Tensor seqlen_k, OptTensor rotary_cos, OptTensor rotary_sin, int64_t rope, OptTensor block_table) {
    const auto et = elem_type(q);
    check_elem(q, "q", et); check_elem(k_cache, "k_cache", et); check_elem(v_cache, "v_cache", et);
    check_elem(knew, "knew", et); check_elem(vnew, "vnew", et); check_elem(seqlen_k, "seqlen_k", at::kInt);
    TORCH_CHECK(rope >= 0 && rope <= 2, "rope must be 0 (none), 1 (interleaved) or 2 (half-rotated)");
    TORCH_CHECK(rope == 0 || (rotary_cos.has_value() && rotary_sin.has_value()), "rotary tables are required unless rope == 0");
    TORCH_CHECK(q.dim() == 4 && knew.dim() == 4 && vnew.dim() == 4 && k_cache.dim() == 4, "batch-mode tensors [b, s, h, d]");
    const int64_t b = q.size(0), sq = q.size(1), hq = q.size(2), d = q.size(3), n = knew.size(1), hkv = knew.size(2), dv = vnew.size(3);
    TORCH_CHECK(seqlen_k.numel() == b && knew.size(0) == b && vnew.size(0) == b && vnew.size(1) == n, "inconsistent batch / new-token counts");
    int64_t rotary_dim = 0;
    if (rope != 0) {
        check_elem(*rotary_cos, "rotary_cos", et); check_elem(*rotary_sin, "rotary_sin", et);
        rotary_dim = 2 * rotary_cos->size(-1);
    }
    int64_t max_pages = 0, page = 0, cap = 0;
    if (block_table.has_value()) {
        check_elem(*block_table, "block_table", at::kInt);
        TORCH_CHECK(block_table->dim() == 2 && block_table->size(0) == b, "block_table must be [b, pages_per_seq]");
        page = k_cache.size(1);
        max_pages = b * block_table->size(1);
    } else {
        cap = k_cache.size(1);
    }
    c10::cuda::CUDAGuard guard(q.device());
    FC_DISPATCH_ELEM(et, naive::fmha_fwd_appendkv<T>(ptr<T>(q), ptr<T>(k_cache), ptr<T>(knew), ptr<T>(v_cache), ptr<T>(vnew),
                                                     ptr<int32_t>(seqlen_k), nullptr, nullptr, ptr<T>(rotary_cos), ptr<T>(rotary_sin),
                                                     ptr<int32_t>(block_table), nullptr, b, sq, cap, n, hq, hkv, d, dv, rotary_dim,
                                                     static_cast<RopeEnum>(rope), max_pages, page, stream(),
                                                     et == at::kHalf ? FLASHCK_DTYPE_FLOAT16 : FLASHCK_DTYPE_BFLOAT16));
    return q;
}

}  // namespace pytorch

PYBIND11_MODULE(flash_ck, m) {
    m.doc() = "FlashCK attention path for B200 (PyTorch extension over libflashck_b200.so)";

    // enums (core/pybind/pybind_helper.h:3-29 binds DataType; the attention enums follow core/profiling/attention/fmha_library.h)
    py::enum_<GenericAttentionMaskEnum>(m, "MaskEnum")
        .value("NO_MASK", GenericAttentionMaskEnum::NO_MASK)
        .value("MASK_FROM_TOP_LEFT", GenericAttentionMaskEnum::MASK_FROM_TOP_LEFT)
        .value("MASK_FROM_BOTTOM_RIGHT", GenericAttentionMaskEnum::MASK_FROM_BOTTOM_RIGHT)
        .value("MASK_GENERIC", GenericAttentionMaskEnum::MASK_GENERIC);
    py::enum_<BiasEnum>(m, "BiasEnum")
        .value("NO_BIAS", BiasEnum::NO_BIAS)
        .value("ELEMENTWISE_BIAS", BiasEnum::ELEMENTWISE_BIAS)
        .value("ALIBI", BiasEnum::ALIBI);
    py::enum_<RopeEnum>(m, "RopeEnum")
        .value("NONE", RopeEnum::NONE)
        .value("INTERLEAVED", RopeEnum::INTERLEAVED)
        .value("HALF_ROTATED", RopeEnum::HALF_ROTATED);
    py::enum_<FmhaOperationMode>(m, "FmhaOperationMode")
        .value("Batch", FmhaOperationMode::Batch)
        .value("Group", FmhaOperationMode::Group);

    // flag API (core/pybind/pybind.cc:21-45); the registry itself is the package's (flashck_b200.utils.flags)
    m.def("get_flag_value", [](const std::string& name) {
        return py::module_::import("flashck_b200.utils.flags").attr("get_flag_value")(name);
    }, py::arg("name"), "Get flag value as string");
    m.def("set_flag_value", [](const std::string& name, const py::object& value) {
        py::module_::import("flashck_b200.utils.flags").attr("set_flag_value")(name, value);
    }, py::arg("name"), py::arg("value"), "Set flag value by name");
    m.def("print_all_flags", [](bool writable_only) {
        py::module_::import("flashck_b200.utils.flags").attr("print_all_flags")(writable_only);
    }, py::arg("writable_only") = false, "Print all flags to stdout");
    m.def("print_flag_info", [](const std::string& name) {
        py::module_::import("flashck_b200.utils.flags").attr("print_flag_info")(name);
    }, py::arg("name"), "Print detailed info for a flag");
    m.def("version", []() { return std::string(FlashckVersion()); });

    using namespace pybind11::literals;
    m.def("fmha_fwd", &pytorch::fmha_fwd, "Dense forward attention -> (o, lse)", "q"_a, "k"_a, "v"_a, "scale"_a = 0.0,
          "causal"_a = false, "window_left"_a = -1, "window_right"_a = -1, "mask_type"_a = -1, "bias"_a = py::none(),
          "alibi_slopes"_a = py::none(), "logits_soft_cap"_a = 0.0);
    m.def("fmha_fwd_varlen", &pytorch::fmha_fwd_varlen, "Varlen forward attention on packed tokens -> (o, lse)", "q"_a, "k"_a,
          "v"_a, "cu_seqlens_q"_a, "cu_seqlens_k"_a, "max_seqlen_q"_a, "scale"_a = 0.0, "causal"_a = false,
          "window_left"_a = -1, "window_right"_a = -1, "mask_type"_a = -1);
    m.def("fmha_batch_prefill", &pytorch::fmha_batch_prefill, "Varlen prefill over an SGLang-style page table -> (o, lse)",
          "q"_a, "k_pool"_a, "v_pool"_a, "cu_seqlens_q"_a, "kv_indptr"_a, "kv_page_indices"_a, "kv_last_page_len"_a,
          "max_seqlen_q"_a, "scale"_a = 0.0, "causal"_a = true, "window_left"_a = -1, "window_right"_a = -1, "mask_type"_a = -1);
    m.def("fmha_fwd_paged_kv_prefill", &pytorch::fmha_fwd_paged_kv_prefill, "Prefill through a block table -> (o, lse)", "q"_a,
          "k_pool"_a, "v_pool"_a, "block_table"_a, "seqlen_k"_a, "cu_seqlens_q"_a = py::none(), "max_seqlen_q"_a = 0,
          "scale"_a = 0.0, "causal"_a = true, "window_left"_a = -1, "window_right"_a = -1, "mask_type"_a = -1);
    m.def("fmha_fwd_splitkv", &pytorch::fmha_fwd_splitkv, "Split-KV attention + combine -> (o, lse)", "q"_a, "k_cache"_a,
          "v_cache"_a, "seqlen_k"_a = py::none(), "block_table"_a = py::none(), "num_splits"_a = 0, "scale"_a = 0.0,
          "causal"_a = false);
    m.def("fmha_fwd_appendkv", &pytorch::fmha_fwd_appendkv, "RoPE + KV-cache write; returns the rotated q", "q"_a, "k_cache"_a,
          "v_cache"_a, "knew"_a, "vnew"_a, "seqlen_k"_a, "rotary_cos"_a = py::none(), "rotary_sin"_a = py::none(), "rope"_a = 1,
          "block_table"_a = py::none());
}

}  // namespace flashck
