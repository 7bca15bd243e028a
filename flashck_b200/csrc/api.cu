// C ABI of libflashck_b200.so: argument checking, stride conventions and dispatch to the kernel instances.
// Mirrors the host code the reference generates around each ck_tile launch (init_args + MakeKargs + GridSize,
// attention_kernels/fmha_fwd/fmha_fwd_jinja.h:186-396, fmha_fwd_split_kv/fmha_fwd_split_kv_jinja.h:241-504,
// fmha_fwd_split_kv_combine/fmha_fwd_split_kv_combine_jinja.h:114-218) with BSHD packed strides.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "kernels.h"

namespace fck {

namespace {
thread_local char g_err[512] = "";
__device__ int g_device_status_word = 0;
constexpr int kMaxDevices = 64;
int* g_status_ptr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
std::mutex g_mu;
}  // namespace

void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_last_error("CUDA error %d (%s) from %s", (int)e, cudaGetErrorString(e), what);
    return FLASHCK_ERR_CUDA;
}

static std::atomic<int64_t> g_use_pdl{1};  // instance parameter "use_pdl"
bool use_pdl() { return g_use_pdl.load() != 0; }

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

int* device_status_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_last_error("cannot query the current device");
        return nullptr;
    }
    if (!g_status_ptr[dev]) {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_status_ptr[dev]) {
            int* ptr = nullptr;
            cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_device_status_word);
            if (e != cudaSuccess) {
                cuda_fail(e, "cudaGetSymbolAddress(status word)");
                return nullptr;
            }
            g_status_ptr[dev] = ptr;
        }
    }
    return g_status_ptr[dev];
}

PFN_encodeTiled get_encode_tiled() {
    static PFN_encodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_encodeTiled>(sym);
    });
    return fn;
}

namespace {

// instance parameters of the split-KV family that belong to the tcgen05 kernel's file
bool split_key_of_sm100(const char* key) {
    return !strcmp(key, "use_sm100_splitkv") || !strcmp(key, "exp_mode_splitkv") || !strcmp(key, "split_item_cost") ||
           !strcmp(key, "split_min_piece_tiles");
}

// how FmhaFwd reads a non-null bias pointer (the reference fixes both per compiled instance)
std::atomic<int64_t> g_bias_enum{1}, g_bias_rank_info{0};

int check_common(const char* fn, int dtype, int64_t hq, int64_t hkv, int64_t d, int64_t dv, const void* bias) {
    FCK_REQUIRE(dtype == FLASHCK_DTYPE_FLOAT16 || dtype == FLASHCK_DTYPE_BFLOAT16, FLASHCK_ERR_UNSUPPORTED,
                "%s: dtype must be 3 (float16) or 4 (bfloat16), got %d", fn, dtype);
    FCK_REQUIRE(hq > 0 && hkv > 0 && hq % hkv == 0, FLASHCK_ERR_INVALID_ARGUMENT,
                "%s: nhead_q (%lld) must be a positive multiple of nhead_k (%lld)", fn, (long long)hq, (long long)hkv);
    FCK_REQUIRE(d > 0 && dv > 0, FLASHCK_ERR_INVALID_ARGUMENT, "%s: head dims must be positive", fn);
    FCK_REQUIRE(bias == nullptr, FLASHCK_ERR_UNSUPPORTED, "%s: bias is not supported (no-bias instances only)", fn);
    return FLASHCK_OK;
}

// The paged and split-KV entry points take a bias pointer only as ALiBi slopes (instance parameter bias_enum = 2;
// bias_rank_info 0 = [1,hq], 1 = [batch,hq]); an elementwise bias has no defined layout over pages.
int alibi_from_bias(const char* fn, const void* bias, const float** slopes, int* rank) {
    *slopes = nullptr;
    *rank = 0;
    if (!bias) return FLASHCK_OK;
    FCK_REQUIRE(g_bias_enum.load() == 2, FLASHCK_ERR_UNSUPPORTED,
                "%s: a bias pointer is read as ALiBi slopes only (set the instance parameter bias_enum of family 0 to 2)", fn);
    FCK_REQUIRE(g_bias_rank_info.load() <= 1, FLASHCK_ERR_INVALID_ARGUMENT, "%s: bias_rank_info must be 0 or 1 for ALiBi", fn);
    *slopes = (const float*)bias;
    *rank = (int)g_bias_rank_info.load();
    return FLASHCK_OK;
}

// The same with the kind of bias stated per call (the ...Ex entry points): nothing process-wide is read.
int alibi_explicit(const char* fn, const void* bias, int bias_enum, int bias_rank_info, const float** slopes, int* rank) {
    *slopes = nullptr;
    *rank = 0;
    FCK_REQUIRE(bias_enum == 0 || bias_enum == 2, FLASHCK_ERR_UNSUPPORTED,
                "%s: bias_enum must be 0 (none) or 2 (alibi); an elementwise bias has no layout over pages", fn);
    if (bias_enum == 0) return FLASHCK_OK;
    FCK_REQUIRE(bias != nullptr, FLASHCK_ERR_INVALID_ARGUMENT, "%s: bias_enum 2 without a slope buffer", fn);
    FCK_REQUIRE(bias_rank_info == 0 || bias_rank_info == 1, FLASHCK_ERR_INVALID_ARGUMENT,
                "%s: bias_rank_info must be 0 ([1,hq]) or 1 ([batch,hq]) for ALiBi", fn);
    *slopes = (const float*)bias;
    *rank = bias_rank_info;
    return FLASHCK_OK;
}

inline float resolve_scale(float scale, int64_t d) {
    return scale == 0.f ? 1.f / sqrtf((float)d) : scale;  // fmha_fwd_jinja.h:57-59
}

// which instance the last forward / prefill call of this process ran on: 1 tcgen05, 0 general (instance parameter
// "last_instance" of family 0, read-only; the tests use it to pin a problem to the instance it is meant for)
std::atomic<int64_t> g_last_fwd_instance{-1};
std::atomic<int64_t> g_log_fallback{0};  // instance parameter "log_fallback": say on stderr why a call left the tcgen05 instance

int run_fwd(const FwdParams& p, cudaStream_t stream) {
    if (fwd_sm100_supported(p)) {
        g_last_fwd_instance = 1;
        return launch_fwd_sm100(p, stream);
    }
    g_last_fwd_instance = 0;
    if (g_log_fallback.load())
        fprintf(stderr,
                "[flashck_b200] forward call on the general (mma.sync) instance: dtype %d, hdim %lld/%lld, batch %lld, max_seqlen_q %lld, "
                "nhead %lld/%lld, bias_type %d, paged %d page %lld (the tcgen05 instances serve hdim 128 and 64, an elementwise bias "
                "only at hdim 128 on contiguous K/V, batch <= 256, <= 1024 work items per SM, nhead_q <= 1023, pages of 16..128 tokens dividing 128 or "
                "multiples; 8-bit operands at hdim 128 with contiguous K/V)\n",
                p.dtype, (long long)p.d, (long long)p.dv, (long long)p.batch, (long long)p.max_seqlen_q, (long long)p.hq,
                (long long)p.hkv, p.bias ? p.bias_type : 0, (p.block_table || p.kv_indptr) ? 1 : 0, (long long)p.page);
    return launch_fwd_generic(p, stream);
}

}  // namespace
}  // namespace fck

using namespace fck;

extern "C" {

const char* FlashckGetLastError(void) { return g_err; }
const char* FlashckVersion(void) { return "flashck_b200 0.1.0 (sm_100a)"; }

int FlashckDeviceStatus(int* status_out) {
    int* ptr = device_status_ptr();
    if (!ptr) return FLASHCK_ERR_CUDA;
    FCK_CUDA(cudaDeviceSynchronize());
    int v = 0;
    FCK_CUDA(cudaMemcpy(&v, ptr, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) {
        int zero = 0;
        FCK_CUDA(cudaMemcpy(ptr, &zero, sizeof(int), cudaMemcpyHostToDevice));
    }
    if (status_out) *status_out = v;
    if (v & FLASHCK_STATUS_TIMEOUT_MASK) {
        set_last_error("a bounded device-side wait ran out (status word 0x%x)", (unsigned)v);
        return FLASHCK_ERR_DEVICE_TIMEOUT;
    }
    if (v != 0) {
        set_last_error("a kernel skipped work: %s%s(status word 0x%x)",
                       (v & FLASHCK_STATUS_WORKLIST_OVERFLOW) ? "on-chip work list overflow " : "",
                       (v & FLASHCK_STATUS_APPEND_OVERFLOW) ? "append past the cache capacity " : "", (unsigned)v);
        return FLASHCK_ERR_UNSUPPORTED;
    }
    return FLASHCK_OK;
}

int FmhaFwd(void* q, void* k, void* v, void* bias, void* o, int64_t* q_seq_start, int64_t* k_seq_start,
            int64_t* k_seq_len, int64_t batch, int64_t q_seq_len, int64_t kv_seq_len, int64_t hq, int64_t hkv,
            int64_t d, int64_t dv, int64_t q_max_seq_len, float scale, int64_t window_left, int64_t window_right,
            uint32_t mask_type, void* stream, void* lse, int dtype) {
    // The reference fixes the kind of bias per compiled instance (bias_enum, bias_rank_info); here the instance
    // parameters of the fmha_fwd family say how a non-null bias pointer is read.
    return FmhaFwdBias(q, k, v, bias, o, q_seq_start, k_seq_start, k_seq_len, batch, q_seq_len, kv_seq_len, hq, hkv, d, dv,
                       q_max_seq_len, scale, window_left, window_right, mask_type, stream, lse, dtype,
                       bias ? (int)g_bias_enum.load() : 0, (int)g_bias_rank_info.load(), 0.f);
}

int FmhaFwdFp8(void* q, void* k, void* v, void* o, int64_t* q_seq_start, int64_t* k_seq_start, int64_t batch,
               int64_t q_seq_len, int64_t kv_seq_len, int64_t hq, int64_t hkv, int64_t d, int64_t dv, int64_t q_max_seq_len,
               float scale_s, float scale_p, float scale_o, int64_t window_left, int64_t window_right, uint32_t mask_type,
               void* stream, void* lse, int dtype, int o_dtype) {
    FCK_REQUIRE(dtype == FLASHCK_DTYPE_FLOAT8 || dtype == FLASHCK_DTYPE_BFLOAT8, FLASHCK_ERR_UNSUPPORTED,
                "FmhaFwdFp8: dtype must be 1 (float8 e4m3) or 2 (bfloat8 e5m2), got %d", dtype);
    FCK_REQUIRE(o_dtype >= FLASHCK_DTYPE_FLOAT8 && o_dtype <= FLASHCK_DTYPE_BFLOAT16, FLASHCK_ERR_UNSUPPORTED,
                "FmhaFwdFp8: o_dtype must be 1, 2, 3 or 4, got %d", o_dtype);
    FCK_REQUIRE(hq > 0 && hkv > 0 && hq % hkv == 0, FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdFp8: nhead_q (%lld) must be a positive multiple of nhead_k (%lld)", (long long)hq, (long long)hkv);
    FCK_REQUIRE(q && k && v && o, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdFp8: q, k, v and o must not be null");
    FCK_REQUIRE(batch >= 0 && q_seq_len >= 0 && kv_seq_len >= 0 && d > 0 && dv > 0, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdFp8: bad size");
    FCK_REQUIRE(mask_type <= 3, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdFp8: mask_type must be 0..3");
    FCK_REQUIRE((q_seq_start == nullptr) == (k_seq_start == nullptr), FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdFp8: group mode needs both seqstart arrays");
    FCK_REQUIRE(scale_p > 0.f && scale_o > 0.f && scale_s >= 0.f, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdFp8: scales must be positive");
    FwdParams p{};
    p.q = q; p.k = k; p.v = v; p.o = o; p.lse = (float*)lse;
    p.seqstart_q = q_seq_start; p.seqstart_k = k_seq_start;
    p.batch = batch; p.seqlen_q = q_seq_len; p.seqlen_k = kv_seq_len; p.hq = hq; p.hkv = hkv; p.d = d; p.dv = dv;
    p.total_q = q_seq_len;
    p.max_seqlen_q = q_seq_start ? (q_max_seq_len > 0 ? q_max_seq_len : q_seq_len) : q_seq_len;
    p.scale = resolve_scale(scale_s, d);
    p.mask_type = (int)mask_type; p.wl = window_left; p.wr = window_right; p.dtype = dtype;
    p.scale_p = scale_p; p.scale_o = scale_o; p.out_dtype = o_dtype;
    return run_fwd(p, (cudaStream_t)stream);  // (hdim 128 contiguous: the kind::f8f6f4 tcgen05 instance; else the general one)
}

int FmhaFwdBias(void* q, void* k, void* v, void* bias, void* o, int64_t* q_seq_start, int64_t* k_seq_start,
                int64_t* k_seq_len, int64_t batch, int64_t q_seq_len, int64_t kv_seq_len, int64_t hq, int64_t hkv,
                int64_t d, int64_t dv, int64_t q_max_seq_len, float scale, int64_t window_left, int64_t window_right,
                uint32_t mask_type, void* stream, void* lse, int dtype, int bias_enum, int bias_rank_info,
                float logits_soft_cap) {
    if (dtype == FLASHCK_DTYPE_FLOAT8 || dtype == FLASHCK_DTYPE_BFLOAT8) {
        FCK_REQUIRE(bias_enum == 0 && logits_soft_cap == 0.f && k_seq_len == nullptr, FLASHCK_ERR_UNSUPPORTED,
                    "FmhaFwd: the 8-bit element types take no bias, soft cap or k_seq_len array");
        return FmhaFwdFp8(q, k, v, o, q_seq_start, k_seq_start, batch, q_seq_len, kv_seq_len, hq, hkv, d, dv, q_max_seq_len,
                          scale, 1.f, 1.f, window_left, window_right, mask_type, stream, lse, dtype, dtype);
    }
    int rc = check_common("FmhaFwd", dtype, hq, hkv, d, dv, nullptr);
    if (rc) return rc;
    FCK_REQUIRE(bias_enum >= 0 && bias_enum <= 2, FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwd: bias_enum must be 0 (none), 1 (elementwise) or 2 (alibi), got %d", bias_enum);
    FCK_REQUIRE(bias_enum == 0 || bias != nullptr, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwd: bias_enum %d without a bias buffer", bias_enum);
    FCK_REQUIRE(bias_rank_info >= 0 && bias_rank_info <= (bias_enum == 2 ? 1 : 2), FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwd: bias_rank_info %d out of range for bias_enum %d", bias_rank_info, bias_enum);
    FCK_REQUIRE(logits_soft_cap >= 0.f, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwd: logits_soft_cap must be >= 0");
    FCK_REQUIRE(q && k && v && o, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwd: q, k, v and o must not be null");
    FCK_REQUIRE(batch >= 0 && q_seq_len >= 0 && kv_seq_len >= 0, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwd: negative size");
    FCK_REQUIRE(mask_type <= 3, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwd: mask_type must be 0..3");
    FCK_REQUIRE(q_seq_start || !k_seq_start, FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwd: k_seq_start_ptr without q_seq_start_ptr (group mode needs both)");
    FwdParams p{};
    p.q = q; p.k = k; p.v = v; p.o = o; p.lse = (float*)lse;
    p.seqstart_q = q_seq_start; p.seqstart_k = k_seq_start; p.seqlen_k64 = k_seq_len;
    p.batch = batch; p.seqlen_q = q_seq_len; p.seqlen_k = kv_seq_len; p.hq = hq; p.hkv = hkv; p.d = d; p.dv = dv;
    // group mode: q_seq_len is the packed total (shape_seqlen), fmha_fwd_jinja.h:189-192
    p.total_q = q_seq_len;
    p.max_seqlen_q = q_seq_start ? (q_max_seq_len > 0 ? q_max_seq_len : q_seq_len) : q_seq_len;
    p.scale = resolve_scale(scale, d);
    p.mask_type = (int)mask_type; p.wl = window_left; p.wr = window_right; p.dtype = dtype;
    p.bias = bias_enum ? bias : nullptr; p.bias_type = bias_enum; p.bias_rank = bias_rank_info;
    p.logits_soft_cap = logits_soft_cap;
    return run_fwd(p, (cudaStream_t)stream);
}

static int batch_prefill_impl(void* q, void* k, void* v, const float* slopes, int slope_rank, void* o, int64_t* q_seq_start,
                              void* kv_indptr, void* kv_page_indices, void* kv_last_page_len, int64_t batch,
                              int64_t q_seq_len, int64_t hq, int64_t hkv, int64_t d, int64_t dv, int64_t q_max_seq_len,
                              int64_t num_total_pages, int64_t paged_block_size, float scale, int64_t window_left,
                              int64_t window_right, uint32_t mask_type, void* stream, void* lse, int dtype) {
    int rc = check_common("FmhaFwdBatchPrefill", dtype, hq, hkv, d, dv, nullptr);
    if (rc) return rc;
    FCK_REQUIRE(q && k && v && o && q_seq_start && kv_indptr && kv_page_indices && kv_last_page_len,
                FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdBatchPrefill: null pointer argument");
    FCK_REQUIRE(paged_block_size > 0 && num_total_pages >= 0 && batch >= 0 && q_max_seq_len >= 0,
                FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdBatchPrefill: bad page geometry");
    FCK_REQUIRE(mask_type <= 3, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdBatchPrefill: mask_type must be 0..3");
    FwdParams p{};
    p.q = q; p.k = k; p.v = v; p.o = o; p.lse = (float*)lse;
    p.seqstart_q = q_seq_start;
    p.kv_indptr = (const int32_t*)kv_indptr; p.kv_page_indices = (const int32_t*)kv_page_indices;
    p.kv_last_page_len = (const int32_t*)kv_last_page_len;
    p.batch = batch; p.hq = hq; p.hkv = hkv; p.d = d; p.dv = dv; p.page = paged_block_size;
    p.max_seqlen_q = q_max_seq_len > 0 ? q_max_seq_len : q_seq_len;
    p.total_q = q_seq_len;  // packed total, like shape_seqlen_q of the other group-mode calls
    p.num_pages = num_total_pages;
    p.scale = resolve_scale(scale, d);
    p.mask_type = (int)mask_type; p.wl = window_left; p.wr = window_right; p.dtype = dtype;
    if (slopes) { p.bias = slopes; p.bias_type = 2; p.bias_rank = slope_rank; }
    return run_fwd(p, (cudaStream_t)stream);
}

int FmhaFwdBatchPrefill(void* q, void* k, void* v, void* bias, void* o, int64_t* q_seq_start, void* kv_indptr,
                        void* kv_page_indices, void* kv_last_page_len, int64_t batch, int64_t q_seq_len, int64_t hq,
                        int64_t hkv, int64_t d, int64_t dv, int64_t q_max_seq_len, int64_t num_total_pages,
                        int64_t paged_block_size, float scale, int64_t window_left, int64_t window_right,
                        uint32_t mask_type, void* stream, void* lse, int dtype) {
    const float* slopes = nullptr;
    int slope_rank = 0;
    if (int rc = alibi_from_bias("FmhaFwdBatchPrefill", bias, &slopes, &slope_rank)) return rc;
    return batch_prefill_impl(q, k, v, slopes, slope_rank, o, q_seq_start, kv_indptr, kv_page_indices, kv_last_page_len,
                              batch, q_seq_len, hq, hkv, d, dv, q_max_seq_len, num_total_pages, paged_block_size, scale,
                              window_left, window_right, mask_type, stream, lse, dtype);
}

int FmhaFwdBatchPrefillEx(void* q, void* k, void* v, void* bias, void* o, int64_t* q_seq_start, void* kv_indptr,
                          void* kv_page_indices, void* kv_last_page_len, int64_t batch, int64_t q_seq_len, int64_t hq,
                          int64_t hkv, int64_t d, int64_t dv, int64_t q_max_seq_len, int64_t num_total_pages,
                          int64_t paged_block_size, float scale, int64_t window_left, int64_t window_right,
                          uint32_t mask_type, void* stream, void* lse, int dtype, int bias_enum, int bias_rank_info) {
    const float* slopes = nullptr;
    int slope_rank = 0;
    if (int rc = alibi_explicit("FmhaFwdBatchPrefillEx", bias, bias_enum, bias_rank_info, &slopes, &slope_rank)) return rc;
    return batch_prefill_impl(q, k, v, slopes, slope_rank, o, q_seq_start, kv_indptr, kv_page_indices, kv_last_page_len,
                              batch, q_seq_len, hq, hkv, d, dv, q_max_seq_len, num_total_pages, paged_block_size, scale,
                              window_left, window_right, mask_type, stream, lse, dtype);
}

static int paged_prefill_impl(void* q, void* k, void* v, const float* slopes, int slope_rank, void* o, int64_t* q_seq_start,
                              void* k_seq_len, void* block_table, int64_t* cache_batch_idx, int64_t batch,
                              int64_t q_seq_len, int64_t hq, int64_t hkv, int64_t d, int64_t dv, int64_t q_max_seq_len,
                              int64_t max_num_page_blocks, int64_t paged_block_size, float scale, int64_t window_left,
                              int64_t window_right, uint32_t mask_type, void* stream, void* lse, int dtype,
                              int64_t num_pool_pages) {
    int rc = check_common("FmhaFwdPagedKVPrefill", dtype, hq, hkv, d, dv, nullptr);
    if (rc) return rc;
    FCK_REQUIRE(num_pool_pages > 0, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdPagedKVPrefill: the K/V pools hold no page");
    FCK_REQUIRE(q && k && v && o && k_seq_len && block_table, FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdPagedKVPrefill: null pointer argument");
    FCK_REQUIRE(batch > 0 && paged_block_size > 0 && max_num_page_blocks % batch == 0, FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdPagedKVPrefill: max_num_page_blocks must be batch * pages_per_sequence");
    FCK_REQUIRE(mask_type <= 3, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdPagedKVPrefill: mask_type must be 0..3");
    FwdParams p{};
    p.q = q; p.k = k; p.v = v; p.o = o; p.lse = (float*)lse;
    p.seqstart_q = q_seq_start; p.seqlen_k32 = (const int32_t*)k_seq_len;
    p.block_table = (const int32_t*)block_table; p.cache_batch_idx = cache_batch_idx;
    p.batch = batch; p.seqlen_q = q_seq_len; p.hq = hq; p.hkv = hkv; p.d = d; p.dv = dv;
    p.total_q = q_seq_len;
    p.max_seqlen_q = q_seq_start ? (q_max_seq_len > 0 ? q_max_seq_len : q_seq_len) : q_seq_len;
    p.bt_stride = max_num_page_blocks / batch;  // fmha_fwd_split_kv_jinja.h:318
    p.page = paged_block_size;
    p.num_pages = num_pool_pages;  // extent of the pools' tensor maps: a page id at or beyond it reads as zeros
    p.scale = resolve_scale(scale, d);
    p.mask_type = (int)mask_type; p.wl = window_left; p.wr = window_right; p.dtype = dtype;
    if (slopes) { p.bias = slopes; p.bias_type = 2; p.bias_rank = slope_rank; }
    return run_fwd(p, (cudaStream_t)stream);
}

int FmhaFwdPagedKVPrefill(void* q, void* k, void* v, void* bias, void* o, int64_t* q_seq_start, void* k_seq_len,
                          void* block_table, int64_t* cache_batch_idx, int64_t batch, int64_t q_seq_len, int64_t hq,
                          int64_t hkv, int64_t d, int64_t dv, int64_t q_max_seq_len, int64_t max_num_page_blocks,
                          int64_t paged_block_size, float scale, int64_t window_left, int64_t window_right,
                          uint32_t mask_type, void* stream, void* lse, int dtype) {
    const float* slopes = nullptr;
    int slope_rank = 0;
    if (int rc = alibi_from_bias("FmhaFwdPagedKVPrefill", bias, &slopes, &slope_rank)) return rc;
    // the reference's pools hold exactly max_num_page_blocks pages (fmha_fwd_split_kv_jinja.h:512-519)
    return paged_prefill_impl(q, k, v, slopes, slope_rank, o, q_seq_start, k_seq_len, block_table, cache_batch_idx, batch,
                              q_seq_len, hq, hkv, d, dv, q_max_seq_len, max_num_page_blocks, paged_block_size, scale,
                              window_left, window_right, mask_type, stream, lse, dtype, max_num_page_blocks);
}

int FmhaFwdPagedKVPrefillEx(void* q, void* k, void* v, void* bias, void* o, int64_t* q_seq_start, void* k_seq_len,
                            void* block_table, int64_t* cache_batch_idx, int64_t batch, int64_t q_seq_len, int64_t hq,
                            int64_t hkv, int64_t d, int64_t dv, int64_t q_max_seq_len, int64_t max_num_page_blocks,
                            int64_t paged_block_size, float scale, int64_t window_left, int64_t window_right,
                            uint32_t mask_type, void* stream, void* lse, int dtype, int bias_enum, int bias_rank_info,
                            int64_t num_pool_pages) {
    const float* slopes = nullptr;
    int slope_rank = 0;
    if (int rc = alibi_explicit("FmhaFwdPagedKVPrefillEx", bias, bias_enum, bias_rank_info, &slopes, &slope_rank)) return rc;
    return paged_prefill_impl(q, k, v, slopes, slope_rank, o, q_seq_start, k_seq_len, block_table, cache_batch_idx, batch,
                              q_seq_len, hq, hkv, d, dv, q_max_seq_len, max_num_page_blocks, paged_block_size, scale,
                              window_left, window_right, mask_type, stream, lse, dtype, num_pool_pages);
}

static int splitkv_impl(void* q, void* k, void* v, const float* slopes, int slope_rank, void* lse_acc, void* o_acc,
                        int64_t* q_seq_start, int64_t* kv_seq_start, void* k_seq_len, void* block_table,
                        int64_t* cache_batch_idx, int64_t batch, int64_t q_seq_len, int64_t kv_seq_len, int64_t hq,
                        int64_t hkv, int64_t d, int64_t dv, int64_t q_max_seq_len, int64_t num_splits,
                        int64_t max_num_page_blocks, int64_t paged_block_size, float scale, int64_t window_left,
                        int64_t window_right, uint32_t mask_type, void* stream, int dtype, int64_t num_pool_pages) {
    int rc = check_common("FmhaFwdSplitKV", dtype, hq, hkv, d, dv, nullptr);
    if (rc) return rc;
    FCK_REQUIRE(!block_table || num_pool_pages > 0, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdSplitKV: the K/V pools hold no page");
    FCK_REQUIRE(q && k && v && o_acc, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdSplitKV: q, k, v and o_acc must not be null");
    FCK_REQUIRE(num_splits >= 1 && num_splits <= 1024, FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdSplitKV: num_splits must be in [1,1024] (got %lld)", (long long)num_splits);
    FCK_REQUIRE(lse_acc || num_splits == 1, FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdSplitKV: lse_acc may be null only when num_splits == 1");
    FCK_REQUIRE(batch > 0 && q_seq_len >= 0, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdSplitKV: bad batch / q_seq_len");
    FCK_REQUIRE(mask_type <= 3, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdSplitKV: mask_type must be 0..3");
    FCK_REQUIRE(!block_table || (paged_block_size > 0 && max_num_page_blocks % batch == 0), FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdSplitKV: max_num_page_blocks must be batch * pages_per_sequence");
    SplitKVParams p{};
    p.alibi_slopes = slopes; p.alibi_rank = slope_rank;
    p.q = q; p.k = k; p.v = v; p.o_acc = (float*)o_acc; p.lse_acc = (float*)lse_acc;
    p.seqstart_q = q_seq_start; p.seqstart_k = block_table ? nullptr : kv_seq_start;
    p.seqlen_k = (const int32_t*)k_seq_len; p.block_table = (const int32_t*)block_table;
    p.cache_batch_idx = cache_batch_idx;
    p.batch = batch; p.seqlen_q = q_seq_len; p.seqlen_k_cap = kv_seq_len; p.hq = hq; p.hkv = hkv; p.d = d; p.dv = dv;
    p.max_seqlen_q = q_seq_start ? (q_max_seq_len > 0 ? q_max_seq_len : q_seq_len) : q_seq_len;
    p.num_splits = num_splits;
    p.total_q = q_seq_len;
    if (block_table) {
        // extent of the pools' tensor maps: a stale or corrupt page id at or beyond it reads as zeros, not as memory
        // outside the pools
        p.num_pages = num_pool_pages;
        p.bt_stride = max_num_page_blocks / batch;
        p.page = paged_block_size;
    } else {
        // contiguous cache [rows, kv_seq_len, hkv, d]: `batch` rows, or (with cache_batch_idx) the row count the caller
        // states through num_pool_pages; 0 = unknown
        p.num_pages = cache_batch_idx ? (num_pool_pages > 0 ? num_pool_pages : 0) : batch;
    }
    p.scale = resolve_scale(scale, d);
    p.mask_type = (int)mask_type; p.wl = window_left; p.wr = window_right; p.dtype = dtype;
    if (splitkv_sm100_supported(p)) return launch_splitkv_sm100(p, (cudaStream_t)stream);
    return launch_splitkv_decode(p, (cudaStream_t)stream);
}

int FmhaFwdSplitKV(void* q, void* k, void* v, void* bias, void* lse_acc, void* o_acc, int64_t* q_seq_start,
                   int64_t* kv_seq_start, void* k_seq_len, void* block_table, int64_t* cache_batch_idx, int64_t batch,
                   int64_t q_seq_len, int64_t kv_seq_len, int64_t hq, int64_t hkv, int64_t d, int64_t dv,
                   int64_t q_max_seq_len, int64_t num_splits, int64_t max_num_page_blocks, int64_t paged_block_size,
                   float scale, int64_t window_left, int64_t window_right, uint32_t mask_type, void* stream,
                   int dtype) {
    const float* slopes = nullptr;
    int slope_rank = 0;
    if (int rc = alibi_from_bias("FmhaFwdSplitKV", bias, &slopes, &slope_rank)) return rc;
    // the reference's pools hold exactly max_num_page_blocks pages (fmha_fwd_split_kv_jinja.h:512-519)
    return splitkv_impl(q, k, v, slopes, slope_rank, lse_acc, o_acc, q_seq_start, kv_seq_start, k_seq_len, block_table,
                        cache_batch_idx, batch, q_seq_len, kv_seq_len, hq, hkv, d, dv, q_max_seq_len, num_splits,
                        max_num_page_blocks, paged_block_size, scale, window_left, window_right, mask_type, stream, dtype,
                        block_table ? max_num_page_blocks : 0);
}

int FmhaFwdSplitKVEx(void* q, void* k, void* v, void* bias, void* lse_acc, void* o_acc, int64_t* q_seq_start,
                     int64_t* kv_seq_start, void* k_seq_len, void* block_table, int64_t* cache_batch_idx, int64_t batch,
                     int64_t q_seq_len, int64_t kv_seq_len, int64_t hq, int64_t hkv, int64_t d, int64_t dv,
                     int64_t q_max_seq_len, int64_t num_splits, int64_t max_num_page_blocks, int64_t paged_block_size,
                     float scale, int64_t window_left, int64_t window_right, uint32_t mask_type, void* stream, int dtype,
                     int bias_enum, int bias_rank_info, int64_t num_pool_pages) {
    const float* slopes = nullptr;
    int slope_rank = 0;
    if (int rc = alibi_explicit("FmhaFwdSplitKVEx", bias, bias_enum, bias_rank_info, &slopes, &slope_rank)) return rc;
    return splitkv_impl(q, k, v, slopes, slope_rank, lse_acc, o_acc, q_seq_start, kv_seq_start, k_seq_len, block_table,
                        cache_batch_idx, batch, q_seq_len, kv_seq_len, hq, hkv, d, dv, q_max_seq_len, num_splits,
                        max_num_page_blocks, paged_block_size, scale, window_left, window_right, mask_type, stream, dtype,
                        num_pool_pages);
}

int FmhaFwdSplitKVCombine(void* lse_acc, void* o_acc, void* o, int64_t* q_seq_start, int64_t batch, int64_t q_seq_len,
                          int64_t hq, int64_t dv, int64_t q_max_seq_len, int64_t num_splits, void* stream, void* lse,
                          int dtype) {
    (void)q_max_seq_len;
    FCK_REQUIRE(dtype == FLASHCK_DTYPE_FLOAT16 || dtype == FLASHCK_DTYPE_BFLOAT16, FLASHCK_ERR_UNSUPPORTED,
                "FmhaFwdSplitKVCombine: dtype must be 3 (float16) or 4 (bfloat16), got %d", dtype);
    FCK_REQUIRE(lse_acc && o_acc && o, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdSplitKVCombine: null pointer argument");
    FCK_REQUIRE(batch >= 0 && q_seq_len >= 0 && hq > 0 && dv > 0, FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdSplitKVCombine: bad sizes");
    CombineParams p{};
    p.lse_acc = (const float*)lse_acc; p.o_acc = (const float*)o_acc; p.o = o; p.lse = (float*)lse;
    // group mode packs all sequences into one batch row of q_seq_len = total tokens (..._combine_jinja.h:118-119)
    p.bs = q_seq_start ? 1 : batch;
    p.rows = q_seq_len; p.hq = hq; p.dv = dv; p.num_splits = num_splits; p.dtype = dtype;
    return launch_combine(p, (cudaStream_t)stream);
}

int FmhaFwdSplitKVCombineStrided(void* lse_acc, void* o_acc, void* o, void* lse, int64_t batch, int64_t rows, int64_t hq,
                                 int64_t dv, int64_t num_splits, const int64_t* lse_strides, const int64_t* o_strides,
                                 int out_dtype, void* stream) {
    FCK_REQUIRE(lse_acc && o_acc && o && lse_strides && o_strides, FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdSplitKVCombineStrided: null pointer argument");
    FCK_REQUIRE(batch >= 0 && rows >= 0 && hq > 0 && dv > 0, FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdSplitKVCombineStrided: bad sizes");
    CombineParams p{};
    p.lse_acc = (const float*)lse_acc; p.o_acc = (const float*)o_acc; p.o = o; p.lse = (float*)lse;
    p.bs = batch; p.rows = rows; p.hq = hq; p.dv = dv; p.num_splits = num_splits; p.dtype = out_dtype;
    p.strided = true;
    for (int i = 0; i < 4; ++i) { p.lse_strides[i] = lse_strides[i]; p.o_strides[i] = o_strides[i]; }
    return launch_combine(p, (cudaStream_t)stream);
}

int FmhaSplitKVCombine(void* lse_acc, void* o_acc, void* o, int64_t* q_seq_start, int64_t batch, int64_t q_seq_len,
                       int64_t hq, int64_t dv, int64_t q_max_seq_len, int64_t num_splits, void* stream, void* lse,
                       int dtype) {
    return FmhaFwdSplitKVCombine(lse_acc, o_acc, o, q_seq_start, batch, q_seq_len, hq, dv, q_max_seq_len, num_splits,
                                 stream, lse, dtype);
}

int FmhaFwdAppendKV(void* q, void* k_cache, void* knew, void* v_cache, void* vnew, void* k_seq_len,
                    int64_t* q_seq_start, int64_t* knew_seq_start, void* rotary_cos, void* rotary_sin,
                    void* block_table, int64_t* cache_batch_idx, int64_t batch, int64_t q_seq_len, int64_t kv_seq_len,
                    int64_t knew_seq_len, int64_t hq, int64_t hkv, int64_t d, int64_t dv, int64_t rotary_dim,
                    int rope_type, int64_t max_num_page_blocks, int64_t paged_block_size, void* stream, int dtype) {
    int rc = check_common("FmhaFwdAppendKV", dtype, hq, hkv, d, dv, nullptr);
    if (rc) return rc;
    FCK_REQUIRE(k_cache && v_cache && k_seq_len, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdAppendKV: null cache or length pointer");
    FCK_REQUIRE(knew_seq_len == 0 || (knew && vnew), FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdAppendKV: knew/vnew must not be null");
    FCK_REQUIRE(rope_type == 0 || (rotary_cos && rotary_sin), FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdAppendKV: rotary tables must not be null when rope_type != 0");
    FCK_REQUIRE(rope_type == 0 || q_seq_len == 0 || q, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdAppendKV: q must not be null");
    FCK_REQUIRE(batch > 0, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdAppendKV: batch must be positive");
    FCK_REQUIRE(!block_table || (paged_block_size > 0 && max_num_page_blocks % batch == 0), FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdAppendKV: max_num_page_blocks must be batch * pages_per_sequence");
    FCK_REQUIRE((q_seq_start == nullptr) == (knew_seq_start == nullptr), FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdAppendKV: q_seq_start_ptr and knew_seq_start_ptr go together (group mode)");
    AppendKVParams p{};
    p.q = q; p.k_cache = k_cache; p.knew = knew; p.v_cache = v_cache; p.vnew = vnew;
    p.seqlen_k = (const int32_t*)k_seq_len; p.seqstart_q = q_seq_start; p.seqstart_knew = knew_seq_start;
    p.rotary_cos = rotary_cos; p.rotary_sin = rotary_sin; p.block_table = (const int32_t*)block_table;
    p.cache_batch_idx = cache_batch_idx;
    p.batch = batch; p.seqlen_q = q_seq_len; p.seqlen_k_cap = kv_seq_len; p.seqlen_knew = knew_seq_len;
    p.hq = hq; p.hkv = hkv; p.d = d; p.dv = dv; p.rotary_dim = rotary_dim; p.rope_type = rope_type;
    p.bt_stride = block_table ? max_num_page_blocks / batch : 0;
    p.page = paged_block_size; p.dtype = dtype;
    return launch_appendkv(p, (cudaStream_t)stream);
}

int FlashckSetInstanceParam(int family, const char* key, int64_t value) {
    FCK_REQUIRE(key != nullptr, FLASHCK_ERR_INVALID_ARGUMENT, "FlashckSetInstanceParam: null key");
    int rc = FLASHCK_ERR_INVALID_ARGUMENT;
    if (family == 0 && !strcmp(key, "bias_enum")) {
        FCK_REQUIRE(value >= 0 && value <= 2, FLASHCK_ERR_INVALID_ARGUMENT, "bias_enum must be 0, 1 or 2");
        g_bias_enum = value;
        return FLASHCK_OK;
    }
    if (family == 0 && !strcmp(key, "bias_rank_info")) {
        FCK_REQUIRE(value >= 0 && value <= 2, FLASHCK_ERR_INVALID_ARGUMENT, "bias_rank_info must be 0, 1 or 2");
        g_bias_rank_info = value;
        return FLASHCK_OK;
    }
    if (family == 0 && !strcmp(key, "log_fallback")) { g_log_fallback = value; return FLASHCK_OK; }
    if (!strcmp(key, "use_pdl")) { g_use_pdl = value; return FLASHCK_OK; }
    if (family == 0) rc = fwd_set_param(key, value);
    else if (family == 2) rc = split_key_of_sm100(key) ? fwd_set_param(key, value) : splitkv_set_param(key, value);
    if (rc) set_last_error("FlashckSetInstanceParam: unknown family/key %d/%s", family, key);
    return rc;
}
int FlashckGetInstanceParam(int family, const char* key, int64_t* value_out) {
    FCK_REQUIRE(key != nullptr && value_out != nullptr, FLASHCK_ERR_INVALID_ARGUMENT, "FlashckGetInstanceParam: null argument");
    int rc = FLASHCK_ERR_INVALID_ARGUMENT;
    if (family == 0 && !strcmp(key, "bias_enum")) { *value_out = g_bias_enum; return FLASHCK_OK; }
    if (family == 0 && !strcmp(key, "bias_rank_info")) { *value_out = g_bias_rank_info; return FLASHCK_OK; }
    if (family == 0 && !strcmp(key, "last_instance")) { *value_out = g_last_fwd_instance; return FLASHCK_OK; }
    if (family == 0 && !strcmp(key, "log_fallback")) { *value_out = g_log_fallback; return FLASHCK_OK; }
    if (!strcmp(key, "use_pdl")) { *value_out = g_use_pdl; return FLASHCK_OK; }
    if (family == 0) rc = fwd_get_param(key, value_out);
    else if (family == 2) rc = split_key_of_sm100(key) ? fwd_get_param(key, value_out) : splitkv_get_param(key, value_out);
    if (rc) set_last_error("FlashckGetInstanceParam: unknown family/key %d/%s", family, key);
    return rc;
}

}  // extern "C"
