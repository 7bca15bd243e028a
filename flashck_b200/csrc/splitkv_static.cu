// FmhaFwdSplitKVStatic: split-KV attention + combine for callers that cannot allocate device memory.
//
// Some callers of this library run where cudaMalloc is off limits: inside a serving loop whose memory is
// fully planned up front, under a framework allocator they must not bypass, or on a thread that is not
// allowed to take the allocator's locks.  The regular path (FmhaFwdSplitKV + FmhaFwdSplitKVCombine) asks
// such a caller for two fp32 workspaces it may have nowhere to get.  This entry point keeps those
// workspaces inside the library instead: a fixed file-scope array in device memory, reserved on every GPU
// that loads the library for as long as the process lives.
//
// Consequences a user has to know:
//   * the workspaces of one call must fit kStaticScratchBytes (16 MiB); larger problems are rejected with
//     FLASHCK_ERR_UNSUPPORTED and a message that states the size asked for;
//   * every call on a device uses the same array, which keeps whatever the previous call left there.  Nothing
//     in it needs to start at zero: the split kernel writes -inf into the LSE slot of every split it does not
//     fill, and the combine never reads the O slot of such a split.  Two calls that overlap on the GPU (different
//     streams, or different host threads) race on the array -- serialise them;
//   * the first call on each device resolves the array's device address (a host-side lookup, no allocation).
//     Make that first call outside any stream capture.
#include "kernels.h"

#include <mutex>

namespace fck {
namespace {

constexpr size_t kStaticScratchBytes = 16u << 20;
// In host code this name is only a handle for the runtime's symbol table, never an address a kernel can use.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDev = 64;
unsigned char* g_scratch_addr[kMaxDev] = {};
std::mutex g_scratch_mu;

// Device address of the scratch array on the current device; resolved once per device.
int scratch_address(unsigned char** out) {
    int dev = 0;
    FCK_CUDA(cudaGetDevice(&dev));
    FCK_REQUIRE(dev >= 0 && dev < kMaxDev, FLASHCK_ERR_UNSUPPORTED, "FmhaFwdSplitKVStatic: device index %d too large", dev);
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    if (!g_scratch_addr[dev]) {
        unsigned char* ptr = nullptr;
        FCK_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
        FCK_REQUIRE(ptr != nullptr, FLASHCK_ERR_CUDA, "FmhaFwdSplitKVStatic: scratch symbol has no device address");
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return FLASHCK_OK;
}

}  // namespace
}  // namespace fck

using namespace fck;

extern "C" FLASHCK_API int FmhaFwdSplitKVStatic(void* q, void* k, void* v, void* o, void* lse, int64_t* q_seq_start,
                                                int64_t* kv_seq_start, void* k_seq_len, void* block_table,
                                                int64_t* cache_batch_idx, int64_t batch, int64_t q_seq_len,
                                                int64_t kv_seq_len, int64_t hq, int64_t hkv, int64_t d, int64_t dv,
                                                int64_t q_max_seq_len, int64_t num_splits,
                                                int64_t max_num_page_blocks, int64_t paged_block_size, float scale,
                                                int64_t window_left, int64_t window_right, uint32_t mask_type,
                                                void* stream, int dtype) {
    FCK_REQUIRE(q && k && v && o, FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdSplitKVStatic: q, k, v and o must not be null");
    FCK_REQUIRE(batch > 0 && q_seq_len >= 0 && hq > 0 && dv > 0 && num_splits >= 1 && num_splits <= 1024,
                FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdSplitKVStatic: bad batch / q_seq_len / heads / num_splits");
    // workspace sizes in the layout of the regular entry points.  The row count is formed in 128 bits from factors below
    // 2^31 each, so that no absurd argument can wrap around and slip under the capacity check.
    constexpr int64_t kFactorMax = 0x7fffffff;
    FCK_REQUIRE(batch <= kFactorMax && q_seq_len <= kFactorMax && hq <= kFactorMax && dv <= kFactorMax,
                FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdSplitKVStatic: a size argument is 2^31 or larger");
    const int64_t bs = q_seq_start ? 1 : batch;
    const unsigned __int128 rows128 = (unsigned __int128)bs * (unsigned __int128)hq * (unsigned __int128)num_splits *
                                      (unsigned __int128)q_seq_len;
    FCK_REQUIRE(rows128 * (unsigned __int128)(dv + 1) * sizeof(float) <= (unsigned __int128)kStaticScratchBytes,
                FLASHCK_ERR_UNSUPPORTED,
                "FmhaFwdSplitKVStatic: workspaces need more than the %zu bytes of the built-in scratch "
                "(batch %lld x heads %lld x splits %lld x rows %lld x (hdim %lld + 1) floats); lower num_splits or use "
                "FmhaFwdSplitKV with caller-owned workspaces",
                kStaticScratchBytes, (long long)bs, (long long)hq, (long long)num_splits, (long long)q_seq_len, (long long)dv);
    const size_t lse_bytes = (size_t)rows128 * sizeof(float);
    const size_t lse_padded = (lse_bytes + 255) & ~(size_t)255;
    const size_t o_bytes = (size_t)rows128 * (size_t)dv * sizeof(float);
    FCK_REQUIRE(lse_padded + o_bytes <= kStaticScratchBytes, FLASHCK_ERR_UNSUPPORTED,
                "FmhaFwdSplitKVStatic: workspaces need %zu bytes, the built-in scratch holds %zu; lower num_splits "
                "or use FmhaFwdSplitKV with caller-owned workspaces",
                lse_padded + o_bytes, kStaticScratchBytes);
    unsigned char* base = nullptr;
    int rc = scratch_address(&base);
    if (rc) return rc;
    float* lse_acc = reinterpret_cast<float*>(base);
    float* o_acc = reinterpret_cast<float*>(base + lse_padded);
    rc = FmhaFwdSplitKV(q, k, v, nullptr, lse_acc, o_acc, q_seq_start, kv_seq_start, k_seq_len, block_table,
                        cache_batch_idx, batch, q_seq_len, kv_seq_len, hq, hkv, d, dv, q_max_seq_len, num_splits,
                        max_num_page_blocks, paged_block_size, scale, window_left, window_right, mask_type, stream,
                        dtype);
    if (rc) return rc;
    return FmhaFwdSplitKVCombine(lse_acc, o_acc, o, q_seq_start, batch, q_seq_len, hq, dv, q_max_seq_len, num_splits,
                                 stream, lse, dtype);
}
