// fmha_fwd_appendkv: rotary embedding of Q (in place) and of the new keys, and the K/V cache write through the
// block table.  The reference names the kind and the rotary modes (core/profiling/attention/fmha_library.h:19,41,
// 195-219) and generates cos/sin tables [positions, rotary_dim/2] in the element dtype
// (attention_kernels/fmha_common_jinja.h:192-227).
//
// Arithmetic contract (bit-exact against the CPU statement): operands widened to fp32; every product, sum and
// difference is one separately rounded fp32 operation (__fmul_rn/__fadd_rn/__fsub_rn are never contracted into
// FMA); results narrowed with round-to-nearest-even.
//
// One CTA per token: CTAs [0, total_new) write K/V rows, CTAs [total_new, total_new + total_q) rotate Q rows.
// Each rotation pair is read and written by exactly one thread, so the in-place Q update has no hazard.
// Traffic is a few MB; the kernel is launch-latency bound.
#include "kernels.h"

namespace fck {

struct AppendDev {
    void* q;
    void* k_cache;
    const void* knew;
    void* v_cache;
    const void* vnew;
    const int32_t* seqlen_k;
    const int64_t* seqstart_q;
    const int64_t* seqstart_knew;
    const void* cosr;
    const void* sinr;
    const int32_t* block_table;
    const int64_t* cache_batch_idx;
    int batch, seqlen_q, seqlen_knew, hq, hkv, d, dv, rotary_dim, rope_type, bt_stride, page;
    int64_t seqlen_k_cap;
    int64_t total_new, total_q;
    int64_t capacity;  // tokens one sequence's cache can hold: pages_per_sequence * page, or the contiguous row length
    int* status;       // device status word: FLASHCK_STATUS_APPEND_OVERFLOW is ORed in when a token is skipped
};

// largest b with seqstart[b] <= t
__device__ __forceinline__ int find_batch(const int64_t* seqstart, int batch, int64_t t) {
    int lo = 0, hi = batch - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (seqstart[mid] <= t) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

template <typename T>
__device__ __forceinline__ void rope_heads(const T* src, T* dst, int heads, int d, int half, int rope_type,
                                           const T* cosr, const T* sinr, bool copy_tail) {
    const int rotary_dim = 2 * half;
    for (int p = threadIdx.x; p < heads * half; p += blockDim.x) {
        const int h = p / half, i = p - h * half;
        const int i0 = rope_type == 1 ? 2 * i : i;
        const int i1 = rope_type == 1 ? 2 * i + 1 : i + half;
        const float x0 = Elem<T>::to_f32(src[h * d + i0]), x1 = Elem<T>::to_f32(src[h * d + i1]);
        const float c = Elem<T>::to_f32(cosr[i]), s = Elem<T>::to_f32(sinr[i]);
        const float y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        const float y1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
        dst[h * d + i0] = Elem<T>::from_f32(y0);
        dst[h * d + i1] = Elem<T>::from_f32(y1);
    }
    if (copy_tail) {
        const int tail = d - rotary_dim;
        for (int p = threadIdx.x; p < heads * tail; p += blockDim.x) {
            const int h = p / tail, x = rotary_dim + (p - h * tail);
            dst[h * d + x] = src[h * d + x];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128) appendkv_kernel(const AppendDev a) {
    const int64_t t = blockIdx.x;
    const int half = a.rope_type == 0 ? 0 : a.rotary_dim / 2;
    if (t < a.total_new) {
        // ---- a new key/value token ----
        int b;
        int64_t j;
        if (a.seqstart_knew) {
            b = find_batch(a.seqstart_knew, a.batch, t);
            j = t - a.seqstart_knew[b];
            if (j >= a.seqstart_knew[b + 1] - a.seqstart_knew[b]) return;  // empty sequences share a start
        } else {
            b = (int)(t / a.seqlen_knew);
            j = t - (int64_t)b * a.seqlen_knew;
        }
        const int64_t pos = (int64_t)a.seqlen_k[b] + j;
        const int64_t bphys = a.cache_batch_idx ? a.cache_batch_idx[b] : b;
        // The lengths live on the device, so a full cache can only be seen here: a token that does not fit its
        // sequence's cache (or whose block-table entry is the negative filler of an unassigned page) is not written --
        // it would land in another sequence's page or past the buffer -- and the status word says so.
        if (pos < 0 || pos >= a.capacity) {
            if (threadIdx.x == 0) atomicOr(a.status, FLASHCK_STATUS_APPEND_OVERFLOW);
            return;
        }
        int64_t row;
        if (a.block_table) {
            const int32_t pg = a.block_table[bphys * a.bt_stride + pos / a.page];
            if (pg < 0) {
                if (threadIdx.x == 0) atomicOr(a.status, FLASHCK_STATUS_APPEND_OVERFLOW);
                return;
            }
            row = (int64_t)pg * a.page + pos % a.page;
        } else {
            row = bphys * a.seqlen_k_cap + pos;
        }
        const T* ksrc = (const T*)a.knew + t * a.hkv * a.d;
        T* kdst = (T*)a.k_cache + row * a.hkv * a.d;
        rope_heads<T>(ksrc, kdst, a.hkv, a.d, half, a.rope_type, (const T*)a.cosr + pos * half,
                      (const T*)a.sinr + pos * half, true);
        // V row: 16-byte copies (dv is a multiple of 8)
        const uint4* vsrc = reinterpret_cast<const uint4*>((const T*)a.vnew + t * a.hkv * a.dv);
        uint4* vdst = reinterpret_cast<uint4*>((T*)a.v_cache + row * a.hkv * a.dv);
        const int nvec = a.hkv * a.dv / 8;
        for (int p = threadIdx.x; p < nvec; p += blockDim.x) vdst[p] = vsrc[p];
    } else {
        // ---- a query token (rotated in place) ----
        if (half == 0) return;
        const int64_t tq = t - a.total_new;
        int b;
        int64_t i, sq, n;
        if (a.seqstart_q) {
            b = find_batch(a.seqstart_q, a.batch, tq);
            i = tq - a.seqstart_q[b];
            sq = a.seqstart_q[b + 1] - a.seqstart_q[b];
            if (i >= sq) return;
        } else {
            b = (int)(tq / a.seqlen_q);
            i = tq - (int64_t)b * a.seqlen_q;
            sq = a.seqlen_q;
        }
        n = a.seqstart_knew ? a.seqstart_knew[b + 1] - a.seqstart_knew[b] : a.seqlen_knew;
        const int64_t pos = (int64_t)a.seqlen_k[b] + n - sq + i;
        T* qrow = (T*)a.q + tq * a.hq * a.d;
        rope_heads<T>(qrow, qrow, a.hq, a.d, half, a.rope_type, (const T*)a.cosr + pos * half,
                      (const T*)a.sinr + pos * half, false);
    }
}

int launch_appendkv(const AppendKVParams& p, cudaStream_t stream) {
    FCK_REQUIRE(p.d % 8 == 0 && p.dv % 8 == 0, FLASHCK_ERR_UNSUPPORTED, "appendkv: head dims must be multiples of 8");
    FCK_REQUIRE(p.rope_type >= 0 && p.rope_type <= 2, FLASHCK_ERR_INVALID_ARGUMENT, "appendkv: rope_type must be 0..2");
    FCK_REQUIRE(p.rope_type == 0 || (p.rotary_dim > 0 && p.rotary_dim <= p.d && p.rotary_dim % 2 == 0),
                FLASHCK_ERR_INVALID_ARGUMENT, "appendkv: rotary_dim must be even and in (0, hdim_q]");
    int* status = device_status_ptr();
    if (!status) return FLASHCK_ERR_CUDA;
    AppendDev a;
    a.status = status;
    a.capacity = p.block_table ? p.bt_stride * p.page : p.seqlen_k_cap;
    a.q = p.q; a.k_cache = p.k_cache; a.knew = p.knew; a.v_cache = p.v_cache; a.vnew = p.vnew;
    a.seqlen_k = p.seqlen_k; a.seqstart_q = p.seqstart_q; a.seqstart_knew = p.seqstart_knew;
    a.cosr = p.rotary_cos; a.sinr = p.rotary_sin; a.block_table = p.block_table;
    a.cache_batch_idx = p.cache_batch_idx;
    a.batch = (int)p.batch; a.seqlen_q = (int)p.seqlen_q; a.seqlen_knew = (int)p.seqlen_knew;
    a.hq = (int)p.hq; a.hkv = (int)p.hkv; a.d = (int)p.d; a.dv = (int)p.dv;
    a.rotary_dim = (int)p.rotary_dim; a.rope_type = p.rope_type; a.bt_stride = (int)p.bt_stride; a.page = (int)p.page;
    a.seqlen_k_cap = p.seqlen_k_cap;
    // group mode: the scalar lengths are the packed totals; batch mode: per-sequence lengths
    a.total_new = p.seqstart_knew ? p.seqlen_knew : p.batch * p.seqlen_knew;
    a.total_q = p.seqstart_q ? p.seqlen_q : p.batch * p.seqlen_q;
    const int64_t blocks = a.total_new + (p.rope_type != 0 ? a.total_q : 0);
    if (blocks == 0) return FLASHCK_OK;
    FCK_REQUIRE(blocks < (1ll << 31), FLASHCK_ERR_UNSUPPORTED, "appendkv: too many tokens");
    if (p.dtype == FLASHCK_DTYPE_BFLOAT16)
        appendkv_kernel<__nv_bfloat16><<<(unsigned)blocks, 128, 0, stream>>>(a);
    else
        appendkv_kernel<__half><<<(unsigned)blocks, 128, 0, stream>>>(a);
    FCK_CUDA(cudaGetLastError());
    return FLASHCK_OK;
}

}  // namespace fck
