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
// Traffic is a few MB; the kernel is bound by its chain of dependent loads, which is kept to three round trips:
// (1) the token's sequence is found by counting the sequence starts at or below it, one start per thread
// (__syncthreads_count), not by a binary search of dependent loads; (2) the sequence's length and starts; (3) the
// block-table entry and the cos/sin row.  The token's own row is read in 16-byte pieces (four or eight rotation pairs
// per thread) when the rotary width allows it.
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
    int vec;           // rows, tables and the rotary width allow the 16-byte form of the rotation
};

// largest b with seqstart[b] <= t, found by the whole CTA: the starts are sorted, so b is the number of entries
// 1 .. batch-1 at or below t.  Every pass is one round of independent loads (one pass up to 129 sequences).
__device__ __forceinline__ int find_batch(const int64_t* seqstart, int batch, int64_t t) {
    int b = 0;
    for (int base = 1; base < batch; base += (int)blockDim.x) {
        const int i = base + (int)threadIdx.x;
        b += __syncthreads_count(i < batch && seqstart[i] <= t);
    }
    return b;
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

// The same rotation on 16-byte pieces: piece c of a head covers elements [8c, 8c + 8).  Interleaved pairs sit inside a
// piece (four pairs, cos/sin entries 4c .. 4c+3); half-rotated pairs are piece c of the first half with piece
// c + half/8 of the second (eight pairs, entries 8c .. 8c+7).  Needs rotary_dim % 8 == 0 (interleaved) or % 16 == 0
// (half-rotated) and 16-byte aligned rows and tables.  The arithmetic per pair is that of rope_heads.
template <typename T>
__device__ __forceinline__ void rope_pair(T x0, T x1, T c_, T s_, T& y0, T& y1) {
    const float a0 = Elem<T>::to_f32(x0), a1 = Elem<T>::to_f32(x1), c = Elem<T>::to_f32(c_), s = Elem<T>::to_f32(s_);
    y0 = Elem<T>::from_f32(__fsub_rn(__fmul_rn(a0, c), __fmul_rn(a1, s)));
    y1 = Elem<T>::from_f32(__fadd_rn(__fmul_rn(a0, s), __fmul_rn(a1, c)));
}
union Piece16 {
    uint4 v;
    uint2 h[2];
};
template <typename T>
__device__ __forceinline__ void rope_heads_vec(const T* src, T* dst, int heads, int d, int half, int rope_type,
                                               const T* cosr, const T* sinr, bool copy_tail) {
    const int rotary_dim = 2 * half, pieces = d / 8;
    for (int p = threadIdx.x; p < heads * pieces; p += blockDim.x) {
        const int h = p / pieces, c = p - h * pieces, e0 = 8 * c;
        const T* srow = src + (int64_t)h * d;
        T* drow = dst + (int64_t)h * d;
        if (e0 >= rotary_dim) {
            if (copy_tail) *reinterpret_cast<uint4*>(drow + e0) = *reinterpret_cast<const uint4*>(srow + e0);
            continue;
        }
        if (rope_type == 1) {
            Piece16 x, y;
            uint2 cw, sw;
            x.v = *reinterpret_cast<const uint4*>(srow + e0);
            cw = *reinterpret_cast<const uint2*>(cosr + e0 / 2);
            sw = *reinterpret_cast<const uint2*>(sinr + e0 / 2);
            const T* xe = reinterpret_cast<const T*>(&x);
            const T* ce = reinterpret_cast<const T*>(&cw);
            const T* se = reinterpret_cast<const T*>(&sw);
            T* ye = reinterpret_cast<T*>(&y);
#pragma unroll
            for (int i = 0; i < 4; ++i) rope_pair<T>(xe[2 * i], xe[2 * i + 1], ce[i], se[i], ye[2 * i], ye[2 * i + 1]);
            *reinterpret_cast<uint4*>(drow + e0) = y.v;
        } else if (e0 < half) {
            Piece16 x0, x1, y0, y1, cw, sw;
            x0.v = *reinterpret_cast<const uint4*>(srow + e0);
            x1.v = *reinterpret_cast<const uint4*>(srow + e0 + half);
            cw.v = *reinterpret_cast<const uint4*>(cosr + e0);
            sw.v = *reinterpret_cast<const uint4*>(sinr + e0);
            const T* a0 = reinterpret_cast<const T*>(&x0);
            const T* a1 = reinterpret_cast<const T*>(&x1);
            const T* ce = reinterpret_cast<const T*>(&cw);
            const T* se = reinterpret_cast<const T*>(&sw);
            T* b0 = reinterpret_cast<T*>(&y0);
            T* b1 = reinterpret_cast<T*>(&y1);
#pragma unroll
            for (int i = 0; i < 8; ++i) rope_pair<T>(a0[i], a1[i], ce[i], se[i], b0[i], b1[i]);
            *reinterpret_cast<uint4*>(drow + e0) = y0.v;
            *reinterpret_cast<uint4*>(drow + e0 + half) = y1.v;
        }
        // (pieces of the second half of a half-rotated head are written by their partners)
    }
}

template <typename T>
__global__ void __launch_bounds__(128) appendkv_kernel(const AppendDev a) {
    pdl_launch_dependents();  // the split-KV kernel that follows may set itself up while the tokens are written
    pdl_wait();               // the kernel before this one has completed (no-op after an ordinary launch)
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
        if (a.vec)
            rope_heads_vec<T>(ksrc, kdst, a.hkv, a.d, half, a.rope_type, (const T*)a.cosr + pos * half,
                              (const T*)a.sinr + pos * half, true);
        else
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
        if (a.vec)
            rope_heads_vec<T>(qrow, qrow, a.hq, a.d, half, a.rope_type, (const T*)a.cosr + pos * half,
                              (const T*)a.sinr + pos * half, false);
        else
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
    {
        const auto al16 = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15u) == 0; };
        const int unit = p.rope_type == 1 ? 8 : 16;  // rotary widths the 16-byte form covers
        a.vec = (p.rope_type == 0 || p.rotary_dim % unit == 0) && al16(p.q) && al16(p.k_cache) && al16(p.knew) &&
                (p.rope_type == 0 || (al16(p.rotary_cos) && al16(p.rotary_sin)));
    }
    const int64_t blocks = a.total_new + (p.rope_type != 0 ? a.total_q : 0);
    if (blocks == 0) return FLASHCK_OK;
    FCK_REQUIRE(blocks < (1ll << 31), FLASHCK_ERR_UNSUPPORTED, "appendkv: too many tokens");
    if (p.dtype == FLASHCK_DTYPE_BFLOAT16)
        FCK_CUDA(launch_dependent(appendkv_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(128), 0, stream, a));
    else
        FCK_CUDA(launch_dependent(appendkv_kernel<__half>, dim3((unsigned)blocks), dim3(128), 0, stream, a));
    return FLASHCK_OK;
}

}  // namespace fck
