// fmha_fwd / batch_prefill / paged-KV prefill -- the general instance.
// Covers every problem the reference's FmhaFwd family describes for the no-bias case
// (attention_kernels/fmha_fwd/fmha_fwd_jinja.h:124-147: batch and group mode, GQA, the four mask types with a
// [left,right] window) plus K/V behind a block table (fmha_fwd_paged_kv_prefill) or an SGLang-style page table
// (fmha_fwd_batch_prefill), for hdim 64/128 in fp16/bf16.  It is the instance the dispatcher falls back to when
// the tcgen05 prefill kernel does not cover a problem (hdim 64, paged K/V, odd masks).
//
// Tiling: one CTA = 64 query rows of one head (4 warps x 16 rows), 64 keys per step.  K and V tiles are
// gathered row by row with 16-byte cp.async (so paging costs one table lookup per row) into a double
// buffer with an XOR swizzle on the 16-byte chunk index, read back with ldmatrix and multiplied with
// mma.sync m16n8k16; fp32 online softmax in base 2 with quad-shuffle row reductions; P is rounded to the
// element dtype before PV and O is accumulated in fp32, as the reference's FmhaFwdTypeConfig prescribes
// (attention_kernels/fmha_common_jinja.h:120-155).  K/V tiles that the mask hides completely are skipped.
#include <cuda_fp8.h>

#include <type_traits>

#include "kernels.h"

namespace fck {

namespace {

constexpr int BM = 64, BN = 64, NWARP = 4;

struct FwdDev {
    const void* q;
    const void* k;
    const void* v;
    void* o;
    float* lse;
    const int64_t* seqstart_q;
    const int64_t* seqstart_k;
    const int64_t* seqlen_k64;
    const int32_t* seqlen_k32;
    const int32_t* block_table;
    const int32_t* kv_indptr;
    const int32_t* kv_page_indices;
    const int32_t* kv_last_page_len;
    const int64_t* cache_batch_idx;
    int batch, seqlen_q, seqlen_k, hq, hkv, total_q, bt_stride, page;
    int mask_type, wl, wr;
    float scale_log2;
    // instances with score additions (template parameter EXTRA)
    const void* bias;
    int bias_type, bias_rank;
    int64_t bias_sk;       // row stride of an elementwise bias (key length, packed total in group mode)
    int64_t bias_sq;       // rows of one head's bias plane
    float soft_cap;        // 0 = off
    float scale;
    // 8-bit instances (template parameter F8): P is stretched by scale_p before it is rounded to 8 bits, the accumulator
    // is taken to the range of O by scale_o (attention_kernels/fmha_fwd/fmha_fwd_jinja.h:326-328); O leaves as out_dtype
    float scale_p, scale_o;
    int out_dtype;
};

// 8 consecutive 8-bit floats (one uint2) as 8 halves (one uint4): exact, every E4M3 / E5M2 value is a half.
template <int F8>
__device__ __forceinline__ uint4 f8x8_to_half8(uint2 v) {
    constexpr __nv_fp8_interpretation_t kind = F8 == 1 ? __NV_E4M3 : __NV_E5M2;
    uint4 r;
    __half2_raw h;
    h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v.x & 0xffffu), kind); r.x = (uint32_t)h.x | ((uint32_t)h.y << 16);
    h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v.x >> 16), kind);     r.y = (uint32_t)h.x | ((uint32_t)h.y << 16);
    h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v.y & 0xffffu), kind); r.z = (uint32_t)h.x | ((uint32_t)h.y << 16);
    h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v.y >> 16), kind);     r.w = (uint32_t)h.x | ((uint32_t)h.y << 16);
    return r;
}
// Two probabilities rounded to the 8-bit type (nearest even, saturating) and handed to the MMA as the halves they equal.
template <int F8>
__device__ __forceinline__ uint32_t quantize_p2(float a, float b) {
    constexpr __nv_fp8_interpretation_t kind = F8 == 1 ? __NV_E4M3 : __NV_E5M2;
    const __nv_fp8x2_storage_t q = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, kind);
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(q, kind);
    return (uint32_t)h.x | ((uint32_t)h.y << 16);
}

// Row-major [rows][D] 16-bit tile; 16-byte chunk index XORed with (row & 7).
template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * (D * 2) + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4));
}

// EXTRA: the instance adds an elementwise bias or ALiBi to the scaled scores and/or soft-caps them (the reference
// compiles these as separate kernel instances too: bias_enum and has_logits_soft_cap are part of the instance name,
// core/profiling/attention/fmha_fwd/fmha_fwd_problem.h:59-64).
// F8: 0 = Q/K/V/O are stored as T.  1 (E4M3) / 2 (E5M2): the 8-bit instances of the reference's FmhaFwdTypeConfig<fp8_t /
// bf8_t> (attention_kernels/fmha_common_jinja.h:157-187): Q, K, V arrive as 8-bit floats and are widened to halves on
// their way into shared memory (exact), so the two GEMMs multiply exactly the 8-bit values with fp32 accumulation; P is
// rounded to the 8-bit type before the second GEMM; T must be __half.  (A tensor-core instance that keeps the operands
// at 8 bits moves half the shared-memory bytes and doubles the MMA rate; this one covers the arithmetic.)
template <typename T, int D, bool EXTRA, int F8 = 0>
__global__ void __launch_bounds__(NWARP * 32)
fmha_fwd_generic_kernel(const FwdDev p) {
    static_assert(F8 == 0 || std::is_same<T, __half>::value, "the 8-bit instances compute in half precision");
    constexpr int CH = D / 8;                    // 16-byte chunks per row
    constexpr int TILE = BN * D * 2;             // bytes of one K or V tile
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* sQ = smem;                          // BM x D
    uint8_t* sK = smem + BM * D * 2;             // 2 x (BN x D)
    uint8_t* sV = sK + 2 * TILE;                 // 2 x (BN x D)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = lane >> 2, qlane = lane & 3, lm = lane >> 3, lr = lane & 7;
    const int b = blockIdx.z, h = blockIdx.y;
    const int mtile = gridDim.x - 1 - blockIdx.x;  // longest (causal) tiles first
    const int G = p.hq / p.hkv, kh = h / G;

    const int64_t q0 = p.seqstart_q ? p.seqstart_q[b] : (int64_t)b * p.seqlen_q;
    const int sq = p.seqstart_q ? (int)(p.seqstart_q[b + 1] - p.seqstart_q[b]) : p.seqlen_q;
    const int m0 = mtile * BM;
    if (m0 >= sq) return;

    // ---- key length and K/V row addressing ----
    const int64_t bphys = p.cache_batch_idx ? p.cache_batch_idx[b] : b;
    int sk;
    const int32_t* pages = nullptr;  // page ids of this sequence (paged modes)
    int64_t row0 = 0;                // first token row (contiguous modes)
    if (p.kv_indptr) {
        const int pb = p.kv_indptr[b], pe = p.kv_indptr[b + 1];
        pages = p.kv_page_indices + pb;
        sk = pe > pb ? (pe - pb - 1) * p.page + p.kv_last_page_len[b] : 0;
    } else if (p.block_table) {
        pages = p.block_table + bphys * p.bt_stride;
        sk = p.seqlen_k32 ? p.seqlen_k32[b] : p.seqlen_k;
    } else {
        if (p.seqstart_k) {
            row0 = p.seqstart_k[b];
            sk = (int)(p.seqstart_k[b + 1] - p.seqstart_k[b]);
        } else {
            row0 = bphys * (int64_t)p.seqlen_k;
            sk = p.seqlen_k;
        }
        if (p.seqlen_k64) sk = (int)p.seqlen_k64[b];
        else if (p.seqlen_k32) sk = p.seqlen_k32[b];
    }
    auto token_row = [&](int j) -> int64_t {
        if (pages) return (int64_t)pages[j / p.page] * p.page + j % p.page;
        return row0 + j;
    };

    // ---- which key tiles can this row tile see ----
    const int m_last = min(sq, m0 + BM) - 1;
    int lo_first, hi_first, lo_last, hi_last;
    visible_range(m0, sq, sk, p.mask_type, p.wl, p.wr, lo_first, hi_first);
    visible_range(m_last, sq, sk, p.mask_type, p.wl, p.wr, lo_last, hi_last);
    const int n_begin = max(0, lo_first) / BN;
    const int n_end = min((sk + BN - 1) / BN, hi_last / BN + 1);  // hi_last < 0 => no tile

    // ---- async loads ----
    auto load_q = [&]() {
        for (int e = tid; e < BM * CH; e += NWARP * 32) {
            const int r = e / CH, c = e % CH;
            const bool ok = m0 + r < sq;
            if constexpr (F8 != 0) {
                const uint8_t* src = (const uint8_t*)p.q + ((q0 + m0 + (ok ? r : 0)) * p.hq + h) * D + c * 8;
                *reinterpret_cast<uint4*>(sQ + swz<D>(r, c)) =
                    ok ? f8x8_to_half8<F8>(*reinterpret_cast<const uint2*>(src)) : make_uint4(0u, 0u, 0u, 0u);
                continue;
            }
            const T* src = (const T*)p.q + ((q0 + m0 + (ok ? r : 0)) * p.hq + h) * D + c * 8;
            cp_async_16(smem_u32(sQ) + swz<D>(r, c), src, ok);
        }
    };
    auto load_kv = [&](int n, int buf) {
        const int c = tid % CH;
#pragma unroll
        for (int r = tid / CH; r < BN; r += (NWARP * 32) / CH) {
            const int j = n * BN + r;
            const bool ok = j < sk;
            const int64_t row = ok ? token_row(j) : 0;
            const size_t off = ((size_t)row * p.hkv + kh) * D + c * 8;
            if constexpr (F8 != 0) {  // (synchronous: the widening happens in registers)
                const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(sK + buf * TILE + swz<D>(r, c)) =
                    ok ? f8x8_to_half8<F8>(*reinterpret_cast<const uint2*>((const uint8_t*)p.k + off)) : zero;
                *reinterpret_cast<uint4*>(sV + buf * TILE + swz<D>(r, c)) =
                    ok ? f8x8_to_half8<F8>(*reinterpret_cast<const uint2*>((const uint8_t*)p.v + off)) : zero;
                continue;
            }
            cp_async_16(smem_u32(sK) + buf * TILE + swz<D>(r, c), (const T*)p.k + off, ok);
            cp_async_16(smem_u32(sV) + buf * TILE + swz<D>(r, c), (const T*)p.v + off, ok);
        }
    };

    load_q();
    if (n_begin < n_end) load_kv(n_begin, 0);
    cp_async_commit();

    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float mrow0 = -INFINITY, mrow1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    uint32_t qa[D / 16][4];

    const int i0 = m0 + warp * 16 + quad, i1 = i0 + 8;  // rows of this thread inside the sequence
    int lo0, hi0, lo1, hi1;
    visible_range(i0, sq, sk, p.mask_type, p.wl, p.wr, lo0, hi0);
    visible_range(i1, sq, sk, p.mask_type, p.wl, p.wr, lo1, hi1);

    // score additions of this (sequence, head): first bias element of the sequence's block, or the head's slope
    const T* bias_el = nullptr;
    float alibi_slope = 0.f;
    if (EXTRA && p.bias_type == 1) {
        const int64_t plane = p.bias_sq * p.bias_sk;
        const int64_t head_off = p.bias_rank >= 1 ? (int64_t)h * plane : 0;
        const int64_t batch_off = (p.bias_rank == 2 && !p.seqstart_q) ? (int64_t)b * p.hq * plane : 0;
        // group mode: the block of this sequence inside the packed [total_q, total_k] plane
        const int64_t blk = p.seqstart_q ? q0 * p.bias_sk + (p.seqstart_k ? p.seqstart_k[b] : 0) : 0;
        bias_el = (const T*)p.bias + batch_off + head_off + blk;
    } else if (EXTRA && p.bias_type == 2) {
        alibi_slope = ((const float*)p.bias)[(p.bias_rank >= 1 ? (int64_t)b * p.hq : 0) + h];
    }

    for (int n = n_begin; n < n_end; ++n) {
        const int buf = (n - n_begin) & 1;
        __syncthreads();  // everyone is done with the buffer the next load overwrites
        if (n + 1 < n_end) load_kv(n + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        if (n == n_begin) {  // Q fragments (each warp reads only its own 16 rows)
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const int r = warp * 16 + (lm & 1) * 8 + lr;
                const int c = 2 * ks + (lm >> 1);
                ldmatrix_x4(qa[ks], smem_u32(sQ) + swz<D>(r, c));
            }
        }
        const uint32_t kb = smem_u32(sK) + buf * TILE, vb = smem_u32(sV) + buf * TILE;

        // ---- S = Q K^T : 16 x 64 per warp ----
        float s[BN / 8][4];
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int jp = 0; jp < BN / 16; ++jp) {
                const int r = jp * 16 + (lm >> 1) * 8 + lr;
                const int c = 2 * ks + (lm & 1);
                uint32_t bfr[4];
                ldmatrix_x4(bfr, kb + swz<D>(r, c));
                mma_16816<T>(s[2 * jp], qa[ks], bfr[0], bfr[1]);
                mma_16816<T>(s[2 * jp + 1], qa[ks], bfr[2], bfr[3]);
            }
        }
        // ---- scale + mask ----
        const int k0 = n * BN;
        const bool need_mask = (k0 + BN > sk) || (p.mask_type != 0 && (k0 + BN - 1 > hi_first || k0 < lo_last));
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float x = s[j][e] * p.scale_log2;
                if (EXTRA) {
                    const int key = k0 + j * 8 + qlane * 2 + (e & 1), row = (e < 2) ? i0 : i1;
                    float y = s[j][e] * p.scale;
                    if (p.soft_cap > 0.f) y = p.soft_cap * tanh_inline(y / p.soft_cap);
                    if (p.bias_type == 1) {
                        if (row < sq && key < sk) y += Elem<T>::to_f32(bias_el[(int64_t)row * p.bias_sk + key]);
                    } else if (p.bias_type == 2) {
                        y -= alibi_slope * fabsf((float)(row + sk - sq - key));
                    }
                    x = y * 1.4426950408889634f;
                }
                if (need_mask) {
                    const int key = k0 + j * 8 + qlane * 2 + (e & 1);
                    const bool vis = (e < 2) ? (key >= lo0 && key <= hi0) : (key >= lo1 && key <= hi1);
                    if (!vis) x = -INFINITY;
                }
                s[j][e] = x;
            }
        }
        // ---- online softmax ----
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(mrow0, mx0), mn1 = fmaxf(mrow1, mx1);
        const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0, ms1 = (mn1 == -INFINITY) ? 0.f : mn1;
        const float a0 = fast_exp2(mrow0 - ms0), a1 = fast_exp2(mrow1 - ms1);
        mrow0 = mn0;
        mrow1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
            s[j][0] = fast_exp2(s[j][0] - ms0);
            s[j][1] = fast_exp2(s[j][1] - ms0);
            s[j][2] = fast_exp2(s[j][2] - ms1);
            s[j][3] = fast_exp2(s[j][3] - ms1);
            ps0 += s[j][0] + s[j][1];
            ps1 += s[j][2] + s[j][3];
        }
        l0 = l0 * a0 + ps0;
        l1 = l1 * a1 + ps1;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            o[j][0] *= a0;
            o[j][1] *= a0;
            o[j][2] *= a1;
            o[j][3] *= a1;
        }
        // ---- O += P V ----
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t pa[4];
            if constexpr (F8 != 0) {
                pa[0] = quantize_p2<F8>(s[2 * kk][0] * p.scale_p, s[2 * kk][1] * p.scale_p);
                pa[1] = quantize_p2<F8>(s[2 * kk][2] * p.scale_p, s[2 * kk][3] * p.scale_p);
                pa[2] = quantize_p2<F8>(s[2 * kk + 1][0] * p.scale_p, s[2 * kk + 1][1] * p.scale_p);
                pa[3] = quantize_p2<F8>(s[2 * kk + 1][2] * p.scale_p, s[2 * kk + 1][3] * p.scale_p);
            } else {
                pa[0] = Elem<T>::pack2(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = Elem<T>::pack2(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = Elem<T>::pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = Elem<T>::pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            }
#pragma unroll
            for (int j = 0; j < D / 16; ++j) {
                const int r = kk * 16 + (lm & 1) * 8 + lr;
                const int c = 2 * j + (lm >> 1);
                uint32_t bfr[4];
                ldmatrix_x4_trans(bfr, vb + swz<D>(r, c));
                mma_16816<T>(o[2 * j], pa, bfr[0], bfr[1]);
                mma_16816<T>(o[2 * j + 1], pa, bfr[2], bfr[3]);
            }
        }
    }
    cp_async_wait<0>();
    if (n_begin >= n_end) __syncthreads();  // no key tile: the Q copies of other threads must land before sQ is reused

    // ---- epilogue ----
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if constexpr (F8 != 0) {
        // O = scale_o * acc / l in the output type the call names: 8-bit (saturating) or 16-bit; each thread stores its
        // two neighbouring columns of its two rows
        const float f0 = inv0 * p.scale_o, f1 = inv1 * p.scale_o;
        auto put = [&](int row, int col, float a, float b) {
            const int64_t idx = ((q0 + row) * p.hq + h) * D + col;
            if (p.out_dtype == FLASHCK_DTYPE_FLOAT8 || p.out_dtype == FLASHCK_DTYPE_BFLOAT8)
                *reinterpret_cast<uint16_t*>((uint8_t*)p.o + idx) = (uint16_t)__nv_cvt_float2_to_fp8x2(
                    make_float2(a, b), __NV_SATFINITE, p.out_dtype == FLASHCK_DTYPE_FLOAT8 ? __NV_E4M3 : __NV_E5M2);
            else if (p.out_dtype == FLASHCK_DTYPE_BFLOAT16)
                *reinterpret_cast<uint32_t*>((__nv_bfloat16*)p.o + idx) = Elem<__nv_bfloat16>::pack2(a, b);
            else
                *reinterpret_cast<uint32_t*>((__half*)p.o + idx) = Elem<__half>::pack2(a, b);
        };
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            if (i0 < sq) put(i0, j * 8 + qlane * 2, o[j][0] * f0, o[j][1] * f0);
            if (i1 < sq) put(i1, j * 8 + qlane * 2, o[j][2] * f1, o[j][3] * f1);
        }
    } else {
    // stage the 16 x D tile of this warp in its own rows of the Q buffer, then store 16-byte vectors
    __syncwarp();
    {
        const int r0 = warp * 16 + quad, r1 = r0 + 8;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            *reinterpret_cast<uint32_t*>(sQ + swz<D>(r0, j) + qlane * 4) = Elem<T>::pack2(o[j][0] * inv0, o[j][1] * inv0);
            *reinterpret_cast<uint32_t*>(sQ + swz<D>(r1, j) + qlane * 4) = Elem<T>::pack2(o[j][2] * inv1, o[j][3] * inv1);
        }
    }
    __syncwarp();
    for (int e = lane; e < 16 * CH; e += 32) {
        const int r = warp * 16 + e / CH, c = e % CH;
        if (m0 + r < sq) {
            const uint4 val = *reinterpret_cast<const uint4*>(sQ + swz<D>(r, c));
            *reinterpret_cast<uint4*>((T*)p.o + ((q0 + m0 + r) * p.hq + h) * D + c * 8) = val;
        }
    }
    }
    if (p.lse && qlane == 0) {
        const float kLn2 = 0.6931471805599453f;
        float* base = p.seqstart_q ? p.lse + (int64_t)h * p.total_q + q0 : p.lse + ((int64_t)b * p.hq + h) * p.seqlen_q;
        if (i0 < sq) base[i0] = l0 > 0.f ? (mrow0 + log2f(l0)) * kLn2 : -INFINITY;
        if (i1 < sq) base[i1] = l1 > 0.f ? (mrow1 + log2f(l1)) * kLn2 : -INFINITY;
    }
}

template <typename T, int D, bool EXTRA>
int launch_inst(const FwdParams& p, const FwdDev& dev, cudaStream_t stream) {
    auto kern = fmha_fwd_generic_kernel<T, D, EXTRA>;
    const size_t smem = (size_t)(BM + 4 * BN) * D * 2;
    static thread_local int configured_device = -1;
    int devid = 0;
    FCK_CUDA(cudaGetDevice(&devid));
    if (configured_device != devid) {
        FCK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured_device = devid;
    }
    const int mtiles = (int)((p.max_seqlen_q + BM - 1) / BM);
    if (mtiles == 0 || p.batch == 0) return FLASHCK_OK;
    FCK_REQUIRE(p.hq <= 65535 && p.batch <= 65535, FLASHCK_ERR_UNSUPPORTED, "fmha_fwd: nhead_q and batch must be <= 65535");
    dim3 grid(mtiles, (unsigned)p.hq, (unsigned)p.batch);
    kern<<<grid, NWARP * 32, smem, stream>>>(dev);
    FCK_CUDA(cudaGetLastError());
    return FLASHCK_OK;
}

}  // namespace

template <int D, int F8>
int launch_inst_f8(const FwdParams& p, const FwdDev& dev, cudaStream_t stream) {
    auto kern = fmha_fwd_generic_kernel<__half, D, false, F8>;
    const size_t smem = (size_t)(BM + 4 * BN) * D * 2;
    static thread_local int configured_device = -1;
    int devid = 0;
    FCK_CUDA(cudaGetDevice(&devid));
    if (configured_device != devid) {
        FCK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured_device = devid;
    }
    const int mtiles = (int)((p.max_seqlen_q + BM - 1) / BM);
    if (mtiles == 0 || p.batch == 0) return FLASHCK_OK;
    FCK_REQUIRE(p.hq <= 65535 && p.batch <= 65535, FLASHCK_ERR_UNSUPPORTED, "fmha_fwd: nhead_q and batch must be <= 65535");
    kern<<<dim3(mtiles, (unsigned)p.hq, (unsigned)p.batch), NWARP * 32, smem, stream>>>(dev);
    FCK_CUDA(cudaGetLastError());
    return FLASHCK_OK;
}

int launch_fwd_generic(const FwdParams& p, cudaStream_t stream) {
    FCK_REQUIRE(p.d == p.dv && (p.d == 64 || p.d == 128), FLASHCK_ERR_UNSUPPORTED,
                "fmha_fwd: hdim_q == hdim_v in {64,128} required (got %lld/%lld)", (long long)p.d, (long long)p.dv);
    FwdDev dev;
    dev.scale_p = p.scale_p; dev.scale_o = p.scale_o; dev.out_dtype = p.out_dtype;
    dev.q = p.q; dev.k = p.k; dev.v = p.v; dev.o = p.o; dev.lse = p.lse;
    dev.seqstart_q = p.seqstart_q; dev.seqstart_k = p.seqstart_k;
    dev.seqlen_k64 = p.seqlen_k64; dev.seqlen_k32 = p.seqlen_k32;
    dev.block_table = p.block_table; dev.kv_indptr = p.kv_indptr; dev.kv_page_indices = p.kv_page_indices;
    dev.kv_last_page_len = p.kv_last_page_len; dev.cache_batch_idx = p.cache_batch_idx;
    dev.batch = (int)p.batch; dev.seqlen_q = (int)p.seqlen_q; dev.seqlen_k = (int)p.seqlen_k;
    dev.hq = (int)p.hq; dev.hkv = (int)p.hkv; dev.total_q = (int)p.total_q;
    dev.bt_stride = (int)p.bt_stride; dev.page = (int)(p.page > 0 ? p.page : 1);
    dev.mask_type = p.mask_type;
    dev.wl = (int)(p.wl < 0 ? -1 : (p.wl > 0x3fffffff ? 0x3fffffff : p.wl));
    dev.wr = (int)(p.wr < 0 ? -1 : (p.wr > 0x3fffffff ? 0x3fffffff : p.wr));
    dev.scale_log2 = p.scale * 1.4426950408889634f;
    dev.bias = p.bias; dev.bias_type = p.bias ? p.bias_type : 0; dev.bias_rank = p.bias_rank;
    dev.bias_sk = p.seqlen_k; dev.bias_sq = p.seqstart_q ? p.total_q : p.seqlen_q;
    dev.soft_cap = p.logits_soft_cap; dev.scale = p.scale;
    if (p.dtype == FLASHCK_DTYPE_FLOAT8 || p.dtype == FLASHCK_DTYPE_BFLOAT8) {
        FCK_REQUIRE(dev.bias_type == 0 && dev.soft_cap == 0.f, FLASHCK_ERR_UNSUPPORTED,
                    "fmha_fwd: the 8-bit instances take no bias and no soft cap");
        if (p.dtype == FLASHCK_DTYPE_FLOAT8)
            return p.d == 128 ? launch_inst_f8<128, 1>(p, dev, stream) : launch_inst_f8<64, 1>(p, dev, stream);
        return p.d == 128 ? launch_inst_f8<128, 2>(p, dev, stream) : launch_inst_f8<64, 2>(p, dev, stream);
    }
    const bool bf16 = p.dtype == FLASHCK_DTYPE_BFLOAT16;
    if (dev.bias_type != 0 || dev.soft_cap > 0.f) {
        FCK_REQUIRE(dev.bias_type != 1 || !(p.block_table || p.kv_indptr || p.cache_batch_idx || p.seqlen_k32 || p.seqlen_k64),
                    FLASHCK_ERR_UNSUPPORTED, "fmha_fwd: an elementwise bias needs contiguous K/V of the stated length");
        if (bf16)
            return p.d == 128 ? launch_inst<__nv_bfloat16, 128, true>(p, dev, stream)
                              : launch_inst<__nv_bfloat16, 64, true>(p, dev, stream);
        return p.d == 128 ? launch_inst<__half, 128, true>(p, dev, stream) : launch_inst<__half, 64, true>(p, dev, stream);
    }
    if (bf16)
        return p.d == 128 ? launch_inst<__nv_bfloat16, 128, false>(p, dev, stream)
                          : launch_inst<__nv_bfloat16, 64, false>(p, dev, stream);
    return p.d == 128 ? launch_inst<__half, 128, false>(p, dev, stream) : launch_inst<__half, 64, false>(p, dev, stream);
}

}  // namespace fck
