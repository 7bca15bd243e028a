// fmha_fwd / batch prefill / paged prefill / multi-token split-KV -- the tcgen05 instance (hdim 128).
// Replaces ck_tile::FmhaFwdKernel<BlockFmhaPipelineQRKSVS...> as instantiated by the reference
// (core/profiling/attention/fmha_fwd/fmha_fwd_codegen.cc:86-118) behind the C symbol FmhaFwd
// (attention_kernels/fmha_fwd/fmha_fwd_jinja.h:124-147), batch and group mode, GQA, fp32 LSE; the paged variants
// (fmha_fwd_batch_prefill_codegen.cc:93-162, fmha_fwd_paged_kv_prefill_codegen.cc:85-144) read K/V through a page list;
// and, behind FmhaFwdSplitKV (fmha_fwd_split_kv_jinja.h:155-184), the calls with more than one 16-row tile of query
// rows per kv head (the "split modes" described at Sm100Dev and at the kernel template).
//
// Persistent kernel: one CTA per SM (384 threads; it owns all 512 TMEM columns) walks a work list that every CTA
// derives on chip from the sequence lengths: items sorted by decreasing row-block index (decreasing cost under a
// causal mask), dealt to the CTAs in snake order.  A work item is two 128-row Q tiles that share their K/V tiles:
// the same rows of two neighbouring q heads of a GQA group when the group size is even (both tiles then run the
// same number of steps and meet the diagonal together), else two consecutive row tiles of one head.  The two
// tiles ping-pong through the pipeline:
//   warp 9      TMA producer: Q tiles of the item (4 boxes of 64 x 128, 128-byte swizzle), then K and V tiles of
//               128 keys into two-slot rings that run on across work items; mbarrier expect-tx.  Paged K/V: one box
//               per page chunk and 64-column half, each lane issuing its own chunk's boxes; the tail of a sequence's
//               last page is kept out of V (its rows are overwritten with zeros once the copy has landed).
//   warp 8      MMA issuer (one elected thread): S_i = Q_i K^T with tcgen05.mma (both operands in shared
//               memory, K-major), O_i += P_i V with the A operand P_i read from tensor memory and V taken
//               MN-major straight from its [key][hdim] tile.  Accumulators live in TMEM: S0,S1 (128 columns
//               each, fp32) and O0,O1 (128 columns each).  tcgen05.commit signals the consumers.  Shared-memory
//               descriptors are built once; per instruction only the start-address field advances.
//   warps 0-3 / 4-7   softmax warpgroup of tile 0 / 1: thread r owns row r (TMEM lane r), so row max and row sum
//               need no shuffles.  tcgen05.ld S -> registers, fp32 online softmax in base 2 with packed f32x2
//               arithmetic, P rounded to the element dtype and stored with tcgen05.st over the first 64 columns
//               of S_i (the next QK^T of the tile is issued after the PV that reads P, and the tensor pipe runs
//               in order).  The running max is only raised -- and O_i rescaled in TMEM -- when it grows by more
//               than 2^8, so the correction is off the steady-state path; the final 1/l normalisation and the
//               O / LSE stores (O through shared memory and TMA stores) are done by the same warpgroup while the
//               MMA warp already starts the next item.
// K/V tiles hidden by the mask are skipped (a left window also skips the tiles before it); only boundary tiles pay
// for masking.  The GQA group's q heads run in neighbouring CTAs and share K/V through L2 (no cluster multicast).
// Every mbarrier wait is bounded; on expiry the CTA records a code in the device status word and drains.
#include <algorithm>
#include <atomic>
#include <string.h>
#include <type_traits>

#include <cuda_fp8.h>

#include "kernels.h"

namespace fck {

namespace {

constexpr int BM = 128;        // rows per Q tile
constexpr int BN = 128;        // keys per K/V tile
constexpr int HD = 128;        // head dim
constexpr int KV_SLOTS = 2;
constexpr int TILE_BYTES = BM * HD * 2;   // 32 KB: one Q, K or V tile
constexpr int HALF_BYTES = BM * 128;      // one 64-column block (128 rows x 128 B); hdim 128 has two, hdim 64 one
constexpr int NTHREADS = 384;
constexpr float kRescaleThreshold = 8.f;  // log2 units; fp32 exponentials: P stays below 2^8
// With the packed f16x2 exp2 the threshold also bounds the rounding of the arguments (f16 spacing grows with the
// magnitude): 2 keeps an argument above the running max within 2^-11, at the price of a few more O rescales in the
// first tiles of a row.  Instance parameter "rescale_log2_x100".
std::atomic<int64_t> g_rescale_half_x100{200};

std::atomic<int64_t> g_use_sm100{1};
std::atomic<int64_t> g_use_sm100_bias{1};    // elementwise bias tensors (hdim 128, contiguous) on the tcgen05 instance (0: general)
std::atomic<int64_t> g_use_sm100_fp8{1};     // 8-bit prefill (hdim 128, contiguous) on the tcgen05 instance (0: general)
std::atomic<int64_t> g_use_sm100_hdim64{1};  // hdim-64 prefill on the tcgen05 instance (0: on the general one)
// exponentials of the softmax (template parameter EXPM of the kernel): 0 fp32 on the exp2 unit, 1 packed f16x2 on the
// exp2 unit, 11 / 12 / 13 fp32 with 1 / 2 / 3 of every 8 column pairs on an FMA-pipe polynomial
// (measured on B200, BASELINE config 2, bf16: 0 -> 962 TFLOP/s; 1 -> 915 at a rescale threshold of 4 and up, 866 at 2,
// with the LSE of a row that one late key dominates off by up to 9.7e-4; 11 / 12 / 13 -> 934 / 916 / 883: the unpacking
// of the packed results and the polynomial both cost the softmax warps more issue slots than the exp2 unit gives back)
std::atomic<int64_t> g_exp_mode{0};
std::atomic<int64_t> g_exp_mode_splitkv{0};
std::atomic<int64_t> g_use_sm100_splitkv{1};  // multi-token split-KV on the tcgen05 instance

struct Sm100Dev {
    void* o;
    float* lse;
    const int64_t* seqstart_q;
    const int64_t* seqstart_k;
    int* status;
    int batch, seqlen_q, seqlen_k, hq, hkv, total_q;
    // paged K/V (page > 0): pools [num_pages, page, hkv, 128]; a sequence's page ids are page_ids[k0 ...] with k0 the
    // sequence's offset into the list (block table row or kv_indptr entry)
    const void* v;
    const int32_t* page_ids;
    const int32_t* kv_indptr;
    const int32_t* kv_last_page_len;
    const int32_t* seqlen_k32;
    const int64_t* cache_batch_idx;
    int page, bt_stride;
    // split mode (FmhaFwdSplitKV with several query rows per kv head): work item = (sequence, kv head, 128-row block,
    // run of key tiles); its Q tile holds the (token, group head) rows of that kv head; the result is one split of the
    // caller's fp32 workspaces.  `piece_tiles` is the shortest piece the work is cut into.
    float* o_acc;
    float* lse_acc;
    int num_splits, piece_tiles, group, sq_cap;
    int item_cost;    // units of the work line that stand for an item's fixed cost (see kItemCostDefault)
    int causal;       // mask type: 0 none, 1 top-left, 2 bottom-right, 3 window with top-left alignment
    int wl, wr;       // window of a masked problem: keys [i + shift - wl, i + shift + wr] of row i; -1 = unbounded
    int num_levels;   // row blocks of the longest sequence (128 rows when heads are paired, else 256)
    int pair_heads;   // the two Q tiles of a work item are two q heads of one kv group
    float scale_log2;
    float scale;            // EXTRA instances: the softmax scale itself
    float soft_cap;         // EXTRA: 0 = off
    const float* alibi;     // EXTRA: fp32 slopes [1,hq] (alibi_rank 0) or [batch,hq] (1), or nullptr
    int alibi_rank;
    float rescale_thr;  // the running max is raised (and O rescaled) when the row max exceeds it by more than this (log2 units)
    // 8-bit instances: P is stretched by scale_p before it is rounded to 8 bits, the accumulator is taken to the range of
    // O by scale_o; O leaves as out_dtype (a FLASHCK_DTYPE_* code: 8-bit saturating, or 16-bit)
    float scale_p, scale_o;
    int out_dtype;
    // BIAS instances: an elementwise bias in the element type, planes of bias_sq rows x bias_sk keys (the packed totals in
    // group mode, where a sequence's block starts at (seqstart_q[b], seqstart_k[b])); rank 0 = one plane, 1 = one per
    // head, 2 = one per (batch, head) (batch mode only)
    const void* bias_el;
    int bias_el_rank;
    int64_t bias_sk, bias_sq;
};

// ---- PTX wrappers ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of sm_100
    d |= (uint64_t)2 << 61;  // 128-byte swizzle
    return d;
}
// F8 = false: kind::f16 (16-bit operands, K = 16 per instruction); true: kind::f8f6f4 (8-bit operands, K = 32).
template <bool F8 = false>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    if constexpr (F8)
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
            : "memory");
    else
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
            : "memory");
}
template <bool F8 = false>
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    if constexpr (F8)
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
            "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
            : "memory");
    else
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
            "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
            : "memory");
}
__device__ __forceinline__ bool elect_one_sync() {  // true in exactly one lane of a converged warp
    uint32_t pred;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
        "%30,%31,%32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3,%4,%5}], [%2];\n" ::
            "r"(smem_u32(smem_dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2,%3,%4}], [%1];\n" ::"l"(map),
                 "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// Element tags of the 8-bit instances (Q, K, V and P in one of the two OCP 8-bit float formats; kind::f8f6f4).
struct f8e4m3_t {};
struct f8e5m2_t {};
template <typename T> struct ElemInfo { static constexpr int bytes = 2; static constexpr bool f8 = false; };
template <> struct ElemInfo<f8e4m3_t> { static constexpr int bytes = 1; static constexpr bool f8 = true; };
template <> struct ElemInfo<f8e5m2_t> { static constexpr int bytes = 1; static constexpr bool f8 = true; };

// Instruction descriptor of tcgen05.mma kind::f16 / kind::f8f6f4: D = f32 (bits 4-5 = 1); A/B format at bits 7-9 /
// 10-12 (kind::f16: 0 = f16, 1 = bf16; kind::f8f6f4: 0 = E4M3, 1 = E5M2); bit 16: B is MN-major; N >> 3 at bits 17-22;
// M >> 4 at bits 24-28.
template <typename T> struct UmmaFmt;
template <> struct UmmaFmt<__half> { static constexpr uint32_t v = 0u; };
template <> struct UmmaFmt<__nv_bfloat16> { static constexpr uint32_t v = 1u; };
template <> struct UmmaFmt<f8e4m3_t> { static constexpr uint32_t v = 0u; };
template <> struct UmmaFmt<f8e5m2_t> { static constexpr uint32_t v = 1u; };
template <typename T>
__device__ __forceinline__ constexpr uint32_t make_idesc(bool b_mn_major, int n = BN) {
    return (1u << 4) | (UmmaFmt<T>::v << 7) | (UmmaFmt<T>::v << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// Eight bias values (16 bytes) of one score row starting at element `row + col`, of which the first `nvalid` exist: one
// 16-byte load when the piece is aligned and whole, element loads (zeros past the end) otherwise.  row == nullptr (a
// row past the end of its sequence): zeros.
__device__ __forceinline__ uint4 load_bias_piece(const unsigned short* row, int col, int nvalid) {
    uint4 r = make_uint4(0u, 0u, 0u, 0u);
    if (row == nullptr || nvalid <= 0) return r;
    const unsigned short* ptr = row + col;
    if (nvalid >= 8 && (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0) return __ldg(reinterpret_cast<const uint4*>(ptr));
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t lo = 2 * j < nvalid ? (uint32_t)__ldg(ptr + 2 * j) : 0u;
        const uint32_t hi = 2 * j + 1 < nvalid ? (uint32_t)__ldg(ptr + 2 * j + 1) : 0u;
        w[j] = lo | (hi << 16);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
template <typename T>
__device__ __forceinline__ float bias_elem(uint32_t w, int hi);
template <>
__device__ __forceinline__ float bias_elem<__nv_bfloat16>(uint32_t w, int hi) {
    return __uint_as_float(hi ? (w & 0xffff0000u) : (w << 16));
}
template <>
__device__ __forceinline__ float bias_elem<__half>(uint32_t w, int hi) {
    return __half2float(__ushort_as_half((unsigned short)(hi ? (w >> 16) : (w & 0xffffu))));
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float ex2_fast(float x) {  // not volatile: the compiler may schedule it freely
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// 2^x for two values on the FMA pipe with packed f32x2 arithmetic: round-to-nearest split x = n + f,
// f in [-0.5, 0.5], cubic for 2^f (max relative error 7.5e-5, far below the rounding of P to 16 bits), then n is
// added to the exponent field.  The exp2 unit delivers 16 results per clock per SM -- as many cycles per
// 128x128 tile as the two MMAs take -- so a share of the elements goes this way instead.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
    x.x = fmaxf(x.x, -126.f);
    x.y = fmaxf(x.y, -126.f);
    const float2 t = __fadd2_rn(x, make_float2(12582912.f, 12582912.f));  // 1.5 * 2^23: n lands in the low mantissa bits
    const float2 nf = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
    const float2 f = __ffma2_rn(nf, make_float2(-1.f, -1.f), x);
    float2 pl = __ffma2_rn(make_float2(0.055171605f, 0.055171605f), f, make_float2(0.24261111f, 0.24261111f));
    pl = __ffma2_rn(pl, f, make_float2(0.69326097f, 0.69326097f));
    pl = __ffma2_rn(pl, f, make_float2(0.99992806f, 0.99992806f));
    float2 r;
    r.x = __int_as_float(__float_as_int(pl.x) + (__float_as_int(t.x) << 23));
    r.y = __int_as_float(__float_as_int(pl.y) + (__float_as_int(t.y) << 23));
    return r;
}

// 2^x for two values with one instruction of the exp2 unit: the arguments are packed to f16x2 and the unit's packed
// half-precision form returns both results, so a 128-column row costs 64 issues of that unit instead of 128 -- at
// hdim 128 the exp2 unit is otherwise busy as long as the tensor pipe.  The arguments are <= the rescale threshold (the
// running max lags the true max by at most that much; 2 with this form), far inside the f16 range; f16 carries 11 significant bits, so an argument
// in [-2, 2] is off by at most 2^-11 (a factor of 1 +- 3.4e-4 in P) and the result is rounded to 11 bits -- P is rounded
// to the 8 (bf16) or 11 (fp16) bits of the element type anyway, and the row sum averages the rounding over the keys.
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;\n" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t ex2_f16x2(uint32_t x) {
    uint32_t y;
    asm("ex2.approx.f16x2 %0, %1;\n" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ float2 unpack_f16x2(uint32_t v) {
    float2 r;
    asm("{\n.reg .f16 l, h;\nmov.b32 {l, h}, %2;\ncvt.f32.f16 %0, l;\ncvt.f32.f16 %1, h;\n}\n" : "=f"(r.x), "=f"(r.y) : "r"(v));
    return r;
}
// acc.x += low half, acc.y += high half, each as one mixed-precision add (f16 operand, fp32 sum)
__device__ __forceinline__ void add_f16x2_to(float2& acc, uint32_t v) {
    asm("{\n.reg .f16 l, h;\nmov.b32 {l, h}, %2;\nadd.f32.f16 %0, l, %0;\nadd.f32.f16 %1, h, %1;\n}\n"
        : "+f"(acc.x), "+f"(acc.y)
        : "r"(v));
}

constexpr int kMaxBatch = 256;    // sequences the on-chip schedule can hold (larger batches use the general instance)
constexpr int kMaxLevels = 512;   // row blocks per sequence the on-chip schedule can hold
constexpr int STAGE_BYTES = 32 * 32 * 2;  // per softmax warp: 32 rows x 32 columns of O on their way to a TMA store
constexpr int kMaxRounds = 1024;  // work items per CTA (the host sends larger problems to the general instance)
constexpr int kSplitItems = 2560; // the same for the split modes (their list needs one word per item)

// One work item = two 128-row Q tiles that share their K/V tiles.  With an even GQA ratio the tiles are the same
// 128 rows of two neighbouring q heads of one kv group: both see the same keys, so they run the same number of
// steps and hit the diagonal together.  Otherwise they are two consecutive row tiles of one head.
struct Item {
    int valid;
    int b, kh, sq, sk, shift, N;
    int h[2];     // q head of each tile
    int row0[2];  // first row (inside the sequence) of each tile
    int nt[2];    // key tiles each Q tile needs (0: the tile does not exist or sees nothing)
    int n0;       // first key tile of the item (a left window skips the tiles before it)
    int q0, k0;   // first row of the sequence in the packed Q / K buffers
};

// Shared-memory control block placed after the tiles.
struct Ctrl {
    uint64_t q_full, q_empty;
    uint64_t k_full[3], k_empty[3], v_full[KV_SLOTS], v_empty[KV_SLOTS];  // (the split modes use a third K slot)
    uint64_t s_full[2], p_full[2], o_full[2];
    uint64_t p_full2[2];  // prefill forms: the second half of P (keys 64-127) has been written (p_full: the first half)
    uint64_t pv_done[2];  // split modes: the PV that read S/P buffer b is complete (buffer b may take the next S)
    uint64_t v_tail;      // paged V: the copies of a tile that holds the end of its sequence (cleaned up before v_full)
    uint32_t tmem_base;
    int abort_flag;
    int num_levels;                     // row-block indices 0 .. num_levels-1
    int level_start[kMaxLevels + 1];    // first work item of each level; level 0 = highest block index
    int nblk[kMaxBatch];                // row blocks of each sequence
    int seq_q0[kMaxBatch], seq_sq[kMaxBatch], seq_k0[kMaxBatch], seq_sk[kMaxBatch];  // first row / length, Q and K
    // this CTA's work list: valid << 31 | sequence << 22 | head index << 12 | row block (split modes: split << 4 | block)
    uint32_t items[kSplitItems];
    int split_w, split_items;           // split modes: length of a CTA's piece of the work stream; items of this CTA
    // split modes: every item takes all key tiles of its stream, except that the first item of the list may start
    // inside its stream (at this tile) and the last one may end inside it (before this tile)
    int split_first_lo, split_last_hi;
};

// Item taken by CTA `cta` in round `rnd` of a grid of `g` CTAs: rounds alternate direction (snake order), so that
// with items sorted by decreasing cost no CTA collects the most expensive item of every round.
__device__ __forceinline__ int item_of_round(int rnd, int cta, int g) {
    return rnd * g + ((rnd & 1) ? (g - 1 - cta) : cta);
}

// Work items are ordered by decreasing row-block index (under a causal mask: decreasing cost), then by sequence,
// then by head, so that the q heads of a GQA group -- which read the same K/V -- run at the same time on
// neighbouring SMs and share those tiles through L2.  Warp-collective.
static_assert(1024 + (2 + 2 * KV_SLOTS) * TILE_BYTES + 8 * STAGE_BYTES + sizeof(Ctrl) <= 227 * 1024,
              "tiles, staging buffers and the control block must fit the 227 KB a CTA can have");

// Split modes.  A stream is the key tiles one (sequence, 128-row block of the packed rows, kv head) needs; all streams,
// in that order, each preceded by item_cost units (kItemCostDefault) that stand for an item's fixed cost (Q load, pipeline fill, epilogue),
// form one line that is cut into equal pieces of split_w units, one per CTA, so that the SMs finish together whatever
// the lengths are.  The part of a stream inside one CTA's piece is a work item and one split of the result; a stream
// cut k times uses splits 0..k.  split_w is raised where needed so that no stream needs more splits than the
// workspace has; with a single split per stream the whole stream goes to the CTA its start falls to.
constexpr int kItemCostDefault = 6;   // instance parameter "split_item_cost" (1 .. 64)
std::atomic<int64_t> g_split_item_cost{kItemCostDefault};
std::atomic<int64_t> g_split_min_piece_tiles{8};  // instance parameter "split_min_piece_tiles": at least 1024 keys per work item

// key tiles the rows of row block `rb` of a sequence see
__device__ __forceinline__ int split_stream_tiles(const Sm100Dev& p, int sq, int sk, int rb) {
    const int first_tok = rb * BM / p.group;
    if (first_tok >= sq || sk <= 0) return 0;
    int hi_key = sk - 1;
    if (p.causal) {
        const int last_tok = min(sq, (rb * BM + BM + p.group - 1) / p.group) - 1;
        hi_key = min(hi_key, last_tok + ((p.causal == 2) ? sk - sq : 0));
    }
    return hi_key >= 0 ? hi_key / BN + 1 : 0;
}

// splits a stream of n tiles starting at unit g0 of the line uses (pieces; the mode with duplicated rows writes two per piece)
__device__ __forceinline__ int split_stream_pieces(int g0, int n, int w, int max_pieces, int item_cost) {
    if (n == 0 || max_pieces == 1) return 1;
    return (g0 + item_cost + n - 1) / w - (g0 + item_cost) / w + 1;
}

__device__ __forceinline__ void expand_item_split(const Ctrl* ctrl, const Sm100Dev& p, uint32_t packed, int rnd, Item& it) {
    it.valid = packed >> 31;
    const int b = (packed >> 22) & 0x1ff, kh = (packed >> 12) & 0x3ff, piece = (packed >> 4) & 0xff, rb = packed & 0xf;
    it.b = b;
    it.q0 = ctrl->seq_q0[b];
    it.sq = ctrl->seq_sq[b];
    it.k0 = ctrl->seq_k0[b];
    it.sk = ctrl->seq_sk[b];
    it.kh = kh;
    it.h[0] = kh * p.group;  // first q head of the group
    it.h[1] = piece;         // split slot of the result
    it.row0[0] = rb * BM;    // first packed row (token * group + group head)
    it.row0[1] = 0x3fffffff; // tile 1 does not exist
    it.shift = (p.causal == 2) ? it.sk - it.sq : 0;
    const int lo = rnd == 0 ? ctrl->split_first_lo : 0;
    const int hi = rnd == ctrl->split_items - 1 ? ctrl->split_last_hi : split_stream_tiles(p, it.sq, it.sk, rb);
    it.n0 = lo;
    it.nt[0] = hi - lo;
    it.nt[1] = 0;
    it.N = it.nt[0];
}

__device__ __forceinline__ uint32_t find_item(const Ctrl* ctrl, const Sm100Dev& p, int w, int lane) {
    int lo = 0, hi = ctrl->num_levels;  // last level whose start is <= w
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (ctrl->level_start[mid] <= w) lo = mid; else hi = mid;
    }
    const int blk = ctrl->num_levels - 1 - lo;
    const int per_seq = p.pair_heads ? p.hq / 2 : p.hq;  // items per (sequence, row block)
    const int j = w - ctrl->level_start[lo];
    int bj = j / per_seq;
    const int hj = j - bj * per_seq;
    int b = 0;
    for (int base = 0; base < p.batch; base += 32) {  // the bj-th sequence that has a block `blk`
        const bool has = (base + lane < p.batch) && ctrl->nblk[base + lane] > blk;
        const uint32_t m = __ballot_sync(0xffffffffu, has);
        const int c = __popc(m);
        if (bj < c) {
            b = base + __fns(m, 0, bj + 1);
            break;
        }
        bj -= c;
    }
    return 0x80000000u | ((uint32_t)b << 22) | ((uint32_t)hj << 12) | (uint32_t)blk;
}

// The fields of a work item from its packed form: a few shared-memory reads and integer operations.
__device__ __forceinline__ void expand_item(const Ctrl* ctrl, const Sm100Dev& p, uint32_t packed, Item& it) {
    it.valid = packed >> 31;
    const int b = (packed >> 22) & 0x1ff, hj = (packed >> 12) & 0x3ff, blk = packed & 0xfff;
    it.b = b;
    it.q0 = ctrl->seq_q0[b];
    it.sq = ctrl->seq_sq[b];
    it.k0 = ctrl->seq_k0[b];
    it.sk = ctrl->seq_sk[b];
    if (p.pair_heads) {
        it.h[0] = 2 * hj;
        it.h[1] = 2 * hj + 1;
        it.row0[0] = it.row0[1] = blk * BM;
    } else {
        it.h[0] = it.h[1] = hj;
        it.row0[0] = blk * 2 * BM;
        it.row0[1] = blk * 2 * BM + BM;
    }
    it.kh = it.h[0] / (p.hq / p.hkv);
    // key tiles each Q tile needs: from the first key its first row sees to the last key its last row sees.  The two
    // tiles of an item walk the same tiles n0 .. n0+N-1, n0 being tile 0's first: with paired heads their ranges are
    // equal; without them (two row blocks of one head) a left window lets tile 1 start one key tile later, and it
    // walks that tile with every key masked instead (P = 0, running max untouched).
    it.shift = (p.causal == 2) ? it.sk - it.sq : 0;
    it.n0 = 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int first = it.row0[i];
        int n = 0;
        if (first < it.sq) {
            int lo_key = 0, hi_key = it.sk - 1;
            if (p.causal) {
                if (p.wl >= 0) lo_key = max(0, first + it.shift - p.wl);
                if (p.wr >= 0) hi_key = min(hi_key, min(it.sq, first + BM) - 1 + it.shift + p.wr);
            }
            if (hi_key >= lo_key) {
                if (i == 0) it.n0 = lo_key / BN;
                n = hi_key / BN - it.n0 + 1;
            }
        }
        it.nt[i] = n;
    }
    if (it.nt[0] == 0) it.n0 = 0;
    it.N = max(it.nt[0], it.nt[1]);
}

// The work item of round `rnd` of this CTA, from the table filled at start-up.
template <int SPLIT = 0>
__device__ __forceinline__ void get_item(const Ctrl* ctrl, const Sm100Dev& p, int rnd, int total_items, int lane, Item& it) {
    if (SPLIT) expand_item_split(ctrl, p, ctrl->items[rnd], rnd, it);
    else expand_item(ctrl, p, ctrl->items[rnd], it);
}

// VAR bit 1 (EXTRA): the scaled scores get the reference's score additions that need no memory traffic -- a logits soft
//          cap (cap * tanh(score / cap), core/profiling/attention/fmha_fwd/fmha_fwd_problem.h:81) and ALiBi
//          (-slope * |i + sk - sq - j|, BiasEnum::ALIBI, fmha_library.h:124) -- applied to the score registers before
//          the mask.
// VAR bit 2 (BIAS): an elementwise bias tensor (BiasEnum::ELEMENTWISE_BIAS) is added to the scaled (and capped) scores.
//          Each softmax thread fetches the 128 bias values of its row and key tile (256 contiguous bytes, sixteen
//          16-byte loads; element loads for unaligned rows and the tail tile) before it waits for S, then reads S 32
//          columns at a time and adds the bias words as it arrives, so that scores and bias are never live in full
//          together.  (Fetching through the warp -- four lanes per row, the block handed on through shared memory --
//          measured the same; fetching a step ahead spilled and lost.)  Implies the score arithmetic of EXTRA.
// VAR bit 0 (WINDOW): the mask has a left window or a right window other than 0 (everything but no mask / causal); a separate
// instance, so that the common masks do not carry the second bound of the visible range through the softmax loop.
// SPLIT 1: the split-KV form described at Sm100Dev (one Q tile per item; work cut as described at kItemCostDefault).  The S
//          columns of tile 1 are a second S buffer, its Q room a third K slot; K, V and Q have a producer warp each
//          (9, 10, 11); warp 8 issues the QK^T, the first thread of warp 4 the PV products, warps 5-7 write LSE = -inf
//          to the splits no work item fills.
// SPLIT 2: the same for at most 64 packed rows: the rows are loaded twice (tile rows 0-63 and 64-127); the copy in rows
//          0-63 takes keys 0-63 of every 128-key tile, the copy in rows 64-127 takes keys 64-127, each as a split of its
//          own (2 * piece, 2 * piece + 1).  Every softmax thread then handles 64 columns instead of 128 with half of the
//          threads idle, which halves the softmax part of the per-tile chain.
// EXPM: how the softmax takes its exponentials.  0: one fp32 exp2 per element on the exp2 unit; 1: two per issue
//       through the unit's packed f16x2 form (see pack_f16x2); 11, 12, 13: fp32, with 1, 2 or 3 of every 8 column pairs
//       on a polynomial on the FMA pipe instead.
#ifndef FCK_P_HALVES
#define FCK_P_HALVES 1
#endif
template <typename T, int EXPM, int VAR, int SPLIT, int HDIM = 128>
__global__ void __launch_bounds__(NTHREADS, 1)
fmha_fwd_sm100_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                      const Sm100Dev p) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // head dim of this instance (128, or 64 for the prefill forms): the names below shadow the file-scope constants
    // RB: bytes of one row of Q, K or V; HB: its 128-byte blocks; XB: elements per block (the TMA x step); KK: keys
    // (PV) or head-dim elements (QK^T) one MMA instruction contracts: 32 bytes of a row either way
    constexpr bool F8 = ElemInfo<T>::f8;
    constexpr int ES = ElemInfo<T>::bytes;
    constexpr int HD = HDIM, RB = HD * ES, TILE_BYTES = BM * RB, HB = RB / 128, XB = 128 / ES, KK = 32 / ES;
    static_assert(HDIM == 128 || (HDIM == 64 && SPLIT == 0), "hdim 64 is built for the prefill forms only");
    static_assert(!F8 || (HDIM == 128 && SPLIT == 0 && (VAR & 6) == 0 && EXPM == 0),
                  "the 8-bit instances: hdim 128, prefill forms, fp32 exponentials, no score additions");
    constexpr bool WINDOW = (VAR & 1) != 0;  // the mask has a second bound (see above)
    constexpr bool BIAS = (VAR & 4) != 0;    // an elementwise bias tensor on the scaled scores
    constexpr bool EXTRA = (VAR & 2) != 0 || BIAS;   // ALiBi and / or a logits soft cap on the scaled scores
    static_assert(!BIAS || (SPLIT == 0 && EXPM == 0 && !F8), "the bias instances are prefill forms with fp32 exponentials");
    constexpr int NPOLY8 = EXPM >= 11 ? EXPM - 10 : 0;
    constexpr bool HEXP = EXPM == 1;
    constexpr bool HALVES = FCK_P_HALVES != 0 && SPLIT == 0;  // P reaches the PV in two halves of 64 keys

    // ---- shared memory carve-up ----
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t* base = smem_raw + (((raw + 1023u) & ~1023u) - raw);
    uint8_t* sQ = base;                                  // 2 tiles
    // The split modes have one Q tile; the room of the second one is a third K slot: with a single tile per item
    // the step is short, and two K tiles ahead keep the loads in flight that the HBM rate needs.
    constexpr int KS = SPLIT ? 3 : 2;
    uint8_t* sK = base + (SPLIT ? 1 : 2) * TILE_BYTES;   // KS tiles
    uint8_t* sV = sK + KS * TILE_BYTES;                  // KV_SLOTS tiles
    uint8_t* sStage = sV + KV_SLOTS * TILE_BYTES;        // 8 x STAGE_BYTES: O chunks of the softmax warps
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(sStage + 8 * STAGE_BYTES);
    volatile int* abort_flag = &ctrl->abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(&ctrl->q_full, 1);
        mbar_init(&ctrl->q_empty, 1);
        mbar_init(&ctrl->v_tail, 1);
        for (int s = 0; s < 3; ++s) {
            mbar_init(&ctrl->k_full[s], 1);
            mbar_init(&ctrl->k_empty[s], 1);
        }
        for (int s = 0; s < KV_SLOTS; ++s) {
            mbar_init(&ctrl->v_full[s], 1);
            mbar_init(&ctrl->v_empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&ctrl->s_full[i], 1);
            mbar_init(&ctrl->p_full[i], 4);  // one arrival per softmax warp
            mbar_init(&ctrl->p_full2[i], 4);
            mbar_init(&ctrl->o_full[i], 1);
            mbar_init(&ctrl->pv_done[i], 1);
        }
        ctrl->abort_flag = 0;
        ctrl->num_levels = p.num_levels;
        mbar_fence_init();
    }
    if (warp == 8) {  // TMEM: all 512 columns (S0 S1 O0 O1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(
            smem_u32(&ctrl->tmem_base)));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    if (p.page > 0) {  // paged: slots start as zeros (rows that are never loaded stay finite)
        for (int idx = threadIdx.x; idx < (KS + KV_SLOTS) * TILE_BYTES / 16; idx += NTHREADS)
            reinterpret_cast<uint4*>(sK)[idx] = make_uint4(0u, 0u, 0u, 0u);
        fence_proxy_async_smem();
    }
    // Barriers, tensor memory and the cleared slots are this CTA's own; everything below reads global memory, which the
    // kernel before this one in the stream (an append, the previous step's merge) may still have been writing.
    pdl_launch_dependents();
    pdl_wait();
    // ---- schedule: blocks per sequence, then the first work item of every level ----
    for (int b = threadIdx.x; b < p.batch; b += NTHREADS) {
        const int64_t q0 = p.seqstart_q ? p.seqstart_q[b] : (int64_t)b * p.seqlen_q;
        const int sq = p.seqstart_q ? (int)(p.seqstart_q[b + 1] - q0) : p.seqlen_q;
        int64_t k0;
        int sk;
        if (p.page > 0) {  // k0 = where the sequence's page ids start in page_ids
            if (p.kv_indptr) {
                const int pb = p.kv_indptr[b], pe = p.kv_indptr[b + 1];
                k0 = pb;
                sk = pe > pb ? (pe - pb - 1) * p.page + p.kv_last_page_len[b] : 0;
            } else {
                // block table row, or (no page list) the first token row of a contiguous cache [rows, seqlen_k, hkv, d]
                k0 = (p.cache_batch_idx ? p.cache_batch_idx[b] : (int64_t)b) * (p.page_ids ? p.bt_stride : p.seqlen_k);
                sk = p.seqlen_k32 ? p.seqlen_k32[b] : p.seqlen_k;
            }
        } else {
            k0 = p.seqstart_k ? p.seqstart_k[b] : (int64_t)b * p.seqlen_k;
            sk = p.seqstart_k ? (int)(p.seqstart_k[b + 1] - k0) : p.seqlen_k;
        }
        ctrl->seq_q0[b] = (int)q0;  // row indices fit 31 bits (checked on the host)
        ctrl->seq_sq[b] = sq;
        ctrl->seq_k0[b] = (int)k0;
        ctrl->seq_sk[b] = sk;
        const int rows_per_block = p.pair_heads ? BM : 2 * BM;
        if (SPLIT) {  // units of the work line this sequence takes, and its longest stream
            const int rbc = (sq * p.group + BM - 1) / BM;
            int cost = 0, nmax = 0;
            for (int rb = 0; rb < rbc; ++rb) {
                const int n = split_stream_tiles(p, sq, sk, rb);
                cost += n + p.item_cost;
                nmax = max(nmax, n);
            }
            ctrl->nblk[b] = cost * p.hkv;
            ctrl->items[b] = (uint32_t)nmax;  // (scratch until the work list is written)
        }
        else ctrl->nblk[b] = min(p.num_levels, (sq + rows_per_block - 1) / rows_per_block);
    }
    __syncthreads();
    if (SPLIT) {
        constexpr int kDup = SPLIT == 2 ? 2 : 1;  // splits per piece
        const int max_pieces = max(1, p.num_splits / kDup);
        if (threadIdx.x == 0) {  // first unit of every sequence; length of a CTA's piece
            int run = 0, nmax = 0;
            for (int b = 0; b < p.batch; ++b) {
                ctrl->level_start[b] = run;
                run += ctrl->nblk[b];
                nmax = max(nmax, (int)ctrl->items[b]);
            }
            ctrl->level_start[p.batch] = run;
            int w = max((run + (int)gridDim.x - 1) / (int)gridDim.x, p.piece_tiles + p.item_cost);
            if (max_pieces >= 2) w = max(w, (nmax + max_pieces - 2) / (max_pieces - 1));  // ceil(n / w) + 1 <= max_pieces
            ctrl->split_w = w;
        }
        __syncthreads();
        const int w = ctrl->split_w;
        if (threadIdx.x == 0) {
            // this CTA's work list: the streams that reach into units [lo, hi) of the line
            const int lo = (int)blockIdx.x * w, hi = lo + w, total = ctrl->level_start[p.batch];
            int cnt = 0;
            bool overflow = false;
            if (lo < total) {
                int b = 0, bh = p.batch;  // last sequence that starts at or before lo
                while (bh - b > 1) {
                    const int mid = (b + bh) >> 1;
                    if (ctrl->level_start[mid] <= lo) b = mid; else bh = mid;
                }
                for (; b < p.batch && ctrl->level_start[b] < hi; ++b) {
                    const int sq = ctrl->seq_sq[b], sk = ctrl->seq_sk[b];
                    const int rbc = (sq * p.group + BM - 1) / BM;
                    int seg0 = ctrl->level_start[b];
                    for (int rb = 0; rb < rbc && seg0 < hi; ++rb) {
                        const int n = split_stream_tiles(p, sq, sk, rb), c = n + p.item_cost;
                        const int kh_lo = max(0, (lo - seg0) / c), kh_hi = min(p.hkv - 1, (hi - 1 - seg0) / c);
                        for (int kh = kh_lo; kh <= kh_hi; ++kh) {
                            const int g0 = seg0 + kh * c;
                            int t_lo = 0, t_hi = n, piece = 0;
                            if (n == 0 || max_pieces == 1) {
                                if (g0 < lo) continue;  // the whole stream belongs to the CTA its start falls to
                            } else {
                                t_lo = max(0, lo - g0 - p.item_cost);
                                t_hi = min(n, hi - g0 - p.item_cost);
                                if (t_hi <= t_lo) continue;
                                piece = (int)blockIdx.x - (g0 + p.item_cost) / w;
                            }
                            if (cnt >= kSplitItems) { overflow = true; break; }
                            ctrl->items[cnt] = 0x80000000u | ((uint32_t)b << 22) | ((uint32_t)kh << 12) | ((uint32_t)piece << 4) | (uint32_t)rb;
                            if (cnt == 0) ctrl->split_first_lo = t_lo;  // (only the first item can start inside its stream)
                            ctrl->split_last_hi = t_hi;                 // (and only the last one end inside it)
                            ++cnt;
                        }
                        seg0 += p.hkv * c;
                    }
                }
            }
            if (overflow) {  // the host checks an upper bound of this; never silently drop work
                atomicOr(p.status, FLASHCK_STATUS_WORKLIST_OVERFLOW);
                cnt = 0;
            }
            ctrl->split_items = cnt;
        }
    }
    for (int lv = threadIdx.x; !SPLIT && lv < p.num_levels; lv += NTHREADS) {  // count of sequences that have block index lv
        int c = 0;
        for (int b = 0; b < p.batch; ++b) c += ctrl->nblk[b] > lv;
        ctrl->level_start[p.num_levels - lv] = c * (p.pair_heads ? p.hq / 2 : p.hq);  // summed up below
    }
    __syncthreads();
    if (!SPLIT && threadIdx.x == 0) {
        int run = 0;
        ctrl->level_start[0] = 0;
        for (int lv = 1; lv <= p.num_levels; ++lv) {
            run += ctrl->level_start[lv];
            ctrl->level_start[lv] = run;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctrl->tmem_base;
    const int total_items = SPLIT ? 0 : ctrl->level_start[p.num_levels];
    int rounds = SPLIT ? ctrl->split_items : (total_items + (int)gridDim.x - 1) / (int)gridDim.x;
    if (!SPLIT && rounds > kMaxRounds) {  // the host checks an upper bound of this; never silently drop work
        if (threadIdx.x == 0) atomicOr(p.status, FLASHCK_STATUS_WORKLIST_OVERFLOW);
        rounds = 0;
    }
    for (int rnd = warp; !SPLIT && rnd < rounds; rnd += NTHREADS / 32) {  // this CTA's work list
        const int w = item_of_round(rnd, blockIdx.x, gridDim.x);
        const uint32_t packed = w >= total_items ? 0u : find_item(ctrl, p, w, lane);
        if (lane == 0) ctrl->items[rnd] = packed;
    }
    __syncthreads();

    if (warp >= 8) {
        // Register budget.  The CTA is launched with 384 x 168 = 64512 registers; setmaxnreg.dec returns registers
        // to the CTA's pool and setmaxnreg.inc waits -- without a bound -- until the pool can serve it, so the sum
        // after the moves must not exceed the launch allocation.  Prefill forms: 256 x 208 + 128 x 88 = 64512, the
        // whole pool -- at 80 registers the producer and the issuing thread spill ~90 bytes, which costs the kernel
        // 1-2 % (the issuing thread's time between MMAs is idle time of the tensor pipe); the softmax warps would need
        // 216 to be free of spills, which the pool does not hold.  Split modes: 256 x 208 + 128 x 80.
        if constexpr (SPLIT == 0) asm volatile("setmaxnreg.dec.sync.aligned.u32 88;\n" ::);
        else asm volatile("setmaxnreg.dec.sync.aligned.u32 80;\n" ::);
        // In the split modes a step is short and the copies are many small boxes whose issue takes a warp a good part
        // of it, so K, V and Q have a producer warp each (9, 10, 11): the K producer then runs ahead into the next item
        // (its first page-id lookup is a round trip to memory) instead of waiting for the Q buffer, which frees late.
        // Prefill steps are long: warp 9 does it all there (measured: extra producer warps cost paged prefill 7 %).
        const bool k_role = warp == 9, v_role = SPLIT ? warp == 10 : warp == 9, q_role = SPLIT ? warp == 11 : warp == 9;
        if (k_role || v_role || q_role) {
            // ================================ TMA producers ================================
            if (lane == 0) {
                tma_prefetch_desc(&map_q);
                tma_prefetch_desc(&map_k);
                tma_prefetch_desc(&map_v);
            }
            uint32_t kv_cnt = 0, q_cnt = 0;  // K/V tiles and Q loads issued so far (ring positions)
            uint32_t tail_cnt = 0;           // tiles that went through v_tail (its parity)
            // Paged pools are read in chunks of min(page, 128) tokens: one TMA box per chunk and 64-column half.
            // A chunk that the sequence only partly fills is the tail of its last page, and what lies behind the
            // sequence end there is whatever the allocator left: for K that is harmless (those scores are masked by
            // index), but P = 0 times a NaN in V is NaN, so the V rows behind the sequence end are overwritten with zeros
            // when such a chunk has landed (a copy of those rows by hand, one 16-byte load after the other, cost up to
            // 16 us per sequence end with pages of 128 tokens).  Chunks wholly behind the end are not loaded at all; the
            // slot then keeps rows of earlier tiles (real data, or the zeros the slots start with).
            const int chunk = p.page > 0 ? min(p.page, BN) : BN;
            const int chunks = BN / chunk;
            for (int rnd = 0; rnd < rounds; ++rnd) {
                Item it;
                get_item<SPLIT>(ctrl, p, rnd, total_items, lane, it);
                if (!it.valid || it.N == 0) continue;
                bool ok = true;
                if (lane == 0 && q_role) {
                    ok = mbar_wait_bounded(&ctrl->q_empty, (q_cnt & 1u) ^ 1u, abort_flag, p.status, 0x08);
                    if (ok && SPLIT) {
                        // one box of (64 columns, group heads, 128/group tokens) per half: the rows land in
                        // (token, group head) order
                        mbar_expect_tx(&ctrl->q_full, TILE_BYTES);
                        for (int hb = 0; hb < HB; ++hb) {
                            if (SPLIT == 2) {  // the box holds 64 rows: once for tile rows 0-63, once for 64-127
                                tma_load_4d(sQ + hb * HALF_BYTES, &map_q, &ctrl->q_full, hb * XB, 0, it.kh, it.q0);
                                tma_load_4d(sQ + hb * HALF_BYTES + 64 * 128, &map_q, &ctrl->q_full, hb * XB, 0, it.kh, it.q0);
                            } else {
                                tma_load_4d(sQ + hb * HALF_BYTES, &map_q, &ctrl->q_full, hb * XB, 0, it.kh, it.q0 + it.row0[0] / p.group);
                            }
                        }
                    } else if (ok) {
                        const int q_tiles = (it.row0[1] < it.sq) ? 2 : 1;
                        mbar_expect_tx(&ctrl->q_full, q_tiles * TILE_BYTES);
                        for (int hb = 0; hb < HB; ++hb)
                            tma_load_3d(sQ + hb * HALF_BYTES, &map_q, &ctrl->q_full, hb * XB, it.h[0], it.q0 + it.row0[0]);
                        if (q_tiles == 2)
                            for (int hb = 0; hb < HB; ++hb)
                                tma_load_3d(sQ + TILE_BYTES + hb * HALF_BYTES, &map_q, &ctrl->q_full, hb * XB, it.h[1],
                                            it.q0 + it.row0[1]);
                    }
                    if (p.page == 0) {  // contiguous K/V: one box per tile and 64-column half
                        for (int n = 0; ok && n < it.N; ++n) {
                            const uint32_t kc = kv_cnt + n;
                            const int s = kc % KV_SLOTS, sk_ = kc % KS;
                            const uint32_t ph = (kc / KV_SLOTS) & 1u, phk = (kc / KS) & 1u;
                            const int row = it.k0 + (it.n0 + n) * BN;
                            if (!(ok = mbar_wait_bounded(&ctrl->k_empty[sk_], phk ^ 1u, abort_flag, p.status, 0x10))) break;
                            mbar_expect_tx(&ctrl->k_full[sk_], TILE_BYTES);
                            for (int hb = 0; hb < HB; ++hb)
                                tma_load_3d(sK + sk_ * TILE_BYTES + hb * HALF_BYTES, &map_k, &ctrl->k_full[sk_], hb * XB, it.kh, row);
                            if (!(ok = mbar_wait_bounded(&ctrl->v_empty[s], ph ^ 1u, abort_flag, p.status, 0x20))) break;
                            mbar_expect_tx(&ctrl->v_full[s], TILE_BYTES);
                            for (int hb = 0; hb < HB; ++hb)
                                tma_load_3d(sV + s * TILE_BYTES + hb * HALF_BYTES, &map_v, &ctrl->v_full[s], hb * XB, it.kh, row);
                        }
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (p.page == 0) kv_cnt += it.N;
                // ---- paged: lane c owns chunk c of the tile: the pool row of its first token and the tokens it holds.
                // Each lane issues the copies of its own chunk (one warp instruction starts up to 8 of them), and the
                // page ids of the next tile are fetched while this tile's slots are awaited.
                auto lookup = [&](int n, int& row, int& valid) {
                    row = 0;
                    valid = 0;
                    if (lane < chunks && n < it.N) {
                        const int key0 = (it.n0 + n) * BN + lane * chunk;
                        valid = max(0, min(chunk, it.sk - key0));
                        if (valid > 0)  // no page list: a contiguous cache read in 128-token chunks
                            row = p.page_ids ? p.page_ids[it.k0 + key0 / p.page] * p.page + key0 % p.page : it.k0 + key0;
                    }
                };
                int my_row = 0, my_valid = 0;
                const bool kv_paged = p.page > 0 && (k_role || v_role);
                if (kv_paged) lookup(0, my_row, my_valid);
                for (int n = 0; kv_paged && ok && n < it.N; ++n, ++kv_cnt) {
                    const int s = kv_cnt % KV_SLOTS, sk_ = kv_cnt % KS;
                    const uint32_t ph = (kv_cnt / KV_SLOTS) & 1u, phk = (kv_cnt / KS) & 1u;
                    int next_row, next_valid;
                    lookup(n + 1, next_row, next_valid);
                    const uint32_t any_mask = __ballot_sync(0xffffffffu, my_valid > 0);
                    const uint32_t full_mask = __ballot_sync(0xffffffffu, my_valid == chunk);
                    if (lane == 0 && k_role) {
                        ok = mbar_wait_bounded(&ctrl->k_empty[sk_], phk ^ 1u, abort_flag, p.status, 0x10);
                        if (ok) mbar_expect_tx(&ctrl->k_full[sk_], __popc(any_mask) * chunk * HD * 2);
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    if (k_role && my_valid > 0)
                        for (int hb = 0; hb < HB; ++hb)
                            tma_load_3d(sK + sk_ * TILE_BYTES + hb * HALF_BYTES + lane * chunk * 128, &map_k, &ctrl->k_full[sk_],
                                        hb * XB, it.kh, my_row);
                    if (!v_role) {
                        my_row = next_row;
                        my_valid = next_valid;
                        continue;
                    }
                    if (lane == 0) ok = mbar_wait_bounded(&ctrl->v_empty[s], ph ^ 1u, abort_flag, p.status, 0x20);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    const uint32_t part_mask = any_mask & ~full_mask;  // at most one chunk: the tail of the last page
                    if (part_mask) {
                        // The tile holds the end of the sequence.  Its copies complete on a barrier of their own; when
                        // they have landed the rows behind the end are overwritten with zeros (shared-memory stores
                        // only), and only then is the slot handed to the MMA thread.
                        if (lane == 0) mbar_expect_tx(&ctrl->v_tail, __popc(any_mask) * chunk * HD * 2);
                        __syncwarp();
                        if (my_valid > 0)
                            for (int hb = 0; hb < HB; ++hb)
                                tma_load_3d(sV + s * TILE_BYTES + hb * HALF_BYTES + lane * chunk * 128, &map_v, &ctrl->v_tail,
                                            hb * XB, it.kh, my_row);
                        if (lane == 0) ok = mbar_wait_bounded(&ctrl->v_tail, tail_cnt & 1u, abort_flag, p.status, 0x21);
                        ++tail_cnt;
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                        if (!ok) break;
                        const int c = __ffs(part_mask) - 1;
                        const int v = __shfl_sync(0xffffffffu, my_valid, c);
                        uint8_t* dst = sV + s * TILE_BYTES + c * chunk * 128;
                        for (int idx = lane; idx < (chunk - v) * (HD / 8); idx += 32) {  // a row is 128 bytes in every 64-column block
                            const int r = v + idx / (HD / 8), piece = idx % (HD / 8);
                            *reinterpret_cast<uint4*>(dst + (piece >> 3) * HALF_BYTES + r * 128 + ((piece & 7) << 4)) =
                                make_uint4(0u, 0u, 0u, 0u);
                        }
                        fence_proxy_async_smem();  // the MMAs read these rows through the async proxy
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&ctrl->v_full[s]);
                    } else {
                        if (lane == 0) mbar_expect_tx(&ctrl->v_full[s], __popc(full_mask) * chunk * HD * 2);
                        __syncwarp();
                        if (my_valid == chunk)
                            for (int hb = 0; hb < HB; ++hb)
                                tma_load_3d(sV + s * TILE_BYTES + hb * HALF_BYTES + lane * chunk * 128, &map_v, &ctrl->v_full[s],
                                            hb * XB, it.kh, my_row);
                    }
                    my_row = next_row;
                    my_valid = next_valid;
                }
                ++q_cnt;
                if (!ok) break;
            }
        } else if (warp == 8) {
            // ================================ MMA issuer ================================
            constexpr uint32_t idesc_qk = make_idesc<T>(false);
            constexpr uint32_t idesc_pv = make_idesc<T>(true, HD);  // N = head dim of V
            const uint32_t tS[2] = {tmem, tmem + 128};
            const uint32_t tO[2] = {tmem + 256, tmem + 384};
            // Descriptors are built once; per MMA only the 14-bit start-address field (16-byte units) advances,
            // by compile-time offsets, so the issuing thread spends a few integer adds per instruction.
            const uint64_t dQ0 = make_smem_desc(smem_u32(sQ), 0, 1024);
            const uint64_t dQ1 = make_smem_desc(smem_u32(sQ + TILE_BYTES), 0, 1024);
            const uint64_t dK0 = make_smem_desc(smem_u32(sK), 0, 1024);
            const uint64_t dV0 = make_smem_desc(smem_u32(sV), HALF_BYTES, 1024);
            const uint64_t dV1 = make_smem_desc(smem_u32(sV + TILE_BYTES), HALF_BYTES, 1024);
            const bool leader = elect_one_sync();
            // A wait of the convergent issuing warp: every lane probes, all leave together with one outcome.  Without the
            // vote a lane could fall two phases of a barrier behind the elected one and then read the parity of a
            // later phase as "not complete yet".
            auto wait_all = [&](uint64_t* bar, uint32_t parity, volatile int* af, int* st, int code) {
                return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity, af, st, code)) != 0;
            };
            auto commit = [&](uint64_t* bar) { if (leader) umma_commit(bar); };
            auto issue_qk = [&](int i, int s) {  // S_i = Q_i K^T : 8 steps of 16 along the head dim
                const uint64_t qd = i ? dQ1 : dQ0, kd = dK0 + (uint64_t)((s * TILE_BYTES) >> 4);
                const uint32_t d = tS[i];
                if (leader) {
#pragma unroll
                    for (int ks = 0; ks < RB / 32; ++ks) {
                        const uint64_t off = (uint64_t)(((ks / 4) * HALF_BYTES + (ks % 4) * 32) >> 4);
                        umma_ss<F8>(d, qd + off, kd + off, idesc_qk, ks > 0 ? 1u : 0u);
                    }
                }
            };
            // O_i += P_i V : 8 steps of 16 keys; `part` 0 / 1 = the steps of keys 0-63 / 64-127, 2 = all of them
            auto issue_pv = [&](int i, int s, bool accumulate, int part = 2) {
                const uint64_t vd = s ? dV1 : dV0;
                const uint32_t d = tO[i], a = tS[i];
                constexpr int STEPS = BN / KK;
                if (leader) {
                    if (part != 1) {
#pragma unroll
                        for (int ks = 0; ks < STEPS / 2; ++ks)  // KK keys = KK rows of 128 bytes of the V tile, 8 columns of P
                            umma_ts<F8>(d, a + ks * 8, vd + (uint64_t)((ks * KK * 128) >> 4), idesc_pv, (accumulate || ks > 0) ? 1u : 0u);
                    }
                    if (part != 0) {
#pragma unroll
                        for (int ks = STEPS / 2; ks < STEPS; ++ks)
                            umma_ts<F8>(d, a + ks * 8, vd + (uint64_t)((ks * KK * 128) >> 4), idesc_pv, 1u);
                    }
                }
            };
            // split modes: tile 0's Q against S buffer `buf` (the S columns of either tile), P read from the same buffer
            auto issue_qk_to = [&](uint32_t buf, int s) {
                const uint64_t kd = dK0 + (uint64_t)((s * TILE_BYTES) >> 4);
                if (leader) {
#pragma unroll
                    for (int ks = 0; ks < RB / 32; ++ks) {
                        const uint64_t off = (uint64_t)(((ks / 4) * HALF_BYTES + (ks % 4) * 32) >> 4);
                        umma_ss<F8>(tS[0] + buf * 128, dQ0 + off, kd + off, idesc_qk, ks > 0 ? 1u : 0u);
                    }
                }
            };
            // running counts give ring slots and barrier parities across work items
            uint32_t kv_cnt = 0, q_cnt = 0, sc0 = 0, sc1 = 0;
            if (SPLIT) {
                // Split modes: this warp issues only the QK^T (all lanes walk the loop, the elected one issues), warp 4 the PV (the warps of tile 1's
                // softmax warpgroup have nothing else to do there).  Each polls its own barriers while the other's
                // block of MMAs runs, which a single issuer could not do (the tensor pipe takes instructions only about
                // one ahead).  The two S buffers are handed back by pv_done: S of step g goes into buffer g & 1 once
                // the PV of step g - 2, which read P from it, is complete.
                for (int rnd = 0; rnd < rounds; ++rnd) {
                    Item it;
                    get_item<SPLIT>(ctrl, p, rnd, total_items, lane, it);
                    if (!it.valid || it.N == 0) continue;
                    const int N = it.N;
                    bool ok = wait_all(&ctrl->q_full, q_cnt & 1u, abort_flag, p.status, 0x40);
                    for (int n = 0; ok && n < N; ++n) {
                        const uint32_t kc = kv_cnt + n, g = sc0 + n, b = g & 1u;
                        const int s = kc % KS;
                        if (!(ok = wait_all(&ctrl->k_full[s], (kc / KS) & 1u, abort_flag, p.status, 0x41))) break;
                        if (g >= 2 && !(ok = wait_all(&ctrl->pv_done[b], ((g >> 1) + 1u) & 1u, abort_flag, p.status, 0x44))) break;
                        tc_fence_after();
                        issue_qk_to(b, s);
                        commit(&ctrl->s_full[b]);
                        commit(&ctrl->k_empty[s]);
                        if (n + 1 == N) commit(&ctrl->q_empty);  // Q may be replaced once these MMAs are done
                    }
                    if (!ok) break;
                    kv_cnt += N;
                    sc0 += N;
                    ++q_cnt;
                }
            } else if (!SPLIT) {
                // All 32 lanes walk the loop and poll the barriers together; one elected lane issues the MMAs and the
                // commits.  The control flow, the counters and the descriptors are then the same in every lane, which
                // lets them live in the warp's uniform registers instead of one thread's vector registers (an item with
                // N == 0 is skipped by every role).
                int N = 0, N0 = 0, N1 = 0;
                if (rounds > 0) {
                    Item it;
                    get_item<SPLIT>(ctrl, p, 0, total_items, lane, it);
                    if (it.valid) { N = it.N; N0 = it.nt[0]; N1 = it.nt[1]; }
                }
                for (int rnd = 0; rnd < rounds; ++rnd) {
                    bool ok = true;
                    int nN = 0, nN0 = 0, nN1 = 0;
                    if (N > 0) {
                        const int s0 = kv_cnt % KS;
                        ok = wait_all(&ctrl->q_full, q_cnt & 1u, abort_flag, p.status, 0x40) &&
                             wait_all(&ctrl->k_full[s0], (kv_cnt / KS) & 1u, abort_flag, p.status, 0x41);
                        if (ok) {
                            tc_fence_after();
                            if (N0 > 0) { issue_qk(0, s0); commit(&ctrl->s_full[0]); }
                            if (N1 > 0) { issue_qk(1, s0); commit(&ctrl->s_full[1]); }
                            commit(&ctrl->k_empty[s0]);
                            if (N == 1) commit(&ctrl->q_empty);  // Q may be replaced once these MMAs are done
                        }
                        // the step counts of the next item, worked out while the first softmax of this one runs
                        if (rnd + 1 < rounds) {
                            Item nx;
                            get_item<SPLIT>(ctrl, p, rnd + 1, total_items, lane, nx);
                            if (nx.valid) { nN = nx.N; nN0 = nx.nt[0]; nN1 = nx.nt[1]; }
                        }
                        for (int n = 0; ok && n < N; ++n) {
                            const uint32_t kc = kv_cnt + n;
                            const int s = kc % KV_SLOTS, s1 = (kc + 1) % KS;           // V slot of this step, K slot of the next
                            const uint32_t ph = (kc / KV_SLOTS) & 1u, ph1 = ((kc + 1) / KS) & 1u;
                            // V of this step and K of the next have been on their way for more than a step: both
                            // barriers are looked at here, under the wait for P that follows, because even a passing
                            // probe costs the issuing thread ~100 clocks -- between PV0 and QK0 those would be idle
                            // clocks of the tensor pipe
                            if (!(ok = wait_all(&ctrl->v_full[s], ph, abort_flag, p.status, 0x42))) break;
                            if (n + 1 < N) {
                                if (!(ok = wait_all(&ctrl->k_full[s1], ph1, abort_flag, p.status, 0x44))) break;
                            }
                            if (n < N0) {
                                if constexpr (HALVES) {
                                    if (!(ok = wait_all(&ctrl->p_full[0], (sc0 + n) & 1u, abort_flag, p.status, 0x43))) break;
                                    tc_fence_after();
                                    issue_pv(0, s, n > 0, 0);
                                    if (!(ok = wait_all(&ctrl->p_full2[0], (sc0 + n) & 1u, abort_flag, p.status, 0x43))) break;
                                    tc_fence_after();
                                    issue_pv(0, s, true, 1);
                                } else {
                                    if (!(ok = wait_all(&ctrl->p_full[0], (sc0 + n) & 1u, abort_flag, p.status, 0x43))) break;
                                    tc_fence_after();
                                    issue_pv(0, s, n > 0);
                                }
                                if (n == N0 - 1) commit(&ctrl->o_full[0]);
                            } else {
                                tc_fence_after();
                            }
                            if (n + 1 < N0) { issue_qk(0, s1); commit(&ctrl->s_full[0]); }
                            if (n < N1) {
                                if constexpr (HALVES) {
                                    if (!(ok = wait_all(&ctrl->p_full[1], (sc1 + n) & 1u, abort_flag, p.status, 0x45))) break;
                                    tc_fence_after();
                                    issue_pv(1, s, n > 0, 0);
                                    if (!(ok = wait_all(&ctrl->p_full2[1], (sc1 + n) & 1u, abort_flag, p.status, 0x45))) break;
                                    tc_fence_after();
                                    issue_pv(1, s, true, 1);
                                } else {
                                    if (!(ok = wait_all(&ctrl->p_full[1], (sc1 + n) & 1u, abort_flag, p.status, 0x45))) break;
                                    tc_fence_after();
                                    issue_pv(1, s, n > 0);
                                }
                                if (n == N1 - 1) commit(&ctrl->o_full[1]);
                            }
                            commit(&ctrl->v_empty[s]);
                            if (n + 1 < N1) { issue_qk(1, s1); commit(&ctrl->s_full[1]); }
                            if (n + 1 < N) commit(&ctrl->k_empty[s1]);
                            if (n + 2 == N) commit(&ctrl->q_empty);  // the last QK^T of the item has been issued
                        }
                        kv_cnt += N;
                        sc0 += N0;
                        sc1 += N1;
                        ++q_cnt;
                    } else if (rnd + 1 < rounds) {
                        Item nx;
                        get_item<SPLIT>(ctrl, p, rnd + 1, total_items, lane, nx);
                        if (nx.valid) { nN = nx.N; nN0 = nx.nt[0]; nN1 = nx.nt[1]; }
                    }
                    if (!ok) break;
                    N = nN; N0 = nN0; N1 = nN1;
                }
            }
        }
    } else {
        // ================================ softmax warpgroups ================================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;\n" ::);
        const int i = warp >> 2;                 // Q tile of this warpgroup
        const int r = (warp & 3) * 32 + lane;    // row inside the tile == TMEM lane
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t tS = lane_addr + i * 128, tO = lane_addr + 256 + i * 128;
        uint32_t sc = 0, oc = 0;  // S tiles and O accumulators consumed so far (barrier parities)
        bool ok = true;
        if (SPLIT && i == 1) {
            // Split modes have no second Q tile; the first thread of this warpgroup issues the PV products instead
            // (the QK^T come from warp 8): O += P V from S/P buffer g & 1 once V has landed and the softmax has
            // handed P over, then pv_done tells the softmax (which may rescale O) and the QK^T issuer (which may
            // overwrite the buffer) that this product is complete.
            if (warp == 4) {  // (all lanes walk the loop, the elected one issues)
                const bool lead4 = elect_one_sync();
                constexpr uint32_t idesc_pv = make_idesc<T>(true);
                const uint64_t dV0 = make_smem_desc(smem_u32(sV), HALF_BYTES, 1024);
                const uint64_t dV1 = make_smem_desc(smem_u32(sV + TILE_BYTES), HALF_BYTES, 1024);
                uint32_t kv_cnt = 0, g = 0;
                for (int rnd = 0; ok && rnd < rounds; ++rnd) {
                    Item it;
                    get_item<SPLIT>(ctrl, p, rnd, total_items, lane, it);
                    if (!it.valid || it.N == 0) continue;
                    const int N = it.N;
                    for (int n = 0; n < N; ++n, ++g) {
                        const uint32_t kc = kv_cnt + n, b = g & 1u;
                        const int s = kc % KV_SLOTS;
                        if (!(ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctrl->v_full[s], (kc / KV_SLOTS) & 1u, abort_flag, p.status, 0x42)))) break;
                        if (!(ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctrl->p_full[b], (g >> 1) & 1u, abort_flag, p.status, 0x43)))) break;
                        tc_fence_after();
                        const uint64_t vd = s ? dV1 : dV0;
                        if (lead4) {
#pragma unroll
                            for (int ks = 0; ks < BN / 16; ++ks)
                                umma_ts(tmem + 256, tmem + b * 128 + ks * 8, vd + (uint64_t)((ks * 2048) >> 4), idesc_pv,
                                        (n > 0 || ks > 0) ? 1u : 0u);
                            umma_commit(&ctrl->pv_done[b]);
                            if (n + 1 == N) umma_commit(&ctrl->o_full[0]);
                            umma_commit(&ctrl->v_empty[s]);
                        }
                    }
                    kv_cnt += N;
                }
            }
            else if (warp > 4 && p.lse_acc) {
                // (warps 5-7, while the others work) splits a stream does not use: LSE = -inf, so that the merge gives
                // them no weight
                constexpr int kDup = SPLIT == 2 ? 2 : 1;
                const int max_pieces = max(1, p.num_splits / kDup), w = ctrl->split_w;
                for (int b = blockIdx.x; b < p.batch; b += gridDim.x) {
                    const int sq = ctrl->seq_sq[b], sk = ctrl->seq_sk[b], q0 = ctrl->seq_q0[b];
                    const int rbc = (sq * p.group + BM - 1) / BM;
                    int seg0 = ctrl->level_start[b];
                    for (int rb = 0; rb < rbc; ++rb) {
                        const int n = split_stream_tiles(p, sq, sk, rb), c = n + p.item_cost;
                        const int rows = min(BM, sq * p.group - rb * BM);
                        for (int kh = 0; kh < p.hkv; ++kh) {
                            const int used = split_stream_pieces(seg0 + kh * c, n, w, max_pieces, p.item_cost) * kDup;
                            const int cnt = (p.num_splits - used) * rows;
                            for (int e = (int)threadIdx.x - 160; e < cnt; e += 96) {
                                const int sp = used + e / rows, pr = rb * BM + e % rows;
                                const int tok = pr / p.group, h = kh * p.group + (pr - tok * p.group);
                                const int64_t slot = p.seqstart_q ? ((int64_t)h * p.num_splits + sp) * p.total_q + q0 + tok
                                                                  : (((int64_t)b * p.hq + h) * p.num_splits + sp) * p.sq_cap + tok;
                                p.lse_acc[slot] = -INFINITY;
                            }
                        }
                        seg0 += p.hkv * c;
                    }
                }
            }
            ok = false;  // nothing else for this warpgroup
        }
        for (int rnd = 0; ok && rnd < rounds; ++rnd) {
            Item it;
            get_item<SPLIT>(ctrl, p, rnd, total_items, lane, it);
            if (!it.valid) continue;
            const int Ni = i ? it.nt[1] : it.nt[0];
            int head = i ? it.h[1] : it.h[0];
            const int sq = it.sq, sk = it.sk, shift = it.shift;
            // split mode packs (token, group head) into the rows; `row` is the query token either way
            const int packed_first = i ? it.row0[1] : it.row0[0];
            const int group = SPLIT ? p.group : 1;
            const int rr = SPLIT == 2 ? (r & 63) : r;   // packed row inside the tile
            const int khalf = SPLIT == 2 ? (r >> 6) : 0;  // which 64 keys of every tile this thread's copy of the row takes
            const int tile_first_row = SPLIT ? packed_first / group : packed_first;
            const int row = SPLIT ? (packed_first + rr) / group : packed_first + r;      // row inside the sequence
            const bool row_ok = row < sq;
            if (SPLIT) head += (packed_first + rr) - row * group;
            // visible keys of this row: [first_key, limit]
            const int wr = WINDOW ? p.wr : 0, wl = WINDOW ? p.wl : -1;
            const int limit = (p.causal && wr >= 0) ? min(sk - 1, row + shift + wr) : sk - 1;
            const int first_key = (WINDOW && p.causal && wl >= 0) ? row + shift - wl : 0;

            float m_used = -INFINITY;  // running max actually subtracted (scaled, base 2)
            float l = 0.f;
            float slope = 0.f;
            if constexpr (EXTRA) {
                if (p.alibi) slope = p.alibi[(p.alibi_rank ? (int64_t)it.b * p.hq : 0) + head];
            }
            [[maybe_unused]] const unsigned short* bias_row = nullptr;  // this row's bias values at key 0 of its sequence
            if constexpr (BIAS) {
                const int64_t plane = p.bias_sq * p.bias_sk;
                int64_t off = p.bias_el_rank >= 1 ? (int64_t)head * plane : 0;
                if (p.seqstart_q) off += (int64_t)(it.q0 + row) * p.bias_sk + it.k0;
                else off += (p.bias_el_rank == 2 ? (int64_t)it.b * p.hq * plane : 0) + (int64_t)row * p.bias_sk;
                if (row_ok) bias_row = reinterpret_cast<const unsigned short*>(p.bias_el) + off;
            }
            for (int n = 0; n < Ni; ++n) {
                // warp-uniform outcome: the loads, votes and stores below are warp-collective
                // The split modes have one Q tile and use the other tile's S columns as a second S buffer: the QK^T of
                // step n+1 is issued before the PV of step n, so the next S is there when P has been handed over.
                // Buffer and barrier index are the step's parity there, the Q tile otherwise.
                const uint32_t gstep = sc + n;
                const int sb = SPLIT ? (int)(gstep & 1u) : i;
                const uint32_t tSb = SPLIT ? lane_addr + sb * 128 : tS;
                const int key0 = (it.n0 + n) * BN + khalf * 64;
                [[maybe_unused]] const bool capped = EXTRA && p.soft_cap > 0.f;
                [[maybe_unused]] const float inv_cap = capped ? 1.f / p.soft_cap : 0.f;
                [[maybe_unused]] uint4 bw[BIAS ? 16 : 1];  // the 128 bias values of this thread's row and key tile
                if constexpr (BIAS) {  // (issued before the wait for S)
#pragma unroll
                    for (int v = 0; v < 16; ++v) bw[v] = load_bias_piece(bias_row, key0 + v * 8, sk - key0 - v * 8);
                }
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctrl->s_full[sb], (SPLIT ? (gstep >> 1) : gstep) & 1u, abort_flag,
                                                               p.status, 0x100 << i));
                if (!ok) break;
                tc_fence_after();
                constexpr int NC = SPLIT == 2 ? 64 : 128;  // columns of the row this thread handles
                uint32_t sreg[NC];
                if constexpr (BIAS) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        tmem_ld32(tSb + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sreg[c * 32]));
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const uint4 q4 = bw[c * 4 + (j >> 3)];
                            const uint32_t w = ((j >> 1) & 3) == 0 ? q4.x : ((j >> 1) & 3) == 1 ? q4.y : ((j >> 1) & 3) == 2 ? q4.z : q4.w;
                            const float bj = bias_elem<T>(w, j & 1), sj = __uint_as_float(sreg[c * 32 + j]);
                            float x;
                            if (capped) x = (p.soft_cap * tanh_inline(sj * p.scale * inv_cap) + bj) * kLog2e;
                            else x = fmaf(sj, p.scale_log2, bj * kLog2e);  // (the two products of the sum in base-2 units)
                            sreg[c * 32 + j] = __float_as_uint(x);
                        }
                    }
                } else {
#pragma unroll
                for (int c = 0; c < NC / 32; ++c)
                    tmem_ld32(tSb + khalf * 64 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sreg[c * 32]));
                tmem_wait_ld();
                }
                if constexpr (EXTRA && !BIAS) {
                    // score additions on the raw scores, before the mask (which must leave -inf behind): the registers
                    // then hold the finished scores in base-2 units, and the scale below becomes 1
                    const float dist0 = (float)(row + sk - sq - key0);  // i + sk - sq - j at the first column
                    const float slope_l2 = slope * kLog2e;
#pragma unroll
                    for (int j = 0; j < NC; ++j) {
                        const float sj = __uint_as_float(sreg[j]), dj = fabsf(dist0 - (float)j);
                        float x;
                        if (capped) x = (p.soft_cap * tanh_inline(sj * p.scale * inv_cap) - slope * dj) * kLog2e;
                        else x = fmaf(-slope_l2, dj, sj * p.scale_log2);  // (scale, slope and distance in base-2 units)
                        sreg[j] = __float_as_uint(x);
                    }
                }
                // mask the diagonal and tail tiles
                const bool need_mask = (key0 + NC > sk) ||
                                       (p.causal && wr >= 0 && key0 + NC - 1 > tile_first_row + shift + wr) ||
                                       (WINDOW && p.causal && wl >= 0 && key0 < tile_first_row + BM - 1 + shift - wl);
                if (need_mask) {
#pragma unroll
                    for (int j = 0; j < NC; ++j)
                        if (key0 + j > limit || (WINDOW && key0 + j < first_key)) sreg[j] = 0xff800000u;  // -inf
                }
                float mx;
                {
                    float a0 = -INFINITY, a1 = -INFINITY, a2 = -INFINITY, a3 = -INFINITY;  // four independent chains
#pragma unroll
                    for (int j = 0; j < NC; j += 8) {
                        a0 = max3(a0, __uint_as_float(sreg[j]), __uint_as_float(sreg[j + 1]));
                        a1 = max3(a1, __uint_as_float(sreg[j + 2]), __uint_as_float(sreg[j + 3]));
                        a2 = max3(a2, __uint_as_float(sreg[j + 4]), __uint_as_float(sreg[j + 5]));
                        a3 = max3(a3, __uint_as_float(sreg[j + 6]), __uint_as_float(sreg[j + 7]));
                    }
                    mx = fmaxf(max3(a0, a1, a2), a3);
                }
                const float scale_eff = EXTRA ? 1.f : p.scale_log2;
                mx *= scale_eff;  // scale > 0: max commutes with scaling
                // raise the running max only on a jump of more than 2^8 (2^2 with the packed exp2); rescale O in TMEM then
                const bool grow = mx > m_used + p.rescale_thr;
                if (n > 0 && __any_sync(0xffffffffu, grow)) {
                    if (SPLIT) {
                        // O must be at rest: the PV of step n-1 may still be running, S of this step was computed ahead
                        // of it.
                        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctrl->pv_done[sb ^ 1], ((gstep - 1u) >> 1) & 1u,
                                                                       abort_flag, p.status, 0x1000));
                        if (!ok) break;
                        tc_fence_after();
                    }
                    const float alpha = grow ? fast_exp2(m_used - mx) : 1.f;  // exp2(-inf) = 0
                    l *= alpha;
#pragma unroll
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t t[32];
                        tmem_ld32(tO + c * 32, t);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) t[j] = __float_as_uint(__uint_as_float(t[j]) * alpha);
                        tmem_st32(tO + c * 32, t);
                    }
                    tmem_wait_st();
                }
                if (grow) m_used = mx;
                const float msub = (m_used == -INFINITY) ? 0.f : m_used;
                const float2 sc2 = make_float2(scale_eff, scale_eff), nm2 = make_float2(-msub, -msub);
                float2 psa = make_float2(0.f, 0.f), psb = make_float2(0.f, 0.f);
                // P = 2^(S * scale - max) for the 128 columns of the row, 64 at a time.  NPOLY8 of every 8 column
                // pairs take the polynomial; tiles with masked (-inf) entries use the exp2 unit only, which returns
                // exact zeros for them.  The two variants are separate straight-line loops so that the scheduler
                // can interleave exp2-unit and FMA-pipe work across column pairs.
                auto exp_half = [&](int c, auto use_poly_tag) {
                    [[maybe_unused]] constexpr int NP = decltype(use_poly_tag)::value;
                    if constexpr (F8) {
                        // 8-bit P: stretched by scale_p, rounded (saturating) to the operand format, four keys per
                        // TMEM column; the row sum takes the unrounded values
                        constexpr __nv_fp8_interpretation_t kind = std::is_same<T, f8e4m3_t>::value ? __NV_E4M3 : __NV_E5M2;
                        const float2 sp2 = make_float2(p.scale_p, p.scale_p);
                        uint32_t pk8[16];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int e = c * 64 + 2 * j;
                            const float2 x = __ffma2_rn(make_float2(__uint_as_float(sreg[e]), __uint_as_float(sreg[e + 1])), sc2, nm2);
                            float2 pr;
                            pr.x = ex2_fast(x.x);
                            pr.y = ex2_fast(x.y);
                            if (j & 1) psb = __fadd2_rn(psb, pr); else psa = __fadd2_rn(psa, pr);
                            const uint32_t q2 = (uint32_t)__nv_cvt_float2_to_fp8x2(__fmul2_rn(pr, sp2), __NV_SATFINITE, kind);
                            if (j & 1) pk8[j >> 1] |= q2 << 16; else pk8[j >> 1] = q2;
                        }
                        tmem_st16(tSb + c * 16, pk8);
                    } else {
                    uint32_t pk[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int e = c * 64 + 2 * j;
                        const float2 x = __ffma2_rn(make_float2(__uint_as_float(sreg[e]), __uint_as_float(sreg[e + 1])), sc2, nm2);
                        if constexpr (HEXP) {
                            const uint32_t ph = ex2_f16x2(pack_f16x2(x.x, x.y));
                            if constexpr (std::is_same<T, __half>::value) {  // P is the unit's result as it stands
                                if (j & 1) add_f16x2_to(psb, ph); else add_f16x2_to(psa, ph);
                                pk[j] = ph;
                            } else {
                                const float2 pr = unpack_f16x2(ph);
                                if (j & 1) psb = __fadd2_rn(psb, pr); else psa = __fadd2_rn(psa, pr);
                                pk[j] = Elem<T>::pack2(pr.x, pr.y);
                            }
                            continue;
                        }
                        float2 pr;
                        if (NP > 0 && ((j * NP) & 7) < NP) pr = exp2_poly2(x);
                        else { pr.x = ex2_fast(x.x); pr.y = ex2_fast(x.y); }
                        if (j & 1) psb = __fadd2_rn(psb, pr); else psa = __fadd2_rn(psa, pr);
                        pk[j] = Elem<T>::pack2(pr.x, pr.y);
                    }
                    tmem_st32(tSb + (SPLIT == 2 ? khalf : c) * 32, pk);
                    }
                };
                // Prefill forms: P is handed over in two halves (a barrier each: with one barrier the second arrival could
                // complete before the issuer has looked at the first), so that the PV of keys 0-63 is on the tensor pipe
                // while the exponentials of keys 64-127 are taken.
                auto hand_over_first_half = [&]() {
                    if constexpr (HALVES) {
                        tmem_wait_st();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&ctrl->p_full[sb]);
                    }
                };
                if (need_mask) {
                    exp_half(0, std::integral_constant<int, 0>{});
                    hand_over_first_half();
                    if (SPLIT != 2) exp_half(1, std::integral_constant<int, 0>{});
                } else {
                    exp_half(0, std::integral_constant<int, NPOLY8>{});
                    hand_over_first_half();
                    if (SPLIT != 2) exp_half(1, std::integral_constant<int, NPOLY8>{});
                }
                if (SPLIT == 2) {  // this copy of the row gives the other 64 keys no weight
                    uint32_t zero[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) zero[j] = 0u;
                    tmem_st32(tSb + (1 - khalf) * 32, zero);
                }
                l += (psa.x + psa.y) + (psb.x + psb.y);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(HALVES ? &ctrl->p_full2[sb] : &ctrl->p_full[sb]);
            }
            if (!ok) break;
            sc += Ni;
            // ---- epilogue: O / l and LSE ----
            if (Ni > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctrl->o_full[i], oc & 1u, abort_flag, p.status, 0x400 << i));
                if (!ok) break;
                ++oc;
                tc_fence_after();
            }
            if (SPLIT) {
                // fp32 partial of this split, normalised inside the split, and its LSE (natural log)
                if (i == 0 && tile_first_row < sq) {
                    const float inv = l > 0.f ? 1.f / l : 0.f;
                    const int split = SPLIT == 2 ? 2 * it.h[1] + khalf : it.h[1];
                    const int64_t slot = p.seqstart_q
                        ? ((int64_t)head * p.num_splits + split) * p.total_q + it.q0 + row
                        : (((int64_t)it.b * p.hq + head) * p.num_splits + split) * p.sq_cap + row;
                    // The rows of a warp go to 32 different places of the workspace (one per token and head), 512
                    // bytes each.  They pass through shared memory (32 rows x 32 columns, 16-byte pieces rotated by
                    // row against bank conflicts) so that eight lanes write one row's 128 bytes together.
                    const unsigned long long my_ptr = row_ok ? (unsigned long long)(p.o_acc + slot * HD) : 0ull;
                    float* stage = reinterpret_cast<float*>(sStage + (warp & 3) * 4096);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t t[32];
                        if (Ni > 0) {
                            tmem_ld32(tO + c * 32, t);
                            tmem_wait_ld();
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) t[j] = 0u;
                        }
                        __syncwarp();  // the previous chunk has been read out of the staging rows
#pragma unroll
                        for (int v4 = 0; v4 < 8; ++v4)
                            *reinterpret_cast<float4*>(stage + lane * 32 + ((v4 ^ (lane & 7)) << 2)) =
                                make_float4(__uint_as_float(t[v4 * 4 + 0]) * inv, __uint_as_float(t[v4 * 4 + 1]) * inv,
                                            __uint_as_float(t[v4 * 4 + 2]) * inv, __uint_as_float(t[v4 * 4 + 3]) * inv);
                        __syncwarp();
#pragma unroll
                        for (int g4 = 0; g4 < 8; ++g4) {  // four rows per pass: lane = (row in the pass, 16-byte piece)
                            const int srow = g4 * 4 + (lane >> 3), piece = lane & 7;
                            const unsigned long long dst = __shfl_sync(0xffffffffu, my_ptr, srow);
                            const float4 val = *reinterpret_cast<const float4*>(stage + srow * 32 + ((piece ^ (srow & 7)) << 2));
                            if (dst) *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + c * 32 + piece * 4) = val;
                        }
                    }
                    if (p.lse_acc && row_ok)
                        p.lse_acc[slot] = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
                }
            } else if (tile_first_row < sq) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                // Whole tiles leave through shared memory and TMA stores (32 rows x 32 columns per warp and store), which
                // keeps the load/store unit free for the other warps; a tile that reaches past the end of its sequence
                // is written row by row, because its surplus rows belong to the next sequence of the packed buffer.
                if constexpr (F8) {
                    // 8-bit instances: O = scale_o * acc / l in the output type the call names, written row by row
                    // (a row of 128 values is 128 or 256 contiguous bytes)
                    const float f = inv * p.scale_o;
                    const int64_t orow_elems = ((int64_t)(it.q0 + row) * p.hq + head) * HD;
#pragma unroll
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t t[32];
                        if (Ni > 0) {
                            tmem_ld32(tO + c * 32, t);
                            tmem_wait_ld();
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) t[j] = 0u;
                        }
                        if (!row_ok) continue;
                        if (p.out_dtype == FLASHCK_DTYPE_FLOAT8 || p.out_dtype == FLASHCK_DTYPE_BFLOAT8) {
                            const __nv_fp8_interpretation_t okind = p.out_dtype == FLASHCK_DTYPE_FLOAT8 ? __NV_E4M3 : __NV_E5M2;
                            uint32_t w[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                                    make_float2(__uint_as_float(t[4 * j]) * f, __uint_as_float(t[4 * j + 1]) * f), __NV_SATFINITE, okind);
                                const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                                    make_float2(__uint_as_float(t[4 * j + 2]) * f, __uint_as_float(t[4 * j + 3]) * f), __NV_SATFINITE, okind);
                                w[j] = lo | (hi << 16);
                            }
                            uint8_t* dst = (uint8_t*)p.o + orow_elems + c * 32;
                            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                            *reinterpret_cast<uint4*>(dst + 16) = make_uint4(w[4], w[5], w[6], w[7]);
                        } else {
                            uint32_t w[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const float a = __uint_as_float(t[2 * j]) * f, b = __uint_as_float(t[2 * j + 1]) * f;
                                w[j] = p.out_dtype == FLASHCK_DTYPE_BFLOAT16 ? Elem<__nv_bfloat16>::pack2(a, b) : Elem<__half>::pack2(a, b);
                            }
                            uint8_t* dst = (uint8_t*)p.o + (orow_elems + c * 32) * 2;
#pragma unroll
                            for (int v4 = 0; v4 < 4; ++v4)
                                *reinterpret_cast<uint4*>(dst + v4 * 16) = make_uint4(w[4 * v4], w[4 * v4 + 1], w[4 * v4 + 2], w[4 * v4 + 3]);
                        }
                    }
                } else {
                const bool whole_tile = tile_first_row + BM <= sq;
                uint8_t* stage = sStage + warp * STAGE_BYTES;
                T* orow = (T*)p.o + ((int64_t)(it.q0 + row) * p.hq + head) * HD;
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t t[32];
                    if (Ni > 0) {
                        tmem_ld32(tO + c * 32, t);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) t[j] = 0u;
                    }
                    uint4 pk[4];
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        pk[v4].x = Elem<T>::pack2(__uint_as_float(t[v4 * 8 + 0]) * inv, __uint_as_float(t[v4 * 8 + 1]) * inv);
                        pk[v4].y = Elem<T>::pack2(__uint_as_float(t[v4 * 8 + 2]) * inv, __uint_as_float(t[v4 * 8 + 3]) * inv);
                        pk[v4].z = Elem<T>::pack2(__uint_as_float(t[v4 * 8 + 4]) * inv, __uint_as_float(t[v4 * 8 + 5]) * inv);
                        pk[v4].w = Elem<T>::pack2(__uint_as_float(t[v4 * 8 + 6]) * inv, __uint_as_float(t[v4 * 8 + 7]) * inv);
                    }
                    if (whole_tile) {
                        if (lane == 0) tma_store_wait_read();  // the previous store has read the staging buffer
                        __syncwarp();
#pragma unroll
                        for (int v4 = 0; v4 < 4; ++v4)  // row `lane` of the chunk: 64 bytes in the 64-byte swizzle of the map
                            *reinterpret_cast<uint4*>(stage + lane * 64 + ((v4 ^ (lane >> 1)) & 3) * 16) = pk[v4];
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_3d(&map_o, stage, c * 32, head, it.q0 + tile_first_row + (warp & 3) * 32);
                            tma_store_commit();
                        }
                    } else if (row_ok) {
#pragma unroll
                        for (int v4 = 0; v4 < 4; ++v4) *reinterpret_cast<uint4*>(orow + c * 32 + v4 * 8) = pk[v4];
                    }
                }
                }
                if (p.lse && row_ok) {
                    float* lp = p.seqstart_q ? p.lse + (int64_t)head * p.total_q + it.q0 + row
                                             : p.lse + ((int64_t)it.b * p.hq + head) * p.seqlen_q + row;
                    *lp = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
                }
                // the O reads above are complete (wait::ld) before this warp's next P store releases the next PV
            }
        }
    }

    if (warp < 8 && lane == 0) tma_store_wait_read();  // shared memory stays valid until the last O store has read it
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;\n" ::"r"(tmem));
    }
}

int make_map_3d(CUtensorMap* map, const void* base, int dtype, int64_t rows, int64_t heads, int box_rows = BM, int hd = HD) {
    PFN_encodeTiled enc = get_encode_tiled();
    FCK_REQUIRE(enc != nullptr, FLASHCK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    // boxes of 128 bytes of a row (64 16-bit or 128 8-bit elements; the 8-bit formats travel as plain bytes)
    const bool f8 = dtype == FLASHCK_DTYPE_FLOAT8 || dtype == FLASHCK_DTYPE_BFLOAT8;
    const int es = f8 ? 1 : 2;
    const cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)(rows > 0 ? rows : 1)};
    const cuuint64_t strides[2] = {(cuuint64_t)(hd * es), (cuuint64_t)(heads * hd * es)};
    const cuuint32_t box[3] = {(cuuint32_t)(128 / es), 1, (cuuint32_t)box_rows};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapDataType dt = f8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
        : dtype == FLASHCK_DTYPE_BFLOAT16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult r = enc(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FCK_REQUIRE(r == CUDA_SUCCESS, FLASHCK_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) rows=%lld heads=%lld", (int)r,
                (long long)rows, (long long)heads);
    return FLASHCK_OK;
}

// O [rows, heads, 128] as 32-row x 32-column boxes (64-byte rows, 64-byte swizzle) for the epilogue's TMA stores.
int make_map_o(CUtensorMap* map, const void* base, int dtype, int64_t rows, int64_t heads, int hd = HD) {
    PFN_encodeTiled enc = get_encode_tiled();
    FCK_REQUIRE(enc != nullptr, FLASHCK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)(rows > 0 ? rows : 1)};
    const cuuint64_t strides[2] = {(cuuint64_t)(hd * 2), (cuuint64_t)(heads * hd * 2)};
    const cuuint32_t box[3] = {32, 1, 32};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapDataType dt =
        dtype == FLASHCK_DTYPE_BFLOAT16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult r = enc(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FCK_REQUIRE(r == CUDA_SUCCESS, FLASHCK_ERR_CUDA, "cuTensorMapEncodeTiled (O) failed (%d) rows=%lld heads=%lld", (int)r,
                (long long)rows, (long long)heads);
    return FLASHCK_OK;
}

template <typename T, int EXPM, int VAR, int SPLIT, int HDIM = 128>
int launch_t(const FwdParams& p, const Sm100Dev& dev, cudaStream_t stream) {
    const int64_t rows_q = p.seqstart_q ? p.total_q : p.batch * p.seqlen_q;
    const bool paged = p.block_table || p.kv_indptr;
    // contiguous: group mode carries the packed total in seqlen_k.  Paged: the token axis of the pools' maps ends with
    // the pool (num_pages pages), so a stale or corrupt page id reads as zeros instead of memory outside the pools.
    const int64_t rows_k = paged ? std::max<int64_t>(p.num_pages, 1) * p.page
                                 : (p.seqstart_k ? p.seqlen_k : p.batch * p.seqlen_k);
    const int box_k = paged ? (int)std::min<int64_t>(p.page, BN) : BN;
    CUtensorMap mq, mk, mv, mo;
    int rc;
    if ((rc = make_map_3d(&mq, p.q, p.dtype, rows_q, p.hq, BM, HDIM))) return rc;
    if ((rc = make_map_3d(&mk, p.k, p.dtype, rows_k, p.hkv, box_k, HDIM))) return rc;
    if ((rc = make_map_3d(&mv, p.v, p.dtype, rows_k, p.hkv, box_k, HDIM))) return rc;
    if constexpr (ElemInfo<T>::f8) mo = mq;  // (the 8-bit instances write O with plain stores: the map is not used)
    else if ((rc = make_map_o(&mo, p.o, p.dtype, rows_q, p.hq, HDIM))) return rc;
    auto kern = fmha_fwd_sm100_kernel<T, EXPM, VAR, SPLIT, HDIM>;
    const size_t smem = 1024 + (size_t)(2 + 2 * KV_SLOTS) * (BM * HDIM * ElemInfo<T>::bytes) + 8 * STAGE_BYTES + sizeof(Ctrl);
    static thread_local int configured_device = -1;
    int devid = 0;
    FCK_CUDA(cudaGetDevice(&devid));
    if (configured_device != devid) {
        FCK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured_device = devid;
    }
    if (p.max_seqlen_q == 0 || p.batch == 0) return FLASHCK_OK;
    // persistent: one CTA per SM walks the device-side work list
    FCK_CUDA(launch_dependent(kern, dim3(sm_count()), dim3(NTHREADS), smem, stream, mq, mk, mv, mo, dev));
    return FLASHCK_OK;
}

}  // namespace

bool fwd_sm100_supported(const FwdParams& p) {
    if (!g_use_sm100.load()) return false;
    if (p.d != p.dv || (p.d != 128 && p.d != 64)) return false;
    if (p.d == 64 && !g_use_sm100_hdim64.load()) return false;
    if (p.dtype == FLASHCK_DTYPE_FLOAT8 || p.dtype == FLASHCK_DTYPE_BFLOAT8) {
        // the 8-bit instances: hdim 128, contiguous K/V, no score additions
        if (!g_use_sm100_fp8.load() || p.d != 128 || p.bias || p.logits_soft_cap > 0.f || p.block_table || p.kv_indptr) return false;
    }
    if (p.bias && p.bias_type == 1) {
        // an elementwise bias tensor: the BIAS instances (hdim 128, contiguous K/V of the stated length, 16-bit elements)
        if (!g_use_sm100_bias.load() || p.d != 128 || p.block_table || p.kv_indptr || p.bias_rank > 2) return false;
        if (p.bias_rank == 2 && p.seqstart_q) return false;
    }
    if (p.bias && p.bias_type == 2 && p.bias_rank > 1) return false;
    const bool paged = p.block_table || p.kv_indptr;
    if (paged) {
        // pages of 16 .. 128 tokens that divide a 128-key tile, or whole multiples of it
        if (p.page < 16 || !((BN % p.page == 0) || (p.page % BN == 0))) return false;
        if (p.seqlen_k64 || p.seqstart_k) return false;
        if (p.kv_indptr && (!p.kv_page_indices || !p.kv_last_page_len || p.cache_batch_idx)) return false;
    } else {
        if (p.cache_batch_idx || p.seqlen_k64 || p.seqlen_k32) return false;
        if ((p.seqstart_q == nullptr) != (p.seqstart_k == nullptr)) return false;
    }
    if (p.mask_type > 3) return false;
    if (p.wl >= (1ll << 30) || p.wr >= (1ll << 30)) return false;
    if (p.batch > kMaxBatch || (p.max_seqlen_q + BM - 1) / BM > kMaxLevels) return false;  // on-chip schedule
    if (p.hq > 1023) return false;
    {   // work items per CTA, bounded from the longest sequence: the on-chip work list holds kMaxRounds
        const bool pair = (p.hq / p.hkv) % 2 == 0;
        const int64_t rows_per_block = pair ? BM : 2 * BM;
        const int64_t items = p.batch * ((p.max_seqlen_q + rows_per_block - 1) / rows_per_block) * (pair ? p.hq / 2 : p.hq);
        if ((items + sm_count() - 1) / sm_count() > kMaxRounds) return false;
    }
    if (p.total_q >= (1ll << 31) || (!paged && p.batch * p.seqlen_k >= (1ll << 31))) return false;
    if (paged && p.num_pages * p.page >= (1ll << 31)) return false;  // token rows of the pools are 31-bit coordinates
    if (p.batch * std::max<int64_t>(p.seqlen_q, 1) >= (1ll << 31)) return false;
    return true;
}

int launch_fwd_sm100(const FwdParams& p, cudaStream_t stream) {
    int* status = device_status_ptr();
    if (!status) return FLASHCK_ERR_CUDA;
    Sm100Dev dev{};
    dev.o = p.o; dev.lse = p.lse; dev.seqstart_q = p.seqstart_q; dev.seqstart_k = p.seqstart_k; dev.status = status;
    dev.batch = (int)p.batch; dev.seqlen_q = (int)p.seqlen_q; dev.seqlen_k = (int)p.seqlen_k;
    dev.hq = (int)p.hq; dev.hkv = (int)p.hkv; dev.total_q = (int)p.total_q;
    dev.v = p.v;
    dev.page_ids = p.kv_indptr ? p.kv_page_indices : p.block_table;
    dev.kv_indptr = p.kv_indptr; dev.kv_last_page_len = p.kv_last_page_len; dev.seqlen_k32 = p.seqlen_k32;
    dev.cache_batch_idx = p.cache_batch_idx;
    dev.page = (p.block_table || p.kv_indptr) ? (int)p.page : 0;
    dev.bt_stride = (int)p.bt_stride;
    dev.causal = p.mask_type;
    dev.wl = p.wl < 0 ? -1 : (int)p.wl;
    dev.wr = p.wr < 0 ? -1 : (int)p.wr;
    dev.pair_heads = ((p.hq / p.hkv) % 2 == 0) ? 1 : 0;
    dev.num_levels = (int)((p.max_seqlen_q + (dev.pair_heads ? BM : 2 * BM) - 1) / (dev.pair_heads ? BM : 2 * BM));
    dev.scale_log2 = p.scale * 1.4426950408889634f;
    const bool bf16 = p.dtype == FLASHCK_DTYPE_BFLOAT16;
    const bool window = p.mask_type != 0 && !(p.wl < 0 && p.wr == 0);
    const bool ebias = p.bias && p.bias_type == 1;
    const bool extra = (p.bias && p.bias_type == 2) || p.logits_soft_cap > 0.f;
    const int expm = extra ? 0 : (int)g_exp_mode.load();
    dev.rescale_thr = expm == 1 ? 0.01f * (float)g_rescale_half_x100.load() : kRescaleThreshold;
    dev.scale = p.scale; dev.soft_cap = p.logits_soft_cap;
    dev.alibi = (p.bias && p.bias_type == 2) ? (const float*)p.bias : nullptr; dev.alibi_rank = p.bias_rank;
    if (p.dtype == FLASHCK_DTYPE_FLOAT8 || p.dtype == FLASHCK_DTYPE_BFLOAT8) {
        // The running max may lag the row max by `thr` (P up to 2^thr) only as far as P * scale_p stays inside the 8-bit
        // format: thr = log2(largest finite value / scale_p), at most the 16-bit instances' threshold, at least 0 (the
        // max then follows every increase).  scale_p = 256: 0.8 for E4M3 (max 448), 7.8 for E5M2 (max 57344).
        {
            const float fmt_max = p.dtype == FLASHCK_DTYPE_FLOAT8 ? 448.f : 57344.f;
            const float thr = log2f(fmt_max / p.scale_p);
            dev.rescale_thr = thr < 0.f ? 0.f : (thr > kRescaleThreshold ? kRescaleThreshold : thr);
        }
        dev.scale_p = p.scale_p; dev.scale_o = p.scale_o; dev.out_dtype = p.out_dtype;
        const bool e4 = p.dtype == FLASHCK_DTYPE_FLOAT8;
        if (window) return e4 ? launch_t<f8e4m3_t, 0, 1, 0>(p, dev, stream) : launch_t<f8e5m2_t, 0, 1, 0>(p, dev, stream);
        return e4 ? launch_t<f8e4m3_t, 0, 0, 0>(p, dev, stream) : launch_t<f8e5m2_t, 0, 0, 0>(p, dev, stream);
    }
    if (ebias) {  // (an elementwise bias: fp32 exponentials on the exp2 unit, with or without a second mask bound)
        dev.rescale_thr = kRescaleThreshold;
        dev.bias_el = p.bias; dev.bias_el_rank = p.bias_rank;
        dev.bias_sk = p.seqlen_k; dev.bias_sq = p.seqstart_q ? p.total_q : p.seqlen_q;
        if (window) return bf16 ? launch_t<__nv_bfloat16, 0, 5, 0>(p, dev, stream) : launch_t<__half, 0, 5, 0>(p, dev, stream);
        return bf16 ? launch_t<__nv_bfloat16, 0, 4, 0>(p, dev, stream) : launch_t<__half, 0, 4, 0>(p, dev, stream);
    }
#define FCK_SM100_LAUNCH(E, V) \
    return bf16 ? launch_t<__nv_bfloat16, E, V, 0>(p, dev, stream) : launch_t<__half, E, V, 0>(p, dev, stream)
    if (p.d == 64) {  // the hdim-64 instances: fp32 exponentials on the exp2 unit, every mask and score addition
        dev.rescale_thr = kRescaleThreshold;
        switch ((window ? 1 : 0) | (extra ? 2 : 0)) {
            case 0: return bf16 ? launch_t<__nv_bfloat16, 0, 0, 0, 64>(p, dev, stream) : launch_t<__half, 0, 0, 0, 64>(p, dev, stream);
            case 1: return bf16 ? launch_t<__nv_bfloat16, 0, 1, 0, 64>(p, dev, stream) : launch_t<__half, 0, 1, 0, 64>(p, dev, stream);
            case 2: return bf16 ? launch_t<__nv_bfloat16, 0, 2, 0, 64>(p, dev, stream) : launch_t<__half, 0, 2, 0, 64>(p, dev, stream);
            default: return bf16 ? launch_t<__nv_bfloat16, 0, 3, 0, 64>(p, dev, stream) : launch_t<__half, 0, 3, 0, 64>(p, dev, stream);
        }
    }
    if (extra) {  // (the score-addition instances take their exponentials in fp32 on the exp2 unit)
        if (window) { FCK_SM100_LAUNCH(0, 3); }
        FCK_SM100_LAUNCH(0, 2);
    }
    if (window) {  // (the window instances come with the two exp2-unit forms only)
        if (expm == 1) { FCK_SM100_LAUNCH(1, 1); }
        FCK_SM100_LAUNCH(0, 1);
    }
    switch (expm) {
        case 1: FCK_SM100_LAUNCH(1, 0);
        case 11: FCK_SM100_LAUNCH(11, 0);
        case 12: FCK_SM100_LAUNCH(12, 0);
        case 13: FCK_SM100_LAUNCH(13, 0);
        default: FCK_SM100_LAUNCH(0, 0);
    }
#undef FCK_SM100_LAUNCH
}

// ---- split-KV with several query rows per kv head (append + decode, speculative decoding, chunked prefill) ----
namespace {


// Q [tokens, hkv, group, 128] as boxes of (64 columns, group heads, 1 kv head, 128/group tokens).
int make_map_q_packed(CUtensorMap* map, const void* base, int dtype, int64_t tokens, int64_t hkv, int64_t group, int rows) {
    PFN_encodeTiled enc = get_encode_tiled();
    FCK_REQUIRE(enc != nullptr, FLASHCK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)group, (cuuint64_t)hkv, (cuuint64_t)(tokens > 0 ? tokens : 1)};
    const cuuint64_t strides[3] = {(cuuint64_t)(HD * 2), (cuuint64_t)(group * HD * 2), (cuuint64_t)(hkv * group * HD * 2)};
    const cuuint32_t box[4] = {64, (cuuint32_t)group, 1, (cuuint32_t)(rows / group)};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt =
        dtype == FLASHCK_DTYPE_BFLOAT16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult r = enc(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FCK_REQUIRE(r == CUDA_SUCCESS, FLASHCK_ERR_CUDA, "cuTensorMapEncodeTiled (packed Q) failed (%d)", (int)r);
    return FLASHCK_OK;
}

int64_t split_cap_tiles(const SplitKVParams& p) {  // key tiles of the longest sequence the cache can hold
    const int64_t cap = p.block_table ? p.bt_stride * p.page : p.seqlen_k_cap;
    return (cap + BN - 1) / BN;
}
// At most 64 packed rows and room for two splits per piece: the rows are duplicated (kernel mode 2).
bool split_duplicates_rows(const SplitKVParams& p) {
    return p.max_seqlen_q * (p.hq / p.hkv) <= 64 && p.num_splits >= 2;
}

template <typename T, int SPLIT, int EXPM>
int launch_split_t(const SplitKVParams& p, const Sm100Dev& dev, cudaStream_t stream) {
    const int64_t tokens = p.seqstart_q ? p.total_q : p.batch * p.seqlen_q;
    const int box_k = p.block_table ? (int)std::min<int64_t>(p.page, BN) : BN;
    CUtensorMap mq, mk, mv;
    int rc;
    if ((rc = make_map_q_packed(&mq, p.q, p.dtype, tokens, p.hkv, p.hq / p.hkv, SPLIT == 2 ? 64 : BM))) return rc;
    // Paged pools: the map ends with the pool (num_pages pages: a page id beyond it reads as zeros), and a copy never
    // leaves its page.  Contiguous cache [batch, capacity, hkv, 128]: the last 128-token chunk of a row reaches past the
    // row's end, and past the end of the buffer in the last row; the map carries the true row count so that those rows
    // are not read (they come as zeros).
    const int64_t cache_rows = p.block_table ? std::max<int64_t>(p.num_pages, 1) * p.page : p.batch * p.seqlen_k_cap;
    if ((rc = make_map_3d(&mk, p.k, p.dtype, cache_rows, p.hkv, box_k))) return rc;
    if ((rc = make_map_3d(&mv, p.v, p.dtype, cache_rows, p.hkv, box_k))) return rc;
    auto kern = fmha_fwd_sm100_kernel<T, EXPM, 0, SPLIT>;
    const size_t smem = 1024 + (size_t)(2 + 2 * KV_SLOTS) * TILE_BYTES + 8 * STAGE_BYTES + sizeof(Ctrl);
    static thread_local int configured_device = -1;
    int devid = 0;
    FCK_CUDA(cudaGetDevice(&devid));
    if (configured_device != devid) {
        FCK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured_device = devid;
    }
    FCK_CUDA(launch_dependent(kern, dim3(sm_count()), dim3(NTHREADS), smem, stream, mq, mk, mv, mq, dev));
    return FLASHCK_OK;
}

}  // namespace

bool splitkv_sm100_supported(const SplitKVParams& p) {
    if (!g_use_sm100_splitkv.load()) return false;
    if (p.alibi_slopes) return false;  // ALiBi runs on the mma.sync decode kernel
    if (p.d != HD || p.dv != HD || p.batch <= 0 || p.batch > kMaxBatch || p.hq > 1023) return false;
    const int64_t group = p.hq / p.hkv;
    if (group > BM || BM % group != 0) return false;
    // one 16-row tile of (token, group head) rows is what the mma.sync decode kernel serves at the HBM rate
    if (p.max_seqlen_q * group <= 16) return false;
    if ((p.max_seqlen_q * group + BM - 1) / BM > 16) return false;
    if (p.seqstart_k) return false;                           // paged or [rows, seqlen_k, hkv, d] caches
    if (p.mask_type > 2 || (p.mask_type != 0 && !(p.wl < 0 && p.wr == 0))) return false;  // none or causal
    if (p.block_table) {
        if (p.page < 16 || !((BN % p.page == 0) || (p.page % BN == 0)) || p.cache_batch_idx) return false;
    } else if (p.seqlen_k_cap <= 0 || p.cache_batch_idx) {
        return false;  // (with cache_batch_idx the number of cache rows is not known here: see the K/V maps)
    }
    if (p.num_splits > 1 && !p.lse_acc) return false;
    if (p.num_splits > 255) return false;  // the split index of a work item has 8 bits
    // The work line (see kItemCostDefault) is indexed with 31 bits, and a CTA's work list holds kSplitItems items: a CTA's
    // piece of w units reaches into at most w / item_cost + 2 streams, and w is at most the larger of the line's
    // 148th, the shortest piece, and what keeps the longest possible stream within the workspace's splits.
    const int64_t cap_tiles = split_cap_tiles(p);
    const int64_t streams = p.batch * p.hkv * ((p.max_seqlen_q * group + BM - 1) / BM);
    const int64_t item_cost = g_split_item_cost.load(), min_piece = g_split_min_piece_tiles.load();
    const int64_t line = streams * (cap_tiles + item_cost);
    if (line >= (1ll << 31)) return false;
    const int64_t max_pieces = std::max<int64_t>(1, split_duplicates_rows(p) ? p.num_splits / 2 : p.num_splits);
    int64_t w_max = std::max<int64_t>(line / sm_count() + 1, min_piece + item_cost);
    if (max_pieces >= 2) w_max = std::max(w_max, cap_tiles / (max_pieces - 1) + 1);
    if (std::min(streams, w_max / item_cost + 2) > kSplitItems) return false;
    const int64_t tokens = p.seqstart_q ? p.total_q : p.batch * p.seqlen_q;
    if (tokens >= (1ll << 31) || (!p.block_table && p.batch * p.seqlen_k_cap >= (1ll << 31))) return false;
    if (p.block_table && p.num_pages * p.page >= (1ll << 31)) return false;
    return true;
}

int launch_splitkv_sm100(const SplitKVParams& p, cudaStream_t stream) {
    int* status = device_status_ptr();
    if (!status) return FLASHCK_ERR_CUDA;
    if (p.batch == 0 || p.max_seqlen_q == 0) return FLASHCK_OK;
    Sm100Dev dev{};
    dev.o = nullptr; dev.lse = nullptr; dev.seqstart_q = p.seqstart_q; dev.seqstart_k = nullptr; dev.status = status;
    dev.batch = (int)p.batch; dev.seqlen_q = (int)p.seqlen_q; dev.seqlen_k = (int)p.seqlen_k_cap;
    dev.hq = (int)p.hq; dev.hkv = (int)p.hkv; dev.total_q = (int)p.total_q;
    dev.v = p.v;
    dev.page_ids = p.block_table; dev.seqlen_k32 = p.seqlen_k; dev.cache_batch_idx = p.cache_batch_idx;
    // a contiguous cache goes through the chunked loader too (chunk = 128 tokens): the rows behind a sequence's end
    // are uninitialised cache, which the loader keeps out of V
    dev.page = p.block_table ? (int)p.page : BN;
    dev.bt_stride = (int)p.bt_stride;
    dev.o_acc = p.o_acc; dev.lse_acc = p.lse_acc; dev.num_splits = (int)p.num_splits;
    dev.piece_tiles = (int)g_split_min_piece_tiles.load();
    dev.item_cost = (int)g_split_item_cost.load();
    dev.group = (int)(p.hq / p.hkv);
    dev.sq_cap = (int)p.seqlen_q;
    dev.causal = p.mask_type; dev.wl = -1; dev.wr = p.mask_type ? 0 : -1;
    dev.pair_heads = 0; dev.num_levels = 1;
    dev.scale_log2 = p.scale * 1.4426950408889634f;
    const bool bf16 = p.dtype == FLASHCK_DTYPE_BFLOAT16;
    const bool hexp = g_exp_mode_splitkv.load() == 1;
    dev.rescale_thr = hexp ? 0.01f * (float)g_rescale_half_x100.load() : kRescaleThreshold;
    if (split_duplicates_rows(p)) {
        if (hexp) return bf16 ? launch_split_t<__nv_bfloat16, 2, 1>(p, dev, stream) : launch_split_t<__half, 2, 1>(p, dev, stream);
        return bf16 ? launch_split_t<__nv_bfloat16, 2, 0>(p, dev, stream) : launch_split_t<__half, 2, 0>(p, dev, stream);
    }
    if (hexp) return bf16 ? launch_split_t<__nv_bfloat16, 1, 1>(p, dev, stream) : launch_split_t<__half, 1, 1>(p, dev, stream);
    return bf16 ? launch_split_t<__nv_bfloat16, 1, 0>(p, dev, stream) : launch_split_t<__half, 1, 0>(p, dev, stream);
}

static bool valid_exp_mode(int64_t v) { return v == 0 || v == 1 || (v >= 11 && v <= 13); }

int fwd_set_param(const char* key, int64_t value) {
    if (!strcmp(key, "use_sm100")) { g_use_sm100 = value; return FLASHCK_OK; }
    if (!strcmp(key, "use_sm100_hdim64")) { g_use_sm100_hdim64 = value; return FLASHCK_OK; }
    if (!strcmp(key, "use_sm100_fp8")) { g_use_sm100_fp8 = value; return FLASHCK_OK; }
    if (!strcmp(key, "use_sm100_bias")) { g_use_sm100_bias = value; return FLASHCK_OK; }
    if (!strcmp(key, "use_sm100_splitkv")) { g_use_sm100_splitkv = value; return FLASHCK_OK; }
    if (!strcmp(key, "exp_mode")) {
        if (!valid_exp_mode(value)) return FLASHCK_ERR_INVALID_ARGUMENT;
        g_exp_mode = value;
        return FLASHCK_OK;
    }
    if (!strcmp(key, "exp_mode_splitkv")) {
        if (value != 0 && value != 1) return FLASHCK_ERR_INVALID_ARGUMENT;
        g_exp_mode_splitkv = value;
        return FLASHCK_OK;
    }
    if (!strcmp(key, "split_item_cost")) {
        if (value < 1 || value > 64) return FLASHCK_ERR_INVALID_ARGUMENT;
        g_split_item_cost = value;
        return FLASHCK_OK;
    }
    if (!strcmp(key, "split_min_piece_tiles")) {
        if (value < 1 || value > 4096) return FLASHCK_ERR_INVALID_ARGUMENT;
        g_split_min_piece_tiles = value;
        return FLASHCK_OK;
    }
    if (!strcmp(key, "rescale_log2_x100")) {
        if (value < 0 || value > 1400) return FLASHCK_ERR_INVALID_ARGUMENT;  // f16 holds 2^15; P < 2^14 leaves headroom
        g_rescale_half_x100 = value;
        return FLASHCK_OK;
    }
    if (!strcmp(key, "poly8")) {  // older spelling: the polynomial share alone (0 = exp2 unit in fp32)
        if (value < 0 || value > 3) return FLASHCK_ERR_INVALID_ARGUMENT;
        g_exp_mode = value ? 10 + value : 0;
        return FLASHCK_OK;
    }
    return FLASHCK_ERR_INVALID_ARGUMENT;
}
int fwd_get_param(const char* key, int64_t* value) {
    if (!strcmp(key, "use_sm100")) { *value = g_use_sm100; return FLASHCK_OK; }
    if (!strcmp(key, "use_sm100_hdim64")) { *value = g_use_sm100_hdim64; return FLASHCK_OK; }
    if (!strcmp(key, "use_sm100_fp8")) { *value = g_use_sm100_fp8; return FLASHCK_OK; }
    if (!strcmp(key, "use_sm100_bias")) { *value = g_use_sm100_bias; return FLASHCK_OK; }
    if (!strcmp(key, "use_sm100_splitkv")) { *value = g_use_sm100_splitkv; return FLASHCK_OK; }
    if (!strcmp(key, "exp_mode")) { *value = g_exp_mode; return FLASHCK_OK; }
    if (!strcmp(key, "exp_mode_splitkv")) { *value = g_exp_mode_splitkv; return FLASHCK_OK; }
    if (!strcmp(key, "rescale_log2_x100")) { *value = g_rescale_half_x100; return FLASHCK_OK; }
    if (!strcmp(key, "split_item_cost")) { *value = g_split_item_cost; return FLASHCK_OK; }
    if (!strcmp(key, "split_min_piece_tiles")) { *value = g_split_min_piece_tiles; return FLASHCK_OK; }
    if (!strcmp(key, "poly8")) { const int64_t m = g_exp_mode; *value = m >= 11 ? m - 10 : 0; return FLASHCK_OK; }
    return FLASHCK_ERR_INVALID_ARGUMENT;
}

}  // namespace fck
