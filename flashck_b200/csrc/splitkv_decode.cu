// fmha_fwd_splitkv: partial attention over contiguous or paged K/V, one partial (O_s, LSE_s) per split.
// Replaces ck_tile::FmhaFwdSplitKVKernel as instantiated by the reference
// (core/profiling/attention/fmha_fwd_split_kv/fmha_fwd_split_kv_codegen.cc:99-130) behind the C symbol
// FmhaFwdSplitKV (attention_kernels/fmha_fwd_split_kv/fmha_fwd_split_kv_jinja.h:155-184).
//
// HBM-bound (4-8 FLOP per K/V byte), so the design is about keeping bytes in flight:
//   * K/V stream through a ring of shared-memory stages filled by TMA.  One 5-D tensor map per pool,
//     dims (64 elements, token-in-page, kv head, hdim/64, page) -- the token axis is placed before the head
//     axis so that the box lands in shared memory as [hdim/64][head][token][64] rows of 128 bytes; with the
//     128-byte swizzle the 8 rows an ldmatrix touches (8 consecutive tokens of one head) fall in 8 different
//     bank groups.  A tile is 16 tokens x HK heads x hdim; with all 8 heads of a 16-token page it is one
//     contiguous 32 KB read of the pool.
//   * One producer warp walks the block table (32 page ids per coalesced load, one tile ahead) and issues
//     the copies; HK consumer warps (one kv head each) run QK^T and PV with mma.sync m16n8k16 on the
//     16-row tile formed by folding the GQA group (x seqlen_q) into M, with an fp32 online softmax whose
//     row reductions are quad shuffles.  full/empty mbarriers per stage; no __syncthreads in the loop.
//   * Work is cut on the device: all 16-token tiles of all sequences form one stream that is divided into
//     equal pieces, one per CTA (one CTA per SM), so the SMs finish together whatever the length
//     distribution.  A piece that spans several sequences emits one split per sequence.  The piece length is
//     raised when needed so that no sequence gets more than num_splits splits.  Splits a sequence does not
//     use get LSE = -inf.
// Every mbarrier wait is bounded; on expiry the CTA sets the device status word and drains.
#include "kernels.h"

#include <algorithm>
#include <atomic>
#include <string.h>
#include <type_traits>

namespace fck {

namespace {

constexpr int kTok = 16;  // tokens per tile

std::atomic<int64_t> g_stages{0};          // 0 = as many as fit
std::atomic<int64_t> g_ctas_per_sm_x100{100};  // grid.x = SMs * this / 100
std::atomic<int64_t> g_heads_per_cta{0};   // kv heads per CTA (8, 4, 2, 1); 0 = the most that divides nhead_k and fits 8 warps
std::atomic<int64_t> g_row_tiles{0};       // 16-row tiles of (token, group head) rows per pass (1, 2, 4); 0 = by the problem

struct DecodeDev {
    const void* q;
    float* o_acc;
    float* lse_acc;
    const int64_t* seqstart_q;
    const int64_t* seqstart_k;
    const int32_t* seqlen_k;
    const int32_t* block_table;
    const int64_t* cache_batch_idx;
    int* status;
    int batch, seqlen_q, seqlen_k_cap, hq, hkv, num_splits, total_q, bt_stride, page;
    int mask_type, wl, wr;
    const float* alibi;  // slopes (see SplitKVParams) or nullptr
    int alibi_rank;
    float scale;
    int stages;
    float scale_log2;
};

__device__ __forceinline__ int seq_len_k(const DecodeDev& p, int b) {
    if (p.seqlen_k) return p.seqlen_k[b];
    if (p.seqstart_k) return (int)(p.seqstart_k[b + 1] - p.seqstart_k[b]);
    return p.seqlen_k_cap;
}
__device__ __forceinline__ int seq_len_q(const DecodeDev& p, int b) {
    return p.seqstart_q ? (int)(p.seqstart_q[b + 1] - p.seqstart_q[b]) : p.seqlen_q;
}

// Shared schedule: for each sequence the first tile it uses (sliding windows skip leading tiles) and the
// prefix sum of tile counts.
struct Sched {
    int* prefix;  // [batch + 1]
    int* tile0;   // [batch]
    int total;    // prefix[batch]
    int piece;    // piece length in tiles (mode A) ; unused in mode B
    bool per_batch;  // mode B: one piece per sequence (num_splits == 1)
};

template <typename T, int D, int HK, int MT>
__global__ void __launch_bounds__((HK * MT + 1) * 32, 1)
splitkv_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const DecodeDev p) {
    constexpr int DH = D / 64;                       // 128-byte column groups per row
    constexpr int TILE_BYTES = kTok * HK * D * 2;    // one K (or V) tile
    constexpr int HEAD_BYTES = kTok * 128;           // one head of one column group
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.hq / p.hkv;
    const int stages = p.stages;

    // ---- carve shared memory -----------------------------------------------------------------
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
    uint8_t* tiles = smem_raw + pad;                                   // stages * 2 * TILE_BYTES
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)stages * 2 * TILE_BYTES);
    uint64_t* full_k = bars;
    uint64_t* full_v = bars + stages;
    uint64_t* empty = bars + 2 * stages;
    int* sm_prefix = reinterpret_cast<int*>(bars + 3 * stages);
    int* sm_tile0 = sm_prefix + p.batch + 1;
    volatile int* abort_flag = sm_tile0 + p.batch;
    int* sm_misc = const_cast<int*>(abort_flag) + 1;  // [0] = max tiles of any sequence

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_k[s], 1);
            mbar_init(&full_v[s], 1);
            mbar_init(&empty[s], HK * MT);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    // the kernel before this one in the stream (an append, the previous step's merge) has completed beyond this point;
    // the merge kernel that follows may take its place on the SMs as their CTAs retire
    pdl_launch_dependents();
    pdl_wait();
    // ---- schedule: tiles per sequence, prefix sum (warp 0) ---------------------------------------
    if (warp == 0) {
        int run = 0, mx = 0;
        for (int base = 0; base < p.batch; base += 32) {
            const int b = base + lane;
            int n = 0, t0 = 0;
            if (b < p.batch) {
                const int len = seq_len_k(p, b);
                if (len > 0) {
                    int first = 0;
                    if (p.mask_type != 0 && p.wl >= 0) {
                        const int shift = (p.mask_type == 2) ? len - seq_len_q(p, b) : 0;
                        first = max(0, min(len - 1, shift - p.wl));  // lowest key any row may see
                    }
                    t0 = first / kTok;
                    n = (len + kTok - 1) / kTok - t0;
                }
                sm_tile0[b] = t0;
            }
            int incl = n;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += y;
            }
            if (b < p.batch) sm_prefix[b] = run + incl - n;
            run += __shfl_sync(0xffffffffu, incl, 31);
            int m = n;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, off));
            mx = max(mx, m);
        }
        if (lane == 0) {
            sm_prefix[p.batch] = run;
            sm_misc[0] = mx;
        }
    }
    __syncthreads();

    Sched sc;
    sc.prefix = sm_prefix;
    sc.tile0 = sm_tile0;
    sc.total = sm_prefix[p.batch];
    sc.per_batch = (p.num_splits <= 1);
    {
        const int even = (sc.total + (int)gridDim.x - 1) / (int)gridDim.x;
        const int cap = sc.per_batch ? 0 : (sm_misc[0] + p.num_splits - 2) / (p.num_splits - 1);
        sc.piece = max(1, max(even, cap));
    }
    const int num_pieces = sc.per_batch ? p.batch : (sc.total + sc.piece - 1) / sc.piece;

    // ---- unused splits get LSE = -inf -------------------------------------------------------------
    if (p.lse_acc && blockIdx.y == 0 && blockIdx.z == 0) {
        for (int b = blockIdx.x; b < p.batch; b += gridDim.x) {
            const int n = sm_prefix[b + 1] - sm_prefix[b];
            int used;
            if (n == 0) used = 0;
            else if (sc.per_batch) used = 1;
            else used = (sm_prefix[b + 1] - 1) / sc.piece - sm_prefix[b] / sc.piece + 1;
            const int sq = seq_len_q(p, b);
            const int64_t q0 = p.seqstart_q ? p.seqstart_q[b] : 0;
            const int cnt = (p.num_splits - used) * sq * p.hq;
            for (int e = threadIdx.x; e < cnt; e += blockDim.x) {
                const int i = e % sq;
                const int s = used + (e / sq) % (p.num_splits - used);
                const int h = e / (sq * (p.num_splits - used));
                const int64_t idx = p.seqstart_q ? ((int64_t)h * p.num_splits + s) * p.total_q + q0 + i
                                                 : (((int64_t)b * p.hq + h) * p.num_splits + s) * p.seqlen_q + i;
                p.lse_acc[idx] = -INFINITY;
            }
        }
    }

    const int hgroup = blockIdx.z;  // kv heads [hgroup*HK, hgroup*HK + HK)

    if (warp == HK * MT) {
        // =========================== producer warp ===========================================
        if (lane == 0) {
            tma_prefetch_desc(&map_k);
            tma_prefetch_desc(&map_v);
        }
        uint32_t it = 0;
        for (int piece = blockIdx.x; piece < num_pieces; piece += gridDim.x) {
            int g_lo, g_hi, b;
            if (sc.per_batch) {
                b = piece;
                g_lo = sm_prefix[b];
                g_hi = sm_prefix[b + 1];
            } else {
                g_lo = piece * sc.piece;
                g_hi = min(sc.total, g_lo + sc.piece);
                int lo = 0, hi = p.batch - 1;  // largest b with prefix[b] <= g_lo
                while (lo < hi) {
                    const int mid = (lo + hi + 1) >> 1;
                    if (sm_prefix[mid] <= g_lo) lo = mid; else hi = mid - 1;
                }
                b = lo;
            }
            for (; b < p.batch && sm_prefix[b] < g_hi; ++b) {
                const int ta = max(g_lo, sm_prefix[b]) - sm_prefix[b];
                const int tb = min(g_hi, sm_prefix[b + 1]) - sm_prefix[b];
                if (tb <= ta) continue;
                // rows of this m-tile exist in this sequence?  (the consumers skip the same segments)
                if ((int)blockIdx.y * MT * 16 >= seq_len_q(p, b) * G) continue;
                const int64_t bphys = p.cache_batch_idx ? p.cache_batch_idx[b] : b;
                const int64_t kstart = p.seqstart_k ? p.seqstart_k[b] : 0;
                const int t0 = sm_tile0[b];
                // page ids for up to 32 tiles per round, loaded one round ahead
                auto load_entry = [&](int t, int& pg, int& tok) {
                    const int token = (t0 + t) * kTok;
                    if (p.block_table) {
                        pg = p.block_table[bphys * p.bt_stride + token / p.page];
                        tok = token % p.page;
                    } else if (p.seqstart_k) {
                        pg = 0;
                        tok = (int)kstart + token;
                    } else {
                        pg = (int)bphys;
                        tok = token;
                    }
                };
                int pg_next = 0, tok_next = 0;
                if (ta + lane < tb) load_entry(ta + lane, pg_next, tok_next);
                for (int base = ta; base < tb; base += 32) {
                    const int pg_cur = pg_next, tok_cur = tok_next;
                    if (base + 32 + lane < tb) load_entry(base + 32 + lane, pg_next, tok_next);
                    const int cnt = min(32, tb - base);
                    for (int j = 0; j < cnt; ++j) {
                        const int pg = __shfl_sync(0xffffffffu, pg_cur, j);
                        const int tok = __shfl_sync(0xffffffffu, tok_cur, j);
                        const int s = it % stages;
                        const uint32_t ph = (it / stages) & 1u;
                        bool ok = true;
                        if (lane == 0) {
                            ok = mbar_wait_bounded(&empty[s], ph ^ 1u, abort_flag, p.status, 1);
                            if (ok) {
                                uint8_t* kdst = tiles + (size_t)s * 2 * TILE_BYTES;
                                mbar_expect_tx(&full_k[s], TILE_BYTES);
                                tma_load_5d(kdst, &map_k, &full_k[s], 0, tok, hgroup * HK, 0, pg);
                                mbar_expect_tx(&full_v[s], TILE_BYTES);
                                tma_load_5d(kdst + TILE_BYTES, &map_v, &full_v[s], 0, tok, hgroup * HK, 0, pg);
                            }
                        }
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                        if (!ok) return;
                        ++it;
                    }
                }
            }
        }
        return;
    }

    // =============================== consumer warps =============================================
    // MT warps share one kv head: warp w works on head w / MT and on 16-row tile w % MT of the (token, group-head)
    // rows, so that up to 16*MT query rows per kv head are served by one pass over the K/V tiles in shared memory
    const int hw = warp / MT;
    const int kh = hgroup * HK + hw;
    const int mt = blockIdx.y * MT + warp % MT;
    const int quad = lane >> 2, qlane = lane & 3;
    const int lm = lane >> 3, lr = lane & 7;  // ldmatrix: matrix id / row within the 8x8 matrix
    uint32_t it = 0;

    for (int piece = blockIdx.x; piece < num_pieces; piece += gridDim.x) {
        int g_lo, g_hi, b;
        if (sc.per_batch) {
            b = piece;
            g_lo = sm_prefix[b];
            g_hi = sm_prefix[b + 1];
        } else {
            g_lo = piece * sc.piece;
            g_hi = min(sc.total, g_lo + sc.piece);
            int lo = 0, hi = p.batch - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (sm_prefix[mid] <= g_lo) lo = mid; else hi = mid - 1;
            }
            b = lo;
        }
        for (; b < p.batch && sm_prefix[b] < g_hi; ++b) {
            const int ta = max(g_lo, sm_prefix[b]) - sm_prefix[b];
            const int tb = min(g_hi, sm_prefix[b + 1]) - sm_prefix[b];
            if (tb <= ta) continue;
            const int sq = seq_len_q(p, b);
            const int rows = sq * G;
            if ((int)blockIdx.y * MT * 16 >= rows) continue;  // no row tile of this CTA exists here (the producer skips too)
            if (MT > 1 && mt * 16 >= rows) {
                // this warp's row tile does not exist in this sequence, but its partners use the tiles: keep the
                // stage accounting in step
                for (int t = ta; t < tb; ++t, ++it) {
                    const int s = it % stages;
                    const uint32_t ph = (it / stages) & 1u;
                    if (!mbar_wait_bounded(&full_k[s], ph, abort_flag, p.status, 2)) return;
                    if (!mbar_wait_bounded(&full_v[s], ph, abort_flag, p.status, 4)) return;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[s]);
                }
                continue;
            }
            const int len = seq_len_k(p, b);
            const int split = sc.per_batch ? 0 : piece - sm_prefix[b] / sc.piece;
            const int64_t q0 = p.seqstart_q ? p.seqstart_q[b] : (int64_t)b * p.seqlen_q;
            const int t0 = sm_tile0[b];

            // ---- Q fragments straight from global memory (row r = token*G + group head) ----
            const int r0 = mt * 16 + quad, r1 = r0 + 8;
            const bool v0 = r0 < rows, v1 = r1 < rows;
            const int i0 = r0 / G, i1 = r1 / G;
            const T* q0p = (const T*)p.q + ((q0 + i0) * p.hq + kh * G + (r0 - i0 * G)) * D;
            const T* q1p = (const T*)p.q + ((q0 + i1) * p.hq + kh * G + (r1 - i1 * G)) * D;
            uint32_t qa[D / 16][4];
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const int c = ks * 16 + qlane * 2;
                qa[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0p + c) : 0u;
                qa[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1p + c) : 0u;
                qa[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0p + c + 8) : 0u;
                qa[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1p + c + 8) : 0u;
            }
            // ALiBi: slope of the head of each of this thread's two rows, and the key its diagonal ends at
            float slope0 = 0.f, slope1 = 0.f;
            if (p.alibi) {
                const float* sl = p.alibi + (p.alibi_rank ? (int64_t)b * p.hq : 0) + kh * G;
                slope0 = v0 ? sl[r0 - i0 * G] : 0.f;
                slope1 = v1 ? sl[r1 - i1 * G] : 0.f;
            }
            // visible key range of the two rows of this thread
            int lo0, hi0, lo1, hi1;
            visible_range(i0, sq, len, p.mask_type, p.wl, p.wr, lo0, hi0);
            visible_range(i1, sq, len, p.mask_type, p.wl, p.wr, lo1, hi1);
            if (!v0) { lo0 = 0; hi0 = len - 1; }
            if (!v1) { lo1 = 0; hi1 = len - 1; }

            float o[D / 8][4];
#pragma unroll
            for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
            float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

            // tiles whose keys all lie at or before `mask_from` and inside the sequence need no masking
            int mask_from = len;  // first key index that some row may not see
            if (p.mask_type != 0) {
                const int shift = (p.mask_type == 2) ? len - sq : 0;
                if (p.wr >= 0) mask_from = min(mask_from, shift + p.wr + 1);
                if (p.wl >= 0) mask_from = 0;
            }
            bool failed = false;
            int tcur = ta;  // next tile of the segment
            // One or two 16-token tiles per step.  Two tiles share the row maxima, the O rescale and the shuffles, and
            // give the dependent mma chains twice the independent work; the steps of a segment are taken in pairs
            // while at least two tiles remain.
            auto step = [&](auto nt_tag) {
                constexpr int NT = decltype(nt_tag)::value;
                uint32_t kbase[NT], vbase[NT], ph[NT];
                int st[NT];
#pragma unroll
                for (int u = 0; u < NT; ++u) {
                    st[u] = (it + u) % stages;
                    ph[u] = ((it + u) / stages) & 1u;
                    kbase[u] = smem_u32(tiles + (size_t)st[u] * 2 * TILE_BYTES);
                    vbase[u] = kbase[u] + TILE_BYTES;
                }
                const int tok0 = (t0 + tcur) * kTok;
                // ---- S = Q K^T ----
                float sacc[2 * NT][4];
#pragma unroll
                for (int n = 0; n < 2 * NT; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
#pragma unroll
                for (int u = 0; u < NT; ++u) {
                    if (!mbar_wait_bounded(&full_k[st[u]], ph[u], abort_flag, p.status, 2)) { failed = true; return; }
                }
                {
                    const int key = (lm >> 1) * 8 + lr;  // token row this lane addresses
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        const int dh = ks / 4;
                        const int c = 2 * (ks % 4) + (lm & 1);
#pragma unroll
                        for (int u = 0; u < NT; ++u) {
                            uint32_t bfr[4];
                            ldmatrix_x4(bfr, kbase[u] + (dh * HK + hw) * HEAD_BYTES + key * 128 + ((c ^ (key & 7)) << 4));
                            mma_16816<T>(sacc[2 * u], qa[ks], bfr[0], bfr[1]);
                            mma_16816<T>(sacc[2 * u + 1], qa[ks], bfr[2], bfr[3]);
                        }
                    }
                }
                // ---- scale, mask, online softmax (base 2) ----
                const bool need_mask = tok0 + NT * kTok > mask_from;
#pragma unroll
                for (int n = 0; n < 2 * NT; ++n) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float x = sacc[n][e] * p.scale_log2;
                        if (p.alibi) {  // (warp-uniform; the common instances pay one predicate per element)
                            const int key = tok0 + n * 8 + qlane * 2 + (e & 1);
                            const float dist = fabsf((float)(((e < 2) ? i0 : i1) + len - sq - key));
                            x = (sacc[n][e] * p.scale - ((e < 2) ? slope0 : slope1) * dist) * 1.4426950408889634f;
                        }
                        if (need_mask) {
                            const int key = tok0 + n * 8 + qlane * 2 + (e & 1);
                            const bool vis = (e < 2) ? (key >= lo0 && key <= hi0) : (key >= lo1 && key <= hi1);
                            if (!vis) x = -INFINITY;
                        }
                        sacc[n][e] = x;
                    }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int n = 0; n < 2 * NT; ++n) {
                    mx0 = fmaxf(mx0, fmaxf(sacc[n][0], sacc[n][1]));
                    mx1 = fmaxf(mx1, fmaxf(sacc[n][2], sacc[n][3]));
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
                const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0, ms1 = (mn1 == -INFINITY) ? 0.f : mn1;
                const float a0 = fast_exp2(m0 - ms0), a1 = fast_exp2(m1 - ms1);  // exp2(-inf) = 0
                m0 = mn0;
                m1 = mn1;
                float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
                for (int n = 0; n < 2 * NT; ++n) {
                    sacc[n][0] = fast_exp2(sacc[n][0] - ms0);
                    sacc[n][1] = fast_exp2(sacc[n][1] - ms0);
                    sacc[n][2] = fast_exp2(sacc[n][2] - ms1);
                    sacc[n][3] = fast_exp2(sacc[n][3] - ms1);
                    ps0 += sacc[n][0] + sacc[n][1];
                    ps1 += sacc[n][2] + sacc[n][3];
                }
                l0 = l0 * a0 + ps0;  // per-thread partial row sums; reduced over the quad at the end
                l1 = l1 * a1 + ps1;
                if (__any_sync(0xffffffffu, (a0 != 1.f) || (a1 != 1.f))) {
#pragma unroll
                    for (int n = 0; n < D / 8; ++n) {
                        o[n][0] *= a0;
                        o[n][1] *= a0;
                        o[n][2] *= a1;
                        o[n][3] *= a1;
                    }
                }
                // ---- O += P V ----
                // A tile that reaches past the end of its sequence holds, behind the end, whatever the cache had there (the
                // tail of the last page, or the unused part of a contiguous row).  Those keys have P = 0, but 0 times a NaN
                // or Inf in V is NaN, so their V rows are cleared in the fragments: this thread's B registers hold keys
                // 2*qlane, 2*qlane + 1 (registers 0 and 2) and the same + 8 (registers 1 and 3) of the 16-key tile.
                const bool v_tail = tok0 + NT * kTok > len;  // (warp-uniform)
#pragma unroll
                for (int u = 0; u < NT; ++u) {
                    uint32_t vm0 = 0xffffffffu, vm1 = 0xffffffffu;
                    if (v_tail) {
                        const int k0 = tok0 + u * kTok + qlane * 2;
                        vm0 = (k0 < len ? 0x0000ffffu : 0u) | (k0 + 1 < len ? 0xffff0000u : 0u);
                        vm1 = (k0 + 8 < len ? 0x0000ffffu : 0u) | (k0 + 9 < len ? 0xffff0000u : 0u);
                    }
                    uint32_t pa[4];
                    pa[0] = Elem<T>::pack2(sacc[2 * u][0], sacc[2 * u][1]);
                    pa[1] = Elem<T>::pack2(sacc[2 * u][2], sacc[2 * u][3]);
                    pa[2] = Elem<T>::pack2(sacc[2 * u + 1][0], sacc[2 * u + 1][1]);
                    pa[3] = Elem<T>::pack2(sacc[2 * u + 1][2], sacc[2 * u + 1][3]);
                    if (!mbar_wait_bounded(&full_v[st[u]], ph[u], abort_flag, p.status, 4)) { failed = true; return; }
                    const int key = (lm & 1) * 8 + lr;
#pragma unroll
                    for (int j = 0; j < D / 16; ++j) {
                        const int g = 2 * j + (lm >> 1);  // 16-byte column chunk of the V row
                        const int dh = g / 8, c = g % 8;
                        uint32_t bfr[4];
                        ldmatrix_x4_trans(bfr,
                                          vbase[u] + (dh * HK + hw) * HEAD_BYTES + key * 128 + ((c ^ (key & 7)) << 4));
                        if (v_tail) {
                            bfr[0] &= vm0;
                            bfr[1] &= vm1;
                            bfr[2] &= vm0;
                            bfr[3] &= vm1;
                        }
                        mma_16816<T>(o[2 * j], pa, bfr[0], bfr[1]);
                        mma_16816<T>(o[2 * j + 1], pa, bfr[2], bfr[3]);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[st[u]]);
                }
                it += NT;
                tcur += NT;
            };
            while (tcur < tb && !failed) {
                if (tb - tcur >= 2) step(std::integral_constant<int, 2>{});
                else step(std::integral_constant<int, 1>{});
            }
            if (failed) return;

            // ---- epilogue: normalise within the split, store fp32 partials ----
            l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
            l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
            const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
            const float kLn2 = 0.6931471805599453f;
            auto acc_index = [&](int r, int i) -> int64_t {  // index of (b, head(r), split, token i)
                const int h = kh * G + (r - i * G);
                return p.seqstart_q ? ((int64_t)h * p.num_splits + split) * p.total_q + (q0 + i)
                                    : (((int64_t)b * p.hq + h) * p.num_splits + split) * p.seqlen_q + i;
            };
            if (v0) {
                const int64_t idx = acc_index(r0, i0);
                float* dst = p.o_acc + idx * D + qlane * 2;
#pragma unroll
                for (int n = 0; n < D / 8; ++n)
                    *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][0] * inv0, o[n][1] * inv0);
                if (p.lse_acc && qlane == 0) p.lse_acc[idx] = l0 > 0.f ? (m0 + log2f(l0)) * kLn2 : -INFINITY;
            }
            if (v1) {
                const int64_t idx = acc_index(r1, i1);
                float* dst = p.o_acc + idx * D + qlane * 2;
#pragma unroll
                for (int n = 0; n < D / 8; ++n)
                    *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2] * inv1, o[n][3] * inv1);
                if (p.lse_acc && qlane == 0) p.lse_acc[idx] = l1 > 0.f ? (m1 + log2f(l1)) * kLn2 : -INFINITY;
            }
        }
    }
}

// Builds the 5-D tensor map of one K or V pool.
int make_pool_map(CUtensorMap* map, const void* base, int dtype, int64_t pages, int64_t page_tokens, int64_t hkv,
                  int D, int HK) {
    PFN_encodeTiled enc = get_encode_tiled();
    FCK_REQUIRE(enc != nullptr, FLASHCK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[5] = {64, (cuuint64_t)page_tokens, (cuuint64_t)hkv, (cuuint64_t)(D / 64), (cuuint64_t)pages};
    const cuuint64_t strides[4] = {(cuuint64_t)(hkv * D * 2), (cuuint64_t)(D * 2), 128,
                                   (cuuint64_t)(page_tokens * hkv * D * 2)};
    const cuuint32_t box[5] = {64, (cuuint32_t)kTok, (cuuint32_t)HK, (cuuint32_t)(D / 64), 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUtensorMapDataType dt =
        dtype == FLASHCK_DTYPE_BFLOAT16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult r = enc(map, dt, 5, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FCK_REQUIRE(r == CUDA_SUCCESS, FLASHCK_ERR_CUDA,
                "cuTensorMapEncodeTiled failed (%d) for pool pages=%lld page=%lld hkv=%lld hdim=%d", (int)r,
                (long long)pages, (long long)page_tokens, (long long)hkv, D);
    return FLASHCK_OK;
}

template <typename T, int D, int HK, int MT>
int launch_inst(const SplitKVParams& p, const DecodeDev& dev_in, cudaStream_t stream) {
    DecodeDev dev = dev_in;
    constexpr int TILE_BYTES = kTok * HK * D * 2;
    const size_t fixed = 1024 /*alignment slack*/ + (size_t)(2 * p.batch + 1 + 4) * sizeof(int);
    const size_t budget = 227 * 1024;
    int stages = (int)((budget - fixed) / (2 * TILE_BYTES + 3 * sizeof(uint64_t)));
    stages = stages > 12 ? 12 : stages;
    const int64_t want = g_stages.load();
    if (want > 0 && want < stages) stages = (int)want;
    FCK_REQUIRE(stages >= 2, FLASHCK_ERR_UNSUPPORTED, "splitkv: batch %lld leaves no room for two K/V stages",
                (long long)p.batch);
    dev.stages = stages;
    const size_t smem = fixed + (size_t)stages * (2 * TILE_BYTES + 3 * sizeof(uint64_t));

    // tensor maps: paged pool, batch-strided cache, or one packed buffer
    int64_t pages, page_tokens;
    if (p.block_table) { pages = p.num_pages; page_tokens = p.page; }
    else if (p.seqstart_k) { pages = 1; page_tokens = p.seqlen_k_cap; /* packed buffer: total key tokens */ }
    else { pages = p.num_pages > 0 ? p.num_pages : (int64_t)1 << 30; page_tokens = p.seqlen_k_cap; }
    CUtensorMap mk, mv;
    int rc = make_pool_map(&mk, p.k, p.dtype, pages, page_tokens, p.hkv, D, HK);
    if (rc) return rc;
    rc = make_pool_map(&mv, p.v, p.dtype, pages, page_tokens, p.hkv, D, HK);
    if (rc) return rc;

    auto kern = splitkv_decode_kernel<T, D, HK, MT>;
    static thread_local int configured_device = -1;  // per instantiation
    int devid = 0;
    FCK_CUDA(cudaGetDevice(&devid));
    if (configured_device != devid) {
        FCK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget));
        configured_device = devid;
    }
    const int G = (int)(p.hq / p.hkv);
    const int mtiles = (int)((p.max_seqlen_q * G + 16 * MT - 1) / (16 * MT));
    int gx = (int)((int64_t)sm_count() * g_ctas_per_sm_x100.load() / 100);
    if (gx < 1) gx = 1;
    dim3 grid(gx, mtiles, (unsigned)(p.hkv / HK));
    FCK_CUDA(launch_dependent(kern, grid, dim3((HK * MT + 1) * 32), smem, stream, mk, mv, dev));
    return FLASHCK_OK;
}

// Instance choice: MT = row tiles (of 16 query rows x group heads) served per pass, HK = kv heads per CTA;
// HK * MT <= 8 consumer warps.  Decode (one token, group <= 16) uses MT = 1 and all 8 heads of a page per CTA;
// multi-token queries (append + decode) trade heads per CTA for row tiles so that K/V still cross HBM once.
template <typename T, int D, int MT>
int launch_hk(const SplitKVParams& p, const DecodeDev& dev, cudaStream_t stream) {
    const int64_t hkv = p.hkv;
    constexpr int kMaxHK = 8 / MT;
    // the instance parameter caps the heads per CTA; a value the problem cannot take (not a divisor of nhead_k, more
    // than 8 warps with this many row tiles) falls through to the next smaller one
    const int64_t want = g_heads_per_cta.load();
    const int cap = want > 0 ? (int)want : 8;
    if constexpr (kMaxHK >= 8) {
        if (cap >= 8 && hkv % 8 == 0) return launch_inst<T, D, 8, MT>(p, dev, stream);
    }
    if constexpr (kMaxHK >= 4) {
        if (cap >= 4 && hkv % 4 == 0) return launch_inst<T, D, 4, MT>(p, dev, stream);
    }
    if constexpr (kMaxHK >= 2) {
        if (cap >= 2 && hkv % 2 == 0) return launch_inst<T, D, 2, MT>(p, dev, stream);
    }
    return launch_inst<T, D, 1, MT>(p, dev, stream);
}

template <typename T, int D>
int launch_mt(const SplitKVParams& p, const DecodeDev& dev, cudaStream_t stream) {
    const int64_t row_tiles = (p.max_seqlen_q * (p.hq / p.hkv) + 15) / 16;
    const int64_t want = g_row_tiles.load();  // more row tiles per pass than the problem has rows only idle warps
    const int64_t mt = want > 0 ? std::min<int64_t>(want, row_tiles <= 1 ? 1 : (row_tiles <= 2 ? 2 : 4)) : row_tiles;
    if (mt <= 1) return launch_hk<T, D, 1>(p, dev, stream);
    if (mt <= 2) return launch_hk<T, D, 2>(p, dev, stream);
    return launch_hk<T, D, 4>(p, dev, stream);
}

}  // namespace

int splitkv_set_param(const char* key, int64_t value) {
    if (!strcmp(key, "stages")) { g_stages = value; return FLASHCK_OK; }
    if (!strcmp(key, "ctas_per_sm_x100")) { g_ctas_per_sm_x100 = value; return FLASHCK_OK; }
    if (!strcmp(key, "heads_per_cta")) {
        if (value != 0 && value != 1 && value != 2 && value != 4 && value != 8) return FLASHCK_ERR_INVALID_ARGUMENT;
        g_heads_per_cta = value;
        return FLASHCK_OK;
    }
    if (!strcmp(key, "row_tiles")) {
        if (value != 0 && value != 1 && value != 2 && value != 4) return FLASHCK_ERR_INVALID_ARGUMENT;
        g_row_tiles = value;
        return FLASHCK_OK;
    }
    return FLASHCK_ERR_INVALID_ARGUMENT;
}
int splitkv_get_param(const char* key, int64_t* value) {
    if (!strcmp(key, "stages")) { *value = g_stages; return FLASHCK_OK; }
    if (!strcmp(key, "ctas_per_sm_x100")) { *value = g_ctas_per_sm_x100; return FLASHCK_OK; }
    if (!strcmp(key, "heads_per_cta")) { *value = g_heads_per_cta; return FLASHCK_OK; }
    if (!strcmp(key, "row_tiles")) { *value = g_row_tiles; return FLASHCK_OK; }
    return FLASHCK_ERR_INVALID_ARGUMENT;
}

int launch_splitkv_decode(const SplitKVParams& p, cudaStream_t stream) {
    FCK_REQUIRE(p.d == p.dv && (p.d == 64 || p.d == 128), FLASHCK_ERR_UNSUPPORTED,
                "splitkv: hdim_q == hdim_v in {64,128} required (got %lld/%lld)", (long long)p.d, (long long)p.dv);
    FCK_REQUIRE(p.batch >= 1 && p.batch <= 8192, FLASHCK_ERR_UNSUPPORTED, "splitkv: batch must be in [1,8192]");
    FCK_REQUIRE(!p.block_table || (p.page > 0 && p.page % kTok == 0), FLASHCK_ERR_UNSUPPORTED,
                "splitkv: page_block_size must be a positive multiple of %d (got %lld)", kTok, (long long)p.page);
    FCK_REQUIRE(!p.block_table || p.seqlen_k, FLASHCK_ERR_INVALID_ARGUMENT,
                "splitkv: paged K/V needs per-sequence lengths (k_seq_len_ptr)");
    int* status = device_status_ptr();
    if (!status) return FLASHCK_ERR_CUDA;
    DecodeDev dev;
    dev.q = p.q; dev.o_acc = p.o_acc; dev.lse_acc = p.lse_acc;
    dev.seqstart_q = p.seqstart_q; dev.seqstart_k = p.seqstart_k; dev.seqlen_k = p.seqlen_k;
    dev.block_table = p.block_table; dev.cache_batch_idx = p.cache_batch_idx; dev.status = status;
    dev.batch = (int)p.batch; dev.seqlen_q = (int)p.seqlen_q; dev.seqlen_k_cap = (int)p.seqlen_k_cap;
    dev.hq = (int)p.hq; dev.hkv = (int)p.hkv; dev.num_splits = (int)p.num_splits; dev.total_q = (int)p.total_q;
    dev.bt_stride = (int)p.bt_stride; dev.page = (int)p.page;
    dev.mask_type = p.mask_type;
    dev.wl = (int)(p.wl < 0 ? -1 : (p.wl > 0x3fffffff ? 0x3fffffff : p.wl));
    dev.wr = (int)(p.wr < 0 ? -1 : (p.wr > 0x3fffffff ? 0x3fffffff : p.wr));
    dev.stages = 0;
    dev.scale_log2 = p.scale * 1.4426950408889634f;
    dev.alibi = p.alibi_slopes; dev.alibi_rank = p.alibi_rank; dev.scale = p.scale;
    if (p.dtype == FLASHCK_DTYPE_BFLOAT16)
        return p.d == 128 ? launch_mt<__nv_bfloat16, 128>(p, dev, stream) : launch_mt<__nv_bfloat16, 64>(p, dev, stream);
    return p.d == 128 ? launch_mt<__half, 128>(p, dev, stream) : launch_mt<__half, 64>(p, dev, stream);
}

}  // namespace fck
