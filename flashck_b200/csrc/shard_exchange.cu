// Sequence-sharded decode: merge of the local splits, exchange of the per-rank partials over NVLink and the final
// merge, in one kernel.
//
// The reference is single-GPU; its combine (attention_kernels/fmha_fwd_split_kv_combine/
// fmha_fwd_split_kv_combine_jinja.h:125-140) merges the splits of one GPU.  When the KV sequence of a request is
// sharded over several GPUs the same LSE-weighted merge runs twice -- over this rank's splits, then over the ranks --
// with an all-gather of (O_r fp32, LSE_r) in between.  Done with library calls that is merge kernel -> collective ->
// merge kernel, three launches whose fixed cost (tens of microseconds) does not shrink with the number of GPUs while
// the split-KV kernel in front of them does.  Here one CTA per (batch, head, row)
//   A. merges this rank's splits in registers (same arithmetic as combine.cu),
//   B. stores the fp32 partial into the exchange buffer of every rank with plain 16-byte stores to peer memory.  Every
//      8 bytes carry 4 bytes of data and a 4-byte flag (the call's epoch), so data and flag arrive together and no
//      fence or separate signal is needed (the "LL" scheme of NCCL's low-latency protocol),
//   C. reads the partials of all ranks out of its own buffer, polling each 16-byte line until both flags show the
//      epoch, and merges them into O (element type) and LSE.
// The polls are bounded (about a second of SM clocks): on expiry the warp ORs a code into the device status word and
// leaves without writing its row, so a rank that never launches cannot hang its peers' GPUs.
// No TMA, no multicast, no multimem: ordinary st.global / ld.global on addresses that cudaIpcOpenMemHandle mapped.
//
// Buffer of one rank: [header 256 B | parity 0: world x items rows | parity 1: the same]; a row is (dv + 2) * 8 bytes
// (dv values and the LSE as (value, flag) pairs, padded to 16 bytes).  Consecutive calls alternate between the two
// halves: a rank can be at most one call ahead of its slowest peer (it needs that peer's partial of the current call to
// finish), so what it writes for the next call never lands in rows a peer is still reading.  The epoch lives in the
// header (device memory) and is advanced by the last CTA of each launch, which keeps the launch parameters constant
// from call to call (the whole decode step can sit in a CUDA graph).
//
// With fewer GPUs than ranks (tests) the same kernel plays several ranks in one cooperative launch: blockIdx.y is the
// local rank, all buffers are local, and co-residency of the CTAs -- which wait on one another -- is guaranteed by the
// launch mode.  Separate launches that wait on one another are never run on one GPU.
#include <string.h>

#include "kernels.h"

namespace fck {

namespace {

constexpr int kMaxRanks = 8;
constexpr int kHeaderBytes = 256;
constexpr int kWarps = 8;
constexpr int kMaxSplitsPerThread = 4;
constexpr int kMaxSplits = kMaxSplitsPerThread * kWarps * 32;  // 1024, the bound of FmhaFwdSplitKV

struct ShardHeader {
    uint32_t counter;  // calls completed on this rank; the running call's epoch is counter + 1
    uint32_t done;     // CTAs of the running call that have finished
};

struct ShardDev {
    const float* lse_acc[kMaxRanks];  // per local rank: [batch, hq, S, rows]
    const float* o_acc[kMaxRanks];    // per local rank: [batch, hq, S, rows, dv]
    void* o[kMaxRanks];               // per local rank: [batch, rows, hq, dv] in the element type
    float* lse[kMaxRanks];            // per local rank: [batch, hq, rows] or nullptr
    uint8_t* buf[kMaxRanks];          // exchange buffer of every rank of the group (peer-mapped or local)
    int* status;
    int64_t items;
    int rows, hq, dv, S;
    int first_rank, world;
    long long wait_cycles;
};

__device__ __forceinline__ uint4 ld_volatile_v4(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_volatile_v4(uint8_t* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// Polls one 16-byte line (value, flag, value, flag) until both flags equal `flag`; false when the time is up.
__device__ __forceinline__ bool ll_wait(const uint8_t* p, uint32_t flag, long long t0, long long limit, float& a, float& b) {
    while (true) {
        const uint4 v = ld_volatile_v4(p);
        if (v.y == flag && v.w == flag) {
            a = __uint_as_float(v.x);
            b = __uint_as_float(v.z);
            return true;
        }
        if (clock64() - t0 > limit) return false;
        __nanosleep(40);
    }
}

template <typename T> struct Store4;
template <> struct Store4<__half> {
    static __device__ __forceinline__ void store(__half* p, float4 v) {
        *reinterpret_cast<uint2*>(p) = make_uint2(Elem<__half>::pack2(v.x, v.y), Elem<__half>::pack2(v.z, v.w));
    }
};
template <> struct Store4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        *reinterpret_cast<uint2*>(p) = make_uint2(Elem<__nv_bfloat16>::pack2(v.x, v.y), Elem<__nv_bfloat16>::pack2(v.z, v.w));
    }
};
template <> struct Store4<float> {
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};

// One CTA of kWarps warps per (batch, head, row): the warps share the splits of the local merge (step A is a chain of
// dependent memory round trips; a single warp per row needs about twenty of them for 75 splits), their sums meet in
// shared memory, each warp stores the partial to its share of the peers (step B) and warp 0 merges the ranks (step C).
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) shard_exchange_kernel(const ShardDev p) {
    __shared__ float4 part[kWarps][64];  // per warp: its share of sum_s w_s * O_s, dv <= 256 floats
    __shared__ float wsm[kMaxSplits];    // exp(LSE_s - max) of every split
    __shared__ float red[2 * kWarps];
    pdl_wait();  // the split-KV kernel's partials (and the previous step's header) are complete and visible
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lr = blockIdx.y;               // local rank played by this CTA
    const int me = p.first_rank + lr;        // its rank in the group
    const int W = p.world;
    ShardHeader* hdr = reinterpret_cast<ShardHeader*>(p.buf[me]);
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(&hdr->counter) + 1u;
    const int64_t item = blockIdx.x;  // = (b*hq + h)*rows + r
    const int64_t row_bytes = (int64_t)(p.dv + 2) * 8;
    const int64_t half_bytes = (int64_t)W * p.items * row_bytes;  // one parity half of a buffer
    const int64_t parity_off = kHeaderBytes + (int64_t)(epoch & 1u) * half_bytes;
    const float ninf = -INFINITY;
    const int r = (int)(item % p.rows);
    const int64_t bh = item / p.rows;
    const int h = (int)(bh % p.hq);
    const int64_t b = bh / p.hq;
    const int S = p.S, nvec = p.dv >> 2;
    const bool c0 = lane < nvec, c1 = lane + 32 < nvec;

    // ---- A. merge of this rank's splits.  The weights of all splits go to shared memory first (one round trip for the
    //         LSE values, read once per thread), then warp w takes splits w, w + kWarps, ... four at a time ----
    const float* lrow = p.lse_acc[lr] + (bh * S) * p.rows + r;                    // stride rows per split
    const float* obase = p.o_acc[lr] + ((bh * S) * p.rows + r) * (int64_t)p.dv;   // stride rows*dv per split
    float lv[kMaxSplitsPerThread];
    float m = ninf;
#pragma unroll
    for (int i = 0; i < kMaxSplitsPerThread; ++i) {
        const int sidx = (int)threadIdx.x + i * kWarps * 32;
        lv[i] = sidx < S ? lrow[(int64_t)sidx * p.rows] : ninf;
        m = fmaxf(m, lv[i]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w2 = 1; w2 < kWarps; ++w2) m = fmaxf(m, red[w2]);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxSplitsPerThread; ++i) {
        const int sidx = (int)threadIdx.x + i * kWarps * 32;
        const float e = (lv[i] == ninf) ? 0.f : expf(lv[i] - m);  // (m == -inf only if every lv is)
        if (sidx < S) wsm[sidx] = e;
        sum += e;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane == 0) red[kWarps + warp] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < kWarps; ++w2) sum += red[kWarps + w2];
    float4 acc[2];
    acc[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    acc[1] = acc[0];
    float lse_local = ninf;
    if (m != ninf) {
        const float inv = 1.f / sum;
        lse_local = m + logf(sum);
        const int64_t os = (int64_t)p.rows * p.dv;
        for (int s0 = warp; s0 < S; s0 += 4 * kWarps) {
            float w[4];
            float4 x[4][2];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int sidx = s0 + u * kWarps;
                w[u] = sidx < S ? wsm[sidx] * inv : 0.f;
                const float4* src = reinterpret_cast<const float4*>(obase + (int64_t)sidx * os);
                // a weight of zero marks an empty split, whose o_acc slot is never read -- it may hold anything
                x[u][0] = (w[u] != 0.f && c0) ? src[lane] : make_float4(0.f, 0.f, 0.f, 0.f);
                x[u][1] = (w[u] != 0.f && c1) ? src[lane + 32] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    acc[j].x += w[u] * x[u][j].x;
                    acc[j].y += w[u] * x[u][j].y;
                    acc[j].z += w[u] * x[u][j].z;
                    acc[j].w += w[u] * x[u][j].w;
                }
            }
        }
    }
    part[warp][lane] = acc[0];
    part[warp][lane + 32] = acc[1];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        float4 t = part[0][lane + 32 * j];
#pragma unroll
        for (int w2 = 1; w2 < kWarps; ++w2) {
            const float4 u = part[w2][lane + 32 * j];
            t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        acc[j] = t;
    }

    // ---- B. this rank's partial into every rank's buffer (own buffer included), the peers shared among the warps,
    //         starting with the next rank ----
    const int64_t my_row = parity_off + ((int64_t)me * p.items + item) * row_bytes;
    for (int k = 1 + warp; k <= W; k += kWarps) {
        uint8_t* dst = p.buf[(me + k) % W] + my_row;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c = lane + 32 * j;
            if (c < nvec) {
                st_volatile_v4(dst + (int64_t)c * 32, make_uint4(__float_as_uint(acc[j].x), epoch, __float_as_uint(acc[j].y), epoch));
                st_volatile_v4(dst + (int64_t)c * 32 + 16, make_uint4(__float_as_uint(acc[j].z), epoch, __float_as_uint(acc[j].w), epoch));
            }
        }
        if (lane == 0) st_volatile_v4(dst + (int64_t)p.dv * 8, make_uint4(__float_as_uint(lse_local), epoch, 0u, epoch));
    }

    // ---- C. (warp 0) the partials of all ranks from this rank's own buffer, then the merge over ranks ----
    if (warp == 0) {
        const long long t0 = clock64();
        const uint8_t* mine = p.buf[me] + parity_off + item * row_bytes;  // + rank * items * row_bytes
        const int64_t rank_stride = p.items * row_bytes;
        float lse_r = ninf, dummy;
        bool ok = true;
        if (lane < W) ok = ll_wait(mine + lane * rank_stride + (int64_t)p.dv * 8, epoch, t0, p.wait_cycles, lse_r, dummy);
        ok = __all_sync(0xffffffffu, ok);
        float mg = lse_r;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, off));
        float wr = (lse_r == ninf) ? 0.f : expf(lse_r - mg);  // (mg == -inf: every weight is 0)
        float sg = wr;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sg += __shfl_xor_sync(0xffffffffu, sg, off);
        if (mg != ninf) wr /= sg;
        float4 out[2];
        out[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        out[1] = out[0];
        for (int rk = 0; ok && rk < W; ++rk) {
            const float w = __shfl_sync(0xffffffffu, wr, rk);
            if (w == 0.f) continue;  // an empty shard: its row is never read
            const uint8_t* src = mine + rk * rank_stride;
            bool got = true;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = lane + 32 * j;
                if (c < nvec) {
                    float a, bb, cc, d;
                    got = got && ll_wait(src + (int64_t)c * 32, epoch, t0, p.wait_cycles, a, bb) &&
                          ll_wait(src + (int64_t)c * 32 + 16, epoch, t0, p.wait_cycles, cc, d);
                    if (got) {
                        out[j].x += w * a;
                        out[j].y += w * bb;
                        out[j].z += w * cc;
                        out[j].w += w * d;
                    }
                }
            }
            ok = __all_sync(0xffffffffu, got);
        }
        if (!ok) {
            if (lane == 0) atomicOr(p.status, 0x2000);  // a peer's partial did not arrive in time
        } else {
            T* orow = (T*)p.o[lr] + ((b * p.rows + r) * p.hq + h) * (int64_t)p.dv;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = lane + 32 * j;
                if (c < nvec) Store4<T>::store(orow + 4 * c, out[j]);
            }
            if (p.lse[lr] && lane == 0) p.lse[lr][item] = (mg == ninf) ? ninf : mg + logf(sg);
        }
    }

    // ---- the last CTA of this rank's launch advances the epoch ----
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t t = atomicAdd(&hdr->done, 1u);
        if (t == gridDim.x - 1) {
            hdr->done = 0u;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(&hdr->counter) = epoch;
        }
    }
}

}  // namespace
}  // namespace fck

using namespace fck;

extern "C" {

int64_t FlashckShardExchangeBytes(int64_t batch, int64_t rows, int64_t q_num_heads, int64_t v_head_dim, int world) {
    if (batch < 0 || rows < 0 || q_num_heads < 0 || v_head_dim < 0 || world < 1) return -1;
    return kHeaderBytes + 2 * (int64_t)world * batch * q_num_heads * rows * (v_head_dim + 2) * 8;
}

int FmhaFwdSplitKVShardedCombine(void* const* lse_acc_ptrs, void* const* o_acc_ptrs, void* const* o_ptrs, void* const* lse_ptrs,
                                 void* const* exchange_bufs, int first_rank, int local_ranks, int world, int64_t batch,
                                 int64_t rows, int64_t hq, int64_t dv, int64_t num_splits, int out_dtype, void* stream) {
    FCK_REQUIRE(lse_acc_ptrs && o_acc_ptrs && o_ptrs && exchange_bufs, FLASHCK_ERR_INVALID_ARGUMENT,
                "FmhaFwdSplitKVShardedCombine: null pointer-array argument");
    FCK_REQUIRE(world >= 1 && world <= kMaxRanks && local_ranks >= 1 && first_rank >= 0 && first_rank + local_ranks <= world,
                FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdSplitKVShardedCombine: ranks [%d, %d) of a group of %d (at most %d)",
                first_rank, first_rank + local_ranks, world, kMaxRanks);
    FCK_REQUIRE(batch >= 0 && rows >= 0 && hq > 0 && dv > 0 && num_splits >= 1 && num_splits <= kMaxSplits,
                FLASHCK_ERR_INVALID_ARGUMENT, "FmhaFwdSplitKVShardedCombine: bad sizes (num_splits must be in [1,%d])", kMaxSplits);
    FCK_REQUIRE(dv % 4 == 0 && dv <= 256, FLASHCK_ERR_UNSUPPORTED,
                "FmhaFwdSplitKVShardedCombine: v_head_dim must be a multiple of 4 and <= 256 (got %lld)", (long long)dv);
    FCK_REQUIRE(out_dtype == FLASHCK_DTYPE_BFLOAT16 || out_dtype == FLASHCK_DTYPE_FLOAT16 || out_dtype == FLASHCK_DTYPE_FLOAT32,
                FLASHCK_ERR_UNSUPPORTED, "FmhaFwdSplitKVShardedCombine: output dtype must be 3, 4 or 7");
    int* status = device_status_ptr();
    if (!status) return FLASHCK_ERR_CUDA;
    ShardDev d{};
    for (int i = 0; i < local_ranks; ++i) {
        FCK_REQUIRE(lse_acc_ptrs[i] && o_acc_ptrs[i] && o_ptrs[i], FLASHCK_ERR_INVALID_ARGUMENT,
                    "FmhaFwdSplitKVShardedCombine: null workspace or output of local rank %d", i);
        d.lse_acc[i] = (const float*)lse_acc_ptrs[i];
        d.o_acc[i] = (const float*)o_acc_ptrs[i];
        d.o[i] = o_ptrs[i];
        d.lse[i] = lse_ptrs ? (float*)lse_ptrs[i] : nullptr;
    }
    for (int i = 0; i < world; ++i) {
        FCK_REQUIRE(exchange_bufs[i] != nullptr, FLASHCK_ERR_INVALID_ARGUMENT,
                    "FmhaFwdSplitKVShardedCombine: no exchange buffer for rank %d", i);
        d.buf[i] = (uint8_t*)exchange_bufs[i];
    }
    d.status = status;
    d.items = batch * hq * rows;
    d.rows = (int)rows; d.hq = (int)hq; d.dv = (int)dv; d.S = (int)num_splits;
    d.first_rank = first_rank; d.world = world;
    d.wait_cycles = kWaitLimitCycles;
    if (d.items == 0) return FLASHCK_OK;
    FCK_REQUIRE(d.items < (1ll << 31), FLASHCK_ERR_UNSUPPORTED, "FmhaFwdSplitKVShardedCombine: too many rows");
    const dim3 grid((unsigned)d.items, (unsigned)local_ranks);
    const dim3 block(kWarps * 32);
    void* kern = out_dtype == FLASHCK_DTYPE_BFLOAT16 ? (void*)shard_exchange_kernel<__nv_bfloat16>
                 : out_dtype == FLASHCK_DTYPE_FLOAT16 ? (void*)shard_exchange_kernel<__half>
                                                      : (void*)shard_exchange_kernel<float>;
    void* args[] = {(void*)&d};
    if (local_ranks > 1) {
        // several ranks in one launch wait on one another: only a cooperative launch guarantees that all of their CTAs
        // are resident together (it fails instead of deadlocking when they do not fit)
        FCK_CUDA(cudaLaunchCooperativeKernel(kern, grid, block, args, 0, (cudaStream_t)stream));
    } else {
        // one rank per launch: the kernel may become resident under the tail of the split-KV kernel before it
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = use_pdl() ? 1 : 0;
        FCK_CUDA(cudaLaunchKernelExC(&cfg, kern, args));
    }
    return FLASHCK_OK;
}

// ---- exchange buffers: device memory that the other ranks' processes can map ----------------------------------------
int FlashckPeerBufferCreate(int64_t bytes, void** ptr_out, void* handle_out64) {
    FCK_REQUIRE(bytes > 0 && ptr_out && handle_out64, FLASHCK_ERR_INVALID_ARGUMENT, "FlashckPeerBufferCreate: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle crosses the C ABI as 64 bytes");
    void* ptr = nullptr;
    FCK_CUDA(cudaMalloc(&ptr, (size_t)bytes));
    cudaError_t e = cudaMemset(ptr, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) {
        cudaFree(ptr);
        return cuda_fail(e, "FlashckPeerBufferCreate");
    }
    memcpy(handle_out64, &h, sizeof(h));
    *ptr_out = ptr;
    return FLASHCK_OK;
}
int FlashckPeerBufferOpen(const void* handle64, void** ptr_out) {
    FCK_REQUIRE(handle64 && ptr_out, FLASHCK_ERR_INVALID_ARGUMENT, "FlashckPeerBufferOpen: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    FCK_CUDA(cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
    return FLASHCK_OK;
}
int FlashckPeerBufferClose(void* ptr) {
    if (ptr) FCK_CUDA(cudaIpcCloseMemHandle(ptr));
    return FLASHCK_OK;
}
int FlashckPeerBufferFree(void* ptr) {
    if (ptr) FCK_CUDA(cudaFree(ptr));
    return FLASHCK_OK;
}

}  // extern "C"
