// Split-KV combine: O = sum_s w_s * O_s / sum_s w_s with w_s = exp(LSE_s - max_s LSE_s);
// LSE = max + log(sum).  Buffer layouts follow the reference's combine arguments
// (attention_kernels/fmha_fwd_split_kv_combine/fmha_fwd_split_kv_combine_jinja.h:125-140).
// One warp per (batch, head, row); HBM-bound on o_acc (read once) -- a few MB, so launch latency dominates.
#include "kernels.h"

namespace fck {

template <typename T>
__global__ void __launch_bounds__(128)
combine_kernel(const float* __restrict__ lse_acc, const float* __restrict__ o_acc, T* __restrict__ o,
               float* __restrict__ lse, int64_t items, int rows, int hq, int dv, int S) {
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    // item = (b*hq + h)*rows + r
    const int r = (int)(item % rows);
    const int64_t bh = item / rows;
    const int h = (int)(bh % hq);
    const int64_t b = bh / hq;
    const float* lrow = lse_acc + bh * S * rows + r;  // stride rows between splits
    const float ninf = -INFINITY;

    float m = ninf;
    for (int s = lane; s < S; s += 32) m = fmaxf(m, lrow[(int64_t)s * rows]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));

    T* orow = o + ((b * rows + r) * hq + h) * (int64_t)dv;
    const int nvec = dv >> 2;  // float4 chunks
    if (m == ninf) {           // no split saw a key: O = 0, LSE = -inf
        for (int c = lane; c < nvec; c += 32) {
            uint2 z = make_uint2(0u, 0u);
            *reinterpret_cast<uint2*>(orow + 4 * c) = z;
        }
        if (lse && lane == 0) lse[item] = ninf;
        return;
    }
    float sum = 0.f;
    for (int s = lane; s < S; s += 32) {
        const float ls = lrow[(int64_t)s * rows];
        sum += (ls == ninf) ? 0.f : expf(ls - m);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float inv = 1.f / sum;

    float4 acc[2];
    acc[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    acc[1] = acc[0];
    const float* obase = o_acc + (bh * S * rows + r) * (int64_t)dv;
    for (int s = 0; s < S; ++s) {
        const float ls = lrow[(int64_t)s * rows];
        if (ls == ninf) continue;  // empty split: its o_acc slot is never read
        const float w = expf(ls - m) * inv;
        const float4* src = reinterpret_cast<const float4*>(obase + (int64_t)s * rows * dv);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c = lane + 32 * j;
            if (c < nvec) {
                const float4 x = src[c];
                acc[j].x += w * x.x;
                acc[j].y += w * x.y;
                acc[j].z += w * x.z;
                acc[j].w += w * x.w;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int c = lane + 32 * j;
        if (c < nvec) {
            uint2 pk;
            pk.x = Elem<T>::pack2(acc[j].x, acc[j].y);
            pk.y = Elem<T>::pack2(acc[j].z, acc[j].w);
            *reinterpret_cast<uint2*>(orow + 4 * c) = pk;
        }
    }
    if (lse && lane == 0) lse[item] = m + logf(sum);
}

int launch_combine(const CombineParams& p, cudaStream_t stream) {
    FCK_REQUIRE(p.dv % 4 == 0 && p.dv <= 256, FLASHCK_ERR_UNSUPPORTED,
                "combine: v_head_dim must be a multiple of 4 and <= 256 (got %lld)", (long long)p.dv);
    FCK_REQUIRE(p.num_splits >= 1, FLASHCK_ERR_INVALID_ARGUMENT, "combine: num_splits must be >= 1");
    const int64_t items = p.bs * p.hq * p.rows;
    if (items == 0) return FLASHCK_OK;
    const int warps = 4;
    const unsigned grid = (unsigned)((items + warps - 1) / warps);
    if (p.dtype == FLASHCK_DTYPE_BFLOAT16)
        combine_kernel<__nv_bfloat16><<<grid, warps * 32, 0, stream>>>(p.lse_acc, p.o_acc, (__nv_bfloat16*)p.o, p.lse,
                                                                      items, (int)p.rows, (int)p.hq, (int)p.dv,
                                                                      (int)p.num_splits);
    else
        combine_kernel<__half><<<grid, warps * 32, 0, stream>>>(p.lse_acc, p.o_acc, (__half*)p.o, p.lse, items,
                                                                (int)p.rows, (int)p.hq, (int)p.dv, (int)p.num_splits);
    FCK_CUDA(cudaGetLastError());
    return FLASHCK_OK;
}

}  // namespace fck
