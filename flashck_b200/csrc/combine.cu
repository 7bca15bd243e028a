// Split-KV combine: O = sum_s w_s * O_s / sum_s w_s with w_s = exp(LSE_s - max_s LSE_s);
// LSE = max + log(sum).  The default strides are those of the reference's combine arguments
// (attention_kernels/fmha_fwd_split_kv_combine/fmha_fwd_split_kv_combine_jinja.h:125-140): lse_acc
// [bs,hq,S,rows], o_acc [bs,hq,S,rows,dv].  The strided form also reads partials gathered from several GPUs
// ([rank][...] layouts) and can leave the result in fp32, which is what a rank contributes to such a gather.
// One warp per (batch, head, row); HBM-bound on o_acc (read once) -- a few MB, so launch latency dominates.
#include "kernels.h"

namespace fck {

namespace {

template <typename T> struct Out4;
template <> struct Out4<__half> {
    static __device__ __forceinline__ void store(__half* p, float4 v) {
        uint2 pk = make_uint2(Elem<__half>::pack2(v.x, v.y), Elem<__half>::pack2(v.z, v.w));
        *reinterpret_cast<uint2*>(p) = pk;
    }
};
template <> struct Out4<__nv_bfloat16> {
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        uint2 pk = make_uint2(Elem<__nv_bfloat16>::pack2(v.x, v.y), Elem<__nv_bfloat16>::pack2(v.z, v.w));
        *reinterpret_cast<uint2*>(p) = pk;
    }
};
template <> struct Out4<float> {
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};

struct CombineDev {
    const float* lse_acc;
    const float* o_acc;
    void* o;
    float* lse;
    int64_t items;
    int rows, hq, dv, S;
    int64_t lb, lh, ls, lr;  // lse_acc strides: batch, head, split, row
    int64_t ob, oh, os, orr; // o_acc strides (elements): batch, head, split, row
};

template <typename T>
__global__ void __launch_bounds__(128) combine_kernel(const CombineDev p) {
    pdl_wait();  // the split kernel's partials are complete and visible (no-op after an ordinary launch)
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= p.items) return;
    // item = (b*hq + h)*rows + r
    const int r = (int)(item % p.rows);
    const int64_t bh = item / p.rows;
    const int h = (int)(bh % p.hq);
    const int64_t b = bh / p.hq;
    const int S = p.S;
    const float* lrow = p.lse_acc + b * p.lb + h * p.lh + r * p.lr;
    const float ninf = -INFINITY;

    float m = ninf;
    for (int s = lane; s < S; s += 32) m = fmaxf(m, lrow[s * p.ls]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));

    T* orow = (T*)p.o + ((b * p.rows + r) * p.hq + h) * (int64_t)p.dv;
    const int nvec = p.dv >> 2;  // float4 chunks
    if (m == ninf) {             // no split saw a key: O = 0, LSE = -inf
        for (int c = lane; c < nvec; c += 32) Out4<T>::store(orow + 4 * c, make_float4(0.f, 0.f, 0.f, 0.f));
        if (p.lse && lane == 0) p.lse[item] = ninf;
        return;
    }
    float sum = 0.f;
    for (int s = lane; s < S; s += 32) {
        const float ls = lrow[s * p.ls];
        sum += (ls == ninf) ? 0.f : expf(ls - m);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float inv = 1.f / sum;

    float4 acc[2];
    acc[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    acc[1] = acc[0];
    const float* obase = p.o_acc + b * p.ob + h * p.oh + r * p.orr;
    const bool c0 = lane < nvec, c1 = lane + 32 < nvec;
    // Lane s of a group of 32 splits holds that split's weight, so the row loop below has no load on its way to the
    // next address: four splits' rows are fetched together.  A weight of zero marks an empty split (LSE = -inf),
    // whose o_acc slot is never read -- it may hold anything.
    for (int s0 = 0; s0 < S; s0 += 32) {
        float wl = 0.f;
        if (s0 + lane < S) {
            const float ls = lrow[(s0 + lane) * p.ls];
            wl = (ls == ninf) ? 0.f : expf(ls - m) * inv;
        }
        const int cnt = min(32, S - s0);
        for (int j0 = 0; j0 < cnt; j0 += 4) {
            float w[4];
            float4 x[4][2];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                w[u] = __shfl_sync(0xffffffffu, wl, (j0 + u) & 31);
                if (j0 + u >= cnt) w[u] = 0.f;
                const float4* src = reinterpret_cast<const float4*>(obase + (int64_t)(s0 + j0 + u) * p.os);
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
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int c = lane + 32 * j;
        if (c < nvec) Out4<T>::store(orow + 4 * c, acc[j]);
    }
    if (p.lse && lane == 0) p.lse[item] = m + logf(sum);
}

}  // namespace

int launch_combine(const CombineParams& p, cudaStream_t stream) {
    FCK_REQUIRE(p.dv % 4 == 0 && p.dv <= 256, FLASHCK_ERR_UNSUPPORTED,
                "combine: v_head_dim must be a multiple of 4 and <= 256 (got %lld)", (long long)p.dv);
    FCK_REQUIRE(p.num_splits >= 1, FLASHCK_ERR_INVALID_ARGUMENT, "combine: num_splits must be >= 1");
    FCK_REQUIRE(p.dtype == FLASHCK_DTYPE_BFLOAT16 || p.dtype == FLASHCK_DTYPE_FLOAT16 || p.dtype == FLASHCK_DTYPE_FLOAT32,
                FLASHCK_ERR_UNSUPPORTED, "combine: output dtype must be 3 (float16), 4 (bfloat16) or 7 (float32)");
    CombineDev d;
    d.lse_acc = p.lse_acc; d.o_acc = p.o_acc; d.o = p.o; d.lse = p.lse;
    d.items = p.bs * p.hq * p.rows;
    d.rows = (int)p.rows; d.hq = (int)p.hq; d.dv = (int)p.dv; d.S = (int)p.num_splits;
    if (p.strided) {
        d.lb = p.lse_strides[0]; d.lh = p.lse_strides[1]; d.ls = p.lse_strides[2]; d.lr = p.lse_strides[3];
        d.ob = p.o_strides[0]; d.oh = p.o_strides[1]; d.os = p.o_strides[2]; d.orr = p.o_strides[3];
        FCK_REQUIRE(d.ob % 4 == 0 && d.oh % 4 == 0 && d.os % 4 == 0 && d.orr % 4 == 0, FLASHCK_ERR_INVALID_ARGUMENT,
                    "combine: o_acc strides must be multiples of 4 elements");
    } else {
        d.lr = 1; d.ls = p.rows; d.lh = p.num_splits * p.rows; d.lb = p.hq * d.lh;
        d.orr = p.dv; d.os = p.rows * p.dv; d.oh = p.num_splits * d.os; d.ob = p.hq * d.oh;
    }
    if (d.items == 0) return FLASHCK_OK;
    const int warps = 4;
    const unsigned grid = (unsigned)((d.items + warps - 1) / warps);
    const dim3 g(grid), b(warps * 32);
    if (p.dtype == FLASHCK_DTYPE_BFLOAT16) FCK_CUDA(launch_dependent(combine_kernel<__nv_bfloat16>, g, b, 0, stream, d));
    else if (p.dtype == FLASHCK_DTYPE_FLOAT16) FCK_CUDA(launch_dependent(combine_kernel<__half>, g, b, 0, stream, d));
    else FCK_CUDA(launch_dependent(combine_kernel<float>, g, b, 0, stream, d));
    return FLASHCK_OK;
}

}  // namespace fck
