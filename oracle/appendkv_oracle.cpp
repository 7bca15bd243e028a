// TEST INFRASTRUCTURE ONLY -- CPU oracle for fmha_fwd_appendkv (RoPE + KV-cache write).
//
// PARITY UNPINNED: the reference tree has no appendkv source, test or fixture; only
// the kind FmhaKind::FwdAppendKV and RopeEnum {NONE, INTERLEAVED, HALF_ROTATED}
// (core/profiling/attention/fmha_library.h:19,41,195-219), the tile schema
// (core/utils/json_config.h:281-312) and the cos/sin table generator
// (core/module/kernels/attention_kernels/fmha_common_jinja.h:192-227: tables
// [positions, rotary_dim/2] in the input dtype).  This file fixes the arithmetic
// contract the CUDA kernel must reproduce bit for bit:
//
//   x0,x1,c,s are widened to fp32; every product and sum is a separately rounded
//   fp32 operation (no fused multiply-add; compile with -ffp-contract=off);
//   y0 = rn(rn(x0*c) - rn(x1*s)), y1 = rn(rn(x0*s) + rn(x1*c)); results are rounded
//   to the storage dtype with round-to-nearest-even.
//   interleaved pairs (x[2i], x[2i+1]); half-rotated pairs (x[i], x[i + rotary_dim/2]);
//   elements at index >= rotary_dim are copied unchanged.
//
// Positions: new key j of batch b sits at pos = seqlen_k[b] + j; query i of batch b
// has pos = seqlen_k[b] + n_new[b] - sq[b] + i (queries are aligned to the end of
// the appended sequence).
#include <cstdint>
#include <cstring>

namespace {
constexpr int kBFloat16 = 4;
inline float bf16_to_f32(uint16_t h) {
    uint32_t u = static_cast<uint32_t>(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            u = sign | ((127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp - 15 + 127) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_f16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return static_cast<uint16_t>(sign | 0x7e00u);
    if (a >= 0x47800000u) return static_cast<uint16_t>(sign | 0x7c00u);
    if (a < 0x38800000u) {
        if (a < 0x33000000u) return static_cast<uint16_t>(sign);
        int e = static_cast<int>(a >> 23);
        uint32_t man = (a & 0x7fffffu) | 0x800000u;
        int shift = 126 - e;
        uint32_t half = man >> shift, rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1u))) ++half;
        return static_cast<uint16_t>(sign | half);
    }
    uint32_t r = a + 0xfffu + ((a >> 13) & 1u);
    r = (r >> 13) - (112u << 10);
    if (r >= 0x7c00u) r = 0x7c00u;
    return static_cast<uint16_t>(sign | r);
}
inline float widen(uint16_t h, int dt) { return dt == kBFloat16 ? bf16_to_f32(h) : f16_to_f32(h); }
inline uint16_t narrow(float f, int dt) { return dt == kBFloat16 ? f32_to_bf16(f) : f32_to_f16(f); }

// rope_type: 0 none, 1 interleaved, 2 half-rotated (RopeEnum).
void rope_row(const uint16_t* x, uint16_t* y, int64_t d, int64_t rotary_dim, int rope_type, const uint16_t* cosr,
              const uint16_t* sinr, int dt) {
    if (rope_type == 0) rotary_dim = 0;
    const int64_t half = rotary_dim / 2;
    for (int64_t i = 0; i < half; ++i) {
        const int64_t i0 = rope_type == 1 ? 2 * i : i;
        const int64_t i1 = rope_type == 1 ? 2 * i + 1 : i + half;
        const float x0 = widen(x[i0], dt), x1 = widen(x[i1], dt);
        const float c = widen(cosr[i], dt), s = widen(sinr[i], dt);
        volatile float a = x0 * c, b = x1 * s, e = x0 * s, f = x1 * c;  // volatile: keep each rounding
        const float y0 = a - b, y1 = e + f;
        y[i0] = narrow(y0, dt);
        y[i1] = narrow(y1, dt);
    }
    for (int64_t i = rotary_dim; i < d; ++i) y[i] = x[i];
}
}  // namespace

extern "C" {

// q: batch mode [b,sq,hq,d] or group mode [total_q,hq,d] (seqstart_q); rotated in place.
// knew/vnew: batch mode [b,n,hkv,d|dv] or group mode [total_new,hkv,*] (seqstart_knew).
// k_cache/v_cache: paged pool [pages,page,hkv,*] with block_table [b,bt_stride], or contiguous
// [b_cache,sk_cap,hkv,*] (block_table == nullptr).  seqlen_k: int32 [b] cached length before the append.
int oracle_fmha_fwd_appendkv(uint16_t* q, uint16_t* k_cache, const uint16_t* knew, uint16_t* v_cache,
                             const uint16_t* vnew, const int32_t* seqlen_k, const int64_t* seqstart_q,
                             const int64_t* seqstart_knew, const uint16_t* rotary_cos, const uint16_t* rotary_sin,
                             const int32_t* block_table, const int64_t* cache_batch_idx, int64_t batch,
                             int64_t seqlen_q, int64_t seqlen_k_cap, int64_t seqlen_knew, int64_t hq, int64_t hkv,
                             int64_t d, int64_t dv, int64_t rotary_dim, int rope_type, int64_t bt_stride,
                             int64_t page_block_size, int dtype) {
    const int64_t half = rotary_dim / 2;
    for (int64_t b = 0; b < batch; ++b) {
        const int64_t q0 = seqstart_q ? seqstart_q[b] : b * seqlen_q;
        const int64_t sq = seqstart_q ? seqstart_q[b + 1] - seqstart_q[b] : seqlen_q;
        const int64_t n0 = seqstart_knew ? seqstart_knew[b] : b * seqlen_knew;
        const int64_t n = seqstart_knew ? seqstart_knew[b + 1] - seqstart_knew[b] : seqlen_knew;
        const int64_t L = seqlen_k[b];
        const int64_t b_phys = cache_batch_idx ? cache_batch_idx[b] : b;
        for (int64_t j = 0; j < n; ++j) {
            const int64_t pos = L + j;
            int64_t row;
            if (block_table)
                row = static_cast<int64_t>(block_table[b_phys * bt_stride + pos / page_block_size]) * page_block_size +
                      pos % page_block_size;
            else
                row = b_phys * seqlen_k_cap + pos;
            for (int64_t h = 0; h < hkv; ++h) {
                rope_row(knew + ((n0 + j) * hkv + h) * d, k_cache + (row * hkv + h) * d, d, rotary_dim, rope_type,
                         rotary_cos + pos * half, rotary_sin + pos * half, dtype);
                std::memcpy(v_cache + (row * hkv + h) * dv, vnew + ((n0 + j) * hkv + h) * dv, dv * 2);
            }
        }
        if (rope_type != 0)
            for (int64_t i = 0; i < sq; ++i) {
                const int64_t pos = L + n - sq + i;
                for (int64_t h = 0; h < hq; ++h) {
                    uint16_t* qr = q + ((q0 + i) * hq + h) * d;
                    rope_row(qr, qr, d, rotary_dim, rope_type, rotary_cos + pos * half, rotary_sin + pos * half, dtype);
                }
            }
    }
    return 0;
}

}  // extern "C"
