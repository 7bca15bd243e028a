// Compile-and-link check of the C++ operator API against libflashck_b200.so; runs without a GPU because every
// call below is rejected by argument validation before any CUDA work.
#include <cstdio>
#include <cstring>
#include "flashck/fmha/fmha_fwd.h"

int main() {
    using namespace flashck;
    typedef unsigned short bf16;  // the reference's carrier type for bfloat16
    int failures = 0;
    try {
        AttentionLayer<bf16> layer(FmhaOperationMode::Batch, /*hq*/ 3, /*hkv*/ 2, 128, 128, 0.f, BiasEnum::NO_BIAS, {-1, 0},
                                   GenericAttentionMaskEnum::MASK_FROM_TOP_LEFT);
        bf16 dummy[8] = {0};
        layer(dummy, dummy, dummy, dummy, 1, 1, 1, 1);
        std::printf("expected a throw for 3 q heads over 2 kv heads\n");
        ++failures;
    } catch (const std::runtime_error& e) {
        if (!std::strstr(e.what(), "multiple")) { std::printf("unexpected message: %s\n", e.what()); ++failures; }
    }
    try {  // a layer built for ALiBi wants its slopes
        AttentionLayer<_Float16> layer(FmhaOperationMode::Batch, 2, 2, 64, 64, 1.f, BiasEnum::ALIBI);
        _Float16 dummy[8] = {0};
        layer(dummy, dummy, dummy, dummy, 1, 1, 1, 1);
        ++failures;
    } catch (const std::runtime_error&) {}
    try {  // the paged wrappers reach the library too (refused: 3 q heads over 2 kv heads)
        bf16 dummy[8] = {0};
        naive::fmha_batch_prefill<bf16>(dummy, dummy, dummy, dummy, nullptr, nullptr, nullptr, nullptr, nullptr, 1, 1, 3, 2,
                                        128, 128, 1, 1, 16);
        ++failures;
    } catch (const std::runtime_error& e) {
        if (!std::strstr(e.what(), "multiple")) { std::printf("unexpected message: %s\n", e.what()); ++failures; }
    }
    try {  // a bias kind without a bias buffer is refused before any CUDA work
        bf16 dummy[8] = {0};
        naive::fmha_fwd_bias<bf16>(dummy, dummy, dummy, nullptr, BiasEnum::ELEMENTWISE_BIAS, 0, 0.f, dummy, nullptr, nullptr,
                                   nullptr, nullptr, 1, 1, 1, 2, 2, 64, 64, 1);
        std::printf("expected a throw for bias_enum without a buffer\n");
        ++failures;
    } catch (const std::runtime_error& e) {
        if (!std::strstr(e.what(), "bias")) { std::printf("unexpected message: %s\n", e.what()); ++failures; }
    }
    static_assert(detail::dtype_code<bf16>() == 4 && detail::dtype_code<_Float16>() == 3, "dtype codes");
    std::printf(failures ? "FAIL\n" : "OK\n");
    return failures;
}
