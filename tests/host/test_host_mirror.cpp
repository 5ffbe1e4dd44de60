// Validation tests of the C++ host mirror, transcribed from the reference's own config tests
// (singe-kernel/src/cuda/attention/tests.rs:88-109, 322-400) plus the matmul span checks
// (singe-kernel/src/cuda/matmul.rs:2977-3020).  Needs no GPU: every case is refused or accepted on the host.
#include <cstdio>
#include <limits>

#include "../../singe_b200/host/singe_kernel.hpp"

using namespace singe_kernel;

static int failures = 0;
#define CHECK(cond)                                                   \
    do {                                                              \
        if (!(cond)) {                                                \
            std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); \
            ++failures;                                               \
        }                                                             \
    } while (0)

int main() {
    {   // test_paged_kv_decode_attention_validation_accepts_exact_lengths / rejects_short_block_table
        PagedKvDecodeAttentionConfig config;
        CHECK(PagedKvDecodeAttentionConfig::contiguous(2, 4, 2, 8, 3, 5, 4, 0.5f, config) == Error::Ok);
        CHECK(config.validate_lengths(64, 64, 240, 240, 2, 8) == Error::Ok);
        CHECK(config.validate_lengths(64, 64, 240, 240, 2, 7) == Error::LengthTooShort);
        CHECK(config.validate_lengths(63, 64, 240, 240, 2, 8) == Error::LengthTooShort);
        CHECK(config.validate_lengths(80, 80, 300, 300, 5, 9) == Error::Ok);  // storage may be longer
        // test_paged_kv_decode_attention_validation_rejects_invalid_head_mapping
        CHECK(PagedKvDecodeAttentionConfig::contiguous(2, 3, 2, 8, 3, 5, 4, 0.5f, config) == Error::InvalidLength);
        CHECK(PagedKvDecodeAttentionConfig::contiguous(2, 4, 2, 8, 0, 5, 4, 0.5f, config) == Error::InvalidLength);
        CHECK(PagedKvDecodeAttentionConfig::contiguous(2, 4, 2, 8, 3, 5, 4, std::numeric_limits<float>::infinity(),
                                                       config) == Error::InvalidLength);
        CHECK(PagedKvDecodeAttentionConfig::contiguous(size_t(1) << 31, 4, 2, 8, 3, 5, 4, 0.5f, config) ==
              Error::LengthExceedsI32);
    }
    {   // paged prefill: accepts exact lengths, rejects short lse and a bad head mapping
        PagedKvPrefillAttentionConfig config;
        CHECK(PagedKvPrefillAttentionConfig::contiguous(2, 7, 4, 2, 8, 3, 5, 4, true, 0.5f, config) == Error::Ok);
        CHECK(config.validate_lengths(224, 28, 224, 240, 240, 2, 2, 2, 8) == Error::Ok);
        CHECK(config.validate_lengths(224, 27, 224, 240, 240, 2, 2, 2, 8) == Error::LengthTooShort);
        CHECK(PagedKvPrefillAttentionConfig::contiguous(2, 7, 3, 2, 8, 3, 5, 4, true, 0.5f, config) ==
              Error::InvalidLength);
    }
    {   // ragged prefill
        RaggedKvPrefillAttentionConfig config;
        CHECK(RaggedKvPrefillAttentionConfig::contiguous(2, 7, 8, 4, 2, 8, true, 0.5f, config) == Error::Ok);
        CHECK(config.validate_lengths(224, 28, 224, 128, 128, 2, 2, 2) == Error::Ok);
        CHECK(config.validate_lengths(224, 28, 224, 127, 128, 2, 2, 2) == Error::LengthTooShort);
        CHECK(RaggedKvPrefillAttentionConfig::contiguous(2, 7, 8, 3, 2, 8, true, 0.5f, config) == Error::InvalidLength);
    }
    {   // test_splitk_reduce_validation_accepts_padded_strides / rejects_short_lse
        SplitKReduceConfig config;
        CHECK(SplitKReduceConfig::contiguous(2, 4, 3, 8, config) == Error::Ok);
        CHECK(config.validate_lengths(64, 192, 24) == Error::Ok);
        CHECK(config.validate_lengths(64, 192, 23) == Error::LengthTooShort);
        config.attn_batch_stride = 104;
        config.attn_head_stride = 25;
        config.lse_batch_stride = 16;
        config.output_batch_stride = 40;
        CHECK(config.validate_lengths(72, 208, 32) == Error::Ok);
    }
    {   // matmul: the linear-layer constructor, strides below the extent, short operands
        MatmulConfig config = MatmulConfig::row_major_transposed_rhs(3, 5, 4);
        CHECK(config.lhs_row_stride == 4 && config.rhs_row_stride == 4 && config.output_row_stride == 5);
        CHECK(config.validate_lengths(15, 12, 20) == Error::Ok);
        CHECK(config.validate_lengths(14, 12, 20) == Error::LengthTooShort);
        CHECK(config.validate_lengths(15, 11, 20) == Error::LengthTooShort);
        config.rhs_row_stride = 3;
        CHECK(config.validate_lengths(15, 12, 20) == Error::InvalidLength);
        config = MatmulConfig::row_major_transposed_rhs(0, 5, 4);
        CHECK(config.validate_lengths(0, 0, 20) == Error::InvalidLength);
    }
    {   // operators validate on the host before they touch the library: a short output never reaches a launch
        PagedKvDecodeAttentionConfig config;
        CHECK(PagedKvDecodeAttentionConfig::contiguous(2, 4, 2, 8, 3, 5, 4, 0.5f, config) == Error::Ok);
        DeviceSlice<void> out{nullptr, 63};
        DeviceSlice<const void> q{nullptr, 64}, kc{nullptr, 240}, vc{nullptr, 240};
        DeviceSlice<const int32_t> lens{nullptr, 2};
        DeviceSlice<const uint32_t> table{nullptr, 8};
        CHECK(cuda::attention::paged_kv_decode_attention_bf16(nullptr, out, q, kc, vc, lens, table, config) ==
              Error::LengthTooShort);
        out.len = 64;  // lengths fine, pointers null: the library refuses with NullPointer, still before any launch
        CHECK(cuda::attention::paged_kv_decode_attention_bf16(nullptr, out, q, kc, vc, lens, table, config) ==
              Error::NullPointer);
    }
    if (failures == 0) std::printf("host mirror ok\n");
    return failures == 0 ? 0 : 1;
}
