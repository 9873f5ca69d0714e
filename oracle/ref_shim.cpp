// C entry points around the reference project's own attention checker, compiled from where
// the reference sources lie.  TEST INFRASTRUCTURE ONLY (built into oracle/_ref/, never linked
// into the product library).
//
// The two `#include`s below do not name files of this repository: oracle/build_oracle.py feeds
// them line ranges of the reference's tests/test_flash_attention.cpp through file descriptors:
//   REF_FN_SRC   = lines 30-97   (compute_reference_attention, a free function)
//   REF_MASK_SRC = lines 523-578 (the masked-attention loop nest of AttentionMaskTest, which
//                  reads `params`, `query_data`, `key_data`, `value_data`, `attention_mask`
//                  and writes `reference_output`)
// so the reference text is compiled unmodified and no copy of it is stored here.
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <limits>
#include <vector>

namespace ref_extract {
#include REF_FN_SRC
}  // namespace ref_extract

namespace {
struct ParamsView {
    size_t batch_size, sequence_length, num_heads, head_dimension;
    float scale_factor;
};
}  // namespace

extern "C" {

__attribute__((visibility("default")))
void ref_compute_reference_attention(const float* q, const float* k, const float* v, float* out,
                                     size_t batch, size_t heads, size_t seq, size_t dim,
                                     float scale, int causal) {
    const size_t n = batch * heads * seq * dim;
    std::vector<float> query(q, q + n), key(k, k + n), value(v, v + n), output(n, 0.0f);
    ref_extract::compute_reference_attention(query, key, value, output, batch, heads, seq, dim,
                                             scale, causal != 0);
    std::copy(output.begin(), output.end(), out);
}

__attribute__((visibility("default")))
void ref_masked_reference_attention(const float* q, const float* k, const float* v, const float* mask,
                                    float* out, size_t batch, size_t heads, size_t seq, size_t dim,
                                    float scale) {
    const size_t n = batch * heads * seq * dim;
    ParamsView params{batch, seq, heads, dim, scale};
    std::vector<float> query_data(q, q + n), key_data(k, k + n), value_data(v, v + n);
    std::vector<float> attention_mask(mask, mask + batch * seq * seq);
    std::vector<float> reference_output(n, 0.0f);
#include REF_MASK_SRC
    std::copy(reference_output.begin(), reference_output.end(), out);
}

}  // extern "C"
