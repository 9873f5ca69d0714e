// attention_hpc::FlashAttention on B200: the class the reference declares in
// src/algorithms/flash_attention.hpp:85-133 (public part), implemented on the C ABI of ahpc.h instead
// of AVX2 loops.  FlashAttentionConfig keeps the reference's fields (:17-36).
#pragma once

#include <string>
#include <utility>
#include <vector>

#include "api/attention_interface.hpp"

#pragma GCC visibility push(default)
namespace attention_hpc {

struct FlashAttentionConfig {
    size_t block_size_q = 64, block_size_k = 64, block_size_v = 64;   // hints: CUDA tiles are 128 x 128
    bool use_causal_mask = false;
    bool apply_dropout = false;           // not supported (forward inference path only)
    float dropout_probability = 0.0f;
    bool use_safe_softmax = true;         // always on: running-maximum softmax
    float softmax_scale = 0.0f;           // 0 = 1/sqrt(head_dim)
    bool prefetch_next_block = true;
    bool use_async_copy = false;
    size_t num_parallel_blocks = 1;
};

// How a {B,S,H,D} dims vector maps to memory (see AHPC_LAYOUT_* in ahpc.h).
enum class TensorMemoryOrder { BHSD = 0, BSHD = 1 };

class FlashAttention : public AttentionInterface {
public:
    FlashAttention();
    ~FlashAttention() override = default;

    void configure(const AttentionParams& params, const PerformanceConfig& perf_config = PerformanceConfig{}) override;
    void configure_flash_attention(const FlashAttentionConfig& flash_config);

    void forward(const TensorShape& query_shape, const void* query_data, const TensorShape& key_shape, const void* key_data,
                 const TensorShape& value_shape, const void* value_data, const TensorShape& output_shape, void* output_data,
                 const void* attention_mask = nullptr) override;

    // Training is outside this library: throws UNSUPPORTED_OPERATION.
    void backward(const TensorShape& grad_output_shape, const void* grad_output_data, const TensorShape& query_shape, const void* query_data,
                  const TensorShape& key_shape, const void* key_data, const TensorShape& value_shape, const void* value_data,
                  const TensorShape& grad_query_shape, void* grad_query_data, const TensorShape& grad_key_shape, void* grad_key_data,
                  const TensorShape& grad_value_shape, void* grad_value_data, const void* attention_mask = nullptr) override;

    size_t get_workspace_size(const AttentionParams& params) const override;
    void set_workspace(void* workspace_ptr, size_t workspace_size) override;

    bool supports_data_type(DataType data_type) const override;
    bool supports_memory_layout(MemoryLayout layout) const override;
    std::string get_backend_name() const override;
    std::string get_version() const override;

    void enable_profiling(bool enable) override;
    std::vector<std::pair<std::string, double>> get_profiling_results() const override;
    void reset_profiling() override;

    AttentionError validate_inputs(const TensorShape& query_shape, const TensorShape& key_shape, const TensorShape& value_shape,
                                   const TensorShape& output_shape, const AttentionParams& params) const override;

    // Additions (no counterpart in the reference): where and how to run.
    void set_device(int device) { device_ = device; }
    void set_stream(void* cuda_stream) { stream_ = cuda_stream; }
    void set_memory_order(TensorMemoryOrder order) { order_ = order; }
    // Name of the kernel the last forward() ran: "tcgen05" or "simt".
    std::string last_kernel() const { return last_kernel_; }

private:
    FlashAttentionConfig flash_config_;
    bool is_configured_ = false;
    size_t configured_elements_ = 0;
    std::vector<std::pair<std::string, double>> profiling_results_;
    int device_ = 0;
    void* stream_ = nullptr;
    TensorMemoryOrder order_ = TensorMemoryOrder::BHSD;
    std::string last_kernel_;
};

}  // namespace attention_hpc
#pragma GCC visibility pop
