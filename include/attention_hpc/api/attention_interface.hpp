// Public types and the abstract interface of the attention library.
//
// Same namespace, names, members and defaults as the reference's src/api/attention_interface.hpp
// (enums :16-26, PerformanceConfig :29-53, AttentionParams :56-71, AttentionError :74-83,
// AttentionException :86-95, TensorShape :98-128, AttentionInterface :131-215), so callers of the
// reference compile against this header unchanged.  There is exactly one TensorShape and one
// AttentionException in this tree.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <numeric>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#pragma GCC visibility push(default)
namespace attention_hpc {

template <typename T> class Tensor;   // declared by the reference; not needed by the hot paths

enum class DataType { FLOAT32, FLOAT16, BFLOAT16 };          // values 0,1,2 == AHPC_F32/F16/BF16
enum class MemoryLayout { ROW_MAJOR, COLUMN_MAJOR };

struct PerformanceConfig {
    size_t block_size_m = 64, block_size_n = 64, block_size_k = 64;   // hints: the CUDA tiles are fixed
    size_t num_threads = 0;                                           // 0 = auto
    bool use_memory_pool = true;
    bool enable_memory_reuse = true;
    bool use_fast_math = false;
    bool enable_mixed_precision = false;
    size_t shared_memory_size = 0;                                    // 0 = auto
    size_t max_workspace_size = size_t(1024) * 1024 * 1024;
    bool enable_profiling = false;
    bool enable_debug_checks = true;
};

struct AttentionParams {
    size_t batch_size;
    size_t sequence_length;
    size_t num_heads;
    size_t head_dimension;
    size_t key_value_heads = 0;         // 0 = num_heads
    float scale_factor = 0.0f;          // 0 = 1/sqrt(head_dimension)
    bool causal_mask = false;
    bool apply_rotary_embedding = false;
    size_t max_sequence_length = 0;     // paged attention
    size_t page_size = 16;              // paged attention
};

enum class AttentionError {
    SUCCESS = 0, INVALID_INPUT, INVALID_PARAMETERS, MEMORY_ALLOCATION_FAILED, COMPUTATION_FAILED,
    BACKEND_NOT_AVAILABLE, UNSUPPORTED_OPERATION, INTERNAL_ERROR
};

class AttentionException : public std::runtime_error {
public:
    explicit AttentionException(AttentionError error_code, const std::string& message)
        : std::runtime_error(message), error_code_(error_code) {}
    AttentionError error_code() const noexcept { return error_code_; }
private:
    AttentionError error_code_;
};

struct TensorShape {
    std::vector<size_t> dimensions;
    DataType data_type = DataType::FLOAT32;
    MemoryLayout layout = MemoryLayout::ROW_MAJOR;

    TensorShape() = default;
    TensorShape(std::vector<size_t> dims, DataType dtype = DataType::FLOAT32, MemoryLayout mem_layout = MemoryLayout::ROW_MAJOR)
        : dimensions(std::move(dims)), data_type(dtype), layout(mem_layout) {}

    size_t total_elements() const {
        return std::accumulate(dimensions.begin(), dimensions.end(), size_t(1), std::multiplies<size_t>());
    }
    size_t element_size() const { return data_type == DataType::FLOAT32 ? 4 : 2; }
    size_t total_bytes() const { return total_elements() * element_size(); }
};

class AttentionInterface {
public:
    virtual ~AttentionInterface() = default;

    virtual void configure(const AttentionParams& params, const PerformanceConfig& perf_config = PerformanceConfig{}) = 0;

    virtual void forward(const TensorShape& query_shape, const void* query_data,
                         const TensorShape& key_shape, const void* key_data,
                         const TensorShape& value_shape, const void* value_data,
                         const TensorShape& output_shape, void* output_data,
                         const void* attention_mask = nullptr) = 0;

    virtual void backward(const TensorShape& grad_output_shape, const void* grad_output_data,
                          const TensorShape& query_shape, const void* query_data,
                          const TensorShape& key_shape, const void* key_data,
                          const TensorShape& value_shape, const void* value_data,
                          const TensorShape& grad_query_shape, void* grad_query_data,
                          const TensorShape& grad_key_shape, void* grad_key_data,
                          const TensorShape& grad_value_shape, void* grad_value_data,
                          const void* attention_mask = nullptr) = 0;

    virtual size_t get_workspace_size(const AttentionParams& params) const = 0;
    virtual void set_workspace(void* workspace_ptr, size_t workspace_size) = 0;

    virtual bool supports_data_type(DataType data_type) const = 0;
    virtual bool supports_memory_layout(MemoryLayout layout) const = 0;
    virtual std::string get_backend_name() const = 0;
    virtual std::string get_version() const = 0;

    virtual void enable_profiling(bool enable) = 0;
    virtual std::vector<std::pair<std::string, double>> get_profiling_results() const = 0;
    virtual void reset_profiling() = 0;

    virtual AttentionError validate_inputs(const TensorShape& query_shape, const TensorShape& key_shape,
                                           const TensorShape& value_shape, const TensorShape& output_shape,
                                           const AttentionParams& params) const = 0;

    // validate_inputs against the configured parameters, then forward / backward
    void safe_forward(const TensorShape& query_shape, const void* query_data,
                      const TensorShape& key_shape, const void* key_data,
                      const TensorShape& value_shape, const void* value_data,
                      const TensorShape& output_shape, void* output_data,
                      const void* attention_mask = nullptr) {
        const AttentionError e = validate_inputs(query_shape, key_shape, value_shape, output_shape, current_params_);
        if (e != AttentionError::SUCCESS) throw AttentionException(e, "Input validation failed in forward pass");
        forward(query_shape, query_data, key_shape, key_data, value_shape, value_data, output_shape, output_data, attention_mask);
    }

    void safe_backward(const TensorShape& grad_output_shape, const void* grad_output_data,
                       const TensorShape& query_shape, const void* query_data,
                       const TensorShape& key_shape, const void* key_data,
                       const TensorShape& value_shape, const void* value_data,
                       const TensorShape& grad_query_shape, void* grad_query_data,
                       const TensorShape& grad_key_shape, void* grad_key_data,
                       const TensorShape& grad_value_shape, void* grad_value_data,
                       const void* attention_mask = nullptr) {
        const AttentionError e = validate_inputs(query_shape, key_shape, value_shape, grad_output_shape, current_params_);
        if (e != AttentionError::SUCCESS) throw AttentionException(e, "Input validation failed in backward pass");
        backward(grad_output_shape, grad_output_data, query_shape, query_data, key_shape, key_data, value_shape, value_data,
                 grad_query_shape, grad_query_data, grad_key_shape, grad_key_data, grad_value_shape, grad_value_data, attention_mask);
    }

protected:
    AttentionParams current_params_{};
    PerformanceConfig current_perf_config_{};
    void* workspace_ptr_ = nullptr;
    size_t workspace_size_ = 0;
    bool profiling_enabled_ = false;
};

inline std::string attention_error_to_string(AttentionError error) {
    static const char* const text[] = {"Success", "Invalid input tensor", "Invalid attention parameters", "Memory allocation failed",
                                       "Computation failed", "Backend not available", "Unsupported operation", "Internal error"};
    const int i = static_cast<int>(error);
    return (i >= 0 && i < 8) ? text[i] : "Unknown error";
}

}  // namespace attention_hpc
#pragma GCC visibility pop
