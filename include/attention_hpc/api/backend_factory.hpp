// Backend registry with the static API of the reference's src/api/backend_factory.hpp:40-115.
//
// Differences in behaviour, all deliberate:
//   - BackendType::CUDA (and AUTO) create working objects backed by the sm_100a kernels; the reference's
//     creators all throw "not implemented yet" (src/api/backend_factory.cpp:90-123).
//   - CPU, OPENCL, OPENGL and VULKAN report "not available": this product has no CPU fallback and no
//     OpenCL / graphics-API dispatch.
//   - No function calls another locking function while holding the registry mutex (the reference
//     re-enters a non-recursive mutex: backend_factory.cpp:66, 368/400, 499-500).
#pragma once

#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "attention_interface.hpp"

#pragma GCC visibility push(default)
namespace attention_hpc {

enum class BackendType { CPU, CUDA, OPENCL, OPENGL, VULKAN, AUTO };

struct BackendCapability {
    bool available = false;
    std::string version;
    std::string device_name;
    size_t memory_size = 0;
    int compute_capability_major = 0;
    int compute_capability_minor = 0;
    std::vector<DataType> supported_data_types;
    std::vector<MemoryLayout> supported_layouts;
    size_t max_threads = 0;
    size_t max_shared_memory = 0;
    bool supports_mixed_precision = false;
    bool supports_tensor_cores = false;
};

class BackendFactory {
public:
    static BackendFactory& getInstance();
    BackendFactory(const BackendFactory&) = delete;
    BackendFactory& operator=(const BackendFactory&) = delete;

    static std::unique_ptr<AttentionInterface> createBackend(BackendType type);
    static std::unique_ptr<AttentionInterface> createFlashAttention(BackendType type);
    static std::unique_ptr<AttentionInterface> createPagedAttention(BackendType type);

    static bool isBackendAvailable(BackendType type);
    static std::vector<BackendType> getAvailableBackends();
    static BackendCapability getBackendCapability(BackendType type);

    static BackendType selectBestBackend(const AttentionParams& params = AttentionParams{});
    static BackendType selectBestBackend(const std::vector<BackendType>& preferred_backends);

    static void setBackendPriority(const std::vector<BackendType>& priority_order);
    static std::vector<BackendType> getBackendPriority();

    using BackendCreator = std::function<std::unique_ptr<AttentionInterface>()>;
    static void registerBackend(BackendType type, const std::string& name, BackendCreator creator);
    static void unregisterBackend(BackendType type);

    static std::string backendTypeToString(BackendType type);
    static BackendType stringToBackendType(const std::string& type_str);
    static std::vector<std::string> getSupportedBackendNames();

    static void printAvailableBackends();
    static std::string getSystemInfo();
    static bool validateBackendCompatibility(BackendType type, const AttentionParams& params);

    static void enableDebugMode(bool enable = true);
    static bool isDebugModeEnabled();
    static void setDefaultBackend(BackendType type);
    static BackendType getDefaultBackend();

private:
    BackendFactory();
    ~BackendFactory() = default;

    struct Entry {
        std::string name;
        BackendCreator flash_creator, paged_creator;
    };
    BackendType resolve(BackendType type) const;          // AUTO -> default backend; call with mutex_ held
    bool available_locked(BackendType type) const;

    mutable std::mutex mutex_;
    std::unordered_map<int, Entry> entries_;
    std::unordered_map<int, BackendCapability> capabilities_;
    std::vector<BackendType> priority_;
    BackendType default_backend_ = BackendType::CUDA;
    bool debug_mode_ = false;

    static int scoreBackend(BackendType type, const AttentionParams& params, const BackendCapability& cap);
};

namespace backend_utils {
double benchmarkBackend(BackendType type, const AttentionParams& params, int num_iterations = 10);
std::vector<std::pair<BackendType, double>> benchmarkAllBackends(const AttentionParams& params, int num_iterations = 10);
size_t estimateMemoryUsage(BackendType type, const AttentionParams& params);
BackendType recommendBackend(const AttentionParams& params, size_t available_memory = 0);
bool checkDataTypeSupport(BackendType type, DataType data_type);
bool checkMemoryLayoutSupport(BackendType type, MemoryLayout layout);
std::string getBackendVersion(BackendType type);
std::string getDriverVersion(BackendType type);
}  // namespace backend_utils

class BackendException : public AttentionException {
public:
    explicit BackendException(BackendType backend_type, const std::string& message)
        : AttentionException(AttentionError::BACKEND_NOT_AVAILABLE,
                             "Backend " + BackendFactory::backendTypeToString(backend_type) + ": " + message),
          backend_type_(backend_type) {}
    BackendType backend_type() const noexcept { return backend_type_; }
private:
    BackendType backend_type_;
};

}  // namespace attention_hpc
#pragma GCC visibility pop
