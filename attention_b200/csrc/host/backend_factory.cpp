// BackendFactory: registry, capability probing and selection, on top of the C ABI.
// Follows the static API of the reference (src/api/backend_factory.hpp:40-115, .cpp:366-504, 647-720).
#include "api/backend_factory.hpp"

#include <algorithm>
#include <cctype>
#include <chrono>
#include <cstdio>
#include <sstream>

#include "ahpc.h"
#include "algorithms/flash_attention.hpp"
#include "algorithms/paged_attention.hpp"

namespace attention_hpc {

namespace {
const BackendType kAllTypes[] = {BackendType::CPU, BackendType::CUDA, BackendType::OPENCL, BackendType::OPENGL, BackendType::VULKAN};

BackendCapability probe_cuda() {
    BackendCapability cap;
    if (ahpc_device_count() <= 0) return cap;
    ahpc_device_info info;
    int dev = -1;
    for (int d = 0; d < 64 && dev < 0; ++d)
        if (ahpc_get_device_info(d, &info) == AHPC_SUCCESS && info.cc_major == 10) dev = d;
    if (dev < 0) return cap;
    cap.available = true;
    cap.version = std::string("CUDA runtime ") + std::to_string(info.runtime_version / 1000) + "." + std::to_string((info.runtime_version % 1000) / 10);
    cap.device_name = info.name;
    cap.memory_size = info.total_memory_bytes;
    cap.compute_capability_major = info.cc_major;
    cap.compute_capability_minor = info.cc_minor;
    cap.supported_data_types = {DataType::FLOAT32, DataType::FLOAT16, DataType::BFLOAT16};
    cap.supported_layouts = {MemoryLayout::ROW_MAJOR};
    cap.max_threads = info.max_threads_per_block;
    cap.max_shared_memory = info.max_shared_memory_per_block;
    cap.supports_mixed_precision = true;
    cap.supports_tensor_cores = true;
    return cap;
}
}  // namespace

BackendFactory& BackendFactory::getInstance() {
    static BackendFactory instance;
    return instance;
}

BackendFactory::BackendFactory() {
    priority_ = {BackendType::CUDA, BackendType::VULKAN, BackendType::OPENCL, BackendType::OPENGL, BackendType::CPU};
    capabilities_[static_cast<int>(BackendType::CUDA)] = probe_cuda();
    for (BackendType t : kAllTypes)
        if (t != BackendType::CUDA) capabilities_[static_cast<int>(t)] = BackendCapability{};   // not part of this product
    Entry cuda;
    cuda.name = "CUDA";
    cuda.flash_creator = [] { return std::unique_ptr<AttentionInterface>(new FlashAttention()); };
    cuda.paged_creator = [] { return std::unique_ptr<AttentionInterface>(new PagedAttention()); };
    entries_[static_cast<int>(BackendType::CUDA)] = std::move(cuda);
}

BackendType BackendFactory::resolve(BackendType type) const { return type == BackendType::AUTO ? default_backend_ : type; }

bool BackendFactory::available_locked(BackendType type) const {
    type = resolve(type);
    auto cap = capabilities_.find(static_cast<int>(type));
    auto ent = entries_.find(static_cast<int>(type));
    return cap != capabilities_.end() && cap->second.available && ent != entries_.end();
}

namespace {
enum class Kind { Generic, Flash, Paged };
}

static std::unique_ptr<AttentionInterface> create_impl(BackendFactory& f, BackendType type, Kind kind,
                                                       std::mutex& mu, const std::function<bool(BackendType)>& available,
                                                       const std::function<BackendFactory::BackendCreator(BackendType, Kind)>& pick) {
    BackendFactory::BackendCreator creator;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!available(type)) throw BackendException(type, "Backend not available");
        creator = pick(type, kind);
    }
    (void)f;
    if (!creator) throw BackendException(type, "No creator function registered");
    try {
        auto obj = creator();                      // runs outside the lock: creators may call back into the factory
        if (!obj) throw BackendException(type, "creator returned null");
        return obj;
    } catch (const BackendException&) {
        throw;
    } catch (const std::exception& e) {
        throw BackendException(type, std::string("Failed to create backend: ") + e.what());
    }
}

std::unique_ptr<AttentionInterface> BackendFactory::createBackend(BackendType type) { return createFlashAttention(type); }

std::unique_ptr<AttentionInterface> BackendFactory::createFlashAttention(BackendType type) {
    BackendFactory& f = getInstance();
    return create_impl(f, type, Kind::Flash, f.mutex_, [&f](BackendType t) { return f.available_locked(t); },
                       [&f](BackendType t, Kind) { return f.entries_[static_cast<int>(f.resolve(t))].flash_creator; });
}

std::unique_ptr<AttentionInterface> BackendFactory::createPagedAttention(BackendType type) {
    BackendFactory& f = getInstance();
    return create_impl(f, type, Kind::Paged, f.mutex_, [&f](BackendType t) { return f.available_locked(t); },
                       [&f](BackendType t, Kind) {
                           Entry& e = f.entries_[static_cast<int>(f.resolve(t))];
                           return e.paged_creator ? e.paged_creator : e.flash_creator;
                       });
}

bool BackendFactory::isBackendAvailable(BackendType type) {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    return f.available_locked(type);
}

std::vector<BackendType> BackendFactory::getAvailableBackends() {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    std::vector<BackendType> out;
    for (BackendType t : kAllTypes)
        if (f.available_locked(t)) out.push_back(t);
    return out;
}

BackendCapability BackendFactory::getBackendCapability(BackendType type) {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    auto it = f.capabilities_.find(static_cast<int>(f.resolve(type)));
    return it == f.capabilities_.end() ? BackendCapability{} : it->second;
}

int BackendFactory::scoreBackend(BackendType type, const AttentionParams& params, const BackendCapability& cap) {
    // Same weights as the reference (backend_factory.cpp:647-696): CUDA 1000, +200 tensor cores, +50 mixed precision.
    if (!cap.available) return -1;
    int score = type == BackendType::CUDA ? 1000 : type == BackendType::VULKAN ? 800 : type == BackendType::OPENCL ? 600
              : type == BackendType::OPENGL ? 400 : 100;
    if (cap.supports_tensor_cores) score += 200;
    if (cap.supports_mixed_precision) score += 50;
    const size_t work = params.batch_size * params.sequence_length * params.num_heads * params.head_dimension;
    if (work > (size_t(1) << 20) && type == BackendType::CUDA) score += 100;
    return score;
}

BackendType BackendFactory::selectBestBackend(const AttentionParams& params) {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    BackendType best = BackendType::CPU;
    int best_score = -1;
    for (BackendType t : kAllTypes) {
        if (!f.available_locked(t)) continue;
        const int s = scoreBackend(t, params, f.capabilities_[static_cast<int>(t)]);
        if (s > best_score) { best_score = s; best = t; }
    }
    return best;
}

BackendType BackendFactory::selectBestBackend(const std::vector<BackendType>& preferred_backends) {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    for (BackendType t : preferred_backends)
        if (f.available_locked(t)) return f.resolve(t);
    for (BackendType t : f.priority_)
        if (f.available_locked(t)) return t;
    return BackendType::CPU;
}

void BackendFactory::setBackendPriority(const std::vector<BackendType>& priority_order) {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    f.priority_ = priority_order;
}

std::vector<BackendType> BackendFactory::getBackendPriority() {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    return f.priority_;
}

void BackendFactory::registerBackend(BackendType type, const std::string& name, BackendCreator creator) {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    Entry& e = f.entries_[static_cast<int>(type)];
    e.name = name;
    e.flash_creator = creator;
    e.paged_creator = nullptr;            // a user backend serves both create* calls, as in the reference
    f.capabilities_[static_cast<int>(type)].available = true;
}

void BackendFactory::unregisterBackend(BackendType type) {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    f.entries_.erase(static_cast<int>(type));
    if (type != BackendType::CUDA) f.capabilities_[static_cast<int>(type)].available = false;
}

std::string BackendFactory::backendTypeToString(BackendType type) {
    switch (type) {
        case BackendType::CPU: return "CPU";
        case BackendType::CUDA: return "CUDA";
        case BackendType::OPENCL: return "OpenCL";
        case BackendType::OPENGL: return "OpenGL";
        case BackendType::VULKAN: return "Vulkan";
        case BackendType::AUTO: return "Auto";
    }
    return "Unknown";
}

BackendType BackendFactory::stringToBackendType(const std::string& type_str) {
    std::string s;
    for (char c : type_str) s.push_back(static_cast<char>(std::tolower(static_cast<unsigned char>(c))));
    if (s == "cpu") return BackendType::CPU;
    if (s == "cuda") return BackendType::CUDA;
    if (s == "opencl") return BackendType::OPENCL;
    if (s == "opengl") return BackendType::OPENGL;
    if (s == "vulkan") return BackendType::VULKAN;
    if (s == "auto") return BackendType::AUTO;
    throw std::invalid_argument("Unknown backend type: " + type_str);
}

std::vector<std::string> BackendFactory::getSupportedBackendNames() { return {"CPU", "CUDA", "OpenCL", "OpenGL", "Vulkan", "Auto"}; }

std::string BackendFactory::getSystemInfo() {
    std::ostringstream os;
    os << "attention_hpc on B200 (library " << ahpc_version() << ")\n";
    for (BackendType t : kAllTypes) {
        const BackendCapability cap = getBackendCapability(t);
        os << "  " << backendTypeToString(t) << ": " << (isBackendAvailable(t) ? "available" : "not available");
        if (cap.available && !cap.device_name.empty())
            os << " - " << cap.device_name << ", sm_" << cap.compute_capability_major << cap.compute_capability_minor << ", "
               << (cap.memory_size >> 20) << " MiB, " << cap.version;
        os << "\n";
    }
    return os.str();
}

void BackendFactory::printAvailableBackends() { std::fputs(getSystemInfo().c_str(), stdout); }

bool BackendFactory::validateBackendCompatibility(BackendType type, const AttentionParams& params) {
    if (!isBackendAvailable(type)) return false;
    if (params.batch_size == 0 || params.sequence_length == 0 || params.num_heads == 0 || params.head_dimension == 0) return false;
    if (params.head_dimension > 256) return false;
    const size_t kvh = params.key_value_heads == 0 ? params.num_heads : params.key_value_heads;
    return kvh == params.num_heads;        // grouped-query attention is not built yet
}

void BackendFactory::enableDebugMode(bool enable) {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    f.debug_mode_ = enable;
}
bool BackendFactory::isDebugModeEnabled() {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    return f.debug_mode_;
}
void BackendFactory::setDefaultBackend(BackendType type) {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    if (type != BackendType::AUTO) f.default_backend_ = type;
}
BackendType BackendFactory::getDefaultBackend() {
    BackendFactory& f = getInstance();
    std::lock_guard<std::mutex> lock(f.mutex_);
    return f.default_backend_;
}

namespace backend_utils {

double benchmarkBackend(BackendType type, const AttentionParams& params, int num_iterations) {
    auto backend = BackendFactory::createFlashAttention(type);
    backend->configure(params);
    const std::vector<size_t> dims = {params.batch_size, params.sequence_length, params.num_heads, params.head_dimension};
    const TensorShape shape(dims, DataType::FLOAT32);
    std::vector<float> q(shape.total_elements(), 0.01f), k(q), v(q), o(q.size());
    backend->forward(shape, q.data(), shape, k.data(), shape, v.data(), shape, o.data());   // warm-up
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < num_iterations; ++i) backend->forward(shape, q.data(), shape, k.data(), shape, v.data(), shape, o.data());
    const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    return ms / std::max(1, num_iterations);
}

std::vector<std::pair<BackendType, double>> benchmarkAllBackends(const AttentionParams& params, int num_iterations) {
    std::vector<std::pair<BackendType, double>> out;
    for (BackendType t : BackendFactory::getAvailableBackends()) out.emplace_back(t, benchmarkBackend(t, params, num_iterations));
    return out;
}

size_t estimateMemoryUsage(BackendType, const AttentionParams& p) {
    return ahpc_fa_workspace_bytes(AHPC_F32, p.batch_size, p.num_heads, p.sequence_length, p.sequence_length, p.head_dimension, 0);
}

BackendType recommendBackend(const AttentionParams& params, size_t available_memory) {
    const BackendType best = BackendFactory::selectBestBackend(params);
    if (available_memory && estimateMemoryUsage(best, params) > available_memory) return BackendType::CPU;
    return best;
}

bool checkDataTypeSupport(BackendType type, DataType data_type) {
    const BackendCapability cap = BackendFactory::getBackendCapability(type);
    return std::find(cap.supported_data_types.begin(), cap.supported_data_types.end(), data_type) != cap.supported_data_types.end();
}

bool checkMemoryLayoutSupport(BackendType type, MemoryLayout layout) {
    const BackendCapability cap = BackendFactory::getBackendCapability(type);
    return std::find(cap.supported_layouts.begin(), cap.supported_layouts.end(), layout) != cap.supported_layouts.end();
}

std::string getBackendVersion(BackendType type) { return type == BackendType::CUDA ? std::string(ahpc_version()) : std::string(); }

std::string getDriverVersion(BackendType type) {
    if (type != BackendType::CUDA) return {};
    ahpc_device_info info;
    if (ahpc_get_device_info(0, &info) != AHPC_SUCCESS) return {};
    return std::to_string(info.driver_version / 1000) + "." + std::to_string((info.driver_version % 1000) / 10);
}

}  // namespace backend_utils
}  // namespace attention_hpc
