// Library-wide host state: the launch stream of the calling thread, cached
// device properties, and the status / model-info entry points kept from the
// reference C ABI (engine/src/capi.cc:44-75) with the build target moved from
// sm_89 to sm_100a.
#include "g4_host.h"

#include "../../include/granite4_b200.h"

#include <atomic>
#include <cstdlib>

namespace g4 {

namespace {
thread_local cudaStream_t t_stream = cudaStreamPerThread;
constexpr int kMaxDevices = 64;
// Per-device caches, filled on first use by whichever host thread gets there first (several may,
// with the same value): relaxed atomics, no lock.
std::atomic<int> g_sm_count[kMaxDevices];  // 0 = not queried yet
std::atomic<unsigned int*> g_status_ptr[kMaxDevices];

// One word per device that loads the library; zero until a kernel reports.
__device__ unsigned int g_device_status;
}  // namespace

unsigned int* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  unsigned int* known = g_status_ptr[dev].load(std::memory_order_relaxed);
  if (known == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    known = static_cast<unsigned int*>(p);
    g_status_ptr[dev].store(known, std::memory_order_relaxed);
  }
  return known;
}

cudaStream_t current_stream() { return t_stream; }
void set_current_stream(cudaStream_t s) { t_stream = s ? s : cudaStreamPerThread; }

namespace {
thread_local bool t_amax_prezeroed = false;
}
bool amax_prezeroed() { return t_amax_prezeroed; }
void set_amax_prezeroed(bool on) { t_amax_prezeroed = on; }

bool pdl_enabled() {
  const char* v = std::getenv("G4_PDL");
  return !(v != nullptr && v[0] == '0');
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = g_sm_count[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

float l2_keep_fraction(double bytes) {
  static const int keep_mb = [] {
    const char* v = std::getenv("G4_L2_KEEP_MB");
    return (v != nullptr && *v != '\0') ? std::atoi(v) : 0;
  }();
  if (keep_mb <= 0 || bytes <= 0.0) return 0.0f;
  const double f = static_cast<double>(keep_mb) * 1048576.0 / bytes;
  return f >= 1.0 ? 1.0f : static_cast<float>(f);
}

}  // namespace g4

namespace {
constexpr int kArchMajor = 10, kArchMinor = 0;
const char kGpuTarget[] = "sm_100a";
const char* const kStatusTexts[] = {"ok", "unimplemented", "no-device", "unavailable"};
}  // namespace

extern "C" {

int granite4_b200_set_stream(void* cuda_stream) {
  g4::set_current_stream(static_cast<cudaStream_t>(cuda_stream));
  return 0;
}

int granite4_b200_device_status(unsigned int* out) {
  if (out == nullptr) return -1;
  unsigned int* p = g4::device_status_ptr();
  if (p == nullptr) return -1;
  // blocking copy: everything enqueued before it on this thread's stream and the
  // legacy stream has finished when it returns
  if (cudaMemcpy(out, p, sizeof *out, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return 0;
}

int granite4_b200_free(void* d_ptr) { return cudaFree(d_ptr) == cudaSuccess ? 0 : -1; }

void granite4_get_model_info(granite4_model_info* out) {
  if (out == nullptr) return;
  // engine/src/model_config.h:18-25
  out->model_id = "granite-4.2-8b";
  out->num_layers = 40;
  out->hidden_size = 4096;
  out->intermediate_size = 12800;
  out->num_attention_heads = 32;
  out->num_key_value_heads = 8;
  out->head_dim = 128;
  out->vocab_size = 100352;
  out->max_context_length = 131072;
  out->gpu_target = kGpuTarget;
}

void granite4_status(granite4_status_info* out) {
  if (out == nullptr) return;
  static thread_local char msg[96];
  msg[0] = '\0';
  int count = 0;
  const cudaError_t err = cudaGetDeviceCount(&count);
  out->cuda_device_present = (err == cudaSuccess && count > 0) ? 1 : 0;
  if (err != cudaSuccess) {
    std::snprintf(msg, sizeof msg, "cudaGetDeviceCount failed");
  } else if (count == 0) {
    std::snprintf(msg, sizeof msg, "no CUDA device");
  } else {
    int major = 0, minor = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, 0) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, 0) != cudaSuccess)
      std::snprintf(msg, sizeof msg, "cannot query compute capability");
    else if (major != kArchMajor || minor != kArchMinor)
      std::snprintf(msg, sizeof msg, "device is sm_%d%d, engine targets %s", major, minor,
                    kGpuTarget);
  }
  // As in the reference, the status is always "unimplemented": this library is
  // the layer-kernel path, whole-model inference is not served through this ABI.
  out->status = granite4_unimplemented;
  out->status_text = kStatusTexts[static_cast<int>(out->status)];
  out->message = msg;
}

}  // extern "C"
