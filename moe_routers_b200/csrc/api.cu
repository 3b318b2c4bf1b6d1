// Library-level entry points: version, error text, workspace helpers.
#include <atomic>
#include <cstdarg>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace moe {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

static std::atomic<long long> g_launches{0};

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) {
    note_launch();
    return MOE_OK;
  }
  return fail(MOE_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

// -1: not decided yet (the environment decides on first use), 0 / 1: off / on
static std::atomic<int> g_pdl{-1};

bool pdl_enabled() {
  int v = g_pdl.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* env = getenv("MOE_B200_PDL");
    v = (env && env[0] == '0') ? 0 : 1;
    g_pdl.store(v, std::memory_order_relaxed);
  }
  return v != 0;
}

}  // namespace moe

extern "C" int moe_version(void) { return 200; }

extern "C" long long moe_launch_count(void) { return moe::g_launches.load(std::memory_order_relaxed); }

extern "C" int moe_set_pdl(int enabled) {
  moe::g_pdl.store(enabled ? 1 : 0, std::memory_order_relaxed);
  return MOE_OK;
}

extern "C" int moe_set_wait_limit(void* workspace, size_t workspace_bytes, unsigned long long limit_ns, void* stream) {
  using namespace moe;
  if (!workspace || workspace_bytes < (size_t)(kStatusBytes + kControlBytes))
    return fail(MOE_ERR_WORKSPACE, "moe_set_wait_limit: workspace too small");
  // the value travels by value inside the launch of a tiny memcpy node: no host buffer has to outlive the call
  const cudaError_t e = cudaMemcpyAsync(static_cast<char*>(workspace) + 2 * sizeof(int32_t), &limit_ns, sizeof(limit_ns),
                                        cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_set_wait_limit: %s", cudaGetErrorString(e));
  return MOE_OK;
}

extern "C" const char* moe_last_error(void) { return moe::g_error; }

extern "C" size_t moe_workspace_bytes(int tokens, int experts, int top_k) {
  if (tokens < 0 || experts <= 0) return 0;
  return moe::workspace_bytes_for(tokens, experts, top_k);
}

extern "C" int moe_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  using namespace moe;
  if (!workspace || workspace_bytes < (size_t)(kStatusBytes + kControlBytes))
    return fail(MOE_ERR_WORKSPACE, "moe_workspace_init: workspace too small");
  const cudaError_t e = cudaMemsetAsync(workspace, 0, kStatusBytes + kControlBytes,
                                        static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_workspace_init: %s", cudaGetErrorString(e));
  return MOE_OK;
}

extern "C" int moe_read_status(const void* workspace, void* stream, int* status_host) {
  using namespace moe;
  if (!workspace || !status_host) return fail(MOE_ERR_ARG, "moe_read_status: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int32_t v = 0;
  cudaError_t e = cudaMemcpyAsync(&v, workspace, sizeof(v), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail(MOE_ERR_LAUNCH, "moe_read_status: %s", cudaGetErrorString(e));
  *status_host = v;
  if (v != 0) {
    const char* what = (v & 0xf00) == kErrMbarTimeout   ? "an mbarrier wait gave up"
                       : (v & 0xf00) == kErrGridBarrier ? "a grid barrier wait gave up"
                       : (v & 0xf00) == kErrBadIndex    ? "an expert index was out of range"
                       : (v & 0xf00) == kErrPeerWait    ? "a wait for a peer rank's signal gave up"
                                                        : "unknown device error";
    return fail(MOE_ERR_DEVICE, "device status 0x%x: %s", v, what);
  }
  return MOE_OK;
}

extern "C" int moe_device_pci_bus_id(int device, char* out, int len) {
  if (out == nullptr || len < 16) return moe::fail(MOE_ERR_ARG, "moe_device_pci_bus_id: buffer of at least 16 bytes needed");
  const cudaError_t e = cudaDeviceGetPCIBusId(out, len, device);
  if (e != cudaSuccess) return moe::fail(MOE_ERR_DEVICE, "moe_device_pci_bus_id: %s", cudaGetErrorString(e));
  return MOE_OK;
}
