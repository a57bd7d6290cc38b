// Peer-memory runtime: device allocations that other ranks (processes) on the same NVLink domain
// map into their address space, so kernels can store straight into a peer's buffers.
//
//   alloc   cudaMalloc + clear; allocations are tracked so that teardown can release them
//   export  64-byte CUDA IPC handle of an allocation (sent to the peers over the bootstrap group)
//   open    map a peer's allocation (lazy peer-access enable); the pointer is valid until close
//   close / free
//
// The reference has no counterpart: it moves rows with torch.distributed all_to_all_single
// (moeflow/fixed.py:234,237; moeflow/comm.py:26-44).  Here NCCL/gloo only carries the handles once.
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "moeflow_b200.h"

namespace {
std::mutex g_mu;
std::unordered_map<void*, unsigned long long> g_allocs;  // ptr -> bytes
std::unordered_map<void*, int> g_opened;                  // peer mappings
}  // namespace

extern "C" {

int mf_peer_alloc(void** ptr, unsigned long long bytes) {
  if (!ptr || bytes == 0) return -1;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return (int)e;
  }
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(p);
    return (int)e;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_allocs[p] = bytes;
  *ptr = p;
  return 0;
}

int mf_peer_free(void* ptr) {
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_allocs.find(ptr);
    if (it == g_allocs.end()) return -1;
    g_allocs.erase(it);
  }
  return (int)cudaFree(ptr);
}

int mf_peer_export(void* ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!ptr || !handle64) return -1;
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  std::memcpy(handle64, &h, 64);
  return 0;
}

int mf_peer_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return -1;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return (int)e;
  std::lock_guard<std::mutex> lk(g_mu);
  g_opened[p] = 1;
  *ptr = p;
  return 0;
}

int mf_peer_close(void* ptr) {
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_opened.find(ptr);
    if (it == g_opened.end()) return -1;
    g_opened.erase(it);
  }
  return (int)cudaIpcCloseMemHandle(ptr);
}

int mf_peer_can_access(int dev, int peer_dev, int* ok) {
  if (!ok) return -1;
  if (dev == peer_dev) {
    *ok = 1;
    return 0;
  }
  return (int)cudaDeviceCanAccessPeer(ok, dev, peer_dev);
}

static int g_pdl = -1;

int mf_pdl_enabled(void) {
  if (g_pdl < 0) {
    const char* v = std::getenv("MOEFLOW_PDL");
    g_pdl = (v && v[0] == '0') ? 0 : 1;
  }
  return g_pdl;
}

void mf_set_pdl(int on) { g_pdl = on ? 1 : 0; }

const char* mf_error_string(int code) {
  if (code < 0) return "moeflow_b200: bad argument";
  return cudaGetErrorString(static_cast<cudaError_t>(code));
}

int mf_device_sm_count(int* out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaDeviceGetAttribute(out, cudaDevAttrMultiProcessorCount, dev);
}

}  // extern "C"
