// nnlib_b200_attention_static: x and alpha in one call, for callers that have
// no way to hand the library a scratch buffer.
//
// Computing both outputs takes two kernels with one float per query (the
// log-sum-exp) passed between them.  Every other entry point expects the
// caller to own that buffer.  Some callers cannot: a serving loop whose memory
// pool has claimed the whole device (a raw cudaMalloc would fail, or stall
// every stream while the driver synchronises), a Julia finalizer or other
// context in which the array allocator must not run, a C host that was given
// input and output pointers and nothing else.  For them the log-sum-exp lives
// in a fixed array that is part of this library's device image.
//
// Cost and rules of that arrangement:
//  * every GPU on which the array has been brought into being holds it
//    (4 MiB) until the process exits.  With eager module loading that is every
//    GPU the library is used on; with CUDA's default lazy loading it is the
//    first call of this entry point on a device (this file holds no kernel, so
//    nothing else touches its module), which may also synchronise the device.
//    Make that first call before a memory pool claims the rest of the device;
//  * a call is limited to NNLIB_B200_STATIC_MAX_QUERIES = 2^20 queries
//    (Lq * H * B); larger problems are refused, nothing is truncated;
//  * all calls on one device share the array.  Each call overwrites the
//    entries it later reads, so nothing has to be cleared between calls and
//    stale values of an earlier call are never observed; but two calls that
//    may run on the GPU at the same time (different streams, or different
//    host threads on the same device) race on it.  Serialise them;
//  * the first call on each device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current).  Make that first call
//    ahead of any stream capture.  Later calls do no set-up.  The address is
//    remembered per device ordinal and assumes the primary context is never
//    reset (cudaDeviceReset would leave a stale address behind).
// No cudaMalloc, cudaFree or any other allocating routine is called from here.
#include <mutex>

#include "common.cuh"
#include "launchers.h"

namespace {

constexpr unsigned long long kMaxQueries = 1ull << 20;
static_assert(kMaxQueries == NNLIB_B200_STATIC_MAX_QUERIES, "header and kernel file disagree on the scratch size");

// Device-side storage.  In HOST code this name is only a handle for
// cudaGetSymbolAddress; it is never passed to a kernel as a pointer.
static __device__ __align__(256) float g_static_lse[kMaxQueries];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
float* g_static_lse_addr[kMaxDevices] = {};

// Device address of g_static_lse on the current device, looked up once per device.
int static_lse_address(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    nb200::set_last_cuda_error(e);
    return NNLIB_B200_CUDA_ERROR;
  }
  if (dev < 0 || dev >= kMaxDevices) return NNLIB_B200_INVALID_ARG;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_static_lse_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_lse);
    if (e != cudaSuccess || p == nullptr) {
      nb200::set_last_cuda_error(e);
      return NNLIB_B200_CUDA_ERROR;
    }
    g_static_lse_addr[dev] = static_cast<float*>(p);
  }
  *out = g_static_lse_addr[dev];
  return NNLIB_B200_OK;
}

}  // namespace

extern "C" int nnlib_b200_static_scratch(void** device_ptr, size_t* bytes) {
  if (!device_ptr || !bytes) return NNLIB_B200_INVALID_ARG;
  float* lse = nullptr;
  const int rc = static_lse_address(&lse);
  if (rc != NNLIB_B200_OK) return rc;
  *device_ptr = lse;
  *bytes = sizeof(float) * kMaxQueries;
  return NNLIB_B200_OK;
}

extern "C" int nnlib_b200_attention_static(const nnlib_b200_attn_params* p, void* stream) {
  if (!p || p->struct_size != sizeof(nnlib_b200_attn_params)) return NNLIB_B200_INVALID_ARG;
  if (p->Lq < 0 || p->H < 1 || p->B < 0) return NNLIB_B200_INVALID_ARG;
  // refuse before touching the device: the scratch array cannot grow
  const unsigned long long lq = (unsigned long long)p->Lq, hh = (unsigned long long)p->H, bb = (unsigned long long)p->B;
  if (lq > kMaxQueries || hh > kMaxQueries || bb > kMaxQueries || lq * hh > kMaxQueries || lq * hh * bb > kMaxQueries)
    return NNLIB_B200_WORKSPACE_TOO_SMALL;
  nnlib_b200_attn_params q = *p;
  q.lse_stride_b = 0;   // dense (Lq, H, B)
  // argument errors are reported before the device is touched: check everything but the pointers' devices
  // with a stand-in for the scratch address, which is looked up only for a call that can run
  q.lse = reinterpret_cast<float*>(uintptr_t(256));
  int rc = nb200::attention_validate(&q, false);
  if (rc != NNLIB_B200_OK) return rc;
  float* lse = nullptr;
  rc = static_lse_address(&lse);
  if (rc != NNLIB_B200_OK) return rc;
  q.lse = lse;          // any lse pointer of the caller is ignored: this variant owns the buffer
  rc = nb200::attention_validate(&q, true);   // both halves, before anything is enqueued
  if (rc != NNLIB_B200_OK) return rc;
  return nb200::attention_both(&q, stream);
}
