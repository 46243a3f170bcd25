// htr_linear_static: the packed linear for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a linear: code that runs while a
// stream is being captured into a CUDA graph (an allocation is not a stream operation and may be refused or
// break the capture), real-time or embedded loops that forbid allocation after start-up, and plugin sandboxes
// whose allocator is owned by the embedding framework.  The GEMV needs scratch (arrival counters and the
// partial sums of the column splits); here that scratch is a fixed array inside the library image, so the
// caller passes inputs and outputs only.
//
// Limits and sharing.  The array is HTR_STATIC_WORKSPACE_BYTES long and every GPU that loads the library
// holds it until the process exits.  Problems whose scratch does not fit are rejected with HTR_ERR_TOO_LARGE.
// All calls on a device share the one array and it keeps what the last call left in it: the counters at its
// start are zeroed by the first call on each device and every launch returns them to zero, the partial sums
// are always rewritten before they are read.  Two calls that are in flight on the GPU at the same time (different
// streams) would race on it; keep them on one stream or use htr_linear with private workspaces.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/htr_b200.h"

namespace {

// scratch in the library image; device code could name it directly, host code may not: the host-side symbol is
// only a handle, its device address comes from cudaGetSymbolAddress
static __device__ __align__(256) unsigned char g_static_scratch[HTR_STATIC_WORKSPACE_BYTES];

struct DeviceSetup {
  bool ready = false;
  void* scratch = nullptr;
};
DeviceSetup g_setup[64];
std::mutex g_setup_mutex;

}  // namespace

extern "C" int htr_linear_static(const void* x, int dtype, int M, const void* qweight, int mt, int nt, int K, const void* scales,
                                 const uint8_t* su, const uint8_t* sv, const void* bias, void* y, htr_stream_t stream) {
  if (M == 0) return HTR_OK;
  // the size check comes first: a call that is going to be refused puts nothing on the stream
  if (mt > 0 && nt > 0 && M > 0 && M <= HTR_GEMV_MAX_ROWS && mt % 8 == 0 && nt % 8 == 0) {
    const size_t need = htr_linear_workspace_bytes(M, mt * 16, nt * 16, K);
    if (need > (size_t)HTR_STATIC_WORKSPACE_BYTES) return HTR_ERR_TOO_LARGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HTR_ERR_CUDA;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    DeviceSetup& s = g_setup[dev];
    if (!s.ready) {
      // once per device, with that device current: resolve the device address of the array and clear the counters
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return HTR_ERR_CUDA;
      if (cudaMemsetAsync(p, 0, htr_linear_counter_bytes(mt * 16), static_cast<cudaStream_t>(stream)) != cudaSuccess) return HTR_ERR_CUDA;
      s.scratch = p;
      s.ready = true;
    }
    scratch = s.scratch;
  }
  return htr_linear_ex(x, dtype, M, qweight, mt, nt, K, scales, su, sv, bias, y, scratch, (size_t)HTR_STATIC_WORKSPACE_BYTES, stream, 0u);
}
