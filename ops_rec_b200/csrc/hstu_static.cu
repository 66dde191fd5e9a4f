// hstu_jagged_fwd_static: the forward for callers that must not allocate device memory.
//
// The regular entry point (hstu_jagged_fwd) needs a caller-provided workspace for the scheduler's work list
// and the status word.  Some callers cannot provide one: a serving process that has frozen its device-memory
// budget after start-up (every byte already handed to a framework pool, or the allocator switched off), a plugin
// whose host forbids allocation inside its enqueue callback, code that holds a lock under which the implicit
// device-wide synchronisation of cudaMalloc / cudaFree is not acceptable.  For them this file keeps one scratch
// block of HSTU_STATIC_SCRATCH_BYTES inside the library image itself: a file-scope __device__ array that every GPU
// which loads the library holds from load until the process exits.
//
// The array's name is only a host-side handle in host code, not an address a kernel may dereference, so the
// device address is looked up with cudaGetSymbolAddress - once per device, with that device current - and it is
// that pointer which reaches the kernels.
#include <mutex>

#include "hstu_common.cuh"

// sets the calling thread's error text (hstu_api.cu) and returns `code`
extern "C" int hstu_set_last_error(int code, const char* text);

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[HSTU_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

}  // namespace

extern "C" {

// The device address of the block on the current device (looked up once per device, with that device current), or
// null with an error code in *rc.
static void* scratch_of_current_device(int* rc) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *rc = hstu_set_last_error(HSTU_E_CUDA, "hstu_jagged_fwd_static: no current device (or more than 64 devices)");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_ptr[dev]) {
    // first call on this device: resolve the device address of the array (the current device is `dev`)
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      *rc = hstu_set_last_error(HSTU_E_CUDA, "hstu_jagged_fwd_static: the address of the built-in scratch block "
                                             "could not be resolved on this device");
      return nullptr;
    }
    g_scratch_ptr[dev] = p;
  }
  *rc = HSTU_OK;
  return g_scratch_ptr[dev];
}

HSTU_API int hstu_jagged_fwd_static(const HstuJaggedArgs* args, void* stream) {
  uint64_t need = 0;
  int rc = hstu_jagged_fwd_get_workspace_size(args, &need);  // validates args; host arithmetic only
  if (rc) return rc;
  if (need > HSTU_STATIC_SCRATCH_BYTES)
    return hstu_set_last_error(HSTU_E_SCRATCH_LIMIT, "hstu_jagged_fwd_static: the work list of this call does not "
                                                     "fit the built-in scratch block; use hstu_jagged_fwd with a "
                                                     "caller workspace");
  void* ptr = scratch_of_current_device(&rc);
  if (!ptr) return rc;
  // Nothing in the block has to be cleared from the host: the scheduling pre-pass that every call enqueues first
  // rewrites the status word, the item count and the work counter before the attention kernel reads them, and
  // the work list is rebuilt up to the new count.  Contents left by the previous call are never read.
  return hstu_jagged_fwd(args, ptr, HSTU_STATIC_SCRATCH_BYTES, stream);
}

// The status word of the last hstu_jagged_fwd_static call on the current device (the caller of that entry point has
// no workspace pointer to hand to hstu_jagged_fwd_status).  Waits for `stream`; allocates nothing.
HSTU_API int hstu_jagged_fwd_static_status(void* stream, uint32_t* status) {
  int rc = HSTU_OK;
  void* ptr = scratch_of_current_device(&rc);
  if (!ptr) return rc;
  return hstu_jagged_fwd_status(ptr, stream, status);
}

}  // extern "C"
