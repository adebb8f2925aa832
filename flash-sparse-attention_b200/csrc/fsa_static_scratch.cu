// Split-KV decode for callers that must not allocate device memory.
//
// The regular decode entry point (fsa_decode) takes its split workspace - the per-split partial
// outputs and log-sum-exps - from the caller, who normally gets it from an allocator. Some callers
// have no allocator to ask: a serving loop that has already handed every free byte of the GPU to its
// own KV-cache pool, a plugin running inside a host framework whose memory plan was frozen at load
// time, or code that runs between other people's kernels and may not trigger the implicit device
// synchronisation a cudaMalloc / cudaFree brings. For them this file keeps ONE fixed workspace inside
// the library image itself (a file-scope __device__ array) and offers a decode call that uses it.
// The array becomes resident on a GPU when that GPU first uses it: with CUDA's lazy module loading that
// is the first call of this entry point on the device, which loads the module holding the array (16 MiB
// taken from the device's free memory, with an implicit synchronisation) and keeps it until the process
// exits. So that first call belongs to start-up, before a pool claims the rest of the GPU and before
// any stream capture; every later call on that device allocates and synchronises nothing. A device with
// less than 16 MiB free at that moment gets FSA_ERR_SCRATCH_UNAVAILABLE.
//
// Consequences of the workspace being a single shared array:
//   * a request whose partials do not fit is refused (FSA_ERR_SCRATCH_TOO_SMALL), never truncated;
//   * the array still holds whatever the previous call left there. Nothing in it needs clearing: the
//     decode kernel writes every (split, sequence, head) slot of the region it is given before the
//     combine kernel reads it, so stale values are never observed;
//   * two calls that can overlap on the GPU (different streams, or graph branches) would write the
//     same bytes: callers must order such calls themselves.
// The first call on each device looks up the array's device address (host code cannot use the
// symbol itself as a pointer). That look-up is not a stream operation: make the first call on a
// device outside of any stream capture.
#include <cuda_runtime.h>
#include <string.h>
#include "../../include/fsa_b200.h"

namespace {

constexpr size_t kScratchFloats = FSA_STATIC_SCRATCH_BYTES / sizeof(float);

static __device__ __align__(256) float g_decode_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the workspace on the current device (resolved once per device).
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FSA_ERR_SCRATCH_UNAVAILABLE;
  float* p = __atomic_load_n(&g_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    void* sym = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&sym, g_decode_scratch);
    if (e != cudaSuccess || !sym) {
      (void)cudaGetLastError();
      return FSA_ERR_SCRATCH_UNAVAILABLE;
    }
    p = static_cast<float*>(sym);
    __atomic_store_n(&g_scratch_addr[dev], p, __ATOMIC_RELEASE);
  }
  *out = p;
  return FSA_OK;
}

}  // namespace

extern "C" {

size_t fsa_static_scratch_bytes(void) { return FSA_STATIC_SCRATCH_BYTES; }

int fsa_decode_static_scratch(const FsaDecArgs* a, void* stream) {
  if (!a) return FSA_ERR_INVALID_ARG;
  if (a->partial_only) return FSA_ERR_INVALID_ARG;  // the partials live in private memory: nothing to hand out
  const int ns = a->num_splits > 0 ? a->num_splits : 1;
  if (a->batch <= 0 || a->heads_q <= 0 || a->head_dim <= 0) return FSA_ERR_INVALID_ARG;
  const size_t slots = (size_t)ns * (size_t)a->batch * (size_t)a->heads_q;
  const size_t need = slots * ((size_t)a->head_dim + 1);  // partial outputs + one log-sum-exp each
  if (need > kScratchFloats) return FSA_ERR_SCRATCH_TOO_SMALL;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != FSA_OK) return rc;
  FsaDecArgs b;
  memcpy(&b, a, sizeof(b));
  b.num_splits = ns;
  b.out_partial = scratch;
  b.lse_partial = scratch + slots * (size_t)a->head_dim;
  return fsa_decode(&b, stream);
}

}  // extern "C"
