// Exchange of decode partials between the GPUs of a context-parallel group without a collective library: every rank
// stores its block of partials straight into the receive buffers of all ranks (plain peer stores over NVLink, no
// multicast) and counts its arrival there; the combine kernel of each rank waits - bounded - for the arrivals of the
// step and merges. The reference has no multi-GPU code; the pieces exchanged are the split-KV partials of its decode
// (flash_sparse_attn/ops/triton/flash_sparse_dec.py:485-489) and the merge is its combine (flash_dec_combine.py:15-153).
//
// One region per rank, allocated here with cudaMalloc so that it can be exported to the other processes:
//   [0, 128)    arrival counters, one 64-bit word per sending rank (only ever incremented)
//   [128, 136)  number of exchanges this rank has sent (device-side, so that a captured graph can be replayed)
//   [136, 140)  CTA counter of the push kernel
//   [256, ...)  two receive buffers of world * block_floats floats each, used alternately: a rank can only send
//               exchange k + 2 after it has received everybody's exchange k + 1, which they send after merging k.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/fsa_b200.h"
#include "fsa_aux.h"
#include "fsa_params.h"

namespace fsa {

namespace {

#ifndef FSA_PUSH_CTAS
#define FSA_PUSH_CTAS 64
#endif
constexpr int PUSH_CTAS = FSA_PUSH_CTAS;
constexpr long long HDR_BYTES = 256;

struct PushParams {
  const float4* src;
  unsigned char* base[FSA_PEER_MAX_RANKS];
  long long block_f4;  // float4 per rank block
  int world, rank;
};

__global__ void __launch_bounds__(256) peer_push_kernel(const PushParams p) {
  unsigned char* mine = p.base[p.rank];
  const unsigned long long step = *reinterpret_cast<const volatile unsigned long long*>(mine + 128);
  const long long slot = ((long long)(step & 1ull) * p.world + p.rank) * p.block_f4;
  // Every element is read once (four independent loads per thread and pass) and stored to all ranks: the stores are
  // fire-and-forget, the loads are what a thread waits for, so reading the block again for every destination (as a
  // rank-by-rank copy would) puts world times the load latency on the path. The destinations are interleaved, so
  // that all of them receive at the same time.
  constexpr int U = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long base = (long long)blockIdx.x * blockDim.x + threadIdx.x; base < p.block_f4; base += stride * U) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = base + u * stride;
      v[u] = i < p.block_f4 ? __ldg(p.src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int r = 0; r < p.world; ++r) {
      float4* dst = reinterpret_cast<float4*>(p.base[r] + HDR_BYTES) + slot;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = base + u * stride;
        if (i < p.block_f4) dst[i] = v[u];
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int r = 0; r < p.world; ++r)
      atomicAdd_system(reinterpret_cast<unsigned long long*>(p.base[r]) + p.rank, 1ull);
    // the last CTA counts the exchange as sent (every CTA has read `step` by then)
    unsigned int* done = reinterpret_cast<unsigned int*>(mine + 136);
    if (atomicAdd(done, 1u) == gridDim.x - 1) {
      *done = 0u;
      *reinterpret_cast<volatile unsigned long long*>(mine + 128) = step + 1;
    }
  }
}

}  // namespace

}  // namespace fsa

extern "C" int fsa_peer_region_bytes(int world, int64_t block_floats, int64_t* bytes) {
  if (!bytes || world <= 0 || world > FSA_PEER_MAX_RANKS || block_floats <= 0 || (block_floats & 3)) return FSA_ERR_INVALID_ARG;
  *bytes = fsa::HDR_BYTES + 2ll * world * block_floats * 4;
  return FSA_OK;
}

extern "C" int fsa_peer_alloc(int64_t bytes, void** region, FsaIpcHandle* handle) {
  if (!region || !handle || bytes <= 0) return FSA_ERR_INVALID_ARG;
  void* ptr = nullptr;
  if (cudaMalloc(&ptr, (size_t)bytes) != cudaSuccess) return FSA_ERR_LAUNCH;
  if (cudaMemset(ptr, 0, (size_t)bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaFree(ptr);
    return FSA_ERR_LAUNCH;
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) {
    cudaFree(ptr);
    return FSA_ERR_UNSUPPORTED;
  }
  static_assert(sizeof(h) == sizeof(handle->bytes), "handle size");
  memcpy(handle->bytes, &h, sizeof(h));
  *region = ptr;
  return FSA_OK;
}

extern "C" int fsa_peer_open(const FsaIpcHandle* handle, void** region) {
  if (!handle || !region) return FSA_ERR_INVALID_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle->bytes, sizeof(h));
  void* ptr = nullptr;
  if (cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    (void)cudaGetLastError();
    return FSA_ERR_UNSUPPORTED;
  }
  *region = ptr;
  return FSA_OK;
}

extern "C" int fsa_peer_close(void* region) {
  if (!region) return FSA_ERR_INVALID_ARG;
  return cudaIpcCloseMemHandle(region) == cudaSuccess ? FSA_OK : FSA_ERR_LAUNCH;
}

extern "C" int fsa_peer_free(void* region) {
  if (!region) return FSA_ERR_INVALID_ARG;
  return cudaFree(region) == cudaSuccess ? FSA_OK : FSA_ERR_LAUNCH;
}

extern "C" int fsa_peer_push(const FsaPeerArgs* a, const float* block, void* stream_) {
  if (!a || !block || a->world <= 0 || a->world > FSA_PEER_MAX_RANKS || a->rank < 0 || a->rank >= a->world ||
      a->block_floats <= 0 || (a->block_floats & 3) || (reinterpret_cast<uintptr_t>(block) & 15))
    return FSA_ERR_INVALID_ARG;
  fsa::PushParams p;
  memset(&p, 0, sizeof(p));
  p.src = reinterpret_cast<const float4*>(block);
  for (int r = 0; r < a->world; ++r) {
    if (!a->region[r] || (reinterpret_cast<uintptr_t>(a->region[r]) & 255)) return FSA_ERR_INVALID_ARG;
    p.base[r] = reinterpret_cast<unsigned char*>(a->region[r]);
  }
  p.block_f4 = a->block_floats / 4;
  p.world = a->world;
  p.rank = a->rank;
  fsa::peer_push_kernel<<<fsa::PUSH_CTAS, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(p);
  return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_LAUNCH;
}

extern "C" int fsa_peer_combine(const FsaPeerArgs* a, void* out, float* lse, int partials_per_rank, int rows, int heads,
                                int head_dim, int dtype, int arrivals_per_step, int* status, void* stream_) {
  if (!a || !out || !lse || !status || a->world <= 0 || a->world > FSA_PEER_MAX_RANKS || a->rank < 0 ||
      a->rank >= a->world || partials_per_rank <= 0 || rows < 0 || heads <= 0 || arrivals_per_step < 0)
    return FSA_ERR_INVALID_ARG;
  if (dtype != FSA_DT_BF16 && dtype != FSA_DT_FP16) return FSA_ERR_UNSUPPORTED;
  const long long per = (long long)rows * heads * (head_dim + 1);  // one partial: outputs, then log-sum-exps
  if (a->block_floats != per * partials_per_rank || !a->region[a->rank]) return FSA_ERR_INVALID_ARG;
  unsigned char* mine = reinterpret_cast<unsigned char*>(a->region[a->rank]);
  const float* recv = reinterpret_cast<const float*>(mine + fsa::HDR_BYTES);
  fsa::CombineParams c;
  memset(&c, 0, sizeof(c));
  c.out_partial = recv;
  c.lse_partial = recv + (long long)rows * heads * head_dim;
  c.out = out;
  c.lse = lse;
  c.op_ss = per;
  c.lp_ss = per;
  c.lp_sh = rows;
  c.o_sb = (long long)heads * head_dim;
  c.o_sm = 0;
  c.o_sh = head_dim;
  c.l_sb = heads;
  c.l_sh = 1;
  c.rows = rows;
  c.rows_per_batch = 1;
  c.heads = heads;
  c.head_dim = head_dim;
  c.num_splits = a->world * partials_per_rank;
  c.peer_flags = reinterpret_cast<const unsigned long long*>(mine);
  c.peer_step = reinterpret_cast<const unsigned long long*>(mine + 128);
  c.status = status;
  c.buf_stride = (long long)a->world * a->block_floats;
  c.peer_world = a->world;
  c.arrivals_per_step = arrivals_per_step > 0 ? arrivals_per_step : fsa::PUSH_CTAS;
  cudaError_t e = fsa::launch_combine(c, dtype, reinterpret_cast<cudaStream_t>(stream_));
  if (e == cudaErrorInvalidValue) return FSA_ERR_UNSUPPORTED;
  return e == cudaSuccess ? FSA_OK : FSA_ERR_LAUNCH;
}
