// Micro-benchmark behind the roofline of the gathered (top-k) decode: how many scattered key / value rows per second
// can the GPU fetch when nothing else is done with them?
//
// A pool of `pool_mb` MB holds rows at a stride of `stride` bytes; a list of row numbers (random, or ascending = one
// sequential sweep) is read by warps that fetch `row` bytes of every listed row with 16-byte loads (as the decode's
// copies do: the lanes of a warp cover whole rows, 512 bytes per warp instruction), eight independent loads in
// flight per lane, and fold the data into one word per thread. Eight CTAs of 256 threads per SM: more loads in
// flight than the decode kernel has, and no arithmetic to speak of. Two more variants fetch the same rows the way a
// kernel that wants them in shared memory can: cp.async (.cg and .ca; 16 bytes per lane, ring of four stages per warp, twelve
// warps per SM) and one cp.async.bulk per row on an mbarrier (four warps per SM). Prints rows per second and bytes
// per second for row sizes of 128 / 256 / 512 bytes at the strides the paged cache has (one position = all KV heads
// side by side).
//
// Build and run (sm_100a):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o row_gather_probe row_gather_probe.cu
//   ./row_gather_probe
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_runtime.h>

namespace {

#define CHECK(x)                                                                  \
  do {                                                                            \
    cudaError_t e_ = (x);                                                         \
    if (e_ != cudaSuccess) {                                                      \
      std::fprintf(stderr, "%s:%d %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
      std::exit(1);                                                               \
    }                                                                             \
  } while (0)

// LPR lanes share one row (LPR * 16 bytes); a warp instruction covers 32 / LPR rows.
template <int LPR>
__global__ void __launch_bounds__(256) gather_kernel(const uint8_t* __restrict__ pool, const int* __restrict__ rows,
                                                     long long n_rows, long long stride, unsigned* __restrict__ sink) {
  constexpr int RPI = 32 / LPR;  // rows per warp instruction
  constexpr int UNROLL = 8;
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long n_warps = (long long)gridDim.x * (blockDim.x >> 5);
  uint4 acc = make_uint4(0, 0, 0, 0);
  for (long long base = warp * (RPI * UNROLL); base < n_rows; base += n_warps * (RPI * UNROLL)) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long i = base + u * RPI + lane / LPR;
      const long long r = i < n_rows ? rows[i] : 0;
      v[u] = *reinterpret_cast<const uint4*>(pool + r * stride + (lane % LPR) * 16);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      acc.x ^= v[u].x;
      acc.y ^= v[u].y;
      acc.z ^= v[u].z;
      acc.w ^= v[u].w;
    }
  }
  if ((acc.x ^ acc.y ^ acc.z ^ acc.w) == 0x12345678u) sink[0] = 1;  // keeps the loads alive
}

// The same fetch through cp.async (16 bytes per lane into a shared-memory ring of four 4 KB stages per warp, as
// the decode kernel does it), four warps per CTA; the data is not read back.
template <int LPR, bool CA>
__global__ void __launch_bounds__(128) gather_cp_async_kernel(const uint8_t* __restrict__ pool,
                                                              const int* __restrict__ rows, long long n_rows,
                                                              long long stride, unsigned* __restrict__ sink) {
  constexpr int RPI = 32 / LPR;
  constexpr int PER_STAGE = 8;  // warp instructions per stage: 4 KB
  constexpr int STAGES = 4;
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + w;
  const long long n_warps = (long long)gridDim.x * (blockDim.x >> 5);
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + w * (STAGES * PER_STAGE * 512);
  int stage = 0;
  for (long long base = warp * (RPI * PER_STAGE); base < n_rows; base += n_warps * (RPI * PER_STAGE)) {
#pragma unroll
    for (int u = 0; u < PER_STAGE; ++u) {
      const long long i = base + u * RPI + lane / LPR;
      const long long r = i < n_rows ? rows[i] : 0;
      const uint8_t* src = pool + r * stride + (lane % LPR) * 16;
      const uint32_t dst = ring + (stage * PER_STAGE + u) * 512 + lane * 16;
      if (CA)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
      else
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 1) : "memory");
    stage = (stage + 1) % STAGES;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (smem[threadIdx.x] == 0x5a && n_rows < 0) sink[0] = 1;
}

// The same fetch with one bulk copy (cp.async.bulk, completion on an mbarrier) per row, issued by one lane per row:
// four stages of 16 rows per warp and four warps per SM, or two stages and twelve warps per SM.
template <int STAGES>
__global__ void __launch_bounds__(128) gather_bulk_kernel(const uint8_t* __restrict__ pool, const int* __restrict__ rows,
                                                          long long n_rows, long long stride, int row_bytes,
                                                          unsigned* __restrict__ sink, unsigned* __restrict__ status) {
  constexpr int ROWS = 16;
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + w;
  const long long n_warps = (long long)gridDim.x * (blockDim.x >> 5);
  uint8_t* ring = smem + 128 + w * (STAGES * ROWS * 512);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem) + w * STAGES;
  if (lane == 0)
    for (int i = 0; i < STAGES; ++i)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(bars + i)));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncwarp();
  long long it = 0;
  bool ok = true;
  auto wait_stage = [&](int st, unsigned parity) {
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(bars + st);
    unsigned done = 0;
    for (int spin = 0; spin < (1 << 18) && !done; ++spin)  // bounded: a wait that runs out is reported, not repeated
      asm volatile(
          "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(done)
          : "r"(bar), "r"(parity)
          : "memory");
    if (!done) ok = false;
  };
  for (long long base = warp * ROWS; base < n_rows && ok; base += n_warps * ROWS, ++it) {
    const int st = (int)(it % STAGES);
    if (it >= STAGES) wait_stage(st, (unsigned)(((it / STAGES) - 1) & 1));  // the stage's previous copies have landed
    if (!ok) break;
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(bars + st);
    const int n_here = (int)((n_rows - base) < ROWS ? (n_rows - base) : ROWS);
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(n_here * row_bytes)
                   : "memory");
    __syncwarp();
    if (lane < n_here) {
      const long long r = rows[base + lane];
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(ring + (st * ROWS + lane) * 512);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                   "l"(pool + r * stride), "r"(row_bytes), "r"(bar)
                   : "memory");
    }
  }
  // drain: every stage that was used has one outstanding phase
  for (int st = 0; st < STAGES && ok; ++st) {
    const long long uses = it > st ? (it - st + STAGES - 1) / STAGES : 0;
    if (uses > 0) wait_stage(st, (unsigned)((uses - 1) & 1));
  }
  if (!ok && lane == 0) atomicExch(status, 1u);
  if (smem[threadIdx.x + 256] == 0x5a && n_rows < 0) sink[0] = 1;
}

// how: 0 = ld.global into registers, 1 = cp.async.cg ring, 2 = one bulk copy per row (4 warps per SM), 3 = cp.async.ca
// ring, 4 = one bulk copy per row (12 warps per SM)
float run(int how, int lpr, const uint8_t* pool, const int* rows, long long n_rows, long long stride, unsigned* sink,
          unsigned* status, int sms) {
  constexpr int kCpSmem = 4 * 4 * 8 * 512, kBulkSmem = 128 + 4 * 4 * 16 * 512, kBulkSmem2 = 128 + 4 * 2 * 16 * 512;
  static bool opted = false;
  if (!opted) {
    CHECK(cudaFuncSetAttribute(gather_cp_async_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCpSmem));
    CHECK(cudaFuncSetAttribute(gather_cp_async_kernel<16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCpSmem));
    CHECK(cudaFuncSetAttribute(gather_cp_async_kernel<32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCpSmem));
    CHECK(cudaFuncSetAttribute(gather_cp_async_kernel<8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCpSmem));
    CHECK(cudaFuncSetAttribute(gather_cp_async_kernel<16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCpSmem));
    CHECK(cudaFuncSetAttribute(gather_cp_async_kernel<32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCpSmem));
    CHECK(cudaFuncSetAttribute(gather_bulk_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmem));
    CHECK(cudaFuncSetAttribute(gather_bulk_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmem2));
    opted = true;
  }
  auto launch = [&]() {
    if (how == 0) {
      const int grid = sms * 8;
      if (lpr == 8) gather_kernel<8><<<grid, 256>>>(pool, rows, n_rows, stride, sink);
      if (lpr == 16) gather_kernel<16><<<grid, 256>>>(pool, rows, n_rows, stride, sink);
      if (lpr == 32) gather_kernel<32><<<grid, 256>>>(pool, rows, n_rows, stride, sink);
    } else if (how == 1) {
      const int grid = sms * 3;  // 64 KB of ring per CTA: three CTAs = twelve warps per SM
      if (lpr == 8) gather_cp_async_kernel<8, false><<<grid, 128, kCpSmem>>>(pool, rows, n_rows, stride, sink);
      if (lpr == 16) gather_cp_async_kernel<16, false><<<grid, 128, kCpSmem>>>(pool, rows, n_rows, stride, sink);
      if (lpr == 32) gather_cp_async_kernel<32, false><<<grid, 128, kCpSmem>>>(pool, rows, n_rows, stride, sink);
    } else if (how == 3) {
      const int grid = sms * 3;
      if (lpr == 8) gather_cp_async_kernel<8, true><<<grid, 128, kCpSmem>>>(pool, rows, n_rows, stride, sink);
      if (lpr == 16) gather_cp_async_kernel<16, true><<<grid, 128, kCpSmem>>>(pool, rows, n_rows, stride, sink);
      if (lpr == 32) gather_cp_async_kernel<32, true><<<grid, 128, kCpSmem>>>(pool, rows, n_rows, stride, sink);
    } else if (how == 4) {
      gather_bulk_kernel<2><<<sms * 3, 128, kBulkSmem2>>>(pool, rows, n_rows, stride, lpr * 16, sink, status);
    } else {
      gather_bulk_kernel<4><<<sms, 128, kBulkSmem>>>(pool, rows, n_rows, stride, lpr * 16, sink, status);
    }
  };
  for (int i = 0; i < 3; ++i) launch();
  CHECK(cudaDeviceSynchronize());
  cudaEvent_t e0, e1;
  CHECK(cudaEventCreate(&e0));
  CHECK(cudaEventCreate(&e1));
  CHECK(cudaEventRecord(e0));
  for (int i = 0; i < 5; ++i) launch();
  CHECK(cudaEventRecord(e1));
  CHECK(cudaEventSynchronize(e1));
  float ms = 0.f;
  CHECK(cudaEventElapsedTime(&ms, e0, e1));
  CHECK(cudaGetLastError());
  return ms / 5;
}

}  // namespace

int main() {
  cudaDeviceProp prop;
  CHECK(cudaGetDeviceProperties(&prop, 0));
  const int sms = prop.multiProcessorCount;
  const long long pool_bytes = 4096ll << 20;  // 4 GB: far above the L2
  uint8_t* pool;
  CHECK(cudaMalloc(&pool, pool_bytes));
  CHECK(cudaMemset(pool, 1, pool_bytes));
  unsigned* sink;
  CHECK(cudaMalloc(&sink, 4));
  const long long n_list = 4ll << 20;  // rows fetched per launch
  int* rows;
  CHECK(cudaMalloc(&rows, n_list * 4));
  std::vector<int> h(n_list);
  std::printf("%s, %d SMs; pool 4096 MB, %lld rows per launch\n", prop.name, sms, n_list);
  unsigned* status;
  CHECK(cudaMalloc(&status, 4));
  CHECK(cudaMemset(status, 0, 4));
  std::printf("%-12s %-10s %-10s %-12s %12s %12s\n", "fetch", "row bytes", "stride", "order", "G rows/s", "TB/s");
  const char* how_names[5] = {"ld.global", "cp.async.cg", "bulk copy", "cp.async.ca", "bulk x12"};
  uint64_t s = 0x9e3779b97f4a7c15ull;
  auto rnd = [&]() {
    s ^= s << 13;
    s ^= s >> 7;
    s ^= s << 17;
    return s;
  };
  const int row_sizes[3] = {128, 256, 512};
  for (int row : row_sizes) {
    // strides: the row itself (rows packed), and one position of 8 KV heads (the paged cache's layout)
    const long long strides[2] = {row, 8ll * row};
    for (long long stride : strides) {
      const long long pool_rows = pool_bytes / stride;
      for (int order = 0; order < 2; ++order) {
        for (long long i = 0; i < n_list; ++i)
          h[i] = order == 0 ? (int)(rnd() % (uint64_t)pool_rows) : (int)(i % pool_rows);
        CHECK(cudaMemcpy(rows, h.data(), n_list * 4, cudaMemcpyHostToDevice));
        for (int how = 0; how < 5; ++how) {
          const float ms = run(how, row / 16, pool, rows, n_list, stride, sink, status, sms);
          std::printf("%-12s %-10d %-10lld %-12s %12.2f %12.3f\n", how_names[how], row, stride,
                      order == 0 ? "random" : "ascending", n_list / ms / 1e6, (double)n_list * row / ms / 1e9);
        }
      }
    }
  }
  unsigned st = 0;
  CHECK(cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost));
  if (st) std::printf("a bounded wait of the bulk-copy variant ran out: its figures are not valid\n");
  return 0;
}
