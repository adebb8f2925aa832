// Micro-benchmark behind the role layout of the backward kernel: how fast does one thread feed the tensor pipe with
// the 40 tcgen05.mma (128 x 128 x 16, bf16) of one backward step, and what slows it down?
//
// One CTA per SM (148), 12 warps. Warp 8 lane 0 issues the MMAs of the step in the operand forms the kernel uses
// (S^T / dP^T: both operands K-major; dV: A from TMEM, B MN-major; dQ: both MN-major; dK: A K-major, B MN-major),
// five commits per step, zero-filled operands. Meanwhile other warps run one kind of "noise":
//   memory kinds run on warps 1-7 and 9-11 (shared-memory stores / loads, TMEM loads, bulk copies into shared
//   memory, bulk reduce-adds out of it); arithmetic kinds run on warps 0 and 4, the two warps that share the
//   issuer's scheduler (warp id mod 4).
// Prints cycles per MMA (64 = the pipe's rate for this shape).
//
// Build and run (sm_100a):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr \
//        -o tcgen05_issue_probe tcgen05_issue_probe.cu && ./tcgen05_issue_probe
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../csrc/fsa_ptx.cuh"
using namespace fsa;

namespace {
constexpr int KT = 32768;                      // one 128 x 128 16-bit operand tile
constexpr int SCRATCH = 6 * KT + 1024;         // noise scratch (32 KB) behind the six operand tiles and the barriers
constexpr int SMEM = SCRATCH + 32768;
enum Noise { NONE, ST_SHARED, LD_SHARED, TMEM_LD, BULK_IN, BULK_RED, FFMA, FFMA2, IMAD, EX2, IADD_XOR, FMAX, PACK_BF16, N_KINDS };
const char* kNames[N_KINDS] = {"none", "st.shared (10 warps)", "ld.shared (10 warps)", "tcgen05.ld (10 warps)",
                               "bulk copy global->shared", "bulk reduce-add shared->global", "scalar FFMA, 32 chains",
                               "packed FFMA2, 16 chains", "IMAD, 32 chains", "ex2 (MUFU), 32 chains",
                               "integer add / xor, 32 chains", "float max, 32 chains", "bf16 pack (cvt), 16 chains"};

__global__ void __launch_bounds__(384) probe(int iters, int noise, uint8_t* gbuf, long long* out, int* err) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * KT);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 6 * KT + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 6 * KT + 128);
  volatile int* done = reinterpret_cast<volatile int*>(smem + 6 * KT + 132);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < 6 * KT / 16; i += 384) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  for (int i = tid; i < 32768 / 16; i += 384) reinterpret_cast<uint4*>(smem + SCRATCH)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    mbar_init(&bars[0], 1);  // completion of everything
    mbar_init(&bars[1], 1);  // per-GEMM commits (nobody waits)
    mbar_init(&bars[2], 1);  // bulk copies of the noise warp
    *abort_flag = 0;
    *done = 0;
    mbar_fence_init();
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ---- the issuer: the step's five GEMMs, lead-lane predicated, descriptors advanced on their low word ----
    const uint32_t sK = smem_u32(smem), sV = smem_u32(smem + KT), sQ = smem_u32(smem + 2 * KT), sDO = smem_u32(smem + 4 * KT),
                   sDS = smem_u32(smem + 5 * KT);
    constexpr uint32_t id_kk = umma_idesc_f16(128, 128, true, false, false);
    constexpr uint32_t id_km = umma_idesc_f16(128, 128, true, false, true);
    constexpr uint32_t id_mm = umma_idesc_f16(128, 128, true, true, true);
    const uint32_t lead = lane == 0;
    const uint32_t k_lo = umma_desc_lo(sK, 16), v_lo = umma_desc_lo(sV, 16), do_lo = umma_desc_lo(sDO, 16),
                   ds_lo = umma_desc_lo(sDS, 16), do_mn = umma_desc_lo(sDO, 128 * 128), ds_mn = umma_desc_lo(sDS, 128 * 128),
                   k_mn = umma_desc_lo(sK, 128 * 128), q_lo0 = umma_desc_lo(sQ, 16), q_mn0 = umma_desc_lo(sQ, 128 * 128);
    bool ok = true;
    const long long t0 = clock64();
    for (int it = 0; it < iters && ok; ++it) {
      const uint32_t q_lo = q_lo0 + (it & 1) * (KT >> 4), q_mn = q_mn0 + (it & 1) * (KT >> 4);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {  // dP^T
        const uint32_t koff = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
        umma_ss_lead(lead, tmem_base + 128, umma_desc_at(v_lo, koff), umma_desc_at(do_lo, koff), id_kk, kk > 0);
      }
      umma_commit_lead(lead, &bars[1]);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)  // dV
        umma_ts_lead(lead, tmem_base + 256, tmem_base + ((kk < 4) ? kk * 8 : 96 + (kk - 4) * 8), umma_desc_at(do_mn, kk * 2048),
                     id_km, 1);
      umma_commit_lead(lead, &bars[1]);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {  // S^T
        const uint32_t koff = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
        umma_ss_lead(lead, tmem_base, umma_desc_at(k_lo, koff), umma_desc_at(q_lo, koff), id_kk, kk > 0);
      }
      umma_commit_lead(lead, &bars[1]);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)  // dQ
        umma_ss_lead(lead, tmem_base + 128, umma_desc_at(ds_mn, kk * 2048), umma_desc_at(k_mn, kk * 2048), id_mm, kk > 0);
      umma_commit_lead(lead, &bars[1]);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)  // dK
        umma_ss_lead(lead, tmem_base + 384, umma_desc_at(ds_lo, (kk >> 2) * (128 * 128) + (kk & 3) * 32),
                     umma_desc_at(q_mn, kk * 2048), id_km, 1);
      umma_commit_lead(lead, &bars[1]);
      if ((it & 63) == 63) ok = !*abort_flag;
    }
    umma_commit_lead(lead, &bars[0]);
    ok = mbar_wait(&bars[0], 0, abort_flag);
    const long long t1 = clock64();
    if (!ok) atomicExch(err, 1);
    if (lane == 0) out[blockIdx.x] = t1 - t0;
    *done = 1;
  } else if (noise >= FFMA) {
    // ---- arithmetic noise on the two warps of the issuer's scheduler ------------------------------------------
    if ((warp & 3) == 0) {
      float a[32];
      int ia[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        a[j] = float(lane + j) * 0.01f;
        ia[j] = lane + j;
      }
      for (int i = 0; i < 2000000 && !*done; ++i) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (noise == FFMA) a[j] = fmaf(a[j], 1.0001f, 0.5f);
            if (noise == IMAD) ia[j] = ia[j] * 3 + 1;
            if (noise == EX2) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(a[j]));
            if (noise == IADD_XOR) ia[j] = (ia[j] + ia[(j + 1) & 31]) ^ 0x55;
            if (noise == FMAX) a[j] = fmaxf(a[j], a[(j + 1) & 31]);
          }
          if (noise == FFMA2 || noise == PACK_BF16) {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              if (noise == FFMA2) {
                const float2 v = fma2(make_float2(a[j], a[j + 1]), make_float2(1.0001f, 1.0001f), make_float2(0.5f, 0.5f));
                a[j] = v.x;
                a[j + 1] = v.y;
              } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(a[j], a[j + 1]);
                a[j] = __low2float(h) + 1.0f;
                a[j + 1] = __high2float(h);
              }
            }
          }
        }
      }
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) sum += a[j] + float(ia[j]);
      if (sum == 1234.5f) out[0] = 1;
    }
  } else if (noise == BULK_IN || noise == BULK_RED) {
    if (warp == 9 && lane == 0) {
      uint8_t* buf = smem + SCRATCH;
      for (int i = 0; i < 2000000 && !*done; ++i) {
        uint8_t* g = gbuf + (size_t)((i * 7 + blockIdx.x) & 1023) * 16384;
        if (noise == BULK_IN) {
          mbar_arrive_expect_tx(&bars[2], 16384);
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                           smem_u32(buf)),
                       "l"(g), "r"(16384), "r"(smem_u32(&bars[2]))
                       : "memory");
          if (!mbar_wait(&bars[2], i & 1, abort_flag)) break;
        } else {
          asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(g),
                       "r"(smem_u32(buf)), "r"(16384)
                       : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  } else if (noise != NONE && warp != 0) {
    // ---- memory noise on ten warps -----------------------------------------------------------------------------
    uint8_t* scr = smem + SCRATCH + (warp > 8 ? warp - 2 : warp - 1) * 2048;
    uint32_t acc = 0;
    for (int i = 0; i < 2000000 && !*done; ++i) {
      if (noise == ST_SHARED) {
#pragma unroll
        for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(scr + (j & 3) * 512 + lane * 16) = make_uint4(i, j, acc, 0);
      } else if (noise == LD_SHARED) {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += reinterpret_cast<volatile uint4*>(scr + (j & 3) * 512 + lane * 16)->x;
      } else {
        uint32_t r[32];
        tmem_ld32(tmem_base + (uint32_t((warp & 3) * 32) << 16) + 384, r);
        tmem_ld_wait();
        acc += r[3];
      }
    }
    if (acc == 0x7fffffffu) out[0] = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}
}  // namespace

int main() {
  long long* out;
  int* err;
  uint8_t* gbuf;
  cudaMalloc(&out, 148 * 8);
  cudaMalloc(&err, 4);
  cudaMalloc(&gbuf, 1024 * 16384);
  cudaMemset(err, 0, 4);
  cudaMemset(gbuf, 0, 1024 * 16384);
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  const int iters = 2000;
  for (int noise = 0; noise < N_KINDS; ++noise) {
    for (int rep = 0; rep < 2; ++rep) {
      probe<<<148, 384, SMEM>>>(iters, noise, gbuf, out, err);
      if (cudaDeviceSynchronize() != cudaSuccess) {
        printf("launch failed\n");
        return 1;
      }
    }
    std::vector<long long> h(148);
    cudaMemcpy(h.data(), out, 148 * 8, cudaMemcpyDeviceToHost);
    long long mx = 0;
    for (auto v : h) mx = v > mx ? v : mx;
    printf("%-34s %6.1f cycles per MMA\n", kNames[noise], double(mx) / (iters * 40.0));
  }
  int herr = 0;
  cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost);
  printf("expired waits: %d\n", herr);
  return herr;
}
