// Bandwidth-bound helper kernels around the attention main loops: split-KV combine.
#include "fsa_ptx.cuh"
#include "fsa_params.h"
#include "fsa_aux.h"
#include "fsa_schedule.h"

namespace fsa {

namespace {

// One warp merges the partial results of one (row, head): running max / sum over the splits in the
// base-2 domain, partials with lse = -inf contribute nothing, final lse is converted to natural log.
// Restates _fwd_combine_kernel (flash_sparse_attn/ops/triton/flash_fwd_combine.py:118-161) and
// _dec_combine_kernel (flash_dec_combine.py:15-153).
template <typename T, int VEC>
__global__ void __launch_bounds__(256) combine_kernel(CombineParams p) {
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  long long buf_off = 0;
  if (p.peer_flags) {
    // partials stored by other GPUs: wait for every rank's arrivals of this step (bounded: on expiry the status word
    // is set and the kernel goes on with whatever is there)
    __shared__ unsigned long long step_s;
    if (threadIdx.x == 0) step_s = *reinterpret_cast<const volatile unsigned long long*>(p.peer_step);
    __syncthreads();
    const unsigned long long step = step_s;
    if (threadIdx.x < p.peer_world) {
      const unsigned long long want = step * (unsigned long long)p.arrivals_per_step;
      const unsigned long long* f = p.peer_flags + threadIdx.x;
      const long long t0 = clock64();
      for (;;) {
        unsigned long long seen;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(f) : "memory");
        if (seen >= want) break;
        if (clock64() - t0 > FSA_WAIT_CYCLES) {
          atomicExch(p.status, 4);
          break;
        }
        __nanosleep(100);
      }
    }
    __syncthreads();
    buf_off = (long long)((step - 1) & 1ull) * p.buf_stride;
  }
  if (item >= (long long)p.rows * p.heads) return;
  const int h = (int)(item % p.heads);
  const long long row = item / p.heads;
  const int b = (int)(row / p.rows_per_batch);
  const long long s = row - (long long)b * p.rows_per_batch;

  const float* lp = p.lse_partial + buf_off + (long long)h * p.lp_sh + row;
  const float* op = p.out_partial + buf_off + (row * p.heads + h) * p.head_dim;
  float e_max = -INFINITY, e_sum = 0.f;
  float acc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
  const int d0 = lane * VEC;
  const bool active = d0 < p.head_dim;
  for (int sp = 0; sp < p.num_splits; ++sp) {
    const float lse_s = lp[(long long)sp * p.lp_ss];
    const float new_max = fmaxf(lse_s, e_max);
    const float old_scale = (e_max == -INFINITY) ? 0.f : exp2f(e_max - new_max);
    const float w = (lse_s == -INFINITY) ? 0.f : exp2f(lse_s - new_max);
    if (active) {
      const float* src = op + (long long)sp * p.op_ss + d0;
#pragma unroll
      for (int i = 0; i < VEC; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(src + i);
        acc[i] = acc[i] * old_scale + w * v.x;
        acc[i + 1] = acc[i + 1] * old_scale + w * v.y;
        acc[i + 2] = acc[i + 2] * old_scale + w * v.z;
        acc[i + 3] = acc[i + 3] * old_scale + w * v.w;
      }
    }
    e_sum = e_sum * old_scale + w;
    e_max = new_max;
  }
  const float inv = (e_sum == 0.f || e_sum != e_sum) ? 0.f : 1.0f / e_sum;
  if (active) {
    T* dst = reinterpret_cast<T*>(p.out) + (long long)b * p.o_sb + s * p.o_sm + (long long)h * p.o_sh + d0;
#pragma unroll
    for (int i = 0; i < VEC; i += 2) {
      *reinterpret_cast<uint32_t*>(dst + i) = pack2<T>(acc[i] * inv, acc[i + 1] * inv);
    }
  }
  if (lane == 0) {
    const float lse = (e_sum > 0.f) ? (e_max + log2f(e_sum)) * 0.6931471805599453f : -INFINITY;
    p.lse[(long long)b * p.l_sb + (long long)h * p.l_sh + s] = lse;
  }
}

template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

// Row position inside the tile-padded workspaces: every sequence starts on a multiple of 128 rows
// (same rule as flash_sparse_attn/ops/triton/seqlen_info.py:86 with TILE_M = 128).
__device__ __forceinline__ long long padded_row(int varlen, const int* cu_q, int b, int sq_static, int q) {
  if (varlen) return (long long)((cu_q[b] + b * 128) / 128) * 128 + q;
  return (long long)b * ((sq_static + 127) / 128) * 128 + q;
}

// Locates one (query row, head) item: batch, position inside the sequence, row in the packed tensor.
struct RowPos {
  int b, q, h;
  long long tok;
};
__device__ __forceinline__ RowPos locate_row(long long item, int heads, int varlen, const int* cu_q, int B, int sq) {
  RowPos r;
  r.h = (int)(item % heads);
  const long long row = item / heads;
  if (varlen) {
    // B is small: linear scan over the sequence starts
    int b = 0;
    while (b + 1 < B && cu_q[b + 1] <= row) ++b;
    r.b = b;
    r.q = (int)(row - cu_q[b]);
    r.tok = row;
  } else {
    r.b = (int)(row / sq);
    r.q = (int)(row - (long long)r.b * sq);
    r.tok = r.q;
  }
  return r;
}

// One warp per tile: max / min of alpha over the 128 rows of a query tile (rows of a packed-GQA tile interleave the
// G heads of a KV head, seqlen_info.py:262-265), or of delta over the 128 keys of a key tile. Rows / keys past
// the sequence count as 0, like the reference's masked loads (scheduler.py:1658-1691).
template <typename T>
__global__ void __launch_bounds__(256) gate_ext_kernel(GateExtParams p) {
  const int lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long n_alpha = (long long)p.B * p.hgrid * p.num_m_blocks;
  const long long n_delta = (long long)p.B * p.Hkv * p.n_tiles_k;
  if (item >= n_alpha + n_delta) return;
  float mx = -INFINITY, mn = INFINITY;
  float* dst;
  if (item < n_alpha) {
    const int mb = (int)(item % p.num_m_blocks);
    const int head = (int)((item / p.num_m_blocks) % p.hgrid);
    const int b = (int)(item / ((long long)p.num_m_blocks * p.hgrid));
    const int off_q = (p.flags & F_VARLEN_Q) ? p.cu_q[b] : 0;
    const int sq = (p.flags & F_USED_Q) ? p.used_q[b] : ((p.flags & F_VARLEN_Q) ? p.cu_q[b + 1] - off_q : p.sq);
    const T* base = reinterpret_cast<const T*>(p.alpha) + ((p.flags & F_VARLEN_Q) ? 0 : (long long)b * p.a_sb);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int offs_m = mb * 128 + j * 32 + lane;
      const int q_idx = offs_m / p.gpack;
      const int q_head = p.gpack > 1 ? head * p.G + (offs_m - q_idx * p.gpack) : head;
      const float v = q_idx < sq ? float(base[(long long)q_head * p.a_sh + off_q + q_idx]) : 0.f;
      mx = fmaxf(mx, v);
      mn = fminf(mn, v);
    }
    dst = p.gate_ws + 2 * item;
  } else {
    item -= n_alpha;
    const int n = (int)(item % p.n_tiles_k);
    const int hkv = (int)((item / p.n_tiles_k) % p.Hkv);
    const int b = (int)(item / ((long long)p.n_tiles_k * p.Hkv));
    const int off_k = (p.flags & F_VARLEN_K) ? p.cu_k[b] : 0;
    const int sk = (p.flags & F_USED_K) ? p.used_k[b] : ((p.flags & F_VARLEN_K) ? p.cu_k[b + 1] - off_k : p.sk);
    const T* base = reinterpret_cast<const T*>(p.delta);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = n * 128 + j * 32 + lane;
      float v = 0.f;
      if (k < sk) {
        long long e;
        if (p.flags & F_PAGED) {
          const int page = p.page_table[(long long)b * p.pt_stride + k / p.page_size];
          e = (long long)page * p.d_sb + (long long)hkv * p.d_sh + (k % p.page_size);
        } else {
          e = (long long)((p.flags & F_VARLEN_K) ? 0 : b) * p.d_sb + (long long)hkv * p.d_sh + off_k + k;
        }
        v = float(base[e]);
      }
      mx = fmaxf(mx, v);
      mn = fminf(mn, v);
    }
    dst = p.gate_ws + 2 * n_alpha + 2 * item;
  }
#pragma unroll
  for (int sft = 16; sft > 0; sft >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sft));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, sft));
  }
  if (lane == 0) *reinterpret_cast<float2*>(dst) = make_float2(mx, mn);
}

constexpr int PP_ITEMS = 1;  // (row, head) items per lane group in the pre / post passes (4 and 8 measured slower: fewer CTAs)

// head_dim / 8 lanes per (query row, head), 16-byte loads; also clears the row of the fp32 dQ accumulator.
// flash_sparse_attn/ops/triton/flash_bwd_preprocess.py:170-195.
template <typename T>
__global__ void __launch_bounds__(256) bwd_pre_kernel(BwdPreParams p) {
  const int lpr = p.head_dim_pad >> 3;  // lanes per row (8 or 16); lanes past the real head size idle
  const int lane = threadIdx.x & 31, sub = lane % lpr;
  const int groups = 32 / lpr;
  const long long first =
      (((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * groups + lane / lpr) * PP_ITEMS;
  const long long rows = p.varlen ? p.total_q : (long long)p.B * p.sq;
  const long long n_items = rows * p.heads;
  RowPos r[PP_ITEMS];
  uint4 a[PP_ITEMS], g[PP_ITEMS];
  bool live[PP_ITEMS];
#pragma unroll
  for (int u = 0; u < PP_ITEMS; ++u) {
    live[u] = first + u < n_items;
    r[u] = RowPos{0, 0, 0, 0};
    a[u] = g[u] = make_uint4(0, 0, 0, 0);
    if (live[u]) {
      r[u] = locate_row(first + u, p.heads, p.varlen, p.cu_q, p.B, p.sq);
      if (sub * 8 < p.head_dim) {
        const T* o = reinterpret_cast<const T*>(p.out) + (p.varlen ? 0 : (long long)r[u].b * p.o_sb) + r[u].tok * p.o_sm +
                     (long long)r[u].h * p.o_sh + sub * 8;
        const T* d = reinterpret_cast<const T*>(p.dout) + (p.varlen ? 0 : (long long)r[u].b * p.do_sb) +
                     r[u].tok * p.do_sm + (long long)r[u].h * p.do_sh + sub * 8;
        a[u] = *reinterpret_cast<const uint4*>(o);
        g[u] = *reinterpret_cast<const uint4*>(d);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < PP_ITEMS; ++u) {
    const uint32_t av[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, gv[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack2<T>(av[i]), y = unpack2<T>(gv[i]);
      acc += x.x * y.x + x.y * y.y;
    }
    for (int s = lpr >> 1; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (!live[u]) continue;
    const long long w = (long long)r[u].h * p.ws_sh + padded_row(p.varlen, p.cu_q, r[u].b, p.sq, r[u].q);
    if (p.dq_accum) {
      float4* z = reinterpret_cast<float4*>(p.dq_accum + w * p.head_dim_pad + sub * 8);
      z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (sub == 0) {
      const float lse = p.lse[(p.varlen ? 0 : (long long)r[u].b * p.l_sb) + (long long)r[u].h * p.l_sh + r[u].tok];
      float l2 = (lse == lse) ? lse * 1.4426950408889634f : 1e6f;
      l2 = fmaxf(l2, -1e6f);
      // both are stored negated: the main kernel then needs one packed fma / add per pair of entries
      p.lse2_ws[w] = -l2;
      p.dpsum_ws[w] = -acc;
      if (p.alpha_ws)
        reinterpret_cast<T*>(p.alpha_ws)[w] = reinterpret_cast<const T*>(
            p.alpha)[(p.varlen ? 0 : (long long)r[u].b * p.a_sb) + (long long)r[u].h * p.a_sh + r[u].tok];
    }
  }
}

// head_dim / 8 lanes per (query row, head). flash_sparse_attn/ops/triton/flash_bwd_postprocess.py:60-148.
template <typename T>
__global__ void __launch_bounds__(256) bwd_post_kernel(BwdPostParams p) {
  const int lpr = p.head_dim_pad >> 3;
  const int lane = threadIdx.x & 31, sub = lane % lpr;
  const int groups = 32 / lpr;
  const long long first =
      (((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * groups + lane / lpr) * PP_ITEMS;
  const long long rows = p.varlen ? p.total_q : (long long)p.B * p.sq;
  const long long n_items = rows * p.heads;
  RowPos r[PP_ITEMS];
  long long wrow[PP_ITEMS];
  float4 v0[PP_ITEMS], v1[PP_ITEMS];
  bool live[PP_ITEMS];
#pragma unroll
  for (int u = 0; u < PP_ITEMS; ++u) {
    live[u] = first + u < n_items;
    r[u] = RowPos{0, 0, 0, 0};
    wrow[u] = 0;
    v0[u] = v1[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live[u]) {
      r[u] = locate_row(first + u, p.heads, p.varlen, p.cu_q, p.B, p.sq);
      wrow[u] = (long long)r[u].h * p.ws_sh + padded_row(p.varlen, p.cu_q, r[u].b, p.sq, r[u].q);
      if (sub * 8 < p.head_dim) {
        const float4* src = reinterpret_cast<const float4*>(p.dq_accum + wrow[u] * p.head_dim_pad + sub * 8);
        v0[u] = __ldcs(src);  // read once: do not keep in cache
        v1[u] = __ldcs(src + 1);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < PP_ITEMS; ++u) {
    if (!live[u]) continue;
    if (p.da && sub == 0)
      reinterpret_cast<T*>(p.da)[(p.varlen ? 0 : (long long)r[u].b * p.da_sb) + (long long)r[u].h * p.da_sh + r[u].tok] =
          T(p.da_accum[wrow[u]] * p.scale);
    if (sub * 8 >= p.head_dim) continue;
    uint4 o;
    o.x = pack2<T>(v0[u].x * p.scale, v0[u].y * p.scale);
    o.y = pack2<T>(v0[u].z * p.scale, v0[u].w * p.scale);
    o.z = pack2<T>(v1[u].x * p.scale, v1[u].y * p.scale);
    o.w = pack2<T>(v1[u].z * p.scale, v1[u].w * p.scale);
    T* dst = reinterpret_cast<T*>(p.dq) + (p.varlen ? 0 : (long long)r[u].b * p.dq_sb) + r[u].tok * p.dq_sm +
             (long long)r[u].h * p.dq_sh + sub * 8;
    *reinterpret_cast<uint4*>(dst) = o;
  }
}

__global__ void __launch_bounds__(128) dq_order_kernel(DqOrderParams p) {
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= (long long)p.B * p.Hkv * p.num_m_blocks) return;
  const int m = (int)(item % p.num_m_blocks);
  const int hkv = (int)((item / p.num_m_blocks) % p.Hkv);
  const int b = (int)(item / ((long long)p.num_m_blocks * p.Hkv));
  const int off_q = (p.flags & F_VARLEN_Q) ? p.cu_q[b] : 0;
  const int off_k = (p.flags & F_VARLEN_K) ? p.cu_k[b] : 0;
  const int sq = (p.flags & F_USED_Q) ? p.used_q[b] : ((p.flags & F_VARLEN_Q) ? p.cu_q[b + 1] - off_q : p.sq);
  const int sk = (p.flags & F_USED_K) ? p.used_k[b] : ((p.flags & F_VARLEN_K) ? p.cu_k[b + 1] - off_k : p.sk);
  const bool causal = p.flags & F_CAUSAL, local = p.flags & F_LOCAL, split_qo = p.flags & F_SPLIT;
  FsaWindow w = {0, 0, 0, 0};
  if (local) {
    const int* wp = p.windows + (long long)hkv * p.win_stride;
    w.sink = wp[0];
    w.left = wp[1];
    w.right = wp[2];
    w.near_ = wp[3];
  }
  unsigned short count = 0;
  for (int n = p.n_tiles_k - 1; n >= 0; --n) {
    if (n * 128 >= sk) continue;
    bool visits = false;
    for (int s = 0; s < p.num_splits && !visits; ++s)
      visits = fsa_bwd_visits(fsa_bwd_schedule(sq, sk, n, s, w, p.num_splits, 128, 128, causal, local, split_qo), m,
                              causal, local);
    if (visits) p.order[(((long long)b * p.Hkv + hkv) * p.n_tiles_k + n) * p.num_m_blocks + m] = count++;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) flat_sum_kernel(FlatSumParams p) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= p.n) return;
  float acc = 0.f;
  for (int s = 0; s < p.num_splits; ++s) acc += p.partial[(long long)s * p.part_ss + i];
  reinterpret_cast<T*>(p.out)[i] = T(acc);
}

// One warp per (key row, head): sum the split partials in split order (fixed order, deterministic).
template <typename T>
__global__ void __launch_bounds__(256) split_sum_kernel(SplitSumParams p) {
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)p.rows * p.heads) return;
  const int h = (int)(item % p.heads);
  const long long row = item / p.heads;
  const int b = (int)(row / p.rows_per_batch);
  const long long n = row - (long long)b * p.rows_per_batch;
  const float* src = p.partial + (row * p.heads + h) * p.head_dim;
  T* dst = reinterpret_cast<T*>(p.out) + (long long)b * p.o_sb + n * p.o_sn + (long long)h * p.o_sh;
  for (int i = lane * 4; i < p.head_dim; i += 128) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < p.num_splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(src + (long long)s * p.part_ss + i);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    uint2 o;
    o.x = pack2<T>(acc.x, acc.y);
    o.y = pack2<T>(acc.z, acc.w);
    *reinterpret_cast<uint2*>(dst + i) = o;
  }
}

}  // namespace

cudaError_t launch_bwd_pre(const BwdPreParams& p, int dtype, cudaStream_t stream) {
  const long long rows = p.varlen ? p.total_q : (long long)p.B * p.sq;
  const long long items = rows * p.heads;
  if (items <= 0) return cudaSuccess;
  if (p.head_dim_pad != 64 && p.head_dim_pad != 128) return cudaErrorInvalidValue;
  const int per_block = 8 * (32 / (p.head_dim_pad >> 3)) * PP_ITEMS;
  const unsigned grid = (unsigned)((items + per_block - 1) / per_block);
  if (dtype == DT_BF16)
    bwd_pre_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else
    bwd_pre_kernel<__half><<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_bwd_post(const BwdPostParams& p, int dtype, cudaStream_t stream) {
  const long long rows = p.varlen ? p.total_q : (long long)p.B * p.sq;
  const long long items = rows * p.heads;
  if (items <= 0) return cudaSuccess;
  if (p.head_dim_pad != 64 && p.head_dim_pad != 128) return cudaErrorInvalidValue;
  const int per_block = 8 * (32 / (p.head_dim_pad >> 3)) * PP_ITEMS;
  const unsigned grid = (unsigned)((items + per_block - 1) / per_block);
  if (dtype == DT_BF16)
    bwd_post_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else
    bwd_post_kernel<__half><<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_gate_ext(const GateExtParams& p, int dtype, cudaStream_t stream) {
  const long long items = (long long)p.B * p.hgrid * p.num_m_blocks + (long long)p.B * p.Hkv * p.n_tiles_k;
  if (items <= 0) return cudaSuccess;
  const unsigned grid = (unsigned)((items + 7) / 8);
  if (dtype == DT_FP16)
    gate_ext_kernel<__half><<<grid, 256, 0, stream>>>(p);
  else
    gate_ext_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_dq_order(const DqOrderParams& p, cudaStream_t stream) {
  const long long items = (long long)p.B * p.Hkv * p.num_m_blocks;
  if (items <= 0) return cudaSuccess;
  dq_order_kernel<<<(unsigned)((items + 127) / 128), 128, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_flat_sum(const FlatSumParams& p, int dtype, cudaStream_t stream) {
  if (p.n <= 0) return cudaSuccess;
  const unsigned grid = (unsigned)((p.n + 255) / 256);
  if (dtype == DT_BF16)
    flat_sum_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else
    flat_sum_kernel<__half><<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_split_sum(const SplitSumParams& p, int dtype, cudaStream_t stream) {
  const long long items = (long long)p.rows * p.heads;
  if (items <= 0) return cudaSuccess;
  const unsigned grid = (unsigned)((items + 7) / 8);
  if (dtype == DT_BF16)
    split_sum_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  else
    split_sum_kernel<__half><<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_combine(const CombineParams& p, int dtype, cudaStream_t stream) {
  const long long items = (long long)p.rows * p.heads;
  if (items <= 0) return cudaSuccess;
  const int warps = 8;
  const unsigned grid = (unsigned)((items + warps - 1) / warps);
  if (p.head_dim % 4 != 0 || p.head_dim > 256) return cudaErrorInvalidValue;
  // VEC floats per lane, 32 lanes: head_dim <= 128 -> 4, <= 256 -> 8
  if (p.head_dim <= 128) {
    if (dtype == DT_BF16)
      combine_kernel<__nv_bfloat16, 4><<<grid, warps * 32, 0, stream>>>(p);
    else
      combine_kernel<__half, 4><<<grid, warps * 32, 0, stream>>>(p);
  } else {
    if (dtype == DT_BF16)
      combine_kernel<__nv_bfloat16, 8><<<grid, warps * 32, 0, stream>>>(p);
    else
      combine_kernel<__half, 8><<<grid, warps * 32, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace fsa
