// Parameter blocks and launchers of the helper kernels (internal).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "fsa_params.h"

namespace fsa {

// out_partial [num_splits, rows, heads, head_dim] fp32 (contiguous), lse_partial addressed as
// split*lp_ss + head*lp_sh + row (base-2 log-sum-exp). `rows` = batch*seqlen (or packed total);
// rows_per_batch splits a row index into (batch, position) for the strided final tensors.
struct CombineParams {
  const float* out_partial;
  const float* lse_partial;
  void* out;
  float* lse;
  long long op_ss, lp_ss, lp_sh;
  long long o_sb, o_sm, o_sh;
  long long l_sb, l_sh;
  int rows, rows_per_batch, heads, head_dim, num_splits;
};

cudaError_t launch_combine(const CombineParams& p, int dtype, cudaStream_t stream);
cudaError_t launch_fwd(const FwdKernelParams& p, int kind, int dtype, int head_dim, cudaStream_t stream);

}  // namespace fsa
