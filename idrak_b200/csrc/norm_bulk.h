// Interface of the bulk-copy norm backward (norm_bulk.cu), used by the launcher in rowops.cu.
#pragma once
#include "common.cuh"

namespace idrak {

struct NormBulkParams {
  const __nv_bfloat16* dy;
  const __nv_bfloat16* x;
  const __nv_bfloat16* w;
  const float* mean;
  const float* rstd;
  const __nv_bfloat16* dres;     // gradient arriving through the residual path, added to dx; or null
  __nv_bfloat16* dx;
  float* dw_part;                // [grid, C]
  float* db_part;                // [grid, C] or null (RMSNorm)
  float* dxs_part;               // [grid, C] column sums of dx, or null
  int rows, C, rms, rows_per_block, stages;
  Status* st;
};

// How many CTAs (= rows of partial sums) a call of these sizes uses; 0 when the sizes do not fit the kernel.
int norm_bwd_bulk_blocks(int rows, int C);
int norm_bwd_bulk_launch(const NormBulkParams& base, int blocks, cudaStream_t stream);

}  // namespace idrak
