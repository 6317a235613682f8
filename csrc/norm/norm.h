// Internal launch entry shared by the exported LayerNorm/RMSNorm backward symbols.
#pragma once
#include <cuda_runtime.h>

namespace st {
// CTAs (= number of partials) used by the entry point that owns its scratch (2 per SM) and by the
// regular entry point (as many as stay resident for this feature dimension).
int norm_bwd_grid(int rows);
int norm_bwd_grid_for(int rows, int d);
// Launches dx + partial dgamma/dbeta + the partial reduction on `s` with `grid` CTAs.  `scratch`
// holds 2 * grid * d floats.
int norm_bwd_launch(int rms, const void* dy, const void* x, const void* gamma, const float* mean,
                    const float* rstd, const void* dres, void* dx, float* dgamma, float* dbeta,
                    int accumulate, float* scratch, int rows, int d, int grid, cudaStream_t s);
}  // namespace st
