// Internal launch entry shared by the exported LayerNorm/RMSNorm backward symbols.
#pragma once
#include <cuda_runtime.h>

namespace st {
// Number of CTAs the backward kernel uses for `rows` rows (also the number of partials).
int norm_bwd_grid(int rows);
// Launches dx + partial dgamma/dbeta + the partial reduction on `s`.  `scratch` holds
// 2 * norm_bwd_grid(rows) * d floats.
int norm_bwd_launch(int rms, const void* dy, const void* x, const void* gamma, const float* mean,
                    const float* rstd, const void* dres, void* dx, float* dgamma, float* dbeta,
                    int accumulate, float* scratch, int rows, int d, cudaStream_t s);
}  // namespace st
