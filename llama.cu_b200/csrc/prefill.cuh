// Multi-row matrix product out(m,N) = lhs(m,K) . W(N,K)^T + beta * out for prompt processing.
#pragma once
#include "common.cuh"
#include "runtime.cuh"

namespace lcu {

// Dispatch: up to 8 rows go through the weight-streaming GEMV; more rows are processed in tiles.
// lhs and out are dense row-major ([m][K], [m][N]); err is the device error word.
int matmul_rows(__half* out, const __half* lhs, const dev_matrix& w, int m, float beta, int* err, cudaStream_t stream);

}  // namespace lcu
