// Multi-row matrix product out(m,N) = lhs(m,K) . W(N,K)^T + beta * out for prompt processing.
#pragma once
#include "common.cuh"
#include "runtime.cuh"

namespace lcu {

struct prefill_tuning {
  int tc_min_rows = 9;  // fp16 weights: this many rows or more go to the tcgen05 GEMM (0 = never)
  int tc_tile_n = 0;    // 0 = pick the tile width per shape; 32 / 64 / 128 forces it
};
prefill_tuning& prefill_tuning_ref();

// Dispatch: fp16 weights with more than 8 rows go to the tcgen05 GEMM (gemm_tc.cu); up to 8 rows, and
// u8 weights in passes of 8 rows, go through the weight-streaming GEMV.
// lhs and out are dense row-major ([m][K], [m][N]); err is the device error word.
int matmul_rows(__half* out, const __half* lhs, const dev_matrix& w, int m, float beta, int* err, cudaStream_t stream);

}  // namespace lcu
