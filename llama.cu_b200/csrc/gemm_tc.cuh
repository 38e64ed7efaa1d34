// tcgen05 / tensor-memory GEMM for prompt processing with fp16 weights (gemm_tc.cu).
#pragma once
#include "common.cuh"
#include "gemv.cuh"

namespace lcu {

// shapes the kernel takes: N a multiple of 32, K a multiple of 64, 16-byte aligned rows
bool gemm_tc_supported(int m, int N, int K, int ldx, const void* lhs, const void* w, const void* out);

// out[m][N] = half(lhs[m][K] . w[N][K]^T + beta * out); out is dense (row stride N), lhs has row stride ldx.
// force_bn: 0 picks the widest tile (128 / 64 / 32 weight rows) that divides N.
int launch_gemm_tc(__half* out, const __half* lhs, int ldx, const __half* w, int m, int N, int K, float beta, int* err, cudaStream_t stream,
                   int force_bn = 0);

}  // namespace lcu
