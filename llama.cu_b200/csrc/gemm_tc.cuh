// tcgen05 / tensor-memory GEMM for prompt processing with fp16 weights (gemm_tc.cu).
#pragma once
#include "common.cuh"
#include "gemv.cuh"

namespace lcu {

// shapes the kernel takes: N a multiple of 32, K a multiple of 64, 16-byte aligned rows
bool gemm_tc_supported(int m, int N, int K, int ldx, const void* lhs, const void* w, const void* out);

// out[m][N] = half(lhs[m][K] . w[N][K]^T + beta * out); out is dense (row stride N), lhs has row stride ldx.
// force_bn: 0 picks the widest one-SM tile (128 / 64 / 32 weight rows) that divides N.
// force_pair: -1 = the two-SM kernel (256-row tiles, 128 or 256 weight rows) whenever m > 128 and N allows it,
//             0 = never, 128 / 256 = always with that tile width.
// force_split: -1 = the one-SM kernel splits K over a cluster of 2 or 4 CTAs when its tiles would fill
//             less than half / a quarter of the SMs; 1 / 2 / 4 forces the factor (128-wide tiles only).
int launch_gemm_tc(__half* out, const __half* lhs, int ldx, const __half* w, int m, int N, int K, float beta, int* err, cudaStream_t stream,
                   int force_bn = 0, int force_pair = -1, int force_split = -1);

}  // namespace lcu
