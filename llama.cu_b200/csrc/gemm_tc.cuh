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

// Wide-tile variant with the K loop balanced over the SM pairs (gemm_tc_sk.cu): 256 x tile_n output tiles (tile_n 256 or
// 512, dividing N), any number of rows.  Partial sums of tiles shared between pairs go through a workspace kept per
// (device, stream) and are added in a fixed order.
// -1 (default) = launch_gemm_tc uses it, with 256- or 512-wide tiles, where its estimate says it wins; 256 / 512 =
// always, with that tile width, where it divides N; 0 = never
int& gemm_tc_sk_mode();
// more than 128 rows: the kernel launch_gemm_tc picks on a GPU of `sms` SMs - 0 whole tiles per SM pair, 256 / 512 the
// balanced kernel with that tile width.  Pure host arithmetic.
int gemm_tc_plan_long(int m, int N, int K, int sms);
// one-SM kernel, up to 128 rows, N a multiple of 128: the tile width (96 to 256) and split-K factor (1, 2, 4; 128-wide
// tiles only) launch_gemm_tc uses on a GPU of `sms` SMs.  Pure host arithmetic.
void gemm_tc_plan_short(int N, int K, int sms, int* tile_n, int* split);
// one-SM kernel: 64-wide k-blocks per stage and tensor copy (0 = as many of 4, 2, 1 as leave four stages)
int& tc_kb_per_stage();
// balanced pair kernel: k-blocks per stage and tensor copy (0 = 2)
int& sk_kb_per_stage();
bool gemm_tc_sk_supported(int m, int N, int K, int ldx, const void* lhs, const void* w, const void* out, int tile_n);
int launch_gemm_tc_sk(__half* out, const __half* lhs, int ldx, const __half* w, int m, int N, int K, float beta, int* err, cudaStream_t stream,
                      int tile_n);

// host walk of the balanced kernel's schedule for n_tiles tiles of nk K steps on C SM pairs: 0 = every K step of every tile
// runs once and the hand-over of partial sums is consistent (gemm_tc_sk.cu)
int gemm_tc_sk_check_schedule(int n_tiles, int nk, int C);

// w1|w3 and the SiLU gate as one launch (gemm_tc_sk.cu): out[m][f] = half(silu(half(lhs . w1^T)) * half(lhs . w3^T)) with
// w13 = [w1; w3] stacked ([2 f][K]); the same bits as the stacked product followed by the gate kernel.
// gemm_tc_gate_mode: -1 = when the estimate favours it, 256 / 512 = from 129 rows with that many accumulator columns per
// tile, 0 = never.  gemm_tc_gated_tile: the tile to use for this shape under that mode, 0 = run product and gate apart.
int& gemm_tc_gate_mode();
int gemm_tc_gated_tile(int m, int f, int K);
bool gemm_tc_gated_supported(int m, int f, int K, int ldx, const void* lhs, const void* w13, const void* out);
// tile_n: accumulator columns per tile (256: 128 output columns, the gate hidden under the next tile; 512: 256 output columns)
int launch_gemm_tc_gated(__half* out, const __half* lhs, int ldx, const __half* w13, int m, int f, int K, int* err, cudaStream_t stream,
                         int tile_n = 256);

}  // namespace lcu
