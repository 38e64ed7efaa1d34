// Multi-row matrix product out(m,N) = lhs(m,K) . W(N,K)^T + beta * out for prompt processing.
#pragma once
#include "common.cuh"
#include "runtime.cuh"

namespace lcu {

struct prefill_tuning {
  // fp16 weights: this many rows or more go to the tcgen05 GEMM (0 = never).  From 2 rows: measured, a 7B prompt of 2 to 8
  // tokens takes 4.2 to 6.7 ms through the multi-row GEMV (seven products per layer) and 3.3 ms through the stacked GEMMs.
  int tc_min_rows = 2;
  int tc_tile_n = 0;    // one-SM kernel: 0 = pick the tile width per shape; a multiple of 32 up to 256 forces it
  int u8_deq_min_rows = 2;   // u8 weights: this many rows or more take a dequantization pass + the tcgen05 GEMM (0 = never);
                             // (GEMV passes of 8 rows: 4.3 to 34 ms for 7B prompts of 2 to 47 tokens)
  int fuse = 1;         // fp16 prompts: wq|wk|wv and w1|w3 as one GEMM each over the stacked matrices
  int attn_tc = 2;      // prompt attention: 2 = one tcgen05 kernel per layer (scores in tensor memory), 1 = three tcgen05 kernels with the
                        // scores in an fp16 buffer (allocated by contexts created while this is 1), 0 = the fused warp-level kernel
  int attn_tc_min_rows = 384;  // rows from which the three-kernel path is used (its three launches per layer cost more below)
  int attn_fused_min_rows = 65;  // rows from which the one-kernel path is used (up to 64 rows: one tile of the warp-level kernel)
  int attn_tiles = 1;   // prompt attention: 1 = 64-row query tiles on tensor cores, 0 = the per-row decode kernel
  int tc_split = -1;    // one-SM kernel: -1 = split K over 2 / 4 CTAs when tiles are few, 1 / 2 / 4 = always that factor
  int tc_pair = -1;     // two-SM kernel: -1 = when m > 128, 0 = never, 128 / 256 = always with that tile width
};
prefill_tuning& prefill_tuning_ref();

// llama_cu::matmul_type (reference llama_cu.h:65-68, llama_cu.cu:28): 4 (the reference's tensor-core kernels) and 0 (its
// cuBLAS path) select the sm_100a kernels of this library; 1 selects the pedantic one-thread-per-output kernels for every
// matrix product, and a context then runs single-token steps through the unfused operator sequence of the prompt path.
int& matmul_type_ref();

// Dispatch: fp16 weights with at least tc_min_rows (2) rows of a shape the tcgen05 GEMM takes go to it (gemm_tc.cu);
// one row, other shapes, and u8 weights without scratch (in passes of 8 rows) go through the weight-streaming GEMV.
// lhs and out are dense row-major ([m][K], [m][N]); err is the device error word.
// deq / deq_halves: scratch for one dequantized matrix; with it, u8 weights and at least u8_deq_min_rows rows are
// expanded to fp16 (the values the reference's tile kernel builds in shared memory, llama_cu.cu:222-300) and
// go through the tcgen05 GEMM as well.
int matmul_rows(__half* out, const __half* lhs, const dev_matrix& w, int m, float beta, int* err, cudaStream_t stream, __half* deq = nullptr,
                size_t deq_halves = 0);

}  // namespace lcu
