// Weight-streaming matrix-vector kernels for batch-1 decode (and up to 8 activation rows).
#pragma once
#include "common.cuh"

namespace lcu {

enum gemv_epilogue : int {
  EPI_PLAIN = 0,    // out[col][row] = half(acc + beta * float(out[col][row]))
  EPI_ROPE_KV = 1,  // three matrices wq|wk|wv: rotate q and k pairs, write k and v into the KV cache
  EPI_SILU = 2      // two matrices w1|w3 interleaved row by row: out[i] = half(silu(half(a_i)) * half(b_i))
};

struct gemv_params {
  // weights: up to three [rows_per_mat][K] matrices that share K; fp16, or u8 with fp16 scales [rows][K/bs]
  const void* w[3];
  const __half* sc[3];
  int n_mats;
  int rows_per_mat;
  int K;
  int bs;  // 0 = fp16 weights
  // activations: m (1..8) rows of K halves, row stride ldx.  With norm_w != nullptr (m == 1) the
  // row is RMS-normalised first: x_i <- norm_w_i *h half(x_i * rsqrt(mean(x^2) + eps)).
  const __half* x;
  int m;
  int ldx;
  const __half* norm_w;
  float eps;
  // EPI_PLAIN / EPI_SILU output
  __half* out;
  int ldo;
  float beta;
  __half* out_peer;     // EPI_PLAIN, optional: the same values are also stored here (another GPU's buffer: the pipeline hop)
  // EPI_ROPE_KV
  const int* pos;       // device scalar: position of the token being decoded
  __half* q_out;        // [dim]
  __half* k_cache;      // [n_heads][ctx_len][head_dim], rotated keys
  __half* v_cache;      // [n_heads][ctx_len][head_dim]
  const float2* rope;   // [ctx_len][head_dim/2] (cos, sin)
  int ctx_len;
  int head_dim;
  int* err;  // device error word
  // ---- tensor-parallel decode (m == 1; all zero on a single GPU).  Every GPU streams its own rows of the matrix and
  // owns the matching slice of the output vector; `out` and the peer pointers are pre-offset to that slice.
  __half* peer_out[7];     // EPI_PLAIN / EPI_SILU: every result is also stored into these buffers of other GPUs (peer stores)
  int n_peer_out;
  int* peer_flag[8];       // this GPU's flag word on each GPU that waits for the slice; written once all stores are out
  int n_peer_flag;
  int* done_count;         // local counter that finds the last CTA of the launch (zero between launches)
  const int* wait_flags;   // local flag words of the n_wait GPUs whose slices the activation row needs
  int n_wait;
  int wait_id;             // the prologue waits until every wait_flags[i] >= *seq * 1024 + wait_id
  int exchange_id;         // the value published is *seq * 1024 + exchange_id
  const int* seq;          // device scalar: number of the decode step in flight (monotonic over the context's life)
};

constexpr int TP_EXCHANGES_PER_STEP = 1024;  // bound of the exchange ids of one decode step

// Launch-shape knobs (defaults chosen by measurement; exposed for experiments)
struct gemv_tuning {
  int nstages = 4;      // shared-memory ring depth (16 rows x 1 KiB per stage)
  int ctas_per_sm = 2;  // grid = SM count x this
  int ctas_per_sm_int8 = 3;  // same for the factored u8 single-row kernel (more resident warps: it is latency-bound)
  int variant = 1;      // m == 1: 1 = per-warp row-pair kernel (gemv1.cu), 0 = 16-row-block kernel (gemv.cu)
  int int8_factored = 1;  // u8 weights: 1 = scale factored out of 64-weight groups (fast), 0 = the reference's per-weight rounding
  int warp_stages = 3;  // gemv1.cu: ring depth of every consumer warp (8 KiB per stage)
  int warp_stages_int8 = 3;  // same for the factored u8 kernel
  int consumer_warps_int8 = 0;  // factored u8 kernel: 0 = five consumer warps per CTA where three CTAs/SM do not fit, 4 = always four
  int prefetch_kb_per_cta = 32;  // L2 look-ahead issued by each CTA's producer at kernel start
};
gemv_tuning& gemv_tuning_ref();

// Launches the kernel on `stream`; pdl != 0 marks it as a programmatic dependent of the
// preceding launch (its weight stream starts while the previous kernel drains).
int launch_gemv(const gemv_params& p, int epilogue, cudaStream_t stream, int pdl);

int gemv_sm_count();
// rows (at most 8) of K activations that one launch with m > 1 can keep in shared memory; long rows (K = 22016: 4) take
// several passes
int gemv_max_rows(int K);

// loads all single-row kernels on the current device ahead of their first launch
int gemv_single_row_preload();
// consumer warps of the single-row launch these arguments lead to
int gemv_single_row_consumer_warps(const gemv_params& p);

// single-row kernel (gemv1.cu); called by launch_gemv after argument checks
int launch_gemv_single_row(const gemv_params& p, int epilogue, cudaStream_t stream, int pdl, int sms);

// pure-read probe with the same bulk-copy ring: mean milliseconds for one pass over `bytes` of HBM
int bench_read_ceiling(uint64_t bytes, int reps, int ncopy, float* ms_per_pass);  // ncopy bulk copies per 16 KiB stage

// bytes one launch must move at minimum (weights + scales + activations in + out)
size_t gemv_algorithmic_bytes(const gemv_params& p, int epilogue);

}  // namespace lcu
