// Fused attention over the head-major fp16 KV cache (decode and prefill rows).
#pragma once
#include <math_constants.h>
#include "common.cuh"

namespace lcu {

struct attn_params {
  const __half* q;        // [m][ldq] rotated queries
  int ldq;
  const __half* k_cache;  // [n_heads][ctx_len][head_dim] rotated keys
  const __half* v_cache;  // [n_heads][ctx_len][head_dim]
  __half* out;            // [m][ldo]
  int ldo;
  const int* pos;         // device scalar: position of query row 0 (row r attends to 0 .. pos + r);
  int pos_value;          // used instead when pos == nullptr
  int ctx_len;
  int n_heads;
  int head_dim;
  int* err;               // device error word for the bounded waits of the streaming kernel (nullptr: that kernel is not used)
  // ---- tensor-parallel decode (cluster kernels only; all zero on a single GPU): this GPU's heads are a slice of the
  // attention row; the slice is also stored into the other GPUs' rows and then published like a GEMV's (gemv.cuh)
  __half* peer_out[7];
  int n_peer_out;
  int* peer_flag[8];
  int n_peer_flag;
  int* done_count;        // local counter that finds the last (row, head) of the launch (zero between launches)
  const int* seq;
  int exchange_id;
  int exchanges_per_step;
};

// m query rows; `cluster` CTAs (1, 2, 4 or 8) share one (row, head); max_T bounds pos + m so that
// shared memory can be sized without reading the device position.
int launch_attention(const attn_params& p, int m, int cluster, int max_T, cudaStream_t stream, int pdl);

int attention_preload();

// -1 = rows through a shared-memory ring of bulk copies when a CTA's slice can exceed 64 rows (default), 0 = never, 1 = always
void attention_set_stream_mode(int mode);

// Prompt rows: 64-row query tiles on tensor cores (attention_prefill.cu); same arithmetic, no clusters.
int launch_attention_prefill(const attn_params& p, int m, int max_T, cudaStream_t stream);

// Prompt rows on tcgen05 (attention_tc.cu): scores to a [heads][m_cap][round_up(ctx_len, 128)] fp16 buffer, softmax in
// place, probabilities times V.  attention_tc_scratch_halves gives the buffer size in elements.
size_t attention_tc_scratch_halves(int n_heads, int m_cap, int ctx_len);
int launch_attention_tc(const attn_params& p, int m, int max_T, __half* scores, int m_cap, cudaStream_t stream);

// Prompt rows on tcgen05 in one kernel (attention_fused.cu): scores, softmax and probabilities x V per (128-row tile,
// head) with the scores in tensor memory and the probabilities in shared memory; no score buffer.
int launch_attention_fused(const attn_params& p, int m, int max_T, cudaStream_t stream);

// one-kernel prompt attention: CTA order, 0 = a head's row tiles together (long first), 1 = all heads' long tiles first
int& attn_fused_order();

}  // namespace lcu
