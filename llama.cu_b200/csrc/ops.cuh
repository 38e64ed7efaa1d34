// Element-wise and row-wise kernels around the matrix products: embedding gather, RMSNorm,
// RoPE + KV-cache scatter, SiLU gate, logits softmax + argmax, the block-absmax quantizer and the
// synthetic-weight generator.
#pragma once
#include "common.cuh"

namespace lcu {

// x[r][:] = table[ids[r]][:]; u8 tables are de-quantised with half((q - 127.5f) * scale) (bs > 0)
int launch_embed(__half* x, int ldx, const void* table, const __half* scales, int bs, const short* ids, int n_ids, int dim,
                 cudaStream_t stream, int pdl);

// out[r][i] = weight[i] *h half(float(in[r][i]) * rsqrt(mean(in[r]^2) + eps))
int launch_rms_norm(__half* out, const __half* in, const __half* weight, int rows, int dim, float eps, cudaStream_t stream);

// (cos, sin) of pos / theta^(2i/head_dim) for first_pos <= pos < ctx_len, i < head_dim/2 (entry index pos * head_dim/2 + i)
int launch_rope_table(float2* table, int ctx_len, int head_dim, float theta, cudaStream_t stream, int first_pos = 0);

// Rotates q rows in place (row r at position *pos + r), rotates the new k rows into the head-major
// key cache and copies the new v rows into the head-major value cache.  The position of row 0 is
// *pos, or pos_value when pos == nullptr.
int launch_rope_scatter(__half* q, const __half* k_new, const __half* v_new, __half* k_cache, __half* v_cache,
                        const float2* rope, const int* pos, int pos_value, int m, int dim, int n_heads, int ctx_len,
                        cudaStream_t stream, int ld = 0);  // ld: row stride of q / k_new / v_new in elements (0 = dim)

// out = half(silu(float(a)) * float(b)) element-wise
int launch_silu(__half* out, const __half* a, const __half* b, size_t n, cudaStream_t stream);
// matmul_type 1 (reference llama_cu.cu:111-145): out(m,n) = lhs(m,k) . w(n,k)^T + beta * out, one thread per output element,
// terms added in index order (fp16 weights: binary32 sum; u8 weights, bs > 0: binary64 terms, sum rounded to binary32
// after every addition).  The on-GPU fp32-accumulate check for the fast kernels; slow by design.
int launch_matmul_nt_pedantic(__half* out, const __half* lhs, const void* w, const __half* scales, int bs, int m, int k, int n, float beta,
                              cudaStream_t stream);
// one warp waiting on an mbarrier that never completes: the wait expires (about a second) and stores its code in *err_word
int run_bounded_wait_probe(int* err_word, cudaStream_t stream);
// rows of [a | b]: out[r][j] = silu(ab[r][j]) * ab[r][f + j] for the fused w1|w3 prompt product
int launch_silu_rows(__half* out, const __half* ab, int m, int f, cudaStream_t stream);

// probs = softmax(logits / temp) rounded to half (written over `probs`), token = first index of the
// maximum probability.  Also advances the decode state for device-chained generation:
// *pos += advance; next_ids[0] = token; if log != nullptr, log[*step] = token and ++*step.
struct head_params {
  const __half* logits;
  __half* probs;  // may alias logits
  int n_vocab;
  float temperature;
  int* token_out;
  short* next_ids;
  int* pos;
  int advance;
  short* log;
  int* step;
  int log_capacity;
};
int launch_logits_head(const head_params& p, cudaStream_t stream, int pdl);
// one-block version of the same computation (any vocabulary size; used when the clustered kernel does not fit)
int launch_logits_head_single(const head_params& p, cudaStream_t stream, int pdl);

// Multinomial sampling over fp16 probabilities (the reference's commented-out discrete_distribution, llama_cu.cu:1202-1203):
// token i with probability p_i / sum(p), by inverting the cumulative sum at u * sum(p).  u comes from a counter-based
// generator (seed, *index) when index != nullptr, else from the argument.  Writes token_out / next_ids[0] and replaces
// the entry the logits head appended to the token log.
int launch_sample(const __half* probs, int n_vocab, uint64_t seed, const int* index, float u, int* token_out, short* next_ids, short* log,
                  const int* step, int log_capacity, cudaStream_t stream);
float sampler_uniform(uint64_t seed, int index);  // the u of launch_sample for (seed, index), on the host
// Context roll-over without a new prompt pass: cached rows [first, first + keep) of every head of one layer move to
// [0, keep); keys are rotated back by `first` positions, values move as they are.
int launch_rollover(__half* k_cache, __half* v_cache, int n_heads, int ctx_len, int head_dim, int first, int keep, float theta, cudaStream_t stream);

// block-absmax quantizer, bit-identical to the reference's (transform.cu:28-72)
int launch_quantize_absmax_uint8(uint8_t* q, __half* scales, const __half* in, size_t h, size_t w, int bs, cudaStream_t stream);
int launch_dequantize_absmax_uint8(__half* out, const __half* scales, const uint8_t* q, size_t h, size_t w, int bs,
                                   cudaStream_t stream);
// stats[0] = mean squared error, [1] = max abs error, [2] = mean abs error; partial is scratch of 3*256 floats
int launch_error_stats(float* stats, float* partial, const __half* a, const __half* b, size_t n, cudaStream_t stream);

// seeded synthetic data: out[i] = half(scale * z(seed, fnv1a(name), first + i)), z ~ approx N(0,1)
int launch_synth_fill(__half* out, size_t n, uint64_t seed, uint64_t stream_id, float scale, uint64_t first, cudaStream_t stream);
int launch_fill_half(__half* out, size_t n, float value, cudaStream_t stream);
uint64_t fnv1a64(const char* s);

// load the kernels of a decode step on the current device ahead of their first launch (ops.cu, head.cu)
int ops_preload();
int head_preload();

// pipeline helpers: *pos += inc; ids[0] = (short)*token (ids may live on a peer GPU)
int launch_bump_pos(int* pos, int inc, cudaStream_t stream);
int launch_token_to_ids(short* ids, const int* token, cudaStream_t stream);

// compares the quantizer's fast arithmetic with the reference's (IEEE division, roundf) for every (value, scale) pair of its
// domain on the device: number of pairs checked and number of differing bytes
int quantizer_arithmetic_check(unsigned long long* checked_out, unsigned long long* differences_out);
// silu_of_half (common.cuh) against a / (1 + expf(-a)) for all 65536 half-precision a: values compared, values that differ
int silu_arithmetic_check(unsigned long long* checked_out, unsigned long long* differences_out);

}  // namespace lcu
