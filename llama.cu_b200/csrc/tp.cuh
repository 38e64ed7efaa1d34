// Tensor-parallel batch-1 decode: every GPU streams its own rows of every matrix; activation slices travel by peer stores
// from the GEMV epilogues (see tp.cu).
#pragma once
#include <memory>
#include <string>

#include "runtime.cuh"

namespace lcu {

struct tp_impl;  // defined in tp.cu

// the row counts of the model must split evenly over the GPUs (whole heads, even row counts); host-only check
int tp_check_split(const model_params& p, int n_gpus);

// measurement switch, see tp.cu (0 = normal operation)
void tp_set_debug(int v);

struct tp_decoder {
  ~tp_decoder();
  // allocates the row shards of the model, the K/V caches of each GPU's heads and the activation rows on the named GPUs
  static int create(std::unique_ptr<tp_decoder>& out, const model_params& p, const int* gpus, int n_gpus, const context_options& opt);
  int fill_synthetic(uint64_t seed, float scale);  // the same values a whole model gets from the same seed
  int load_dir(const std::string& dir);            // every GPU reads its run of rows of every file of a weight directory
  // feeds n new tokens (a prompt runs as n single-token steps), returns the greedy next token
  int next_token(const short* tokens, int n, int* token_out);
  // n_steps greedy steps chained on the devices; device time of the loop from CUDA events on GPU 0's stream
  int decode_chained(short first_token, int n_steps, short* tokens_out, float* ms_out);
  int read_probs(__half* out_host);
  void clear_tokens();
  int tokens_left() const;
  int n_gpus() const;
  int kernels_per_step() const;
  size_t weight_bytes_per_gpu() const;
  size_t memory_usage() const;
  std::unique_ptr<tp_impl> impl;
};

}  // namespace lcu
