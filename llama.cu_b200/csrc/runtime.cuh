// Host runtime of the inference core: model weights in per-GPU arenas, the KV cache and scratch of
// one context, and the forward pass (prefill and batch-1 decode) over a layer partition.
#pragma once
#include <memory>
#include <string>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace lcu {

// makes `dev` the current device for the lifetime of the object, then restores the previous one
struct device_guard {
  int prev = 0;
  explicit device_guard(int dev) {
    cudaGetDevice(&prev);
    cudaSetDevice(dev);
  }
  ~device_guard() { cudaSetDevice(prev); }
  device_guard(const device_guard&) = delete;
  device_guard& operator=(const device_guard&) = delete;
};

int* device_scratch_words();  // 64 zeroed ints on the current device (error word of the stand-alone operators)

#pragma pack(push, 1)
// The 40-byte `params` file of a weight directory (reference llama_cu.h:280-291, extract.py:30-41).
struct model_params {
  uint64_t magic;
  uint32_t fourcc;
  uint32_t dim;
  uint32_t multiple_of;
  uint32_t n_heads;
  uint32_t n_layers;
  uint32_t n_vocab;
  float norm_eps;
  uint8_t q_type;  // 0 fp16, 1 uint8 block-absmax
  uint8_t reserved0;
  uint16_t quantization_block_size;
};
#pragma pack(pop)
static_assert(sizeof(model_params) == 40, "params file layout");

constexpr uint64_t PARAMS_MAGIC = 0x000041524F525541ull;  // "AURORA\0\0"
constexpr uint32_t PARAMS_FOURCC = 0x414D4C4Cu;           // "LLMA"

uint32_t ffn_dim_of(const model_params& p);  // round_up(dim * 8 / 3, multiple_of), reference llama_cu.cu:765-767

// layer -> GPU map (reference llama_cu.h:301-314): embedding lives with the first layer, the final
// norm and the output matrix with the last one.
struct partition {
  std::vector<int> layer_gpus;
  int embedding_gpu() const { return layer_gpus.front(); }
  int output_gpu() const { return layer_gpus.back(); }
  std::vector<int> used_gpus() const;  // in order of first use
};

// true when every GPU holds one contiguous run of layers (a GPU does not reappear after another one was used)
bool partition_is_contiguous(const std::vector<int>& layer_gpus);

struct dev_matrix {
  void* w = nullptr;       // fp16 [rows][cols] or u8 [rows][cols]
  __half* sc = nullptr;    // fp16 [rows][cols / bs] when bs > 0
  size_t rows = 0, cols = 0;
  int bs = 0;
  size_t weight_bytes() const { return bs ? rows * cols : rows * cols * 2; }
  size_t scale_bytes() const { return bs ? rows * (cols / bs) * 2 : 0; }
};

struct layer_weights {
  dev_matrix wq, wk, wv, wo, w1, w2, w3;
  __half* attn_norm = nullptr;
  __half* ffn_norm = nullptr;
};

struct model {
  model_params params{};
  uint32_t ffn = 0;
  partition part;
  dev_matrix tok_embeddings, output;
  __half* norm = nullptr;
  std::vector<layer_weights> layers;
  std::vector<std::pair<int, void*>> arenas;  // (device, base) one allocation per GPU
  size_t weight_bytes_total = 0;
  // tensor-parallel shard: rows [tp_rank, tp_rank + 1) * rows / tp_size of every layer matrix and of the output matrix
  // (whole heads of wq / wk / wv); norm vectors and the embedding table are whole.  tp_size 1 = the whole model.
  int tp_rank = 0, tp_size = 1;

  // fp16 shadow of the u8 layer matrices, for prompt GEMMs.  A prompt of 9 rows or more runs its products on tcgen05
  // over fp16 operands; expanding every u8 matrix into scratch on every pass costs a 7B prompt about 100 us per layer
  // at any length (11.0 against 7.7 ms at 512 tokens).  Where the GPU has the room (the shadow takes 2 bytes per
  // weight: 13 GB for 7B, and is kept only if 6 GB stay free after it) the expansion is done once, by the same
  // kernel, so prompts read the same halves either way; decode keeps streaming the u8 matrices.  Set up when the
  // model's first context is created; refreshed by the next long prompt after a tensor was handed out (it may have
  // been rewritten).
  std::vector<layer_weights> shadow_layers;  // as `layers`, bs = 0, wq|wk|wv and w1|w3 back to back
  std::vector<std::pair<int, void*>> shadow_arenas;
  size_t shadow_bytes = 0;
  int shadow_state = 0;  // 0 not tried, 1 current, 2 stale, -1 does not fit / not wanted
  std::mutex shadow_mu;
  // true = usable (refreshed if stale); false = use the per-pass expansion.  Allocates only when told it may
  // (context creation): a prompt never does.
  bool shadow_ready(bool may_allocate);
  void shadow_touch();   // a tensor may have been written

  ~model();
  // allocates all tensors (uninitialised) according to params and the partition
  static int create(std::unique_ptr<model>& out, const model_params& p, const partition& part, int tp_rank = 0, int tp_size = 1);
  // reads a weight directory in the reference's layout (llama_cu.cu:929-984)
  int load_dir(const std::string& dir);
  // fills every tensor with seeded synthetic data (matrices ~ scale * z, norm weights 1.0); a
  // quantized model is generated in fp16 tensor by tensor and quantized on the device
  int fill_synthetic(uint64_t seed, float scale);
  // looks a tensor up by its file stem ("layers.3.attention.wq", "norm", ...): which 0 = values, 1 = scales
  int find_tensor(const std::string& name, int which, void** ptr, size_t* bytes, int* device);
  // writes params and every tensor as a weight directory in the reference's layout
  int save_dir(const std::string& dir);
};

// fp16 shadow of u8 models for prompts (model::shadow_ready): 1 (default) = where it fits, 0 = never
int& u8_shadow_mode();

// weight-directory loader: 1 (default) = pieces through two pinned buffers with asynchronous copies overlapping the file
// reads; 0 = the reference's way, a file mapping handed to one blocking copy from pageable memory (llama_cu.cu:699-702)
void set_loader_staged(int on);

// `transform quantize` (reference transform.cu:220-263): fp16 weight directory -> uint8 weight
// directory, one tensor at a time on the current device
int quantize_dir(const std::string& in_dir, const std::string& out_dir, int bs);

// greedy fill of the visible GPUs by free memory (reference llama_cu.cu:819-880); layer_gpus gets
// n_layers entries; fails if the model does not fit
int autopipe(const model_params& p, int context_len, std::vector<int>& layer_gpus);

// bytes of the scratch arena a context allocates on every GPU it uses, and of one layer's K and V caches
size_t context_scratch_bytes(const model_params& p, int context_len);
size_t context_kv_bytes_per_layer(const model_params& p, int context_len);

struct context_options {
  int context_len = 2048;
  float temperature = 0.9f;
  int use_graph = 1;     // replay one CUDA graph per decode step
  int use_pdl = 1;       // programmatic dependent launch between the kernels of a step
  int attn_cluster = 8;  // CTAs per (row, head) in decode attention
  int sampling = 0;      // 0 = greedy (first maximum, what the reference runs); 1 = multinomial over the fp16 probabilities
  uint64_t sample_seed = 0;
};

struct context_impl;  // defined in runtime.cu

struct context {
  ~context();
  static int create(std::unique_ptr<context>& out, model* m, const context_options& opt);
  void clear_tokens();
  size_t memory_usage() const;
  int tokens_left() const;
  int position() const;
  // feeds n new tokens (prefill when n > 1), returns the greedy next token in *token_out
  int next_token(const short* tokens, int n, int* token_out);
  // device-chained greedy decode: n_steps single-token steps starting from first_token, each
  // step's argmax feeding the next without a host round trip.  Returns the tokens and the device
  // time of the whole loop (CUDA events on the launching stream).
  int decode_chained(short first_token, int n_steps, short* tokens_out, float* ms_out);
  int read_probs(__half* out_host);    // softmax output of the last step (n_vocab halves)
  int read_hidden(__half* out_host);   // residual stream of the last token before the final norm
  int kernels_per_step() const;        // kernel launches of one decode step
  // times one decode kernel class over all layers in rotation (see lcu_bench_decode_kernel)
  int bench_kernel(int which, int reps, float* ms_per_launch, uint64_t* bytes_per_launch);
  int device_error();                  // non-zero if a kernel gave up on a bounded wait
  // 0 = greedy, 1 = multinomial sampling with a counter-based generator keyed by (seed, sequence length)
  int set_sampling(int mode, uint64_t seed);
  // Context roll-over without a new prompt pass: keeps the last `keep` cached positions (keys rotated back to
  // positions 0 .. keep-1, values moved) and continues at position `keep`.
  int rollover(int keep);
  std::unique_ptr<context_impl> impl;
};

}  // namespace lcu
