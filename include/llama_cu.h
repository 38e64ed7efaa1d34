// C++ interface of the B200-native llama.cu inference core.
//
// Source-compatible with the public part of the reference's llama_cu.h (eiz/llama.cu): a program
// written against that header - the reference's own main.cpp for one - compiles against this one
// and links with libllama_cu_b200.so unchanged.  Each declaration names the reference lines it
// mirrors.  Everything here is a thin layer over the C ABI in llama_cu_c.h; the device code is
// sm_100a only and there is no CPU fallback.
//
// Not carried over: the LLAMA_CU_IMPLEMENTATION section of the reference header (tensor4d,
// gpu_buffer, generic_tensor, CHECK_CUDA ...).  Those are internals of the reference's own
// translation units; the equivalent operator seam (matmul_nt and friends) is exported through
// llama_cu_c.h on plain device pointers instead.
#pragma once

#if __cplusplus < 201703L
#error "C++17 or higher is required"
#endif

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

namespace llama_cu {

// reference llama_cu.h:65-68.  0 (cuBLAS in the reference) and 4 (its tensor-core kernels) both
// select the native sm_100a kernels; 1 (its naive kernels) is accepted and means the same.
extern int matmul_type;

// reference llama_cu.h:392, llama_cu.cu:1525-1542: prints the device properties
void initialize();

// reference llama_cu.h:70-95: read-only file mapping, read-write file of a given size, or
// anonymous memory.  Move-only.
class mapped_buffer {
 public:
  mapped_buffer();
  explicit mapped_buffer(std::string const& path);
  mapped_buffer(std::string const& path, size_t size);
  explicit mapped_buffer(size_t size);
  ~mapped_buffer();
  mapped_buffer(mapped_buffer&& other);
  mapped_buffer& operator=(mapped_buffer&& other);
  mapped_buffer(mapped_buffer const&) = delete;
  mapped_buffer& operator=(mapped_buffer const&) = delete;
  bool is_ok() const { return base_ != nullptr; }
  void* data() const { return base_; }
  size_t size() const { return length_; }

 private:
  void release();
  void* base_ = nullptr;
  size_t length_ = 0;
  int file_ = -1;
};

// reference llama_cu.h:136-139
enum class quantization_type : uint8_t { fp16, uint8 };

#define LLAMA_CU_MAGIC 0x000041524F525541       // "AURORA\0\0"
#define LLAMA_CU_MODEL_FOURCC_LLAMA 0x414D4C4C  // "LLMA"

// reference llama_cu.h:280-299: the 40-byte params record, read by raw cast in main.cpp:34
struct llama_params {
  uint64_t magic;
  uint32_t fourcc;
  uint32_t dim;
  uint32_t multiple_of;
  uint32_t n_heads;
  uint32_t n_layers;
  uint32_t n_vocab;
  float norm_eps;
  quantization_type q_type;
  uint8_t reserved0[1];
  uint16_t quantization_block_size;

  bool load(mapped_buffer const& buffer);
  uint32_t ffn_dim() const;
  size_t layer_size() const;
  size_t embedding_size() const;
  size_t output_size() const;
  size_t shared_context_memory_size(size_t context_len) const;
  size_t kv_cache_size(size_t context_len) const;
};
static_assert(sizeof(llama_params) == 40, "llama_params must match the params file");

// reference llama_cu.h:301-314: layer -> GPU map with public fields
struct llama_partition {
  llama_partition() {}
  void use_default(llama_params const& params);
  void autopipe(llama_params const& params, size_t context_len);
  bool is_valid();
  void debug_print();
  std::vector<int> used_gpus;
  int embedding_gpu{-1};
  std::vector<int> layer_gpus;
  int output_gpu{-1};
};

// reference llama_cu.h:316-327
struct llama_token {
  short id;
  float score;
  std::string text;
};

struct llama_vocabulary {
  explicit llama_vocabulary(mapped_buffer const& buffer);
  std::vector<short> tokenize(std::string_view text, bool bos);
  std::unordered_map<std::string, llama_token*> token_lookup;
  std::vector<llama_token> tokens;
};

// reference llama_cu.h:329-358: greedy highest-score pair merging with byte fallback
class llama_tokenizer {
 public:
  explicit llama_tokenizer(llama_vocabulary const& vocab) : vocab_(vocab) {}
  void tokenize(std::string_view text, std::vector<short>& output);

 private:
  llama_vocabulary const& vocab_;
};

struct llama_model_impl;

// reference llama_cu.h:362-372
struct llama_model {
  static std::unique_ptr<llama_model> load(llama_params params, llama_partition partition, std::string const& path);
  virtual ~llama_model() = default;
  llama_params params;
  llama_partition partition;

 protected:
  llama_model(llama_params params, llama_partition partition) : params(params), partition(partition) {}
};

// reference llama_cu.h:374-390
struct llama_context {
  static std::unique_ptr<llama_context> create(llama_model* model, int context_len = 2048, float temperature = 0.9);
  virtual ~llama_context() = default;
  virtual void clear_tokens() = 0;
  virtual size_t context_memory_usage() = 0;
  virtual short next_token(std::vector<short> const& new_tokens) = 0;
  size_t tokens_left() { return context_len_ - start_pos_; }

 protected:
  llama_context(llama_model_impl* model, int context_len, float temperature)
      : model_(model), context_len_(context_len), temperature_(temperature) {}
  llama_model_impl* model_;
  int context_len_;
  int start_pos_{0};
  float temperature_;
};

}  // namespace llama_cu
