// The llama_cu:: C++ classes of include/llama_cu.h on top of the internal runtime.
#define LLAMA_CU_IMPLEMENTATION
#include "../../include/llama_cu.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cassert>
#include <cstdio>
#include <cstring>
#include <queue>

#include "prefill.cuh"
#include "runtime.cuh"

namespace llama_cu {

int matmul_type = 4;

void initialize() {
  int device = 0;
  cudaDeviceProp prop;
  if (cudaGetDevice(&device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    fprintf(stderr, "llama_cu: no CUDA device available\n");
    return;
  }
  printf("Device name: %s\n", prop.name);
  printf("Number of SMs: %d\n", prop.multiProcessorCount);
  printf("Shared mem size per SM: %zu bytes\n", prop.sharedMemPerMultiprocessor);
  printf("Shared mem size per block: %zu bytes\n", prop.sharedMemPerBlock);
  printf("Shared mem size per block (optin): %zu bytes\n", prop.sharedMemPerBlockOptin);
  printf("Shared mem size per block (reserved): %zu bytes\n", prop.reservedSharedMemPerBlock);
  printf("L2 cache size: %d bytes\n", prop.l2CacheSize);
}

// ------------------------------------------------------------------ mapped_buffer
mapped_buffer::mapped_buffer() {}
mapped_buffer::mapped_buffer(std::string const& path) {
  file_ = open(path.c_str(), O_RDONLY);
  if (file_ < 0) return;
  struct stat st;
  if (fstat(file_, &st) == 0 && st.st_size > 0) {
    void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_SHARED, file_, 0);
    if (p != MAP_FAILED) {
      base_ = p;
      length_ = (size_t)st.st_size;
      return;
    }
  }
  release();
}
mapped_buffer::mapped_buffer(std::string const& path, size_t size) {
  file_ = open(path.c_str(), O_RDWR | O_CREAT | O_TRUNC, 0644);
  if (file_ < 0) return;
  if (ftruncate(file_, (off_t)size) == 0) {
    void* p = mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_SHARED, file_, 0);
    if (p != MAP_FAILED) {
      base_ = p;
      length_ = size;
      return;
    }
  }
  release();
}
mapped_buffer::mapped_buffer(size_t size) {
  void* p = mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (p != MAP_FAILED) {
    base_ = p;
    length_ = size;
  }
}
void mapped_buffer::release() {
  if (base_) munmap(base_, length_);
  if (file_ >= 0) close(file_);
  base_ = nullptr;
  length_ = 0;
  file_ = -1;
}
mapped_buffer::~mapped_buffer() { release(); }
mapped_buffer::mapped_buffer(mapped_buffer&& other) { *this = std::move(other); }
mapped_buffer& mapped_buffer::operator=(mapped_buffer&& other) {
  if (this != &other) {
    release();
    base_ = other.base_;
    length_ = other.length_;
    file_ = other.file_;
    other.base_ = nullptr;
    other.length_ = 0;
    other.file_ = -1;
  }
  return *this;
}

// ------------------------------------------------------------------ scoped_gpu, gpu_buffer (reference llama_cu.cu:691-736)
scoped_gpu::scoped_gpu(int device) {
  CHECK_CUDA(cudaGetDevice(&prev_device_));
  CHECK_CUDA(cudaSetDevice(device));
}
scoped_gpu::~scoped_gpu() { CHECK_CUDA(cudaSetDevice(prev_device_)); }

void gpu_buffer_view::copy_from(mapped_buffer const& buffer) {
  assert(buffer.size() == size_);
  CHECK_CUDA(cudaMemcpyAsync(dev_ptr_, buffer.data(), size_, cudaMemcpyHostToDevice));
}
void gpu_buffer_view::copy_from(void const* buffer, size_t size) {
  assert(size <= size_);
  CHECK_CUDA(cudaMemcpyAsync(dev_ptr_, buffer, size, cudaMemcpyHostToDevice));
}
void gpu_buffer_view::copy_to(void* buffer, size_t size) {
  assert(size <= size_);
  CHECK_CUDA(cudaMemcpy(buffer, dev_ptr_, size, cudaMemcpyDeviceToHost));
}
gpu_buffer::gpu_buffer(size_t size) {
  CHECK_CUDA(cudaMalloc(&dev_ptr_, size ? size : 1));
  size_ = size;
}
gpu_buffer::gpu_buffer(gpu_buffer&& other) : gpu_buffer_view(other.dev_ptr_, other.size_) {
  other.dev_ptr_ = nullptr;
  other.size_ = 0;
}
gpu_buffer& gpu_buffer::operator=(gpu_buffer&& other) {
  if (this == &other) return *this;
  if (dev_ptr_) CHECK_CUDA(cudaFree(dev_ptr_));
  dev_ptr_ = other.dev_ptr_;
  size_ = other.size_;
  other.dev_ptr_ = nullptr;
  other.size_ = 0;
  return *this;
}
gpu_buffer::~gpu_buffer() {
  if (dev_ptr_) CHECK_CUDA(cudaFree(dev_ptr_));
}

// ------------------------------------------------------------------ the operator seam (reference llama_cu.cu:1463-1523)
namespace {
void seam_matmul(tensor4d_view<__half>& out, tensor4d_view<__half>& lhs, lcu::dev_matrix const& w, __half beta, cudaStream_t stream) {
  // the reference's kernels index rows densely and ignore the strides; the same contract holds here
  assert(lhs.w == w.cols && out.w == w.rows && out.h >= lhs.h);
  lcu::matmul_type_ref() = matmul_type;
  if (lcu::matmul_rows(out.data(), lhs.data(), w, (int)lhs.h, __half2float(beta), lcu::device_scratch_words(), stream) != lcu::LCU_OK) {
    fprintf(stderr, "matmul_nt: %s\n", lcu::last_error());
    raise(SIGSEGV);  // contract violations and CUDA errors are fatal in the reference too (assert / CHECK_CUDA)
  }
}
}  // namespace

void matmul_nt(tensor4d_view<__half> out, tensor4d_view<__half> lhs, tensor4d_view<__half> rhs, __half beta, cudaStream_t stream) {
  lcu::dev_matrix w;
  w.w = rhs.data();
  w.rows = rhs.h;
  w.cols = rhs.w;
  seam_matmul(out, lhs, w, beta, stream);
}
void matmul_nt(tensor4d_view<__half> out, tensor4d_view<__half> lhs, generic_tensor& rhs, __half beta, cudaStream_t stream) {
  if (!rhs.is_quantized()) return matmul_nt(out, lhs, rhs.as_fp16().view(), beta, stream);
  quantized_tensor& q = rhs.as_quantized();
  lcu::dev_matrix w;
  w.w = q.q_values.data();
  w.sc = q.scales.data();
  w.rows = q.q_values.h;
  w.cols = q.q_values.w;
  w.bs = q.quantization_block_size;
  seam_matmul(out, lhs, w, beta, stream);
}

// ------------------------------------------------------------------ llama_params
namespace {
lcu::model_params to_internal(llama_params const& p) {
  lcu::model_params q;
  static_assert(sizeof(q) == sizeof(p), "params layouts must agree");
  memcpy(&q, &p, sizeof(q));
  return q;
}
size_t matrix_bytes(llama_params const& p, size_t rows, size_t cols) {
  if (p.q_type == quantization_type::uint8) return rows * cols + rows * (cols / p.quantization_block_size) * 2;
  return rows * cols * 2;
}
}  // namespace

bool llama_params::load(mapped_buffer const& buffer) {
  if (buffer.size() != sizeof(llama_params)) return false;
  llama_params tmp;
  memcpy(&tmp, buffer.data(), sizeof(tmp));
  if (tmp.magic != LLAMA_CU_MAGIC || tmp.fourcc != LLAMA_CU_MODEL_FOURCC_LLAMA) return false;
  *this = tmp;
  return true;
}
uint32_t llama_params::ffn_dim() const { return lcu::ffn_dim_of(to_internal(*this)); }
// Bytes of one layer's weights (norms + 7 matrices).  The reference's own figure for uint8 models
// leaves out part of the scale bytes (llama_cu.cu:775-779); this one counts them all.
size_t llama_params::layer_size() const {
  const size_t d = dim, f = ffn_dim();
  return 2 * d * 2 + 4 * matrix_bytes(*this, d, d) + 2 * matrix_bytes(*this, f, d) + matrix_bytes(*this, d, f);
}
size_t llama_params::embedding_size() const { return matrix_bytes(*this, n_vocab, dim); }
size_t llama_params::output_size() const { return matrix_bytes(*this, n_vocab, dim) + (size_t)dim * 2; }
// what a context allocates on every GPU it uses: activations for context_len rows, the prompt path's score and
// dequantization buffers, tables (the same figure context::create and the partitioner use)
size_t llama_params::shared_context_memory_size(size_t context_len) const {
  return lcu::context_scratch_bytes(to_internal(*this), (int)context_len);
}
size_t llama_params::kv_cache_size(size_t context_len) const { return context_len * dim * 2 * 2; }

// ------------------------------------------------------------------ llama_partition
void llama_partition::use_default(llama_params const& params) {
  used_gpus = {0};
  embedding_gpu = 0;
  output_gpu = 0;
  layer_gpus.assign(params.n_layers, 0);
}
void llama_partition::autopipe(llama_params const& params, size_t context_len) {
  std::vector<int> lg;
  layer_gpus.clear();
  used_gpus.clear();
  embedding_gpu = output_gpu = -1;
  if (lcu::autopipe(to_internal(params), (int)context_len, lg) != lcu::LCU_OK) {
    layer_gpus.assign(params.n_layers, -1);
    return;
  }
  layer_gpus = lg;
  embedding_gpu = lg.front();
  output_gpu = lg.back();
  for (int g : lg)
    if (std::find(used_gpus.begin(), used_gpus.end(), g) == used_gpus.end()) used_gpus.push_back(g);
}
bool llama_partition::is_valid() {
  if (embedding_gpu < 0 || output_gpu < 0 || layer_gpus.empty()) return false;
  return std::all_of(layer_gpus.begin(), layer_gpus.end(), [](int g) { return g >= 0; });
}
void llama_partition::debug_print() {
  fprintf(stderr, "Model partition:\n  Embedding GPU: %d\n  Output GPU: %d\n  Layers:\n    ", embedding_gpu, output_gpu);
  for (size_t i = 0; i < layer_gpus.size(); ++i) {
    fprintf(stderr, "% 3zu: %d ", i, layer_gpus[i]);
    if (i % 8 == 7 && i + 1 != layer_gpus.size()) fprintf(stderr, "\n    ");
  }
  fprintf(stderr, "\n");
}

// ------------------------------------------------------------------ vocabulary / tokenizer
// vocab file (extract.py:44-61): int32 count, then count x {int32 offset, float score}, then the
// zero-terminated pieces.  Ids 3..258 are the byte tokens (reference llama_cu.cu:1331-1337).
llama_vocabulary::llama_vocabulary(mapped_buffer const& buffer) {
  const char* base = static_cast<const char*>(buffer.data());
  uint32_t count = 0;
  memcpy(&count, base, 4);
  tokens.resize(count);
  for (uint32_t i = 0; i < count; ++i) {
    uint32_t offset;
    float score;
    memcpy(&offset, base + 4 + 8 * (size_t)i, 4);
    memcpy(&score, base + 8 + 8 * (size_t)i, 4);
    llama_token& t = tokens[i];
    t.id = (short)i;
    t.score = score;
    if (i >= 3 && i < 259)
      t.text = std::string(1, (char)(i - 3));
    else
      t.text = std::string(base + offset);
  }
  for (uint32_t i = 259; i < count; ++i) token_lookup.emplace(tokens[i].text, &tokens[i]);
}

std::vector<short> llama_vocabulary::tokenize(std::string_view text, bool bos) {
  std::vector<short> out;
  if (bos) out.push_back(1);
  if (text.empty()) return out;
  llama_tokenizer tk(*this);
  if (text.front() == ' ') {
    tk.tokenize(text, out);
  } else {  // sentencepiece's dummy prefix (reference llama_cu.cu:1353-1358)
    std::string padded(" ");
    padded.append(text);
    tk.tokenize(padded, out);
  }
  return out;
}

// Pair merging: split into UTF-8 characters, repeatedly join the adjacent pair whose concatenation
// is the highest-scoring vocabulary piece (leftmost on ties), emit bytes for what is left over
// (reference llama_cu.cu:1365-1437).
void llama_tokenizer::tokenize(std::string_view text, std::vector<short>& output) {
  struct piece {
    size_t begin, len;
    int prev, next;
  };
  struct candidate {
    float score;
    int left, right;
    size_t len;
    bool operator<(candidate const& o) const { return score < o.score || (score == o.score && left > o.left); }
  };
  std::vector<piece> pieces;
  for (size_t at = 0; at < text.size();) {
    const unsigned char lead = (unsigned char)text[at];
    size_t n = lead < 0xC0 ? 1 : lead < 0xE0 ? 2 : lead < 0xF0 ? 3 : 4;
    n = std::min(n, text.size() - at);
    pieces.push_back({at, n, (int)pieces.size() - 1, -1});
    at += n;
  }
  for (size_t i = 0; i + 1 < pieces.size(); ++i) pieces[i].next = (int)i + 1;
  std::priority_queue<candidate> heap;
  auto consider = [&](int l, int r) {
    if (l < 0 || r < 0) return;
    const size_t len = pieces[l].len + pieces[r].len;
    auto hit = vocab_.token_lookup.find(std::string(text.substr(pieces[l].begin, len)));
    if (hit != vocab_.token_lookup.end()) heap.push({hit->second->score, l, r, len});
  };
  for (size_t i = 1; i < pieces.size(); ++i) consider((int)i - 1, (int)i);
  while (!heap.empty()) {
    const candidate c = heap.top();
    heap.pop();
    piece& a = pieces[c.left];
    piece& b = pieces[c.right];
    if (a.len == 0 || b.len == 0 || a.len + b.len != c.len) continue;  // stale entry
    a.len += b.len;
    b.len = 0;
    a.next = b.next;
    if (b.next >= 0) pieces[b.next].prev = c.left;
    consider(a.prev, c.left);
    consider(c.left, a.next);
  }
  for (int i = pieces.empty() ? -1 : 0; i != -1; i = pieces[i].next) {
    const std::string_view s = text.substr(pieces[i].begin, pieces[i].len);
    auto hit = vocab_.token_lookup.find(std::string(s));
    if (hit != vocab_.token_lookup.end()) {
      output.push_back(hit->second->id);
    } else {
      for (unsigned char ch : s) output.push_back((short)(ch + 3));
    }
  }
}

// ------------------------------------------------------------------ model / context
struct llama_model_impl : public llama_model {
  llama_model_impl(llama_params p, llama_partition part) : llama_model(p, part) {}
  std::unique_ptr<lcu::model> core;
};

std::unique_ptr<llama_model> llama_model::load(llama_params params, llama_partition partition, std::string const& path) {
  auto m = std::make_unique<llama_model_impl>(params, partition);
  lcu::partition part;
  part.layer_gpus = partition.layer_gpus;
  if (lcu::model::create(m->core, to_internal(params), part) != lcu::LCU_OK || m->core->load_dir(path) != lcu::LCU_OK) {
    fprintf(stderr, "%s\n", lcu::last_error());
    return nullptr;
  }
  return m;
}

namespace {
struct context_on_b200 final : public llama_context {
  context_on_b200(llama_model_impl* model, int context_len, float temperature) : llama_context(model, context_len, temperature) {
    lcu::context_options opt;
    opt.context_len = context_len;
    opt.temperature = temperature;
    if (lcu::context::create(core, model->core.get(), opt) != lcu::LCU_OK) {
      fprintf(stderr, "%s\n", lcu::last_error());
      abort();
    }
  }
  void clear_tokens() override {
    core->clear_tokens();
    start_pos_ = 0;
  }
  size_t context_memory_usage() override { return core->memory_usage(); }
  short next_token(std::vector<short> const& new_tokens) override {
    assert(new_tokens.size() + start_pos_ <= (size_t)context_len_);  // reference llama_cu.cu:1074
    lcu::matmul_type_ref() = matmul_type;  // the reference reads its global at every matmul (llama_cu.cu:1467, 1504)
    int token = 0;
    if (core->next_token(new_tokens.data(), (int)new_tokens.size(), &token) != lcu::LCU_OK) {
      fprintf(stderr, "%s\n", lcu::last_error());
      abort();
    }
    start_pos_ += (int)new_tokens.size();
    return (short)token;
  }
  std::unique_ptr<lcu::context> core;
};
}  // namespace

std::unique_ptr<llama_context> llama_context::create(llama_model* model, int context_len, float temperature) {
  return std::make_unique<context_on_b200>(static_cast<llama_model_impl*>(model), context_len, temperature);
}

}  // namespace llama_cu

// llama_vocabulary::tokenize for foreign-function callers (declared in llama_cu_c.h)
extern "C" int lcu_tokenize(const char* vocab_path, const char* text, int bos, int16_t* ids_out, int capacity) {
  if (!vocab_path || !text || (capacity > 0 && !ids_out)) {
    lcu::set_last_error("tokenize: null argument");
    return -1;
  }
  llama_cu::mapped_buffer file{std::string(vocab_path)};
  if (!file.is_ok() || file.size() < 4) {
    lcu::set_last_error("tokenize: cannot map vocabulary file %s", vocab_path);
    return -1;
  }
  llama_cu::llama_vocabulary vocab(file);
  const std::vector<short> ids = vocab.tokenize(text, bos != 0);
  for (size_t i = 0; i < ids.size() && (int)i < capacity; ++i) ids_out[i] = ids[i];
  return (int)ids.size();
}
