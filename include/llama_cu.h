// C++ interface of the B200-native llama.cu inference core.
//
// Source-compatible with the public part of the reference's llama_cu.h (eiz/llama.cu): a program
// written against that header - the reference's own main.cpp for one - compiles against this one
// and links with libllama_cu_b200.so unchanged.  Each declaration names the reference lines it
// mirrors.  Everything here is a thin layer over the C ABI in llama_cu_c.h; the device code is
// sm_100a only and there is no CPU fallback.
//
// A translation unit that defines LLAMA_CU_IMPLEMENTATION before including this header also gets
// the reference's internal vocabulary (reference llama_cu.h:29-62, 141-272): CHECK_CUDA,
// RETURN_UNLESS, tensor4d / tensor4d_view, quantized_tensor, generic_tensor - and the operator
// seam matmul_nt(out, lhs, rhs, beta, stream) (reference llama_cu.cu:738-747), which this library
// exports with the reference's C++ signatures on top of the same sm_100a kernels.
#pragma once

#if __cplusplus < 201703L
#error "C++17 or higher is required"
#endif

#include <cstddef>
#include <cstdint>
#include <memory>
#include <queue>
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

#ifdef LLAMA_CU_IMPLEMENTATION
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <variant>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

// reference llama_cu.h:48-56: a failed CUDA call is fatal (message, then SIGSEGV)
#define CHECK_CUDA(expr)                                                                                       \
  do {                                                                                                         \
    cudaError_t llama_cu_status_ = (expr);                                                                     \
    if (llama_cu_status_ != cudaSuccess) {                                                                     \
      fprintf(stderr, "%s(%d): cuda error: %s (source: " #expr ")\n", __func__, __LINE__,                      \
              cudaGetErrorString(llama_cu_status_));                                                           \
      raise(SIGSEGV);                                                                                          \
    }                                                                                                          \
  } while (0)
// reference llama_cu.h:57-60
#define RETURN_UNLESS(x) \
  if (!(x)) {            \
    return false;        \
  }
#ifdef __CUDACC__
#define LLAMA_CU_HD __host__ __device__ __forceinline__
#else
#define LLAMA_CU_HD inline
#endif
#endif  // LLAMA_CU_IMPLEMENTATION

namespace llama_cu {

// reference llama_cu.h:65-68.  0 (cuBLAS in the reference) and 4 (its tensor-core kernels) both
// select the native sm_100a kernels; 1 selects the pedantic one-thread-per-output kernels (the
// reference's naive pair, llama_cu.cu:111-145) for every matrix product.
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

// reference llama_cu.h:97-108: makes `device` current until the end of the scope
struct scoped_gpu {
  scoped_gpu(int device);
  ~scoped_gpu();
  scoped_gpu(scoped_gpu const&) = delete;
  scoped_gpu& operator=(scoped_gpu const&) = delete;

 private:
  int prev_device_;
};

// reference llama_cu.h:110-123: a device pointer and its size in bytes (not owning)
struct gpu_buffer_view {
  gpu_buffer_view() {}
  gpu_buffer_view(void* dev_ptr, size_t size) : dev_ptr_(dev_ptr), size_(size) {}
  void copy_from(mapped_buffer const& buffer);          // sizes must agree; asynchronous like the reference's
  void copy_from(void const* buffer, size_t size);      // size <= size()
  void copy_to(void* buffer, size_t size);              // blocking
  bool is_ok() const { return dev_ptr_ != nullptr; }
  void* data() const { return dev_ptr_; }
  size_t size() const { return size_; }

 protected:
  void* dev_ptr_{nullptr};
  size_t size_{0};
};

// reference llama_cu.h:125-134: owning device allocation, move-only
struct gpu_buffer : public gpu_buffer_view {
  gpu_buffer() {}
  explicit gpu_buffer(size_t size);
  gpu_buffer(gpu_buffer&& other);
  gpu_buffer& operator=(gpu_buffer&& other);
  ~gpu_buffer();
  gpu_buffer(gpu_buffer const&) = delete;
  gpu_buffer& operator=(gpu_buffer const&) = delete;
};

// reference llama_cu.h:136-139
enum class quantization_type : uint8_t { fp16, uint8 };

#ifdef LLAMA_CU_IMPLEMENTATION
// reference llama_cu.h:141-157
LLAMA_CU_HD size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }
LLAMA_CU_HD size_t round_up(size_t a, size_t b) { return ceil_div(a, b) * b; }
template <typename T>
inline float to_float(T value);
template <>
inline float to_float(float value) {
  return value;
}
template <>
inline float to_float(__half value) {
  return __half2float(value);
}

// reference llama_cu.h:162-234: a 4-D window (n, c, h, w) with element strides over device memory.
// take() keeps the origin and shrinks the extents; as in the reference the view's byte size then
// becomes take_n * stride_n elements.  skip() moves the origin forward and shrinks the extents.
template <typename T>
struct tensor4d_view {
  tensor4d_view() = default;
  tensor4d_view(size_t n, size_t c, size_t h, size_t w, size_t stride_n, size_t stride_c, size_t stride_h, gpu_buffer_view gpu)
      : n(n), c(c), h(h), w(w), stride_n(stride_n), stride_c(stride_c), stride_h(stride_h), gpu(gpu) {}
  size_t size() { return n * c * h * w; }
  T* data() { return static_cast<T*>(gpu.data()); }
  tensor4d_view<T> skip(int skip_n, int skip_c, int skip_h, int skip_w) {
    const size_t first = skip_n * stride_n + skip_c * stride_c + skip_h * stride_h + skip_w;
    return tensor4d_view<T>(n - skip_n, c - skip_c, h - skip_h, w - skip_w, stride_n, stride_c, stride_h,
                            gpu_buffer_view(static_cast<char*>(gpu.data()) + first * sizeof(T), gpu.size() - first * sizeof(T)));
  }
  tensor4d_view<T> take(int take_n, int take_c, int take_h, int take_w) {
    return tensor4d_view<T>(take_n, take_c, take_h, take_w, stride_n, stride_c, stride_h,
                            gpu_buffer_view(gpu.data(), take_n * stride_n * sizeof(T)));
  }
  // reference llama_cu.h:206-227: copies the window to the host and prints the corners of every channel
  void debug_print(char const* title, float divisor = 1.0) {
    T* host = static_cast<T*>(malloc(gpu.size()));
    gpu.copy_to(host, gpu.size());
    printf("==%s (%zu,%zu,%zu,%zu) (%zu,%zu,%zu)==\n", title, n, c, h, w, stride_n, stride_c, stride_h);
    for (size_t ch = 0; ch < c; ++ch) {
      printf("channel %zu\n", ch);
      for (size_t row = 0; row < h; ++row) {
        printf("% 4d ", (int)row);
        for (size_t col = 0; col < w; ++col) {
          printf("% 9.6f, ", to_float(host[ch * stride_c + row * stride_h + col]) / divisor);
          if (w > 3 && col > 1 && col + 4 < w) {  // the first three and the last four columns only
            printf(" ... ");
            col = w - 4;
          }
        }
        printf("\n");
      }
      printf("\n\n\n");
    }
    free(host);
  }
  size_t n = 0, c = 0, h = 0, w = 0;
  size_t stride_n = 0, stride_c = 0, stride_h = 0;
  gpu_buffer_view gpu;
};

// reference llama_cu.h:236-252: owning dense tensor.  gutter_h adds zeroed rows behind the last one: the reference's
// tile kernels read and write past the logical rows; the kernels of this library never do, the argument is kept for
// source compatibility.
template <typename T>
struct tensor4d {
  tensor4d() = default;
  tensor4d(size_t n, size_t c, size_t h, size_t w, size_t gutter_h = 0)
      : n(n), c(c), h(h), w(w), gpu(gpu_buffer(n * c * (h + gutter_h) * w * sizeof(T))) {
    if (gutter_h > 0) cudaMemset(gpu.data(), 0, gpu.size());
  }
  size_t size() const { return n * c * h * w; }
  operator tensor4d_view<T>() { return tensor4d_view<T>(n, c, h, w, c * h * w, h * w, w, gpu); }
  tensor4d_view<T> view() { return *this; }
  T* data() { return static_cast<T*>(gpu.data()); }
  T const* data() const { return static_cast<T const*>(gpu.data()); }
  size_t n = 0, c = 0, h = 0, w = 0;
  gpu_buffer gpu;
};

// reference llama_cu.h:254-259: u8 values [h][w] and fp16 scales [h][w / block size]
struct quantized_tensor {
  tensor4d<uint8_t> q_values;
  tensor4d<half> scales;
  quantization_type q_type{quantization_type::fp16};
  uint16_t quantization_block_size{0};
};

// reference llama_cu.h:261-272: a weight matrix in either storage
struct generic_tensor {
  std::variant<tensor4d<half>, quantized_tensor> v;
  generic_tensor() {}
  generic_tensor(tensor4d<half> t) : v(std::move(t)) {}
  generic_tensor(quantized_tensor t) : v(std::move(t)) {}
  bool is_quantized() const { return std::holds_alternative<quantized_tensor>(v); }
  bool is_fp16() const { return std::holds_alternative<tensor4d<half>>(v); }
  tensor4d<half>& as_fp16() { return std::get<tensor4d<half>>(v); }
  quantized_tensor& as_quantized() { return std::get<quantized_tensor>(v); }
  tensor4d<half> const& as_fp16() const { return std::get<tensor4d<half>>(v); }
  quantized_tensor const& as_quantized() const { return std::get<quantized_tensor>(v); }
};

// The operator seam (reference llama_cu.cu:738-747, 1463-1523; declared there, not in its header):
// out(m, n) = lhs(m, k) . rhs(n, k)^T + beta * out with m = lhs.h, k = lhs.w, n = rhs.h; rows dense; fp16 in and out,
// fp32 accumulation; dispatch on llama_cu::matmul_type.  No gutter rows are needed behind out or lhs.
constexpr int GUTTER = 128;  // reference llama_cu.cu:749, for callers that size their tensors with it
void matmul_nt(tensor4d_view<__half> out, tensor4d_view<__half> lhs, tensor4d_view<__half> rhs, __half beta = 0.0f, cudaStream_t stream = 0);
void matmul_nt(tensor4d_view<__half> out, tensor4d_view<__half> lhs, generic_tensor& rhs, __half beta = 0.0f, cudaStream_t stream = 0);
#endif  // LLAMA_CU_IMPLEMENTATION

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
