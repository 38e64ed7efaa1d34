// C-ABI shim around the UNMODIFIED reference implementation (eiz/llama.cu, llama_cu.cu + llama_cu.h).
//
// TEST INFRASTRUCTURE ONLY.  The reference translation unit is pulled in from where it lies (the
// include path is given on the command line by oracle/Makefile); no reference source is copied.
// The shim lets the Python tests and the benchmark's reference arm drive the reference's own
// kernels and its own forward pass (llama_context::next_token) on the same inputs as the new
// library, so that golden vectors come from the reference itself.
//
// The reference keeps its kernels and the context's logits buffer file-local / private, so the
// standard headers are included first and then the access keywords are opened up for the one
// include below.
#include <algorithm>
#include <cassert>
#include <cfloat>
#include <chrono>
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <memory>
#include <queue>
#include <random>
#include <string>
#include <string_view>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <variant>
#include <vector>
#include <fcntl.h>
#include <signal.h>
#include <sys/mman.h>
#include <unistd.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <mma.h>

#define private public
#define protected public
#include "llama_cu.cu"
#undef private
#undef protected

using namespace llama_cu;

namespace {
bool g_attr_set = false;
void ensure_smem_attr() {  // the two 16x128x256 kernels need the opt-in the context constructor does (llama_cu.cu:1035-1038)
  if (g_attr_set) return;
  cudaFuncSetAttribute(kernel::matmul_nt_wmma_16x128x256, cudaFuncAttributeMaxDynamicSharedMemorySize, 78336);
  cudaFuncSetAttribute(kernel::matmul_nt_wmma_16x128x256_fp16u8, cudaFuncAttributeMaxDynamicSharedMemorySize, 78336);
  g_attr_set = true;
}

struct ref_model_handle {
  std::unique_ptr<llama_model> model;
  llama_model_impl* impl() { return reinterpret_cast<llama_model_impl*>(model.get()); }
};

generic_tensor alloc_matrix(const llama_params& p, size_t h, size_t w) {
  if (p.q_type == quantization_type::fp16) return generic_tensor(tensor4d<half>(1, 1, h, w));
  quantized_tensor q;
  q.q_values = tensor4d<uint8_t>(1, 1, h, w);
  q.scales = tensor4d<half>(1, 1, h, w / p.quantization_block_size);
  q.q_type = p.q_type;
  q.quantization_block_size = p.quantization_block_size;
  return generic_tensor(std::move(q));
}

generic_tensor* find_matrix(llama_model_impl* m, const std::string& name, tensor4d<half>** vec) {
  *vec = nullptr;
  if (name == "tok_embeddings") return &m->tok_embeddings;
  if (name == "output") return &m->output;
  if (name == "norm") {
    *vec = &m->norm;
    return nullptr;
  }
  if (name.rfind("layers.", 0) != 0) return nullptr;
  size_t dot = name.find('.', 7);
  if (dot == std::string::npos) return nullptr;
  int li = atoi(name.substr(7, dot - 7).c_str());
  if (li < 0 || li >= (int)m->layers.size()) return nullptr;
  std::string rest = name.substr(dot + 1);
  llama_layer& L = m->layers[li];
  if (rest == "attention_norm") { *vec = &L.attn_norm; return nullptr; }
  if (rest == "ffn_norm") { *vec = &L.ffn_norm; return nullptr; }
  if (rest == "attention.wq") return &L.wq;
  if (rest == "attention.wk") return &L.wk;
  if (rest == "attention.wv") return &L.wv;
  if (rest == "attention.wo") return &L.wo;
  if (rest == "feed_forward.w1") return &L.w1;
  if (rest == "feed_forward.w2") return &L.w2;
  if (rest == "feed_forward.w3") return &L.w3;
  return nullptr;
}

llama_partition make_partition(const llama_params& p, const int* layer_gpus) {
  llama_partition part;
  if (!layer_gpus) {
    part.use_default(p);
    return part;
  }
  std::unordered_set<int> used;
  for (uint32_t i = 0; i < p.n_layers; ++i) {
    part.layer_gpus.push_back(layer_gpus[i]);
    used.insert(layer_gpus[i]);
  }
  part.embedding_gpu = part.layer_gpus.front();
  part.output_gpu = part.layer_gpus.back();
  part.used_gpus.assign(used.begin(), used.end());
  return part;
}
}  // namespace

extern "C" {

void ref_initialize() { initialize(); }

// out(m,n) = lhs(m,k) * rhs(n,k)^T + beta*out through the reference's matmul_nt dispatch
// (llama_cu.cu:1463-1496).  Host buffers; activations get the reference's 128-row gutter.
// If ms_out != nullptr the call is repeated `reps` times and the mean device time is returned.
int ref_matmul_nt_f16(uint16_t* out, const uint16_t* lhs, const uint16_t* rhs, int m, int k, int n, float beta,
                      int type, int reps, float* ms_out) {
  ensure_smem_attr();
  matmul_type = type;
  tensor4d<half> t_out(1, 1, m, n, GUTTER), t_lhs(1, 1, m, k, GUTTER), t_rhs(1, 1, n, k);
  cudaMemcpy(t_lhs.data(), lhs, (size_t)m * k * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(t_rhs.data(), rhs, (size_t)n * k * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(t_out.data(), out, (size_t)m * n * 2, cudaMemcpyHostToDevice);
  auto v_out = t_out.view().take(1, 1, m, n);
  auto v_lhs = t_lhs.view().take(1, 1, m, k);
  matmul_nt(v_out, v_lhs, t_rhs.view(), __float2half(beta), 0);
  if (cudaDeviceSynchronize() != cudaSuccess) return 1;
  cudaMemcpy(out, t_out.data(), (size_t)m * n * 2, cudaMemcpyDeviceToHost);
  if (ms_out) {
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, 0);
    for (int i = 0; i < reps; ++i) matmul_nt(v_out, v_lhs, t_rhs.view(), __float2half(0.f), 0);
    cudaEventRecord(e1, 0);
    cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    *ms_out = ms / reps;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  }
  return cudaGetLastError() != cudaSuccess;
}

// int8-weight variant (llama_cu.cu:1498-1523); type 4 = tensor-core kernel, 1 = naive kernel
int ref_matmul_nt_fp16u8(uint16_t* out, const uint16_t* lhs, const uint8_t* q, const uint16_t* scales, int m, int k,
                         int n, int bs, float beta, int type, int reps, float* ms_out) {
  ensure_smem_attr();
  matmul_type = type;
  tensor4d<half> t_out(1, 1, m, n, GUTTER), t_lhs(1, 1, m, k, GUTTER);
  quantized_tensor qt;
  qt.q_values = tensor4d<uint8_t>(1, 1, n, k);
  qt.scales = tensor4d<half>(1, 1, n, k / bs);
  qt.q_type = quantization_type::uint8;
  qt.quantization_block_size = (uint16_t)bs;
  cudaMemcpy(qt.q_values.data(), q, (size_t)n * k, cudaMemcpyHostToDevice);
  cudaMemcpy(qt.scales.data(), scales, (size_t)n * (k / bs) * 2, cudaMemcpyHostToDevice);
  generic_tensor rhs(std::move(qt));
  cudaMemcpy(t_lhs.data(), lhs, (size_t)m * k * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(t_out.data(), out, (size_t)m * n * 2, cudaMemcpyHostToDevice);
  auto v_out = t_out.view().take(1, 1, m, n);
  auto v_lhs = t_lhs.view().take(1, 1, m, k);
  matmul_nt(v_out, v_lhs, rhs, __float2half(beta), 0);
  if (cudaDeviceSynchronize() != cudaSuccess) return 1;
  cudaMemcpy(out, t_out.data(), (size_t)m * n * 2, cudaMemcpyDeviceToHost);
  if (ms_out) {
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, 0);
    for (int i = 0; i < reps; ++i) matmul_nt(v_out, v_lhs, rhs, __float2half(0.f), 0);
    cudaEventRecord(e1, 0);
    cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    *ms_out = ms / reps;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  }
  return cudaGetLastError() != cudaSuccess;
}

// Timed loop of the reference matmul over `copies` distinct device-resident weight matrices
// (rotating through more bytes than L2 holds).  Returns mean milliseconds per call.
float ref_matmul_rotating_ms(int m, int k, int n, int bs, int type, int copies, int reps) {
  ensure_smem_attr();
  matmul_type = type;
  tensor4d<half> t_out(1, 1, m, n, GUTTER), t_lhs(1, 1, m, k, GUTTER);
  std::vector<generic_tensor> ws;
  for (int i = 0; i < copies; ++i) {
    if (bs == 0) {
      tensor4d<half> t(1, 1, n, k);
      cudaMemset(t.data(), 0x11 + i, (size_t)n * k * 2);
      ws.emplace_back(std::move(t));
    } else {
      quantized_tensor qt;
      qt.q_values = tensor4d<uint8_t>(1, 1, n, k);
      qt.scales = tensor4d<half>(1, 1, n, k / bs);
      qt.q_type = quantization_type::uint8;
      qt.quantization_block_size = (uint16_t)bs;
      cudaMemset(qt.q_values.data(), 0x11 + i, (size_t)n * k);
      cudaMemset(qt.scales.data(), 0x11, (size_t)n * (k / bs) * 2);
      ws.emplace_back(std::move(qt));
    }
  }
  auto v_out = t_out.view().take(1, 1, m, n);
  auto v_lhs = t_lhs.view().take(1, 1, m, k);
  for (int i = 0; i < copies; ++i) matmul_nt(v_out, v_lhs, ws[i], __float2half(0.f), 0);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaEventRecord(e0, 0);
  for (int i = 0; i < reps; ++i) matmul_nt(v_out, v_lhs, ws[i % copies], __float2half(0.f), 0);
  cudaEventRecord(e1, 0);
  cudaEventSynchronize(e1);
  float ms = 0;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return cudaGetLastError() == cudaSuccess ? ms / reps : -1.f;
}

int ref_rms_norm(uint16_t* out, const uint16_t* in, const uint16_t* weight, int h, int w, float eps) {
  tensor4d<half> t_in(1, 1, h, w), t_out(1, 1, h, w), t_w(1, 1, 1, w);
  cudaMemcpy(t_in.data(), in, (size_t)h * w * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(t_w.data(), weight, (size_t)w * 2, cudaMemcpyHostToDevice);
  kernel::rms_norm<<<h, 256>>>(t_out.data(), t_in.data(), t_w.data(), h, w, eps);
  cudaMemcpy(out, t_out.data(), (size_t)h * w * 2, cudaMemcpyDeviceToHost);
  return cudaGetLastError() != cudaSuccess;
}

int ref_rotary(uint16_t* out, const uint16_t* in, int h, int w, int n_heads, int pos_offset) {
  tensor4d<half> t_in(1, 1, h, w), t_out(1, 1, h, w);
  cudaMemcpy(t_in.data(), in, (size_t)h * w * 2, cudaMemcpyHostToDevice);
  dim3 grid(ceil_div(w, 32), ceil_div(h, 32)), block(32, 32);
  kernel::rotary<<<grid, block>>>(t_out.data(), t_in.data(), h, w, n_heads, pos_offset);
  cudaMemcpy(out, t_out.data(), (size_t)h * w * 2, cudaMemcpyDeviceToHost);
  return cudaGetLastError() != cudaSuccess;
}

int ref_silu(uint16_t* out, const uint16_t* a, const uint16_t* b, size_t n) {
  tensor4d<half> t_a(1, 1, 1, n), t_b(1, 1, 1, n), t_o(1, 1, 1, n);
  cudaMemcpy(t_a.data(), a, n * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(t_b.data(), b, n * 2, cudaMemcpyHostToDevice);
  kernel::silu<<<ceil_div(n, 256), 256>>>(t_o.data(), t_a.data(), t_b.data(), (int)n);
  cudaMemcpy(out, t_o.data(), n * 2, cudaMemcpyDeviceToHost);
  return cudaGetLastError() != cudaSuccess;
}

// the reference's attention chain (llama_cu.cu:1161-1171) on q (m,dim), rotated k (T,dim), v (T,dim)
int ref_attention(uint16_t* out, const uint16_t* q, const uint16_t* k, const uint16_t* v, int m, int T, int dim,
                  int n_heads, int start_pos) {
  tensor4d<half> t_q(1, 1, m, dim), t_k(1, 1, T, dim), t_v(1, 1, T, dim), t_o(1, 1, m, dim), t_qk(1, n_heads, m, T);
  cudaMemcpy(t_q.data(), q, (size_t)m * dim * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(t_k.data(), k, (size_t)T * dim * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(t_v.data(), v, (size_t)T * dim * 2, cudaMemcpyHostToDevice);
  const dim3 block(32, 32);
  dim3 grid(ceil_div(T, 32), ceil_div(m, 32), n_heads);
  kernel::matmul_qk<<<grid, block>>>(t_qk.data(), t_q.data(), t_k.data(), m, T, dim, n_heads, start_pos);
  kernel::softmax_rows<<<dim3(m, n_heads), 256>>>(t_qk.data(), t_qk.data(), m, T);
  grid = dim3(ceil_div(dim, 32), ceil_div(T, 32));
  kernel::matmul_qkv<<<grid, block>>>(t_o.data(), t_qk.data(), t_v.data(), m, T, dim, n_heads);
  cudaMemcpy(out, t_o.data(), (size_t)m * dim * 2, cudaMemcpyDeviceToHost);
  return cudaGetLastError() != cudaSuccess;
}

// ---- model / context ------------------------------------------------------------------------
// Allocates the reference's llama_model_impl with uninitialised device tensors (no files): the
// caller fills them in place through ref_model_tensor().  layer_gpus == NULL puts all on GPU 0.
void* ref_model_alloc(uint32_t dim, uint32_t multiple_of, uint32_t n_heads, uint32_t n_layers, uint32_t n_vocab,
                      float norm_eps, int block_size, const int* layer_gpus) {
  llama_params p{};
  p.magic = LLAMA_CU_MAGIC;
  p.fourcc = LLAMA_CU_MODEL_FOURCC_LLAMA;
  p.dim = dim;
  p.multiple_of = multiple_of;
  p.n_heads = n_heads;
  p.n_layers = n_layers;
  p.n_vocab = n_vocab;
  p.norm_eps = norm_eps;
  p.q_type = block_size > 0 ? quantization_type::uint8 : quantization_type::fp16;
  p.quantization_block_size = (uint16_t)block_size;
  llama_partition part = make_partition(p, layer_gpus);
  auto impl = std::make_unique<llama_model_impl>(p, part);
  {
    scoped_gpu g(part.embedding_gpu);
    impl->tok_embeddings = alloc_matrix(p, n_vocab, dim);
  }
  {
    scoped_gpu g(part.output_gpu);
    impl->output = alloc_matrix(p, n_vocab, dim);
    impl->norm = tensor4d<half>(1, 1, 1, dim);
  }
  for (uint32_t i = 0; i < n_layers; ++i) {
    scoped_gpu g(part.layer_gpus[i]);
    llama_layer L;
    L.attn_norm = tensor4d<half>(1, 1, 1, dim);
    L.ffn_norm = tensor4d<half>(1, 1, 1, dim);
    L.wq = alloc_matrix(p, dim, dim);
    L.wk = alloc_matrix(p, dim, dim);
    L.wv = alloc_matrix(p, dim, dim);
    L.wo = alloc_matrix(p, dim, dim);
    L.w1 = alloc_matrix(p, p.ffn_dim(), dim);
    L.w2 = alloc_matrix(p, dim, p.ffn_dim());
    L.w3 = alloc_matrix(p, p.ffn_dim(), dim);
    impl->layers.emplace_back(std::move(L));
  }
  auto* h = new ref_model_handle();
  h->model = std::move(impl);
  return h;
}

// which: 0 = fp16 matrix / norm vector / u8 values, 1 = fp16 scales.  Returns 0 on success.
int ref_model_tensor(void* model, const char* name, int which, void** dev_ptr, uint64_t* bytes) {
  auto* h = (ref_model_handle*)model;
  tensor4d<half>* vec = nullptr;
  generic_tensor* g = find_matrix(h->impl(), name, &vec);
  if (vec) {
    *dev_ptr = vec->data();
    *bytes = vec->gpu.size();
    return 0;
  }
  if (!g) return 1;
  if (g->is_fp16()) {
    if (which != 0) return 1;
    *dev_ptr = g->as_fp16().data();
    *bytes = g->as_fp16().gpu.size();
  } else if (which == 0) {
    *dev_ptr = g->as_quantized().q_values.data();
    *bytes = g->as_quantized().q_values.gpu.size();
  } else {
    *dev_ptr = g->as_quantized().scales.data();
    *bytes = g->as_quantized().scales.gpu.size();
  }
  return 0;
}

}  // extern "C"

// ---- seeded synthetic weights, generated on the device inside this library --------------------
// The benchmark's reference arm must not map the product library, so the generator the product
// uses for its synthetic models is restated here (test infrastructure; same recipe, same bits):
// one Philox4x32-10 block per element keyed by the seed, counter = (element index, FNV-1a of the
// tensor name), the eight 16-bit lanes summed (Irwin-Hall) and scaled to unit variance, times
// `scale`, rounded to half.  Norm vectors are 1.0.  u8 models: each matrix is generated in fp16 and
// quantized with the reference's own quantizer kernel (ref_quantize_device, transform.cu:28-72).
__global__ void shim_synth_kernel(half* out, size_t n, uint64_t seed, uint64_t stream_id, float scale) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    uint32_t c0 = (uint32_t)i, c1 = (uint32_t)(i >> 32), c2 = (uint32_t)stream_id, c3 = (uint32_t)(stream_id >> 32);
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    for (int r = 0; r < 10; ++r) {
      const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
      const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
      c0 = n0; c1 = (uint32_t)p1; c2 = n2; c3 = (uint32_t)p0;
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
    const int sum = (int)(c0 & 0xffffu) + (int)(c0 >> 16) + (int)(c1 & 0xffffu) + (int)(c1 >> 16) + (int)(c2 & 0xffffu) + (int)(c2 >> 16) +
                    (int)(c3 & 0xffffu) + (int)(c3 >> 16);
    const float z = __fmul_rn((float)(sum - 262140), 0x1.3988e2p-16f);
    out[i] = __float2half(__fmul_rn(z, scale));
  }
}
__global__ void shim_fill_kernel(half* out, size_t n, half v) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = v;
}
extern "C" int ref_quantize_device(void* q_dev, void* scales_dev, const void* in_dev, uint64_t h, uint64_t w, int bs);

extern "C" int ref_model_fill_synthetic(void* model, uint64_t seed, float scale) {
  auto* hnd = (ref_model_handle*)model;
  llama_model_impl* m = hnd->impl();
  const llama_params& p = m->params;
  std::vector<std::string> names = {"tok_embeddings", "output", "norm"};
  for (uint32_t i = 0; i < p.n_layers; ++i)
    for (const char* t : {"attention_norm", "ffn_norm", "attention.wq", "attention.wk", "attention.wv", "attention.wo", "feed_forward.w1",
                          "feed_forward.w2", "feed_forward.w3"})
      names.push_back("layers." + std::to_string(i) + "." + t);
  for (const std::string& name : names) {
    tensor4d<half>* vec = nullptr;
    generic_tensor* g = find_matrix(m, name, &vec);
    int dev = m->partition.output_gpu;
    if (name == "tok_embeddings") dev = m->partition.embedding_gpu;
    if (name.rfind("layers.", 0) == 0) dev = m->partition.layer_gpus[atoi(name.c_str() + 7)];
    scoped_gpu sg(dev);
    if (vec) {
      shim_fill_kernel<<<64, 256>>>(vec->data(), vec->size(), __float2half(1.0f));
      continue;
    }
    if (!g) return 1;
    uint64_t sid = 0xcbf29ce484222325ull;  // FNV-1a of the tensor name
    for (unsigned char ch : name) sid = (sid ^ ch) * 0x100000001b3ull;
    if (g->is_fp16()) {
      shim_synth_kernel<<<148 * 32, 256>>>(g->as_fp16().data(), g->as_fp16().size(), seed, sid, scale);
    } else {
      quantized_tensor& q = g->as_quantized();
      tensor4d<half> tmp(1, 1, q.q_values.h, q.q_values.w);
      shim_synth_kernel<<<148 * 32, 256>>>(tmp.data(), tmp.size(), seed, sid, scale);
      if (ref_quantize_device(q.q_values.data(), q.scales.data(), tmp.data(), q.q_values.h, q.q_values.w, q.quantization_block_size)) return 1;
    }
    if (cudaDeviceSynchronize() != cudaSuccess) return 1;
  }
  return cudaGetLastError() != cudaSuccess;
}

// llama_vocabulary::tokenize (llama_cu.cu:1344-1437) on a vocab file in extract.py's layout (44-61).
// Returns the number of ids (at most cap are written), or -1 if the file cannot be mapped.
extern "C" int ref_tokenize(const char* vocab_path, const char* text, int bos, int16_t* out, int cap) {
  mapped_buffer buf{std::string(vocab_path)};
  if (!buf.is_ok()) return -1;
  llama_vocabulary vocab(buf);
  std::vector<short> ids = vocab.tokenize(text, bos != 0);
  for (int i = 0; i < (int)ids.size() && i < cap; ++i) out[i] = ids[i];
  return (int)ids.size();
}

extern "C" {
// llama_model::load on a weight directory (llama_cu.cu:987-997); params are read from <dir>/params
void* ref_model_load(const char* dir, const int* layer_gpus) {
  mapped_buffer pb(std::string(dir) + "/params");
  llama_params p;
  if (!pb.is_ok() || !p.load(pb)) return nullptr;
  auto m = llama_model::load(p, make_partition(p, layer_gpus), dir);
  if (!m) return nullptr;
  cudaDeviceSynchronize();
  auto* h = new ref_model_handle();
  h->model = std::move(m);
  return h;
}

void ref_model_free(void* model) { delete (ref_model_handle*)model; }

void* ref_context_create(void* model, int context_len, float temperature, int type) {
  matmul_type = type;
  auto* h = (ref_model_handle*)model;
  return llama_context::create(h->model.get(), context_len, temperature).release();
}
void ref_context_free(void* ctx) { delete static_cast<llama_context_impl*>((llama_context*)ctx); }
void ref_context_clear(void* ctx) { ((llama_context*)ctx)->clear_tokens(); }
uint64_t ref_context_memory_usage(void* ctx) { return ((llama_context*)ctx)->context_memory_usage(); }

int ref_next_token(void* ctx, const int16_t* tokens, int n, int type) {
  matmul_type = type;
  std::vector<short> t(tokens, tokens + n);
  return ((llama_context*)ctx)->next_token(t);
}

// softmax output of the last step (the logits buffer is overwritten in place, llama_cu.cu:1196)
int ref_get_probs(void* ctx, uint16_t* out) {
  auto* c = static_cast<llama_context_impl*>((llama_context*)ctx);
  scoped_gpu g(c->model_->partition.output_gpu);
  return cudaMemcpy(out, c->t_logits_.data(), (size_t)c->model_->params.n_vocab * 2, cudaMemcpyDeviceToHost) != cudaSuccess;
}

// Greedy generation loop timed like main.cpp:80-100 (steady_clock around next_token).
// Returns the wall seconds of the n_steps single-token calls; tokens_out gets the n_steps results.
double ref_decode_timed(void* ctx, int16_t first_token, int n_steps, int16_t* tokens_out, int type) {
  matmul_type = type;
  auto* c = (llama_context*)ctx;
  std::vector<short> t{first_token};
  auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < n_steps; ++i) {
    short nt = c->next_token(t);
    tokens_out[i] = nt;
    t[0] = nt;
  }
  auto t1 = std::chrono::steady_clock::now();
  return std::chrono::duration<double>(t1 - t0).count();
}

}  // extern "C"
