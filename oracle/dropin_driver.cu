// Drop-in proof.  TEST INFRASTRUCTURE ONLY.
//
// ONE client source written against the reference's C++ interface (llama_cu.h with
// LLAMA_CU_IMPLEMENTATION: tensor4d, generic_tensor, the matmul_nt operator seam, llama_model,
// llama_context, llama_vocabulary).  oracle/Makefile compiles it twice without changing a line:
//   oracle/_ref/dropin_ref  against the reference's own header, linked with the reference built for sm_100a;
//   oracle/_ref/dropin_new  against include/llama_cu.h, linked with libllama_cu_b200.so.
// The GPU test runs both on the same weight directory and compares what they print.
//
//   dropin_driver run <model_dir> <report_file> [forced_tokens_file]
//   dropin_driver tokenize <vocab_file> <text>
#define LLAMA_CU_IMPLEMENTATION
#include "llama_cu.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace llama_cu {
// the seam is declared in the reference's llama_cu.cu (738-747), not in its header
void matmul_nt(tensor4d_view<__half> out, tensor4d_view<__half> lhs, tensor4d_view<__half> rhs, __half beta, cudaStream_t stream);
void matmul_nt(tensor4d_view<__half> out, tensor4d_view<__half> lhs, generic_tensor& rhs, __half beta, cudaStream_t stream);
}  // namespace llama_cu
using namespace llama_cu;

namespace {
struct lcg {  // the same numbers in both binaries
  uint64_t s;
  explicit lcg(uint64_t seed) : s(seed) {}
  uint32_t next() {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    return (uint32_t)(s >> 33);
  }
  float uniform() { return (float)(next() & 0xffffff) / 16777216.0f - 0.5f; }  // [-0.5, 0.5)
};

std::vector<__half> random_halves(size_t n, float scale, uint64_t seed) {
  lcg g(seed);
  std::vector<__half> v(n);
  for (auto& x : v) x = __float2half(scale * (g.uniform() + g.uniform() + g.uniform()));
  return v;
}

void report(FILE* f, const char* name, tensor4d<__half>& t, size_t rows, size_t cols) {
  std::vector<__half> host(rows * cols);
  cudaDeviceSynchronize();
  cudaMemcpy(host.data(), t.data(), host.size() * 2, cudaMemcpyDeviceToHost);
  fprintf(f, "matmul %s %zu %zu", name, rows, cols);
  for (__half h : host) {
    unsigned short bits;
    memcpy(&bits, &h, 2);
    fprintf(f, " %u", bits);
  }
  fprintf(f, "\n");
}

// out(m, n) = x(m, k) . w(n, k)^T (+ out) through both overloads of the seam
void matmul_section(FILE* f) {
  const size_t k = 1024, n = 512;
  for (size_t m : {(size_t)1, (size_t)20}) {
    for (int quantized = 0; quantized < 2; ++quantized) {
      for (float beta : {0.0f, 1.0f}) {
        tensor4d<__half> x(1, 1, m, k, 128), out(1, 1, m, n, 128);
        auto hx = random_halves(m * k, 1.0f, 11 + m);
        auto hout = random_halves(m * n, 1.0f, 13 + m);
        x.gpu.copy_from(hx.data(), hx.size() * 2);
        out.gpu.copy_from(hout.data(), hout.size() * 2);
        generic_tensor w;
        if (quantized) {
          quantized_tensor q;
          q.q_values = tensor4d<uint8_t>(1, 1, n, k);
          q.scales = tensor4d<__half>(1, 1, n, k / 128);
          q.q_type = quantization_type::uint8;
          q.quantization_block_size = 128;
          lcg g(17);
          std::vector<uint8_t> bytes(n * k);
          for (auto& b : bytes) b = (uint8_t)(g.next() & 0xff);
          std::vector<__half> sc(n * k / 128);
          for (auto& s : sc) s = __float2half(0.0002f + 0.0004f * (g.uniform() + 0.5f));
          q.q_values.gpu.copy_from(bytes.data(), bytes.size());
          q.scales.gpu.copy_from(sc.data(), sc.size() * 2);
          w = generic_tensor(std::move(q));
        } else {
          tensor4d<__half> t(1, 1, n, k);
          auto hw = random_halves(n * k, 0.05f, 19);
          t.gpu.copy_from(hw.data(), hw.size() * 2);
          w = generic_tensor(std::move(t));
        }
        cudaDeviceSynchronize();
        auto v_out = out.view().take(1, 1, m, n);
        auto v_x = x.view().take(1, 1, m, k);
        if (quantized)
          matmul_nt(v_out, v_x, w, __float2half(beta), 0);
        else
          matmul_nt(v_out, v_x, w.as_fp16().view(), __float2half(beta), 0);
        char name[64];
        snprintf(name, sizeof name, "m%zu_%s_beta%d", m, quantized ? "u8" : "f16", (int)beta);
        report(f, name, out, m, n);
      }
    }
  }
}

int run(const char* dir, const char* report_path, const char* forced_path) {
  initialize();
  mapped_buffer params_file(std::string(dir) + "/params");
  llama_params params;
  if (!params_file.is_ok() || !params.load(params_file)) {
    fprintf(stderr, "cannot read %s/params\n", dir);
    return 1;
  }
  llama_partition partition;
  partition.use_default(params);
  if (!partition.is_valid()) return 1;
  auto model = llama_model::load(params, partition, dir);
  if (!model) return 1;
  auto context = llama_context::create(model.get(), 128, 0.8f);
  FILE* f = fopen(report_path, "w");
  if (!f) return 1;
  matmul_type = 4;
  matmul_section(f);  // (after the context exists: the reference's constructor opts its kernels into large shared memory)

  std::vector<short> forced;
  if (forced_path) {
    std::ifstream in(forced_path);
    for (int t; in >> t;) forced.push_back((short)t);
  }
  lcg g(1234);
  std::vector<short> prompt(16);
  for (auto& t : prompt) t = (short)(3 + g.next() % (params.n_vocab - 3));
  std::vector<short> produced;
  short token = context->next_token(prompt);
  produced.push_back(token);
  for (int step = 0; step < 24; ++step) {
    const short fed = step < (int)forced.size() ? forced[step] : token;
    token = context->next_token({fed});
    produced.push_back(token);
  }
  fprintf(f, "tokens");
  for (short t : produced) fprintf(f, " %d", (int)t);
  fprintf(f, "\ntokens_left %zu\ncontext_bytes %zu\n", context->tokens_left(), context->context_memory_usage());
  context->clear_tokens();
  fprintf(f, "tokens_left_after_clear %zu\n", context->tokens_left());
  fclose(f);
  return 0;
}

int tokenize(const char* vocab_path, const char* text) {
  mapped_buffer vocab_file{std::string(vocab_path)};
  if (!vocab_file.is_ok()) return 1;
  llama_vocabulary vocab(vocab_file);
  for (short id : vocab.tokenize(text, true)) printf("%d ", (int)id);
  printf("\n");
  return 0;
}
}  // namespace

int main(int argc, char** argv) {
  if (argc >= 4 && !strcmp(argv[1], "run")) return run(argv[2], argv[3], argc > 4 ? argv[4] : nullptr);
  if (argc == 4 && !strcmp(argv[1], "tokenize")) return tokenize(argv[2], argv[3]);
  fprintf(stderr, "usage: %s run <model_dir> <report_file> [forced_tokens_file] | tokenize <vocab_file> <text>\n", argv[0]);
  return 2;
}
