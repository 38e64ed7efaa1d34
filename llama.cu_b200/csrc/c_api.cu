// extern "C" surface of libllama_cu_b200.so (declared in include/llama_cu_c.h).
#include "../../include/llama_cu_c.h"

#include <cuda_profiler_api.h>

#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "attention.cuh"
#include "gemm_tc.cuh"
#include "gemv.cuh"
#include "ops.cuh"
#include "prefill.cuh"
#include "runtime.cuh"
#include "tp.cuh"

using namespace lcu;

namespace {
context_options g_default_opts;  // "use_graph", "use_pdl", "attn_cluster" knobs apply to contexts created afterwards

int require_device() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    cudaGetLastError();
    set_last_error("no CUDA device is visible: this library has no CPU path");
    return LCU_ERR_CUDA;
  }
  return LCU_OK;
}
#define NEED_DEVICE()             \
  do {                            \
    int _r = require_device();    \
    if (_r) return _r;            \
  } while (0)

partition make_partition(const model_params& p, const int* layer_gpus) {
  partition part;
  int cur = 0;
  cudaGetDevice(&cur);  // no partition given: everything on the calling thread's current device
  for (uint32_t i = 0; i < p.n_layers; ++i) part.layer_gpus.push_back(layer_gpus ? layer_gpus[i] : cur);
  return part;
}

int* scratch_err() { return device_scratch_words(); }
}  // namespace

extern "C" {

const char* lcu_last_error(void) { return last_error(); }

int lcu_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int lcu_initialize(int verbose) {
  const int n = lcu_device_count();
  if (verbose && n > 0) {
    int device = 0;
    cudaDeviceProp prop;
    cudaGetDevice(&device);
    cudaGetDeviceProperties(&prop, device);
    printf("Device name: %s\n", prop.name);
    printf("Number of SMs: %d\n", prop.multiProcessorCount);
    printf("Shared mem size per SM: %zu bytes\n", prop.sharedMemPerMultiprocessor);
    printf("Shared mem size per block: %zu bytes\n", prop.sharedMemPerBlock);
    printf("Shared mem size per block (optin): %zu bytes\n", prop.sharedMemPerBlockOptin);
    printf("Shared mem size per block (reserved): %zu bytes\n", prop.reservedSharedMemPerBlock);
    printf("L2 cache size: %d bytes\n", prop.l2CacheSize);
  }
  return n;
}

int lcu_set_matmul_type(int type) {
  LCU_REQUIRE(type == 0 || type == 1 || type == 4, "matmul_type %d is not one of 0, 1, 4", type);
  matmul_type_ref() = type;
  return LCU_OK;
}

int lcu_set_tuning(const char* key, int value) {
  const std::string k(key ? key : "");
  if (k == "gemv_stages") gemv_tuning_ref().nstages = value;
  else if (k == "gemv_ctas_per_sm") gemv_tuning_ref().ctas_per_sm = value;
  else if (k == "gemv_ctas_per_sm_int8") gemv_tuning_ref().ctas_per_sm_int8 = value;
  else if (k == "int8_factored") gemv_tuning_ref().int8_factored = value;
  else if (k == "gemv_warp_stages_int8") gemv_tuning_ref().warp_stages_int8 = value;
  else if (k == "gemv_warp_stages") gemv_tuning_ref().warp_stages = value;
  else if (k == "gemv_consumer_warps_int8") gemv_tuning_ref().consumer_warps_int8 = value;
  else if (k == "gemv_variant") gemv_tuning_ref().variant = value;
  else if (k == "gemv_prefetch_kb") gemv_tuning_ref().prefetch_kb_per_cta = value;
  else if (k == "prefill_tc_min_rows") prefill_tuning_ref().tc_min_rows = value;
  else if (k == "prefill_tc_tile_n") prefill_tuning_ref().tc_tile_n = value;
  else if (k == "prefill_u8_deq_min_rows") prefill_tuning_ref().u8_deq_min_rows = value;
  else if (k == "prefill_u8_shadow") u8_shadow_mode() = value;
  else if (k == "attn_stream") attention_set_stream_mode(value);
  else if (k == "prefill_fuse") prefill_tuning_ref().fuse = value;
  else if (k == "prefill_attn_tc") prefill_tuning_ref().attn_tc = value;
  else if (k == "prefill_attn_tc_min_rows") prefill_tuning_ref().attn_tc_min_rows = value;
  else if (k == "prefill_attn_fused_min_rows") prefill_tuning_ref().attn_fused_min_rows = value;
  else if (k == "prefill_attn_tiles") prefill_tuning_ref().attn_tiles = value;
  else if (k == "prefill_tc_split") prefill_tuning_ref().tc_split = value;
  else if (k == "prefill_tc_pair") prefill_tuning_ref().tc_pair = value;
  else if (k == "prefill_tc_sk") gemm_tc_sk_mode() = value;
  else if (k == "prefill_tc_kb") tc_kb_per_stage() = value;
  else if (k == "prefill_sk_kb") sk_kb_per_stage() = value;
  else if (k == "prefill_attn_fused_order") attn_fused_order() = value;
  else if (k == "prefill_gate_fused") gemm_tc_gate_mode() = value;
  else if (k == "prompt_pdl") prompt_pdl() = value;
  else if (k == "tp_debug") tp_set_debug(value);
  else if (k == "loader_staged") set_loader_staged(value);
  else if (k == "use_graph") g_default_opts.use_graph = value;
  else if (k == "use_pdl") g_default_opts.use_pdl = value;
  else if (k == "attn_cluster") g_default_opts.attn_cluster = value;
  else LCU_REQUIRE(false, "unknown tuning key %s", k.c_str());
  return LCU_OK;
}

int lcu_malloc(void** dev_out, uint64_t bytes) {
  NEED_DEVICE();
  LCU_CUDA(cudaMalloc(dev_out, bytes ? bytes : 1));
  return LCU_OK;
}
int lcu_free(void* dev) {
  LCU_CUDA(cudaFree(dev));
  return LCU_OK;
}
int lcu_memcpy_h2d(void* dev, const void* host, uint64_t bytes) {
  LCU_CUDA(cudaMemcpy(dev, host, bytes, cudaMemcpyHostToDevice));
  LCU_CUDA(cudaStreamSynchronize(0));  // complete on return, whatever stream uses the buffer next
  return LCU_OK;
}
int lcu_memcpy_d2h(void* host, const void* dev, uint64_t bytes) {
  LCU_CUDA(cudaMemcpy(host, dev, bytes, cudaMemcpyDeviceToHost));
  return LCU_OK;
}
int lcu_memcpy_d2d(void* dst_dev, const void* src_dev, uint64_t bytes) {
  LCU_CUDA(cudaMemcpy(dst_dev, src_dev, bytes, cudaMemcpyDefault));
  LCU_CUDA(cudaStreamSynchronize(0));
  return LCU_OK;
}
int lcu_memset(void* dev, int value, uint64_t bytes) {
  LCU_CUDA(cudaMemset(dev, value, bytes));
  LCU_CUDA(cudaStreamSynchronize(0));
  return LCU_OK;
}
int lcu_mem_info(uint64_t* free_bytes_out, uint64_t* total_bytes_out) {
  NEED_DEVICE();
  size_t f = 0, t = 0;
  LCU_CUDA(cudaMemGetInfo(&f, &t));
  if (free_bytes_out) *free_bytes_out = f;
  if (total_bytes_out) *total_bytes_out = t;
  return LCU_OK;
}
int lcu_set_device(int device) {
  LCU_CUDA(cudaSetDevice(device));
  return LCU_OK;
}
int lcu_synchronize(void) {
  LCU_CUDA(cudaDeviceSynchronize());
  return LCU_OK;
}

// ---- quantizer
int lcu_quantize_absmax_uint8(void* q_dev, void* scales_dev, const void* in_dev, uint64_t h, uint64_t w, int bs, void* stream) {
  NEED_DEVICE();
  return launch_quantize_absmax_uint8((uint8_t*)q_dev, (__half*)scales_dev, (const __half*)in_dev, h, w, bs, (cudaStream_t)stream);
}
int lcu_dequantize_absmax_uint8(void* out_dev, const void* scales_dev, const void* q_dev, uint64_t h, uint64_t w, int bs, void* stream) {
  NEED_DEVICE();
  return launch_dequantize_absmax_uint8((__half*)out_dev, (const __half*)scales_dev, (const uint8_t*)q_dev, h, w, bs, (cudaStream_t)stream);
}
int lcu_error_stats(float* stats_host, const void* a_dev, const void* b_dev, uint64_t n, void* stream) {
  NEED_DEVICE();
  float* d = nullptr;
  LCU_CUDA(cudaMalloc(&d, (3 * 256 + 4) * sizeof(float)));
  int rc = launch_error_stats(d + 3 * 256, d, (const __half*)a_dev, (const __half*)b_dev, n, (cudaStream_t)stream);
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
  if (!rc && e == cudaSuccess) e = cudaMemcpy(stats_host, d + 3 * 256, 12, cudaMemcpyDeviceToHost);
  cudaFree(d);
  if (rc) return rc;
  LCU_CUDA(e);
  return LCU_OK;
}
int lcu_quantize_host(uint8_t* q_host, uint16_t* scales_host, const uint16_t* in_host, uint64_t h, uint64_t w, int bs, float* stats_host) {
  NEED_DEVICE();
  LCU_REQUIRE(bs > 0 && w % bs == 0, "quantize: block size %d does not divide the row length", bs);
  const size_t n = h * w;
  __half *d_in = nullptr, *d_sc = nullptr, *d_dq = nullptr;
  uint8_t* d_q = nullptr;
  int rc = LCU_OK;
  cudaError_t e = cudaMalloc(&d_in, n * 2 + 16);
  if (e == cudaSuccess) e = cudaMalloc(&d_q, n + 16);
  if (e == cudaSuccess) e = cudaMalloc(&d_sc, n / bs * 2 + 16);
  if (e == cudaSuccess) e = cudaMemcpy(d_in, in_host, n * 2, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) rc = launch_quantize_absmax_uint8(d_q, d_sc, d_in, h, w, bs, 0);
  if (!rc && e == cudaSuccess) e = cudaMemcpy(q_host, d_q, n, cudaMemcpyDeviceToHost);
  if (!rc && e == cudaSuccess) e = cudaMemcpy(scales_host, d_sc, n / bs * 2, cudaMemcpyDeviceToHost);
  if (!rc && e == cudaSuccess && stats_host) {  // the round-trip report of quantize_one (transform.cu:173-178)
    e = cudaMalloc(&d_dq, n * 2 + 16);
    if (e == cudaSuccess) rc = launch_dequantize_absmax_uint8(d_dq, d_sc, d_q, h, w, bs, 0);
    if (!rc && e == cudaSuccess) rc = lcu_error_stats(stats_host, d_in, d_dq, n, nullptr);
  }
  cudaFree(d_in);
  cudaFree(d_q);
  cudaFree(d_sc);
  if (d_dq) cudaFree(d_dq);
  if (rc) return rc;
  LCU_CUDA(e);
  return LCU_OK;
}
int lcu_quantize_model_dir(const char* in_dir, const char* out_dir, int bs) {
  NEED_DEVICE();
  return quantize_dir(in_dir, out_dir, bs);
}

// ---- operators
int lcu_matmul_nt_f16(void* out_dev, const void* lhs_dev, const void* rhs_dev, int m, int k, int n, float beta, void* stream) {
  NEED_DEVICE();
  LCU_REQUIRE(m >= 1, "matmul_nt: m must be positive");
  dev_matrix w;
  w.w = const_cast<void*>(rhs_dev);
  w.rows = n;
  w.cols = k;
  w.bs = 0;
  return matmul_rows((__half*)out_dev, (const __half*)lhs_dev, w, m, beta, scratch_err(), (cudaStream_t)stream);
}
int lcu_matmul_nt_f16_gated(void* out_dev, const void* lhs_dev, const void* w13_dev, int m, int k, int f, int tile, void* stream) {
  NEED_DEVICE();
  return launch_gemm_tc_gated((__half*)out_dev, (const __half*)lhs_dev, k, (const __half*)w13_dev, m, f, k, scratch_err(), (cudaStream_t)stream, tile);
}
int lcu_matmul_nt_fp16u8(void* out_dev, const void* lhs_dev, const void* q_dev, const void* scales_dev, int m, int k, int n, int bs,
                         float beta, void* stream) {
  NEED_DEVICE();
  LCU_REQUIRE(m >= 1, "matmul_nt: m must be positive");
  dev_matrix w;
  w.w = const_cast<void*>(q_dev);
  w.sc = (__half*)const_cast<void*>(scales_dev);
  w.rows = n;
  w.cols = k;
  w.bs = bs;
  return matmul_rows((__half*)out_dev, (const __half*)lhs_dev, w, m, beta, scratch_err(), (cudaStream_t)stream);
}
int lcu_rms_norm(void* out_dev, const void* in_dev, const void* weight_dev, int rows, int dim, float eps, void* stream) {
  NEED_DEVICE();
  return launch_rms_norm((__half*)out_dev, (const __half*)in_dev, (const __half*)weight_dev, rows, dim, eps, (cudaStream_t)stream);
}
int lcu_silu(void* out_dev, const void* a_dev, const void* b_dev, uint64_t n, void* stream) {
  NEED_DEVICE();
  return launch_silu((__half*)out_dev, (const __half*)a_dev, (const __half*)b_dev, n, (cudaStream_t)stream);
}
int lcu_rope_scatter(void* q_dev, const void* k_new_dev, const void* v_new_dev, void* k_cache_dev, void* v_cache_dev, int pos0, int m,
                     int dim, int n_heads, int ctx_len, void* stream) {
  NEED_DEVICE();
  LCU_REQUIRE(pos0 >= 0 && pos0 + m <= ctx_len, "rope_scatter: positions %d..%d outside the context length %d", pos0, pos0 + m, ctx_len);
  const int hd = dim / n_heads;
  float2* table = nullptr;
  LCU_CUDA(cudaMalloc(&table, (size_t)ctx_len * (hd / 2) * sizeof(float2)));
  int rc = launch_rope_table(table, ctx_len, hd, 10000.0f, (cudaStream_t)stream);
  if (!rc)
    rc = launch_rope_scatter((__half*)q_dev, (const __half*)k_new_dev, (const __half*)v_new_dev, (__half*)k_cache_dev, (__half*)v_cache_dev,
                             table, nullptr, pos0, m, dim, n_heads, ctx_len, (cudaStream_t)stream);
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
  cudaFree(table);
  if (rc) return rc;
  LCU_CUDA(e);
  return LCU_OK;
}
int lcu_attention(void* out_dev, const void* q_dev, const void* k_cache_dev, const void* v_cache_dev, int pos0, int m, int dim,
                  int n_heads, int ctx_len, int cluster, void* stream) {
  NEED_DEVICE();
  attn_params at{};
  at.q = (const __half*)q_dev;
  at.ldq = dim;
  at.k_cache = (const __half*)k_cache_dev;
  at.v_cache = (const __half*)v_cache_dev;
  at.out = (__half*)out_dev;
  at.ldo = dim;
  at.pos = nullptr;
  at.pos_value = pos0;
  at.ctx_len = ctx_len;
  at.n_heads = n_heads;
  at.head_dim = dim / n_heads;
  at.err = scratch_err();
  if (cluster == 0) return launch_attention_prefill(at, m, pos0 + m, (cudaStream_t)stream);
  if (cluster == -2) return launch_attention_fused(at, m, pos0 + m, (cudaStream_t)stream);  // tcgen05, one kernel
  if (cluster == -1) {  // tcgen05 path; this stand-alone entry owns no scratch, so the score buffer lives for the call only
    const size_t halves = attention_tc_scratch_halves(n_heads, m, ctx_len);
    __half* scores = nullptr;
    LCU_CUDA(cudaMalloc(&scores, halves * 2));
    cudaMemsetAsync(scores, 0, halves * 2, (cudaStream_t)stream);
    int rc = launch_attention_tc(at, m, pos0 + m, scores, m, (cudaStream_t)stream);
    cudaStreamSynchronize((cudaStream_t)stream);
    cudaFree(scores);
    return rc;
  }
  return launch_attention(at, m, cluster, pos0 + m, (cudaStream_t)stream, 0);
}
int lcu_logits_head(void* probs_dev, const void* logits_dev, int n_vocab, float temperature, int* token_host, void* stream) {
  NEED_DEVICE();
  int* d_tok = scratch_err();
  LCU_REQUIRE(d_tok != nullptr, "logits_head: no scratch");
  head_params h{};
  h.logits = (const __half*)logits_dev;
  h.probs = (__half*)probs_dev;
  h.n_vocab = n_vocab;
  h.temperature = temperature;
  h.token_out = d_tok + 8;
  int rc = launch_logits_head(h, (cudaStream_t)stream, 0);
  if (rc) return rc;
  LCU_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  LCU_CUDA(cudaMemcpy(token_host, d_tok + 8, 4, cudaMemcpyDeviceToHost));
  return LCU_OK;
}

int lcu_synth_fill_f16(void* out_dev, uint64_t n, uint64_t seed, const char* name, float scale, uint64_t first, void* stream) {
  NEED_DEVICE();
  return launch_synth_fill((__half*)out_dev, n, seed, fnv1a64(name), scale, first, (cudaStream_t)stream);
}

// ---- model
int lcu_model_create(const void* params40, const int* layer_gpus, void** model_out) {
  NEED_DEVICE();
  model_params p;
  memcpy(&p, params40, sizeof(p));
  std::unique_ptr<model> m;
  int rc = model::create(m, p, make_partition(p, layer_gpus));
  if (rc) return rc;
  *model_out = m.release();
  return LCU_OK;
}
int lcu_model_load(const char* dir, const int* layer_gpus, void** model_out) {
  NEED_DEVICE();
  model_params p;
  FILE* f = fopen((std::string(dir) + "/params").c_str(), "rb");
  if (!f || fread(&p, 1, sizeof(p), f) != sizeof(p) || fgetc(f) != EOF) {
    if (f) fclose(f);
    set_last_error("cannot read a 40-byte params record from %s/params", dir);
    return LCU_ERR_IO;
  }
  fclose(f);
  std::unique_ptr<model> m;
  int rc = model::create(m, p, make_partition(p, layer_gpus));
  if (rc) return rc;
  rc = m->load_dir(dir);
  if (rc) return rc;
  *model_out = m.release();
  return LCU_OK;
}
int lcu_model_fill_synthetic(void* mdl, uint64_t seed, float scale) { return ((model*)mdl)->fill_synthetic(seed, scale); }
int lcu_model_save(void* mdl, const char* dir) { return ((model*)mdl)->save_dir(dir); }
int lcu_model_tensor(void* mdl, const char* name, int which, void** dev_out, uint64_t* bytes_out, int* device_out) {
  size_t bytes = 0;
  int rc = ((model*)mdl)->find_tensor(name, which, dev_out, &bytes, device_out);
  if (bytes_out) *bytes_out = bytes;
  return rc;
}
int lcu_model_params(void* mdl, void* params40_out) {
  memcpy(params40_out, &((model*)mdl)->params, sizeof(model_params));
  return LCU_OK;
}
uint64_t lcu_model_shadow_bytes(void* mdl) {
  model* m = (model*)mdl;
  if (!m) return 0;
  std::lock_guard<std::mutex> lock(m->shadow_mu);
  return m->shadow_state > 0 ? m->shadow_bytes : 0;
}
uint64_t lcu_model_weight_bytes(void* mdl) { return ((model*)mdl)->weight_bytes_total; }
void lcu_model_free(void* mdl) { delete (model*)mdl; }
uint32_t lcu_ffn_dim(uint32_t dim, uint32_t multiple_of) {
  model_params p{};
  p.dim = dim;
  p.multiple_of = multiple_of;
  return ffn_dim_of(p);
}
int lcu_partition_autopipe(const void* params40, int context_len, int* layer_gpus_out) {
  NEED_DEVICE();
  model_params p;
  memcpy(&p, params40, sizeof(p));
  std::vector<int> lg;
  int rc = autopipe(p, context_len, lg);
  if (rc) return rc;
  memcpy(layer_gpus_out, lg.data(), lg.size() * sizeof(int));
  return LCU_OK;
}
int lcu_partition_is_contiguous(const int* layer_gpus, int n_layers) {
  if (!layer_gpus || n_layers < 1) return 0;
  return partition_is_contiguous(std::vector<int>(layer_gpus, layer_gpus + n_layers)) ? 1 : 0;
}
uint64_t lcu_context_scratch_bytes(const void* params40, int context_len) {
  model_params p;
  memcpy(&p, params40, sizeof(p));
  if (p.dim == 0 || p.n_heads == 0 || p.multiple_of == 0 || context_len < 1) return 0;
  return context_scratch_bytes(p, context_len);
}
uint64_t lcu_context_kv_bytes_per_layer(const void* params40, int context_len) {
  model_params p;
  memcpy(&p, params40, sizeof(p));
  return context_kv_bytes_per_layer(p, context_len);
}
int lcu_partition_even(int n_layers, int n_gpus, int* layer_gpus_out) {
  LCU_REQUIRE(n_layers >= 1 && n_gpus >= 1 && n_gpus <= n_layers, "partition: %d layers over %d GPUs", n_layers, n_gpus);
  for (int l = 0; l < n_layers; ++l) layer_gpus_out[l] = (int)(((long long)l * n_gpus) / n_layers);
  return LCU_OK;
}

// ---- context
int lcu_context_create(void* mdl, int context_len, float temperature, void** ctx_out) {
  NEED_DEVICE();
  context_options opt = g_default_opts;
  opt.context_len = context_len;
  opt.temperature = temperature;
  std::unique_ptr<context> c;
  int rc = context::create(c, (model*)mdl, opt);
  if (rc) return rc;
  *ctx_out = c.release();
  return LCU_OK;
}
void lcu_context_free(void* ctx) { delete (context*)ctx; }
void lcu_context_clear_tokens(void* ctx) { ((context*)ctx)->clear_tokens(); }
uint64_t lcu_context_memory_usage(void* ctx) { return ((context*)ctx)->memory_usage(); }
int lcu_context_tokens_left(void* ctx) { return ((context*)ctx)->tokens_left(); }
int lcu_context_next_token(void* ctx, const int16_t* tokens_host, int n_tokens, int* token_out) {
  return ((context*)ctx)->next_token(tokens_host, n_tokens, token_out);
}
int lcu_context_decode_chained(void* ctx, int16_t first_token, int n_steps, int16_t* tokens_host_out, float* ms_out) {
  return ((context*)ctx)->decode_chained(first_token, n_steps, tokens_host_out, ms_out);
}
int lcu_context_read_probs(void* ctx, uint16_t* probs_host) { return ((context*)ctx)->read_probs((__half*)probs_host); }
int lcu_context_read_hidden(void* ctx, uint16_t* hidden_host) { return ((context*)ctx)->read_hidden((__half*)hidden_host); }
int lcu_context_set_sampling(void* ctx, int mode, uint64_t seed) { return ((context*)ctx)->set_sampling(mode, seed); }
int lcu_context_rollover(void* ctx, int keep) { return ((context*)ctx)->rollover(keep); }
float lcu_sampler_uniform(uint64_t seed, int index) { return sampler_uniform(seed, index); }
int lcu_sample_token(const void* probs_dev, int n_vocab, float u, int* token_host, void* stream) {
  NEED_DEVICE();
  int* d_tok = scratch_err();
  LCU_REQUIRE(d_tok != nullptr && token_host != nullptr, "sample_token: no scratch");
  LCU_REQUIRE(u >= 0.f && u < 1.f, "sample_token: u = %f outside [0, 1)", u);
  int rc = launch_sample((const __half*)probs_dev, n_vocab, 0, nullptr, u, d_tok + 9, nullptr, nullptr, nullptr, 0, (cudaStream_t)stream);
  if (rc) return rc;
  LCU_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  LCU_CUDA(cudaMemcpy(token_host, d_tok + 9, 4, cudaMemcpyDeviceToHost));
  return LCU_OK;
}
int lcu_rollover(void* k_cache_dev, void* v_cache_dev, int n_heads, int ctx_len, int head_dim, int first, int keep, void* stream) {
  NEED_DEVICE();
  LCU_REQUIRE(n_heads >= 1 && head_dim >= 2 && head_dim % 2 == 0, "rollover: bad head shape");
  return launch_rollover((__half*)k_cache_dev, (__half*)v_cache_dev, n_heads, ctx_len, head_dim, first, keep, 10000.0f, (cudaStream_t)stream);
}
int lcu_context_kernels_per_step(void* ctx) { return ((context*)ctx)->kernels_per_step(); }

// ---- tensor-parallel decode
int lcu_tp_check_split(const void* params40, int n_gpus) {
  model_params p;
  memcpy(&p, params40, sizeof(p));
  return tp_check_split(p, n_gpus);
}
int lcu_tp_create(const void* params40, const int* gpus, int n_gpus, int context_len, float temperature, void** tp_out) {
  NEED_DEVICE();
  LCU_REQUIRE(params40 && tp_out && n_gpus >= 1 && n_gpus <= 8, "tp_create: bad arguments");
  model_params p;
  memcpy(&p, params40, sizeof(p));
  int ids[8];
  for (int i = 0; i < n_gpus; ++i) ids[i] = gpus ? gpus[i] : i;
  context_options opt = g_default_opts;
  opt.context_len = context_len;
  opt.temperature = temperature;
  std::unique_ptr<tp_decoder> d;
  int rc = tp_decoder::create(d, p, ids, n_gpus, opt);
  if (rc) return rc;
  *tp_out = d.release();
  return LCU_OK;
}
int lcu_tp_fill_synthetic(void* tp, uint64_t seed, float scale) { return ((tp_decoder*)tp)->fill_synthetic(seed, scale); }
int lcu_tp_load(void* tp, const char* dir) { return ((tp_decoder*)tp)->load_dir(dir); }
int lcu_tp_next_token(void* tp, const int16_t* tokens_host, int n_tokens, int* token_out) {
  return ((tp_decoder*)tp)->next_token(tokens_host, n_tokens, token_out);
}
int lcu_tp_decode_chained(void* tp, int16_t first_token, int n_steps, int16_t* tokens_host_out, float* ms_out) {
  return ((tp_decoder*)tp)->decode_chained(first_token, n_steps, tokens_host_out, ms_out);
}
int lcu_tp_read_probs(void* tp, uint16_t* probs_host) { return ((tp_decoder*)tp)->read_probs((__half*)probs_host); }
void lcu_tp_clear_tokens(void* tp) { ((tp_decoder*)tp)->clear_tokens(); }
int lcu_tp_tokens_left(void* tp) { return ((tp_decoder*)tp)->tokens_left(); }
int lcu_tp_kernels_per_step(void* tp) { return ((tp_decoder*)tp)->kernels_per_step(); }
uint64_t lcu_tp_weight_bytes_per_gpu(void* tp) { return ((tp_decoder*)tp)->weight_bytes_per_gpu(); }
void lcu_tp_free(void* tp) { delete (tp_decoder*)tp; }

// ---- measurement
int lcu_bench_decode_kernel(void* ctx, int which, int reps, float* ms_per_launch_out, uint64_t* bytes_per_launch_out) {
  return ((context*)ctx)->bench_kernel(which, reps, ms_per_launch_out, bytes_per_launch_out);
}
int lcu_profiler_start(void) {
  LCU_CUDA(cudaProfilerStart());
  return LCU_OK;
}
int lcu_profiler_stop(void) {
  LCU_CUDA(cudaProfilerStop());
  return LCU_OK;
}
int lcu_selftest_quantizer_arithmetic(uint64_t* checked_out, uint64_t* differences_out) {
  NEED_DEVICE();
  unsigned long long a = 0, b = 0;
  int rc = quantizer_arithmetic_check(&a, &b);
  *checked_out = a;
  *differences_out = b;
  return rc;
}
int lcu_selftest_balanced_schedule(int n_tiles, int k_steps, int sm_pairs) { return gemm_tc_sk_check_schedule(n_tiles, k_steps, sm_pairs); }
int lcu_plan_long_prompt_gemm(int m, int n, int k, int sms, int* kernel_out) {
  LCU_REQUIRE(m > 128 && n >= 128 && n % 128 == 0 && k >= 64 && k % 64 == 0 && sms >= 2 && kernel_out, "plan_long_prompt_gemm: bad arguments");
  *kernel_out = gemm_tc_plan_long(m, n, k, sms);
  return LCU_OK;
}
int lcu_plan_short_prompt_gemm(int n, int k, int sms, int* tile_n_out, int* split_out) {
  LCU_REQUIRE(n >= 128 && n % 128 == 0 && k >= 64 && k % 64 == 0 && sms >= 2 && tile_n_out && split_out, "plan_short_prompt_gemm: bad arguments");
  gemm_tc_plan_short(n, k, sms, tile_n_out, split_out);
  return LCU_OK;
}
int lcu_selftest_silu_arithmetic(uint64_t* checked_out, uint64_t* differences_out) {
  NEED_DEVICE();
  unsigned long long a = 0, b = 0;
  int rc = silu_arithmetic_check(&a, &b);
  *checked_out = a;
  *differences_out = b;
  return rc;
}
int lcu_selftest_bounded_wait(int* device_code_out) {
  NEED_DEVICE();
  int* err = scratch_err();
  LCU_REQUIRE(err != nullptr, "selftest: no scratch");
  LCU_CUDA(cudaMemset(err, 0, 4));
  int rc = run_bounded_wait_probe(err, 0);
  if (rc) return rc;
  LCU_CUDA(cudaDeviceSynchronize());
  int code = 0;
  LCU_CUDA(cudaMemcpy(&code, err, 4, cudaMemcpyDeviceToHost));
  LCU_CUDA(cudaMemset(err, 0, 4));
  if (device_code_out) *device_code_out = code;
  if (code != 0) {
    set_last_error("a kernel gave up on a bounded wait (device code 0x%x)", code);
    return LCU_ERR_DEVICE_WAIT;
  }
  return LCU_OK;
}
int lcu_bench_matmul_f16(void* out_dev, const void* lhs_dev, const void* rhs_dev, int m, int k, int n, int reps, float* ms_per_launch_out) {
  NEED_DEVICE();
  LCU_REQUIRE(reps >= 1 && ms_per_launch_out, "bench_matmul: bad arguments");
  cudaEvent_t e0, e1;
  LCU_CUDA(cudaEventCreate(&e0));
  LCU_CUDA(cudaEventCreate(&e1));
  int rc = lcu_matmul_nt_f16(out_dev, lhs_dev, rhs_dev, m, k, n, 0.f, nullptr);  // warm: attributes, tensor maps
  if (rc == LCU_OK) {
    cudaEventRecord(e0, 0);
    for (int i = 0; i < reps && rc == LCU_OK; ++i) rc = lcu_matmul_nt_f16(out_dev, lhs_dev, rhs_dev, m, k, n, 0.f, nullptr);
    cudaEventRecord(e1, 0);
    if (cudaEventSynchronize(e1) != cudaSuccess) rc = LCU_ERR_CUDA;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    *ms_per_launch_out = ms / reps;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return rc;
}
int lcu_bench_quantize(uint64_t h, uint64_t w, int bs, int reps, float* ms_per_launch_out) {
  NEED_DEVICE();
  LCU_REQUIRE(reps >= 1 && ms_per_launch_out && bs > 0 && w % bs == 0 && h > 0, "bench_quantize: bad arguments");
  const size_t n = h * w;
  __half *d_in = nullptr, *d_sc = nullptr;
  uint8_t* d_q = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaError_t e = cudaMalloc(&d_in, n * 2);
  if (e == cudaSuccess) e = cudaMalloc(&d_q, n);
  if (e == cudaSuccess) e = cudaMalloc(&d_sc, n / bs * 2);
  if (e == cudaSuccess) e = cudaEventCreate(&e0);
  if (e == cudaSuccess) e = cudaEventCreate(&e1);
  int rc = LCU_OK;
  if (e == cudaSuccess) rc = launch_synth_fill(d_in, n, 1234, fnv1a64("bench.quantize"), 0.02f, 0, 0);
  if (e == cudaSuccess && !rc) rc = launch_quantize_absmax_uint8(d_q, d_sc, d_in, h, w, bs, 0);  // warm
  if (e == cudaSuccess && !rc) {
    cudaEventRecord(e0, 0);
    for (int i = 0; i < reps && !rc; ++i) rc = launch_quantize_absmax_uint8(d_q, d_sc, d_in, h, w, bs, 0);
    cudaEventRecord(e1, 0);
    e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    *ms_per_launch_out = ms / reps;
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(d_in);
  cudaFree(d_q);
  cudaFree(d_sc);
  if (rc) return rc;
  LCU_CUDA(e);
  return LCU_OK;
}
int lcu_bench_read_ceiling(uint64_t bytes, int reps, int copies_per_stage, float* ms_per_pass_out) {
  NEED_DEVICE();
  return bench_read_ceiling(bytes, reps, copies_per_stage, ms_per_pass_out);
}

}  // extern "C"
