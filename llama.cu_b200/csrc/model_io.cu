// Weight-directory output, the directory-to-directory quantizer and the memory-based partitioner.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <vector>

#include "ops.cuh"
#include "runtime.cuh"

namespace lcu {
namespace {

int write_file(const std::string& path, const void* data, size_t bytes) {
  FILE* f = fopen(path.c_str(), "wb");
  if (!f) {
    set_last_error("cannot create %s", path.c_str());
    return LCU_ERR_IO;
  }
  const size_t done = bytes ? fwrite(data, 1, bytes, f) : 0;
  if (fclose(f) != 0 || done != bytes) {
    set_last_error("short write to %s", path.c_str());
    return LCU_ERR_IO;
  }
  return LCU_OK;
}

int read_file(const std::string& path, void* data, size_t bytes) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) {
    set_last_error("cannot open %s", path.c_str());
    return LCU_ERR_IO;
  }
  fseek(f, 0, SEEK_END);
  const long sz = ftell(f);
  fseek(f, 0, SEEK_SET);
  const bool ok = (size_t)sz == bytes && fread(data, 1, bytes, f) == bytes;
  fclose(f);
  if (!ok) {
    set_last_error("%s: expected %zu bytes, file has %ld", path.c_str(), bytes, sz);
    return LCU_ERR_IO;
  }
  return LCU_OK;
}

int save_device(const std::string& path, const void* dev, size_t bytes, std::vector<char>& host) {
  host.resize(bytes);
  LCU_CUDA(cudaMemcpy(host.data(), dev, bytes, cudaMemcpyDeviceToHost));
  return write_file(path, host.data(), bytes);
}

struct named_shape {
  std::string name;
  size_t rows, cols;  // cols == 0: vector of `rows` elements
};

// tensor list of a weight directory (reference llama_cu.cu:893-918)
std::vector<named_shape> shapes_of(const model_params& p) {
  const size_t d = p.dim, f = ffn_dim_of(p), v = p.n_vocab;
  std::vector<named_shape> out;
  out.push_back({"tok_embeddings", v, d});
  out.push_back({"output", v, d});
  out.push_back({"norm", d, 0});
  for (uint32_t i = 0; i < p.n_layers; ++i) {
    const std::string b = "layers." + std::to_string(i) + ".";
    out.push_back({b + "attention_norm", d, 0});
    out.push_back({b + "ffn_norm", d, 0});
    out.push_back({b + "attention.wq", d, d});
    out.push_back({b + "attention.wk", d, d});
    out.push_back({b + "attention.wv", d, d});
    out.push_back({b + "attention.wo", d, d});
    out.push_back({b + "feed_forward.w1", f, d});
    out.push_back({b + "feed_forward.w2", d, f});
    out.push_back({b + "feed_forward.w3", f, d});
  }
  return out;
}

}  // namespace

int model::save_dir(const std::string& dir) {
  LCU_REQUIRE(tp_size == 1, "model: a tensor-parallel shard cannot be saved as a weight directory");
  mkdir(dir.c_str(), 0777);
  std::vector<char> host;
  int rc = write_file(dir + "/params", &params, sizeof(params));
  if (rc) return rc;
  for (const named_shape& s : shapes_of(params)) {
    void* ptr = nullptr;
    size_t bytes = 0;
    int dev = 0;
    rc = find_tensor(s.name, 0, &ptr, &bytes, &dev);
    if (rc) return rc;
    device_guard dg(dev);  // the tensor's GPU for the copy; the caller's current device is left as it was
    const std::string base = dir + "/" + s.name;
    if (s.cols == 0) {
      rc = save_device(base + ".weight__" + std::to_string(s.rows), ptr, bytes, host);
    } else {
      rc = save_device(base + ".weight__" + std::to_string(s.rows) + "_" + std::to_string(s.cols), ptr, bytes, host);
      if (!rc && params.q_type) {
        rc = find_tensor(s.name, 1, &ptr, &bytes, &dev);
        if (!rc)
          rc = save_device(base + ".scale__" + std::to_string(s.rows) + "_" + std::to_string(s.cols / params.quantization_block_size),
                           ptr, bytes, host);
      }
    }
    if (rc) return rc;
  }
  return LCU_OK;
}

int quantize_dir(const std::string& in_dir, const std::string& out_dir, int bs) {
  model_params p;
  int rc = read_file(in_dir + "/params", &p, sizeof(p));
  if (rc) return rc;
  LCU_REQUIRE(p.magic == PARAMS_MAGIC && p.fourcc == PARAMS_FOURCC, "quantize: bad magic in %s/params", in_dir.c_str());
  LCU_REQUIRE(p.q_type == 0, "quantize: input model is not fp16");  // transform.cu:224-227
  LCU_REQUIRE(bs > 0 && bs % 4 == 0 && p.dim % bs == 0 && ffn_dim_of(p) % bs == 0, "quantize: block size %d does not divide the row lengths", bs);
  mkdir(out_dir.c_str(), 0777);
  std::vector<char> host;
  size_t max_elems = 0;
  for (const named_shape& s : shapes_of(p)) max_elems = std::max(max_elems, s.cols ? s.rows * s.cols : 0);
  __half* d_in = nullptr;
  uint8_t* d_q = nullptr;
  __half* d_sc = nullptr;
  cudaError_t ea = cudaMalloc(&d_in, max_elems * 2);
  if (ea == cudaSuccess) ea = cudaMalloc(&d_q, max_elems);
  if (ea == cudaSuccess) ea = cudaMalloc(&d_sc, max_elems / bs * 2);
  if (ea != cudaSuccess) {  // nothing stays allocated when one of the three fails
    cudaFree(d_in);
    cudaFree(d_q);
    cudaFree(d_sc);
    LCU_CUDA(ea);
  }
  for (const named_shape& s : shapes_of(p)) {
    const std::string ib = in_dir + "/" + s.name, ob = out_dir + "/" + s.name;
    if (s.cols == 0) {  // norm vectors are copied verbatim (transform.cu:198-218)
      host.resize(s.rows * 2);
      rc = read_file(ib + ".weight__" + std::to_string(s.rows), host.data(), host.size());
      if (!rc) rc = write_file(ob + ".weight__" + std::to_string(s.rows), host.data(), host.size());
    } else {
      const size_t n = s.rows * s.cols;
      const std::string dims = std::to_string(s.rows) + "_" + std::to_string(s.cols);
      host.resize(n * 2);
      rc = read_file(ib + ".weight__" + dims, host.data(), n * 2);
      if (rc) break;
      if (cudaMemcpy(d_in, host.data(), n * 2, cudaMemcpyHostToDevice) != cudaSuccess) rc = LCU_ERR_CUDA;
      if (!rc) rc = launch_quantize_absmax_uint8(d_q, d_sc, d_in, s.rows, s.cols, bs, 0);
      if (!rc) rc = save_device(ob + ".weight__" + dims, d_q, n, host);
      if (!rc) rc = save_device(ob + ".scale__" + std::to_string(s.rows) + "_" + std::to_string(s.cols / bs), d_sc, n / bs * 2, host);
    }
    if (rc) break;
  }
  cudaFree(d_in);
  cudaFree(d_q);
  cudaFree(d_sc);
  if (rc) return rc;
  model_params q = p;  // transform.cu:253-261
  q.q_type = 1;
  q.quantization_block_size = (uint16_t)bs;
  return write_file(out_dir + "/params", &q, sizeof(q));
}

int autopipe(const model_params& p, int context_len, std::vector<int>& layer_gpus) {
  int ndev = 0;
  LCU_CUDA(cudaGetDeviceCount(&ndev));
  const size_t d = p.dim, f = ffn_dim_of(p), v = p.n_vocab;
  const size_t bs = p.q_type ? p.quantization_block_size : 0;
  auto mat = [&](size_t r, size_t c) { return bs ? r * c + r * (c / bs) * 2 : r * c * 2; };
  const size_t layer_bytes = 4 * mat(d, d) + 2 * mat(f, d) + mat(d, f) + 2 * d * 2 + 9 * 256  // weights + norms (256-byte aligned)
                             + context_kv_bytes_per_layer(p, context_len);                    // + K and V cache of the layer
  // what context::create allocates on every GPU it uses (activations, the prompt path's score and dequantization
  // buffers, tables) + a margin for the CUDA context's own growth (graphs, module loading)
  const size_t scratch = context_scratch_bytes(p, context_len) + (64u << 20);
  const size_t embed_bytes = mat(v, d), out_bytes = mat(v, d) + d * 2;
  layer_gpus.clear();
  int gpu = 0;
  size_t used = scratch + embed_bytes;
  auto free_on = [&](int g) {
    size_t a = 0, t = 0;
    cudaSetDevice(g);
    cudaMemGetInfo(&a, &t);
    return a;
  };
  int prev = 0;
  cudaGetDevice(&prev);
  size_t avail = ndev ? free_on(0) : 0;
  for (uint32_t l = 0; l < p.n_layers && gpu < ndev; ++l) {
    const size_t need = layer_bytes + (l + 1 == p.n_layers ? out_bytes : 0);
    while (gpu < ndev && used + need > avail) {
      ++gpu;
      used = scratch;
      if (gpu < ndev) avail = free_on(gpu);
    }
    if (gpu < ndev) {
      layer_gpus.push_back(gpu);
      used += need;
    }
  }
  cudaSetDevice(prev);
  LCU_REQUIRE(layer_gpus.size() == p.n_layers, "autopipe: the model does not fit the %d visible GPUs", ndev);
  return LCU_OK;
}

}  // namespace lcu
