// Model storage and the forward pass.
//
// Drop-in scope: what the reference does in llama_model_impl (llama_cu.cu:888-997) and
// llama_context_impl (llama_cu.cu:999-1304), re-planned for B200:
//   * all weights of a GPU live in one arena (one cudaMalloc), tensors 256-byte aligned, in the
//     reference's own [rows][K] row-major layout, so the files of a weight directory load as is;
//   * the KV cache is head-major [head][position][head_dim] with keys stored already rotated
//     (the reference re-rotates the whole prefix every step, llama_cu.cu:1150-1153);
//   * a decode step is 5 kernels per layer (fused norm+QKV+RoPE+cache write, attention,
//     wo+residual, norm+w1|w3+SiLU, w2+residual) instead of 15, no allocation, no host
//     synchronisation, replayed as one CUDA graph with programmatic dependent launches;
//   * the position is read from device memory, so the same graph serves every step and greedy
//     decoding can run chained on the device.
#include "runtime.cuh"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstring>
#include <thread>

#include "attention.cuh"
#include "gemm_tc.cuh"
#include "gemv.cuh"
#include "ops.cuh"
#include "prefill.cuh"

namespace lcu {

// ------------------------------------------------------------------ error text
static thread_local char g_err[512] = "";
void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_err; }

#define LCU_TRY(expr)      \
  do {                     \
    int _rc = (expr);      \
    if (_rc) return _rc;   \
  } while (0)

// 64 zeroed device words per GPU for the stand-alone operator entry points (word 0: error word of their kernels;
// word 8: token of lcu_logits_head); allocated at the first use on a device
int* device_scratch_words() {
  static int* ptr[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptr[dev]) {
    if (cudaMalloc(&ptr[dev], 256) != cudaSuccess) return nullptr;
    cudaMemset(ptr[dev], 0, 256);
    cudaStreamSynchronize(0);  // the kernels that get this word run on other streams
  }
  return ptr[dev];
}

uint32_t ffn_dim_of(const model_params& p) {
  uint32_t a = p.dim * 8 / 3;
  return (a + p.multiple_of - 1) / p.multiple_of * p.multiple_of;
}

// A pipeline stage is one contiguous run of layers: the forward pass keeps the final norm and the output matrix on the
// GPU of the last layer and hands the residual row from stage to stage, so a GPU may not reappear once it was left.
bool partition_is_contiguous(const std::vector<int>& layer_gpus) {
  std::vector<int> seen;
  for (size_t i = 0; i < layer_gpus.size(); ++i) {
    if (i > 0 && layer_gpus[i] == layer_gpus[i - 1]) continue;
    if (std::find(seen.begin(), seen.end(), layer_gpus[i]) != seen.end()) return false;
    seen.push_back(layer_gpus[i]);
  }
  return true;
}

std::vector<int> partition::used_gpus() const {
  std::vector<int> out;
  for (int g : layer_gpus)
    if (std::find(out.begin(), out.end(), g) == out.end()) out.push_back(g);
  return out;
}

// ------------------------------------------------------------------ model
namespace {
constexpr size_t ALIGN = 256;
struct carve {
  size_t off = 0;
  size_t take(size_t bytes) {
    size_t o = off;
    off += round_up(bytes, ALIGN);
    return o;
  }
};

struct tensor_slot {  // one named tensor of the weight directory
  std::string name;
  dev_matrix* mat;    // matrix, or
  __half** vec;       // norm vector
  size_t len;         // vector length
  int device;
  size_t full_rows = 0;  // rows of the whole matrix as named in the weight directory
  size_t row0 = 0;       // first of them held by this model (a tensor-parallel shard holds full_rows / tp_size rows)
};

std::vector<tensor_slot> enumerate(model& m) {
  const model_params& p = m.params;
  std::vector<tensor_slot> out;
  // every layer matrix and the output matrix are split by rows over the tensor-parallel ranks; the embedding table
  // (one row is read per token) stays whole on every rank
  auto mat = [&](const std::string& name, dev_matrix& d, size_t rows, size_t cols, int dev, bool sharded = true) {
    const size_t local = sharded ? rows / m.tp_size : rows;
    d.rows = local;
    d.cols = cols;
    d.bs = p.q_type ? p.quantization_block_size : 0;
    tensor_slot t{name, &d, nullptr, 0, dev};
    t.full_rows = rows;
    t.row0 = sharded ? local * m.tp_rank : 0;
    out.push_back(t);
  };
  auto vec = [&](const std::string& name, __half*& v, size_t len, int dev) { out.push_back({name, nullptr, &v, len, dev}); };
  mat("tok_embeddings", m.tok_embeddings, p.n_vocab, p.dim, m.part.embedding_gpu(), false);
  for (uint32_t i = 0; i < p.n_layers; ++i) {
    layer_weights& L = m.layers[i];
    const int dev = m.part.layer_gpus[i];
    const std::string b = "layers." + std::to_string(i) + ".";
    vec(b + "attention_norm", L.attn_norm, p.dim, dev);
    vec(b + "ffn_norm", L.ffn_norm, p.dim, dev);
    mat(b + "attention.wq", L.wq, p.dim, p.dim, dev);
    mat(b + "attention.wk", L.wk, p.dim, p.dim, dev);
    mat(b + "attention.wv", L.wv, p.dim, p.dim, dev);
    mat(b + "attention.wo", L.wo, p.dim, p.dim, dev);
    mat(b + "feed_forward.w1", L.w1, m.ffn, p.dim, dev);
    mat(b + "feed_forward.w3", L.w3, m.ffn, p.dim, dev);
    mat(b + "feed_forward.w2", L.w2, p.dim, m.ffn, dev);
  }
  vec("norm", m.norm, p.dim, m.part.output_gpu());
  mat("output", m.output, p.n_vocab, p.dim, m.part.output_gpu());
  return out;
}
}  // namespace

model::~model() {
  for (auto& a : arenas) {
    device_guard g(a.first);
    cudaFree(a.second);
  }
  for (auto& a : shadow_arenas) {
    device_guard g(a.first);
    cudaFree(a.second);
  }
}

int& u8_shadow_mode() {
  static int mode = 1;
  return mode;
}

void model::shadow_touch() {
  std::lock_guard<std::mutex> lock(shadow_mu);
  if (shadow_state == 1) shadow_state = 2;
}

bool model::shadow_ready(bool may_allocate) {
  std::lock_guard<std::mutex> lock(shadow_mu);
  if (shadow_state == 1) return true;
  if (shadow_state < 0) return false;
  const model_params& p = params;
  const int bs = p.q_type ? (int)p.quantization_block_size : 0;
  if (bs == 0 || tp_size != 1 || !u8_shadow_mode()) return false;  // (not remembered: the mode may be switched on later)
  const size_t d = p.dim, f = ffn;
  const size_t per_layer = (3 * d * d + d * d + 2 * f * d + d * f) * 2;
  if (shadow_state == 0 && !may_allocate) return false;
  if (shadow_state == 0) {
    // one allocation per GPU that holds layers; all or nothing
    std::vector<std::pair<int, size_t>> need;
    for (uint32_t l = 0; l < p.n_layers; ++l) {
      const int dev = part.layer_gpus[l];
      auto it = std::find_if(need.begin(), need.end(), [&](const std::pair<int, size_t>& a) { return a.first == dev; });
      if (it == need.end()) need.emplace_back(dev, per_layer);
      else it->second += per_layer;
    }
    bool fits = true;
    for (auto& n : need) {
      device_guard g(n.first);
      size_t free_b = 0, total_b = 0;
      if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess || free_b < n.second + ((size_t)6 << 30)) fits = false;
    }
    if (fits)
      for (auto& n : need) {
        device_guard g(n.first);
        void* base = nullptr;
        if (cudaMalloc(&base, n.second) != cudaSuccess) {
          cudaGetLastError();
          fits = false;
          break;
        }
        shadow_arenas.emplace_back(n.first, base);
      }
    if (!fits) {
      for (auto& a : shadow_arenas) {
        device_guard g(a.first);
        cudaFree(a.second);
      }
      shadow_arenas.clear();
      shadow_state = -1;
      return false;
    }
    shadow_layers = layers;
    std::vector<size_t> used(shadow_arenas.size(), 0);
    shadow_bytes = 0;
    for (uint32_t l = 0; l < p.n_layers; ++l) {
      size_t ai = 0;
      while (shadow_arenas[ai].first != part.layer_gpus[l]) ++ai;
      __half* at = reinterpret_cast<__half*>((char*)shadow_arenas[ai].second + used[ai]);
      layer_weights& S = shadow_layers[l];
      dev_matrix* order[7] = {&S.wq, &S.wk, &S.wv, &S.wo, &S.w1, &S.w3, &S.w2};
      for (dev_matrix* mt : order) {
        mt->w = at;
        mt->sc = nullptr;
        mt->bs = 0;
        at += mt->rows * mt->cols;
      }
      used[ai] += per_layer;
      shadow_bytes += per_layer;
    }
  }
  // (re)fill: the kernel the per-pass expansion uses, the values the reference's tile kernel builds in shared
  // memory (llama_cu.cu:287-289)
  bool ok = true;
  for (uint32_t l = 0; l < p.n_layers && ok; ++l) {
    device_guard g(part.layer_gpus[l]);
    const layer_weights& L = layers[l];
    const layer_weights& S = shadow_layers[l];
    const dev_matrix* src[7] = {&L.wq, &L.wk, &L.wv, &L.wo, &L.w1, &L.w3, &L.w2};
    const dev_matrix* dst[7] = {&S.wq, &S.wk, &S.wv, &S.wo, &S.w1, &S.w3, &S.w2};
    for (int i = 0; i < 7 && ok; ++i)
      ok = launch_dequantize_absmax_uint8((__half*)dst[i]->w, src[i]->sc, (const uint8_t*)src[i]->w, src[i]->rows, src[i]->cols, bs, nullptr) == LCU_OK;
  }
  for (auto& a : shadow_arenas) {
    device_guard g(a.first);
    if (cudaDeviceSynchronize() != cudaSuccess) ok = false;
  }
  shadow_state = ok ? 1 : -1;
  return ok;
}

int model::create(std::unique_ptr<model>& out, const model_params& p, const partition& part, int tp_rank, int tp_size) {
  LCU_REQUIRE(p.magic == PARAMS_MAGIC && p.fourcc == PARAMS_FOURCC, "model: bad magic in params");
  LCU_REQUIRE(p.dim > 0 && p.n_heads > 0 && p.n_layers > 0 && p.n_vocab > 0 && p.multiple_of > 0, "model: empty dimension in params");
  LCU_REQUIRE(p.dim % p.n_heads == 0, "model: dim %u not divisible by n_heads %u", p.dim, p.n_heads);
  LCU_REQUIRE(p.dim % 256 == 0, "model: dim %u must be a multiple of 256", p.dim);
  LCU_REQUIRE(p.n_vocab <= 32768 && p.n_vocab % 2 == 0, "model: n_vocab %u must be even and fit a 16-bit token id", p.n_vocab);
  LCU_REQUIRE(p.q_type <= 1, "model: unsupported quantization type %u", p.q_type);
  const uint32_t ffn = ffn_dim_of(p);
  LCU_REQUIRE(ffn % 256 == 0, "model: ffn dim %u must be a multiple of 256", ffn);
  if (p.q_type) {
    const int bs = p.quantization_block_size;
    LCU_REQUIRE(bs == 32 || bs == 64 || bs == 128, "model: quantization block size %d not in {32,64,128}", bs);
  }
  LCU_REQUIRE(part.layer_gpus.size() == p.n_layers, "model: partition has %zu layers, params %u", part.layer_gpus.size(), p.n_layers);
  int ndev = 0;
  LCU_CUDA(cudaGetDeviceCount(&ndev));
  for (int g : part.layer_gpus) LCU_REQUIRE(g >= 0 && g < ndev, "model: partition names GPU %d but %d are visible", g, ndev);
  LCU_REQUIRE(partition_is_contiguous(part.layer_gpus),
              "model: partition returns to a GPU after leaving it; every GPU must hold one contiguous range of layers");

  LCU_REQUIRE(tp_size >= 1 && tp_rank >= 0 && tp_rank < tp_size, "model: tensor-parallel rank %d of %d", tp_rank, tp_size);
  if (tp_size > 1) {
    LCU_REQUIRE(p.n_heads % tp_size == 0, "model: %u heads do not split over %d GPUs", p.n_heads, tp_size);
    LCU_REQUIRE((ffn / tp_size) * tp_size == ffn && (ffn / tp_size) % 2 == 0 && (p.n_vocab / tp_size) * tp_size == p.n_vocab &&
                    (p.n_vocab / tp_size) % 2 == 0,
                "model: ffn dim %u and vocabulary %u must split into even row counts over %d GPUs", ffn, p.n_vocab, tp_size);
  }
  auto m = std::make_unique<model>();
  m->params = p;
  m->ffn = ffn;
  m->part = part;
  m->tp_rank = tp_rank;
  m->tp_size = tp_size;
  m->layers.resize(p.n_layers);
  auto slots = enumerate(*m);
  // size and carve one arena per GPU
  for (int dev : part.used_gpus()) {
    carve c;
    for (auto& s : slots)
      if (s.device == dev) {
        if (s.mat) {
          c.take(s.mat->weight_bytes());
          c.take(s.mat->scale_bytes());
        } else {
          c.take(s.len * 2);
        }
      }
    device_guard g(dev);
    void* base = nullptr;
    LCU_CUDA(cudaMalloc(&base, c.off));
    m->arenas.push_back({dev, base});
    m->weight_bytes_total += c.off;
    carve c2;
    for (auto& s : slots)
      if (s.device == dev) {
        if (s.mat) {
          s.mat->w = (char*)base + c2.take(s.mat->weight_bytes());
          size_t so = c2.take(s.mat->scale_bytes());
          s.mat->sc = s.mat->bs ? (__half*)((char*)base + so) : nullptr;
        } else {
          *s.vec = (__half*)((char*)base + c2.take(s.len * 2));
        }
      }
  }
  out = std::move(m);
  return LCU_OK;
}

int model::find_tensor(const std::string& name, int which, void** ptr, size_t* bytes, int* device) {
  shadow_touch();  // (the caller gets a writable pointer)
  for (auto& s : enumerate(*this)) {
    if (s.name != name) continue;
    if (device) *device = s.device;
    if (s.mat) {
      LCU_REQUIRE(which == 0 || s.mat->bs, "tensor %s has no scales", name.c_str());
      *ptr = which == 0 ? s.mat->w : (void*)s.mat->sc;
      *bytes = which == 0 ? s.mat->weight_bytes() : s.mat->scale_bytes();
    } else {
      LCU_REQUIRE(which == 0, "tensor %s has no scales", name.c_str());
      *ptr = *s.vec;
      *bytes = s.len * 2;
    }
    return LCU_OK;
  }
  LCU_REQUIRE(false, "no tensor named %s", name.c_str());
}

namespace {
// copies a whole file of exactly `bytes` bytes into device memory: the reference's way (llama_cu.cu:699-702, 929-971),
// a file mapping handed to one blocking copy from pageable memory.  Kept as the baseline of the loader measurement.
// (`file_bytes` is the size the whole file must have; [file_off, file_off + bytes) is the part that is loaded)
int load_file_mapped(const std::string& path, void* dst, size_t bytes, size_t file_off, size_t file_bytes) {
  int fd = open(path.c_str(), O_RDONLY);
  if (fd < 0) {
    set_last_error("cannot open %s", path.c_str());
    return LCU_ERR_IO;
  }
  struct stat st;
  if (fstat(fd, &st) != 0 || (size_t)st.st_size != file_bytes) {
    close(fd);
    set_last_error("%s: expected %zu bytes, file has %lld", path.c_str(), file_bytes, (long long)st.st_size);
    return LCU_ERR_IO;
  }
  void* map = file_bytes ? mmap(nullptr, file_bytes, PROT_READ, MAP_PRIVATE, fd, 0) : nullptr;
  close(fd);
  if (file_bytes && map == MAP_FAILED) {
    set_last_error("cannot map %s", path.c_str());
    return LCU_ERR_IO;
  }
  // a copy from pageable memory may return while its last piece is still on the way to the device, and the
  // contexts' streams do not wait for the default stream: finish it here
  cudaError_t e = bytes ? cudaMemcpy(dst, (const char*)map + file_off, bytes, cudaMemcpyHostToDevice) : cudaSuccess;
  if (bytes && e == cudaSuccess) e = cudaStreamSynchronize(0);
  if (file_bytes) munmap(map, file_bytes);
  if (e != cudaSuccess) {
    set_last_error("copy of %s to the device failed: %s", path.c_str(), cudaGetErrorString(e));
    return LCU_ERR_CUDA;
  }
  return LCU_OK;
}

// Staged loader: files are read in pieces into two pinned buffers; while one piece travels to the device
// (cudaMemcpyAsync on the loader's stream, one copy per piece) the next one is read from the file.  One loader per
// GPU of the partition; finish() waits for the last copies.
struct staged_loader {
  static constexpr size_t PIECE = (size_t)64 << 20;
  static constexpr int READERS = 8;
  int device = 0;
  void* pin[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
  bool in_flight[2] = {false, false};
  cudaStream_t stream = nullptr;
  int cur = 0;

  int init(int dev) {
    device = dev;
    device_guard g(dev);
    LCU_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      LCU_CUDA(cudaMallocHost(&pin[i], PIECE));
      LCU_CUDA(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
    }
    return LCU_OK;
  }
  ~staged_loader() {
    device_guard g(device);
    if (stream) cudaStreamSynchronize(stream);
    for (int i = 0; i < 2; ++i) {
      if (pin[i]) cudaFreeHost(pin[i]);
      if (done[i]) cudaEventDestroy(done[i]);
    }
    if (stream) cudaStreamDestroy(stream);
  }
  int copy_file(const std::string& path, void* dst, size_t bytes, size_t file_off, size_t file_bytes) {
    int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) {
      set_last_error("cannot open %s", path.c_str());
      return LCU_ERR_IO;
    }
    struct stat st;
    if (fstat(fd, &st) != 0 || (size_t)st.st_size != file_bytes) {
      close(fd);
      set_last_error("%s: expected %zu bytes, file has %lld", path.c_str(), file_bytes, (long long)st.st_size);
      return LCU_ERR_IO;
    }
#ifdef POSIX_FADV_SEQUENTIAL
    posix_fadvise(fd, 0, 0, POSIX_FADV_SEQUENTIAL);
#endif
    device_guard g(device);
    for (size_t off = 0; off < bytes;) {
      const size_t n = std::min(PIECE, bytes - off);
      if (in_flight[cur]) {  // the buffer's previous piece must have left it
        if (cudaEventSynchronize(done[cur]) != cudaSuccess) {
          close(fd);
          set_last_error("copy of %s to the device failed", path.c_str());
          return LCU_ERR_CUDA;
        }
        in_flight[cur] = false;
      }
      // the piece is read by several threads at once (a single reader copies out of the page cache at a fraction of
      // what the host-to-device link takes)
      const int n_readers = n >= ((size_t)4 << 20) ? READERS : 1;
      const size_t share = (n / n_readers + 4095) & ~(size_t)4095;
      std::atomic<int> failed{0};
      auto read_range = [&](size_t lo, size_t hi) {
        while (lo < hi) {
          const ssize_t r = pread(fd, (char*)pin[cur] + lo, hi - lo, (off_t)(file_off + off + lo));
          if (r <= 0) {
            failed = 1;
            return;
          }
          lo += (size_t)r;
        }
      };
      std::vector<std::thread> readers;
      for (int t = 1; t < n_readers; ++t) readers.emplace_back(read_range, std::min(n, t * share), std::min(n, (t + 1) * share));
      read_range(0, std::min(n, share));
      for (auto& th : readers) th.join();
      if (failed) {
        close(fd);
        set_last_error("short read from %s", path.c_str());
        return LCU_ERR_IO;
      }
      cudaError_t e = cudaMemcpyAsync((char*)dst + off, pin[cur], n, cudaMemcpyHostToDevice, stream);
      if (e == cudaSuccess) e = cudaEventRecord(done[cur], stream);
      if (e != cudaSuccess) {
        close(fd);
        set_last_error("copy of %s to the device failed: %s", path.c_str(), cudaGetErrorString(e));
        return LCU_ERR_CUDA;
      }
      in_flight[cur] = true;
      cur ^= 1;
      off += n;
    }
    close(fd);
    return LCU_OK;
  }
  int finish() {
    device_guard g(device);
    LCU_CUDA(cudaStreamSynchronize(stream));
    in_flight[0] = in_flight[1] = false;
    return LCU_OK;
  }
};

int g_loader_staged = 1;
}  // namespace

void set_loader_staged(int on) { g_loader_staged = on; }

int model::load_dir(const std::string& dir) {
  shadow_touch();
  std::vector<std::unique_ptr<staged_loader>> loaders;  // one per GPU that holds tensors
  auto loader_for = [&](int dev, staged_loader*& out) {
    for (auto& l : loaders)
      if (l->device == dev) {
        out = l.get();
        return (int)LCU_OK;
      }
    loaders.push_back(std::make_unique<staged_loader>());
    out = loaders.back().get();
    return out->init(dev);
  };
  for (auto& s : enumerate(*this)) {
    device_guard g(s.device);
    staged_loader* ld = nullptr;
    if (g_loader_staged) {
      int rc = loader_for(s.device, ld);
      if (rc) return rc;
    }
    auto load = [&](const std::string& path, void* dst, size_t bytes, size_t file_off, size_t file_bytes) {
      return ld ? ld->copy_file(path, dst, bytes, file_off, file_bytes) : load_file_mapped(path, dst, bytes, file_off, file_bytes);
    };
    const std::string base = dir + "/" + s.name;
    int rc;
    if (s.mat) {
      // files carry the whole matrix (and are named after its shape); a tensor-parallel shard reads its run of rows
      const size_t wrow = s.mat->bs ? s.mat->cols : s.mat->cols * 2, srow = s.mat->bs ? (s.mat->cols / s.mat->bs) * 2 : 0;
      const std::string dims = std::to_string(s.full_rows) + "_" + std::to_string(s.mat->cols);
      rc = load(base + ".weight__" + dims, s.mat->w, s.mat->weight_bytes(), s.row0 * wrow, s.full_rows * wrow);
      if (rc == LCU_OK && s.mat->bs)
        rc = load(base + ".scale__" + std::to_string(s.full_rows) + "_" + std::to_string(s.mat->cols / s.mat->bs), s.mat->sc,
                  s.mat->scale_bytes(), s.row0 * srow, s.full_rows * srow);
    } else {
      rc = load(base + ".weight__" + std::to_string(s.len), *s.vec, s.len * 2, 0, s.len * 2);
    }
    if (rc != LCU_OK) return rc;
  }
  for (auto& l : loaders) {
    int rc = l->finish();
    if (rc) return rc;
  }
  return LCU_OK;
}

int model::fill_synthetic(uint64_t seed, float scale) {
  shadow_touch();
  for (auto& s : enumerate(*this)) {
    device_guard g(s.device);
    if (!s.mat) {
      int rc = launch_fill_half(*s.vec, s.len, 1.0f, 0);
      if (rc) return rc;
      continue;
    }
    const size_t n = s.mat->rows * s.mat->cols;
    const uint64_t sid = fnv1a64(s.name.c_str());
    const uint64_t first = (uint64_t)s.row0 * s.mat->cols;  // a shard holds a run of whole rows: the same values the whole matrix has there
    if (s.mat->bs == 0) {
      int rc = launch_synth_fill((__half*)s.mat->w, n, seed, sid, scale, first, 0);
      if (rc) return rc;
    } else {
      __half* tmp = nullptr;
      LCU_CUDA(cudaMalloc(&tmp, n * 2));
      int rc = launch_synth_fill(tmp, n, seed, sid, scale, first, 0);
      if (!rc) rc = launch_quantize_absmax_uint8((uint8_t*)s.mat->w, s.mat->sc, tmp, s.mat->rows, s.mat->cols, s.mat->bs, 0);
      cudaError_t e = cudaDeviceSynchronize();
      cudaFree(tmp);
      if (rc) return rc;
      LCU_CUDA(e);
    }
  }
  for (auto& a : arenas) {
    device_guard g(a.first);
    LCU_CUDA(cudaDeviceSynchronize());
  }
  return LCU_OK;
}

// ------------------------------------------------------------------ context
namespace {
// Offsets of everything a context keeps in its per-GPU scratch arena.  One function sizes the arena for
// context::create, for the memory-based partitioner and for llama_params::shared_context_memory_size.
struct scratch_layout {
  size_t o_x, o_norm, o_q, o_kn, o_vn, o_att, o_h1, o_h3, o_hs, o_deq, o_deq2, o_scores, o_rope, o_state, o_ids, o_log, o_logits, o_probs;
  size_t deq_halves, score_halves, total;
};
scratch_layout scratch_layout_of(const model_params& p, uint32_t ffn, int context_len) {
  const size_t ctxl = context_len, d = p.dim, f = ffn, hd = p.dim / p.n_heads;
  scratch_layout s{};
  carve cv;
  s.o_x = cv.take(ctxl * d * 2); s.o_norm = cv.take(ctxl * d * 2); s.o_q = cv.take(ctxl * d * 2);
  s.o_kn = cv.take(ctxl * d * 2); s.o_vn = cv.take(ctxl * d * 2); s.o_att = cv.take(ctxl * d * 2);
  s.o_h1 = cv.take(ctxl * f * 2); s.o_h3 = cv.take(ctxl * f * 2); s.o_hs = cv.take(ctxl * f * 2);
  // u8 models: two buffers, each with room for the stacked w1|w3 or wq|wk|wv expanded to fp16 (one feeds the prompt GEMM
  // in flight while the next matrix is expanded into the other)
  s.deq_halves = p.q_type ? std::max((size_t)2 * f * d, (size_t)3 * d * d) : 0;
  s.o_deq = cv.take(s.deq_halves * 2);
  s.o_deq2 = cv.take(s.deq_halves * 2);
  // score buffer of the three-kernel tcgen05 prompt attention: only when that path is selected ("prefill_attn_tc" = 1);
  // the one-kernel path (2, the default) keeps scores in tensor memory
  s.score_halves = (prefill_tuning_ref().attn_tc == 1 && context_len <= 4096) ? attention_tc_scratch_halves(p.n_heads, context_len, context_len) : 0;
  s.o_scores = cv.take(s.score_halves * 2);
  s.o_rope = cv.take(ctxl * (hd / 2) * sizeof(float2));
  s.o_state = cv.take(64);
  s.o_ids = cv.take(ctxl * 2); s.o_log = cv.take(ctxl * 2);
  s.o_logits = cv.take((size_t)p.n_vocab * 2); s.o_probs = cv.take((size_t)p.n_vocab * 2);
  s.total = cv.off;
  return s;
}
}  // namespace

size_t context_scratch_bytes(const model_params& p, int context_len) { return scratch_layout_of(p, ffn_dim_of(p), context_len).total; }
size_t context_kv_bytes_per_layer(const model_params& p, int context_len) { return 2 * round_up((size_t)context_len * p.dim * 2, ALIGN); }

struct gpu_state {
  int device = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev = nullptr;
  void* arena = nullptr;
  size_t arena_bytes = 0;
  __half *x = nullptr, *norm = nullptr, *q = nullptr, *kn = nullptr, *vn = nullptr, *att = nullptr;
  __half *h1 = nullptr, *h3 = nullptr, *hs = nullptr;
  __half* scores = nullptr;  // prompt attention on tcgen05: [heads][context_len][round_up(context_len, 128)] scores / probabilities
  __half* deq = nullptr;  // u8 models: the dequantized matrix (or stack of matrices) of the prompt GEMM in flight
  size_t deq_halves = 0;
  // prompt path of u8 models: matrices are expanded to fp16 one job ahead on a side stream, into two alternating buffers
  __half* deq_buf[2] = {nullptr, nullptr};
  cudaStream_t side = nullptr;
  cudaEvent_t deq_done[2] = {nullptr, nullptr}, gemm_done[2] = {nullptr, nullptr};
  long deq_issued = 0, deq_used = 0;  // jobs expanded / consumed so far (job j lives in buffer j % 2)
  float2* rope = nullptr;
  int* state = nullptr;  // [0] position, [1] step counter, [2] last token, [3] error word
};

struct context_impl {
  model* m = nullptr;
  context_options opt;
  int start_pos = 0;
  std::vector<gpu_state> gpus;           // in order of first use
  std::vector<int> layer_slot;           // layer -> index into gpus
  std::vector<__half*> k_cache, v_cache; // per layer, on the layer's GPU
  std::vector<void*> kv_arenas;          // one per GPU
  size_t kv_bytes = 0;
  short* ids = nullptr;                  // token ids on the embedding GPU [context_len]
  __half* logits = nullptr;              // on the output GPU
  __half* probs = nullptr;
  short* log = nullptr;                  // generated tokens of a chained run [context_len]
  int* h_stage = nullptr;                // pinned: [0] position, [1] zero, [2] token read-back
  short* h_ids = nullptr;                // pinned token staging [context_len]
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  // two captured decode steps: [0] for positions whose attention slices stay within the register-path kernel's
  // 64 rows per CTA, [1] for longer contexts (streaming attention kernel); the host knows the position of every step
  cudaGraphExec_t graph[2] = {nullptr, nullptr};
  bool graph_failed = false;
  bool warmed_variant[2] = {false, false};
  int last_row = 0;                      // row of x that holds the last token's residual stream

  gpu_state& first() { return gpus.front(); }
  gpu_state& last() { return gpus.back(); }

  gemv_params params_base(gpu_state& g, int K);
  gemv_params params_qkv(int l);
  gemv_params params_wo(int l);
  gemv_params params_w13(int l);
  gemv_params params_w2(int l);
  gemv_params params_out(int row);
  int enqueue_hop(int from, int to, int m_rows);
  int enqueue_decode_step(int long_ctx);
  int enqueue_prefill(int m_rows);
  int build_graph(int variant);
  int run_decode_step(int n_keys);
  int stage_inputs(const short* tokens, int n);
};

context::~context() {
  if (!impl) return;
  context_impl& c = *impl;
  for (int v = 0; v < 2; ++v)
    if (c.graph[v]) cudaGraphExecDestroy(c.graph[v]);
  for (size_t i = 0; i < c.gpus.size(); ++i) {
    device_guard g(c.gpus[i].device);
    cudaDeviceSynchronize();
    if (c.gpus[i].arena) cudaFree(c.gpus[i].arena);
    if (i < c.kv_arenas.size() && c.kv_arenas[i]) cudaFree(c.kv_arenas[i]);
    if (c.gpus[i].side) cudaStreamDestroy(c.gpus[i].side);
    for (int e = 0; e < 2; ++e) {
      if (c.gpus[i].deq_done[e]) cudaEventDestroy(c.gpus[i].deq_done[e]);
      if (c.gpus[i].gemm_done[e]) cudaEventDestroy(c.gpus[i].gemm_done[e]);
    }
    if (c.gpus[i].stream) cudaStreamDestroy(c.gpus[i].stream);
    if (c.gpus[i].ev) cudaEventDestroy(c.gpus[i].ev);
  }
  if (c.t0) cudaEventDestroy(c.t0);
  if (c.t1) cudaEventDestroy(c.t1);
  if (c.h_stage) cudaFreeHost(c.h_stage);
  if (c.h_ids) cudaFreeHost(c.h_ids);
}

int context::create(std::unique_ptr<context>& out, model* m, const context_options& opt) {
  LCU_REQUIRE(m != nullptr, "context: null model");
  LCU_REQUIRE(opt.context_len >= 1 && opt.context_len <= 32768, "context: context length %d outside 1..32768", opt.context_len);
  LCU_REQUIRE(opt.temperature > 0.f, "context: temperature must be positive");
  const model_params& p = m->params;
  const int hd = p.dim / p.n_heads;
  LCU_REQUIRE(hd == 64 || hd == 128, "context: head_dim %d not supported (64 or 128)", hd);
  auto ctx = std::make_unique<context>();
  ctx->impl = std::make_unique<context_impl>();
  context_impl& c = *ctx->impl;
  c.m = m;
  c.opt = opt;
  const size_t ctxl = opt.context_len, d = p.dim;
  const std::vector<int> used = m->part.used_gpus();
  c.gpus.resize(used.size());
  c.kv_arenas.assign(used.size(), nullptr);
  c.layer_slot.resize(p.n_layers);
  for (uint32_t l = 0; l < p.n_layers; ++l)
    c.layer_slot[l] = (int)(std::find(used.begin(), used.end(), m->part.layer_gpus[l]) - used.begin());
  c.k_cache.resize(p.n_layers);
  c.v_cache.resize(p.n_layers);

  for (size_t gi = 0; gi < used.size(); ++gi) {
    gpu_state& g = c.gpus[gi];
    g.device = used[gi];
    device_guard dg(g.device);
    for (int other : used)
      if (other != g.device) {
        cudaError_t e = cudaDeviceEnablePeerAccess(other, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
          set_last_error("context: GPU %d cannot access GPU %d: %s", g.device, other, cudaGetErrorString(e));
          return LCU_ERR_CUDA;
        }
        cudaGetLastError();
      }
    LCU_CUDA(cudaStreamCreateWithFlags(&g.stream, cudaStreamNonBlocking));
    LCU_CUDA(cudaEventCreateWithFlags(&g.ev, cudaEventDisableTiming));
    // scratch arena: activations for up to context_len rows, rope table, state words,
    // and (first / last GPU) token ids, logits, probabilities, token log
    const scratch_layout sl = scratch_layout_of(p, m->ffn, opt.context_len);
    const size_t o_x = sl.o_x, o_norm = sl.o_norm, o_q = sl.o_q, o_kn = sl.o_kn, o_vn = sl.o_vn, o_att = sl.o_att;
    const size_t o_h1 = sl.o_h1, o_h3 = sl.o_h3, o_hs = sl.o_hs, o_deq = sl.o_deq, o_scores = sl.o_scores, o_rope = sl.o_rope;
    const size_t o_state = sl.o_state, o_ids = sl.o_ids, o_log = sl.o_log, o_logits = sl.o_logits, o_probs = sl.o_probs;
    const size_t deq_halves = sl.deq_halves, score_halves = sl.score_halves;
    carve cv;
    cv.off = sl.total;
    LCU_CUDA(cudaMalloc(&g.arena, cv.off));
    g.arena_bytes = cv.off;
    // on the context's own stream: that stream does not synchronise with the default stream, and the table kernel
    // below writes into this arena
    LCU_CUDA(cudaMemsetAsync(g.arena, 0, cv.off, g.stream));
    char* b = (char*)g.arena;
    g.x = (__half*)(b + o_x);
    g.norm = (__half*)(b + o_norm);
    g.q = (__half*)(b + o_q);
    g.kn = (__half*)(b + o_kn);
    g.vn = (__half*)(b + o_vn);
    g.att = (__half*)(b + o_att);
    g.h1 = (__half*)(b + o_h1);
    g.h3 = (__half*)(b + o_h3);
    g.hs = (__half*)(b + o_hs);
    g.scores = score_halves ? (__half*)(b + o_scores) : nullptr;
    g.deq = deq_halves ? (__half*)(b + o_deq) : nullptr;
    g.deq_halves = deq_halves;
    if (deq_halves) {
      g.deq_buf[0] = g.deq;
      g.deq_buf[1] = (__half*)(b + sl.o_deq2);
      LCU_CUDA(cudaStreamCreateWithFlags(&g.side, cudaStreamNonBlocking));
      for (int i = 0; i < 2; ++i) {
        LCU_CUDA(cudaEventCreateWithFlags(&g.deq_done[i], cudaEventDisableTiming));
        LCU_CUDA(cudaEventCreateWithFlags(&g.gemm_done[i], cudaEventDisableTiming));
      }
    }
    g.rope = (float2*)(b + o_rope);
    g.state = (int*)(b + o_state);
    if (gi == 0) c.ids = (short*)(b + o_ids);
    if (gi + 1 == used.size()) {
      c.logits = (__half*)(b + o_logits);
      c.probs = (__half*)(b + o_probs);
      c.log = (short*)(b + o_log);
    }
    int rc = launch_rope_table(g.rope, opt.context_len, hd, 10000.0f, g.stream);
    if (rc) return rc;
    // KV cache of this GPU's layers
    size_t n_local = 0;
    for (uint32_t l = 0; l < p.n_layers; ++l) n_local += c.layer_slot[l] == (int)gi;
    const size_t per = round_up(ctxl * d * 2, ALIGN);
    LCU_CUDA(cudaMalloc(&c.kv_arenas[gi], std::max<size_t>(per * 2 * n_local, ALIGN)));
    LCU_CUDA(cudaMemsetAsync(c.kv_arenas[gi], 0, std::max<size_t>(per * 2 * n_local, ALIGN), g.stream));
    c.kv_bytes += per * 2 * n_local;
    size_t k = 0;
    for (uint32_t l = 0; l < p.n_layers; ++l)
      if (c.layer_slot[l] == (int)gi) {
        c.k_cache[l] = (__half*)((char*)c.kv_arenas[gi] + per * (2 * k));
        c.v_cache[l] = (__half*)((char*)c.kv_arenas[gi] + per * (2 * k + 1));
        ++k;
      }
    LCU_CUDA(cudaStreamSynchronize(g.stream));
  }
  {
    device_guard dg(c.first().device);
    LCU_CUDA(cudaMallocHost(&c.h_stage, 64));
    LCU_CUDA(cudaMallocHost(&c.h_ids, ctxl * 2));
    memset(c.h_stage, 0, 64);
    LCU_CUDA(cudaEventCreate(&c.t0));
    LCU_CUDA(cudaEventCreate(&c.t1));
  }
  // u8 models: the fp16 shadow for prompts is set up here, next to the context's own arenas, so that next_token never
  // allocates (a stale shadow is refreshed in place by the next long prompt)
  if (p.q_type && c.opt.context_len >= 2) m->shadow_ready(true);
  out = std::move(ctx);
  return LCU_OK;
}

void context::clear_tokens() { impl->start_pos = 0; }  // the reference re-allocates everything here (llama_cu.cu:1004-1049)

size_t context::memory_usage() const {
  size_t n = impl->kv_bytes;
  for (auto& g : impl->gpus) n += g.arena_bytes;
  return n;
}
int context::tokens_left() const { return impl->opt.context_len - impl->start_pos; }
int context::position() const { return impl->start_pos; }
int context::kernels_per_step() const { return 1 + 5 * (int)impl->m->params.n_layers + 2 + (impl->opt.sampling ? 1 : 0); }

int context::set_sampling(int mode, uint64_t seed) {
  LCU_REQUIRE(mode == 0 || mode == 1, "set_sampling: mode %d (0 = greedy, 1 = multinomial)", mode);
  context_impl& c = *impl;
  c.opt.sampling = mode;
  c.opt.sample_seed = seed;
  for (int v = 0; v < 2; ++v)  // the captured steps hold the old choice
    if (c.graph[v]) {
      device_guard dg(c.first().device);
      LCU_CUDA(cudaStreamSynchronize(c.first().stream));
      cudaGraphExecDestroy(c.graph[v]);
      c.graph[v] = nullptr;
    }
  return LCU_OK;
}

int context::rollover(int keep) {
  context_impl& c = *impl;
  LCU_REQUIRE(keep >= 1 && keep < c.start_pos, "rollover: keep %d of %d cached positions", keep, c.start_pos);
  const model_params& p = c.m->params;
  const int first = c.start_pos - keep;
  for (uint32_t l = 0; l < p.n_layers; ++l) {
    gpu_state& g = c.gpus[c.layer_slot[l]];
    device_guard dg(g.device);
    LCU_TRY(launch_rollover(c.k_cache[l], c.v_cache[l], p.n_heads, c.opt.context_len, p.dim / p.n_heads, first, keep, 10000.0f, g.stream));
  }
  for (auto& g : c.gpus) {
    device_guard dg(g.device);
    LCU_CUDA(cudaStreamSynchronize(g.stream));
  }
  c.start_pos = keep;
  return LCU_OK;
}

// Error words of all stages (every stage's kernels report into their own GPU's word).  A word that is set is
// cleared here, so that one expired wait is reported once and the context stays usable.
int context::device_error() {
  int worst = 0;
  for (auto& g : impl->gpus) {
    int e = 0;
    device_guard dg(g.device);
    if (cudaMemcpy(&e, g.state + 3, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (e) {
      worst = e;
      if (cudaMemset(g.state + 3, 0, 4) != cudaSuccess) return -1;
    }
  }
  return worst;
}

// After the step's stream has been synchronised: the last stage's word came back with the token (h_stage[3]); with
// more than one stage the other stages' words are read as well.
static int finish_step(context& ctx, const char* who) {
  context_impl& c = *ctx.impl;
  int code = c.h_stage[3];
  if (code != 0 || c.gpus.size() > 1) {
    const int all = ctx.device_error();
    if (all < 0) {
      set_last_error("%s: cannot read the device error words", who);
      return LCU_ERR_CUDA;
    }
    if (all) code = all;
  }
  if (code != 0) {
    set_last_error("%s: a kernel gave up on a bounded wait (device error 0x%x)", who, code);
    return LCU_ERR_DEVICE_WAIT;
  }
  return LCU_OK;
}

// residual stream hand-off between pipeline stages: m_rows x dim halves over NVLink
// (the reference copies the whole context-length buffer, llama_cu.cu:1110-1114)
int context_impl::enqueue_hop(int from, int to, int m_rows) {
  gpu_state& a = gpus[from];
  gpu_state& b = gpus[to];
  LCU_CUDA(cudaMemcpyPeerAsync(b.x, b.device, a.x, a.device, (size_t)m_rows * m->params.dim * 2, a.stream));
  LCU_CUDA(cudaEventRecord(a.ev, a.stream));
  LCU_CUDA(cudaStreamWaitEvent(b.stream, a.ev, 0));
  return LCU_OK;
}


// ---- kernel arguments of the decode step
gemv_params context_impl::params_base(gpu_state& g, int K) {
  gemv_params a{};
  a.K = K;
  a.bs = m->params.q_type ? m->params.quantization_block_size : 0;
  a.m = 1;
  a.ldx = K;
  a.eps = m->params.norm_eps;
  a.err = g.state + 3;
  a.pos = g.state;
  return a;
}
gemv_params context_impl::params_qkv(int l) {
  gpu_state& g = gpus[layer_slot[l]];
  const layer_weights& L = m->layers[l];
  const int d = m->params.dim;
  gemv_params a = params_base(g, d);
  a.w[0] = L.wq.w; a.w[1] = L.wk.w; a.w[2] = L.wv.w;
  a.sc[0] = L.wq.sc; a.sc[1] = L.wk.sc; a.sc[2] = L.wv.sc;
  a.n_mats = 3;
  a.rows_per_mat = d;
  a.x = g.x;
  a.norm_w = L.attn_norm;
  a.q_out = g.q;
  a.k_cache = k_cache[l];
  a.v_cache = v_cache[l];
  a.rope = g.rope;
  a.ctx_len = opt.context_len;
  a.head_dim = d / m->params.n_heads;
  return a;
}
gemv_params context_impl::params_wo(int l) {
  gpu_state& g = gpus[layer_slot[l]];
  const layer_weights& L = m->layers[l];
  const int d = m->params.dim;
  gemv_params a = params_base(g, d);
  a.w[0] = L.wo.w; a.sc[0] = L.wo.sc; a.n_mats = 1; a.rows_per_mat = d;
  a.x = g.att; a.out = g.x; a.ldo = d; a.beta = 1.0f;
  return a;
}
gemv_params context_impl::params_w13(int l) {
  gpu_state& g = gpus[layer_slot[l]];
  const layer_weights& L = m->layers[l];
  const int d = m->params.dim, f = m->ffn;
  gemv_params a = params_base(g, d);
  a.w[0] = L.w1.w; a.w[1] = L.w3.w; a.sc[0] = L.w1.sc; a.sc[1] = L.w3.sc;
  a.n_mats = 2; a.rows_per_mat = f;
  a.x = g.x; a.norm_w = L.ffn_norm; a.out = g.hs; a.ldo = f;
  return a;
}
gemv_params context_impl::params_w2(int l) {
  gpu_state& g = gpus[layer_slot[l]];
  const layer_weights& L = m->layers[l];
  const int d = m->params.dim, f = m->ffn;
  gemv_params a = params_base(g, f);
  a.w[0] = L.w2.w; a.sc[0] = L.w2.sc; a.n_mats = 1; a.rows_per_mat = d;
  a.x = g.hs; a.out = g.x; a.ldo = d; a.beta = 1.0f;
  // last layer of a pipeline stage: the residual row is also written straight into the next stage's buffer
  if (l + 1 < (int)m->params.n_layers && layer_slot[l + 1] != layer_slot[l]) a.out_peer = gpus[layer_slot[l + 1]].x;
  return a;
}
gemv_params context_impl::params_out(int row) {
  gpu_state& g = last();
  const int d = m->params.dim;
  gemv_params a = params_base(g, d);
  a.w[0] = m->output.w; a.sc[0] = m->output.sc; a.n_mats = 1; a.rows_per_mat = m->params.n_vocab;
  a.x = g.x + (size_t)row * d; a.norm_w = m->norm; a.out = logits; a.ldo = m->params.n_vocab;
  return a;
}

int context_impl::enqueue_decode_step(int long_ctx) {
  const model_params& p = m->params;
  const int d = p.dim, hd = d / p.n_heads, bs = p.q_type ? p.quantization_block_size : 0;
  const int pdl = opt.use_pdl;
  {
    gpu_state& g = first();
    device_guard dg(g.device);
    LCU_TRY(launch_embed(g.x, d, m->tok_embeddings.w, m->tok_embeddings.sc, bs, ids, 1, d, g.stream, 0));
  }
  for (uint32_t l = 0; l < p.n_layers; ++l) {
    const int gi = layer_slot[l];
    bool hopped = false;
    if (l > 0 && layer_slot[l - 1] != gi) {
      // the stage being left advances its own position word, then hands the residual row over
      gpu_state& prev = gpus[layer_slot[l - 1]];
      {
        device_guard dgp(prev.device);
        LCU_TRY(launch_bump_pos(prev.state, 1, prev.stream));
      }
      // the row itself arrived with the previous layer's w2 kernel (peer stores); only the ordering is left
      LCU_CUDA(cudaEventRecord(prev.ev, prev.stream));
      LCU_CUDA(cudaStreamWaitEvent(gpus[gi].stream, prev.ev, 0));
      hopped = true;
    }
    gpu_state& g = gpus[gi];
    device_guard dg(g.device);
    const layer_weights& L = m->layers[l];
    // fused RMSNorm + wq|wk|wv + RoPE + cache write (reference llama_cu.cu:1129-1156)
    LCU_TRY(launch_gemv(params_qkv(l), EPI_ROPE_KV, g.stream, pdl && !hopped));
    // attention over the cache (reference llama_cu.cu:1161-1171)
    attn_params at{};
    at.q = g.q; at.ldq = d;
    at.k_cache = k_cache[l]; at.v_cache = v_cache[l];
    at.out = g.att; at.ldo = d;
    at.pos = g.state;
    at.ctx_len = opt.context_len; at.n_heads = p.n_heads; at.head_dim = hd; at.err = g.state + 3;
    // max_T sizes the kernel's shared memory and picks its variant: up to 64 rows per CTA the register-path kernel
    LCU_TRY(launch_attention(at, 1, opt.attn_cluster, long_ctx ? opt.context_len : std::min(opt.context_len, 64 * opt.attn_cluster), g.stream, pdl));
    LCU_TRY(launch_gemv(params_wo(l), EPI_PLAIN, g.stream, pdl));   // wo + residual (llama_cu.cu:1174)
    LCU_TRY(launch_gemv(params_w13(l), EPI_SILU, g.stream, pdl));   // RMSNorm + w1|w3 + SiLU gate (llama_cu.cu:1176-1183)
    LCU_TRY(launch_gemv(params_w2(l), EPI_PLAIN, g.stream, pdl));   // w2 + residual (llama_cu.cu:1185)
  }
  {
    // final RMSNorm + output matrix, softmax(T) + first-maximum token (llama_cu.cu:1191-1209)
    gpu_state& g = last();
    device_guard dg(g.device);
    LCU_TRY(launch_gemv(params_out(0), EPI_PLAIN, g.stream, pdl));
    head_params h{};
    h.logits = logits; h.probs = probs; h.n_vocab = p.n_vocab; h.temperature = opt.temperature;
    h.token_out = g.state + 2; h.next_ids = gpus.size() == 1 ? ids : nullptr;
    h.pos = g.state; h.advance = 1; h.log = log; h.step = g.state + 1; h.log_capacity = opt.context_len;
    LCU_TRY(launch_logits_head(h, g.stream, pdl));
    if (opt.sampling)  // the reference's discrete_distribution over the probabilities (llama_cu.cu:1202-1203) instead of the argmax
      LCU_TRY(launch_sample(probs, p.n_vocab, opt.sample_seed, g.state, 0.f, g.state + 2, h.next_ids, log, g.state + 1, opt.context_len, g.stream));
    if (gpus.size() > 1) {
      // multi-GPU: the token returns to stage 0 (the other stages advanced their position word on the way)
      LCU_TRY(launch_token_to_ids(ids, g.state + 2, g.stream));  // peer store into stage 0's id buffer
      LCU_CUDA(cudaEventRecord(g.ev, g.stream));
      LCU_CUDA(cudaStreamWaitEvent(first().stream, g.ev, 0));
    }
  }
  return LCU_OK;
}

int context_impl::enqueue_prefill(int m_rows) {
  const model_params& p = m->params;
  const int d = p.dim, hd = d / p.n_heads, f = m->ffn, bs = p.q_type ? p.quantization_block_size : 0;
  // u8 weights, prompts long enough for the tcgen05 GEMM: every matrix (or stack of matrices) is expanded to fp16 - the
  // exact values the reference's tile kernel builds in shared memory, llama_cu.cu:287-289 - on a side stream, one GEMM
  // ahead, into two alternating buffers: the expansion streams from HBM while the GEMM before it keeps the tensor
  // cores busy, instead of the two taking turns.  Job j of a GPU lives in buffer j % 2.
  for (auto& g : gpus) g.deq_issued = g.deq_used = 0;
  // (or, where the GPU has room, from the fp16 shadow of the whole model: model::shadow_ready)
  const bool shadow = bs > 0 && matmul_type_ref() != 1 && prefill_tuning_ref().fuse && prefill_tuning_ref().u8_deq_min_rows > 0 &&
                      m_rows >= prefill_tuning_ref().u8_deq_min_rows && m->shadow_ready(false);
  auto expand = [&](gpu_state& g, const dev_matrix* const* mats, int n_mats) -> int {
    const int b = (int)(g.deq_issued % 2);
    if (g.deq_issued >= 2) LCU_CUDA(cudaStreamWaitEvent(g.side, g.gemm_done[b], 0));  // the GEMM that read this buffer last
    size_t off = 0;
    for (int i = 0; i < n_mats; ++i) {
      LCU_TRY(launch_dequantize_absmax_uint8(g.deq_buf[b] + off, mats[i]->sc, (const uint8_t*)mats[i]->w, mats[i]->rows, mats[i]->cols, bs, g.side));
      off += mats[i]->rows * mats[i]->cols;
    }
    LCU_CUDA(cudaEventRecord(g.deq_done[b], g.side));
    ++g.deq_issued;
    return LCU_OK;
  };
  // job k of layer l: 0 = wq|wk|wv, 1 = wo, 2 = w1|w3, 3 = w2
  auto expand_job = [&](gpu_state& g, uint32_t l, int k) -> int {
    const layer_weights& W = m->layers[l];
    const dev_matrix* qkv[3] = {&W.wq, &W.wk, &W.wv};
    const dev_matrix* w13[2] = {&W.w1, &W.w3};
    const dev_matrix* one[1] = {k == 1 ? &W.wo : &W.w2};
    return k == 0 ? expand(g, qkv, 3) : k == 2 ? expand(g, w13, 2) : expand(g, one, 1);
  };
  // the GEMM of the oldest expanded job: waits for its expansion, runs, releases the buffer
  // (gate: the buffer holds w1|w3 and out takes silu(lhs . w1^T) * (lhs . w3^T), rows = 2 f; the value is the tile width)
  auto gemm_expanded = [&](gpu_state& g, __half* out, const __half* lhs, size_t rows, size_t cols, float beta, int gate = 0) -> int {
    const int b = (int)(g.deq_used % 2);
    LCU_CUDA(cudaStreamWaitEvent(g.stream, g.deq_done[b], 0));
    dev_matrix w;
    w.w = g.deq_buf[b];
    w.rows = rows;
    w.cols = cols;
    if (gate) LCU_TRY(launch_gemm_tc_gated(out, lhs, (int)cols, g.deq_buf[b], m_rows, (int)(rows / 2), (int)cols, g.state + 3, g.stream, gate));
    else LCU_TRY(matmul_rows(out, lhs, w, m_rows, beta, g.state + 3, g.stream));
    LCU_CUDA(cudaEventRecord(g.gemm_done[b], g.stream));
    ++g.deq_used;
    return LCU_OK;
  };
  {
    gpu_state& g = first();
    device_guard dg(g.device);
    LCU_TRY(launch_embed(g.x, d, m->tok_embeddings.w, m->tok_embeddings.sc, bs, ids, m_rows, d, g.stream, 0));
  }
  for (uint32_t l = 0; l < p.n_layers; ++l) {
    const int gi = layer_slot[l];
    if (l > 0 && layer_slot[l - 1] != gi) LCU_TRY(enqueue_hop(layer_slot[l - 1], gi, m_rows));
    gpu_state& g = gpus[gi];
    device_guard dg(g.device);
    const layer_weights& L = shadow ? m->shadow_layers[l] : m->layers[l];
    int* err = g.state + 3;
    LCU_TRY(launch_rms_norm(g.norm, g.x, L.attn_norm, m_rows, d, p.norm_eps, g.stream));
    // fp16 weights lie back to back in the arena (wq, wk, wv; w1, w3), and so do the q / new-k / new-v and the h1 / h3
    // scratch buffers: the three (two) products run as one GEMM over the stacked matrix into rows of [q | k | v]
    // ([h1 | h3]) - more tiles per launch, fewer launches
    const prefill_tuning& pt = prefill_tuning_ref();
    const bool rows_stacked = g.kn == g.q + (size_t)opt.context_len * d && g.vn == g.kn + (size_t)opt.context_len * d &&
                              g.h3 == g.h1 + (size_t)opt.context_len * f;
    // u8 weights: the same, with the matrices expanded to fp16 one after the other into the scratch buffer
    const bool pedantic = matmul_type_ref() == 1;  // u8 weights then stay u8 all the way into the pedantic kernel
    const bool fuse_u8 = !shadow && !pedantic && pt.fuse && bs > 0 && rows_stacked && pt.u8_deq_min_rows > 0 && m_rows >= pt.u8_deq_min_rows &&
                         g.deq != nullptr;
    const bool fuse = pt.fuse && (bs == 0 || shadow) && pt.tc_min_rows > 0 && m_rows >= pt.tc_min_rows && rows_stacked;
    const bool qkv_stacked = fuse_u8 || (fuse && (char*)L.wk.w == (char*)L.wq.w + (size_t)d * d * 2 && (char*)L.wv.w == (char*)L.wk.w + (size_t)d * d * 2);
    const int ldq = qkv_stacked ? 3 * d : d;
    if (qkv_stacked) {
      dev_matrix wqkv = L.wq;
      wqkv.rows = 3 * (size_t)d;
      if (fuse_u8) {
        if (g.deq_issued == g.deq_used) LCU_TRY(expand_job(g, l, 0));  // first layer of this GPU in this prompt: nothing was expanded ahead
        LCU_TRY(gemm_expanded(g, g.q, g.norm, 3 * (size_t)d, d, 0.f));
        LCU_TRY(expand_job(g, l, 1));
      } else {
        LCU_TRY(matmul_rows(g.q, g.norm, wqkv, m_rows, 0.f, err, g.stream));
      }
      LCU_TRY(launch_rope_scatter(g.q, g.q + d, g.q + 2 * d, k_cache[l], v_cache[l], g.rope, g.state, 0, m_rows, d, p.n_heads, opt.context_len,
                                  g.stream, ldq));
    } else {
      LCU_TRY(matmul_rows(g.q, g.norm, L.wq, m_rows, 0.f, err, g.stream, g.deq, g.deq_halves));
      LCU_TRY(matmul_rows(g.kn, g.norm, L.wk, m_rows, 0.f, err, g.stream, g.deq, g.deq_halves));
      LCU_TRY(matmul_rows(g.vn, g.norm, L.wv, m_rows, 0.f, err, g.stream, g.deq, g.deq_halves));
      LCU_TRY(launch_rope_scatter(g.q, g.kn, g.vn, k_cache[l], v_cache[l], g.rope, g.state, 0, m_rows, d, p.n_heads, opt.context_len, g.stream));
    }
    attn_params at{};
    at.q = g.q; at.ldq = ldq;
    at.k_cache = k_cache[l]; at.v_cache = v_cache[l];
    at.out = g.att; at.ldo = d;
    at.pos = g.state;
    at.ctx_len = opt.context_len; at.n_heads = p.n_heads; at.head_dim = hd; at.err = g.state + 3;
    if (pt.attn_tc == 2 && m_rows >= pt.attn_fused_min_rows)
      LCU_TRY(launch_attention_fused(at, m_rows, start_pos + m_rows, g.stream));
    else if (pt.attn_tc == 1 && g.scores != nullptr && m_rows >= pt.attn_tc_min_rows)
      LCU_TRY(launch_attention_tc(at, m_rows, start_pos + m_rows, g.scores, opt.context_len, g.stream));
    else if (pt.attn_tiles)
      LCU_TRY(launch_attention_prefill(at, m_rows, start_pos + m_rows, g.stream));
    else
      LCU_TRY(launch_attention(at, m_rows, 1, start_pos + m_rows, g.stream, 0));
    if (fuse_u8) {
      LCU_TRY(gemm_expanded(g, g.x, g.att, d, d, 1.0f));
      LCU_TRY(expand_job(g, l, 2));
    } else {
      LCU_TRY(matmul_rows(g.x, g.att, L.wo, m_rows, 1.0f, err, g.stream, g.deq, g.deq_halves));
    }
    LCU_TRY(launch_rms_norm(g.norm, g.x, L.ffn_norm, m_rows, d, p.norm_eps, g.stream));
    if (fuse_u8 || (fuse && (char*)L.w3.w == (char*)L.w1.w + (size_t)f * d * 2)) {
      dev_matrix w13 = L.w1;
      w13.rows = 2 * (size_t)f;
      // the tensor-core GEMM is on and no kernel is forced: w1|w3 and the gate may run as one launch (tile width, 0 = apart)
      const bool gate_allowed = pt.tc_min_rows > 0 && m_rows >= pt.tc_min_rows && pt.tc_tile_n == 0 && pt.tc_pair < 0 && gemm_tc_sk_mode() != 0;
      int gate_tile = gate_allowed ? gemm_tc_gated_tile(m_rows, (int)f, (int)d) : 0;
      if (fuse_u8) {
        if (!gemm_tc_gated_supported(m_rows, (int)f, (int)d, (int)d, g.norm, g.deq_buf[0], g.hs) || ((uintptr_t)g.deq_buf[1] & 15)) gate_tile = 0;
        LCU_TRY(gemm_expanded(g, gate_tile ? g.hs : g.h1, g.norm, 2 * (size_t)f, d, 0.f, gate_tile));
        LCU_TRY(expand_job(g, l, 3));
      } else if (gate_tile && gemm_tc_gated_supported(m_rows, (int)f, (int)d, (int)d, g.norm, w13.w, g.hs)) {
        LCU_TRY(launch_gemm_tc_gated(g.hs, g.norm, (int)d, (const __half*)w13.w, m_rows, (int)f, (int)d, err, g.stream, gate_tile));
      } else {
        gate_tile = 0;
        LCU_TRY(matmul_rows(g.h1, g.norm, w13, m_rows, 0.f, err, g.stream));
      }
      if (!gate_tile) LCU_TRY(launch_silu_rows(g.hs, g.h1, m_rows, f, g.stream));
    } else {
      LCU_TRY(matmul_rows(g.h1, g.norm, L.w1, m_rows, 0.f, err, g.stream, g.deq, g.deq_halves));
      LCU_TRY(matmul_rows(g.h3, g.norm, L.w3, m_rows, 0.f, err, g.stream, g.deq, g.deq_halves));
      LCU_TRY(launch_silu(g.hs, g.h1, g.h3, (size_t)m_rows * f, g.stream));
    }
    if (fuse_u8) {
      LCU_TRY(gemm_expanded(g, g.x, g.hs, d, f, 1.0f));
      if (l + 1 < p.n_layers && layer_slot[l + 1] == gi) LCU_TRY(expand_job(g, l + 1, 0));  // the next layer's first job, while this GEMM runs
    } else {
      LCU_TRY(matmul_rows(g.x, g.hs, L.w2, m_rows, 1.0f, err, g.stream, g.deq, g.deq_halves));
    }
  }
  {
    gpu_state& g = last();
    device_guard dg(g.device);
    // only the last row's logits are used (llama_cu.cu:1194-1195)
    if (matmul_type_ref() == 1) {
      LCU_TRY(launch_rms_norm(g.norm, g.x + (size_t)(m_rows - 1) * d, m->norm, 1, d, p.norm_eps, g.stream));
      LCU_TRY(matmul_rows(logits, g.norm, m->output, 1, 0.f, g.state + 3, g.stream));
    } else {
      LCU_TRY(launch_gemv(params_out(m_rows - 1), EPI_PLAIN, g.stream, 0));
    }
    head_params h{};
    h.logits = logits; h.probs = probs; h.n_vocab = p.n_vocab; h.temperature = opt.temperature;
    h.token_out = g.state + 2; h.next_ids = nullptr;
    h.pos = g.state; h.advance = m_rows; h.log = nullptr; h.step = nullptr; h.log_capacity = 0;
    LCU_TRY(launch_logits_head(h, g.stream, 0));
    if (opt.sampling) LCU_TRY(launch_sample(probs, p.n_vocab, opt.sample_seed, g.state, 0.f, g.state + 2, nullptr, nullptr, nullptr, 0, g.stream));
    if (gpus.size() > 1) {
      LCU_CUDA(cudaEventRecord(g.ev, g.stream));
      LCU_CUDA(cudaStreamWaitEvent(first().stream, g.ev, 0));
    }
  }
  return LCU_OK;
}

int context_impl::build_graph(int variant) {
  gpu_state& g0 = first();
  device_guard dg(g0.device);
  cudaGraph_t graph = nullptr;
  if (cudaStreamBeginCapture(g0.stream, cudaStreamCaptureModeRelaxed) != cudaSuccess) {
    cudaGetLastError();
    return LCU_ERR_CUDA;
  }
  int rc = enqueue_decode_step(variant);
  cudaError_t e = cudaStreamEndCapture(g0.stream, &graph);
  if (rc != LCU_OK || e != cudaSuccess || graph == nullptr) {
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    return rc ? rc : LCU_ERR_CUDA;
  }
  e = cudaGraphInstantiate(&this->graph[variant], graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    cudaGetLastError();
    this->graph[variant] = nullptr;
    set_last_error("cudaGraphInstantiate: %s", cudaGetErrorString(e));
    return LCU_ERR_CUDA;
  }
  return LCU_OK;
}

int context_impl::run_decode_step(int n_keys) {
  const int variant = n_keys > 64 * opt.attn_cluster ? 1 : 0;
  if (!warmed_variant[variant]) {  // first use of a variant runs un-captured (function attributes, tensor maps, ...)
    warmed_variant[variant] = true;
    return enqueue_decode_step(variant);
  }
  if (opt.use_graph && !graph[variant] && !graph_failed) {
    if (build_graph(variant) != LCU_OK) {
      graph_failed = true;
      fprintf(stderr, "llama_cu_b200: CUDA graph capture of the decode step failed (%s); launching kernels directly\n",
              last_error());
    }
  }
  if (graph[variant]) {
    device_guard dg(first().device);
    LCU_CUDA(cudaGraphLaunch(graph[variant], first().stream));
    return LCU_OK;
  }
  return enqueue_decode_step(variant);
}

// position word (and a zeroed step counter) to every stage, token ids to stage 0
int context_impl::stage_inputs(const short* tokens, int n) {
  h_stage[0] = start_pos;
  h_stage[1] = 0;
  for (size_t gi = 0; gi < gpus.size(); ++gi) {
    gpu_state& g = gpus[gi];
    device_guard dg(g.device);
    if (gi > 0) {  // order the other stages' copies after stage 0's stream position
      LCU_CUDA(cudaEventRecord(first().ev, first().stream));
      LCU_CUDA(cudaStreamWaitEvent(g.stream, first().ev, 0));
    }
    LCU_CUDA(cudaMemcpyAsync(g.state, h_stage, 8, cudaMemcpyHostToDevice, g.stream));
  }
  memcpy(h_ids, tokens, (size_t)n * 2);
  device_guard dg(first().device);
  LCU_CUDA(cudaMemcpyAsync(ids, h_ids, (size_t)n * 2, cudaMemcpyHostToDevice, first().stream));
  if (gpus.size() > 1) {
    // stage 0 must not start before every stage has its position word
    for (size_t gi = 1; gi < gpus.size(); ++gi) {
      device_guard dg2(gpus[gi].device);
      LCU_CUDA(cudaEventRecord(gpus[gi].ev, gpus[gi].stream));
      LCU_CUDA(cudaStreamWaitEvent(first().stream, gpus[gi].ev, 0));
    }
  }
  return LCU_OK;
}

int context::next_token(const short* tokens, int n, int* token_out) {
  context_impl& c = *impl;
  LCU_REQUIRE(n >= 1, "next_token: no tokens given");
  LCU_REQUIRE(n + c.start_pos <= c.opt.context_len, "next_token: %d new tokens at position %d exceed the context length %d", n,
              c.start_pos, c.opt.context_len);
  for (int i = 0; i < n; ++i)
    LCU_REQUIRE(tokens[i] >= 0 && (uint32_t)tokens[i] < c.m->params.n_vocab, "next_token: token id %d outside the vocabulary", tokens[i]);
  LCU_TRY(c.stage_inputs(tokens, n));
  if (n == 1 && matmul_type_ref() != 1)  // (the pedantic matmul type has no fused decode kernels: it takes the operator sequence below)
    LCU_TRY(c.run_decode_step(c.start_pos + 1));
  else
    LCU_TRY(c.enqueue_prefill(n));
  c.last_row = n == 1 ? 0 : n - 1;
  device_guard dg(c.first().device);
  LCU_CUDA(cudaMemcpyAsync(c.h_stage + 2, c.last().state + 2, 8, cudaMemcpyDeviceToHost, c.first().stream));
  LCU_CUDA(cudaStreamSynchronize(c.first().stream));
  LCU_TRY(finish_step(*this, "next_token"));
  c.start_pos += n;
  *token_out = c.h_stage[2];
  return LCU_OK;
}

int context::decode_chained(short first_token, int n_steps, short* tokens_out, float* ms_out) {
  context_impl& c = *impl;
  LCU_REQUIRE(n_steps >= 1 && n_steps + c.start_pos <= c.opt.context_len, "decode_chained: %d steps at position %d exceed the context length %d",
              n_steps, c.start_pos, c.opt.context_len);
  LCU_REQUIRE(first_token >= 0 && (uint32_t)first_token < c.m->params.n_vocab, "decode_chained: token id %d outside the vocabulary", first_token);
  LCU_REQUIRE(matmul_type_ref() != 1, "decode_chained: matmul_type 1 runs host-driven steps only (lcu_context_next_token)");
  LCU_TRY(c.stage_inputs(&first_token, 1));
  device_guard dg(c.first().device);
  LCU_CUDA(cudaEventRecord(c.t0, c.first().stream));
  for (int i = 0; i < n_steps; ++i) LCU_TRY(c.run_decode_step(c.start_pos + i + 1));
  LCU_CUDA(cudaEventRecord(c.t1, c.first().stream));
  LCU_CUDA(cudaMemcpyAsync(c.h_ids, c.log, (size_t)n_steps * 2, cudaMemcpyDeviceToHost, c.first().stream));
  LCU_CUDA(cudaMemcpyAsync(c.h_stage + 2, c.last().state + 2, 8, cudaMemcpyDeviceToHost, c.first().stream));
  LCU_CUDA(cudaStreamSynchronize(c.first().stream));
  LCU_TRY(finish_step(*this, "decode_chained"));
  c.start_pos += n_steps;
  c.last_row = 0;
  memcpy(tokens_out, c.h_ids, (size_t)n_steps * 2);
  if (ms_out) LCU_CUDA(cudaEventElapsedTime(ms_out, c.t0, c.t1));
  return LCU_OK;
}

int context::read_probs(__half* out_host) {
  context_impl& c = *impl;
  device_guard dg(c.last().device);
  LCU_CUDA(cudaMemcpy(out_host, c.probs, (size_t)c.m->params.n_vocab * 2, cudaMemcpyDeviceToHost));
  return LCU_OK;
}

int context::read_hidden(__half* out_host) {
  context_impl& c = *impl;
  device_guard dg(c.last().device);
  // decode leaves the token's row at x[0]; a prefill of n rows leaves it at x[n-1] - the caller
  // reads right after next_token, so the row index is kept
  LCU_CUDA(cudaMemcpy(out_host, c.last().x + (size_t)c.last_row * c.m->params.dim, (size_t)c.m->params.dim * 2, cudaMemcpyDeviceToHost));
  return LCU_OK;
}

int context::bench_kernel(int which, int reps, float* ms_per_launch, uint64_t* bytes_per_launch) {
  context_impl& c = *impl;
  LCU_REQUIRE(which >= 0 && which <= 4 && reps >= 1, "bench_kernel: bad arguments");
  // layers of one pipeline stage in rotation: the first stage, or the last one for the output matrix
  const int stage = which == 4 ? (int)c.gpus.size() - 1 : 0;
  std::vector<int> stage_layers;
  for (int l = 0; l < (int)c.m->params.n_layers; ++l)
    if (c.layer_slot[l] == stage && !(which == 3 && l + 1 < (int)c.m->params.n_layers && c.layer_slot[l + 1] != stage))
      stage_layers.push_back(l);  // (a w2 that also stores into the next stage is left out of the rotation)
  LCU_REQUIRE(!stage_layers.empty(), "bench_kernel: no layer to rotate over");
  auto params_of = [&](int i, int& epi) {
    const int l = stage_layers[i % stage_layers.size()];
    switch (which) {
      case 0: epi = EPI_ROPE_KV; return c.params_qkv(l);
      case 1: epi = EPI_PLAIN; return c.params_wo(l);
      case 2: epi = EPI_SILU; return c.params_w13(l);
      case 3: epi = EPI_PLAIN; return c.params_w2(l);
      default: epi = EPI_PLAIN; return c.params_out(0);
    }
  };
  gpu_state& g = c.gpus[stage];
  device_guard dg(g.device);
  c.h_stage[0] = 0;
  c.h_stage[1] = 0;
  LCU_CUDA(cudaMemcpyAsync(g.state, c.h_stage, 8, cudaMemcpyHostToDevice, g.stream));
  int epi = 0;
  for (int i = 0; i < std::min(reps, 8); ++i) {  // warm-up
    gemv_params a = params_of(i, epi);
    LCU_TRY(launch_gemv(a, epi, g.stream, 0));
  }
  cudaEvent_t e0 = nullptr, e1 = nullptr;  // on this stage's device
  LCU_CUDA(cudaEventCreate(&e0));
  LCU_CUDA(cudaEventCreate(&e1));
  LCU_CUDA(cudaEventRecord(e0, g.stream));
  for (int i = 0; i < reps; ++i) {
    gemv_params a = params_of(i, epi);
    LCU_TRY(launch_gemv(a, epi, g.stream, c.opt.use_pdl));
  }
  LCU_CUDA(cudaEventRecord(e1, g.stream));
  LCU_CUDA(cudaStreamSynchronize(g.stream));
  float ms = 0.f;
  LCU_CUDA(cudaEventElapsedTime(&ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *ms_per_launch = ms / reps;
  gemv_params a0 = params_of(0, epi);
  *bytes_per_launch = gemv_algorithmic_bytes(a0, epi);
  // the launches above wrote position 0 of the K/V caches and the q / residual scratch rows: whatever the context held
  // is gone, so it is left cleared
  c.start_pos = 0;
  return LCU_OK;
}

}  // namespace lcu
