// Tensor-parallel batch-1 decode over the GPUs of one box (one process, one stream per GPU).
//
// The reference's only multi-GPU scheme is the layer pipeline (llama_partition, llama_cu.cu:810-880, 1099-1114): at batch 1
// one stage works at a time, so more GPUs add capacity and no speed (its README.md:25).  This file is the scheme that does
// speed a single token up: every GPU holds a run of ROWS of every matrix (whole heads of wq / wk / wv, a slice of w1 / w3
// rows, of wo / w2 / output rows), streams only those rows from its own HBM, and owns the matching slice of each
// activation row.  Rows keep their full length, so the weight-streaming GEMV runs exactly as on one GPU and every output
// element is computed by the same instructions in the same order: tokens and probabilities are bit-identical to the
// single-GPU run.
//
// Exchange, inside the producing kernel: the GEMV epilogue (and the attention kernel) stores each result into its own
// row AND into the same place of every other GPU's row (plain peer stores over NVLink; no TMA multicast, no library
// kernel on peer memory).  The last warp of the launch - found by counting behind fences that widen from CTA to device
// scope - fences once at system scope and writes step * 1024 + exchange_id into a flag word in every GPU's memory; the
// kernel that needs the whole row polls its own GPU's flag words (bounded: ~1 s, then the error word is set and the
// step ends).
// Per layer: the attention output, x after wo, the gated hidden row after w1|w3, x after w2.
// The logits slices go to GPU 0, which runs the softmax / argmax head and sends the token back to every GPU.
// A step is captured once as a CUDA graph spanning all GPUs (fork / join by events on stream 0); inside it the GPUs are
// ordered by the flags alone.
#include "tp.cuh"

#include <algorithm>
#include <cstring>

#include "attention.cuh"
#include "gemv.cuh"
#include "ops.cuh"

namespace lcu {
namespace {

constexpr int TP_MAX = 8;
// measurement switch (lcu_set_tuning "tp_debug"; results are wrong when set): 1 = kernels do not wait for the other GPUs'
// slices, 2 = kernels neither send their slices nor publish, 4 = no peer stores of results but flags are still published
int g_tp_debug = 0;
constexpr size_t ALIGN = 256;
struct carve {
  size_t off = 0;
  size_t take(size_t bytes) {
    size_t o = off;
    off += round_up(bytes, ALIGN);
    return o;
  }
};

#define LCU_TRY(expr)    \
  do {                   \
    int _rc = (expr);    \
    if (_rc) return _rc; \
  } while (0)

// state words of a GPU: [0] position, [1] step counter of a chained run, [2] last token, [3] error word,
// [4] number of the decode step in flight (monotonic), [5] "last CTA" counter of the GEMV launches, [6] of the attention launches,
// [8 .. 15] flag words: [8 + src] = step * 1024 + id of the last exchange GPU `src` has completed
constexpr int ST_POS = 0, ST_STEP = 1, ST_TOKEN = 2, ST_ERR = 3, ST_SEQ = 4, ST_DONE = 5, ST_FLAGS = 8, ST_WORDS = 16;

__global__ void tp_begin_kernel(int* state) { state[ST_SEQ] += 1; }

// holds the stream until the n flag words have reached step * 1024 + wait_id (the kernel behind it reads what arrived)
__global__ void tp_wait_kernel(const int* flags, int n, const int* seq, int wait_id, int* err) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)threadIdx.x < n) flag_wait_at_least(flags + threadIdx.x, *seq * TP_EXCHANGES_PER_STEP + wait_id, err);
}

// the chosen token goes to every other GPU's id buffer (ordering to their next step: the join / fork events of the steps)
struct id_list {
  short* ids[TP_MAX];
  int n;
};
__global__ void tp_token_kernel(id_list peers, const int* token) {
  const short t = (short)*token;
  for (int q = 0; q < peers.n; ++q) peers.ids[q][0] = t;
}

template <typename... Args>
int launch_small(void (*kernel)(Args...), int threads, cudaStream_t stream, int pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(threads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  LCU_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
  return LCU_OK;
}

struct tp_gpu {
  int device = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev = nullptr;
  std::unique_ptr<model> shard;
  void* arena = nullptr;
  void* kv = nullptr;
  size_t arena_bytes = 0, kv_bytes = 0;
  __half *x = nullptr, *att = nullptr, *hs = nullptr, *q = nullptr, *logits = nullptr, *probs = nullptr;
  float2* rope = nullptr;
  short *ids = nullptr, *log = nullptr;
  int* state = nullptr;
  std::vector<__half*> k_cache, v_cache;
};

}  // namespace

void tp_set_debug(int v) { g_tp_debug = v; }

struct tp_impl {
  model_params p{};
  uint32_t ffn = 0;
  int n = 0;
  context_options opt;
  int start_pos = 0;
  std::vector<tp_gpu> g;
  int* h_stage = nullptr;   // pinned: [0] token read-back, [1] error word; [2 ..] staging of positions
  short* h_ids = nullptr;   // pinned token staging [context_len]
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  cudaGraphExec_t graph[2] = {nullptr, nullptr};
  bool warmed[2] = {false, false}, graph_failed = false;

  gemv_params base(int gi, int K) const;
  void exchange(gemv_params& a, int gi, size_t slice_off, __half* tp_gpu::*row, int exchange_id) const;
  int enqueue_step(int long_ctx);
  int build_graph(int variant);
  int run_step(int n_keys);
  int stage(const short* tokens, int n_first);
  int finish(const char* who);
};

tp_decoder::~tp_decoder() {
  if (!impl) return;
  tp_impl& c = *impl;
  for (int v = 0; v < 2; ++v)
    if (c.graph[v]) cudaGraphExecDestroy(c.graph[v]);
  for (auto& g : c.g) {
    device_guard dg(g.device);
    cudaDeviceSynchronize();
    if (g.arena) cudaFree(g.arena);
    if (g.kv) cudaFree(g.kv);
    if (g.stream) cudaStreamDestroy(g.stream);
    if (g.ev) cudaEventDestroy(g.ev);
    g.shard.reset();
  }
  if (c.t0) cudaEventDestroy(c.t0);
  if (c.t1) cudaEventDestroy(c.t1);
  if (c.h_stage) cudaFreeHost(c.h_stage);
  if (c.h_ids) cudaFreeHost(c.h_ids);
}

int tp_check_split(const model_params& p, int n_gpus) {
  LCU_REQUIRE(n_gpus >= 2 && n_gpus <= TP_MAX, "tensor parallel: %d GPUs (2 .. %d)", n_gpus, TP_MAX);
  LCU_REQUIRE(p.dim > 0 && p.n_heads > 0 && p.multiple_of > 0 && p.n_vocab > 0, "tensor parallel: empty dimension in params");
  const uint32_t ffn = ffn_dim_of(p);
  LCU_REQUIRE(p.n_heads % n_gpus == 0, "tensor parallel: %u heads do not split over %d GPUs", p.n_heads, n_gpus);
  LCU_REQUIRE(ffn % n_gpus == 0 && (ffn / n_gpus) % 8 == 0, "tensor parallel: ffn dim %u does not split into rows of 8 over %d GPUs", ffn, n_gpus);
  LCU_REQUIRE(p.n_vocab % n_gpus == 0 && (p.n_vocab / n_gpus) % 2 == 0, "tensor parallel: vocabulary %u does not split evenly over %d GPUs", p.n_vocab, n_gpus);
  LCU_REQUIRE((p.dim / n_gpus) % 8 == 0, "tensor parallel: dim %u does not split into slices of 8 over %d GPUs", p.dim, n_gpus);
  return LCU_OK;
}

int tp_decoder::create(std::unique_ptr<tp_decoder>& out, const model_params& p, const int* gpus, int n_gpus, const context_options& opt) {
  LCU_TRY(tp_check_split(p, n_gpus));
  LCU_REQUIRE(opt.context_len >= 1 && opt.context_len <= 32768 && opt.temperature > 0.f, "tensor parallel: bad context length or temperature");
  const int hd = p.dim / p.n_heads;
  LCU_REQUIRE(hd == 64 || hd == 128, "tensor parallel: head_dim %d not supported (64 or 128)", hd);
  int ndev = 0;
  LCU_CUDA(cudaGetDeviceCount(&ndev));
  for (int i = 0; i < n_gpus; ++i) {
    LCU_REQUIRE(gpus[i] >= 0 && gpus[i] < ndev, "tensor parallel: GPU %d named but %d are visible", gpus[i], ndev);
    for (int j = 0; j < i; ++j) LCU_REQUIRE(gpus[i] != gpus[j], "tensor parallel: GPU %d named twice", gpus[i]);
  }
  auto dec = std::make_unique<tp_decoder>();
  dec->impl = std::make_unique<tp_impl>();
  tp_impl& c = *dec->impl;
  c.p = p;
  c.ffn = ffn_dim_of(p);
  c.n = n_gpus;
  c.opt = opt;
  c.g.resize(n_gpus);
  const size_t ctxl = opt.context_len, d = p.dim, f = c.ffn, V = p.n_vocab, L = p.n_layers;
  for (int gi = 0; gi < n_gpus; ++gi) {
    tp_gpu& g = c.g[gi];
    g.device = gpus[gi];
    device_guard dg(g.device);
    for (int j = 0; j < n_gpus; ++j)
      if (j != gi) {
        cudaError_t e = cudaDeviceEnablePeerAccess(gpus[j], 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
          set_last_error("tensor parallel: GPU %d cannot access GPU %d: %s", g.device, gpus[j], cudaGetErrorString(e));
          return LCU_ERR_CUDA;
        }
        cudaGetLastError();
      }
    partition part;
    part.layer_gpus.assign(p.n_layers, g.device);
    LCU_TRY(model::create(g.shard, p, part, gi, n_gpus));
    LCU_CUDA(cudaStreamCreateWithFlags(&g.stream, cudaStreamNonBlocking));
    LCU_CUDA(cudaEventCreateWithFlags(&g.ev, cudaEventDisableTiming));
    carve cv;
    const size_t o_x = cv.take(d * 2), o_att = cv.take(d * 2), o_hs = cv.take(f * 2), o_q = cv.take(d / n_gpus * 2);
    const size_t o_logits = cv.take(V * 2), o_probs = cv.take(V * 2), o_rope = cv.take(ctxl * (hd / 2) * sizeof(float2));
    const size_t o_ids = cv.take(ctxl * 2), o_log = cv.take(ctxl * 2), o_state = cv.take(ST_WORDS * 4);
    LCU_CUDA(cudaMalloc(&g.arena, cv.off));
    g.arena_bytes = cv.off;
    LCU_CUDA(cudaMemsetAsync(g.arena, 0, cv.off, g.stream));
    char* b = (char*)g.arena;
    g.x = (__half*)(b + o_x);
    g.att = (__half*)(b + o_att);
    g.hs = (__half*)(b + o_hs);
    g.q = (__half*)(b + o_q);
    g.logits = (__half*)(b + o_logits);
    g.probs = (__half*)(b + o_probs);
    g.rope = (float2*)(b + o_rope);
    g.ids = (short*)(b + o_ids);
    g.log = (short*)(b + o_log);
    g.state = (int*)(b + o_state);
    LCU_TRY(launch_rope_table(g.rope, opt.context_len, hd, 10000.0f, g.stream));
    // every kernel of a step is loaded on this GPU now: in the first step no launch may stall in kernel loading while
    // the other GPUs' kernels are already waiting for this GPU's slices
    LCU_TRY(gemv_single_row_preload());
    LCU_TRY(attention_preload());
    LCU_TRY(ops_preload());
    LCU_TRY(head_preload());
    {
      cudaFuncAttributes fa;
      LCU_CUDA(cudaFuncGetAttributes(&fa, tp_begin_kernel));
      LCU_CUDA(cudaFuncGetAttributes(&fa, tp_wait_kernel));
      LCU_CUDA(cudaFuncGetAttributes(&fa, tp_token_kernel));
    }
    // K and V caches of this GPU's heads: [layer][K | V][local head][position][head_dim]
    const size_t per = round_up(ctxl * (d / n_gpus) * 2, ALIGN);
    g.kv_bytes = per * 2 * L;
    LCU_CUDA(cudaMalloc(&g.kv, g.kv_bytes));
    LCU_CUDA(cudaMemsetAsync(g.kv, 0, g.kv_bytes, g.stream));
    g.k_cache.resize(L);
    g.v_cache.resize(L);
    for (size_t l = 0; l < L; ++l) {
      g.k_cache[l] = (__half*)((char*)g.kv + per * (2 * l));
      g.v_cache[l] = (__half*)((char*)g.kv + per * (2 * l + 1));
    }
    LCU_CUDA(cudaStreamSynchronize(g.stream));
  }
  {
    device_guard dg(c.g[0].device);
    LCU_CUDA(cudaMallocHost(&c.h_stage, (2 + ctxl) * sizeof(int)));
    LCU_CUDA(cudaMallocHost(&c.h_ids, ctxl * 2));
    memset(c.h_stage, 0, (2 + ctxl) * sizeof(int));
    LCU_CUDA(cudaEventCreate(&c.t0));
    LCU_CUDA(cudaEventCreate(&c.t1));
  }
  out = std::move(dec);
  return LCU_OK;
}

int tp_decoder::fill_synthetic(uint64_t seed, float scale) {
  for (auto& g : impl->g) LCU_TRY(g.shard->fill_synthetic(seed, scale));
  return LCU_OK;
}
int tp_decoder::load_dir(const std::string& dir) {
  for (auto& g : impl->g) LCU_TRY(g.shard->load_dir(dir));
  return LCU_OK;
}
size_t tp_decoder::weight_bytes_per_gpu() const { return impl->g[0].shard->weight_bytes_total; }
size_t tp_decoder::memory_usage() const {
  size_t n = 0;
  for (auto& g : impl->g) n += g.arena_bytes + g.kv_bytes;
  return n;
}
int tp_decoder::n_gpus() const { return impl->n; }
int tp_decoder::tokens_left() const { return impl->opt.context_len - impl->start_pos; }
void tp_decoder::clear_tokens() { impl->start_pos = 0; }
// per GPU: begin, embed, 5 per layer (QKV, attention, wo, w1|w3, w2), output rows, + on GPU 0 wait, head, token
int tp_decoder::kernels_per_step() const { return impl->n * (3 + 5 * (int)impl->p.n_layers) + 3 + (impl->n - 1); }

gemv_params tp_impl::base(int gi, int K) const {
  const tp_gpu& g = this->g[gi];
  gemv_params a{};
  a.K = K;
  a.bs = p.q_type ? p.quantization_block_size : 0;
  a.m = 1;
  a.ldx = K;
  a.eps = p.norm_eps;
  a.err = g.state + ST_ERR;
  a.pos = g.state + ST_POS;
  a.seq = g.state + ST_SEQ;
  a.wait_flags = g.state + ST_FLAGS;
  return a;
}

// results of this launch also go into `row` of every other GPU at element offset slice_off, and once the launch is
// complete every GPU (this one included) gets the flag exchange_id in its slot for this GPU
void tp_impl::exchange(gemv_params& a, int gi, size_t slice_off, __half* tp_gpu::*row, int exchange_id) const {
  a.n_peer_out = 0;
  a.n_peer_flag = 0;
  if (g_tp_debug & 2) return;
  for (int j = 0; j < n; ++j) {
    if (j != gi && !(g_tp_debug & 4)) a.peer_out[a.n_peer_out++] = g[j].*row + slice_off;
    a.peer_flag[a.n_peer_flag++] = g[j].state + ST_FLAGS + gi;
  }
  a.done_count = g[gi].state + ST_DONE;
  a.exchange_id = exchange_id;
}

int tp_impl::enqueue_step(int long_ctx) {
  const int d = p.dim, hd = d / p.n_heads, f = ffn, V = p.n_vocab, L = p.n_layers, bs = p.q_type ? p.quantization_block_size : 0;
  const int dl = d / n, fl = f / n, vl = V / n, pdl = opt.use_pdl;
  LCU_REQUIRE(4 * L + 2 < TP_EXCHANGES_PER_STEP, "tensor parallel: %d layers exceed the exchange numbering", L);
  // fork: the other GPUs' streams join stream 0's place in the step sequence
  {
    device_guard dg(g[0].device);
    LCU_CUDA(cudaEventRecord(g[0].ev, g[0].stream));
  }
  for (int gi = 1; gi < n; ++gi) {
    device_guard dg(g[gi].device);
    LCU_CUDA(cudaStreamWaitEvent(g[gi].stream, g[0].ev, 0));
  }
  // The launches of all GPUs are interleaved layer by layer: a GPU's kernels wait (on the device) for the other GPUs'
  // slices, so no GPU may get far ahead of what has been enqueued for the others.
  for (int gi = 0; gi < n; ++gi) {
    tp_gpu& me = g[gi];
    device_guard dg(me.device);
    const model& m = *me.shard;
    tp_begin_kernel<<<1, 1, 0, me.stream>>>(me.state);
    LCU_CUDA(cudaGetLastError());
    LCU_TRY(launch_embed(me.x, d, m.tok_embeddings.w, m.tok_embeddings.sc, bs, me.ids, 1, d, me.stream, 0));
  }
  for (int l = 0; l < L; ++l) {
    for (int gi = 0; gi < n; ++gi) {
      tp_gpu& me = g[gi];
      device_guard dg(me.device);
      const model& m = *me.shard;
      const layer_weights& W = m.layers[l];
      const int id0 = 4 * l;
      {  // RMSNorm + this GPU's heads of wq | wk | wv + RoPE + cache write (llama_cu.cu:1129-1156)
        gemv_params a = base(gi, d);
        a.w[0] = W.wq.w; a.w[1] = W.wk.w; a.w[2] = W.wv.w;
        a.sc[0] = W.wq.sc; a.sc[1] = W.wk.sc; a.sc[2] = W.wv.sc;
        a.n_mats = 3;
        a.rows_per_mat = dl;
        a.x = me.x;
        a.norm_w = W.attn_norm;
        a.q_out = me.q;
        a.k_cache = me.k_cache[l];
        a.v_cache = me.v_cache[l];
        a.rope = me.rope;
        a.ctx_len = opt.context_len;
        a.head_dim = hd;
        if (l > 0) {  // x of the previous layer's w2: slices of every GPU
          a.n_wait = (g_tp_debug & 1) ? 0 : n;
          a.wait_id = id0;
        }
        LCU_TRY(launch_gemv(a, EPI_ROPE_KV, me.stream, pdl));
      }
      {  // attention of this GPU's heads (llama_cu.cu:1161-1171), then the slice to every GPU
        attn_params at{};
        at.q = me.q; at.ldq = dl;
        at.k_cache = me.k_cache[l]; at.v_cache = me.v_cache[l];
        at.out = me.att + (size_t)gi * dl; at.ldo = dl;
        at.pos = me.state + ST_POS;
        at.ctx_len = opt.context_len; at.n_heads = p.n_heads / n; at.head_dim = hd; at.err = me.state + ST_ERR;
        for (int j = 0; j < n && !(g_tp_debug & 2); ++j) {
          if (j != gi && !(g_tp_debug & 4)) at.peer_out[at.n_peer_out++] = g[j].att + (size_t)gi * dl;
          at.peer_flag[at.n_peer_flag++] = g[j].state + ST_FLAGS + gi;
        }
        if (!(g_tp_debug & 2)) at.done_count = me.state + ST_DONE + 1;
        at.seq = me.state + ST_SEQ;
        at.exchange_id = id0 + 1;
        at.exchanges_per_step = TP_EXCHANGES_PER_STEP;
        LCU_TRY(launch_attention(at, 1, opt.attn_cluster, long_ctx ? opt.context_len : std::min(opt.context_len, 64 * opt.attn_cluster), me.stream, pdl));
      }
      {  // this GPU's rows of wo + residual (llama_cu.cu:1174)
        gemv_params a = base(gi, d);
        a.w[0] = W.wo.w; a.sc[0] = W.wo.sc; a.n_mats = 1; a.rows_per_mat = dl;
        a.x = me.att; a.out = me.x + (size_t)gi * dl; a.ldo = d; a.beta = 1.0f;
        a.n_wait = (g_tp_debug & 1) ? 0 : n; a.wait_id = id0 + 1;
        exchange(a, gi, (size_t)gi * dl, &tp_gpu::x, id0 + 2);
        LCU_TRY(launch_gemv(a, EPI_PLAIN, me.stream, pdl));
      }
      {  // RMSNorm + this GPU's rows of w1 | w3 + SiLU gate (llama_cu.cu:1176-1183)
        gemv_params a = base(gi, d);
        a.w[0] = W.w1.w; a.w[1] = W.w3.w; a.sc[0] = W.w1.sc; a.sc[1] = W.w3.sc;
        a.n_mats = 2; a.rows_per_mat = fl;
        a.x = me.x; a.norm_w = W.ffn_norm; a.out = me.hs + (size_t)gi * fl; a.ldo = f;
        a.n_wait = (g_tp_debug & 1) ? 0 : n; a.wait_id = id0 + 2;
        exchange(a, gi, (size_t)gi * fl, &tp_gpu::hs, id0 + 3);
        LCU_TRY(launch_gemv(a, EPI_SILU, me.stream, pdl));
      }
      {  // this GPU's rows of w2 + residual (llama_cu.cu:1185)
        gemv_params a = base(gi, f);
        a.w[0] = W.w2.w; a.sc[0] = W.w2.sc; a.n_mats = 1; a.rows_per_mat = dl;
        a.x = me.hs; a.out = me.x + (size_t)gi * dl; a.ldo = d; a.beta = 1.0f;
        a.n_wait = (g_tp_debug & 1) ? 0 : n; a.wait_id = id0 + 3;
        exchange(a, gi, (size_t)gi * dl, &tp_gpu::x, id0 + 4);
        LCU_TRY(launch_gemv(a, EPI_PLAIN, me.stream, pdl));
      }
    }
  }
  for (int gi = 0; gi < n; ++gi) {
    tp_gpu& me = g[gi];
    device_guard dg(me.device);
    const model& m = *me.shard;
    {  // final RMSNorm + this GPU's rows of the output matrix; the logits slice goes to GPU 0 (llama_cu.cu:1191-1195)
      gemv_params a = base(gi, d);
      a.w[0] = m.output.w; a.sc[0] = m.output.sc; a.n_mats = 1; a.rows_per_mat = vl;
      a.x = me.x; a.norm_w = m.norm; a.out = me.logits + (size_t)gi * vl; a.ldo = V;
      a.n_wait = (g_tp_debug & 1) ? 0 : n; a.wait_id = 4 * L;
      if (gi != 0) a.peer_out[a.n_peer_out++] = g[0].logits + (size_t)gi * vl;
      a.peer_flag[a.n_peer_flag++] = g[0].state + ST_FLAGS + gi;
      a.done_count = me.state + ST_DONE;
      a.exchange_id = 4 * L + 1;
      LCU_TRY(launch_gemv(a, EPI_PLAIN, me.stream, pdl));
    }
  }
  // (everything the head waits for is enqueued before the head itself: the host must never sit between a waiting
  // kernel and the launch it waits for)
  for (int gi = n - 1; gi >= 0; --gi) {
    tp_gpu& me = g[gi];
    device_guard dg(me.device);
    if (gi == 0) {  // softmax(T) + first-maximum token (llama_cu.cu:1196-1209), the token to every GPU
      LCU_TRY(launch_small(tp_wait_kernel, 32, me.stream, pdl, (const int*)(me.state + ST_FLAGS), (g_tp_debug & 1) ? 0 : n, (const int*)(me.state + ST_SEQ), 4 * L + 1,
                           me.state + ST_ERR));
      head_params h{};
      h.logits = me.logits; h.probs = me.probs; h.n_vocab = V; h.temperature = opt.temperature;
      h.token_out = me.state + ST_TOKEN; h.next_ids = me.ids;
      h.pos = me.state + ST_POS; h.advance = 1; h.log = me.log; h.step = me.state + ST_STEP; h.log_capacity = opt.context_len;
      LCU_TRY(launch_logits_head(h, me.stream, 0));
      id_list il{};
      for (int j = 1; j < n; ++j) il.ids[il.n++] = g[j].ids;
      tp_token_kernel<<<1, 1, 0, me.stream>>>(il, me.state + ST_TOKEN);
      LCU_CUDA(cudaGetLastError());
    } else {
      LCU_TRY(launch_bump_pos(me.state + ST_POS, 1, me.stream));
    }
  }
  // join: stream 0 continues when every GPU has finished the step
  for (int gi = 1; gi < n; ++gi) {
    device_guard dg(g[gi].device);
    LCU_CUDA(cudaEventRecord(g[gi].ev, g[gi].stream));
  }
  {
    device_guard dg(g[0].device);
    for (int gi = 1; gi < n; ++gi) LCU_CUDA(cudaStreamWaitEvent(g[0].stream, g[gi].ev, 0));
  }
  return LCU_OK;
}

int tp_impl::build_graph(int variant) {
  device_guard dg(g[0].device);
  cudaGraph_t gr = nullptr;
  if (cudaStreamBeginCapture(g[0].stream, cudaStreamCaptureModeRelaxed) != cudaSuccess) {
    cudaGetLastError();
    return LCU_ERR_CUDA;
  }
  int rc = enqueue_step(variant);
  cudaError_t e = cudaStreamEndCapture(g[0].stream, &gr);
  if (rc != LCU_OK || e != cudaSuccess || gr == nullptr) {
    if (gr) cudaGraphDestroy(gr);
    cudaGetLastError();
    return rc ? rc : LCU_ERR_CUDA;
  }
  e = cudaGraphInstantiate(&graph[variant], gr, 0);
  cudaGraphDestroy(gr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    graph[variant] = nullptr;
    set_last_error("cudaGraphInstantiate: %s", cudaGetErrorString(e));
    return LCU_ERR_CUDA;
  }
  return LCU_OK;
}

int tp_impl::run_step(int n_keys) {
  const int variant = n_keys > 64 * opt.attn_cluster ? 1 : 0;
  if (!warmed[variant]) {  // first use of a variant runs un-captured (function attributes)
    warmed[variant] = true;
    return enqueue_step(variant);
  }
  if (opt.use_graph && !graph[variant] && !graph_failed && build_graph(variant) != LCU_OK) {
    graph_failed = true;
    fprintf(stderr, "llama_cu_b200: CUDA graph capture of the tensor-parallel step failed (%s); launching kernels directly\n", last_error());
  }
  if (graph[variant]) {
    device_guard dg(g[0].device);
    LCU_CUDA(cudaGraphLaunch(graph[variant], g[0].stream));
    return LCU_OK;
  }
  return enqueue_step(variant);
}

// position and token of step `i` of this call to every GPU (pinned staging slots i are written once per call)
int tp_impl::stage(const short* tokens, int i) {
  h_stage[2 + i] = start_pos + i;
  h_ids[i] = tokens[i];
  {
    device_guard dg(g[0].device);
    if (i == 0) LCU_CUDA(cudaMemsetAsync(g[0].state + ST_STEP, 0, 4, g[0].stream));  // the token log of this call starts empty
    LCU_CUDA(cudaEventRecord(g[0].ev, g[0].stream));
  }
  for (int gi = 0; gi < n; ++gi) {
    device_guard dg(g[gi].device);
    if (gi > 0) LCU_CUDA(cudaStreamWaitEvent(g[gi].stream, g[0].ev, 0));
    LCU_CUDA(cudaMemcpyAsync(g[gi].state + ST_POS, h_stage + 2 + i, 4, cudaMemcpyHostToDevice, g[gi].stream));
    LCU_CUDA(cudaMemcpyAsync(g[gi].ids, h_ids + i, 2, cudaMemcpyHostToDevice, g[gi].stream));
    if (gi > 0) LCU_CUDA(cudaEventRecord(g[gi].ev, g[gi].stream));
  }
  device_guard dg(g[0].device);
  for (int gi = 1; gi < n; ++gi) LCU_CUDA(cudaStreamWaitEvent(g[0].stream, g[gi].ev, 0));
  return LCU_OK;
}

// after stream 0 has been synchronised: token and GPU 0's error word came back in h_stage; the other GPUs' words are read
int tp_impl::finish(const char* who) {
  int code = h_stage[1];
  for (int gi = 0; gi < n; ++gi) {
    device_guard dg(g[gi].device);
    int e = 0;
    LCU_CUDA(cudaMemcpy(&e, g[gi].state + ST_ERR, 4, cudaMemcpyDeviceToHost));
    if (e) {
      code = e;
      LCU_CUDA(cudaMemset(g[gi].state + ST_ERR, 0, 4));
    }
  }
  if (code != 0) {
    set_last_error("%s: a kernel gave up on a bounded wait (device error 0x%x)", who, code);
    return LCU_ERR_DEVICE_WAIT;
  }
  return LCU_OK;
}

int tp_decoder::next_token(const short* tokens, int n_tokens, int* token_out) {
  tp_impl& c = *impl;
  LCU_REQUIRE(n_tokens >= 1, "next_token: no tokens given");
  LCU_REQUIRE(n_tokens + c.start_pos <= c.opt.context_len, "next_token: %d new tokens at position %d exceed the context length %d", n_tokens,
              c.start_pos, c.opt.context_len);
  for (int i = 0; i < n_tokens; ++i)
    LCU_REQUIRE(tokens[i] >= 0 && (uint32_t)tokens[i] < c.p.n_vocab, "next_token: token id %d outside the vocabulary", tokens[i]);
  // a prompt runs as single-token steps (each one sharded over all GPUs); only the last step's token is returned
  for (int i = 0; i < n_tokens; ++i) {
    LCU_TRY(c.stage(tokens, i));
    LCU_TRY(c.run_step(c.start_pos + i + 1));
  }
  device_guard dg(c.g[0].device);
  LCU_CUDA(cudaMemcpyAsync(c.h_stage, c.g[0].state + ST_TOKEN, 8, cudaMemcpyDeviceToHost, c.g[0].stream));
  LCU_CUDA(cudaStreamSynchronize(c.g[0].stream));
  LCU_TRY(c.finish("next_token"));
  c.start_pos += n_tokens;
  *token_out = c.h_stage[0];
  return LCU_OK;
}

int tp_decoder::decode_chained(short first_token, int n_steps, short* tokens_out, float* ms_out) {
  tp_impl& c = *impl;
  LCU_REQUIRE(n_steps >= 1 && n_steps + c.start_pos <= c.opt.context_len, "decode_chained: %d steps at position %d exceed the context length %d",
              n_steps, c.start_pos, c.opt.context_len);
  LCU_REQUIRE(first_token >= 0 && (uint32_t)first_token < c.p.n_vocab, "decode_chained: token id %d outside the vocabulary", first_token);
  LCU_TRY(c.stage(&first_token, 0));
  device_guard dg(c.g[0].device);
  LCU_CUDA(cudaEventRecord(c.t0, c.g[0].stream));
  for (int i = 0; i < n_steps; ++i) LCU_TRY(c.run_step(c.start_pos + i + 1));
  LCU_CUDA(cudaEventRecord(c.t1, c.g[0].stream));
  LCU_CUDA(cudaMemcpyAsync(c.h_ids, c.g[0].log, (size_t)n_steps * 2, cudaMemcpyDeviceToHost, c.g[0].stream));
  LCU_CUDA(cudaMemcpyAsync(c.h_stage, c.g[0].state + ST_TOKEN, 8, cudaMemcpyDeviceToHost, c.g[0].stream));
  LCU_CUDA(cudaStreamSynchronize(c.g[0].stream));
  LCU_TRY(c.finish("decode_chained"));
  c.start_pos += n_steps;
  memcpy(tokens_out, c.h_ids, (size_t)n_steps * 2);
  if (ms_out) LCU_CUDA(cudaEventElapsedTime(ms_out, c.t0, c.t1));
  return LCU_OK;
}

int tp_decoder::read_probs(__half* out_host) {
  tp_impl& c = *impl;
  device_guard dg(c.g[0].device);
  LCU_CUDA(cudaMemcpy(out_host, c.g[0].probs, (size_t)c.p.n_vocab * 2, cudaMemcpyDeviceToHost));
  return LCU_OK;
}

}  // namespace lcu
