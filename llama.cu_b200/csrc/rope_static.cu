// lcu_rope_scatter_static: the RoPE + cache-write operator for callers that must not allocate.
//
// lcu_rope_scatter builds its cos/sin table in a buffer it cudaMallocs and frees on every call.
// Some callers cannot afford that: a serving process that has already handed every spare byte of
// HBM to its own KV-cache pool (the allocation would fail), a loop that must not stall (cudaMalloc
// and cudaFree synchronise the whole device), or a host that forbids allocation after start-up.
// This variant keeps the table in a fixed file-scope device array instead, so it allocates
// nothing: no cudaMalloc, no cudaFree, no allocating library routine.
//
// Cost and limits: the table covers at most ROPE_STATIC_MAX_ENTRIES = 262144 (position, pair)
// entries, e.g. 4096 positions at head_dim 128; larger requests are rejected.  All calls share the
// one array and it keeps the previous call's contents: each call rewrites the entries of the
// positions it is about to use, so nothing has to be cleared, but two calls whose kernels overlap
// on the GPU (different streams) race on it.
//
// When the 2 MiB are taken: the array belongs to this file's device module, and the CUDA runtime
// loads a module the first time something in it is used.  That first use is the first call on a
// device (cudaGetSymbolAddress with that device current), so it is the FIRST CALL that reserves the
// 2 MiB and may synchronise - not the loading of the library.  Make one call per device at start-up
// (a one-row call is enough), before the process hands the rest of HBM to its own pool and outside
// any stream capture; from then on the array stays until the process exits and a call takes no
// device memory at all.
#include "../../include/llama_cu_c.h"
#include "ops.cuh"

namespace {
constexpr size_t ROPE_STATIC_MAX_ENTRIES = 262144;
// In host code this name is only a handle for the runtime, not an address a kernel could use.
static __device__ __align__(256) float2 g_rope_static[ROPE_STATIC_MAX_ENTRIES];

// device address of g_rope_static on the current device, resolved once per device
int static_table(float2** out) {
  static float2* addr[64] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  LCU_REQUIRE(dev >= 0 && dev < 64, "rope_scatter_static: device index %d not supported", dev);
  if (!addr[dev]) {
    float2* p = nullptr;
    LCU_CUDA(cudaGetSymbolAddress((void**)&p, g_rope_static));
    addr[dev] = p;
  }
  *out = addr[dev];
  return lcu::LCU_OK;
}
}  // namespace

extern "C" int lcu_rope_scatter_static(void* q_dev, const void* k_new_dev, const void* v_new_dev, void* k_cache_dev, void* v_cache_dev,
                                       int pos0, int m, int dim, int n_heads, int ctx_len, void* stream) {
  using namespace lcu;
  {
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) {
      cudaGetLastError();
      set_last_error("no CUDA device is visible: this library has no CPU path");
      return LCU_ERR_CUDA;
    }
  }
  LCU_REQUIRE(n_heads >= 1 && dim >= 2 && dim % n_heads == 0 && (dim / n_heads) % 2 == 0, "rope_scatter_static: bad dim %d / n_heads %d", dim, n_heads);
  LCU_REQUIRE(m >= 1 && pos0 >= 0 && pos0 + m <= ctx_len, "rope_scatter_static: positions %d..%d outside the context length %d", pos0, pos0 + m, ctx_len);
  const int hd = dim / n_heads;
  // only positions < pos0 + m are used, so only those count against the table size
  const size_t need = (size_t)(pos0 + m) * (hd / 2);
  LCU_REQUIRE(need <= ROPE_STATIC_MAX_ENTRIES,
              "rope_scatter_static: %d positions x %d pairs = %zu table entries exceed the static table of %zu entries; use lcu_rope_scatter",
              pos0 + m, hd / 2, need, ROPE_STATIC_MAX_ENTRIES);
  float2* table = nullptr;
  int rc = static_table(&table);
  if (rc) return rc;
  rc = launch_rope_table(table, pos0 + m, hd, 10000.0f, (cudaStream_t)stream, pos0);  // only the rows this call reads
  if (rc) return rc;
  return launch_rope_scatter((__half*)q_dev, (const __half*)k_new_dev, (const __half*)v_new_dev, (__half*)k_cache_dev, (__half*)v_cache_dev,
                             table, nullptr, pos0, m, dim, n_heads, ctx_len, (cudaStream_t)stream);
}
