// Logits head on a thread-block cluster: softmax with temperature over the logits, probabilities
// rounded to half, and the first index of the maximum probability - what the reference does with
// softmax_rows (llama_cu.cu:433-499), a 64 KB device-to-host copy and std::max_element on the host
// (llama_cu.cu:1196-1209).
//
// The reference's exp-sum order is kept exactly: its 256 threads sum elements t, t+256, ... one
// after the other, 8 warps reduce with xor trees, one warp reduces the 8 warp sums with an xor
// tree.  Here CTA r of an 8-CTA cluster plays the reference's warp r: it owns the elements with
// (i mod 256) / 32 == r, computes their exponentials in parallel into shared memory, lets 32
// threads add them in the reference's order, and the 8 warp sums are exchanged through distributed
// shared memory.  One block doing all of this alone takes ~27 us on a B200 (it is bound by one
// SM's instruction issue); the cluster takes a few microseconds.
#include <math_constants.h>

#include "ops.cuh"

namespace lcu {
namespace {

constexpr int HC_THREADS = 512;
constexpr int HC_WARPS = HC_THREADS / 32;
constexpr int HC_CLUSTER = 8;

__device__ __forceinline__ void st_dsmem_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void st_dsmem_s32(uint32_t addr, int v) {
  asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

__global__ void __cluster_dims__(HC_CLUSTER, 1, 1) __launch_bounds__(HC_THREADS) logits_head_cluster_kernel(const head_params p, int J) {
  extern __shared__ float e_buf[];      // [J][32]: element (j, l) is logit index 256*j + 32*rank + l
  __shared__ float x_max[HC_CLUSTER];   // pushed by every rank
  __shared__ float x_wsum[HC_CLUSTER];  // the reference's 8 warp sums, pushed by every rank
  __shared__ float x_best[HC_CLUSTER];  // rank 0 only: best probability of every rank
  __shared__ int x_idx[HC_CLUSTER];     //              and its first index
  __shared__ float s_red[HC_WARPS];
  __shared__ int s_redi[HC_WARPS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int V = p.n_vocab;
  const float temp = p.temperature;
  const int n_local = J * 32;

  pdl_launch_dependents();
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");  // peers must run before remote stores
  pdl_wait();

  // ---- v = float(x) / temp (llama_cu.cu:445), kept in shared memory; maximum
  float mx = -CUDART_INF_F;
  for (int e = tid; e < n_local; e += HC_THREADS) {
    const int i = 256 * (e >> 5) + 32 * (int)rank + (e & 31);
    float v = -CUDART_INF_F;
    if (i < V) v = __half2float(p.logits[i]) / temp;
    e_buf[e] = v;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  if (lane == 0) s_red[warp] = mx;
  __syncthreads();
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
  if (tid < HC_CLUSTER) {
    float m = s_red[0];
    for (int w = 1; w < HC_WARPS; ++w) m = fmaxf(m, s_red[w]);
    st_dsmem_f32(mapa(smem_u32(&x_max[rank]), tid), m);
  }
  cluster_sync();
  mx = x_max[0];
#pragma unroll
  for (int r = 1; r < HC_CLUSTER; ++r) mx = fmaxf(mx, x_max[r]);

  // ---- exponentials in parallel, then the reference's summation order
  for (int e = tid; e < n_local; e += HC_THREADS) {
    const float v = e_buf[e];
    e_buf[e] = v == -CUDART_INF_F ? 0.f : expf(v - mx);  // padding beyond n_vocab adds nothing
  }
  __syncthreads();
  if (warp == 0) {
    float s = 0.f;
    for (int j = 0; j < J; ++j) {
      const int i = 256 * j + 32 * (int)rank + lane;
      if (i < V) s += e_buf[j * 32 + lane];  // thread (32*rank + lane) of the reference: i, i+256, ...
    }
    s = warp_sum(s);                         // xor tree 16, 8, 4, 2, 1 as llama_cu.cu:477-479
    if (lane < HC_CLUSTER) st_dsmem_f32(mapa(smem_u32(&x_wsum[rank]), lane), s);
  }
  cluster_sync();
  float sum;
  {
    float t = lane < 8 ? x_wsum[lane] : 0.f;  // xor tree 4, 2, 1 over the 8 warp sums (llama_cu.cu:486-489)
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    sum = __shfl_sync(0xffffffffu, t, 0);
  }

  // ---- probabilities (half), their maximum, and the first index that attains it
  float best = -1.f;
  int best_i = 0x7fffffff;
  for (int e = tid; e < n_local; e += HC_THREADS) {
    const int i = 256 * (e >> 5) + 32 * (int)rank + (e & 31);
    if (i < V) {
      const __half ph = __float2half(e_buf[e] / sum);
      p.probs[i] = ph;
      const float pf = __half2float(ph);
      if (pf > best || (pf == best && i < best_i)) {
        best = pf;
        best_i = i;
      }
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
    }
  }
  if (lane == 0) {
    s_red[warp] = best;
    s_redi[warp] = best_i;
  }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < HC_WARPS; ++w)
      if (s_red[w] > best || (s_red[w] == best && s_redi[w] < best_i)) {
        best = s_red[w];
        best_i = s_redi[w];
      }
    st_dsmem_f32(mapa(smem_u32(&x_best[rank]), 0), best);
    st_dsmem_s32(mapa(smem_u32(&x_idx[rank]), 0), best_i);
  }
  cluster_sync();
  if (rank == 0 && tid == 0) {
    best = x_best[0];
    best_i = x_idx[0];
    for (int r = 1; r < HC_CLUSTER; ++r)
      if (x_best[r] > best || (x_best[r] == best && x_idx[r] < best_i)) {
        best = x_best[r];
        best_i = x_idx[r];
      }
    if (p.token_out) *p.token_out = best_i;
    if (p.next_ids) p.next_ids[0] = (short)best_i;
    if (p.pos) *p.pos += p.advance;
    if (p.log && p.step) {
      if (*p.step < p.log_capacity) p.log[*p.step] = (short)best_i;
      *p.step += 1;
    }
  }
}

}  // namespace

int head_preload() {
  cudaFuncAttributes fa;
  LCU_CUDA(cudaFuncGetAttributes(&fa, logits_head_cluster_kernel));
  return LCU_OK;
}

int launch_logits_head(const head_params& p, cudaStream_t stream, int pdl) {
  const int J = (p.n_vocab + 255) / 256;
  const size_t smem = (size_t)J * 32 * sizeof(float);
  if (p.n_vocab < 256 || smem > 160 * 1024) return launch_logits_head_single(p, stream, pdl);
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(logits_head_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(HC_CLUSTER);
  cfg.blockDim = dim3(HC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  LCU_CUDA(cudaLaunchKernelEx(&cfg, logits_head_cluster_kernel, p, J));
  return LCU_OK;
}

}  // namespace lcu
