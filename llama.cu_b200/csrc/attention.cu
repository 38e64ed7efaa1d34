// Fused attention over the fp16 KV cache for sm_100a.
//
// Replaces the reference's matmul_qk -> softmax_rows -> matmul_qkv chain (llama_cu.cu:400-531,
// called at 1161-1171) and its per-layer score tensor with one kernel that keeps scores and
// probabilities on chip.  The reference's rounding points are kept ("parity" arithmetic):
//   score  s_t = half( (sum_i q_i k_ti) / sqrtf(head_dim) )                    llama_cu.cu:420-425
//   prob   p_t = half( expf(s_t - max) / sum_t' expf(s_t' - max) )             llama_cu.cu:443-498
//   out    o_j = half( sum_t float(p_t) float(v_tj) )                          llama_cu.cu:524-529
// which needs the row's max and sum before any probability is formed, so the kernel is two-pass
// over the scores (held in shared memory as halves), not an online-softmax.
//
// One thread-block cluster of CS CTAs serves one (query row, head): each CTA takes a contiguous
// slice of the cached positions.  K and V are stored head-major ([head][position][head_dim], keys
// already rotated), so a slice is one contiguous run of 2*head_dim-byte rows.  Latency plan for
// decode (short slices): the K rows AND the V rows of the first rounds are requested up front, so
// there is one trip to memory instead of two; every CTA pushes its (max, sum) pair into all peers'
// shared memory (st.shared::cluster) and its partial output into CTA 0's, which leaves two cluster
// barriers in the kernel.  Slice sums are combined as sum_r lsum_r * expf(lmax_r - max) in rank order.
#include "attention.cuh"

namespace lcu {
namespace {

constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int PRE_ROUNDS = 4;  // rounds of K and V rows requested together at kernel start
constexpr int BATCH = 4;       // rounds whose row loads are issued before the first of them is used

__device__ __forceinline__ void st_dsmem_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// Tensor-parallel decode: the CTA that wrote a head's output (into this GPU's row and, as peer stores, into the other
// GPUs' rows) counts itself behind a device-scope fence; the last one of the launch fences at system scope - cumulative
// over everything counted before it - and writes this GPU's flag into the memory of every GPU that waits for the row.
__device__ __forceinline__ void publish_when_last(const attn_params& p, int tid, int n_ctas) {
  __syncthreads();  // the storing threads' writes are ordered before thread 0's fence
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(p.done_count, 1) == n_ctas - 1) {
      atomicExch(p.done_count, 0);
      fence_acq_rel_sys();
      const int stamp = *p.seq * p.exchanges_per_step + p.exchange_id;
      for (int q = 0; q < p.n_peer_flag; ++q) st_relaxed_sys(p.peer_flag[q], stamp);
    }
  }
}

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) attn_kernel(const attn_params p) {
  constexpr int LPR = HD / 8;    // lanes that share one cached row (8 halves = 16 bytes each)
  constexpr int RPW = 32 / LPR;  // rows a warp handles per round
  constexpr int RPR = ATT_WARPS * RPW;  // rows per round of the whole CTA
  extern __shared__ __align__(16) uint8_t smem[];
  float* xmax = reinterpret_cast<float*>(smem);  // [8] slice maxima of all ranks (pushed by the peers)
  float* xsum = xmax + 8;                        // [8] slice exp-sums relative to the slice maximum
  float* rpart = xsum + 8;                       // [8][HD] partial outputs of all ranks (used on rank 0)
  float* wpart = rpart + 8 * HD;                 // [ATT_WARPS][HD]
  float* wred = wpart + ATT_WARPS * HD;          // [2 * ATT_WARPS] scratch
  __half* sc = reinterpret_cast<__half*>(wred + 2 * ATT_WARPS);  // [chunk] scores of this CTA's slice

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = lane / LPR, gl = lane % LPR;
  const uint32_t rank = cluster_ctarank(), cs = cluster_nctarank();
  const int head = blockIdx.y, qrow = blockIdx.z;

  pdl_launch_dependents();
  // Remote shared-memory stores need the target CTA to have started: arrive now, wait right before
  // the first push (split-phase, so the wait is free by then).
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  pdl_wait();

  const int start_pos = p.pos ? *p.pos : p.pos_value;
  const int T = start_pos + qrow + 1;  // causal: row r sees positions 0 .. start_pos + r
  const int chunk = (T + (int)cs - 1) / (int)cs;
  const int t0 = min(T, (int)rank * chunk), t1 = min(T, t0 + chunk);
  const int n = t1 - t0;

  const __half* kbase = p.k_cache + ((size_t)head * p.ctx_len + t0) * HD + gl * 8;
  const __half* vbase = p.v_cache + ((size_t)head * p.ctx_len + t0) * HD + gl * 8;

  // requests for the first rounds of K and V go out together
  uint4 kreg[PRE_ROUNDS], vreg[PRE_ROUNDS];
#pragma unroll
  for (int r = 0; r < PRE_ROUNDS; ++r) {
    const int t = r * RPR + warp * RPW + grp;
    kreg[r] = make_uint4(0, 0, 0, 0);
    vreg[r] = make_uint4(0, 0, 0, 0);
    if (t < n) {
      kreg[r] = *reinterpret_cast<const uint4*>(kbase + (size_t)t * HD);
      vreg[r] = *reinterpret_cast<const uint4*>(vbase + (size_t)t * HD);
    }
  }
  float q[8];
  {
    const uint4 qv = *reinterpret_cast<const uint4*>(p.q + (size_t)qrow * p.ldq + head * HD + gl * 8);
    const __half2* h = reinterpret_cast<const __half2*>(&qv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      q[2 * i] = f.x;
      q[2 * i + 1] = f.y;
    }
  }
  const float scale_div = sqrtf((float)HD);

  // ---- pass 1: scores of the slice, rounded to half, and the slice maximum.  Rounds are taken BATCH at a time with
  // all their row loads issued before the first use (long slices would otherwise pay one memory latency per round).
  float lmax = -CUDART_INF_F;
  for (int base = 0; base < n; base += BATCH * RPR) {
    uint4 kv[BATCH];
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
      const int t = base + j * RPR + warp * RPW + grp;
      if (base == 0 && j < PRE_ROUNDS) kv[j] = kreg[j < PRE_ROUNDS ? j : 0];
      else if (t < n) kv[j] = *reinterpret_cast<const uint4*>(kbase + (size_t)t * HD);
      else kv[j] = make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
      const int t = base + j * RPR + warp * RPW + grp;
      float s = 0.f;
      const __half2* h = reinterpret_cast<const __half2*>(&kv[j]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(h[i]);
        s += q[2 * i] * f.x;
        s += q[2 * i + 1] * f.y;
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (t < n) {
        const __half sh = __float2half(s / scale_div);
        if (gl == 0) sc[t] = sh;
        lmax = fmaxf(lmax, __half2float(sh));
      }
    }
  }
  lmax = warp_max(lmax);
  if (lane == 0) wred[warp] = lmax;
  __syncthreads();
  lmax = wred[0];
#pragma unroll
  for (int w = 1; w < ATT_WARPS; ++w) lmax = fmaxf(lmax, wred[w]);

  // slice exp-sum relative to the slice maximum (fixed order: lanes, then warps)
  float lsum = 0.f;
  for (int t = tid; t < n; t += ATT_THREADS) lsum += expf(__half2float(sc[t]) - lmax);
  lsum = warp_sum(lsum);
  if (lane == 0) wred[ATT_WARPS + warp] = lsum;
  __syncthreads();
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
  if (tid < (int)cs) {  // thread r pushes this slice's pair into rank r's table
    float s = 0.f;
    for (int w = 0; w < ATT_WARPS; ++w) s += wred[ATT_WARPS + w];
    st_dsmem_f32(mapa(smem_u32(&xmax[rank]), tid), lmax);
    st_dsmem_f32(mapa(smem_u32(&xsum[rank]), tid), s);
  }
  cluster_sync();
  float gmax = -CUDART_INF_F;
  for (uint32_t r = 0; r < cs; ++r) gmax = fmaxf(gmax, xmax[r]);
  float gsum = 0.f;
  for (uint32_t r = 0; r < cs; ++r) {
    const float m = xmax[r];
    if (m > -CUDART_INF_F) gsum += xsum[r] * expf(m - gmax);  // an empty slice contributes nothing
  }

  // ---- pass 2: probabilities rounded to half, times V (rounds in batches, as above)
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int base = 0; base < n; base += BATCH * RPR) {
    uint4 vv[BATCH];
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
      const int t = base + j * RPR + warp * RPW + grp;
      if (base == 0 && j < PRE_ROUNDS) vv[j] = vreg[j < PRE_ROUNDS ? j : 0];
      else if (t < n) vv[j] = *reinterpret_cast<const uint4*>(vbase + (size_t)t * HD);
      else vv[j] = make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
      const int t = base + j * RPR + warp * RPW + grp;
      if (t < n) {
        const float pr = __half2float(__float2half(expf(__half2float(sc[t]) - gmax) / gsum));
        const __half2* h = reinterpret_cast<const __half2*>(&vv[j]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __half22float2(h[i]);
          acc[2 * i] += pr * f.x;
          acc[2 * i + 1] += pr * f.y;
        }
      }
    }
  }
  // combine the row groups of a warp, then the warps, then the cluster ranks (all in fixed order)
#pragma unroll
  for (int i = 0; i < 8; ++i)
    for (int o = LPR; o < 32; o <<= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  if (grp == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) wpart[warp * HD + gl * 8 + i] = acc[i];
  }
  __syncthreads();
  if (tid < HD) {
    float s = 0.f;
    for (int w = 0; w < ATT_WARPS; ++w) s += wpart[w * HD + tid];
    st_dsmem_f32(mapa(smem_u32(&rpart[rank * HD + tid]), 0), s);  // into rank 0's table
  }
  cluster_sync();
  if (rank == 0 && tid < HD) {
    float s = 0.f;
    for (uint32_t r = 0; r < cs; ++r) s += rpart[r * HD + tid];
    const __half o = __float2half(s);
    const size_t at = (size_t)qrow * p.ldo + head * HD + tid;
    p.out[at] = o;
    for (int q = 0; q < p.n_peer_out; ++q) p.peer_out[q][at] = o;  // tensor-parallel: into every GPU's row (peer stores)
  }
  if (rank == 0 && p.done_count != nullptr) publish_when_last(p, tid, (int)(gridDim.y * gridDim.z));
}

// ---------------------------------------------------------------------------------------------------
// Streaming variant for long slices.  Same arithmetic, same thread-to-row assignment and summation order as
// attn_kernel (the two give identical bits), but the rows come through shared memory: a producer warp brings the
// slice in as contiguous bulk copies of up to 64 rows (the cache is head-major, so a slice is one contiguous run),
// K chunks first, then V chunks, through a ring of three buffers with full/empty mbarriers.  With per-thread
// loads a CTA has at most 4 rows per thread in flight and a 260-row slice pays a memory latency every few rounds;
// here the ring keeps 48 KB per CTA requested at all times.
constexpr int AS_CH = 64;  // rows per chunk
constexpr int AS_NB = 3;   // ring buffers
constexpr int AS_THREADS = ATT_THREADS + 32;

template <int HD>
__global__ void __launch_bounds__(AS_THREADS, 3) attn_stream_kernel(const attn_params p) {
  constexpr int LPR = HD / 8, RPW = 32 / LPR, RPR = ATT_WARPS * RPW;
  constexpr int CHUNK_BYTES = AS_CH * HD * 2;
  extern __shared__ __align__(16) uint8_t smem[];
  float* xmax = reinterpret_cast<float*>(smem);
  float* xsum = xmax + 8;
  float* rpart = xsum + 8;
  float* wpart = rpart + 8 * HD;
  float* wred = wpart + ATT_WARPS * HD;
  uint64_t* bars = reinterpret_cast<uint64_t*>(wred + 2 * ATT_WARPS);  // full[AS_NB], empty[AS_NB]
  uint8_t* ring = reinterpret_cast<uint8_t*>(bars + 8);                // 16-byte aligned (bulk-copy destination)
  __half* sc = reinterpret_cast<__half*>(ring + AS_NB * CHUNK_BYTES);  // [slice] scores

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = lane / LPR, gl = lane % LPR;
  const uint32_t rank = cluster_ctarank(), cs = cluster_nctarank();
  const int head = blockIdx.y, qrow = blockIdx.z;

  pdl_launch_dependents();
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  if (tid == 0) {
    for (int i = 0; i < AS_NB; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);
      mbar_init(smem_u32(&bars[AS_NB + i]), ATT_WARPS);
    }
    fence_mbar_init();
  }
  __syncthreads();
  pdl_wait();

  const int start_pos = p.pos ? *p.pos : p.pos_value;
  const int T = start_pos + qrow + 1;
  const int chunk = (T + (int)cs - 1) / (int)cs;
  const int t0 = min(T, (int)rank * chunk), t1 = min(T, t0 + chunk);
  const int n = t1 - t0;
  const int nch = (n + AS_CH - 1) / AS_CH, total = 2 * nch;

  if (warp == ATT_WARPS) {
    // ---- producer: chunk i < nch is K chunk i, chunk nch + j is V chunk j.  Chunks up to nch + AS_NB - 1 need only
    // buffers that pass 1 releases; the rest wait for pass 2 and are issued after the first cluster barrier.
    const __half* kb = p.k_cache + ((size_t)head * p.ctx_len + t0) * HD;
    const __half* vb = p.v_cache + ((size_t)head * p.ctx_len + t0) * HD;
    auto issue = [&](int i) {
      const int b = i % AS_NB, use = i / AS_NB;
      if (use > 0 && !mbar_wait(smem_u32(&bars[AS_NB + b]), (use - 1) & 1, p.err, DEV_ERR_EMPTY_WAIT)) return false;
      const int c = i < nch ? i : i - nch;
      const uint32_t bytes = (uint32_t)min(AS_CH, n - c * AS_CH) * (HD * 2);
      const uint32_t full = smem_u32(&bars[b]);
      mbar_arrive_expect_tx(full, bytes);
      bulk_g2s(smem_u32(ring + b * CHUNK_BYTES), (i < nch ? kb : vb) + (size_t)c * AS_CH * HD, bytes, full);
      return true;
    };
    const int first_part = min(total, nch + AS_NB);
    bool ok = true;
    if (lane == 0)
      for (int i = 0; i < first_part && ok; ++i) ok = issue(i);
    __syncwarp();
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    cluster_sync();
    if (lane == 0)
      for (int i = first_part; i < total && ok; ++i) ok = issue(i);
    __syncwarp();
    cluster_sync();
    return;
  }

  float q[8];
  {
    const uint4 qv = *reinterpret_cast<const uint4*>(p.q + (size_t)qrow * p.ldq + head * HD + gl * 8);
    const __half2* h = reinterpret_cast<const __half2*>(&qv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      q[2 * i] = f.x;
      q[2 * i + 1] = f.y;
    }
  }
  const float scale_div = sqrtf((float)HD);
  bool ok = true;

  // ---- pass 1: scores of the slice, rounded to half, and the slice maximum
  float lmax = -CUDART_INF_F;
  for (int c = 0; c < nch; ++c) {
    const int b = c % AS_NB;
    ok = ok && mbar_wait(smem_u32(&bars[b]), (c / AS_NB) & 1, p.err, DEV_ERR_FULL_WAIT);
    const uint8_t* buf = ring + b * CHUNK_BYTES;
#pragma unroll
    for (int r0 = 0; r0 < AS_CH; r0 += RPR) {
      const int r = r0 + warp * RPW + grp;
      const int t = c * AS_CH + r;
      uint4 kv = make_uint4(0, 0, 0, 0);
      if (ok && t < n) kv = *reinterpret_cast<const uint4*>(buf + (size_t)r * (HD * 2) + gl * 16);
      float s = 0.f;
      const __half2* h = reinterpret_cast<const __half2*>(&kv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __half22float2(h[i]);
        s += q[2 * i] * f.x;
        s += q[2 * i + 1] * f.y;
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (t < n) {
        const __half sh = __float2half(s / scale_div);
        if (gl == 0) sc[t] = sh;
        lmax = fmaxf(lmax, __half2float(sh));
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bars[AS_NB + b]));
  }
  lmax = warp_max(lmax);
  if (lane == 0) wred[warp] = lmax;
  bar_sync(1, ATT_THREADS);
  lmax = wred[0];
#pragma unroll
  for (int w = 1; w < ATT_WARPS; ++w) lmax = fmaxf(lmax, wred[w]);

  float lsum = 0.f;
  for (int t = tid; t < n; t += ATT_THREADS) lsum += expf(__half2float(sc[t]) - lmax);
  lsum = warp_sum(lsum);
  if (lane == 0) wred[ATT_WARPS + warp] = lsum;
  bar_sync(1, ATT_THREADS);
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
  if (tid < (int)cs) {
    float s = 0.f;
    for (int w = 0; w < ATT_WARPS; ++w) s += wred[ATT_WARPS + w];
    st_dsmem_f32(mapa(smem_u32(&xmax[rank]), tid), lmax);
    st_dsmem_f32(mapa(smem_u32(&xsum[rank]), tid), s);
  }
  cluster_sync();
  float gmax = -CUDART_INF_F;
  for (uint32_t r = 0; r < cs; ++r) gmax = fmaxf(gmax, xmax[r]);
  float gsum = 0.f;
  for (uint32_t r = 0; r < cs; ++r) {
    const float m = xmax[r];
    if (m > -CUDART_INF_F) gsum += xsum[r] * expf(m - gmax);
  }

  // ---- pass 2: probabilities rounded to half, times V
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int c = 0; c < nch; ++c) {
    const int i = nch + c, b = i % AS_NB;
    ok = ok && mbar_wait(smem_u32(&bars[b]), (i / AS_NB) & 1, p.err, DEV_ERR_FULL_WAIT);
    const uint8_t* buf = ring + b * CHUNK_BYTES;
#pragma unroll
    for (int r0 = 0; r0 < AS_CH; r0 += RPR) {
      const int r = r0 + warp * RPW + grp;
      const int t = c * AS_CH + r;
      if (ok && t < n) {
        const float pr = __half2float(__float2half(expf(__half2float(sc[t]) - gmax) / gsum));
        const uint4 vv = *reinterpret_cast<const uint4*>(buf + (size_t)r * (HD * 2) + gl * 16);
        const __half2* h = reinterpret_cast<const __half2*>(&vv);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float2 f = __half22float2(h[k]);
          acc[2 * k] += pr * f.x;
          acc[2 * k + 1] += pr * f.y;
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bars[AS_NB + b]));
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    for (int o = LPR; o < 32; o <<= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  if (grp == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) wpart[warp * HD + gl * 8 + i] = acc[i];
  }
  bar_sync(1, ATT_THREADS);
  if (tid < HD) {
    float s = 0.f;
    for (int w = 0; w < ATT_WARPS; ++w) s += wpart[w * HD + tid];
    st_dsmem_f32(mapa(smem_u32(&rpart[rank * HD + tid]), 0), s);
  }
  cluster_sync();
  if (rank == 0 && tid < HD) {
    float s = 0.f;
    for (uint32_t r = 0; r < cs; ++r) s += rpart[r * HD + tid];
    const __half o = __float2half(s);
    const size_t at = (size_t)qrow * p.ldo + head * HD + tid;
    p.out[at] = o;
    for (int q = 0; q < p.n_peer_out; ++q) p.peer_out[q][at] = o;  // tensor-parallel: into every GPU's row (peer stores)
  }
  if (rank == 0 && p.done_count != nullptr) publish_when_last(p, tid, (int)(gridDim.y * gridDim.z));
}

template <int HD>
int launch_hd(const attn_params& p, int m, int cs, int max_T, cudaStream_t stream, int pdl) {
  const int chunk = (max_T + cs - 1) / cs;
  const size_t smem = (16 + 8 * HD + ATT_WARPS * HD + 2 * ATT_WARPS) * sizeof(float) + (size_t)chunk * 2 + 16;
  LCU_REQUIRE(smem <= 200 * 1024, "attention: %d positions per CTA do not fit in shared memory", chunk);
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(attn_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cs, p.n_heads, m);
  cfg.blockDim = dim3(ATT_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  LCU_CUDA(cudaLaunchKernelEx(&cfg, attn_kernel<HD>, p));
  return LCU_OK;
}

template <int HD>
int launch_stream_hd(const attn_params& p, int m, int cs, int max_T, cudaStream_t stream, int pdl) {
  const int chunk = (max_T + cs - 1) / cs;
  const size_t smem = (16 + 8 * HD + ATT_WARPS * HD + 2 * ATT_WARPS) * sizeof(float) + 64 + (size_t)AS_NB * AS_CH * HD * 2 +
                      (((size_t)chunk * 2 + 15) & ~(size_t)15);
  LCU_REQUIRE(smem <= 200 * 1024, "attention: %d positions per CTA do not fit in shared memory", chunk);
  LCU_REQUIRE(p.err != nullptr, "attention: the streaming kernel needs a device error word");
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(attn_stream_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cs, p.n_heads, m);
  cfg.blockDim = dim3(AS_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  LCU_CUDA(cudaLaunchKernelEx(&cfg, attn_stream_kernel<HD>, p));
  return LCU_OK;
}

int g_attn_stream = -1;  // -1 = streaming kernel when a CTA's slice can exceed 64 rows, 0 = never, 1 = always

}  // namespace

void attention_set_stream_mode(int mode) { g_attn_stream = mode; }

// loads the decode attention kernels on the current device ahead of their first launch (see gemv_single_row_preload)
int attention_preload() {
  cudaFuncAttributes fa;
  LCU_CUDA(cudaFuncGetAttributes(&fa, attn_kernel<128>));
  LCU_CUDA(cudaFuncGetAttributes(&fa, attn_kernel<64>));
  LCU_CUDA(cudaFuncGetAttributes(&fa, attn_stream_kernel<128>));
  LCU_CUDA(cudaFuncGetAttributes(&fa, attn_stream_kernel<64>));
  return LCU_OK;
}

int launch_attention(const attn_params& p, int m, int cluster, int max_T, cudaStream_t stream, int pdl) {
  LCU_REQUIRE(m >= 1 && p.n_heads >= 1, "attention: empty problem");
  LCU_REQUIRE(cluster >= 1 && cluster <= 8 && (cluster & (cluster - 1)) == 0, "attention: cluster size %d not in {1,2,4,8}", cluster);
  LCU_REQUIRE(max_T >= 1 && max_T <= p.ctx_len, "attention: %d positions exceed the context length %d", max_T, p.ctx_len);
  const bool streaming = p.err != nullptr && (g_attn_stream == 1 || (g_attn_stream < 0 && (max_T + cluster - 1) / cluster > AS_CH));
  if (streaming) {
    if (p.head_dim == 128) return launch_stream_hd<128>(p, m, cluster, max_T, stream, pdl);
    if (p.head_dim == 64) return launch_stream_hd<64>(p, m, cluster, max_T, stream, pdl);
  }
  if (p.head_dim == 128) return launch_hd<128>(p, m, cluster, max_T, stream, pdl);
  if (p.head_dim == 64) return launch_hd<64>(p, m, cluster, max_T, stream, pdl);
  LCU_REQUIRE(false, "attention: head_dim %d not supported (64 or 128)", p.head_dim);
}

}  // namespace lcu
