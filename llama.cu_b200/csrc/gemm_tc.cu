// Prompt-processing GEMM on the 5th-generation tensor cores: out(m,N) = A(m,K) . W(N,K)^T + beta * out.
//
// Replaces the reference's prefill tile kernel (matmul_nt_wmma_128x64x64, llama_cu.cu:150-220) for
// fp16 weights.  Both operands are K-major (the reference's own layout), fp16 in, fp32 accumulation
// in tensor memory, one rounding to fp16 on the way out (with the residual add when beta = 1).
//
// One CTA computes one 128 x BN output tile (BN = the widest of 128, 64, 32 weight rows that divides N).  Warp roles:
//   warp 0  - one lane issues the TMA loads: per 64-wide K step a 128 x 64 activation box and a
//             BN x 64 weight box (cp.async.bulk.tensor.2d, 128-byte swizzle, zero fill past the last row)
//             into a ring of shared-memory stages, completion on `full` mbarriers;
//   warp 1  - allocates BN tensor-memory columns; one lane issues tcgen05.mma (M = 128, N = BN, K = 16,
//             four per stage) from shared-memory descriptors and releases each stage with
//             tcgen05.commit on its `empty` mbarrier; a last commit signals the epilogue;
//   warps 2-5 - epilogue: each warp reads its 32-lane quadrant of the accumulator with tcgen05.ld
//             (32 columns at a time), adds beta * out, rounds to half and stores 64-byte row pieces.
// Two kernels share these roles: gemm_tc_kernel (one SM per tile, optionally a cluster of 2 or 4 CTAs that
// splits K and reduces through distributed shared memory - for few rows) and gemm_tc_pair_kernel (two SMs per
// 256-row tile with tcgen05.mma.cta_group::2, persistent, two accumulators in tensor memory - for many rows).
// No TMA multicast anywhere.  Every mbarrier wait is bounded: on expiry the kernel records a code in the error
// word, skips ahead and still frees its tensor memory.
#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <unordered_map>

#include "gemm_tc.cuh"
#include "tc_common.cuh"

namespace lcu {
namespace {

constexpr int BM = 128;      // output rows (tokens) per tile = TMEM lanes
constexpr int BK = 64;       // K per stage: 64 halves = one 128-byte swizzled row
constexpr int TC_THREADS = 192;
constexpr int TC_MAX_STAGES = 12;  // one-SM kernel: barrier slots for the ring

// half(acc + beta * previous) for 32 consecutive outputs of one row (64 bytes, 16-byte aligned)
__device__ __forceinline__ void store_row_piece(__half* o, const float (&acc)[32], float beta) {
  uint4 v[4];
  if (beta != 0.f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = reinterpret_cast<const uint4*>(o)[i];
  }
  __half2* h = reinterpret_cast<__half2*>(v);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float a0 = acc[2 * i], a1 = acc[2 * i + 1];
    if (beta != 0.f) {
      const float2 prev = __half22float2(h[i]);
      a0 = fmaf(beta, prev.x, a0);
      a1 = fmaf(beta, prev.y, a1);
    }
    h[i] = __floats2half2_rn(a0, a1);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(o)[i] = v[i];
}
__device__ __forceinline__ void st_dsmem_f4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// One-SM kernel.  S > 1 splits K over a cluster of S CTAs that share one output tile (few rows and a
// narrow matrix would otherwise leave most SMs without a tile while the weights stream from HBM):
// CTA r accumulates k-blocks [r nk / S, (r+1) nk / S), then owns the BN / S output columns starting at
// r BN / S: every CTA pushes its fp32 partials of the columns it does not own into the owner's shared
// memory (distributed shared memory), one cluster barrier, and the owner adds them in rank order.
template <int BN, int S>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                                __half* out, int m, int N, int K, float beta, int nstages, int a_box_rows,
                                                                int kbs, int* err) {
  // A stage holds the activation box (a_box_rows rows, 2 to 16 KB) and the BN weight rows.  The MMA reads 128 operand rows
  // from the box's address: with a short box the rest comes from whatever follows in the ring, reaches output rows >= m
  // only, and those are never stored.  Short prompts so get up to 12 stages of weights in flight instead of 6.
  // A stage is kbs (1, 2 or 4) 64-wide k-blocks, brought in by ONE tensor copy per operand (a three-dimensional box:
  // 64 halves x rows x k-blocks, which lands as kbs swizzled operand tiles one after the other): the copies, not the
  // bytes, set the pace of a CTA that streams weights for few rows - 0.28 us per k-block with one box per k-block
  // whether the tile is 32 or 128 wide, on 32 or 148 SMs, with 6 or 11 stages.
  constexpr uint32_t B_BYTES = BN * BK * 2;
  const uint32_t A_BYTES = (uint32_t)a_box_rows * (BK * 2), STAGE = (uint32_t)kbs * (A_BYTES + B_BYTES);
  constexpr int MAXS = TC_MAX_STAGES;
  constexpr uint32_t TM_COLS = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;  // tensor memory comes in powers of two
  // instruction descriptor: fp32 accumulate, fp16 x fp16, both K-major, N = BN, M = 128
  constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  constexpr int CW = BN / S;        // columns owned by each CTA of the cluster
  constexpr int CPR = CW / 32;      // 32-column pieces per owner
  constexpr uint32_t RED_BYTES = S > 1 ? (S - 1) * BM * CW * 4 : 0;
  static_assert(CW % 32 == 0, "each CTA of a split-K cluster owns whole 32-column pieces");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms are 1024-byte aligned
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t red = base + (uint32_t)nstages * STAGE;  // [S-1 senders][CW/4][128 rows] float4
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)nstages * STAGE + RED_BYTES);  // full[MAXS], empty[MAXS], tmem_full
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAXS + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = S > 1 ? (int)cluster_ctarank() : 0;
  const int n0 = (blockIdx.x / S) * BN, m0 = blockIdx.y * BM;
  const int groups = (K / BK + kbs - 1) / kbs;  // (k-blocks past K in the last group arrive as zeros)
  const int kb0 = rank * groups / S, nk = (rank + 1) * groups / S - kb0;  // this CTA's groups of k-blocks

  if (threadIdx.x == 0) {
    for (int i = 0; i < nstages; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);
      mbar_init(smem_u32(&bars[MAXS + i]), 1);
    }
    mbar_init(smem_u32(&bars[2 * MAXS]), 1);
    fence_mbar_init();
  }
  if (warp == 1) {  // tensor-memory allocation: BN fp32 columns x 128 lanes
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (S > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");  // waited for before the first remote store
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();  // everything above ran under the previous kernel's tail; nothing before this line touches global memory

  float own[S == 1 ? 1 : CPR][32];  // epilogue warps: this CTA's partial of the columns it owns
  bool go = false;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer
      for (int kb = 0; kb < nk; ++kb) {
        const int s = kb % nstages, use = kb / nstages;
        if (use > 0 && !mbar_wait(smem_u32(&bars[MAXS + s]), (use - 1) & 1, err, DEV_ERR_EMPTY_WAIT)) break;
        const uint32_t full = smem_u32(&bars[s]);
        const uint32_t dst = base + (uint32_t)s * STAGE;
        mbar_arrive_expect_tx(full, STAGE);
        tma_load_3d(dst, &map_a, 0, m0, (kb0 + kb) * kbs, full);
        tma_load_3d(dst + (uint32_t)kbs * A_BYTES, &map_b, 0, n0, (kb0 + kb) * kbs, full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer
      bool ok = true;
      for (int kb = 0; kb < nk && ok; ++kb) {
        const int s = kb % nstages, use = kb / nstages;
        ok = mbar_wait(smem_u32(&bars[s]), use & 1, err, DEV_ERR_FULL_WAIT);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = base + (uint32_t)s * STAGE, b_addr = a_addr + (uint32_t)kbs * A_BYTES;
        for (int j = 0; j < kbs; ++j) {
          const uint64_t a_desc = smem_desc_sw128(a_addr + (uint32_t)j * A_BYTES), b_desc = smem_desc_sw128(b_addr + (uint32_t)j * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)  // 16 halves = 32 bytes = 2 descriptor address units per K step
            tc_mma_f16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, IDESC, (kb | j | k) != 0);
        }
        tc_commit(smem_u32(&bars[MAXS + s]));  // the stage is free once these MMAs have read it
      }
      tc_commit(smem_u32(&bars[2 * MAXS]));  // accumulator complete (also on the error path: lets the epilogue leave)
    }
  } else {
    // ---- epilogue: warp w may touch TMEM lanes 32 * (w % 4) ... + 31 only
    const int quad = warp & 3;
    const int trow = quad * 32 + lane;  // row of the tile = TMEM lane
    const bool ok = mbar_wait(smem_u32(&bars[2 * MAXS]), 0, err, DEV_ERR_TMEM_WAIT);
    tc_fence_after();
    go = __all_sync(0xffffffffu, ok && *(volatile int*)err == 0);  // warp-uniform: tcgen05.ld is .aligned
    if (S > 1) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");  // every CTA of the cluster is running
    if (go) {
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int owner = c / CPR;
        if (S == 1 || owner == rank) {
#pragma unroll
          for (int i = 0; i < 32; ++i) own[S == 1 ? 0 : c % CPR][i] = __uint_as_float(r[i]);
          if (S == 1) {
            // (a tile width that does not divide N: the last tile's columns past N hold products with zero-filled rows)
            if (m0 + trow < m && n0 + c * 32 < N) store_row_piece(out + (size_t)(m0 + trow) * N + n0 + c * 32, own[0], beta);
          }
        } else {
          // float4 number j4 of this row goes to ((j4 * 128 + row) * 16) so that a warp's stores are contiguous
          const uint32_t slot = (uint32_t)(rank < owner ? rank : rank - 1);
          const uint32_t dst = mapa(red + slot * (uint32_t)(BM * CW * 4), (uint32_t)owner);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4)
            st_dsmem_f4(dst + (uint32_t)((((c % CPR) * 8 + j4) * BM + trow) * 16), __uint_as_float(r[4 * j4]), __uint_as_float(r[4 * j4 + 1]),
                        __uint_as_float(r[4 * j4 + 2]), __uint_as_float(r[4 * j4 + 3]));
        }
      }
    }
  }
  if (S > 1) {
    __syncwarp();
    if (warp < 2) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");  // complete the start barrier (epilogue warps did already)
    cluster_sync();  // all partials have landed in their owners' shared memory
    if (warp >= 2 && go && *(volatile int*)err == 0) {
      const int trow = (warp & 3) * 32 + lane;
      const float4* part = reinterpret_cast<const float4*>(smem + (size_t)nstages * STAGE);
#pragma unroll
      for (int cc = 0; cc < CPR; ++cc) {
#pragma unroll
        for (int s = 0; s < S - 1; ++s) {  // senders in rank order
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 v = part[(size_t)s * (BM * CW / 4) + (cc * 8 + j4) * BM + trow];
            own[cc][4 * j4] += v.x;
            own[cc][4 * j4 + 1] += v.y;
            own[cc][4 * j4 + 2] += v.z;
            own[cc][4 * j4 + 3] += v.w;
          }
        }
        if (m0 + trow < m) store_row_piece(out + (size_t)(m0 + trow) * N + n0 + rank * CW + cc * 32, own[cc], beta);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------
// Two-SM variant for more than 128 rows: a cluster of two CTAs owns a 256 x BN output tile
// (tcgen05.mma.cta_group::2, M = 256).  Each CTA loads its own 128 activation rows and its own half of
// the BN weight rows, so a stage costs each SM (128 + BN/2) x 128 bytes of L2 traffic for
// 128 x BN x 64 multiply-adds - half of what the one-SM kernel needs, which is what bounds that kernel.
// The pair is persistent: it walks the tile list with a stride of the number of clusters and keeps two
// accumulators in tensor memory, so the epilogue of one tile runs under the main loop of the next.
//
// Barriers (all waits bounded):
//   full[s]       leader CTA only; the leader's producer arrives with the byte count of both CTAs' boxes,
//                 both producers' TMA loads complete on it (the peer addresses it through the cluster window)
//   empty[s]      one per CTA; the leader's MMA thread commits to both (commit with a CTA mask)
//   acc_full[b]   one per CTA; committed to both when a tile's last MMA has been issued
//   acc_empty[b]  leader only, 8 arrivals: the four epilogue warps of both CTAs
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(cta_mask)
               : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

template <int BN>  // weight rows per pair tile: 128 or 256
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
    gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, __half* out, int m, int N, int K,
                        float beta, int nstages, int tiles_m, int n_tiles, int kbs, int* err) {
  // (a stage is kbs k-blocks, one three-dimensional tensor copy per operand, as in the one-SM kernel)
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2;
  const uint32_t STAGE = (uint32_t)kbs * (A_BYTES + B_BYTES);
  constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
  constexpr uint32_t TMEM_COLS = 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)nstages * STAGE);  // full[8] empty[8] acc_full[2] acc_empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int n_clusters = gridDim.x / 2, cluster_id = blockIdx.x / 2;
  const int nk = K / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < nstages; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);
      mbar_init(smem_u32(&bars[8 + i]), 1);
    }
    mbar_init(smem_u32(&bars[16]), 1);
    mbar_init(smem_u32(&bars[17]), 1);
    mbar_init(smem_u32(&bars[18]), 8);
    mbar_init(smem_u32(&bars[19]), 8);
    fence_mbar_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();  // everything above ran under the previous kernel's tail; nothing before this line touches global memory

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer (both CTAs)
      int it = 0;
      bool ok = true;
      for (int t = cluster_id; t < n_tiles && ok; t += n_clusters) {
        const int m0 = (t % tiles_m) * (2 * BM) + (int)rank * BM;
        const int n0 = (t / tiles_m) * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < nk; kb += kbs, ++it) {  // (k-blocks past K arrive as zeros)
          const int s = it % nstages;
          const uint32_t ph = (uint32_t)(it / nstages) & 1u;
          ok = mbar_wait(smem_u32(&bars[8 + s]), ph ^ 1u, err, DEV_ERR_EMPTY_WAIT);
          if (!ok) break;
          const uint32_t full_leader = mapa(smem_u32(&bars[s]), 0);
          const uint32_t dst = base + (uint32_t)s * STAGE;
          if (rank == 0) mbar_arrive_expect_tx(smem_u32(&bars[s]), 2 * STAGE);
          tma_load_3d_pair(dst, &map_a, 0, m0, kb, full_leader);
          tma_load_3d_pair(dst + (uint32_t)kbs * A_BYTES, &map_b, 0, n0, kb, full_leader);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {  // ---- MMA issuer (leader CTA only)
      int it = 0, ti = 0;
      bool ok = true;
      for (int t = cluster_id; t < n_tiles && ok; t += n_clusters, ++ti) {
        const int b = ti & 1;
        const uint32_t acc_ph = (uint32_t)(ti >> 1) & 1u;
        ok = mbar_wait(smem_u32(&bars[18 + b]), acc_ph ^ 1u, err, DEV_ERR_TMEM_WAIT);  // both epilogues have drained buffer b
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * BN);
        for (int kb = 0; kb < nk; kb += kbs, ++it) {
          const int s = it % nstages;
          const uint32_t ph = (uint32_t)(it / nstages) & 1u;
          ok = mbar_wait(smem_u32(&bars[s]), ph, err, DEV_ERR_FULL_WAIT);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = base + (uint32_t)s * STAGE, b_addr = a_addr + (uint32_t)kbs * A_BYTES;
          for (int j = 0; j < kbs && kb + j < nk; ++j) {
            const uint64_t a_desc = smem_desc_sw128(a_addr + (uint32_t)j * A_BYTES), b_desc = smem_desc_sw128(b_addr + (uint32_t)j * B_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) tc_mma_f16_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, (kb | j | k) != 0);
          }
          tc_commit_pair(smem_u32(&bars[8 + s]), 3);  // frees the stage in both CTAs
        }
        tc_commit_pair(smem_u32(&bars[16 + b]), 3);  // accumulator b complete (also after a failed wait: lets the epilogues leave)
      }
    }
  } else {
    // ---- epilogue (both CTAs): warp w reads TMEM lanes 32 * (w % 4) ... + 31 of its own CTA
    const int quad = warp & 3;
    const uint32_t acc_empty_leader = mapa(smem_u32(&bars[18]), 0);
    int ti = 0;
    bool go = true;
    for (int t = cluster_id; t < n_tiles && go; t += n_clusters, ++ti) {
      const int b = ti & 1;
      const uint32_t acc_ph = (uint32_t)(ti >> 1) & 1u;
      const int row = (t % tiles_m) * (2 * BM) + (int)rank * BM + quad * 32 + lane;
      const int n0 = (t / tiles_m) * BN;
      const bool ok = mbar_wait(smem_u32(&bars[16 + b]), acc_ph, err, DEV_ERR_TMEM_WAIT);
      tc_fence_after();
      go = __all_sync(0xffffffffu, ok && *(volatile int*)err == 0);
      if (!go) break;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tc_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * BN + c), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < m) {
          float acc[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = __uint_as_float(r[i]);
          store_row_piece(out + (size_t)row * N + n0 + c, acc, beta);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader + (uint32_t)(b * 8));  // buffer b may be overwritten
    }
  }
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync();  // nobody leaves while the other CTA's MMAs, loads or arrivals may still touch this CTA
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// cuTensorMapEncodeTiled through the runtime's driver entry-point lookup (no link against libcuda)
using encode_fn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encoder(encode_fn* out) {
  static encode_fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    LCU_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    LCU_REQUIRE(q == cudaDriverEntryPointSuccess && p, "cuTensorMapEncodeTiled is not available in this driver");
    fn = reinterpret_cast<encode_fn>(p);
  }
  *out = fn;
  return LCU_OK;
}

// [rows][K] halves, row-major; box = box_rows x 64 halves with 128-byte swizzle; rows past the end read as zero.
// Encoded maps are kept (a map depends on address and shape only), so that a prompt's 7 products per layer
// do not pay for two driver calls each.
struct map_key {
  const void* ptr;
  uint64_t rows, K, ld;
  uint32_t box_rows;
  bool operator==(const map_key& o) const { return ptr == o.ptr && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows; }
};
struct map_key_hash {
  size_t operator()(const map_key& k) const {
    uint64_t h = (uint64_t)(uintptr_t)k.ptr * 0x9e3779b97f4a7c15ull;
    h ^= (k.rows + 0x632be59bd9b4e019ull) * 0xff51afd7ed558ccdull;
    h ^= (k.K * 31 + k.ld * 17 + k.box_rows) * 0xc4ceb9fe1a85ec53ull;
    return (size_t)(h ^ (h >> 29));
  }
};

int make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t K, uint64_t ld, uint32_t box_rows, bool streamed) {
  static std::mutex mu;
  static std::unordered_map<map_key, CUtensorMap, map_key_hash> cache;
  const map_key key{ptr, rows, K, ld, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *map = it->second;
    return LCU_OK;
  }
  encode_fn enc;
  int rc = get_encoder(&enc);
  if (rc) return rc;
  const cuuint64_t dims[2] = {K, rows};
  const cuuint64_t strides[1] = {ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, streamed ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  LCU_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d (ptr %p rows %llu K %llu ld %llu)", (int)r, ptr,
              (unsigned long long)rows, (unsigned long long)K, (unsigned long long)ld);
  if (cache.size() >= 8192) cache.clear();
  cache.emplace(key, *map);
  return LCU_OK;
}

template <int BN, int S>
int launch_bn(__half* out, const __half* lhs, int ldx, const __half* w, int m, int N, int K, float beta, int* err, cudaStream_t stream) {
  CUtensorMap map_a, map_b;
  const int a_box_rows = m > 64 ? BM : m > 32 ? 64 : m > 16 ? 32 : 16;
  constexpr size_t RED = S > 1 ? (size_t)(S - 1) * BM * (BN / S) * 4 : 0;
  // k-blocks per stage: as many as still leave four stages and two stages' worth of work per CTA
  int kbs = tc_kb_per_stage();
  if (kbs <= 0) {
    kbs = 4;
    while (kbs > 1 && ((200 * 1024 - RED) / ((size_t)kbs * (a_box_rows + BN) * BK * 2) < 3 || K / BK / S < 2 * kbs)) kbs /= 2;
  }
  LCU_REQUIRE(kbs == 1 || kbs == 2 || kbs == 4, "gemm_tc: %d k-blocks per stage is not 1, 2 or 4", kbs);
  {
    const uint64_t dims_a[3] = {(uint64_t)BK, (uint64_t)m, (uint64_t)(K / BK)}, str_a[2] = {(uint64_t)ldx * 2, (uint64_t)BK * 2};
    const uint32_t box_a[3] = {(uint32_t)BK, (uint32_t)a_box_rows, (uint32_t)kbs};
    int rc = tc_encode_map(&map_a, lhs, 3, dims_a, str_a, box_a);
    if (rc) return rc;
    const uint64_t dims_b[3] = {(uint64_t)BK, (uint64_t)N, (uint64_t)(K / BK)}, str_b[2] = {(uint64_t)K * 2, (uint64_t)BK * 2};
    const uint32_t box_b[3] = {(uint32_t)BK, (uint32_t)BN, (uint32_t)kbs};
    rc = tc_encode_map(&map_b, w, 3, dims_b, str_b, box_b, true);
    if (rc) return rc;
  }
  const size_t STAGE = (size_t)kbs * (a_box_rows + BN) * BK * 2;
  const int groups = (K / BK + kbs - 1) / kbs;
  int nstages = (int)((200 * 1024 - RED) / STAGE);
  if (nstages > TC_MAX_STAGES) nstages = TC_MAX_STAGES;
  if (nstages > groups) nstages = groups;
  // (the MMA reads BM operand rows from the last stage's box too: the slack below covers what a short box leaves out)
  const size_t smem = nstages * STAGE + RED + (size_t)(BM - a_box_rows) * BK * 2 + 1024 /* alignment slack */ + 256 /* barriers, tmem slot */;
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(((N + BN - 1) / BN) * S, (m + BM - 1) / BM);
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (S > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = S;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (prompt_pdl()) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  LCU_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, S>, map_a, map_b, out, m, N, K, beta, nstages, a_box_rows, kbs, err));
  return LCU_OK;
}

template <int BN>
int launch_pair(__half* out, const __half* lhs, int ldx, const __half* w, int m, int N, int K, float beta, int* err, cudaStream_t stream) {
  CUtensorMap map_a, map_b;
  int kbs = sk_kb_per_stage();  // k-blocks per stage and tensor copy
  if (kbs <= 0) kbs = 2;
  if (kbs > 2 || K / BK < 2) kbs = 1;
  {
    const uint64_t dims_a[3] = {(uint64_t)BK, (uint64_t)m, (uint64_t)(K / BK)}, str_a[2] = {(uint64_t)ldx * 2, (uint64_t)BK * 2};
    const uint32_t box_a[3] = {(uint32_t)BK, (uint32_t)BM, (uint32_t)kbs};
    int rc = tc_encode_map(&map_a, lhs, 3, dims_a, str_a, box_a);
    if (rc) return rc;
    const uint64_t dims_b[3] = {(uint64_t)BK, (uint64_t)N, (uint64_t)(K / BK)}, str_b[2] = {(uint64_t)K * 2, (uint64_t)BK * 2};
    const uint32_t box_b[3] = {(uint32_t)BK, (uint32_t)(BN / 2), (uint32_t)kbs};
    rc = tc_encode_map(&map_b, w, 3, dims_b, str_b, box_b, true);
    if (rc) return rc;
  }
  const size_t STAGE = (size_t)kbs * (BM + BN / 2) * BK * 2;
  int nstages = (int)((200 * 1024) / STAGE);
  if (nstages > 8) nstages = 8;
  const size_t smem = nstages * STAGE + 1024 /* alignment slack */ + 256 /* barriers, tmem slot */;
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(gemm_tc_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_done[dev] = true;
  }
  const int tiles_m = (m + 2 * BM - 1) / (2 * BM), n_tiles = tiles_m * (N / BN);
  int clusters = gemv_sm_count() / 2;
  if (clusters > n_tiles) clusters = n_tiles;
  LCU_CUDA(launch_after(gemm_tc_pair_kernel<BN>, dim3(2 * clusters), dim3(TC_THREADS), smem, stream, map_a, map_b, out, m, N, K, beta, nstages, tiles_m,
                        n_tiles, kbs, err));
  return LCU_OK;
}

}  // namespace

int tc_encode_map(CUtensorMap* map, const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                  bool streamed) {
  LCU_REQUIRE(rank == 2 || rank == 3, "tensor map: rank %d not supported", rank);
  // encoded maps are kept (a map depends on address, shape and box only)
  static std::mutex mu;
  static std::unordered_map<std::string, CUtensorMap> cache;
  std::string key(reinterpret_cast<const char*>(&ptr), sizeof ptr);
  key.append(reinterpret_cast<const char*>(dims), sizeof(uint64_t) * rank);
  key.append(reinterpret_cast<const char*>(strides_bytes), sizeof(uint64_t) * (rank - 1));
  key.append(reinterpret_cast<const char*>(box), sizeof(uint32_t) * rank);
  key.push_back(streamed ? 's' : 'r');
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *map = it->second;
    return LCU_OK;
  }
  encode_fn enc;
  int rc = get_encoder(&enc);
  if (rc) return rc;
  cuuint64_t d[3], st[2];
  cuuint32_t b[3], es[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    if (i > 0) st[i - 1] = strides_bytes[i - 1];
  }
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, streamed ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  LCU_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (rank %d) failed with code %d", rank, (int)r);
  if (cache.size() >= 8192) cache.clear();
  cache.emplace(std::move(key), *map);
  return LCU_OK;
}

// Up to 128 rows the product streams the weights once and an SM takes in about 50 GB/s whatever its tile's width, so
// what counts is that all SMs stream the same number of bytes: tile widths from 96 to 256 (the last tile may hang
// over N) and split-K for the 128-wide tile are compared by waves x max(bytes per CTA / 50 GB/s, 0.27 us per K step)
// + 7 us per wave, against the whole matrix at 5.8 TB/s.  7B: w1|w3 (N = 22016) takes 160-wide tiles (138 CTAs, one
// wave, instead of 172 in two: 51 -> 32 us at 16 rows); N = 4096 keeps 128-wide tiles with K split four ways.
void gemm_tc_plan_short(int N, int K, int sms, int* tile_n, int* split) {
  const double nk = K / BK;
  double best = 1e30;
  int bn = 128, sp_best = 1;
  const int widths[6] = {128, 96, 160, 192, 224, 256};
  for (int i = 0; i < 6; ++i)
    for (int sp = 1; sp <= (widths[i] == 128 ? 4 : 1); sp *= 2) {
      if (nk < 8 * sp) continue;
      const long ctas = (long)((N + widths[i] - 1) / widths[i]) * sp, waves = (ctas + sms - 1) / sms;
      const double per_cta = std::max(widths[i] * 128.0 * nk / sp / 50e3, nk / sp * 0.27);
      const double est = std::max(waves * per_cta, (double)N * K * 2 / 5.8e6) + 7.0 * waves + (sp > 1 ? 1.5 : 0.0);
      if (est < best - 0.5) {  // (ties stay with the earlier candidate)
        best = est;
        bn = widths[i];
        sp_best = sp;
      }
    }
  *tile_n = bn;
  *split = sp_best;
}

int& tc_kb_per_stage() {
  static int kb = 0;
  return kb;
}

int& gemm_tc_sk_mode() {
  static int mode = -1;
  return mode;
}

// Estimated duration (microseconds) of an [m][K] x [N][K]^T product, m > 128, on the three kernels: whole tiles per SM
// pair, and the balanced kernel with 256- and 512-wide tiles.  Fitted to timings of the 7B, 13B and 65B products at 200 to
// 2048 rows (56 shapes; the picks sum to 10.45 ms against 10.26 ms for the best of the three each time, 11.10 ms for whole
// tiles alone and 10.51 ms for the balanced 256-wide kernel alone).
static void gemm_tc_estimates(int m, int N, int K, int sms, double* whole_us, double* t256_us, double* t512_us) {
  const long C = sms / 2, nk = K / BK, tm = (m + 2 * BM - 1) / (2 * BM);
  auto ceil_div_l = [](long a, long b) { return (a + b - 1) / b; };
  double whole;
  if ((m > 2 * BM || N > 8192) && N % 128 == 0) {
    const long n256 = tm * (N / 256);
    // (several hundred tiles of a short K: the whole-tile kernel's epilogues weigh more, 0.42 us per K step measured)
    if (N % 256 == 0 && n256 * 4 >= C * 3) whole = ceil_div_l(n256, C) * nk * (n256 > 300 && nk <= 80 ? 0.42 : n256 > 40 ? 0.38 : 0.34) + 5;
    else whole = ceil_div_l(tm * (N / 128), C) * nk * 0.37 + 5;
  } else {
    const long n128 = (long)((m + BM - 1) / BM) * (N / 128);
    long sp = n128 * 4 <= sms ? 4 : n128 * 2 <= sms ? 2 : 1;
    if (nk < 8 * sp) sp = 1;
    whole = ceil_div_l(n128 * sp, sms) * ((double)nk / sp) * 0.40 + 6;
  }
  auto balanced = [&](int bn) -> double {
    if (N % bn) return 1e30;
    const long n = tm * (N / bn), full = n / C, rest = n - full * C;
    const double per = bn == 256 ? 0.41 : 0.80;
    double t = full * (nk * per + (bn == 512 ? 4 : 0)) + 5;
    if (rest) {
      const long cs = std::min(C, std::min(rest * nk, rest * 3));
      const double per_s = cs > 40 ? per : (bn == 256 ? 0.36 : 0.72);
      t += (double)(rest * nk) / cs * per_s + (bn == 256 ? 8 : 26);
      if (bn == 256 && full == 0) t += 6;  // no whole wave: every tile is handed over, and nothing hides the first wait
    }
    return t;
  };
  *whole_us = whole;
  *t256_us = balanced(256);
  *t512_us = N >= 2 * K ? balanced(512) : 1e30;
}

// More than 128 rows: 0 = whole tiles per SM pair, 256 / 512 = the balanced kernel with that tile width (the one whose
// estimate is lowest; a balanced kernel has to beat whole tiles by 3 %).
int gemm_tc_plan_long(int m, int N, int K, int sms) {
  double whole, t256, t512;
  gemm_tc_estimates(m, N, K, sms, &whole, &t256, &t512);
  double best = whole;
  int tile = 0;
  if (t256 < 0.97 * whole && t256 < best) {
    best = t256;
    tile = 256;
  }
  if (t512 < 0.97 * whole && t512 < best) tile = 512;
  return tile;
}

int& gemm_tc_gate_mode() {
  static int mode = -1;
  return mode;
}

int gemm_tc_gated_tile(int m, int f, int K) {
  const int mode = gemm_tc_gate_mode();
  if (m <= BM || mode == 0) return 0;
  if (mode > 0) return mode == 512 && f % 256 == 0 ? 512 : 256;
  // the one launch (256 accumulator columns per tile: the gate's arithmetic runs under the next tile's main loop, so
  // its duration is the balanced kernel's for the stacked product plus about 3 us measured, more beyond 1024 rows)
  // against the best kernel for the stacked product plus the gate kernel's pass over the result (6 bytes per output
  // element at about 5 TB/s, and a launch).  7B shapes: the one launch wins 4 to 8 us per layer from 129 to 1024 rows.
  double whole, t256, t512;
  gemm_tc_estimates(m, 2 * f, K, gemv_sm_count(), &whole, &t256, &t512);
  const double gate_us = (double)m * f * 6.0 / 5.0e6 + 2;
  const double one_launch = t256 + 3 + (m > 1024 ? (m - 1024) * 0.016 : 0.0);
  return one_launch < std::min(whole, t512) + gate_us ? 256 : 0;
}

bool gemm_tc_supported(int m, int N, int K, int ldx, const void* lhs, const void* w, const void* out) {
  return m >= 1 && N % 32 == 0 && K % BK == 0 && ldx % 8 == 0 && ((uintptr_t)lhs & 15) == 0 && ((uintptr_t)w & 15) == 0 &&
         ((uintptr_t)out & 15) == 0;
}

int launch_gemm_tc(__half* out, const __half* lhs, int ldx, const __half* w, int m, int N, int K, float beta, int* err, cudaStream_t stream,
                   int force_bn, int force_pair, int force_split) {
  LCU_REQUIRE(gemm_tc_supported(m, N, K, ldx, lhs, w, out), "gemm_tc: unsupported shape m=%d N=%d K=%d ldx=%d or unaligned pointers", m, N, K, ldx);
  const int sms = gemv_sm_count();
  // More than 128 rows: three kernels can run the product - whole tiles per SM pair (below), the kernel that deals the
  // K steps of the last, partial wave evenly over the pairs (gemm_tc_sk.cu, 256-wide tiles), and the same with
  // 512-wide tiles (a third less operand traffic per multiply-add, no overlap of epilogue and main loop).  Which one is
  // fastest depends on how the tile count meets the 74 pairs (gemm_tc_estimates).  Mode -1 = that rule; 256 / 512 force
  // the balanced kernel with that tile width; 0 = never.
  if (force_pair < 0 && !force_bn && (m > BM || gemm_tc_sk_mode() > 0)) {
    const int mode = gemm_tc_sk_mode();
    int tile = mode > 0 ? mode : 0;
    if (mode < 0) tile = gemm_tc_plan_long(m, N, K, sms);
    if (tile && gemm_tc_sk_supported(m, N, K, ldx, lhs, w, out, tile)) return launch_gemm_tc_sk(out, lhs, ldx, w, m, N, K, beta, err, stream, tile);
  }
  // Large products: the two-SM kernel, with its 256-wide tile when that still gives (nearly) every SM pair a tile.
  // Up to 256 rows of a matrix with few tiles stay on the one-SM kernel, which can split K to fill the SMs.
  int pair = force_pair;
  if (pair < 0) {
    pair = 0;
    if (m > BM && N % 128 == 0 && !force_bn && (m > 2 * BM || N > 8192)) {
      const long tiles_m = (m + 2 * BM - 1) / (2 * BM), clusters = sms / 2;
      pair = (N % 256 == 0 && tiles_m * (N / 256) * 4 >= clusters * 3) ? 256 : 128;
    }
  }
  if (pair) {
    LCU_REQUIRE((pair == 128 || pair == 256) && N % pair == 0, "gemm_tc: pair tile width %d does not divide N=%d", pair, N);
    return pair == 256 ? launch_pair<256>(out, lhs, ldx, w, m, N, K, beta, err, stream) : launch_pair<128>(out, lhs, ldx, w, m, N, K, beta, err, stream);
  }
  int bn = force_bn, split = force_split;
  if (!bn) bn = N % 128 == 0 ? 128 : N % 64 == 0 ? 64 : 32;  // measured: the widest tile wins even when it leaves SMs idle
  if (!force_bn && force_split < 0 && m <= BM && N % 128 == 0) gemm_tc_plan_short(N, K, sms, &bn, &split);
  LCU_REQUIRE(bn % 32 == 0 && bn >= 32 && bn <= 256, "gemm_tc: tile width %d is not a multiple of 32 up to 256", bn);
  if (bn == 128 && N % 128) split = 1;  // (the split-K clusters own whole 128-wide tiles)
  if (bn == 128) {
    if (split < 0) {
      const long tiles = (long)(N / 128) * ((m + BM - 1) / BM);
      split = tiles * 4 <= sms ? 4 : tiles * 2 <= sms ? 2 : 1;
    }
    if (K / BK < 8 * split) split = 1;  // every CTA of the cluster needs k-blocks of its own
    LCU_REQUIRE(split == 1 || split == 2 || split == 4, "gemm_tc: split-K factor %d is not 1, 2 or 4", split);
    if (split == 4) return launch_bn<128, 4>(out, lhs, ldx, w, m, N, K, beta, err, stream);
    if (split == 2) return launch_bn<128, 2>(out, lhs, ldx, w, m, N, K, beta, err, stream);
    return launch_bn<128, 1>(out, lhs, ldx, w, m, N, K, beta, err, stream);
  }
  switch (bn) {
    case 32: return launch_bn<32, 1>(out, lhs, ldx, w, m, N, K, beta, err, stream);
    case 64: return launch_bn<64, 1>(out, lhs, ldx, w, m, N, K, beta, err, stream);
    case 96: return launch_bn<96, 1>(out, lhs, ldx, w, m, N, K, beta, err, stream);
    case 160: return launch_bn<160, 1>(out, lhs, ldx, w, m, N, K, beta, err, stream);
    case 192: return launch_bn<192, 1>(out, lhs, ldx, w, m, N, K, beta, err, stream);
    case 224: return launch_bn<224, 1>(out, lhs, ldx, w, m, N, K, beta, err, stream);
    default: return launch_bn<256, 1>(out, lhs, ldx, w, m, N, K, beta, err, stream);
  }
}

}  // namespace lcu
