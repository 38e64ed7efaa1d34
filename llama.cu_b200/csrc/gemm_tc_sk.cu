// Prompt-processing GEMM, wide tiles with the K loop balanced over the SM pairs ("stream-K").
//
// out(m,N) = A(m,K) . W(N,K)^T + beta * out, fp16 operands, fp32 accumulation in tensor memory (the reference's
// prefill tile kernel, llama_cu.cu:150-220, is what it replaces).
//
// Two things bound the 256 x 256 pair kernel of gemm_tc.cu below the tensor-core rate.  (1) Operand traffic: every
// SM pulls (128 + 128) x 64 halves from L2 per 128 x 256 x 64 multiply-adds; measured, the kernel settles where that
// traffic meets the L2 bandwidth.  Here a pair's tile is 256 x 512: each CTA's 128 activation rows serve two
// tcgen05.mma.cta_group::2 of N = 256, which is 48 KiB of operands per CTA and K step instead of 64 KiB for the same
// arithmetic.  The two accumulators fill all 512 tensor-memory columns, so the epilogue does not overlap the next
// tile's main loop (a few per cent of a tile at K = 4096).  (2) Wave quantisation: a 512-row prompt times the 7B
// w1|w3 stack is 86 such tiles for 74 SM pairs.  Work is therefore dealt in units of one K step of one tile: pair c
// runs units [U c / C, U (c+1) / C) of the tile-major list.  A pair whose range starts inside a tile computes that
// tile's tail first and writes its fp32 partial sums to a workspace slot of its own, then raises a flag; the pair
// that ran the tile's first K step owns the tile and adds the partials of the pairs after it, in pair order, in its
// epilogue.  Ranges ascend, so a partial is the first thing its writer produces and the last thing its reader needs.
// Every wait (mbarriers, flags) is bounded and reports through the error word; no TMA multicast.
#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "gemm_tc.cuh"

#include <algorithm>
#include <vector>
#include "tc_common.cuh"

namespace lcu {
namespace {

constexpr int SK_BM = 128;  // rows per CTA (the pair's tile has 256)
constexpr int SK_BK = 64;
constexpr int SK_THREADS = 192;
constexpr int DEV_ERR_PARTIAL_WAIT = 0x107;  // a tile's owner timed out waiting for another pair's partial sums

__device__ __forceinline__ void sk_tma_load_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void sk_tma_load_pair_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void sk_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(cta_mask)
               : "memory");
}
__device__ __forceinline__ void sk_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void sk_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ int sk_ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void sk_st_release(int* p, int v) { asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

// tile store shared memory -> global (rows and columns past the tensor's end are not written)
__device__ __forceinline__ void sk_tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void sk_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void sk_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// bounded wait for *flag == value (one thread)
__device__ __forceinline__ bool sk_flag_wait(const int* flag, int value, int* err) {
  if (sk_ld_acquire(flag) == value) return true;
  const long long t0 = clock64();
  long long next_check = 400000;
  for (;;) {
    if (sk_ld_acquire(flag) == value) return true;
    const long long dt = clock64() - t0;
    if (dt > next_check) {
      if (*(volatile int*)err != 0) return false;
      if (dt > 2000000000ll) {
        atomicCAS(err, 0, DEV_ERR_PARTIAL_WAIT);
        return false;
      }
      next_check += 400000;
    }
  }
}

// pair c of C runs units [U c / C, U (c + 1) / C)
__host__ __device__ __forceinline__ long long sk_first_unit(long long U, int c, int C) { return U * c / C; }
__host__ __device__ __forceinline__ long long sk_min(long long a, long long b) { return a < b ? a : b; }

// A pair's schedule: first whole tiles, tile w C + c in wave w (at any time the pairs work on neighbouring tiles, which
// share weight panels and keep the working set inside L2), then its share of the K steps of the tiles that do not fill
// a wave.  Every role of the kernel walks the same list.
struct sk_schedule {
  int C, Cs, c, nk, full_waves, first_split_tile;  // Cs: pairs that take part in the split tiles (every one of them has a K step)
  long long U, u, u1;  // units of the split tiles: all, next of this pair, end of this pair's range
  int wave;
  __host__ __device__ void init(int n_tiles, int nk_, int C_, int c_) {
    C = C_;
    c = c_;
    nk = nk_;
    full_waves = n_tiles / C;
    first_split_tile = full_waves * C;
    U = (long long)(n_tiles - first_split_tile) * nk;
    // at most three pairs per shared tile: its owner adds the other pairs' sums one after the other at the very end of
    // the kernel, and what it reads of the first two is requested ahead (eight pairs per tile were slower even for
    // prompts of 16 rows, whose sums are small: 59 against 46 us on the 7B w1|w3)
    const long long split_pairs = (long long)(n_tiles - first_split_tile) * 3;
    Cs = (int)sk_min(sk_min((long long)C, U), split_pairs);
    u = c < Cs ? sk_first_unit(U, c, Cs) : 0;
    u1 = c < Cs ? sk_first_unit(U, c + 1, Cs) : 0;
    wave = 0;
  }
  // next segment: K steps [kb0, kb1) of tile `tile`; split = the tile is shared with other pairs
  __host__ __device__ bool next(int& tile, int& kb0, int& kb1, bool& split) {
    if (wave < full_waves) {
      tile = wave * C + c;
      kb0 = 0;
      kb1 = nk;
      split = false;
      ++wave;
      return true;
    }
    if (u >= u1) return false;
    const int lt = (int)(u / nk);
    tile = first_split_tile + lt;
    kb0 = (int)(u - (long long)lt * nk);
    kb1 = (int)sk_min((long long)nk, kb0 + (u1 - u));
    split = true;
    u += kb1 - kb0;
    return true;
  }
  // pairs after this one that hold later K steps of split tile `tile` (this pair ran its first)
  __host__ __device__ int peers_of(int tile) const {
    const long long tile_end = (long long)(tile - first_split_tile + 1) * nk;
    int n = 0;
    while (c + 1 + n < Cs && sk_first_unit(U, c + 1 + n, Cs) < tile_end) ++n;
    return n;
  }
};

// NB: 256-column accumulators per tile (1: the tile is 256 x 256 and tensor memory holds two of them).
// GATE: the two halves of a tile's accumulator columns are the same BN / 2 output columns of two matrices stacked in W -
// rows [n, n + BN / 2) and [gate_rows + n, gate_rows + n + BN / 2) - and the epilogue stores half(silu(half(a)) * half(b))
// (llama_cu.cu:533-539 on the half-rounded products, what the separate gate kernel computes from the stored halves): w1|w3
// and the SiLU gate as one launch, without the [rows][2 f] intermediate.  With NB = 1 each CTA of the pair loads one
// matrix's 128 rows, and the gate's arithmetic (a division and an exponential per element on four warps) runs under the
// next tile's main loop.
template <int NB, bool GATE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(SK_THREADS, 1)
    gemm_tc_sk_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_out, int m, int N, int K,
                      float beta, int nstages, int tiles_m, int n_tiles, float* workspace, int* flags, int seq, int* err, int gate_rows,
                      int kbs) {
  constexpr int BN = 256 * NB;
  constexpr int BN_OUT = GATE ? BN / 2 : BN;  // output columns per tile
  // a stage holds kbs (1 or 2) k-blocks: [kbs] A tiles, then per accumulator [kbs] B tiles, each operand brought in by one
  // three-dimensional tensor copy (64 halves x 128 rows x kbs k-blocks)
  constexpr uint32_t A_BYTES = SK_BM * SK_BK * 2, B_BYTES = 128 * SK_BK * 2;
  const uint32_t STAGE = (uint32_t)kbs * (A_BYTES + NB * B_BYTES);
  constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);  // fp32 acc, fp16 x fp16, K-major, N = 256, M = 256
  constexpr int NBUF = NB == 1 ? 2 : 1;  // accumulator buffers: the epilogue of one segment runs under the main loop of the next
  constexpr uint32_t TMEM_COLS = BN * NBUF;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  // output staging: per epilogue warp two buffers of 32 rows x 64 halves (128-byte swizzled rows, as the tensor maps want them)
  constexpr uint32_t STG_WARP = 2 * 4096, STG_BYTES = 4 * STG_WARP;
  const uint32_t stg_base = base + (uint32_t)nstages * STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)nstages * STAGE + STG_BYTES);  // full[8] empty[8] acc_full[2] acc_empty[2] part_done prev[4][2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 30);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int C = gridDim.x / 2, cluster_id = blockIdx.x / 2;
  const int nk = K / SK_BK;
  sk_schedule sched;
  sched.init(n_tiles, nk, C, cluster_id);
  int tile, kb0, kb1;
  bool split;

  if (threadIdx.x == 0) {
    for (int i = 0; i < nstages; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);
      mbar_init(smem_u32(&bars[8 + i]), 1);
    }
    mbar_init(smem_u32(&bars[16]), 1);  // acc_full[b] (each CTA)
    mbar_init(smem_u32(&bars[17]), 1);
    mbar_init(smem_u32(&bars[18]), 8);  // acc_empty[b] (leader): the four epilogue warps of both CTAs
    mbar_init(smem_u32(&bars[19]), 8);
    mbar_init(smem_u32(&bars[20]), 8);  // part_done (leader): the same eight warps have stored their partial sums
    for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&bars[21 + i]), 1);  // prev[warp][buffer]: the previous output values (beta != 0) have landed
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
      while (ok && sched.next(tile, kb0, kb1, split)) {
        const int m0 = (tile % tiles_m) * (2 * SK_BM) + (int)rank * SK_BM;
        // rows of W for this CTA's 128 columns of accumulator h: n0 + h * n_step
        const int n0 = (tile / tiles_m) * BN_OUT + (int)rank * ((GATE && NB == 1) ? gate_rows : 128);
        const int n_step = GATE ? gate_rows : 256;
        for (int kb = kb0; kb < kb1; kb += kbs, ++it) {  // (a segment of odd length loads one k-block it does not use)
          const int s = it % nstages;
          const uint32_t ph = (uint32_t)(it / nstages) & 1u;
          ok = mbar_wait(smem_u32(&bars[8 + s]), ph ^ 1u, err, DEV_ERR_EMPTY_WAIT);
          if (!ok) break;
          const uint32_t full_leader = mapa(smem_u32(&bars[s]), 0);
          const uint32_t dst = base + (uint32_t)s * STAGE;
          if (rank == 0) mbar_arrive_expect_tx(smem_u32(&bars[s]), 2 * STAGE);
          sk_tma_load_pair_3d(dst, &map_a, 0, m0, kb, full_leader);
#pragma unroll
          for (int h = 0; h < NB; ++h)
            sk_tma_load_pair_3d(dst + (uint32_t)kbs * (A_BYTES + h * B_BYTES), &map_b, 0, n0 + h * n_step, kb, full_leader);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {  // ---- MMA issuer (leader CTA only)
      int it = 0, si = 0;
      bool ok = true;
      for (; ok && sched.next(tile, kb0, kb1, split); ++si) {
        const int b = si % NBUF;
        const uint32_t acc_ph = (uint32_t)(si / NBUF) & 1u;
        ok = mbar_wait(smem_u32(&bars[18 + b]), acc_ph ^ 1u, err, DEV_ERR_TMEM_WAIT);  // the epilogues have drained buffer b
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * BN);
        for (int kb = kb0; kb < kb1; kb += kbs, ++it) {
          const int s = it % nstages;
          const uint32_t ph = (uint32_t)(it / nstages) & 1u;
          ok = mbar_wait(smem_u32(&bars[s]), ph, err, DEV_ERR_FULL_WAIT);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = base + (uint32_t)s * STAGE, b_addr = a_addr + (uint32_t)kbs * A_BYTES;
          for (int j = 0; j < kbs && kb + j < kb1; ++j) {
            const uint64_t a_desc = smem_desc_sw128(a_addr + (uint32_t)j * A_BYTES);
#pragma unroll
            for (int k = 0; k < SK_BK / 16; ++k) {
#pragma unroll
              for (int h = 0; h < NB; ++h)
                sk_mma_pair(d_tmem + (uint32_t)(h * 256), a_desc + 2 * k, smem_desc_sw128(b_addr + (uint32_t)(h * kbs + j) * B_BYTES) + 2 * k, IDESC,
                            (kb + j > kb0 || k > 0) ? 1u : 0u);
            }
          }
          sk_commit_pair(smem_u32(&bars[8 + s]), 3);  // frees the stage in both CTAs
        }
        sk_commit_pair(smem_u32(&bars[16 + b]), 3);  // the segment's accumulators are complete (also after a failed wait: lets the epilogues leave)
      }
    }
  } else {
    // ---- epilogue (both CTAs): warp w reads TMEM lanes 32 * (w % 4) ... + 31 of its own CTA
    const int quad = warp & 3;
    const uint32_t acc_empty_leader = mapa(smem_u32(&bars[18]), 0);
    const uint32_t part_done_leader = mapa(smem_u32(&bars[20]), 0);
    const int trow = (int)rank * SK_BM + quad * 32 + lane;  // row within the pair's tile
    const uint32_t stg = stg_base + (uint32_t)quad * STG_WARP;
    const uint32_t prev_bar = smem_u32(&bars[21 + quad * 2]);
    uint32_t prev_uses[2] = {0, 0};  // loads of previous values completed on each buffer's barrier
    int si = 0;
    bool go = true;
    for (; go && sched.next(tile, kb0, kb1, split); ++si) {
      const int row = (tile % tiles_m) * (2 * SK_BM) + trow;
      const int n0 = (tile / tiles_m) * BN_OUT;
      const int b = si % NBUF;
      const uint32_t acc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * BN);
      const bool ok = mbar_wait(smem_u32(&bars[16 + b]), (uint32_t)(si / NBUF) & 1u, err, DEV_ERR_TMEM_WAIT);
      tc_fence_after();
      go = __all_sync(0xffffffffu, ok && *(volatile int*)err == 0);
      if (!go) break;
      if (kb0 > 0) {
        // the tail of a tile that another pair owns: fp32 partial sums into this pair's workspace slot
        float* slot = workspace + (size_t)cluster_id * (256 * BN);
        // (rows past the last one are neither written here nor read by the owner: a short prompt hands over m rows, not 256)
#pragma unroll 1
        for (int c = 0; c < BN && row - lane < m; c += 32) {
          uint32_t r[32];
          tc_ld_32x32(acc + (uint32_t)c, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          // float4 number ((piece * 8 + i) * 256 + row): the 32 lanes of a warp store 512 contiguous bytes
          float4* dst = reinterpret_cast<float4*>(slot) + (size_t)(c >> 5) * 8 * 256 + trow;
          if (row < m) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[i * 256] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
          }
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) sk_arrive_cluster(part_done_leader);
        if (rank == 0 && quad == 0 && lane == 0) {  // all eight warps have stored: raise this pair's flag
          if (mbar_wait(smem_u32(&bars[20]), 0, err, DEV_ERR_TMEM_WAIT)) sk_st_release(flags + cluster_id, seq);
        }
      } else {
        // a whole tile, or the head of one: the pairs after this one that ran its later K steps hand their sums over
        int n_peers = 0;
        if (kb1 < nk) {
          n_peers = sched.peers_of(tile);
          bool got = true;
          if (lane == 0)
            for (int q = 0; q < n_peers && got; ++q) got = sk_flag_wait(flags + cluster_id + 1 + q, seq, err);
          got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
          if (!got) n_peers = 0;  // (the error word is set: the result is not used)
        }
        // the first two peers' sums of a piece are requested one piece ahead (an L2 round trip per piece otherwise)
        float4 nxt[2][8];
        auto peer_piece = [&](int q, int piece) {
          return reinterpret_cast<const float4*>(workspace + (size_t)(cluster_id + 1 + q) * (256 * BN)) + (size_t)piece * 8 * 256 + trow;
        };
        auto fetch = [&](int piece) {
#pragma unroll
          for (int q = 0; q < 2; ++q)
            if (q < n_peers) {
              const float4* src = peer_piece(q, piece);
              if (row < m) {
#pragma unroll
                for (int i = 0; i < 8; ++i) nxt[q][i] = __ldcg(src + i * 256);
              }
            }
        };
        const int row0w = row - lane;  // first of this warp's 32 rows
        const bool rows_live = row0w < m;  // a warp whose rows all lie past the last one has nothing to add or store
        if (n_peers > 0 && rows_live) fetch(0);
        if (beta != 0.f && rows_live) {
          if (lane == 0) {
            sk_store_wait_read<0>();
            mbar_arrive_expect_tx(prev_bar, 4096);
            tma_load_2d(stg, &map_out, n0, row0w, prev_bar);
          }
          __syncwarp();
        }
        // GATE: the pieces are visited as (first matrix, second matrix) pairs of the same output columns
        auto piece_of = [](int idx) { return GATE ? (idx >> 1) + (idx & 1) * (BN / 64) : idx; };
        uint32_t first[16];  // GATE: the half-rounded products of the first matrix for the piece in flight
#pragma unroll 1
        for (int idx = 0; idx < BN / 32 && rows_live; ++idx) {
          const int piece = piece_of(idx);
          uint32_t r[32];
          tc_ld_32x32(acc + (uint32_t)(piece * 32), r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          float sum[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) sum[i] = __uint_as_float(r[i]);
          if (n_peers > 0) {  // in pair order: the sum does not depend on who was ready first
            float4 cur[2][8];
#pragma unroll
            for (int q = 0; q < 2; ++q)
#pragma unroll
              for (int i = 0; i < 8; ++i) cur[q][i] = nxt[q][i];
            if (idx + 1 < BN / 32) fetch(piece_of(idx + 1));
#pragma unroll
            for (int q = 0; q < 2; ++q)
              if (q < n_peers) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  sum[4 * i] += cur[q][i].x;
                  sum[4 * i + 1] += cur[q][i].y;
                  sum[4 * i + 2] += cur[q][i].z;
                  sum[4 * i + 3] += cur[q][i].w;
                }
              }
            for (int q = 2; q < n_peers && row < m; ++q) {
              const float4* src = peer_piece(q, piece);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 v = __ldcg(src + i * 256);
                sum[4 * i] += v.x;
                sum[4 * i + 1] += v.y;
                sum[4 * i + 2] += v.z;
                sum[4 * i + 3] += v.w;
              }
            }
          }
          if (GATE && (idx & 1) == 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const __half2 h = __floats2half2_rn(sum[2 * i], sum[2 * i + 1]);
              first[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
            continue;
          }
          uint32_t outw[16];  // the piece's 32 output halves (beta = 0 paths)
          if (GATE) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&first[i]));
              const float2 bq = __half22float2(__floats2half2_rn(sum[2 * i], sum[2 * i + 1]));
              const __half2 gt = __halves2half2(__float2half(silu_of_half(a.x) * bq.x), __float2half(silu_of_half(a.y) * bq.y));
              outw[i] = *reinterpret_cast<const uint32_t*>(&gt);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const __half2 h = __floats2half2_rn(sum[2 * i], sum[2 * i + 1]);
              outw[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
          }
          // results go out through shared memory: the warp's 32 rows x 64 columns are stored by one bulk tensor copy
          // (rows are 44 KB apart in memory; stores of 64 bytes per thread kept the load/store unit busy for longer
          // than the tile's arithmetic left room for)
          const int c = (GATE ? idx >> 1 : idx) * 32;  // output column of the piece within the tile
          const int chunk = c >> 6, buf = chunk & 1;
          const uint32_t sb = stg + (uint32_t)buf * 4096;
          if ((c & 32) == 0) {
            if (!GATE && beta != 0.f) {
              if (lane == 0) {
                sk_store_wait_read<0>();  // the other buffer's last store has read it: it may take the next chunk's previous values
                if (c + 64 < BN_OUT) {
                  mbar_arrive_expect_tx(prev_bar + (uint32_t)(buf ^ 1) * 8, 4096);
                  tma_load_2d(stg + (uint32_t)(buf ^ 1) * 4096, &map_out, n0 + c + 64, row0w, prev_bar + (uint32_t)(buf ^ 1) * 8);
                }
              }
              __syncwarp();
              mbar_wait(prev_bar + (uint32_t)buf * 8, prev_uses[buf] & 1u, err, DEV_ERR_FULL_WAIT);
              ++prev_uses[buf];
            } else {
              if (lane == 0) sk_store_wait_read<1>();  // the store before last, which used this buffer, has read it
              __syncwarp();
            }
          }
          const uint32_t rowb = sb + (uint32_t)lane * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t at = rowb + ((uint32_t)((((c & 32) >> 3) + i) ^ (lane & 7)) << 4);
            uint4 v = make_uint4(outw[4 * i], outw[4 * i + 1], outw[4 * i + 2], outw[4 * i + 3]);
            if (!GATE && beta != 0.f) {
              __half2* h = reinterpret_cast<__half2*>(&v);
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(at) : "memory");
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 prev = __half22float2(h[e]);
                h[e] = __floats2half2_rn(fmaf(beta, prev.x, sum[8 * i + 2 * e]), fmaf(beta, prev.y, sum[8 * i + 2 * e + 1]));
              }
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(at), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
          }
          if (c & 32) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) sk_tma_store_2d(&map_out, n0 + c - 32, row0w, sb);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) sk_arrive_cluster(acc_empty_leader + (uint32_t)(b * 8));
    }
    if (lane == 0) sk_store_wait_all();  // this warp's bulk stores are complete before its shared memory goes away
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

// workspace of partial sums and flags, one per (device, stream): launches on one stream run in order, so a slot is
// free again when the next launch starts; launches on different streams must not share slots
struct sk_workspace {
  float* partials = nullptr;
  int* flags = nullptr;
  size_t partial_floats = 0;
  int n_flags = 0;
  int seq = 0;
};
struct sk_key {
  int dev;
  cudaStream_t stream;
  bool operator==(const sk_key& o) const { return dev == o.dev && stream == o.stream; }
};
struct sk_key_hash {
  size_t operator()(const sk_key& k) const { return (size_t)k.dev * 1000003u ^ (size_t)(uintptr_t)k.stream; }
};

int sk_get_workspace(int dev, cudaStream_t stream, size_t partial_floats, int n_flags, sk_workspace** out) {
  static std::mutex mu;
  static std::unordered_map<sk_key, sk_workspace, sk_key_hash> table;
  std::lock_guard<std::mutex> lock(mu);
  sk_workspace& w = table[sk_key{dev, stream}];
  if (w.partial_floats < partial_floats || w.n_flags < n_flags) {
    // (grows only; the old buffers may still be read by a launch in flight on this stream, so they are released in
    // stream order)
    if (w.partials) LCU_CUDA(cudaFreeAsync(w.partials, stream));
    if (w.flags) LCU_CUDA(cudaFreeAsync(w.flags, stream));
    partial_floats = std::max(partial_floats, w.partial_floats);  // (both only grow, whichever of the two asked for more)
    n_flags = std::max(n_flags, w.n_flags);
    w = sk_workspace{};
    LCU_CUDA(cudaMalloc(&w.partials, partial_floats * sizeof(float)));
    LCU_CUDA(cudaMalloc(&w.flags, (size_t)n_flags * sizeof(int)));
    LCU_CUDA(cudaMemsetAsync(w.flags, 0, (size_t)n_flags * sizeof(int), stream));
    w.partial_floats = partial_floats;
    w.n_flags = n_flags;
  }
  *out = &w;
  return LCU_OK;
}

}  // namespace

int& sk_kb_per_stage() {
  static int kb = 0;
  return kb;
}

namespace {

// GATE: w is the stack [w1; w3] of two [N][K] matrices and out is [m][N]
template <int NB, bool GATE>
int launch_sk(__half* out, const __half* lhs, int ldx, const __half* w, int m, int N, int K, float beta, int* err, cudaStream_t stream) {
  constexpr int BN = 256 * NB;
  constexpr int BN_OUT = GATE ? BN / 2 : BN;
  CUtensorMap map_a, map_b;
  int kbs = sk_kb_per_stage();  // k-blocks per stage and tensor copy
  if (kbs <= 0) kbs = 2;
  if (kbs > 2 || K / SK_BK < 2) kbs = 1;
  {
    const uint64_t dims[3] = {(uint64_t)SK_BK, (uint64_t)m, (uint64_t)(K / SK_BK)}, strides[2] = {(uint64_t)ldx * 2, (uint64_t)SK_BK * 2};
    const uint32_t box[3] = {(uint32_t)SK_BK, (uint32_t)SK_BM, (uint32_t)kbs};
    int rc = tc_encode_map(&map_a, lhs, 3, dims, strides, box);
    if (rc) return rc;
  }
  {
    const uint64_t dims[3] = {(uint64_t)SK_BK, (uint64_t)(GATE ? 2 * N : N), (uint64_t)(K / SK_BK)}, strides[2] = {(uint64_t)K * 2, (uint64_t)SK_BK * 2};
    const uint32_t box[3] = {(uint32_t)SK_BK, 128u, (uint32_t)kbs};
    int rc = tc_encode_map(&map_b, w, 3, dims, strides, box, true);
    if (rc) return rc;
  }
  CUtensorMap map_out;
  {
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)m}, strides[1] = {(uint64_t)N * 2};
    const uint32_t box[2] = {64u, 32u};
    int rc = tc_encode_map(&map_out, out, 2, dims, strides, box);
    if (rc) return rc;
  }
  const size_t STAGE = (size_t)kbs * (SK_BM + NB * 128) * SK_BK * 2;
  int nstages = (int)((192 * 1024) / STAGE);
  if (nstages > 8) nstages = 8;
  const size_t smem = nstages * STAGE + 32768 /* output staging */ + 1024 /* alignment slack */ + 256 /* barriers, tmem slot */;
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(gemm_tc_sk_kernel<NB, GATE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_done[dev] = true;
  }
  const int tiles_m = (m + 2 * SK_BM - 1) / (2 * SK_BM), n_tiles = tiles_m * (N / BN_OUT);
  int clusters = gemv_sm_count() / 2;
  if (clusters > n_tiles) clusters = n_tiles < 1 ? 1 : std::min<long long>(clusters, (long long)n_tiles * (K / SK_BK));
  sk_workspace* ws = nullptr;
  int rc = sk_get_workspace(dev, stream, (size_t)clusters * 256 * BN, clusters, &ws);
  if (rc) return rc;
  const int seq = ++ws->seq;
  LCU_CUDA(launch_after(gemm_tc_sk_kernel<NB, GATE>, dim3(2 * clusters), dim3(SK_THREADS), smem, stream, map_a, map_b, map_out, m, N, K, beta, nstages,
                        tiles_m, n_tiles, ws->partials, ws->flags, seq, err, GATE ? N : 0, kbs));
  return LCU_OK;
}

}  // namespace

bool gemm_tc_sk_supported(int m, int N, int K, int ldx, const void* lhs, const void* w, const void* out, int tile_n) {
  return (tile_n == 256 || tile_n == 512) && m >= 1 && N % tile_n == 0 && K % SK_BK == 0 && ldx % 8 == 0 && ((uintptr_t)lhs & 15) == 0 &&
         ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0;
}

int launch_gemm_tc_sk(__half* out, const __half* lhs, int ldx, const __half* w, int m, int N, int K, float beta, int* err, cudaStream_t stream,
                      int tile_n) {
  LCU_REQUIRE(gemm_tc_sk_supported(m, N, K, ldx, lhs, w, out, tile_n), "gemm_tc_sk: unsupported shape m=%d N=%d K=%d ldx=%d tile %d", m, N, K, ldx,
              tile_n);
  return tile_n == 512 ? launch_sk<2, false>(out, lhs, ldx, w, m, N, K, beta, err, stream) : launch_sk<1, false>(out, lhs, ldx, w, m, N, K, beta, err, stream);
}

bool gemm_tc_gated_supported(int m, int f, int K, int ldx, const void* lhs, const void* w, const void* out) {
  return m >= 1 && f % 128 == 0 && K % SK_BK == 0 && ldx % 8 == 0 && ((uintptr_t)lhs & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0;
}

int launch_gemm_tc_gated(__half* out, const __half* lhs, int ldx, const __half* w13, int m, int f, int K, int* err, cudaStream_t stream, int tile_n) {
  LCU_REQUIRE(gemm_tc_gated_supported(m, f, K, ldx, lhs, w13, out) && (tile_n == 256 || (tile_n == 512 && f % 256 == 0)),
              "gemm_tc_gated: unsupported shape m=%d f=%d K=%d ldx=%d tile=%d", m, f, K, ldx, tile_n);
  return tile_n == 512 ? launch_sk<2, true>(out, lhs, ldx, w13, m, f, K, 0.f, err, stream) : launch_sk<1, true>(out, lhs, ldx, w13, m, f, K, 0.f, err, stream);
}

// The schedule, walked on the host for every pair of a launch: 0 when every K step of every tile is run exactly once,
// a pair starts inside a tile (and so hands partial sums over) at most once and only with its first shared segment, and
// the pair that ran a shared tile's first K step finds exactly the pairs after it that ran the rest, in order.
int gemm_tc_sk_check_schedule(int n_tiles, int nk, int C) {
  if (n_tiles < 1 || nk < 1 || C < 1) return -1;
  std::vector<int> owner((size_t)n_tiles * nk, -1);
  struct seg { int tile, kb0, kb1; };
  std::vector<std::vector<seg>> segs(C);
  for (int c = 0; c < C; ++c) {
    sk_schedule sc;
    sc.init(n_tiles, nk, C, c);
    int tile, kb0, kb1, writer_segments = 0, shared_segments = 0;
    bool split;
    while (sc.next(tile, kb0, kb1, split)) {
      if (tile < 0 || tile >= n_tiles || kb0 < 0 || kb1 > nk || kb0 >= kb1) return 1;
      if (split) ++shared_segments;
      if (kb0 > 0) {
        if (!split || shared_segments != 1) return 2;  // only a pair's first shared segment may start inside a tile
        ++writer_segments;
      }
      for (int kb = kb0; kb < kb1; ++kb) {
        if (owner[(size_t)tile * nk + kb] != -1) return 3;
        owner[(size_t)tile * nk + kb] = c;
      }
      segs[c].push_back({tile, kb0, kb1});
    }
    if (writer_segments > 1) return 4;
    if (c < sc.Cs && shared_segments == 0) return 5;  // every pair counted for the shared tiles has a K step of them
  }
  for (int v : owner)
    if (v < 0) return 6;
  for (int c = 0; c < C; ++c)
    for (const seg& sg : segs[c]) {
      if (sg.kb0 != 0) continue;
      sk_schedule sc;
      sc.init(n_tiles, nk, C, c);
      if (sg.kb1 == nk) continue;  // ran the whole tile
      if (sg.tile < sc.first_split_tile) return 7;
      const int peers = sc.peers_of(sg.tile);
      if (peers < 1 || c + peers >= C) return 8;
      int at = sg.kb1;
      for (int q = 1; q <= peers; ++q) {  // the next pairs continue the tile, one after the other
        if (segs[c + q].empty()) return 9;
        const seg& first_shared = *std::find_if(segs[c + q].begin(), segs[c + q].end(), [&](const seg& x) { return x.tile == sg.tile; });
        if (first_shared.tile != sg.tile || first_shared.kb0 != at) return 10;
        at = first_shared.kb1;
      }
      if (at != nk) return 11;
    }
  return 0;
}

}  // namespace lcu
