// Prompt attention in one kernel on tcgen05: scores, softmax and probabilities x V of the reference's three-step chain
// (matmul_qk -> softmax_rows -> matmul_qkv, llama_cu.cu:400-531) without the [heads][rows][keys] score buffer.
//
// The reference's rounding points need a row's maximum and exp-sum before any probability is formed:
//   s_t = half((q . k_t) / sqrtf(head_dim)),  p_t = half(e^(s_t - max) / sum),  out_j = half(sum_t float(p_t) float(v_tj))
// so the kernel makes two passes over the key tiles of a (128-row tile, head) and computes the scores twice - the
// contraction over head_dim is cheap next to writing and re-reading 2 bytes per score:
//   pass 1  S = Q K_j^T into tensor memory; the epilogue warps round the scores to half and keep a running maximum and
//           exp-sum per row (the sum is rescaled when the maximum moves);
//   pass 2  S again; the epilogue warps form the half-rounded probabilities and store them into shared memory as a
//           K-major operand tile; a second tcgen05.mma multiplies that tile with V_j (read as it lies in the cache: an
//           MN-major operand) into the output accumulator, which stays in tensor memory over all key tiles.
// Warp roles: warp 0 issues the TMA loads (Q once, then K tiles, in pass 2 K and V tiles alternately, through one ring),
// warp 1 issues the MMAs, warps 2-9 are the epilogue (a thread owns one row and 64 of a tile's 128 keys).  Two score
// accumulators and two probability tiles let the exponentials of one key tile run under the MMAs of its neighbours.
// Key tiles above the causal diagonal are not visited.  Every mbarrier wait is bounded.
#include <algorithm>

#include "attention.cuh"
#include "tc_common.cuh"

namespace lcu {

int& attn_fused_order() {
  static int v = 1;  // measured: 2000 rows, 7B: 135 -> 104 us per layer against 0 (the heavy tiles of the last heads end the kernel)
  return v;
}

namespace {

constexpr int FA_BM = 128;       // query rows per CTA
constexpr int FA_BN = 128;       // keys per tile
constexpr int FA_EPI_WARPS = 16;  // four per tensor-memory lane quadrant: a thread owns one row and 32 of a tile's 128 keys
constexpr int FA_THREADS = 64 + 32 * FA_EPI_WARPS;  // warp 0: TMA, warp 1: MMA + tensor memory, then the epilogue warps
constexpr int FA_RING = 4;       // ring stages of one 128-key operand each
constexpr uint32_t FA_P_BYTES = FA_BM * FA_BN * 2;  // one probability tile: two K-major blocks of 128 rows x 64 keys

struct fused_params {
  __half* out;  // [m][ldo]
  int ldo;
  const int* pos;  // device scalar: position of query row 0 (nullptr: pos_value)
  int pos_value;
  int m;
  int* err;
};

// barrier indices
constexpr int B_Q = 0;                       // Q landed
constexpr int B_FULL = 1;                    // [FA_RING] ring stage landed
constexpr int B_EMPTY = B_FULL + FA_RING;    // [FA_RING] ring stage free
constexpr int B_S_FULL = B_EMPTY + FA_RING;  // [2] score accumulator ready
constexpr int B_S_EMPTY = B_S_FULL + 2;      // [2] score accumulator read out (8 warps)
constexpr int B_P_READY = B_S_EMPTY + 2;     // [2] probability tile written (8 warps)
constexpr int B_P_FREE = B_P_READY + 2;      // [2] probability tile consumed by its MMAs
constexpr int B_O_FULL = B_P_FREE + 2;       // output accumulator complete
constexpr int B_COUNT = B_O_FULL + 1;

__device__ __forceinline__ float2 fa_unpack(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2*>(&w)); }
constexpr uint16_t FA_MASKED = 0xfbff;  // -65504: a key above the diagonal (its exponential is 0 for every row maximum)

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1) attn_fused_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                                                   const __grid_constant__ CUtensorMap map_v, const fused_params p, int t_tiles, int m_tiles,
                                                                   int head_fastest) {
  constexpr int NKB = HD / 64;                       // 64-wide blocks of the head dimension
  constexpr uint32_t BLOCK_BYTES = 128 * 64 * 2;     // 128 rows (or keys) x 64 dims
  constexpr uint32_t OPERAND = NKB * BLOCK_BYTES;    // Q tile, K tile, or V tile (2 x NKB atoms of 64 keys x 64 dims)
  constexpr uint32_t V_ATOM = 64 * 64 * 2;
  constexpr uint32_t IDESC_QK = (1u << 4) | ((uint32_t)(FA_BN >> 3) << 17) | ((uint32_t)(FA_BM >> 4) << 24);
  // A K-major, B MN-major (bit 16), N = HD, M = 128
  constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(FA_BM >> 4) << 24);
  constexpr uint32_t TMEM_COLS = 512;                // S[2]: columns 0..255, O: columns 256..256+HD
  constexpr uint32_t O_COL = 256;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_addr = base, ring_addr = base + OPERAND, p_addr = ring_addr + FA_RING * OPERAND;
  // [128 rows][2 halves][max, sum], handed over between the passes: in the second probability tile, which is first
  // written after every thread has read its row's pair
  float* stats = reinterpret_cast<float*>(smem + OPERAND + FA_RING * OPERAND + FA_P_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OPERAND + FA_RING * OPERAND + 2 * FA_P_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // long row tiles first: over all heads (head_fastest: the kernel then ends with every head's short tiles), or within
  // each head
  const int n_heads_grid = (int)gridDim.x / m_tiles;
  const int mt = head_fastest ? (int)blockIdx.x / n_heads_grid : (int)blockIdx.x % m_tiles;
  const int head = head_fastest ? (int)blockIdx.x % n_heads_grid : (int)blockIdx.x / m_tiles;
  const int m0 = (m_tiles - 1 - mt) * FA_BM;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars[B_Q]), 1);
    for (int i = 0; i < FA_RING; ++i) {
      mbar_init(smem_u32(&bars[B_FULL + i]), 1);
      mbar_init(smem_u32(&bars[B_EMPTY + i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars[B_S_FULL + i]), 1);
      mbar_init(smem_u32(&bars[B_S_EMPTY + i]), FA_EPI_WARPS);
      mbar_init(smem_u32(&bars[B_P_READY + i]), FA_EPI_WARPS);
      mbar_init(smem_u32(&bars[B_P_FREE + i]), 1);
    }
    mbar_init(smem_u32(&bars[B_O_FULL]), 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();  // (the position word and the operands are read after this line)
  const int pos0 = p.pos ? *p.pos : p.pos_value;
  const int n_tiles = min(t_tiles, (pos0 + m0 + FA_BM + FA_BN - 1) / FA_BN);       // key tiles that hold a visible key

  if (warp == 0) {
    if (lane == 0) {
      // ---- loads: Q; pass 1: K_0 .. K_{n-1}; pass 2: K_0, V_0, K_1, V_1, ...  (item i lives in ring stage i % FA_RING)
      mbar_arrive_expect_tx(smem_u32(&bars[B_Q]), OPERAND);
      for (int kb = 0; kb < NKB; ++kb) tma_load_3d(q_addr + kb * BLOCK_BYTES, &map_q, kb * 64, head, m0, smem_u32(&bars[B_Q]));
      const int items = 3 * n_tiles;
      for (int it = 0; it < items; ++it) {
        const int s = it % FA_RING, use = it / FA_RING;
        if (use > 0 && !mbar_wait(smem_u32(&bars[B_EMPTY + s]), (use - 1) & 1, p.err, DEV_ERR_EMPTY_WAIT)) break;
        const uint32_t full = smem_u32(&bars[B_FULL + s]);
        const uint32_t dst = ring_addr + (uint32_t)s * OPERAND;
        mbar_arrive_expect_tx(full, OPERAND);
        const bool is_v = it >= n_tiles && ((it - n_tiles) & 1);
        const int j = it < n_tiles ? it : (it - n_tiles) >> 1;
        if (!is_v) {
          for (int kb = 0; kb < NKB; ++kb) tma_load_3d(dst + kb * BLOCK_BYTES, &map_k, kb * 64, j * FA_BN, head, full);  // [128 keys][64 dims]
        } else {
          for (int kb2 = 0; kb2 < 2; ++kb2)
            for (int a = 0; a < NKB; ++a)
              tma_load_3d(dst + (kb2 * NKB + a) * V_ATOM, &map_v, a * 64, j * FA_BN + kb2 * 64, head, full);  // [64 keys][64 dims]
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMAs.  sidx counts score tiles over both passes: tile sidx uses accumulator sidx & 1.
      bool ok = mbar_wait(smem_u32(&bars[B_Q]), 0, p.err, DEV_ERR_FULL_WAIT);
      int sidx = 0;
      auto scores = [&](int item) {  // S[sidx & 1] = Q K^T with the K tile of ring item `item`
        const int s = item % FA_RING, b = sidx & 1;
        ok = ok && mbar_wait(smem_u32(&bars[B_S_EMPTY + b]), ((uint32_t)(sidx >> 1) & 1u) ^ 1u, p.err, DEV_ERR_TMEM_WAIT);
        ok = ok && mbar_wait(smem_u32(&bars[B_FULL + s]), (uint32_t)(item / FA_RING) & 1u, p.err, DEV_ERR_FULL_WAIT);
        if (!ok) return;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < NKB; ++kb) {
          const uint64_t a_desc = smem_desc_sw128(q_addr + kb * BLOCK_BYTES), b_desc = smem_desc_sw128(ring_addr + (uint32_t)s * OPERAND + kb * BLOCK_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma_f16(tmem_base + (uint32_t)(b * FA_BN), a_desc + 2 * k, b_desc + 2 * k, IDESC_QK, (kb | k) != 0);
        }
        tc_commit(smem_u32(&bars[B_EMPTY + s]));
        tc_commit(smem_u32(&bars[B_S_FULL + b]));
        ++sidx;
      };
      for (int j = 0; j < n_tiles && ok; ++j) scores(j);  // pass 1
      if (ok) scores(n_tiles);                            // pass 2, tile 0
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) scores(n_tiles + 2 * (j + 1));
        const int item = n_tiles + 2 * j + 1, s = item % FA_RING, pb = j & 1;
        ok = ok && mbar_wait(smem_u32(&bars[B_P_READY + pb]), (uint32_t)(j >> 1) & 1u, p.err, DEV_ERR_FULL_WAIT);
        ok = ok && mbar_wait(smem_u32(&bars[B_FULL + s]), (uint32_t)(item / FA_RING) & 1u, p.err, DEV_ERR_FULL_WAIT);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kb2 = 0; kb2 < 2; ++kb2) {
          const uint64_t a_desc = smem_desc_sw128(p_addr + (uint32_t)pb * FA_P_BYTES + kb2 * BLOCK_BYTES);
          const uint64_t b_desc = smem_desc_sw128_mn(ring_addr + (uint32_t)s * OPERAND + kb2 * NKB * V_ATOM, V_ATOM);
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 16 keys per instruction: 32 bytes along P's rows, two 8-key groups (2 x 1024 bytes) of V
            tc_mma_f16(tmem_base + O_COL, a_desc + 2 * k, b_desc + (uint64_t)(k * 2048 >> 4), IDESC_PV, (j | kb2 | k) != 0);
        }
        tc_commit(smem_u32(&bars[B_EMPTY + s]));
        tc_commit(smem_u32(&bars[B_P_FREE + pb]));
      }
      tc_commit(smem_u32(&bars[B_O_FULL]));  // (also after a failed wait: lets the epilogue warps leave)
      if (!ok) {
        tc_commit(smem_u32(&bars[B_S_FULL]));
        tc_commit(smem_u32(&bars[B_S_FULL + 1]));
      }
    }
  } else {
    // ---- epilogue: a thread owns row `row` of the tile and the 32 keys [cq * 32, +32) of every key tile.  (With eight
    // warps of 64 keys per thread the kernel was bound by the latency of its own instruction chain: 186 us per 7B layer
    // at 2000 rows, what the three kernels it replaces took together.)
    const int quad = warp & 3, cq = (warp - 2) >> 2;
    const int row = quad * 32 + lane, grow = m0 + row;
    const int last_key = pos0 + grow;  // the row sees keys 0 .. last_key
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    // x / sqrt(head_dim) as one multiplication and a residual correction: RN(x / d) in all but vanishingly rare
    // double-rounding cases (the result is rounded to half right after)
    const float scale_div = sqrtf((float)HD), scale_rcp = __frcp_rn(scale_div);
    auto scaled = [&](uint32_t bits) {
      const float x = __uint_as_float(bits), q = x * scale_rcp;
      return fmaf(fmaf(-q, scale_div, x), scale_rcp, q);
    };
    auto ex2 = [](float y) {
      float r;
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(y));
      return r;
    };
    constexpr float LOG2E = 1.4426950408889634f;
    int sidx = 0;
    bool go = true;
    // the scores of this thread's 32 keys of tile j, rounded to half (masked keys: -inf), as 16 half2 words
    auto load_scores = [&](int j, uint32_t (&h)[16]) {
      const int b = sidx & 1;
      const bool ok = mbar_wait(smem_u32(&bars[B_S_FULL + b]), (uint32_t)(sidx >> 1) & 1u, p.err, DEV_ERR_TMEM_WAIT);
      tc_fence_after();
      go = __all_sync(0xffffffffu, ok && *(volatile int*)p.err == 0);
      if (!go) return;
      const int key0 = j * FA_BN + cq * 32;
      uint32_t r[32];
      tc_ld_32x32(lane_base + (uint32_t)(b * FA_BN + cq * 32), r);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (key0 + 31 <= pos0 + m0 + quad * 32) {  // every key of the piece is visible to every row of this warp
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const __half2 v = __floats2half2_rn(scaled(r[2 * i]), scaled(r[2 * i + 1]));
          h[i] = *reinterpret_cast<const uint32_t*>(&v);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          __half2 v = __floats2half2_rn(scaled(r[2 * i]), scaled(r[2 * i + 1]));
          const int k = key0 + 2 * i;
          if (k + 1 > last_key) {
            const __half gone = __ushort_as_half(FA_MASKED);
            v = __halves2half2(k > last_key ? gone : __low2half(v), gone);
          }
          h[i] = *reinterpret_cast<const uint32_t*>(&v);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[B_S_EMPTY + b]));  // the accumulator may take the next tile
      ++sidx;
    };

    // ---- pass 1: running maximum and exp-sum of the row's half-rounded scores
    float mx = -CUDART_INF_F, sum = 0.f;
    for (int j = 0; j < n_tiles && go; ++j) {
      uint32_t h[16];
      load_scores(j, h);
      if (!go) break;
      __half2 hm = *reinterpret_cast<const __half2*>(&h[0]);
#pragma unroll
      for (int i = 1; i < 16; ++i) hm = __hmax2(hm, *reinterpret_cast<const __half2*>(&h[i]));
      const float2 hmf = fa_unpack(*reinterpret_cast<const uint32_t*>(&hm));
      const float tmax = fmaxf(hmf.x, hmf.y);
      if (tmax > mx) {
        sum *= ex2((mx - tmax) * LOG2E);  // (mx = -inf at the first tile: the factor is 0 and so is the sum)
        mx = tmax;
      }
      const float off = -mx * LOG2E;
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 f = fa_unpack(h[i]);
        s0 += ex2(fmaf(f.x, LOG2E, off));
        s1 += ex2(fmaf(f.y, LOG2E, off));
      }
      sum += s0 + s1;
    }
    // the four threads of a row put their parts together (left to right)
    stats[(row * 4 + cq) * 2] = mx;
    stats[(row * 4 + cq) * 2 + 1] = sum;
    bar_sync(1, 32 * FA_EPI_WARPS);
    {
      float part_m[4], part_s[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        part_m[q] = stats[(row * 4 + q) * 2];
        part_s[q] = stats[(row * 4 + q) * 2 + 1];
      }
      mx = fmaxf(fmaxf(part_m[0], part_m[1]), fmaxf(part_m[2], part_m[3]));  // (finite: the first part holds key 0)
      sum = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q)
        sum += part_s[q] * ex2((part_m[q] - mx) * LOG2E);  // (a part with every key above the diagonal: factor 0)
    }
    bar_sync(1, 32 * FA_EPI_WARPS);  // (the pairs lie where pass 2 writes probabilities)
    const float rsum = __frcp_rn(sum);
    // e / sum as one multiplication and a residual correction (RN(e / sum) in all but vanishingly rare cases)
    const float off2 = -mx * LOG2E;
    auto prob = [&](float x) {
      const float e = ex2(fmaf(x, LOG2E, off2)), q = e * rsum;
      return fmaf(fmaf(-q, sum, e), rsum, q);
    };

    // ---- pass 2: probabilities rounded to half into the K-major operand tile (128-byte swizzled rows of 64 keys)
    for (int j = 0; j < n_tiles && go; ++j) {
      uint32_t h[16];
      load_scores(j, h);
      if (!go) break;
      const int pb = j & 1;
      const bool ok = mbar_wait(smem_u32(&bars[B_P_FREE + pb]), ((uint32_t)(j >> 1) & 1u) ^ 1u, p.err, DEV_ERR_TMEM_WAIT);  // the MMAs of tile j - 2 have read it
      go = __all_sync(0xffffffffu, ok);
      if (!go) break;
      const uint32_t prow = p_addr + (uint32_t)pb * FA_P_BYTES + (uint32_t)(cq >> 1) * BLOCK_BYTES + (uint32_t)row * 128;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const int cidx = (cq & 1) * 4 + c4;
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = fa_unpack(h[c4 * 4 + e]);
          const __half2 pr = __floats2half2_rn(prob(f.x), prob(f.y));
          o[e] = *reinterpret_cast<const uint32_t*>(&pr);
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + (uint32_t)((cidx ^ (row & 7)) << 4)), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                     "r"(o[3])
                     : "memory");
      }
      fence_proxy_async();  // the tile is read by the tensor core (async proxy)
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[B_P_READY + pb]));
    }

    // ---- output: half(sum_t p_t v_tj); the row's first HD / 32 threads store 32 columns each
    {
      const bool ok = mbar_wait(smem_u32(&bars[B_O_FULL]), 0, p.err, DEV_ERR_TMEM_WAIT);
      tc_fence_after();
      if (__all_sync(0xffffffffu, ok && go && *(volatile int*)p.err == 0)) {
        if (cq * 32 < HD) {
          const int c = cq * 32;
          uint32_t r[32];
          tc_ld_32x32(lane_base + O_COL + (uint32_t)c, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (grow < p.m) {
            __align__(16) __half2 hv[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) hv[i] = __floats2half2_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
            __half* o = p.out + (size_t)grow * p.ldo + head * HD + c;
#pragma unroll
            for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(o)[i] = reinterpret_cast<const uint4*>(hv)[i];
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <int HD>
int launch_fused_hd(const attn_params& p, int m, int max_T, cudaStream_t stream) {
  CUtensorMap map_q, map_k, map_v;
  const uint64_t H = (uint64_t)p.n_heads, ctx = (uint64_t)p.ctx_len;
  {
    // q rows [m][ldq], head h at column h * HD: dims (HD, heads, rows)
    const uint64_t dims[3] = {(uint64_t)HD, H, (uint64_t)m}, strides[2] = {(uint64_t)HD * 2, (uint64_t)p.ldq * 2};
    const uint32_t box[3] = {64, 1, 128};
    int rc = tc_encode_map(&map_q, p.q, 3, dims, strides, box);
    if (rc) return rc;
  }
  {
    // caches [heads][ctx][HD]: dims (HD, positions, heads)
    const uint64_t dims[3] = {(uint64_t)HD, ctx, H}, strides[2] = {(uint64_t)HD * 2, ctx * HD * 2};
    const uint32_t box_k[3] = {64, 128, 1}, box_v[3] = {64, 64, 1};
    int rc = tc_encode_map(&map_k, p.k_cache, 3, dims, strides, box_k);
    if (rc) return rc;
    rc = tc_encode_map(&map_v, p.v_cache, 3, dims, strides, box_v);
    if (rc) return rc;
  }
  fused_params q{};
  q.out = p.out; q.ldo = p.ldo; q.pos = p.pos; q.pos_value = p.pos_value; q.m = m; q.err = p.err;
  constexpr size_t OPERAND = (size_t)(HD / 64) * 128 * 64 * 2;
  constexpr size_t SMEM = (1 + FA_RING) * OPERAND + 2 * FA_P_BYTES + 256 /* barriers, tensor-memory slot */ + 1024 /* alignment slack */;
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(attn_fused_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    attr_done[dev] = true;
  }
  const int m_tiles = (m + FA_BM - 1) / FA_BM, t_tiles = (max_T + FA_BN - 1) / FA_BN;
  LCU_CUDA(launch_after(attn_fused_kernel<HD>, dim3(m_tiles * p.n_heads), dim3(FA_THREADS), SMEM, stream, map_q, map_k, map_v, q, t_tiles, m_tiles,
                        attn_fused_order()));
  return LCU_OK;
}

}  // namespace

int launch_attention_fused(const attn_params& p, int m, int max_T, cudaStream_t stream) {
  LCU_REQUIRE(m >= 1 && p.n_heads >= 1, "attention: no rows");
  LCU_REQUIRE(max_T >= 1 && max_T <= p.ctx_len, "attention: %d positions exceed the context length %d", max_T, p.ctx_len);
  LCU_REQUIRE(p.err != nullptr, "attention: the tensor-core path needs an error word");
  LCU_REQUIRE(p.ldq % 8 == 0 && p.ldo % 8 == 0 && ((uintptr_t)p.q & 15) == 0 && ((uintptr_t)p.out & 15) == 0, "attention: rows must be 16-byte aligned");
  if (p.head_dim == 128) return launch_fused_hd<128>(p, m, max_T, stream);
  if (p.head_dim == 64) return launch_fused_hd<64>(p, m, max_T, stream);
  LCU_REQUIRE(false, "attention: head_dim %d not supported (64 or 128)", p.head_dim);
}

}  // namespace lcu
