// Prompt attention on tcgen05: the reference's three-step chain (matmul_qk -> softmax_rows -> matmul_qkv,
// llama_cu.cu:400-531) with both contractions on the 5th-generation tensor cores.
//
//   1. attn_qk_kernel   S[h][r][t] = half( (q_r . k_t) / sqrtf(head_dim) )    128 x 128 tiles, K = head_dim, key tiles
//                       above the causal diagonal are not visited; Q and K tiles arrive by 3-D TMA (heads are one coordinate)
//   2. attn_softmax_kernel  P = softmax over t <= pos0 + r of every row, in place (one warp per row, the row held in
//                       registers); columns after the row's last key up to the end of its row tile's key range are
//                       zeroed so that step 3 can multiply whole key blocks
//   3. attn_pv_kernel   out[r][h*hd + j] = half( sum_t float(P[h][r][t]) float(v[t][j]) )   A = P (K-major, from the
//                       score buffer), B = V read as it lies in the cache ([t][j]: an MN-major operand), K loop over the
//                       64-key blocks up to the row tile's causal limit
//
// The score / probability buffer [heads][rows][keys] lives in HBM as in the reference (fp16, written once, read twice);
// the rounding points are the reference's.  Every mbarrier wait is bounded.
#include <algorithm>

#include "attention.cuh"
#include "tc_common.cuh"

namespace lcu {
namespace {

constexpr int AT_BM = 128;   // query rows per tile
constexpr int AT_BN = 128;   // keys per score tile
constexpr int AT_THREADS = 192;  // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue

struct attn_tc_params {
  __half* scores;     // [heads][m_cap][t_cap]
  __half* out;        // [m][ldo]
  int ldo;
  const int* pos;     // device scalar: position of query row 0 (nullptr: pos_value)
  int pos_value;
  int m, m_cap, t_cap, n_heads;
  int* err;
};

// ------------------------------------------------------------------------------------------------ 1. scores
// One CTA per (128-row tile, head), persistent over the key tiles up to the tile's causal limit: Q is loaded once,
// K tiles stream through a ring, two accumulators in tensor memory let the epilogue of one key tile (8 warps: scale,
// round to half, store) run under the loads and MMAs of the next.
constexpr int QK_THREADS = 320;  // warp 0: TMA, warp 1: MMA + TMEM, warps 2-9: epilogue
constexpr int QK_STAGES = 3;

template <int HD>
__global__ void __launch_bounds__(QK_THREADS, 1) attn_qk_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                                                const attn_tc_params p, int t_tiles) {
  constexpr int NKB = HD / 64;  // 64-wide k-blocks of the head dimension
  constexpr uint32_t TILE_BYTES = 128 * 64 * 2;
  constexpr uint32_t OPERAND = NKB * TILE_BYTES;  // one 128 x HD operand
  constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(AT_BN >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  // [0] Q landed, [1..3] K stage landed, [4..6] K stage free, [7..8] accumulator ready, [9..10] accumulator drained
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (1 + QK_STAGES) * OPERAND);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * AT_BM, head = blockIdx.y;  // long row tiles first
  const int pos0 = p.pos ? *p.pos : p.pos_value;
  const int n_tiles = min(t_tiles, (pos0 + m0 + AT_BM + AT_BN - 1) / AT_BN);       // key tiles that hold a visible key

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars[0]), 1);
    for (int i = 0; i < QK_STAGES; ++i) {
      mbar_init(smem_u32(&bars[1 + i]), 1);
      mbar_init(smem_u32(&bars[4 + i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars[7 + i]), 1);
      mbar_init(smem_u32(&bars[9 + i]), 8);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(2 * AT_BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(smem_u32(&bars[0]), OPERAND);
      for (int kb = 0; kb < NKB; ++kb) tma_load_3d(base + kb * TILE_BYTES, &map_q, kb * 64, head, m0, smem_u32(&bars[0]));  // [128 rows][64] of this head
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % QK_STAGES, use = j / QK_STAGES;
        if (use > 0 && !mbar_wait(smem_u32(&bars[4 + s]), (use - 1) & 1, p.err, DEV_ERR_EMPTY_WAIT)) break;
        const uint32_t full = smem_u32(&bars[1 + s]);
        mbar_arrive_expect_tx(full, OPERAND);
        for (int kb = 0; kb < NKB; ++kb) tma_load_3d(base + (1 + s) * OPERAND + kb * TILE_BYTES, &map_k, kb * 64, j * AT_BN, head, full);  // [128 keys][64]
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(smem_u32(&bars[0]), 0, p.err, DEV_ERR_FULL_WAIT);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % QK_STAGES, b = j & 1;
        ok = mbar_wait(smem_u32(&bars[9 + b]), ((uint32_t)(j >> 1) & 1u) ^ 1u, p.err, DEV_ERR_TMEM_WAIT);  // accumulator b drained
        ok = ok && mbar_wait(smem_u32(&bars[1 + s]), (uint32_t)(j / QK_STAGES) & 1u, p.err, DEV_ERR_FULL_WAIT);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < NKB; ++kb) {
          const uint64_t a_desc = smem_desc_sw128(base + kb * TILE_BYTES), b_desc = smem_desc_sw128(base + (1 + s) * OPERAND + kb * TILE_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma_f16(tmem_base + (uint32_t)(b * AT_BN), a_desc + 2 * k, b_desc + 2 * k, IDESC, (kb | k) != 0);
        }
        tc_commit(smem_u32(&bars[4 + s]));
        tc_commit(smem_u32(&bars[7 + b]));
      }
      if (!ok) {  // let the epilogue warps leave
        tc_commit(smem_u32(&bars[7]));
        tc_commit(smem_u32(&bars[8]));
      }
    }
  } else {
    const int quad = warp & 3, chalf = (warp - 2) >> 2;  // TMEM lane quadrant of this warp; it takes 64 of the 128 columns
    const int row = m0 + quad * 32 + lane;
    // x / sqrt(head_dim) as one multiplication and a residual correction: RN(x / d) in all but vanishingly rare
    // double-rounding cases (the result is rounded to half right after), a third of the division's instructions
    const float scale_div = sqrtf((float)HD), scale_rcp = __frcp_rn(scale_div);
    auto scaled = [&](uint32_t bits) {
      const float x = __uint_as_float(bits), q = x * scale_rcp;
      return fmaf(fmaf(-q, scale_div, x), scale_rcp, q);
    };
    bool go = true;
    for (int j = 0; j < n_tiles && go; ++j) {
      const int b = j & 1;
      const bool ok = mbar_wait(smem_u32(&bars[7 + b]), (uint32_t)(j >> 1) & 1u, p.err, DEV_ERR_TMEM_WAIT);
      tc_fence_after();
      go = __all_sync(0xffffffffu, ok && *(volatile int*)p.err == 0);
      if (!go) break;
      __half* srow = p.scores + ((size_t)head * p.m_cap + row) * p.t_cap + j * AT_BN;
#pragma unroll 1
      for (int c = chalf * 64; c < chalf * 64 + 64; c += 32) {
        uint32_t r[32];
        tc_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(b * AT_BN + c), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < p.m) {
          __align__(16) __half2 h[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) h[i] = __floats2half2_rn(scaled(r[2 * i]), scaled(r[2 * i + 1]));
#pragma unroll
          for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(srow + c)[i] = reinterpret_cast<const uint4*>(h)[i];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[9 + b]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * AT_BN)) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ 2. softmax
// One warp per (row, head): the row (up to SM_VEC x 256 keys) is read once into registers as 16-byte vectors, the
// maximum and the exp-sum are warp reductions, the probabilities are written back in place.  Arithmetic of the
// reference's softmax_rows (llama_cu.cu:433-499) with temperature 1 over the row's causal prefix: max, e^(x - max),
// sum, e^(x - max) / sum rounded to half; the sum is taken in a different order than its 256-thread tree.
constexpr int SM_VEC_MAX = 16;  // vectors of 8 keys per lane: rows of up to 4096 keys
// SM_VEC (4, 8 or 16) is picked from the longest row of the call: fewer registers, more rows in flight per SM
template <int SM_VEC>
__global__ void __launch_bounds__(256) attn_softmax_kernel(const attn_tc_params p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + warp, head = blockIdx.y;
  if (r >= p.m) return;
  const int pos0 = p.pos ? *p.pos : p.pos_value;
  const int L = pos0 + r + 1;                                                     // keys this row sees
  const int m0 = (r / AT_BM) * AT_BM;
  const int k_end = min(p.t_cap, ((pos0 + m0 + AT_BM + 63) / 64) * 64);           // key range step 3 walks for this row tile
  __half* row = p.scores + ((size_t)head * p.m_cap + r) * p.t_cap;
  uint4 v[SM_VEC];
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int j = 0; j < SM_VEC; ++j) {
    const int i0 = (j * 32 + lane) * 8;
    v[j] = make_uint4(0, 0, 0, 0);
    if (i0 < L) v[j] = *reinterpret_cast<const uint4*>(row + i0);
  }
  // The one vector that holds the row's last key gets its tail overwritten with -inf (maximum ignores it, 2^(-inf) = 0,
  // probability 0), so that every pass below works on whole vectors without per-element checks.
  {
    const int jb = (L - 1) >> 8, lb = ((L - 1) >> 3) & 31, keep = ((L - 1) & 7) + 1;
    if (lane == lb && keep < 8) {
#pragma unroll
      for (int j = 0; j < SM_VEC; ++j)
        if (j == jb) {
          __half* h = reinterpret_cast<__half*>(&v[j]);
#pragma unroll
          for (int e = 1; e < 8; ++e)
            if (e >= keep) h[e] = __ushort_as_half(0xfc00);
        }
    }
  }
#pragma unroll
  for (int j = 0; j < SM_VEC; ++j) {
    const int i0 = (j * 32 + lane) * 8;
    if (i0 < L) {
      const __half2* h2 = reinterpret_cast<const __half2*>(&v[j]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h2[e]);
        mx = fmaxf(mx, fmaxf(f.x, f.y));
      }
    }
  }
  mx = warp_max(mx);
  // e^(x - max) as 2^((x - max) log2 e): one multiplication and the hardware exponential (2 ulp) instead of expf's
  // longer sequence (1 ulp); every element is exponentiated twice here, so this is what bounds the kernel
  auto ex = [&](float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"((x - mx) * 1.4426950408889634f));
    return y;
  };
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int j = 0; j < SM_VEC; ++j) {
    const int i0 = (j * 32 + lane) * 8;
    if (i0 < L) {
      const __half2* h2 = reinterpret_cast<const __half2*>(&v[j]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h2[e]);
        sum0 += ex(f.x);
        sum1 += ex(f.y);
      }
    }
  }
  const float sum = warp_sum(sum0 + sum1);
  const float rsum = __frcp_rn(sum);
  // e / sum as one multiplication and a residual correction (RN(e / sum) in all but vanishingly rare cases)
  auto prob = [&](float x) {
    const float e = ex(x), q = e * rsum;
    return fmaf(fmaf(-q, sum, e), rsum, q);
  };
#pragma unroll
  for (int j = 0; j < SM_VEC; ++j) {
    const int i0 = (j * 32 + lane) * 8;
    if (i0 >= k_end) continue;  // probabilities, then zeros from the row's last key to the end of the row tile's key range
    __align__(16) __half2 o[4];
    if (i0 < L) {
      const __half2* h2 = reinterpret_cast<const __half2*>(&v[j]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h2[e]);
        o[e] = __floats2half2_rn(prob(f.x), prob(f.y));
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = __floats2half2_rn(0.f, 0.f);
    }
    *reinterpret_cast<uint4*>(row + i0) = *reinterpret_cast<const uint4*>(o);
  }
}

// ------------------------------------------------------------------------------------------------ 3. P . V
template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 1) attn_pv_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_v,
                                                                const attn_tc_params p, int nstages) {
  constexpr int ND = HD / 64;                       // 64-wide blocks of the head dimension (the operand's N atoms)
  constexpr uint32_t A_BYTES = AT_BM * 64 * 2;      // P: 128 rows x 64 keys
  constexpr uint32_t V_ATOM = 64 * 64 * 2;          // V: 64 keys x 64 dims
  constexpr uint32_t STAGE = A_BYTES + ND * V_ATOM;
  // fp32 accumulate, fp16 operands, A K-major, B MN-major (bit 16), N = HD, M = 128
  constexpr uint32_t IDESC = (1u << 4) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)nstages * STAGE);  // full[8], empty[8], accumulator ready
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * AT_BM, head = blockIdx.y;
  const int pos0 = p.pos ? *p.pos : p.pos_value;
  const int nk = min(p.t_cap, ((pos0 + m0 + AT_BM + 63) / 64) * 64) / 64;  // 64-key blocks up to this row tile's causal limit

  if (threadIdx.x == 0) {
    for (int i = 0; i < nstages; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);
      mbar_init(smem_u32(&bars[8 + i]), 1);
    }
    mbar_init(smem_u32(&bars[16]), 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(HD < 32 ? 32 : HD)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < nk; ++kb) {
        const int s = kb % nstages, use = kb / nstages;
        if (use > 0 && !mbar_wait(smem_u32(&bars[8 + s]), (use - 1) & 1, p.err, DEV_ERR_EMPTY_WAIT)) break;
        const uint32_t full = smem_u32(&bars[s]);
        const uint32_t dst = base + (uint32_t)s * STAGE;
        mbar_arrive_expect_tx(full, STAGE);
        tma_load_3d(dst, &map_p, kb * 64, m0, head, full);  // probabilities [128 rows][64 keys]
        for (int j = 0; j < ND; ++j) tma_load_3d(dst + A_BYTES + j * V_ATOM, &map_v, j * 64, kb * 64, head, full);  // V [64 keys][64 dims]
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < nk && ok; ++kb) {
        const int s = kb % nstages, use = kb / nstages;
        ok = mbar_wait(smem_u32(&bars[s]), use & 1, p.err, DEV_ERR_FULL_WAIT);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = base + (uint32_t)s * STAGE;
        const uint64_t a_desc = smem_desc_sw128(a_addr);
        const uint64_t b_desc = smem_desc_sw128_mn(a_addr + A_BYTES, V_ATOM);
#pragma unroll
        for (int k = 0; k < 4; ++k)  // 16 keys per instruction: 32 bytes along A's rows, two 8-key groups (2 x 1024 bytes) of V
          tc_mma_f16(tmem_base, a_desc + 2 * k, b_desc + (uint64_t)(k * 2048 >> 4), IDESC, (kb | k) != 0);
        tc_commit(smem_u32(&bars[8 + s]));
      }
      tc_commit(smem_u32(&bars[16]));
    }
  } else {
    const int quad = warp & 3;
    const int row = m0 + quad * 32 + lane;
    const bool ok = mbar_wait(smem_u32(&bars[16]), 0, p.err, DEV_ERR_TMEM_WAIT);
    tc_fence_after();
    if (__all_sync(0xffffffffu, ok && *(volatile int*)p.err == 0)) {
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        uint32_t r[32];
        tc_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < p.m) {
          __align__(16) __half2 h[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) h[i] = __floats2half2_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
          __half* o = p.out + (size_t)row * p.ldo + head * HD + c;
#pragma unroll
          for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(o)[i] = reinterpret_cast<const uint4*>(h)[i];
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(HD < 32 ? 32 : HD)) : "memory");
  }
}

template <int HD>
int launch_tc_hd(const attn_params& p, int m, int max_T, __half* scores, int m_cap, int t_cap, cudaStream_t stream) {
  CUtensorMap map_q, map_k, map_p, map_v;
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
  {
    // scores / probabilities [heads][m_cap][t_cap]: dims (keys, rows, heads)
    const uint64_t dims[3] = {(uint64_t)t_cap, (uint64_t)m_cap, H}, strides[2] = {(uint64_t)t_cap * 2, (uint64_t)m_cap * t_cap * 2};
    const uint32_t box[3] = {64, 128, 1};
    int rc = tc_encode_map(&map_p, scores, 3, dims, strides, box);
    if (rc) return rc;
  }
  attn_tc_params q{};
  q.scores = scores; q.out = p.out; q.ldo = p.ldo; q.pos = p.pos; q.pos_value = p.pos_value;
  q.m = m; q.m_cap = m_cap; q.t_cap = t_cap; q.n_heads = p.n_heads; q.err = p.err;
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  constexpr size_t QK_SMEM = (size_t)(1 + QK_STAGES) * (HD / 64) * 128 * 64 * 2 + 1024 + 128;
  constexpr size_t PV_STAGE = 128 * 64 * 2 + (HD / 64) * 64 * 64 * 2;
  const int nstages = 6;
  const size_t pv_smem = nstages * PV_STAGE + 1024 + 256;
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(attn_qk_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)QK_SMEM));
    LCU_CUDA(cudaFuncSetAttribute(attn_pv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pv_smem));
    attr_done[dev] = true;
  }
  const int m_tiles = (m + AT_BM - 1) / AT_BM, t_tiles = (max_T + AT_BN - 1) / AT_BN;
  attn_qk_kernel<HD><<<dim3(m_tiles, p.n_heads), QK_THREADS, QK_SMEM, stream>>>(map_q, map_k, q, t_tiles);
  LCU_CUDA(cudaGetLastError());
  const int k_max = std::min(t_cap, (max_T + 63) / 64 * 64);  // longest key range a row's probabilities cover
  if (k_max <= 4 * 256)
    attn_softmax_kernel<4><<<dim3((m + 7) / 8, p.n_heads), 256, 0, stream>>>(q);
  else if (k_max <= 8 * 256)
    attn_softmax_kernel<8><<<dim3((m + 7) / 8, p.n_heads), 256, 0, stream>>>(q);
  else
    attn_softmax_kernel<16><<<dim3((m + 7) / 8, p.n_heads), 256, 0, stream>>>(q);
  LCU_CUDA(cudaGetLastError());
  attn_pv_kernel<HD><<<dim3(m_tiles, p.n_heads), AT_THREADS, pv_smem, stream>>>(map_p, map_v, q, nstages);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

}  // namespace

size_t attention_tc_scratch_halves(int n_heads, int m_cap, int ctx_len) {
  const size_t t_cap = ((size_t)ctx_len + 127) / 128 * 128;
  return (size_t)n_heads * m_cap * t_cap;
}

int launch_attention_tc(const attn_params& p, int m, int max_T, __half* scores, int m_cap, cudaStream_t stream) {
  LCU_REQUIRE(m >= 1 && m <= m_cap && p.n_heads >= 1, "attention: %d rows do not fit the score buffer (%d)", m, m_cap);
  LCU_REQUIRE(max_T >= 1 && max_T <= p.ctx_len, "attention: %d positions exceed the context length %d", max_T, p.ctx_len);
  LCU_REQUIRE(p.ctx_len <= SM_VEC_MAX * 256, "attention: the tensor-core path holds rows of up to %d keys", SM_VEC_MAX * 256);
  LCU_REQUIRE(p.err != nullptr && scores != nullptr, "attention: the tensor-core path needs an error word and a score buffer");
  LCU_REQUIRE(p.ldq % 8 == 0 && p.ldo % 8 == 0 && ((uintptr_t)p.q & 15) == 0 && ((uintptr_t)p.out & 15) == 0, "attention: rows must be 16-byte aligned");
  const int t_cap = (p.ctx_len + 127) / 128 * 128;
  if (p.head_dim == 128) return launch_tc_hd<128>(p, m, max_T, scores, m_cap, t_cap, stream);
  if (p.head_dim == 64) return launch_tc_hd<64>(p, m, max_T, scores, m_cap, t_cap, stream);
  LCU_REQUIRE(false, "attention: head_dim %d not supported (64 or 128)", p.head_dim);
}

}  // namespace lcu
