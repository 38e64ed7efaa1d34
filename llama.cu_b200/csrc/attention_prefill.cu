// Prompt attention: many query rows against the fp16 KV cache, causal.
//
// Replaces the reference's matmul_qk -> softmax_rows -> matmul_qkv chain (llama_cu.cu:400-531, called at
// 1161-1171) for m > 1 rows.  The reference's rounding points are kept, as in the decode kernel:
//   score  s_t = half( (sum_i q_i k_ti) / sqrtf(head_dim) )
//   prob   p_t = half( expf(s_t - max) / sum_t' expf(s_t' - max) )
//   out    o_j = half( sum_t float(p_t) float(v_tj) )
// The probabilities need the row's final max and sum, so the kernel goes over the keys twice: pass 1 forms the
// score tiles and keeps a running (max, sum) per row, pass 2 forms the same score tiles again, turns them into
// half probabilities and multiplies them with V.  Scores never leave the SM (the reference writes an
// [heads][m][T] tensor per layer).
//
// One CTA = 64 query rows of one head, 4 warps x 16 rows.  Tiles of 64 keys are staged in shared memory with
// cp.async (double-buffered; rows past the last needed key are zero-filled), Q fragments stay in registers, the
// products run on warp-level m16n8k16 tensor-core instructions with fp32 accumulation; the score accumulators of
// a 16 x 16 block are exactly the A fragment of the P.V product, so P never goes through memory.
#include "attention.cuh"

namespace lcu {
namespace {

constexpr int PA_QM = 64;       // query rows per CTA
constexpr int PA_KT = 64;       // keys per tile
constexpr int PA_THREADS = 128;

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// x / d from r = RN(1 / d): one multiplication and one residual correction.  This is the core of the correctly
// rounded division sequence without its special-case handling (operands here are finite, d >= 1): it returns
// RN(x / d) in all but vanishingly rare double-rounding cases, at a third of the instructions.
__device__ __forceinline__ float div_by(float x, float d, float r) {
  const float q = x * r;
  return fmaf(fmaf(-q, d, x), r, q);
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int HD>
__global__ void __launch_bounds__(PA_THREADS) attn_prefill_kernel(const attn_params p, int m) {
  constexpr int LDS = HD + 8;             // padded row (halves): conflict-free fragment loads
  constexpr int TILE = PA_KT * LDS;       // halves per staged K or V tile
  constexpr int CPR = HD / 8;             // 16-byte chunks per row
  extern __shared__ __align__(16) __half pa_smem[];  // [2 stages][K tile | V tile]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int head = blockIdx.y, q0 = blockIdx.x * PA_QM;
  const int start_pos = p.pos ? *p.pos : p.pos_value;
  const int rows_here = min(PA_QM, m - q0);
  const int nkeys = start_pos + q0 + rows_here;  // the last row of this CTA sees keys 0 .. nkeys - 1
  const int ntiles = (nkeys + PA_KT - 1) / PA_KT;
  const __half* kb = p.k_cache + (size_t)head * p.ctx_len * HD;
  const __half* vb = p.v_cache + (size_t)head * p.ctx_len * HD;
  const float scale_div = sqrtf((float)HD), scale_rcp = __frcp_rn(scale_div);

  // Q fragments (A operand, 16 rows x HD per warp): rows g and g + 8 of the warp's block
  const int r_lo = q0 + warp * 16 + g, r_hi = r_lo + 8;
  uint32_t qa[HD / 16][4];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    const int d = ks * 16 + 2 * c;
    const __half* ql = p.q + (size_t)r_lo * p.ldq + head * HD + d;
    const __half* qh = p.q + (size_t)r_hi * p.ldq + head * HD + d;
    qa[ks][0] = r_lo < m ? *reinterpret_cast<const uint32_t*>(ql) : 0u;
    qa[ks][1] = r_hi < m ? *reinterpret_cast<const uint32_t*>(qh) : 0u;
    qa[ks][2] = r_lo < m ? *reinterpret_cast<const uint32_t*>(ql + 8) : 0u;
    qa[ks][3] = r_hi < m ? *reinterpret_cast<const uint32_t*>(qh + 8) : 0u;
  }
  const int last_lo = start_pos + r_lo, last_hi = start_pos + r_hi;  // last key each row may see
  const int warp_last = start_pos + q0 + warp * 16 + 15;

  auto stage_tile = [&](int tile, int stage, bool with_v) {
    __half* ks = pa_smem + (size_t)stage * 2 * TILE;
    __half* vs = ks + TILE;
    const int t0 = tile * PA_KT;
    for (int i = tid; i < PA_KT * CPR; i += PA_THREADS) {
      const int r = i / CPR, ch = i % CPR;
      const bool valid = t0 + r < nkeys;
      const size_t off = (size_t)(valid ? t0 + r : 0) * HD + ch * 8;
      cp_async16_zfill(smem_u32(ks + r * LDS + ch * 8), kb + off, valid);
      if (with_v) cp_async16_zfill(smem_u32(vs + r * LDS + ch * 8), vb + off, valid);
    }
    cp_async_commit();
  };

  // scores of one 16 x 64 block: s[j][0..1] = row g, keys 8j + 2c, +1; s[j][2..3] = row g + 8; masked keys = -inf
  auto score_tile = [&](const __half* ks, int t0, float (&s)[8][4]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk += 2) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // four 8x8 blocks of keys 8j .. 8j+7: d = 16kk, 16kk + 8, 16kk + 16, 16kk + 24
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(smem_u32(ks + (j * 8 + (lane & 7)) * LDS + kk * 16 + (lane >> 3) * 8), b0, b1, b2, b3);
        mma_16816(s[j], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
        mma_16816(s[j], qa[kk + 1][0], qa[kk + 1][1], qa[kk + 1][2], qa[kk + 1][3], b2, b3);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int t = t0 + j * 8 + 2 * c;
      s[j][0] = t <= last_lo ? __half2float(__float2half(div_by(s[j][0], scale_div, scale_rcp))) : -CUDART_INF_F;
      s[j][1] = t + 1 <= last_lo ? __half2float(__float2half(div_by(s[j][1], scale_div, scale_rcp))) : -CUDART_INF_F;
      s[j][2] = t <= last_hi ? __half2float(__float2half(div_by(s[j][2], scale_div, scale_rcp))) : -CUDART_INF_F;
      s[j][3] = t + 1 <= last_hi ? __half2float(__float2half(div_by(s[j][3], scale_div, scale_rcp))) : -CUDART_INF_F;
    }
  };

  // ---- pass 1: running maximum and exp-sum of every row
  float mx_lo = -CUDART_INF_F, mx_hi = -CUDART_INF_F, sum_lo = 0.f, sum_hi = 0.f;
  stage_tile(0, 0, false);
  for (int tile = 0; tile < ntiles; ++tile) {
    if (tile + 1 < ntiles) {
      stage_tile(tile + 1, (tile + 1) & 1, false);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (tile * PA_KT > warp_last) {  // every key of the tile lies in the future of all 16 rows of this warp
      __syncthreads();
      continue;
    }
    float s[8][4];
    score_tile(pa_smem + (size_t)(tile & 1) * 2 * TILE, tile * PA_KT, s);
    float tm_lo = -CUDART_INF_F, tm_hi = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      tm_lo = fmaxf(tm_lo, fmaxf(s[j][0], s[j][1]));
      tm_hi = fmaxf(tm_hi, fmaxf(s[j][2], s[j][3]));
    }
    tm_lo = fmaxf(tm_lo, __shfl_xor_sync(0xffffffffu, tm_lo, 1));
    tm_lo = fmaxf(tm_lo, __shfl_xor_sync(0xffffffffu, tm_lo, 2));
    tm_hi = fmaxf(tm_hi, __shfl_xor_sync(0xffffffffu, tm_hi, 1));
    tm_hi = fmaxf(tm_hi, __shfl_xor_sync(0xffffffffu, tm_hi, 2));
    const float nm_lo = fmaxf(mx_lo, tm_lo), nm_hi = fmaxf(mx_hi, tm_hi);
    float ts_lo = 0.f, ts_hi = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // expf(-inf - x) = 0 for masked keys; a fully masked row keeps sum 0
      if (nm_lo > -CUDART_INF_F) ts_lo += expf(s[j][0] - nm_lo) + expf(s[j][1] - nm_lo);
      if (nm_hi > -CUDART_INF_F) ts_hi += expf(s[j][2] - nm_hi) + expf(s[j][3] - nm_hi);
    }
    ts_lo += __shfl_xor_sync(0xffffffffu, ts_lo, 1);
    ts_lo += __shfl_xor_sync(0xffffffffu, ts_lo, 2);
    ts_hi += __shfl_xor_sync(0xffffffffu, ts_hi, 1);
    ts_hi += __shfl_xor_sync(0xffffffffu, ts_hi, 2);
    sum_lo = (mx_lo > -CUDART_INF_F ? sum_lo * expf(mx_lo - nm_lo) : 0.f) + ts_lo;
    sum_hi = (mx_hi > -CUDART_INF_F ? sum_hi * expf(mx_hi - nm_hi) : 0.f) + ts_hi;
    mx_lo = nm_lo;
    mx_hi = nm_hi;
    __syncthreads();  // the stage is overwritten two tiles later
  }

  // ---- pass 2: probabilities (half) times V
  const float rs_lo = __frcp_rn(sum_lo), rs_hi = __frcp_rn(sum_hi);
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  stage_tile(0, 0, true);
  for (int tile = 0; tile < ntiles; ++tile) {
    if (tile + 1 < ntiles) {
      stage_tile(tile + 1, (tile + 1) & 1, true);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (tile * PA_KT > warp_last) {
      __syncthreads();
      continue;
    }
    const __half* ks = pa_smem + (size_t)(tile & 1) * 2 * TILE;
    const __half* vs = ks + TILE;
    float s[8][4];
    score_tile(ks, tile * PA_KT, s);
    // probabilities of rows that see nothing in this tile are expf(-inf) = 0
    uint32_t pa[4][4];  // A fragments of the 16 x 64 probability block, 16 keys each
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      pa[kk][0] = pack_half2(div_by(expf(s[2 * kk][0] - mx_lo), sum_lo, rs_lo), div_by(expf(s[2 * kk][1] - mx_lo), sum_lo, rs_lo));
      pa[kk][1] = pack_half2(div_by(expf(s[2 * kk][2] - mx_hi), sum_hi, rs_hi), div_by(expf(s[2 * kk][3] - mx_hi), sum_hi, rs_hi));
      pa[kk][2] = pack_half2(div_by(expf(s[2 * kk + 1][0] - mx_lo), sum_lo, rs_lo), div_by(expf(s[2 * kk + 1][1] - mx_lo), sum_lo, rs_lo));
      pa[kk][3] = pack_half2(div_by(expf(s[2 * kk + 1][2] - mx_hi), sum_hi, rs_hi), div_by(expf(s[2 * kk + 1][3] - mx_hi), sum_hi, rs_hi));
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int dj = 0; dj < HD / 16; ++dj) {
        // transposed 8x8 loads: matrices (keys 16kk.., d 16dj..), (keys +8, same d), (keys, d + 8), (keys + 8, d + 8)
        const int mrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int mcol = dj * 16 + (lane >> 4) * 8;
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(smem_u32(vs + mrow * LDS + mcol), b0, b1, b2, b3);
        mma_16816(o[2 * dj], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
        mma_16816(o[2 * dj + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) {
    const int d = head * HD + j * 8 + 2 * c;
    if (r_lo < m) *reinterpret_cast<uint32_t*>(p.out + (size_t)r_lo * p.ldo + d) = pack_half2(o[j][0], o[j][1]);
    if (r_hi < m) *reinterpret_cast<uint32_t*>(p.out + (size_t)r_hi * p.ldo + d) = pack_half2(o[j][2], o[j][3]);
  }
}

template <int HD>
int launch_prefill_hd(const attn_params& p, int m, cudaStream_t stream) {
  const size_t smem = (size_t)2 * 2 * PA_KT * (HD + 8) * sizeof(__half);
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done[dev] = true;
  }
  attn_prefill_kernel<HD><<<dim3((m + PA_QM - 1) / PA_QM, p.n_heads), PA_THREADS, smem, stream>>>(p, m);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

}  // namespace

int launch_attention_prefill(const attn_params& p, int m, int max_T, cudaStream_t stream) {
  LCU_REQUIRE(m >= 1 && p.n_heads >= 1, "attention: empty problem");
  LCU_REQUIRE(max_T >= 1 && max_T <= p.ctx_len, "attention: %d positions exceed the context length %d", max_T, p.ctx_len);
  LCU_REQUIRE(p.ldq % 2 == 0 && p.ldo % 2 == 0, "attention: row strides must be even");
  if (p.head_dim == 128) return launch_prefill_hd<128>(p, m, stream);
  if (p.head_dim == 64) return launch_prefill_hd<64>(p, m, stream);
  LCU_REQUIRE(false, "attention: head_dim %d not supported (64 or 128)", p.head_dim);
}

}  // namespace lcu
