// Single-row (batch-1) weight-streaming GEMV: every consumer warp is an independent streaming
// dot-product engine with a private shared-memory ring; no block-wide synchronisation in the loop.
//
// Measured on B200 with this library's read probe (bench_read_ceiling): a 16 KiB ring stage
// fetched as sixteen 1 KiB bulk copies tops out near 4.4 TB/s with one CTA per SM, while copies
// of 4 KiB or more reach the read ceiling of ~7.2 TB/s.  So a stage here is TWO bulk copies: one
// contiguous 4 KiB chunk (2048 fp16 / 4096 u8 weights) from each row of a row pair, and the chunk
// is mapped onto the tensor-core tile like this:
//
//   m16n8k16 tile row  m = 8*rr + seg : segment `seg` (1/8 of the chunk, 512 B) of row `rr` of the pair
//   tile column        n = seg        : the activation values of that same segment
//
// D[m][n] is wanted only on the "diagonal" n == seg(m): lane (g, c = g/2) ends up with the partial
// dot products of segment g for both rows.  All 16 tile rows still consume distinct weight bytes.
// Odd segments walk their 64-byte steps in swapped order (step ^ 1) on both operands, so the eight
// lanes of a quarter warp hit eight distinct 16-byte bank groups without padding the staged rows.
//
// A row pair (the unit RoPE and the SiLU gate need) belongs to ONE warp from its first chunk to its
// epilogue: the warp waits on its own mbarriers, accumulates in registers, reduces with shuffles and
// writes the result.  The producer warp deals chunks to the warps' rings round-robin.  As in the
// multi-row kernel (gemv.cu) the producer does not depend on the activations, so under programmatic
// dependent launch the rings of kernel n+1 fill while kernel n drains; every wait is bounded; int8
// weights are de-quantised in registers bit-identically to half((q - 127.5f) * scale)
// (reference llama_cu.cu:287-289); the RMSNorm prologue keeps the reference's summation order.
#include "gemv.cuh"

namespace lcu {
namespace {

// Consumer warps per CTA (template parameter of the kernel): 4, or 5 for u8 kernels whose activation row leaves room
// for two CTAs per SM only - ten consumer warps per SM instead of eight, the u8 kernels being latency-bound.
constexpr int NW_MAX = 5;
// Stage geometry per weight type: 4 KiB of each row per stage (measured: 2 KiB stages in a ring twice as deep lose a
// third of the u8 throughput - the per-stage cost of the producer counts).
template <int WT>
struct geom {
  static constexpr int ROWB = 4096;                    // bytes of one row per stage (one bulk copy)
  static constexpr int SEG = ROWB / 8;                 // the chunk is cut into 8 segments, one per tile column
  static constexpr int NSTEPS = SEG / 64;              // 64-byte steps per segment
  static constexpr int SC_ROW = WT == 2 ? ROWB / 64 * 2 : 256;  // scale bytes reserved per row per stage (block size >= 64 / >= 32)
  static constexpr int SEG_SHIFT = 9;                  // log2(SEG)
};
constexpr int MAX_SW = 4;                   // ring depth per warp
constexpr int NACC = 4;                     // independent accumulator sets (no chain on one result)
constexpr int EMPTY_BASE = NW_MAX * MAX_SW;  // barriers: full[w * MAX_SW + s], empty[EMPTY_BASE + w * MAX_SW + s]
constexpr int BAR_BYTES = 2 * EMPTY_BASE * 8;
constexpr int SMEM_FIXED = BAR_BYTES + 64;  // barriers; scratch of the RMSNorm reduction

template <int EPI>
__device__ __forceinline__ void map_row(const gemv_params& p, int vrow, int& mat, int& row) {
  if (EPI == EPI_SILU) {
    mat = vrow & 1;
    row = vrow >> 1;
  } else if (EPI == EPI_ROPE_KV) {  // three matrices: two comparisons instead of a division
    mat = (vrow >= p.rows_per_mat) + (vrow >= 2 * p.rows_per_mat);
    row = vrow - mat * p.rows_per_mat;
  } else {
    mat = 0;
    row = vrow;
  }
}

__device__ __forceinline__ uint32_t dequant_pair(uint32_t word, uint32_t selector, __half2 scale2) {
  uint32_t v = __byte_perm(word, 0x64646464u, selector);  // bytes -> halves 1024 + q
  __half2 h = *reinterpret_cast<__half2*>(&v);
  h = __hsub2(h, __half2half2(__ushort_as_half(0x6400)));  // - 1024   (exact)
  h = __hsub2(h, __half2half2(__ushort_as_half(0x57f8)));  // - 127.5  (exact)
  h = __hmul2(h, scale2);                                  // one rounding, as the reference
  return *reinterpret_cast<uint32_t*>(&h);
}

// One 64-byte step of every segment: 16 tile rows x 32 (fp16) or 64 (u8) weights per lane group.
template <int WT, bool FULL>
__device__ __forceinline__ void step(float (&accs)[NACC][4], const int s, const int flip, const int c, const int g, const int vb,
                                     const uint8_t* seg0, const uint8_t* xseg, const uint8_t* st, const float* xs64, const int ci,
                                     const int bs) {
  constexpr int ESZ = WT == 0 ? 2 : 1;
  constexpr int ROWB = geom<WT>::ROWB, SEG = geom<WT>::SEG, NSTEPS = geom<WT>::NSTEPS;
  constexpr int CHUNK_K = ROWB / ESZ;
  float* acc = accs[(2 * s) % NACC];
  float* acc_b = accs[(2 * s + 1) % NACC];
  const int off = ((s ^ flip) << 6) + c * 16;  // byte offset inside the segment
  const bool ok = FULL || off < vb;
  uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
  if (ok) {
    lo = *reinterpret_cast<const uint4*>(seg0 + off);
    hi = *reinterpret_cast<const uint4*>(seg0 + ROWB + off);
  }
  if (WT == 0) {
    uint4 xb = make_uint4(0, 0, 0, 0);
    if (ok) xb = *reinterpret_cast<const uint4*>(xseg + off);
    mma_16816(acc, lo.x, hi.x, lo.y, hi.y, xb.x, xb.y);
    mma_16816(acc_b, lo.z, hi.z, lo.w, hi.w, xb.z, xb.w);
  } else {
    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
    __half sc_lo = __ushort_as_half(0), sc_hi = sc_lo;
    float corr = 0.f;
    if (ok) {
      x0 = *reinterpret_cast<const uint4*>(xseg + 2 * off);
      x1 = *reinterpret_cast<const uint4*>(xseg + 2 * off + 16);
      const __half* scs = reinterpret_cast<const __half*>(st + 2 * ROWB);
      const int si = (g * SEG + off) >> bs;  // k offset inside the chunk / block size (bs is log2 of it here)
      sc_lo = scs[si];
      sc_hi = scs[geom<WT>::SC_ROW / 2 + si];
      // WT 2: sum of x over this lane's segment and step (the diagonal column of the tile)
      if (WT == 2) corr = 1151.5f * xs64[ci * (CHUNK_K / 64) + g * NSTEPS + (s ^ flip)];
    }
    if (WT == 2) {
      float ta[4] = {0.f, 0.f, 0.f, 0.f}, tb[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t M = 0x64646464u;  // bytes -> halves 1024 + q
      mma_16816(ta, __byte_perm(lo.x, M, 0x4140), __byte_perm(hi.x, M, 0x4140), __byte_perm(lo.x, M, 0x4342), __byte_perm(hi.x, M, 0x4342), x0.x, x0.y);
      mma_16816(tb, __byte_perm(lo.y, M, 0x4140), __byte_perm(hi.y, M, 0x4140), __byte_perm(lo.y, M, 0x4342), __byte_perm(hi.y, M, 0x4342), x0.z, x0.w);
      mma_16816(ta, __byte_perm(lo.z, M, 0x4140), __byte_perm(hi.z, M, 0x4140), __byte_perm(lo.z, M, 0x4342), __byte_perm(hi.z, M, 0x4342), x1.x, x1.y);
      mma_16816(tb, __byte_perm(lo.w, M, 0x4140), __byte_perm(hi.w, M, 0x4140), __byte_perm(lo.w, M, 0x4342), __byte_perm(hi.w, M, 0x4342), x1.z, x1.w);
      // only the diagonal entries (column == this lane's segment) are meaningful, and they share `corr`
      const float sl = __half2float(sc_lo), sh = __half2float(sc_hi);
      acc[0] += sl * ((ta[0] + tb[0]) - corr);
      acc[1] += sl * ((ta[1] + tb[1]) - corr);
      acc[2] += sh * ((ta[2] + tb[2]) - corr);
      acc[3] += sh * ((ta[3] + tb[3]) - corr);
    } else {
      const __half2 s_lo = __half2half2(sc_lo), s_hi = __half2half2(sc_hi);
      mma_16816(acc, dequant_pair(lo.x, 0x4140, s_lo), dequant_pair(hi.x, 0x4140, s_hi), dequant_pair(lo.x, 0x4342, s_lo),
                dequant_pair(hi.x, 0x4342, s_hi), x0.x, x0.y);
      mma_16816(acc_b, dequant_pair(lo.y, 0x4140, s_lo), dequant_pair(hi.y, 0x4140, s_hi), dequant_pair(lo.y, 0x4342, s_lo),
                dequant_pair(hi.y, 0x4342, s_hi), x0.z, x0.w);
      mma_16816(acc, dequant_pair(lo.z, 0x4140, s_lo), dequant_pair(hi.z, 0x4140, s_hi), dequant_pair(lo.z, 0x4342, s_lo),
                dequant_pair(hi.z, 0x4342, s_hi), x1.x, x1.y);
      mma_16816(acc_b, dequant_pair(lo.w, 0x4140, s_lo), dequant_pair(hi.w, 0x4140, s_hi), dequant_pair(lo.w, 0x4342, s_lo),
                dequant_pair(hi.w, 0x4342, s_hi), x1.z, x1.w);
    }
  }
}

// Factored u8, block size >= 128: the two 64-byte steps of a 128-weight block share their scale, so the eight
// tensor-core products of both steps are summed before the one multiplication by the scale.
template <bool FULL>
__device__ __forceinline__ void step_pair_factored(float (&accs)[NACC][4], const int sp, const int flip, const int c, const int g, const int vb,
                                                   const uint8_t* seg0, const uint8_t* xseg, const uint8_t* st, const float* xs64, const int ci,
                                                   const int bs) {
  constexpr int ROWB = geom<2>::ROWB, SEG = geom<2>::SEG, NSTEPS = geom<2>::NSTEPS;
  constexpr int CHUNK_K = ROWB;
  float* acc = accs[sp % NACC];
  const uint32_t M = 0x64646464u;  // bytes -> halves 1024 + q
  // a row's last chunk may be short; its length is a multiple of the block size, so a 128-byte pair is valid or not as a whole
  const bool ok = FULL || (sp << 7) < vb;
  // the correction term is the start value of one accumulator chain: sum - 1151.5 * sum(x) costs no instruction of its own
  float negcorr = 0.f;
  if (ok) {
    const float2 xs2 = *reinterpret_cast<const float2*>(xs64 + ci * (CHUNK_K / 64) + g * NSTEPS + 2 * sp);
    negcorr = -1151.5f * (xs2.x + xs2.y);
  }
  float ta[4], tb[4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int off = (((2 * sp + h) ^ flip) << 6) + c * 16;  // odd segments take the two steps in swapped order (bank spread)
    uint4 lo = make_uint4(0, 0, 0, 0), hi = lo, x0 = lo, x1 = lo;
    if (ok) {
      lo = *reinterpret_cast<const uint4*>(seg0 + off);
      hi = *reinterpret_cast<const uint4*>(seg0 + ROWB + off);
      x0 = *reinterpret_cast<const uint4*>(xseg + 2 * off);
      x1 = *reinterpret_cast<const uint4*>(xseg + 2 * off + 16);
    }
    if (h == 0) {  // the block's first products start the two chains
      mma_16816_from(ta, __byte_perm(lo.x, M, 0x4140), __byte_perm(hi.x, M, 0x4140), __byte_perm(lo.x, M, 0x4342), __byte_perm(hi.x, M, 0x4342), x0.x, x0.y, negcorr);
      mma_16816_from(tb, __byte_perm(lo.y, M, 0x4140), __byte_perm(hi.y, M, 0x4140), __byte_perm(lo.y, M, 0x4342), __byte_perm(hi.y, M, 0x4342), x0.z, x0.w, 0.f);
    } else {
      mma_16816(ta, __byte_perm(lo.x, M, 0x4140), __byte_perm(hi.x, M, 0x4140), __byte_perm(lo.x, M, 0x4342), __byte_perm(hi.x, M, 0x4342), x0.x, x0.y);
      mma_16816(tb, __byte_perm(lo.y, M, 0x4140), __byte_perm(hi.y, M, 0x4140), __byte_perm(lo.y, M, 0x4342), __byte_perm(hi.y, M, 0x4342), x0.z, x0.w);
    }
    mma_16816(ta, __byte_perm(lo.z, M, 0x4140), __byte_perm(hi.z, M, 0x4140), __byte_perm(lo.z, M, 0x4342), __byte_perm(hi.z, M, 0x4342), x1.x, x1.y);
    mma_16816(tb, __byte_perm(lo.w, M, 0x4140), __byte_perm(hi.w, M, 0x4140), __byte_perm(lo.w, M, 0x4342), __byte_perm(hi.w, M, 0x4342), x1.z, x1.w);
  }
  if (!ok) return;  // (after the warp-wide tensor-core instructions)
  const __half* scs = reinterpret_cast<const __half*>(st + 2 * ROWB);
  const int si = (g * SEG + (sp << 7)) >> bs;
  const float sl = __half2float(scs[si]), sh = __half2float(scs[geom<2>::SC_ROW / 2 + si]);
  acc[0] += sl * (ta[0] + tb[0]);
  acc[1] += sl * (ta[1] + tb[1]);
  acc[2] += sh * (ta[2] + tb[2]);
  acc[3] += sh * (ta[3] + tb[3]);
}

// Weight types (WT): 0 = fp16; 1 = u8, every weight rounded to half((q - 127.5) * scale) before the
// product exactly as the reference's tensor-core kernel does (llama_cu.cu:287-289, 332-341); 2 = u8
// with the scale factored out of each 64-weight group: sum_k x_k (q_k - 127.5) s = s * (sum_k x_k
// (1024 + q_k) - 1151.5 * sum_k x_k), the bytes going to the tensor core as the exact halves
// 1024 + q (one PRMT per two weights) and the group sums of x coming from the prologue.  Mode 2 has
// no per-weight rounding: it is closer to the exact product but is not the reference's rounding.
template <int WT, int EPI, int NW>
__global__ void __launch_bounds__((NW + 1) * 32, NW == 4 ? 3 : 2) gemv1_kernel(const gemv_params p, const int sw, const int pf_bytes) {
  constexpr int NCONS = NW * 32;
  static_assert(NW >= 4 && NW <= NW_MAX, "the RMSNorm reduction uses the first four consumer warps");
  constexpr int ESZ = WT == 0 ? 2 : 1;
  constexpr int ROWB = geom<WT>::ROWB, SEG = geom<WT>::SEG, NSTEPS = geom<WT>::NSTEPS;
  constexpr int CHUNK_K = ROWB / ESZ;        // weights of one row per stage
  constexpr int STAGE_BYTES = 2 * ROWB + (WT ? 2 * geom<WT>::SC_ROW : 0);

  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // full: [w * MAX_SW + s], empty: [EMPTY_BASE + w * MAX_SW + s]
  float* scratch = reinterpret_cast<float*>(smem + BAR_BYTES);  // [8] floats of the RMSNorm reduction, then the activation row's barrier
  const uint32_t xbar = smem_u32(smem + BAR_BYTES + 32);
  int* cta_done = reinterpret_cast<int*>(smem + BAR_BYTES + 40);  // consumer warps of this CTA that are through (tensor-parallel)
  uint8_t* xs = smem + SMEM_FIXED;                     // activation row, K halves (u8 kernels: skewed, see xoff)
  // u8 kernels read 32 activation bytes per 16 weight bytes; with the row stored flat, the two segments of a
  // quarter warp would meet on the same banks.  The activations of every segment are therefore shifted by 16 more
  // bytes than those of the one before (vector i of eight halves lives at byte 16 * (i + i / (SEG / 8))).
  auto xoff = [](int vec_index) { return WT == 0 ? vec_index * 16 : (vec_index + (vec_index >> (geom<WT>::SEG_SHIFT - 3))) * 16; };
  const int xbytes = WT == 0 ? p.K * 2 : p.K * 2 + (p.K >> geom<WT>::SEG_SHIFT) * 16 + 16;
  float* xs64 = reinterpret_cast<float*>(xs + ((xbytes + 127) & ~127));  // sums of x over aligned groups of 64
  // norm weights beyond what the consumers hold in registers (rows longer than NVEC * 8 * consumer threads) are staged here
  uint8_t* nws = reinterpret_cast<uint8_t*>(xs64) + ((p.K / 64 * 4 + 127) & ~127);
  uint8_t* stages = nws + (p.norm_w != nullptr && p.K > 4096 ? (((p.K - 4096) * 2 + 127) & ~127) : 0);  // [NW][sw][STAGE_BYTES]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();

  const int pairs = (p.n_mats * p.rows_per_mat) >> 1;
  const int pr0 = (int)(((long long)pairs * blockIdx.x) / gridDim.x);
  const int npairs = (int)(((long long)pairs * (blockIdx.x + 1)) / gridDim.x) - pr0;
  const int rowbytes = p.K * ESZ;
  const int nchunks = (rowbytes + ROWB - 1) / ROWB;

  // Scales of a row chunk are one contiguous run; when rows start 16-byte aligned they travel as one more bulk copy
  // per row on the same barrier, otherwise as 4-byte cp.async pieces issued by all lanes (32 more barrier arrivals).
  const bool sc_bulk = WT != 0 && ((p.K / p.bs) & 7) == 0 && ((ROWB / p.bs) & 7) == 0;
  if (tid == 0) {
    for (int i = 0; i < NW * MAX_SW; ++i) {
      mbar_init(smem_u32(&bars[i]), (WT == 0 || sc_bulk) ? 1 : 33);
      mbar_init(smem_u32(&bars[EMPTY_BASE + i]), 1);
    }
    mbar_init(xbar, 1);
    *cta_done = 0;
    fence_mbar_init();
  }
  __syncthreads();

  const int bs_shift = p.bs > 0 ? 31 - __clz(p.bs) : 0;  // block size is a power of two (32, 64, 128, ...)
  if (warp == NW) {
    // ------------------------------------------------------------ producer
    // (this warp's instruction chain per stage bounds the u8 kernels: shifts, no divisions)
    const uint64_t pol = policy_evict_first();
    if (pf_bytes > 0) {  // L2 look-ahead over the first rows of this CTA
      const int rows_pf = max(1, min(pf_bytes / rowbytes, 2 * npairs));
      for (int r = lane; r < rows_pf; r += 32) {
        int mat, row;
        map_row<EPI>(p, 2 * pr0 + r, mat, row);
        l2_prefetch(reinterpret_cast<const uint8_t*>(p.w[mat]) + (size_t)row * rowbytes, (uint32_t)rowbytes);
      }
    }
    int slot[NW];
    uint32_t par[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      slot[w] = 0;
      par[w] = 0;
    }
    const int full_rounds = npairs / NW, r_tail = npairs - full_rounds * NW;
    // one stage for consumer warp w: `cbytes` bytes of both rows of a pair (lanes 0 and 1 hold the row addresses,
    // the half warps the scale addresses) and their scales
    // Copies of a stage are issued by one predicated instruction: lanes 0 and 1 copy the two rows, lanes 2 and 16 the
    // scale runs of rows 0 and 1 when those travel as bulk copies (scale addresses are held per half warp).
    const uint32_t bars_u32 = smem_u32(bars), stages_u32 = smem_u32(stages);
    const bool lane_sc = lane >= 2;
    const bool lane_copies = lane < 2 || (sc_bulk && (lane == 2 || lane == 16));
    const uint32_t lane_dst = lane_sc ? 2 * ROWB + (lane >> 4) * (WT ? geom<WT>::SC_ROW : 0) : lane * ROWB;
    auto issue = [&](const int w, const uint8_t* row_src, const __half* sc_src, const int cbytes) {
      const uint32_t full = bars_u32 + (uint32_t)(w * MAX_SW + slot[w]) * 8;
      mbar_wait(full + EMPTY_BASE * 8, par[w] ^ 1, p.err, DEV_ERR_EMPTY_WAIT);
      const uint32_t st = stages_u32 + (uint32_t)(w * sw + slot[w]) * STAGE_BYTES;
      const uint32_t scbytes = WT != 0 ? (uint32_t)(cbytes >> bs_shift) * 2 : 0;  // scale bytes per row of this chunk
      if (lane == 0) mbar_arrive_expect_tx(full, (uint32_t)(2 * cbytes) + (sc_bulk ? 2 * scbytes : 0));
      __syncwarp();
      if (lane_copies)
        bulk_g2s_hint(st + lane_dst, lane_sc ? (const void*)sc_src : (const void*)row_src, lane_sc ? scbytes : (uint32_t)cbytes, full, pol);
      if (WT != 0 && !sc_bulk) {
        const int ppr = (cbytes >> bs_shift) >> 1;  // 4-byte pieces per row
        for (int j = lane & 15; j < ppr; j += 16) cp_async4(st + 2 * ROWB + (lane >> 4) * geom<WT>::SC_ROW + j * 4, sc_src + 2 * j);
        cp_async_mbar_arrive_noinc(full);
      }
      if (++slot[w] == sw) {
        slot[w] = 0;
        par[w] ^= 1;
      }
    };
    auto pair_sources = [&](const int pr, const uint8_t*& row_src, const __half*& sc_src) {
      int mat, row;
      map_row<EPI>(p, 2 * pr + (lane & 1), mat, row);
      row_src = reinterpret_cast<const uint8_t*>(p.w[mat]) + (size_t)row * rowbytes;
      sc_src = nullptr;
      if (WT) {
        int m2, r2;
        map_row<EPI>(p, 2 * pr + (lane >> 4), m2, r2);
        sc_src = p.sc[m2] + (size_t)r2 * (p.K >> bs_shift);
      }
    };
    // full rounds: chunk ci of the pairs base .. base+NW-1 goes to warps 0 .. NW-1 in turn
    for (int rd = 0; rd < full_rounds; ++rd) {
      const uint8_t* src_row[NW];
      const __half* src_sc[NW];
#pragma unroll
      for (int w = 0; w < NW; ++w) pair_sources(pr0 + rd * NW + w, src_row[w], src_sc[w]);
      for (int ci = 0; ci < nchunks; ++ci) {
        const int cbytes = min(ROWB, rowbytes - ci * ROWB);
#pragma unroll
        for (int w = 0; w < NW; ++w) issue(w, src_row[w] + (size_t)ci * ROWB, WT ? src_sc[w] + ((ci * CHUNK_K) >> bs_shift) : nullptr, cbytes);
      }
    }
    // tail round: the pairs left over go to warps 0 .. r_tail-1
    if (r_tail > 0) {
      const uint8_t* src_row[NW];
      const __half* src_sc[NW];
#pragma unroll
      for (int w = 0; w < NW; ++w)
        if (w < r_tail) pair_sources(pr0 + full_rounds * NW + w, src_row[w], src_sc[w]);
      for (int ci = 0; ci < nchunks; ++ci) {
        const int cbytes = min(ROWB, rowbytes - ci * ROWB);
#pragma unroll
        for (int w = 0; w < NW; ++w)
          if (w < r_tail) issue(w, src_row[w] + (size_t)ci * ROWB, WT ? src_sc[w] + ((ci * CHUNK_K) >> bs_shift) : nullptr, cbytes);
      }
    }
    if (WT != 0) cp_async_wait<0>();
    return;
  }

  // -------------------------------------------------------------- consumers
  // The norm weights do not depend on the previous kernel: their loads are in flight while this one waits for it.
  constexpr int NVEC = 4;  // 16-byte vectors of norm weights per thread kept in registers (covers K <= 4096 with four warps)
  const int vec = p.K >> 3;
  uint4 nw[NVEC];
  if (p.norm_w != nullptr && npairs > 0) {
#pragma unroll
    for (int j = 0; j < NVEC; ++j) {
      const int i = tid + j * NCONS;
      nw[j] = i < vec ? *reinterpret_cast<const uint4*>(p.norm_w + i * 8) : make_uint4(0, 0, 0, 0);
    }
    // the rest of a long row's norm weights: asynchronous 16-byte copies into shared memory, no registers held
    for (int i = tid + NVEC * NCONS; i < vec; i += NCONS) cp_async16(smem_u32(nws) + (uint32_t)(i - NVEC * NCONS) * 16, p.norm_w + i * 8);
    cp_async_commit();
  }
  pdl_wait();
  if (npairs > 0) {
    // Rows that fit the consumers' registers (NVEC vectors per thread: K <= 4096 with four warps) are loaded by the
    // threads themselves and stay in registers for the normalisation.  Longer rows come in as bulk copies of one
    // 512-element segment each: one trip to L2 whatever the row length, where per-thread loads paid a round trip per
    // batch of vectors - several microseconds for rows of 8192 and more.  Both read past L1 (L2 is where another GPU's
    // peer stores land).
    const bool row_in_regs = vec <= NVEC * NCONS;
    uint4 xv[NVEC];
    if (row_in_regs) {
      if (p.n_wait > 0) {
        // tensor-parallel: parts of the row come from other GPUs; wait for their flags first
        if (tid < p.n_wait) flag_wait_at_least(p.wait_flags + tid, *p.seq * TP_EXCHANGES_PER_STEP + p.wait_id, p.err);
        bar_sync(1, NCONS);
      }
#pragma unroll
      for (int j = 0; j < NVEC; ++j) {
        const int i = tid + j * NCONS;
        if (i < vec) {
          xv[j] = __ldcg(reinterpret_cast<const uint4*>(p.x + i * 8));
          *reinterpret_cast<uint4*>(xs + xoff(i)) = xv[j];
        }
      }
      bar_sync(1, NCONS);
    } else {
      if (warp == 0) {
        if (p.n_wait > 0) {
          if (lane < p.n_wait) flag_wait_at_least(p.wait_flags + lane, *p.seq * TP_EXCHANGES_PER_STEP + p.wait_id, p.err);
          __syncwarp();
        }
        if (lane == 0) mbar_arrive_expect_tx(xbar, (uint32_t)p.K * 2);
        __syncwarp();
        const int nseg = (p.K + 511) >> 9;
        for (int sg = lane; sg < nseg; sg += 32)
          bulk_g2s(smem_u32(xs + xoff(sg * 64)), p.x + sg * 512, (uint32_t)min(1024, (p.K - sg * 512) * 2), xbar);
      }
      mbar_wait(xbar, 0, p.err, DEV_ERR_FULL_WAIT);
    }
    if (p.norm_w != nullptr) {
      // RMSNorm with the reference's summation order (llama_cu.cu:72-106): 256 strided partial sums,
      // xor trees inside 8 warps, xor tree over the 8 warp sums.  Each of the 128 threads here plays
      // two of the reference's threads (t and t + 128), each warp two of its warps (w and w + 4).
      auto xat = [&](int i) { return __half2float(*reinterpret_cast<const __half*>(xs + xoff(i >> 3) + (i & 7) * 2)); };
      if (warp < 4) {  // (a fifth consumer warp only joins the barriers and the normalisation below)
        float s0 = 0.f, s1 = 0.f;
        for (int i = tid; i < p.K; i += 256) {
          float v = xat(i);
          s0 += v * v;
        }
        for (int i = tid + 128; i < p.K; i += 256) {
          float v = xat(i);
          s1 += v * v;
        }
        s0 = warp_sum(s0);
        s1 = warp_sum(s1);
        if (lane == 0) {
          scratch[warp] = s0;
          scratch[warp + 4] = s1;
        }
      }
      bar_sync(1, NCONS);
      float t = lane < 8 ? scratch[lane] : 0.f;  // every warp repeats the last tree: no second hand-over
      for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      const float rinv = rsqrtf(__shfl_sync(0xffffffffu, t, 0) / p.K + p.eps);
      // x_i <- norm_w_i *h half(x_i * rinv), eight elements at a time from the registers filled above
      auto norm8 = [&](uint4 xq, uint4 wq) {
        __half2* xq2 = reinterpret_cast<__half2*>(&xq);
        const __half2* wq2 = reinterpret_cast<const __half2*>(&wq);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(xq2[e]);
          xq2[e] = __hmul2(wq2[e], __floats2half2_rn(f.x * rinv, f.y * rinv));
        }
        return xq;
      };
#pragma unroll
      for (int j = 0; j < NVEC; ++j) {
        const int i = tid + j * NCONS;
        if (i < vec) *reinterpret_cast<uint4*>(xs + xoff(i)) = norm8(row_in_regs ? xv[j] : *reinterpret_cast<const uint4*>(xs + xoff(i)), nw[j]);
      }
      cp_async_wait<0>();  // (each thread reads back the staged norm weights it copied itself)
      for (int i = tid + NVEC * NCONS; i < vec; i += NCONS)
        *reinterpret_cast<uint4*>(xs + xoff(i)) =
            norm8(*reinterpret_cast<const uint4*>(xs + xoff(i)), *reinterpret_cast<const uint4*>(nws + (size_t)(i - NVEC * NCONS) * 16));
      bar_sync(1, NCONS);
    }
    if (WT == 2) {  // sums of the (normalised) activations over aligned groups of 64: eight lanes per group, 16 bytes per lane
#pragma unroll 3
      for (int grp64 = warp * 4 + (lane >> 3); grp64 < p.K / 64; grp64 += NW * 4) {
        const uint4 q = *reinterpret_cast<const uint4*>(xs + xoff(grp64 * 8 + (lane & 7)));
        const __half2* h = reinterpret_cast<const __half2*>(&q);
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(h[e]);
          s += f.x + f.y;
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if ((lane & 7) == 0) xs64[grp64] = s;
      }
      bar_sync(1, NCONS);
    }
  }

  const int g = lane >> 2, c = lane & 3;
  const int flip = g & 1;
  const bool diag = c == (g >> 1);
  int pos = 0;
  if (EPI == EPI_ROPE_KV) pos = *p.pos;

  int slot = 0;
  uint32_t par = 0;
  for (int i = warp; i < npairs; i += NW) {
    float accs[NACC][4];
#pragma unroll
    for (int a = 0; a < NACC; ++a) accs[a][0] = accs[a][1] = accs[a][2] = accs[a][3] = 0.f;
    // u8 kernels (latency-bound): what the epilogue reads from global memory is requested now, one address for the
    // whole warp, so that its latency passes under the row's products instead of after them.  The fp16 kernels run at
    // the memory roofline, where the early loads measured no difference; they fetch in the epilogue.
    constexpr bool EARLY = WT != 0;
    const int vrow = 2 * (pr0 + i);
    __half2 prev = __half2half2(__ushort_as_half(0));
    float2 cs = make_float2(1.f, 0.f);
    int mat = 0, row = vrow, head = 0, j = 0;
    auto fetch_epilogue_operands = [&]() {
      if (EPI == EPI_PLAIN) {
        if (p.beta != 0.f) prev = *reinterpret_cast<const __half2*>(p.out + vrow);
      } else if (EPI == EPI_ROPE_KV) {
        map_row<EPI_ROPE_KV>(p, vrow, mat, row);
        head = row / p.head_dim;
        j = row - head * p.head_dim;
        if (mat < 2) cs = p.rope[(size_t)pos * (p.head_dim >> 1) + (j >> 1)];
      }
    };
    if (EARLY) fetch_epilogue_operands();
    for (int ci = 0; ci < nchunks; ++ci) {
      mbar_wait(smem_u32(&bars[warp * MAX_SW + slot]), par, p.err, DEV_ERR_FULL_WAIT);
      const int cbytes = min(ROWB, rowbytes - ci * ROWB);
      const int vb = min(max(cbytes - g * SEG, 0), SEG);  // valid bytes of this lane's segment
      const uint8_t* st = stages + (size_t)(warp * sw + slot) * STAGE_BYTES;
      const uint8_t* seg0 = st + g * SEG;
      const uint8_t* xseg = xs + xoff((ci * CHUNK_K + g * (SEG / ESZ)) >> 3);
      // A full chunk (every chunk but possibly the last of a row) takes the branch-free path, so that the
      // shared loads of all eight steps can be issued ahead of the tensor-core instructions.
      if (WT == 2 && cbytes == ROWB && bs_shift >= 7) {
#pragma unroll
        for (int sp = 0; sp < NSTEPS / 2; ++sp) step_pair_factored<true>(accs, sp, flip, c, g, SEG, seg0, xseg, st, xs64, ci, bs_shift);
      } else if (WT == 2 && bs_shift >= 7) {
#pragma unroll
        for (int sp = 0; sp < NSTEPS / 2; ++sp) step_pair_factored<false>(accs, sp, flip, c, g, vb, seg0, xseg, st, xs64, ci, bs_shift);
      } else if (cbytes == ROWB) {
#pragma unroll
        for (int s = 0; s < NSTEPS; ++s) step<WT, true>(accs, s, flip, c, g, SEG, seg0, xseg, st, xs64, ci, bs_shift);
      } else {
#pragma unroll
        for (int s = 0; s < NSTEPS; ++s) step<WT, false>(accs, s, flip, c, g, vb, seg0, xseg, st, xs64, ci, bs_shift);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[EMPTY_BASE + warp * MAX_SW + slot]));
      if (++slot == sw) {
        slot = 0;
        par ^= 1;
      }
    }

    // the diagonal lanes hold segment g of row 0 (d0/d1) and of row 1 (d2/d3): fixed-order shuffle tree
    float v0 = 0.f, v1 = 0.f;
    if (diag) {
      const float a0 = (accs[0][0] + accs[1][0]) + (accs[2][0] + accs[3][0]), a1 = (accs[0][1] + accs[1][1]) + (accs[2][1] + accs[3][1]);
      const float a2 = (accs[0][2] + accs[1][2]) + (accs[2][2] + accs[3][2]), a3 = (accs[0][3] + accs[1][3]) + (accs[2][3] + accs[3][3]);
      v0 = (g & 1) ? a1 : a0;
      v1 = (g & 1) ? a3 : a2;
    }
    v0 = warp_sum(v0);
    v1 = warp_sum(v1);
    if (lane == 0) {
      const int pr = pr0 + i;
      if (!EARLY) fetch_epilogue_operands();
      if (EPI == EPI_PLAIN) {
        float a0 = v0, a1 = v1;
        __half* o = p.out + vrow;
        if (p.beta != 0.f) {
          a0 = a0 + p.beta * __low2float(prev);
          a1 = a1 + p.beta * __high2float(prev);
        }
        const __half2 r2 = __halves2half2(__float2half(a0), __float2half(a1));
        *reinterpret_cast<__half2*>(o) = r2;
        if (p.out_peer) *reinterpret_cast<__half2*>(p.out_peer + vrow) = r2;  // peer store over NVLink
        for (int q = 0; q < p.n_peer_out; ++q) *reinterpret_cast<__half2*>(p.peer_out[q] + vrow) = r2;  // tensor-parallel: into every GPU's row
      } else {
        const __half a = __float2half(v0), bq = __float2half(v1);  // the matmul's own output rounding
        if (EPI == EPI_SILU) {
          const float val = __half2float(a);  // llama_cu.cu:536-537 on the half-rounded w1 / w3 outputs
          const __half gated = __float2half(val / (1.0f + expf(-val)) * __half2float(bq));
          p.out[pr] = gated;
          for (int q = 0; q < p.n_peer_out; ++q) p.peer_out[q][pr] = gated;
        } else {
          __half o0 = a, o1 = bq;
          if (mat < 2) {  // llama_cu.cu:381-387, cos/sin from the context's table (fetched above)
            const float real = __half2float(a), imag = __half2float(bq);
            const float a_cos = cs.x, a_sin = cs.y;
            o0 = __float2half(real * a_cos - imag * a_sin);
            o1 = __float2half(real * a_sin + imag * a_cos);
          }
          const __half2 pr2 = __halves2half2(o0, o1);
          if (mat == 0) {
            *reinterpret_cast<__half2*>(p.q_out + row) = pr2;
          } else {
            __half* cache = mat == 1 ? p.k_cache : p.v_cache;
            *reinterpret_cast<__half2*>(cache + ((size_t)head * p.ctx_len + pos) * p.head_dim + j) = pr2;
          }
        }
      }
    }
  }
  // tensor-parallel: the last consumer warp of the launch to get here publishes this GPU's slice (every result went into
  // the other GPUs' rows as a peer store in the epilogue above, made by lane 0 of its warp).  The fences widen with the
  // counting: a warp counts itself inside its CTA behind a CTA-scope fence (shared memory), the last warp of a CTA
  // counts the CTA behind a device-scope fence (global memory), and only the last warp of the launch pays for the
  // system-scope fence - cumulative over everything counted before it - ahead of the flags it writes into the waiting
  // GPUs' memory.  (A system-scope fence in every warp serialises for more than 10 us per launch.)
  if (p.done_count != nullptr && lane == 0) {
    __threadfence_block();
    if (atomicAdd_block(cta_done, 1) == NW - 1) {
      __threadfence();
      if (atomicAdd(p.done_count, 1) == (int)gridDim.x - 1) {
        atomicExch(p.done_count, 0);  // (the next launch counts from zero; its warps arrive after this kernel has ended)
        fence_acq_rel_sys();
        const int stamp = *p.seq * TP_EXCHANGES_PER_STEP + p.exchange_id;
        for (int q = 0; q < p.n_peer_flag; ++q) st_relaxed_sys(p.peer_flag[q], stamp);
      }
    }
  }
}

template <int WT, int EPI, int NW>
int launch_one(const gemv_params& p, cudaStream_t stream, int pdl, size_t smem, int grid, int sw, int pf_bytes) {
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(gemv1_kernel<WT, EPI, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3((NW + 1) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  LCU_CUDA(cudaLaunchKernelEx(&cfg, gemv1_kernel<WT, EPI, NW>, p, sw, pf_bytes));
  return LCU_OK;
}

}  // namespace

namespace {
struct gemv1_config {
  int wt, nw, sw, grid, pf;
  size_t smem;
};
int configure(const gemv_params& p, int sms, gemv1_config& c) {
  const gemv_tuning& t = gemv_tuning_ref();
  const bool q = p.bs != 0;
  // weight type of the kernel: fp16; u8 with the reference's per-weight rounding; u8 with factored scales
  const int wt = !q ? 0 : ((t.int8_factored && p.bs >= 64) ? 2 : 1);
  const size_t stage_bytes = wt == 2 ? 2 * geom<2>::ROWB + 2 * geom<2>::SC_ROW : wt == 1 ? 2 * geom<1>::ROWB + 2 * geom<1>::SC_ROW : 2 * geom<0>::ROWB;
  const int seg_shift = wt == 2 ? geom<2>::SEG_SHIFT : geom<1>::SEG_SHIFT;
  const size_t xbytes = wt == 0 ? (size_t)p.K * 2 : (size_t)p.K * 2 + ((size_t)p.K >> seg_shift) * 16 + 16;  // u8: skewed activation row
  const size_t nw_stage = p.norm_w != nullptr && p.K > 4096 ? ((((size_t)p.K - 4096) * 2 + 127) & ~(size_t)127) : 0;
  const size_t fixed = SMEM_FIXED + ((xbytes + 127) & ~(size_t)127) + (((size_t)p.K / 64 * 4 + 127) & ~(size_t)127) + nw_stage;
  // CTAs per SM: as many as asked for that still fit with a two-deep ring per warp (the factored u8 kernel is
  // latency-bound and compiled for three); then the deepest ring that keeps them resident
  int cps = wt == 2 ? t.ctas_per_sm_int8 : t.ctas_per_sm;
  if (cps < 1) cps = 1;
  if (cps > 3) cps = 3;
  auto fits = [&](int warps, int stages, int ctas) { return fixed + (size_t)warps * stages * stage_bytes <= (size_t)(228 * 1024) / ctas - 1024; };
  while (cps > 1 && !fits(4, 2, cps)) --cps;
  // factored u8 kernels that cannot have three CTAs of four consumer warps per SM take five consumer warps per CTA
  // when those fit (a long activation row: w2 of every model, every matrix of the larger models)
  int nw = 4;
  if (wt == 2 && cps < 3 && t.consumer_warps_int8 != 4 && fits(5, 2, cps)) nw = 5;
  const int want_sw = wt == 2 ? t.warp_stages_int8 : t.warp_stages;
  int sw = want_sw < 2 ? 2 : (want_sw > MAX_SW ? MAX_SW : want_sw);
  while (sw > 2 && !fits(nw, sw, cps)) --sw;
  const size_t smem = fixed + (size_t)nw * sw * stage_bytes;
  LCU_REQUIRE(smem <= 227 * 1024, "gemv: a row of K=%d does not fit in shared memory", p.K);
  const int pairs = p.n_mats * p.rows_per_mat / 2;
  c.wt = wt;
  c.nw = nw;
  c.sw = sw;
  c.grid = sms * cps > pairs ? pairs : sms * cps;
  c.pf = t.prefetch_kb_per_cta * 1024;
  c.smem = smem;
  return LCU_OK;
}
}  // namespace

// Loads every single-row kernel on the current device (the CUDA runtime loads a kernel at its first use; a first decode
// step whose launches stall one after the other in that loading would leave the other GPUs of a tensor-parallel step
// waiting far longer than their bounded waits allow).
int gemv_single_row_preload() {
  cudaFuncAttributes fa;
#define LCU_PRELOAD(WTV, E, NWV) LCU_CUDA(cudaFuncGetAttributes(&fa, gemv1_kernel<WTV, E, NWV>));
#define LCU_PRELOAD_E(E) LCU_PRELOAD(0, E, 4) LCU_PRELOAD(1, E, 4) LCU_PRELOAD(2, E, 4) LCU_PRELOAD(2, E, 5)
  LCU_PRELOAD_E(EPI_PLAIN)
  LCU_PRELOAD_E(EPI_ROPE_KV)
  LCU_PRELOAD_E(EPI_SILU)
#undef LCU_PRELOAD_E
#undef LCU_PRELOAD
  return LCU_OK;
}

// consumer warps of the launch launch_gemv would make for these arguments (each counts itself once on the waiting GPUs'
// counters in tensor-parallel decode); 0 if the arguments cannot be launched
int gemv_single_row_consumer_warps(const gemv_params& p) {
  gemv1_config c;
  if (configure(p, gemv_sm_count(), c) != LCU_OK) return 0;
  return c.grid * c.nw;
}

// m == 1 entry used by launch_gemv (argument checks are done there)
int launch_gemv_single_row(const gemv_params& p, int epilogue, cudaStream_t stream, int pdl, int sms) {
  gemv1_config c;
  int rc = configure(p, sms, c);
  if (rc) return rc;
  const int wt = c.wt, nw = c.nw, sw = c.sw, grid = c.grid, pf = c.pf;
  const size_t smem = c.smem;
#define LCU_GEMV1_CASE(E)                                                                  \
  case E:                                                                                  \
    if (wt == 0) return launch_one<0, E, 4>(p, stream, pdl, smem, grid, sw, pf);           \
    if (wt == 1) return launch_one<1, E, 4>(p, stream, pdl, smem, grid, sw, pf);           \
    if (nw == 5) return launch_one<2, E, 5>(p, stream, pdl, smem, grid, sw, pf);           \
    return launch_one<2, E, 4>(p, stream, pdl, smem, grid, sw, pf);
  switch (epilogue) {
    LCU_GEMV1_CASE(EPI_PLAIN)
    LCU_GEMV1_CASE(EPI_ROPE_KV)
    LCU_GEMV1_CASE(EPI_SILU)
  }
#undef LCU_GEMV1_CASE
  LCU_REQUIRE(false, "gemv: unknown epilogue %d", epilogue);
}

}  // namespace lcu
