// Batch-1 decode GEMV for sm_100a: out = W . x with W streamed once from HBM.
//
// Replaces the reference's small-m tile kernels (llama_cu.cu:225-285 fp16, 287-366 int8) and the
// element-wise kernels around them (rms_norm 66-107, rotary 368-389, silu 533-539) for m <= 8.
//
// Structure of one CTA (one per SM, persistent over a contiguous range of output rows):
//   * a producer warp keeps a ring of shared-memory stages full with 1-D bulk copies (TMA,
//     cp.async.bulk) of 16 weight rows x KCB bytes; int8 scales ride along with 4-byte cp.async
//     handed to the same mbarrier.  The producer never waits for activations, so under
//     programmatic dependent launch the weight stream of kernel n+1 starts while kernel n drains.
//   * consumer warps read the staged rows with conflict-free 128-bit loads, de-quantise int8 in
//     registers with the reference's rounding (half((q - 127.5) * scale), llama_cu.cu:287-289)
//     and feed an m16n8k16 tensor-core product whose B operand holds the (up to 8) activation
//     rows; the k index is permuted identically on both operands, which a dot product allows.
//     Each warp owns a k-slice of every stage; partial sums are combined in a fixed order.
//   * epilogues fuse what the reference does in separate kernels: residual add (beta = 1),
//     RoPE + KV-cache write, SiLU gate.  The RMSNorm of the input row is fused as a prologue.
#include "gemv.cuh"

namespace lcu {
namespace {

constexpr int NCW = 8;                  // consumer warps
constexpr int NTHREADS = (NCW + 1) * 32;
constexpr int RB = 16;                  // weight rows per stage (one MMA row block)
constexpr int KCB = 1024;               // bytes per weight row per stage
constexpr int ROWSTRIDE = KCB + 64;     // == 64 (mod 128): 128-bit loads of 8 lanes hit 8 distinct 16-byte bank groups
constexpr int SCROW = KCB / 16;         // scale bytes reserved per row per stage (bs >= 32)
constexpr int STAGE_W = RB * ROWSTRIDE;
constexpr int STAGE_BYTES = STAGE_W + RB * SCROW;
constexpr int MAX_STAGES = 8;
constexpr int NACC = 4;                  // independent accumulator sets per warp
constexpr int RED_FLOATS = NCW * 16 * 8;  // per-warp partial sums of a row block, double buffered
constexpr int SMEM_FIXED = 256 /*barriers: 2 x MAX_STAGES x 8 bytes, padded*/ + 2 * RED_FLOATS * 4 + 64 /*reduction scratch*/;

__host__ __device__ inline int x_stride_bytes(int K) { return K * 2 + 64; }

template <int EPI>
__device__ __forceinline__ void map_row(const gemv_params& p, int vrow, int& mat, int& row) {
  if (EPI == EPI_SILU) {
    mat = vrow & 1;
    row = vrow >> 1;
  } else if (EPI == EPI_ROPE_KV) {
    mat = vrow / p.rows_per_mat;
    row = vrow - mat * p.rows_per_mat;
  } else {
    mat = 0;
    row = vrow;
  }
}

__device__ __forceinline__ uint32_t dequant_pair(uint32_t word, uint32_t selector, __half2 scale2) {
  // bytes (q_lo, q_hi) -> halves 1024+q (exact), minus 1024, minus 127.5 (both exact), times scale (one rounding)
  uint32_t v = __byte_perm(word, 0x64646464u, selector);
  __half2 h = *reinterpret_cast<__half2*>(&v);
  h = __hsub2(h, __half2half2(__ushort_as_half(0x6400)));  // 1024
  h = __hsub2(h, __half2half2(__ushort_as_half(0x57f8)));  // 127.5
  h = __hmul2(h, scale2);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int WT /*0 fp16, 1 u8*/, int EPI>
__global__ void __launch_bounds__(NTHREADS, 2) gemv_kernel(const gemv_params p, const int nstages, const int pf_bytes) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // full[MAX_STAGES], empty[MAX_STAGES]
  float* red = reinterpret_cast<float*>(smem + 256);
  float* scratch = red + 2 * RED_FLOATS;  // 16 floats
  uint8_t* xs = smem + SMEM_FIXED;
  const int xstride = x_stride_bytes(p.K);
  uint8_t* stages = xs + (size_t)p.m * xstride;  // SMEM_FIXED and xstride are multiples of 64

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  pdl_launch_dependents();

  // rows of this CTA: contiguous range in units of two rows (pairs stay together)
  const int n_total = p.n_mats * p.rows_per_mat;
  const int units = n_total >> 1;
  const int r0 = (int)(((long long)units * blockIdx.x) / gridDim.x) * 2;
  const int r1 = (int)(((long long)units * (blockIdx.x + 1)) / gridDim.x) * 2;
  const int nblocks = (r1 - r0 + RB - 1) / RB;
  const int rowbytes = WT == 0 ? p.K * 2 : p.K;
  const int nchunks = (rowbytes + KCB - 1) / KCB;

  if (tid == 0) {
    for (int i = 0; i < nstages; ++i) {
      mbar_init(smem_u32(&bars[i]), WT == 0 ? 1 : 33);
      mbar_init(smem_u32(&bars[MAX_STAGES + i]), NCW);
    }
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == NCW) {
    // ------------------------------------------------------------ producer
    const uint64_t pol = policy_evict_first();
    // Look-ahead into L2: the first pf_bytes of this CTA's rows are requested before the ring starts.
    // Under programmatic dependent launch this runs while the previous kernels are still busy (or,
    // like attention, latency-bound), so HBM keeps streaming across kernel boundaries.
    if (pf_bytes > 0) {
      int rows_pf = pf_bytes / rowbytes;
      rows_pf = max(1, min(rows_pf, r1 - r0));
      for (int r = lane; r < rows_pf; r += 32) {
        int mat, row;
        map_row<EPI>(p, r0 + r, mat, row);
        l2_prefetch(reinterpret_cast<const uint8_t*>(p.w[mat]) + (size_t)row * rowbytes, (uint32_t)rowbytes);
      }
    }
    int stage = 0;
    uint32_t phase = 0;
    for (int b = 0; b < nblocks; ++b) {
      const int rb = r0 + b * RB;
      const int nr = min(RB, r1 - rb);
      // source of this lane's row (lanes 0..15 copy one row each)
      const uint8_t* src_row = nullptr;
      if (lane < nr) {
        int mat, row;
        map_row<EPI>(p, rb + lane, mat, row);
        src_row = reinterpret_cast<const uint8_t*>(p.w[mat]) + (size_t)row * rowbytes;
      }
      for (int ci = 0; ci < nchunks; ++ci) {
        const uint32_t full = smem_u32(&bars[stage]);
        const uint32_t empty = smem_u32(&bars[MAX_STAGES + stage]);
        mbar_wait(empty, phase ^ 1, p.err, DEV_ERR_EMPTY_WAIT);
        const int cbytes = min(KCB, rowbytes - ci * KCB);
        uint8_t* st = stages + (size_t)stage * STAGE_BYTES;
        if (lane == 0) mbar_arrive_expect_tx(full, (uint32_t)(nr * cbytes));
        __syncwarp();
        if (lane < nr) bulk_g2s_hint(smem_u32(st + lane * ROWSTRIDE), src_row + (size_t)ci * KCB, (uint32_t)cbytes, full, pol);
        if (WT == 1) {
          // scales of this chunk: cbytes / bs halves per row, copied as 4-byte pieces
          const int nb_row = p.K / p.bs;
          const int ppr = (cbytes / p.bs) >> 1;  // pieces per row
          const int first = (ci * KCB) / p.bs;
          for (int q = lane; q < nr * ppr; q += 32) {
            const int r = q / ppr, j = q - r * ppr;
            int mat, row;
            map_row<EPI>(p, rb + r, mat, row);
            cp_async4(smem_u32(st + STAGE_W + r * SCROW + j * 4), p.sc[mat] + (size_t)row * nb_row + first + 2 * j);
          }
          cp_async_mbar_arrive_noinc(full);
        }
        if (++stage == nstages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (WT == 1) cp_async_wait<0>();
    return;
  }

  // -------------------------------------------------------------- consumers
  const int ct = tid;  // 0 .. NCW*32-1
  pdl_wait();          // activations (and the buffers the epilogue updates) come from the previous kernel

  if (nblocks > 0) {
    // stage the activation rows in shared memory (row stride K*2+64 bytes)
    const int vec_per_row = p.K >> 3;
    for (int r = 0; r < p.m; ++r)
      for (int i = ct; i < vec_per_row; i += NCW * 32)
        *reinterpret_cast<uint4*>(xs + (size_t)r * xstride + i * 16) =
            *reinterpret_cast<const uint4*>(p.x + (size_t)r * p.ldx + i * 8);
    bar_sync(1, NCW * 32);
    if (p.norm_w != nullptr) {
      // RMSNorm prologue, summation order of the reference kernel (llama_cu.cu:72-100): 256 strided
      // partial sums, xor trees inside each warp, xor tree over the 8 warp sums.
      __half* xh = reinterpret_cast<__half*>(xs);
      float s = 0.f;
      for (int i = ct; i < p.K; i += 256) {
        float v = __half2float(xh[i]);
        s += v * v;
      }
      s = warp_sum(s);
      if (lane == 0) scratch[warp] = s;
      bar_sync(1, NCW * 32);
      if (warp == 0) {
        float t = lane < 8 ? scratch[lane] : 0.f;
        for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) scratch[8] = rsqrtf(t / p.K + p.eps);
      }
      bar_sync(1, NCW * 32);
      const float rinv = scratch[8];
      for (int i = ct; i < p.K; i += 256) {
        float v = __half2float(xh[i]);
        xh[i] = __hmul(p.norm_w[i], __float2half(v * rinv));
      }
      bar_sync(1, NCW * 32);
    }
  }

  const int g = lane >> 2, c = lane & 3;
  int pos = 0;
  if (EPI == EPI_ROPE_KV) pos = *p.pos;

  // every consumer warp takes 1/8 of the 64-byte steps of every stage
  int stage = 0;
  uint32_t phase = 0;
  for (int b = 0; b < nblocks; ++b) {
    const int rb = r0 + b * RB;
    // Independent accumulators: consecutive tensor-core instructions of a warp must not wait for
    // each other's result (a chain on one accumulator serialises on the instruction's latency).
    float accs[NACC][4];
#pragma unroll
    for (int a = 0; a < NACC; ++a) accs[a][0] = accs[a][1] = accs[a][2] = accs[a][3] = 0.f;
    for (int ci = 0; ci < nchunks; ++ci) {
      mbar_wait(smem_u32(&bars[stage]), phase, p.err, DEV_ERR_FULL_WAIT);
      const int cbytes = min(KCB, rowbytes - ci * KCB);
      const int nsteps = cbytes >> 6;
      const uint8_t* st = stages + (size_t)stage * STAGE_BYTES;
      const int s_first = warp, s_stride = NCW;
#pragma unroll
      for (int it = 0; it < KCB / 64; ++it) {
        const int s = s_first + it * s_stride;
        if (s >= nsteps) break;
        float* acc = accs[(it * 2) % NACC];
        float* acc_b = accs[(it * 2 + 1) % NACC];
        const uint8_t* pa = st + g * ROWSTRIDE + s * 64 + c * 16;
        const uint4 lo = *reinterpret_cast<const uint4*>(pa);
        const uint4 hi = *reinterpret_cast<const uint4*>(pa + 8 * ROWSTRIDE);
        if (WT == 0) {
          const int kx = (ci * KCB >> 1) + s * 32 + c * 8;
          uint4 xb = make_uint4(0, 0, 0, 0);
          if (g < p.m) xb = *reinterpret_cast<const uint4*>(xs + (size_t)g * xstride + kx * 2);
          mma_16816(acc, lo.x, hi.x, lo.y, hi.y, xb.x, xb.y);
          mma_16816(acc_b, lo.z, hi.z, lo.w, hi.w, xb.z, xb.w);
        } else {
          const int kl = s * 64 + c * 16;  // k offset inside the chunk
          const int kx = ci * KCB + kl;
          uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
          if (g < p.m) {
            const uint8_t* px = xs + (size_t)g * xstride + kx * 2;
            x0 = *reinterpret_cast<const uint4*>(px);
            x1 = *reinterpret_cast<const uint4*>(px + 16);
          }
          const int si = kl / p.bs;
          const __half* scs = reinterpret_cast<const __half*>(st + STAGE_W);
          const __half2 s_lo = __half2half2(scs[g * (SCROW / 2) + si]);
          const __half2 s_hi = __half2half2(scs[(g + 8) * (SCROW / 2) + si]);
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
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[MAX_STAGES + stage]));
      if (++stage == nstages) {
        stage = 0;
        phase ^= 1;
      }
    }

    // combine the accumulators, then the warps' k-slices (fixed order), and run the epilogue
    float acc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float t = accs[0][i];
#pragma unroll
      for (int a = 1; a < NACC; ++a) t += accs[a][i];
      acc[i] = t;
    }
    float* rbuf = red + (b & 1) * RED_FLOATS;
    {
      float* mine = rbuf + warp * 128;
      if (2 * c < p.m) {
        mine[g * 8 + 2 * c] = acc[0];
        mine[(g + 8) * 8 + 2 * c] = acc[2];
      }
      if (2 * c + 1 < p.m) {
        mine[g * 8 + 2 * c + 1] = acc[1];
        mine[(g + 8) * 8 + 2 * c + 1] = acc[3];
      }
    }
    bar_sync(1, NCW * 32);
    if (EPI == EPI_PLAIN) {
      for (int item = ct; item < RB * p.m; item += NCW * 32) {
        const int row = item / p.m, col = item - row * p.m;
        const int vrow = rb + row;
        if (vrow < r1) {
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < NCW; ++w) sum += rbuf[w * 128 + row * 8 + col];
          __half* o = p.out + (size_t)col * p.ldo + vrow;
          if (p.beta != 0.f) sum = sum + p.beta * __half2float(*o);
          *o = __float2half(sum);
          if (p.out_peer) p.out_peer[(size_t)col * p.ldo + vrow] = __float2half(sum);
        }
      }
    } else if (ct < RB / 2) {
      const int vrow = rb + 2 * ct;
      if (vrow < r1) {
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int w = 0; w < NCW; ++w) {
          s0 += rbuf[w * 128 + (2 * ct) * 8];
          s1 += rbuf[w * 128 + (2 * ct + 1) * 8];
        }
        const __half a = __float2half(s0), bq = __float2half(s1);  // the matmul's own output rounding
        if (EPI == EPI_SILU) {
          // llama_cu.cu:536-537 on the half-rounded w1 / w3 outputs
          const float val = __half2float(a);
          p.out[vrow >> 1] = __float2half(val / (1.0f + expf(-val)) * __half2float(bq));
        } else {
          int mat, row;
          map_row<EPI_ROPE_KV>(p, vrow, mat, row);
          const int head = row / p.head_dim, j = row - head * p.head_dim;
          __half o0 = a, o1 = bq;
          if (mat < 2) {
            // llama_cu.cu:381-387 with the angle's cos/sin taken from the context's table
            const float2 cs = p.rope[(size_t)pos * (p.head_dim >> 1) + (j >> 1)];
            const float real = __half2float(a), imag = __half2float(bq);
            const float a_cos = cs.x, a_sin = cs.y;
            o0 = __float2half(real * a_cos - imag * a_sin);
            o1 = __float2half(real * a_sin + imag * a_cos);
          }
          __half2 pr = __halves2half2(o0, o1);
          if (mat == 0) {
            *reinterpret_cast<__half2*>(p.q_out + row) = pr;
          } else {
            __half* cache = mat == 1 ? p.k_cache : p.v_cache;
            *reinterpret_cast<__half2*>(cache + ((size_t)head * p.ctx_len + pos) * p.head_dim + j) = pr;
          }
        }
      }
    }
  }
}

template <int WT, int EPI>
int launch_one(const gemv_params& p, cudaStream_t stream, int pdl, size_t smem, int grid, int nstages, int pf_bytes) {
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(gemv_kernel<WT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  LCU_CUDA(cudaLaunchKernelEx(&cfg, gemv_kernel<WT, EPI>, p, nstages, pf_bytes));
  return LCU_OK;
}

// Read-only ceiling probe: the same bulk-copy ring as the GEMV with consumers that only release
// the stages, so its time is what the memory system allows for a pure stream of `bytes`.
__global__ void __launch_bounds__(64, 2) read_ring_kernel(const uint8_t* src, size_t bytes, int nstages, int ncopy, int* err) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  uint8_t* stages = smem + 256;
  constexpr int PIECE = 16384;
  const size_t pieces = bytes / PIECE;
  const size_t p0 = pieces * blockIdx.x / gridDim.x, p1 = pieces * (blockIdx.x + 1) / gridDim.x;
  if (threadIdx.x == 0) {
    for (int i = 0; i < nstages; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);
      mbar_init(smem_u32(&bars[MAX_STAGES + i]), 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  int stage = 0;
  uint32_t phase = 0;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    // producer warp: each 16 KiB stage arrives as `ncopy` bulk copies issued by the first ncopy lanes
    const uint64_t pol = policy_evict_first();
    const int sub = PIECE / ncopy;
    for (size_t i = p0; i < p1; ++i) {
      mbar_wait(smem_u32(&bars[MAX_STAGES + stage]), phase ^ 1, err, DEV_ERR_EMPTY_WAIT);
      if (lane == 0) mbar_arrive_expect_tx(smem_u32(&bars[stage]), PIECE);
      __syncwarp();
      if (lane < ncopy)
        bulk_g2s_hint(smem_u32(stages + (size_t)stage * PIECE + lane * sub), src + i * PIECE + (size_t)lane * sub, sub, smem_u32(&bars[stage]), pol);
      if (++stage == nstages) {
        stage = 0;
        phase ^= 1;
      }
    }
  } else if (threadIdx.x == 32) {
    for (size_t i = p0; i < p1; ++i) {
      mbar_wait(smem_u32(&bars[stage]), phase, err, DEV_ERR_FULL_WAIT);
      mbar_arrive(smem_u32(&bars[MAX_STAGES + stage]));
      if (++stage == nstages) {
        stage = 0;
        phase ^= 1;
      }
    }
  }
}

int sm_count() {
  static int cached[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && cached[dev]) return cached[dev];
  int n = 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (dev < 16) cached[dev] = n;
  return n;
}

}  // namespace

int gemv_sm_count() { return sm_count(); }

gemv_tuning& gemv_tuning_ref() {
  static gemv_tuning t;
  return t;
}

int bench_read_ceiling(uint64_t bytes, int reps, int ncopy, float* ms_per_pass) {
  LCU_REQUIRE(ncopy == 1 || ncopy == 2 || ncopy == 4 || ncopy == 8 || ncopy == 16 || ncopy == 32, "read ceiling: copies per stage must be a power of two <= 32");
  LCU_REQUIRE(bytes >= (1u << 20) && reps >= 1, "read ceiling: need at least 1 MiB and one repetition");
  const gemv_tuning& t = gemv_tuning_ref();
  const int nstages = t.nstages < 2 ? 2 : (t.nstages > MAX_STAGES ? MAX_STAGES : t.nstages);
  const size_t smem = 256 + (size_t)nstages * 16384;
  uint8_t* buf = nullptr;
  int* err = nullptr;
  LCU_CUDA(cudaMalloc(&buf, bytes));
  LCU_CUDA(cudaMalloc(&err, 4));
  LCU_CUDA(cudaMemset(buf, 1, bytes));
  LCU_CUDA(cudaMemset(err, 0, 4));
  LCU_CUDA(cudaFuncSetAttribute(read_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  const int grid = sm_count() * (t.ctas_per_sm < 1 ? 1 : t.ctas_per_sm);
  cudaEvent_t e0, e1;
  LCU_CUDA(cudaEventCreate(&e0));
  LCU_CUDA(cudaEventCreate(&e1));
  for (int i = 0; i < 3; ++i) read_ring_kernel<<<grid, 64, smem>>>(buf, bytes, nstages, ncopy, err);
  LCU_CUDA(cudaEventRecord(e0, 0));
  for (int i = 0; i < reps; ++i) read_ring_kernel<<<grid, 64, smem>>>(buf, bytes, nstages, ncopy, err);
  LCU_CUDA(cudaEventRecord(e1, 0));
  cudaError_t e = cudaEventSynchronize(e1);
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  int dev_err = 0;
  if (e == cudaSuccess) e = cudaMemcpy(&dev_err, err, 4, cudaMemcpyDeviceToHost);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(buf);
  cudaFree(err);
  LCU_CUDA(e);
  LCU_REQUIRE(dev_err == 0, "read ceiling: a bounded wait gave up (0x%x)", dev_err);
  *ms_per_pass = ms / reps;
  return LCU_OK;
}

size_t gemv_algorithmic_bytes(const gemv_params& p, int epilogue) {
  size_t n = (size_t)p.n_mats * p.rows_per_mat;
  size_t w = p.bs == 0 ? n * p.K * 2 : n * p.K + n * (p.K / p.bs) * 2;
  size_t io = (size_t)p.m * p.K * 2;
  if (epilogue == EPI_SILU)
    io += n;  // n/2 halves
  else
    io += (size_t)p.m * n * 2 * (p.beta != 0.f ? 2 : 1);
  if (p.norm_w) io += (size_t)p.K * 2;
  return w + io;
}

// most activation rows (1..8) of length K one pass of the multi-row kernel can hold next to a two-deep ring
int gemv_max_rows(int K) {
  const size_t room = 227 * 1024 - SMEM_FIXED - 2 * (size_t)STAGE_BYTES;
  const size_t rows = room / (size_t)x_stride_bytes(K);
  return rows > 8 ? 8 : (int)rows;
}

int launch_gemv(const gemv_params& p, int epilogue, cudaStream_t stream, int pdl) {
  LCU_REQUIRE(p.m >= 1 && p.m <= 8, "gemv: m=%d outside 1..8", p.m);
  LCU_REQUIRE(p.K > 0 && p.K % 256 == 0, "gemv: K=%d must be a positive multiple of 256", p.K);
  LCU_REQUIRE(p.rows_per_mat > 0 && p.rows_per_mat % 2 == 0, "gemv: row count %d must be even", p.rows_per_mat);
  LCU_REQUIRE(p.bs == 0 || p.bs == 32 || p.bs == 64 || p.bs == 128, "gemv: quantization block size %d not in {32,64,128}", p.bs);
  LCU_REQUIRE(epilogue == EPI_PLAIN || p.m == 1, "gemv: fused epilogues need m == 1");
  LCU_REQUIRE(p.norm_w == nullptr || p.m == 1, "gemv: fused RMSNorm needs m == 1");
  LCU_REQUIRE(p.ldx % 8 == 0 && ((uintptr_t)p.x & 15) == 0, "gemv: activation rows must be 16-byte aligned");
  for (int i = 0; i < p.n_mats; ++i) {
    LCU_REQUIRE(((uintptr_t)p.w[i] & 15) == 0, "gemv: weight matrix %d is not 16-byte aligned", i);
    LCU_REQUIRE(p.bs == 0 || ((uintptr_t)p.sc[i] & 3) == 0, "gemv: scale matrix %d is not 4-byte aligned", i);
  }
  const gemv_tuning& t = gemv_tuning_ref();
  if (p.m == 1 && t.variant == 1) {
    LCU_REQUIRE((epilogue == EPI_PLAIN && p.n_mats == 1) || (epilogue == EPI_ROPE_KV && p.n_mats == 3 && p.head_dim % 2 == 0 && p.rows_per_mat % p.head_dim == 0) ||
                    (epilogue == EPI_SILU && p.n_mats == 2),
                "gemv: matrix count %d does not fit epilogue %d", p.n_mats, epilogue);
    return launch_gemv_single_row(p, epilogue, stream, pdl, sm_count());
  }
  int nstages = t.nstages < 2 ? 2 : (t.nstages > MAX_STAGES ? MAX_STAGES : t.nstages);
  size_t smem = SMEM_FIXED + (size_t)p.m * x_stride_bytes(p.K) + (size_t)nstages * STAGE_BYTES;
  while (smem > 227 * 1024 && nstages > 2) {
    --nstages;
    smem -= STAGE_BYTES;
  }
  LCU_REQUIRE(smem <= 227 * 1024, "gemv: m=%d rows of K=%d do not fit in shared memory", p.m, p.K);
  const int units = p.n_mats * p.rows_per_mat / 2;
  const int pf_bytes = t.prefetch_kb_per_cta * 1024;
  int grid = sm_count() * (t.ctas_per_sm < 1 ? 1 : t.ctas_per_sm);
  if (grid > units) grid = units;
  const bool q = p.bs != 0;
  switch (epilogue) {
    case EPI_PLAIN:
      LCU_REQUIRE(p.n_mats == 1, "gemv: plain epilogue takes one matrix");
      return q ? launch_one<1, EPI_PLAIN>(p, stream, pdl, smem, grid, nstages, pf_bytes) : launch_one<0, EPI_PLAIN>(p, stream, pdl, smem, grid, nstages, pf_bytes);
    case EPI_ROPE_KV:
      LCU_REQUIRE(p.n_mats == 3 && p.head_dim % 2 == 0 && p.rows_per_mat % p.head_dim == 0, "gemv: bad q/k/v shapes");
      return q ? launch_one<1, EPI_ROPE_KV>(p, stream, pdl, smem, grid, nstages, pf_bytes) : launch_one<0, EPI_ROPE_KV>(p, stream, pdl, smem, grid, nstages, pf_bytes);
    case EPI_SILU:
      LCU_REQUIRE(p.n_mats == 2, "gemv: SiLU-gate epilogue takes w1 and w3");
      return q ? launch_one<1, EPI_SILU>(p, stream, pdl, smem, grid, nstages, pf_bytes) : launch_one<0, EPI_SILU>(p, stream, pdl, smem, grid, nstages, pf_bytes);
  }
  LCU_REQUIRE(false, "gemv: unknown epilogue %d", epilogue);
}

}  // namespace lcu
