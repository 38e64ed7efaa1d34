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
// No multicast, no clusters.  Every mbarrier wait is bounded: on expiry the kernel records a code in
// the error word, skips ahead and still frees its tensor memory.
#include <cuda.h>

#include "gemm_tc.cuh"

namespace lcu {
namespace {

constexpr int BM = 128;      // output rows (tokens) per tile = TMEM lanes
constexpr int BK = 64;       // K per stage: 64 halves = one 128-byte swizzled row
constexpr int TC_THREADS = 192;

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 32 columns of fp32: thread t of the warp gets row (quadrant base + t), 32 consecutive columns
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// shared-memory matrix descriptor of a K-major tile stored as 128-byte swizzled rows:
// start address (16-byte units), leading byte offset 1 (unused for swizzled K-major), stride byte offset
// 1024 (eight 128-byte rows form one swizzle atom), descriptor version 1, layout type 2 = 128-byte swizzle
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                                __half* out, int m, int N, int K, float beta, int nstages, int* err) {
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE = A_BYTES + B_BYTES;
  // instruction descriptor: fp32 accumulate, fp16 x fp16, both K-major, N = BN, M = 128
  constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms are 1024-byte aligned
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)nstages * STAGE);  // full[8], empty[8], tmem_full
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  const int nk = K / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < nstages; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);
      mbar_init(smem_u32(&bars[8 + i]), 1);
    }
    mbar_init(smem_u32(&bars[16]), 1);
    fence_mbar_init();
  }
  if (warp == 1) {  // tensor-memory allocation: BN fp32 columns x 128 lanes
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer
      for (int kb = 0; kb < nk; ++kb) {
        const int s = kb % nstages, use = kb / nstages;
        if (use > 0 && !mbar_wait(smem_u32(&bars[8 + s]), (use - 1) & 1, err, DEV_ERR_EMPTY_WAIT)) break;
        const uint32_t full = smem_u32(&bars[s]);
        const uint32_t dst = base + (uint32_t)s * STAGE;
        mbar_arrive_expect_tx(full, STAGE);
        tma_load_2d(dst, &map_a, kb * BK, m0, full);
        tma_load_2d(dst + A_BYTES, &map_b, kb * BK, n0, full);
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
        const uint32_t a_addr = base + (uint32_t)s * STAGE;
        const uint64_t a_desc = smem_desc_sw128(a_addr), b_desc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)  // 16 halves = 32 bytes = 2 descriptor address units per K step
          tc_mma_f16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, IDESC, (kb | k) != 0);
        tc_commit(smem_u32(&bars[8 + s]));  // the stage is free once these MMAs have read it
      }
      tc_commit(smem_u32(&bars[16]));  // accumulator complete (also on the error path: lets the epilogue leave)
    }
  } else {
    // ---- epilogue: warp w may touch TMEM lanes 32 * (w % 4) ... + 31 only
    const int quad = warp & 3;
    const int row = m0 + quad * 32 + lane;
    const bool ok = mbar_wait(smem_u32(&bars[16]), 0, err, DEV_ERR_TMEM_WAIT);
    tc_fence_after();
    if (__all_sync(0xffffffffu, ok && *(volatile int*)err == 0)) {  // warp-uniform: tcgen05.ld is .aligned
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tc_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < m) {
          __half* o = out + (size_t)row * N + n0 + c;
          uint4 v[4];
          if (beta != 0.f) {
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = reinterpret_cast<const uint4*>(o)[i];
          }
          __half2* h = reinterpret_cast<__half2*>(v);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float a0 = __uint_as_float(r[2 * i]), a1 = __uint_as_float(r[2 * i + 1]);
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
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
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

// [rows][K] halves, row-major; box = box_rows x 64 halves with 128-byte swizzle; rows past the end read as zero
int make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t K, uint64_t ld, uint32_t box_rows, bool streamed) {
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
  return LCU_OK;
}

template <int BN>
int launch_bn(__half* out, const __half* lhs, int ldx, const __half* w, int m, int N, int K, float beta, int* err, cudaStream_t stream) {
  CUtensorMap map_a, map_b;
  int rc = make_map(&map_a, lhs, (uint64_t)m, (uint64_t)K, (uint64_t)ldx, BM, false);
  if (rc) return rc;
  rc = make_map(&map_b, w, (uint64_t)N, (uint64_t)K, (uint64_t)K, BN, true);
  if (rc) return rc;
  constexpr size_t STAGE = (size_t)(BM + BN) * BK * 2;
  int nstages = (int)((200 * 1024) / STAGE);
  if (nstages > 8) nstages = 8;
  if (nstages > K / BK) nstages = K / BK;
  const size_t smem = nstages * STAGE + 1024 /* alignment slack */ + 256 /* barriers, tmem slot */;
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_done[dev] = true;
  }
  const dim3 grid(N / BN, (m + BM - 1) / BM);
  gemm_tc_kernel<BN><<<grid, TC_THREADS, smem, stream>>>(map_a, map_b, out, m, N, K, beta, nstages, err);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

}  // namespace

bool gemm_tc_supported(int m, int N, int K, int ldx, const void* lhs, const void* w, const void* out) {
  return m >= 1 && N % 32 == 0 && K % BK == 0 && ldx % 8 == 0 && ((uintptr_t)lhs & 15) == 0 && ((uintptr_t)w & 15) == 0 &&
         ((uintptr_t)out & 15) == 0;
}

int launch_gemm_tc(__half* out, const __half* lhs, int ldx, const __half* w, int m, int N, int K, float beta, int* err, cudaStream_t stream,
                   int force_bn) {
  LCU_REQUIRE(gemm_tc_supported(m, N, K, ldx, lhs, w, out), "gemm_tc: unsupported shape m=%d N=%d K=%d ldx=%d or unaligned pointers", m, N, K, ldx);
  int bn = force_bn;
  if (!bn) bn = N % 128 == 0 ? 128 : N % 64 == 0 ? 64 : 32;  // measured: the widest tile wins even when it leaves SMs idle
  LCU_REQUIRE((bn == 32 || bn == 64 || bn == 128) && N % bn == 0, "gemm_tc: tile width %d does not divide N=%d", bn, N);
  if (bn == 128) return launch_bn<128>(out, lhs, ldx, w, m, N, K, beta, err, stream);
  if (bn == 64) return launch_bn<64>(out, lhs, ldx, w, m, N, K, beta, err, stream);
  return launch_bn<32>(out, lhs, ldx, w, m, N, K, beta, err, stream);
}

}  // namespace lcu
