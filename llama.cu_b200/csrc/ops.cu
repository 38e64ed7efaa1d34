// Row-wise and element-wise kernels of the forward pass, the quantizer and the data generator.
// Each kernel keeps the arithmetic (operation order inside an element, rounding points, libdevice
// functions) of the reference kernel it replaces, cited beside it.
#include "ops.cuh"

#include <algorithm>

#include <math_constants.h>

namespace lcu {
namespace {

template <typename F>
int launch_simple(F kernel_launch) {
  kernel_launch();
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

// ------------------------------------------------------------------ embedding (llama_cu.cu:32-62)
__global__ void embed_kernel(__half* x, int ldx, const void* table, const __half* scales, int bs, const short* ids, int dim) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const size_t id = (size_t)ids[r];
  if (bs == 0) {
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(table) + id * dim);
    uint4* dst = reinterpret_cast<uint4*>(x + (size_t)r * ldx);
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) dst[i] = src[i];
  } else {
    const uint8_t* src = reinterpret_cast<const uint8_t*>(table) + id * dim;
    const __half* sc = scales + id * (dim / bs);
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
      x[(size_t)r * ldx + i] = __float2half((float(src[i]) - 127.5f) * __half2float(sc[i / bs]));
  }
}

// ------------------------------------------------------------------ RMSNorm (llama_cu.cu:66-107)
// Same launch shape (one 256-thread block per row) and the same reduction order as the reference.
__global__ void __launch_bounds__(256) rms_norm_kernel(__half* out, const __half* in, const __half* weight, int w, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const __half* x = in + (size_t)row * w;
  __shared__ float s_warp[8];
  __shared__ float s_rinv;
  float s = 0.f;
  for (int i = tid; i < w; i += 256) {
    float v = __half2float(x[i]);
    s += v * v;
  }
  s = warp_sum(s);
  if (lane == 0) s_warp[warp] = s;
  __syncthreads();
  if (warp == 0) {
    float t = lane < 8 ? s_warp[lane] : 0.f;
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) s_rinv = rsqrtf(t / w + eps);
  }
  __syncthreads();
  const float rinv = s_rinv;
  for (int i = tid; i < w; i += 256) {
    float v = __half2float(x[i]);
    out[(size_t)row * w + i] = __hmul(weight[i], __float2half(v * rinv));
  }
}

// Same arithmetic and summation order with one trip to memory: every thread brings 16-byte vectors of the row into
// registers and into shared memory, the 256 strided partial sums of the reference are formed from shared memory, and the
// normalised row is written from the registers.  Rows of up to 8 * 256 * RN_VEC elements, 16-byte aligned.
constexpr int RN_VEC = 4;
__global__ void __launch_bounds__(256) rms_norm_vec_kernel(__half* out, const __half* in, const __half* weight, int w, float eps) {
  extern __shared__ __align__(16) uint8_t rn_row[];  // the row as halves
  __shared__ float s_warp[8];
  const int row = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int vec = w >> 3;
  pdl_launch_dependents();
  pdl_wait();
  const uint4* x = reinterpret_cast<const uint4*>(in + (size_t)row * w);
  uint4 xv[RN_VEC], wv[RN_VEC];
#pragma unroll
  for (int j = 0; j < RN_VEC; ++j) {
    const int i = tid + j * 256;
    if (i < vec) {
      xv[j] = x[i];
      wv[j] = reinterpret_cast<const uint4*>(weight)[i];
      reinterpret_cast<uint4*>(rn_row)[i] = xv[j];
    }
  }
  __syncthreads();
  const __half* xr = reinterpret_cast<const __half*>(rn_row);
  float s = 0.f;
  for (int i = tid; i < w; i += 256) {
    const float v = __half2float(xr[i]);
    s += v * v;
  }
  s = warp_sum(s);
  if (lane == 0) s_warp[warp] = s;
  __syncthreads();
  float t = lane < 8 ? s_warp[lane] : 0.f;  // every warp repeats the last tree
  for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  const float rinv = rsqrtf(__shfl_sync(0xffffffffu, t, 0) / w + eps);
#pragma unroll
  for (int j = 0; j < RN_VEC; ++j) {
    const int i = tid + j * 256;
    if (i < vec) {
      uint4 o = xv[j];
      __half2* o2 = reinterpret_cast<__half2*>(&o);
      const __half2* w2 = reinterpret_cast<const __half2*>(&wv[j]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(o2[e]);
        o2[e] = __hmul2(w2[e], __floats2half2_rn(f.x * rinv, f.y * rinv));
      }
      reinterpret_cast<uint4*>(out + (size_t)row * w)[i] = o;
    }
  }
}

// ------------------------------------------------------------------ RoPE (llama_cu.cu:368-389)
__global__ void rope_table_kernel(float2* table, int ctx_len, int head_dim, float theta, int first_pos) {
  const int half_dim = head_dim >> 1;
  const int idx = first_pos * half_dim + blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= ctx_len * half_dim) return;
  const int pos = idx / half_dim, i = idx - pos * half_dim;
  const int head_c = 2 * i;
  const float angle = pos / powf(theta, float(head_c) / head_dim);
  table[idx] = make_float2(cosf(angle), sinf(angle));
}

__global__ void rope_scatter_kernel(__half* q, const __half* k_new, const __half* v_new, __half* k_cache, __half* v_cache,
                                    const float2* rope, const int* pos_ptr, int pos_value, int m, int dim, int n_heads, int ctx_len, int ld) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y;
  const int c = 2 * (blockIdx.x * blockDim.x + threadIdx.x);
  if (c >= dim) return;
  const int hd = dim / n_heads;
  const int head = c / hd, j = c - head * hd;
  const int pos = (pos_ptr ? *pos_ptr : pos_value) + r;
  const float2 cs = rope[(size_t)pos * (hd >> 1) + (j >> 1)];
  const float a_cos = cs.x, a_sin = cs.y;
  const size_t src = (size_t)r * ld + c;
  const size_t dst = ((size_t)head * ctx_len + pos) * hd + j;
  {
    const float real = __half2float(q[src]), imag = __half2float(q[src + 1]);
    q[src] = __float2half(real * a_cos - imag * a_sin);
    q[src + 1] = __float2half(real * a_sin + imag * a_cos);
  }
  {
    const float real = __half2float(k_new[src]), imag = __half2float(k_new[src + 1]);
    k_cache[dst] = __float2half(real * a_cos - imag * a_sin);
    k_cache[dst + 1] = __float2half(real * a_sin + imag * a_cos);
  }
  *reinterpret_cast<__half2*>(v_cache + dst) = *reinterpret_cast<const __half2*>(v_new + src);
}

// Same arithmetic, eight consecutive columns (four rotation pairs, inside one head) per thread with 16-byte accesses.
__global__ void __launch_bounds__(128) rope_scatter_vec_kernel(__half* q, const __half* k_new, const __half* v_new, __half* k_cache, __half* v_cache,
                                                               const float2* rope, const int* pos_ptr, int pos_value, int m, int dim, int n_heads,
                                                               int ctx_len, int ld) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y;
  const int c = 8 * (blockIdx.x * blockDim.x + threadIdx.x);
  if (c >= dim) return;
  const int hd = dim / n_heads;
  const int head = c / hd, j = c - head * hd;
  const int pos = (pos_ptr ? *pos_ptr : pos_value) + r;
  const float4* tab = reinterpret_cast<const float4*>(rope + (size_t)pos * (hd >> 1) + (j >> 1));
  const float4 t0 = tab[0], t1 = tab[1];
  const float cs[4][2] = {{t0.x, t0.y}, {t0.z, t0.w}, {t1.x, t1.y}, {t1.z, t1.w}};
  const size_t src = (size_t)r * ld + c;
  const size_t dst = ((size_t)head * ctx_len + pos) * hd + j;
  auto rotate = [&](uint4 v) {
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float real = __low2float(h[e]), imag = __high2float(h[e]);
      h[e] = __halves2half2(__float2half(real * cs[e][0] - imag * cs[e][1]), __float2half(real * cs[e][1] + imag * cs[e][0]));
    }
    return v;
  };
  const uint4 qv = *reinterpret_cast<const uint4*>(q + src), kv = *reinterpret_cast<const uint4*>(k_new + src);
  const uint4 vv = *reinterpret_cast<const uint4*>(v_new + src);
  *reinterpret_cast<uint4*>(q + src) = rotate(qv);
  *reinterpret_cast<uint4*>(k_cache + dst) = rotate(kv);
  *reinterpret_cast<uint4*>(v_cache + dst) = vv;
}

// ------------------------------------------------------------------ SiLU gate (llama_cu.cu:533-539)
__global__ void silu_kernel(__half* out, const __half* a, const __half* b, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float val = __half2float(a[i]);
    out[i] = __float2half(val / (1.0f + expf(-val)) * __half2float(b[i]));
  }
}
// same arithmetic, eight elements per thread (16-byte loads and stores); n % 8 == 0 and 16-byte aligned pointers
__global__ void __launch_bounds__(256) silu8_kernel(__half* out, const __half* a, const __half* b, size_t n8) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 av = reinterpret_cast<const uint4*>(a)[i], bv = reinterpret_cast<const uint4*>(b)[i];
  const __half* ah = reinterpret_cast<const __half*>(&av);
  const __half* bh = reinterpret_cast<const __half*>(&bv);
  __align__(16) __half o[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float val = __half2float(ah[e]);
    o[e] = __float2half(val / (1.0f + expf(-val)) * __half2float(bh[e]));
  }
  reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<const uint4*>(o);
}

// ------------------------------------------------------------------ logits head
// softmax_rows with temperature (llama_cu.cu:433-499) followed by the host's first-maximum search
// over the half probabilities (llama_cu.cu:1205-1209), in one block.  The exp-sum keeps the
// reference's order: 256 strided partial sums, xor trees in 8 warps, xor tree over the warp sums.
constexpr int HEAD_THREADS = 1024;
__global__ void __launch_bounds__(HEAD_THREADS) logits_head_kernel(const head_params p, int cache_exp) {
  extern __shared__ float e_cache[];
  __shared__ float s_red[32];
  __shared__ int s_idx[32];
  __shared__ float s_bcast[2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int V = p.n_vocab;
  const float temp = p.temperature;
  pdl_launch_dependents();
  pdl_wait();

  float mx = -CUDART_INF_F;
  for (int i = tid; i < V; i += HEAD_THREADS) mx = fmaxf(mx, __half2float(p.logits[i]) / temp);
  mx = warp_max(mx);
  if (lane == 0) s_red[warp] = mx;
  __syncthreads();
  if (tid == 0) {
    float m = s_red[0];
    for (int w = 1; w < HEAD_THREADS / 32; ++w) m = fmaxf(m, s_red[w]);
    s_bcast[0] = m;
  }
  __syncthreads();
  mx = s_bcast[0];

  if (cache_exp)
    for (int i = tid; i < V; i += HEAD_THREADS) e_cache[i] = expf(__half2float(p.logits[i]) / temp - mx);
  __syncthreads();
  float sum = 0.f;
  if (tid < 256) {
    if (cache_exp)
      for (int i = tid; i < V; i += 256) sum += e_cache[i];
    else
      for (int i = tid; i < V; i += 256) sum += expf(__half2float(p.logits[i]) / temp - mx);
    sum = warp_sum(sum);
    if (lane == 0) s_red[warp] = sum;
  }
  __syncthreads();
  if (warp == 0) {
    float t = lane < 8 ? s_red[lane] : 0.f;
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) s_bcast[1] = t;
  }
  __syncthreads();
  sum = s_bcast[1];

  // probabilities (half), their maximum, and the first index that attains it
  float best = -1.f;
  int best_i = 0x7fffffff;
  for (int i = tid; i < V; i += HEAD_THREADS) {
    const float e = cache_exp ? e_cache[i] : expf(__half2float(p.logits[i]) / temp - mx);
    const __half ph = __float2half(e / sum);
    p.probs[i] = ph;
    const float pf = __half2float(ph);
    if (pf > best) {  // strided ascending i: keeps the first index of this thread's maximum
      best = pf;
      best_i = i;
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
    s_idx[warp] = best_i;
  }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < HEAD_THREADS / 32; ++w)
      if (s_red[w] > best || (s_red[w] == best && s_idx[w] < best_i)) {
        best = s_red[w];
        best_i = s_idx[w];
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

// ------------------------------------------------------------------ quantizer (transform.cu:28-87)
// One warp per (row, K-block).  scale = half(absmax / 127.5f); q = u8(roundf(127.5f + x / float(scale))).
__global__ void __launch_bounds__(256) quantize_kernel(uint8_t* q, __half* scales, const __half* in, size_t n_blocks, int bs) {
  const int lane = threadIdx.x & 31;
  const size_t warp0 = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const size_t nwarps = (size_t)gridDim.x * (blockDim.x >> 5);
  for (size_t blk = warp0; blk < n_blocks; blk += nwarps) {
    const __half* x = in + blk * bs;
    float absmax_val = 0;
    for (int i = lane * 4; i < bs; i += 128) {
      const uint2 raw = *reinterpret_cast<const uint2*>(x + i);
      const __half2* h = reinterpret_cast<const __half2*>(&raw);
      absmax_val = fmaxf(absmax_val, fabsf(__low2float(h[0])));
      absmax_val = fmaxf(absmax_val, fabsf(__high2float(h[0])));
      absmax_val = fmaxf(absmax_val, fabsf(__low2float(h[1])));
      absmax_val = fmaxf(absmax_val, fabsf(__high2float(h[1])));
    }
    absmax_val = warp_max(absmax_val);
    const __half s_absmax = __float2half(absmax_val / 127.5f);
    if (lane == 0) scales[blk] = s_absmax;
    const float sf = __half2float(s_absmax);
    for (int i = lane * 4; i < bs; i += 128) {
      const uint2 raw = *reinterpret_cast<const uint2*>(x + i);
      const __half* h = reinterpret_cast<const __half*>(&raw);
      uchar4 o;
      o.x = static_cast<uint8_t>(roundf(127.5f + __half2float(h[0]) / sf));
      o.y = static_cast<uint8_t>(roundf(127.5f + __half2float(h[1]) / sf));
      o.z = static_cast<uint8_t>(roundf(127.5f + __half2float(h[2]) / sf));
      o.w = static_cast<uint8_t>(roundf(127.5f + __half2float(h[3]) / sf));
      *reinterpret_cast<uchar4*>(q + blk * bs + i) = o;
    }
  }
}

__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// q = u8(roundf(127.5f + x / s)) costs an IEEE division and a roundf per element - about 25 instructions, which is what
// bounded the kernel at half the copy bandwidth.  For the inputs the quantizer can see - x a finite half, s a positive
// finite half, |x| within the absmax that rounds to s - the same byte comes out of a reciprocal multiply with one
// residual correction (the correctly rounded quotient) and trunc(v + 0.5f) for the non-negative v = 127.5f + quotient:
// 7 instructions.  "The same byte" is not argued, it is checked: quantizer_check_kernel compares the two for every such
// pair (2 x 10^9 of them) on the device, and tests/test_gpu_kernels.py requires zero differences.
__device__ __forceinline__ uint32_t quant_byte_reference(float x, float s) { return static_cast<uint8_t>(roundf(127.5f + x / s)); }
__device__ __forceinline__ uint32_t quant_byte_fast(float x, float s, float rcp) {
  const float t = x * rcp;
  const float quo = fmaf(fmaf(-t, s, x), rcp, t);
  return static_cast<uint8_t>(quo + 128.0f);  // trunc((127.5f + quo) + 0.5f) in one addition (conversion truncates); checked like the rest
}

// every (x, s) pair of the quantizer's domain: s = positive finite half number blockIdx.x * 256 + threadIdx.x..., x every
// finite half with |x| <= the largest absmax whose scale rounds to s.  counts[0] = pairs checked, counts[1] = differences.
__global__ void __launch_bounds__(256) quantizer_check_kernel(unsigned long long* counts) {
  unsigned long long checked = 0, diff = 0;
  for (uint32_t sb = blockIdx.x + 1; sb < 0x7c00u; sb += gridDim.x) {  // bit patterns of the positive finite halves
    const float s = __half2float(__ushort_as_half((unsigned short)sb));
    const float rcp = __frcp_rn(s);
    for (uint32_t xb = threadIdx.x; xb < 0x10000u; xb += 256) {
      if ((xb & 0x7c00u) == 0x7c00u) continue;  // inf / nan
      const __half xh = __ushort_as_half((unsigned short)xb);
      const float x = __half2float(xh);
      // in the domain iff a block with this absmax would get this scale
      if (__half_as_ushort(__float2half(fabsf(x) / 127.5f)) > sb) continue;
      ++checked;
      if (quant_byte_reference(x, s) != quant_byte_fast(x, s, rcp)) ++diff;
    }
  }
  checked = warp_sum_u64(checked);
  diff = warp_sum_u64(diff);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(counts, checked);
    atomicAdd(counts + 1, diff);
  }
}

// The same arithmetic with 16-byte loads: a thread holds eight consecutive halves in registers (read once), the
// BS / 8 neighbouring lanes that share a block agree on the block's absmax with xor shuffles, and every thread stores
// its eight bytes at once.  Block sizes 32 .. 256 (4 .. 32 lanes per block); n_vec = elements / 8.
template <int LANES>
__global__ void __launch_bounds__(256) quantize8_kernel(uint8_t* q, __half* scales, const __half* in, size_t n_vec) {
  constexpr int UNROLL = 2;  // vectors per thread whose loads are in flight together
  const size_t stride = (size_t)gridDim.x * 256;
  const size_t n_round = (n_vec + 31) / 32 * 32;  // whole warps take part in the shuffles
  for (size_t v0 = (size_t)blockIdx.x * 256 + threadIdx.x; v0 < n_round; v0 += UNROLL * stride) {
    uint4 raw[UNROLL];
#pragma unroll
    for (int r = 0; r < UNROLL; ++r) {
      const size_t v = v0 + r * stride;
      raw[r] = v < n_vec ? *reinterpret_cast<const uint4*>(in + v * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int r = 0; r < UNROLL; ++r) {
      const size_t v = v0 + r * stride;
      if (v >= n_round) break;  // (warp-uniform: v and n_round are multiples of 32 apart from the lane)
      const bool valid = v < n_vec;
      const __half2* h2 = reinterpret_cast<const __half2*>(&raw[r]);
      float f[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 p = __half22float2(h2[e]);
        f[2 * e] = p.x;
        f[2 * e + 1] = p.y;
      }
      // absmax on the packed halves (the maximum of halves is exact in any format; NaNs are passed over as fmaxf does)
      __half2 am2 = __hmax2(__hmax2(__habs2(h2[0]), __habs2(h2[1])), __hmax2(__habs2(h2[2]), __habs2(h2[3])));
      float absmax_val = fmaxf(0.f, fmaxf(__low2float(am2), __high2float(am2)));
#pragma unroll
      for (int o = LANES / 2; o > 0; o >>= 1) absmax_val = fmaxf(absmax_val, __shfl_xor_sync(0xffffffffu, absmax_val, o));
      const __half s_absmax = __float2half(absmax_val / 127.5f);
      const float sf = __half2float(s_absmax);
      if (!valid) continue;
      if ((v & (LANES - 1)) == 0) scales[v / LANES] = s_absmax;
      uint32_t lo = 0, hi = 0;
      if (sf > 0.f && absmax_val < CUDART_INF_F) {  // (block-uniform) the checked domain: finite values, positive scale
        const float rcp = __frcp_rn(sf);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          lo |= quant_byte_fast(f[e], sf, rcp) << (8 * e);
          hi |= quant_byte_fast(f[e + 4], sf, rcp) << (8 * e);
        }
      } else {  // an all-zero block (0 / 0), infinities or NaNs: the reference's own instructions
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          lo |= quant_byte_reference(f[e], sf) << (8 * e);
          hi |= quant_byte_reference(f[e + 4], sf) << (8 * e);
        }
      }
      *reinterpret_cast<uint2*>(q + v * 8) = make_uint2(lo, hi);
    }
  }
}

__global__ void __launch_bounds__(256) dequantize_kernel(__half* out, const __half* scales, const uint8_t* q, size_t n, int bs) {
  const size_t i4 = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 >= n) return;
  const uchar4 v = *reinterpret_cast<const uchar4*>(q + i4);
  const float s = __half2float(scales[i4 / bs]);  // bs % 4 == 0: the four share a block
  __half2 lo = __halves2half2(__float2half((float(v.x) - 127.5f) * s), __float2half((float(v.y) - 127.5f) * s));
  __half2 hi = __halves2half2(__float2half((float(v.z) - 127.5f) * s), __float2half((float(v.w) - 127.5f) * s));
  *reinterpret_cast<__half2*>(out + i4) = lo;
  *reinterpret_cast<__half2*>(out + i4 + 2) = hi;
}

// same, 16 weights per thread (one 16-byte load, two 16-byte stores); needs bs % 16 == 0
__global__ void __launch_bounds__(256) dequantize16_kernel(__half* out, const __half* scales, const uint8_t* q, size_t n, int bs) {
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 16;
  if (i >= n) return;
  const uint4 v = *reinterpret_cast<const uint4*>(q + i);
  const float s = __half2float(scales[i / bs]);
  const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
  __align__(16) __half2 o[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t u = wds[j];
    o[2 * j] = __halves2half2(__float2half((float(u & 0xff) - 127.5f) * s), __float2half((float((u >> 8) & 0xff) - 127.5f) * s));
    o[2 * j + 1] = __halves2half2(__float2half((float((u >> 16) & 0xff) - 127.5f) * s), __float2half((float(u >> 24) - 127.5f) * s));
  }
  reinterpret_cast<uint4*>(out + i)[0] = reinterpret_cast<const uint4*>(o)[0];
  reinterpret_cast<uint4*>(out + i)[1] = reinterpret_cast<const uint4*>(o)[1];
}

// error statistics (transform.cu:100-150) with a fixed-order two-stage reduction instead of float atomics
__global__ void __launch_bounds__(256) error_partial_kernel(float* partial, const __half* a, const __half* b, size_t n) {
  __shared__ float s_sq[8], s_mx[8], s_ab[8];
  float sq = 0, mx = 0, ab = 0;
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
    const float d = __half2float(a[i]) - __half2float(b[i]);
    sq += d * d;
    mx = fmaxf(mx, fabsf(d));
    ab += fabsf(d);
  }
  sq = warp_sum(sq);
  ab = warp_sum(ab);
  mx = warp_max(mx);
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) {
    s_sq[warp] = sq;
    s_mx[warp] = mx;
    s_ab[warp] = ab;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) {
      sq += s_sq[w];
      ab += s_ab[w];
      mx = fmaxf(mx, s_mx[w]);
    }
    partial[blockIdx.x * 3 + 0] = sq;
    partial[blockIdx.x * 3 + 1] = mx;
    partial[blockIdx.x * 3 + 2] = ab;
  }
}
__global__ void error_final_kernel(float* stats, const float* partial, int nparts, size_t n) {
  double sq = 0, ab = 0;
  float mx = 0;
  for (int i = 0; i < nparts; ++i) {
    sq += partial[i * 3];
    mx = fmaxf(mx, partial[i * 3 + 1]);
    ab += partial[i * 3 + 2];
  }
  stats[0] = (float)(sq / (double)n);
  stats[1] = mx;
  stats[2] = (float)(ab / (double)n);
}

// ------------------------------------------------------------------ synthetic data
// Philox4x32-10 block per element, keyed by the seed, counter = (index, stream id); the eight
// 16-bit lanes are summed (Irwin-Hall) and scaled to unit variance.  Integer arithmetic plus two
// binary32 multiplications: a host implementation of the same recipe yields identical bits.
__device__ __forceinline__ void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0;
    c[1] = lo1;
    c[2] = n2;
    c[3] = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}
__global__ void synth_kernel(__half* out, size_t n, uint64_t seed, uint64_t stream_id, float scale, uint64_t first) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t idx = first + i;
    uint32_t c[4] = {(uint32_t)idx, (uint32_t)(idx >> 32), (uint32_t)stream_id, (uint32_t)(stream_id >> 32)};
    philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
    int s = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) s += (int)(c[k] & 0xffffu) + (int)(c[k] >> 16);
    const float z = __fmul_rn((float)(s - 262140), 0x1.3988e2p-16f);  // 1 / sqrt(8 * (65536^2 - 1) / 12)
    out[i] = __float2half(__fmul_rn(z, scale));
  }
}
__global__ void bump_pos_kernel(int* pos, int inc) { *pos += inc; }
__global__ void token_to_ids_kernel(short* ids, const int* token) { ids[0] = (short)*token; }
__global__ void fill_half_kernel(__half* out, size_t n, __half v) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = v;
}

}  // namespace

uint64_t fnv1a64(const char* s) {
  uint64_t h = 0xcbf29ce484222325ull;
  for (; *s; ++s) {
    h ^= (uint8_t)*s;
    h *= 0x100000001b3ull;
  }
  return h;
}

int launch_embed(__half* x, int ldx, const void* table, const __half* scales, int bs, const short* ids, int n_ids, int dim,
                 cudaStream_t stream, int pdl) {
  LCU_REQUIRE(dim % 8 == 0 && ldx % 8 == 0, "embed: dim must be a multiple of 8");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_ids);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  LCU_CUDA(cudaLaunchKernelEx(&cfg, embed_kernel, x, ldx, table, scales, bs, ids, dim));
  return LCU_OK;
}

int launch_rms_norm(__half* out, const __half* in, const __half* weight, int rows, int dim, float eps, cudaStream_t stream) {
  if (dim % 8 == 0 && dim <= 8 * 256 * RN_VEC && ((((uintptr_t)out | (uintptr_t)in | (uintptr_t)weight)) & 15) == 0)
    LCU_CUDA(launch_after(rms_norm_vec_kernel, dim3(rows), dim3(256), (size_t)dim * 2, stream, out, in, weight, dim, eps));
  else
    LCU_CUDA(launch_after(rms_norm_kernel, dim3(rows), dim3(256), 0, stream, out, in, weight, dim, eps));
  return LCU_OK;
}

int launch_rope_table(float2* table, int ctx_len, int head_dim, float theta, cudaStream_t stream, int first_pos) {
  const int n = (ctx_len - first_pos) * (head_dim / 2);
  if (n <= 0) return LCU_OK;
  rope_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(table, ctx_len, head_dim, theta, first_pos);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

int launch_rope_scatter(__half* q, const __half* k_new, const __half* v_new, __half* k_cache, __half* v_cache,
                        const float2* rope, const int* pos, int pos_value, int m, int dim, int n_heads, int ctx_len,
                        cudaStream_t stream, int ld) {
  const int row_ld = ld > 0 ? ld : dim;
  const int hd = dim / n_heads;
  const uintptr_t all = (uintptr_t)q | (uintptr_t)k_new | (uintptr_t)v_new | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)rope;
  if (hd % 8 == 0 && row_ld % 8 == 0 && (all & 15) == 0) {
    dim3 grid((dim / 8 + 127) / 128, m);
    LCU_CUDA(launch_after(rope_scatter_vec_kernel, grid, dim3(128), 0, stream, q, k_new, v_new, k_cache, v_cache, rope, pos, pos_value, m, dim, n_heads,
                          ctx_len, row_ld));
  } else {
    dim3 grid((dim / 2 + 127) / 128, m);
    LCU_CUDA(launch_after(rope_scatter_kernel, grid, dim3(128), 0, stream, q, k_new, v_new, k_cache, v_cache, rope, pos, pos_value, m, dim, n_heads, ctx_len,
                          row_ld));
  }
  return LCU_OK;
}

// rows of [a | b] pairs: out[r][j] = silu(ab[r][j]) * ab[r][f + j], f % 8 == 0
__global__ void __launch_bounds__(256) silu_rows_kernel(__half* out, const __half* ab, int m, int f) {
  pdl_launch_dependents();
  pdl_wait();
  const int fv = f >> 3;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)m * fv) return;
  const size_t r = i / fv, jv = i - r * fv;
  const uint4 av = reinterpret_cast<const uint4*>(ab + r * 2 * f)[jv], bv = reinterpret_cast<const uint4*>(ab + r * 2 * f + f)[jv];
  const __half* ah = reinterpret_cast<const __half*>(&av);
  const __half* bh = reinterpret_cast<const __half*>(&bv);
  __align__(16) __half o[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float val = __half2float(ah[e]);
    o[e] = __float2half(val / (1.0f + expf(-val)) * __half2float(bh[e]));
  }
  reinterpret_cast<uint4*>(out + r * f)[jv] = *reinterpret_cast<const uint4*>(o);
}

// Self-test of the bounded wait every pipeline in this library relies on: one warp waits on an mbarrier that nothing
// will ever complete.  The wait gives up after about a second of SM clock, records its code and the kernel ends.
__global__ void bounded_wait_probe_kernel(int* err) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  __syncthreads();
  mbar_wait(smem_u32(&bar), 0, err, DEV_ERR_FULL_WAIT);
}

int run_bounded_wait_probe(int* err_word, cudaStream_t stream) {
  bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(err_word);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

int launch_silu_rows(__half* out, const __half* ab, int m, int f, cudaStream_t stream) {
  LCU_REQUIRE(f % 8 == 0 && (((uintptr_t)out | (uintptr_t)ab) & 15) == 0, "silu_rows: rows of %d elements are not 16-byte vectors", f);
  const size_t n = (size_t)m * (f / 8);
  LCU_CUDA(launch_after(silu_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, out, ab, m, f));
  return LCU_OK;
}

// ------------------------------------------------------------------ matmul_type 1: the pedantic product
// The reference keeps a pair of deliberately plain kernels as "a trivial reference point for optimized kernels"
// (llama_cu.cu:110-145) and runs them when matmul_type == 1.  Same contract here: one thread owns one output element
// and adds its K terms strictly in index order.  fp16 weights: binary32 running sum (a product of two halves is exact
// in binary32).  u8 weights: every term x * (q - 127.5) * scale is formed in binary64 - the reference's 127.5 literal is
// a double - added to the running sum in binary64, and the sum is rounded back to binary32 after each addition.
__global__ void __launch_bounds__(256) pedantic_matmul_f16_kernel(__half* out, const __half* lhs, const __half* w, int m, int k, int n, float beta) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)m * n) return;
  const __half* x = lhs + (idx / n) * (size_t)k;
  const __half* wr = w + (idx % n) * (size_t)k;
  float acc = 0.f;
  for (const __half* end = x + k; x != end; ++x, ++wr) acc = __fmaf_rn(__half2float(*x), __half2float(*wr), acc);
  out[idx] = __float2half(beta == 0.f ? acc : __fmaf_rn(beta, __half2float(out[idx]), acc));
}
__global__ void __launch_bounds__(256) pedantic_matmul_u8_kernel(__half* out, const __half* lhs, const uint8_t* q, const __half* scales, int m, int k,
                                                                 int n, int bs, float beta) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)m * n) return;
  const size_t row = idx % n;
  const __half* x = lhs + (idx / n) * (size_t)k;
  const uint8_t* qr = q + row * (size_t)k;
  const __half* sr = scales + row * (size_t)(k / bs);
  float acc = 0.f;
  for (int b = 0; b < k / bs; ++b) {
    const double scale = (double)__half2float(sr[b]);
    for (int i = b * bs; i < (b + 1) * bs; ++i) {
      const double term = __dmul_rn(__dmul_rn((double)__half2float(x[i]), (double)(float)qr[i] - 127.5), scale);
      acc = (float)__dadd_rn((double)acc, term);
    }
  }
  out[idx] = __float2half(beta == 0.f ? acc : __fmaf_rn(beta, __half2float(out[idx]), acc));
}

int launch_matmul_nt_pedantic(__half* out, const __half* lhs, const void* w, const __half* scales, int bs, int m, int k, int n, float beta,
                              cudaStream_t stream) {
  LCU_REQUIRE(m >= 1 && k >= 1 && n >= 1, "matmul_nt (pedantic): empty shape %d x %d x %d", m, k, n);
  LCU_REQUIRE(bs == 0 || (bs > 0 && k % bs == 0 && scales != nullptr), "matmul_nt (pedantic): block size %d does not divide K=%d", bs, k);
  const unsigned grid = (unsigned)(((size_t)m * n + 255) / 256);
  if (bs == 0)
    pedantic_matmul_f16_kernel<<<grid, 256, 0, stream>>>(out, lhs, (const __half*)w, m, k, n, beta);
  else
    pedantic_matmul_u8_kernel<<<grid, 256, 0, stream>>>(out, lhs, (const uint8_t*)w, scales, m, k, n, bs, beta);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

int launch_silu(__half* out, const __half* a, const __half* b, size_t n, cudaStream_t stream) {
  if (n % 8 == 0 && (((uintptr_t)out | (uintptr_t)a | (uintptr_t)b) & 15) == 0)
    silu8_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, stream>>>(out, a, b, n / 8);
  else
    silu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(out, a, b, n);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

int launch_logits_head_single(const head_params& p, cudaStream_t stream, int pdl) {
  static bool attr_done[16] = {};
  int dev = 0;
  LCU_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !attr_done[dev]) {
    LCU_CUDA(cudaFuncSetAttribute(logits_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_done[dev] = true;
  }
  const size_t need = (size_t)p.n_vocab * sizeof(float);
  const int cache_exp = need <= 200 * 1024;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(HEAD_THREADS);
  cfg.dynamicSmemBytes = cache_exp ? need : 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  LCU_CUDA(cudaLaunchKernelEx(&cfg, logits_head_kernel, p, cache_exp));
  return LCU_OK;
}

int launch_quantize_absmax_uint8(uint8_t* q, __half* scales, const __half* in, size_t h, size_t w, int bs, cudaStream_t stream) {
  LCU_REQUIRE(bs > 0 && bs % 4 == 0 && w % bs == 0, "quantize: block size %d must be a multiple of 4 that divides the row length %zu", bs, w);
  LCU_REQUIRE(((uintptr_t)in & 7) == 0 && ((uintptr_t)q & 3) == 0, "quantize: buffers must be 8-byte (input) and 4-byte (output) aligned");
  const size_t n_blocks = h * (w / bs);
  if (n_blocks == 0) return LCU_OK;
  const bool vec_ok = (((uintptr_t)in & 15) | ((uintptr_t)q & 7)) == 0;
  if (vec_ok && (bs == 32 || bs == 64 || bs == 128 || bs == 256)) {
    const size_t n_vec = n_blocks * (size_t)(bs / 8);
    size_t grid8 = (n_vec + 255) / 256;
    if (grid8 > 148 * 8) grid8 = 148 * 8;
    if (bs == 32) quantize8_kernel<4><<<(unsigned)grid8, 256, 0, stream>>>(q, scales, in, n_vec);
    else if (bs == 64) quantize8_kernel<8><<<(unsigned)grid8, 256, 0, stream>>>(q, scales, in, n_vec);
    else if (bs == 128) quantize8_kernel<16><<<(unsigned)grid8, 256, 0, stream>>>(q, scales, in, n_vec);
    else quantize8_kernel<32><<<(unsigned)grid8, 256, 0, stream>>>(q, scales, in, n_vec);
    LCU_CUDA(cudaGetLastError());
    return LCU_OK;
  }
  size_t grid = (n_blocks + 7) / 8;
  if (grid > 148 * 16) grid = 148 * 16;
  quantize_kernel<<<(unsigned)grid, 256, 0, stream>>>(q, scales, in, n_blocks, bs);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

// every half-precision a: silu_of_half against the division it replaces, bit for bit (NaN = NaN)
__global__ void silu_check_kernel(unsigned long long* counts) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 65536u) return;
  const float a = __half2float(__ushort_as_half((unsigned short)i));
  const float want = a / (1.0f + expf(-a)), got = silu_of_half(a);
  const bool same = (want != want && got != got) || __float_as_uint(want) == __float_as_uint(got);
  atomicAdd(counts, 1ull);
  if (!same) atomicAdd(counts + 1, 1ull);
}

int silu_arithmetic_check(unsigned long long* checked_out, unsigned long long* differences_out) {
  unsigned long long* d = nullptr;
  LCU_CUDA(cudaMalloc(&d, 16));
  LCU_CUDA(cudaMemset(d, 0, 16));
  silu_check_kernel<<<256, 256>>>(d);
  unsigned long long h[2] = {0, 0};
  cudaError_t e = cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
  cudaFree(d);
  LCU_CUDA(e);
  *checked_out = h[0];
  *differences_out = h[1];
  return LCU_OK;
}

int quantizer_arithmetic_check(unsigned long long* checked_out, unsigned long long* differences_out) {
  unsigned long long* d = nullptr;
  LCU_CUDA(cudaMalloc(&d, 16));
  LCU_CUDA(cudaMemset(d, 0, 16));
  quantizer_check_kernel<<<148 * 4, 256>>>(d);
  unsigned long long h[2] = {0, 0};
  cudaError_t e = cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
  cudaFree(d);
  LCU_CUDA(e);
  *checked_out = h[0];
  *differences_out = h[1];
  return LCU_OK;
}

int launch_dequantize_absmax_uint8(__half* out, const __half* scales, const uint8_t* q, size_t h, size_t w, int bs,
                                   cudaStream_t stream) {
  LCU_REQUIRE(bs > 0 && bs % 4 == 0 && w % bs == 0, "dequantize: block size %d must be a multiple of 4 that divides the row length %zu", bs, w);
  const size_t n = h * w;
  if (n == 0) return LCU_OK;
  if (bs % 16 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0)
    dequantize16_kernel<<<(unsigned)((n / 16 + 255) / 256), 256, 0, stream>>>(out, scales, q, n, bs);
  else
    dequantize_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, stream>>>(out, scales, q, n, bs);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

int launch_error_stats(float* stats, float* partial, const __half* a, const __half* b, size_t n, cudaStream_t stream) {
  error_partial_kernel<<<256, 256, 0, stream>>>(partial, a, b, n);
  error_final_kernel<<<1, 1, 0, stream>>>(stats, partial, 256, n);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

int launch_synth_fill(__half* out, size_t n, uint64_t seed, uint64_t stream_id, float scale, uint64_t first, cudaStream_t stream) {
  if (n == 0) return LCU_OK;
  size_t grid = (n + 255) / 256;
  if (grid > 148 * 32) grid = 148 * 32;
  synth_kernel<<<(unsigned)grid, 256, 0, stream>>>(out, n, seed, stream_id, scale, first);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

// ------------------------------------------------------------------ sampler
// The reference's next_token ends in `std::discrete_distribution<short> dist(probs.begin(), probs.end()); return dist(rng_);`
// - commented out in favour of the argmax (llama_cu.cu:1202-1209).  Same distribution here, on the device: token i
// with probability float(p_i) / sum_j float(p_j) over the fp16 probabilities, chosen by inverting the cumulative sum at
// u * total.  Every sum is binary32 in a fixed order (32-element chunks in index order, then the chunk sums in index
// order), so a host restatement gives the same token for the same u.
__device__ __host__ inline float sampler_uniform_from(uint32_t word) { return (float)(word >> 8) * 0x1p-24f; }  // [0, 1)

__global__ void __launch_bounds__(1024) sample_kernel(const __half* probs, int n, uint64_t seed, const int* index_ptr, float u_given, int* token_out,
                                                      short* next_ids, short* log, const int* step, int log_capacity) {
  __shared__ float chunk[1024];
  __shared__ int s_pick;
  __shared__ float s_before, s_target;
  const int tid = threadIdx.x;
  const int per = (n + 1023) / 1024;  // elements per chunk
  const int lo = tid * per, hi = min(n, lo + per);
  float s = 0.f;
  for (int i = lo; i < hi; ++i) s += __half2float(probs[i]);
  chunk[tid] = s;
  __syncthreads();
  if (tid == 0) {
    float u = u_given;
    if (index_ptr != nullptr) {  // counter-based: one Philox block per (seed, index)
      uint32_t c[4] = {(uint32_t)*index_ptr, 0u, 0x73616d70u, 0x6c657221u};
      philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
      u = sampler_uniform_from(c[0]);
    }
    float total = 0.f;
    for (int c = 0; c < 1024; ++c) total += chunk[c];
    const float target = u * total;
    float run = 0.f;
    int pick = -1;
    for (int c = 0; c < 1024; ++c) {
      if (run + chunk[c] > target) {
        pick = c;
        break;
      }
      run += chunk[c];
    }
    s_pick = pick;
    s_before = run;
    s_target = target;
  }
  __syncthreads();
  if (tid == 0) {
    int token = -1;
    if (s_pick >= 0) {
      float run = s_before;
      const int c_lo = s_pick * per, c_hi = min(n, c_lo + per);
      for (int i = c_lo; i < c_hi; ++i) {
        const float w = __half2float(probs[i]);
        run += w;
        if (run > s_target && w > 0.f) {
          token = i;
          break;
        }
      }
    }
    if (token < 0)  // rounding left the target at or past the total: the last token with a non-zero probability
      for (int i = n - 1; i >= 0; --i)
        if (__half2float(probs[i]) > 0.f) {
          token = i;
          break;
        }
    if (token < 0) token = 0;
    if (token_out) *token_out = token;
    if (next_ids) next_ids[0] = (short)token;
    if (log && step && *step >= 1 && *step - 1 < log_capacity) log[*step - 1] = (short)token;  // over the head's argmax entry
  }
}

// block rotation of cached keys for a context roll-over: key rows [first, first + keep) of every head move to positions
// [0, keep), each pair (2i, 2i+1) rotated back by `first` positions (the angle of llama_cu.cu:375-388 with pos = -first),
// value rows move unchanged.  One CTA per (destination position, head); in-place is safe row by row in ascending order
// only when first > 0, so the kernel reads from the source row into registers before any thread writes the destination
// row of another CTA is touched: rows are disjoint per CTA and destination < source.
__global__ void rollover_kernel(__half* k_cache, __half* v_cache, int ctx_len, int head_dim, int first, float theta) {
  const int dst = blockIdx.x, head = blockIdx.y, src = dst + first;
  __half* kd = k_cache + ((size_t)head * ctx_len + dst) * head_dim;
  const __half* ks = k_cache + ((size_t)head * ctx_len + src) * head_dim;
  __half* vd = v_cache + ((size_t)head * ctx_len + dst) * head_dim;
  const __half* vs = v_cache + ((size_t)head * ctx_len + src) * head_dim;
  for (int i = threadIdx.x; i < head_dim / 2; i += blockDim.x) {
    const float re = __half2float(ks[2 * i]), im = __half2float(ks[2 * i + 1]);
    const float angle = -(float)first / powf(theta, float(2 * i) / head_dim);
    const float c = cosf(angle), sn = sinf(angle);
    const __half v0 = vs[2 * i], v1 = vs[2 * i + 1];
    kd[2 * i] = __float2half(re * c - im * sn);
    kd[2 * i + 1] = __float2half(re * sn + im * c);
    vd[2 * i] = v0;
    vd[2 * i + 1] = v1;
  }
}

// loads the small kernels of a decode step on the current device ahead of their first launch
int ops_preload() {
  cudaFuncAttributes fa;
  LCU_CUDA(cudaFuncGetAttributes(&fa, embed_kernel));
  LCU_CUDA(cudaFuncGetAttributes(&fa, bump_pos_kernel));
  LCU_CUDA(cudaFuncGetAttributes(&fa, token_to_ids_kernel));
  LCU_CUDA(cudaFuncGetAttributes(&fa, logits_head_kernel));
  return LCU_OK;
}

int launch_sample(const __half* probs, int n_vocab, uint64_t seed, const int* index, float u, int* token_out, short* next_ids, short* log,
                  const int* step, int log_capacity, cudaStream_t stream) {
  LCU_REQUIRE(n_vocab >= 1 && probs != nullptr, "sample: empty distribution");
  sample_kernel<<<1, 1024, 0, stream>>>(probs, n_vocab, seed, index, u, token_out, next_ids, log, step, log_capacity);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

float sampler_uniform(uint64_t seed, int index) {
  uint32_t c[4] = {(uint32_t)index, 0u, 0x73616d70u, 0x6c657221u};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) {  // Philox4x32-10, as philox4x32_10 on the device
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
    c[0] = n0; c[1] = (uint32_t)p1; c[2] = n2; c[3] = (uint32_t)p0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return sampler_uniform_from(c[0]);
}

// Rows are processed in ascending destination order by independent CTAs; a CTA's source row (dst + first) may be the
// destination row of a later CTA, so the move runs in waves of `first` rows: wave w moves rows [w*first, (w+1)*first),
// whose sources [(w+1)*first, (w+2)*first) no earlier wave has written.
int launch_rollover(__half* k_cache, __half* v_cache, int n_heads, int ctx_len, int head_dim, int first, int keep, float theta, cudaStream_t stream) {
  LCU_REQUIRE(first >= 1 && keep >= 1 && first + keep <= ctx_len, "rollover: rows %d..%d outside the context length %d", first, first + keep, ctx_len);
  for (int done = 0; done < keep; done += first) {
    const int rows = std::min(first, keep - done);
    const size_t off = (size_t)done * head_dim;  // shifts both source and destination by `done` rows
    rollover_kernel<<<dim3(rows, n_heads), 64, 0, stream>>>(k_cache + off, v_cache + off, ctx_len, head_dim, first, theta);
  }
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

int launch_bump_pos(int* pos, int inc, cudaStream_t stream) {
  bump_pos_kernel<<<1, 1, 0, stream>>>(pos, inc);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}
int launch_token_to_ids(short* ids, const int* token, cudaStream_t stream) {
  token_to_ids_kernel<<<1, 1, 0, stream>>>(ids, token);
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

int launch_fill_half(__half* out, size_t n, float value, cudaStream_t stream) {
  if (n == 0) return LCU_OK;
  size_t grid = (n + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  fill_half_kernel<<<(unsigned)grid, 256, 0, stream>>>(out, n, __float2half(value));
  LCU_CUDA(cudaGetLastError());
  return LCU_OK;
}

}  // namespace lcu
