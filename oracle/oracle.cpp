// CPU oracle for the llama.cu forward pass, quantizer and synthetic-weight generator.
//
// TEST INFRASTRUCTURE ONLY.  This file is a scalar host restatement of the arithmetic that
// eiz/llama.cu performs in its CUDA kernels; it exists so that the sm_100a kernels can be checked
// against an independent implementation.  Nothing in the shipped library links, includes or calls
// it: only the test-suite, the smoke check and the benchmark's cpu_baseline leg load it.
//
// Pinning: the reference ships no tests or golden vectors, so this restatement is pinned by
// vectors produced by running the reference's own kernels on a B200 (tests/golden/*.json, made by
// tests/golden/make_golden.py) - quantizer bytes, single-matmul outputs and greedy token streams.
//
// Every function cites the reference lines it restates (paths relative to the reference repo).
// All storage is IEEE binary16 held in uint16_t; arithmetic is binary32 unless the reference
// itself uses double.  Built with -ffp-contract=off: fused multiply-adds appear only where they
// are written out with fmaf(), at the places where nvcc contracts the reference's expressions.

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---------------------------------------------------------------- binary16 <-> binary32
float g_h2f[65536];
bool g_h2f_ready = false;

float h2f_slow(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while ((man & 0x400u) == 0);
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

void init_tables() {
  if (g_h2f_ready) return;
  for (uint32_t i = 0; i < 65536; ++i) g_h2f[i] = h2f_slow((uint16_t)i);
  g_h2f_ready = true;
}

inline float h2f(uint16_t h) { return g_h2f[h]; }

// round-to-nearest-even binary32 -> binary16 (what __float2half / __float2half_rn do)
inline uint16_t f2h(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  x &= 0x7fffffffu;
  if (x > 0x7f800000u) return 0x7fffu;               // NaN (CUDA returns the canonical 0x7fff)
  if (x >= 0x477ff000u) return sign | 0x7c00u;        // >= 65520 rounds to inf
  if (x >= 0x38800000u) {                             // normal half
    uint32_t man = x & 0x7fffffu;
    uint32_t h = (((x >> 23) - 112u) << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return sign | (uint16_t)h;
  }
  if (x < 0x33000000u) return sign;                   // < 2^-25 rounds to zero (tie at 2^-25 -> even = 0)
  uint32_t man = (x & 0x7fffffu) | 0x800000u;
  uint32_t shift = 126u - (x >> 23);                  // 14..24: man >> shift is in units of 2^-24
  uint32_t h = man >> shift;
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (h & 1u))) ++h;
  return sign | (uint16_t)h;
}

// ---------------------------------------------------------------- synthetic data generator
// Counter-based: Philox4x32-10 keyed by the seed, counter = (element index, stream id) where the
// stream id is the FNV-1a hash of the tensor name.  The eight 16-bit lanes of one Philox block are
// summed (Irwin-Hall, n = 8) to an approximately normal variate; only integer arithmetic and two
// binary32 multiplications are involved, so host and device produce identical bits.
inline void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
  for (int r = 0; r < 10; ++r) {
    uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
    uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
    uint32_t n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
    uint32_t n3 = (uint32_t)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

uint64_t fnv1a64(const char* s) {
  uint64_t h = 0xcbf29ce484222325ull;
  for (; *s; ++s) {
    h ^= (uint8_t)*s;
    h *= 0x100000001b3ull;
  }
  return h;
}

// 1 / sqrt(8 * (65536^2 - 1) / 12): scales the centred 8-lane sum to unit variance
const float kIrwinHallScale = 0x1.3988e2p-16f;  // 1.8688124e-05

inline uint16_t synth_half(uint64_t seed, uint64_t stream, uint64_t idx, float scale) {
  uint32_t c[4] = {(uint32_t)idx, (uint32_t)(idx >> 32), (uint32_t)stream, (uint32_t)(stream >> 32)};
  philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
  int32_t s = 0;
  for (int i = 0; i < 4; ++i) s += (int32_t)(c[i] & 0xffffu) + (int32_t)(c[i] >> 16);
  float z = (float)(s - 262140) * kIrwinHallScale;
  return f2h(z * scale);
}

// ---------------------------------------------------------------- model structures
#pragma pack(push, 1)
struct params_t {  // llama_cu.h:280-291, extract.py:30-41 ("<QIiiiiifi")
  uint64_t magic;
  uint32_t fourcc;
  uint32_t dim, multiple_of, n_heads, n_layers, n_vocab;
  float norm_eps;
  uint8_t q_type;
  uint8_t reserved0;
  uint16_t block_size;
};
#pragma pack(pop)
static_assert(sizeof(params_t) == 40, "params file is 40 bytes");

struct weight_t {  // fp16 matrix, or u8 matrix + fp16 per-block scales (llama_cu.h:252-270)
  size_t h = 0, w = 0;
  int bs = 0;  // 0 = fp16
  std::vector<uint16_t> f16;
  std::vector<uint8_t> q;
  std::vector<uint16_t> scales;
};

struct layer_t {
  weight_t wq, wk, wv, wo, w1, w2, w3;
  std::vector<uint16_t> attn_norm, ffn_norm;
};

struct model_t {
  params_t p;
  uint32_t ffn;
  weight_t tok_embeddings, output;
  std::vector<uint16_t> norm;
  std::vector<layer_t> layers;
};

struct context_t {
  model_t* m;
  int ctx_len;
  float temperature;
  int start_pos = 0;
  int wmma_rounding = 1;   // 1: int8 weights rounded to half before the product (matmul_type 4)
  int fp32_attention = 0;  // 1: keep scores/probabilities in binary32 (not what the reference does)
  std::vector<std::vector<uint16_t>> k_cache, v_cache;  // [layer][ctx*dim], K stored un-rotated
  std::vector<uint16_t> probs;                          // last softmax output (n_vocab)
  std::vector<uint16_t> logits;                         // last logits before softmax (n_vocab)
  std::vector<uint16_t> last_hidden;                    // residual stream of the last new token
  double t_layers = 0, t_head = 0;                      // wall seconds of the last call: layer loop / final norm + logits + softmax
};

uint32_t ffn_dim(const params_t& p) {  // llama_cu.cu:765-767 (integer division first)
  uint32_t a = p.dim * 8 / 3;
  return (a + p.multiple_of - 1) / p.multiple_of * p.multiple_of;
}

// ---------------------------------------------------------------- operators
// llama_cu.cu:287-289  half((float(q) - 127.5f) * float(scale))
inline uint16_t dequant_one(uint8_t q, uint16_t scale) { return f2h(((float)q - 127.5f) * h2f(scale)); }

// llama_cu.cu:66-107.  Sum of squares in binary32 (nvcc contracts `sum += v*v` to an fma),
// r = rsqrt(sum/w + eps), out = weight *_half half(x * r).
void rms_norm(uint16_t* out, const uint16_t* in, const uint16_t* weight, int h, int w, float eps) {
  for (int r = 0; r < h; ++r) {
    const uint16_t* x = in + (size_t)r * w;
    // the kernel's summation order: 256 threads stride the row, then xor-shuffle trees
    float part[256];
    for (int t = 0; t < 256; ++t) {
      float s = 0.f;
      for (int i = t; i < w; i += 256) s = fmaf(h2f(x[i]), h2f(x[i]), s);
      part[t] = s;
    }
    float warp[8];
    for (int wi = 0; wi < 8; ++wi) {
      float v[32];
      for (int l = 0; l < 32; ++l) v[l] = part[wi * 32 + l];
      for (int off = 16; off > 0; off /= 2) {
        float n[32];
        for (int l = 0; l < 32; ++l) n[l] = v[l] + v[l ^ off];
        memcpy(v, n, sizeof v);
      }
      warp[wi] = v[0];
    }
    float v[8];
    memcpy(v, warp, sizeof v);
    for (int off = 4; off > 0; off /= 2) {
      float n[8];
      for (int l = 0; l < 8; ++l) n[l] = v[l] + v[l ^ off];
      memcpy(v, n, sizeof v);
    }
    float rinv = 1.0f / sqrtf(v[0] / (float)w + eps);
    for (int i = 0; i < w; ++i) {
      uint16_t xn = f2h(h2f(x[i]) * rinv);
      out[(size_t)r * w + i] = f2h(h2f(weight[i]) * h2f(xn));  // __hmul: exact product, one rounding
    }
  }
}

// llama_cu.cu:111-122 (naive kernel = the specification of matmul_nt).
// out(m,n) = half( sum_k float(lhs[r,k]) * float(rhs[c,k])  + beta * float(out) ), binary32 sum in k order.
// acc64 != 0 evaluates the sum in double instead ("gold" evaluation for error metrics).
void matmul_nt_f16(uint16_t* out, const uint16_t* lhs, const uint16_t* rhs, int m, int k, int n, float beta, int acc64) {
#pragma omp parallel for schedule(static)
  for (int c = 0; c < n; ++c) {
    const uint16_t* w = rhs + (size_t)c * k;
    for (int r = 0; r < m; ++r) {
      const uint16_t* x = lhs + (size_t)r * k;
      float res;
      if (acc64) {
        double s = 0;
        for (int i = 0; i < k; ++i) s += (double)h2f(x[i]) * (double)h2f(w[i]);
        res = (float)s;
      } else {
        float s = 0;
        for (int i = 0; i < k; ++i) s += h2f(x[i]) * h2f(w[i]);  // products of two halves are exact
        res = s;
      }
      size_t o = (size_t)r * n + c;
      out[o] = f2h(beta == 0.f ? res : fmaf(beta, h2f(out[o]), res));
    }
  }
}

// int8-weight product.  mode 0: weights rounded to half first (llama_cu.cu:287-289, 332-341: the
// tensor-core kernel, matmul_type 4).  mode 1: the naive kernel llama_cu.cu:125-145 whose
// `127.5` literal is a double, so each term is evaluated in double and added to a float sum.
// mode 2: double accumulation over the half-rounded weights; mode 3: double accumulation over the
// un-rounded (q-127.5)*scale ("gold" evaluations).
void matmul_nt_fp16u8(uint16_t* out, const uint16_t* lhs, const uint8_t* q, const uint16_t* scales, int m, int k,
                      int n, int bs, float beta, int mode) {
  int nb = k / bs;
#pragma omp parallel for schedule(static)
  for (int c = 0; c < n; ++c) {
    const uint8_t* wq = q + (size_t)c * k;
    const uint16_t* sc = scales + (size_t)c * nb;
    for (int r = 0; r < m; ++r) {
      const uint16_t* x = lhs + (size_t)r * k;
      float res;
      if (mode == 0) {
        float s = 0;
        for (int i = 0; i < k; ++i) s += h2f(x[i]) * h2f(dequant_one(wq[i], sc[i / bs]));
        res = s;
      } else if (mode == 1) {
        float s = 0;
        for (int i = 0; i < k; ++i)
          s = (float)((double)s + (double)h2f(x[i]) * ((double)(float)wq[i] - 127.5) * (double)h2f(sc[i / bs]));
        res = s;
      } else if (mode == 2) {
        double s = 0;
        for (int i = 0; i < k; ++i) s += (double)h2f(x[i]) * (double)h2f(dequant_one(wq[i], sc[i / bs]));
        res = (float)s;
      } else {
        double s = 0;
        for (int i = 0; i < k; ++i) s += (double)h2f(x[i]) * ((double)wq[i] - 127.5) * (double)h2f(sc[i / bs]);
        res = (float)s;
      }
      size_t o = (size_t)r * n + c;
      out[o] = f2h(beta == 0.f ? res : fmaf(beta, h2f(out[o]), res));
    }
  }
}

void matmul_w(uint16_t* out, const uint16_t* lhs, const weight_t& w, int m, float beta, int wmma_rounding) {
  if (w.bs == 0)
    matmul_nt_f16(out, lhs, w.f16.data(), m, (int)w.w, (int)w.h, beta, 0);
  else
    matmul_nt_fp16u8(out, lhs, w.q.data(), w.scales.data(), m, (int)w.w, (int)w.h, w.bs, beta,
                     wmma_rounding ? 0 : 1);
}

// llama_cu.cu:368-389.  Pairs (c, c+1), angle = (pos_offset + r) / powf(theta, float(c % hd) / hd).
void rotary(uint16_t* out, const uint16_t* in, int h, int w, int n_heads, int pos_offset, float theta) {
  int hd = w / n_heads;
  for (int r = 0; r < h; ++r)
    for (int c = 0; c < w; c += 2) {
      int hc = c % hd;
      float angle = (float)(pos_offset + r) / powf(theta, (float)hc / (float)hd);
      float re = h2f(in[(size_t)r * w + c]);
      float im = h2f(in[(size_t)r * w + c + 1]);
      float cs = cosf(angle), sn = sinf(angle);
      out[(size_t)r * w + c] = f2h(fmaf(re, cs, -(im * sn)));
      out[(size_t)r * w + c + 1] = f2h(fmaf(re, sn, im * cs));
    }
}

// llama_cu.cu:400-428.  out is (n_heads, m, T) with row stride T (the stride the consumers use,
// llama_cu.cu:437,526; the producer's own `r*seq_len_new` stride coincides whenever m == 1 or start_pos == 0).
void matmul_qk(uint16_t* out, const uint16_t* q, const uint16_t* k, int m, int T, int dim, int n_heads, int start_pos) {
  int hd = dim / n_heads;
  float inv = sqrtf((float)hd);
  for (int hh = 0; hh < n_heads; ++hh)
    for (int r = 0; r < m; ++r)
      for (int c = 0; c < T; ++c) {
        size_t o = (size_t)hh * m * T + (size_t)r * T + c;
        if (c > r + start_pos) {
          out[o] = 0xfc00u;  // -inf
        } else {
          float s = 0;
          for (int i = 0; i < hd; ++i) s += h2f(q[(size_t)r * dim + hh * hd + i]) * h2f(k[(size_t)c * dim + hh * hd + i]);
          out[o] = f2h(s / inv);
        }
      }
}

// llama_cu.cu:433-499.  v = float(x)/temp; max; sum expf(v-max); out = half(expf(v-max)/sum).
void softmax_rows(uint16_t* out, const uint16_t* in, size_t rows, int w, float temp) {
  for (size_t r = 0; r < rows; ++r) {
    const uint16_t* x = in + r * w;
    float mx = -INFINITY;
    for (int i = 0; i < w; ++i) mx = fmaxf(mx, h2f(x[i]) / temp);
    // kernel order: 256 strided partial sums, warp xor trees, then 8-way tree
    float part[256];
    for (int t = 0; t < 256; ++t) {
      float s = 0.f;
      for (int i = t; i < w; i += 256) s += expf(h2f(x[i]) / temp - mx);
      part[t] = s;
    }
    float warp[8];
    for (int wi = 0; wi < 8; ++wi) {
      float v[32];
      for (int l = 0; l < 32; ++l) v[l] = part[wi * 32 + l];
      for (int off = 16; off > 0; off /= 2) {
        float n[32];
        for (int l = 0; l < 32; ++l) n[l] = v[l] + v[l ^ off];
        memcpy(v, n, sizeof v);
      }
      warp[wi] = v[0];
    }
    float v[8];
    memcpy(v, warp, sizeof v);
    for (int off = 4; off > 0; off /= 2) {
      float n[8];
      for (int l = 0; l < 8; ++l) n[l] = v[l] + v[l ^ off];
      memcpy(v, n, sizeof v);
    }
    float sum = v[0];
    for (int i = 0; i < w; ++i) out[r * w + i] = f2h(expf(h2f(x[i]) / temp - mx) / sum);
  }
}

// llama_cu.cu:511-531.  out(m,dim) = half( sum_t float(p[head,r,t]) * float(v[t,c]) ), head = c / hd.
void matmul_qkv(uint16_t* out, const uint16_t* p, const uint16_t* v, int m, int T, int dim, int n_heads) {
  int hd = dim / n_heads;
  for (int r = 0; r < m; ++r)
    for (int c = 0; c < dim; ++c) {
      int hh = c / hd;
      float s = 0;
      for (int t = 0; t < T; ++t) s += h2f(p[(size_t)hh * m * T + (size_t)r * T + t]) * h2f(v[(size_t)t * dim + c]);
      out[(size_t)r * dim + c] = f2h(s);
    }
}

// fp32 variant of the attention chain (no half rounding of scores / probabilities): what a fused
// kernel computes if it does not mirror the reference's intermediate storage.  Diagnostic only.
void attention_fp32(uint16_t* out, const uint16_t* q, const uint16_t* k, const uint16_t* v, int m, int T, int dim,
                    int n_heads, int start_pos) {
  int hd = dim / n_heads;
  std::vector<float> s(T);
  for (int hh = 0; hh < n_heads; ++hh)
    for (int r = 0; r < m; ++r) {
      int lim = std::min(T, r + start_pos + 1);
      float mx = -INFINITY;
      for (int c = 0; c < lim; ++c) {
        float a = 0;
        for (int i = 0; i < hd; ++i) a += h2f(q[(size_t)r * dim + hh * hd + i]) * h2f(k[(size_t)c * dim + hh * hd + i]);
        s[c] = a / sqrtf((float)hd);
        mx = fmaxf(mx, s[c]);
      }
      float sum = 0;
      for (int c = 0; c < lim; ++c) {
        s[c] = expf(s[c] - mx);
        sum += s[c];
      }
      for (int i = 0; i < hd; ++i) {
        float a = 0;
        for (int c = 0; c < lim; ++c) a += s[c] * h2f(v[(size_t)c * dim + hh * hd + i]);
        out[(size_t)r * dim + hh * hd + i] = f2h(a / sum);
      }
    }
}

// llama_cu.cu:533-539
void silu(uint16_t* out, const uint16_t* a, const uint16_t* b, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    float v = h2f(a[i]);
    out[i] = f2h(v / (1.0f + expf(-v)) * h2f(b[i]));
  }
}

// llama_cu.cu:32-62
void embed(uint16_t* out, const weight_t& table, const int16_t* ids, int n_ids) {
  size_t d = table.w;
  for (int t = 0; t < n_ids; ++t) {
    size_t id = (size_t)ids[t];
    if (table.bs == 0) {
      memcpy(out + t * d, table.f16.data() + id * d, d * 2);
    } else {
      size_t nb = d / table.bs;
      for (size_t i = 0; i < d; ++i) out[t * d + i] = dequant_one(table.q[id * d + i], table.scales[id * nb + i / table.bs]);
    }
  }
}

// transform.cu:28-72.  Per (row, K-block): scale = half(absmax / 127.5f); q = (u8) roundf(127.5f + x / float(scale)).
// An all-zero block gives 0/0 = NaN, which the device's float->u8 conversion turns into 0.
void quantize_absmax_uint8(uint8_t* q, uint16_t* scales, const uint16_t* in, size_t h, size_t w, int bs) {
  size_t nb = w / bs;
#pragma omp parallel for schedule(static)
  for (size_t r = 0; r < h; ++r)
    for (size_t b = 0; b < nb; ++b) {
      const uint16_t* x = in + r * w + b * bs;
      float amax = 0;
      for (int i = 0; i < bs; ++i) amax = fmaxf(amax, fabsf(h2f(x[i])));
      uint16_t sc = f2h(amax / 127.5f);
      scales[r * nb + b] = sc;
      float s = h2f(sc);
      for (int i = 0; i < bs; ++i) {
        float v = roundf(127.5f + h2f(x[i]) / s);
        q[r * w + b * bs + i] = std::isnan(v) ? 0 : (uint8_t)(v < 0 ? 0.f : (v > 255.f ? 255.f : v));
      }
    }
}

// transform.cu:74-87
void dequantize_absmax_uint8(uint16_t* out, const uint16_t* scales, const uint8_t* q, size_t h, size_t w, int bs) {
  size_t nb = w / bs;
#pragma omp parallel for schedule(static)
  for (size_t r = 0; r < h; ++r)
    for (size_t i = 0; i < w; ++i) out[r * w + i] = dequant_one(q[r * w + i], scales[r * nb + i / bs]);
}

// transform.cu:100-150: mean squared error, max abs error, mean abs error (order of the float
// atomics in the kernel is unspecified; summed in double here and compared with a tolerance).
void error_stats(float out[3], const uint16_t* a, const uint16_t* b, size_t n) {
  double ss = 0, sa = 0;
  float mx = 0;
  for (size_t i = 0; i < n; ++i) {
    float d = h2f(a[i]) - h2f(b[i]);
    ss += (double)d * d;
    sa += fabs(d);
    mx = fmaxf(mx, fabsf(d));
  }
  out[0] = (float)(ss / (double)n);
  out[1] = mx;
  out[2] = (float)(sa / (double)n);
}

// ---------------------------------------------------------------- model construction
void quantize_weight(weight_t& w, int bs) {
  w.q.resize(w.h * w.w);
  w.scales.resize(w.h * (w.w / bs));
  quantize_absmax_uint8(w.q.data(), w.scales.data(), w.f16.data(), w.h, w.w, bs);
  w.f16.clear();
  w.f16.shrink_to_fit();
  w.bs = bs;
}

void synth_weight(weight_t& w, size_t h, size_t width, uint64_t seed, const std::string& name, float scale) {
  w.h = h;
  w.w = width;
  w.bs = 0;
  w.f16.resize(h * width);
  uint64_t stream = fnv1a64(name.c_str());
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < h * width; ++i) w.f16[i] = synth_half(seed, stream, i, scale);
}

bool read_file(const std::string& path, void* dst, size_t bytes) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return false;
  fseek(f, 0, SEEK_END);
  size_t sz = (size_t)ftell(f);
  fseek(f, 0, SEEK_SET);
  bool ok = sz == bytes && fread(dst, 1, bytes, f) == bytes;
  fclose(f);
  return ok;
}

// weight directory layout: llama_cu.cu:929-984
bool load_weight(weight_t& w, const params_t& p, const std::string& dir, const std::string& name, size_t h, size_t width) {
  w.h = h;
  w.w = width;
  std::string base = dir + "/" + name;
  std::string dims = std::to_string(h) + "_" + std::to_string(width);
  if (p.q_type == 0) {
    w.bs = 0;
    w.f16.resize(h * width);
    return read_file(base + ".weight__" + dims, w.f16.data(), h * width * 2);
  }
  w.bs = p.block_size;
  w.q.resize(h * width);
  w.scales.resize(h * (width / w.bs));
  return read_file(base + ".weight__" + dims, w.q.data(), h * width) &&
         read_file(base + ".scale__" + std::to_string(h) + "_" + std::to_string(width / w.bs), w.scales.data(),
                   w.scales.size() * 2);
}

bool load_vec(std::vector<uint16_t>& v, const std::string& dir, const std::string& name, size_t w) {
  v.resize(w);
  return read_file(dir + "/" + name + ".weight__" + std::to_string(w), v.data(), w * 2);
}

// the forward pass, llama_cu.cu:1073-1210, in the reference's order and with its rounding points
int next_token(context_t* c, const int16_t* tokens, int m) {
  model_t& M = *c->m;
  const params_t& p = M.p;
  int d = (int)p.dim, H = (int)p.n_heads, f = (int)M.ffn, V = (int)p.n_vocab;
  int sp = c->start_pos, T = sp + m;
  if (T > c->ctx_len) return -1;
  std::vector<uint16_t> x((size_t)m * d), nrm((size_t)m * d), xq((size_t)m * d), xk((size_t)T * d), att((size_t)m * d);
  std::vector<uint16_t> qk((size_t)H * m * T), h1((size_t)m * f), h3((size_t)m * f), hs((size_t)m * f);
  embed(x.data(), M.tok_embeddings, tokens, m);  // :1086-1097
  auto clk0 = std::chrono::steady_clock::now();
  for (size_t l = 0; l < M.layers.size(); ++l) {
    layer_t& L = M.layers[l];
    uint16_t* kc = c->k_cache[l].data();
    uint16_t* vc = c->v_cache[l].data();
    rms_norm(nrm.data(), x.data(), L.attn_norm.data(), m, d, p.norm_eps);         // :1129
    matmul_w(xq.data(), nrm.data(), L.wq, m, 0.f, c->wmma_rounding);               // :1144
    rotary(xq.data(), xq.data(), m, d, H, sp, 10000.0f);                           // :1146
    matmul_w(kc + (size_t)sp * d, nrm.data(), L.wk, m, 0.f, c->wmma_rounding);     // :1150 (into the cache)
    rotary(xk.data(), kc, T, d, H, 0, 10000.0f);                                   // :1152 (whole prefix)
    matmul_w(vc + (size_t)sp * d, nrm.data(), L.wv, m, 0.f, c->wmma_rounding);     // :1156
    if (c->fp32_attention) {
      attention_fp32(att.data(), xq.data(), xk.data(), vc, m, T, d, H, sp);
    } else {
      matmul_qk(qk.data(), xq.data(), xk.data(), m, T, d, H, sp);                  // :1163
      softmax_rows(qk.data(), qk.data(), (size_t)H * m, T, 1.0f);                  // :1166
      matmul_qkv(att.data(), qk.data(), vc, m, T, d, H);                           // :1170
    }
    matmul_w(x.data(), att.data(), L.wo, m, 1.0f, c->wmma_rounding);               // :1174 residual
    rms_norm(nrm.data(), x.data(), L.ffn_norm.data(), m, d, p.norm_eps);           // :1176
    matmul_w(h1.data(), nrm.data(), L.w1, m, 0.f, c->wmma_rounding);               // :1180
    matmul_w(h3.data(), nrm.data(), L.w3, m, 0.f, c->wmma_rounding);               // :1181
    silu(hs.data(), h1.data(), h3.data(), (size_t)m * f);                          // :1183
    matmul_w(x.data(), hs.data(), L.w2, m, 1.0f, c->wmma_rounding);                // :1185 residual
  }
  auto clk1 = std::chrono::steady_clock::now();
  c->last_hidden.assign(x.begin() + (size_t)(m - 1) * d, x.end());
  rms_norm(nrm.data(), x.data() + (size_t)(m - 1) * d, M.norm.data(), 1, d, p.norm_eps);  // :1191 (only the last row is used)
  c->logits.resize(V);
  c->probs.resize(V);
  matmul_w(c->logits.data(), nrm.data(), M.output, 1, 0.f, c->wmma_rounding);      // :1195
  softmax_rows(c->probs.data(), c->logits.data(), 1, V, c->temperature);          // :1196
  c->start_pos += m;                                                               // :1201
  auto clk2 = std::chrono::steady_clock::now();
  c->t_layers = std::chrono::duration<double>(clk1 - clk0).count();
  c->t_head = std::chrono::duration<double>(clk2 - clk1).count();
  int best = 0;                                                                    // :1205-1209 first maximum
  for (int i = 1; i < V; ++i)
    if (h2f(c->probs[best]) < h2f(c->probs[i])) best = i;
  return best;
}

}  // namespace

// ================================================================== C interface (ctypes)
extern "C" {

void orc_init() { init_tables(); }

uint16_t orc_f2h(float f) { return f2h(f); }
float orc_h2f(uint16_t h) {
  init_tables();
  return h2f(h);
}

uint64_t orc_fnv1a64(const char* name) { return fnv1a64(name); }

void orc_synth_fill_f16(uint16_t* out, uint64_t n, uint64_t seed, const char* name, float scale, uint64_t first) {
  init_tables();
  uint64_t stream = fnv1a64(name);
#pragma omp parallel for schedule(static)
  for (uint64_t i = 0; i < n; ++i) out[i] = synth_half(seed, stream, first + i, scale);
}

// token ids uniform in [lo, hi): lo + word0 % (hi - lo)
void orc_synth_tokens(int16_t* out, int n, uint64_t seed, const char* name, int lo, int hi) {
  uint64_t stream = fnv1a64(name);
  for (int i = 0; i < n; ++i) {
    uint32_t c[4] = {(uint32_t)i, 0u, (uint32_t)stream, (uint32_t)(stream >> 32)};
    philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
    out[i] = (int16_t)(lo + (int)(c[0] % (uint32_t)(hi - lo)));
  }
}

void orc_quantize_absmax_uint8(uint8_t* q, uint16_t* scales, const uint16_t* in, uint64_t h, uint64_t w, int bs) {
  init_tables();
  quantize_absmax_uint8(q, scales, in, h, w, bs);
}
void orc_dequantize_absmax_uint8(uint16_t* out, const uint16_t* scales, const uint8_t* q, uint64_t h, uint64_t w, int bs) {
  init_tables();
  dequantize_absmax_uint8(out, scales, q, h, w, bs);
}
void orc_error_stats(float* out3, const uint16_t* a, const uint16_t* b, uint64_t n) {
  init_tables();
  error_stats(out3, a, b, n);
}
void orc_matmul_nt_f16(uint16_t* out, const uint16_t* lhs, const uint16_t* rhs, int m, int k, int n, float beta, int acc64) {
  init_tables();
  matmul_nt_f16(out, lhs, rhs, m, k, n, beta, acc64);
}
void orc_matmul_nt_fp16u8(uint16_t* out, const uint16_t* lhs, const uint8_t* q, const uint16_t* scales, int m, int k,
                          int n, int bs, float beta, int mode) {
  init_tables();
  matmul_nt_fp16u8(out, lhs, q, scales, m, k, n, bs, beta, mode);
}
// double-precision result vector (no final rounding) for error metrics: out64[r*n+c]
void orc_matmul_nt_gold(double* out64, const uint16_t* lhs, const uint16_t* rhs_f16, const uint8_t* q,
                        const uint16_t* scales, int m, int k, int n, int bs, int round_weights) {
  init_tables();
#pragma omp parallel for schedule(static)
  for (int c = 0; c < n; ++c)
    for (int r = 0; r < m; ++r) {
      double s = 0;
      for (int i = 0; i < k; ++i) {
        double w;
        if (rhs_f16) {
          w = h2f(rhs_f16[(size_t)c * k + i]);
        } else if (round_weights) {
          w = h2f(dequant_one(q[(size_t)c * k + i], scales[(size_t)c * (k / bs) + i / bs]));
        } else {
          w = ((double)q[(size_t)c * k + i] - 127.5) * (double)h2f(scales[(size_t)c * (k / bs) + i / bs]);
        }
        s += (double)h2f(lhs[(size_t)r * k + i]) * w;
      }
      out64[(size_t)r * n + c] = s;
    }
}
void orc_rms_norm(uint16_t* out, const uint16_t* in, const uint16_t* weight, int h, int w, float eps) {
  init_tables();
  rms_norm(out, in, weight, h, w, eps);
}
void orc_rotary(uint16_t* out, const uint16_t* in, int h, int w, int n_heads, int pos_offset, float theta) {
  init_tables();
  rotary(out, in, h, w, n_heads, pos_offset, theta);
}
void orc_matmul_qk(uint16_t* out, const uint16_t* q, const uint16_t* k, int m, int T, int dim, int n_heads, int start_pos) {
  init_tables();
  matmul_qk(out, q, k, m, T, dim, n_heads, start_pos);
}
void orc_softmax_rows(uint16_t* out, const uint16_t* in, uint64_t rows, int w, float temp) {
  init_tables();
  softmax_rows(out, in, rows, w, temp);
}
void orc_matmul_qkv(uint16_t* out, const uint16_t* p, const uint16_t* v, int m, int T, int dim, int n_heads) {
  init_tables();
  matmul_qkv(out, p, v, m, T, dim, n_heads);
}
// the reference's attention chain on row-major q (m,dim), rotated k (T,dim), v (T,dim)
void orc_attention(uint16_t* out, const uint16_t* q, const uint16_t* k, const uint16_t* v, int m, int T, int dim,
                   int n_heads, int start_pos, int fp32_mode) {
  init_tables();
  if (fp32_mode) {
    attention_fp32(out, q, k, v, m, T, dim, n_heads, start_pos);
    return;
  }
  std::vector<uint16_t> qk((size_t)n_heads * m * T);
  matmul_qk(qk.data(), q, k, m, T, dim, n_heads, start_pos);
  softmax_rows(qk.data(), qk.data(), (size_t)n_heads * m, T, 1.0f);
  matmul_qkv(out, qk.data(), v, m, T, dim, n_heads);
}
void orc_silu(uint16_t* out, const uint16_t* a, const uint16_t* b, uint64_t n) {
  init_tables();
  silu(out, a, b, n);
}

// The feed-forward's first half as the reference runs it for a prompt (llama_cu.cu:1180-1183): matmul_nt with w1, matmul_nt
// with w3 - each product stored as halves - then silu on the stored halves.  w13 = [w1; w3], (2 f, k).
void orc_matmul_nt_f16_gated(uint16_t* out, const uint16_t* lhs, const uint16_t* w13, int m, int k, int f, int acc64) {
  init_tables();
  std::vector<uint16_t> a((size_t)m * f), b((size_t)m * f);
  matmul_nt_f16(a.data(), lhs, w13, m, k, f, 0.f, acc64);
  matmul_nt_f16(b.data(), lhs, w13 + (size_t)f * k, m, k, f, 0.f, acc64);
  silu(out, a.data(), b.data(), (uint64_t)m * f);
}

uint32_t orc_ffn_dim(uint32_t dim, uint32_t multiple_of) {
  params_t p{};
  p.dim = dim;
  p.multiple_of = multiple_of;
  return ffn_dim(p);
}

// Synthetic model in the reference's tensor naming: every matrix ~ scale * z, norm weights 1.0.
// block_size > 0 quantizes every matrix (embedding and output included, transform.cu:228-231).
void* orc_model_create_synth(uint32_t dim, uint32_t multiple_of, uint32_t n_heads, uint32_t n_layers, uint32_t n_vocab,
                             float norm_eps, int block_size, uint64_t seed, float scale) {
  init_tables();
  model_t* M = new model_t();
  params_t& p = M->p;
  p.magic = 0x000041524F525541ull;
  p.fourcc = 0x414D4C4Cu;
  p.dim = dim; p.multiple_of = multiple_of; p.n_heads = n_heads; p.n_layers = n_layers; p.n_vocab = n_vocab;
  p.norm_eps = norm_eps;
  p.q_type = block_size > 0 ? 1 : 0;
  p.reserved0 = 0;
  p.block_size = (uint16_t)block_size;
  M->ffn = ffn_dim(p);
  auto mk = [&](weight_t& w, const std::string& name, size_t h, size_t width) {
    synth_weight(w, h, width, seed, name, scale);
    if (block_size > 0) quantize_weight(w, block_size);
  };
  mk(M->tok_embeddings, "tok_embeddings", n_vocab, dim);
  mk(M->output, "output", n_vocab, dim);
  M->norm.assign(dim, 0x3c00u);
  M->layers.resize(n_layers);
  for (uint32_t i = 0; i < n_layers; ++i) {
    layer_t& L = M->layers[i];
    std::string b = "layers." + std::to_string(i) + ".";
    L.attn_norm.assign(dim, 0x3c00u);
    L.ffn_norm.assign(dim, 0x3c00u);
    mk(L.wq, b + "attention.wq", dim, dim);
    mk(L.wk, b + "attention.wk", dim, dim);
    mk(L.wv, b + "attention.wv", dim, dim);
    mk(L.wo, b + "attention.wo", dim, dim);
    mk(L.w1, b + "feed_forward.w1", M->ffn, dim);
    mk(L.w2, b + "feed_forward.w2", dim, M->ffn);
    mk(L.w3, b + "feed_forward.w3", M->ffn, dim);
  }
  return M;
}

void* orc_model_load(const char* dir) {
  init_tables();
  model_t* M = new model_t();
  std::string d(dir);
  if (!read_file(d + "/params", &M->p, sizeof(params_t)) || M->p.magic != 0x000041524F525541ull ||
      M->p.fourcc != 0x414D4C4Cu) {
    delete M;
    return nullptr;
  }
  const params_t& p = M->p;
  M->ffn = ffn_dim(p);
  bool ok = load_weight(M->tok_embeddings, p, d, "tok_embeddings", p.n_vocab, p.dim) &&
            load_weight(M->output, p, d, "output", p.n_vocab, p.dim) && load_vec(M->norm, d, "norm", p.dim);
  M->layers.resize(p.n_layers);
  for (uint32_t i = 0; ok && i < p.n_layers; ++i) {
    layer_t& L = M->layers[i];
    std::string b = "layers." + std::to_string(i) + ".";
    ok = load_vec(L.attn_norm, d, b + "attention_norm", p.dim) && load_vec(L.ffn_norm, d, b + "ffn_norm", p.dim) &&
         load_weight(L.wq, p, d, b + "attention.wq", p.dim, p.dim) && load_weight(L.wk, p, d, b + "attention.wk", p.dim, p.dim) &&
         load_weight(L.wv, p, d, b + "attention.wv", p.dim, p.dim) && load_weight(L.wo, p, d, b + "attention.wo", p.dim, p.dim) &&
         load_weight(L.w1, p, d, b + "feed_forward.w1", M->ffn, p.dim) &&
         load_weight(L.w2, p, d, b + "feed_forward.w2", p.dim, M->ffn) &&
         load_weight(L.w3, p, d, b + "feed_forward.w3", M->ffn, p.dim);
  }
  if (!ok) {
    delete M;
    return nullptr;
  }
  return M;
}

void orc_model_free(void* m) { delete (model_t*)m; }

void* orc_context_create(void* model, int context_len, float temperature) {
  context_t* c = new context_t();
  c->m = (model_t*)model;
  c->ctx_len = context_len;
  c->temperature = temperature;
  size_t n = (size_t)context_len * c->m->p.dim;
  c->k_cache.assign(c->m->layers.size(), std::vector<uint16_t>(n, 0));
  c->v_cache.assign(c->m->layers.size(), std::vector<uint16_t>(n, 0));
  return c;
}
void orc_context_free(void* c) { delete (context_t*)c; }
void orc_context_clear(void* c) { ((context_t*)c)->start_pos = 0; }
void orc_context_set_modes(void* c, int wmma_rounding, int fp32_attention) {
  ((context_t*)c)->wmma_rounding = wmma_rounding;
  ((context_t*)c)->fp32_attention = fp32_attention;
}
int orc_context_pos(void* c) { return ((context_t*)c)->start_pos; }
int orc_next_token(void* c, const int16_t* tokens, int n) { return next_token((context_t*)c, tokens, n); }
void orc_get_probs(void* c, uint16_t* out) {
  context_t* x = (context_t*)c;
  memcpy(out, x->probs.data(), x->probs.size() * 2);
}
void orc_get_logits(void* c, uint16_t* out) {
  context_t* x = (context_t*)c;
  memcpy(out, x->logits.data(), x->logits.size() * 2);
}
void orc_get_last_hidden(void* c, uint16_t* out) {
  context_t* x = (context_t*)c;
  memcpy(out, x->last_hidden.data(), x->last_hidden.size() * 2);
}
// wall seconds of the last orc_next_token call: which 0 = all layers, 1 = final norm + logits + softmax
double orc_last_timing(void* c, int which) { return which == 0 ? ((context_t*)c)->t_layers : ((context_t*)c)->t_head; }
// Multinomial sampling over fp16 probabilities: the distribution of the reference's commented-out
// `std::discrete_distribution<short> dist(probs.begin(), probs.end())` (llama_cu.cu:1202-1203), token i with probability
// p_i / sum(p), restated as the inversion of the cumulative sum at u * sum(p) with binary32 sums in a fixed order:
// chunks of ceil(n / 1024) elements summed in index order, the chunk sums added in index order, then a running sum
// inside the chunk that crosses the target.  Falls back to the last token with a non-zero probability.
int orc_sample_token(const uint16_t* probs, int n, float u) {
  init_tables();
  const int per = (n + 1023) / 1024;
  std::vector<float> chunk(1024, 0.f);
  for (int c = 0; c < 1024; ++c) {
    float s = 0.f;
    for (int i = c * per; i < std::min(n, (c + 1) * per); ++i) s += h2f(probs[i]);
    chunk[c] = s;
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
  if (pick >= 0)
    for (int i = pick * per; i < std::min(n, (pick + 1) * per); ++i) {
      const float w = h2f(probs[i]);
      run += w;
      if (run > target && w > 0.f) return i;
    }
  for (int i = n - 1; i >= 0; --i)
    if (h2f(probs[i]) > 0.f) return i;
  return 0;
}
// u in [0, 1) for (seed, index): word 0 of the Philox4x32-10 block with counter (index, 0, "samp", "ler!"), top 24 bits
float orc_sampler_uniform(uint64_t seed, int index) {
  uint32_t c[4] = {(uint32_t)index, 0u, 0x73616d70u, 0x6c657221u};
  philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
  return (float)(c[0] >> 8) * 0x1p-24f;
}

// number of OpenMP threads used by the calls that follow (1 = the scalar single-thread evaluation); returns the previous value
int orc_set_num_threads(int n) {
#ifdef _OPENMP
  const int prev = omp_get_max_threads();
  if (n >= 1) omp_set_num_threads(n);
  return prev;
#else
  (void)n;
  return 1;
#endif
}
int orc_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

}  // extern "C"
