// Prompt-processing matrix product (reference: matmul_nt dispatch, llama_cu.cu:1463-1523).
#include "prefill.cuh"

#include "gemm_tc.cuh"
#include "gemv.cuh"
#include "ops.cuh"

namespace lcu {

prefill_tuning& prefill_tuning_ref() {
  static prefill_tuning t;
  return t;
}

int& prompt_pdl() {
  static int on = 1;
  return on;
}

int& matmul_type_ref() {
  static int type = 4;
  return type;
}

int matmul_rows(__half* out, const __half* lhs, const dev_matrix& w, int m, float beta, int* err, cudaStream_t stream, __half* deq,
                size_t deq_halves) {
  const int K = (int)w.cols, N = (int)w.rows;
  const prefill_tuning& pt = prefill_tuning_ref();
  if (matmul_type_ref() == 1) return launch_matmul_nt_pedantic(out, lhs, w.w, w.sc, w.bs, m, K, N, beta, stream);
  if (w.bs == 0 && pt.tc_min_rows > 0 && m >= pt.tc_min_rows && gemm_tc_supported(m, N, K, K, lhs, w.w, out))
    return launch_gemm_tc(out, lhs, K, (const __half*)w.w, m, N, K, beta, err, stream, pt.tc_tile_n, pt.tc_pair, pt.tc_split);
  if (w.bs > 0 && deq && pt.u8_deq_min_rows > 0 && m >= pt.u8_deq_min_rows && (size_t)N * K <= deq_halves &&
      gemm_tc_supported(m, N, K, K, lhs, deq, out)) {
    int rc = launch_dequantize_absmax_uint8(deq, w.sc, (const uint8_t*)w.w, (size_t)N, (size_t)K, w.bs, stream);
    if (rc) return rc;
    return launch_gemm_tc(out, lhs, K, deq, m, N, K, beta, err, stream, pt.tc_tile_n, pt.tc_pair, pt.tc_split);
  }
  const int pass_rows = gemv_max_rows(K);  // 8, fewer where the activation rows are long
  LCU_REQUIRE(pass_rows >= 1, "matmul_nt: a row of K=%d does not fit in shared memory", K);
  for (int t = 0; t < m; t += pass_rows) {
    gemv_params p{};
    p.w[0] = w.w;
    p.sc[0] = w.sc;
    p.n_mats = 1;
    p.rows_per_mat = N;
    p.K = K;
    p.bs = w.bs;
    p.x = lhs + (size_t)t * K;
    p.m = m - t < pass_rows ? m - t : pass_rows;
    p.ldx = K;
    p.out = out + (size_t)t * N;
    p.ldo = N;
    p.beta = beta;
    p.err = err;
    int rc = launch_gemv(p, EPI_PLAIN, stream, 0);
    if (rc) return rc;
  }
  return LCU_OK;
}

}  // namespace lcu
