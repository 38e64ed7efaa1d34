/* C ABI of the B200-native llama.cu inference core (libllama_cu_b200.so).
 *
 * Plain pointers and sizes only.  Every entry point names the reference interface it stands in
 * for (file:line in eiz/llama.cu).  The reference has no C ABI of its own: its boundary is the
 * C++ header llama_cu.h; the C++ classes of that header are provided by include/llama_cu.h on top
 * of the same library, and this C layer is what a foreign-function binding (ctypes, cgo, JNI ...)
 * loads.
 *
 * Conventions: functions return 0 on success or a non-zero lcu status (1 CUDA error, 2 invalid
 * argument, 3 I/O error, 4 a kernel gave up on a bounded wait); lcu_last_error() returns the
 * message of the calling thread's last failure.  `stream` is a cudaStream_t passed as void*
 * (NULL = the legacy default stream).  "dev" pointers are device memory of the current device,
 * "host" pointers are host memory.  All fp16 data is IEEE binary16.  There is no CPU fallback:
 * every compute entry point launches sm_100a kernels and fails if no such device is present.
 */
#ifndef LLAMA_CU_C_H
#define LLAMA_CU_C_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- library ------------------------------------------------------------------------------ */
const char* lcu_last_error(void);
/* llama_cu::initialize (llama_cu.cu:1525-1542): prints the device properties; returns the device count. */
int lcu_initialize(int verbose);
int lcu_device_count(void);
/* llama_cu::matmul_type (llama_cu.h:65-68, llama_cu.cu:28): 4 (the reference's tensor-core kernels) and 0 (its cuBLAS
 * path) select the sm_100a kernels.  1 selects the pedantic pair of llama_cu.cu:111-145 for every matrix product
 * (lcu_matmul_nt_* and every product inside lcu_context_next_token): one thread per output element, terms added in
 * index order, binary32 sum (u8 weights: binary64 terms); a context then runs single-token steps through the unfused
 * operator sequence.  It is the on-GPU check for the fast kernels and is slow by design. */
int lcu_set_matmul_type(int type);
/* launch-shape knobs used for the measurements (defaults are the measured best): "gemv_stages", "gemv_ctas_per_sm",
 * "gemv_ctas_per_sm_int8", "gemv_variant", "gemv_warp_stages", "gemv_warp_stages_int8", "gemv_consumer_warps_int8", "gemv_prefetch_kb",
 * "int8_factored" (0 = round every dequantized weight to half as the reference does), "prefill_tc_min_rows",
 * "prefill_tc_tile_n", "prefill_tc_pair", "prefill_tc_split", "prefill_tc_sk", "prefill_tc_kb", "prefill_sk_kb" (k-blocks per
 * stage and tensor copy of the one-SM / the pair GEMMs), "prefill_gate_fused", "prefill_u8_deq_min_rows", "prefill_u8_shadow", "prefill_fuse",
 * "prefill_attn_tc", "prefill_attn_tc_min_rows", "prefill_attn_fused_min_rows", "prefill_attn_fused_order", "prefill_attn_tiles", "prompt_pdl", "attn_stream",
 * "use_graph", "use_pdl", "attn_cluster", "loader_staged" (lcu_model_load: 1 = pinned double-buffered asynchronous copies, 0 = a file mapping and one
 * blocking pageable copy per tensor as the reference does).  Unknown keys are rejected. */
int lcu_set_tuning(const char* key, int value);

/* device memory helpers for callers that have no CUDA binding of their own */
int lcu_malloc(void** dev_out, uint64_t bytes);
int lcu_free(void* dev);
int lcu_memcpy_h2d(void* dev, const void* host, uint64_t bytes);
int lcu_memcpy_d2h(void* host, const void* dev, uint64_t bytes);
int lcu_memcpy_d2d(void* dst_dev, const void* src_dev, uint64_t bytes); /* any two devices */
int lcu_memset(void* dev, int value, uint64_t bytes);
int lcu_mem_info(uint64_t* free_bytes_out, uint64_t* total_bytes_out); /* cudaMemGetInfo of the current device */
int lcu_set_device(int device);
int lcu_synchronize(void);

/* ---- quantizer (transform.cu) --------------------------------------------------------------- */
/* quantize_absmax_uint8 kernel, transform.cu:28-72, launched by quantize_one at transform.cu:171.
 * in: fp16 [h][w]; q: u8 [h][w]; scales: fp16 [h][w/bs].  Bit-identical to the reference. */
int lcu_quantize_absmax_uint8(void* q_dev, void* scales_dev, const void* in_dev, uint64_t h, uint64_t w, int bs, void* stream);
/* dequantize_absmax_uint8 kernel, transform.cu:74-87 */
int lcu_dequantize_absmax_uint8(void* out_dev, const void* scales_dev, const void* q_dev, uint64_t h, uint64_t w, int bs, void* stream);
/* error_stats kernel, transform.cu:100-150: stats_host[0..2] = mean squared / max / mean absolute error */
int lcu_error_stats(float* stats_host, const void* a_dev, const void* b_dev, uint64_t n, void* stream);
/* quantize_one, transform.cu:152-196, on host buffers (copies in, quantizes, copies out; stats_host may be NULL) */
int lcu_quantize_host(uint8_t* q_host, uint16_t* scales_host, const uint16_t* in_host, uint64_t h, uint64_t w, int bs, float* stats_host);
/* do_quantize, transform.cu:220-263 (`transform quantize <in> <out> <bs>`): weight directory -> weight directory */
int lcu_quantize_model_dir(const char* in_dir, const char* out_dir, int bs);

/* ---- operators (the reference's internal seam) ---------------------------------------------- */
/* matmul_nt(out, lhs, rhs, beta, stream), llama_cu.cu:738-742 / 1463-1496:
 * out(m,n) = lhs(m,k) . rhs(n,k)^T + beta * out, fp16 in/out, fp32 accumulation.  No gutter rows needed. */
int lcu_matmul_nt_f16(void* out_dev, const void* lhs_dev, const void* rhs_dev, int m, int k, int n, float beta, void* stream);
/* The feed-forward's first half as one launch: matmul_nt of lhs(m,k) with w1 and with w3 (llama_cu.cu:1180-1181; w13 =
 * [w1; w3], (2 f, k), k a multiple of 64) and silu (llama_cu.cu:533-539, 1182-1183) on the half-rounded products: out(m,f).
 * The same bits as lcu_matmul_nt_f16 on each matrix followed by lcu_silu.  tile = accumulator columns per output tile:
 * 256 (f a multiple of 128; the gate runs under the next tile's main loop) or 512 (f a multiple of 256).  Prompt passes
 * use it as the tuning key "prefill_gate_fused" says (-1 = when estimated faster, 256 / 512 = from 129 rows with that
 * tile, 0 = never). */
int lcu_matmul_nt_f16_gated(void* out_dev, const void* lhs_dev, const void* w13_dev, int m, int k, int f, int tile, void* stream);
/* matmul_nt(out, lhs, generic_tensor& rhs, beta, stream) with a quantized rhs, llama_cu.cu:743-747 / 1498-1523 */
int lcu_matmul_nt_fp16u8(void* out_dev, const void* lhs_dev, const void* q_dev, const void* scales_dev, int m, int k, int n, int bs,
                         float beta, void* stream);
/* kernel::rms_norm, llama_cu.cu:66-107 (launch at 1129) */
int lcu_rms_norm(void* out_dev, const void* in_dev, const void* weight_dev, int rows, int dim, float eps, void* stream);
/* kernel::silu, llama_cu.cu:533-539 (launch at 1183) */
int lcu_silu(void* out_dev, const void* a_dev, const void* b_dev, uint64_t n, void* stream);
/* kernel::rotary, llama_cu.cu:368-389 (launches at 1146 and 1152), together with the cache write:
 * rotates q rows in place at positions pos0+r, rotates k_new into k_cache and copies v_new into
 * v_cache, both head-major [n_heads][ctx_len][dim/n_heads]. */
int lcu_rope_scatter(void* q_dev, const void* k_new_dev, const void* v_new_dev, void* k_cache_dev, void* v_cache_dev, int pos0, int m,
                     int dim, int n_heads, int ctx_len, void* stream);
/* Same operator for callers that cannot allocate device memory (a server whose memory pool owns
 * all of HBM, a loop that must not hit cudaMalloc's device-wide synchronisation, a host that forbids
 * allocation after start-up).  No counterpart in the reference.  The cos/sin table lives in a fixed
 * 2 MiB device array inside the library instead of a per-call allocation; (pos0 + m) * (dim / n_heads / 2)
 * must not exceed 262144 entries (4096 positions at head_dim 128) or the call is rejected.  All calls
 * share that array: calls whose kernels overlap on the GPU race.  The first call on each device resolves
 * the array's address, which is also what makes the CUDA runtime load the module that holds the array: that
 * first call reserves the 2 MiB (and may synchronise), so make it at start-up - one small call per device -
 * before HBM is exhausted and outside stream capture.  Later calls take no device memory and return without
 * synchronising. */
int lcu_rope_scatter_static(void* q_dev, const void* k_new_dev, const void* v_new_dev, void* k_cache_dev, void* v_cache_dev, int pos0,
                            int m, int dim, int n_heads, int ctx_len, void* stream);
/* matmul_qk + softmax_rows + matmul_qkv, llama_cu.cu:400-531 (launches at 1163-1171), fused:
 * q [m][dim] rotated, caches head-major as above holding positions 0 .. pos0+m-1; out [m][dim].
 * cluster = 1, 2, 4, 8: one thread-block cluster of that many CTAs per (row, head), the decode kernel;
 * cluster = 0: 64-row query tiles on warp-level tensor-core instructions (one fused kernel);
 * cluster = -1: the prompt path on tcgen05 as three kernels (scores to a temporary fp16 buffer, softmax, probabilities x V);
 * cluster = -2: the prompt path on tcgen05 as one kernel (scores in tensor memory, no buffer). */
int lcu_attention(void* out_dev, const void* q_dev, const void* k_cache_dev, const void* v_cache_dev, int pos0, int m, int dim,
                  int n_heads, int ctx_len, int cluster, void* stream);
/* softmax_rows with temperature on the logits + the host-side first-maximum search,
 * llama_cu.cu:1196-1209: probs_dev (fp16 [n_vocab], may alias logits_dev), *token_host = argmax */
int lcu_logits_head(void* probs_dev, const void* logits_dev, int n_vocab, float temperature, int* token_host, void* stream);

/* ---- synthetic data ------------------------------------------------------------------------- */
/* out[i] = fp16(scale * z(seed, name, first + i)), z approximately N(0,1), reproducible on any host */
int lcu_synth_fill_f16(void* out_dev, uint64_t n, uint64_t seed, const char* name, float scale, uint64_t first, void* stream);

/* ---- model (llama_model, llama_cu.h:362-372) -------------------------------------------------- */
/* params40: the 40-byte params record (llama_cu.h:280-291).  layer_gpus: n_layers device indices
 * (llama_partition::layer_gpus, llama_cu.h:301-314; embedding on the first, output on the last),
 * NULL = every layer on the calling thread's current device (lcu_set_device; device 0 unless changed, which is
 * llama_partition::use_default, llama_cu.cu:810-818). */
int lcu_model_create(const void* params40, const int* layer_gpus, void** model_out);
/* llama_model::load, llama_cu.cu:987-997: reads <dir>/params and the tensor files (llama_cu.cu:929-984) */
int lcu_model_load(const char* dir, const int* layer_gpus, void** model_out);
/* seeded synthetic weights in place of a checkpoint (matrices scale*z, norm weights 1.0) */
int lcu_model_fill_synthetic(void* model, uint64_t seed, float scale);
/* writes the model as a weight directory in the reference's layout (extract.py:16-41, transform.cu:179-261) */
int lcu_model_save(void* model, const char* dir);
/* device pointer of a tensor by file stem, e.g. "layers.0.attention.wq"; which: 0 values, 1 scales */
int lcu_model_tensor(void* model, const char* name, int which, void** dev_out, uint64_t* bytes_out, int* device_out);
int lcu_model_params(void* model, void* params40_out);
uint64_t lcu_model_weight_bytes(void* model);
/* u8 models: bytes of the fp16 copy of the layer matrices that prompts of 2 tokens or more read (the same halves the
 * per-pass expansion of llama_cu.cu:287-289 produces, expanded once).  It is allocated when the model's first context is
 * created, where the GPU keeps 6 GB free after it, and not at all with the tuning key "prefill_u8_shadow" = 0 (prompts
 * then expand into the context's scratch on every pass); 0 while it does not exist. */
uint64_t lcu_model_shadow_bytes(void* model);
void lcu_model_free(void* model);
/* llama_params::ffn_dim, llama_cu.cu:765-767 */
uint32_t lcu_ffn_dim(uint32_t dim, uint32_t multiple_of);
/* llama_partition::autopipe, llama_cu.cu:819-837: fills layer_gpus_out[n_layers] greedily by free memory; returns 0 if it fits */
int lcu_partition_autopipe(const void* params40, int context_len, int* layer_gpus_out);
/* 1 if every GPU of the map holds one contiguous run of layers (what lcu_model_create / lcu_model_load accept: the
 * reference's forward pass asserts embedding on the first and output on the last layer's GPU, llama_cu.cu:1076-1079,
 * and a GPU that reappears later would run the head against another stage's buffers), else 0.  Host only. */
int lcu_partition_is_contiguous(const int* layer_gpus, int n_layers);
/* llama_params::shared_context_memory_size / kv_cache_size (llama_cu.cu:781-808): bytes of the scratch arena
 * lcu_context_create allocates on every GPU it uses (activations, prompt-path score and dequantization buffers, tables)
 * and of one layer's K and V caches; lcu_partition_autopipe packs with the same figures.  Host only. */
uint64_t lcu_context_scratch_bytes(const void* params40, int context_len);
uint64_t lcu_context_kv_bytes_per_layer(const void* params40, int context_len);
/* contiguous equal split over n_gpus devices (the hand-built partitions of the pipelined configurations) */
int lcu_partition_even(int n_layers, int n_gpus, int* layer_gpus_out);

/* ---- context (llama_context, llama_cu.h:374-390) ---------------------------------------------- */
/* llama_context::create(model, context_len, temperature), llama_cu.cu:1306-1310 */
int lcu_context_create(void* model, int context_len, float temperature, void** ctx_out);
void lcu_context_free(void* ctx);
/* llama_context::clear_tokens, llama_cu.cu:1004-1049 (resets the position; nothing is re-allocated) */
void lcu_context_clear_tokens(void* ctx);
/* llama_context::context_memory_usage, llama_cu.cu:1051-1072 */
uint64_t lcu_context_memory_usage(void* ctx);
/* llama_context::tokens_left, llama_cu.h:381 */
int lcu_context_tokens_left(void* ctx);
/* llama_context::next_token(new_tokens), llama_cu.cu:1073-1210: host token ids in, greedy token out */
int lcu_context_next_token(void* ctx, const int16_t* tokens_host, int n_tokens, int* token_out);
/* n_steps greedy single-token steps chained on the device (the loop of main.cpp:80-100 without the
 * per-token host round trip); tokens_host_out[n_steps]; *ms_out = device time of the loop */
int lcu_context_decode_chained(void* ctx, int16_t first_token, int n_steps, int16_t* tokens_host_out, float* ms_out);
/* probabilities of the last step (what the reference leaves in its logits buffer, llama_cu.cu:1196-1200) */
int lcu_context_read_probs(void* ctx, uint16_t* probs_host);
/* residual stream row of the last token before the final norm (diagnostics) */
int lcu_context_read_hidden(void* ctx, uint16_t* hidden_host);
int lcu_context_kernels_per_step(void* ctx);
/* The sampler the reference has commented out (llama_cu.cu:1202-1203: std::discrete_distribution over the fp16
 * probabilities in place of the argmax), on the device.  mode 0 = greedy (default, what the reference runs), 1 = token i
 * with probability p_i / sum(p): the cumulative sum (binary32, fixed order) is inverted at u * sum(p), u from a
 * counter-based generator keyed by (seed, sequence length after the step), so a run repeats for the same seed.
 * The reference draws from std::random_device and cannot be repeated; no parity of tokens is claimed in mode 1. */
int lcu_context_set_sampling(void* ctx, int mode, uint64_t seed);
/* the u of mode 1 for a sequence length (host only), and the same inversion as a stand-alone operator on device probabilities */
float lcu_sampler_uniform(uint64_t seed, int index);
int lcu_sample_token(const void* probs_dev, int n_vocab, float u, int* token_host, void* stream);
/* Context roll-over without a new prompt pass.  The reference's client clears the context when it is full and feeds the
 * last context_len / 2 tokens again (main.cpp:83-87).  This call keeps the last `keep` cached positions instead: values
 * move to positions 0 .. keep-1, keys are rotated back by the dropped length (they are cached rotated), and decoding
 * continues at position `keep`.  The kept rows still carry what they attended to before, so the continuation is not the
 * one a fresh prompt pass over the kept tokens gives. */
int lcu_context_rollover(void* ctx, int keep);
/* the same move on one layer's caches ([n_heads][ctx_len][head_dim], keys rotated): rows [first, first + keep) to [0, keep) */
int lcu_rollover(void* k_cache_dev, void* v_cache_dev, int n_heads, int ctx_len, int head_dim, int first, int keep, void* stream);

/* ---- tensor-parallel decode (one process, 2 / 4 / 8 GPUs of one box) ---------------------------- */
/* No counterpart in the reference: its only multi-GPU scheme is the layer pipeline (llama_partition, llama_cu.cu:810-880,
 * 1099-1114), which keeps one GPU busy at a time at batch 1.  Here every GPU holds a run of rows of every layer matrix and
 * of the output matrix (whole heads of wq / wk / wv) and streams only those from its HBM; the slices of each activation row
 * travel as peer stores over NVLink from the GEMV epilogues, ordered by flag words with bounded waits (status 4 if a wait
 * expires).  Every output element is computed exactly as on one GPU, so tokens and probabilities equal those of an
 * lcu_context fed the same tokens one at a time.  n_heads, the ffn dim and n_vocab must split evenly
 * (lcu_tp_check_split, host only).  gpus: n_gpus device indices, NULL = 0 .. n_gpus-1.  A prompt runs as single-token steps. */
int lcu_tp_check_split(const void* params40, int n_gpus);
int lcu_tp_create(const void* params40, const int* gpus, int n_gpus, int context_len, float temperature, void** tp_out);
/* the values lcu_model_fill_synthetic gives the whole model, generated shard by shard */
int lcu_tp_fill_synthetic(void* tp, uint64_t seed, float scale);
/* every GPU reads its rows of every tensor file of a weight directory (llama_cu.cu:929-984 layout) */
int lcu_tp_load(void* tp, const char* dir);
/* llama_context::next_token / the chained loop / probabilities / clear_tokens / tokens_left, as for lcu_context_* */
int lcu_tp_next_token(void* tp, const int16_t* tokens_host, int n_tokens, int* token_out);
int lcu_tp_decode_chained(void* tp, int16_t first_token, int n_steps, int16_t* tokens_host_out, float* ms_out);
int lcu_tp_read_probs(void* tp, uint16_t* probs_host);
void lcu_tp_clear_tokens(void* tp);
int lcu_tp_tokens_left(void* tp);
int lcu_tp_kernels_per_step(void* tp);
uint64_t lcu_tp_weight_bytes_per_gpu(void* tp);
void lcu_tp_free(void* tp);

/* ---- tokenizer (host only) ------------------------------------------------------------------- */
/* llama_vocabulary(vocab file) + llama_vocabulary::tokenize(text, bos), llama_cu.cu:1319-1437: greedy highest-score pair
 * merging over UTF-8 characters with byte fallback (id = byte + 3), a leading space added when the text has none, id 1
 * first when bos != 0.  vocab file layout: extract.py:44-61.  Returns the number of ids (the first `capacity` of them are
 * written to ids_out), or -1 if the file cannot be mapped. */
int lcu_tokenize(const char* vocab_path, const char* text, int bos, int16_t* ids_out, int capacity);

/* ---- measurement ---------------------------------------------------------------------------- */
/* Times one decode kernel class over all layers of `model` in rotation (distinct weights every
 * launch, more than L2 holds), CUDA events on the launching stream.
 * which: 0 fused norm+wq|wk|wv+RoPE, 1 wo+residual, 2 fused norm+w1|w3+SiLU, 3 w2+residual, 4 output matrix.
 * Returns mean milliseconds per launch and the algorithmic bytes of one launch. */
int lcu_bench_decode_kernel(void* ctx, int which, int reps, float* ms_per_launch_out, uint64_t* bytes_per_launch_out);
/* cudaProfilerStart / cudaProfilerStop, so that a profiler attached with --profile-from-start off sees only the timed region */
int lcu_profiler_start(void);
int lcu_profiler_stop(void);
/* Self-test of the failure path: launches one warp that waits on an mbarrier nothing completes.  The bounded wait
 * expires after about one second of SM clock, the kernel ends normally, and the call returns status 4
 * (LCU_ERR_DEVICE_WAIT) with the device code (0x101) in *device_code_out; the context stays usable.  No counterpart
 * in the reference (its kernels have no waits). */
int lcu_selftest_bounded_wait(int* device_code_out);
/* The quantizer forms q = u8(roundf(127.5f + x / scale)) (transform.cu:60-80) with a reciprocal multiply, one residual
 * correction and trunc(v + 0.5f).  This entry compares that with the reference's IEEE division and roundf for EVERY pair
 * (x a finite half, scale a positive finite half, |x| within the absmax that rounds to the scale) on the device and
 * returns the number of pairs checked and the number of differing bytes (0). */
int lcu_selftest_quantizer_arithmetic(uint64_t* checked_out, uint64_t* differences_out);
/* Host arithmetic only (no device needed): how lcu_matmul_nt_f16 cuts out(m,n) = lhs(m,k) . rhs(n,k)^T for m <= 128 rows on
 * a GPU of `sms` SMs - the tile width (96 to 256 columns; the last tile may hang over n) and the split-K factor (1, 2 or 4,
 * 128-wide tiles only) - chosen so that one wave of CTAs streams the matrix in equal shares.  n a multiple of 128, k of 64. */
int lcu_plan_short_prompt_gemm(int n, int k, int sms, int* tile_n_out, int* split_out);
/* The same for m > 128 rows: *kernel_out = 0 for whole 256-row tiles per SM pair, 256 or 512 for the kernel that deals the K
 * steps of the last wave's tiles evenly over the pairs, with tiles that wide (estimates fitted to timings on B200). */
int lcu_plan_long_prompt_gemm(int m, int n, int k, int sms, int* kernel_out);
/* Host walk of that kernel's work list (no device needed) for n_tiles output tiles of k_steps 64-wide K steps on sm_pairs
 * pairs of SMs: 0 when every K step of every tile is run by exactly one pair, a pair hands partial sums over at most once,
 * and each shared tile's owner finds exactly the pairs that ran the rest of it, in order; a positive code names the rule
 * that failed, -1 bad arguments. */
int lcu_selftest_balanced_schedule(int n_tiles, int k_steps, int sm_pairs);
/* lcu_matmul_nt_f16_gated forms silu's a / (1 + expf(-a)) (llama_cu.cu:533-539) with a refined reciprocal and one
 * residual correction instead of the IEEE division.  This entry compares the two on the device for all 65536
 * half-precision a (the only values the gate meets) and returns how many were compared and how many differ (0). */
int lcu_selftest_silu_arithmetic(uint64_t* checked_out, uint64_t* differences_out);
/* lcu_matmul_nt_f16 (beta = 0, default stream) launched `reps` times back to back between two CUDA events on that
 * stream: mean milliseconds per launch.  Used to put the prompt GEMM against the tensor-core roofline. */
int lcu_bench_matmul_f16(void* out_dev, const void* lhs_dev, const void* rhs_dev, int m, int k, int n, int reps, float* ms_per_launch_out);
/* lcu_quantize_absmax_uint8 on a seeded fp16 matrix [h][w] resident in device memory, `reps` launches between two CUDA
 * events on the launching stream: mean milliseconds per launch (algorithmic traffic: 2 bytes read, 1 + 2/bs written per
 * element; use a matrix larger than the L2 cache) */
int lcu_bench_quantize(uint64_t h, uint64_t w, int bs, int reps, float* ms_per_launch_out);
/* pure-read ceiling: a kernel that only streams `bytes` from HBM with the same bulk-copy ring (16 KiB stages, each
 * fetched as copies_per_stage bulk copies, 1..32); ms per pass */
int lcu_bench_read_ceiling(uint64_t bytes, int reps, int copies_per_stage, float* ms_per_pass_out);

#ifdef __cplusplus
}
#endif
#endif /* LLAMA_CU_C_H */
