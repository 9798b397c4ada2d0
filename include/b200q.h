/*
 * b200q.h — C ABI of libb200q.so, the B200-native (sm_100a) generation engine that
 * replaces the arithmetic behind llmq's vLLM worker.
 *
 * The reference (iPieter/llmq) has NO FFI of its own: its hot path is four Python calls
 * into the un-vendored vLLM package (ref:llmq/workers/vllm_worker.py:105-123 engine
 * construction, :146 tokenizer, :161-165 sampling params, :183-186 engine.generate).
 * Each group of entry points below cites the reference call (or the vLLM op behind it)
 * that it replaces.  INTEGRATION.md shows the ctypes binding a maintainer would add.
 *
 * Conventions
 *   - extern "C", plain pointers and sizes, no torch / C++ types in any signature.
 *   - every function returns 0 on success or a negative B200Q_E* code; it never throws.
 *     b200q_last_error() returns a thread-local message for the last failure.
 *   - all `dev` pointers are device pointers owned by the caller (PyTorch is only the
 *     allocator); the library owns TMA descriptors, small metadata buffers and its
 *     scheduler state.
 *   - no hidden synchronisation in the op-level and model-level calls: work is enqueued
 *     on `stream` (a cudaStream_t passed as void*; NULL = legacy default stream).
 *     Engine-level calls (b200q_engine_step) synchronise their own stream because they
 *     hand token ids back to the host.
 *   - bf16 tensors are passed as `void*` / `const void*` (2-byte elements, row-major).
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200Q_VERSION 5

#define B200Q_OK 0
#define B200Q_EINVAL (-1)   /* bad argument / unsupported shape            */
#define B200Q_ECUDA (-2)    /* CUDA runtime / driver error                 */
#define B200Q_ENOMEM (-3)   /* KV pool or workspace exhausted              */
#define B200Q_ESTATE (-4)   /* call made in the wrong state (unbound etc.) */
#define B200Q_ENODEV (-5)   /* no sm_100 device present                    */

int b200q_version(void);
const char* b200q_last_error(void);
/* 0 if a CUDA device with compute capability 10.x is current, else B200Q_ENODEV. */
int b200q_device_check(void);

/* ------------------------------------------------------------------------------------
 * Op-level entry points (used by the parity tests and by b200q_model_forward).
 * Each replaces one op vLLM dispatches for the reference worker.
 * ---------------------------------------------------------------------------------- */

/* K1  embedding gather: out[t,:] = table[ids[t],:]            (vLLM VocabParallelEmbedding) */
int b200q_embed(const int32_t* ids_dev, const void* table_dev, void* out_dev,
                int T, int H, void* stream);
/* same, where ids[t] < 0 stands for prev_out_dev[-1 - ids[t]] — a token the previous step sampled
 * and left on the device (the engine enqueues step k+1 before reading step k's ids back, as
 * vLLM's async scheduling does: vllm/v1/worker/gpu_model_runner.py prev_sampled_token_ids);
 * scale > 0 and != 1 multiplies the row (Gemma normaliser), 0 = plain gather */
int b200q_embed_ex(const int32_t* ids_dev, const int32_t* prev_out_dev, const void* table_dev,
                   void* out_dev, int T, int H, float scale, void* stream);

/* K2  RMSNorm: y = bf16(bf16(x * rsqrt(mean(x^2)+eps)) * w)      (vllm/ir/ops/layernorm.py:9-21) */
int b200q_rmsnorm(const void* x_dev, const void* w_dev, void* y_dev,
                  int T, int H, float eps, void* stream);

/* K2' fused residual add + RMSNorm, in place:
 *     residual <- bf16(x + residual);  x <- rmsnorm(residual) * w
 *     (vllm/ir/ops/layernorm.py:39-58; rounding of the sum as in vLLM's _C kernel / HF) */
int b200q_add_rmsnorm(void* x_dev, void* residual_dev, const void* w_dev,
                      int T, int H, float eps, void* stream);

/* K4+K5  neox RoPE on q,k (in place on the fused qkv rows) and scatter of k,v into the
 *     paged KV cache.  qkv: [T, (n_q + 2*n_kv) * D]; cos_sin: bf16 [max_pos, D] (cos | sin);
 *     slot_mapping[t] = block * block_size + offset, or < 0 to skip the cache write.
 *     (vllm rotary_embedding/base.py:140-180 + _C_cache_ops.reshape_and_cache_flash) */
int b200q_rope_kvwrite(void* qkv_dev, const void* cos_sin_dev, const int32_t* positions_dev,
                       const int32_t* slot_mapping_dev, void* kv_layer_dev,
                       int T, int n_q, int n_kv, int D, int block_size, void* stream);

/* K7  paged decode attention (one query token per sequence, GQA).
 *     q rows are the first n_seqs rows of the fused qkv buffer (row stride q_stride elems);
 *     out: [n_seqs, n_q * D].  kv_layer: [num_blocks][2][n_kv][block_size][D] bf16, each
 *     token row stored with its 16-byte chunks XOR-swizzled by (token_in_block & 7).
 *     (replaces flashinfer trtllm_batch_decode_with_kv_cache, vllm flashinfer.py:1803) */
int b200q_decode_attn(const void* q_dev, int q_stride, void* out_dev, const void* kv_layer_dev,
                      const int32_t* block_table_dev, int bt_stride, const int32_t* ctx_lens_dev,
                      int n_seqs, int n_q, int n_kv, int D, int block_size, float scale,
                      void* stream);

/* K6  paged causal prefill attention over q-tiles of <=16 consecutive tokens of one sequence.
 *     tiles: int32[n_tiles][4] = {block_table_row, first_batch_row, n_rows, first_position}.
 *     (replaces flashinfer trtllm_batch_context_with_kv_cache, vllm flashinfer.py:1665) */
int b200q_prefill_attn(const void* q_dev, int q_stride, void* out_dev, const void* kv_layer_dev,
                       const int32_t* block_table_dev, int bt_stride, const int32_t* tiles_dev,
                       int n_tiles, int n_q, int n_kv, int D, int block_size, float scale,
                       void* stream);

/* K3/K8/K9/K11/K12  C[M,N] = A[M,K] * W[N,K]^T, bf16 in, fp32 accumulate in TMEM (tcgen05),
 *     bf16 out.  A, W, C row-major and contiguous; K % 64 == 0, N % 64 == 0.
 *     (replaces F.linear -> cuBLASLt, vllm/model_executor/layers/utils.py:92-98) */
int b200q_gemm_bf16(const void* A_dev, const void* W_dev, void* C_dev,
                    int M, int N, int K, void* stream);

/* Decode-sized batches: the split-K form of b200q_gemm_bf16 WITHOUT its reduce pass.  If the library
 *     would split the reduction for this shape, the fp32 partial tiles are left in its scratch
 *     (*partials = [splits][M][N], valid until the next split-K GEMM on the stream) and *splits > 1;
 *     the caller folds sum-in-split-order + bf16 rounding into the consumer (the two *_splitk ops
 *     below).  *splits == 1: nothing was launched, call b200q_gemm_bf16.  Results are bit-identical
 *     to the unfused sequence. */
int b200q_gemm_bf16_splitk(const void* A_dev, const void* W_dev, int M, int N, int K, void* stream,
                           const float** partials_dev, int* splits);
/* K2' reading x from split-K partials: residual <- bf16(bf16(sum_s partials[s]) + residual);
 *     x <- rmsnorm(residual) * w        (o-projection / down-projection -> next norm, one launch) */
int b200q_add_rmsnorm_splitk(void* x_dev, void* residual_dev, const void* w_dev,
                             const float* partials_dev, int splits, int T, int H, float eps,
                             void* stream);
/* K4+K5 reading the qkv rows from split-K partials (rotated q is written to qkv_dev) */
int b200q_rope_kvwrite_splitk(void* qkv_dev, const float* partials_dev, int splits,
                              const void* cos_sin_dev, const int32_t* positions_dev,
                              const int32_t* slot_mapping_dev, void* kv_layer_dev,
                              int T, int n_q, int n_kv, int D, int block_size, void* stream);

/* K9+K10 fused: out[M, N/2] = SwiGLU(A . W^T); W [N=2I, K] holds gate/up rows INTERLEAVED in blocks
 *     of 128: rows [256j, 256j+128) = gate rows [128j, 128j+128), rows [256j+128, 256j+256) = the
 *     matching up rows.  Rounding identical to b200q_gemm_bf16 followed by b200q_swiglu. */
int b200q_gemm_swiglu_bf16(const void* A_dev, const void* W_dev, void* C_dev,
                           int M, int N, int K, void* stream);

/* K10 SwiGLU: out[t,i] = bf16(bf16(silu(g[t,i])) * u[t,i]), gate_up = [T, 2I] = (g | u)
 *     (vllm activation.py:138-141 SiluAndMul.forward_native) */
int b200q_swiglu(const void* gate_up_dev, void* out_dev, int T, int I, void* stream);

/* row gather: out[i,:] = x[rows[i],:]  (last-token selection before the LM head) */
int b200q_gather_rows(const void* x_dev, const int32_t* rows_dev, void* out_dev,
                      int n, int H, void* stream);

/* K13 greedy sampler: ids[b] = argmax_v logits[b,v] over bf16 logits, lowest index wins ties
 *     (vllm/v1/sample/sampler.py:91,235-236 in the oracle's temperature-0 mode) */
int b200q_argmax_bf16(const void* logits_dev, int32_t* ids_dev, int B, int V, void* stream);

/* K13 sampler, the reference's default (temperature 0.7, no top-p/k;
 *     ref:llmq/workers/vllm_worker.py:161-165; vllm/v1/sample/ops/topk_topp_sampler.py:395-416:
 *     probs.div_(q).argmax, q ~ Exp(1)): ids[b] = argmax_v (logits[b,v]/T_b - log q_bv) with
 *     q_bv = -log(u), u from Philox4x32-10(key = seed_b, counter = (v/4, position_b, 0, 0)).
 *     params_dev: int32[B][4] = {float bits of temperature, seed lo, seed hi, position};
 *     temperature <= 0 selects the greedy argmax for that row. */
int b200q_sample_bf16(const void* logits_dev, const int32_t* params_dev, int32_t* ids_dev,
                      int B, int V, void* stream);

/* ---- Gemma-2 family (vllm/model_executor/models/gemma2.py) ----------------- */

/* embedding gather with the Gemma normaliser: out[t,:] = bf16(table[ids[t],:] * scale), scale =
 *     bf16(sqrt(H))                                                    (gemma2.py embed_tokens * normalizer) */
int b200q_embed_scaled(const int32_t* ids_dev, const void* table_dev, void* out_dev,
                       int T, int H, float scale, void* stream);

/* GemmaRMSNorm: y = bf16(x * rsqrt(mean(x^2)+eps) * (1 + w)), ONE rounding
 *     (vllm/model_executor/layers/layernorm.py GemmaRMSNorm.forward_static) */
int b200q_gemma_rmsnorm(const void* x_dev, const void* w_dev, void* y_dev,
                        int T, int H, float eps, void* stream);

/* Gemma-2 sandwich norms around the residual add, fused, in place:
 *     residual <- bf16(residual + gemma_rmsnorm(x, w_post));  x <- gemma_rmsnorm(residual, w_next)
 *     (post_attention_layernorm + pre_feedforward_layernorm, or post_feedforward_layernorm + the
 *     next layer's input_layernorm / the final norm; gemma2.py Gemma2DecoderLayer.forward) */
int b200q_gemma_norm_add_norm(void* x_dev, void* residual_dev, const void* w_post_dev,
                              const void* w_next_dev, int T, int H, float eps, void* stream);

/* K7/K6 with Gemma-2's attention extras: scores <- softcap * tanh(scores * scale / softcap)
 *     (softcap <= 0: off) and a sliding window: the query at position p sees keys j with
 *     p - window < j <= p (window <= 0: off).  D in {64, 128, 256}. */
int b200q_decode_attn_ex(const void* q_dev, int q_stride, void* out_dev, const void* kv_layer_dev,
                         const int32_t* block_table_dev, int bt_stride, const int32_t* ctx_lens_dev,
                         int n_seqs, int n_q, int n_kv, int D, int block_size, float scale,
                         float softcap, int window, void* stream);
int b200q_prefill_attn_ex(const void* q_dev, int q_stride, void* out_dev, const void* kv_layer_dev,
                          const int32_t* block_table_dev, int bt_stride, const int32_t* tiles_dev,
                          int n_tiles, int n_q, int n_kv, int D, int block_size, float scale,
                          float softcap, int window, void* stream);

/* fused gate_up GEMM + GeGLU: out = bf16(bf16(gelu_tanh(g)) * u), weight rows interleaved exactly as
 *     for b200q_gemm_swiglu_bf16                          (vllm activation.py GeluAndMul, approximate="tanh") */
int b200q_gemm_geglu_bf16(const void* A_dev, const void* W_dev, void* C_dev,
                          int M, int N, int K, void* stream);

/* final-logit soft-capping in place over n bf16 values, with the bf16 rounding of every eager op:
 *     l <- bf16(bf16(tanh(bf16(l / cap))) * cap)               (vllm logits_processor.py:66-69) */
int b200q_softcap_bf16(void* logits_dev, int64_t n, float cap, void* stream);

/* ---- layered architectures (B200Q_ARCH_RAMOPEL): op-level entry points ---------------------------
 * `dtype` (B200Q_DTYPE_*) is the element type of every `void*` matrix, activation and cache argument;
 * `float*` arguments are fp32 in both modes.  What the design wants exact (residual sum, norms, scores
 * and softmax, router, recurrent state and its gates) is fp32 in both; angles are fp64. */

/* x[t,:] = table[ids[t],:] * scale into the fp32 residual; ids < 0 as in b200q_embed_ex */
int b200q_embed_f32(const int32_t* ids_dev, const int32_t* prev_out_dev, const void* table_dev,
                    float* out_dev, int T, int W, float scale, int dtype, void* stream);
/* zero-centred RMS norm of fp32 rows, one or two weights at once (the two branches of a parallel
 * layer): y_k = x / sqrt(mean(x^2) + eps) * (1 + w_k); y2/w2 may be NULL; rows != NULL gathers
 * x[rows[i]] into y[i] */
int b200q_centered_rmsnorm(const float* x_dev, const int32_t* rows_dev, const float* w1_dev,
                           const float* w2_dev, void* y1_dev, void* y2_dev, int n, int W, float eps,
                           int dtype, void* stream);
/* C[m,n] = sum_k A[m,k] W[n,k] (+ bias[n]) for ANY M, N, K (fp32 accumulation in ascending k; true
 * fp32 products for fp32 operands).  bf16 shapes the tcgen05 GEMM takes (K, N multiples of 64, dense
 * rows, no bias, bf16 out) run on it.  out_f32: C is fp32 whatever dtype says. */
int b200q_linear(const void* A_dev, int lda, const void* W_dev, const float* bias_dev, void* C_dev, int ldc,
                 int M, int N, int K, int dtype, int out_f32, void* stream);
/* the same per batch index b (per-head weights): A + b*a_bs, W + b*w_bs, C + b*c_bs (strides in elements) */
int b200q_linear_batched(const void* A_dev, int lda, long long a_bs, const void* W_dev, long long w_bs,
                         void* C_dev, int ldc, long long c_bs, int M, int N, int K, int batch, int dtype,
                         int out_f32, void* stream);
/* the same per group g (expert): rows [group_off[g], group_off[g+1]) of C use W + g*w_gs and read row
 * a_rows[r] of A (a_rows NULL: row r); max_rows bounds a group's rows.  With the tile table of
 * b200q_moe_route (tile_tab / n_tiles, may be NULL), a_rows NULL and bf16 shapes the tensor-core form takes,
 * the groups run on b200q_gemm_grouped_bf16. */
int b200q_linear_grouped(const void* A_dev, int lda, const int32_t* a_rows_dev, const void* W_dev,
                         long long w_gs, void* C_dev, int ldc, const int32_t* group_off_dev, int groups,
                         int max_rows, int N, int K, int dtype, const void* tile_tab_dev,
                         const int32_t* n_tiles_dev, void* stream);
/* the tensor-core form behind the batched and grouped linears (bf16 operands, fp32 accumulation; C bf16 or
 * fp32):  C[row, g*c_gx + n] = sum_k A[row, g*a_gx + k] * W[g*N + n, k].  tab_dev != NULL: the m-tiles
 * {group, first row, end row, 0} as b200q_moe_route wrote them (n_mt_dev of them, at most max_mtiles);
 * tab_dev == NULL: `groups` groups of rows [0, M).  A is [a_rows, lda].  b200q_gemm_grouped_ok says whether
 * the shapes are taken (K, N multiples of 64; operands and slices 16-byte aligned). */
int b200q_gemm_grouped_bf16(const void* A_dev, long long a_rows, long long lda, int a_gx, const void* W_dev,
                            int groups, void* C_dev, long long ldc, int c_gx, int M, int N, int K,
                            const void* tab_dev, const int32_t* n_mt_dev, int max_mtiles, int out_f32,
                            void* stream);
int b200q_gemm_grouped_ok(const void* A_dev, long long lda, int a_gx, const void* W_dev, const void* C_dev,
                          long long ldc, int c_gx, int N, int K, int out_f32);
/* latent attention 1/3: proj row = [query latent | kv latent | shared rotated key part];
 *     cq = rmsnorm(query latent) * w_qn;  cache row slot_mapping[t] = [rmsnorm(kv latent) * w_kvn |
 *     rotate(key part)], pairs (2i, 2i+1) of the first rot_dims entries turned by position * freq[i]
 *     (freq: fp64 [rot_dims/2]).  has_kv = 0: query part only (the layer reads another layer's cache). */
int b200q_latent_prep(const void* proj_dev, int ldp, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                      const double* freq_dev, const int32_t* positions_dev, const int32_t* slot_mapping_dev,
                      const float* w_qn_dev, const float* w_kvn_dev, void* cq_dev, void* cache_dev,
                      int has_kv, int T, float eps, int dtype, void* stream);
/* latent attention 2/3: rotated query parts, turned, into qa[t, h, kv_rank:] (qa: fp32 [T, heads,
 *     kv_rank + rot_dim]; its first kv_rank entries are W_uk[h]^T q_unrotated, written by a batched linear) */
int b200q_rope_pairs_q(const void* q_dev, int heads, int dim, int rot_dim, int rot_dims, const double* freq_dev,
                       const int32_t* positions_dev, float* qa_dev, int kv_rank, int T, int dtype, void* stream);
/* latent attention 3/3: out[t,h,:] = softmax_j(scale * qa[t,h] . row_j) . latent_j over the keys
 *     max(0, p - window + 1) <= j <= p of the token's sequence (window 0: all), rows read through the
 *     block table (cache: [blocks][block_size][kv_rank + rot_dim]); out [T, heads, kv_rank] */
int b200q_latent_attn(const float* qa_dev, const void* cache_dev, const int32_t* block_table_dev, int bt_stride,
                      const int32_t* row_seq_dev, const int32_t* positions_dev, int T, int heads, int kv_rank,
                      int rot_dim, int block_size, int window, float scale, void* out_dev, int dtype,
                      void* stream);
/* generalized delta rule over the sequences of a step (seq_desc as in b200q_batch); proj row =
 *     [r | k | v | g | a | z] (heads*D each, z: Rk); state: fp32 [slots] x slot_stride, this layer's part
 *     [heads][D][D] at the start of a slot.  Per token and head:
 *     w = exp(-e^-1/2 sigmoid(w0 + W2 tanh z)), a = sigmoid(a + a_bias), u = k / sqrt(sum k^2 + 1e-6),
 *     S <- diag(w) S - (a*u)(u^T S) + k v^T, o = S^T r, out = o / rms(o) * out_norm * sigmoid(g).
 *     scratch (fp32, 6*T*heads*D, may be NULL) with the step's row count T lets D = 32/64/128 run as three
 *     launches: the state-independent vectors of all T rows at once, the bare recurrence, norm and gate */
int b200q_delta_rule(const void* proj_dev, int ldp, const void* w2_dev, const float* w0_dev,
                     const float* a_bias_dev, const float* out_norm_dev, float* state_dev, long long slot_stride,
                     const int32_t* seq_desc_dev, int n_seqs, int heads, int D, int Rk, float eps, void* out_dev,
                     int dtype, float* scratch_dev, int T, void* stream);
/* PolyNorm over rows of F values: y = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3, N(v) = v / sqrt(mean(v^2) + eps) */
int b200q_polynorm(const void* z_dev, const float* coef_dev, void* y_dev, int rows, int F, float eps, int dtype,
                   void* stream);
/* clamped gated unit: gate_up row = [g (F) | u (F)]; y = g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit),
 *     u' = clamp(u, -limit, limit) */
int b200q_clamped_glu(const void* gate_up_dev, void* y_dev, int64_t rows, int F, float limit, int dtype,
                      void* stream);
/* top-k routing over fp32 router logits [T, E]: idx/wts [T, top] (softmax over the chosen logits), and the
 *     grouping of the T*top (token, choice) pairs by expert: group_off [E+1], perm_tok [T*top] (token of the
 *     pair at each sorted position), pair_pos [T*top] (sorted position of pair t*top+k); optionally (NULL: not
 *     written) the 128-row tiles of the groups for b200q_gemm_grouped_bf16: tile_tab [(T*top)/128 + E][4] =
 *     {expert, first sorted row, end row of the expert, 0} and their count n_tiles [1] */
int b200q_moe_route(const float* logits_dev, int T, int E, int top, int32_t* idx_dev, float* wts_dev,
                    int32_t* group_off_dev, int32_t* perm_tok_dev, int32_t* pair_pos_dev, int32_t* tile_tab_dev,
                    int32_t* n_tiles_dev, void* stream);
/* end of a parallel layer: x += mix + ff; ff = f (dense) or sum_k wts[t,k] expert_out[pair_pos[t*top+k]]
 *     (+ sigmoid(shared_gate[t]) shared_out[t]); unused parts NULL */
int b200q_layer_sum(float* x_dev, const void* mix_dev, const void* f_dev, const void* expert_out_dev,
                    const int32_t* pair_pos_dev, const float* wts_dev, int top, const void* shared_out_dev,
                    const float* shared_gate_dev, int T, int W, int dtype, void* stream);
/* moe_route with the scoring of the chosen experts selectable: score_mode 0 = softmax over the chosen logits,
 * 1 = sigmoid of each chosen logit (not renormalised) */
int b200q_moe_route_ex(const float* logits_dev, int T, int E, int top, int score_mode, int32_t* idx_dev,
                       float* wts_dev, int32_t* group_off_dev, int32_t* perm_tok_dev, int32_t* pair_pos_dev,
                       int32_t* tile_tab_dev, int32_t* n_tiles_dev, void* stream);

/* ---- post-norm layers, carried convolutions, and mixers 3-5 (sequence_ops.cu, chunk_attn.cu) ------------------------------
 * seq_desc / row_seq as in b200q_batch.  `state` arguments point at the op's own region inside slot 0 of the
 * fp32 state pool; slot s is `slot_stride` floats further.  A sequence whose portion starts at position 0
 * starts from zeros whatever its slot holds. */

/* x[t,:] = table[ids[t],:] + pos_table[positions[t],:] into the fp32 residual (pos_table NULL: none) */
int b200q_embed_pos_f32(const int32_t* ids_dev, const int32_t* prev_out_dev, const void* table_dev,
                        const void* pos_table_dev, const int32_t* positions_dev, float* out_dev, int T, int W,
                        int dtype, void* stream);
/* grouped RMS norm of v = alpha * x + scale * add:  y = v / sqrt(mean_part(v^2) + eps) * w, the mean taken
 * over each of `groups` equal consecutive parts of the row.  add (model dtype, may be NULL): row r, or with
 * pair_pos the sum over k < top of rows pair_pos[r*top + k] (the routed experts' outputs).  scale NULL = 1.
 * rows != NULL gathers x[rows[i]] into output row i.  y_f32 and / or y_t (model dtype) receive the result;
 * y_f32 may be x itself. */
int b200q_group_rmsnorm(const float* x_dev, const int32_t* rows_dev, const void* add_dev,
                        const int32_t* pair_pos_dev, int top, const float* scale_dev, float alpha,
                        const float* w_dev, int groups, float eps, float* y_f32_dev, void* y_t_dev, int n, int W,
                        int dtype, void* stream);
/* per-channel causal convolution over the tokens of each sequence's portion, continued from the last
 * taps - 1 inputs the sequence left in its state slot:
 *   y[t,c] = act( bias[c] + sum_j w[c,j] * in[t - taps + 1 + j, c] ) (+ in[t,c] if add_input)
 * in: [T, ld_in] (fp32 if in_f32, else model dtype), w: fp32 [C, taps], out: [T, ld_out] (fp32 if out_f32).
 * act 0 = none, 1 = SiLU.  The state is advanced by a second launch after the outputs are written. */
int b200q_causal_conv(const void* in_dev, int ld_in, int in_f32, const float* w_dev, const float* bias_dev,
                      int C, int taps, int act, int add_input, float* state_dev, long long slot_stride,
                      const int32_t* seq_desc_dev, const int32_t* row_seq_dev, int n_seqs, void* out_dev,
                      int ld_out, int out_f32, int T, int dtype, void* stream);
/* gated delta rule.  qkv: fp32 [T, 2*kv_heads*dim + heads*vdim] = (q | k | v) after convolution and SiLU
 * (q and k are normalised in place); ba: fp32 [T, 2*heads] = (beta logits | decay inputs), turned into
 * (beta | g) in place; raw: fp32 scratch [T, heads*vdim]; gate: model dtype rows (ld_gate) of heads*vdim
 * output gate logits.  Per head h (q/k head h / (heads/kv_heads)):
 *   q <- q / sqrt(sum q^2 + 1e-6) * dim^-1/2,  k <- k / sqrt(sum k^2 + 1e-6),  beta = sigmoid(.),
 *   g = exp(-exp(a_log[h]) * softplus(a + dt_bias[h]));  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;
 *   o = S^T q;  out = o / sqrt(mean(o^2) + eps) * out_norm * silu(gate)
 * state: fp32 [heads][dim][vdim] per slot. */
int b200q_gated_delta(float* qkv_dev, float* ba_dev, float* raw_dev, const void* gate_dev, int ld_gate,
                      const float* a_log_dev, const float* dt_bias_dev, const float* out_norm_dev,
                      float* state_dev, long long slot_stride, const int32_t* seq_desc_dev, int n_seqs, int heads,
                      int kv_heads, int dim, int vdim, float eps, void* out_dev, int T, int dtype, void* stream);
/* chunk attention 1/2: proj row = [q (heads*dim) | k (kv_heads*dim) | ...];  qs[t,h,:] = q / rms(q) * w_qn *
 * w_kn (fp32; the key norm's weight is carried by the query so that the cache holds the raw keys, which are
 * also the values);  cache row slot_mapping[t] = k as projected (model dtype, [kv_heads*dim]) */
int b200q_chunk_attn_prep(const void* proj_dev, int ldp, int heads, int kv_heads, int dim, const float* w_qn_dev,
                          const float* w_kn_dev, const int32_t* slot_mapping_dev, float* qs_dev, void* cache_dev,
                          int T, float eps, int dtype, void* stream);
/* chunk attention 2/2: for token t at position p of its sequence, over keys j in [lo, p], lo = p - p % chunk
 * (chunk 0: lo = 0):  s_j = (qs . k_j) / sqrt(mean(k_j^2) + eps) * scale;  s_j <- softcap tanh(s_j / softcap);
 * s_j -= r1[h] * log(1 + r2[h] * (p - j));  w_j = exp(s_j) / (1 + sum exp(s));  out[t,h,:] = (sum_j w_j k_j) *
 * sigmoid(gate[t,h,:]).  gate: model dtype rows with stride ld_gate. */
int b200q_chunk_attn(const float* qs_dev, const void* cache_dev, const int32_t* block_table_dev, int bt_stride,
                     const int32_t* row_seq_dev, const int32_t* positions_dev, int T, int heads, int kv_heads,
                     int dim, int block_size, int chunk, float scale, float softcap, const float* r1_dev,
                     const float* r2_dev, const void* gate_dev, int ld_gate, float eps, void* out_dev, int dtype,
                     void* stream);
/* the same with the per-sequence view of the step (seq_desc / n_seqs; row r of the block table is sequence r):
 * bf16 caches with a head size of 64 or 128 then run on the tensor cores, 16 consecutive tokens of a sequence per
 * tile (results equal the form above up to rounding: the queries and the softmax weights are rounded to bf16) */
int b200q_chunk_attn_seq(const float* qs_dev, const void* cache_dev, const int32_t* block_table_dev, int bt_stride,
                         const int32_t* row_seq_dev, const int32_t* positions_dev, const int32_t* seq_desc_dev,
                         int n_seqs, int T, int heads, int kv_heads, int dim, int block_size, int chunk, float scale,
                         float softcap, const float* r1_dev, const float* r2_dev, const void* gate_dev, int ld_gate,
                         float eps, void* out_dev, int dtype, void* stream);
/* selective scan.  x: model dtype [T, inner] (after convolution and SiLU); dt_raw: fp32 [T, inner] (before
 * softplus), dt_bias: fp32 [inner] added to it (NULL: none); bc: model dtype rows (ld_bc) whose entries [b_off, b_off + N) are B and
 * [b_off + N, b_off + 2N) are C; z: model dtype rows (ld_z); a_log: fp32 [inner, N]; d: fp32 [inner].
 *   dt = softplus(dt_raw + dt_bias);  S[c,n] <- exp(dt_c * -exp(a_log[c,n])) S[c,n] + dt_c x_c B_n;
 *   y_c = sum_n S[c,n] C_n + d_c x_c;  out = y * silu(z).     state: fp32 [N][inner] per slot.  T = rows of the
 *   step (T > n_seqs: prompt portions are present and a channel's state is split over four lanes). */
int b200q_selective_scan(const void* x_dev, const float* dt_raw_dev, const float* dt_bias_dev, const void* bc_dev,
                         int ld_bc, int b_off,
                         const void* z_dev, int ld_z, const float* a_log_dev, const float* d_dev, float* state_dev,
                         long long slot_stride, const int32_t* seq_desc_dev, int n_seqs, int inner, int N,
                         void* out_dev, int T, int dtype, void* stream);
/* routed experts whose weight scales the INPUT: dst[pair_pos[p], :] = src[p / top, :] * wts[p] for every
 * (token, choice) pair p < T*top (rows land in expert order for the grouped linear) */
int b200q_scatter_scaled_rows(const void* src_dev, const int32_t* pair_pos_dev, const float* wts_dev, int top,
                              void* dst_dev, int T, int W, int dtype, void* stream);
/* gated unit: gate_up row = [g (F) | u (F)]; y = silu(g) * u */
int b200q_silu_glu(const void* gate_up_dev, void* y_dev, int64_t rows, int F, int dtype, void* stream);
/* ---- pre-norm layers, token shift, and mixers 6-8 (prenorm_ops.cu, decay_attn.cu, window_attn.cu) -------------------------
 * seq_desc / row_seq / state conventions as above. */

/* plain RMS norm of fp32 rows, optionally followed by a token shift:
 *   n[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w;   y[t] = n[t] + (n[t-1] - n[t]) * shift       (shift NULL: y = n)
 * n[t-1] of a portion's first token is read from the sequence's state slot (zeros at position 0).  The n of a
 * sequence's last token replaces it: a portion of ONE token stores it in the slot itself (reader and writer are
 * the same thread), a longer portion leaves it in carry [n_seqs, W], and b200q_store_carry (skip_single = 1) moves
 * it into the slot once every reader of the old value has run — a step of single tokens needs no second launch.
 * rows != NULL (only without shift) gathers x[rows[i]] into output row i.
 * y_t (model dtype) and / or y_f32 receive the result. */
int b200q_rmsnorm_shift(const float* x_dev, const int32_t* rows_dev, const float* w_dev, const float* shift_dev,
                        float* state_dev, long long slot_stride, const int32_t* seq_desc_dev,
                        const int32_t* row_seq_dev, int n_seqs, float* carry_dev, void* y_t_dev, float* y_f32_dev,
                        int n, int W, float eps, int dtype, void* stream);
/* state[slot of sequence s][0..W) <- src row of s: last_rows = 1: the last row of the sequence's portion in a
 * [T, W] buffer; 0: row s of a [n_seqs, W] buffer.  skip_single = 1 leaves portions of one token alone. */
int b200q_store_carry(const float* src_dev, int last_rows, float* state_dev, long long slot_stride,
                      const int32_t* seq_desc_dev, int n_seqs, int W, int skip_single, void* stream);
/* n_mix blends of every row with the previous token's row: out[t, s*W + c] = h[t,c] + (h[t-1,c] - h[t,c]) *
 * mu[s*W + c]; h fp32 [T, W]; h[t-1] of a portion's first token from the state slot (zeros at position 0);
 * out [T, n_mix*W] in the model dtype.  store_single = 1: a portion of one token also stores its row in the slot
 * (the rows of longer portions are stored by b200q_store_carry with last_rows = 1, skip_single = 1) */
int b200q_shift_blend(const float* h_dev, const float* mu_dev, int n_mix, float* state_dev,
                      long long slot_stride, const int32_t* seq_desc_dev, const int32_t* row_seq_dev, int store_single,
                      void* out_dev, int T, int W, int dtype, void* stream);
/* z <- relu(z)^2 in place over n values */
int b200q_relu2(void* z_dev, int64_t n, int dtype, void* stream);
/* out = tanh(in) (fp32 in, model dtype out) */
int b200q_tanh_cast(const float* in_dev, void* out_dev, int64_t n, int dtype, void* stream);
/* out[t, 0..C) = act(in[t, 0..C)) into fp32 rows; act 0 = none, 1 = SiLU */
int b200q_act_to_f32(const void* in_dev, int ld_in, float* out_dev, int ld_out, int C, int act, int T, int dtype,
                     void* stream);
/* w <- exp(-exp(w + w0)) in place over fp32 rows of C values (row stride ldw; the fp32 model evaluates it
 * through fp64) */
int b200q_decay_from_logits(float* w_dev, int ldw, const float* w0_dev, int C, int T, int dtype, void* stream);
/* linear attention with decay over the sequences of a step.  qkv: fp32 rows (ldq) holding q at q_off (heads*dim), k at
 * k_off (heads*dim), v at v_off (heads*vdim).  state: fp32 [heads][dim][vdim] per slot.
 *   head_decay != NULL (fp32 [heads]):    S <- decay_h S + k v^T;  o = S^T q
 *   w != NULL (fp32 rows ldw, [heads*dim]), bonus fp32 [heads*dim]:   o = (S + diag(bonus) k v^T)^T q;  S <- diag(w) S + k v^T
 * raw: fp32 [T, heads*vdim] */
int b200q_decay_attn(const float* qkv_dev, int ldq, int q_off, int k_off, int v_off, const float* head_decay_dev,
                     const float* w_dev, int ldw, const float* bonus_dev, float* state_dev, long long slot_stride,
                     const int32_t* seq_desc_dev, int n_seqs, int heads, int dim, int vdim, float* raw_dev,
                     void* stream);
/* out[t, c] = raw[t, c] / sqrt(mean over c's group of raw^2 + eps) * w[c] * act(gate[t, c]); groups are `group`
 * consecutive values of the C in a row; gate: model dtype rows (ld_gate); gate_act 0 = sigmoid, 1 = SiLU */
int b200q_gated_rmsnorm(const float* raw_dev, int C, int group, const float* w_dev, const void* gate_dev,
                        int ld_gate, int gate_act, float eps, void* out_dev, int T, int dtype, void* stream);
/* window attention 1/2: proj row = [q (heads*dim) | k (kv_heads*dim) | v (kv_heads*vdim) | ...].  The first rot_dims
 * dimensions of every q and k head are turned, dimension i with i + rot_dims/2, by position * freq[i] (freq: fp64
 * [rot_dims/2]; rot_dims 0: none).  qs[t,h,:] = turned q * scale * temp[h] (fp32; temp NULL = 1); cache row
 * slot_mapping[t] = [turned k | v] in the model dtype ([kv_heads*dim + kv_heads*vdim]) */
int b200q_window_attn_prep(const void* proj_dev, int ldp, int heads, int kv_heads, int dim, int vdim, int rot_dims,
                           const double* freq_dev, const int32_t* positions_dev, const int32_t* slot_mapping_dev,
                           const float* temp_dev, float scale, float* qs_dev, void* cache_dev, int T, int dtype,
                           void* stream);
/* window attention 2/2: for token t at position p over keys max(0, p - window + 1) <= j <= p (window 0: all):
 * out[t,h,:] = softmax_j(qs[t,h] . k_j) . v_j * sigmoid(gate[t,h]) (gate: model dtype rows with one value per
 * head, stride ld_gate; NULL: no gate).  bf16 caches with dim, vdim in {64, 128} run on the tensor cores. */
int b200q_window_attn(const float* qs_dev, const void* cache_dev, const int32_t* block_table_dev, int bt_stride,
                      const int32_t* row_seq_dev, const int32_t* positions_dev, const int32_t* seq_desc_dev,
                      int n_seqs, int T, int heads, int kv_heads, int dim, int vdim, int block_size, int window,
                      const void* gate_dev, int ld_gate, void* out_dev, int dtype, void* stream);
/* routing of the grouped mixture over fp32 router logits [T, E]: s = softmax(logits); choice = s + correction;
 * only experts of the keep best of n_groups equal groups (group score = largest choice in it) may be chosen;
 * the top largest choices (ties: lowest index) -> idx; wts = s of the chosen / (their sum + 1e-20).  Grouping
 * outputs as in b200q_moe_route over E groups; the tile table lists the first e_gemm experts only (the rest are
 * identity experts that run no product). */
int b200q_moe_route_grouped(const float* logits_dev, const float* correction_dev, int T, int E, int e_gemm, int top,
                            int n_groups, int keep, int32_t* idx_dev, float* wts_dev, int32_t* group_off_dev,
                            int32_t* perm_tok_dev, int32_t* pair_pos_dev, int32_t* tile_tab_dev,
                            int32_t* n_tiles_dev, void* stream);
/* x += a_scale * a (+ b_scale * b, b may be NULL); a, b in the model dtype */
int b200q_residual_add(float* x_dev, const void* a_dev, float a_scale, const void* b_dev, float b_scale, int T, int W,
                       int dtype, void* stream);
/* x += a_scale * a (+ b_scale * b), then y = x / sqrt(mean(x^2) + eps) * w (model dtype) in the same pass */
int b200q_residual_add_rmsnorm(float* x_dev, const void* a_dev, float a_scale, const void* b_dev, float b_scale,
                               const float* w_dev, void* y_dev, int T, int W, float eps, int dtype, void* stream);
/* x[t] += sum_k wts[t,k] * (idx[t,k] < n_real ? expert_out[pair_pos[t*top+k]] : h[t]) */
int b200q_residual_add_routed(float* x_dev, const void* expert_out_dev, const int32_t* pair_pos_dev,
                              const int32_t* idx_dev, const float* wts_dev, int top, int n_real, const void* h_dev,
                              int T, int W, int dtype, void* stream);
/* out[t] = [a[t] | b[t]] (fp32 rows of W each) in the model dtype, [T, 2W] */
int b200q_concat_cast(const float* a_dev, const float* b_dev, void* out_dev, int T, int W, int dtype, void* stream);
/* l <- cap * tanh(l / cap) in place over n fp32 values */
int b200q_softcap_f32(float* logits_dev, int64_t n, float cap, void* stream);
int b200q_argmax_f32(const float* logits_dev, int32_t* ids_dev, int B, int V, void* stream);
int b200q_f32_to_bf16(const float* in_dev, void* out_dev, int64_t n, void* stream);
int b200q_copy_f32(const float* in_dev, float* out_dev, int64_t n, void* stream);

/* ---- sandwich layers and the options of window / latent attention (sandwich_ops.cu) ----------------------------- */

/* rotation frequencies as b200q_layer_desc describes them (host only): freq_out fp64 [rot_dims/2], *mag_out the
 * factor of sine and cosine */
int b200q_rot_frequencies(int rot_dims, double base, double factor, double original, double fast, double slow,
                          double* freq_out, float* mag_out);
/* y[i] = norm(x[rows ? rows[i] : i]) in the model dtype; kind B200Q_NORM_DYT (w = [w | b | alpha]), B200Q_NORM_RMS
 * (w = [w]) or B200Q_NORM_CAST (w unused) */
int b200q_row_norm(const float* x_dev, const int32_t* rows_dev, int kind, const float* w_dev, void* y_dev, int n,
                   int W, float eps, int dtype, void* stream);
/* x[t] += mult * post(y[t] + bias) over fp32 rows x and model-dtype rows y (bias fp32 [W] or NULL; post_kind
 * B200Q_NORM_DYT or B200Q_NORM_RMS with weights post_w), then out[t] = next(x[t]) in the model dtype (next_kind any
 * B200Q_NORM_*; B200Q_NORM_NONE: no output) — the sum that closes a sublayer and the norm that opens the next */
int b200q_sandwich_add(float* x_dev, const void* y_dev, const float* bias_dev, int post_kind, const float* post_w_dev,
                       float mult, int next_kind, const float* next_w_dev, void* out_dev, int T, int W, float eps,
                       int dtype, void* stream);
/* v[i] *= a */
int b200q_scale_f32(float* v_dev, int64_t n, float a, void* stream);
/* gated unit: gate_up row = [g (F) | u (F)]; y = gelu_tanh(g) * u */
int b200q_gelu_glu(const void* gate_up_dev, void* y_dev, int64_t rows, int F, int dtype, void* stream);
/* the same over rows whose gate and up values are interleaved in blocks of `block` columns ([g | u | g | u ...], the
 * layout of b200q_gemm_geglu_bf16's weight rows; block 0 = [g (F) | u (F)]; block must divide F) */
int b200q_gelu_glu_ex(const void* gate_up_dev, void* y_dev, int64_t rows, int F, int block, int dtype, void* stream);
/* per-layer token input: out[t, j] = gelu_tanh(g[t, j]) * table[id(t), col0 + j], j < D (ids < 0 as in b200q_embed_ex;
 * g rows of stride ldg, table rows of stride ld_table, both in the model dtype) */
int b200q_token_side_gate(const void* g_dev, int ldg, const int32_t* ids_dev, const int32_t* prev_out_dev,
                          const void* table_dev, int ld_table, int col0, void* out_dev, int T, int D, int dtype,
                          void* stream);
/* b200q_window_attn_prep with options: proj row = [q | k | v] at q_off / k_off / v_off (k_off < 0: the layer reads
 * another layer's cache and writes none); bias fp32 (indexed like a proj row) or NULL; qk_norm as in
 * b200q_layer_desc with weights w_qn / w_kn, before rotation; sine and cosine times mag; the query at position p
 * also times 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (temp_every 0: off) */
int b200q_window_attn_prep_ex(const void* proj_dev, int ldp, int q_off, int k_off, int v_off, const float* bias_dev,
                              int heads, int kv_heads, int dim, int vdim, int qk_norm, const float* w_qn_dev,
                              const float* w_kn_dev, float eps, int rot_dims, const double* freq_dev, float mag,
                              const int32_t* positions_dev, const int32_t* slot_mapping_dev, const float* temp_dev,
                              float scale, float temp_coef, int temp_every, float* qs_dev, void* cache_dev, int T,
                              int dtype, void* stream);
/* b200q_window_attn with options: key j <= p is visible when p - j < window or j < keep_first (window 0: every
 * j <= p); scores <- softcap * tanh(scores / softcap) before the softmax (softcap 0: off) */
int b200q_window_attn_ex(const float* qs_dev, const void* cache_dev, const int32_t* block_table_dev, int bt_stride,
                         const int32_t* row_seq_dev, const int32_t* positions_dev, const int32_t* seq_desc_dev,
                         int n_seqs, int T, int heads, int kv_heads, int dim, int vdim, int block_size, int window,
                         int keep_first, float softcap, const void* gate_dev, int ld_gate, void* out_dev, int dtype,
                         void* stream);
/* b200q_latent_prep with q_rank = 0 allowed (full-rank queries: no query latent) and sine / cosine times mag */
int b200q_latent_prep_ex(const void* proj_dev, int ldp, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                         const double* freq_dev, float mag, const int32_t* positions_dev,
                         const int32_t* slot_mapping_dev, const float* w_qn_dev, const float* w_kvn_dev, void* cq_dev,
                         void* cache_dev, int has_kv, int T, float eps, int dtype, void* stream);
/* b200q_rope_pairs_q over query rows of stride ldq, sine / cosine times mag */
int b200q_rope_pairs_q_ex(const void* q_dev, int ldq, int heads, int dim, int rot_dim, int rot_dims,
                          const double* freq_dev, float mag, const int32_t* positions_dev, float* qa_dev, int kv_rank,
                          int T, int dtype, void* stream);
/* b200q_latent_attn whose head outputs are multiplied by sigmoid(gate[t, h]) (model dtype rows of stride ld_gate; NULL:
 * no gate) */
int b200q_latent_attn_ex(const float* qa_dev, const void* cache_dev, const int32_t* block_table_dev, int bt_stride,
                         const int32_t* row_seq_dev, const int32_t* positions_dev, int T, int heads, int kv_rank,
                         int rot_dim, int block_size, int window, float scale, const void* gate_dev, int ld_gate,
                         void* out_dev, int dtype, void* stream);

/* ------------------------------------------------------------------------------------
 * Model-level: one forward step over a mixed decode+prefill token batch.
 * Replaces GPUModelRunner.execute_model for LlamaForCausalLM
 * (vllm/model_executor/models/llama.py:316-333,395-431).
 * ---------------------------------------------------------------------------------- */

typedef struct b200q_model_config {
  int32_t hidden;        /* H                              */
  int32_t n_layers;      /* L                              */
  int32_t n_q_heads;
  int32_t n_kv_heads;
  int32_t head_dim;      /* 64, 128 or 256                 */
  int32_t intermediate;  /* I                              */
  int32_t vocab;         /* V                              */
  int32_t block_size;    /* KV page size in tokens (16)    */
  int32_t max_tokens;    /* workspace capacity: max tokens per step */
  int32_t max_seqs;      /* max sequences per step (block-table rows, sampled rows) */
  int32_t max_pos;       /* rows of the RoPE table         */
  int32_t tie_embeddings;/* 1: lm_head shares embed_tokens */
  float rms_eps;
  float attn_scale;      /* 1/sqrt(head_dim); gemma2: query_pre_attn_scalar^-0.5 */
  /* architecture extras; all zero = Llama */
  int32_t arch;           /* B200Q_ARCH_LLAMA | B200Q_ARCH_GEMMA2                                   */
  int32_t sliding_window; /* gemma2: even layers see only the last `sliding_window` keys; 0 = off   */
  float attn_softcap;     /* attention logit soft-capping (gemma2: 50); 0 = off                     */
  float final_softcap;    /* final logit soft-capping (gemma2: 30); 0 = off                         */
  float embed_scale;      /* embeddings are multiplied by this value (gemma2: bf16(sqrt(H))); 0 = off */
  /* layered architectures (B200Q_ARCH_RAMOPEL); zero elsewhere */
  int32_t dtype;          /* B200Q_DTYPE_BF16 | B200Q_DTYPE_F32: element type of matrices, activations, cache */
  int32_t max_logit_rows; /* rows of the fp32 logits buffer (0 = max_seqs); a replayed step may ask for the
                             logits of any of its rows                                                     */
  int32_t state_slots;    /* recurrent-state slots (one per live sequence); 0 = max_seqs                    */
  /* form of a layer (layered architectures); all zero = parallel pre-norm layers                            */
  int32_t layer_form;     /* B200Q_FORM_PARALLEL | B200Q_FORM_POSTNORM                                       */
  int32_t norm_groups;    /* post-norm form: the RMS norms (layers and final) are taken over this many equal
                             consecutive parts of a row; 0 / 1 = the whole row                               */
  float residual_alpha;   /* post-norm form: x <- norm(alpha * x + scale * sublayer(x))                      */
  int32_t input_taps;     /* post-norm form: every sublayer reads h + conv(h), a per-channel causal
                             convolution over time with this many taps ("canon1" / "canon2"); 0 = reads x    */
  int32_t learned_pos;    /* 1: a learned position table "pos" [>= max_pos, W] is added to the embedding     */
  int32_t token_shift;    /* pre-norm form, 1: the mixer reads h + (h_prev - h) * shift ("shift" [1, W] per layer),
                             h_prev = the previous token's normed row (zeros before the first token)           */
  float logit_softcap;    /* layered architectures: logits <- cap * tanh(logits / cap); 0 = off                */
  /* sandwich form (zero elsewhere) */
  int32_t norm_kind;      /* B200Q_NORM_RMS | B200Q_NORM_DYT: the norm on both sides of every sublayer and the final one */
  float residual_mult;    /* every sublayer's normed output is multiplied by this before it joins x; 0 = 1      */
  int32_t side_dim;       /* per-layer token input: columns of the second embedding table a layer reads; 0 = none */
  float logit_scale;      /* layered architectures: logits are multiplied by this; 0 = 1                        */
} b200q_model_config;

#define B200Q_ARCH_LLAMA 0
#define B200Q_ARCH_GEMMA2 1
/* Ramopel: a layered decoder.  Every layer is  x <- x + mixer(norm1 x) + ff(norm2 x)  with the residual
 * x in fp32; the mixer and the feed-forward of each layer are chosen by its b200q_layer_desc. */
#define B200Q_ARCH_RAMOPEL 2
/* Noridra: a layered decoder in post-norm form.  Every layer is
 *   x <- norm1(alpha x + ls1 * mixer(x + conv1 x));  x <- norm2(alpha x + ls2 * ff(x + conv2 x))
 * with grouped RMS norms, per-channel layer scales ls and causal input convolutions whose last inputs are
 * carried in the sequence's state slot; mixers and feed-forwards again come from b200q_layer_desc. */
#define B200Q_ARCH_NORIDRA 3
/* Paluzen: a layered decoder in sequential pre-norm form.  Every layer is
 *   x <- x + a * mixer(shift(norm1 x)) (+ b * side_mixer(shift(norm1 x)));  x <- x + ff(norm2 x)
 * with plain RMS norms (x / rms * w), an optional token shift of the mixer's input (a per-channel blend with
 * the previous token's normed row, carried in the state slot), optional re-injection of the embedding output
 * before a layer (x <- W_in [x; x0]), a tied output matrix and soft-capped logits. */
#define B200Q_ARCH_PALUZEN 4

/* Kabavik: a layered decoder with a norm on BOTH sides of every sublayer and a residual multiplier m,
 *   x <- x + m * norm1b(mixer(norm1 x));  x <- x + m * norm2b(ff(norm2 x));
 *   x <- x + m * rms(P (gelu(G x) * e)) * s      (e = the layer's columns of a second embedding row of the token)
 * with dynamic-tanh norms (tanh(alpha x) * w + b: no statistics of the row), grouped-query attention with biases,
 * query / key norms, kept first keys behind the window, soft-capped scores, a query temperature that grows with the
 * logarithm of the position, keys and values shared with an earlier layer; latent attention with full-rank queries,
 * YaRN-scaled frequencies and a sigmoid gate per head; gated GELU feed-forwards; scaled logits. */
#define B200Q_ARCH_KABAVIK 5

#define B200Q_FORM_PARALLEL 0  /* x <- x + mixer(norm1 x) + ff(norm2 x)                                  */
#define B200Q_FORM_POSTNORM 1  /* x <- norm1(alpha x + ls1 mixer(x~)); x <- norm2(alpha x + ls2 ff(x~)) */
#define B200Q_FORM_PRENORM 2   /* x <- x + a mixer(h) (+ b side(h)), h = shift(norm1 x); x <- x + ff(norm2 x)     */
#define B200Q_FORM_SANDWICH 3  /* x <- x + m norm1b(mixer(norm1 x)); x <- x + m norm2b(ff(norm2 x)) (+ token input) */

#define B200Q_NORM_RMS 0       /* x / sqrt(mean(x^2) + eps) * w                                                    */
#define B200Q_NORM_DYT 1       /* tanh(alpha * x) * w + b  (weights as one fp32 row [w (W) | b (W) | alpha])       */
#define B200Q_NORM_CAST 2      /* op-level only: the row itself, in the model dtype                                */
#define B200Q_NORM_NONE 3      /* op-level only: nothing                                                           */

#define B200Q_DTYPE_BF16 0
#define B200Q_DTYPE_F32 1

#define B200Q_MIXER_LATENT_ATTN 1   /* low-rank (latent) queries and keys/values, sliding window, paged latent cache */
#define B200Q_MIXER_GENERAL_DELTA 2 /* generalized delta-rule recurrence, fp32 state per (sequence, head)            */
/* gated delta rule: per head a [dim x vdim] fp32 state, S <- g S + k (beta (v - S^T k))^T, o = S^T q; q, k
 * (kv_heads x dim) and v (heads x vdim) pass a short causal convolution + SiLU, q and k are unit vectors    */
#define B200Q_MIXER_GATED_DELTA 3
/* grouped-query attention over a paged cache of raw keys that also serve as values; per-head RMS norm of
 * queries and keys, soft-capped scores, a logarithmic distance penalty per head, visibility limited to the
 * query's own chunk of `chunk` positions, a softmax with a silent sink (denominator + 1), a sigmoid gate   */
#define B200Q_MIXER_CHUNK_ATTN 4
/* selective scan: per channel a [state_dim] fp32 state, S <- exp(dt A) S + dt x B, y = S.C + D x           */
#define B200Q_MIXER_SELECTIVE_SCAN 5
/* linear attention with a constant decay per head: q, k (heads x dim), v (heads x vdim) pass SiLU;
 * S <- decay_h S + k v^T, o = S^T q; the concatenated heads take one RMS norm and a sigmoid gate              */
#define B200Q_MIXER_LIGHTNING 6
/* rotary grouped-query attention over a sliding window: keys (rotated) and values in a paged cache, the first
 * rot_dims dimensions of every head turned in the half-split layout (i with i + rot_dims/2), a per-head score
 * temperature, ordinary softmax, one sigmoid gate number per head                                              */
#define B200Q_MIXER_WINDOW_ATTN 7
/* time mixing with a data-dependent decay per key channel: r, k, v, gate and decay each read their own blend of
 * the input with the previous token's input; w = exp(-exp(w0 + W2 tanh(W1 .))); o = (S + diag(u) k v^T)^T r,
 * S <- diag(w) S + k v^T; per-head RMS, a weight, a SiLU gate                                                  */
#define B200Q_MIXER_DECAY_MIX 8
#define B200Q_FF_NONE 0
#define B200Q_FF_POLYNORM 1         /* down(PolyNorm(up h))                                                          */
#define B200Q_FF_MOE 2              /* top-k of clamped gated experts + an optional gated shared expert              */
#define B200Q_FF_MOE_SIGMOID 3      /* top-k by sigmoid score, weights = the scores (not renormalised) applied to the
                                       expert's INPUT; expert = down(silu(gate h) * up h)                            */
#define B200Q_FF_RELU2 4            /* down(relu(up h)^2)                                                            */
/* top-k of relu^2 experts by softmax score over all experts: the choice adds a per-expert correction to the
 * score and is limited to the best `keep_groups` of `n_groups` equal groups of neighbouring experts (a group's
 * score = its largest choice score); weights = the chosen scores without correction, divided by their sum.  The
 * last `n_identity` router outputs are identity experts: they return their input.                               */
#define B200Q_FF_MOE_GROUPED 5
#define B200Q_FF_GEGLU 6            /* down(gelu_tanh(gate h) * up h); "mlp.gate_up" [2*ff, W] = gate rows, then up rows,
                                       or "mlp.gate_up_il" = the same rows interleaved in blocks of 128 (ff a multiple
                                       of 128), which a bf16 model runs with the unit in the product's epilogue */

typedef struct b200q_layer_desc {
  int32_t mixer;        /* B200Q_MIXER_*                                                               */
  int32_t heads;
  int32_t dim;          /* latent attention: unrotated q/k dims per head; delta: key = value dims       */
  int32_t rot_dim;      /* latent attention: rotated q/k dims per head (one key part shared by heads)   */
  int32_t vdim;         /* latent attention: value dims per head                                        */
  int32_t q_rank;       /* latent attention: rows of the query down-projection                          */
  int32_t kv_rank;      /* latent attention: size of the cached latent                                  */
  int32_t kv_from;      /* latent attention: layer whose cached latents are read; -1 = its own          */
  int32_t window;       /* keys seen: 0 <= i - j < window; 0 = all earlier keys                         */
  int32_t rot_dims;     /* leading dims of the rotated part that are rotated (pairs 2i, 2i+1)           */
  double rot_base;     /* pair i turns by position * rot_base^(-2i/rot_dims)                           */
  float attn_scale;
  int32_t decay_rank;   /* delta: inner size of the low-rank decay projection                           */
  int32_t ff;           /* B200Q_FF_*                                                                   */
  int32_t ff_dim;       /* dense: ff size; moe: ff size of one expert                                   */
  int32_t n_experts;
  int32_t top_k;
  float expert_limit;
  int32_t shared_dim;   /* moe: ff size of the shared expert, 0 = none                                  */
  float shared_limit;
  /* mixers 3-5 (zero elsewhere) */
  int32_t kv_heads;     /* gated delta / chunk attention: heads of q and k (delta) or of k (attention)    */
  int32_t conv_taps;    /* gated delta / selective scan: taps of the mixer's short convolution            */
  float softcap;        /* chunk attention: scores <- softcap * tanh(scores / softcap); 0 = off           */
  int32_t chunk;        /* chunk attention: i sees j <= i with floor(i/chunk) == floor(j/chunk); 0 = all  */
  int32_t inner;        /* selective scan: channels                                                       */
  int32_t state_dim;    /* selective scan: state size per channel                                         */
  int32_t dt_rank;      /* selective scan: rank of the step-size projection                               */
  /* pre-norm form and mixers 6-8 (zero elsewhere) */
  int32_t inject;       /* 1: before this layer x <- W_in [x; x0] ("inject" [W, 2W]; x0 = the embedding output) */
  float mix_scale;      /* the mixer's output is multiplied by this (0 = 1)                               */
  int32_t n_identity;   /* grouped mixture: identity experts behind the n_experts real ones               */
  int32_t n_groups;     /* grouped mixture: groups of neighbouring experts (identity ones included)       */
  int32_t keep_groups;  /* grouped mixture: groups a token may choose from                                */
  /* a second mixer beside the first, reading the same input (weights "side.*"); 0 = none */
  int32_t side_mixer;   /* B200Q_MIXER_LIGHTNING | B200Q_MIXER_DECAY_MIX                                  */
  int32_t side_heads;
  int32_t side_dim;
  int32_t side_vdim;
  int32_t side_decay_rank;
  float side_scale;
  /* options of window attention and latent attention (zero = off) */
  int32_t keep_first;   /* window attention: the first keep_first keys of a sequence stay visible behind the window  */
  int32_t qk_norm;      /* window attention: RMS norm of q and k before rotation, plain weights "mix.q_norm" /
                           "mix.k_norm": 1 = over the whole projection ([heads*dim], [kv_heads*dim]), 2 = per head
                           (one [dim] weight shared by the heads)                                                  */
  int32_t proj_bias;    /* window attention: 1 = q, k, v ("mix.proj_b" [rows of mix.proj]) and the output
                           projection ("mix.o_b" [W]) have biases                                                  */
  int32_t bare;         /* window attention: 1 = no temperature per head ("mix.temp") and no gate number per head
                           (mix.proj = [q | k | v] rows, padded to a multiple of 64)                               */
  int32_t head_gate;    /* latent attention: 1 = head h's output is multiplied by sigmoid of a gate number
                           (mix.down gains `heads` rows behind the latents)                                        */
  float q_temp_coef;    /* window attention: the query at position p is multiplied by                              */
  int32_t q_temp_every; /*   1 + q_temp_coef * ln(floor((p + 1) / q_temp_every) + 1); q_temp_every 0 = off         */
  /* rotation frequencies f_i = rot_base^(-2i/rot_dims), then: rot_factor > 0 and rot_original == 0: f_i / rot_factor;
   * rot_original > 0 (YaRN): with dim(t) = rot_dims ln(rot_original / (2 pi t)) / (2 ln rot_base), lo = max(floor(
   * dim(rot_fast)), 0), hi = min(ceil(dim(rot_slow)), rot_dims - 1), r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1):
   * f_i / rot_factor * r_i + f_i (1 - r_i), and sine and cosine are multiplied by 0.1 ln(rot_factor) + 1 */
  double rot_factor, rot_original, rot_fast, rot_slow;
} b200q_layer_desc;

typedef struct b200q_model* b200q_model_t;

/* device metadata for one step; every pointer is a device pointer to int32 data */
typedef struct b200q_batch {
  int32_t T;             /* total tokens this step; decode tokens occupy rows [0, n_dec)        */
  int32_t n_dec;         /* decode sequences (1 token each); block-table rows [0, n_dec)        */
  int32_t n_tiles;       /* prefill q-tiles                                                     */
  int32_t n_sample;      /* rows for which a next token is sampled                              */
  int32_t bt_stride;     /* int32 elements per block-table row                                  */
  const int32_t* token_ids;     /* [T]                                                          */
  const int32_t* positions;     /* [T]                                                          */
  const int32_t* slot_mapping;  /* [T]                                                          */
  const int32_t* block_table;   /* [rows][bt_stride]                                            */
  const int32_t* ctx_lens;      /* [n_dec] context length including the current token           */
  const int32_t* tiles;         /* [n_tiles][4]                                                 */
  const int32_t* sample_rows;   /* [n_sample] batch rows whose hidden state feeds the LM head   */
  int32_t* out_ids;             /* [n_sample] sampled token ids                                 */
  const int32_t* sample_params; /* [n_sample][4] {temperature bits, seed lo, seed hi, position};
                                   NULL = greedy argmax for every row                           */
  /* host-side bookkeeping for the profiler (algorithmic work of this step's attention) */
  int64_t sum_ctx_dec;          /* sum of ctx_lens over the decode sequences                    */
  int64_t prefill_flops_per_layer; /* causal QK^T + PV flops of the prefill tiles, one layer     */
  /* async stepping: token_ids[t] < 0 stands for prev_out_ids[-1 - token_ids[t]], a token the
   * previous step sampled and the host has not read back yet; NULL when no id is negative      */
  const int32_t* prev_out_ids;
  /* per-sequence view of the same step (used by the layered architectures): row r of the block table is
   * sequence r; seq_desc[r] = {first batch row, tokens this step, position of the first of them,
   * recurrent-state slot}; row_seq[t] = sequence of batch row t.  NULL for callers that only run
   * llama / gemma2 models. */
  int32_t n_rows;
  const int32_t* seq_desc;      /* [n_rows][4]                                                   */
  const int32_t* row_seq;       /* [T]                                                           */
  int32_t no_sampling;          /* 1: stop after the logits (sample_rows may then hold up to max_logit_rows rows) */
} b200q_batch;

int b200q_model_create(const b200q_model_config* cfg, b200q_model_t* out);
/* B200Q_ARCH_RAMOPEL: cfg gives hidden (width), n_layers, vocab, block_size, max_tokens, max_seqs, max_pos,
 * rms_eps, embed_scale, dtype; layers[n_layers] the mixer and feed-forward of every layer.
 * Weights (b200q_model_bind_weight; matrices in cfg.dtype, row-major [out, in]; every vector and the
 * PolyNorm constants in fp32 as one row):
 *   "embed" [V, W], "final_norm" [1, W], "lm_head" [V, W]; per layer i, prefix "layers.i.":
 *   "norm1", "norm2" [1, W]
 *   latent attention: "mix.down" [q_rank (+ kv_rank + rot_dim if kv_from < 0), W] (query rows first),
 *     "mix.q_norm" [1, q_rank], "mix.kv_norm" [1, kv_rank], "mix.uq" [heads*(dim+rot_dim), q_rank],
 *     "mix.uk_t" [heads*kv_rank, dim] (each head's key up-projection TRANSPOSED: the query is carried into
 *     the latent space, so scores are taken against the cached latent directly),
 *     "mix.uv" [heads*vdim, kv_rank], "mix.o" [W, heads*vdim]
 *   general delta: "mix.proj" [5*heads*dim + decay_rank, W] (rows: r, k, v, g, a, w1), "mix.w2"
 *     [heads*dim, decay_rank], "mix.w0", "mix.a_bias", "mix.out_norm" [1, heads*dim], "mix.o" [W, heads*dim]
 *   PolyNorm ff: "mlp.up" [ff, W], "mlp.act" [1, 4], "mlp.down" [W, ff]
 *   MoE ff: "mlp.router" [E, W], "mlp.router_bias" [1, E], "mlp.experts_gate_up" [E*2*ff, W] (per expert:
 *     gate rows then up rows), "mlp.experts_down" [E*W, ff], and with a shared expert
 *     "mlp.shared_gate_up" [2*ffs, W], "mlp.shared_down" [W, ffs], "mlp.shared_gate" [1, W]
 * B200Q_ARCH_NORIDRA (cfg.layer_form = B200Q_FORM_POSTNORM, with norm_groups, residual_alpha, input_taps,
 * learned_pos): "pos" [>= max_pos, W] beside "embed"; per layer "norm1", "ls1" [1, W] (and "norm2", "ls2" with a
 * feed-forward), "canon1" / "canon2" [1, W*input_taps] (fp32 tap table [W][taps], last tap = current token), and
 *   gated delta: "mix.proj" [2*kv_heads*dim + 2*heads*vdim, W] (rows: q, k, v, gate), "mix.ba" [2*heads, W] (rows:
 *     beta, decay input), "mix.conv" [1, (2*kv_heads*dim + heads*vdim)*conv_taps] (taps of the channels q | k | v),
 *     "mix.a_log", "mix.dt_bias" [1, heads], "mix.out_norm" [1, vdim], "mix.o" [W, heads*vdim]
 *   chunk attention: "mix.proj" [(2*heads + kv_heads)*dim, W] (rows: q, k, gate), "mix.q_norm", "mix.k_norm"
 *     [1, dim], "mix.r1", "mix.r2" [1, heads], "mix.o" [W, heads*dim]
 *   selective scan: "mix.proj" [2*inner, W] (rows: x, z), "mix.conv" [1, inner*conv_taps], "mix.conv_b" [1, inner],
 *     "mix.x" [roundup64(dt_rank + 2*state_dim), inner] (rows: dt, B, C, then zero rows), "mix.dt" [inner, dt_rank],
 *     "mix.dt_b" [1, inner], "mix.a_log" [1, inner*state_dim], "mix.d" [1, inner], "mix.o" [W, inner]
 *   sigmoid-routed experts: "mlp.router" [E, W], "mlp.experts_gate_up" [E*2*ff, W], "mlp.experts_down" [E*W, ff] */
int b200q_model_create_layered(const b200q_model_config* cfg, const b200q_layer_desc* layers,
                               b200q_model_t* out);
/* layered models: bytes of one cache block over all layers that own a latent cache (the caller allocates
 * num_blocks times this, zeroed, and binds it with b200q_model_bind_kv), and bytes of one recurrent-state
 * slot over all recurrent layers (fp32; bound with b200q_model_bind_state) */
int64_t b200q_model_kv_block_bytes(b200q_model_t m);
int64_t b200q_model_state_slot_bytes(b200q_model_t m);
int b200q_model_bind_state(b200q_model_t m, void* dev_ptr, int64_t n_slots);
/* layered models: fp32 logits of the last forward, [n_sample, V] */
const float* b200q_model_logits_f32_ptr(b200q_model_t m);
/* layered models: copy the fp32 residual stream after every layer of the NEXT forwards into dev_ptr
 * ([n_layers][T][W], the caller sizes it for the steps it runs); NULL switches it off */
int b200q_model_set_layer_tap(b200q_model_t m, float* dev_ptr);
int b200q_model_destroy(b200q_model_t m);
/* names: "embed", "final_norm", "lm_head", and per layer i: "layers.i.input_norm",
 * "layers.i.qkv" [(n_q+2n_kv)D, H], "layers.i.o" [H, n_q D], "layers.i.post_norm",
 * "layers.i.gate_up" [2I, H] (gate/up rows interleaved in 128-row blocks, see
 * b200q_gemm_swiglu_bf16), "layers.i.down" [H, I].  bf16, row-major, contiguous.
 * B200Q_ARCH_GEMMA2 replaces "post_norm" by the three norms "layers.i.post_attn_norm",
 * "layers.i.pre_ffn_norm", "layers.i.post_ffn_norm" (weights as stored: the kernels add the 1). */
int b200q_model_bind_weight(b200q_model_t m, const char* name, const void* dev_ptr,
                            int64_t rows, int64_t cols);
/* kv: [L][num_blocks][2][n_kv][block_size][D] bf16, zero-initialised by the caller */
int b200q_model_bind_kv(b200q_model_t m, void* dev_ptr, int64_t num_blocks);
/* cos_sin: bf16 [max_pos][D] */
int b200q_model_bind_rope(b200q_model_t m, const void* dev_ptr);
/* bytes needed for activations at cfg.max_tokens; caller allocates and binds */
int64_t b200q_model_workspace_bytes(const b200q_model_config* cfg);
/* the same for a created model of any architecture (a layered model's need depends on its layers) */
int64_t b200q_model_workspace_bytes_of(b200q_model_t m);
int b200q_model_bind_workspace(b200q_model_t m, void* dev_ptr, int64_t bytes);
int b200q_model_forward(b200q_model_t m, const b200q_batch* batch, void* stream);
/* debugging / parity: copy the bf16 logits of the last forward ([n_sample, V]) location */
const void* b200q_model_logits_ptr(b200q_model_t m);
/* per-category device timing: CUDA events recorded on the forward's stream around every launch
 * (bench.py's live roofline numbers).  work = algorithmic flops (GEMM, prefill attention) or
 * bytes (decode attention, elementwise) summed over the timed launches. */
#define B200Q_PROF_GEMM 0
#define B200Q_PROF_DECODE_ATTN 1
#define B200Q_PROF_PREFILL_ATTN 2
#define B200Q_PROF_ELEMENTWISE 3
typedef struct b200q_profile {
  double ms[4];
  double work[4];
  int64_t launches[4];
} b200q_profile;
int b200q_model_set_profiling(b200q_model_t m, int on);
int b200q_model_profile_collect(b200q_model_t m, b200q_profile* out, int reset);
/* number of kernels launched by this library since load (gpu_launches evidence) */
int64_t b200q_launch_count(void);

/* ------------------------------------------------------------------------------------
 * Engine-level: continuous-batching scheduler + paged-KV block manager + step loop.
 * Replaces AsyncLLMEngine.generate / EngineCore.step for the reference worker
 * (ref:llmq/workers/vllm_worker.py:183-186; vllm/v1/core/sched/scheduler.py:329-340
 * behaviour: running requests first, then waiting/prefill under a token budget, chunked
 * prefill, preempt-by-recompute when the KV pool is exhausted).
 * ---------------------------------------------------------------------------------- */

typedef struct b200q_engine_config {
  int32_t max_num_seqs;            /* VLLM_MAX_NUM_SEQS  (ref:llmq/core/config.py:27-32)  */
  int32_t max_num_batched_tokens;  /* token budget per step (<= model max_tokens)          */
  int32_t max_model_len;           /* VLLM_MAX_MODEL_LEN (ref:llmq/core/config.py:34-39)  */
  int32_t eos_token_id;            /* -1: none                                            */
  int32_t policy;                  /* 0: running requests first (vLLM order); 1: prefill first */
} b200q_engine_config;

typedef struct b200q_engine* b200q_engine_t;

#define B200Q_FLAG_FINISHED_EOS 1
#define B200Q_FLAG_FINISHED_LENGTH 2
#define B200Q_FLAG_FINISHED_ABORT 4

typedef struct b200q_engine_stats {
  int64_t steps;
  int64_t tokens_prefilled;
  int64_t tokens_decoded;
  int64_t preemptions;
  int32_t running;
  int32_t waiting;
  int32_t free_blocks;
  int32_t total_blocks;
  int32_t last_step_tokens;
  int32_t last_step_seqs;
  int64_t h2d_bytes;   /* per-step metadata copies (token ids, block tables, ...) */
  int64_t d2h_bytes;   /* sampled token ids read back                              */
} b200q_engine_stats;

int b200q_engine_create(b200q_model_t model, const b200q_engine_config* cfg, b200q_engine_t* out);
/* Scheduler self-test engine (host-logic tests on machines without a GPU): no model, no CUDA.
 * step() builds the per-step metadata exactly as in production, checks its invariants (budget,
 * unique KV slots, tile cover, positions) and fabricates each "sampled" token as
 * (previous token + 1) mod vocab.  It cannot run a model and is never used by the worker. */
int b200q_engine_create_dryrun(const b200q_engine_config* cfg, int32_t vocab, int32_t block_size,
                               int32_t num_blocks, b200q_engine_t* out);
int b200q_engine_destroy(b200q_engine_t e);
/* prompt ids are copied.  Returns B200Q_EINVAL if n_prompt + 1 > max_model_len (the worker
 * turns that into ValueError => job dropped, ref:llmq/workers/base.py:228-235). */
int b200q_engine_add_request(b200q_engine_t e, int64_t req_id, const int32_t* prompt_ids,
                             int32_t n_prompt, int32_t max_new_tokens, int32_t ignore_eos);
/* same, with the sampling the reference worker uses: temperature (0 = greedy) and a per-request
 * seed; token t of the request is drawn with Philox counter position t, so the result does not
 * depend on batching, chunking or preemption. */
int b200q_engine_add_request_sampled(b200q_engine_t e, int64_t req_id, const int32_t* prompt_ids,
                                     int32_t n_prompt, int32_t max_new_tokens, int32_t ignore_eos,
                                     float temperature, uint64_t seed);
/* every id in ids[0..n) ends a request (replaces the single cfg.eos_token_id): vLLM stops on
 * tokenizer.eos_token_id plus all eos ids of generation_config.json (vllm/sampling_params.py
 * update_from_generation_config), which the reference worker inherits (vllm_worker.py:161-165). */
int b200q_engine_set_stop_ids(b200q_engine_t e, const int32_t* ids, int32_t n);
int b200q_engine_abort(b200q_engine_t e, int64_t req_id);
/* Async stepping (default on; env B200Q_ASYNC=0 or on=0 turns it off): b200q_engine_step enqueues
 * step k+1 BEFORE it reads step k's sampled ids back, so the events a call returns are those of
 * the step enqueued by the PREVIOUS call, and b200q_engine_has_work stays 1 while a step is in
 * flight.  Off: every call returns the events of the step it ran (one sync per step).  Token
 * sequences are identical in both modes.  Only while no step is in flight (B200Q_ESTATE else). */
int b200q_engine_set_async(b200q_engine_t e, int32_t on);
/* 1 if any request is waiting or running */
int b200q_engine_has_work(b200q_engine_t e);
/* run one scheduler step + forward; writes up to cap (req_id, token, flags) events — those of this
 * step (sync mode) or of the previously enqueued step (async mode, see b200q_engine_set_async).
 * cap must be >= max_num_seqs. */
int b200q_engine_step(b200q_engine_t e, int64_t* out_req_ids, int32_t* out_tokens,
                      int32_t* out_flags, int32_t cap, int32_t* n_out);
/* Replay (teacher forcing): one step whose work the CALLER lays down instead of the scheduler — entry i
 * appends n_tokens[i] given tokens to request req_ids[i] (admitted on its first entry: pages and a state
 * slot are taken from the same pools the scheduler uses) and runs them through the same metadata
 * builder, forward and kernels as a scheduled step, all entries as one batch.  want[] lists, per entry,
 * the entry-relative token places whose logits are wanted; they are written, fp32, to logits_out
 * [sum n_want][vocab] (host memory) in the order of the entries.  Nothing is sampled.  A request stays
 * live (and may sit a step out) until b200q_engine_abort gives its pages and slot back.  Not to be mixed
 * with b200q_engine_step on the same engine while requests are live.  B200Q_ENOMEM: the pool cannot hold
 * the step. */
int b200q_engine_step_replay(b200q_engine_t e, int32_t n_entries, const int64_t* req_ids,
                             const int32_t* n_tokens, const int32_t* tokens, const int32_t* n_want,
                             const int32_t* want, float* logits_out);
int b200q_engine_get_stats(b200q_engine_t e, b200q_engine_stats* out);
/* the engine's CUDA stream (cudaStream_t) so callers can record their own events on it */
void* b200q_engine_stream(b200q_engine_t e);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
