// model_types.cuh — the model object behind b200q_model_t, shared by model.cu (llama / gemma2 forward)
// and layered.cu (layered architectures).
#pragma once
#include <string>
#include <vector>

#include "common.cuh"

using b200q::bf16;

// one layer of a layered architecture: its description, bound weights and where its cache / state live
struct b200q_layered_layer {
  b200q_layer_desc d{};
  const float *norm1 = nullptr, *norm2 = nullptr;
  // latent attention
  const void *down = nullptr, *uq = nullptr, *uk_t = nullptr, *uv = nullptr;
  const float *q_norm = nullptr, *kv_norm = nullptr;
  // general delta
  const void *proj = nullptr, *w2 = nullptr;
  const float *w0 = nullptr, *a_bias = nullptr, *out_norm = nullptr;
  const void* o = nullptr;  // output projection of either mixer
  // feed-forward
  const void *up = nullptr, *ff_down = nullptr;
  const float* act = nullptr;
  const void* router = nullptr;
  const float* router_bias = nullptr;
  const void *experts_gate_up = nullptr, *experts_down = nullptr, *shared_gate_up = nullptr,
             *shared_down = nullptr, *shared_gate = nullptr;
  // post-norm form: layer scales and input convolutions of the two sublayers
  const float *ls1 = nullptr, *ls2 = nullptr, *canon1 = nullptr, *canon2 = nullptr;
  // gated delta (proj = [q | k | v | gate] rows), chunk attention (proj = [q | k | gate] rows; q_norm / kv_norm
  // are the per-head norms of queries and keys), selective scan (proj = [x | z] rows)
  const void* ba = nullptr;  // gated delta: [beta | decay input] rows
  const float *conv_w = nullptr, *conv_b = nullptr, *a_log = nullptr, *dt_bias = nullptr, *r1 = nullptr, *r2 = nullptr;
  const void *x_proj = nullptr, *dt_proj = nullptr;
  const float *dt_b = nullptr, *dvec = nullptr;
  // pre-norm form: token-shift weights and the re-injection matrix; lightning (proj = [q | k | v | gate] rows,
  // head_decay), window attention (proj = [q | k | v | gate number per head] rows, temp), decay mix (mu: five
  // blend weights; proj = [r | k | v | gate] rows, each product reading its own blend; w1, w2, w0: the decay's
  // low-rank path; bonus)
  const float *shift = nullptr, *head_decay = nullptr, *temp = nullptr, *mu = nullptr, *bonus = nullptr;
  const void *inject = nullptr, *w1 = nullptr, *experts_up = nullptr;
  // sandwich form: the norms behind the two sublayers (dynamic tanh rows [w | b | alpha], like norm1 / norm2 there),
  // the gated GELU feed-forward (gate_up = [gate | up] rows), the per-layer token input; biases of window attention
  const float *norm1b = nullptr, *norm2b = nullptr, *proj_b = nullptr, *o_b = nullptr, *tok_norm = nullptr;
  const void *gate_up = nullptr, *tok_gate = nullptr, *tok_proj = nullptr;
  float mag = 1.f;  // factor of sine and cosine (YaRN)
  bool gate_up_il = false;  // gate_up rows interleaved in blocks of 128 (the fused product + gated unit's layout)
  std::vector<b200q_layered_layer> side;  // the mixer beside the first one (none or one)
  int64_t shift_off = 0, prev_off = 0;    // floats into a state slot: carried normed row, carried mixer input
  int64_t cache_block_off = 0;  // bytes per block of the cache regions before this layer's (own cache only)
  int64_t state_off = 0;        // floats into a state slot: the recurrent state
  int64_t conv_off = 0, canon1_off = 0, canon2_off = 0;  // ... the carried inputs of the convolutions
  double* freq = nullptr;       // device, [rot_dims/2]
};

struct b200q_layered {
  std::vector<b200q_layered_layer> layers;
  int64_t kv_block_bytes = 0;
  int64_t state_slot_floats = 0;
  float* state = nullptr;
  int64_t n_slots = 0;
  float* tap = nullptr;
  const void* pos = nullptr;  // learned position table [pos_rows, W]
  int64_t pos_rows = 0;
  float *cvf = nullptr, *baf = nullptr, *dtr = nullptr;  // fp32: convolved q|k|v (+ raw outputs), beta|g, step sizes
  void *xc = nullptr, *xp = nullptr;                     // selective scan: convolved x, [dt | B | C] rows
  // workspace views (element type = cfg.dtype unless float)
  float *dscr = nullptr;  // delta rule: per-token vectors and raw outputs of a step (fp32)
  float *x = nullptr, *qa = nullptr, *rlog = nullptr, *wts = nullptr, *sgate = nullptr, *logits = nullptr;
  void *h1 = nullptr, *h2 = nullptr, *mix = nullptr, *ffo = nullptr, *proj = nullptr, *cq = nullptr, *q = nullptr,
       *olat = nullptr, *attn = nullptr, *ffh = nullptr, *ffa = nullptr, *egu = nullptr, *eact = nullptr,
       *eout = nullptr, *shout = nullptr, *sel = nullptr, *logits_bf16 = nullptr;
  int32_t *idx = nullptr, *group_off = nullptr, *perm_tok = nullptr, *pair_pos = nullptr, *tile_tab = nullptr,
          *n_tiles = nullptr;
  void* esrc = nullptr;  // the routed pairs' inputs gathered into expert order (bf16 path)
  // pre-norm form: fp32 mixer input, embedding output, carried rows of a step, side mixer's output, [x | x0], blends
  float *hf = nullptr, *x0 = nullptr, *carry = nullptr;
  void *mix2 = nullptr, *cat = nullptr, *blend = nullptr;
  // sandwich form: the second embedding table [V, n_layers * side_dim] and the token input's two small activations
  const void* tok_embed = nullptr;
  int64_t tok_cols = 0;
  void *tg = nullptr, *ta = nullptr;
};

struct b200q_layer {
  const void* input_norm = nullptr;
  const void* qkv = nullptr;
  const void* o = nullptr;
  const void* post_norm = nullptr;  // llama: post_attention_layernorm (= the pre-MLP norm)
  const void* gate_up = nullptr;
  const void* down = nullptr;
  // gemma2: the sandwich norms
  const void* post_attn_norm = nullptr;
  const void* pre_ffn_norm = nullptr;
  const void* post_ffn_norm = nullptr;
};

struct b200q_model {
  b200q_model_config cfg;
  const void* embed = nullptr;
  const void* final_norm = nullptr;
  const void* lm_head = nullptr;
  std::vector<b200q_layer> layers;
  uint8_t* kv = nullptr;
  int64_t num_blocks = 0;
  const void* rope = nullptr;
  // workspace views
  uint8_t* ws = nullptr;
  int64_t ws_bytes = 0;
  // (no [T, 2I] gate_up buffer: the SwiGLU is applied in the gate_up GEMM's epilogue)
  bf16 *x = nullptr, *residual = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr,
       *sel = nullptr, *logits = nullptr;
  // fold the split-K reduce of decode-sized projections into the consuming kernel (B200Q_FUSE_SPLITK=0: off)
  bool fuse_splitk = true;
  b200q_layered* lay = nullptr;  // B200Q_ARCH_RAMOPEL: everything layer-specific lives here
  // optional per-category device timing (CUDA events on the forward's stream)
  bool profiling = false;
  std::vector<cudaEvent_t> ev_pool;
  struct Span { int cat; double work; int e0, e1; };
  std::vector<Span> spans;
  int ev_used = 0;
  b200q_profile prof{};
  int get_event() {
    if (ev_used == (int)ev_pool.size()) {
      cudaEvent_t e;
      cudaEventCreate(&e);
      ev_pool.push_back(e);
    }
    return ev_used++;
  }
};

