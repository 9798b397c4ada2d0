// layered.cu — model-level code of the layered architectures (B200Q_ARCH_RAMOPEL): creation from a list
// of b200q_layer_desc, weight binding by name, cache / state / workspace layout, and one forward step over
// a mixed batch (single decoded tokens beside portions of prompts), composed from the kernels of
// layered_ops.cu.  The step's metadata is the engine's own (b200q_batch): block table, slot mapping,
// positions, per-sequence descriptors.
//
// Layout.  Latent cache: one region per layer that owns latents, [num_blocks][block_size][kv_rank +
// rot_dim] in the model's dtype — a layer with kv_from reads the region of the layer it names.  Recurrent
// state: fp32 [slots][sum over delta layers of heads*dim*dim]; a slot belongs to one live sequence.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include "model_types.cuh"

using namespace b200q;

namespace {

int64_t al256(int64_t v) { return (v + 255) & ~(int64_t)255; }
int esize(const b200q_model_config& c) { return c.dtype == B200Q_DTYPE_F32 ? 4 : 2; }
int logit_rows(const b200q_model_config& c) { return std::max(c.max_logit_rows, c.max_seqs); }

// the description of the mixer that stands beside a layer's first one, as a description of its own
b200q_layer_desc side_desc(const b200q_layer_desc& d) {
  b200q_layer_desc s{};
  s.mixer = d.side_mixer;
  s.heads = d.side_heads;
  s.kv_heads = d.side_heads;
  s.dim = d.side_dim;
  s.vdim = d.side_vdim;
  s.decay_rank = d.side_decay_rank;
  s.mix_scale = d.side_scale;
  s.kv_from = -1;
  return s;
}

int check_sequence_mixer(int i, const b200q_layer_desc& d) {
  if (d.mixer == B200Q_MIXER_LIGHTNING) {
    B200Q_CHECK_ARG(d.heads > 0 && d.dim > 0 && d.dim <= 256 && d.vdim > 0, "layer %d: bad lightning sizes (dim <= 256)", i);
  } else if (d.mixer == B200Q_MIXER_DECAY_MIX) {
    B200Q_CHECK_ARG(d.heads > 0 && d.dim > 0 && d.dim <= 256 && d.vdim == d.dim && d.decay_rank > 0,
                    "layer %d: bad decay-mix sizes (dim <= 256, values as wide as keys)", i);
  } else {
    B200Q_CHECK_ARG(d.heads > 0 && d.kv_heads > 0 && d.heads % d.kv_heads == 0 && d.dim > 0 && d.dim <= 512 &&
                        d.vdim > 0 && d.vdim <= 512 && d.window >= 0 && d.rot_dims >= 0 && d.rot_dims % 2 == 0 &&
                        d.rot_dims <= d.dim && (d.rot_dims == 0 || d.rot_base > 0.0),
                    "layer %d: bad window-attention sizes (dim, vdim <= 512, even rot.dims <= dim, kv_heads divides heads)",
                    i);
    B200Q_CHECK_ARG(d.keep_first >= 0 && d.qk_norm >= 0 && d.qk_norm <= 2 && d.softcap >= 0.f && d.q_temp_every >= 0 &&
                        d.rot_factor >= 0.0 && d.rot_original >= 0.0 &&
                        (d.bare || (d.proj_bias == 0 && d.qk_norm == 0 && d.q_temp_every == 0 && d.kv_from < 0)),
                    "layer %d: bad window-attention options (biases, query / key norms, a query temperature by "
                    "position and borrowed keys go with the bare projection layout)", i);
  }
  return B200Q_OK;
}

int check_layered(const b200q_model_config* c, const b200q_layer_desc* L) {
  B200Q_CHECK_ARG(c && L, "layered config is null");
  B200Q_CHECK_ARG(c->arch == B200Q_ARCH_RAMOPEL || c->arch == B200Q_ARCH_NORIDRA || c->arch == B200Q_ARCH_PALUZEN ||
                      c->arch == B200Q_ARCH_KABAVIK,
                  "create_layered: arch=%d is not a layered architecture", c->arch);
  B200Q_CHECK_ARG(c->layer_form == B200Q_FORM_PARALLEL || c->layer_form == B200Q_FORM_POSTNORM ||
                      c->layer_form == B200Q_FORM_PRENORM || c->layer_form == B200Q_FORM_SANDWICH,
                  "layer_form=%d unknown", c->layer_form);
  const bool sandwich = c->layer_form == B200Q_FORM_SANDWICH;
  B200Q_CHECK_ARG(sandwich ? ((c->norm_kind == B200Q_NORM_RMS || c->norm_kind == B200Q_NORM_DYT) && c->side_dim >= 0 &&
                              c->residual_mult >= 0.f && c->learned_pos == 0)
                           : (c->norm_kind == 0 && c->side_dim == 0 && c->residual_mult == 0.f),
                  "norm kind (%d), residual multiplier and per-layer token input belong to the sandwich form",
                  c->norm_kind);
  B200Q_CHECK_ARG(c->logit_softcap >= 0.f && (c->token_shift == 0 || c->layer_form == B200Q_FORM_PRENORM),
                  "bad logit soft cap, or a token shift outside the pre-norm form");
  B200Q_CHECK_ARG(c->norm_groups >= 0 && (c->norm_groups <= 1 || c->hidden % c->norm_groups == 0) &&
                      c->input_taps >= 0 && c->input_taps <= 16,
                  "bad norm groups (%d must divide the width %d) or input taps (%d, at most 16)", c->norm_groups,
                  c->hidden, c->input_taps);
  B200Q_CHECK_ARG(c->dtype == B200Q_DTYPE_BF16 || c->dtype == B200Q_DTYPE_F32, "dtype=%d unknown", c->dtype);
  B200Q_CHECK_ARG(c->hidden > 0 && c->vocab > 0 && c->n_layers > 0 && c->max_tokens > 0 && c->max_seqs > 0 &&
                      c->max_pos > 0 && c->block_size > 0 && c->rms_eps > 0.f,
                  "bad sizes width=%d vocab=%d L=%d max_tokens=%d max_seqs=%d max_pos=%d block=%d", c->hidden,
                  c->vocab, c->n_layers, c->max_tokens, c->max_seqs, c->max_pos, c->block_size);
  for (int i = 0; i < c->n_layers; ++i) {
    const b200q_layer_desc& d = L[i];
    if (d.mixer == B200Q_MIXER_LATENT_ATTN) {
      B200Q_CHECK_ARG(d.heads > 0 && d.dim >= 0 && d.rot_dim >= 0 && d.dim + d.rot_dim > 0 && d.vdim > 0 &&
                          d.q_rank >= 0 && d.kv_rank > 0 && d.kv_rank <= 1024 && d.window >= 0 && d.rot_dims >= 0 &&
                          d.rot_dims % 2 == 0 && d.rot_dims <= d.rot_dim && d.rot_factor >= 0.0 && d.rot_original >= 0.0,
                      "layer %d: bad latent attention sizes (kv_rank <= 1024, even rot.dims <= rot_dim)", i);
      // full-rank queries (q_rank 0) and the gate number per head come as one fused projection of the layer's input
      B200Q_CHECK_ARG((d.q_rank == 0) == (d.head_gate != 0) && (d.q_rank > 0 || d.kv_from < 0),
                      "layer %d: full-rank queries (q_rank 0) come with a gate per head and latents of their own", i);
      if (d.kv_from >= 0) {
        B200Q_CHECK_ARG(d.kv_from < i && L[d.kv_from].mixer == B200Q_MIXER_LATENT_ATTN && L[d.kv_from].kv_from < 0 &&
                            L[d.kv_from].kv_rank == d.kv_rank && L[d.kv_from].rot_dim == d.rot_dim,
                        "layer %d: kv_from=%d must name an earlier latent-attention layer with its own latents "
                        "of the same sizes", i, d.kv_from);
      }
    } else if (d.mixer == B200Q_MIXER_GENERAL_DELTA) {
      B200Q_CHECK_ARG(d.heads > 0 && d.dim > 0 && d.dim <= 1024 && d.decay_rank > 0,
                      "layer %d: bad delta-rule sizes", i);
    } else if (d.mixer == B200Q_MIXER_GATED_DELTA) {
      B200Q_CHECK_ARG(d.heads > 0 && d.kv_heads > 0 && d.heads % d.kv_heads == 0 && d.dim > 0 && d.dim <= 256 &&
                          d.vdim > 0 && d.vdim <= 1024 && d.conv_taps >= 1 && d.conv_taps <= 16,
                      "layer %d: bad gated-delta sizes (dim <= 256, vdim <= 1024, taps <= 16, kv_heads divides heads)", i);
    } else if (d.mixer == B200Q_MIXER_CHUNK_ATTN) {
      B200Q_CHECK_ARG(d.heads > 0 && d.kv_heads > 0 && d.heads % d.kv_heads == 0 && d.dim > 0 && d.dim <= 512 &&
                          d.vdim == d.dim && d.chunk >= 0 && d.softcap >= 0.f,
                      "layer %d: bad chunk-attention sizes (dim <= 512; the values are the keys, so vdim == dim)", i);
    } else if (d.mixer == B200Q_MIXER_SELECTIVE_SCAN) {
      B200Q_CHECK_ARG(d.inner > 0 && d.state_dim > 0 && d.state_dim <= 256 && d.dt_rank > 0 && d.conv_taps >= 1 &&
                          d.conv_taps <= 16,
                      "layer %d: bad selective-scan sizes (state <= 256, taps <= 16)", i);
    } else if (d.mixer == B200Q_MIXER_LIGHTNING || d.mixer == B200Q_MIXER_DECAY_MIX ||
               d.mixer == B200Q_MIXER_WINDOW_ATTN) {
      if (int rc = check_sequence_mixer(i, d)) return rc;
      if (d.mixer == B200Q_MIXER_WINDOW_ATTN && d.kv_from >= 0) {
        const b200q_layer_desc& o = L[d.kv_from < i ? d.kv_from : 0];
        B200Q_CHECK_ARG(d.kv_from < i && o.mixer == B200Q_MIXER_WINDOW_ATTN && o.kv_from < 0 && o.kv_heads == d.kv_heads &&
                            o.dim == d.dim && o.vdim == d.vdim,
                        "layer %d: kv_from=%d must name an earlier window-attention layer with keys and values of its "
                        "own and the same sizes", i, d.kv_from);
      }
    } else {
      set_error("layer %d: unknown mixer %d", i, d.mixer);
      return B200Q_EINVAL;
    }
    if (d.side_mixer != 0) {
      B200Q_CHECK_ARG(d.side_mixer == B200Q_MIXER_LIGHTNING || d.side_mixer == B200Q_MIXER_DECAY_MIX,
                      "layer %d: side mixer %d is not one that can stand beside another", i, d.side_mixer);
      if (int rc = check_sequence_mixer(i, side_desc(d))) return rc;
    }
    B200Q_CHECK_ARG((d.inject == 0 && d.side_mixer == 0 && d.mix_scale == 0.f) || c->layer_form == B200Q_FORM_PRENORM,
                    "layer %d: re-injection, side mixers and mixer scales belong to the pre-norm form", i);
    B200Q_CHECK_ARG(!sandwich || d.ff == B200Q_FF_GEGLU || d.ff == B200Q_FF_NONE,
                    "layer %d: feed-forward %d is not built for the sandwich form", i, d.ff);
    B200Q_CHECK_ARG(!sandwich || d.mixer == B200Q_MIXER_LATENT_ATTN || d.mixer == B200Q_MIXER_WINDOW_ATTN,
                    "layer %d: mixer %d is not built for the sandwich form", i, d.mixer);
    if (d.ff == B200Q_FF_GEGLU) {
      B200Q_CHECK_ARG(d.ff_dim > 0 && sandwich, "layer %d: bad gated-GELU feed-forward", i);
    } else if (d.ff == B200Q_FF_RELU2) {
      B200Q_CHECK_ARG(d.ff_dim > 0 && c->layer_form == B200Q_FORM_PRENORM, "layer %d: bad squared-ReLU feed-forward", i);
    } else if (d.ff == B200Q_FF_MOE_GROUPED) {
      const int E = d.n_experts + d.n_identity;
      B200Q_CHECK_ARG(d.ff_dim > 0 && d.n_experts >= 0 && d.n_identity >= 0 && E > 0 && E <= 4096 && d.top_k > 0 &&
                          d.top_k <= 32 && d.n_groups > 0 && d.n_groups <= 256 && E % d.n_groups == 0 &&
                          d.keep_groups > 0 && d.keep_groups <= d.n_groups &&
                          d.top_k <= d.keep_groups * (E / d.n_groups) && c->layer_form == B200Q_FORM_PRENORM,
                      "layer %d: bad grouped mixture (experts + identity <= 4096, top <= 32, at most 256 groups that "
                      "divide the experts, top fits the kept groups)", i);
    } else if (d.ff == B200Q_FF_MOE_SIGMOID) {
      B200Q_CHECK_ARG(d.ff_dim > 0 && d.n_experts > 0 && d.n_experts <= 4096 && d.top_k > 0 && d.top_k <= 32 &&
                          d.top_k <= d.n_experts,
                      "layer %d: bad mixture sizes (experts <= 4096, top <= 32)", i);
      B200Q_CHECK_ARG(c->layer_form == B200Q_FORM_POSTNORM, "layer %d: this mixture belongs to the post-norm form", i);
    } else if (d.ff == B200Q_FF_POLYNORM) {
      B200Q_CHECK_ARG(d.ff_dim > 0, "layer %d: bad ff size", i);
    } else if (d.ff == B200Q_FF_MOE) {
      B200Q_CHECK_ARG(d.ff_dim > 0 && d.n_experts > 0 && d.n_experts <= 4096 && d.top_k > 0 && d.top_k <= 32 &&
                          d.top_k <= d.n_experts && d.shared_dim >= 0,
                      "layer %d: bad mixture sizes (experts <= 4096, top <= 32)", i);
    } else {
      B200Q_CHECK_ARG(d.ff == B200Q_FF_NONE, "layer %d: unknown feed-forward %d", i, d.ff);
    }
  }
  return B200Q_OK;
}

// widest use of every workspace buffer over the layers
struct Widths {
  int64_t proj = 1, cq = 1, q = 1, qa = 1, olat = 1, attn = 1, ffh = 1, ffa = 1, experts = 1, pairs = 1, egu = 1,
          eact = 1, delta = 0, cvf = 0, baf = 0, dtr = 0, xc = 0, xp = 0, blend = 0;
  bool moe = false, shared = false, hf = false, side = false, inject = false;
};
int64_t pad64(int64_t v) { return (v + 63) & ~(int64_t)63; }
// rows of window attention's fused projection: [q | k | v (own keys and values) | gate number per head (not bare)],
// with zero rows up to a multiple of 64
int64_t window_proj_rows(const b200q_layer_desc& d) {
  return pad64((int64_t)d.heads * d.dim + (d.kv_from < 0 ? (int64_t)d.kv_heads * (d.dim + d.vdim) : 0) +
               (d.bare ? 0 : d.heads));
}
// rows of latent attention's fused projection with full-rank queries: [q | latent | shared rotated key | gate number
// per head], with zero rows up to a multiple of 64
int64_t latent_full_rows(const b200q_layer_desc& d) {
  return pad64((int64_t)d.heads * (d.dim + d.rot_dim) + d.kv_rank + d.rot_dim + d.heads);
}
void sequence_mixer_widths(const b200q_layer_desc& d, int64_t W, Widths& w) {
  const int64_t HD = (int64_t)d.heads * d.dim, HV = (int64_t)d.heads * d.vdim;
  if (d.mixer == B200Q_MIXER_LIGHTNING) {
    w.proj = std::max<int64_t>(w.proj, 2 * HD + 2 * HV);
    w.cvf = std::max<int64_t>(w.cvf, 2 * HD + 2 * HV);  // q | k | v in fp32 and, behind them, the raw outputs
    w.attn = std::max<int64_t>(w.attn, HV);
  } else if (d.mixer == B200Q_MIXER_DECAY_MIX) {
    w.hf = true;
    w.blend = std::max<int64_t>(w.blend, 5 * W);
    w.proj = std::max<int64_t>(w.proj, 4 * HD);
    w.baf = std::max<int64_t>(w.baf, d.decay_rank);
    w.cq = std::max<int64_t>(w.cq, d.decay_rank);
    w.cvf = std::max<int64_t>(w.cvf, 5 * HD);  // r | k | v | w and the raw outputs
    w.attn = std::max<int64_t>(w.attn, HD);
  } else if (d.mixer == B200Q_MIXER_WINDOW_ATTN) {
    w.proj = std::max<int64_t>(w.proj, window_proj_rows(d));
    w.qa = std::max<int64_t>(w.qa, HD);
    w.attn = std::max<int64_t>(w.attn, HV);
  }
}
Widths widths_of(const b200q_model_config& c, const std::vector<b200q_layered_layer>& Ls) {
  Widths w;
  for (const auto& l : Ls) {
    const b200q_layer_desc& d = l.d;
    if (d.mixer == B200Q_MIXER_LATENT_ATTN) {
      const int64_t RP = d.kv_rank + d.rot_dim;
      w.proj = std::max<int64_t>(w.proj, d.q_rank > 0 ? d.q_rank + (d.kv_from < 0 ? RP : 0) : latent_full_rows(d));
      w.cq = std::max<int64_t>(w.cq, d.q_rank);
      if (d.q_rank > 0) w.q = std::max<int64_t>(w.q, (int64_t)d.heads * (d.dim + d.rot_dim));
      w.qa = std::max<int64_t>(w.qa, (int64_t)d.heads * RP);
      w.olat = std::max<int64_t>(w.olat, (int64_t)d.heads * d.kv_rank);
      w.attn = std::max<int64_t>(w.attn, (int64_t)d.heads * d.vdim);
    } else if (d.mixer == B200Q_MIXER_GENERAL_DELTA) {
      w.proj = std::max<int64_t>(w.proj, 5 * (int64_t)d.heads * d.dim + d.decay_rank);
      w.attn = std::max<int64_t>(w.attn, (int64_t)d.heads * d.dim);
      w.delta = std::max<int64_t>(w.delta, (int64_t)d.heads * d.dim);
    } else if (d.mixer == B200Q_MIXER_GATED_DELTA) {
      const int64_t GD = (int64_t)d.kv_heads * d.dim, HV = (int64_t)d.heads * d.vdim;
      w.proj = std::max<int64_t>(w.proj, 2 * GD + 2 * HV);
      w.cvf = std::max<int64_t>(w.cvf, 2 * GD + 2 * HV);  // convolved q|k|v and, behind them, the raw outputs
      w.baf = std::max<int64_t>(w.baf, 2 * (int64_t)d.heads);
      w.attn = std::max<int64_t>(w.attn, HV);
    } else if (d.mixer == B200Q_MIXER_CHUNK_ATTN) {
      const int64_t HD = (int64_t)d.heads * d.dim;
      w.proj = std::max<int64_t>(w.proj, 2 * HD + (int64_t)d.kv_heads * d.dim);
      w.qa = std::max<int64_t>(w.qa, HD);
      w.attn = std::max<int64_t>(w.attn, HD);
    } else if (d.mixer == B200Q_MIXER_SELECTIVE_SCAN) {
      w.proj = std::max<int64_t>(w.proj, 2 * (int64_t)d.inner);
      w.xc = std::max<int64_t>(w.xc, d.inner);
      w.xp = std::max<int64_t>(w.xp, (d.dt_rank + 2 * (int64_t)d.state_dim + 63) & ~(int64_t)63);
      w.dtr = std::max<int64_t>(w.dtr, d.inner);
      w.attn = std::max<int64_t>(w.attn, d.inner);
    } else {
      sequence_mixer_widths(d, c.hidden, w);
    }
    if (d.side_mixer) {
      w.side = true;
      sequence_mixer_widths(side_desc(d), c.hidden, w);
    }
    if (d.inject) w.inject = true;
    if (d.ff == B200Q_FF_GEGLU) {
      w.ffh = std::max<int64_t>(w.ffh, 2 * (int64_t)d.ff_dim);
      w.ffa = std::max<int64_t>(w.ffa, d.ff_dim);
    } else if (d.ff == B200Q_FF_RELU2) {
      w.ffh = std::max<int64_t>(w.ffh, d.ff_dim);
    } else if (d.ff == B200Q_FF_MOE_GROUPED) {
      w.moe = true;
      w.experts = std::max<int64_t>(w.experts, d.n_experts + d.n_identity);
      w.pairs = std::max<int64_t>(w.pairs, d.top_k);
      w.egu = std::max<int64_t>(w.egu, (int64_t)d.top_k * d.ff_dim);
    }
    if (d.ff == B200Q_FF_MOE_SIGMOID) {
      w.moe = true;
      w.experts = std::max<int64_t>(w.experts, d.n_experts);
      w.pairs = std::max<int64_t>(w.pairs, d.top_k);
      w.egu = std::max<int64_t>(w.egu, (int64_t)d.top_k * 2 * d.ff_dim);
      w.eact = std::max<int64_t>(w.eact, (int64_t)d.top_k * d.ff_dim);
    } else if (d.ff == B200Q_FF_POLYNORM) {
      w.ffh = std::max<int64_t>(w.ffh, d.ff_dim);
      w.ffa = std::max<int64_t>(w.ffa, d.ff_dim);
    } else if (d.ff == B200Q_FF_MOE) {
      w.moe = true;
      w.experts = std::max<int64_t>(w.experts, d.n_experts);
      w.pairs = std::max<int64_t>(w.pairs, d.top_k);
      w.egu = std::max<int64_t>(w.egu, (int64_t)d.top_k * 2 * d.ff_dim);
      w.eact = std::max<int64_t>(w.eact, (int64_t)d.top_k * d.ff_dim);
      if (d.shared_dim > 0) {
        w.shared = true;
        w.ffh = std::max<int64_t>(w.ffh, 2 * (int64_t)d.shared_dim);
        w.ffa = std::max<int64_t>(w.ffa, d.shared_dim);
      }
    }
  }
  return w;
}

// one pass lays the workspace out; with base == nullptr it only measures
int64_t layout(b200q_model* m, uint8_t* base) {
  const b200q_model_config& c = m->cfg;
  b200q_layered* y = m->lay;
  const Widths w = widths_of(c, y->layers);
  const int64_t T = c.max_tokens, W = c.hidden, es = esize(c), LR = logit_rows(c);
  int64_t off = 0;
  auto take = [&](int64_t bytes) -> void* {
    void* r = base ? base + off : nullptr;
    off += al256(bytes);
    return r;
  };
  y->x = (float*)take(T * W * 4);
  y->h1 = take(T * W * es);
  y->h2 = take(T * W * es);
  y->mix = take(T * W * es);
  y->ffo = take(T * W * es);
  y->proj = take(T * w.proj * es);
  y->cq = take(T * w.cq * es);
  y->q = take(T * w.q * es);
  y->qa = (float*)take(T * w.qa * 4);
  y->olat = take(T * w.olat * es);
  y->attn = take(T * w.attn * es);
  y->dscr = (float*)take(w.delta ? T * w.delta * 6 * 4 : 1);
  y->cvf = (float*)take(w.cvf ? T * w.cvf * 4 : 1);
  y->baf = (float*)take(w.baf ? T * w.baf * 4 : 1);
  y->dtr = (float*)take(w.dtr ? T * w.dtr * 4 : 1);
  y->xc = take(w.xc ? T * w.xc * es : 1);
  y->xp = take(w.xp ? T * w.xp * es : 1);
  y->ffh = take(T * w.ffh * es);
  y->ffa = take(T * w.ffa * es);
  y->rlog = (float*)take(T * w.experts * 4);
  y->idx = (int32_t*)take(T * w.pairs * 4);
  y->wts = (float*)take(T * w.pairs * 4);
  y->perm_tok = (int32_t*)take(T * w.pairs * 4);
  y->pair_pos = (int32_t*)take(T * w.pairs * 4);
  y->group_off = (int32_t*)take((w.experts + 1) * 4);
  y->tile_tab = (int32_t*)take((T * w.pairs / 128 + w.experts + 1) * 16);
  y->n_tiles = (int32_t*)take(16);
  y->esrc = take(w.moe ? T * w.pairs * W * es : 1);
  y->egu = take(T * w.egu * es);
  y->eact = take(T * w.eact * es);
  y->eout = take(w.moe ? T * w.pairs * W * es : 1);
  y->shout = take(w.shared ? T * W * es : 1);
  y->sgate = (float*)take(T * 4);
  y->hf = (float*)take(w.hf ? T * W * 4 : 1);
  y->x0 = (float*)take(w.inject ? T * W * 4 : 1);
  y->cat = take(w.inject ? T * 2 * W * es : 1);
  y->carry = (float*)take(c.token_shift ? (int64_t)c.max_seqs * W * 4 : 1);
  y->mix2 = take(w.side ? T * W * es : 1);
  y->blend = take(w.blend ? T * w.blend * es : 1);
  y->tg = take(c.side_dim > 0 ? T * c.side_dim * es : 1);
  y->ta = take(c.side_dim > 0 ? T * c.side_dim * es : 1);
  y->sel = take(LR * W * es);
  y->logits = (float*)take(LR * (int64_t)c.vocab * 4);
  y->logits_bf16 = take((int64_t)c.max_seqs * c.vocab * 2);
  return off;
}

// the layer's rotation frequencies (fp64, on the device) and the factor of sine and cosine
int upload_frequencies(b200q_layered_layer& l) {
  const b200q_layer_desc& d = l.d;
  const int half = d.rot_dims / 2;
  if (half <= 0) return B200Q_OK;
  std::vector<double> f(half);
  int rc = b200q_rot_frequencies(d.rot_dims, d.rot_base, d.rot_factor, d.rot_original, d.rot_fast, d.rot_slow, f.data(),
                                 &l.mag);
  if (rc) return rc;
  if (cudaMalloc(&l.freq, half * sizeof(double)) != cudaSuccess ||
      cudaMemcpy(l.freq, f.data(), half * sizeof(double), cudaMemcpyHostToDevice) != cudaSuccess) {
    set_error("create_layered: CUDA allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
    return B200Q_ECUDA;
  }
  return B200Q_OK;
}

}  // namespace

namespace b200q {

int layered_create(const b200q_model_config* cfg, const b200q_layer_desc* layers, b200q_model_t* out) {
  B200Q_CHECK_ARG(out != nullptr, "out is null");
  int rc = check_layered(cfg, layers);
  if (rc) return rc;
  rc = b200q_device_check();
  if (rc) return rc;
  b200q_model* m = new b200q_model();
  m->cfg = *cfg;
  m->lay = new b200q_layered();
  m->lay->layers.resize(cfg->n_layers);
  const int es = esize(*cfg);
  for (int i = 0; i < cfg->n_layers; ++i) {
    b200q_layered_layer& l = m->lay->layers[i];
    l.d = layers[i];
    if (l.d.mixer == B200Q_MIXER_LATENT_ATTN) {
      if (l.d.kv_from < 0) {
        l.cache_block_off = m->lay->kv_block_bytes;
        m->lay->kv_block_bytes += (int64_t)cfg->block_size * (l.d.kv_rank + l.d.rot_dim) * es;
      } else {
        l.cache_block_off = m->lay->layers[l.d.kv_from].cache_block_off;
      }
      if ((rc = upload_frequencies(l))) {
        b200q_model_destroy(m);
        return rc;
      }
    } else if (l.d.mixer == B200Q_MIXER_GENERAL_DELTA) {
      l.state_off = m->lay->state_slot_floats;
      m->lay->state_slot_floats += (int64_t)l.d.heads * l.d.dim * l.d.dim;
    } else if (l.d.mixer == B200Q_MIXER_GATED_DELTA) {
      l.state_off = m->lay->state_slot_floats;
      m->lay->state_slot_floats += (int64_t)l.d.heads * l.d.dim * l.d.vdim;
      l.conv_off = m->lay->state_slot_floats;
      m->lay->state_slot_floats += (int64_t)(l.d.conv_taps - 1) * (2 * l.d.kv_heads * l.d.dim + l.d.heads * l.d.vdim);
    } else if (l.d.mixer == B200Q_MIXER_CHUNK_ATTN) {
      l.cache_block_off = m->lay->kv_block_bytes;
      m->lay->kv_block_bytes += (int64_t)cfg->block_size * l.d.kv_heads * l.d.dim * es;
    } else if (l.d.mixer == B200Q_MIXER_SELECTIVE_SCAN) {
      l.state_off = m->lay->state_slot_floats;
      m->lay->state_slot_floats += (int64_t)l.d.inner * l.d.state_dim;
      l.conv_off = m->lay->state_slot_floats;
      m->lay->state_slot_floats += (int64_t)(l.d.conv_taps - 1) * l.d.inner;
    } else if (l.d.mixer == B200Q_MIXER_WINDOW_ATTN) {
      if (l.d.kv_from < 0) {
        l.cache_block_off = m->lay->kv_block_bytes;
        m->lay->kv_block_bytes += (int64_t)cfg->block_size * l.d.kv_heads * (l.d.dim + l.d.vdim) * es;
      } else {  // the keys and values of an earlier layer, as its cache holds them
        l.cache_block_off = m->lay->layers[l.d.kv_from].cache_block_off;
      }
      if ((rc = upload_frequencies(l))) {
        b200q_model_destroy(m);
        return rc;
      }
    }
    if (l.d.side_mixer) {
      l.side.resize(1);
      l.side[0].d = side_desc(l.d);
    }
    // recurrent mixers of the pre-norm form, first or side: the state, and for the decay mix the carried input
    for (b200q_layered_layer* q : {&l, l.side.empty() ? (b200q_layered_layer*)nullptr : &l.side[0]}) {
      if (!q || (q->d.mixer != B200Q_MIXER_LIGHTNING && q->d.mixer != B200Q_MIXER_DECAY_MIX)) continue;
      m->lay->state_slot_floats = (m->lay->state_slot_floats + 3) & ~(int64_t)3;
      q->state_off = m->lay->state_slot_floats;
      m->lay->state_slot_floats += (int64_t)q->d.heads * q->d.dim * q->d.vdim;
      if (q->d.mixer == B200Q_MIXER_DECAY_MIX) {
        q->prev_off = m->lay->state_slot_floats;
        m->lay->state_slot_floats += cfg->hidden;
      }
    }
    if (cfg->token_shift) {
      l.shift_off = m->lay->state_slot_floats;
      m->lay->state_slot_floats += cfg->hidden;
    }
    if (cfg->layer_form == B200Q_FORM_POSTNORM && cfg->input_taps > 1) {
      // the last inputs of the two sublayers' input convolutions travel with the sequence
      l.canon1_off = m->lay->state_slot_floats;
      m->lay->state_slot_floats += (int64_t)(cfg->input_taps - 1) * cfg->hidden;
      if (l.d.ff != B200Q_FF_NONE) {
        l.canon2_off = m->lay->state_slot_floats;
        m->lay->state_slot_floats += (int64_t)(cfg->input_taps - 1) * cfg->hidden;
      }
    }
    m->lay->state_slot_floats = (m->lay->state_slot_floats + 3) & ~(int64_t)3;  // regions stay 16-byte aligned
  }
  *out = m;
  return B200Q_OK;
}

void layered_destroy(b200q_model* m) {
  if (!m->lay) return;
  for (auto& l : m->lay->layers)
    if (l.freq) cudaFree(l.freq);
  delete m->lay;
  m->lay = nullptr;
}

int64_t layered_workspace_bytes(b200q_model* m) { return layout(m, nullptr); }

int layered_bind_workspace(b200q_model* m, void* p, int64_t bytes) {
  const int64_t need = layout(m, nullptr);
  B200Q_CHECK_ARG(bytes >= need, "workspace too small: %lld < %lld", (long long)bytes, (long long)need);
  B200Q_CHECK_ARG((reinterpret_cast<uintptr_t>(p) & 255) == 0, "workspace must be 256-byte aligned");
  m->ws = (uint8_t*)p;
  m->ws_bytes = bytes;
  layout(m, (uint8_t*)p);
  return B200Q_OK;
}

int layered_bind_weight(b200q_model* m, const char* name, const void* p, int64_t rows, int64_t cols) {
  const b200q_model_config& c = m->cfg;
  const int64_t W = c.hidden;
  auto expect = [&](int64_t r, int64_t cc) -> int {
    B200Q_CHECK_ARG(rows == r && cols == cc, "weight %s has shape [%lld,%lld], expected [%lld,%lld]", name,
                    (long long)rows, (long long)cols, (long long)r, (long long)cc);
    return B200Q_OK;
  };
  int rc;
  if (!strcmp(name, "embed")) { if ((rc = expect(c.vocab, W))) return rc; m->embed = p; return B200Q_OK; }
  if (!strcmp(name, "final_norm")) {
    const bool dyt = c.layer_form == B200Q_FORM_SANDWICH && c.norm_kind == B200Q_NORM_DYT;
    if ((rc = expect(1, dyt ? 2 * W + 1 : W))) return rc;
    m->final_norm = p;
    return B200Q_OK;
  }
  if (!strcmp(name, "lm_head")) { if ((rc = expect(c.vocab, W))) return rc; m->lm_head = p; return B200Q_OK; }
  if (!strcmp(name, "tok_embed")) {
    B200Q_CHECK_ARG(c.side_dim > 0 && rows == c.vocab && cols >= (int64_t)c.n_layers * c.side_dim,
                    "weight tok_embed has shape [%lld,%lld], expected [%d, >= %lld]", (long long)rows, (long long)cols,
                    c.vocab, (long long)c.n_layers * c.side_dim);
    m->lay->tok_embed = p;
    m->lay->tok_cols = cols;
    return B200Q_OK;
  }
  if (!strcmp(name, "pos")) {
    B200Q_CHECK_ARG(c.learned_pos && cols == W && rows >= c.max_pos, "weight pos has shape [%lld,%lld], expected [>= %d,%lld]",
                    (long long)rows, (long long)cols, c.max_pos, (long long)W);
    m->lay->pos = p;
    m->lay->pos_rows = rows;
    return B200Q_OK;
  }
  int li = -1;
  char field[48] = {0};
  if (sscanf(name, "layers.%d.%47s", &li, field) != 2 || li < 0 || li >= c.n_layers) {
    set_error("bind_weight: unknown weight name '%s'", name);
    return B200Q_EINVAL;
  }
  b200q_layered_layer& l = m->lay->layers[li];
  const b200q_layer_desc& d = l.d;
  const int64_t HD = (int64_t)d.heads * d.dim;
#define FIELD(fname, slot, r, cc)                        \
  if (!strcmp(field, fname)) {                           \
    if ((rc = expect((r), (cc)))) return rc;             \
    *(const void**)&(slot) = p;                          \
    return B200Q_OK;                                     \
  }
  if (c.layer_form == B200Q_FORM_SANDWICH) {
    // norm rows: dynamic tanh [w | b | alpha], RMS [w]
    const int64_t NW = c.norm_kind == B200Q_NORM_DYT ? 2 * W + 1 : W;
    FIELD("norm1", l.norm1, 1, NW)
    FIELD("norm1b", l.norm1b, 1, NW)
    if (d.ff != B200Q_FF_NONE) {
      FIELD("norm2", l.norm2, 1, NW)
      FIELD("norm2b", l.norm2b, 1, NW)
    }
    if (c.side_dim > 0) {
      FIELD("tok.gate", l.tok_gate, c.side_dim, W)
      FIELD("tok.proj", l.tok_proj, W, c.side_dim)
      FIELD("tok.norm", l.tok_norm, 1, W)
    }
  }
  FIELD("norm1", l.norm1, 1, W)
  if (d.ff != B200Q_FF_NONE) FIELD("norm2", l.norm2, 1, W)
  if (c.token_shift) FIELD("shift", l.shift, 1, W)
  if (d.inject) FIELD("inject", l.inject, W, 2 * W)
  // the mixers of the pre-norm form, as a layer's first mixer ("mix.*") or beside it ("side.*")
  for (int which = 0; which < 2; ++which) {
    b200q_layered_layer* q = which == 0 ? &l : (l.side.empty() ? nullptr : &l.side[0]);
    const char* pre = which == 0 ? "mix." : "side.";
    if (!q || strncmp(field, pre, strlen(pre)) != 0) continue;
    const char* f = field + strlen(pre);
    const b200q_layer_desc& e = q->d;
    const int64_t QD = (int64_t)e.heads * e.dim, QV = (int64_t)e.heads * e.vdim;
#define SUB(fname, slot, r, cc)                          \
  if (!strcmp(f, fname)) {                               \
    if ((rc = expect((r), (cc)))) return rc;             \
    *(const void**)&(slot) = p;                          \
    return B200Q_OK;                                     \
  }
    if (e.mixer == B200Q_MIXER_LIGHTNING) {
      SUB("proj", q->proj, 2 * QD + 2 * QV, W)
      SUB("decay", q->head_decay, 1, e.heads)
      SUB("out_norm", q->out_norm, 1, QV)
      SUB("o", q->o, W, QV)
    } else if (e.mixer == B200Q_MIXER_DECAY_MIX) {
      SUB("mu", q->mu, 1, 5 * W)
      SUB("proj", q->proj, 4 * QD, W)
      SUB("w1", q->w1, e.decay_rank, W)
      SUB("w2", q->w2, QD, e.decay_rank)
      SUB("w0", q->w0, 1, QD)
      SUB("bonus", q->bonus, 1, QD)
      SUB("out_norm", q->out_norm, 1, QD)
      SUB("o", q->o, W, QD)
    } else if (e.mixer == B200Q_MIXER_WINDOW_ATTN) {
      SUB("proj", q->proj, window_proj_rows(e), W)
      if (!e.bare) SUB("temp", q->temp, 1, e.heads)
      if (e.proj_bias) {
        SUB("proj_b", q->proj_b, 1, window_proj_rows(e))
        SUB("o_b", q->o_b, 1, W)
      }
      if (e.qk_norm) {
        SUB("q_norm", q->q_norm, 1, e.qk_norm == 1 ? QD : e.dim)
        if (e.kv_from < 0) SUB("k_norm", q->kv_norm, 1, e.qk_norm == 1 ? (int64_t)e.kv_heads * e.dim : e.dim)
      }
      SUB("o", q->o, W, QV)
    }
#undef SUB
  }
  if (c.layer_form == B200Q_FORM_POSTNORM) {
    FIELD("ls1", l.ls1, 1, W)
    if (d.ff != B200Q_FF_NONE) FIELD("ls2", l.ls2, 1, W)
    if (c.input_taps > 0) {
      FIELD("canon1", l.canon1, 1, W * c.input_taps)
      if (d.ff != B200Q_FF_NONE) FIELD("canon2", l.canon2, 1, W * c.input_taps)
    }
  }
  if (d.mixer == B200Q_MIXER_GATED_DELTA) {
    const int64_t GD = (int64_t)d.kv_heads * d.dim, HV = (int64_t)d.heads * d.vdim;
    FIELD("mix.proj", l.proj, 2 * GD + 2 * HV, W)
    FIELD("mix.ba", l.ba, 2 * d.heads, W)
    FIELD("mix.conv", l.conv_w, 1, (2 * GD + HV) * d.conv_taps)
    FIELD("mix.a_log", l.a_log, 1, d.heads)
    FIELD("mix.dt_bias", l.dt_bias, 1, d.heads)
    FIELD("mix.out_norm", l.out_norm, 1, d.vdim)
    FIELD("mix.o", l.o, W, HV)
  } else if (d.mixer == B200Q_MIXER_CHUNK_ATTN) {
    FIELD("mix.proj", l.proj, 2 * HD + (int64_t)d.kv_heads * d.dim, W)
    FIELD("mix.q_norm", l.q_norm, 1, d.dim)
    FIELD("mix.k_norm", l.kv_norm, 1, d.dim)
    FIELD("mix.r1", l.r1, 1, d.heads)
    FIELD("mix.r2", l.r2, 1, d.heads)
    FIELD("mix.o", l.o, W, HD)
  } else if (d.mixer == B200Q_MIXER_SELECTIVE_SCAN) {
    FIELD("mix.proj", l.proj, 2 * d.inner, W)
    FIELD("mix.conv", l.conv_w, 1, (int64_t)d.inner * d.conv_taps)
    FIELD("mix.conv_b", l.conv_b, 1, d.inner)
    FIELD("mix.x", l.x_proj, (d.dt_rank + 2 * d.state_dim + 63) & ~63, d.inner)  // zero rows up to a multiple of 64
    FIELD("mix.dt", l.dt_proj, d.inner, d.dt_rank)
    FIELD("mix.dt_b", l.dt_b, 1, d.inner)
    FIELD("mix.a_log", l.a_log, 1, (int64_t)d.inner * d.state_dim)
    FIELD("mix.d", l.dvec, 1, d.inner)
    FIELD("mix.o", l.o, W, d.inner)
  } else if (d.mixer == B200Q_MIXER_LATENT_ATTN) {
    const int64_t RP = d.kv_rank + d.rot_dim;
    if (d.q_rank > 0) {
      FIELD("mix.down", l.down, d.q_rank + (d.kv_from < 0 ? RP : 0), W)
      FIELD("mix.q_norm", l.q_norm, 1, d.q_rank)
      FIELD("mix.uq", l.uq, (int64_t)d.heads * (d.dim + d.rot_dim), d.q_rank)
    } else {
      FIELD("mix.down", l.down, latent_full_rows(d), W)
    }
    if (d.kv_from < 0) FIELD("mix.kv_norm", l.kv_norm, 1, d.kv_rank)
    FIELD("mix.uk_t", l.uk_t, (int64_t)d.heads * d.kv_rank, d.dim)
    FIELD("mix.uv", l.uv, (int64_t)d.heads * d.vdim, d.kv_rank)
    FIELD("mix.o", l.o, W, (int64_t)d.heads * d.vdim)
  } else if (d.mixer == B200Q_MIXER_GENERAL_DELTA) {
    FIELD("mix.proj", l.proj, 5 * HD + d.decay_rank, W)
    FIELD("mix.w2", l.w2, HD, d.decay_rank)
    FIELD("mix.w0", l.w0, 1, HD)
    FIELD("mix.a_bias", l.a_bias, 1, HD)
    FIELD("mix.out_norm", l.out_norm, 1, HD)
    FIELD("mix.o", l.o, W, HD)
  }
  if (d.ff == B200Q_FF_GEGLU) {
    FIELD("mlp.gate_up", l.gate_up, 2 * (int64_t)d.ff_dim, W)
    if (!strcmp(field, "mlp.gate_up_il")) {
      B200Q_CHECK_ARG(d.ff_dim % 128 == 0, "layer %d: interleaved gate / up rows need ff (%d) to be a multiple of 128", li,
                      d.ff_dim);
      if ((rc = expect(2 * (int64_t)d.ff_dim, W))) return rc;
      l.gate_up = p;
      l.gate_up_il = true;
      return B200Q_OK;
    }
    FIELD("mlp.down", l.ff_down, W, d.ff_dim)
  } else if (d.ff == B200Q_FF_RELU2) {
    FIELD("mlp.up", l.up, d.ff_dim, W)
    FIELD("mlp.down", l.ff_down, W, d.ff_dim)
  } else if (d.ff == B200Q_FF_MOE_GROUPED) {
    FIELD("mlp.router", l.router, d.n_experts + d.n_identity, W)
    FIELD("mlp.router_bias", l.router_bias, 1, d.n_experts + d.n_identity)
    if (d.n_experts > 0) {
      FIELD("mlp.experts_up", l.experts_up, (int64_t)d.n_experts * d.ff_dim, W)
      FIELD("mlp.experts_down", l.experts_down, (int64_t)d.n_experts * W, d.ff_dim)
    }
  } else if (d.ff == B200Q_FF_MOE_SIGMOID) {
    FIELD("mlp.router", l.router, d.n_experts, W)
    FIELD("mlp.experts_gate_up", l.experts_gate_up, (int64_t)d.n_experts * 2 * d.ff_dim, W)
    FIELD("mlp.experts_down", l.experts_down, (int64_t)d.n_experts * W, d.ff_dim)
  } else if (d.ff == B200Q_FF_POLYNORM) {
    FIELD("mlp.up", l.up, d.ff_dim, W)
    FIELD("mlp.act", l.act, 1, 4)
    FIELD("mlp.down", l.ff_down, W, d.ff_dim)
  } else if (d.ff == B200Q_FF_MOE) {
    FIELD("mlp.router", l.router, d.n_experts, W)
    FIELD("mlp.router_bias", l.router_bias, 1, d.n_experts)
    FIELD("mlp.experts_gate_up", l.experts_gate_up, (int64_t)d.n_experts * 2 * d.ff_dim, W)
    FIELD("mlp.experts_down", l.experts_down, (int64_t)d.n_experts * W, d.ff_dim)
    if (d.shared_dim > 0) {
      FIELD("mlp.shared_gate_up", l.shared_gate_up, 2 * (int64_t)d.shared_dim, W)
      FIELD("mlp.shared_down", l.shared_down, W, d.shared_dim)
      FIELD("mlp.shared_gate", l.shared_gate, 1, W)
    }
  }
#undef FIELD
  set_error("bind_weight: layer %d has no weight '%s'", li, field);
  return B200Q_EINVAL;
}

static int check_bound(b200q_model* m) {
  if (!m->embed || !m->final_norm || !m->lm_head || !m->ws || (m->cfg.learned_pos && !m->lay->pos)) {
    set_error("forward: model not fully bound (embed/pos/final_norm/lm_head/workspace)");
    return B200Q_ESTATE;
  }
  bool need_kv = false, need_state = false;
  for (size_t i = 0; i < m->lay->layers.size(); ++i) {
    const b200q_layered_layer& l = m->lay->layers[i];
    const b200q_layer_desc& d = l.d;
    bool ok = l.norm1 && l.o && (d.ff == B200Q_FF_NONE || l.norm2);
    if (m->cfg.layer_form == B200Q_FORM_POSTNORM) {
      ok = ok && l.ls1 && (d.ff == B200Q_FF_NONE || l.ls2);
      if (m->cfg.input_taps > 0) ok = ok && l.canon1 && (d.ff == B200Q_FF_NONE || l.canon2);
      if (m->cfg.input_taps > 1) need_state = true;
    }
    if (d.mixer == B200Q_MIXER_LATENT_ATTN) {
      need_kv = true;
      ok = ok && l.down && (d.q_rank == 0 || (l.q_norm && l.uq)) && (d.kv_from >= 0 || l.kv_norm) && l.uk_t && l.uv;
    } else if (d.mixer == B200Q_MIXER_GENERAL_DELTA) {
      need_state = true;
      ok = ok && l.proj && l.w2 && l.w0 && l.a_bias && l.out_norm;
    } else if (d.mixer == B200Q_MIXER_GATED_DELTA) {
      need_state = true;
      ok = ok && l.proj && l.ba && l.conv_w && l.a_log && l.dt_bias && l.out_norm;
    } else if (d.mixer == B200Q_MIXER_CHUNK_ATTN) {
      need_kv = true;
      ok = ok && l.proj && l.q_norm && l.kv_norm && l.r1 && l.r2;
    } else if (d.mixer == B200Q_MIXER_SELECTIVE_SCAN) {
      need_state = true;
      ok = ok && l.proj && l.conv_w && l.conv_b && l.x_proj && l.dt_proj && l.dt_b && l.a_log && l.dvec;
    }
    if (m->cfg.token_shift) {
      need_state = true;
      ok = ok && l.shift;
    }
    if (d.inject) ok = ok && l.inject;
    for (const b200q_layered_layer* q : {&l, l.side.empty() ? (const b200q_layered_layer*)nullptr : &l.side[0]}) {
      if (!q) continue;
      if (q != &l) ok = ok && q->o;
      if (q->d.mixer == B200Q_MIXER_LIGHTNING) {
        need_state = true;
        ok = ok && q->proj && q->head_decay && q->out_norm;
      } else if (q->d.mixer == B200Q_MIXER_DECAY_MIX) {
        need_state = true;
        ok = ok && q->mu && q->proj && q->w1 && q->w2 && q->w0 && q->bonus && q->out_norm;
      } else if (q->d.mixer == B200Q_MIXER_WINDOW_ATTN) {
        need_kv = true;
        ok = ok && q->proj && (q->d.bare || q->temp) && (!q->d.proj_bias || (q->proj_b && q->o_b)) &&
             (!q->d.qk_norm || (q->q_norm && (q->d.kv_from >= 0 || q->kv_norm)));
      }
    }
    if (d.ff == B200Q_FF_RELU2) ok = ok && l.up && l.ff_down;
    if (d.ff == B200Q_FF_GEGLU) ok = ok && l.gate_up && l.ff_down;
    if (m->cfg.layer_form == B200Q_FORM_SANDWICH)
      ok = ok && l.norm1b && (d.ff == B200Q_FF_NONE || l.norm2b) &&
           (m->cfg.side_dim == 0 || (l.tok_gate && l.tok_proj && l.tok_norm && m->lay->tok_embed));
    if (d.ff == B200Q_FF_MOE_GROUPED)
      ok = ok && l.router && l.router_bias && (d.n_experts == 0 || (l.experts_up && l.experts_down));
    if (d.ff == B200Q_FF_MOE_SIGMOID) ok = ok && l.router && l.experts_gate_up && l.experts_down;
    if (d.ff == B200Q_FF_POLYNORM) ok = ok && l.up && l.act && l.ff_down;
    if (d.ff == B200Q_FF_MOE)
      ok = ok && l.router && l.router_bias && l.experts_gate_up && l.experts_down &&
           (d.shared_dim == 0 || (l.shared_gate_up && l.shared_down && l.shared_gate));
    if (!ok) {
      set_error("forward: layer %d has unbound weights", (int)i);
      return B200Q_ESTATE;
    }
  }
  if ((need_kv && !m->kv) || (need_state && !m->lay->state)) {
    set_error("forward: cache / recurrent state not bound");
    return B200Q_ESTATE;
  }
  return B200Q_OK;
}

int layered_forward(b200q_model* m, const b200q_batch* b, void* stream) {
  int rc = check_bound(m);
  if (rc) return rc;
  const b200q_model_config& c = m->cfg;
  b200q_layered* y = m->lay;
  const int T = b->T, W = c.hidden, dt = c.dtype, es = esize(c);
  B200Q_CHECK_ARG(T >= 0 && T <= c.max_tokens, "forward: T=%d exceeds workspace (%d)", T, c.max_tokens);
  B200Q_CHECK_ARG(b->n_sample >= 0 && b->n_sample <= (b->no_sampling ? logit_rows(c) : c.max_seqs),
                  "forward: n_sample=%d exceeds the logits buffer", b->n_sample);
  B200Q_CHECK_ARG(b->seq_desc && b->row_seq && b->n_rows > 0, "forward: a layered model needs the per-sequence "
                  "view of the step (seq_desc / row_seq)");
  if (T == 0) return B200Q_OK;
  cudaStream_t cst = as_stream(stream);
#define TRY(cat, work, call)                                \
  do {                                                      \
    int _e0 = -1;                                           \
    if (m->profiling) {                                     \
      _e0 = m->get_event();                                 \
      cudaEventRecord(m->ev_pool[_e0], cst);                \
    }                                                       \
    rc = (call);                                            \
    if (rc) return rc;                                      \
    if (m->profiling) {                                     \
      int _e1 = m->get_event();                             \
      cudaEventRecord(m->ev_pool[_e1], cst);                \
      m->spans.push_back({(cat), (double)(work), _e0, _e1}); \
    }                                                       \
  } while (0)
#define LIN(Aptr, lda, Wptr, bias, Cptr, ldc, N, K, f32)                                                     \
  TRY(B200Q_PROF_GEMM, 2.0 * T * (double)(N) * (K),                                                          \
      b200q_linear((Aptr), (lda), (Wptr), (bias), (Cptr), (ldc), T, (N), (K), dt, (f32), stream))
  const int EW = B200Q_PROF_ELEMENTWISE;

  const bool post = c.layer_form == B200Q_FORM_POSTNORM, pre = c.layer_form == B200Q_FORM_PRENORM,
             sandwich = c.layer_form == B200Q_FORM_SANDWICH;
  const float mult = c.residual_mult > 0.f ? c.residual_mult : 1.f;
  const int groups = c.norm_groups > 0 ? c.norm_groups : 1;
  if (c.learned_pos)
    TRY(EW, (double)T * W * (2 * es + 4),
        b200q_embed_pos_f32(b->token_ids, b->prev_out_ids, m->embed, y->pos, b->positions, y->x, T, W, dt, stream));
  else
    TRY(EW, (double)T * W * (es + 4),
        b200q_embed_f32(b->token_ids, b->prev_out_ids, m->embed, y->x, T, W, c.embed_scale > 0.f ? c.embed_scale : 1.f,
                        dt, stream));

  // ---- mixers 6-8: read y->h1 [T, W] (model dtype; the decay mix reads the fp32 rows y->hf), write outp [T, W] ----
  auto run_sequence_mixer = [&](const b200q_layered_layer& l, void* outp) -> int {
    const b200q_layer_desc& d = l.d;
    const int H = d.heads, HD = H * d.dim, HV = H * d.vdim;
    if (d.mixer == B200Q_MIXER_LIGHTNING) {
      const int NC = 2 * HD + HV, NP = NC + HV;
      LIN(y->h1, W, l.proj, nullptr, y->proj, NP, NP, W, 0);  // [q | k | v | gate]
      TRY(EW, (double)T * NC * (es + 4), b200q_act_to_f32(y->proj, NP, y->cvf, NC, NC, 1, T, dt, stream));
      float* raw = y->cvf + (int64_t)T * NC;
      TRY(B200Q_PROF_PREFILL_ATTN, 4.0 * T * H * (double)d.dim * d.vdim,
          b200q_decay_attn(y->cvf, NC, 0, HD, 2 * HD, l.head_decay, nullptr, 0, nullptr, y->state + l.state_off,
                           y->state_slot_floats, b->seq_desc, b->n_rows, H, d.dim, d.vdim, raw, stream));
      TRY(EW, (double)T * HV * (4 + 2 * es),
          b200q_gated_rmsnorm(raw, HV, HV, l.out_norm, (uint8_t*)y->proj + (size_t)NC * es, NP, 0, c.rms_eps, y->attn, T,
                              dt, stream));
      LIN(y->attn, HV, l.o, nullptr, outp, W, W, HV, 0);
    } else if (d.mixer == B200Q_MIXER_DECAY_MIX) {
      const int R = d.decay_rank, NQ = 4 * HD;
      TRY(EW, (double)T * W * (4 + 5 * es),
          b200q_shift_blend(y->hf, l.mu, 5, y->state + l.prev_off, y->state_slot_floats, b->seq_desc, b->row_seq, 1,
                            y->blend, T, W, dt, stream));
      // every reader of the carried input has run: the last row of each longer portion takes its place (single
      // tokens stored theirs while blending, so a step of single tokens launches nothing here)
      if (T > b->n_rows)
        TRY(EW, 8.0 * b->n_rows * W,
            b200q_store_carry(y->hf, 1, y->state + l.prev_off, y->state_slot_floats, b->seq_desc, b->n_rows, W, 1, stream));
      // r, k, v, gate: product g reads blend g (a column slice of the blend rows)
      TRY(B200Q_PROF_GEMM, 2.0 * T * 4.0 * HD * W,
          b200q_linear_batched(y->blend, 5 * W, W, l.proj, (long long)HD * W, y->proj, NQ, HD, T, HD, W, 4, dt, 0, stream));
      LIN((uint8_t*)y->blend + (size_t)4 * W * es, 5 * W, l.w1, nullptr, y->baf, R, R, W, 1);
      TRY(EW, (double)T * R * (4 + es), b200q_tanh_cast(y->baf, y->cq, (int64_t)T * R, dt, stream));
      float* rkvw = y->cvf;  // [T, 4*HD] = r | k | v | w
      LIN(y->cq, R, l.w2, nullptr, rkvw + 3 * HD, NQ, HD, R, 1);
      TRY(EW, (double)T * HD * 8, b200q_decay_from_logits(rkvw + 3 * HD, NQ, l.w0, HD, T, dt, stream));
      TRY(EW, (double)T * 3 * HD * (es + 4), b200q_act_to_f32(y->proj, NQ, rkvw, NQ, 3 * HD, 0, T, dt, stream));
      float* raw = y->cvf + (int64_t)T * NQ;
      TRY(B200Q_PROF_PREFILL_ATTN, 6.0 * T * H * (double)d.dim * d.dim,
          b200q_decay_attn(rkvw, NQ, 0, HD, 2 * HD, nullptr, rkvw + 3 * HD, NQ, l.bonus, y->state + l.state_off,
                           y->state_slot_floats, b->seq_desc, b->n_rows, H, d.dim, d.dim, raw, stream));
      TRY(EW, (double)T * HD * (4 + 2 * es),
          b200q_gated_rmsnorm(raw, HD, d.dim, l.out_norm, (uint8_t*)y->proj + (size_t)3 * HD * es, NQ, 1, c.rms_eps,
                              y->attn, T, dt, stream));
      LIN(y->attn, HD, l.o, nullptr, outp, W, W, HD, 0);
    } else {  // B200Q_MIXER_WINDOW_ATTN
      const int G = d.kv_heads, GD = G * d.dim, GV = G * d.vdim, NP = (int)window_proj_rows(d);
      const bool own = d.kv_from < 0;
      const int n_kv = own ? GD + GV : 0;
      uint8_t* cache = m->kv + m->num_blocks * l.cache_block_off;  // a borrowing layer's offset is the lender's
      // [q | k | v (own keys and values) | gate number per head (not bare) | zero rows]; biases join in the next step
      LIN(y->h1, W, l.proj, nullptr, y->proj, NP, NP, W, 0);
      if (!d.bare && d.rot_factor == 0.0)
        TRY(EW, (double)T * ((HD + 2 * GD + 2 * GV) * es + HD * 4),
            b200q_window_attn_prep(y->proj, NP, H, G, d.dim, d.vdim, d.rot_dims, l.freq, b->positions, b->slot_mapping,
                                   l.temp, d.attn_scale, y->qa, cache, T, dt, stream));
      else
        TRY(EW, (double)T * ((HD + 2 * n_kv) * es + HD * 4),
            b200q_window_attn_prep_ex(y->proj, NP, 0, own ? HD : -1, HD + GD, d.proj_bias ? l.proj_b : nullptr, H, G,
                                      d.dim, d.vdim, d.qk_norm, l.q_norm, l.kv_norm, c.rms_eps, d.rot_dims, l.freq, l.mag,
                                      b->positions, b->slot_mapping, d.bare ? nullptr : l.temp, d.attn_scale,
                                      d.q_temp_coef, d.q_temp_every, y->qa, cache, T, dt, stream));
      TRY(B200Q_PROF_DECODE_ATTN, (double)b->sum_ctx_dec * (GD + GV) * es,
          b200q_window_attn_ex(y->qa, cache, b->block_table, b->bt_stride, b->row_seq, b->positions, b->seq_desc,
                               b->n_rows, T, H, G, d.dim, d.vdim, c.block_size, d.window, d.keep_first, d.softcap,
                               d.bare ? nullptr : (uint8_t*)y->proj + (size_t)(HD + n_kv) * es, NP, y->attn, dt, stream));
      LIN(y->attn, HV, l.o, nullptr, outp, W, W, HV, 0);  // the output bias, if any, joins in the layer's sum
    }
    return B200Q_OK;
  };

  // ---- the mixers: read y->h1 [T, W] (model dtype), write y->mix [T, W] ----
  auto run_mixer = [&](const b200q_layered_layer& l) -> int {
    const b200q_layer_desc& d = l.d;
    if (d.mixer == B200Q_MIXER_LIGHTNING || d.mixer == B200Q_MIXER_DECAY_MIX || d.mixer == B200Q_MIXER_WINDOW_ATTN)
      return run_sequence_mixer(l, y->mix);
    if (d.mixer == B200Q_MIXER_LATENT_ATTN) {
      const int R = d.kv_rank, P = d.rot_dim, RP = R + P, H = d.heads, QD = d.dim + P;
      const bool own = d.kv_from < 0, full = d.q_rank == 0;
      uint8_t* cache = m->kv + m->num_blocks * l.cache_block_off;
      const void* q = y->q;   // the heads' queries [unrotated | rotated], rows of stride ldq
      int ldq = H * QD;
      const void* gate = nullptr;  // one gate number per head, rows of stride ldq
      if (full) {
        // full-rank queries: one projection of the layer's input gives [q | latent | shared rotated key | gates]
        const int nd = (int)latent_full_rows(d);
        LIN(y->h1, W, l.down, nullptr, y->proj, nd, nd, W, 0);
        TRY(EW, (double)T * 2 * RP * es,
            b200q_latent_prep_ex((uint8_t*)y->proj + (size_t)H * QD * es, nd, 0, R, P, d.rot_dims, l.freq, l.mag,
                                 b->positions, b->slot_mapping, nullptr, l.kv_norm, nullptr, cache, 1, T, c.rms_eps, dt,
                                 stream));
        q = y->proj;
        ldq = nd;
        gate = (uint8_t*)y->proj + (size_t)(H * QD + RP) * es;
      } else {
        const int nd = d.q_rank + (own ? RP : 0);
        LIN(y->h1, W, l.down, nullptr, y->proj, nd, nd, W, 0);
        TRY(EW, (double)T * (nd + d.q_rank + RP) * es,
            b200q_latent_prep_ex(y->proj, nd, d.q_rank, R, P, d.rot_dims, l.freq, l.mag, b->positions, b->slot_mapping,
                                 l.q_norm, l.kv_norm, y->cq, cache, own ? 1 : 0, T, c.rms_eps, dt, stream));
        LIN(y->cq, d.q_rank, l.uq, nullptr, y->q, H * QD, H * QD, d.q_rank, 0);
      }
      TRY(EW, (double)T * H * P * (es + 4),
          b200q_rope_pairs_q_ex(q, ldq, H, d.dim, P, d.rot_dims, l.freq, l.mag, b->positions, y->qa, R, T, dt, stream));
      // the unrotated query of every head, carried into the latent space: qa[t,h,:R] = W_uk[h]^T q[t,h,:dim]
      if (d.dim > 0)
        TRY(B200Q_PROF_GEMM, 2.0 * T * H * (double)R * d.dim,
            b200q_linear_batched(q, ldq, QD, l.uk_t, (long long)R * d.dim, y->qa, H * RP, RP, T, R, d.dim, H, dt, 1,
                                 stream));
      else
        B200Q_CUDA(cudaMemsetAsync(y->qa, 0, (size_t)T * H * RP * 4, cst));
      TRY(B200Q_PROF_DECODE_ATTN, 0.0,
          b200q_latent_attn_ex(y->qa, cache, b->block_table, b->bt_stride, b->row_seq, b->positions, T, H, R, P,
                               c.block_size, d.window, d.attn_scale, gate, ldq, y->olat, dt, stream));
      TRY(B200Q_PROF_GEMM, 2.0 * T * H * (double)R * d.vdim,
          b200q_linear_batched(y->olat, H * R, R, l.uv, (long long)d.vdim * R, y->attn, H * d.vdim, d.vdim, T, d.vdim, R,
                               H, dt, 0, stream));
      LIN(y->attn, H * d.vdim, l.o, nullptr, y->mix, W, W, H * d.vdim, 0);
    } else if (d.mixer == B200Q_MIXER_GENERAL_DELTA) {
      const int HD = d.heads * d.dim, NP = 5 * HD + d.decay_rank;
      LIN(y->h1, W, l.proj, nullptr, y->proj, NP, NP, W, 0);
      TRY(B200Q_PROF_PREFILL_ATTN, 0.0,
          b200q_delta_rule(y->proj, NP, l.w2, l.w0, l.a_bias, l.out_norm, y->state + l.state_off,
                           y->state_slot_floats, b->seq_desc, b->n_rows, d.heads, d.dim, d.decay_rank, c.rms_eps,
                           y->attn, dt, T > b->n_rows ? y->dscr : nullptr /* portions of prompts: three launches */, T,
                           stream));
      LIN(y->attn, HD, l.o, nullptr, y->mix, W, W, HD, 0);
    } else if (d.mixer == B200Q_MIXER_GATED_DELTA) {
      const int H = d.heads, GD = d.kv_heads * d.dim, HV = H * d.vdim, NC = 2 * GD + HV, NP = NC + HV;
      LIN(y->h1, W, l.proj, nullptr, y->proj, NP, NP, W, 0);          // [q | k | v | gate]
      LIN(y->h1, W, l.ba, nullptr, y->baf, 2 * H, 2 * H, W, 1);       // [beta | decay input], fp32
      TRY(EW, (double)T * NC * (es + 4),
          b200q_causal_conv(y->proj, NP, 0, l.conv_w, nullptr, NC, d.conv_taps, 1, 0, y->state + l.conv_off,
                            y->state_slot_floats, b->seq_desc, b->row_seq, b->n_rows, y->cvf, NC, 1, T, dt, stream));
      uint8_t* gate = (uint8_t*)y->proj + (size_t)NC * es;
      TRY(B200Q_PROF_PREFILL_ATTN, 8.0 * b->n_rows * H * (double)d.dim * d.vdim,
          b200q_gated_delta(y->cvf, y->baf, y->cvf + (int64_t)T * NC, gate, NP, l.a_log, l.dt_bias, l.out_norm,
                            y->state + l.state_off, y->state_slot_floats, b->seq_desc, b->n_rows, H, d.kv_heads, d.dim,
                            d.vdim, c.rms_eps, y->attn, T, dt, stream));
      LIN(y->attn, HV, l.o, nullptr, y->mix, W, W, HV, 0);
    } else if (d.mixer == B200Q_MIXER_CHUNK_ATTN) {
      const int H = d.heads, G = d.kv_heads, D = d.dim, HD = H * D, NP = 2 * HD + G * D;
      uint8_t* cache = m->kv + m->num_blocks * l.cache_block_off;
      LIN(y->h1, W, l.proj, nullptr, y->proj, NP, NP, W, 0);          // [q | k | gate]
      TRY(EW, (double)T * ((HD + G * D) * es + HD * 4 + G * D * es),
          b200q_chunk_attn_prep(y->proj, NP, H, G, D, l.q_norm, l.kv_norm, b->slot_mapping, y->qa, cache, T, c.rms_eps, dt,
                                stream));
      uint8_t* gate = (uint8_t*)y->proj + (size_t)(HD + G * D) * es;
      TRY(B200Q_PROF_DECODE_ATTN, (double)b->sum_ctx_dec * G * D * es,
          b200q_chunk_attn_seq(y->qa, cache, b->block_table, b->bt_stride, b->row_seq, b->positions, b->seq_desc,
                               b->n_rows, T, H, G, D, c.block_size, d.chunk, d.attn_scale, d.softcap, l.r1, l.r2, gate, NP,
                               c.rms_eps, y->attn, dt, stream));
      LIN(y->attn, HD, l.o, nullptr, y->mix, W, W, HD, 0);
    } else {  // B200Q_MIXER_SELECTIVE_SCAN
      // the rows of the [dt | B | C] projection are padded with zero rows to a multiple of 64 at load time, so
      // that both small projections take the tensor-core path whenever the other sizes allow it
      const int I = d.inner, N = d.state_dim, R = d.dt_rank, NX = (R + 2 * N + 63) & ~63;
      LIN(y->h1, W, l.proj, nullptr, y->proj, 2 * I, 2 * I, W, 0);    // [x | z]
      TRY(EW, 2.0 * T * I * es,
          b200q_causal_conv(y->proj, 2 * I, 0, l.conv_w, l.conv_b, I, d.conv_taps, 1, 0, y->state + l.conv_off,
                            y->state_slot_floats, b->seq_desc, b->row_seq, b->n_rows, y->xc, I, 0, T, dt, stream));
      LIN(y->xc, I, l.x_proj, nullptr, y->xp, NX, NX, I, 0);          // [dt | B | C]
      LIN(y->xp, NX, l.dt_proj, nullptr, y->dtr, I, I, R, 1);         // step sizes before bias and softplus, fp32
      uint8_t* z = (uint8_t*)y->proj + (size_t)I * es;
      TRY(B200Q_PROF_PREFILL_ATTN, 8.0 * b->n_rows * (double)I * N,
          b200q_selective_scan(y->xc, y->dtr, l.dt_b, y->xp, NX, R, z, 2 * I, l.a_log, l.dvec, y->state + l.state_off,
                               y->state_slot_floats, b->seq_desc, b->n_rows, I, N, y->attn, T, dt, stream));
      LIN(y->attn, I, l.o, nullptr, y->mix, W, W, I, 0);
    }
    return B200Q_OK;
  };

  // ---- sigmoid-routed experts of the post-norm form: read y->h2, leave the pairs' outputs in y->eout ----
  auto run_moe_sigmoid = [&](const b200q_layered_layer& l) -> int {
    const b200q_layer_desc& d = l.d;
    const int E = d.n_experts, K = d.top_k, F = d.ff_dim, P = T * K;
    LIN(y->h2, W, l.router, nullptr, y->rlog, E, E, W, 1);
    TRY(EW, (double)T * E * 4,
        b200q_moe_route_ex(y->rlog, T, E, K, 1, y->idx, y->wts, y->group_off, y->perm_tok, y->pair_pos, y->tile_tab,
                           y->n_tiles, stream));
    // every (token, choice) pair's input, scaled by its routing weight, in expert order
    TRY(EW, 2.0 * P * W * es, b200q_scatter_scaled_rows(y->h2, y->pair_pos, y->wts, K, y->esrc, T, W, dt, stream));
    TRY(B200Q_PROF_GEMM, 2.0 * P * 2.0 * F * W,
        b200q_linear_grouped(y->esrc, W, nullptr, l.experts_gate_up, 2LL * F * W, y->egu, 2 * F, y->group_off, E, P,
                             2 * F, W, dt, y->tile_tab, y->n_tiles, stream));
    TRY(EW, 3.0 * P * F * es, b200q_silu_glu(y->egu, y->eact, P, F, dt, stream));
    TRY(B200Q_PROF_GEMM, 2.0 * P * (double)F * W,
        b200q_linear_grouped(y->eact, F, nullptr, l.experts_down, (long long)W * F, y->eout, W, y->group_off, E, P, W, F,
                             dt, y->tile_tab, y->n_tiles, stream));
    return B200Q_OK;
  };

  bool keep_x0 = false;
  for (const auto& l : y->layers) keep_x0 = keep_x0 || l.d.inject;
  if (keep_x0) TRY(EW, 8.0 * T * W, b200q_copy_f32(y->x, y->x0, (int64_t)T * W, stream));

  for (int li = 0; li < c.n_layers; ++li) {
    const b200q_layered_layer& l = y->layers[li];
    const b200q_layer_desc& d = l.d;
    const bool has_ff = d.ff != B200Q_FF_NONE;
    if (pre) {
      // (x <- W_in [x; x0]);  x <- x + a mixer(h) (+ b side(h)), h = shift(norm1 x);  x <- x + ff(norm2 x)
      if (d.inject) {
        TRY(EW, (double)T * W * (8 + 2 * es), b200q_concat_cast(y->x, y->x0, y->cat, T, W, dt, stream));
        LIN(y->cat, 2 * W, l.inject, nullptr, y->x, W, W, 2 * W, 1);
      }
      const bool side = !l.side.empty();
      const bool want_f32 = d.mixer == B200Q_MIXER_DECAY_MIX || (side && l.side[0].d.mixer == B200Q_MIXER_DECAY_MIX);
      TRY(EW, (double)T * W * (8 + es),
          b200q_rmsnorm_shift(y->x, nullptr, l.norm1, c.token_shift ? l.shift : nullptr, y->state + l.shift_off,
                              y->state_slot_floats, b->seq_desc, b->row_seq, b->n_rows, y->carry, y->h1,
                              want_f32 ? y->hf : nullptr, T, W, c.rms_eps, dt, stream));
      if (c.token_shift && T > b->n_rows)
        TRY(EW, 8.0 * b->n_rows * W,
            b200q_store_carry(y->carry, 0, y->state + l.shift_off, y->state_slot_floats, b->seq_desc, b->n_rows, W, 1,
                              stream));
      if ((rc = run_mixer(l))) return rc;
      if (side && (rc = run_sequence_mixer(l.side[0], y->mix2))) return rc;
      const float sa = d.mix_scale != 0.f ? d.mix_scale : 1.f;
      const float sb = side && l.side[0].d.mix_scale != 0.f ? l.side[0].d.mix_scale : 1.f;
      if (!has_ff)
        TRY(EW, (double)T * W * (8 + (side ? 2 : 1) * es),
            b200q_residual_add(y->x, y->mix, sa, side ? y->mix2 : nullptr, sb, T, W, dt, stream));
      if (has_ff) {
        // the sum that closes the mixer and the norm that opens the feed-forward, one pass
        TRY(EW, (double)T * W * (8 + (side ? 3 : 2) * es),
            b200q_residual_add_rmsnorm(y->x, y->mix, sa, side ? y->mix2 : nullptr, sb, l.norm2, y->h2, T, W, c.rms_eps, dt,
                                       stream));
        if (d.ff == B200Q_FF_RELU2) {
          const int F = d.ff_dim;
          LIN(y->h2, W, l.up, nullptr, y->ffh, F, F, W, 0);
          TRY(EW, 2.0 * T * F * es, b200q_relu2(y->ffh, (int64_t)T * F, dt, stream));
          LIN(y->ffh, F, l.ff_down, nullptr, y->ffo, W, W, F, 0);
          TRY(EW, (double)T * W * (8 + es), b200q_residual_add(y->x, y->ffo, 1.f, nullptr, 0.f, T, W, dt, stream));
        } else {
          B200Q_CHECK_ARG(d.ff == B200Q_FF_MOE_GROUPED, "layer %d: feed-forward %d is not built for the pre-norm form", li,
                          d.ff);
          const int E = d.n_experts, ET = E + d.n_identity, K = d.top_k, F = d.ff_dim, P = T * K;
          LIN(y->h2, W, l.router, nullptr, y->rlog, ET, ET, W, 1);
          TRY(EW, (double)T * ET * 4,
              b200q_moe_route_grouped(y->rlog, l.router_bias, T, ET, E, K, d.n_groups, d.keep_groups, y->idx, y->wts,
                                      y->group_off, y->perm_tok, y->pair_pos, y->tile_tab, y->n_tiles, stream));
          if (E > 0) {
            const bool sorted = dt == B200Q_DTYPE_BF16 && W % 8 == 0;
            if (sorted) TRY(EW, 2.0 * P * W * es, b200q_gather_rows(y->h2, y->perm_tok, y->esrc, P, W, stream));
            TRY(B200Q_PROF_GEMM, 2.0 * P * (double)F * W,
                b200q_linear_grouped(sorted ? y->esrc : y->h2, W, sorted ? nullptr : y->perm_tok, l.experts_up,
                                     (long long)F * W, y->egu, F, y->group_off, E, P, F, W, dt, y->tile_tab, y->n_tiles,
                                     stream));
            TRY(EW, 2.0 * P * F * es, b200q_relu2(y->egu, (int64_t)P * F, dt, stream));
            TRY(B200Q_PROF_GEMM, 2.0 * P * (double)F * W,
                b200q_linear_grouped(y->egu, F, nullptr, l.experts_down, (long long)W * F, y->eout, W, y->group_off, E, P, W,
                                     F, dt, y->tile_tab, y->n_tiles, stream));
          }
          TRY(EW, (double)T * W * (8 + (1 + K) * es),
              b200q_residual_add_routed(y->x, y->eout, y->pair_pos, y->idx, y->wts, K, E, y->h2, T, W, dt, stream));
        }
      }
      if (y->tap) TRY(EW, 8.0 * T * W, b200q_copy_f32(y->x, y->tap + (int64_t)li * T * W, (int64_t)T * W, stream));
      continue;
    }
    if (sandwich) {
      // x <- x + m n1b(mixer(n1 x) + o_b);  x <- x + m n2b(ff(n2 x));  x <- x + m rms(P (gelu(G x) * e)) s.
      // Every sum also writes what reads the new x next: the following norm's output, or x itself in the model dtype.
      const int NK = c.norm_kind, D = c.side_dim;
      const bool last = li + 1 == c.n_layers;
      const int next_kind = last ? B200Q_NORM_NONE : NK;
      const float* next_w = last ? nullptr : y->layers[li + 1].norm1;
      if (li == 0)
        TRY(EW, (double)T * W * (4 + es), b200q_row_norm(y->x, nullptr, NK, l.norm1, y->h1, T, W, c.rms_eps, dt, stream));
      if ((rc = run_mixer(l))) return rc;
      const float* o_b = d.mixer == B200Q_MIXER_WINDOW_ATTN && d.proj_bias ? l.o_b : nullptr;
      const int after_kind = D > 0 ? B200Q_NORM_CAST : next_kind;  // what follows the layer's last sublayer
      const float* after_w = D > 0 ? nullptr : next_w;
      if (has_ff) {
        const int F = d.ff_dim;
        TRY(EW, (double)T * W * (8 + 2 * es),
            b200q_sandwich_add(y->x, y->mix, o_b, NK, l.norm1b, mult, NK, l.norm2, y->h2, T, W, c.rms_eps, dt, stream));
        // (steps of few tokens keep the plain product: its 128-wide tiles put twice as many SMs on the weight stream)
        if (l.gate_up_il && dt == B200Q_DTYPE_BF16 && W % 64 == 0 && T >= 512 &&
            ((reinterpret_cast<uintptr_t>(y->h2) | reinterpret_cast<uintptr_t>(l.gate_up) |
              reinterpret_cast<uintptr_t>(y->ffa)) & 15) == 0) {
          // the gated unit in the product's epilogue: the [T, 2F] activations are never written
          TRY(B200Q_PROF_GEMM, 2.0 * T * 2.0 * F * W, b200q_gemm_geglu_bf16(y->h2, l.gate_up, y->ffa, T, 2 * F, W, stream));
        } else {
          LIN(y->h2, W, l.gate_up, nullptr, y->ffh, 2 * F, 2 * F, W, 0);  // [gate | up], or blocks of 128 of each
          TRY(EW, 3.0 * T * F * es, b200q_gelu_glu_ex(y->ffh, y->ffa, T, F, l.gate_up_il ? 128 : 0, dt, stream));
        }
        LIN(y->ffa, F, l.ff_down, nullptr, y->ffo, W, W, F, 0);
        TRY(EW, (double)T * W * (8 + 2 * es),
            b200q_sandwich_add(y->x, y->ffo, nullptr, NK, l.norm2b, mult, after_kind, after_w, y->h1, T, W, c.rms_eps, dt,
                               stream));
      } else {
        TRY(EW, (double)T * W * (8 + 2 * es),
            b200q_sandwich_add(y->x, y->mix, o_b, NK, l.norm1b, mult, after_kind, after_w, y->h1, T, W, c.rms_eps, dt,
                               stream));
      }
      if (D > 0) {  // the per-layer token input reads x (in y->h1, model dtype) and the layer's columns of the table
        LIN(y->h1, W, l.tok_gate, nullptr, y->tg, D, D, W, 0);
        TRY(EW, (double)T * D * 3 * es,
            b200q_token_side_gate(y->tg, D, b->token_ids, b->prev_out_ids, y->tok_embed, (int)y->tok_cols, li * D, y->ta,
                                  T, D, dt, stream));
        LIN(y->ta, D, l.tok_proj, nullptr, y->ffo, W, W, D, 0);
        TRY(EW, (double)T * W * (8 + 2 * es),
            b200q_sandwich_add(y->x, y->ffo, nullptr, B200Q_NORM_RMS, l.tok_norm, mult, next_kind, next_w, y->h1, T, W,
                               c.rms_eps, dt, stream));
      }
      if (y->tap) TRY(EW, 8.0 * T * W, b200q_copy_f32(y->x, y->tap + (int64_t)li * T * W, (int64_t)T * W, stream));
      continue;
    }
    if (post) {
      // x <- norm1(alpha x + ls1 * mixer(x + conv1 x));  x <- norm2(alpha x + ls2 * ff(x + conv2 x))
      for (int sub = 0; sub < (has_ff ? 2 : 1); ++sub) {
        void* hin = sub ? y->h2 : y->h1;
        if (c.input_taps > 0)
          TRY(EW, (double)T * W * (4 + es),
              b200q_causal_conv(y->x, W, 1, sub ? l.canon2 : l.canon1, nullptr, W, c.input_taps, 0, 1,
                                y->state + (sub ? l.canon2_off : l.canon1_off), y->state_slot_floats, b->seq_desc,
                                b->row_seq, b->n_rows, hin, W, 0, T, dt, stream));
        else if (dt == B200Q_DTYPE_F32)
          TRY(EW, 8.0 * T * W, b200q_copy_f32(y->x, (float*)hin, (int64_t)T * W, stream));
        else
          TRY(EW, 6.0 * T * W, b200q_f32_to_bf16(y->x, hin, (int64_t)T * W, stream));
        if (sub == 0) {
          if ((rc = run_mixer(l))) return rc;
          TRY(EW, (double)T * W * (8 + es),
              b200q_group_rmsnorm(y->x, nullptr, y->mix, nullptr, 0, l.ls1, c.residual_alpha, l.norm1, groups, c.rms_eps,
                                  y->x, nullptr, T, W, dt, stream));
        } else {
          B200Q_CHECK_ARG(d.ff == B200Q_FF_MOE_SIGMOID, "layer %d: feed-forward %d is not built for the post-norm form",
                          li, d.ff);
          if ((rc = run_moe_sigmoid(l))) return rc;
          TRY(EW, (double)T * W * (8 + d.top_k * es),
              b200q_group_rmsnorm(y->x, nullptr, y->eout, y->pair_pos, d.top_k, l.ls2, c.residual_alpha, l.norm2, groups,
                                  c.rms_eps, y->x, nullptr, T, W, dt, stream));
        }
      }
      if (y->tap) TRY(EW, 8.0 * T * W, b200q_copy_f32(y->x, y->tap + (int64_t)li * T * W, (int64_t)T * W, stream));
      continue;
    }
    TRY(EW, (double)T * W * (4 + 2 * es),
        b200q_centered_rmsnorm(y->x, nullptr, l.norm1, l.norm2, y->h1, has_ff ? y->h2 : nullptr, T, W, c.rms_eps, dt,
                               stream));
    if ((rc = run_mixer(l))) return rc;
    // ---- feed-forward and the layer's sum ----
    if (d.ff == B200Q_FF_POLYNORM) {
      LIN(y->h2, W, l.up, nullptr, y->ffh, d.ff_dim, d.ff_dim, W, 0);
      TRY(EW, 2.0 * T * d.ff_dim * es, b200q_polynorm(y->ffh, l.act, y->ffa, T, d.ff_dim, c.rms_eps, dt, stream));
      LIN(y->ffa, d.ff_dim, l.ff_down, nullptr, y->ffo, W, W, d.ff_dim, 0);
      TRY(EW, (double)T * W * (8 + 2 * es),
          b200q_layer_sum(y->x, y->mix, y->ffo, nullptr, nullptr, nullptr, 0, nullptr, nullptr, T, W, dt, stream));
    } else if (d.ff == B200Q_FF_MOE) {
      const int E = d.n_experts, K = d.top_k, F = d.ff_dim, P = T * K;
      LIN(y->h2, W, l.router, l.router_bias, y->rlog, E, E, W, 1);
      TRY(EW, (double)T * E * 4,
          b200q_moe_route(y->rlog, T, E, K, y->idx, y->wts, y->group_off, y->perm_tok, y->pair_pos, y->tile_tab,
                          y->n_tiles, stream));
      // bf16: the pairs' inputs are gathered into expert order once, so that each expert's rows are one
      // dense block the tensor-core GEMM can fetch by TMA; fp32 reads them through perm_tok
      const bool sorted = dt == B200Q_DTYPE_BF16 && W % 8 == 0;
      if (sorted) TRY(EW, 2.0 * P * W * es, b200q_gather_rows(y->h2, y->perm_tok, y->esrc, P, W, stream));
      TRY(B200Q_PROF_GEMM, 2.0 * P * 2.0 * F * W,
          b200q_linear_grouped(sorted ? y->esrc : y->h2, W, sorted ? nullptr : y->perm_tok, l.experts_gate_up,
                               2LL * F * W, y->egu, 2 * F, y->group_off, E, P, 2 * F, W, dt, y->tile_tab, y->n_tiles,
                               stream));
      TRY(EW, 3.0 * P * F * es, b200q_clamped_glu(y->egu, y->eact, P, F, d.expert_limit, dt, stream));
      TRY(B200Q_PROF_GEMM, 2.0 * P * (double)F * W,
          b200q_linear_grouped(y->eact, F, nullptr, l.experts_down, (long long)W * F, y->eout, W, y->group_off, E, P, W,
                               F, dt, y->tile_tab, y->n_tiles, stream));
      const bool sh = d.shared_dim > 0;
      if (sh) {
        const int FS = d.shared_dim;
        LIN(y->h2, W, l.shared_gate_up, nullptr, y->ffh, 2 * FS, 2 * FS, W, 0);
        TRY(EW, 3.0 * T * FS * es, b200q_clamped_glu(y->ffh, y->ffa, T, FS, d.shared_limit, dt, stream));
        LIN(y->ffa, FS, l.shared_down, nullptr, y->shout, W, W, FS, 0);
        LIN(y->h2, W, l.shared_gate, nullptr, y->sgate, 1, 1, W, 1);
      }
      TRY(EW, (double)T * W * (8 + (2 + K) * es),
          b200q_layer_sum(y->x, y->mix, nullptr, y->eout, y->pair_pos, y->wts, K, sh ? y->shout : nullptr,
                          sh ? y->sgate : nullptr, T, W, dt, stream));
    } else {
      TRY(EW, (double)T * W * (8 + es),
          b200q_layer_sum(y->x, y->mix, nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, T, W, dt, stream));
    }
    if (y->tap) TRY(EW, 8.0 * T * W, b200q_copy_f32(y->x, y->tap + (int64_t)li * T * W, (int64_t)T * W, stream));
  }
  if (b->n_sample > 0) {
    const int n = b->n_sample;
    if (sandwich)
      TRY(EW, (double)n * W * (4 + es),
          b200q_row_norm(y->x, b->sample_rows, c.norm_kind, (const float*)m->final_norm, y->sel, n, W, c.rms_eps, dt,
                         stream));
    else if (post)
      TRY(EW, (double)n * W * (4 + es),
          b200q_group_rmsnorm(y->x, b->sample_rows, nullptr, nullptr, 0, nullptr, 1.f, (const float*)m->final_norm, groups,
                              c.rms_eps, nullptr, y->sel, n, W, dt, stream));
    else if (pre)
      TRY(EW, (double)n * W * (4 + es),
          b200q_rmsnorm_shift(y->x, b->sample_rows, (const float*)m->final_norm, nullptr, nullptr, 0, nullptr, nullptr, 0,
                              nullptr, y->sel, nullptr, n, W, c.rms_eps, dt, stream));
    else
      TRY(EW, (double)n * W * (4 + es),
          b200q_centered_rmsnorm(y->x, b->sample_rows, (const float*)m->final_norm, nullptr, y->sel, nullptr, n, W,
                                 c.rms_eps, dt, stream));
    TRY(B200Q_PROF_GEMM, 2.0 * n * (double)c.vocab * W,
        b200q_linear(y->sel, W, m->lm_head, nullptr, y->logits, c.vocab, n, c.vocab, W, dt, 1, stream));
    if (c.logit_scale > 0.f && c.logit_scale != 1.f)
      TRY(EW, 8.0 * n * c.vocab, b200q_scale_f32(y->logits, (int64_t)n * c.vocab, c.logit_scale, stream));
    if (c.logit_softcap > 0.f)
      TRY(EW, 8.0 * n * c.vocab, b200q_softcap_f32(y->logits, (int64_t)n * c.vocab, c.logit_softcap, stream));
    if (!b->no_sampling) {
      if (b->sample_params) {
        TRY(EW, 6.0 * n * c.vocab, b200q_f32_to_bf16(y->logits, y->logits_bf16, (int64_t)n * c.vocab, stream));
        TRY(EW, 2.0 * n * c.vocab, b200q_sample_bf16(y->logits_bf16, b->sample_params, b->out_ids, n, c.vocab, stream));
      } else {
        TRY(EW, 4.0 * n * c.vocab, b200q_argmax_f32(y->logits, b->out_ids, n, c.vocab, stream));
      }
    }
  }
#undef LIN
#undef TRY
  return B200Q_OK;
}

}  // namespace b200q

extern "C" {

int b200q_model_create_layered(const b200q_model_config* cfg, const b200q_layer_desc* layers, b200q_model_t* out) {
  return layered_create(cfg, layers, out);
}

int64_t b200q_model_kv_block_bytes(b200q_model_t m) { return m && m->lay ? m->lay->kv_block_bytes : -1; }

int64_t b200q_model_state_slot_bytes(b200q_model_t m) { return m && m->lay ? m->lay->state_slot_floats * 4 : -1; }

int b200q_model_bind_state(b200q_model_t m, void* p, int64_t n_slots) {
  B200Q_CHECK_ARG(m && m->lay && p && n_slots > 0, "bind_state: bad argument");
  B200Q_CHECK_ARG((reinterpret_cast<uintptr_t>(p) & 15) == 0, "recurrent state must be 16-byte aligned");
  m->lay->state = (float*)p;
  m->lay->n_slots = n_slots;
  return B200Q_OK;
}

const float* b200q_model_logits_f32_ptr(b200q_model_t m) { return m && m->lay ? m->lay->logits : nullptr; }

int b200q_model_set_layer_tap(b200q_model_t m, float* p) {
  B200Q_CHECK_ARG(m && m->lay, "set_layer_tap: not a layered model");
  m->lay->tap = p;
  return B200Q_OK;
}

}  // extern "C"
