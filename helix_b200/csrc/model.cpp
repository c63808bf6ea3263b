#include "model.h"

#include <math.h>
#include <string.h>

#include <algorithm>

namespace hb {

namespace {
constexpr size_t kAlign = 256;
size_t up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

// Walks the tensors of a model in arena order. `visit(name, rows, cols, mode, group, kind)`;
// fused tensors are visited once per checkpoint tensor that lands in them.
struct Carver {
  uint8_t* base;
  size_t off = 0;
  bf16* take(size_t elems) {
    bf16* p = base ? reinterpret_cast<bf16*>(base + off) : nullptr;
    off += up(elems * sizeof(bf16));
    return p;
  }
};
}  // namespace

std::string validate_desc(const hb_model_desc& d) {
  if (d.arch != HB_ARCH_LLAMA && d.arch != HB_ARCH_BERT) return "unknown arch";
  if (d.hidden <= 0 || d.layers <= 0 || d.heads <= 0 || d.ffn <= 0 || d.vocab <= 0) return "non-positive dimension";
  if (d.head_dim != 64 && d.head_dim != 128) return "head_dim must be 64 or 128";
  if (d.hidden % 64) return "hidden must be a multiple of 64";
  if (d.hidden > 4096 * 4) return "hidden too large";
  if (d.arch == HB_ARCH_LLAMA) {
    if (d.kv_heads <= 0 || d.heads % d.kv_heads) return "heads must be a multiple of kv_heads";
    const int g = d.heads / d.kv_heads;
    if (g != 1 && g != 2 && g != 3 && g != 4 && g != 6 && g != 8) return "GQA group (heads/kv_heads) must be 1, 2, 3, 4, 6 or 8";
    if (d.ffn % 128) return "ffn must be a multiple of 128 (SwiGLU tile packing)";
    if (d.rope_theta <= 0.f) return "rope_theta must be positive";
    if (d.vocab % 4) return "vocab must be a multiple of 4 (16-byte rows of the fp32 logits)";
    if (d.hidden > 8192) return "hidden > 8192 unsupported (decode residual+RMSNorm register budget)";
  } else {
    if (d.heads * d.head_dim != d.hidden) return "BERT needs heads*head_dim == hidden";
    if (d.hidden > 4096) return "BERT hidden > 4096 unsupported (LayerNorm register budget)";
    if (d.ffn % 64) return "ffn must be a multiple of 64";
    if (d.max_pos <= 0) return "max_pos required";
  }
  return "";
}

static size_t carve(Model* m, const hb_model_desc& d, uint8_t* base) {
  Carver c{base};
  auto put = [&](const std::string& name, bf16* dst, size_t rows, size_t cols, int mode = 0, bool gain = false,
                 bool bias = false) {
    if (!m) return;
    Placement p;
    p.dst = dst;
    p.rows = rows;
    p.cols = cols;
    p.mode = mode;
    p.is_norm_gain = gain;
    p.is_bias = bias;
    m->placements[name] = p;
  };
  const size_t H = d.hidden, F = d.ffn, V = d.vocab, D = d.head_dim;
  if (d.arch == HB_ARCH_LLAMA) {
    const size_t QD = (size_t)d.heads * D, KD = (size_t)d.kv_heads * D;
    bf16* embed = c.take(V * H);
    put("model.embed_tokens.weight", embed, V, H);
    if (m) {
      m->embed = embed;
      m->ll.resize(d.layers);
    }
    for (int i = 0; i < d.layers; ++i) {
      const std::string p = "model.layers." + std::to_string(i) + ".";
      LlamaLayerW w;
      w.attn_norm = c.take(H);
      w.wqkv = c.take((QD + 2 * KD) * H);
      if (d.qkv_bias) w.bqkv = c.take(QD + 2 * KD);
      w.wo = c.take(H * QD);
      w.mlp_norm = c.take(H);
      w.wgu = c.take(2 * F * H);
      w.wdown = c.take(H * F);
      put(p + "input_layernorm.weight", w.attn_norm, H, 1, 0, true);
      put(p + "self_attn.q_proj.weight", w.wqkv, QD, H);
      put(p + "self_attn.k_proj.weight", w.wqkv ? w.wqkv + QD * H : nullptr, KD, H);
      put(p + "self_attn.v_proj.weight", w.wqkv ? w.wqkv + (QD + KD) * H : nullptr, KD, H);
      if (d.qkv_bias) {
        put(p + "self_attn.q_proj.bias", w.bqkv, QD, 1, 0, false, true);
        put(p + "self_attn.k_proj.bias", w.bqkv ? w.bqkv + QD : nullptr, KD, 1, 0, false, true);
        put(p + "self_attn.v_proj.bias", w.bqkv ? w.bqkv + QD + KD : nullptr, KD, 1, 0, false, true);
      }
      put(p + "self_attn.o_proj.weight", w.wo, H, QD);
      put(p + "post_attention_layernorm.weight", w.mlp_norm, H, 1, 0, true);
      put(p + "mlp.gate_proj.weight", w.wgu, F, H, 1);
      put(p + "mlp.up_proj.weight", w.wgu, F, H, 2);
      put(p + "mlp.down_proj.weight", w.wdown, H, F);
      if (m) m->ll[i] = w;
    }
    bf16* fn = c.take(H);
    put("model.norm.weight", fn, H, 1, 0, true);
    bf16* head = embed;
    if (!d.tie_embeddings) {
      head = c.take(V * H);
      put("lm_head.weight", head, V, H);
    }
    if (m) {
      m->final_norm = fn;
      m->lm_head = head;
    }
  } else {
    const size_t P = d.max_pos, TV = d.type_vocab > 0 ? d.type_vocab : 2;
    bf16* word = c.take(V * H);
    bf16* pos = c.take(P * H);
    bf16* type = c.take(TV * H);
    bf16* g = c.take(H);
    bf16* b = c.take(H);
    put("embeddings.word_embeddings.weight", word, V, H);
    put("embeddings.position_embeddings.weight", pos, P, H);
    put("embeddings.token_type_embeddings.weight", type, TV, H);
    put("embeddings.LayerNorm.weight", g, H, 1, 0, true);
    put("embeddings.LayerNorm.bias", b, H, 1, 0, false, true);
    if (m) {
      m->word = word;
      m->pos = pos;
      m->type = type;
      m->emb_ln_g = g;
      m->emb_ln_b = b;
      m->bl.resize(d.layers);
    }
    for (int i = 0; i < d.layers; ++i) {
      const std::string p = "encoder.layer." + std::to_string(i) + ".";
      BertLayerW w;
      w.wqkv = c.take(3 * H * H);
      w.bqkv = c.take(3 * H);
      w.wo = c.take(H * H);
      w.bo = c.take(H);
      w.ln1_g = c.take(H);
      w.ln1_b = c.take(H);
      w.w1 = c.take(F * H);
      w.b1 = c.take(F);
      w.w2 = c.take(H * F);
      w.b2 = c.take(H);
      w.ln2_g = c.take(H);
      w.ln2_b = c.take(H);
      put(p + "attention.self.query.weight", w.wqkv, H, H);
      put(p + "attention.self.key.weight", w.wqkv ? w.wqkv + H * H : nullptr, H, H);
      put(p + "attention.self.value.weight", w.wqkv ? w.wqkv + 2 * H * H : nullptr, H, H);
      put(p + "attention.self.query.bias", w.bqkv, H, 1, 0, false, true);
      put(p + "attention.self.key.bias", w.bqkv ? w.bqkv + H : nullptr, H, 1, 0, false, true);
      put(p + "attention.self.value.bias", w.bqkv ? w.bqkv + 2 * H : nullptr, H, 1, 0, false, true);
      put(p + "attention.output.dense.weight", w.wo, H, H);
      put(p + "attention.output.dense.bias", w.bo, H, 1, 0, false, true);
      put(p + "attention.output.LayerNorm.weight", w.ln1_g, H, 1, 0, true);
      put(p + "attention.output.LayerNorm.bias", w.ln1_b, H, 1, 0, false, true);
      put(p + "intermediate.dense.weight", w.w1, F, H);
      put(p + "intermediate.dense.bias", w.b1, F, 1, 0, false, true);
      put(p + "output.dense.weight", w.w2, H, F);
      put(p + "output.dense.bias", w.b2, H, 1, 0, false, true);
      put(p + "output.LayerNorm.weight", w.ln2_g, H, 1, 0, true);
      put(p + "output.LayerNorm.bias", w.ln2_b, H, 1, 0, false, true);
      if (m) m->bl[i] = w;
    }
  }
  return c.off;
}

// ------------------------------------------------------------------ layer-list decoders
std::string validate_stack(const hb_stack_desc& d, const hb_layer_desc* L) {
  if (!L) return "no layer list";
  if (d.width <= 0 || d.vocab <= 0 || d.n_layers <= 0) return "non-positive dimension";
  if (!(d.norm_eps > 0.f)) return "norm_eps must be positive";
  for (int i = 0; i < d.n_layers; ++i) {
    const hb_layer_desc& l = L[i];
    const std::string at = " (layer " + std::to_string(i) + ")";
    if (l.heads <= 0 || l.dim <= 0 || l.vdim <= 0) return "non-positive head size" + at;
    if (l.mixer == HB_MIXER_GLA) {
      if (l.dim > 256) return "GLA key channels per head > 256 unsupported (one warp per 16 channels, 512 threads per block)" + at;
      if (!(l.tau > 0.f) || l.decay_rank <= 0) return "GLA needs tau > 0 and a decay rank" + at;
    } else if (l.mixer == HB_MIXER_LATENT) {
      if (l.q_rank <= 0 || l.kv_rank <= 0 || l.rot_dim < 0 || l.window <= 0) return "latent attention sizes" + at;
      if (l.rope_dims < 0 || l.rope_dims % 2 || l.rope_dims > l.rot_dim) return "rope_dims must be even and <= rot_dim" + at;
      if (l.rope_dims > 0 && !(l.rope_base > 0.f)) return "rope_base must be positive" + at;
      if ((size_t)(4 * (l.kv_rank + l.rot_dim + 4) + 5 * l.window + 8 * 1024 + 136) * 4 > 200 * 1024) return "window + latent row exceed the attention kernel's shared memory" + at;
      if (l.kv_from >= 0) {
        if (l.kv_from >= i) return "kv_from must name an earlier layer" + at;
        const hb_layer_desc& s = L[l.kv_from];
        if (s.mixer != HB_MIXER_LATENT || s.kv_from >= 0) return "kv_from must name a latent layer with its own cache rows" + at;
        if (s.kv_rank != l.kv_rank || s.rot_dim != l.rot_dim) return "kv_from layer has a different latent row" + at;
      }
    } else if (l.mixer == HB_MIXER_GQA) {
      if (l.kv_heads <= 0 || l.heads % l.kv_heads) return "heads must be a multiple of kv_heads" + at;
      if ((l.attn_flags & HB_ATTN_V_IS_K) && l.vdim != l.dim) return "values that are the keys need vdim == dim" + at;
      if (l.rope_dims < 0 || l.rope_dims % 2 || l.rope_dims > l.dim) return "rope_dims must be even and <= dim" + at;
      if (l.rope_dims > 0 && !(l.rope_base > 0.f)) return "rope_base must be positive" + at;
      if (l.rope_pairing != 0 && l.rope_pairing != 1) return "unknown rope_pairing" + at;
      if (l.rope_factor > 0.f && (l.rope_original <= 0 || !(l.rope_high > l.rope_low))) return "rope scaling needs original > 0 and high > low" + at;
      if (l.mask != HB_MASK_WINDOW && l.mask != HB_MASK_CHUNK && l.mask != HB_MASK_CAUSAL) return "unknown mask" + at;
      if (l.mask != HB_MASK_CAUSAL && l.window <= 0) return "window / chunk size must be positive" + at;
      if (l.dim > 512 || l.vdim > 512) return "head size > 512 unsupported" + at;
      if (l.kv_from >= 0) return "kv_from is a latent-attention option" + at;
      if ((l.attn_flags & HB_ATTN_QK_PROJ_NORM) && (l.attn_flags & HB_ATTN_QK_UNIT_NORM)) return "two q / k norms" + at;
      if ((l.attn_flags & HB_ATTN_LEARNED_SINK) && (l.attn_flags & HB_ATTN_UNIT_SINK)) return "two softmax sinks" + at;
      if ((l.attn_flags & HB_ATTN_V_BLEND) && (l.attn_flags & HB_ATTN_V_IS_K)) return "blended values need a value projection" + at;
      if (l.attn_flags & HB_ATTN_V_BLEND)
        for (int j = 0; j < i; ++j)
          if (L[j].mixer == HB_MIXER_GQA && (L[j].attn_flags & HB_ATTN_V_BLEND) && L[j].kv_heads * L[j].vdim != l.kv_heads * l.vdim)
            return "layers that blend values need equal kv_heads * vdim" + at;
      if ((size_t)(l.heads + l.kv_heads) * l.dim + (size_t)l.kv_heads * l.vdim > 24 * 1024) return "q + k + v row > 24576 entries unsupported" + at;
    } else if (l.mixer == HB_MIXER_DELTA) {
      if (l.kv_heads <= 0 || l.heads % l.kv_heads) return "heads must be a multiple of kv_heads" + at;
      if (l.dim > 256) return "delta-rule key channels per head > 256 unsupported" + at;
      if (l.conv_taps < 1 || l.conv_taps > 16) return "convolution taps must be 1..16" + at;
    } else if (l.mixer == HB_MIXER_MAMBA2) {
      if (l.kv_heads <= 0 || l.heads % l.kv_heads) return "heads must be a multiple of the groups" + at;
      if (l.dim > 256) return "state size > 256 unsupported" + at;
      if (l.conv_taps < 1 || l.conv_taps > 16) return "convolution taps must be 1..16" + at;
      if (l.norm_groups < 1 || (l.heads * l.vdim) % l.norm_groups) return "norm_groups must divide heads * vdim" + at;
    } else if (l.mixer == HB_MIXER_MLSTM) {
      if (l.dim > 256) return "matrix-memory key channels per head > 256 unsupported" + at;
      if (!(l.gate_cap > 0.f)) return "gate_cap must be positive" + at;
    } else {
      return "unknown mixer" + at;
    }
    if (l.mixer == HB_MIXER_GQA) {
      if ((l.attn_flags & HB_ATTN_QKV_CONV) && (l.conv_taps < 1 || l.conv_taps > 16)) return "convolution taps must be 1..16" + at;
      if ((l.attn_flags & HB_ATTN_QKV_CONV) && (l.attn_flags & (HB_ATTN_QK_PROJ_NORM | HB_ATTN_V_BLEND | HB_ATTN_V_IS_K)))
        return "convolved projections with a whole-projection norm, blended values or values that are the keys are unsupported" + at;
      if ((l.attn_flags & HB_ATTN_OUT_GATE) && (l.attn_flags & HB_ATTN_HEAD_GATE)) return "two output gates" + at;
    }
    if (l.side_heads < 0) return "negative side_heads" + at;
    if (l.side_heads > 0) {
      if (l.mixer != HB_MIXER_GQA) return "a second mixer stands beside a grouped-query mixer only" + at;
      if (l.side_mixer != HB_MIXER_MLSTM) return "the second mixer must be a matrix memory" + at;
      if (l.side_dim <= 0 || l.side_vdim <= 0 || l.side_dim > 256) return "second mixer head sizes" + at;
      if (!(l.side_gate_cap > 0.f)) return "side_gate_cap must be positive" + at;
      if (l.attn_flags & HB_ATTN_HEAD_GATE) return "a second mixer with a per-head gate on the first is unsupported" + at;
    }
    if (l.weights_of < 0 || l.weights_of > d.n_layers || l.weights_of == i + 1) return "weights_of must name another layer" + at;
    if (l.weights_of > 0) {
      hb_layer_desc a = l, b = L[l.weights_of - 1];
      if (b.weights_of > 0) return "weights_of must name a layer with tensors of its own" + at;
      a.weights_of = b.weights_of = 0;
      if (memcmp(&a, &b, sizeof a) != 0) return "a layer that uses another layer's tensors must have its description" + at;
      if (l.attn_flags & HB_ATTN_V_BLEND) return "shared tensors with blended values are unsupported" + at;
      if (l.mixer == HB_MIXER_LATENT) return "shared tensors for latent attention are unsupported" + at;
    }
    if (l.ff < 0) return "negative ff" + at;
    if (l.ff > 0) {
      if (l.ff_kind == HB_FF_MOE) {
        if (l.experts <= 0 || l.identity_experts < 0 || l.top_k <= 0 || l.top_k > l.experts + l.identity_experts) return "mixture-of-experts sizes" + at;
        if (l.experts + l.identity_experts > 1024 || l.top_k > 32) return "more than 1024 router outputs or top_k > 32 unsupported" + at;
        if (l.router_kind != HB_ROUTER_SOFTMAX && l.router_kind != HB_ROUTER_SIGMOID) return "unknown router kind" + at;
        if (l.expert_kind != HB_EXPERT_SILU && l.expert_kind != HB_EXPERT_CLAMPED) return "unknown expert kind" + at;
        if (l.route_groups > 1) {
          const int R = l.experts + l.identity_experts;
          if (R % l.route_groups) return "router outputs must divide into the groups" + at;
          if (l.route_keep <= 0 || l.route_keep > l.route_groups) return "groups kept must be 1..groups" + at;
          if (l.route_keep * (R / l.route_groups) < l.top_k) return "the kept groups hold fewer outputs than top_k" + at;
        }
        if (l.shared_ff < 0) return "negative shared_ff" + at;
      } else if (l.ff_kind != HB_FF_CLAMPED && l.ff_kind != HB_FF_GELU_TANH && l.ff_kind != HB_FF_SILU && l.ff_kind != HB_FF_RELU2) {
        return "unknown feed-forward kind" + at;
      }
    }
  }
  if (d.norm_place != HB_NORM_OF_SUM && d.norm_place != HB_NORM_OF_OUTPUT && d.norm_place != HB_NORM_BOTH_SIDES &&
      d.norm_place != HB_NORM_PARALLEL)
    return "unknown norm_place";
  if (d.norm_place == HB_NORM_PARALLEL) {
    if (d.norm_kind != HB_NORM_RMS) return "parallel sublayers need RMS norms";
    for (int i = 0; i < d.n_layers; ++i)
      if (L[i].ff > 0 && (L[i].ff_kind == HB_FF_MOE || L[i].ff_kind == HB_FF_CLAMPED)) return "parallel sublayers with a mixture or a biased feed-forward are unsupported";
  }
  if (d.norm_kind != HB_NORM_RMS && d.norm_kind != HB_NORM_TANH) return "unknown norm_kind";
  for (int i = 0; i < d.n_layers; ++i) {
    if (L[i].mixer != HB_MIXER_GQA || !(L[i].attn_flags & HB_ATTN_OUT_BIAS)) continue;
    if (d.norm_kind == HB_NORM_TANH) return "tanh norms with a biased output projection are unsupported";
    if (d.norm_place != HB_NORM_PARALLEL && L[i].side_heads > 0 && L[i].mix_scale != 0.f && L[i].mix_scale != 1.f)
      return "a weighted first mixer with a biased output projection needs parallel sublayers";
  }
  for (int i = 0; i < d.n_layers; ++i)
    if (L[i].side_heads > 0 && !(L[i].attn_flags & HB_ATTN_OUT_GATE)) return "a second mixer needs the entry-wise output gate on the first";
  if (d.norm_kind == HB_NORM_TANH && d.norm_place == HB_NORM_OF_SUM) return "tanh norms of the sum are unsupported";
  if (d.norm_kind == HB_NORM_TANH && !d.plain_gains) return "tanh norms store their gains plainly";
  if (d.norm_kind == HB_NORM_TANH)
    for (int i = 0; i < d.n_layers; ++i)
      if (L[i].ff > 0 && L[i].ff_kind == HB_FF_CLAMPED) return "tanh norms with a biased feed-forward are unsupported";
  return "";
}

std::vector<double> stack_rope_freqs(const hb_layer_desc& l) {
  const int half = l.rope_dims / 2;
  std::vector<double> f(half);
  for (int i = 0; i < half; ++i) f[i] = pow((double)l.rope_base, -2.0 * i / (double)l.rope_dims);
  if (l.rope_linear > 0.f)
    for (int i = 0; i < half; ++i) f[i] /= (double)l.rope_linear;
  if (l.rope_factor > 0.f) {
    const double factor = l.rope_factor, lo = l.rope_low, hi = l.rope_high, orig = l.rope_original;
    for (int i = 0; i < half; ++i) {
      const double wl = 2.0 * M_PI / f[i];
      if (wl < orig / hi) continue;
      if (wl > orig / lo) {
        f[i] /= factor;
      } else {
        const double s = (orig / wl - lo) / (hi - lo);
        f[i] = (1.0 - s) * f[i] / factor + s * f[i];
      }
    }
  }
  return f;
}

static size_t carve_stack(Model* m, const hb_stack_desc& d, const hb_layer_desc* L, uint8_t* base) {
  const size_t es = d.compute_f32 ? 4 : 2;
  size_t off = 0;
  auto take = [&](size_t elems) -> uint8_t* {
    uint8_t* p = base ? base + off : nullptr;
    off += up(elems * es);
    return p;
  };
  bool muted = false;  // a layer that uses another layer's tensors lays out nothing of its own
  size_t put_ld = 0;   // destination row stride of the next placements (0: rows are contiguous)
  auto put = [&](const std::string& name, uint8_t* dst, size_t row_off, size_t rows, size_t cols, bool gain = false, float fill = 1.f,
                 bool bias = false, int mode = 0) {
    if (!m || muted) return;
    Placement p;
    p.mode = mode;
    p.ld = put_ld;
    p.dst = reinterpret_cast<bf16*>(dst ? dst + row_off * (put_ld ? put_ld : cols) * es : nullptr);
    p.rows = rows;
    p.cols = cols;
    p.is_norm_gain = gain;
    p.is_bias = bias;
    p.fill = fill;
    p.elem = (int)es;
    m->placements[name] = p;
  };
  const size_t W = d.width, V = d.vocab;
  const float gain_fill = d.plain_gains ? 1.f : 0.f;  // neutral value of a stored residual-norm gain
  const bool tanh_norm = d.norm_kind == HB_NORM_TANH, both = d.norm_place == HB_NORM_BOTH_SIDES;
  // a norm of the stream: its gain, and for tanh norms the offset vector and the scalar behind it in one block
  auto norm_block = [&](const std::string& name) -> uint8_t* {
    uint8_t* p = take(tanh_norm ? 2 * W + 1 : W);
    put(name, p, 0, W, 1, true, gain_fill);
    if (tanh_norm) {
      put(name + ".b", p ? p + W * es : nullptr, 0, W, 1, true, 0.f);
      put(name + ".alpha", p ? p + 2 * W * es : nullptr, 0, 1, 1, true, 1.f);
    }
    return p;
  };
  uint8_t* embed = take(V * W);
  put("embed", embed, 0, V, W);
  uint8_t* embed_norm = d.embed_norm ? norm_block("embed.norm") : nullptr;
  if (m) {
    m->s_embed = embed;
    m->s_embed_norm = embed_norm;
    m->sw.assign(d.n_layers, StackLayerW{});
    m->state_floats = 0;
    m->plane_row.clear();
    m->elem = (int)es;
  }
  std::vector<int> plane_of(d.n_layers, -1);
  int planes = 0;
  for (int i = 0; i < d.n_layers; ++i) {
    const hb_layer_desc& l = L[i];
    const std::string p = "l" + std::to_string(i) + ".";
    StackLayerW w;
    const size_t H = l.heads, Dk = l.dim, Dv = l.vdim;
    const bool shared_w = l.weights_of > 0;
    const size_t off_before = off;
    muted = shared_w;
    w.norm1 = norm_block(p + "norm1");
    if (both) w.norm1b = norm_block(p + "norm1b");
    // a matrix memory: rows [q | k | v | g | i | f] from row `row0` of the fused projection `in`, gate biases in `bias`
    auto carve_mlstm = [&](const std::string& pm, uint8_t* in, uint8_t* bias, size_t row0, size_t Hm, size_t Dm, size_t Dvm, float cap) {
      MlstmW& q = w.ml;
      q.H = (int)Hm; q.D = (int)Dm; q.Dv = (int)Dvm; q.cap = cap;
      q.off_q = (int)row0;
      q.off_k = q.off_q + (int)(Hm * Dm);
      q.off_v = q.off_k + (int)(Hm * Dm);
      q.off_g = q.off_v + (int)(Hm * Dvm);
      q.off_i = q.off_g + (int)(Hm * Dvm);
      q.off_f = q.off_i + (int)Hm;
      put(pm + "q", in, q.off_q, Hm * Dm, W);
      put(pm + "k", in, q.off_k, Hm * Dm, W);
      put(pm + "v", in, q.off_v, Hm * Dvm, W);
      put(pm + "g", in, q.off_g, Hm * Dvm, W);
      put(pm + "i", in, q.off_i, Hm, W);
      put(pm + "f", in, q.off_f, Hm, W);
      put(pm + "i.b", bias ? bias + (size_t)q.off_i * es : nullptr, 0, Hm, 1, false, 1.f, true);
      put(pm + "f.b", bias ? bias + (size_t)q.off_f * es : nullptr, 0, Hm, 1, false, 1.f, true);
      uint8_t* hn = take(Hm * Dvm);
      put(pm + "norm", hn, 0, Hm * Dvm, 1, true, 1.f);
      q.hnorm = hn;
      if (m) {
        q.state_off = m->state_floats;
        q.n_off = q.state_off + Hm * Dm * Dvm;
        q.m_off = q.n_off + Hm * Dm;
        m->state_floats += Hm * Dm * Dvm + Hm * Dm + Hm;
        m->state_floats = (m->state_floats + 3) & ~size_t(3);
      }
      return (size_t)q.off_f + Hm - row0;  // rows taken
    };
    if (l.mixer == HB_MIXER_MAMBA2) {
      const size_t G = l.kv_heads, N = Dk, inner = H * Dv, C = inner + 2 * G * N, taps = l.conv_taps;
      w.off_g = 0;                       // z
      w.off_v = (int)inner;              // x
      w.off_k = (int)(2 * inner);        // B
      w.off_q = (int)(2 * inner + G * N);  // C
      w.off_a = (int)(2 * inner + 2 * G * N);  // dt
      w.n_in = w.off_a + (int)H;
      uint8_t* in = take((size_t)w.n_in * W);
      w.w_in = in;
      put(p + "mix.in", in, 0, (size_t)w.n_in, W);
      uint8_t* cw = take(C * taps);
      uint8_t* cb = take(C);
      put(p + "mix.conv", cw, 0, C, taps);
      put(p + "mix.conv.b", cb, 0, C, 1, false, 1.f, true);
      uint8_t* adt = take(3 * H);
      put(p + "mix.A_log", adt, 0, H, 1, false, 1.f, true);
      put(p + "mix.dt_bias", adt ? adt + H * es : nullptr, 0, H, 1, false, 1.f, true);
      put(p + "mix.D", adt ? adt + 2 * H * es : nullptr, 0, H, 1, true, 1.f);
      uint8_t* hn = take(inner);
      uint8_t* o = take(W * inner);
      put(p + "mix.norm", hn, 0, inner, 1, true, 1.f);
      put(p + "mix.o", o, 0, W, inner);
      w.conv_w = cw; w.conv_b = cb; w.a_dt = adt; w.hnorm = hn; w.wo = o; w.o_cols = (int)inner;
      if (m) {
        w.state_off = m->state_floats;
        w.tail_off = w.state_off + H * N * Dv;
        m->state_floats += H * N * Dv + (taps - 1) * C;
        m->state_floats = (m->state_floats + 3) & ~size_t(3);
      }
    } else if (l.mixer == HB_MIXER_MLSTM) {
      const size_t rows = 2 * H * Dk + 2 * H * Dv + 2 * H;
      uint8_t* in = take(rows * W);
      uint8_t* b = take(rows);
      w.w_in = in; w.b_in = b; w.n_in = (int)rows;
      carve_mlstm(p + "mix.", in, b, 0, H, Dk, Dv, l.gate_cap);
      uint8_t* o = take(W * H * Dv);
      put(p + "mix.o", o, 0, W, H * Dv);
      w.wo = o; w.o_cols = (int)(H * Dv);
    } else if (l.mixer == HB_MIXER_DELTA) {
      const size_t G = l.kv_heads, C = 2 * G * Dk + H * Dv, taps = l.conv_taps;
      w.off_q = 0;
      w.off_k = (int)(G * Dk);
      w.off_v = (int)(2 * G * Dk);
      w.off_g = (int)(2 * G * Dk + H * Dv);
      w.off_b = (int)(2 * G * Dk + 2 * H * Dv);
      w.off_a = w.off_b + (int)H;
      w.n_in = w.off_a + (int)H;
      uint8_t* in = take((size_t)w.n_in * W);
      w.w_in = in;
      put(p + "mix.q", in, w.off_q, G * Dk, W);
      put(p + "mix.k", in, w.off_k, G * Dk, W);
      put(p + "mix.v", in, w.off_v, H * Dv, W);
      put(p + "mix.g", in, w.off_g, H * Dv, W);
      put(p + "mix.b", in, w.off_b, H, W);
      put(p + "mix.a", in, w.off_a, H, W);
      uint8_t* cw = take(C * taps);
      put(p + "mix.q.conv", cw, 0, G * Dk, taps);
      put(p + "mix.k.conv", cw, G * Dk, G * Dk, taps);
      put(p + "mix.v.conv", cw, 2 * G * Dk, H * Dv, taps);
      uint8_t* adt = take(2 * H);
      put(p + "mix.A_log", adt, 0, H, 1, false, 1.f, true);
      put(p + "mix.dt_bias", adt ? adt + H * es : nullptr, 0, H, 1, false, 1.f, true);
      uint8_t* hn = take(Dv);
      uint8_t* o = take(W * H * Dv);
      put(p + "mix.norm", hn, 0, Dv, 1, true, 1.f);
      put(p + "mix.o", o, 0, W, H * Dv);
      w.conv_w = cw; w.a_dt = adt; w.hnorm = hn; w.wo = o;
      if (m) {
        w.state_off = m->state_floats;
        w.tail_off = w.state_off + H * Dk * Dv;
        m->state_floats += H * Dk * Dv + (taps - 1) * C;
      }
    } else if (l.mixer == HB_MIXER_GLA) {
      const size_t r = l.decay_rank;
      w.off_q = 0;
      w.off_k = (int)(H * Dk);
      w.off_v = (int)(2 * H * Dk);
      w.off_g = (int)(2 * H * Dk + H * Dv);
      w.off_a1 = (int)(2 * H * Dk + 2 * H * Dv);
      w.n_in = (int)(2 * H * Dk + 2 * H * Dv + r);
      uint8_t* in = take((size_t)w.n_in * W);
      w.w_in = in;
      put(p + "mix.q", in, w.off_q, H * Dk, W);
      put(p + "mix.k", in, w.off_k, H * Dk, W);
      put(p + "mix.v", in, w.off_v, H * Dv, W);
      put(p + "mix.g", in, w.off_g, H * Dv, W);
      put(p + "mix.a1", in, w.off_a1, r, W);
      uint8_t* a2 = take(H * Dk * r);
      uint8_t* a2b = take(H * Dk);
      uint8_t* hn = take(Dv);
      uint8_t* o = take(W * H * Dv);
      put(p + "mix.a2", a2, 0, H * Dk, r);
      put(p + "mix.a2.b", a2b, 0, H * Dk, 1, false, 1.f, true);
      put(p + "mix.norm", hn, 0, Dv, 1, true, 1.f);
      put(p + "mix.o", o, 0, W, H * Dv);
      w.a2 = a2; w.a2b = a2b; w.hnorm = hn; w.wo = o;
      if (m) {
        w.state_off = m->state_floats;
        m->state_floats += H * Dk * Dv;
      }
    } else if (l.mixer == HB_MIXER_GQA) {
      const size_t G = l.kv_heads;
      const bool own_v = !(l.attn_flags & HB_ATTN_V_IS_K), gated = (l.attn_flags & HB_ATTN_HEAD_GATE) != 0;
      const bool out_gate = (l.attn_flags & HB_ATTN_OUT_GATE) != 0, side = l.side_heads > 0;
      const std::string pm = p + (side ? "mix.left." : "mix.");  // with a second mixer the first one's tensors are mix.left.*
      w.off_q = 0;
      w.off_k = (int)(H * Dk);
      w.off_v = own_v ? (int)(H * Dk + G * Dk) : w.off_k;
      w.off_g = (int)(H * Dk + G * Dk + (own_v ? G * Dv : 0));
      w.n_in = w.off_g + (gated ? (int)H : 0) + (out_gate ? (int)(H * Dv) : 0);
      const size_t first_rows = (size_t)w.n_in;
      if (side) w.n_in += (int)(2 * (size_t)l.side_heads * l.side_dim + 2 * (size_t)l.side_heads * l.side_vdim + 2 * (size_t)l.side_heads);
      uint8_t* in = take((size_t)w.n_in * W);
      w.w_in = in;
      put(pm + "q", in, w.off_q, H * Dk, W);
      put(pm + "k", in, w.off_k, G * Dk, W);
      if (own_v) put(pm + "v", in, w.off_v, G * Dv, W);
      if (gated) put(pm + "g", in, w.off_g, H, W);
      if (out_gate) put(pm + "g", in, w.off_g, H * Dv, W);
      if ((l.attn_flags & HB_ATTN_QKV_BIAS) || side) {
        uint8_t* b = take((size_t)w.n_in);
        w.b_in = b;
        if (l.attn_flags & HB_ATTN_QKV_BIAS) {
          put(pm + "q.b", b ? b + (size_t)w.off_q * es : nullptr, 0, H * Dk, 1, false, 1.f, true);
          put(pm + "k.b", b ? b + (size_t)w.off_k * es : nullptr, 0, G * Dk, 1, false, 1.f, true);
          if (own_v) put(pm + "v.b", b ? b + (size_t)w.off_v * es : nullptr, 0, G * Dv, 1, false, 1.f, true);
        }
      }
      if (side) carve_mlstm(p + "mix.right.", in, (uint8_t*)w.b_in, first_rows, l.side_heads, l.side_dim, l.side_vdim, l.side_gate_cap);
      if (l.attn_flags & HB_ATTN_QKV_CONV) {
        const size_t taps = l.conv_taps, C = H * Dk + G * Dk + G * Dv;
        uint8_t* cw = take(C * taps);
        w.conv_w = cw;
        put(pm + "q.conv", cw, 0, H * Dk, taps);
        put(pm + "k.conv", cw, H * Dk, G * Dk, taps);
        put(pm + "v.conv", cw, H * Dk + G * Dk, G * Dv, taps);
        if (m) {
          w.tail_off = m->state_floats;
          m->state_floats += (taps - 1) * C;
          m->state_floats = (m->state_floats + 3) & ~size_t(3);
        }
      }
      if (l.attn_flags & HB_ATTN_QK_PROJ_NORM) {
        uint8_t* gn = take((H + G) * Dk);
        w.qk_gain = gn;
        put(pm + "q.norm", gn, 0, H * Dk, 1, true, 1.f);
        put(pm + "k.norm", gn ? gn + H * Dk * es : nullptr, 0, G * Dk, 1, true, 1.f);
      }
      if (l.attn_flags & HB_ATTN_LEARNED_SINK) {
        uint8_t* sk = take(H);
        w.sink = sk;
        put(pm + "sink", sk, 0, H, 1, false, 1.f, true);
      }
      if (l.attn_flags & HB_ATTN_V_BLEND) {
        bool earlier = false;
        for (int j = 0; j < i; ++j) earlier |= L[j].mixer == HB_MIXER_GQA && (L[j].attn_flags & HB_ATTN_V_BLEND);
        w.blend_role = earlier ? 2 : 1;
        if (earlier) {  // the first blending layer keeps its own values: it has no use for a blend weight
          uint8_t* vm = take(1);
          w.vmix = vm;
          put(pm + "vmix", vm, 0, 1, 1, false, 1.f, true);
        }
      }
      // the output projections of both mixers side by side in every row: one product over [first | second] inputs
      const size_t KL = H * Dv, KR = side ? (size_t)l.side_heads * l.side_vdim : 0;
      uint8_t* o = take(W * (KL + KR));
      w.wo = o; w.o_cols = (int)(KL + KR);
      if (side) {
        put_ld = KL + KR;
        put(pm + "o", o, 0, W, KL);
        put(p + "mix.right.o", o ? o + KL * es : nullptr, 0, W, KR);
        put_ld = 0;
      } else {
        put(pm + "o", o, 0, W, KL);
      }
      if (l.attn_flags & HB_ATTN_OUT_BIAS) {
        uint8_t* ob = take(W);
        w.o_bias = ob;
        put(pm + "o.b", ob, 0, W, 1, false, 1.f, true);
      }
      w.cache_plane = planes++;
      w.cache_plane_v = planes++;
      if (m) {
        m->plane_row.push_back((int)(G * Dk));
        m->plane_row.push_back((int)(G * Dv));
      }
    } else {
      const size_t Q = l.q_rank, R = l.kv_rank, Dr = l.rot_dim;
      const bool own = l.kv_from < 0;
      w.off_dq = 0;
      w.off_dkv = own ? (int)Q : -1;
      w.off_g = (int)(Q + (own ? R + Dr : 0));
      w.n_in = (int)(w.off_g + H * Dv);
      uint8_t* in = take((size_t)w.n_in * W);
      w.w_in = in;
      put(p + "mix.dq", in, 0, Q, W);
      if (own) put(p + "mix.dkv", in, Q, R + Dr, W);
      put(p + "mix.g", in, w.off_g, H * Dv, W);
      uint8_t* dqn = take(Q);
      uint8_t* uq = take(H * (Dk + Dr) * Q);
      uint8_t* dkvn = own ? take(R) : nullptr;
      uint8_t* uk = take(H * Dk * R);
      uint8_t* uv = take(H * Dv * R);
      uint8_t* ukT = d.compute_f32 ? nullptr : take(H * Dk * R);
      w.ukT = ukT;
      uint8_t* sink = take(H);
      uint8_t* o = take(W * H * Dv);
      put(p + "mix.dq.norm", dqn, 0, Q, 1, true, 1.f);
      put(p + "mix.uq", uq, 0, H * (Dk + Dr), Q);
      if (own) put(p + "mix.dkv.norm", dkvn, 0, R, 1, true, 1.f);
      put(p + "mix.uk", uk, 0, H * Dk, R);
      put(p + "mix.uv", uv, 0, H * Dv, R);
      put(p + "mix.sink", sink, 0, H, 1, false, 1.f, true);
      put(p + "mix.o", o, 0, W, H * Dv);
      w.dq_norm = dqn; w.uq = uq; w.dkv_norm = dkvn; w.uk = uk; w.uv = uv; w.sink = sink; w.wo = o;
      if (own) {
        plane_of[i] = planes++;
        if (m) m->plane_row.push_back((int)(R + Dr));
      } else {
        plane_of[i] = plane_of[l.kv_from];
      }
      w.cache_plane = plane_of[i];
    }
    if (l.ff > 0 && l.ff_kind == HB_FF_MOE) {
      const size_t Fn = l.ff, E = l.experts, R = (size_t)l.experts + l.identity_experts;
      uint8_t* n2 = norm_block(p + "norm2");
      if (both) w.norm2b = norm_block(p + "norm2b");
      uint8_t* router = take(std::max<size_t>(R, 64) * W);  // at least one MMA tile of rows; the arena is zeroed at load
      uint8_t* corr = take(R);
      uint8_t* gu = take(E * 2 * Fn * W);
      uint8_t* dn = take(E * W * Fn);
      put(p + "mlp.router", router, 0, R, W);
      put(p + "mlp.correction", corr, 0, R, 1, false, 1.f, true);
      if (l.shared_ff > 0) {
        const size_t Fs = l.shared_ff;
        uint8_t* sg = take(2 * Fs * W);
        uint8_t* sd = take(W * Fs);
        const bool spk = !d.compute_f32 && Fs % 128 == 0;
        put(p + "mlp.shared.gate", sg, 0, Fs, W, false, 1.f, false, spk ? 1 : 0);
        put(p + "mlp.shared.up", sg, spk ? 0 : Fs, Fs, W, false, 1.f, false, spk ? 2 : 0);
        put(p + "mlp.shared.down", sd, 0, W, Fs);
        w.w_gu_sh = sg; w.w_down_sh = sd; w.sh_packed = spk;
      }
      const bool packed = !d.compute_f32 && Fn % 128 == 0;
      for (size_t e = 0; e < E; ++e) {
        const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
        put(pe + "gate", gu, e * 2 * Fn, Fn, W, false, 1.f, false, packed ? 1 : 0);
        put(pe + "up", gu, e * 2 * Fn + (packed ? 0 : Fn), Fn, W, false, 1.f, false, packed ? 2 : 0);
        put(pe + "down", dn, e * W, W, Fn);
      }
      w.gu_packed = packed;
      w.norm2 = n2; w.router = router; w.correction = corr; w.w_gu = gu; w.w_down = dn;
    } else if (l.ff > 0 && (l.ff_kind == HB_FF_GELU_TANH || l.ff_kind == HB_FF_SILU)) {
      const size_t Fn = l.ff;
      uint8_t* n2 = norm_block(p + "norm2");
      if (both) w.norm2b = norm_block(p + "norm2b");
      uint8_t* gu = take(2 * Fn * W);
      uint8_t* dn = take(W * Fn);
      const bool packed = !d.compute_f32 && Fn % 128 == 0;
      put(p + "mlp.gate", gu, 0, Fn, W, false, 1.f, false, packed ? 1 : 0);
      put(p + "mlp.up", gu, packed ? 0 : Fn, Fn, W, false, 1.f, false, packed ? 2 : 0);
      put(p + "mlp.down", dn, 0, W, Fn);
      w.gu_packed = packed;
      w.norm2 = n2; w.w_gu = gu; w.w_down = dn;
    } else if (l.ff > 0 && l.ff_kind == HB_FF_RELU2) {
      const size_t Fn = l.ff;
      uint8_t* n2 = norm_block(p + "norm2");
      if (both) w.norm2b = norm_block(p + "norm2b");
      uint8_t* up_w = take(Fn * W);
      uint8_t* dn = take(W * Fn);
      put(p + "mlp.up", up_w, 0, Fn, W);
      put(p + "mlp.down", dn, 0, W, Fn);
      w.norm2 = n2; w.w_gu = up_w; w.w_down = dn;
    } else if (l.ff > 0) {
      const size_t Fn = l.ff;
      uint8_t* n2 = norm_block(p + "norm2");
      if (both) w.norm2b = norm_block(p + "norm2b");
      uint8_t* gu = take(2 * Fn * W);
      uint8_t* bgu = take(2 * Fn);
      uint8_t* dn = take(W * Fn);
      uint8_t* bdn = take(W);
      put(p + "mlp.gate", gu, 0, Fn, W);
      put(p + "mlp.up", gu, Fn, Fn, W);
      put(p + "mlp.gate.b", bgu, 0, Fn, 1, false, 1.f, true);
      put(p + "mlp.up.b", bgu, Fn, Fn, 1, false, 1.f, true);
      put(p + "mlp.down", dn, 0, W, Fn);
      put(p + "mlp.down.b", bdn, 0, W, 1, false, 1.f, true);
      w.norm2 = n2; w.w_gu = gu; w.b_gu = bgu; w.w_down = dn; w.b_down = bdn;
    }
    if (shared_w) {
      // the tensors are the named layer's; the arena space walked through above is handed back.  What stays the layer's own:
      // its cache planes and its offsets inside a state slot
      off = off_before;
      muted = false;
    }
    if (m) m->sw[i] = w;
  }
  if (m)
    for (int i = 0; i < d.n_layers; ++i) {  // the named layer may stand before or behind the one that uses its tensors
      if (L[i].weights_of <= 0) continue;
      const StackLayerW w = m->sw[i];
      StackLayerW o = m->sw[L[i].weights_of - 1];
      o.state_off = w.state_off; o.tail_off = w.tail_off;
      o.cache_plane = w.cache_plane; o.cache_plane_v = w.cache_plane_v;
      o.ml.state_off = w.ml.state_off; o.ml.n_off = w.ml.n_off; o.ml.m_off = w.ml.m_off;
      m->sw[i] = o;
    }
  if (m) m->state_floats = (m->state_floats + 3) & ~size_t(3);  // slots start on 16-byte boundaries
  uint8_t* fn = norm_block("final.norm");
  uint8_t* head = d.tie_head ? embed : take(V * W);
  if (!d.tie_head) put("head", head, 0, V, W);
  if (m) {
    m->s_final_norm = fn;
    m->s_head = head;
  }
  return off;
}

size_t arena_bytes_for_stack(const hb_stack_desc& d, const hb_layer_desc* layers) { return carve_stack(nullptr, d, layers, nullptr); }

void layout_stack(Model& m) {
  m.placements.clear();
  m.filled.clear();
  carve_stack(&m, m.sd, m.sl.data(), reinterpret_cast<uint8_t*>(m.arena));
}

size_t arena_bytes_for(const hb_model_desc& d) { return carve(nullptr, d, nullptr); }

void layout_model(Model& m) {
  m.placements.clear();
  m.filled.clear();
  carve(&m, m.d, reinterpret_cast<uint8_t*>(m.arena));
}

std::vector<float> rope_inv_freq(const hb_model_desc& d) {
  const int dim = d.head_dim;
  std::vector<float> f(dim / 2);
  for (int i = 0; i < dim / 2; ++i) {
    // HF: 1.0 / (base ** (arange(0, dim, 2).float() / dim)), evaluated in fp32
    const float e = (float)(2 * i) / (float)dim;
    f[i] = 1.0f / powf(d.rope_theta, e);
  }
  if (d.rope_factor > 0.f) {
    const float factor = d.rope_factor, lo = d.rope_low_freq_factor, hi = d.rope_high_freq_factor;
    const float old_len = (float)d.rope_orig_max_pos;
    const float low_wl = old_len / lo, high_wl = old_len / hi;
    for (int i = 0; i < dim / 2; ++i) {
      const float inv = f[i];
      const float wl = 2.0f * (float)M_PI / inv;
      float v = (wl > low_wl) ? inv / factor : inv;
      const float smooth = (old_len / wl - lo) / (hi - lo);
      const float smoothed = (1.0f - smooth) * v / factor + smooth * v;
      const bool medium = !(wl < high_wl) && !(wl > low_wl);
      f[i] = medium ? smoothed : v;
    }
  }
  return f;
}

}  // namespace hb
