// Weight arena: every tensor of a ModelInstance lives in ONE device allocation (so a replica can be
// filled by a single NCCL broadcast — SURVEY.md §8e) with projections pre-fused the way the kernels
// consume them:  wqkv = [q;k;v] rows,  w_gate_up packed per 256-row tile as [128 gate | 128 up].
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/helix_b200.h"
#include "kernels.h"

namespace hb {

struct LlamaLayerW {
  bf16 *attn_norm, *wqkv, *wo, *mlp_norm, *wgu, *wdown;
  bf16* bqkv = nullptr;  // [q;k;v] projection biases (hb_model_desc.qkv_bias), else null
};
struct BertLayerW {
  bf16 *wqkv, *bqkv, *wo, *bo, *ln1_g, *ln1_b, *w1, *b1, *w2, *b2, *ln2_g, *ln2_b;
};

// One layer of a layer-list decoder (HB_ARCH_RISEPEL).  Pointers are arena addresses of elements of Model::elem bytes.
// Projections that read the same input are stacked into one weight (w_in) so one GEMM produces all of them:
//   GLA:    rows [q | k | v | g | a1]            LATENT: rows [dq | dkv (own cache only) | g]
//   GQA:    rows [q | k | v (unless the values are the keys) | g (one row per head, when gated)]
//   DELTA:  rows [q | k | v | g | b (one row per head) | a (one row per head)]
// Norms of kind HB_NORM_TANH are blocks [gain (width) | offset (width) | alpha (1)] behind one pointer.
// A matrix-memory mixer (HB_MIXER_MLSTM) as a layer's only mixer or beside its first one: columns of the layer's fused
// projection, gain over all heads' entries, float offsets of S [H][D][Dv], n [H][D] and m [H] inside a state slot.
struct MlstmW {
  int H = 0, D = 0, Dv = 0;  // H == 0: the layer has none
  float cap = 0.f;
  int off_q = 0, off_k = 0, off_v = 0, off_g = 0, off_i = 0, off_f = 0;
  void* hnorm = nullptr;
  size_t state_off = 0, n_off = 0, m_off = 0;
};

struct StackLayerW {
  void *norm1 = nullptr, *norm2 = nullptr;
  void *norm1b = nullptr, *norm2b = nullptr;  // HB_NORM_BOTH_SIDES: the norms of the sublayers' outputs (norm1 / norm2: of their inputs)
  void* w_in = nullptr;
  int n_in = 0;
  int off_q = 0, off_k = 0, off_v = 0, off_g = 0, off_a1 = 0, off_dq = 0, off_dkv = -1;  // columns of the fused projection
  void *a2 = nullptr, *a2b = nullptr, *hnorm = nullptr;                                          // GLA
  void *dq_norm = nullptr, *uq = nullptr, *dkv_norm = nullptr, *uk = nullptr, *uv = nullptr, *sink = nullptr;  // LATENT
  void* ukT = nullptr;  // LATENT, bf16 mode: [heads][kv_rank][dim] copy of uk (built after load; no checkpoint tensor)
  void* b_in = nullptr;     // GQA with biases: [n_in] in the order of w_in's rows
  void* qk_gain = nullptr;  // GQA with whole-projection norms: [heads * dim | kv_heads * dim]
  void* vmix = nullptr;     // GQA with blended values: the blend weight (1 element)
  int blend_role = 0;       // 0: no blending; 1: the first blending layer (keeps its values, publishes them); 2: blends
  int off_b = 0, off_a = 0;                      // DELTA: columns of the write-strength and decay rows
  void *conv_w = nullptr, *a_dt = nullptr;       // DELTA: [2 kv_heads dim + heads vdim][taps] in q, k, v order; [A_log (heads) | dt_bias (heads)]
  size_t tail_off = 0;                           // DELTA: float offset of the [taps - 1][channels] convolution inputs inside a state slot
  void *w_gu_sh = nullptr, *w_down_sh = nullptr;  // mixture of experts: the unit every token uses, rows [gate | up] and down
  // MAMBA2: rows [z | x | B | C | dt] of w_in; conv_w [heads vdim + 2 kv_heads dim][taps] and its bias conv_b; a_dt =
  // [A_log (heads) | dt_bias (heads) | D (heads)]; hnorm [heads vdim]; state_off: S [heads][dim][vdim], tail_off: the convolution's
  // last inputs.  GQA with convolved projections: conv_w [q | k | v channels][taps], tail_off.
  void* conv_b = nullptr;
  MlstmW ml;                 // MLSTM as the only mixer, or the second mixer of the layer
  void* o_bias = nullptr;    // GQA: bias of the output projection [width]
  int o_cols = 0;            // columns of wo: the first mixer's heads * vdim (+ the second's, stored behind them in every row)
  void* wo = nullptr;
  void *w_gu = nullptr, *b_gu = nullptr, *w_down = nullptr, *b_down = nullptr;  // feed-forward: rows [gate | up]
  size_t state_off = 0;  // GLA: float offset of this layer's [heads][dim][vdim] block inside a state slot
  int cache_plane = -1;  // LATENT: plane of the latent pool this layer reads (its own, or the kv_from layer's); GQA: its key plane
  int cache_plane_v = -1;  // GQA: its value plane.  Both are [page][kv_head][page_size][dim | vdim]
  // mixture of experts: router rows and choice corrections for experts + identity outputs; expert e's [gate | up] rows at
  // w_gu + e * 2 ff * width, its down-projection at w_down + e * width * ff
  void *router = nullptr, *correction = nullptr;
  // bf16 mode, ff a multiple of 128 (tanh-GELU unit, experts): [gate | up] rows stored per 256-row tile as [128 gate | 128 up],
  // the layout the gated epilogue of the tcgen05 GEMM reads; every other consumer indexes through it
  bool gu_packed = false;
  bool sh_packed = false;  // the same for the unit every token of a mixture uses
};

// where an uploaded checkpoint tensor lands inside the arena
struct Placement {
  bf16* dst = nullptr;
  size_t rows = 0, cols = 0;   // checkpoint tensor shape (cols == 1 for vectors)
  int mode = 0;                // 0: contiguous copy; 1: gate rows -> tile*256 + r%128; 2: up rows -> tile*256+128 + r%128
  bool is_norm_gain = false;   // random init sets these to 1
  bool is_bias = false;        // random init keeps these small
  size_t ld = 0;               // row stride of the destination in elements (0: cols, rows are contiguous)
  int elem = 2;                // bytes per arena element (4: layer-list decoders in fp32 mode; payloads are widened on upload)
  float fill = 1.0f;           // random init value of norm gains (0 where the stored gain is an offset from one)
};

struct Model {
  hb_model_desc d{};
  bf16* arena = nullptr;
  size_t arena_bytes = 0;
  float* inv_freq = nullptr;  // [head_dim/2] device (llama)
  // llama
  bf16 *embed = nullptr, *final_norm = nullptr, *lm_head = nullptr;
  std::vector<LlamaLayerW> ll;
  // bert
  bf16 *word = nullptr, *pos = nullptr, *type = nullptr, *emb_ln_g = nullptr, *emb_ln_b = nullptr;
  std::vector<BertLayerW> bl;
  // layer-list decoders
  hb_stack_desc sd{};
  std::vector<hb_layer_desc> sl;
  std::vector<StackLayerW> sw;
  void *s_embed = nullptr, *s_embed_norm = nullptr, *s_final_norm = nullptr, *s_head = nullptr;
  size_t state_floats = 0;              // fp32 state of one sequence over all GLA layers
  std::vector<int> plane_row;           // cache pool planes: elements per cached position (kv_rank + rot_dim; kv_heads * dim)
  int elem = 2;
  std::unordered_map<std::string, Placement> placements;  // HF checkpoint name -> arena slot
  std::unordered_map<std::string, bool> filled;

  int qkv_cols() const { return (d.heads + 2 * d.kv_heads) * d.head_dim; }
};

// Validates the description against what the kernels support; returns "" when fine.
std::string validate_desc(const hb_model_desc& d);
// Layer-list decoders: validation, arena size, layout (fills m.sw, m.placements, m.state_floats, m.plane_row).
std::string validate_stack(const hb_stack_desc& d, const hb_layer_desc* layers);
size_t arena_bytes_for_stack(const hb_stack_desc& d, const hb_layer_desc* layers);
void layout_stack(Model& m);
// Arena size in bytes for a description (also used by hb_memory_estimate).
size_t arena_bytes_for(const hb_model_desc& d);
// Carves `m.arena` (already allocated, m.arena_bytes long) into tensors and fills m.placements.
void layout_model(Model& m);
// Host inverse frequencies incl. llama3 scaling (HF transformers `_compute_llama3_parameters`).
std::vector<float> rope_inv_freq(const hb_model_desc& d);
// Rotation frequencies of a layer-list attention layer: base^(-2i/dims), i < dims/2, with the wavelength-dependent scaling
// of hb_layer_desc (rope_factor <= 0: none), in double precision.
std::vector<double> stack_rope_freqs(const hb_layer_desc& l);

}  // namespace hb
