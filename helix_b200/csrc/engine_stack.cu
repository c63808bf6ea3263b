// Layer-list decoders (HB_ARCH_STACK: the Risepel, Lurepel, Latanex and Funudra designs) inside hb::Engine: model load, the page pool's planes and recurrent state slots,
// the step's forward pass and the driven-sequence entry points.  Scheduling, page bookkeeping, the step block, sampling
// and request records are the engine's own (engine.cu); this file adds what differs from the Llama path:
//   * the residual stream is fp32 and post-normed; every sublayer reads the stream itself;
//   * ONE forward serves every step shape: each batch entry is a run of tokens [first, first + n) of a sequence whose
//     earlier tokens live in the latent pool (attention) and in its state slot (recurrence), so a prompt, a portion of a
//     prompt and a single decoded token are the same code with different n;
//   * attention layers cache one latent row per token ([c | k_rot]); a layer may read the rows of an earlier layer;
//   * recurrent layers keep one fp32 matrix per head in a state slot; an entry that starts at position 0 starts from zero,
//     so a slot needs no clearing when it changes hands.
//   * grouped-query layers keep two planes of the pool (rotated unit-norm keys, raw values) in the Llama path's
//     [page][kv_head][64][D] layout, so prompt portions and single-token steps run on that path's fused tcgen05 attention
//     kernels (block mask, unit sink and head gate are parameters of both); other shapes, short portions and the exact
//     mode take the per-token kernel;
//   * the residual step norms the sum (x <- norm(alpha x + f(x))), the sublayer's output (x <- x + norm(f(x))), or both sides
//     (x <- x + norm_b(f(norm_a(x))): the sublayers then read the normed copy of the stream, and one launch adds a sublayer's
//     normed output and norms the next sublayer's input); norms are RMS norms or element-wise tanh norms;
//   * grouped-query layers may carry projection biases, a norm over the whole q / k projection, capped scores, learned sinks,
//     sliding windows (all parameters of the fused attention kernels too) and values blended with an earlier layer's;
//   * gated-delta-rule layers keep, per sequence slot, one fp32 matrix per head and the last inputs of their short
//     convolutions; like the GLA state both start from zero inside the kernels when an entry starts at position 0;
//   * feed-forwards: clamped, silu and tanh-GELU gated units (gated epilogues of the GEMM), mixture of experts (softmax or
//     sigmoid router with an optional restriction to the best groups of experts, choice in fp32, items sorted by expert into
//     128-row segments on the device, two grouped tcgen05 products, an optional unit every token uses; nothing returns to the
//     host, so decode graphs stay static).
//   * stacks whose two sublayers read the same stream (x <- x + mixer(norm1 x) + ff(norm2 x)): one launch adds both outputs and
//     forms both normed inputs of the next layer from one row statistic; state-space layers and matrix memories (scalar-decay
//     recurrences on one kernel, state and convolution inputs in the slot); a second mixer beside a grouped-query one, their
//     output projections as one product over the concatenated inputs; layers that use an earlier layer's tensors with planes
//     and state of their own; logits from the embedding table.
#include "engine.h"
#include "launch.h"

#include <string.h>

#include <algorithm>

namespace hb {

namespace {
size_t al256(size_t x) { return (x + 255) & ~size_t(255); }
int up8(int x) { return (x + 7) / 8 * 8; }

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
template <typename T>
__global__ void fill_uniform_kernel(T* p, size_t n, uint64_t seed, float amp, float mean, size_t cols, size_t ld) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const uint64_t h = mix64(seed ^ (i * 0xD1B54A32D192ED03ull));
    const float u = (float)(h >> 40) * (1.0f / 16777216.0f) * 2.0f - 1.0f;
    const float v = __bfloat162float(__float2bfloat16(u * amp + mean));  // bf16-representable in either mode
    const size_t at = ld == cols ? i : i / cols * ld + i % cols;         // rows of `cols` elements, `ld` apart
    if constexpr (sizeof(T) == 4) p[at] = v; else p[at] = __float2bfloat16(v);
  }
}
}  // namespace

#define CU(expr)                                         \
  do {                                                   \
    cudaError_t e_ = (expr);                             \
    if (e_ != cudaSuccess) return fail_cuda(e_, #expr);  \
  } while (0)
#define LAUNCH(expr)                                     \
  do {                                                   \
    cudaError_t e_ = (expr);                             \
    launches_.fetch_add(1, std::memory_order_relaxed);   \
    if (e_ != cudaSuccess) return fail_cuda(e_, #expr);  \
  } while (0)
#define SPAN(cat, work, expr) \
  do {                        \
    span_begin(cat, work);    \
    LAUNCH(expr);             \
    span_end();               \
  } while (0)

// ------------------------------------------------------------------ load
int Engine::load_begin_stack(const hb_stack_desc& sd, const hb_layer_desc* layers) {
  std::lock_guard<std::mutex> g(gpu_mu_);
  if (loaded_ || load_open_) return fail(HB_ERR_STATE, "model already loaded on this engine");
  if (!layers || sd.n_layers <= 0) return fail(HB_ERR_INVALID, "unsupported model description: no layer list");
  // no position reaches max_ctx, so a longer window sees what a window of max_ctx sees: size the kernels for the shorter one
  std::vector<hb_layer_desc> lv(layers, layers + sd.n_layers);
  for (hb_layer_desc& l : lv) {
    if (l.mixer == HB_MIXER_LATENT && l.window > cfg_.max_ctx) l.window = cfg_.max_ctx;
    if (l.mixer == HB_MIXER_GQA) {  // a block or window that no sequence outgrows is the causal mask
      if (l.mask == HB_MASK_CAUSAL || l.window >= cfg_.max_ctx) { l.mask = HB_MASK_WINDOW; l.window = cfg_.max_ctx; }
    }
  }
  layers = lv.data();
  const std::string why = validate_stack(sd, layers);
  if (!why.empty()) return fail(HB_ERR_INVALID, "unsupported model description: " + why);
  // the per-token attention kernel keeps one position's scores in shared memory.  Steps replayed from graphs fix that size at
  // capture, so a full context has to fit; otherwise each launch is sized by its step's longest context and a sequence that
  // outgrows the kernel fails in its step, not here
  for (const hb_layer_desc& l : lv)
    if (l.mixer == HB_MIXER_GQA && gqa_attn_smem(l.dim, l.vdim, cfg_.use_cuda_graphs ? l.window : std::min(l.window, 256)) > 200 * 1024)
      return fail(HB_ERR_INVALID, "unsupported model description: the keys one position sees exceed the attention kernel's shared memory");
  CU(cudaSetDevice(cfg_.device));
  size_t free_b = 0, total_b = 0;
  CU(cudaMemGetInfo(&free_b, &total_b));
  budget_ = cfg_.memory_budget_bytes ? cfg_.memory_budget_bytes : (free_b > (1ull << 30) ? free_b - (1ull << 30) : free_b);
  model_.sd = sd;
  model_.sl.assign(layers, layers + sd.n_layers);
  hb_model_desc d{};
  d.arch = HB_ARCH_RISEPEL;
  d.hidden = sd.width;
  d.layers = sd.n_layers;
  d.vocab = sd.vocab;
  d.norm_eps = sd.norm_eps;
  d.max_pos = cfg_.max_ctx;
  model_.d = d;
  model_.arena_bytes = arena_bytes_for_stack(sd, layers);
  if (model_.arena_bytes > budget_) return fail(HB_ERR_OOM, "weights alone exceed the memory budget");
  if (model_.arena_bytes > free_b) return fail(HB_ERR_OOM, "weights exceed free device memory");
  CU(cudaMalloc(&model_.arena, model_.arena_bytes));
  CU(cudaMemset(model_.arena, 0, model_.arena_bytes));  // padding rows (routers below one MMA tile) must read as zero
  layout_stack(model_);
  load_open_ = true;
  return HB_OK;
}

int Engine::load_random_stack(const hb_stack_desc& sd, const hb_layer_desc* layers, uint64_t seed) {
  int rc = load_begin_stack(sd, layers);
  if (rc != HB_OK) return rc;
  std::lock_guard<std::mutex> g(gpu_mu_);
  CU(cudaSetDevice(cfg_.device));
  uint64_t k = 0;
  for (auto& kv : model_.placements) {
    const Placement& p = kv.second;
    const size_t n = p.rows * p.cols;
    // projections ~ U(+-sqrt(3/in)) so activations keep unit scale through any width; gains at their neutral value
    const float amp = p.is_norm_gain ? 0.f : (p.is_bias ? 0.1f : sqrtf(3.0f / (float)p.cols));
    const float mean = p.is_norm_gain ? p.fill : 0.f;
    const uint64_t sk = seed * 0x9E3779B97F4A7C15ull + (++k) * 0xD1B54A32D192ED03ull + std::hash<std::string>{}(kv.first);
    // [128 gate | 128 up] tiles: the gate and up placements share a base; random values need no interleaving, the up
    // tensor's share of the block is simply its second half
    bf16* dst = p.dst + (p.mode == 2 ? n : 0);
    const size_t ld = p.ld ? p.ld : p.cols;
    if (p.elem == 4) fill_uniform_kernel<float><<<148 * 4, 256, 0, stream_>>>((float*)p.dst, n, sk, amp, mean, p.cols, ld);
    else fill_uniform_kernel<bf16><<<148 * 4, 256, 0, stream_>>>(dst, n, sk, amp, mean, p.cols, ld);
    CU(cudaGetLastError());
    model_.filled[kv.first] = true;
  }
  CU(cudaStreamSynchronize(stream_));
  int rc2 = alloc_runtime();
  if (rc2 != HB_OK) return rc2;
  load_open_ = false;
  loaded_ = true;
  return HB_OK;
}

// ------------------------------------------------------------------ sizing
// fp32 partial slabs of the weight-streaming GEMM that serves steps of <= 256 tokens (every projection it may be given)
static size_t stack_skinny_floats(const Model& m) {
  size_t f = 0;
  auto shape = [&](size_t N, size_t K) { f = std::max(f, (size_t)gemm_skinny_max_segs((int)N, (int)K, 148) * 256 * N); };
  const size_t W = m.sd.width;
  for (int i = 0; i < m.sd.n_layers; ++i) {
    const hb_layer_desc& l = m.sl[i];
    shape(m.sw[i].n_in, W);
    shape(W, m.sw[i].o_cols ? (size_t)m.sw[i].o_cols : (size_t)l.heads * l.vdim);
    if (l.ff > 0 && l.ff_kind == HB_FF_RELU2) shape(l.ff, W);
    if (l.mixer == HB_MIXER_LATENT) shape((size_t)l.heads * (l.dim + l.rot_dim), l.q_rank);
    if (l.ff > 0) {
      shape(2 * (size_t)l.ff, W);
      shape(W, l.ff);
    }
    if (l.ff > 0 && l.ff_kind == HB_FF_MOE && l.shared_ff > 0) {
      shape(2 * (size_t)l.shared_ff, W);
      shape(W, l.shared_ff);
    }
  }
  shape(m.sd.vocab, W);
  return f;
}

// Dense-product attention (bf16 mode, prompt portions of >= kAttDenseMin tokens): capacity of one query block over all
// latent layers.  Returns false when no layer qualifies (row sizes that are not 16-byte multiples).
constexpr int kAttDenseMin = 64;
static bool stack_att_caps(const Model& m, int* qb, size_t* rows, size_t* keys, size_t* rmax, size_t* dmax, size_t* qa16) {
  *qb = 512; *rows = *keys = *rmax = *dmax = *qa16 = 0;
  if (m.sd.compute_f32) return false;
  bool any = false;
  for (const hb_layer_desc& l : m.sl) {
    if (l.mixer != HB_MIXER_LATENT || (l.kv_rank + l.rot_dim) % 8 || l.kv_rank % 8) continue;
    any = true;
    int q = 512;
    while (q > 64 && (size_t)q * l.heads * (l.window + q) * 4 > (size_t(64) << 20)) q /= 2;  // scores of a block <= 64 MB
    *qb = std::min(*qb, q);
  }
  if (!any) return false;
  for (const hb_layer_desc& l : m.sl) {
    if (l.mixer != HB_MIXER_LATENT || (l.kv_rank + l.rot_dim) % 8 || l.kv_rank % 8) continue;
    *rows = std::max(*rows, (size_t)*qb * l.heads);
    *keys = std::max(*keys, (size_t)(l.window + *qb + 7) / 8 * 8);
    *rmax = std::max(*rmax, (size_t)l.kv_rank);
    *dmax = std::max(*dmax, (size_t)l.kv_rank + l.rot_dim);
    *qa16 = std::max(*qa16, (size_t)l.heads * (l.kv_rank + l.rot_dim));
  }
  return true;
}

// widest buffers any layer needs (columns per token)
struct StackDims {
  int n1 = 0, n2 = 0, q = 0, qa = 0, cx = 0, mo = 0;
  int moe_r = 0, moe_top = 0, rope_half = 0;
  int gu = 0;                // widest [gate | up] row of a plain gated unit (bf16 intermediate of the tensor-core path)
  int att_heads = 0, att_dim = 0;  // ... and their most heads / widest head (split workspace of the decode kernel)
  int att = 0;               // grouped-query layers the fused tcgen05 attention takes: widest heads * vdim
  int moe_e = 0, moe_f = 0;  // grouped tensor-core experts: most experts / widest expert over the layers that qualify
  int vf = 0;                // layers that blend values: kv_heads * vdim
  bool shared = false;       // some mixture has a unit every token uses
  int cv = 0;                // widest convolved row (state-space layers, grouped-query layers with convolved projections)
  int ab = 0;                // most heads of a scalar-decay recurrence (decay, input weight, exp(-m), n . q per head and token)
};
// Grouped-query layers whose prompt portions run on the fused tcgen05 attention kernel (the one the Llama path uses, with
// the mask — blocks, a sliding window or plain causal —, the score cap and the sinks of the denominator as parameters): bf16
// mode, its head sizes, the pool's 64-position pages.
static bool gqa_fused_ok(const Model& m, const hb_layer_desc& l, int max_ctx) {
  static const bool off = [] { const char* e = getenv("HB_STACK_FUSED_ATTN"); return e && atoi(e) == 0; }();
  (void)max_ctx;
  return !off && !m.sd.compute_f32 && l.mixer == HB_MIXER_GQA && l.dim == l.vdim && (l.dim == 64 || l.dim == 128);
}
// experts run as grouped tcgen05 products when the mode and the shapes allow (16-byte TMA strides, at least one MMA tile)
static bool moe_grouped_ok(const Model& m, const hb_layer_desc& l) {
  static const bool off = [] { const char* e = getenv("HB_STACK_MOE_GROUPED"); return e && atoi(e) == 0; }();
  return !off && !m.sd.compute_f32 && l.ff > 0 && l.ff_kind == HB_FF_MOE && m.sd.width % 8 == 0 && l.ff % 8 == 0 && m.sd.width >= 64 &&
         l.ff >= 64;
}
static StackDims stack_dims(const Model& m, int max_ctx) {
  StackDims d;
  for (int i = 0; i < m.sd.n_layers; ++i) {
    const hb_layer_desc& l = m.sl[i];
    d.n1 = std::max(d.n1, std::max(m.sw[i].n_in, 2 * l.ff));
    d.mo = std::max(d.mo, std::max(l.heads * l.vdim, l.ff));
    if (l.ff > 0 && l.ff_kind == HB_FF_MOE && l.shared_ff > 0) {
      d.n1 = std::max(d.n1, 2 * l.shared_ff);
      d.mo = std::max(d.mo, l.shared_ff);
      d.gu = std::max(d.gu, 2 * l.shared_ff);
      d.shared = true;
    }
    d.mo = std::max(d.mo, m.sw[i].o_cols);
    if (l.ff > 0 && l.ff_kind == HB_FF_RELU2) d.gu = std::max(d.gu, l.ff);
    if (m.sw[i].ml.H > 0) {
      d.cx = std::max(d.cx, m.sw[i].ml.H * m.sw[i].ml.Dv);
      d.ab = std::max(d.ab, m.sw[i].ml.H);
    }
    if (l.mixer == HB_MIXER_MAMBA2) {
      d.cx = std::max(d.cx, l.heads * l.vdim);
      d.cv = std::max(d.cv, l.heads * l.vdim + 2 * l.kv_heads * l.dim);
      d.ab = std::max(d.ab, l.heads);
    } else if (l.mixer == HB_MIXER_MLSTM) {
    } else if (l.mixer == HB_MIXER_DELTA) {
      d.n2 = std::max(d.n2, 2 * l.kv_heads * l.dim + l.heads * l.vdim + 2 * l.heads + l.kv_heads);
      d.cx = std::max(d.cx, l.heads * l.vdim);
    } else if (l.mixer == HB_MIXER_GLA) {
      d.n2 = std::max(d.n2, l.heads * l.dim);
      d.cx = std::max(d.cx, l.heads * l.vdim);
    } else if (l.mixer == HB_MIXER_GQA) {
      d.n2 = std::max(d.n2, l.heads * l.dim);
      d.rope_half += l.rope_dims / 2;
      if (l.attn_flags & HB_ATTN_QKV_CONV) d.cv = std::max(d.cv, (l.heads + l.kv_heads) * l.dim + l.kv_heads * l.vdim);
      if ((l.attn_flags & HB_ATTN_OUT_GATE) || l.side_heads > 0) d.cx = std::max(d.cx, l.heads * l.vdim);
      if (l.attn_flags & HB_ATTN_V_BLEND) d.vf = std::max(d.vf, l.kv_heads * l.vdim);
      if (gqa_fused_ok(m, l, max_ctx)) {
        d.att = std::max(d.att, l.heads * l.vdim);
        d.att_heads = std::max(d.att_heads, l.heads);
        d.att_dim = std::max(d.att_dim, l.dim);
      }
    } else {
      d.n2 = std::max(d.n2, l.heads * (l.dim + l.rot_dim));
      d.q = std::max(d.q, l.q_rank);
      d.qa = std::max(d.qa, l.heads * (l.kv_rank + l.rot_dim));
      d.cx = std::max(d.cx, std::max(l.heads * l.kv_rank, l.heads * l.vdim));
    }
    if (l.ff > 0 && (l.ff_kind == HB_FF_GELU_TANH || l.ff_kind == HB_FF_SILU)) d.gu = std::max(d.gu, 2 * l.ff);
    if (l.ff > 0 && l.ff_kind == HB_FF_MOE) {
      d.moe_r = std::max(d.moe_r, l.experts + l.identity_experts);
      d.moe_top = std::max(d.moe_top, l.top_k);
      if (moe_grouped_ok(m, l)) {
        d.moe_e = std::max(d.moe_e, l.experts);
        d.moe_f = std::max(d.moe_f, l.ff);
      }
    }
  }
  return d;
}

size_t Engine::workspace_bytes_stack() const {
  const hb_stack_desc& sd = model_.sd;
  const size_t T = t_cap_, W = sd.width;
  const StackDims dm = stack_dims(model_, cfg_.max_ctx);
  const int n1 = dm.n1, n2 = dm.n2, q = dm.q, qa = dm.qa, cx = dm.cx, mo = dm.mo;
  size_t b = 0;
  b += al256((size_t)std::max(dm.rope_half, 1) * 8) + al256(T * 2 * (size_t)std::max(dm.rope_half, 1) * 4);
  if (dm.att > 0) b += al256(T * (size_t)up8(dm.att) * 2) + al256(attn_decode_workspace_floats(cfg_.max_seqs, dm.att_heads, dm.att_dim, 16) * 4);
  if (dm.moe_r > 0) {
    const size_t rows = dm.moe_e > 0 ? (size_t)moe_group_max_rows((int)T * dm.moe_top, dm.moe_e) : T * (size_t)dm.moe_top;
    b += al256(T * (size_t)std::max(64, up8(dm.moe_r)) * 4) + 2 * al256(T * (size_t)dm.moe_top * 4) + al256(T * (size_t)dm.moe_top * W * 4);
    if (dm.moe_e > 0)
      b += al256(T * (size_t)dm.moe_top * 4) + al256(rows * 4) + al256(rows / 128 * 4) + 2 * al256(rows * W * 2) + al256(rows * dm.moe_f * 2) +
           al256((size_t)3 * dm.moe_e * 4);
  }
  if (!sd.compute_f32) {
    const size_t rows = dm.moe_e > 0 ? (size_t)moe_group_max_rows((int)T * dm.moe_top, dm.moe_e) : 0;
    b += al256(std::max(T * (size_t)up8(dm.gu), rows * 2 * (size_t)dm.moe_f) * 2 + 256);
  }
  b += 2 * al256(T * W * 4) + al256(T * W * 2);                       // x, y, x16
  if (sd.norm_place == HB_NORM_BOTH_SIDES || sd.norm_place == HB_NORM_PARALLEL) b += al256(T * W * 4);     // hn
  if (sd.norm_place == HB_NORM_PARALLEL) b += al256(T * W * 4) + al256(T * W * 2);  // hn2, x16b
  if (dm.shared || sd.norm_place == HB_NORM_PARALLEL) b += al256(T * W * 4);                               // y2
  b += al256(T * (size_t)up8(dm.cv) * 4) + al256(T * (size_t)up8(4 * dm.ab) * 4);  // cv, ab
  if (dm.vf > 0) b += al256(T * (size_t)dm.vf * 4);                   // vfirst
  b += al256(T * (size_t)up8(n1) * 4) + al256(T * (size_t)up8(n2) * 4);  // p1, p2
  b += al256(T * (size_t)up8(q) * 4) + al256(T * (size_t)up8(q) * 2);     // cq, cq16
  b += al256(T * (size_t)up8(qa) * 4) + 2 * al256(T * (size_t)up8(cx) * 4);  // qabs, ctx (+ per-head value output)
  b += al256(T * (size_t)up8(mo) * 4) + al256(T * (size_t)up8(mo) * 2);   // mo, mo16
  b += al256((size_t)cfg_.max_seqs * sd.vocab * 4);                   // logits
  b += al256((size_t)cfg_.max_seqs * 4);                              // sampled
  b += al256(sample_scratch_bytes(cfg_.max_seqs, sd.vocab));
  b += 2 * al256((size_t)cfg_.max_seqs * HB_MAX_LOGPROBS * 4);
  if (!sd.compute_f32) b += al256(stack_skinny_floats(model_) * 4) + al256(T * (size_t)up8(n2) * 2) + al256(T * (size_t)up8(cx) * 2);
  {
    int qb; size_t rows, keys, rmax, dmax, qa16;
    if (stack_att_caps(model_, &qb, &rows, &keys, &rmax, &dmax, &qa16))
      b += al256(T * qa16 * 2) + al256(keys * dmax * 2) + al256(rmax * keys * 2) + al256(rows * keys * 2) + al256(rows * keys * 4);
  }
  return b;
}

int Engine::alloc_runtime_stack() {
  const hb_stack_desc& sd = model_.sd;
  cfg_.enable_prefix_cache = 0;  // a page of latent rows does not carry the recurrent layers' state of its prefix
  CU(stack_ops_init());
  CU(stack_gqa_init());
  CU(stack_moe_init());
  CU(stack_delta_init());
  CU(stack_ssm_init());
  if (!sd.compute_f32) {  // stream-K plans allocate on first use of a shape: make them now, not inside a graph capture
    SmLimitScope sm_scope(cfg_.sm_budget);
    SkinnyPlan pl{};
    for (int i = 0; i < sd.n_layers; ++i) {
      const hb_layer_desc& l = model_.sl[i];
      CU(gemm_skinny_plan(model_.sw[i].n_in, sd.width, &pl));
      CU(gemm_skinny_plan(sd.width, model_.sw[i].o_cols ? model_.sw[i].o_cols : l.heads * l.vdim, &pl));
      if (l.ff > 0 && l.ff_kind == HB_FF_RELU2) CU(gemm_skinny_plan(l.ff, sd.width, &pl));
      if (l.mixer == HB_MIXER_LATENT) CU(gemm_skinny_plan(l.heads * (l.dim + l.rot_dim), l.q_rank, &pl));
      if (l.ff > 0) {
        CU(gemm_skinny_plan(2 * l.ff, sd.width, &pl));
        CU(gemm_skinny_plan(sd.width, l.ff, &pl));
      }
      if (l.ff > 0 && l.ff_kind == HB_FF_MOE && l.shared_ff > 0) {
        CU(gemm_skinny_plan(2 * l.shared_ff, sd.width, &pl));
        CU(gemm_skinny_plan(sd.width, l.shared_ff, &pl));
      }
    }
    CU(gemm_skinny_plan(sd.vocab, sd.width, &pl));
  }
  t_cap_ = cfg_.max_batched_tokens;
  b_cap_ = cfg_.max_seqs;
  max_pages_per_seq_ = (cfg_.max_ctx + page_ - 1) / page_;
  ws_bytes_ = workspace_bytes_stack();
  CU(cudaMalloc(&ws_, ws_bytes_));
  uint8_t* p = ws_;
  auto take = [&](size_t bytes) {
    uint8_t* r = p;
    p += al256(bytes);
    return r;
  };
  const size_t T = t_cap_, W = sd.width;
  const StackDims dm = stack_dims(model_, cfg_.max_ctx);
  const int n1 = dm.n1, n2 = dm.n2, q = dm.q, qa = dm.qa, cx = dm.cx, mo = dm.mo;
  {  // rotation frequencies of the grouped-query layers (double precision, formed on the host)
    double* fq = (double*)take((size_t)std::max(dm.rope_half, 1) * 8);
    float* cs = (float*)take(T * 2 * (size_t)std::max(dm.rope_half, 1) * 4);
    sk_.layer_set.assign(sd.n_layers, -1);
    sk_.freq_sets.clear(); sk_.freq_half.clear(); sk_.rope_cs.clear();
    std::vector<std::vector<double>> sets;
    size_t at = 0;
    for (int i = 0; i < sd.n_layers; ++i) {
      const hb_layer_desc& l = model_.sl[i];
      if (l.mixer != HB_MIXER_GQA || l.rope_dims <= 0) continue;
      const std::vector<double> f = stack_rope_freqs(l);
      size_t sidx = 0;
      while (sidx < sets.size() && sets[sidx] != f) ++sidx;
      if (sidx == sets.size()) {
        CU(cudaMemcpy(fq + at, f.data(), f.size() * 8, cudaMemcpyHostToDevice));
        sets.push_back(f);
        sk_.freq_sets.push_back(fq + at);
        sk_.freq_half.push_back((int)f.size());
        sk_.rope_cs.push_back(cs + T * 2 * at);
        at += f.size();
      }
      sk_.layer_set[i] = (int)sidx;
    }
  }
  if (dm.att > 0) {
    sk_.ldatt = up8(dm.att);
    sk_.att16 = (bf16*)take(T * (size_t)sk_.ldatt * 2);
    sk_.dec_ws = (float*)take(attn_decode_workspace_floats(cfg_.max_seqs, dm.att_heads, dm.att_dim, 16) * 4);
  }
  if (dm.moe_r > 0) {
    sk_.ldz = std::max(64, up8(dm.moe_r));
    sk_.moe_z = (float*)take(T * (size_t)sk_.ldz * 4);
    sk_.moe_ids = (int32_t*)take(T * (size_t)dm.moe_top * 4);
    sk_.moe_w = (float*)take(T * (size_t)dm.moe_top * 4);
    const size_t rows = dm.moe_e > 0 ? (size_t)moe_group_max_rows((int)T * dm.moe_top, dm.moe_e) : T * (size_t)dm.moe_top;
    sk_.moe_y = (float*)take(T * (size_t)dm.moe_top * W * 4);  // per-item outputs of the GEMV path
    if (dm.moe_e > 0) {
      sk_.moe_rows = (int)rows;
      sk_.moe_row_of = (int32_t*)take(T * (size_t)dm.moe_top * 4);
      sk_.moe_src = (int32_t*)take(rows * 4);
      sk_.moe_tiles = (int32_t*)take(rows / 128 * 4);
      sk_.moe_a16 = (bf16*)take(rows * W * 2);
      sk_.moe_h16 = (bf16*)take(rows * dm.moe_f * 2);
      sk_.moe_y16 = (bf16*)take(rows * W * 2);
      sk_.moe_scratch = (int32_t*)take((size_t)3 * dm.moe_e * 4);
    }
  }
  if (!sd.compute_f32) {
    const size_t rows = dm.moe_e > 0 ? (size_t)moe_group_max_rows((int)T * dm.moe_top, dm.moe_e) : 0;
    sk_.gu16 = (bf16*)take(std::max(T * (size_t)up8(dm.gu), rows * 2 * (size_t)dm.moe_f) * 2 + 256);
  }
  sk_.ld1 = up8(n1); sk_.ld2 = up8(n2); sk_.ldcq = up8(q); sk_.ldqa = up8(qa); sk_.ldctx = up8(cx); sk_.ldmo = up8(mo);
  sk_.x = (float*)take(T * W * 4);
  sk_.y = (float*)take(T * W * 4);
  sk_.x16 = (bf16*)take(T * W * 2);
  const bool par = sd.norm_place == HB_NORM_PARALLEL;
  sk_.hn = (sd.norm_place == HB_NORM_BOTH_SIDES || par) ? (float*)take(T * W * 4) : nullptr;
  sk_.hn2 = par ? (float*)take(T * W * 4) : nullptr;
  sk_.x16b = par ? (bf16*)take(T * W * 2) : nullptr;
  sk_.y2 = (dm.shared || par) ? (float*)take(T * W * 4) : nullptr;
  sk_.ldcv = up8(dm.cv); sk_.ldab = up8(4 * dm.ab); sk_.ab_heads = dm.ab;
  sk_.cv = (float*)take(T * (size_t)sk_.ldcv * 4);
  sk_.ab = (float*)take(T * (size_t)sk_.ldab * 4);
  sk_.vfirst = dm.vf > 0 ? (float*)take(T * (size_t)dm.vf * 4) : nullptr;
  sk_.p1 = (float*)take(T * (size_t)sk_.ld1 * 4);
  sk_.p2 = (float*)take(T * (size_t)sk_.ld2 * 4);
  sk_.cq = (float*)take(T * (size_t)sk_.ldcq * 4);
  sk_.cq16 = (bf16*)take(T * (size_t)sk_.ldcq * 2);
  sk_.qabs = (float*)take(T * (size_t)sk_.ldqa * 4);
  sk_.ctx = (float*)take(2 * al256(T * (size_t)sk_.ldctx * 4));
  sk_.mo = (float*)take(T * (size_t)sk_.ldmo * 4);
  sk_.mo16 = (bf16*)take(T * (size_t)sk_.ldmo * 2);
  logits_ = (float*)take((size_t)cfg_.max_seqs * sd.vocab * 4);
  sampled_ = (int32_t*)take((size_t)cfg_.max_seqs * 4);
  sample_ws_ = take(sample_scratch_bytes(cfg_.max_seqs, sd.vocab));
  lp_ids_ = (int32_t*)take((size_t)cfg_.max_seqs * HB_MAX_LOGPROBS * 4);
  lp_vals_ = (float*)take((size_t)cfg_.max_seqs * HB_MAX_LOGPROBS * 4);
  skinny_ws_ = sd.compute_f32 ? nullptr : (float*)take(stack_skinny_floats(model_) * 4);
  if (!sd.compute_f32) {
    sk_.q16 = (bf16*)take(T * (size_t)sk_.ld2 * 2);
    sk_.ctx16 = (bf16*)take(T * (size_t)sk_.ldctx * 2);
    for (int i = 0; i < sd.n_layers; ++i) {  // per-head transposed key up-projections (arena slots without a checkpoint tensor)
      const hb_layer_desc& l = model_.sl[i];
      if (l.mixer == HB_MIXER_LATENT && model_.sw[i].ukT)
        CU(transpose_heads_bf16(stream_, (const bf16*)model_.sw[i].uk, (bf16*)model_.sw[i].ukT, l.heads, l.dim, l.kv_rank));
    }
    CU(cudaStreamSynchronize(stream_));
  }
  {
    int qb; size_t rows, keys, rmax, dmax, qa16;
    if (stack_att_caps(model_, &qb, &rows, &keys, &rmax, &dmax, &qa16)) {
      sk_.att_qb = qb; sk_.att_rows = rows; sk_.att_keys = keys;
      sk_.qabs16 = (bf16*)take(T * qa16 * 2);
      sk_.kbuf = (bf16*)take(keys * dmax * 2);
      sk_.ct = (bf16*)take(rmax * keys * 2);
      sk_.P = (bf16*)take(rows * keys * 2);
      sk_.S = (float*)take(rows * keys * 4);
    }
  }

  pen_cap_ = std::min<size_t>((size_t)cfg_.max_seqs * cfg_.max_ctx, size_t(4) << 20);
  step_bytes_ = layout(t_cap_, b_cap_, pen_cap_).total;
  CU(cudaMalloc(&d_step_, step_bytes_));
  CU(cudaMallocHost(&h_step_, step_bytes_));
  CU(cudaMallocHost(&h_sampled_, (size_t)b_cap_ * 4));
  CU(cudaMallocHost(&h_lp_ids_, (size_t)cfg_.max_seqs * HB_MAX_LOGPROBS * 4));
  CU(cudaMallocHost(&h_lp_vals_, (size_t)cfg_.max_seqs * HB_MAX_LOGPROBS * 4));

  // recurrent state: one slot per admissible sequence
  const size_t state_bytes = (size_t)cfg_.max_seqs * std::max<size_t>(model_.state_floats, 1) * 4;
  CU(cudaMalloc(&state_, state_bytes));
  CU(cudaMemsetAsync(state_, 0, state_bytes, stream_));
  free_slots_.resize(cfg_.max_seqs);
  for (int i = 0; i < cfg_.max_seqs; ++i) free_slots_[i] = cfg_.max_seqs - 1 - i;

  // latent pool: every plane holds num_pages pages of page_ rows; one page id addresses the same positions in all planes
  uint64_t page_bytes = 0;
  for (int r : model_.plane_row) page_bytes += (uint64_t)page_ * r * model_.elem;
  page_bytes = std::max<uint64_t>(page_bytes, 16);
  const uint64_t used = model_.arena_bytes + ws_bytes_ + step_bytes_ + state_bytes;
  if (used >= budget_) return fail(HB_ERR_OOM, "weights + workspace exceed the memory budget");
  size_t free_b = 0, total_b = 0;
  CU(cudaMemGetInfo(&free_b, &total_b));
  uint64_t avail = std::min<uint64_t>(budget_ - used, free_b > (256ull << 20) ? free_b - (256ull << 20) : 0);
  uint64_t pages = avail / page_bytes;
  const uint64_t want = (uint64_t)cfg_.max_seqs * max_pages_per_seq_;
  if (pages > want) pages = want;
  if (cfg_.kv_pool_tokens > 0) pages = std::min<uint64_t>(pages, std::max<uint64_t>((cfg_.kv_pool_tokens + page_ - 1) / page_, max_pages_per_seq_));
  if (pages < (uint64_t)max_pages_per_seq_) return fail(HB_ERR_OOM, "memory budget leaves no room for one full-context sequence of cache");
  num_pages_ = (int)pages;
  kv_bytes_ = pages * page_bytes;
  CU(cudaMalloc(&kv_, kv_bytes_));
  CU(cudaMemsetAsync(kv_, 0, kv_bytes_, stream_));
  CU(cudaStreamSynchronize(stream_));
  plane_off_.clear();
  size_t off = 0;
  for (int r : model_.plane_row) {
    plane_off_.push_back(off);
    off += (size_t)num_pages_ * page_ * r * model_.elem;
  }
  pmeta_.assign(num_pages_, PageMeta{});
  cache_.clear();
  lru_.clear();
  free_pages_.resize(num_pages_);
  for (int i = 0; i < num_pages_; ++i) free_pages_[i] = num_pages_ - 1 - i;
  return HB_OK;
}

int Engine::take_slot() {
  if (free_slots_.empty()) return -1;
  const int s = free_slots_.back();
  free_slots_.pop_back();
  return s;
}
void Engine::drop_slot(Request* r) {
  if (r->state_slot >= 0) free_slots_.push_back(r->state_slot);
  r->state_slot = -1;
}

// ------------------------------------------------------------------ forward
bool Engine::stack_tc(int N, int K, int lda, int ldc) const {
  static const bool simt_only = [] { const char* e = getenv("HB_STACK_SIMT"); return e && atoi(e) != 0; }();
  return !model_.sd.compute_f32 && !simt_only && K % 8 == 0 && lda % 8 == 0 && K >= 64 && N >= 64 && ldc % 4 == 0;
}

int Engine::stack_gemm(const float* A, const bf16* A16, int lda, const void* Wt, int N, int K, float* C, int ldc, int M, const void* bias) {
  const bool f32 = model_.sd.compute_f32 != 0;
  static const bool simt_only = [] { const char* e = getenv("HB_STACK_SIMT"); return e && atoi(e) != 0; }();  // A/B and bring-up
  const double flops = 2.0 * M * N * K;
  const bool tc = !f32 && !simt_only && A16 && !bias && K % 8 == 0 && lda % 8 == 0 && K >= 64 && N >= 64;
  static const bool no_skinny = [] { const char* e = getenv("HB_STACK_SKINNY"); return e && atoi(e) == 0; }();
  if (tc && M <= 256 && skinny_ws_ && !no_skinny) {
    // steps of a few tokens (decoding): the weights are the MMA's M operand and stream through every SM once (stream-K over
    // (tile, k-block) units, fp32 slabs summed in slab order: the result does not depend on who finishes first)
    SkinnyPlan plan{};
    CU(gemm_skinny_plan(N, K, &plan));
    if (gemm_skinny_ws_floats(plan, M, N) <= stack_skinny_floats(model_)) {
      SPAN(4, 2.0 * N * K + 2.0 * M * K + 4.0 * M * N, gemm_skinny(stream_, plan, A16, lda, (const bf16*)Wt, K, skinny_ws_, M, N, K));
      SPAN(3, 8.0 * M * N, dec_sum_slabs(stream_, skinny_ws_, plan, C, ldc, M, N));
      return HB_OK;
    }
  }
  if (tc && ldc % 4 == 0) {
    GemmArgs g{A16, lda, (const bf16*)Wt, K, C, ldc, nullptr, 0, nullptr, M, N, K, EPI_F32, 0};
    SPAN(0, flops, gemm_bf16_tn(stream_, g));
    return HB_OK;
  }
  GemmRtArgs g{A, lda, 0, Wt, K, 1, 0, C, ldc, 0, bias, M, N, K, 1, f32};
  SPAN(5, flops, gemm_rt(stream_, g));
  return HB_OK;
}

int Engine::forward_stack(int T, int B, const StepLayout& L, const int32_t* extra_rows, int n_extra, float* extra_out, bool sample) {
  const hb_stack_desc& sd = model_.sd;
  const bool f32 = sd.compute_f32 != 0;
  const int W = sd.width, V = sd.vocab;
  const int32_t* tokens = (const int32_t*)(d_step_ + L.tokens);
  const int32_t* positions = (const int32_t*)(d_step_ + L.positions);
  const int32_t* slots = (const int32_t*)(d_step_ + L.slots);
  const int32_t* cu = (const int32_t*)(d_step_ + L.cu);
  const int32_t* last = (const int32_t*)(d_step_ + L.last);
  const int32_t* pt = (const int32_t*)(d_step_ + L.pt);
  const int32_t* sslot = (const int32_t*)(d_step_ + L.sslot);
  const int32_t* first = (const int32_t*)(d_step_ + L.first);
  const int32_t* seqof = (const int32_t*)(d_step_ + L.seqof);
  StackWs& k = sk_;
  bf16* x16 = f32 ? nullptr : k.x16;
  bf16* cq16 = f32 ? nullptr : k.cq16;
  bf16* mo16 = f32 ? nullptr : k.mo16;
  const double rowb = 4.0 * T * W;

  const float goff = sd.plain_gains ? 0.f : 1.f;  // stored norm gains are offsets from one unless plain
  const bool both = sd.norm_place == HB_NORM_BOTH_SIDES, tnorm = sd.norm_kind == HB_NORM_TANH;
  const bool par = sd.norm_place == HB_NORM_PARALLEL;
  // what a sublayer reads: the stream itself, or (norms on both sides, parallel sublayers) its normed copy; x16 is the bf16
  // copy of that.  With parallel sublayers the feed-forward has a normed copy of its own (hn2 / x16b).
  const float* xin = (both || par) ? k.hn : k.x;
  const float* ff_in = par ? k.hn2 : xin;
  const bf16* ff_in16 = par ? (f32 ? nullptr : k.x16b) : x16;
  // parallel sublayers: x += mixer + feed-forward (+ bias), and the two normed inputs of the layer `next` (none behind the last)
  auto par_step = [&](const float* y, const float* y2, const void* bias, float bias_scale, int next) -> cudaError_t {
    const void* w1 = next < sd.n_layers ? model_.sw[next].norm1 : nullptr;
    const void* w2 = next < sd.n_layers && model_.sl[next].ff > 0 ? model_.sw[next].norm2 : nullptr;
    // the fp32 copies are written only where a product of the next layer reads them (shapes the tensor-core GEMMs do not take)
    bool h1_f32 = true, h2_f32 = true;
    if (next < sd.n_layers) {
      const hb_layer_desc& nl = model_.sl[next];
      const int n_in = model_.sw[next].n_in;
      h1_f32 = !stack_tc(n_in, W, W, nl.mixer == HB_MIXER_GQA ? up8(n_in) : k.ld1);
      h2_f32 = !stack_tc(nl.ff_kind == HB_FF_RELU2 ? nl.ff : 2 * nl.ff, W, W, k.ld1);
    }
    return parallel_step(stream_, k.x, nullptr, y, y2, bias, bias_scale, w1, w2, f32, sd.norm_eps, y ? k.x : nullptr, h1_f32 ? k.hn : nullptr, x16,
                         h2_f32 ? k.hn2 : nullptr, f32 ? nullptr : k.x16b, T, W);
  };
  // the residual step: the norm covers the sum (post-norm stream) or the sublayer's output alone; with norms on both sides
  // the same launch also norms the input of the sublayer that follows (`pre`, null behind the last one)
  auto resid = [&](const void* bias, const void* gain, const void* pre) -> cudaError_t {
    if (tnorm) {
      cudaError_t e = tanh_norm_step(stream_, k.x, nullptr, k.y, W, gain, both ? pre : nullptr, f32, k.x, both && pre ? k.hn : nullptr,
                                     both && pre ? x16 : nullptr, T, W);
      if (e == cudaSuccess && !both && x16) e = to_bf16_rows(stream_, k.x, W, x16, W, T, W);
      return e;
    }
    if (both) {
      cudaError_t e = resid_add_normed(stream_, k.x, nullptr, k.y, W, bias, gain, f32, goff, sd.norm_eps, T, W);
      if (e == cudaSuccess && pre) e = norm_rows_f32(stream_, k.x, nullptr, pre, f32, goff, sd.norm_eps, k.hn, x16, T, W);
      return e;
    }
    if (sd.norm_place == HB_NORM_OF_OUTPUT) return resid_add_normed(stream_, k.x, x16, k.y, W, bias, gain, f32, goff, sd.norm_eps, T, W);
    return resid_postnorm(stream_, k.x, x16, k.y, W, bias, gain, f32, sd.resid_alpha, goff, sd.norm_eps, T, W);
  };
  // a row norm outside the residual step (embedding, first sublayer's input, final norm)
  auto norm_rows = [&](const float* src, const int32_t* idx, const void* nw, float* out, bf16* out16, int rows) -> cudaError_t {
    if (tnorm) return tanh_norm_step(stream_, src, idx, nullptr, 0, nullptr, nw, f32, nullptr, out, out16, rows, W);
    return norm_rows_f32(stream_, src, idx, nw, f32, goff, sd.norm_eps, out, out16, rows, W);
  };
  // gated unit y = down(act(gate) * up) of inner size F from the sublayer's input (dense feed-forwards, the unit every token
  // of a mixture uses).  Steps of many tokens: both products on the tcgen05 GEMM, the gated pair applied on the accumulators'
  // way out (packed [128 gate | 128 up] weight tiles) or on the bf16 [gate | up] rows between them.
  auto gated_ff = [&](const void* w_gu, const void* w_down, int F, int act, float limit, bool packed, float* out) -> int {
    int rc;
    if (T > 256 && k.gu16 && F % 8 == 0 && stack_tc(2 * F, W, W, W) && stack_tc(W, F, F, W)) {
      if (packed) {
        GemmArgs g{ff_in16, W, (const bf16*)w_gu, W, mo16, F, nullptr, 0, nullptr, T, 2 * F, W,
                   act == GLU_GELU_TANH ? EPI_GEGLU : (act == GLU_CLAMPED ? EPI_CLAMPGLU : EPI_SWIGLU), 0};
        g.glu_limit = limit;
        SPAN(0, 4.0 * T * F * W, gemm_bf16_tn(stream_, g));
      } else {
        GemmArgs g{ff_in16, W, (const bf16*)w_gu, W, k.gu16, 2 * F, nullptr, 0, nullptr, T, 2 * F, W, EPI_NONE, 0};
        SPAN(0, 4.0 * T * F * W, gemm_bf16_tn(stream_, g));
        SPAN(3, 6.0 * T * F, gated_unit_b16(stream_, k.gu16, 2 * F, act, mo16, T, F, limit));
      }
    } else {
      rc = stack_gemm(ff_in, ff_in16, W, w_gu, 2 * F, W, k.p1, k.ld1, T);
      if (rc != HB_OK) return rc;
      SPAN(3, 12.0 * T * F, gated_unit(stream_, k.p1, k.ld1, act, k.mo, mo16, T, F, packed, limit));
    }
    return stack_gemm(k.mo, mo16, F, w_down, W, F, out, W, T);
  };
  // ungated unit y = down(relu(up h)^2)
  auto relu2_ff = [&](const void* w_up, const void* w_down, int F, float* out) -> int {
    if (T > 256 && k.gu16 && F % 8 == 0 && stack_tc(F, W, W, F) && stack_tc(W, F, F, W)) {
      GemmArgs g{ff_in16, W, (const bf16*)w_up, W, mo16, F, nullptr, 0, nullptr, T, F, W, EPI_RELU2, 0};
      SPAN(0, 2.0 * T * F * W, gemm_bf16_tn(stream_, g));
    } else {
      int rc = stack_gemm(ff_in, ff_in16, W, w_up, F, W, k.p1, k.ld1, T);
      if (rc != HB_OK) return rc;
      SPAN(3, 10.0 * T * F, relu2_rows(stream_, k.p1, k.ld1, k.mo, mo16, T, F));
    }
    return stack_gemm(k.mo, mo16, F, w_down, W, F, out, W, T);
  };
  // a matrix memory over the columns of the layer's fused projection (row stride ldin): gates and their running maximum,
  // the recurrence, then normalisation, per-head unit RMS, gain, sigmoid gate and `scale` into columns col0.. of the output
  // projection's input (row stride ldout)
  auto run_memory = [&](const StackLayerW& w, int ldin, int col0, int ldout, float scale, float* out_f32) -> int {
    const MlstmW& q = w.ml;
    GateScanArgs ga{};
    ga.p = k.p1; ga.ldp = ldin; ga.off_i = q.off_i; ga.off_f = q.off_f; ga.bias = w.b_in; ga.f32 = f32; ga.cap = q.cap;
    ga.ab = k.ab; ga.ldab = k.ldab;
    ga.state = state_; ga.slot_stride = (long)model_.state_floats; ga.m_off = q.m_off;
    ga.cu = cu; ga.first_pos = first; ga.slots = sslot; ga.B = B; ga.H = q.H;
    SPAN(3, 24.0 * T * q.H, exp_gate_scan(stream_, ga));
    LinRecArgs ra{};
    ra.q = k.p1; ra.ldq = ldin; ra.q_off = q.off_q;
    ra.k = k.p1; ra.ldk = ldin; ra.k_off = q.off_k;
    ra.v = k.p1; ra.ldv = ldin; ra.v_off = q.off_v;
    ra.ab = k.ab; ra.ldab = k.ldab;
    ra.out = k.ctx; ra.ldo = k.ldctx;
    ra.nq = k.ab + 3 * q.H; ra.ldn = k.ldab;
    ra.skip = nullptr; ra.f32 = f32; ra.q_scale = 1.0f / sqrtf((float)q.D);
    ra.state = state_; ra.slot_stride = (long)model_.state_floats; ra.s_off = q.state_off; ra.n_off = q.n_off;
    ra.cu = cu; ra.first_pos = first; ra.slots = sslot;
    ra.B = B; ra.H = q.H; ra.G = q.H; ra.Dk = q.D; ra.Dv = q.Dv;
    SPAN(6, 4.0 * T * q.H * q.D * q.Dv, lin_recurrence(stream_, ra));
    SPAN(3, 16.0 * T * q.H * q.Dv, memory_readout(stream_, k.ctx, k.ldctx, k.ab + 3 * q.H, k.ldab, k.ab, k.ldab, k.p1 + q.off_g, ldin, q.hnorm, f32,
                                                  sd.norm_eps, scale, out_f32, mo16, ldout, col0, T, q.H, q.Dv));
    return HB_OK;
  };
  SPAN(3, rowb, embed_rows_f32(stream_, tokens, model_.s_embed, f32, k.x, x16, T, W, sd.embed_scale != 0.f ? sd.embed_scale : 1.f));
  if (sd.embed_norm) SPAN(3, 2 * rowb, norm_rows(k.x, nullptr, model_.s_embed_norm, k.x, both ? nullptr : x16, T));
  if (both) SPAN(3, 2 * rowb, norm_rows(k.x, nullptr, model_.sw[0].norm1, k.hn, x16, T));
  if (par) SPAN(3, 3 * rowb, par_step(nullptr, nullptr, nullptr, 0.f, 0));
  for (size_t si = 0; si < k.freq_sets.size(); ++si)  // cos / sin of the step's positions, once per distinct rotation
    SPAN(3, 8.0 * T * k.freq_half[si], stack_rope_table(stream_, positions, k.freq_sets[si], k.freq_half[si], k.rope_cs[si], T));
  for (int i = 0; i < sd.n_layers; ++i) {
    const hb_layer_desc& l = model_.sl[i];
    const StackLayerW& w = model_.sw[i];
    const int H = l.heads, Dk = l.dim, Dv = l.vdim;
    // every projection that reads the stream, in one GEMM
    // (grouped-query layers keep the rows of this product dense: the buffer's stride is sized for the widest gated unit)
    const int ldin = l.mixer == HB_MIXER_GQA ? up8(w.n_in) : k.ld1;
    int rc = stack_gemm(xin, x16, W, w.w_in, w.n_in, W, k.p1, ldin, T);
    if (rc != HB_OK) return rc;
    // the norm that prepares the input of whatever follows a sublayer (norms on both sides)
    const void* pre_next = i + 1 < sd.n_layers ? model_.sw[i + 1].norm1 : nullptr;
    const int ocols = w.o_cols ? w.o_cols : H * Dv;  // columns of the output projection (both mixers' when there are two)
    float* mo_f32 = stack_tc(W, ocols, ocols, W) ? nullptr : k.mo;  // the output projection's fp32 input, when it reads one
    if (l.mixer == HB_MIXER_MAMBA2) {
      const int G = l.kv_heads, N = Dk, inner = H * Dv, C = inner + 2 * G * N;
      ConvArgs ca{};
      ca.in = k.p1; ca.ldi = k.ld1; ca.off = w.off_v; ca.in_bias = nullptr; ca.bias_off = 0;
      ca.w = w.conv_w; ca.bias = w.conv_b; ca.f32 = f32; ca.taps = l.conv_taps; ca.act = 1;
      ca.out = k.cv; ca.ldo = k.ldcv;
      ca.state = state_; ca.slot_stride = (long)model_.state_floats; ca.tail_off = w.tail_off;
      ca.cu = cu; ca.first_pos = first; ca.slots = sslot; ca.seq_of = seqof; ca.T = T; ca.B = B; ca.C = C;
      SPAN(3, 4.0 * T * C * (l.conv_taps + 1), short_conv(stream_, ca));
      SPAN(3, 8.0 * B * C * l.conv_taps, conv_tails(stream_, ca));
      SPAN(3, 12.0 * T * H, ssm_steps(stream_, k.p1, k.ld1, w.off_a, w.a_dt, f32, k.ab, k.ldab, T, H));
      LinRecArgs ra{};
      ra.q = k.cv; ra.ldq = k.ldcv; ra.q_off = inner + G * N;
      ra.k = k.cv; ra.ldk = k.ldcv; ra.k_off = inner;
      ra.v = k.cv; ra.ldv = k.ldcv; ra.v_off = 0;
      ra.ab = k.ab; ra.ldab = k.ldab;
      ra.out = k.ctx; ra.ldo = k.ldctx;
      ra.nq = nullptr; ra.ldn = 0;
      ra.skip = (const uint8_t*)w.a_dt + (size_t)2 * H * model_.elem; ra.f32 = f32; ra.q_scale = 1.f;
      ra.state = state_; ra.slot_stride = (long)model_.state_floats; ra.s_off = w.state_off; ra.n_off = 0;
      ra.cu = cu; ra.first_pos = first; ra.slots = sslot;
      ra.B = B; ra.H = H; ra.G = G; ra.Dk = N; ra.Dv = Dv;
      SPAN(6, 4.0 * T * H * N * Dv, lin_recurrence(stream_, ra));
      SPAN(3, 16.0 * T * inner, gated_group_norm(stream_, k.ctx, k.ldctx, k.p1 + w.off_g, k.ld1, w.hnorm, f32, sd.norm_eps, l.norm_groups, mo_f32,
                                                 mo16, T, inner));
    } else if (l.mixer == HB_MIXER_MLSTM) {
      rc = run_memory(w, k.ld1, 0, ocols, 1.f, mo_f32);
      if (rc != HB_OK) return rc;
    } else if (l.mixer == HB_MIXER_DELTA) {
      const int G = l.kv_heads, GD = G * Dk, C = 2 * GD + H * Dv;
      DeltaPrepArgs pa{};
      pa.p = k.p1; pa.ldp = k.ld1; pa.off_qkv = w.off_q; pa.off_b = w.off_b; pa.off_a = w.off_a;
      pa.conv_w = w.conv_w; pa.a_dt = w.a_dt; pa.f32 = f32; pa.taps = l.conv_taps;
      pa.out = k.p2; pa.ldo = k.ld2;
      pa.state = state_; pa.slot_stride = (long)model_.state_floats; pa.tail_off = w.tail_off;
      pa.cu = cu; pa.first_pos = first; pa.slots = sslot; pa.seq_of = seqof;
      pa.T = T; pa.B = B; pa.H = H; pa.G = G; pa.D = Dk; pa.Dv = Dv;
      SPAN(3, 8.0 * T * C * (l.conv_taps + 1), delta_prep(stream_, pa));
      SPAN(3, 8.0 * B * C * l.conv_taps, delta_conv_tails(stream_, pa));
      DeltaArgs da{};
      da.in = k.p2; da.ld = k.ld2;
      da.off_q = 0; da.off_k = GD; da.off_v = 2 * GD; da.off_beta = C; da.off_decay = C + H; da.off_kq = C + 2 * H;
      da.out = k.ctx; da.ldo = k.ldctx;
      da.state = state_ + w.state_off; da.slot_stride = (long)model_.state_floats;
      da.cu = cu; da.first_pos = first; da.slots = sslot;
      da.B = B; da.H = H; da.G = G; da.D = Dk; da.Dv = Dv;
      SPAN(6, 6.0 * T * H * Dk * Dv, delta_recurrence(stream_, da));
      SPAN(3, 12.0 * T * H * Dv, headnorm_silu_gate(stream_, k.ctx, k.ldctx, k.p1 + w.off_g, k.ld1, w.hnorm, f32, sd.norm_eps, k.mo, mo16, T, H, Dv));
    } else if (l.mixer == HB_MIXER_GLA) {
      // decay: z = a2 (a1 x) + b -> sigmoid(z)^(1/tau), fp32
      rc = stack_gemm(k.p1 + w.off_a1, nullptr, k.ld1, w.a2, H * Dk, l.decay_rank, k.p2, k.ld2, T);
      if (rc != HB_OK) return rc;
      SPAN(3, 8.0 * T * H * Dk, gla_decay(stream_, k.p2, k.ld2, w.a2b, f32, l.tau, T, H * Dk));
      GlaArgs a{};
      a.q = k.p1 + w.off_q; a.k = k.p1 + w.off_k; a.v = k.p1 + w.off_v; a.ld = k.ld1;
      a.decay = k.p2; a.ldd = k.ld2;
      a.out = k.ctx; a.ldo = k.ldctx;
      a.state = state_ + w.state_off; a.slot_stride = (long)model_.state_floats;
      a.cu = cu; a.first_pos = first; a.slots = sslot;
      a.B = B; a.H = H; a.Dk = Dk; a.Dv = Dv;
      a.q_scale = 1.0f / sqrtf((float)Dk);
      SPAN(6, 4.0 * T * H * Dk * Dv, gla_recurrence(stream_, a));
      SPAN(3, 12.0 * T * H * Dv, headnorm_silu_gate(stream_, k.ctx, k.ldctx, k.p1 + w.off_g, k.ld1, w.hnorm, f32, sd.norm_eps, k.mo, mo16, T, H, Dv));
    } else if (l.mixer == HB_MIXER_GQA) {
      const int G = l.kv_heads;
      void* kplane = (uint8_t*)kv_ + plane_off_[w.cache_plane];
      void* vplane = (uint8_t*)kv_ + plane_off_[w.cache_plane_v];
      GqaPrepArgs pa{};
      pa.p = k.p1; pa.ldp = ldin; pa.q_off = w.off_q; pa.k_off = w.off_k; pa.v_off = w.off_v;
      const bool conv = (l.attn_flags & HB_ATTN_QKV_CONV) != 0;
      if (conv) {
        // q | k | v columns (biases added on the way in) through their short convolutions; what follows reads the convolved rows
        const int C = (H + G) * Dk + G * Dv;
        ConvArgs ca{};
        ca.in = k.p1; ca.ldi = ldin; ca.off = w.off_q;
        ca.in_bias = (l.attn_flags & HB_ATTN_QKV_BIAS) ? w.b_in : nullptr; ca.bias_off = w.off_q;
        ca.w = w.conv_w; ca.bias = nullptr; ca.f32 = f32; ca.taps = l.conv_taps; ca.act = 0;
        ca.out = k.cv; ca.ldo = k.ldcv;
        ca.state = state_; ca.slot_stride = (long)model_.state_floats; ca.tail_off = w.tail_off;
        ca.cu = cu; ca.first_pos = first; ca.slots = sslot; ca.seq_of = seqof; ca.T = T; ca.B = B; ca.C = C;
        SPAN(3, 4.0 * T * C * (l.conv_taps + 1), short_conv(stream_, ca));
        SPAN(3, 8.0 * B * C * l.conv_taps, conv_tails(stream_, ca));
        pa.p = k.cv; pa.ldp = k.ldcv; pa.q_off = 0; pa.k_off = H * Dk; pa.v_off = (H + G) * Dk;
      }
      // an entry-wise output gate or a second mixer: the attention output passes one more kernel on its way to the output
      // projection's input (gate, weight of the mixer, its columns of the concatenated row)
      const bool post = (l.attn_flags & HB_ATTN_OUT_GATE) || w.ml.H > 0;
      const float mix_scale = l.mix_scale != 0.f ? l.mix_scale : 1.f;
      // prompt portions (any entry of >= kAttDenseMin tokens): the whole step runs on the fused tcgen05 kernel over the paged
      // planes; steps of single tokens and short portions, other masks, head sizes and the exact mode take the per-token kernel
      bool fused = gqa_fused_ok(model_, l, cfg_.max_ctx) && k.att16 && k.q16 && (H * Dk) % 8 == 0 && page_ == 64;
      int longest = 0;
      for (const StepEntry& en : step_entries_) longest = std::max(longest, en.n);
      // steps of single tokens: the Llama path's tensor-core decode kernel (keys and values streamed once per kv head by TMA)
      // with the block start, the unit of the denominator and the gate as parameters
      const int rep = H / G;
      static const bool dec_off = [] { const char* e = getenv("HB_STACK_TC_DECODE"); return e && atoi(e) == 0; }();
      const bool tc_dec = fused && !dec_off && longest == 1 && T == B && B <= cfg_.max_seqs && k.dec_ws && stack_tc(W, H * Dv, H * Dv, W) &&
                          (rep == 1 || rep == 2 || rep == 3 || rep == 4 || rep == 6 || rep == 8);
      fused = fused && longest >= kAttDenseMin;
      pa.q = (fused || tc_dec) ? nullptr : k.p2; pa.ldq = H * Dk; pa.q_b16 = (fused || tc_dec) ? k.q16 : nullptr;
      pa.k_cache = kplane; pa.v_cache = vplane; pa.f32 = f32;
      pa.slots = slots; pa.positions = positions;
      pa.cs = k.layer_set[i] >= 0 ? k.rope_cs[k.layer_set[i]] : nullptr; pa.rope_dims = l.rope_dims; pa.pairing = l.rope_pairing;
      pa.H = H; pa.G = G; pa.D = Dk; pa.Dv = Dv; pa.page_size = page_;
      pa.unit_norm = (l.attn_flags & HB_ATTN_QK_UNIT_NORM) != 0; pa.eps = sd.norm_eps; pa.T = T;
      pa.bias = ((l.attn_flags & HB_ATTN_QKV_BIAS) && !conv) ? w.b_in : nullptr;
      pa.proj_norm = (l.attn_flags & HB_ATTN_QK_PROJ_NORM) != 0; pa.qk_gain = w.qk_gain;
      pa.blend_role = w.blend_role; pa.vmix = w.vmix; pa.v_first = k.vfirst;
      SPAN(3, 8.0 * T * (H + 2 * G) * Dk, gqa_prep(stream_, pa));
      if (tc_dec) {
        AttnDecodeArgs da{};
        da.q = k.q16; da.ldq = H * Dk;
        da.k_cache = (const bf16*)kplane; da.v_cache = (const bf16*)vplane;
        da.page_table = pt; da.max_pages = max_pages_per_seq_;
        da.ctx_lens = (const int32_t*)(d_step_ + L.ctx);
        da.out = post ? k.att16 : mo16; da.ldo = H * Dv;
        da.workspace = k.dec_ws;
        da.B = B; da.Hq = H; da.Hkv = G; da.D = Dk; da.page_size = page_;
        const int want = (int)(0.8 * 2 * (cfg_.sm_budget > 0 ? cfg_.sm_budget : 148));
        da.num_splits = std::max(1, std::min(16, (want + B * G - 1) / (B * G)));
        da.scale = l.scale; da.num_pages = num_pages_;
        da.block_mask = l.mask == HB_MASK_CHUNK ? l.window : 0;
        da.window = (l.mask == HB_MASK_WINDOW && l.window < cfg_.max_ctx) ? l.window : 0;
        da.softcap = l.score_cap; da.sink = (l.attn_flags & HB_ATTN_LEARNED_SINK) ? (const bf16*)w.sink : nullptr;
        da.unit_sink = (l.attn_flags & HB_ATTN_UNIT_SINK) ? 1 : 0;
        if (l.attn_flags & HB_ATTN_HEAD_GATE) { da.head_gate = k.p1 + w.off_g; da.ldg = ldin; }
        SPAN(2, 2.0 * B * G * (double)std::min(l.window, cfg_.max_ctx) * (Dk + Dv), attn_decode(stream_, da));
        if (da.num_splits > 1) launches_.fetch_add(1, std::memory_order_relaxed);  // combine kernel
      } else if (fused) {
        AttnPrefillArgs fa{};
        fa.q = k.q16; fa.ldq = H * Dk;
        fa.k = nullptr; fa.ldk = 0; fa.v = nullptr; fa.ldv = 0;
        const bool direct = !post && stack_tc(W, H * Dv, H * Dv, W);  // the output projection reads the bf16 copy only
        fa.out = direct ? mo16 : k.att16; fa.ldo = H * Dv;
        if (direct && (l.attn_flags & HB_ATTN_HEAD_GATE)) { fa.head_gate = k.p1 + w.off_g; fa.ldg = ldin; }
        fa.cu_seqlens = cu; fa.B = B; fa.T = T; fa.max_seqlen = longest;
        fa.Hq = H; fa.Hkv = G; fa.D = Dk; fa.causal = 1; fa.scale = l.scale;
        fa.k_cache = (const bf16*)kplane; fa.v_cache = (const bf16*)vplane;
        fa.page_table = pt; fa.kv_lens = (const int32_t*)(d_step_ + L.ctx);
        fa.max_pages = max_pages_per_seq_; fa.num_pages = num_pages_; fa.page_size = page_;
        fa.block_mask = l.mask == HB_MASK_CHUNK ? l.window : 0;
        fa.window = (l.mask == HB_MASK_WINDOW && l.window < cfg_.max_ctx) ? l.window : 0;
        fa.softcap = l.score_cap; fa.sink = (l.attn_flags & HB_ATTN_LEARNED_SINK) ? (const bf16*)w.sink : nullptr;
        fa.unit_sink = (l.attn_flags & HB_ATTN_UNIT_SINK) ? 1 : 0;
        SPAN(1, 2.0 * T * H * (double)std::min(l.window, cfg_.max_ctx) * (Dk + Dv) * 0.5, attn_prefill(stream_, fa));
        if (!direct && !post)
          SPAN(3, 10.0 * T * H * Dv, head_gate_rows(stream_, k.att16, H * Dv, (l.attn_flags & HB_ATTN_HEAD_GATE) ? k.p1 + w.off_g : nullptr,
                                                    ldin, k.mo, mo16, T, H, Dv));
      } else {
      GqaAttnArgs aa{};
      aa.q = k.p2; aa.ldq = H * Dk;
      aa.k_cache = kplane; aa.v_cache = vplane; aa.f32 = f32;
      aa.page_table = pt; aa.max_pages = max_pages_per_seq_; aa.page_size = page_;
      aa.positions = positions; aa.seq_of = seqof;
      aa.gate = (l.attn_flags & HB_ATTN_HEAD_GATE) ? k.p1 + w.off_g : nullptr; aa.ldg = ldin;
      aa.out = post ? k.ctx : k.mo; aa.ldo = H * Dv; aa.out_b16 = post ? nullptr : mo16;
      aa.T = T; aa.H = H; aa.G = G; aa.D = Dk; aa.Dv = Dv; aa.mask = l.mask; aa.window = l.window;
      aa.unit_sink = (l.attn_flags & HB_ATTN_UNIT_SINK) != 0; aa.scale = l.scale;
      aa.softcap = l.score_cap; aa.sink = (l.attn_flags & HB_ATTN_LEARNED_SINK) ? w.sink : nullptr;
      if (!cfg_.use_cuda_graphs && gqa_attn_smem(Dk, Dv, l.window) > 200 * 1024) {
        for (const StepEntry& en : step_entries_) aa.longest_ctx = std::max(aa.longest_ctx, en.first + en.n);
        if (gqa_attn_smem(Dk, Dv, std::min(l.window, (aa.longest_ctx + 255) / 256 * 256)) > 200 * 1024)
          return fail(HB_ERR_INVALID, "a position sees more keys than the attention kernel's shared memory holds");
      }
      SPAN(7, 2.0 * T * H * (double)std::min(l.window, cfg_.max_ctx) * (Dk + Dv), gqa_attn(stream_, aa));
      }
      if (post) {
        const bool from16 = tc_dec || fused;
        if (l.attn_flags & HB_ATTN_OUT_GATE)
          SPAN(3, 12.0 * T * H * Dv, gate_scale_rows(stream_, from16 ? nullptr : k.ctx, from16 ? k.att16 : nullptr, H * Dv, k.p1 + w.off_g, ldin,
                                                     mix_scale, mo_f32, mo16, ocols, 0, T, H * Dv));
        else
          return fail(HB_ERR_INVALID, "a second mixer needs the entry-wise output gate on the first");
        if (w.ml.H > 0) {
          rc = run_memory(w, ldin, H * Dv, ocols, l.side_scale != 0.f ? l.side_scale : 1.f, mo_f32);
          if (rc != HB_OK) return rc;
        }
      }
    } else {
      const int R = l.kv_rank, Dr = l.rot_dim, Q = l.q_rank;
      uint8_t* plane = (uint8_t*)kv_ + plane_off_[w.cache_plane];
      LatentPrepArgs pa{};
      pa.p = k.p1; pa.ldp = k.ld1; pa.q_off = w.off_dq; pa.kv_off = w.off_dkv;
      pa.wq = w.dq_norm; pa.wkv = w.dkv_norm; pa.f32 = f32; pa.eps = sd.norm_eps;
      pa.cq = k.cq; pa.cq_b16 = cq16; pa.Q = Q;
      pa.cache = plane; pa.slots = slots; pa.positions = positions;
      pa.R = R; pa.Dr = Dr; pa.rope_dims = l.rope_dims; pa.rope_base = l.rope_base; pa.T = T;
      SPAN(3, 8.0 * T * (Q + R + Dr), latent_prep(stream_, pa));
      rc = stack_gemm(k.cq, cq16, Q, w.uq, H * (Dk + Dr), Q, k.p2, k.ld2, T);
      if (rc != HB_OK) return rc;
      const int D = R + Dr, ldqa = H * D, ldcx = H * R;  // (token, head) rows are contiguous: row stride D / R
      // keys are never expanded: q_h is carried into the latent space instead (q_h^T W_uk,h), one product per head —
      // on the tensor cores for steps of many tokens (bf16 copy of q, W_uk transposed per head at load), else one batched
      // CUDA-core launch
      const bool head_tc = !f32 && T > 256 && w.ukT && k.q16 && (Dk + Dr) % 8 == 0 && Dk % 8 == 0 && Dk >= 64 && R % 8 == 0 &&
                           R >= 64 && D % 4 == 0 && Dv % 4 == 0 && Dv >= 64 && !getenv("HB_STACK_SIMT");
      if (head_tc) {
        SPAN(3, 6.0 * T * H * (Dk + Dr), to_bf16_rows(stream_, k.p2, k.ld2, k.q16, k.ld2, T, H * (Dk + Dr)));
        for (int h = 0; h < H; ++h) {
          GemmArgs g{k.q16 + (size_t)h * (Dk + Dr), k.ld2, (const bf16*)w.ukT + (size_t)h * R * Dk, Dk, k.qabs + (size_t)h * D, ldqa,
                     nullptr, 0, nullptr, T, R, Dk, EPI_F32, 0};
          SPAN(0, 2.0 * T * R * Dk, gemm_bf16_tn(stream_, g));
        }
      } else {
        GemmRtArgs g{k.p2, k.ld2, (long)(Dk + Dr), w.uk, 1, (long)R, (long)Dk * R, k.qabs, ldqa, (long)D, nullptr, T, R, Dk, H, f32};
        SPAN(5, 2.0 * T * H * Dk * R, gemm_rt(stream_, g));
      }
      SPAN(3, 8.0 * T * H * Dr, latent_q_rope(stream_, k.p2, k.ld2, k.qabs, ldqa, positions, T, H, Dk, Dr, R, l.rope_dims, l.rope_base));
      // Long prompt portions (bf16 mode): scores and weighted latents as two tcgen05 products per block of att_qb tokens over
      // the block's gathered keys, softmax (mask, sink) between them.  Everything else — single tokens, short portions, the
      // exact mode — goes through the per-token kernel.  Both read the same cache rows, written by latent_prep above.
      static const bool dense_off = [] { const char* e = getenv("HB_STACK_DENSE_ATTN"); return e && atoi(e) == 0; }();
      const bool dense_ok = !f32 && !dense_off && k.S && D % 8 == 0 && R % 8 == 0 && (size_t)k.att_qb * H <= k.att_rows &&
                            (size_t)l.window + k.att_qb <= k.att_keys;
      bool any_dense = false;
      if (dense_ok)
        for (const StepEntry& en : step_entries_) any_dense |= en.n >= kAttDenseMin;
      if (any_dense) SPAN(3, 6.0 * T * ldqa, to_bf16_rows(stream_, k.qabs, ldqa, k.qabs16, ldqa, T, ldqa));
      int run0 = -1;  // start of the current run of tokens that take the per-token kernel
      auto flush = [&](int t_end) -> int {
        if (run0 < 0 || t_end <= run0) { run0 = -1; return HB_OK; }
        LatentAttnArgs aa{};
        aa.qabs = k.qabs + (size_t)run0 * ldqa; aa.ldqa = ldqa; aa.cache = plane; aa.f32 = f32; aa.sink = w.sink;
        aa.page_table = pt; aa.max_pages = max_pages_per_seq_; aa.page_size = page_;
        aa.positions = positions + run0; aa.seq_of = seqof + run0;
        aa.ctx = k.ctx + (size_t)run0 * ldcx; aa.ldc = ldcx;
        aa.T = t_end - run0; aa.H = H; aa.R = R; aa.Dr = Dr; aa.window = l.window; aa.scale = l.scale;
        SPAN(7, 2.0 * aa.T * H * (double)std::min(l.window, cfg_.max_ctx) * (2.0 * R + Dr), latent_attn(stream_, aa));
        run0 = -1;
        return HB_OK;
      };
      for (size_t b = 0; b < step_entries_.size(); ++b) {
        const StepEntry& en = step_entries_[b];
        if (!(dense_ok && en.n >= kAttDenseMin)) {
          if (run0 < 0) run0 = en.t0;
          continue;
        }
        rc = flush(en.t0);
        if (rc != HB_OK) return rc;
        for (int q0 = 0; q0 < en.n; q0 += k.att_qb) {
          const int nq = std::min(k.att_qb, en.n - q0);
          const int p0 = en.first + q0;                       // position of the block's first query
          const int k0 = std::max(0, p0 - l.window + 1);      // first key any of its queries sees
          const int nk = p0 + nq - k0;                        // ... through the block's last token
          const int ldk = (nk + 7) / 8 * 8;
          const int rows = nq * H;
          SPAN(3, 4.0 * nk * D, latent_gather(stream_, (const bf16*)plane, pt + b * max_pages_per_seq_, page_, k0, nk, R, Dr, k.kbuf, k.ct, ldk));
          GemmArgs g1{k.qabs16 + (size_t)(en.t0 + q0) * ldqa, D, k.kbuf, D, k.S, ldk, nullptr, 0, nullptr, rows, nk, D, EPI_F32, 0};
          SPAN(1, 2.0 * rows * nk * D, gemm_bf16_tn(stream_, g1));
          SPAN(3, 6.0 * rows * ldk, latent_softmax(stream_, k.S, k.P, ldk, rows, H, p0, k0, nk, l.window, l.scale, (const bf16*)w.sink));
          GemmArgs g2{k.P, ldk, k.ct, ldk, k.ctx + (size_t)(en.t0 + q0) * ldcx, R, nullptr, 0, nullptr, rows, R, ldk, EPI_F32, 0};
          SPAN(1, 2.0 * rows * ldk * R, gemm_bf16_tn(stream_, g2));
        }
      }
      rc = flush(T);
      if (rc != HB_OK) return rc;
      const int ldov = H * Dv;
      float* ov = k.ctx + al256((size_t)t_cap_ * k.ldctx * 4) / 4;  // per-head values out of the weighted latent
      if (head_tc) {
        SPAN(3, 6.0 * T * ldcx, to_bf16_rows(stream_, k.ctx, ldcx, k.ctx16, ldcx, T, ldcx));
        for (int h = 0; h < H; ++h) {
          GemmArgs g{k.ctx16 + (size_t)h * R, ldcx, (const bf16*)w.uv + (size_t)h * Dv * R, R, ov + (size_t)h * Dv, ldov,
                     nullptr, 0, nullptr, T, Dv, R, EPI_F32, 0};
          SPAN(0, 2.0 * T * Dv * R, gemm_bf16_tn(stream_, g));
        }
      } else {
        GemmRtArgs g{k.ctx, ldcx, (long)R, w.uv, (long)R, 1, (long)Dv * R, ov, ldov, (long)Dv, nullptr, T, Dv, R, H, f32};
        SPAN(5, 2.0 * T * H * Dv * R, gemm_rt(stream_, g));
      }
      SPAN(3, 12.0 * T * H * Dv, sigmoid_gate(stream_, ov, ldov, k.p1 + w.off_g, k.ld1, k.mo, mo16, T, H * Dv));
    }
    rc = stack_gemm(k.mo, mo16, ocols, w.wo, W, ocols, k.y, W, T);
    if (rc != HB_OK) return rc;
    if (par) {
      // both sublayers read the same stream: the feed-forward runs on its own normed copy, one launch adds both outputs
      // (and the first mixer's output bias, times that mixer's weight) and norms the next layer's inputs
      const float* y2 = nullptr;
      if (l.ff > 0) {
        if (l.ff_kind == HB_FF_RELU2) rc = relu2_ff(w.w_gu, w.w_down, l.ff, k.y2);
        else rc = gated_ff(w.w_gu, w.w_down, l.ff, l.ff_kind == HB_FF_SILU ? GLU_SILU : GLU_GELU_TANH, 0.f, w.gu_packed, k.y2);
        if (rc != HB_OK) return rc;
        y2 = k.y2;
      }
      SPAN(3, 5 * rowb, par_step(k.y, y2, w.o_bias, l.mix_scale != 0.f ? l.mix_scale : 1.f, i + 1));
      continue;
    }
    SPAN(3, 3 * rowb, resid(w.o_bias, both ? w.norm1b : w.norm1, l.ff > 0 ? w.norm2 : pre_next));
    if (l.ff > 0 && l.ff_kind == HB_FF_RELU2) {
      rc = relu2_ff(w.w_gu, w.w_down, l.ff, k.y);
      if (rc != HB_OK) return rc;
      SPAN(3, 3 * rowb, resid(nullptr, both ? w.norm2b : w.norm2, pre_next));
    } else if (l.ff > 0 && l.ff_kind == HB_FF_MOE) {
      // router in fp32 on the stream itself; experts per (token, choice); identity outputs and weights in the combination
      const int E = l.experts, R = l.experts + l.identity_experts, F = l.ff;
      RouteOpts ro;
      ro.sigmoid = l.router_kind == HB_ROUTER_SIGMOID; ro.groups = l.route_groups; ro.keep = l.route_keep; ro.renorm = l.route_renorm;
      ro.scale = l.route_scale != 0.f ? l.route_scale : 1.f;
      const int eact = l.expert_kind == HB_EXPERT_CLAMPED ? GLU_CLAMPED : GLU_SILU;
      const float* add = nullptr;
      if (l.shared_ff > 0) {  // the unit every token uses; the combination below starts from its output
        rc = gated_ff(w.w_gu_sh, w.w_down_sh, l.shared_ff, eact, l.shared_limit, w.sh_packed, k.y2);
        if (rc != HB_OK) return rc;
        add = k.y2;
      }
      if (T > 256 && R <= 64 && stack_tc(64, W, W, k.ldz) && k.ldz >= 64) {
        // steps of many tokens: logits on the tensor cores from the bf16 copy of the stream (fp32 accumulation; the router's
        // rows are padded with zero rows to one MMA tile), then the choice in fp32
        GemmArgs g{x16, W, (const bf16*)w.router, W, k.moe_z, k.ldz, nullptr, 0, nullptr, T, 64, W, EPI_F32, 0};
        SPAN(0, 2.0 * T * 64 * W, gemm_bf16_tn(stream_, g));
        SPAN(3, 8.0 * T * R, moe_route(stream_, k.moe_z, k.ldz, w.correction, f32, R, l.top_k, k.moe_ids, k.moe_w, T, ro));
      } else if (moe_router_smem(R, W, f32) <= 200 * 1024) {
        SPAN(3, 4.0 * T * W, moe_router(stream_, xin, w.router, w.correction, f32, R, W, l.top_k, k.moe_ids, k.moe_w, T,
                                        cfg_.sm_budget > 0 ? cfg_.sm_budget : 148, ro));
      } else {  // a router too large for shared memory: product, then choice
        GemmRtArgs g{xin, W, 0, w.router, W, 1, 0, k.moe_z, k.ldz, 0, nullptr, T, R, W, 1, f32};
        SPAN(5, 2.0 * T * R * W, gemm_rt(stream_, g));
        SPAN(3, 8.0 * T * R, moe_route(stream_, k.moe_z, k.ldz, w.correction, f32, R, l.top_k, k.moe_ids, k.moe_w, T, ro));
      }
      const int items = T * l.top_k;
      if (moe_grouped_ok(model_, l) && k.moe_a16 && items >= 2 * E) {
        // items sorted by expert into 128-row segments; both products of every expert in two grouped tcgen05 launches
        const int rows = moe_group_max_rows(items, E);
        SPAN(3, 12.0 * items, moe_group_rows(stream_, k.moe_ids, items, l.top_k, E, k.moe_row_of, k.moe_src, k.moe_tiles, k.moe_scratch));
        if (items > 4096) launches_.fetch_add(2, std::memory_order_relaxed);  // three kernels behind one call
        SPAN(3, 4.0 * rows * W, moe_gather_rows(stream_, x16, W, k.moe_src, k.moe_a16, rows));
        if (w.gu_packed) {  // silu(gate) * up on the accumulators' way out
          GemmArgs g1{k.moe_a16, W, (const bf16*)w.w_gu, W, k.moe_h16, F, nullptr, 0, nullptr, rows, 2 * F, W,
                      eact == GLU_CLAMPED ? EPI_CLAMPGLU : EPI_SWIGLU, 0};
          g1.m_tile_group = k.moe_tiles; g1.groups = E; g1.glu_limit = l.ff_limit;
          SPAN(0, 4.0 * rows * F * W, gemm_bf16_tn(stream_, g1));
        } else {
          GemmArgs g1{k.moe_a16, W, (const bf16*)w.w_gu, W, k.gu16, 2 * F, nullptr, 0, nullptr, rows, 2 * F, W, EPI_NONE, 0};
          g1.m_tile_group = k.moe_tiles; g1.groups = E;
          SPAN(0, 4.0 * rows * F * W, gemm_bf16_tn(stream_, g1));
          SPAN(3, 6.0 * rows * F, gated_unit_b16(stream_, k.gu16, 2 * F, eact, k.moe_h16, rows, F, l.ff_limit));
        }
        GemmArgs g2{k.moe_h16, F, (const bf16*)w.w_down, F, k.moe_y16, W, nullptr, 0, nullptr, rows, W, F, EPI_NONE, 0};
        g2.m_tile_group = k.moe_tiles; g2.groups = E;
        SPAN(0, 2.0 * rows * F * W, gemm_bf16_tn(stream_, g2));
        SPAN(3, 2.0 * T * (l.top_k + 4) * W, moe_combine_rows(stream_, xin, k.moe_y16, k.moe_row_of, k.moe_w, l.top_k, k.y, T, W, add));
      } else {
        SPAN(5, 6.0 * items * F * W, moe_expert_rows(stream_, xin, x16, w.w_gu, w.w_down, f32, k.moe_ids, l.top_k, E, F, W, k.moe_y, T, w.gu_packed,
                                                     eact, l.ff_limit));
        SPAN(3, 4.0 * T * (l.top_k + 2) * W, moe_combine(stream_, xin, k.moe_y, k.moe_ids, k.moe_w, l.top_k, E, k.y, T, W, add));
      }
      SPAN(3, 3 * rowb, resid(nullptr, both ? w.norm2b : w.norm2, pre_next));
    } else if (l.ff > 0 && (l.ff_kind == HB_FF_GELU_TANH || l.ff_kind == HB_FF_SILU)) {
      rc = gated_ff(w.w_gu, w.w_down, l.ff, l.ff_kind == HB_FF_SILU ? GLU_SILU : GLU_GELU_TANH, 0.f, w.gu_packed, k.y);
      if (rc != HB_OK) return rc;
      SPAN(3, 3 * rowb, resid(nullptr, both ? w.norm2b : w.norm2, pre_next));
    } else if (l.ff > 0) {
      const int F = l.ff;
      rc = stack_gemm(xin, x16, W, w.w_gu, 2 * F, W, k.p1, k.ld1, T);
      if (rc != HB_OK) return rc;
      const void* bu = (const uint8_t*)w.b_gu + (size_t)F * model_.elem;
      SPAN(3, 12.0 * T * F, clamped_glu(stream_, k.p1, k.ld1, w.b_gu, bu, f32, l.ff_limit, 1.702f, k.mo, mo16, T, F));
      rc = stack_gemm(k.mo, mo16, F, w.w_down, W, F, k.y, W, T);
      if (rc != HB_OK) return rc;
      SPAN(3, 3 * rowb, resid(w.b_down, both ? w.norm2b : w.norm2, pre_next));
    }
  }
  // logits: final norm -> head -> soft cap, for the entries' last rows (sampling) and for the rows asked for
  auto head = [&](const int32_t* rows, int n, float* out) -> int {
    for (int r0 = 0; r0 < n; r0 += t_cap_) {  // the normed rows go through the (free) projection buffers, t_cap_ rows at a time
      const int m = std::min(t_cap_, n - r0);
      const int32_t* idx = rows ? rows + r0 : nullptr;
      const float* src = rows ? k.x : k.x + (size_t)r0 * W;
      LAUNCH(norm_rows(src, idx, model_.s_final_norm, k.y, x16, m));
      int rc = stack_gemm(k.y, x16, W, model_.s_head, V, W, out + (size_t)r0 * V, V, m);
      if (rc != HB_OK) return rc;
    }
    LAUNCH(softcap_rows(stream_, out, (size_t)n * V, sd.logit_softcap, sd.logit_scale != 0.f ? sd.logit_scale : 1.f));
    return HB_OK;
  };
  if (n_extra > 0) {
    int rc = head(extra_rows, n_extra, extra_out);
    if (rc != HB_OK) return rc;
  }
  if (sample) {
    int rc = head(last, B, logits_);
    if (rc != HB_OK) return rc;
    return sample_step(B, L);
  }
  return HB_OK;
}

// ------------------------------------------------------------------ driven sequences
int Engine::seq_open(uint64_t* id) {
  if (!id) return fail(HB_ERR_INVALID, "null argument");
  if (!loaded_ || !is_stack()) return fail(HB_ERR_STATE, "driven sequences need a loaded layer-list decoder");
  if (thread_running_) return fail(HB_ERR_STATE, "driven sequences and the step-loop thread exclude each other");
  std::lock_guard<std::mutex> g(mu_);
  const int slot = take_slot();
  if (slot < 0) return fail(HB_ERR_BUSY, "no free state slot");
  auto r = std::make_unique<Request>();
  r->driven = true;
  r->state_slot = slot;
  r->state = ReqState::RUNNING;
  r->id = next_id_++;
  *id = r->id;
  reqs_[r->id] = std::move(r);
  return HB_OK;
}

int Engine::seq_close(uint64_t id) {
  std::lock_guard<std::mutex> gg(gpu_mu_);
  std::lock_guard<std::mutex> g(mu_);
  auto it = reqs_.find(id);
  if (it == reqs_.end() || !it->second->driven) return fail(HB_ERR_NOT_FOUND, "unknown sequence id");
  finish_request(it->second.get(), ReqState::FINISHED);  // pages and state slot go back
  reqs_.erase(it);
  return HB_OK;
}

int Engine::seq_step(const hb_seq_feed* entries, int n, float* out, size_t cap, int* rows_out) {
  if (rows_out) *rows_out = 0;
  if (!entries || n <= 0) return fail(HB_ERR_INVALID, "null/empty argument");
  if (!loaded_ || !is_stack()) return fail(HB_ERR_STATE, "driven sequences need a loaded layer-list decoder");
  if (thread_running_) return fail(HB_ERR_STATE, "driven sequences and the step-loop thread exclude each other");
  if (cuda_error_.load()) return fail(HB_ERR_CUDA, "engine is in a sticky CUDA error state");
  if (n > b_cap_) return fail(HB_ERR_INVALID, "more entries than max_seqs");
  std::lock_guard<std::mutex> gg(gpu_mu_);
  CU(cudaSetDevice(cfg_.device));
  SmLimitScope sm_scope(cfg_.sm_budget);
  std::vector<Request*> batch;
  int T = 0, R = 0;
  {
    std::lock_guard<std::mutex> g(mu_);
    int need_pages = 0;
    for (int i = 0; i < n; ++i) {  // validate everything before anything changes hands
      const hb_seq_feed& f = entries[i];
      auto it = reqs_.find(f.seq);
      if (it == reqs_.end() || !it->second->driven) return fail(HB_ERR_NOT_FOUND, "unknown sequence id");
      Request* r = it->second.get();
      if (std::find(batch.begin(), batch.end(), r) != batch.end()) return fail(HB_ERR_INVALID, "a sequence appears twice in one step");
      if (!f.tokens || f.n_tokens <= 0) return fail(HB_ERR_INVALID, "an entry without tokens");
      if (f.n_want < 0 || (f.n_want > 0 && !f.want)) return fail(HB_ERR_INVALID, "bad want list");
      for (int j = 0; j < f.n_tokens; ++j)
        if (f.tokens[j] < 0 || f.tokens[j] >= model_.d.vocab) return fail(HB_ERR_INVALID, "token id out of range");
      for (int j = 0; j < f.n_want; ++j)
        if (f.want[j] < 0 || f.want[j] >= f.n_tokens) return fail(HB_ERR_INVALID, "want index outside the entry");
      if (r->kv_len + f.n_tokens > cfg_.max_ctx) return fail(HB_ERR_INVALID, "sequence exceeds context_length");
      need_pages += (r->kv_len + f.n_tokens + page_ - 1) / page_ - (int)r->pages.size();
      T += f.n_tokens;
      R += f.n_want;
      batch.push_back(r);
    }
    if (T > t_cap_) return fail(HB_ERR_INVALID, "step exceeds max_batched_tokens");
    if (need_pages > pages_available()) return fail(HB_ERR_BUSY, "not enough free cache pages");
    if (out == nullptr ? R > 0 : (size_t)R * model_.d.vocab > cap) return fail(HB_ERR_INVALID, "logits buffer too small");
    for (int i = 0; i < n; ++i) {
      const hb_seq_feed& f = entries[i];
      Request* r = batch[i];
      r->prompt.insert(r->prompt.end(), f.tokens, f.tokens + f.n_tokens);
      while ((int)r->pages.size() * page_ < (int)r->prompt.size()) r->pages.push_back(take_page());
      r->prefilled = r->kv_len;
      r->chunk = f.n_tokens;
      r->target = r->kv_len + f.n_tokens;
      r->want.assign(f.want, f.want + f.n_want);
    }
  }
  step_driven_ = true;
  step_decode_rows_ = 0;
  int rc = run_prefill(batch);
  step_driven_ = false;
  if (rc != HB_OK) return rc;  // a CUDA failure is sticky; the sequences keep their records for hb_seq_close
  if (R > 0) CU(cudaMemcpy(out, all_logits_, (size_t)R * model_.d.vocab * 4, cudaMemcpyDeviceToHost));
  {
    std::lock_guard<std::mutex> g(mu_);
    for (Request* r : batch) {
      r->kv_len += r->chunk;
      r->prefilled = r->kv_len;
      r->want.clear();
    }
  }
  if (rows_out) *rows_out = R;
  return HB_OK;
}

}  // namespace hb
