// Internal C++ interface to the sm_100a kernels (the C ABI in include/helix_b200.h sits on top).
// All pointers are device pointers; every launcher is asynchronous on `stream` and returns the
// launch status.  Shapes follow the reference backends' conventions (SURVEY.md §2.3, K1–K11).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hb {

typedef __nv_bfloat16 bf16;

// Sets the opt-in shared-memory attribute of every kernel instantiation; call once per process/device.
cudaError_t kernels_init();
cudaError_t gemm_init();
cudaError_t attn_prefill_init();
cudaError_t attn_decode_init();

// ---- GEMM: C[M,N] = A[M,K] · W[N,K]^T (both K-major, bf16 in, fp32 accumulate in TMEM) ----
enum Epi : int {
  EPI_NONE = 0,        // C = acc                              (bf16)
  EPI_BIAS = 1,        // C = acc + bias[n]                    (bf16)
  EPI_BIAS_GELU = 2,   // C = gelu_erf(acc + bias[n])          (bf16)
  EPI_RESID = 3,       // C = acc + R[m,n]                     (bf16, R may alias C)
  EPI_BIAS_RESID = 4,  // C = acc + bias[n] + R[m,n]           (bf16)
  EPI_SWIGLU = 5,      // W rows packed per 256-row tile as [128 gate | 128 up];
                       // C[m, tile*128+j] = silu(gate_j) * up_j   (bf16, ldc counts N/2 columns)
  EPI_F32 = 6,         // C = acc                              (fp32)
  EPI_GEGLU = 8,       // as EPI_SWIGLU with gelu_tanh(gate_j) * up_j
  EPI_CLAMPGLU = 9,    // as EPI_SWIGLU with g = min(gate_j, limit), u = clamp(up_j, -limit, limit): g sigmoid(1.702 g) (u + 1)
                       // (limit = GemmArgs::glu_limit)
  EPI_RELU2 = 10,      // C = relu(acc)^2                      (bf16)
  EPI_ROPE = 7,        // fused QKV projection of a decoder: C = bf16(acc [+ bias]) with the q and k heads rotated
                       // (RopeEpi) and the k / v rows also scattered into the paged KV cache
};

// What EPI_ROPE needs beyond the GEMM itself (the job of rope_kv_write, done on the accumulators' way out).
struct RopeEpi {
  bf16* out = nullptr;             // == GemmArgs::C, written with plain stores (row stride ldc elements)
  int ldc = 0;
  const float* cs = nullptr;       // [M][D]: cos(pos*inv_freq[i]) for i < D/2, then sin (rope_table)
  const int32_t* slots = nullptr;  // slot_mapping as in rope_kv_write; null or < 0: no cache write for the row
  bf16* k_cache = nullptr;
  bf16* v_cache = nullptr;
  int Hq = 0, Hkv = 0, D = 0, page_size = 0;
};

struct GemmArgs {
  const bf16* A;
  int lda;
  const bf16* W;
  int ldw;
  void* C;
  int ldc;
  const bf16* R;
  int ldr;
  const bf16* bias;
  int M, N, K;
  Epi epi;
  int block_n;  // 0 = choose
  RopeEpi rope{};  // EPI_ROPE only
  // Grouped weights (mixtures of experts): W holds `groups` matrices of N rows each, one after the other; the 128 rows of m
  // tile i of A multiply the matrix m_tile_group[i] (device array, ceil(M / 128) entries, every entry a valid group).
  const int32_t* m_tile_group = nullptr;
  int groups = 1;
  float glu_limit = 0.f;  // EPI_CLAMPGLU
};
cudaError_t gemm_bf16_tn(cudaStream_t stream, const GemmArgs& a);
// Debug/test-only CUDA-core GEMM (same contract, EPI_NONE/EPI_F32 only); used by tests as an on-device checker.
cudaError_t gemm_naive_check(cudaStream_t stream, const GemmArgs& a);


// ---- HBM-bound row kernels (K1, K2, K4, K10 sampling, K11) ----
// x[t,:] = table[tokens[t],:]
cudaError_t embed_gather(cudaStream_t s, const int32_t* tokens, const bf16* table, bf16* x, int T, int H);
// BERT: x[t,:] = LayerNorm(word[tok[t]] + pos[positions[t]] + type[0]) * g + b
cudaError_t bert_embed_ln(cudaStream_t s, const int32_t* tokens, const int32_t* positions, const bf16* word,
                          const bf16* pos, const bf16* type0, const bf16* gamma, const bf16* beta, bf16* x, int T, int H,
                          float eps);
// out[r,:] = x[row_index ? row_index[r] : r, :] * rsqrt(mean(x^2)+eps) * w    (fp32 math, one bf16 rounding)
cudaError_t rmsnorm(cudaStream_t s, const bf16* x, const bf16* w, bf16* out, const int32_t* row_index, int rows, int H,
                    float eps);
// out[r,:] = (x[r,:]-mean)/sqrt(var+eps)*g + b   (in-place allowed)
cudaError_t layernorm(cudaStream_t s, const bf16* x, const bf16* gamma, const bf16* beta, bf16* out, int rows, int H,
                      float eps);
// In-place rotary embedding (HF rotate_half convention) on the q and k column blocks of the fused
// qkv[T, (Hq+2*Hkv)*D] buffer, then scatter of the rotated k and of v into the paged KV cache:
//   slot = slot_mapping[t] = page*page_size + offset;  cache layout [page][Hkv][page_size][D].
// slot < 0 skips the cache write (embedding-only models never call this).
cudaError_t rope_kv_write(cudaStream_t s, bf16* qkv, const int32_t* positions, const int32_t* slot_mapping,
                          const float* inv_freq, bf16* k_cache, bf16* v_cache, int T, int Hq, int Hkv, int D,
                          int page_size);
// cs[t][0..D/2) = cos(positions[t] * inv_freq[i]), cs[t][D/2..D) = sin(...): the table EPI_ROPE reads (once per step,
// shared by every layer).
cudaError_t rope_table(cudaStream_t s, const int32_t* positions, const float* inv_freq, float* cs, int T, int D);
// Greedy / Gumbel-max sampling over fp32 logits[B,V]: out[b] = argmax_v(logits[b,v]/temp[b] + g(seed[b],v)),
// temp[b] <= 0 -> pure argmax (lowest index wins ties).
cudaError_t sample_tokens(cudaStream_t s, const float* logits, int ldl, const float* temperature, const uint64_t* seed,
                          int32_t* out, int B, int V, void* scratch, const int32_t* top_k = nullptr,
                          const float* top_p = nullptr);  // per-row top-k (<=0 off) / top-p (outside (0,1) off), sampled rows only
size_t sample_scratch_bytes(int B, int V);  // two-stage argmax partials
// logits[b, tok] -= val for the entries {int32 tok; float val} [pen_off[b], pen_off[b+1]) of row b (distinct tokens per row)
cudaError_t apply_penalties(cudaStream_t s, float* logits, int ldl, const int32_t* pen_off, const void* pen, int B, int V);
// rows with width[b] > 0: out_ids/out_lp[b][0] = sampled token and its log-softmax, [1..width) = most likely tokens (desc)
cudaError_t logprob_topk(cudaStream_t s, const float* logits, int ldl, int V, const int32_t* sampled, const int32_t* width,
                         int32_t* out_ids, float* out_lp, int B, int max_width);
// out[b,:] = l2normalize(x[first_row[b], :]) as fp32 (CLS pooling for bge-style encoders)
cudaError_t cls_pool_l2(cudaStream_t s, const bf16* x, const int32_t* first_row, float* out, int B, int H);


// ---- K5: varlen flash attention over contiguous q/k/v rows (whole-prompt prefill, BERT encoder) ----
struct AttnPrefillArgs {
  const bf16* q; int ldq;   // [T, >=Hq*D], head h at column h*D
  const bf16* k; int ldk;   // [T, >=Hkv*D]
  const bf16* v; int ldv;
  bf16* out; int ldo;       // [T, Hq*D]
  const int32_t* cu_seqlens;  // [B+1] token offsets
  int B, T, max_seqlen;
  int Hq, Hkv, D;
  int causal;
  float scale;              // 1/sqrt(D)
  // chunked prefill (optional; k_cache != nullptr selects it): the q rows are the last rows of kv_lens[b]-long sequences
  // whose K/V are read from the paged pool instead of k/v
  const bf16* k_cache = nullptr;   // [num_pages][Hkv][64][D] plane of one layer
  const bf16* v_cache = nullptr;
  const int32_t* page_table = nullptr;  // [B, max_pages]
  const int32_t* kv_lens = nullptr;     // [B] kv length including this step's q rows
  int max_pages = 0, num_pages = 0, page_size = 64;
  // paged + causal only.  block_mask > 0: a position sees only the keys of its own block of block_mask positions (blocks
  // counted from position 0 of the sequence).  unit_sink: one unit added to the softmax denominator (a key of score 0 that
  // carries no value)
  int block_mask = 0, unit_sink = 0;
  const float* head_gate = nullptr; int ldg = 0;  // optional [T][>= Hq] fp32: head h of token t leaves times sigmoid(head_gate[t][h])
  // paged + causal only.  window > 0: position i sees j with 0 <= i - j < window.  softcap > 0: scores pass
  // softcap * tanh(scale * s / softcap).  sink: [Hq] learned logits, exp(sink[h]) joins head h's softmax denominator.
  int window = 0;
  float softcap = 0.f;
  const bf16* sink = nullptr;
};
cudaError_t attn_prefill(cudaStream_t stream, const AttnPrefillArgs& a);
// test-only CUDA-core checker, fp32 output [T, ldo]
cudaError_t attn_naive_check(cudaStream_t stream, const AttnPrefillArgs& a, float* out_f32);

// Stream hand-over between consecutive HBM-streaming kernels of a decode step (see ptx.cuh sig_*): `wait` is the counter
// the PREVIOUS streaming kernel bumps once per CTA when its last load is issued (`wait_count` = its CTA count), `done`
// is this kernel's own counter, `bank_bytes` how much of its own stream the kernel may prefetch into L2 once the
// predecessor's loads have ended.  All-zero = feature off.
// Data dependency of a decode-step kernel on its predecessor as a release/acquire counter (ptx.cuh dep_*): `wait` is the
// predecessor's counter, `wait_count` how many of its CTAs report, `done` this kernel's own counter.  wait == nullptr:
// the kernel uses griddepcontrol.wait (every standalone / prefill use).
struct DepSig {
  const int* wait = nullptr;
  int wait_count = 0;
  int* done = nullptr;
};
struct StreamSig {
  const int* wait = nullptr;
  int wait_count = 0;
  int* done = nullptr;
  size_t bank_bytes = 0;
  unsigned long long* trace = nullptr;  // 16 event slots of this launch (HB_DEC_TRACE), written by CTA 0
  DepSig dep;                           // data dependency on the previous kernel of the step (optional)
};

// ---- K6: paged-KV decode attention (one query token per sequence), split-KV + combine ----
// Optional prologue of the decode-attention kernel (one split only): each CTA (sequence b, kv head) is the ONLY consumer of
// that sequence's q heads of the group and of its new K/V row, so it builds them itself from the QKV GEMM's slabs — slab sum
// (+ bias), bf16 rounding, RoPE, K/V written into the paged cache, q staged straight into shared memory — and the separate
// RoPE / KV-write kernel (and its kernel boundary) disappears from the layer.  Same arithmetic as dec_qkv_rope_kvwrite.
struct DecodeRope {
  const float* ws = nullptr;        // QKV GEMM slabs [seg][M][N]; nullptr = q is read from AttnDecodeArgs::q as usual
  const uint8_t* segs = nullptr;    // slabs per 128-column tile
  int M = 0, N = 0;                 // batch rows, (Hq + 2 Hkv) * D
  const bf16* bias = nullptr;       // [N] or null
  const int32_t* positions = nullptr;
  const int32_t* slots = nullptr;
  const float* inv_freq = nullptr;
  bf16* k_cache = nullptr;          // writable views of the layer's planes
  bf16* v_cache = nullptr;
};
struct AttnDecodeArgs {
  const bf16* q; int ldq;          // [B, >=Hq*D] (post-RoPE)
  const bf16* k_cache;             // [num_pages][Hkv][page_size][D]
  const bf16* v_cache;
  const int32_t* page_table;       // [B, max_pages]
  int max_pages;
  const int32_t* ctx_lens;         // [B] kv length including the current token
  bf16* out; int ldo;              // [B, Hq*D]
  float* workspace;                // >= B*Hq*num_splits*(D+2) floats
  int B, Hq, Hkv, D, page_size, num_splits;
  float scale;
  int num_pages;                   // pages in the pool (TMA tensor-map extent)
  StreamSig sig;                   // HBM hand-over with the neighbouring streaming kernels (optional)
  DecodeRope rope;                 // build q / K / V from the QKV GEMM's slabs inside the kernel (num_splits == 1 only)
  // block_mask > 0: the token sees only the keys of its own block of block_mask positions (blocks counted from position 0);
  // unit_sink: one unit added to the softmax denominator; head_gate: optional [B][>= Hq] fp32, head h leaves times its sigmoid
  int block_mask = 0, unit_sink = 0;
  const float* head_gate = nullptr; int ldg = 0;
  // window > 0: the token sees the last `window` positions; softcap > 0: scores pass softcap * tanh(scale * s / softcap);
  // sink: [Hq] learned logits whose exponential joins the head's softmax denominator
  int window = 0;
  float softcap = 0.f;
  const bf16* sink = nullptr;
};
cudaError_t attn_decode(cudaStream_t stream, const AttnDecodeArgs& a);
size_t attn_decode_workspace_floats(int B, int Hq, int D, int num_splits);


// ---- decode-step GEMM (M <= 256): swap-AB + deterministic stream-K, fp32 partial slabs ----
struct SkinnyPlan {
  int grid;                  // CTAs (== SMs unless the problem is tiny)
  int n_tiles;               // ceil(N/128)
  int max_segs;              // max #slabs any tile is split into
  const uint8_t* seg_count;  // device [n_tiles]: slabs of each 128-column tile
};
// Tile finisher of the decode GEMM: the LAST CTA that contributes a slab to an output tile (one counter per tile) sums
// the tile's slabs in slab order — bit-deterministic whoever finishes — and applies the op that follows the projection
// in the decoder layer, so no separate row kernel (and no kernel boundary) sits between two projections.
enum SkinnyEpiMode : int {
  SK_SLABS = 0,       // no finisher: slabs only (legacy path, consumed by the dec_* row kernels)
  SK_F32 = 1,         // out[m, n] = rstd[m] * sum                                   (LM head -> logits)
  SK_QKV_ROPE = 2,    // bf16(rstd[m] * sum) -> RoPE on q / k heads -> q to qkv_out, k / v into the paged cache
  SK_RESID_NORM = 3,  // x = bf16(x + sum); xg = bf16(x * gain[n]); ss_out[tile][m] = sum_n x^2 over the tile's columns
  SK_SWIGLU = 4,      // tiles (2t, 2t+1) = gate / up rows of block t:  h[m, t*128+j] = silu(rstd*gate) * (rstd*up)
};
constexpr int kSkinnySsStride = 256;  // row stride of the per-tile sum-of-squares partials ([tile][m], m < 256)
struct SkinnyEpi {
  int mode = SK_SLABS;
  int* tile_cnt = nullptr;          // per-engine arrival counters (zero between launches; the finisher re-zeroes its own)
  // rstd[m] = rsqrt(sum_t ss_in[t * 256 + m] / norm_h + eps): RMSNorm statistics of the INPUT rows, carried as per-tile
  // partials by the SK_RESID_NORM finisher of the previous projection (the GEMM is linear in the row factor); null: 1
  const float* ss_in = nullptr;
  int ss_tiles = 0, norm_h = 0;
  float eps = 0.f;
  float* out_f32 = nullptr; int ldo = 0;                                        // SK_F32
  bf16* qkv_out = nullptr; const int32_t* positions = nullptr; const int32_t* slots = nullptr;  // SK_QKV_ROPE
  const float* inv_freq = nullptr; bf16* k_cache = nullptr; bf16* v_cache = nullptr;
  int Hq = 0, Hkv = 0, D = 0, page_size = 64;
  bf16* x = nullptr; const bf16* gain = nullptr; bf16* xg = nullptr; float* ss_out = nullptr;   // SK_RESID_NORM
  bf16* h = nullptr; int F = 0;                                                  // SK_SWIGLU
};
// x = table[token]; xg = bf16(x * gain); ss_out[tile][m] = per-128-column sums of x^2 (what SK_RESID_NORM leaves behind)
cudaError_t dec_embed_prep(cudaStream_t s, const int32_t* tokens, const bf16* table, const bf16* gain, bf16* x, bf16* xg,
                           float* ss_out, int M, int H);
cudaError_t gemm_skinny_init();
cudaError_t gemm_skinny_plan(int N, int K, SkinnyPlan* out);  // cached per (device, N, K)
size_t gemm_skinny_ws_floats(const SkinnyPlan& p, int M, int N);
int gemm_skinny_max_segs(int N, int K, int sms);  // pure host arithmetic (memory estimates)
// ws[seg][m][n] (seg < seg_count[n/128]) = partial sums of X[M,K] . W[N,K]^T
cudaError_t gemm_skinny(cudaStream_t stream, const SkinnyPlan& plan, const bf16* X, int ldx, const bf16* W, int ldw,
                        float* ws, int M, int N, int K, const StreamSig* sig = nullptr, const SkinnyEpi* epi = nullptr);
// consumers of the slabs (each sums the slabs in fixed order, then applies its fused epilogue)
cudaError_t dec_sum_slabs(cudaStream_t s, const float* ws, const SkinnyPlan& p, float* out, int ldo, int M, int N);
// the dec_* kernels below take an optional DepSig; *ctas (when given) receives the number of CTAs that will report
cudaError_t dec_qkv_rope_kvwrite(cudaStream_t s, const float* ws, const SkinnyPlan& p, bf16* qkv_out,
                                 const int32_t* positions, const int32_t* slot_mapping, const float* inv_freq,
                                 bf16* k_cache, bf16* v_cache, int M, int Hq, int Hkv, int D, int page_size,
                                 const DepSig* dep = nullptr, const bf16* qkv_bias = nullptr);
int dec_qkv_rope_ctas(int M, int Hq, int Hkv);
int dec_swiglu_ctas(int M, int F);
// x = bf16(x + sum); xn = rmsnorm(x) * w (w may be null: residual update only)
cudaError_t dec_resid_rmsnorm(cudaStream_t s, const float* ws, const SkinnyPlan& p, bf16* x, const bf16* w, bf16* xn,
                              int M, int H, float eps, const DepSig* dep = nullptr);
// h[m, t*128+j] = silu(sum[m, t*256+j]) * sum[m, t*256+128+j]
cudaError_t dec_swiglu(cudaStream_t s, const float* ws, const SkinnyPlan& p, bf16* h, int M, int F, const DepSig* dep = nullptr);

// ==================================================================================================================
// Mechanisms of hybrid decoder stacks (recurrent + windowed-attention layers on a 32-bit residual stream).
// Activations between kernels are fp32; weights and cache rows are bf16 or fp32 (`f32` selects the element type of
// every `const void*` weight / cache argument of a call).  Each launcher optionally writes a bf16 copy of its output
// for the tensor-core GEMM that consumes it (`*_b16`, may be null).
// ==================================================================================================================

// C[z][m, n] = sum_k A[z][m, k] * W[z](n, k) (+ bias[n]): CUDA-core fp32 FMA GEMM for shapes or precisions the tcgen05
// GEMMs do not take (true 32-bit mode, strides that are not 16-byte multiples, per-head batched products).
// W(n, k) = W[z * w_bs + n * w_sn + k * w_sk]; k runs sequentially inside a thread, so a row's result does not depend on M.
cudaError_t stack_ops_init();  // opt-in shared-memory attributes of the kernels below (once, outside any graph capture)
struct GemmRtArgs {
  const float* A; long lda; long a_bs;
  const void* W; long w_sn, w_sk, w_bs;
  float* C; long ldc; long c_bs;
  const void* bias;   // [N] of the weight type, or null
  int M, N, K, batch;
  bool f32;           // element type of W / bias
};
cudaError_t gemm_rt(cudaStream_t s, const GemmRtArgs& a);

// x[t, :] = table[tokens[t], :] * scale as fp32 (+ bf16 copy)
cudaError_t embed_rows_f32(cudaStream_t s, const int32_t* tokens, const void* table, bool f32, float* x, bf16* x_b16, int T, int W,
                           float scale = 1.f);
// Residual step between element-wise norms N(v) = tanh(alpha v) * w + b; `post` / `pre` are blocks [w (W) | b (W) | alpha] of
// the weight type or null.  v = x[row_index ? row_index[r] : r]; with y: v += post ? N_post(y[r]) : y[r] and x_out[r] = v
// (x_out may be x); with pre: h[r] = N_pre(v) as fp32 (h) and / or bf16 (h_b16).
cudaError_t tanh_norm_step(cudaStream_t s, const float* x, const int32_t* row_index, const float* y, long ldy, const void* post,
                           const void* pre, bool f32, float* x_out, float* h, bf16* h_b16, int rows, int W);
// Post-norm residual step: x[t] <- rmsnorm(alpha * x[t] + y[t] (+ bias)) * (gain_offset + w);  rows of y have stride ldy
cudaError_t resid_postnorm(cudaStream_t s, float* x, bf16* x_b16, const float* y, long ldy, const void* bias, const void* w,
                           bool f32, float alpha, float gain_offset, float eps, int T, int W);
// Residual step with the norm on the sublayer's output only: x[t] <- x[t] + rmsnorm(y[t] (+ bias)) * (gain_offset + w)
cudaError_t resid_add_normed(cudaStream_t s, float* x, bf16* x_b16, const float* y, long ldy, const void* bias, const void* w,
                             bool f32, float gain_offset, float eps, int T, int W);
// out[r] = rmsnorm(x[row_index ? row_index[r] : r]) * (gain_offset + w)   (out may be x itself when row_index is null)
cudaError_t norm_rows_f32(cudaStream_t s, const float* x, const int32_t* row_index, const void* w, bool f32, float gain_offset,
                          float eps, float* out, bf16* out_b16, int rows, int W);
// logits <- scale * logits, then cap * tanh(logits / cap) when cap > 0; in place on [rows, V]
cudaError_t softcap_rows(cudaStream_t s, float* logits, size_t n, float cap, float scale = 1.f);
// Clamped gated unit: g = min(G + bg, limit); u = clamp(U + bu, -limit, limit); out = g * sigmoid(act_alpha * g) * (u + 1)
// with G = gu[t, j], U = gu[t, F + j] (row stride ldg)
cudaError_t clamped_glu(cudaStream_t s, const float* gu, long ldg, const void* bias_g, const void* bias_u, bool f32, float limit,
                        float act_alpha, float* out, bf16* out_b16, int T, int F);

// ---- gated linear attention: S_t = diag(decay_t) S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t * q_scale, one fp32 state per
//      (sequence slot, head).  Step entries are token ranges [cu[b], cu[b+1]) of a packed batch; an entry whose first
//      position is 0 starts from the zero state, any other from its slot.
// decay[t, n] = sigmoid(z[t, n] + bias[n])^(1/tau) in fp32, in place on z (row stride ldz)
cudaError_t gla_decay(cudaStream_t s, float* z, long ldz, const void* bias, bool f32, float tau, int T, int N);
struct GlaArgs {
  const float* q; const float* k; const float* v; long ld;   // row stride shared by q / k / v (columns of one projection buffer)
  const float* decay; long ldd;                               // [T, H*Dk]
  float* out; long ldo;                                        // [T, H*Dv]
  float* state; long slot_stride;                              // state + slot * slot_stride -> [H][Dk][Dv] fp32 of this layer
  const int32_t* cu; const int32_t* first_pos; const int32_t* slots;  // [B+1], [B], [B]
  int B, H, Dk, Dv;
  float q_scale;
};
cudaError_t gla_recurrence(cudaStream_t s, const GlaArgs& a);
// out[t, h, :] = rmsnorm(o[t, h, :]) * w[:] * silu(g[t, h, :])   (per-head norm over Dv, gain shared by heads)
cudaError_t headnorm_silu_gate(cudaStream_t s, const float* o, long ldo, const float* g, long ldg, const void* w, bool f32, float eps,
                               float* out, bf16* out_b16, int T, int H, int Dv);

// ---- latent attention: the cache keeps, per token, the normed latent c [R] and one rotated key part [Dr] shared by all
//      heads (row = [c | k_rot], R + Dr elements, page-major: row index = page * page_size + offset).
// From the fused down-projection p[t] = [dq (Q) | dkv (R + Dr) | ...]: cq = rmsnorm(dq) * wq; c = rmsnorm(dkv[:R]) * wkv and
// k_rot = rotate(dkv[R:], pos) written to cache row slots[t].  kv_off < 0: the layer reads another layer's cache (no write).
struct LatentPrepArgs {
  const float* p; long ldp; int q_off, kv_off;
  const void* wq; const void* wkv; bool f32;
  float eps;
  float* cq; bf16* cq_b16; int Q;
  void* cache; const int32_t* slots; const int32_t* positions;
  int R, Dr, rope_dims; float rope_base;
  int T;
};
cudaError_t latent_prep(cudaStream_t s, const LatentPrepArgs& a);
// qabs[t, h, R:R+Dr] = rotate(q[t, h, Dk:Dk+Dr], pos)   (the absorbed part qabs[t, h, :R] comes from a batched GEMM with W_uk)
cudaError_t latent_q_rope(cudaStream_t s, const float* q, long ldq, float* qabs, long ldqa, const int32_t* positions, int T, int H,
                          int Dk, int Dr, int R, int rope_dims, float rope_base);
// Sliding-window attention of every head over the shared latent rows, softmax with a per-head sink in the denominator:
// ctx[t, h, :] = sum_j p_j c_j,  p_j = exp(s_j - m) / (sum_i exp(s_i - m) + exp(sink_h - m)),
// s_j = scale * qabs[t, h] . [c_j | k_rot_j] over 0 <= pos_t - j < window.
struct LatentAttnArgs {
  const float* qabs; long ldqa;     // [T, H*(R+Dr)]
  const void* cache; bool f32;      // [rows][R+Dr]
  const void* sink;                 // [H] weight type
  const int32_t* page_table; int max_pages, page_size;
  const int32_t* positions;         // [T]
  const int32_t* seq_of;            // [T] batch entry of each token
  float* ctx; long ldc;             // [T, H*R]
  int T, H, R, Dr, window;
  float scale;
};
cudaError_t latent_attn(cudaStream_t s, const LatentAttnArgs& a);
// The same attention as three dense products for a block of consecutive tokens of ONE sequence (long prompt portions in the
// bf16 mode; the two products run on the tcgen05 GEMM):
//   latent_gather:  kbuf[jj] = cache row of position k0 + jj (jj < nk), ct[r][jj] = its latent entry r (columns nk..ldk zero)
//   S = qabs16 . kbuf^T  (rows (token, head))        -> latent_softmax: masked, sink-normalised probabilities as bf16
//   ctx = P . ct^T
cudaError_t latent_gather(cudaStream_t s, const bf16* cache, const int32_t* page_table_row, int page_size, int k0, int nk, int R,
                          int Dr, bf16* kbuf, bf16* ct, int ldk);
// P[(tq, h), jj] = softmax over the keys position q0 + tq sees (0 <= q0 + tq - (k0 + jj) < window) with sink_h in the
// denominator; S and P have row stride ld, columns >= nk of P are written as zero
cudaError_t latent_softmax(cudaStream_t s, const float* S, bf16* P, int ld, int rows, int H, int q0, int k0, int nk, int window,
                           float scale, const bf16* sink);
// dst[h][r][d] = src[h][d][r] (bf16): the key up-projection per head, transposed once at load time
cudaError_t transpose_heads_bf16(cudaStream_t s, const bf16* src, bf16* dst, int H, int Dk, int R);
// out = o * sigmoid(g)
cudaError_t sigmoid_gate(cudaStream_t s, const float* o, long ldo, const float* g, long ldg, float* out, bf16* out_b16, int T, int N);
// f32 -> bf16 copy of a [T, N] block (row strides lds / ldd)
cudaError_t to_bf16_rows(cudaStream_t s, const float* src, long lds, bf16* dst, long ldd, int T, int N);

// ---- grouped-query attention over per-head key / value planes [page][kv_head][page_size][D | Dv] (stack_gqa.cu).
cudaError_t stack_gqa_init();
enum StackMask : int { MASK_WINDOW = 0, MASK_CHUNK = 1, MASK_CAUSAL = 2 };  // == hb_mask
// From the fused projection p[t] = [q (H*D) | k (G*D) | v (G*Dv, or the k columns again) | ...]: the first rope_dims entries of
// every q and k head turn by the angles of the step's table cs (pairing 1: entries (2i, 2i+1); 0: (i, i + rope_dims/2)),
// then q and k are divided by their root mean square over D when unit_norm.  q goes to q[t, h*D..] and / or its
// bf16 copy (either may be null),
// k and the UNTOUCHED v columns to the cache rows of slots[t] (slot < 0: no cache write).
struct GqaPrepArgs {
  const float* p; long ldp; int q_off, k_off, v_off;
  float* q; long ldq; bf16* q_b16;
  void* k_cache; void* v_cache; bool f32;
  const int32_t* slots; const int32_t* positions;
  const float* cs; int rope_dims, pairing;   // cs[t][2i], cs[t][2i+1] = cos, sin of positions[t] * f_i (stack_rope_table)
  int H, G, D, Dv, page_size;
  bool unit_norm; float eps;
  int T;
  // Options served by one block per token (any of them set): bias [q | k | v columns of p] of the cache element type added
  // first; proj_norm: q (and k) divided by the root mean square over ALL their heads' entries and multiplied by
  // qk_gain [H*D | G*D] (instead of unit_norm per head); blend_role 1: the (biased) values also go to v_first[t][G*Dv];
  // 2: values become (1 - l) v + l v_first[t], l = vmix[0], before they are cached.
  const void* bias = nullptr;
  bool proj_norm = false; const void* qk_gain = nullptr;
  int blend_role = 0; const void* vmix = nullptr; float* v_first = nullptr;
};
cudaError_t gqa_prep(cudaStream_t s, const GqaPrepArgs& a);
// cs[t][2i] = cos(a), cs[t][2i+1] = sin(a), a = positions[t] * freqs[i], i < half: the angle and its reduction to one turn in
// double precision, sine and cosine of the remainder in fp32.  Once per step and per distinct frequency set, shared by every
// layer and head that rotates with it.
cudaError_t stack_rope_table(cudaStream_t s, const int32_t* positions, const double* freqs, int half, float* cs, int T);
// out[t, h, :] = gate_h * sum_j p_j v_j over the keys position pos_t sees, p_j = exp(s_j) / (sum_i exp(s_i) + sink),
// s_j = scale * q[t, h] . k_j (head h reads kv head h / (H / G)).  Visible keys: mask 0 (window) pos - window < j <= pos;
// 1 (chunk) j <= pos in the block of `window` positions that holds pos; 2 (causal) j <= pos.  sink = 1 when unit_sink
// (a key with score 0 and no value), else 0.  gate_h = sigmoid(gate[t, h]) or 1 when gate is null.
struct GqaAttnArgs {
  const float* q; long ldq;
  const void* k_cache; const void* v_cache; bool f32;
  const int32_t* page_table; int max_pages, page_size;
  const int32_t* positions; const int32_t* seq_of;
  const float* gate; long ldg;
  float* out; long ldo; bf16* out_b16;
  int T, H, G, D, Dv, mask, window;
  bool unit_sink; float scale;
  float softcap = 0.f;         // > 0: s <- softcap * tanh(s / softcap) after the scale
  const void* sink = nullptr;  // [H] of the cache element type: exp(sink_h) joins the denominator (instead of unit_sink)
  // > 0: no position of this launch is beyond longest_ctx - 1, so the scores' shared memory is sized for that many keys instead
  // of a full context (launches that are not replayed from a graph, whose shared memory is fixed at capture)
  int longest_ctx = 0;
};
cudaError_t gqa_attn(cudaStream_t s, const GqaAttnArgs& a);
size_t gqa_attn_smem(int D, int Dv, int max_keys);  // dynamic shared memory the kernel needs to see max_keys keys
// out[t, h*Dv + i] = o[t, h*Dv + i] * sigmoid(gate[t, h])  (gate null: copy), o in bf16, out as fp32 + bf16 copy
cudaError_t head_gate_rows(cudaStream_t s, const bf16* o, long ldo, const float* gate, long ldg, float* out, bf16* out_b16, int T, int H,
                           int Dv);

// ---- gated delta rule (stack_delta.cu).  Step entries as for gla_recurrence; a state slot holds, per layer, S [H][D][Dv] and
//      the last taps - 1 inputs of the convolutions [taps - 1][2 G D + H Dv] (at float offset tail_off of the slot).
cudaError_t stack_delta_init();
// From the fused projection p[t] = [.. q (G*D) | k (G*D) | v (H*Dv) at off_qkv .. | b (H) at off_b | a (H) at off_a]:
// causal convolution over `taps` tokens per channel (conv_w [channels][taps], last tap = the token itself; inputs before the
// entry come from the slot, zeros before position 0), silu; q and k to unit vectors per head (q also times D^-1/2);
// out[t] = [q | k | v | beta = sigmoid(b) (H) | decay = exp(-exp(A_log) softplus(a + dt_bias)) (H) | k . q (G)]
struct DeltaPrepArgs {
  const float* p; long ldp; int off_qkv, off_b, off_a;
  const void* conv_w; const void* a_dt; bool f32;   // a_dt = [A_log (H) | dt_bias (H)]
  int taps;
  float* out; long ldo;
  float* state; long slot_stride; size_t tail_off;
  const int32_t* cu; const int32_t* first_pos; const int32_t* slots; const int32_t* seq_of;
  int T, B, H, G, D, Dv;
};
cudaError_t delta_prep(cudaStream_t s, const DeltaPrepArgs& a);
// after delta_prep of the same step: the slots' convolution inputs advance by the entries' tokens
cudaError_t delta_conv_tails(cudaStream_t s, const DeltaPrepArgs& a);
// S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q per (entry, head); query / key head of head h: h / (H / G)
struct DeltaArgs {
  const float* in; long ld;                       // delta_prep's rows
  int off_q, off_k, off_v, off_beta, off_decay, off_kq;
  float* out; long ldo;                           // [T, H*Dv]
  float* state; long slot_stride;                 // state + slot * slot_stride -> this layer's [H][D][Dv]
  const int32_t* cu; const int32_t* first_pos; const int32_t* slots;
  int B, H, G, D, Dv;
};
cudaError_t delta_recurrence(cudaStream_t s, const DeltaArgs& a);

// ---- short convolutions, scalar-decay linear recurrences (state-space layers, matrix memories), sublayers that share one
//      residual step (stack_ssm.cu).  Step entries as for gla_recurrence.
cudaError_t stack_ssm_init();
// Causal convolution over `taps` tokens per channel of C neighbouring columns of a projection buffer:
//   u_t[c] = in[t, off + c] (+ in_bias[bias_off + c]);  y_t[c] = act(sum_j w[c][j] u_(t - taps + 1 + j)[c] (+ bias[c]))
// with zeros before position 0; the taps - 1 inputs before an entry come from the slot ([taps - 1][C] at tail_off), and
// conv_tails (after short_conv of the same step) moves the slot's inputs on by the entry's tokens.  act: 0 none, 1 silu.
struct ConvArgs {
  const float* in; long ldi; int off;
  const void* in_bias; int bias_off;   // weight type, or null
  const void* w; const void* bias; bool f32;
  int taps, act;
  float* out; long ldo;
  float* state; long slot_stride; size_t tail_off;
  const int32_t* cu; const int32_t* first_pos; const int32_t* slots; const int32_t* seq_of;
  int T, B, C;
};
cudaError_t short_conv(cudaStream_t s, const ConvArgs& a);
cudaError_t conv_tails(cudaStream_t s, const ConvArgs& a);
// State-space step sizes: dt = softplus(p[t, off_dt + h] + dt_bias[h]); ab[t, h] = exp(-exp(A_log[h]) dt), ab[t, H + h] = dt
// (a_dt = [A_log (H) | dt_bias (H) | ...] of the weight type)
cudaError_t ssm_steps(cudaStream_t s, const float* p, long ldp, int off_dt, const void* a_dt, bool f32, float* ab, long ldab, int T, int H);
// Exponential gates of a matrix memory with their running maximum, one warp per (entry, head) scanning the entry's tokens:
//   i = cap tanh((p[t, off_i + h] + bias[off_i + h]) / cap);  f = logsigmoid(cap tanh((p[t, off_f + h] + bias[off_f + h]) / cap))
//   m_t = max(f + m_(t-1), i);  ab[t, h] = exp(f + m_(t-1) - m_t);  ab[t, H + h] = exp(i - m_t);  ab[t, 2H + h] = exp(-m_t)
// m lives in the slot ([H] floats at m_off) and starts at 0 when the entry starts at position 0.
struct GateScanArgs {
  const float* p; long ldp; int off_i, off_f;
  const void* bias; bool f32;   // [.. off_i .. off_f ..] of the weight type, or null
  float cap;
  float* ab; long ldab;
  float* state; long slot_stride; size_t m_off;
  const int32_t* cu; const int32_t* first_pos; const int32_t* slots;
  int B, H;
};
cudaError_t exp_gate_scan(cudaStream_t s, const GateScanArgs& a);
// S_t = a_t S_(t-1) + b_t k_t v_t^T;  out_t = q_scale * S_t^T q_t (+ skip[h] v_t) per (entry, head); query / key head of
// head h: h / (H / G); a_t = ab[t, h], b_t = ab[t, H + h].  With nq: the vector n_t = a_t n_(t-1) + b_t k_t ([H][Dk] at
// n_off of the slot) is carried too and nq[t, h] = q_scale * n_t . q_t.  S: [H][Dk][Dv] fp32 at s_off of the slot.
struct LinRecArgs {
  const float* q; long ldq; int q_off;
  const float* k; long ldk; int k_off;
  const float* v; long ldv; int v_off;
  const float* ab; long ldab;
  float* out; long ldo;
  float* nq; long ldn;
  const void* skip; bool f32;
  float q_scale;
  float* state; long slot_stride; size_t s_off, n_off;
  const int32_t* cu; const int32_t* first_pos; const int32_t* slots;
  int B, H, G, Dk, Dv;
};
cudaError_t lin_recurrence(cudaStream_t s, const LinRecArgs& a);
// Matrix memory read-out: o = num[t, h, :] / (max(|nq[t, h]|, ab[t, 2H + h]) + 1e-6); out[t, col0 + h Dv + i] =
// o_i / rms(o) * w[h Dv + i] * sigmoid(g[t, h Dv + i]) * scale (+ bf16 copy at the same place of out_b16)
cudaError_t memory_readout(cudaStream_t s, const float* num, long ldnum, const float* nq, long ldn, const float* ab, long ldab,
                           const float* g, long ldg, const void* w, bool f32, float eps, float scale, float* out, bf16* out_b16,
                           long ldout, int col0, int T, int H, int Dv);
// State-space read-out: u = y[t, :] * silu(z[t, :]) over n entries, divided by its root mean square in `parts` equal parts,
// times w; out [T, n] (+ bf16 copy)
cudaError_t gated_group_norm(cudaStream_t s, const float* y, long ldy, const float* z, long ldz, const void* w, bool f32, float eps,
                             int parts, float* out, bf16* out_b16, int T, int n);
// out[t, col0 + e] = in[t, e] * sigmoid(g[t, e]) * scale, e < n (in: fp32, or bf16 when in_b16 is given instead)
cudaError_t gate_scale_rows(cudaStream_t s, const float* in, const bf16* in_b16, long ldi, const float* g, long ldg, float scale,
                            float* out, bf16* out_b16, long ldout, int col0, int T, int n);
// Sublayers that read the same stream and are added in one step:
//   v = x[row_index ? row_index[r] : r] (+ y[r]) (+ y2[r]) (+ bias_scale * bias);  x_out[r] = v (when given; may be x);
//   h1[r] = v / rms(v) * w1, h2[r] = v / rms(v) * w2 as fp32 and / or bf16 (each optional): one statistic serves both norms
cudaError_t parallel_step(cudaStream_t s, const float* x, const int32_t* row_index, const float* y, const float* y2, const void* bias,
                          float bias_scale, const void* w1, const void* w2, bool f32, float eps, float* x_out, float* h1, bf16* h1_b16,
                          float* h2, bf16* h2_b16, int rows, int W);
// out = relu(in)^2 (fp32 in, row stride ldi; fp32 and / or bf16 out, dense rows of n)
cudaError_t relu2_rows(cudaStream_t s, const float* in, long ldi, float* out, bf16* out_b16, int T, int n);
// the same on bf16 rows (tensor-core path)
cudaError_t relu2_rows_b16(cudaStream_t s, const bf16* in, long ldi, bf16* out, int T, int n);

// ---- gated feed-forward units and mixtures of experts (stack_moe.cu).
cudaError_t stack_moe_init();
enum GluAct : int { GLU_SILU = 0, GLU_GELU_TANH = 1, GLU_CLAMPED = 2 };
// GLU_CLAMPED: g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1); the others act(gate) * up.
// How a router turns logits into a choice.  softmax or sigmoid scores; the top_k largest of (score + correction) among the
// eligible outputs are chosen, lowest index first among equals: with groups > 1 the outputs form that many equal groups of
// neighbours, a group scores the sum of its two largest corrected scores and only the `keep` best groups are eligible.
// The weights are the chosen outputs' uncorrected scores, divided by their sum (+ 1e-20) when renorm, times scale.
struct RouteOpts {
  int sigmoid = 0, groups = 0, keep = 0, renorm = 0;
  float scale = 1.f;
};
// out[t, j] = act(gu[t, j]) * gu[t, F + j]   (row stride ldg; out may be null when only the bf16 copy is wanted)
// packed: the columns come from weights stored per 256-row tile as [128 gate | 128 up] (the layout of EPI_SWIGLU / EPI_GEGLU):
// gate j of tile i at column 256 i + j, its up at 256 i + 128 + j, output column 128 i + j (F a multiple of 128)
cudaError_t gated_unit(cudaStream_t s, const float* gu, long ldg, int act, float* out, bf16* out_b16, int T, int F, bool packed = false,
                       float limit = 0.f);
// Router: scores = softmax(z[t, :R]) in fp32; the top_k largest of (score + correction) are chosen, lowest index first among
// equals; ids[t, k] = chosen output, wts[t, k] = its score (not renormalised)
cudaError_t moe_route(cudaStream_t s, const float* z, long ldz, const void* correction, bool f32, int R, int top_k, int32_t* ids,
                      float* wts, int T, const RouteOpts& ro = RouteOpts());
// moe_route fused with the router's product: z = router x[t] in fp32 (router [R][W] of the weight type, held in shared
// memory: moe_router_smem(R, W, f32) <= 200 KB, else use gemm_rt + moe_route), then the same choice.  sms: blocks to launch
size_t moe_router_smem(int R, int W, bool f32);
cudaError_t moe_router(cudaStream_t s, const float* x, const void* router, const void* correction, bool f32, int R, int W, int top_k,
                       int32_t* ids, float* wts, int T, int sms, const RouteOpts& ro = RouteOpts());
// bf16 form of gated_unit for the tensor-core path: gu and out are bf16, F and ldg multiples of eight
cudaError_t gated_unit_b16(cudaStream_t s, const bf16* gu, long ldg, int act, bf16* out, int T, int F, float limit = 0.f);
// One block per (token, choice): y[(t, k), :] = down_e(silu(gate_e x_t) * (up_e x_t)) for ids[t, k] = e < E (rows of choices
// that name an identity output are left alone).  x_b16 != null: the unit reads the bf16 copy of x and rounds its inner
// activation to bf16, as the tensor-core path does.  w_gu: [E][2F][W] ([gate | up] rows), w_down: [E][W][F].
cudaError_t moe_expert_rows(cudaStream_t s, const float* x, const bf16* x_b16, const void* w_gu, const void* w_down, bool f32,
                            const int32_t* ids, int top_k, int E, int F, int W, float* y, int T, bool packed = false, int act = GLU_SILU,
                            float limit = 0.f);
// The same experts as grouped tensor-core products (bf16 mode): moe_group_rows sorts the (token, choice) items by expert into
// a row buffer of moe_group_max_rows(items, E) rows whose per-expert segments start on multiples of 128 rows (row_of[item] =
// its row or -1 for an identity output, src_of_row[row] = its token or -1, tile_group[row / 128] = the expert whose weights
// multiply that m tile — GemmArgs::m_tile_group); moe_gather_rows copies the tokens' bf16 rows into it (zeros elsewhere);
// moe_combine_rows is moe_combine over the row buffer (the experts' outputs as bf16, the sum in fp32).
int moe_group_max_rows(int n_items, int E);
cudaError_t moe_group_rows(cudaStream_t s, const int32_t* ids, int n_items, int top_k, int E, int32_t* row_of, int32_t* src_of_row,
                           int32_t* tile_group, int32_t* scratch);  // scratch: 3 E ints
cudaError_t moe_gather_rows(cudaStream_t s, const bf16* x16, int W, const int32_t* src_of_row, bf16* a16, int rows);
cudaError_t moe_combine_rows(cudaStream_t s, const float* x, const bf16* y, const int32_t* row_of, const float* wts, int top_k,
                             float* out, int T, int W, const float* add = nullptr);
// out[t, :] = (add ? add[t, :] : 0) + sum_k wts[t, k] * (ids[t, k] < E ? y[(t, k), :] : x[t, :]), k in order (add may be out)
cudaError_t moe_combine(cudaStream_t s, const float* x, const float* y, const int32_t* ids, const float* wts, int top_k, int E,
                        float* out, int T, int W, const float* add = nullptr);

}  // namespace hb
