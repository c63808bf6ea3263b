// Mechanisms of hybrid decoder stacks on a 32-bit residual stream: CUDA-core GEMM for exact / odd-shaped products,
// post-norm residual step, gated-linear-attention recurrence, windowed latent attention with a softmax sink, clamped
// gated unit, soft-capped logits.  Everything the recurrence and the softmax touch is fp32; weights and cache rows are
// bf16 or fp32 (template parameter WT / CT).  Summation orders are fixed per output element and do not depend on the
// batch a row travels in, so a position's result is the same whatever else the step carries.
#include <math.h>

#include "kernels.h"
#include "launch.h"
#include "stack_common.cuh"

namespace hb {
namespace {

// ------------------------------------------------------------------ CUDA-core GEMM
constexpr int GT = 64, GK = 16;
template <typename WT>
__global__ void __launch_bounds__(256) gemm_rt_kernel(const float* __restrict__ A, long lda, long a_bs, const WT* __restrict__ W,
                                                      long w_sn, long w_sk, long w_bs, float* __restrict__ C, long ldc, long c_bs,
                                                      const WT* __restrict__ bias, int M, int N, int K) {
  __shared__ float As[GK][GT + 4];
  __shared__ float Ws[GK][GT + 4];
  const int z = blockIdx.z;
  A += (size_t)z * a_bs;
  W += (size_t)z * w_bs;
  C += (size_t)z * c_bs;
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;  // loader: row lr of the tile, 4 consecutive k
  for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int m = m0 + lr, n = n0 + lr;
      As[lk + i][lr] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.f;
      Ws[lk + i][lr] = (n < N && k < K) ? ldf<WT>(W, (size_t)n * w_sn + (size_t)k * w_sk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j] + (bias ? ldf<WT>(bias, n) : 0.f);
    }
  }
}

// ------------------------------------------------------------------ row kernels
template <typename WT>
__global__ void embed_rows_kernel(const int32_t* __restrict__ tokens, const WT* __restrict__ table, float* __restrict__ x,
                                  bf16* __restrict__ xb, int W, float scale) {
  const int t = blockIdx.x;
  const WT* src = table + (size_t)tokens[t] * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = ldf<WT>(src, i) * scale;
    x[(size_t)t * W + i] = v;
    if (xb) xb[(size_t)t * W + i] = __float2bfloat16(v);
  }
}

// out = rmsnorm(alpha * x + y + bias) * (off + w); y == nullptr: plain norm of x (alpha = 1).  add_x: the norm covers the
// sublayer's output only and the stream is added afterwards, out = x + rmsnorm(y + bias) * (off + w).
// dynamic smem: W floats + 32.  x / out are not __restrict__: the residual steps update the stream in place.
template <typename WT>
__global__ void __launch_bounds__(256) postnorm_kernel(const float* x, const int32_t* __restrict__ row_index,
                                                       const float* __restrict__ y, long ldy, const WT* __restrict__ bias,
                                                       const WT* __restrict__ w, float alpha, float off, float eps,
                                                       float* out, bf16* __restrict__ outb, int W, int add_x) {
  extern __shared__ float sm[];
  float* row = sm;
  float* red = sm + W;
  const int r = blockIdx.x;
  const size_t src = row_index ? (size_t)row_index[r] : (size_t)r;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = add_x ? 0.f : x[src * W + i];
    if (y) v = alpha * v + y[(size_t)r * ldy + i] + (bias ? ldf<WT>(bias, i) : 0.f);
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float rs = 1.f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = row[i] * rs * (off + ldf<WT>(w, i));
    if (add_x) v += x[src * W + i];
    out[(size_t)r * W + i] = v;
    if (outb) outb[(size_t)r * W + i] = __float2bfloat16(v);
  }
}

// The same step with the row held in registers as float4 (W a multiple of 4, W <= 4 * 256 * kPnChunks)
constexpr int kPnChunks = 8;
template <typename WT>
__global__ void __launch_bounds__(256) postnorm_vec_kernel(const float* x, const int32_t* __restrict__ row_index,
                                                           const float* __restrict__ y, long ldy, const WT* __restrict__ bias,
                                                           const WT* __restrict__ w, float alpha, float off, float eps,
                                                           float* out, bf16* __restrict__ outb, int W, int add_x) {
  __shared__ float red[32];
  const int r = blockIdx.x;
  const size_t src = row_index ? (size_t)row_index[r] : (size_t)r;
  const int nv = W / 4;
  float4 v[kPnChunks];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kPnChunks; ++c) {
    const int i = threadIdx.x + c * 256;
    if (i < nv) {
      float4 a = add_x ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(x + src * W + 4 * i);
      if (y) {
        const float4 b = *reinterpret_cast<const float4*>(y + (size_t)r * ldy + 4 * i);
        a.x = alpha * a.x + b.x + (bias ? ldf<WT>(bias, 4 * i) : 0.f);
        a.y = alpha * a.y + b.y + (bias ? ldf<WT>(bias, 4 * i + 1) : 0.f);
        a.z = alpha * a.z + b.z + (bias ? ldf<WT>(bias, 4 * i + 2) : 0.f);
        a.w = alpha * a.w + b.w + (bias ? ldf<WT>(bias, 4 * i + 3) : 0.f);
      }
      v[c] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  ss = block_sum(ss, red);
  const float rs = 1.f / sqrtf(ss / (float)W + eps);
#pragma unroll
  for (int c = 0; c < kPnChunks; ++c) {
    const int i = threadIdx.x + c * 256;
    if (i < nv) {
      float4 a = v[c];
      a.x *= rs * (off + ldf<WT>(w, 4 * i));
      a.y *= rs * (off + ldf<WT>(w, 4 * i + 1));
      a.z *= rs * (off + ldf<WT>(w, 4 * i + 2));
      a.w *= rs * (off + ldf<WT>(w, 4 * i + 3));
      if (add_x) {
        const float4 b = *reinterpret_cast<const float4*>(x + src * W + 4 * i);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
      }
      *reinterpret_cast<float4*>(out + (size_t)r * W + 4 * i) = a;
      if (outb) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
        uint2 pk;
        pk.x = *reinterpret_cast<unsigned*>(&lo);
        pk.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(outb + (size_t)r * W + 4 * i) = pk;
      }
    }
  }
}

__global__ void softcap_kernel(float* __restrict__ z, size_t n, float cap, float scale) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = z[i] * scale;
    z[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}

// Element-wise norms N(v) = tanh(alpha v) * w + b (a block [w (W) | b (W) | alpha] of the weight type; no row statistic) around
// the residual step: v = x[src]; with y: v += post ? N_post(y[r]) : y[r], stored to x_out[r]; with pre: h[r] = N_pre(v) as
// fp32 and / or bf16.  One launch serves "add the normed output of one sublayer and norm the input of the next".
// x / x_out are not __restrict__: the step updates the stream in place.
template <typename WT, int VEC>
__global__ void __launch_bounds__(256) tanh_norm_kernel(const float* x, const int32_t* __restrict__ row_index, const float* __restrict__ y,
                                                        long ldy, const WT* __restrict__ post, const WT* __restrict__ pre, float* x_out,
                                                        float* __restrict__ h, bf16* __restrict__ hb, int W) {
  const size_t r = blockIdx.y;
  const size_t src = row_index ? (size_t)row_index[r] : r;
  const int i0 = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (i0 >= W) return;
  const float a_post = post ? ldf<WT>(post, 2 * (size_t)W) : 0.f, a_pre = pre ? ldf<WT>(pre, 2 * (size_t)W) : 0.f;
  float v[VEC], hv[VEC];
  if (VEC == 4) {
    const float4 t4 = *reinterpret_cast<const float4*>(x + src * W + i0);
    v[0] = t4.x; v[1] = t4.y; v[2] = t4.z; v[VEC - 1] = t4.w;
  } else {
    v[0] = x[src * W + i0];
  }
  if (y) {
    float yv[VEC];
    if (VEC == 4) {
      const float4 t4 = *reinterpret_cast<const float4*>(y + r * ldy + i0);
      yv[0] = t4.x; yv[1] = t4.y; yv[2] = t4.z; yv[VEC - 1] = t4.w;
    } else {
      yv[0] = y[r * ldy + i0];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      v[e] += post ? fmaf(tanhf(a_post * yv[e]), ldf<WT>(post, i0 + e), ldf<WT>(post, (size_t)W + i0 + e)) : yv[e];
    if (VEC == 4) *reinterpret_cast<float4*>(x_out + r * W + i0) = make_float4(v[0], v[1], v[2], v[VEC - 1]);
    else x_out[r * W + i0] = v[0];
  }
  if (pre) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) hv[e] = fmaf(tanhf(a_pre * v[e]), ldf<WT>(pre, i0 + e), ldf<WT>(pre, (size_t)W + i0 + e));
    if (VEC == 4) {
      if (h) *reinterpret_cast<float4*>(h + r * W + i0) = make_float4(hv[0], hv[1], hv[2], hv[VEC - 1]);
      if (hb) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(hv[0], hv[1]), hi = __floats2bfloat162_rn(hv[2], hv[VEC - 1]);
        uint2 pk;
        pk.x = *reinterpret_cast<unsigned*>(&lo);
        pk.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(hb + r * W + i0) = pk;
      }
    } else {
      if (h) h[r * W + i0] = hv[0];
      if (hb) hb[r * W + i0] = __float2bfloat16(hv[0]);
    }
  }
}

__device__ __forceinline__ float clamped_glu_one(float g, float u, float limit, float act_alpha) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * sigmoidf_(act_alpha * g) * (u + 1.f);
}
// VEC = 4: F and ldg are multiples of four (16-byte loads and stores)
template <typename WT, int VEC>
__global__ void clamped_glu_kernel(const float* __restrict__ gu, long ldg, const WT* __restrict__ bg, const WT* __restrict__ bu,
                                   float limit, float act_alpha, float* __restrict__ out, bf16* __restrict__ outb, int F) {
  const int t = blockIdx.y;
  const int j = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (j >= F) return;
  if (VEC == 4) {
    const float4 g4 = *reinterpret_cast<const float4*>(gu + (size_t)t * ldg + j);
    const float4 u4 = *reinterpret_cast<const float4*>(gu + (size_t)t * ldg + F + j);
    const float g[4] = {g4.x, g4.y, g4.z, g4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w};
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      v[e] = clamped_glu_one(g[e] + (bg ? ldf<WT>(bg, j + e) : 0.f), u[e] + (bu ? ldf<WT>(bu, j + e) : 0.f), limit, act_alpha);
    *reinterpret_cast<float4*>(out + (size_t)t * F + j) = make_float4(v[0], v[1], v[2], v[3]);
    if (outb) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<unsigned*>(&lo);
      pk.y = *reinterpret_cast<unsigned*>(&hi);
      *reinterpret_cast<uint2*>(outb + (size_t)t * F + j) = pk;
    }
  } else {
    const float v = clamped_glu_one(gu[(size_t)t * ldg + j] + (bg ? ldf<WT>(bg, j) : 0.f),
                                    gu[(size_t)t * ldg + F + j] + (bu ? ldf<WT>(bu, j) : 0.f), limit, act_alpha);
    out[(size_t)t * F + j] = v;
    if (outb) outb[(size_t)t * F + j] = __float2bfloat16(v);
  }
}

__global__ void sigmoid_gate_kernel(const float* __restrict__ o, long ldo, const float* __restrict__ g, long ldg,
                                    float* __restrict__ out, bf16* __restrict__ outb, int N) {
  const int t = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= N) return;
  const float v = o[(size_t)t * ldo + j] * sigmoidf_(g[(size_t)t * ldg + j]);
  out[(size_t)t * N + j] = v;
  if (outb) outb[(size_t)t * N + j] = __float2bfloat16(v);
}

// VEC = 4: N, both strides and both bases are multiples of four elements (16-byte loads, 8-byte stores)
template <int VEC>
__global__ void to_bf16_kernel(const float* __restrict__ src, long lds, bf16* __restrict__ dst, long ldd, int N) {
  const int t = blockIdx.y;
  const int j = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (j >= N) return;
  if (VEC == 4) {
    const float4 v = *reinterpret_cast<const float4*>(src + (size_t)t * lds + j);
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo);
    u.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(dst + (size_t)t * ldd + j) = u;
  } else {
    dst[(size_t)t * ldd + j] = __float2bfloat16(src[(size_t)t * lds + j]);
  }
}

// ------------------------------------------------------------------ gated linear attention
template <typename WT>
__global__ void gla_decay_kernel(float* __restrict__ z, long ldz, const WT* __restrict__ bias, float inv_tau, int N) {
  const int t = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= N) return;
  const float v = z[(size_t)t * ldz + j] + (bias ? ldf<WT>(bias, j) : 0.f);
  // log sigmoid(v) = -softplus(-v), evaluated without overflow on either side
  const float ls = (v >= 0.f) ? -log1pf(expf(-v)) : v - log1pf(expf(v));
  z[(size_t)t * ldz + j] = expf(ls * inv_tau);
}

constexpr int kGlaTch = 16;  // tokens per shared-memory stage of the recurrence
__device__ __forceinline__ void cp_async4(float* smem_dst, const float* gsrc) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Block = (entry, head, 32 value columns), DKP/16 warps: warp w owns key channels [16w, 16w+16) of the state (16 fp32
// registers per thread), so a block of one slice still puts several warps on every scheduler.  Tokens are staged 16 at a
// time through a cp.async double buffer; each warp leaves its partial dot products in shared memory and the block adds
// them in warp order once per stage.
template <int DKP>
__global__ void __launch_bounds__(DKP * 2) gla_recurrence_kernel(GlaArgs a) {
  constexpr int KS = DKP / 16;
  constexpr int per_tok = 3 * DKP + 32, stage_floats = kGlaTch * per_tok;
  extern __shared__ float sm[];  // 2 stages x [kGlaTch][3 * DKP + 32] + partial outputs [kGlaTch][KS][32]
  float* obuf = sm + 2 * stage_floats;
  const int b = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int j = blockIdx.z * 32 + lane;
  const bool live = j < a.Dv;
  const int t0 = a.cu[b], t1 = a.cu[b + 1];
  const int Dk = a.Dk, i0 = w * 16;
  float* st = a.state + (size_t)a.slots[b] * a.slot_stride + (size_t)h * Dk * a.Dv;
  float S[16];
  const bool fresh = a.first_pos[b] == 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) S[i] = (!fresh && live && i0 + i < Dk) ? st[(size_t)(i0 + i) * a.Dv + j] : 0.f;
  // padded key channels read zeros: clear the stages once, the copies below only touch i < Dk
  for (int e = threadIdx.x; e < 2 * stage_floats; e += blockDim.x) sm[e] = 0.f;
  __syncthreads();
  auto issue = [&](int tc, int stage) {
    const int nt = min(kGlaTch, t1 - tc);
    float* base = sm + stage * stage_floats;
    for (int e = threadIdx.x; e < nt * Dk; e += blockDim.x) {
      const int tt = e / Dk, i = e % Dk;
      const size_t row = (size_t)(tc + tt);
      float* dst = base + tt * per_tok;
      cp_async4(dst + i, a.q + row * a.ld + h * Dk + i);
      cp_async4(dst + DKP + i, a.k + row * a.ld + h * Dk + i);
      cp_async4(dst + 2 * DKP + i, a.decay + row * a.ldd + h * Dk + i);
    }
    for (int e = threadIdx.x; e < nt * 32; e += blockDim.x) {
      const int tt = e >> 5, c = e & 31;
      if (blockIdx.z * 32 + c < a.Dv) cp_async4(base + tt * per_tok + 3 * DKP + c, a.v + (size_t)(tc + tt) * a.ld + (size_t)h * a.Dv + blockIdx.z * 32 + c);
    }
    cp_async_commit();
  };
  if (t0 < t1) issue(t0, 0);
  int stage = 0;
  for (int tc = t0; tc < t1; tc += kGlaTch, stage ^= 1) {
    const int nt = min(kGlaTch, t1 - tc);
    if (tc + kGlaTch < t1) {
      issue(tc + kGlaTch, stage ^ 1);  // next tokens travel while these are consumed
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* base = sm + stage * stage_floats;
    for (int tt = 0; tt < nt; ++tt) {
      const float* tk = base + tt * per_tok;
      const float vj = tk[3 * DKP + lane];
      const float4* q4 = reinterpret_cast<const float4*>(tk + i0);
      const float4* k4 = reinterpret_cast<const float4*>(tk + DKP + i0);
      const float4* d4 = reinterpret_cast<const float4*>(tk + 2 * DKP + i0);
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 q = q4[i], k = k4[i], d = d4[i];
        S[4 * i + 0] = fmaf(d.x, S[4 * i + 0], k.x * vj); o0 = fmaf(S[4 * i + 0], q.x, o0);
        S[4 * i + 1] = fmaf(d.y, S[4 * i + 1], k.y * vj); o1 = fmaf(S[4 * i + 1], q.y, o1);
        S[4 * i + 2] = fmaf(d.z, S[4 * i + 2], k.z * vj); o2 = fmaf(S[4 * i + 2], q.z, o2);
        S[4 * i + 3] = fmaf(d.w, S[4 * i + 3], k.w * vj); o3 = fmaf(S[4 * i + 3], q.w, o3);
      }
      obuf[(tt * KS + w) * 32 + lane] = (o0 + o1) + (o2 + o3);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < nt * 32; e += blockDim.x) {
      const int tt = e >> 5, c = e & 31;
      float o = 0.f;
#pragma unroll
      for (int ww = 0; ww < KS; ++ww) o += obuf[(tt * KS + ww) * 32 + c];
      if (blockIdx.z * 32 + c < a.Dv) a.out[(size_t)(tc + tt) * a.ldo + (size_t)h * a.Dv + blockIdx.z * 32 + c] = o * a.q_scale;
    }
    __syncthreads();  // the stage and the partial outputs are rewritten in the next iteration
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i0 + i < Dk) st[(size_t)(i0 + i) * a.Dv + j] = S[i];
  }
}

// one warp per (token, head)
template <typename WT>
__global__ void headnorm_gate_kernel(const float* __restrict__ o, long ldo, const float* __restrict__ g, long ldg,
                                     const WT* __restrict__ w, float eps, float* __restrict__ out, bf16* __restrict__ outb, int T,
                                     int H, int Dv) {
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= T * H) return;
  const int t = item / H, h = item % H, l = threadIdx.x & 31;
  const float* src = o + (size_t)t * ldo + (size_t)h * Dv;
  const float* gs = g + (size_t)t * ldg + (size_t)h * Dv;
  float ss = 0.f;
  for (int i = l; i < Dv; i += 32) ss += src[i] * src[i];
  ss = warp_sum(ss);
  const float rs = 1.f / sqrtf(ss / (float)Dv + eps);
  for (int i = l; i < Dv; i += 32) {
    const float gv = gs[i];
    const float v = src[i] * rs * ldf<WT>(w, i) * (gv * sigmoidf_(gv));
    const size_t d = (size_t)t * H * Dv + (size_t)h * Dv + i;
    out[d] = v;
    if (outb) outb[d] = __float2bfloat16(v);
  }
}

// ------------------------------------------------------------------ latent attention
// angle of pair i at position p: p * base^(-2i/dims), in fp32
__device__ __forceinline__ void rope_pair(float u, float v, int pos, int i, int dims, float base, float* ou, float* ov) {
  const float f = powf(base, -2.f * (float)i / (float)dims);
  float s, c;
  sincosf((float)pos * f, &s, &c);
  *ou = u * c - v * s;
  *ov = v * c + u * s;
}

template <typename WT, typename CT>
__global__ void __launch_bounds__(128) latent_prep_kernel(LatentPrepArgs a) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const float* p = a.p + (size_t)t * a.ldp;
  {
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.Q; i += blockDim.x) ss += p[a.q_off + i] * p[a.q_off + i];
    ss = block_sum(ss, red);
    const float rs = 1.f / sqrtf(ss / (float)a.Q + a.eps);
    for (int i = threadIdx.x; i < a.Q; i += blockDim.x) {
      const float v = p[a.q_off + i] * rs * ldf<WT>((const WT*)a.wq, i);
      a.cq[(size_t)t * a.Q + i] = v;
      if (a.cq_b16) a.cq_b16[(size_t)t * a.Q + i] = __float2bfloat16(v);
    }
  }
  if (a.kv_off < 0) return;
  const int slot = a.slots[t];
  if (slot < 0) return;
  CT* row = (CT*)a.cache + (size_t)slot * (a.R + a.Dr);
  const float* kv = p + a.kv_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < a.R; i += blockDim.x) ss += kv[i] * kv[i];
  ss = block_sum(ss, red);
  const float rs = 1.f / sqrtf(ss / (float)a.R + a.eps);
  for (int i = threadIdx.x; i < a.R; i += blockDim.x) stf<CT>(row, i, kv[i] * rs * ldf<WT>((const WT*)a.wkv, i));
  const int half = a.rope_dims / 2, pos = a.positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float u, v;
    rope_pair(kv[a.R + i], kv[a.R + half + i], pos, i, a.rope_dims, a.rope_base, &u, &v);
    stf<CT>(row, a.R + i, u);
    stf<CT>(row, a.R + half + i, v);
  }
  for (int i = a.rope_dims + threadIdx.x; i < a.Dr; i += blockDim.x) stf<CT>(row, a.R + i, kv[a.R + i]);
}

__global__ void latent_q_rope_kernel(const float* __restrict__ q, long ldq, float* __restrict__ qabs, long ldqa,
                                     const int32_t* __restrict__ positions, int H, int Dk, int Dr, int R, int rope_dims, float base) {
  const int t = blockIdx.x, pos = positions[t], half = rope_dims / 2;
  for (int e = threadIdx.x; e < H * Dr; e += blockDim.x) {
    const int h = e / Dr, i = e % Dr;
    const float* src = q + (size_t)t * ldq + (size_t)h * (Dk + Dr) + Dk;
    float* dst = qabs + (size_t)t * ldqa + (size_t)h * (R + Dr) + R;
    if (i < half) {
      float u, v;
      rope_pair(src[i], src[half + i], pos, i, rope_dims, base, &u, &v);
      dst[i] = u;
      dst[half + i] = v;
    } else if (i >= rope_dims) {
      dst[i] = src[i];
    }
  }
}

// One block per (token, group of kLatHG heads), kLatThreads threads.  Every head of a token reads the same cache rows, so a
// block serves several heads from one pass over them.  dynamic smem: q [HG][D] + scores [window][HG] + page-resolved row
// index [window] + group partials [threads][HG] + 32.
// Scores: one warp per key (16-byte loads of bf16 rows when the row length allows), HG dot products per loaded row.
// Weighted sum: thread (g, r) adds the keys jj = g mod G of latent entry r for all HG heads; groups are then summed in group
// order — fixed per (R, threads), independent of the batch.
constexpr int kLatThreads = 1024;
constexpr int kLatHG = 4;
template <typename WT, typename CT>
__global__ void __launch_bounds__(kLatThreads) latent_attn_kernel(LatentAttnArgs a) {
  constexpr int HG = kLatHG;
  extern __shared__ float sm[];
  const int D = a.R + a.Dr, Dp = (D + 3) / 4 * 4;
  float* qs = sm;                       // [HG][Dp]
  float* sc = qs + HG * Dp;             // [window][HG]
  float* part = sc + HG * a.window;     // [8 * threads]: group partials of the weighted sum
  float* red = part + 8 * blockDim.x;   // [32 * HG]
  int* rowoff = reinterpret_cast<int*>(red + 32 * HG);  // [window] cache row of every visible key (page lookup done once)
  const int t = blockIdx.x, h0 = blockIdx.y * HG;
  const int nh = min(HG, a.H - h0);
  const int pos = a.positions[t];
  const int n = min(pos + 1, a.window), j0 = pos - n + 1;  // keys j0 .. pos
  const int32_t* pt = a.page_table + (size_t)a.seq_of[t] * a.max_pages;
  const CT* cache = (const CT*)a.cache;
  for (int e = threadIdx.x; e < HG * Dp; e += blockDim.x) {
    const int hh = e / Dp, i = e % Dp;
    qs[e] = (hh < nh && i < D) ? a.qabs[(size_t)t * a.ldqa + (size_t)(h0 + hh) * D + i] : 0.f;
  }
  for (int jj = threadIdx.x; jj < n; jj += blockDim.x) {
    const int j = j0 + jj;
    rowoff[jj] = pt[j / a.page_size] * a.page_size + j % a.page_size;
  }
  __syncthreads();
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (sizeof(CT) == 2 && (D & 7) == 0) {
    // bf16 rows that start on 16-byte boundaries: two keys per iteration, their loads issued together
    for (int jj = w; jj < n; jj += 2 * nw) {
      const int jb = jj + nw;
      const bool two = jb < n;
      const bf16* ra = reinterpret_cast<const bf16*>(cache) + (size_t)rowoff[jj] * D;
      const bf16* rb = reinterpret_cast<const bf16*>(cache) + (size_t)rowoff[two ? jb : jj] * D;
      float sa[HG] = {}, sb[HG] = {};
      for (int i = l * 8; i < D; i += 256) {
        const uint4 ua = *reinterpret_cast<const uint4*>(ra + i), ub = *reinterpret_cast<const uint4*>(rb + i);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ua);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&ub);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fa = __bfloat1622float2(pa[e]), fb = __bfloat1622float2(pb[e]);
#pragma unroll
          for (int hh = 0; hh < HG; ++hh) {
            const float2 q = *reinterpret_cast<const float2*>(qs + hh * Dp + i + 2 * e);
            sa[hh] = fmaf(q.x, fa.x, sa[hh]); sa[hh] = fmaf(q.y, fa.y, sa[hh]);
            sb[hh] = fmaf(q.x, fb.x, sb[hh]); sb[hh] = fmaf(q.y, fb.y, sb[hh]);
          }
        }
      }
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) {
        sa[hh] = warp_sum(sa[hh]);
        sb[hh] = warp_sum(sb[hh]);
      }
      if (l == 0) {
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) {
          sc[jj * HG + hh] = sa[hh] * a.scale;
          if (two) sc[jb * HG + hh] = sb[hh] * a.scale;
        }
      }
    }
  }
  for (int jj = (sizeof(CT) == 2 && (D & 7) == 0) ? n : w; jj < n; jj += nw) {  // rows read element by element
    const CT* row = cache + (size_t)rowoff[jj] * D;
    float s[HG] = {};
    for (int i = l; i < D; i += 32) {
      const float kv = ldf<CT>(row, i);
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) s[hh] = fmaf(qs[hh * Dp + i], kv, s[hh]);
    }
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) s[hh] = warp_sum(s[hh]);
    if (l == 0) {
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) sc[jj * HG + hh] = s[hh] * a.scale;
    }
  }
  __syncthreads();
  // fp32 softmax with the sink in the denominator; the HG heads share each block reduction
  float inv[HG], mx[HG], sink[HG];
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) mx[hh] = sink[hh] = hh < nh ? ldf<WT>((const WT*)a.sink, h0 + hh) : 0.f;
  for (int jj = threadIdx.x; jj < n; jj += blockDim.x) {
    const float4 v = *reinterpret_cast<const float4*>(sc + jj * HG);
    mx[0] = fmaxf(mx[0], v.x); mx[1] = fmaxf(mx[1], v.y); mx[2] = fmaxf(mx[2], v.z); mx[3] = fmaxf(mx[3], v.w);
  }
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) mx[hh] = warp_max(mx[hh]);
  __syncthreads();
  if (l == 0) {
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) red[w * HG + hh] = mx[hh];
  }
  __syncthreads();
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) mx[hh] = warp_max(l < nw ? red[l * HG + hh] : -INFINITY);
  float sum[HG] = {};
  for (int jj = threadIdx.x; jj < n; jj += blockDim.x) {
    float4 v = *reinterpret_cast<const float4*>(sc + jj * HG);
    v.x = expf(v.x - mx[0]); v.y = expf(v.y - mx[1]); v.z = expf(v.z - mx[2]); v.w = expf(v.w - mx[3]);
    *reinterpret_cast<float4*>(sc + jj * HG) = v;
    sum[0] += v.x; sum[1] += v.y; sum[2] += v.z; sum[3] += v.w;
  }
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) sum[hh] = warp_sum(sum[hh]);
  __syncthreads();  // every thread has read the maxima
  if (l == 0) {
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) red[w * HG + hh] = sum[hh];
  }
  __syncthreads();  // also publishes the exponentials in sc[]
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) inv[hh] = 1.f / (warp_sum(l < nw ? red[l * HG + hh] : 0.f) + expf(sink[hh] - mx[hh]));
  if (sizeof(CT) == 2 && (D & 7) == 0 && (a.R & 7) == 0 && a.R / 8 <= (int)blockDim.x) {
    // bf16 rows: a thread owns 8 consecutive latent entries (one 16-byte load per key), the block's threads form G groups
    // that take every G-th key, so many loads are in flight per SM; groups are summed in group order, one head at a time
    const int RC = a.R / 8, G = blockDim.x / RC, g = threadIdx.x / RC, c = threadIdx.x % RC;
    const bf16* base = reinterpret_cast<const bf16*>(cache) + c * 8;
    float acc[HG][8] = {};
    auto add_key = [&](const uint4& u, const float4& p) {
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&u);
      const float pw[HG] = {p.x, p.y, p.z, p.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p2[e]);
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) {
          acc[hh][2 * e] = fmaf(pw[hh], f.x, acc[hh][2 * e]);
          acc[hh][2 * e + 1] = fmaf(pw[hh], f.y, acc[hh][2 * e + 1]);
        }
      }
    };
    if (g < G) {
      int jj = g;
      for (; jj + G < n; jj += 2 * G) {  // two rows in flight; added in key order
        const uint4 u0 = *reinterpret_cast<const uint4*>(base + (size_t)rowoff[jj] * D);
        const uint4 u1 = *reinterpret_cast<const uint4*>(base + (size_t)rowoff[jj + G] * D);
        add_key(u0, *reinterpret_cast<const float4*>(sc + jj * HG));
        add_key(u1, *reinterpret_cast<const float4*>(sc + (jj + G) * HG));
      }
      if (jj < n) add_key(*reinterpret_cast<const uint4*>(base + (size_t)rowoff[jj] * D), *reinterpret_cast<const float4*>(sc + jj * HG));
    }
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) {
      __syncthreads();
      if (g < G) {
#pragma unroll
        for (int e = 0; e < 8; ++e) part[g * a.R + c * 8 + e] = acc[hh][e];
      }
      __syncthreads();
      if (hh < nh)
        for (int r = threadIdx.x; r < a.R; r += blockDim.x) {
          float tot = 0.f;
          for (int gg = 0; gg < G; ++gg) tot += part[gg * a.R + r];
          a.ctx[(size_t)t * a.ldc + (size_t)(h0 + hh) * a.R + r] = tot * inv[hh];
        }
    }
    return;
  }
  const int Rp = (a.R + 31) / 32 * 32;
  const int G = max(1, (int)blockDim.x / Rp);
  for (int r0 = 0; r0 < a.R; r0 += blockDim.x) {  // one pass unless the latent is wider than the block
    const int g = (G > 1) ? threadIdx.x / Rp : 0, r = r0 + ((G > 1) ? threadIdx.x % Rp : threadIdx.x);
    float acc[HG] = {};
    if (g < G && r < a.R) {
      const CT* col = cache + r;
      int jj = g;
      for (; jj + G < n; jj += 2 * G) {  // two independent loads in flight; the sum keeps key order
        const float c0 = ldf<CT>(col, (size_t)rowoff[jj] * D), c1 = ldf<CT>(col, (size_t)rowoff[jj + G] * D);
        const float4 p0 = *reinterpret_cast<const float4*>(sc + jj * HG), p1 = *reinterpret_cast<const float4*>(sc + (jj + G) * HG);
        acc[0] = fmaf(p0.x, c0, acc[0]); acc[1] = fmaf(p0.y, c0, acc[1]); acc[2] = fmaf(p0.z, c0, acc[2]); acc[3] = fmaf(p0.w, c0, acc[3]);
        acc[0] = fmaf(p1.x, c1, acc[0]); acc[1] = fmaf(p1.y, c1, acc[1]); acc[2] = fmaf(p1.z, c1, acc[2]); acc[3] = fmaf(p1.w, c1, acc[3]);
      }
      for (; jj < n; jj += G) {
        const float c0 = ldf<CT>(col, (size_t)rowoff[jj] * D);
        const float4 p0 = *reinterpret_cast<const float4*>(sc + jj * HG);
        acc[0] = fmaf(p0.x, c0, acc[0]); acc[1] = fmaf(p0.y, c0, acc[1]); acc[2] = fmaf(p0.z, c0, acc[2]); acc[3] = fmaf(p0.w, c0, acc[3]);
      }
    }
    if (G > 1) {
      __syncthreads();
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) part[threadIdx.x * HG + hh] = acc[hh];
      __syncthreads();
      if (threadIdx.x < a.R) {
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) {
          float tot = 0.f;
          for (int gg = 0; gg < G; ++gg) tot += part[(gg * Rp + threadIdx.x) * HG + hh];
          if (hh < nh) a.ctx[(size_t)t * a.ldc + (size_t)(h0 + hh) * a.R + threadIdx.x] = tot * inv[hh];
        }
      }
    } else if (r < a.R) {
#pragma unroll
      for (int hh = 0; hh < HG; ++hh)
        if (hh < nh) a.ctx[(size_t)t * a.ldc + (size_t)(h0 + hh) * a.R + r] = acc[hh] * inv[hh];
    }
  }
}

// dst[h][r][d] = src[h][d][r]: per-head transposed copy of the key up-projection (bf16), so that carrying a query into the
// latent space is a K-major product for the tensor-core GEMM
__global__ void transpose_heads_kernel(const bf16* __restrict__ src, bf16* __restrict__ dst, int Dk, int R) {
  const size_t h = blockIdx.z;
  const int r = blockIdx.x * 32 + threadIdx.x, d0 = blockIdx.y * 32;
  __shared__ bf16 tile[32][33];
  for (int i = threadIdx.y; i < 32; i += blockDim.y)
    if (d0 + i < Dk && r < R) tile[i][threadIdx.x] = src[(h * Dk + d0 + i) * R + r];
  __syncthreads();
  const int d = d0 + threadIdx.x;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int rr = blockIdx.x * 32 + i;
    if (rr < R && d < Dk) dst[(h * R + rr) * Dk + d] = tile[threadIdx.x][i];
  }
}

// block per key row jj
__global__ void __launch_bounds__(128) latent_gather_kernel(const bf16* __restrict__ cache, const int32_t* __restrict__ pt, int page_size,
                                                            int k0, int nk, int R, int Dr, bf16* __restrict__ kbuf,
                                                            bf16* __restrict__ ct, int ldk) {
  const int jj = blockIdx.x, D = R + Dr;
  if (jj >= nk) {  // padding columns of ct must be exact zeros: they meet the zero tail of P in the second product
    for (int r = threadIdx.x; r < R; r += blockDim.x) ct[(size_t)r * ldk + jj] = __float2bfloat16(0.f);
    return;
  }
  const int pos = k0 + jj;
  const bf16* row = cache + ((size_t)pt[pos / page_size] * page_size + pos % page_size) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const bf16 v = row[i];
    kbuf[(size_t)jj * D + i] = v;
    if (i < R) ct[(size_t)i * ldk + jj] = v;
  }
}

// one warp per row (token, head)
__global__ void __launch_bounds__(128) latent_softmax_kernel(const float* __restrict__ S, bf16* __restrict__ P, int ld, int rows, int H,
                                                             int q0, int k0, int nk, int window, float scale,
                                                             const bf16* __restrict__ sink) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int l = threadIdx.x & 31;
  const int pos = q0 + row / H, h = row % H;
  const int lo = max(pos - window + 1, k0) - k0, hi = min(pos, k0 + nk - 1) - k0;  // visible columns [lo, hi]
  const float* s = S + (size_t)row * ld;
  bf16* p = P + (size_t)row * ld;
  const float snk = __bfloat162float(sink[h]);
  float m = snk;
  for (int j = lo + l; j <= hi; j += 32) m = fmaxf(m, s[j] * scale);
  m = warp_max(m);
  float sum = 0.f;
  for (int j = lo + l; j <= hi; j += 32) sum += expf(s[j] * scale - m);
  sum = warp_sum(sum) + expf(snk - m);
  const float inv = 1.f / sum;
  for (int j = l; j < ld; j += 32) p[j] = __float2bfloat16((j >= lo && j <= hi) ? expf(s[j] * scale - m) * inv : 0.f);
}

}  // namespace

#define KERR() cudaGetLastError()

cudaError_t transpose_heads_bf16(cudaStream_t s, const bf16* src, bf16* dst, int H, int Dk, int R) {
  transpose_heads_kernel<<<dim3((R + 31) / 32, (Dk + 31) / 32, H), dim3(32, 8), 0, s>>>(src, dst, Dk, R);
  return KERR();
}
cudaError_t latent_gather(cudaStream_t s, const bf16* cache, const int32_t* pt, int page_size, int k0, int nk, int R, int Dr, bf16* kbuf,
                          bf16* ct, int ldk) {
  if (nk <= 0 || ldk < nk) return cudaErrorInvalidValue;
  latent_gather_kernel<<<ldk, 128, 0, s>>>(cache, pt, page_size, k0, nk, R, Dr, kbuf, ct, ldk);
  return KERR();
}
cudaError_t latent_softmax(cudaStream_t s, const float* S, bf16* P, int ld, int rows, int H, int q0, int k0, int nk, int window,
                           float scale, const bf16* sink) {
  if (rows <= 0) return cudaSuccess;
  latent_softmax_kernel<<<(rows + 3) / 4, 128, 0, s>>>(S, P, ld, rows, H, q0, k0, nk, window, scale, sink);
  return KERR();
}

// opt-in shared-memory sizes of every kernel here; called once per process before the first launch (never inside a capture)
cudaError_t stack_ops_init() {
  cudaError_t e;
  const int big = 200 * 1024;
#define HB_SMEM(k, n) if ((e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, n)) != cudaSuccess) return e
  HB_SMEM(postnorm_kernel<float>, big);
  HB_SMEM(postnorm_kernel<bf16>, big);
  HB_SMEM((latent_attn_kernel<float, float>), big);
  HB_SMEM((latent_attn_kernel<bf16, bf16>), big);
  HB_SMEM(gla_recurrence_kernel<16>, 80 * 1024);
  HB_SMEM(gla_recurrence_kernel<32>, 80 * 1024);
  HB_SMEM(gla_recurrence_kernel<64>, 80 * 1024);
  HB_SMEM(gla_recurrence_kernel<128>, 80 * 1024);
  HB_SMEM(gla_recurrence_kernel<256>, 160 * 1024);
#undef HB_SMEM
  return cudaSuccess;
}

cudaError_t gemm_rt(cudaStream_t s, const GemmRtArgs& a) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) return cudaErrorInvalidValue;
  dim3 grid((a.N + GT - 1) / GT, (a.M + GT - 1) / GT, a.batch);
  if (a.f32)
    gemm_rt_kernel<float><<<grid, 256, 0, s>>>(a.A, a.lda, a.a_bs, (const float*)a.W, a.w_sn, a.w_sk, a.w_bs, a.C, a.ldc, a.c_bs,
                                               (const float*)a.bias, a.M, a.N, a.K);
  else
    gemm_rt_kernel<bf16><<<grid, 256, 0, s>>>(a.A, a.lda, a.a_bs, (const bf16*)a.W, a.w_sn, a.w_sk, a.w_bs, a.C, a.ldc, a.c_bs,
                                              (const bf16*)a.bias, a.M, a.N, a.K);
  return KERR();
}

cudaError_t tanh_norm_step(cudaStream_t s, const float* x, const int32_t* row_index, const float* y, long ldy, const void* post,
                           const void* pre, bool f32, float* x_out, float* h, bf16* hb, int rows, int W) {
  if (rows <= 0) return cudaSuccess;
  if ((y && !x_out) || (!y && !pre)) return cudaErrorInvalidValue;
  const bool vec = W % 4 == 0 && ldy % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)x_out & 15) == 0 &&
                   ((uintptr_t)h & 15) == 0 && ((uintptr_t)hb & 7) == 0;
  dim3 grid(((vec ? W / 4 : W) + 255) / 256, rows);
  if (f32) {
    if (vec) tanh_norm_kernel<float, 4><<<grid, 256, 0, s>>>(x, row_index, y, ldy, (const float*)post, (const float*)pre, x_out, h, hb, W);
    else tanh_norm_kernel<float, 1><<<grid, 256, 0, s>>>(x, row_index, y, ldy, (const float*)post, (const float*)pre, x_out, h, hb, W);
  } else {
    if (vec) tanh_norm_kernel<bf16, 4><<<grid, 256, 0, s>>>(x, row_index, y, ldy, (const bf16*)post, (const bf16*)pre, x_out, h, hb, W);
    else tanh_norm_kernel<bf16, 1><<<grid, 256, 0, s>>>(x, row_index, y, ldy, (const bf16*)post, (const bf16*)pre, x_out, h, hb, W);
  }
  return cudaGetLastError();
}

cudaError_t embed_rows_f32(cudaStream_t s, const int32_t* tokens, const void* table, bool f32, float* x, bf16* xb, int T, int W, float scale) {
  if (T <= 0) return cudaSuccess;
  if (f32) embed_rows_kernel<float><<<T, 128, 0, s>>>(tokens, (const float*)table, x, xb, W, scale);
  else embed_rows_kernel<bf16><<<T, 128, 0, s>>>(tokens, (const bf16*)table, x, xb, W, scale);
  return KERR();
}

static cudaError_t postnorm_launch(cudaStream_t s, const float* x, const int32_t* idx, const float* y, long ldy, const void* bias,
                                   const void* w, bool f32, float alpha, float off, float eps, float* out, bf16* outb, int rows, int W,
                                   int add_x = 0) {
  if (rows <= 0) return cudaSuccess;
  if (W % 4 == 0 && W <= 4 * 256 * kPnChunks && (!y || ldy % 4 == 0) && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0 &&
      ((uintptr_t)out & 15) == 0 && ((uintptr_t)outb & 7) == 0) {
    if (f32)
      postnorm_vec_kernel<float><<<rows, 256, 0, s>>>(x, idx, y, ldy, (const float*)bias, (const float*)w, alpha, off, eps, out, outb, W, add_x);
    else
      postnorm_vec_kernel<bf16><<<rows, 256, 0, s>>>(x, idx, y, ldy, (const bf16*)bias, (const bf16*)w, alpha, off, eps, out, outb, W, add_x);
    return KERR();
  }
  const size_t smem = (size_t)(W + 32) * 4;
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  if (f32)
    postnorm_kernel<float><<<rows, 256, smem, s>>>(x, idx, y, ldy, (const float*)bias, (const float*)w, alpha, off, eps, out, outb, W, add_x);
  else
    postnorm_kernel<bf16><<<rows, 256, smem, s>>>(x, idx, y, ldy, (const bf16*)bias, (const bf16*)w, alpha, off, eps, out, outb, W, add_x);
  return KERR();
}
cudaError_t resid_postnorm(cudaStream_t s, float* x, bf16* xb, const float* y, long ldy, const void* bias, const void* w, bool f32,
                           float alpha, float off, float eps, int T, int W) {
  if (!y) return cudaErrorInvalidValue;
  return postnorm_launch(s, x, nullptr, y, ldy, bias, w, f32, alpha, off, eps, x, xb, T, W);
}
cudaError_t resid_add_normed(cudaStream_t s, float* x, bf16* xb, const float* y, long ldy, const void* bias, const void* w, bool f32,
                             float off, float eps, int T, int W) {
  if (!y) return cudaErrorInvalidValue;
  return postnorm_launch(s, x, nullptr, y, ldy, bias, w, f32, 1.f, off, eps, x, xb, T, W, 1);
}
cudaError_t norm_rows_f32(cudaStream_t s, const float* x, const int32_t* row_index, const void* w, bool f32, float off, float eps,
                          float* out, bf16* outb, int rows, int W) {
  return postnorm_launch(s, x, row_index, nullptr, 0, nullptr, w, f32, 1.f, off, eps, out, outb, rows, W);
}

cudaError_t softcap_rows(cudaStream_t s, float* logits, size_t n, float cap, float scale) {
  if (n == 0 || (!(cap > 0.f) && scale == 1.f)) return cudaSuccess;
  softcap_kernel<<<(unsigned)std::min<size_t>((n + 255) / 256, 148 * 16), 256, 0, s>>>(logits, n, cap, scale);
  return KERR();
}

cudaError_t clamped_glu(cudaStream_t s, const float* gu, long ldg, const void* bg, const void* bu, bool f32, float limit,
                        float act_alpha, float* out, bf16* outb, int T, int F) {
  if (T <= 0) return cudaSuccess;
  const bool vec = F % 4 == 0 && ldg % 4 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)outb & 7) == 0;
  dim3 grid(((vec ? F / 4 : F) + 255) / 256, T);
  if (f32 && vec) clamped_glu_kernel<float, 4><<<grid, 256, 0, s>>>(gu, ldg, (const float*)bg, (const float*)bu, limit, act_alpha, out, outb, F);
  else if (f32) clamped_glu_kernel<float, 1><<<grid, 256, 0, s>>>(gu, ldg, (const float*)bg, (const float*)bu, limit, act_alpha, out, outb, F);
  else if (vec) clamped_glu_kernel<bf16, 4><<<grid, 256, 0, s>>>(gu, ldg, (const bf16*)bg, (const bf16*)bu, limit, act_alpha, out, outb, F);
  else clamped_glu_kernel<bf16, 1><<<grid, 256, 0, s>>>(gu, ldg, (const bf16*)bg, (const bf16*)bu, limit, act_alpha, out, outb, F);
  return KERR();
}

cudaError_t sigmoid_gate(cudaStream_t s, const float* o, long ldo, const float* g, long ldg, float* out, bf16* outb, int T, int N) {
  if (T <= 0) return cudaSuccess;
  sigmoid_gate_kernel<<<dim3((N + 255) / 256, T), 256, 0, s>>>(o, ldo, g, ldg, out, outb, N);
  return KERR();
}
cudaError_t to_bf16_rows(cudaStream_t s, const float* src, long lds, bf16* dst, long ldd, int T, int N) {
  if (T <= 0) return cudaSuccess;
  if (N % 4 == 0 && lds % 4 == 0 && ldd % 4 == 0 && ((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 7) == 0)
    to_bf16_kernel<4><<<dim3((N / 4 + 255) / 256, T), 256, 0, s>>>(src, lds, dst, ldd, N);
  else
    to_bf16_kernel<1><<<dim3((N + 255) / 256, T), 256, 0, s>>>(src, lds, dst, ldd, N);
  return KERR();
}

cudaError_t gla_decay(cudaStream_t s, float* z, long ldz, const void* bias, bool f32, float tau, int T, int N) {
  if (T <= 0) return cudaSuccess;
  dim3 grid((N + 255) / 256, T);
  if (f32) gla_decay_kernel<float><<<grid, 256, 0, s>>>(z, ldz, (const float*)bias, 1.f / tau, N);
  else gla_decay_kernel<bf16><<<grid, 256, 0, s>>>(z, ldz, (const bf16*)bias, 1.f / tau, N);
  return KERR();
}

template <int DKP>
static cudaError_t gla_launch(cudaStream_t s, const GlaArgs& a) {
  constexpr int KS = DKP / 16;
  dim3 grid(a.B, a.H, (a.Dv + 31) / 32);
  const size_t smem = (size_t)(2 * kGlaTch * (3 * DKP + 32) + kGlaTch * KS * 32) * 4;  // 65 KB at DKP = 128, 131 KB at 256
  gla_recurrence_kernel<DKP><<<grid, 32 * KS, smem, s>>>(a);
  return KERR();
}
cudaError_t gla_recurrence(cudaStream_t s, const GlaArgs& a) {
  if (a.B <= 0) return cudaSuccess;
  if (a.Dk <= 16) return gla_launch<16>(s, a);
  if (a.Dk <= 32) return gla_launch<32>(s, a);
  if (a.Dk <= 64) return gla_launch<64>(s, a);
  if (a.Dk <= 128) return gla_launch<128>(s, a);
  if (a.Dk <= 256) return gla_launch<256>(s, a);
  return cudaErrorInvalidValue;  // more key channels per head than one block's warps cover
}

cudaError_t headnorm_silu_gate(cudaStream_t s, const float* o, long ldo, const float* g, long ldg, const void* w, bool f32, float eps,
                               float* out, bf16* outb, int T, int H, int Dv) {
  if (T <= 0) return cudaSuccess;
  const int items = T * H, grid = (items + 3) / 4;
  if (f32) headnorm_gate_kernel<float><<<grid, 128, 0, s>>>(o, ldo, g, ldg, (const float*)w, eps, out, outb, T, H, Dv);
  else headnorm_gate_kernel<bf16><<<grid, 128, 0, s>>>(o, ldo, g, ldg, (const bf16*)w, eps, out, outb, T, H, Dv);
  return KERR();
}

cudaError_t latent_prep(cudaStream_t s, const LatentPrepArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  if (a.rope_dims % 2 || a.rope_dims > a.Dr) return cudaErrorInvalidValue;
  if (a.f32) latent_prep_kernel<float, float><<<a.T, 128, 0, s>>>(a);
  else latent_prep_kernel<bf16, bf16><<<a.T, 128, 0, s>>>(a);
  return KERR();
}

cudaError_t latent_q_rope(cudaStream_t s, const float* q, long ldq, float* qabs, long ldqa, const int32_t* positions, int T, int H,
                          int Dk, int Dr, int R, int rope_dims, float base) {
  if (T <= 0) return cudaSuccess;
  latent_q_rope_kernel<<<T, 128, 0, s>>>(q, ldq, qabs, ldqa, positions, H, Dk, Dr, R, rope_dims, base);
  return KERR();
}

cudaError_t latent_attn(cudaStream_t s, const LatentAttnArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  const size_t smem = (size_t)(kLatHG * ((a.R + a.Dr + 3) / 4 * 4) + (kLatHG + 1) * a.window + 8 * kLatThreads + 32 * kLatHG) * 4;
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  dim3 grid(a.T, (a.H + kLatHG - 1) / kLatHG);
  if (a.f32) latent_attn_kernel<float, float><<<grid, kLatThreads, smem, s>>>(a);
  else latent_attn_kernel<bf16, bf16><<<grid, kLatThreads, smem, s>>>(a);
  return KERR();
}

}  // namespace hb
