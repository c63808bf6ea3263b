// State-space and matrix-memory layers of layer-list decoders (HB_MIXER_MAMBA2, HB_MIXER_MLSTM), the short causal
// convolutions in front of them (and in front of grouped-query attention with HB_ATTN_QKV_CONV), and the residual step of
// stacks whose two sublayers read the same stream (HB_NORM_PARALLEL).
//
// Both recurrences have one scalar decay per head and token,
//   S_t = a_t S_(t-1) + b_t k_t v_t^T,   o_t = S_t^T q_t            (S [dim][vdim] fp32 per head and sequence)
// and run on one kernel (lin_recurrence):
//   state-space layer:  a = exp(-exp(A) dt), b = dt, k = B, q = C, v = x, o += D x       (ssm_steps makes a, b)
//   matrix memory:      a = exp(f + m' - m), b = exp(i - m) with the running maximum m = max(f + m', i) of the log gates
//                       (exp_gate_scan: a warp scan over the tokens of an entry, since m -> max(m + f, i) composes
//                       associatively); the normaliser n_t = a n + b k is carried as one more state vector.
// Step entries are runs of tokens [first, first + n) of sequences whose state lives in their slot; an entry that starts at
// position 0 starts from zeros inside the kernels (m from 0), so a slot needs no clearing when it changes hands.
// Everything here is fp32; every sum has a fixed order per output element.
#include <math.h>
#include <stdlib.h>

#include <algorithm>

#include "kernels.h"
#include "launch.h"
#include "stack_common.cuh"

namespace hb {
namespace {

__device__ __forceinline__ float softplus_(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// ------------------------------------------------------------------ short convolutions
template <typename WT>
__global__ void __launch_bounds__(256) short_conv_kernel(ConvArgs a) {
  const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const int b = a.seq_of[t], t0 = a.cu[b], taps = a.taps;
  const bool fresh = a.first_pos[b] == 0;
  const float* tail = a.state + (size_t)a.slots[b] * a.slot_stride + a.tail_off;  // inputs of positions first - (taps - 1) ..
  const float ib = a.in_bias ? ldf<WT>((const WT*)a.in_bias, a.bias_off + c) : 0.f;
  const WT* w = (const WT*)a.w + (size_t)c * taps;
  float acc = 0.f;
  for (int j = 0; j < taps; ++j) {  // tap j multiplies the input of token t - (taps - 1 - j), oldest first
    const int tau = t - (taps - 1 - j);
    float x;
    if (tau >= t0) x = a.in[(size_t)tau * a.ldi + a.off + c] + ib;
    else x = fresh ? 0.f : tail[(size_t)(tau - t0 + taps - 1) * a.C + c];
    acc = fmaf(ldf<WT>(w, j), x, acc);
  }
  if (a.bias) acc += ldf<WT>((const WT*)a.bias, c);
  if (a.act == 1) acc = acc * sigmoidf_(acc);
  a.out[(size_t)t * a.ldo + c] = acc;
}

// The same for rows whose pieces start on 16-byte boundaries and up to four taps: thread = four neighbouring channels x kConvRun
// consecutive tokens, the last TAPS - 1 inputs in registers, so a row is read once per run instead of once per tap.  A run may
// cross entries: the window is refilled (from the slot or with zeros) wherever an entry starts.
constexpr int kConvRun = 8;
__device__ __forceinline__ float4 f4add(const float4& a, const float4& b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
template <typename WT, int TAPS>
__global__ void __launch_bounds__(128) short_conv_run_kernel(ConvArgs a) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= a.C) return;
  const int tb = blockIdx.y * kConvRun;
  float w[4][TAPS];
#pragma unroll
  for (int e = 0; e < 4; ++e)
#pragma unroll
    for (int j = 0; j < TAPS; ++j) w[e][j] = ldf<WT>((const WT*)a.w, (size_t)(c + e) * TAPS + j);
  float4 ib = make_float4(0.f, 0.f, 0.f, 0.f), cb = ib;
  if (a.in_bias) {
    const WT* p = (const WT*)a.in_bias + a.bias_off + c;
    ib = make_float4(ldf<WT>(p, 0), ldf<WT>(p, 1), ldf<WT>(p, 2), ldf<WT>(p, 3));
  }
  if (a.bias) {
    const WT* p = (const WT*)a.bias + c;
    cb = make_float4(ldf<WT>(p, 0), ldf<WT>(p, 1), ldf<WT>(p, 2), ldf<WT>(p, 3));
  }
  float4 win[TAPS > 1 ? TAPS - 1 : 1];
  int t0 = 0, t1 = -1;
  bool fresh = false;
  const float* tail = nullptr;
#pragma unroll
  for (int tt = 0; tt < kConvRun; ++tt) {
    const int t = tb + tt;
    if (t >= a.T) break;
    bool refill = tt == 0;
    if (t >= t1) {
      const int b = a.seq_of[t];
      t0 = a.cu[b]; t1 = a.cu[b + 1];
      fresh = a.first_pos[b] == 0;
      tail = a.state + (size_t)a.slots[b] * a.slot_stride + a.tail_off;
      refill = true;
    }
    if (refill) {
#pragma unroll
      for (int j = 0; j < TAPS - 1; ++j) {
        const int tau = t - (TAPS - 1 - j);
        if (tau >= t0) win[j] = f4add(*reinterpret_cast<const float4*>(a.in + (size_t)tau * a.ldi + a.off + c), ib);
        else if (!fresh) win[j] = *reinterpret_cast<const float4*>(tail + (size_t)(tau - t0 + TAPS - 1) * a.C + c);
        else win[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    const float4 x = f4add(*reinterpret_cast<const float4*>(a.in + (size_t)t * a.ldi + a.off + c), ib);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < TAPS - 1; ++j) {  // oldest tap first, as the per-channel kernel
      acc[0] = fmaf(w[0][j], win[j].x, acc[0]); acc[1] = fmaf(w[1][j], win[j].y, acc[1]);
      acc[2] = fmaf(w[2][j], win[j].z, acc[2]); acc[3] = fmaf(w[3][j], win[j].w, acc[3]);
    }
    acc[0] = fmaf(w[0][TAPS - 1], x.x, acc[0]); acc[1] = fmaf(w[1][TAPS - 1], x.y, acc[1]);
    acc[2] = fmaf(w[2][TAPS - 1], x.z, acc[2]); acc[3] = fmaf(w[3][TAPS - 1], x.w, acc[3]);
    if (a.bias) { acc[0] += cb.x; acc[1] += cb.y; acc[2] += cb.z; acc[3] += cb.w; }
    if (a.act == 1) {
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] = acc[e] * sigmoidf_(acc[e]);
    }
    *reinterpret_cast<float4*>(a.out + (size_t)t * a.ldo + c) = make_float4(acc[0], acc[1], acc[2], acc[3]);
#pragma unroll
    for (int j = 0; j + 1 < TAPS - 1; ++j) win[j] = win[j + 1];
    if (TAPS > 1) win[TAPS - 2] = x;
  }
}

// Thread = one channel of one entry: the slot's last taps - 1 inputs become those behind the entry's last token.
constexpr int kMaxConvTail = 15;
template <typename WT>
__global__ void __launch_bounds__(256) conv_tails_kernel(ConvArgs a) {
  const int b = blockIdx.y, nt = a.taps - 1;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.C || nt <= 0) return;
  const int t0 = a.cu[b], n = a.cu[b + 1] - t0;
  const bool fresh = a.first_pos[b] == 0;
  const float ib = a.in_bias ? ldf<WT>((const WT*)a.in_bias, a.bias_off + c) : 0.f;
  float* tail = a.state + (size_t)a.slots[b] * a.slot_stride + a.tail_off;
  float v[kMaxConvTail];
#pragma unroll
  for (int i = 0; i < kMaxConvTail; ++i) {
    if (i >= nt) break;
    const int e = n + i;  // index into [old tail (nt rows) ; the entry's rows (n)]
    v[i] = e < nt ? (fresh ? 0.f : tail[(size_t)e * a.C + c]) : a.in[(size_t)(t0 + e - nt) * a.ldi + a.off + c] + ib;
  }
#pragma unroll
  for (int i = 0; i < kMaxConvTail; ++i) {
    if (i >= nt) break;
    tail[(size_t)i * a.C + c] = v[i];
  }
}

// ------------------------------------------------------------------ decays and gates
template <typename WT>
__global__ void ssm_steps_kernel(const float* __restrict__ p, long ldp, int off_dt, const WT* __restrict__ a_dt, float* __restrict__ ab,
                                 long ldab, int T, int H) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)T * H) return;
  const int t = (int)(idx / H), h = (int)(idx % H);
  const float dt = softplus_(p[(size_t)t * ldp + off_dt + h] + ldf<WT>(a_dt, H + h));
  ab[(size_t)t * ldab + h] = expf(-expf(ldf<WT>(a_dt, h)) * dt);
  ab[(size_t)t * ldab + H + h] = dt;
}

// One warp per (entry, head).  The step m -> max(m + f, i) is the pair (f, i); two steps compose to
// (f1 + f2, max(i1 + f2, i2)), so the running maxima of 32 tokens come from one inclusive warp scan.
template <typename WT>
__global__ void __launch_bounds__(32) exp_gate_scan_kernel(GateScanArgs a) {
  const int b = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
  const int t0 = a.cu[b], t1 = a.cu[b + 1];
  float* ms = a.state + (size_t)a.slots[b] * a.slot_stride + a.m_off + h;
  float m = a.first_pos[b] == 0 ? 0.f : *ms;
  const float bi = a.bias ? ldf<WT>((const WT*)a.bias, a.off_i + h) : 0.f, bf = a.bias ? ldf<WT>((const WT*)a.bias, a.off_f + h) : 0.f;
  const float cap = a.cap, icap = 1.f / cap;
  for (int tc = t0; tc < t1; tc += 32) {
    const int t = tc + lane;
    const bool live = t < t1;
    float gi = -INFINITY, gf = 0.f;
    if (live) {
      const float* pr = a.p + (size_t)t * a.ldp;
      gi = cap * tanhf((pr[a.off_i + h] + bi) * icap);
      const float z = cap * tanhf((pr[a.off_f + h] + bf) * icap);
      gf = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));  // log sigmoid
    }
    float F = gf, I = gi;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float Fp = __shfl_up_sync(0xffffffffu, F, o), Ip = __shfl_up_sync(0xffffffffu, I, o);
      if (lane >= o) {
        I = fmaxf(Ip + F, I);
        F = Fp + F;
      }
    }
    const float mt = fmaxf(m + F, I);
    float mp = __shfl_up_sync(0xffffffffu, mt, 1);
    if (lane == 0) mp = m;
    if (live) {
      float* o = a.ab + (size_t)t * a.ldab;
      o[h] = expf(gf + mp - mt);
      o[a.H + h] = expf(gi - mt);
      o[2 * a.H + h] = expf(-mt);
    }
    m = __shfl_sync(0xffffffffu, mt, min(31, t1 - tc - 1));
  }
  if (lane == 0 && t1 > t0) *ms = m;
}

// ------------------------------------------------------------------ the recurrence
__device__ __forceinline__ void cpa4(float* smem_dst, const float* gsrc) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cpa16(float* smem_dst, const float* gsrc) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cpa_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cpa_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Block = (entry, head, 32 NC value columns), DKP / 16 warps: warp w keeps key channels [16 w, 16 w + 16) of the block's
// state columns in registers (lane = NC neighbouring columns; pairs of neighbouring channels as packed f32x2 operands, so one
// instruction serves two state elements, and one 16-byte broadcast read of q or k feeds 4 NC of them).  Tokens are staged
// 16 / NC at a time through a cp.async double buffer (q | k | the block's v columns | a, b); every warp leaves its partial dot
// products in shared memory and the block adds them in warp order once per stage.  The block of the first column slice also
// carries the normaliser vector: lane l of warp w keeps channel 16 w + (l & 15), the 16 lanes' products are added by a
// butterfly.
template <int DKP, int NC>
__global__ void __launch_bounds__(DKP * 2, 512 / DKP) lin_recurrence_kernel(LinRecArgs a) {
  // (64 registers per thread and four 256-thread blocks per SM: a step of 8 sequences x 64 heads x 64 columns is one wave)
  constexpr int kRecTch = 16 / NC;  // tokens per shared-memory stage
  constexpr int KS = DKP / 16, BC = 32 * NC;
  constexpr int per_tok = 2 * DKP + BC + 4, stage_floats = kRecTch * per_tok;
  extern __shared__ __align__(16) float sm[];  // 2 stages | partial outputs [kRecTch][KS][BC] | partial n . q [kRecTch][KS]
  float* obuf = sm + 2 * stage_floats;
  float* nbuf = obuf + kRecTch * KS * BC;
  const int b = blockIdx.x, h = blockIdx.y, kvh = h / (a.H / a.G);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c0 = blockIdx.z * BC, j0 = c0 + lane * NC;
  const int t0 = a.cu[b], t1 = a.cu[b + 1];
  const int Dk = a.Dk, i0 = w * 16;
  float* slot = a.state + (size_t)a.slots[b] * a.slot_stride;
  float* st = slot + a.s_off + (size_t)h * Dk * a.Dv;
  const bool fresh = a.first_pos[b] == 0;
  const bool do_n = a.nq != nullptr && blockIdx.z == 0;
  const int nch = i0 + (lane & 15);
  float* nst = slot + a.n_off + (size_t)h * Dk + nch;
  float2 S[NC][8];
#pragma unroll
  for (int e = 0; e < NC; ++e)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      auto ld = [&](int ch) { return (!fresh && j0 + e < a.Dv && ch < Dk) ? st[(size_t)ch * a.Dv + j0 + e] : 0.f; };
      S[e][i] = make_float2(ld(i0 + 2 * i), ld(i0 + 2 * i + 1));
    }
  float nreg = (do_n && !fresh && nch < Dk) ? *nst : 0.f;
  for (int e = threadIdx.x; e < 2 * stage_floats; e += blockDim.x) sm[e] = 0.f;  // padded key channels and columns read zeros
  __syncthreads();
  const bool vec = ((Dk | a.Dv | (int)a.ldq | (int)a.ldk | (int)a.ldv | a.q_off | a.k_off | a.v_off) & 3) == 0 && ((uintptr_t)a.q & 15) == 0 &&
                   ((uintptr_t)a.k & 15) == 0 && ((uintptr_t)a.v & 15) == 0;
  auto issue = [&](int tc, int stage) {  // warp w stages the tokens w, w + KS, ...
    const int nt = min(kRecTch, t1 - tc);
    float* base = sm + stage * stage_floats;
    for (int tt = w; tt < nt; tt += KS) {
      const size_t row = (size_t)(tc + tt);
      const float* sq = a.q + row * a.ldq + a.q_off + (size_t)kvh * Dk;
      const float* sk = a.k + row * a.ldk + a.k_off + (size_t)kvh * Dk;
      const float* sv = a.v + row * a.ldv + a.v_off + (size_t)h * a.Dv + c0;
      float* dst = base + tt * per_tok;
      if (vec) {
        for (int i = lane * 4; i < Dk; i += 128) {
          cpa16(dst + i, sq + i);
          cpa16(dst + DKP + i, sk + i);
        }
        if (lane < 8 * NC && c0 + lane * 4 < a.Dv) cpa16(dst + 2 * DKP + lane * 4, sv + lane * 4);
      } else {
        for (int i = lane; i < Dk; i += 32) {
          cpa4(dst + i, sq + i);
          cpa4(dst + DKP + i, sk + i);
        }
#pragma unroll
        for (int e = 0; e < NC; ++e)
          if (c0 + lane + 32 * e < a.Dv) cpa4(dst + 2 * DKP + lane + 32 * e, sv + lane + 32 * e);
      }
      if (lane == 8 * NC) cpa4(dst + 2 * DKP + BC, a.ab + row * a.ldab + h);
      if (lane == 8 * NC + 1) cpa4(dst + 2 * DKP + BC + 1, a.ab + row * a.ldab + a.H + h);
    }
    cpa_commit();
  };
  const float skip = a.skip ? (a.f32 ? ((const float*)a.skip)[h] : __bfloat162float(((const bf16*)a.skip)[h])) : 0.f;
  if (t0 < t1) issue(t0, 0);
  int stage = 0;
  for (int tc = t0; tc < t1; tc += kRecTch, stage ^= 1) {
    const int nt = min(kRecTch, t1 - tc);
    if (tc + kRecTch < t1) {
      issue(tc + kRecTch, stage ^ 1);  // the next tokens travel while these are consumed
      cpa_wait<1>();
    } else {
      cpa_wait<0>();
    }
    __syncthreads();
    const float* base = sm + stage * stage_floats;
    for (int tt = 0; tt < nt; ++tt) {
      const float* tk = base + tt * per_tok;
      const float2 dab = *reinterpret_cast<const float2*>(tk + 2 * DKP + BC);
      const float da = dab.x, db = dab.y;
      const float2 da2 = make_float2(da, da);
      float2 bv2[NC], oa[NC];
#pragma unroll
      for (int e = 0; e < NC; ++e) {
        const float bv = db * tk[2 * DKP + lane * NC + e];
        bv2[e] = make_float2(bv, bv);
        oa[e] = make_float2(0.f, 0.f);
      }
      const float4* q4 = reinterpret_cast<const float4*>(tk + i0);
      const float4* k4 = reinterpret_cast<const float4*>(tk + DKP + i0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 q = q4[i], k = k4[i];
        const float2 k01 = make_float2(k.x, k.y), k23 = make_float2(k.z, k.w), q01 = make_float2(q.x, q.y), q23 = make_float2(q.z, q.w);
#pragma unroll
        for (int e = 0; e < NC; ++e) {
          S[e][2 * i] = __ffma2_rn(da2, S[e][2 * i], __fmul2_rn(k01, bv2[e]));
          oa[e] = __ffma2_rn(S[e][2 * i], q01, oa[e]);
          S[e][2 * i + 1] = __ffma2_rn(da2, S[e][2 * i + 1], __fmul2_rn(k23, bv2[e]));
          oa[e] = __ffma2_rn(S[e][2 * i + 1], q23, oa[e]);
        }
      }
#pragma unroll
      for (int e = 0; e < NC; ++e) obuf[(tt * KS + w) * BC + lane * NC + e] = oa[e].x + oa[e].y;
      if (do_n) {
        nreg = fmaf(da, nreg, db * tk[DKP + nch]);
        float pn = nreg * tk[nch];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) pn += __shfl_xor_sync(0xffffffffu, pn, o);
        if (lane == 0) nbuf[tt * KS + w] = pn;
      }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < nt * BC; e += blockDim.x) {
      const int tt = e / BC, c = e % BC;
      float o = 0.f;
#pragma unroll
      for (int ww = 0; ww < KS; ++ww) o += obuf[(tt * KS + ww) * BC + c];
      if (c0 + c < a.Dv) a.out[(size_t)(tc + tt) * a.ldo + (size_t)h * a.Dv + c0 + c] = fmaf(skip, base[tt * per_tok + 2 * DKP + c], o * a.q_scale);
    }
    if (do_n) {
      for (int tt = threadIdx.x; tt < nt; tt += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int ww = 0; ww < KS; ++ww) o += nbuf[tt * KS + ww];
        a.nq[(size_t)(tc + tt) * a.ldn + h] = o * a.q_scale;
      }
    }
    __syncthreads();  // the stage and the partial outputs are rewritten in the next iteration
  }
  if (t1 <= t0) return;
#pragma unroll
  for (int e = 0; e < NC; ++e) {
    if (j0 + e >= a.Dv) continue;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (i0 + 2 * i < Dk) st[(size_t)(i0 + 2 * i) * a.Dv + j0 + e] = S[e][i].x;
      if (i0 + 2 * i + 1 < Dk) st[(size_t)(i0 + 2 * i + 1) * a.Dv + j0 + e] = S[e][i].y;
    }
  }
  if (do_n && lane < 16 && nch < Dk) *nst = nreg;
}

template <int DKP, int NC>
cudaError_t launch_rec(cudaStream_t s, const LinRecArgs& a) {
  constexpr int KS = DKP / 16, BC = 32 * NC, kRecTch = 16 / NC;
  const size_t smem = (size_t)(2 * kRecTch * (2 * DKP + BC + 4) + kRecTch * KS * BC + kRecTch * KS) * 4;
  dim3 grid(a.B, a.H, (a.Dv + BC - 1) / BC);
  lin_recurrence_kernel<DKP, NC><<<grid, DKP * 2, smem, s>>>(a);
  return cudaGetLastError();
}

// ------------------------------------------------------------------ read-outs
// one warp per (token, head)
template <typename WT>
__global__ void memory_readout_kernel(const float* __restrict__ num, long ldnum, const float* __restrict__ nq, long ldn,
                                      const float* __restrict__ ab, long ldab, const float* __restrict__ g, long ldg, const WT* __restrict__ w,
                                      float eps, float scale, float* __restrict__ out, bf16* __restrict__ outb, long ldout, int col0, int T,
                                      int H, int Dv) {
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= T * H) return;
  const int t = item / H, h = item % H, l = threadIdx.x & 31;
  const float den = fmaxf(fabsf(nq[(size_t)t * ldn + h]), ab[(size_t)t * ldab + 2 * H + h]) + 1e-6f;
  const float* src = num + (size_t)t * ldnum + (size_t)h * Dv;
  const float* gs = g + (size_t)t * ldg + (size_t)h * Dv;
  float ss = 0.f;
  for (int i = l; i < Dv; i += 32) {
    const float o = src[i] / den;
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  const float rs = 1.f / sqrtf(ss / (float)Dv + eps);
  for (int i = l; i < Dv; i += 32) {
    const float v = src[i] / den * rs * ldf<WT>(w, (size_t)h * Dv + i) * sigmoidf_(gs[i]) * scale;
    const size_t d = (size_t)t * ldout + col0 + (size_t)h * Dv + i;
    if (out) out[d] = v;
    if (outb) outb[d] = __float2bfloat16(v);
  }
}

// one block per (part, token)
template <typename WT>
__global__ void __launch_bounds__(256) gated_group_norm_kernel(const float* __restrict__ y, long ldy, const float* __restrict__ z, long ldz,
                                                               const WT* __restrict__ w, float eps, int parts, float* __restrict__ out,
                                                               bf16* __restrict__ outb, int n) {
  __shared__ float red[32];
  const int t = blockIdx.y, part = blockIdx.x, len = n / parts, c0 = part * len;
  const float* ys = y + (size_t)t * ldy + c0;
  const float* zs = z + (size_t)t * ldz + c0;
  constexpr int kKeep = 8;  // gated values a thread keeps between the two passes (parts of up to 2048 entries are read once)
  float keep[kKeep];
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < kKeep; ++r) {
    const int i = threadIdx.x + r * 256;
    keep[r] = 0.f;
    if (i < len) {
      const float zv = zs[i];
      keep[r] = ys[i] * (zv * sigmoidf_(zv));
    }
    ss = fmaf(keep[r], keep[r], ss);
  }
  for (int i = threadIdx.x + kKeep * 256; i < len; i += blockDim.x) {
    const float zv = zs[i], u = ys[i] * (zv * sigmoidf_(zv));
    ss = fmaf(u, u, ss);
  }
  ss = block_sum(ss, red);
  const float rs = 1.f / sqrtf(ss / (float)len + eps);
#pragma unroll
  for (int r = 0; r < kKeep; ++r) {
    const int i = threadIdx.x + r * 256;
    if (i >= len) break;
    const float v = keep[r] * rs * ldf<WT>(w, c0 + i);
    const size_t d = (size_t)t * n + c0 + i;
    if (out) out[d] = v;
    if (outb) outb[d] = __float2bfloat16(v);
  }
  for (int i = threadIdx.x + kKeep * 256; i < len; i += blockDim.x) {
    const float zv = zs[i], u = ys[i] * (zv * sigmoidf_(zv));
    const float v = u * rs * ldf<WT>(w, c0 + i);
    const size_t d = (size_t)t * n + c0 + i;
    if (out) out[d] = v;
    if (outb) outb[d] = __float2bfloat16(v);
  }
}

__global__ void gate_scale_kernel(const float* __restrict__ in, const bf16* __restrict__ inb, long ldi, const float* __restrict__ g, long ldg,
                                  float scale, float* __restrict__ out, bf16* __restrict__ outb, long ldout, int col0, int n) {
  const int t = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const float x = in ? in[(size_t)t * ldi + e] : __bfloat162float(inb[(size_t)t * ldi + e]);
  const float v = x * sigmoidf_(g[(size_t)t * ldg + e]) * scale;
  const size_t d = (size_t)t * ldout + col0 + e;
  if (out) out[d] = v;
  if (outb) outb[d] = __float2bfloat16(v);
}

// ------------------------------------------------------------------ residual step of parallel sublayers
// one block per row; dynamic smem: the summed row [W]
template <typename WT>
__global__ void __launch_bounds__(256) parallel_step_kernel(const float* x, const int32_t* __restrict__ row_index,
                                                            const float* __restrict__ y, const float* __restrict__ y2,
                                                            const WT* __restrict__ bias, float bias_scale, const WT* __restrict__ w1,
                                                            const WT* __restrict__ w2, float eps, float* x_out,
                                                            float* __restrict__ h1, bf16* __restrict__ h1b, float* __restrict__ h2,
                                                            bf16* __restrict__ h2b, int W) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[32];
  const size_t r = blockIdx.x;
  const float* xs = x + (row_index ? (size_t)row_index[r] : r) * W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = xs[i];
    if (y) v += y2 ? y[r * W + i] + y2[r * W + i] : y[r * W + i];
    if (bias) v = fmaf(bias_scale, ldf<WT>(bias, i), v);
    row[i] = v;
    if (x_out) x_out[r * W + i] = v;
    ss = fmaf(v, v, ss);
  }
  if (!w1 && !w2) return;
  ss = block_sum(ss, red);
  const float rs = 1.f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float u = row[i] * rs;
    if (w1) {
      const float v = u * ldf<WT>(w1, i);
      if (h1) h1[r * W + i] = v;
      if (h1b) h1b[r * W + i] = __float2bfloat16(v);
    }
    if (w2) {
      const float v = u * ldf<WT>(w2, i);
      if (h2) h2[r * W + i] = v;
      if (h2b) h2b[r * W + i] = __float2bfloat16(v);
    }
  }
}

__global__ void relu2_kernel(const float* __restrict__ in, long ldi, float* __restrict__ out, bf16* __restrict__ outb, int n) {
  const int t = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const float r = fmaxf(in[(size_t)t * ldi + e], 0.f), v = r * r;
  if (out) out[(size_t)t * n + e] = v;
  if (outb) outb[(size_t)t * n + e] = __float2bfloat16(v);
}
__global__ void relu2_b16_kernel(const bf16* __restrict__ in, long ldi, bf16* __restrict__ out, int n) {
  const int t = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const float r = fmaxf(__bfloat162float(in[(size_t)t * ldi + e]), 0.f);
  out[(size_t)t * n + e] = __float2bfloat16(r * r);
}

}  // namespace

cudaError_t stack_ssm_init() {
  cudaError_t e;
#define HB_SMEM(k, n) if ((e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, n)) != cudaSuccess) return e
  HB_SMEM((lin_recurrence_kernel<16, 1>), 64 * 1024);
  HB_SMEM((lin_recurrence_kernel<32, 1>), 64 * 1024);
  HB_SMEM((lin_recurrence_kernel<64, 1>), 64 * 1024);
  HB_SMEM((lin_recurrence_kernel<128, 1>), 96 * 1024);
  HB_SMEM((lin_recurrence_kernel<256, 1>), 160 * 1024);
  HB_SMEM((lin_recurrence_kernel<16, 2>), 64 * 1024);
  HB_SMEM((lin_recurrence_kernel<32, 2>), 64 * 1024);
  HB_SMEM((lin_recurrence_kernel<64, 2>), 96 * 1024);
  HB_SMEM((lin_recurrence_kernel<128, 2>), 128 * 1024);
  HB_SMEM((lin_recurrence_kernel<256, 2>), 200 * 1024);
  HB_SMEM(parallel_step_kernel<float>, 200 * 1024);
  HB_SMEM(parallel_step_kernel<bf16>, 200 * 1024);
#undef HB_SMEM
  return cudaSuccess;
}

cudaError_t short_conv(cudaStream_t s, const ConvArgs& a) {
  if (a.T <= 0 || a.C <= 0) return cudaSuccess;
  if (a.taps < 1 || a.taps - 1 > kMaxConvTail) return cudaErrorInvalidValue;
  const bool vec = a.taps <= 4 && ((a.C | (int)a.ldi | a.off | (int)a.ldo | (int)a.slot_stride | (int)a.tail_off) & 3) == 0 &&
                   ((uintptr_t)a.in & 15) == 0 && ((uintptr_t)a.out & 15) == 0 && ((uintptr_t)a.state & 15) == 0;
  if (vec) {
    dim3 g((a.C / 4 + 127) / 128, (a.T + kConvRun - 1) / kConvRun);
#define HB_CONV(WT, TP) short_conv_run_kernel<WT, TP><<<g, 128, 0, s>>>(a)
    if (a.f32) { if (a.taps == 1) HB_CONV(float, 1); else if (a.taps == 2) HB_CONV(float, 2); else if (a.taps == 3) HB_CONV(float, 3); else HB_CONV(float, 4); }
    else { if (a.taps == 1) HB_CONV(bf16, 1); else if (a.taps == 2) HB_CONV(bf16, 2); else if (a.taps == 3) HB_CONV(bf16, 3); else HB_CONV(bf16, 4); }
#undef HB_CONV
    return cudaGetLastError();
  }
  dim3 grid((a.C + 255) / 256, a.T);
  if (a.f32) short_conv_kernel<float><<<grid, 256, 0, s>>>(a);
  else short_conv_kernel<bf16><<<grid, 256, 0, s>>>(a);
  return cudaGetLastError();
}

cudaError_t conv_tails(cudaStream_t s, const ConvArgs& a) {
  if (a.B <= 0 || a.taps <= 1 || a.C <= 0) return cudaSuccess;
  dim3 grid((a.C + 255) / 256, a.B);
  if (a.f32) conv_tails_kernel<float><<<grid, 256, 0, s>>>(a);
  else conv_tails_kernel<bf16><<<grid, 256, 0, s>>>(a);
  return cudaGetLastError();
}

cudaError_t ssm_steps(cudaStream_t s, const float* p, long ldp, int off_dt, const void* a_dt, bool f32, float* ab, long ldab, int T, int H) {
  if (T <= 0 || H <= 0) return cudaSuccess;
  const unsigned blocks = (unsigned)(((long)T * H + 255) / 256);
  if (f32) ssm_steps_kernel<float><<<blocks, 256, 0, s>>>(p, ldp, off_dt, (const float*)a_dt, ab, ldab, T, H);
  else ssm_steps_kernel<bf16><<<blocks, 256, 0, s>>>(p, ldp, off_dt, (const bf16*)a_dt, ab, ldab, T, H);
  return cudaGetLastError();
}

cudaError_t exp_gate_scan(cudaStream_t s, const GateScanArgs& a) {
  if (a.B <= 0 || a.H <= 0) return cudaSuccess;
  if (!(a.cap > 0.f)) return cudaErrorInvalidValue;
  if (a.f32) exp_gate_scan_kernel<float><<<dim3(a.B, a.H), 32, 0, s>>>(a);
  else exp_gate_scan_kernel<bf16><<<dim3(a.B, a.H), 32, 0, s>>>(a);
  return cudaGetLastError();
}

cudaError_t lin_recurrence(cudaStream_t s, const LinRecArgs& a) {
  if (a.B <= 0) return cudaSuccess;
  if (a.G <= 0 || a.H % a.G || a.Dk > 256 || a.Dk <= 0) return cudaErrorInvalidValue;
  // two columns per lane (blocks of 64 columns) halve the shared-memory reads per product; heads of up to 32 value columns
  // keep one.  HB_REC_COLS=1 forces the narrow blocks (A/B measurements)
  // (the arithmetic per column is the same either way, so the choice never shows in a result; narrow blocks for small grids
  // measured no faster)
  static const bool narrow = [] { const char* e = getenv("HB_REC_COLS"); return e && atoi(e) == 1; }();
  if (a.Dv > 32 && !narrow) {
    if (a.Dk <= 16) return launch_rec<16, 2>(s, a);
    if (a.Dk <= 32) return launch_rec<32, 2>(s, a);
    if (a.Dk <= 64) return launch_rec<64, 2>(s, a);
    if (a.Dk <= 128) return launch_rec<128, 2>(s, a);
    return launch_rec<256, 2>(s, a);
  }
  if (a.Dk <= 16) return launch_rec<16, 1>(s, a);
  if (a.Dk <= 32) return launch_rec<32, 1>(s, a);
  if (a.Dk <= 64) return launch_rec<64, 1>(s, a);
  if (a.Dk <= 128) return launch_rec<128, 1>(s, a);
  return launch_rec<256, 1>(s, a);
}

cudaError_t memory_readout(cudaStream_t s, const float* num, long ldnum, const float* nq, long ldn, const float* ab, long ldab,
                           const float* g, long ldg, const void* w, bool f32, float eps, float scale, float* out, bf16* outb, long ldout,
                           int col0, int T, int H, int Dv) {
  if (T <= 0) return cudaSuccess;
  const unsigned blocks = (unsigned)(((long)T * H + 7) / 8);
  if (f32) memory_readout_kernel<float><<<blocks, 256, 0, s>>>(num, ldnum, nq, ldn, ab, ldab, g, ldg, (const float*)w, eps, scale, out, outb, ldout, col0, T, H, Dv);
  else memory_readout_kernel<bf16><<<blocks, 256, 0, s>>>(num, ldnum, nq, ldn, ab, ldab, g, ldg, (const bf16*)w, eps, scale, out, outb, ldout, col0, T, H, Dv);
  return cudaGetLastError();
}

cudaError_t gated_group_norm(cudaStream_t s, const float* y, long ldy, const float* z, long ldz, const void* w, bool f32, float eps, int parts,
                             float* out, bf16* outb, int T, int n) {
  if (T <= 0) return cudaSuccess;
  if (parts < 1 || n % parts) return cudaErrorInvalidValue;
  dim3 grid(parts, T);
  if (f32) gated_group_norm_kernel<float><<<grid, 256, 0, s>>>(y, ldy, z, ldz, (const float*)w, eps, parts, out, outb, n);
  else gated_group_norm_kernel<bf16><<<grid, 256, 0, s>>>(y, ldy, z, ldz, (const bf16*)w, eps, parts, out, outb, n);
  return cudaGetLastError();
}

cudaError_t gate_scale_rows(cudaStream_t s, const float* in, const bf16* inb, long ldi, const float* g, long ldg, float scale, float* out,
                            bf16* outb, long ldout, int col0, int T, int n) {
  if (T <= 0 || n <= 0) return cudaSuccess;
  if ((in == nullptr) == (inb == nullptr)) return cudaErrorInvalidValue;
  gate_scale_kernel<<<dim3((n + 255) / 256, T), 256, 0, s>>>(in, inb, ldi, g, ldg, scale, out, outb, ldout, col0, n);
  return cudaGetLastError();
}

cudaError_t parallel_step(cudaStream_t s, const float* x, const int32_t* row_index, const float* y, const float* y2, const void* bias,
                          float bias_scale, const void* w1, const void* w2, bool f32, float eps, float* x_out, float* h1, bf16* h1b, float* h2,
                          bf16* h2b, int rows, int W) {
  if (rows <= 0) return cudaSuccess;
  if ((y2 && !y) || (size_t)W * 4 > 200 * 1024) return cudaErrorInvalidValue;
  const size_t smem = (size_t)W * 4;
  if (f32)
    parallel_step_kernel<float><<<rows, 256, smem, s>>>(x, row_index, y, y2, (const float*)bias, bias_scale, (const float*)w1, (const float*)w2,
                                                        eps, x_out, h1, h1b, h2, h2b, W);
  else
    parallel_step_kernel<bf16><<<rows, 256, smem, s>>>(x, row_index, y, y2, (const bf16*)bias, bias_scale, (const bf16*)w1, (const bf16*)w2, eps,
                                                       x_out, h1, h1b, h2, h2b, W);
  return cudaGetLastError();
}

cudaError_t relu2_rows(cudaStream_t s, const float* in, long ldi, float* out, bf16* outb, int T, int n) {
  if (T <= 0 || n <= 0) return cudaSuccess;
  relu2_kernel<<<dim3((n + 255) / 256, T), 256, 0, s>>>(in, ldi, out, outb, n);
  return cudaGetLastError();
}
cudaError_t relu2_rows_b16(cudaStream_t s, const bf16* in, long ldi, bf16* out, int T, int n) {
  if (T <= 0 || n <= 0) return cudaSuccess;
  relu2_b16_kernel<<<dim3((n + 255) / 256, T), 256, 0, s>>>(in, ldi, out, n);
  return cudaGetLastError();
}

}  // namespace hb
