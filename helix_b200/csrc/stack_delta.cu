// Gated delta rule layers of layer-list decoders (HB_MIXER_DELTA): short causal convolutions over the q / k / v projections,
// silu, unit-length q and k, the per-head write strength and decay, and the recurrence itself
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (S [dim][vdim] fp32 per head and sequence)
// over the entries of a step: an entry is a run of tokens [first, first + n) of a sequence whose state (S and the last
// taps - 1 inputs of the convolutions) lives in its state slot; an entry that starts at position 0 starts from zeros inside
// the kernels, so a slot is never cleared when it changes hands.  Everything here is fp32.  Every sum has a fixed order per
// output element: a token's result does not depend on what else the step carries or on how the sequence was cut.
#include <math.h>

#include <algorithm>

#include "kernels.h"
#include "launch.h"
#include "stack_common.cuh"

namespace hb {
namespace {

__device__ __forceinline__ float softplusf_(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// One block per token.  dynamic smem: the token's convolved, activated q | k | v row [C]
template <typename WT>
__global__ void __launch_bounds__(256) delta_prep_kernel(DeltaPrepArgs a) {
  extern __shared__ __align__(16) float row[];
  const int t = blockIdx.x;
  const int b = a.seq_of[t], t0 = a.cu[b];
  const int GD = a.G * a.D, C = 2 * GD + a.H * a.Dv, taps = a.taps;
  const bool fresh = a.first_pos[b] == 0;
  const float* tail = a.state + (size_t)a.slots[b] * a.slot_stride + a.tail_off;  // [taps - 1][C]: inputs of positions first - (taps - 1) ..
  const WT* cw = (const WT*)a.conv_w;
  if (((C | (int)a.ldp | a.off_qkv) & 3) == 0 && ((uintptr_t)a.p & 15) == 0 && ((uintptr_t)a.state & 15) == 0 &&
      ((a.slot_stride | (long)a.tail_off) & 3) == 0) {
    // four neighbouring channels per thread: 16-byte loads of the projection rows and of the slot's tail
    for (int c = threadIdx.x * 4; c < C; c += blockDim.x * 4) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < taps; ++j) {
        const int tau = t - (taps - 1 - j);
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tau >= t0) x = *reinterpret_cast<const float4*>(a.p + (size_t)tau * a.ldp + a.off_qkv + c);
        else if (!fresh) x = *reinterpret_cast<const float4*>(tail + (size_t)(tau - t0 + taps - 1) * C + c);
        acc[0] = fmaf(ldf<WT>(cw, (size_t)c * taps + j), x.x, acc[0]);
        acc[1] = fmaf(ldf<WT>(cw, (size_t)(c + 1) * taps + j), x.y, acc[1]);
        acc[2] = fmaf(ldf<WT>(cw, (size_t)(c + 2) * taps + j), x.z, acc[2]);
        acc[3] = fmaf(ldf<WT>(cw, (size_t)(c + 3) * taps + j), x.w, acc[3]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) row[c + e] = acc[e] * sigmoidf_(acc[e]);
    }
  } else {
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {  // tap j multiplies the input of token t - (taps - 1 - j), oldest first
      const int tau = t - (taps - 1 - j);
      float x;
      if (tau >= t0) x = a.p[(size_t)tau * a.ldp + a.off_qkv + c];
      else x = fresh ? 0.f : tail[(size_t)(tau - t0 + taps - 1) * C + c];
      acc = fmaf(ldf<WT>(cw, (size_t)c * taps + j), x, acc);
    }
    row[c] = acc * sigmoidf_(acc);
  }
  }
  __syncthreads();
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  float* out = a.out + (size_t)t * a.ldo;
  const float qs = 1.f / sqrtf((float)a.D);
  for (int g = w; g < a.G; g += nw) {  // q and k of one head pair: unit vectors, and their dot product
    const float* q = row + (size_t)g * a.D;
    const float* k = row + GD + (size_t)g * a.D;
    float sq = 0.f, sk = 0.f, qk = 0.f;
    for (int i = l; i < a.D; i += 32) {
      sq = fmaf(q[i], q[i], sq);
      sk = fmaf(k[i], k[i], sk);
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float rq = qs / sqrtf(sq + 1e-6f), rk = 1.f / sqrtf(sk + 1e-6f);
    for (int i = l; i < a.D; i += 32) {
      const float qv = q[i] * rq, kv = k[i] * rk;
      out[(size_t)g * a.D + i] = qv;
      out[GD + (size_t)g * a.D + i] = kv;
      qk = fmaf(qv, kv, qk);
    }
    qk = warp_sum(qk);
    if (l == 0) out[C + 2 * a.H + g] = qk;
  }
  if (((GD | (a.H * a.Dv) | (int)a.ldo) & 3) == 0 && ((uintptr_t)a.out & 15) == 0) {
    for (int i = threadIdx.x * 4; i < a.H * a.Dv; i += blockDim.x * 4)
      *reinterpret_cast<float4*>(out + 2 * GD + i) = *reinterpret_cast<const float4*>(row + 2 * GD + i);
  } else {
    for (int i = threadIdx.x; i < a.H * a.Dv; i += blockDim.x) out[2 * GD + i] = row[2 * GD + i];
  }
  const WT* adt = (const WT*)a.a_dt;
  for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
    const float* pr = a.p + (size_t)t * a.ldp;
    out[C + h] = sigmoidf_(pr[a.off_b + h]);
    out[C + a.H + h] = expf(-expf(ldf<WT>(adt, h)) * softplusf_(pr[a.off_a + h] + ldf<WT>(adt, a.H + h)));
  }
}

// After delta_prep: the slots' convolution inputs move on by the entries' tokens.  Thread = one channel of one entry.
constexpr int kMaxTail = 15;
__global__ void __launch_bounds__(256) delta_tails_kernel(DeltaPrepArgs a) {
  const int b = blockIdx.y;
  const int C = 2 * a.G * a.D + a.H * a.Dv, nt = a.taps - 1;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C || nt <= 0) return;
  const int t0 = a.cu[b], n = a.cu[b + 1] - t0;
  const bool fresh = a.first_pos[b] == 0;
  float* tail = a.state + (size_t)a.slots[b] * a.slot_stride + a.tail_off;
  float v[kMaxTail];
#pragma unroll
  for (int i = 0; i < kMaxTail; ++i) {
    if (i >= nt) break;
    const int e = n + i;  // index into [old tail (nt rows) ; the entry's rows (n)]
    v[i] = e < nt ? (fresh ? 0.f : tail[(size_t)e * C + c]) : a.p[(size_t)(t0 + e - nt) * a.ldp + a.off_qkv + c];
  }
#pragma unroll
  for (int i = 0; i < kMaxTail; ++i) {
    if (i >= nt) break;
    tail[(size_t)i * C + c] = v[i];
  }
}

constexpr int kDelTch = 16;  // tokens per shared-memory stage
__device__ __forceinline__ void cp_async4(float* smem_dst, const float* gsrc) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gsrc) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Block = (entry, head, 32 value columns), 128 threads: a group of 8 lanes owns TWO state columns (c and c + 16 of the slice),
// lane `sub` of the group keeps the key channels 4 (sub + 8 i) .. + 3, i < CPL / 4, of both in registers as packed pairs of
// neighbouring channels, so one 16-byte read of q or k from shared memory feeds four f32x2 products and the 8 lanes of a
// group read 128 contiguous bytes.  Per token both products with the OLD state, S^T k and S^T q, are formed in one pass and
// added over the 8 lanes by a butterfly; the write u and the output o = g S^T q + (k . q) u follow from them, then the state
// is updated in place (g S + k u: one multiply and one fused multiply-add per pair).  Tokens are staged kDelTch at a time
// through a cp.async double buffer.
constexpr int kDelThreads = 128;
template <int CPL>
__global__ void __launch_bounds__(kDelThreads) delta_recurrence_kernel(DeltaArgs a) {
  constexpr int DP = 8 * CPL;                     // padded key channels
  constexpr int per_tok = 2 * DP + 32 + 4;        // q | k | v (this block's columns) | beta, decay, k.q, pad
  constexpr int stage_floats = kDelTch * per_tok;
  extern __shared__ __align__(16) float sm[];     // 2 stages + outputs [kDelTch][32]
  float* obuf = sm + 2 * stage_floats;
  const int b = blockIdx.x, h = blockIdx.y, kvh = h / (a.H / a.G);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, sub = lane & 7;
  const int col = w * 4 + (lane >> 3);            // first column of this group inside the slice; the second is col + 16
  const int j0 = blockIdx.z * 32 + col, j1 = j0 + 16;
  const bool live0 = j0 < a.Dv, live1 = j1 < a.Dv;
  const int t0 = a.cu[b], t1 = a.cu[b + 1];
  const int D = a.D;
  float* st = a.state + (size_t)a.slots[b] * a.slot_stride + (size_t)h * D * a.Dv;
  const bool fresh = a.first_pos[b] == 0;
  float2 Sa[CPL / 2], Sb[CPL / 2];
#pragma unroll
  for (int i = 0; i < CPL / 4; ++i)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int ch = 4 * (sub + 8 * i) + 2 * e;
      auto ld = [&](int c, int j, bool live) { return (!fresh && live && c < D) ? st[(size_t)c * a.Dv + j] : 0.f; };
      Sa[2 * i + e] = make_float2(ld(ch, j0, live0), ld(ch + 1, j0, live0));
      Sb[2 * i + e] = make_float2(ld(ch, j1, live1), ld(ch + 1, j1, live1));
    }
  for (int e = threadIdx.x; e < 2 * stage_floats; e += blockDim.x) sm[e] = 0.f;  // padded channels read zeros
  __syncthreads();
  // 16-byte copies when every row piece starts on a 16-byte boundary
  const bool vec = ((D | a.Dv | (int)a.ld | a.off_q | a.off_k | a.off_v) & 3) == 0 && ((uintptr_t)a.in & 15) == 0;
  const int nw = blockDim.x >> 5;
  auto issue = [&](int tc, int stage) {  // warp w stages the tokens w, w + nw, ...: no index arithmetic beyond adds
    const int nt = min(kDelTch, t1 - tc);
    float* base = sm + stage * stage_floats;
    for (int tt = w; tt < nt; tt += nw) {
      const float* src = a.in + (size_t)(tc + tt) * a.ld;
      const float* sq = src + a.off_q + kvh * D;
      const float* sk = src + a.off_k + kvh * D;
      const float* sv = src + a.off_v + (size_t)h * a.Dv + blockIdx.z * 32;
      float* dst = base + tt * per_tok;
      if (vec) {
        for (int i = lane * 4; i < D; i += 128) {
          cp_async16(dst + i, sq + i);
          cp_async16(dst + DP + i, sk + i);
        }
        if (lane < 8 && blockIdx.z * 32 + lane * 4 < a.Dv) cp_async16(dst + 2 * DP + lane * 4, sv + lane * 4);
      } else {
        for (int i = lane; i < D; i += 32) {
          cp_async4(dst + i, sq + i);
          cp_async4(dst + DP + i, sk + i);
        }
        if (blockIdx.z * 32 + lane < a.Dv) cp_async4(dst + 2 * DP + lane, sv + lane);
      }
      if (lane == 8) cp_async4(dst + 2 * DP + 32, src + a.off_beta + h);
      if (lane == 9) cp_async4(dst + 2 * DP + 33, src + a.off_decay + h);
      if (lane == 10) cp_async4(dst + 2 * DP + 34, src + a.off_kq + kvh);
    }
    cp_async_commit();
  };
  if (t0 < t1) issue(t0, 0);
  int stage = 0;
  for (int tc = t0; tc < t1; tc += kDelTch, stage ^= 1) {
    const int nt = min(kDelTch, t1 - tc);
    if (tc + kDelTch < t1) {
      issue(tc + kDelTch, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* base = sm + stage * stage_floats;
    for (int tt = 0; tt < nt; ++tt) {
      const float* tk = base + tt * per_tok;
      const float4* q4 = reinterpret_cast<const float4*>(tk);
      const float4* k4 = reinterpret_cast<const float4*>(tk + DP);
      const float va = tk[2 * DP + col], vb = tk[2 * DP + col + 16];
      const float beta = tk[2 * DP + 32], g = tk[2 * DP + 33], kq = tk[2 * DP + 34];
      float2 kk[CPL / 2];
      float2 ka = make_float2(0.f, 0.f), qa = ka, kb = ka, qb = ka;  // S^T k and S^T q of the two columns, even / odd channels
#pragma unroll
      for (int i = 0; i < CPL / 4; ++i) {
        const float4 q = q4[sub + 8 * i], kv = k4[sub + 8 * i];
        const float2 q0 = make_float2(q.x, q.y), q1 = make_float2(q.z, q.w);
        kk[2 * i] = make_float2(kv.x, kv.y);
        kk[2 * i + 1] = make_float2(kv.z, kv.w);
        ka = __ffma2_rn(Sa[2 * i], kk[2 * i], ka); ka = __ffma2_rn(Sa[2 * i + 1], kk[2 * i + 1], ka);
        qa = __ffma2_rn(Sa[2 * i], q0, qa);        qa = __ffma2_rn(Sa[2 * i + 1], q1, qa);
        kb = __ffma2_rn(Sb[2 * i], kk[2 * i], kb); kb = __ffma2_rn(Sb[2 * i + 1], kk[2 * i + 1], kb);
        qb = __ffma2_rn(Sb[2 * i], q0, qb);        qb = __ffma2_rn(Sb[2 * i + 1], q1, qb);
      }
      float ska = ka.x + ka.y, sqa = qa.x + qa.y, skb = kb.x + kb.y, sqb = qb.x + qb.y;
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) {
        ska += __shfl_xor_sync(0xffffffffu, ska, o);
        sqa += __shfl_xor_sync(0xffffffffu, sqa, o);
        skb += __shfl_xor_sync(0xffffffffu, skb, o);
        sqb += __shfl_xor_sync(0xffffffffu, sqb, o);
      }
      const float ua = beta * (va - g * ska), ub = beta * (vb - g * skb);
      const float2 ua2 = make_float2(ua, ua), ub2 = make_float2(ub, ub), g2 = make_float2(g, g);
#pragma unroll
      for (int i = 0; i < CPL / 2; ++i) {
        Sa[i] = __ffma2_rn(kk[i], ua2, __fmul2_rn(g2, Sa[i]));
        Sb[i] = __ffma2_rn(kk[i], ub2, __fmul2_rn(g2, Sb[i]));
      }
      if (sub == 0) {
        obuf[tt * 32 + col] = fmaf(kq, ua, g * sqa);
        obuf[tt * 32 + col + 16] = fmaf(kq, ub, g * sqb);
      }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < nt * 32; e += blockDim.x) {
      const int tt = e >> 5, c = e & 31;
      if (blockIdx.z * 32 + c < a.Dv) a.out[(size_t)(tc + tt) * a.ldo + (size_t)h * a.Dv + blockIdx.z * 32 + c] = obuf[e];
    }
    __syncthreads();  // the stage and the outputs are rewritten in the next iteration
  }
#pragma unroll
  for (int i = 0; i < CPL / 4; ++i)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int ch = 4 * (sub + 8 * i) + 2 * e;
      if (live0 && ch < D) st[(size_t)ch * a.Dv + j0] = Sa[2 * i + e].x;
      if (live0 && ch + 1 < D) st[(size_t)(ch + 1) * a.Dv + j0] = Sa[2 * i + e].y;
      if (live1 && ch < D) st[(size_t)ch * a.Dv + j1] = Sb[2 * i + e].x;
      if (live1 && ch + 1 < D) st[(size_t)(ch + 1) * a.Dv + j1] = Sb[2 * i + e].y;
    }
}

template <int CPL>
cudaError_t launch_delta(cudaStream_t s, const DeltaArgs& a) {
  constexpr int DP = 8 * CPL;
  const size_t smem = (size_t)(2 * kDelTch * (2 * DP + 36) + kDelTch * 32) * 4;
  dim3 grid(a.B, a.H, (a.Dv + 31) / 32);
  delta_recurrence_kernel<CPL><<<grid, kDelThreads, smem, s>>>(a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t stack_delta_init() {
  cudaError_t e;
  if ((e = cudaFuncSetAttribute(delta_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(delta_prep_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(delta_recurrence_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(delta_recurrence_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024)) != cudaSuccess) return e;
  return cudaSuccess;
}

cudaError_t delta_prep(cudaStream_t s, const DeltaPrepArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  const size_t C = 2 * (size_t)a.G * a.D + (size_t)a.H * a.Dv;
  if (a.taps < 1 || a.taps - 1 > kMaxTail || C * 4 > 160 * 1024 || a.G <= 0 || a.H % a.G) return cudaErrorInvalidValue;
  if (a.f32) delta_prep_kernel<float><<<a.T, 256, C * 4, s>>>(a);
  else delta_prep_kernel<bf16><<<a.T, 256, C * 4, s>>>(a);
  return cudaGetLastError();
}

cudaError_t delta_conv_tails(cudaStream_t s, const DeltaPrepArgs& a) {
  if (a.B <= 0 || a.taps <= 1) return cudaSuccess;
  const int C = 2 * a.G * a.D + a.H * a.Dv;
  delta_tails_kernel<<<dim3((C + 255) / 256, a.B), 256, 0, s>>>(a);
  return cudaGetLastError();
}

cudaError_t delta_recurrence(cudaStream_t s, const DeltaArgs& a) {
  if (a.B <= 0) return cudaSuccess;
  if (a.G <= 0 || a.H % a.G || a.D > 256) return cudaErrorInvalidValue;
  if (a.D <= 32) return launch_delta<4>(s, a);
  if (a.D <= 64) return launch_delta<8>(s, a);
  if (a.D <= 128) return launch_delta<16>(s, a);
  return launch_delta<32>(s, a);
}

}  // namespace hb
