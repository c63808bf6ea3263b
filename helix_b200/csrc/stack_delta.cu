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
  extern __shared__ float row[];
  const int t = blockIdx.x;
  const int b = a.seq_of[t], t0 = a.cu[b];
  const int GD = a.G * a.D, C = 2 * GD + a.H * a.Dv, taps = a.taps;
  const bool fresh = a.first_pos[b] == 0;
  const float* tail = a.state + (size_t)a.slots[b] * a.slot_stride + a.tail_off;  // [taps - 1][C]: inputs of positions first - (taps - 1) ..
  const WT* cw = (const WT*)a.conv_w;
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
  for (int i = threadIdx.x; i < a.H * a.Dv; i += blockDim.x) out[2 * GD + i] = row[2 * GD + i];
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
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Block = (entry, head, 32 value columns), 256 threads: a state column is shared by 8 lanes, lane `sub` of them keeps the key
// channels 4 (sub + 8 i) .. + 3, i < CPL / 4, in registers (the 8 lanes of a column read 128 contiguous bytes of q or k per
// step).  Per token both products with the OLD state, S^T k and S^T q, are formed in one pass and added over the 8 lanes by a
// butterfly; the write u and the output o = g S^T q + (k . q) u follow from them, then the state is updated in place.
// Tokens are staged kDelTch at a time through a cp.async double buffer.
template <int CPL>
__global__ void __launch_bounds__(256) delta_recurrence_kernel(DeltaArgs a) {
  constexpr int DP = 8 * CPL;                     // padded key channels
  constexpr int per_tok = 2 * DP + 32 + 4;        // q | k | v (this block's columns) | beta, decay, k.q, pad
  constexpr int stage_floats = kDelTch * per_tok;
  extern __shared__ float sm[];                   // 2 stages + outputs [kDelTch][32]
  float* obuf = sm + 2 * stage_floats;
  const int b = blockIdx.x, h = blockIdx.y, kvh = h / (a.H / a.G);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, sub = lane & 7;
  const int col = w * 4 + (lane >> 3);            // column of this block's slice
  const int j = blockIdx.z * 32 + col;
  const bool live = j < a.Dv;
  const int t0 = a.cu[b], t1 = a.cu[b + 1];
  const int D = a.D;
  float* st = a.state + (size_t)a.slots[b] * a.slot_stride + (size_t)h * D * a.Dv;
  const bool fresh = a.first_pos[b] == 0;
  float S[CPL];
#pragma unroll
  for (int i = 0; i < CPL / 4; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int ch = 4 * (sub + 8 * i) + e;
      S[4 * i + e] = (!fresh && live && ch < D) ? st[(size_t)ch * a.Dv + j] : 0.f;
    }
  for (int e = threadIdx.x; e < 2 * stage_floats; e += blockDim.x) sm[e] = 0.f;  // padded channels read zeros
  __syncthreads();
  auto issue = [&](int tc, int stage) {
    const int nt = min(kDelTch, t1 - tc);
    float* base = sm + stage * stage_floats;
    for (int e = threadIdx.x; e < nt * D; e += blockDim.x) {
      const int tt = e / D, i = e % D;
      const float* src = a.in + (size_t)(tc + tt) * a.ld;
      float* dst = base + tt * per_tok;
      cp_async4(dst + i, src + a.off_q + kvh * D + i);
      cp_async4(dst + DP + i, src + a.off_k + kvh * D + i);
    }
    for (int e = threadIdx.x; e < nt * 32; e += blockDim.x) {
      const int tt = e >> 5, c = e & 31;
      if (blockIdx.z * 32 + c < a.Dv)
        cp_async4(base + tt * per_tok + 2 * DP + c, a.in + (size_t)(tc + tt) * a.ld + a.off_v + (size_t)h * a.Dv + blockIdx.z * 32 + c);
    }
    for (int tt = threadIdx.x; tt < nt; tt += blockDim.x) {
      const float* src = a.in + (size_t)(tc + tt) * a.ld;
      float* dst = base + tt * per_tok + 2 * DP + 32;
      cp_async4(dst, src + a.off_beta + h);
      cp_async4(dst + 1, src + a.off_decay + h);
      cp_async4(dst + 2, src + a.off_kq + kvh);
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
      const float vj = tk[2 * DP + col];
      const float beta = tk[2 * DP + 32], g = tk[2 * DP + 33], kq = tk[2 * DP + 34];
      float4 kk[CPL / 4];
      float sk0 = 0.f, sk1 = 0.f, sq0 = 0.f, sq1 = 0.f;
#pragma unroll
      for (int i = 0; i < CPL / 4; ++i) {
        const float4 q = q4[sub + 8 * i];
        kk[i] = k4[sub + 8 * i];
        sk0 = fmaf(S[4 * i + 0], kk[i].x, sk0); sk1 = fmaf(S[4 * i + 1], kk[i].y, sk1);
        sk0 = fmaf(S[4 * i + 2], kk[i].z, sk0); sk1 = fmaf(S[4 * i + 3], kk[i].w, sk1);
        sq0 = fmaf(S[4 * i + 0], q.x, sq0); sq1 = fmaf(S[4 * i + 1], q.y, sq1);
        sq0 = fmaf(S[4 * i + 2], q.z, sq0); sq1 = fmaf(S[4 * i + 3], q.w, sq1);
      }
      float sk = sk0 + sk1, sq = sq0 + sq1;
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) {
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
      }
      const float u = beta * (vj - g * sk);
#pragma unroll
      for (int i = 0; i < CPL / 4; ++i) {
        S[4 * i + 0] = fmaf(kk[i].x, u, g * S[4 * i + 0]);
        S[4 * i + 1] = fmaf(kk[i].y, u, g * S[4 * i + 1]);
        S[4 * i + 2] = fmaf(kk[i].z, u, g * S[4 * i + 2]);
        S[4 * i + 3] = fmaf(kk[i].w, u, g * S[4 * i + 3]);
      }
      if (sub == 0) obuf[tt * 32 + col] = fmaf(kq, u, g * sq);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < nt * 32; e += blockDim.x) {
      const int tt = e >> 5, c = e & 31;
      if (blockIdx.z * 32 + c < a.Dv) a.out[(size_t)(tc + tt) * a.ldo + (size_t)h * a.Dv + blockIdx.z * 32 + c] = obuf[e];
    }
    __syncthreads();  // the stage and the outputs are rewritten in the next iteration
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < CPL / 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ch = 4 * (sub + 8 * i) + e;
        if (ch < D) st[(size_t)ch * a.Dv + j] = S[4 * i + e];
      }
  }
}

template <int CPL>
cudaError_t launch_delta(cudaStream_t s, const DeltaArgs& a) {
  constexpr int DP = 8 * CPL;
  const size_t smem = (size_t)(2 * kDelTch * (2 * DP + 36) + kDelTch * 32) * 4;
  dim3 grid(a.B, a.H, (a.Dv + 31) / 32);
  delta_recurrence_kernel<CPL><<<grid, 256, smem, s>>>(a);
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
