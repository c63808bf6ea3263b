// Feed-forward units of layer-list decoders beyond the clamped one: the plain gated unit (act(gate) * up with silu or
// tanh-GELU) and the mixture of experts — router softmax and corrected top-k choice in fp32, expert units per (token,
// choice), weighted combination with identity outputs.  Every sum has a fixed order per output element.
#include <math.h>

#include <algorithm>

#include "kernels.h"
#include "launch.h"
#include "stack_common.cuh"

namespace hb {
namespace {

__device__ __forceinline__ float gelu_tanh_(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
// one gated pair: act(gate) * up, or the clamped form min(g, limit) sigmoid(1.702 g) (clamp(u, +-limit) + 1)
__device__ __forceinline__ float glu_pair(float g, float u, int act, float limit) {
  if (act == GLU_CLAMPED) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoidf_(1.702f * g) * (u + 1.f);
  }
  return (act == GLU_GELU_TANH ? gelu_tanh_(g) : g * sigmoidf_(g)) * u;
}

// VEC = 4: F and ldg are multiples of four (16-byte loads and stores).  PACKED: gate j of tile i sits at column 256 i + j and
// its up at 256 i + 128 + j (weights stored per 256-row tile as [128 gate | 128 up]); the output column is 128 i + j
template <int VEC, bool PACKED>
__global__ void gated_unit_kernel(const float* __restrict__ gu, long ldg, int act, float* __restrict__ out, bf16* __restrict__ outb, int F,
                                  float limit) {
  const size_t t = blockIdx.x;
  const int j = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (j >= F) return;
  const size_t gi = PACKED ? (size_t)(j >> 7) * 256 + (j & 127) : (size_t)j, ui = PACKED ? gi + 128 : (size_t)F + j;
  if (VEC == 4) {
    const float4 g = *reinterpret_cast<const float4*>(gu + t * ldg + gi);
    const float4 u = *reinterpret_cast<const float4*>(gu + t * ldg + ui);
    const float v0 = glu_pair(g.x, u.x, act, limit), v1 = glu_pair(g.y, u.y, act, limit), v2 = glu_pair(g.z, u.z, act, limit),
                v3 = glu_pair(g.w, u.w, act, limit);
    if (out) *reinterpret_cast<float4*>(out + t * F + j) = make_float4(v0, v1, v2, v3);
    if (outb) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v0, v1), hi = __floats2bfloat162_rn(v2, v3);
      uint2 pk;
      pk.x = *reinterpret_cast<unsigned*>(&lo);
      pk.y = *reinterpret_cast<unsigned*>(&hi);
      *reinterpret_cast<uint2*>(outb + t * F + j) = pk;
    }
  } else {
    const float v = glu_pair(gu[t * ldg + gi], gu[t * ldg + ui], act, limit);
    if (out) out[t * F + j] = v;
    if (outb) outb[t * F + j] = __float2bfloat16(v);
  }
}

// The choice of one token by one warp: zr[R] router logits (global or shared memory), pick[2 R] scratch in shared memory
// (choice scores, then group scores).
template <typename WT>
__device__ __forceinline__ void route_one(const float* zr, const WT* __restrict__ corr, int R, int top_k, float* pick,
                                          int32_t* __restrict__ ids, float* __restrict__ wts, int l, const RouteOpts& ro) {
  float mx = 0.f, inv = 1.f;
  if (!ro.sigmoid) {
    mx = -INFINITY;
    for (int i = l; i < R; i += 32) mx = fmaxf(mx, zr[i]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = l; i < R; i += 32) sum += expf(zr[i] - mx);
    sum = warp_sum(sum);
    inv = 1.f / sum;
  }
  auto score = [&](int i) { return ro.sigmoid ? sigmoidf_(zr[i]) : expf(zr[i] - mx) * inv; };
  for (int i = l; i < R; i += 32) pick[i] = score(i) + ldf<WT>(corr, i);
  __syncwarp();
  if (ro.groups > 1 && ro.keep < ro.groups) {
    float* gs = pick + R;
    const int per = R / ro.groups;
    for (int g = l; g < ro.groups; g += 32) {  // a group scores the sum of its two largest choice scores
      float a = -INFINITY, b = -INFINITY;
      for (int i = g * per; i < (g + 1) * per; ++i) {
        const float v = pick[i];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      gs[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    for (int k = 0; k < ro.keep; ++k) {  // the kept groups are marked with -inf (a real score is finite)
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = l; g < ro.groups; g += 32) {
        const float v = gs[g];
        if (v > best) { best = v; bi = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      if (l == 0 && bi < ro.groups) gs[bi] = -INFINITY;
      __syncwarp();
    }
    for (int i = l; i < R; i += 32)
      if (gs[i / per] != -INFINITY) pick[i] = -INFINITY;  // outputs of dropped groups cannot be chosen
    __syncwarp();
  }
  float wsum = 0.f;
  for (int k = 0; k < top_k; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = l; i < R; i += 32) {
      const float v = pick[i];
      if (v > best) { best = v; bi = i; }  // ascending i: the lowest index among equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (l == 0) {
      if (bi >= R) bi = 0;  // fewer eligible outputs than top_k (excluded at load): stay inside the tables
      const float sc = score(bi);  // the score itself, without the correction
      ids[k] = bi;
      wts[k] = sc;
      wsum += sc;
      pick[bi] = -INFINITY;
    }
    __syncwarp();
  }
  if (l == 0) {
    const float f = (ro.renorm ? 1.f / (wsum + 1e-20f) : 1.f) * ro.scale;
    if (f != 1.f)
      for (int k = 0; k < top_k; ++k) wts[k] *= f;
  }
}

// One warp per token.  dynamic smem: per warp 2 R floats (the choice scores while the top-k is taken, group scores)
template <typename WT>
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ z, long ldz, const WT* __restrict__ corr, int R,
                                                        int top_k, int32_t* __restrict__ ids, float* __restrict__ wts, int T, RouteOpts ro) {
  extern __shared__ float sm[];
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + w;
  if (t >= T) return;
  route_one<WT>(z + (size_t)t * ldz, corr, R, top_k, sm + (size_t)w * 2 * R, ids + (size_t)t * top_k, wts + (size_t)t * top_k, l, ro);
}

// Router logits and choice in one kernel: the router's rows stay in shared memory, every warp takes tokens in turn and
// forms the R dot products of its token's fp32 row (lanes stride the row four entries at a time, kRouterRT outputs per pass
// so that a pass keeps many independent loads in flight), then chooses.
// dynamic smem: router [R][W] of WT | per warp: logits [R] + scratch [2 R]
constexpr int kRouterWarps = 16;
constexpr int kRouterRT = 16;
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename WT>
__global__ void __launch_bounds__(kRouterWarps * 32) moe_router_kernel(const float* __restrict__ x, const WT* __restrict__ router,
                                                                       const WT* __restrict__ corr, int R, int W, int top_k,
                                                                       int32_t* __restrict__ ids, float* __restrict__ wts, int T, RouteOpts ro) {
  extern __shared__ float sm[];
  WT* rw = reinterpret_cast<WT*>(sm);
  float* zs = sm + ((size_t)R * W * sizeof(WT) + 15) / 16 * 4;
  {
    const size_t bytes = (size_t)R * W * sizeof(WT), n16 = ((uintptr_t)router & 15) ? 0 : bytes / 16;
    const uint4* src = reinterpret_cast<const uint4*>(router);
    uint4* dst = reinterpret_cast<uint4*>(sm);
    for (size_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
    for (size_t i = n16 * 16 / sizeof(WT) + threadIdx.x; i < (size_t)R * W; i += blockDim.x) rw[i] = router[i];
  }
  __syncthreads();
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  float* z = zs + (size_t)w * 3 * R;
  for (int t = blockIdx.x * kRouterWarps + w; t < T; t += gridDim.x * kRouterWarps) {
    const float* xr = x + (size_t)t * W;
    for (int r0 = 0; r0 < R; r0 += kRouterRT) {
      float acc[kRouterRT] = {};
      if ((W & 3) == 0) {
#pragma unroll 2
        for (int i = l * 4; i < W; i += 128) {
          const float4 xv = ld4(xr + i);
#pragma unroll
          for (int c = 0; c < kRouterRT; ++c)
            if (r0 + c < R) {
              const float4 wv = ld4(rw + (size_t)(r0 + c) * W + i);
              acc[c] = fmaf(xv.x, wv.x, acc[c]); acc[c] = fmaf(xv.y, wv.y, acc[c]);
              acc[c] = fmaf(xv.z, wv.z, acc[c]); acc[c] = fmaf(xv.w, wv.w, acc[c]);
            }
        }
      } else {
        for (int i = l; i < W; i += 32) {
          const float xv = xr[i];
#pragma unroll
          for (int c = 0; c < kRouterRT; ++c)
            if (r0 + c < R) acc[c] = fmaf(xv, ldf<WT>(rw, (size_t)(r0 + c) * W + i), acc[c]);
        }
      }
#pragma unroll
      for (int c = 0; c < kRouterRT; ++c) {
        const float v = warp_sum(acc[c]);
        if (l == 0 && r0 + c < R) z[r0 + c] = v;
      }
    }
    __syncwarp();
    route_one<WT>(z, corr, R, top_k, z + R, ids + (size_t)t * top_k, wts + (size_t)t * top_k, l, ro);
    __syncwarp();
  }
}

// Steps of few tokens: one block per token, warp w forms the outputs w, w + warps, ... straight from the router's rows in
// global memory (each row is read once per block), warp 0 chooses.  dynamic smem: logits [R] + scratch [2 R]
template <typename WT>
__global__ void __launch_bounds__(kRouterWarps * 32) moe_router_small_kernel(const float* __restrict__ x, const WT* __restrict__ router,
                                                                             const WT* __restrict__ corr, int R, int W, int top_k,
                                                                             int32_t* __restrict__ ids, float* __restrict__ wts, RouteOpts ro) {
  extern __shared__ float sm[];
  const int t = blockIdx.x, w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const float* xr = x + (size_t)t * W;
  const bool vec = (W & 3) == 0 && ((uintptr_t)router & 15) == 0;
  for (int r = w; r < R; r += kRouterWarps) {
    const WT* row = router + (size_t)r * W;
    float acc = 0.f;
    if (vec) {
      for (int i = l * 4; i < W; i += 128) {
        const float4 xv = ld4(xr + i), wv = ld4(row + i);
        acc = fmaf(xv.x, wv.x, acc); acc = fmaf(xv.y, wv.y, acc); acc = fmaf(xv.z, wv.z, acc); acc = fmaf(xv.w, wv.w, acc);
      }
    } else {
      for (int i = l; i < W; i += 32) acc = fmaf(xr[i], ldf<WT>(row, i), acc);
    }
    acc = warp_sum(acc);
    if (l == 0) sm[r] = acc;
  }
  __syncthreads();
  if (w == 0) route_one<WT>(sm, corr, R, top_k, sm + R, ids + (size_t)t * top_k, wts + (size_t)t * top_k, l, ro);
}

// bf16 in, bf16 out: h[t, j] = act(gu[t, j]) * gu[t, F + j], eight columns per thread (F and ldg multiples of eight)
__global__ void gated_unit_b16_kernel(const bf16* __restrict__ gu, long ldg, int act, bf16* __restrict__ out, int F, float limit) {
  const size_t t = blockIdx.x;
  const int j = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (j >= F) return;
  const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * ldg + j);
  const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * ldg + F + j);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
  uint4 o4;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
    o2[e] = __floats2bfloat162_rn(glu_pair(g.x, u.x, act, limit), glu_pair(g.y, u.y, act, limit));
  }
  *reinterpret_cast<uint4*>(out + t * F + j) = o4;
}

// dot product of a weight row with a vector in shared memory, lanes striding the row; every lane gets the sum
template <typename WT>
__device__ __forceinline__ float warp_dot(const WT* __restrict__ wrow, const float* __restrict__ xs, int n, int lane) {
  float s = 0.f;
  if (sizeof(WT) == 2 && (n & 7) == 0 && ((uintptr_t)wrow & 15) == 0) {
    for (int i = lane * 8; i < n; i += 256) {
      const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(wrow) + i);
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p2[e]);
        s = fmaf(f.x, xs[i + 2 * e], s);
        s = fmaf(f.y, xs[i + 2 * e + 1], s);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) s = fmaf(ldf<WT>(wrow, i), xs[i], s);
  }
  return warp_sum(s);
}

// block per (token, choice).  dynamic smem: x [Wp] + inner activation [F]
template <typename WT>
__global__ void __launch_bounds__(256) moe_expert_rows_kernel(const float* __restrict__ x, const bf16* __restrict__ xb,
                                                              const WT* __restrict__ w_gu, const WT* __restrict__ w_down,
                                                              const int32_t* __restrict__ ids, int E, int F, int W,
                                                              float* __restrict__ y, int packed, int act, float limit) {
  extern __shared__ float sm[];
  const int t = blockIdx.x;
  const size_t item = (size_t)t * gridDim.y + blockIdx.y;  // (token, choice)
  const int e = ids[item];
  if (e >= E) return;
  float* xs = sm;
  float* hs = sm + (W + 3) / 4 * 4;
  for (int i = threadIdx.x; i < W; i += blockDim.x) xs[i] = xb ? __bfloat162float(xb[(size_t)t * W + i]) : x[(size_t)t * W + i];
  __syncthreads();
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  const WT* gu = w_gu + (size_t)e * 2 * F * W;
  for (int f = w; f < F; f += nw) {
    const size_t gr = packed ? (size_t)(f >> 7) * 256 + (f & 127) : (size_t)f, ur = packed ? gr + 128 : (size_t)F + f;
    const float g = warp_dot<WT>(gu + gr * W, xs, W, l);
    const float u = warp_dot<WT>(gu + ur * W, xs, W, l);
    if (l == 0) {
      float v = glu_pair(g, u, act, limit);
      if (xb) v = __bfloat162float(__float2bfloat16(v));
      hs[f] = v;
    }
  }
  __syncthreads();
  const WT* dn = w_down + (size_t)e * W * F;
  for (int c = w; c < W; c += nw) {
    const float v = warp_dot<WT>(dn + (size_t)c * F, hs, F, l);
    if (l == 0) y[item * W + c] = v;
  }
}

__global__ void moe_combine_kernel(const float* __restrict__ x, const float* __restrict__ y, const int32_t* __restrict__ ids,
                                   const float* __restrict__ wts, int top_k, int E, float* out, int W, const float* add) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float acc = add ? add[(size_t)t * W + c] : 0.f;
    for (int k = 0; k < top_k; ++k) {
      const size_t item = (size_t)t * top_k + k;
      const float v = ids[item] < E ? y[item * W + c] : x[(size_t)t * W + c];
      acc = fmaf(wts[item], v, acc);
    }
    out[(size_t)t * W + c] = acc;
  }
}

// Groups the (token, choice) items by expert for the grouped tensor-core products, in three small launches: count per
// expert (and mark every row of the buffer empty), offsets and the m tiles' experts, rows.  Expert e's items get the rows
// [off_e, off_e + count_e) of a row buffer whose per-expert segments start on multiples of 128 rows (one m tile never mixes
// experts); rows between segments and behind the last one stay empty (src -1) and belong to expert 0's tiles, so every tile
// of the buffer can be multiplied without the host knowing the counts.  Which row of its segment an item gets depends on
// arrival order; a row's product does not depend on where the row sits.  scratch: [E] counts | [E] offsets | [E] cursors.
__global__ void moe_count_kernel(const int32_t* __restrict__ ids, int n_items, int E, int max_rows, int32_t* __restrict__ src_of_row,
                                 int32_t* __restrict__ scratch) {
  const int stride = gridDim.x * blockDim.x;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < max_rows; i += stride) {
    src_of_row[i] = -1;
    if (i < n_items) {
      const int e = ids[i];
      if (e < E) atomicAdd(&scratch[e], 1);
    }
  }
}
__global__ void moe_offsets_kernel(int E, int max_rows, int32_t* __restrict__ scratch, int32_t* __restrict__ tile_group) {
  __shared__ int s_off[4097];
  if (threadIdx.x == 0) {
    int o = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = o;
      o += (scratch[e] + 127) / 128 * 128;
    }
    s_off[E] = o;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    scratch[E + e] = s_off[e];
    scratch[2 * E + e] = 0;
    for (int tl = s_off[e] / 128; tl < s_off[e + 1] / 128; ++tl) tile_group[tl] = e;
  }
  for (int tl = s_off[E] / 128 + threadIdx.x; tl < max_rows / 128; tl += blockDim.x) tile_group[tl] = 0;
}
__global__ void moe_rows_kernel(const int32_t* __restrict__ ids, int n_items, int top_k, int E, int32_t* __restrict__ scratch,
                                int32_t* __restrict__ row_of, int32_t* __restrict__ src_of_row) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_items) return;
  const int e = ids[i];
  int r = -1;
  if (e < E) {
    r = scratch[E + e] + atomicAdd(&scratch[2 * E + e], 1);
    src_of_row[r] = i / top_k;
  }
  row_of[i] = r;
}

// The same grouping by one block (steps of few items: one launch instead of three).
__global__ void __launch_bounds__(1024) moe_group_small_kernel(const int32_t* __restrict__ ids, int n_items, int top_k, int E, int max_rows,
                                                         int32_t* __restrict__ row_of, int32_t* __restrict__ src_of_row,
                                                         int32_t* __restrict__ tile_group) {
  extern __shared__ int smi[];
  int* cnt = smi;
  int* off = smi + E;
  int* cur = smi + 2 * E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
    const int e = ids[i];
    if (e < E) atomicAdd(&cnt[e], 1);
  }
  for (int r = threadIdx.x; r < max_rows; r += blockDim.x) src_of_row[r] = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o;
      cur[e] = 0;
      const int nt = (cnt[e] + 127) / 128;
      for (int k = 0; k < nt; ++k) tile_group[o / 128 + k] = e;
      o += nt * 128;
    }
    for (int tl = o / 128; tl < max_rows / 128; ++tl) tile_group[tl] = 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
    const int e = ids[i];
    int r = -1;
    if (e < E) {
      r = off[e] + atomicAdd(&cur[e], 1);
      src_of_row[r] = i / top_k;
    }
    row_of[i] = r;
  }
}

// a16[r, :] = x16[src_of_row[r], :], zeros for empty rows.  W is a multiple of 8 (16-byte pieces)
__global__ void __launch_bounds__(128) moe_gather_kernel(const bf16* __restrict__ x16, int W, const int32_t* __restrict__ src_of_row,
                                                         bf16* __restrict__ a16) {
  const size_t r = blockIdx.x;
  const int src = src_of_row[r];
  uint4* dst = reinterpret_cast<uint4*>(a16 + r * W);
  const uint4* from = reinterpret_cast<const uint4*>(x16 + (size_t)(src < 0 ? 0 : src) * W);
  for (int i = threadIdx.x; i < W / 8; i += blockDim.x) dst[i] = src < 0 ? make_uint4(0, 0, 0, 0) : from[i];
}

__global__ void moe_combine_rows_kernel(const float* __restrict__ x, const bf16* __restrict__ y, const int32_t* __restrict__ row_of,
                                        const float* __restrict__ wts, int top_k, float* out, int W, const float* add) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float acc = add ? add[(size_t)t * W + c] : 0.f;
    for (int k = 0; k < top_k; ++k) {
      const size_t item = (size_t)t * top_k + k;
      const int r = row_of[item];
      const float v = r >= 0 ? __bfloat162float(y[(size_t)r * W + c]) : x[(size_t)t * W + c];
      acc = fmaf(wts[item], v, acc);
    }
    out[(size_t)t * W + c] = acc;
  }
}

}  // namespace

int moe_group_max_rows(int n_items, int E) { return (n_items + 127) / 128 * 128 + E * 128; }

cudaError_t moe_group_rows(cudaStream_t s, const int32_t* ids, int n_items, int top_k, int E, int32_t* row_of, int32_t* src_of_row,
                           int32_t* tile_group, int32_t* scratch) {
  if (n_items <= 0) return cudaSuccess;
  if (E > 4096) return cudaErrorInvalidValue;
  const int max_rows = moe_group_max_rows(n_items, E);
  if (n_items <= 4096) {
    moe_group_small_kernel<<<1, 1024, (size_t)3 * E * 4, s>>>(ids, n_items, top_k, E, max_rows, row_of, src_of_row, tile_group);
    return cudaGetLastError();
  }
  cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)E * 4, s);
  if (e != cudaSuccess) return e;
  moe_count_kernel<<<std::min((max_rows + 255) / 256, 1184), 256, 0, s>>>(ids, n_items, E, max_rows, src_of_row, scratch);
  moe_offsets_kernel<<<1, 256, 0, s>>>(E, max_rows, scratch, tile_group);
  moe_rows_kernel<<<(n_items + 255) / 256, 256, 0, s>>>(ids, n_items, top_k, E, scratch, row_of, src_of_row);
  return cudaGetLastError();
}

cudaError_t moe_gather_rows(cudaStream_t s, const bf16* x16, int W, const int32_t* src_of_row, bf16* a16, int rows) {
  if (rows <= 0) return cudaSuccess;
  if (W % 8) return cudaErrorInvalidValue;
  moe_gather_kernel<<<rows, 128, 0, s>>>(x16, W, src_of_row, a16);
  return cudaGetLastError();
}

cudaError_t moe_combine_rows(cudaStream_t s, const float* x, const bf16* y, const int32_t* row_of, const float* wts, int top_k,
                             float* out, int T, int W, const float* add) {
  if (T <= 0) return cudaSuccess;
  moe_combine_rows_kernel<<<T, 256, 0, s>>>(x, y, row_of, wts, top_k, out, W, add);
  return cudaGetLastError();
}

cudaError_t stack_moe_init() {
  cudaError_t e;
  const int big = 200 * 1024;
  if ((e = cudaFuncSetAttribute(moe_router_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, big)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(moe_router_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(moe_expert_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, big)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(moe_expert_rows_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big)) != cudaSuccess) return e;
  return cudaSuccess;
}

cudaError_t gated_unit(cudaStream_t s, const float* gu, long ldg, int act, float* out, bf16* outb, int T, int F, bool packed, float limit) {
  if (T <= 0) return cudaSuccess;
  if (packed && F % 128) return cudaErrorInvalidValue;
  const bool vec = F % 4 == 0 && ldg % 4 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)outb & 7) == 0;
  dim3 grid(T, ((vec ? F / 4 : F) + 255) / 256);
  if (vec && packed) gated_unit_kernel<4, true><<<grid, 256, 0, s>>>(gu, ldg, act, out, outb, F, limit);
  else if (vec) gated_unit_kernel<4, false><<<grid, 256, 0, s>>>(gu, ldg, act, out, outb, F, limit);
  else if (packed) gated_unit_kernel<1, true><<<grid, 256, 0, s>>>(gu, ldg, act, out, outb, F, limit);
  else gated_unit_kernel<1, false><<<grid, 256, 0, s>>>(gu, ldg, act, out, outb, F, limit);
  return cudaGetLastError();
}

cudaError_t moe_route(cudaStream_t s, const float* z, long ldz, const void* corr, bool f32, int R, int top_k, int32_t* ids, float* wts,
                      int T, const RouteOpts& ro) {
  if (T <= 0) return cudaSuccess;
  if (R <= 0 || top_k <= 0 || top_k > R || R > 1024 || (ro.groups > 1 && R % ro.groups)) return cudaErrorInvalidValue;
  const size_t smem = (size_t)4 * 2 * R * 4;
  if (f32) moe_route_kernel<float><<<(T + 3) / 4, 128, smem, s>>>(z, ldz, (const float*)corr, R, top_k, ids, wts, T, ro);
  else moe_route_kernel<bf16><<<(T + 3) / 4, 128, smem, s>>>(z, ldz, (const bf16*)corr, R, top_k, ids, wts, T, ro);
  return cudaGetLastError();
}

size_t moe_router_smem(int R, int W, bool f32) {
  return ((size_t)R * W * (f32 ? 4 : 2) + 15) / 16 * 16 + (size_t)kRouterWarps * 3 * R * 4;
}
cudaError_t moe_router(cudaStream_t s, const float* x, const void* router, const void* corr, bool f32, int R, int W, int top_k,
                       int32_t* ids, float* wts, int T, int sms, const RouteOpts& ro) {
  if (T <= 0) return cudaSuccess;
  if (R <= 0 || top_k <= 0 || top_k > R || (ro.groups > 1 && R % ro.groups)) return cudaErrorInvalidValue;
  if (T <= 2 * (sms > 0 ? sms : 148) && R <= 4096) {  // few tokens: a block per token, no staging of the router
    const size_t sm_small = (size_t)3 * R * 4;
    if (f32) moe_router_small_kernel<float><<<T, kRouterWarps * 32, sm_small, s>>>(x, (const float*)router, (const float*)corr, R, W, top_k, ids, wts, ro);
    else moe_router_small_kernel<bf16><<<T, kRouterWarps * 32, sm_small, s>>>(x, (const bf16*)router, (const bf16*)corr, R, W, top_k, ids, wts, ro);
    return cudaGetLastError();
  }
  const size_t smem = moe_router_smem(R, W, f32);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  const int grid = std::max(1, std::min((T + kRouterWarps - 1) / kRouterWarps, sms > 0 ? sms : 148));
  if (f32) moe_router_kernel<float><<<grid, kRouterWarps * 32, smem, s>>>(x, (const float*)router, (const float*)corr, R, W, top_k, ids, wts, T, ro);
  else moe_router_kernel<bf16><<<grid, kRouterWarps * 32, smem, s>>>(x, (const bf16*)router, (const bf16*)corr, R, W, top_k, ids, wts, T, ro);
  return cudaGetLastError();
}

cudaError_t gated_unit_b16(cudaStream_t s, const bf16* gu, long ldg, int act, bf16* out, int T, int F, float limit) {
  if (T <= 0) return cudaSuccess;
  if (F % 8 || ldg % 8 || ((uintptr_t)gu & 15) || ((uintptr_t)out & 15)) return cudaErrorInvalidValue;
  gated_unit_b16_kernel<<<dim3(T, (F / 8 + 255) / 256), 256, 0, s>>>(gu, ldg, act, out, F, limit);
  return cudaGetLastError();
}

cudaError_t moe_expert_rows(cudaStream_t s, const float* x, const bf16* xb, const void* w_gu, const void* w_down, bool f32,
                            const int32_t* ids, int top_k, int E, int F, int W, float* y, int T, bool packed, int act, float limit) {
  if (T <= 0) return cudaSuccess;
  const size_t smem = ((size_t)(W + 3) / 4 * 4 + F) * 4;
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  dim3 grid(T, top_k);
  if (f32) moe_expert_rows_kernel<float><<<grid, 256, smem, s>>>(x, xb, (const float*)w_gu, (const float*)w_down, ids, E, F, W, y, packed ? 1 : 0, act, limit);
  else moe_expert_rows_kernel<bf16><<<grid, 256, smem, s>>>(x, xb, (const bf16*)w_gu, (const bf16*)w_down, ids, E, F, W, y, packed ? 1 : 0, act, limit);
  return cudaGetLastError();
}

cudaError_t moe_combine(cudaStream_t s, const float* x, const float* y, const int32_t* ids, const float* wts, int top_k, int E, float* out,
                        int T, int W, const float* add) {
  if (T <= 0) return cudaSuccess;
  moe_combine_kernel<<<T, 256, 0, s>>>(x, y, ids, wts, top_k, E, out, W, add);
  return cudaGetLastError();
}

}  // namespace hb
