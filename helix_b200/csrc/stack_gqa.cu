// Grouped-query attention of layer-list decoders over per-head key / value planes of the page pool
// ([page][kv_head][page_size][D | Dv], bf16 or fp32): rotation + unit normalisation + cache write of a step's tokens, and the
// attention of every token of a step — single decoded tokens and prompt portions alike — under a sliding-window, block
// ("chunk") or causal mask, optionally with one extra unit in the softmax denominator and a sigmoid gate per head.
// Softmax, normalisation and every sum are fp32; rotation angles are formed and reduced to one turn in double precision
// (position * frequency loses bits that matter at positions in the thousands), once per step in a cos / sin table.  Summation orders are fixed per output element: a position's result does
// not depend on what else the step carries.
#include <math.h>

#include <algorithm>

#include "kernels.h"
#include "launch.h"
#include "stack_common.cuh"

namespace hb {
namespace {

// One warp per run of kPrepUnits (token, head) units — query heads, then key heads (a key head's unit also writes the value
// row).  Warps are independent (no block-wide phase) and issue the loads of all their units before they work on the first,
// so an SM keeps hundreds of rows in flight.  Cosines and sines come from the step's table (stack_rope_table).
constexpr int kPrepWarps = 8;
constexpr int kPrepUnits = 4;

template <typename CT>
__global__ void __launch_bounds__(kPrepWarps * 32) gqa_prep_kernel(GqaPrepArgs a) {
  extern __shared__ float sm[];
  const int half = a.rope_dims / 2, Dp = (a.D + 3) / 4 * 4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_tok = a.H + a.G;
  const long total = (long)a.T * per_tok;
  const long unit0 = ((long)blockIdx.x * kPrepWarps + warp) * kPrepUnits;
  if (unit0 >= total) return;
  float* bufs = sm + (size_t)warp * kPrepUnits * Dp;
  // 16-byte loads when every head row starts on a 16-byte boundary
  const bool vec = (a.D & 3) == 0 && (a.ldp & 3) == 0 && (a.q_off & 3) == 0 && (a.k_off & 3) == 0 && ((uintptr_t)a.p & 15) == 0;
#pragma unroll
  for (int k = 0; k < kPrepUnits; ++k) {
    const long unit = unit0 + k;
    if (unit >= total) break;
    const int t = (int)(unit / per_tok), u = (int)(unit % per_tok);
    const float* src = a.p + (size_t)t * a.ldp + (u < a.H ? a.q_off + (size_t)u * a.D : a.k_off + (size_t)(u - a.H) * a.D);
    float* buf = bufs + k * Dp;
    if (vec) {
      for (int i = lane * 4; i < a.D; i += 128) *reinterpret_cast<float4*>(buf + i) = *reinterpret_cast<const float4*>(src + i);
    } else {
      for (int i = lane; i < a.D; i += 32) buf[i] = src[i];
    }
  }
  __syncwarp();
  for (int k = 0; k < kPrepUnits; ++k) {
    const long unit = unit0 + k;
    if (unit >= total) break;
    const int t = (int)(unit / per_tok), u = (int)(unit % per_tok);
    const int slot = a.slots ? a.slots[t] : -1;
    const size_t page = slot >= 0 ? slot / a.page_size : 0, off = slot >= 0 ? slot % a.page_size : 0;
    const bool isq = u < a.H;
    const int head = isq ? u : u - a.H;
    float* buf = bufs + k * Dp;
    if (!isq && slot >= 0) {  // values leave the projection untouched
      const float* vsrc = a.v_off == a.k_off && a.Dv == a.D ? buf : a.p + (size_t)t * a.ldp + a.v_off + (size_t)head * a.Dv;
      CT* vrow = (CT*)a.v_cache + ((page * a.G + head) * a.page_size + off) * a.Dv;
      for (int i = lane; i < a.Dv; i += 32) stf<CT>(vrow, i, vsrc[i]);
      __syncwarp();
    }
    for (int i = lane; i < half; i += 32) {
      const float2 sc2 = *reinterpret_cast<const float2*>(a.cs + (size_t)t * a.rope_dims + 2 * i);
      const float c = sc2.x, s = sc2.y;
      const int i0 = a.pairing ? 2 * i : i, i1 = a.pairing ? 2 * i + 1 : i + half;
      const float x = buf[i0], y = buf[i1];
      buf[i0] = x * c - y * s;
      buf[i1] = y * c + x * s;
    }
    __syncwarp();
    float rs = 1.f;
    if (a.unit_norm) {
      float ss = 0.f;
      for (int i = lane; i < a.D; i += 32) ss += buf[i] * buf[i];
      ss = warp_sum(ss);
      rs = 1.f / sqrtf(ss / (float)a.D + a.eps);
    }
    if (isq) {
      float* dst = a.q ? a.q + (size_t)t * a.ldq + (size_t)head * a.D : nullptr;
      bf16* dstb = a.q_b16 ? a.q_b16 + (size_t)t * a.ldq + (size_t)head * a.D : nullptr;
      for (int i = lane; i < a.D; i += 32) {
        const float v = buf[i] * rs;
        if (dst) dst[i] = v;
        if (dstb) dstb[i] = __float2bfloat16(v);
      }
    } else if (slot >= 0) {
      CT* row = (CT*)a.k_cache + ((page * a.G + head) * a.page_size + off) * a.D;
      for (int i = lane; i < a.D; i += 32) stf<CT>(row, i, buf[i] * rs);
    }
  }
}

// The same step for the common layouts — head rows that start on 16-byte boundaries; neighbouring pairs (2i, 2i+1), or halves
// (i, i + dims/2) with dims a multiple of 8 and at most 128; values that are the keys, or value rows of their own (one more
// unit per kv head that copies the row): a lane owns four consecutive entries of a head row in registers (with halves the
// partner entries come from the lane dims/8 away by shuffles); no shared memory, one 16-byte load and one 8- or 16-byte
// store per lane and row.  One warp per (token, head) unit; D, Dv <= 512.
template <typename CT>
__global__ void __launch_bounds__(256) gqa_prep_vec_kernel(GqaPrepArgs a) {
  const int lane = threadIdx.x & 31;
  const unsigned unit = blockIdx.x * 8u + (threadIdx.x >> 5);
  const bool sep_v = a.v_off != a.k_off;  // value rows of their own: units H + G .. H + 2G copy them into the cache
  const unsigned per_tok = a.H + a.G + (sep_v ? a.G : 0);
  if (unit >= (unsigned)a.T * per_tok) return;
  const int t = unit / per_tok, u = unit % per_tok;
  if (u >= a.H + a.G) {
    const int head = u - a.H - a.G, slot = a.slots ? a.slots[t] : -1;
    if (slot < 0) return;
    const float* vs = a.p + (size_t)t * a.ldp + a.v_off + (size_t)head * a.Dv;
    CT* vrow = (CT*)a.v_cache + (((size_t)(slot / a.page_size) * a.G + head) * a.page_size + slot % a.page_size) * a.Dv;
    for (int e = 4 * lane; e < a.Dv; e += 128) {
      const float4 x = *reinterpret_cast<const float4*>(vs + e);
      if (sizeof(CT) == 4) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(vrow) + e) = x;
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
        uint2 pk;
        pk.x = *reinterpret_cast<unsigned*>(&lo);
        pk.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(vrow) + e) = pk;
      }
    }
    return;
  }
  const bool isq = u < a.H;
  const int head = isq ? u : u - a.H;
  const int half = a.rope_dims / 2;
  const float* src = a.p + (size_t)t * a.ldp + (isq ? a.q_off : a.k_off) + (size_t)head * a.D;
  float4 v[4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = 4 * lane + 128 * j;
    v[j] = e < a.D ? *reinterpret_cast<const float4*>(src + e) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int slot = (!isq && a.slots) ? a.slots[t] : -1;
  const size_t rowi = slot >= 0 ? ((size_t)(slot / a.page_size) * a.G + head) * a.page_size + slot % a.page_size : 0;
  auto put16 = [](bf16* row, int e, const float4& x) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
    uint2 pk;
    pk.x = *reinterpret_cast<unsigned*>(&lo);
    pk.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(row + e) = pk;
  };
  auto put = [&](CT* row, int e, const float4& x) {
    if (sizeof(CT) == 4) *reinterpret_cast<float4*>(reinterpret_cast<float*>(row) + e) = x;
    else put16(reinterpret_cast<bf16*>(row), e, x);
  };
  if (slot >= 0 && !sep_v) {  // values: the key projection as it is
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = 4 * lane + 128 * j;
      if (e < a.D) put((CT*)a.v_cache + rowi * a.Dv, e, v[j]);
    }
  }
  if (a.pairing == 0 && half > 0) {
    // halves: the rotating entries lie in the first 128 of the row (v[0]); quad `lane` of the first half pairs with quad
    // lane + half / 4 of the second.  Every lane takes part in the shuffles.
    const int hq = half / 4;
    const bool first = lane < hq, second = lane >= hq && lane < 2 * hq;
    const int partner = first ? lane + hq : lane - hq;
    const float4 o = v[0];
    float4 pr;
    pr.x = __shfl_sync(0xffffffffu, o.x, partner & 31); pr.y = __shfl_sync(0xffffffffu, o.y, partner & 31);
    pr.z = __shfl_sync(0xffffffffu, o.z, partner & 31); pr.w = __shfl_sync(0xffffffffu, o.w, partner & 31);
    if (first || second) {
      const int qi = first ? lane : lane - hq;  // angles 4 qi .. 4 qi + 3
      const float4 c0 = *reinterpret_cast<const float4*>(a.cs + (size_t)t * a.rope_dims + 8 * qi);      // cos, sin, cos, sin
      const float4 c1 = *reinterpret_cast<const float4*>(a.cs + (size_t)t * a.rope_dims + 8 * qi + 4);
      if (first) {  // x cos - y sin, y = the partner's entries
        v[0] = make_float4(o.x * c0.x - pr.x * c0.y, o.y * c0.z - pr.y * c0.w, o.z * c1.x - pr.z * c1.y, o.w * c1.z - pr.w * c1.w);
      } else {      // y cos + x sin, x = the partner's entries
        v[0] = make_float4(o.x * c0.x + pr.x * c0.y, o.y * c0.z + pr.y * c0.w, o.z * c1.x + pr.z * c1.y, o.w * c1.z + pr.w * c1.w);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = 4 * lane + 128 * j;
    if (e < a.D && a.pairing == 1) {
      // the lane's two pairs are neighbours in the table: cos, sin, cos, sin (rope_dims is even; a 16-byte load when both rotate)
      float c4[4] = {1.f, 0.f, 1.f, 0.f};
      if (e / 2 + 1 < half) {
        const float4 tq = *reinterpret_cast<const float4*>(a.cs + (size_t)t * a.rope_dims + e);
        c4[0] = tq.x; c4[1] = tq.y; c4[2] = tq.z; c4[3] = tq.w;
      } else if (e / 2 < half) {
        const float2 tq = *reinterpret_cast<const float2*>(a.cs + (size_t)t * a.rope_dims + e);
        c4[0] = tq.x; c4[1] = tq.y;
      }
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int pr = e / 2 + h2;
        if (pr < half) {
          const float cs = c4[2 * h2], sn = c4[2 * h2 + 1];
          float& x = h2 ? v[j].z : v[j].x;
          float& y = h2 ? v[j].w : v[j].y;
          const float x0 = x, y0 = y;
          x = x0 * cs - y0 * sn;
          y = y0 * cs + x0 * sn;
        }
      }
    }
    if (e < a.D) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  }
  float rs = 1.f;
  if (a.unit_norm) rs = 1.f / sqrtf(warp_sum(ss) / (float)a.D + a.eps);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = 4 * lane + 128 * j;
    if (e >= a.D) continue;
    const float4 o = make_float4(v[j].x * rs, v[j].y * rs, v[j].z * rs, v[j].w * rs);
    if (isq) {
      const size_t at = (size_t)t * a.ldq + (size_t)head * a.D;
      if (a.q) *reinterpret_cast<float4*>(a.q + at + e) = o;
      if (a.q_b16) put16(a.q_b16 + at, e, o);
    } else if (slot >= 0) {
      put((CT*)a.k_cache + rowi * a.D, e, o);
    }
  }
}

// One block per token, for the options the warp-per-head kernels do not take: projection biases, a norm over the whole q (and
// k) projection with a gain per entry, values blended with an earlier layer's.  Order: bias, rotation, norm.
// dynamic smem: the token's q | k rows [(H + G) * D] + per-head factors [H + G]
template <typename CT>
__global__ void __launch_bounds__(256) gqa_prep_token_kernel(GqaPrepArgs a) {
  extern __shared__ __align__(16) float sm[];
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int nq = a.H * a.D, nk = a.G * a.D, nv = a.G * a.Dv;
  float* rsh = sm + nq + nk;
  const float* pr = a.p + (size_t)t * a.ldp;
  const CT* bias = (const CT*)a.bias;
  // 16-byte pieces when q, k and v rows start on 16-byte boundaries and the sizes are multiples of four
  const bool vec = ((nq | nk | nv | a.D | a.Dv | (int)a.ldp | a.q_off | a.k_off | a.v_off | (int)a.ldq) & 3) == 0 && ((uintptr_t)a.p & 15) == 0 &&
                   ((uintptr_t)a.q & 15) == 0 && ((uintptr_t)a.q_b16 & 7) == 0 && ((uintptr_t)a.v_first & 15) == 0 &&
                   ((uintptr_t)a.k_cache & 15) == 0 && ((uintptr_t)a.v_cache & 15) == 0;
  if (vec) {
    for (int i = threadIdx.x * 4; i < nq + nk; i += blockDim.x * 4) {
      const int col = i < nq ? a.q_off + i : a.k_off + (i - nq);
      float4 v = *reinterpret_cast<const float4*>(pr + col);
      if (bias) { v.x += ldf<CT>(bias, col); v.y += ldf<CT>(bias, col + 1); v.z += ldf<CT>(bias, col + 2); v.w += ldf<CT>(bias, col + 3); }
      *reinterpret_cast<float4*>(sm + i) = v;
    }
  } else {
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
      const int col = i < nq ? a.q_off + i : a.k_off + (i - nq);
      sm[i] = pr[col] + (bias ? ldf<CT>(bias, col) : 0.f);
    }
  }
  __syncthreads();
  const int half = a.rope_dims / 2;
  if (half > 0) {
    for (int u = threadIdx.x; u < (a.H + a.G) * half; u += blockDim.x) {
      const int head = u / half, i = u % half;
      const float2 cs = *reinterpret_cast<const float2*>(a.cs + (size_t)t * a.rope_dims + 2 * i);
      float* hp = sm + (size_t)head * a.D;
      const int i0 = a.pairing ? 2 * i : i, i1 = a.pairing ? 2 * i + 1 : i + half;
      const float x = hp[i0], y = hp[i1];
      hp[i0] = x * cs.x - y * cs.y;
      hp[i1] = y * cs.x + x * cs.y;
    }
    __syncthreads();
  }
  float rq = 1.f, rk = 1.f;
  if (a.proj_norm) {
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) sq = fmaf(sm[i], sm[i], sq);
    for (int i = threadIdx.x; i < nk; i += blockDim.x) sk = fmaf(sm[nq + i], sm[nq + i], sk);
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    rq = 1.f / sqrtf(sq / (float)nq + a.eps);
    rk = 1.f / sqrtf(sk / (float)nk + a.eps);
  } else if (a.unit_norm) {
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    for (int head = w; head < a.H + a.G; head += blockDim.x >> 5) {
      float ss = 0.f;
      for (int i = l; i < a.D; i += 32) ss = fmaf(sm[head * a.D + i], sm[head * a.D + i], ss);
      ss = warp_sum(ss);
      if (l == 0) rsh[head] = 1.f / sqrtf(ss / (float)a.D + a.eps);
    }
    __syncthreads();
  }
  const CT* gain = (const CT*)a.qk_gain;
  const int slot = a.slots ? a.slots[t] : -1;
  const size_t page = slot >= 0 ? slot / a.page_size : 0, off = slot >= 0 ? slot % a.page_size : 0;
  const float lam = a.blend_role == 2 ? ldf<CT>((const CT*)a.vmix, 0) : 0.f;
  auto put4 = [](CT* dst, const float4& x) {  // four neighbouring cache / weight-typed elements
    if (sizeof(CT) == 4) {
      *reinterpret_cast<float4*>(dst) = x;
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
      uint2 pk;
      pk.x = *reinterpret_cast<unsigned*>(&lo);
      pk.y = *reinterpret_cast<unsigned*>(&hi);
      *reinterpret_cast<uint2*>(dst) = pk;
    }
  };
  if (vec) {
    for (int i = threadIdx.x * 4; i < nq + nk; i += blockDim.x * 4) {
      const bool isq = i < nq;
      const int head = isq ? i / a.D : a.H + (i - nq) / a.D;
      float4 v = *reinterpret_cast<const float4*>(sm + i);
      if (a.proj_norm) {
        const float r = isq ? rq : rk;
        v.x *= r * ldf<CT>(gain, i); v.y *= r * ldf<CT>(gain, i + 1); v.z *= r * ldf<CT>(gain, i + 2); v.w *= r * ldf<CT>(gain, i + 3);
      } else if (a.unit_norm) {
        const float r = rsh[head];
        v.x *= r; v.y *= r; v.z *= r; v.w *= r;
      }
      if (isq) {
        if (a.q) *reinterpret_cast<float4*>(a.q + (size_t)t * a.ldq + i) = v;
        if (a.q_b16) {
          __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
          uint2 pk;
          pk.x = *reinterpret_cast<unsigned*>(&lo);
          pk.y = *reinterpret_cast<unsigned*>(&hi);
          *reinterpret_cast<uint2*>(a.q_b16 + (size_t)t * a.ldq + i) = pk;
        }
      } else if (slot >= 0) {
        const int kh = head - a.H, e = (i - nq) % a.D;
        put4((CT*)a.k_cache + ((page * a.G + kh) * a.page_size + off) * a.D + e, v);
      }
    }
    for (int i = threadIdx.x * 4; i < nv; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(pr + a.v_off + i);
      if (bias) { v.x += ldf<CT>(bias, a.v_off + i); v.y += ldf<CT>(bias, a.v_off + i + 1); v.z += ldf<CT>(bias, a.v_off + i + 2); v.w += ldf<CT>(bias, a.v_off + i + 3); }
      if (a.blend_role == 1) {
        *reinterpret_cast<float4*>(a.v_first + (size_t)t * nv + i) = v;
      } else if (a.blend_role == 2) {
        const float4 f = *reinterpret_cast<const float4*>(a.v_first + (size_t)t * nv + i);
        v.x = (1.f - lam) * v.x + lam * f.x; v.y = (1.f - lam) * v.y + lam * f.y;
        v.z = (1.f - lam) * v.z + lam * f.z; v.w = (1.f - lam) * v.w + lam * f.w;
      }
      if (slot >= 0) put4((CT*)a.v_cache + ((page * a.G + i / a.Dv) * a.page_size + off) * a.Dv + i % a.Dv, v);
    }
    return;
  }
  for (int i = threadIdx.x; i < nq; i += blockDim.x) {
    const float v = sm[i] * (a.proj_norm ? rq * ldf<CT>(gain, i) : (a.unit_norm ? rsh[i / a.D] : 1.f));
    if (a.q) a.q[(size_t)t * a.ldq + i] = v;
    if (a.q_b16) a.q_b16[(size_t)t * a.ldq + i] = __float2bfloat16(v);
  }
  if (slot >= 0) {
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
      const int head = i / a.D;
      const float v = sm[nq + i] * (a.proj_norm ? rk * ldf<CT>(gain, nq + i) : (a.unit_norm ? rsh[a.H + head] : 1.f));
      stf<CT>((CT*)a.k_cache, ((page * a.G + head) * a.page_size + off) * a.D + i % a.D, v);
    }
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float v = pr[a.v_off + i] + (bias ? ldf<CT>(bias, a.v_off + i) : 0.f);
    if (a.blend_role == 1) a.v_first[(size_t)t * nv + i] = v;
    else if (a.blend_role == 2) v = (1.f - lam) * v + lam * a.v_first[(size_t)t * nv + i];
    if (slot >= 0) stf<CT>((CT*)a.v_cache, ((page * a.G + i / a.Dv) * a.page_size + off) * a.Dv + i % a.Dv, v);
  }
}

// One block per (token, kv head, group of up to kHG of its query heads): the heads of a group read the same key and value
// rows, so one pass over them serves the group.
//   scores:       one warp per key, lanes stride the row, HG dot products per loaded row
//   softmax:      fp32, the optional unit of the denominator enters as a key of score 0 without a value
//   weighted sum: thread (slice, column) adds the keys of its slice for all HG heads; slices are added in slice order
// dynamic smem (floats): q [HG][Dp] | scores [max_keys][HG] | partials [threads][HG] | red [32 * HG] | row index [max_keys]
constexpr int kAttThreads = 512;
constexpr int kHG = 4;

template <typename CT>
__global__ void __launch_bounds__(kAttThreads) gqa_attn_kernel(GqaAttnArgs a, int max_keys) {
  constexpr int HG = kHG;
  extern __shared__ float sm[];
  const int D = a.D, Dv = a.Dv, Dp = (D + 3) / 4 * 4;
  float* qs = sm;
  float* sc = qs + HG * Dp;
  float* part = sc + (size_t)HG * max_keys;
  float* red = part + HG * blockDim.x;
  int* rowoff = reinterpret_cast<int*>(red + 32 * HG);
  const int rep = a.H / a.G, parts = (rep + HG - 1) / HG;
  const int t = blockIdx.x, g = blockIdx.y / parts, h0 = g * rep + (blockIdx.y % parts) * HG;
  const int nh = min(HG, g * rep + rep - h0);
  const int pos = a.positions[t];
  int j0 = 0;
  if (a.mask == MASK_CHUNK) j0 = pos / a.window * a.window;
  else if (a.mask == MASK_WINDOW) j0 = max(0, pos - a.window + 1);
  const int n = pos - j0 + 1;  // keys j0 .. pos (the host sized max_keys for the longest run any position can see)
  const int32_t* pt = a.page_table + (size_t)a.seq_of[t] * a.max_pages;
  for (int e = threadIdx.x; e < HG * Dp; e += blockDim.x) {
    const int hh = e / Dp, i = e % Dp;
    qs[e] = (hh < nh && i < D) ? a.q[(size_t)t * a.ldq + (size_t)(h0 + hh) * D + i] : 0.f;
  }
  for (int jj = threadIdx.x; jj < n; jj += blockDim.x) {
    const int j = j0 + jj;
    rowoff[jj] = (pt[j / a.page_size] * a.G + g) * a.page_size + j % a.page_size;
  }
  __syncthreads();
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  const CT* kc = (const CT*)a.k_cache;
  const CT* vc = (const CT*)a.v_cache;
  const float cap = a.softcap, icap = cap > 0.f ? 1.f / cap : 0.f;
  auto fin = [&](float sdot) {  // scale, then the optional tanh cap
    const float v = sdot * a.scale;
    return cap > 0.f ? cap * tanhf(v * icap) : v;
  };
  const int lpk = D / 8;  // lanes that cover one bf16 key row with one 16-byte load each
  if (sizeof(CT) == 2 && (D & 7) == 0 && (lpk == 4 || lpk == 8 || lpk == 16 || lpk == 32)) {
    // several keys per warp iteration: sub-warp `sub` of lpk lanes takes key base + sub; partial dot products are added
    // inside the sub-warp by a butterfly, so a key's sum does not depend on which sub-warp took it
    const int kpw = 32 / lpk, sub = l / lpk, li = l % lpk;
    for (int base = w * kpw; base < n; base += nw * kpw) {
      const int jj = base + sub;
      const bool live = jj < n;
      const bf16* row = reinterpret_cast<const bf16*>(kc) + (size_t)rowoff[live ? jj : n - 1] * D;
      const uint4 u = *reinterpret_cast<const uint4*>(row + li * 8);
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&u);
      float s[HG] = {};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p2[e]);
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) {
          const float2 q = *reinterpret_cast<const float2*>(qs + hh * Dp + li * 8 + 2 * e);
          s[hh] = fmaf(q.x, f.x, s[hh]);
          s[hh] = fmaf(q.y, f.y, s[hh]);
        }
      }
      for (int o = lpk >> 1; o > 0; o >>= 1) {
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) s[hh] += __shfl_xor_sync(0xffffffffu, s[hh], o);
      }
      if (live && li == 0) {
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) sc[jj * HG + hh] = fin(s[hh]);
      }
    }
  } else if (sizeof(CT) == 2 && (D & 7) == 0) {
    // bf16 rows that start on 16-byte boundaries: a lane takes 8 consecutive entries per load
    for (int jj = w; jj < n; jj += nw) {
      const bf16* row = reinterpret_cast<const bf16*>(kc) + (size_t)rowoff[jj] * D;
      float s[HG] = {};
      for (int i = l * 8; i < D; i += 256) {
        const uint4 u = *reinterpret_cast<const uint4*>(row + i);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(p2[e]);
#pragma unroll
          for (int hh = 0; hh < HG; ++hh) {
            const float2 q = *reinterpret_cast<const float2*>(qs + hh * Dp + i + 2 * e);
            s[hh] = fmaf(q.x, f.x, s[hh]);
            s[hh] = fmaf(q.y, f.y, s[hh]);
          }
        }
      }
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) s[hh] = warp_sum(s[hh]);
      if (l == 0) {
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) sc[jj * HG + hh] = fin(s[hh]);
      }
    }
  } else {
    for (int jj = w; jj < n; jj += nw) {
      const CT* row = kc + (size_t)rowoff[jj] * D;
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
        for (int hh = 0; hh < HG; ++hh) sc[jj * HG + hh] = fin(s[hh]);
      }
    }
  }
  __syncthreads();
  float mx[HG], inv[HG], snk[HG];
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) {  // a sink is a key without a value: the unit's score is 0, a learned one's is stored per head
    snk[hh] = a.sink ? ldf<CT>((const CT*)a.sink, h0 + (hh < nh ? hh : 0)) : (a.unit_sink ? 0.f : -INFINITY);
    mx[hh] = snk[hh];
  }
  for (int jj = threadIdx.x; jj < n; jj += blockDim.x) {
    const float4 v = *reinterpret_cast<const float4*>(sc + jj * HG);
    mx[0] = fmaxf(mx[0], v.x); mx[1] = fmaxf(mx[1], v.y); mx[2] = fmaxf(mx[2], v.z); mx[3] = fmaxf(mx[3], v.w);
  }
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) mx[hh] = warp_max(mx[hh]);
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
  for (int hh = 0; hh < HG; ++hh) {
    const float tot = warp_sum(l < nw ? red[l * HG + hh] : 0.f) + ((a.unit_sink || a.sink) ? expf(snk[hh] - mx[hh]) : 0.f);
    float gate = 1.f;
    if (a.gate && hh < nh) gate = sigmoidf_(a.gate[(size_t)t * a.ldg + h0 + hh]);
    inv[hh] = gate / tot;
  }
  const int ncg = Dv / 16;  // groups of 16 value columns (one 32-byte piece of a bf16 row)
  if (sizeof(CT) == 2 && (Dv & 15) == 0 && ncg <= nw) {
    // warp (column group cg, half): its 32 lanes take every (32 * halves)-th key and keep 16 columns x HG heads in registers;
    // lanes are added by a butterfly, halves in order through shared memory
    const int halves = nw / ncg, cg = w % ncg, half = w / ncg, NSv = halves * 32;
    float acc[HG][16] = {};
    if (half < halves) {
      for (int jj = half * 32 + l; jj < n; jj += NSv) {
        const uint4* vrow = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(vc) + (size_t)rowoff[jj] * Dv + cg * 16);
        const uint4 u0 = vrow[0], u1 = vrow[1];
        const float4 p = *reinterpret_cast<const float4*>(sc + jj * HG);
        const float pw[HG] = {p.x, p.y, p.z, p.w};
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&u0);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&u1);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fa = __bfloat1622float2(a2[e]), fb = __bfloat1622float2(b2[e]);
#pragma unroll
          for (int hh = 0; hh < HG; ++hh) {
            acc[hh][2 * e] = fmaf(pw[hh], fa.x, acc[hh][2 * e]);
            acc[hh][2 * e + 1] = fmaf(pw[hh], fa.y, acc[hh][2 * e + 1]);
            acc[hh][8 + 2 * e] = fmaf(pw[hh], fb.x, acc[hh][8 + 2 * e]);
            acc[hh][8 + 2 * e + 1] = fmaf(pw[hh], fb.y, acc[hh][8 + 2 * e + 1]);
          }
        }
      }
#pragma unroll
      for (int hh = 0; hh < HG; ++hh)
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float v = warp_sum(acc[hh][e]);
          if (l == e) part[((size_t)half * Dv + cg * 16 + e) * HG + hh] = v;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < Dv * HG; e += blockDim.x) {
      const int r = e / HG, hh = e % HG;
      if (hh >= nh) continue;
      float tot = 0.f;
      for (int hf = 0; hf < halves; ++hf) tot += part[((size_t)hf * Dv + r) * HG + hh];
      const size_t o = (size_t)t * a.ldo + (size_t)(h0 + hh) * Dv + r;
      const float v = tot * inv[hh];
      a.out[o] = v;
      if (a.out_b16) a.out_b16[o] = __float2bfloat16(v);
    }
    return;
  }
  const int Rp = (Dv + 31) / 32 * 32;
  const int NS = max(1, (int)blockDim.x / Rp);  // key slices
  for (int r0 = 0; r0 < Dv; r0 += blockDim.x) {  // one pass unless a value row is wider than the block
    const int sl = (NS > 1) ? threadIdx.x / Rp : 0, r = r0 + ((NS > 1) ? threadIdx.x % Rp : threadIdx.x);
    float acc[HG] = {};
    if (sl < NS && r < Dv) {
      const CT* col = vc + r;
      int jj = sl;
      for (; jj + NS < n; jj += 2 * NS) {  // two independent loads in flight; the sum keeps key order
        const float c0 = ldf<CT>(col, (size_t)rowoff[jj] * Dv), c1 = ldf<CT>(col, (size_t)rowoff[jj + NS] * Dv);
        const float4 p0 = *reinterpret_cast<const float4*>(sc + jj * HG), p1 = *reinterpret_cast<const float4*>(sc + (jj + NS) * HG);
        acc[0] = fmaf(p0.x, c0, acc[0]); acc[1] = fmaf(p0.y, c0, acc[1]); acc[2] = fmaf(p0.z, c0, acc[2]); acc[3] = fmaf(p0.w, c0, acc[3]);
        acc[0] = fmaf(p1.x, c1, acc[0]); acc[1] = fmaf(p1.y, c1, acc[1]); acc[2] = fmaf(p1.z, c1, acc[2]); acc[3] = fmaf(p1.w, c1, acc[3]);
      }
      for (; jj < n; jj += NS) {
        const float c0 = ldf<CT>(col, (size_t)rowoff[jj] * Dv);
        const float4 p0 = *reinterpret_cast<const float4*>(sc + jj * HG);
        acc[0] = fmaf(p0.x, c0, acc[0]); acc[1] = fmaf(p0.y, c0, acc[1]); acc[2] = fmaf(p0.z, c0, acc[2]); acc[3] = fmaf(p0.w, c0, acc[3]);
      }
    }
    if (NS > 1) {
      __syncthreads();
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) part[threadIdx.x * HG + hh] = acc[hh];
      __syncthreads();
      if (threadIdx.x < Dv) {
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) {
          float tot = 0.f;
          for (int ss = 0; ss < NS; ++ss) tot += part[(ss * Rp + threadIdx.x) * HG + hh];
          if (hh < nh) {
            const size_t o = (size_t)t * a.ldo + (size_t)(h0 + hh) * Dv + threadIdx.x;
            const float v = tot * inv[hh];
            a.out[o] = v;
            if (a.out_b16) a.out_b16[o] = __float2bfloat16(v);
          }
        }
      }
    } else if (r < Dv) {
#pragma unroll
      for (int hh = 0; hh < HG; ++hh)
        if (hh < nh) {
          const size_t o = (size_t)t * a.ldo + (size_t)(h0 + hh) * Dv + r;
          const float v = acc[hh] * inv[hh];
          a.out[o] = v;
          if (a.out_b16) a.out_b16[o] = __float2bfloat16(v);
        }
    }
  }
}

__global__ void head_gate_kernel(const bf16* __restrict__ o, long ldo, const float* __restrict__ gate, long ldg, float* __restrict__ out,
                                 bf16* __restrict__ outb, int H, int Dv) {
  const size_t t = blockIdx.x;
  for (int e = threadIdx.x; e < H * Dv; e += blockDim.x) {
    const float g = gate ? sigmoidf_(gate[t * ldg + e / Dv]) : 1.f;
    const float v = __bfloat162float(o[t * ldo + e]) * g;
    out[t * H * Dv + e] = v;
    if (outb) outb[t * H * Dv + e] = __float2bfloat16(v);
  }
}

__global__ void rope_table_kernel(const int32_t* __restrict__ positions, const double* __restrict__ freqs, int half,
                                  float* __restrict__ cs, int T) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)T * half) return;
  const int t = (int)(idx / half), i = (int)(idx % half);
  const double ang = (double)positions[t] * freqs[i];
  const double red = fma(-6.283185307179586476925, rint(ang * 0.15915494309189533577), ang);
  float s, c;
  sincosf((float)red, &s, &c);
  *reinterpret_cast<float2*>(cs + 2 * idx) = make_float2(c, s);
}

}  // namespace

cudaError_t stack_rope_table(cudaStream_t s, const int32_t* positions, const double* freqs, int half, float* cs, int T) {
  if (T <= 0 || half <= 0) return cudaSuccess;
  rope_table_kernel<<<(unsigned)(((long)T * half + 255) / 256), 256, 0, s>>>(positions, freqs, half, cs, T);
  return cudaGetLastError();
}

cudaError_t head_gate_rows(cudaStream_t s, const bf16* o, long ldo, const float* gate, long ldg, float* out, bf16* outb, int T, int H,
                           int Dv) {
  if (T <= 0) return cudaSuccess;
  head_gate_kernel<<<T, 256, 0, s>>>(o, ldo, gate, ldg, out, outb, H, Dv);
  return cudaGetLastError();
}

size_t gqa_attn_smem(int D, int Dv, int max_keys) {
  (void)Dv;
  return ((size_t)kHG * ((D + 3) / 4 * 4) + (size_t)(kHG + 1) * max_keys + (size_t)kHG * kAttThreads + 32 * kHG) * 4;
}

cudaError_t stack_gqa_init() {
  cudaError_t e;
  const int big = 200 * 1024;
  if ((e = cudaFuncSetAttribute(gqa_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, big)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(gqa_attn_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, big)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(gqa_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(gqa_prep_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(gqa_prep_token_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(gqa_prep_token_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)) != cudaSuccess) return e;
  return cudaSuccess;
}

cudaError_t gqa_prep(cudaStream_t s, const GqaPrepArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  if (a.rope_dims % 2 || a.rope_dims > a.D || (a.rope_dims > 0 && !a.cs)) return cudaErrorInvalidValue;
  if (a.bias || a.proj_norm || a.blend_role) {
    if ((a.proj_norm && !a.qk_gain) || (a.blend_role && !a.v_first) || (a.blend_role == 2 && !a.vmix)) return cudaErrorInvalidValue;
    const size_t smem = ((size_t)(a.H + a.G) * a.D + a.H + a.G) * 4;
    if (smem > 100 * 1024) return cudaErrorInvalidValue;
    if (a.f32) gqa_prep_token_kernel<float><<<a.T, 256, smem, s>>>(a);
    else gqa_prep_token_kernel<bf16><<<a.T, 256, smem, s>>>(a);
    return cudaGetLastError();
  }
  const bool aligned = (a.D & 3) == 0 && a.D <= 512 && (a.ldp & 3) == 0 && (a.q_off & 3) == 0 && (a.k_off & 3) == 0 && (a.ldq & 3) == 0 &&
                       ((uintptr_t)a.p & 15) == 0 && ((uintptr_t)a.q & 15) == 0 && ((uintptr_t)a.q_b16 & 7) == 0 &&
                       ((uintptr_t)a.k_cache & 15) == 0 && ((uintptr_t)a.v_cache & 15) == 0 && ((uintptr_t)a.cs & 15) == 0 &&
                       (a.rope_dims & 3) == 0;
  const bool own_v = a.v_off != a.k_off, v_ok = own_v ? ((a.Dv | a.v_off) & 3) == 0 && a.Dv <= 512 : a.Dv == a.D;
  const bool pairs_ok = a.pairing == 1 || a.rope_dims == 0 || (a.pairing == 0 && a.rope_dims % 8 == 0 && a.rope_dims <= 128);
  if (aligned && pairs_ok && v_ok) {
    const unsigned blocks = (unsigned)(((long)a.T * (a.H + a.G + (own_v ? a.G : 0)) + 7) / 8);
    if (a.f32) gqa_prep_vec_kernel<float><<<blocks, 256, 0, s>>>(a);
    else gqa_prep_vec_kernel<bf16><<<blocks, 256, 0, s>>>(a);
    return cudaGetLastError();
  }
  const size_t smem = (size_t)kPrepWarps * kPrepUnits * ((a.D + 3) / 4 * 4) * 4;
  if (smem > 72 * 1024) return cudaErrorInvalidValue;
  const long units = (long)a.T * (a.H + a.G);
  const unsigned grid = (unsigned)((units + kPrepWarps * kPrepUnits - 1) / (kPrepWarps * kPrepUnits));
  if (a.f32) gqa_prep_kernel<float><<<grid, kPrepWarps * 32, smem, s>>>(a);
  else gqa_prep_kernel<bf16><<<grid, kPrepWarps * 32, smem, s>>>(a);
  return cudaGetLastError();
}

cudaError_t gqa_attn(cudaStream_t s, const GqaAttnArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  if (a.G <= 0 || a.H % a.G || (a.mask != MASK_CAUSAL && a.window <= 0)) return cudaErrorInvalidValue;
  // the longest run of keys any position of a sequence can see: window / block length, never more than a sequence holds
  const int ctx = a.max_pages * a.page_size;
  int max_keys = a.mask == MASK_CAUSAL ? ctx : std::min(a.window, ctx);
  if (a.longest_ctx > 0) max_keys = std::min(max_keys, (a.longest_ctx + 255) / 256 * 256);  // sized by what this step's positions see
  const size_t smem = gqa_attn_smem(a.D, a.Dv, max_keys);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  const int rep = a.H / a.G;
  dim3 grid(a.T, a.G * ((rep + kHG - 1) / kHG));
  if (a.f32) gqa_attn_kernel<float><<<grid, kAttThreads, smem, s>>>(a, max_keys);
  else gqa_attn_kernel<bf16><<<grid, kAttThreads, smem, s>>>(a, max_keys);
  return cudaGetLastError();
}

}  // namespace hb
