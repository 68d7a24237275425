// Mixture-of-experts feed-forward of layer-list decoders (layerlist.cu).
//
//  * moe_route_kernel      one CTA per token: fp32 router logits over experts + identity slots (a warp per slice of the
//                          input's coordinates, eight slots at a time, slices summed in a fixed order), softmax, the choice
//                          scores (score + correction), group limitation (only slots of the `keep` groups with the
//                          largest best choice score stay eligible), the `top` largest choices (ties: lower slot),
//                          weights = scale * score.  Emits the chosen slots and weights, the dense [rows, E] weight
//                          table of the masked-dense path and the summed weight of the chosen identity slots.
//  * moe_act_mask_kernel   masked-dense path (many rows): the up projection of ALL experts is one GEMM of the shared
//                          projection kernels, this kernel turns it into relu(u)^2 * weight(row, expert) - zero for
//                          experts the row did not choose - and one GEMM over K = experts * ff sums the experts.
//  * moe_up_rows / moe_down_rows   few rows (decode): a warp per output reads only the chosen experts' rows.
//  * moe_identity_kernel   x += (weight of the chosen identity slots) * h
//  Router kind 1 (sigmoid scores, the largest win, weight = score, applied to the expert's INPUT) with gated experts
//  down(silu(w g) * (w u)) and a shared expert:
//  * moe_glu_act_kernel    masked-dense path: [rows, 2 F] interleaved (gate, up) of all experts and the shared one ->
//                          [rows, F] hidden values, zero where the row did not choose the expert
//  * moe_glu_up_rows / moe_glu_down_rows   few rows: only the chosen experts' and the shared expert's rows are read
#include "common.cuh"
#include "mixer.h"

namespace {

constexpr int MOE_MAX_SLOTS = 1024;

// w . v over K entries by one warp; rows of whole 16-byte vectors (aligned base) take vector loads, four in flight
template <typename WT>
__device__ __forceinline__ float warp_dot(const WT* __restrict__ w, const float* __restrict__ v, int K, int lane) {
  constexpr int VEC = Vec16<WT>::N;
  float acc = 0.f;
  if (K % VEC == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)v & 15) == 0) {
#pragma unroll 4
    for (int k = lane * VEC; k < K; k += 32 * VEC) {
      float f[VEC];
      Vec16<WT>::load(w + k, f);
#pragma unroll
      for (int x = 0; x < VEC; x += 4) {
        const float4 a = *reinterpret_cast<const float4*>(v + k + x);
        acc = fmaf(f[x], a.x, acc); acc = fmaf(f[x + 1], a.y, acc); acc = fmaf(f[x + 2], a.z, acc); acc = fmaf(f[x + 3], a.w, acc);
      }
    }
  } else {
#pragma unroll 4
    for (int k = lane; k < K; k += 32) acc = fmaf(to_f32(w[k]), v[k], acc);
  }
  return warp_sum(acc);
}


__global__ void __launch_bounds__(256) moe_route_kernel(MoeRouteArgs a) {
  __shared__ float s_score[MOE_MAX_SLOTS];   // logits, then softmax scores
  __shared__ float s_choice[MOE_MAX_SLOTS];  // score + correction; -inf once taken or out of the kept groups
  __shared__ float s_group[MOE_MAX_SLOTS];
  __shared__ float s_part[MOE_MAX_SLOTS * 8];  // [slot][warp] partial logits
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int n = a.E + a.I, D = a.D;
  const float* h = a.h + (size_t)r * D;
  // logits: every warp takes one slice of the input's coordinates for ALL slots (eight slots at a time, so that eight
  // independent weight loads are in flight per input load), the slices' partial sums meet in shared memory and are added
  // in slice order - the same arithmetic whatever the number of rows in the launch
  const int per_w = ((D + nw - 1) / nw + 3) & ~3;
  const int k_lo = min(D, warp * per_w), k_hi = min(D, k_lo + per_w);
  const bool vec4 = (D % 4 == 0) && (((uintptr_t)h & 15) == 0) && (((uintptr_t)a.router & 15) == 0);
  for (int e0 = 0; e0 < n; e0 += 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (vec4) {
      for (int k = k_lo + lane * 4; k < k_hi; k += 128) {
        const float4 hv = *reinterpret_cast<const float4*>(h + k);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (e0 + j < n) {
            const float4 wv = *reinterpret_cast<const float4*>(a.router + (size_t)(e0 + j) * D + k);
            acc[j] = fmaf(wv.x, hv.x, acc[j]); acc[j] = fmaf(wv.y, hv.y, acc[j]);
            acc[j] = fmaf(wv.z, hv.z, acc[j]); acc[j] = fmaf(wv.w, hv.w, acc[j]);
          }
      }
    } else {
      for (int k = k_lo + lane; k < k_hi; k += 32) {
        const float hv = h[k];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (e0 + j < n) acc[j] = fmaf(a.router[(size_t)(e0 + j) * D + k], hv, acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float t = warp_sum(acc[j]);
      if (lane == 0 && e0 + j < n) s_part[(e0 + j) * 8 + warp] = t;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    float t = 0.f;
    for (int w = 0; w < nw; ++w) t += s_part[e * 8 + w];
    s_score[e] = t;
  }
  __syncthreads();
  if (warp != 0) return;
  if (a.kind == 1) {  // independent sigmoid scores; the largest win
    for (int e = lane; e < n; e += 32) { const float sc = 1.0f / (1.0f + expf(-s_score[e])); s_score[e] = sc; s_choice[e] = sc; }
    __syncwarp();
  } else {
  float mx = -INFINITY;
  for (int e = lane; e < n; e += 32) mx = fmaxf(mx, s_score[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < n; e += 32) { const float p = expf(s_score[e] - mx); s_score[e] = p; sum += p; }
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
  for (int e = lane; e < n; e += 32) {
    const float sc = s_score[e] * inv;
    s_score[e] = sc;
    s_choice[e] = sc + a.correction[e];
  }
  __syncwarp();
  }
  const int per = n / a.groups;
  if (a.groups > 1 && a.keep < a.groups) {
    for (int g = lane; g < a.groups; g += 32) {
      float best = -INFINITY;
      for (int j = 0; j < per; ++j) best = fmaxf(best, s_choice[g * per + j]);
      s_group[g] = best;
    }
    __syncwarp();
    // the keep best groups get +inf as a mark, the others lose their slots
    for (int k = 0; k < a.keep; ++k) {
      float bv = -INFINITY; int bi = 0x7fffffff;
      for (int g = lane; g < a.groups; g += 32) {
        const float v = s_group[g];
        if (v != INFINITY && (bi == 0x7fffffff || v > bv)) { bv = v; bi = g; }
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(L3_FULL, bv, o);
        const int oi = __shfl_xor_sync(L3_FULL, bi, o);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
      }
      if (lane == 0 && bi != 0x7fffffff) s_group[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < n; e += 32)
      if (s_group[e / per] != INFINITY) s_choice[e] = -INFINITY;
    __syncwarp();
  }
  if (a.dense)
    for (int e = lane; e < a.E; e += 32) a.dense[(size_t)r * a.E + e] = 0.f;
  __syncwarp();
  float idw = 0.f;
  for (int k = 0; k < a.top; ++k) {
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < n; e += 32) {
      const float v = s_choice[e];
      if (v > bv) { bv = v; bi = e; }  // ascending e: the first of equal values stays
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(L3_FULL, bv, o);
      const int oi = __shfl_xor_sync(L3_FULL, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      // fewer eligible slots than `top`: the surplus picks get weight 0 on slot 0
      const bool ok = bi != 0x7fffffff;
      const int e = ok ? bi : 0;
      const float w = ok ? s_score[e] * a.scale : 0.f;
      a.sel[(size_t)r * a.top + k] = e;
      a.w[(size_t)r * a.top + k] = w;
      if (ok) {
        s_choice[e] = -INFINITY;
        if (e >= a.E) idw += w;
        else if (a.dense) a.dense[(size_t)r * a.E + e] = w;
      }
    }
    __syncwarp();
  }
  if (lane == 0) a.idw[r] = idw;
}

__global__ void moe_act_mask_kernel(float* __restrict__ u, const float* __restrict__ dense, int64_t n, int E, int ff,
                                    bf16* __restrict__ out16) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t width = (int64_t)E * ff;
  const int64_t r = i / width;
  const int e = (int)((i - r * width) / ff);
  const float w = dense[r * E + e];
  const float v = fmaxf(u[i], 0.f);
  const float o = w != 0.f ? v * v * w : 0.f;
  u[i] = o;
  if (out16) out16[i] = __float2bfloat16_rn(o);
}

__global__ void moe_identity_kernel(float* __restrict__ x, const float* __restrict__ h, const float* __restrict__ idw, int64_t n,
                                    int D) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float w = idw[i / D];
  if (w != 0.f) x[i] = fmaf(w, h[i], x[i]);
}

// grid (ceil(ff / 8), rows * top): hid[pair, j] = relu(up_e[j] . h[row])^2
template <typename WT>
__global__ void __launch_bounds__(256) moe_up_rows_kernel(const float* __restrict__ h, const WT* __restrict__ w_up,
                                                          const int32_t* __restrict__ sel, int D, int E, int ff, int top,
                                                          float* __restrict__ hid) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pair = blockIdx.y, j = blockIdx.x * 8 + warp;
  const int e = sel[pair];
  if (j >= ff || e >= E) return;
  const float d = warp_dot(w_up + ((size_t)e * ff + j) * D, h + (size_t)(pair / top) * D, D, lane);
  if (lane == 0) { const float v = fmaxf(d, 0.f); hid[(size_t)pair * ff + j] = v * v; }
}

// grid (ceil(D / 8), rows): x[row, i] += sum_k w_k down_e[i] . hid[pair_k] + idw[row] h[row, i]
template <typename WT>
__global__ void __launch_bounds__(256) moe_down_rows_kernel(const float* __restrict__ h, const WT* __restrict__ w_down,
                                                            const int32_t* __restrict__ sel, const float* __restrict__ w,
                                                            const float* __restrict__ idw, int D, int E, int ff, int top,
                                                            const float* __restrict__ hid, float* __restrict__ x) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.y, i = blockIdx.x * 8 + warp;
  if (i >= D) return;
  float acc = 0.f;
  for (int k = 0; k < top; ++k) {
    const int pair = row * top + k, e = sel[pair];
    if (e >= E) continue;
    acc = fmaf(w[pair], warp_dot(w_down + (size_t)i * E * ff + (size_t)e * ff, hid + (size_t)pair * ff, ff, lane), acc);
  }
  if (lane == 0) x[(size_t)row * D + i] += acc + idw[row] * h[(size_t)row * D + i];
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

__global__ void moe_glu_act_kernel(const float* __restrict__ gu, const float* __restrict__ dense, int64_t n, int E, int ff, int sff,
                                   float* __restrict__ hid, bf16* __restrict__ hid16) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t F = (int64_t)E * ff + sff;
  const int64_t r = i / F;
  const int64_t c = i - r * F;
  const float w = c < (int64_t)E * ff ? dense[r * E + c / ff] : 1.0f;
  float o = 0.f;
  if (w != 0.f) {
    const float2 p = *reinterpret_cast<const float2*>(gu + 2 * i);
    o = silu_f(w * p.x) * (w * p.y);
  }
  hid[i] = o;
  if (hid16) hid16[i] = __float2bfloat16_rn(o);
}

// grid (ceil(max(ff, sff) / 8), rows * (top + 1)): slot k < top of a row is its k-th chosen expert, slot top the shared expert
template <typename WT>
__global__ void __launch_bounds__(256) moe_glu_up_rows_kernel(const float* __restrict__ h, const WT* __restrict__ w_gu,
                                                              const int32_t* __restrict__ sel, const float* __restrict__ wsel,
                                                              int D, int E, int ff, int sff, int top, int hs,
                                                              float* __restrict__ hid) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slot = blockIdx.y, row = slot / (top + 1), k = slot - row * (top + 1);
  const int j = blockIdx.x * 8 + warp;
  const bool shared = k == top;
  const int e = shared ? E : sel[row * top + k];
  const int width = shared ? sff : ff;
  if (j >= width || e > E || (!shared && e >= E)) return;
  const float w = shared ? 1.0f : wsel[row * top + k];
  const WT* wr = w_gu + ((size_t)2 * ((size_t)e * ff + j)) * D;
  const float* hr = h + (size_t)row * D;
  const float g = warp_dot(wr, hr, D, lane), u = warp_dot(wr + D, hr, D, lane);
  if (lane == 0) hid[(size_t)slot * hs + j] = silu_f(w * g) * (w * u);
}

// grid (ceil(D / 8), rows): y[row, i] = sum over the row's slots of down_e[i] . hid[slot]
template <typename WT>
__global__ void __launch_bounds__(256) moe_glu_down_rows_kernel(const WT* __restrict__ w_down, const int32_t* __restrict__ sel,
                                                                int D, int E, int ff, int sff, int top, int hs,
                                                                const float* __restrict__ hid, float* __restrict__ y) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.y, i = blockIdx.x * 8 + warp;
  if (i >= D) return;
  const size_t F = (size_t)E * ff + sff;
  float acc = 0.f;
  for (int k = 0; k <= top; ++k) {
    const bool shared = k == top;
    if (shared && sff == 0) break;
    const int e = shared ? E : sel[row * top + k];
    if (!shared && e >= E) continue;
    acc += warp_dot(w_down + (size_t)i * F + (size_t)e * ff, hid + ((size_t)row * (top + 1) + k) * hs, shared ? sff : ff, lane);
  }
  if (lane == 0) y[(size_t)row * D + i] = acc;
}

}  // namespace

cudaError_t launch_moe_glu_act(const float* gu, const float* dense, int rows, int E, int ff, int sff, float* hid, bf16* hid16,
                               cudaStream_t s) {
  const int64_t n = (int64_t)rows * ((int64_t)E * ff + sff);
  return launch_k(moe_glu_act_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, gu, dense, n, E, ff, sff, hid, hid16);
}

cudaError_t launch_moe_glu_rows(const float* h, const void* w_gu, const void* w_down, bool w_bf16, const int32_t* sel,
                                const float* w, int rows, int D, int E, int ff, int sff, int top, float* hid, float* y,
                                cudaStream_t s) {
  const int hs = ff > sff ? ff : sff;
  const dim3 gu((hs + 7) / 8, rows * (top + 1)), gd((D + 7) / 8, rows);
  cudaError_t e;
  if (w_bf16) {
    e = launch_k(moe_glu_up_rows_kernel<bf16>, gu, dim3(256), 0, s, h, (const bf16*)w_gu, sel, w, D, E, ff, sff, top, hs, hid);
    if (e != cudaSuccess) return e;
    return launch_k(moe_glu_down_rows_kernel<bf16>, gd, dim3(256), 0, s, (const bf16*)w_down, sel, D, E, ff, sff, top, hs, (const float*)hid, y);
  }
  e = launch_k(moe_glu_up_rows_kernel<float>, gu, dim3(256), 0, s, h, (const float*)w_gu, sel, w, D, E, ff, sff, top, hs, hid);
  if (e != cudaSuccess) return e;
  return launch_k(moe_glu_down_rows_kernel<float>, gd, dim3(256), 0, s, (const float*)w_down, sel, D, E, ff, sff, top, hs, (const float*)hid, y);
}

cudaError_t launch_moe_route(const MoeRouteArgs& a, int rows, cudaStream_t s) {
  if (a.E + a.I > MOE_MAX_SLOTS || a.groups < 1 || (a.E + a.I) % a.groups) return cudaErrorInvalidValue;
  return launch_k(moe_route_kernel, dim3(rows), dim3(256), 0, s, a);
}

cudaError_t launch_moe_act_mask(float* u, const float* dense, int rows, int E, int ff, bf16* out16, cudaStream_t s) {
  const int64_t n = (int64_t)rows * E * ff;
  return launch_k(moe_act_mask_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, u, dense, n, E, ff, out16);
}

cudaError_t launch_moe_identity(float* x, const float* h, const float* idw, int rows, int D, cudaStream_t s) {
  const int64_t n = (int64_t)rows * D;
  return launch_k(moe_identity_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, x, h, idw, n, D);
}

cudaError_t launch_moe_rows(const float* h, const void* w_up, const void* w_down, bool w_bf16, const int32_t* sel,
                            const float* w, const float* idw, int rows, int D, int E, int ff, int top, float* hid, float* x,
                            cudaStream_t s) {
  cudaError_t e;
  const dim3 gu((ff + 7) / 8, rows * top), gd((D + 7) / 8, rows);
  if (w_bf16) {
    e = launch_k(moe_up_rows_kernel<bf16>, gu, dim3(256), 0, s, h, (const bf16*)w_up, sel, D, E, ff, top, hid);
    if (e != cudaSuccess) return e;
    return launch_k(moe_down_rows_kernel<bf16>, gd, dim3(256), 0, s, h, (const bf16*)w_down, sel, w, idw, D, E, ff, top,
                    (const float*)hid, x);
  }
  e = launch_k(moe_up_rows_kernel<float>, gu, dim3(256), 0, s, h, (const float*)w_up, sel, D, E, ff, top, hid);
  if (e != cudaSuccess) return e;
  return launch_k(moe_down_rows_kernel<float>, gd, dim3(256), 0, s, h, (const float*)w_down, sel, w, idw, D, E, ff, top,
                  (const float*)hid, x);
}
