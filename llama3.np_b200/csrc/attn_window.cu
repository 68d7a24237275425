// Sliding-window attention that may keep the first tokens (L3_MIX_WINDOW): GQA with key size DK and value size DV,
// the weight of a visible key either a softmax term whose denominator also holds a per-head sink, or sigmoid(score +
// per-head bias) without any normalisation over keys.  Everything fp32 (FFMA): scores, weights, accumulation.
//
//  * win_prep_kernel     a warp per head vector of a token: rotary turn of the leading rot_dims entries at the token's
//                        position (pairs (2i, 2i + 1) or (i, i + rot_dims / 2); angle = position * frequency in fp32,
//                        sincosf), optional division by the vector's root mean square, q to the query buffer, k and the
//                        value row to the caches
//  * win_attn_kernel     a CTA holds 32 query rows of ONE key head - row = (token, query head of the group), token-major,
//                        so the heads of a group share every key / value tile - and walks the keys the tile can see, 32 at
//                        a time: first the kept tokens that lie ahead of the window, then the window.  A warp owns 4 rows;
//                        in the score phase a lane is a key (16-byte shared loads, key rows padded by 4 floats), in the
//                        output phase a lane owns value columns lane, lane + 32, ...  Softmax rows run the online form,
//                        started at (max = sink, sum = 1) so that the sink needs no key; sigmoid rows just accumulate.
//                        Calls of few tokens split the key tiles over CTAs (win_attn_combine_kernel merges).
#include <algorithm>

#include "common.cuh"
#include "mixer.h"
#include "../../include/llama3_b200.h"

namespace {

constexpr int WA_ROWS = 32, WA_KEYS = 32, WA_WARPS = 8, WA_QW = WA_ROWS / WA_WARPS;

template <typename KVT>
__global__ void __launch_bounds__(256) win_prep_kernel(WinPrepArgs a) {
  extern __shared__ float sm[];  // [warps][DK]
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int b = r / a.L, t = r - b * a.L;
  const int pos = *a.pos_ptr + t;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float* row = a.proj + (size_t)r * a.ld;
  float* buf = sm + (size_t)warp * a.DK;
  const int half = a.rot_dims / 2;
  for (int v = warp; v < a.H + a.G; v += nw) {
    const bool is_q = v < a.H;
    const float* src = row + (is_q ? a.q_off + (size_t)v * a.DK : a.k_off + (size_t)(v - a.H) * a.DK);
    for (int i = lane; i < half; i += 32) {
      const int i0 = a.rot_layout ? i : 2 * i, i1 = a.rot_layout ? i + half : 2 * i + 1;
      float sn, cs;
      sincosf((float)pos * a.inv_freq[i], &sn, &cs);
      const float u = src[i0], w = src[i1];
      buf[i0] = u * cs - w * sn;
      buf[i1] = w * cs + u * sn;
    }
    for (int i = a.rot_dims + lane; i < a.DK; i += 32) buf[i] = src[i];
    __syncwarp();
    float mul = 1.0f;
    if (a.unit_norm) {
      float ss = 0.f;
      for (int i = lane; i < a.DK; i += 32) ss = fmaf(buf[i], buf[i], ss);
      mul = 1.0f / sqrtf(warp_sum(ss) / (float)a.DK + a.eps);
    }
    if (is_q) {
      float* dst = a.q_out + ((size_t)r * a.H + v) * a.DK;
      for (int i = lane; i < a.DK; i += 32) dst[i] = buf[i] * mul;
    } else {
      KVT* dst = (KVT*)a.cache_k + (((size_t)b * a.G + (v - a.H)) * a.M + pos) * a.DK;
      for (int i = lane; i < a.DK; i += 32) dst[i] = from_f32<KVT>(buf[i] * mul);
    }
    __syncwarp();
  }
  for (int i = threadIdx.x; i < a.G * a.DV; i += blockDim.x) {
    const int g = i / a.DV, d = i - g * a.DV;
    ((KVT*)a.cache_v)[(((size_t)b * a.G + g) * a.M + pos) * a.DV + d] = from_f32<KVT>(row[a.v_off + i]);
  }
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// NJ: value columns per lane (DV <= 32 NJ)
template <typename KVT, int NJ>
__global__ void __launch_bounds__(256) win_attn_kernel(WinAttnArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int DKP = (a.DK + 3) & ~3, KS = DKP + 4, DVP = 32 * NJ;
  float* sQ = sm;                                  // [32][DKP]
  float* sK = sQ + (size_t)WA_ROWS * DKP;          // [32][DKP + 4]
  float* sV = sK + (size_t)WA_KEYS * KS;           // [32][DVP]
  float* sP = sV + (size_t)WA_KEYS * DVP;          // [warps][QW][32]
  pdl_launch();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rep = a.H / a.G;
  const int g = blockIdx.y;
  const int b = blockIdx.z / a.nsplit, split = blockIdx.z - b * a.nsplit;
  const int nrows = a.L * rep;                     // rows of this (sequence, key head): row = t * rep + head in group
  const int row0 = blockIdx.x * WA_ROWS;
  const int pos0 = *a.pos_ptr;
  const int t_lo = row0 / rep, t_hi = min(a.L - 1, (row0 + WA_ROWS - 1) / rep);
  const int p_lo = pos0 + t_lo, p_hi = pos0 + t_hi;
  // keys the tile can see: [0, ka) kept tokens ahead of the window, then [w_lo, p_hi]
  const int w_lo = a.window > 0 ? max(0, p_lo - a.window + 1) : 0;
  const int ka = min(a.keep_first, w_lo);
  const int nkeys = ka + (p_hi + 1 - w_lo);
  const int ntiles = (nkeys + WA_KEYS - 1) / WA_KEYS;
  const int per = (ntiles + a.nsplit - 1) / a.nsplit;
  const int tile_lo = split * per, tile_hi = min(ntiles, tile_lo + per);

  // queries
  for (int idx = tid; idx < WA_ROWS * DKP; idx += 256) {
    const int rr = idx / DKP, d = idx - rr * DKP;
    const int row = row0 + rr;
    float v = 0.f;
    if (row < nrows && d < a.DK) {
      const int t = row / rep, h = g * rep + (row - t * rep);
      v = a.q[(((size_t)b * a.L + t) * a.H + h) * a.DK + d];
    }
    sQ[idx] = v;
  }
  // per-row state: rows warp, warp + 8, warp + 16, warp + 24 of the tile
  float o[WA_QW][NJ], mx[WA_QW], sum[WA_QW], hv[WA_QW];
  int rpos[WA_QW];
#pragma unroll
  for (int qi = 0; qi < WA_QW; ++qi) {
    const int row = row0 + warp + qi * WA_WARPS;
    const bool live = row < nrows;
    const int t = live ? row / rep : 0, h = g * rep + (live ? row - t * rep : 0);
    rpos[qi] = live ? pos0 + t : -1;
    hv[qi] = a.head_vec ? a.head_vec[h] : 0.f;
    const bool sink_here = a.kind == L3_ATTN_SINK && a.head_vec && split == 0;
    mx[qi] = sink_here ? hv[qi] : -INFINITY;
    sum[qi] = sink_here ? 1.f : 0.f;
#pragma unroll
    for (int j = 0; j < NJ; ++j) o[qi][j] = 0.f;
  }
  const KVT* ck = (const KVT*)a.cache_k + ((size_t)b * a.G + g) * a.M * a.DK;
  const KVT* cv = (const KVT*)a.cache_v + ((size_t)b * a.G + g) * a.M * a.DV;
  float* myP = sP + (size_t)warp * WA_QW * WA_KEYS;

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    __syncthreads();  // the previous tile has been used (and sQ is complete)
    const int v0 = tile * WA_KEYS;
    for (int idx = tid; idx < WA_KEYS * DKP; idx += 256) {
      const int kk = idx / DKP, d = idx - kk * DKP;
      const int vi = v0 + kk;
      float v = 0.f;
      if (vi < nkeys && d < a.DK) {
        const int j = vi < ka ? vi : w_lo + (vi - ka);
        v = to_f32(ck[(size_t)j * a.DK + d]);
      }
      sK[kk * KS + d] = v;
    }
    for (int idx = tid; idx < WA_KEYS * DVP; idx += 256) {
      const int kk = idx / DVP, d = idx - kk * DVP;
      const int vi = v0 + kk;
      float v = 0.f;
      if (vi < nkeys && d < a.DV) {
        const int j = vi < ka ? vi : w_lo + (vi - ka);
        v = to_f32(cv[(size_t)j * a.DV + d]);
      }
      sV[idx] = v;
    }
    __syncthreads();
    // scores: lane = key
    const int vi = v0 + lane;
    const int kj = vi < nkeys ? (vi < ka ? vi : w_lo + (vi - ka)) : -1;
    float sc[WA_QW];
#pragma unroll
    for (int qi = 0; qi < WA_QW; ++qi) sc[qi] = 0.f;
    const float4* k4 = reinterpret_cast<const float4*>(sK + (size_t)lane * KS);
    for (int d4 = 0; d4 < DKP / 4; ++d4) {
      const float4 kv = k4[d4];
#pragma unroll
      for (int qi = 0; qi < WA_QW; ++qi) {
        const float4 qv = reinterpret_cast<const float4*>(sQ + (size_t)(warp + qi * WA_WARPS) * DKP)[d4];
        sc[qi] = fmaf(qv.x, kv.x, sc[qi]);
        sc[qi] = fmaf(qv.y, kv.y, sc[qi]);
        sc[qi] = fmaf(qv.z, kv.z, sc[qi]);
        sc[qi] = fmaf(qv.w, kv.w, sc[qi]);
      }
    }
#pragma unroll
    for (int qi = 0; qi < WA_QW; ++qi) {
      const int p = rpos[qi];
      const bool vis = kj >= 0 && kj <= p && ((a.window <= 0 || p - kj < a.window) || kj < a.keep_first);
      const float s = sc[qi] * a.scale;
      float w;
      if (a.kind == L3_ATTN_SIGMOID) {
        w = vis ? sigmoid_f(s + hv[qi]) : 0.f;
      } else {
        const float mnew = fmaxf(mx[qi], warp_max(vis ? s : -INFINITY));
        const float alpha = mnew == -INFINITY ? 1.f : expf(mx[qi] - mnew);
        w = vis ? expf(s - mnew) : 0.f;
        sum[qi] = sum[qi] * alpha + warp_sum(w);
        mx[qi] = mnew;
#pragma unroll
        for (int j = 0; j < NJ; ++j) o[qi][j] *= alpha;
      }
      myP[qi * WA_KEYS + lane] = w;
    }
    __syncwarp();
    // outputs: lane = value columns lane + 32 j
    for (int k0 = 0; k0 < WA_KEYS; k0 += 4) {
      float4 pw[WA_QW];
#pragma unroll
      for (int qi = 0; qi < WA_QW; ++qi) pw[qi] = *reinterpret_cast<const float4*>(myP + qi * WA_KEYS + k0);
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const float v0f = sV[(k0 + 0) * DVP + lane + 32 * j], v1f = sV[(k0 + 1) * DVP + lane + 32 * j];
        const float v2f = sV[(k0 + 2) * DVP + lane + 32 * j], v3f = sV[(k0 + 3) * DVP + lane + 32 * j];
#pragma unroll
        for (int qi = 0; qi < WA_QW; ++qi) {
          o[qi][j] = fmaf(pw[qi].x, v0f, o[qi][j]);
          o[qi][j] = fmaf(pw[qi].y, v1f, o[qi][j]);
          o[qi][j] = fmaf(pw[qi].z, v2f, o[qi][j]);
          o[qi][j] = fmaf(pw[qi].w, v3f, o[qi][j]);
        }
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int qi = 0; qi < WA_QW; ++qi) {
    const int row = row0 + warp + qi * WA_WARPS;
    if (row >= nrows) continue;
    const int t = row / rep, h = g * rep + (row - t * rep);
    const size_t r = (size_t)b * a.L + t;
    if (a.nsplit > 1) {  // partial (o, max, sum) of this split
      const size_t pi = (r * a.H + h) * a.nsplit + split;
#pragma unroll
      for (int j = 0; j < NJ; ++j)
        if (lane + 32 * j < a.DV) a.part_o[pi * a.DV + lane + 32 * j] = o[qi][j];
      if (lane == 0) { a.part_ml[pi * 2] = mx[qi]; a.part_ml[pi * 2 + 1] = sum[qi]; }
      continue;
    }
    const float mul = a.out_scale * (a.kind == L3_ATTN_SIGMOID ? 1.f : (sum[qi] > 0.f ? 1.0f / sum[qi] : 0.f));
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int d = lane + 32 * j;
      if (d < a.DV) {
        const float v = o[qi][j] * mul;
        const size_t oi = r * a.ld_out + (size_t)h * a.DV + d;
        a.out[oi] = v;
        if (a.out16) a.out16[oi] = __float2bfloat16_rn(v);
      }
    }
  }
}

// a warp per (row, head): merges the splits' partials
__global__ void __launch_bounds__(128) win_attn_combine_kernel(WinAttnArgs a) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const size_t rh = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (rh >= (size_t)a.B * a.L * a.H) return;
  const size_t r = rh / a.H;
  const int h = (int)(rh - r * a.H);
  float M = -INFINITY;
  if (a.kind != L3_ATTN_SIGMOID)
    for (int s = 0; s < a.nsplit; ++s) M = fmaxf(M, a.part_ml[(rh * a.nsplit + s) * 2]);
  float den = 0.f;
  for (int d = lane; d < a.DV; d += 32) {
    float acc = 0.f;
    den = 0.f;
    for (int s = 0; s < a.nsplit; ++s) {
      const size_t pi = rh * a.nsplit + s;
      float f = 1.f;
      if (a.kind != L3_ATTN_SIGMOID) {
        const float ms = a.part_ml[pi * 2];
        f = ms == -INFINITY ? 0.f : expf(ms - M);
        den = fmaf(a.part_ml[pi * 2 + 1], f, den);
      }
      acc = fmaf(a.part_o[pi * a.DV + d], f, acc);
    }
    const float mul = a.out_scale * (a.kind == L3_ATTN_SIGMOID ? 1.f : (den > 0.f ? 1.0f / den : 0.f));
    const float v = acc * mul;
    const size_t oi = r * a.ld_out + (size_t)h * a.DV + d;
    a.out[oi] = v;
    if (a.out16) a.out16[oi] = __float2bfloat16_rn(v);
  }
}

size_t win_attn_smem(int DK, int NJ) {
  const int DKP = (DK + 3) & ~3;
  return ((size_t)WA_ROWS * DKP + (size_t)WA_KEYS * (DKP + 4) + (size_t)WA_KEYS * 32 * NJ + (size_t)WA_WARPS * WA_QW * WA_KEYS) * sizeof(float);
}

int win_nj(int DV) { return DV <= 32 ? 1 : DV <= 64 ? 2 : DV <= 128 ? 4 : 8; }

template <typename KVT, int NJ>
cudaError_t launch_win_nj(const WinAttnArgs& a, dim3 grid, cudaStream_t s) {
  const size_t smem = win_attn_smem(a.DK, NJ);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(win_attn_kernel<KVT, NJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  return launch_k(win_attn_kernel<KVT, NJ>, grid, dim3(256), smem, s, a);
}

template <typename KVT>
cudaError_t launch_win_t(const WinAttnArgs& a, dim3 grid, cudaStream_t s) {
  switch (win_nj(a.DV)) {
    case 1: return launch_win_nj<KVT, 1>(a, grid, s);
    case 2: return launch_win_nj<KVT, 2>(a, grid, s);
    case 4: return launch_win_nj<KVT, 4>(a, grid, s);
    default: return launch_win_nj<KVT, 8>(a, grid, s);
  }
}

}  // namespace

bool win_attn_supported(int DK, int DV) {
  return DK >= 1 && DV >= 1 && DV <= 256 && win_attn_smem(DK, win_nj(DV)) <= 200 * 1024;
}

int win_attn_splits(int B, int L, int H, int G, int window, int keep_first, int max_keys, int max_split) {
  if (L > 8) return 1;
  const int rep = H / G;
  const int ctas = B * G * ((L * rep + WA_ROWS - 1) / WA_ROWS);
  int keys = max_keys;
  if (window > 0) keys = std::min(keys, window + L + keep_first);
  const int tiles = (keys + WA_KEYS - 1) / WA_KEYS;
  // at least two key tiles per split, aimed at two CTAs per SM
  return std::max(1, std::min(std::min(max_split, tiles / 2), (2 * 148) / std::max(1, ctas)));
}

size_t win_attn_part_floats(int max_rows, int H, int DV, int max_split) { return (size_t)max_rows * H * max_split * DV; }

cudaError_t launch_win_prep(const WinPrepArgs& a, int rows, bool kv_bf16, cudaStream_t s) {
  const int vecs = a.H + a.G;
  const int threads = std::min(256, 32 * std::max(1, std::min(vecs, 8)));
  const size_t smem = (size_t)(threads / 32) * a.DK * sizeof(float);
  if (kv_bf16) return launch_k(win_prep_kernel<bf16>, dim3(rows), dim3(threads), smem, s, a);
  return launch_k(win_prep_kernel<float>, dim3(rows), dim3(threads), smem, s, a);
}

cudaError_t launch_win_attn(const WinAttnArgs& a, bool kv_bf16, cudaStream_t s) {
  if (!win_attn_supported(a.DK, a.DV) || a.H % a.G != 0 || a.nsplit < 1) return cudaErrorInvalidValue;
  if (a.nsplit > 1 && (!a.part_o || !a.part_ml)) return cudaErrorInvalidValue;
  const int rep = a.H / a.G;
  const dim3 grid((a.L * rep + WA_ROWS - 1) / WA_ROWS, a.G, a.B * a.nsplit);
  cudaError_t e = kv_bf16 ? launch_win_t<bf16>(a, grid, s) : launch_win_t<float>(a, grid, s);
  if (e != cudaSuccess || a.nsplit == 1) return e;
  const int64_t rh = (int64_t)a.B * a.L * a.H;
  return launch_k(win_attn_combine_kernel, dim3((unsigned)((rh + 3) / 4)), dim3(128), 0, s, a);
}
