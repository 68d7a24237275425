// Sliding-window attention that may keep the first tokens (L3_MIX_WINDOW): GQA with key size DK and value size DV,
// the weight of a visible key either a softmax term whose denominator also holds a per-head sink, or sigmoid(score +
// per-head bias) without any normalisation over keys.  Everything fp32 (FFMA): scores, weights, accumulation.
//
//  * win_prep_kernel     a warp per head vector of a token: rotary turn of the leading rot_dims entries at the token's
//                        position (pairs (2i, 2i + 1) or (i, i + rot_dims / 2); angle = position * frequency in fp32,
//                        sincosf), optional division by the vector's root mean square, q to the query buffer, k and the
//                        value row to the caches
//  * win_attn_kernel     a CTA holds 32 query rows of ONE key head - row = (token, query head of the group), token-major,
//                        so the heads of a group share every key / value tile - and walks the keys the tile can see, 64 at
//                        a time: first the kept tokens that lie ahead of the window, then the window.  A
//                        warp owns 4 rows; in the score phase a lane holds two keys (16-byte shared loads, key rows padded by
//                        4 floats), in the output phase a lane owns value columns read as 16-byte pieces while the weights
//                        arrive as 16-byte broadcasts.  Softmax rows run the online form,
//                        started at (max = sink, sum = 1) so that the sink needs no key; sigmoid rows just accumulate.
//                        Calls of few tokens split the key tiles over CTAs (win_attn_combine_kernel merges).
#include <algorithm>

#include "common.cuh"
#include "mixer.h"
#include "../../include/llama3_b200.h"

namespace {

constexpr int WA_ROWS = 32, WA_KEYS = 64, WA_WARPS = 8, WA_QW = WA_ROWS / WA_WARPS;

template <typename KVT>
__global__ void __launch_bounds__(256) win_prep_kernel(WinPrepArgs a) {
  extern __shared__ float sm[];  // [warps][DK] | cosines and sines of the row's angles [rot_dims / 2] each
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int b = r / a.L, t = r - b * a.L;
  const int pos = *a.pos_ptr + t;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float* row = a.proj + (size_t)r * a.ld;
  float* buf = sm + (size_t)warp * a.DK;
  const int half = a.rot_dims / 2;
  float* cs = sm + (size_t)nw * a.DK;
  float* sn = cs + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * a.inv_freq[i], &sn[i], &cs[i]);  // once per row, every head reads them
  __syncthreads();
  for (int v = warp; v < a.H + a.G; v += nw) {
    const bool is_q = v < a.H;
    const float* src = row + (is_q ? a.q_off + (size_t)v * a.DK : a.k_off + (size_t)(v - a.H) * a.DK);
    for (int i = lane; i < half; i += 32) {
      const int i0 = a.rot_layout ? i : 2 * i, i1 = a.rot_layout ? i + half : 2 * i + 1;
      const float u = src[i0], w = src[i1];
      buf[i0] = u * cs[i] - w * sn[i];
      buf[i1] = w * cs[i] + u * sn[i];
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

// One row of a key / value tile from the cache into shared memory as floats: `n` values (dst padded with zeros up to np).
// 16-byte global loads where the row length allows them.
template <typename KVT>
__device__ __forceinline__ void stage_row(const KVT* __restrict__ src, int n, int np, float* __restrict__ dst, int part, int nparts) {
  constexpr int VEC = 16 / (int)sizeof(KVT);
  if (src && n % VEC == 0) {
    for (int c = part; c < n / VEC; c += nparts) {
      float v[VEC];
      Vec16<KVT>::load(src + c * VEC, v);
#pragma unroll
      for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4*>(dst + c * VEC + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
    for (int i = n + part; i < np; i += nparts) dst[i] = 0.f;
  } else {
    for (int i = part; i < np; i += nparts) dst[i] = (src && i < n) ? to_f32(src[i]) : 0.f;
  }
}

// value column j (< NJ) of a lane: lanes read 16-byte (8-byte, 4-byte) pieces that tile a row without bank conflicts
template <int NJ>
__device__ __forceinline__ int win_col(int lane, int j) {
  return NJ == 1 ? lane : NJ == 2 ? 2 * lane + j : (j >> 2) * 128 + 4 * lane + (j & 3);
}

// NJ: value columns per lane (DV <= 32 NJ)
template <typename KVT, int NJ>
__global__ void __launch_bounds__(256) win_attn_kernel(WinAttnArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int DKP = (a.DK + 3) & ~3, KS = DKP + 4, DVP = 32 * NJ;
  float* sQ = sm;                                  // [32][DKP]
  float* sK = sQ + (size_t)WA_ROWS * DKP;          // [64][DKP + 4]
  float* sV = sK + (size_t)WA_KEYS * KS;           // [64][DVP]
  float* sP = sV + (size_t)WA_KEYS * DVP;          // [warps][QW][64]
  pdl_launch();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rep = a.H / a.G;
  const int g = blockIdx.y;
  const int b = blockIdx.z / a.nsplit, split = blockIdx.z - b * a.nsplit;
  const int nrows = a.L * rep;                     // rows of this (sequence, key head): row = t * rep + head in group
  const int row0 = (gridDim.x - 1 - blockIdx.x) * WA_ROWS;  // late tokens see the most keys: their tiles start first
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

  // queries: 8 threads per row
  for (int rr = tid >> 3; rr < WA_ROWS; rr += 32) {
    const int row = row0 + rr;
    const float* src = nullptr;
    if (row < nrows) {
      const int t = row / rep, h = g * rep + (row - t * rep);
      src = a.q + (((size_t)b * a.L + t) * a.H + h) * a.DK;
    }
    stage_row<float>(src, a.DK, DKP, sQ + (size_t)rr * DKP, tid & 7, 8);
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
    for (int kk = tid >> 3; kk < WA_KEYS; kk += 32) {  // 8 threads per key / value row
      const int vi = v0 + kk;
      const int j = vi < nkeys ? (vi < ka ? vi : w_lo + (vi - ka)) : -1;
      stage_row<KVT>(j >= 0 ? ck + (size_t)j * a.DK : nullptr, a.DK, DKP, sK + (size_t)kk * KS, tid & 7, 8);
      stage_row<KVT>(j >= 0 ? cv + (size_t)j * a.DV : nullptr, a.DV, DVP, sV + (size_t)kk * DVP, tid & 7, 8);
    }
    __syncthreads();
    // scores: a lane holds keys lane and lane + 32 of the tile
    int kj[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int vi = v0 + lane + 32 * u;
      kj[u] = vi < nkeys ? (vi < ka ? vi : w_lo + (vi - ka)) : -1;
    }
    float sc[WA_QW][2];
#pragma unroll
    for (int qi = 0; qi < WA_QW; ++qi) sc[qi][0] = sc[qi][1] = 0.f;
    const float4* kA = reinterpret_cast<const float4*>(sK + (size_t)lane * KS);
    const float4* kB = reinterpret_cast<const float4*>(sK + (size_t)(lane + 32) * KS);
#pragma unroll 2
    for (int d4 = 0; d4 < DKP / 4; ++d4) {
      const float4 ka4 = kA[d4], kb4 = kB[d4];
#pragma unroll
      for (int qi = 0; qi < WA_QW; ++qi) {
        const float4 qv = reinterpret_cast<const float4*>(sQ + (size_t)(warp + qi * WA_WARPS) * DKP)[d4];
        sc[qi][0] = fmaf(qv.x, ka4.x, sc[qi][0]); sc[qi][1] = fmaf(qv.x, kb4.x, sc[qi][1]);
        sc[qi][0] = fmaf(qv.y, ka4.y, sc[qi][0]); sc[qi][1] = fmaf(qv.y, kb4.y, sc[qi][1]);
        sc[qi][0] = fmaf(qv.z, ka4.z, sc[qi][0]); sc[qi][1] = fmaf(qv.z, kb4.z, sc[qi][1]);
        sc[qi][0] = fmaf(qv.w, ka4.w, sc[qi][0]); sc[qi][1] = fmaf(qv.w, kb4.w, sc[qi][1]);
      }
    }
#pragma unroll
    for (int qi = 0; qi < WA_QW; ++qi) {
      const int p = rpos[qi];
      bool vis[2];
      float s2[2], w[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        vis[u] = kj[u] >= 0 && kj[u] <= p && ((a.window <= 0 || p - kj[u] < a.window) || kj[u] < a.keep_first);
        s2[u] = sc[qi][u] * a.scale;
      }
      if (a.kind == L3_ATTN_SIGMOID) {
        w[0] = vis[0] ? sigmoid_f(s2[0] + hv[qi]) : 0.f;
        w[1] = vis[1] ? sigmoid_f(s2[1] + hv[qi]) : 0.f;
      } else {
        const float mnew = fmaxf(mx[qi], warp_max(fmaxf(vis[0] ? s2[0] : -INFINITY, vis[1] ? s2[1] : -INFINITY)));
        const float alpha = mnew == -INFINITY ? 1.f : expf(mx[qi] - mnew);
        w[0] = vis[0] ? expf(s2[0] - mnew) : 0.f;
        w[1] = vis[1] ? expf(s2[1] - mnew) : 0.f;
        sum[qi] = sum[qi] * alpha + warp_sum(w[0] + w[1]);
        mx[qi] = mnew;
#pragma unroll
        for (int j = 0; j < NJ; ++j) o[qi][j] *= alpha;
      }
      myP[qi * WA_KEYS + lane] = w[0];
      myP[qi * WA_KEYS + lane + 32] = w[1];
    }
    __syncwarp();
    // outputs: a lane owns NJ value columns (win_col), read as 16-byte pieces
    for (int k0 = 0; k0 < WA_KEYS; k0 += 4) {
      float4 pw[WA_QW];
#pragma unroll
      for (int qi = 0; qi < WA_QW; ++qi) pw[qi] = *reinterpret_cast<const float4*>(myP + qi * WA_KEYS + k0);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        float vv[NJ];
        const float* vr = sV + (size_t)(k0 + kk) * DVP;
        if (NJ == 1) vv[0] = vr[lane];
        else if (NJ == 2) { const float2 t2 = *reinterpret_cast<const float2*>(vr + 2 * lane); vv[0] = t2.x; vv[1] = t2.y; }
        else {
#pragma unroll
          for (int c = 0; c < NJ / 4; ++c) {
            const float4 t4 = *reinterpret_cast<const float4*>(vr + c * 128 + 4 * lane);
            vv[4 * c] = t4.x; vv[4 * c + 1] = t4.y; vv[4 * c + 2] = t4.z; vv[4 * c + 3] = t4.w;
          }
        }
#pragma unroll
        for (int qi = 0; qi < WA_QW; ++qi) {
          const float pk = kk == 0 ? pw[qi].x : kk == 1 ? pw[qi].y : kk == 2 ? pw[qi].z : pw[qi].w;
#pragma unroll
          for (int j = 0; j < NJ; ++j) o[qi][j] = fmaf(pk, vv[j], o[qi][j]);
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
      for (int j = 0; j < NJ; ++j) {
        const int d = win_col<NJ>(lane, j);
        if (d < a.DV) a.part_o[pi * a.DV + d] = o[qi][j];
      }
      if (lane == 0) { a.part_ml[pi * 2] = mx[qi]; a.part_ml[pi * 2 + 1] = sum[qi]; }
      continue;
    }
    const float mul = a.out_scale * (a.kind == L3_ATTN_SIGMOID ? 1.f : (sum[qi] > 0.f ? 1.0f / sum[qi] : 0.f));
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int d = win_col<NJ>(lane, j);
      if (d < a.DV) {
        const float v = o[qi][j] * mul;
        const size_t oi = r * a.ld_out + (size_t)h * a.DV + d;
        a.out[oi] = v;
        if (a.out16) a.out16[oi] = __float2bfloat16_rn(v);
      }
    }
  }
}

// a thread per (row, head, value column): merges the splits' partials
__global__ void __launch_bounds__(128) win_attn_combine_kernel(WinAttnArgs a) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.B * a.L * a.H * a.DV) return;
  const size_t rh = (size_t)(i / a.DV);
  const int d = (int)(i - (int64_t)rh * a.DV);
  const size_t r = rh / a.H;
  const int h = (int)(rh - r * a.H);
  float M = -INFINITY;
  if (a.kind != L3_ATTN_SIGMOID)
    for (int s = 0; s < a.nsplit; ++s) M = fmaxf(M, a.part_ml[(rh * a.nsplit + s) * 2]);
  float acc = 0.f, den = 0.f;
#pragma unroll 4
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

size_t win_attn_smem(int DK, int NJ) {
  const int DKP = (DK + 3) & ~3;
  return ((size_t)WA_ROWS * DKP + (size_t)WA_KEYS * (DKP + 4) + (size_t)WA_KEYS * 32 * NJ + (size_t)WA_WARPS * WA_QW * WA_KEYS) * sizeof(float);
}

int win_nj(int DV) { return DV <= 32 ? 1 : DV <= 64 ? 2 : DV <= 128 ? 4 : DV <= 256 ? 8 : 16; }

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
    case 8: return launch_win_nj<KVT, 8>(a, grid, s);
    default: return launch_win_nj<KVT, 16>(a, grid, s);
  }
}

}  // namespace

bool win_attn_supported(int DK, int DV) {
  return DK >= 1 && DV >= 1 && DV <= 512 && win_attn_smem(DK, win_nj(DV)) <= 220 * 1024;
}

int win_attn_splits(int B, int L, int H, int G, int window, int keep_first, int max_keys, int max_split) {
  if (L > 8) return 1;
  const int rep = H / G;
  const int ctas = B * G * ((L * rep + WA_ROWS - 1) / WA_ROWS);
  int keys = max_keys;
  if (window > 0) keys = std::min(keys, window + L + keep_first);
  const int tiles = (keys + WA_KEYS - 1) / WA_KEYS;
  // a key tile or more per split, aimed at two CTAs per SM
  return std::max(1, std::min(std::min(max_split, tiles), (2 * 148) / std::max(1, ctas)));
}

size_t win_attn_part_floats(int max_rows, int H, int DV, int max_split) { return (size_t)max_rows * H * max_split * DV; }

cudaError_t launch_win_prep(const WinPrepArgs& a, int rows, bool kv_bf16, cudaStream_t s) {
  const int vecs = a.H + a.G;
  const int threads = std::min(256, 32 * std::max(1, std::min(vecs, 8)));
  const size_t smem = ((size_t)(threads / 32) * a.DK + a.rot_dims) * sizeof(float);
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
  const int64_t n = (int64_t)a.B * a.L * a.H * a.DV;
  return launch_k(win_attn_combine_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, s, a);
}
