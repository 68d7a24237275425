// Differential sliding-window attention (L3_MIX_DIFF, include/llama3_b200.h).
//
// Every query head holds two maps [map 1 | map 2] of size DK; key head g likewise; both maps of a query head attend over
// the SAME values (size DV) of its key head with a softmax of their own, and the head's output is
//     o = a1 - lambda a2,   o <- o / sqrt(mean(o^2) + eps) * (1 - diff).
// Query i sees keys j with 0 <= i - j < window.  Scores, softmax weights, sums and the norm are fp32 in both modes.
//
//  * diff_lambda_kernel      lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, once per layer at finalize
//  * diff_prep_kernel        bias, RMS norm per head and map (one weight vector), rotary turn of the first rot_dims entries of
//                            each map (entry i with entry i + rot_dims / 2; the row's angles position * f_i, cosines and sines
//                            computed once in fp32 and shared by all heads), append of the keys
//                            [maxB, 2 G, M, DK] (head g, map m at 2 g + m) and of the biased values [maxB, G, M, DV]
//  * attn_diff_tile_kernel   prompts: 64 queries x 64 keys per tile for one head, both maps at once - two score tiles, two
//                            online softmaxes, two accumulators fed by the same value rows; tiles outside the window are
//                            never visited; the combination and the head norm are the epilogue
//  * attn_diff_cta_kernel    decode, short portions and head sizes outside the tiled list: a CTA per (token, head), its warps
//                            split the visible keys (a lane scores one key for both maps), merged through shared memory
#include <algorithm>

#include "common.cuh"
#include "mixer.h"

namespace {

__global__ void diff_lambda_kernel(const float* __restrict__ v, int n, float diff, float* __restrict__ out) {
  // v = lq1 | lk1 | lq2 | lk2, n entries each; one warp
  const int lane = threadIdx.x;
  float s1 = 0.f, s2 = 0.f;
  for (int i = lane; i < n; i += 32) { s1 = fmaf(v[i], v[n + i], s1); s2 = fmaf(v[2 * n + i], v[3 * n + i], s2); }
  s1 = warp_sum(s1);
  s2 = warp_sum(s2);
  if (lane == 0) *out = expf(s1) - expf(s2) + diff;
}

template <typename KVT>
__global__ void __launch_bounds__(256) diff_prep_kernel(DiffPrepArgs a) {
  extern __shared__ float sm[];  // the row's cosines and sines [2][rot_dims / 2]
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const size_t r = blockIdx.x;
  const int b = (int)(r / a.L), t = (int)(r - (size_t)b * a.L);
  const int pos = *a.pos_ptr + t;
  const int DK = a.DK, half = a.rot_dims >> 1;
  const float* pr = a.proj + r * a.ld;
  float* cs_tab = sm;
  float* sn_tab = cs_tab + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * a.inv_freq[i], &sn_tab[i], &cs_tab[i]);  // every head turns by the same angles
  __syncthreads();
  const int nq = 2 * a.H, nk = 2 * a.G;
  for (int vec = blockIdx.y * nw + warp; vec < nq + nk; vec += gridDim.y * nw) {  // a row's vectors spread over gridDim.y CTAs
    const bool isq = vec < nq;
    const int col = isq ? a.q_off + vec * DK : a.k_off + (vec - nq) * DK;
    const float* src = pr + col;
    const float* bs = a.bias + col;
    const float* w = isq ? a.wq : a.wk;
    float ss = 0.f;
    for (int d = lane; d < DK; d += 32) { const float v = src[d] + bs[d]; ss = fmaf(v, v, ss); }
    const float rinv = 1.0f / sqrtf(warp_sum(ss) / (float)DK + a.eps);
    KVT* kdst = isq ? nullptr : (KVT*)a.cache_k + (((size_t)b * nk + (vec - nq)) * a.M + pos) * DK;
    float* qdst = isq ? a.q_out + r * ((size_t)nq * DK) + (size_t)vec * DK : nullptr;
    // a lane holds both entries of a rotated pair (i, i + half): no exchange between lanes
    for (int i = lane; i < half; i += 32) {
      const float lo = (src[i] + bs[i]) * rinv * w[i], hi = (src[i + half] + bs[i + half]) * rinv * w[i + half];
      const float sn = sn_tab[i], cs = cs_tab[i];
      const float o_lo = lo * cs - hi * sn, o_hi = hi * cs + lo * sn;
      if (isq) { qdst[i] = o_lo; qdst[i + half] = o_hi; }
      else { kdst[i] = from_f32<KVT>(o_lo); kdst[i + half] = from_f32<KVT>(o_hi); }
    }
    for (int d = a.rot_dims + lane; d < DK; d += 32) {
      const float o = (src[d] + bs[d]) * rinv * w[d];
      if (isq) qdst[d] = o;
      else kdst[d] = from_f32<KVT>(o);
    }
  }
  const int nv = a.G * a.DV;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < nv; i += gridDim.y * blockDim.x) {
    const int g = i / a.DV, d = i - g * a.DV;
    ((KVT*)a.cache_v)[(((size_t)b * a.G + g) * a.M + pos) * a.DV + d] = from_f32<KVT>(pr[a.v_off + i] + a.bias[a.v_off + i]);
  }
}

// ---------------------------------------------------------------------------------------------- generic CTA kernel
template <typename KVT>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const KVT* __restrict__ k, int n) {
  constexpr int VEC = Vec16<KVT>::N;
  float acc = 0.f;
  if (n % VEC == 0) {
    for (int d = 0; d < n; d += VEC) {
      float f[VEC];
      Vec16<KVT>::unpack(*reinterpret_cast<const uint4*>(k + d), f);
#pragma unroll
      for (int x = 0; x < VEC; ++x) acc = fmaf(q[d + x], f[x], acc);
    }
  } else {
    for (int d = 0; d < n; ++d) acc = fmaf(q[d], to_f32(k[d]), acc);
  }
  return acc;
}

constexpr int DIFF_CTA_WARPS = 8;
constexpr int DIFF_DEC_MAX_L = 8;     // rows per sequence the decode kernel takes
constexpr int DIFF_DEC_CTAS = 296;    // CTAs a split decode launch aims at

template <typename KVT>
__global__ void __launch_bounds__(DIFF_CTA_WARPS * 32) attn_diff_cta_kernel(DiffAttnArgs a) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NW = DIFF_CTA_WARPS;
  const int DK = a.DK, DV = a.DV;
  float* qs = sm;                       // [2][DK]
  float* os = qs + 2 * DK;              // [NW][2][DV]
  float* st = os + (size_t)NW * 2 * DV; // [NW][4]: m1, l1, m2, l2
  float* red = st + NW * 4;             // [32]
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.x % a.H;
  const size_t row = blockIdx.x / a.H;
  const int b = (int)(row / a.L), t = (int)(row - (size_t)b * a.L);
  const int last = *a.pos_ptr + t;
  const int lo = a.window > 0 ? max(0, last - a.window + 1) : 0;
  const int g = head / (a.H / a.G);
  for (int d = threadIdx.x; d < 2 * DK; d += blockDim.x) qs[d] = a.q[(row * a.H + head) * (size_t)(2 * DK) + d];
  float* o1 = os + (size_t)warp * 2 * DV;
  float* o2 = o1 + DV;
  for (int d = lane; d < 2 * DV; d += 32) o1[d] = 0.f;
  __syncthreads();
  const KVT* k1 = (const KVT*)a.cache_k + ((size_t)b * 2 * a.G + 2 * g) * a.M * DK;
  const KVT* k2 = k1 + (size_t)a.M * DK;
  const KVT* vb = (const KVT*)a.cache_v + ((size_t)b * a.G + g) * a.M * DV;
  float m1 = -INFINITY, l1 = 0.f, m2 = -INFINITY, l2 = 0.f;
  for (int j0 = lo + warp * 32; j0 <= last; j0 += NW * 32) {
    const int j = j0 + lane;
    float s1 = -INFINITY, s2 = -INFINITY;
    if (j <= last) {
      s1 = dot_row<KVT>(qs, k1 + (size_t)j * DK, DK) * a.scale;
      s2 = dot_row<KVT>(qs + DK, k2 + (size_t)j * DK, DK) * a.scale;
    }
    const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
    const float p1 = j <= last ? expf(s1 - n1) : 0.f, p2 = j <= last ? expf(s2 - n2) : 0.f;
    const float al1 = expf(m1 - n1), al2 = expf(m2 - n2);  // first batch: exp(-inf) = 0 and o, l are 0
    l1 = l1 * al1 + warp_sum(p1);
    l2 = l2 * al2 + warp_sum(p2);
    m1 = n1; m2 = n2;
    const int nb = min(32, last + 1 - j0);
    for (int d0 = 0; d0 < DV; d0 += 32) {  // every lane runs every round: the shuffles name the full warp
      const int d = d0 + lane;
      const bool ok = d < DV;
      float c1 = ok ? o1[d] * al1 : 0.f, c2 = ok ? o2[d] * al2 : 0.f;
      for (int u = 0; u < nb; ++u) {
        const float pu1 = __shfl_sync(L3_FULL, p1, u), pu2 = __shfl_sync(L3_FULL, p2, u);
        if (ok) {
          const float v = to_f32(vb[(size_t)(j0 + u) * DV + d]);
          c1 = fmaf(pu1, v, c1);
          c2 = fmaf(pu2, v, c2);
        }
      }
      if (ok) { o1[d] = c1; o2[d] = c2; }
    }
  }
  if (lane == 0) { st[warp * 4] = m1; st[warp * 4 + 1] = l1; st[warp * 4 + 2] = m2; st[warp * 4 + 3] = l2; }
  __syncthreads();
  // merge the warps' partial softmaxes (a warp without keys has m = -inf, l = 0 and weighs nothing)
  float M1 = -INFINITY, M2 = -INFINITY;
  for (int w = 0; w < NW; ++w) { M1 = fmaxf(M1, st[w * 4]); M2 = fmaxf(M2, st[w * 4 + 2]); }
  float L1 = 0.f, L2 = 0.f;
  for (int w = 0; w < NW; ++w) { L1 += st[w * 4 + 1] * expf(st[w * 4] - M1); L2 += st[w * 4 + 3] * expf(st[w * 4 + 2] - M2); }
  const float lam = *a.lambda;
  float ss = 0.f;
  for (int d = threadIdx.x; d < DV; d += blockDim.x) {
    float c1 = 0.f, c2 = 0.f;
    for (int w = 0; w < NW; ++w) {
      c1 = fmaf(os[((size_t)w * 2) * DV + d], expf(st[w * 4] - M1), c1);
      c2 = fmaf(os[((size_t)w * 2 + 1) * DV + d], expf(st[w * 4 + 2] - M2), c2);
    }
    const float o = c1 / L1 - lam * (c2 / L2);
    os[d] = o;                     // warp 0's map-1 slot: every d is written by exactly one thread after its reads
    ss = fmaf(o, o, ss);
  }
  // block sum of ss
  ss = warp_sum(ss);
  __syncthreads();
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < NW; ++w) tot += red[w];
  const float mul = (1.0f - a.diff) / sqrtf(tot / (float)DV + a.eps);
  for (int d = threadIdx.x; d < DV; d += blockDim.x) {
    const float v = os[d] * mul;
    const size_t oi = (row * a.H + head) * (size_t)DV + d;
    a.out[oi] = v;
    if (a.out16) a.out16[oi] = __float2bfloat16_rn(v);
  }
}

// ---------------------------------------------------------------------------------------------- tiled prompt kernel
template <typename KVT> __device__ __forceinline__ float4 ld_kv4(const KVT* p);
template <> __device__ __forceinline__ float4 ld_kv4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ld_kv4<bf16>(const bf16* p) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u), __uint_as_float(r.y << 16),
                     __uint_as_float(r.y & 0xffff0000u));
}

constexpr int DT_ROWS = 64, DT_TK = 64, DT_LDS = DT_TK + 4;

template <int DK, int DV>
constexpr size_t diff_tile_smem() {
  return (size_t)(2 * DT_ROWS * (DK + 4) + 2 * DT_TK * (DK + 4) + DT_TK * DV + 2 * DT_ROWS * DT_LDS + 6 * DT_ROWS) * sizeof(float);
}

// TXN lanes share a group of four queries: 16 (256 threads, four keys and 4 x DV / 64 output columns per thread) or, for values
// of 128 and more, 32 (512 threads, two keys per thread; a warp then reads ONE query row - a broadcast - per load)
template <int DK, int DV, int TXN, typename KVT>
__global__ void __launch_bounds__(16 * TXN) attn_diff_tile_kernel(DiffAttnArgs a) {
  constexpr int NT = 16 * TXN, KPT = DT_TK / TXN, NWARP = NT / 32, RPW = 2 * DT_ROWS / NWARP;
  constexpr int LDK = DK + 4, DK4 = DK / 4, DV4 = DV / 4, NCH = (DV + 4 * TXN - 1) / (4 * TXN);
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                           // [2][ROWS][LDK]
  float* Ks = Qs + 2 * DT_ROWS * LDK;       // [2][TK][LDK]
  float* Vs = Ks + 2 * DT_TK * LDK;         // [TK][DV]
  float* Ss = Vs + DT_TK * DV;              // [2][ROWS][LDS]
  float* St = Ss + 2 * DT_ROWS * DT_LDS;    // [2][ROWS][3]: running max, running sum, rescale of this tile
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ty = tid / TXN, tx = tid % TXN;
  const int head = blockIdx.y, b = blockIdx.z;
  const int g = head / (a.H / a.G);
  pdl_launch();
  pdl_wait();
  const int start = *a.pos_ptr;
  const int q0 = (gridDim.x - 1 - blockIdx.x) * DT_ROWS;  // long tiles first
  const int nq = min(DT_ROWS, a.L - q0);
  const int t_hi = start + q0 + nq;  // one past the last visible key
  const int k_lo = a.window > 0 ? max(0, start + q0 - a.window + 1) : 0;
  for (int i = tid; i < 2 * DT_ROWS * DK4; i += NT) {
    const int mp = i / (DT_ROWS * DK4), rem = i - mp * (DT_ROWS * DK4);
    const int r = rem / DK4, d4 = rem - r * DK4;
    float4 v = make_float4(0, 0, 0, 0);
    if (r < nq) v = *reinterpret_cast<const float4*>(a.q + (((size_t)b * a.L + q0 + r) * a.H + head) * (2 * DK) + mp * DK + d4 * 4);
    *reinterpret_cast<float4*>(Qs + (mp * DT_ROWS + r) * LDK + d4 * 4) = v;
  }
  for (int i = tid; i < 2 * DT_ROWS; i += NT) { St[i * 3] = -INFINITY; St[i * 3 + 1] = 0.f; St[i * 3 + 2] = 1.f; }
  float4 acc[2][4][NCH];
#pragma unroll
  for (int mp = 0; mp < 2; ++mp)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < NCH; ++c) acc[mp][i][c] = make_float4(0, 0, 0, 0);
  const KVT* kbase = (const KVT*)a.cache_k + ((size_t)b * 2 * a.G + 2 * g) * a.M * DK;
  const KVT* vbase = (const KVT*)a.cache_v + ((size_t)b * a.G + g) * a.M * DV;

  for (int k0 = k_lo; k0 < t_hi; k0 += DT_TK) {
    __syncthreads();
    for (int i = tid; i < 2 * DT_TK * DK4; i += NT) {
      const int mp = i / (DT_TK * DK4), rem = i - mp * (DT_TK * DK4);
      const int key = rem / DK4, d4 = rem - key * DK4;
      const int t = k0 + key;
      float4 kv = make_float4(0, 0, 0, 0);
      if (t < t_hi) kv = ld_kv4<KVT>(kbase + ((size_t)mp * a.M + t) * DK + d4 * 4);
      *reinterpret_cast<float4*>(Ks + (mp * DT_TK + key) * LDK + d4 * 4) = kv;
    }
    for (int i = tid; i < DT_TK * DV4; i += NT) {
      const int key = i / DV4, d4 = i - key * DV4;
      const int t = k0 + key;
      float4 vv = make_float4(0, 0, 0, 0);
      if (t < t_hi) vv = ld_kv4<KVT>(vbase + (size_t)t * DV + d4 * 4);
      *reinterpret_cast<float4*>(Vs + key * DV + d4 * 4) = vv;
    }
    __syncthreads();
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {  // scores of both maps: queries ty * 4 + i, keys tx + TXN j
      float s[4][KPT];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < KPT; ++j) s[i][j] = 0.f;
      const float* Qm = Qs + mp * DT_ROWS * LDK;
      const float* Km = Ks + mp * DT_TK * LDK;
#pragma unroll 2
      for (int d4 = 0; d4 < DK4; ++d4) {
        float4 qv[4], kv[KPT];
#pragma unroll
        for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4*>(Qm + (ty * 4 + i) * LDK + d4 * 4);
#pragma unroll
        for (int j = 0; j < KPT; ++j) kv[j] = *reinterpret_cast<const float4*>(Km + (tx + TXN * j) * LDK + d4 * 4);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < KPT; ++j) {
            s[i][j] = fmaf(qv[i].x, kv[j].x, s[i][j]); s[i][j] = fmaf(qv[i].y, kv[j].y, s[i][j]);
            s[i][j] = fmaf(qv[i].z, kv[j].z, s[i][j]); s[i][j] = fmaf(qv[i].w, kv[j].w, s[i][j]);
          }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        const int qpos = start + q0 + r;
#pragma unroll
        for (int j = 0; j < KPT; ++j) {
          const int key = tx + TXN * j, kp = k0 + key;
          const bool vis = r < nq && kp <= qpos && (a.window <= 0 || qpos - kp < a.window);
          Ss[(mp * DT_ROWS + r) * DT_LDS + key] = vis ? s[i][j] * a.scale : -INFINITY;
        }
      }
    }
    __syncthreads();
    for (int rr = 0; rr < RPW; ++rr) {  // online softmax: every warp owns RPW of the 128 (map, query) rows
      const int r = warp * RPW + rr;
      float* srow = Ss + r * DT_LDS;
      const float mold = St[r * 3];
      const float s0 = srow[lane], s1 = srow[lane + 32];
      const float mnew = fmaxf(mold, warp_max(fmaxf(s0, s1)));
      float p0 = 0.f, p1 = 0.f, alpha = 1.f;
      if (mnew > -INFINITY) {
        p0 = expf(s0 - mnew);
        p1 = expf(s1 - mnew);
        alpha = expf(mold - mnew);
      }
      const float ps = warp_sum(p0 + p1);
      srow[lane] = p0;
      srow[lane + 32] = p1;
      if (lane == 0) { St[r * 3 + 1] = St[r * 3 + 1] * alpha + ps; St[r * 3] = mnew; St[r * 3 + 2] = alpha; }
    }
    __syncthreads();
    {  // o_m = o_m * alpha_m + P_m V for both maps; a value row read once feeds both
#pragma unroll
      for (int mp = 0; mp < 2; ++mp)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float alpha = St[(mp * DT_ROWS + ty * 4 + i) * 3 + 2];
#pragma unroll
          for (int c = 0; c < NCH; ++c) { acc[mp][i][c].x *= alpha; acc[mp][i][c].y *= alpha; acc[mp][i][c].z *= alpha; acc[mp][i][c].w *= alpha; }
        }
#pragma unroll 2
      for (int k4 = 0; k4 < DT_TK / 4; ++k4) {
        float4 p[2][4];
#pragma unroll
        for (int mp = 0; mp < 2; ++mp)
#pragma unroll
          for (int i = 0; i < 4; ++i) p[mp][i] = *reinterpret_cast<const float4*>(Ss + (mp * DT_ROWS + ty * 4 + i) * DT_LDS + k4 * 4);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const int d = tx * 4 + 4 * TXN * c;
          if (d < DV) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const float4 v = *reinterpret_cast<const float4*>(Vs + (k4 * 4 + kk) * DV + d);
#pragma unroll
              for (int mp = 0; mp < 2; ++mp)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float pw = kk == 0 ? p[mp][i].x : kk == 1 ? p[mp][i].y : kk == 2 ? p[mp][i].z : p[mp][i].w;
                  acc[mp][i][c].x = fmaf(pw, v.x, acc[mp][i][c].x); acc[mp][i][c].y = fmaf(pw, v.y, acc[mp][i][c].y);
                  acc[mp][i][c].z = fmaf(pw, v.z, acc[mp][i][c].z); acc[mp][i][c].w = fmaf(pw, v.w, acc[mp][i][c].w);
                }
            }
          }
        }
      }
    }
  }
  __syncthreads();
  const float lam = *a.lambda;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    const float i1 = 1.0f / St[r * 3 + 1], i2 = lam / St[(DT_ROWS + r) * 3 + 1];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      float4& o = acc[0][i][c];
      const float4 o2 = acc[1][i][c];
      o.x = o.x * i1 - o2.x * i2; o.y = o.y * i1 - o2.y * i2; o.z = o.z * i1 - o2.z * i2; o.w = o.w * i1 - o2.w * i2;
      if (tx * 4 + 4 * TXN * c < DV) ss += o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w;
    }
    // the TXN threads of a query row are adjacent lanes
#pragma unroll
    for (int off = TXN / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(L3_FULL, ss, off);
    const float mul = (1.0f - a.diff) / sqrtf(ss / (float)DV + a.eps);
    if (r >= nq) continue;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int d = tx * 4 + 4 * TXN * c;
      if (d >= DV) continue;
      float4 o = acc[0][i][c];
      o.x *= mul; o.y *= mul; o.z *= mul; o.w *= mul;
      const size_t oi = (((size_t)b * a.L + q0 + r) * a.H + head) * DV + d;
      *reinterpret_cast<float4*>(a.out + oi) = o;
      if (a.out16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo);
        pk.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(a.out16 + oi) = pk;
      }
    }
  }
}


// ---------------------------------------------------------------------------------------------- decode kernel
// Few rows (L <= 8): a CTA per (key split, key head, row).  All REP query heads of the key head and both maps run against
// the same staged work: a lane reads one key row per map ONCE and scores it for every query head, a value row read once
// by the warp feeds all 2 REP accumulators.  Every split leaves (max, sum, o) per (head, map); attn_diff_combine_kernel
// merges the splits, forms a1 - lambda a2 and norms the head.
constexpr int DEC_WARPS = 4;

// N = 1, 2 or 4 consecutive cache values at an N-element aligned index, as one load
template <int N> __device__ __forceinline__ void load_vals(const float* p, float (&v)[N]) {
  if constexpr (N == 4) { const float4 r = *reinterpret_cast<const float4*>(p); v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w; }
  else if constexpr (N == 2) { const float2 r = *reinterpret_cast<const float2*>(p); v[0] = r.x; v[1] = r.y; }
  else { for (int x = 0; x < N; ++x) v[x] = p[x]; }
}
template <int N> __device__ __forceinline__ void load_vals(const bf16* p, float (&v)[N]) {
  if constexpr (N == 4) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
  } else if constexpr (N == 2) {
    const uint32_t r = *reinterpret_cast<const uint32_t*>(p);
    v[0] = __uint_as_float(r << 16); v[1] = __uint_as_float(r & 0xffff0000u);
  } else { for (int x = 0; x < N; ++x) v[x] = __bfloat162float(p[x]); }
}

template <int DK, int DV, int REP, typename KVT>
__global__ void __launch_bounds__(DEC_WARPS * 32) attn_diff_decode_kernel(DiffAttnArgs a, int nsplit, float* __restrict__ part_o,
                                                                          float* __restrict__ part_ml) {
  constexpr int NR = 2 * REP;        // (map, head) rows: index mp * REP + r
  constexpr int VPL = DV / 32;       // value dims per lane
  constexpr int VEC = Vec16<KVT>::N;
  extern __shared__ __align__(16) float sm[];
  float* qs = sm;                          // [NR][DK]
  float* mo = qs + NR * DK;                // [DEC_WARPS][NR][DV]
  float* mml = mo + DEC_WARPS * NR * DV;   // [DEC_WARPS][NR][2]
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int split = blockIdx.x, g = blockIdx.y;
  const size_t row = blockIdx.z;
  const int b = (int)(row / a.L), t = (int)(row - (size_t)b * a.L);
  const int last = *a.pos_ptr + t;
  const int lo = a.window > 0 ? max(0, last - a.window + 1) : 0;
  const int chunk = (((last - lo + 1) + nsplit - 1) / nsplit + 31) & ~31;
  const int k_begin = lo + split * chunk, k_end = min(last, k_begin + chunk - 1);
  for (int i = threadIdx.x; i < NR * DK; i += blockDim.x) {
    const int mp = i / (REP * DK), rem = i - mp * (REP * DK), r = rem / DK, d = rem - r * DK;
    qs[i] = a.q[((row * a.H + (size_t)g * REP + r) * 2 + mp) * DK + d] * a.scale;
  }
  __syncthreads();
  const KVT* kb = (const KVT*)a.cache_k + ((size_t)b * 2 * a.G + 2 * g) * a.M * DK;
  const KVT* vb = (const KVT*)a.cache_v + ((size_t)b * a.G + g) * a.M * DV;
  float mx[NR], ls[NR], acc[NR][VPL];
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    mx[i] = -INFINITY; ls[i] = 0.f;
#pragma unroll
    for (int x = 0; x < VPL; ++x) acc[i][x] = 0.f;
  }
  for (int j0 = k_begin + warp * 32; j0 <= k_end; j0 += DEC_WARPS * 32) {
    const int j = j0 + lane;
    const bool live = j <= k_end;
    float p[NR];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
      float sc[REP];
#pragma unroll
      for (int r = 0; r < REP; ++r) sc[r] = 0.f;
      if (live) {
        const KVT* kr = kb + ((size_t)mp * a.M + j) * DK;
#pragma unroll 4
        for (int d = 0; d < DK; d += VEC) {
          float f[VEC];
          Vec16<KVT>::unpack(*reinterpret_cast<const uint4*>(kr + d), f);
#pragma unroll
          for (int r = 0; r < REP; ++r) {
            const float* qr = qs + (mp * REP + r) * DK + d;
#pragma unroll
            for (int x = 0; x < VEC; x += 4) {
              const float4 qv = *reinterpret_cast<const float4*>(qr + x);
              sc[r] = fmaf(qv.x, f[x], sc[r]); sc[r] = fmaf(qv.y, f[x + 1], sc[r]);
              sc[r] = fmaf(qv.z, f[x + 2], sc[r]); sc[r] = fmaf(qv.w, f[x + 3], sc[r]);
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < REP; ++r) {
        const int i = mp * REP + r;
        const float s = live ? sc[r] : -INFINITY;
        const float mn = fmaxf(mx[i], warp_max(s));
        const float pv = live ? expf(s - mn) : 0.f;
        const float al = expf(mx[i] - mn);  // the warp's first batch holds its first key: mn is finite
        ls[i] = ls[i] * al + warp_sum(pv);
        mx[i] = mn;
        p[i] = pv;
#pragma unroll
        for (int x = 0; x < VPL; ++x) acc[i][x] *= al;
      }
    }
    // eight value rows in flight at a time; rows past the split's end are read clamped and weigh nothing (their p is 0)
    const int nb = min(32, k_end + 1 - j0);
    for (int u0 = 0; u0 < nb; u0 += 8) {
      float v[8][VPL];
#pragma unroll
      for (int u = 0; u < 8; ++u) load_vals<VPL>(vb + (size_t)min(j0 + u0 + u, k_end) * DV + lane * VPL, v[u]);
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const float pu = __shfl_sync(L3_FULL, p[i], u0 + u);
#pragma unroll
          for (int x = 0; x < VPL; ++x) acc[i][x] = fmaf(pu, v[u][x], acc[i][x]);
        }
    }
  }
#pragma unroll
  for (int i = 0; i < NR; ++i) {
#pragma unroll
    for (int x = 0; x < VPL; ++x) mo[((size_t)warp * NR + i) * DV + lane * VPL + x] = acc[i][x];
    if (lane == 0) { mml[(warp * NR + i) * 2] = mx[i]; mml[(warp * NR + i) * 2 + 1] = ls[i]; }
  }
  __syncthreads();
  // merge the warps (one without keys has max = -inf, sum = 0 and weighs nothing); an empty split leaves (-inf, 0, 0)
  for (int i = warp; i < NR; i += DEC_WARPS) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, mml[(w * NR + i) * 2]);
    float Lsum = 0.f, wgt[DEC_WARPS];
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      wgt[w] = M > -INFINITY ? expf(mml[(w * NR + i) * 2] - M) : 0.f;
      Lsum = fmaf(mml[(w * NR + i) * 2 + 1], wgt[w], Lsum);
    }
    const int mp = i / REP, r = i - mp * REP;
    const size_t pi = (((row * a.H + (size_t)g * REP + r) * 2 + mp) * nsplit + split);
    for (int d = lane; d < DV; d += 32) {
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) o = fmaf(mo[((size_t)w * NR + i) * DV + d], wgt[w], o);
      part_o[pi * DV + d] = o;
    }
    if (lane == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = Lsum; }
  }
}

// grid: rows * H; merges the splits of both maps of one (row, head), combines and norms
__global__ void __launch_bounds__(128) attn_diff_combine_kernel(DiffAttnArgs a, int nsplit, const float* __restrict__ part_o,
                                                                const float* __restrict__ part_ml) {
  __shared__ float red[4];
  __shared__ float wgt[2][64];
  pdl_launch();
  pdl_wait();
  const size_t item = blockIdx.x;  // row * H + head
  const int DV = a.DV, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float inv[2];
  for (int mp = 0; mp < 2; ++mp) {
    const float* ml = part_ml + (item * 2 + mp) * nsplit * 2;
    float M = -INFINITY, Ls = 0.f;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, ml[s * 2]);
    for (int s = 0; s < nsplit; ++s) {
      const float w = expf(ml[s * 2] - M);
      Ls = fmaf(ml[s * 2 + 1], w, Ls);
      if (threadIdx.x == 0) wgt[mp][s] = w;
    }
    inv[mp] = 1.0f / Ls;
  }
  __syncthreads();
  const float lam = *a.lambda;
  float ss = 0.f;
  float keep[4];  // DV <= 512
  int n = 0;
  for (int d = threadIdx.x; d < DV; d += blockDim.x, ++n) {
    float o1 = 0.f, o2 = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      o1 = fmaf(part_o[((item * 2) * nsplit + s) * DV + d], wgt[0][s], o1);
      o2 = fmaf(part_o[((item * 2 + 1) * nsplit + s) * DV + d], wgt[1][s], o2);
    }
    const float o = o1 * inv[0] - lam * (o2 * inv[1]);
    keep[n] = o;
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  const float tot = red[0] + red[1] + red[2] + red[3];
  const float mul = (1.0f - a.diff) / sqrtf(tot / (float)DV + a.eps);
  n = 0;
  for (int d = threadIdx.x; d < DV; d += blockDim.x, ++n) {
    const float v = keep[n] * mul;
    a.out[item * DV + d] = v;
    if (a.out16) a.out16[item * DV + d] = __float2bfloat16_rn(v);
  }
}

template <int DK, int DV, int REP, typename KVT>
cudaError_t launch_decode(const DiffAttnArgs& a, int nsplit, float* part_o, float* part_ml, cudaStream_t s) {
  auto kern = attn_diff_decode_kernel<DK, DV, REP, KVT>;
  constexpr size_t smem = (size_t)(2 * REP * DK + DEC_WARPS * 2 * REP * DV + DEC_WARPS * 2 * REP * 2) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  cudaError_t e = launch_k(kern, dim3(nsplit, a.G, a.B * a.L), dim3(DEC_WARPS * 32), smem, s, a, nsplit, part_o, part_ml);
  if (e != cudaSuccess) return e;
  return launch_k(attn_diff_combine_kernel, dim3(a.B * a.L * a.H), dim3(128), 0, s, a, nsplit, (const float*)part_o, (const float*)part_ml);
}

template <int DK, int DV, typename KVT>
cudaError_t launch_decode_rep(const DiffAttnArgs& a, int nsplit, float* part_o, float* part_ml, cudaStream_t s) {
  switch (a.H / a.G) {
    case 1: return launch_decode<DK, DV, 1, KVT>(a, nsplit, part_o, part_ml, s);
    case 2: return launch_decode<DK, DV, 2, KVT>(a, nsplit, part_o, part_ml, s);
    case 4: return launch_decode<DK, DV, 4, KVT>(a, nsplit, part_o, part_ml, s);
    default: return cudaErrorInvalidValue;
  }
}

template <typename KVT>
cudaError_t launch_decode_t(const DiffAttnArgs& a, int nsplit, float* part_o, float* part_ml, cudaStream_t s) {
  if (a.DK == 32 && a.DV == 32) return launch_decode_rep<32, 32, KVT>(a, nsplit, part_o, part_ml, s);
  if (a.DK == 32 && a.DV == 64) return launch_decode_rep<32, 64, KVT>(a, nsplit, part_o, part_ml, s);
  if (a.DK == 64 && a.DV == 64) return launch_decode_rep<64, 64, KVT>(a, nsplit, part_o, part_ml, s);
  if (a.DK == 64 && a.DV == 128) return launch_decode_rep<64, 128, KVT>(a, nsplit, part_o, part_ml, s);
  if (a.DK == 128 && a.DV == 128) return launch_decode_rep<128, 128, KVT>(a, nsplit, part_o, part_ml, s);
  return cudaErrorInvalidValue;
}

template <int DK, int DV, typename KVT>
cudaError_t launch_tile(const DiffAttnArgs& a, cudaStream_t s) {
  constexpr int TXN = DV >= 128 ? 32 : 16;
  auto kern = attn_diff_tile_kernel<DK, DV, TXN, KVT>;
  constexpr size_t smem = diff_tile_smem<DK, DV>();
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return launch_k(kern, dim3((a.L + DT_ROWS - 1) / DT_ROWS, a.H, a.B), dim3(16 * TXN), smem, s, a);
}

template <typename KVT>
cudaError_t launch_tile_t(const DiffAttnArgs& a, cudaStream_t s) {
  if (a.DK == 32 && a.DV == 32) return launch_tile<32, 32, KVT>(a, s);
  if (a.DK == 32 && a.DV == 64) return launch_tile<32, 64, KVT>(a, s);
  if (a.DK == 64 && a.DV == 64) return launch_tile<64, 64, KVT>(a, s);
  if (a.DK == 64 && a.DV == 128) return launch_tile<64, 128, KVT>(a, s);
  if (a.DK == 128 && a.DV == 128) return launch_tile<128, 128, KVT>(a, s);
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_diff_lambda(const float* vecs, int n, float diff, float* out, cudaStream_t s) {
  diff_lambda_kernel<<<1, 32, 0, s>>>(vecs, n, diff, out);
  return cudaGetLastError();
}

cudaError_t launch_diff_prep(const DiffPrepArgs& a, int rows, bool kv_bf16, cudaStream_t s) {
  const int nvec = 2 * (a.H + a.G);
  const int warps = std::max(2, std::min(8, nvec));
  const size_t smem = (size_t)std::max(1, a.rot_dims) * sizeof(float);
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  const dim3 grid(rows, rows <= 64 ? (nvec + warps - 1) / warps : 1);  // few rows: a row's vectors spread over several CTAs
  if (kv_bf16) return launch_k(diff_prep_kernel<bf16>, grid, dim3(warps * 32), smem, s, a);
  return launch_k(diff_prep_kernel<float>, grid, dim3(warps * 32), smem, s, a);
}

bool diff_attn_tiled(int DK, int DV) {
  return (DK == 32 && (DV == 32 || DV == 64)) || (DK == 64 && (DV == 64 || DV == 128)) || (DK == 128 && DV == 128);
}

size_t diff_attn_cta_smem(int DK, int DV) {
  return (size_t)(2 * DK + DIFF_CTA_WARPS * 2 * DV + DIFF_CTA_WARPS * 4 + 32) * sizeof(float);
}

bool diff_attn_supported(int DK, int DV) { return diff_attn_cta_smem(DK, DV) <= 200 * 1024 && DK <= 12 * 1024 / 4; }

bool diff_attn_decode_shape(int DK, int DV, int rep) { return diff_attn_tiled(DK, DV) && (rep == 1 || rep == 2 || rep == 4); }

size_t diff_attn_part_floats(int max_rows, int H, int DV) { return (size_t)std::max(max_rows, DIFF_DEC_CTAS) * H * 2 * DV; }

cudaError_t launch_diff_attn(const DiffAttnArgs& a, bool kv_bf16, float* part_o, float* part_ml, cudaStream_t s) {
  static const int tile_min = [] { const char* v = getenv("L3_DIFF_TILE_MIN"); return v ? atoi(v) : DIFF_DEC_MAX_L + 1; }();
  static const bool dec_on = !(getenv("L3_DIFF_DECODE") && atoi(getenv("L3_DIFF_DECODE")) == 0);
  if (tile_min > 0 && a.L >= tile_min && diff_attn_tiled(a.DK, a.DV))
    return kv_bf16 ? launch_tile_t<bf16>(a, s) : launch_tile_t<float>(a, s);
  if (dec_on && part_o && a.L <= DIFF_DEC_MAX_L && diff_attn_decode_shape(a.DK, a.DV, a.H / a.G)) {
    // enough CTAs for two per SM; a split has at least 128 keys of the longest range a row can see (a batch of 32 per warp)
    const int rows = a.B * a.L, keys = a.window > 0 ? std::min(a.window, a.M) : a.M;
    const int nsplit = std::max(1, std::min(std::min(64, keys / (DEC_WARPS * 32)), DIFF_DEC_CTAS / std::max(1, rows * a.G)));
    return kv_bf16 ? launch_decode_t<bf16>(a, nsplit, part_o, part_ml, s) : launch_decode_t<float>(a, nsplit, part_o, part_ml, s);
  }
  const size_t smem = diff_attn_cta_smem(a.DK, a.DV);
  const dim3 grid((unsigned)((size_t)a.B * a.L * a.H));
  if (kv_bf16) {
    auto kern = attn_diff_cta_kernel<bf16>;
    if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
    return launch_k(kern, grid, dim3(DIFF_CTA_WARPS * 32), smem, s, a);
  }
  auto kern = attn_diff_cta_kernel<float>;
  if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
  return launch_k(kern, grid, dim3(DIFF_CTA_WARPS * 32), smem, s, a);
}
