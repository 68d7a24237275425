// Row kernels of pre-norm layer-list decoders (layerlist.cu): everything fp32.
//
//  * prenorm_shift_kernel   h = x / rms(x) * w, optionally mixed with the previous token's h (token shift):
//                           out = h + (h_prev - h) * shift.  The previous token's h is the un-shifted one; for the
//                           first token of a call it comes from the slot's state, which the same CTA then replaces
//                           by the h of the call's last token (so no other CTA reads or writes that state row).
//  * scale_add_rows_kernel  x = x * mul + vec   (embedding multiplier, the per-pass vector of a looped block)
//  * mingru_scan_kernel     the element-wise gated recurrence over the tokens of a call, one thread per channel;
//                           prompts run as mingru_gates_kernel (all gates at once) + mingru_chain_kernel (S <- a S + b)
#include "common.cuh"
#include "mixer.h"

namespace {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nw; ++w) t += red[w];
  return t;
}

// 1 / rms of every one of `groups` equal consecutive parts of a row, into out[groups] (shared memory).  The CTA's warps
// share the groups: with fewer groups than warps several warps sum one group, and a round of the loop settles as many
// groups as fit (one round for up to 8 groups of a 256-thread CTA).
__device__ __forceinline__ void row_rinv(const float* __restrict__ row, int D, int groups, float eps, float* red, float* out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  const int gs = D / groups;
  const int wpg = max(1, nw / groups), gpr = nw / wpg;  // warps per group, groups per round
  for (int g0 = 0; g0 < groups; g0 += gpr) {
    const int g = g0 + warp / wpg, sub = warp % wpg;
    float ss = 0.f;
    if (g < groups && warp < gpr * wpg)
      for (int i = sub * 32 + lane; i < gs; i += wpg * 32) { const float v = row[g * gs + i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    __syncthreads();  // red may still be read from the previous round
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (g < groups && warp < gpr * wpg && sub == 0 && lane == 0) {
      float tot = 0.f;
      for (int w = 0; w < wpg; ++w) tot += red[warp + w];
      out[g] = 1.0f / sqrtf(tot / (float)gs + eps);
    }
  }
  __syncthreads();
}

constexpr int NORM_GROUPS_MAX = 128;

__global__ void __launch_bounds__(256) prenorm_shift_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps,
                                                            const float* __restrict__ shift, float* __restrict__ hprev, int L,
                                                            int D, int groups, float* __restrict__ out, bf16* __restrict__ out16) {
  __shared__ float red[32];
  __shared__ float rc[NORM_GROUPS_MAX], rp[NORM_GROUPS_MAX], rl[NORM_GROUPS_MAX];
  pdl_launch();
  pdl_wait();
  const size_t r = blockIdx.x;
  const int b = (int)(r / L), t = (int)(r - (size_t)b * L);
  const int gs = D / groups;
  const float* xr = x + r * D;
  row_rinv(xr, D, groups, eps, red, rc);
  if (!shift) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      const float h = xr[i] * rc[i / gs] * w[i];
      out[r * D + i] = h;
      if (out16) out16[r * D + i] = __float2bfloat16_rn(h);
    }
    return;
  }
  const float* xp = xr - D;  // previous token of the same sequence (t > 0)
  if (t > 0) row_rinv(xp, D, groups, eps, red, rp);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float h = xr[i] * rc[i / gs] * w[i];
    const float prev = t > 0 ? xp[i] * rp[i / gs] * w[i] : hprev[(size_t)b * D + i];
    const float v = h + (prev - h) * shift[i];
    out[r * D + i] = v;
    if (out16) out16[r * D + i] = __float2bfloat16_rn(v);
  }
  if (t == 0) {  // this CTA alone touches hprev[b]: read above, replaced here
    const float* xl = xr + (size_t)(L - 1) * D;
    __syncthreads();  // every thread has read its hprev entries
    if (L > 1) row_rinv(xl, D, groups, eps, red, rl);
    const float* rlast = L > 1 ? rl : rc;
    for (int i = threadIdx.x; i < D; i += blockDim.x) hprev[(size_t)b * D + i] = xl[i] * rlast[i / gs] * w[i];
  }
}

__global__ void scale_add_rows_kernel(float* __restrict__ x, float mul, const float* __restrict__ vec, int64_t n, int D) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  x[i] = fmaf(x[i], mul, vec ? vec[i % D] : 0.f);
}

// One thread per (sequence, channel); the loads of the next GRU_AHEAD tokens are in flight while a token's chain of
// dependent operations runs, so that the chain, not the memory latency, sets the pace.
constexpr int GRU_AHEAD = 8;
__global__ void __launch_bounds__(128) mingru_scan_kernel(const float* __restrict__ proj, int ld, int z_off, int x_off, int g_off,
                                                          const float* __restrict__ bias, float* __restrict__ S, int L, int n,
                                                          float* __restrict__ out, bf16* __restrict__ out16) {
  pdl_launch();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (c >= n) return;
  const float bz = bias[c], bx = bias[n + c];
  float s = S[(size_t)b * n + c];
  const float* p = proj + (size_t)b * L * ld;
  // a ring of GRU_AHEAD tokens in registers: the loads of token t + GRU_AHEAD are issued while token t is computed
  float zq[GRU_AHEAD], uq[GRU_AHEAD], gq[GRU_AHEAD];
#pragma unroll
  for (int i = 0; i < GRU_AHEAD; ++i)
    if (i < L) { const float* pn = p + (size_t)i * ld; zq[i] = pn[z_off + c]; uq[i] = pn[x_off + c]; gq[i] = pn[g_off + c]; }
  for (int t0 = 0; t0 < L; t0 += GRU_AHEAD) {
#pragma unroll
    for (int i = 0; i < GRU_AHEAD; ++i) {
      const int t = t0 + i;
      if (t >= L) break;
      const float zc = zq[i], uc = uq[i], gc = gq[i];
      if (t + GRU_AHEAD < L) {
        const float* pn = p + (size_t)(t + GRU_AHEAD) * ld;
        zq[i] = pn[z_off + c]; uq[i] = pn[x_off + c]; gq[i] = pn[g_off + c];
      }
      const float z = sigmoid_f(zc + bz);
      const float u = uc + bx;
      const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
      s = (1.0f - z) * s + z * cand;
      const float o = s * (gc * sigmoid_f(gc));
      const size_t oi = ((size_t)b * L + t) * n + c;
      out[oi] = o;
      if (out16) out16[oi] = __float2bfloat16_rn(o);
    }
  }
  S[(size_t)b * n + c] = s;
}

// Prompts: the gates of all tokens at once (every (token, channel) on its own), in place over the projection:
// z column <- 1 - z, x column <- z * candidate, g column <- silu(g) ...
__global__ void mingru_gates_kernel(float* __restrict__ proj, int ld, int z_off, int x_off, int g_off,
                                    const float* __restrict__ bias, int64_t rows, int n) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * n) return;
  const int64_t r = i / n;
  const int c = (int)(i - r * n);
  float* p = proj + r * ld;
  const float z = sigmoid_f(p[z_off + c] + bias[c]);
  const float u = p[x_off + c] + bias[n + c];
  const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
  const float g = p[g_off + c];
  p[z_off + c] = 1.0f - z;
  p[x_off + c] = z * cand;
  p[g_off + c] = g * sigmoid_f(g);
}

// ... and then the chain alone: S <- a S + b per token, a thread per (sequence, channel), GRU_AHEAD tokens of loads in flight
__global__ void __launch_bounds__(128) mingru_chain_kernel(const float* __restrict__ proj, int ld, int z_off, int x_off, int g_off,
                                                           float* __restrict__ S, int L, int n, float* __restrict__ out,
                                                           bf16* __restrict__ out16) {
  pdl_launch();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (c >= n) return;
  float s = S[(size_t)b * n + c];
  const float* p = proj + (size_t)b * L * ld + c;
  float aq[GRU_AHEAD], bq[GRU_AHEAD], gq[GRU_AHEAD];
  const int Lfull = L / GRU_AHEAD * GRU_AHEAD;
  if (Lfull) {
#pragma unroll
    for (int i = 0; i < GRU_AHEAD; ++i) { const float* pn = p + (size_t)i * ld; aq[i] = pn[z_off]; bq[i] = pn[x_off]; gq[i] = pn[g_off]; }
  }
  for (int t0 = 0; t0 < Lfull; t0 += GRU_AHEAD) {
    const bool more = t0 + GRU_AHEAD < Lfull;
#pragma unroll
    for (int i = 0; i < GRU_AHEAD; ++i) {
      const float a = aq[i], bb = bq[i], g = gq[i];
      if (more) { const float* pn = p + (size_t)(t0 + GRU_AHEAD + i) * ld; aq[i] = pn[z_off]; bq[i] = pn[x_off]; gq[i] = pn[g_off]; }
      s = a * s + bb;
      const float o = s * g;
      const size_t oi = ((size_t)b * L + t0 + i) * n + c;
      out[oi] = o;
      if (out16) out16[oi] = __float2bfloat16_rn(o);
    }
  }
  for (int t = Lfull; t < L; ++t) {
    const float* pn = p + (size_t)t * ld;
    s = pn[z_off] * s + pn[x_off];
    const float o = s * pn[g_off];
    const size_t oi = ((size_t)b * L + t) * n + c;
    out[oi] = o;
    if (out16) out16[oi] = __float2bfloat16_rn(o);
  }
  S[(size_t)b * n + c] = s;
}

int row_threads(int D) { return D >= 1024 ? 256 : D >= 256 ? 128 : 64; }

}  // namespace

cudaError_t launch_prenorm_shift(const float* x, const float* w, float eps, const float* shift, float* hprev, int B, int L,
                                 int D, float* out, bf16* out16, cudaStream_t s, int groups) {
  if (groups < 1 || groups > NORM_GROUPS_MAX || D % groups != 0) return cudaErrorInvalidValue;
  return launch_k(prenorm_shift_kernel, dim3(B * L), dim3(row_threads(D)), 0, s, x, w, eps, shift, hprev, L, D, groups, out, out16);
}

cudaError_t launch_scale_add_rows(float* x, float mul, const float* vec, int rows, int D, cudaStream_t s) {
  const int64_t n = (int64_t)rows * D;
  return launch_k(scale_add_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, x, mul, vec, n, D);
}

cudaError_t launch_mingru_scan(float* proj, int ld, int z_off, int x_off, int g_off, const float* bias, float* S, int B,
                               int L, int n, float* out, bf16* out16, cudaStream_t s) {
  if (L > 16) {  // a prompt: gates in parallel, then the bare chain
    const int64_t tot = (int64_t)B * L * n;
    cudaError_t e = launch_k(mingru_gates_kernel, dim3((unsigned)((tot + 255) / 256)), dim3(256), 0, s, proj, ld, z_off, x_off, g_off,
                             bias, (int64_t)B * L, n);
    if (e != cudaSuccess) return e;
    return launch_k(mingru_chain_kernel, dim3((n + 127) / 128, B), dim3(128), 0, s, (const float*)proj, ld, z_off, x_off, g_off, S, L,
                    n, out, out16);
  }
  return launch_k(mingru_scan_kernel, dim3((n + 127) / 128, B), dim3(128), 0, s, proj, ld, z_off, x_off, g_off, bias, S, L, n, out,
                  out16);
}
