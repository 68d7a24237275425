// Row kernels of the state-space (L3_MIX_SSD) and gated-linear (L3_MIX_GLA) mixers, the shared output stage of the
// recurrent mixers of pre-norm stacks, and two small stream kernels.  Everything fp32.
//
//  * ssd_prep_kernel     a CTA per token: causal convolution with bias + silu over the x | B | C channels (inputs ahead of
//                        the call from the slot's tail), dt = softplus(dt + bias), decay = exp(-exp(A_log) dt) per head,
//                        and the recurrence's operands: keys B, queries C, values dt * x, plus x itself for the skip term
//  * gla_prep_kernel     q * dim^(-1/2) and the per-channel decay sigmoid(z + b)^(1 / tau) = exp(-softplus(-(z + b)) / tau)
//  * mix_out_kernel      skip term, gate (ahead of or behind the norm, sigmoid or silu), RMS norm in groups, weight, scale;
//                        writes into a slice of a wider row so that two mixers side by side share one output projection
//  * softcap_kernel      c tanh(x / c)
//  * concat_rows_kernel  [a | b] row by row (+ bf16 mirror): the input of the looped block's entry projection
#include <algorithm>

#include "common.cuh"
#include "mixer.h"

namespace {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

__global__ void __launch_bounds__(256) ssd_prep_kernel(SsdPrepArgs a) {
  extern __shared__ float sdt[];  // [H] dt of this row
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int b = r / a.L, t = r - b * a.L;
  const int inner = a.H * a.DV, gn = a.G * a.N, C = inner + 2 * gn, T1 = a.taps - 1;
  const float* row = a.proj + (size_t)r * a.ld;
  for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
    const float dt = softplus_f(row[a.dt_off + h] + a.dt_bias[h]);
    sdt[h] = dt;
    if (blockIdx.y == 0) {
      const float ld = -expf(a.A_log[h]) * dt;
      a.decay_out[(size_t)r * a.H + h] = expf(ld);
      if (a.logdecay_out) a.logdecay_out[(size_t)r * a.H + h] = ld;
    }
  }
  __syncthreads();
  float* tail = a.conv_tail + (size_t)b * C * T1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float acc = a.conv_b ? a.conv_b[c] : 0.f;
    for (int j = 0; j < a.taps; ++j) {
      const int tt = t - T1 + j;  // time inside this call; negative: from the tail
      const float xin = tt >= 0 ? a.proj[(size_t)(b * a.L + tt) * a.ld + a.xbc_off + c] : tail[(size_t)c * T1 + (T1 + tt)];
      acc = fmaf(a.conv_w[(size_t)c * a.taps + j], xin, acc);
      // a call of one token moves the tail on here: this thread alone reads and writes channel c's entries
      if (a.update_tail && j >= 1 && j <= T1) tail[(size_t)c * T1 + (j - 1)] = xin;
    }
    const float s = silu_ref(acc);
    if (c < inner) {
      a.x_out[(size_t)r * inner + c] = s;
      a.v_out[(size_t)r * inner + c] = sdt[c / a.DV] * s;
    } else if (c < inner + gn) {
      a.k_out[(size_t)r * gn + (c - inner)] = s;
    } else {
      a.q_out[(size_t)r * gn + (c - inner - gn)] = s;
    }
  }
}

__global__ void gla_prep_kernel(const float* __restrict__ q, int ld, float q_mul, const float* __restrict__ z, int ld_z,
                                const float* __restrict__ bias, float inv_tau, int64_t rows, int n, float* __restrict__ q_out,
                                float* __restrict__ g_out) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * n) return;
  const int64_t r = i / n;
  const int c = (int)(i - r * n);
  q_out[i] = q[r * ld + c] * q_mul;
  const float zz = z[r * ld_z + c] + (bias ? bias[c] : 0.f);
  g_out[i] = expf(-softplus_f(-zz) * inv_tau);  // log sigmoid(z) = -softplus(-z)
}

// wpg warps share a group (wpg in 1, 2, 4, 8); a CTA of 8 warps holds 8 / wpg groups, blockIdx.y walks the groups
__global__ void __launch_bounds__(256) mix_out_kernel(MixOutArgs a, int wpg) {
  __shared__ float red[8];
  pdl_launch();
  pdl_wait();
  const size_t r = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gpc = 8 / wpg, g = blockIdx.y * gpc + warp / wpg, sub = warp % wpg;
  const bool live = g * a.group < a.n;
  const float* orow = a.o + r * a.n;
  const float* grow = a.gate ? a.gate + r * a.ld_gate : nullptr;
  const float* xrow = a.skip_d ? a.skip_x + r * a.n : nullptr;
  auto act = [&](float z) { return a.gate_act ? z * sigmoid_f(z) : sigmoid_f(z); };
  auto val = [&](int i) {
    float y = orow[i];
    if (xrow) y = fmaf(a.skip_d[i / a.DV], xrow[i], y);
    if (grow && a.pre_gate) y *= act(grow[i]);
    return y;
  };
  const int base = g * a.group;
  float ss = 0.f;
  if (live)
    for (int i = sub * 32 + lane; i < a.group; i += wpg * 32) { const float y = val(base + i); ss = fmaf(y, y, ss); }
  ss = warp_sum(ss);
  if (wpg > 1) {
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    ss = 0.f;
    for (int w = 0; w < wpg; ++w) ss += red[(warp / wpg) * wpg + w];
  }
  if (!live) return;
  const float rinv = 1.0f / sqrtf(ss / (float)a.group + a.eps);
  for (int i = sub * 32 + lane; i < a.group; i += wpg * 32) {
    const int c = base + i;
    float v = val(c) * rinv * a.w[c % a.wlen];
    if (grow && !a.pre_gate) v *= act(grow[c]);
    v *= a.out_scale;
    a.out[r * a.ld_out + c] = v;
    if (a.out16) a.out16[r * a.ld_out + c] = __float2bfloat16_rn(v);
  }
}

__global__ void softcap_kernel(float* __restrict__ x, int64_t n, float cap) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

__global__ void concat_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, int64_t rows, int D,
                                   float* __restrict__ out, bf16* __restrict__ out16) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * 2 * D) return;
  const int64_t r = i / (2 * D);
  const int c = (int)(i - r * 2 * D);
  const float v = c < D ? a[r * D + c] : b[r * D + (c - D)];
  out[i] = v;
  if (out16) out16[i] = __float2bfloat16_rn(v);
}

}  // namespace

cudaError_t launch_ssd_prep(const SsdPrepArgs& a, int rows, cudaStream_t s) {
  if (a.update_tail && a.L != 1) return cudaErrorInvalidValue;
  const int C = a.H * a.DV + 2 * a.G * a.N;
  const int parts = rows <= 8 ? std::max(1, std::min(32, C / 256)) : 1;  // few rows: a row's channels spread over CTAs
  return launch_k(ssd_prep_kernel, dim3(rows, parts), dim3(256), (size_t)a.H * sizeof(float), s, a);
}

cudaError_t launch_gla_prep(const float* q, int ld, float q_mul, const float* z, int ld_z, const float* bias, float tau, int rows,
                            int n, float* q_out, float* g_out, cudaStream_t s) {
  const int64_t tot = (int64_t)rows * n;
  return launch_k(gla_prep_kernel, dim3((unsigned)((tot + 255) / 256)), dim3(256), 0, s, q, ld, q_mul, z, ld_z, bias, 1.0f / tau,
                  (int64_t)rows, n, q_out, g_out);
}

cudaError_t launch_mix_out(const MixOutArgs& a, int rows, cudaStream_t s) {
  if (a.group < 1 || a.n % a.group != 0) return cudaErrorInvalidValue;
  const int groups = a.n / a.group;
  const int wpg = a.group >= 1024 ? 8 : a.group >= 512 ? 4 : a.group >= 256 ? 2 : 1;  // warps per group
  const int gpc = 8 / wpg;
  return launch_k(mix_out_kernel, dim3(rows, (groups + gpc - 1) / gpc), dim3(256), 0, s, a, wpg);
}

cudaError_t launch_softcap(float* x, int64_t n, float cap, cudaStream_t s) {
  return launch_k(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, x, n, cap);
}

cudaError_t launch_concat_rows(const float* a, const float* b, int rows, int D, float* out, bf16* out16, cudaStream_t s) {
  const int64_t tot = (int64_t)rows * 2 * D;
  return launch_k(concat_rows_kernel, dim3((unsigned)((tot + 255) / 256)), dim3(256), 0, s, a, b, (int64_t)rows, D, out, out16);
}
