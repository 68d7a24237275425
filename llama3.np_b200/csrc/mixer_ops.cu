// Row kernels around the token mixers of layer-list decoders (layerlist.cu): everything here is fp32 - norms,
// gates, the residual sum - whatever the model's weight type is.
//
//  * resid_postnorm_kernel   x += mult * y / rms(y) * w        (norm on the sublayer's OUTPUT), emits the bf16
//                            mirror of the new residual row for the tensor-core projections that read it next
//  * gated_rmsnorm_kernel    out = o / rms_group(o) * w * sigmoid(gate)   over the whole row or per head
//  * qk_norm_cache_kernel    RMS norm over the WHOLE q / k projection, append k (normalised) and the raw k
//                            (the values of this attention) to the KV cache
//  * side_mul_kernel         act(g) * E[token, layer slice]    (per-layer token input)
//  * delta_prep_kernel       short causal convolutions + silu, unit-length q / k, decay and write strength of
//                            the gated delta rule; conv_tail_kernel moves the convolutions' tails on (a call of one
//                            token lets delta_prep_kernel do that itself)
//  * rmsnorm_rows_kernel     plain RMS norm of chosen rows, any width (ahead of the LM head)
//  * to_bf16_kernel          bf16 mirror of fp32 rows
#include <algorithm>

#include "common.cuh"
#include "mixer.h"

namespace {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// sum over the CTA (every thread gets the total; same order of additions in every thread)
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // red may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nw; ++w) t += red[w];
  return t;
}

__global__ void __launch_bounds__(256) resid_postnorm_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                             const float* __restrict__ w, float mult, float eps, int D,
                                                             bf16* __restrict__ x16) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const size_t r = blockIdx.x;
  const float* yr = y + r * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) { const float v = yr[i]; ss = fmaf(v, v, ss); }
  const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = x[r * D + i] + mult * (yr[i] * rinv * w[i]);
    x[r * D + i] = v;
    if (x16) x16[r * D + i] = __float2bfloat16_rn(v);
  }
}

// group == O: one norm over the row (block-wide sum); group < O: one norm per group (a warp per group).
__global__ void __launch_bounds__(256) gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                                                            int ld_gate, const float* __restrict__ w, int wlen, int group,
                                                            float eps, int O, float* __restrict__ out,
                                                            bf16* __restrict__ out16) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const size_t r = blockIdx.x;
  const float* orow = o + r * O;
  const float* grow = gate + r * ld_gate;
  if (group >= O) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < O; i += blockDim.x) { const float v = orow[i]; ss = fmaf(v, v, ss); }
    const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)O + eps);
    for (int i = threadIdx.x; i < O; i += blockDim.x) {
      const float v = orow[i] * rinv * w[i % wlen] * sigmoid_f(grow[i]);
      out[r * O + i] = v;
      if (out16) out16[r * O + i] = __float2bfloat16_rn(v);
    }
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int g = warp; g * group < O; g += nw) {
    const int base = g * group;
    float ss = 0.f;
    for (int i = lane; i < group; i += 32) { const float v = orow[base + i]; ss = fmaf(v, v, ss); }
    const float rinv = 1.0f / sqrtf(warp_sum(ss) / (float)group + eps);
    for (int i = lane; i < group; i += 32) {
      const float v = orow[base + i] * rinv * w[(base + i) % wlen] * sigmoid_f(grow[base + i]);
      out[r * O + base + i] = v;
      if (out16) out16[r * O + base + i] = __float2bfloat16_rn(v);
    }
  }
}

template <typename KVT>
__global__ void __launch_bounds__(256) qk_norm_cache_kernel(QkNormArgs a) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int b = r / a.L, t = r - b * a.L;
  const int pos = *a.pos_ptr + t;
  const float* row = a.proj + (size_t)r * a.ld;
  const int nq = a.HN * a.HD, nk = a.KVHN * a.HD;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = row[i]; ss = fmaf(v, v, ss); }
  const float rq = 1.0f / sqrtf(block_sum(ss, red) / (float)nq + a.eps);
  for (int i = threadIdx.x; i < nq; i += blockDim.x) a.q_out[(size_t)r * nq + i] = row[i] * rq * a.wq[i];
  const float* krow = row + a.k_off;
  ss = 0.f;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = krow[i]; ss = fmaf(v, v, ss); }
  const float rk = 1.0f / sqrtf(block_sum(ss, red) / (float)nk + a.eps);
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const int h = i / a.HD, d = i - h * a.HD;
    const size_t ci = (((size_t)b * a.KVHN + h) * a.M + pos) * a.HD + d;
    const float v = krow[i];
    ((KVT*)a.cache_k)[ci] = from_f32<KVT>(v * rk * a.wk[i]);
    ((KVT*)a.cache_v)[ci] = from_f32<KVT>(v);
  }
}

template <typename WT>
__global__ void side_mul_kernel(float* __restrict__ g, int n, int rows, const WT* __restrict__ table, int table_ld,
                                int col0, const int32_t* __restrict__ ids, int ids_ld, int ids_off, int L, int vocab,
                                int act, bf16* __restrict__ out16) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)rows * n) return;
  const int r = (int)(i / n), j = (int)(i - (int64_t)r * n);
  const int b = r / L, t = r - b * L;
  const int id = min(max(ids[(size_t)b * ids_ld + ids_off + t], 0), vocab - 1);
  const float z = g[i];
  const float a = act == GLU_GELU_TANH ? gelu_tanh_ref(z) : silu_ref(z);
  const float v = a * to_f32(table[(size_t)id * table_ld + col0 + j]);
  g[i] = v;
  if (out16) out16[i] = __float2bfloat16_rn(v);
}

// Input of channel c at time t' < 0 of the call comes from the tail [C][taps-1] (oldest first) that earlier calls left.
// The work of a token row is a list of items - a q or k head (convolution + silu + unit length), a v head (convolution +
// silu), a head's decays, the write strengths - and every warp of the row's CTAs (blockIdx.y of them: few rows spread a
// row over several CTAs) takes items round-robin; no item needs another warp.
__global__ void __launch_bounds__(256) delta_prep_kernel(DeltaPrepArgs a) {
  extern __shared__ float sm[];  // [warps][DK] the convolved head a warp works on
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int b = r / a.L, t = r - b * a.L;
  const int nq = a.G * a.DK, nv = a.H * a.DV, C = 2 * nq + nv, T1 = a.taps - 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float* tail = a.conv_tail + (size_t)b * C * T1;
  float* buf = sm + (size_t)warp * a.DK;
  auto conv = [&](int c) {
    float acc = 0.f;
    for (int j = 0; j < a.taps; ++j) {
      const int tt = t - T1 + j;  // time inside this call; negative: from the tail
      const float xin = tt >= 0 ? a.proj[(size_t)(b * a.L + tt) * a.ld + c] : tail[(size_t)c * T1 + (T1 + tt)];
      acc = fmaf(a.conv_w[(size_t)c * a.taps + j], xin, acc);
      // a call of one token moves the tail on here: this thread alone reads and writes channel c's entries
      if (a.update_tail && j >= 1 && j <= T1) tail[(size_t)c * T1 + (j - 1)] = xin;
    }
    return silu_ref(acc);
  };
  const int n_items = 2 * a.G + 2 * a.H + 1;
  for (int item = blockIdx.y * nw + warp; item < n_items; item += gridDim.y * nw) {
    if (item < 2 * a.G) {  // a q or k head: unit length; q also times DK^-1/2
      float ss = 0.f;
      for (int i = lane; i < a.DK; i += 32) { const float v = conv(item * a.DK + i); buf[i] = v; ss = fmaf(v, v, ss); }
      float rinv = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
      const bool is_q = item < a.G;
      if (is_q) rinv *= 1.0f / sqrtf((float)a.DK);
      float* dst = is_q ? a.q_out + (size_t)r * nq + (size_t)item * a.DK : a.k_out + (size_t)r * nq + (size_t)(item - a.G) * a.DK;
      for (int i = lane; i < a.DK; i += 32) dst[i] = buf[i] * rinv;  // a lane reads back what it wrote itself
    } else if (item < 2 * a.G + a.H) {
      const int h = item - 2 * a.G;
      for (int i = lane; i < a.DV; i += 32) a.v_out[(size_t)r * nv + (size_t)h * a.DV + i] = conv(2 * nq + h * a.DV + i);
    } else if (item < 2 * a.G + 2 * a.H) {  // decay per key channel of a head
      const int h = item - 2 * a.G - a.H;
      const float rate = expf(a.A_log[h]);
      for (int i = lane; i < a.DK; i += 32) {
        const int c = h * a.DK + i;
        a.decay_out[(size_t)r * a.H * a.DK + c] = expf(-rate * softplus_f(a.dt_in[(size_t)r * a.ld_dt + c] + a.dt_bias[c]));
      }
    } else {
      for (int h = lane; h < a.H; h += 32) a.beta_out[(size_t)r * a.H + h] = sigmoid_f(a.proj[(size_t)r * a.ld + a.beta_off + h]);
    }
  }
}

// new tail[r] = element L + r of (old tail | the call's L inputs); ascending r never reads what it wrote
__global__ void conv_tail_kernel(float* __restrict__ tail, const float* __restrict__ proj, int ld, int B, int L, int C, int T1) {
  pdl_launch();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * C) return;
  const int b = i / C, c = i - b * C;
  float* tl = tail + ((size_t)b * C + c) * T1;
  for (int r = 0; r < T1; ++r) {
    const int v = L + r;  // index into the virtual sequence
    tl[r] = v < T1 ? tl[v] : proj[(size_t)(b * L + (v - T1)) * ld + c];
  }
}

// out[r] = x[source row of r] / rms * w, any D; source row = src_rows[r] or r * src_mul + src_add; groups > 1: the row is
// cut into that many equal parts, each over its own root mean square
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps,
                                                           int D, int src_mul, int src_add, const int32_t* __restrict__ src_rows,
                                                           int groups, float* __restrict__ out, bf16* __restrict__ out16) {
  __shared__ float red[32];
  __shared__ float rg[128];
  pdl_launch();
  pdl_wait();
  const size_t r = blockIdx.x;
  const float* xr = x + (src_rows ? (size_t)src_rows[r] : r * src_mul + src_add) * D;
  const int gs = D / groups;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  const int wpg = max(1, nw / groups), gpr = nw / wpg;  // warps per group, groups settled per round
  for (int g0 = 0; g0 < groups; g0 += gpr) {
    const int g = g0 + warp / wpg, sub = warp % wpg;
    float ss = 0.f;
    if (g < groups && warp < gpr * wpg)
      for (int i = sub * 32 + lane; i < gs; i += wpg * 32) { const float v = xr[g * gs + i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    __syncthreads();
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (g < groups && warp < gpr * wpg && sub == 0 && lane == 0) {
      float tot = 0.f;
      for (int w = 0; w < wpg; ++w) tot += red[warp + w];
      rg[g] = 1.0f / sqrtf(tot / (float)gs + eps);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = xr[i] * rg[i / gs] * w[i];
    out[r * D + i] = v;
    if (out16) out16[r * D + i] = __float2bfloat16_rn(v);
  }
}

__global__ void to_bf16_kernel(const float* __restrict__ in, int64_t n, bf16* __restrict__ out) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16_rn(in[i]);
}

__global__ void add_one_kernel(float* __restrict__ p, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] += 1.0f;
}

}  // namespace

static int row_threads(int n) { return n >= 1024 ? 256 : n >= 256 ? 128 : 64; }

cudaError_t launch_resid_postnorm(float* x, const float* y, const float* w, float mult, float eps, int rows, int D,
                                  bf16* x16, cudaStream_t s) {
  return launch_k(resid_postnorm_kernel, dim3(rows), dim3(row_threads(D)), 0, s, x, y, w, mult, eps, D, x16);
}

cudaError_t launch_gated_rmsnorm(const float* o, const float* gate, int ld_gate, const float* w, int wlen, int group,
                                 float eps, int rows, int O, float* out, bf16* out16, cudaStream_t s) {
  const int threads = group >= O ? row_threads(O) : std::min(256, std::max(32, 32 * (O / group)));
  return launch_k(gated_rmsnorm_kernel, dim3(rows), dim3(threads), 0, s, o, gate, ld_gate, w, wlen, group, eps, O, out, out16);
}

cudaError_t launch_qk_norm_cache(const QkNormArgs& a, int rows, bool kv_bf16, cudaStream_t s) {
  const int threads = row_threads(a.HN * a.HD);
  if (kv_bf16) return launch_k(qk_norm_cache_kernel<bf16>, dim3(rows), dim3(threads), 0, s, a);
  return launch_k(qk_norm_cache_kernel<float>, dim3(rows), dim3(threads), 0, s, a);
}

cudaError_t launch_side_mul(float* g, int n, int rows, const void* table, bool table_bf16, int table_ld, int col0,
                            const int32_t* ids, int ids_ld, int ids_off, int L, int vocab, int act, bf16* out16,
                            cudaStream_t s) {
  const int64_t tot = (int64_t)rows * n;
  const dim3 grid((unsigned)((tot + 255) / 256));
  if (table_bf16)
    return launch_k(side_mul_kernel<bf16>, grid, dim3(256), 0, s, g, n, rows, (const bf16*)table, table_ld, col0, ids, ids_ld, ids_off, L, vocab, act, out16);
  return launch_k(side_mul_kernel<float>, grid, dim3(256), 0, s, g, n, rows, (const float*)table, table_ld, col0, ids, ids_ld, ids_off, L, vocab, act, out16);
}

cudaError_t launch_delta_prep(const DeltaPrepArgs& a, int rows, cudaStream_t s) {
  if (a.update_tail && a.L != 1) return cudaErrorInvalidValue;
  const size_t smem = (size_t)8 * a.DK * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  const int items = 2 * a.G + 2 * a.H + 1;
  const int parts = rows <= 8 ? std::max(1, std::min(32, (items + 7) / 8)) : 1;  // few rows: a row's items spread over CTAs
  return launch_k(delta_prep_kernel, dim3(rows, parts), dim3(256), smem, s, a);
}

cudaError_t launch_conv_tail(float* tail, const float* proj, int ld, int B, int L, int C, int T1, cudaStream_t s) {
  if (T1 <= 0) return cudaSuccess;
  return launch_k(conv_tail_kernel, dim3((B * C + 127) / 128), dim3(128), 0, s, tail, proj, ld, B, L, C, T1);
}

cudaError_t launch_rmsnorm_rows(const float* x, const float* w, float eps, int rows, int D, int src_mul, int src_add,
                                const int32_t* src_rows, float* out, bf16* out16, cudaStream_t s, int groups) {
  if (groups < 1 || groups > 128 || D % groups != 0) return cudaErrorInvalidValue;
  return launch_k(rmsnorm_rows_kernel, dim3(rows), dim3(row_threads(D)), 0, s, x, w, eps, D, src_mul, src_add, src_rows, groups, out, out16);
}

cudaError_t launch_to_bf16(const float* in, int64_t n, bf16* out, cudaStream_t s) {
  return launch_k(to_bf16_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, in, n, out);
}

cudaError_t launch_add_one(float* p, int n, cudaStream_t s) {
  add_one_kernel<<<(n + 255) / 256, 256, 0, s>>>(p, n);
  return cudaGetLastError();
}
