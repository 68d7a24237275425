// Row kernels of parallel layers (layerlist.cu, L3StackConfig::parallel): one norm per layer, both sublayers read it.
// Everything here is fp32; the bf16 mirrors feed the tensor-core projections.
//
//  * layernorm_rows_kernel    (x - mean) / sqrt(var + eps) * w over chosen rows (var = mean of the squared deviations);
//                             center = 0 gives the plain RMS norm.  The layers' norm1 and the final norm.
//  * canon_kernel             the causal convolution over time ahead of each sublayer, for both sublayers at once:
//                             out_s[t] = h[t] + sum_j w_s[:, j] h[t - T + 1 + j]; rows ahead of the call come from the
//                             slot's tail (the last T - 1 rows of h, moved on by conv_tail_kernel of mixer_ops.cu)
//  * polynorm_kernel          a N(z) + b N(z^2) + c N(z^3) + e over a token's feed-forward values, N = RMS norm
//  * parallel_combine_kernel  X_new = x + ls1 * y1 + ls2 * y2, stored as layer result i + 1, and the stream handed on:
//                             x = sum_j dwa[j] X_j over the embedding output and every layer result so far
#include <algorithm>

#include "common.cuh"
#include "mixer.h"

namespace {

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

__global__ void __launch_bounds__(256) layernorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps,
                                                             int D, int center, int src_mul, int src_add,
                                                             const int32_t* __restrict__ src_rows, float* __restrict__ out,
                                                             bf16* __restrict__ out16) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const size_t r = blockIdx.x;
  const float* xr = x + (src_rows ? (size_t)src_rows[r] : r * src_mul + src_add) * D;
  float mean = 0.f;
  if (center) {
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) s += xr[i];
    mean = block_sum(s, red) / (float)D;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) { const float v = xr[i] - mean; ss = fmaf(v, v, ss); }
  const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = (xr[i] - mean) * rinv * w[i];
    out[r * D + i] = v;
    if (out16) out16[r * D + i] = __float2bfloat16_rn(v);
  }
}

// one thread per (row, channel); w1 / w2 [T, D] (tap-major copies made at finalize), last tap = the current token;
// tail [maxB, D, T - 1], oldest first
__global__ void __launch_bounds__(256) canon_kernel(const float* __restrict__ h, const float* __restrict__ tail,
                                                    const float* __restrict__ w1, const float* __restrict__ w2, int L, int D, int T,
                                                    int64_t n, float* __restrict__ out1, bf16* __restrict__ out1_16,
                                                    float* __restrict__ out2, bf16* __restrict__ out2_16) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t r = i / D;
  const int c = (int)(i - r * D);
  const int b = (int)(r / L), t = (int)(r - (int64_t)b * L);
  const float cur = h[i];
  float a1 = cur, a2 = cur;
  for (int j = 0; j < T; ++j) {
    const int v = t - (T - 1) + j;  // row of this call, or (negative) a row of the tail
    const float hv = v >= 0 ? h[((int64_t)b * L + v) * D + c] : tail[((size_t)b * D + c) * (T - 1) + (T - 1 + v)];
    a1 = fmaf(w1[(size_t)j * D + c], hv, a1);
    if (out2) a2 = fmaf(w2[(size_t)j * D + c], hv, a2);
  }
  out1[i] = a1;
  if (out1_16) out1_16[i] = __float2bfloat16_rn(a1);
  if (out2) {
    out2[i] = a2;
    if (out2_16) out2_16[i] = __float2bfloat16_rn(a2);
  }
}

// the same for four adjacent channels per thread (D % 4 == 0): 16-byte loads and stores
__global__ void __launch_bounds__(256) canon4_kernel(const float* __restrict__ h, const float* __restrict__ tail,
                                                     const float* __restrict__ w1, const float* __restrict__ w2, int L, int D, int T,
                                                     int64_t n4, float* __restrict__ out1, bf16* __restrict__ out1_16,
                                                     float* __restrict__ out2, bf16* __restrict__ out2_16) {
  pdl_launch();
  pdl_wait();
  const int64_t i4 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i4 >= n4) return;
  const int D4 = D >> 2;
  const int64_t r = i4 / D4;
  const int c = (int)(i4 - r * D4) * 4;
  const int b = (int)(r / L), t = (int)(r - (int64_t)b * L);
  const float4 cur = *reinterpret_cast<const float4*>(h + r * D + c);
  float a1[4] = {cur.x, cur.y, cur.z, cur.w}, a2[4] = {cur.x, cur.y, cur.z, cur.w};
  for (int j = 0; j < T; ++j) {
    const int v = t - (T - 1) + j;
    float hv[4];
    if (v >= 0) {
      const float4 q = *reinterpret_cast<const float4*>(h + ((int64_t)b * L + v) * D + c);
      hv[0] = q.x; hv[1] = q.y; hv[2] = q.z; hv[3] = q.w;
    } else {
#pragma unroll
      for (int x = 0; x < 4; ++x) hv[x] = tail[((size_t)b * D + c + x) * (T - 1) + (T - 1 + v)];
    }
    const float4 k1 = *reinterpret_cast<const float4*>(w1 + (size_t)j * D + c);
    a1[0] = fmaf(k1.x, hv[0], a1[0]); a1[1] = fmaf(k1.y, hv[1], a1[1]); a1[2] = fmaf(k1.z, hv[2], a1[2]); a1[3] = fmaf(k1.w, hv[3], a1[3]);
    if (out2) {
      const float4 k2 = *reinterpret_cast<const float4*>(w2 + (size_t)j * D + c);
      a2[0] = fmaf(k2.x, hv[0], a2[0]); a2[1] = fmaf(k2.y, hv[1], a2[1]); a2[2] = fmaf(k2.z, hv[2], a2[2]); a2[3] = fmaf(k2.w, hv[3], a2[3]);
    }
  }
  const int64_t o = r * D + c;
  *reinterpret_cast<float4*>(out1 + o) = make_float4(a1[0], a1[1], a1[2], a1[3]);
  if (out1_16) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a1[0], a1[1]), hi = __floats2bfloat162_rn(a1[2], a1[3]);
    *reinterpret_cast<uint2*>(out1_16 + o) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  }
  if (out2) {
    *reinterpret_cast<float4*>(out2 + o) = make_float4(a2[0], a2[1], a2[2], a2[3]);
    if (out2_16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a2[0], a2[1]), hi = __floats2bfloat162_rn(a2[2], a2[3]);
      *reinterpret_cast<uint2*>(out2_16 + o) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

// Few rows (L <= NORM_CANON_MAX_L tokens per sequence, T <= NORM_CANON_MAX_T taps): norm, both convolutions and the tail's
// update in ONE launch.  A CTA per sequence: the rows' statistics first, then every thread walks its channels through the
// call's tokens with the last T - 1 normed inputs in registers (read from the tail, written back at the end).
constexpr int NORM_CANON_MAX_L = 8, NORM_CANON_MAX_T = 8;
__global__ void __launch_bounds__(1024) norm_canon_rows_kernel(float* __restrict__ x, const float* __restrict__ nw, float eps,
                                                              int center, float* __restrict__ tail, const float* __restrict__ w1,
                                                              const float* __restrict__ w2, int L, int D, int T,
                                                              float* __restrict__ out1, float* __restrict__ out2,
                                                              ParallelCombineArgs pre) {
  __shared__ float red[32];
  __shared__ float s_mean[NORM_CANON_MAX_L], s_rinv[NORM_CANON_MAX_L];
  pdl_launch();
  pdl_wait();
  const int b = blockIdx.x;
  float* xb = x + (size_t)b * L * D;
  if (pre.y1) {  // the previous layer's result and the stream it hands on, for this sequence's rows (as parallel_combine_kernel)
    for (int i = threadIdx.x; i < L * D; i += blockDim.x) {
      const size_t gi = (size_t)b * L * D + i;
      const int c = i % D;
      float v = xb[i];
      v = fmaf(pre.ls1 ? pre.ls1[c] : 1.0f, pre.y1[gi], v);
      if (pre.y2) v = fmaf(pre.ls2 ? pre.ls2[c] : 1.0f, pre.y2[gi], v);
      if (pre.Xs) {
        pre.Xs[(int64_t)pre.n_prev * pre.x_stride + gi] = v;
        float acc = 0.f;
        for (int j = 0; j < pre.n_prev; ++j) acc = fmaf(pre.dwa[j], pre.Xs[(int64_t)j * pre.x_stride + gi], acc);
        v = fmaf(pre.dwa[pre.n_prev], v, acc);
      }
      xb[i] = v;
    }
    __syncthreads();
  }
  for (int t = 0; t < L; ++t) {
    const float* xr = xb + (size_t)t * D;
    float mean = 0.f;
    if (center) {
      float s = 0.f;
      for (int i = threadIdx.x; i < D; i += blockDim.x) s += xr[i];
      mean = block_sum(s, red) / (float)D;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { const float v = xr[i] - mean; ss = fmaf(v, v, ss); }
    const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps);
    if (threadIdx.x == 0) { s_mean[t] = mean; s_rinv[t] = rinv; }
  }
  __syncthreads();
  const int T1 = T - 1;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float win[NORM_CANON_MAX_T];  // win[0 .. T - 2]: the last inputs, oldest first; win[T - 1]: the current one
    float k1[NORM_CANON_MAX_T], k2[NORM_CANON_MAX_T];
    float* tl = tail + ((size_t)b * D + c) * T1;
#pragma unroll
    for (int j = 0; j < NORM_CANON_MAX_T; ++j) {
      win[j] = j < T1 ? tl[j] : 0.f;
      k1[j] = j < T ? w1[(size_t)j * D + c] : 0.f;
      k2[j] = (w2 && j < T) ? w2[(size_t)j * D + c] : 0.f;
    }
    const float wn = nw[c];
    for (int t = 0; t < L; ++t) {
      const float hv = (xb[(size_t)t * D + c] - s_mean[t]) * s_rinv[t] * wn;
      float a1 = hv, a2 = hv;
#pragma unroll
      for (int j = 0; j < NORM_CANON_MAX_T; ++j) {
        if (j == T1) win[j] = hv;
        if (j < T) { a1 = fmaf(k1[j], win[j], a1); a2 = fmaf(k2[j], win[j], a2); }
      }
      out1[((size_t)b * L + t) * D + c] = a1;
      if (out2) out2[((size_t)b * L + t) * D + c] = a2;
#pragma unroll
      for (int j = 0; j + 1 < NORM_CANON_MAX_T; ++j) win[j] = win[j + 1];
    }
#pragma unroll
    for (int j = 0; j < NORM_CANON_MAX_T; ++j)
      if (j < T1) tl[j] = win[j];
  }
}

__global__ void __launch_bounds__(1024) polynorm_kernel(float* __restrict__ z, const float* __restrict__ coef, float eps, int n,
                                                       bf16* __restrict__ out16) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  float* zr = z + (size_t)blockIdx.x * n;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = zr[i], v2 = v * v, v3 = v2 * v;
    s2 += v2; s4 = fmaf(v2, v2, s4); s6 = fmaf(v3, v3, s6);
  }
  const float r1 = 1.0f / sqrtf(block_sum(s2, red) / (float)n + eps);
  const float r2 = 1.0f / sqrtf(block_sum(s4, red) / (float)n + eps);
  const float r3 = 1.0f / sqrtf(block_sum(s6, red) / (float)n + eps);
  const float a = coef[0] * r1, b = coef[1] * r2, c = coef[2] * r3, e = coef[3];
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = zr[i], v2 = v * v;
    const float o = fmaf(a, v, fmaf(b, v2, fmaf(c, v2 * v, e)));
    zr[i] = o;
    if (out16) out16[(size_t)blockIdx.x * n + i] = __float2bfloat16_rn(o);
  }
}

__global__ void __launch_bounds__(256) parallel_combine_kernel(float* __restrict__ x, const float* __restrict__ y1,
                                                               const float* __restrict__ y2, const float* __restrict__ ls1,
                                                               const float* __restrict__ ls2, float* __restrict__ Xs,
                                                               int64_t x_stride, const float* __restrict__ dwa, int n_prev,
                                                               int64_t n, int D) {
  pdl_launch();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int c = (int)(i % D);
  float v = x[i];
  v = fmaf(ls1 ? ls1[c] : 1.0f, y1[i], v);
  if (y2) v = fmaf(ls2 ? ls2[c] : 1.0f, y2[i], v);
  if (!Xs) { x[i] = v; return; }
  Xs[(int64_t)n_prev * x_stride + i] = v;
  float acc = 0.f;
  for (int j = 0; j < n_prev; ++j) acc = fmaf(dwa[j], Xs[(int64_t)j * x_stride + i], acc);
  x[i] = fmaf(dwa[n_prev], v, acc);
}

__global__ void transpose_kernel(const float* __restrict__ src, int rows, int cols, float* __restrict__ dst) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < rows * cols) dst[(size_t)(i % cols) * rows + i / cols] = src[i];
}

int row_threads(int n) { return n >= 1024 ? 256 : n >= 256 ? 128 : 64; }
// a launch of a few CTAs only (decode): as many threads as the row has pairs of entries, up to 1024
int few_row_threads(int n) { return std::min(1024, std::max(64, (n / 2 + 31) & ~31)); }

}  // namespace

cudaError_t launch_layernorm_rows(const float* x, const float* w, float eps, int center, int rows, int D, int src_mul,
                                  int src_add, const int32_t* src_rows, float* out, bf16* out16, cudaStream_t s) {
  return launch_k(layernorm_rows_kernel, dim3(rows), dim3(row_threads(D)), 0, s, x, w, eps, D, center, src_mul, src_add, src_rows,
                  out, out16);
}

cudaError_t launch_canon(const float* h, const float* tail, const float* w1, const float* w2, int B, int L, int D, int T,
                         float* out1, bf16* out1_16, float* out2, bf16* out2_16, cudaStream_t s) {
  const int64_t n = (int64_t)B * L * D;
  if (D % 4 == 0)
    return launch_k(canon4_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, s, h, tail, w1, w2, L, D, T, n / 4, out1, out1_16,
                    out2, out2_16);
  return launch_k(canon_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, h, tail, w1, w2, L, D, T, n, out1, out1_16, out2,
                  out2_16);
}

cudaError_t launch_transpose_f32(const float* src, int rows, int cols, float* dst, cudaStream_t s) {
  transpose_kernel<<<(rows * cols + 255) / 256, 256, 0, s>>>(src, rows, cols, dst);
  return cudaGetLastError();
}

bool norm_canon_rows_supported(int L, int T) { return L <= NORM_CANON_MAX_L && T >= 1 && T <= NORM_CANON_MAX_T; }

cudaError_t launch_norm_canon_rows(float* x, const float* nw, float eps, int center, float* tail, const float* w1,
                                   const float* w2, int B, int L, int D, int T, float* out1, float* out2,
                                   const ParallelCombineArgs* pre, cudaStream_t s) {
  ParallelCombineArgs p{};
  if (pre) p = *pre;
  return launch_k(norm_canon_rows_kernel, dim3(B), dim3(few_row_threads(D)), 0, s, x, nw, eps, center, tail, w1, w2, L, D, T, out1, out2, p);
}

cudaError_t launch_polynorm(float* z, const float* coef, float eps, int rows, int n, bf16* out16, cudaStream_t s) {
  return launch_k(polynorm_kernel, dim3(rows), dim3(rows <= 8 ? few_row_threads(n) : row_threads(n)), 0, s, z, coef, eps, n, out16);
}

cudaError_t launch_parallel_combine(float* x, const float* y1, const float* y2, const float* ls1, const float* ls2, float* Xs,
                                    int64_t x_stride, const float* dwa, int n_prev, int rows, int D, cudaStream_t s) {
  const int64_t n = (int64_t)rows * D;
  return launch_k(parallel_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, x, y1, y2, ls1, ls2, Xs, x_stride, dwa,
                  n_prev, n, D);
}
