// Chunk-parallel form of the linear-attention recurrences whose decay is ONE number per head - fixed (RecurArgs mode 0)
// or a new one for every token (mode 2 with g_head: the state-space mixer) - for prompts.
//
//   S_t = lam S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t
//
// (written below for a fixed lam; with a decay a_t per token every power lam^(i-j) becomes the product a_(j+1) .. a_i,
// formed as exp(c_i - c_j) from the running sums c of the decays' logarithms inside the chunk, so that no product of
// many small numbers is ever divided by another one.)
//
// Inside a chunk of CH tokens that starts from the state P, token i (0-based) reads
//   o_i = lam^(i+1) P^T q_i + sum_{j <= i} lam^(i-j) (q_i . k_j) v_j
// and the chunk leaves  lam^n P + sum_j lam^(n-1-j) k_j v_j^T  behind (n = tokens in the chunk).  Nothing in the two
// sums depends on another chunk, so a prompt runs as three launches over all (sequence, head, chunk) at once instead
// of one dependent chain over its tokens:
//   1. lin_chunk_state_kernel   D_c = sum_j lam^(n-1-j) k_j v_j^T           one CTA per (chunk, head, sequence)
//   2. lin_chunk_scan_kernel    P_c = state before chunk c, in place of D_c; the slot's state after the last chunk
//   3. lin_chunk_out_kernel     A = (Q K^T) .* lam^(i-j) (causal), o = lam^(i+1) Q P_c + A V
// Every product is an fp32 FFMA chain over shared-memory tiles (4 x 4 outputs per thread, operands stored with the
// summed index outermost so that both are read as 16-byte vectors); the powers of lam come from double precision.
// The sums run in another order than the token-by-token kernel, so the two agree to fp32 rounding, not bit for bit.
#include <stdint.h>

#include "common.cuh"
#include "mixer.h"

namespace {

constexpr int CH = 64;       // tokens per chunk
constexpr int LDT = CH + 4;  // row length of a transposed [channel][token] tile: 16-byte rows, 4-bank skew

__device__ __forceinline__ float act_silu(int act_in, float x) {
  return act_in == 0 ? x : act_in == 2 ? __fdividef(x, 1.0f + __expf(-x)) : silu_ref(x);
}

// acc[r][c] += sum_kk X[kk * ldx + r] * Y[kk * ldy + c]; X, Y already point at this thread's four rows / columns
__device__ __forceinline__ void mm44(const float* __restrict__ X, int ldx, const float* __restrict__ Y, int ldy, int K,
                                     float (&acc)[4][4]) {
#pragma unroll 8
  for (int kk = 0; kk < K; ++kk) {
    const float4 x = *reinterpret_cast<const float4*>(X + (size_t)kk * ldx);
    const float4 y = *reinterpret_cast<const float4*>(Y + (size_t)kk * ldy);
    acc[0][0] += x.x * y.x; acc[0][1] += x.x * y.y; acc[0][2] += x.x * y.z; acc[0][3] += x.x * y.w;
    acc[1][0] += x.y * y.x; acc[1][1] += x.y * y.y; acc[1][2] += x.y * y.z; acc[1][3] += x.y * y.w;
    acc[2][0] += x.z * y.x; acc[2][1] += x.z * y.y; acc[2][2] += x.z * y.z; acc[2][3] += x.z * y.w;
    acc[3][0] += x.w * y.x; acc[3][1] += x.w * y.y; acc[3][2] += x.w * y.z; acc[3][3] += x.w * y.w;
  }
}

__device__ __forceinline__ void zero44(float (&acc)[4][4]) {
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
}

// powers lam^0 .. lam^CH of this head's decay, from double precision
__device__ __forceinline__ void fill_powers(float* pw, float lam) {
  for (int p = threadIdx.x; p <= CH; p += blockDim.x) pw[p] = (float)pow((double)lam, (double)p);
}

// cl[j] = sum over t <= j of the chunk's log decays (tokens >= n add nothing): warp 0 scans, 32 tokens at a time
__device__ __forceinline__ void fill_cumlog(float* cl, const float* __restrict__ lg, size_t stride, int n) {
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  float carry = 0.f;
  for (int j0 = 0; j0 < CH; j0 += 32) {
    const int j = j0 + lane;
    float v = j < n ? lg[(size_t)j * stride] : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(L3_FULL, v, o);
      if (lane >= o) v += t;
    }
    v += carry;
    cl[j] = v;
    carry = __shfl_sync(L3_FULL, v, 31);
  }
}

// where the chunks' total decays live inside the workspace: behind the chunk states
__device__ __forceinline__ float* chunk_decays(const RecurArgs& a, int NC) { return a.ws + (size_t)a.B * a.H * NC * a.DK * a.DV; }

// rows [n, CH) of a natural [token][cols] tile and tokens >= n of the operands are zero: they add nothing
__device__ __forceinline__ void load_natural(float* dst, int ld_dst, const float* src, size_t ld_src, int n, int cols, int act_in,
                                             const float* row_scale) {
  const int c4 = cols / 4;
  for (int idx = threadIdx.x; idx < CH * c4; idx += blockDim.x) {
    const int j = idx / c4, c = (idx - j * c4) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < n) {
      v = *reinterpret_cast<const float4*>(src + (size_t)j * ld_src + c);
      const float s = row_scale ? row_scale[j] : 1.f;
      v.x = act_silu(act_in, v.x) * s; v.y = act_silu(act_in, v.y) * s;
      v.z = act_silu(act_in, v.z) * s; v.w = act_silu(act_in, v.w) * s;
    }
    *reinterpret_cast<float4*>(dst + (size_t)j * ld_dst + c) = v;
  }
}

// dst[channel][token] from rows [token][channel]: a lane takes four channels of one token (one 16-byte load), and
// adjacent lanes take adjacent tokens, so the four scalar stores of a warp fall into distinct banks
__device__ __forceinline__ void load_transposed(float* dst, const float* src, size_t ld_src, int n, int cols, int act_in) {
  const int c4 = cols / 4;
  for (int idx = threadIdx.x; idx < CH * c4; idx += blockDim.x) {
    const int j = idx % CH, c = (idx / CH) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < n) {
      v = *reinterpret_cast<const float4*>(src + (size_t)j * ld_src + c);
      v.x = act_silu(act_in, v.x); v.y = act_silu(act_in, v.y); v.z = act_silu(act_in, v.z); v.w = act_silu(act_in, v.w);
    }
    dst[(size_t)(c + 0) * LDT + j] = v.x;
    dst[(size_t)(c + 1) * LDT + j] = v.y;
    dst[(size_t)(c + 2) * LDT + j] = v.z;
    dst[(size_t)(c + 3) * LDT + j] = v.w;
  }
}

// ---------------------------------------------------------------------------- 1. what a chunk adds to the state
template <bool DEC>
__global__ void __launch_bounds__(256) lin_chunk_state_kernel(RecurArgs a, int NC) {
  extern __shared__ __align__(16) float sm[];
  float* pw = sm;                 // [CH + 1] + scale per token [CH]
  float* sc = pw + CH + 4;        // lam^(n - 1 - j)
  float* Ks = sc + CH;            // [CH][DK]
  float* Vs = Ks + (size_t)CH * a.DK;  // [CH][DV]
  pdl_launch();
  pdl_wait();
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
  const int n = min(CH, a.L - c * CH);
  const size_t row0 = (size_t)b * a.L + (size_t)c * CH;
  if (DEC) fill_cumlog(pw, a.log_g + row0 * a.H + h, a.H, n);
  else fill_powers(pw, a.head_decay[h]);
  __syncthreads();
  for (int j = tid; j < CH; j += blockDim.x) sc[j] = j < n ? (DEC ? expf(pw[n - 1] - pw[j]) : pw[n - 1 - j]) : 0.f;
  if (DEC && tid == 0) chunk_decays(a, NC)[((size_t)b * a.H + h) * NC + c] = expf(pw[n - 1]);
  __syncthreads();
  load_natural(Ks, a.DK, a.k + row0 * a.ld_k + (size_t)(h / a.rep) * a.DK, a.ld_k, n, a.DK, a.act_in, sc);
  load_natural(Vs, a.DV, a.v + row0 * a.ld_v + (size_t)h * a.DV, a.ld_v, n, a.DV, a.act_in, nullptr);
  __syncthreads();
  const int tx = tid & 15, ty = tid >> 4;
  float* D = a.ws + (((size_t)b * a.H + h) * NC + c) * a.DK * a.DV;
  for (int d0 = 0; d0 < a.DK; d0 += 64)
    for (int e0 = 0; e0 < a.DV; e0 += 64) {
      float acc[4][4];
      zero44(acc);
      mm44(Ks + d0 + ty * 4, a.DK, Vs + e0 + tx * 4, a.DV, CH, acc);
#pragma unroll
      for (int r = 0; r < 4; ++r)
        *reinterpret_cast<float4*>(D + (size_t)(d0 + ty * 4 + r) * a.DV + e0 + tx * 4) =
            make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
}

// ---------------------------------------------------------------------------- 2. the states between the chunks
template <bool DEC>
__global__ void __launch_bounds__(256) lin_chunk_scan_kernel(RecurArgs a, int NC) {
  pdl_launch();
  pdl_wait();
  const int h = blockIdx.y, b = blockIdx.z;
  const size_t n4 = (size_t)a.DK * a.DV / 4;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float lam = DEC ? 0.f : a.head_decay[h];
  const float full = DEC ? 0.f : (float)pow((double)lam, (double)CH);
  const float last = DEC ? 0.f : (float)pow((double)lam, (double)(a.L - (NC - 1) * CH));
  const float* cdec = DEC ? chunk_decays(a, NC) + ((size_t)b * a.H + h) * NC : nullptr;
  float4* st = reinterpret_cast<float4*>(a.state + ((size_t)b * a.H + h) * a.DK * a.DV) + i;
  float4* W = reinterpret_cast<float4*>(a.ws + ((size_t)b * a.H + h) * NC * a.DK * a.DV) + i;
  float4 S = *st;
  // the chunk sums do not depend on S: four loads stay in flight ahead of the chain
  constexpr int AHEAD = 4;
  float4 d[AHEAD];
#pragma unroll
  for (int u = 0; u < AHEAD; ++u) d[u] = u < NC ? W[(size_t)u * n4] : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c0 = 0; c0 < NC; c0 += AHEAD) {
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      const int c = c0 + u;
      if (c < NC) {
        const float4 cur = d[u];
        if (c + AHEAD < NC) d[u] = W[(size_t)(c + AHEAD) * n4];
        W[(size_t)c * n4] = S;
        const float f = DEC ? cdec[c] : c == NC - 1 ? last : full;
        S.x = f * S.x + cur.x; S.y = f * S.y + cur.y; S.z = f * S.z + cur.z; S.w = f * S.w + cur.w;
      }
    }
  }
  *st = S;
}

// ---------------------------------------------------------------------------- 3. the outputs of a chunk
template <bool DEC>
__global__ void __launch_bounds__(256) lin_chunk_out_kernel(RecurArgs a, int NC) {
  extern __shared__ __align__(16) float sm[];
  float* pw = sm;                            // [CH + 1]
  float* Qt = pw + CH + 4;                   // [DK][LDT]
  float* Kt = Qt + (size_t)a.DK * LDT;       // [DK][LDT]
  float* At = Kt + (size_t)a.DK * LDT;       // [CH][LDT]: At[j][i] = lam^(i-j) q_i . k_j for j <= i
  float* Vs = At + (size_t)CH * LDT;         // [CH][64]
  float* Ps = Kt;                            // [DK][64]: the keys are done with once A stands
  pdl_launch();
  pdl_wait();
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
  const int n = min(CH, a.L - c * CH);
  const size_t row0 = (size_t)b * a.L + (size_t)c * CH;
  if (DEC) fill_cumlog(pw, a.log_g + row0 * a.H + h, a.H, n);
  else fill_powers(pw, a.head_decay[h]);
  load_transposed(Qt, a.q + row0 * a.ld_q + (size_t)(h / a.rep) * a.DK, a.ld_q, n, a.DK, a.act_in);
  load_transposed(Kt, a.k + row0 * a.ld_k + (size_t)(h / a.rep) * a.DK, a.ld_k, n, a.DK, a.act_in);
  __syncthreads();
  const int tx = tid & 15, ty = tid >> 4;
  {
    float acc[4][4];  // acc[r][cc]: query i = ty * 4 + r, key j = tx * 4 + cc
    zero44(acc);
    mm44(Qt + ty * 4, LDT, Kt + tx * 4, LDT, a.DK, acc);
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int j = tx * 4 + cc;
      float4 o;
      float* op = &o.x;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int i = ty * 4 + r;
        op[r] = j <= i ? acc[r][cc] * (DEC ? expf(pw[i] - pw[j]) : pw[i - j]) : 0.f;
      }
      *reinterpret_cast<float4*>(At + (size_t)j * LDT + ty * 4) = o;
    }
  }
  const float* P = a.ws + (((size_t)b * a.H + h) * NC + c) * a.DK * a.DV;
  const int O = a.H * a.DV;
  for (int e0 = 0; e0 < a.DV; e0 += 64) {
    __syncthreads();  // At is written; the previous tile's Vs / Ps are no longer read
    load_natural(Vs, 64, a.v + row0 * a.ld_v + (size_t)h * a.DV + e0, a.ld_v, n, 64, a.act_in, nullptr);
    for (int idx = tid; idx < a.DK * 16; idx += blockDim.x) {
      const int d = idx >> 4, e = (idx & 15) * 4;
      *reinterpret_cast<float4*>(Ps + (size_t)d * 64 + e) = *reinterpret_cast<const float4*>(P + (size_t)d * a.DV + e0 + e);
    }
    __syncthreads();
    float acc[4][4];
    zero44(acc);
    mm44(Qt + ty * 4, LDT, Ps + tx * 4, 64, a.DK, acc);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float f = DEC ? expf(pw[ty * 4 + r]) : pw[ty * 4 + r + 1];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) acc[r][cc] *= f;
    }
    mm44(At + ty * 4, LDT, Vs + tx * 4, 64, CH, acc);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = ty * 4 + r;
      if (i < n)
        *reinterpret_cast<float4*>(a.out + (row0 + i) * O + (size_t)h * a.DV + e0 + tx * 4) =
            make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
  }
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

size_t recur_chunk_ws_floats(int B, int L, int H, int DK, int DV) {
  const size_t NC = (L + CH - 1) / CH;
  return (size_t)B * H * NC * DK * DV + (size_t)B * H * NC;  // chunk states, then the chunks' total decays
}

bool recur_chunk_shape(int DK, int DV) { return (DK == 64 || DK == 128) && DV % 64 == 0 && DV >= 64 && DV <= 512; }

bool recur_chunk_supported(const RecurArgs& a) {
  const bool per_token = a.mode == 2 && a.g_head && a.log_g;  // one decay per head and token
  if ((a.mode != 0 && !per_token) || !a.ws || a.L < 2 * CH) return false;
  if (!recur_chunk_shape(a.DK, a.DV)) return false;
  if (a.ld_q % 4 || a.ld_k % 4 || a.ld_v % 4 || (a.H * a.DV) % 4) return false;
  if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned16(a.out) || !aligned16(a.ws) || !aligned16(a.state)) return false;
  return recur_chunk_ws_floats(a.B, a.L, a.H, a.DK, a.DV) <= a.ws_floats;
}

cudaError_t launch_recur_chunk(const RecurArgs& a, cudaStream_t s) {
  if (!recur_chunk_supported(a)) return cudaErrorInvalidValue;
  const int NC = (a.L + CH - 1) / CH;
  const dim3 grid(NC, a.H, a.B);
  const size_t sm1 = (size_t)(CH + 4 + CH + CH * a.DK + CH * a.DV) * sizeof(float);
  const size_t sm3 = (size_t)(CH + 4 + 2 * a.DK * LDT + CH * LDT + CH * 64) * sizeof(float);
  cudaError_t e;
  const int n4 = a.DK * a.DV / 4;
  if (a.mode == 2) {
    if ((e = cudaFuncSetAttribute(lin_chunk_state_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm1)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(lin_chunk_out_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm3)) != cudaSuccess) return e;
    if ((e = launch_k(lin_chunk_state_kernel<true>, grid, dim3(256), sm1, s, a, NC)) != cudaSuccess) return e;
    if ((e = launch_k(lin_chunk_scan_kernel<true>, dim3((n4 + 255) / 256, a.H, a.B), dim3(256), 0, s, a, NC)) != cudaSuccess) return e;
    return launch_k(lin_chunk_out_kernel<true>, grid, dim3(256), sm3, s, a, NC);
  }
  if ((e = cudaFuncSetAttribute(lin_chunk_state_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm1)) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(lin_chunk_out_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm3)) != cudaSuccess) return e;
  if ((e = launch_k(lin_chunk_state_kernel<false>, grid, dim3(256), sm1, s, a, NC)) != cudaSuccess) return e;
  if ((e = launch_k(lin_chunk_scan_kernel<false>, dim3((n4 + 255) / 256, a.H, a.B), dim3(256), 0, s, a, NC)) != cudaSuccess) return e;
  return launch_k(lin_chunk_out_kernel<false>, grid, dim3(256), sm3, s, a, NC);
}
