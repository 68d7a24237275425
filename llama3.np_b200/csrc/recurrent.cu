// Matrix-state recurrences over time for the recurrent token mixers of layer-list decoders: linear attention
// with a fixed decay per head, and the gated delta rule with a decay per head and key channel.  One fp32
// state matrix S [DK, DV] per (sequence slot, head), carried in HBM between calls.
//
//   mode 0   S <- decay_h S + k v^T                                   o = S^T q
//   mode 1   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T    o = S^T q   (o sees this token's write)
//   mode 2   S <- diag(g) S + k v^T                                   o = S^T q   (g per key channel, or one per head)
//
// The columns of S never mix: column j needs v_j, the token's k, q, g (shared by all columns) and nothing of
// any other column.  So a CTA owns a tile of CPB columns of one (slot, head) for the whole call; a column is
// held by TPC adjacent lanes, each with R rows of it in registers (row i = lane + r TPC), and the two inner
// products over the key dimension are R FMAs plus log2(TPC) shuffles.  Tokens are staged TCH at a time in
// shared memory by the whole CTA (coalesced), outputs leave the same way.  The state is read once at the
// start and written once at the end: a decode step (L = 1) moves 2 x DK x DV x 4 bytes per head and nothing
// else of size - it is HBM-bound on the state; a prompt is a dependent chain over its tokens, the same
// arithmetic in the same order however the prompt is cut into calls, so cutting it changes no bit.
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"
#include "mixer.h"

namespace {

template <int R, int MODE>
__global__ void __launch_bounds__(256) recur_kernel(RecurArgs a, int TPC, int CPB, int TCH) {
  extern __shared__ float sm[];
  const int DKP = R * TPC;  // padded key dimension: rows >= DK hold zeros
  float* sq = sm;                                   // [TCH][DKP]
  float* sk = sq + (size_t)TCH * DKP;               // [TCH][DKP]
  float* sg = sk + (size_t)TCH * DKP;               // [TCH][DKP]   (modes 1, 2)
  float* sv = sg + (MODE >= 1 ? (size_t)TCH * DKP : 0);  // [TCH][CPB]
  float* so = sv + (size_t)TCH * CPB;               // [TCH][CPB]
  float* sb = so + (size_t)TCH * CPB;               // [TCH]        (mode 1)
  pdl_launch();
  pdl_wait();
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int ntile = (a.DV + CPB - 1) / CPB;
  const int h = blockIdx.x / ntile, tile = blockIdx.x - h * ntile, b = blockIdx.y;
  const int kvh = h / a.rep;
  const int cl = tid / TPC, s = tid - cl * TPC;
  const int j = tile * CPB + cl;
  const bool live = cl < CPB;  // a CTA is padded to a whole warp when CPB * TPC < 32
  const bool col_ok = live && j < a.DV;
  float* Sg = a.state + ((size_t)b * a.H + h) * a.DK * a.DV;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = s + r * TPC;
    S[r] = (col_ok && i < a.DK) ? Sg[(size_t)i * a.DV + j] : 0.f;
  }
  const float lam = MODE == 0 ? a.head_decay[h] : 0.f;

  for (int t0 = 0; t0 < a.L; t0 += TCH) {
    const int n = min(TCH, a.L - t0);
    __syncthreads();  // the previous chunk's outputs have left
    for (int idx = tid; idx < n * DKP; idx += nthr) {
      const int tok = idx / DKP, i = idx - tok * DKP;
      const size_t row = (size_t)b * a.L + t0 + tok;
      float qv = 0.f, kv = 0.f, gv = 0.f;
      if (i < a.DK) {
        qv = a.q[row * a.ld_q + (size_t)kvh * a.DK + i];
        kv = a.k[row * a.ld_k + (size_t)kvh * a.DK + i];
        if (a.act_in) { qv = silu_ref(qv); kv = silu_ref(kv); }
        if (MODE >= 1) gv = a.g_head ? a.g[row * (size_t)a.H + h] : a.g[row * ((size_t)a.H * a.DK) + (size_t)h * a.DK + i];
      }
      sq[idx] = qv;
      sk[idx] = kv;
      if (MODE >= 1) sg[idx] = gv;
    }
    for (int idx = tid; idx < n * CPB; idx += nthr) {
      const int tok = idx / CPB, c = idx - tok * CPB;
      const int jj = tile * CPB + c;
      float vv = 0.f;
      if (jj < a.DV) {
        vv = a.v[((size_t)b * a.L + t0 + tok) * a.ld_v + (size_t)h * a.DV + jj];
        if (a.act_in) vv = silu_ref(vv);
      }
      sv[idx] = vv;
    }
    if (MODE == 1)
      for (int tok = tid; tok < n; tok += nthr) sb[tok] = a.beta[((size_t)b * a.L + t0 + tok) * a.H + h];
    __syncthreads();

    for (int tok = 0; tok < n; ++tok) {
      const float* qk = sq + (size_t)tok * DKP + s;
      const float* kk = sk + (size_t)tok * DKP + s;
      const float vj = live ? sv[tok * CPB + cl] : 0.f;
      float acc = 0.f;
      if (MODE == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          S[r] = fmaf(lam, S[r], kk[r * TPC] * vj);
          acc = fmaf(S[r], qk[r * TPC], acc);
        }
      } else if (MODE == 2) {
        const float* gk = sg + (size_t)tok * DKP + s;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          S[r] = fmaf(gk[r * TPC], S[r], kk[r * TPC] * vj);
          acc = fmaf(S[r], qk[r * TPC], acc);
        }
      } else {
        const float* gk = sg + (size_t)tok * DKP + s;
        float kr[R];
        float pred = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          kr[r] = kk[r * TPC];
          S[r] *= gk[r * TPC];
          pred = fmaf(S[r], kr[r], pred);
        }
        for (int o = TPC >> 1; o > 0; o >>= 1) pred += __shfl_xor_sync(L3_FULL, pred, o);
        const float u = sb[tok] * (vj - pred);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          S[r] = fmaf(kr[r], u, S[r]);
          acc = fmaf(S[r], qk[r * TPC], acc);
        }
      }
      for (int o = TPC >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(L3_FULL, acc, o);
      if (s == 0 && live) so[tok * CPB + cl] = acc;
    }
    __syncthreads();
    for (int idx = tid; idx < n * CPB; idx += nthr) {
      const int tok = idx / CPB, c = idx - tok * CPB;
      const int jj = tile * CPB + c;
      if (jj < a.DV) a.out[((size_t)b * a.L + t0 + tok) * ((size_t)a.H * a.DV) + (size_t)h * a.DV + jj] = so[idx];
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = s + r * TPC;
    if (col_ok && i < a.DK) Sg[(size_t)i * a.DV + j] = S[r];
  }
}


// The same recurrences for the common shapes (256 threads: CPB * TPC = 256, R = 8, 2 <= TPC <= 32), software-pipelined:
// while the CTA runs the TCH tokens staged in one shared-memory buffer, every thread already holds its share of the next
// TCH tokens in registers (the global loads were issued before the compute), and stores it - through silu where asked -
// into the other buffer afterwards.  A lane's R rows are two float4 groups (rows 4 (s + rr TPC) + 0..3), so a token costs
// two 16-byte shared-memory loads per operand instead of eight scalar ones, without bank conflicts.  The arithmetic per
// (column, row) and its order over the tokens are those of recur_kernel; only the order in which a column's row partials
// are summed differs (another lane-to-row map), i.e. rounding.
constexpr int RP_TCH = 16;

template <int TPC, int MODE>
__global__ void __launch_bounds__(256) recur_pipe_kernel(RecurArgs a) {
  constexpr int R = 8, DKP = R * TPC, CPB = 256 / TPC, TCH = RP_TCH;
  constexpr int NA = MODE >= 1 ? 3 : 2;               // staged operand arrays of DKP floats per token: q, k (, g)
  constexpr int NPF = TCH * DKP / 256;                // floats per thread and array in the register stage
  constexpr int NV = (TCH * CPB + 255) / 256;
  constexpr int BUF = TCH * (NA * DKP + CPB) + TCH;   // floats per buffer: q | k | (g) | v | beta
  extern __shared__ __align__(16) float sm[];
  float* so = sm + 2 * BUF;                           // [TCH][CPB] outputs of the chunk
  pdl_launch();
  pdl_wait();
  const int tid = threadIdx.x;
  constexpr int ntile_den = CPB;
  const int ntile = (a.DV + ntile_den - 1) / ntile_den;
  const int h = blockIdx.x / ntile, tile = blockIdx.x - h * ntile, b = blockIdx.y;
  const int kvh = h / a.rep;
  const int cl = tid / TPC, s = tid % TPC;
  const int j = tile * CPB + cl;
  const bool col_ok = j < a.DV;
  float* Sg = a.state + ((size_t)b * a.H + h) * a.DK * a.DV;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = 4 * (s + (r >> 2) * TPC) + (r & 3);
    S[r] = (col_ok && i < a.DK) ? Sg[(size_t)i * a.DV + j] : 0.f;
  }
  const float lam = MODE == 0 ? a.head_decay[h] : 0.f;
  const size_t row0 = (size_t)b * a.L;

  float pq[NPF], pk[NPF], pg[MODE >= 1 ? NPF : 1], pv[NV], pb = 0.f;
  // A thread's share of a chunk: operand element i_f of tokens tok_f, tok_f + TSTEP, ... (DKP divides 256, so i_f never
  // changes) and value column c_f of tokens tok_v, tok_v + VSTEP, ...: the addresses advance by a constant per load.
  constexpr int TSTEP = 256 / DKP, VSTEP = CPB >= 256 ? 1 : 256 / CPB;
  const int i_f = tid % DKP, tok_f = tid / DKP, c_f = tid % CPB, tok_v = tid / CPB;
  const bool i_ok = i_f < a.DK, c_ok = tile * CPB + c_f < a.DV;
  const float* q_f = a.q + (row0 + tok_f) * a.ld_q + (size_t)kvh * a.DK + i_f;
  const float* k_f = a.k + (row0 + tok_f) * a.ld_k + (size_t)kvh * a.DK + i_f;
  // the decays: one per (head, key channel), or with g_head one per head
  const size_t g_row = a.g_head ? (size_t)a.H : (size_t)a.H * a.DK;
  const float* g_f = MODE >= 1 ? a.g + (row0 + tok_f) * g_row + (a.g_head ? (size_t)h : (size_t)h * a.DK + i_f) : nullptr;
  const float* v_f = a.v + (row0 + tok_v) * a.ld_v + (size_t)h * a.DV + tile * CPB + c_f;
  const size_t q_st = (size_t)TSTEP * a.ld_q, k_st = (size_t)TSTEP * a.ld_k, g_st = (size_t)TSTEP * g_row, v_st = (size_t)VSTEP * a.ld_v;
  auto fetch = [&](int t0) {  // global -> registers, tokens [t0, t0 + TCH) clipped to L
    const float* qp = q_f + (size_t)t0 * a.ld_q;
    const float* kp = k_f + (size_t)t0 * a.ld_k;
    const float* gp = MODE >= 1 ? g_f + (size_t)t0 * g_row : nullptr;
#pragma unroll
    for (int n = 0; n < NPF; ++n) {
      const bool ok = i_ok && t0 + tok_f + n * TSTEP < a.L;
      pq[n] = ok ? qp[n * q_st] : 0.f;
      pk[n] = ok ? kp[n * k_st] : 0.f;
      if (MODE >= 1) pg[n] = ok ? gp[n * g_st] : 0.f;
    }
    const float* vp = v_f + (size_t)t0 * a.ld_v;
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const bool ok = c_ok && tok_v + n * VSTEP < TCH && t0 + tok_v + n * VSTEP < a.L;
      pv[n] = ok ? vp[n * v_st] : 0.f;
    }
    if (MODE == 1 && tid < TCH) pb = t0 + tid < a.L ? a.beta[(row0 + t0 + tid) * a.H + h] : 0.f;
  };
  // silu of the staged operands: the exact form in fp32 mode (act_in 1), exp2-based with a fast divide where the
  // operands are bf16-rounded projections anyway (act_in 2)
  auto act = [&](float x) { return a.act_in == 2 ? __fdividef(x, 1.0f + __expf(-x)) : silu_ref(x); };
  auto stash = [&](float* buf) {  // registers -> shared memory (silu on the way where asked)
#pragma unroll
    for (int n = 0; n < NPF; ++n) {
      const int e = tid + n * 256;
      buf[e] = a.act_in ? act(pq[n]) : pq[n];
      buf[TCH * DKP + e] = a.act_in ? act(pk[n]) : pk[n];
      if (MODE >= 1) buf[2 * TCH * DKP + e] = pg[n];
    }
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int e = tid + n * 256;
      if (e < TCH * CPB) buf[NA * TCH * DKP + e] = a.act_in ? act(pv[n]) : pv[n];
    }
    if (MODE == 1 && tid < TCH) buf[TCH * (NA * DKP + CPB) + tid] = pb;
  };

  fetch(0);
  stash(sm);
  __syncthreads();
  int cur = 0;
  for (int t0 = 0; t0 < a.L; t0 += TCH, cur ^= 1) {
    const int n = min(TCH, a.L - t0);
    const bool more = t0 + TCH < a.L;
    if (more) fetch(t0 + TCH);  // in flight during the compute below
    const float* buf = sm + cur * BUF;
    const float4* q4 = reinterpret_cast<const float4*>(buf);
    const float4* k4 = reinterpret_cast<const float4*>(buf + TCH * DKP);
    const float4* g4 = reinterpret_cast<const float4*>(buf + 2 * TCH * DKP);
    const float* vb = buf + NA * TCH * DKP;
    const float* bb = buf + TCH * (NA * DKP + CPB);
    int tok_first = 0;
    if (MODE != 1 && TPC >= 4) {
      // No delta step: nothing a token needs waits for a reduction, so four tokens' row partials are summed together -
      // a butterfly that halves the values a lane carries at the first two levels (5 shuffles for four tokens at
      // TPC = 16 instead of 16), after which lane s holds the complete sum of token s & 3.
      for (; tok_first + 4 <= n; tok_first += 4) {
        float part[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int o4 = (tok_first + u) * (DKP / 4) + s;
          const float4 ka = k4[o4], kb = k4[o4 + TPC], qa = q4[o4], qb = q4[o4 + TPC];
          const float kr[R] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
          const float qr[R] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
          const float vj = vb[(tok_first + u) * CPB + cl];
          float a0 = 0.f, a1 = 0.f;
          if (MODE == 0) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              S[r] = fmaf(lam, S[r], kr[r] * vj);
              S[r + 4] = fmaf(lam, S[r + 4], kr[r + 4] * vj);
              a0 = fmaf(S[r], qr[r], a0);
              a1 = fmaf(S[r + 4], qr[r + 4], a1);
            }
          } else {  // a decay per token and key channel
            const float4 ga = g4[o4], gb = g4[o4 + TPC];
            const float gr[R] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              S[r] = fmaf(gr[r], S[r], kr[r] * vj);
              S[r + 4] = fmaf(gr[r + 4], S[r + 4], kr[r + 4] * vj);
              a0 = fmaf(S[r], qr[r], a0);
              a1 = fmaf(S[r + 4], qr[r + 4], a1);
            }
          }
          part[u] = a0 + a1;
        }
        // level xor 1: lanes with bit 0 clear keep tokens 0 and 2, the others 1 and 3
        const bool b0 = s & 1, b1 = s & 2;
        const float send0 = b0 ? part[0] : part[1], send1 = b0 ? part[2] : part[3];
        const float r0 = __shfl_xor_sync(L3_FULL, send0, 1), r1 = __shfl_xor_sync(L3_FULL, send1, 1);
        const float lo = (b0 ? part[1] : part[0]) + r0;  // token (s & 1)
        const float hi = (b0 ? part[3] : part[2]) + r1;  // token 2 + (s & 1)
        // level xor 2: bit 1 clear keeps the low token, set keeps the high one
        const float r2 = __shfl_xor_sync(L3_FULL, b1 ? lo : hi, 2);
        float acc = (b1 ? hi : lo) + r2;                 // token (s & 3)
#pragma unroll
        for (int o = 4; o < TPC; o <<= 1) acc += __shfl_xor_sync(L3_FULL, acc, o);
        if (s < 4) so[(tok_first + s) * CPB + cl] = acc;
      }
    }
#pragma unroll 2
    for (int tok = tok_first; tok < n; ++tok) {
      const int o4 = tok * (DKP / 4) + s;
      const float4 ka = k4[o4], kb = k4[o4 + TPC], qa = q4[o4], qb = q4[o4 + TPC];
      const float kr[R] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
      const float qr[R] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
      const float vj = vb[tok * CPB + cl];
      float acc0 = 0.f, acc1 = 0.f;
      if (MODE == 0) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          S[r] = fmaf(lam, S[r], kr[r] * vj);
          S[r + 4] = fmaf(lam, S[r + 4], kr[r + 4] * vj);
          acc0 = fmaf(S[r], qr[r], acc0);
          acc1 = fmaf(S[r + 4], qr[r + 4], acc1);
        }
      } else if (MODE == 2) {
        const float4 ga = g4[o4], gb = g4[o4 + TPC];
        const float gr[R] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          S[r] = fmaf(gr[r], S[r], kr[r] * vj);
          S[r + 4] = fmaf(gr[r + 4], S[r + 4], kr[r + 4] * vj);
          acc0 = fmaf(S[r], qr[r], acc0);
          acc1 = fmaf(S[r + 4], qr[r + 4], acc1);
        }
      } else {
        const float4 ga = g4[o4], gb = g4[o4 + TPC];
        const float gr[R] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
        float p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          S[r] *= gr[r];
          S[r + 4] *= gr[r + 4];
          p0 = fmaf(S[r], kr[r], p0);
          p1 = fmaf(S[r + 4], kr[r + 4], p1);
        }
        float pred = p0 + p1;
#pragma unroll
        for (int o = TPC >> 1; o > 0; o >>= 1) pred += __shfl_xor_sync(L3_FULL, pred, o);
        const float u = bb[tok] * (vj - pred);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          S[r] = fmaf(kr[r], u, S[r]);
          S[r + 4] = fmaf(kr[r + 4], u, S[r + 4]);
          acc0 = fmaf(S[r], qr[r], acc0);
          acc1 = fmaf(S[r + 4], qr[r + 4], acc1);
        }
      }
      float acc = acc0 + acc1;
#pragma unroll
      for (int o = TPC >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(L3_FULL, acc, o);
      if (s == 0) so[tok * CPB + cl] = acc;
    }
    if (more) stash(sm + (cur ^ 1) * BUF);
    __syncthreads();  // outputs of this chunk and the next chunk's operands are in shared memory
    for (int e = tid; e < n * CPB; e += 256) {
      const int tok = e / CPB, c = e % CPB;
      const int jj = tile * CPB + c;
      if (jj < a.DV) a.out[(row0 + t0 + tok) * ((size_t)a.H * a.DV) + (size_t)h * a.DV + jj] = so[e];
    }
    __syncthreads();  // the next chunk's compute writes `so` again
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = 4 * (s + (r >> 2) * TPC) + (r & 3);
    if (col_ok && i < a.DK) Sg[(size_t)i * a.DV + j] = S[r];
  }
}

template <int TPC>
cudaError_t launch_recur_pipe(const RecurArgs& a, cudaStream_t s) {
  constexpr int DKP = 8 * TPC, CPB = 256 / TPC;
  const int NA = a.mode >= 1 ? 3 : 2;
  const size_t smem = (size_t)(2 * (RP_TCH * (NA * DKP + CPB) + RP_TCH) + RP_TCH * CPB) * sizeof(float);
  const dim3 grid(a.H * ((a.DV + CPB - 1) / CPB), a.B);
  auto go = [&](auto kern) {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
    }
    return launch_k(kern, grid, dim3(256), smem, s, a);
  };
  return a.mode == 0 ? go(recur_pipe_kernel<TPC, 0>) : a.mode == 1 ? go(recur_pipe_kernel<TPC, 1>) : go(recur_pipe_kernel<TPC, 2>);
}

int pow2_at_least(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

template <int R>
cudaError_t launch_recur_r(const RecurArgs& a, cudaStream_t s) {
  const int TPC = std::min(32, pow2_at_least((a.DK + R - 1) / R));
  const int CPB = std::max(1, std::min(256 / TPC, pow2_at_least(a.DV)));
  const int threads = std::max(32, CPB * TPC);  // CPB * TPC is a power of two: whole warps once it reaches 32
  const int DKP = R * TPC;
  const int per_tok = (a.mode >= 1 ? 3 : 2) * DKP + 2 * CPB + 1;
  const int TCH = std::max(1, std::min(32, 11000 / per_tok));
  const size_t smem = (size_t)TCH * per_tok * sizeof(float);
  const int ntile = (a.DV + CPB - 1) / CPB;
  const dim3 grid(a.H * ntile, a.B);
  if (a.mode == 0) return launch_k(recur_kernel<R, 0>, grid, dim3(threads), smem, s, a, TPC, CPB, TCH);
  if (a.mode == 2) return launch_k(recur_kernel<R, 2>, grid, dim3(threads), smem, s, a, TPC, CPB, TCH);
  return launch_k(recur_kernel<R, 1>, grid, dim3(threads), smem, s, a, TPC, CPB, TCH);
}

}  // namespace

bool recur_supported(int DK, int DV) { return DK >= 1 && DK <= 1024 && DV >= 1; }

cudaError_t launch_recur(const RecurArgs& a, cudaStream_t s) {
  if (!recur_supported(a.DK, a.DV)) return cudaErrorInvalidValue;
  static const bool chunk_on = !(getenv("L3_RECUR_CHUNK") && atoi(getenv("L3_RECUR_CHUNK")) == 0);
  if (chunk_on && recur_chunk_supported(a)) return launch_recur_chunk(a, s);  // prompts of the common shapes
  static const bool pipe_on = !(getenv("L3_RECUR_PIPE") && atoi(getenv("L3_RECUR_PIPE")) == 0);
  if (pipe_on && a.DK <= 256) {  // the pipelined kernel: its 256 threads must all own a column slice
    const int TPC = std::min(32, pow2_at_least((a.DK + 7) / 8));
    if (TPC >= 2 && a.DV >= 256 / TPC) {
      switch (TPC) {
        case 2: return launch_recur_pipe<2>(a, s);
        case 4: return launch_recur_pipe<4>(a, s);
        case 8: return launch_recur_pipe<8>(a, s);
        case 16: return launch_recur_pipe<16>(a, s);
        default: return launch_recur_pipe<32>(a, s);
      }
    }
  }
  if (a.DK <= 256) return launch_recur_r<8>(a, s);
  return launch_recur_r<32>(a, s);
}
