// Kernel-launch interface of the token mixers of layer-list decoders (mixer_ops.cu, recurrent.cu, attn_any.cu).
#pragma once
#include "common.cuh"

// ---- row kernels (mixer_ops.cu)
// x[r] += mult * y[r] / sqrt(mean(y[r]^2) + eps) * w; x16 (may be null) receives the bf16 mirror of the new x
cudaError_t launch_resid_postnorm(float* x, const float* y, const float* w, float mult, float eps, int rows, int D,
                                  bf16* x16, cudaStream_t s);
// out[r, i] = o[r, i] / rms(group of i) * w[i % wlen] * sigmoid(gate[r * ld_gate + i]); group = O: one norm per row
cudaError_t launch_gated_rmsnorm(const float* o, const float* gate, int ld_gate, const float* w, int wlen, int group,
                                 float eps, int rows, int O, float* out, bf16* out16, cudaStream_t s);

struct QkNormArgs {
  const float* proj;   // [rows, ld]: q at column 0 (HN * HD), k at column k_off (KVHN * HD)
  int ld, k_off;
  const float* wq;     // [HN * HD], [KVHN * HD] plain norm weights over the whole projection
  const float* wk;
  float eps;
  float* q_out;        // [rows, HN * HD] normalised q
  void* cache_k;       // [maxB, KVHN, M, HD]: normalised k
  void* cache_v;       // same shape: k as projected
  const int* pos_ptr;  // device scalar: position of token 0 of every sequence in this call
  int L, HN, KVHN, HD, M;
};
cudaError_t launch_qk_norm_cache(const QkNormArgs& a, int rows, bool kv_bf16, cudaStream_t s);

// g[r, j] = act(g[r, j]) * table[token(r), col0 + j], in place (+ bf16 mirror)
cudaError_t launch_side_mul(float* g, int n, int rows, const void* table, bool table_bf16, int table_ld, int col0,
                            const int32_t* ids, int ids_ld, int ids_off, int L, int vocab, int act, bf16* out16,
                            cudaStream_t s);

struct DeltaPrepArgs {
  const float* proj;      // [rows, ld]: q | k | v channels at columns [0, C), write-strength logits at beta_off
  int ld, beta_off;
  const float* dt_in;     // [rows, ld_dt]: decay logits per (head, key channel) before the bias
  int ld_dt;
  const float* conv_w;    // [C, taps], last tap = current token
  float* conv_tail;       // [maxB, C, taps - 1]
  const float* A_log;     // [H]
  const float* dt_bias;   // [H * DK]
  float *q_out, *k_out;   // [rows, G * DK]
  float* v_out;           // [rows, H * DV]
  float* decay_out;       // [rows, H * DK]
  float* beta_out;        // [rows, H]
  int L, H, G, DK, DV, taps;
  int update_tail;        // L == 1 only: the kernel also moves conv_tail on by this token (no launch_conv_tail afterwards)
};
cudaError_t launch_delta_prep(const DeltaPrepArgs& a, int rows, cudaStream_t s);
cudaError_t launch_conv_tail(float* tail, const float* proj, int ld, int B, int L, int C, int T1, cudaStream_t s);
// out[r] = x[src_rows ? src_rows[r] : r * src_mul + src_add] / rms * w  (+ bf16 mirror); any D
cudaError_t launch_rmsnorm_rows(const float* x, const float* w, float eps, int rows, int D, int src_mul, int src_add,
                                const int32_t* src_rows, float* out, bf16* out16, cudaStream_t s, int groups = 1);
cudaError_t launch_to_bf16(const float* in, int64_t n, bf16* out, cudaStream_t s);
cudaError_t launch_add_one(float* p, int n, cudaStream_t s);

// ---- recurrences over time (recurrent.cu): one fp32 state matrix [DK, DV] per (sequence slot, head)
struct RecurArgs {
  int mode;               // 0: S <- decay_h S + k v^T, o = S^T q  (q, k, v read through silu when act_in)
                          // 1: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q
                          // 2: S <- diag(g) S + k v^T; o = S^T q
  const float *q, *k, *v; // rows [B * L, ld_*]; head h of q / k at column (h / rep) * DK, of v at column h * DV
  int ld_q, ld_k, ld_v;
  int act_in;             // silu on q, k, v as they are read: 0 no, 1 exact form, 2 fast exponential and divide (pipelined kernel)
  const float* head_decay;  // mode 0: [H]
  const float* g;         // mode 1, 2: [B * L, H * DK]; with g_head [B * L, H], one decay for all key channels of a head
  int g_head;
  const float* log_g;     // mode 2 with g_head, may be null: [B * L, H] the decays' natural logarithms (finite); with it and
                          // `ws`, prompts of the common shapes run in the chunk-parallel form
  const float* beta;      // mode 1: [B * L, H]
  float* state;           // [maxB, H, DK, DV]
  float* out;             // [B * L, H * DV]
  int B, L, H, rep, DK, DV;
  float* ws;              // mode 0, may be null: room for one state matrix per (sequence, head, chunk of 64 tokens);
  size_t ws_floats;       // with it, prompts of the common shapes run in the chunk-parallel form (recur_chunk.cu)
};
bool recur_supported(int DK, int DV);
cudaError_t launch_recur(const RecurArgs& a, cudaStream_t s);
// chunk-parallel form of mode 0 (recur_chunk.cu): floats of workspace a call needs, whether a call can take it, the launch
size_t recur_chunk_ws_floats(int B, int L, int H, int DK, int DV);
bool recur_chunk_shape(int DK, int DV);
bool recur_chunk_supported(const RecurArgs& a);
cudaError_t launch_recur_chunk(const RecurArgs& a, cudaStream_t s);

// ---- attention for head sizes the tiled kernels do not take (attn_any.cu): same arguments, any HD
cudaError_t launch_attn_any(const AttnArgs& a, bool kv_bf16, cudaStream_t s);

// ---- pre-norm layers (prenorm_ops.cu)
// out[r] = n(x[r]) + (prev - n(x[r])) * shift with n(v) = v / rms(v) * w (w: D weights) and prev = n(x[r - 1]) inside a
// sequence, hprev[b] for its first token; the CTA of a sequence's first token then stores n(x[last row]) to hprev[b].
// shift == null: plain norm.  out16 (may be null): bf16 mirror.
// groups > 1: the norm cuts a row into that many equal consecutive parts, each over its own root mean square
cudaError_t launch_prenorm_shift(const float* x, const float* w, float eps, const float* shift, float* hprev, int B, int L,
                                 int D, float* out, bf16* out16, cudaStream_t s, int groups = 1);
// x[r, i] = x[r, i] * mul + (vec ? vec[i] : 0)
cudaError_t launch_scale_add_rows(float* x, float mul, const float* vec, int rows, int D, cudaStream_t s);

// ---- latent attention (attn_latent.cu)
struct LatentPrepArgs {
  const float* proj;     // [rows, ld]: query latent at column 0 (q_rank), key latent at k_off (kv_rank), rotated key part behind it (rot_dim)
  int ld, k_off;
  const float *wq, *wk;  // norm weights [q_rank], [kv_rank]
  float eps;
  float* cq;             // [rows, q_rank] normed query latent (+ bf16 mirror, may be null)
  bf16* cq16;
  void* cache;           // [maxB, M, kv_rank + rot_dim] of KVT
  const float* inv_freq; // [rot_dims / 2]
  const int* pos_ptr;
  int L, M, q_rank, kv_rank, rot_dim, rot_dims;
};
cudaError_t launch_latent_prep(const LatentPrepArgs& a, int rows, bool kv_bf16, cudaStream_t s);
// rotated part of the queries: qlat[r, h, kv_rank + j] = rot(q[r, h, dim + j]) at the row's position
cudaError_t launch_latent_q_rope(const float* q, float* qlat, const float* inv_freq, const int* pos_ptr, int rows, int L,
                                 int H, int dim, int rot_dim, int rot_dims, int kv_rank, cudaStream_t s);
// Batched per-head product  C[r, h, j] = sum_k A[r * lda + h * a_hs + k] * W[h * w_hs + k * w_ks + j * w_js]
// for r < rows, h < H, j < J, k < K; C at c[r * ldc + h * c_hs + j] (+ bf16 mirror).  One of w_ks, w_js is 1.
struct HeadGemmArgs {
  const float* A; int lda, a_hs;
  const void* W; int64_t w_hs; int w_ks, w_js;
  float* C; bf16* C16; int ldc, c_hs;
  int rows, H, J, K;
};
cudaError_t launch_head_gemm(const HeadGemmArgs& a, bool w_bf16, cudaStream_t s);
struct LatentAttnArgs {
  const float* q;        // [B * L, H, Dk] folded queries
  const void* cache;     // [maxB, M, Dk] of KVT; a row's first Dv entries are also its value
  float* out;            // [B * L, H, Dv]
  const float* gate;     // head h of row r is multiplied by sigmoid(gate[r * ld_gate + h]) (null: none)
  int ld_gate;
  const int* pos_ptr;    // keys [0, *pos_ptr + t] are visible to token t
  float scale;
  int B, L, H, Dk, Dv, M;
  int nsplit;            // > 1 (L == 1 only): every split writes (o, m, l) to part_o / part_ml, the combine kernel merges
  float *part_o, *part_ml;
};
size_t latent_attn_smem(int Dk);
bool latent_attn_supported(int Dk, int Dv);
cudaError_t launch_latent_attn(const LatentAttnArgs& a, bool kv_bf16, cudaStream_t s);

// ---- minGRU (mingru.cu): proj [rows, ld] = z | x | g logits of width n each at z_off, x_off, g_off; bias [2 n] (z, x)
// S [maxB, n] is read and written; out[r, c] = S_t[c] * silu(g) (+ bf16 mirror).  Prompts overwrite proj with the gates.
cudaError_t launch_mingru_scan(float* proj, int ld, int z_off, int x_off, int g_off, const float* bias, float* S, int B,
                               int L, int n, float* out, bf16* out16, cudaStream_t s);

// ---- parallel layers (parallel_ops.cu)
// out[r] = (x[src] - mean) / sqrt(var + eps) * w  (center 0: x / rms * w); source rows as launch_rmsnorm_rows
cudaError_t launch_layernorm_rows(const float* x, const float* w, float eps, int center, int rows, int D, int src_mul,
                                  int src_add, const int32_t* src_rows, float* out, bf16* out16, cudaStream_t s);
// dst [cols, rows] = src [rows, cols]^T (small fp32 tables at finalize)
cudaError_t launch_transpose_f32(const float* src, int rows, int cols, float* dst, cudaStream_t s);
// out_s[t] = h[t] + sum_j w_s[j] h[t - T + 1 + j] for s = 1, 2 (out2 null: one sublayer); h [B * L, D]; w_s [T, D] (tap-major);
// tail [maxB, D, T - 1] holds the rows ahead of the call, oldest first (moved on by launch_conv_tail afterwards)
cudaError_t launch_canon(const float* h, const float* tail, const float* w1, const float* w2, int B, int L, int D, int T,
                         float* out1, bf16* out1_16, float* out2, bf16* out2_16, cudaStream_t s);
// few rows per sequence (norm_canon_rows_supported): launch_layernorm_rows + launch_canon + launch_conv_tail as one launch, fp32 only
// pre (may be null): the previous layer's launch_parallel_combine, applied to x by the same launch first
struct ParallelCombineArgs {
  const float *y1, *y2, *ls1, *ls2, *dwa;
  float* Xs;
  int64_t x_stride;
  int n_prev;
};
bool norm_canon_rows_supported(int L, int T);
cudaError_t launch_norm_canon_rows(float* x, const float* nw, float eps, int center, float* tail, const float* w1,
                                   const float* w2, int B, int L, int D, int T, float* out1, float* out2,
                                   const ParallelCombineArgs* pre, cudaStream_t s);
// z[r] <- a N(z) + b N(z^2) + c N(z^3) + e in place (+ bf16 mirror), N = RMS norm over the n values of a row; coef = (a, b, c, e)
cudaError_t launch_polynorm(float* z, const float* coef, float eps, int rows, int n, bf16* out16, cudaStream_t s);
// v = x + ls1 * y1 + ls2 * y2 (y2 null: no second sublayer; ls null: ones).  Xs null: x <- v.  Else Xs[n_prev] <- v and
// x <- sum_(j < n_prev) dwa[j] Xs[j] + dwa[n_prev] v, Xs[j] at Xs + j * x_stride
cudaError_t launch_parallel_combine(float* x, const float* y1, const float* y2, const float* ls1, const float* ls2, float* Xs,
                                    int64_t x_stride, const float* dwa, int n_prev, int rows, int D, cudaStream_t s);

// ---- differential sliding-window attention (attn_diff.cu)
struct DiffPrepArgs {
  const float* proj;     // [rows, ld]: q (H heads of [map 1 | map 2], DK each) at q_off, k (G heads likewise) at k_off, v (G x DV) at v_off
  int ld, q_off, k_off, v_off;
  const float* bias;     // [ld] biases of the projection's columns
  const float *wq, *wk;  // [DK] norm weights shared by all heads and maps
  float eps;
  const float* inv_freq; // [rot_dims / 2]
  float* q_out;          // [rows, H, 2, DK]
  void* cache_k;         // [maxB, 2 G, M, DK] of KVT: head g, map m at index 2 g + m
  void* cache_v;         // [maxB, G, M, DV]
  const int* pos_ptr;
  int L, H, G, DK, DV, M, rot_dims;
};
cudaError_t launch_diff_prep(const DiffPrepArgs& a, int rows, bool kv_bf16, cudaStream_t s);
// out = exp(v[0:n] . v[n:2n]) - exp(v[2n:3n] . v[3n:4n]) + diff
cudaError_t launch_diff_lambda(const float* vecs, int n, float diff, float* out, cudaStream_t s);
struct DiffAttnArgs {
  const float* q;        // [B * L, H, 2, DK]
  const void* cache_k;   // [maxB, 2 G, M, DK]
  const void* cache_v;   // [maxB, G, M, DV]
  float* out;            // [B * L, H, DV] (+ bf16 mirror, may be null)
  bf16* out16;
  const float* lambda;   // device scalar
  const int* pos_ptr;    // token t of the call sits at *pos_ptr + t
  float scale, diff, eps;
  int window;            // query i sees keys j with 0 <= i - j < window; 0: every key up to i
  int B, L, H, G, DK, DV, M;
};
bool diff_attn_supported(int DK, int DV);
bool diff_attn_tiled(int DK, int DV);
// floats of split scratch (part_o; part_ml needs a DV-th of it, times 2) for calls of up to max_rows rows of <= 8 tokens per sequence
size_t diff_attn_part_floats(int max_rows, int H, int DV);
// part_o / part_ml: scratch of the split decode kernel (null: the decode kernel is not used)
cudaError_t launch_diff_attn(const DiffAttnArgs& a, bool kv_bf16, float* part_o, float* part_ml, cudaStream_t s);

// ---- mixture of experts (moe.cu)
struct MoeRouteArgs {
  const float* h;        // [rows, D] router input
  const float* router;   // [E + I, D] fp32
  const float* correction;
  int D, E, I, top, groups, keep;
  int kind;              // 0: softmax scores + correction + groups; 1: scores = sigmoid(logit), the top scores win, weight = score
  float scale;
  int32_t* sel;          // [rows, top] chosen slots, best first
  float* w;              // [rows, top] their weights
  float* dense;          // [rows, E] weight of every expert (0: not chosen); may be null
  float* idw;            // [rows] summed weight of the chosen identity slots
};
cudaError_t launch_moe_route(const MoeRouteArgs& a, int rows, cudaStream_t s);
// u[r, c] <- relu(u[r, c])^2 * dense[r, c / ff]  (+ bf16 mirror)
cudaError_t launch_moe_act_mask(float* u, const float* dense, int rows, int E, int ff, bf16* out16, cudaStream_t s);
// x[r, i] += idw[r] * h[r, i]
cudaError_t launch_moe_identity(float* x, const float* h, const float* idw, int rows, int D, cudaStream_t s);
// few rows: only the chosen experts' weights are read.  hid [rows * top, ff] = relu(up_e h)^2;
// x[r] += sum_k w_k down_e hid_k + idw[r] h[r]
cudaError_t launch_moe_rows(const float* h, const void* w_up, const void* w_down, bool w_bf16, const int32_t* sel,
                            const float* w, const float* idw, int rows, int D, int E, int ff, int top, float* hid, float* x,
                            cudaStream_t s);

// Gated experts whose routing weight multiplies their INPUT (L3_ROUTE_SIGMOID_IN): expert e = down_e(silu(w gate_e h) * (w up_e h)).
// Weights: w_gu [2 (E ff + sff), D] rows interleaved (gate_j, up_j), expert e at rows [2 e ff, 2 (e + 1) ff), the shared expert
// (width sff, weight 1, every token; sff 0: none) behind them; w_down [D, E ff + sff].
// masked-dense path: gu [rows, 2 F] (F = E ff + sff) -> hid [rows, F] = silu(w g) * (w u), zero where the row did not choose the expert
cudaError_t launch_moe_glu_act(const float* gu, const float* dense, int rows, int E, int ff, int sff, float* hid, bf16* hid16,
                               cudaStream_t s);
// few rows: only the chosen experts' (and the shared expert's) weights are read.  hid [rows * (top + 1), max(ff, sff)] scratch;
// y[r] = sum over the row's experts of down_e hid
cudaError_t launch_moe_glu_rows(const float* h, const void* w_gu, const void* w_down, bool w_bf16, const int32_t* sel,
                                const float* w, int rows, int D, int E, int ff, int sff, int top, float* hid, float* y,
                                cudaStream_t s);

// ---- sliding-window attention with kept first tokens, sink softmax or sigmoid weights (attn_window.cu)
struct WinPrepArgs {
  const float* proj;     // [rows, ld]: q (H x DK) at q_off, k (G x DK) at k_off, v (G x DV) at v_off
  int ld, q_off, k_off, v_off;
  const float* inv_freq; // [rot_dims / 2]
  int rot_dims, rot_layout;  // layout 0: entries (2i, 2i + 1) turn together; 1: entries (i, i + rot_dims / 2)
  int unit_norm;         // 1: q and k over their root mean square per head, after the rotation
  float eps;
  float* q_out;          // [rows, H, DK]
  void* cache_k;         // [maxB, G, M, DK] of KVT
  void* cache_v;         // [maxB, G, M, DV]
  const int* pos_ptr;
  int L, H, G, DK, DV, M;
};
cudaError_t launch_win_prep(const WinPrepArgs& a, int rows, bool kv_bf16, cudaStream_t s);
struct WinAttnArgs {
  const float* q;        // [B * L, H, DK]
  const void* cache_k;   // [maxB, G, M, DK]
  const void* cache_v;   // [maxB, G, M, DV]
  float* out;            // out[r * ld_out + h * DV + d] (+ bf16 mirror, may be null), times out_scale
  bf16* out16;
  int ld_out;
  float out_scale;
  const float* head_vec; // [H]: the sink's logit (softmax; null: no sink) or the bias inside the sigmoid
  const int* pos_ptr;    // token t of the call sits at *pos_ptr + t
  float scale;
  int kind;              // L3_ATTN_SINK | L3_ATTN_SIGMOID
  int window, keep_first;  // query i sees key j <= i with i - j < window (0: all) or j < keep_first
  int B, L, H, G, DK, DV, M;
  int nsplit;            // > 1: the key tiles of a query spread over that many CTAs; partials in part_o / part_ml
  float *part_o, *part_ml;
};
bool win_attn_supported(int DK, int DV);
int win_attn_splits(int B, int L, int H, int G, int window, int keep_first, int max_keys, int max_split);
size_t win_attn_part_floats(int max_rows, int H, int DV, int max_split);
cudaError_t launch_win_attn(const WinAttnArgs& a, bool kv_bf16, cudaStream_t s);

// ---- state-space and gated-linear mixers, output stage, small row kernels (hybrid_ops.cu)
struct SsdPrepArgs {
  const float* proj;      // [rows, ld]: x | B | C channels (H DV + 2 G N) at xbc_off, dt logits (H) at dt_off
  int ld, xbc_off, dt_off;
  const float* conv_w;    // [C, taps], last tap = current token
  const float* conv_b;    // [C]
  float* conv_tail;       // [maxB, C, taps - 1]
  const float* A_log;     // [H]
  const float* dt_bias;   // [H]
  float* x_out;           // [rows, H * DV] convolved x (the skip term reads it)
  float* v_out;           // [rows, H * DV] dt * x
  float *k_out, *q_out;   // [rows, G * N] B and C
  float* decay_out;       // [rows, H] exp(-exp(A_log) dt)
  float* logdecay_out;    // [rows, H] -exp(A_log) dt (may be null)
  int L, H, G, N, DV, taps;
  int update_tail;        // L == 1 only: the kernel also moves conv_tail on by this token (no launch_conv_tail afterwards)
};
cudaError_t launch_ssd_prep(const SsdPrepArgs& a, int rows, cudaStream_t s);
// q_out[r, i] = q[r * ld + i] * q_mul;  g_out[r, i] = sigmoid(z[r * ld_z + i] + bias[i])^(1 / tau)   (i < n)
cudaError_t launch_gla_prep(const float* q, int ld, float q_mul, const float* z, int ld_z, const float* bias, float tau, int rows,
                            int n, float* q_out, float* g_out, cudaStream_t s);
// Output stage of a recurrent mixer, a CTA per row of n = H * DV values:
//   y = o + skip_d[i / DV] * skip_x[r, i]                       (skip_d null: y = o)
//   pre_gate 1:  y <- y * act(gate), then out = y / rms_group(y) * w[i % wlen]
//   pre_gate 0:  out = y / rms_group(y) * w[i % wlen] * act(gate)
// with groups of `group` consecutive values, act = sigmoid (gate_act 0) or silu (1); out[r * ld_out + i] * out_scale
struct MixOutArgs {
  const float* o; int n;
  const float* skip_d; const float* skip_x; int DV;
  const float* gate; int ld_gate; int gate_act, pre_gate;
  const float* w; int wlen, group;
  float eps, out_scale;
  float* out; bf16* out16; int ld_out;
};
cudaError_t launch_mix_out(const MixOutArgs& a, int rows, cudaStream_t s);
// x <- cap * tanh(x / cap), n values
cudaError_t launch_softcap(float* x, int64_t n, float cap, cudaStream_t s);
// out[r] = [a[r] | b[r]] (D values each; + bf16 mirror)
cudaError_t launch_concat_rows(const float* a, const float* b, int rows, int D, float* out, bf16* out16, cudaStream_t s);
