// Layer-list decoders (l3_create_stack, include/llama3_b200.h): a decoder described as a list of layers, each
// with its own token mixer, an optional gated feed-forward and an optional per-layer token input, sharing the
// handle, the entry points, the generate loop, the graphs and the projection kernels of the Llama path.
#pragma once
#include <set>
#include <string>
#include <vector>

#include "model.h"

struct LLLayer {
  L3LayerSpec spec{};
  // ---- weights (WT = model dtype unless noted)
  void* w_in = nullptr;    // [n_in, width]: every projection that reads the mixer's input, fused row-wise
  int n_in = 0;
  // row / column offsets of the segments inside w_in / its output
  int off_q = 0, off_k = 0, off_v = 0, off_g = 0, off_b = 0, off_a1 = 0, off_g1 = 0;
  void* w_o = nullptr;     // [width, heads * vdim]
  void* w_a2 = nullptr;    // gated delta: [heads * dim, rank_decay]
  void* w_g2 = nullptr;    // gated delta: [heads * vdim, rank_gate]
  void* w13 = nullptr;     // [2 ff, width] rows interleaved gate_j, up_j
  void* w2 = nullptr;      // [width, ff]
  void* side_gate = nullptr;  // [side_dim, width]
  void* side_proj = nullptr;  // [width, side_dim]
  // fp32 vectors
  float *norm1 = nullptr, *norm2 = nullptr, *side_norm = nullptr;  // norm1 / norm2 hold 1 + w when norm_one_plus
  float* mix_norm = nullptr;  // decay-linear: [heads * vdim]; gated delta: [vdim]
  float *q_norm = nullptr, *k_norm = nullptr;  // softmax: over the whole projection
  float* conv_w = nullptr;    // gated delta: [2 kv_heads dim + heads vdim, taps]
  float *A_log = nullptr, *dt_bias = nullptr;
  float* decay = nullptr;     // decay-linear: [heads]
  // latent attention: w_in = dq | dkv | g rows; q_norm / k_norm hold the two latent norms' weights
  void* w_uq = nullptr;       // [heads * (dim + rot_dim), q_rank]
  void* w_uk = nullptr;       // [heads * dim, kv_rank]
  void* w_uv = nullptr;       // [heads * vdim, kv_rank]
  float* inv_freq = nullptr;  // [rot_dims / 2] rot_base^(-2 i / rot_dims), rounded from double
  float* in_bias = nullptr;   // minGRU: [2 dim] biases of the z and x segments of w_in
  float* shift = nullptr;     // token shift: [width]
  // mixture of experts: w13 = [experts * ff, width] up rows expert by expert, w2 = [width, experts * ff]
  float* router = nullptr;      // [experts + identity, width] fp32
  float* correction = nullptr;  // [experts + identity]
  // parallel layers: convolutions ahead of the sublayers [width, taps], layer scales [width], depth-average weights [layer + 2]
  float *canon1 = nullptr, *canon2 = nullptr, *ls1 = nullptr, *ls2 = nullptr, *dwa = nullptr;
  float *canon1t = nullptr, *canon2t = nullptr;  // [taps, width] copies the kernels read (made at finalize)
  // differential attention: w_in = q | k | v rows with in_bias [n_in]; q_norm / k_norm [dim]; lam_vec = lq1 | lk1 | lq2 | lk2
  float *lam_vec = nullptr, *lambda = nullptr;
  float* poly = nullptr;        // PolyNorm coefficients (a, b, c, e); w13 is then the plain up matrix [ff, width]
  // sigmoid-routed gated experts: w13 = [2 (experts ff + shared_ff), width] rows interleaved (gate_j, up_j), expert by
  // expert, the shared expert last; w2 = [width, experts ff + shared_ff]
  int ff_total = 0;
  // window attention: head_vec [heads] the sinks' logits or the sigmoid's biases; state-space mixer: conv_b [channels],
  // skip_d [heads] (the D of y += D x), dt_bias [heads]; gated linear attention: a2_bias [heads * dim]
  float *head_vec = nullptr, *conv_b = nullptr, *skip_d = nullptr, *a2_bias = nullptr;
  // Two mixers side by side: `pair` is the second one (its mixer fields only).  Both read ONE fused input projection -
  // w_in holds in_ld rows, this mixer's segment starts at row / output column in_base - and feed ONE output projection:
  // w_o is [width, ctx_ld], this mixer's columns start at ctx_base.  A single mixer has in_base = ctx_base = 0.
  // The pair's w_in / w_o point into the first mixer's allocations.
  LLLayer* pair = nullptr;
  int in_base = 0, in_ld = 0, ctx_base = 0, ctx_ld = 0, n_ctx = 0;
  float mix_scale = 1.f;  // multiplier of this mixer's result (applied to its slice of the output projection's input)
};

// What one layer RUN keeps per sequence slot (a layer inside the loop has one of these per pass).
struct LLState {
  void *ck = nullptr, *cv = nullptr;  // softmax: [maxB, kv_heads, M, dim] of KVT (cv = keys as projected)
  float* S = nullptr;                 // recurrent: [maxB, heads, dim, vdim]
  float* conv_tail = nullptr;         // gated delta: [maxB, channels, taps - 1]
  void* lat = nullptr;                // latent attention: [maxB, M, kv_rank + rot_dim] of KVT
  float* hprev = nullptr;             // token shift: [maxB, width] the last token's normed mixer input
  // differential attention: ck [maxB, 2 kv_heads, M, dim] (head g, map m at 2 g + m), cv [maxB, kv_heads, M, vdim];
  // parallel layers with a convolution: conv_tail [maxB, width, taps - 1] the last rows of the layer's normed input
  // window attention: ck [maxB, kv_heads, M, dim], cv [maxB, kv_heads, M, vdim]; state-space mixer: S [maxB, heads, state, vdim],
  // conv_tail [maxB, heads vdim + 2 groups state, taps - 1]; gated linear attention: S
  LLState* pair = nullptr;            // state of the layer's second mixer
};

struct LLRun {
  int layer = 0;
  int pass = -1;       // >= 0: first layer of pass `pass` of the loop - the pass's step vector is added ahead of it
};

struct LayerList {
  L3StackConfig cfg{};
  std::vector<LLLayer> layers;
  std::vector<LLRun> runs;       // execution order
  std::vector<LLState> state;    // per run
  float* loop_step = nullptr;    // [loop_times, width] fp32
  void* loop_in = nullptr;       // [width, 2 width] of WT: the looped block's entry projection (loop_in)
  float* embed_norm = nullptr;   // [width]
  float *x0 = nullptr, *cat = nullptr;  // the embedding output [cap_tok, width]; [x | x0] rows [cap_tok, 2 width]
  void* cat16 = nullptr;
  float *win_part_o = nullptr, *win_part_ml = nullptr;  // split scratch of the window attention
  float* xs = nullptr;           // state-space mixer: the convolved x [cap_tok, heads * vdim]
  void* side_embed = nullptr;  // [vocab, n_layers * side_dim] of WT
  std::set<std::string> loaded;
  std::vector<int> slot_pos;   // next position of every sequence slot (host copy)
  // workspace beyond the shared buffers of L3Model (x, xn = sublayer output, q, ctx, h + bf16 mirrors)
  float *pin = nullptr, *aux = nullptr, *rk = nullptr, *rv = nullptr, *rg = nullptr, *rbeta = nullptr, *o = nullptr;
  float* sg = nullptr;
  float* chunk_ws = nullptr;               // chunk states of the chunk-parallel decay-linear recurrence (prompts)
  size_t chunk_ws_floats = 0;
  float* x2 = nullptr;                     // second residual buffer, 8 rows (fused post-norm step of the GEMV path)
  float *xcur = nullptr, *xalt = nullptr;  // where the residual stream of the running step lives / the other buffer
  void* sg16 = nullptr;
  // pre-norm / latent / mixture-of-experts workspace
  float* qlat = nullptr;                   // [rows, heads, kv_rank + rot_dim] queries folded onto the latent
  void* aux16 = nullptr;                   // bf16 mirror of aux (the query latent)
  float *moe_w = nullptr, *moe_dense = nullptr, *moe_idw = nullptr;  // [rows, top] | [rows, experts] | [rows]
  int32_t* moe_sel = nullptr;              // [rows, top]
  // parallel layers
  float* Xs = nullptr;                     // [n_layers + 1][cap_tok, width] embedding output and every layer's own result
  float *hn = nullptr, *hf = nullptr;      // normed rows ahead of the convolutions; the feed-forward's input
  void* hf16 = nullptr;
  float *y1 = nullptr, *y2 = nullptr;      // the two sublayers' results [cap_tok, width]
  float* moe_gu = nullptr;                 // [cap_tok, 2 ff_total] gate | up of every expert
  float *diff_part_o = nullptr, *diff_part_ml = nullptr;  // split scratch of the differential decode attention
  int max_in = 0, max_o = 0, max_ff = 0;
  int head_rows = 0;  // rows the LM head's buffers hold
};

int ll_fill_random(L3Model* m, uint64_t seed);
// final norm + LM head over `rows` source rows of m->x (d_rows, or row b * L + L - 1 of every sequence) -> m->logits
int ll_enqueue_head(L3Model* m, int B, int L, const int32_t* d_rows, int n_rows);
// room for n rows in the LM head's buffers (xlast, its mirror, logits)
int ll_ensure_head_rows(L3Model* m, int n);
int ll_finalize(L3Model* m);
void ll_destroy(L3Model* m);
// zero the KV caches and recurrent state of slots [slot0, slot0 + n) (all layers)
int ll_reset_slots(L3Model* m, int slot0, int n, bool kv_too);
// position bookkeeping of a call that feeds L tokens to slots [0, B) at start_pos; start_pos 0 zeroes their state
int ll_begin_call(L3Model* m, int B, int L, int start_pos);
// all layers of one chunk; x in m->x (and its bf16 mirror) on entry and exit.  d_resid: null, or
// [n_layers, B * L, width] receiving the residual stream after every layer
int ll_enqueue_layers(L3Model* m, const int32_t* d_ids, int ids_ld, int ids_off, int B, int L, float* d_resid);
