// Layer-list decoders: creation, tensors by checkpoint name, per-slot state, and the layers of one step.
//
// A layer is  x += m N1(mixer(x));  x += m N2(ff(x)) [if it has one];  x += m Ns(token_input(x)) [if side_dim]
// with the norm on the sublayer's OUTPUT (N = RMS norm, weight w or 1 + w), the residual stream x in fp32.
// Three mixers (include/llama3_b200.h, L3_MIX_*), each a chain of launches that share the projection kernels of
// the Llama path (row-streaming GEMV for <= 8 rows, tcgen05 GEMMs in bf16 mode, FFMA GEMMs in fp32 mode):
//
//   softmax       fused q|k|gate projection -> whole-projection q / k norm + KV append (values = raw keys)
//                 -> causal attention with the score multiplier and the per-head sigmoid gate in its epilogue
//   decay-linear  fused q|k|v|gate projection -> recurrence (recurrent.cu, silu on load) -> row norm * gate
//   gated delta   fused q|k|v|beta|a1|g1 projection -> a2, g2 -> convolutions, unit vectors, decays
//                 (delta_prep_kernel) -> recurrence -> per-head norm * gate
//   then the output projection and the post-norm residual kernel, which also emits the bf16 mirror of the new
//   residual rows for the next tensor-core projection.
//
//
// Pre-norm stacks (L3StackConfig::norm_input):  x += mixer(shift(norm1(x)));  x += ff(norm2(x)), the norms with one
// weight or one per coordinate, the mixer's input optionally mixed with the previous token's (token shift, one saved
// row per sequence slot and layer run), the output projections adding into x in their epilogue.  Two mixers:
//
//   latent        fused dq|dkv|g projection -> norms of both latents, rotation of the shared key part, append of the
//                 [latent | rotated part] row to the run's cache -> query up-projection -> queries folded onto the
//                 latent per head (Wuk^T q) -> attention over the cache rows themselves, all heads of a token against
//                 the same rows (attn_latent.cu), gate per head -> values out of the latent per head (Wuv o)
//   minGRU        fused z|x|g projection -> element-wise gated recurrence (prenorm_ops.cu)
//   and a feed-forward that is a mixture of experts (moe.cu): fp32 router -> few rows: only the chosen experts' weights
//   are read; many rows: ONE up-projection over all experts, relu^2 times the routing weight (zero where not chosen),
//   ONE down-projection whose K runs over all experts and so sums them.
// Parallel stacks (L3StackConfig::parallel, ll_enqueue_parallel):  h = norm1(x);  X_new = x + ls1 mixer(h + conv1(h)) +
// ls2 ff(h + conv2(h));  x <- sum_j dwa[j] X_j over the embedding output and every layer result so far.  One mixer:
//
//   differential  fused q|k|v projection -> biases, RMS norm per head and map, rotary turn, append of both maps' keys and of
//                 the values (attn_diff.cu) -> two softmax maps per head over a sliding window of the same values, combined
//                 as a1 - lambda a2 and normed per head
//   and a feed-forward that is dense with the PolyNorm activation (parallel_ops.cu) or a mixture of gated experts routed by
//   sigmoid scores whose weights scale the experts' input, with a shared expert (moe.cu), or none.
// A block of layers can run several times per token (loop_*): the execution order is a list of layer RUNS, every run
// with its own cache / state (LLState); the pass's step vector is added ahead of the block's first layer.
//
// Precision: norms, gates, decays, scores, softmax, router, recurrent state and the residual sum are fp32 in both
// modes; bf16 mode rounds only GEMM operands (weights, and activations on the tensor-core path) and the KV cache.
#include "layerlist.h"

#include <math.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>

#include "common.cuh"
#include "gemm_tc.h"
#include "internal.h"
#include "mixer.h"

static size_t wb(const L3Model* m) { return m->bf16 ? 2 : 4; }
static int pad8(int v) { return (v + 7) & ~7; }

// ------------------------------------------------------------------------------ create
// the mixers that pre-norm stacks run through ll_mix_unit, alone or two side by side
static bool unit_mixer(int mixer) { return mixer == L3_MIX_WINDOW || mixer == L3_MIX_SSD || mixer == L3_MIX_GLA || mixer == L3_MIX_GATED_DELTA; }

static int check_unit(const L3LayerSpec& s, int i) {
  REQUIRE(nullptr, s.heads >= 1 && s.dim >= 1 && s.vdim >= 1, "layer %d: bad sizes", i);
  if (s.mixer == L3_MIX_WINDOW) {
    REQUIRE(nullptr, s.kv_heads >= 1 && s.heads % s.kv_heads == 0, "layer %d: heads %% kv_heads != 0", i);
    REQUIRE(nullptr, s.rot_dims >= 0 && s.rot_dims <= s.dim && s.rot_dims % 2 == 0 && (s.rot_dims == 0 || s.rot_base > 0), "layer %d: bad rotary sizes", i);
    REQUIRE(nullptr, s.window >= 0 && s.keep_first >= 0 && (s.attn_kind == L3_ATTN_SINK || s.attn_kind == L3_ATTN_SIGMOID), "layer %d: bad window / kind", i);
    REQUIRE(nullptr, win_attn_supported(s.dim, s.vdim), "layer %d: head sizes %d, %d unsupported", i, s.dim, s.vdim);
  } else if (s.mixer == L3_MIX_SSD) {
    REQUIRE(nullptr, s.kv_heads >= 1 && s.heads % s.kv_heads == 0, "layer %d: heads %% groups != 0", i);
    REQUIRE(nullptr, s.conv_taps >= 1 && s.conv_taps <= 64, "layer %d: bad conv size", i);
    REQUIRE(nullptr, s.out_norm_groups >= 1 && (s.heads * s.vdim) % s.out_norm_groups == 0, "layer %d: bad output norm groups", i);
    REQUIRE(nullptr, recur_supported(s.dim, s.vdim), "layer %d: state %d x %d unsupported", i, s.dim, s.vdim);
  } else if (s.mixer == L3_MIX_GLA) {
    REQUIRE(nullptr, s.rank_decay >= 1 && s.tau > 0.f, "layer %d: bad decay rank / tau", i);
    REQUIRE(nullptr, recur_supported(s.dim, s.vdim), "layer %d: state %d x %d unsupported", i, s.dim, s.vdim);
  } else {
    REQUIRE(nullptr, s.kv_heads >= 1 && s.heads % s.kv_heads == 0, "layer %d: heads %% kv_heads != 0", i);
    REQUIRE(nullptr, s.conv_taps >= 1 && s.conv_taps <= 64 && s.rank_decay >= 1 && s.rank_gate >= 1, "layer %d: bad conv / rank sizes", i);
    REQUIRE(nullptr, recur_supported(s.dim, s.vdim), "layer %d: state %d x %d unsupported", i, s.dim, s.vdim);
  }
  return L3_OK;
}

static int check_spec(const L3StackConfig* c, const L3LayerSpec& s, int i) {
  REQUIRE(nullptr, s.mixer >= L3_MIX_SOFTMAX && s.mixer <= L3_MIX_GLA, "layer %d: unknown mixer %d", i, s.mixer);
  REQUIRE(nullptr, s.mixer < L3_MIX_WINDOW || (c->norm_input && !c->parallel), "layer %d: this mixer is built for pre-norm layers (norm_input)", i);
  REQUIRE(nullptr, !s.pair || (c->norm_input && !c->parallel && unit_mixer(s.mixer) && unit_mixer(s.pair->mixer) && !s.pair->pair),
          "layer %d: two mixers side by side need a pre-norm stack and mixers of the window / state-space / gated-linear / gated-delta kinds", i);
  if (c->norm_input && !c->parallel && unit_mixer(s.mixer)) {
    int rc = check_unit(s, i);
    if (rc == L3_OK && s.pair) rc = check_unit(*s.pair, i);
    if (rc != L3_OK) return rc;
  }
  REQUIRE(nullptr, (s.mixer == L3_MIX_DIFF) == (c->parallel != 0), "layer %d: differential attention and parallel layers come together", i);
  REQUIRE(nullptr, s.ff_kind == L3_FF_GLU || (s.ff_kind == L3_FF_POLYNORM && c->parallel), "layer %d: this feed-forward kind is built for parallel layers", i);
  REQUIRE(nullptr, s.router_kind == L3_ROUTE_SOFTMAX || (s.router_kind == L3_ROUTE_SIGMOID_IN && c->parallel), "layer %d: this router kind is built for parallel layers", i);
  REQUIRE(nullptr, !(c->parallel && s.experts > 0) || s.router_kind == L3_ROUTE_SIGMOID_IN, "layer %d: parallel layers take the sigmoid router", i);
  REQUIRE(nullptr, s.heads >= 1 && s.dim >= 1 && s.vdim >= 1 && s.ff >= 0, "layer %d: bad sizes", i);
  REQUIRE(nullptr, s.mixer <= L3_MIX_GATED_DELTA || c->norm_input, "layer %d: this mixer is built for pre-norm layers (norm_input)", i);
  REQUIRE(nullptr, !(c->norm_input && !c->parallel) || s.mixer == L3_MIX_LATENT || s.mixer == L3_MIX_MINGRU || unit_mixer(s.mixer),
          "layer %d: mixer %d is not built for pre-norm layers", i, s.mixer);
  if (s.experts > 0) {
    const int n = s.experts + s.identity;
    REQUIRE(nullptr, c->norm_input, "layer %d: the mixture of experts is built for pre-norm layers (norm_input)", i);
    REQUIRE(nullptr, s.ff >= 1 && s.identity >= 0 && s.top >= 1 && s.top <= n && n <= 1024, "layer %d: bad expert counts", i);
    REQUIRE(nullptr, s.router_kind == L3_ROUTE_SOFTMAX || (s.identity == 0 && s.top <= s.experts && s.shared_ff >= 0), "layer %d: bad sigmoid-router sizes", i);
    REQUIRE(nullptr, s.groups >= 1 && n % s.groups == 0 && s.groups_keep >= 1 && s.groups_keep <= s.groups, "layer %d: bad expert groups", i);
  }
  if (s.mixer == L3_MIX_LATENT) {
    REQUIRE(nullptr, s.q_rank >= 1 && s.kv_rank >= 1 && s.rot_dim >= 0 && s.rot_dims >= 0 && s.rot_dims <= s.rot_dim && s.rot_dims % 2 == 0,
            "layer %d: bad latent / rotary sizes", i);
    REQUIRE(nullptr, s.rot_dims == 0 || s.rot_base > 0, "layer %d: rotary base must be positive", i);
    REQUIRE(nullptr, latent_attn_supported(s.kv_rank + s.rot_dim, s.kv_rank), "layer %d: latent row of %d + %d entries unsupported", i, s.kv_rank, s.rot_dim);
  } else if (s.mixer == L3_MIX_DIFF) {
    REQUIRE(nullptr, s.kv_heads >= 1 && s.heads % s.kv_heads == 0, "layer %d: heads %% kv_heads != 0", i);
    REQUIRE(nullptr, s.rot_dims >= 0 && s.rot_dims <= s.dim && s.rot_dims % 2 == 0 && (s.rot_dims == 0 || s.rot_base > 0), "layer %d: bad rotary sizes", i);
    REQUIRE(nullptr, s.rot_scale_original == 0 || (s.rot_scale_factor > 0 && s.rot_scale_high != s.rot_scale_low && s.rot_scale_low > 0 && s.rot_scale_high > 0),
            "layer %d: bad rotary scaling", i);
    REQUIRE(nullptr, s.window >= 0 && diff_attn_supported(s.dim, s.vdim), "layer %d: window %d / head sizes %d, %d unsupported", i, s.window, s.dim, s.vdim);
  } else if (s.mixer == L3_MIX_MINGRU) {
    REQUIRE(nullptr, s.heads == 1 && s.vdim == 1, "layer %d: the element-wise recurrence has heads = vdim = 1", i);
  } else if (s.mixer == L3_MIX_SOFTMAX) {
    REQUIRE(nullptr, s.kv_heads >= 1 && s.heads % s.kv_heads == 0, "layer %d: heads %% kv_heads != 0", i);
    REQUIRE(nullptr, s.vdim == s.dim, "layer %d: the values of this attention are its keys, so vdim must equal dim", i);
  } else if (s.mixer == L3_MIX_DECAY_LINEAR) {
    REQUIRE(nullptr, s.decay != nullptr, "layer %d: decay-linear mixer without decays", i);
    REQUIRE(nullptr, recur_supported(s.dim, s.vdim), "layer %d: state %d x %d unsupported", i, s.dim, s.vdim);
  } else if (s.mixer == L3_MIX_GATED_DELTA) {
    REQUIRE(nullptr, s.kv_heads >= 1 && s.heads % s.kv_heads == 0, "layer %d: heads %% kv_heads != 0", i);
    REQUIRE(nullptr, s.conv_taps >= 1 && s.conv_taps <= 64 && s.rank_decay >= 1 && s.rank_gate >= 1, "layer %d: bad conv / rank sizes", i);
    REQUIRE(nullptr, recur_supported(s.dim, s.vdim), "layer %d: state %d x %d unsupported", i, s.dim, s.vdim);
  }
  (void)c;
  return L3_OK;
}

// Segment layout of a unit mixer's share of the fused input projection (offsets relative to the unit's first column),
// the width of its share of the output projection's input, and its small fp32 tensors.
static int ll_alloc_unit(LLLayer& L, size_t w) {
  const L3LayerSpec& s = L.spec;
  const int H = s.heads, G = s.kv_heads, DK = s.dim, DV = s.vdim;
  cudaError_t e = cudaSuccess;
  auto al = [&](void** p, size_t bytes) { if (e == cudaSuccess) e = cudaMalloc(p, std::max<size_t>(16, bytes)); };
  L.n_ctx = H * DV;
  if (s.mixer == L3_MIX_WINDOW) {
    L.off_q = 0; L.off_k = H * DK; L.off_v = L.off_k + G * DK; L.n_in = pad8(L.off_v + G * DV);  // q | k | v
    al((void**)&L.head_vec, (size_t)H * 4);
    al((void**)&L.inv_freq, (size_t)std::max(1, s.rot_dims / 2) * 4);
    std::vector<float> f(std::max(1, s.rot_dims / 2), 0.f);
    for (int j = 0; j < s.rot_dims / 2; ++j) f[j] = (float)pow(s.rot_base, -2.0 * j / s.rot_dims);
    if (e == cudaSuccess) e = cudaMemcpy(L.inv_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice);
  } else if (s.mixer == L3_MIX_SSD) {
    // z | x | B | C | dt as the checkpoint lays them out: x, B, C stay contiguous (a convolution channel is a column)
    const int inner = H * DV, gn = G * DK;
    L.off_g = 0; L.off_q = inner; L.off_b = 2 * inner + 2 * gn; L.n_in = pad8(L.off_b + H);
    al((void**)&L.conv_w, (size_t)(inner + 2 * gn) * s.conv_taps * 4);
    al((void**)&L.conv_b, (size_t)(inner + 2 * gn) * 4);
    al((void**)&L.A_log, (size_t)H * 4);
    al((void**)&L.dt_bias, (size_t)H * 4);
    al((void**)&L.skip_d, (size_t)H * 4);
    al((void**)&L.mix_norm, (size_t)inner * 4);
  } else if (s.mixer == L3_MIX_GLA) {
    L.off_q = 0; L.off_k = H * DK; L.off_v = 2 * H * DK; L.off_g = L.off_v + H * DV;
    L.off_a1 = pad8(L.off_g + H * DV); L.n_in = pad8(L.off_a1 + s.rank_decay);
    al((void**)&L.mix_norm, (size_t)DV * 4);
    al(&L.w_a2, (size_t)H * DK * s.rank_decay * w);
    al((void**)&L.a2_bias, (size_t)H * DK * 4);
  } else {
    // q | k | v stay contiguous (a convolution channel is a column); the inner projections start on a
    // multiple of 8 columns so that the second-stage projections read 16-byte aligned rows
    L.off_q = 0; L.off_k = G * DK; L.off_v = 2 * G * DK; L.off_b = L.off_v + H * DV;
    L.off_a1 = pad8(L.off_b + H); L.off_g1 = pad8(L.off_a1 + s.rank_decay); L.n_in = pad8(L.off_g1 + s.rank_gate);
    al((void**)&L.mix_norm, (size_t)DV * 4);
    al(&L.w_a2, (size_t)H * DK * s.rank_decay * w);
    al(&L.w_g2, (size_t)H * DV * s.rank_gate * w);
    al((void**)&L.conv_w, (size_t)(2 * G * DK + H * DV) * s.conv_taps * 4);
    al((void**)&L.A_log, (size_t)H * 4);
    al((void**)&L.dt_bias, (size_t)H * DK * 4);
  }
  if (e != cudaSuccess) { set_err(nullptr, "cudaMalloc of a mixer's tensors failed: %s", cudaGetErrorString(e)); return L3_ENOMEM; }
  return L3_OK;
}

extern "C" int l3_create_stack(const L3StackConfig* c, const L3LayerSpec* specs, L3Model** out) {
  *out = nullptr;
  REQUIRE(nullptr, c && specs && c->width >= 1 && c->vocab >= 1 && c->n_layers >= 1, "bad stack config");
  REQUIRE(nullptr, c->max_batch_size >= 1 && c->max_seq_len >= 1, "bad sizes");
  REQUIRE(nullptr, c->dtype == L3_DTYPE_F32 || c->dtype == L3_DTYPE_BF16, "bad dtype");
  REQUIRE(nullptr, c->side_dim >= 0 && (c->glu_act == GLU_SILU || c->glu_act == GLU_GELU_TANH), "bad side_dim / glu_act");
  for (int i = 0; i < c->n_layers; ++i) {
    const int rc = check_spec(c, specs[i], i);
    if (rc != L3_OK) return rc;
  }
  REQUIRE(nullptr, c->loop_times >= 0 && (c->loop_times == 0 || (c->loop_start >= 0 && c->loop_start <= c->loop_stop && c->loop_stop <= c->n_layers)),
          "bad loop bounds");
  REQUIRE(nullptr, !c->norm_input || c->side_dim == 0, "pre-norm stacks have no per-layer token input");
  REQUIRE(nullptr, c->norm_input || (!c->token_shift && !c->norm_scalar), "token shift and single-weight norms are built for pre-norm stacks");
  REQUIRE(nullptr, !c->parallel || (c->norm_input && !c->token_shift && !c->norm_scalar && c->loop_times == 0), "parallel layers are pre-norm layers without token shift, single-weight norms or loops");
  REQUIRE(nullptr, c->parallel || (!c->norm_center && !c->layer_scale && !c->canon_taps && !c->depth_avg), "centred norms, layer scales, input convolutions and the depth average are built for parallel layers");
  REQUIRE(nullptr, c->canon_taps >= 0 && c->canon_taps <= 64, "bad canon_taps");
  REQUIRE(nullptr, c->norm_groups >= 0 && c->norm_groups <= 128 && (c->norm_groups <= 1 || c->width % c->norm_groups == 0), "bad norm_groups");
  REQUIRE(nullptr, (c->norm_input && !c->parallel) || (c->norm_groups <= 1 && !c->embed_norm && !c->loop_in && !(c->logit_softcap > 0.f)),
          "grouped norms, the embedding norm, the loop's entry projection and the logit cap are built for pre-norm stacks");
  REQUIRE(nullptr, !c->loop_in || c->loop_times > 0, "loop_in without a loop");
  REQUIRE(nullptr, !(c->norm_groups > 1 && c->norm_scalar), "grouped norms have one weight per coordinate");
  L3Model* m = new L3Model();
  LayerList* ll = m->ll = new LayerList();
  ll->cfg = *c;
  m->cfg.dim = c->width; m->cfg.n_layers = c->n_layers; m->cfg.n_heads = 1; m->cfg.n_kv_heads = 1;
  m->cfg.vocab_size = c->vocab; m->cfg.max_seq_len = c->max_seq_len; m->cfg.max_batch_size = c->max_batch_size;
  m->cfg.hidden_dim = 0; m->cfg.norm_eps = c->norm_eps; m->cfg.dtype = c->dtype; m->cfg.device = c->device;
  m->cfg.tp_rank = 0; m->cfg.tp_world = 1; m->cfg.flags = c->flags;
  m->bf16 = c->dtype == L3_DTYPE_BF16;
  m->D = c->width; m->HD = 0; m->G = 1; m->HN = 0; m->KVHN = 0; m->FD = 0; m->VS = c->vocab; m->M = c->max_seq_len;
  m->maxB = c->max_batch_size;
  if (cudaSetDevice(c->device) != cudaSuccess) {
    set_err(nullptr, "cudaSetDevice(%d) failed: %s", c->device, cudaGetErrorString(cudaGetLastError()));
    delete ll; delete m;
    return L3_ECUDA;
  }
  cudaError_t e = cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) { set_err(nullptr, "stream: %s", cudaGetErrorString(e)); delete ll; delete m; return L3_ECUDA; }
  cudaEventCreate(&m->ev0);
  cudaEventCreate(&m->ev1);
  const size_t w = wb(m);
  const int W = c->width, sd = c->side_dim;
#define AL(p, bytes)                                                                          \
  if ((e = cudaMalloc((void**)&(p), std::max<size_t>(16, (bytes)))) != cudaSuccess) {          \
    set_err(nullptr, "cudaMalloc(%zu) failed: %s", (size_t)(bytes), cudaGetErrorString(e));   \
    l3_destroy(m);                                                                            \
    return L3_ENOMEM;                                                                         \
  }
  AL(m->embed, (size_t)c->vocab * W * w);
  AL(m->lm_head, (size_t)c->vocab * W * w);
  AL(m->norm_final, (size_t)W * 4);
  if (sd) AL(ll->side_embed, (size_t)c->vocab * c->n_layers * sd * w);
  ll->layers.resize(c->n_layers);
  for (int i = 0; i < c->n_layers; ++i) {
    LLLayer& L = ll->layers[i];
    L.spec = specs[i];
    const L3LayerSpec& s = L.spec;
    const int H = s.heads, G = s.mixer == L3_MIX_DECAY_LINEAR ? s.heads : s.kv_heads, DK = s.dim, DV = s.vdim;
    L.spec.kv_heads = G;
    if (s.pair) {  // the second mixer of the layer: its own record, sharing the first one's projections
      L.pair = new LLLayer();
      L.pair->spec = *s.pair;
      L.pair->spec.pair = nullptr; L.pair->spec.ff = 0; L.pair->spec.experts = 0; L.pair->spec.decay = nullptr;
      L.pair->mix_scale = s.pair_scale;
      L.mix_scale = s.mix_scale;
      L.spec.pair = nullptr;  // the caller's record is not kept
    }
    if (unit_mixer(s.mixer) && c->norm_input) {
      int rc = ll_alloc_unit(L, w);
      if (rc == L3_OK && L.pair) rc = ll_alloc_unit(*L.pair, w);
      if (rc != L3_OK) { l3_destroy(m); return rc; }
    } else if (s.mixer == L3_MIX_LATENT) {
      // dq | dkv | g rows, every segment on a multiple of 8 columns of the projection's output
      const int Dk = s.kv_rank + s.rot_dim;
      L.off_q = 0; L.off_k = pad8(s.q_rank); L.off_g = pad8(L.off_k + Dk); L.n_in = pad8(L.off_g + H);
      AL(L.q_norm, (size_t)s.q_rank * 4);
      AL(L.k_norm, (size_t)s.kv_rank * 4);
      AL(L.w_uq, (size_t)H * (DK + s.rot_dim) * s.q_rank * w);
      AL(L.w_uk, (size_t)H * DK * s.kv_rank * w);
      AL(L.w_uv, (size_t)H * DV * s.kv_rank * w);
      AL(L.inv_freq, (size_t)std::max(1, s.rot_dims / 2) * 4);
      std::vector<float> f(std::max(1, s.rot_dims / 2), 0.f);
      for (int j = 0; j < s.rot_dims / 2; ++j) f[j] = (float)pow(s.rot_base, -2.0 * j / s.rot_dims);
      if ((e = cudaMemcpy(L.inv_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess) {
        set_err(nullptr, "rotary table upload: %s", cudaGetErrorString(e)); l3_destroy(m); return L3_ECUDA;
      }
    } else if (s.mixer == L3_MIX_DIFF) {
      L.off_q = 0; L.off_k = 2 * H * DK; L.off_v = L.off_k + 2 * G * DK; L.n_in = pad8(L.off_v + G * DV);  // q | k | v
      AL(L.in_bias, (size_t)L.n_in * 4);
      cudaMemset(L.in_bias, 0, (size_t)L.n_in * 4);
      AL(L.q_norm, (size_t)DK * 4);
      AL(L.k_norm, (size_t)DK * 4);
      AL(L.lam_vec, (size_t)4 * DK * 4);
      AL(L.lambda, 4);
      AL(L.inv_freq, (size_t)std::max(1, s.rot_dims / 2) * 4);
      std::vector<float> f(std::max(1, s.rot_dims / 2), 0.f);
      const double two_pi = 6.283185307179586476925286766559;
      for (int j = 0; j < s.rot_dims / 2; ++j) {
        double fr = pow(s.rot_base, -2.0 * j / s.rot_dims);
        if (s.rot_scale_original > 0) {  // wavelength-dependent rescaling
          const double wl = two_pi / fr, orig = s.rot_scale_original;
          if (wl > orig / s.rot_scale_low) fr = fr / s.rot_scale_factor;
          else if (!(wl < orig / s.rot_scale_high)) {
            const double sm = (orig / wl - s.rot_scale_low) / ((double)s.rot_scale_high - s.rot_scale_low);
            fr = (1.0 - sm) * fr / s.rot_scale_factor + sm * fr;
          }
        }
        f[j] = (float)fr;
      }
      if ((e = cudaMemcpy(L.inv_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess) {
        set_err(nullptr, "rotary table upload: %s", cudaGetErrorString(e)); l3_destroy(m); return L3_ECUDA;
      }
    } else if (s.mixer == L3_MIX_MINGRU) {
      L.off_b = 0; L.off_v = pad8(DK); L.off_g = pad8(L.off_v + DK); L.n_in = pad8(L.off_g + DK);  // z | x | g
      AL(L.in_bias, (size_t)2 * DK * 4);
    } else if (s.mixer == L3_MIX_SOFTMAX) {
      L.off_q = 0; L.off_k = H * DK; L.off_g = L.off_k + G * DK; L.n_in = L.off_g + H;
      AL(L.q_norm, (size_t)H * DK * 4);
      AL(L.k_norm, (size_t)G * DK * 4);
    } else if (s.mixer == L3_MIX_DECAY_LINEAR) {
      L.off_q = 0; L.off_k = H * DK; L.off_v = 2 * H * DK; L.off_g = L.off_v + H * DV; L.n_in = L.off_g + H * DV;
      AL(L.mix_norm, (size_t)H * DV * 4);
      AL(L.decay, (size_t)H * 4);
      if ((e = cudaMemcpy(L.decay, s.decay, (size_t)H * 4, cudaMemcpyHostToDevice)) != cudaSuccess) {
        set_err(nullptr, "decay upload: %s", cudaGetErrorString(e)); l3_destroy(m); return L3_ECUDA;
      }
      L.spec.decay = nullptr;  // the caller's array is not kept
    } else {
      // q | k | v stay contiguous (a convolution channel is a column); the inner projections start on a
      // multiple of 8 columns so that the second-stage projections read 16-byte aligned rows
      L.off_q = 0; L.off_k = G * DK; L.off_v = 2 * G * DK; L.off_b = L.off_v + H * DV;
      L.off_a1 = pad8(L.off_b + H); L.off_g1 = pad8(L.off_a1 + s.rank_decay); L.n_in = pad8(L.off_g1 + s.rank_gate);
      AL(L.mix_norm, (size_t)DV * 4);
      AL(L.w_a2, (size_t)H * DK * s.rank_decay * w);
      AL(L.w_g2, (size_t)H * DV * s.rank_gate * w);
      AL(L.conv_w, (size_t)(2 * G * DK + H * DV) * s.conv_taps * 4);
      AL(L.A_log, (size_t)H * 4);
      AL(L.dt_bias, (size_t)H * DK * 4);
    }
    const int n_ctx = (s.mixer == L3_MIX_MINGRU ? DK : H * DV) + (L.pair ? L.pair->n_ctx : 0);  // columns the output projection reads
    L.n_ctx = n_ctx - (L.pair ? L.pair->n_ctx : 0);
    L.in_base = 0; L.ctx_base = 0; L.ctx_ld = n_ctx;
    if (L.pair) { L.pair->in_base = L.n_in; L.pair->ctx_base = L.n_ctx; L.pair->ctx_ld = n_ctx; L.n_in += L.pair->n_in; L.pair->in_ld = L.n_in; }
    L.in_ld = L.n_in;  // n_in: the rows of the whole fused projection
    AL(L.w_in, (size_t)L.n_in * W * w);
    cudaMemset(L.w_in, 0, (size_t)L.n_in * W * w);  // padding rows project to zero
    AL(L.w_o, (size_t)W * n_ctx * w);
    if (L.pair) { L.pair->w_in = (char*)L.w_in + (size_t)L.pair->in_base * W * w; L.pair->w_o = (char*)L.w_o + (size_t)L.pair->ctx_base * w; }
    AL(L.norm1, (size_t)W * 4);
    if (c->token_shift) AL(L.shift, (size_t)W * 4);
    if (c->layer_scale) { AL(L.ls1, (size_t)W * 4); if (s.ff > 0) AL(L.ls2, (size_t)W * 4); }
    if (c->canon_taps > 0) { AL(L.canon1, (size_t)W * c->canon_taps * 4); if (s.ff > 0) AL(L.canon2, (size_t)W * c->canon_taps * 4); }
    if (c->depth_avg) AL(L.dwa, (size_t)(i + 2) * 4);
    if (s.experts > 0 && s.router_kind == L3_ROUTE_SIGMOID_IN) {
      L.ff_total = s.experts * s.ff + s.shared_ff;
      AL(L.w13, (size_t)2 * L.ff_total * W * w);
      AL(L.w2, (size_t)W * L.ff_total * w);
      AL(L.router, (size_t)s.experts * W * 4);
    } else if (s.ff > 0 && s.ff_kind == L3_FF_POLYNORM) {
      AL(L.w13, (size_t)s.ff * W * w);
      AL(L.w2, (size_t)W * s.ff * w);
      AL(L.poly, 4 * 4);
    } else if (s.experts > 0) {
      AL(L.w13, (size_t)s.experts * s.ff * W * w);
      AL(L.w2, (size_t)W * s.experts * s.ff * w);
      AL(L.norm2, (size_t)W * 4);
      AL(L.router, (size_t)(s.experts + s.identity) * W * 4);
      AL(L.correction, (size_t)(s.experts + s.identity) * 4);
    } else if (s.ff > 0) {
      AL(L.w13, (size_t)2 * s.ff * W * w);
      AL(L.w2, (size_t)W * s.ff * w);
      if (!c->parallel) AL(L.norm2, (size_t)W * 4);
    }
    if (sd) {
      AL(L.side_gate, (size_t)sd * W * w);
      AL(L.side_proj, (size_t)W * sd * w);
      AL(L.side_norm, (size_t)W * 4);
    }
    ll->max_in = std::max(ll->max_in, L.n_in);
    ll->max_o = std::max(ll->max_o, std::max(std::max(H * DV, H * DK), n_ctx));
    if (L.pair) ll->max_o = std::max(ll->max_o, std::max(L.pair->spec.heads * L.pair->spec.vdim, L.pair->spec.heads * L.pair->spec.dim));
    if (L.ff_total) ll->max_ff = std::max(ll->max_ff, L.ff_total);
    if (s.mixer == L3_MIX_LATENT) ll->max_o = std::max(ll->max_o, H * s.kv_rank);
    ll->max_ff = std::max(ll->max_ff, s.experts > 0 ? s.experts * s.ff : s.ff);
  }
  if (c->loop_times > 0 && !c->loop_in) AL(ll->loop_step, (size_t)c->loop_times * W * 4);
  if (c->loop_in) AL(ll->loop_in, (size_t)W * 2 * W * w);
  if (c->embed_norm) AL(ll->embed_norm, (size_t)W * 4);
#undef AL
  // execution order: the layers ahead of the loop, the looped block loop_times times, the rest
  auto run = [&](int layer, int pass) { LLRun r; r.layer = layer; r.pass = pass; ll->runs.push_back(r); };
  if (c->loop_times > 0) {
    for (int i = 0; i < c->loop_start; ++i) run(i, -1);
    for (int t = 0; t < c->loop_times; ++t)
      for (int i = c->loop_start; i < c->loop_stop; ++i) run(i, i == c->loop_start ? t : -1);
    for (int i = c->loop_stop; i < c->n_layers; ++i) run(i, -1);
  } else {
    for (int i = 0; i < c->n_layers; ++i) run(i, -1);
  }
  ll->state.resize(ll->runs.size());
  ll->slot_pos.assign(c->max_batch_size, 0);
  *out = m;
  return L3_OK;
}

// ------------------------------------------------------------------------------ tensors by name
// Where a named tensor lives: destination, its logical shape, and the row mapping inside a fused matrix.
struct LLPlace {
  void* dst = nullptr;
  bool wt = true;        // stored in the model dtype (false: fp32 vector / table)
  int64_t rows = 0, cols = 1;
  int row0 = 0, row_stride = 1, ld = 1;
  bool one_plus = false; // stored as 1 + w
  bool broadcast = false;  // the checkpoint holds one number, the device vector `rows` copies of it
  float scale = 0.f, bias = 0.f;  // random init
};

// Tensors of a unit mixer (window attention, state-space, gated linear attention, gated delta rule); r = "mix.<name>"
static bool ll_place_unit(L3Model* m, LLLayer& L, const std::string& r, LLPlace* p) {
  const int W = m->ll->cfg.width;
  const L3LayerSpec& s = L.spec;
  const int H = s.heads, G = s.kv_heads, DK = s.dim, DV = s.vdim;
  auto mat = [&](void* d, int64_t rows, int64_t cols, int row0 = 0) {
    p->dst = d; p->wt = true; p->rows = rows; p->cols = cols; p->row0 = row0; p->row_stride = 1; p->ld = (int)cols;
    p->scale = 1.0f / sqrtf((float)cols);
    return d != nullptr;
  };
  auto vec = [&](float* d, int64_t n, float bias, float scale) {
    p->dst = d; p->wt = false; p->rows = n; p->cols = 1; p->ld = 1; p->bias = bias; p->scale = scale;
    return d != nullptr;
  };
  auto seg = [&](int off, int64_t rows, float mul = 1.f) { const bool ok = mat(L.w_in, rows, W, off); p->scale *= mul; return ok; };
  auto conv = [&](int ch0, int64_t rows) {
    p->dst = L.conv_w + (size_t)ch0 * s.conv_taps; p->wt = false; p->rows = rows; p->cols = s.conv_taps; p->ld = s.conv_taps;
    p->scale = 1.0f / sqrtf((float)s.conv_taps);
    return true;
  };
  if (r == "mix.o") {  // this mixer's columns of the layer's output projection
    const bool ok = mat(L.w_o, W, L.n_ctx);
    p->ld = L.ctx_ld;
    return ok;
  }
  if (s.mixer == L3_MIX_WINDOW) {
    if (r == "mix.q") return seg(L.off_q, (int64_t)H * DK, 2.f);
    if (r == "mix.k") return seg(L.off_k, (int64_t)G * DK, 2.f);
    if (r == "mix.v") return seg(L.off_v, (int64_t)G * DV);
    if (r == "mix.sink") return s.attn_kind == L3_ATTN_SINK && vec(L.head_vec, H, 0.5f, 0.5f);
    if (r == "mix.pb") return s.attn_kind == L3_ATTN_SIGMOID && vec(L.head_vec, H, -2.f, 0.5f);
    return false;
  }
  if (s.mixer == L3_MIX_SSD) {
    const int inner = H * DV, gn = G * DK;
    if (r == "mix.in") return seg(0, (int64_t)2 * inner + 2 * gn + H);
    if (r == "mix.conv") return conv(0, inner + 2 * gn);
    if (r == "mix.conv.b") return vec(L.conv_b, inner + 2 * gn, 0.f, 0.1f);
    if (r == "mix.dt_bias") return vec(L.dt_bias, H, -1.f, 0.5f);
    if (r == "mix.A_log") return vec(L.A_log, H, 0.f, 0.5f);
    if (r == "mix.D") return vec(L.skip_d, H, 1.f, 0.2f);
    if (r == "mix.norm") return vec(L.mix_norm, inner, 1.f, 0.1f);
    return false;
  }
  if (s.mixer == L3_MIX_GLA) {
    if (r == "mix.q") return seg(L.off_q, (int64_t)H * DK, 2.f);
    if (r == "mix.k") return seg(L.off_k, (int64_t)H * DK, 2.f);
    if (r == "mix.v") return seg(L.off_v, (int64_t)H * DV);
    if (r == "mix.g") return seg(L.off_g, (int64_t)H * DV);
    if (r == "mix.a1") return seg(L.off_a1, s.rank_decay);
    if (r == "mix.a2") return mat(L.w_a2, (int64_t)H * DK, s.rank_decay);
    if (r == "mix.a2.b") return vec(L.a2_bias, (int64_t)H * DK, 3.f, 1.f);
    if (r == "mix.norm") return vec(L.mix_norm, DV, 1.f, 0.1f);
    return false;
  }
  const int nq = G * DK, nv = H * DV;
  if (r == "mix.q") return seg(L.off_q, nq, 2.f);
  if (r == "mix.k") return seg(L.off_k, nq, 2.f);
  if (r == "mix.v") return seg(L.off_v, nv, 2.f);
  if (r == "mix.b") return seg(L.off_b, H);
  if (r == "mix.a1") return seg(L.off_a1, s.rank_decay);
  if (r == "mix.g1") return seg(L.off_g1, s.rank_gate);
  if (r == "mix.a2") return mat(L.w_a2, (int64_t)H * DK, s.rank_decay);
  if (r == "mix.g2") return mat(L.w_g2, nv, s.rank_gate);
  if (r == "mix.norm") return vec(L.mix_norm, DV, 1.f, 0.1f);
  if (r == "mix.A_log") return vec(L.A_log, H, 0.f, 0.5f);
  if (r == "mix.dt_bias") return vec(L.dt_bias, (int64_t)H * DK, -1.f, 0.5f);
  if (r == "mix.q.conv") return conv(0, nq);
  if (r == "mix.k.conv") return conv(nq, nq);
  if (r == "mix.v.conv") return conv(2 * nq, nv);
  return false;
}

static std::vector<const char*> ll_unit_names(const L3LayerSpec& s) {
  if (s.mixer == L3_MIX_WINDOW) return {"q", "k", "v", s.attn_kind == L3_ATTN_SIGMOID ? "pb" : "sink", "o"};
  if (s.mixer == L3_MIX_SSD) return {"in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o"};
  if (s.mixer == L3_MIX_GLA) return {"q", "k", "v", "g", "a1", "a2", "a2.b", "norm", "o"};
  return {"q", "k", "v", "b", "a1", "a2", "g1", "g2", "norm", "A_log", "dt_bias", "q.conv", "k.conv", "v.conv", "o"};
}

static bool ll_place(L3Model* m, const std::string& name, LLPlace* p) {
  LayerList* ll = m->ll;
  const int W = ll->cfg.width, V = ll->cfg.vocab, sd = ll->cfg.side_dim, NL = ll->cfg.n_layers;
  const bool op = ll->cfg.norm_one_plus != 0;
  *p = LLPlace{};
  auto mat = [&](void* d, int64_t r, int64_t c, int row0 = 0, int stride = 1) {
    p->dst = d; p->wt = true; p->rows = r; p->cols = c; p->row0 = row0; p->row_stride = stride; p->ld = (int)c;
    p->scale = 1.0f / sqrtf((float)c);
    return d != nullptr;
  };
  auto vec = [&](float* d, int64_t n, float bias, float scale, bool one_plus = false) {
    p->dst = d; p->wt = false; p->rows = n; p->cols = 1; p->ld = 1; p->bias = bias; p->scale = scale; p->one_plus = one_plus;
    return d != nullptr;
  };
  const bool pre = ll->cfg.norm_input != 0;
  // a layer norm's weight: [width], or one number spread over the vector
  auto norm = [&](float* d) {
    const bool ok = vec(d, W, op && !pre ? 0.f : 1.f, 0.1f, op && !pre);
    p->broadcast = ll->cfg.norm_scalar != 0;
    return ok;
  };
  // fp32 matrix (router tables, step vectors)
  auto fmat = [&](float* d, int64_t r, int64_t c, float scale) {
    p->dst = d; p->wt = false; p->rows = r; p->cols = c; p->ld = (int)c; p->scale = scale;
    return d != nullptr;
  };
  if (name == "embed") { const bool ok = mat(m->embed, V, W); p->scale = pre ? 0.1f : 1.0f; return ok; }
  if (name == "head") return mat(m->lm_head, V, W);
  if (name == "final.norm") return norm(m->norm_final);
  if (name == "loop.step") return ll->loop_step && fmat(ll->loop_step, ll->cfg.loop_times, W, 0.3f);
  if (name == "loop.in") { const bool ok = ll->loop_in && mat(ll->loop_in, W, (int64_t)2 * W); p->scale *= 1.4f; return ok; }
  if (name == "embed.norm") return ll->embed_norm && norm(ll->embed_norm);
  if (name == "side.embed") { const bool ok = sd && mat(ll->side_embed, V, (int64_t)NL * sd); p->scale = 1.0f; return ok; }
  int li = -1, n = 0;
  if (sscanf(name.c_str(), "l%d.%n", &li, &n) < 1 || n == 0 || li < 0 || li >= NL) return false;
  const std::string r = name.substr(n);
  LLLayer& L = ll->layers[li];
  const L3LayerSpec& s = L.spec;
  const int H = s.heads, G = s.kv_heads, DK = s.dim, DV = s.vdim;
  if (r == "norm1") return norm(L.norm1);
  if (r == "norm2") return s.ff > 0 && L.norm2 && norm(L.norm2);
  if (r == "ls1") return L.ls1 && vec(L.ls1, W, 1.f, 0.2f);
  if (r == "ls2") return L.ls2 && vec(L.ls2, W, 1.f, 0.2f);
  if (r == "canon1") return L.canon1 && fmat(L.canon1, W, ll->cfg.canon_taps, 0.3f / (float)ll->cfg.canon_taps);
  if (r == "canon2") return L.canon2 && fmat(L.canon2, W, ll->cfg.canon_taps, 0.3f / (float)ll->cfg.canon_taps);
  if (r == "dwa") return L.dwa && vec(L.dwa, li + 2, 1.f / (float)(li + 2), 0.3f / (float)(li + 2));
  if (L.ff_total) {  // sigmoid-routed gated experts + shared expert: gate / up rows interleaved, expert by expert
    if (r == "mlp.router") return fmat(L.router, s.experts, W, 3.0f / sqrtf((float)W));
    int e = -1, n2 = 0;
    std::string part;
    int off = -1, width = 0;
    if (sscanf(r.c_str(), "mlp.e%d.%n", &e, &n2) >= 1 && n2 > 0 && e >= 0 && e < s.experts) { part = r.substr(n2); off = e * s.ff; width = s.ff; }
    else if (s.shared_ff > 0 && r.compare(0, 11, "mlp.shared.") == 0) { part = r.substr(11); off = s.experts * s.ff; width = s.shared_ff; }
    if (off >= 0) {
      if (part == "gate") return mat(L.w13, width, W, 2 * off, 2);
      if (part == "up") return mat(L.w13, width, W, 2 * off + 1, 2);
      if (part == "down") {
        const bool ok = mat((char*)L.w2 + (size_t)off * wb(m), W, width);
        p->ld = L.ff_total;
        return ok;
      }
    }
    if (r.compare(0, 4, "mlp.") == 0) return false;
  }
  if (L.poly) {
    if (r == "mlp.up") return mat(L.w13, s.ff, W);
    if (r == "mlp.down") return mat(L.w2, W, s.ff);
    if (r == "mlp.act") return vec(L.poly, 4, 0.4f, 0.2f);
    if (r.compare(0, 4, "mlp.") == 0) return false;
  }
  if (r == "shift") return L.shift && vec(L.shift, W, 0.5f, 0.5f);
  if (s.experts > 0) {
    const int n = s.experts + s.identity;
    if (r == "mlp.router") return fmat(L.router, n, W, 3.0f / sqrtf((float)W));
    if (r == "mlp.correction") return vec(L.correction, n, 0.f, 0.05f);
    int e = -1, n2 = 0;
    if (sscanf(r.c_str(), "mlp.e%d.%n", &e, &n2) >= 1 && n2 > 0 && e >= 0 && e < s.experts) {
      const std::string part = r.substr(n2);
      if (part == "up") return mat(L.w13, s.ff, W, e * s.ff, 1);
      if (part == "down") {  // columns [e ff, (e + 1) ff) of the [width, experts * ff] matrix
        const bool ok = mat((char*)L.w2 + (size_t)e * s.ff * wb(m), W, s.ff);
        p->ld = s.experts * s.ff;
        return ok;
      }
    }
    if (r.compare(0, 4, "mlp.") == 0) return false;
  } else {
    if (r == "mlp.gate") return s.ff > 0 && mat(L.w13, s.ff, W, 0, 2);
    if (r == "mlp.up") return s.ff > 0 && mat(L.w13, s.ff, W, 1, 2);
    if (r == "mlp.down") return s.ff > 0 && mat(L.w2, W, s.ff);
  }
  if (r == "side.gate") return sd && mat(L.side_gate, sd, W);
  if (r == "side.proj") return sd && mat(L.side_proj, W, sd);
  if (r == "side.norm") return sd && vec(L.side_norm, W, 1.f, 0.1f);
  if (pre && !ll->cfg.parallel && unit_mixer(s.mixer)) {
    if (!L.pair) return ll_place_unit(m, L, r, p);
    if (r.compare(0, 9, "mix.left.") == 0) return ll_place_unit(m, L, "mix." + r.substr(9), p);
    if (r.compare(0, 10, "mix.right.") == 0) return ll_place_unit(m, *L.pair, "mix." + r.substr(10), p);
    return false;
  }
  if (r == "mix.o") return mat(L.w_o, W, s.mixer == L3_MIX_MINGRU ? (int64_t)DK : (int64_t)H * DV);
  auto seg = [&](int off, int64_t rows) { const bool ok = mat(L.w_in, rows, W, off, 1); return ok; };
  if (s.mixer == L3_MIX_LATENT) {
    if (r == "mix.dq") return seg(L.off_q, s.q_rank);
    if (r == "mix.dkv") { const bool ok = seg(L.off_k, (int64_t)s.kv_rank + s.rot_dim); p->scale *= 2.f; return ok; }
    if (r == "mix.g") return seg(L.off_g, H);
    if (r == "mix.dq.norm") return vec(L.q_norm, s.q_rank, 1.f, 0.1f);
    if (r == "mix.dkv.norm") return vec(L.k_norm, s.kv_rank, 1.f, 0.1f);
    if (r == "mix.uq") { const bool ok = mat(L.w_uq, (int64_t)H * (DK + s.rot_dim), s.q_rank); p->scale *= 2.f; return ok; }
    if (r == "mix.uk") { const bool ok = mat(L.w_uk, (int64_t)H * DK, s.kv_rank); p->scale *= 2.f; return ok; }
    if (r == "mix.uv") return mat(L.w_uv, (int64_t)H * DV, s.kv_rank);
    return false;
  }
  if (s.mixer == L3_MIX_DIFF) {
    auto bias = [&](int off, int64_t n) { return vec(L.in_bias + off, n, 0.f, 0.2f); };
    if (r == "mix.q") return seg(L.off_q, (int64_t)2 * H * DK);
    if (r == "mix.k") return seg(L.off_k, (int64_t)2 * G * DK);
    if (r == "mix.v") return seg(L.off_v, (int64_t)G * DV);
    if (r == "mix.q.b") return bias(L.off_q, (int64_t)2 * H * DK);
    if (r == "mix.k.b") return bias(L.off_k, (int64_t)2 * G * DK);
    if (r == "mix.v.b") return bias(L.off_v, (int64_t)G * DV);
    if (r == "mix.q.norm") return vec(L.q_norm, DK, 1.f, 0.1f);
    if (r == "mix.k.norm") return vec(L.k_norm, DK, 1.f, 0.1f);
    if (r == "mix.lq1") return vec(L.lam_vec, DK, 0.f, 0.2f);
    if (r == "mix.lk1") return vec(L.lam_vec + DK, DK, 0.f, 0.2f);
    if (r == "mix.lq2") return vec(L.lam_vec + 2 * DK, DK, 0.f, 0.2f);
    if (r == "mix.lk2") return vec(L.lam_vec + 3 * DK, DK, 0.f, 0.2f);
    return false;
  }
  if (s.mixer == L3_MIX_MINGRU) {
    if (r == "mix.z") return seg(L.off_b, DK);
    if (r == "mix.x") return seg(L.off_v, DK);
    if (r == "mix.g") return seg(L.off_g, DK);
    if (r == "mix.z.b") return vec(L.in_bias, DK, 0.f, 1.0f);
    if (r == "mix.x.b") return vec(L.in_bias + DK, DK, 0.f, 0.5f);
    return false;
  }
  if (s.mixer == L3_MIX_SOFTMAX) {
    if (r == "mix.q") return seg(L.off_q, (int64_t)H * DK);
    if (r == "mix.k") return seg(L.off_k, (int64_t)G * DK);
    if (r == "mix.g") return seg(L.off_g, H);
    if (r == "mix.q.norm") return vec(L.q_norm, (int64_t)H * DK, 1.f, 0.1f);
    if (r == "mix.k.norm") return vec(L.k_norm, (int64_t)G * DK, 1.f, 0.1f);
    return false;
  }
  if (s.mixer == L3_MIX_DECAY_LINEAR) {
    if (r == "mix.q") { const bool ok = seg(L.off_q, (int64_t)H * DK); p->scale *= 2.f; return ok; }
    if (r == "mix.k") { const bool ok = seg(L.off_k, (int64_t)H * DK); p->scale *= 2.f; return ok; }
    if (r == "mix.v") { const bool ok = seg(L.off_v, (int64_t)H * DV); p->scale *= 2.f; return ok; }
    if (r == "mix.g") return seg(L.off_g, (int64_t)H * DV);
    if (r == "mix.norm") return vec(L.mix_norm, (int64_t)H * DV, 1.f, 0.1f);
    return false;
  }
  const int nq = G * DK, nv = H * DV;
  if (r == "mix.q") { const bool ok = seg(L.off_q, nq); p->scale *= 2.f; return ok; }
  if (r == "mix.k") { const bool ok = seg(L.off_k, nq); p->scale *= 2.f; return ok; }
  if (r == "mix.v") { const bool ok = seg(L.off_v, nv); p->scale *= 2.f; return ok; }
  if (r == "mix.b") return seg(L.off_b, H);
  if (r == "mix.a1") return seg(L.off_a1, s.rank_decay);
  if (r == "mix.g1") return seg(L.off_g1, s.rank_gate);
  if (r == "mix.a2") return mat(L.w_a2, (int64_t)H * DK, s.rank_decay);
  if (r == "mix.g2") return mat(L.w_g2, nv, s.rank_gate);
  if (r == "mix.norm") return vec(L.mix_norm, DV, 1.f, 0.1f);
  if (r == "mix.A_log") return vec(L.A_log, H, 0.f, 0.5f);
  if (r == "mix.dt_bias") return vec(L.dt_bias, (int64_t)H * DK, -1.f, 0.5f);
  auto conv = [&](int ch0, int64_t rows) {
    p->dst = L.conv_w + (size_t)ch0 * s.conv_taps; p->wt = false; p->rows = rows; p->cols = s.conv_taps; p->ld = s.conv_taps;
    p->scale = 1.0f / sqrtf((float)s.conv_taps);
    return true;
  };
  if (r == "mix.q.conv") return conv(0, nq);
  if (r == "mix.k.conv") return conv(nq, nq);
  if (r == "mix.v.conv") return conv(2 * nq, nv);
  return false;
}

static std::vector<std::string> ll_expected(const L3Model* m) {
  const LayerList* ll = m->ll;
  std::vector<std::string> v = {"embed", "head", "final.norm"};
  if (ll->cfg.side_dim) v.push_back("side.embed");
  if (ll->loop_step) v.push_back("loop.step");
  if (ll->loop_in) v.push_back("loop.in");
  if (ll->embed_norm) v.push_back("embed.norm");
  for (int i = 0; i < ll->cfg.n_layers; ++i) {
    const L3LayerSpec& s = ll->layers[i].spec;
    const std::string p = "l" + std::to_string(i) + ".";
    const bool unit = ll->cfg.norm_input && !ll->cfg.parallel && unit_mixer(s.mixer);
    std::vector<const char*> names = {"norm1"};
    if (!unit) names.push_back("mix.o");
    if (ll->cfg.token_shift) names.push_back("shift");
    if (unit) {
      const LLLayer& Lu = ll->layers[i];
      for (auto nme : ll_unit_names(s)) v.push_back(p + (Lu.pair ? "mix.left." : "mix.") + nme);
      if (Lu.pair) for (auto nme : ll_unit_names(Lu.pair->spec)) v.push_back(p + "mix.right." + nme);
    } else if (s.mixer == L3_MIX_LATENT) names.insert(names.end(), {"mix.dq", "mix.dq.norm", "mix.uq", "mix.dkv", "mix.dkv.norm", "mix.uk", "mix.uv", "mix.g"});
    else if (s.mixer == L3_MIX_MINGRU) names.insert(names.end(), {"mix.z", "mix.z.b", "mix.x", "mix.x.b", "mix.g"});
    else if (s.mixer == L3_MIX_DIFF) names.insert(names.end(), {"mix.q", "mix.q.b", "mix.k", "mix.k.b", "mix.v", "mix.v.b", "mix.q.norm", "mix.k.norm",
                                                                "mix.lq1", "mix.lk1", "mix.lq2", "mix.lk2"});
    else if (s.mixer == L3_MIX_SOFTMAX) names.insert(names.end(), {"mix.q", "mix.k", "mix.g", "mix.q.norm", "mix.k.norm"});
    else if (s.mixer == L3_MIX_DECAY_LINEAR) names.insert(names.end(), {"mix.q", "mix.k", "mix.v", "mix.g", "mix.norm"});
    else names.insert(names.end(), {"mix.q", "mix.k", "mix.v", "mix.b", "mix.a1", "mix.a2", "mix.g1", "mix.g2", "mix.norm",
                                    "mix.A_log", "mix.dt_bias", "mix.q.conv", "mix.k.conv", "mix.v.conv"});
    const LLLayer& Lx = ll->layers[i];
    if (Lx.ls1) names.push_back("ls1");
    if (Lx.ls2) names.push_back("ls2");
    if (Lx.canon1) names.push_back("canon1");
    if (Lx.canon2) names.push_back("canon2");
    if (Lx.dwa) names.push_back("dwa");
    if (Lx.ff_total) {
      names.push_back("mlp.router");
      for (int e = 0; e <= s.experts; ++e) {
        if (e == s.experts && s.shared_ff == 0) break;
        const std::string ep = p + (e == s.experts ? std::string("mlp.shared.") : "mlp.e" + std::to_string(e) + ".");
        v.push_back(ep + "gate"); v.push_back(ep + "up"); v.push_back(ep + "down");
      }
    } else if (Lx.poly) {
      names.insert(names.end(), {"mlp.up", "mlp.down", "mlp.act"});
    } else if (s.experts > 0) {
      names.insert(names.end(), {"norm2", "mlp.router", "mlp.correction"});
      for (int e = 0; e < s.experts; ++e) {
        v.push_back(p + "mlp.e" + std::to_string(e) + ".up");
        v.push_back(p + "mlp.e" + std::to_string(e) + ".down");
      }
    } else if (s.ff > 0) {
      if (Lx.norm2) names.push_back("norm2");
      names.insert(names.end(), {"mlp.gate", "mlp.up", "mlp.down"});
    }
    if (ll->cfg.side_dim) names.insert(names.end(), {"side.gate", "side.proj", "side.norm"});
    for (auto nme : names) v.push_back(p + nme);
  }
  return v;
}

extern "C" int l3_load_tensor(L3Model* m, const char* name, const float* host, const int64_t* shape, int ndim) {
  if (!m) return L3_EINVAL;
  REQUIRE(m, m->ll != nullptr, "l3_load_tensor needs a handle made by l3_create_stack");
  REQUIRE(m, !m->finalized, "l3_load_tensor after l3_finalize");
  CK(m, cudaSetDevice(m->cfg.device));
  LLPlace p;
  REQUIRE(m, ll_place(m, name, &p), "tensor '%s' does not belong to this model", name);
  REQUIRE(m, ndim == 1 || ndim == 2, "'%s': expected a vector or a matrix, got %d dimensions", name, ndim);
  const int64_t rows = shape[0], cols = ndim > 1 ? shape[1] : 1;
  if (p.broadcast) {
    REQUIRE(m, rows * cols == 1, "'%s': expected a single number, got [%lld, %lld]", name, (long long)rows, (long long)cols);
    const std::vector<float> v((size_t)p.rows, host[0]);
    CK(m, cudaMemcpy(p.dst, v.data(), v.size() * 4, cudaMemcpyHostToDevice));
    m->ll->loaded.insert(name);
    return L3_OK;
  }
  REQUIRE(m, rows == p.rows && cols == p.cols, "shape mismatch for '%s': got [%lld, %lld], want [%lld, %lld]", name,
          (long long)rows, (long long)cols, (long long)p.rows, (long long)p.cols);
  const size_t STAGE = (size_t)256 << 20;
  if (!m->stage) CK(m, cudaMalloc((void**)&m->stage, STAGE));
  const int64_t rows_per = std::max<int64_t>(1, (int64_t)(STAGE / (cols * sizeof(float))));
  for (int64_t r0 = 0; r0 < rows; r0 += rows_per) {
    const int64_t nr = std::min(rows_per, rows - r0);
    CK(m, cudaMemcpyAsync(m->stage, host + r0 * cols, (size_t)nr * cols * sizeof(float), cudaMemcpyHostToDevice, m->stream));
    CK(m, launch_pack_rows(m->stage, (int)nr, (int)cols, p.dst, p.wt && m->bf16, p.row0 + (int)r0 * p.row_stride, p.row_stride,
                           p.ld, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
  }
  if (p.one_plus) {
    CK(m, launch_add_one((float*)p.dst, (int)rows, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
  }
  m->ll->loaded.insert(name);
  return L3_OK;
}

// l3_fill_random for a layer-list handle: every expected tensor, deterministic in (seed, tensor index)
int ll_fill_random(L3Model* m, uint64_t seed) {
  uint32_t id = 1;
  for (const auto& name : ll_expected(m)) {
    LLPlace p;
    if (!ll_place(m, name, &p)) { set_err(m, "no place for '%s'", name.c_str()); return L3_ESTATE; }
    const float bias = p.one_plus ? p.bias + 1.0f : p.bias;
    CK(m, launch_fill_random(p.dst, p.wt && m->bf16, p.rows, p.cols, p.cols, 0, 0, p.row0, p.row_stride, p.ld, seed, id++,
                             p.scale, bias, m->stream));
    m->ll->loaded.insert(name);
  }
  CK(m, cudaStreamSynchronize(m->stream));
  return L3_OK;
}

// ------------------------------------------------------------------------------ finalize / destroy / state
// channels of a unit mixer's short convolutions (0: it has none)
static int unit_conv_channels(const L3LayerSpec& s) {
  if (s.mixer == L3_MIX_SSD) return s.heads * s.vdim + 2 * s.kv_heads * s.dim;
  if (s.mixer == L3_MIX_GATED_DELTA) return 2 * s.kv_heads * s.dim + s.heads * s.vdim;
  return 0;
}

// what a unit mixer keeps per sequence slot: KV caches (window attention) or a state matrix per head (+ convolution tail)
static int ll_alloc_unit_state(L3Model* m, const L3LayerSpec& s, LLState& St) {
  const size_t kvb = m->bf16 ? 2 : 4;
  if (s.mixer == L3_MIX_WINDOW) {
    CK(m, cudaMalloc(&St.ck, (size_t)m->maxB * s.kv_heads * m->M * s.dim * kvb));
    CK(m, cudaMalloc(&St.cv, (size_t)m->maxB * s.kv_heads * m->M * s.vdim * kvb));
    return L3_OK;
  }
  CK(m, cudaMalloc((void**)&St.S, (size_t)m->maxB * s.heads * s.dim * s.vdim * 4));
  const int C = unit_conv_channels(s);
  if (C) CK(m, cudaMalloc((void**)&St.conv_tail, std::max<size_t>(16, (size_t)m->maxB * C * (s.conv_taps - 1) * 4)));
  return L3_OK;
}

static int ll_reset_unit_state(L3Model* m, const L3LayerSpec& s, LLState& St, int slot0, int n, bool kv_too) {
  const size_t kvb = m->bf16 ? 2 : 4;
  if (s.mixer == L3_MIX_WINDOW) {
    if (!kv_too) return L3_OK;  // rows past a slot's position are never read: a new sequence overwrites them
    const size_t pk = (size_t)s.kv_heads * m->M * s.dim * kvb, pv = (size_t)s.kv_heads * m->M * s.vdim * kvb;
    CK(m, cudaMemsetAsync((char*)St.ck + slot0 * pk, 0, n * pk, m->stream));
    CK(m, cudaMemsetAsync((char*)St.cv + slot0 * pv, 0, n * pv, m->stream));
    return L3_OK;
  }
  const size_t per = (size_t)s.heads * s.dim * s.vdim;
  CK(m, cudaMemsetAsync(St.S + slot0 * per, 0, n * per * 4, m->stream));
  const size_t pc = (size_t)unit_conv_channels(s) * (s.conv_taps - 1);
  if (pc) CK(m, cudaMemsetAsync(St.conv_tail + slot0 * pc, 0, n * pc * 4, m->stream));
  return L3_OK;
}

int ll_finalize(L3Model* m) {
  LayerList* ll = m->ll;
  for (const auto& name : ll_expected(m))
    if (!ll->loaded.count(name)) { set_err(m, "tensor '%s' was never loaded", name.c_str()); return L3_ESTATE; }
  if (m->stage) { cudaFree(m->stage); m->stage = nullptr; }
  const size_t kvb = m->bf16 ? 2 : 4;
  int max_rq = 1, max_rk = 1, max_rv = 1, max_rg = 1, max_h = 1, max_aux = 1, max_qlat = 0, max_top = 0, max_exp = 0, max_hid = 1, max_gu = 0;
  for (size_t ri = 0; ri < ll->runs.size(); ++ri) {
    const LLLayer& L = ll->layers[ll->runs[ri].layer];
    LLState& St = ll->state[ri];
    const L3LayerSpec& s = L.spec;
    const int H = s.heads, G = s.kv_heads, DK = s.dim, DV = s.vdim;
    if (ll->cfg.token_shift) CK(m, cudaMalloc((void**)&St.hprev, (size_t)m->maxB * m->D * 4));
    if (ll->cfg.canon_taps > 1) CK(m, cudaMalloc((void**)&St.conv_tail, (size_t)m->maxB * m->D * (ll->cfg.canon_taps - 1) * 4));
    if (ll->cfg.norm_input && !ll->cfg.parallel && unit_mixer(s.mixer)) {
      int rc = ll_alloc_unit_state(m, s, St);
      if (rc == L3_OK && L.pair) { St.pair = new LLState(); rc = ll_alloc_unit_state(m, L.pair->spec, *St.pair); }
      if (rc != L3_OK) return rc;
    } else if (s.mixer == L3_MIX_LATENT) {
      CK(m, cudaMalloc(&St.lat, (size_t)m->maxB * m->M * (s.kv_rank + s.rot_dim) * kvb));
    } else if (s.mixer == L3_MIX_DIFF) {
      CK(m, cudaMalloc(&St.ck, (size_t)m->maxB * 2 * G * m->M * DK * kvb));
      CK(m, cudaMalloc(&St.cv, (size_t)m->maxB * G * m->M * DV * kvb));
    } else if (s.mixer == L3_MIX_SOFTMAX) {
      const size_t bytes = (size_t)m->maxB * G * m->M * DK * kvb;
      CK(m, cudaMalloc(&St.ck, bytes));
      CK(m, cudaMalloc(&St.cv, bytes));
    } else {
      CK(m, cudaMalloc((void**)&St.S, (size_t)m->maxB * H * DK * DV * 4));
      if (s.mixer == L3_MIX_GATED_DELTA) {
        const int C = 2 * G * DK + H * DV;
        CK(m, cudaMalloc((void**)&St.conv_tail, std::max<size_t>(16, (size_t)m->maxB * C * (s.conv_taps - 1) * 4)));
      }
    }
  }
  const bool units = ll->cfg.norm_input && !ll->cfg.parallel;
  int max_xs = 0;
  size_t win_part = 0;
  for (auto& L0 : ll->layers)
    for (const LLLayer* U = &L0; units && U; U = U->pair) {  // the unit mixers' share of the workspace
      const L3LayerSpec& s = U->spec;
      const int H = s.heads, G = s.kv_heads, DK = s.dim, DV = s.vdim;
      if (s.mixer == L3_MIX_WINDOW) {
        max_rq = std::max(max_rq, H * DK);
        win_part = std::max(win_part, win_attn_part_floats(m->maxB * 8, H, DV, 32));
      } else if (s.mixer == L3_MIX_SSD) {
        max_rq = std::max(max_rq, G * DK); max_rk = std::max(max_rk, G * DK); max_rv = std::max(max_rv, H * DV);
        max_rg = std::max(max_rg, 2 * H); max_xs = std::max(max_xs, H * DV);  // decays and their logarithms
      } else if (s.mixer == L3_MIX_GLA) {
        max_rq = std::max(max_rq, H * DK); max_rg = std::max(max_rg, H * DK); max_aux = std::max(max_aux, H * DK);
      }
    }
  for (auto& L : ll->layers) {
    const L3LayerSpec& s = L.spec;
    const int H = s.heads, G = s.kv_heads, DK = s.dim, DV = s.vdim;
    if (L.pair && L.pair->spec.mixer == L3_MIX_GATED_DELTA) {
      const L3LayerSpec& r = L.pair->spec;
      max_rq = std::max(max_rq, r.kv_heads * r.dim); max_rk = std::max(max_rk, r.kv_heads * r.dim); max_rv = std::max(max_rv, r.heads * r.vdim);
      max_rg = std::max(max_rg, r.heads * r.dim); max_h = std::max(max_h, r.heads); max_aux = std::max(max_aux, r.heads * r.dim + r.heads * r.vdim);
    }
    for (int k = 0; k < 2; ++k) {  // the convolutions' taps, tap-major for the kernels
      float* src = k ? L.canon2 : L.canon1;
      float** dst = k ? &L.canon2t : &L.canon1t;
      if (!src) continue;
      if (!*dst) CK(m, cudaMalloc((void**)dst, (size_t)m->D * ll->cfg.canon_taps * 4));
      LAUNCH(m, launch_transpose_f32(src, m->D, ll->cfg.canon_taps, *dst, m->stream));
    }
    if (s.mixer == L3_MIX_SOFTMAX) {
      max_rq = std::max(max_rq, H * DK);
    } else if (s.mixer == L3_MIX_DIFF) {
      max_rq = std::max(max_rq, 2 * H * DK);
      LAUNCH(m, launch_diff_lambda(L.lam_vec, DK, s.diff, L.lambda, m->stream));
    } else if (s.mixer == L3_MIX_GATED_DELTA) {
      max_rq = std::max(max_rq, G * DK); max_rk = std::max(max_rk, G * DK); max_rv = std::max(max_rv, H * DV);
      max_rg = std::max(max_rg, H * DK); max_h = std::max(max_h, H); max_aux = std::max(max_aux, H * DK + H * DV);
    } else if (s.mixer == L3_MIX_LATENT) {
      max_rq = std::max(max_rq, H * (DK + s.rot_dim));
      max_aux = std::max(max_aux, s.q_rank);
      max_qlat = std::max(max_qlat, H * (s.kv_rank + s.rot_dim));
    }
    if (s.experts > 0) { max_top = std::max(max_top, s.top); max_exp = std::max(max_exp, s.experts); max_hid = std::max(max_hid, (s.top + 1) * std::max(s.ff, s.shared_ff)); }
    max_gu = std::max(max_gu, 2 * L.ff_total);
  }
  const int W = m->D, sd = ll->cfg.side_dim;
  const int64_t want = (int64_t)m->maxB * m->M;
  m->cap_tok = (int)std::max<int64_t>(m->maxB, std::min<int64_t>(want, 8192));
  const size_t ct = (size_t)m->cap_tok;
  CK(m, cudaMalloc((void**)&m->x, ct * W * 4));
  CK(m, cudaMalloc((void**)&ll->x2, (size_t)8 * W * 4));  // second residual buffer of the fused post-norm step (<= 8 rows)
  CK(m, cudaMalloc((void**)&m->xn, ct * W * 4));  // sublayer output before its norm
  CK(m, cudaMalloc((void**)&m->q, ct * max_rq * 4));
  CK(m, cudaMalloc((void**)&m->ctx, ct * ll->max_o * 4));
  CK(m, cudaMalloc((void**)&m->h, std::max(ct * std::max(1, ll->max_ff), (size_t)8 * max_hid) * 4));
  CK(m, cudaMalloc((void**)&m->xlast, (size_t)m->maxB * W * 4));
  CK(m, cudaMalloc((void**)&m->logits, (size_t)m->maxB * m->VS * 4));
  CK(m, cudaMalloc((void**)&ll->pin, ct * ll->max_in * 4));
  CK(m, cudaMalloc((void**)&ll->aux, ct * max_aux * 4));
  CK(m, cudaMalloc((void**)&ll->rk, ct * max_rk * 4));
  CK(m, cudaMalloc((void**)&ll->rv, ct * max_rv * 4));
  CK(m, cudaMalloc((void**)&ll->rg, ct * max_rg * 4));
  CK(m, cudaMalloc((void**)&ll->rbeta, ct * max_h * 4));
  CK(m, cudaMalloc((void**)&ll->o, ct * ll->max_o * 4));
  CK(m, cudaMalloc((void**)&ll->sg, ct * std::max(1, sd) * 4));
  if (max_qlat) CK(m, cudaMalloc((void**)&ll->qlat, ct * max_qlat * 4));
  if (max_xs) CK(m, cudaMalloc((void**)&ll->xs, ct * max_xs * 4));
  if (win_part) {
    CK(m, cudaMalloc((void**)&ll->win_part_o, win_part * 4));
    CK(m, cudaMalloc((void**)&ll->win_part_ml, win_part * 4));
  }
  if (ll->cfg.loop_in) {
    CK(m, cudaMalloc((void**)&ll->x0, ct * W * 4));
    CK(m, cudaMalloc((void**)&ll->cat, ct * 2 * W * 4));
  }
  if (ll->cfg.parallel) {
    if (ll->cfg.depth_avg) CK(m, cudaMalloc((void**)&ll->Xs, (size_t)(ll->cfg.n_layers + 1) * ct * W * 4));
    if (ll->cfg.canon_taps > 0) {
      CK(m, cudaMalloc((void**)&ll->hn, ct * W * 4));
      CK(m, cudaMalloc((void**)&ll->hf, ct * W * 4));
    }
    CK(m, cudaMalloc((void**)&ll->y1, ct * W * 4));
    CK(m, cudaMalloc((void**)&ll->y2, ct * W * 4));
    if (max_gu) CK(m, cudaMalloc((void**)&ll->moe_gu, ct * max_gu * 4));
    size_t part = 0;
    for (auto& L : ll->layers)
      if (L.spec.mixer == L3_MIX_DIFF) part = std::max(part, diff_attn_part_floats(m->maxB * 8, L.spec.heads, L.spec.vdim));
    if (part) {
      CK(m, cudaMalloc((void**)&ll->diff_part_o, part * 4));
      CK(m, cudaMalloc((void**)&ll->diff_part_ml, part * 4));
    }
  }
  if (max_top) {
    CK(m, cudaMalloc((void**)&ll->moe_sel, ct * max_top * 4));
    CK(m, cudaMalloc((void**)&ll->moe_w, ct * max_top * 4));
    CK(m, cudaMalloc((void**)&ll->moe_dense, ct * max_exp * 4));
    CK(m, cudaMalloc((void**)&ll->moe_idw, ct * 4));
  }
  for (const LLLayer& L0 : ll->layers)
    for (const LLLayer* U = &L0; U; U = U->pair) {
      const L3LayerSpec& s = U->spec;
      const bool chunked = s.mixer == L3_MIX_DECAY_LINEAR || (units && s.mixer == L3_MIX_SSD);
      if (chunked && recur_chunk_shape(s.dim, s.vdim) && ct >= 128)
        ll->chunk_ws_floats = std::max(ll->chunk_ws_floats, (ct / 64 + m->maxB) * ((size_t)s.heads * s.dim * s.vdim + s.heads));
    }
  if (ll->chunk_ws_floats) CK(m, cudaMalloc((void**)&ll->chunk_ws, ll->chunk_ws_floats * 4));
  // tensor cores: bf16 mode only.  fp32 mode is the exact mode of this family: every product is an fp32 FFMA chain
  // (the 3xTF32 scheme of the Llama path would need a (hi, lo) copy of the residual stream beside the stream itself).
  m->tc_ok = m->bf16 && !(m->cfg.flags & L3_FLAG_NO_TENSORCORE) && tc_gemm_supported(W);
  if (m->tc_ok) {
    if (!(getenv("L3_GEMM_KSPLIT") && atoi(getenv("L3_GEMM_KSPLIT")) == 0)) {
      CK(m, cudaMalloc((void**)&m->gemm_part, (size_t)32 << 20));
      CK(m, cudaMalloc((void**)&m->gemm_cnt, 1024 * sizeof(int)));
      CK(m, cudaMemsetAsync(m->gemm_cnt, 0, 1024 * sizeof(int), m->stream));
    }
    CK(m, cudaMalloc(&m->xn16, ct * W * 2));  // mirror of the residual stream
    CK(m, cudaMalloc(&m->ctx16, ct * ll->max_o * 2));
    CK(m, cudaMalloc(&m->h16, ct * std::max(1, ll->max_ff) * 2));
    CK(m, cudaMalloc(&m->xlast16, (size_t)m->maxB * W * 2));
    CK(m, cudaMalloc(&ll->sg16, ct * std::max(1, sd) * 2));
    if (max_qlat) CK(m, cudaMalloc(&ll->aux16, ct * max_aux * 2));
    if (ll->hf) CK(m, cudaMalloc(&ll->hf16, ct * W * 2));
    if (ll->cat) CK(m, cudaMalloc(&ll->cat16, ct * 2 * W * 2));
  }
  m->max_split = 32;
  int max_hn = 1, max_hd = 1;
  for (auto& L : ll->layers)
    if (L.spec.mixer == L3_MIX_SOFTMAX || L.spec.mixer == L3_MIX_DIFF) { max_hn = std::max(max_hn, L.spec.heads); max_hd = std::max(max_hd, L.spec.dim); }
    else if (L.spec.mixer == L3_MIX_LATENT) { max_hn = std::max(max_hn, L.spec.heads); max_hd = std::max(max_hd, L.spec.kv_rank); }
  CK(m, cudaMalloc((void**)&m->part_o, (size_t)m->maxB * max_hn * m->max_split * max_hd * 4));
  CK(m, cudaMalloc((void**)&m->part_ml, (size_t)m->maxB * max_hn * m->max_split * 2 * 4));
  CK(m, cudaMalloc((void**)&m->attn_cnt, (size_t)m->maxB * max_hn * 4));
  CK(m, cudaMemsetAsync(m->attn_cnt, 0, (size_t)m->maxB * max_hn * 4, m->stream));
  CK(m, cudaMalloc((void**)&m->d_ids, (size_t)m->maxB * m->M * 4));
  CK(m, cudaMalloc((void**)&m->d_next, (size_t)m->maxB * 4));
  CK(m, cudaMalloc((void**)&m->d_fwd_next, (size_t)m->maxB * 4));
  CK(m, cudaMalloc((void**)&m->d_fwd_ids, (size_t)m->maxB * m->M * 4));
  CK(m, cudaMalloc((void**)&m->d_scal, 16 * 4));
  CK(m, cudaMemsetAsync(m->d_scal, 0, 16 * 4, m->stream));
  CK(m, cudaMalloc((void**)&m->d_tokens, (size_t)m->maxB * m->M * 8));
  CK(m, cudaMalloc((void**)&m->d_fwd_arg, (size_t)m->maxB * 8));
  CK(m, cudaMalloc((void**)&m->d_best, (size_t)m->maxB * 8));
  CK(m, cudaMemsetAsync(m->d_best, 0, (size_t)m->maxB * 8, m->stream));
  CK(m, cudaMallocHost((void**)&m->h_next, (size_t)m->maxB * 4));
  cudaDeviceProp prop;
  CK(m, cudaGetDeviceProperties(&prop, m->cfg.device));
  m->n_sm = prop.multiProcessorCount;
  ll->head_rows = m->maxB;
  m->finalized = true;
  const int rc = ll_reset_slots(m, 0, m->maxB, true);
  if (rc != L3_OK) { m->finalized = false; return rc; }
  CK(m, cudaStreamSynchronize(m->stream));
  return L3_OK;
}

void ll_destroy(L3Model* m) {
  LayerList* ll = m->ll;
  if (!ll) return;
  auto fr = [](void* p) { if (p) cudaFree(p); };
  fr(ll->side_embed);
  for (auto& L : ll->layers) {
    fr(L.w_in); fr(L.w_o); fr(L.w_a2); fr(L.w_g2); fr(L.w13); fr(L.w2); fr(L.side_gate); fr(L.side_proj);
    fr(L.norm1); fr(L.norm2); fr(L.side_norm); fr(L.mix_norm); fr(L.q_norm); fr(L.k_norm); fr(L.conv_w);
    fr(L.A_log); fr(L.dt_bias); fr(L.decay);
    fr(L.w_uq); fr(L.w_uk); fr(L.w_uv); fr(L.inv_freq); fr(L.in_bias); fr(L.shift); fr(L.router); fr(L.correction);
    fr(L.canon1); fr(L.canon2); fr(L.canon1t); fr(L.canon2t); fr(L.ls1); fr(L.ls2); fr(L.dwa); fr(L.lam_vec); fr(L.lambda); fr(L.poly);
    fr(L.head_vec); fr(L.conv_b); fr(L.skip_d); fr(L.a2_bias);
    if (LLLayer* R = L.pair) {  // its w_in / w_o are views of the first mixer's
      fr(R->w_a2); fr(R->w_g2); fr(R->mix_norm); fr(R->conv_w); fr(R->A_log); fr(R->dt_bias); fr(R->inv_freq);
      fr(R->head_vec); fr(R->conv_b); fr(R->skip_d); fr(R->a2_bias);
      delete R;
      L.pair = nullptr;
    }
  }
  for (auto& St : ll->state) {
    fr(St.ck); fr(St.cv); fr(St.S); fr(St.conv_tail); fr(St.lat); fr(St.hprev);
    if (LLState* P = St.pair) { fr(P->ck); fr(P->cv); fr(P->S); fr(P->conv_tail); delete P; St.pair = nullptr; }
  }
  fr(ll->loop_in); fr(ll->embed_norm); fr(ll->x0); fr(ll->cat); fr(ll->cat16); fr(ll->win_part_o); fr(ll->win_part_ml); fr(ll->xs);
  fr(ll->diff_part_o); fr(ll->diff_part_ml);
  fr(ll->Xs); fr(ll->hn); fr(ll->hf); fr(ll->hf16); fr(ll->y1); fr(ll->y2); fr(ll->moe_gu);
  fr(ll->loop_step); fr(ll->qlat); fr(ll->aux16); fr(ll->moe_sel); fr(ll->moe_w); fr(ll->moe_dense); fr(ll->moe_idw);
  fr(ll->pin); fr(ll->aux); fr(ll->rk); fr(ll->rv); fr(ll->rg); fr(ll->rbeta); fr(ll->o); fr(ll->sg); fr(ll->sg16); fr(ll->x2); fr(ll->chunk_ws);
  delete ll;
  m->ll = nullptr;
}

int ll_reset_slots(L3Model* m, int slot0, int n, bool kv_too) {
  LayerList* ll = m->ll;
  const size_t kvb = m->bf16 ? 2 : 4;
  for (size_t ri = 0; ri < ll->runs.size(); ++ri) {
    const L3LayerSpec& s = ll->layers[ll->runs[ri].layer].spec;
    LLState& St = ll->state[ri];
    if (St.hprev) CK(m, cudaMemsetAsync(St.hprev + (size_t)slot0 * m->D, 0, (size_t)n * m->D * 4, m->stream));
    if (ll->cfg.norm_input && !ll->cfg.parallel && unit_mixer(s.mixer)) {
      int rc = ll_reset_unit_state(m, s, St, slot0, n, kv_too);
      if (rc == L3_OK && St.pair) rc = ll_reset_unit_state(m, ll->layers[ll->runs[ri].layer].pair->spec, *St.pair, slot0, n, kv_too);
      if (rc != L3_OK) return rc;
      continue;
    }
    if (s.mixer == L3_MIX_DIFF) {
      if (St.conv_tail) {  // zeros ahead of a sequence's first token
        const size_t pc = (size_t)m->D * (ll->cfg.canon_taps - 1);
        CK(m, cudaMemsetAsync(St.conv_tail + slot0 * pc, 0, n * pc * 4, m->stream));
      }
      if (!kv_too) continue;  // rows past a slot's position are never read
      const size_t pk = (size_t)2 * s.kv_heads * m->M * s.dim * kvb, pv = (size_t)s.kv_heads * m->M * s.vdim * kvb;
      CK(m, cudaMemsetAsync((char*)St.ck + slot0 * pk, 0, n * pk, m->stream));
      CK(m, cudaMemsetAsync((char*)St.cv + slot0 * pv, 0, n * pv, m->stream));
      continue;
    }
    if (s.mixer == L3_MIX_LATENT) {
      if (!kv_too) continue;  // rows past a slot's position are never read: a new sequence overwrites them
      const size_t per = (size_t)m->M * (s.kv_rank + s.rot_dim) * kvb;
      CK(m, cudaMemsetAsync((char*)St.lat + slot0 * per, 0, n * per, m->stream));
    } else if (s.mixer == L3_MIX_SOFTMAX) {
      if (!kv_too) continue;
      const size_t per = (size_t)s.kv_heads * m->M * s.dim * kvb;
      CK(m, cudaMemsetAsync((char*)St.ck + slot0 * per, 0, n * per, m->stream));
      CK(m, cudaMemsetAsync((char*)St.cv + slot0 * per, 0, n * per, m->stream));
    } else {
      const size_t per = (size_t)s.heads * s.dim * s.vdim;
      CK(m, cudaMemsetAsync(St.S + slot0 * per, 0, n * per * 4, m->stream));
      if (s.mixer == L3_MIX_GATED_DELTA && s.conv_taps > 1) {
        const size_t pc = (size_t)(2 * s.kv_heads * s.dim + s.heads * s.vdim) * (s.conv_taps - 1);
        CK(m, cudaMemsetAsync(St.conv_tail + slot0 * pc, 0, n * pc * 4, m->stream));
      }
    }
  }
  for (int b = slot0; b < slot0 + n; ++b) ll->slot_pos[b] = 0;
  return L3_OK;
}

int ll_begin_call(L3Model* m, int B, int L, int start_pos) {
  LayerList* ll = m->ll;
  if (start_pos == 0) {
    const int rc = ll_reset_slots(m, 0, B, false);
    if (rc != L3_OK) return rc;
  } else {
    for (int b = 0; b < B; ++b)
      if (ll->slot_pos[b] != start_pos) {
        set_err(m, "slot %d is at position %d, the call starts at %d: a recurrent state cannot be moved", b, ll->slot_pos[b], start_pos);
        return L3_ESTATE;
      }
  }
  for (int b = 0; b < B; ++b) ll->slot_pos[b] = start_pos + L;
  return L3_OK;
}

extern "C" int l3_stack_runs(L3Model* m, int* n_runs_out) {
  if (!m || !n_runs_out) return L3_EINVAL;
  REQUIRE(m, m->ll != nullptr, "l3_stack_runs needs a handle made by l3_create_stack");
  *n_runs_out = (int)m->ll->runs.size();
  return L3_OK;
}

extern "C" int l3_read_state(L3Model* m, int layer, int slot, float* S_out, float* conv_out) {
  if (!m || !m->finalized) return L3_ESTATE;
  REQUIRE(m, m->ll != nullptr, "l3_read_state needs a handle made by l3_create_stack");
  REQUIRE(m, layer >= 0 && layer < (int)m->ll->runs.size() && slot >= 0 && slot < m->maxB, "layer run / slot out of range");
  const LLLayer* Lp = &m->ll->layers[m->ll->runs[layer].layer];
  const LLState* Sp = &m->ll->state[layer];
  if (Lp->pair && Lp->spec.mixer == L3_MIX_WINDOW) { Lp = Lp->pair; Sp = Sp->pair; }  // two mixers side by side: the recurrent one
  const LLLayer& L = *Lp;
  const LLState& St = *Sp;
  const L3LayerSpec& s = L.spec;
  REQUIRE(m, s.mixer != L3_MIX_SOFTMAX && s.mixer != L3_MIX_DIFF && s.mixer != L3_MIX_WINDOW, "layer run %d keeps a KV cache, not a recurrent state (l3_read_cache)", layer);
  CK(m, cudaSetDevice(m->cfg.device));
  CK(m, cudaStreamSynchronize(m->stream));
  if (s.mixer == L3_MIX_LATENT) {
    REQUIRE(m, !conv_out, "layer run %d has no convolution", layer);
    const size_t per = (size_t)m->M * (s.kv_rank + s.rot_dim);
    if (!S_out) return L3_OK;
    if (!m->bf16) { CK(m, cudaMemcpy(S_out, (const float*)St.lat + slot * per, per * 4, cudaMemcpyDeviceToHost)); return L3_OK; }
    float* tmp = nullptr;
    CK(m, cudaMalloc((void**)&tmp, per * 4));
    cudaError_t e = launch_unpack_bf16((const bf16*)St.lat + slot * per, (int64_t)per, tmp, m->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(S_out, tmp, per * 4, cudaMemcpyDeviceToHost, m->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    cudaFree(tmp);
    CK(m, e);
    return L3_OK;
  }
  const size_t per = (size_t)s.heads * s.dim * s.vdim;
  if (S_out) CK(m, cudaMemcpy(S_out, St.S + slot * per, per * 4, cudaMemcpyDeviceToHost));
  if (conv_out) {
    REQUIRE(m, unit_conv_channels(s) > 0, "layer run %d has no convolution", layer);
    const size_t pc = (size_t)unit_conv_channels(s) * (s.conv_taps - 1);
    if (pc) CK(m, cudaMemcpy(conv_out, St.conv_tail + slot * pc, pc * 4, cudaMemcpyDeviceToHost));
  }
  return L3_OK;
}

// ------------------------------------------------------------------------------ projections
// A post-norm residual step  x += mult * y / rms(y) * w  that has been deferred: the next projection that reads x
// through the row-streaming GEMV applies it while staging its input (linear.cu) and writes the new rows to the other
// residual buffer; any other consumer has it applied by resid_postnorm_kernel first (ll_settle).
struct LLPending {
  const float* y = nullptr;
  const float* w = nullptr;
};

static int ll_settle(L3Model* m, LLPending& pd, int rows) {
  if (!pd.y) return L3_OK;
  LayerList* ll = m->ll;
  LAUNCH(m, launch_resid_postnorm(ll->xcur, pd.y, pd.w, ll->cfg.residual_mult, ll->cfg.norm_eps, rows, m->D, (bf16*)m->xn16, m->stream));
  pd.y = nullptr;
  return L3_OK;
}

// y = x W^T (+ epilogue).  x32: fp32 rows with stride lda (0 = K); x16: bf16 mirror with stride K, or null.
// pd: non-null when x32 is the residual stream (ll->xcur) - a deferred step is applied on the way.
static int ll_linear(L3Model* m, const void* W, const float* x32, const void* x16, int lda, int rows, int N, int K, int epi,
                     const EpiArgs& e, LLPending* pd = nullptr) {
  LayerList* ll = m->ll;
  LinearArgs a{};
  a.W = W; a.x = x32; a.lda = lda; a.rows = rows; a.N = N; a.K = K; a.src_mul = 1; a.src_add = 0; a.epi = epi; a.e = e;
  const int ld = lda ? lda : K;
  if (linear_rows_supported(rows, K) && ld % 4 == 0) {
    // the fused form costs every CTA a pass over x, y and w per row: it wins for one or two rows (0.85 -> 0.75 ms per
    // decode step of a 12-layer width-2048 model) and loses from four rows on (8 rows: 1.87 -> 2.08 ms)
    if (pd && pd->y && rows > 2) {
      const int rc = ll_settle(m, *pd, rows);
      if (rc != L3_OK) return rc;
    }
    if (pd && pd->y) {
      a.x = ll->xcur;
      a.post_y = pd->y; a.post_w = pd->w; a.post_mult = ll->cfg.residual_mult; a.post_eps = ll->cfg.norm_eps; a.post_out = ll->xalt;
      std::swap(ll->xcur, ll->xalt);
      pd->y = nullptr;
    } else if (pd) a.x = ll->xcur;
    LAUNCH(m, launch_linear_rows(a, m->bf16, m->bf16, m->stream));
    return L3_OK;
  }
  if (pd) {
    const int rc = ll_settle(m, *pd, rows);
    if (rc != L3_OK) return rc;
    a.x = ll->xcur;
  }
  if (m->tc_ok && x16 && ld == K && K % 8 == 0 && K >= 64 && N >= 64) {
    TcGemmArgs t{};
    t.kind = TC_BF16; t.A[0] = x16; t.W[0] = W;
    t.rows = rows; t.N = N; t.K = K; t.epi = epi; t.e = e; t.bn = 0;
    t.part = m->gemm_part; t.part_bytes = (size_t)32 << 20; t.tile_cnt = m->gemm_cnt; t.tile_cnt_len = 1024;
    static const bool swap_on = !(getenv("L3_GEMM_SWAP") && atoi(getenv("L3_GEMM_SWAP")) == 0);
    if (swap_on && gemm_swap_supported(rows, N)) LAUNCH(m, launch_gemm_swap(t, m->stream));
    else LAUNCH(m, launch_gemm_tc(t, m->stream));
    return L3_OK;
  }
  if (K % 4 == 0 && ld % 4 == 0) LAUNCH(m, launch_linear_simt(a, m->bf16, m->bf16, m->stream));
  else LAUNCH(m, launch_linear_any(a, m->bf16, m->stream));
  return L3_OK;
}

static EpiArgs store_to(float* out, void* out16, int ld) {
  EpiArgs e{};
  e.out = out; e.out_bf16 = (bf16*)out16; e.ld_out = ld;
  return e;
}

// ------------------------------------------------------------------------------ pre-norm layers
// x <- x + mixer(shift(norm1(x)));  x <- x + ff(norm2(x)).  The residual stream stays in m->x (fp32); the normed rows
// live in m->xn (+ the bf16 mirror m->xn16 for the tensor-core projections); the sublayers' output projections add
// into x in their epilogue.
static EpiArgs resid_into(float* x, int ld) {
  EpiArgs e{};
  e.out = x; e.resid = x; e.ld_out = ld;
  return e;
}

// One unit mixer (window attention, state-space, gated linear attention, gated delta rule) of a pre-norm layer: from its
// columns of the fused input projection (pin, row stride ld) to its columns of the output projection's input (m->ctx, row
// stride Ly.ctx_ld, already times the mixer's scale).
static int ll_mix_unit(L3Model* m, LLLayer& Ly, LLState& St, const float* pin, int ld, int B, int L) {
  LayerList* ll = m->ll;
  const L3LayerSpec& s = Ly.spec;
  const int ntok = B * L, H = s.heads, G = s.kv_heads, DK = s.dim, DV = s.vdim, O = H * DV;
  const float eps = ll->cfg.norm_eps;
  int* d_pos = m->d_scal + 0;
  float* ctx = m->ctx + Ly.ctx_base;
  bf16* ctx16 = m->ctx16 ? (bf16*)m->ctx16 + Ly.ctx_base : nullptr;
  int rc;
  if (s.mixer == L3_MIX_WINDOW) {
    WinPrepArgs pa{};
    pa.proj = pin; pa.ld = ld; pa.q_off = Ly.off_q; pa.k_off = Ly.off_k; pa.v_off = Ly.off_v; pa.inv_freq = Ly.inv_freq;
    pa.rot_dims = s.rot_dims; pa.rot_layout = s.rot_layout; pa.unit_norm = s.qk_unit; pa.eps = eps;
    pa.q_out = m->q; pa.cache_k = St.ck; pa.cache_v = St.cv; pa.pos_ptr = d_pos;
    pa.L = L; pa.H = H; pa.G = G; pa.DK = DK; pa.DV = DV; pa.M = m->M;
    LAUNCH(m, launch_win_prep(pa, ntok, m->bf16, m->stream));
    WinAttnArgs at{};
    at.q = m->q; at.cache_k = St.ck; at.cache_v = St.cv; at.out = ctx; at.out16 = ctx16; at.ld_out = Ly.ctx_ld; at.out_scale = Ly.mix_scale;
    at.head_vec = Ly.head_vec; at.pos_ptr = d_pos; at.scale = s.scale; at.kind = s.attn_kind; at.window = s.window; at.keep_first = s.keep_first;
    at.B = B; at.L = L; at.H = H; at.G = G; at.DK = DK; at.DV = DV; at.M = m->M;
    at.nsplit = win_attn_splits(B, L, H, G, s.window, s.keep_first, m->M, 32);
    at.part_o = ll->win_part_o; at.part_ml = ll->win_part_ml;
    LAUNCH(m, launch_win_attn(at, m->bf16, m->stream));
    if (at.nsplit > 1) m->launch_acc += 1;
    return L3_OK;
  }
  MixOutArgs mo{};
  mo.o = ll->o; mo.n = O; mo.DV = DV; mo.eps = eps; mo.out_scale = Ly.mix_scale; mo.out = ctx; mo.out16 = ctx16; mo.ld_out = Ly.ctx_ld;
  RecurArgs ra{};
  ra.state = St.S; ra.out = ll->o; ra.B = B; ra.L = L; ra.H = H; ra.DK = DK; ra.DV = DV;
  if (s.mixer == L3_MIX_SSD) {
    const int gn = G * DK;
    SsdPrepArgs pa{};
    pa.proj = pin; pa.ld = ld; pa.xbc_off = Ly.off_q; pa.dt_off = Ly.off_b; pa.conv_w = Ly.conv_w; pa.conv_b = Ly.conv_b;
    pa.conv_tail = St.conv_tail; pa.A_log = Ly.A_log; pa.dt_bias = Ly.dt_bias;
    pa.x_out = ll->xs; pa.v_out = ll->rv; pa.k_out = ll->rk; pa.q_out = m->q; pa.decay_out = ll->rg;
    pa.logdecay_out = ll->rg + (size_t)ntok * H;
    pa.L = L; pa.H = H; pa.G = G; pa.N = DK; pa.DV = DV; pa.taps = s.conv_taps; pa.update_tail = L == 1;
    LAUNCH(m, launch_ssd_prep(pa, ntok, m->stream));
    if (s.conv_taps > 1 && L > 1) LAUNCH(m, launch_conv_tail(St.conv_tail, pin + Ly.off_q, ld, B, L, O + 2 * gn, s.conv_taps - 1, m->stream));
    ra.mode = 2; ra.q = m->q; ra.k = ll->rk; ra.v = ll->rv; ra.ld_q = ra.ld_k = gn; ra.ld_v = O; ra.g = ll->rg; ra.g_head = 1; ra.rep = H / G;
    ra.log_g = pa.logdecay_out; ra.ws = ll->chunk_ws; ra.ws_floats = ll->chunk_ws_floats;  // prompts: chunk-parallel where the shape allows
    LAUNCH(m, launch_recur(ra, m->stream));
    mo.skip_d = Ly.skip_d; mo.skip_x = ll->xs; mo.gate = pin + Ly.off_g; mo.ld_gate = ld; mo.gate_act = 1; mo.pre_gate = 1;
    mo.w = Ly.mix_norm; mo.wlen = O; mo.group = O / s.out_norm_groups;
  } else if (s.mixer == L3_MIX_GLA) {
    const int nd = H * DK;
    float* z = ll->aux;  // [ntok, H * DK] decay logits
    if ((rc = ll_linear(m, Ly.w_a2, pin + Ly.off_a1, nullptr, ld, ntok, nd, s.rank_decay, EPI_STORE, store_to(z, nullptr, nd))) != L3_OK) return rc;
    LAUNCH(m, launch_gla_prep(pin + Ly.off_q, ld, 1.0f / sqrtf((float)DK), z, nd, Ly.a2_bias, s.tau, ntok, nd, m->q, ll->rg, m->stream));
    ra.mode = 2; ra.q = m->q; ra.ld_q = nd; ra.k = pin + Ly.off_k; ra.ld_k = ld; ra.v = pin + Ly.off_v; ra.ld_v = ld; ra.g = ll->rg; ra.rep = 1;
    LAUNCH(m, launch_recur(ra, m->stream));
    mo.gate = pin + Ly.off_g; mo.ld_gate = ld; mo.gate_act = 1; mo.pre_gate = 0; mo.w = Ly.mix_norm; mo.wlen = DV; mo.group = DV;
  } else {
    const int nq = G * DK, nd = H * DK;
    float* dt = ll->aux;                          // [ntok, H * DK] decay logits
    float* og = ll->aux + (size_t)ntok * nd;      // [ntok, H * DV] output-gate logits
    if ((rc = ll_linear(m, Ly.w_a2, pin + Ly.off_a1, nullptr, ld, ntok, nd, s.rank_decay, EPI_STORE, store_to(dt, nullptr, nd))) != L3_OK) return rc;
    if ((rc = ll_linear(m, Ly.w_g2, pin + Ly.off_g1, nullptr, ld, ntok, O, s.rank_gate, EPI_STORE, store_to(og, nullptr, O))) != L3_OK) return rc;
    DeltaPrepArgs pa{};
    pa.proj = pin; pa.ld = ld; pa.beta_off = Ly.off_b; pa.dt_in = dt; pa.ld_dt = nd;
    pa.conv_w = Ly.conv_w; pa.conv_tail = St.conv_tail; pa.A_log = Ly.A_log; pa.dt_bias = Ly.dt_bias;
    pa.q_out = m->q; pa.k_out = ll->rk; pa.v_out = ll->rv; pa.decay_out = ll->rg; pa.beta_out = ll->rbeta;
    pa.L = L; pa.H = H; pa.G = G; pa.DK = DK; pa.DV = DV; pa.taps = s.conv_taps; pa.update_tail = L == 1;
    LAUNCH(m, launch_delta_prep(pa, ntok, m->stream));
    if (s.conv_taps > 1 && L > 1) LAUNCH(m, launch_conv_tail(St.conv_tail, pin, ld, B, L, 2 * nq + O, s.conv_taps - 1, m->stream));
    ra.mode = 1; ra.q = m->q; ra.k = ll->rk; ra.v = ll->rv; ra.ld_q = ra.ld_k = nq; ra.ld_v = O;
    ra.g = ll->rg; ra.beta = ll->rbeta; ra.rep = H / G;
    LAUNCH(m, launch_recur(ra, m->stream));
    mo.gate = og; mo.ld_gate = O; mo.gate_act = 0; mo.pre_gate = 0; mo.w = Ly.mix_norm; mo.wlen = DV; mo.group = DV;
  }
  LAUNCH(m, launch_mix_out(mo, ntok, m->stream));
  return L3_OK;
}

static int ll_enqueue_prenorm(L3Model* m, int B, int L, float* d_resid) {
  LayerList* ll = m->ll;
  const int ntok = B * L, W = m->D;
  const float eps = ll->cfg.norm_eps;
  int* d_pos = m->d_scal + 0;
  float* hn = m->xn;
  bf16* hn16 = (bf16*)m->xn16;  // null in fp32 mode
  int rc;
  ll->xcur = m->x;
  if (ll->cfg.embed_scale != 0.f && ll->cfg.embed_scale != 1.f) LAUNCH(m, launch_scale_add_rows(m->x, ll->cfg.embed_scale, nullptr, ntok, W, m->stream));
  const int ng = std::max(1, ll->cfg.norm_groups);
  if (ll->embed_norm) LAUNCH(m, launch_rmsnorm_rows(m->x, ll->embed_norm, eps, ntok, W, 1, 0, nullptr, m->x, nullptr, m->stream, ng));  // in place, row by row
  if (ll->x0) CK(m, cudaMemcpyAsync(ll->x0, m->x, (size_t)ntok * W * 4, cudaMemcpyDeviceToDevice, m->stream));  // the embedding output
  for (int ri = 0; ri < (int)ll->runs.size(); ++ri) {
    LLLayer& Ly = ll->layers[ll->runs[ri].layer];
    LLState& St = ll->state[ri];
    const L3LayerSpec& s = Ly.spec;
    const int H = s.heads, DK = s.dim, DV = s.vdim;
    if (ll->runs[ri].pass >= 0 && ll->loop_in) {  // a pass starts: x <- W_in [x ; x0]
      LAUNCH(m, launch_concat_rows(m->x, ll->x0, ntok, W, ll->cat, (bf16*)ll->cat16, m->stream));
      if ((rc = ll_linear(m, ll->loop_in, ll->cat, ll->cat16, 0, ntok, W, 2 * W, EPI_STORE, store_to(m->x, nullptr, W))) != L3_OK) return rc;
    } else if (ll->runs[ri].pass >= 0)
      LAUNCH(m, launch_scale_add_rows(m->x, 1.0f, ll->loop_step + (size_t)ll->runs[ri].pass * W, ntok, W, m->stream));
    LAUNCH(m, launch_prenorm_shift(m->x, Ly.norm1, eps, Ly.shift, St.hprev, B, L, W, hn, hn16, m->stream, ng));
    // every projection of the mixer's input in one GEMM
    if ((rc = ll_linear(m, Ly.w_in, hn, hn16, 0, ntok, Ly.n_in, W, EPI_STORE, store_to(ll->pin, nullptr, Ly.n_in))) != L3_OK) return rc;
    int n_ctx = H * DV;
    if (unit_mixer(s.mixer)) {
      n_ctx = Ly.ctx_ld;
      if ((rc = ll_mix_unit(m, Ly, St, ll->pin, Ly.in_ld, B, L)) != L3_OK) return rc;
      if (Ly.pair && (rc = ll_mix_unit(m, *Ly.pair, *St.pair, ll->pin + Ly.pair->in_base, Ly.in_ld, B, L)) != L3_OK) return rc;
    } else if (s.mixer == L3_MIX_LATENT) {
      const int Dk = s.kv_rank + s.rot_dim, nq = H * (DK + s.rot_dim);
      LatentPrepArgs pa{};
      pa.proj = ll->pin; pa.ld = Ly.n_in; pa.k_off = Ly.off_k; pa.wq = Ly.q_norm; pa.wk = Ly.k_norm; pa.eps = eps;
      pa.cq = ll->aux; pa.cq16 = (bf16*)ll->aux16; pa.cache = St.lat; pa.inv_freq = Ly.inv_freq; pa.pos_ptr = d_pos;
      pa.L = L; pa.M = m->M; pa.q_rank = s.q_rank; pa.kv_rank = s.kv_rank; pa.rot_dim = s.rot_dim; pa.rot_dims = s.rot_dims;
      LAUNCH(m, launch_latent_prep(pa, ntok, m->bf16, m->stream));
      if ((rc = ll_linear(m, Ly.w_uq, ll->aux, ll->aux16, 0, ntok, nq, s.q_rank, EPI_STORE, store_to(m->q, nullptr, nq))) != L3_OK) return rc;
      // queries onto the latent: qlat[r, h] = [Wuk_h^T q_c | rot(q_r)]
      HeadGemmArgs ga{};
      ga.A = m->q; ga.lda = nq; ga.a_hs = DK + s.rot_dim;
      ga.W = Ly.w_uk; ga.w_hs = (int64_t)DK * s.kv_rank; ga.w_ks = s.kv_rank; ga.w_js = 1;
      ga.C = ll->qlat; ga.C16 = nullptr; ga.ldc = H * Dk; ga.c_hs = Dk;
      ga.rows = ntok; ga.H = H; ga.J = s.kv_rank; ga.K = DK;
      LAUNCH(m, launch_head_gemm(ga, m->bf16, m->stream));
      if (s.rot_dim > 0)
        LAUNCH(m, launch_latent_q_rope(m->q, ll->qlat, Ly.inv_freq, d_pos, ntok, L, H, DK, s.rot_dim, s.rot_dims, s.kv_rank, m->stream));
      LatentAttnArgs at{};
      at.q = ll->qlat; at.cache = St.lat; at.out = ll->o; at.gate = ll->pin + Ly.off_g; at.ld_gate = Ly.n_in;
      at.pos_ptr = d_pos; at.scale = s.scale; at.B = B; at.L = L; at.H = H; at.Dk = Dk; at.Dv = s.kv_rank; at.M = m->M;
      at.part_o = m->part_o; at.part_ml = m->part_ml;
      at.nsplit = 1;
      if (L == 1) {  // decode: the keys of a sequence spread over CTAs
        const int ctas = B * ((H + 31) / 32);
        at.nsplit = std::max(1, std::min(std::min(m->max_split, m->M / 64), (2 * 148) / std::max(1, ctas)));
      }
      LAUNCH(m, launch_latent_attn(at, m->bf16, m->stream));
      if (at.nsplit > 1) m->launch_acc += 1;
      // values out of the latent: ctx[r, h] = Wuv_h o[r, h]
      HeadGemmArgs gv{};
      gv.A = ll->o; gv.lda = H * s.kv_rank; gv.a_hs = s.kv_rank;
      gv.W = Ly.w_uv; gv.w_hs = (int64_t)DV * s.kv_rank; gv.w_ks = 1; gv.w_js = s.kv_rank;
      gv.C = m->ctx; gv.C16 = (bf16*)m->ctx16; gv.ldc = H * DV; gv.c_hs = DV;
      gv.rows = ntok; gv.H = H; gv.J = DV; gv.K = s.kv_rank;
      LAUNCH(m, launch_head_gemm(gv, m->bf16, m->stream));
    } else if (s.mixer == L3_MIX_MINGRU) {
      n_ctx = DK;
      LAUNCH(m, launch_mingru_scan(ll->pin, Ly.n_in, Ly.off_b, Ly.off_v, Ly.off_g, Ly.in_bias, St.S, B, L, DK, m->ctx, (bf16*)m->ctx16, m->stream));
    } else {
      set_err(m, "mixer %d is not built for pre-norm layers", s.mixer);
      return L3_EINVAL;
    }
    if ((rc = ll_linear(m, Ly.w_o, m->ctx, m->ctx16, 0, ntok, W, n_ctx, EPI_RESID, resid_into(m->x, W))) != L3_OK) return rc;
    if (s.experts > 0) {
      const int E = s.experts, ff = s.ff;
      LAUNCH(m, launch_prenorm_shift(m->x, Ly.norm2, eps, nullptr, nullptr, B, L, W, hn, hn16, m->stream, ng));
      const bool few = ntok <= 8;  // few rows read only their chosen experts' weights; many share one GEMM over all experts
      MoeRouteArgs ra{};
      ra.h = hn; ra.router = Ly.router; ra.correction = Ly.correction; ra.D = W; ra.E = E; ra.I = s.identity; ra.top = s.top;
      ra.groups = s.groups; ra.keep = s.groups_keep; ra.scale = s.router_scale;
      ra.sel = ll->moe_sel; ra.w = ll->moe_w; ra.dense = few ? nullptr : ll->moe_dense; ra.idw = ll->moe_idw;
      LAUNCH(m, launch_moe_route(ra, ntok, m->stream));
      if (few) {
        LAUNCH(m, launch_moe_rows(hn, Ly.w13, Ly.w2, m->bf16, ll->moe_sel, ll->moe_w, ll->moe_idw, ntok, W, E, ff, s.top, m->h, m->x, m->stream));
        m->launch_acc += 1;
      } else {
        if ((rc = ll_linear(m, Ly.w13, hn, hn16, 0, ntok, E * ff, W, EPI_STORE, store_to(m->h, nullptr, E * ff))) != L3_OK) return rc;
        LAUNCH(m, launch_moe_act_mask(m->h, ll->moe_dense, ntok, E, ff, (bf16*)m->h16, m->stream));
        if ((rc = ll_linear(m, Ly.w2, m->h, m->h16, 0, ntok, W, E * ff, EPI_RESID, resid_into(m->x, W))) != L3_OK) return rc;
        if (s.identity > 0) LAUNCH(m, launch_moe_identity(m->x, hn, ll->moe_idw, ntok, W, m->stream));
      }
    } else if (s.ff > 0) {
      LAUNCH(m, launch_prenorm_shift(m->x, Ly.norm2, eps, nullptr, nullptr, B, L, W, hn, hn16, m->stream, ng));
      EpiArgs e = store_to(m->h, m->h16, s.ff);
      e.act = ll->cfg.glu_act;
      if ((rc = ll_linear(m, Ly.w13, hn, hn16, 0, ntok, 2 * s.ff, W, EPI_SWIGLU, e)) != L3_OK) return rc;
      if ((rc = ll_linear(m, Ly.w2, m->h, m->h16, 0, ntok, W, s.ff, EPI_RESID, resid_into(m->x, W))) != L3_OK) return rc;
    }
    if (d_resid) CK(m, cudaMemcpyAsync(d_resid + (size_t)ri * ntok * W, m->x, (size_t)ntok * W * 4, cudaMemcpyDeviceToDevice, m->stream));
  }
  return L3_OK;
}

// ------------------------------------------------------------------------------ parallel layers
// h = norm1(x);  X_new = x + ls1 * mixer(h + conv1(h)) + ls2 * ff(h + conv2(h));  x <- sum_j dwa[j] X_j (depth average).
// One norm per layer; both sublayers' output projections store into y1 / y2 and ONE kernel forms the layer's result,
// keeps it for the later layers' averages and writes the stream that goes on.
static int ll_enqueue_parallel(L3Model* m, int B, int L, float* d_resid) {
  LayerList* ll = m->ll;
  const int ntok = B * L, W = m->D, T = ll->cfg.canon_taps;
  const float eps = ll->cfg.norm_eps;
  int* d_pos = m->d_scal + 0;
  const int64_t xs = (int64_t)m->cap_tok * W;
  int rc;
  ll->xcur = m->x;
  if (ll->Xs) CK(m, cudaMemcpyAsync(ll->Xs, m->x, (size_t)ntok * W * 4, cudaMemcpyDeviceToDevice, m->stream));
  // few rows: norm, convolutions and tail are one launch, which also applies the PREVIOUS layer's combination first
  const bool few_fused = T > 0 && ntok <= 8 && norm_canon_rows_supported(L, T) && (!m->bf16 || linear_rows_supported(ntok, W));
  ParallelCombineArgs pre{};
  bool have_pre = false;
  for (int ri = 0; ri < (int)ll->runs.size(); ++ri) {
    LLLayer& Ly = ll->layers[ll->runs[ri].layer];
    LLState& St = ll->state[ri];
    const L3LayerSpec& s = Ly.spec;
    const int H = s.heads, G = s.kv_heads, DK = s.dim, DV = s.vdim;
    const bool has_ff = s.ff > 0;
    float *hm = m->xn, *hf = m->xn;
    bf16 *hm16 = (bf16*)m->xn16, *hf16 = (bf16*)m->xn16;  // null in fp32 mode
    // rows that go through the row-streaming GEMV need no bf16 mirror: norm, convolutions and tail in one launch
    if (few_fused) {
      hf = ll->hf; hf16 = (bf16*)ll->hf16;
      LAUNCH(m, launch_norm_canon_rows(m->x, Ly.norm1, eps, ll->cfg.norm_center, St.conv_tail, Ly.canon1t, has_ff ? Ly.canon2t : nullptr, B, L, W, T,
                                       hm, has_ff ? hf : nullptr, have_pre ? &pre : nullptr, m->stream));
      have_pre = false;
    } else if (T > 0) {
      hf = ll->hf; hf16 = (bf16*)ll->hf16;
      LAUNCH(m, launch_layernorm_rows(m->x, Ly.norm1, eps, ll->cfg.norm_center, ntok, W, 1, 0, nullptr, ll->hn, nullptr, m->stream));
      LAUNCH(m, launch_canon(ll->hn, St.conv_tail, Ly.canon1t, has_ff ? Ly.canon2t : nullptr, B, L, W, T, hm, hm16, has_ff ? hf : nullptr, hf16, m->stream));
      if (T > 1) LAUNCH(m, launch_conv_tail(St.conv_tail, ll->hn, W, B, L, W, T - 1, m->stream));
    } else {
      LAUNCH(m, launch_layernorm_rows(m->x, Ly.norm1, eps, ll->cfg.norm_center, ntok, W, 1, 0, nullptr, hm, hm16, m->stream));
    }
    if (s.mixer != L3_MIX_DIFF) { set_err(m, "mixer %d is not built for parallel layers", s.mixer); return L3_EINVAL; }
    if ((rc = ll_linear(m, Ly.w_in, hm, hm16, 0, ntok, Ly.n_in, W, EPI_STORE, store_to(ll->pin, nullptr, Ly.n_in))) != L3_OK) return rc;
    DiffPrepArgs pa{};
    pa.proj = ll->pin; pa.ld = Ly.n_in; pa.q_off = Ly.off_q; pa.k_off = Ly.off_k; pa.v_off = Ly.off_v; pa.bias = Ly.in_bias;
    pa.wq = Ly.q_norm; pa.wk = Ly.k_norm; pa.eps = eps; pa.inv_freq = Ly.inv_freq; pa.q_out = m->q; pa.cache_k = St.ck; pa.cache_v = St.cv;
    pa.pos_ptr = d_pos; pa.L = L; pa.H = H; pa.G = G; pa.DK = DK; pa.DV = DV; pa.M = m->M; pa.rot_dims = s.rot_dims;
    LAUNCH(m, launch_diff_prep(pa, ntok, m->bf16, m->stream));
    DiffAttnArgs at{};
    at.q = m->q; at.cache_k = St.ck; at.cache_v = St.cv; at.out = m->ctx; at.out16 = (bf16*)m->ctx16; at.lambda = Ly.lambda;
    at.pos_ptr = d_pos; at.scale = s.scale; at.diff = s.diff; at.eps = eps; at.window = s.window;
    at.B = B; at.L = L; at.H = H; at.G = G; at.DK = DK; at.DV = DV; at.M = m->M;
    LAUNCH(m, launch_diff_attn(at, m->bf16, ll->diff_part_o, ll->diff_part_ml, m->stream));
    if ((rc = ll_linear(m, Ly.w_o, m->ctx, m->ctx16, 0, ntok, W, H * DV, EPI_STORE, store_to(ll->y1, nullptr, W))) != L3_OK) return rc;
    if (Ly.ff_total) {
      const int E = s.experts, ff = s.ff, F = Ly.ff_total;
      const bool few = ntok <= 8;  // few rows read only their chosen experts' weights; many share one GEMM over all experts
      MoeRouteArgs ra{};
      ra.h = hf; ra.router = Ly.router; ra.correction = nullptr; ra.D = W; ra.E = E; ra.I = 0; ra.top = s.top;
      ra.groups = 1; ra.keep = 1; ra.kind = 1; ra.scale = 1.0f;
      ra.sel = ll->moe_sel; ra.w = ll->moe_w; ra.dense = few ? nullptr : ll->moe_dense; ra.idw = ll->moe_idw;
      LAUNCH(m, launch_moe_route(ra, ntok, m->stream));
      if (few) {
        LAUNCH(m, launch_moe_glu_rows(hf, Ly.w13, Ly.w2, m->bf16, ll->moe_sel, ll->moe_w, ntok, W, E, ff, s.shared_ff, s.top, m->h, ll->y2, m->stream));
        m->launch_acc += 1;
      } else {
        // gate | up of every expert and of the shared one in ONE projection, then the routing weight (zero for experts the
        // row did not choose) and silu(g) * u in a streaming kernel.  L3_MOE_EPI=1 moves that step into the GEMM's epilogue:
        // measured slower (width 2048, 2048 tokens: 13.65 against 12.95 ms per prompt) - the epilogue then does a weight
        // lookup and an exponential per output pair while the tensor pipe waits.
        static const bool fused = getenv("L3_MOE_EPI") && atoi(getenv("L3_MOE_EPI")) == 1;
        if (fused) {
          EpiArgs e = store_to(m->h, m->h16, F);
          e.act = GLU_SILU; e.glu_w = ll->moe_dense; e.glu_w_ld = E; e.glu_group = ff; e.glu_groups = E;
          if ((rc = ll_linear(m, Ly.w13, hf, hf16, 0, ntok, 2 * F, W, EPI_SWIGLU, e)) != L3_OK) return rc;
        } else {
          if ((rc = ll_linear(m, Ly.w13, hf, hf16, 0, ntok, 2 * F, W, EPI_STORE, store_to(ll->moe_gu, nullptr, 2 * F))) != L3_OK) return rc;
          LAUNCH(m, launch_moe_glu_act(ll->moe_gu, ll->moe_dense, ntok, E, ff, s.shared_ff, m->h, (bf16*)m->h16, m->stream));
        }
        if ((rc = ll_linear(m, Ly.w2, m->h, m->h16, 0, ntok, W, F, EPI_STORE, store_to(ll->y2, nullptr, W))) != L3_OK) return rc;
      }
    } else if (Ly.poly) {
      if ((rc = ll_linear(m, Ly.w13, hf, hf16, 0, ntok, s.ff, W, EPI_STORE, store_to(m->h, nullptr, s.ff))) != L3_OK) return rc;
      LAUNCH(m, launch_polynorm(m->h, Ly.poly, eps, ntok, s.ff, (bf16*)m->h16, m->stream));
      if ((rc = ll_linear(m, Ly.w2, m->h, m->h16, 0, ntok, W, s.ff, EPI_STORE, store_to(ll->y2, nullptr, W))) != L3_OK) return rc;
    } else if (has_ff) {
      EpiArgs e = store_to(m->h, m->h16, s.ff);
      e.act = ll->cfg.glu_act;
      if ((rc = ll_linear(m, Ly.w13, hf, hf16, 0, ntok, 2 * s.ff, W, EPI_SWIGLU, e)) != L3_OK) return rc;
      if ((rc = ll_linear(m, Ly.w2, m->h, m->h16, 0, ntok, W, s.ff, EPI_STORE, store_to(ll->y2, nullptr, W))) != L3_OK) return rc;
    }
    if (few_fused && !d_resid && ri + 1 < (int)ll->runs.size()) {  // left to the next layer's first launch
      pre.y1 = ll->y1; pre.y2 = has_ff ? ll->y2 : nullptr; pre.ls1 = Ly.ls1; pre.ls2 = Ly.ls2; pre.dwa = Ly.dwa;
      pre.Xs = ll->Xs; pre.x_stride = xs; pre.n_prev = ri + 1;
      have_pre = true;
      continue;
    }
    LAUNCH(m, launch_parallel_combine(m->x, ll->y1, has_ff ? ll->y2 : nullptr, Ly.ls1, Ly.ls2, ll->Xs, xs, Ly.dwa, ri + 1, ntok, W, m->stream));
    if (d_resid) CK(m, cudaMemcpyAsync(d_resid + (size_t)ri * ntok * W, m->x, (size_t)ntok * W * 4, cudaMemcpyDeviceToDevice, m->stream));
  }
  return L3_OK;
}

// ------------------------------------------------------------------------------ the layers of one chunk
int ll_enqueue_layers(L3Model* m, const int32_t* d_ids, int ids_ld, int ids_off, int B, int L, float* d_resid) {
  LayerList* ll = m->ll;
  const int ntok = B * L, W = m->D, sd = ll->cfg.side_dim;
  const float eps = ll->cfg.norm_eps;
  int* d_pos = m->d_scal + 0;
  bf16* x16 = (bf16*)m->xn16;  // null in fp32 mode; written by resid_postnorm_kernel, read by the tensor-core projections
  float* y = m->xn;
  int rc;
  // the residual stream lives in xcur; a fused post-norm step (LLPending) moves it to the other buffer
  ll->xcur = m->x;
  ll->xalt = ll->x2;
  LLPending pd;
  if (ll->cfg.parallel) return ll_enqueue_parallel(m, B, L, d_resid);
  // rows <= 8 never reach a tensor-core projection of the residual stream: no mirror needed
  if (x16 && !linear_rows_supported(ntok, W)) LAUNCH(m, launch_to_bf16(m->x, (int64_t)ntok * W, x16, m->stream));
  if (ll->cfg.norm_input) return ll_enqueue_prenorm(m, B, L, d_resid);
  for (int ri = 0; ri < (int)ll->runs.size(); ++ri) {
    const int li = ll->runs[ri].layer;
    LLLayer& Ly = ll->layers[li];
    LLState& St = ll->state[ri];
    const L3LayerSpec& s = Ly.spec;
    const int H = s.heads, G = s.kv_heads, DK = s.dim, DV = s.vdim, O = H * DV;
    if (ll->runs[ri].pass >= 0) {  // a pass of the looped block starts: its step vector joins the stream
      if ((rc = ll_settle(m, pd, ntok)) != L3_OK) return rc;
      LAUNCH(m, launch_scale_add_rows(ll->xcur, 1.0f, ll->loop_step + (size_t)ll->runs[ri].pass * W, ntok, W, m->stream));
      if (x16 && !linear_rows_supported(ntok, W)) LAUNCH(m, launch_to_bf16(ll->xcur, (int64_t)ntok * W, x16, m->stream));
    }
    // every projection of the mixer's input in one GEMM
    if ((rc = ll_linear(m, Ly.w_in, ll->xcur, x16, 0, ntok, Ly.n_in, W, EPI_STORE, store_to(ll->pin, nullptr, Ly.n_in), &pd)) != L3_OK) return rc;
    if (s.mixer == L3_MIX_SOFTMAX) {
      QkNormArgs qa{};
      qa.proj = ll->pin; qa.ld = Ly.n_in; qa.k_off = Ly.off_k; qa.wq = Ly.q_norm; qa.wk = Ly.k_norm; qa.eps = eps;
      qa.q_out = m->q; qa.cache_k = St.ck; qa.cache_v = St.cv; qa.pos_ptr = d_pos;
      qa.L = L; qa.HN = H; qa.KVHN = G; qa.HD = DK; qa.M = m->M;
      LAUNCH(m, launch_qk_norm_cache(qa, ntok, m->bf16, m->stream));
      AttnArgs at{};
      at.q = m->q; at.cache_k = St.ck; at.cache_v = St.cv; at.pos_ptr = d_pos;
      at.B = B; at.L = L; at.HN = H; at.KVHN = G; at.HD = DK; at.M = m->M;
      at.part_o = m->part_o; at.part_ml = m->part_ml; at.counters = m->attn_cnt;
      at.out = m->ctx; at.out_bf16 = (bf16*)m->ctx16;
      at.scale = s.scale; at.head_gate = ll->pin + Ly.off_g; at.ld_gate = Ly.n_in;
      at.force_exact = 1;  // scores and softmax weights stay fp32
      at.nsplit = 1;
      if (!attn_head_dim_supported(DK)) LAUNCH(m, launch_attn_any(at, m->bf16, m->stream));
      else if (L == 1) {
        at.nsplit = std::max(1, std::min(std::min(m->max_split, m->M / 16), (4 * 148) / std::max(1, B * G)));
        LAUNCH(m, launch_attn_decode(at, m->bf16, m->stream));
      } else LAUNCH(m, launch_attn_prefill(at, m->bf16, m->stream));
    } else if (s.mixer == L3_MIX_DECAY_LINEAR) {
      RecurArgs ra{};
      ra.mode = 0; ra.q = ll->pin + Ly.off_q; ra.k = ll->pin + Ly.off_k; ra.v = ll->pin + Ly.off_v;
      ra.ld_q = ra.ld_k = ra.ld_v = Ly.n_in; ra.act_in = m->bf16 ? 2 : 1; ra.head_decay = Ly.decay;
      ra.state = St.S; ra.out = ll->o; ra.B = B; ra.L = L; ra.H = H; ra.rep = 1; ra.DK = DK; ra.DV = DV;
      ra.ws = ll->chunk_ws; ra.ws_floats = ll->chunk_ws_floats;
      LAUNCH(m, launch_recur(ra, m->stream));
      LAUNCH(m, launch_gated_rmsnorm(ll->o, ll->pin + Ly.off_g, Ly.n_in, Ly.mix_norm, O, O, eps, ntok, O, m->ctx, (bf16*)m->ctx16, m->stream));
    } else {
      const int nq = G * DK, nd = H * DK;
      float* dt = ll->aux;                          // [ntok, H * DK] decay logits
      float* og = ll->aux + (size_t)ntok * nd;      // [ntok, H * DV] output-gate logits
      if ((rc = ll_linear(m, Ly.w_a2, ll->pin + Ly.off_a1, nullptr, Ly.n_in, ntok, nd, s.rank_decay, EPI_STORE, store_to(dt, nullptr, nd))) != L3_OK) return rc;
      if ((rc = ll_linear(m, Ly.w_g2, ll->pin + Ly.off_g1, nullptr, Ly.n_in, ntok, O, s.rank_gate, EPI_STORE, store_to(og, nullptr, O))) != L3_OK) return rc;
      DeltaPrepArgs pa{};
      pa.proj = ll->pin; pa.ld = Ly.n_in; pa.beta_off = Ly.off_b; pa.dt_in = dt; pa.ld_dt = nd;
      pa.conv_w = Ly.conv_w; pa.conv_tail = St.conv_tail; pa.A_log = Ly.A_log; pa.dt_bias = Ly.dt_bias;
      pa.q_out = m->q; pa.k_out = ll->rk; pa.v_out = ll->rv; pa.decay_out = ll->rg; pa.beta_out = ll->rbeta;
      pa.L = L; pa.H = H; pa.G = G; pa.DK = DK; pa.DV = DV; pa.taps = s.conv_taps;
      LAUNCH(m, launch_delta_prep(pa, ntok, m->stream));
      if (s.conv_taps > 1) LAUNCH(m, launch_conv_tail(St.conv_tail, ll->pin, Ly.n_in, B, L, 2 * nq + O, s.conv_taps - 1, m->stream));
      RecurArgs ra{};
      ra.mode = 1; ra.q = m->q; ra.k = ll->rk; ra.v = ll->rv; ra.ld_q = ra.ld_k = nq; ra.ld_v = O;
      ra.g = ll->rg; ra.beta = ll->rbeta; ra.state = St.S; ra.out = ll->o;
      ra.B = B; ra.L = L; ra.H = H; ra.rep = H / G; ra.DK = DK; ra.DV = DV;
      LAUNCH(m, launch_recur(ra, m->stream));
      LAUNCH(m, launch_gated_rmsnorm(ll->o, og, O, Ly.mix_norm, DV, DV, eps, ntok, O, m->ctx, (bf16*)m->ctx16, m->stream));
    }
    if ((rc = ll_linear(m, Ly.w_o, m->ctx, m->ctx16, 0, ntok, W, O, EPI_STORE, store_to(y, nullptr, W))) != L3_OK) return rc;
    pd.y = y; pd.w = Ly.norm1;  // x += mult * N1(y): applied by whoever reads x next
    if (s.ff > 0) {
      EpiArgs e = store_to(m->h, m->h16, s.ff);
      e.act = ll->cfg.glu_act;
      if ((rc = ll_linear(m, Ly.w13, ll->xcur, x16, 0, ntok, 2 * s.ff, W, EPI_SWIGLU, e, &pd)) != L3_OK) return rc;
      if ((rc = ll_linear(m, Ly.w2, m->h, m->h16, 0, ntok, W, s.ff, EPI_STORE, store_to(y, nullptr, W))) != L3_OK) return rc;
      pd.y = y; pd.w = Ly.norm2;
    }
    if (sd) {
      if ((rc = ll_linear(m, Ly.side_gate, ll->xcur, x16, 0, ntok, sd, W, EPI_STORE, store_to(ll->sg, nullptr, sd), &pd)) != L3_OK) return rc;
      LAUNCH(m, launch_side_mul(ll->sg, sd, ntok, ll->side_embed, m->bf16, (int)ll->layers.size() * sd, li * sd, d_ids, ids_ld, ids_off, L,
                                m->cfg.vocab_size, ll->cfg.glu_act, (bf16*)ll->sg16, m->stream));
      if ((rc = ll_linear(m, Ly.side_proj, ll->sg, ll->sg16, 0, ntok, W, sd, EPI_STORE, store_to(y, nullptr, W))) != L3_OK) return rc;
      pd.y = y; pd.w = Ly.side_norm;
    }
    if (d_resid) {
      if ((rc = ll_settle(m, pd, ntok)) != L3_OK) return rc;
      CK(m, cudaMemcpyAsync(d_resid + (size_t)ri * ntok * W, ll->xcur, (size_t)ntok * W * 4, cudaMemcpyDeviceToDevice, m->stream));
    }
  }
  return ll_settle(m, pd, ntok);  // the LM head reads ll->xcur
}

int ll_ensure_head_rows(L3Model* m, int n) {
  LayerList* ll = m->ll;
  if (n <= ll->head_rows) return L3_OK;
  CK(m, cudaStreamSynchronize(m->stream));
  cudaFree(m->xlast); cudaFree(m->logits);
  m->xlast = m->logits = nullptr;
  CK(m, cudaMalloc((void**)&m->xlast, (size_t)n * m->D * 4));
  CK(m, cudaMalloc((void**)&m->logits, (size_t)n * m->VS * 4));
  if (m->xlast16) {
    cudaFree(m->xlast16);
    m->xlast16 = nullptr;
    CK(m, cudaMalloc(&m->xlast16, (size_t)n * m->D * 2));
  }
  ll->head_rows = n;
  return L3_OK;
}

int ll_enqueue_head(L3Model* m, int B, int L, const int32_t* d_rows, int n_rows) {
  const int rows = d_rows ? n_rows : B;
  if (m->ll->cfg.norm_center)
    LAUNCH(m, launch_layernorm_rows(m->ll->xcur, m->norm_final, m->ll->cfg.norm_eps, 1, rows, m->D, L, L - 1, d_rows, m->xlast, (bf16*)m->xlast16, m->stream));
  else
    LAUNCH(m, launch_rmsnorm_rows(m->ll->xcur, m->norm_final, m->ll->cfg.norm_eps, rows, m->D, L, L - 1, d_rows, m->xlast, (bf16*)m->xlast16, m->stream,
                                  std::max(1, m->ll->cfg.norm_groups)));
  const int rc = ll_linear(m, m->lm_head, m->xlast, m->xlast16, 0, rows, m->VS, m->D, EPI_STORE, store_to(m->logits, nullptr, m->VS));
  if (rc != L3_OK) return rc;
  if (m->ll->cfg.logit_softcap > 0.f) LAUNCH(m, launch_softcap(m->logits, (int64_t)rows * m->VS, m->ll->cfg.logit_softcap, m->stream));
  return L3_OK;
}
