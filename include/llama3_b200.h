/* llama3_b200.h - C-ABI of the B200-native (sm_100a) Llama-3 forward / greedy-generate path.
 *
 * The reference (swap357/llama3.np) is pure Python + NumPy and has no FFI of its own; the
 * boundary it exposes is its Python surface.  Every entry point below names the reference
 * behaviour it replaces (file:line relative to the reference checkout).  The Python host
 * (`llama3.np_b200/llama3.py`) binds these with ctypes and mirrors `Llama` / `ModelArgs`.
 *
 * Conventions: plain pointers and sizes only; every function returns 0 on success and a
 * negative L3_E* code on failure, with a message retrievable through l3_last_error().
 * One handle = one CUDA device + one stream; a handle is not re-entrant.  All host
 * buffers may be pageable; "dev" variants take device pointers and never touch the host.
 */
#ifndef LLAMA3_B200_H
#define LLAMA3_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define L3_OK 0
#define L3_EINVAL (-1)   /* bad argument (maps to ValueError)              */
#define L3_ECUDA (-2)    /* CUDA runtime / launch failure (RuntimeError)    */
#define L3_ESTATE (-3)   /* call out of order (e.g. forward before finalize) */
#define L3_ENOMEM (-4)
#define L3_ENCCL (-5)

#define L3_DTYPE_F32 0   /* fp32 weights, activations, KV cache: token-identical mode */
#define L3_DTYPE_BF16 1  /* bf16 weights / KV cache / GEMM operands, fp32 accumulation  */

/* ModelArgs (reference config.py:5-19) + the FFN width the reference infers from the
 * up_proj weight shape (llama3.py:86-95).  rope base is fixed at 10000 (llama3.py:31). */
typedef struct L3Config {
  int32_t dim;
  int32_t n_layers;
  int32_t n_heads;
  int32_t n_kv_heads;     /* already resolved: n_heads when ModelArgs.n_kv_heads is None */
  int32_t vocab_size;
  int32_t max_seq_len;
  int32_t max_batch_size;
  int32_t hidden_dim;
  float norm_eps;
  int32_t dtype;          /* L3_DTYPE_* */
  int32_t device;         /* CUDA ordinal */
  int32_t tp_rank;        /* tensor-parallel rank / world (1 = single GPU) */
  int32_t tp_world;
  int32_t flags;          /* L3_FLAG_* */
} L3Config;

#define L3_FLAG_NO_GRAPH 1      /* never capture CUDA graphs (debug)                      */
#define L3_FLAG_NO_TENSORCORE 2 /* keep SIMT GEMMs (A/B against the tcgen05 kernels)         */
#define L3_FLAG_NO_PDL 4        /* process-wide: no programmatic dependent launch           */
#define L3_FLAG_NO_MEGA 8       /* batch-1 decode as one kernel per projection (A/B against
                                   the persistent single-kernel step)                       */

typedef struct L3Model L3Model;

/* Library-level (no handle): version string, and the last error of a failed l3_create. */
const char* l3_version(void);
const char* l3_last_error(const L3Model* m); /* m may be NULL */
int l3_device_count(int* out);

/* -- lifetime: replaces Llama.__init__ (llama3.py:265-283) -------------------------- */
int l3_create(const L3Config* cfg, L3Model** out);
/* Upload one tensor of the reference's .npz key layout (llama3.py:219-235, 269, 280-281):
 * float32, C-contiguous, stored [out, in].  Keys are the reference's HF-style names. */
int l3_load_weight(L3Model* m, const char* key, const float* host, const int64_t* shape, int ndim);
/* Random-init on the device for shapes that are impractical to build on the host
 * (8B-shaped benches).  Same scales as synth.make_weights, different stream of numbers. */
int l3_fill_random(L3Model* m, uint64_t seed);
/* Packed device-layout weight cache (replaces a repeat of np.load + per-tensor packing,
 * llama3.py:269 / utils.py:4-5, on the second and later starts).  l3_save_packed writes the weight matrices
 * exactly as they sit on the device after the l3_load_weight calls (fused q|k|v rows, interleaved gate/up rows,
 * this rank's tensor-parallel slices, model dtype) to `path` (atomically: temp file + rename) together with
 * `source_digest`, the caller's hex digest of the checkpoint they came from.  l3_load_packed, called INSTEAD of
 * the l3_load_weight calls and before l3_finalize, streams such a file into the device buffers; it fails with
 * L3_EINVAL - leaving the model unloaded - if shape, dtype, tensor-parallel placement, digest or any tensor
 * checksum differ.  l3_packed_info reads a file's header without a model (hidden_dim is needed for l3_create). */
int l3_save_packed(L3Model* m, const char* path, const char* source_digest);
int l3_load_packed(L3Model* m, const char* path, const char* source_digest /* NULL: accept any */);
int l3_packed_info(const char* path, L3Config* cfg_out, char* digest_out, int digest_cap);
/* RoPE tables as computed by compute_cos_sin_cache in float64 on the host
 * (llama3.py:31-38), [max_seq_len, head_dim/2] each. */
int l3_set_rope_tables(L3Model* m, const double* cos_tab, const double* sin_tab);
/* Pack (fused QKV rows, interleaved gate/up rows, optional bf16 copies), allocate and
 * zero the KV caches (llama3.py:138-153) and the activation workspace. */
int l3_finalize(L3Model* m);
int l3_destroy(L3Model* m);
/* Zero the KV caches (the reference never does; a new Llama instance starts at zero). */
int l3_reset_cache(L3Model* m);
/* Tensor parallel: hand the handle an initialised NCCL communicator (ncclComm_t) made by
 * the caller, or let it create one from a 128-byte ncclUniqueId. */
int l3_tp_init(L3Model* m, const void* nccl_unique_id_128);
int l3_nccl_unique_id(void* out_128);

/* -- the forward step: replaces Llama.__call__ (llama3.py:285-308) ------------------- */
/* ids [B, L] int32 row-major (host).  logits_out: [B, vocab] float32 or NULL.
 * argmax_out: [B] int64 (first maximum wins, llama3.py:320) or NULL. */
int l3_forward(L3Model* m, const int32_t* ids, int B, int L, int start_pos,
               float* logits_out, int64_t* argmax_out);
/* Same, all pointers on the device; enqueues on the handle's stream and returns. */
int l3_forward_dev(L3Model* m, const int32_t* d_ids, int B, int L, int start_pos,
                   float* d_logits_out, int64_t* d_argmax_out);

/* -- the greedy loop: replaces Llama.generate (llama3.py:310-321) -------------------- */
/* Runs prefill at pos 0 and then decode steps with pos = L + i (the reference's schedule,
 * including its skipped slot L).  out: [B, max_new_tokens - L] int64 row-major.
 * Returns L3_EINVAL when max_new_tokens > max_seq_len or L >= max_new_tokens yields nothing
 * (n_out = 0 is allowed and writes nothing). */
int l3_generate_greedy(L3Model* m, const int32_t* ids, int B, int L, int max_new_tokens,
                       int64_t* out);
int l3_generate_greedy_dev(L3Model* m, const int32_t* d_ids, int B, int L, int max_new_tokens,
                           int64_t* d_out);
/* Incremental form used by the lazy Python generator: start enqueues the prefill,
 * each next() runs one step and copies that step's [B] token ids to the host. */
int l3_generate_begin(L3Model* m, const int32_t* ids, int B, int L);
/* pos_offset 0: decode step i at pos = L + i (Llama.generate, llama3.py:316-318);
 * pos_offset -1: pos = L + i - 1 (llama_generate of llama3_simple.py:272-280). */
int l3_generate_begin_ex(L3Model* m, const int32_t* ids, int B, int L, int pos_offset);
int l3_generate_next(L3Model* m, int64_t* out_B);
/* Extension (the reference generates equal-length prompts only and checks EOS for row 0 in the caller,
 * llama3.py:341-343): prompts of different lengths in one batch.  ids [B, Lmax] int32, right-padded
 * (padding values ignored); lens [B]; out [B, max_new_tokens] int64.  Sequence b yields exactly what it
 * would yield alone: Llama.generate(ids_b, lens[b] + max_new_tokens) for pos_offset 0, llama_generate for
 * pos_offset -1.  eos_id >= 0: a sequence that emitted eos_id keeps emitting it. */
int l3_generate_ragged(L3Model* m, const int32_t* ids, const int32_t* lens, int B, int Lmax, int max_new_tokens,
                       int pos_offset, int eos_id, int64_t* out);


/* -- layer-list decoders (hybrid stacks) ---------------------------------------------------------------
 * A second way to make a model, for decoders that are a LIST of layers, each with its own token mixer
 * (no counterpart in the reference, which has the one Llama block, llama3.py:238-262).  A handle made by
 * l3_create_stack goes through the same calls as a Llama handle: l3_load_tensor (instead of l3_load_weight),
 * l3_fill_random, l3_finalize, l3_forward / l3_forward_dev / l3_forward_rows, the l3_generate_* loop
 * (always at contiguous positions L + i - 1), l3_reset_cache, l3_destroy and the measurement helpers.
 * Every sequence slot b < max_batch_size owns a KV-cache region per attention layer and a recurrent state
 * (fp32 matrix per head, plus the short convolution's tail) per recurrent layer.  A call at start_pos 0
 * starts slot b afresh (its recurrent state is zeroed); a call at start_pos > 0 must continue exactly where
 * the slot's previous call ended (L3_ESTATE otherwise: a recurrent state cannot be rewound). */
#define L3_MIX_SOFTMAX 0       /* causal softmax attention, GQA, no positions, values = un-normalised keys,
                                  RMS norm over the whole q / k projection, sigmoid gate per head            */
#define L3_MIX_DECAY_LINEAR 1  /* linear attention, one fixed decay per head: S <- decay S + k v^T, o = S^T q */
#define L3_MIX_GATED_DELTA 2   /* gated delta rule, one data-dependent decay per head and key channel,
                                  short causal convolutions on q, k, v                                       */
#define L3_MIX_LATENT 3        /* causal softmax attention over ONE cached latent row per token: queries through a
                                  normed latent of width q_rank; the cache row is [normed latent (kv_rank) | rotated key
                                  part (rot_dim)] shared by all heads; per-head keys / values are expanded from the latent
                                  (here: folded into the query and the output); rotary pairs (2i, 2i + 1) on the first
                                  rot_dims entries of the rotated part; sigmoid gate per head                          */
#define L3_MIX_MINGRU 4        /* element-wise gated recurrence of width dim (heads = vdim = 1):
                                  S <- (1 - z) S + z c,  z = sigmoid(Wz h + bz),  c = u + 1/2 (u >= 0) | sigmoid(u),
                                  u = Wx h + bx;  output Wo (S * silu(Wg h))                                            */
#define L3_MIX_DIFF 5          /* differential sliding-window attention: every query / key head holds two maps of size dim
                                  ([map 1 | map 2]) that attend over the same values (GQA, value size vdim) and are combined
                                  as a1 - lambda a2, lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, followed by an RMS
                                  norm without weight over the head's values times (1 - diff); q / k / v have biases;
                                  q and k get an RMS norm per head and map (one weight vector of size dim each) and then
                                  rotary positions on the first rot_dims entries of each map, entry i paired with entry
                                  i + rot_dims / 2, frequencies rot_base^(-2 i / rot_dims) rescaled by wavelength
                                  (rot_scale_*); query i sees keys j with 0 <= i - j < window (window 0: every earlier key).
                                  Built for parallel layers (L3StackConfig::parallel)                                     */
#define L3_MIX_WINDOW 6        /* sliding-window attention, GQA, key size dim and value size vdim: query i sees key j <= i with
                                  i - j < window (window 0: every earlier key) or j < keep_first (the first tokens stay visible at
                                  their true positions); rotary positions on the first rot_dims entries of every head, pairs
                                  (2i, 2i + 1) (rot_layout 0) or (i, i + rot_dims / 2) (rot_layout 1), frequencies
                                  rot_base^(-2 i / rot_dims); qk_unit 1: q and k are divided by their root mean square per head
                                  after the rotation (no weight); score = q . k * scale; attn_kind L3_ATTN_SINK: softmax whose
                                  denominator also holds exp(sink_h) (tensor mix.sink [heads]), L3_ATTN_SIGMOID: the weight of a
                                  visible key is sigmoid(score + pb_h) (tensor mix.pb [heads]), not normalised over keys       */
#define L3_MIX_SSD 7           /* Mamba-2 state-space mixer: one projection laid out [z | x | B | C | dt] (heads * vdim twice,
                                  kv_heads * dim twice, heads); x | B | C pass a causal convolution of conv_taps taps with bias
                                  and silu; dt <- softplus(dt + dt_bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T
                                  (S is dim x vdim, dim = the state size, kv_heads = the B / C groups), y = S^T C + D x; then
                                  y * silu(z), an RMS norm in out_norm_groups equal parts with weight mix.norm, mix.o           */
#define L3_MIX_GLA 8           /* gated linear attention: q dim^(-1/2), k (heads x dim), v (heads x vdim); a decay per key channel
                                  alpha = sigmoid(a2 (a1 h) + a2.b)^(1 / tau); S <- diag(alpha) S + k v^T, o = S^T q; RMS norm per
                                  head with weight mix.norm [vdim], times silu(g h), mix.o                                    */
/* weights of L3_MIX_WINDOW (L3LayerSpec::attn_kind) */
#define L3_ATTN_SINK 0
#define L3_ATTN_SIGMOID 1
/* feed-forward kinds (L3LayerSpec::ff_kind) */
#define L3_FF_GLU 0            /* down(act(gate x) * (up x)), act = L3StackConfig::glu_act; experts: down relu(up x)^2 */
#define L3_FF_POLYNORM 1       /* down(P(up x)),  P(z) = a N(z) + b N(z^2) + c N(z^3) + e with element-wise powers and
                                  N(v) = v / sqrt(mean(v^2) + eps) over the ff values of a token; tensor l<i>.mlp.act = (a, b, c, e) */
/* router kinds (L3LayerSpec::router_kind) */
#define L3_ROUTE_SOFTMAX 0     /* softmax scores, correction, groups, identity slots; the weight multiplies the expert's output */
#define L3_ROUTE_SIGMOID_IN 1  /* scores = sigmoid(logits); the `top` largest are chosen (ties: lower slot), their weights are
                                  the scores themselves; the weight multiplies the expert's INPUT; experts are gated units
                                  down(silu(gate x) * (up x)); a shared expert of width shared_ff (0: none) runs for every token */
typedef struct L3LayerSpec {
  int32_t mixer;        /* L3_MIX_* */
  int32_t heads;        /* value heads (query heads for L3_MIX_SOFTMAX) */
  int32_t kv_heads;     /* key heads (L3_MIX_DECAY_LINEAR: = heads) */
  int32_t dim;          /* per-head query / key size */
  int32_t vdim;         /* per-head value size */
  int32_t conv_taps;    /* L3_MIX_GATED_DELTA: taps of the short convolutions */
  int32_t rank_decay;   /* L3_MIX_GATED_DELTA: inner width of the two-matrix decay projection */
  int32_t rank_gate;    /* L3_MIX_GATED_DELTA: inner width of the two-matrix output-gate projection */
  int32_t ff;           /* width of the gated feed-forward; 0 = the layer has none */
  float scale;          /* L3_MIX_SOFTMAX: multiplier of q . k */
  const float* decay;   /* L3_MIX_DECAY_LINEAR: [heads] decays (host memory, copied by l3_create_stack) */
  /* L3_MIX_LATENT: dim = un-rotated query / key size per head, vdim = value size per head */
  int32_t q_rank, kv_rank;   /* widths of the query latent and of the cached key / value latent */
  int32_t rot_dim, rot_dims; /* rotated query / key size per head; how many of its leading entries rotate (even) */
  double rot_base;           /* pair i turns by position * rot_base^(-2 i / rot_dims) */
  /* feed-forward as a mixture of experts (experts > 0; ff is then one expert's width):
   * expert e = down_e relu(up_e x)^2; the router scores experts + identity slots with a softmax, picks `top` of them by
   * score + correction inside the `groups_keep` best of `groups` equal groups of neighbours, and weighs the picked
   * ones by router_scale * score (not renormalised); an identity slot returns its input */
  int32_t experts, top, identity, groups, groups_keep;
  float router_scale;
  /* L3_MIX_DIFF (also uses heads, kv_heads, dim, vdim, scale, rot_dims, rot_base) */
  int32_t window;            /* keys a query sees, itself included; 0 = all */
  float diff;                /* constant of lambda and of the output multiplier (1 - diff) */
  /* wavelength-dependent rescaling of the rotary frequencies (rot_scale_original 0: none): with l = 2 pi / f, f stays
   * where l < original / high, becomes f / factor where l > original / low, and in between
   * (1 - s) f / factor + s f with s = (original / l - low) / (high - low) */
  float rot_scale_factor, rot_scale_low, rot_scale_high;
  int32_t rot_scale_original;
  int32_t ff_kind;           /* L3_FF_* of the dense feed-forward */
  int32_t router_kind;       /* L3_ROUTE_* of the mixture of experts */
  int32_t shared_ff;         /* L3_ROUTE_SIGMOID_IN: width of the shared expert; 0 = none */
  /* L3_MIX_WINDOW (also uses heads, kv_heads, dim, vdim, scale, window, rot_dims, rot_base) */
  int32_t keep_first;        /* the first keep_first tokens stay visible behind the window */
  int32_t attn_kind;         /* L3_ATTN_* */
  int32_t rot_layout;        /* 0: entry 2i turns with 2i + 1; 1: entry i with i + rot_dims / 2 */
  int32_t qk_unit;           /* 1: q and k over their root mean square per head, after the rotation */
  int32_t out_norm_groups;   /* L3_MIX_SSD: parts of the output norm */
  float tau;                 /* L3_MIX_GLA: the decay is sigmoid(.)^(1 / tau) */
  /* Two mixers side by side (pre-norm stacks): `pair` (may be null) names a second mixer that reads the same input; the
   * layer's mixer result is mix_scale * mixer + pair_scale * pair mixer.  The first mixer's tensors are then named
   * l<i>.mix.left.*, the second's l<i>.mix.right.*; of the pair spec only the mixer fields are read (no ff, no pair). */
  const struct L3LayerSpec* pair;
  float mix_scale, pair_scale;
} L3LayerSpec;

typedef struct L3StackConfig {
  int32_t width, vocab, n_layers;
  int32_t max_seq_len, max_batch_size;
  int32_t dtype, device, flags;   /* as in L3Config */
  float norm_eps;
  float residual_mult;   /* x <- x + residual_mult * norm(sublayer(x)): the norm sits on the sublayer's OUTPUT */
  int32_t norm_one_plus; /* 1: the layer norms and the final norm multiply by (1 + w) */
  int32_t glu_act;       /* activation of the feed-forward's gate: 0 silu, 1 tanh-GELU */
  int32_t side_dim;      /* per-layer token input: width of each layer's slice of the side embedding; 0 = none */
  int32_t norm_input;    /* 1: pre-norm layers  x <- x + sublayer(norm(x))  (residual_mult, norm_one_plus, side_dim unused) */
  int32_t norm_scalar;   /* 1: every layer norm and the final norm has ONE weight for all coordinates */
  int32_t token_shift;   /* 1: the mixer reads h + (h_prev - h) * shift, h_prev = the previous token's normed input
                               (zeros ahead of position 0; kept per sequence slot and layer run); tensor l<i>.shift */
  float embed_scale;     /* multiplier of the embedding rows; 0 = 1 */
  /* layers [loop_start, loop_stop) run loop_times times in a row with the same weights, every pass with its own
   * caches and states; ahead of pass t the row t of the tensor "loop.step" [loop_times, width] is added to x.
   * loop_times 0 = no loop.  A "layer run" is one execution of a layer; runs are numbered in execution order. */
  int32_t loop_start, loop_stop, loop_times;
  /* parallel layers (needs norm_input): ONE norm per layer, h = norm1(x), and both sublayers read it:
   *   X_(i+1) = x + ls1 * mixer(h + conv1(h)) + ls2 * ff(h + conv2(h))
   * norm_center 1: the norms (layer norms and the final norm) subtract the mean first (layer norm with a weight, no bias);
   * layer_scale 1: tensors l<i>.ls1 / ls2 [width] multiply the sublayers' results (0: ones);
   * canon_taps T > 0: every sublayer reads h + conv(h), conv(h)_t = sum_j w[:, j] h_(t - T + 1 + j), a causal convolution
   *   over time per channel (tensors l<i>.canon1 / canon2 [width, T], zeros ahead of position 0; the last T - 1 rows of h
   *   are kept per sequence slot and layer run);
   * depth_avg 1: what goes on to the next layer (and to the final norm) is sum_(j <= i+1) dwa_i[j] X_j with X_0 the
   *   embedding output and X_(i+1) layer i's own result (tensor l<i>.dwa [i + 2]). */
  int32_t parallel, norm_center, layer_scale, canon_taps, depth_avg;
  /* pre-norm stacks: norm_groups G > 1: every layer norm, the embedding norm and the final norm cut the vector into G equal
   * consecutive parts and divide each by its own root mean square;
   * embed_norm 1: the embedding rows pass such a norm (tensor embed.norm) before the first layer;
   * loop_in 1: ahead of every pass of the looped block the stream becomes W [x ; x0] (tensor loop.in [width, 2 width],
   *   x0 = the embedding output) instead of x + loop.step[pass];
   * logit_softcap c > 0: logits <- c tanh(logits / c). */
  int32_t norm_groups, embed_norm, loop_in;
  float logit_softcap;
} L3StackConfig;

int l3_create_stack(const L3StackConfig* cfg, const L3LayerSpec* layers, L3Model** out);
/* One tensor by its checkpoint name ("embed", "side.embed", "l<i>.norm1", "l<i>.mix.q", "l<i>.mlp.gate",
 * "l<i>.side.proj", "final.norm", "head", ...): float32, C-contiguous, matrices stored [out, in]. */
int l3_load_tensor(L3Model* m, const char* name, const float* host, const int64_t* shape, int ndim);
/* l3_forward with the logits of chosen rows: rows[i] = b * L + t of the [B, L] block, logits_out
 * [n_rows, vocab] float32.  resid_out (may be NULL, stack handles only): the residual stream after every
 * layer run, [n_runs, B * L, width] float32 (l3_stack_runs; = n_layers without a loop). */
int l3_forward_rows(L3Model* m, const int32_t* ids, int B, int L, int start_pos, const int32_t* rows, int n_rows,
                    float* logits_out, float* resid_out);
/* Number of layer runs of a stack handle (a layer inside the loop counts once per pass). */
int l3_stack_runs(L3Model* m, int* n_runs_out);
/* Recurrent state of one layer run and slot (tests): S [heads, dim, vdim] float32; conv_out (may be NULL)
 * [channels, taps - 1] float32, the convolution's tail, oldest input first.  L3_MIX_LATENT: S receives the
 * slot's latent cache [max_seq_len, kv_rank + rot_dim].  `layer` counts layer runs. */
int l3_read_state(L3Model* m, int layer, int slot, float* S_out, float* conv_out);

/* -- state inspection (tests): the layer's caches in the reference's layout
 * [max_batch, max_seq_len, n_kv_heads, head_dim] (llama3.py:138-153), as float32. */
int l3_read_cache(L3Model* m, int layer, float* k_out, float* v_out);

/* -- per-op entry points (parity tests against the reference's functions) ------------
 * All take HOST float32 buffers, run the same kernels the model path launches. */
/* RMSNorm.__call__ (llama3.py:111-114): x [rows, dim] */
int l3_op_rmsnorm(int device, const float* x, const float* w, float eps, int rows, int dim, float* out);
/* y = x @ W.T with W [n, k] (the `x @ self.*_weight` lines, llama3.py:99-102,166-168,211,307).
 * path: 0 auto, 1 row-streaming GEMV, 2 SIMT tiled GEMM, 3 tcgen05 (bf16 or 3xTF32 operands),
 * 4 tcgen05 with swapped operand roles (rows <= 128, n >= 128).
 * w_bf16 != 0 rounds W (and for path 3 x) to bf16 first. */
int l3_op_linear(int device, const float* x, const float* w, int rows, int n, int k,
                 int path, int w_bf16, float* out);
/* apply_rotary_emb (llama3.py:41-76) on one tensor x [B, L, heads, head_dim] at positions
 * start_pos..start_pos+L-1; tables [max_pos, head_dim/2] float64. */
int l3_op_rope(int device, const float* x, const double* cos_tab, const double* sin_tab,
               int B, int L, int heads, int head_dim, int start_pos, float* out);
/* silu(gate) * up (llama3.py:27-28, 99-101) elementwise over n values */
int l3_op_swiglu(int device, const float* gate, const float* up, int64_t n, float* out);
/* Attention core (llama3.py:190-207): q [B, L, HN, HD]; k, v caches in the reference layout
 * [B, T, KVHN, HD] holding T = start_pos + L valid positions; out [B, L, HN*HD]. */
int l3_op_attention(int device, const float* q, const float* k, const float* v,
                    int B, int L, int n_heads, int n_kv_heads, int head_dim, int start_pos,
                    int kv_bf16 /* 0 fp32 cache, 1 bf16 cache, 2 bf16 tensor-core prefill (L > 1, head_dim 64/128),
                                   3 bf16 cache, decode through the exact (non tensor-core) kernels */,
                    int nsplit /* decode split-KV factor, 0 = auto */, float* out);
/* logits[:, -1, :].argmax(-1) (llama3.py:320): first maximum wins. */
int l3_op_argmax(int device, const float* logits, int rows, int n, int64_t* out);

/* Debug: switch the tcgen05 GEMM's clock64 milestone stamps on/off and read the last 64
 * stamps of CTA (0,0) (indices documented in gemm_tc.cu). */
int l3_debug_tc_timeline(int device, int enable, uint64_t* out64);

/* -- measurement helpers (bench.py): CUDA events on the handle's own stream ---------- */
int l3_sync(L3Model* m);
int l3_timer_start(L3Model* m);
int l3_timer_stop(L3Model* m, float* ms_out);      /* records, synchronises, returns ms */
int l3_dev_alloc(L3Model* m, int64_t bytes, void** out);
int l3_dev_free(L3Model* m, void* p);
int l3_memcpy_h2d(L3Model* m, void* dst, const void* src, int64_t bytes);
int l3_memcpy_d2h(L3Model* m, void* dst, const void* src, int64_t bytes);
int l3_flush_l2(L3Model* m);                        /* writes a buffer larger than L2 */
/* Number of kernel launches (graph nodes count individually) since the last call. */
int l3_launch_count(L3Model* m, int64_t* out, int reset);
/* Time one kernel family in isolation on the current model state (bench roofline leg):
 * which: 0 = decode attention at position `pos` for batch B, 1 = LM head for B rows, 2 = the FFN leg of a
 * layer (RMSNorm + gate|up + down), 3 = the two residual projections of a layer (Wo, Wdown: one kernel symbol);
 * batched decode path (decode_stack.cu), each launch timed alone after an L2 flush: 4 = the cluster-resident kernel
 * (every layer of one decode step at `pos`), 5 = its LM head with the fused argmax.
 * Runs `iters` launches bracketed by events; returns average ms. */
int l3_bench_kernel(L3Model* m, int which, int B, int pos, int iters, float* avg_ms);

/* Debug: %globaltimer stamps of the last persistent decode step, [n_sm][512] (layout in decode_mega.cu);
 * needs L3_MEGA_DBG=1 in the environment when the model is created. */
int l3_debug_mega_timeline(L3Model* m, uint64_t* out, int64_t capacity);

/* Debug of the cluster-resident batched-decode kernel (decode_stack.cu), last step; needs L3_STACK_DBG=1 when the
 * model is created.  which 0: %globaltimer stamps uint64 [clusters * 8][128] (row = CTA, layout in the kernel);
 * which 1: float [n_layers][max_batch_size][dim], the residual stream after every layer. */
int l3_debug_stack(L3Model* m, int which, void* out, int64_t capacity_bytes);

/* Micro-benchmark of the row-streaming GEMV (y = W x, W [n, k]) at one shape, weights rotated
 * over more copies than fit the L2: average ms per launch over `iters` launches. */
int l3_bench_gemv(int device, int n, int k, int w_bf16, int rows, int iters, float* avg_ms);

/* Micro-benchmark of the tensor pipe alone (csrc/mma_probe.cu, scripts/mma_cost.py): cycles per
 * tcgen05.mma of M = 128, K = 32 bytes, width n (16..256), kind 0 = bf16 / 1 = tf32, issued by one thread
 * rotating over nacc TMEM accumulators (nacc * n <= 512), `iters` groups of four, on `ctas` CTAs at once.
 * cycles_per_mma[0] = issue loop, [1] = issue + completion (maximum over the CTAs).  No reference
 * counterpart: a design input for the GEMM kernels. */
int l3_probe_mma(int device, int kind, int n, int nacc, int iters, int ctas, double* cycles_per_mma);

#ifdef __cplusplus
}
#endif
#endif /* LLAMA3_B200_H */
