"""Layer-list decoders on the C-ABI's stack handles (`l3_create_stack`, include/llama3_b200.h).

`StackDecoder` is the host side every such model shares: the handle's lifetime, tensors by checkpoint
name, the forward call (logits of the last token, or of chosen rows), the greedy generate loop of the
library (CUDA-graph replays, next ids on the device) and the per-slot state rules - a call at
`start_pos` 0 starts its sequence slots afresh, any other call continues them.  A model family (e.g.
`risalix.Risalix`) only turns its configuration into a `StackConfig` and a list of `LayerSpec`s.
The reference has one fixed block (llama3.py:238-262) and no counterpart of this.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Mapping, Optional, Sequence, Tuple

import numpy as np

from . import _cabi

SOFTMAX, DECAY_LINEAR, GATED_DELTA = _cabi.MIX_SOFTMAX, _cabi.MIX_DECAY_LINEAR, _cabi.MIX_GATED_DELTA
LATENT, MINGRU, DIFF = _cabi.MIX_LATENT, _cabi.MIX_MINGRU, _cabi.MIX_DIFF
WINDOW, SSD, GLA = _cabi.MIX_WINDOW, _cabi.MIX_SSD, _cabi.MIX_GLA
ATTN_SINK, ATTN_SIGMOID = _cabi.ATTN_SINK, _cabi.ATTN_SIGMOID
FF_GLU, FF_POLYNORM = _cabi.FF_GLU, _cabi.FF_POLYNORM
ROUTE_SOFTMAX, ROUTE_SIGMOID_IN = _cabi.ROUTE_SOFTMAX, _cabi.ROUTE_SIGMOID_IN
_DTYPES = {"float32": _cabi.DTYPE_F32, "fp32": _cabi.DTYPE_F32, "bfloat16": _cabi.DTYPE_BF16, "bf16": _cabi.DTYPE_BF16}


@dataclass
class LayerSpec:
    mixer: int                    # SOFTMAX | DECAY_LINEAR | GATED_DELTA | LATENT | MINGRU
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0             # 0: = heads
    conv_taps: int = 0            # GATED_DELTA
    rank_decay: int = 0           # GATED_DELTA: inner width of the decay projection pair
    rank_gate: int = 0            # GATED_DELTA: inner width of the output-gate projection pair
    ff: int = 0                   # 0: no feed-forward in this layer
    scale: float = 0.0            # SOFTMAX: multiplier of q . k
    decay: Sequence[float] = ()   # DECAY_LINEAR: one per head
    q_rank: int = 0               # LATENT: width of the query latent
    kv_rank: int = 0              # LATENT: width of the cached key / value latent
    rot_dim: int = 0              # LATENT: rotated query / key size per head (dim is the un-rotated size)
    rot_dims: int = 0             # LATENT: leading entries of the rotated part that turn
    rot_base: float = 10000.0
    experts: int = 0              # > 0: the feed-forward is a mixture of experts of width ff each
    top: int = 0
    identity: int = 0             # router slots behind the experts that return their input
    groups: int = 1
    groups_keep: int = 1
    router_scale: float = 1.0
    window: int = 0               # DIFF: keys a query sees, itself included; 0 = all
    diff: float = 0.0             # DIFF: constant of lambda and of the output multiplier 1 - diff
    rot_scaling: Optional[Tuple[float, float, float, int]] = None   # DIFF: (factor, low, high, original) or None
    ff_kind: int = 0              # FF_GLU | FF_POLYNORM
    router_kind: int = 0          # ROUTE_SOFTMAX | ROUTE_SIGMOID_IN
    shared_ff: int = 0            # ROUTE_SIGMOID_IN: width of the shared expert
    keep_first: int = 0           # WINDOW: the first tokens that stay visible behind the window
    attn_kind: int = 0            # WINDOW: ATTN_SINK (softmax with a sink per head) | ATTN_SIGMOID (sigmoid(score + bias), not normalised)
    rot_layout: int = 0           # WINDOW: 0 = entries (2i, 2i + 1) turn together, 1 = entries (i, i + rot_dims / 2)
    qk_unit: bool = False         # WINDOW: q and k over their root mean square per head, after the rotation
    out_norm_groups: int = 1      # SSD: parts of the output norm
    tau: float = 1.0              # GLA: the decay is sigmoid(.)^(1 / tau)
    pair: Optional["LayerSpec"] = None   # a second mixer on the same input (tensors mix.left.* / mix.right.*)
    mix_scale: float = 1.0        # with `pair`: result = mix_scale * mixer + pair_scale * pair mixer
    pair_scale: float = 1.0


@dataclass
class StackConfig:
    width: int
    vocab: int
    layers: List[LayerSpec] = field(default_factory=list)
    norm_eps: float = 1e-5
    residual_mult: float = 1.0
    norm_one_plus: bool = True
    glu_act: str = "gelu_tanh"    # "silu" | "gelu_tanh"
    side_dim: int = 0
    norm_input: bool = False      # pre-norm layers: x += sublayer(norm(x))
    norm_scalar: bool = False     # every norm has one weight
    token_shift: bool = False     # the mixer reads its input mixed with the previous token's
    embed_scale: float = 1.0
    loop: Optional[Tuple[int, int, int]] = None   # (start, stop, times): layers [start, stop) run `times` times
    parallel: bool = False        # one norm per layer, the mixer and the feed-forward both read it
    norm_center: bool = False     # norms subtract the mean (layer norm with a weight, no bias)
    layer_scale: bool = False     # per-channel multipliers l<i>.ls1 / ls2 on the sublayers' results
    canon_taps: int = 0           # taps of the causal convolution ahead of every sublayer; 0 = none
    depth_avg: bool = False       # the stream handed on is a weighted sum of every earlier layer's result
    norm_groups: int = 1          # pre-norm stacks: every norm cuts the vector into this many parts, each over its own RMS
    embed_norm: bool = False      # the embedding rows pass a norm (tensor embed.norm)
    loop_in: bool = False         # ahead of every pass of the loop x <- W [x ; x0] (tensor loop.in) instead of x + loop.step[pass]
    logit_softcap: float = 0.0    # c > 0: logits <- c tanh(logits / c)
    max_seq_len: int = 256
    max_batch_size: int = 1
    dtype: str = "float32"


class StackDecoder:
    def __init__(self, cfg: StackConfig, *, device: int = 0, flags: int = 0):
        if cfg.dtype not in _DTYPES:
            raise ValueError(f"unsupported dtype {cfg.dtype!r}; use 'float32' or 'bfloat16'")
        if cfg.glu_act not in ("silu", "gelu_tanh"):
            raise ValueError(f"unsupported activation {cfg.glu_act!r}")
        self.cfg = cfg
        self._lib = _cabi.lib()
        self._h = C.c_void_p()
        self._finalized = False
        specs = (_cabi.L3LayerSpec * len(cfg.layers))()
        keep = []

        def c_spec(i, l):
            dec = (C.c_float * max(1, len(l.decay)))(*[float(x) for x in l.decay])
            keep.append(dec)
            if l.mixer == DECAY_LINEAR and len(l.decay) != l.heads:
                raise ValueError(f"layer {i}: {len(l.decay)} decays for {l.heads} heads")
            pair = None
            if l.pair is not None:
                pair = c_spec(i, l.pair)
                keep.append(pair)
            return _cabi.L3LayerSpec(mixer=l.mixer, heads=l.heads, kv_heads=l.kv_heads or l.heads, dim=l.dim, vdim=l.vdim,
                                         conv_taps=l.conv_taps, rank_decay=l.rank_decay, rank_gate=l.rank_gate, ff=l.ff,
                                         scale=l.scale, decay=C.cast(dec, C.POINTER(C.c_float)) if len(l.decay) else None,
                                         q_rank=l.q_rank, kv_rank=l.kv_rank, rot_dim=l.rot_dim, rot_dims=l.rot_dims,
                                         rot_base=float(l.rot_base), experts=l.experts, top=l.top, identity=l.identity,
                                         groups=l.groups, groups_keep=l.groups_keep, router_scale=float(l.router_scale),
                                         window=l.window, diff=float(l.diff),
                                         rot_scale_factor=float(l.rot_scaling[0]) if l.rot_scaling else 1.0,
                                         rot_scale_low=float(l.rot_scaling[1]) if l.rot_scaling else 0.0,
                                         rot_scale_high=float(l.rot_scaling[2]) if l.rot_scaling else 0.0,
                                         rot_scale_original=int(l.rot_scaling[3]) if l.rot_scaling else 0,
                                         ff_kind=l.ff_kind, router_kind=l.router_kind, shared_ff=l.shared_ff,
                                         keep_first=l.keep_first, attn_kind=l.attn_kind, rot_layout=l.rot_layout,
                                         qk_unit=int(l.qk_unit), out_norm_groups=l.out_norm_groups, tau=float(l.tau),
                                         pair=C.pointer(pair) if pair is not None else None,
                                         mix_scale=float(l.mix_scale), pair_scale=float(l.pair_scale))

        for i, l in enumerate(cfg.layers):
            specs[i] = c_spec(i, l)
        c = _cabi.L3StackConfig(width=cfg.width, vocab=cfg.vocab, n_layers=len(cfg.layers), max_seq_len=cfg.max_seq_len,
                                max_batch_size=cfg.max_batch_size, dtype=_DTYPES[cfg.dtype], device=device, flags=flags,
                                norm_eps=cfg.norm_eps, residual_mult=cfg.residual_mult, norm_one_plus=int(cfg.norm_one_plus),
                                glu_act=_cabi.GLU_GELU_TANH if cfg.glu_act == "gelu_tanh" else _cabi.GLU_SILU,
                                side_dim=cfg.side_dim, norm_input=int(cfg.norm_input), norm_scalar=int(cfg.norm_scalar),
                                token_shift=int(cfg.token_shift), embed_scale=float(cfg.embed_scale),
                                loop_start=cfg.loop[0] if cfg.loop else 0, loop_stop=cfg.loop[1] if cfg.loop else 0,
                                loop_times=cfg.loop[2] if cfg.loop else 0, parallel=int(cfg.parallel),
                                norm_center=int(cfg.norm_center), layer_scale=int(cfg.layer_scale),
                                canon_taps=int(cfg.canon_taps), depth_avg=int(cfg.depth_avg), norm_groups=int(cfg.norm_groups),
                                embed_norm=int(cfg.embed_norm), loop_in=int(cfg.loop_in), logit_softcap=float(cfg.logit_softcap))
        _cabi.check(self._lib.l3_create_stack(C.byref(c), specs, C.byref(self._h)))
        n = C.c_int()
        _cabi.check(self._lib.l3_stack_runs(self._h, C.byref(n)), self._h)
        self.n_runs = n.value  # executions of a layer per token: a layer inside the loop counts once per pass

    # ---------------------------------------------------------------- lifetime / weights
    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.l3_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load_tensors(self, tensors: Mapping[str, np.ndarray]) -> None:
        """Upload every tensor of the mapping (checkpoint names) and finish the model.  A tensor of the wrong shape
        or one the model does not know is an error, as is a missing tensor."""
        try:
            for name in tensors.keys():
                w = np.ascontiguousarray(tensors[name], dtype=np.float32)
                if w.ndim == 0:  # a single number travels as a vector of one
                    w = w.reshape(1)
                shape = (C.c_int64 * max(1, w.ndim))(*w.shape)
                _cabi.check(self._lib.l3_load_tensor(self._h, name.encode(), _cabi.f32p(w), shape, w.ndim), self._h)
            self.finalize()
        except Exception:
            self.close()
            raise

    def fill_random(self, seed: int) -> None:
        """Random weights on the device (benchmarks of shapes no checkpoint exists for), then finish the model."""
        try:
            _cabi.check(self._lib.l3_fill_random(self._h, int(seed)), self._h)
            self.finalize()
        except Exception:
            self.close()
            raise

    def finalize(self) -> None:
        _cabi.check(self._lib.l3_finalize(self._h), self._h)
        self._finalized = True

    def reset(self) -> None:
        """Zero every slot's KV cache and recurrent state."""
        _cabi.check(self._lib.l3_reset_cache(self._h), self._h)

    # ---------------------------------------------------------------- forward
    @staticmethod
    def _ids(input_ids):
        ids = np.asarray(input_ids)
        if ids.ndim != 2:
            raise ValueError(f"input_ids must be [B, L], got shape {ids.shape}")
        if not np.issubdtype(ids.dtype, np.integer):
            raise ValueError("input_ids must be integers")
        return np.ascontiguousarray(ids, dtype=np.int32)

    def forward(self, input_ids, start_pos: int) -> np.ndarray:
        """`[B, L]` ids for slots 0..B-1 at `start_pos` -> float32 logits `[B, vocab]` of the last token."""
        ids = self._ids(input_ids)
        B, L = ids.shape
        logits = np.empty((B, self.cfg.vocab), dtype=np.float32)
        _cabi.check(self._lib.l3_forward(self._h, _cabi.i32p(ids), B, L, int(start_pos), _cabi.f32p(logits), None), self._h)
        return logits

    __call__ = forward

    def forward_rows(self, input_ids, start_pos: int, rows, want_residual: bool = False):
        """As `forward`, returning the logits `[len(rows), vocab]` of the chosen rows (`b * L + t`); with
        `want_residual` also the residual stream after every layer run, `[n_runs, B * L, width]`."""
        ids = self._ids(input_ids)
        B, L = ids.shape
        rows = np.ascontiguousarray(np.asarray(rows, dtype=np.int32).reshape(-1))
        logits = np.empty((len(rows), self.cfg.vocab), dtype=np.float32)
        resid = np.empty((self.n_runs, B * L, self.cfg.width), dtype=np.float32) if want_residual else None
        _cabi.check(self._lib.l3_forward_rows(self._h, _cabi.i32p(ids), B, L, int(start_pos),
                                              _cabi.i32p(rows) if len(rows) else None, len(rows),
                                              _cabi.f32p(logits) if len(rows) else None,
                                              _cabi.f32p(resid) if want_residual else None), self._h)
        return (logits, resid) if want_residual else logits

    # ---------------------------------------------------------------- generate (greedy, the library's loop)
    def generate(self, input_ids, max_new_tokens: int):
        """Lazy greedy generator: prefill at position 0, then one decode step per `next()`; yields
        `max_new_tokens` arrays `[B, 1]` int64 (the library's step function and CUDA graphs)."""
        ids = self._ids(input_ids)
        B, L = ids.shape
        if max_new_tokens <= 0:
            return
        if L + max_new_tokens - 1 > self.cfg.max_seq_len:
            raise ValueError(f"prompt {L} + {max_new_tokens} new tokens exceed max_seq_len {self.cfg.max_seq_len}")
        _cabi.check(self._lib.l3_generate_begin(self._h, _cabi.i32p(ids), B, L), self._h)
        for _ in range(max_new_tokens):
            nxt = np.empty((B,), dtype=np.int64)
            _cabi.check(self._lib.l3_generate_next(self._h, _cabi.i64p(nxt)), self._h)
            yield nxt[:, None]

    def generate_all(self, input_ids, max_new_tokens: int) -> np.ndarray:
        """The whole greedy loop on the device; returns `[B, max_new_tokens]` int64."""
        ids = self._ids(input_ids)
        B, L = ids.shape
        out = np.empty((B, max(0, max_new_tokens)), dtype=np.int64)
        if max_new_tokens > 0:
            if L + max_new_tokens - 1 > self.cfg.max_seq_len:
                raise ValueError(f"prompt {L} + {max_new_tokens} new tokens exceed max_seq_len {self.cfg.max_seq_len}")
            # the C entry point counts the total length (prompt included), as the reference's generate does
            _cabi.check(self._lib.l3_generate_greedy(self._h, _cabi.i32p(ids), B, L, L + int(max_new_tokens), _cabi.i64p(out)),
                        self._h)
        return out

    def generate_ragged(self, prompts, max_new_tokens: int, eos_id: Optional[int] = None):
        """Greedy generation for prompts of different lengths: a list with `max_new_tokens` new ids per prompt (cut
        after the first `eos_id`, if given).  The recurrent layers take one length per call, so the scheduler here is
        length bucketing on the host: prompts of one length share a batch (at most `max_batch_size` of them), the
        buckets run one after another through `generate_all`, and every prompt yields what it yields alone."""
        seqs = [np.ascontiguousarray(np.asarray(p).reshape(-1), dtype=np.int32) for p in prompts]
        if not seqs or any(len(p) == 0 for p in seqs):
            raise ValueError("need at least one non-empty prompt")
        buckets = {}
        for i, p in enumerate(seqs):
            buckets.setdefault(len(p), []).append(i)
        out = [None] * len(seqs)
        for length in sorted(buckets):
            idx = buckets[length]
            for lo in range(0, len(idx), self.cfg.max_batch_size):
                part = idx[lo:lo + self.cfg.max_batch_size]
                toks = self.generate_all(np.stack([seqs[i] for i in part]), max_new_tokens)
                for row, i in zip(toks, part):
                    if eos_id is not None and (row == eos_id).any():
                        row = row[: int(np.argmax(row == eos_id)) + 1]
                    out[i] = row.copy()
        return out

    # ---------------------------------------------------------------- state inspection / measurement
    def run_layer(self, run: int) -> int:
        """Index of the layer that layer run `run` executes."""
        n = len(self.cfg.layers)
        if not self.cfg.loop:
            return run
        start, stop, times = self.cfg.loop
        span = stop - start
        if run < start:
            return run
        if run < start + span * times:
            return start + (run - start) % span
        return run - span * (times - 1)

    def read_state(self, layer: int, slot: int = 0):
        """(S [heads, dim, vdim], conv tail [channels, taps - 1] or None) of a recurrent layer run's slot; for a
        latent-attention run S is its cache `[max_seq_len, kv_rank + rot_dim]`.  `layer` counts layer runs."""
        l = self.cfg.layers[self.run_layer(layer)]
        if l.pair is not None and l.mixer == WINDOW:   # two mixers side by side: the recurrent one
            l = l.pair
        if l.mixer == LATENT:
            S = np.empty((self.cfg.max_seq_len, l.kv_rank + l.rot_dim), dtype=np.float32)
            _cabi.check(self._lib.l3_read_state(self._h, layer, slot, _cabi.f32p(S), None), self._h)
            return S, None
        S = np.empty((l.heads, l.dim, l.vdim), dtype=np.float32)
        tail = None
        if l.mixer in (GATED_DELTA, SSD):
            g = l.kv_heads or l.heads
            ch = 2 * g * l.dim + l.heads * l.vdim
            tail = np.empty((ch, max(0, l.conv_taps - 1)), dtype=np.float32)
        _cabi.check(self._lib.l3_read_state(self._h, layer, slot, _cabi.f32p(S), _cabi.f32p(tail) if tail is not None and tail.size else None),
                    self._h)
        return S, tail

    def read_cache(self, layer: int):
        """(keys, values) `[max_batch, max_seq_len, kv_heads, dim]` float32 of a softmax layer."""
        l = self.cfg.layers[self.run_layer(layer)]
        shape = (self.cfg.max_batch_size, self.cfg.max_seq_len, l.kv_heads or l.heads, l.dim)
        k = np.empty(shape, dtype=np.float32)
        v = np.empty(shape, dtype=np.float32)
        _cabi.check(self._lib.l3_read_cache(self._h, layer, _cabi.f32p(k), _cabi.f32p(v)), self._h)
        return k, v

    def sync(self):
        _cabi.check(self._lib.l3_sync(self._h), self._h)

    def launch_count(self, reset: bool = False) -> int:
        n = C.c_int64()
        _cabi.check(self._lib.l3_launch_count(self._h, C.byref(n), int(reset)), self._h)
        return n.value


class SlotTable:
    """Which sequence slot a live request holds.  Slots are handed out lowest-first and come back on release;
    a released slot's state is overwritten by the next sequence that starts in it (position 0)."""

    def __init__(self, n_slots: int):
        self.free = list(range(n_slots))
        self.slot = {}
        self.pos = {}

    def acquire(self, key) -> int:
        if key not in self.slot:
            if not self.free:
                raise RuntimeError("every sequence slot is taken")
            self.slot[key] = self.free.pop(0)
            self.pos[key] = 0
        return self.slot[key]

    def advance(self, key, n: int) -> None:
        self.pos[key] += n

    def release(self, key) -> None:
        if key in self.slot:
            self.free.append(self.slot.pop(key))
            self.free.sort()
            self.pos.pop(key, None)
