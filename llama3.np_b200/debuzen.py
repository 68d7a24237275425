"""Debuzen: a pre-norm decoder of hybrid layers.  Every norm is an RMS norm in groups (the vector is cut into
`norm.groups` equal parts, each over its own root mean square); the embedding rows pass such a norm; the mixer
reads its input mixed with the previous token's (token shift); a block of layers may run several times with one
set of weights, and ahead of every pass the stream becomes `W [x ; x0]` with x0 the embedding output; the
feed-forward is a silu-gated unit; the logits pass a tanh soft cap.  Layer types:

* `parallel`: two mixers side by side on the same input, summed with fixed weights - sliding-window attention that
  keeps the first tokens visible, rotary pairs (2i, 2i + 1), q and k over their root mean square, un-normalised
  sigmoid weights with a bias per head; and a gated delta rule behind short convolutions;
* `parallel_2`: sliding-window softmax attention with a sink per head in the denominator, rotary pairs
  (i, i + dims / 2); and a Mamba-2 state-space mixer;
* `gla`: gated linear attention with a decay per key channel.

The arithmetic lives in the library's layer-list path (csrc/layerlist.cu, attn_window.cu, hybrid_ops.cu,
recurrent.cu); this file reads `config.json`, names the tensors and builds the `StackConfig`.  Sizes that the
configuration does not spell out (the inner widths of the two-matrix projections) come from the tensors' shapes.
The reference has one fixed block (llama3.py:238-262) and no counterpart of this.

A checkpoint folder holds `config.json` (keys: architecture, vocab, width, norm.eps / groups, loop.start / stop /
times, logit_softcap, layers[].type / mixer / mlp) and `model.safetensors` (tensor names `embed`, `embed.norm`,
`loop.in`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.shift`, `l<i>.mix.*` or `l<i>.mix.left.*` / `l<i>.mix.right.*`,
`l<i>.mlp.gate / up / down`, `final.norm`, `head`).
"""
from __future__ import annotations

import json
import os
from typing import Mapping, Optional

import numpy as np

from .stack import (ATTN_SIGMOID, ATTN_SINK, GATED_DELTA, GLA, SSD, WINDOW, LayerSpec, StackConfig, StackDecoder)
from .utils import read_safetensors

DEFAULT_RANK = 16   # inner width of a two-matrix projection when neither a tensor nor the configuration gives it


def _window(mc: Mapping, kind: int, layout: int) -> LayerSpec:
    rot, mask = mc.get("rot") or {}, mc.get("mask") or {}
    return LayerSpec(mixer=WINDOW, heads=int(mc["heads"]), kv_heads=int(mc.get("kv_heads", mc["heads"])), dim=int(mc["dim"]),
                     vdim=int(mc["vdim"]), scale=float(mc["scale"]), window=int(mask.get("size", 0)),
                     keep_first=int(mask.get("keep_first", 0)), rot_dims=int(rot.get("dims", 0)),
                     rot_base=float(rot.get("base", 10000.0)), rot_layout=layout, attn_kind=kind, qk_unit=kind == ATTN_SIGMOID)


def _rank(shapes, name: str, mc: Mapping, key: str) -> int:
    if shapes is not None and name in shapes:
        return int(shapes[name][0])
    return int(mc.get(key, DEFAULT_RANK))


def stack_config(config: Mapping, shapes: Optional[Mapping] = None, *, max_seq_len: int = 256, max_batch_size: int = 1,
                 dtype: str = "float32") -> StackConfig:
    """`config.json` (as a dict) and the tensors' shapes (name -> shape; None: ranks from the configuration) -> StackConfig."""
    layers = []
    for i, lc in enumerate(config["layers"]):
        kind, mc, p = lc["type"], lc["mixer"], f"l{i}.mix."
        if kind in ("parallel", "parallel_2"):
            r, rp = mc["right"], p + "right."
            if kind == "parallel":
                spec = _window(mc["left"], ATTN_SIGMOID, 0)
                right = LayerSpec(mixer=GATED_DELTA, heads=int(r["heads"]), kv_heads=int(r.get("kv_heads", r["heads"])),
                                  dim=int(r["dim"]), vdim=int(r["vdim"]), conv_taps=int(r["conv"]),
                                  rank_decay=_rank(shapes, rp + "a1", r, "rank_decay"), rank_gate=_rank(shapes, rp + "g1", r, "rank_gate"))
            else:
                spec = _window(mc["left"], ATTN_SINK, 1)
                right = LayerSpec(mixer=SSD, heads=int(r["heads"]), kv_heads=int(r.get("groups", 1)), dim=int(r["state"]),
                                  vdim=int(r["vdim"]), conv_taps=int(r["conv"]), out_norm_groups=int(r.get("norm_groups", 1)))
            spec.pair, spec.mix_scale, spec.pair_scale = right, float(mc.get("left_scale", 1.0)), float(mc.get("right_scale", 1.0))
        elif kind == "gla":
            spec = LayerSpec(mixer=GLA, heads=int(mc["heads"]), dim=int(mc["dim"]), vdim=int(mc["vdim"]), tau=float(mc["tau"]),
                             rank_decay=_rank(shapes, p + "a1", mc, "rank_decay"))
        else:
            raise ValueError(f"layer {i}: unknown layer type {kind!r}")
        mlp = lc.get("mlp")
        if mlp is not None:
            if mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            spec.ff = int(mlp["ff"])
        layers.append(spec)
    lp = config.get("loop")
    loop = (int(lp["start"]), int(lp["stop"]), int(lp["times"])) if lp and int(lp.get("times", 0)) > 0 else None
    norm = config.get("norm") or {}
    return StackConfig(width=int(config["width"]), vocab=int(config["vocab"]), layers=layers,
                       norm_eps=float(norm.get("eps", 1e-6)), norm_one_plus=False, glu_act="silu", norm_input=True,
                       token_shift=True, loop=loop, norm_groups=int(norm.get("groups", 1)), embed_norm=True,
                       loop_in=loop is not None, logit_softcap=float(config.get("logit_softcap") or 0.0),
                       max_seq_len=max_seq_len, max_batch_size=max_batch_size, dtype=dtype)


class Debuzen(StackDecoder):
    architecture = "Debuzen"

    def __init__(self, config: Mapping, tensors: Optional[Mapping[str, np.ndarray]] = None, *, max_seq_len: int = 256,
                 max_batch_size: int = 1, dtype: str = "float32", device: int = 0, random_seed: Optional[int] = None,
                 flags: int = 0):
        """`tensors`: checkpoint name -> array; or None with `random_seed` for random weights on the device."""
        if tensors is None and random_seed is None:
            raise ValueError("tensors=None needs random_seed")
        self.config = dict(config)
        shapes = {k: np.shape(v) for k, v in tensors.items()} if tensors is not None else None
        lp = config.get("loop")
        if tensors is not None and not (lp and int(lp.get("times", 0)) > 0) and "loop.in" in tensors:
            tensors = {k: v for k, v in tensors.items() if k != "loop.in"}   # no pass ever starts: the entry projection is unused
        super().__init__(stack_config(config, shapes, max_seq_len=max_seq_len, max_batch_size=max_batch_size, dtype=dtype),
                         device=device, flags=flags)
        if tensors is not None:
            self.load_tensors(tensors)
        else:
            self.fill_random(random_seed)

    @classmethod
    def from_pretrained(cls, model_dir, **kw) -> "Debuzen":
        with open(os.path.join(model_dir, "config.json")) as f:
            config = json.load(f)
        return cls(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), **kw)
