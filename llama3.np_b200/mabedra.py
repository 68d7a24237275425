"""Mabedra: a decoder of parallel layers.  Every layer has ONE norm (a layer norm with a weight, no bias) whose output
both sublayers read, each through a short causal convolution over time of its own (`h + conv(h)`); the sublayers'
results are scaled per channel (layer scale) and added to the stream together; what goes on to the next layer is a
learned weighted sum of the embedding output and every layer's own result so far (depth average).  The mixer is
differential sliding-window attention: two attention maps per head over the same values, combined as
`a1 - lambda a2` and normed per head, with biased q / k / v, an RMS norm per head and map, rotary positions in the
rotate-half layout on the leading part of each map with wavelength-dependent frequency scaling, and GQA.  The
feed-forward is either dense with the PolyNorm activation or a mixture of gated silu experts routed by sigmoid
scores whose weights multiply the experts' INPUT, plus a shared expert; a layer may also have none.  The arithmetic
lives in the library's layer-list path (csrc/layerlist.cu `ll_enqueue_parallel`, attn_diff.cu, parallel_ops.cu,
moe.cu); this file reads `config.json`, names the tensors and builds the `StackConfig`.

A checkpoint folder holds `config.json` (keys: architecture, vocab, width, norm.eps, canon.taps, layers[].type /
mixer {heads, kv_heads, dim, vdim, scale, diff, mask.size, rot {base, dims, scaling {factor, low, high, original}}} /
mlp {kind: dense | moe, ff | expert.ff, router {experts, top}, shared.ff} or null) and `model.safetensors`
(`embed`, `l<i>.norm1`, `l<i>.mix.q|k|v` + `.b`, `l<i>.mix.q.norm|k.norm`, `l<i>.mix.lq1|lk1|lq2|lk2`, `l<i>.mix.o`,
`l<i>.mlp.up|down|act` or `l<i>.mlp.router`, `l<i>.mlp.e<k>.gate|up|down`, `l<i>.mlp.shared.gate|up|down`,
`l<i>.ls1|ls2`, `l<i>.canon1|canon2`, `l<i>.dwa`, `final.norm`, `head`).
"""
from __future__ import annotations

import json
import os
from typing import Mapping, Optional

import numpy as np

from .stack import DIFF, FF_POLYNORM, ROUTE_SIGMOID_IN, LayerSpec, StackConfig, StackDecoder
from .utils import read_safetensors


def stack_config(config: Mapping, *, max_seq_len: int = 256, max_batch_size: int = 1, dtype: str = "float32") -> StackConfig:
    """`config.json` (as a dict) -> StackConfig."""
    layers = []
    for i, lc in enumerate(config["layers"]):
        kind, mc = lc["type"], lc["mixer"]
        if kind != "attention":
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        rot = mc.get("rot") or {}
        sc = rot.get("scaling")
        heads = int(mc["heads"])
        spec = LayerSpec(mixer=DIFF, heads=heads, kv_heads=int(mc.get("kv_heads", heads)), dim=int(mc["dim"]),
                         vdim=int(mc.get("vdim", mc["dim"])), scale=float(mc["scale"]), diff=float(mc["diff"]),
                         window=int((mc.get("mask") or {}).get("size", 0)), rot_dims=int(rot.get("dims", 0)),
                         rot_base=float(rot.get("base", 10000.0)),
                         rot_scaling=(float(sc["factor"]), float(sc["low"]), float(sc["high"]), int(sc["original"])) if sc else None)
        mlp = lc.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                spec.ff = int(mlp["ff"])
                spec.ff_kind = FF_POLYNORM
            elif mlp["kind"] == "moe":
                spec.ff = int(mlp["expert"]["ff"])
                spec.experts = int(mlp["router"]["experts"])
                spec.top = int(mlp["router"]["top"])
                spec.router_kind = ROUTE_SIGMOID_IN
                spec.shared_ff = int((mlp.get("shared") or {}).get("ff", 0))
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
        layers.append(spec)
    return StackConfig(width=int(config["width"]), vocab=int(config["vocab"]), layers=layers,
                       norm_eps=float(config["norm"]["eps"]), norm_one_plus=False, norm_input=True, parallel=True,
                       norm_center=True, layer_scale=True, canon_taps=int((config.get("canon") or {}).get("taps", 0)),
                       depth_avg=True, glu_act="silu", max_seq_len=max_seq_len, max_batch_size=max_batch_size, dtype=dtype)


class Mabedra(StackDecoder):
    architecture = "Mabedra"

    def __init__(self, config: Mapping, tensors: Optional[Mapping[str, np.ndarray]] = None, *, max_seq_len: int = 256,
                 max_batch_size: int = 1, dtype: str = "float32", device: int = 0, random_seed: Optional[int] = None,
                 flags: int = 0):
        """`tensors`: checkpoint name -> array; or None with `random_seed` for random weights on the device."""
        if tensors is None and random_seed is None:
            raise ValueError("tensors=None needs random_seed")
        self.config = dict(config)
        super().__init__(stack_config(config, max_seq_len=max_seq_len, max_batch_size=max_batch_size, dtype=dtype),
                         device=device, flags=flags)
        if tensors is not None:
            self.load_tensors(tensors)
        else:
            self.fill_random(random_seed)

    @classmethod
    def from_pretrained(cls, model_dir, **kw) -> "Mabedra":
        with open(os.path.join(model_dir, "config.json")) as f:
            config = json.load(f)
        return cls(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), **kw)
