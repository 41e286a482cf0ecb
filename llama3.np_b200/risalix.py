"""Risalix: a decoder whose layers alternate three token mixers - softmax attention without positions
(values are the un-normalised keys, one sigmoid gate per head), linear attention with a fixed decay per
head, and a gated delta rule with a decay per head and key channel behind short convolutions - around a
post-norm residual stream (`x += m * norm(sublayer(x))`), a tanh-GELU gated feed-forward in some layers
and a per-layer token input after each.  The arithmetic lives in the library's layer-list path
(csrc/layerlist.cu, recurrent.cu, mixer_ops.cu); this file reads `config.json`, names the tensors and
builds the `StackConfig`.

A checkpoint folder holds `config.json` (keys: architecture, vocab, width, residual_mult, norm.eps,
token_side.dim, layers[].type / mixer / mlp) and `model.safetensors` (tensor names `embed`, `side.embed`,
`l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.side.*`, `final.norm`, `head`).  Sizes the config does
not state (the inner widths of the two-matrix projections) come from the tensors' shapes.
"""
from __future__ import annotations

import json
import os
from typing import Mapping, Optional

import numpy as np

from .stack import DECAY_LINEAR, GATED_DELTA, SOFTMAX, LayerSpec, StackConfig, StackDecoder
from .utils import read_safetensors

_MIXERS = {"attention": SOFTMAX, "lightning": DECAY_LINEAR, "channel_delta": GATED_DELTA}


def stack_config(config: Mapping, shapes: Optional[Mapping[str, tuple]] = None, *, max_seq_len: int = 256,
                 max_batch_size: int = 1, dtype: str = "float32") -> StackConfig:
    """`config.json` (as a dict) -> StackConfig.  `shapes`: tensor name -> shape, for the sizes only tensors state;
    without it the mixer entries may carry `rank_decay` / `rank_gate` (random-weight benches)."""
    layers = []
    for i, lc in enumerate(config["layers"]):
        kind = lc["type"]
        if kind not in _MIXERS:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mc = lc["mixer"]
        mlp = lc.get("mlp")
        if mlp is not None and mlp.get("kind", "dense") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        spec = LayerSpec(mixer=_MIXERS[kind], heads=int(mc["heads"]), dim=int(mc["dim"]), vdim=int(mc.get("vdim", mc["dim"])),
                         kv_heads=int(mc.get("kv_heads", mc["heads"])), ff=int(mlp["ff"]) if mlp is not None else 0)
        if kind == "attention":
            spec.scale = float(mc["scale"])
        elif kind == "lightning":
            d = mc["decay"]  # one value per head; a single number serves every head
            spec.decay = [float(x) for x in d] if isinstance(d, (list, tuple)) else [float(d)] * spec.heads
            if len(spec.decay) != spec.heads:
                raise ValueError(f"layer {i}: {len(spec.decay)} decays for {spec.heads} heads")
        else:
            spec.conv_taps = int(mc["conv"])
            if shapes is not None:
                spec.rank_decay = int(shapes[f"l{i}.mix.a1"][0])
                spec.rank_gate = int(shapes[f"l{i}.mix.g1"][0])
            else:
                spec.rank_decay = int(mc.get("rank_decay", max(8, config["width"] // 8)))
                spec.rank_gate = int(mc.get("rank_gate", max(8, config["width"] // 8)))
        layers.append(spec)
    side = config.get("token_side") or {}
    return StackConfig(width=int(config["width"]), vocab=int(config["vocab"]), layers=layers,
                       norm_eps=float(config["norm"]["eps"]), residual_mult=float(config["residual_mult"]),
                       norm_one_plus=True, glu_act="gelu_tanh", side_dim=int(side.get("dim", 0)),
                       max_seq_len=max_seq_len, max_batch_size=max_batch_size, dtype=dtype)


class Risalix(StackDecoder):
    architecture = "Risalix"

    def __init__(self, config: Mapping, tensors: Optional[Mapping[str, np.ndarray]] = None, *, max_seq_len: int = 256,
                 max_batch_size: int = 1, dtype: str = "float32", device: int = 0, random_seed: Optional[int] = None,
                 flags: int = 0):
        """`tensors`: checkpoint name -> array; or None with `random_seed` for random weights on the device."""
        if tensors is None and random_seed is None:
            raise ValueError("tensors=None needs random_seed")
        shapes = {k: tuple(np.shape(tensors[k])) for k in tensors.keys()} if tensors is not None else None
        self.config = dict(config)
        super().__init__(stack_config(config, shapes, max_seq_len=max_seq_len, max_batch_size=max_batch_size, dtype=dtype),
                         device=device, flags=flags)
        if tensors is not None:
            self.load_tensors(tensors)
        else:
            self.fill_random(random_seed)

    @classmethod
    def from_pretrained(cls, model_dir, **kw) -> "Risalix":
        with open(os.path.join(model_dir, "config.json")) as f:
            config = json.load(f)
        return cls(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), **kw)
