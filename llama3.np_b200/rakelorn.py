"""Rakelorn: a pre-norm decoder whose layers mix tokens either by latent attention - one cached row per token
(a normed latent and a rotated key part shared by all heads), queries through a latent of their own, rotary
pairs (2i, 2i + 1), a sigmoid gate per head - or by minGRU, an element-wise gated recurrence; every layer
norm is a single number, the mixer reads its input mixed with the previous token's (token shift), the
feed-forward is a mixture of relu^2 experts with identity slots, a score correction and group-limited
choice, and a block of layers may run several times with one set of weights, each pass with its own
caches and a step vector added ahead of it.  The arithmetic lives in the library's layer-list path
(csrc/layerlist.cu, attn_latent.cu, prenorm_ops.cu, moe.cu); this file reads `config.json`, names the
tensors and builds the `StackConfig`.

A checkpoint folder holds `config.json` (keys: architecture, vocab, width, embedding.scale, norm.eps,
loop.start / stop / times, layers[].type / mixer / mlp) and `model.safetensors` (tensor names `embed`,
`loop.step`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.shift`, `l<i>.mix.*`, `l<i>.mlp.e<k>.up / down`,
`l<i>.mlp.router`, `l<i>.mlp.correction`, `final.norm`, `head`).
"""
from __future__ import annotations

import json
import os
from typing import Mapping, Optional

import numpy as np

from .stack import LATENT, MINGRU, LayerSpec, StackConfig, StackDecoder
from .utils import read_safetensors


def stack_config(config: Mapping, *, max_seq_len: int = 256, max_batch_size: int = 1, dtype: str = "float32") -> StackConfig:
    """`config.json` (as a dict) -> StackConfig."""
    layers = []
    for i, lc in enumerate(config["layers"]):
        kind, mc = lc["type"], lc["mixer"]
        if kind == "latent_attention":
            rot = mc.get("rot") or {}
            rot_dim = int(mc.get("rot_dim", 0))
            spec = LayerSpec(mixer=LATENT, heads=int(mc["heads"]), dim=int(mc["dim"]), vdim=int(mc["vdim"]),
                             q_rank=int(mc["q_rank"]), kv_rank=int(mc["kv_rank"]), rot_dim=rot_dim,
                             rot_dims=int(rot.get("dims", rot_dim)), rot_base=float(rot.get("base", 10000.0)),
                             scale=float(mc["scale"]))
        elif kind == "mingru":
            spec = LayerSpec(mixer=MINGRU, heads=1, dim=int(mc["width"]), vdim=1)
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = lc.get("mlp")
        if mlp is not None:
            if mlp.get("kind", "moe") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            rc = mlp["router"]
            groups = rc.get("groups") or {}
            spec.ff = int(mlp["expert"]["ff"])
            spec.experts = int(rc["experts"])
            spec.top = int(rc["top"])
            spec.identity = int(rc.get("identity", 0))
            spec.groups = int(groups.get("count", 1))
            spec.groups_keep = int(groups.get("keep", spec.groups))
            spec.router_scale = float(rc.get("scale", 1.0))
        layers.append(spec)
    lp = config.get("loop")
    loop = (int(lp["start"]), int(lp["stop"]), int(lp["times"])) if lp else None
    return StackConfig(width=int(config["width"]), vocab=int(config["vocab"]), layers=layers,
                       norm_eps=float(config["norm"]["eps"]), norm_one_plus=False, norm_input=True, norm_scalar=True,
                       token_shift=True, embed_scale=float((config.get("embedding") or {}).get("scale", 1.0)), loop=loop,
                       max_seq_len=max_seq_len, max_batch_size=max_batch_size, dtype=dtype)


class Rakelorn(StackDecoder):
    architecture = "Rakelorn"

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
    def from_pretrained(cls, model_dir, **kw) -> "Rakelorn":
        with open(os.path.join(model_dir, "config.json")) as f:
            config = json.load(f)
        return cls(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), **kw)
