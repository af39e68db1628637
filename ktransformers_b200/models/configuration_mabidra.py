"""Configuration of the Mabidra decoder family: a list of layers, each a mixer ("attention": sigmoid attention with a learned
distance bias, or "gla": gated linear attention with a recurrent state) and a feed-forward (xIELU dense, relu-squared mixture
of experts, or none); a span of layers that runs several times in a row with the same weights and separate caches; grouped
RMS norms on both sides of every sublayer.  Every size and constant is read from the checkpoint's `config.json` (or from a
tensor's shape at load time); nothing is assumed equal between layers."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional, Tuple


@dataclass
class SigmoidAttentionSpec:
    heads: int
    kv_heads: int
    dim: int                       # query / key size per head
    vdim: int
    scale: float                   # multiplies q . k (not the distance bias)
    bias_max: float                # distance from which the last row of the bias table applies
    temp_coef: float               # query temperature 1 + coef * ln(floor((pos + 1) / every) + 1)
    temp_every: int

    @classmethod
    def from_dict(cls, d: dict) -> "SigmoidAttentionSpec":
        heads = int(d["heads"])
        temp = d.get("q_temp") or {}
        return cls(heads=heads, kv_heads=int(d.get("kv_heads", heads)), dim=int(d["dim"]), vdim=int(d.get("vdim", d["dim"])),
                   scale=float(d.get("scale", int(d["dim"]) ** -0.5)), bias_max=float(d["bias_max"]), temp_coef=float(temp.get("coef", 0.0)),
                   temp_every=int(temp.get("every", 1)))

    def cache_row_width(self) -> int:
        return self.kv_heads * (self.dim + self.vdim)

    def state_width(self) -> int:
        return 0


@dataclass
class GatedLinearAttentionSpec:
    heads: int
    dim: int                       # key channels per head (the decay is per key channel)
    vdim: int
    tau: float                     # decay = sigmoid(z) ** (1 / tau)

    @classmethod
    def from_dict(cls, d: dict) -> "GatedLinearAttentionSpec":
        return cls(heads=int(d["heads"]), dim=int(d["dim"]), vdim=int(d.get("vdim", d["dim"])), tau=float(d["tau"]))

    def cache_row_width(self) -> int:
        return 0

    def state_width(self) -> int:
        return self.heads * self.dim * self.vdim


@dataclass
class MlpSpec:
    kind: str                      # "dense" (xIELU) or "moe" (top-k router, soft-max over the chosen logits, relu-squared experts)
    ff: int
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> Optional["MlpSpec"]:
        if d is None:
            return None
        if d["kind"] == "dense":
            return cls("dense", int(d["ff"]))
        if d["kind"] == "moe":
            return cls("moe", int(d["expert"]["ff"]), int(d["router"]["experts"]), int(d["router"]["top"]))
        raise ValueError(f"unknown feed-forward kind {d['kind']!r}")


@dataclass
class LayerSpec:
    type: str
    mixer: object
    mlp: Optional[MlpSpec]


@dataclass
class LoopSpec:
    start: int
    stop: int
    times: int


MIXER_SPECS = {"attention": SigmoidAttentionSpec, "gla": GatedLinearAttentionSpec}


@dataclass
class MabidraConfig:
    architecture: str = "Mabidra"
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    norm_groups: int = 1
    embedding_scale: float = 1.0
    layers: List[LayerSpec] = field(default_factory=list)
    loop: Optional[LoopSpec] = None

    @classmethod
    def from_dict(cls, d: dict) -> "MabidraConfig":
        layers = []
        for i, l in enumerate(d["layers"]):
            if l["type"] not in MIXER_SPECS:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            layers.append(LayerSpec(l["type"], MIXER_SPECS[l["type"]].from_dict(l["mixer"]), MlpSpec.from_dict(l.get("mlp"))))
        norm = d.get("norm") or {}
        loop = d.get("loop")
        if loop is not None:
            loop = LoopSpec(int(loop["start"]), int(loop["stop"]), int(loop["times"]))
            if not (0 <= loop.start < loop.stop <= len(layers)) or loop.times < 1:
                raise ValueError(f"loop {loop} does not fit {len(layers)} layers")
        return cls(architecture=d.get("architecture", "Mabidra"), vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(norm.get("eps", 1e-5)),
                   norm_groups=int(norm.get("groups", 1)), embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)), layers=layers, loop=loop)

    @classmethod
    def from_pretrained(cls, path: str) -> "MabidraConfig":
        with open(os.path.join(path, "config.json") if os.path.isdir(path) else path) as f:
            return cls.from_dict(json.load(f))

    def layer_runs(self) -> List[Tuple[int, Optional[int]]]:
        """The order in which layers run: (layer index, number of the pass that this run OPENS or None).  A looped span
        contributes `times` runs of each of its layers; every run has a cache layer of its own."""
        n, lp = len(self.layers), self.loop
        if lp is None:
            return [(i, None) for i in range(n)]
        runs = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            runs += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return runs + [(i, None) for i in range(lp.stop, n)]

    # what the cache manager asks of a model
    @property
    def num_hidden_layers(self) -> int:
        return len(self.layer_runs())

    def cache_row_widths(self) -> List[int]:
        return [self.layers[i].mixer.cache_row_width() for i, _ in self.layer_runs()]

    def state_widths(self) -> List[int]:
        return [self.layers[i].mixer.state_width() for i, _ in self.layer_runs()]

    def max_window(self) -> Optional[int]:
        """No layer of this family forgets keys: attention layers see every earlier position."""
        return None
