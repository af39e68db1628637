"""Mabidra — a decoder whose layers norm both sides of every sublayer,

    x <- x + norm1b(mixer(norm1(x))) ;  x <- x + norm2b(ff(norm2(x)))          (grouped RMS norms, fp32 residual stream)

with sigmoid attention under a learned distance bias or gated linear attention as the mixer, an xIELU feed-forward or a
relu-squared mixture of experts (or none) as the feed-forward, and a span of layers that runs several times in a row with the
same weights: each pass opens with x <- W_in [x ; x0] + step[pass] (x0: the scaled embedding) and keeps caches and states of
its own.  The layer list, the span, every size and every constant come from `MabidraConfig`.

The model is assembled from the framework's operators (operators/norm.py, attention.py, linear_attention.py, mlp.py,
experts.py, gate.py); its `forward(batch, cache)` is the step function the engine drives: a flattened ragged batch of prompt
portions and decode tokens (models/custom_cache.ForwardBatch) against the paged cache rows and per-sequence state rows of
models/custom_cache.PagedStateCache, one cache layer per layer RUN.  Every residual sum is folded into a norm launch: a
sublayer's output is normed, added, and the next sublayer's input normed in one kernel."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..operators.attention import KSigmoidBiasAttention
from ..operators.experts import KTopKSoftmaxMoE
from ..operators.linear_attention import KGatedLinearAttention
from ..operators.mlp import KXIELUMLP
from ..operators.norm import KGroupRMSNorm
from .configuration_mabidra import MabidraConfig
from .custom_cache import ForwardBatch, PagedStateCache

MIXERS = {"attention": KSigmoidBiasAttention, "gla": KGatedLinearAttention}


class MabidraDecoderLayer(nn.Module):
    def __init__(self, config: MabidraConfig, layer_idx: int, dtype, device):
        super().__init__()
        spec = config.layers[layer_idx]
        norm = lambda: KGroupRMSNorm(config.width, config.norm_groups, config.norm_eps, dtype=dtype, device=device)
        self.layer_idx = layer_idx
        self.norm1, self.norm1b = norm(), norm()
        self.mix = MIXERS[spec.type](config.width, spec.mixer, config.norm_eps, dtype=dtype, device=device)
        if spec.mlp is None:
            self.mlp = self.norm2 = self.norm2b = None
        else:
            self.norm2, self.norm2b = norm(), norm()
            if spec.mlp.kind == "dense":
                self.mlp = KXIELUMLP(config.width, spec.mlp.ff, dtype=dtype, device=device)
            else:
                self.mlp = KTopKSoftmaxMoE(config.width, spec.mlp.ff, spec.mlp.experts, spec.mlp.top, dtype=dtype, device=device)

    def load(self, loader, prefix: str):
        for name in ("norm1", "norm1b") + (("norm2", "norm2b") if self.mlp is not None else ()):
            getattr(self, name).load(loader, prefix + name)
        self.mix.load(loader, prefix + "mix.")
        if self.mlp is not None:
            self.mlp.load(loader, prefix + "mlp.")


class MabidraForCausalLM(nn.Module):
    config_class = MabidraConfig

    def __init__(self, config: MabidraConfig, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        self.config, self.dtype, self.device = config, dtype, torch.device(device)
        P = lambda *shape, dt=dtype: nn.Parameter(torch.empty(shape, dtype=dt, device=device), requires_grad=False)
        self.embed = P(config.vocab, config.width)
        self.layers = nn.ModuleList([MabidraDecoderLayer(config, i, dtype, device) for i in range(len(config.layers))])
        self.runs = config.layer_runs()
        if config.loop is not None:
            self.loop_in = P(config.width, 2 * config.width)
            self.loop_step = P(config.loop.times, config.width, dt=torch.float32)
        self.final_norm = KGroupRMSNorm(config.width, config.norm_groups, config.norm_eps, dtype=dtype, device=device)
        self.head = P(config.vocab, config.width)

    def load(self, loader):
        self.embed.data.copy_(loader.load_tensor("embed", "cpu"))
        for i, layer in enumerate(self.layers):
            layer.load(loader, f"l{i}.")
        if self.config.loop is not None:
            self.loop_in.data.copy_(loader.load_tensor("loop.in", "cpu"))
            self.loop_step.data.copy_(loader.load_tensor("loop.step", "cpu").float())
        self.final_norm.load(loader, "final.norm")
        self.head.data.copy_(loader.load_tensor("head", "cpu"))

    def make_cache(self, max_tokens: int, max_slots: int = 8, page_size: int = 64) -> PagedStateCache:
        c = self.config
        return PagedStateCache(c.cache_row_widths(), c.state_widths(), max_tokens, max_slots, self.device, dtype=self.dtype, page_size=page_size, window=None)

    def decode_is_capturable(self, max_batch: int = 47) -> bool:
        """Whether a decode step of up to `max_batch` sequences makes no host read (then the engine may replay it as a CUDA
        graph)."""
        for layer in self.layers:
            e = getattr(layer.mlp, "experts", None)
            if e is not None and not e.small_batches_stay_on_device(layer.mlp.router.top, self.dtype, max_batch):
                return False
        return True

    @torch.no_grad()
    def forward(self, batch: ForwardBatch, cache: PagedStateCache, residual_trace: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        """Runs the batch's tokens from the cache and state earlier steps left; returns fp32 logits [len(batch.want), vocab]."""
        x0 = self.embed.index_select(0, batch.tokens).float() * self.config.embedding_scale
        # (x, y, post): the residual before the pending sublayer output y, whose norm `post` has not been applied yet
        x, y, post = None, x0, None
        for run, (i, opens_pass) in enumerate(self.runs):
            layer = self.layers[i]
            if opens_pass is not None:
                if post is not None or x is not None:
                    x, _ = KGroupRMSNorm.fused(x, y, post, None)
                else:
                    x = y
                y = F.linear(torch.cat([x, x0], -1).to(self.dtype), self.loop_in)
                x, h = KGroupRMSNorm.fused(None, y, None, layer.norm1, row_add=self.loop_step[opens_pass])
            else:
                x, h = KGroupRMSNorm.fused(x, y, post, layer.norm1)
            y, post = layer.mix(h, batch, cache, run), layer.norm1b
            if layer.mlp is not None:
                x, h = KGroupRMSNorm.fused(x, y, post, layer.norm2)
                y, post = layer.mlp(h), layer.norm2b
            if residual_trace is not None:
                residual_trace.append(KGroupRMSNorm.fused(x, y, post, None)[0])
        want_rows = batch.want
        if x is not None:
            x = x.index_select(0, want_rows)
        _, h = KGroupRMSNorm.fused(x, y.index_select(0, want_rows), post, self.final_norm, keep_x=False)
        return F.linear(h, self.head).float()
