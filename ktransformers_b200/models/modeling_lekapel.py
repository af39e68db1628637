"""Lekapel — a decoder whose layers run their mixer and their feed-forward in parallel off ONE grouped RMS norm,

    h = norm(x) ;  x <- x + m * (mixer(shift(h)) + ff(h))

with a token shift in front of the mixer, latent attention with a sliding window, a soft-max sink and an output gate as the
mixer, and either a PolyNorm feed-forward or a soft-max top-k mixture of gated-SiLU experts (or none) as the feed-forward.
The layer list, every size and every constant come from `LekapelConfig`.

The model is assembled from the framework's operators (operators/norm.py, attention.py, mlp.py, experts.py, gate.py); its
`forward(batch, cache)` is the step function the engine drives: a flattened ragged batch of prompt portions and decode
tokens (models/custom_cache.ForwardBatch) against the paged cache and state rows of models/custom_cache.PagedStateCache.
The residual stream is fp32; the sum `x + m * (a + b)` of a layer is folded into the next norm launch."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..operators.attention import KLatentWindowAttention
from ..operators.experts import KSoftmaxTopKMoE
from ..operators.mlp import KPolyNormMLP
from ..operators.norm import KGroupRMSNormShift
from .configuration_lekapel import LekapelConfig
from .custom_cache import ForwardBatch, PagedStateCache

MIXERS = {"latent_attention": KLatentWindowAttention}


class LekapelDecoderLayer(nn.Module):
    def __init__(self, config: LekapelConfig, layer_idx: int, dtype, device):
        super().__init__()
        spec = config.layers[layer_idx]
        self.layer_idx = layer_idx
        self.norm1 = KGroupRMSNormShift(config.width, config.norm_groups, config.norm_eps, shift=True, dtype=dtype, device=device)
        self.mix = MIXERS[spec.type](config.width, spec.mixer, config.norm_eps, layer_idx, dtype=dtype, device=device)
        if spec.mlp is None:
            self.mlp = None
        elif spec.mlp.kind == "dense":
            self.mlp = KPolyNormMLP(config.width, spec.mlp.ff, config.norm_eps, dtype=dtype, device=device)
        else:
            self.mlp = KSoftmaxTopKMoE(config.width, spec.mlp.ff, spec.mlp.experts, spec.mlp.top, dtype=dtype, device=device)

    def load(self, loader, prefix: str):
        self.norm1.load(loader, prefix + "norm1", prefix + "shift")
        self.mix.load(loader, prefix + "mix.")
        if self.mlp is not None:
            self.mlp.load(loader, prefix + "mlp.")


class LekapelForCausalLM(nn.Module):
    config_class = LekapelConfig

    def __init__(self, config: LekapelConfig, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        self.config, self.dtype, self.device = config, dtype, torch.device(device)
        self.embed = nn.Parameter(torch.empty((config.vocab, config.width), dtype=dtype, device=device), requires_grad=False)
        self.layers = nn.ModuleList([LekapelDecoderLayer(config, i, dtype, device) for i in range(len(config.layers))])
        self.final_norm = KGroupRMSNormShift(config.width, config.norm_groups, config.norm_eps, shift=False, dtype=dtype, device=device)
        self.head = nn.Parameter(torch.empty((config.vocab, config.width), dtype=dtype, device=device), requires_grad=False)

    def load(self, loader):
        self.embed.data.copy_(loader.load_tensor("embed", "cpu"))
        for i, layer in enumerate(self.layers):
            layer.load(loader, f"l{i}.")
        self.final_norm.load(loader, "final.norm")
        self.head.data.copy_(loader.load_tensor("head", "cpu"))

    def make_cache(self, max_tokens: int, max_slots: int = 8, page_size: int = 64) -> PagedStateCache:
        c = self.config
        return PagedStateCache(c.cache_row_widths(), c.width, max_tokens, max_slots, self.device, dtype=self.dtype, page_size=page_size, window=c.max_window())

    def decode_is_capturable(self, max_batch: int = 47) -> bool:
        """Whether a decode step of up to `max_batch` sequences makes no host read (then the engine may replay it as a CUDA
        graph): the experts' small-batch kernels never do; experts whose rows are too long for them do, unless the library's
        grouped GEMM applies."""
        for layer in self.layers:
            e = getattr(layer.mlp, "experts", None)
            if e is not None and not e.small_batches_stay_on_device(layer.mlp.router.top, self.dtype, max_batch):
                return False
        return True

    @torch.no_grad()
    def forward(self, batch: ForwardBatch, cache: PagedStateCache, residual_trace: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        """Runs the batch's tokens from the cache and state earlier steps left; returns fp32 logits [len(batch.want), vocab]."""
        m = self.config.residual_mult
        x = self.embed.index_select(0, batch.tokens).float()
        a = b = None
        for layer in self.layers:
            x, h, hs = layer.norm1(x, a, b, m, batch, cache.state[layer.layer_idx], want_h=layer.mlp is not None)
            if residual_trace is not None and a is not None:
                residual_trace.append(x.clone())
            a = layer.mix(hs, batch, cache)
            b = layer.mlp(h) if layer.mlp is not None else None
        x, h, _ = self.final_norm(x, a, b, m)
        if residual_trace is not None:
            residual_trace.append(x.clone())
        return F.linear(h.index_select(0, batch.want), self.head).float() * self.config.logit_scale
