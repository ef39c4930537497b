"""Residual stack of PoM layers with a GELU feed-forward block, run frame by frame with the layers'
running-mean state — the block-causal video pattern of the reference's README (README.md:28-35, 48-61):

    for each frame:  for each layer:  x = x + pom.state_forward(x, x, state[l]);  x = x + W2·gelu(W1·x)

This is inference plumbing around ``PoM.state_forward`` (no autograd through the feed-forward block): the two
feed-forward products run on the tcgen05 GEMM with the GELU and the residual add fused into its epilogue,
and a whole multi-frame pass can be captured once into a CUDA graph and replayed, which removes the
per-launch host latency that dominates at a few hundred tokens per frame.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from . import ops
from .functional import BlockCausal, eager_only, on_tensor_device
from .pom import PoM


class PoMStack(nn.Module):
    """``n_layers`` x (PoM + 4·D GELU feed-forward), no normalisation layers, bf16 inference."""

    def __init__(self, dim: int, degree: int, expand: int, n_layers: int, ffn_mult: int = 4, n_sel_heads: int = 1):
        super().__init__()
        self.dim = dim
        self.mixers = nn.ModuleList([PoM(dim, degree, expand, 1, n_sel_heads) for _ in range(n_layers)])
        self.ffn_in = nn.ModuleList([nn.Linear(dim, ffn_mult * dim, bias=False) for _ in range(n_layers)])
        self.ffn_out = nn.ModuleList([nn.Linear(ffn_mult * dim, dim, bias=False) for _ in range(n_layers)])

    @eager_only
    @on_tensor_device
    @torch.no_grad()
    def frame_forward(self, x: torch.Tensor, states: Optional[List[Optional[dict]]] = None):
        """One frame (B, L, D) bf16 through all layers; ``states`` is the per-layer list returned by the
        previous frame (None for the first).  Returns (output, new states)."""
        if x.dtype != torch.bfloat16 or not x.is_cuda:
            raise TypeError("PoMStack runs on CUDA bfloat16 tensors")
        B, L, D = x.shape
        states = list(states) if states is not None else [None] * len(self.mixers)
        h = x.contiguous()
        for i, mixer in enumerate(self.mixers):
            y, states[i] = mixer.state_forward(h, None, states[i], residual=h)  # x + mixer(x), add fused
            h2 = y.view(B * L, D)
            u = ops.gemm(h2, self.ffn_in[i].weight, act="gelu")
            h = ops.gemm(u, self.ffn_out[i].weight, residual=h2).view(B, L, D)
        return h, states

    @eager_only
    @on_tensor_device
    @torch.no_grad()
    def forward_single_pass(self, x: torch.Tensor, frame_len: int) -> torch.Tensor:
        """Same result as :meth:`forward`, all frames at once: each mixer runs with ``BlockCausal(frame_len)``, so
        every GEMM sees the whole (B·N)-row batch instead of one frame's rows."""
        if x.dtype != torch.bfloat16 or not x.is_cuda:
            raise TypeError("PoMStack runs on CUDA bfloat16 tensors")
        B, N, D = x.shape
        mask = BlockCausal(frame_len)
        h = x.contiguous()
        for i, mixer in enumerate(self.mixers):
            y = mixer(h, None, mask, residual=h)
            h2 = y.view(B * N, D)
            u = ops.gemm(h2, self.ffn_in[i].weight, act="gelu")
            h = ops.gemm(u, self.ffn_out[i].weight, residual=h2).view(B, N, D)
        return h

    @eager_only
    @on_tensor_device
    @torch.no_grad()
    def forward(self, x: torch.Tensor, frame_len: int) -> torch.Tensor:
        """Full sequence (B, F·frame_len, D), processed frame by frame with state carried across frames."""
        outs, states = [], None
        for f in range(x.shape[1] // frame_len):
            y, states = self.frame_forward(x[:, f * frame_len:(f + 1) * frame_len], states)
            outs.append(y)
        return torch.cat(outs, dim=1)

