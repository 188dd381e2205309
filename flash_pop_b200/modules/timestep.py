"""Sinusoidal timestep embedding + MLP for diffusion conditioning (flash_pop/modules/timestep.py:18-56)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn


class TimestepEmbedder(nn.Module):
    """Embeds (possibly fractional) scalar timesteps of any shape (B, [T], [tokens]) into vectors."""

    def __init__(self, hidden_size, frequency_embedding_size=256, device=None, dtype=None):
        super().__init__()
        kw = dict(bias=True, device=device, dtype=dtype)
        self.mlp = nn.Sequential(nn.Linear(frequency_embedding_size, hidden_size, **kw), nn.SiLU(),
                                 nn.Linear(hidden_size, hidden_size, **kw))
        self.frequency_embedding_size = frequency_embedding_size

    @staticmethod
    def timestep_embedding(t, dim, max_period=10000):
        """[cos(t f_0..f_{h-1}), sin(t f_0..f_{h-1})] with f_i = max_period^(-i/h), h = dim // 2."""
        half = dim // 2
        freqs = torch.exp(torch.arange(half, dtype=torch.float32, device=t.device) * (-math.log(max_period) / half))
        angles = t.reshape(-1, 1).float() * freqs
        emb = torch.cat((angles.cos(), angles.sin()), dim=-1)
        if dim % 2:
            emb = torch.nn.functional.pad(emb, (0, 1))
        return emb.reshape(*t.shape, dim)

    def forward(self, t):
        return self.mlp(self.timestep_embedding(t, self.frequency_embedding_size).to(dtype=t.dtype))
