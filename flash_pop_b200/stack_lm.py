"""A token-level language-model wrapper around ``RetNetDecoder``: embedding -> decoder stack -> LayerNorm -> vocabulary
head.  The reference has no such wrapper (its decoders consume embeddings, tests/test_retention_layer.py:97-101);
this is the harness for the full-stack training configuration (12 layers, d_model 1024, 8 heads of 128, FFN 4096,
vocabulary 32000) and for users who want the same."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from flash_pop_b200.layer_ops import norm_in_fp32
from flash_pop_b200.recurrent_state import RecurrentState
from flash_pop_b200.retnet import RetNetDecoder, RetNetDecoderLayer


class RetNetLM(nn.Module):
    def __init__(self, vocab_size: int = 32000, num_layers: int = 12, num_heads: int = 8, head_dim: int = 128,
                 dim_feedforward: int = 4096, dropout: float = 0.0, device="cuda", dtype=torch.bfloat16):
        super().__init__()
        d_model = num_heads * head_dim
        cfg = RetNetDecoderLayer.Config(num_heads=num_heads, head_dim_v=head_dim, head_dim_qk=head_dim,
                                        dim_feedforward=dim_feedforward, dropout=dropout, device=device, dtype=dtype)
        self.embed = nn.Embedding(vocab_size, d_model, device=device, dtype=dtype)
        self.decoder = RetNetDecoder(cfg, num_layers)
        self.norm = nn.LayerNorm(d_model, device=device, dtype=torch.float32)
        self.head = nn.Linear(d_model, vocab_size, bias=False, device=device, dtype=dtype)
        nn.init.normal_(self.embed.weight, std=d_model ** -0.5)
        nn.init.normal_(self.head.weight, std=d_model ** -0.5)

    def forward(self, tokens: torch.Tensor, recurrent_state: Optional[RecurrentState] = None):
        """tokens: (B, T) int64 -> logits (B, T, vocab), new RecurrentState."""
        x, state = self.decoder(self.embed(tokens), recurrent_state)
        return self.head(norm_in_fp32(self.norm, x)), state

    def loss(self, tokens: torch.Tensor) -> torch.Tensor:
        """Next-token cross entropy of `tokens` (B, T)."""
        logits, _ = self(tokens[:, :-1])
        return F.cross_entropy(logits.float().flatten(0, 1), tokens[:, 1:].flatten())

    def flops_per_token(self, seq_len: int) -> float:
        """Training (forward + backward) FLOPs per token: 6 x matmul parameters + the retention operator."""
        layer = self.decoder.layers[0]
        d = layer.retention.embed_dim
        per_layer = 5 * d * d + 2 * d * layer.linear1.out_features
        matmul = len(self.decoder.layers) * per_layer + d * self.head.out_features
        H, dk, dv = layer.retention.num_heads, layer.retention.head_dim_qk, layer.retention.head_dim_v
        ch = 32.5
        retention = len(self.decoder.layers) * H * ((2 * ch * (dk + dv) + 4 * dk * dv) + (2 * ch * (3 * dk + 2 * dv) + 8 * dk * dv))
        return 6.0 * matmul + retention
