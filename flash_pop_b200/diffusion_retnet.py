"""Diffusion RetNet (DiT-style): RetNet layers whose norms are AdaLN-Zero blocks driven by a conditioning
signal.  Names, ``Config`` fields and arithmetic follow the reference (flash_pop/diffusion_retnet.py:27-286);
the retention inside is the B200 operator through ``MultiScaleRetention``.  Unlike the reference, the
recurrent walk takes the conditioning it needs (the reference's drops it, diffusion_retnet.py:236-246)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple, Union

import torch
import torch.nn as nn
from torch import Tensor

from flash_pop_b200.modules.adaln import AdaLayerNorm, AdaLayerNormZero, _to_tokens, gated_residual
from flash_pop_b200.recurrent_state import RecurrentState
from flash_pop_b200.retnet import ActivationString, MultiScaleRetention, RetNetDecoder, _get_activation_fn
from flash_pop_b200.xpos_emb import XPos


class DiffusionRetNetDecoderLayer(nn.Module):
    @dataclass(kw_only=True)
    class Config:
        num_heads: int
        head_dim_v: int
        head_dim_qk: int = None
        dim_feedforward: int = 2048
        dropout: float = 0.1
        use_post_retention_dropout: bool = True
        head_decays_range: tuple[float, float] = None
        activation: Union[ActivationString, Callable[[Tensor], Tensor]] = "swish"
        layer_norm_eps: float = 1e-6
        ada_ln_lora_dim: Optional[int] = None
        device: Optional[Union[torch.device, str]] = torch.device("cuda")
        dtype: Optional[torch.dtype] = torch.bfloat16
        use_fused_version: bool = True
        chunk_size: int = 512  # accepted for compatibility; unused

    def __init__(self, config: Config, xpos_embedder: Optional[XPos] = None) -> None:
        super().__init__()
        self.config = config
        self.activation = _get_activation_fn(config.activation) if isinstance(config.activation, str) else config.activation
        self.dropout = nn.Dropout(config.dropout)
        self.use_post_retention_dropout = config.use_post_retention_dropout
        d_model = config.num_heads * config.head_dim_v
        ada = dict(eps=config.layer_norm_eps, lora_hidden_dim=config.ada_ln_lora_dim, device=config.device, dtype=config.dtype)
        self.ada_ln1 = AdaLayerNormZero(d_model, **ada)
        self.retention = self._build_multi_scale_retention(xpos_embedder=xpos_embedder)
        self.ada_ln2 = AdaLayerNormZero(d_model, **ada)
        self.linear1 = nn.Linear(d_model, config.dim_feedforward, device=config.device, dtype=config.dtype)
        self.linear2 = nn.Linear(config.dim_feedforward, d_model, device=config.device, dtype=config.dtype)
        self._reset_parameters()

    def _build_multi_scale_retention(self, xpos_embedder: Optional[XPos] = None):
        c = self.config
        return MultiScaleRetention(MultiScaleRetention.Config(
            num_heads=c.num_heads, head_dim_v=c.head_dim_v, head_dim_qk=c.head_dim_qk, dropout=c.dropout,
            head_decays_range=c.head_decays_range, activation=self.activation, device=c.device, dtype=c.dtype,
            use_fused_version=c.use_fused_version, chunk_size=c.chunk_size), xpos_embedder=xpos_embedder)

    def _reset_parameters(self):
        for lin in (self.linear1, self.linear2):
            nn.init.xavier_normal_(lin.weight)
            nn.init.constant_(lin.bias, 0)

    def _feedforward_block(self, x: Tensor) -> Tensor:
        x = self.dropout(self.activation(self.linear1(x)))
        return self.dropout(self.linear2(x))

    def _blocks(self, x: Tensor, c: Tensor, retention_fn) -> Tuple[Tensor, Tensor]:
        # the gates stay (B, Tm, D) rows of the modulation MLP's output; norm + modulation and gate + residual are one
        # kernel each (flash_pop_b200.layer_ops)
        x, gate = self.ada_ln1.forward_rows(x, c)
        y, state = retention_fn(x)
        if self.use_post_retention_dropout and self.training and self.dropout.p > 0:
            x = x + self.dropout(y * _to_tokens(gate, x.size(1)))
        else:
            x = gated_residual(x, y, gate)
        x, gate = self.ada_ln2.forward_rows(x, c)
        return gated_residual(x, self._feedforward_block(x), gate), state

    def forward_chunkwise(self, x: Tensor, c: Tensor, start_idx: int, prev_state: Optional[Tensor] = None):
        return self._blocks(x, c, lambda h: self.retention.forward_chunkwise(h, start_idx=start_idx, prev_state=prev_state))

    def forward_recurrent(self, x: Tensor, c: Tensor, seq_idx: int, prev_state: Optional[Tensor] = None):
        """x: (B, D) one token per row; c: (B, D)."""
        def step(h):
            y, state = self.retention.forward_recurrent(h.squeeze(1), seq_idx=seq_idx, prev_state=prev_state)
            return y.unsqueeze(1), state
        out, state = self._blocks(x.unsqueeze(1), c, step)
        return out.squeeze(1), state

    def forward(self, x: Tensor, c: Tensor, start_idx: int = 0, prev_state: Optional[Tensor] = None):
        return self.forward_chunkwise(x, c, start_idx=start_idx, prev_state=prev_state)


class DiffusionRetNetFinalLayer(nn.Module):
    @dataclass(kw_only=True)
    class Config:
        layer_config: DiffusionRetNetDecoderLayer.Config
        out_dim: int

    def __init__(self, config: Config):
        super().__init__()
        lc = config.layer_config
        d_model = lc.head_dim_v * lc.num_heads
        self.final_ada_ln = AdaLayerNorm(d_model, eps=lc.layer_norm_eps, lora_hidden_dim=lc.ada_ln_lora_dim,
                                         device=lc.device, dtype=lc.dtype)
        self.final_linear = nn.Linear(d_model, config.out_dim, device=lc.device, dtype=lc.dtype)

    def forward(self, x: Tensor, c: Tensor):
        return self.final_linear(self.final_ada_ln(x, c))


class DiffusionRetNetDecoder(nn.Module):
    """The stack without its final layer (AdaLN + Linear), which the user adds per output modality."""

    @dataclass(kw_only=True)
    class Config:
        layer_config: DiffusionRetNetDecoderLayer.Config
        num_layers: int

    def __init__(self, config: Config):
        super().__init__()
        lc = config.layer_config
        if lc.head_dim_qk is None:
            lc.head_dim_qk = lc.head_dim_v
        self.layer_config = lc
        self.num_layers = config.num_layers
        self.xpos_embedder = XPos(lc.head_dim_qk, device=lc.device, dtype=lc.dtype)
        self.layers = nn.ModuleList(self._build_layers(config.num_layers))

    def _build_layers(self, num_layers: int):
        return [DiffusionRetNetDecoderLayer(self.layer_config, self.xpos_embedder) for _ in range(num_layers)]

    _validate_and_init_state = RetNetDecoder._validate_and_init_state

    def _walk(self, x, recurrent_state, step, advance):
        rs = self._validate_and_init_state(recurrent_state)
        states: List[Tensor] = []
        for layer, state_i in zip(self.layers, rs.state):
            x, state = step(layer, x, rs.index, state_i)
            states.append(state)
        return x, RecurrentState(torch.stack(states), rs.index + advance)

    def forward_recurrent(self, x: Tensor, c: Tensor, recurrent_state: RecurrentState = None):
        return self._walk(x, recurrent_state, lambda layer, h, idx, st: layer.forward_recurrent(h, c, idx, st), 1)

    def forward_chunkwise(self, x: Tensor, c: Tensor, recurrent_state: RecurrentState = None):
        """x: (B, T, D).  c: (B, T, D), (B, T', D) with T % T' == 0 (shared inside fixed-length frames) or (B, D)."""
        return self._walk(x, recurrent_state, lambda layer, h, idx, st: layer.forward_chunkwise(h, c, idx, st), x.size(1))

    def forward(self, x: Tensor, c: Tensor, recurrent_state: RecurrentState = None):
        return self.forward_chunkwise(x=x, c=c, recurrent_state=recurrent_state)
