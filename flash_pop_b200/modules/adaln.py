"""Adaptive LayerNorm (AdaLN / AdaLN-Zero) conditioning blocks of the diffusion RetNet, with the optional
low-rank (LoRA) modulation; same parameter names and arithmetic as the reference
(flash_pop/modules/adaln.py:13-166)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from flash_pop_b200.layer_ops import adaln_modulate, gate_residual


def modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    assert x.shape == shift.shape == scale.shape, f"Got x: {x.shape}, shift: {shift.shape}, scale: {scale.shape}"
    return x * (1 + scale) + shift


def apply_modulation(c: torch.Tensor, modulation_op, x_shape) -> torch.Tensor:
    """Run the modulation MLP on the conditioning and broadcast it to the (B, T, D) activations:
    c is (B, D) (shared by all steps), (B, T', D) with T % T' == 0 (one per frame) or (B, T, D)."""
    assert len(x_shape) == 3, f"Expected x to have 3 dims, got {len(x_shape)}"
    B, T = x_shape[0], x_shape[1]
    if c.dim() == 2:
        return modulation_op(c.unsqueeze(1)).expand(B, T, -1)
    assert c.dim() == 3, f"Got c.dim={c.dim()}"
    if c.size(1) == T:
        assert c.shape == tuple(x_shape), f"Shape mismatch: {c.shape}!={x_shape}"
        return modulation_op(c)
    assert T % c.size(1) == 0, f"Got incompatible shapes: {x_shape}, {c.shape}"
    return modulation_op(c).repeat_interleave(T // c.size(1), dim=1)


class _AdaNormBase(nn.Module):
    n_chunks = 2

    def __init__(self, hidden_size: int, lora_hidden_dim: Optional[int] = None, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.lora_hidden_dim = lora_hidden_dim
        out = self.n_chunks * hidden_size
        kw = dict(device=device, dtype=dtype)
        if lora_hidden_dim is None:
            layers = [nn.SiLU(), nn.Linear(hidden_size, out, bias=True, **kw)]
        else:
            layers = [nn.SiLU(), nn.Linear(hidden_size, lora_hidden_dim, bias=False, **kw),
                      nn.Linear(lora_hidden_dim, out, bias=True, **kw)]
        self.modulation = nn.Sequential(*layers)
        self.norm = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=eps, device=device, dtype=torch.float32)
        self.initialize_weights()

    def initialize_weights(self):
        nn.init.zeros_(self.modulation[-1].weight)
        nn.init.zeros_(self.modulation[-1].bias)
        if self.lora_hidden_dim is not None:
            nn.init.zeros_(self.modulation[-2].weight)

    def modulation_rows(self, x: torch.Tensor, c: torch.Tensor):
        """The modulation MLP on the conditioning, NOT broadcast to the activations: `n_chunks` tensors (B, Tm, D), each
        row shared by T / Tm consecutive tokens of x - Tm = 1 for c (B, D), T' for c (B, T', D), T for c (B, T, D)."""
        assert x.dim() == 3, f"Expected x to have 3 dims, got {x.dim()}"
        B, T = x.shape[0], x.shape[1]
        if c.dim() == 2:
            c = c.unsqueeze(1)
        assert c.dim() == 3, f"Got c.dim={c.dim()}"
        assert c.size(1) == T or T % c.size(1) == 0, f"Got incompatible shapes: {tuple(x.shape)}, {tuple(c.shape)}"
        return self.modulation(c).chunk(self.n_chunks, dim=-1)

    def modulated_norm(self, x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        """norm(x) * (1 + scale) + shift, the fp32 LayerNorm and the modulation in one kernel each way on CUDA."""
        return adaln_modulate(x, shift, scale, self.norm.eps)


def _to_tokens(m: torch.Tensor, T: int) -> torch.Tensor:
    """(B, Tm, D) modulation rows as the (B, T, D) tensor the reference's modules hand out."""
    return m.expand(-1, T, -1) if m.size(1) == 1 else (m if m.size(1) == T else m.repeat_interleave(T // m.size(1), dim=1))


class AdaLayerNorm(_AdaNormBase):
    """x: (B, T, D), c: conditioning.  Returns norm(x) * (1 + scale) + shift."""
    n_chunks = 2

    def forward(self, x: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
        shift, scale = self.modulation_rows(x, c)
        return self.modulated_norm(x, shift, scale)


class AdaLayerNormZero(_AdaNormBase):
    """As AdaLayerNorm, and also returns the gate for the branch that follows."""
    n_chunks = 3

    def forward(self, x: torch.Tensor, c: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        shift, scale, gate = self.modulation_rows(x, c)
        return self.modulated_norm(x, shift, scale), _to_tokens(gate, x.size(1))

    def forward_rows(self, x: torch.Tensor, c: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """As forward, with the gate left as its (B, Tm, D) rows for `gated_residual`."""
        shift, scale, gate = self.modulation_rows(x, c)
        return self.modulated_norm(x, shift, scale), gate


def gated_residual(x: torch.Tensor, branch: torch.Tensor, gate_rows: torch.Tensor) -> torch.Tensor:
    """x + branch * gate with the gate given as (B, Tm, D) rows (AdaLayerNormZero.forward_rows)."""
    return gate_residual(x, branch, gate_rows)
