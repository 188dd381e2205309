"""Rotary position embedding applied to queries and keys before retention.

Same call and numerics as the reference's ``XPos`` (flash_pop/xpos_emb.py:12-129): channel pairs
(2i, 2i+1) are rotated by the angle ``position * theta_i`` with ``theta_i = 10000^(-linspace(0,1,d/2))``;
``start_idx`` is an int (all rows share the offset) or a LongTensor with one offset per batch row (the
POP suffixes, whose rows start at different positions).  Computed in fp32 from cached phasor tables that grow on
demand: on CUDA tensors by the library's rotation kernel (q and k in one launch), elsewhere as an eager complex
multiplication.
"""
from __future__ import annotations

from typing import Optional, Union

import torch
from torch import Tensor

from flash_pop_b200.layer_ops import rotary_qk, rotary_supported


class XPos:
    def __init__(self, head_dim_qk: int, seq_len_estimate: int = 2 ** 12, start_idx: Union[int, Tensor] = 0,
                 device=None, dtype=None, scale: float = 10000.0) -> None:
        assert head_dim_qk % 2 == 0, "rotary embedding needs an even head dimension"
        self.head_dim = head_dim_qk
        exponents = torch.linspace(0, 1, steps=head_dim_qk // 2, device=device, dtype=torch.float32)
        self.thetas = 1.0 / (scale ** exponents)            # (d/2,)
        self._table: Optional[Tensor] = None                 # complex64 (L, d/2) for positions 0..L-1
        self._rows_key: Optional[Tensor] = None
        self._rows_table: Optional[Tensor] = None
        self.seq_len = 0
        self.fused = True            # CUDA tensors take the library's rotation kernel
        self._grow(seq_len_estimate)

    # -- tables -------------------------------------------------------------------------------------
    def _phasors(self, positions: Tensor) -> Tensor:
        angles = positions.to(self.thetas.device, torch.float32).unsqueeze(-1) * self.thetas
        return torch.polar(torch.ones_like(angles), angles)

    def _grow(self, length: int) -> None:
        if length > self.seq_len:
            self._table = self._phasors(torch.arange(length, device=self.thetas.device))
            self.seq_len = length

    def _move(self, device) -> None:
        if self.thetas.device != device:
            self.thetas = self.thetas.to(device)
            self._table = None if self._table is None else self._table.to(device)
            self._rows_key = self._rows_table = None

    def get_sin_cos(self, seq_len: int, start_idx: Union[int, Tensor]):
        """sin, cos of shape (1 or B, seq_len, 1, d) with each angle repeated for its channel pair."""
        ph = self._rotation(seq_len, start_idx)
        return (ph.imag.repeat_interleave(2, dim=-1).unsqueeze(2), ph.real.repeat_interleave(2, dim=-1).unsqueeze(2))

    def _rotation(self, seq_len: int, start_idx: Union[int, Tensor]) -> Tensor:
        if isinstance(start_idx, int):
            self._grow(start_idx + seq_len)
            return self._table[start_idx:start_idx + seq_len].unsqueeze(0)          # (1, T, d/2)
        assert isinstance(start_idx, Tensor) and start_idx.dim() == 1, "start_idx: int or 1-D LongTensor"
        key = self._rows_key
        if key is None or key.shape != start_idx.shape or self._rows_table.shape[1] != seq_len or not torch.equal(key, start_idx):
            pos = start_idx.view(-1, 1) + torch.arange(seq_len, device=start_idx.device).view(1, -1)
            self._rows_table = self._phasors(pos)                                    # (B, T, d/2)
            self._rows_key = start_idx.clone()
        return self._rows_table

    # -- application --------------------------------------------------------------------------------
    def _rotate(self, x: Tensor, ph: Tensor) -> Tensor:
        xc = torch.view_as_complex(x.float().unflatten(-1, (-1, 2)))
        if x.dim() == 4:                       # (B, T, H, d): broadcast over heads
            ph = ph.unsqueeze(2)
        else:                                  # (B, H, d) single step: ph is (1, 1, d/2) or (B, 1, d/2)
            ph = ph.reshape(ph.shape[0], 1, -1)
        return torch.view_as_real(xc * ph).flatten(-2).to(x.dtype)

    def __call__(self, q: Tensor, k: Tensor, start_idx: Union[int, Tensor], *args, **kwargs):
        self._move(q.device)
        seq_len = q.size(1) if q.dim() == 4 else 1
        ph = self._rotation(seq_len, start_idx)
        if self.fused and rotary_supported(q) and k.shape == q.shape:
            # one kernel for both tensors (and one for their gradients) instead of the eager complex product
            return rotary_qk(q, k, torch.view_as_real(ph).contiguous())
        return self._rotate(q, ph), self._rotate(k, ph)
