"""Carried retention state of a decoder stack, same fields and layout as the reference's container
(flash_pop/recurrent_state.py:5-35): ``state`` is (num_layers, B, H, dk, dv), ``index`` the number of
tokens already consumed (an int, or a LongTensor with one entry per batch row)."""
from __future__ import annotations

from typing import Optional, Union

from torch import LongTensor, Tensor


class RecurrentState:
    def __init__(self, state: Optional[Tensor] = None, index: Optional[Union[int, LongTensor]] = None):
        self.state = state
        self.index = index

    def to_dict(self):
        return {"state": self.state, "index": self.index}

    def clone(self):
        return RecurrentState(None if self.state is None else self.state.clone(),
                              self.index.clone() if isinstance(self.index, Tensor) else self.index)

    def cpu_clone(self):
        idx = self.index if isinstance(self.index, int) else self.index.detach().clone().cpu()
        return RecurrentState(self.state.detach().clone().cpu(), idx)

    def to_device(self, device):
        if self.state is not None:
            self.state = self.state.to(device)
        if isinstance(self.index, Tensor):
            self.index = self.index.to(device)
        else:
            assert isinstance(self.index, int)
        return self
