"""POP (parallel observation prediction) RetNet layers over the B200 operators.

Class names, ``Config`` fields and call signatures follow the reference (flash_pop/pop_retnet.py:15-243).
The observation stream goes through ``flash_pop_retention`` (outputs + the state after every full block);
the prediction-token suffixes go through ``pop_suffix_retention``, which reads each suffix's start state
in place from the stream's start state / block states instead of concatenating them into a new batch of
states as the reference does (flash_pop/pop_retnet.py:160-168), and never writes a state.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
from torch import Tensor

from flash_pop_b200.pop_retention import flash_pop_retention, pop_suffix_retention
from flash_pop_b200.fused_retention import cuda_core_kernels
from flash_pop_b200.recurrent_state import RecurrentState
from flash_pop_b200.retnet import MultiScaleRetention, RetNetDecoder, RetNetDecoderLayer
from flash_pop_b200.xpos_emb import XPos


class POPMultiScaleRetention(MultiScaleRetention):
    @dataclass(kw_only=True)
    class Config(MultiScaleRetention.Config):
        block_size: int

    def __init__(self, config: Config, xpos_embedder: Optional[XPos] = None):
        super().__init__(config, xpos_embedder=xpos_embedder)
        self.config = config

    def _maybe_cuda_core(self):
        import contextlib
        return contextlib.nullcontext() if self.config.use_fused_version else cuda_core_kernels()

    def _pop_retention_kernel(self, q: Tensor, k: Tensor, v: Tensor, prev_state: Tensor):
        with self._maybe_cuda_core():
            return flash_pop_retention(q, k, v, prev_state, self.head_decays, self.config.block_size)

    def pop_chunkwise(self, x: Tensor, start_index: int, prev_state: Optional[Tensor]):
        """Returns the layer output and block_states (B, T // block_size, H, dk, dv)."""
        return self._retention_chunkwise(x, start_index, prev_state, self._pop_retention_kernel)

    def suffixes_chunkwise(self, suffixes: Tensor, start_indices: Tensor, prev_state: Optional[Tensor], states: Tensor,
                           xpos_embedder: Optional[XPos]) -> Tensor:
        """suffixes: (B*M, P, H*dv), M suffixes per stream row.  Suffix m starts from prev_state (m == 0) or
        states[:, m-1]."""
        B, N = states.shape[:2]
        M = suffixes.size(0) // B

        def kernel(q, k, v, _unused_state):
            unf = lambda t: t.unflatten(0, (B, M))
            s0 = None if prev_state is None else prev_state.to(q.dtype)
            with self._maybe_cuda_core():
                out = pop_suffix_retention(unf(q), unf(k), unf(v), s0, states.to(q.dtype), self.head_decays)
            return out.flatten(0, 1), out.new_empty(0)

        # the start states are handed to the kernel through the closure, not through `prev_state`
        placeholder = suffixes.new_empty(0)
        out, _ = self._retention_chunkwise(suffixes, start_indices, placeholder, kernel, xpos_embedder)
        return out


class POPDecoderLayer(RetNetDecoderLayer):
    @dataclass(kw_only=True)
    class Config(RetNetDecoderLayer.Config):
        block_size: int

    def __init__(self, config: Config, xpos_embedder: Optional[XPos] = None, suffixes_xpos_embedder: Optional[XPos] = None):
        super().__init__(config, xpos_embedder)
        self.suffixes_xpos_embedder = suffixes_xpos_embedder
        self.config = config

    def _build_multi_scale_retention(self, xpos_embedder: Optional[XPos] = None):
        cfg = POPMultiScaleRetention.Config(block_size=self.config.block_size, use_fused_version=self.config.use_fused_version,
                                            **self._retention_config_kwargs())
        return POPMultiScaleRetention(cfg, xpos_embedder=xpos_embedder)

    def _post(self, y: Tensor) -> Tensor:
        return self.dropout(y) if self.config.use_post_retention_dropout else y

    def pop_forward(self, x: Tensor, start_index: int, prev_state: Optional[Tensor], suffixes: Optional[Tensor] = None,
                    suffixes_start_indices: Optional[Tensor] = None):
        """x: (B, T, H*dv) observation stream.  suffixes: (B*(N+1), P, H*dv) or None.
        Without suffixes returns (x, block_states, None); with suffixes (x, last block state, suffixes)."""
        assert x.dim() == 3, f"Got {x.dim()}"
        captured = {}

        def stream_branch(h):
            y, states = self.retention.pop_chunkwise(h, start_index=start_index, prev_state=prev_state)
            captured["states"] = states
            return self._post(y), states

        x, states = self._residual_blocks(x, stream_branch, fp32_norm=True)
        if suffixes is None:
            return x, states, None

        def suffix_branch(h):
            y, last = self._suffixes_forward(h, suffixes_start_indices, prev_state, states, x.size(0), self.suffixes_xpos_embedder)
            return self._post(y), last

        suffixes, last_state = self._residual_blocks(suffixes, suffix_branch, fp32_norm=True)
        return x, last_state, suffixes

    def _suffixes_forward(self, suffixes, start_indices, prev_state, states, batch_size, xpos_embedder=None):
        assert start_indices is not None and isinstance(start_indices, Tensor)
        assert suffixes.dim() == 3, f"Got {suffixes.dim()}"
        num_blocks = suffixes.size(0) // batch_size
        assert states.size(1) + 1 >= num_blocks, (f"got {states.size(1)} block states for {num_blocks} suffix blocks; "
                                                  "each suffix block after the first needs the state of the block before it")
        out = self.retention.suffixes_chunkwise(suffixes, start_indices, prev_state, states,
                                                xpos_embedder or self.suffixes_xpos_embedder)
        return out, states[:, -1].clone()


def _get_suffixes_start_indices(batch_size, num_blocks, start_index: int, block_size: int, device):
    start = start_index + torch.arange(num_blocks, device=device) * block_size
    return start.repeat(batch_size)


class POPRetNetDecoder(RetNetDecoder):
    def __init__(self, layer_config: POPDecoderLayer.Config, num_layers: int):
        self.suffixes_xpos_embedder = XPos(layer_config.head_dim_qk or layer_config.head_dim_v, device=layer_config.device,
                                           dtype=layer_config.dtype)
        super().__init__(layer_config, num_layers)

    def _build_layers(self, num_layers: int):
        return [POPDecoderLayer(self.layer_config, xpos_embedder=self.xpos_embedder,
                                suffixes_xpos_embedder=self.suffixes_xpos_embedder) for _ in range(num_layers)]

    def pop_forward(self, x: Tensor, recurrent_state: RecurrentState = None, suffixes: Optional[Tensor] = None):
        """x: (B, T, H*dv); suffixes: (B, N+1, P, H*dv) or None.
        Returns (x, new RecurrentState, suffixes (B, N+1, P, H*dv) or None)."""
        rs = self._validate_and_init_state(recurrent_state)
        start_indices = None
        if suffixes is not None:
            assert suffixes.dim() == 4, f"Got {suffixes.dim()}"
            start_indices = _get_suffixes_start_indices(x.size(0), suffixes.size(1), rs.index, self.layer_config.block_size, x.device)
            suffixes = suffixes.flatten(0, 1)
        states = []
        for layer, state_i in zip(self.layers, rs.state):
            x, state, suffixes = layer.pop_forward(x, rs.index, state_i, suffixes, suffixes_start_indices=start_indices)
            states.append(state)
        if suffixes is not None:
            suffixes = suffixes.unflatten(0, (x.size(0), -1))
        return x, RecurrentState(state=torch.stack(states), index=rs.index + x.size(1)), suffixes
