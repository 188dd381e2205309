"""RetNet layers that call the B200 retention operator.

Thin PyTorch callers with the reference's class names, ``Config`` fields and defaults, parameter names
(so reference checkpoints load) and arithmetic (flash_pop/retnet.py:104-575): q/k/v projections, rotary
embedding, the retention operator in bf16, per-head GroupNorm in fp32, swish gate, output projection,
pre-norm residual blocks with fp32 LayerNorm.  Only the operator underneath differs.

Differences from the reference, none of which changes results of a working call:
  * ``use_fused_version=False`` selects the fp32-arithmetic CUDA-core kernels of this library instead of a
    PyTorch implementation (``chunk_size`` is accepted and ignored) — the package has no non-CUDA path;
  * the decoder creates the zero start state itself when called without one, and the recurrent walk
    iterates the per-layer states (the reference discards the state it creates and zips over the container,
    flash_pop/retnet.py:535-575);
  * per-head decays are a non-persistent buffer, so they follow ``module.to(device)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache
from typing import Callable, List, Literal, Optional, Tuple, Union

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from flash_pop_b200.fused_retention import cuda_core_kernels, fused_chunk_retention, retention_step
from flash_pop_b200.layer_ops import groupnorm_gate, groupnorm_gate_supported, norm_in_fp32
from flash_pop_b200.recurrent_state import RecurrentState
from flash_pop_b200.xpos_emb import XPos

ActivationString = Literal["swish", "gelu", "relu"]
_ACTIVATIONS = {"swish": F.silu, "gelu": F.gelu, "relu": F.relu}


def _get_activation_fn(activation: str) -> Callable[[Tensor], Tensor]:
    try:
        return _ACTIVATIONS[activation]
    except KeyError:
        raise RuntimeError(f"Unsupported activation string '{activation}'. Supported: 'swish', 'gelu', 'relu'") from None


@lru_cache(maxsize=8)
def get_decays(num_heads: int, decay_range: Optional[Tuple[float, float]] = None) -> np.ndarray:
    """gamma_h = 1 - 2^(-5-h), or 1 - 2^(-linspace(lo, hi, H)) for decay_range=(lo, hi).
    (flash_pop/retnet.py:70-76)"""
    expo = -5.0 - np.arange(num_heads) if decay_range is None else -np.linspace(decay_range[0], decay_range[1], num_heads)
    return 1.0 - np.exp2(expo)


def retention_recurrent(query: Tensor, key: Tensor, value: Tensor, head_decays: Tensor, prev_state: Optional[Tensor],
                        scale: Optional[float] = None, decays: Optional[Tuple[float, ...]] = None) -> Tuple[Tensor, Tensor]:
    """One decoding step: S = gamma S_prev + k^T v / sqrt(dk); o = q S.  q, k: (B,H,dk), v: (B,H,dv),
    head_decays: (1,H,1,1).  (flash_pop/retnet.py:79-101)

    On CUDA tensors outside autograd this is the library's streaming step kernel (``decays``: the same decays as
    Python floats, which saves reading ``head_decays`` back from the device); where a gradient is being recorded it
    is the differentiable PyTorch expression."""
    assert head_decays.dim() == 4 and head_decays.shape[0] == 1 and head_decays.shape[2:] == (1, 1)
    needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (query, key, value, prev_state))
    if query.is_cuda and not needs_grad and scale is None and query.dtype in (torch.bfloat16, torch.float32):
        common = torch.promote_types(torch.promote_types(query.dtype, key.dtype), value.dtype)
        if common in (torch.bfloat16, torch.float32):
            if decays is None:
                decays = tuple(head_decays.flatten().tolist())
            state_dtype = common if prev_state is None else torch.promote_types(prev_state.dtype, head_decays.dtype)
            if state_dtype not in (torch.bfloat16, torch.float32):
                state_dtype = torch.float32
            return retention_step(query.to(common), key.to(common), value.to(common), decays, prev_state,
                                  state_dtype=state_dtype)
    key = key / (key.size(-1) ** 0.5 if scale is None else scale)
    state = key.unsqueeze(-1) * value.unsqueeze(-2)
    if prev_state is not None:
        state = state + prev_state * head_decays
    return torch.einsum("bhk,bhkv->bhv", query, state), state


def _split_heads(x: Tensor, num_heads: int) -> Tensor:
    return x.unflatten(-1, (num_heads, -1))


class MultiScaleRetention(nn.Module):
    """Multi-scale retention: H heads with different decays, GroupNorm over each head, swish gate."""

    @dataclass(kw_only=True)
    class Config:
        num_heads: int
        head_dim_v: int
        head_dim_qk: int = None
        dropout: float = 0.0
        head_decays_range: Optional[Tuple[float, float]] = None
        relative_position: bool = True
        bias: bool = True
        activation: Union[ActivationString, Callable[[Tensor], Tensor]] = "swish"
        group_norm_eps: float = 1e-6
        device: Optional[Union[torch.device, str]] = torch.device("cuda")
        dtype: Optional[torch.dtype] = torch.bfloat16
        use_fused_version: bool = True
        chunk_size: int = 512  # accepted for compatibility; unused

    def __init__(self, config: Config, xpos_embedder: Optional[XPos] = None):
        super().__init__()
        self.config = config
        self.num_heads = config.num_heads
        self.head_dim_v = config.head_dim_v
        self.head_dim_qk = config.head_dim_v if config.head_dim_qk is None else config.head_dim_qk
        self.embed_dim = embed_dim = self.head_dim_v * self.num_heads
        if self.head_dim_v % 8 != 0:
            raise ValueError(f"head_dim (embed_dim / num_heads = {self.head_dim_v}) must be divisible by 8")
        self.dropout = config.dropout
        self.relative_position = config.relative_position
        self.bias = config.bias
        self.activation = _get_activation_fn(config.activation) if isinstance(config.activation, str) else config.activation
        self.xpos_embedder = xpos_embedder if xpos_embedder is not None else XPos(self.head_dim_qk, device=config.device,
                                                                                   dtype=torch.float32)
        self.head_decays = tuple(get_decays(self.num_heads, config.head_decays_range).tolist())
        self.register_buffer("head_decays_torch",
                             torch.tensor(self.head_decays, dtype=torch.float32, device=config.device).view(1, -1, 1, 1),
                             persistent=False)

        kw = dict(bias=config.bias, device=config.device, dtype=config.dtype)
        qk_dim = self.num_heads * self.head_dim_qk
        self.q_proj = nn.Linear(embed_dim, qk_dim, **kw)
        self.k_proj = nn.Linear(embed_dim, qk_dim, **kw)
        self.v_proj = nn.Linear(embed_dim, embed_dim, **kw)
        self.group_norm = nn.GroupNorm(num_groups=self.num_heads, num_channels=embed_dim, affine=False,
                                       eps=config.group_norm_eps, device=config.device, dtype=torch.float32)
        self.g_proj = nn.Linear(embed_dim, embed_dim, **kw)
        self.out_proj = nn.Linear(embed_dim, embed_dim, **kw)
        self._reset_parameters()

    def _reset_parameters(self):
        for lin in (self.q_proj, self.k_proj, self.v_proj, self.out_proj, self.g_proj):
            nn.init.xavier_normal_(lin.weight)
            if lin.bias is not None:
                nn.init.constant_(lin.bias, 0)

    # -- operator call ------------------------------------------------------------------------------
    def _compute_chunkwise_retention_kernel(self, q: Tensor, k: Tensor, v: Tensor, prev_state: Tensor):
        if self.config.use_fused_version:
            return fused_chunk_retention(q, k, v, prev_state, self.head_decays)
        with cuda_core_kernels():
            return fused_chunk_retention(q, k, v, prev_state, self.head_decays)

    def _gate_and_project(self, retention: Tensor, x: Tensor) -> Tensor:
        """GroupNorm over each head of each token (fp32), swish gate, output projection."""
        shape = retention.shape[:-2]
        dropping = self.dropout > 0 and self.training
        z = self.g_proj(x)
        o4 = retention.reshape(-1, 1, self.num_heads, self.head_dim_v) if retention.dim() == 3 else retention
        if retention.dim() in (3, 4) and not dropping and z.dtype == retention.dtype:
            z4 = z.reshape(o4.shape)
            if groupnorm_gate_supported(o4, z4):
                swish = self.activation is F.silu
                gated = groupnorm_gate(o4, z4 if swish else self.activation(z4), self.group_norm.eps, swish)
                return self.out_proj(gated.reshape(*shape, self.embed_dim))
        flat = retention.reshape(-1, self.embed_dim)
        flat = F.dropout(flat, p=self.dropout, training=self.training)
        flat = self.group_norm(flat.float()).to(dtype=x.dtype)
        return self.out_proj(flat.view(*shape, self.embed_dim) * self.activation(z))

    def _retention_chunkwise(self, x: Tensor, start_idx: Union[int, torch.LongTensor], prev_state: Optional[Tensor] = None,
                             retention_kernel: Optional[Callable] = None, xpos_embedder: Optional[XPos] = None):
        """x: (B, T, H*dv).  Returns the layer output (B, T, H*dv) and whatever state(s) the kernel returns."""
        q = _split_heads(self.q_proj(x).to(dtype=x.dtype), self.num_heads)
        k = _split_heads(self.k_proj(x).to(dtype=x.dtype), self.num_heads)
        v = _split_heads(self.v_proj(x).to(dtype=x.dtype), self.num_heads)
        if self.relative_position:
            q, k = (xpos_embedder or self.xpos_embedder)(q, k, start_idx)
        if prev_state is None:
            prev_state = torch.zeros((x.size(0), self.num_heads, self.head_dim_qk, self.head_dim_v), device=x.device, dtype=x.dtype)
        kernel = retention_kernel or self._compute_chunkwise_retention_kernel
        retention, state = kernel(q.bfloat16(), k.bfloat16(), v.bfloat16(), prev_state.bfloat16())
        retention, state = retention.to(dtype=x.dtype), state.to(dtype=x.dtype)
        return self._gate_and_project(retention, x).to(dtype=x.dtype), state

    def forward_chunkwise(self, x: Tensor, start_idx: Union[int, torch.LongTensor], prev_state: Optional[Tensor] = None):
        return self._retention_chunkwise(x, start_idx, prev_state)

    def forward_recurrent(self, x: Tensor, seq_idx: int, prev_state: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
        """x: (B, H*dv), one token per row."""
        q = _split_heads(self.q_proj(x), self.num_heads)
        k = _split_heads(self.k_proj(x), self.num_heads)
        v = _split_heads(self.v_proj(x), self.num_heads)
        if self.relative_position:
            q, k = self.xpos_embedder(q, k, seq_idx)
        retention, state = retention_recurrent(q, k, v, self.head_decays_torch.to(x.device), prev_state=prev_state,
                                               decays=self.head_decays)
        return self._gate_and_project(retention, x), state


class RetNetDecoderLayer(nn.Module):
    """Pre-norm (default) residual block: retention, then a two-layer feed-forward."""

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
        norm_first: bool = True
        layer_norm_eps: float = 1e-6
        device: Optional[Union[torch.device, str]] = torch.device("cuda")
        dtype: Optional[torch.dtype] = torch.bfloat16
        use_fused_version: bool = True
        chunk_size: int = 512  # accepted for compatibility; unused

    def __init__(self, config: Config, xpos_embedder: Optional[XPos] = None) -> None:
        super().__init__()
        self.config = config
        self.activation = _get_activation_fn(config.activation) if isinstance(config.activation, str) else config.activation
        self.dropout = nn.Dropout(config.dropout)
        self.norm_first = config.norm_first
        d_model = config.num_heads * config.head_dim_v
        ln = dict(eps=config.layer_norm_eps, device=config.device, dtype=torch.float32)   # fp32 norms, as the reference
        self.norm1 = nn.LayerNorm(d_model, **ln)
        self.retention = self._build_multi_scale_retention(xpos_embedder=xpos_embedder)
        self.norm2 = nn.LayerNorm(d_model, **ln)
        self.linear1 = nn.Linear(d_model, config.dim_feedforward, device=config.device, dtype=config.dtype)
        self.linear2 = nn.Linear(config.dim_feedforward, d_model, device=config.device, dtype=config.dtype)
        self._reset_parameters()

    def _retention_config_kwargs(self) -> dict:
        c = self.config
        return dict(num_heads=c.num_heads, head_dim_v=c.head_dim_v, head_dim_qk=c.head_dim_qk, dropout=c.dropout,
                    head_decays_range=c.head_decays_range, activation=self.activation, device=c.device, dtype=c.dtype)

    def _build_multi_scale_retention(self, xpos_embedder: Optional[XPos] = None):
        cfg = MultiScaleRetention.Config(use_fused_version=self.config.use_fused_version, chunk_size=self.config.chunk_size,
                                         **self._retention_config_kwargs())
        return MultiScaleRetention(cfg, xpos_embedder=xpos_embedder)

    def _reset_parameters(self):
        for lin in (self.linear1, self.linear2):
            nn.init.xavier_normal_(lin.weight)
            nn.init.constant_(lin.bias, 0)

    def _feedforward_block(self, x: Tensor) -> Tensor:
        x = self.dropout(self.activation(self.linear1(x)))
        return self.dropout(self.linear2(x))

    def _residual_blocks(self, x: Tensor, retention_fn: Callable[[Tensor], Tuple[Tensor, Tensor]], fp32_norm: bool):
        """x + retention, x + feed-forward, with the norm before (pre-norm) or after each branch."""
        dtype = self.config.dtype
        norm = (lambda m, t: norm_in_fp32(m, t).to(dtype=dtype)) if fp32_norm else (lambda m, t: m(t))
        if self.norm_first:
            y, state = retention_fn(norm(self.norm1, x))
            x = x + y
            x = x + self._feedforward_block(norm(self.norm2, x))
        else:
            y, state = retention_fn(x)
            x = x + norm(self.norm1, y)
            x = x + norm(self.norm2, self._feedforward_block(x))
        return x, state

    def forward_chunkwise(self, x: Tensor, start_idx: int, prev_state: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
        def branch(h):
            y, state = self.retention.forward_chunkwise(h, start_idx=start_idx, prev_state=prev_state)
            return (self.dropout(y) if self.config.use_post_retention_dropout else y), state
        return self._residual_blocks(x, branch, fp32_norm=True)

    def forward_recurrent(self, x: Tensor, seq_idx: int, prev_state: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
        def branch(h):
            y, state = self.retention.forward_recurrent(h.to(self.config.dtype), seq_idx=seq_idx, prev_state=prev_state)
            return self.dropout(y), state
        return self._residual_blocks(x, branch, fp32_norm=True)

    def forward(self, x: Tensor, start_idx: int = 0, prev_state: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
        return self.forward_chunkwise(x, start_idx, prev_state)


class RetNetDecoder(nn.Module):
    """A stack of decoder layers that carries one retention state per layer in a ``RecurrentState``."""

    def __init__(self, layer_config: RetNetDecoderLayer.Config, num_layers: int):
        super().__init__()
        if layer_config.head_dim_qk is None:
            layer_config.head_dim_qk = layer_config.head_dim_v
        self.layer_config = layer_config
        self.num_layers = num_layers
        self.xpos_embedder = XPos(layer_config.head_dim_qk, device=layer_config.device, dtype=layer_config.dtype)
        self.layers = nn.ModuleList(self._build_layers(num_layers))

    def _build_layers(self, num_layers: int):
        return [RetNetDecoderLayer(self.layer_config, self.xpos_embedder) for _ in range(num_layers)]

    def _validate_and_init_state(self, recurrent_state: Optional[RecurrentState]) -> RecurrentState:
        if recurrent_state is None:
            recurrent_state = RecurrentState()
        if recurrent_state.state is None:
            return RecurrentState([None] * self.num_layers, 0 if recurrent_state.index is None else recurrent_state.index)
        if len(recurrent_state.state) != len(self.layers):
            raise ValueError(f"Expected {len(self.layers)} previous states, got {len(recurrent_state.state)}")
        assert recurrent_state.index is not None
        return recurrent_state

    def _walk_layers(self, x: Tensor, recurrent_state: Optional[RecurrentState], step: Callable, advance: int):
        rs = self._validate_and_init_state(recurrent_state)
        states: List[Tensor] = []
        for layer, state_i in zip(self.layers, rs.state):
            x, state = step(layer, x, rs.index, state_i)
            states.append(state)
        return x, RecurrentState(torch.stack(states), rs.index + advance)

    def forward_recurrent(self, x: Tensor, recurrent_state: RecurrentState = None) -> Tuple[Tensor, RecurrentState]:
        return self._walk_layers(x, recurrent_state, lambda layer, h, idx, st: layer.forward_recurrent(h, idx, st), 1)

    def forward_chunkwise(self, x: Tensor, recurrent_state: RecurrentState = None) -> Tuple[Tensor, RecurrentState]:
        return self._walk_layers(x, recurrent_state, lambda layer, h, idx, st: layer.forward_chunkwise(h, idx, st), x.size(1))

    def forward(self, x: Tensor, recurrent_state: RecurrentState = None) -> Tuple[Tensor, RecurrentState]:
        return self.forward_chunkwise(x, recurrent_state=recurrent_state)
