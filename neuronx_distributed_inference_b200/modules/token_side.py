"""Per-layer token input: every layer owns a slice of a second, narrow embedding table and feeds it into the residual stream through
a gated bottleneck, ``x <- x + rms_unit(W_proj (act(W_gate x) * e)) * w`` with ``e`` the layer's slice of the token's row.  The lookup is
done once per forward for all layers (``meta.extras['token_side']``, ``[B, T, layers * dim]``); a layer that runs several times reads
the same slice every time.  The closing norm and the sum belong to the stream kernel (``ops.stream_add_rmsnorm``), so this module
returns the projected rows and exposes ``norm_weight``."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear


class TokenSideInput(nn.Module):
    def __init__(self, hidden_size: int, dim: int, index: int, act: str = "gelu_tanh", dtype=torch.bfloat16, device=None, tp_group=None):
        super().__init__()
        self.lo, self.dim, self.act = index * dim, dim, act
        self.gate = ColumnParallelLinear(hidden_size, dim, bias=False, gather_output=False, dtype=dtype, device=device,
                                         tensor_model_parallel_group=tp_group)
        self.proj = RowParallelLinear(dim, hidden_size, bias=False, input_is_parallel=True, dtype=dtype, device=device,
                                      tensor_model_parallel_group=tp_group)
        self.norm_weight = nn.Parameter(torch.ones(hidden_size, dtype=torch.float32, device=device), requires_grad=False)

    def forward(self, x, meta):
        e = meta.extras["token_side"][..., self.lo:self.lo + self.dim]
        return self.proj(ops.gated_act_mul(self.gate(x), e, self.act))
