"""Mamba-2 mixer on ragged rows with carried state (chunked prompts, mixed prefill / decode batches).

``in_proj`` rows are ``[z: inner | x: inner | B: G N | C: G N | dt: heads]``.  x, B and C pass a depthwise causal convolution (+bias)
and SiLU; ``dt = softplus(dt + dt_bias)``; per head ``S <- exp(-exp(A_log) dt) S + dt B x^T`` (fp32, ``[N, head_dim]``),
``y = S^T C + D x``; the heads are gated by ``silu(z)`` FIRST and then RMS-normalised in ``norm_groups`` equal parts, times a weight.
Decays, step sizes, the state and the norm are fp32 whatever the activation dtype.  The convolution tail and the state of a
sequence live in its state line (``RecurrentStateCache``), so a prompt may arrive in portions of any size and rows of one batch may be
at different places of their sequences.  The per-token PyTorch loop of ``contrib/models/hybrid_family.py::Mamba2Mixer`` serves
whole-prompt prefill only; this module is the kernel path (csrc/seqmix.cu: short_conv, ssd_scan, group_rmsnorm).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear


class RaggedMamba2Mixer(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, state_size: int, groups: int, norm_groups: int,
                 conv_taps: int, eps: float, layer_idx: int, dtype=torch.bfloat16, device=None, tp_group=None):
        super().__init__()
        if num_heads % groups or (num_heads * head_dim) % norm_groups:
            raise ValueError("Mamba-2: heads must divide into groups and the inner width into norm groups")
        if tp_group is not None and tp_group.size != 1:
            raise NotImplementedError("ragged Mamba-2 mixer: tensor parallel degree 1")
        self.nh, self.P, self.N, self.G, self.norm_groups = num_heads, head_dim, state_size, groups, norm_groups
        self.taps, self.eps, self.layer_idx = conv_taps, eps, layer_idx
        self.inner = num_heads * head_dim
        self.conv_dim = self.inner + 2 * groups * state_size
        self.in_proj = ColumnParallelLinear(hidden_size, self.inner + self.conv_dim + num_heads, bias=False, gather_output=False,
                                            dtype=dtype, device=device, tensor_model_parallel_group=tp_group)
        self.out_proj = RowParallelLinear(self.inner, hidden_size, bias=False, input_is_parallel=True, dtype=dtype, device=device,
                                          tensor_model_parallel_group=tp_group)
        f32 = dict(dtype=torch.float32, device=device)
        self.conv_weight = nn.Parameter(torch.zeros(self.conv_dim, conv_taps, **f32), requires_grad=False)
        self.conv_bias = nn.Parameter(torch.zeros(self.conv_dim, **f32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(num_heads, **f32), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(num_heads, **f32), requires_grad=False)
        self.D = nn.Parameter(torch.ones(num_heads, **f32), requires_grad=False)
        self.norm_weight = nn.Parameter(torch.ones(self.inner, **f32), requires_grad=False)
        self.conv_state, self.ssm_state = f"ssm_conv{layer_idx}", f"ssm_state{layer_idx}"

    def state_specs(self):
        return {self.conv_state: (self.taps - 1, self.conv_dim), self.ssm_state: ((self.nh, self.N, self.P), torch.float32)}

    def forward(self, x, meta, kv_mgr):
        ex = meta.extras
        ctx, qlen, lines = ex["ctx_len"], ex["q_len"], ex["state_lines"]
        p = self.in_proj(x)
        I, Cd = self.inner, self.conv_dim
        z, u, dt = p[..., :I], p[..., I:I + Cd], p[..., I + Cd:]
        states = kv_mgr.states
        cst = states.tensor(self.conv_state)
        sst = states.tensor(self.ssm_state)
        xBC = ops.short_conv(u, self.conv_weight, self.conv_bias, cst, lines, ctx, qlen, silu=True)
        ops.short_conv_update(u, cst, lines, ctx, qlen)
        y = ops.ssd_scan(xBC, dt, z, self.A_log, self.dt_bias, self.D, sst, lines, ctx, qlen, self.nh, self.P, self.N, self.G)
        y = ops.group_rmsnorm(y, self.norm_weight, self.norm_groups, self.eps, out_dtype=x.dtype)
        return self.out_proj(y)
