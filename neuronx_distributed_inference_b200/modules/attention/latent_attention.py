"""Latent attention with a softmax sink and per-head output gates, on ragged rows and the paged cache.

Keys and values of every head are linear images of ONE low-rank row per token, ``c = rms_norm(W_dkv x)``: ``k_h = U_h c``,
``v_h = V_h c``.  Only ``c`` is cached (``kv_rank`` numbers per token and layer instead of ``heads * (dim + vdim)``), and neither
keys nor values are ever materialised: with ``a_h = U_h^T q_h`` the score is ``q_h . k_h = a_h . c`` and the head's output is
``V_h (sum_j p_j c_j)``, so attention runs as multi-query attention over the latent rows, which serve as keys AND values.  There are
no positional rotations.  Constructor parameters, so that other stacks can combine them:

* ``sink``: one learned logit per head joins the softmax denominator (a slot without key or value; not scaled);
* ``head_gate``: head ``h``'s output is multiplied by ``sigmoid(W_g x)_h`` — one factor per head, read from the mixer's input;
* ``scale``: multiplies the scores.

Data flow (CUDA: csrc/seqmix.cu for the two middle steps, GEMMs around them):

    p   = W_in x                          q | latent | head gates in ONE GEMM
          latent_norm_append(p)           fp32 RMS norm of the latent slice + paged cache write
    a   = q_h U_h                         batched over heads
    l   = paged_window_attention(a)       fp32 softmax (+ sink) over the latent cache, times sigmoid(gate_h)
    y   = W_o [V_h l_h]                   batched over heads, then the output projection

DeepSeek-style caches in this package (models/deepseek) keep expanded keys and values; this module is the compressed-cache form.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ... import ops
from ...parallel.layers import ColumnParallelLinear, RowParallelLinear


class LatentSinkAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, kv_rank: int, *, scale: float, eps: float,
                 sink: bool = True, head_gate: bool = True, layer_idx: int = 0, dtype=torch.bfloat16, device=None, tp_group=None):
        super().__init__()
        if tp_group is not None and tp_group.size != 1:
            raise NotImplementedError("latent attention: the latent row is shared by all heads; tensor parallel degree 1")
        self.n_q, self.head_dim, self.v_head_dim, self.kv_rank = num_heads, head_dim, v_head_dim, kv_rank
        self.scale, self.eps, self.layer_idx = float(scale), float(eps), layer_idx
        self.Cq, self.Cg = num_heads * head_dim, (num_heads if head_gate else 0)
        self.in_proj = ColumnParallelLinear(hidden_size, self.Cq + kv_rank + self.Cg, bias=False, gather_output=False, dtype=dtype,
                                            device=device, tensor_model_parallel_group=tp_group)
        self.o_proj = RowParallelLinear(num_heads * v_head_dim, hidden_size, bias=False, input_is_parallel=True, dtype=dtype,
                                        device=device, tensor_model_parallel_group=tp_group)
        self.k_up = nn.Parameter(torch.zeros(num_heads, head_dim, kv_rank, dtype=dtype, device=device), requires_grad=False)
        self.v_up = nn.Parameter(torch.zeros(num_heads, v_head_dim, kv_rank, dtype=dtype, device=device), requires_grad=False)
        f32 = dict(dtype=torch.float32, device=device)
        self.latent_norm_weight = nn.Parameter(torch.ones(kv_rank, **f32), requires_grad=False)
        self.sinks = nn.Parameter(torch.zeros(num_heads, **f32), requires_grad=False) if sink else None

    def kv_shape(self):
        """One kv head whose key row is also its value row."""
        return (1, self.kv_rank, None)

    def forward(self, x, meta, kv_mgr, cache_index=None):
        B, T, _ = x.shape
        ex = meta.extras
        ctx, qlen = ex["ctx_len"], ex["q_len"]
        H, R = self.n_q, self.kv_rank
        p = self.in_proj(x)
        cache, _ = kv_mgr.get_kv_by_layer_id(self.layer_idx if cache_index is None else cache_index)
        # whole prompts (no row brings earlier context): the new rows are all the keys there are, so attention can read them in token
        # order with the contiguous-key tcgen05 kernel; every other step (portions after a prefix, decoded tokens) reads the paged cache
        whole = meta.is_prefill and not meta.has_prefix and T >= 16 and ops.latent_prefill_on_tensor_cores(p, R)
        rows = ops.latent_norm_append(p, self.Cq, R, self.latent_norm_weight, self.eps, cache, meta.block_table, ctx, qlen, emit_rows=whole)
        # batched over heads with strided operands and results: the products land in [B, T, H, .] layout, no transposing copies
        a = torch.empty(B, T, H, R, dtype=p.dtype, device=p.device)
        torch.bmm(p.view(B * T, -1)[:, :self.Cq].unflatten(1, (H, self.head_dim)).transpose(0, 1), self.k_up, out=a.view(B * T, H, R).transpose(0, 1))
        gate = p[..., self.Cq + R:] if self.Cg else None
        if whole:
            lat = ops.attention_prefill(a, rows, rows, self.scale, True, sinks=self.sinks)
            lat = ops.head_gate_mul(lat, gate) if gate is not None else lat
        else:
            lat = ops.paged_window_attention(a, cache, cache, meta.block_table, ctx, qlen, self.scale, None, None, 0, gate, self.sinks,
                                             gate_per_head=True)
        o = torch.empty(B, T, H * self.v_head_dim, dtype=p.dtype, device=p.device)
        torch.bmm(lat.view(B * T, H, R).transpose(0, 1), self.v_up.transpose(1, 2), out=o.view(B * T, H, self.v_head_dim).transpose(0, 1))
        return self.o_proj(o)
