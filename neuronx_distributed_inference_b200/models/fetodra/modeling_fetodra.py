"""Fetodra: a post-norm hybrid decoder.

``config.json`` lists the layers one by one (``layers[i] = {type, mixer, mlp}``); a layer is
``x <- norm1(alpha x + mixer(x))`` followed, when it has an MLP, by ``x <- norm2(alpha x + mlp(x))`` (:class:`PostNormDecoderLayer`,
norms with weights stored as deviations from one).  Mixers:

* ``attention`` — :class:`ConvWindowAttention`: biased q / k / v with a short causal convolution, row-wide q / k RMS norm, partial
  interleaved rotary positions, soft-capped scores, sliding window that keeps the first tokens, sigmoid output gate, optional reuse of
  an earlier layer's keys and values (``kv_from``);
* ``mamba2`` — :class:`RaggedMamba2Mixer`: gate before the grouped norm, state carried per sequence.

MLP: :class:`ClampedGLUMLP`.  Every size and constant comes from the checkpoint's ``config.json``; nothing here depends on a
particular stack.  The engine side: paged KV cache with per-layer shapes (:class:`LayeredBlockKVCacheManager`), state lines for the
convolution tails and recurrent states, ragged rows (prompt portions beside single decoded tokens) in one forward.
"""
from __future__ import annotations

import json
import os
from typing import List

import torch
import torch.nn as nn

from ... import ops
from ...config import InferenceConfig, NeuronConfig
from ...modules.attention.conv_window_attention import ConvWindowAttention
from ...modules.kvcache import LayeredBlockKVCacheManager
from ...modules.mlp import ClampedGLUMLP
from ...modules.norm import RMSNorm
from ...modules.sampling import Sampler
from ...modules.ssm import RaggedMamba2Mixer
from ...parallel.layers import ColumnParallelLinear, ParallelEmbedding
from ..application_base import NeuronBaseForCausalLM
from ..model_base import NeuronBaseModel, PostNormDecoderLayer

GLU_ALPHA = 1.702        # slope of the sigmoid in the gate product (fixed by the design)


class FetodraInferenceConfig(InferenceConfig):
    def get_required_attributes(self) -> List[str]:
        return ["layers", "norm", "postln_alpha", "vocab", "width"]

    def add_derived_config(self):
        self.num_cores_per_group = 1
        # names the engine's generic code looks up
        self.hidden_size, self.vocab_size, self.num_hidden_layers = self.width, self.vocab, len(self.layers)
        self.rms_norm_eps = float(self.norm["eps"])
        for i, layer in enumerate(self.layers):
            if layer["type"] not in ("attention", "mamba2"):
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown mlp kind {mlp.get('kind')!r}")
            src = layer["mixer"].get("kv_from")
            if src is not None:
                m, s = layer["mixer"], self.layers[src]["mixer"]
                if self.layers[src]["type"] != "attention" or s.get("kv_from") is not None or src >= i:
                    raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with keys of its own")
                shape = lambda x: (x.get("kv_heads", x["heads"]), x["dim"], x.get("vdim", x["dim"]))      # noqa: E731
                if shape(m) != shape(s):
                    raise ValueError(f"layer {i}: key / value shape differs from layer {src}")

    @classmethod
    def get_neuron_config_cls(cls):
        return NeuronConfig

    @classmethod
    def from_pretrained(cls, model_path: str, neuron_config: NeuronConfig) -> "FetodraInferenceConfig":
        with open(os.path.join(model_path, "config.json")) as f:
            d = json.load(f)

        def load(self):
            for k, v in d.items():
                setattr(self, k, v)
        return cls(neuron_config, load_config=load)


class NeuronFetodraModel(NeuronBaseModel):
    meta_extra_keys = ("computed_context_lens",)
    # decode steps (one token per row) replay from a CUDA graph: these per-step tensors are staged into the graph's static inputs
    graph_tensor_kwargs = ("slot_mapping", "block_table", "computed_context_lens", "gather_positions")

    def __init__(self, config, device=None):
        super().__init__(config, device)
        # every op of a step is a sync-free kernel launch or a torch op on static shapes; rows with seq_id -1 (graph warm-up, batch
        # padding) have q_len 0 and touch neither cache nor state
        self.graph_safe = device is not None and torch.device(device).type == "cuda"

    def setup_attr_for_model(self, config):
        nc = config.neuron_config
        if nc.tp_degree != 1:
            raise NotImplementedError("Fetodra: tensor parallel degree 1 (row-wide q/k norms and the grouped scan are not sharded)")
        if not nc.is_block_kv_layout:
            raise ValueError("Fetodra runs on the paged KV cache: set is_block_kv_layout=True, pa_block_size, pa_num_blocks")
        self.tp_degree, self.hidden_size = 1, config.width
        self.max_batch_size, self.buckets = nc.max_batch_size, nc.buckets

    def init_model(self, config):
        nc = config.neuron_config
        dev, dt = self.device_, nc.torch_dtype
        W, eps = config.width, config.rms_norm_eps
        self.embed_tokens = ParallelEmbedding(config.vocab, W, None, dtype=dt, device=dev, shard_across_embedding=True, pad=True,
                                              tensor_model_parallel_group=self.tp_group)
        norm = lambda: RMSNorm(W, eps, torch.float32, offset=1.0, device=dev)       # noqa: E731  (weights stored around zero)
        layers = []
        for i, spec in enumerate(config.layers):
            m = spec["mixer"]
            if spec["type"] == "attention":
                mask, rot = m.get("mask") or {}, m.get("rot") or {}
                mixer = ConvWindowAttention(W, m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"]),
                                            conv_taps=int(m.get("conv") or 1), rot_dims=int(rot.get("dims") or 0),
                                            rot_base=float(rot.get("base") or 10000.0),
                                            scale=float(m["scale"]) if m.get("scale") is not None else m["dim"] ** -0.5,
                                            softcap=m.get("softcap"), window=mask.get("size"), keep_first=int(mask.get("keep_first") or 0),
                                            eps=eps, layer_idx=i, kv_source=m.get("kv_from"), dtype=dt, device=dev, tp_group=self.tp_group)
            else:
                mixer = RaggedMamba2Mixer(W, m["heads"], m["vdim"], m["state"], int(m.get("groups") or 1), int(m.get("norm_groups") or 1),
                                          int(m.get("conv") or 1), eps, i, dtype=dt, device=dev, tp_group=self.tp_group)
            f = spec.get("mlp")
            mlp = ClampedGLUMLP(W, f["ff"], f["limit"], GLU_ALPHA, dt, self.tp_group, dev) if f is not None else None
            layers.append(PostNormDecoderLayer(mixer, mlp, norm(), norm() if f is not None else None, config.postln_alpha, i))
        self.layers = nn.ModuleList(layers)
        self.norm = norm()
        self.lm_head = ColumnParallelLinear(W, config.vocab, bias=False, gather_output=False, dtype=dt, device=dev, pad=True,
                                            tensor_model_parallel_group=self.tp_group)

    def _kernels_cover_decode(self) -> bool:
        return False

    def init_inference_optimization(self, config):
        nc = self.neuron_config
        if self.on_device_sampling:
            self.sampler = Sampler(nc, self.tp_group, vocab_shard=False)
        shapes, share, specs = {}, {}, {}
        for i, layer in enumerate(self.layers):
            specs.update(layer.state_specs())
            mx = layer.mixer
            if isinstance(mx, ConvWindowAttention):
                if mx.owns_kv:
                    shapes[i] = mx.kv_shape()
                else:
                    share[i] = mx.kv_source
        self.kv_mgr = LayeredBlockKVCacheManager(shapes, share, nc.pa_num_blocks, nc.pa_block_size, nc.torch_dtype, self.device_,
                                                 state_specs=specs, num_slots=nc.kv_cache_batch_size, state_dtype=nc.torch_dtype)

    # ---- forward hooks ---------------------------------------------------------------------------------------------------
    def build_meta(self, input_ids, attention_mask, position_ids, seq_ids, is_prefill, **kw):
        meta = super().build_meta(input_ids, attention_mask, position_ids, seq_ids, is_prefill, **kw)
        if meta.block_table is None:
            raise ValueError("Fetodra: every forward needs block_table (paged KV cache)")
        B, T = input_ids.shape[:2]
        dev = input_ids.device
        q_len = meta.key_valid.sum(-1).to(torch.int32) if meta.key_valid is not None else torch.full((B,), T, dtype=torch.int32, device=dev)
        q_len = torch.where(meta.seq_ids < 0, torch.zeros_like(q_len), q_len)
        ctx = meta.extras.get("computed_context_lens")
        ctx = meta.position_ids[:, 0] if ctx is None else ctx.to(dev)
        meta.extras.update(q_len=q_len.contiguous(), ctx_len=ctx.to(torch.int32).contiguous(),
                           state_lines=self.kv_mgr.lines_for(meta.seq_ids).to(torch.int32).contiguous(),
                           act_dtype=self.neuron_config.torch_dtype)
        return meta

    def embed(self, input_ids, inputs_embeds=None, vision_embeddings=None, vision_mask=None):
        return super().embed(input_ids, inputs_embeds, vision_embeddings, vision_mask).float()      # fp32 residual stream

    def final_hidden(self, h):
        return ops.scaled_add_rmsnorm(h.float(), None, self.norm.weight, 1.0, self.norm.variance_epsilon, self.norm.offset)[0]

    def compute_logits(self, h):
        dt = self.neuron_config.torch_dtype
        out, lp = ops.scaled_add_rmsnorm(h.float(), None, self.norm.weight, 1.0, self.norm.variance_epsilon, self.norm.offset, dt)
        return self.lm_head(out if lp is None else lp)


class NeuronFetodraForCausalLM(NeuronBaseForCausalLM):
    _model_cls = NeuronFetodraModel
    _STATE_DICT_MODEL_PREFIX = ""

    @classmethod
    def get_config_cls(cls):
        return FetodraInferenceConfig

    @classmethod
    def from_pretrained(cls, model_path: str, neuron_config: NeuronConfig):
        return cls(model_path, FetodraInferenceConfig.from_pretrained(model_path, neuron_config))

    @staticmethod
    def convert_hf_to_neuron_state_dict(sd: dict, config) -> dict:
        """Checkpoint names (``l<i>.mix.q`` ...) -> module parameters; q | k | v | gate (and their biases, zero for the gate) and
        gate | up are stacked for the fused projections."""
        out = {"embed_tokens.weight": sd["embed"], "lm_head.weight": sd["head"], "norm.weight": sd["final.norm"]}
        for i, spec in enumerate(config.layers):
            a, b = f"l{i}.", f"layers.{i}."
            out[b + "norm1.weight"] = sd[a + "norm1"]
            x, y = a + "mix.", b + "mixer."
            if spec["type"] == "attention":
                own = spec["mixer"].get("kv_from") is None
                names = ["q", "k", "v"] if own else ["q"]
                g = sd[x + "g"]
                out[y + "in_proj.weight"] = torch.cat([sd[x + n] for n in names] + [g], 0)
                zeros = lambda n: torch.zeros(sd[x + n].shape[0], dtype=g.dtype)                               # noqa: E731
                ident = lambda n: torch.ones(sd[x + n].shape[0], 1, dtype=g.dtype)                               # noqa: E731
                out[y + "in_proj.bias"] = torch.cat([sd.get(x + n + ".b", zeros(n)) for n in names] + [torch.zeros(g.shape[0], dtype=g.dtype)], 0)
                out[y + "conv_weight"] = torch.cat([sd.get(x + n + ".conv", ident(n)) for n in names], 0)
                out[y + "q_norm_weight"] = sd[x + "q.norm"]
                if own:
                    out[y + "k_norm_weight"] = sd[x + "k.norm"]
                out[y + "o_proj.weight"] = sd[x + "o"]
            else:
                for src, dst in (("in", "in_proj.weight"), ("conv", "conv_weight"), ("conv.b", "conv_bias"), ("dt_bias", "dt_bias"),
                                 ("A_log", "A_log"), ("D", "D"), ("norm", "norm_weight"), ("o", "out_proj.weight")):
                    if x + src in sd:
                        out[y + dst] = sd[x + src]
                if x + "conv" not in sd:                                 # a stack without the short convolution: one tap of weight one
                    m = spec["mixer"]
                    cd = m["heads"] * m["vdim"] + 2 * int(m.get("groups") or 1) * m["state"]
                    out[y + "conv_weight"] = torch.ones(cd, 1, dtype=sd[x + "in"].dtype)
            if spec.get("mlp") is not None:
                out[b + "norm2.weight"] = sd[a + "norm2"]
                out[b + "mlp.gate_up_proj.weight"] = torch.cat([sd[a + "mlp.gate"], sd[a + "mlp.up"]], 0)
                out[b + "mlp.down_proj.weight"] = sd[a + "mlp.down"]
        return out

    def init_random_weights(self, seed: int = 0):
        """Benchmarks: N(0, 0.02) projections; norms, decays and step biases at values that keep the stream well scaled."""
        super().init_random_weights(seed)
        with torch.no_grad():
            for name, p in self.model.named_parameters():
                if name.endswith(("norm1.weight", "norm2.weight")) or name == "norm.weight":
                    p.zero_()
                elif name.endswith(("q_norm_weight", "k_norm_weight", "mixer.norm_weight", "mixer.D")):
                    p.fill_(1.0)
                elif name.endswith("conv_weight"):
                    p.fill_(1.0 / p.shape[1])
                elif name.endswith("A_log"):
                    p.zero_()
                elif name.endswith("dt_bias"):
                    p.fill_(-2.0)
