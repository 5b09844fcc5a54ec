"""Sodudra: a decoder of parallel blocks over latent attention and routed experts, with a repeated span of layers.

``config.json`` lists the layers one by one (``layers[i] = {type, mixer, mlp}``).  A block is :class:`ParallelDecoderLayer`:
``h = norm1(x)``, ``x <- x + mixer(h) + mlp(h)``, then the layer's token input (:class:`TokenSideInput`, a slice of a second embedding
table gated by the stream).  Parts:

* mixer ``latent_attention`` — :class:`LatentSinkAttention`: one normalised low-rank row per token is all the cache holds; scores and
  outputs are formed against it directly (absorbed up-projections), softmax with a learned sink per head, sigmoid gate per head;
* feed-forward ``moe`` — :class:`MoE` with a sigmoid router whose chosen scores are renormalised, two-matrix squared-ReLU experts and
  an always-on shared expert of the same form;
* ``loop`` — layers ``start .. stop-1`` run ``times`` times in a row with the same weights; every run of a layer has a cache of its
  own, and ``loop_step[t]`` is added to the stream right before pass ``t``;
* input: embedding followed by an RMS norm; output: final norm, head, ``logit_scale``, then ``cap * tanh(logits / cap)``.

Every size and constant comes from the checkpoint's ``config.json``.  The engine side is the one the other hybrid stacks use: the
paged cache with per-layer shapes (:class:`LayeredBlockKVCacheManager`, here one latent row per token and layer RUN), ragged rows
(prompt portions beside single decoded tokens) in one forward, decode steps replayed from CUDA graphs.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from ... import ops
from ...config import InferenceConfig, NeuronConfig
from ...modules.attention.latent_attention import LatentSinkAttention
from ...modules.kvcache import LayeredBlockKVCacheManager
from ...modules.mlp import PlainMLP
from ...modules.moe import ExpertMLPs, MoE, RouterTopK
from ...modules.norm import RMSNorm
from ...modules.sampling import Sampler
from ...modules.token_side import TokenSideInput
from ...parallel.layers import ColumnParallelLinear, ParallelEmbedding
from ..application_base import NeuronBaseForCausalLM
from ..model_base import NeuronBaseModel, ParallelDecoderLayer

ROUTER_SUM_EPS = 1e-20       # added to the sum of the chosen scores before the division (fixed by the design)
EXPERT_ACT = "relu2"         # experts: down(relu(up x)^2)
SIDE_ACT = "gelu_tanh"


def layer_runs(n_layers: int, loop: Optional[dict]) -> List[Tuple[int, Optional[int]]]:
    """The order in which layers run: ``(layer, pass)`` with ``pass = t`` on the first layer of pass ``t`` of the repeated span (the
    place where ``loop_step[t]`` enters) and ``None`` everywhere else."""
    if not loop or int(loop.get("times", 1)) < 1 or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n_layers)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    if not (0 <= a < b <= n_layers):
        raise ValueError(f"loop {a}..{b} outside the {n_layers} layers")
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n_layers)]


class SodudraInferenceConfig(InferenceConfig):
    def get_required_attributes(self) -> List[str]:
        return ["layers", "norm", "vocab", "width"]

    def add_derived_config(self):
        self.num_cores_per_group = 1
        self.hidden_size, self.vocab_size, self.num_hidden_layers = self.width, self.vocab, len(self.layers)
        self.rms_norm_eps = float(self.norm["eps"])
        for name, default in (("loop", None), ("token_side", None), ("logit_scale", 1.0), ("logit_softcap", None)):
            if not hasattr(self, name):
                setattr(self, name, default)
        for i, layer in enumerate(self.layers):
            if layer["type"] != "latent_attention":
                raise ValueError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "moe") != "moe":
                raise ValueError(f"layer {i}: unknown mlp kind {mlp.get('kind')!r}")
        self.runs = layer_runs(len(self.layers), self.loop)

    @classmethod
    def get_neuron_config_cls(cls):
        return NeuronConfig

    @classmethod
    def from_pretrained(cls, model_path: str, neuron_config: NeuronConfig) -> "SodudraInferenceConfig":
        with open(os.path.join(model_path, "config.json")) as f:
            d = json.load(f)

        def load(self):
            for k, v in d.items():
                setattr(self, k, v)
        return cls(neuron_config, load_config=load)


class NeuronSodudraModel(NeuronBaseModel):
    meta_extra_keys = ("computed_context_lens",)
    graph_tensor_kwargs = ("slot_mapping", "block_table", "computed_context_lens", "gather_positions")

    def __init__(self, config, device=None):
        super().__init__(config, device)
        # every op of a step is a sync-free kernel launch or a torch op on static shapes (the routed experts run on a device-side
        # permutation with a static row bound); rows with seq_id -1 have q_len 0 and write nothing
        self.graph_safe = device is not None and torch.device(device).type == "cuda"

    def setup_attr_for_model(self, config):
        nc = config.neuron_config
        if nc.tp_degree != 1:
            raise NotImplementedError("Sodudra: tensor parallel degree 1")
        if not nc.is_block_kv_layout:
            raise ValueError("Sodudra runs on the paged KV cache: set is_block_kv_layout=True, pa_block_size, pa_num_blocks")
        self.tp_degree, self.hidden_size = 1, config.width
        self.max_batch_size, self.buckets = nc.max_batch_size, nc.buckets

    def init_model(self, config):
        nc = config.neuron_config
        dev, dt = self.device_, nc.torch_dtype
        W, eps = config.width, config.rms_norm_eps
        emb = lambda rows, cols: ParallelEmbedding(rows, cols, None, dtype=dt, device=dev, shard_across_embedding=True, pad=True,      # noqa: E731
                                                   tensor_model_parallel_group=self.tp_group)
        norm = lambda: RMSNorm(W, eps, torch.float32, device=dev)       # noqa: E731
        self.embed_tokens = emb(config.vocab, W)
        self.embed_norm = norm()
        side_dim = int((config.token_side or {}).get("dim") or 0)
        self.side_embed = emb(config.vocab, side_dim * len(config.layers)) if side_dim else None
        times = int((config.loop or {}).get("times") or 0)
        self.loop_step = nn.Parameter(torch.zeros(times, W, dtype=torch.float32, device=dev), requires_grad=False) if times else None
        layers = []
        for i, spec in enumerate(config.layers):
            m = spec["mixer"]
            mixer = LatentSinkAttention(W, m["heads"], m["dim"], m.get("vdim", m["dim"]), m["kv_rank"],
                                        scale=float(m["scale"]) if m.get("scale") is not None else m["dim"] ** -0.5, eps=eps, layer_idx=i,
                                        dtype=dt, device=dev, tp_group=self.tp_group)
            f, mlp = spec.get("mlp"), None
            if f is not None:
                r = f["router"]
                router = RouterTopK(r["experts"], r["top"], W, dt, "sigmoid", False, False, False, dev, renorm_eps=ROUTER_SUM_EPS)
                experts = ExpertMLPs(r["experts"], W, f["expert"]["ff"], EXPERT_ACT, dt, False, dev, gated=False)
                shared = PlainMLP(W, f["shared"]["ff"], EXPERT_ACT, dt, False, self.tp_group, dev) if f.get("shared") else None
                mlp = MoE(router, experts, shared)
            side = TokenSideInput(W, side_dim, i, SIDE_ACT, dt, dev, self.tp_group) if side_dim else None
            layers.append(ParallelDecoderLayer(mixer, mlp, norm(), side, i))
        self.layers = nn.ModuleList(layers)
        self.runs = list(config.runs)
        self.norm = norm()
        self.lm_head = ColumnParallelLinear(W, config.vocab, bias=False, gather_output=False, dtype=dt, device=dev, pad=True,
                                            tensor_model_parallel_group=self.tp_group)

    def _kernels_cover_decode(self) -> bool:
        return False

    def init_inference_optimization(self, config):
        nc = self.neuron_config
        if self.on_device_sampling:
            self.sampler = Sampler(nc, self.tp_group, vocab_shard=False)
        # one latent cache per layer RUN: a layer of the repeated span sees different streams in different passes
        shapes = {r: self.layers[i].mixer.kv_shape() for r, (i, _) in enumerate(self.runs)}
        self.kv_mgr = LayeredBlockKVCacheManager(shapes, {}, nc.pa_num_blocks, nc.pa_block_size, nc.torch_dtype, self.device_,
                                                 state_specs={}, num_slots=nc.kv_cache_batch_size, state_dtype=nc.torch_dtype)

    # ---- forward hooks ---------------------------------------------------------------------------------------------------
    def build_meta(self, input_ids, attention_mask, position_ids, seq_ids, is_prefill, **kw):
        meta = super().build_meta(input_ids, attention_mask, position_ids, seq_ids, is_prefill, **kw)
        if meta.block_table is None:
            raise ValueError("Sodudra: every forward needs block_table (paged KV cache)")
        B, T = input_ids.shape[:2]
        dev = input_ids.device
        q_len = meta.key_valid.sum(-1).to(torch.int32) if meta.key_valid is not None else torch.full((B,), T, dtype=torch.int32, device=dev)
        q_len = torch.where(meta.seq_ids < 0, torch.zeros_like(q_len), q_len)
        ctx = meta.extras.get("computed_context_lens")
        ctx = meta.position_ids[:, 0] if ctx is None else ctx.to(dev)
        meta.extras.update(q_len=q_len.contiguous(), ctx_len=ctx.to(torch.int32).contiguous(), act_dtype=self.neuron_config.torch_dtype)
        if self.side_embed is not None:
            meta.extras["token_side"] = self.side_embed(input_ids)          # [B, T, layers * dim]: one lookup serves every layer
        return meta

    def _before(self, run):
        """What enters the stream right before run ``run``: (the pass vector or None, the block's norm weight)."""
        i, t = self.runs[run]
        return (None if t is None or self.loop_step is None else self.loop_step[t]), self.layers[i].norm1.weight

    def run_layers(self, emb, meta):
        dt, eps = meta.extras["act_dtype"], self.config.rms_norm_eps
        fuse = meta.capture is None          # capturing the stream after every run keeps the pass vector out of the captured value
        vec, w = self._before(0)
        x, _, h = ops.stream_add_rmsnorm(None, normed=emb, normed_weight=self.embed_norm.weight, vec=vec, weight=w, eps=eps, lp_dtype=dt)
        for r, (i, _) in enumerate(self.runs):
            vec, w = self._before(r + 1) if r + 1 < len(self.runs) else (None, None)
            if fuse:
                x, h = self.layers[i](x, h, meta, self.kv_mgr, r, next_weight=w, next_vec=vec)
            else:
                x, _ = self.layers[i](x, h, meta, self.kv_mgr, r)
                meta.capture[f"runs.{r}.out"] = x
                if w is not None:
                    x, _, h = ops.stream_add_rmsnorm(x, vec=vec, weight=w, eps=eps, lp_dtype=dt)
        return x

    def final_hidden(self, h):
        return ops.stream_add_rmsnorm(h.float(), weight=self.norm.weight, eps=self.norm.variance_epsilon)[2]

    def compute_logits(self, h):
        dt = self.neuron_config.torch_dtype
        hn = ops.stream_add_rmsnorm(h.float(), weight=self.norm.weight, eps=self.norm.variance_epsilon, lp_dtype=dt)[2]
        logits = self.lm_head(hn).float() * float(self.config.logit_scale)
        cap = self.config.logit_softcap
        return logits if not cap else float(cap) * torch.tanh(logits / float(cap))


class NeuronSodudraForCausalLM(NeuronBaseForCausalLM):
    _model_cls = NeuronSodudraModel
    _STATE_DICT_MODEL_PREFIX = ""

    @classmethod
    def get_config_cls(cls):
        return SodudraInferenceConfig

    @classmethod
    def from_pretrained(cls, model_path: str, neuron_config: NeuronConfig):
        return cls(model_path, SodudraInferenceConfig.from_pretrained(model_path, neuron_config))

    @staticmethod
    def convert_hf_to_neuron_state_dict(sd: dict, config) -> dict:
        """Checkpoint names (``l<i>.mix.q`` ...) -> module parameters: q | latent | head gates stacked for the fused input
        projection, the up-projections viewed per head, the experts' matrices stacked along a leading expert axis."""
        out = {"embed_tokens.weight": sd["embed"], "embed_norm.weight": sd["embed.norm"], "lm_head.weight": sd["head"],
               "norm.weight": sd["final.norm"]}
        if "side.embed" in sd:
            out["side_embed.weight"] = sd["side.embed"]
        if "loop.step" in sd:
            out["loop_step"] = sd["loop.step"]
        for i, spec in enumerate(config.layers):
            a, b = f"l{i}.", f"layers.{i}."
            out[b + "norm1.weight"] = sd[a + "norm1"]
            x, y, m = a + "mix.", b + "mixer.", spec["mixer"]
            H, R = m["heads"], m["kv_rank"]
            out[y + "in_proj.weight"] = torch.cat([sd[x + "q"], sd[x + "dkv"], sd[x + "g"]], 0)
            out[y + "latent_norm_weight"] = sd[x + "dkv.norm"]
            out[y + "k_up"] = sd[x + "uk"].reshape(H, m["dim"], R)
            out[y + "v_up"] = sd[x + "uv"].reshape(H, m.get("vdim", m["dim"]), R)
            out[y + "sinks"] = sd[x + "sink"]
            out[y + "o_proj.weight"] = sd[x + "o"]
            f = spec.get("mlp")
            if f is not None:
                x, y, E = a + "mlp.", b + "mlp.", f["router"]["experts"]
                out[y + "router.linear_router.weight"] = sd[x + "router"]
                out[y + "expert_mlps.gate_up_proj"] = torch.stack([sd[f"{x}e{e}.up"] for e in range(E)], 0)
                out[y + "expert_mlps.down_proj"] = torch.stack([sd[f"{x}e{e}.down"] for e in range(E)], 0)
                if f.get("shared"):
                    out[y + "shared_experts.fc1.weight"] = sd[x + "shared.up"]
                    out[y + "shared_experts.fc2.weight"] = sd[x + "shared.down"]
            if a + "side.gate" in sd:
                out[b + "side.gate.weight"] = sd[a + "side.gate"]
                out[b + "side.proj.weight"] = sd[a + "side.proj"]
                out[b + "side.norm_weight"] = sd[a + "side.norm"]
        return out

    def init_random_weights(self, seed: int = 0):
        """Benchmarks: N(0, 0.02) projections, unit norm weights, zero sinks and pass vectors."""
        super().init_random_weights(seed)
        with torch.no_grad():
            for name, p in self.model.named_parameters():
                if name.endswith(("norm1.weight", "norm_weight", "embed_norm.weight")) or name == "norm.weight":
                    p.fill_(1.0)
                elif name.endswith("sinks") or name == "loop_step":
                    p.zero_()
