"""Continuous batching over the paged KV cache: page and state-slot pools, ragged step batches, a token-budget scheduler.

The reference leaves scheduling to the serving layer above it (vLLM hands it ``slot_mapping`` / ``block_table`` /
``computed_context_lens``, reference models/model_base.py:3314-3460); this module is that layer for stand-alone use:

* :class:`PagePool` / :class:`SlotPool` — free lists of KV pages and of per-sequence state lines (convolution tails, recurrent states);
  both are handed out lowest-first and returned on release, so pages and lines are reused across requests;
* :class:`PagedBatchEngine` — ``step(entries)`` runs ONE forward over a ragged batch: each entry brings the next tokens of a request
  (a portion of its prompt of any size, or one decoded token), rows are right-padded to the longest entry and the application is
  called with position ids, slot mapping, block table, ``computed_context_lens`` and the token indices whose logits are wanted.
  The kernels read true lengths, so a row's result does not depend on its neighbours or on its padding;
* :meth:`PagedBatchEngine.generate` — a scheduler on top of ``step``: every iteration decodes one token for each running request and
  spends what is left of ``max_step_tokens`` on prompt portions of waiting requests (chunked prefill), admitting new requests while
  state slots and pages last; sampling is the application's on-device sampler.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple
from typing import Sequence as Seq

import numpy as np
import torch


class PagePool:
    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))

    @property
    def available(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise MemoryError(f"KV cache exhausted: {n} pages wanted, {len(self._free)} free of {self.num_pages}")
        return [self._free.pop() for _ in range(n)]

    def give(self, pages: Iterable[int]):
        self._free.extend(sorted(pages, reverse=True))
        self._free.sort(reverse=True)


class SlotPool(PagePool):
    """State lines; same discipline as pages."""


@dataclass
class Sequence:
    rid: object
    slot: int
    pages: List[int] = field(default_factory=list)
    length: int = 0                                  # tokens already in the cache / folded into the state
    prompt: List[int] = field(default_factory=list)  # generate(): tokens not yet fed
    output: List[int] = field(default_factory=list)
    max_new_tokens: int = 0
    last_token: Optional[int] = None


class PagedBatchEngine:
    def __init__(self, app):
        nc = app.neuron_config
        if not nc.is_block_kv_layout:
            raise ValueError("PagedBatchEngine drives the paged KV cache (is_block_kv_layout)")
        self.app = app
        self.page = nc.pa_block_size
        self.pages = PagePool(nc.pa_num_blocks)
        self.slots = SlotPool(nc.kv_cache_batch_size)
        self.max_rows = min(nc.ctx_batch_size, nc.tkg_batch_size)
        self.max_row_tokens = nc.max_context_length
        self.live: Dict[object, Sequence] = {}
        self.device = torch.device(app.device) if app.device is not None else torch.device("cpu")
        self._host = None
        self._sp: Dict[int, torch.Tensor] = {}

    def _staging(self, n: int) -> torch.Tensor:
        """Reusable int32 host buffer of ``n`` elements; safe to refill every step because a step ends by reading its result back."""
        if self._host is None or self._host.numel() < n:
            self._host = torch.empty(max(n, 4096), dtype=torch.int32)
            if self.device.type == "cuda":
                self._host = self._host.pin_memory()
        return self._host[:n]

    def _sampling_rows(self, B: int) -> torch.Tensor:
        """The configured sampling parameters for ``B`` rows, resident on the engine's device."""
        if B not in self._sp:
            from ..modules.sampling import prepare_sampling_params
            c = self.app.neuron_config.on_device_sampling_config
            sp = prepare_sampling_params(B, c.top_k, c.top_p, c.temperature) if c is not None else prepare_sampling_params(B)
            self._sp[B] = sp.to(self.device)
        return self._sp[B]

    # ---- requests ----------------------------------------------------------------------------------------------------
    def admit(self, rid) -> Sequence:
        if rid in self.live:
            return self.live[rid]
        seq = Sequence(rid, self.slots.take(1)[0])
        self.live[rid] = seq
        return seq

    def release(self, rid):
        seq = self.live.pop(rid, None)
        if seq is not None:
            self.pages.give(seq.pages)
            self.slots.give([seq.slot])

    def _reserve(self, seq: Sequence, n_new: int):
        need = -(-(seq.length + n_new) // self.page) - len(seq.pages)
        if need > 0:
            seq.pages.extend(self.pages.take(need))

    # ---- one forward -------------------------------------------------------------------------------------------------
    def step(self, entries: Seq[Tuple[object, Seq[int], Seq[int]]], sample: bool = False):
        """``entries``: (request id, next tokens, indices among them whose logits are wanted).  Returns one fp32 tensor
        ``[len(want), vocab]`` per entry (CPU), or with ``sample`` the token sampled after each entry's LAST token."""
        if not entries:
            return []
        if any(len(toks) == 0 for _, toks, _ in entries):
            # an entry without tokens takes no part in the forward (its request stays admitted)
            full = [e for e in entries if len(e[1])]
            done = iter(self.step(full, sample))
            for rid, toks, _ in entries:
                if not len(toks):
                    self.admit(rid)
            return [next(done) if len(toks) else (None if sample else torch.zeros(0, 0)) for _, toks, _ in entries]
        if len(entries) > self.max_rows:
            raise ValueError(f"{len(entries)} rows in one step; the engine was sized for {self.max_rows}")
        seqs = [self.admit(rid) for rid, _, _ in entries]
        B = len(entries)
        T = max(len(toks) for _, toks, _ in entries)
        if T < 1 or any(len(toks) < 1 for _, toks, _ in entries):
            raise ValueError("every entry of a step brings at least one token")
        if T > self.max_row_tokens:
            raise ValueError(f"a portion of {T} tokens exceeds max_context_length={self.max_row_tokens}")
        for seq, (_, toks, _) in zip(seqs, entries):
            self._reserve(seq, len(toks))
        K = 1 if sample else max(1, max(len(w) for _, _, w in entries))
        P = max(len(s.pages) for s in seqs)
        P = 1 << (P - 1).bit_length()                    # block-table width in powers of two: few distinct decode graphs
        # every integer input of the step is laid out in ONE staging buffer (pinned on a GPU engine) and reaches the device in one copy:
        # ids | mask | positions | slot mapping (each [B, T]) | block table [B, P] | wanted indices [B, K] | state slots [B]
        sizes = [B * T] * 4 + [B * P, B * K, B]
        offs = np.cumsum([0] + sizes)
        host = self._staging(int(offs[-1]))
        flat = host.numpy()
        flat[:] = 0
        ids, mask, pos, slot_map = (flat[offs[i]:offs[i + 1]].reshape(B, T) for i in range(4))
        table, gather, slots = flat[offs[4]:offs[5]].reshape(B, P), flat[offs[5]:offs[6]].reshape(B, K), flat[offs[6]:offs[7]]
        slot_map[:] = -1
        ctx = np.zeros(B, dtype=np.int32)
        for b, (seq, (_, toks, want)) in enumerate(zip(seqs, entries)):
            n = len(toks)
            ids[b, :n] = np.asarray(toks, dtype=np.int32)
            mask[b, :n] = 1
            p = np.arange(seq.length, seq.length + n, dtype=np.int32)
            pos[b, :n] = p
            pg = np.asarray(seq.pages, dtype=np.int32)
            table[b, :len(pg)] = pg
            slot_map[b, :n] = pg[p // self.page] * self.page + p % self.page
            ctx[b] = seq.length
            slots[b] = seq.slot
            w = [n - 1] if sample else list(want)
            if w:
                gather[b, :len(w)] = np.asarray(w, dtype=np.int32)
        dev = host.to(self.device, non_blocking=True) if self.device.type == "cuda" else host.clone()
        part = lambda i, *shape: dev[int(offs[i]):int(offs[i + 1])].view(*shape)          # noqa: E731
        out = self.app(part(0, B, T), attention_mask=part(1, B, T), position_ids=part(2, B, T), seq_ids=part(6, B),
                       sampling_params=self._sampling_rows(B), slot_mapping=part(3, B, T), block_table=part(4, B, P),
                       computed_context_lens=torch.from_numpy(ctx), gather_positions=part(5, B, K), output_logits=not sample)
        for seq, (_, toks, _) in zip(seqs, entries):
            seq.length += len(toks)
        if sample:
            return [int(t) for t in out.tokens.reshape(B, -1)[:, 0].tolist()]
        logits = out.logits.float().cpu()
        return [logits[b, :len(want)] for b, (_, _, want) in enumerate(entries)]

    # ---- scheduler ---------------------------------------------------------------------------------------------------
    def generate(self, prompts: Seq[Seq[int]], max_new_tokens: int, max_step_tokens: int = 256,
                 eos_token_id: Optional[int] = None) -> List[List[int]]:
        """Greedy / sampled generation for a list of prompts with continuous batching and chunked prefill."""
        waiting = [Sequence(("gen", i), -1, prompt=list(p), max_new_tokens=max_new_tokens) for i, p in enumerate(prompts)]
        waiting.reverse()
        running: List[Sequence] = []
        done: Dict[object, List[int]] = {}
        while waiting or running:
            budget = max_step_tokens
            batch: List[Tuple[Sequence, List[int]]] = []
            for seq in running:
                if not seq.prompt:                               # decoding: one token each
                    batch.append((seq, [seq.last_token]))
                    budget -= 1
            for seq in running:
                if seq.prompt and budget > 0 and len(batch) < self.max_rows:
                    take = self._portion(seq, budget)
                    if take:
                        batch.append((seq, take))
                        budget -= len(take)
            while waiting and budget > 0 and len(batch) < self.max_rows and self.slots.available:
                cand = waiting[-1]
                total = -(-(len(cand.prompt) + cand.max_new_tokens) // self.page)
                held = sum(-(-(len(s.prompt) + s.length + s.max_new_tokens - len(s.output)) // self.page) - len(s.pages) for s in running)
                if total + held > self.pages.available:
                    break                                        # not enough pages to finish it: wait for a release
                waiting.pop()
                cand.slot = self.slots.take(1)[0]
                self.live[cand.rid] = cand
                running.append(cand)
                take = self._portion(cand, budget)
                batch.append((cand, take))
                budget -= len(take)
            if not batch:
                raise MemoryError("no request fits the KV cache")
            toks = self.step([(s.rid, t, ()) for s, t in batch], sample=True)
            for (seq, _), tok in zip(batch, toks):
                if seq.prompt:
                    continue                                     # mid-prompt: nothing to emit yet
                seq.output.append(tok)
                seq.last_token = tok
                if len(seq.output) >= seq.max_new_tokens or (eos_token_id is not None and tok == eos_token_id):
                    done[seq.rid] = seq.output
                    running.remove(seq)
                    self.release(seq.rid)
        return [done[("gen", i)] for i in range(len(prompts))]

    def _portion(self, seq: Sequence, budget: int) -> List[int]:
        n = min(len(seq.prompt), budget, self.max_row_tokens)
        take, seq.prompt = seq.prompt[:n], seq.prompt[n:]
        return take


def build_engine(model_path: str, dtype: str = "bfloat16", max_tokens: int = 4096, max_requests: int = 4, page_size: int = 64,
                 device: Optional[str] = None, max_portion: Optional[int] = None, sampling=None) -> PagedBatchEngine:
    """Load the checkpoint in ``model_path`` (model class chosen from its config.json) on the paged cache sized for ``max_tokens``
    live tokens (rounded up to whole pages per request) and ``max_requests`` state slots, and wrap it in an engine."""
    from ..config import NeuronConfig, OnDeviceSamplingConfig
    from ..utils.constants import get_model_cls, model_type_of
    cls = get_model_cls(model_type_of(model_path))
    dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
    mcl = max_portion or max_tokens
    ladder = [b for b in (8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384, 32768) if b < mcl] + [mcl]
    nc = cls.get_neuron_config_cls()(
        batch_size=max_requests, ctx_batch_size=max_requests, tkg_batch_size=max_requests, max_batch_size=max_requests,
        kv_cache_batch_size=max_requests, seq_len=max(max_tokens, mcl), max_context_length=mcl, torch_dtype=dtype,
        on_cpu=(dev == "cpu"), is_block_kv_layout=True, pa_block_size=page_size, pa_num_blocks=-(-max_tokens // page_size),
        enable_bucketing=True, context_encoding_buckets=ladder, is_continuous_batching=True, output_logits=True,
        on_device_sampling_config=sampling or OnDeviceSamplingConfig(top_k=1), skip_warmup=True)
    if hasattr(cls, "from_pretrained"):
        app = cls.from_pretrained(model_path, nc)
    else:
        from ..config import load_pretrained_config
        app = cls(model_path, cls.get_config_cls()(nc, load_config=load_pretrained_config(model_path)))
    app.load(None, skip_warmup=True)
    return PagedBatchEngine(app)
