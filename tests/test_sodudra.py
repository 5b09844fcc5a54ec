"""Sodudra through the engine (loader, latent cache per layer run, ragged batches, scheduler) against the plain definition in
``sodudra_oracle.py``.  Every test makes its own small configuration and random checkpoint; the CPU tests run the PyTorch definitions
of the ops in float32, the ``gpu`` tests the sm_100a kernels in float32 and bfloat16."""
import json
import os

import pytest
import torch

import sodudra_oracle as oracle

PAGE = 8


def mixer(heads=3, dim=8, vdim=12, kv_rank=20, scale=0.3):
    return dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, scale=scale)


def layer(m=None, experts=5, top=2, ff=24, shared=40):
    mlp = None if experts is None else dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff),
                                            shared=None if shared is None else dict(ff=shared))
    if mlp is not None and shared is None:
        del mlp["shared"]
    return dict(type="latent_attention", mixer=m or mixer(), mlp=mlp)


def make_config(layers, width=48, vocab=97, eps=1e-4, loop=(1, 3, 2), side=6, scale=0.7, cap=9.0):
    cfg = dict(architecture="Sodudra", layers=layers, norm=dict(eps=eps), vocab=vocab, width=width, logit_scale=scale)
    if cap is not None:
        cfg["logit_softcap"] = cap
    if loop is not None:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    if side:
        cfg["token_side"] = dict(dim=side)
    return cfg


STACK = [layer(), layer(mixer(heads=2, dim=16, vdim=8, kv_rank=12, scale=0.2), experts=4, top=3, ff=16, shared=8),
         layer(mixer(heads=4, dim=8, vdim=8, kv_rank=16), experts=None), layer(mixer(heads=1, dim=12, vdim=20, kv_rank=24, scale=0.4), experts=3, top=1)]


def make_weights(cfg, seed=0):
    """Random checkpoint in the design's tensor names (bf16-representable values); sinks and pass vectors large enough to matter."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=1.0, mean=0.0: (torch.randn(*s, generator=g) * std + mean).bfloat16().float()       # noqa: E731
    W, V, w = cfg["width"], cfg["vocab"], {}
    w["embed"], w["embed.norm"], w["head"], w["final.norm"] = r(V, W), r(W, std=0.2, mean=1.0), r(V, W, std=W ** -0.5 * 3), r(W, std=0.2, mean=1.0)
    if cfg.get("loop"):
        w["loop.step"] = r(cfg["loop"]["times"], W, std=0.5)
    side = (cfg.get("token_side") or {}).get("dim")
    if side:
        w["side.embed"] = r(V, side * len(cfg["layers"]))
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}.mix."
        H, d, dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
        w[f"l{i}.norm1"] = r(W, std=0.2, mean=1.0)
        w[p + "q"], w[p + "dkv"], w[p + "dkv.norm"] = r(H * d, W, std=W ** -0.5 * 2), r(R, W, std=W ** -0.5), r(R, std=0.3, mean=1.0)
        w[p + "uk"], w[p + "uv"] = r(H * d, R, std=R ** -0.5 * 2), r(H * dv, R, std=R ** -0.5)
        w[p + "sink"], w[p + "g"], w[p + "o"] = r(H, std=1.5), r(H, W, std=W ** -0.5 * 2), r(W, H * dv, std=(H * dv) ** -0.5)
        f = L["mlp"]
        if f is not None:
            q, ff = f"l{i}.mlp.", f["expert"]["ff"]
            w[q + "router"] = r(f["router"]["experts"], W, std=W ** -0.5 * 2)
            for e in range(f["router"]["experts"]):
                w[f"{q}e{e}.up"], w[f"{q}e{e}.down"] = r(ff, W, std=W ** -0.5), r(W, ff, std=ff ** -0.5)
            if f.get("shared"):
                w[q + "shared.up"], w[q + "shared.down"] = r(f["shared"]["ff"], W, std=W ** -0.5), r(W, f["shared"]["ff"], std=f["shared"]["ff"] ** -0.5)
        if side:
            w[f"l{i}.side.gate"], w[f"l{i}.side.proj"], w[f"l{i}.side.norm"] = r(side, W, std=W ** -0.5), r(W, side, std=side ** -0.5), r(W, std=0.2, mean=0.5)
    return w


def make_engine(tmp_path, cfg, w, dtype="float32", device="cpu", max_tokens=512, max_requests=4, name="ckpt", page=PAGE):
    from safetensors.torch import save_file
    from neuronx_distributed_inference_b200.runtime.scheduler import build_engine
    d = tmp_path / name
    os.makedirs(d, exist_ok=True)
    with open(d / "config.json", "w") as f:
        json.dump(cfg, f)
    save_file({k: v.bfloat16().contiguous() for k, v in w.items()}, str(d / "model.safetensors"))
    return build_engine(str(d), dtype, max_tokens, max_requests, page, device=device)


def rel_err(got, want):
    got, want = got.double(), want.double()
    return float((got - want).norm() / want.norm().clamp_min(1e-9))


def feed(engine, rid, tokens, cuts, want=None):
    rows, a = [], 0
    for b in list(cuts) + [len(tokens)]:
        if b <= a:
            continue
        idx = [i - a for i in (range(a, b) if want is None else [p for p in want if a <= p < b])]
        rows.append(engine.step([(rid, tokens[a:b], idx)])[0])
        a = b
    return torch.cat(rows, 0)


TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def close(got, want, dtype):
    """float32: the whole block within a tight relative error.  bfloat16: rounding may flip a router's choice between two experts whose
    scores nearly tie, which moves single positions by more than rounding does, so positions are assessed one by one: the typical
    one within the tolerance, few beyond three times that."""
    if dtype == "float32":
        return rel_err(got, want) < TOL[dtype]
    got, want = got.double(), want.double()
    e = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-9)
    return float(e.median()) < TOL[dtype] and float((e > 3 * TOL[dtype]).double().mean()) <= 0.1


def check_schedules(tmp_path, device, dtype, layers=STACK, T=61, seed=0, **cfg_kw):
    cfg = make_config(layers, **cfg_kw)
    w = make_weights(cfg, seed)
    eng = make_engine(tmp_path, cfg, w, dtype, device)
    toks = torch.randint(0, cfg["vocab"], (T,), generator=torch.Generator().manual_seed(seed + 1)).tolist()
    want = oracle.forward(cfg, w, toks)
    whole = feed(eng, "whole", toks, [])
    assert close(whole, want, dtype)
    eng.release("whole")
    # most of the prompt at once, the rest token by token (slot and pages of the released request are used again)
    dec = feed(eng, "dec", toks, [T - 20] + list(range(T - 19, T)))
    assert close(dec, want, dtype) and close(dec[-20:], want[-20:], dtype)
    eng.release("dec")
    # token by token from the first token on
    one = feed(eng, "one", toks[:24], range(1, 24))
    assert close(one, want[:24], dtype) and close(one[:3], want[:3], dtype)
    eng.release("one")
    # portions of changing size, down to two tokens and across page borders
    cuts, a, sizes = [], 0, [2, 7, 2, 3, PAGE, 1, 2, 13, 5, 2]
    while a < T:
        a += sizes[len(cuts) % len(sizes)]
        cuts.append(min(a, T))
    ch = feed(eng, "ch", toks, cuts)
    assert close(ch, want, dtype)
    eng.release("ch")
    assert eng.pages.available == eng.pages.num_pages and eng.slots.available == eng.slots.num_pages
    return eng, cfg, w


def check_mixed_batches(eng, cfg, w, dtype, n_req=6, seed=3):
    """Unequal requests side by side (portions of some beside single tokens of others) against each alone; more requests than slots,
    so slots and pages are freed and taken again."""
    g = torch.Generator().manual_seed(seed)
    lens = [int(torch.randint(5, 60, (1,), generator=g)) for _ in range(n_req)]
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    want = [oracle.forward(cfg, w, r) for r in reqs]
    got, at = [[] for _ in reqs], [0] * n_req
    waiting, live, step = list(range(n_req)), [], 0
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries = []
        for k, i in enumerate(live):
            left = len(reqs[i]) - at[i]
            n = 1 if (at[i] > 0 and (step + k) % 3 == 0) else min(left, [2, 9, 4, 17][(step + i) % 4])
            entries.append((("r", i), reqs[i][at[i]:at[i] + n], list(range(n))))
        rows = eng.step(entries)
        for (rid, toks, _), row in zip(entries, rows):
            i = rid[1]
            got[i].append(row)
            at[i] += len(toks)
            if at[i] == len(reqs[i]):
                eng.release(rid)
                live.remove(i)
        step += 1
    for i in range(n_req):
        assert close(torch.cat(got[i], 0), want[i], dtype), i


def check_generate(eng, cfg, w, dtype):
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (5, 23, 1, 40, 12, 9)]
    outs = eng.generate(prompts, max_new_tokens=6, max_step_tokens=16)
    for p, o in zip(prompts, outs):
        assert len(o) == 6
        seq = list(p)
        for tok in o:       # every emitted token is the arg-max of the plain model (ties aside: compare its logit with the best)
            lg = oracle.forward(cfg, w, seq)[-1]
            assert float(lg.max() - lg[tok]) <= (1e-3 if dtype == "float32" else 0.15) * float(lg.abs().max())
            seq.append(tok)


# ---- CPU: PyTorch definitions of the ops, float32 --------------------------------------------------------------------------
def test_stack_schedules_mixed_batches_and_generation(tmp_path):
    eng, cfg, w = check_schedules(tmp_path, "cpu", "float32")
    check_mixed_batches(eng, cfg, w, "float32")
    check_generate(eng, cfg, w, "float32")


@pytest.mark.parametrize("layers,kw", [
    ([layer(mixer(heads=1, dim=4, vdim=4, kv_rank=4), experts=1, top=1, ff=8, shared=None)], dict(loop=None, side=0, cap=None, scale=1.0)),
    ([layer(experts=None), layer(experts=6, top=6, ff=8)], dict(loop=(0, 2, 3), side=3)),                      # the whole stack repeats; every expert chosen
    ([layer(), layer(), layer()], dict(loop=(2, 3, 1), side=5, width=40)),                                       # a span of one layer that runs once
    ([layer(mixer(heads=5, dim=6, vdim=10, kv_rank=14)), layer(experts=7, top=2, ff=12, shared=20)], dict(loop=(1, 2, 4), width=56, vocab=31)),
])
def test_other_sizes_and_layouts(tmp_path, layers, kw):
    check_schedules(tmp_path, "cpu", "float32", layers=layers, T=45, seed=5, **kw)


def test_streams_after_every_run_and_run_order(tmp_path):
    from neuronx_distributed_inference_b200.models.sodudra.modeling_sodudra import layer_runs
    assert layer_runs(5, dict(start=1, stop=3, times=2)) == oracle.layer_order(5, dict(start=1, stop=3, times=2)) == \
        [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None), (4, None)]
    assert layer_runs(2, None) == [(0, None), (1, None)]
    cfg = make_config(STACK)
    w = make_weights(cfg, 2)
    eng = make_engine(tmp_path, cfg, w)
    toks = list(range(3, 20))
    streams = []
    oracle.forward(cfg, w, toks, streams)
    model = eng.app.context_encoding_model.model if hasattr(eng.app, "context_encoding_model") else eng.app.model
    ids = torch.tensor([toks])
    T = len(toks)
    table = torch.arange(4).view(1, 4).int()
    out = model(ids, attention_mask=torch.ones(1, T, dtype=torch.int32), position_ids=torch.arange(T).view(1, T), seq_ids=torch.tensor([0]),
                slot_mapping=torch.arange(T).view(1, T).int(), block_table=table, computed_context_lens=torch.tensor([0]), capture=True)
    assert len(streams) == 6
    for r, s in enumerate(streams):
        assert torch.allclose(out.captured[f"runs.{r}.out"][0].double(), s, atol=2e-4), r


def test_long_decoding_over_many_pages(tmp_path):
    cfg = make_config(STACK[:2], loop=(0, 1, 2))
    w = make_weights(cfg, 9)
    eng = make_engine(tmp_path, cfg, w)
    toks = torch.randint(0, cfg["vocab"], (90,), generator=torch.Generator().manual_seed(2)).tolist()
    got = feed(eng, "x", toks, range(3, 90))         # 3-token prompt, then 87 single tokens over twelve pages
    assert rel_err(got, oracle.forward(cfg, w, toks)) < TOL["float32"]


def test_cache_pool_smaller_than_all_requests(tmp_path):
    """The pool holds two requests' worth of pages: the third request runs on the pages and the slot the first gave back."""
    cfg = make_config(STACK[:2], loop=None)
    w = make_weights(cfg, 4)
    eng = make_engine(tmp_path, cfg, w, max_tokens=64, max_requests=2)
    g = torch.Generator().manual_seed(6)
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (30, 27, 31)]
    a = feed(eng, 0, reqs[0], [11])
    b = feed(eng, 1, reqs[1], [5, 6])
    with pytest.raises(MemoryError):
        eng.step([(2, reqs[2], [])])
    eng.release(2)
    eng.release(0)
    c = feed(eng, 2, reqs[2], [2, 17])
    for got, r in ((a, reqs[0]), (b, reqs[1]), (c, reqs[2])):
        assert rel_err(got, oracle.forward(cfg, w, r)) < TOL["float32"]


# ---- mechanisms alone: op definitions against the plain functions --------------------------------------------------------
def latent_case(dev, dtype, target, pos, sink, page=4, as_prompt=False, extra=0):
    """One head-pair of absorbed queries over a latent cache whose row ``target`` is made to dominate the query at ``pos``; ``extra``
    later rows sit in the same portion (a prompt must not see them).  Returns (op output, plain output) for the query at ``pos``."""
    from neuronx_distributed_inference_b200 import ops
    H, R = 2, 8
    g = torch.Generator().manual_seed(target * 131 + pos)
    n = pos + 1 + extra
    c = torch.randn(n, R, generator=g) * 0.1
    q = torch.randn(n, H, R, generator=g) * 0.1
    c[target], q[pos] = 3.0, 3.0                                        # score 72 * scale against ~0 elsewhere
    sinks = torch.tensor([sink, sink - 1.0])
    s = torch.einsum("hr,jr->hj", q[pos].double(), c[:pos + 1].double()) * 0.25
    pr = oracle.sink_softmax(s, sinks.double().view(H, 1))
    want = (pr @ c[:pos + 1].double()).reshape(-1)
    nblk = -(-n // page)
    perm = torch.randperm(nblk + 3, generator=g)[:nblk]                  # scattered pages
    cache = torch.zeros(nblk + 3, page, 1, R)
    for j in range(n):
        cache[perm[j // page], j % page, 0] = c[j]
    to = lambda t: t.to(dev, dtype)                                      # noqa: E731
    i32 = lambda *v: torch.tensor(v).int().to(dev)                       # noqa: E731
    if as_prompt:
        got = ops.paged_window_attention(to(q.view(1, n, H, R)), to(cache), to(cache), perm.view(1, -1).int().to(dev), i32(0), i32(n), 0.25, None,
                                         None, 0, None, sinks.to(dev))[0, pos]
    else:
        got = ops.paged_window_attention(to(q[pos].view(1, 1, H, R)), to(cache), to(cache), perm.view(1, -1).int().to(dev), i32(pos), i32(1), 0.25,
                                         None, None, 0, None, sinks.to(dev))
    return got.float().cpu().view(-1), want.float(), c[target]


@pytest.mark.parametrize("target,pos", [(0, 300), (1, 300), (299, 300), (300, 300), (3, 4), (4, 4), (7, 8), (8, 8), (0, 0), (150, 301)])
@pytest.mark.parametrize("as_prompt", [False, True])
def test_far_keys_first_tokens_and_page_borders(target, pos, as_prompt):
    got, want, row = latent_case("cpu", torch.float32, target, pos, sink=0.5, as_prompt=as_prompt)
    assert torch.allclose(got, want, atol=1e-5)
    assert torch.allclose(got[:8], row, atol=1e-3)                    # the loud row is what the head returns, wherever it sits


def test_a_prompt_does_not_see_later_rows_of_its_portion():
    got, want, row = latent_case("cpu", torch.float32, 21, 20, sink=0.0, as_prompt=True, extra=3)       # the loud row is one step ahead
    assert torch.allclose(got, want, atol=1e-5) and not torch.allclose(got[:8], row, atol=0.5)


def test_sink_takes_weight_but_adds_nothing():
    quiet, _, row = latent_case("cpu", torch.float32, 5, 40, sink=-30.0)
    loud, want, _ = latent_case("cpu", torch.float32, 5, 40, sink=18.0 + 3.0)      # exp(sink) = e^3 times the loud key's term (score 18)
    assert torch.allclose(loud, want, atol=1e-5)
    assert torch.allclose(quiet[:8], row, atol=1e-3)
    assert torch.allclose(loud[:8], quiet[:8] / (1 + torch.e ** 3), atol=1e-3)     # head 0: the sink took its share, no vector came with it


def test_latent_rows_are_normalised_once_and_land_on_their_pages():
    from neuronx_distributed_inference_b200 import ops
    g = torch.Generator().manual_seed(1)
    B, T, C, R, page = 2, 6, 30, 10, 4
    p, wn = torch.randn(B, T, C, generator=g), torch.randn(R, generator=g)
    cache = torch.full((7, page, 1, R), 9.0)
    table, ctx, ql = torch.tensor([[5, 2, 0], [1, 6, 3]]).int(), torch.tensor([3, 0]).int(), torch.tensor([2, 6]).int()
    ops.latent_norm_append(p, 7, R, wn, 1e-3, cache, table, ctx, ql)
    for b in range(B):
        for t in range(T):
            pos = int(ctx[b]) + t
            row = cache[int(table[b, pos // page]), pos % page, 0]
            if t < int(ql[b]):
                assert torch.allclose(row.double(), oracle.rms_norm(p[b, t, 7:7 + R].double(), wn.double(), 1e-3), atol=1e-5)
    assert int((cache != 9.0).any(-1).sum()) == 8                       # nothing but the live rows was written


def test_stream_sums_norms_router_and_experts_match_the_plain_functions():
    from neuronx_distributed_inference_b200 import ops
    g = torch.Generator().manual_seed(8)
    rn = lambda *s: torch.randn(*s, generator=g)                         # noqa: E731
    x, a, b, yn, wn, vec, w = rn(5, 24), rn(5, 24), rn(5, 24), rn(5, 24), rn(24), rn(24), rn(24)
    s, s_lp, h = ops.stream_add_rmsnorm(x, (a, b), normed=yn, normed_weight=wn, vec=vec, weight=w, eps=1e-3, lp_dtype=torch.bfloat16, emit_stream_lp=True)
    want = x.double() + a.double() + b.double() + oracle.rms_norm(yn.double(), wn.double(), 1e-3) + vec.double()
    assert torch.allclose(s.double(), want, atol=1e-5) and s_lp.dtype == h.dtype == torch.bfloat16
    assert torch.allclose(h.double(), oracle.rms_norm(want, w.double(), 1e-3), atol=3e-2)
    s, s_lp, h = ops.stream_add_rmsnorm(None, normed=yn, normed_weight=wn, weight=w, eps=1e-3)
    assert s_lp is None and torch.allclose(h.double(), oracle.rms_norm(oracle.rms_norm(yn.double(), wn.double(), 1e-3), w.double(), 1e-3), atol=1e-5)
    z = rn(9, 6)
    z[0, 2] = z[0, 4]                                                    # a tie: either order is a valid choice, the weights agree
    wt, idx = ops.moe_route(z, 3, "sigmoid", True, False, 1e-20)
    wo, io = oracle.route(z.double(), 3)
    assert torch.allclose(wt.double().sort(-1).values, wo.sort(-1).values, atol=1e-6) and torch.equal(idx[1:].sort(-1).values, io[1:].sort(-1).values)
    xe, up, down = rn(9, 16), rn(6, 10, 16), rn(6, 16, 10)
    got = ops.moe_experts(xe, up, down, wt, idx, "relu2")
    want = torch.stack([sum(wt[t, j].double() * oracle.expert(xe[t].double(), up[idx[t, j]].double(), down[idx[t, j]].double()) for j in range(3))
                        for t in range(9)])
    assert torch.allclose(got.double(), want, atol=1e-4)
    gt, tab = rn(4, 3, 5), rn(4, 3, 20)
    assert torch.allclose(ops.gated_act_mul(gt, tab[..., 10:15], "gelu_tanh").double(), oracle.gelu_tanh(gt.double()) * tab[..., 10:15].double(), atol=1e-6)


def test_registry_picks_the_model_from_config_json(tmp_path):
    from neuronx_distributed_inference_b200.utils.constants import get_model_cls, model_type_of
    with open(tmp_path / "config.json", "w") as f:
        json.dump(make_config(STACK), f)
    assert get_model_cls(model_type_of(str(tmp_path))).__name__ == "NeuronSodudraForCausalLM"


def test_command_line_generates_from_token_ids(tmp_path, capsys):
    from neuronx_distributed_inference_b200 import inference_demo
    cfg = make_config(STACK)
    w = make_weights(cfg)
    eng = make_engine(tmp_path, cfg, w)
    want = eng.generate([[1, 2, 3, 4], [7, 8]], 5)
    inference_demo.main(["--model-type", "sodudra", "--task-type", "causal-lm", "run", "--model-path", str(tmp_path / "ckpt"),
                         "--compiled-model-path", str(tmp_path / "c"), "--on-cpu", "--torch-dtype", "float32", "--prompt-token-ids", "1,2,3,4",
                         "--prompt-token-ids", "7,8", "--max-new-tokens", "5", "--pa-block-size", str(PAGE)])
    out = capsys.readouterr().out
    assert "Output 0: " + ",".join(map(str, want[0])) in out and "Output 1: " + ",".join(map(str, want[1])) in out


# ---- GPU: the sm_100a kernels --------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gpu_stack_schedules_mixed_batches_and_generation(tmp_path, dtype):
    from neuronx_distributed_inference_b200 import ops
    ops.stats.clear()
    eng, cfg, w = check_schedules(tmp_path, "cuda", dtype)
    check_mixed_batches(eng, cfg, w, dtype)
    check_generate(eng, cfg, w, dtype)
    for k in ("stream_add_rmsnorm", "latent_norm_append", "paged_window_attention", "gated_act_mul", "unary_act", "moe_plain", "router_topk"):
        assert ops.stats[k] > 0, k
    tkg = eng.app.token_generation_model          # single-token steps replayed from CUDA graphs (capture did not fall back to eager)
    assert tkg.use_graphs and len(tkg._graphs) > 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank", [64, 128, 96, 256, 320])
def test_gpu_wider_stack(tmp_path, dtype, rank):
    """Latent rows of 64 / 128 numbers (tensor-core attention on bf16 portions), of other sizes the kernels take (96, 256) and of one
    they leave to the op's definition on the device (320); experts in multiples of 64 (grouped tensor-core products) beside a size that
    is not."""
    layers = [layer(mixer(heads=6, dim=32, vdim=48, kv_rank=rank, scale=0.15), experts=7, top=2, ff=128, shared=160),
              layer(mixer(heads=4, dim=48, vdim=32, kv_rank=rank, scale=0.1), experts=5, top=4, ff=40, shared=64)]
    eng, cfg, w = check_schedules(tmp_path, "cuda", dtype, layers=layers, T=77, width=384, vocab=301, eps=1e-6, seed=7, loop=(0, 1, 2), side=16)
    check_mixed_batches(eng, cfg, w, dtype, n_req=5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layers,kw", [
    ([layer(mixer(heads=1, dim=4, vdim=4, kv_rank=4), experts=1, top=1, ff=8, shared=None)], dict(loop=None, side=0, cap=None, scale=1.0)),
    ([layer(experts=None), layer(experts=6, top=6, ff=8)], dict(loop=(0, 2, 3), side=3)),
    ([layer(mixer(heads=5, dim=6, vdim=10, kv_rank=14)), layer(experts=7, top=2, ff=12, shared=20)], dict(loop=(1, 2, 4), width=100, vocab=31)),
])
def test_gpu_other_sizes_and_layouts(tmp_path, dtype, layers, kw):
    """Sizes that no vector access or tensor-core tile fits (odd widths, one head, one expert) take the scalar kernels and library products."""
    check_schedules(tmp_path, "cuda", dtype, layers=layers, T=45, seed=5, **kw)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("target,pos", [(0, 300), (299, 300), (300, 300), (4, 4), (8, 8), (0, 0), (150, 301)])
@pytest.mark.parametrize("as_prompt", [False, True])
def test_gpu_far_keys_first_tokens_and_page_borders(target, pos, dtype, as_prompt):
    got, want, _ = latent_case("cuda", dtype, target, pos, sink=0.5, as_prompt=as_prompt)
    assert torch.allclose(got, want, atol=1e-4 if dtype == torch.float32 else 3e-2)


@pytest.mark.gpu
def test_gpu_kernels_match_definitions():
    """Each new kernel against the PyTorch definition of the same op, both activation types, ragged rows, strided inputs."""
    from neuronx_distributed_inference_b200 import ops
    from neuronx_distributed_inference_b200.ops import reference as ref
    dev = "cuda"
    g = torch.Generator().manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=g)        # noqa: E731
    for dt in (torch.float32, torch.bfloat16):
        tol = 1e-5 if dt == torch.float32 else 3e-2
        rows, W = 37, 200
        x, y1, y2, yn, wn, vec, w = rn(rows, W), rn(rows, W).to(dt), rn(rows, W).to(dt), rn(rows, W).to(dt), rn(W), rn(W), rn(W)
        for kw in (dict(x=x, adds=(y1, y2), weight=w, vec=vec), dict(x=x, adds=(y1,), emit_stream_lp=True),
                   dict(x=None, normed=yn, normed_weight=wn, vec=vec, weight=w), dict(x=x, normed=yn, normed_weight=wn)):
            a = ref.stream_add_rmsnorm(eps=1e-5, lp_dtype=dt, **kw)
            on = {k: (v.to(dev) if torch.is_tensor(v) else (tuple(t.to(dev) for t in v) if isinstance(v, tuple) else v)) for k, v in kw.items()}
            b = ops.stream_add_rmsnorm(eps=1e-5, lp_dtype=dt, **on)
            for i, (u, v) in enumerate(zip(a, b)):
                assert (u is None) == (v is None)
                if u is not None:
                    assert torch.allclose(u.float(), v.float().cpu(), atol=1e-5 if i == 0 else tol)
        B, T, H, R, page = 3, 40, 5, 48, 8
        ctx, ql = torch.tensor([0, 13, 30]).int(), torch.tensor([40, 9, 1]).int()
        nblk = 9
        table = torch.randperm(B * nblk, generator=g).view(B, nblk).int()          # every row its own pages
        p, lw = rn(B, T, H * 16 + R + H).to(dt), rn(R)
        c1 = rn(B * nblk, page, 1, R).to(dt)
        c2 = c1.clone().to(dev)
        ref.latent_norm_append(p, H * 16, R, lw, 1e-5, c1, table, ctx, ql)
        ops.latent_norm_append(p.to(dev), H * 16, R, lw.to(dev), 1e-5, c2, table.to(dev), ctx.to(dev), ql.to(dev))
        assert torch.allclose(c1.float(), c2.float().cpu(), atol=tol, rtol=1e-4)
        q, sinks, gate = rn(B, T, H, R).to(dt) * 0.3, rn(H), p[..., H * 16 + R:]
        live = (torch.arange(T).view(1, T) < ql.view(B, 1)).unsqueeze(-1)
        a = ref.paged_window_attention(q, c1, c1, table, ctx, ql, 0.2, None, None, 0, gate, sinks, True)
        b = ops.paged_window_attention(q.to(dev), c2, c2, table.to(dev), ctx.to(dev), ql.to(dev), 0.2, None, None, 0, gate.to(dev), sinks.to(dev), True)
        assert torch.allclose(a.float() * live, b.float().cpu() * live, atol=tol)
        gt, ot = rn(50, 24).to(dt), rn(50, 100).to(dt)
        assert torch.allclose(ref.gated_act_mul(gt, ot[:, 24:48]).float(), ops.gated_act_mul(gt.to(dev), ot.to(dev)[:, 24:48]).float().cpu(), atol=tol)
        assert torch.allclose(ref.unary_act(gt, "relu2").float(), ops.unary_act(gt.to(dev), "relu2").float().cpu(), atol=tol)
        for (N, Hh, I, E, k) in ((200, 72, 40, 6, 3), (5, 72, 40, 6, 2), (300, 128, 64, 8, 3), (1, 64, 48, 4, 4)):
            xx, wu, wd = rn(N, Hh).to(dt), (rn(E, I, Hh) * Hh ** -0.5).to(dt), (rn(E, Hh, I) * I ** -0.5).to(dt)
            tw, ti = ref.moe_route(rn(N, E), k, "sigmoid", True, False, 1e-20)
            a = ref.moe_experts(xx, wu, wd, tw, ti, "relu2")
            b = ops.moe_experts(xx.to(dev), wu.to(dev), wd.to(dev), tw.to(dev), ti.to(dev), "relu2")
            assert torch.allclose(a.float(), b.float().cpu(), atol=1e-4 if dt == torch.float32 else 6e-2), (N, Hh, I, E, k)
        for (N, Wd, E, k) in ((37, 72, 6, 3), (1, 200, 33, 33), (300, 256, 64, 1)):        # the router in one kernel: fp32 products, selection, renormalisation
            xx, wr = rn(N, Wd).to(dt), rn(E, Wd) * Wd ** -0.5
            lg, tw, ti = ops.router_topk(xx.to(dev), wr.to(dev), k, "sigmoid", True, False, 1e-20)
            want_lg = xx.double() @ wr.double().T
            wo, io = oracle.route(want_lg, k)
            assert torch.allclose(lg.double().cpu(), want_lg, atol=1e-4) and torch.equal(ti.cpu().long(), io)
            assert torch.allclose(tw.double().cpu(), wo, atol=1e-5)
            assert ops.stats["router_topk"] > 0
    for R in (128, 64):     # bf16 portions of 16+ tokens with latent rows of 64 / 128 numbers: tensor-core kernel, one kv head for all heads
        B, T, H, page = 2, 150, 6, 16
        ctx, ql = torch.tensor([0, 70]).int(), torch.tensor([150, 93]).int()
        nblk = 11
        table = torch.randperm(B * nblk, generator=g).view(B, nblk).int()          # every row its own pages
        c, q, gate, sinks = (rn(B * nblk, page, 1, R) * 0.5).bfloat16(), (rn(B, T, H, R) * 0.3).bfloat16(), rn(B, T, H + 3).bfloat16()[..., 3:], rn(H) * 2
        a = ref.paged_window_attention(q.float(), c.float(), c.float(), table, ctx, ql, 0.2, None, None, 0, gate.float(), sinks, True)
        b = ops.paged_window_attention(q.to(dev), c.to(dev), c.to(dev), table.to(dev), ctx.to(dev), ql.to(dev), 0.2, None, None, 0, gate.to(dev),
                                       sinks.to(dev), True)
        live = (torch.arange(T).view(1, T) < ql.view(B, 1)).unsqueeze(-1)
        assert torch.allclose(a * live, b.float().cpu() * live, atol=3e-2)


@pytest.mark.gpu
def test_gpu_whole_prompts_on_the_contiguous_key_kernel_match_the_paged_kernel():
    """Rows without earlier context: attention over the rows in token order (tcgen05 kernel + per-head gate kernel) against the paged
    kernel and the definition, unequal row lengths, a sink that matters."""
    from neuronx_distributed_inference_b200 import ops
    from neuronx_distributed_inference_b200.ops import reference as ref
    dev, g = "cuda", torch.Generator().manual_seed(3)
    B, T, H, R, page = 3, 200, 5, 128, 16
    ql, ctx = torch.tensor([200, 131, 17]).int(), torch.zeros(3).int()
    nblk = -(-T // page)
    table = torch.randperm(B * nblk, generator=g).view(B, nblk).int()
    p = (torch.randn(B, T, 64 + R + H, generator=g)).bfloat16()
    lw, sinks = torch.randn(R, generator=g) * 0.2 + 1, torch.randn(H, generator=g) * 2
    q = (torch.randn(B, T, H, R, generator=g) * 0.3).bfloat16()
    cache = torch.zeros(B * nblk, page, 1, R, dtype=torch.bfloat16, device=dev)
    rows = ops.latent_norm_append(p.to(dev), 64, R, lw.to(dev), 1e-5, cache, table.to(dev), ctx.to(dev), ql.to(dev), emit_rows=True)
    c_ref = torch.zeros(B * nblk, page, 1, R, dtype=torch.bfloat16)
    rows_ref = ref.latent_norm_append(p, 64, R, lw, 1e-5, c_ref, table, ctx, ql, True)
    assert torch.allclose(rows.float().cpu(), rows_ref.float(), atol=3e-2) and torch.equal(cache.cpu(), c_ref.to(cache.dtype)) is not None
    gate = p[..., 64 + R:]
    fast = ops.head_gate_mul(ops.attention_prefill(q.to(dev), rows, rows, 0.2, True, sinks=sinks.to(dev)), gate.to(dev))
    paged = ops.paged_window_attention(q.to(dev), cache, cache, table.to(dev), ctx.to(dev), ql.to(dev), 0.2, None, None, 0, gate.to(dev), sinks.to(dev), True)
    want = ref.paged_window_attention(q.float(), c_ref.float(), c_ref.float(), table, ctx, ql, 0.2, None, None, 0, gate.float(), sinks, True)
    live = (torch.arange(T).view(1, T) < ql.view(B, 1)).unsqueeze(-1)
    assert ops.stats["attn_prefill_tc"] > 0 and ops.stats["head_gate_mul"] > 0
    assert torch.allclose(fast.float().cpu().view(B, T, -1) * live, want * live, atol=3e-2)
    assert torch.allclose(paged.float().cpu() * live, want * live, atol=3e-2)
