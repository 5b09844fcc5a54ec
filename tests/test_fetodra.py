"""Fetodra through the engine (loader, paged cache, state lines, ragged batches, scheduler) against the plain definition in
``fetodra_oracle.py``.  Every test makes its own small configuration and random checkpoint; the CPU tests run the PyTorch
definitions of the ops in float32, the ``gpu`` tests the sm_100a kernels in float32 and bfloat16."""
import json
import math
import os

import pytest
import torch

import fetodra_oracle as oracle

PAGE = 8


def attn(heads=4, kv_heads=2, dim=16, vdim=8, conv=4, rot=8, base=500.0, scale=0.3, softcap=5.0, window=9, keep=3, kv_from=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, rot=dict(dims=rot, base=base), scale=scale, softcap=softcap,
             mask=dict(size=window, keep_first=keep))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mamba(heads=4, vdim=12, state=8, groups=2, norm_groups=2, conv=2):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=norm_groups, conv=conv)


def layer(kind, mixer, ff=48, limit=0.7):
    return dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff, limit=limit))


def make_config(layers, width=64, vocab=97, alpha=1.5, eps=1e-4):
    return dict(architecture="Fetodra", layers=layers, norm=dict(eps=eps), postln_alpha=alpha, vocab=vocab, width=width)


HYBRID = [layer("mamba2", mamba()), layer("attention", attn()), layer("attention", attn(kv_from=1), ff=None),
          layer("mamba2", mamba(heads=2, vdim=16, state=16, groups=1, norm_groups=1, conv=4), ff=None),
          layer("attention", attn(heads=3, kv_heads=1, dim=8, vdim=16, conv=2, rot=8, window=5, keep=0, softcap=2.0, scale=0.5)),
          layer("attention", attn(kv_from=1))]


def make_weights(cfg, seed=0):
    """Random checkpoint in the design's tensor names (bf16-representable values)."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=1.0, mean=0.0: (torch.randn(*s, generator=g) * std + mean).bfloat16().float()       # noqa: E731
    W, w = cfg["width"], {}
    w["embed"], w["head"], w["final.norm"] = r(cfg["vocab"], W), r(cfg["vocab"], W, std=W ** -0.5), r(W, std=0.2)
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}.mix."
        w[f"l{i}.norm1"] = r(W, std=0.2)
        if L["type"] == "attention":
            Cq, Ck, Cv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            names = [("q", Cq)] + ([("k", Ck), ("v", Cv)] if m.get("kv_from") is None else [])
            for n, C in names:
                w[p + n], w[p + n + ".b"], w[p + n + ".conv"] = r(C, W, std=W ** -0.5), r(C, std=0.3), r(C, m["conv"], std=0.6)
            w[p + "q.norm"] = r(Cq, std=0.3, mean=1.0)
            if m.get("kv_from") is None:
                w[p + "k.norm"] = r(Ck, std=0.3, mean=1.0)
            w[p + "g"], w[p + "o"] = r(m["heads"] * m["vdim"], W, std=W ** -0.5), r(W, m["heads"] * m["vdim"], std=(m["heads"] * m["vdim"]) ** -0.5)
        else:
            inner, GN = m["heads"] * m["vdim"], m["groups"] * m["state"]
            w[p + "in"] = r(2 * inner + 2 * GN + m["heads"], W, std=W ** -0.5)
            w[p + "conv"], w[p + "conv.b"] = r(inner + 2 * GN, m["conv"], std=0.6), r(inner + 2 * GN, std=0.2)
            w[p + "dt_bias"], w[p + "A_log"], w[p + "D"] = r(m["heads"], mean=-1.0), r(m["heads"], mean=-1.0), r(m["heads"], std=0.3, mean=1.0)
            w[p + "norm"], w[p + "o"] = r(inner, std=0.2, mean=1.0), r(W, inner, std=inner ** -0.5)
        if L["mlp"] is not None:
            f = L["mlp"]["ff"]
            w[f"l{i}.norm2"] = r(W, std=0.2)
            w[f"l{i}.mlp.gate"], w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"] = r(f, W, std=W ** -0.5), r(f, W, std=W ** -0.5), r(W, f, std=f ** -0.5)
    return w


def make_engine(tmp_path, cfg, w, dtype="float32", device="cpu", max_tokens=512, max_requests=4, name="ckpt"):
    from safetensors.torch import save_file
    from neuronx_distributed_inference_b200.runtime.scheduler import build_engine
    d = tmp_path / name
    os.makedirs(d, exist_ok=True)
    with open(d / "config.json", "w") as f:
        json.dump(cfg, f)
    save_file({k: v.bfloat16().contiguous() for k, v in w.items()}, str(d / "model.safetensors"))
    return build_engine(str(d), dtype, max_tokens, max_requests, PAGE, device=device)


def rel_err(got, want):
    got, want = got.double(), want.double()
    return float((got - want).norm() / want.norm().clamp_min(1e-9))


def feed(engine, rid, tokens, cuts, want=None):
    """Feed ``tokens`` in portions ending at ``cuts``; returns logits at every position (or those in ``want``)."""
    rows, a = [], 0
    for b in list(cuts) + [len(tokens)]:
        if b <= a:
            continue
        idx = [i - a for i in (range(a, b) if want is None else [p for p in want if a <= p < b])]
        rows.append(engine.step([(rid, tokens[a:b], idx)])[0])
        a = b
    return torch.cat(rows, 0)


TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def check_schedules(tmp_path, device, dtype, layers=HYBRID, T=61, seed=0, **cfg_kw):
    cfg = make_config(layers, **cfg_kw)
    w = make_weights(cfg, seed)
    eng = make_engine(tmp_path, cfg, w, dtype, device)
    g = torch.Generator().manual_seed(seed + 1)
    toks = torch.randint(0, cfg["vocab"], (T,), generator=g).tolist()
    want = oracle.forward(cfg, w, toks)
    tol = TOL[dtype]
    whole = feed(eng, "whole", toks, [])
    assert rel_err(whole, want) < tol
    eng.release("whole")
    # most of the prompt at once, the rest token by token (slot and pages of the released request are used again)
    dec = feed(eng, "dec", toks, [T - 20] + list(range(T - 19, T)))
    assert rel_err(dec, want) < tol
    assert rel_err(dec[-20:], want[-20:]) < tol
    eng.release("dec")
    # token by token from the first token on
    one = feed(eng, "one", toks[:24], range(1, 24))
    assert rel_err(one, want[:24]) < tol
    eng.release("one")
    # portions of changing size, down to two tokens and across page borders
    cuts, a, sizes = [], 0, [2, 7, 2, 3, PAGE, 1, 2, 13, 5, 2]
    while a < T:
        a += sizes[len(cuts) % len(sizes)]
        cuts.append(min(a, T))
    ch = feed(eng, "ch", toks, cuts)
    assert rel_err(ch, want) < tol
    eng.release("ch")
    assert eng.pages.available == eng.pages.num_pages and eng.slots.available == eng.slots.num_pages
    return eng, cfg, w


def check_mixed_batches(eng, cfg, w, dtype, n_req=6, seed=3):
    """Unequal requests side by side (portions of some beside single tokens of others) against each alone; more requests than
    slots, so slots and pages are freed and taken again."""
    g = torch.Generator().manual_seed(seed)
    lens = [int(torch.randint(5, 60, (1,), generator=g)) for _ in range(n_req)]
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    want = [oracle.forward(cfg, w, r) for r in reqs]
    got = [[] for _ in reqs]
    at = [0] * n_req
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
        assert rel_err(torch.cat(got[i], 0), want[i]) < TOL[dtype], i


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
def test_hybrid_stack_schedules_mixed_batches_and_generation(tmp_path):
    eng, cfg, w = check_schedules(tmp_path, "cpu", "float32")
    check_mixed_batches(eng, cfg, w, "float32")
    check_generate(eng, cfg, w, "float32")


@pytest.mark.parametrize("layers", [
    [layer("attention", attn(heads=2, kv_heads=2, dim=8, vdim=8, conv=1, rot=8, window=4, keep=2))],          # no convolution, full rotation
    [layer("attention", attn(heads=4, kv_heads=1, dim=12, vdim=4, conv=3, rot=4, window=200, keep=0, softcap=50.0), ff=None)],   # window never reached
    [layer("mamba2", mamba(heads=3, vdim=5, state=6, groups=3, norm_groups=3, conv=3))],
    [layer("mamba2", mamba(heads=4, vdim=8, state=4, groups=1, norm_groups=4, conv=1), ff=None)],
])
def test_single_mixer_stacks(tmp_path, layers):
    check_schedules(tmp_path, "cpu", "float32", layers=layers, T=45, width=32, vocab=53, alpha=1.0, eps=1e-5, seed=5)


def test_long_decoding_past_window_and_kept_tokens(tmp_path):
    cfg = make_config([layer("attention", attn(window=6, keep=2)), layer("mamba2", mamba())], alpha=2.5)
    w = make_weights(cfg, 9)
    eng = make_engine(tmp_path, cfg, w)
    toks = torch.randint(0, cfg["vocab"], (70,), generator=torch.Generator().manual_seed(2)).tolist()
    got = feed(eng, "x", toks, range(3, 70))         # 3-token prompt, then 67 single tokens over eight pages
    assert rel_err(got, oracle.forward(cfg, w, toks)) < TOL["float32"]


# ---- mechanisms alone: op definitions against the plain functions --------------------------------------------------------
def _ragged(B=3):
    return torch.tensor([0, 5, 11]), torch.tensor([7, 1, 4]), torch.tensor([2, 0, 1])       # ctx_len, q_len, state lines


def test_short_conv_portions_match_one_pass():
    from neuronx_distributed_inference_b200 import ops
    C, K, T = 6, 4, 19
    u, wt, bias = torch.randn(T, C), torch.randn(C, K), torch.randn(C)
    want = oracle.short_causal_conv(u.double(), wt.double(), bias.double())
    state = torch.randn(3, K - 1, C)                 # stale contents of a reused line must not leak into a new sequence
    line, got, a = torch.tensor([1]), [], 0
    for n in (2, 1, 1, 5, 2, 8):
        part = torch.zeros(1, 8, C)
        part[0, :n] = u[a:a + n]
        ctx, ql = torch.tensor([a]), torch.tensor([n])
        got.append(ops.short_conv(part, wt, bias, state, line, ctx, ql)[0, :n])
        ops.short_conv_update(part, state, line, ctx, ql)
        a += n
    assert torch.allclose(torch.cat(got).double(), want, atol=1e-5)


def test_rotation_pairs_and_partial_width():
    from neuronx_distributed_inference_b200.ops import reference as ref
    x, pos = torch.randn(5, 2, 8, dtype=torch.float64), torch.tensor([0, 1, 7, 300, 4000])
    want = oracle.rotate_interleaved(x, pos, 4, 100.0)
    ang = pos.double()[:, None] * (100.0 ** (-torch.arange(0, 4, 2).double() / 4))
    got = ref.rope_partial_interleaved(x.unsqueeze(0), torch.cos(ang).unsqueeze(0), torch.sin(ang).unsqueeze(0))[0]
    assert torch.allclose(got, want.float(), atol=1e-6) and torch.equal(got[..., 4:], x[..., 4:].float())


def window_case(dev, dtype, target, pos, window, keep, page=4, as_prompt=False):
    """One query at ``pos`` whose key at ``target`` is made to dominate: returns (op output, plain output)."""
    from neuronx_distributed_inference_b200 import ops
    H, G, D, Dv = 2, 1, 8, 4
    g = torch.Generator().manual_seed(target * 131 + pos)
    n = pos + 1
    k, v = torch.randn(n, G, D, generator=g) * 0.1, torch.randn(n, G, Dv, generator=g)
    q = torch.randn(n, H, D, generator=g) * 0.1
    k[target], q[pos] = 3.0, 3.0                                        # score 72 * scale against ~0 elsewhere
    want = oracle.softcapped_window_attention(q.double(), k.double(), v.double(), 0.25, 40.0, window, keep)[pos]
    nblk = -(-n // page)
    perm = torch.randperm(nblk + 3, generator=g)[:nblk]                  # scattered pages
    kc, vc = torch.zeros(nblk + 3, page, G, D), torch.zeros(nblk + 3, page, G, Dv)
    for j in range(n):
        kc[perm[j // page], j % page], vc[perm[j // page], j % page] = k[j], v[j]
    to = lambda t: t.to(dev, dtype)                                      # noqa: E731
    if as_prompt:        # all positions 0 .. pos in one portion; the last row is the query under test
        got = ops.paged_window_attention(to(q.view(1, n, H, D)), to(kc), to(vc), perm.view(1, -1).int().to(dev), torch.tensor([0]).int().to(dev),
                                         torch.tensor([n]).int().to(dev), 0.25, 40.0, window, keep)[0, -1]
    else:                # decoded alone against the cache
        got = ops.paged_window_attention(to(q[pos].view(1, 1, H, D)), to(kc), to(vc), perm.view(1, -1).int().to(dev),
                                         torch.tensor([pos]).int().to(dev), torch.tensor([1]).int().to(dev), 0.25, 40.0, window, keep)
    return got.float().cpu().view(-1), want.float()


@pytest.mark.parametrize("target,pos,visible", [(0, 90, True), (2, 90, True), (3, 90, False), (90 - 11, 90, True), (90 - 12, 90, False),
                                                (40, 90, False), (15, 16, True), (4, 15, True), (3, 15, False), (7, 8, True)])
@pytest.mark.parametrize("as_prompt", [False, True])
def test_window_edges_kept_tokens_and_page_borders(target, pos, visible, as_prompt):
    got, want = window_case("cpu", torch.float32, target, pos, window=12, keep=3, as_prompt=as_prompt)
    assert torch.allclose(got, want, atol=1e-5)
    # the dominant key decides the output exactly when it is visible
    got_far, _ = window_case("cpu", torch.float32, target, pos, window=10 ** 6, keep=0, as_prompt=as_prompt)
    assert (torch.allclose(got, got_far, atol=1e-3)) == visible


def test_norms_and_gate_product_match_the_plain_functions():
    from neuronx_distributed_inference_b200 import ops
    g = torch.Generator().manual_seed(8)
    x, y, wn = torch.randn(5, 24, generator=g), torch.randn(5, 24, generator=g), torch.randn(24, generator=g) * 0.2
    out, lp = ops.scaled_add_rmsnorm(x, y, wn, 1.7, 1e-3, 1.0, torch.bfloat16)
    want = oracle.offset_rms_norm(1.7 * x.double() + y.double(), wn.double(), 1e-3)
    assert torch.allclose(out.double(), want, atol=1e-5) and lp.dtype == torch.bfloat16 and torch.allclose(lp.double(), want, atol=2e-2)
    yv, wg = torch.randn(5, 24, generator=g), torch.randn(24, generator=g)
    want = oracle.rms_unit(yv.double().view(5, 3, 8), 1e-3).reshape(5, 24) * wg.double()
    assert torch.allclose(ops.group_rmsnorm(yv, wg, 3, 1e-3).double(), want, atol=1e-5)
    W, F = 6, 10
    h, wt = torch.randn(4, W, generator=g).double() * 2, {"gate": torch.randn(F, W, generator=g).double(), "up": torch.randn(F, W, generator=g).double(),
                                                         "down": torch.eye(F).double()}
    gu = torch.cat([h @ wt["gate"].T, h @ wt["up"].T], -1)
    assert (gu.abs() > 0.9).any()                                        # both clamps bite
    assert torch.allclose(ops.clamped_glu(gu.float(), 0.9, 1.702).double(), oracle.clamped_glu(h, wt, "", dict(limit=0.9)), atol=1e-5)


def test_scan_state_carries_across_portions_and_reused_lines():
    from neuronx_distributed_inference_b200 import ops
    m = mamba(heads=2, vdim=3, state=4, groups=1, norm_groups=1, conv=2)
    nh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, T = nh * P, 13
    g = torch.Generator().manual_seed(4)
    xBC, dt, z = torch.randn(T, inner + 2 * G * N, generator=g), torch.randn(T, nh, generator=g), torch.randn(T, inner, generator=g)
    A_log, dtb, Dk = torch.randn(nh, generator=g), torch.randn(nh, generator=g), torch.randn(nh, generator=g)
    S, ys = torch.zeros(nh, N, P, dtype=torch.float64), []
    for t in range(T):                                                   # the recurrence written out
        for h in range(nh):
            step = math.log1p(math.exp(float(dt[t, h] + dtb[h])))
            x, Bv, Cv = xBC[t, h * P:(h + 1) * P].double(), xBC[t, inner:inner + N].double(), xBC[t, inner + N:].double()
            S[h] = math.exp(-math.exp(float(A_log[h])) * step) * S[h] + step * torch.outer(Bv, x)
            ys.append(S[h].T @ Cv + float(Dk[h]) * x)
    want = torch.stack(ys).view(T, inner) * torch.nn.functional.silu(z.double())
    state = torch.randn(2, nh, N, P)                                     # stale line
    got, a = [], 0
    for n in (1, 4, 2, 6):
        pad = lambda t: torch.cat([t[a:a + n], torch.zeros(7 - n, t.shape[1])]).unsqueeze(0)          # noqa: E731
        got.append(ops.ssd_scan(pad(xBC), pad(dt), pad(z), A_log, dtb, Dk, state, torch.tensor([1]), torch.tensor([a]), torch.tensor([n]),
                                nh, P, N, G)[0, :n])
        a += n
    assert torch.allclose(torch.cat(got).double(), want, atol=1e-4)
    assert torch.allclose(state[1].double(), S, atol=1e-4)


def test_registry_picks_the_model_from_config_json(tmp_path):
    from neuronx_distributed_inference_b200.utils.constants import get_model_cls, model_type_of
    with open(tmp_path / "config.json", "w") as f:
        json.dump(make_config(HYBRID), f)
    assert get_model_cls(model_type_of(str(tmp_path))).__name__ == "NeuronFetodraForCausalLM"


def test_pools_hand_pages_back():
    from neuronx_distributed_inference_b200.runtime.scheduler import PagePool
    p = PagePool(5)
    a = p.take(3)
    assert a == [0, 1, 2] and p.available == 2
    p.give([1])
    assert p.take(2) == [1, 3]
    with pytest.raises(MemoryError):
        p.take(2)


# ---- GPU: the sm_100a kernels --------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gpu_hybrid_stack_schedules_mixed_batches_and_generation(tmp_path, dtype):
    from neuronx_distributed_inference_b200 import ops
    ops.stats.clear()
    eng, cfg, w = check_schedules(tmp_path, "cuda", dtype)
    check_mixed_batches(eng, cfg, w, dtype)
    check_generate(eng, cfg, w, dtype)
    for k in ("scaled_add_rmsnorm", "short_conv", "short_conv_update", "conv_qknorm_rope_append", "paged_window_attention", "ssd_scan",
              "group_rmsnorm", "clamped_glu"):
        assert ops.stats[k] > 0, k
    tkg = eng.app.token_generation_model          # single-token steps replayed from CUDA graphs (capture did not fall back to eager)
    assert tkg.use_graphs and len(tkg._graphs) > 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gpu_wider_stack(tmp_path, dtype):
    """Head sizes with 16-byte rows (vector loads), more heads than a warp's value lanes need, several norm groups."""
    layers = [layer("attention", attn(heads=6, kv_heads=2, dim=64, vdim=96, conv=4, rot=16, window=20, keep=4, softcap=20.0, scale=0.1), ff=320),
              layer("mamba2", mamba(heads=8, vdim=40, state=48, groups=2, norm_groups=4, conv=4), ff=None),
              layer("attention", attn(heads=6, kv_heads=2, dim=64, vdim=96, conv=4, rot=16, window=20, keep=4, softcap=20.0, scale=0.1, kv_from=0),
                    ff=320)]
    eng, cfg, w = check_schedules(tmp_path, "cuda", dtype, layers=layers, T=77, width=256, vocab=301, alpha=1.25, eps=1e-6, seed=7)
    check_mixed_batches(eng, cfg, w, dtype, n_req=5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("target,pos", [(0, 90), (2, 90), (3, 90), (79, 90), (78, 90), (40, 90), (15, 16), (7, 8)])
def test_gpu_window_edges(target, pos, dtype):
    got, want = window_case("cuda", dtype, target, pos, window=12, keep=3)
    assert torch.allclose(got, want, atol=1e-4 if dtype == torch.float32 else 3e-2)


@pytest.mark.gpu
def test_gpu_kernels_match_definitions_on_ragged_rows():
    """Each kernel against the PyTorch definition of the same op (fp32), rows of unequal length and stale state lines."""
    from neuronx_distributed_inference_b200 import ops
    from neuronx_distributed_inference_b200.ops import reference as ref
    dev = "cuda"
    g = torch.Generator().manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=g)        # noqa: E731
    ctx, ql, lines = (t.int() for t in _ragged())
    B, T = 3, 8
    for dt in (torch.float32, torch.bfloat16):
        tol = 1e-5 if dt == torch.float32 else 2e-2
        C, K = 40, 3
        u, wt, bias, st = rn(B, T, C + 5).to(dt), rn(C, K), rn(C), rn(4, K - 1, C).to(dt)
        cpu = ref.short_conv(u[..., 2:2 + C], wt, bias, st.clone(), lines, ctx, ql, True)
        gpu = ops.short_conv(u.to(dev)[..., 2:2 + C], wt.to(dev), bias.to(dev), st.to(dev), lines.to(dev), ctx.to(dev), ql.to(dev), True)
        live = (torch.arange(T).view(1, T) < ql.view(B, 1)).unsqueeze(-1)
        assert torch.allclose(gpu.cpu() * live, cpu * live, atol=tol)
        s1, s2 = st.clone(), st.clone().to(dev)
        ref.short_conv_update(u[..., 2:2 + C], s1, lines, ctx, ql)
        ops.short_conv_update(u.to(dev)[..., 2:2 + C], s2, lines.to(dev), ctx.to(dev), ql.to(dev))
        assert torch.equal(s1, s2.cpu())
        x, y, wn = rn(B * T, 72), rn(B * T, 72).to(dt), rn(72)
        a, a_lp = ref.scaled_add_rmsnorm(x, y, wn, 1.7, 1e-5, 1.0, dt)
        b, b_lp = ops.scaled_add_rmsnorm(x.to(dev), y.to(dev), wn.to(dev), 1.7, 1e-5, 1.0, dt)
        assert torch.allclose(a, b.cpu(), atol=1e-5) and (a_lp is None or torch.allclose(a_lp.float(), b_lp.float().cpu(), atol=2e-2))
        gu = rn(B * T, 2 * 36).to(dt)
        assert torch.allclose(ref.clamped_glu(gu, 0.8, 1.702).float(), ops.clamped_glu(gu.to(dev), 0.8, 1.702).float().cpu(), atol=tol)
        yv, wg = rn(B * T, 48), rn(48)
        assert torch.allclose(ref.group_rmsnorm(yv, wg, 3, 1e-5, dt).float(), ops.group_rmsnorm(yv.to(dev), wg.to(dev), 3, 1e-5, dt).float().cpu(), atol=tol)
        nh, P, N, G = 4, 20, 24, 2
        inner = nh * P
        pz = rn(B, T, inner + nh + 3).to(dt)
        xBC, Al, db, Dk, S = rn(B, T, inner + 2 * G * N), rn(nh), rn(nh), rn(nh), rn(4, nh, N, P)
        S1, S2 = S.clone(), S.clone().to(dev)
        c = ref.ssd_scan(xBC, pz[..., inner:inner + nh], pz[..., :inner], Al, db, Dk, S1, lines, ctx, ql, nh, P, N, G)
        d = ops.ssd_scan(xBC.to(dev), pz.to(dev)[..., inner:inner + nh], pz.to(dev)[..., :inner], Al.to(dev), db.to(dev), Dk.to(dev), S2,
                         lines.to(dev), ctx.to(dev), ql.to(dev), nh, P, N, G)
        assert torch.allclose(c * live, d.cpu() * live, atol=1e-4, rtol=1e-4) and torch.allclose(S1, S2.cpu(), atol=1e-4, rtol=1e-4)
    # more rows / tokens than one grid axis other than x can index
    yv, wg = rn(70000, 16), rn(16)
    assert torch.allclose(ref.group_rmsnorm(yv, wg, 2, 1e-5), ops.group_rmsnorm(yv.to(dev), wg.to(dev), 2, 1e-5).cpu(), atol=1e-5)
    u, wt, st = rn(1, 70000, 8), rn(8, 2), rn(2, 1, 8)
    one, zero = torch.tensor([70000]).int(), torch.tensor([0]).int()
    assert torch.allclose(ref.short_conv(u, wt, None, st, zero, zero, one), ops.short_conv(u.to(dev), wt.to(dev), None, st.to(dev), zero.to(dev), zero.to(dev),
                                                                                           one.to(dev)).cpu(), atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("D,Dv", [(64, 64), (128, 128), (64, 128), (128, 64)])
def test_gpu_tensor_core_attention_on_prompt_portions(D, Dv):
    """bf16 portions of 16+ tokens take the mma kernel: ragged rows that start mid-sequence, scattered pages, window and kept-token
    edges inside and across key tiles, one dominant far key per row."""
    from neuronx_distributed_inference_b200 import ops
    from neuronx_distributed_inference_b200.ops import reference as ref
    g = torch.Generator().manual_seed(D + Dv)
    B, T, H, G, page = 3, 150, 4, 2, 16
    ctx, ql = torch.tensor([0, 70, 129]), torch.tensor([150, 93, 17])
    nblk = -(-(int((ctx + ql).max())) // page)
    table = torch.stack([torch.randperm(B * nblk, generator=g)[b * nblk:(b + 1) * nblk] for b in range(B)]).int()
    kc, vc = torch.randn(B * nblk, page, G, D, generator=g) * 0.5, torch.randn(B * nblk, page, G, Dv, generator=g)
    q, gate = torch.randn(B, T, H, D, generator=g) * 0.5, torch.randn(B, T, H * Dv + 8, generator=g)
    # row 0: make key 2 (kept) and key 40 (out of window for late queries) loud
    for j in (2, 40):
        kc[table[0, j // page].long(), j % page] = 2.0
    q[0, 100:] = 1.0
    for window, keep in ((37, 3), (64, 0), (0, 0), (200, 5)):
        want = ref.paged_window_attention(q.bfloat16().float(), kc.bfloat16().float(), vc.bfloat16().float(), table, ctx, ql, 0.2, 25.0, window, keep,
                                          gate[..., 8:].bfloat16().float())
        got = ops.paged_window_attention(q.bfloat16().cuda(), kc.bfloat16().cuda(), vc.bfloat16().cuda(), table.cuda(), ctx.int().cuda(), ql.int().cuda(),
                                         0.2, 25.0, window, keep, gate.bfloat16().cuda()[..., 8:])
        assert torch.allclose(got.float().cpu(), want, atol=2e-2, rtol=2e-2), (window, keep, float((got.float().cpu() - want).abs().max()))


def test_command_line_generates_from_token_ids(tmp_path, capsys):
    """``inference_demo --model-type fetodra ... --prompt-token-ids`` runs the engine's scheduler and prints the generated ids."""
    from neuronx_distributed_inference_b200 import inference_demo
    cfg = make_config(HYBRID)
    w = make_weights(cfg)
    eng = make_engine(tmp_path, cfg, w)
    want = eng.generate([[1, 2, 3, 4], [7, 8]], 5)
    inference_demo.main(["--model-type", "fetodra", "--task-type", "causal-lm", "run", "--model-path", str(tmp_path / "ckpt"),
                         "--compiled-model-path", str(tmp_path / "c"), "--on-cpu", "--torch-dtype", "float32", "--prompt-token-ids", "1,2,3,4",
                         "--prompt-token-ids", "7,8", "--max-new-tokens", "5", "--pa-block-size", str(PAGE)])
    out = capsys.readouterr().out
    assert "Output 0: " + ",".join(map(str, want[0])) in out and "Output 1: " + ",".join(map(str, want[1])) in out


def test_step_accepts_an_entry_without_tokens(tmp_path):
    cfg = make_config(HYBRID[:2])
    eng = make_engine(tmp_path, cfg, make_weights(cfg))
    rows = eng.step([("a", [1, 2, 3], [2]), ("b", [], [])])
    assert rows[0].shape == (1, cfg["vocab"]) and rows[1].shape[0] == 0 and "b" in eng.live
