"""Prefill / decode throughput of the Fetodra stack beside the closest stack the engine already had (Bamba: Mamba-2 + GQA attention +
gated MLP after every mixer) at equal layer sizes, random weights, plus a per-kernel table: every ragged-mixer kernel timed alone
(CUDA events, L2 flushed between iterations) with its algorithmic bytes as a fraction of the measured copy bandwidth, next to the like
kernel of the closest stack.  Run through ``bench.py --config fetodra``."""
from __future__ import annotations

import json
import os
import tempfile

import torch

SIZES = {
    # width, q heads, kv heads, head size, ff, Mamba-2 heads x head size, state, groups
    "1b": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, m_heads=64, m_dim=64, state=128, groups=1),
    "8b": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, m_heads=128, m_dim=64, state=128, groups=8),
}
PATTERN = ("attention", "mamba2", "attention", "mamba2")
VOCAB = 32000


def fetodra_config(s, window, keep_first):
    layers = []
    for kind in PATTERN:
        if kind == "attention":
            mixer = dict(heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], vdim=s["dim"], conv=4, rot=dict(dims=s["dim"] // 2, base=1e6),
                         scale=s["dim"] ** -0.5, softcap=30.0, mask=dict(size=window, keep_first=keep_first))
        else:
            mixer = dict(heads=s["m_heads"], vdim=s["m_dim"], state=s["state"], groups=s["groups"], norm_groups=1, conv=4)
        layers.append(dict(type=kind, mixer=mixer, mlp=dict(kind="dense", ff=s["ff"], limit=7.0)))
    return dict(architecture="Fetodra", layers=layers, norm=dict(eps=1e-5), postln_alpha=1.0, vocab=VOCAB, width=s["width"])


def build_fetodra(s, batch, max_tokens, window, keep_first):
    from ..config import NeuronConfig, OnDeviceSamplingConfig
    from ..models.fetodra.modeling_fetodra import FetodraInferenceConfig, NeuronFetodraForCausalLM
    from ..runtime.scheduler import PagedBatchEngine
    d = tempfile.mkdtemp()
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(fetodra_config(s, window, keep_first), f)
    page = 64
    ladder = [b for b in (64, 256, 1024, 4096) if b < max_tokens] + [max_tokens]
    nc = NeuronConfig(batch_size=batch, ctx_batch_size=batch, tkg_batch_size=batch, max_batch_size=batch, kv_cache_batch_size=batch,
                      seq_len=max_tokens, max_context_length=max_tokens, torch_dtype="bfloat16", is_block_kv_layout=True, pa_block_size=page,
                      pa_num_blocks=batch * (-(-max_tokens // page)), enable_bucketing=True, context_encoding_buckets=ladder,
                      is_continuous_batching=True, on_device_sampling_config=OnDeviceSamplingConfig(top_k=1), skip_warmup=True)
    app = NeuronFetodraForCausalLM(d, FetodraInferenceConfig.from_pretrained(d, nc))
    app.load(None, skip_warmup=True, random_weights=True)
    return PagedBatchEngine(app)


def build_bamba(s, batch, max_tokens):
    from ..contrib.models.hybrid_family import NeuronBambaForCausalLM
    from .testing import build_random_llama
    hf = dict(hidden_size=s["width"], intermediate_size=s["ff"], num_hidden_layers=len(PATTERN), num_attention_heads=s["heads"],
              num_key_value_heads=s["kv_heads"], head_dim=s["dim"], vocab_size=VOCAB, mamba_n_heads=s["m_heads"], mamba_d_head=s["m_dim"],
              mamba_d_state=s["state"], mamba_n_groups=s["groups"], mamba_d_conv=4, mamba_expand=s["m_heads"] * s["m_dim"] / s["width"],
              mamba_d_ssm=s["m_heads"] * s["m_dim"], layers_block_type=["attention" if k == "attention" else "mamba" for k in PATTERN],
              partial_rotary_factor=0.5, rope_theta=1e6)
    return build_random_llama(hf, batch_size=batch, seq_len=max_tokens, max_context_length=max_tokens, device="cuda", app_cls=NeuronBambaForCausalLM)


def _time(fn, n=3, warm=1):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best


def model_numbers(size, batch, prompt, decode_steps, warmup):
    """tokens/s of one prefill step (batch rows x prompt tokens, host-resident ids in, tokens out) and of decode steps at that context,
    through each stack's public entry point."""
    s = SIZES[size]
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, VOCAB, (batch, prompt), generator=g)
    out = {}
    eng = build_fetodra(s, batch, prompt + decode_steps + warmup + 64, window=prompt + decode_steps + warmup + 64, keep_first=4)

    def f_prefill():
        for b in range(batch):
            eng.release(b)
        return eng.step([(b, ids[b].tolist(), ()) for b in range(batch)], sample=True)
    ms = _time(f_prefill, n=3, warm=max(1, min(warmup, 2)))
    out["fetodra_prefill_tok_s"] = batch * prompt * 1e3 / ms
    tok = f_prefill()

    def f_decode(n):
        nonlocal tok
        for _ in range(n):
            tok = eng.step([(b, [tok[b]], ()) for b in range(batch)], sample=True)
    f_decode(warmup)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    f_decode(decode_steps)
    e1.record()
    torch.cuda.synchronize()
    out["fetodra_decode_tok_s"] = batch * decode_steps * 1e3 / e0.elapsed_time(e1)
    out["fetodra_decode_ms_per_step"] = e0.elapsed_time(e1) / decode_steps
    del eng
    torch.cuda.empty_cache()
    app = build_bamba(s, batch, prompt + decode_steps + warmup + 64)
    mask = torch.ones_like(ids, dtype=torch.int32)

    def b_prefill():
        app.reset()
        return app(ids, attention_mask=mask).tokens
    ms = _time(b_prefill, n=2, warm=1)
    out["bamba_prefill_tok_s"] = batch * prompt * 1e3 / ms
    tokb = b_prefill().cpu()
    pos = torch.full((batch, 1), prompt, dtype=torch.int32)

    def b_decode(n):
        nonlocal tokb, pos
        for _ in range(n):
            tokb = app(tokb.view(batch, 1), position_ids=pos).tokens.cpu()
            pos = pos + 1
    b_decode(warmup)
    torch.cuda.synchronize()
    e0.record()
    b_decode(decode_steps)
    e1.record()
    torch.cuda.synchronize()
    out["bamba_decode_tok_s"] = batch * decode_steps * 1e3 / e0.elapsed_time(e1)
    out["bamba_decode_ms_per_step"] = e0.elapsed_time(e1) / decode_steps
    del app
    torch.cuda.empty_cache()
    return out


def kernel_table(size, batch, prompt, hbm_gbs):
    """Each ragged-mixer kernel alone at the layer's shapes: [name, ms, GB moved (algorithmic), fraction of the measured copy
    bandwidth], prefill (batch x prompt tokens) and decode (batch x 1 token at context ``prompt``); then the like kernels of the
    Llama / Bamba path on the same shapes."""
    from .. import ops
    s = SIZES[size]
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def run(name, fn, nbytes, n=5):
        best = float("inf")
        for i in range(n + 2):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 2:
                best = min(best, e0.elapsed_time(e1))
        rows.append(dict(kernel=name, ms=round(best, 4), gb=round(nbytes / 1e9, 4), frac_of_measured_hbm=round(nbytes / 1e6 / best / hbm_gbs, 3)))

    W, H, G, D, F = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"]
    nh, P, N, Gm = s["m_heads"], s["m_dim"], s["state"], s["groups"]
    inner, K, page = nh * P, 4, 64
    for phase, T, ctx0 in (("prefill", prompt, 0), ("decode", 1, prompt)):
        B = batch
        R = B * T
        ctx = torch.full((B,), ctx0, dtype=torch.int32, device=dev)
        ql = torch.full((B,), T, dtype=torch.int32, device=dev)
        lines = torch.arange(B, dtype=torch.int32, device=dev)
        nblk = -(-(ctx0 + T) // page)
        table = torch.arange(B * nblk, dtype=torch.int32, device=dev).view(B, nblk)
        x32, y = torch.randn(R, W, device=dev), torch.randn(R, W, device=dev, dtype=bf)
        wn = torch.randn(W, device=dev)
        run(f"{phase}: scaled_add_rmsnorm", lambda: ops.scaled_add_rmsnorm(x32, y, wn, 1.0, 1e-5, 1.0, bf), R * W * (4 + 2 + 4 + 2))
        xb, wb = torch.randn(R, W, device=dev, dtype=bf), torch.randn(W, device=dev, dtype=bf)
        run(f"{phase}: rmsnorm+residual (Llama path)", lambda: ops.rmsnorm(xb, wb, 1e-5, 0.0, xb), R * W * 2 * 4)
        C = (H + 2 * G) * D
        p = torch.randn(B, T, C + H * D, device=dev, dtype=bf)
        cw, st = torch.randn(C, K, device=dev), torch.zeros(B + 1, K - 1, C, device=dev, dtype=bf)
        cos, sin = torch.randn(B, T, D // 4, device=dev), torch.randn(B, T, D // 4, device=dev)
        kc, vc = (torch.randn(B * nblk, page, G, D, device=dev, dtype=bf) for _ in range(2))
        qn, kn = torch.ones(H * D, device=dev), torch.ones(G * D, device=dev)
        run(f"{phase}: conv_qknorm_rope_append", lambda: ops.conv_qknorm_rope_append(p, cw, st, lines, ctx, ql, qn, kn, 1e-5, H, G, D, D, cos, sin, kc, vc, table),
            R * C * 2 * 2)
        if phase == "prefill":
            qkv = torch.randn(B, T, C, device=dev, dtype=bf)
            cf, sf = torch.randn(B, T, D // 2, device=dev), torch.randn(B, T, D // 2, device=dev)
            kcl, vcl = (torch.zeros(B + 1, G, T, D, device=dev, dtype=bf) for _ in range(2))
            posl = torch.arange(T, dtype=torch.int32, device=dev).view(1, T).expand(B, T).contiguous()
            if ops.rope_kv_split_append(qkv, cf, sf, kcl, vcl, lines, posl, H, G, D) is not None:
                run("prefill: rope_kv_split_append (Llama path: split + rotate + cache write, no convolution / row norm)",
                    lambda: ops.rope_kv_split_append(qkv, cf, sf, kcl, vcl, lines, posl, H, G, D), R * C * 2 * 2 + R * 2 * G * D * 2)
        run(f"{phase}: short_conv_update (q|k|v)", lambda: ops.short_conv_update(p[..., :C], st, lines, ctx, ql), B * (K - 1) * C * 2 * 2)
        q = torch.randn(B, T, H, D, device=dev, dtype=bf)
        keys = ctx0 + T
        attn_bytes = (B * keys * G * D * 2 * 2) + R * H * D * 2 * 3
        run(f"{phase}: paged_window_attention (window >= context)", lambda: ops.paged_window_attention(q, kc, vc, table, ctx, ql, D ** -0.5, 30.0, 0, 0, p[..., C:]),
            attn_bytes)
        if phase == "prefill":
            k2, v2 = torch.randn(B, T, G, D, device=dev, dtype=bf), torch.randn(B, T, G, D, device=dev, dtype=bf)
            run("prefill: attention_prefill (Llama path, tcgen05)", lambda: ops.attention_prefill(q, k2, v2, D ** -0.5, True), attn_bytes)
        else:
            S = -(-(keys + 1) // 64) * 64
            kcc, vcc = (torch.randn(B + 1, G, S, D, device=dev, dtype=bf) for _ in range(2))
            pos = torch.full((B, 1), ctx0, dtype=torch.int32, device=dev)
            run("decode: attention_decode (Llama path)", lambda: ops.attention_decode(q, kcc, vcc, lines, pos, D ** -0.5), attn_bytes)
        gu = torch.randn(R, 2 * F, device=dev, dtype=bf)
        run(f"{phase}: clamped_glu", lambda: ops.clamped_glu(gu, 7.0), R * F * 2 * 3)
        Cd = inner + 2 * Gm * N
        pm = torch.randn(B, T, inner + Cd + nh, device=dev, dtype=bf)
        mw, mb, mst = torch.randn(Cd, K, device=dev) * 0.3, torch.zeros(Cd, device=dev), torch.zeros(B + 1, K - 1, Cd, device=dev, dtype=bf)
        run(f"{phase}: short_conv+silu (x|B|C)", lambda: ops.short_conv(pm[..., inner:inner + Cd], mw, mb, mst, lines, ctx, ql, True), R * Cd * (2 + 4))
        xBC = torch.randn(B, T, Cd, device=dev) * 0.3
        Al, db, Dk = torch.zeros(nh, device=dev), torch.full((nh,), -2.0, device=dev), torch.ones(nh, device=dev)
        S0 = torch.zeros(B + 1, nh, N, P, device=dev)
        run(f"{phase}: ssd_scan", lambda: ops.ssd_scan(xBC, pm[..., inner + Cd:], pm[..., :inner], Al, db, Dk, S0, lines, ctx, ql, nh, P, N, Gm),
            R * (Cd * 4 + inner * (2 + 4)) + B * nh * N * P * 4 * 2, n=3)
        yv, wg = torch.randn(R, inner, device=dev), torch.ones(inner, device=dev)
        run(f"{phase}: group_rmsnorm", lambda: ops.group_rmsnorm(yv, wg, 1, 1e-5, bf), R * inner * (4 + 2))
    return rows


def run(size="1b", batch=4, prompt=1024, decode_steps=32, warmup=3):
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            peaks = json.load(f)
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    res = dict(size=size, shapes=SIZES[size], layers=list(PATTERN), batch=batch, prompt=prompt, decode_steps=decode_steps,
               hbm_gbs=hbm, hbm_source="measured" if peaks else "fallback")
    res.update(model_numbers(size, batch, prompt, decode_steps, warmup))
    res["kernels"] = kernel_table(size, batch, prompt, hbm)
    return res
