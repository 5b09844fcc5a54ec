"""Prefill / decode throughput of the Sodudra stack (latent attention with a compressed cache, squared-ReLU routed experts) beside the
closest stack the engine already had — DeepSeek: latent attention with expanded keys and values in the cache, sigmoid-routed gated
experts plus a shared expert — at equal layer sizes, random weights, plus a per-kernel table: every kernel the new stack added, timed
alone (CUDA events, L2 flushed between iterations) with its algorithmic bytes or FLOPs as a fraction of the measured copy bandwidth /
bf16 GEMM rate, next to the like kernel of the engine's other stacks.  Run through ``bench.py --config sodudra``."""
from __future__ import annotations

import json
import os
import tempfile

import torch

SIZES = {
    # width, heads, q/k head size, value head size, latent rank, experts, chosen, expert ff, shared ff, side width
    "small": dict(width=2048, heads=16, dim=128, vdim=128, rank=128, experts=32, top=4, ff=1024, shared=2048, side=64),
    "large": dict(width=4096, heads=32, dim=128, vdim=128, rank=128, experts=64, top=6, ff=1408, shared=2816, side=128),
}
LAYERS = 4
VOCAB = 32000


def sodudra_config(s):
    layer = dict(type="latent_attention", mixer=dict(heads=s["heads"], dim=s["dim"], vdim=s["vdim"], kv_rank=s["rank"], scale=s["dim"] ** -0.5),
                 mlp=dict(kind="moe", router=dict(experts=s["experts"], top=s["top"]), expert=dict(ff=s["ff"]), shared=dict(ff=s["shared"])))
    return dict(architecture="Sodudra", layers=[layer] * LAYERS, norm=dict(eps=1e-5), vocab=VOCAB, width=s["width"], logit_scale=1.0,
                logit_softcap=30.0, loop=dict(start=1, stop=3, times=1), token_side=dict(dim=s["side"]))


def build_sodudra(s, batch, max_tokens):
    from ..config import NeuronConfig, OnDeviceSamplingConfig
    from ..models.sodudra.modeling_sodudra import NeuronSodudraForCausalLM, SodudraInferenceConfig
    from ..runtime.scheduler import PagedBatchEngine
    d = tempfile.mkdtemp()
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(sodudra_config(s), f)
    page = 64
    ladder = [b for b in (64, 256, 1024, 4096) if b < max_tokens] + [max_tokens]
    nc = NeuronConfig(batch_size=batch, ctx_batch_size=batch, tkg_batch_size=batch, max_batch_size=batch, kv_cache_batch_size=batch,
                      seq_len=max_tokens, max_context_length=max_tokens, torch_dtype="bfloat16", is_block_kv_layout=True, pa_block_size=page,
                      pa_num_blocks=batch * (-(-max_tokens // page)), enable_bucketing=True, context_encoding_buckets=ladder,
                      is_continuous_batching=True, on_device_sampling_config=OnDeviceSamplingConfig(top_k=1), skip_warmup=True)
    app = NeuronSodudraForCausalLM(d, SodudraInferenceConfig.from_pretrained(d, nc))
    app.load(None, skip_warmup=True, random_weights=True)
    return PagedBatchEngine(app)


def build_deepseek(s, batch, max_tokens):
    """Same widths: q/k head = 3/4 unrotated + 1/4 rotated channels, the same latent rank, experts and chosen count; its experts are
    gated (three matrices of the same ff instead of two)."""
    from ..models.deepseek.modeling_deepseek import NeuronDeepseekForCausalLM
    from .testing import build_random_llama
    rope = s["dim"] // 4
    hf = dict(hidden_size=s["width"], intermediate_size=s["shared"], num_hidden_layers=LAYERS, num_attention_heads=s["heads"],
              num_key_value_heads=s["heads"], vocab_size=VOCAB, kv_lora_rank=s["rank"], q_lora_rank=None, qk_nope_head_dim=s["dim"] - rope,
              qk_rope_head_dim=rope, v_head_dim=s["vdim"], n_routed_experts=s["experts"], num_experts_per_tok=s["top"], n_shared_experts=1,
              moe_intermediate_size=s["ff"], first_k_dense_replace=0, n_group=1, topk_group=1, norm_topk_prob=True)
    return build_random_llama(hf, batch_size=batch, seq_len=max_tokens, max_context_length=max_tokens, device="cuda",
                              app_cls=NeuronDeepseekForCausalLM)


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
    eng = build_sodudra(s, batch, prompt + decode_steps + warmup + 64)

    def f_prefill():
        for b in range(batch):
            eng.release(b)
        return eng.step([(b, ids[b].tolist(), ()) for b in range(batch)], sample=True)
    ms = _time(f_prefill, n=3, warm=max(1, min(warmup, 2)))
    out["sodudra_prefill_tok_s"] = batch * prompt * 1e3 / ms
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
    out["sodudra_decode_tok_s"] = batch * decode_steps * 1e3 / e0.elapsed_time(e1)
    out["sodudra_decode_ms_per_step"] = e0.elapsed_time(e1) / decode_steps
    del eng
    torch.cuda.empty_cache()
    app = build_deepseek(s, batch, prompt + decode_steps + warmup + 64)
    mask = torch.ones_like(ids, dtype=torch.int32)

    def d_prefill():
        app.reset()
        return app(ids, attention_mask=mask).tokens
    ms = _time(d_prefill, n=2, warm=1)
    out["deepseek_prefill_tok_s"] = batch * prompt * 1e3 / ms
    tokb = d_prefill().cpu()
    pos = torch.full((batch, 1), prompt, dtype=torch.int32)

    def d_decode(n):
        nonlocal tokb, pos
        for _ in range(n):
            tokb = app(tokb.view(batch, 1), position_ids=pos).tokens.cpu()
            pos = pos + 1
    d_decode(warmup)
    torch.cuda.synchronize()
    e0.record()
    d_decode(decode_steps)
    e1.record()
    torch.cuda.synchronize()
    out["deepseek_decode_tok_s"] = batch * decode_steps * 1e3 / e0.elapsed_time(e1)
    out["deepseek_decode_ms_per_step"] = e0.elapsed_time(e1) / decode_steps
    del app
    torch.cuda.empty_cache()
    return out


def kernel_table(size, batch, prompt, hbm_gbs, tflops):
    """Each kernel alone at the layer's shapes: name, ms, algorithmic GB and GFLOP, the fraction of the measured copy bandwidth and of
    the measured bf16 GEMM rate; prefill (batch x prompt tokens) and decode (batch x 1 token at context ``prompt``); after every new
    kernel the like kernel of another stack on the same shapes."""
    from .. import ops
    from ..ops import reference as ref
    s = SIZES[size]
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def run(name, fn, nbytes, flops=0.0, n=5):
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
        rows.append(dict(kernel=name, ms=round(best, 4), gb=round(nbytes / 1e9, 4), frac_of_measured_hbm=round(nbytes / 1e6 / best / hbm_gbs, 3),
                         tflops=round(flops / 1e9 / best, 1), frac_of_measured_bf16=round(flops / 1e9 / best / tflops, 3)))

    W, H, D, Dv, R = s["width"], s["heads"], s["dim"], s["vdim"], s["rank"]
    E, k, F, page = s["experts"], s["top"], s["ff"], 64
    for phase, T, ctx0 in (("prefill", prompt, 0), ("decode", 1, prompt)):
        B = batch
        N = B * T
        ctx = torch.full((B,), ctx0, dtype=torch.int32, device=dev)
        ql = torch.full((B,), T, dtype=torch.int32, device=dev)
        nblk = -(-(ctx0 + T) // page)
        table = torch.arange(B * nblk, dtype=torch.int32, device=dev).view(B, nblk)
        x32, y1, y2 = torch.randn(N, W, device=dev), torch.randn(N, W, device=dev, dtype=bf), torch.randn(N, W, device=dev, dtype=bf)
        wn = torch.randn(W, device=dev)
        run(f"{phase}: stream_add_rmsnorm (x + a + b -> stream, bf16 copy)", lambda: ops.stream_add_rmsnorm(x32, (y1, y2), eps=1e-5, lp_dtype=bf, emit_stream_lp=True),
            N * W * (4 + 2 + 2 + 4 + 2))
        run(f"{phase}: stream_add_rmsnorm (x + unit(y) w -> stream, next norm)",
            lambda: ops.stream_add_rmsnorm(x32, normed=y1, normed_weight=wn, weight=wn, eps=1e-5, lp_dtype=bf), N * W * (4 + 2 + 4 + 2))
        run(f"{phase}: like: scaled_add_rmsnorm (post-norm stack)", lambda: ops.scaled_add_rmsnorm(x32, y1, wn, 1.0, 1e-5, 0.0, bf), N * W * (4 + 2 + 4 + 2))
        C = H * D + R + H
        p = torch.randn(B, T, C, device=dev, dtype=bf)
        cache = torch.randn(B * nblk, page, 1, R, device=dev, dtype=bf)
        lw = torch.ones(R, device=dev)
        run(f"{phase}: latent_norm_append", lambda: ops.latent_norm_append(p, H * D, R, lw, 1e-5, cache, table, ctx, ql), N * R * 2 * 2)
        k_new, v_new = torch.randn(N, 1, R, device=dev, dtype=bf), torch.randn(N, 1, R, device=dev, dtype=bf)
        slots = (torch.arange(N, device=dev, dtype=torch.int32) % T + ctx0).view(B, T) + (torch.arange(B, device=dev, dtype=torch.int32) * nblk * page).view(B, 1)
        if hasattr(ops, "paged_kv_append"):
            run(f"{phase}: like: paged_kv_append (one kv head of the same width, no norm)",
                lambda: ops.paged_kv_append(cache, cache, k_new, v_new, slots.reshape(-1)), N * R * 2 * 3)
        q = torch.randn(B, T, H, R, device=dev, dtype=bf) * 0.2
        gate, sinks = p[..., H * D + R:], torch.zeros(H, device=dev)
        keys = ctx0 + T
        attn_bytes = B * keys * R * 2 + N * H * R * 2 * 2
        attn_flops = 4.0 * B * H * R * (T * (T + 1) / 2 + T * ctx0)
        run(f"{phase}: paged_window_attention (latent rows as keys and values, sink, head gate)",
            lambda: ops.paged_window_attention(q, cache, cache, table, ctx, ql, D ** -0.5, None, None, 0, gate, sinks, True), attn_bytes, attn_flops)
        G = max(1, H // 4)
        kc, vc = (torch.randn(B * nblk, page, G, R, device=dev, dtype=bf) for _ in range(2))
        run(f"{phase}: like: paged_window_attention (grouped kv heads of the same size, no sink / gate)",
            lambda: ops.paged_window_attention(q, kc, vc, table, ctx, ql, D ** -0.5, None, None, 0), B * keys * G * R * 2 * 2 + N * H * R * 2 * 2, attn_flops)
        if phase == "prefill" and ops.latent_prefill_on_tensor_cores(q, R):
            rows_t = torch.randn(B, T, 1, R, device=dev, dtype=bf)
            run("prefill: whole prompts: attention_prefill over the rows in token order (tcgen05, sink)",
                lambda: ops.attention_prefill(q, rows_t, rows_t, D ** -0.5, True, sinks=sinks), attn_bytes, attn_flops)
            o_t = torch.randn(B, T, H, R, device=dev, dtype=bf)
            run("prefill: whole prompts: head_gate_mul", lambda: ops.head_gate_mul(o_t, gate), N * H * R * 2 * 2)
        if phase == "prefill":
            k2, v2 = torch.randn(B, T, G, R, device=dev, dtype=bf), torch.randn(B, T, G, R, device=dev, dtype=bf)
            run("prefill: like: attention_prefill (Llama path, tcgen05, contiguous keys)", lambda: ops.attention_prefill(q, k2, v2, D ** -0.5, True),
                B * keys * G * R * 2 * 2 + N * H * R * 2 * 2, attn_flops)
        x = torch.randn(N, W, device=dev, dtype=bf)
        w_up, w_dn = torch.randn(E, F, W, device=dev, dtype=bf) * W ** -0.5, torch.randn(E, W, F, device=dev, dtype=bf) * F ** -0.5
        w_gu = torch.randn(E, 2 * F, W, device=dev, dtype=bf) * W ** -0.5
        wr = torch.randn(E, W, device=dev) * W ** -0.5
        run(f"{phase}: router_topk (fp32 products + selection + renormalisation, two kernels)", lambda: ops.router_topk(x, wr, k, "sigmoid", True, False, 1e-20),
            N * W * 2 + E * W * 4, 2.0 * N * E * W)
        run(f"{phase}: like: cast + fp32 library GEMM + sigmoid / top-k / sum / divide (torch)",
            lambda: ref.moe_route(torch.nn.functional.linear(x.float(), wr), k, "sigmoid", True, False, 1e-20), N * W * 2 + E * W * 4, 2.0 * N * E * W)
        tw, ti = ref.moe_route(torch.randn(N, E, device=dev), k, "sigmoid", True, False, 1e-20)
        ti = ti.to(torch.int32)
        used = min(E, N * k)
        run(f"{phase}: moe experts, two matrices, squared ReLU", lambda: ops.moe_experts(x, w_up, w_dn, tw, ti, "relu2"),
            used * 2 * F * W * 2 + N * W * 2 * 2, 4.0 * N * k * F * W)
        run(f"{phase}: like: moe experts, gated SiLU (three matrices)", lambda: ops.moe_experts(x, w_gu, w_dn, tw, ti, "silu_mul"),
            used * 3 * F * W * 2 + N * W * 2 * 2, 6.0 * N * k * F * W)
        Fs = s["shared"]
        hs = torch.randn(N, Fs, device=dev, dtype=bf)
        run(f"{phase}: unary_act (squared ReLU, shared expert)", lambda: ops.unary_act(hs, "relu2"), N * Fs * 2 * 2)
        gu = torch.randn(N, 2 * Fs, device=dev, dtype=bf)
        run(f"{phase}: like: clamped_glu", lambda: ops.clamped_glu(gu, 7.0), N * Fs * 2 * 3)
        sd = s["side"]
        gt, tab = torch.randn(N, sd, device=dev, dtype=bf), torch.randn(N, sd * LAYERS, device=dev, dtype=bf)
        run(f"{phase}: gated_act_mul (token input)", lambda: ops.gated_act_mul(gt, tab[:, sd:2 * sd], "gelu_tanh"), N * sd * 2 * 3)
    return rows


def run(size="small", batch=4, prompt=1024, decode_steps=32, warmup=3):
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            peaks = json.load(f)
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    tf = float(peaks.get("bf16_tflops", 1590.0))
    res = dict(size=size, shapes=SIZES[size], layers=LAYERS, batch=batch, prompt=prompt, decode_steps=decode_steps, hbm_gbs=hbm, bf16_tflops=tf,
               peaks_source="measured" if peaks else "fallback")
    res.update(model_numbers(size, batch, prompt, decode_steps, warmup))
    res["kernels"] = kernel_table(size, batch, prompt, hbm, tf)
    return res
