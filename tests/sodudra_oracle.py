"""Plain definition of the Sodudra decoder, one function per mechanism, float64, whole sequences, no cache.  Shares nothing with the
engine: tests compare the engine (loader, latent cache, ragged batches, kernels) against these functions."""
import math

import torch


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sink_softmax(scores, sink):
    """Softmax over the last axis whose denominator also holds exp(sink); returns the weights of the real entries."""
    top = torch.maximum(scores.max(-1, keepdim=True).values, sink)
    e = torch.exp(scores - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))


def latent_attention(h, w, p, m, eps):
    """h [T, W].  Keys and values are expanded from the normalised latent row; causal; sink per head; sigmoid gate per head."""
    T, H, d, dv = h.shape[0], m["heads"], m["dim"], m.get("vdim", m["dim"])
    q = (h @ w[p + "q"].T).view(T, H, d)
    c = rms_norm(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)
    k = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    gate = torch.sigmoid(h @ w[p + "g"].T)                                    # [T, H]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        for a in range(H):
            s = (k[:i + 1, a] @ q[i, a]) * m["scale"]
            pr = sink_softmax(s, w[p + "sink"][a])
            out[i, a] = (pr.unsqueeze(-1) * v[:i + 1, a]).sum(0) * gate[i, a]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def expert(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


def route(z, top):
    """Sigmoid scores, the ``top`` largest, divided by their sum."""
    s = torch.sigmoid(z)
    val, idx = torch.sort(s, dim=-1, descending=True, stable=True)
    val, idx = val[..., :top], idx[..., :top]
    return val / (val.sum(-1, keepdim=True) + 1e-20), idx


def moe(h, w, p, f):
    wt, idx = route(h @ w[p + "router"].T, f["router"]["top"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * expert(h[t], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
    if f.get("shared"):
        out = out + expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


def token_side(x, tokens, w, i, dim, eps):
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ w[f"l{i}.side.gate"].T) * e) @ w[f"l{i}.side.proj"].T
    return x + rms_norm(y, w[f"l{i}.side.norm"], eps)


def layer_order(n, loop):
    """[(layer, pass or None)]: the pass number stands on the first layer of every pass of the repeated span."""
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, t if i == loop["start"] else None))
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, streams=None):
    """Logits [T, vocab] (float64) of one whole sequence; ``streams`` collects the residual stream after every layer run."""
    w = {k: v.double() for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(tokens)
    x = rms_norm(w["embed"][tok], w["embed.norm"], eps)
    side = (cfg.get("token_side") or {}).get("dim")
    for i, t in layer_order(len(cfg["layers"]), cfg.get("loop")):
        if t is not None:
            x = x + w["loop.step"][t]
        spec = cfg["layers"][i]
        h = rms_norm(x, w[f"l{i}.norm1"], eps)
        y = latent_attention(h, w, f"l{i}.mix.", spec["mixer"], eps)
        if spec.get("mlp") is not None:
            y = y + moe(h, w, f"l{i}.mlp.", spec["mlp"])
        x = x + y
        if side:
            x = token_side(x, tok, w, i, side, eps)
        if streams is not None:
            streams.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
