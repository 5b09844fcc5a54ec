"""Plain, slow definition of the Fetodra decoder, one function per mechanism, for the tests.

Everything is evaluated token by token or with dense masks in float64 (or float32) on the CPU; nothing here is shared with the
package.  ``cfg`` is the checkpoint's ``config.json`` as a dict and ``w`` maps checkpoint tensor names to tensors.

Notation: ``h`` is a sublayer's input ``[T, width]`` for ONE sequence whose first row is position 0.
"""
import math

import torch


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_rms_norm(x, weight, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return rms_unit(x, eps) * (1.0 + weight)


def short_causal_conv(u, taps_w, bias=None):
    """u [T, C], taps_w [C, K]: y_t = sum_j taps_w[:, j] * u_{t-K+1+j}; rows before the start are zero."""
    T, C = u.shape
    K = taps_w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(K):
            s = t - K + 1 + j
            if s >= 0:
                y[t] += taps_w[:, j] * u[s]
    if bias is not None:
        y = y + bias
    return y


def rotate_interleaved(x, positions, n_rot, base):
    """x [T, heads, D]: channels (2i, 2i+1), i < n_rot/2, of every head turn by angle p * base^(-2i/n_rot)."""
    out = x.clone()
    for i in range(n_rot // 2):
        f = base ** (-2.0 * i / n_rot)
        ang = positions.to(x.dtype) * f
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def visible(i, j, window, keep_first):
    """Query position i sees key position j."""
    return j <= i and (i - j < window or j < keep_first)


def softcapped_window_attention(q, k, v, scale, softcap, window, keep_first):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] (already convolved / normed / rotated) -> [T, H * Dv]."""
    T, H, D = q.shape
    G = k.shape[1]
    see = torch.tensor([[visible(i, j, window, keep_first) for j in range(T)] for i in range(T)])
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ k[:, g].T) * scale
        s = softcap * torch.tanh(s / softcap)
        p = torch.softmax(s.masked_fill(~see, -math.inf), -1)
        out[:, hq] = p @ v[:, g]
    return out.reshape(T, -1)


def attention_keys_values(h, w, pre, m, eps):
    """The keys (convolved, normed over the whole projection, rotated) and values (convolved only) a layer stores."""
    T = h.shape[0]
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    k = short_causal_conv(h @ w[pre + "k"].T + w[pre + "k.b"], w[pre + "k.conv"])
    v = short_causal_conv(h @ w[pre + "v"].T + w[pre + "v.b"], w[pre + "v.conv"])
    k = rms_unit(k, eps) * w[pre + "k.norm"]
    k = rotate_interleaved(k.view(T, G, D), pos, m["rot"]["dims"], m["rot"]["base"])
    return k, v.view(T, G, Dv)


def attention_mixer(h, w, pre, m, eps, shared_kv=None):
    """``shared_kv``: (k, v) of the layer named by ``kv_from``; otherwise this layer makes its own.  Returns (out, (k, v))."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    pos = torch.arange(T)
    q = short_causal_conv(h @ w[pre + "q"].T + w[pre + "q.b"], w[pre + "q.conv"])
    q = rms_unit(q, eps) * w[pre + "q.norm"]
    q = rotate_interleaved(q.view(T, H, D), pos, m["rot"]["dims"], m["rot"]["base"])
    k, v = shared_kv if shared_kv is not None else attention_keys_values(h, w, pre, m, eps)
    o = softcapped_window_attention(q, k, v, m["scale"], m["softcap"], m["mask"]["size"], m["mask"]["keep_first"])
    o = o * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T, (k, v)


def mamba2_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    nh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = nh * P
    zxbcdt = h @ w[pre + "in"].T
    z, xBC, dt = zxbcdt.split([inner, inner + 2 * G * N, nh], -1)
    xBC = torch.nn.functional.silu(short_causal_conv(xBC, w[pre + "conv"], w[pre + "conv.b"]))
    x, Bm, Cm = xBC.split([inner, G * N, G * N], -1)
    dt = torch.nn.functional.softplus(dt + w[pre + "dt_bias"], threshold=1e9)
    A = torch.exp(w[pre + "A_log"])
    y = torch.zeros(T, nh, P, dtype=h.dtype)
    for hd in range(nh):
        g = hd // (nh // G)
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            xt = x[t, hd * P:(hd + 1) * P]
            Bt, Ct = Bm[t, g * N:(g + 1) * N], Cm[t, g * N:(g + 1) * N]
            S = torch.exp(-A[hd] * dt[t, hd]) * S + dt[t, hd] * torch.outer(Bt, xt)
            y[t, hd] = S.T @ Ct + w[pre + "D"][hd] * xt
    y = y.reshape(T, inner) * torch.nn.functional.silu(z)
    ng = m["norm_groups"]
    y = rms_unit(y.view(T, ng, inner // ng), eps).reshape(T, inner) * w[pre + "norm"]
    return y @ w[pre + "o"].T


def clamped_glu(h, w, pre, f):
    lim = f["limit"]
    g = (h @ w[pre + "gate"].T).clamp(max=lim)
    u = (h @ w[pre + "up"].T).clamp(-lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def forward(cfg, w, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][torch.as_tensor(tokens)]
    kv, per_layer = {}, []
    for i, layer in enumerate(cfg["layers"]):
        m, pre = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "attention":
            src = m.get("kv_from")
            y, kv[i] = attention_mixer(x, w, pre, m, eps, kv[src] if src is not None else None)
        elif layer["type"] == "mamba2":
            y = mamba2_mixer(x, w, pre, m, eps)
        else:
            raise ValueError(layer["type"])
        x = offset_rms_norm(alpha * x + y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = offset_rms_norm(alpha * x + clamped_glu(x, w, f"l{i}.mlp.", layer["mlp"]), w[f"l{i}.norm2"], eps)
        per_layer.append(x)
    logits = offset_rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(per_layer)) if return_layers else logits
