"""A plain, slow statement of the Daborax decoder: whole sequences, no cache, float64, one function a
mechanism.  It shares no code with the engine; the tests compare the engine with it.

Notation: T tokens, W the model width, rows are tokens, positions p = 0, 1, ...  Linear weights are [out, in].

* embedding:         x_p = E[token] * s + pe(p),  pe(p)[2i] = sin(p * 10000^(-2i/W)),  pe(p)[2i+1] = cos(same)
* RMS norm:          N(x) = x / sqrt(mean(x^2) + eps) (* w)
* a layer:           x += m * ls1 * N_1(mixer(x)),   x += m * ls2 * N_2(ff(x))      (sublayers read x itself)
* selective scan:    S_t = exp(-exp(A) dt_t) S_(t-1) + dt_t B_t x_t^T,   y_t = S_t^T C_t + D x_t,
                     dt = softplus(dt_raw + dt_bias);  x, B, C pass a causal convolution with bias and SiLU first;
                     y * silu(z) is RMS-normed in equal parts before the output projection
* decayed linear attention:  S_t = lambda S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t,  q, k, v through SiLU; the heads
                     together are RMS-normed, gated by sigmoid(W_g h) and projected
* window attention:  biases; q and k of every head divided by their root mean square; score = cap * tanh(q.k * scale / cap);
                     a query sees its own key and the window - 1 before it; the softmax's denominator also holds
                     exp(sink) of the head
* feed-forward:      g = min(W_g h, L), u = clamp(W_u h, -L, L), y = g * sigmoid(1.702 g) * (u + 1), W_d y
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def position_vectors(T, width, start=0):
    p = torch.arange(start, start + T, dtype=F64)[:, None]
    i = torch.arange((width + 1) // 2, dtype=F64)[None, :]
    ang = p * 10000.0 ** (-2 * i / width)
    out = torch.zeros(T, width, dtype=F64)
    out[:, 0::2] = torch.sin(ang)
    out[:, 1::2] = torch.cos(ang)[:, : width // 2]
    return out


def embed(tokens, table, scale, start=0):
    return table[torch.as_tensor(tokens)] * scale + position_vectors(len(tokens), table.shape[1], start)


def causal_conv(u, w, b):
    """u [T, C], w [C, taps], b [C]: out_t = b + sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    out = b.expand(T, -1).clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out


def selective_scan(x, B, C, dt, A_log, D, groups):
    """x [T, H, P], B and C [T, G, N], dt [T, H] (after softplus).  Returns y [T, H, P] and the last state."""
    T, H, P = x.shape
    N = B.shape[-1]
    S = torch.zeros(H, N, P, dtype=x.dtype)
    y = torch.zeros(T, H, P, dtype=x.dtype)
    group_of = torch.arange(H) // (H // groups)
    a = torch.exp(A_log)
    for t in range(T):
        Bt, Ct = B[t][group_of], C[t][group_of]                      # [H, N]
        S = torch.exp(-a * dt[t])[:, None, None] * S + dt[t][:, None, None] * Bt[:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, Ct) + D[:, None] * x[t]
    return y, S


def mamba2_mixer(h, p, heads, vdim, state, groups, norm_groups, eps):
    """p: in, conv, conv.b, dt_bias, A_log, D, norm, o."""
    T = h.shape[0]
    inner, GN = heads * vdim, groups * state
    proj = h @ p["in"].T
    z, xBC, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * GN], proj[:, 2 * inner + 2 * GN:]
    xBC = silu(causal_conv(xBC, p["conv"], p["conv.b"]))
    x = xBC[:, :inner].reshape(T, heads, vdim)
    B = xBC[:, inner:inner + GN].reshape(T, groups, state)
    C = xBC[:, inner + GN:].reshape(T, groups, state)
    dt = softplus(dt + p["dt_bias"])
    y, _ = selective_scan(x, B, C, dt, p["A_log"], p["D"], groups)
    y = y.reshape(T, inner) * silu(z)
    y = rms_norm(y.reshape(T, norm_groups, inner // norm_groups), None, eps).reshape(T, inner) * p["norm"]
    return y @ p["o"].T


def decayed_linear_attention(q, k, v, decay):
    """q, k [T, H, d], v [T, H, e], decay [H]."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=q.dtype)
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out


def lightning_mixer(h, p, heads, dim, vdim, decay, eps):
    """p: q, k, v, g, norm, o."""
    T = h.shape[0]
    q = silu(h @ p["q"].T).reshape(T, heads, dim)
    k = silu(h @ p["k"].T).reshape(T, heads, dim)
    v = silu(h @ p["v"].T).reshape(T, heads, vdim)
    o = decayed_linear_attention(q, k, v, torch.as_tensor(decay, dtype=h.dtype)).reshape(T, heads * vdim)
    o = rms_norm(o, p["norm"], eps) * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T


def window_sink_attention(q, k, v, sink, scale, softcap, window):
    """q [T, H, d], k [T, G, d], v [T, G, e], sink [H]."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        i = torch.arange(T)[:, None]
        j = torch.arange(T)[None, :]
        seen = (j <= i) & ((i - j) < window if window else True)
        s = s.masked_fill(~seen, -math.inf)
        m = torch.maximum(s.max(-1, keepdim=True).values, sink[h])
        e = torch.exp(s - m)
        out[:, h] = (e @ v[:, g]) / (e.sum(-1, keepdim=True) + torch.exp(sink[h] - m))
    return out


def attention_mixer(h, p, heads, kv_heads, dim, vdim, scale, softcap, window, eps):
    """p: q, q.b, k, k.b, v, v.b, sink, o, o.b."""
    T = h.shape[0]
    q = (h @ p["q"].T + p["q.b"]).reshape(T, heads, dim)
    k = (h @ p["k"].T + p["k.b"]).reshape(T, kv_heads, dim)
    v = (h @ p["v"].T + p["v.b"]).reshape(T, kv_heads, vdim)
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    o = window_sink_attention(q, k, v, p["sink"], scale, softcap, window)
    return o.reshape(T, heads * vdim) @ p["o"].T + p["o.b"]


def clamped_glu(h, p, limit):
    """p: gate, up, down."""
    g = torch.clamp(h @ p["gate"].T, max=limit)
    u = torch.clamp(h @ p["up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ p["down"].T


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def run_mixer(layer, h, p, eps):
    m = layer["mixer"]
    if layer["type"] == "mamba2":
        return mamba2_mixer(h, p, m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"], eps)
    if layer["type"] == "lightning":
        return lightning_mixer(h, p, m["heads"], m["dim"], m["vdim"], m["decay"], eps)
    if layer["type"] == "attention":
        return attention_mixer(h, p, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], m.get("softcap"),
                               (m.get("mask") or {}).get("size"), eps)
    raise ValueError(layer["type"])


def forward(config, weights, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence; ``weights`` {name: float64 tensor}.  ``layers_out`` (a list) receives the
    stream after every layer."""
    eps, m = config["norm"]["eps"], config.get("residual_mult", 1.0)
    x = embed(tokens, weights["embed"], config["embedding"]["scale"])
    for i, layer in enumerate(config["layers"]):
        src = layer.get("weights_of", i)
        pre = f"l{src}."
        y = run_mixer(layer, x, sub(weights, pre + "mix."), eps)
        x = x + m * rms_norm(y, weights[pre + "norm1"], eps) * weights[pre + "ls1"]
        if layer.get("mlp") is not None:
            y = clamped_glu(x, sub(weights, pre + "mlp."), layer["mlp"]["limit"])
            x = x + m * rms_norm(y, weights[pre + "norm2"], eps) * weights[pre + "ls2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, weights["final.norm"], eps) @ weights["head"].T
