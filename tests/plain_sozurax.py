"""A plain, slow statement of the Sozurax decoder: whole sequences, no cache, float64, one function a
mechanism.  It shares no code with the engine; the tests compare the engine with it.

Notation: T tokens, W the model width, rows are tokens.  Linear weights are [out, in].

* layer norm:        y = (x - mean) / sqrt(var + eps) * w + b,  var = mean((x - mean)^2)
* RMS norm:          y = x / sqrt(mean(x^2) + eps) (* w)
* input convolution: g_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j)      (zeros before the sequence)
* gated recurrence:  S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,  o_t = S_t^T q_t,
                     f = l + (1 - l) * sigmoid(W_f h + b_f),  q = silu(W_q h)
* latent attention:  keys and values are made from a per-token latent c = rms(W_dkv h)[:rank] and one rotated
                     key part shared by the heads; a query sees the last `window` positions
* PolyNorm:          a N(z) + b N(z^2) + c N(z^3) + e,   N(u) = u / sqrt(mean(u^2) + eps)
* routed experts:    the `top` largest router logits choose experts, weights softmax over the chosen logits
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def input_conv(h, w):
    """h [T, W], w [W, taps] -> h + causal depthwise convolution of h."""
    T, taps = h.shape[0], w.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def hgrn2_mixer(h, p, heads, dim, vdim, eps):
    """p: dict with q, f, f.b, lower, v, norm, o."""
    T = h.shape[0]
    q = silu(h @ p["q"].T).view(T, heads, dim)
    v = (h @ p["v"].T).view(T, heads, vdim)
    low = p["lower"]
    f = (low + (1 - low) * torch.sigmoid(h @ p["f"].T + p["f.b"])).view(T, heads, dim)
    S = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    out = rms_norm(out, p["norm"], eps)
    return out.reshape(T, heads * vdim) @ p["o"].T


def rotate_interleaved(x, positions, base, dims):
    """x [T, ..., D]: the first `dims` entries of the last axis are rotated in pairs (2i, 2i+1) by the angle
    position * base^(-2i/dims)."""
    T = x.shape[0]
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F64)
    freq = base ** (-2 * i / dims)
    ang = positions.to(F64)[:, None] * freq[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_kv(h, p, kv_rank, rot_dim, rot_base, rot_dims, eps):
    """The per-token latent and the rotated shared key part, from the layer that owns W_dkv."""
    T = h.shape[0]
    d = h @ p["dkv"].T
    c = rms_norm(d[:, :kv_rank], p["dkv.norm"], eps)
    kr = rotate_interleaved(d[:, kv_rank:kv_rank + rot_dim], torch.arange(T), rot_base, rot_dims)
    return c, kr


def latent_attention_mixer(h, p, m, eps, shared_kv=None):
    """m: the mixer's sizes and constants (heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mask.size,
    rot.base, rot.dims).  shared_kv: (c, rotated key part) of another layer, or None to make one's own.
    Returns (output, (c, kr))."""
    T = h.shape[0]
    H, dim, rd, vd, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, rdims, window = m["rot"]["base"], m["rot"]["dims"], m["mask"]["size"]
    cq = rms_norm(h @ p["dq"].T, p["dq.norm"], eps)
    q = (cq @ p["uq"].T).view(T, H, dim + rd)
    q_plain, q_rot = q[..., :dim], rotate_interleaved(q[..., dim:], torch.arange(T), base, rdims)
    c, kr = shared_kv if shared_kv is not None else latent_kv(h, p, R, rd, base, rdims, eps)
    k_plain = (c @ p["uk"].T).view(T, H, dim)
    val = (c @ p["uv"].T).view(T, H, vd)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thd,sd->hts", q_rot, kr)) * m["scale"]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = (i - j >= 0) & (i - j < window)
    scores = scores.masked_fill(~visible, float("-inf"))
    w = torch.softmax(scores, dim=-1)
    out = torch.einsum("hts,shv->thv", w, val).reshape(T, H * vd)
    return out @ p["o"].T, (c, kr)


def polynorm(z, coef, eps):
    a, b, c, e = [coef[i] for i in range(4)]
    return a * rms_norm(z, None, eps) + b * rms_norm(z ** 2, None, eps) + c * rms_norm(z ** 3, None, eps) + e


def dense_ff(h, p, eps):
    return polynorm(h @ p["up"].T, p["act"], eps) @ p["down"].T


def gated_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def routed_ff(h, p, n_experts, top, has_shared):
    logits = h @ p["router"].T + p["router.b"]
    vals, idx = torch.topk(logits, top, dim=-1)
    wts = torch.softmax(vals, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(idx[t, k])
            out[t] += wts[t, k] * gated_expert(h[t:t + 1], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    if has_shared:
        out = out + gated_expert(h, p["shared.gate"], p["shared.up"], p["shared.down"])
    return out


def sub(weights, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, ids, return_layers=False):
    """Logits [T, vocab] of a whole sequence.  weights: {name: tensor}, any float type."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(ids)] * config.get("embedding", {}).get("scale", 1.0)
    kv_of = {}
    per_layer = []
    for i, layer in enumerate(config["layers"]):
        L = f"l{i}."
        m = layer["mixer"]
        h = input_conv(layer_norm(x, w[L + "norm1"], w[L + "norm1.b"], eps), w[L + "canon1"])
        p = sub(w, L + "mix.")
        if layer["type"] == "hgrn2":
            x = x + hgrn2_mixer(h, p, m["heads"], m["dim"], m["vdim"], eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            out, kv = latent_attention_mixer(h, p, m, eps, kv_of[src] if src is not None else None)
            if src is None:
                kv_of[i] = kv
            x = x + out
        else:
            raise ValueError(layer["type"])
        ff = layer.get("mlp")
        if ff is not None:
            h = input_conv(layer_norm(x, w[L + "norm2"], w[L + "norm2.b"], eps), w[L + "canon2"])
            p = sub(w, L + "mlp.")
            if ff["kind"] == "dense":
                x = x + dense_ff(h, p, eps)
            else:
                x = x + routed_ff(h, p, ff["router"]["experts"], ff["router"]["top"], ff.get("shared") is not None)
        per_layer.append(x.clone())
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    if return_layers:
        return logits, torch.stack(per_layer)
    return logits
