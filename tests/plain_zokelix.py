"""Plain, slow float64 implementation of the Zokelix design, one function per mechanism,
written from the design's equations with torch on the CPU.  It shares no code with the
package: it reads ``config.json`` as a dictionary and the checkpoint by tensor name.

Notation: h [T, width] is what a sublayer reads (the residual stream itself); every layer
does x <- x + norm1(mixer(x)) and then, if it has a feed-forward, x <- x + norm2(ff(x)).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


# ---------------------------------------------------------------------- feed-forwards
def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dense_ff(h, W, p):
    """down(gelu_tanh(gate h + b) * (up h + b)) + b."""
    g = h @ W[p + "gate"].T + W[p + "gate.b"]
    u = h @ W[p + "up"].T + W[p + "up.b"]
    return (gelu_tanh(g) * u) @ W[p + "down"].T + W[p + "down.b"]


def expert_ff(x, W, p, limit):
    """One expert: g = min(gate x, limit), u = clamp(up x, +-limit), down(g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(x @ W[p + "gate"].T, max=limit)
    u = torch.clamp(x @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def router_choice(h, W, p, top):
    """(ids [T, top], scores [T, top]): the largest sigmoid(router h), not renormalised."""
    s = torch.sigmoid(h @ W[p + "router"].T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val


def routed_ff(h, W, p, ml):
    """sum over a token's chosen experts of expert(score * h): the score scales the INPUT."""
    top, limit = ml["router"]["top"], ml["expert"]["limit"]
    idx, val = router_choice(h, W, p, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += expert_ff(val[t, j] * h[t], W, f"{p}e{e}.", limit)
    return out


# ---------------------------------------------------------------------- rotary
def rotary_frequencies(rot):
    """(f [dims/2], factor on cos and sin).  With scaling: d(t) = dims ln(original / (2 pi t))
    / (2 ln base); lo = max(floor(d(fast)), 0); hi = min(ceil(d(slow)), dims - 1); the pair i is
    blended towards f_i / factor by clamp((i - lo) / max(hi - lo, 0.001), 0, 1)."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def d(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(d(sc["fast"])), 0)
    hi = min(math.ceil(d(sc["slow"])), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_pairs(x, positions, f, factor):
    """Dimension 2i pairs with 2i + 1: (u, v) -> (u cos a - v sin a, v cos a + u sin a),
    a = position * f_i, cos and sin times ``factor``.  x [T, ..., 2 len(f)]."""
    a = positions.to(F64)[:, None] * f[None, :]
    c, s = torch.cos(a) * factor, torch.sin(a) * factor
    while c.dim() < x.dim():
        c, s = c.unsqueeze(1), s.unsqueeze(1)
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


# ---------------------------------------------------------------------- latent attention
def latent_rows(h, W, p, mx, eps, positions):
    """What the design keeps per token: the normed latent c [T, rank] and the rotated shared
    key part [T, rot_dim]."""
    r, nrot = mx["kv_rank"], mx["rot"]["dims"]
    ckr = h @ W[p + "dkv"].T
    c = rms_norm(ckr[:, :r], W[p + "dkv.norm"], eps)
    kr = ckr[:, r:].clone()
    f, factor = rotary_frequencies(mx["rot"])
    kr[:, :nrot] = rotate_pairs(kr[:, :nrot], positions, f, factor)
    return c, kr


def latent_attention(h, W, p, mx, eps):
    """Per head: key = [W_uk c | shared rotated part], value = W_uv c, causal softmax of
    (q . key) * scale; then W_o on the concatenated heads."""
    T = h.shape[0]
    H, dn, dr, dv = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"]
    nrot = mx["rot"]["dims"]
    positions = torch.arange(T)
    q = (h @ W[p + "q"].T).view(T, H, dn + dr)
    f, factor = rotary_frequencies(mx["rot"])
    q_rot = q[..., dn:].clone()
    q_rot[..., :nrot] = rotate_pairs(q_rot[..., :nrot], positions, f, factor)
    c, kr = latent_rows(h, W, p, mx, eps, positions)
    k_nope = (c @ W[p + "uk"].T).view(T, H, dn)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        s = (torch.einsum("hd,jhd->hj", q[t, :, :dn], k_nope[:t + 1])
             + torch.einsum("hd,jd->hj", q_rot[t], kr[:t + 1])) * mx["scale"]
        out[t] = torch.einsum("hj,jhd->hd", torch.softmax(s, -1), v[:t + 1])
    return out.reshape(T, H * dv) @ W[p + "o"].T


# ---------------------------------------------------------------------- channel delta
def short_conv_silu(x, w):
    """y[t, c] = silu(sum_j w[c, j] x[t - (taps - 1) + j, c]), zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=F64), x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y += xp[j:j + T] * w[:, j][None, :]
    return y * torch.sigmoid(y)


def delta_scan(q, k, v, beta, g):
    """One head: q, k, g [T, dk], v [T, dv], beta [T].  S <- g (.) S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q (after the write)."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=F64)
    o = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o


def channel_delta(h, W, p, mx, eps):
    T = h.shape[0]
    H, KH, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = short_conv_silu(h @ W[p + "q"].T, W[p + "q.conv"]).view(T, KH, dk)
    k = short_conv_silu(h @ W[p + "k"].T, W[p + "k.conv"]).view(T, KH, dk)
    v = short_conv_silu(h @ W[p + "v"].T, W[p + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    a = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    g = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None]
                  * torch.nn.functional.softplus(a).view(T, H, dk))
    gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).view(T, H, dv)
    o = torch.stack([delta_scan(q[:, hh // (H // KH)], k[:, hh // (H // KH)], v[:, hh],
                                beta[:, hh], g[:, hh]) for hh in range(H)], dim=1)
    o = rms_norm(o, W[p + "norm"], eps) * gate
    return o.reshape(T, H * dv) @ W[p + "o"].T


# ---------------------------------------------------------------------- the model
def forward_layers(cfg, weights, tokens):
    """(residual after every layer [layers, T, width], logits [T, vocab]), float64."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(list(tokens))]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mixer = {"latent_attention": latent_attention, "channel_delta": channel_delta}[layer["type"]]
        x = x + rms_norm(mixer(x, W, p + "mix.", layer["mixer"], eps), W[p + "norm1"], eps)
        ml = layer.get("mlp")
        if ml:
            y = dense_ff(x, W, p + "mlp.") if ml["kind"] == "dense" else routed_ff(x, W, p + "mlp.", ml)
            x = x + rms_norm(y, W[p + "norm2"], eps)
        after.append(x.clone())
    return torch.stack(after), rms_norm(x, W["final.norm"], eps) @ W["head"].T


def forward_logits(cfg, weights, tokens):
    return forward_layers(cfg, weights, tokens)[1]
