"""Plain, slow float64 implementation of the Mizerax design, one function per mechanism,
written from the design's equations with torch on the CPU.  It shares no code with the
package: it reads ``config.json`` as a dictionary and the checkpoint by tensor name.

Notation: x [T, width] is the residual stream of ONE request whose tokens stand at
positions 0 .. T-1; a layer does  x <- x + m (ls1 * mixer(h) + ls2 * ff(h))  with
h = layer_norm(x): both sublayers read the same normed rows.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------------- norms
def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * weight + bias over the last dimension."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * weight + bias


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


# ---------------------------------------------------------------------- attention
def head_slopes(heads):
    """slope of head h = 2 ^ (-8 (h + 1) / heads)."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F64)


def query_temperature(positions, coef, every):
    """1 + coef ln(floor((p + 1) / every) + 1) for every position p."""
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(F64) + 1.0)


def sink_softmax(scores):
    """exp(s_j) / (1 + sum_j exp(s_j)) over the last dimension; masked entries are -inf.
    The one stands for a key whose score is 0 and that carries no value."""
    m = torch.clamp(scores.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(scores - m)
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def attention_scores(q, k, scale, slopes):
    """q [T, H, d], k [S, H, d] (keys already repeated per query head), query i at position
    S - T + i: q.k * scale - slope_h (i - j) for j <= i, -inf beyond."""
    T, S = q.shape[0], k.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(S - T, S).view(1, T, 1)
    j = torch.arange(S).view(1, 1, S)
    s = s - slopes.view(-1, 1, 1) * (i - j).to(F64)
    return s.masked_fill(j > i, float("-inf"))


def attention_mixer(h, W, p, mx, eps, start=0, past=None):
    """The mixer on rows h [T, width] at positions start .. start + T - 1.  ``past`` = (k, v) of
    the positions before (already normed), or None.  Returns (out [T, width], (k, v) of all
    positions so far)."""
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].T).view(T, H, d)
    k = (h @ W[p + "k"].T).view(T, G, d)
    v = (h @ W[p + "v"].T).view(T, G, dv)
    q = rms_norm(q, W[p + "q.norm"], eps)
    k = rms_norm(k, W[p + "k.norm"], eps)
    pos = torch.arange(start, start + T)
    qt = mx.get("q_temp")
    if qt:
        q = q * query_temperature(pos, qt["coef"], qt["every"]).view(T, 1, 1)
    if past is not None:
        k = torch.cat([past[0], k], 0)
        v = torch.cat([past[1], v], 0)
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    w = sink_softmax(attention_scores(q, kk, mx["scale"], head_slopes(H)))
    o = torch.einsum("hij,jhd->ihd", w, vv)
    gate = torch.sigmoid(h @ W[p + "g"].T)                      # [T, H]
    o = o * gate.unsqueeze(-1)
    return o.reshape(T, H * dv) @ W[p + "o"].T, (k, v)


# ---------------------------------------------------------------------- feed-forward
def silu_expert(x, W, p):
    """down(silu(gate x) * (up x))."""
    g = x @ W[p + "gate"].T
    return (g * torch.sigmoid(g) * (x @ W[p + "up"].T)) @ W[p + "down"].T


def router_choice(h, W, p, top):
    """(ids [T, top], weights [T, top]): s = softmax(router h) over all outputs; chosen by
    s + correction, weighted by s itself."""
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    _, idx = torch.topk(s + W[p + "correction"], top, dim=-1)
    return idx, torch.gather(s, -1, idx)


def routed_ff(h, W, p, ml):
    """sum over the chosen outputs of weight * expert(h); the last ``identity`` router outputs
    stand for experts that return h itself; plus the shared expert on every row."""
    ro = ml["router"]
    n_real = ro["experts"]
    idx, val = router_choice(h, W, p, ro["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ro["top"]):
            e = int(idx[t, j])
            y = silu_expert(h[t], W, f"{p}e{e}.") if e < n_real else h[t]
            out[t] += val[t, j] * y
    if ml.get("shared"):
        out = out + silu_expert(h, W, p + "shared.")
    return out


# ---------------------------------------------------------------------- the model
def layer_runs(cfg):
    """Indices of the layers in the order they run: the layers before the loop once, the
    loop's layers ``times`` times over, the rest once.  Yields (layer, pass_begins)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(cfg, weights, tokens, start=0, past=None, want_layers=False):
    """Logits [T, vocab] (float64) of one request's tokens at positions start ...; ``past``
    is the list (one entry a layer run) of (k, v) this function returned for the positions
    before.  Returns (logits, new past[, residual after every layer run])."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    m = cfg.get("residual_mult", 1.0)
    ids = torch.as_tensor(tokens, dtype=torch.long)
    T = ids.numel()
    x = W["embed"][ids] + W["pos"][start:start + T]
    x0 = x.clone()
    new_past, after = [], []
    for r, (i, begins) in enumerate(layer_runs(cfg)):
        layer, p = cfg["layers"][i], f"l{i}."
        if begins:
            x = torch.cat([x, x0], -1) @ W["loop.in"].T
        h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        mix, kv = attention_mixer(h, W, p + "mix.", layer["mixer"], eps, start,
                                  None if past is None else past[r])
        new_past.append(kv)
        y = W[p + "ls1"] * mix
        if layer.get("mlp"):
            y = y + W[p + "ls2"] * routed_ff(h, W, p + "mlp.", layer["mlp"])
        x = x + m * y
        after.append(x.clone())
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["embed"].T
    if want_layers:
        return logits, new_past, torch.stack(after)
    return logits, new_past
