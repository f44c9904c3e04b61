"""A plain, slow Vebisun decoder: whole sequences, no cache, one function per mechanism.

Nothing here is shared with the library under test.  It reads ``config.json`` keys from a
plain dictionary and tensors from a plain name -> tensor mapping and computes on the CPU in
the dtype it is given (float64 by default, so that it is the more exact side of a comparison).

The design in this file's notation (T tokens, width d):

* x0 = E[ids] * c_embed.
* a layer: x += m * LN1b(mixer(LN1(x))); x += m * LN2b(ff(LN2(x))); LN is the layer norm with
  weight and bias, m a constant of the model.
* layers lo..hi-1 are run R times in a row with the same weights; before every pass after the
  first, x += x0.  Then the remaining layers, the final norm and the head.
* mixer: grouped-query attention with a short causal convolution over time on q, k and v right
  after their projections, rotation of the leading r dimensions of q and k in neighbouring pairs
  (frequencies rescaled by wavelength), scores * c then cap * tanh(. / cap), a sliding window of
  w keys (own position included), softmax, output projection.
* feed-forward: a mixture of small gated feed-forwards; the router's softmax scores choose the
  ``top`` best experts among the ``keep`` best groups of neighbouring experts (a group counts by
  its best expert); the chosen experts' outputs are added with their scores as weights.
"""
from __future__ import annotations

import math
from typing import List, Mapping, Sequence

import torch


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w.to(x.dtype) + b.to(x.dtype)


def short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y[t] = sum_j w[:, j] * u[t - taps + 1 + j], zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j].to(u.dtype) * u[s]
    return y


def rotary_frequencies(r: int, base: float, scaling: Mapping) -> torch.Tensor:
    """f_i = base^(-2i/r), then by wavelength l = 2 pi / f: kept when l < orig/high, divided by
    ``factor`` when l > orig/low, blended linearly in orig/l between."""
    out = []
    for i in range(r // 2):
        f = float(base) ** (-2.0 * i / r)
        if scaling:
            factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
            orig = float(scaling["original"])
            l = 2.0 * math.pi / f
            if l < orig / high:
                pass
            elif l > orig / low:
                f = f / factor
            else:
                s = (orig / l - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def rotate_pairs(x: torch.Tensor, positions: Sequence[int], freqs: torch.Tensor) -> torch.Tensor:
    """x [T, heads, dim]; dimensions (2i, 2i+1), i < len(freqs), are turned by position * f_i."""
    r = 2 * len(freqs)
    ang = torch.tensor(list(positions), dtype=torch.float64)[:, None] * freqs[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:r:2], x[..., 1:r:2]
    out[..., 0:r:2] = a * c - b * s
    out[..., 1:r:2] = b * c + a * s
    return out


def attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, cap=None, window=None) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, Dv] of one sequence -> [T, H, Dv]: scores * scale, capped by
    cap * tanh(. / cap), position i sees j with 0 <= i - j < window, softmax, weighted values."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window:
        seen = seen & (i - j < window)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * float(scale)
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~seen, float("-inf"))
        out[:, hh] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def attention_mixer(h: torch.Tensor, mc: Mapping, w: Mapping[str, torch.Tensor], prefix: str) -> torch.Tensor:
    T = h.shape[0]
    dt = h.dtype
    H, G, D, Dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    q = h @ w[prefix + "q"].to(dt).T
    k = h @ w[prefix + "k"].to(dt).T
    v = h @ w[prefix + "v"].to(dt).T
    if mc.get("conv"):
        q = short_conv(q, w[prefix + "q.conv"])
        k = short_conv(k, w[prefix + "k.conv"])
        v = short_conv(v, w[prefix + "v.conv"])
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, Dv)
    rot = mc.get("rot")
    if rot:
        f = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_pairs(q, range(T), f), rotate_pairs(k, range(T), f)
    out = attention_core(q, k, v, mc["scale"], mc.get("softcap"), (mc.get("mask") or {}).get("size"))
    return out.reshape(T, H * Dv) @ w[prefix + "o"].to(dt).T


def route(h: torch.Tensor, rc: Mapping, w_router: torch.Tensor):
    """Returns (chosen experts [T, top], their weights [T, top])."""
    E, top = rc["experts"], rc["top"]
    s = torch.softmax(h @ w_router.to(h.dtype).T, dim=-1)
    groups = rc.get("groups")
    allowed = torch.ones_like(s, dtype=torch.bool)
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        best = s.view(-1, n, per).max(-1).values
        kept = best.topk(keep, dim=-1).indices
        gmask = torch.zeros_like(best, dtype=torch.bool)
        gmask.scatter_(1, kept, True)
        allowed = gmask[:, :, None].expand(-1, n, per).reshape(-1, E)
    chosen = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    return chosen, s.gather(1, chosen)


def expert_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str) -> torch.Tensor:
    dt = h.dtype
    g = h @ w[prefix + "gate"].to(dt).T
    u = h @ w[prefix + "up"].to(dt).T
    return (g * torch.sigmoid(g) * u) @ w[prefix + "down"].to(dt).T


def moe_ff(h: torch.Tensor, fc: Mapping, w: Mapping[str, torch.Tensor], prefix: str) -> torch.Tensor:
    chosen, weight = route(h, fc["router"], w[prefix + "router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(chosen[t].tolist(), weight[t]):
            out[t] += p * expert_ff(h[t:t + 1], w, f"{prefix}e{e}.")[0]
    return out


def layer(x: torch.Tensor, i: int, cfg: Mapping, w: Mapping[str, torch.Tensor]) -> torch.Tensor:
    lc, eps, m = cfg["layers"][i], float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    p = f"l{i}."

    def ln(name, z):
        return layer_norm(z, w[p + name], w[p + name + ".b"], eps)

    if lc["type"] != "attention":
        raise ValueError(f"unknown mixer {lc['type']!r}")
    x = x + m * ln("norm1b", attention_mixer(ln("norm1", x), lc["mixer"], w, p + "mix."))
    if lc.get("mlp") is not None:
        if lc["mlp"]["kind"] != "moe":
            raise ValueError(f"unknown feed-forward {lc['mlp']['kind']!r}")
        x = x + m * ln("norm2b", moe_ff(ln("norm2", x), lc["mlp"], w, p + "mlp."))
    return x


def layer_runs(cfg: Mapping) -> List[tuple]:
    """(layer, adds the embedding output first) for every run, in order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    lo, hi, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(lo)]
    for r in range(times):
        runs += [(i, r > 0 and i == lo) for i in range(lo, hi)]
    runs += [(i, False) for i in range(hi, n)]
    return runs


def forward(ids: Sequence[int], cfg: Mapping, w: Mapping[str, torch.Tensor], dtype=torch.float64, trace=None):
    """Logits [T, vocab] of one whole sequence.  ``trace``: a list that receives x after every layer run."""
    x0 = w["embed"].to(dtype)[torch.as_tensor(list(ids), dtype=torch.long)] * float(cfg["embedding"]["scale"])
    x = x0.clone()
    for i, add in layer_runs(cfg):
        if add:
            x = x + x0
        x = layer(x, i, cfg, w)
        if trace is not None:
            trace.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], float(cfg["norm"]["eps"]))
    return x @ w["head"].to(dtype).T
