"""A plain, slow Tiralix decoder: whole sequences, no cache, one function per mechanism.

Nothing here is shared with the library under test.  It reads ``config.json`` keys from a
plain dictionary and tensors from a plain name -> tensor mapping and computes on the CPU in
the dtype it is given (float64 by default, so that it is the more exact side of a comparison).

The design in this file's notation (T tokens, width d):

* x = E[ids].
* a layer: x += s1 * N1(mixer(x)); x += s2 * N2(ff(x)).  The sublayers read x as it is; N is the RMS norm
  with a weight, s1 and s2 are vectors of the layer ("layer scale").
* mixer ``parallel``: cl * softmax_attention(x) + cr * decayed_linear_attention(x).
  - softmax attention: grouped heads; q and k are RMS-normed over their whole projections (all heads
    at once) with weights; the leading r dimensions of every head are rotated in pairs (i, i + r/2) with
    frequencies that are slowed down by wavelength (see ``rotary_frequencies``) and with cos and sin enlarged by
    one constant; scores * c; causal softmax; every head's result times sigmoid of one number per
    head (a projection of x); output projection.
  - decayed linear attention: q, k, v = silu(projections); per head S <- a_h S + k v^T; o = S^T q; the
    heads' results together are RMS-normed with a weight, multiplied by sigmoid(projection of x), projected.
* mixer ``mamba1``: [u | z] = W_in x; u <- silu(causal convolution per channel with bias);
  [r | B | C] = W_x u; delta = softplus(W_dt r + b); A = -exp(A_log);
  S[c, n] <- exp(delta_c A[c, n]) S[c, n] + delta_c u_c B_n; y_c = sum_n S[c, n] C_n + D_c u_c;
  out = W_o (y * silu(z)).
* feed-forward: g = min(W_g x, L); u = clamp(W_u x, -L, L); W_d (g * sigmoid(1.702 g) * (u + 1)).
* logits = cap * tanh(scale * E N(x) / cap).
"""
from __future__ import annotations

import math
from typing import Mapping, Optional, Sequence

import torch


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w.to(x.dtype)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def rotary_frequencies(r: int, base: float, scaling: Optional[Mapping]):
    """(f_i for i < r/2, magnitude).  Unscaled f_i = base^(-2i/r).  With scaling (factor s, original
    length L, turn counts fast and slow): the dimension at which a frequency makes t turns over L is
    D(t) = r ln(L / (2 pi t)) / (2 ln base); lo = max(floor(D(fast)), 0), hi = min(ceil(D(slow)), r - 1);
    the blend weight of dimension i is clamp((i - lo) / max(hi - lo, 0.001), 0, 1); the frequency becomes
    f_i / s * weight + f_i * (1 - weight), and cos and sin are multiplied by 0.1 ln(s) + 1."""
    out, mag = [], 1.0
    if scaling:
        s, L = float(scaling["factor"]), float(scaling["original"])

        def D(t):
            return r * math.log(L / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(D(float(scaling["fast"]))), 0)
        hi = min(math.ceil(D(float(scaling["slow"]))), r - 1)
        mag = 0.1 * math.log(s) + 1.0
    for i in range(r // 2):
        f = float(base) ** (-2.0 * i / r)
        if scaling:
            wgt = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f = f / s * wgt + f * (1.0 - wgt)
        out.append(f)
    return out, mag


def rotate(x: torch.Tensor, positions: Sequence[int], r: int, freqs: Sequence[float], mag: float) -> torch.Tensor:
    """x [T, heads, dim]: the pair (i, i + r/2) of every head's leading r dimensions turns by p * f_i."""
    y = x.clone()
    h = r // 2
    p = torch.tensor(list(positions), dtype=x.dtype)[:, None, None]
    f = torch.tensor(list(freqs), dtype=x.dtype)[None, None, :]
    c, s = torch.cos(p * f) * mag, torch.sin(p * f) * mag
    a, b = x[..., :h], x[..., h:r]
    y[..., :h] = a * c - b * s
    y[..., h:r] = b * c + a * s
    return y


def softmax_attention(x: torch.Tensor, m: Mapping, W: Mapping[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    T, dt = x.shape[0], x.dtype
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(x @ W[pre + "q"].to(dt).T, W[pre + "q.norm"], eps).view(T, H, dk)
    k = rms_norm(x @ W[pre + "k"].to(dt).T, W[pre + "k.norm"], eps).view(T, G, dk)
    v = (x @ W[pre + "v"].to(dt).T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        freqs, mag = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q = rotate(q, range(T), rot["dims"], freqs, mag)
        k = rotate(k, range(T), rot["dims"], freqs, mag)
    gate = torch.sigmoid(x @ W[pre + "g"].to(dt).T)                     # [T, H]
    out = torch.zeros(T, H, dv, dtype=dt)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ W[pre + "o"].to(dt).T


def decayed_linear_attention(x: torch.Tensor, m: Mapping, W: Mapping[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    T, dt = x.shape[0], x.dtype
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(x @ W[pre + "q"].to(dt).T).view(T, H, dk)
    k = silu(x @ W[pre + "k"].to(dt).T).view(T, H, dk)
    v = silu(x @ W[pre + "v"].to(dt).T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=dt)
    for h in range(H):
        S = torch.zeros(dk, dv, dtype=dt)
        a = float(m["decay"][h])
        for t in range(T):
            S = a * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    y = rms_norm(out.reshape(T, H * dv), W[pre + "norm"], eps) * torch.sigmoid(x @ W[pre + "g"].to(dt).T)
    return y @ W[pre + "o"].to(dt).T


def parallel_mixer(x, m, W, pre, eps):
    left = softmax_attention(x, m["left"], W, pre + "left.", eps)
    right = decayed_linear_attention(x, m["right"], W, pre + "right.", eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def causal_conv(u: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y[t] = b + sum_j w[:, j] u[t - taps + 1 + j], zeros before the start."""
    T = u.shape[0]
    taps = w.shape[1]
    y = b.to(u.dtype).expand(T, -1).clone()
    for j in range(taps):
        shift = taps - 1 - j
        if shift < T:
            y[shift:] += w[:, j].to(u.dtype) * u[:T - shift]
    return y


def selective_scan_mixer(x: torch.Tensor, m: Mapping, W: Mapping[str, torch.Tensor], pre: str) -> torch.Tensor:
    T, dt = x.shape[0], x.dtype
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    uz = x @ W[pre + "in"].to(dt).T
    u, z = uz[:, :inner], uz[:, inner:]
    u = silu(causal_conv(u, W[pre + "conv"], W[pre + "conv.b"]))
    rbc = u @ W[pre + "x"].to(dt).T
    r, B, C = rbc[:, :R], rbc[:, R:R + N], rbc[:, R + N:]
    delta = softplus(r @ W[pre + "dt"].to(dt).T + W[pre + "dt.b"].to(dt))
    A = -torch.exp(W[pre + "A_log"].to(dt))
    D = W[pre + "D"].to(dt)
    S = torch.zeros(inner, N, dtype=dt)
    y = torch.zeros(T, inner, dtype=dt)
    for t in range(T):
        S = torch.exp(delta[t][:, None] * A) * S + (delta[t] * u[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * u[t]
    return (y * silu(z)) @ W[pre + "o"].to(dt).T


def clamped_gated_ff(x: torch.Tensor, f: Mapping, W: Mapping[str, torch.Tensor], pre: str) -> torch.Tensor:
    dt, L = x.dtype, float(f["limit"])
    g = torch.clamp(x @ W[pre + "gate"].to(dt).T, max=L)
    u = torch.clamp(x @ W[pre + "up"].to(dt).T, min=-L, max=L)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[pre + "down"].to(dt).T


def forward(cfg: Mapping, W: Mapping[str, torch.Tensor], ids: Sequence[int], dtype=torch.float64, streams=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``streams``: a list that receives x after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"].to(dtype)[torch.tensor(list(ids), dtype=torch.long)]
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        if l["type"] == "parallel":
            y = parallel_mixer(x, l["mixer"], W, p + "mix.", eps)
        elif l["type"] == "mamba1":
            y = selective_scan_mixer(x, l["mixer"], W, p + "mix.")
        else:
            raise ValueError(l["type"])
        x = x + W[p + "ls1"].to(dtype) * rms_norm(y, W[p + "norm1"], eps)
        if l.get("mlp") is not None:
            y = clamped_gated_ff(x, l["mlp"], W, p + "mlp.")
            x = x + W[p + "ls2"].to(dtype) * rms_norm(y, W[p + "norm2"], eps)
        if streams is not None:
            streams.append(x.clone())
    xn = rms_norm(x, W["final.norm"], eps)
    logits = xn @ W["embed"].to(dtype).T * float(cfg["logit_scale"])
    cap = float(cfg["logit_softcap"])
    return cap * torch.tanh(logits / cap)
