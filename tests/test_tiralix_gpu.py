"""The Tiralix decoder and its mechanisms against the plain implementation (tests/plain/tiralix_plain.py).

Small configurations with weights made here (large enough that every non-linearity is at work).  Per mechanism:
the kernel against the plain function, also across two steps where it carries a state.  Whole models: prompts
against token-by-token decoding, portions down to two tokens, batches of unequal requests against each alone, slots
and pages that are used again, long decoding, and greedy generation through the engine's own loop.  Where random
weights would hide a fault (a far key among hundreds, a state that was lost on the way), the weights are made so
that one early token decides the result.
"""
import json
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from helpers import REL, random_ids, rel_err, run_schedule
from plain import tiralix_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _left(heads, kv, dim, vdim, rot=None, scale=0.5):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    return m


def _par(left, right, cl, cr):
    return {"left": left, "right": right, "left_scale": cl, "right_scale": cr}


YARN = {"base": 500.0, "dims": 8, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 2.0}}

# unlike layers in another order than any usual one: a layer without feed-forward, kv heads equal to heads and to one,
# the whole head rotated and a part of it, equal and unequal key/value sizes, a decay of exactly 1, a value size that is
# no multiple of 32, a key size above 32, one tap and three, a state size that is no multiple of 8
CFG_A = {
    "architecture": "Tiralix", "vocab": 101, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 0.5, "logit_softcap": 8.0,
    "layers": [
        {"type": "parallel", "mixer": _par(_left(6, 2, 16, 8, YARN, 0.3), {"heads": 2, "dim": 24, "vdim": 40, "decay": [1.0, 0.9]}, 1.3, 0.7),
         "mlp": {"kind": "dense", "ff": 88, "limit": 1.5}},
        {"type": "mamba1", "mixer": {"inner": 96, "state": 5, "dt_rank": 3, "conv": 3}, "mlp": None},
        {"type": "parallel", "mixer": _par(_left(2, 2, 32, 32, {"base": 10000.0, "dims": 32}, 0.2),
                                           {"heads": 3, "dim": 40, "vdim": 16, "decay": [0.97, 0.5, 0.999]}, 0.6, 1.1),
         "mlp": {"kind": "dense", "ff": 40, "limit": 0.5}},
        {"type": "mamba1", "mixer": {"inner": 80, "state": 20, "dt_rank": 8, "conv": 1}, "mlp": {"kind": "dense", "ff": 64, "limit": 3.0}},
    ],
}
# one head everywhere, no rotation at all, a step-size rank of one, four taps, no cap on the logits worth the name
CFG_B = {
    "architecture": "Tiralix", "vocab": 67, "width": 48, "norm": {"eps": 1e-6}, "logit_scale": 1.0, "logit_softcap": 50.0,
    "layers": [
        {"type": "mamba1", "mixer": {"inner": 48, "state": 16, "dt_rank": 1, "conv": 4}, "mlp": {"kind": "dense", "ff": 56, "limit": 2.5}},
        {"type": "parallel", "mixer": _par(_left(1, 1, 64, 16, None, 0.15), {"heads": 1, "dim": 8, "vdim": 32, "decay": [0.8]}, 1.0, 1.0),
         "mlp": None},
    ],
}
CONFIGS = {"A": CFG_A, "B": CFG_B}


def make_tensors(cfg, seed):
    """Weights by name with the shapes the library asks for; scales chosen so that activations are of order one."""
    from ithaca_b200.config import config_from_dict
    from ithaca_b200.engine.model import weight_manifest
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, req in weight_manifest(config_from_dict(cfg)[1].model_spec()).items():
        shape = tuple(req.shape)
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif name.endswith((".ls1", ".ls2")):
            t = 0.5 + 0.2 * r
        elif "norm" in name or name.endswith(".D"):
            t = 1.0 + 0.1 * r
        elif name.endswith(".conv"):
            t = 0.5 * r
        elif name.endswith((".conv.b", ".dt.b")):
            t = 0.3 * r - (0.5 if name.endswith(".dt.b") else 0.0)
        elif name.endswith(".A_log"):
            t = 0.5 * r
        else:
            t = r * (1.2 / shape[1] ** 0.5)
        out[name] = t.bfloat16()
    return out


def _write(tmp, cfg, tensors, tag):
    from ithaca_b200.weights.safetensors_io import write_file
    d = os.path.join(str(tmp), tag)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(d, "model.safetensors"), tensors, {"format": "pt"})
    return d


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("tiralix")
    out = {}
    for i, (n, c) in enumerate(CONFIGS.items()):
        t = make_tensors(c, 40 + i)
        out[n] = (_write(root, c, t, n), t)
    return out


def _close(got, want, dtype):
    """float32: every logit within the tolerance.  bfloat16: these weights are large enough that every non-linearity
    bends, and 16-bit operands then leave single rows at two or three hundredths of the logits' range: the median row
    must hold the tolerance and none may pass two and a half times it (a wrong key or a lost state moves a row by tens
    of hundredths, see the needle tests)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape and np.all(np.isfinite(got))
    rows = np.abs(got - want).reshape(-1, want.shape[-1]).max(-1) / max(np.abs(want).max(), 1e-30)
    if dtype == "float32":
        return bool(rows.max() < REL[dtype])
    return bool(np.median(rows) < REL[dtype] and rows.max() < 2.5 * REL[dtype])


def _plain(cfg, t, ids):
    return P.forward(cfg, t, ids).numpy()


def _ctx(lo, hi, slots):
    """The device arrays of a step in which sequence b brings positions lo[b] .. hi[b] - 1."""
    new = [h - l for l, h in zip(lo, hi)]
    i32 = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    return SimpleNamespace(
        n_seqs=len(lo), is_decode=all(n == 1 for n in new), slots=i32(slots), cu_seqlens=i32(np.concatenate([[0], np.cumsum(new)])),
        kv_lens=i32(hi), token_seq=i32(np.repeat(np.arange(len(lo)), new)),
        token_pos=i32(np.concatenate([np.arange(l, h) for l, h in zip(lo, hi)]) if sum(new) else []))


STEPS = [([0, 0, 0], [67, 1, 60]), ([67, 1, 60], [70, 2, 131]), ([70, 2, 131], [71, 3, 132]), ([71, 3, 132], [72, 4, 133])]
TOTAL = [72, 4, 133]


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("d", [48, 256, 1100])
def test_norm_behind_a_sublayer_with_layer_scale(d):
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(d)
    y, res = torch.randn(9, d, generator=g) * 3, torch.randn(9, d, generator=g)
    w, ls = torch.randn(d, generator=g), torch.randn(d, generator=g)
    want = res.double() + ls.double() * P.rms_norm(y.double(), w, 1e-5)
    r = res.clone().to(DEV)
    copy = torch.empty(9, d, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm_add(y.to(DEV), w.to(DEV), 1e-5, r, scale=ls.to(DEV), copy=copy)
    assert rel_err(r.cpu().numpy(), want.numpy()) < 2e-6
    assert torch.equal(copy.cpu(), r.cpu().bfloat16())
    r2 = res.clone().to(DEV)
    ops.rmsnorm_add(y.to(DEV), w.to(DEV), 1e-5, r2, mult=0.25)                      # no scale vector, a constant instead
    assert rel_err(r2.cpu().numpy(), (res.double() + 0.25 * P.rms_norm(y.double(), w, 1e-5)).numpy()) < 2e-6


def test_yarn_frequencies_and_magnitude():
    from ithaca_b200.parts.position import inverse_frequencies, magnitude
    for dims, base, sc in [(8, 500.0, YARN["scaling"]), (64, 10000.0, {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}),
                           (6, 30.0, {"factor": 1.5, "original": 16, "fast": 3.0, "slow": 0.5})]:
        mine = {"rope_type": "yarn", "factor": sc["factor"], "original_max_position_embeddings": sc["original"],
                "fast_turns": sc["fast"], "slow_turns": sc["slow"]}
        f, mag = P.rotary_frequencies(dims, base, sc)
        assert np.allclose(inverse_frequencies(dims, base, mine), np.array(f), rtol=1e-6)
        assert abs(magnitude(mine) - mag) < 1e-12 and mag > 1.0
        assert not np.allclose(np.array(f), np.array(P.rotary_frequencies(dims, base, None)[0]))       # the scaling does something


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,hdv,rot,pairing,norm", [(6, 2, 16, 8, 8, 0, True), (2, 2, 32, 32, 32, 0, True), (3, 1, 24, 40, 0, 0, True),
                                                           (4, 2, 16, 16, 12, 1, False), (1, 1, 64, 16, 64, 0, True)])
def test_projection_norm_rotation_append_kernel(dtype, nh, nkv, hd, hdv, rot, pairing, norm):
    """q and k normed over all their heads at once, rotated by half-split or neighbouring pairs with a magnitude, k and v
    into scrambled pages; the inputs are a column range of a wider matrix."""
    from test_kernels_gpu import Paged
    from ithaca_b200.csrc import ops
    lens, new = [70, 5, 130], [3, 5, 66]
    T, pad = sum(new), 7
    g = torch.Generator().manual_seed(hd + rot)
    wide = torch.randn(T, pad + (nh + nkv) * hd + nkv * hdv + 3, generator=g)
    qw, kw = torch.randn(nh * hd, generator=g), torch.randn(nkv * hd, generator=g)
    freqs, mag = P.rotary_frequencies(rot, 300.0, {"factor": 3.0, "original": 40, "fast": 6.0, "slow": 1.0}) if rot else ([], 1.0)
    pk, pv = Paged(lens, nkv, hd, dtype, 5), Paged(lens, nkv, hdv, dtype, 5)
    k_d, v_d, tab = pk.dev()[0], pv.dev()[0], pk.dev()[2]
    seq = torch.from_numpy(np.repeat(np.arange(3), new).astype(np.int32)).to(DEV)
    posn = np.concatenate([np.arange(l - n, l) for l, n in zip(lens, new)])
    q_out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    p = wide.to(DEV)[:, pad:]
    ops.norm_rope_append(p, 0, nh * hd, (nh + nkv) * hd, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None, 1e-5, q_out,
                         k_d, v_d, seq, torch.from_numpy(posn.astype(np.int32)).to(DEV), tab,
                         torch.tensor(freqs, dtype=torch.float32, device=DEV) if rot else None, mag, nh, rot, pairing, True, status)
    assert status.item() == 0
    x = wide[:, pad:].double()
    q, k, v = x[:, :nh * hd], x[:, nh * hd:(nh + nkv) * hd], x[:, (nh + nkv) * hd:(nh + nkv) * hd + nkv * hdv]
    if norm:
        q, k = P.rms_norm(q, qw, 1e-5), P.rms_norm(k, kw, 1e-5)
    q, k = q.reshape(T, nh, hd), k.reshape(T, nkv, hd)
    if rot:
        if pairing == 1:                                       # neighbouring pairs: to half-split order, rotate, back
            order = torch.stack((torch.arange(rot // 2) * 2, torch.arange(rot // 2) * 2 + 1), 0).reshape(-1)
            back = torch.argsort(order)
            turn = lambda a: torch.cat((P.rotate(a[..., order], posn, rot, freqs, mag)[..., back], a[..., rot:]), -1)
            q, k = turn(q), turn(k)
        else:
            q, k = P.rotate(q, posn, rot, freqs, mag), P.rotate(k, posn, rot, freqs, mag)
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    assert rel_err(q_out.float().cpu().numpy(), q.reshape(T, -1).numpy()) < tol
    t = 0
    for b, (l, n) in enumerate(zip(lens, new)):
        for j in range(l - n, l):
            kk, vv = k_d.cpu()[pk.table[b, j // 64], :, j % 64].float(), v_d.cpu()[pk.table[b, j // 64], :, j % 64].float()
            assert rel_err(kk.numpy(), k[t].numpy()) < tol and rel_err(vv.numpy(), v[t].reshape(nkv, hdv).numpy()) < tol
            t += 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_gate_and_gated_norm_kernels(dtype):
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    T, H, hdv = 11, 5, 24
    att = torch.randn(T, H * hdv, generator=g).to(dtype)
    p = torch.randn(T, 3 + H + H * hdv, generator=g)
    mid = torch.zeros(T, 10 + 2 * H * hdv, dtype=dtype, device=DEV)
    ops.head_gate(att.to(DEV), p.to(DEV), 3, mid[:, 10:10 + H * hdv], H, 0.8)
    want = att.double().view(T, H, hdv) * torch.sigmoid(p[:, 3:3 + H].double())[:, :, None] * 0.8
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    assert rel_err(mid[:, 10:10 + H * hdv].float().cpu().numpy(), want.reshape(T, -1).numpy()) < tol
    x, w = torch.randn(T, H * hdv, generator=g) * 5, torch.randn(H * hdv, generator=g)
    ops.gated_rmsnorm(x.to(DEV), w.to(DEV), 1e-5, p.to(DEV), 3 + H, mid[:, 10 + H * hdv:], 1.7)
    want = P.rms_norm(x.double(), w, 1e-5) * torch.sigmoid(p[:, 3 + H:].double()) * 1.7
    assert rel_err(mid[:, 10 + H * hdv:].float().cpu().numpy(), want.numpy()) < tol
    assert float(mid[:, :10].abs().max()) == 0.0                       # nothing outside the column ranges is touched


def test_gate_with_limits_and_logit_cap_kernels():
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(4)
    gu = torch.randn(13, 2 * 40, generator=g) * 3
    got = ops.glu_act(gu.to(DEV), torch.float32, 1.702, 1.5, 1.0)
    gg, uu = torch.clamp(gu[:, :40].double(), max=1.5), torch.clamp(gu[:, 40:].double(), -1.5, 1.5)
    assert rel_err(got.cpu().numpy(), (gg * torch.sigmoid(1.702 * gg) * (uu + 1)).numpy()) < 2e-6
    inter = torch.stack((gu[:, :40], gu[:, 40:]), 2).reshape(13, 80).contiguous()
    assert torch.equal(ops.glu_act(inter.to(DEV), torch.float32, 1.702, 1.5, 1.0, interleaved=True), got)
    v = (torch.randn(5, 77, generator=g) * 20).to(DEV)
    want = 15.0 * torch.tanh(v.double().cpu() * 2.0 / 15.0)
    assert rel_err(ops.scale_softcap_(v.clone(), 2.0, 15.0).cpu().numpy(), want.numpy()) < 2e-6
    assert rel_err(ops.scale_softcap_(v.clone(), 0.5, 0.0).cpu().numpy(), (v.cpu().double() * 0.5).numpy()) < 1e-7


@pytest.mark.parametrize("T", [5, 12, 40, 300, 700])
def test_gate_with_limits_in_the_products_epilogues(monkeypatch, T):
    """The 16-bit feed-forward joins gate and up inside the product that makes them: the warp-level kernel for a few tokens,
    the tcgen05 kernel above, its pair mode for many.  Inputs large enough that the limits bite."""
    from ithaca_b200.config.spec import PartSpec
    from ithaca_b200.csrc import ops
    from ithaca_b200.parts import FEED_FORWARDS, Runtime
    d, ff = 128, 328
    g = torch.Generator().manual_seed(T)
    spec = PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": ff, "activation": "swish", "alpha": 1.702, "limit": 1.0,
                                  "up_shift": 1.0}, {"gate": "gate", "up": "up", "down": "down"})
    t = {"gate": (torch.randn(ff, d, generator=g) * 0.15).bfloat16(), "up": (torch.randn(ff, d, generator=g) * 0.15).bfloat16(),
         "down": (torch.randn(d, ff, generator=g) * 0.1).bfloat16()}
    part = FEED_FORWARDS.get("gated_mlp")(spec, t, Runtime(dtype="bfloat16", device=DEV))

    def never(*a, **k):
        raise AssertionError("the gate ran as a kernel of its own")
    monkeypatch.setattr(ops, "glu_act", never)
    x = torch.randn(T, d, generator=g).bfloat16()
    want = P.clamped_gated_ff(x.double(), {"limit": 1.0}, t, "")
    out = torch.full((T, d), 7.0, device=DEV)
    part.forward(x.to(DEV), None, out, accumulate=False)
    assert rel_err(out.cpu().numpy(), want.numpy()) < 2e-2
    free = P.clamped_gated_ff(x.double(), {"limit": 100.0}, t, "")
    assert rel_err(free.numpy(), want.numpy()) > 0.1                      # the limits matter here


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 2, 4])
def test_causal_convolution_with_its_ring(dtype, taps):
    """Three sequences in four steps (a prompt, a portion, two single tokens: the last steps read everything older from
    the ring) against the plain convolution of the whole sequences; the ring starts with another user's leftovers."""
    from ithaca_b200.csrc import ops
    C, pad = 40, 5
    g = torch.Generator().manual_seed(taps)
    u = [torch.randn(l, pad + C, generator=g) for l in TOTAL]
    w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    ring = torch.full((6, taps, C), 9.0, device=DEV) if taps > 1 else None
    got = [[] for _ in TOTAL]
    for lo, hi in STEPS:
        ctx = _ctx(lo, hi, [2, 0, 5])
        x = torch.cat([a[l:h] for a, l, h in zip(u, lo, hi)]).to(DEV)
        y = ops.causal_conv(x[:, pad:], w.t().contiguous().to(DEV), b.to(DEV), ring, ctx, dtype)
        for i, part in enumerate(torch.split(y.float().cpu(), [h - l for l, h in zip(lo, hi)])):
            got[i].append(part)
    for i in range(3):
        want = P.silu(P.causal_conv(u[i][:, pad:].double(), w, b))
        assert rel_err(torch.cat(got[i]).numpy(), want.numpy()) < (3e-6 if dtype == torch.float32 else 8e-3), i


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,N", [(40, 5), (96, 16), (33, 20), (64, 64)])
def test_selective_scan_kernel(dtype, inner, N):
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(inner + N)
    R = 3
    u = [(torch.randn(l, inner, generator=g)).to(dtype) for l in TOTAL]
    dt = [torch.randn(l, inner, generator=g) - 1.0 for l in TOTAL]
    bc = [torch.randn(l, R + 2 * N, generator=g) for l in TOTAL]
    z = [torch.randn(l, 2 * inner, generator=g) for l in TOTAL]
    A, D, bias = -torch.exp(torch.randn(inner, N, generator=g) * 0.5), torch.randn(inner, generator=g), torch.randn(inner, generator=g) * 0.3
    state = torch.full((6, 2, inner, N), 7.0, device=DEV)                   # leftovers that a new sequence must not see
    got = [[] for _ in TOTAL]
    for lo, hi in STEPS:
        ctx = _ctx(lo, hi, [2, 0, 5])
        cat = lambda xs: torch.cat([a[l:h] for a, l, h in zip(xs, lo, hi)]).to(DEV)
        y = ops.selective_scan(cat(u), cat(dt), bias.to(DEV), A.to(DEV), cat(bc), R, R + N, D.to(DEV), cat(z)[:, inner:], state, ctx, dtype)
        for i, part in enumerate(torch.split(y.float().cpu(), [h - l for l, h in zip(lo, hi)])):
            got[i].append(part)
    for i, l in enumerate(TOTAL):
        S, want = torch.zeros(inner, N, dtype=torch.float64), []
        ud, dd = u[i].double(), P.softplus(dt[i].double() + bias.double())
        for t in range(l):
            S = torch.exp(dd[t][:, None] * A.double()) * S + (dd[t] * ud[t])[:, None] * bc[i][t, R:R + N].double()[None, :]
            want.append((S @ bc[i][t, R + N:].double() + D.double() * ud[t]) * P.silu(z[i][t, inner:].double()))
        assert rel_err(torch.cat(got[i]).numpy(), torch.stack(want).numpy()) < (5e-6 if dtype == torch.float32 else 8e-3), i


@pytest.mark.parametrize("H,dk,dv", [(2, 24, 40), (3, 40, 16), (1, 8, 32), (2, 96, 64), (1, 130, 33)])
def test_decayed_linear_attention_kernel(H, dk, dv):
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(dk + dv)
    pad = 3
    p = [torch.randn(l, pad + H * (2 * dk + dv), generator=g) for l in TOTAL]
    decay = torch.tensor([1.0, 0.9, 0.5][:H])
    state = torch.full((6, 2, H, dk, dv), 7.0, device=DEV)
    got = [[] for _ in TOTAL]
    for lo, hi in STEPS:
        ctx = _ctx(lo, hi, [2, 0, 5])
        x = torch.cat([a[l:h] for a, l, h in zip(p, lo, hi)]).to(DEV)
        o = ops.decay_attention(x[:, pad:], 0, H * dk, 2 * H * dk, decay.to(DEV), state, ctx, H, dk, dv, True)
        for i, part in enumerate(torch.split(o.cpu(), [h - l for l, h in zip(lo, hi)])):
            got[i].append(part)
    for i, l in enumerate(TOTAL):
        x = P.silu(p[i][:, pad:].double())
        q, k, v = x[:, :H * dk].view(l, H, dk), x[:, H * dk:2 * H * dk].view(l, H, dk), x[:, 2 * H * dk:].view(l, H, dv)
        want = torch.zeros(l, H, dv, dtype=torch.float64)
        for h in range(H):
            S = torch.zeros(dk, dv, dtype=torch.float64)
            for t in range(l):
                S = float(decay[h]) * S + torch.outer(k[t, h], v[t, h])
                want[t, h] = S.T @ q[t, h]
        assert rel_err(torch.cat(got[i]).numpy(), want.reshape(l, -1).numpy()) < 5e-6, i


# ------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompt_matches_plain(models, name, dtype):
    from ithaca_b200 import Engine
    d, t = models[name]
    ids = random_ids(150, CONFIGS[name]["vocab"], 3)
    want = _plain(CONFIGS[name], t, ids)
    eng = Engine(d, dtype=dtype, max_tokens=1024)
    s = eng.alloc_slot()
    got = eng.step([s], [ids], "all").cpu().numpy()
    eng.check_status()
    assert _close(got, want, dtype)
    for n in (1, 2, 3):                                                 # the first tokens of a sequence alone
        s2 = eng.alloc_slot()
        assert _close(eng.step([s2], [ids[:n]], "all").cpu().numpy(), want[:n], dtype)
        eng.free_slot(s2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_schedules_agree_with_plain(models, name, dtype):
    """Token by token; portions of 2, 3, 7, 64 and 65 tokens; a prompt and then decoding across page edges; unequal
    requests in one batch and decoded together; every position against the plain whole sequence."""
    from ithaca_b200 import Engine
    d, t = models[name]
    V = CONFIGS[name]["vocab"]
    reqs = {"a": random_ids(140, V, 11), "b": random_ids(67, V, 12), "c": random_ids(1, V, 13), "d": random_ids(9, V, 14)}
    want = {r: _plain(CONFIGS[name], t, ids) for r, ids in reqs.items()}
    eng = Engine(d, dtype=dtype, max_tokens=2048)

    def portions(r, sizes):
        out, left = [], len(reqs[r])
        while left:
            for n in sizes:
                n = min(n, left)
                if n:
                    out.append([(r, n)])
                    left -= n
        return out

    schedules = {
        "token by token": [[("b", 1)] for _ in range(67)],
        "portions": portions("a", [2, 3, 7, 64, 65]),
        "pairs": portions("b", [2]),
        "prompt then decode": [[("a", 60)]] + [[("a", 1)] for _ in range(80)],
        "batch": [[("c", 1), ("a", 100), ("d", 5), ("b", 30)]] + [[("a", 1), ("d", 1), ("b", 1)] for _ in range(4)]
                 + [[("a", 1), ("b", 1)] for _ in range(33)] + [[("a", 1)] for _ in range(3)],
        "mixed portions": [[("a", 64), ("b", 1)], [("b", 64), ("a", 3)], [("a", 73), ("b", 2)]],
    }
    for label, sched in schedules.items():
        got = run_schedule(eng, reqs, sched)
        for r, lg in got.items():
            assert _close(lg, want[r], dtype), (label, r)
        eng.cache.table.check_consistent()
        assert eng.cache.table.n_slots_in_use() == 0


def test_float32_does_not_depend_on_the_cutting(models):
    """The recurrences run token by token and every sum's order is fixed by sizes alone: in float32 two cuttings of the
    same tokens, alone or beside others, give the same bits."""
    from ithaca_b200 import Engine
    d, t = models["A"]
    reqs = {"a": random_ids(150, 101, 21), "b": random_ids(40, 101, 22)}
    eng = Engine(d, dtype="float32", max_tokens=2048)
    whole = run_schedule(eng, reqs, [[("a", 150)], [("b", 40)]])
    cut = run_schedule(eng, reqs, [[("a", 63), ("b", 2)], [("a", 2), ("b", 38)], [("a", 1)], [("a", 84)]])
    for r in reqs:
        assert np.array_equal(whole[r], cut[r]), r


def test_slots_pages_and_states_are_used_again(models):
    """A small cache: requests come and go, so slots, pages, states and rings are handed out again, also to shorter
    sequences whose first tokens must see nothing of what lay there before."""
    from ithaca_b200 import Engine
    d, t = models["A"]
    eng = Engine(d, dtype="float32", max_tokens=64 * 6, max_slots=2)
    for round_ in range(4):
        reqs = {"x": random_ids(130 - 40 * round_, 101, 20 + round_), "y": random_ids(3 + round_, 101, 30 + round_)}
        got = run_schedule(eng, reqs, [[("x", len(reqs["x"]) - 2), ("y", 2)], [("x", 1), ("y", 1)], [("x", 1)]]
                           + [[("y", 1)] for _ in range(round_)])
        for r, ids in reqs.items():
            assert rel_err(got[r], _plain(CFG_A, t, ids)) < REL["float32"], (round_, r)
        eng.cache.table.check_consistent()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    from ithaca_b200 import Engine
    d, t = models["A"]
    ids = random_ids(330, 101, 77)
    want = _plain(CFG_A, t, ids)
    eng = Engine(d, dtype=dtype, max_tokens=1024)
    got = run_schedule(eng, {"a": ids}, [[("a", 10)]] + [[("a", 1)] for _ in range(320)])["a"]
    assert _close(got, want, dtype)


# ------------------------------------------------------------------------------------------ one early token decides
D = 32


def _needle_tensors(cfg):
    """Token 1 (the needle) and token 2 (the query) point along axis 0, every other token along an axis of its own."""
    t = make_tensors(cfg, 9)
    g = torch.Generator().manual_seed(1)
    emb = torch.randn(40, D, generator=g) * 0.05
    for i in range(3, 40):
        emb[i, 8 + i % 20] += 4.0
    emb[1] += torch.eye(D)[0] * 4 + torch.eye(D)[5] * 2
    emb[2] += torch.eye(D)[0] * 4 - torch.eye(D)[5] * 2
    t["embed"] = emb.bfloat16()
    for n in ("l0.norm1", "final.norm"):
        t[n] = torch.ones(D).bfloat16()
    t["l0.ls1"] = torch.full((D,), 3.0).bfloat16()                      # what the mixer adds outweighs the token's own embedding
    return t


def _needle_attention():
    """The softmax branch alone decides: k copies the input and q copies it with the mark's axis turned over (after the
    projection-wide norm: a token's own axes), so the query's best match is the needle, ahead of itself and of hundreds of
    others, and the value it fetches carries the needle's mark."""
    cfg = {"architecture": "Tiralix", "vocab": 40, "width": D, "norm": {"eps": 1e-6}, "logit_scale": 1.0, "logit_softcap": 30.0,
           "layers": [{"type": "parallel", "mlp": None,
                       "mixer": _par(_left(1, 1, D, D, None, 0.6), {"heads": 1, "dim": 8, "vdim": 8, "decay": [0.9]}, 1.0, 0.0)}]}
    t = _needle_tensors(cfg)
    for r in "qkvo":
        t[f"l0.mix.left.{r}"] = torch.eye(D).bfloat16()
    flip = torch.eye(D)
    flip[5, 5] = -1.0
    t["l0.mix.left.q"] = flip.bfloat16()
    t["l0.mix.left.q.norm"] = t["l0.mix.left.k.norm"] = torch.ones(D).bfloat16()
    t["l0.mix.left.g"] = torch.zeros(1, D).bfloat16()
    return cfg, t


def _needle_linear():
    """The decayed branch alone decides, with a decay of one: only the needle's key has weight along axis 0, where the
    query looks, so what the query reads from the state is the needle's value, however long ago it was added."""
    cfg = {"architecture": "Tiralix", "vocab": 40, "width": D, "norm": {"eps": 1e-6}, "logit_scale": 1.0, "logit_softcap": 30.0,
           "layers": [{"type": "parallel", "mlp": None,
                       "mixer": _par(_left(1, 1, 8, 8, None, 0.5), {"heads": 1, "dim": D, "vdim": D, "decay": [1.0]}, 0.0, 1.0)}]}
    t = _needle_tensors(cfg)
    pick = torch.zeros(D, D)
    pick[0, 0] = 2.0                                                    # q and k: axis 0 only; silu(0) = 0 elsewhere
    t["l0.mix.right.q"] = t["l0.mix.right.k"] = pick.bfloat16()
    mark = torch.eye(D)
    mark[5, 5] = 3.0                                                    # the mark's axis counts: silu(6) against silu(-6)
    t["l0.mix.right.v"], t["l0.mix.right.o"] = mark.bfloat16(), torch.eye(D).bfloat16()
    t["l0.mix.right.g"] = torch.zeros(D, D).bfloat16()
    t["l0.mix.right.norm"] = torch.ones(D).bfloat16()
    return cfg, t


def _needle_scan():
    """A selective scan that forgets slowly (tiny step sizes, small A): the needle's large embedding is written into the
    state once and is still most of it hundreds of tokens later."""
    cfg = {"architecture": "Tiralix", "vocab": 40, "width": D, "norm": {"eps": 1e-6}, "logit_scale": 1.0, "logit_softcap": 30.0,
           "layers": [{"type": "mamba1", "mlp": None, "mixer": {"inner": 48, "state": 12, "dt_rank": 4, "conv": 3}}]}
    t = _needle_tensors(cfg)
    t["embed"][1] *= 12
    t["l0.mix.dt.b"] = torch.full((48,), -4.0).bfloat16()
    t["l0.mix.dt"] = (t["l0.mix.dt"].float() * 0.05).bfloat16()
    t["l0.mix.A_log"] = torch.full((48, 12), -4.0).bfloat16()
    t["l0.mix.D"] = torch.zeros(48).bfloat16()
    return cfg, t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("make", [_needle_attention, _needle_linear, _needle_scan])
def test_the_one_early_token_that_matters(tmp_path, make, dtype):
    """The needle sits at the very start, at a page's last and first place and elsewhere far back; the query comes at the
    end of a prompt, is decoded alone after it, or follows a short portion; a batch neighbour runs beside it."""
    from ithaca_b200 import Engine
    cfg, t = make()
    d = _write(tmp_path, cfg, t, "needle")
    eng = Engine(d, dtype=dtype, max_tokens=4096)
    n = 400
    hay = [3 + (i * 7) % 37 for i in range(n)]
    tol = REL[dtype] if dtype == "float32" else 6e-2
    none = list(hay)
    none[n - 1] = 2
    base = _plain(cfg, t, none)[n - 1]
    for at in (0, 1, 63, 64, 127, 128, 300):
        ids = list(hay)
        ids[at], ids[n - 1] = 1, 2
        want = _plain(cfg, t, ids)[n - 1]
        assert rel_err(want, base) > 0.15, at                              # the test has teeth: without the needle, other logits
        for cut in (n, n - 1, n - 5, 65):
            s, other = eng.alloc_slot(), eng.alloc_slot()
            lg = eng.step([other, s], [hay[:7], ids[:cut]], "last")
            for x in ids[cut:]:
                lg = eng.step([s, other], [[x], [5]], "last")
            eng.free_slot(s)
            eng.free_slot(other)
            row = lg.cpu().numpy()[1 if cut == n else 0]
            assert rel_err(row, want) < tol, (at, cut)
    eng.check_status()


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_engine(models, name, graphs):
    """More prompts than slots, unequal lengths, the generation loop's own batching (and its graph-replayed decode
    steps, which launch a step ahead and may drop it: the states are kept by parity so that this changes nothing)."""
    from ithaca_b200 import Engine
    d, t = models[name]
    V = CONFIGS[name]["vocab"]
    prompts = [random_ids(n, V, 60 + n) for n in (1, 6, 70, 20)]
    eng = Engine(d, dtype="float32", max_tokens=64 * 12, max_slots=3, graphs=graphs)
    assert (eng._decoder is not None) == graphs                            # every part of the design may be replayed
    got = eng.generate(prompts, max_tokens=12, temp=0.0, rep_pen=1.0, stop_token_ids=[])
    for p, g in zip(prompts, got):
        assert len(g) == 12
        lgs = P.forward(CONFIGS[name], t, list(p) + g[:-1])
        for i, tok in enumerate(g):
            lg = lgs[len(p) - 1 + i]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > 1e-4 * float(lg.abs().max()):
                assert tok == int(lg.argmax()), (len(p), i)
    assert eng.cache.table.n_slots_in_use() == 0
    # requests that end at different times: the step launched ahead is dropped when the batch changes
    got = eng.generate(prompts[:3], max_tokens=9, temp=0.0, rep_pen=1.0, stop_token_ids=[got[0][4], got[2][6]])
    for p, g in zip(prompts, got):
        lgs = P.forward(CONFIGS[name], t, list(p) + g)
        for i, tok in enumerate(g):
            lg = lgs[len(p) - 1 + i]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > 1e-4 * float(lg.abs().max()):
                assert tok == int(lg.argmax()), (len(p), i)


# ------------------------------------------------------------------------------------------ the programs
def test_trace_replay_and_command_line(models, tmp_path):
    import subprocess
    import sys
    from helpers import ROOT
    d, t = models["A"]
    V = 101
    reqs = {"p": random_ids(70, V, 90), "q": random_ids(3, V, 91), "r": random_ids(130, V, 92)}
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": reqs["p"][:66], "want": [0, 65]}, {"id": "q", "tokens": reqs["q"][:1], "want": []},
                                     {"id": "r", "tokens": reqs["r"][:126], "want": [125]}], "end": []}]
    for i in range(4):
        ent = [{"id": "p", "tokens": [reqs["p"][66 + i]], "want": [0]}, {"id": "r", "tokens": [reqs["r"][126 + i]], "want": [0]}]
        if i < 2:
            ent.insert(1, {"id": "q", "tokens": [reqs["q"][1 + i]], "want": [0] if i == 1 else []})
        steps.append({"step": 1 + i, "entries": ent, "end": (["q"] if i == 1 else []) + (["p", "r"] if i == 3 else [])})
    out = tmp_path / "out"
    for dtype in ("float32", "bfloat16"):
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "210"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                           timeout=900)
        assert p.returncode == 0, p.stderr[-3000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(5)]
        want = {r: _plain(CFG_A, t, ids) for r, ids in reqs.items()}
        tol = REL[dtype] * (1 if dtype == "float32" else 2)
        got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, V)
        assert rel_err(got0, np.stack([want["p"][0], want["p"][65], want["r"][125]])) < tol
        got2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(3, V)
        assert rel_err(got2, np.stack([want["p"][67], want["q"][2], want["r"][127]])) < tol
        got4 = np.fromfile(out / "4.f32", dtype="<f4").reshape(2, V)
        assert rel_err(got4, np.stack([want["p"][69], want["r"][129]])) < tol

    cli = [sys.executable, os.path.join(ROOT, "bin", "ithaca"), "--model", d, "--dtype", "float32"]
    p = subprocess.run(cli + ["--describe"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and p.stdout.count("outnorm") == 4 and p.stdout.count("parallel") == 2 and p.stdout.count("mamba1") == 2, p.stderr[-2000:]
    prompt = random_ids(11, V, 93)
    p = subprocess.run(cli + ["--prompt", ",".join(map(str, prompt)), "-n", "5", "--rep-pen", "1.0", "--stop-ids", ""],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    from ithaca_b200 import Engine
    eng = Engine(d, dtype="float32", max_tokens=512)
    assert [int(x) for x in p.stdout.strip().split(",")] == eng.generate([prompt], max_tokens=5, temp=0.0, rep_pen=1.0, stop_token_ids=[])[0]
