"""The Vebisun decoder and its mechanisms against the plain implementation (tests/plain/vebisun_plain.py).

Small configurations with random weights, made here.  Per mechanism: the kernel against the plain
function.  Whole models: prompts against token-by-token decoding, portions down to two tokens, batches of
unequal requests against each alone, slots and pages that are used again, keys at page and window edges in
prompts and in decoding, long decoding, and greedy generation through the engine's own loop.  Where random
weights would hide a fault (a window one key off, a far key), the weights are made so that one key decides
the result.
"""
import json
import os

import numpy as np
import pytest
import torch

from helpers import REL, random_ids, rel_err, run_schedule
from plain import vebisun_plain as P

pytestmark = pytest.mark.gpu

ROT = {"base": 1000.0, "dims": 8, "scaling": {"factor": 4.0, "high": 4.0, "low": 1.0, "original": 24}}


def _moe(E, top, ff, groups=None):
    r = {"experts": E, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def _mixer(heads, kv, dim, vdim, conv=None, rot=None, window=None, softcap=None, scale=8.0):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if conv is not None:
        m["conv"] = conv
    if rot is not None:
        m["rot"] = rot
    if window is not None:
        m["mask"] = {"size": window}
    if softcap is not None:
        m["softcap"] = softcap
    return m


# three unlike layers, a loop over the last two that runs three times
CFG_A = {
    "architecture": "Vebisun", "vocab": 97, "width": 64, "embedding": {"scale": 2.5}, "residual_mult": 0.7,
    "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _mixer(4, 2, 16, 24, conv=3, rot=ROT, window=9, softcap=3.0),
         "mlp": _moe(8, 3, 40, groups=(4, 2))},
        {"type": "attention", "mixer": _mixer(2, 2, 32, 32, conv=2, rot={"base": 50.0, "dims": 32}), "mlp": None},
        {"type": "attention", "mixer": _mixer(3, 1, 16, 16, window=70, softcap=5.0), "mlp": _moe(4, 1, 24)},
    ],
    "loop": {"start": 1, "stop": 3, "times": 3},
}
# no loop; a window of exactly one page and of one key; four taps and one tap; every expert used; one group kept of one
CFG_B = {
    "architecture": "Vebisun", "vocab": 61, "width": 48, "embedding": {"scale": 1.0}, "residual_mult": 1.0,
    "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _mixer(3, 3, 16, 8, conv=4, rot={"base": 10000.0, "dims": 16}, window=64, softcap=2.0),
         "mlp": _moe(3, 3, 20, groups=(1, 1))},
        {"type": "attention", "mixer": _mixer(1, 1, 32, 48, conv=1, rot=ROT, window=1), "mlp": _moe(6, 2, 16, groups=(3, 3))},
    ],
}
CONFIGS = {"A": CFG_A, "B": CFG_B}


def _write(tmp, cfg, seed, tensors=None):
    from ithaca_b200.weights import write_random_model
    d = os.path.join(str(tmp), f"m{abs(hash(json.dumps(cfg, sort_keys=True))) % 10**8}_{seed}")
    write_random_model(d, cfg, seed)
    if tensors is not None:
        from ithaca_b200.weights.safetensors_io import write_file
        write_file(os.path.join(d, "model.safetensors"), tensors, {"format": "pt"})
    return d


def _load(d):
    from safetensors import safe_open
    t = {}
    with safe_open(os.path.join(d, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            t[k] = f.get_tensor(k)
    with open(os.path.join(d, "config.json")) as f:
        return json.load(f), t


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("vebisun")
    return {n: _write(root, c, seed=5 + i) for i, (n, c) in enumerate(CONFIGS.items())}


def _close(got, want, dtype):
    """float32: every logit within the tolerance.  bfloat16: a router reads the 16-bit rounding of its input, so among
    hundreds of random tokens a few sit close enough to a tie to choose another expert than the float64 side; such
    a token's row is off by more than rounding.  Nine rows in ten must hold the tolerance and none may be far off
    (a wrong key or a lost state moves a row by tens of percent, see the one-key test, which has no router)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape and np.all(np.isfinite(got))
    rows = np.abs(got - want).reshape(-1, want.shape[-1]).max(-1) / max(np.abs(want).max(), 1e-30)
    if dtype == "float32":
        return bool(rows.max() < REL[dtype])
    return bool(np.mean(rows < REL[dtype]) >= 0.9 and rows.max() < 5 * REL[dtype])


def _plain(d, ids):
    cfg, t = _load(d)
    return P.forward(ids, cfg, t).numpy()


# ------------------------------------------------------------------------------------------ configuration
def test_config_reads_every_size_from_the_file(models):
    from ithaca_b200.config import config_from_model_dir, validate_schedule
    arch, cfg = config_from_model_dir(models["A"])
    spec = cfg.model_spec()
    validate_schedule(spec)
    assert arch.name == "Vebisun" and spec.vocab_size == 97 and spec.hidden_size == 64
    runs = [(e.layer, e.adds_input) for e in spec.schedule]
    assert runs == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False)]
    assert len({e.cache for e in spec.schedule}) == len(spec.schedule)            # every pass has its own cache
    assert runs == P.layer_runs(CFG_A)
    assert spec.layers[1].feed_forward is None and spec.layers[0].mixer["v_head_dim"] == 24


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("d", [48, 256, 5000])
def test_layer_norm_kernel(d):
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(d)
    x = (torch.randn(7, d, generator=g) * 3 + 1.5).cuda()
    w, b = torch.randn(d, generator=g).cuda(), torch.randn(d, generator=g).cuda()
    want = P.layer_norm(x.double().cpu(), w.cpu(), b.cpu(), 1e-5)
    got = ops.layernorm(x, w, b, 1e-5, torch.float32)
    assert rel_err(got.cpu().numpy(), want.numpy()) < 2e-6
    rows = torch.tensor([5, 0, 5], dtype=torch.int32).cuda()
    assert torch.equal(ops.layernorm(x, w, b, 1e-5, torch.float32, rows_in=rows), got[rows.long()])
    assert rel_err(ops.layernorm(x, w, b, 1e-5, torch.bfloat16).float().cpu().numpy(), want.numpy()) < 1e-2
    stream = torch.randn(7, d, generator=g).cuda()
    want2 = stream.double().cpu() + 0.3 * want
    ops.layernorm(x, w, b, 1e-5, torch.float32, into=stream, mult=0.3)
    assert rel_err(stream.cpu().numpy(), want2.numpy()) < 2e-6


@pytest.mark.parametrize("E,top,groups", [(8, 3, (4, 2)), (20, 2, (2, 1)), (6, 6, None), (5, 1, None), (12, 4, (3, 3)), (64, 8, (8, 3))])
def test_router_kernel(E, top, groups):
    from ithaca_b200.csrc import ops
    g = torch.Generator().manual_seed(E * 10 + top)
    z = torch.randn(50, E, generator=g) * 2
    rc = {"experts": E, "top": top}
    if groups:
        rc["groups"] = {"count": groups[0], "keep": groups[1]}
    want_e, want_w = P.route(z.double(), rc, torch.eye(E))
    got_e, got_w = ops.moe_route(z.cuda(), top, *(groups or (0, 0)))
    assert torch.equal(got_e.cpu().long(), want_e)
    assert rel_err(got_w.cpu().numpy(), want_w.numpy()) < 1e-6


def test_router_prefers_the_better_group_over_the_better_expert():
    """Two groups of two; the best single expert sits in group 0, but only one group is kept and two experts are
    chosen: both come from the group whose best is best, whatever the other group's second holds."""
    from ithaca_b200.csrc import ops
    z = torch.tensor([[3.0, -5.0, 2.5, 2.4], [0.0, 1.0, 5.0, -9.0]]).cuda()
    e, w = ops.moe_route(z, 2, 2, 1)
    assert e.cpu().tolist() == [[0, 1], [2, 3]]
    s = torch.softmax(z.cpu(), -1)
    assert torch.allclose(w.cpu(), torch.stack([s[0, [0, 1]], s[1, [2, 3]]]), atol=1e-7)          # not renormalized


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top,ff,d", [(1, 4, 2, 24, 32), (70, 8, 3, 40, 64), (300, 3, 1, 100, 72)])
def test_mixture_of_experts_part(dtype, T, E, top, ff, d):
    from ithaca_b200.config.spec import PartSpec
    from ithaca_b200.parts import FEED_FORWARDS, Runtime
    g = torch.Generator().manual_seed(T)
    spec = PartSpec("moe", {"hidden_size": d, "intermediate_size": ff, "n_experts": E, "top": top},
                    {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down"})
    t = {"router": (torch.randn(E, d, generator=g) * 0.4).bfloat16()}
    for e in range(E):
        t[f"e{e}.gate"] = (torch.randn(ff, d, generator=g) * 0.3).bfloat16()
        t[f"e{e}.up"] = (torch.randn(ff, d, generator=g) * 0.3).bfloat16()
        t[f"e{e}.down"] = (torch.randn(d, ff, generator=g) * 0.3).bfloat16()
    rt = Runtime(dtype=dtype, device="cuda:0")
    part = FEED_FORWARDS.get("moe")(spec, t, rt)
    x = torch.randn(T, d, generator=g).bfloat16()
    want = P.moe_ff(x.double(), {"router": {"experts": E, "top": top}}, t, "")
    out = torch.full((T, d), 7.0, device="cuda")
    part.forward(x.cuda().to(rt.act_dtype), None, out, accumulate=False)
    assert rel_err(out.cpu().numpy(), want.numpy()) < (2e-5 if dtype == "float32" else 2e-2)
    base = torch.ones(T, d, device="cuda")
    part.forward(x.cuda().to(rt.act_dtype), None, base, accumulate=True)
    assert torch.allclose(base - 1.0, out, atol=1e-5 * float(out.abs().max()))


def _paged_case(nh, nkv, hd, hdv, lens, new, dtype, seed, scale, cap, window):
    """Random q, k, v of sequences with the given lengths laid into scrambled pages; the last ``new[b]`` positions
    of each are the step's queries.  Keys and values get page pools of their own sizes."""
    from test_kernels_gpu import DEV, Paged
    g = torch.Generator().manual_seed(seed)
    qs = [torch.randn(l, nh, hd, generator=g).to(dtype) for l in lens]
    ks = [torch.randn(l, nkv, hd, generator=g).to(dtype) for l in lens]
    vs = [torch.randn(l, nkv, hdv, generator=g).to(dtype) for l in lens]
    pk, pv = Paged(lens, nkv, hd, dtype, seed), Paged(lens, nkv, hdv, dtype, seed)       # same seed: same block table
    pk.fill(ks, ks)
    pv.fill(vs, vs)
    ref = torch.cat([P.attention_core(q.double(), k.double(), v.double(), scale, cap, window)[l - n:]
                     for q, k, v, l, n in zip(qs, ks, vs, lens, new)]).reshape(sum(new), nh * hdv)
    q = torch.cat([q[l - n:] for q, l, n in zip(qs, lens, new)]).reshape(sum(new), nh * hd).to(DEV)
    seq = torch.from_numpy(np.repeat(np.arange(len(lens)), new).astype(np.int32)).to(DEV)
    pos = torch.from_numpy(np.concatenate([np.arange(l - n, l) for l, n in zip(lens, new)]).astype(np.int32)).to(DEV)
    cu = torch.from_numpy(np.concatenate([[0], np.cumsum(new)]).astype(np.int32)).to(DEV)
    return dict(q=q, k=pk.dev()[0], v=pv.dev()[0], tab=pk.dev()[2], ref=ref, seq=seq, pos=pos, cu=cu,
                lens=torch.tensor(lens, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,hdv,cap,window", [(4, 2, 16, 24, 3.0, 9), (3, 3, 32, 8, 0.0, 70), (6, 1, 48, 48, 1.5, 0),
                                                      (2, 1, 8, 130, 20.0, 64)])
def test_attention_with_capped_scores_and_its_own_value_size(dtype, nh, nkv, hd, hdv, cap, window):
    from ithaca_b200.csrc import ops
    lens, new = [1, 70, 200, 129], [1, 70, 3, 1]
    c = _paged_case(nh, nkv, hd, hdv, lens, new, dtype, 40, 0.7, cap or None, window or None)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ops.attention_simt(c["q"], c["k"], c["v"], c["seq"], c["pos"], c["tab"], nh, 0.7, window, status, softcap=cap)
    assert status.item() == 0 and got.shape == (sum(new), nh * hdv)
    assert rel_err(got.float().cpu().numpy(), c["ref"].numpy()) < (3e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("nh,nkv,hd,kind", [(4, 4, 16, "mma"), (6, 2, 32, "mma"), (8, 2, 64, "tc"), (8, 4, 128, "tc"), (6, 2, 128, "mma")])
@pytest.mark.parametrize("cap,window", [(2.0, 0), (40.0, 70), (0.5, 40)])
def test_tensor_core_attention_with_capped_scores(nh, nkv, hd, kind, cap, window):
    """Prefill (both kernels) and decode.  The scale makes raw scores of several units, so a cap of 0.5 or 2 bends most
    of them and a missing cap would show."""
    from ithaca_b200.csrc import attention_bf16 as A
    scale = 3.0 / hd ** 0.5
    lens, new = [1, 70, 200, 129, 64, 700], [1, 70, 67, 129, 5, 450]
    c = _paged_case(nh, nkv, hd, hd, lens, new, torch.bfloat16, 41, scale, cap, window or None)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = A.prefill(c["q"], c["k"], c["v"], c["cu"], c["lens"], c["tab"], len(lens), max(new), nh, scale, window, status,
                    kind=kind, softcap=cap)
    assert status.item() == 0
    assert rel_err(got.float().cpu().numpy(), c["ref"].numpy()) < 8e-3
    lens = [1, 70, 200, 129, 64, 700]
    d = _paged_case(nh, nkv, hd, hd, lens, [1] * len(lens), torch.bfloat16, 42, scale, cap, window or None)
    for chunk in (1, 4):
        got = A.decode(d["q"], d["k"], d["v"], d["lens"], d["tab"], len(lens), max(lens), nh, scale, window, status,
                       chunk_pages=chunk, softcap=cap)
        assert status.item() == 0
        assert rel_err(got.float().cpu().numpy(), d["ref"].numpy()) < 8e-3
    # the test has teeth: without the cap the result is another one
    if cap <= 2.0:
        free = A.decode(d["q"], d["k"], d["v"], d["lens"], d["tab"], len(lens), max(lens), nh, scale, window, status)
        assert rel_err(free.float().cpu().numpy(), d["ref"].numpy()) > 5e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,rot,pairing,hd,hdv", [(3, 8, 1, 16, 24), (4, 16, 0, 16, 16), (1, 0, 1, 8, 8), (2, 32, 1, 32, 8), (0, 8, 1, 16, 24),
                                                      (3, 6, 1, 10, 6), (4, 12, 1, 12, 12), (2, 0, 0, 20, 36)])
def test_convolution_rotation_append_kernel(dtype, taps, rot, pairing, hd, hdv):
    """Three sequences fed in two steps (the second reads the first's last values from the ring, for one sequence a
    single new token, for one more tokens than taps) against the plain convolution and rotation of the whole sequences."""
    from test_kernels_gpu import DEV, Paged
    from ithaca_b200.csrc import ops
    nh, nkv = 4, 2
    ctot = (nh + nkv) * hd + nkv * hdv
    total, first = [70, 9, 131], [67, 8, 60]
    g = torch.Generator().manual_seed(taps * 7 + rot)
    u = [torch.randn(l, ctot, generator=g) for l in total]
    w = torch.randn(ctot, max(taps, 1), generator=g)
    freqs = P.rotary_frequencies(rot, 100.0, None) if rot else None
    pk, pv = Paged(total, nkv, hd, dtype, 3), Paged(total, nkv, hdv, dtype, 3)
    k_d, v_d, tab = pk.dev()[0], pv.dev()[0], pk.dev()[2]
    slots = torch.tensor([2, 0, 5], dtype=torch.int32, device=DEV)
    ring = torch.full((6, taps, ctot), 9.0, device=DEV) if taps > 1 else None          # what an earlier user left there
    inv = torch.tensor(freqs.numpy(), dtype=torch.float32, device=DEV) if rot else None
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    q_got = [[] for _ in total]
    for lo, hi in ([0] * 3, first), (first, total):
        new = [h - l for l, h in zip(lo, hi)]
        qkv = torch.cat([x[l:h] for x, l, h in zip(u, lo, hi)]).to(DEV)
        seq = torch.from_numpy(np.repeat(np.arange(3), new).astype(np.int32)).to(DEV)
        pos = torch.from_numpy(np.concatenate([np.arange(l, h) for l, h in zip(lo, hi)]).astype(np.int32)).to(DEV)
        cu = torch.from_numpy(np.concatenate([[0], np.cumsum(new)]).astype(np.int32)).to(DEV)
        q_out = torch.empty(sum(new), nh * hd, dtype=dtype, device=DEV)
        ops.conv_rope_append(qkv, w.t().contiguous().to(DEV) if taps else None, ring, slots, cu, torch.tensor(hi, dtype=torch.int32, device=DEV),
                             q_out, k_d, v_d, seq, pos, tab, inv, nh, nkv, rot, pairing, True, status)
        for b, part in enumerate(torch.split(q_out.float().cpu(), new)):
            q_got[b].append(part)
    assert status.item() == 0
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    for b, l in enumerate(total):
        y = P.short_conv(u[b].double(), w.double()) if taps else u[b].double()
        q = y[:, :nh * hd].reshape(l, nh, hd)
        k = y[:, nh * hd:(nh + nkv) * hd].reshape(l, nkv, hd)
        v = y[:, (nh + nkv) * hd:].reshape(l, nkv, hdv)
        if rot:
            if pairing == 0:                                   # pairs (i, i + rot/2): bring them side by side, turn, and back
                order = torch.stack((torch.arange(rot // 2), torch.arange(rot // 2) + rot // 2), 1).reshape(-1)
                back = torch.argsort(order)
                turn = lambda x: torch.cat((P.rotate_pairs(x[..., order], range(l), freqs)[..., back], x[..., rot:]), -1)
                q, k = turn(q), turn(k)
            else:
                q, k = P.rotate_pairs(q, range(l), freqs), P.rotate_pairs(k, range(l), freqs)
        assert rel_err(torch.cat(q_got[b]).numpy(), q.reshape(l, -1).numpy()) < tol
        kk = torch.stack([k_d.cpu()[pk.table[b, j // 64], :, j % 64] for j in range(l)]).float()
        vv = torch.stack([v_d.cpu()[pk.table[b, j // 64], :, j % 64] for j in range(l)]).float()
        assert rel_err(kk.numpy(), k.numpy()) < tol and rel_err(vv.numpy(), v.numpy()) < tol


@pytest.mark.parametrize("T,E,top,ff,d", [(5, 12, 2, 88, 192), (700, 4, 2, 200, 128), (2500, 2, 1, 64, 64), (200, 64, 1, 48, 64),
                                          (64, 8, 8, 72, 200)])
def test_mixture_of_experts_on_the_grouped_tensor_core_product(monkeypatch, T, E, top, ff, d):
    """Tile heights of 16, 128 and 256 rows; experts that get no token; widths that are no multiple of the 128-row
    weight tile or the 64-wide K block.  The CUDA-core product must not run."""
    from ithaca_b200.config.spec import PartSpec
    from ithaca_b200.csrc import ops
    from ithaca_b200.parts import FEED_FORWARDS, Runtime
    g = torch.Generator().manual_seed(T + E)
    spec = PartSpec("moe", {"hidden_size": d, "intermediate_size": ff, "n_experts": E, "top": top},
                    {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down"})
    t = {"router": (torch.randn(E, d, generator=g) * 0.4).bfloat16()}
    for e in range(E):
        t[f"e{e}.gate"] = (torch.randn(ff, d, generator=g) * 0.2).bfloat16()
        t[f"e{e}.up"] = (torch.randn(ff, d, generator=g) * 0.2).bfloat16()
        t[f"e{e}.down"] = (torch.randn(d, ff, generator=g) * 0.2).bfloat16()
    rt = Runtime(dtype="bfloat16", device="cuda:0")
    part = FEED_FORWARDS.get("moe")(spec, t, rt)
    assert part.tensor_cores

    def never(*a, **k):
        raise AssertionError("the CUDA-core grouped product ran")
    monkeypatch.setattr(ops, "moe_gemm", never)
    x = torch.randn(T, d, generator=g).bfloat16()
    want = P.moe_ff(x.double(), {"router": {"experts": E, "top": top}}, t, "")
    out = torch.full((T, d), 7.0, device="cuda")
    part.forward(x.cuda(), None, out, accumulate=False)
    assert int(rt.status.item()) == 0
    assert rel_err(out.cpu().numpy(), want.numpy()) < 2e-2


# ------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompt_matches_plain(models, name, dtype):
    from ithaca_b200 import Engine
    ids = random_ids(150, CONFIGS[name]["vocab"], 3)
    want = _plain(models[name], ids)
    eng = Engine(models[name], dtype=dtype, max_tokens=1024)
    s = eng.alloc_slot()
    got = eng.step([s], [ids], "all").cpu().numpy()
    eng.check_status()
    assert _close(got, want, dtype)
    # the first tokens of a sequence alone
    for n in (1, 2, 3):
        s2 = eng.alloc_slot()
        assert _close(eng.step([s2], [ids[:n]], "all").cpu().numpy(), want[:n], dtype)
        eng.free_slot(s2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_schedules_agree_with_plain(models, name, dtype):
    """Token by token; portions of 2, 3, 7, 64 and 65 tokens; a prompt and then decoding across page and window
    edges; unequal requests in one batch and decoded together; every position against the plain whole sequence."""
    from ithaca_b200 import Engine
    V = CONFIGS[name]["vocab"]
    reqs = {"a": random_ids(140, V, 11), "b": random_ids(67, V, 12), "c": random_ids(1, V, 13), "d": random_ids(9, V, 14)}
    want = {r: _plain(models[name], ids) for r, ids in reqs.items()}
    eng = Engine(models[name], dtype=dtype, max_tokens=2048)

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


def test_slots_and_pages_are_used_again(models):
    """A small cache: requests come and go, so slots, pages and convolution rings are handed out again, also to
    shorter sequences whose first tokens must see nothing of what lay there before."""
    from ithaca_b200 import Engine
    V = CFG_A["vocab"]
    eng = Engine(models["A"], dtype="float32", max_tokens=64 * 6, max_slots=2)
    for round_ in range(4):
        reqs = {"x": random_ids(130 - 40 * round_, V, 20 + round_), "y": random_ids(3 + round_, V, 30 + round_)}
        got = run_schedule(eng, reqs, [[("x", len(reqs["x"]) - 2), ("y", 2)], [("x", 1), ("y", 1)], [("x", 1)]]
                           + [[("y", 1)] for _ in range(round_)])
        for r, ids in reqs.items():
            assert rel_err(got[r], _plain(models["A"], ids)) < REL["float32"], (round_, r)
        eng.cache.table.check_consistent()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    from ithaca_b200 import Engine
    ids = random_ids(330, CFG_A["vocab"], 77)
    want = _plain(models["A"], ids)
    eng = Engine(models["A"], dtype=dtype, max_tokens=1024)
    got = run_schedule(eng, {"a": ids}, [[("a", 10)]] + [[("a", 1)] for _ in range(320)])["a"]
    assert _close(got, want, dtype)


# ------------------------------------------------------------------------------------------ one key decides
def _needle_model(tmp, window, conv):
    """One layer whose attention output is, to good approximation, the value of the one earlier 'needle' token
    that the query token matches: needle and query point along axis 0, every other token along an axis of its own,
    and q and k copy axis 0 of the normed input.  If a window or a page edge is one key off, the logits at the query
    change completely."""
    from ithaca_b200.config import config_from_dict
    from ithaca_b200.engine.model import weight_manifest
    from ithaca_b200.weights.random_init import random_tensors
    d = 32
    cfg = {"architecture": "Vebisun", "vocab": 40, "width": d, "embedding": {"scale": 1.0}, "residual_mult": 1.0,
           "norm": {"eps": 1e-6},
           "layers": [{"type": "attention", "mixer": _mixer(1, 1, d, d, conv=conv, window=window, scale=0.05), "mlp": None}]}
    t = random_tensors(weight_manifest(config_from_dict(cfg)[1].model_spec()), 3, "bfloat16")
    g = torch.Generator().manual_seed(1)
    emb = torch.randn(40, d, generator=g) * 0.05
    for i in range(3, 40):
        emb[i, 8 + i % 20] += 4.0
    emb[1] += torch.eye(d)[0] * 4 + torch.eye(d)[5] * 2          # the needle's token
    emb[2] += torch.eye(d)[0] * 4 - torch.eye(d)[5] * 2          # the query's token: matches the needle along axis 0
    t["embed"] = emb.bfloat16()
    t["l0.norm1"], t["l0.norm1.b"] = torch.ones(d).bfloat16(), torch.zeros(d).bfloat16()
    t["l0.mix.q"] = t["l0.mix.k"] = (torch.eye(d)[0][None, :] * torch.eye(d)[0][:, None] * 4).bfloat16()
    t["l0.mix.v"] = torch.eye(d).bfloat16()
    if conv:
        for r in "qkv":                                            # the tap at the token itself is 1, the others small
            w = torch.full((d, conv), 0.05)
            w[:, -1] = 1.0
            t[f"l0.mix.{r}.conv"] = w.bfloat16()
    return _write(tmp, cfg, 3, tensors=t), cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,conv", [(75, 3), (64, None), (None, 2), (130, None)])
def test_the_one_key_that_matters(tmp_path, window, conv, dtype):
    """The needle sits far back, at a page's last and first place, and just inside and just outside the window; the
    query comes at the end of a prompt or is decoded alone after it."""
    from ithaca_b200 import Engine
    d, cfg = _needle_model(tmp_path, window, conv)
    eng = Engine(d, dtype=dtype, max_tokens=4096)
    n = 400
    places = [0, 63, 64, 127, 128, n - 2]
    if window:
        places += [n - 1 - window, n - window, n - window + 1, n - 1 - 64, n - 64]
    hay = [3 + (i * 7) % 37 for i in range(n)]
    for at in sorted(set(p for p in places if 0 <= p < n - 1)):
        ids = list(hay)
        ids[at], ids[n - 1] = 1, 2
        want = _plain(d, ids)[n - 1]
        for cut in (n, n - 1, n - 5):                              # whole prompt; the query decoded alone; a short portion
            s = eng.alloc_slot()
            steps = [ids[:cut]] + [[x] for x in ids[cut:]]
            for st in steps:
                lg = eng.step([s], [st], "last")
            eng.free_slot(s)
            # bfloat16: the attention output here is ONE cached value vector whose two large components carry the
            # rounding of 16 bits (0.4 % of 5) into a layer norm over otherwise small components: up to 3 % of the
            # logits' scale, the same for every cutting; a wrong key moves them by 30 % (checked below)
            assert rel_err(lg.cpu().numpy()[0], want) < (REL[dtype] if dtype == "float32" else 6e-2), (at, cut)
    eng.check_status()
    if window:                                                     # the test has teeth: inside and outside differ widely
        ids_in, ids_out = list(hay), list(hay)
        ids_in[n - window], ids_out[n - 1 - window] = 1, 1
        ids_in[n - 1] = ids_out[n - 1] = 2
        a, b = _plain(d, ids_in)[n - 1], _plain(d, ids_out)[n - 1]
        assert rel_err(a, b) > 0.2


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_engine(models, name, graphs):
    """More prompts than slots, unequal lengths, the generation loop's own batching (and its graph-replayed decode
    steps, which launch a step ahead and may drop it)."""
    from ithaca_b200 import Engine
    V = CONFIGS[name]["vocab"]
    cfg, t = _load(models[name])
    prompts = [random_ids(n, V, 60 + n) for n in (1, 6, 70, 20)]
    eng = Engine(models[name], dtype="float32", max_tokens=64 * 12, max_slots=3, graphs=graphs)
    got = eng.generate(prompts, max_tokens=12, temp=0.0, rep_pen=1.0, stop_token_ids=[])
    for p, g in zip(prompts, got):
        assert len(g) == 12
        lgs = P.forward(list(p) + g[:-1], cfg, t)                  # every generated token is the plain model's greedy pick
        for i, tok in enumerate(g):
            lg = lgs[len(p) - 1 + i]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > 1e-4 * float(lg.abs().max()):
                assert tok == int(lg.argmax()), (len(p), i)
    assert eng.cache.table.n_slots_in_use() == 0


# ------------------------------------------------------------------------------------------ the programs
def test_trace_replay_and_command_line(models, tmp_path):
    """bin/trace_run on a batch of unequal prompts decoded together, against the plain implementation; bin/ithaca
    describes the looped schedule and generates greedily what the engine generates."""
    import subprocess
    import sys
    from helpers import ROOT
    d, V = models["A"], CFG_A["vocab"]
    reqs = {"p": random_ids(70, V, 90), "q": random_ids(3, V, 91), "r": random_ids(130, V, 92)}
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": reqs["p"][:66], "want": [0, 65]}, {"id": "q", "tokens": reqs["q"][:1], "want": []},
                                     {"id": "r", "tokens": reqs["r"][:126], "want": [125]}], "end": []}]
    for i in range(4):
        ent = [{"id": "p", "tokens": [reqs["p"][66 + i]], "want": [0]}, {"id": "r", "tokens": [reqs["r"][126 + i]], "want": [0]}]
        if i < 2:
            ent.insert(1, {"id": "q", "tokens": [reqs["q"][1 + i]], "want": [0] if i == 1 else []})
        steps.append({"step": 1 + i, "entries": ent, "end": (["q"] if i == 1 else []) + (["p", "r"] if i == 3 else [])})
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "210"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                       timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(5)]
    want = {r: _plain(d, ids) for r, ids in reqs.items()}
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, V)
    assert rel_err(got0, np.stack([want["p"][0], want["p"][65], want["r"][125]])) < REL["float32"]
    got2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(3, V)
    assert rel_err(got2, np.stack([want["p"][67], want["q"][2], want["r"][127]])) < REL["float32"]
    got4 = np.fromfile(out / "4.f32", dtype="<f4").reshape(2, V)
    assert rel_err(got4, np.stack([want["p"][69], want["r"][129]])) < REL["float32"]

    cli = [sys.executable, os.path.join(ROOT, "bin", "ithaca"), "--model", d, "--dtype", "float32"]
    p = subprocess.run(cli + ["--describe"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and p.stdout.count("sandwich") == 7 and p.stdout.count("input added first") == 2, p.stderr[-2000:]
    prompt = random_ids(11, V, 93)
    p = subprocess.run(cli + ["--prompt", ",".join(map(str, prompt)), "-n", "5", "--rep-pen", "1.0", "--stop-ids", ""],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    from ithaca_b200 import Engine
    eng = Engine(d, dtype="float32", max_tokens=512)
    assert [int(x) for x in p.stdout.strip().split(",")] == eng.generate([prompt], max_tokens=5, temp=0.0, rep_pen=1.0, stop_token_ids=[])[0]
