"""Vebisun without a device: the configuration reader, the description built from it, the tensors it asks
for, a random model folder read back, and the plain implementation's parts against closed forms."""
import copy
import math

import pytest
import torch

from plain import vebisun_plain as P
from test_vebisun_gpu import CFG_A, CFG_B, _load, _write


def test_layers_sizes_and_schedule_come_from_the_file():
    from ithaca_b200.config import config_from_dict, describe, validate_schedule
    from ithaca_b200.engine.model import weight_manifest
    arch, cfg = config_from_dict(CFG_A)
    spec = cfg.model_spec()
    validate_schedule(spec)
    m = weight_manifest(spec)
    assert tuple(m["l0.mix.v"].shape) == (2 * 24, 64) and tuple(m["l0.mix.o"].shape) == (64, 4 * 24)
    assert tuple(m["l0.mix.q.conv"].shape) == (64, 3) and "l2.mix.q.conv" not in m
    assert tuple(m["l2.mlp.router"].shape) == (4, 64) and tuple(m["l0.mlp.e7.down"].shape) == (64, 40)
    assert not any(n.startswith("l1.mlp") or n.startswith("l1.norm2") for n in m)
    assert {"embed", "head", "final.norm", "final.norm.b", "l1.norm1b.b"} <= set(m)
    assert len(describe(spec)) == 7 and "input added first" in describe(spec)[3]
    att = spec.layers[0].mixer
    assert att["window"] == 9 and att["softcap"] == 3.0 and att["scale"] == 8.0 and att["conv_taps"] == 3
    assert spec.layers[0].position["pairing"] == "interleaved" and spec.layers[2].position is None
    assert spec.layers[0].feed_forward["n_groups"] == 4 and spec.layers[0].feed_forward["group_keep"] == 2
    # the same file without a loop: every layer once
    plain = copy.deepcopy(CFG_A)
    del plain["loop"]
    assert [e.layer for e in config_from_dict(plain)[1].model_spec().schedule] == [0, 1, 2]
    assert config_from_dict(cfg.to_dict())[1].model_spec() == spec


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].__setitem__("type", "recurrent"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 3), "groups"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][2]["mlp"].__setitem__("kind", "dense"), "kind"),
])
def test_config_errors_name_the_key(change, word):
    from ithaca_b200.config import ConfigError, config_from_dict
    c = copy.deepcopy(CFG_A)
    change(c)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(c)


def test_random_model_folder_round_trip(tmp_path):
    from ithaca_b200.config import config_from_model_dir
    from ithaca_b200.engine.model import weight_manifest
    from ithaca_b200.weights.loader import load_checkpoint
    d = _write(tmp_path, CFG_B, 9)
    arch, cfg = config_from_model_dir(d)
    t = load_checkpoint(d, weight_manifest(cfg.model_spec()))
    assert t["l1.mix.v"].shape == (48, 48) and t["l0.mix.q.conv"].shape == (48, 4) and t["embed"].dtype == torch.bfloat16
    logits = P.forward([1, 2, 3, 4], *_load(d))
    assert logits.shape == (4, 61) and bool(torch.isfinite(logits).all())


def test_plain_short_convolution_is_causal_and_matches_conv1d():
    g = torch.Generator().manual_seed(0)
    u, w = torch.randn(12, 5, generator=g, dtype=torch.float64), torch.randn(5, 3, generator=g, dtype=torch.float64)
    y = P.short_conv(u, w)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (2, 0)), w[:, None, :], groups=5)[0].T
    assert torch.allclose(y, ref, atol=1e-12)
    u2 = u.clone()
    u2[7:] += 1.0
    assert torch.equal(P.short_conv(u2, w)[:7], y[:7])
    assert torch.allclose(y[0], w[:, 2] * u[0])


def test_plain_rotation_keeps_lengths_and_relative_angles():
    f = P.rotary_frequencies(8, 1000.0, {"factor": 4.0, "high": 4.0, "low": 1.0, "original": 64})
    raw = P.rotary_frequencies(8, 1000.0, None)
    # wavelengths 6.3, 35.3, 199, 1117 against 64/4 and 64/1: kept, blended, slowed, slowed
    assert float(f[0]) == float(raw[0]) == 1.0 and math.isclose(float(f[3]), float(raw[3]) / 4.0)
    mix = (64.0 * float(raw[1]) / (2 * math.pi) - 1.0) / 3.0
    assert 0 < mix < 1 and math.isclose(float(f[1]), (1 - mix) * float(raw[1]) / 4.0 + mix * float(raw[1]))
    g = torch.Generator().manual_seed(1)
    x = torch.randn(6, 2, 12, generator=g, dtype=torch.float64)
    a = P.rotate_pairs(x, range(6), f)
    assert torch.allclose(a.norm(dim=-1), x.norm(dim=-1)) and torch.equal(a[..., 8:], x[..., 8:])
    b = P.rotate_pairs(x, range(10, 16), f)
    assert torch.allclose(a[2, 0] @ a[5, 1], b[2, 0] @ b[5, 1])        # depends on the distance only


def test_plain_router_weights_are_scores_of_all_experts():
    z = torch.tensor([[1.0, 2.0, 3.0, 0.0]], dtype=torch.float64)
    e, w = P.route(z, {"experts": 4, "top": 2}, torch.eye(4, dtype=torch.float64))
    s = torch.softmax(z, -1)
    assert e.tolist() == [[2, 1]] and torch.allclose(w, s[:, [2, 1]]) and float(w.sum()) < 1.0
