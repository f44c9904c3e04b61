"""Tiralix without a device: the configuration reader, the description built from it, the tensors it asks for,
what its mixers keep in the cache, and the plain implementation's parts against closed forms."""
import copy
import math

import pytest
import torch

from plain import tiralix_plain as P
from test_tiralix_gpu import CFG_A, CFG_B, make_tensors


def test_layers_sizes_and_constants_come_from_the_file():
    from ithaca_b200.config import config_from_dict, describe, validate_schedule
    from ithaca_b200.engine.model import weight_manifest
    arch, cfg = config_from_dict(CFG_A)
    spec = cfg.model_spec()
    validate_schedule(spec)
    assert arch.name == "Tiralix" and spec.vocab_size == 101 and spec.hidden_size == 64
    m = weight_manifest(spec)
    assert tuple(m["l0.mix.left.q"].shape) == (6 * 16, 64) and tuple(m["l0.mix.left.v"].shape) == (2 * 8, 64)
    assert tuple(m["l0.mix.left.o"].shape) == (64, 6 * 8) and tuple(m["l0.mix.left.g"].shape) == (6, 64)
    assert tuple(m["l0.mix.left.q.norm"].shape) == (96,) and tuple(m["l0.mix.left.k.norm"].shape) == (32,)
    assert tuple(m["l0.mix.right.k"].shape) == (2 * 24, 64) and tuple(m["l0.mix.right.g"].shape) == (2 * 40, 64)
    assert tuple(m["l0.mix.right.norm"].shape) == (80,) and tuple(m["l0.mix.right.o"].shape) == (64, 80)
    assert tuple(m["l1.mix.in"].shape) == (192, 64) and tuple(m["l1.mix.x"].shape) == (3 + 2 * 5, 96)
    assert tuple(m["l1.mix.dt"].shape) == (96, 3) and tuple(m["l1.mix.conv"].shape) == (96, 3) and tuple(m["l3.mix.conv"].shape) == (80, 1)
    assert tuple(m["l1.mix.A_log"].shape) == (96, 5) and tuple(m["l0.mlp.down"].shape) == (64, 88)
    assert not any(n.startswith("l1.mlp") or n.startswith("l1.norm2") or n.startswith("l1.ls2") for n in m)
    assert {"embed", "final.norm", "l1.ls1", "l3.ls2", "l3.mix.dt.b", "l3.mix.conv.b", "l3.mix.D"} <= set(m) and "head" not in m
    assert [b.mixer.kind for b in spec.layers] == ["parallel", "mamba1", "parallel", "mamba1"]
    assert all(b.kind == "outnorm" for b in spec.layers) and len(describe(spec)) == 4
    left, right = spec.layers[0].mixer["branches"]
    assert spec.layers[0].mixer["scales"] == [1.3, 0.7] and left["scale"] == 0.3 and right["decay"] == [1.0, 0.9]
    assert left["position"]["pairing"] == "half" and left["position"]["rotary_dim"] == 8
    assert left["position"]["scaling"]["rope_type"] == "yarn" and spec.layers[2].mixer["branches"][0]["position"]["scaling"] is None
    ff = spec.layers[2].feed_forward
    assert ff["limit"] == 0.5 and ff["alpha"] == 1.702 and ff["up_shift"] == 1.0 and spec.layers[1].feed_forward is None
    assert spec.head["scale"] == 0.5 and spec.head["softcap"] == 8.0 and spec.head.weights["weight"] == spec.embedding.weights["weight"]
    assert config_from_dict(cfg.to_dict())[1].model_spec() == spec
    assert config_from_dict(CFG_B)[1].model_spec().layers[1].mixer["branches"][0]["position"] is None


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].__setitem__("type", "attention"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 4), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][1]["mixer"].pop("dt_rank"), "dt_rank"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "mlp.kind"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_a_wrong_file_is_refused_with_the_key_named(change, word):
    from ithaca_b200.config import ConfigError, config_from_dict
    bad = copy.deepcopy(CFG_A)
    change(bad)
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    assert word in str(e.value)


def test_what_the_mixers_keep_per_sequence():
    """Keys and values for the softmax branch; for the recurrences a float state kept twice (by position parity) and the
    convolution's ring where there is more than one tap.  Equal shapes share a group."""
    from ithaca_b200.cache.cache import KVRequest, StateRequest, SequenceCache
    from ithaca_b200.config import config_from_dict
    from ithaca_b200.parts import MIXERS, Runtime
    spec = config_from_dict(CFG_A)[1].model_spec()
    t = make_tensors(CFG_A, 1)
    rt = Runtime(dtype="float32", device="cpu")
    reqs = {i: MIXERS.get(b.mixer.kind)(b.mixer, t, rt).cache_requests() for i, b in enumerate(spec.layers)}
    assert reqs[0] == [KVRequest(2, 16, None, 8), StateRequest("decay_state", (2, 2, 24, 40), "float32")]
    assert reqs[1] == [StateRequest("scan_state", (2, 96, 5), "float32"), StateRequest("scan_conv_ring", (3, 96), "float32")]
    assert reqs[2] == [KVRequest(2, 32, None, None), StateRequest("decay_state", (2, 3, 40, 16), "float32")]
    assert reqs[3] == [StateRequest("scan_state", (2, 80, 20), "float32")]                 # one tap: no ring
    cache = SequenceCache(reqs, max_tokens=256, max_slots=3, device=None)
    assert len(cache.kv_groups) == 2 and len(cache.state_groups) == 5
    s = cache.alloc_slot()
    cache.reserve([s], [70])
    cache.commit([s], [70])
    with pytest.raises(Exception):
        cache.truncate(s, 10)                                            # a fixed-size state cannot be rolled back
    cache.truncate(s, 0)


def test_plain_parts_against_closed_forms():
    # a decay of one and constant inputs: the state grows linearly, o_t = (t + 1) * (k . q) * v
    m = {"heads": 1, "dim": 2, "vdim": 3, "decay": [1.0]}
    eye = lambda r, c: torch.eye(max(r, c))[:r, :c].double()
    W = {"q": eye(2, 4), "k": eye(2, 4), "v": eye(3, 4), "g": torch.zeros(3, 4).double(), "o": torch.eye(3).double(), "norm": torch.ones(3).double()}
    x = torch.tensor([[1.0, 2.0, 0.5, 0.0]] * 4, dtype=torch.float64)
    out = P.decayed_linear_attention(x, m, W, "", 0.0)
    s = P.silu(x[0])
    want = P.rms_norm((s[:2] @ s[:2]) * s[:3], None, 0.0) * 0.5           # the norm removes the factor t + 1
    assert torch.allclose(out, want.expand(4, 3))
    # convolution: the last column meets the current token, zeros stand before the start
    u = torch.arange(1.0, 5.0, dtype=torch.float64)[:, None]
    y = P.causal_conv(u, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64), torch.tensor([0.5], dtype=torch.float64))
    assert y[:, 0].tolist() == [1.5, 12.5, 123.5, 234.5]
    # the feed-forward's gate: limits, the constant 1.702 and the shift by one
    W = {"gate": torch.tensor([[1.0]]), "up": torch.tensor([[1.0]]), "down": torch.tensor([[1.0]])}
    f = lambda v: float(P.clamped_gated_ff(torch.tensor([[v]], dtype=torch.float64), {"limit": 2.0}, W, "")[0, 0])
    assert abs(f(5.0) - 2.0 / (1 + math.exp(-3.404)) * 3.0) < 1e-12 and abs(f(-5.0) - (-5.0 / (1 + math.exp(8.51))) * -1.0) < 1e-12
    # rotation: frequencies without scaling are base^(-2i/r); a pair turns by p * f and grows by the magnitude
    f, mag = P.rotary_frequencies(4, 100.0, None)
    assert mag == 1.0 and abs(f[1] - 0.1) < 1e-15
    x = torch.tensor([[[1.0, 0.0, 0.0, 1.0, 7.0]]], dtype=torch.float64).expand(3, 1, 5)
    r = P.rotate(x, [0, 1, 2], 4, f, 2.0)
    assert torch.allclose(r[2, 0], torch.tensor([2 * math.cos(2.0), -2 * math.sin(0.2), 2 * math.sin(2.0), 2 * math.cos(0.2), 7.0], dtype=torch.float64))
