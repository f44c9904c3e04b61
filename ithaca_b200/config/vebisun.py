"""Typed configuration of the Vebisun decoder, read from ``config.json``.

A Vebisun model lists its layers one by one; every size and constant that can differ between two
models of the design is in the file.  The keys:

* ``vocab``, ``width``, ``embedding.scale``, ``residual_mult``, ``norm.eps``;
* ``layers``: per layer ``type`` (the mixer, ``attention``), ``mixer`` (its sizes) and ``mlp`` (the
  feed-forward, or null for none);
* ``loop``: layers ``start`` .. ``stop`` - 1 run ``times`` times in a row with the same weights, each pass
  with a cache of its own; before every pass after the first the embedding's output joins the stream.

A layer is norm, sublayer, norm, scaled add, for the mixer and then for the feed-forward, with layer
norms (weight and bias).  The attention mixer has grouped heads with key size ``dim`` and value size
``vdim``, a short causal convolution of ``conv`` taps on q, k and v, rotation of the first ``rot.dims``
dimensions in neighbouring pairs with wavelength-dependent frequency scaling, a constant score
``scale``, a ``softcap`` on the scores and a sliding window of ``mask.size`` keys.  The feed-forward is
a mixture of ``router.experts`` gated feed-forwards of width ``expert.ff``, ``router.top`` per token,
chosen among the ``router.groups.keep`` best of ``router.groups.count`` groups of neighbours.

Tensor names: ``embed``, ``head``, ``final.norm`` (+ ``.b``), and per layer i ``l<i>.norm1``, ``norm1b``,
``norm2``, ``norm2b`` (+ ``.b``), ``l<i>.mix.{q,k,v,o}``, ``l<i>.mix.{q,k,v}.conv``, ``l<i>.mlp.router``,
``l<i>.mlp.e<n>.{gate,up,down}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, need_float, need_int
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

# no key of the file bounds a sequence's length; this sizes nothing, it only stops a runaway caller
MAX_POSITION = 1 << 20


def _obj(d: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = d.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object, found {v!r}")
    return v


@dataclass(frozen=True)
class VebisunConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding_scale: float
    residual_mult: float
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]        # as validated from the file
    loop_start: int
    loop_stop: int
    loop_times: int
    raw: Dict[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Vebisun"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VebisunConfig":
        width = need_int(d, "width")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, l in enumerate(layers):
            where = f"layers[{i}]."
            if not isinstance(l, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            if l.get("type") != "attention":
                raise ConfigError(f"config.json: {where}type {l.get('type')!r} is not supported (attention)")
            m = _obj(l, "mixer", where)
            heads, kv = need_int(m, "heads"), need_int(m, "kv_heads")
            if heads % kv:
                raise ConfigError(f"config.json: {where}mixer: {heads} heads cannot share {kv} kv_heads evenly")
            need_int(m, "dim"), need_int(m, "vdim"), need_float(m, "scale")
            if m.get("conv") is not None:
                need_int(m, "conv")
            if m.get("softcap") is not None and need_float(m, "softcap") <= 0:
                raise ConfigError(f"config.json: {where}mixer.softcap must be > 0")
            mask = _obj(m, "mask", where + "mixer.", optional=True)
            if mask is not None:
                need_int(mask, "size")
            rot = _obj(m, "rot", where + "mixer.", optional=True)
            if rot is not None:
                dims = need_int(rot, "dims")
                if dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"config.json: {where}mixer.rot.dims must be even and at most dim, found {dims}")
                if need_float(rot, "base") <= 0:
                    raise ConfigError(f"config.json: {where}mixer.rot.base must be > 0")
                sc = _obj(rot, "scaling", where + "mixer.rot.", optional=True)
                if sc is not None:
                    f, lo, hi = need_float(sc, "factor"), need_float(sc, "low"), need_float(sc, "high")
                    need_int(sc, "original")
                    if f <= 0 or hi <= lo:
                        raise ConfigError(f"config.json: {where}mixer.rot.scaling needs factor > 0 and low < high")
            mlp = l.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} "
                                      "is not supported (moe, or null for none)")
                need_int(_obj(mlp, "expert", where + "mlp."), "ff")
                r = _obj(mlp, "router", where + "mlp.")
                E, top = need_int(r, "experts"), need_int(r, "top")
                if top > E:
                    raise ConfigError(f"config.json: {where}mlp.router.top exceeds the number of experts")
                g = _obj(r, "groups", where + "mlp.router.", optional=True)
                if g is not None:
                    n, keep = need_int(g, "count"), need_int(g, "keep")
                    if E % n or keep > n or top > keep * (E // n):
                        raise ConfigError(f"config.json: {where}mlp.router.groups: {E} experts, {n} groups, {keep} kept, "
                                          f"{top} chosen do not fit together")
        loop = _obj(d, "loop", "", optional=True) or {"start": 0, "stop": 0, "times": 1}
        lo, hi = need_int(loop, "start", minimum=0), need_int(loop, "stop", minimum=0)
        times = need_int(loop, "times", minimum=1)
        if not lo <= hi <= len(layers):
            raise ConfigError(f"config.json: loop {lo}..{hi} does not lie within the {len(layers)} layers")
        return cls(
            architecture=cls.ARCHITECTURE,
            vocab_size=need_int(d, "vocab"),
            hidden_size=width,
            embedding_scale=need_float(_obj(d, "embedding", "", optional=True) or {}, "scale", 1.0),
            residual_mult=need_float(d, "residual_mult", 1.0),
            norm_eps=need_float(_obj(d, "norm", ""), "eps"),
            layers=tuple(copy.deepcopy(layers)),
            loop_start=lo, loop_stop=hi, loop_times=times,
            raw=copy.deepcopy(d),
        )

    def to_dict(self) -> Dict[str, Any]:
        return {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "embedding": {"scale": self.embedding_scale}, "residual_mult": self.residual_mult,
            "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers)),
            "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times},
        }

    # -- the architecture-neutral description --------------------------------------------------
    def layer_runs(self) -> List[Tuple[int, bool]]:
        """(layer, joins the embedding's output first) for every run, in order."""
        lo, hi = self.loop_start, self.loop_stop
        runs = [(i, False) for i in range(lo)]
        for r in range(self.loop_times if hi > lo else 0):
            runs += [(i, r > 0 and i == lo) for i in range(lo, hi)]
        return runs + [(i, False) for i in range(hi, len(self.layers))]

    def model_spec(self) -> ModelSpec:
        d = self.hidden_size

        def ln(name: str) -> PartSpec:
            return PartSpec("layernorm", {"size": d, "eps": self.norm_eps}, {"weight": name, "bias": name + ".b"})

        blocks = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}", l["mixer"]
            rot, position = m.get("rot"), None
            if rot is not None:
                sc = rot.get("scaling")
                position = PartSpec("rotary", {
                    "rotary_dim": rot["dims"], "theta": rot["base"], "pairing": "interleaved", "max_position": MAX_POSITION,
                    "scaling": None if sc is None else {
                        "rope_type": "llama3", "factor": sc["factor"], "low_freq_factor": sc["low"],
                        "high_freq_factor": sc["high"], "original_max_position_embeddings": sc["original"]},
                })
            taps = m.get("conv") or 0
            weights = {r: f"{p}.mix.{r}" for r in "qkvo"}
            if taps:
                weights.update({f"{r}_conv": f"{p}.mix.{r}.conv" for r in "qkv"})
            mixer = PartSpec("attention", {
                "hidden_size": d, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_head_dim": m["vdim"], "window": (m.get("mask") or {}).get("size"), "scale": m["scale"],
                "softcap": m.get("softcap"), "conv_taps": taps,
            }, weights)
            ff, norms = None, {"mixer": ln(f"{p}.norm1"), "mixer_out": ln(f"{p}.norm1b")}
            if l.get("mlp") is not None:
                r = l["mlp"]["router"]
                g = r.get("groups") or {}
                ff = PartSpec("moe", {
                    "hidden_size": d, "intermediate_size": l["mlp"]["expert"]["ff"], "n_experts": r["experts"],
                    "top": r["top"], "n_groups": g.get("count", 0), "group_keep": g.get("keep", 0),
                    "renormalize": False, "activation": "silu",
                }, {"router": f"{p}.mlp.router", "gate": f"{p}.mlp.e{{e}}.gate", "up": f"{p}.mlp.e{{e}}.up",
                    "down": f"{p}.mlp.e{{e}}.down"})
                norms.update({"feed_forward": ln(f"{p}.norm2"), "feed_forward_out": ln(f"{p}.norm2b")})
            blocks.append(BlockSpec(kind="sandwich", mixer=mixer, feed_forward=ff, norms=norms, position=position,
                                    params={"residual_mult": self.residual_mult}))
        schedule = tuple(ScheduleEntry(layer=i, cache=n, adds_input=add) for n, (i, add) in enumerate(self.layer_runs()))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=d,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": d, "scale": self.embedding_scale},
                               {"weight": "embed"}),
            layers=tuple(blocks), schedule=schedule, final_norm=ln("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": d, "tied": False}, {"weight": "head"}),
            max_position=MAX_POSITION,
        )
