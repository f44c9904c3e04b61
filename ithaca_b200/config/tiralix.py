"""Typed configuration of the Tiralix decoder, read from ``config.json``.

A Tiralix model lists its layers one by one; every size and constant that can differ between two models
of the design is in the file.  The keys:

* ``vocab``, ``width``, ``norm.eps``, ``logit_scale``, ``logit_softcap``;
* ``layers``: per layer ``type`` (the mixer: ``parallel`` or ``mamba1``), ``mixer`` (its sizes and constants)
  and ``mlp`` (``kind: dense`` with ``ff`` and ``limit``, or null for none).

A layer adds each sublayer's result to the stream through an RMS norm and a per-channel scale; the
sublayers read the stream as it is.  The ``parallel`` mixer is the weighted sum (``left_scale``,
``right_scale``) of a softmax attention (``left``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot`` with
``dims``, ``base`` and ``scaling`` = ``factor``, ``original``, ``fast``, ``slow``) whose q and k are normed over their
whole projections and whose heads are gated, and a linear attention with one decay per head (``right``:
``heads``, ``dim``, ``vdim``, ``decay``).  The ``mamba1`` mixer is a selective scan (``inner``, ``state``, ``dt_rank``,
``conv``).  The output matrix is the embedding matrix; logits are scaled and capped.

Tensor names: ``embed``, ``final.norm``, and per layer i ``l<i>.norm1``, ``norm2``, ``ls1``, ``ls2``,
``l<i>.mix.left.{q,k,v,g,o,q.norm,k.norm}``, ``l<i>.mix.right.{q,k,v,g,o,norm}``,
``l<i>.mix.{in,conv,conv.b,x,dt,dt.b,A_log,D,o}``, ``l<i>.mlp.{gate,up,down}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, need_float, need_int
from .spec import BlockSpec, ModelSpec, PartSpec, default_schedule

# no key of the file bounds a sequence's length; this sizes nothing, it only stops a runaway caller
MAX_POSITION = 1 << 20

SWISH_ALPHA = 1.702        # the feed-forward's gate is g * sigmoid(1.702 g)
UP_SHIFT = 1.0             # ... times (u + 1)


def _obj(d: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = d.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object, found {v!r}")
    return v


def _check_left(m: Dict[str, Any], where: str) -> None:
    heads, kv = need_int(m, "heads"), need_int(m, "kv_heads")
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads cannot share {kv} kv_heads evenly")
    dim = need_int(m, "dim")
    need_int(m, "vdim"), need_float(m, "scale")
    rot = _obj(m, "rot", where + ".", optional=True)
    if rot is not None:
        dims = need_int(rot, "dims")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim, found {dims}")
        if need_float(rot, "base") <= 1:
            raise ConfigError(f"config.json: {where}.rot.base must be > 1")
        sc = _obj(rot, "scaling", where + ".rot.", optional=True)
        if sc is not None:
            if need_float(sc, "factor") <= 0 or need_float(sc, "fast") <= 0 or need_float(sc, "slow") <= 0:
                raise ConfigError(f"config.json: {where}.rot.scaling needs positive factor, fast and slow")
            need_int(sc, "original")


def _check_right(m: Dict[str, Any], where: str) -> None:
    heads = need_int(m, "heads")
    need_int(m, "dim"), need_int(m, "vdim")
    decay = m.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(a, (int, float)) and not isinstance(a, bool) for a in decay):
        raise ConfigError(f"config.json: {where}.decay must list one number per head ({heads})")


@dataclass(frozen=True)
class TiralixConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    logit_scale: float
    logit_softcap: float
    layers: Tuple[Dict[str, Any], ...]        # as validated from the file
    raw: Dict[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Tiralix"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TiralixConfig":
        width = need_int(d, "width")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, l in enumerate(layers):
            where = f"layers[{i}]."
            if not isinstance(l, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            m = _obj(l, "mixer", where)
            if l.get("type") == "parallel":
                _check_left(_obj(m, "left", where + "mixer."), where + "mixer.left")
                _check_right(_obj(m, "right", where + "mixer."), where + "mixer.right")
                need_float(m, "left_scale"), need_float(m, "right_scale")
            elif l.get("type") == "mamba1":
                need_int(m, "inner"), need_int(m, "state"), need_int(m, "dt_rank"), need_int(m, "conv")
            else:
                raise ConfigError(f"config.json: {where}type {l.get('type')!r} is not supported (parallel, mamba1)")
            mlp = l.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} "
                                      "is not supported (dense, or null for none)")
                need_int(mlp, "ff")
                if need_float(mlp, "limit") <= 0:
                    raise ConfigError(f"config.json: {where}mlp.limit must be > 0")
        cap = need_float(d, "logit_softcap", 0.0)
        if cap < 0:
            raise ConfigError("config.json: 'logit_softcap' cannot be negative")
        return cls(
            architecture=cls.ARCHITECTURE, vocab_size=need_int(d, "vocab"), hidden_size=width,
            norm_eps=need_float(_obj(d, "norm", ""), "eps"), logit_scale=need_float(d, "logit_scale", 1.0),
            logit_softcap=cap, layers=tuple(copy.deepcopy(layers)), raw=copy.deepcopy(d),
        )

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap,
                "layers": copy.deepcopy(list(self.layers))}

    # -- the architecture-neutral description --------------------------------------------------
    def _parallel(self, p: str, m: Dict[str, Any]) -> PartSpec:
        d, left, right = self.hidden_size, m["left"], m["right"]
        rot, position = left.get("rot"), None
        if rot is not None:
            sc = rot.get("scaling")
            position = PartSpec("rotary", {
                "rotary_dim": rot["dims"], "theta": rot["base"], "pairing": "half", "max_position": MAX_POSITION,
                "scaling": None if sc is None else {
                    "rope_type": "yarn", "factor": sc["factor"], "original_max_position_embeddings": sc["original"],
                    "fast_turns": sc["fast"], "slow_turns": sc["slow"]},
            })
        lw = {r: f"{p}.mix.left.{r}" for r in "qkvgo"}
        lw.update({"q_norm": f"{p}.mix.left.q.norm", "k_norm": f"{p}.mix.left.k.norm"})
        softmax = PartSpec("attention", {
            "hidden_size": d, "n_heads": left["heads"], "n_kv_heads": left["kv_heads"], "head_dim": left["dim"],
            "v_head_dim": left["vdim"], "scale": left["scale"], "qk_norm": "projection", "norm_eps": self.norm_eps,
            "head_gate": True, "position": position,
        }, lw)
        linear = PartSpec("decay_attention", {
            "hidden_size": d, "n_heads": right["heads"], "head_dim": right["dim"], "v_head_dim": right["vdim"],
            "decay": [float(a) for a in right["decay"]], "norm_eps": self.norm_eps, "activation": "silu", "gate": True,
        }, {**{r: f"{p}.mix.right.{r}" for r in "qkvgo"}, "norm": f"{p}.mix.right.norm"})
        return PartSpec("parallel", {"hidden_size": d, "branches": [softmax, linear],
                                     "scales": [float(m["left_scale"]), float(m["right_scale"])]})

    def _mamba(self, p: str, m: Dict[str, Any]) -> PartSpec:
        return PartSpec("mamba1", {"hidden_size": self.hidden_size, "inner": m["inner"], "state": m["state"],
                                   "dt_rank": m["dt_rank"], "conv_taps": m["conv"]},
                        {"in": f"{p}.mix.in", "conv": f"{p}.mix.conv", "conv_bias": f"{p}.mix.conv.b", "x": f"{p}.mix.x",
                         "dt": f"{p}.mix.dt", "dt_bias": f"{p}.mix.dt.b", "A_log": f"{p}.mix.A_log", "D": f"{p}.mix.D",
                         "o": f"{p}.mix.o"})

    def model_spec(self) -> ModelSpec:
        d = self.hidden_size

        def norm(name: str, scale: Optional[str] = None) -> PartSpec:
            w = {"weight": name}
            if scale is not None:
                w["scale"] = scale
            return PartSpec("rmsnorm", {"size": d, "eps": self.norm_eps}, w)

        blocks = []
        for i, l in enumerate(self.layers):
            p = f"l{i}"
            mixer = self._parallel(p, l["mixer"]) if l["type"] == "parallel" else self._mamba(p, l["mixer"])
            ff, norms = None, {"mixer_out": norm(f"{p}.norm1", f"{p}.ls1")}
            if l.get("mlp") is not None:
                ff = PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": l["mlp"]["ff"], "activation": "swish",
                                            "alpha": SWISH_ALPHA, "limit": float(l["mlp"]["limit"]), "up_shift": UP_SHIFT},
                              {"gate": f"{p}.mlp.gate", "up": f"{p}.mlp.up", "down": f"{p}.mlp.down"})
                norms["feed_forward_out"] = norm(f"{p}.norm2", f"{p}.ls2")
            blocks.append(BlockSpec(kind="outnorm", mixer=mixer, feed_forward=ff, norms=norms))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=d,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": d}, {"weight": "embed"}),
            layers=tuple(blocks), schedule=default_schedule(len(blocks)), final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": d, "tied": True,
                                      "scale": self.logit_scale, "softcap": self.logit_softcap}, {"weight": "embed"}),
            max_position=MAX_POSITION,
        )
