"""Govuvik: configuration, layer plan and tensor names.

A decoder whose ``config.json`` lists its layers one by one (``layers``: ``type``, ``mixer`` sizes, ``mlp`` or
null).  What it is put together from:

* the embedding's rows pass an RMS norm (``embed.norm``) before the first layer (``token_embedding`` with ``norm``);
* a layer is a ``sandwich`` block: a norm before and after each sublayer (``norm1`` / ``norm1b`` around the mixer,
  ``norm2`` / ``norm2b`` around the feed-forward), and the mixer's input ``h`` becomes ``h + conv(h)``, a causal
  convolution over time of ``canon.taps`` taps per channel (``canon1``) whose last inputs are per-request state;
* ``type`` ``mlstm``: the matrix memory with exponential gating (part ``mlstm``); ``parallel``: two mixers side by
  side (part ``side_by_side``), each RMS-normed with a weight of its own, averaged: ``left`` is grouped-query
  attention (the engine's ``attention`` mixer) whose projections pass a short convolution over time, with ONE norm
  over all heads of q and of k, a rotation of the first ``rot.dims`` entries of a head (entry i with i + dims/2,
  slow frequencies divided by ``rot.scaling.factor`` with a ramp by wavelength), a number per head on the scores
  (``temp``), the heads' scores mixed by ``talk``, a sliding window of ``mask.size`` and a sink in the softmax's
  divisor; ``right`` is gated linear attention (part ``gla``) with a decay per key channel;
* ``mlp.kind`` ``moe``: experts without a gate, ``W_down relu(W_up h)^2``, the ``top`` largest router logits pick,
  weights = the softmax over the picked logits alone;
* the head's logits are capped, ``logit_softcap * tanh(logits / logit_softcap)``.

Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.canon1``, ``l<i>.mix.*``
(``mlstm``: ``q k v g o norm i i.b f f.b``; ``parallel``: ``left.q|k|v|o``, ``left.q.conv|k.conv|v.conv``,
``left.q.norm|k.norm``, ``left.temp|talk|sink``, ``left.out``, ``right.q|k|v|g|o|norm|a1|a2|a2.b``, ``right.out``),
``l<i>.mlp.router``, ``l<i>.mlp.e<k>.up|down``, ``final.norm``, ``head``.  Every size and every constant that can
differ between models comes from ``config.json`` or from a tensor's shape (the decay's inner size is ``a1``'s rows:
the weight file's header is asked for it when a model folder is loaded; a configuration without a folder gives it
as ``mixer.right.decay_rank``).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Any, Dict, Tuple

from ..config.base import ConfigError, ConfigReader, ModelConfig, register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

ARCHITECTURE = "Govuvik"
MIXER_TYPES = ("mlstm", "parallel")
MLSTM_FLOOR = 1e-6            # added to the divisor of the matrix memory's read-out
DEFAULT_DECAY_RANK = 16


@dataclass(frozen=True)
class GovuvikConfig(ModelConfig):
    width: int
    vocab: int
    norm_eps: float
    canon_taps: int
    logit_softcap: float
    layers_json: str              # ``layers`` as canonical JSON (a frozen dataclass holds no dicts)
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def layers(self):
        return json.loads(self.layers_json)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "GovuvikConfig":
        raw = r.raw
        arch = raw["architectures"][0] if "architectures" in raw else raw["architecture"]
        norm = raw.get("norm")
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError(f"{r.source}: required key 'norm.eps' is missing")
        eps = _number(r.source, "norm.eps", norm["eps"])
        canon = raw.get("canon")
        taps = 0                      # no 'canon': the mixer reads the normed row as it is
        if canon is not None:
            _need_ints(r.source, "canon", canon, ("taps",))
            taps = canon["taps"]
        cap = raw.get("logit_softcap")
        cap = 0.0 if cap is None else _number(r.source, "logit_softcap", cap)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{r.source}: required key 'layers' is missing or is not a list of layers")
        # sizes that only a tensor's shape gives are read from the weight file's header, when there is one
        folder = os.path.dirname(r.source)
        shapes = _tensor_shapes(folder) if folder and r.source.endswith("config.json") else {}
        layers = json.loads(json.dumps(layers))
        for i, layer in enumerate(layers):
            _check_layer(r.source, i, layer)
            if layer["type"] == "parallel":
                right = layer["mixer"]["right"]
                shape = shapes.get(f"l{i}.mix.right.a1")
                if shape is not None:
                    right["decay_rank"] = int(shape[0])
                elif "decay_rank" not in right:
                    right["decay_rank"] = DEFAULT_DECAY_RANK
        return cls(architecture=arch, width=r.integer("width", minimum=1), vocab=r.integer("vocab", minimum=1), norm_eps=eps,
                   canon_taps=taps, logit_softcap=cap, layers_json=json.dumps(layers, sort_keys=True),
                   eos_token_ids=tuple(r.integer_list("eos_token_id", ())))

    def to_json_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                             "norm": {"eps": self.norm_eps}, "layers": self.layers}
        if self.canon_taps:
            d["canon"] = {"taps": self.canon_taps}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


def _tensor_shapes(model_dir: str) -> Dict[str, Tuple[int, ...]]:
    """Names and shapes from the header of ``model.safetensors`` (8 bytes of length, then JSON); {} without a file."""
    path = os.path.join(model_dir, "model.safetensors")
    if not os.path.isfile(path):
        return {}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    return {k: tuple(v["shape"]) for k, v in header.items() if k != "__metadata__"}


def _need_ints(source: str, where: str, d: Any, keys, minimum: int = 1) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{source}: {where} must be an object")
    for k in keys:
        v = d.get(k)
        if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
            raise ConfigError(f"{source}: {where}.{k} must be an integer >= {minimum}, found {v!r}")


def _number(source: str, where: str, v: Any, positive: bool = True) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and v <= 0):
        raise ConfigError(f"{source}: {where} must be a{' positive' if positive else ''} number, found {v!r}")
    return float(v)


def _check_layer(source: str, i: int, layer: Any) -> None:
    where = f"layers[{i}]"
    if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
        raise ConfigError(f"{source}: {where}.type must be one of {', '.join(MIXER_TYPES)}, "
                          f"found {layer.get('type') if isinstance(layer, dict) else layer!r}")
    m = layer.get("mixer")
    if layer["type"] == "mlstm":
        _need_ints(source, f"{where}.mixer", m, ("heads", "dim", "vdim"))
        _number(source, f"{where}.mixer.gate_cap", m.get("gate_cap"))
    else:
        if not isinstance(m, dict):
            raise ConfigError(f"{source}: {where}.mixer must be an object")
        left, right = m.get("left"), m.get("right")
        _need_ints(source, f"{where}.mixer.left", left, ("heads", "kv_heads", "dim", "vdim"))
        if left["heads"] % left["kv_heads"] != 0:
            raise ConfigError(f"{source}: {where}.mixer.left: heads {left['heads']} is not a multiple of kv_heads {left['kv_heads']}")
        _number(source, f"{where}.mixer.left.scale", left.get("scale"))
        if left.get("conv") is not None:
            _need_ints(source, f"{where}.mixer.left", left, ("conv",))
        if left.get("mask") is not None:
            _need_ints(source, f"{where}.mixer.left.mask", left["mask"], ("size",))
        rot = left.get("rot")
        if rot is not None:
            _need_ints(source, f"{where}.mixer.left.rot", rot, ("dims",))
            if rot["dims"] % 2 != 0 or rot["dims"] > left["dim"] or _number(source, f"{where}.mixer.left.rot.base", rot.get("base")) <= 1.0:
                raise ConfigError(f"{source}: {where}.mixer.left.rot: dims must be even and at most dim, base larger than 1")
            sc = rot.get("scaling")
            if sc is not None:
                if not isinstance(sc, dict):
                    raise ConfigError(f"{source}: {where}.mixer.left.rot.scaling must be an object")
                for k in ("factor", "high", "original"):
                    _number(source, f"{where}.mixer.left.rot.scaling.{k}", sc.get(k))
                _number(source, f"{where}.mixer.left.rot.scaling.low", sc.get("low"), positive=False)
        _need_ints(source, f"{where}.mixer.right", right, ("heads", "dim", "vdim"))
        _number(source, f"{where}.mixer.right.tau", right.get("tau"))
        if right.get("decay_rank") is not None:
            _need_ints(source, f"{where}.mixer.right", right, ("decay_rank",))
    ff = layer.get("mlp")
    if ff is None:
        return
    if not isinstance(ff, dict) or ff.get("kind") != "moe":
        raise ConfigError(f"{source}: {where}.mlp.kind must be 'moe' (or mlp null for no feed-forward)")
    _need_ints(source, f"{where}.mlp.expert", ff.get("expert"), ("ff",))
    _need_ints(source, f"{where}.mlp.router", ff.get("router"), ("experts", "top"))
    if ff["router"]["top"] > ff["router"]["experts"]:
        raise ConfigError(f"{source}: {where}.mlp.router.top is larger than .experts")


def _left_spec(h: int, eps: float, m: Dict[str, Any]) -> PartSpec:
    params: Dict[str, Any] = {
        "hidden_size": h, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
        "window": (m.get("mask") or {}).get("size", 0), "scale": float(m["scale"]),
        "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "position": PartSpec("none"),
        "qk_norm": {"q": "q.norm", "k": "k.norm", "eps": eps, "whole": True},
        "head_temp": "temp", "talk": "talk", "sink": "sink"}
    if m.get("conv"):
        params["proj_conv"] = {"taps": m["conv"], "q": "q.conv", "k": "k.conv", "v": "v.conv"}
    rot = m.get("rot")
    if rot is not None:
        sc = rot.get("scaling")
        scaling = dict(sc, kind="wavelength") if sc else None
        params["position"] = PartSpec("rope", {"head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": float(rot["base"]),
                                               "scaling": scaling})
    return PartSpec("attention", params)


def _mixer_spec(h: int, eps: float, kind: str, m: Dict[str, Any]) -> PartSpec:
    if kind == "mlstm":
        return PartSpec("mlstm", {"hidden_size": h, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                  "gate_cap": float(m["gate_cap"]), "floor": MLSTM_FLOOR, "eps": eps})
    r = m["right"]
    right = PartSpec("gla", {"hidden_size": h, "heads": r["heads"], "dim": r["dim"], "vdim": r["vdim"],
                             "decay_rank": r.get("decay_rank", DEFAULT_DECAY_RANK), "tau": float(r["tau"]), "eps": eps})
    return PartSpec("side_by_side", {"hidden_size": h, "eps": eps, "coef": 0.5, "left": _left_spec(h, eps, m["left"]), "right": right,
                                     "left_name": "left", "right_name": "right", "left_out": "left.out", "right_out": "right.out"})


def _feed_forward_spec(h: int, ff: Any):
    if ff is None:
        return None
    return PartSpec("sparse_moe", {
        "hidden_size": h, "num_experts": ff["router"]["experts"], "top_k": ff["router"]["top"],
        "expert_intermediate_size": ff["expert"]["ff"], "activation": "relu2",
        # the softmax over the picked logits alone = the picked probabilities renormalised
        "norm_topk_prob": True, "score": "softmax", "weight_on": "output",
        "names": {"router": "router", "up": "e{e}.up", "down": "e{e}.down"}})


def build_plan(cfg: GovuvikConfig) -> ModelPlan:
    h, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rmsnorm", {"dim": h, "eps": eps, "weight_name": ""})
    block_params = {"hidden_size": h, "mixer_norm_name": "norm1", "mixer_post_norm_name": "norm1b",
                    "feed_forward_norm_name": "norm2", "feed_forward_post_norm_name": "norm2b",
                    "mixer_name": "mix", "feed_forward_name": "mlp"}
    if cfg.canon_taps >= 1:
        block_params["input_conv"] = {"taps": cfg.canon_taps, "name": "canon1"}
    block = PartSpec("sandwich", block_params)
    layers = []
    for i, layer in enumerate(cfg.layers):
        ffn = _feed_forward_spec(h, layer.get("mlp"))
        layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=_mixer_spec(h, eps, layer["type"], layer["mixer"]),
                                feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm if ffn is not None else None))
    plan = ModelPlan(architecture=cfg.architecture, hidden_size=h, vocab_size=cfg.vocab, embedding_name="embed",
                     layers=tuple(layers), schedule=tuple(ScheduleEntry(layer=i) for i in range(len(layers))),
                     final_norm=norm, final_norm_prefix="final.norm", lm_head_name="head", eog_token_ids=cfg.eos_token_ids,
                     max_position=None, embedding=PartSpec("token_embedding", {"norm": {"eps": eps, "weight_name": "embed.norm"}}),
                     head=PartSpec("linear_head", {"softcap": cfg.logit_softcap}))
    plan.validate()
    return plan


register_architecture(ARCHITECTURE, GovuvikConfig, build_plan, replace=True)
