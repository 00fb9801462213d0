"""Dimuvik: configuration, layer plan and tensor names.

A decoder whose ``config.json`` lists its layers one by one (``layers``: ``type``, ``mixer`` sizes, ``mlp`` or
null).  What it is put together from:

* the embedding's rows are multiplied by ``embedding.scale`` (``token_embedding`` with ``scale``);
* a layer is a ``sandwich`` block, a norm before and after each sublayer, and every norm (the final one too) is
  Dynamic Tanh (part ``dyt``): ``tanh(alpha x) w + b`` with the scalar and the bias stored beside the weight as
  ``<name>.alpha`` and ``<name>.b``;
* ``type`` ``attention``: differential attention (part ``differential_attention``): two softmax maps per head over
  the same values, biases on q, k and v, a short causal convolution on every projected channel, no rotation, a
  query temperature that grows with the position, the difference of the maps normed per head; ``kv_from: j`` lets a
  layer attend over layer j's keys and values with its own queries;
* ``type`` ``latent_attention``: attention over a compressed latent (part ``latent_attention``) whose queries pass a
  latent of their own (``q_rank``), with a rotation of the shared key part in interleaved pairs and a sink per head in
  the softmax's divisor; no gate on the heads;
* ``mlp.kind`` ``dense``: ``W_down relu(W_up h)^2`` (part ``dense_relu2``); ``moe``: gated SiLU experts behind a softmax
  router whose choice adds a correction per expert to the scores while the weights are the scores themselves times
  ``router.scale``, not renormalised, plus a shared expert that every token runs (part ``sparse_moe``).

Tensor names: ``embed``, ``l<i>.norm1|norm1b|norm2|norm2b`` (each with ``.alpha`` and ``.b``), ``l<i>.mix.*``
(``attention``: ``q k v`` with ``.b`` and ``.conv``, ``lq1 lk1 lq2 lk2``, ``o``; ``latent_attention``: ``dq dq.norm uq
dkv dkv.norm uk uv sink o``), ``l<i>.mlp.up|down`` or ``l<i>.mlp.router|correction``, ``l<i>.mlp.e<k>.gate|up|down``,
``l<i>.mlp.shared.gate|up|down``, ``final.norm``, ``head``.  Every size and every constant that can differ between
models comes from ``config.json``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, Tuple

from ..config.base import ConfigError, ConfigReader, ModelConfig, register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

ARCHITECTURE = "Dimuvik"
MIXER_TYPES = ("attention", "latent_attention")


@dataclass(frozen=True)
class DimuvikConfig(ModelConfig):
    width: int
    vocab: int
    norm_eps: float
    embedding_scale: float
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
    def from_reader(cls, r: ConfigReader) -> "DimuvikConfig":
        raw = r.raw
        arch = raw["architectures"][0] if "architectures" in raw else raw["architecture"]
        norm = raw.get("norm")
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError(f"{r.source}: required key 'norm.eps' is missing")
        eps = _number(r.source, "norm.eps", norm["eps"])
        emb = raw.get("embedding")
        scale = 1.0
        if emb is not None:
            if not isinstance(emb, dict):
                raise ConfigError(f"{r.source}: embedding must be an object")
            if emb.get("scale") is not None:
                scale = _number(r.source, "embedding.scale", emb["scale"])
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{r.source}: required key 'layers' is missing or is not a list of layers")
        for i, layer in enumerate(layers):
            _check_layer(r.source, i, layer, layers)
        return cls(architecture=arch, width=r.integer("width", minimum=1), vocab=r.integer("vocab", minimum=1), norm_eps=eps,
                   embedding_scale=scale, layers_json=json.dumps(layers, sort_keys=True),
                   eos_token_ids=tuple(r.integer_list("eos_token_id", ())))

    def to_json_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "layers": self.layers}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


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


def _check_source(source: str, where: str, i: int, m: Dict[str, Any], layers, same) -> None:
    """``kv_from`` names an earlier layer of the same type that owns its cache and whose cached sizes equal this layer's."""
    src = m.get("kv_from")
    if src is None:
        return
    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
        raise ConfigError(f"{source}: {where}.mixer.kv_from must name an earlier layer, found {src!r}")
    other = layers[src]
    om = other.get("mixer") if isinstance(other, dict) else None
    if not isinstance(om, dict) or other.get("type") != layers[i]["type"] or om.get("kv_from") is not None:
        raise ConfigError(f"{source}: {where}.mixer.kv_from names layer {src}, which owns no cache of this kind")
    for k in same:
        if om.get(k) != m.get(k):
            raise ConfigError(f"{source}: {where}.mixer.{k} must equal that of layer {src}, whose cache it reads")


def _check_layer(source: str, i: int, layer: Any, layers) -> None:
    where = f"layers[{i}]"
    if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
        raise ConfigError(f"{source}: {where}.type must be one of {', '.join(MIXER_TYPES)}, "
                          f"found {layer.get('type') if isinstance(layer, dict) else layer!r}")
    m = layer.get("mixer")
    if layer["type"] == "attention":
        _need_ints(source, f"{where}.mixer", m, ("heads", "kv_heads", "dim", "vdim"))
        if m["heads"] % m["kv_heads"] != 0:
            raise ConfigError(f"{source}: {where}.mixer: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
        _number(source, f"{where}.mixer.scale", m.get("scale"))
        _number(source, f"{where}.mixer.diff", m.get("diff"), positive=False)
        if m.get("conv") is not None:
            _need_ints(source, f"{where}.mixer", m, ("conv",))
        qt = m.get("q_temp")
        if qt is not None:
            _need_ints(source, f"{where}.mixer.q_temp", qt, ("every",))
            _number(source, f"{where}.mixer.q_temp.coef", qt.get("coef"), positive=False)
        _check_source(source, where, i, m, layers, ("kv_heads", "dim", "vdim", "conv"))
    else:
        _need_ints(source, f"{where}.mixer", m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"))
        rot = m.get("rot")
        if not isinstance(rot, dict):
            raise ConfigError(f"{source}: {where}.mixer.rot must give 'base' and 'dims'")
        _need_ints(source, f"{where}.mixer.rot", rot, ("dims",))
        _number(source, f"{where}.mixer.rot.base", rot.get("base"))
        if rot["dims"] % 2 != 0 or rot["dims"] > m["rot_dim"]:
            raise ConfigError(f"{source}: {where}.mixer.rot.dims must be even and at most rot_dim")
        _number(source, f"{where}.mixer.scale", m.get("scale"))
        _check_source(source, where, i, m, layers, ("kv_rank", "rot_dim", "rot"))
    ff = layer.get("mlp")
    if ff is None:
        return
    if not isinstance(ff, dict) or ff.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{source}: {where}.mlp.kind must be 'dense' or 'moe' (or mlp null for no feed-forward)")
    if ff["kind"] == "dense":
        _need_ints(source, f"{where}.mlp", ff, ("ff",))
        return
    _need_ints(source, f"{where}.mlp.expert", ff.get("expert"), ("ff",))
    _need_ints(source, f"{where}.mlp.router", ff.get("router"), ("experts", "top"))
    if ff["router"]["top"] > ff["router"]["experts"]:
        raise ConfigError(f"{source}: {where}.mlp.router.top is larger than .experts")
    if ff["router"].get("scale") is not None:
        _number(source, f"{where}.mlp.router.scale", ff["router"]["scale"])
    if ff.get("shared") is not None:
        _need_ints(source, f"{where}.mlp.shared", ff["shared"], ("ff",))


def _mixer_spec(h: int, eps: float, kind: str, m: Dict[str, Any]) -> PartSpec:
    owns = m.get("kv_from") is None
    if kind == "attention":
        params: Dict[str, Any] = {
            "hidden_size": h, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
            "scale": float(m["scale"]), "lambda_init": float(m["diff"]), "eps": eps, "bias": True, "owns_cache": owns}
        if m.get("conv"):
            params["proj_conv"] = {"taps": m["conv"]}
        if m.get("q_temp"):
            params["q_temp"] = {"coef": float(m["q_temp"]["coef"]), "every": int(m["q_temp"]["every"])}
        return PartSpec("differential_attention", params)
    position = PartSpec("rope", {"head_dim": m["rot_dim"], "rotary_dim": m["rot"]["dims"], "theta": float(m["rot"]["base"])})
    return PartSpec("latent_attention", {
        "hidden_size": h, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"], "kv_rank": m["kv_rank"],
        "q_rank": m["q_rank"], "scale": float(m["scale"]), "eps": eps, "position": position, "owns_cache": owns, "gate": False,
        "sink": "sink"})


def _feed_forward_spec(h: int, ff: Any):
    if ff is None:
        return None
    if ff["kind"] == "dense":
        return PartSpec("dense_relu2", {"hidden_size": h, "intermediate_size": ff["ff"], "names": {"up": "up", "down": "down"}})
    shared = ff.get("shared") or {}
    return PartSpec("sparse_moe", {
        "hidden_size": h, "num_experts": ff["router"]["experts"], "top_k": ff["router"]["top"],
        "expert_intermediate_size": ff["expert"]["ff"], "shared_intermediate_size": int(shared.get("ff", 0)), "shared_gate": False,
        "norm_topk_prob": False, "score": "softmax", "weight_on": "output", "correction": "correction",
        "route_scale": float(ff["router"].get("scale", 1.0)),
        "names": {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down",
                  "shared_gate": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down"}})


def build_plan(cfg: DimuvikConfig) -> ModelPlan:
    h, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("dyt", {"dim": h, "weight_name": ""})
    block = PartSpec("sandwich", {"hidden_size": h, "mixer_norm_name": "norm1", "mixer_post_norm_name": "norm1b",
                                  "feed_forward_norm_name": "norm2", "feed_forward_post_norm_name": "norm2b",
                                  "mixer_name": "mix", "feed_forward_name": "mlp"})
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        ffn = _feed_forward_spec(h, layer.get("mlp"))
        layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=_mixer_spec(h, eps, layer["type"], layer["mixer"]),
                                feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm if ffn is not None else None))
        # the schedule runs the layers in order, so a layer's index is its schedule entry's
        schedule.append(ScheduleEntry(layer=i, cache_from=layer["mixer"].get("kv_from")))
    plan = ModelPlan(architecture=cfg.architecture, hidden_size=h, vocab_size=cfg.vocab, embedding_name="embed",
                     layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, final_norm_prefix="final.norm",
                     lm_head_name="head", eog_token_ids=cfg.eos_token_ids, max_position=None,
                     embedding=PartSpec("token_embedding", {"scale": 0.0 if cfg.embedding_scale == 1.0 else cfg.embedding_scale}))
    plan.validate()
    return plan


register_architecture(ARCHITECTURE, DimuvikConfig, build_plan, replace=True)
