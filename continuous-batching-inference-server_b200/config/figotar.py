"""Typed configuration of Figotar folders.

A Figotar model is a list of unlike layers.  Every layer normalises before AND after each of its two parts
(x += post(mixer(pre(x))), then x += post(feed_forward(pre(x)))); all norms are root-mean-square norms whose weights
are stored around zero.  The mixer is windowed attention with a distance bias, a query temperature and a gate per head
("attention"), causal attention over a cached latent with a rotated key part shared by the heads, a sink in the
softmax and a gate per head ("latent_attention"), or a matrix memory with exponential gates ("mlstm").  The
feed-forward is a gated one with biases (tanh GELU), or absent.  Every size and every constant that may differ between
two models comes from ``config.json``; the tensor names are the format's.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec
from .vekedra import _get, _int, _num, _only

MIXERS = ("attention", "latent_attention", "mlstm")
SLOPE_POWER = 8.0          # the distance bias of head h of H: 2^(-8 (h + 1) / H) per token of distance


def _parse_mixer(kind: str, m: Dict[str, Any], i: int) -> Dict[str, Any]:
    where = f"layers[{i}].mixer."
    if kind == "attention":
        _only(m, ("dim", "heads", "kv_heads", "mask", "q_temp", "scale", "vdim"), where)
        out = {k: _int(m, k, where) for k in ("dim", "heads", "kv_heads", "vdim")}
        out["scale"] = _num(m, "scale", where)
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"config.json: {where}heads={out['heads']} is not a multiple of kv_heads={out['kv_heads']}")
        out["window"] = 0
        if m.get("mask") is not None:
            _only(m["mask"], ("size",), where + "mask.")
            out["window"] = _int(m["mask"], "size", where + "mask.")
        out["q_temp"] = None
        if m.get("q_temp") is not None:
            _only(m["q_temp"], ("coef", "every"), where + "q_temp.")
            out["q_temp"] = (_num(m["q_temp"], "coef", where + "q_temp.", False), _int(m["q_temp"], "every", where + "q_temp."))
        return out
    if kind == "latent_attention":
        _only(m, ("dim", "heads", "kv_rank", "q_rank", "rot", "rot_dim", "scale", "vdim"), where)
        out = {k: _int(m, k, where) for k in ("dim", "heads", "kv_rank", "q_rank", "rot_dim", "vdim")}
        out["scale"] = _num(m, "scale", where)
        rot = _get(m, "rot", where)
        _only(rot, ("base", "dims"), where + "rot.")
        out["rot_base"], out["rot_dims"] = _num(rot, "base", where + "rot."), _int(rot, "dims", where + "rot.")
        if out["rot_dims"] % 2 or out["rot_dims"] > out["rot_dim"]:
            raise ConfigError(f"config.json: {where}rot.dims={out['rot_dims']} must be even and at most rot_dim={out['rot_dim']}")
        return out
    if kind == "mlstm":
        _only(m, ("dim", "gate_cap", "heads", "vdim"), where)
        out = {k: _int(m, k, where) for k in ("dim", "heads", "vdim")}
        out["gate_cap"] = _num(m, "gate_cap", where)
        return out
    raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not one of {sorted(MIXERS)}")


def _parse_mlp(f: Optional[Dict[str, Any]], i: int) -> Optional[Dict[str, Any]]:
    if f is None:
        return None
    where = f"layers[{i}].mlp."
    kind = _get(f, "kind", where)
    if kind != "dense":
        raise ConfigError(f"config.json: {where}'kind' {kind!r} is not one of ['dense']")
    _only(f, ("kind", "ff"), where)
    return {"kind": "dense", "ff": _int(f, "ff", where)}


@dataclass(frozen=True)
class FigotarLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]      # the mixer's sizes and constants, as sorted items
    mlp: Optional[Tuple[Tuple[str, Any], ...]]

    def mixer_dict(self) -> Dict[str, Any]:
        return dict(self.mixer)

    def mlp_dict(self) -> Optional[Dict[str, Any]]:
        return None if self.mlp is None else dict(self.mlp)


@dataclass(frozen=True)
class FigotarConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[FigotarLayer, ...]
    architecture: str = "Figotar"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FigotarConfig":
        _only(d, ("architecture", "architectures", "model_type", "layers", "norm", "vocab", "width"), "")
        norm = _get(d, "norm", "")
        _only(norm, ("eps",), "norm.")
        raw = _get(d, "layers", "")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            _only(entry, ("type", "mixer", "mlp"), f"layers[{i}].")
            kind = _get(entry, "type", f"layers[{i}].")
            mixer = _parse_mixer(kind, _get(entry, "mixer", f"layers[{i}]."), i)
            mlp = _parse_mlp(entry.get("mlp"), i)
            layers.append(FigotarLayer(kind, tuple(sorted(mixer.items(), key=lambda kv: kv[0])),
                                       None if mlp is None else tuple(sorted(mlp.items()))))
        return cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), norm_eps=_num(norm, "eps", "norm."),
                   layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        out = []
        for layer in self.layers:
            m = layer.mixer_dict()
            if layer.type == "attention":
                window, temp = m.pop("window"), m.pop("q_temp")
                if window:
                    m["mask"] = {"size": window}
                if temp is not None:
                    m["q_temp"] = {"coef": temp[0], "every": temp[1]}
            elif layer.type == "latent_attention":
                m["rot"] = {"base": m.pop("rot_base"), "dims": m.pop("rot_dims")}
            out.append({"type": layer.type, "mixer": m, "mlp": layer.mlp_dict()})
        return {"architecture": self.architecture, "layers": out, "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
                "width": self.width}

    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        norm = PartSpec("rmsnorm", {"width": W, "eps": eps, "offset": 1.0, "name": ""})
        none = PartSpec("none", {"width": W})
        specs, ignored = [], []
        for i, layer in enumerate(self.layers):
            m = layer.mixer_dict()
            if layer.type == "attention":
                mixer = PartSpec("gated_attention", {"width": W, "n_head": m["heads"], "n_kv_head": m["kv_heads"],
                                                     "head_dim": m["dim"], "v_head_dim": m["vdim"], "scale": m["scale"],
                                                     "window": m["window"], "qkv_bias": True, "slope_power": SLOPE_POWER,
                                                     "q_temp": m["q_temp"], "head_gate": True})
            elif layer.type == "latent_attention":
                mixer = PartSpec("latent_attention", {"width": W, "n_head": m["heads"], "qk_dim": m["dim"],
                                                      "v_dim": m["vdim"], "rank": m["kv_rank"], "scale": m["scale"],
                                                      "window": 0, "eps": eps, "own_latent": True, "q_rank": m["q_rank"],
                                                      "rot_dim": m["rot_dim"], "rot_base": m["rot_base"],
                                                      "rot_dims": m["rot_dims"], "sinks": True, "gate": "head"})
            else:
                mixer = PartSpec("mlstm", {"width": W, "heads": m["heads"], "dim": m["dim"], "v_dim": m["vdim"],
                                           "gate_cap": m["gate_cap"], "eps": eps})
            f = layer.mlp_dict()
            if f is None:
                ff = PartSpec("nothing", {"width": W})
                ignored.append(rf"l{i}\.norm2b?")      # a folder may still carry the norms of the part that is absent
            else:
                ff = PartSpec("gated", {"width": W, "inner": f["ff"], "activation": "gelu_tanh", "biases": True})
            specs.append(LayerSpec(prefix=f"l{i}.", arrangement="sandwich", mixer=mixer, feed_forward=ff,
                                   norm_mixer=norm, norm_feed_forward=norm if f is not None else none,
                                   norm_prefixes=("norm1", "norm2"), post_norm_mixer=norm,
                                   post_norm_feed_forward=norm if f is not None else None,
                                   post_norm_prefixes=("norm1b", "norm2b")))
        return ModelSpec(width=W, vocab_size=self.vocab, max_positions=0,      # 0: the design sets no limit; the engine's holds
                         token_embedding=PartSpec("token_table", {"vocab_size": self.vocab, "width": W, "tensor": "embed"}),
                         position=PartSpec("none", {"width": W}),
                         layers=tuple(specs), schedule=tuple(range(len(specs))),
                         final_norm=norm, final_norm_prefix="final.norm", head="head", ignored_tensors=tuple(ignored))
