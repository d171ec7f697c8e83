"""Typed configuration of Vekedra folders.

A Vekedra model is a list of unlike layers.  Every layer is a parallel block (one LayerNorm whose
output feeds both the mixer and the feed-forward; both results are added to the stream together).  The
mixer is a state-space layer ("mamba2") or windowed attention over a cached latent ("latent_attention",
which may read the latent of an earlier layer); the feed-forward is a gated one, a routed mixture of
such, or absent.  There is no position encoding and no position limit.  Every size and every constant
that may differ between two models comes from ``config.json``; the tensor names are the format's.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec


def _get(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where}'{key}' is missing")
    return d[key]


def _int(d, key, where, minimum=1) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}'{key}' must be an integer >= {minimum}, got {v!r}")
    return v


def _num(d, key, where, positive=True) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"config.json: {where}'{key}' must be a{' positive' if positive else ''} number, got {v!r}")
    return float(v)


def _only(d: Dict[str, Any], allowed, where: str) -> None:
    """Keys the design does not have are reported and passed over: a folder may carry notes of its own."""
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where.rstrip('.') or 'the top level'} must be an object, got {d!r}")
    extra = sorted(set(d) - set(allowed))
    if extra:
        warnings.warn(f"config.json: {where}unknown keys {extra} are ignored; known: {sorted(allowed)}", stacklevel=3)


@dataclass(frozen=True)
class VekedraLayer:
    type: str                               # "mamba2" | "latent_attention"
    mixer: Tuple[Tuple[str, Any], ...]      # the mixer's sizes and constants, as sorted items
    mlp: Optional[Tuple[Tuple[str, Any], ...]]

    def mixer_dict(self) -> Dict[str, Any]:
        return dict(self.mixer)

    def mlp_dict(self) -> Optional[Dict[str, Any]]:
        return None if self.mlp is None else dict(self.mlp)


def _parse_mixer(kind: str, m: Dict[str, Any], i: int, n_before) -> Dict[str, Any]:
    where = f"layers[{i}].mixer."
    if kind == "mamba2":
        _only(m, ("conv", "groups", "heads", "norm_groups", "state", "vdim"), where)
        out = {k: _int(m, k, where) for k in ("conv", "groups", "heads", "norm_groups", "state", "vdim")}
        if out["heads"] % out["groups"]:
            raise ConfigError(f"config.json: {where}heads={out['heads']} is not a multiple of groups={out['groups']}")
        if (out["heads"] * out["vdim"]) % out["norm_groups"]:
            raise ConfigError(f"config.json: {where}heads*vdim={out['heads'] * out['vdim']} is not a multiple of "
                              f"norm_groups={out['norm_groups']}")
        return out
    if kind == "latent_attention":
        _only(m, ("dim", "heads", "kv_rank", "kv_from", "mask", "scale", "vdim"), where)
        out = {k: _int(m, k, where) for k in ("dim", "heads", "kv_rank", "vdim")}
        out["scale"] = _num(m, "scale", where)
        mask = _get(m, "mask", where)
        _only(mask, ("size",), where + "mask.")
        out["window"] = _int(mask, "size", where + "mask.")
        src = m.get("kv_from")
        if src is not None:
            if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                raise ConfigError(f"config.json: {where}'kv_from' must name an earlier layer, got {src!r}")
            other = n_before[src]
            if other.type != "latent_attention" or other.mixer_dict().get("kv_from") is not None:
                raise ConfigError(f"config.json: {where}'kv_from'={src}: that layer keeps no latent of its own")
            if other.mixer_dict()["kv_rank"] != out["kv_rank"]:
                raise ConfigError(f"config.json: {where}kv_rank={out['kv_rank']} differs from layer {src}'s "
                                  f"{other.mixer_dict()['kv_rank']}")
            out["kv_from"] = src
        return out
    raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not one of ['latent_attention', 'mamba2']")


def _parse_mlp(f: Optional[Dict[str, Any]], i: int) -> Optional[Dict[str, Any]]:
    if f is None:
        return None
    where = f"layers[{i}].mlp."
    kind = _get(f, "kind", where)
    if kind == "dense":
        _only(f, ("kind", "ff"), where)
        return {"kind": "dense", "ff": _int(f, "ff", where)}
    if kind == "moe":
        _only(f, ("kind", "expert", "router"), where)
        expert, router = _get(f, "expert", where), _get(f, "router", where)
        _only(expert, ("ff",), where + "expert.")
        _only(router, ("experts", "top"), where + "router.")
        out = {"kind": "moe", "ff": _int(expert, "ff", where + "expert."),
               "experts": _int(router, "experts", where + "router."), "top": _int(router, "top", where + "router.")}
        if out["top"] > out["experts"]:
            raise ConfigError(f"config.json: {where}router.top={out['top']} exceeds experts={out['experts']}")
        return out
    raise ConfigError(f"config.json: {where}'kind' {kind!r} is not one of ['dense', 'moe']")


@dataclass(frozen=True)
class VekedraConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[VekedraLayer, ...]
    architecture: str = "Vekedra"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VekedraConfig":
        _only(d, ("architecture", "architectures", "model_type", "embedding", "layers", "norm", "vocab", "width"), "")
        emb, norm = _get(d, "embedding", ""), _get(d, "norm", "")
        _only(emb, ("scale",), "embedding.")
        _only(norm, ("eps",), "norm.")
        raw = _get(d, "layers", "")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            _only(entry, ("type", "mixer", "mlp"), f"layers[{i}].")
            kind = _get(entry, "type", f"layers[{i}].")
            mixer = _parse_mixer(kind, _get(entry, "mixer", f"layers[{i}]."), i, layers)
            mlp = _parse_mlp(entry.get("mlp"), i)
            layers.append(VekedraLayer(kind, tuple(sorted(mixer.items())),
                                       None if mlp is None else tuple(sorted(mlp.items()))))
        return cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), embedding_scale=_num(emb, "scale", "embedding.", False),
                   norm_eps=_num(norm, "eps", "norm."), layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        out = []
        for layer in self.layers:
            m = layer.mixer_dict()
            if layer.type == "latent_attention":
                m["mask"] = {"size": m.pop("window")}
            f = layer.mlp_dict()
            if f is not None and f["kind"] == "moe":
                f = {"kind": "moe", "expert": {"ff": f["ff"]}, "router": {"experts": f["experts"], "top": f["top"]}}
            out.append({"type": layer.type, "mixer": m, "mlp": f})
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale}, "layers": out,
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    def model_spec(self) -> ModelSpec:
        W = self.width
        norm = PartSpec("layernorm", {"width": W, "eps": self.norm_eps, "names": ("", ".b")})
        none = PartSpec("none", {"width": W})
        specs = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer_dict()
            source = None
            if layer.type == "mamba2":
                mixer = PartSpec("mamba2", {"width": W, "heads": m["heads"], "head_dim": m["vdim"], "state": m["state"],
                                            "groups": m["groups"], "taps": m["conv"], "norm_groups": m["norm_groups"],
                                            "eps": self.norm_eps})
            else:
                source = m.get("kv_from")
                mixer = PartSpec("latent_attention", {"width": W, "n_head": m["heads"], "qk_dim": m["dim"],
                                                      "v_dim": m["vdim"], "rank": m["kv_rank"], "scale": m["scale"],
                                                      "window": m["window"], "eps": self.norm_eps,
                                                      "own_latent": source is None})
            f = layer.mlp_dict()
            if f is None:
                ff = PartSpec("nothing", {"width": W})
            elif f["kind"] == "dense":
                ff = PartSpec("gated", {"width": W, "inner": f["ff"], "activation": "silu"})
            else:
                ff = PartSpec("routed", {"width": W, "inner": f["ff"], "experts": f["experts"], "top": f["top"],
                                         "activation": "silu", "score": "sigmoid", "renormalize": False,
                                         "weight_on": "input"})
            specs.append(LayerSpec(prefix=f"l{i}.", arrangement="parallel", mixer=mixer, feed_forward=ff,
                                   norm_mixer=norm, norm_feed_forward=none, cache_source=source,
                                   norm_prefixes=("norm1", "norm2")))
        return ModelSpec(width=W, vocab_size=self.vocab, max_positions=0,      # 0: the design sets no limit; the engine's holds
                         token_embedding=PartSpec("token_table", {"vocab_size": self.vocab, "width": W, "tensor": "embed",
                                                                  "multiplier": self.embedding_scale}),
                         position=PartSpec("none", {"width": W}),
                         layers=tuple(specs), schedule=tuple(range(len(specs))),
                         final_norm=norm, final_norm_prefix="final.norm", head="head")
