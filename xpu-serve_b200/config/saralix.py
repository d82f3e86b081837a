"""Typed configuration of Saralix, read from config.json's own keys.

config.json gives the model's `width`, `vocab` and `norm.eps`, and under `layers` one entry per layer:
`type` (which mixer), `mixer` (its sizes and constants) and `mlp` (its feed-forward, or null for none).
Every size and every constant that can differ between two models of the design is read from there;
what the design fixes (the activation constants of the dense feed-forward, the factor in the rotation's
stretch) lives in the specs' defaults (config/spec.py).

Layer types:
  latent_attention     latent attention over every earlier position, softmax, a sigmoid gate per head
  latent_attention_2   latent attention over a window (`mask.size`), softmax with a sink per head, no gate
  mamba2               a state-space recurrence behind a short convolution
Feed-forwards (`mlp.kind`): `dense` (a clamped gated unit, `ff`, `limit`) and `moe` (`expert.ff`,
`router.experts`, `router.top`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .json_util import ConfigError, get_float, get_int, get_str
from .spec import (ClampedGLUSpec, LatentAttentionSpec, LayerCall, LayerSpec, Mamba2Spec, ModelSpec, NormSpec,
                   RopeScalingSpec, RoutedExpertsSpec, ScaledRopeSpec)

LATENT, LATENT_WINDOW, MAMBA2 = "latent_attention", "latent_attention_2", "mamba2"
# No key of config.json limits a sequence's length; the cache's own limit is what bounds one.
MAX_POSITION = 1 << 22


def _obj(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: missing object '{key}'")
    return v


@dataclass(frozen=True)
class SaralixLayer:
    type: str
    mixer: object                    # LatentAttentionSpec | Mamba2Spec, names and all
    mlp: Optional[object]            # ClampedGLUSpec | RoutedExpertsSpec | None
    raw: dict                        # the entry as read (written back by to_json)


@dataclass(frozen=True)
class SaralixConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[SaralixLayer, ...]
    architecture: str = "Saralix"

    # ---------------------------------------------------------------- parsing
    @staticmethod
    def _rotation(m: dict, rot_dim: int, where: str) -> ScaledRopeSpec:
        rot = _obj(m, "rot", where)
        rw = f"{where} rot"
        dims = get_int(rot, "dims", rw)
        if dims <= 0 or dims % 2 != 0 or dims > rot_dim:
            raise ConfigError(f"{rw}: dims {dims} must be even and at most rot_dim {rot_dim}")
        base = get_float(rot, "base", rw)
        if not base > 1.0:
            raise ConfigError(f"{rw}: base must be larger than 1")
        scaling = None
        if rot.get("scaling") is not None:
            sc, sw = _obj(rot, "scaling", rw), f"{rw} scaling"
            scaling = RopeScalingSpec(get_float(sc, "factor", sw), get_float(sc, "original", sw),
                                      get_float(sc, "fast", sw), get_float(sc, "slow", sw))
            if not (scaling.factor > 0 and scaling.original > 0 and scaling.fast > 0 and scaling.slow > 0):
                raise ConfigError(f"{sw}: factor, original, fast and slow must be positive")
        return ScaledRopeSpec(head_dim=rot_dim, theta=base, dims=dims, scaling=scaling)

    @classmethod
    def _latent(cls, m: dict, width: int, eps: float, kind: str, where: str) -> LatentAttentionSpec:
        rot_dim = get_int(m, "rot_dim", where)
        sizes = {k: get_int(m, k, where) for k in ("heads", "dim", "vdim", "kv_rank")}
        if min(sizes.values()) <= 0 or rot_dim <= 0 or rot_dim % 2 != 0:
            raise ConfigError(f"{where}: heads, dim, vdim and kv_rank must be positive and rot_dim even")
        window = 0
        if kind == LATENT_WINDOW:
            window = get_int(_obj(m, "mask", where), "size", f"{where} mask")
            if window <= 0:
                raise ConfigError(f"{where} mask: size must be positive")
        return LatentAttentionSpec(
            hidden=width, heads=sizes["heads"], dim=sizes["dim"], rot_dim=rot_dim, vdim=sizes["vdim"],
            kv_rank=sizes["kv_rank"], scale=get_float(m, "scale", where), eps=eps,
            position=cls._rotation(m, rot_dim, where), window=window, sink=kind == LATENT_WINDOW,
            head_gate=kind == LATENT)

    @staticmethod
    def _mamba2(m: dict, width: int, eps: float, where: str) -> Mamba2Spec:
        s = Mamba2Spec(hidden=width, heads=get_int(m, "heads", where), vdim=get_int(m, "vdim", where),
                       state=get_int(m, "state", where), groups=get_int(m, "groups", where),
                       taps=get_int(m, "conv", where), norm_groups=get_int(m, "norm_groups", where), eps=eps)
        if min(s.heads, s.vdim, s.state, s.groups, s.taps, s.norm_groups) <= 0:
            raise ConfigError(f"{where}: every size must be positive")
        if s.heads % s.groups != 0:
            raise ConfigError(f"{where}: {s.heads} heads over {s.groups} groups")
        if s.inner % s.norm_groups != 0:
            raise ConfigError(f"{where}: {s.inner} channels in {s.norm_groups} norm groups")
        return s

    @staticmethod
    def _mlp(f: Optional[dict], width: int, where: str):
        if f is None:
            return None
        if not isinstance(f, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        kind = get_str(f, "kind", where)
        if kind == "dense":
            spec = ClampedGLUSpec(hidden=width, intermediate=get_int(f, "ff", where), limit=get_float(f, "limit", where))
            if spec.intermediate <= 0 or not spec.limit > 0:
                raise ConfigError(f"{where}: ff and limit must be positive")
            return spec
        if kind == "moe":
            router = _obj(f, "router", where)
            spec = RoutedExpertsSpec(hidden=width, intermediate=get_int(_obj(f, "expert", where), "ff", f"{where} expert"),
                                     experts=get_int(router, "experts", f"{where} router"),
                                     top=get_int(router, "top", f"{where} router"))
            if spec.intermediate <= 0 or not 0 < spec.top <= spec.experts:
                raise ConfigError(f"{where}: expert.ff must be positive and 0 < router.top <= router.experts")
            return spec
        raise ConfigError(f"{where}: unknown feed-forward kind '{kind}' (dense, moe)")

    @classmethod
    def from_json(cls, cfg: dict) -> "SaralixConfig":
        w = "config.json"
        width, vocab = get_int(cfg, "width", w), get_int(cfg, "vocab", w)
        eps = get_float(_obj(cfg, "norm", w), "eps", f"{w} norm")
        if width <= 0 or vocab <= 0 or not eps > 0:
            raise ConfigError(f"{w}: width, vocab and norm.eps must be positive")
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(f"{w}: 'layers' must be a list with at least one entry")
        layers = []
        for i, e in enumerate(entries):
            where = f"{w} layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"{where}: must be an object")
            kind = get_str(e, "type", where)
            m = _obj(e, "mixer", where)
            if kind in (LATENT, LATENT_WINDOW):
                mixer: object = cls._latent(m, width, eps, kind, f"{where} mixer")
            elif kind == MAMBA2:
                mixer = cls._mamba2(m, width, eps, f"{where} mixer")
            else:
                raise ConfigError(f"{where}: unknown layer type '{kind}' ({LATENT}, {LATENT_WINDOW}, {MAMBA2})")
            layers.append(SaralixLayer(kind, mixer, cls._mlp(e.get("mlp"), width, f"{where} mlp"), e))
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers))

    def to_json(self) -> dict:
        return {"architecture": self.architecture, "layers": [l.raw for l in self.layers],
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    # ------------------------------------------------------- to a model spec
    def model_spec(self) -> ModelSpec:
        norm = NormSpec(self.width, self.norm_eps, kind="layernorm")
        layers = tuple(
            LayerSpec(prefix=f"l{i}.", mixer=l.mixer, ffn=l.mlp, norm=norm, sandwich=True,
                      names={"pre_mixer": "norm1", "post_mixer": "norm1b", "pre_ffn": "norm2", "post_ffn": "norm2b"})
            for i, l in enumerate(self.layers))
        spec = ModelSpec(arch="saralix", vocab=self.vocab, hidden=self.width, max_position=MAX_POSITION, layers=layers,
                         order=tuple(LayerCall(i) for i in range(len(layers))), final_norm=norm, tied_head=True,
                         init_std=0.05, prefixes=("",),
                         # a layer without a feed-forward may still carry the norms of one
                         ignorable=tuple(rf"^l{i}\.norm2b?$" for i, l in enumerate(self.layers) if l.mlp is None),
                         names={"embed": "embed", "final_norm": "final.norm", "head": "head"})
        spec.validate()
        return spec
