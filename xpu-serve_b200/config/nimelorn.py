"""Typed configuration of Nimelorn, read from config.json's own keys.

config.json gives the model's `width`, `vocab`, `norm.eps`, the embedding's constants (`embedding.scale` and
`embedding.bigram`: `buckets`, `mul_prev`, `mul_cur`) and under `layers` one entry per layer: `type` (which mixer),
`mixer` (its sizes and constants) and `mlp` (its feed-forward, or null for none). Every size and every constant that can
differ between two models of the design is read from there; what the design fixes (the base of the position vector, the
clamped unit's alpha and shift, the recurrence's 1e-6) lives in the specs' defaults and in the kernels.

Layer types:
  attention   grouped-query attention without rotation, per-head RMS norms on q and k, a sigmoid gate per head, value
              heads of their own size (`vdim`); a query sees the earlier keys of its own block of `mask.size` positions.
              With `kv_from: j` the layer has no keys and values of its own and reads layer j's cache.
  mlstm       the matrix-memory recurrence of xLSTM (`heads`, `dim`, `vdim`, `gate_cap`)
Feed-forwards (`mlp.kind`): `dense` (squared ReLU, `ff`) and `moe` (`expert.ff`, `expert.limit`, `router.experts`,
`router.top`, `router.scale`, and optionally `shared.ff`, `shared.limit`).
A layer is h += norm1(mixer(h)); h += norm2(ff(h)) with RMS norms on the branches only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .json_util import ConfigError, get_float, get_float_or, get_int, get_str
from .spec import (AttentionSpec, ClampedGLUSpec, LayerCall, LayerSpec, MLstmSpec, ModelSpec, NormSpec,
                   PairHashEmbeddingSpec, RoutedExpertsSpec, SquaredReluSpec)

ATTENTION, MLSTM = "attention", "mlstm"
# No key of config.json limits a sequence's length; the cache's own limit is what bounds one.
MAX_POSITION = 1 << 22

_ATTENTION_NAMES = {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "gate": "mix.g", "q_norm": "mix.q.norm",
                    "k_norm": "mix.k.norm", "q_bias": "mix.q.b", "k_bias": "mix.k.b", "v_bias": "mix.v.b"}


def _obj(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: missing object '{key}'")
    return v


@dataclass(frozen=True)
class NimelornLayer:
    type: str
    mixer: object                    # AttentionSpec | MLstmSpec
    mlp: Optional[object]            # SquaredReluSpec | RoutedExpertsSpec | None
    kv_from: Optional[int]           # attention: the layer whose keys and values this one reads
    raw: dict                        # the entry as read (written back by to_json)


@dataclass(frozen=True)
class NimelornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding: PairHashEmbeddingSpec
    layers: Tuple[NimelornLayer, ...]
    raw_embedding: dict
    architecture: str = "Nimelorn"

    # ---------------------------------------------------------------- parsing
    @staticmethod
    def _attention(m: dict, width: int, eps: float, where: str) -> Tuple[AttentionSpec, Optional[int]]:
        heads, kv_heads = get_int(m, "heads", where), get_int(m, "kv_heads", where)
        dim, vdim = get_int(m, "dim", where), get_int(m, "vdim", where)
        if min(heads, kv_heads, dim, vdim) <= 0 or heads % kv_heads != 0:
            raise ConfigError(f"{where}: heads, kv_heads, dim and vdim must be positive and kv_heads divide heads")
        size = get_int(_obj(m, "mask", where), "size", f"{where} mask")
        if size <= 0:
            raise ConfigError(f"{where} mask: size must be positive")
        kv_from = m.get("kv_from")
        if kv_from is not None:
            if isinstance(kv_from, bool) or not isinstance(kv_from, (int, float)) or kv_from != int(kv_from):
                raise ConfigError(f"{where}: kv_from must be a layer's number")
            kv_from = int(kv_from)
        spec = AttentionSpec(hidden=width, heads=heads, kv_heads=kv_heads, head_dim=dim, qk_norm=True, qk_norm_eps=eps,
                             position=None, window=0, head_gate=True, scale=get_float(m, "scale", where),
                             names=dict(_ATTENTION_NAMES), v_dim=vdim, chunk=size, own_kv=kv_from is None)
        return spec, kv_from

    @staticmethod
    def _mlstm(m: dict, width: int, eps: float, where: str) -> MLstmSpec:
        s = MLstmSpec(hidden=width, heads=get_int(m, "heads", where), dim=get_int(m, "dim", where),
                      vdim=get_int(m, "vdim", where), gate_cap=get_float(m, "gate_cap", where), eps=eps)
        if min(s.heads, s.dim, s.vdim) <= 0 or not s.gate_cap > 0:
            raise ConfigError(f"{where}: heads, dim, vdim and gate_cap must be positive")
        return s

    @staticmethod
    def _mlp(f: Optional[dict], width: int, where: str):
        if f is None:
            return None
        if not isinstance(f, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        kind = get_str(f, "kind", where)
        if kind == "dense":
            spec = SquaredReluSpec(hidden=width, intermediate=get_int(f, "ff", where))
            if spec.intermediate <= 0:
                raise ConfigError(f"{where}: ff must be positive")
            return spec
        if kind == "moe":
            router, expert = _obj(f, "router", where), _obj(f, "expert", where)
            shared = None
            if f.get("shared") is not None:
                sh = _obj(f, "shared", where)
                shared = ClampedGLUSpec(hidden=width, intermediate=get_int(sh, "ff", f"{where} shared"),
                                        limit=get_float(sh, "limit", f"{where} shared"),
                                        names={"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"})
                if shared.intermediate <= 0 or not shared.limit > 0:
                    raise ConfigError(f"{where} shared: ff and limit must be positive")
            spec = RoutedExpertsSpec(hidden=width, intermediate=get_int(expert, "ff", f"{where} expert"),
                                     experts=get_int(router, "experts", f"{where} router"),
                                     top=get_int(router, "top", f"{where} router"),
                                     route_scale=get_float_or(router, "scale", 1.0, f"{where} router"),
                                     limit=get_float(expert, "limit", f"{where} expert"), shared=shared)
            if spec.intermediate <= 0 or not 0 < spec.top <= spec.experts or not spec.limit > 0:
                raise ConfigError(f"{where}: expert.ff and expert.limit must be positive and 0 < router.top <= router.experts")
            return spec
        raise ConfigError(f"{where}: unknown feed-forward kind '{kind}' (dense, moe)")

    @classmethod
    def from_json(cls, cfg: dict) -> "NimelornConfig":
        w = "config.json"
        width, vocab = get_int(cfg, "width", w), get_int(cfg, "vocab", w)
        eps = get_float(_obj(cfg, "norm", w), "eps", f"{w} norm")
        if width <= 0 or vocab <= 0 or not eps > 0:
            raise ConfigError(f"{w}: width, vocab and norm.eps must be positive")
        emb = _obj(cfg, "embedding", w)
        big = _obj(emb, "bigram", f"{w} embedding")
        bw = f"{w} embedding bigram"
        embedding = PairHashEmbeddingSpec(width=width, vocab=vocab, scale=get_float(emb, "scale", f"{w} embedding"),
                                          buckets=get_int(big, "buckets", bw), mul_prev=get_int(big, "mul_prev", bw),
                                          mul_cur=get_int(big, "mul_cur", bw), eps=eps)
        if embedding.buckets <= 0 or embedding.mul_prev < 0 or embedding.mul_cur < 0:
            raise ConfigError(f"{bw}: buckets must be positive, mul_prev and mul_cur not negative")
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
            kv_from = None
            if kind == ATTENTION:
                mixer, kv_from = cls._attention(m, width, eps, f"{where} mixer")
                if kv_from is not None:
                    if not 0 <= kv_from < i or layers[kv_from].type != ATTENTION or layers[kv_from].kv_from is not None:
                        raise ConfigError(f"{where} mixer: kv_from {kv_from} must name an earlier attention layer with keys and values of its own")
                    src = layers[kv_from].mixer
                    if (src.kv_heads, src.head_dim, src.v_dim, src.heads) != (mixer.kv_heads, mixer.head_dim, mixer.v_dim, mixer.heads):
                        raise ConfigError(f"{where} mixer: its head counts and sizes must equal those of layer {kv_from}, whose keys and values it reads")
            elif kind == MLSTM:
                mixer = cls._mlstm(m, width, eps, f"{where} mixer")
            else:
                raise ConfigError(f"{where}: unknown layer type '{kind}' ({ATTENTION}, {MLSTM})")
            layers.append(NimelornLayer(kind, mixer, cls._mlp(e.get("mlp"), width, f"{where} mlp"), kv_from, e))
        return cls(vocab=vocab, width=width, norm_eps=eps, embedding=embedding, layers=tuple(layers), raw_embedding=emb)

    def to_json(self) -> dict:
        return {"architecture": self.architecture, "embedding": self.raw_embedding, "layers": [l.raw for l in self.layers],
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    # ------------------------------------------------------- to a model spec
    def model_spec(self) -> ModelSpec:
        norm = NormSpec(self.width, self.norm_eps)
        layers = tuple(
            LayerSpec(prefix=f"l{i}.", mixer=l.mixer, ffn=l.mlp, norm=norm, sandwich=True, kind="branch_norm",
                      names={"post_mixer": "norm1", "post_ffn": "norm2"})
            for i, l in enumerate(self.layers))
        spec = ModelSpec(arch="nimelorn", vocab=self.vocab, hidden=self.width, max_position=MAX_POSITION, layers=layers,
                         order=tuple(LayerCall(i, cache_of=l.kv_from) for i, l in enumerate(self.layers)),
                         final_norm=norm, tied_head=False, init_std=0.05, prefixes=("",),
                         # a layer without a feed-forward may still carry the norm of one
                         ignorable=tuple(rf"^l{i}\.norm2$" for i, l in enumerate(self.layers) if l.mlp is None),
                         names={"embed": "embed", "final_norm": "final.norm", "head": "head"},
                         embedding=self.embedding)
        spec.validate()
        return spec
