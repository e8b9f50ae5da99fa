"""Typed configuration of the Bepuzen design, read from config.json.

The file lists the layers one by one: each entry names its mixer (`type`), the mixer's sizes and
constants (`mixer`) and its feed-forward (`mlp`, or null).  Nothing is assumed about their order,
and no size or constant has a stand-in in code: what a layer needs and the file lacks is an error
that names the key.

    architecture   "Bepuzen"
    vocab, width   vocabulary and residual width
    norm.eps       eps of every RMS norm
    token_side.dim width of the per-layer token input (the key may be absent: no such input)
    layers[i].type "latent_attention" (rotated key part shared by the heads, sink, output gate) or
                   "latent_attention_2" (no positions, plain softmax, no gate)
    layers[i].mixer  heads, dim, vdim, kv_rank, scale; with positions also rot_dim and rot.base / rot.dims
    layers[i].mlp    null, or kind "dense" with ff
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .qwen3 import ConfigError
from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec

# Positions are 32-bit numbers and exact far beyond this; the design itself names no longest sequence.  The engine
# sizes its block tables for this many tokens unless `EngineConfig.max_model_len` says less.
MAX_POSITIONS = 1 << 20


def _need(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"config.json lacks required key(s): {where}{key}")
    return d[key]


def _pos_int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config key '{where}{key}' must be a positive integer, got {v!r}")
    return v


def _pos_float(d: Mapping[str, Any], key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not v > 0:
        raise ConfigError(f"config key '{where}{key}' must be a positive number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class LatentMixerConfig:
    kind: str                   # "latent_attention" | "latent_attention_2"
    heads: int
    dim: int                    # unrotated query/key size per head
    vdim: int
    kv_rank: int
    scale: float
    rot_dim: int = 0            # rotated query/key size per head (one key part shared by all heads)
    rot_base: float = 0.0
    rot_dims: int = 0           # how many of the rot_dim coordinates are rotated (the rest pass unchanged)

    @property
    def rotary(self) -> bool:
        return self.kind == "latent_attention"


@dataclass(frozen=True)
class BepuzenConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    side_dim: int                                   # 0: no per-layer token input
    mixers: Tuple[LatentMixerConfig, ...]
    ff_sizes: Tuple[int, ...]                       # per layer; 0: the layer has no feed-forward
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    ARCHITECTURE = "Bepuzen"
    MIXERS = ("latent_attention", "latent_attention_2")

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BepuzenConfig":
        layers = _need(d, "layers", "")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config key 'layers' must be a non-empty list")
        eps = _pos_float(_need(d, "norm", ""), "eps", "norm.")
        side = d.get("token_side")
        side_dim = _pos_int(side, "dim", "token_side.") if side is not None else 0
        mixers, ffs = [], []
        for i, L in enumerate(layers):
            at = f"layers[{i}]."
            kind = _need(L, "type", at)
            if kind not in cls.MIXERS:
                raise ConfigError(f"{at}type={kind!r} is not a mixer of this design ({', '.join(cls.MIXERS)})")
            m = _need(L, "mixer", at)
            mat = at + "mixer."
            kw = dict(kind=kind, heads=_pos_int(m, "heads", mat), dim=_pos_int(m, "dim", mat), vdim=_pos_int(m, "vdim", mat),
                      kv_rank=_pos_int(m, "kv_rank", mat), scale=_pos_float(m, "scale", mat))
            if kind == "latent_attention":
                rot = _need(m, "rot", mat)
                kw.update(rot_dim=_pos_int(m, "rot_dim", mat), rot_base=_pos_float(rot, "base", mat + "rot."),
                          rot_dims=_pos_int(rot, "dims", mat + "rot."))
                if kw["rot_dims"] % 2 or kw["rot_dims"] > kw["rot_dim"]:
                    raise ConfigError(f"{mat}rot.dims={kw['rot_dims']} must be even and at most rot_dim={kw['rot_dim']}")
            mixers.append(LatentMixerConfig(**kw))
            mlp = L.get("mlp")                   # null, or no such key: the layer has no feed-forward
            if mlp is None:
                ffs.append(0)
            else:
                kind = _need(mlp, "kind", at + "mlp.")
                if kind != "dense":
                    raise ConfigError(f"{at}mlp.kind={kind!r} is not a feed-forward of this design (dense)")
                ffs.append(_pos_int(mlp, "ff", at + "mlp."))
        eos = d.get("eos_token_id")
        return cls(architecture=cls.ARCHITECTURE, vocab_size=_pos_int(d, "vocab", ""), hidden_size=_pos_int(d, "width", ""),
                   norm_eps=eps, side_dim=side_dim, mixers=tuple(mixers), ff_sizes=tuple(ffs),
                   eos_token_id=eos if isinstance(eos, int) else None,
                   torch_dtype=str(d.get("torch_dtype", "bfloat16")))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for m, ff in zip(self.mixers, self.ff_sizes):
            mixer: Dict[str, Any] = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale}
            if m.rotary:
                mixer.update(rot_dim=m.rot_dim, rot={"base": m.rot_base, "dims": m.rot_dims})
            layers.append({"type": m.kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None})
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                             "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    # ------------------------------------------------------------------ the model as parts
    @property
    def num_hidden_layers(self) -> int:
        return len(self.mixers)

    def model_spec(self) -> ModelSpec:
        D = self.hidden_size
        norm = PartSpec("rmsnorm_scalar", {"size": D, "eps": self.norm_eps, "leaf": ""})
        layers = []
        for i, (m, ff) in enumerate(zip(self.mixers, self.ff_sizes)):
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "num_heads": m.heads, "nope_dim": m.dim, "rot_dim": m.rot_dim if m.rotary else 0,
                "v_dim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": self.norm_eps,
                "position_encoding": (PartSpec("rotary_partial", {"dims": m.rot_dims, "base": m.rot_base})
                                      if m.rotary else None),
                "sink": m.rotary, "output_gate": m.rotary})
            parts = {"mixer": mixer, "norm": norm}
            if ff:
                parts["feed_forward"] = PartSpec("dense_xielu", {"hidden_size": D, "intermediate_size": ff})
            if self.side_dim:
                parts["token_side"] = PartSpec("token_side_input", {
                    "hidden_size": D, "dim": self.side_dim, "offset": i * self.side_dim,
                    "table_width": self.num_hidden_layers * self.side_dim, "vocab_size": self.vocab_size,
                    "eps": self.norm_eps, "table": "side.embed"})
            layers.append(LayerSpec(prefix=f"l{i}", block=PartSpec("parallel_residual", {
                "norm_name": "norm1", "mixer_name": "mix", "feed_forward_name": "mlp", "token_side_name": "side"}),
                parts=parts))
        embedding = {"vocab_size": self.vocab_size, "hidden_size": D, "leaf": ""}
        if self.side_dim:
            embedding["extra_tables"] = {"side.embed": self.num_hidden_layers * self.side_dim}
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=D, vocab_size=self.vocab_size, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", embedding), layers=tuple(layers),
            order=tuple(LayerRun(i) for i in range(len(layers))), final_norm=norm,
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": D, "leaf": ""}),
            embedding_prefix="embed", final_norm_prefix="final.norm", lm_head_prefix="head")
        spec.validate()
        return spec

    @staticmethod
    def canonical_tensor_name(name: str) -> str:
        return name
