"""Typed configuration of the Torisun design, read from config.json.

The file lists the layers one by one: each entry names its mixer (`type`), the mixer's sizes and constants
(`mixer`) and its feed-forward (`mlp`, or null).  Nothing is assumed about their order, and no size or
constant has a stand-in in code: what a layer needs and the file lacks is an error that names the key.

    architecture   "Torisun"
    vocab, width   vocabulary and residual width
    norm.eps       eps of every RMS norm
    layers[i].type "attention"
    layers[i].mixer  heads, kv_heads, dim (query/key size per head), vdim (value size per head), scale,
                     mask.size (window), mask.keep_first (first positions every query sees),
                     rot.base, rot.dims and optionally rot.scaling {factor, original, fast, slow},
                     kv_from (optional): the layer whose cached keys and values this layer reads
    layers[i].mlp    null; or kind "dense" with ff and limit; or kind "moe" with expert.ff,
                     router.{experts, top, scale} and optionally shared.ff
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .bepuzen import MAX_POSITIONS, _need, _pos_float, _pos_int
from .qwen3 import ConfigError
from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec


def _count(d: Mapping[str, Any], key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"config key '{where}{key}' must be a non-negative integer, got {v!r}")
    return v


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    keep_first: int
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotaryScaling] = None
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                   # "dense" | "moe"
    ff: int                     # dense: its size; moe: the size of one expert
    limit: float = 0.0          # dense
    experts: int = 0            # moe
    top: int = 0
    route_scale: float = 0.0
    shared_ff: int = 0          # 0: no shared expert


@dataclass(frozen=True)
class TorisunConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    mixers: Tuple[AttentionMixerConfig, ...]
    mlps: Tuple[Optional[FeedForwardConfig], ...]
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    ARCHITECTURE = "Torisun"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "TorisunConfig":
        layers = _need(d, "layers", "")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config key 'layers' must be a non-empty list")
        eps = _pos_float(_need(d, "norm", ""), "eps", "norm.")
        mixers, mlps = [], []
        for i, L in enumerate(layers):
            at = f"layers[{i}]."
            kind = _need(L, "type", at)
            if kind != "attention":
                raise ConfigError(f"{at}type={kind!r} is not a mixer of this design (attention)")
            mixers.append(cls._mixer(_need(L, "mixer", at), at + "mixer.", i, mixers))
            mlps.append(cls._mlp(L.get("mlp"), at + "mlp."))
        eos = d.get("eos_token_id")
        return cls(architecture=cls.ARCHITECTURE, vocab_size=_pos_int(d, "vocab", ""), hidden_size=_pos_int(d, "width", ""),
                   norm_eps=eps, mixers=tuple(mixers), mlps=tuple(mlps), eos_token_id=eos if isinstance(eos, int) else None,
                   torch_dtype=str(d.get("torch_dtype", "bfloat16")))

    @staticmethod
    def _mixer(m: Mapping[str, Any], at: str, index: int, earlier) -> AttentionMixerConfig:
        mask, rot = _need(m, "mask", at), _need(m, "rot", at)
        sc = rot.get("scaling") if isinstance(rot, Mapping) else None
        scaling = None
        if sc is not None:
            w = at + "rot.scaling."
            scaling = RotaryScaling(_pos_float(sc, "factor", w), _pos_float(sc, "original", w), _pos_float(sc, "fast", w),
                                    _pos_float(sc, "slow", w))
        c = AttentionMixerConfig(
            heads=_pos_int(m, "heads", at), kv_heads=_pos_int(m, "kv_heads", at), dim=_pos_int(m, "dim", at),
            vdim=_pos_int(m, "vdim", at), scale=_pos_float(m, "scale", at), window=_pos_int(mask, "size", at + "mask."),
            keep_first=_count(mask, "keep_first", at + "mask."), rot_base=_pos_float(rot, "base", at + "rot."),
            rot_dims=_pos_int(rot, "dims", at + "rot."), rot_scaling=scaling,
            kv_from=None if m.get("kv_from") is None else _count(m, "kv_from", at))
        if c.heads % c.kv_heads:
            raise ConfigError(f"{at}heads={c.heads} must be a multiple of kv_heads={c.kv_heads}")
        if c.rot_dims % 2 or c.rot_dims > c.dim:
            raise ConfigError(f"{at}rot.dims={c.rot_dims} must be even and at most dim={c.dim}")
        if c.kv_from is not None:
            if c.kv_from >= index:
                raise ConfigError(f"{at}kv_from={c.kv_from} must name an earlier layer")
            o = earlier[c.kv_from]
            if o.kv_from is not None:
                raise ConfigError(f"{at}kv_from={c.kv_from} names a layer that has no keys and values of its own")
            if (o.kv_heads, o.dim, o.vdim) != (c.kv_heads, c.dim, c.vdim):
                raise ConfigError(f"{at}kv_from={c.kv_from}: kv_heads, dim and vdim must equal that layer's")
        return c

    @staticmethod
    def _mlp(mlp: Optional[Mapping[str, Any]], at: str) -> Optional[FeedForwardConfig]:
        if mlp is None:
            return None
        kind = _need(mlp, "kind", at)
        if kind == "dense":
            return FeedForwardConfig("dense", _pos_int(mlp, "ff", at), limit=_pos_float(mlp, "limit", at))
        if kind == "moe":
            r = _need(mlp, "router", at)
            sh = mlp.get("shared")
            c = FeedForwardConfig("moe", _pos_int(_need(mlp, "expert", at), "ff", at + "expert."),
                                  experts=_pos_int(r, "experts", at + "router."), top=_pos_int(r, "top", at + "router."),
                                  route_scale=_pos_float(r, "scale", at + "router."),
                                  shared_ff=_pos_int(sh, "ff", at + "shared.") if sh is not None else 0)
            if c.top > c.experts:
                raise ConfigError(f"{at}router.top={c.top} exceeds router.experts={c.experts}")
            return c
        raise ConfigError(f"{at}kind={kind!r} is not a feed-forward of this design (dense, moe)")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for m, f in zip(self.mixers, self.mlps):
            rot: Dict[str, Any] = {"base": m.rot_base, "dims": m.rot_dims}
            if m.rot_scaling is not None:
                s = m.rot_scaling
                rot["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                                     "mask": {"size": m.window, "keep_first": m.keep_first}, "rot": rot}
            if m.kv_from is not None:
                mixer["kv_from"] = m.kv_from
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff, "limit": f.limit}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.ff},
                       "router": {"experts": f.experts, "top": f.top, "scale": f.route_scale}}
                if f.shared_ff:
                    mlp["shared"] = {"ff": f.shared_ff}
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                             "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    # ------------------------------------------------------------------ the model as parts
    @property
    def num_hidden_layers(self) -> int:
        return len(self.mixers)

    def _retention(self, owner: int) -> Tuple[int, int]:
        """What the cache of layer `owner` must keep: the widest window and the most first positions among the
        layer itself and the layers that read its keys and values."""
        users = [m for i, m in enumerate(self.mixers) if i == owner or m.kv_from == owner]
        return max(m.window for m in users), max(m.keep_first for m in users)

    def model_spec(self) -> ModelSpec:
        D, eps = self.hidden_size, self.norm_eps
        norm = PartSpec("rmsnorm", {"size": D, "eps": eps, "leaf": ""})
        layers = []
        for i, (m, f) in enumerate(zip(self.mixers, self.mlps)):
            window, first = self._retention(i if m.kv_from is None else m.kv_from)
            scaling = None
            if m.rot_scaling is not None:
                s = m.rot_scaling
                scaling = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            mixer = PartSpec("gqa_window_sink", {
                "hidden_size": D, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "qk_dim": m.dim, "v_dim": m.vdim,
                "scale": m.scale, "norm_eps": eps, "window": m.window, "keep_first": m.keep_first, "sink": True,
                "own_kv": m.kv_from is None, "retain_window": window, "retain_first": first,
                "position_encoding": PartSpec("rotary_partial", {"dims": m.rot_dims, "base": m.rot_base, "scaling": scaling})})
            parts = {"mixer": mixer, "mixer_norm": norm}
            if f is not None:
                if f.kind == "dense":
                    parts["feed_forward"] = PartSpec("gated_dense", {
                        "hidden_size": D, "intermediate_size": f.ff, "activation": "clamped_swish", "limit": f.limit})
                else:
                    parts["feed_forward"] = PartSpec("routed_experts", {
                        "hidden_size": D, "num_experts": f.experts, "top_k": f.top, "expert_size": f.ff,
                        "route_scale": f.route_scale, "shared_size": f.shared_ff})
                parts["feed_forward_norm"] = norm
            layers.append(LayerSpec(prefix=f"l{i}", block=PartSpec("postnorm_residual", {
                "mixer_name": "mix", "feed_forward_name": "mlp", "mixer_norm_name": "norm1", "feed_forward_norm_name": "norm2"}),
                parts=parts))
        # the order is the layer order; a layer with kv_from reads the run (= layer) of that index
        order = tuple(LayerRun(i, cache_from=m.kv_from) for i, m in enumerate(self.mixers))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=D, vocab_size=self.vocab_size, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": D, "leaf": "",
                                                   "norm_leaf": "norm", "norm_eps": eps}),
            layers=tuple(layers), order=order, final_norm=norm,
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": D, "leaf": "", "tied_to": "embed"}),
            embedding_prefix="embed", final_norm_prefix="final.norm", lm_head_prefix="head")
        spec.validate()
        return spec

    @staticmethod
    def canonical_tensor_name(name: str) -> str:
        return name

    def ignorable_tensor(self, name: str) -> bool:
        """A norm gain stored for a feed-forward that the layer does not have."""
        return any(f is None and name == f"l{i}.norm2" for i, f in enumerate(self.mlps))
