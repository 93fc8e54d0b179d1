"""Configuration of the Tibepel decoder: pre-norm layers on a float32 residual stream whose mixer is either a
mamba1 selective scan or two mixers side by side - chunked attention whose softmax weights are mixed across
the heads, and a gated delta rule - followed by a clamped gated feed-forward and a small input that depends
on the token's id alone.

config.json keys (every size and every constant that may differ between models is read, none is assumed):

    architecture            "Tibepel"
    width, vocab            model width and vocabulary size
    embedding.scale         factor on the embedded tokens (a sinusoidal position vector is added after it)
    norm.eps                eps of every RMS norm
    logit_softcap           optional: logits <- c tanh(logits / c)
    token_side.dim          optional: width of the per-layer slice of the table `side.embed`
    layers[i].type          "mamba1" | "parallel"
    layers[i].mixer         mamba1:   inner, state, dt_rank, conv
                            parallel: left_scale, right_scale,
                                      left  {heads, kv_heads, dim, vdim, scale, mask.size}
                                      right {heads, kv_heads, dim, vdim, conv}
    layers[i].mlp           null | {"kind": "dense", "ff": n, "limit": L}
    max_positions           optional: the longest sequence the engine is ever asked for

Tensor names: embed, head, final.norm, side.embed, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.{gate,up,down}(.b),
l<i>.side.{gate,proj,norm}.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

DEFAULT_MAX_POSITIONS = 1 << 17       # the design sets no limit

_MAMBA1_KEYS = ("inner", "state", "dt_rank", "conv")
_LEFT_INTS = ("heads", "kv_heads", "dim", "vdim")
_RIGHT_INTS = ("heads", "kv_heads", "dim", "vdim", "conv")


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@dataclass(frozen=True)
class TibepelLayer:
    type: str                              # "mamba1" | "parallel"
    mixer: Dict[str, Any]
    ff: Optional[int]                      # width of the feed-forward, None for a layer without one
    limit: Optional[float] = None          # the feed-forward's clamp


@dataclass(frozen=True)
class TibepelConfig:
    width: int
    vocab: int
    eps: float
    embedding_scale: float
    layers: Tuple[TibepelLayer, ...]
    logit_softcap: Optional[float] = None
    side_dim: Optional[int] = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    ARCHITECTURE = "Tibepel"

    @property
    def architecture(self) -> str:
        return self.ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    # ---- reading -------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, obj: Dict[str, Any], where: str = "config.json") -> "TibepelConfig":
        p: List[str] = []

        def integer(d, key, what, minimum=1):
            v = d.get(key) if isinstance(d, dict) else None
            if not _is_int(v) or v < minimum:
                p.append(f"{what}`{key}` must be an integer >= {minimum}, got {v!r}")
                return minimum
            return v

        def number(d, key, what, positive=True):
            v = d.get(key) if isinstance(d, dict) else None
            if not _is_num(v) or (positive and not v > 0):
                p.append(f"{what}`{key}` must be a number{' > 0' if positive else ''}, got {v!r}")
                return 1.0
            return float(v)

        width = integer(obj, "width", "")
        vocab = integer(obj, "vocab", "")
        eps = number(obj.get("norm"), "eps", "norm: ")
        emb = obj.get("embedding")
        scale = number(emb, "scale", "embedding: ") if emb is not None else 1.0
        cap = obj.get("logit_softcap")
        if cap is not None and (not _is_num(cap) or not cap > 0):
            p.append(f"`logit_softcap` must be a number > 0 or absent, got {cap!r}")
            cap = None
        side = obj.get("token_side")
        side_dim = None
        if side is not None:
            side_dim = integer(side, "dim", "token_side: ")
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(p + ["`layers` must be a non-empty list"], where)
        layers: List[TibepelLayer] = []
        for i, e in enumerate(raw_layers):
            at = f"layers[{i}]: "
            if not isinstance(e, dict):
                p.append(at + "must be an object")
                continue
            kind, m = e.get("type"), e.get("mixer")
            if not isinstance(m, dict):
                p.append(at + "`mixer` must be an object")
                m = {}
            mixer: Dict[str, Any] = {}
            if kind == "mamba1":
                for key in _MAMBA1_KEYS:
                    mixer[key] = integer(m, key, at)
            elif kind == "parallel":
                mixer["left_scale"] = number(m, "left_scale", at, positive=False)
                mixer["right_scale"] = number(m, "right_scale", at, positive=False)
                left, right = m.get("left"), m.get("right")
                lm: Dict[str, Any] = {key: integer(left, key, at + "left: ") for key in _LEFT_INTS}
                lm["scale"] = number(left, "scale", at + "left: ")
                lm["chunk"] = integer(left.get("mask") if isinstance(left, dict) else None, "size", at + "left: mask: ")
                if lm["heads"] % lm["kv_heads"]:
                    p.append(at + f"left: `heads` {lm['heads']} is not a multiple of `kv_heads` {lm['kv_heads']}")
                rm: Dict[str, Any] = {key: integer(right, key, at + "right: ") for key in _RIGHT_INTS}
                if rm["heads"] % rm["kv_heads"]:
                    p.append(at + f"right: `heads` {rm['heads']} is not a multiple of `kv_heads` {rm['kv_heads']}")
                mixer["left"], mixer["right"] = lm, rm
            else:
                p.append(at + f"`type` = {kind!r} is not known (mamba1, parallel)")
            mlp, ff, limit = e.get("mlp"), None, None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    p.append(at + f"`mlp` must be null or an object of kind \"dense\", got {mlp!r}")
                else:
                    ff = integer(mlp, "ff", at + "mlp: ")
                    limit = number(mlp, "limit", at + "mlp: ")
            layers.append(TibepelLayer(kind if kind in ("mamba1", "parallel") else "mamba1", mixer, ff, limit))
        max_pos = obj.get("max_positions", DEFAULT_MAX_POSITIONS)
        if not _is_int(max_pos) or max_pos < 1:
            p.append(f"`max_positions` must be a positive integer, got {max_pos!r}")
            max_pos = DEFAULT_MAX_POSITIONS
        eos = obj.get("eos_token_id")
        eos_ids: Tuple[int, ...] = ()
        if _is_int(eos):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(_is_int(t) for t in eos):
            eos_ids = tuple(eos)
        elif eos is not None:
            p.append(f"`eos_token_id` must be an integer or a list of integers, got {eos!r}")
        if p:
            raise ConfigError(p, where)
        return cls(width=width, vocab=vocab, eps=eps, embedding_scale=scale, layers=tuple(layers),
                   logit_softcap=None if cap is None else float(cap), side_dim=side_dim, max_positions=max_pos,
                   eos_token_ids=eos_ids, raw=dict(obj))

    # ---- writing -------------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        out_layers = []
        for layer in self.layers:
            if layer.type == "mamba1":
                m: Dict[str, Any] = dict(layer.mixer)
            else:
                left = dict(layer.mixer["left"])
                left["mask"] = {"size": left.pop("chunk")}
                m = {"left": left, "left_scale": layer.mixer["left_scale"], "right": dict(layer.mixer["right"]),
                     "right_scale": layer.mixer["right_scale"]}
            out_layers.append({"type": layer.type, "mixer": m,
                               "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff, "limit": layer.limit}})
        d: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "width": self.width, "vocab": self.vocab,
                             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "layers": out_layers}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.side_dim is not None:
            d["token_side"] = {"dim": self.side_dim}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- the model this configuration describes ----------------------------------------------------
    def to_spec(self) -> ModelSpec:
        n_layers = len(self.layers)
        norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "tensor": "", "unit_offset": True}, "norm")
        specs = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "mamba1":
                mixer = PartSpec("mamba1", {"hidden_size": self.width, "inner": m["inner"], "state": m["state"],
                                            "dt_rank": m["dt_rank"], "conv": m["conv"]}, "mixer")
            else:
                lm, rm = m["left"], m["right"]
                left = {"kind": "talking_heads_attention", "prefix": "left.", "scale": m["left_scale"], "params": {
                    "hidden_size": self.width, "num_heads": lm["heads"], "num_kv_heads": lm["kv_heads"], "head_dim": lm["dim"],
                    "value_dim": lm["vdim"], "scale": lm["scale"], "chunk": lm["chunk"], "value_norm_eps": self.eps,
                    "distance_bias": True, "talk": True, "bias": True}}
                right = {"kind": "gated_delta_rule", "prefix": "right.", "scale": m["right_scale"], "params": {
                    "hidden_size": self.width, "heads": rm["heads"], "qk_heads": rm["kv_heads"], "head_dim": rm["dim"],
                    "value_dim": rm["vdim"], "conv": rm["conv"], "eps": self.eps}}
                mixer = PartSpec("parallel_mixers", {"branches": (left, right)}, "mixer")
            parts = {"mixer": mixer, "mixer_norm": norm}
            names = {"mixer": "mix.", "mixer_norm": "norm1"}
            if layer.ff is not None:
                parts["feed_forward"] = PartSpec("clamped_glu_mlp", {
                    "hidden_size": self.width, "intermediate_size": layer.ff, "limit": layer.limit, "alpha": 1.702,
                    "names": ("gate", "up", "down")}, "feed_forward")
                parts["feed_forward_norm"] = norm
                names.update({"feed_forward": "mlp.", "feed_forward_norm": "norm2"})
            if self.side_dim is not None:
                parts["token_input"] = PartSpec("token_side_input", {
                    "hidden_size": self.width, "dim": self.side_dim, "column": i * self.side_dim, "eps": self.eps,
                    "table": "token_side"}, "feed_forward")
                names["token_input"] = "side."
            specs.append(LayerSpec(f"l{i}.", PartSpec("prenorm_stream_residual"), parts, names))
        hooks = ()
        if self.side_dim is not None:
            hooks = (PartSpec("token_table_rows", {"rows": self.vocab, "width": n_layers * self.side_dim,
                                                   "tensor": "side.embed", "key": "token_side"}),)
        return ModelSpec(
            architecture=self.ARCHITECTURE, hidden_size=self.width, vocab_size=self.vocab,
            max_position_embeddings=self.max_positions, embedding_name="embed", layers=tuple(specs),
            run_order=tuple(RunEntry(layer=i, cache=i) for i in range(n_layers)),
            final_norm=PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "tensor": "", "unit_offset": True}),
            final_norm_prefix="final.norm", lm_head_name="head",
            position_encodings={"sinusoid": PartSpec("sinusoidal", {"width": self.width, "base": 10000.0,
                                                                    "input_scale": self.embedding_scale})},
            embedding_hooks=hooks,
            logit_hooks=() if self.logit_softcap is None else (PartSpec("logit_softcap", {"cap": self.logit_softcap}),),
            residual_dtype="float32", eos_token_ids=self.eos_token_ids)
