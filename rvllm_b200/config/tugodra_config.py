"""Configuration of the Tugodra decoder: layers listed one by one, each with one of three mixers (grouped-query attention
inside a sliding window, whose queries and keys are rotated and then made unit-RMS vectors and whose heads are gated,
optionally reading the keys and values that an earlier layer cached; latent attention with a sink in the softmax; an
mLSTM matrix memory) and, optionally, a routed mixture of experts with a gated shared expert.  Every sublayer has a
Dynamic-Tanh norm in front of it and one on what it returns; the residual stream is float32; the embedding is scaled;
the LM head is a tensor of its own.

config.json keys (all sizes and every constant that may differ between models are read, none is assumed):

    architecture            "Tugodra"
    width, vocab            model width and vocabulary size
    norm.eps                eps of the unit-RMS norms inside the mixers (the layer norms use none)
    embedding.scale         factor on the embedded tokens
    layers[i].type          "attention" | "latent_attention" | "mlstm"
    layers[i].mixer         attention: heads, kv_heads, dim, vdim, scale, mask.size (absent: every earlier key), rot.dims,
                                       rot.base, kv_from (optional: the earlier attention layer whose keys and values are read)
                            latent_attention: heads, dim, rot_dim, vdim, kv_rank, scale, rot.dims, rot.base
                            mlstm: heads, dim, vdim, gate_cap
    layers[i].mlp           null | {"kind": "moe", "expert": {"ff": n}, "router": {"experts": E, "top": k,
                                    "groups": {"count": c, "keep": m} (optional)}, "shared": {"ff": m} | null}
    max_positions           optional: the longest sequence the rotation tables are ever built for

Tensor names: embed, head, final.norm (+ .b, .alpha), l<i>.norm1 / norm1b / norm2 / norm2b (+ .b, .alpha),
l<i>.mix.{q,k,v,g,o} | {q,dkv,dkv.norm,uk,uv,sink,o} | {q,k,v,g,o,norm,i,i.b,f,f.b},
l<i>.mlp.{router, correction, e<j>.up, e<j>.down, shared.up, shared.down, shared.sg}.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

DEFAULT_MAX_POSITIONS = 1 << 17       # the design sets no limit; the engine's tables are built for max_model_len
MIXERS = ("attention", "latent_attention", "mlstm")


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@dataclass(frozen=True)
class TugodraLayer:
    type: str                              # one of MIXERS
    mixer: Dict[str, Any]                  # the mixer's sizes and constants, flat (rot_dims, rot_base, window, kv_from, ...)
    mlp: Optional[Dict[str, Any]]          # None | {ff, experts, top, groups, keep, shared_ff | None}


@dataclass(frozen=True)
class TugodraConfig:
    width: int
    vocab: int
    eps: float
    embedding_scale: float
    layers: Tuple[TugodraLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    ARCHITECTURE = "Tugodra"

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
    def from_dict(cls, obj: Dict[str, Any], where: str = "config.json") -> "TugodraConfig":
        p: List[str] = []

        def integer(d, key, what, minimum=1):
            v = d.get(key) if isinstance(d, dict) else None
            if not _is_int(v) or v < minimum:
                p.append(f"{what}`{key}` must be an integer >= {minimum}, got {v!r}")
                return max(minimum, 1)
            return v

        def number(d, key, what):
            v = d.get(key) if isinstance(d, dict) else None
            if not _is_num(v) or not v > 0:
                p.append(f"{what}`{key}` must be a number > 0, got {v!r}")
                return 1.0
            return float(v)

        def rotation(m, at, inside, what):
            rot = m.get("rot")
            dims = integer(rot, "dims", at + "rot: ", minimum=2)
            base = number(rot, "base", at + "rot: ")
            if dims % 2 or dims > inside:
                p.append(at + f"`rot.dims` must be even and at most {what} = {inside}, got {dims}")
            return dims, base

        width = integer(obj, "width", "")
        vocab = integer(obj, "vocab", "")
        eps = number(obj.get("norm"), "eps", "norm: ")
        scale = number(obj.get("embedding"), "scale", "embedding: ")
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(p + ["`layers` must be a non-empty list"], where)
        layers: List[TugodraLayer] = []
        for i, e in enumerate(raw_layers):
            at = f"layers[{i}]: "
            if not isinstance(e, dict):
                p.append(at + "must be an object")
                continue
            kind, m = e.get("type"), e.get("mixer")
            if kind not in MIXERS:
                p.append(at + f"`type` = {kind!r} is not known ({', '.join(MIXERS)})")
                kind = "mlstm"
            if not isinstance(m, dict):
                p.append(at + "`mixer` must be an object")
                m = {}
            if kind == "attention":
                mixer: Dict[str, Any] = {key: integer(m, key, at) for key in ("heads", "kv_heads", "dim", "vdim")}
                mixer["scale"] = number(m, "scale", at)
                mixer["rot_dims"], mixer["rot_base"] = rotation(m, at, mixer["dim"], "dim")
                if mixer["heads"] % mixer["kv_heads"]:
                    p.append(at + f"{mixer['heads']} query heads cannot share {mixer['kv_heads']} key/value heads")
                mask = m.get("mask")
                mixer["window"] = None if mask is None else integer(mask, "size", at + "mask: ")
                src = m.get("kv_from")
                mixer["kv_from"] = None
                if src is not None:
                    if not _is_int(src) or not 0 <= src < i:
                        p.append(at + f"`kv_from` must name an earlier layer, got {src!r}")
                    else:
                        other = layers[src] if src < len(layers) else None
                        if other is None or other.type != "attention" or other.mixer.get("kv_from") is not None:
                            p.append(at + f"`kv_from` = {src}: that layer is no attention layer with keys and values of its own")
                        elif any(other.mixer[key] != mixer[key] for key in ("heads", "kv_heads", "dim", "vdim", "rot_dims", "rot_base")):
                            p.append(at + f"`kv_from` = {src}: head counts, head sizes and rotation must equal that layer's")
                        else:
                            mixer["kv_from"] = src
            elif kind == "latent_attention":
                mixer = {key: integer(m, key, at) for key in ("heads", "dim", "vdim", "kv_rank")}
                mixer["rot_dim"] = integer(m, "rot_dim", at, minimum=2)
                mixer["scale"] = number(m, "scale", at)
                mixer["rot_dims"], mixer["rot_base"] = rotation(m, at, mixer["rot_dim"], "rot_dim")
            else:
                mixer = {key: integer(m, key, at) for key in ("heads", "dim", "vdim")}
                mixer["gate_cap"] = number(m, "gate_cap", at)
            raw_mlp, mlp = e.get("mlp"), None
            if raw_mlp is not None:
                if not isinstance(raw_mlp, dict) or raw_mlp.get("kind") != "moe":
                    p.append(at + f"`mlp` must be null or an object of kind \"moe\", got {raw_mlp!r}")
                else:
                    router = raw_mlp.get("router")
                    mlp = {"ff": integer(raw_mlp.get("expert"), "ff", at + "mlp.expert: "),
                           "experts": integer(router, "experts", at + "mlp.router: "),
                           "top": integer(router, "top", at + "mlp.router: "), "groups": 1, "keep": 1, "shared_ff": None}
                    groups = router.get("groups") if isinstance(router, dict) else None
                    if groups is not None:
                        mlp["groups"] = integer(groups, "count", at + "mlp.router.groups: ")
                        mlp["keep"] = integer(groups, "keep", at + "mlp.router.groups: ")
                    if mlp["experts"] % mlp["groups"] or mlp["keep"] > mlp["groups"]:
                        p.append(at + f"mlp.router: {mlp['experts']} experts in {mlp['groups']} equal groups of which {mlp['keep']} are kept")
                    elif mlp["top"] > mlp["keep"] * (mlp["experts"] // mlp["groups"]):
                        p.append(at + f"mlp.router: `top` {mlp['top']} exceeds the experts of the {mlp['keep']} kept groups")
                    if raw_mlp.get("shared") is not None:
                        mlp["shared_ff"] = integer(raw_mlp.get("shared"), "ff", at + "mlp.shared: ")
            layers.append(TugodraLayer(kind, mixer, mlp))
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
        return cls(width=width, vocab=vocab, eps=eps, embedding_scale=scale, layers=tuple(layers), max_positions=max_pos,
                   eos_token_ids=eos_ids, raw=dict(obj))

    # ---- writing -------------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        out_layers = []
        for layer in self.layers:
            m = dict(layer.mixer)
            if layer.type != "mlstm":
                m["rot"] = {"dims": m.pop("rot_dims"), "base": m.pop("rot_base")}
            if layer.type == "attention":
                window, src = m.pop("window"), m.pop("kv_from")
                if window is not None:
                    m["mask"] = {"size": window}
                if src is not None:
                    m["kv_from"] = src
            mlp = None
            if layer.mlp is not None:
                f = layer.mlp
                mlp = {"kind": "moe", "expert": {"ff": f["ff"]},
                       "router": {"experts": f["experts"], "top": f["top"], "groups": {"count": f["groups"], "keep": f["keep"]}},
                       "shared": None if f["shared_ff"] is None else {"ff": f["shared_ff"]}}
            out_layers.append({"type": layer.type, "mixer": m, "mlp": mlp})
        d: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "width": self.width, "vocab": self.vocab,
                             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "layers": out_layers}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- the model this configuration describes ----------------------------------------------------
    def kept_window(self, i: int) -> Optional[int]:
        """How many keys the cache of attention layer `i` must keep: the widest window among the layer itself and the
        layers that read its keys and values (None: all of them)."""
        windows = [self.layers[i].mixer["window"]]
        windows += [l.mixer["window"] for l in self.layers if l.type == "attention" and l.mixer["kv_from"] == i]
        return None if any(w is None for w in windows) else max(windows)

    def to_spec(self) -> ModelSpec:
        rotations: Dict[Tuple[int, float], str] = {}
        norm = PartSpec("dynamic_tanh", {"size": self.width, "tensor": ""}, "norm")
        specs, run_order = [], []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            position = None
            if layer.type != "mlstm":
                position = rotations.setdefault((m["rot_dims"], m["rot_base"]), f"rot{len(rotations)}")
            cache = i
            if layer.type == "attention":
                owner = i if m["kv_from"] is None else m["kv_from"]
                cache = owner
                mixer = PartSpec("unit_qk_attention", {
                    "hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                    "value_dim": m["vdim"], "scale": m["scale"], "eps": self.eps, "window": m["window"],
                    "kept_window": self.kept_window(owner), "gate": True, "pairs": "neighbours", "own_kv": m["kv_from"] is None,
                    "position": position}, "mixer")
            elif layer.type == "latent_attention":
                mixer = PartSpec("latent_attention", {
                    "hidden_size": self.width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                    "value_dim": m["vdim"], "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": self.eps, "gate": False,
                    "sink": True, "pairs": "halves", "position": position, "suffix": ""}, "mixer")
            else:
                mixer = PartSpec("mlstm", {"hidden_size": self.width, "heads": m["heads"], "head_dim": m["dim"],
                                           "value_dim": m["vdim"], "gate_cap": m["gate_cap"], "eps": self.eps}, "mixer")
            parts = {"mixer": mixer, "mixer_norm": norm, "mixer_out_norm": norm}
            names = {"mixer": "mix.", "mixer_norm": "norm1", "mixer_out_norm": "norm1b"}
            if layer.mlp is not None:
                f = layer.mlp
                parts["feed_forward"] = PartSpec("routed_moe", {
                    "hidden_size": self.width, "intermediate_size": f["ff"], "experts": f["experts"], "top": f["top"],
                    "groups": f["groups"], "keep_groups": f["keep"], "shared_intermediate_size": f["shared_ff"],
                    "activation": "relu2"}, "feed_forward")
                parts.update({"feed_forward_norm": norm, "feed_forward_out_norm": norm})
                names.update({"feed_forward": "mlp.", "feed_forward_norm": "norm2", "feed_forward_out_norm": "norm2b"})
            specs.append(LayerSpec(f"l{i}.", PartSpec("sandwich_norm_residual"), parts, names))
            run_order.append(RunEntry(layer=i, cache=cache, writes_cache=cache == i))
        return ModelSpec(
            architecture=self.ARCHITECTURE, hidden_size=self.width, vocab_size=self.vocab,
            max_position_embeddings=self.max_positions, embedding_name="embed", layers=tuple(specs), run_order=tuple(run_order),
            final_norm=PartSpec("dynamic_tanh", {"size": self.width, "tensor": ""}), final_norm_prefix="final.norm",
            lm_head_name="head",
            position_encodings={key: PartSpec("rotary", {"head_dim": dims, "theta": base, "rotary_dim": dims})
                                for (dims, base), key in rotations.items()},
            embedding_hooks=(PartSpec("embedding_scale", {"scale": self.embedding_scale}),),
            residual_dtype="float32", eos_token_ids=self.eos_token_ids,
            # steps of this design at real layer widths stopped answering, rarely, with programmatic dependent launch on
            # and never with it off; one cause was found and removed (a kernel that signalled its dependents before it
            # held its tensor memory), another may remain: its kernels follow one another strictly
            programmatic_launch=False)
