"""The Sitelorn configuration: a decoder whose config.json lists its layers one by one.

Keys read: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and ``layers``, a list whose entries give ``type``
(the mixer: ``lightning``, ``gla`` or ``attention``), ``mixer`` (that mixer's sizes and constants) and ``mlp`` (``kind``
``dense`` with ``ff``, or null for a layer without feed-forward).  Every layer is x += norm1(mixer(x)); x += norm2(ff(x))
with layer norms (weight and bias) on the sublayers' outputs; the model ends with a layer norm and the output matrix.

    lightning   linear attention with a constant decay per head (``decay``), silu on q, k and v, one RMS norm over all
                heads, a sigmoid gate                                          heads, dim, vdim, decay
    gla         linear attention with a decay per key channel and token, sigmoid(W2 W1 h + b) ** (1 / tau), q scaled by
                dim ** -0.5, an RMS norm per head with a shared weight, a silu gate        heads, dim, vdim, tau
    attention   grouped softmax attention with a short convolution on q, k and v, RMS norms over the whole q and k,
                rotation of the first rot.dims elements in pairs, a window, a sink and a gate per head; ``kv_from`` j:
                the layer has queries only and reads layer j's keys and values
                                         heads, kv_heads, dim, vdim, conv, rot.base, rot.dims, scale, mask.size, kv_from

Tensor names: ``embed``, ``head``, ``final.norm`` (+ ``.b``), and below ``l<i>.``: ``norm1``, ``norm2`` (+ ``.b``),
``mix.<name>``, ``mlp.gate / up / down``.  The configuration names no longest sequence: the engine's is given when the
configuration is read (``max_tokens``), nothing in the model depends on it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional, Tuple

from .specs import (ConfigError, ConvAttentionSpec, GLUSpec, LayerNormSpec, LinearAttentionSpec, ModelSpec, PairRotarySpec,
                    PostNormBlockSpec, RunEntry)

DEFAULT_MAX_POSITIONS = 32768
LOW_RANK_OF = "a1"


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _pos_int(d: dict, key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, found {v!r}")
    return int(v)


@dataclass(frozen=True)
class SitelornConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[dict, ...]           # the entries of config.json's ``layers``, checked
    max_positions: int = DEFAULT_MAX_POSITIONS
    model_type: str = "sitelorn"
    # The width of a gla layer's decay projection stands in no key: a tensor's shape gives it.  ``read_config`` therefore
    # hands this class the checkpoint's shapes; the width is kept as ``mixer.rank`` of the layer (``to_dict`` writes it).
    reads_shapes: ClassVar[bool] = True

    # ---- reading -------------------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict, max_tokens: Optional[int] = None, shapes: Optional[dict] = None) -> "SitelornConfig":
        layers = _need(cfg, "layers", "the configuration")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one entry")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            m = dict(_need(layer, "mixer", where))
            if kind == "lightning":
                heads = _pos_int(m, "heads", where); _pos_int(m, "dim", where); _pos_int(m, "vdim", where)
                decay = _need(m, "decay", where)
                if not isinstance(decay, (list, tuple)) or len(decay) != heads:
                    raise ConfigError(f"config.json: {where}.mixer.decay must list one decay for each of the {heads} heads")
            elif kind == "gla":
                _pos_int(m, "heads", where); _pos_int(m, "dim", where); _pos_int(m, "vdim", where)
                if float(_need(m, "tau", where)) <= 0:
                    raise ConfigError(f"config.json: {where}.mixer.tau must be positive")
                if "rank" not in m and shapes is not None and f"l{i}.mix.{LOW_RANK_OF}" in shapes:
                    m["rank"] = int(shapes[f"l{i}.mix.{LOW_RANK_OF}"][0])
            elif kind == "attention":
                heads, kv = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
                if heads % kv:
                    raise ConfigError(f"config.json: {where}: {heads} heads are no multiple of {kv} key/value heads")
                dim = _pos_int(m, "dim", where); _pos_int(m, "vdim", where); _pos_int(m, "conv", where)
                _pos_int(_need(m, "mask", where), "size", where + ".mask")
                rot = _need(m, "rot", where)
                dims = int(_need(rot, "dims", where + ".rot"))
                if dims < 0 or dims % 2 or dims > dim:
                    raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even and at most dim {dim}")
                if float(_need(rot, "base", where + ".rot")) <= 0:
                    raise ConfigError(f"config.json: {where}.rot.base must be positive")
                float(_need(m, "scale", where))
                src = m.get("kv_from")
                if src is not None:
                    if not isinstance(src, int) or not 0 <= src < i or layers[src].get("type") != "attention" \
                            or layers[src]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}.kv_from {src!r} must name an earlier attention layer with keys of its own")
                    other = layers[src]["mixer"]
                    if any(other.get(k) != m.get(k) for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"config.json: {where} borrows layer {src}'s keys and values but differs in their sizes")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is none of lightning, gla, attention")
            mlp = layer.get("mlp")
            if mlp is not None:
                if _need(mlp, "kind", where + ".mlp") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not built (dense is)")
                _pos_int(mlp, "ff", where + ".mlp")
            checked.append({"type": kind, "mixer": m, "mlp": None if mlp is None else dict(mlp)})
        return cls(vocab=_pos_int(cfg, "vocab", "the configuration"), width=_pos_int(cfg, "width", "the configuration"),
                   embedding_scale=float(_need(_need(cfg, "embedding", "the configuration"), "scale", "embedding")),
                   norm_eps=float(_need(_need(cfg, "norm", "the configuration"), "eps", "norm")),
                   layers=tuple(checked),
                   max_positions=int(max_tokens) if max_tokens else int(cfg.get("max_positions", DEFAULT_MAX_POSITIONS)))

    # what the entry points ask of any configuration
    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @property
    def tie_word_embeddings(self) -> bool:
        return False

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> dict:
        """config.json contents that read back to this configuration."""
        return {"architecture": "Sitelorn", "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "vocab": self.vocab, "width": self.width,
                "layers": [{"type": l["type"], "mixer": dict(l["mixer"]), "mlp": None if l["mlp"] is None else dict(l["mlp"])}
                           for l in self.layers]}

    # ---- the model as parts ------------------------------------------------------------------------------------------
    def _mixer_spec(self, kind: str, m: dict):
        if kind == "lightning":
            return LinearAttentionSpec(hidden_size=self.width, num_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                       norm_eps=self.norm_eps, qkv_act="silu", q_scale=1.0,
                                       decay=tuple(float(d) for d in m["decay"]), norm_per_head=False, gate_act="sigmoid")
        if kind == "gla":
            if "rank" not in m:
                raise ConfigError("a gla layer's decay projection has no width: config.json gives no mixer.rank and no "
                                  f"checkpoint was at hand to read the shape of mix.{LOW_RANK_OF} from")
            return LinearAttentionSpec(hidden_size=self.width, num_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                       norm_eps=self.norm_eps, qkv_act="none", q_scale=float(m["dim"]) ** -0.5, decay=None,
                                       decay_rank=int(m["rank"]), decay_tau=float(m["tau"]), norm_per_head=True, gate_act="silu")
        rot = m["rot"]
        return ConvAttentionSpec(hidden_size=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                 v_head_dim=m["vdim"], softmax_scale=float(m["scale"]), window=int(m["mask"]["size"]),
                                 conv_taps=int(m["conv"]), qk_norm=True, qk_norm_eps=self.norm_eps,
                                 position=PairRotarySpec(dims=int(rot["dims"]), base=float(rot["base"])) if int(rot["dims"]) else None,
                                 sink=True, head_gate=True, shares_kv=m.get("kv_from") is not None)

    def model_spec(self) -> ModelSpec:
        norm = LayerNormSpec(size=self.width, eps=self.norm_eps, weight_name="", bias_name=".b")
        blocks, order = [], []
        for i, layer in enumerate(self.layers):
            mlp = layer["mlp"]
            ffn = None if mlp is None else GLUSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]), act="gelu_tanh")
            blocks.append(PostNormBlockSpec(mixer=self._mixer_spec(layer["type"], layer["mixer"]), feed_forward=ffn,
                                            mixer_norm=norm, ffn_norm=None if ffn is None else norm))
            src = layer["mixer"].get("kv_from") if layer["type"] == "attention" else None
            order.append(RunEntry(layer=i, cache=i if src is None else src, writes_cache=src is None))
        return ModelSpec(architecture="sitelorn", hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
                         layers=tuple(blocks), order=tuple(order), final_norm=norm, embed_scale=self.embedding_scale,
                         logit_scale=1.0, tie_embeddings=False, embed_name="embed", lm_head_name="head",
                         final_norm_prefix="final.norm", layer_prefix="l{}.", eos_token_ids=())
