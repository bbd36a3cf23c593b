"""The Vunelix configuration: a decoder whose config.json lists its layers one by one and may run a span of them
several times.

Keys read: ``vocab``, ``width``, ``norm.eps``, ``logit_softcap``, ``loop`` (``start``, ``stop``, ``times``; absent or null:
every layer runs once) and ``layers``, a list whose entries give ``type`` (the mixer), ``mixer`` (its sizes and constants)
and ``mlp`` (the feed-forward, or null for none).  Every layer is x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x)))
with RMS norms; the model ends with an RMS norm, the embedding table as the output matrix, and c tanh(logits / c).

    latent_attention   attention over one latent vector and one shared rotated key part per position; rotation in pairs
                       with stretched frequencies; a sigmoid gate on the heads' outputs
                                heads, dim, rot_dim, vdim, kv_rank, scale, rot.base, rot.dims, rot.scaling.{factor, original, fast, slow}
    mamba1             a selective scan behind a short convolution                        inner, state, dt_rank, conv
    mlp.kind dense     down(relu(gate h) * up h)                                                                 ff
    mlp.kind moe       router.experts gated silu units of expert.ff, router.top a row by sigmoid scores that multiply the
                       unit's input; shared.ff: one more unit that every row passes

Layers ``loop.start`` .. ``loop.stop`` - 1 run ``loop.times`` times in a row with the same weights, each pass with a cache
and state of its own; before the first layer of every pass x <- loop.in [x | embedding output] + loop.step[pass].

Tensor names: ``embed``, ``final.norm``, ``loop.in``, ``loop.step`` and below ``l<i>.``: ``norm1``, ``norm1b``, ``norm2``,
``norm2b``, ``mix.<name>``, ``mlp.gate / up / down``, ``mlp.router``, ``mlp.e<j>.gate / up / down``, ``mlp.shared.gate / up /
down``.  The configuration names no longest sequence: the engine's is given when the configuration is read.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .specs import (ConfigError, FrequencyRampSpec, GLUSpec, LatentAttentionSpec, ModelSpec, PairRotarySpec, ReinjectSpec,
                    RMSNormSpec, RoutedExpertsSpec, RunEntry, SandwichBlockSpec, SelectiveScanSpec)

DEFAULT_MAX_POSITIONS = 32768


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _pos_int(d, key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, found {v!r}")
    return int(v)


def _pos_float(d, key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not v > 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive number, found {v!r}")
    return float(v)


@dataclass(frozen=True)
class VunelixConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float               # 0: none
    layers: Tuple[dict, ...]           # the entries of config.json's ``layers``, checked
    loop: Optional[Tuple[int, int, int]] = None        # (start, stop, times)
    max_positions: int = DEFAULT_MAX_POSITIONS
    model_type: str = "vunelix"

    # ---- reading -------------------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict, max_tokens: Optional[int] = None) -> "VunelixConfig":
        layers = _need(cfg, "layers", "the configuration")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one entry")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            m = dict(_need(layer, "mixer", where))
            if kind == "latent_attention":
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    _pos_int(m, key, where + ".mixer")
                _pos_float(m, "scale", where + ".mixer")
                rot = _need(m, "rot", where + ".mixer")
                dims = _pos_int(rot, "dims", where + ".mixer.rot")
                if dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims {dims} must be even and at most rot_dim {m['rot_dim']}")
                _pos_float(rot, "base", where + ".mixer.rot")
                if rot.get("scaling") is not None:
                    for key in ("factor", "original", "fast", "slow"):
                        _pos_float(rot["scaling"], key, where + ".mixer.rot.scaling")
            elif kind == "mamba1":
                for key in ("inner", "state", "dt_rank", "conv"):
                    _pos_int(m, key, where + ".mixer")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is none of latent_attention, mamba1")
            mlp = layer.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                form = _need(mlp, "kind", where + ".mlp")
                if form == "dense":
                    _pos_int(mlp, "ff", where + ".mlp")
                elif form == "moe":
                    router = _need(mlp, "router", where + ".mlp")
                    n, top = _pos_int(router, "experts", where + ".mlp.router"), _pos_int(router, "top", where + ".mlp.router")
                    if top > n:
                        raise ConfigError(f"config.json: {where}.mlp.router takes {top} of {n} experts")
                    _pos_int(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert")
                    if mlp.get("shared") is not None:
                        _pos_int(mlp["shared"], "ff", where + ".mlp.shared")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {form!r} is none of dense, moe")
            checked.append({"type": kind, "mixer": m, "mlp": mlp})
        loop = cfg.get("loop")
        if loop is not None:
            start, stop = int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop"))
            times = _pos_int(loop, "times", "loop")
            if not 0 <= start < stop <= len(checked):
                raise ConfigError(f"config.json: loop {start} .. {stop} does not lie within the {len(checked)} layers")
            loop = (start, stop, times)
        cap = cfg.get("logit_softcap")
        return cls(vocab=_pos_int(cfg, "vocab", "the configuration"), width=_pos_int(cfg, "width", "the configuration"),
                   norm_eps=float(_need(_need(cfg, "norm", "the configuration"), "eps", "norm")),
                   logit_softcap=float(cap) if cap else 0.0, layers=tuple(checked), loop=loop,
                   max_positions=int(max_tokens) if max_tokens else int(cfg.get("max_positions", DEFAULT_MAX_POSITIONS)))

    # what the entry points ask of any configuration
    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @property
    def tie_word_embeddings(self) -> bool:
        return True

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> dict:
        """config.json contents that read back to this configuration."""
        out = {"architecture": "Vunelix", "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width,
               "logit_softcap": self.logit_softcap or None,
               "layers": [{"type": l["type"], "mixer": dict(l["mixer"]), "mlp": None if l["mlp"] is None else dict(l["mlp"])}
                          for l in self.layers]}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    # ---- the model as parts ------------------------------------------------------------------------------------------
    def _mixer_spec(self, kind: str, m: dict):
        if kind == "mamba1":
            return SelectiveScanSpec(hidden_size=self.width, inner=int(m["inner"]), state_size=int(m["state"]),
                                     dt_rank=int(m["dt_rank"]), conv_taps=int(m["conv"]))
        rot, scaling = m["rot"], None
        if rot.get("scaling") is not None:
            s = rot["scaling"]
            scaling = FrequencyRampSpec(factor=float(s["factor"]), original=float(s["original"]), fast=float(s["fast"]),
                                        slow=float(s["slow"]), magnitude_slope=0.1)
        return LatentAttentionSpec(hidden_size=self.width, num_heads=int(m["heads"]), head_dim=int(m["dim"]), rot_dim=int(m["rot_dim"]),
                                   v_head_dim=int(m["vdim"]), latent_size=int(m["kv_rank"]), softmax_scale=float(m["scale"]),
                                   norm_eps=self.norm_eps, output_gate=True,
                                   position=PairRotarySpec(dims=int(rot["dims"]), base=float(rot["base"]), scaling=scaling))

    def _ffn_spec(self, mlp: Optional[dict]):
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return GLUSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]), act="relu")
        shared = mlp.get("shared")
        return RoutedExpertsSpec(hidden_size=self.width, num_experts=int(mlp["router"]["experts"]), top=int(mlp["router"]["top"]),
                                 expert_size=int(mlp["expert"]["ff"]), act="silu", scale_input=True,
                                 shared=None if shared is None else GLUSpec(hidden_size=self.width, intermediate_size=int(shared["ff"]), act="silu"))

    def run_order(self):
        """(layer, pass number or None, whether the pass starts here) for every layer run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None, False) for i in range(n)]
        start, stop, times = self.loop
        runs = [(i, None, False) for i in range(start)]
        for t in range(times):
            runs += [(i, t, i == start) for i in range(start, stop)]
        return runs + [(i, None, False) for i in range(stop, n)]

    def model_spec(self) -> ModelSpec:
        norm = RMSNormSpec(size=self.width, eps=self.norm_eps, weight_name="")
        blocks = []
        for layer in self.layers:
            ffn = self._ffn_spec(layer["mlp"])
            blocks.append(SandwichBlockSpec(mixer=self._mixer_spec(layer["type"], layer["mixer"]), feed_forward=ffn,
                                            mixer_norm=norm, mixer_post_norm=norm, ffn_norm=None if ffn is None else norm,
                                            ffn_post_norm=None if ffn is None else norm))
        order = []
        for run, (i, t, opens) in enumerate(self.run_order()):       # every run of a layer has a cache and state of its own
            before = ReinjectSpec(hidden_size=self.width, steps=self.loop[2], step_index=t) if opens else None
            order.append(RunEntry(layer=i, cache=run, writes_cache=True, before=before))
        return ModelSpec(architecture="vunelix", hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
                         layers=tuple(blocks), order=tuple(order), final_norm=norm, embed_scale=1.0, logit_scale=1.0,
                         logit_softcap=self.logit_softcap, tie_embeddings=True, embed_name="embed", lm_head_name="head",
                         final_norm_prefix="final.norm", layer_prefix="l{}.", eos_token_ids=())
