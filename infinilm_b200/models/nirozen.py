"""Nirozen described as data: a decoder of latent-attention layers with routed feed-forwards, of which a run of layers
may be passed through several times.

config.json: `vocab`, `width`, `norm.eps`, `embedding` (`scale`, `bigram`: `buckets`, `mul_prev`, `mul_cur`), `layers` (per
layer `type`, `mixer` with its sizes, `mlp` or null) and `loop` (`start`, `stop`, `times`: layers start..stop-1 run `times`
times in a row with the same weights, each pass with a cache of its own and a pass vector added to the residual stream
before its first layer). Tensors: `embed`, `bigram`, `loop.step`, `l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.*`,
`final.norm`, `head`. Block norms hold a deviation from one as their weight (y = x / rms * (1 + w)); positions enter only as a
sinusoid added to the embedding (base 10000).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..config.model_config import ConfigError, ModelConfig, take
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep

SINUSOID_BASE = 10000.0
MIXERS = ("latent_attention",)
FEED_FORWARDS = ("moe",)


def _obj(raw: Dict[str, Any], key: str, required: bool = True) -> Optional[Dict[str, Any]]:
    v = raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: key '{key}' must be an object")
    return v


@dataclass
class NirozenConfig(ModelConfig):
    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    bigram: Optional[Dict[str, int]] = None       # buckets, mul_prev, mul_cur
    layers: List[Dict[str, Any]] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0

    @classmethod
    def from_json(cls, raw: Dict[str, Any]) -> "NirozenConfig":
        raw = dict(raw)
        emb = _obj(raw, "embedding")
        big = _obj(emb, "bigram", required=False)
        bigram = None if big is None else {k: take(big, k, int) for k in ("buckets", "mul_prev", "mul_cur")}
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out_layers = []
        for i, L in enumerate(layers):
            typ = take(L, "type", str)
            if typ not in MIXERS:
                raise ConfigError(f"config.json: layer {i} has mixer type {typ!r} (known: {', '.join(MIXERS)})")
            m = _obj(L, "mixer")
            mixer = {k: take(m, k, int) for k in ("heads", "dim", "vdim", "q_rank", "kv_rank")}
            mixer["scale"] = take(m, "scale", float)
            mlp = None
            f = _obj(L, "mlp", required=False)
            if f is not None:
                kind = take(f, "kind", str)
                if kind not in FEED_FORWARDS:
                    raise ConfigError(f"config.json: layer {i} has feed-forward kind {kind!r} (known: {', '.join(FEED_FORWARDS)})")
                router, shared = _obj(f, "router"), _obj(f, "shared", required=False)
                mlp = {"kind": kind, "experts": take(router, "experts", int), "top": take(router, "top", int),
                       "ff": take(_obj(f, "expert"), "ff", int), "shared_ff": None if shared is None else take(shared, "ff", int)}
            out_layers.append({"type": typ, "mixer": mixer, "mlp": mlp})
        loop = _obj(raw, "loop", required=False)
        start = stop = times = 0
        if loop is not None:
            start, stop, times = take(loop, "start", int), take(loop, "stop", int), take(loop, "times", int)
            if not (0 <= start <= stop <= len(out_layers)) or times < 1:
                raise ConfigError(f"config.json: loop {start}..{stop} x {times} does not fit {len(out_layers)} layers")
        cfg = cls(architecture="Nirozen", model_type="nirozen", vocab_size=take(raw, "vocab", int), hidden_size=take(raw, "width", int),
                  max_position_embeddings=1 << 30, torch_dtype="bfloat16", eos_token_ids=[], raw=raw,
                  norm_eps=take(_obj(raw, "norm"), "eps", float), embedding_scale=take(emb, "scale", float, 1.0), bigram=bigram,
                  layers=out_layers, loop_start=start, loop_stop=stop, loop_times=times)
        if cfg.vocab_size <= 0 or cfg.hidden_size <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        return cfg

    @property
    def looped(self) -> bool:
        return self.loop_times > 0 and self.loop_stop > self.loop_start


def run_order(cfg: NirozenConfig) -> List[RunStep]:
    n = len(cfg.layers)
    if not cfg.looped:
        return [RunStep(i) for i in range(n)]
    a, b = cfg.loop_start, cfg.loop_stop
    order = [RunStep(i) for i in range(a)]
    for t in range(cfg.loop_times):                 # every pass keeps a cache of its own; its vector comes before its first layer
        order += [RunStep(i, add_row=t if i == a else None) for i in range(a, b)]
    return order + [RunStep(i) for i in range(b, n)]


def describe(cfg: NirozenConfig) -> ModelSpec:
    W, eps = cfg.hidden_size, cfg.norm_eps

    def block_norm(prefix: str, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": eps, "weight_offset": 1.0, "name": name}, prefix)
    layers = []
    for i, L in enumerate(cfg.layers):
        m, f = L["mixer"], L["mlp"]
        mixer = PartSpec("latent_attention", {"hidden": W, "n_heads": m["heads"], "qk_dim": m["dim"], "v_dim": m["vdim"],
                                              "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps,
                                              "sink": True, "gate": True}, f"l{i}.mix")
        ffn = ffn_norm = None
        if f is not None:
            ffn = PartSpec("routed_experts", {"hidden": W, "n_experts": f["experts"], "top": f["top"], "expert_ff": f["ff"],
                                              "shared_ff": f["shared_ff"], "router_bias": True}, f"l{i}.mlp")
            ffn_norm = block_norm(f"l{i}", "norm2")
        layers.append(LayerSpec("prenorm_residual", block_norm(f"l{i}", "norm1"), mixer, ffn_norm, ffn, {"residual_scale": 1.0}))
    pair = None if cfg.bigram is None else dict(cfg.bigram, name="bigram")
    return ModelSpec(
        embedding=PartSpec("pair_position_embedding", {"vocab": cfg.vocab_size, "hidden": W, "scale": cfg.embedding_scale, "name": "embed",
                                                       "pair": pair, "sinusoid_base": SINUSOID_BASE}, ""),
        layers=layers, order=run_order(cfg),
        final_norm=block_norm("final", "norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": W, "scale": 1.0, "tied_to": None, "name": "head"}, ""),
        pass_vectors=PartSpec("row_table", {"rows": cfg.loop_times, "hidden": W, "name": "step"}, "loop") if cfg.looped else None)


register_architecture(["Nirozen", "nirozen"], NirozenConfig, describe)
