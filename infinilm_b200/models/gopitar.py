"""Gopitar described as data: a decoder whose layers mix tokens either by two mixers side by side - softmax attention over
a sliding window, its queries, keys and values passed through a short convolution, beside a decayed linear attention - or
by the gated delta rule; gated feed-forwards with the tanh form of GELU; a run of layers that may be passed through several
times, the embedding's output added again before every later pass; logits under a soft cap.

config.json: `vocab`, `width`, `norm.eps`, `embedding.scale`, `logit_softcap`, `layers` (per layer `type` - "parallel" or
"delta" -, `mixer` with its sizes and constants, `mlp` - `kind` "dense" with `ff` - or null) and `loop` (`start`, `stop`,
`times`: layers start..stop-1 run `times` times in a row with the same weights, each pass with caches and states of its own).
Tensors: `embed`, `l<i>.norm1|norm2`, `l<i>.mix.*` (`left.*` and `right.*` in a parallel layer), `l<i>.mlp.gate|up|down`,
`final.norm`, `head`. The constant of the design that is not in config.json: 1e-6 inside the root that makes the delta rule's
queries and keys unit vectors.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..config.model_config import ConfigError, ModelConfig, take
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep

UNIT_EPS = 1e-6
MIXERS = ("parallel", "delta")
FEED_FORWARDS = ("dense",)


def _obj(raw: Dict[str, Any], key: str, required: bool = True) -> Optional[Dict[str, Any]]:
    v = raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: key '{key}' must be an object")
    return v


def _softmax_branch(m: Dict[str, Any]) -> Dict[str, Any]:
    out = {k: take(m, k, int) for k in ("heads", "kv_heads", "dim", "vdim")}
    out["conv"] = take(m, "conv", int, None)
    out["scale"] = take(m, "scale", float)
    mask, rot = _obj(m, "mask", required=False), _obj(m, "rot", required=False)
    out["window"] = None if mask is None else take(mask, "size", int)
    out["rot_dims"] = 0 if rot is None else take(rot, "dims", int)
    out["rot_base"] = 10000.0 if rot is None else take(rot, "base", float)
    return out


def _linear_branch(m: Dict[str, Any]) -> Dict[str, Any]:
    out = {k: take(m, k, int) for k in ("heads", "dim", "vdim")}
    decay = m.get("decay")
    if not isinstance(decay, list) or len(decay) != out["heads"] or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
        raise ConfigError("config.json: 'decay' must list one number per head")
    out["decay"] = [float(x) for x in decay]
    return out


@dataclass
class GopitarConfig(ModelConfig):
    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    logit_softcap: Optional[float] = None
    layers: List[Dict[str, Any]] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0

    @classmethod
    def from_json(cls, raw: Dict[str, Any]) -> "GopitarConfig":
        raw = dict(raw)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out_layers = []
        for i, L in enumerate(layers):
            typ = take(L, "type", str)
            if typ not in MIXERS:
                raise ConfigError(f"config.json: layer {i} has mixer type {typ!r} (known: {', '.join(MIXERS)})")
            m = _obj(L, "mixer")
            if typ == "parallel":
                mixer = {"left": _softmax_branch(_obj(m, "left")), "right": _linear_branch(_obj(m, "right")),
                         "left_scale": take(m, "left_scale", float, 1.0), "right_scale": take(m, "right_scale", float, 1.0)}
            else:
                mixer = {k: take(m, k, int) for k in ("heads", "kv_heads", "dim", "vdim")}
                mixer["conv"] = take(m, "conv", int, None)
            mlp = None
            f = _obj(L, "mlp", required=False)
            if f is not None:
                kind = take(f, "kind", str)
                if kind not in FEED_FORWARDS:
                    raise ConfigError(f"config.json: layer {i} has feed-forward kind {kind!r} (known: {', '.join(FEED_FORWARDS)})")
                mlp = {"kind": kind, "ff": take(f, "ff", int)}
            out_layers.append({"type": typ, "mixer": mixer, "mlp": mlp})
        loop = _obj(raw, "loop", required=False)
        start = stop = times = 0
        if loop is not None:
            start, stop, times = take(loop, "start", int), take(loop, "stop", int), take(loop, "times", int)
            if not (0 <= start <= stop <= len(out_layers)) or times < 1:
                raise ConfigError(f"config.json: loop {start}..{stop} x {times} does not fit {len(out_layers)} layers")
        cap = take(raw, "logit_softcap", float, None)
        cfg = cls(architecture="Gopitar", model_type="gopitar", vocab_size=take(raw, "vocab", int), hidden_size=take(raw, "width", int),
                  max_position_embeddings=1 << 30, torch_dtype="bfloat16", eos_token_ids=[], raw=raw,
                  norm_eps=take(_obj(raw, "norm"), "eps", float), embedding_scale=take(_obj(raw, "embedding", required=False) or {}, "scale", float, 1.0),
                  logit_softcap=cap if cap else None, layers=out_layers, loop_start=start, loop_stop=stop, loop_times=times)
        if cfg.vocab_size <= 0 or cfg.hidden_size <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        return cfg

    @property
    def looped(self) -> bool:
        return self.loop_times > 1 and self.loop_stop > self.loop_start


def run_order(cfg: GopitarConfig) -> List[RunStep]:
    n = len(cfg.layers)
    if not cfg.looped:
        return [RunStep(i) for i in range(n)]
    a, b = cfg.loop_start, cfg.loop_stop
    order = [RunStep(i) for i in range(a)]
    for t in range(cfg.loop_times):                 # every pass has caches and states of its own; later passes take the input in again
        order += [RunStep(i, add_embedding=(t > 0 and i == a)) for i in range(a, b)]
    return order + [RunStep(i) for i in range(b, n)]


def describe(cfg: GopitarConfig) -> ModelSpec:
    W, eps = cfg.hidden_size, cfg.norm_eps

    def norm(prefix: str, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": eps, "name": name}, prefix)
    layers = []
    for i, L in enumerate(cfg.layers):
        m, f = L["mixer"], L["mlp"]
        if L["type"] == "parallel":
            l, r = m["left"], m["right"]
            left = PartSpec("conv_gated_attention", {
                "hidden": W, "n_heads": l["heads"], "n_kv_heads": l["kv_heads"], "qk_dim": l["dim"], "v_dim": l["vdim"], "scale": l["scale"],
                "window": l["window"], "conv_taps": l["conv"], "qkv_bias": True, "out_bias": True, "head_gate": True,
                "position": PartSpec("rope", {"rot_dim": l["rot_dims"], "theta": l["rot_base"]}) if l["rot_dims"] else None}, "left")
            right = PartSpec("decay_linear_attention", {"hidden": W, "n_heads": r["heads"], "qk_dim": r["dim"], "v_dim": r["vdim"],
                                                        "decay": r["decay"], "eps": eps}, "right")
            mixer = PartSpec("parallel", {"branches": [(left, m["left_scale"]), (right, m["right_scale"])]}, f"l{i}.mix")
        else:
            mixer = PartSpec("gated_delta_rule", {"hidden": W, "n_heads": m["heads"], "n_qk_heads": m["kv_heads"], "qk_dim": m["dim"],
                                                  "v_dim": m["vdim"], "conv_taps": m["conv"], "eps": eps, "unit_eps": UNIT_EPS}, f"l{i}.mix")
        ffn = ffn_norm = None
        if f is not None:
            ffn = PartSpec("swiglu", {"hidden": W, "intermediate": f["ff"], "activation": "gelu_tanh",
                                      "names": {"gate": "gate", "up": "up", "down": "down"}}, f"l{i}.mlp")
            ffn_norm = norm(f"l{i}", "norm2")
        layers.append(LayerSpec("prenorm_residual", norm(f"l{i}", "norm1"), mixer, ffn_norm, ffn, {"residual_scale": 1.0}))
    return ModelSpec(
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": W, "scale": cfg.embedding_scale, "name": "embed", "exact": True}, ""),
        layers=layers, order=run_order(cfg), final_norm=norm("final", "norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": W, "scale": 1.0, "tied_to": None, "name": "head",
                                      "softcap": cfg.logit_softcap}, ""))


register_architecture(["Gopitar", "gopitar"], GopitarConfig, describe)
