"""Ronelorn: a decoder-only language model whose layers mix three kinds of sequence mixer — grouped-query attention with a sliding
window and POOLED BLOCKS before it (per-head query / key norm, rotated values, tanh-capped scores), grouped-query attention with a
sliding window that KEEPS THE FIRST TOKENS (whole-projection query / key norm, a softmax sink) and a minGRU recurrence — with a dense
squared-relu feed-forward or none.  Pre-norm residual layers with a residual multiplier, norm gains stored around zero, a scaled
embedding, and layers that may run on an earlier layer's weights.  This module only reads the checkpoint's config.json into the
generic layer list of leopard_b200/seqlm.py and names its tensors; the mechanisms themselves are the shared ones.

config.json keys: architecture, vocab, width, norm.eps, residual_mult, embedding.scale, layers[] = {type: "attention" | "attention_2" |
"mingru", mixer: {...}, mlp: null | {kind: "dense", ff}, weights_of: j (optional)}.
  attention / attention_2 mixer: heads, kv_heads, dim, vdim, scale, softcap (optional), rot.{base, dims, scaling.factor (optional)},
  mask.{size, pool (attention) | keep_first (attention_2)}.   mingru mixer: width.
Tensor names: embed, head, final.norm, and per layer l<i>.{norm1, norm2, mix.{q, k, v, o, q.norm, k.norm | z, z.b, x, x.b, g, o}, mlp.{up, down}}.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

from .safetensors_io import SafetensorsFile
from .seqlm import (DenseFFConfig, LayerConfig, LinearScaling, MinGRUConfig, RotaryConfig, SeqLMConfig, SeqLMEngine, SeqLMWeights,
                    WindowAttentionConfig)

ARCHITECTURE = "Ronelorn"


def _rotary(d: Optional[dict]) -> RotaryConfig:
    """Rotate-half pairing; linear scaling divides every frequency by its factor."""
    if not d:
        return RotaryConfig(dims=0, base=10000.0, layout="half")
    s = d.get("scaling")
    return RotaryConfig(dims=int(d["dims"]), base=float(d["base"]), layout="half",
                        scaling=LinearScaling(float(s["factor"])) if s and s.get("factor") else None)


def _attention(kind: str, m: dict) -> WindowAttentionConfig:
    mask = m.get("mask") or {}
    rot = _rotary(m.get("rot"))
    common = dict(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])),
                  scale=float(m["scale"]), rot=rot, window=int(mask["size"]) if mask.get("size") else None,
                  softcap=float(m.get("softcap") or 0.0))
    if kind == "attention":
        # pooled blocks before the window; per-head norm; the values are rotated over all of vdim, unscaled, in the same pairing
        return WindowAttentionConfig(qk_norm="head", pool=int(mask.get("pool") or 0),
                                     value_rot=RotaryConfig(dims=common["vdim"], base=rot.base, layout=rot.layout), **common)
    # attention_2: the first tokens stay visible; norm over the whole projection; a sink in the softmax
    return WindowAttentionConfig(qk_norm="full", keep_first=int(mask.get("keep_first") or 0), sink=True, **common)


def _mixer(kind: str, m: dict):
    if kind in ("attention", "attention_2"):
        return _attention(kind, m)
    if kind == "mingru":
        return MinGRUConfig(width=int(m["width"]))
    raise ValueError(f"unknown mixer type {kind!r}")


def _ff(f: Optional[dict]):
    if f is None:
        return None
    if f["kind"] == "dense":
        return DenseFFConfig(ff=int(f["ff"]), act="relu2")
    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")


def config_from_dict(d: dict) -> SeqLMConfig:
    if d.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: architecture = {d.get('architecture')!r}")
    layers = tuple(LayerConfig(mixer=_mixer(l["type"], l["mixer"]), ff=_ff(l.get("mlp")),
                               weights_of=int(l["weights_of"]) if l.get("weights_of") is not None else None) for l in d["layers"])
    return SeqLMConfig(architecture=ARCHITECTURE, vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]), layers=layers,
                       norm="pre", residual_mult=float(d.get("residual_mult", 1.0)),
                       embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)))


def tensor_name(layer: Optional[int], key: str) -> str:
    return key if layer is None else f"l{layer}.{key}"


def load(path, dtype: str = "bfloat16", device="cuda", lib=None, **engine_kw) -> SeqLMEngine:
    """A folder with config.json and model.safetensors -> an engine ready to step."""
    path = Path(path)
    cfg = config_from_dict(json.loads((path / "config.json").read_text()))
    st = SafetensorsFile(path / "model.safetensors")
    try:
        weights = SeqLMWeights(cfg, lambda n: st[n], tensor_name, device)
    finally:
        st.close()
    return SeqLMEngine(cfg, weights, dtype=dtype, lib=lib, **engine_kw)


def from_state_dict(cfg: SeqLMConfig, tensors: dict, dtype: str = "bfloat16", device="cuda", lib=None, **engine_kw) -> SeqLMEngine:
    return SeqLMEngine(cfg, SeqLMWeights(cfg, lambda n: tensors[n], tensor_name, device), dtype=dtype, lib=lib, **engine_kw)
