"""Zudalorn: a decoder-only language model that interleaves retention layers (linear attention with a fixed decay per head and a
32-bit recurrent state) with sliding-window latent-attention layers (a cached low-rank latent plus one shared rotated key part), each
followed by a dense xIELU feed-forward or a grouped-choice mixture of experts with a gated shared expert; every sublayer sits between
two scalar-gain RMS norms.  This module only reads the checkpoint's config.json into the generic layer list of leopard_b200/seqlm.py
and names its tensors; the mechanisms themselves are the shared ones.

config.json keys: architecture, vocab, width, norm.eps, layers[] = {type: "retention" | "latent_attention", mixer: {...}, mlp: null |
{kind: "dense", ff} | {kind: "moe", expert.ff, router.{experts, top, groups.{count, keep}}, shared.ff}}.
Tensor names: embed, head, final.norm, and per layer l<i>.{norm1, norm1b, norm2, norm2b, mix.*, mlp.*}.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

from .safetensors_io import SafetensorsFile
from .seqlm import (DenseFFConfig, LatentAttentionConfig, LayerConfig, MoEConfig, RetentionConfig, RotaryConfig, SeqLMConfig,
                    SeqLMEngine, SeqLMWeights, YarnScaling)

ARCHITECTURE = "Zudalorn"


def _rotary(d: dict, layout: str) -> RotaryConfig:
    s = d.get("scaling")
    scaling = None if not s else YarnScaling(factor=float(s["factor"]), original=float(s["original"]), fast=float(s["fast"]),
                                             slow=float(s["slow"]))
    return RotaryConfig(dims=int(d["dims"]), base=float(d["base"]), layout=layout, scaling=scaling)


def _mixer(kind: str, m: dict):
    if kind == "retention":
        # retention rotates in the rotate-half pairing
        return RetentionConfig(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), decay=tuple(float(x) for x in m["decay"]),
                               rot=_rotary(m["rot"], "half"))
    if kind == "latent_attention":
        # latent attention rotates adjacent pairs; only the rot_dim part of a head is rotated
        mask = m.get("mask") or {}
        return LatentAttentionConfig(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                                     kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), rot=_rotary(m["rot"], "interleaved"),
                                     window=int(mask["size"]) if mask.get("size") else None)
    raise ValueError(f"unknown mixer type {kind!r}")


def _ff(f: Optional[dict]):
    if f is None:
        return None
    if f["kind"] == "dense":
        return DenseFFConfig(ff=int(f["ff"]))
    if f["kind"] == "moe":
        r = f["router"]
        g = r.get("groups") or {"count": 1, "keep": 1}
        sh = f.get("shared")
        return MoEConfig(experts=int(r["experts"]), top=int(r["top"]), expert_ff=int(f["expert"]["ff"]), n_groups=int(g["count"]),
                         keep_groups=int(g["keep"]), shared_ff=int(sh["ff"]) if sh else 0)
    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")


def config_from_dict(d: dict) -> SeqLMConfig:
    if d.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: architecture = {d.get('architecture')!r}")
    layers = tuple(LayerConfig(mixer=_mixer(l["type"], l["mixer"]), ff=_ff(l.get("mlp"))) for l in d["layers"])
    return SeqLMConfig(architecture=ARCHITECTURE, vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]), layers=layers)


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
