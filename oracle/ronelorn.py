"""Plain, slow float64 implementation of the Ronelorn layers: what the tests compare the window-attention, minGRU and pre-norm paths
of leopard_b200/seqlm.py with.  One function per mechanism, whole sequences from position 0 only, explicit loops over queries and keys,
nothing shared with the product path: it takes the parsed config.json and a {name: tensor} dict.

Notation: T tokens, H query heads, G key / value heads (query head h reads group h // (H // G)), d key size, e value size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def one_plus_norm(x, w, eps):
    """the gain is stored around zero"""
    return unit_rms(x, eps) * (1.0 + w)


def turn(x: torch.Tensor, angles_of: torch.Tensor, n: int, base: float, divide: float = 1.0) -> torch.Tensor:
    """x [T, heads, D]; the first n entries of each head are turned: entry i is coupled with entry i + n/2, the couple at row t turns
    by angles_of[t] * base^(-2i/n) / divide.  Negative angles_of turn back."""
    out = x.clone()
    for t in range(x.shape[0]):
        for i in range(n // 2):
            ang = float(angles_of[t]) * base ** (-2.0 * i / n) / divide
            c, s = math.cos(ang), math.sin(ang)
            a, b = x[t, :, i], x[t, :, i + n // 2]
            out[t, :, i] = a * c - b * s
            out[t, :, i + n // 2] = b * c + a * s
    return out


def _project(h, w, p, m):
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return (h @ w[p + "q"].T), (h @ w[p + "k"].T), (h @ w[p + "v"].T).view(T, G, e), (T, H, G, d, e)


def pooled_window_attention(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """mixer 'attention': per-head q / k norm, rotation of q, k (frequencies divided by the scaling factor) and of v (all of e, never
    divided), capped scores, window of `size` tokens plus the mean key / value of every block of `pool` tokens wholly before it."""
    q, k, v, (T, H, G, d, e) = _project(h, w, p, m)
    q = unit_rms(q.view(T, H, d), eps) * w[p + "q.norm"]
    k = unit_rms(k.view(T, G, d), eps) * w[p + "k.norm"]
    pos = torch.arange(T, dtype=DT)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    divide = (rot.get("scaling") or {}).get("factor", 1.0)
    q, k = turn(q, pos, rot["dims"], rot["base"], divide), turn(k, pos, rot["dims"], rot["base"], divide)
    v = turn(v, pos, e, rot["base"])
    mask = m.get("mask") or {}
    size, P = mask.get("size"), mask.get("pool") or 0
    cap = m.get("softcap") or 0.0
    out = torch.zeros(T, H, e, dtype=DT)
    for i in range(T):
        tokens = [j for j in range(i + 1) if not size or i - j < size]
        blocks = [b for b in range(T) if size and P and b * P + P - 1 <= i - size]
        for hd in range(H):
            g = hd // (H // G)
            keys = [k[b * P:(b + 1) * P, g].mean(0) for b in blocks] + [k[j, g] for j in tokens]
            vals = [v[b * P:(b + 1) * P, g].mean(0) for b in blocks] + [v[j, g] for j in tokens]
            sc = torch.stack([q[i, hd] @ kk for kk in keys]) * m["scale"]
            if cap:
                sc = cap * torch.tanh(sc / cap)
            out[i, hd] = torch.softmax(sc, 0) @ torch.stack(vals)
    out = turn(out, -pos, e, rot["base"])
    return out.reshape(T, H * e) @ w[p + "o"].T


def sink_window_attention(h, w, p: str, m: dict, eps: float):
    """mixer 'attention_2': q / k norm over the whole projection, rotation of q and k only, window of `size` tokens plus the first
    `keep_first` tokens of the sequence, and a softmax whose denominator has one added."""
    q, k, v, (T, H, G, d, e) = _project(h, w, p, m)
    q = (unit_rms(q, eps) * w[p + "q.norm"]).view(T, H, d)
    k = (unit_rms(k, eps) * w[p + "k.norm"]).view(T, G, d)
    pos = torch.arange(T, dtype=DT)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    divide = (rot.get("scaling") or {}).get("factor", 1.0)
    q, k = turn(q, pos, rot["dims"], rot["base"], divide), turn(k, pos, rot["dims"], rot["base"], divide)
    mask = m.get("mask") or {}
    size, first = mask.get("size"), mask.get("keep_first") or 0
    cap = m.get("softcap") or 0.0
    out = torch.zeros(T, H, e, dtype=DT)
    for i in range(T):
        seen = [j for j in range(i + 1) if not size or i - j < size or j < first]
        for hd in range(H):
            g = hd // (H // G)
            sc = torch.stack([q[i, hd] @ k[j, g] for j in seen]) * m["scale"]
            if cap:
                sc = cap * torch.tanh(sc / cap)
            ex = torch.exp(sc)
            out[i, hd] = (ex / (1.0 + ex.sum())) @ v[seen, g]
    return out.reshape(T, H * e) @ w[p + "o"].T


def mingru(h, w, p: str, m: dict, eps: float):
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = h @ w[p + "g"].T
    S = torch.zeros(m["width"], dtype=DT)
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S * gate[t] * torch.sigmoid(gate[t]))
    return torch.stack(rows) @ w[p + "o"].T


def squared_relu_ff(h, w, p: str):
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


MIXERS = {"attention": pooled_window_attention, "attention_2": sink_window_attention, "mingru": mingru}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None) -> torch.Tensor:
    """logits float64 [len(tokens), vocab] of one sequence from position 0."""
    w = {k: v.to(DT) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = w["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer['weights_of'] if layer.get('weights_of') is not None else i}."
        x = x + mult * MIXERS[layer["type"]](one_plus_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + mult * squared_relu_ff(one_plus_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        if residuals is not None:
            residuals.append(x.clone())
    return one_plus_norm(x, w["final.norm"], eps) @ w["head"].T


def random_weights(cfg: dict, seed: int = 0, scale: float = 1.0, sharp: float = 1.0) -> Dict[str, torch.Tensor]:
    """Seeded bf16 weights with every tensor a Ronelorn checkpoint of this config holds.  `sharp` multiplies the query / key norm gains:
    larger values make each softmax lean on few keys, so that a key wrongly seen or missed changes the result visibly."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    out: Dict[str, torch.Tensor] = {}

    def lin(name, n_out, n_in):
        out[name] = (torch.randn(n_out, n_in, generator=g) * scale / math.sqrt(n_in)).to(torch.bfloat16)

    def around(name, n, mid=0.0, spread=0.3):
        out[name] = (mid + torch.empty(n).uniform_(-spread, spread, generator=g)).to(torch.bfloat16)

    out["embed"] = torch.randn(cfg["vocab"], D, generator=g).to(torch.bfloat16)
    lin("head", cfg["vocab"], D)
    around("final.norm", D)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        around(p + "norm1", D)
        if layer["type"] == "mingru":
            for n in ("z", "x", "g"):
                lin(p + "mix." + n, m["width"], D)
            out[p + "mix.x"] = (out[p + "mix.x"].float() * 2).to(torch.bfloat16)      # candidates on both sides of zero
            around(p + "mix.z.b", m["width"], spread=1.0)
            around(p + "mix.x.b", m["width"], spread=0.5)
            lin(p + "mix.o", D, m["width"])
        else:
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            lin(p + "mix.q", H * d, D)
            lin(p + "mix.k", G * d, D)
            lin(p + "mix.v", G * e, D)
            lin(p + "mix.o", D, H * e)
            n_q, n_k = (d, d) if layer["type"] == "attention" else (H * d, G * d)
            around(p + "mix.q.norm", n_q, mid=sharp)
            around(p + "mix.k.norm", n_k, mid=sharp)
        if layer.get("mlp") is not None:
            around(p + "norm2", D)
            lin(p + "mlp.up", layer["mlp"]["ff"], D)
            lin(p + "mlp.down", D, layer["mlp"]["ff"])
    return out
