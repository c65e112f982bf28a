"""Plain, slow float64 implementation of the layer-list language models (retention, windowed latent attention, xIELU feed-forward,
grouped-choice mixture of experts, scalar-gain RMS norms) — the checker of leopard_b200/seqlm.py.  One function per mechanism,
whole sequences only, nothing shared with the product path: it takes plain dicts (the parsed config.json of a Zudalorn checkpoint)
and a {name: tensor} dict, and loops over tokens where the definition does."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, gain, eps):
    return rms_unit(x, eps) * gain


def rotary_frequencies(rot: dict):
    """(frequencies per pair, factor on cos and sin)"""
    dims, base = rot["dims"], rot["base"]
    idx = torch.arange(dims // 2, dtype=DT)
    freq = base ** (-2.0 * idx / dims)
    factor = 1.0
    sc = rot.get("scaling")
    if sc:
        def where(turns):
            return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), dims - 1)
        blend = ((idx - lo) / max(hi - lo, 0.001)).clamp(0, 1)
        freq = freq / sc["factor"] * blend + freq * (1 - blend)
        factor = 0.1 * math.log(sc["factor"]) + 1.0
    return freq, factor


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict, pairing: str) -> torch.Tensor:
    """x [T, heads, D]: the first rot.dims entries of every head turn by position * frequency; pairing 'half' couples entry i with
    i + dims/2, 'adjacent' couples 2i with 2i + 1."""
    dims = rot["dims"]
    freq, factor = rotary_frequencies(rot)
    out = x.clone()
    for t in range(x.shape[0]):
        ang = float(positions[t]) * freq
        c, s = torch.cos(ang) * factor, torch.sin(ang) * factor
        for i in range(dims // 2):
            a, b = (i, i + dims // 2) if pairing == "half" else (2 * i, 2 * i + 1)
            u, v = x[t, :, a], x[t, :, b]
            out[t, :, a] = u * c[i] - v * s[i]
            out[t, :, b] = v * c[i] + u * s[i]
    return out


def retention(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, positions=None):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    positions = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    g = h @ w[p + "g"].T
    q = rotate(q, positions, m["rot"], "half")
    k = rotate(k, positions, m["rot"], "half") / math.sqrt(dk)
    o = torch.zeros(T, H, dv, dtype=DT)
    for head in range(H):
        S = torch.zeros(dk, dv, dtype=DT)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            o[t, head] = q[t, head] @ S
    o = rms_unit(o, eps).reshape(T, H * dv) * (g * torch.sigmoid(g))
    return o @ w[p + "o"].T


def latent_attention(h, w, p: str, m: dict, eps: float, positions=None):
    T = h.shape[0]
    H, dk, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T).view(T, H, dk + dr)
    down = h @ w[p + "dkv"].T
    c = rms_unit(down[:, :R], eps) * w[p + "dkv.norm"]
    k_shared = rotate(down[:, R:].reshape(T, 1, dr), positions, m["rot"], "adjacent")[:, 0]
    q_plain, q_turn = q[..., :dk], rotate(q[..., dk:].contiguous(), positions, m["rot"], "adjacent")
    k_plain = (c @ w[p + "uk"].T).view(T, H, dk)
    val = (c @ w[p + "uv"].T).view(T, H, dv)
    size = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, dv, dtype=DT)
    for t in range(T):
        first = 0 if not size else max(0, t - size + 1)
        for head in range(H):
            sc = torch.stack([(q_plain[t, head] @ k_plain[j, head] + q_turn[t, head] @ k_shared[j]) * m["scale"] for j in range(first, t + 1)])
            pr = torch.softmax(sc, 0)
            out[t, head] = pr @ val[first:t + 1, head]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def xielu(z, p: float, q: float):
    ap = math.log1p(math.exp(p))
    an = 0.5 + math.log1p(math.exp(q))
    return torch.where(z > 0, ap * z * z + z / 2, an * (torch.expm1(torch.clamp(z, max=0.0)) - z) + z / 2)


def gated_expert(h, w, p: str):
    a = h @ w[p + "gate"].T
    return ((a * torch.sigmoid(a)) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p: str, r: dict):
    """-> (chosen experts [T, top], weights [T, top])"""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    pick = s + w[p + "correction"] if (p + "correction") in w else s.clone()
    g = r.get("groups") or {"count": 1, "keep": 1}
    G, keep = g["count"], g["keep"]
    size = E // G
    chosen, weights = [], []
    for t in range(h.shape[0]):
        score = pick[t].clone()
        if G > 1 and keep < G:
            gs = [score[a * size:(a + 1) * size].sort(descending=True).values[:2].sum() for a in range(G)]
            best = sorted(range(G), key=lambda a: (-float(gs[a]), a))[:keep]
            for a in range(G):
                if a not in best:
                    score[a * size:(a + 1) * size] = float("-inf")
        order = sorted(range(E), key=lambda e: (-float(score[e]), e))[:top]
        wt = s[t, order]
        chosen.append(order)
        weights.append(wt / (wt.sum() + 1e-20))
    return chosen, torch.stack(weights)


def feed_forward(h, w, p: str, f: dict):
    if f["kind"] == "dense":
        a = w[p + "act"]
        return xielu(h @ w[p + "up"].T, float(a[0]), float(a[1])) @ w[p + "down"].T
    chosen, weights = route(h, w, p, f["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k, e in enumerate(chosen[t]):
            out[t] += weights[t, k] * gated_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if f.get("shared"):
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].reshape(-1, 1)) * gated_expert(h, w, p + "shared.")
    return out


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None) -> torch.Tensor:
    """logits float64 [len(tokens), vocab] of one sequence from position 0."""
    w = {k: v.to(DT) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = scalar_norm(x, w[p + "norm1"], eps)
        mix = retention if layer["type"] == "retention" else latent_attention
        x = x + scalar_norm(mix(h, w, p + "mix.", layer["mixer"], eps), w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = scalar_norm(x, w[p + "norm2"], eps)
            x = x + scalar_norm(feed_forward(h, w, p + "mlp.", layer["mlp"]), w[p + "norm2b"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return scalar_norm(x, w["final.norm"], eps) @ w["head"].T


def random_weights(cfg: dict, seed: int = 0, scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """Seeded bf16 weights with every tensor a Zudalorn checkpoint of this config holds."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    out: Dict[str, torch.Tensor] = {}

    def lin(name, n_out, n_in):
        out[name] = (torch.randn(n_out, n_in, generator=g) * scale / math.sqrt(n_in)).to(torch.bfloat16)

    def one(name, lo=0.6, hi=1.4):
        out[name] = torch.empty(()).uniform_(lo, hi, generator=g).to(torch.bfloat16)

    out["embed"] = torch.randn(cfg["vocab"], D, generator=g).to(torch.bfloat16)
    lin("head", cfg["vocab"], D)
    one("final.norm")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        one(p + "norm1")
        one(p + "norm1b")
        if layer["type"] == "retention":
            lin(p + "mix.q", m["heads"] * m["dim"], D)
            lin(p + "mix.k", m["heads"] * m["dim"], D)
            lin(p + "mix.v", m["heads"] * m["vdim"], D)
            lin(p + "mix.g", m["heads"] * m["vdim"], D)
            lin(p + "mix.o", D, m["heads"] * m["vdim"])
        else:
            lin(p + "mix.q", m["heads"] * (m["dim"] + m["rot_dim"]), D)
            lin(p + "mix.dkv", m["kv_rank"] + m["rot_dim"], D)
            out[p + "mix.dkv.norm"] = torch.empty(m["kv_rank"]).uniform_(0.5, 1.5, generator=g).to(torch.bfloat16)
            lin(p + "mix.uk", m["heads"] * m["dim"], m["kv_rank"])
            lin(p + "mix.uv", m["heads"] * m["vdim"], m["kv_rank"])
            lin(p + "mix.o", D, m["heads"] * m["vdim"])
        f = layer.get("mlp")
        if f is None:
            continue
        one(p + "norm2")
        one(p + "norm2b")
        if f["kind"] == "dense":
            lin(p + "mlp.up", f["ff"], D)
            lin(p + "mlp.down", D, f["ff"])
            out[p + "mlp.act"] = torch.empty(2).uniform_(-1.0, 1.0, generator=g).to(torch.bfloat16)
        else:
            r = f["router"]
            for e in range(r["experts"]):
                lin(f"{p}mlp.e{e}.gate", f["expert"]["ff"], D)
                lin(f"{p}mlp.e{e}.up", f["expert"]["ff"], D)
                lin(f"{p}mlp.e{e}.down", D, f["expert"]["ff"])
            lin(p + "mlp.router", r["experts"], D)
            out[p + "mlp.router"] = (out[p + "mlp.router"].float() * 4).to(torch.bfloat16)      # spread the scores: no close calls
            out[p + "mlp.correction"] = torch.empty(r["experts"]).uniform_(-0.3, 0.3, generator=g).to(torch.bfloat16)
            if f.get("shared"):
                lin(p + "mlp.shared.gate", f["shared"]["ff"], D)
                lin(p + "mlp.shared.up", f["shared"]["ff"], D)
                lin(p + "mlp.shared.down", D, f["shared"]["ff"])
                lin(p + "mlp.shared.sg", 1, D)
    return out
