"""Decoder-only language models described as a LIST OF LAYERS, on the 32-bit residual-stream kernels.

A model is a `SeqLMConfig`: vocabulary, width, norm epsilon and a tuple of `LayerConfig`s, each naming its sequence mixer
(`RetentionConfig` or `LatentAttentionConfig`) and its feed-forward (`DenseFFConfig`, `MoEConfig` or none).  Every mechanism is a
separate native entry point with its constants as arguments (include/leopard_b200.h, "32-BIT RESIDUAL-STREAM MODELS"), so another
design is another list.  The residual stream, norms, routers, rotary angles, attention scores and recurrent state are fp32; matrix
products take bf16 weights and, in the serving precision, bf16 activations with fp32 accumulation ("bfloat16"), or fp32 activations
on fp32 FMAs ("float32": a true 32-bit forward, no tensor-core rounding).

`SeqLMEngine.step(entries)` is THE step function: a packed batch of requests, each bringing its next tokens (a whole prompt, a
portion of one, or one token), runs from the cache and state that earlier steps left (leopard_b200/seqcache.py) and returns the
logits of the rows asked for.  The scheduler (leopard_b200/scheduler.py), greedy generation and the trace replayer
(leopard_b200/cli.py) all drive this function.  Host code does allocation, shapes and index tables only; there is no CPU fallback
(a CPU device is accepted only together with an injected library: the tests run the kernel sources under their CPU emulator).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import _lib
from .seqcache import SequenceCache

F32, BF16, I32 = torch.float32, torch.bfloat16, torch.int32
TENSOR_CORE_MIN_ROWS = 64
MOE_PAIRS_MAX = 64             # up to this many (token, choice) pairs the experts run as one-row weight-streaming problems
MAX_DECODE_GRAPHS = 32         # captured decode layouts kept at a time
PAGE_TABLE_STEP = 16           # decode batches round their page-table width up to a multiple of this


# ---------------------------------------------------------------------------------------------------------------- configuration
@dataclass(frozen=True)
class YarnScaling:
    """Frequency rescale for context extension: high-frequency pairs keep their frequency, low-frequency pairs are divided by
    `factor`, with a linear ramp between the pair indices at which `original` positions make `fast` / `slow` full turns; cos and sin
    are multiplied by 0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RotaryConfig:
    dims: int                      # leading dimensions of a head that are rotated
    base: float
    layout: str = "half"           # "half": i pairs with i + dims/2; "interleaved": 2i pairs with 2i + 1
    scaling: Optional[YarnScaling] = None


def rotary_table(rot: RotaryConfig) -> Tuple[torch.Tensor, float]:
    """(inv_freq fp32 [dims/2], magnitude factor) — computed in float64, rounded once."""
    if rot.dims % 2:
        raise ValueError("rotary dims must be even")
    n = rot.dims // 2
    i = np.arange(n, dtype=np.float64)
    f = rot.base ** (-2.0 * i / rot.dims) if n else np.zeros(0)
    mag = 1.0
    s = rot.scaling
    if s is not None:
        def pair_index(turns):      # the (fractional) pair index whose wavelength fits `turns` times into the original context
            return rot.dims * math.log(s.original / (2 * math.pi * turns)) / (2 * math.log(rot.base))
        lo = max(math.floor(pair_index(s.fast)), 0)
        hi = min(math.ceil(pair_index(s.slow)), rot.dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / s.factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(s.factor) + 1.0
    return torch.from_numpy(f.astype(np.float32)), float(mag)


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: RotaryConfig

    @property
    def k_scale(self) -> float:
        return self.dim ** -0.5


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                       # unrotated query / key dimensions per head
    rot_dim: int                   # rotated dimensions per head (the key's are shared by all heads)
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig
    window: Optional[int] = None   # position i sees j with 0 <= i - j < window; None: every earlier position


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int


@dataclass(frozen=True)
class MoEConfig:
    experts: int
    top: int
    expert_ff: int
    n_groups: int = 1
    keep_groups: int = 1
    shared_ff: int = 0             # 0: no shared expert


@dataclass(frozen=True)
class LayerConfig:
    mixer: Union[RetentionConfig, LatentAttentionConfig]
    ff: Union[DenseFFConfig, MoEConfig, None]


@dataclass(frozen=True)
class SeqLMConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: Tuple[LayerConfig, ...]


def softplus(x: float) -> float:
    return math.log1p(math.exp(-abs(x))) + max(x, 0.0)


# ---------------------------------------------------------------------------------------------------------------- weights
class SeqLMWeights:
    """Device tensors in the layout the kernels read.  `get(name)` returns a checkpoint tensor; `name(layer, key)` maps the generic
    keys used here (norm1, norm1b, norm2, norm2b, mix.*, mlp.*; embed, final.norm, head with layer None) to checkpoint names."""

    def __init__(self, cfg: SeqLMConfig, get: Callable[[str], torch.Tensor], name: Callable[[Optional[int], str], str], device):
        self.cfg, self.device = cfg, torch.device(device)
        dev = self.device

        def w(layer, key, shape=None):
            t = get(name(layer, key))
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"{name(layer, key)}: shape {tuple(t.shape)}, expected {tuple(shape)}")
            return t

        def mat(t):
            return t.to(BF16).contiguous().to(dev)

        def num(layer, key):
            return float(w(layer, key).float().reshape(-1)[0])

        D = cfg.width
        self.embed = mat(w(None, "embed", (cfg.vocab, D)))
        self.head = mat(w(None, "head", (cfg.vocab, D)))
        self.final_gain = num(None, "final.norm")
        self.layers: List[Dict[str, object]] = []
        for i, lc in enumerate(cfg.layers):
            lw: Dict[str, object] = {k: num(i, k) for k in ("norm1", "norm1b")}
            m = lc.mixer
            inv_freq, mag = rotary_table(m.rot)
            lw["inv_freq"], lw["rot_mag"] = inv_freq.to(dev), mag
            if isinstance(m, RetentionConfig):
                if len(m.decay) != m.heads:
                    raise ValueError(f"layer {i}: {len(m.decay)} decays for {m.heads} heads")
                lw["w_qkvg"] = mat(torch.cat([w(i, "mix.q", (m.heads * m.dim, D)), w(i, "mix.k", (m.heads * m.dim, D)),
                                              w(i, "mix.v", (m.heads * m.vdim, D)), w(i, "mix.g", (m.heads * m.vdim, D))], 0))
                lw["w_o"] = mat(w(i, "mix.o", (D, m.heads * m.vdim)))
                lw["decay"] = torch.tensor(m.decay, dtype=torch.float64).to(F32).to(dev)
            else:
                per = m.dim + m.rot_dim
                lw["w_qdkv"] = mat(torch.cat([w(i, "mix.q", (m.heads * per, D)), w(i, "mix.dkv", (m.kv_rank + m.rot_dim, D))], 0))
                lw["c_gain"] = w(i, "mix.dkv.norm", (m.kv_rank,)).float().contiguous().to(dev)
                uk = w(i, "mix.uk", (m.heads * m.dim, m.kv_rank))
                lw["w_ukT"] = mat(uk.reshape(m.heads, m.dim, m.kv_rank).transpose(1, 2))       # [heads][kv_rank, dim]
                lw["w_uv"] = mat(w(i, "mix.uv", (m.heads * m.vdim, m.kv_rank)))                 # [heads][vdim, kv_rank]
                lw["w_o"] = mat(w(i, "mix.o", (D, m.heads * m.vdim)))
            f = lc.ff
            if f is not None:
                lw.update({k: num(i, k) for k in ("norm2", "norm2b")})
            if isinstance(f, DenseFFConfig):
                lw["w_up"] = mat(w(i, "mlp.up", (f.ff, D)))
                lw["w_down"] = mat(w(i, "mlp.down", (D, f.ff)))
                act = w(i, "mlp.act", (2,)).float()
                lw["act_a"], lw["act_b"] = softplus(float(act[0])), 0.5 + softplus(float(act[1]))
            elif isinstance(f, MoEConfig):
                lw["w_router"] = mat(w(i, "mlp.router", (f.experts, D)))
                try:
                    corr = w(i, "mlp.correction", (f.experts,)).float()
                except KeyError:                     # a router without a choice bias
                    corr = torch.zeros(f.experts)
                lw["correction"] = corr.contiguous().to(dev)
                gu = [torch.cat([w(i, f"mlp.e{e}.gate", (f.expert_ff, D)), w(i, f"mlp.e{e}.up", (f.expert_ff, D))], 0)
                      for e in range(f.experts)]
                lw["w_gu"] = mat(torch.stack(gu, 0))                                           # [experts][2 ff, D]
                lw["w_edown"] = mat(torch.stack([w(i, f"mlp.e{e}.down", (D, f.expert_ff)) for e in range(f.experts)], 0))
                if f.shared_ff:
                    lw["ws_gu"] = mat(torch.cat([w(i, "mlp.shared.gate", (f.shared_ff, D)), w(i, "mlp.shared.up", (f.shared_ff, D))], 0))
                    lw["ws_down"] = mat(w(i, "mlp.shared.down", (D, f.shared_ff)))
                    lw["w_sg"] = mat(w(i, "mlp.shared.sg").reshape(D))
            self.layers.append(lw)


# ---------------------------------------------------------------------------------------------------------------- batches
@dataclass
class StepEntry:
    key: Hashable                  # the request
    tokens: Sequence[int]          # its next tokens
    want: Sequence[int] = ()       # indices into `tokens` whose logits are returned


class _Batch:
    """Index tables of one step, built on the host and copied to the device in one transfer."""

    def __init__(self, eng: "SeqLMEngine", entries: Sequence[StepEntry], static: Optional[Dict] = None):
        """static: {(n, table width): device int32 buffer} — a decode batch whose layout has been seen before is copied into the same
        device buffer again, so that a captured graph of the step finds its tables where they were."""
        cache = eng.cache
        seqs = []
        for e in entries:
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.key!r} brings no tokens")
            s = cache.get(e.key) or cache.open(e.key)
            cache.reserve(s, len(e.tokens))
            seqs.append(s)
        self.seqs = seqs
        n = len(entries)
        lens = [len(e.tokens) for e in entries]
        R = sum(lens)
        self.R, self.n, self.lens = R, n, lens
        self.decode = all(ln == 1 for ln in lens)
        row0 = np.zeros(n + 1, np.int32)
        row0[1:] = np.cumsum(lens)
        pos0 = np.array([s.length for s in seqs], np.int32)
        slot = np.array([s.slot for s in seqs], np.int32)
        tokens = np.concatenate([np.asarray(e.tokens, np.int64) for e in entries])
        if tokens.min() < 0 or tokens.max() >= eng.cfg.vocab:
            raise ValueError("token id outside the vocabulary")
        row_seq = np.repeat(np.arange(n, dtype=np.int32), lens)
        row_pos = np.concatenate([np.arange(p, p + ln, dtype=np.int32) for p, ln in zip(pos0, lens)])
        max_pages = max([len(s.pages) for s in seqs] + [1])
        if self.decode:
            max_pages = -(-max_pages // PAGE_TABLE_STEP) * PAGE_TABLE_STEP      # the width is a launch argument: change it rarely
        table = np.full((n, max_pages), -1, np.int32)
        for i, s in enumerate(seqs):
            table[i, : len(s.pages)] = s.pages
        ch = _lib.RETENTION_CHUNK
        c_seq, c_row0, c_len, seq_c0 = [], [], [], [0]
        for i, ln in enumerate(lens):
            for a in range(0, ln, ch):
                c_seq.append(i)
                c_row0.append(int(row0[i]) + a)
                c_len.append(min(ch, ln - a))
            seq_c0.append(len(c_seq))
        self.n_chunks = len(c_seq)
        self.max_pages = max_pages
        want = [int(row0[i]) + int(k) for i, e in enumerate(entries) for k in e.want]
        for i, e in enumerate(entries):
            if any(k < 0 or k >= lens[i] for k in e.want):
                raise ValueError(f"request {e.key!r}: a wanted index is outside its tokens")
        self.n_want = len(want)
        parts = [tokens.astype(np.int32), row_seq, row_pos, row0, pos0, slot, table.reshape(-1), np.asarray(c_seq, np.int32),
                 np.asarray(c_row0, np.int32), np.asarray(c_len, np.int32), np.asarray(seq_c0, np.int32)]
        tables = torch.from_numpy(np.concatenate(parts).astype(np.int32))
        want_t = torch.from_numpy(np.asarray(want, np.int32))
        self.layout = (n, max_pages) if self.decode else None      # fixes the size of every table of a decode batch
        if eng.device.type == "cuda":
            host = tables.pin_memory()
            if static is not None and self.decode:
                tables = static.get(self.layout)
                if tables is None:
                    tables = static[self.layout] = torch.empty(len(host), dtype=I32, device=eng.device)
                tables.copy_(host, non_blocking=True)
            else:
                tables = host.to(eng.device, non_blocking=True)
            if len(want):
                want_t = want_t.pin_memory().to(eng.device, non_blocking=True)
        views, o = [], 0
        for p in parts:
            views.append(tables[o:o + len(p)])
            o += len(p)
        (self.tokens, self.row_seq, self.row_pos, self.seq_row0, self.seq_pos0, self.seq_slot, self.page_table, self.chunk_seq,
         self.chunk_row0, self.chunk_len, self.seq_chunk0) = views
        self.want_rows = want_t
        self._tables = tables


# ---------------------------------------------------------------------------------------------------------------- engine
class SeqLMEngine:
    def __init__(self, cfg: SeqLMConfig, weights: SeqLMWeights, dtype: str = "bfloat16", max_tokens: int = 4096, page_size: int = 64,
                 max_seqs: int = 8, lib=None):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        self.cfg, self.w, self.device = cfg, weights, weights.device
        if lib is None:
            if self.device.type != "cuda" or not torch.cuda.is_available():
                raise _lib.NativeError("leopard_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
            lib = _lib.stream32_lib()
        self.L = lib
        self.dtype = dtype
        self.act = BF16 if dtype == "bfloat16" else F32
        lat = [lc.mixer for lc in cfg.layers if isinstance(lc.mixer, LatentAttentionConfig)]
        ret = [lc.mixer for lc in cfg.layers if isinstance(lc.mixer, RetentionConfig)]
        window = None if any(m.window is None or m.window <= 0 for m in lat) else max([m.window for m in lat], default=None)
        self.cache = SequenceCache([m.kv_rank + m.rot_dim for m in lat], [(m.heads, m.dim, m.vdim) for m in ret], window, self.device,
                                   max_tokens=max_tokens, page_size=page_size, max_seqs=max_seqs)
        self._cache_index, self._state_index, a, b = [], [], 0, 0
        for lc in cfg.layers:
            is_lat = isinstance(lc.mixer, LatentAttentionConfig)
            self._cache_index.append(a if is_lat else -1)
            self._state_index.append(-1 if is_lat else b)
            a, b = a + is_lat, b + (not is_lat)
        self.tile_rows = int(self.L.lp_linear_tile_rows())
        # large bf16 products of the serving precision go to the tcgen05 GEMM when the library has it (the native ones do)
        self.tensor_core_rows = TENSOR_CORE_MIN_ROWS if dtype == "bfloat16" and hasattr(self.L, "lp_gemm_bf16") else None
        self.tap: Optional[Callable[[int, torch.Tensor], None]] = None   # called with (layer, residual stream) after every layer
        # decode steps are launch-bound: a batch layout (requests, page-table width) that comes back is captured into a CUDA graph on
        # its second appearance and replayed from then on; only the index tables change between replays (LEOPARD_DECODE_GRAPH=0: off)
        import os
        self.use_graphs = self.device.type == "cuda" and os.environ.get("LEOPARD_DECODE_GRAPH", "1") != "0"
        self._static_tables: Dict = {}
        self._graphs: Dict = {}
        self._seen: Dict = {}

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream().cuda_stream) if self.device.type == "cuda" else None

    def _check(self, rc, what):
        _lib.check_on(self.L, rc, what)

    def _empty(self, shape, dtype):
        return torch.empty(shape, dtype=dtype, device=self.device)

    def _on_tensor_cores(self, a, w, M, N, K) -> bool:
        """The tcgen05 GEMM takes a product when it is large enough to fill tiles and meets the 16-byte rules of its TMA loads."""
        return (self.tensor_core_rows is not None and M >= self.tensor_core_rows and a.dtype == BF16 and N >= 128 and K >= 64
                and N % 8 == 0 and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def linear(self, a: torch.Tensor, w: torch.Tensor, out_dtype, epi=_lib.EPI_NONE, epi_a=0.0, epi_b=0.0, out=None):
        """out[M, N'] = epi(a[M, K] @ w[N, K].T)."""
        M, K = a.shape
        N = w.shape[0]
        n_out = N // 2 if epi == _lib.EPI_SILU_GATE else N
        if out is None:
            out = self._empty((M, n_out), out_dtype)
        if self._on_tensor_cores(a, w, M, N, K) and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0:
            raw = out if epi == _lib.EPI_NONE else self._empty((M, N), F32)
            rc = self.L.lp_gemm_bf16(_lib.ptr(a), a.stride(0), _lib.ptr(w), w.stride(0), _lib.ptr(raw), raw.stride(0), M, N, K, None, None,
                                     0, 0, _lib.ACT_NONE, int(raw.dtype == F32), 0, self._stream())
            self._check(rc, "lp_gemm_bf16")
            if epi != _lib.EPI_NONE:
                rc = self.L.lp_glu_f32(_lib.ptr(raw), raw.stride(0), 1, _lib.ptr(out), out.stride(0), int(out.dtype == F32), M, n_out, epi,
                                       epi_a, epi_b, self._stream())
                self._check(rc, "lp_glu_f32")
            return out
        d = _lib.LinearDesc(A=_lib.ptr(a), lda=a.stride(0), a_batch=0, a_fp32=int(a.dtype == F32), W=_lib.ptr(w), ldw=w.stride(0),
                            w_batch=0, C=_lib.ptr(out), ldc=out.stride(0), c_batch=0, c_fp32=int(out.dtype == F32), M=M, N=N, K=K,
                            batch=1, epi=epi, epi_a=epi_a, epi_b=epi_b)
        self._check(self.L.lp_linear(C.byref(d), self._stream()), "lp_linear")
        return out

    def linear_heads(self, a: torch.Tensor, a_head: int, w: torch.Tensor, out: torch.Tensor, out_head: int):
        """Per head h: out[:, h*out_head : +N] = a[:, h*a_head : +K] @ w[h].T with w [heads, N, K]."""
        heads, N, K = w.shape
        d = _lib.LinearDesc(A=_lib.ptr(a), lda=a.stride(0), a_batch=a_head, a_fp32=int(a.dtype == F32), W=_lib.ptr(w), ldw=w.stride(1),
                            w_batch=w.stride(0), C=_lib.ptr(out), ldc=out.stride(0), c_batch=out_head, c_fp32=int(out.dtype == F32),
                            M=a.shape[0], N=N, K=K, batch=heads, epi=_lib.EPI_NONE, epi_a=0.0, epi_b=0.0)
        self._check(self.L.lp_linear(C.byref(d), self._stream()), "lp_linear")
        return out

    def norm(self, x: torch.Tensor, gain: float, out_dtype=None, accum: Optional[torch.Tensor] = None):
        """RMS norm with one gain for all coordinates; `accum`: add the result to it instead of returning it."""
        M, D = x.shape
        out = None if accum is not None else self._empty((M, D), out_dtype)
        rc = self.L.lp_rmsnorm_f32(_lib.ptr(x), x.stride(0), M, D, gain, None, self.cfg.eps, _lib.ptr(out),
                                   out.stride(0) if out is not None else 0, int(out is not None and out.dtype == F32), _lib.ptr(accum),
                                   accum.stride(0) if accum is not None else 0, self._stream())
        self._check(rc, "lp_rmsnorm_f32")
        return out

    # ------------------------------------------------------------------ mixers
    def _retention(self, li: int, m: RetentionConfig, lw, h: torch.Tensor, b: _Batch) -> torch.Tensor:
        qkvg = self.linear(h, lw["w_qkvg"], F32)
        hd, hv = m.heads * m.dim, m.heads * m.vdim
        out = self._empty((b.R, hv), self.act)
        state = self.cache.states[self._state_index[li]]
        d = _lib.RetentionDesc(qkvg=_lib.ptr(qkvg), ld=qkvg.stride(0), q_off=0, k_off=hd, v_off=2 * hd, g_off=2 * hd + hv, heads=m.heads,
                               dim=m.dim, vdim=m.vdim, decay=_lib.ptr(lw["decay"]), inv_freq=_lib.ptr(lw["inv_freq"]), rot_dims=m.rot.dims,
                               rot_layout=_lib.ROT_INTERLEAVED if m.rot.layout == "interleaved" else _lib.ROT_HALF,
                               rot_mscale=lw["rot_mag"], k_scale=m.k_scale, eps=self.cfg.eps, state=_lib.ptr(state),
                               slot_stride=state.stride(0), out=_lib.ptr(out), ldo=out.stride(0), out_fp32=int(out.dtype == F32))
        if b.decode:
            rc = self.L.lp_retention_decode(C.byref(d), b.n, _lib.ptr(b.seq_row0), _lib.ptr(b.seq_pos0), _lib.ptr(b.seq_slot), self._stream())
            self._check(rc, "lp_retention_decode")
        else:
            nbytes = int(self.L.lp_retention_workspace_bytes(b.n_chunks, m.heads, m.dim, m.vdim))
            ws = self._empty((nbytes // 4,), F32)
            rc = self.L.lp_retention_prefill(C.byref(d), b.n, b.n_chunks, _lib.ptr(b.seq_row0), _lib.ptr(b.seq_pos0), _lib.ptr(b.seq_slot),
                                             _lib.ptr(b.seq_chunk0), _lib.ptr(b.chunk_seq), _lib.ptr(b.chunk_row0), _lib.ptr(b.chunk_len),
                                             _lib.ptr(ws), nbytes, self._stream())
            self._check(rc, "lp_retention_prefill")
        return self.linear(out, lw["w_o"], F32)

    def _latent(self, li: int, m: LatentAttentionConfig, lw, h: torch.Tensor, b: _Batch) -> torch.Tensor:
        per = m.dim + m.rot_dim
        qd = self.linear(h, lw["w_qdkv"], F32)
        q, dkv = qd[:, : m.heads * per], qd[:, m.heads * per:]
        pool = self.cache.pools[self._cache_index[li]]
        d = _lib.LatentDesc(q=_lib.ptr(q), ldq=qd.stride(0), dkv=_lib.ptr(dkv), lddkv=qd.stride(0), heads=m.heads, dim=m.dim,
                            rot_dim=m.rot_dim, kv_rank=m.kv_rank, c_gain=_lib.ptr(lw["c_gain"]), eps=self.cfg.eps,
                            inv_freq=_lib.ptr(lw["inv_freq"]), rot_dims=m.rot.dims,
                            rot_layout=_lib.ROT_INTERLEAVED if m.rot.layout == "interleaved" else _lib.ROT_HALF,
                            rot_mscale=lw["rot_mag"], cache=_lib.ptr(pool), page_size=self.cache.page_size,
                            page_table=_lib.ptr(b.page_table), max_pages=b.max_pages, window=m.window or 0, scale=m.scale)
        self._check(self.L.lp_latent_prep(C.byref(d), b.R, _lib.ptr(b.row_seq), _lib.ptr(b.row_pos), self._stream()), "lp_latent_prep")
        q_abs = self._empty((b.R, m.heads * m.kv_rank), F32)
        self.linear_heads(q, per, lw["w_ukT"], q_abs, m.kv_rank)
        lat = self._empty((b.R, m.heads * m.kv_rank), self.act)
        rc = self.L.lp_latent_attend(C.byref(d), b.R, _lib.ptr(b.row_seq), _lib.ptr(b.row_pos), _lib.ptr(q_abs), q_abs.stride(0),
                                     _lib.ptr(lat), lat.stride(0), int(lat.dtype == F32), self._stream())
        self._check(rc, "lp_latent_attend")
        o = self._empty((b.R, m.heads * m.vdim), self.act)
        self.linear_heads(lat, m.kv_rank, lw["w_uv"].view(m.heads, m.vdim, m.kv_rank), o, m.vdim)
        return self.linear(o, lw["w_o"], F32)

    # ------------------------------------------------------------------ feed-forwards
    def _dense(self, f: DenseFFConfig, lw, h: torch.Tensor) -> torch.Tensor:
        up = self.linear(h, lw["w_up"], self.act, _lib.EPI_XIELU, lw["act_a"], lw["act_b"])
        return self.linear(up, lw["w_down"], F32)

    def _moe(self, f: MoEConfig, lw, h: torch.Tensor) -> torch.Tensor:
        T, D = h.shape
        L, st = self.L, self._stream()
        idx = self._empty((T, f.top), I32)
        wts = self._empty((T, f.top), F32)
        gate = self._empty((T,), F32) if f.shared_ff else None
        rc = L.lp_moe_route(_lib.ptr(h), h.stride(0), int(h.dtype == F32), T, D, _lib.ptr(lw["w_router"]), lw["w_router"].stride(0),
                            f.experts, _lib.ptr(lw["correction"]), f.n_groups, f.keep_groups, f.top,
                            _lib.ptr(lw["w_sg"]) if f.shared_ff else None, _lib.ptr(idx), _lib.ptr(wts), _lib.ptr(gate), st)
        self._check(rc, "lp_moe_route")
        n_pairs = T * f.top
        if n_pairs <= MOE_PAIRS_MAX:
            # few (token, choice) pairs (decoding): no sorting — every pair streams its expert's weights once, pair z = row z
            w_gu, w_dn = lw["w_gu"], lw["w_edown"]
            h1 = self._empty((n_pairs, f.expert_ff), self.act)
            d1 = _lib.LinearDesc(A=_lib.ptr(h), lda=h.stride(0), a_batch=0, a_fp32=int(h.dtype == F32), W=_lib.ptr(w_gu), ldw=w_gu.stride(1),
                                 w_batch=w_gu.stride(0), C=_lib.ptr(h1), ldc=h1.stride(0), c_batch=0, c_fp32=int(h1.dtype == F32), M=1,
                                 N=2 * f.expert_ff, K=D, batch=1, epi=_lib.EPI_SILU_GATE, epi_a=0.0, epi_b=0.0)
            self._check(L.lp_linear_pairs(C.byref(d1), _lib.ptr(idx), f.top, n_pairs, st), "lp_linear_pairs")
            y = self._empty((n_pairs, D), F32)
            d2 = _lib.LinearDesc(A=_lib.ptr(h1), lda=h1.stride(0), a_batch=0, a_fp32=int(h1.dtype == F32), W=_lib.ptr(w_dn),
                                 ldw=w_dn.stride(1), w_batch=w_dn.stride(0), C=_lib.ptr(y), ldc=y.stride(0), c_batch=0, c_fp32=1, M=1, N=D,
                                 K=f.expert_ff, batch=1, epi=_lib.EPI_NONE, epi_a=0.0, epi_b=0.0)
            self._check(L.lp_linear_pairs(C.byref(d2), _lib.ptr(idx), 1, n_pairs, st), "lp_linear_pairs")
            return self._moe_combine(f, lw, h, y, self._pair_identity(n_pairs), wts, gate)
        tiles = int(L.lp_moe_max_tiles(n_pairs, f.experts, self.tile_rows))
        tile_group = self._empty((tiles,), I32)
        sorted_token = self._empty((tiles * self.tile_rows,), I32)
        pair_row = self._empty((n_pairs,), I32)
        rc = L.lp_moe_align(_lib.ptr(idx), n_pairs, f.top, f.experts, self.tile_rows, tiles, _lib.ptr(tile_group), _lib.ptr(sorted_token),
                            _lib.ptr(pair_row), st)
        self._check(rc, "lp_moe_align")
        rows = tiles * self.tile_rows
        h1 = self._empty((rows, f.expert_ff), self.act)
        y = self._empty((rows, D), F32)
        w_gu, w_dn = lw["w_gu"], lw["w_edown"]
        if self.tensor_core_rows is not None and n_pairs >= f.experts * self.tensor_core_rows and h.dtype == BF16:
            # prefill in the serving precision: enough rows per expert to fill tensor-core tiles.  The segment bounds come to the host
            # (one small device -> host copy), the rows are gathered into expert order and every expert runs two tcgen05 GEMMs.
            groups = tile_group.cpu().tolist()
            a_sorted = h.index_select(0, sorted_token.clamp_min(0).long())
            t0 = 0
            while t0 < tiles:
                e, t1 = groups[t0], t0 + 1
                while t1 < tiles and groups[t1] == e:
                    t1 += 1
                if e >= 0:
                    r0, r1 = t0 * self.tile_rows, t1 * self.tile_rows
                    self.linear(a_sorted[r0:r1], w_gu[e], self.act, _lib.EPI_SILU_GATE, out=h1[r0:r1])
                    self.linear(h1[r0:r1], w_dn[e], F32, out=y[r0:r1])
                t0 = t1
        else:
            d1 = _lib.LinearDesc(A=_lib.ptr(h), lda=h.stride(0), a_batch=0, a_fp32=int(h.dtype == F32), W=_lib.ptr(w_gu), ldw=w_gu.stride(1),
                                 w_batch=w_gu.stride(0), C=_lib.ptr(h1), ldc=h1.stride(0), c_batch=0, c_fp32=int(h1.dtype == F32), M=rows,
                                 N=2 * f.expert_ff, K=D, batch=1, epi=_lib.EPI_SILU_GATE, epi_a=0.0, epi_b=0.0)
            self._check(L.lp_linear_grouped(C.byref(d1), _lib.ptr(tile_group), tiles, _lib.ptr(sorted_token), st), "lp_linear_grouped")
            d2 = _lib.LinearDesc(A=_lib.ptr(h1), lda=h1.stride(0), a_batch=0, a_fp32=int(h1.dtype == F32), W=_lib.ptr(w_dn),
                                 ldw=w_dn.stride(1), w_batch=w_dn.stride(0), C=_lib.ptr(y), ldc=y.stride(0), c_batch=0, c_fp32=1, M=rows,
                                 N=D, K=f.expert_ff, batch=1, epi=_lib.EPI_NONE, epi_a=0.0, epi_b=0.0)
            self._check(L.lp_linear_grouped(C.byref(d2), _lib.ptr(tile_group), tiles, None, st), "lp_linear_grouped")
        return self._moe_combine(f, lw, h, y, pair_row, wts, gate)

    def _pair_identity(self, n: int) -> torch.Tensor:
        t = getattr(self, "_arange", None)
        if t is None or t.numel() < n:
            t = self._arange = torch.arange(max(n, 256), dtype=I32, device=self.device)
        return t

    def _moe_combine(self, f: MoEConfig, lw, h, y, pair_row, wts, gate) -> torch.Tensor:
        T, D = h.shape
        shared = None
        if f.shared_ff:
            s1 = self.linear(h, lw["ws_gu"], self.act, _lib.EPI_SILU_GATE)
            shared = self.linear(s1, lw["ws_down"], F32)
        out = self._empty((T, D), F32)
        rc = self.L.lp_moe_combine(_lib.ptr(y), y.stride(0), _lib.ptr(pair_row), _lib.ptr(wts), f.top, _lib.ptr(shared),
                                   shared.stride(0) if shared is not None else 0, _lib.ptr(gate), _lib.ptr(out), out.stride(0), T, D,
                                   self._stream())
        self._check(rc, "lp_moe_combine")
        return out

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the tokens each entry brings, from the cache and state earlier steps left; returns fp32 logits [wanted rows, vocab]
        in the order of the entries and of their `want` lists (None when nothing is wanted)."""
        if not entries:
            return None
        if len({e.key for e in entries}) != len(entries):
            raise ValueError("a request appears twice in one step")
        b = _Batch(self, entries, self._static_tables if self.use_graphs else None)
        if b.decode and self.use_graphs and self.tap is None:
            logits = self._decode_replay(b)
        else:
            logits = self._forward(b, b.want_rows if b.n_want else None)
        for s, ln in zip(b.seqs, b.lens):
            self.cache.advance(s, ln)
        return logits

    def _decode_replay(self, b: _Batch) -> Optional[torch.Tensor]:
        """One-token-per-request steps: eager the first time a layout is seen, captured the second time, replayed afterwards.  The
        graph computes the logits of every row; the wanted ones are picked afterwards."""
        key = (b.layout, self.cache.generation)
        g = self._graphs.get(key)
        if g is None:
            self._seen[key] = self._seen.get(key, 0) + 1
            if self._seen[key] < 2:
                return self._forward(b, b.want_rows if b.n_want else None)
            for old in [k for k in self._graphs if k[1] != self.cache.generation]:
                del self._graphs[old]                      # pools were reallocated: those graphs point at freed memory
            if len(self._graphs) >= MAX_DECODE_GRAPHS:      # a bound on what the captured layouts may hold
                self._graphs.clear()
                self._seen.clear()
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph):
                out = self._forward(b, "all")
            g = self._graphs[key] = (graph, out)
        g[0].replay()
        if b.n_want == 0:
            return None
        return g[1].index_select(0, b.want_rows.long()) if b.n_want != b.R else g[1].clone()

    def _forward(self, b: _Batch, want) -> Optional[torch.Tensor]:
        """embedding -> layers -> (final norm, head) over the rows `want` (a device index tensor, "all", or None)"""
        cfg, D = self.cfg, self.cfg.width
        x = self._empty((b.R, D), F32)
        rc = self.L.lp_embed_rows_f32(_lib.ptr(b.tokens), b.R, _lib.ptr(self.w.embed), self.w.embed.stride(0), cfg.vocab, _lib.ptr(x),
                                      x.stride(0), D, self._stream())
        self._check(rc, "lp_embed_rows_f32")
        for li, (lc, lw) in enumerate(zip(cfg.layers, self.w.layers)):
            h = self.norm(x, lw["norm1"], self.act)
            if isinstance(lc.mixer, RetentionConfig):
                mixed = self._retention(li, lc.mixer, lw, h, b)
            else:
                mixed = self._latent(li, lc.mixer, lw, h, b)
            self.norm(mixed, lw["norm1b"], accum=x)
            if lc.ff is not None:
                h = self.norm(x, lw["norm2"], self.act)
                y = self._dense(lc.ff, lw, h) if isinstance(lc.ff, DenseFFConfig) else self._moe(lc.ff, lw, h)
                self.norm(y, lw["norm2b"], accum=x)
            if self.tap is not None:
                self.tap(li, x)
        if want is None:
            return None
        rows = x if isinstance(want, str) else x.index_select(0, want.long())
        hn = self.norm(rows, self.w.final_gain, self.act)
        return self.linear(hn, self.w.head, F32)

    def finish(self, key: Hashable) -> None:
        """The request is over: its pages and its slot go back to the pools."""
        self.cache.close(key)
