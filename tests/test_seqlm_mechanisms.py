"""Each mechanism of the 32-bit residual-stream models alone, against the plain implementation in oracle/seqlm.py: the general linear
layer (both kernels, every epilogue, per-head batches, ragged shapes), scalar-gain RMS norm with the residual update, rotary tables
with frequency rescaling, retention, windowed latent attention, the grouped-choice router, the expert feed-forward and xIELU.  Every
test runs on the kernel SOURCES under the CPU emulator (tests/emu) and, marked gpu, on the native library."""
import math

import pytest
import torch

from leopard_b200 import _lib
from leopard_b200.seqlm import RotaryConfig, StepEntry, YarnScaling, rotary_table
from oracle import seqlm as O
from seqlm_common import (TOL, backend, dense, emu_lib, latent_layer, make_engine, model, moe, rel_err,  # noqa: F401
                          retention_layer)

F32, BF16 = torch.float32, torch.bfloat16


def _tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def _engine_1layer(layer, backend, dtype="float32", seed=1, **kw):
    cfg = model([layer])
    w = O.random_weights(cfg, seed=seed)
    return cfg, w, make_engine(cfg, w, backend, dtype, **kw)


@pytest.mark.parametrize("M", [3, 70])
def test_linear_kernels(backend, M):
    device, _ = backend
    cfg, w, eng = _engine_1layer(retention_layer(), backend)
    g = torch.Generator().manual_seed(M)
    for K, N in ((20, 13), (64, 72)):
        a = torch.randn(M, K, generator=g)
        wt = torch.randn(N, K, generator=g).to(BF16)
        want = a.double() @ wt.double().T
        for a_dt, c_dt, tol in ((F32, F32, 1e-6), (BF16, F32, 1e-2), (F32, BF16, 1e-2)):
            got = eng.linear(a.to(a_dt).to(device), wt.to(device), c_dt)
            assert rel_err(got, want) < tol, (M, K, N, a_dt, c_dt)
        # xIELU epilogue and the gated epilogue (weight = gate rows, then up rows)
        got = eng.linear(a.to(device), wt.to(device), F32, _lib.EPI_XIELU, 0.7, 0.9)
        z = want
        ref = torch.where(z > 0, 0.7 * z * z + z / 2, 0.9 * (torch.expm1(z.clamp(max=0)) - z) + z / 2)
        assert rel_err(got, ref) < 1e-5
        if N % 2 == 0:
            got = eng.linear(a.to(device), wt.to(device), F32, _lib.EPI_SILU_GATE)
            gate, up = want[:, : N // 2], want[:, N // 2:]
            assert rel_err(got, gate * torch.sigmoid(gate) * up) < 1e-5
    # per-head batches with strided operands
    heads, K, N = 3, 5, 6
    a = torch.randn(M, heads * 7, generator=g)
    wt = torch.randn(heads, N, K, generator=g).to(BF16)
    out = torch.zeros(M, heads * N, device=device)
    eng.linear_heads(a.to(device), 7, wt.to(device), out, N)
    want = torch.cat([a[:, h * 7:h * 7 + K].double() @ wt[h].double().T for h in range(heads)], 1)
    assert rel_err(out, want) < 1e-6


def test_scalar_norm_and_residual_update(backend):
    device, _ = backend
    cfg, w, eng = _engine_1layer(retention_layer(), backend)
    x = torch.randn(5, 32) * 3
    want = O.scalar_norm(x.double(), 1.3, cfg["norm"]["eps"])
    assert rel_err(eng.norm(x.to(device), 1.3, F32), want) < 1e-6
    assert rel_err(eng.norm(x.to(device), 1.3, BF16), want) < 1e-2
    acc = torch.ones(5, 32, device=device)
    eng.norm(x.to(device), 1.3, accum=acc)
    assert rel_err(acc, want + 1) < 1e-6
    # eps inside the root: an all-zero row stays zero instead of dividing by zero
    assert float(eng.norm(torch.zeros(2, 32, device=device), 2.0, F32).abs().max()) == 0.0


def test_rotary_table_with_rescaling():
    for dims, base, sc in ((4, 5000.0, dict(factor=4.0, original=64, fast=16.0, slow=1.0)), (16, 1e4, None),
                           (32, 1e6, dict(factor=8.0, original=512, fast=32.0, slow=2.0))):
        rot = {"dims": dims, "base": base}
        if sc:
            rot["scaling"] = sc
        f, mag = rotary_table(RotaryConfig(dims=dims, base=base, scaling=YarnScaling(**sc) if sc else None))
        want_f, want_mag = O.rotary_frequencies(rot)
        assert torch.allclose(f.double(), want_f, rtol=1e-6, atol=0) and abs(mag - want_mag) < 1e-12
        if sc:      # the lowest frequency is fully rescaled, the highest is not touched
            assert abs(float(f[0]) - 1.0) < 1e-6 and abs(float(f[-1]) * sc["factor"] / base ** (-(dims - 2) / dims) - 1) < 1e-5


@pytest.mark.parametrize("layer", [retention_layer(), retention_layer(heads=1, dim=6, vdim=40, rot_dims=6, decay=(0.999,)),
                                   latent_layer(), latent_layer(heads=3, dim=2, rot_dim=6, vdim=3, kv_rank=40, window=3, scaling=False),
                                   latent_layer(window=None), latent_layer(heads=2, dim=2, rot_dim=36, vdim=3, kv_rank=8, window=4)],
                         ids=["retention", "retention-wide-v", "latent", "latent-rank40-w3", "latent-no-window", "latent-rot-wider-than-rank"])
def test_mixer_alone_prefill_and_decode(backend, layer):
    """one mixer between its norms, no feed-forward: a whole prompt (several retention chunks / windows), then token by token"""
    cfg, w, eng = _engine_1layer(layer, backend)
    toks = _tokens(41, cfg["vocab"], seed=3)
    want = O.forward(cfg, w, toks)
    got = eng.step([StepEntry("p", toks[:37], list(range(37)))])
    assert rel_err(got, want[:37]) < TOL["float32"]
    for t in range(37, 41):
        got = eng.step([StepEntry("p", [toks[t]], [0])])
        assert rel_err(got, want[t:t + 1]) < TOL["float32"], t


def test_router_choices_and_weights(backend):
    device, lib = backend
    cfg, w, eng = _engine_1layer(retention_layer(mlp=moe(experts=8, top=3, groups=4, keep=2, ff=4, shared=6)), backend)
    f, lw = eng.cfg.layers[0].ff, eng.w.layers[0]
    # negative choice scores everywhere: an excluded group must count as minus infinity, not as zero
    lw["correction"] = lw["correction"] - 2.0
    w = dict(w)
    w["l0.mlp.correction"] = (w["l0.mlp.correction"].float() - 2.0)
    h = torch.randn(9, 32)
    idx = torch.zeros(9, 3, dtype=torch.int32, device=device)
    wt = torch.zeros(9, 3, device=device)
    gate = torch.zeros(9, device=device)
    L = eng.L
    rc = L.lp_moe_route(_lib.ptr(h.to(device)), 32, 1, 9, 32, _lib.ptr(lw["w_router"]), 32, 8, _lib.ptr(lw["correction"]), 4, 2, 3,
                        _lib.ptr(lw["w_sg"]), _lib.ptr(idx), _lib.ptr(wt), _lib.ptr(gate), eng._stream())
    assert rc == 0
    wd = {k: v.double() for k, v in w.items()}
    chosen, weights = O.route(h.double(), wd, "l0.mlp.", cfg["layers"][0]["mlp"]["router"])
    assert idx.cpu().tolist() == chosen
    assert rel_err(wt, weights) < 1e-5
    assert rel_err(gate, torch.sigmoid(h.double() @ wd["l0.mlp.shared.sg"].reshape(-1))) < 1e-5
    for row in chosen:                     # never more than the kept groups
        assert len({e // 2 for e in row}) <= 2


@pytest.mark.parametrize("T", [1, 5, 70])
@pytest.mark.parametrize("ff", [moe(), moe(experts=4, top=1, groups=1, keep=1, ff=6, shared=0), dense(ff=9)], ids=["moe", "moe-top1", "dense"])
def test_feed_forward_alone(backend, T, ff):
    device, _ = backend
    cfg, w, eng = _engine_1layer(retention_layer(mlp=ff), backend)
    h = torch.randn(T, 32)
    want = O.feed_forward(h.double(), {k: v.double() for k, v in w.items()}, "l0.mlp.", ff)
    f, lw = eng.cfg.layers[0].ff, eng.w.layers[0]
    got = eng._dense(f, lw, h.to(device)) if ff["kind"] == "dense" else eng._moe(f, lw, h.to(device))
    assert rel_err(got, want) < 1e-5


@pytest.mark.gpu
def test_large_bf16_products_run_on_the_tensor_cores():
    """in the serving precision a product of 64 rows or more goes to the tcgen05 GEMM; same result as the fp32-FMA kernels up to
    the rounding of the accumulation order, ragged N and K included, with and without an epilogue"""
    cfg = model([retention_layer()])
    w = O.random_weights(cfg, seed=2)
    eng = make_engine(cfg, w, ("cuda", None), "bfloat16")
    assert eng.tensor_core_rows == 64
    g = torch.Generator().manual_seed(5)
    for M, N, K in ((64, 128, 64), (130, 128, 64), (333, 328, 136), (1000, 784, 320)):
        a = torch.randn(M, K, generator=g).to(BF16).cuda()
        wt = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(BF16).cuda()
        want = a.double() @ wt.double().T
        assert eng._on_tensor_cores(a, wt, M, N, K)
        for c_dt, tol in ((F32, 1e-5), (BF16, 1e-2)):
            assert rel_err(eng.linear(a, wt, c_dt), want) < tol, (M, N, K, c_dt)
        gate, up = want[:, : N // 2], want[:, N // 2:]
        assert rel_err(eng.linear(a, wt, F32, _lib.EPI_SILU_GATE), gate * torch.sigmoid(gate) * up) < 1e-5
        eng.tensor_core_rows = None                 # the same call on the fp32-FMA kernel
        assert rel_err(eng.linear(a, wt, F32), want) < 1e-5
        eng.tensor_core_rows = 64
