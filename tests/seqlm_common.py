"""Shared pieces of the language-model tests: small configurations (the parsed-JSON form a Zudalorn checkpoint carries), the two
backends (the kernel sources under the CPU emulator; the native library on a GPU) and the error measure."""
import copy
import ctypes as C
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]

BACKENDS = ["emu", pytest.param("cuda", marks=pytest.mark.gpu)]


def retention_layer(heads=2, dim=8, vdim=4, rot_dims=4, decay=(0.9, 0.99), mlp=None, base=10000.0):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay),
                                           "rot": {"base": base, "dims": rot_dims}}, "mlp": mlp}


def latent_layer(heads=2, dim=6, rot_dim=4, vdim=5, kv_rank=12, window=5, scaling=True, mlp=None, base=5000.0):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": (dim + rot_dim) ** -0.5, "rot": rot}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def dense(ff=24):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, groups=3, keep=2, ff=8, shared=10):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def model(layers, width=32, vocab=61, eps=1e-5):
    return {"architecture": "Zudalorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}


def mixed_model():
    return model([retention_layer(mlp=dense()), latent_layer(mlp=moe()), retention_layer(heads=1, dim=4, vdim=6, rot_dims=2, decay=(0.97,))])


def plain_model():
    """sizes that happen to be 1 or equal: one head, top 1, one group, no shared expert, no window, no rescaling, width not a multiple of 8"""
    return model([latent_layer(heads=1, dim=4, rot_dim=2, vdim=4, kv_rank=7, window=None, scaling=False,
                               mlp=moe(experts=4, top=1, groups=1, keep=1, ff=6, shared=0)),
                  retention_layer(heads=1, dim=4, vdim=4, rot_dims=4, decay=(0.5,), mlp=dense(ff=9))], width=20, vocab=37, eps=1e-6)


@pytest.fixture(scope="session")
def emu_lib(tmp_path_factory):
    sys.path.insert(0, str(ROOT / "tests/emu"))
    from stream32_build import build_emulated
    from leopard_b200 import _lib
    return _lib.bind_stream32(C.CDLL(str(build_emulated(tmp_path_factory.mktemp("emu_stream32")))))


@pytest.fixture(params=BACKENDS)
def backend(request):
    """(device, library or None for the native one)"""
    if request.param == "emu":
        return "cpu", request.getfixturevalue("emu_lib")
    return "cuda", None


def make_engine(cfg: dict, weights: dict, backend, dtype="float32", **kw):
    from leopard_b200 import zudalorn
    device, lib = backend
    kw.setdefault("page_size", 4)
    kw.setdefault("max_tokens", 32)
    kw.setdefault("max_seqs", 2)
    return zudalorn.from_state_dict(zudalorn.config_from_dict(cfg), weights, dtype=dtype, device=device, lib=lib, **kw)


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    return float((got - want).pow(2).mean().sqrt() / (want.pow(2).mean().sqrt() + 1e-30))


TOL = {"float32": 2e-5, "bfloat16": 4e-2}
