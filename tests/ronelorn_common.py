"""Shared pieces of the Ronelorn tests: small configurations in the parsed-JSON form a checkpoint carries, and the engine builder for
the two backends of seqlm_common (kernel sources under the CPU emulator; the native library on a GPU)."""
import copy

from seqlm_common import BACKENDS, TOL, backend, emu_lib, rel_err  # noqa: F401  (fixtures)


def pooled_layer(heads=4, kv_heads=2, dim=8, vdim=8, window=7, pool=3, rot_dims=4, base=100.0, factor=2.0, softcap=5.0, scale=0.3,
                 mlp=None, weights_of=None):
    rot = {"base": base, "dims": rot_dims}
    if factor:
        rot["scaling"] = {"factor": factor}
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot,
             "mask": {"size": window, "pool": pool}}
    if softcap:
        mixer["softcap"] = softcap
    layer = {"type": "attention", "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def sink_layer(heads=4, kv_heads=1, dim=8, vdim=4, window=5, keep_first=3, rot_dims=8, base=50.0, scale=0.4, mlp=None, weights_of=None):
    layer = {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                              "rot": {"base": base, "dims": rot_dims}, "mask": {"size": window, "keep_first": keep_first}},
             "mlp": mlp}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def gru_layer(width=24, mlp=None, weights_of=None):
    layer = {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def dense(ff=28):
    return {"kind": "dense", "ff": ff}


def model(layers, width=20, vocab=53, eps=1e-5, residual_mult=0.5, embed_scale=3.0):
    return {"architecture": "Ronelorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": residual_mult,
            "embedding": {"scale": embed_scale}, "layers": copy.deepcopy(layers)}


def mixed_model():
    """every mixer, a layer without feed-forward, and a layer that runs on an earlier layer's weights"""
    return model([pooled_layer(mlp=dense()), sink_layer(mlp=dense(12)), gru_layer(), pooled_layer(mlp=dense(), weights_of=0)])


def make_engine(cfg: dict, weights: dict, backend, dtype="float32", **kw):
    from leopard_b200 import ronelorn
    device, lib = backend
    kw.setdefault("page_size", 4)
    kw.setdefault("max_tokens", 32)
    kw.setdefault("max_seqs", 2)
    return ronelorn.from_state_dict(ronelorn.config_from_dict(cfg), weights, dtype=dtype, device=device, lib=lib, **kw)
