"""Ronelorn on the step engine against the plain implementation (oracle/ronelorn.py): every mechanism alone, whole prompts against
token-by-token decoding, prompts cut into portions down to two tokens, batches of unequal requests, pages / summary pages / slots
that are given back and taken again, keys just inside and just outside the window, pooled blocks that are just seen or not yet, the
kept first tokens and the ones after them, page borders, the first tokens of a sequence, long decoding, sizes that happen to be equal
or one, both precisions, and greedy generation through the scheduler and the command line.  Where random weights would hide a wrong
key, the query / key norm gains are raised so that every softmax leans on few keys, and the test first shows on the oracle itself that
a window one token off would be noticed.  On the kernel sources under the CPU emulator and, marked gpu, on the native library."""
import copy
import json

import pytest
import torch

from leopard_b200 import ronelorn
from leopard_b200.scheduler import Request, Scheduler, generate
from leopard_b200.seqlm import StepEntry
from oracle import ronelorn as O
from ronelorn_common import (TOL, backend, dense, emu_lib, gru_layer, make_engine, mixed_model, model, pooled_layer,  # noqa: F401
                             rel_err, sink_layer)


def _tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def _all(n):
    return list(range(n))


def _rows(got, want):
    """relative error of every row"""
    got, want = got.double().cpu(), want.double()
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()


def _prompt_then_decode(eng, toks, n_prompt, key="r"):
    got = [eng.step([StepEntry(key, toks[:n_prompt], _all(n_prompt))])]
    for t in toks[n_prompt:]:
        got.append(eng.step([StepEntry(key, [t], [0])]))
    return torch.cat(got, 0)


LAYERS = {
    "pooled": pooled_layer(),
    "pooled, odd sizes": pooled_layer(heads=3, kv_heads=3, dim=6, vdim=10, window=4, pool=3, rot_dims=6, factor=None, softcap=None),
    "pooled, blocks of one": pooled_layer(heads=2, kv_heads=1, dim=4, vdim=4, window=3, pool=1, rot_dims=2),
    "pooled, heads of sixteen": pooled_layer(heads=4, kv_heads=1, dim=16, vdim=8, window=9, pool=4, rot_dims=8),
    "sink": sink_layer(),
    "sink, heads of sixteen": sink_layer(heads=2, kv_heads=1, dim=16, vdim=12, window=6, keep_first=2, rot_dims=16),
    "sink, nothing kept": sink_layer(heads=2, kv_heads=2, dim=4, vdim=6, window=6, keep_first=0, rot_dims=2),
    "sink, eight heads a group": sink_layer(heads=8, kv_heads=1, dim=4, vdim=4, window=4, keep_first=5, rot_dims=4),
    "mingru": gru_layer(),
    "mingru + squared relu": gru_layer(width=7, mlp=dense(9)),
}


@pytest.mark.parametrize("name", list(LAYERS))
def test_each_mechanism_alone(backend, name):
    """a one-layer model: the whole prompt in one step, and the same tokens with the last ones decoded through cache and state"""
    cfg = model([LAYERS[name]])
    w = O.random_weights(cfg, seed=3, sharp=2.0)
    toks = _tokens(14, cfg["vocab"], seed=1)
    res = []
    want = O.forward(cfg, w, toks, residuals=res)
    eng = make_engine(cfg, w, backend)
    taps = []
    eng.tap = lambda li, x: taps.append(x.clone())
    got = eng.step([StepEntry("p", toks, _all(14))])
    assert rel_err(taps[0], res[0]) < TOL["float32"]              # the residual stream after the layer
    assert float(_rows(got, want).max()) < 5 * TOL["float32"]
    eng.tap = None
    eng.finish("p")
    assert float(_rows(_prompt_then_decode(eng, toks, 8), want).max()) < 5 * TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_long_decoding(backend, dtype):
    """a prompt, then 15 tokens one by one (7 in the serving precision): past both windows, over many page borders, with blocks that
    complete while decoding"""
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=11)
    toks = _tokens(24 if dtype == "float32" else 16, cfg["vocab"], seed=2)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend, dtype)
    got = _prompt_then_decode(eng, toks, 9)
    assert rel_err(got, want) < TOL[dtype]
    if dtype == "float32":
        assert float(_rows(got, want).max()) < 5 * TOL[dtype]


@pytest.mark.parametrize("cuts", [(2, 2, 3, 9, 2, 4), (7, 15), (1, 2, 19)])
def test_portions_of_a_prompt(backend, cuts):
    """a prompt fed in portions: blocks that start in one portion and end in another, windows that reach into earlier portions"""
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=12, sharp=2.0)
    toks = _tokens(sum(cuts), cfg["vocab"], seed=3)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend)
    got, at = [], 0
    for n in cuts:
        got.append(eng.step([StepEntry("r", toks[at:at + n], _all(n))]))
        at += n
    assert float(_rows(torch.cat(got, 0), want).max()) < 5 * TOL["float32"]


def test_batch_of_unequal_requests_and_reuse(backend):
    """three requests of different lengths in one batch, decoded together while the short ones end; then a new request takes the
    pages, summary pages and slot that were given back (the pools are sized so that it must)"""
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=13)
    lens = {"a": (1, 3), "b": (11, 4), "c": (14, 2)}            # prompt length, decoded tokens
    toks = {k: _tokens(p + d, cfg["vocab"], seed=30 + i) for i, (k, (p, d)) in enumerate(lens.items())}
    want = {k: O.forward(cfg, w, toks[k]) for k in lens}
    eng = make_engine(cfg, w, backend, max_tokens=8, max_seqs=3)
    got = {k: [] for k in lens}
    out = eng.step([StepEntry(k, toks[k][:p], [p - 1]) for k, (p, d) in lens.items()])
    for i, k in enumerate(lens):
        got[k].append(out[i:i + 1])
    live = list(lens)
    for step in range(4):
        live = [k for k in live if step < lens[k][1]]
        out = eng.step([StepEntry(k, [toks[k][lens[k][0] + step]], [0]) for k in live])
        for i, k in enumerate(live):
            got[k].append(out[i:i + 1])
        for k in live:
            if step + 1 == lens[k][1]:
                eng.finish(k)
    for k, (p, d) in lens.items():
        assert float(_rows(torch.cat(got[k], 0), want[k][p - 1:]).max()) < 5 * TOL["float32"], k
    c = eng.cache
    assert c.pages_in_use() == 0 and len(c.free_slots) == c.n_slots and len(c.summary_free[0]) == c.summary_n_pages[0]
    before = (c.n_slots, c.n_pages, tuple(c.summary_n_pages))
    t2 = _tokens(15, cfg["vocab"], seed=77)
    again = eng.step([StepEntry("a", t2, _all(15))])           # the name of an ended request, a used slot, used pages
    assert float(_rows(again, O.forward(cfg, w, t2)).max()) < 5 * TOL["float32"]
    assert (c.n_slots, c.n_pages, tuple(c.summary_n_pages)) == before


def test_pages_given_back_while_running_and_kept_pages_stay(backend):
    """the window bounds the token pages a request holds, except the pages of the kept first tokens; summary pages stay; two pooled
    layers with different block sizes keep two summary page tables"""
    cfg = model([sink_layer(window=5, keep_first=3), pooled_layer(window=6, pool=2), pooled_layer(heads=2, kv_heads=2, window=4, pool=3)])
    w = O.random_weights(cfg, seed=14, sharp=2.0)
    toks = _tokens(25, cfg["vocab"], seed=4)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend, max_tokens=16, max_seqs=1)
    got = [eng.step([StepEntry("r", toks[:6], _all(6))])]
    for i, t in enumerate(toks[6:]):
        got.append(eng.step([StepEntry("r", [t], [0])]))
        seq = eng.cache.get("r")
        assert seq.pages[0] >= 0                             # tokens 0..2 live in page 0 for ever
        assert eng.cache.pages_in_use() <= 1 + 3             # one kept page + a window of 6 rows over pages of 4
    assert eng.cache.summary_every == [2, 3]
    assert [len(p) for p in eng.cache.get("r").summary_pages] == [-(-(25 // 2) // 4), -(-(25 // 3) // 4)]
    assert float(_rows(torch.cat(got, 0), want).max()) < 5 * TOL["float32"]


def _edited(layer, **mask):
    out = copy.deepcopy(layer)
    out["mixer"]["mask"].update(mask)
    return out


@pytest.mark.parametrize("mode", ["prompt", "decoded"])
@pytest.mark.parametrize("kind", ["window", "pool", "kept"])
def test_edges_of_what_is_visible(backend, mode, kind):
    """Sharp softmaxes (norm gains of 4): first the oracle itself shows that a window one token longer, blocks one token wider or one
    more kept token change rows by far more than the tolerance; then the engine matches the right oracle on EVERY row, so the last
    key inside and the first outside each edge are right at every position, in a prompt and when decoded one by one."""
    if kind == "kept":
        layer, wrong = sink_layer(window=4, keep_first=2), {"keep_first": 3}
    elif kind == "pool":
        layer, wrong = pooled_layer(window=5, pool=3, softcap=None), {"pool": 4}
    else:
        layer, wrong = pooled_layer(window=5, pool=3), {"size": 6}
    cfg = model([layer], residual_mult=1.0)
    w = O.random_weights(cfg, seed=15, sharp=4.0)
    toks = _tokens(20, cfg["vocab"], seed=5)
    want = O.forward(cfg, w, toks)
    off = O.forward(model([_edited(layer, **wrong)], residual_mult=1.0), w, toks)
    assert float(_rows(off, want).max()) > 200 * TOL["float32"]
    eng = make_engine(cfg, w, backend)
    got = eng.step([StepEntry("r", toks, _all(20))]) if mode == "prompt" else _prompt_then_decode(eng, toks, 3)
    assert float(_rows(got, want).max()) < 5 * TOL["float32"]


def test_a_far_key_that_stands_out(backend):
    """With large values and sharp scores one early token, 40 positions back and 10 pages away, still shapes the late rows: it reaches
    them only through its pooled block (pooled layer) or as a kept first token (sink layer), and it must."""
    for layer, at in ((pooled_layer(heads=2, kv_heads=1, window=6, pool=4, softcap=None), 5), (sink_layer(window=6, keep_first=3), 1)):
        cfg = model([layer], vocab=40, residual_mult=1.0)
        w = O.random_weights(cfg, seed=16, sharp=3.0)
        w["l0.mix.v"] = (w["l0.mix.v"].float() * 3).to(torch.bfloat16)
        toks = _tokens(46, 39, seed=6)
        toks[at] = 39
        quiet = list(toks)
        quiet[at] = 0
        want = O.forward(cfg, w, toks)
        assert float(_rows(O.forward(cfg, w, quiet)[40:], want[40:]).max()) > 100 * TOL["float32"]    # the far token matters there
        eng = make_engine(cfg, w, backend, max_tokens=64)
        got = [eng.step([StepEntry("r", toks[:41], [40])])] + [eng.step([StepEntry("r", [t], [0])]) for t in toks[41:]]
        assert float(_rows(torch.cat(got, 0), want[40:]).max()) < 5 * TOL["float32"]


def test_state_of_the_recurrence_over_chunks_and_slots(backend):
    """minGRU with update gates near zero keeps a token alive for long: a prompt over several scan chunks, fed in two portions, then
    decoded; a second request on a used slot starts from zero"""
    cfg = model([gru_layer(width=10)], vocab=30, residual_mult=1.0)
    w = O.random_weights(cfg, seed=17)
    w["l0.mix.z.b"] = torch.full((10,), -4.0).to(torch.bfloat16)
    toks = _tokens(86, 30, seed=7)
    want = O.forward(cfg, w, toks)
    other = list(toks)
    other[2] = (toks[2] + 1) % 30
    assert float(_rows(O.forward(cfg, w, other)[80:], want[80:]).max()) > 100 * TOL["float32"]
    eng = make_engine(cfg, w, backend, max_seqs=1)
    got = [eng.step([StepEntry("r", toks[:45], [44])]), eng.step([StepEntry("r", toks[45:80], [34])])]
    got += [eng.step([StepEntry("r", [t], [0])]) for t in toks[80:]]
    assert float(_rows(torch.cat(got, 0), want[[44] + list(range(79, 86))]).max()) < 5 * TOL["float32"]
    eng.finish("r")
    t2 = _tokens(5, 30, seed=8)
    assert float(_rows(eng.step([StepEntry("s", t2, _all(5))]), O.forward(cfg, w, t2)).max()) < 5 * TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_equal_or_one(backend, dtype):
    """one head, as many key heads as query heads, no window at all, a window longer than the sequence, no cap, no frequency scaling,
    no rotation, multipliers of one, an odd width"""
    cfg = model([pooled_layer(heads=1, kv_heads=1, dim=4, vdim=2, window=64, pool=2, rot_dims=0, factor=None, softcap=None, mlp=dense(5)),
                 sink_layer(heads=2, kv_heads=2, dim=2, vdim=2, window=None, keep_first=0, rot_dims=2),
                 gru_layer(width=1)], width=9, vocab=17, residual_mult=1.0, embed_scale=1.0)
    del cfg["embedding"], cfg["residual_mult"]
    w = O.random_weights(cfg, seed=18)
    toks = _tokens(13, cfg["vocab"], seed=9)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend, dtype)
    assert rel_err(_prompt_then_decode(eng, toks, 7), want) < TOL[dtype]


def test_greedy_generation_through_the_scheduler(backend):
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=19)
    prompts = [_tokens(n, cfg["vocab"], seed=40 + n) for n in (3, 9, 1)]
    eng = make_engine(cfg, w, backend, max_seqs=2)
    outs = generate(eng, prompts, max_new_tokens=3)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for t in o:                                   # every generated token is the oracle's arg-max given what came before
            lg = O.forward(cfg, w, seq)[-1]
            top2 = lg.topk(2).values
            assert int(lg.argmax()) == t or float(top2[0] - top2[1]) < 1e-3
            seq.append(t)
        assert len(o) == 3
    assert eng.cache.pages_in_use() == 0
    sched = Scheduler(eng, max_running=1)
    first = outs[0][0]
    sched.add(Request("x", prompts[0], max_new_tokens=3, eos={first}))
    sched.add(Request("y", prompts[1], max_new_tokens=2))
    done = sched.run()
    assert done["x"].output == [first] and done["y"].output == outs[1][:2]


@pytest.mark.gpu
def test_command_line_generate_and_trace(tmp_path):
    """the registry picks the loader from config.json; `generate` and `trace` run the same step engine"""
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    from leopard_b200.safetensors_io import save_file
    root = Path(__file__).resolve().parents[1]
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=20)
    (tmp_path / "m").mkdir()
    (tmp_path / "m/config.json").write_text(json.dumps(cfg))
    save_file(w, tmp_path / "m/model.safetensors")
    toks = _tokens(12, cfg["vocab"], seed=8)
    r = subprocess.run([sys.executable, "-m", "leopard_b200", "generate", "--model", str(tmp_path / "m"), "--dtype", "float32", "--prompt",
                        ",".join(map(str, toks)), "--max-new-tokens", "3"], cwd=root, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])["output"]
    assert out[0] == int(O.forward(cfg, w, toks)[-1].argmax())
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": toks[:9], "want": [0, 8]}, {"id": "s", "tokens": toks[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": toks[9:10], "want": []}, {"id": "s", "tokens": toks[2:3], "want": [0]}],
              "end": ["s"]},
             {"step": 2, "entries": [{"id": "q", "tokens": toks[10:11], "want": [0]}], "end": ["q"]}]
    for dtype in ("float32", "bfloat16"):
        r = subprocess.run([str(root / "bin/trace_run"), "--model", str(tmp_path / "m"), "--dtype", dtype, "--out", str(tmp_path / dtype),
                            "--max-tokens", "64"], input="\n".join(map(json.dumps, steps)) + "\n", cwd=root, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        want = O.forward(cfg, w, toks)
        got = [torch.from_numpy(np.fromfile(tmp_path / dtype / f"{i}.f32", dtype="<f4").reshape(n, -1)) for i, n in ((0, 2), (1, 1), (2, 1))]
        assert rel_err(got[0], want[[0, 8]]) < TOL[dtype] and rel_err(got[1], want[2:3]) < TOL[dtype]
        assert rel_err(got[2], want[10:11]) < TOL[dtype]


def test_registry_and_config_reader():
    from leopard_b200 import registry
    from leopard_b200.seqlm import DenseFFConfig, LinearScaling, MinGRUConfig, WindowAttentionConfig, rotary_table
    assert "Ronelorn" in registry.architectures()
    cfg = ronelorn.config_from_dict(mixed_model())
    assert (cfg.norm, cfg.residual_mult, cfg.embed_scale) == ("pre", 0.5, 3.0)
    a, b, c, d = cfg.layers
    assert isinstance(a.mixer, WindowAttentionConfig) and (a.mixer.qk_norm, a.mixer.window, a.mixer.pool, a.mixer.keep_first) == ("head", 7, 3, 0)
    assert a.mixer.softcap == 5.0 and not a.mixer.sink and a.mixer.value_rot.dims == a.mixer.vdim and a.mixer.value_rot.scaling is None
    assert a.mixer.rot.scaling == LinearScaling(2.0) and isinstance(a.ff, DenseFFConfig) and a.ff.act == "relu2"
    assert (b.mixer.qk_norm, b.mixer.keep_first, b.mixer.pool, b.mixer.sink, b.mixer.value_rot) == ("full", 3, 0, True, None)
    assert isinstance(c.mixer, MinGRUConfig) and c.ff is None and d.weights_of == 0 and a.weights_of is None
    f, mag = rotary_table(a.mixer.rot)
    assert mag == 1.0 and torch.allclose(f.double(), torch.tensor([1.0, 100.0 ** -0.5]).double() / 2.0, rtol=1e-7)
    with pytest.raises(ValueError):
        ronelorn.config_from_dict({"architecture": "other"})
    bad = mixed_model()
    bad["layers"][3]["mixer"]["mask"]["size"] = 9                # a layer that borrows weights must equal their owner
    with pytest.raises(ValueError):
        w = O.random_weights(mixed_model(), seed=1)
        ronelorn.from_state_dict(ronelorn.config_from_dict(bad), w, device="cpu", lib=object())
