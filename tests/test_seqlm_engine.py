"""The step engine of the layer-list language models against the plain implementation (oracle/seqlm.py): whole prompts, token-by-token
decoding through cache and state, prompts cut into portions, batches of unequal requests, pages and slots that are given back and
taken again, keys at the edges of a sliding window and of cache pages, a far token that only a slow decay keeps alive, sizes that
happen to be one, both precisions, and greedy generation through the scheduler and the command line.  On the kernel sources under
the CPU emulator and, marked gpu, on the native library."""
import json

import pytest
import torch

from leopard_b200 import zudalorn
from leopard_b200.scheduler import Request, Scheduler, generate
from leopard_b200.seqlm import StepEntry
from oracle import seqlm as O
from seqlm_common import (TOL, backend, emu_lib, latent_layer, make_engine, mixed_model, model, plain_model,  # noqa: F401  (fixtures)
                          rel_err, retention_layer)


def _tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def _all(n):
    return list(range(n))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_decoding(backend, dtype):
    """whole prompt in one step, then 12 tokens one by one: past the window (5) and over three page borders (pages of 4)"""
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=11)
    toks = _tokens(22, cfg["vocab"], seed=1)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend, dtype)
    got = [eng.step([StepEntry("r", toks[:10], _all(10))])]
    for t in range(10, 22):
        got.append(eng.step([StepEntry("r", [toks[t]], [0])]))
    got = torch.cat(got, 0)
    assert rel_err(got, want) < TOL[dtype]
    if dtype == "float32":           # no position stands out: the first tokens, the window's edge and page borders included
        per_row = (got.double().cpu() - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()
        assert float(per_row.max()) < 10 * TOL[dtype], per_row


@pytest.mark.parametrize("cuts", [(2, 2, 3, 9, 2), (7, 11), (1, 17)])
def test_portions_of_a_prompt(backend, cuts):
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=12)
    toks = _tokens(sum(cuts), cfg["vocab"], seed=2)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend)
    got, at = [], 0
    for n in cuts:
        got.append(eng.step([StepEntry("r", toks[at:at + n], _all(n))]))
        at += n
    assert rel_err(torch.cat(got, 0), want) < TOL["float32"]


def test_batch_of_unequal_requests_and_reuse(backend):
    """three requests of different lengths in one batch, decoded together while the short ones end; then a new request takes the
    pages and the slot that were given back (the pool is sized so that it must)"""
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=13)
    lens = {"a": (1, 3), "b": (9, 6), "c": (14, 2)}            # prompt length, decoded tokens
    toks = {k: _tokens(p + d, cfg["vocab"], seed=30 + i) for i, (k, (p, d)) in enumerate(lens.items())}
    want = {k: O.forward(cfg, w, toks[k]) for k in lens}
    eng = make_engine(cfg, w, backend, max_tokens=8, max_seqs=3)
    got = {k: [] for k in lens}
    out = eng.step([StepEntry(k, toks[k][:p], [p - 1]) for k, (p, d) in lens.items()])
    for i, k in enumerate(lens):
        got[k].append(out[i:i + 1])
    live = list(lens)
    for step in range(6):
        live = [k for k in live if step < lens[k][1]]
        out = eng.step([StepEntry(k, [toks[k][lens[k][0] + step]], [0]) for k in live])
        for i, k in enumerate(live):
            got[k].append(out[i:i + 1])
        for k in live:
            if step + 1 == lens[k][1]:
                eng.finish(k)
    for k, (p, d) in lens.items():
        assert rel_err(torch.cat(got[k], 0), want[k][p - 1:]) < TOL["float32"], k
    assert eng.cache.pages_in_use() == 0 and len(eng.cache.free_slots) == eng.cache.n_slots
    slots_before, pages_before = eng.cache.n_slots, eng.cache.n_pages
    t2 = _tokens(13, cfg["vocab"], seed=77)
    again = eng.step([StepEntry("a", t2, _all(13))])           # the name of an ended request, a used slot, used pages
    assert rel_err(again, O.forward(cfg, w, t2)) < TOL["float32"]
    assert (eng.cache.n_slots, eng.cache.n_pages) == (slots_before, pages_before)


def test_window_pages_are_given_back_while_running(backend):
    cfg = model([latent_layer(window=5, mlp=None)])
    w = O.random_weights(cfg, seed=14)
    toks = _tokens(30, cfg["vocab"], seed=4)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend, max_tokens=12, max_seqs=1)
    pages = eng.cache.n_pages
    got = [eng.step([StepEntry("r", toks[:6], _all(6))])]
    for t in range(6, 30):
        got.append(eng.step([StepEntry("r", [toks[t]], [0])]))
        assert eng.cache.pages_in_use() <= 3                  # a window of 5 rows touches at most 3 pages of 4
    assert rel_err(torch.cat(got, 0), want) < TOL["float32"]
    assert eng.cache.n_pages == pages                          # the pool never had to grow


@pytest.mark.parametrize("mode", ["prompt", "decoded"])
def test_window_edge_with_a_key_that_stands_out(backend, mode):
    """One token's latent is made large (its embedding row is scaled), so wherever it is visible it takes most of the softmax: a
    window that is one position too long or too short changes the logits at the edge by far more than the tolerance."""
    W, loud_at = 6, 3
    cfg = model([latent_layer(heads=2, dim=6, rot_dim=4, vdim=5, kv_rank=12, window=W, mlp=None)], vocab=40)
    w = O.random_weights(cfg, seed=15)
    w["embed"][39] = (w["embed"][39].float() * 6).to(torch.bfloat16)
    w["l0.mix.dkv.norm"] = (w["l0.mix.dkv.norm"].float() * 3).to(torch.bfloat16)
    toks = _tokens(14, 39, seed=5)
    toks[loud_at] = 39
    want = O.forward(cfg, w, toks)
    quiet = list(toks)
    quiet[loud_at] = 0
    other = O.forward(cfg, w, quiet)
    last_in, first_out = loud_at + W - 1, loud_at + W
    # the loud key matters at the last position that sees it, and the position after it does not see it at all
    assert rel_err(other[last_in], want[last_in]) > 0.05
    eng = make_engine(cfg, w, backend)
    if mode == "prompt":
        got = eng.step([StepEntry("r", toks, _all(14))])
    else:
        got = [eng.step([StepEntry("r", toks[:5], _all(5))])] + [eng.step([StepEntry("r", [t], [0])]) for t in toks[5:]]
        got = torch.cat(got, 0)
    for p in (last_in, first_out):
        assert rel_err(got[p], want[p]) < TOL["float32"], p
    eng_q = make_engine(cfg, w, backend)
    got_q = eng_q.step([StepEntry("r", quiet, [first_out])])
    assert rel_err(got[first_out], got_q[0]) < TOL["float32"]       # out of the window: as if it had never been there


def test_far_token_kept_by_a_slow_decay(backend):
    """retention with decay 0.999 on one head: a scaled token 150 positions back still shapes the output; it crosses five chunks
    of the chunked prompt kernel and then the decode kernel"""
    cfg = model([retention_layer(heads=2, dim=4, vdim=4, rot_dims=4, decay=(0.999, 0.5), mlp=None)], vocab=30)
    w = O.random_weights(cfg, seed=16)
    w["embed"][29] = (w["embed"][29].float() * 8).to(torch.bfloat16)
    toks = _tokens(160, 29, seed=6)
    toks[4] = 29
    want = O.forward(cfg, w, toks)
    quiet = list(toks)
    quiet[4] = 1
    assert rel_err(O.forward(cfg, w, quiet)[155:], want[155:]) > 0.01      # a thousand times the tolerance
    eng = make_engine(cfg, w, backend, max_tokens=200)
    got = [eng.step([StepEntry("r", toks[:150], [149])])] + [eng.step([StepEntry("r", [t], [0])]) for t in toks[150:]]
    assert rel_err(torch.cat(got, 0), want[149:]) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_one(backend, dtype):
    cfg = plain_model()
    w = O.random_weights(cfg, seed=17)
    del w["l0.mlp.correction"]                     # a router without a choice bias
    toks = _tokens(11, cfg["vocab"], seed=7)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend, dtype)
    got = torch.cat([eng.step([StepEntry("r", toks[:7], _all(7))])] + [eng.step([StepEntry("r", [t], [0])]) for t in toks[7:]], 0)
    assert rel_err(got, want) < TOL[dtype]


def test_greedy_generation_through_the_scheduler(backend):
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=18)
    prompts = [_tokens(n, cfg["vocab"], seed=40 + n) for n in (3, 8, 1)]
    eng = make_engine(cfg, w, backend, max_seqs=2)
    outs = generate(eng, prompts, max_new_tokens=5)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for t in o:                                   # every generated token is the oracle's arg-max given what came before
            lg = O.forward(cfg, w, seq)[-1]
            top2 = lg.topk(2).values
            assert int(lg.argmax()) == t or float(top2[0] - top2[1]) < 1e-3
            seq.append(t)
        assert len(o) == 5
    assert eng.cache.pages_in_use() == 0
    # an end-of-sequence id stops a request and frees what it held; a waiting request is admitted later
    sched = Scheduler(eng, max_running=1)
    first = outs[0][0]
    sched.add(Request("x", prompts[0], max_new_tokens=5, eos={first}))
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
    w = O.random_weights(cfg, seed=19)
    (tmp_path / "m").mkdir()
    (tmp_path / "m/config.json").write_text(json.dumps(cfg))
    save_file(w, tmp_path / "m/model.safetensors")
    toks = _tokens(9, cfg["vocab"], seed=8)
    r = subprocess.run([sys.executable, "-m", "leopard_b200", "generate", "--model", str(tmp_path / "m"), "--dtype", "float32", "--prompt",
                        ",".join(map(str, toks)), "--max-new-tokens", "3"], cwd=root, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])["output"]
    assert out[0] == int(O.forward(cfg, w, toks)[-1].argmax())
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": toks[:6], "want": [0, 5]}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": toks[6:7], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "q", "tokens": toks[7:8], "want": [0]}], "end": ["q"]}]
    r = subprocess.run([str(root / "bin/trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32", "--out", str(tmp_path / "o"),
                        "--max-tokens", "64"], input="\n".join(map(json.dumps, steps)) + "\n", cwd=root, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = O.forward(cfg, w, toks)
    got0 = torch.from_numpy(np.fromfile(tmp_path / "o/0.f32", dtype="<f4").reshape(2, -1))
    got2 = torch.from_numpy(np.fromfile(tmp_path / "o/2.f32", dtype="<f4").reshape(1, -1))
    assert rel_err(got0, want[[0, 5]]) < TOL["float32"] and rel_err(got2, want[7:8]) < TOL["float32"]
    assert not (tmp_path / "o/1.f32").exists()


def test_registry_and_config_reader(tmp_path):
    from leopard_b200 import registry
    from leopard_b200.seqlm import LatentAttentionConfig, MoEConfig, RetentionConfig
    assert "Zudalorn" in registry.architectures()
    cfg = zudalorn.config_from_dict(mixed_model())
    assert isinstance(cfg.layers[0].mixer, RetentionConfig) and cfg.layers[0].mixer.rot.layout == "half"
    lat = cfg.layers[1].mixer
    assert isinstance(lat, LatentAttentionConfig) and lat.window == 5 and lat.rot.layout == "interleaved" and lat.rot.scaling.factor == 4.0
    assert isinstance(cfg.layers[1].ff, MoEConfig) and cfg.layers[1].ff.shared_ff == 10 and cfg.layers[2].ff is None
    with pytest.raises(ValueError):
        zudalorn.config_from_dict({"architecture": "other"})
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "nothing-known"}))
    with pytest.raises(KeyError):
        registry.load_model(tmp_path)
