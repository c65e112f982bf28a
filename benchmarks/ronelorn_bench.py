"""bench.py --workload ronelorn: prefill and decode throughput of the Ronelorn layers (pooled-window attention, sink-window attention,
minGRU, squared-relu feed-forward; leopard_b200/ronelorn.py) at a few sizes that resemble a real model's layers, beside the framework's
closest existing model, the Zudalorn stack of benchmarks/seqlm_bench.py, at the same width, head count, feed-forward size and vocabulary
on the same step engine.  Random weights, synthetic token ids, one GPU.

Per size: a 4-layer stack [pooled-window attention + dense, sink-window attention + dense, minGRU, pooled-window attention + dense on
layer 0's weights];
  prefill   one request of `prompt` tokens per step through SeqLMEngine.step (cache, summaries and state written), tokens/s;
  decode    `batch` running requests with 512 tokens of history advanced by one token per step, tokens/s, for batch 1, 8 and 64;
  kernels   device time per native entry point of one prefill step and one decode step (CUDA events around every call) and the rate
            each reaches against its ceiling: the fp32 FMA peak for the attention kernel (its scores, softmax and sums are fp32), the
            measured copy bandwidth for the recurrence, the projection prologue and the weight-streaming decode products, the measured
            cuBLAS bf16 peak for the tcgen05 GEMM.  The same figures of the Zudalorn stack's like kernels stand beside them.
One JSON line in the shape bench.py prints for its other workloads; `value` is the prefill throughput of the middle size.
"""
from __future__ import annotations

import json

import torch

from benchmarks.seqlm_bench import FP32_FMA_TFLOPS, HEAD, SIZES, TimedLib, _time, bench_size

POOL, KEEP = 64, 4


def ronelorn_config(s):
    H, G = s["heads"], max(s["heads"] // 4, 1)
    pooled = {"heads": H, "kv_heads": G, "dim": HEAD, "vdim": HEAD, "scale": HEAD ** -0.5, "softcap": 30.0,
              "rot": {"base": 1e6, "dims": 64, "scaling": {"factor": 4.0}}, "mask": {"size": s["window"], "pool": POOL}}
    sink = {"heads": H, "kv_heads": G, "dim": HEAD, "vdim": HEAD, "scale": HEAD ** -0.5, "rot": {"base": 1e6, "dims": 64},
            "mask": {"size": s["window"], "keep_first": KEEP}}
    dense = {"kind": "dense", "ff": s["ff"]}
    layers = [{"type": "attention", "mixer": pooled, "mlp": dense}, {"type": "attention_2", "mixer": sink, "mlp": dense},
              {"type": "mingru", "mixer": {"width": s["width"]}, "mlp": None},
              {"type": "attention", "mixer": pooled, "mlp": dense, "weights_of": 0}]
    return {"architecture": "Ronelorn", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "embedding": {"scale": s["width"] ** 0.5}, "layers": layers}


def random_getter(cfg, dev, seed=1):
    g = torch.Generator(device=dev).manual_seed(seed)
    D = cfg["width"]
    shapes = {"embed": (cfg["vocab"], D), "head": (cfg["vocab"], D), "final.norm": (D,)}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (D,)
        if layer["type"] == "mingru":
            for n in ("z", "x", "g"):
                shapes[p + "mix." + n] = (m["width"], D)
            shapes[p + "mix.z.b"] = shapes[p + "mix.x.b"] = (m["width"],)
            shapes[p + "mix.o"] = (D, m["width"])
        else:
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * d, D), p + "mix.k": (G * d, D), p + "mix.v": (G * e, D), p + "mix.o": (D, H * e)})
            full = layer["type"] == "attention_2"
            shapes[p + "mix.q.norm"], shapes[p + "mix.k.norm"] = ((H * d,), (G * d,)) if full else ((d,), (d,))
        if layer["mlp"] is not None:
            shapes.update({p + "norm2": (D,), p + "mlp.up": (layer["mlp"]["ff"], D), p + "mlp.down": (D, layer["mlp"]["ff"])})

    def get(name):
        shape = shapes[name]
        if len(shape) == 2:
            return (torch.randn(shape, device=dev, generator=g) * shape[1] ** -0.5).to(torch.bfloat16)
        if name.endswith(".q.norm") or name.endswith(".k.norm"):
            return (torch.rand(shape, device=dev, generator=g) * 0.5 + 0.75).to(torch.bfloat16)
        return ((torch.rand(shape, device=dev, generator=g) - 0.5) * 0.2).to(torch.bfloat16)
    return get


def visible(pos, window, keep=0, pool=0):
    """keys a query at `pos` reads"""
    lo = max(pos - window + 1, 0)
    return pos - lo + 1 + min(keep, lo) + (lo // pool if pool else 0)


def bench_ronelorn(name, s, dev, steps, warmup, peaks, prompt):
    from leopard_b200 import ronelorn
    from leopard_b200.seqlm import SeqLMEngine, SeqLMWeights, StepEntry
    cfg_d = ronelorn_config(s)
    cfg = ronelorn.config_from_dict(cfg_d)
    eng = SeqLMEngine(cfg, SeqLMWeights(cfg, random_getter(cfg_d, dev), ronelorn.tensor_name, dev), dtype="bfloat16",
                      max_tokens=64 * 600 + prompt, max_seqs=64)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, s["vocab"], (prompt,), generator=g).tolist()
    D, H, G, R, W = s["width"], s["heads"], max(s["heads"] // 4, 1), prompt, s["window"]
    out = {"size": name, "width": D, "heads": H, "kv_heads": G, "ff": s["ff"], "window": W, "pool": POOL, "keep_first": KEEP, "prompt": prompt}

    def prefill():
        eng.step([StepEntry("p", toks, [prompt - 1])])
        eng.finish("p")
    ms = _time(prefill, steps, warmup)
    out["prefill_ms"], out["prefill_tokens_per_s"] = round(ms, 3), round(prompt / ms * 1e3, 1)
    plain = eng.L
    eng.L = TimedLib(plain)
    prefill()
    kp = eng.L.collect()
    eng.L = plain
    qkv_n = (H + 2 * G) * HEAD
    flops_gemm = 3 * (2.0 * R * D * qkv_n + 2.0 * R * D * H * HEAD + 2 * 2.0 * R * D * s["ff"]) + 2.0 * R * D * 3 * D + 2.0 * R * D * D
    keys = 2 * sum(visible(p, W, pool=POOL) for p in range(R)) + sum(visible(p, W, keep=KEEP) for p in range(R))
    attn_flops = H * keys * 4.0 * HEAD
    gru_bytes = R * D * 4.0 * (2 + 3) + R * D * 2.0           # pass 1 reads z, x; pass 3 reads z, x, g and writes bf16
    prep_bytes = 3 * R * (qkv_n * 4.0 + H * HEAD * 4.0 + 2 * G * HEAD * 4.0)

    def per_s(key, amount, unit):
        return round(amount / (kp[key]["ms"] * 1e-3) / unit, 2) if key in kp and kp[key]["ms"] > 0 else None
    attn_key = "lp_window_attn_tiles" if "lp_window_attn_tiles" in kp else "lp_window_attn"      # prompts run the row-tile kernel
    r = {"lp_gemm_bf16_tflops": per_s("lp_gemm_bf16", flops_gemm, 1e12), "lp_window_attn_tflops": per_s(attn_key, attn_flops, 1e12),
         "lp_mingru_prefill_gbs": per_s("lp_mingru_prefill", gru_bytes, 1e9), "lp_window_attn_prep_gbs": per_s("lp_window_attn_prep", prep_bytes, 1e9)}
    r["lp_gemm_bf16_of_bf16_peak"] = round(r["lp_gemm_bf16_tflops"] / peaks["bf16_burst"], 3) if r["lp_gemm_bf16_tflops"] else None
    r["lp_window_attn_of_fp32_fma_peak"] = round(r["lp_window_attn_tflops"] / FP32_FMA_TFLOPS, 3) if r["lp_window_attn_tflops"] else None
    for k in ("lp_mingru_prefill", "lp_window_attn_prep"):
        r[k + "_of_copy_peak"] = round(r[k + "_gbs"] / peaks["hbm_gbs"], 3) if r[k + "_gbs"] else None
    out["prefill_kernels"], out["prefill_rates"] = kp, r
    out["decode"] = {}
    for batch in (1, 8, 64):
        keys_ = [("d", i) for i in range(batch)]
        eng.step([StepEntry(k, toks[:512], []) for k in keys_])
        nxt = [int(t) for t in torch.randint(0, s["vocab"], (batch,), generator=g)]

        def decode():
            eng.step([StepEntry(k, [t], [0]) for k, t in zip(keys_, nxt)])
        ms = _time(decode, steps, warmup)
        d = {"ms_per_step": round(ms, 3), "tokens_per_s": round(batch / ms * 1e3, 1)}
        if batch in (1, 8):
            eng.L, eng.use_graphs = TimedLib(plain), False      # the breakdown needs the launches one by one
            decode()
            kd = eng.L.collect()
            eng.L, eng.use_graphs = plain, True
            d["kernels"] = kd
            wbytes = 2.0 * (3 * (D * qkv_n + D * H * HEAD + 2 * D * s["ff"]) + 4 * D * D + D * s["vocab"])
            if "lp_linear" in kd:
                d["lp_linear_gbs"] = round(wbytes / (kd["lp_linear"]["ms"] * 1e-3) / 1e9, 1)
                d["lp_linear_of_copy_peak"] = round(d["lp_linear_gbs"] / peaks["hbm_gbs"], 3)
            # the rows of the cache one decode step reads: window (+ blocks, + kept tokens) x [keys | values] of every key head
            kv_bytes = batch * 4.0 * 2 * G * HEAD * (2 * visible(512, W, pool=POOL) + visible(512, W, keep=KEEP))
            if "lp_window_attn" in kd:
                d["lp_window_attn_gbs"] = round(kv_bytes / (kd["lp_window_attn"]["ms"] * 1e-3) / 1e9, 1)
        out["decode"][str(batch)] = d
        for k in keys_:
            eng.finish(k)
    del eng
    torch.cuda.empty_cache()
    return out


def run(args):
    import bench
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference has no model of this kind; the comparison arm of this "
                                                              "workload is the framework's own Zudalorn stack"}), flush=True)
        return 0
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: leopard_b200 has no CPU fallback")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = bench.load_peaks()
    from leopard_b200 import _lib
    L = _lib.stream32_lib()
    n0 = L.lp_launch_count()
    only = [x for x in (getattr(args, "seqlm_sizes", None) or "").split(",") if x]
    prompt, sizes, beside = 4096, [], []
    for name, s in SIZES.items():
        if only and name not in only:
            continue
        sizes.append(bench_ronelorn(name, s, dev, args.steps, max(args.warmup, 3), peaks, prompt))
        z = bench_size(name, s, dev, args.steps, max(args.warmup, 3), peaks, prompt)
        beside.append({k: z[k] for k in ("size", "prefill_ms", "prefill_tokens_per_s", "prefill_kernels", "prefill_rates", "decode")})
    mid = sizes[min(1, len(sizes) - 1)]
    line = {"metric": "ronelorn_prefill_tokens_per_s", "value": mid["prefill_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": mid["prefill_ms"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, random token ids)",
            "config": {"model": f"Ronelorn 4-layer stack, {mid['size']}", "global_batch": 1, "seq_len": prompt, "parallelism": "single GPU",
                       "cache_policy": "weights + activations of a step exceed L2 at every size"},
            "gpu_launches": int(L.lp_launch_count() - n0), "peaks": peaks, "fp32_fma_peak_tflops": round(FP32_FMA_TFLOPS, 1),
            "sizes": sizes, "zudalorn_stack": beside}
    print(json.dumps(line), flush=True)
    return 0
