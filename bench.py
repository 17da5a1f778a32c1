#!/usr/bin/env python3
"""Headline benchmark: decode tokens per second (and prefill of 2,048 tokens) at the layer
sizes of Qwen2.5-7B with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  The default run is a
batch of 8 sequences with 2,048-token prompts in a 4,096-token context; decode at batch 1 and
64 goes into "points".  `value` is timed on the device with CUDA events around K steps of the
engine's decode loop; `e2e` is the same loop driven through the Python entry point with the
step's token ids copied from pinned host memory and the new ids read back every step.
The decode step reads every weight once (14 GB, far above the 126 MB L2), so no L2 flush is
needed between steps; `config` says so.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Layer sizes of Qwen2.5-7B (the benchmark configuration).
QWEN25_7B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=3584,
                 num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
                 intermediate_size=18944, vocab_size=152064, rope_theta=1000000.0,
                 rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False,
                 max_position_embeddings=32768)
PROMPT_LEN, CONTEXT = 2048, 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        def find(d, key):
            """The number under `key`, at the top or one dictionary down."""
            if isinstance(d, dict):
                if isinstance(d.get(key), (int, float)):
                    return float(d[key])
                for v in d.values():
                    if isinstance(v, dict) and isinstance(v.get(key), (int, float)):
                        return float(v[key])
            raise KeyError(key)
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": find(d, "hbm_gbs"), "bf16_tflops": find(d, "bf16_tflops"),
                    "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples the SM clock and the throttle reasons (read-only NVML queries) every 50 ms while
    a timed region runs."""
    REASONS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20,
               "hw_thermal_slowdown": 0x40}

    def __init__(self):
        self.samples, self.max_mhz, self._stop, self._thread = [], None, None, None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:
            return self
        self._stop = threading.Event()

        def poll():
            while not self._stop.is_set():
                try:
                    mhz = int(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                    try:
                        why = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                    except Exception:
                        why = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                    self.samples.append((mhz, why))
                except Exception:
                    pass
                self._stop.wait(0.05)
        self._thread = threading.Thread(target=poll, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._stop is not None:
            self._stop.set()
            self._thread.join(timeout=2)

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples"]}
        mhz = sorted(m for m, _ in self.samples)
        reasons = [n for n, bit in self.REASONS.items() if any(w & bit for _, w in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(self.samples)}


def reference_arm() -> int:
    """The reference is a CMake/C++ project (no Python package): it cannot be installed with
    pip, needs its MLIR submodule and GGUF model files to build, and serves one sequence of
    quantized weights at a time."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "hardenedlinux/SonicBoom has no pip-installable package (pip install of the "
                      "source tree fails: no setup.py/pyproject.toml); its build needs the empty "
                      "third_party/llvm-project submodule and GGUF model files"}))
    return 0


def weight_bytes(model) -> int:
    seen, total = set(), 0
    def add(t):
        nonlocal total
        if t is not None and t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    for b in model.blocks:
        for part in b.parts:
            for v in vars(part).values():
                if hasattr(v, "data_ptr"):
                    add(v)
    add(model.final_norm.weight)
    add(model.head)                       # the embedding table is read for B rows only
    return total


def decode_flops_per_token(cfg) -> float:
    d, ff = cfg["hidden_size"], cfg["intermediate_size"]
    qw = cfg["num_attention_heads"] * (d // cfg["num_attention_heads"])
    kvw = cfg["num_key_value_heads"] * (d // cfg["num_attention_heads"])
    per_layer = 2 * d * (qw + 2 * kvw) + 2 * qw * d + 2 * d * 2 * ff + 2 * ff * d
    return per_layer * cfg["num_hidden_layers"]


def run(args) -> int:
    import torch
    import sonicboom_b200 as sb
    from sonicboom_b200.engine.decode import DecodeLoop
    from sonicboom_b200 import llm, ops

    torch.cuda.set_device(0)
    dev = "cuda:0"
    cfg = dict(QWEN25_7B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    t0 = time.time()
    model = sb.random_model(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    wbytes = weight_bytes(model)
    kv_bytes_per_token = sum(g.bytes_per_token() for g in
                             sb.Engine(model, max_tokens=64).cache.groups)
    gen = torch.Generator().manual_seed(1)

    def prompts(n):
        return [torch.randint(0, cfg["vocab_size"], (PROMPT_LEN,), generator=gen).tolist()
                for _ in range(n)]

    def decode_point(batch, steps, warmup, clocks=None, graph=True):
        """Prefills `batch` prompts (8 at a time), then times `steps` steps of the decode loop
        on the device with CUDA events."""
        engine = sb.Engine(model, max_tokens=batch * CONTEXT, n_slots=batch)
        slots = [engine.open() for _ in range(batch)]
        ps = prompts(batch)
        first = []
        for i in range(0, batch, 8):
            lg = engine.step([(s, p, [len(p) - 1]) for s, p in zip(slots[i:i + 8], ps[i:i + 8])])
            first += lg.argmax(dim=-1).tolist()
        # The sequences decode from 2,048 to 4,096 positions; the timed steps are the ones
        # around the middle of that stretch.  Instead of decoding every token up to there, the
        # sequences' lengths are moved forward (the skipped positions hold zeros in the cache;
        # a step reads the same bytes either way).
        skip = max(0, (CONTEXT + PROMPT_LEN) // 2 - (warmup + steps) // 2 - PROMPT_LEN)
        skip = min(skip, CONTEXT - PROMPT_LEN - (warmup + steps + 2))
        for s in slots:
            engine.cache.reserve(s, PROMPT_LEN + skip)
            engine.cache.advance(s, PROMPT_LEN + skip)
        loop = DecodeLoop(engine, slots, warmup + steps + 2, use_graph=graph)
        loop.run_device(first, warmup)
        torch.cuda.synchronize()
        ctx_start = engine.length(slots[0]) + warmup
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if clocks is not None:
            clocks.__enter__()
        start.record()
        loop.run_device(None, steps)
        end.record()
        torch.cuda.synchronize()
        if clocks is not None:
            clocks.__exit__()
        ms = start.elapsed_time(end)
        launches = loop.launches_per_step * steps
        loop.close()
        for s in slots:
            engine.close(s)
        del engine, loop
        torch.cuda.empty_cache()
        return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
                "bytes_per_step": wbytes + batch * (ctx_start + steps / 2.0) * kv_bytes_per_token}

    def e2e_point(batch, steps, warmup):
        """The same through the Python entry point: host token ids in, host token ids out.
        generate_batch prefills the prompts and runs the decode loop; every step copies the
        step's ids from pinned host memory and reads the new ids back.  The time between
        the callbacks of token `warmup` and token `warmup + steps` is what is reported."""
        engine = sb.Engine(model, max_tokens=batch * CONTEXT, n_slots=batch)
        stamps = []

        def on_token(i, tok):
            if i == 0:
                stamps.append(time.perf_counter())
            return 0
        # decode from 2,048 up to the same stretch around position 3072 that `value` times
        first = (CONTEXT - PROMPT_LEN) // 2 - steps // 2
        outs = llm.generate_batch(llm.Model(model), prompts(batch), max_tokens=first + steps + 1,
                                  ignore_eos=True, engine=engine, on_token=on_token, max_batch=batch)
        assert all(len(o) == first + steps + 1 for o in outs)
        dt = stamps[first + steps] - stamps[first]
        del engine
        torch.cuda.empty_cache()
        return {"tok_s": batch * steps / dt, "h2d": 4 * batch, "d2h": 4 * batch}

    if args.only == "decode":
        # a small case for profilers: the decode point alone (with --eager: kernel by kernel)
        r = decode_point(args.batch, args.steps, args.warmup, graph=not args.eager)
        print(json.dumps({"only": "decode", "layers": cfg["num_hidden_layers"], "batch": args.batch,
                          "ms_per_step": round(r["ms_per_step"], 4), "tok_s": round(r["tok_s"], 1)}))
        return 0

    # prefill of one 2,048-token prompt
    engine = sb.Engine(model, max_tokens=PROMPT_LEN, n_slots=1)
    (p,) = prompts(1)
    times = []
    for i in range(1 + args.prefill_reps):
        s = engine.open()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([(s, p, [PROMPT_LEN - 1])])
        end.record()
        torch.cuda.synchronize()
        engine.close(s)
        if i > 0:
            times.append(start.elapsed_time(end))
    prefill_ms = sorted(times)[len(times) // 2]
    hd = cfg["hidden_size"] // cfg["num_attention_heads"]
    prefill_flops = PROMPT_LEN * decode_flops_per_token(cfg) + \
        cfg["num_hidden_layers"] * 4 * cfg["num_attention_heads"] * hd * PROMPT_LEN * PROMPT_LEN / 2 + \
        2 * cfg["hidden_size"] * cfg["vocab_size"]
    del engine
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "layers": cfg["num_hidden_layers"], "tokens": PROMPT_LEN,
                          "ms": round(prefill_ms, 3)}))
        return 0

    clocks = ClockSampler()
    main = decode_point(args.batch, args.steps, args.warmup, clocks=clocks)
    e2e = e2e_point(args.batch, args.steps, args.warmup)
    points = {}
    for b in (1, 64):
        points[f"decode_b{b}"] = round(decode_point(b, args.steps, args.warmup)["tok_s"], 1)
    achieved = main["bytes_per_step"] / (main["ms_per_step"] / 1e3) / 1e9
    out = {
        "metric": "decode tok/s at batch 8 (Qwen2.5-7B sizes, 2,048-token prompts, context 4,096)",
        "value": round(main["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights, uniform random token ids", "impl": "ours",
        "config": {"model": "Qwen2.5-7B sizes", "layers": cfg["num_hidden_layers"],
                   "layers_full_model": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": hd, "intermediate": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "global_batch": args.batch, "seq_len": CONTEXT,
                   "prompt_len": PROMPT_LEN, "parallelism": "none (1 GPU)",
                   "decode_positions": "timed steps centred on position 3072 of 2048..4096",
                   "l2": "inputs larger than L2 (weights read once per step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tok/s",
                "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": int(main["launches"]),
        "clocks": clocks.summary(),
        "prefill": {"value": round(PROMPT_LEN / (prefill_ms / 1e3), 1), "tokens": PROMPT_LEN,
                    "ms": round(prefill_ms, 3),
                    "frac": round(prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "load_s": round(load_s, 1),
    }
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the model has (both numbers go into config)")
    ap.add_argument("--prefill-reps", type=int, default=3)
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one phase only and print a short line (small cases for profilers)")
    ap.add_argument("--eager", action="store_true",
                    help="with --only decode: launch the step kernel by kernel, not as a graph")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        print("bench.py: this library runs on one GPU; --gpus N with N > 1 is not built")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    return run(args)


if __name__ == "__main__":
    sys.exit(main())
