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


QWEN25_1P5B = dict(QWEN25_7B, hidden_size=1536, num_attention_heads=12, num_key_value_heads=2,
                   intermediate_size=8960, vocab_size=151936, tie_word_embeddings=True)
QWEN25_32B = dict(QWEN25_7B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=40,
                  num_key_value_heads=8, intermediate_size=27648)
REPETITIONS = 3       # timed regions of K steps each; the median is reported


def run(args) -> int:
    import torch
    import sonicboom_b200 as sb
    from sonicboom_b200.engine.decode import DecodeLoop
    from sonicboom_b200 import llm, ops
    from sonicboom_b200.sampling import Sampling

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
    gen = torch.Generator().manual_seed(1)

    def kv_bytes_per_token(m):
        return sum(g.bytes_per_token() for g in sb.Engine(m, max_tokens=64).cache.groups)

    def prompts(n, length=PROMPT_LEN, vocab=None):
        return [torch.randint(0, vocab or cfg["vocab_size"], (length,), generator=gen).tolist()
                for _ in range(n)]

    def decode_point(m, batch, steps, warmup, clocks=None, graph=True, prompt_len=PROMPT_LEN,
                     context=CONTEXT, real_prompt=None, reps=REPETITIONS):
        """Prefills `batch` prompts (8 at a time), then times regions of `steps` steps of the
        decode loop on the device with CUDA events: after `warmup` steps and one untimed region,
        `reps` regions back to back; the median region is the result.
        The sequences decode from prompt_len to context positions; the timed steps are the ones
        around the middle of that stretch.  Instead of decoding every token up to there, the
        sequences' lengths are moved forward (the skipped positions hold zeros in the cache; a
        step reads the same bytes either way).  `real_prompt` < prompt_len prefills only that
        many tokens of each prompt and moves the lengths forward over the rest as well."""
        real = real_prompt or prompt_len
        engine = sb.Engine(m, max_tokens=batch * context, n_slots=batch)
        slots = [engine.open() for _ in range(batch)]
        ps = prompts(batch, real, m.spec.vocab)
        first = []
        for i in range(0, batch, 8):
            lg = engine.step([(s, p, [len(p) - 1]) for s, p in zip(slots[i:i + 8], ps[i:i + 8])])
            first += lg.argmax(dim=-1).tolist()
        room = context - prompt_len
        reps = max(1, min(reps, (room - warmup - 2) // steps - 1))
        total = warmup + (reps + 1) * steps
        skip = max(0, min((context + prompt_len) // 2 - total // 2 - real, context - real - total - 2))
        for s in slots:
            engine.cache.reserve(s, real + skip)
            engine.cache.advance(s, real + skip)
        loop = DecodeLoop(engine, slots, total + 2, use_graph=graph)
        loop.run_device(first, warmup + steps)               # warm-up, and one untimed region
        torch.cuda.synchronize()
        ctx_start = engine.length(slots[0]) + warmup + steps
        if clocks is not None:
            clocks.__enter__()
        times = []
        for _ in range(reps):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            loop.run_device(None, steps)
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
        if clocks is not None:
            clocks.__exit__()
        mid = sorted(range(reps), key=lambda i: times[i])[reps // 2]      # the median region
        ms = times[mid]
        launches = loop.launches_per_step * steps
        loop.close()
        for s in slots:
            engine.close(s)
        del engine, loop
        torch.cuda.empty_cache()
        nbytes = weight_bytes(m) + batch * (ctx_start + mid * steps + steps / 2.0) * kv_bytes_per_token(m)
        return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
                "bytes_per_step": nbytes, "frac": nbytes / (ms / steps / 1e3) / 1e9 / pk["hbm_gbs"],
                "repetitions": reps, "all_ms_per_step": [t / steps for t in times]}

    def point_record(r):
        return {"tok_s": round(r["tok_s"], 1), "ms_per_step": round(r["ms_per_step"], 4),
                "bytes_per_step": int(r["bytes_per_step"]), "frac": round(r["frac"], 4)}

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

    def session_point(steps, warmup):
        """Batch 1 through llm.Session (`boom_llm_prefill` / `boom_llm_decode`): wall time
        per token of one decode call, after `warmup` tokens."""
        sess = llm.session_new(llm.Model(model), CONTEXT)
        sess.prefill(prompts(1)[0])
        stamps = []
        sess.decode(Sampling(max_tokens=warmup + steps + 1), cb=lambda t: stamps.append(time.perf_counter()) or 0)
        sess.free()
        dt = stamps[warmup + steps] - stamps[warmup]
        del sess
        torch.cuda.empty_cache()
        return {"tok_s": round(steps / dt, 1), "ms_per_step": round(dt / steps * 1e3, 4),
                "positions": f"{PROMPT_LEN}..{PROMPT_LEN + warmup + steps}"}

    if args.only == "decode":
        # a small case for profilers: the decode point alone (with --eager: kernel by kernel)
        r = decode_point(model, args.batch, args.steps, args.warmup, graph=not args.eager, reps=1)
        print(json.dumps({"only": "decode", "layers": cfg["num_hidden_layers"], "batch": args.batch,
                          "ms_per_step": round(r["ms_per_step"], 4), "tok_s": round(r["tok_s"], 1)}))
        return 0

    def prefill_point(m, n_tokens, reps):
        engine = sb.Engine(m, max_tokens=n_tokens, n_slots=1)
        (p,) = prompts(1, n_tokens, m.spec.vocab)
        times = []
        for i in range(1 + reps):
            s = engine.open()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step([(s, p, [n_tokens - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.close(s)
            if i > 0:
                times.append(start.elapsed_time(end))
        del engine
        torch.cuda.empty_cache()
        return sorted(times)[len(times) // 2]

    def prefill_flops(c, n_tokens):
        hd_ = c["hidden_size"] // c["num_attention_heads"]
        return n_tokens * decode_flops_per_token(c) + \
            c["num_hidden_layers"] * 4 * c["num_attention_heads"] * hd_ * n_tokens * n_tokens / 2 + \
            2 * c["hidden_size"] * c["vocab_size"]

    # prefill of one 2,048-token prompt
    prefill_ms = prefill_point(model, PROMPT_LEN, args.prefill_reps)
    hd = cfg["hidden_size"] // cfg["num_attention_heads"]
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "layers": cfg["num_hidden_layers"], "tokens": PROMPT_LEN,
                          "ms": round(prefill_ms, 3)}))
        return 0

    clocks = ClockSampler()
    main = decode_point(model, args.batch, args.steps, args.warmup, clocks=clocks)
    e2e = e2e_point(args.batch, args.steps, args.warmup)
    points = {}
    for b in (1, 64):
        points[f"decode_b{b}"] = point_record(decode_point(model, b, args.steps, args.warmup))
    if not args.no_extras:
        points["session_decode_b1"] = session_point(min(args.steps, 128), 8)
    ops.check_status()

    if not args.no_extras:
        # Further sizes of the same architecture; they do not enter `value`.
        del model
        torch.cuda.empty_cache()
        # Qwen2.5-1.5B sizes: 64 prompts of 16..1,024 tokens, 256 new tokens each at temperature
        # 0.7, through generate_batch (prefill, sampling and the host loop included)
        m15 = sb.random_model(QWEN25_1P5B, seed=0, dtype="bfloat16", device=dev, std=0.02)
        lens = torch.randint(16, 1025, (64,), generator=gen).tolist()
        ps = [torch.randint(0, QWEN25_1P5B["vocab_size"], (n,), generator=gen).tolist() for n in lens]
        llm.generate_batch(llm.Model(m15), ps[:4], max_tokens=8, ignore_eos=True, temperature=0.7, seed=1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate_batch(llm.Model(m15), ps, max_tokens=256, ignore_eos=True,
                                  temperature=0.7, seed=1)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        points["qwen2.5-1.5b_generate_64x256_t0.7"] = {
            "tok_s": round(sum(len(o) for o in outs) / dt, 1), "seconds": round(dt, 3),
            "prompt_tokens": sum(lens), "new_tokens": sum(len(o) for o in outs), "layers": 28}
        del m15
        torch.cuda.empty_cache()
        # Qwen2.5-32B sizes: prefill of 8,192 tokens; decode at batch 1 and 16 around position
        # 12,288 of 8,192..16,384 (64 tokens of each prompt are prefilled, the lengths are moved
        # forward over the rest: the cache holds zeros there and a step reads the same bytes)
        c32 = dict(QWEN25_32B)
        if args.layers_32b:
            c32["num_hidden_layers"] = args.layers_32b
        m32 = sb.random_model(c32, seed=0, dtype="bfloat16", device=dev, std=0.02)
        ms32 = prefill_point(m32, 8192, 1)
        rec = {"layers": c32["num_hidden_layers"], "layers_full_model": 64,
               "prefill_8192": {"tok_s": round(8192 / (ms32 / 1e3), 1), "ms": round(ms32, 2),
                                "frac": round(prefill_flops(c32, 8192) / (ms32 / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}}
        for b in (1, 16):
            rec[f"decode_b{b}"] = point_record(decode_point(m32, b, 16, 4, prompt_len=8192, context=16384,
                                                            real_prompt=64))
        points["qwen2.5-32b"] = rec
        del m32
        torch.cuda.empty_cache()
        ops.check_status()

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
                   "peaks": pk["source"],
                   "repetitions": f"median of {main['repetitions']} timed regions of {args.steps} steps "
                                  f"after {args.warmup} + {args.steps} untimed steps"},
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tok/s",
                "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": int(main["launches"]),
        "clocks": clocks.summary(),
        "prefill": {"value": round(PROMPT_LEN / (prefill_ms / 1e3), 1), "tokens": PROMPT_LEN,
                    "ms": round(prefill_ms, 3),
                    "frac": round(prefill_flops(cfg, PROMPT_LEN) / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "load_s": round(load_s, 1),
        "build": sb.build_info_line(),
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
    ap.add_argument("--no-extras", action="store_true",
                    help="leave out the points beyond the headline configuration (the session "
                         "entry point, the 1.5B and 32B sizes)")
    ap.add_argument("--layers-32b", type=int, default=0,
                    help="run the 32B sizes with fewer than their 64 layers (both numbers are recorded)")
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
