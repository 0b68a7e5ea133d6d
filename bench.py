"""Decode and prefill throughput of the Llama-3.1-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 with a
2,048-token prompt in a cache sized for 4,096 tokens per sequence, timed on the
device with CUDA events around K replays of the captured decode step; ``e2e`` is
the same through ``Engine.generate`` (host token lists in and out; each step copies
its input tokens from pinned host memory and reads the sampled tokens back), from
the call's own per-step timings of a run that decodes K tokens after the first
(``e2e.by_difference``: against a run that stops after the first; ``e2e.sm_mhz``: the
clocks sampled during those calls; ``e2e.step_call``: the per-step call underneath,
``Engine.run``, once the clocks are back up).  ``prefill`` is one
2,048-token prompt; ``points`` hold decode at batch 1 and 64; ``roofline`` compares
the decode step with the bytes it has to read (each weight it uses once, plus the
keys and values of the live sequences).  Weights are seeded random values of the
real shape (there is no checkpoint offline); inputs exceed L2, so nothing stays
cached between steps.  Between the prompts' prefill and the W warm-up steps the
process pauses for a quarter of a second: the prefill of eight prompts runs at
the power cap and leaves the SM clock low for some tens of milliseconds, which
a short timed region would otherwise measure instead of decoding (``e2e`` keeps
that shadow, prompts and steps being one call, and reports its clocks).

Other workloads than the default run's: ``--model NAME`` takes another shipped or
registered configuration's layer sizes (``llama-3.2-1b``, ``llama-3.2-3b``; whatever
architecture its config.json names), ``--prompt-tokens N`` (with ``--context C``) other prompt
and cache lengths, ``--batch B`` another batch; the line then names them in ``metric``
and ``config``.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PROMPT_TOKENS = 2048
CONTEXT = 4096
SETTLE_S = 0.25        # pause between the prompts' prefill and the decode warm-up (see decode_at)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"])}, "measured"
        except Exception:  # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:  # noqa: BLE001
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "sm_mhz_min": min(sm) if sm else None, "reasons": sorted(reasons), "samples": len(sm)}


def main() -> int:
    global PROMPT_TOKENS, CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--model", default="llama-3.1-8b",
                    help="the shipped or registered configuration whose layer sizes run (the default run's is llama-3.1-8b)")
    ap.add_argument("--prompt-tokens", type=int, default=PROMPT_TOKENS,
                    help="tokens of every prompt, also of the timed prefill (other context lengths than the default run's)")
    ap.add_argument("--context", type=int, default=0,
                    help="cache tokens per sequence (default: 4,096, or the prompt and the decoded tokens rounded up to 1,024)")
    ap.add_argument("--no-pdl", action="store_true", help="launch kernels in plain stream order (no programmatic dependent launch)")
    ap.add_argument("--cuda-profiler-range", nargs="?", const="decode", default=None, choices=["decode", "prefill"],
                    help="bracket the timed decode replays (or the timed prefill steps) with cudaProfilerStart/Stop, "
                         "for ncu --profile-from-start off")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pip cannot install the reference offline (setuptools: multiple top-level packages in a "
                          "flat layout); its public API also downloads weights with huggingface_hub (no network) "
                          "and it has no random-weights mode"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    PROMPT_TOKENS = args.prompt_tokens
    need = PROMPT_TOKENS + args.warmup + args.steps + 64
    CONTEXT = args.context or max(CONTEXT, (need + 1023) // 1024 * 1024)
    if CONTEXT < need:
        print(f"bench.py: --context {CONTEXT} holds no prompt of {PROMPT_TOKENS} tokens plus {args.warmup + args.steps} steps")
        return 2

    import dataclasses

    import torch

    import simple_inference_autoresearch_b200 as siar
    from simple_inference_autoresearch_b200 import registry
    from simple_inference_autoresearch_b200.config import preset_path
    from simple_inference_autoresearch_b200.engine import generation
    from simple_inference_autoresearch_b200.kernels import ops

    if args.no_pdl:
        ops.set_programmatic_launch(False)
    try:
        _arch, full = registry.resolve_path(preset_path(args.model))      # the class the preset's architecture names
    except FileNotFoundError as e:
        print(f"bench.py: {e}")
        return 2
    if args.layers:
        if not (dataclasses.is_dataclass(full) and hasattr(full, "num_hidden_layers")):
            print("bench.py: --layers needs a configuration with num_hidden_layers")
            return 2
        cfg = dataclasses.replace(full, num_hidden_layers=args.layers)
    else:
        cfg = full
    pk, pk_src = peaks()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)

    loaded = siar.init_random(siar.build_model(cfg, torch.bfloat16, dev), seed=0)
    model = loaded.model
    # Sizes the arithmetic below needs, taken from the model itself (its tensors, its cache needs and its
    # mixers), so that another registered architecture's configuration runs through the same lines.
    from simple_inference_autoresearch_b200.parts.base import KVNeed
    spec = model.spec
    h, v, L = spec.hidden_size, spec.vocab_size, len(model.schedule)
    kv_token_bytes = sum(n.n_kv_heads * (n.head_dim + (n.v_head_dim or n.head_dim)) * 2       # bfloat16 keys and values
                         for n in model.cache_needs if isinstance(n, KVNeed))
    matrix_params = sum(t.shape[0] * t.shape[1] for t in model.tensor_specs() if t.role == "matrix" and len(t.shape) == 2)
    table_params = v * h * (1 if spec.head_name is None else 2)          # embedding table (and the head when untied)
    layer_matrix_params = (matrix_params - table_params) * L // max(len(model.layers), 1)     # per run of the schedule
    attn_flops_per_token_pair = sum(4 * getattr(model.layers[e.layer].mixer, "n_heads", 0) *
                                    getattr(model.layers[e.layer].mixer, "head_dim", 0)
                                    for e in model.schedule if hasattr(model.layers[e.layer], "mixer"))
    if not args.no_points and 64 * CONTEXT * kv_token_bytes > 100e9:
        print(f"bench.py: the batch 1 / 64 points are left out: 64 sequences of {CONTEXT:,} tokens would hold "
              f"{64 * CONTEXT * kv_token_bytes / 1e9:.0f} GB of keys and values", file=sys.stderr)
        args.no_points = True
    max_b = max(args.batch, 1 if args.no_points else 64)
    engine = siar.Engine(model, max_batch=max_b, max_seq_len=CONTEXT, use_cuda_graph=True)
    gen = torch.Generator().manual_seed(0)
    rand_tokens = lambda n: torch.randint(0, v, (n,), generator=gen).tolist()  # noqa: E731

    # ---------------------------------------------------------------- prefill, one prompt
    def prefill_once():
        s = engine.open()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        toks = rand_tokens(PROMPT_TOKENS)
        torch.cuda.synchronize()
        e0.record()
        engine.step([siar.StepEntry(s, toks, [PROMPT_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        engine.close(s)
        return e0.elapsed_time(e1)

    for _ in range(2):
        prefill_once()
    if args.cuda_profiler_range == "prefill":
        torch.cuda.profiler.start()
    prefill_ms = statistics.median(prefill_once() for _ in range(3))
    if args.cuda_profiler_range == "prefill":
        torch.cuda.profiler.stop()
    T = PROMPT_TOKENS
    # the layers' products on every token, causal attention (half of T x T), the head on the one wanted row
    prefill_flops = 2 * T * layer_matrix_params + attn_flops_per_token_pair * T * T / 2 + 2 * v * h
    prefill = {"value": round(T / (prefill_ms * 1e-3), 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---------------------------------------------------------------- decode at a batch size
    embed_bytes = v * h * 2
    # every weight a step uses, once: the embedding table is only read as the head, when the two are tied
    weight_bytes = model.weight_bytes() - embed_bytes * (0 if spec.head_name is None else 1)

    def decode_at(batch, steps, warmup, e2e):
        slots_reqs = []
        for b in range(batch):
            r = generation.Request(rand_tokens(PROMPT_TOKENS), 10 ** 9, siar.SamplingParams(temperature=0.0), index=b)
            r.slot = engine.open()
            slots_reqs.append(r)
        for g0 in range(0, batch, 8):   # real prefill, eight prompts to a step
            grp = slots_reqs[g0:g0 + 8]
            engine.step([siar.StepEntry(r.slot, r.prompt, []) for r in grp])
        # The prompts' prefill runs at the power cap and leaves the SM clock low for some tens of
        # milliseconds; the warm-up and the timed steps measure decoding, not that shadow (the e2e
        # figure below, prompts and steps in one call, keeps it and says so).
        torch.cuda.synchronize()
        time.sleep(SETTLE_S)
        feed = [[1] for _ in slots_reqs]
        for _ in range(warmup):
            out = engine.run(slots_reqs, feed)
            feed = [[t] for t in out]
        # device-timed: K replays of the captured step (tokens, lengths and sampling stay on the device)
        graph = engine._graphs[(batch, engine._graph_state.bucket)]
        engine.cache.reserve([r.slot for r in slots_reqs], [steps] * batch)    # pages for the replays below
        sampler = ClockSampler()
        sampler.start()
        before = ops.launch_count
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if args.cuda_profiler_range == "decode" and e2e:
            torch.cuda.profiler.start()
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        if args.cuda_profiler_range == "decode" and e2e:
            torch.cuda.profiler.stop()
        dev_ms = e0.elapsed_time(e1) / steps
        launches = ops.launch_count - before
        kv_mid = PROMPT_TOKENS + warmup + steps / 2
        engine.cache.commit([r.slot for r in slots_reqs], [steps] * batch)
        engine._graph_state.invalidate()
        res = {"ms": dev_ms, "tok_s": batch / (dev_ms * 1e-3), "launches": launches,
               "bytes": weight_bytes + batch * h * 2 + batch * kv_mid * kv_token_bytes}
        if e2e:
            feed = [[1] for _ in slots_reqs]
            for _ in range(3):
                out = engine.run(slots_reqs, feed)
                feed = [[t] for t in out]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                out = engine.run(slots_reqs, feed)
                feed = [[t] for t in out]
            torch.cuda.synchronize()
            res["e2e_tok_s"] = batch * steps / (time.perf_counter() - t0)
        sampler.stop()
        res["clocks"] = sampler.summary()
        for r in slots_reqs:
            engine.close(r.slot)
        return res

    head = decode_at(args.batch, args.steps, args.warmup, e2e=True)

    # ---------------------------------------------------------------- end to end through Engine.generate
    # The public call: host token lists in, host token lists out.  Every decode step inside it copies
    # its input tokens from pinned host memory, runs, reads the drawn tokens back and synchronises;
    # the call's own statistics time each of those steps with the host clock (the reference's
    # generate_with_stats reports decode tok/s the same way, generate.py:193-237).  The value is the
    # median of three calls that decode `steps` tokens after the first.  As a cross-check, the
    # difference between such a call and one that stops after the first token (`by_difference`:
    # it also carries what the two prefills differ by, a few milliseconds at the power cap).
    prompts = [rand_tokens(PROMPT_TOKENS) for _ in range(args.batch)]
    greedy = siar.SamplingParams(temperature=0.0)
    engine.generate(prompts, greedy, max_new_tokens=1 + args.warmup, ignore_eos=True)      # warm-up
    diffs, in_call = [], []
    e2e_clock = ClockSampler()               # the clocks the decode steps of these calls run at (read-only sampling)
    e2e_clock.start()
    for _ in range(3):                       # the median of three pairs: one pair alone moves by a few per cent
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        engine.generate(prompts, greedy, max_new_tokens=1, ignore_eos=True)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        outs, gen_stats = engine.generate(prompts, greedy, max_new_tokens=1 + args.steps, ignore_eos=True,
                                          return_stats=True)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        assert all(len(o) == 1 + args.steps for o in outs)
        diffs.append((t2 - t1) - (t1 - t0))
        in_call.append(gen_stats["decode_tok_s"])
    e2e_clock.stop()
    e2e_clocks = e2e_clock.summary()
    generate_tok_s = sorted(in_call)[1]
    by_difference = args.batch * args.steps / max(sorted(diffs)[1], 1e-9)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(decode_at(b, max(8, args.steps // 2), args.warmup, e2e=False)["tok_s"], 1)

    def config_record():
        """Every size of the run, flat and at most 20 keys: the run's own numbers, then the configuration's
        keys as config.json names them (a nested block such as rope_scaling becomes one string)."""
        rec = {"model": f"{args.model} shape", "global_batch": args.batch, "seq_len": CONTEXT,
               "prompt_tokens": PROMPT_TOKENS, "parallelism": "single GPU", "layers": L,
               "layers_of_full_model": getattr(full, "num_hidden_layers", L)}
        skip = {"architectures", "model_type", "bos_token_id", "eos_token_id", "torch_dtype", "hidden_act", "attention_bias",
                "mlp_bias", "num_hidden_layers", "initializer_range", "max_position_embeddings", "norm_weight_init"}
        for key, val in cfg.to_dict().items():
            if key in skip or isinstance(val, (list, tuple)) or len(rec) >= 18:
                continue
            if isinstance(val, dict):
                val = " ".join(f"{k}={x}" for k, x in val.items())
            rec[key] = val
        rec["l2"] = "inputs larger than L2 (weights + cache read every step)"
        rec["peaks"] = pk_src
        return rec

    achieved = head["bytes"] / (head["ms"] * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s @ batch {args.batch} ({args.model.replace('llama', 'Llama').upper().replace('LLAMA', 'Llama')} shape, bf16, {PROMPT_TOKENS:,}-token prompts, "
                  f"{CONTEXT:,}-token cache)",
        "value": round(head["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(head["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)",
        "impl": "ours",
        "config": config_record(),
        "e2e": {"value": round(generate_tok_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * args.batch,
                "d2h_bytes_per_step": 4 * args.batch + 4, "via": "Engine.generate: its decode steps timed by the call's own statistics (host clock around every step), median of 3 calls",
                "by_difference": round(by_difference, 1),
                "step_ms_first16": gen_stats["tpot_ms_first16"], "step_ms_last16": gen_stats["tpot_ms_last16"],
                "note": "the steps right after the prompts run at the clocks the prefill left (power cap)",
                "sm_mhz": e2e_clocks["sm_mhz"], "sm_mhz_min": e2e_clocks.get("sm_mhz_min"),       # over the calls: prompts and decode steps
                "step_call": round(head["e2e_tok_s"], 1)},
        "gpu_launches": head["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_src},
        "points": points,
        "clocks": head["clocks"],
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
