#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Qwen3-8B shape with random weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--shape 8b|0.6b|32b] [--impl ours|reference]
    python bench.py --design bozosun|sizizen|zerusun|vokepel [--size 1k|2k|4k]   (another design beside the Qwen3 layers of equal size; see below)

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 from 2,048-token prefixes, timed on the
device (CUDA events on the engine's stream) over exactly K decode steps after W warm-up steps, each step fed its
token ids from the host and ending in the greedy sampling kernel; ``e2e`` is the same through the Python entry point
(purhie_b200.api: streams, host token ids in and sampled tokens out every step) by the wall clock; ``prefill`` is
one 2,048-token prompt from submit to logits; ``roofline`` is the decode step's bytes (every weight once plus the
live requests' cache) over its time; ``points`` holds decode at batch 1 and 64 and a mixed step (32 decoded tokens
beside a 512-token prompt chunk).  Token ids are uniform random (synthetic).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the headline benchmark configuration: the Qwen3-8B shape
QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096, intermediate_size=12288,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936,
                max_position_embeddings=4096, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False)
# the two other benchmark shapes (Qwen3-0.6B and Qwen3-32B); the default run stays the 8B shape
QWEN3_06B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, intermediate_size=3072, num_attention_heads=16,
                 num_key_value_heads=8, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, intermediate_size=25600, num_attention_heads=64,
                 num_key_value_heads=8)
SHAPES = {"8b": ("Qwen3-8B", QWEN3_8B, 2, 0.02, (1, 64)), "0.6b": ("Qwen3-0.6B", QWEN3_06B, 3, 0.02, (1, 64)),
          "32b": ("Qwen3-32B", QWEN3_32B, 4, 0.015, (1, 32))}
CONTEXT, PREFIX, PREFILL_TOKENS = 4096, 2048, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    """The roofline denominators: the measured copy bandwidth, and the cuBLAS bf16 rate as a burst (a kernel timed
    alone, which is how the prefill is timed here) and sustained under the power cap."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained") or d["bf16_tflops"]), "source": "measured"}
        except (ValueError, KeyError, OSError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                clocks.append(float(f[0])); mx = float(f[1])
            except ValueError:
                continue
            for name, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks)}


# ---- another design beside the closest existing one -------------------------------------------------------------------
# Layer sizes that resemble a real model's, random weights.  Four layers, one of every pairing of the design's mixers
# and feed-forwards; the twin is four Qwen3 layers of the same width, heads and feed-forward width.
DESIGN_SIZES = {
    "1k": dict(width=1024, heads=8, kv_heads=2, dim=128, ff=4096, inner=2048, state=16, dt_rank=64, conv=4, experts=8, top=2,
               expert_ff=2048, vocab=32768),
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, inner=4096, state=16, dt_rank=128, conv=4, experts=8, top=2,
               expert_ff=4096, vocab=32768),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, inner=8192, state=16, dt_rank=256, conv=4, experts=16, top=4,
               expert_ff=3072, vocab=32768),
}


def bozosun_config(z):
    rot = {"base": 5e5, "dims": z["dim"], "scaling": {"factor": 8.0, "original": 4096, "fast": 24.0, "slow": 2.0}}
    att = lambda: {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                                                  "rot": rot, "scale": z["dim"] ** -0.5, "v_mix": True}}
    ssm = lambda: {"type": "mamba1", "mixer": {"inner": z["inner"], "state": z["state"], "dt_rank": z["dt_rank"], "conv": z["conv"]}}
    dense = {"kind": "dense", "ff": z["ff"], "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"], "limit": 7.0}, "router": {"experts": z["experts"], "top": z["top"]}}
    layers = [dict(att(), mlp=dense), dict(ssm(), mlp=moe), dict(att(), mlp=moe), dict(ssm(), mlp=dense)]
    return {"architecture": "Bozosun", "vocab": z["vocab"], "width": z["width"], "residual_mult": 0.5, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "layers": layers, "max_position": CONTEXT}


def sizizen_config(z):
    """Four layers of two mixers side by side (attention under a mask of blocks of 1,024 positions with heads of 128
    rotated over half their width; gated linear attention with half as many heads of 128 x 128 state), a dense gated unit
    in the first and last, routed ungated experts with a shared one in between."""
    left = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "rot": {"base": 5e5, "dims": z["dim"] // 2},
            "mask": {"size": 1024}, "scale": z["dim"] ** -0.5}
    right = {"heads": z["heads"] // 2, "dim": 128, "vdim": 128, "tau": 16.0, "rank": 64}
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": 4, "keep": 2}},
           "shared": {"ff": z["expert_ff"]}}
    layers = [{"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp} for mlp in (dense, moe, moe, dense)]
    return {"architecture": "Sizizen", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "layers": layers, "max_position": CONTEXT}


def zerusun_config(z):
    """Four parallel layers under dynamic-tanh norms: attention through a latent (query latent of 3/4 of the width, a
    cached row of 512 + 64 numbers, heads of 128 + 64 rotated dimensions, a window of 1,024 positions) in the first and
    last, lightning attention with half as many heads of 128 x 128 state in between; a dense gated unit in the first and
    last, routed experts with a gated shared one in between.  The two middle layers are the repeated stretch, run once,
    so that the reinjection in front of it is in the step and the number of layer runs equals the twin's."""
    rot = {"base": 5e5, "dims": 64, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    latent = {"heads": z["heads"], "dim": z["dim"], "rot_dim": 64, "vdim": z["dim"], "q_rank": 3 * z["width"] // 4, "kv_rank": 512,
              "mask": {"size": 1024}, "rot": rot, "scale": (z["dim"] + 64) ** -0.5}
    heads = z["heads"] // 2
    lightning = {"heads": heads, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-3.0 - 5.0 * h / max(heads - 1, 1)) for h in range(heads)]}
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "shared": {"ff": z["expert_ff"]},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 2.5, "groups": {"count": 4, "keep": 2}}}
    layers = [{"type": "latent_attention", "mixer": latent, "mlp": dense}, {"type": "lightning", "mixer": lightning, "mlp": moe},
              {"type": "lightning", "mixer": lightning, "mlp": moe}, {"type": "latent_attention", "mixer": latent, "mlp": dense}]
    return {"architecture": "Zerusun", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "layers": layers,
            "loop": {"start": 1, "stop": 3, "times": 1}, "max_position": CONTEXT}


def vokepel_config(z):
    """Four pre-norm layers with a factor on the residual and squared-relu feed-forwards: attention whose heads talk before
    the softmax (capped scores, a distance bias, a window of 1,024 positions, keys that double as values, a sigmoid gate)
    in the first and third, attention with a sink (heads of 128 rotated over their whole width in interleaved pairs, the
    same window) side by side with a minimal gated recurrent unit as wide as the model in the second and fourth.  The two
    middle layers are the repeated stretch, run once, so that the reinjection in front of it is in the step and the
    number of layer runs equals the twin's."""
    att = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "mask": {"size": 1024},
           "scale": z["dim"] ** -0.5, "softcap": 25.0}
    left = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "mask": {"size": 1024},
            "rot": {"base": 1e6, "dims": z["dim"]}, "scale": z["dim"] ** -0.5}
    both = {"left": left, "right": {"width": z["width"]}, "left_scale": 0.8, "right_scale": 1.2}
    dense = {"kind": "dense", "ff": z["ff"]}
    layers = [{"type": "attention", "mixer": att, "mlp": dense}, {"type": "parallel", "mixer": both, "mlp": dense},
              {"type": "attention", "mixer": att, "mlp": dense}, {"type": "parallel", "mixer": both, "mlp": dense}]
    return {"architecture": "Vokepel", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.6,
            "logit_scale": 1.5, "logit_softcap": 40.0, "layers": layers, "loop": {"start": 1, "stop": 3, "times": 1}, "max_position": CONTEXT}


DESIGN_CONFIGS = {"bozosun": bozosun_config, "sizizen": sizizen_config, "zerusun": zerusun_config, "vokepel": vokepel_config}


def design_bench(args):
    """Prefill and decode throughput of the design at real layer sizes beside its twin, and, kernel class by kernel
    class, the time per call with the fraction of the roofline (bytes over the copy bandwidth or flops over the
    cuBLAS rate, whichever is longer) from one profiled prompt and eight profiled decode steps."""
    import numpy as np
    from purhie_b200 import native
    from purhie_b200.engine import Engine, StepEntry
    z = DESIGN_SIZES[args.size]
    pk = peaks()
    twin = dict(QWEN3_8B, num_hidden_layers=4, hidden_size=z["width"], intermediate_size=z["ff"], num_attention_heads=z["heads"],
                num_key_value_heads=z["kv_heads"], head_dim=z["dim"], vocab_size=z["vocab"])
    rng = np.random.default_rng(5)
    batch, steps, warmup = args.batch, min(args.steps, 32), max(args.warmup, 3)
    result = {"design": args.design, "size": args.size, "sizes": z, "batch": batch, "prefix": PREFIX, "prefill_tokens": PREFILL_TOKENS,
              "peaks": pk, "models": {}}
    for name, config in ((args.design, DESIGN_CONFIGS[args.design](z)), ("qwen3_twin", twin)):
        vocab = z["vocab"]
        ids = lambda n: rng.integers(0, vocab, size=n).tolist()
        eng = Engine.from_random(config, 3, "bfloat16", std=0.02, page_size=16, max_requests=batch + 2,
                                 max_tokens=(batch + 1) * (PREFIX + 256) + PREFILL_TOKENS)
        prompt = ids(PREFILL_TOKENS)

        def prefill_once():
            eng.add_request("p")
            ms = eng.time_step([StepEntry("p", prompt, [PREFILL_TOKENS - 1])])
            eng.release("p")
            return ms
        for _ in range(2):
            prefill_once()
        prefill_ms = sorted(prefill_once() for _ in range(5))[2]
        for i in range(batch):
            eng.add_request(i)
            eng.step([StepEntry(i, ids(PREFIX), [])])
        sampler = ClockSampler()
        sampler.start()
        ms_step, launches = eng.time_decode_steps(list(range(batch)), [ids(steps + warmup) for _ in range(batch)], warmup, steps, sample=True)
        clocks = sampler.stop()
        # one profiled prompt and eight profiled decode steps: every launcher between events, graphs off
        native.lib().qe_profile_enable(1)
        native.profile_report(True)
        prefill_once()
        prof_prefill = native.profile_report(True)
        for _ in range(8):
            eng.step([StepEntry(i, ids(1), [0]) for i in range(batch)])
        prof_decode = native.profile_report(True)
        native.lib().qe_profile_enable(0)

        def classes(report):
            out = {}
            for k, v in sorted(report.items(), key=lambda kv: -kv[1]["ms"]):
                us = 1e3 * v["ms"] / max(v["calls"], 1)
                floor_us = max(v["bytes"] / v["calls"] / (pk["hbm_gbs"] * 1e3), v["flops"] / v["calls"] / (pk["bf16_tflops"] * 1e6)) if v["calls"] else 0.0
                out[k] = {"calls": v["calls"], "us_per_call": round(us, 2), "roofline_us": round(floor_us, 2),
                          "frac": round(floor_us / us, 3) if us > 0 and floor_us > 0 else None}
            return out
        result["models"][name] = {"prefill_ms": round(prefill_ms, 3), "prefill_tok_s": round(PREFILL_TOKENS / prefill_ms * 1e3, 1),
                                  "decode_ms_per_step": round(ms_step, 4), "decode_tok_s": round(batch / ms_step * 1e3, 1),
                                  "decode_launches": launches, "clocks": clocks,
                                  "prefill_kernels": classes(prof_prefill), "decode_kernels": classes(prof_decode)}
        eng.close()
    print(json.dumps(result))
    return 0


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a HIP engine for AMD gfx1151 (Makefile + hipcc, GGUF models); it has no Python "
                      "package to install (pip finds neither setup.py nor pyproject.toml) and no CUDA path"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: the headline 8B shape or another")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has (named in config); layer sizes stay")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64 and the mixed step")
    ap.add_argument("--phase", default="all", choices=["all", "decode", "prefill"],
                    help="run one phase only, with few launches around it (for profiling under ncu)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (the benchmark's configuration has 16)")
    ap.add_argument("--step-options", default="", metavar="JSON",
                    help="kernel choices of the step, for comparing two forms of it on one box, e.g. '{\"norm_ahead\": \"off\"}'")
    ap.add_argument("--design", default="", choices=["", "bozosun", "sizizen", "zerusun", "vokepel"],
                    help="instead of the headline workload: prefill and decode of this design at real layer sizes beside four "
                         "Qwen3 layers of equal size, with the time and roofline fraction of every kernel class")
    ap.add_argument("--size", default="4k", choices=sorted(DESIGN_SIZES), help="with --design: the layer sizes")
    ap.add_argument("--leave-out", default="", metavar="NAMES",
                    help="with --phase decode: launchers (comma separated, e.g. add_rmsnorm,decode_bulk) that the timed steps "
                         "skip; the difference to a run without shows what they cost inside the graph (no benchmark value)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.design:
        return design_bench(args)

    import numpy as np
    from purhie_b200.api import GenOptions, load_model_random
    from purhie_b200.config import Qwen3Config
    from purhie_b200.engine import Engine, StepEntry
    from purhie_b200.sampling import SamplerParams

    shape_name, shape, SEED, STD, point_batches = SHAPES[args.shape]
    if args.layers is None:
        args.layers = shape["num_hidden_layers"]
    cfg = Qwen3Config.from_dict(dict(shape, num_hidden_layers=args.layers))
    pk = peaks()
    model = load_model_random(cfg, SEED, "bfloat16", std=STD)
    max_batch = args.batch if args.phase != "all" else max(max(point_batches), args.batch)
    if args.phase != "all":
        args.no_points = True
    kv_tokens = max_batch * (PREFIX + 2 * (args.steps + args.warmup) + 256) + PREFILL_TOKENS + 64
    step_options = {"step": json.loads(args.step_options)} if args.step_options else {}
    model.kv_cache_init(CONTEXT, max_sequences=max_batch + 2, page_size=args.page_size, kv_tokens=kv_tokens, **step_options)
    eng = Engine.attach(model)
    rng = np.random.default_rng(SEED)
    ids = lambda n: rng.integers(0, cfg.vocab_size, size=n).tolist()
    median = lambda xs: sorted(xs)[len(xs) // 2]

    # ---- prefill of one 2,048-token prompt ----------------------------------------------------------
    prompt = ids(PREFILL_TOKENS)

    def prefill_once():
        eng.add_request("prefill")
        ms = eng.time_step([StepEntry("prefill", prompt, [PREFILL_TOKENS - 1])])
        eng.release("prefill")
        return ms

    if args.phase == "decode":
        prefill_ms = float("nan")
    else:
        for _ in range(3 if args.phase == "all" else 1):
            prefill_once()
        from purhie_b200 import native as _native
        if _native.profile_enabled():
            _native.profile_report(True)             # the warm-up runs do not count
        prefill_ms = median([prefill_once() for _ in range(5 if args.phase == "all" else 1)])
    if args.phase == "prefill":
        from purhie_b200 import native
        if native.profile_enabled():
            sys.stderr.write(native.format_profile(native.profile_report(), f"prefill of {PREFILL_TOKENS} tokens, {args.layers} layers") + "\n")
        print(json.dumps({"phase": "prefill", "ms": prefill_ms, "layers": args.layers}))
        return 0
    T, E, FF, V = PREFILL_TOKENS, cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    qw, kvw, D = cfg.q_width, cfg.kv_width, cfg.head_dim
    layer_mm = E * (qw + 2 * kvw) + qw * E + 3 * E * FF
    prefill_flops = cfg.num_hidden_layers * (2.0 * T * layer_mm + 4.0 * cfg.num_attention_heads * D * T * (T + 1) / 2) + 2.0 * V * E
    tflops = prefill_flops / (prefill_ms * 1e-3) / 1e12
    prefill = {"value": round(T / prefill_ms * 1e3, 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(tflops / pk["bf16_tflops"], 4), "frac_of_sustained": round(tflops / pk["bf16_tflops_sustained"], 4),
               "tflops": round(tflops, 1), "peak": pk["source"]}

    # ---- prefixes of 2,048 tokens for every request ---------------------------------------------------
    for i in range(max_batch):
        eng.add_request(i)
        eng.step([StepEntry(i, ids(PREFIX), [])])

    weight_bytes = 2.0 * (cfg.num_hidden_layers * layer_mm + V * E)       # the embedding table is gathered, not streamed
    kv_bytes_per_token = 2.0 * 2 * cfg.num_hidden_layers * kvw

    def decode_run(batch, steps, warmup):
        ctx0 = eng.length(0) + warmup
        toks = [ids(steps + warmup) for _ in range(batch)]
        ms, launches = eng.time_decode_steps(list(range(batch)), toks, warmup, steps, sample=True)
        bytes_step = weight_bytes + batch * (ctx0 + steps / 2.0) * kv_bytes_per_token
        return ms, launches, bytes_step

    if args.leave_out:
        if args.phase != "decode":
            print("bench.py: --leave-out goes with --phase decode")
            return 2
        from purhie_b200 import native
        native.lib().qe_profile_leave_out(args.leave_out.encode())     # the graphs are captured after this
    from purhie_b200 import native as _native
    if _native.profile_enabled():
        _native.profile_report(True)                 # what came before the timed steps does not count
    sampler = ClockSampler()
    sampler.start()
    ms_step, launches, bytes_step = decode_run(args.batch, args.steps, args.warmup)
    clocks = sampler.stop()
    points = {}
    if not args.no_points:
        for b in point_batches:
            ms_b, _, by = decode_run(b, min(args.steps, 32), 3)
            points[f"decode_b{b}"] = round(b / ms_b * 1e3, 1)
            points[f"decode_b{b}_hbm_frac"] = round(by / (ms_b * 1e-3) / (pk["hbm_gbs"] * 1e9), 4)
        # a step of 32 decoded tokens beside one 512-token prompt chunk (the small shape's benchmark workload),
        # launched kernel by kernel every time
        n_dec, chunk = min(32, max_batch), 512
        chunk_ids = ids(chunk)

        def mixed_once():
            eng.add_request("chunk")
            ms = eng.time_step([StepEntry(i, [chunk_ids[i]], [0]) for i in range(n_dec)] + [StepEntry("chunk", chunk_ids, [chunk - 1])])
            eng.release("chunk")
            return ms

        for _ in range(3):
            mixed_once()
        points[f"mixed_b{n_dec}_chunk{chunk}_ms"] = round(median([mixed_once() for _ in range(5)]), 3)
    if args.phase == "decode":
        from purhie_b200 import native
        if native.profile_enabled():             # PURHIE_PROFILE=1: every launch between events, graphs off
            sys.stderr.write(native.format_profile(native.profile_report(), f"decode, batch {args.batch}, {args.layers} layers") + "\n")
        print(json.dumps({"phase": "decode", "batch": args.batch, "ms_per_step": ms_step, "layers": args.layers,
                          "left_out": args.leave_out or None}))
        return 0

    # ---- end to end through the Python entry point ------------------------------------------------------
    for i in range(max_batch):
        eng.release(i)
    streams = []
    opts = GenOptions(sampler=SamplerParams.greedy(), max_new_tokens=args.steps + args.warmup + 8, ignore_eog=True)
    for i in range(args.batch):
        seq = model.seq_new()
        model.seq_select(seq)
        streams.append(model.stream_begin(ids(PREFIX), opts))
    model.stream_run(streams, args.warmup)
    model.synchronize()
    t0 = time.perf_counter()
    done = model.stream_run(streams, args.steps)          # host token ids in, every step's sampled ids out
    model.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    assert len(done) == args.steps and all(tok is not None for step in done for _, tok in step)
    h2d = model.engine_info()["upload_bytes"]                   # the step's packed int32 metadata (ids, positions, tables)
    e2e = {"value": round(args.batch / e2e_ms * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch + 8}

    # ---- the small shape is bound by launches: the same decode with every kernel launched by the host -----------
    if args.shape == "0.6b" and not args.no_points:
        for st in streams:
            st.free()
        model.kv_cache_init(CONTEXT, max_sequences=3, page_size=args.page_size, kv_tokens=2 * (PREFIX + 256), cuda_graphs=False)
        eng2 = Engine.attach(model)
        eng2.add_request(0)
        eng2.step([StepEntry(0, ids(PREFIX), [])])
        ms_off, launches_off = eng2.time_decode_steps([0], [ids(35)], 3, 32, sample=True)
        points["decode_b1_graphs_off"] = round(1 / ms_off * 1e3, 1)
        points["decode_b1_launches_per_step"] = launches_off // 32

    value = args.batch / ms_step * 1e3
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {args.batch} from 2,048-token prefixes ({shape_name} shape)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": f"{shape_name} shape, random weights seed {SEED}", "global_batch": args.batch, "seq_len": PREFIX,
                   "context": CONTEXT, "parallelism": "single GPU", "layers": args.layers,
                   "layers_of_config": shape["num_hidden_layers"], "hidden": E, "q_heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": D, "intermediate": FF, "vocab": V,
                   "kv_page_tokens": args.page_size, "kv_dtype": "bf16", "l2": f"weights ({weight_bytes / 1e9:.1f} GB) exceed L2 every step",
                   "cuda_graphs": True, "prefill_tokens": PREFILL_TOKENS, "sampling": "greedy, inside the timed step"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"]},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
