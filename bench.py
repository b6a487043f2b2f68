#!/usr/bin/env python3
"""Benchmark of the library's serving step on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default workload: the layer sizes of Llama-3.1-8B with random weights (bfloat16), a batch of 8
sequences with 512-token prompts in a cache sized for a context of 4096, K decode steps.
Prints ONE JSON line.  ``value`` is decoded tokens per second, timed on the device with CUDA
events; ``e2e`` is the same loop by the wall clock, through the public Python entry point with
host token ids in and out every step.  The line also carries the mean and the median step, the
prefill of one 2,048-token prompt, the decode step's roofline fraction against the measured HBM
bandwidth, and further points: decode at batch 1 and 64, decode after prompts of 2,048 and 3,900
tokens, the true 32-bit path (decode and prefill at a stated number of layers), and the
generation workloads of the 1B and 13B size sets.
A step reads all 15 GB of weights, far more than the 126 MB L2, so no L2 flush is needed
between timed iterations (``config.l2`` says so).

``--impl reference`` measures artalis-io/bitnet.c itself (unmodified, built from baseline/_ref with
its own Makefile) on the same sizes through baseline/ref_harness.c.
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

LLAMA_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 4096,
    "intermediate_size": 14336, "num_hidden_layers": 32, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256, "max_position_embeddings": 4096,
    "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
}
LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 2048,
    "intermediate_size": 8192, "num_hidden_layers": 16, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256, "max_position_embeddings": 8192,
    "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "hidden_act": "silu",
}
LLAMA_13B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 5120,
    "intermediate_size": 13824, "num_hidden_layers": 40, "num_attention_heads": 40,
    "num_key_value_heads": 40, "head_dim": 128, "vocab_size": 32000, "max_position_embeddings": 4096,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
}
PROMPT_LEN = 512
FP32_LAYERS = 8  # layers of the float32 points (the sizes of each layer are the full ones)
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs.

    nvidia-smi needs a moment before its first line, and a timed region of a few dozen decode
    steps is shorter than that: ``launch`` starts it before the warm-up steps, every line is
    stamped when it arrives, and ``stop`` keeps the lines between ``start`` and ``stop``.  If
    fewer than three fall into the timed region, the lines of the warm-up steps (the same steps,
    directly before) are counted too, and ``window`` says so."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    PERIOD_MS = 20

    def __init__(self):
        self.lines, self.proc = [], None
        self.t_launch = self.t_start = self.t_stop = None

    def launch(self):
        if self.proc is not None:
            return
        self.t_launch = time.monotonic()
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.PERIOD_MS)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def start(self):
        self.launch()
        self.t_start = time.monotonic()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

    def stop(self):
        self.t_stop = time.monotonic()
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        timed = [l for t, l in self.lines if self.t_start <= t <= self.t_stop]
        window = "timed steps"
        if len(timed) < 3:
            timed = [l for t, l in self.lines if t <= self.t_stop]
            window = "warm-up and timed steps"
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in timed:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm), "window": window}


REF_DIR = os.path.join(ROOT, "baseline", "_ref")
# where an unmodified checkout of artalis-io/bitnet.c lies if baseline/_ref does not hold one yet
REF_SOURCE = os.environ.get("BITNET_C_SOURCE") or os.path.join(os.path.dirname(ROOT), "reference")
REF_PREFILL_BUDGET_S = 200.0  # the 2,048-token prompt is left out if the 512-token one says it would take longer
REF_CUDA_NOTE = ("its CUDA backend cannot be built: nvcc 12.9 stops on src/gpu_cuda.cu with 119 errors in the source "
                 "itself (BnCudaBlockQ8_1 used at line 104 before its definition at line 179, 115 calls that pass "
                 "'&ctx->runtime_policy' where a 'const BnBackendRuntimePolicy *' is expected, an undefined identifier "
                 "'gpu' at line 18869, a call with too few arguments at line 15883)")


def _cpu_stamp():
    """What the reference's objects were built for: its Makefile compiles with -march=native."""
    flags = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = line
                    break
    except OSError:
        pass
    import hashlib
    return hashlib.sha256(flags.encode()).hexdigest()[:16]


def build_reference():
    """An unmodified copy of the reference under baseline/_ref, built with its own Makefile (CPU
    engine: ``make bitnet``), and this repository's harness linked against its objects.  Returns
    the harness's path; raises RuntimeError with the reason if something is missing or fails."""
    import glob
    import shutil
    if not os.path.isfile(os.path.join(REF_DIR, "Makefile")):
        if not os.path.isfile(os.path.join(REF_SOURCE, "Makefile")):
            raise RuntimeError("no copy of artalis-io/bitnet.c under baseline/_ref and none to copy from")
        shutil.copytree(REF_SOURCE, REF_DIR, dirs_exist_ok=True)
    stamp_path = os.path.join(REF_DIR, ".built_for_cpu")
    stamp = _cpu_stamp()
    built = os.path.isfile(stamp_path) and open(stamp_path).read().strip() == stamp
    exe = os.path.join(ROOT, "baseline", "_ref", "ref_harness")
    env = dict(os.environ, NVCC="/usr/local/cuda/bin/nvcc")
    if not built:
        subprocess.run(["make", "clean"], cwd=REF_DIR, env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        r = subprocess.run(["make", "bitnet", f"-j{max(2, os.cpu_count() or 2)}"], cwd=REF_DIR, env=env,
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("the reference's 'make bitnet' failed: " + r.stdout.strip().splitlines()[-1][:200])
    harness_src = os.path.join(ROOT, "baseline", "ref_harness.c")
    if not built or not os.path.isfile(exe) or os.path.getmtime(exe) < os.path.getmtime(harness_src):
        objs = [o for o in glob.glob(os.path.join(REF_DIR, "src", "**", "*.o"), recursive=True)
                if not o.endswith(os.sep + "main.o")]
        r = subprocess.run([os.environ.get("CC", "gcc"), "-O2", "-std=c11", "-D_GNU_SOURCE", "-I", os.path.join(REF_DIR, "include"),
                            "-I", os.path.join(REF_DIR, "src"), harness_src, *objs, "-lm", "-lpthread", "-o", exe],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("linking the harness against the reference's objects failed: " + r.stdout.strip()[-300:])
        with open(stamp_path, "w") as f:
            f.write(stamp + "\n")
    return exe


def reference_arm(args):
    """The same metric from artalis-io/bitnet.c itself, unmodified, through its public calls
    (bn_session_create, bn_prefill, bn_prompt_cache_*, bn_transformer_forward, bn_sampler_sample),
    on the same sizes with random BF16 weights.  It runs on the host's cores: the reference is a
    CPU-first engine and the CUDA backend of this checkout does not compile."""
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    try:
        exe = build_reference()
    except (RuntimeError, OSError) as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)[:400]}))
        return 0
    cfg = dict(LLAMA_8B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    warmup = max(3, args.warmup)
    B = args.batch
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    cmd = [exe] + [str(v) for v in (
        cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"],
        cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"], cfg["max_position_embeddings"],
        cfg["rope_theta"], cfg["rms_norm_eps"], B, PROMPT_LEN, args.steps, warmup,
        0 if args.skip_points else PREFILL_TOKENS, threads, REF_PREFILL_BUDGET_S * 1e3)]
    t0 = time.perf_counter()
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    if r.returncode != 0:
        print(json.dumps({"impl": "reference", "unavailable": f"the harness exited with {r.returncode}: "
                          + (r.stderr.strip().splitlines() or ["no message"])[-1][:300]}))
        return 0
    res = json.loads(r.stdout.strip().splitlines()[-1])
    steps_ms = sorted(res["step_ms"])
    total_ms = sum(steps_ms)
    value = B * len(steps_ms) / (total_ms / 1e3)
    out = {
        "metric": f"decode tokens/s at batch {B} (Llama-3.1-8B sizes, bf16)", "value": round(value, 3), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(total_ms / len(steps_ms), 3),
        "ms_per_step_median": round(steps_ms[len(steps_ms) // 2], 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 weights, float32 activations and cache",
        "data": "synthetic", "impl": "reference",
        "config": {"model": "llama-3.1-8b-sizes-random", "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": B, "seq_len": cfg["max_position_embeddings"], "prompt_len": PROMPT_LEN,
                   "rope_theta": cfg["rope_theta"], "rms_norm_eps": cfg["rms_norm_eps"], "tied": False,
                   "parallelism": "single-gpu", "l2": "inputs larger than any cache (15 GB of weights per forward)",
                   "peaks": "none"},
        "device": f"host CPU, {res['threads']} threads: the reference's CPU engine; " + REF_CUDA_NOTE,
        "batching": "one BnSession per request, each stepped once per decode step; the prompt is run once by "
                    "bn_prefill and restored into the other sessions by the reference's prompt cache "
                    "(all but the last token, which differs per request)",
        "e2e": {"value": round(value, 3), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "host engine: token ids never leave the host; the timed loop includes the greedy choice"},
        "gpu_launches": 0,
        "clocks": {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "no GPU work in this arm"},
        "prompt_prefill": {"tokens": PROMPT_LEN, "ms": round(res["prompt_ms"], 1),
                           "value": round(PROMPT_LEN / (res["prompt_ms"] / 1e3), 2)},
        "wall_s": round(time.perf_counter() - t0, 1),
    }
    if res.get("prefill_ms", -1) > 0:
        out["prefill"] = {"value": round(res["prefill_tokens"] / (res["prefill_ms"] / 1e3), 2), "tokens": res["prefill_tokens"],
                          "ms": round(res["prefill_ms"], 1)}
    if res.get("b1_step_ms"):
        b1 = sorted(res["b1_step_ms"])
        out["points"] = {"decode_b1": round(1e3 * len(b1) / sum(b1), 3)}
    print(json.dumps(out))
    return 0


def weight_bytes(model):
    seen, total = set(), 0
    tensors = [model.embedding, model.head]
    for blk in model.blocks:
        tensors += [blk.mixer.w_qkv, blk.mixer.w_o, blk.ffn.w_gate_up, blk.ffn.w_down, blk.mixer_norm.weight,
                    blk.ffn_norm.weight]
    tensors.append(model.final_norm.weight)
    for t in tensors:
        if t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    return total


def decode_read_bytes(model, cfg, batch, context_len):
    """Bytes a decode step has to read: every weight it uses once (the embedding table only the
    rows it gathers) and the cached keys and values of the live sequences."""
    emb = model.embedding.numel() * model.embedding.element_size()
    w = weight_bytes(model) - (emb if model.head is not model.embedding else 0)
    w += batch * cfg["hidden_size"] * model.embedding.element_size() if model.head is not model.embedding else 0
    kv_per_token = 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * model.embedding.element_size()
    return w + batch * context_len * kv_per_token


def prefill_flops(cfg, T):
    d, I, L, H, KV, hs, V = (cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"],
                             cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"])
    per_layer = 2 * T * d * (H * hs + 2 * KV * hs) + 2 * T * H * hs * d + 3 * 2 * T * d * I
    attn = 2 * 2 * (T * (T + 1) // 2) * hs * H
    return L * (per_layer + attn) + 2 * V * d


def run_decode(model, cfg, batch, steps, warmup, prompt_len=PROMPT_LEN, clock=None):
    """Prefill ``batch`` prompts of ``prompt_len`` tokens, then time ``steps`` decode steps through
    the public engine: every step's token ids go in from the host (copied from pinned memory even
    where the device already holds them from its own sampling, which the library would skip) and
    the sampled ids come back to the host.  One loop, two clocks: CUDA events around the steps
    (device time) and the wall clock around the same steps (end to end); an event between steps
    gives the per-step times."""
    import torch
    from bitnet_c_b200.engine import ModelEngine
    from bitnet_c_b200.engine.batch import SeqStep
    from bitnet_c_b200.sampling import SamplingParams
    from bitnet_c_b200.csrc import ops

    g = torch.Generator().manual_seed(1234 + batch)
    prompts = torch.randint(0, cfg["vocab_size"], (batch, prompt_len), generator=g).tolist()
    cache = model.new_cache(max_tokens=batch * cfg["max_position_embeddings"], max_seqs=batch)
    eng = ModelEngine(model, cache, SamplingParams(temperature=0.0), always_upload=True)
    eng.start_batch(0, prompts)
    slots = [eng.open() for _ in range(batch)]
    rows = list(range(batch))
    # prompts in groups so that the activations of many long prompts need not live at once
    group = max(1, 4096 // prompt_len)
    toks = []
    for a in range(0, batch, group):
        idx = list(range(a, min(batch, a + group)))
        toks += eng.step_and_sample([SeqStep(slots[i], prompts[i], [prompt_len - 1]) for i in idx], idx)

    def one_step(t):
        return eng.step_and_sample([SeqStep(slots[i], [t[i]], [0]) for i in range(batch)], rows)

    if clock is not None:
        clock.launch()
    for _ in range(warmup):
        toks = one_step(toks)
    torch.cuda.synchronize()
    ops.LAUNCHES = 0
    h2d_before = eng.h2d_bytes()
    if clock is not None:
        clock.start()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    t0 = time.perf_counter()
    marks[0].record()
    for i in range(steps):
        toks = one_step(toks)
        marks[i + 1].record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    dev_ms = marks[0].elapsed_time(marks[-1])
    per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
    clocks = clock.stop() if clock is not None else None
    launches = ops.LAUNCHES
    ctx_len = prompt_len + warmup + steps // 2
    h2d = (eng.h2d_bytes() - h2d_before) // max(1, steps)
    for s in slots:
        eng.close(s)
    del cache, eng
    torch.cuda.empty_cache()
    return {"dev_ms": dev_ms, "wall_ms": wall_ms, "median_ms": per_step[len(per_step) // 2], "launches": launches,
            "clocks": clocks, "context": ctx_len, "h2d": h2d, "d2h": 4 * batch}


def run_prefill(model, cfg, warmup=3, iters=5):
    import torch
    from bitnet_c_b200.engine.batch import SeqStep
    g = torch.Generator().manual_seed(99)
    prompt = torch.randint(0, cfg["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
    cache = model.new_cache(max_tokens=cfg["max_position_embeddings"], max_seqs=1)
    times = []
    for i in range(warmup + iters):
        slot = cache.open()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        logits = model.step(cache, [SeqStep(slot, prompt, [PREFILL_TOKENS - 1])])
        e.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(s.elapsed_time(e))
        cache.close(slot)
    del cache, logits
    torch.cuda.empty_cache()
    times.sort()
    return times[len(times) // 2]


WORKLOADS = {
    # name: (configuration, prompt lengths or None for 64 drawn from 1..2,048, new tokens per request)
    "1b": (LLAMA_1B, None, 256),
    "13b": (LLAMA_13B, [2048, 1024, 512, 256, 128, 64, 16, 1], 1024),
}


def run_workload(name, repeats=2):
    """The generation workloads of the two other size sets, through the Python entry point:
    1b: 64 requests with prompts of 1 to 2,048 tokens (one ragged prefill step), 256 greedy tokens
    each; 13b: 8 requests with prompts of 2,048 down to 1 tokens, 1,024 greedy tokens each.  The
    first run warms libraries, recorded steps and memory pools; the fastest of the others counts."""
    import torch
    import bitnet_c_b200 as bn
    from bitnet_c_b200.engine import Model
    base, lens, new = WORKLOADS[name]
    cfg = dict(base)
    g = torch.Generator().manual_seed(7)
    if lens is None:
        lens = torch.randint(1, 2049, (64,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    model = Model.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0", norm_std=0.0)
    times = []
    for _ in range(1 + repeats):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = bn.generate(model, prompts, max_new_tokens=new, temperature=0.0, stop_ids=[])
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
    made = sum(len(c.tokens) for c in out)
    # what the decode steps alone had to read, at the batch's mean length over the run
    kv_per_token = 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    mean_live = sum(lens) + len(lens) * new / 2
    step_bytes = weight_bytes(model) - (0 if model.head is model.embedding else model.embedding.numel() * 2) + mean_live * kv_per_token
    del model
    torch.cuda.empty_cache()
    best = min(times[1:])
    return {"metric": f"generated tokens/s, {name} workload (prefill of {sum(lens)} prompt tokens included)",
            "value": round(made / best, 1), "unit": "tokens/s", "seconds": round(best, 3),
            "seconds_all": [round(t, 3) for t in times], "generated": made, "prompt_tokens": sum(lens),
            "requests": len(lens), "decode_step_gb": round(step_bytes / 1e9, 2), "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {"model": f"llama-{name}-sizes-random", "layers": cfg["num_hidden_layers"],
                       "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                       "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                       "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                       "seq_len": cfg["max_position_embeddings"], "new_tokens": new}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--skip-points", action="store_true", help="only the main decode run (quick runs, profiling)")
    ap.add_argument("--only-prefill", action="store_true", help="run only the 2,048-token prefill and print its record (profiling)")
    ap.add_argument("--batch", type=int, default=8, help="batch of the main decode run (default 8; other values for profiling)")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), help="run the generation workload of another size set instead")
    ap.add_argument("--own-gemm", choices=["off", "fused", "all"],
                    help="which many-row products run on the library's own tcgen05 kernel (gemm_tc.cu) instead of cuBLAS: "
                         "none, those whose epilogue replaces a separate kernel (the library's default), or all "
                         "(comparisons, profiling)")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="compute type of the main decode run (float32: profiling of the 32-bit path, with --skip-points)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload:
        print(json.dumps(run_workload(args.workload)))
        return 0
    warmup = max(3, args.warmup)

    import torch
    from bitnet_c_b200.engine import Model

    cfg = dict(LLAMA_8B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    if args.own_gemm:
        from bitnet_c_b200.csrc import ops
        ops.USE_OWN_GEMM = {"off": False, "fused": "fused", "all": True}[args.own_gemm]
    if args.dtype == "float32":
        if not (args.skip_points or args.only_prefill):
            print("bench.py: --dtype float32 times the main run only; give --skip-points or --only-prefill")
            return 2
        torch.backends.cuda.matmul.allow_tf32 = False
    model = Model.from_random(cfg, seed=0, dtype=args.dtype, device="cuda:0", norm_std=0.0)

    def prefill_record(m, c, ms, peak_tflops):
        fl = prefill_flops(c, PREFILL_TOKENS)
        return {"value": round(PREFILL_TOKENS / (ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                "frac": round(fl / (ms / 1e3) / (peak_tflops * 1e12), 4)}

    if args.only_prefill:
        rec = prefill_record(model, cfg, run_prefill(model, cfg, warmup=2, iters=3), pk["bf16_tflops"])
        rec["layers"] = cfg["num_hidden_layers"]
        from bitnet_c_b200.csrc import ops as _ops
        rec["many_row_products"] = {False: "library", "fused": "gemm_tc where its epilogue replaces a kernel, else library",
                                    True: "gemm_tc"}[_ops.USE_OWN_GEMM]
        print(json.dumps({"prefill": rec}))
        return 0
    B = args.batch
    short_dtype = "bf16" if args.dtype == "bfloat16" else "fp32"
    # the prefill first: it is a burst of matrix products of a seventh of a second, and what it is
    # compared with is the burst peak; after seconds of decoding the GPU sits at its power cap
    pre_ms = None if args.skip_points else run_prefill(model, cfg)
    run = run_decode(model, cfg, B, args.steps, warmup, clock=ClockSampler())
    ms_per_step = run["dev_ms"] / args.steps
    value = B * args.steps / (run["dev_ms"] / 1e3)
    e2e_value = B * args.steps / (run["wall_ms"] / 1e3)
    read_bytes = decode_read_bytes(model, cfg, B, run["context"])
    achieved = read_bytes / (ms_per_step / 1e3) / 1e9

    out = {
        "metric": f"decode tokens/s at batch {B} (Llama-3.1-8B sizes, {short_dtype})", "value": round(value, 2), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms_per_step, 4),
        "ms_per_step_median": round(run["median_ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": short_dtype, "data": "synthetic", "impl": "ours",
        "config": {"model": "llama-3.1-8b-sizes-random", "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": B, "seq_len": cfg["max_position_embeddings"], "prompt_len": PROMPT_LEN,
                   "rope_theta": cfg["rope_theta"], "rms_norm_eps": cfg["rms_norm_eps"], "tied": False,
                   "parallelism": "single-gpu", "l2": "inputs larger than L2 (15 GB of weights per step)",
                   "peaks": pk["source"], "fp32_layers": FP32_LAYERS,
                   "timing": "one loop: value by CUDA events around its steps, e2e by the wall clock around the same steps"},
        "clocks": run["clocks"],
        "e2e": {"value": round(e2e_value, 2), "unit": "tokens/s", "h2d_bytes_per_step": run["h2d"],
                "d2h_bytes_per_step": run["d2h"]},
        "gpu_launches": run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if not args.skip_points:
        out["prefill"] = prefill_record(model, cfg, pre_ms, pk["bf16_tflops"])
        points, fracs = {}, {}
        short = min(args.steps, 32)  # the further points take fewer steps each

        def point(name, m, c, b, steps, prompt_len):
            r = run_decode(m, c, b, steps, warmup, prompt_len=prompt_len)
            points[name] = round(b * steps / (r["dev_ms"] / 1e3), 2)
            fracs[name] = round(decode_read_bytes(m, c, b, r["context"]) / (r["dev_ms"] / steps / 1e3) / 1e9 / pk["hbm_gbs"], 4)

        for b in (1, 64):
            point(f"decode_b{b}", model, cfg, b, args.steps, PROMPT_LEN)
        for ctx in (2048, 3900):  # longer contexts: the cache of the live requests becomes the larger part
            for b in (1, 8, 64):
                point(f"decode_b{b}_ctx{ctx}", model, cfg, b, short, ctx)
        del model
        torch.cuda.empty_cache()
        # the true 32-bit path at the same layer sizes, FP32_LAYERS of the layers (named in config)
        cfg32 = dict(cfg, num_hidden_layers=min(FP32_LAYERS, cfg["num_hidden_layers"]))
        torch.backends.cuda.matmul.allow_tf32 = False
        m32 = Model.from_random(cfg32, seed=0, dtype="float32", device="cuda:0", norm_std=0.0)
        point("decode_b8_fp32", m32, cfg32, 8, short, PROMPT_LEN)
        p32 = run_prefill(m32, cfg32, warmup=1, iters=3)
        out["prefill_fp32"] = {"value": round(PREFILL_TOKENS / (p32 / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(p32, 3),
                               "layers": cfg32["num_hidden_layers"]}
        del m32
        torch.cuda.empty_cache()
        for name in sorted(WORKLOADS):
            w = run_workload(name, repeats=2)
            points[f"workload_{name}"] = w["value"]
            new = WORKLOADS[name][2]
            # the whole run's time (prefill included) spread over its decode steps: a lower bound of the
            # decode steps' fraction of the copy bandwidth
            fracs[f"workload_{name}"] = round(w["decode_step_gb"] / (w["seconds"] / new) / pk["hbm_gbs"], 4)
            out[f"workload_{name}"] = {"seconds": w["seconds"], "generated": w["generated"], "prompt_tokens": w["prompt_tokens"],
                                       "requests": w["requests"], "decode_step_gb": w["decode_step_gb"]}
        out["points"] = points
        out["points_frac"] = fracs
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
