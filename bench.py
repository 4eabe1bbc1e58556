#!/usr/bin/env python
"""Benchmark of the forward-pass hot path: Qwen3-4B-shaped Q4_K_M decode (and prefill) tok/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0). A step is one single-token decode step at batch 1 after a 512-token prompt
(el bench --pp 512 --tg K of the reference, src/main.cpp:621-648, seeded synthetic weights, LCG token stream).
  value      decode tok/s with tokens and weights resident on the device (CUDA events around K back-to-back steps)
  e2e        the same K steps through Backend.eval: host token in, host logits out, copies inside the timed region
  roofline   the dominant kernel of the timed region: the persistent decode-step kernel (algorithmic bytes = all
             weights once + the KV rows read), live CUDA-event time; roofline_gemv is the Q4_K matvec 2560 x 9728
             (4 limbs) timed alone over 24 weight copies in rotation
  cpu_baseline  the reference's CPU path on the host cores, bounded sample (N=1, rank 0 only)
--impl reference times only that CPU path.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from exactinfer_b200 import synth  # noqa: E402

PROMPT = 512
SEED = 20251125
MICRO_ROWS, MICRO_N = 2560, 9728
MICRO_BYTES = MICRO_ROWS * (MICRO_N // 256) * 144  # 14 008 320 algorithmic bytes per matvec
INT8_PEAK_TOPS = 4500.0  # nominal dense int8
# The measured-peaks file has no int8 figure. A library int8 GEMM (torch._int_mm, 8192^3 and 16384x8192x8192, 20 launches
# by CUDA events) reached 2857-2890 TOP/s on this pool's B200s: the practical ceiling of the int8 tensor pipe here.
INT8_PROBE_TOPS = 2870.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu captures summarised under profiles/: the figures
# live in profiles/dram_traffic.txt (JSON) next to the summaries they were read from (kernel -> workload -> bytes)
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "dram_traffic.txt")


def traffic_table():
    try:
        return json.load(open(TRAFFIC_FILE))
    except (OSError, ValueError):
        return {}


def micro_traffic():
    t = traffic_table().get("k_gemv", {}).get("q4_k_2560x9728")
    return None if t is None else float(t["bytes_per_launch"])


def decode_traffic(spec):
    """DRAM bytes per k_decode_step launch, scaled per layer from the captures on 4 and 8 layers of the same shape
    (fixed part for head and embedding row + a per-layer part, at positions ~517). None for shapes not captured."""
    t = traffic_table().get("k_decode_step", {}).get(spec.name)
    return None if t is None else float(t["fixed_bytes"]) + float(t["per_layer_bytes"]) * spec.n_layer


def metric_name(spec):
    return f"{spec.name} decode tok/s (batch 1, after pp{PROMPT}; prefill tok/s under \"prefill\")"


def workload_name(spec, K):
    return (f"{spec.name}: {spec.n_layer} layers, E{spec.n_embd} F{spec.n_ff} H{spec.n_head}/{spec.n_head_kv} "
            f"V{spec.n_vocab}, batch 1, pp{PROMPT} then tg{K}")


def big_model(spec):
    return spec_macs_per_token(spec) > 8e9


def spec_macs_per_token(spec):
    """Multiply-accumulates of the linear layers for one token (head excluded: prefill computes it once per chunk)."""
    qd, kd = spec.n_head * spec.head_dim, spec.n_head_kv * spec.head_dim
    per_layer = spec.n_embd * (qd + 2 * kd) + qd * spec.n_embd + 3 * spec.n_embd * spec.n_ff
    return float(spec.n_layer * per_layer)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--workload", default="qwen3-4b-q4_k_m", choices=sorted(synth.SPECS))
    ap.add_argument("--layers", type=int, default=0, help="truncate the model to this many layers (debugging only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tp32b", action="store_true", help="skip the 32B-shaped block (tp_32b) of the default workload")
    ap.add_argument("--cpu-seconds", type=float, default=20.0)
    ap.add_argument("--cpu-full", action="store_true",
                    help="time the reference CPU build on its whole benchmark procedure (warm-up, 512-token prompt pass, "
                         "128 single-token steps from position 0) instead of a bounded sample")
    ap.add_argument("--batch", type=int, default=1,
                    help="concurrent sequences: above 1 the run is the batched workload (each sequence a --prompt-token "
                         "prompt, then --steps batched steps, one row per sequence)")
    ap.add_argument("--prompt", type=int, default=4096, help="prompt length of the batched workload")
    ap.add_argument("--gemm-micro", action="store_true",
                    help="only time the prompt-chunk GEMM on the five linear shapes of the 4B model at 512 tokens")
    return ap.parse_args()


def int8_probe(device: int):
    """Peak of the int8 tensor pipe as a library GEMM reaches it on this GPU, measured in this run: torch._int_mm at
    8192^3, best of 10 launches by CUDA events (TOP/s = 2 N^3 / t). The denominator of the prompt pass's roofline: the
    driver-written peaks file has no int8 figure. None when the probe cannot run."""
    try:
        import torch
        dev = torch.device("cuda", device)
        n = 8192
        a = torch.randint(-127, 127, (n, n), dtype=torch.int8, device=dev)
        b = torch.randint(-127, 127, (n, n), dtype=torch.int8, device=dev)
        for _ in range(3):
            torch._int_mm(a, b)
        best = None
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            e1.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        del a, b
        torch.cuda.empty_cache()
        return 2.0 * n ** 3 / (best / 1000.0) / 1e12
    except Exception as exc:  # noqa: BLE001 - a missing probe must not cost the benchmark line
        print(f"bench: int8 probe unavailable ({exc})", file=sys.stderr)
        return None


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.remove(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return rank, local, world


def get_spec(args):
    spec = synth.SPECS[args.workload]
    if args.layers:
        import dataclasses
        spec = dataclasses.replace(spec, n_layer=args.layers)
    return spec


def model_tensors(spec):
    t0 = time.time()
    # models above ~8 GB reuse the random blocks of layers 0 and 1 for the later layers of the same parity (types and
    # shapes unchanged, every layer still has its own copy in HBM): host generation time only
    tens = list(synth.generate(spec, SEED, share_layers=big_model(spec)))
    return tens, time.time() - t0


# ---------------------------------------------------------------- CPU baseline (the reference's CPU path)

def physical_cores() -> int:
    """Physical cores this process may run on: distinct (package, core) pairs of /proc/cpuinfo among the CPUs of the
    affinity mask; the size of the mask when that cannot be read."""
    try:
        allowed = os.sched_getaffinity(0)
    except AttributeError:
        allowed = set(range(os.cpu_count() or 1))
    try:
        cores, cpu, pkg = set(), None, 0
        for line in open("/proc/cpuinfo"):
            k, _, v = line.partition(":")
            k, v = k.strip(), v.strip()
            if k == "processor":
                cpu, pkg = int(v), 0
            elif k == "physical id":
                pkg = int(v)
            elif k == "core id" and cpu in allowed:
                cores.add((pkg, int(v)))
        if cores:
            return len(cores)
    except (OSError, ValueError):
        pass
    return max(1, len(allowed))


def cpu_decode_baseline(spec, tens, seconds: float, max_steps: int, gpu_context: int = PROMPT):
    """Decode tok/s of the reference CPU backend on the host cores, on a bounded sample: one warm-up token, then
    single-token steps from position 1 until `seconds` have passed (at most max_steps). Uses the reference's own code
    (oracle/_ref/libelref.so over a GGUF written to a temporary file) when that build is present, else the restated
    oracle (bit-identical, same OpenMP structure)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol

    toks = synth.lcg_tokens(max_steps + 1, spec.n_vocab)
    n_ctx = max_steps + 2
    tmp = None
    want = physical_cores()
    if ol.have_ref():
        kind = "reference"
        tmp = tempfile.mkdtemp(prefix="elb_bench_")
        path = os.path.join(tmp, "model.gguf")
        synth.write_gguf(path, spec, tens)
        # the thread count is set explicitly (a launcher such as torch.distributed.run exports OMP_NUM_THREADS=1)
        ol.ref().ref_set_threads(want)
        model = ol.RefModel(path, n_ctx)
        cores = ol.ref().ref_threads()
    else:
        kind = "port"
        ol.oracle().orc_set_threads(want)
        model = ol.OracleModel(spec, tens, n_ctx)
        cores = ol.oracle().orc_threads()
    model.eval(toks[:1], 0)  # warm-up
    t0 = time.perf_counter()
    done = 0
    while done < max_steps and (done < 2 or time.perf_counter() - t0 < seconds):
        model.eval(toks[done + 1:done + 2], done + 1)
        done += 1
    dt = time.perf_counter() - t0
    model.close()
    if tmp:
        import shutil
        shutil.rmtree(tmp, ignore_errors=True)
    return {"value": done / dt, "unit": "tok/s", "cores": int(cores), "physical_cores": int(want), "kind": kind,
            "sample": f"{done} single-token decode steps at positions 1..{done} of the same model (1 warm-up token; "
                      f"context shorter than the GPU run's {gpu_context}+), {dt:.1f} s"}, done, dt


def cpu_full_bench(spec, tens, pp=PROMPT, tg=128):
    """The reference's own benchmark procedure (`bench --backend cpu --pp 512 --tg 128`, src/main.cpp:621-647 of the
    reference) on its CPU backend, all physical cores: 8 warm-up tokens, one timed pass over pp prompt tokens at position
    0, then tg timed single-token evaluations at positions 0..tg-1 of the same token stream."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    import shutil

    want = physical_cores()
    toks = synth.lcg_tokens(max(pp, tg), spec.n_vocab)
    tmp = None
    if ol.have_ref():
        kind = "reference"
        tmp = tempfile.mkdtemp(prefix="elb_bench_")
        path = os.path.join(tmp, "model.gguf")
        synth.write_gguf(path, spec, tens)
        ol.ref().ref_set_threads(want)
        model = ol.RefModel(path, max(pp, tg) + 1)
        cores = ol.ref().ref_threads()
    else:
        kind = "port"
        ol.oracle().orc_set_threads(want)
        model = ol.OracleModel(spec, tens, max(pp, tg) + 1)
        cores = ol.oracle().orc_threads()
    model.eval(toks[:8], 0)
    t0 = time.perf_counter()
    model.eval(toks[:pp], 0)
    t1 = time.perf_counter()
    for i in range(tg):
        model.eval(toks[i:i + 1], i)
    t2 = time.perf_counter()
    model.close()
    if tmp:
        shutil.rmtree(tmp, ignore_errors=True)
    return {"value": tg / (t2 - t1), "unit": "tok/s", "prefill_tok_s": pp / (t1 - t0), "cores": int(cores),
            "physical_cores": int(want), "kind": kind,
            "sample": f"the whole procedure of the reference's bench command: 8 warm-up tokens, pp{pp} in {t1 - t0:.1f} s, "
                      f"tg{tg} (positions 0..{tg - 1}) in {t2 - t1:.1f} s"}


def run_reference(args):
    rank, local, world = dist_env()
    if rank != 0:
        return
    spec = get_spec(args)
    tens, _ = model_tensors(spec)
    budget = 150.0
    if args.cpu_full:
        base = cpu_full_bench(spec, tens)
        done, dt = 128, 128 / base["value"]
    else:
        base, done, dt = cpu_decode_baseline(spec, tens, budget, max(2, args.steps))
    out = {"impl": "reference", "metric": metric_name(spec), "value": base["value"], "unit": "tok/s",
           "n_gpus": args.gpus, "steps": done, "steps_requested": args.steps, "warmup": 1,
           "ms_per_step": 1000.0 * dt / done, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic", "config": {"workload": workload_name(spec, args.steps),
                      "sample": base["sample"] if args.cpu_full else
                      "CPU path, single-token steps from position 1 (no 512-token prompt: it alone would "
                      "take minutes on the host), bounded to 150 s"},
           "cpu_baseline": base,
           "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(json.dumps(out))


# ---------------------------------------------------------------- the dominant kernel alone (roofline)

def microbench_matvec(e, device, iters=480, copies=24):
    """Q4_K matvec 2560 x 9728 with a 4-limb N(0,1) activation, `copies` distinct weights in rotation (336 MB, larger
    than the 126 MB L2) so that every launch streams its weight from HBM. Average device time per launch in ms."""
    import ctypes as C
    from exactinfer_b200 import capi
    rng = np.random.default_rng(SEED + 1)
    ws = [e.Weight(synth.Q4_K, MICRO_ROWS, MICRO_N, synth.rand_q4_k(rng, MICRO_ROWS, MICRO_N), device=device)
          for _ in range(copies)]
    x = e.DeviceBuffer.from_array(rng.normal(size=MICRO_N).astype(np.float32), device)
    y = e.DeviceBuffer(MICRO_ROWS * 4, device)
    arr = (C.c_void_p * copies)(*[w._h for w in ws])
    ms = C.c_float()
    capi.check(capi.lib().elb_bench_matvec(arr, copies, x.ptr, y.ptr, 4, iters, C.byref(ms)))
    for w in ws:
        w.close()
    return ms.value


def microbench_gemm(args):
    """The limb GEMM (split of the 512 fp32 rows + k_gemm_tc) on the linear shapes of the Qwen3-4B layer with the limb
    counts the model uses, 4 weight copies in rotation, best of 3 runs of 40 launches; one JSON line."""
    import ctypes as C
    import exactinfer_b200 as e
    from exactinfer_b200 import capi
    shapes = (("q", 4096, 2560, 4), ("k", 1024, 2560, 4), ("attn_output", 2560, 4096, 3), ("gate|up", 19456, 2560, 3),
              ("ffn_down", 2560, 9728, 4))
    rng = np.random.default_rng(SEED + 2)
    out = {"metric": "k_gemm_tc microbenchmark, Q4_K, 512 tokens (limb split included)", "unit": "us", "shapes": {}}
    for name, rows, n, nl in shapes:
        base = synth.rand_q4_k(rng, rows, n)
        ws = [e.Weight(synth.Q4_K, rows, n, base, planes=True) for _ in range(4)]
        x = e.DeviceBuffer.from_array(rng.normal(size=(PROMPT, n)).astype(np.float32))
        y = e.DeviceBuffer(rows * PROMPT * 4)
        arr = (C.c_void_p * 4)(*[w._h for w in ws])
        ms, best = C.c_float(), 1e9
        for _ in range(3):
            capi.check(capi.lib().elb_bench_matmul(arr, 4, x.ptr, PROMPT, y.ptr, nl, 40, C.byref(ms)))
            best = min(best, ms.value)
        out["shapes"][f"{name} {rows}x{n} nl{nl}"] = {"us": best * 1e3, "tops_single_count": 2.0 * rows * n * PROMPT / best / 1e9}
        for w in ws:
            w.close()
    emit(json.dumps(out))


# ---------------------------------------------------------------- tensor parallelism: parity first, then the 32B shape

TP_REL_TOL, TP_LOGPROB_TOL = 2e-4, 3e-5  # the bars of tests/test_gpu_tp.py


def tp_parity(e, make_tp, local):
    """Every rank evaluates a small model (uneven FFN cut, vocabulary not a multiple of 16) through the tensor-parallel
    backend - the persistent decode kernel with its peer-memory exchange, then the kernel-per-op path - and compares the
    gathered logits with the CPU oracle's whole-model result: the check of tests/tp_gpu_worker.py, run where the
    multi-GPU numbers are taken. Returns (worst relative logit error, worst |delta logprob|, ok)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol

    # 8 KV heads (2, 4 and 8 ranks divide them), 11 FFN blocks (an uneven cut at every rank count), odd vocabulary
    spec = synth.Spec(name="tp-small", n_layer=3, n_embd=512, n_ff=2816, n_head=16, n_head_kv=8, n_vocab=2043,
                      layout="q4_k_m", head_sigma=2e-5)
    tens = list(synth.generate(spec, 33))
    n_prompt, n_decode = 40, 5
    cpu = ol.OracleModel(spec, tens, n_prompt + n_decode + 1)
    toks = list(synth.lcg_tokens(n_prompt, spec.n_vocab))
    ref = [cpu.eval(toks, 0)]
    for i in range(n_decode):
        toks.append(int(np.argmax(ref[-1])))
        ref.append(cpu.eval(toks[-1:], n_prompt + i))
    cpu.close()

    def rel(a, b):
        return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(np.abs(b).max(), 1e-30))

    def logprobs(l):
        return l.astype(np.float64) - ol.logsumexp(l)

    worst_rel = worst_lp = 0.0
    paths = []
    for no_mega in ("0", "1"):
        os.environ["ELB_TP_NO_MEGA"] = no_mega
        gpu = e.Backend(spec, tens, n_prompt + n_decode + 1, device=local, tp=make_tp())
        got = [gpu.eval(toks[:n_prompt], 0)]
        for i in range(n_decode):
            got.append(gpu.eval(toks[n_prompt + i:n_prompt + i + 1], n_prompt + i))
        paths.append(int(gpu.last_eval_stats()[1]))
        gpu.close()
        for g, r in zip(got, ref):
            top = np.argsort(r)[-8:]
            worst_rel = max(worst_rel, rel(g, r))
            worst_lp = max(worst_lp, float(np.abs(logprobs(g)[top] - logprobs(r)[top]).max()))
    os.environ.pop("ELB_TP_NO_MEGA", None)
    return worst_rel, worst_lp, bool(worst_rel <= TP_REL_TOL and worst_lp <= TP_LOGPROB_TOL), paths


def bench_32b(e, tp, local, world, dist, barrier, max_over_ranks, hbm, steps):
    """The configuration tensor parallelism is meant for: the 32B shape, one sequence (2048-token prompt, then single-token
    steps) and sixteen sequences (512-token prompts, then batched steps), on `world` GPUs."""
    spec = synth.SPECS["qwen3-32b-q4_k_m"]
    tens = list(synth.generate(spec, SEED, share_layers=True))
    P1, PB, NB = 2048, 512, 16
    out = {"workload": f"{spec.name}: {spec.n_layer} layers, E{spec.n_embd} F{spec.n_ff} H{spec.n_head}/{spec.n_head_kv}, "
                       f"prompt {P1} then {steps} steps (batch 1); {NB} sequences with {PB}-token prompts then {steps} batched steps"}
    model = e.Backend(spec, tens, P1 + steps + 4, device=local, tp=tp, max_batch=PROMPT, n_seq=NB)  # one upload for both parts
    toks = synth.lcg_tokens(P1 + steps + 3 + NB, spec.n_vocab)
    # ---- sixteen sequences: rows of a batch carry their own sequence and position; no logits are read back
    for sq in range(NB):
        model.eval_batch(toks[:PB], np.full(PB, sq, np.int32), np.arange(PB, dtype=np.int32), want_logits=False)
    seq = np.arange(NB, dtype=np.int32)
    model.eval_batch(toks[PB:PB + NB], seq, np.full(NB, PB, np.int32), want_logits=False)  # warm-up step
    barrier()
    dev = []
    for i in range(steps):
        model.eval_batch(toks[PB + i:PB + i + NB], seq, np.full(NB, PB + 1 + i, np.int32), want_logits=False)
        dev.append(model.last_eval_stats()[0])
    ms16 = max_over_ranks(float(np.sum(dev)))
    out["batch16"] = {"decode_ms_per_step": ms16 / steps, "decode_tok_s": NB * steps / (ms16 / 1000.0),
                      "note": "one row per sequence and step, head not evaluated (no logits read back)"}
    # ---- batch 1 (sequence 0 again, from position 0)
    barrier()
    t1 = time.perf_counter()
    model.eval(toks[:P1], 0, want_logits=False)
    pp_s = max_over_ranks(time.perf_counter() - t1)
    model.eval_steps(toks[P1:P1 + 3], P1)
    barrier()
    ms = max_over_ranks(model.eval_steps(toks[P1 + 3:P1 + 3 + steps], P1 + 3))
    step_bytes = model.weight_bytes + model.kv_bytes_per_token * (P1 + 3 + steps / 2.0)
    step_s = ms / steps / 1000.0
    out["batch1"] = {"decode_ms_per_step": ms / steps, "decode_tok_s": steps / (ms / 1000.0), "prefill_tok_s": P1 / pp_s,
                     "per_gpu_bytes_per_step": step_bytes, "per_gpu_gbs": step_bytes / step_s / 1e9,
                     "hbm_frac_of_per_gpu_share": step_bytes / step_s / 1e9 / hbm,
                     "kernels_per_step": model.last_eval_stats()[1] / float(steps)}
    model.close()
    return out


# ---------------------------------------------------------------- our arm

def pinned_array(e, n_floats):
    import ctypes as C
    from exactinfer_b200 import capi
    p = C.c_void_p()
    capi.check(capi.lib().elb_host_alloc(n_floats * 4, C.byref(p)))
    return np.ctypeslib.as_array((C.c_float * n_floats).from_address(p.value)), p


def run_ours(args):
    rank, local, world = dist_env()
    n_gpus = world  # one rank per GPU; started without a launcher, --gpus N > 1 still runs the single-GPU path
    if args.gpus != world and rank == 0:
        print(f"bench: --gpus {args.gpus} but WORLD_SIZE is {world}; running on {world} GPU(s)", file=sys.stderr)
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import exactinfer_b200 as e
    ok, why = e.cuda_available()
    if not ok:
        raise SystemExit(f"bench: the CUDA path is unavailable ({why}); there is no CPU fallback")
    K, W = args.steps, max(args.warmup, 3)
    spec = get_spec(args)
    tens, gen_s = model_tensors(spec)
    t0 = time.time()
    def make_tp():
        """Tensor parallel: rank 0 makes the NCCL id of the library's own communicator, all ranks join it. An id serves
        one communicator, so every model gets its own."""
        if world == 1:
            return None
        box = [e.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return (rank, world, box[0])

    tp = make_tp()
    parity = None
    if world > 1:  # correctness of the tensor-parallel paths on these GPUs, before anything is timed
        r, lp, ok_tp, paths = tp_parity(e, make_tp, local)
        flags = [None] * world
        dist.all_gather_object(flags, (r, lp, ok_tp))
        parity = {"rel": max(f[0] for f in flags), "logprob": max(f[1] for f in flags), "ok": all(f[2] for f in flags),
                  "bars": {"rel": TP_REL_TOL, "logprob": TP_LOGPROB_TOL}, "kernels_per_step": paths,
                  "against": "CPU oracle, whole model, every rank; persistent kernel and kernel-per-op path"}
        if not parity["ok"]:
            if rank == 0:
                emit(json.dumps({"metric": metric_name(spec), "value": None, "n_gpus": n_gpus, "tp_parity": parity,
                                 "error": "tensor-parallel parity failed: nothing was timed"}))
            dist.barrier()
            dist.destroy_process_group()
            raise SystemExit(3)
        t0 = time.time()
    model = e.Backend(spec, tens, PROMPT + W + K + 1, device=local, tp=tp)
    load_s = time.time() - t0
    toks = synth.lcg_tokens(PROMPT + W + K, spec.n_vocab)
    logits, _pin = pinned_array(e, spec.n_vocab)

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v):
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- prefill pp512: one warm-up pass, then 3 timed passes (median); weights (GBs) exceed L2 between passes
    model.eval(toks[:PROMPT], 0, out=logits)
    pp_dev, pp_wall = [], []
    for _ in range(3):
        barrier()
        t1 = time.perf_counter()
        model.eval(toks[:PROMPT], 0, out=logits)
        pp_wall.append(time.perf_counter() - t1)
        pp_dev.append(model.last_eval_stats()[0] / 1000.0)
    pp_launches = model.last_eval_stats()[1]
    pp_dev_s, pp_wall_s = max_over_ranks(statistics.median(pp_dev)), max_over_ranks(statistics.median(pp_wall))

    # ---- decode: W warm-up steps, then exactly K timed steps (device events inside the library, on its stream)
    model.eval_steps(toks[PROMPT:PROMPT + W], PROMPT)
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    dev_ms = model.eval_steps(toks[PROMPT + W:PROMPT + W + K], PROMPT + W)
    launches = model.last_eval_stats()[1]
    barrier()
    dev_ms = max_over_ranks(dev_ms)

    # ---- the same K steps end to end: host token in, host logits out (pinned), each call synchronous
    barrier()
    t1 = time.perf_counter()
    for i in range(K):
        p = PROMPT + W + i
        model.eval(toks[p:p + 1], p, out=logits)
    e2e_s = max_over_ranks(time.perf_counter() - t1)
    clocks = sampler.stop() if rank == 0 else None

    peaks, peak_kind = measured_peaks()
    hbm = float(peaks["hbm_gbs"])
    weight_bytes, kv_bytes_per_token = model.weight_bytes, model.kv_bytes_per_token
    tp32 = None
    if args.workload == "qwen3-4b-q4_k_m" and not args.layers and not args.no_tp32b:
        model.close()  # the 32B shape takes the memory
        model = None
        tp32 = bench_32b(e, make_tp(), local, world, dist, barrier, max_over_ranks, hbm, max(8, min(K, 32)))
    if rank != 0:
        if model is not None:
            model.close()
        dist.barrier()
        dist.destroy_process_group()
        return
    micro_ms = microbench_matvec(e, local) if spec.layout != "f16" else None
    step_bytes = weight_bytes + kv_bytes_per_token * (PROMPT + W + K / 2.0)
    tok_s = K / (dev_ms / 1000.0)  # one sequence: under tensor parallelism the ranks share every step
    out = {
        "metric": metric_name(spec), "value": tok_s, "unit": "tok/s",
        "n_gpus": n_gpus, "steps": K, "warmup": W, "ms_per_step": dev_ms / K, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 limbs x quantized ints -> int32, fp32 scales",
        "data": "synthetic",
        "config": {"workload": workload_name(spec, K),
                   "parallelism": "single GPU" if world == 1 else
                   f"tp{world}: heads and FFN columns cut over {world} GPUs; decode: one persistent kernel per rank, partial "
                   "sums of attn_output and ffn_down and the logits rows exchanged through peer memory (kernel-per-op with "
                   "a peer-memory all-reduce when the step does not fit the kernel); prompt chunks: NCCL all-reduce",
                   "l2": "inputs larger than L2: every step streams all weights (GBs) from HBM",
                   "seed": SEED, "tokens": "reference LCG stream, seed 12345",
                   "weights": "two sets of random blocks shared by the layers of equal parity" if big_model(spec)
                   else "every layer drawn separately"},
        "e2e": {"value": K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 8,
                "d2h_bytes_per_step": spec.n_vocab * 4},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "prefill": {"value": PROMPT / pp_dev_s, "unit": "tok/s", "ms": pp_dev_s * 1000.0,
                    "e2e_tok_s": PROMPT / pp_wall_s, "gpu_launches": int(pp_launches)},
        "decode_hbm": {"per": "GPU (rank 0's share of the weights and KV rows)", "bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (dev_ms / K / 1000.0) / 1e9,
                       "frac_of_measured_copy": step_bytes / (dev_ms / K / 1000.0) / 1e9 / hbm,
                       "frac_of_8tbs": step_bytes / (dev_ms / K / 1000.0) / 1e9 / 8000.0},
        "setup_s": {"generate": gen_s, "upload": load_s},
        "reference_published": None if spec.name != "qwen3-4b-q4_k_m" else {"note": "the reference's own figures for this metric, on other hardware and real weights; "
                                        "nothing is published for B200, hence vs_baseline null",
                                "hardware": "RTX 2060 (docs/performance.md:18 of the reference)",
                                "decode_tok_s": [76, 81], "prefill_tok_s": [1100, 1140]},
    }
    # dominant kernel of the timed region: with one persistent launch per token it is the decode step itself
    step_s = dev_ms / K / 1000.0
    per_step = launches / float(K)
    if per_step < 4:
        ach = step_bytes / step_s / 1e9
        out["roofline"] = {"bound": "hbm", "kernel": "k_decode_step (one persistent launch per token: every matvec, "
                           "norm, RoPE, attention and SwiGLU of the step)", "achieved": ach, "peak": hbm, "unit": "GB/s",
                           "frac": ach / hbm, "peak_kind": peak_kind, "frac_of_8tbs": ach / 8000.0,
                           "bytes_per_launch": step_bytes, "us_per_launch": step_s * 1e6, "traffic": decode_traffic(spec)}
    if micro_ms is not None:
        ach = MICRO_BYTES / (micro_ms / 1000.0) / 1e9
        micro = {"bound": "hbm", "kernel": "k_gemv<Q4_K> 2560x9728, 4 limbs, alone (24 weight copies in rotation)",
                 "achieved": ach, "peak": hbm, "unit": "GB/s", "frac": ach / hbm, "peak_kind": peak_kind,
                 "frac_of_8tbs": ach / 8000.0, "bytes_per_launch": MICRO_BYTES, "us_per_launch": micro_ms * 1000.0,
                 "traffic": micro_traffic()}
        out["roofline_gemv"] = micro
        out.setdefault("roofline", micro)
    ops = 2.0 * spec_macs_per_token(spec)
    ach_tops = ops * out["prefill"]["value"] / 1e12
    if spec.layout in ("f16", "q8_0"):  # fp16 tensor pipe: the driver-measured bf16 GEMM peak is the denominator
        issued = 2 if spec.layout == "f16" else 3
        peak = float(peaks.get("bf16_tflops", 1590.0))
        out["prefill"]["roofline"] = {"bound": "tensor", "kernel": "k_gemm_f16_tc (tcgen05 kind::f16) + attention + splits",
                                      "achieved": ach_tops, "peak": peak, "unit": "TFLOP/s", "frac": ach_tops / peak,
                                      "peak_kind": peak_kind + " (bf16 GEMM burst figure of MEASURED_PEAKS.json)",
                                      "issued_over_counted": issued,
                                      "note": f"2*M*N*K counted once; the fp16 halves issue {issued}x that on the tensor pipe"}
    else:
        probe = int8_probe(local)
        out["prefill"]["roofline"] = {"bound": "tensor", "kernel": "k_gemm_tc (tcgen05 kind::i8) + attention + splits",
                                      "achieved": ach_tops, "peak": probe if probe else INT8_PROBE_TOPS, "unit": "TOP/s",
                                      "frac": ach_tops / (probe if probe else INT8_PROBE_TOPS),
                                      "peak_kind": "library int8 GEMM (torch._int_mm 8192^3) measured in this run" if probe else
                                      "library int8 GEMM measured earlier on this pool (the probe could not run)",
                                      "frac_of_nominal": ach_tops / INT8_PEAK_TOPS, "nominal_dense_int8": INT8_PEAK_TOPS,
                                      "note": "2*M*N*K counted once; the digit planes and limb columns issue 2*(NL+1) = 8-10x "
                                              "that on the tensor pipe"}
    if model is not None:
        model.close()
    if parity is not None:
        out["tp_parity"] = parity
    if tp32 is not None:
        out["tp_32b"] = tp32
    if n_gpus == 1 and not args.no_cpu_baseline:
        if args.cpu_full:
            out["cpu_baseline"] = cpu_full_bench(spec, tens)
        else:
            out["cpu_baseline"] = cpu_decode_baseline(spec, tens, args.cpu_seconds, 64)[0]
    emit(json.dumps(out))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_batched(args):
    """Many sequences on one GPU: --batch sequences, each with a --prompt-token prompt (chunks of 512 rows), then
    --steps batched decode steps with one row per sequence. value = rows per second of the timed steps up to the last
    layer; e2e evaluates the head as well and copies every row's logits to the host."""
    import exactinfer_b200 as e
    ok, why = e.cuda_available()
    if not ok:
        raise SystemExit(f"bench: the CUDA path is unavailable ({why}); there is no CPU fallback")
    spec = get_spec(args)
    tens, gen_s = model_tensors(spec)
    NB, P, K, W = args.batch, args.prompt, args.steps, max(args.warmup, 3)
    CH = 512
    t0 = time.time()
    model = e.Backend(spec, tens, P + W + K + 1, max_batch=CH, n_seq=NB)
    load_s = time.time() - t0
    toks = synth.lcg_tokens(P + W + K + NB + 1, spec.n_vocab)
    seq = np.arange(NB, dtype=np.int32)
    # ---- prompts: sequence s reads the token stream from offset s
    pp_ms, pp_launch = 0.0, 0
    t1 = time.perf_counter()
    for s in range(NB):
        for c0 in range(0, P, CH):
            n = min(CH, P - c0)
            model.eval_batch(toks[s + c0:s + c0 + n], np.full(n, s, np.int32), np.arange(c0, c0 + n, dtype=np.int32),
                             want_logits=False)
            st = model.last_eval_stats()
            pp_ms += st[0]
            pp_launch += st[1]
    pp_wall = time.perf_counter() - t1
    for i in range(W):
        model.eval_batch(toks[P + i:P + i + NB], seq, np.full(NB, P + i, np.int32), want_logits=False)
    sampler = ClockSampler(0)
    sampler.start()
    dev, launches = 0.0, 0
    t1 = time.perf_counter()
    for i in range(K):
        model.eval_batch(toks[P + W + i:P + W + i + NB], seq, np.full(NB, P + W + i, np.int32), want_logits=False)
        st = model.last_eval_stats()
        dev += st[0]
        launches += st[1]
    wall = time.perf_counter() - t1
    # the same step end to end, as a sampler would call it: head evaluated, every row's logits reduced on the device to
    # its best token and log-sum-exp (elb_model_eval_batch_top), host tokens in, 16 bytes per row out
    KH = min(K, 32)
    t1 = time.perf_counter()
    for i in range(KH):
        model.eval_batch_top(toks[P + W + i:P + W + i + NB], seq, np.full(NB, P + W + i, np.int32), k=1)
    head_wall = time.perf_counter() - t1
    # ... and with every row's full logits copied to the host instead (39 MB per step at 64 rows)
    KL = min(K, 4)
    t1 = time.perf_counter()
    for i in range(KL):
        model.eval_batch(toks[P + W + i:P + W + i + NB], seq, np.full(NB, P + W + i, np.int32), want_logits=True)
    logits_wall = time.perf_counter() - t1
    clocks = sampler.stop()
    peaks, peak_kind = measured_peaks()
    hbm = float(peaks["hbm_gbs"])
    step_s = dev / K / 1000.0
    kv_step = NB * model.kv_bytes_per_token * (P + W + K / 2.0)
    step_bytes = model.weight_bytes + kv_step
    out = {"metric": f"{spec.name} batched decode tok/s ({NB} sequences)", "value": NB * K / (dev / 1000.0), "unit": "tok/s",
           "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": dev / K, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "int8 limbs x quantized ints -> int32, fp32 scales", "data": "synthetic",
           "config": {"workload": f"{spec.name}: {spec.n_layer} layers, E{spec.n_embd} F{spec.n_ff} H{spec.n_head}/{spec.n_head_kv}, "
                                  f"{NB} sequences x {P}-token prompts, then {K} batched steps (one row per sequence)",
                      "l2": "inputs larger than L2: every step streams the weights and all sequences' KV rows from HBM",
                      "seed": SEED, "head": "timed steps stop at the last layer (no logits); e2e evaluates the head and reduces "
                                            "every row's logits on the device"},
           "e2e": {"value": NB * KH / head_wall, "unit": "tok/s", "h2d_bytes_per_step": NB * 12,
                   "d2h_bytes_per_step": NB * 16, "steps": KH,
                   "call": "elb_model_eval_batch_top(k = 1): head evaluated, best token and log-sum-exp of every row",
                   "full_logits_to_host_tok_s": NB * KL / logits_wall, "full_logits_bytes_per_step": NB * spec.n_vocab * 4,
                   "without_head_tok_s": NB * K / wall},
           "gpu_launches": int(launches), "clocks": clocks,
           "prefill": {"value": NB * P / (pp_ms / 1000.0), "unit": "tok/s", "ms": pp_ms, "e2e_tok_s": NB * P / pp_wall,
                       "gpu_launches": int(pp_launch)},
           "roofline": {"bound": "hbm", "kernel": "the batched step as a whole (attention over every sequence's KV rows "
                        "dominates the bytes)", "achieved": step_bytes / step_s / 1e9, "peak": hbm, "unit": "GB/s",
                        "frac": step_bytes / step_s / 1e9 / hbm, "peak_kind": peak_kind, "bytes_per_launch": step_bytes,
                        "kv_bytes_per_step": kv_step, "weight_bytes": model.weight_bytes, "us_per_launch": step_s * 1e6,
                        "traffic": None},
           "setup_s": {"generate": gen_s, "upload": load_s}}
    model.close()
    if not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_decode_baseline(spec, tens, args.cpu_seconds, 64, P)[0]
        out["cpu_baseline"]["sample"] += " (one sequence: the reference has no batched path)"
    emit(json.dumps(out))


def emit(line: str):
    os.write(REAL_STDOUT, (line + "\n").encode())


if __name__ == "__main__":
    # libraries (NCCL's version banner, for one) print to stdout: send file descriptor 1 to stderr for the whole run and
    # keep the real one for the single JSON line
    sys.stdout.flush()
    REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    a = parse_args()
    if a.gemm_micro:
        microbench_gemm(a)
    elif a.impl == "reference":
        run_reference(a)
    elif a.batch > 1:
        run_batched(a)
    else:
        run_ours(a)
