#!/usr/bin/env python
"""Benchmark of the hot path: LLaMA-7B-shaped batch-1 greedy decode (tok/s) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload 7b-fp16|7b-int8]

One "step" is one decode step (one new token through all layers, position advancing).  The
workload is the 7B configuration the metric is quoted on: random-init fp16 weights ~N(0, 0.02)
(seeded generator), 128-token seeded prompt, context 2048, K greedy steps after W warm-up steps.
Weights streamed per step (13.2 GB fp16) are far larger than the 126 MB L2, so no flush is needed.

Printed JSON line (rank 0):
  value     tok/s of K device-chained steps (token fed back on the device), CUDA events, max over ranks
  e2e       tok/s of K calls of the reference-facing entry point (lcu_context_next_token: host token
            in, host token out, one synchronisation per token), wall clock around the loop
  roofline  the dominant kernel (fused RMSNorm + w1|w3 + SiLU GEMV) timed alone over all layers in
            rotation with CUDA events: algorithmic bytes per launch / mean launch time vs the measured
            HBM copy bandwidth
  prefill   (N = 1) the prompt path: tok/s of a 512-token prompt through lcu_context_next_token, and the largest
            prompt GEMM (the stacked w1|w3 product, 512 x 4096 x 22016, tcgen05 kernel) timed alone with CUDA events against the measured
            dense bf16 tensor peak
  cpu_baseline  the CPU oracle on a bounded sample (one of the 32 layers + the output head), host threads
With N > 1 (torchrun) every rank runs an independent replica on its own GPU (the path does not
shard at batch 1: layers are sequentially dependent), value = N*K / max-rank time, scaling "weak".

--impl reference times the unmodified reference (its CUDA build for sm_100a, oracle/_ref) on the same
weights, prompt and step count through its own llama_context::next_token, timed as its main.cpp does.
"""
import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "tests"))

WORKLOADS = {
    "7b-fp16": dict(dim=4096, n_heads=32, n_layers=32, n_vocab=32000, block_size=0),
    "7b-int8": dict(dim=4096, n_heads=32, n_layers=32, n_vocab=32000, block_size=128),
    "13b-fp16": dict(dim=5120, n_heads=40, n_layers=40, n_vocab=32000, block_size=0),
    "65b-int8": dict(dim=8192, n_heads=64, n_layers=80, n_vocab=32000, block_size=128),
    "7b-l4-fp16": dict(dim=4096, n_heads=32, n_layers=4, n_vocab=32000, block_size=0),   # 7B kernel shapes, 4 layers: profiler captures
    "7b-l4-int8": dict(dim=4096, n_heads=32, n_layers=4, n_vocab=32000, block_size=128),
    "tiny-fp16": dict(dim=512, n_heads=4, n_layers=4, n_vocab=2000, block_size=0),  # plumbing checks only
}
SEED, SCALE, PROMPT_LEN, CONTEXT_LEN, TEMPERATURE = 1234, 0.02, 128, 2048, 0.8
# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu
# captures summarised in profiles/gemv_w13_7b_fp16.md and profiles/gemv_w13_7b_int8.md
NCU_TRAFFIC_BYTES = {"7b-fp16": 180413440 + 3508736, "7b-int8": 91672832 + 2845952}
PREFILL_LEN = 512


def load_package():
    if "llama_cu_b200" in sys.modules:
        return sys.modules["llama_cu_b200"]
    spec = importlib.util.spec_from_file_location("llama_cu_b200", os.path.join(ROOT, "llama.cu_b200", "__init__.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["llama_cu_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def decode_bytes_per_token(cfg, ffn, t_cached):
    """Algorithmic HBM bytes of one decode step at `t_cached` cached positions."""
    d, L, V, bs = cfg["dim"], cfg["n_layers"], cfg["n_vocab"], cfg["block_size"]
    p = L * (4 * d * d + 3 * d * ffn) + V * d
    w = 2 * p if bs == 0 else p + p // bs * 2
    norms = (2 * L + 1) * d * 2
    kv = 2 * L * d * 2 * (t_cached + 1) + 2 * L * d * 2
    return w + norms + d * 2 + kv


class ClockSampler:
    """nvidia-smi sampling (200 ms) of SM clock and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
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
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, copy bandwidth)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def measured_tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, cuBLAS burst)"
        except Exception:
            pass
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def prefill_sample(lcu, ctx, cfg, ffn, profile=False, PREFILL_LEN=PREFILL_LEN):
    """Prompt path: a PREFILL_LEN-token prompt through the public call (wall clock, host tokens in, token out),
    and the largest prompt GEMM alone (CUDA events) against the dense tensor peak."""
    import oracle_lib as O
    prompt = O.synth_tokens(PREFILL_LEN, SEED + 1, lo=3, hi=min(32000, cfg["n_vocab"]))
    best = None
    for _ in range(3):
        ctx.clear_tokens()
        lcu.check(lcu.lib.lcu_synchronize())
        t0 = time.perf_counter()
        ctx.next_token(prompt)
        dt = time.perf_counter() - t0
        best = dt if best is None or dt < best else best
    out = {"prompt_tokens": PREFILL_LEN, "ms": round(best * 1e3, 3), "tok_s": round(PREFILL_LEN / best, 1)}
    if profile:  # one more prompt pass and a few GEMM launches inside the profiler's window
        ctx.clear_tokens()
        lcu.check(lcu.lib.lcu_profiler_start())
        ctx.next_token(prompt)
        if cfg["block_size"] == 0:
            lcu.bench_matmul_f16_ms(2048, cfg["dim"], ffn, reps=2)
        lcu.check(lcu.lib.lcu_profiler_stop())
    if cfg["block_size"] == 0:
        peak, src = measured_tensor_peak()
        m, k, n = PREFILL_LEN, cfg["dim"], 2 * ffn  # the stacked w1|w3 product, the largest GEMM of a prompt pass
        ms = lcu.bench_matmul_f16_ms(m, k, n, reps=50)
        tf = 2.0 * m * k * n / (ms * 1e-3) / 1e12
        m2 = 2048
        ms2 = lcu.bench_matmul_f16_ms(m2, k, n, reps=20)
        tf2 = 2.0 * m2 * k * n / (ms2 * 1e-3) / 1e12
        out["gemm_roofline"] = {"bound": "tensor", "kernel": "gemm_tc_pair_kernel (tcgen05.mma cta_group::2, TMA-fed, accumulator in TMEM)",
                                "shape": [m, k, n], "us_per_launch": round(ms * 1e3, 2), "achieved": round(tf, 1), "peak": peak, "unit": "TFLOP/s",
                                "frac": round(tf / peak, 4), "peak_source": src,
                                "at_2048_rows": {"shape": [m2, k, n], "us_per_launch": round(ms2 * 1e3, 2), "achieved": round(tf2, 1),
                                                 "frac": round(tf2 / peak, 4)}}
    return out


def cpu_baseline_sample(cfg, ffn, steps=6):
    """CPU oracle on one layer + the head of the same shapes; extrapolated to all layers."""
    import numpy as np
    import oracle_lib as O

    t0 = time.time()
    om = O.OracleModel(dim=cfg["dim"], multiple_of=256, n_heads=cfg["n_heads"], n_layers=1, n_vocab=cfg["n_vocab"],
                       block_size=cfg["block_size"], seed=SEED, scale=SCALE, context_len=PROMPT_LEN + steps + 1, temperature=TEMPERATURE)
    gen_s = time.time() - t0
    tok = int(O.synth_tokens(1, SEED)[0])
    # a short prefix instead of the 128-token prompt keeps the sample bounded; attention is <1 % of a step here
    om.next_token([tok])
    lay, head = [], []
    for _ in range(steps):
        tok = om.next_token([tok])
        tl, th = O.lib().orc_last_timing(om.ctx, 0), O.lib().orc_last_timing(om.ctx, 1)
        lay.append(tl)
        head.append(th)
    om.close()
    t_token = cfg["n_layers"] * min(lay) + min(head)
    return {"value": 1.0 / t_token, "unit": "tok/s", "cores": O.lib().orc_num_threads(), "kind": "port",
            "sample": f"CPU oracle (oracle/oracle.cpp, OpenMP over output rows): 1 of {cfg['n_layers']} layers + output head of the "
                      f"{cfg['dim']}-dim model, best of {steps} decode steps, layer time x {cfg['n_layers']} + head time; "
                      f"weights generated in {gen_s:.1f} s (not timed)"}


def dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
        dist_mod.init_process_group(backend="nccl" if torch.cuda.is_available() else "gloo")
        dist = dist_mod
    return world, rank, local, dist


def reduce_max_time(ms, dist, device=None):
    """max over ranks of a per-rank duration (the job ends when the slowest replica ends)"""
    if dist is None:
        return ms
    import torch
    t = torch.tensor([ms], dtype=torch.float64, device=device or ("cuda" if torch.cuda.is_available() and dist.get_backend() == "nccl" else "cpu"))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync(dist, lcu):
    lcu.check(lcu.lib.lcu_synchronize())
    if dist is not None:
        dist.barrier()
    lcu.check(lcu.lib.lcu_synchronize())


def run_ours(args):
    import numpy as np
    import oracle_lib as O

    world, rank, local, dist = dist_setup(args.gpus)
    lcu = load_package()
    if lcu.lib.lcu_device_count() < 1:
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    lcu.check(lcu.lib.lcu_set_device(local))
    cfg = WORKLOADS[args.workload]
    ffn = lcu.lib.lcu_ffn_dim(cfg["dim"], 256)
    K, W = args.steps, args.warmup
    PROMPT_LEN = args.prompt_len
    ctx_len = max(CONTEXT_LEN, PROMPT_LEN + W + K + 2)
    layer_gpus = None
    if args.pipeline > 1:  # one process, layers split evenly over the first P devices (the reference's pipelined configurations)
        if world > 1:
            raise SystemExit("--pipeline is a single-process mode; launch it without torchrun")
        if lcu.lib.lcu_device_count() < args.pipeline:
            raise SystemExit(f"--pipeline {args.pipeline} needs {args.pipeline} GPUs")
        per = (cfg["n_layers"] + args.pipeline - 1) // args.pipeline
        layer_gpus = [min(i // per, args.pipeline - 1) for i in range(cfg["n_layers"])]
    t_gen0 = time.perf_counter()
    model = lcu.Model.synthetic(seed=SEED, scale=SCALE, layer_gpus=layer_gpus, **cfg)
    gen_s = time.perf_counter() - t_gen0
    ctx = lcu.Context(model, context_len=ctx_len, temperature=TEMPERATURE)
    prompt = O.synth_tokens(PROMPT_LEN, SEED, lo=3, hi=min(32000, cfg["n_vocab"]))

    # ---- device-chained decode: `value`
    t_prefill0 = time.perf_counter()
    first = ctx.next_token(prompt)
    prefill_s = time.perf_counter() - t_prefill0
    warm_tokens, _ = ctx.decode_chained(first, W)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier_sync(dist, lcu)
    if args.profile == "decode":
        lcu.check(lcu.lib.lcu_profiler_start())
    tokens, ms = ctx.decode_chained(int(warm_tokens[-1]), K)
    if args.profile == "decode":
        lcu.check(lcu.lib.lcu_profiler_stop())
    barrier_sync(dist, lcu)
    ms_all = reduce_max_time(ms, dist)
    value = world * K / (ms_all / 1e3)

    # ---- end to end through the reference-facing call: host token in, host token out, every step
    ctx.clear_tokens()
    tok = ctx.next_token(prompt)
    for _ in range(W):
        tok = ctx.next_token([tok])
    barrier_sync(dist, lcu)
    t0 = time.perf_counter()
    e2e_tokens = []
    for _ in range(K):
        tok = ctx.next_token([tok])
        e2e_tokens.append(tok)
    lcu.check(lcu.lib.lcu_synchronize())
    e2e_ms = (time.perf_counter() - t0) * 1e3
    barrier_sync(dist, lcu)
    clocks = sampler.stop() if rank == 0 else None
    e2e_ms_all = reduce_max_time(e2e_ms, dist)
    e2e_value = world * K / (e2e_ms_all / 1e3)
    same_tokens = bool((np.array(e2e_tokens, np.int16) == tokens).all())

    # ---- roofline of the dominant kernel, timed alone with CUDA events on the launching stream
    peak, peak_src = measured_peak()
    reps = 10 * cfg["n_layers"]
    names = ["norm+wq|wk|wv+rope", "wo+residual", "norm+w1|w3+silu", "w2+residual", "norm+output"]
    kernels = {}
    for which, name in enumerate(names):
        kms, kbytes = ctx.bench_kernel(which, reps if which < 4 else 20)
        kernels[name] = {"us": round(kms * 1e3, 3), "bytes": kbytes, "gbs": round(kbytes / (kms * 1e-3) / 1e9, 1)}
    dom = kernels["norm+w1|w3+silu"]
    roofline = {"bound": "hbm", "kernel": "gemv1_kernel<WT, EPI_SILU> (fused RMSNorm + w1|w3 + SiLU gate)", "achieved": dom["gbs"], "peak": peak,
                "unit": "GB/s", "frac": round(dom["gbs"] / peak, 4), "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                "algorithmic_bytes_per_launch": dom["bytes"], "us_per_launch": dom["us"], "peak_source": peak_src,
                "frac_of_nominal_8tbs": round(dom["gbs"] / 8000.0, 4)}
    t_mid = PROMPT_LEN + W + K // 2
    step_bytes = decode_bytes_per_token(cfg, ffn, t_mid)
    whole_step = {"bytes_per_token": step_bytes, "achieved_gbs": round(step_bytes * (K / (ms_all / 1e3)) / 1e9, 1),
                  "frac_of_measured_peak": round(step_bytes * (K / (ms_all / 1e3)) / 1e9 / peak, 4),
                  "frac_of_nominal_8tbs": round(step_bytes * (K / (ms_all / 1e3)) / 1e9 / 8000.0, 4)}
    kps = ctx.kernels_per_step()
    prefill = prefill_sample(lcu, ctx, cfg, ffn, args.profile == "prefill", args.prefill_len) if world == 1 and ctx_len >= args.prefill_len + 2 else None
    ctx.close()
    model.close()

    line = {
        "metric": "7B batch-1 decode tok/s" if args.workload.startswith("7b") else f"{args.workload} batch-1 decode tok/s",
        "value": round(value, 2), "unit": "tok/s", "n_gpus": world if args.pipeline <= 1 else args.pipeline, "steps": K, "warmup": W,
        "ms_per_step": round(ms_all / K, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16" if cfg["block_size"] == 0 else "u8 weights x f16 activations, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"llama-{args.workload} greedy decode, batch 1, {PROMPT_LEN}-token seeded prompt, context {ctx_len}",
                   "parallelism": (f"layer pipeline over {args.pipeline} GPUs in one process (one stage active at a time at batch 1)" if args.pipeline > 1
                                   else "1 GPU" if world == 1 else f"{world} independent replicas (replicas only: batch-1 decode does not shard)"),
                   "weights_generated_s": round(gen_s, 1),
                   "l2": "inputs larger than L2: each step streams its weights once, far more than the 126 MB L2",
                   "weights": f"random-init ~N(0,{SCALE}) (Irwin-Hall, seed {SEED}), RMSNorm weights 1.0", "prefill_s": round(prefill_s, 4)},
        "e2e": {"value": round(e2e_value, 2), "unit": "tok/s", "h2d_bytes_per_step": 10, "d2h_bytes_per_step": 8,
                "ms_per_step": round(e2e_ms_all / K, 5), "tokens_equal_chained_run": same_tokens},
        "gpu_launches": K * kps, "kernels_per_step": kps,
        "roofline": roofline, "kernels": kernels, "whole_step": whole_step, "clocks": clocks,
    }
    if prefill is not None:
        line["prefill"] = prefill
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_sample(cfg, ffn)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    import numpy as np
    import oracle_lib as O
    import ref_lib as R

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    cfg = WORKLOADS[args.workload]
    K, W = args.steps, args.warmup
    base = {"impl": "reference", "metric": "7B batch-1 decode tok/s", "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
            "dtype": "f16" if cfg["block_size"] == 0 else "u8 weights x f16 activations, f32 accumulate"}
    lcu = load_package()
    if not R.available() or lcu.lib.lcu_device_count() < 1:
        # no reference build travelled to this machine: time the CPU restatement on a bounded sample
        ffn = O.lib().orc_ffn_dim(cfg["dim"], 256)
        cb = cpu_baseline_sample(cfg, ffn)
        base.update(value=round(cb["value"], 4), ms_per_step=round(1e3 / cb["value"], 3), cpu_baseline=cb,
                    config={"workload": f"llama-{args.workload} greedy decode, batch 1 (CPU restatement of the reference, bounded sample)"},
                    e2e={"value": round(cb["value"], 4), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
        print(json.dumps(base), flush=True)
        return
    ctx_len = max(CONTEXT_LEN, PROMPT_LEN + W + K + 2)
    R.lib().ref_initialize()
    model = lcu.Model.synthetic(seed=SEED, scale=SCALE, **cfg)  # same seeded weights, copied device to device
    ref = R.RefModel(lcu, model, cfg["dim"], 256, cfg["n_heads"], cfg["n_layers"], cfg["n_vocab"], 1e-6, cfg["block_size"], ctx_len,
                     TEMPERATURE, mtype=4)
    model.close()
    prompt = O.synth_tokens(PROMPT_LEN, SEED, lo=3, hi=min(32000, cfg["n_vocab"]))
    t0 = time.perf_counter()
    tok = ref.next_token(prompt)
    prefill_s = time.perf_counter() - t0
    warm, _ = ref.decode_timed(tok, W)
    lcu.check(lcu.lib.lcu_synchronize())
    tokens, secs = ref.decode_timed(int(warm[-1]), K)
    lcu.check(lcu.lib.lcu_synchronize())
    ref.close()
    value = K / secs
    base.update(value=round(value, 2), ms_per_step=round(secs / K * 1e3, 4),
                config={"workload": f"llama-{args.workload} greedy decode, batch 1, {PROMPT_LEN}-token seeded prompt, context {ctx_len}",
                        "reference": "unmodified eiz/llama.cu built for sm_100a (oracle/_ref), matmul_type 4, llama_context::next_token "
                                     "timed with steady_clock as main.cpp:80-100 does; the reference has no CPU path",
                        "prefill_s": round(prefill_s, 3)},
                cpu_baseline={"value": round(value, 2), "unit": "tok/s", "cores": 1, "kind": "reference",
                              "sample": f"all {K} decode steps; one host thread driving the reference's CUDA kernels on the same B200"},
                e2e={"value": round(value, 2), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                first_tokens=[int(t) for t in tokens[:8]])
    print(json.dumps(base), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="7b-fp16", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="seeded prompt length (128 for the headline configuration)")
    ap.add_argument("--prefill-len", type=int, default=PREFILL_LEN, help="prompt length of the prefill sample (512; from 768 rows the tcgen05 attention path runs)")
    ap.add_argument("--pipeline", type=int, default=1, help="single process: split the layers evenly over this many GPUs")
    ap.add_argument("--profile", nargs="?", const="decode", default=None, choices=["decode", "prefill"],
                    help="cudaProfilerStart/Stop around the device-chained timed region (decode) or around the prompt pass and GEMM (prefill)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
