#!/usr/bin/env python
"""Benchmark driver: GPT fp32 training throughput (fwd + bwd + AdamW), tokens/s.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload gpt180m|gpt90m|tiny|kernels]

Default workload "gpt180m": 12 layers, d_model 1024, 16 heads, d_ff 4096, seq 1024, vocab 32768, 32 sequences per GPU
(LayerNorm + GELU, learned positions, tied head), Zipf(1.1) synthetic tokens, seeded N(0, 0.02) weights.
One "step" = zero_grad + forward + Tensor::backward() + AdamW over one batch.  For N > 1 the script runs under
torch.distributed.run (one rank per GPU); gradients are averaged by bucketed NCCL all-reduce overlapped with backward.

Prints one JSON line (rank 0):
  value     whole-job tokens/s with the token batches already resident in HBM, CUDA-event timed on the compute stream;
  e2e       the same through the public trainer call with pinned HOST token buffers, the H2D copies and a D2H read of
            the loss inside the timed region;
  roofline  the GEMM engine (dominant kernel): algorithmic FLOP/s over the launches of the timed region vs the measured
            dense tensor peak;
  kernels   (1 GPU) every bandwidth-bound backward / optimizer kernel at the microbenchmark shapes: achieved HBM GB/s over the
            measured copy peak ("bwd kernel % HBM peak", the second half of the metric);
  reference_cuda / vs_reference_cuda  (1 GPU) the reference's own CUDA path built for sm_100a, same model and batch, and
            value over it;
  cpu_baseline  the reference's own CPU path (oracle/_ref) timed on the host cores on a bounded sample;
  dp        (N > 1) exposed communication time per step, GEMM time per step with NCCL in flight, and whether every rank
            ends with bit-identical weights.
`--impl reference` times the reference's CPU path alone on the same metric; `--impl reference-cuda` its CUDA path.
`--workload kernels` prints the kernel table alone, `--workload gemm` every GEMM shape of the step.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TRAFFIC_PROFILE = "gemm_tc_pair_kernel_linear_fwd_32768x1024x1024.md"
WORKLOADS = {
    # name: arch, V, T, C, H, L, F, B per GPU, micro-batches per step
    "gpt180m": ("lngelu", 32768, 1024, 1024, 16, 12, 4096, 32, 1),
    "gpt90m": ("lngelu", 16384, 512, 768, 12, 12, 3072, 32, 16),
    "tiny": ("lngelu", 512, 64, 128, 4, 2, 512, 4, 1),
}
HYPER = dict(lr=3e-4, beta1=0.9, beta2=0.95, wd=0.1, eps=1e-5, norm_eps=1e-5, ce_eps=1e-5)
CLIP = 1.0  # GlobalNormClipper threshold, as train.cpp:158 of the reference runs it: the clip is part of the timed step


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], tensor_tflops=d.get("bf16_tflops_sustained", d["bf16_tflops"]), tensor_tflops_burst=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, tensor_tflops=1400.0, tensor_tflops_burst=1590.0, source="fallback")


def profile_traffic(name):
    """DRAM read + write bytes of one captured launch, from the table row `dram__bytes_read.sum + dram__bytes_write.sum | a MB + b MB = c MB`
    of a committed ncu summary under profiles/ (None when the file or the row is missing)."""
    import re

    try:
        text = open(os.path.join(ROOT, "profiles", name)).read()
    except OSError:
        return None
    m = re.search(r"dram__bytes_read\.sum \+ dram__bytes_write\.sum\s*\|\s*[\d.]+ MB \+ [\d.]+ MB = ([\d.]+) MB", text)
    return float(m.group(1)) * 1e6 if m else None


def flops_per_token(V, T, C, L, F):
    """6 * (L * (4 C^2 + 2 C F) + C V) + 12 L T C: dense fwd + bwd contractions, non-causal attention as the reference computes it."""
    return 6 * (L * (4 * C * C + 2 * C * F) + C * V) + 12 * L * T * C


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        mhz, reasons, mx = [], set(), None
        for r in self.rows:
            try:
                mhz.append(float(r[0]))
                mx = float(r[1])
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "samples": len(mhz), "reasons": sorted(reasons)}


# ---- reference CPU arm -------------------------------------------------------------------------------------
CPU_SAMPLE_T = None  # tokens per CPU step: None = one full sequence (~16 s of host work per step for gpt180m on 16 cores; shorter samples would
                     # overweight the optimizer pass over all parameters, whose cost does not depend on the number of tokens)


def reference_cpu_run(workload, steps, warmup, sample_B=1, sample_T=None):
    """Times oracle/_ref/ref_harness (GradCraft's CPUBackend + OpenBLAS) on exactly `warmup` untimed + `steps` timed steps of a
    bounded sample: the workload's model with its seeded weights, sample_B sequences of sample_T tokens per step.
    Returns (tokens/s, cores, description, kind, ms per timed step)."""
    arch, V, T, C, H, L, F, B, accum = WORKLOADS[workload]
    sample_T = min(T, sample_T or CPU_SAMPLE_T or T)
    harness = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
    cores = os.cpu_count() or 1
    if not os.path.exists(harness):
        return None, cores, "oracle/_ref/ref_harness is not built", "reference", None
    import numpy as np

    from gradcraft_b200 import synth
    from oracle import ckpt

    n_steps = steps + warmup
    with tempfile.TemporaryDirectory() as tmp:
        # the harness reads T tokens per sequence from the file only when it runs full sequences; with a shorter sample it reads sample_T
        synth.token_batches(99, n_steps, sample_B, sample_T, V).tofile(os.path.join(tmp, "tok.i64"))
        ckpt.save(os.path.join(tmp, "w.ckpt"), synth.gpt_weights(arch, V, T, C, H, L, F, seed=0))  # the weights the GPU arm trains from
        h = HYPER
        cmd = [harness, "gpt", arch] + [str(v) for v in (V, T, C, H, L, F, sample_B, n_steps, 1, h["lr"], h["beta1"], h["beta2"], h["wd"], h["eps"], CLIP)]
        cmd += [os.path.join(tmp, "w.ckpt"), os.path.join(tmp, "tok.i64"), os.path.join(tmp, "out"), str(h["norm_eps"])]
        env = dict(os.environ, REF_BLAS_THREADS=str(cores), OPENBLAS_NUM_THREADS=str(cores), REF_HARNESS_NO_DUMP="1", REF_HARNESS_SAMPLE_T=str(sample_T))
        r = subprocess.run(cmd, env=env, capture_output=True, text=True)
        if r.returncode != 0:
            return None, cores, "ref_harness failed: " + (r.stderr.strip().splitlines() or ["?"])[-1], "reference", None
        ms = np.loadtxt(os.path.join(tmp, "out_time.txt"), ndmin=1)
    ms = ms[warmup:]
    ms_step = float(np.mean(ms))
    tok_s = sample_B * sample_T / (ms_step / 1e3)
    desc = "%s model with the GPU arm's seeded weights, %d sequence(s) of %d tokens per step (the model's sequence length is %d), %d warm-up + %d timed steps incl. clip and AdamW, OpenBLAS threads=%d, elementwise code single-threaded as the reference has it" % (
        workload, sample_B, sample_T, T, warmup, len(ms), cores)
    return tok_s, cores, desc, "reference", ms_step


def reference_cuda_run(workload, steps, warmup, batch=0):
    """The reference's own CUDA path (its two .cu files built for sm_100a by oracle/build_ref.sh; cuBLAS in TF32 tensor-op mode as
    the reference sets it) on the same model, batch size and token shapes, one GPU.  Returns a dict with `value` (tokens/s) or
    `unavailable`."""
    arch, V, T, C, H, L, F, B, accum = WORKLOADS[workload]
    harness = os.path.join(ROOT, "oracle", "_ref", "ref_harness_cuda")
    if not os.path.exists(harness):
        return {"unavailable": "oracle/_ref/ref_harness_cuda is not built"}
    from gradcraft_b200 import synth

    Bs = batch or B
    with tempfile.TemporaryDirectory() as tmp:
        synth.token_batches(99, 1, Bs, T, V).tofile(os.path.join(tmp, "tok.i64"))
        cmd = [harness, "gptcuda", arch] + [str(v) for v in (V, T, C, H, L, F, Bs, steps, warmup)] + [os.path.join(tmp, "tok.i64")]
        t0 = time.time()
        r = subprocess.run(cmd, capture_output=True, text=True)
    out = [l for l in r.stdout.splitlines() if l.startswith("tokens_per_s")]
    if r.returncode != 0 or not out:
        return {"unavailable": "ref_harness_cuda failed: " + ((r.stderr.strip().splitlines() or r.stdout.strip().splitlines() or ["?"])[-1])[:300]}
    f = out[-1].split()
    return {"value": float(f[1]), "unit": "tokens/s", "ms_per_step": float(f[3]), "steps": steps, "warmup": warmup, "batch": Bs, "pool_high_water_gb": float(f[5]), "last_loss": float(f[7]),
            "wall_s": time.time() - t0, "what": "the reference's CUDA path (kernels_math.cu / kernels_utils.cu built with -O3 -use_fast_math for sm_100a, cuBLAS TF32 tensor-op GEMMs), "
            "same model and batch, one fixed batch of synthetic tokens, wall clock around %d steps after %d warm-up" % (steps, warmup)}


def run_reference_cuda_arm(args, rank):
    if rank != 0:
        return
    arch, V, T, C, H, L, F, B, accum = WORKLOADS[args.workload]
    res = reference_cuda_run(args.workload, args.steps, args.warmup, args.ref_batch)
    if "unavailable" in res:
        print(json.dumps({"impl": "reference-cuda", "unavailable": res["unavailable"]}))
        return
    print(json.dumps({"impl": "reference-cuda", "metric": "GPT fp32 train tokens/s (fwd+bwd+AdamW)", "value": res["value"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                      "ms_per_step": res["ms_per_step"], "higher_is_better": True, "dtype": "f32 (cuBLAS TF32 tensor-op mode, as the reference sets it)", "data": "synthetic Zipf(1.1) tokens, one fixed batch",
                      "config": {"workload": args.workload, "arch": arch, "layers": L, "d_model": C, "heads": H, "d_ff": F, "seq_len": T, "vocab": V, "batch": res["batch"]},
                      "pool_high_water_gb": res["pool_high_water_gb"], "last_loss": res["last_loss"], "wall_s": res["wall_s"]}))


def run_reference_arm(args, rank):
    """The reference's CPU implementation on the host cores: --warmup untimed and --steps timed steps, each a bounded sample (one
    sequence instead of the GPU arm's 32); steps beyond what fits in about four minutes are cut, and the line reports the counts
    and the per-step time that were actually run (the requested ones go to steps_requested / warmup_requested)."""
    if rank != 0:
        return
    arch, V, T, C, H, L, F, B, accum = WORKLOADS[args.workload]
    t0 = time.time()
    Ts = min(T, CPU_SAMPLE_T or T)
    est_s = 18.7 * (flops_per_token(V, Ts, C, L, F) * Ts) / (flops_per_token(32768, 1024, 1024, 12, 4096) * 1024)  # ~18.7 s per full-sequence step (with clip) for gpt180m on 16 cores
    fit = max(2, int(190.0 / max(est_s, 1e-3)))
    warm = min(args.warmup, max(1, fit // 5))
    steps = max(1, min(args.steps, fit - warm))
    tok_s, cores, desc, kind, ms_step = reference_cpu_run(args.workload, steps, warm)
    if tok_s is None:
        print(json.dumps({"impl": "reference", "unavailable": desc}))
        return
    line = {
        "impl": "reference", "metric": "GPT fp32 train tokens/s (fwd+bwd+AdamW)", "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "steps_requested": args.steps, "warmup_requested": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic Zipf(1.1) tokens, N(0,0.02) weights (seed 0)",
        "config": {"workload": args.workload, "arch": arch, "layers": L, "d_model": C, "heads": H, "d_ff": F, "seq_len": T, "vocab": V, "clip": CLIP, "sample": desc},
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.time() - t0,
    }
    print(json.dumps(line))


# ---- our arm ----------------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import numpy as np
    import torch

    from gradcraft_b200 import capi, synth
    from gradcraft_b200.trainer import Trainer

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the training path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    arch, V, T, C, H, L, F, B, accum = WORKLOADS[args.workload]
    K, W = args.steps, args.warmup
    pk = peaks()

    tr = Trainer(arch, V, T, C, H, L, F, lr=HYPER["lr"], beta1=HYPER["beta1"], beta2=HYPER["beta2"], wd=HYPER["wd"], eps=HYPER["eps"], norm_eps=HYPER["norm_eps"], ce_eps=HYPER["ce_eps"],
                 clip=CLIP, device=local_rank)
    tr.load(synth.gpt_weights(arch, V, T, C, H, L, F, seed=0))  # identical on every rank
    lib = capi.lib()
    ctx = tr.context()
    if world > 1:
        uid = torch.zeros(capi.DP_ID_BYTES, dtype=torch.uint8)
        if rank == 0:
            buf = np.zeros(capi.DP_ID_BYTES, np.uint8)
            lib.dp_unique_id(buf)
            uid = torch.from_numpy(buf)
        uid = uid.cuda()
        dist.broadcast(uid, 0)
        tr.dp_init(uid.cpu().numpy(), rank, world, accum)

    # token streams: rank r draws from seed base + r; W + K steps of `accum` micro-batches, twice (device-resident pass, host pass)
    n_mb = (W + K) * accum
    host = torch.from_numpy(synth.token_batches(1000 + rank, n_mb, B, T, V)).pin_memory()
    resident = host.cuda()
    stream = torch.cuda.ExternalStream(tr.stream(), device=local_rank)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def one_step(i, src, on_device, want_loss):
        tr.zero_grad()
        loss = 0.0
        for mb in range(accum):
            x, y = src[i * accum + mb, 0], src[i * accum + mb, 1]
            l = tr.forward_backward(x, y, accum, want_loss, on_device)
            loss += l if want_loss else 0.0
        tr.optimizer_step()
        return loss

    def timed(src, on_device, want_loss, profile_gemm):
        for i in range(W):
            one_step(i, src, on_device, want_loss)
        barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        launches0 = tr.launch_count()
        if profile_gemm:
            lib.profile_gemm_begin(ctx)
            if world > 1:
                lib.dp_timing_begin(ctx)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        last = 0.0
        for i in range(W, W + K):
            last = one_step(i, src, on_device, want_loss)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop()
        prof = None
        if profile_gemm:
            import ctypes

            n, tms, fl = ctypes.c_int64(), ctypes.c_double(), ctypes.c_double()
            lib.profile_gemm_end(ctx, ctypes.byref(n), ctypes.byref(tms), ctypes.byref(fl))
            waits, exposed = ctypes.c_int64(), ctypes.c_double()
            if world > 1:
                lib.dp_timing_end(ctx, ctypes.byref(waits), ctypes.byref(exposed))
            prof = (n.value, tms.value, fl.value, waits.value, exposed.value)
        if dist is not None:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, clocks, tr.launch_count() - launches0, prof, last

    ms_dev, clocks, launches, prof, _ = timed(resident, True, False, True)
    if args.no_e2e:
        ms_e2e, last_loss = float("nan"), float("nan")
    else:
        ms_e2e, _, _, _, last_loss = timed(host, False, True, False)
    engine = lib.ctx_last_gemm_engine(ctx)
    split_mode = lib.ctx_gemm_split_mode(ctx)
    units = 4 if split_mode == 2 else 6  # tensor time per product in bf16-MMA units
    tokens_per_step = B * T * accum * world
    value = tokens_per_step * K / (ms_dev / 1e3)
    e2e = tokens_per_step * K / (ms_e2e / 1e3)
    n_gemm, gemm_ms, gemm_flops, dp_waits, dp_exposed_ms = prof
    achieved = gemm_flops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else 0.0
    fpt = flops_per_token(V, T, C, L, F)
    hwm = tr.high_water_bytes()
    nparams = tr.num_params()
    nbuckets = tr.num_buckets()
    dp = None
    if world > 1:
        # every rank must hold the same weights after the same reduced gradients: a digest of all parameters, gathered from every rank
        import hashlib

        hsh = hashlib.blake2b(digest_size=16)
        params = tr.get("param")
        for name in sorted(params):
            hsh.update(params[name].tobytes())
        mine = torch.frombuffer(bytearray(hsh.digest()), dtype=torch.uint8).cuda()
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        t = torch.tensor([dp_exposed_ms, gemm_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dp = {"dp_weights_identical": bool(all(torch.equal(e, every[0]) for e in every)), "weights_digest_rank0": bytes(every[0].cpu().numpy()).hex(),
              "exposed_comm_ms_per_step": float(t[0]) / K, "gemm_ms_per_step_with_comm_in_flight": float(t[1]) / K,
              "note": "exposed = time the compute stream waits for the last reduced bucket after backward has been queued (events on both streams, max over ranks); "
                      "compare gemm_ms_per_step with the 1-GPU line's roofline.kernel figure for the slowdown of the GEMMs while NCCL runs beside them",
              "nccl_max_ctas": os.environ.get("NCCL_MAX_CTAS")}
    tr.close()

    cpu = kernels = ref_cuda = None
    if rank == 0 and world == 1 and not args.no_kernels:
        torch.cuda.synchronize()
        lib.arena_release_cached(ctx)  # the trainer's arena (tens of GB) goes back to the driver before the microbenchmarks allocate
        kernels = kernel_suite(5, 3, local_rank)
    if rank == 0 and world == 1 and not args.no_reference_cuda:
        torch.cuda.synchronize()
        lib.arena_release_cached(ctx)
        torch.cuda.empty_cache()
        ref_cuda = reference_cuda_run(args.workload, 3, 1)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tok_s, cores, desc, kind, _ = reference_cpu_run(args.workload, 1, 1)
        cpu = {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": desc}
    if rank == 0:
        line = {
            "metric": "GPT fp32 train tokens/s (fwd+bwd+AdamW)", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_dev / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic: Zipf(1.1) tokens (seed 1000+rank), N(0,0.02) weights (seed 0)",
            "config": {"workload": args.workload, "arch": arch, "layers": L, "d_model": C, "heads": H, "d_ff": F, "seq_len": T, "vocab": V, "batch_per_gpu": B, "micro_batches_per_step": accum,
                       "global_batch": B * accum * world, "params": nparams, "clip": CLIP, "parallelism": "dp%d" % world, "gradient_buckets": nbuckets,
                       "l2": "working set per step (%.1f GB arena high-water) far exceeds the 126 MB L2" % (hwm / 1e9), "gemm_engine": {1: "simt_fp32", 2: "tcgen05_split_fp32(mode %d)" % split_mode}.get(engine, "none"),
                       "algorithmic_gflop_per_token": fpt / 1e9, "step_tflops": fpt * tokens_per_step / world / (ms_dev / K / 1e3) / 1e12},
            "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * T * 8 * accum, "d2h_bytes_per_step": 4 * accum, "ms_per_step": ms_e2e / K, "last_loss": last_loss},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["tensor_tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tensor_tflops"],
                         "traffic": profile_traffic(TRAFFIC_PROFILE), "traffic_note": "dram read+write of one captured launch of the most frequent shape (M=32768, N=K=1024; algorithmic 272.6 MB), read from profiles/" + TRAFFIC_PROFILE,
                         "frac_of_split_ceiling": achieved / (pk["tensor_tflops"] / units),
                         "kernel": "gemm (%d launches, %.1f ms of the timed region)" % (n_gemm, gemm_ms),
                         "peak_source": "%s dense bf16, sustained; split mode %d spends the tensor time of %d bf16 MMAs per product (a tf32 MMA counts 2), so its ceiling is 1/%d of this" % (pk["source"], split_mode, units, units),
                         "gemm_share_of_step": gemm_ms / ms_dev},
            "cpu_baseline": cpu,
        }
        if kernels is not None:
            # the second half of the metric: every bandwidth-bound backward / optimizer kernel against the measured HBM peak
            line["kernels"] = kernels
            line["bwd_kernel_frac_of_hbm_peak"] = {k: round(v["frac_of_hbm_peak"], 4) for k, v in kernels.items()}
            line["peak_hbm_gbs"] = pk["hbm_gbs"]
        if ref_cuda is not None:
            line["reference_cuda"] = ref_cuda
            line["vs_reference_cuda"] = (value / ref_cuda["value"]) if "value" in ref_cuda else None
        if dp is not None:
            line["dp"] = dp
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


# ---- fused backward kernels vs the HBM roofline -----------------------------------------------------------------------
def kernel_suite(steps, warmup, device=0, only="", small=False):
    """The bandwidth-bound kernels of the backward pass and the optimizer at the microbenchmark shapes, each timed alone with
    CUDA events (L2 flushed by a 256 MB write before every sample): {name: {ms, algorithmic_bytes, achieved_gbs,
    frac_of_hbm_peak}}.  Algorithmic bytes count every operand once."""
    import numpy as np
    import torch

    from gradcraft_b200 import capi, synth

    ctx = capi.Context(device)
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timeit(fn, calls=1):
        """Median ms per call.  calls > 1: that many back-to-back launches per sample, fn(i) working on the i-th of `calls`
        disjoint buffer sets (so no launch finds its data in L2)."""
        for _ in range(max(3, warmup)):
            for i in range(calls):
                fn(i)
        ts = []
        for _ in range(max(5, steps)):
            flush.zero_()  # evict L2 between timed samples
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for i in range(calls):
                fn(i)
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) / calls)
        return float(np.median(ts))

    out, notes = {}, {}
    want = lambda name: (not only) or only in name  # --only: run the kernels whose name contains the text (profiling runs)
    M, V = (2048 if small else 16384), 32768  # --small: an eighth of the rows, for captures that must stay within a few GB
    if want("softmax_ce"):
        P = torch.rand(M, V, device="cuda")
        P /= P.sum(-1, keepdim=True)
        Tg = torch.randint(0, V, (M,), dtype=torch.int32, device="cuda")
        out["softmax_ce_bwd [%d,32768]" % M] = (timeit(lambda i: ctx.softmax_ce_bwd_f32(P, P, Tg, capi.IDX_I32, 1.0, M, V, 0)), 2 * M * V * 4 + M * 4)
        lossbuf = torch.empty(1, device="cuda")
        out["softmax_ce_fwd [%d,32768]" % M] = (timeit(lambda i: ctx.softmax_ce_fwd_f32(lossbuf, P, P, Tg, capi.IDX_I32, M, V, 1e-5)), 2 * M * V * 4 + M * 4)
        del P
    M, C = 16384, 1024
    if want("layernorm rmsnorm"):
        g, b, dg, db = torch.ones(C, device="cuda"), torch.zeros(C, device="cuda"), torch.empty(C, device="cuda"), torch.empty(C, device="cuda")
        sets = []
        for _ in range(4):  # four disjoint (x, dy, dx, mean, rstd) sets, 201 MB each
            x, dy = torch.randn(M, C, device="cuda"), torch.randn(M, C, device="cuda") * 1e-2
            y, mu, rs, dx = torch.empty_like(x), torch.empty(M, device="cuda"), torch.empty(M, device="cuda"), torch.empty_like(x)
            ctx.layernorm_fwd_f32(y, mu, rs, x, g, b, M, C, 1e-5)
            sets.append((x, dy, dx, mu, rs))
            del y
        ln = lambda i: ctx.layernorm_bwd_f32(sets[i][2], dg, db, sets[i][1], sets[i][0], g, sets[i][3], sets[i][4], M, C, 0, 0)
        ln_bytes = 3 * M * C * 4 + 2 * M * 4 + 3 * C * 4
        if want("layernorm"):
            out["layernorm_bwd [16384,1024]"] = (timeit(ln), ln_bytes)  # one isolated call per sample: the headline
            out["layernorm_bwd [16384,1024] pipelined x4"] = (timeit(ln, calls=4), ln_bytes)
            notes["layernorm_bwd [16384,1024] pipelined x4"] = "four back-to-back calls on four disjoint buffer sets per sample: launch latency hidden, as inside a training step"
            lna = lambda i: ctx.layernorm_bwd_f32(sets[i][2], dg, db, sets[i][1], sets[i][0], g, sets[i][3], sets[i][4], M, C, 1, 1)
            out["layernorm_bwd accumulating into dx [16384,1024] pipelined x4"] = (timeit(lna, calls=4), ln_bytes + M * C * 4)
            notes["layernorm_bwd accumulating into dx [16384,1024] pipelined x4"] = "the form the residual stream's gradient takes in the step: dx is read, added to and written back (four arrays of traffic)"
        if want("rmsnorm"):
            rms = lambda i: ctx.rmsnorm_bwd_f32(sets[i][2], dg, sets[i][1], sets[i][0], g, sets[i][4], M, C, 0, 0)
            out["rmsnorm_bwd [16384,1024]"] = (timeit(rms), 3 * M * C * 4 + M * 4 + 2 * C * 4)
        del sets
    M, F = 16384, 4096
    if want("gelu") or want("reduce_rows"):
        x, dy = torch.randn(M, F, device="cuda"), torch.randn(M, F, device="cuda") * 1e-2
        dx = torch.empty_like(x)
        if want("gelu"):
            out["gelu_bwd [16384,4096]"] = (timeit(lambda i: ctx.gelu_bwd_f32(dx, dy, x, M * F, 0)), 3 * M * F * 4)
        if want("reduce_rows"):
            red = torch.empty(F, device="cuda")
            out["reduce_rows (bias gradient) [16384,4096]"] = (timeit(lambda i: ctx.reduce_rows_f32(red, dy, M, F, 0)), M * F * 4 + F * 4)
        del x, dy, dx
    if want("causal_softmax"):
        Bn, H, T = 16, 16, 1024
        rows = Bn * H * T
        S = torch.randn(rows, T, device="cuda")
        tri = 4 * Bn * H * T * ((T + 1) // 2)  # bytes of one pass over the entries at or below the diagonal
        out["causal_softmax_fwd [16,16,1024,1024]"] = (timeit(lambda i: ctx.causal_softmax_fwd_f32(S, S, 0.125, rows, T)), tri + 4 * rows * T)
        dP = torch.randn(rows, T, device="cuda") * 1e-2
        out["causal_softmax_bwd [16,16,1024,1024]"] = (timeit(lambda i: ctx.causal_softmax_bwd_f32(dP, dP, S, 0.125, rows, T, 0)), 2 * tri + 4 * rows * T)
        del S, dP
    if want("scatter_add"):
        n, Vv, Wd = 32768, 32768, 1024
        idx_h = synth.zipf_tokens(4321, n, Vv).astype(np.int64)
        idx = torch.from_numpy(idx_h).cuda()
        dyv, table = torch.randn(n, Wd, device="cuda") * 1e-2, torch.zeros(Vv, Wd, device="cuda")
        hit = int(np.unique(idx_h).size)
        out["scatter_add [32768 Zipf(1.1) tokens, 32768 x 1024 table]"] = (timeit(lambda i: ctx.scatter_add_f32(table, idx, capi.IDX_I64, dyv, n, Wd, Vv)), n * Wd * 4 + 2 * hit * Wd * 4)
        notes["scatter_add [32768 Zipf(1.1) tokens, 32768 x 1024 table]"] = "%d distinct rows hit; bytes = dy once + read-modify-write of the rows hit" % hit
        del dyv, table
    if want("adamw"):
        npar = 185759744 // (8 if small else 1)
        npar_pad = (npar + capi.ADAMW_CHUNK - 1) // capi.ADAMW_CHUNK * capi.ADAMW_CHUNK
        w, m, v, gr = (torch.randn(npar_pad, device="cuda") * 0.02 for _ in range(4))
        v.abs_()
        mask = torch.ones(npar_pad // capi.ADAMW_CHUNK, dtype=torch.uint8, device="cuda")
        out["adamw_arena [%.1f M parameters]" % (npar / 1e6)] = (timeit(lambda i: ctx.adamw_arena_f32(w, m, v, gr, mask, npar_pad, 3e-4, 0.9, 0.95, 0.9, 0.95, 0.1, 1e-5, 1.0)), 28 * npar_pad)
        del w, m, v, gr
    ctx.sync()
    kernels = {k: {"ms": ms, "algorithmic_bytes": by, "achieved_gbs": by / ms / 1e6, "frac_of_hbm_peak": by / ms / 1e6 / pk["hbm_gbs"]} for k, (ms, by) in out.items()}
    for k, t in notes.items():
        kernels[k]["note"] = t
    ctx.close()
    del flush
    torch.cuda.empty_cache()
    return kernels


def run_kernels(args):
    pk = peaks()
    kernels = kernel_suite(args.steps, args.warmup, only=args.only, small=args.small)
    if not kernels:
        raise SystemExit("bench.py: --only %r matches no kernel of the kernels workload" % args.only)
    worst = min(kernels.values(), key=lambda d: d["frac_of_hbm_peak"])
    print(json.dumps({"metric": "fused backward kernels, achieved HBM GB/s vs measured peak", "value": worst["frac_of_hbm_peak"], "unit": "fraction of HBM peak (worst kernel)", "n_gpus": 1,
                      "steps": max(5, args.steps), "warmup": max(3, args.warmup), "higher_is_better": True, "dtype": "f32", "data": "synthetic N(0,1) activations, N(0,1e-2) upstream gradients",
                      "config": {"workload": "kernels", "l2": "flushed between timed launches (256 MB write)"}, "peak_hbm_gbs": pk["hbm_gbs"], "peak_source": pk["source"], "kernels": kernels}))


# ---- the GEMM shapes of one gpt180m step vs the tensor roofline -------------------------------------------------------------
def run_gemm(args):
    import numpy as np
    import torch

    from gradcraft_b200 import capi

    ctx = capi.Context(0)
    pk = peaks()
    units = 4 if ctx.ctx_gemm_split_mode() == 2 else 6  # tensor time per product in bf16-MMA units
    M, C, F, V, T, D, BH = 32768, 1024, 4096, 32768, 1024, 64, 512
    # name, opa, opb, M, N, K, batches (attention shapes are strided over (B, T, H*D) buffers exactly as the step runs them: causal
    # variants that skip known zeros; their TFLOP/s are quoted on the dense 2*M*N*K count, as the reference computes them)
    shapes = [
        ("linear_fwd_NN_CxC", 0, 0, M, C, C, 1), ("linear_dX_NT_CxC", 0, 1, M, C, C, 1), ("linear_dW_TN_CxC_splitk", 1, 0, C, C, M, 1),
        ("fc1_fwd_NN_CxF", 0, 0, M, F, C, 1), ("fc2_dW_TN_FxC", 1, 0, F, C, M, 1), ("head_fwd_NT_CxV", 0, 1, M, V, C, 1), ("head_dE_TN_VxC", 1, 0, V, C, M, 1),
        ("attn_scores_NT_batched", 0, 1, T, T, D, BH), ("attn_dS_NT_batched_softmax_bwd", 0, 1, T, T, D, BH), ("attn_pv_NN_batched", 0, 0, T, D, T, BH), ("attn_dV_TN_batched", 1, 0, T, D, T, BH),
    ]
    out = {}
    for name, opa, opb, m, n, k, nb in shapes:
        if args.only and args.only not in name:
            continue
        if nb == 1:
            A = torch.randn((k, m) if opa else (m, k), device="cuda")
            B = torch.randn((n, k) if opb else (k, n), device="cuda")
            Cm = torch.empty(m, n, device="cuda")
            fn = lambda: ctx.gemm_f32(opa, opb, m, n, k, 1.0, A, A.shape[1], B, B.shape[1], 0.0, Cm, n, None)
            is_weight = "_fwd_" in name or "_dX_" in name  # B is a weight matrix there: registered for pre-split companions, as Module::to does
            if is_weight:
                ctx.weight_twins_register(B, B.shape[0], B.shape[1])
        else:
            Bn, H = 32, 16
            Cw = H * D
            q = torch.randn(Bn, T, Cw, device="cuda")
            kk = torch.randn(Bn, T, Cw, device="cuda")
            S = torch.randn(Bn * H, T, T, device="cuda")
            O = torch.empty(Bn, T, Cw, device="cuda")
            if name.startswith("attn_scores"):
                fn = lambda: ctx.gemm_batched_causal_f32(0, 1, T, T, D, 1.0, q, Cw, T * Cw, D, kk, Cw, T * Cw, D, 0.0, S, T, H * T * T, T * T, Bn, H, 1)
            elif name.startswith("attn_dS"):
                Pm = torch.rand(Bn * H, T, T, device="cuda").tril_()
                rdot = torch.randn(Bn * H * T, device="cuda")
                fn = lambda: ctx.gemm_batched_softmax_bwd_f32(0, 1, T, D, 1.0, q, Cw, T * Cw, D, kk, Cw, T * Cw, D, S, T, H * T * T, T * T, Bn, H, Pm, rdot, 0.125)
            elif name.startswith("attn_pv"):
                fn = lambda: ctx.gemm_batched_causal_f32(0, 0, T, D, T, 1.0, S, T, H * T * T, T * T, kk, Cw, T * Cw, D, 0.0, O, Cw, T * Cw, D, Bn, H, 2)
            else:
                fn = lambda: ctx.gemm_batched_causal_f32(1, 0, T, D, T, 1.0, S, T, H * T * T, T * T, q, Cw, T * Cw, D, 0.0, O, Cw, T * Cw, D, Bn, H, 3)
        for _ in range(max(3, args.warmup)):
            fn()
        ts = []
        for _ in range(max(3, args.steps)):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ms = float(np.median(ts))
        fl = 2.0 * m * n * k * nb
        if nb == 1 and is_weight:
            ctx.weight_twins_drop(B, B.numel() * 4)
        out[name] = {"ms": ms, "tflops": fl / ms / 1e9, "frac_of_bf16_peak": fl / ms / 1e9 / pk["tensor_tflops_burst"], "frac_of_split_ceiling": fl / ms / 1e9 / (pk["tensor_tflops_burst"] / units), "engine": ctx.ctx_last_gemm_engine()}
        del fn
    ctx.sync()
    worst = min(out.values(), key=lambda d: d["tflops"])
    print(json.dumps({"metric": "GEMM engine, algorithmic TFLOP/s on the shapes of one gpt180m step", "value": worst["tflops"], "unit": "TFLOP/s (slowest shape)", "n_gpus": 1, "steps": max(3, args.steps),
                      "warmup": max(3, args.warmup), "higher_is_better": True, "dtype": "f32 (split mode %d)" % ctx.ctx_gemm_split_mode(), "data": "synthetic N(0,1)", "config": {"workload": "gemm", "l2": "operands of the large shapes exceed the 126 MB L2"},
                      "peak_tflops": pk["tensor_tflops_burst"], "peak_source": pk["source"] + " dense bf16 burst", "shapes": out}))
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda"])
    ap.add_argument("--ref-batch", type=int, default=0, help="sequences per step for --impl reference-cuda (default: the workload's)")
    ap.add_argument("--workload", default="gpt180m", choices=list(WORKLOADS) + ["kernels", "gemm"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernels", action="store_true", help="skip the fused-kernel microbenchmarks of the default line")
    ap.add_argument("--no-reference-cuda", action="store_true", help="skip the reference-CUDA leg of the default line")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass (profiling runs)")
    ap.add_argument("--only", default="", help="gemm / kernels workloads: run only the entries whose name contains this text")
    ap.add_argument("--small", action="store_true", help="kernels workload: an eighth of the loss rows / optimizer parameters (profiler captures)")
    args = ap.parse_args()
    rank, world, local_rank = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference-cuda":
        run_reference_cuda_arm(args, int(os.environ.get("RANK", "0")))
        return
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.workload == "kernels":
        run_kernels(args)
        return
    if args.workload == "gemm":
        run_gemm(args)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
