#!/usr/bin/env python
"""Decode throughput of the B200 engine on the Qwen2.5-0.5B-architecture workload
(--workload selects the other measured configurations; the default is the headline).

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference --gpus N --steps K ...   # the reference's algorithm on host cores

A step is one greedy decode step (one new token per sequence, batch 1 per GPU) after a
128-token prompt, on seeded random-init bf16 weights written as config.json + safetensors
(no checkpoints or datasets exist where this runs).  With N > 1 every rank holds a replica on
its own GPU and decodes its own sequence; there is no collective on the token path, the ranks
only meet at the barriers around the timed region (weak scaling).

Prints ONE JSON line (rank 0):
  value      whole-job tokens/s with everything resident in HBM, device-timed (CUDA events on the
             engine's stream, max over ranks);
  e2e        the same metric through the per-token C-ABI call with host buffers: token id in,
             next token id out, one synchronisation per token;
  roofline   the projection kernel (all weight streaming of a step): algorithmic bytes / device
             time of its launches (CUDA events around graph replays of each kernel class, taken
             live after the timed region), against the measured HBM copy bandwidth;
  e2e_logits the same per-token call with the [vocab] f32 logits copied back every step, which is what
             the reference's trait returns (decode_step -> Vec<f32>, src/hf/model.rs:359-371);
  e2e_sampled  hm_generate at the reference's default sampling settings (batch-1 workloads), prefill excluded;
  c5         the batched configuration (Qwen2.5-1.5B architecture, 64 sequences per GPU, 512-token
             prompts) timed the same way on bf16 and on f32 KV pages, with its prefill rate;
  cpu_baseline  the CPU oracle (a restatement of Homura's CPU path) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np  # noqa: E402

PROMPT_LEN = 128
SEED = 20251
FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0
# DRAM bytes of the 97 projection launches of one headline decode step, summed from the ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum per launch) summarised in the file below; the algorithmic
# figure is 987.9 MB, so every weight byte is read once.
HEADLINE_PROJECTION_DRAM_BYTES_PER_STEP = 997.0e6
HEADLINE_PROJECTION_LAUNCHES = 97
TRAFFIC_SOURCE = "profiles/ncu_full_gemv_lmhead_and_small_kernels.md"


def log(*a):
    print(*a, file=sys.stderr, flush=True)


# The contract is ONE JSON line on stdout.  Libraries (NCCL prints its version there) must not add
# to it, so file descriptor 1 is pointed at stderr for the whole run and the line goes to the saved one.
_OUT_FD = None


def claim_stdout():
    global _OUT_FD
    if _OUT_FD is None:
        sys.stdout.flush()
        _OUT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(obj):
    data = (json.dumps(obj) + "\n").encode()
    if _OUT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_OUT_FD, data)


# name -> (config attribute in homura_b200.synth, checkpoint format, sequences per GPU, description);
# prompt lengths of the workloads: PROMPTS below
WORKLOADS = {
    "qwen25-05b": ("QWEN25_05B", "bf16", 1, "Qwen2.5-0.5B-architecture decoder (24 layers, hidden 896, 14/2 heads, hd 64, SwiGLU 4864, vocab 151936, tied, QKV bias), batch 1 per GPU"),
    "tinyllama-q8_0": ("TINYLLAMA_11B", "q8_0", 1, "TinyLlama-1.1B-architecture decoder (22 layers, hidden 2048, 32/4 heads, hd 64, SwiGLU 5632, vocab 32000), GGUF Q8_0, batch 1 per GPU"),
    "tinyllama-q4_0": ("TINYLLAMA_11B", "q4_0", 1, "TinyLlama-1.1B-architecture decoder (22 layers, hidden 2048, 32/4 heads, hd 64, SwiGLU 5632, vocab 32000), GGUF Q4_0, batch 1 per GPU"),
    "tinyllama-q4_k_m": ("TINYLLAMA_11B", "q4_k_m", 1, "TinyLlama-1.1B-architecture decoder (22 layers, hidden 2048, 32/4 heads, hd 64, SwiGLU 5632, vocab 32000), GGUF Q4_K with attn_v / ffn_down / output in Q6_K (the Q4_K_M mix), batch 1 per GPU"),
    "qwen25-15b-x64": ("QWEN25_15B", "bf16", 64, "Qwen2.5-1.5B-architecture decoder (28 layers, hidden 1536, 12/2 heads, hd 128, SwiGLU 8960, vocab 151936, tied, QKV bias), 64 sequences per GPU"),
}
HEADLINE = "qwen25-05b"
PROMPTS = {"qwen25-05b": 128, "tinyllama-q8_0": 256, "tinyllama-q4_0": 256, "tinyllama-q4_k_m": 256, "qwen25-15b-x64": 512}


def model_dir(cfg, seed, rank, world, name=HEADLINE, fmt="bf16"):
    """Rank 0 writes the seeded checkpoint once; the other ranks wait for the marker file.
    Returns a directory (config.json + safetensors) or, for the GGUF formats, the file's path."""
    from homura_b200 import synth

    tag = "qwen25_05b" if name == HEADLINE else name.replace("-", "_")
    d = os.path.join(tempfile.gettempdir(), f"homura_b200_bench_{tag}_seed{seed}")
    marker = os.path.join(d, ".complete")
    gguf = os.path.join(d, "model.gguf")
    if rank == 0 and not os.path.exists(marker):
        t = time.time()
        if fmt == "bf16":
            synth.write_hf_model(d, cfg, seed)
        else:
            os.makedirs(d, exist_ok=True)
            if fmt == "q4_k_m":
                synth.write_gguf_model(gguf, cfg, seed, synth.GGML_Q4_K, k_mix=True, quant_embed=True)
            else:
                synth.write_gguf_model(gguf, cfg, seed, synth.GGML_Q8_0 if fmt == "q8_0" else synth.GGML_Q4_0)
        open(marker, "w").write("ok")
        log(f"[bench] wrote synthetic checkpoint to {d} in {time.time() - t:.1f}s")
    while not os.path.exists(marker):
        time.sleep(0.5)
    return d if fmt == "bf16" else gguf


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU during the timed region."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except Exception:
                continue
            for nm, v in zip(names, r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


def dist_setup(n_gpus):
    """(rank, world, local_rank, barrier, max_over_ranks, close).  torch.distributed only as plumbing."""
    from homura_b200.replicas import Rendezvous

    rv = Rendezvous()
    return rv.rank, rv.world, rv.local, rv.barrier, rv.max, rv.close


def cpu_sample(d, cfg, steps, warmup, prompt_len):
    """Decode tokens/s of the CPU oracle on the same checkpoint (all host threads, one sequence)."""
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use every host core this
    # process may run on, so the variable is reset before the OpenMP runtime of the oracle library loads
    try:
        ncores = len(os.sched_getaffinity(0))
    except Exception:
        ncores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(ncores)
    os.environ.setdefault("OMP_PROC_BIND", "close")
    os.environ.setdefault("OMP_PLACES", "cores")
    import oracle as orc
    from homura_b200 import synth

    try:
        orc.use_native_build()  # -march=native on the machine that runs the baseline
    except RuntimeError:
        pass  # already loaded in this process

    n = prompt_len + warmup + steps + 1
    om = orc.OracleModel.from_hf_dir(d, max_seq_len=n) if os.path.isdir(d) else orc.OracleModel.from_gguf(d, max_seq_len=n)
    ids = synth.prompt_ids(SEED, prompt_len, cfg.vocab_size)
    tok, _ = om.prefill(ids)
    for _ in range(warmup):
        tok = orc.argmax(om.decode_step(tok))
    t = time.perf_counter()
    for _ in range(steps):
        tok = orc.argmax(om.decode_step(tok))
    dt = time.perf_counter() - t
    return steps / dt, dt, orc.num_threads()


def headline_config(world, kv_dtype, weight_mb):
    """The `config` object of the headline workload: identical for this engine and for the reference arm."""
    _, _, _, wl_desc = WORKLOADS[HEADLINE]
    return {
        "workload": wl_desc + f", {PROMPTS[HEADLINE]}-token prompt, greedy decode",
        "kv_cache": f"paged, 16 tokens/page, {kv_dtype}", "l2": f"inputs larger than L2: {weight_mb:.0f} MB of weights are streamed once per step (L2 is 126 MB)",
        "parallelism": f"replicas x{world}, independent sequences, no collective on the token path", "seed": SEED,
    }


def run_reference(args):
    """The reference's CPU implementation of the path = the oracle port, timed on host cores: same checkpoint,
    same 128-token prompt, same warm-up and step counts as this engine's arm."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from homura_b200 import synth

    cfg = synth.QWEN25_05B
    d = model_dir(cfg, SEED, 0, 1)
    steps, warmup = args.steps, max(args.warmup, 3)
    prompt = PROMPTS[HEADLINE]
    tps, dt, threads = cpu_sample(d, cfg, steps, warmup, prompt)
    sample = f"{steps} greedy decode steps after a {prompt}-token prompt and {warmup} warm-up steps, same seeded weights (bf16), {threads} OpenMP threads (OMP_PROC_BIND=close), oracle built -march=native"
    out = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": tps, "unit": "tok/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": 1000.0 * dt / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over bf16 weights",
        "data": "synthetic", "config": headline_config(args.gpus, "f32", 987_922_432 / 1e6),
        "reference_kind": "CPU oracle = restated Homura CPU path (the reference itself needs Rust + LLVM 21, absent here)",
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(out)


def run_c5(hm, synth, rank, world, local, barrier, vmax, K, W, peak):
    """The batched configuration: Qwen2.5-1.5B architecture, 64 sequences per GPU, 512-token prompts, greedy
    decode, on bf16 and on f32 KV pages.  Every rank runs its own 64 sequences on its replica."""
    name = "qwen25-15b-x64"
    cfg_name, fmt, B, wl_desc = WORKLOADS[name]
    cfg = getattr(synth, cfg_name)
    PL = PROMPTS[name]
    d = model_dir(cfg, SEED, rank, world, name, fmt)
    barrier()
    m = hm.HfModel.load_with_dtype(d, hm.DType.BF16, device=local)
    prompts = [synth.prompt_ids(SEED + 1000 + rank * B + b, PL, cfg.vocab_size) for b in range(B)]
    max_seq = PL + W + K + 8 + 24
    out = {"workload": wl_desc + f", {PL}-token prompts, greedy decode", "sequences_per_gpu": B, "steps": K, "warmup": W, "weight_bytes_per_step": m.weight_bytes(), "pages": {}}
    for kv in ("bf16", "f32"):
        m.init_kv_cache(max_seq, batch=B, kv_dtype=hm.DType.BF16 if kv == "bf16" else hm.DType.F32)
        barrier()
        t = time.perf_counter()
        first = [m.prefill(prompts[b], seq=b) for b in range(B)]
        pf_s = vmax(time.perf_counter() - t)
        m.decode_greedy_n(first, 0)
        barrier()
        ms = vmax(m.time_decode(W, K))
        barrier()
        prof = m.profile_decode(4)
        T_avg = PL + W + (K + 1) / 2.0
        kv_tok = cfg.num_hidden_layers * 2 * cfg.kv_dim * (2 if kv == "bf16" else 4)
        step_bytes = m.weight_bytes() + B * (kv_tok * T_avg + kv_tok)
        gbs = step_bytes / (ms / K * 1e-3) / 1e9
        out["pages"][kv] = {
            "tok_per_s": world * B * K / (ms / 1e3), "ms_per_step": ms / K, "bytes_per_step": step_bytes, "achieved_gbs": gbs, "frac_of_measured": gbs / peak,
            "frac_of_nominal_8TBs": gbs / NOMINAL_HBM_GBS, "prefill_tok_per_s": world * B * PL / pf_s,
            "kernels": [{"name": p["name"], "launches": p["launches_per_step"], "us": round(1e3 * p["ms_per_step"], 2), "MB": round(p["bytes_per_step"] / 1e6, 3)} for p in prof],
        }
    out["launches_per_step"] = m.launches_per_step()
    m.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kv-dtype", default="f32", choices=["f32", "bf16"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-c5", action="store_true", help="skip the batched Qwen2.5-1.5B x 64 block of the headline line")
    ap.add_argument("--prompt-len", type=int, default=None, help="prompt tokens before the timed decode steps (default: the workload's own, 128 for the headline)")
    ap.add_argument("--workload", default=HEADLINE, choices=sorted(WORKLOADS), help="default: the headline workload; the others are the remaining measured configurations")
    ap.add_argument("--device-only", action="store_true", help="only the device-timed region: skips the end-to-end loop, the per-kernel pass and the CPU baseline (for profiler runs)")
    args = ap.parse_args()
    claim_stdout()
    if args.impl == "reference":
        return run_reference(args)

    import homura_b200 as hm
    from homura_b200 import synth

    rank, world, local, barrier, vmax, close = dist_setup(args.gpus)
    K, W = args.steps, max(args.warmup, 3)
    cfg_name, fmt, B, wl_desc = WORKLOADS[args.workload]
    cfg = getattr(synth, cfg_name)
    d = model_dir(cfg, SEED, rank, world, args.workload, fmt)
    barrier()

    t0 = time.time()
    m = hm.HfModel.load_with_dtype(d, hm.DType.BF16, device=local) if fmt == "bf16" else hm.HfModel.load_gguf(d, device=local)
    kv_dtype = hm.DType.F32 if args.kv_dtype == "f32" else hm.DType.BF16
    PL = args.prompt_len if args.prompt_len is not None else PROMPTS[args.workload]
    max_seq = PL + 3 * (W + K) + 24
    if max_seq > cfg.max_position_embeddings:
        raise SystemExit(f"--steps/--warmup need {max_seq} positions; the checkpoint has {cfg.max_position_embeddings}")
    m.init_kv_cache(max_seq, batch=B, kv_dtype=kv_dtype)
    if rank == 0:
        log(f"[bench] engine ready in {time.time() - t0:.1f}s; {m.launches_per_step()} launches/step; weight bytes/step {m.weight_bytes()}")
    # every sequence of every rank decodes its own prompt
    prompts = [synth.prompt_ids(SEED + rank * B + b, PL, cfg.vocab_size) for b in range(B)]

    # ---- device-timed region: K steps, inputs resident, token fed back on the device ----
    first = [m.prefill(prompts[b], seq=b) for b in range(B)]
    m.decode_greedy_n(first, 0)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    rt = None
    if args.device_only:
        # a profiler started with `--profile-from-start off` sees the timed decode steps only (not the load and prefill launches)
        try:
            import torch

            rt = torch.cuda.cudart()
            rt.cudaProfilerStart()
        except Exception:
            rt = None
    ms = m.time_decode(W, K)
    if rt is not None:
        rt.cudaProfilerStop()
    barrier()
    clocks = sampler.stop() if sampler else None
    ms_max = vmax(ms)
    tok_per_s = world * B * K / (ms_max / 1e3)

    if args.device_only:
        if rank == 0:
            emit({"metric": "decode_tokens_per_s", "value": tok_per_s, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_max / K,
                  "config": {"workload": f"device-only run, prompt {PL}"}, "clocks": clocks})
        close()
        return

    # ---- end to end through the per-token C-ABI call (host token in, host token out) ----
    for b in range(B):
        m.reset_kv_cache(seq=b)
    t = time.perf_counter()
    cur = [m.prefill(prompts[b], seq=b) for b in range(B)]
    prefill_s = time.perf_counter() - t  # hm_prefill per sequence: host ids in, first token out (the kernels are warm from the device-timed region)
    for _ in range(W):
        _, nxt = m.decode_step(cur, want_logits=False)
        cur = [int(v) for v in nxt]
    barrier()
    t = time.perf_counter()
    for _ in range(K):
        _, nxt = m.decode_step(cur, want_logits=False)
        cur = [int(v) for v in nxt]
    e2e_s = time.perf_counter() - t
    barrier()
    e2e_tps = world * B * K / vmax(e2e_s)
    # the reference trait's decode_step returns the logits (Vec<f32> of vocab entries): the same loop with that copy
    t = time.perf_counter()
    for _ in range(K):
        _, nxt = m.decode_step(cur, want_logits=True)
        cur = [int(v) for v in nxt]
    e2e_lg_s = time.perf_counter() - t
    barrier()
    e2e_lg_tps = world * B * K / vmax(e2e_lg_s)
    # sampled generation at the reference's default settings (temperature 0.7, top-k 50, top-p 0.9, repetition
    # penalty 1.1; src/generate.rs:648-683) through hm_generate, the sampler on the device
    e2e_smp = None
    if B == 1:
        # two generations from an empty cache that differ only in length: the difference leaves the prefill out, as the
        # reference's decode rate does (src/generate.rs:820-841)
        n_short = 8
        n_long = min(n_short + K, max_seq - PL - 1)
        times = []
        for n_new in (n_short, n_long):
            m.reset_kv_cache(seq=0)
            t = time.perf_counter()
            got = m.generate_ids(prompts[0], n_new, hm.SamplingConfig(seed=SEED))
            times.append((time.perf_counter() - t, len(got)))
        barrier()
        (t_s, g_s), (t_l, g_l) = times
        if g_l > g_s and t_l > t_s:
            e2e_smp = {"value": world * (g_l - g_s) / vmax(t_l - t_s), "unit": "tok/s", "new_tokens": g_l - g_s, "d2h_bytes_per_step": 4,
                       "api": "hm_generate with SamplingConfig defaults, sampler on the device; rate over the tokens by which a long generation exceeds a short one (prefill excluded)"}

    # ---- per-kernel-class device times (launch by launch, CUDA events) ----
    prof = m.profile_decode(8)
    proj = [p for p in prof if p["name"] in ("qkv_rope_kvwrite", "o_proj_residual", "gate_up_swiglu", "down_residual", "lm_head")]
    proj_bytes = sum(p["bytes_per_step"] for p in proj)
    proj_ms = sum(p["ms_per_step"] for p in proj)
    proj_launches = sum(p["launches_per_step"] for p in proj)
    peak, peak_kind = measured_peak()
    achieved = proj_bytes / (proj_ms * 1e-3) / 1e9 if proj_ms > 0 else 0.0
    weight_bytes, launches_per_step = m.weight_bytes(), m.launches_per_step()

    c5 = None
    if args.workload == HEADLINE and not args.no_c5:
        m.close()
        m = None
        c5 = run_c5(hm, synth, rank, world, local, barrier, vmax, K, W, peak)

    close()
    if rank != 0:
        return
    T_avg = PL + W + (K + 1) / 2.0
    kv_bytes_tok = cfg.num_hidden_layers * 2 * cfg.kv_dim * (4 if args.kv_dtype == "f32" else 2)
    step_bytes = weight_bytes + B * (kv_bytes_tok * T_avg + kv_bytes_tok)  # weights once per step, every sequence's cache
    step_gbs = step_bytes * (tok_per_s / world / B) / 1e9
    if fmt != "bf16":
        kern = "gemv_kquant_kernel<1> (Q4_K/Q6_K projections: Q8_K activations, dp4a; LM head in f32)" if fmt == "q4_k_m" else "gemv_quant_kernel<1> (Q8_0/Q4_0 projections, block dots on mma.sync s8; LM head included)"
    elif B > 8:
        kern = "gemm_tc_kernel (tcgen05 projections over 64 rows; LM head included)"
    else:
        kern = "gemv_bf16_kernel<1> (QKV, O, gate/up, down and LM-head projections)"
    # DRAM bytes per projection launch from the ncu capture summarised under profiles/ (headline workload
    # only): 997.0 MB summed over the 97 projection launches of a step, against 987.9 MB algorithmic.
    known_traffic = args.workload == HEADLINE and proj_launches == HEADLINE_PROJECTION_LAUNCHES
    traffic = HEADLINE_PROJECTION_DRAM_BYTES_PER_STEP / HEADLINE_PROJECTION_LAUNCHES if known_traffic else None
    out = {
        "metric": "decode_tokens_per_s", "value": tok_per_s, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_max / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 accumulate over bf16 weights" if fmt == "bf16" else f"f32 accumulate over {fmt} blocks", "data": "synthetic",
        "config": headline_config(world, args.kv_dtype, weight_bytes / 1e6) if (args.workload == HEADLINE and PL == PROMPTS[HEADLINE]) else {
            "workload": wl_desc + f", {PL}-token prompt, greedy decode",
            "kv_cache": f"paged, 16 tokens/page, {args.kv_dtype}", "l2": f"inputs larger than L2: {weight_bytes / 1e6:.0f} MB of weights are streamed once per step (L2 is 126 MB)",
            "parallelism": f"replicas x{world}, independent sequences, no collective on the token path", "seed": SEED,
        },
        "clocks": clocks,
        "e2e": {"value": e2e_tps, "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B, "api": "hm_decode_step (host token ids in, greedy next token ids out, one stream sync per step)"},
        "e2e_logits": {"value": e2e_lg_tps, "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B + 4 * B * cfg.vocab_size,
                       "api": "hm_decode_step with the [vocab] f32 logits returned (the reference trait's decode_step -> Vec<f32>)"},
        "e2e_sampled": e2e_smp,
        "prefill": {"tok_per_s": world * B * PL / vmax(prefill_s), "prompt_tokens": PL, "api": "hm_prefill, one call per sequence, end to end"},
        "gpu_launches": launches_per_step * K,
        "roofline": {
            "bound": "hbm", "kernel": kern, "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "peak_source": f"{peak_kind} copy bandwidth", "traffic": traffic, "traffic_source": TRAFFIC_SOURCE if known_traffic else None,
            "per_launch": {"algorithmic_bytes": proj_bytes / max(proj_launches, 1), "device_us": 1e3 * proj_ms / max(proj_launches, 1)},
            "timing": "CUDA events on the engine's stream around graph replays of each kernel class (8 steps each), run after the timed region",
            "launches_per_step": proj_launches, "algorithmic_bytes_per_step": proj_bytes, "device_ms_per_step": proj_ms,
        },
        "step_roofline": {"bytes_per_step": step_bytes, "achieved_gbs": step_gbs, "frac_of_measured": step_gbs / peak, "frac_of_nominal_8TBs": step_gbs / NOMINAL_HBM_GBS},
        "kernels": [{"name": p["name"], "launches": p["launches_per_step"], "us": round(1e3 * p["ms_per_step"], 2), "MB": round(p["bytes_per_step"] / 1e6, 3),
                     "GBs": round(p["bytes_per_step"] / (p["ms_per_step"] * 1e-3) / 1e9, 1) if p["ms_per_step"] > 0 else None} for p in prof],
    }
    if c5 is not None:
        out["c5"] = c5
    if world == 1 and not args.no_cpu_baseline:
        if m is not None:
            m.close()
        steps_c, prompt_c = (32, 8) if args.workload == HEADLINE else (12, 4)
        tps, dt, threads = cpu_sample(d, cfg, steps_c, 2, prompt_c)
        out["cpu_baseline"] = {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port",
                               "sample": f"{steps_c} greedy decode steps of one sequence after an {prompt_c}-token prompt on the same weights ({dt:.1f} s of CPU time, {threads} OpenMP threads)"}
    else:
        out["cpu_baseline"] = None
    emit(out)


if __name__ == "__main__":
    main()
