"""Per-kernel sweeps of the decode path on one GPU: `python -m homura_b200.sweeps projections|attention`.

Each line of output is one JSON record.  Timing is by CUDA events around replays of a CUDA graph
that holds one rotation of launches; the weights (or KV pages) of consecutive launches come from a rotation of copies
larger than the L2 cache, so every launch streams from HBM.  Shapes are the projection and attention
shapes of Qwen2.5-0.5B / 1.5B / Qwen3-0.6B (src/hf/config.rs:11-38 gives the fields they come from); the
attention sweep defaults to the Qwen3-0.6B geometry (16 query / 8 KV heads, head_dim 128) on bf16 pages.
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np

import homura_b200 as hm
from homura_b200 import synth

# (K, N): qkv / gate_up / down of Qwen2.5-0.5B, gate_up / down of Qwen2.5-1.5B, one LM-head shape
PROJECTION_SHAPES = [(896, 1152), (896, 9728), (4864, 896), (1536, 17920), (8960, 1536), (1024, 151936)]
ROTATE_BYTES = 256 << 20


def _events():
    import torch

    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), torch


def _time_launches(fn, n_rot: int, target_ms: float = 30.0):
    """fn(i, stream) launches once using rotation slot i % n_rot.  The launches of one rotation are
    captured into a CUDA graph (so that small kernels are not timed by the host's launch rate) and
    the graph is replayed between two events.  Returns (microseconds per launch, launches, mode)."""
    e0, e1, torch = _events()
    side = torch.cuda.Stream()
    sp = side.cuda_stream
    per_graph = max(n_rot, 8)
    with torch.cuda.stream(side):
        for i in range(max(3, n_rot)):  # warm-up touches every slot and sizes the library's scratch
            fn(i, sp)
    hm.dev_sync()
    graph = None
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(per_graph):
                fn(i, sp)
        graph = g
    except Exception as ex:  # capture refused: time plain stream launches instead
        print(f"[sweeps] graph capture failed ({ex}); timing stream launches", file=sys.stderr)
        hm.dev_sync()
    reps = 1
    while True:
        with torch.cuda.stream(side):
            e0.record(side)
            for r in range(reps):
                if graph is not None:
                    graph.replay()
                else:
                    for i in range(per_graph):
                        fn(i, sp)
            e1.record(side)
        hm.dev_sync()
        ms = e0.elapsed_time(e1)
        if ms >= target_ms or reps >= 4096:
            return ms * 1000.0 / (reps * per_graph), reps * per_graph, "graph" if graph is not None else "stream"
        reps = min(4096, max(reps * 2, int(reps * target_ms / max(ms, 1e-3)) + 1))


def projections(ms: list[int], peak_gbs: float, shapes=None, profile_launches: int = 0):
    rng = np.random.default_rng(5)
    for (K, N) in (shapes or PROJECTION_SHAPES):
        w = synth.f32_to_bf16_rne(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.02))
        slab = hm.pack_bf16_slabs(w).reshape(-1)
        tc = hm.pack_bf16_tc(w)
        n_rot = max(2, -(-ROTATE_BYTES // (2 * K * N)) + 1)
        bufs = {}
        for name, arr in (("slab", slab), ("tc", tc)):
            b = hm.DeviceBuffer(arr.nbytes * n_rot)
            for r in range(n_rot):
                b.upload(arr, r * arr.nbytes)
            bufs[name] = (b, arr.nbytes)
        xb = hm.DeviceBuffer(64 * K * 4)
        xb.upload(rng.standard_normal((64, K), dtype=np.float32))
        yb = hm.DeviceBuffer(64 * N * 4)
        for M in ms:
            paths = []
            if M <= 16:
                paths.append("gemv")
            if M >= 9:
                paths.append("tcgen05")
            for path in paths:
                if path == "gemv":
                    b, nb = bufs["slab"]
                    fn = lambda i, st: hm.gemv_bf16((xb.ptr, M), b.ptr + (i % n_rot) * nb, hm.LAYOUT_SLAB128, K=K, N=N, y=yb.ptr, stream=st)
                else:
                    b, nb = bufs["tc"]
                    fn = lambda i, st: hm.gemm_bf16_tc((xb.ptr, M), b.ptr + (i % n_rot) * nb, N, K=K, y=yb.ptr, stream=st)
                if profile_launches:  # a few plain launches for a profiler run, no timing
                    for i in range(profile_launches):
                        fn(i, None)
                    hm.dev_sync()
                    print(json.dumps({"sweep": "projection", "path": path, "M": M, "K": K, "N": N, "profile_launches": profile_launches}), flush=True)
                    continue
                us, iters, mode = _time_launches(fn, n_rot)
                alg = 2 * K * N  # weight bytes, read once per launch
                gbs = alg / us / 1e3
                print(json.dumps({"sweep": "projection", "path": path, "M": M, "K": K, "N": N, "us": round(us, 2), "GBps": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak_gbs, 3), "tflops": round(2.0 * M * K * N / us / 1e6, 2), "launches": iters, "rotation": n_rot, "timing": mode}), flush=True)
        for b, _ in bufs.values():
            b.free()
        xb.free()
        yb.free()


ATTENTION_GEOMETRY = {"qwen3-0.6b": (16, 8, 128), "qwen2.5-0.5b": (14, 2, 64), "qwen2.5-1.5b": (12, 2, 128), "tinyllama-1.1b": (32, 4, 64)}


def attention(kv_lens: list[int], batches: list[int], kv_dtype: str, peak_gbs: float, geometry: str = "qwen3-0.6b", profile_launches: int = 0):
    heads, kvh, hd = ATTENTION_GEOMETRY[geometry]  # query heads, KV heads, head_dim
    page = 16
    rng = np.random.default_rng(6)
    dt = hm.DType.F32 if kv_dtype == "f32" else hm.DType.BF16
    esz = 4 if kv_dtype == "f32" else 2
    for L in kv_lens:
        for B in batches:
            pages_per_seq = -(-L // page)
            page_bytes = kvh * page * hd * esz
            seq_bytes = 2 * pages_per_seq * page_bytes
            n_rot = max(1, min(8, -(-ROTATE_BYTES // (seq_bytes * B))))
            total_pages = pages_per_seq * B * n_rot
            if 2 * total_pages * page_bytes > (24 << 30):
                continue
            kb = hm.DeviceBuffer(total_pages * page_bytes)
            vb = hm.DeviceBuffer(total_pages * page_bytes)
            chunk = rng.standard_normal(min(total_pages * page_bytes // esz, 1 << 24), dtype=np.float32)
            src = chunk if kv_dtype == "f32" else synth.f32_to_bf16_rne(chunk)
            off = 0
            while off < total_pages * page_bytes:
                n = min(src.nbytes, total_pages * page_bytes - off)
                kb.upload(src.view(np.uint8)[:n], off)
                vb.upload(src.view(np.uint8)[:n], off)
                off += n
            pts = []
            for r in range(n_rot):
                perm = rng.permutation(pages_per_seq * B).astype(np.int32) + r * pages_per_seq * B
                pts.append(perm.reshape(B, pages_per_seq))
            pt = hm.DeviceBuffer(n_rot * B * pages_per_seq * 4)
            pt.upload(np.stack(pts))
            kl = hm.DeviceBuffer(B * 4)
            kl.upload(np.full(B, L, np.int32))
            q = hm.DeviceBuffer(B * heads * hd * 4)
            q.upload(rng.standard_normal((B, heads * hd), dtype=np.float32))
            out = hm.DeviceBuffer(B * heads * hd * 4)
            lib = hm.load_library()
            import ctypes as C

            def fn(i, st):
                r = i % n_rot
                rc = lib.hm_attn_decode_paged(C.c_void_p(q.ptr), C.c_void_p(kb.ptr), C.c_void_p(vb.ptr), int(dt), C.c_void_p(pt.ptr + r * B * pages_per_seq * 4), C.c_void_p(kl.ptr), B, heads, kvh, hd, page, pages_per_seq, C.c_void_p(out.ptr), C.c_void_p(st))
                if rc != 0:
                    raise hm.HomuraError(lib.hm_last_error_global())

            if profile_launches:  # a few plain launches for a profiler run, no timing
                for i in range(profile_launches):
                    fn(i, None)
                hm.dev_sync()
                print(json.dumps({"sweep": "attention", "geometry": geometry, "kv_dtype": kv_dtype, "kv_len": L, "batch": B, "profile_launches": profile_launches}), flush=True)
                for b in (kb, vb, pt, kl, q, out):
                    b.free()
                continue
            us, iters, mode = _time_launches(fn, n_rot, target_ms=20.0)
            alg = 2 * B * L * kvh * hd * esz
            gbs = alg / us / 1e3
            print(json.dumps({"sweep": "attention", "geometry": geometry, "kv_dtype": kv_dtype, "kv_len": L, "batch": B, "us": round(us, 2), "GBps": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak_gbs, 3), "launches": iters, "rotation": n_rot, "timing": mode}), flush=True)
            for b in (kb, vb, pt, kl, q, out):
                b.free()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("which", choices=["projections", "attention"])
    ap.add_argument("--m", type=int, nargs="*", default=[1, 4, 16, 64])
    ap.add_argument("--kv-len", type=int, nargs="*", default=[512, 4096, 32768])
    ap.add_argument("--batch", type=int, nargs="*", default=[1, 8, 64])
    ap.add_argument("--kv-dtype", choices=["f32", "bf16"], default="bf16")
    ap.add_argument("--geometry", choices=sorted(ATTENTION_GEOMETRY), default="qwen3-0.6b", help="attention: query heads / KV heads / head_dim of the named architecture")
    ap.add_argument("--shape", action="append", default=None, help="K,N of a projection; repeatable; default: the built-in shapes")
    ap.add_argument("--profile-launches", type=int, default=0, help="issue this many plain launches per case and exit (for ncu)")
    ap.add_argument("--hbm-peak-gbs", type=float, default=6545.6, help="copy bandwidth to report fractions against")
    a = ap.parse_args(argv)
    if a.which == "projections":
        shapes = [tuple(int(v) for v in sh.split(",")) for sh in a.shape] if a.shape else None
        projections(a.m, a.hbm_peak_gbs, shapes, a.profile_launches)
    else:
        attention(a.kv_len, a.batch, a.kv_dtype, a.hbm_peak_gbs, a.geometry, a.profile_launches)
    return 0


if __name__ == "__main__":
    sys.exit(main())
