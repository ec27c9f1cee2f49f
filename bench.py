#!/usr/bin/env python
"""Benchmark of the hierarchical sparse attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one pass of the span-attention forward over one batch of synthetic Q/K/V (the layer
shape of the N=4096 headline: bf16, H=16, head_dim=128, radius 16, causal, batch 32 per GPU).
Under torchrun every rank runs its own batch shard (weak scaling, no data-path collective);
time is the max over ranks of CUDA-event time between barriers.  Prints ONE JSON line on rank 0.

Keys beyond the base contract:
  roofline      the dominant kernel against the measured HBM copy bandwidth (MEASURED_PEAKS.json)
  cpu_baseline  the CPU oracle (a port of the reference's eager layer math) timed on this box's
                host cores on a bounded sample of the same workload
  e2e           same metric through the public Python API with host (pinned) inputs copied in
                and the result copied out inside the timed region
  extras        parent-node build and forward+backward figures on the same shape
`--impl reference` times the CPU oracle instead (the reference has no GPU-independent compiled
path; its own implementation of this layer on a CPU is eager PyTorch, which the oracle restates).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B per GPU, N, H, D, R, causal, dtype)
    "layer_n4096": (32, 4096, 16, 128, 16, True, torch.bfloat16),
    "layer_n4096_small": (4, 4096, 16, 128, 16, True, torch.bfloat16),     # for profiler captures
    "config2": (16, 512, 8, 64, 8, True, torch.bfloat16),
}
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the forward kernel, measured with ncu on
# `--workload layer_n4096_small` (profiles/), scaled by batch (traffic is proportional to batch).
NCU_TRAFFIC_BYTES_PER_BATCH_ELEM = {"layer_n4096": 317.2e6 / 4, "layer_n4096_small": 317.2e6 / 4}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def algorithmic_bytes_fwd(B, N, H, D, esize, causal):
    """Rows that must cross HBM once: Q, Out, and the attended K/V rows (module docstring of DESIGN.md)."""
    row = H * D * esize
    return B * row * ((5 * N - 2) if causal else (6 * N - 4))


def algorithmic_bytes_bwd(B, N, H, D, esize, causal):
    row = H * D * esize
    return B * row * ((11 * N - 4) if causal else (12 * N - 6))


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            # honour CUDA_VISIBLE_DEVICES when mapping the torch index to an NVML handle
            uuid = torch.cuda.get_device_properties(index).uuid
            self._h = None
            for i in range(pynvml.nvmlDeviceGetCount()):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                u = pynvml.nvmlDeviceGetUUID(h)
                u = u.decode() if isinstance(u, bytes) else u
                if str(uuid) in u:
                    self._h = h
            if self._h is None:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None
        self.period = period_s

    def _loop(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def dist_setup(gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return world, rank, local


def make_inputs(B, N, H, D, dtype, seed, device, pinned=False):
    """Q/K/V ~ N(0,1) from a CPU generator (identical bits for the oracle and the GPU)."""
    gen = torch.Generator().manual_seed(seed)
    out = []
    for rows in (N, 2 * N - 1, 2 * N - 1):
        t = torch.randn(B, rows, H, D, generator=gen, dtype=torch.float32).to(dtype)
        if pinned:
            t = t.pin_memory()
        out.append(t if device is None else t.to(device))
    return out


def time_cuda(fn, steps, warmup, barrier):
    """CUDA-event time of `steps` calls of fn on the current stream, in ms (this rank)."""
    for _ in range(warmup):
        fn()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1)


def oracle_tokens_per_s(workload, budget_s: float, threads: int):
    """CPU oracle on a bounded sample of the workload's leaves (all heads, one batch entry)."""
    from oracle import hsa_oracle as orc
    B, N, H, D, R, causal, dtype = WORKLOADS[workload]
    torch.set_num_threads(threads)
    Q, K, V = make_inputs(1, N, H, D, dtype, 1234, None)
    orc.span_candidates(N, R, causal)           # topology tables are cached by the layer, not per call
    chunk = 256
    done, t0 = 0, time.perf_counter()
    start = 0
    while True:
        leaves = (torch.arange(chunk) + start) % N
        orc.hierarchical_attention(Q, K, V, R, causal, leaves=leaves)
        done += chunk
        start += chunk
        el = time.perf_counter() - t0
        if el > budget_s or done >= 8 * N:
            break
    return done / el, done, el


def run_reference(args):
    world, rank, local = dist_setup(args.gpus)
    if rank != 0:
        return
    B, N, H, D, R, causal, dtype = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    per_step = max(0.5, min(10.0, 120.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        oracle_tokens_per_s(args.workload, per_step, cores)
    vals, toks, secs = [], 0, 0.0
    for _ in range(args.steps):
        v, n, s = oracle_tokens_per_s(args.workload, per_step, cores)
        vals.append(v); toks += n; secs += s
    value = toks / secs if secs > 0 else 0.0
    line = {
        "impl": "reference", "metric": "hier-attn layer tokens/s (span attention forward, N=4096)",
        "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * secs / max(1, args.steps), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "B_per_gpu": B, "N": N, "H": H, "D": D, "radius": R, "causal": causal,
                   "sharding": "rank 0 only", "l2": "cpu run on a bounded sample of the workload's leaves"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{toks} leaves x {H} heads of one batch entry over {args.steps} steps "
                                   f"(eager PyTorch CPU oracle, {cores} threads)"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


LM_CONFIGS = {
    # BASELINE configs 3 and 4: 6 layers, d_model 512, 8 heads, FFN 2048, window 16, vocab 50257, bf16
    "lm_8x2048": dict(batch=8, seq=2048), "lm_8x4096": dict(batch=8, seq=4096),
}


def run_lm(args, device, world, rank, barrier, use_dist, strong=False):
    """Training step (forward, loss, backward, gradient all-reduce, clip, AdamW) of the hierarchical LM
    on Zipf(1.1) token ids.  Per-GPU batch fixed (weak scaling) unless `strong`, which splits the config's
    batch over the ranks (global batch fixed).  Returns whole-job tokens/s."""
    import torch.distributed as dist
    from sparseattention_b200.dp import BucketedGradAverager
    from sparseattention_b200.lm import TransformerLM, lm_loss, zipf_tokens

    cfg = dict(LM_CONFIGS[args.lm])
    if strong:
        cfg["batch"] //= world
    vocab = 50257
    torch.manual_seed(0)
    model = TransformerLM(vocab, 512, 8, 2048, 6, dropout=0.1, window_size=16).to(device)
    avg = BucketedGradAverager(model.parameters())
    use_graph = not args.no_cuda_graph
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, fused=True, capturable=use_graph)
    host_tokens = zipf_tokens(cfg["batch"], cfg["seq"] + 1, vocab, seed=4321 + rank).pin_memory()
    tokens = torch.empty(host_tokens.shape, dtype=host_tokens.dtype, device=device)
    loss_buf = torch.zeros((), device=device)
    losses = []

    def body():
        tokens.copy_(host_tokens, non_blocking=True)        # this step's inputs come from pinned host memory
        avg.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = lm_loss(model, tokens)
        loss.backward()
        avg.finish()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        loss_buf.copy_(loss.detach())

    # The whole step is captured once in a CUDA graph and replayed (the launches of the ~2500 small kernels of
    # a step otherwise cost more host time than the GPU needs); eager launching is used if capture is refused.
    graph = None
    if use_graph:
        try:
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                for _ in range(3):
                    body()
            torch.cuda.current_stream(device).wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                body()
        except Exception as exc:                              # pragma: no cover - depends on the runtime
            graph = None
            graph_error = f"{type(exc).__name__}: {exc}"[:200]
            torch.cuda.synchronize()
    if use_dist:                                              # every rank must take the same path
        flag = torch.tensor([1 if graph is not None else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            graph = None

    def step():
        if graph is not None:
            graph.replay()
        else:
            body()
        losses.append(loss_buf.clone())

    steps = max(3, min(args.steps, 10))
    ms = time_cuda(step, steps, 3, barrier)
    if use_dist:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms /= steps
    tok = cfg["batch"] * cfg["seq"] * world
    nparams = sum(p.numel() for p in model.parameters())
    out = {"config": args.lm, "scaling": "strong" if strong else "weak", "tokens_per_s": tok / (ms * 1e-3),
           "ms_per_step": ms, "steps": steps,
           "global_batch": cfg["batch"] * world, "seq_len": cfg["seq"], "params": nparams,
           "allreduce_bytes_per_step": avg.bytes_per_step() if world > 1 else 0,
           "loss_first": float(losses[0]), "loss_last": float(losses[-1]),
           "step": "fwd + label-smoothed CE + bwd + NCCL grad all-reduce + clip + AdamW, bf16 autocast",
           "cuda_graph": graph is not None}
    del model, opt, avg, graph
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    import sparseattention_b200 as hsa
    from sparseattention_b200 import _lib
    from sparseattention_b200.ops import functional as F

    world, rank, local = dist_setup(args.gpus)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in the library)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"          # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=device)

        def barrier():
            dist.barrier()
    else:
        def barrier():
            pass

    B, N, H, D, R, causal, dtype = WORKLOADS[args.workload]
    esize = torch.finfo(dtype).bits // 8
    _lib.load()
    Qh, Kh, Vh = make_inputs(B, N, H, D, dtype, 1234 + rank, None, pinned=True)
    Q, K, V = (t.to(device) for t in (Qh, Kh, Vh))
    tables = hsa.build_tree_topology(N, causal, device=device)
    footprint = sum(t.numel() * t.element_size() for t in (Q, K, V)) + Q.numel() * esize

    # ---- device-resident: raw forward (inference form: no LSE) -------------------------------
    def step():
        F.span_attention_forward(Q, K, V, R, causal, need_lse=False)

    with ClockSampler(local) as clk:
        ms = time_cuda(step, args.steps, args.warmup, barrier)
    if use_dist:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    tokens_step = B * N * world
    value = tokens_step / (ms_step * 1e-3)
    peak, peak_kind = measured_peaks()
    alg = algorithmic_bytes_fwd(B, N, H, D, esize, causal)
    achieved = alg / (ms_step * 1e-3) / 1e9
    traffic = NCU_TRAFFIC_BYTES_PER_BATCH_ELEM.get(args.workload)

    # ---- end to end through the public API with host buffers -----------------------------------
    out_host = torch.empty((B, N, H, D), dtype=dtype).pin_memory()
    e2e_steps = max(2, min(args.steps, 5))

    def e2e_step():
        # public host-side entry point: pinned inputs in, pinned result out, copies overlapped with compute
        F.hierarchical_attention_from_host(Qh, Kh, Vh, R, causal, out=out_host, device=device)

    e2e_ms = time_cuda(e2e_step, e2e_steps, 1, barrier)
    if use_dist:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = tokens_step / (e2e_ms / e2e_steps * 1e-3)
    h2d = sum(t.numel() * t.element_size() for t in (Qh, Kh, Vh))
    d2h = out_host.numel() * out_host.element_size()

    # ---- extras: training forward (+LSE), backward, parent build on the same shape -------------
    extras = {}
    launches_per_step = 1
    if rank == 0 and not args.no_extras:
        out, lse = F.span_attention_forward(Q, K, V, R, causal, need_lse=True)
        go = torch.randn_like(out)
        bsteps = max(3, min(args.steps, 20))
        bms = time_cuda(lambda: F.span_attention_backward(Q, K, V, out, lse, go, R, causal), bsteps, 3,
                        lambda: None) / bsteps
        balg = algorithmic_bytes_bwd(B, N, H, D, esize, causal)
        extras["span_bwd"] = {"ms": bms, "tokens_per_s": B * N / (bms * 1e-3), "achieved_gbs": balg / (bms * 1e-3) / 1e9,
                              "frac_of_hbm": balg / (bms * 1e-3) / 1e9 / peak}
        del out, lse, go
        # parent build: all levels, op level (8 rows per parent forward)
        sizes = []
        n = N
        while n > 1:
            n //= 2
            sizes.append(n)
        gen = torch.Generator(device=device).manual_seed(7)
        Pq, Pk, Pv = (torch.randn(B, N - 1, H, D, generator=gen, device=device, dtype=dtype) for _ in range(3))
        Ck, Cv = (torch.randn(B, N, H, D, generator=gen, device=device, dtype=dtype) for _ in range(2))
        qs, ks, vs = (torch.split(t, sizes, dim=1) for t in (Pq, Pk, Pv))

        def parents():
            kc, vc = Ck, Cv
            for lvl, P in enumerate(sizes):
                hsa.build_parent_nodes(qs[lvl], ks[lvl], vs[lvl], kc[:, :2 * P], vc[:, :2 * P])

        with torch.no_grad():
            pms = time_cuda(parents, bsteps, 3, lambda: None) / bsteps
        palg = B * H * D * esize * 8 * (N - 1)
        extras["parent_build_fwd_all_levels"] = {
            "ms": pms, "launches": len(sizes), "achieved_gbs": palg / (pms * 1e-3) / 1e9,
            "frac_of_hbm": palg / (pms * 1e-3) / 1e9 / peak}
        # backward of every level through the C ABI directly (15 rows per parent)
        lib = _lib.load()
        grads = [torch.empty_like(t) for t in (Pq, Pk, Pv, Ck, Cv)]
        gq, gk, gv = (torch.split(t, sizes, dim=1) for t in grads[:3])
        gout = torch.randn_like(Pq)
        gos = torch.split(gout, sizes, dim=1)
        dt = _lib.dtype_code(Pq)

        def parents_bwd():
            for lvl, P in enumerate(sizes):
                views = [_lib.rows_view(t) for t in (gos[lvl], qs[lvl], ks[lvl], vs[lvl], Ck[:, :2 * P], Cv[:, :2 * P],
                                                     gq[lvl], gk[lvl], gv[lvl], grads[3][:, :2 * P], grads[4][:, :2 * P])]
                _lib.check(lib.hsa_parent_nodes_bwd(*views, B, P, H, D, dt, _lib.stream_ptr(device)), "hsa_parent_nodes_bwd")

        pbms = time_cuda(parents_bwd, bsteps, 3, lambda: None) / bsteps
        pbalg = B * H * D * esize * 15 * (N - 1)
        extras["parent_build_bwd_all_levels"] = {
            "ms": pbms, "launches": len(sizes), "achieved_gbs": pbalg / (pbms * 1e-3) / 1e9,
            "frac_of_hbm": pbalg / (pbms * 1e-3) / 1e9 / peak}
        del Pq, Pk, Pv, Ck, Cv, grads, gout

    # ---- the model that calls the layer: data-parallel LM training step (all ranks) ---------------
    if not args.no_lm:
        extras["lm_train"] = run_lm(args, device, world, rank, barrier, use_dist)
        if world > 1 and LM_CONFIGS[args.lm]["batch"] % world == 0:
            # secondary line: the same global batch as one GPU, split over the ranks
            extras["lm_train_strong"] = run_lm(args, device, world, rank, barrier, use_dist, strong=True)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        v, n, s = oracle_tokens_per_s(args.workload, args.cpu_seconds, cores)
        cpu = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"{n} leaves x {H} heads of one batch entry, {s:.1f} s "
                         f"(eager PyTorch CPU oracle, {cores} threads)"}

    if rank == 0:
        line = {
            "metric": "hier-attn layer tokens/s (span attention forward, N=4096)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if dtype == torch.bfloat16 else str(dtype).replace("torch.", ""),
            "data": "synthetic",
            "config": {"workload": args.workload, "B_per_gpu": B, "N": N, "H": H, "D": D, "radius": R,
                       "causal": causal, "sharding": "batch shards, no collective",
                       "l2": f"inputs+outputs {footprint / 1e6:.0f} MB per GPU exceed the 126 MB L2; no flush"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": peak_kind,
                         "traffic": None if traffic is None else traffic * B,
                         "algorithmic_bytes_per_launch": alg, "kernel_ms": ms_step},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "steps": e2e_steps},
            "gpu_launches": args.steps * launches_per_step,
            "clocks": clk.summary(),
            "extras": extras,
        }
        emit(line)
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()


def run_sweep(args):
    """BASELINE config 5: forward-only bf16 sweep over N and batch (H=16, D=128, causal, radius 16 and 32).
    Prints a markdown table: achieved algorithmic GB/s and fraction of the measured HBM copy bandwidth."""
    from sparseattention_b200.ops import functional as F
    torch.cuda.set_device(0)
    peak, kind = measured_peaks()
    H, D = 16, 128
    print(f"| N | B | radius | ms | tokens/s | GB/s (algorithmic) | of {kind} {peak:.0f} GB/s | footprint MB |")
    print("|---|---|---|---|---|---|---|---|")
    for N in (1024, 2048, 4096, 8192, 16384, 32768):
        for B in (1, 8, 32):
            if 6 * B * N * H * D * 2 > 40e9:
                continue
            gen = torch.Generator(device="cuda").manual_seed(N + B)
            Q = torch.randn(B, N, H, D, generator=gen, device="cuda", dtype=torch.bfloat16)
            K = torch.randn(B, 2 * N - 1, H, D, generator=gen, device="cuda", dtype=torch.bfloat16)
            V = torch.randn(B, 2 * N - 1, H, D, generator=gen, device="cuda", dtype=torch.bfloat16)
            for R in (16, 32):
                ms = time_cuda(lambda: F.span_attention_forward(Q, K, V, R, True, need_lse=False), 30, 5, lambda: None) / 30
                alg = algorithmic_bytes_fwd(B, N, H, D, 2, True)
                gbs = alg / (ms * 1e-3) / 1e9
                foot = 6 * B * N * H * D * 2 / 1e6
                print(f"| {N} | {B} | {R} | {ms:.4f} | {B * N / (ms * 1e-3):.3e} | {gbs:.0f} | {gbs / peak:.3f} | {foot:.0f} |")
            del Q, K, V


_JSON_OUT = None


def emit(line: dict) -> None:
    out = _JSON_OUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="layer_n4096", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-lm", action="store_true")
    ap.add_argument("--no-cuda-graph", action="store_true", help="launch the LM step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--lm", default="lm_8x4096", choices=sorted(LM_CONFIGS))
    ap.add_argument("--sweep", action="store_true", help="print the forward sweep over N and batch instead of the JSON line")
    args = ap.parse_args()
    if args.sweep:
        run_sweep(args)
        return
    # Libraries (NCCL's version banner, for one) write to file descriptor 1; keep the real stdout for the
    # single JSON line and send everything else to stderr.
    global _JSON_OUT
    sys.stdout.flush()
    _JSON_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
