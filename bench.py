#!/usr/bin/env python
"""Benchmark of the hierarchical sparse attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
                    [--only fwd|bwd|parents|parent_tree|lm|reference_triton]

One step = one pass of the span-attention forward over one batch of synthetic Q/K/V (the layer
shape of the N=4096 headline: bf16, H=16, head_dim=128, radius 16, causal, batch 32 per GPU).
Under torchrun every rank runs its own batch shard (weak scaling, no data-path collective);
time is the max over ranks of CUDA-event time between barriers.  Prints ONE JSON line on rank 0.

Keys beyond the base contract:
  roofline      the dominant kernel against the measured HBM copy bandwidth (MEASURED_PEAKS.json):
                `achieved` / `frac` are EFFECTIVE bandwidth (algorithmic bytes / kernel time),
                `frac_dram` is measured DRAM traffic (ncu, scaled by batch) / kernel time / peak
  cpu_baseline  the CPU oracle (a port of the reference's eager layer math) timed on this box's
                host cores on a bounded sample of the same workload
  e2e           same metric through the public Python API with host (pinned) inputs copied in
                and the result copied out inside the timed region
  extras        backward, parent-node build, a multi-second loop of the headline kernel with the
                sampled SM clock, the LM training step (8x4096 and 8x2048 per GPU; tensor roofline,
                exposed all-reduce time) and the reference's Triton package timed on the same GPU
`--impl reference` times the CPU oracle instead (the reference has no GPU-independent compiled
path; its own implementation of this layer on a CPU is eager PyTorch, which the oracle restates).
`--only X` runs just one kernel loop on the chosen workload and prints a short JSON line: the
command profiler captures are taken from.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
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
    "layer_n4096_b8": (8, 4096, 16, 128, 16, True, torch.bfloat16),        # for profiler captures
    "b16_h8_n512": (16, 512, 8, 64, 8, True, torch.bfloat16),
}
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS_SUSTAINED = 1400.0

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of span_fwd_tc128_kernel at batch 4
# (`--workload layer_n4096_small`, ncu --set full): 316.6 MB.  Traffic is proportional to batch, because
# every (batch, head, tile) thread block reads its own rows.
NCU_TRAFFIC_BYTES_PER_BATCH_ELEM = 316.6e6 / 4
NCU_TRAFFIC_WORKLOADS = ("layer_n4096", "layer_n4096_small", "layer_n4096_b8")

REF_TRITON_DIR = os.path.join(ROOT, "baseline", "_ref", "hierarchical_attention")


def measured_peaks():
    """(HBM GB/s, sustained bf16 TFLOP/s, "measured" | "fallback")."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", FALLBACK_BF16_TFLOPS_SUSTAINED)), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS_SUSTAINED, "fallback"


def algorithmic_bytes_fwd(B, N, H, D, esize, causal):
    """Rows that must cross HBM once: Q, Out, and the attended K/V rows (causal: leaves + left children)."""
    row = H * D * esize
    return B * row * ((5 * N - 2) if causal else (6 * N - 4))


def algorithmic_bytes_bwd(B, N, H, D, esize, causal):
    """Read Q, Out, dOut and the attended K/V rows; write dQ and every row of dK, dV."""
    row = H * D * esize
    return B * row * ((11 * N - 4) if causal else (12 * N - 6))


def lm_flops_per_token(d=512, d_ff=2048, layers=6, vocab=50257):
    """Forward matrix-multiply flops per token of the LM: per layer 14 d x d projections (bottom-up: Q/K/V of the
    parents, K/V of the leaves, K/V of the refreshed parents, out_proj_y; top-down: Q, K/V of leaves and parents,
    out_proj_x) and the feed-forward pair, plus the LM head."""
    return layers * (14 * 2 * d * d + 4 * d * d_ff) + 2 * d * vocab


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


def time_graph(fn, per_graph=10, reps=5, warmup=2):
    """Device time per call of fn, in ms, from a replayed CUDA graph of `per_graph` calls: what a captured training step
    pays for the call, without the host time an eager launch from Python adds (tens of microseconds through ctypes)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            for _ in range(per_graph):
                keep = fn()
    torch.cuda.current_stream().wait_stream(side)
    ms = time_cuda(graph.replay, reps, warmup, lambda: None) / reps / per_graph
    del graph, keep
    return ms


def max_over_ranks(ms, device, use_dist):
    if not use_dist:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


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


# The LM of the training-step metric: 6 layers, d_model 512, 8 heads, FFN 2048, window 16, vocabulary 50257, bf16
# autocast; batch x sequence per GPU.
LM_CONFIGS = {"lm_8x2048": dict(batch=8, seq=2048), "lm_8x4096": dict(batch=8, seq=4096)}
LM_VOCAB = 50257


def run_lm(args, device, world, rank, barrier, use_dist, name, strong=False, allreduce=True, attention_cls=None,
           graph=True, steps=None, fused=True):
    """Training step (forward, loss, backward, gradient all-reduce, clip, AdamW) of the hierarchical LM
    on Zipf(1.1) token ids.  Per-GPU batch fixed (weak scaling) unless `strong`, which splits the config's
    batch over the ranks (global batch fixed).  `allreduce=False` leaves the collective out (to see what it
    costs on the same ranks).  `fused=False` runs the decoder layers and the LM head op by op under autocast (library
    products, separate element-wise kernels) instead of the library's fused nodes: the step as it was before them.
    Returns whole-job tokens/s and the step's share of the tensor roofline."""
    import torch.distributed as dist
    from sparseattention_b200.dp import BucketedGradAverager
    from sparseattention_b200.lm import TransformerLM, lm_loss, zipf_tokens
    from sparseattention_b200.train import GraphedStep

    cfg = dict(LM_CONFIGS[name])
    if strong:
        cfg["batch"] //= world
    torch.manual_seed(0)
    kwargs = {} if attention_cls is None else {"attention_cls": attention_cls}
    model = TransformerLM(LM_VOCAB, 512, 8, 2048, 6, dropout=0.1, window_size=16, **kwargs).to(device)
    if not fused:
        model.fused_head = False
        for layer in model.layers:
            layer.fused = False
    avg = BucketedGradAverager(model.parameters(), communicate=allreduce)
    use_graph = graph and not args.no_cuda_graph
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, fused=True, capturable=use_graph)
    host_tokens = zipf_tokens(cfg["batch"], cfg["seq"] + 1, LM_VOCAB, seed=4321 + rank).pin_memory()
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

    runner = GraphedStep(body, device, enabled=use_graph)
    if use_dist:                                              # every rank must take the same path
        flag = torch.tensor([1 if runner.captured else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            runner.drop_graph()

    def step():
        runner()
        losses.append(loss_buf.clone())

    steps = steps or max(3, min(args.steps, 10))
    ms = max_over_ranks(time_cuda(step, steps, 3, barrier), device, use_dist) / steps
    tok = cfg["batch"] * cfg["seq"] * world
    nparams = sum(p.numel() for p in model.parameters())
    _, tf_peak, peak_kind = measured_peaks()
    flops_step = 3 * lm_flops_per_token() * cfg["batch"] * cfg["seq"]        # per GPU: forward + backward (2x)
    tflops = flops_step / (ms * 1e-3) / 1e12
    out = {"config": name, "scaling": "strong" if strong else "weak", "tokens_per_s": tok / (ms * 1e-3),
           "ms_per_step": ms, "steps": steps,
           "global_batch": cfg["batch"] * world, "seq_len": cfg["seq"], "params": nparams,
           "allreduce_bytes_per_step": avg.bytes_per_step() if (world > 1 and allreduce) else 0,
           "loss_first": float(losses[0]), "loss_last": float(losses[-1]),
           "step": "fwd + label-smoothed CE + bwd + NCCL grad all-reduce + clip + AdamW, bf16 autocast",
           "cuda_graph": runner.captured, "fused_nodes": bool(fused and attention_cls is None),
           "roofline": {"bound": "tensor", "achieved": tflops, "peak": tf_peak, "unit": "TFLOP/s",
                        "frac": tflops / tf_peak, "peak_source": peak_kind + " (sustained bf16 matmul)",
                        "flops_per_step_per_gpu": flops_step,
                        "flops": "3 x forward matrix-multiply flops (120.7 MFLOP per token)"}}
    del model, opt, avg, runner
    torch.cuda.empty_cache()
    return out


def sizes_of(N):
    sizes, n = [], N
    while n > 1:
        n //= 2
        sizes.append(n)
    return sizes


def kernel_loops(workload, device):
    """Closures that run one kernel (or one kernel per tree level) of the hot path on `workload`:
    {"fwd", "bwd", "parents", "parents_bwd"} -> (callable, algorithmic bytes, launches per call)."""
    import sparseattention_b200 as hsa
    from sparseattention_b200 import _lib
    from sparseattention_b200.ops import functional as F

    B, N, H, D, R, causal, dtype = WORKLOADS[workload]
    esize = torch.finfo(dtype).bits // 8
    lib = _lib.load()
    state = {}

    def qkv():
        if "qkv" not in state:
            state["qkv"] = make_inputs(B, N, H, D, dtype, 1234, device)
        return state["qkv"]

    def fwd():
        Q, K, V = qkv()
        F.span_attention_forward(Q, K, V, R, causal, need_lse=False)

    def bwd():
        Q, K, V = qkv()
        if "bwd" not in state:
            out, lse = F.span_attention_forward(Q, K, V, R, causal, need_lse=True)
            state["bwd"] = (out, lse, torch.randn_like(out))
        out, lse, go = state["bwd"]
        F.span_attention_backward(Q, K, V, out, lse, go, R, causal)

    sizes = sizes_of(N)

    def parent_tensors():
        if "par" not in state:
            gen = torch.Generator(device=device).manual_seed(7)
            Pq, Pk, Pv = (torch.randn(B, N - 1, H, D, generator=gen, device=device, dtype=dtype) for _ in range(3))
            Ck, Cv = (torch.randn(B, N, H, D, generator=gen, device=device, dtype=dtype) for _ in range(2))
            state["par"] = (Pq, Pk, Pv, Ck, Cv)
        return state["par"]

    def parents():
        Pq, Pk, Pv, Ck, Cv = parent_tensors()
        qs, ks, vs = (torch.split(t, sizes, dim=1) for t in (Pq, Pk, Pv))
        with torch.no_grad():
            for lvl, P in enumerate(sizes):
                hsa.build_parent_nodes(qs[lvl], ks[lvl], vs[lvl], Ck[:, :2 * P], Cv[:, :2 * P])

    def parents_bwd():
        Pq, Pk, Pv, Ck, Cv = parent_tensors()
        if "pgrads" not in state:
            state["pgrads"] = ([torch.empty_like(t) for t in (Pq, Pk, Pv, Ck, Cv)], torch.randn_like(Pq))
        grads, gout = state["pgrads"]
        qs, ks, vs = (torch.split(t, sizes, dim=1) for t in (Pq, Pk, Pv))
        gq, gk, gv = (torch.split(t, sizes, dim=1) for t in grads[:3])
        gos = torch.split(gout, sizes, dim=1)
        dt = _lib.dtype_code(Pq)
        for lvl, P in enumerate(sizes):
            views = [_lib.rows_view(t) for t in (gos[lvl], qs[lvl], ks[lvl], vs[lvl], Ck[:, :2 * P], Cv[:, :2 * P],
                                                 gq[lvl], gk[lvl], gv[lvl], grads[3][:, :2 * P], grads[4][:, :2 * P])]
            _lib.check(lib.hsa_parent_nodes_bwd(*views, B, P, H, D, dt, _lib.stream_ptr(device)), "hsa_parent_nodes_bwd")

    row = B * H * D * esize
    return {
        "fwd": (fwd, algorithmic_bytes_fwd(B, N, H, D, esize, causal), 1),
        "bwd": (bwd, algorithmic_bytes_bwd(B, N, H, D, esize, causal), 2),
        "parents": (parents, row * 8 * (N - 1), len(sizes)),
        "parents_bwd": (parents_bwd, row * 15 * (N - 1), len(sizes)),
    }, state


def gemm_table(device, steps=20):
    """The dense products of one LM training step (8 x 4096 tokens, d_model 512, FFN 2048, padded vocabulary 50304) on
    the library's tcgen05 kernel and, beside it, on torch.matmul (the vendor library): TFLOP/s each, device time per call
    inside a replayed CUDA graph."""
    from sparseattention_b200.ops.gemm import gemm
    rows = 8 * 4096
    shapes = [("qkv_y  Y=XW^T", rows, 1536, 512), ("kv     Y=XW^T", rows, 1024, 512), ("proj   Y=XW^T", rows, 512, 512),
              ("fc1    Y=XW^T", rows, 2048, 512), ("fc2    Y=XW^T", rows, 512, 2048), ("head   Y=XW^T", rows, 50304, 512)]
    _, tf_peak, _ = measured_peaks()
    out = []
    gen = torch.Generator(device=device).manual_seed(3)
    for name, M, N, K in shapes:
        X = torch.randn(M, K, generator=gen, device=device, dtype=torch.bfloat16)
        W = torch.randn(N, K, generator=gen, device=device, dtype=torch.bfloat16)
        dY = torch.randn(M, N, generator=gen, device=device, dtype=torch.bfloat16)
        flops = 2.0 * M * N * K
        rec = {"product": name.split()[0], "M": M, "N": N, "K": K}
        for kind, ours, lib in (
                ("fwd", lambda: gemm(X, W), lambda: torch.matmul(X, W.t())),
                ("dx", lambda: gemm(dY, W, b_t=True), lambda: torch.matmul(dY, W)),
                ("dw", lambda: gemm(dY.unsqueeze(0), X.unsqueeze(0), a_t=True, b_t=True, out_dtype=torch.float32),
                 lambda: torch.matmul(dY.t(), X))):
            # both inside replayed graphs: an eager call of the small shapes is bound by the host on either side
            mo = time_graph(ours)
            ml = time_graph(lib)
            rec[kind] = {"ours_ms": mo, "ours_tflops": flops / (mo * 1e-3) / 1e12, "library_ms": ml,
                         "library_tflops": flops / (ml * 1e-3) / 1e12,
                         "frac_of_sustained_peak": flops / (mo * 1e-3) / 1e12 / tf_peak}
        out.append(rec)
        del X, W, dY
    return out


def parent_tree_table(device, steps=20, B=8, N=4096, H=8, D=64):
    """The bottom-up refresh above level 0 at the LM's shape (8 sequences of 4096 leaves, 8 heads of 64): one cooperative
    launch per tree and direction against one projection + one attention launch per level (what it replaces)."""
    import sparseattention_b200.fused_layer as fl
    from sparseattention_b200.ops.gemm import gemm
    d, M = H * D, N - 1
    gen = torch.Generator(device=device).manual_seed(11)
    rnd = lambda *s: torch.randn(*s, generator=gen, device=device).bfloat16()          # noqa: E731
    QKVp, Rb, KVc, W = rnd(B, M, 3 * d), rnd(B, M, d), rnd(B, M, 2 * d), (rnd(2 * d, d) * 0.05)
    dRf = torch.randn(B, M, d, generator=gen, device=device)
    dRb, dQKVp, dKVc = dRf.bfloat16(), torch.empty_like(QKVp), torch.empty_like(KVc)
    sizes, offs = fl.level_layout(N)
    L = len(sizes)

    def per_level_fwd():
        for lvl in range(1, L):
            po, pp, off, P = offs[lvl - 1], sizes[lvl - 1], offs[lvl], sizes[lvl]
            gemm(Rb[:, po:po + pp], W, out=KVc[:, po:po + pp])
            sl = QKVp[:, off:off + P]
            fl._parent_fwd(sl[..., :d], sl[..., d:2 * d], sl[..., 2 * d:], KVc[:, po:po + pp, :d], KVc[:, po:po + pp, d:],
                           Rb[:, off:off + P], H)

    def per_level_bwd():
        for lvl in range(L - 1, 0, -1):
            po, pp, off, P = offs[lvl - 1], sizes[lvl - 1], offs[lvl], sizes[lvl]
            sl, dsl, dkv = QKVp[:, off:off + P], dQKVp[:, off:off + P], dKVc[:, po:po + pp]
            fl._parent_bwd(dRb[:, off:off + P], sl[..., :d], sl[..., d:2 * d], sl[..., 2 * d:], KVc[:, po:po + pp, :d],
                           KVc[:, po:po + pp, d:], dsl[..., :d], dsl[..., d:2 * d], dsl[..., 2 * d:], dkv[..., :d], dkv[..., d:], H)
            gemm(dkv, W, b_t=True, out=dRf[:, po:po + pp], accumulate=True, copy_bf16=dRb[:, po:po + pp])

    out = {"shape": {"B": B, "N": N, "H": H, "D": D, "levels_fused": L - 1}}
    for name, fn, launches in (
            ("parent_tree_fwd", lambda: fl._parent_tree_fwd(QKVp, Rb, KVc, W, N, H, 1, None), 1),
            ("per_level_fwd", per_level_fwd, 2 * (L - 1)),
            ("parent_tree_bwd", lambda: fl._parent_tree_bwd(QKVp, KVc, dRf, dRb, dQKVp, dKVc, W, N, H, 1, None), 1),
            ("per_level_bwd", per_level_bwd, 2 * (L - 1))):
        ms = time_cuda(fn, steps, 3, lambda: None) / steps
        out[name] = {"ms": ms, "launches": launches}
    out["status_word"] = fl.parent_tree_status(fl._parent_tree_fwd(QKVp, Rb, KVc, W, N, H, 1, None))
    return out


def run_only(args):
    """One kernel loop on the chosen workload (what profiler captures are taken from)."""
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    if args.only == "gemm":
        emit({"only": "gemm", "products": gemm_table(device, max(3, min(args.steps, 20)))})
        return
    if args.only == "parent_tree":
        emit({"only": "parent_tree", **parent_tree_table(device, max(3, min(args.steps, 20)))})
        return
    if args.only == "reference_triton":
        emit(reference_triton_child(args, device))
        return
    if args.only == "lm":
        out = run_lm(args, device, 1, 0, lambda: None, False, args.lm, graph=not args.no_cuda_graph, fused=not args.lm_eager)
        emit({"only": "lm", **out})
        return
    loops, _ = kernel_loops(args.workload, device)
    fn, alg, launches = loops[args.only]
    ms = time_cuda(fn, args.steps, args.warmup, lambda: None) / args.steps
    peak, _, kind = measured_peaks()
    emit({"only": args.only, "workload": args.workload, "ms": ms, "launches_per_call": launches,
          "achieved_gbs": alg / (ms * 1e-3) / 1e9, "frac_of_hbm": alg / (ms * 1e-3) / 1e9 / peak, "peak_source": kind})


# ---------------------------------------------------------------------------------------------------------------
# The reference project's own Triton package, unmodified, on this GPU (a copy of its `hierarchical_attention`
# directory under baseline/_ref/, made by __graft_entry__.build() where the reference checkout is mounted).
# Runs in a child process with a time limit: a failure of Triton's JIT on this GPU, or a fault in code this
# repository does not control, must not take the benchmark with it.
# ---------------------------------------------------------------------------------------------------------------
def load_reference_package():
    init = os.path.join(REF_TRITON_DIR, "__init__.py")
    if not os.path.exists(init):
        return None
    spec = importlib.util.spec_from_file_location("reference_hierarchical_attention", init,
                                                  submodule_search_locations=[REF_TRITON_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["reference_hierarchical_attention"] = mod
    spec.loader.exec_module(mod)
    return mod


def reference_triton_child(args, device):
    ref = load_reference_package()
    if ref is None:
        return {"unavailable": "baseline/_ref/hierarchical_attention is not there (reference checkout absent at build time)"}
    import sparseattention_b200 as hsa
    out = {"package": "reference hierarchical_attention (Triton JIT), unmodified", "triton": None}
    try:
        import triton
        out["triton"] = triton.__version__
    except Exception as exc:
        return {"unavailable": f"triton does not import: {exc}"[:200]}
    B, N, H, D, R, causal, dtype = WORKLOADS[args.workload]
    nsteps, nwarm = 10, 3

    def timed(fn):
        return time_cuda(fn, nsteps, nwarm, lambda: None) / nsteps

    def section(name, fn):
        try:
            out[name] = fn()
        except Exception as exc:                      # JIT failure, unsupported shape, out of memory ...
            out[name] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
            torch.cuda.synchronize()

    # ---- op level: span attention forward and forward+backward on the benchmark's Q/K/V
    def span_ops():
        Q, K, V = make_inputs(B, N, H, D, dtype, 1234, device)
        res = {"shape": {"B": B, "N": N, "H": H, "D": D, "radius": R, "causal": causal, "dtype": "bf16"}}
        for label, pkg in (("reference", ref), ("ours", hsa)):
            t = pkg.build_tree_topology(N, is_causal=causal, device=device)
            mask = t["forward_mask"] if causal else None
            with torch.no_grad():
                fwd_ms = timed(lambda: pkg.hierarchical_attention(Q, K, V, t["forward_idx"], t["backward_gather"], mask, R))
            q, k, v = (x.clone().requires_grad_() for x in (Q, K, V))
            go = torch.randn_like(Q)

            def fb():
                o = pkg.hierarchical_attention(q, k, v, t["forward_idx"], t["backward_gather"], mask, R)
                o.backward(go)
                q.grad = k.grad = v.grad = None
            res[label] = {"fwd_ms": fwd_ms, "fwd_tokens_per_s": B * N / (fwd_ms * 1e-3), "fwd_bwd_ms": timed(fb)}
            del q, k, v, go
            torch.cuda.empty_cache()
        res["speedup_fwd"] = res["reference"]["fwd_ms"] / res["ours"]["fwd_ms"]
        res["speedup_fwd_bwd"] = res["reference"]["fwd_bwd_ms"] / res["ours"]["fwd_bwd_ms"]
        return res

    # ---- module level: cross_update_Y forward+backward at the shape the reference's own benchmark uses
    # (hierarchical_attention_project/Hierarchical_Attention_Triton_Test.py:504: B 32, N 4096, 8 heads of 64)
    def bottom_up():
        Bm, Nm, Hm, Dm = 32, 4096, 8, 64
        dim = Hm * Dm
        res = {"shape": {"B": Bm, "N": Nm, "H": Hm, "D": Dm, "dtype": "bf16"}}
        x = torch.randn(Bm, Nm, dim, device=device, dtype=dtype, requires_grad=True)
        y = torch.randn(Bm, Nm - 1, dim, device=device, dtype=dtype, requires_grad=True)
        dout = torch.randn(Bm, Nm - 1, dim, device=device, dtype=dtype)
        for label, pkg in (("reference", ref), ("ours", hsa)):
            torch.manual_seed(0)
            m = pkg.HierarchicalAttention(dim, Hm, dropout=0.0).to(device).to(dtype).eval()

            def fb():
                o = m.cross_update_Y(x, y)
                o.backward(dout)
                m.zero_grad(); x.grad = None; y.grad = None
            res[label] = {"fwd_bwd_ms": timed(fb)}
            del m
        res["speedup"] = res["reference"]["fwd_bwd_ms"] / res["ours"]["fwd_bwd_ms"]
        return res

    # ---- model level: one LM training step with the reference's module injected, both launched eagerly
    def lm_step():
        res = {"config": args.lm, "launch": "eager (no CUDA graph) for both"}
        for label, cls in (("reference", ref.HierarchicalAttention), ("ours", None)):
            r = run_lm(args, device, 1, 0, lambda: None, False, args.lm, attention_cls=cls, graph=False, steps=5)
            res[label] = {"ms_per_step": r["ms_per_step"], "tokens_per_s": r["tokens_per_s"], "loss_last": r["loss_last"]}
        res["speedup"] = res["reference"]["ms_per_step"] / res["ours"]["ms_per_step"]
        return res

    section("span_attention", span_ops)
    section("cross_update_Y", bottom_up)
    section("lm_train_step", lm_step)
    return out


def reference_triton_parent(args):
    """Run `--only reference_triton` in a child with a time limit and return its JSON (or why there is none)."""
    if not os.path.exists(os.path.join(REF_TRITON_DIR, "__init__.py")):
        return {"unavailable": "baseline/_ref/hierarchical_attention is not there (reference checkout absent at build time)"}
    cmd = [sys.executable, os.path.abspath(__file__), "--only", "reference_triton", "--workload", args.workload, "--lm", args.lm]
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=args.reference_triton_seconds)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"no result within {args.reference_triton_seconds} s (child process stopped)"}
    for ln in reversed(res.stdout.strip().splitlines()):
        try:
            return json.loads(ln)
        except Exception:
            continue
    return {"unavailable": f"child exited {res.returncode}: {res.stderr.strip()[-300:]}"}


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
    footprint = sum(t.numel() * t.element_size() for t in (Q, K, V)) + Q.numel() * esize

    # ---- device-resident: raw forward (inference form: no LSE) -------------------------------
    def step():
        F.span_attention_forward(Q, K, V, R, causal, need_lse=False)

    with ClockSampler(local) as clk:
        ms = time_cuda(step, args.steps, args.warmup, barrier)
    ms = max_over_ranks(ms, device, use_dist)
    ms_step = ms / args.steps
    tokens_step = B * N * world
    value = tokens_step / (ms_step * 1e-3)
    peak, tf_peak, peak_kind = measured_peaks()
    alg = algorithmic_bytes_fwd(B, N, H, D, esize, causal)
    achieved = alg / (ms_step * 1e-3) / 1e9
    traffic = NCU_TRAFFIC_BYTES_PER_BATCH_ELEM * B if args.workload in NCU_TRAFFIC_WORKLOADS else None

    extras = {}
    # ---- the same kernel back to back for >= 2 s, with the SM clock sampled while it runs ------------
    if world == 1 and not args.no_extras:
        per_round = max(1, int(200.0 / ms_step))                      # ~0.2 s of launches between host checks
        with ClockSampler(local, period_s=0.05) as sclk:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t_start, launches = time.perf_counter(), 0
            e0.record()
            while time.perf_counter() - t_start < args.sustained_seconds:
                for _ in range(per_round):
                    step()
                launches += per_round
                torch.cuda.synchronize()
            e1.record()
            torch.cuda.synchronize()
        sms = e0.elapsed_time(e1) / launches
        extras["fwd_sustained"] = {"seconds": e0.elapsed_time(e1) / 1e3, "launches": launches, "ms": sms,
                                   "tokens_per_s": B * N / (sms * 1e-3), "achieved_gbs": alg / (sms * 1e-3) / 1e9,
                                   "frac_of_hbm": alg / (sms * 1e-3) / 1e9 / peak, "clocks": sclk.summary()}

    # ---- end to end through the public API with host buffers -----------------------------------
    out_host = torch.empty((B, N, H, D), dtype=dtype).pin_memory()
    e2e_steps = max(2, min(args.steps, 5))

    def e2e_step():
        # public host-side entry point: pinned inputs in, pinned result out, copies overlapped with compute
        F.hierarchical_attention_from_host(Qh, Kh, Vh, R, causal, out=out_host, device=device)

    e2e_ms = max_over_ranks(time_cuda(e2e_step, e2e_steps, 1, barrier), device, use_dist)
    e2e_value = tokens_step / (e2e_ms / e2e_steps * 1e-3)
    h2d = F.host_entry_h2d_bytes(B, N, H, D, esize, causal)
    d2h = out_host.numel() * out_host.element_size()

    # ---- extras: backward and parent build on the same shape -------------
    launches_per_step = 1
    del Q, K, V
    torch.cuda.empty_cache()
    if rank == 0 and not args.no_extras:
        loops, state = kernel_loops(args.workload, device)
        bsteps = max(3, min(args.steps, 20))
        for key, name in (("bwd", "span_bwd"), ("parents", "parent_build_fwd_all_levels"),
                          ("parents_bwd", "parent_build_bwd_all_levels")):
            fn, kalg, launches = loops[key]
            kms = time_cuda(fn, bsteps, 3, lambda: None) / bsteps
            extras[name] = {"ms": kms, "launches": launches, "achieved_gbs": kalg / (kms * 1e-3) / 1e9,
                            "frac_of_hbm": kalg / (kms * 1e-3) / 1e9 / peak}
            if key == "bwd":
                extras[name]["tokens_per_s"] = B * N / (kms * 1e-3)
        state.clear()
        del loops
        torch.cuda.empty_cache()
        if world == 1:
            extras["parent_tree"] = parent_tree_table(device, bsteps)
            table = gemm_table(device, 10)
            extras["tcgen05_products"] = {
                "note": "the dense products of one LM step (32768 tokens) on the library's tcgen05 kernel; TFLOP/s, and the "
                        "vendor library (torch.matmul) on the same shapes beside it",
                "products": [{"product": r["product"], "M": r["M"], "N": r["N"], "K": r["K"],
                              **{k: {"ours_tflops": round(r[k]["ours_tflops"], 1), "library_tflops": round(r[k]["library_tflops"], 1),
                                     "frac_of_sustained_peak": round(r[k]["frac_of_sustained_peak"], 3)} for k in ("fwd", "dx", "dw")}}
                             for r in table]}
            torch.cuda.empty_cache()

    # ---- the model that calls the layer: data-parallel LM training step (all ranks) ---------------
    if not args.no_lm:
        lm = run_lm(args, device, world, rank, barrier, use_dist, args.lm)
        extras["lm_train"] = lm
        if world > 1:
            # the same step on the same ranks without the collective: the difference is what the all-reduce
            # adds to the step after overlap with the backward
            quiet = run_lm(args, device, world, rank, barrier, use_dist, args.lm, allreduce=False)
            lm["ms_per_step_without_allreduce"] = quiet["ms_per_step"]
            lm["allreduce_exposed_ms"] = lm["ms_per_step"] - quiet["ms_per_step"]
            if LM_CONFIGS[args.lm]["batch"] % world == 0:
                # secondary line: the same global batch as one GPU, split over the ranks
                extras["lm_train_strong"] = run_lm(args, device, world, rank, barrier, use_dist, args.lm, strong=True)
        if world == 1:
            # the same step with the decoder layers and the head run op by op (library products, separate element-wise
            # kernels), i.e. without the fused nodes: what they buy
            eager = run_lm(args, device, world, rank, barrier, use_dist, args.lm, fused=False)
            lm["ms_per_step_unfused"] = eager["ms_per_step"]
        other = "lm_8x2048" if args.lm != "lm_8x2048" else "lm_8x4096"
        extras["lm_train_" + other[3:]] = run_lm(args, device, world, rank, barrier, use_dist, other)
        extras["lm_scaling"] = {"n_gpus": world, "tokens_per_s": lm["tokens_per_s"], "ms_per_step": lm["ms_per_step"],
                                "allreduce_exposed_ms": lm.get("allreduce_exposed_ms", 0.0),
                                "frac_of_tensor_roofline": lm["roofline"]["frac"]}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        v, n, s = oracle_tokens_per_s(args.workload, args.cpu_seconds, cores)
        cpu = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"{n} leaves x {H} heads of one batch entry, {s:.1f} s "
                         f"(eager PyTorch CPU oracle, {cores} threads)"}
    if rank == 0 and world == 1 and not args.no_extras and not args.no_reference_triton:
        extras["reference_triton"] = reference_triton_parent(args)

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
                         "achieved_kind": "effective bandwidth: algorithmic bytes / kernel time",
                         "traffic": traffic,
                         "frac_dram": None if traffic is None else traffic / (ms_step * 1e-3) / 1e9 / peak,
                         "traffic_source": "ncu dram bytes of span_fwd_tc128_kernel at batch 4, scaled by batch",
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
    """Forward-only bf16 sweep over N and batch (H=16, D=128, causal, radius 16 and 32).
    Prints a markdown table: achieved algorithmic GB/s and fraction of the measured HBM copy bandwidth.  `ms` is the
    device time per launch, the smaller of two measurements: inside a replayed CUDA graph of 20 launches (what a captured
    model step sees) and issued from Python one by one (the last column), which for the small cases is bound by the host
    (about 30 us per call through ctypes), not by the kernel."""
    from sparseattention_b200.ops import functional as F
    torch.cuda.set_device(0)
    peak, _, kind = measured_peaks()
    H, D = 16, 128
    print(f"| N | B | radius | ms | tokens/s | GB/s (algorithmic) | of {kind} {peak:.0f} GB/s | footprint MB | eager call ms |")
    print("|---|---|---|---|---|---|---|---|---|")
    side = torch.cuda.Stream()
    for N in (1024, 2048, 4096, 8192, 16384, 32768):
        for B in (1, 8, 32):
            if 6 * B * N * H * D * 2 > 40e9:
                continue
            gen = torch.Generator(device="cuda").manual_seed(N + B)
            Q = torch.randn(B, N, H, D, generator=gen, device="cuda", dtype=torch.bfloat16)
            K = torch.randn(B, 2 * N - 1, H, D, generator=gen, device="cuda", dtype=torch.bfloat16)
            V = torch.randn(B, 2 * N - 1, H, D, generator=gen, device="cuda", dtype=torch.bfloat16)
            for R in (16, 32):
                call = lambda: F.span_attention_forward(Q, K, V, R, True, need_lse=False)   # noqa: E731
                eager = time_cuda(call, 30, 5, lambda: None) / 30
                per_graph = 20
                graph = torch.cuda.CUDAGraph()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    call()
                    torch.cuda.synchronize()
                    with torch.cuda.graph(graph):
                        for _ in range(per_graph):
                            out = call()
                torch.cuda.current_stream().wait_stream(side)
                reps = max(2, min(10, int(400 / (eager * per_graph + 1e-3))))
                ms_graph = time_cuda(graph.replay, reps, 2, lambda: None) / reps / per_graph
                del graph, out
                ms = min(ms_graph, eager)             # long launches: the two agree; the shorter one ran at the higher clock
                alg = algorithmic_bytes_fwd(B, N, H, D, 2, True)
                gbs = alg / (ms * 1e-3) / 1e9
                foot = 6 * B * N * H * D * 2 / 1e6
                print(f"| {N} | {B} | {R} | {ms:.4f} | {B * N / (ms * 1e-3):.3e} | {gbs:.0f} | {gbs / peak:.3f} | {foot:.0f} | {eager:.4f} |")
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
    ap.add_argument("--only", default=None, choices=["fwd", "bwd", "parents", "parents_bwd", "lm", "reference_triton", "gemm", "parent_tree"],
                    help="run one kernel loop (or the LM step, or the reference's Triton package) and print a short JSON line")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--sustained-seconds", type=float, default=2.5)
    ap.add_argument("--reference-triton-seconds", type=int, default=420)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-lm", action="store_true")
    ap.add_argument("--no-reference-triton", action="store_true")
    ap.add_argument("--no-cuda-graph", action="store_true", help="launch the LM step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--lm", default="lm_8x4096", choices=sorted(LM_CONFIGS))
    ap.add_argument("--lm-eager", action="store_true", help="with --only lm: layers and head op by op (library products) instead of the fused nodes")
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
    if args.only is not None:
        run_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
