"""Benchmark of the alpha-entmax attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0).  A "step" is one forward + backward of alpha-entmax attention over
one batch of seeded synthetic input.  Metric: dense-equivalent TFLOP/s,
F = 3.5 * 4 * H * D * sum_b L_b^2 * c  (c = 0.5 causal), no credit for tau iterations or recompute.

  value      inputs resident in HBM, K steps between CUDA events, max over ranks
  e2e        the same step through the operator API from pinned HOST buffers: every step copies
             q, k, v, dO host->device and out, dq, dk, dv device->host inside the timed region
  roofline   the step against the measured bf16 tensor peak (MEASURED_PEAKS.json); `kernels` holds the
             duration every library kernel clocked for itself (GPU global timer, first CTA start to last
             CTA end) and names the dominant one
  cpu_baseline  the dense PyTorch CPU path (oracle port: scores -> 10-step bisection entmax -> PV,
             Jacobian backward) timed on the host cores on one (batch, head) pair of the same workload,
             rank 0, N=1 only; `config1` beside it is BASELINE.json's CPU configuration timed exactly

Multi-GPU: one process per GPU (torchrun), every rank runs the per-GPU workload on its own
(batch, head) shard; there is no collective on the data path ("weak" scaling).
--impl reference times the reference's dense CPU path (the oracle port) instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, H, L, D, alpha, causal)
    "headline": (8, 32, 8192, 128, 1.5, True),     # the shape the metric is quoted on (L=8K, alpha=1.5)
    "config2": (8, 16, 4096, 64, 1.5, True),
    "mid": (2, 16, 4096, 128, 1.5, True),          # profiling case: 4 x 32 MiB of inputs, kernels of a few ms
    "config3": (16, 16, 8192, 128, 2.0, False),    # varlen U[512, 8192], non-causal, alpha = 2
    "config5": (8, 32, 32768, 128, 1.5, True),     # long context (alpha also 1.333 / 2.0 via --alpha)
    "lazy": (4, 32, 16384, 128, None, True),       # Lazy Attention: RoPE'd q,k, bias [H,512] ~ N(0,0.02), tau = -1, W = 512
    "lazy_mid": (2, 16, 4096, 128, None, True),
    "small": (2, 8, 2048, 128, 1.5, True),
    "tiny": (1, 4, 1024, 128, 1.5, True),
}
METRIC = "entmax-attn fwd+bwd TFLOP/s (dense-equiv) & % bf16 tensor peak, L=8K alpha=1.5"


def flops_fwd(B, H, L, D, causal):
    return 4.0 * H * D * B * float(L) * L * (0.5 if causal else 1.0)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id: str):
        # nvidia-smi orders GPUs by PCI bus and ignores CUDA_VISIBLE_DEVICES: select by UUID
        self.index, self.rows, self.stamps, self.proc, self.note = gpu_id, [], [], None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6 and parts[0].isdigit():
                self.rows.append(parts)
                self.stamps.append(time.monotonic())

    def window(self, t0, t1):
        """Keep the samples read between t0 and t1 (host monotonic seconds); returns how many there are."""
        keep = [i for i, t in enumerate(self.stamps[:len(self.rows)]) if t0 <= t <= t1]
        self.rows = [self.rows[i] for i in keep]
        self.stamps = [self.stamps[i] for i in keep]
        return len(self.rows)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"], "gpu": self.index}
        sm = [int(r[0]) for r in self.rows]
        busy = [x for x in sm if x > 0.5 * max(sm)] or sm
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        out = {"sm_mhz": statistics.median(busy), "sm_max_mhz": int(self.rows[0][1]), "reasons": reasons,
               "samples": len(sm), "gpu": self.index}
        if self.note:
            out["sampled"] = self.note
        return out


def cpu_reference(L, D, alpha, causal, steps, warmup, threads=None, B=1, H=1, median=False):
    """Times the dense CPU path on [B,H,L,D] fp32 (default: one (batch, head) pair) per step; returns
    (dense-equivalent TFLOP/s, seconds per step, threads)."""
    import torch
    from oracle import cpu_reference_fwd_bwd
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    q, k, v, do = (torch.randn(B, H, L, D, generator=g) for _ in range(4))
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        cpu_reference_fwd_bwd(q, k, v, do, alpha=alpha, is_causal=causal, n_iter=10)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = statistics.median(times) if median else sum(times) / len(times)
    return 3.5 * flops_fwd(B, H, L, D, causal) / sec / 1e12, sec, threads


def cpu_config1():
    """BASELINE.json's CPU configuration, exactly: B=1 H=8 L=128 D=64 fp32, causal, alpha=1.5, bisection
    n_iter=10, forward + backward w.r.t. q, k, v; 3 warm-ups, median of 50."""
    tf, sec, threads = cpu_reference(128, 64, 1.5, True, 50, 3, B=1, H=8, median=True)
    return {"workload": "B=1 H=8 L=128 D=64 fp32 causal alpha=1.5 bisection n_iter=10, fwd+bwd", "ms": sec * 1e3,
            "gflops": tf * 1e3, "cores": threads, "statistic": "median of 50 after 3 warm-ups"}


def run_reference(args):
    """The reference arm: the dense CPU path (oracle port; the reference's own entmax kernels are not in its
    checkout) on the host cores.  Every step is ONE (batch, head) pair of the workload at its full length;
    exactly --warmup untimed and --steps timed steps are run."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    B, H, L, D, alpha, causal = WORKLOADS[args.workload]
    alpha = 1.5 if alpha is None else alpha
    Ls = min(L, args.cpu_len)
    tf, sec, threads = cpu_reference(Ls, D, alpha, causal, args.steps, args.warmup)
    sample = (f"1 of {B * H} (batch, head) pairs per step at L={Ls}, fp32, dense bisection n_iter=10 + Jacobian backward; "
              f"{args.warmup} warm-up and {args.steps} timed steps")
    line = {"metric": METRIC, "impl": "reference", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: B={B} H={H} L={L} D={D} alpha={alpha} causal={causal}",
                       "reference_arm": "dense PyTorch CPU path (oracle port)"},
            "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def rows_table(steps, warmup):
    """Stand-alone entmax over rows (the HBM-bound operator of the path): achieved bandwidth per shape, one JSON
    line each.  Algorithmic bytes: forward rows x cols x (in + out), backward rows x cols x 3."""
    import torch

    import flash_lazy_attention_b200 as fla
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = 6650.0   # fallback: an earlier copy-bandwidth measurement on the same pool
    if os.path.exists(path):
        with open(path) as fh:
            peak = float(json.load(fh).get("hbm_gbs", peak))

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    for dtype, name in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        for rows, cols in ((1 << 19, 256), (1 << 17, 1024), (1 << 16, 4096), (1 << 14, 16384), (1 << 12, 65536)):
            x = torch.randn(rows, cols, device="cuda", dtype=dtype).requires_grad_(True)
            dy = torch.randn(rows, cols, device="cuda", dtype=dtype)
            y = fla.triton_entmax(x, 1.5, 10)
            ms_f = timed(lambda: fla.triton_entmax(x, 1.5, 10))

            def bwd():
                x.grad = None
                y.backward(dy, retain_graph=True)
            ms_b = timed(bwd)
            nb = rows * cols * x.element_size()
            print(json.dumps({"op": "entmax_rows", "dtype": name, "rows": rows, "cols": cols,
                              "fwd_ms": round(ms_f, 4), "fwd_gbs": round(2 * nb / ms_f / 1e6, 1),
                              "bwd_ms": round(ms_b, 4), "bwd_gbs": round(3 * nb / ms_b / 1e6, 1),
                              "peak_gbs": peak}), flush=True)
            del x, dy, y
    # rotary embedding of q and k in one launch (the step before attention in the layers): read + write of both
    for B, L, H, Hk, D in ((8, 8192, 32, 32, 128), (4, 16384, 32, 8, 128), (8, 4096, 16, 16, 64)):
        q = torch.randn(B, L, H, D, device="cuda", dtype=torch.bfloat16).transpose(1, 2)    # b l h d storage
        k = torch.randn(B, L, Hk, D, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
        ms = timed(lambda: fla.rope_qk(q, k, 10000.0, 0))
        nb = 2 * (q.numel() + k.numel()) * q.element_size()
        print(json.dumps({"op": "rope_qk", "dtype": "bf16", "B": B, "L": L, "H": H, "Hkv": Hk, "D": D,
                          "ms": round(ms, 4), "gbs": round(nb / ms / 1e6, 1), "peak_gbs": peak}), flush=True)
        del q, k


def lazy_compare(steps, warmup):
    """Same-box comparator for the Lazy Attention path: the reference's own Triton module, JIT-compiled for this
    GPU (oracle/_ref/lazy_attention_triton.py, put there by oracle/make_ref.py), against this library on the same
    bf16 inputs: forward + backward time with frozen and with trained bias / tau, and the largest difference
    between the two implementations' outputs and gradients.  One JSON line per case."""
    import torch

    import flash_lazy_attention_b200 as fla
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "lazy_attention_triton.py")):
        print(json.dumps({"lazy_compare": "unavailable", "why": "oracle/_ref/lazy_attention_triton.py is missing: "
                          "run `python oracle/make_ref.py <reference checkout>` first"}), flush=True)
        return
    sys.path.insert(0, ref_dir)
    try:
        import lazy_attention_triton as ref_mod
    except Exception as exc:   # Triton missing or unusable on this box
        print(json.dumps({"lazy_compare": "unavailable", "why": f"{type(exc).__name__}: {exc}"}), flush=True)
        return
    dev = torch.device("cuda", 0)

    def rope(x):
        L, D = x.shape[-2], x.shape[-1]
        half = D // 2
        inv = 1.0 / (10000.0 ** (torch.arange(half, device=dev, dtype=torch.float32) / half))
        ang = torch.arange(L, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
        return x * cos + torch.cat([-x[..., half:], x[..., :half]], -1) * sin

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    for name, (B, H, L, D, W) in (("B2 H8 L4096 D128 W512", (2, 8, 4096, 128, 512)),
                                  ("config 4: B4 H32 L16384 D128 W512", (4, 32, 16384, 128, 512))):
        gen = torch.Generator(device=dev).manual_seed(0)
        q, k = (rope(torch.randn(B, H, L, D, generator=gen, device=dev)).to(torch.bfloat16) for _ in range(2))
        v, do = (torch.randn(B, H, L, D, generator=gen, device=dev).to(torch.bfloat16) for _ in range(2))
        bias = torch.randn(H, W, generator=gen, device=dev) * 0.02
        tau = torch.full((H,), -1.0, device=dev)
        F = 3.5 * flops_fwd(B, H, L, D, True)
        for trained in (False, True):
            def run(fn):
                leaves = [t.detach().clone().requires_grad_(True) for t in (q, k, v)]
                bp, tp = bias.clone().requires_grad_(trained), tau.clone().requires_grad_(trained)
                out = fn(*leaves, bp.to(torch.bfloat16), tp.to(torch.bfloat16), window_size=W)
                out.backward(do)
                return [out.detach()] + [t.grad for t in leaves] + ([bp.grad, tp.grad] if trained else [])
            line = {"lazy_compare": name, "trained_params": trained}
            try:
                ref_ms = timed(lambda: run(ref_mod.lazy_attention_triton))
                ref_res = run(ref_mod.lazy_attention_triton)
                line.update({"reference_triton_ms": ref_ms, "reference_triton_tflops": F / ref_ms / 1e9})
            except Exception as exc:
                ref_res = None
                line["reference_triton"] = f"failed: {type(exc).__name__}: {str(exc)[:200]}"
            ours_ms = timed(lambda: run(fla.lazy_attention_triton))
            ours = run(fla.lazy_attention_triton)
            line.update({"ours_ms": ours_ms, "ours_tflops": F / ours_ms / 1e9})
            if ref_res is not None:
                line["speedup"] = ref_ms / ours_ms
                names = ["out", "dq", "dk", "dv", "dbias", "dtau"][:len(ours)]
                line["max_abs_diff"] = {n: float((a.float() - b.float()).abs().max()) for n, a, b in zip(names, ours, ref_res)}
                line["max_abs_ref"] = {n: float(b.float().abs().max()) for n, b in zip(names, ref_res)}
            print(json.dumps(line), flush=True)
            del ours, ref_res
        del q, k, v, do
        torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="headline", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-len", type=int, default=8192, help="longest row of the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--alpha", type=float, default=None, help="override the workload's alpha")
    ap.add_argument("--frozen", action="store_true", help="lazy workloads: bias/tau without gradients")
    ap.add_argument("--clusters", type=int, default=0,
                    help="entmax workloads: q, k drawn around this many well separated centres in contiguous "
                         "segments of --seg tokens, so that most (query block, key block) pairs are empty")
    ap.add_argument("--seg", type=int, default=512, help="segment length of --clusters")
    ap.add_argument("--flags", type=int, default=0,
                    help="fla_attn_geom.flags for the run (include/fla.h: 1 thresholds by passes over recomputed scores, "
                         "4 by candidates kept in the row-max pass; 0 = the library's choice)")
    ap.add_argument("--niter", type=int, default=10,
                    help="entmax workloads: cap on the threshold iterations (the metric is defined at the default, 10; "
                         "0, 1, 2 ... time the forward with that many threshold passes and leave the thresholds "
                         "unconverged: for the per-pass breakdown under profiles/ only)")
    ap.add_argument("--partition", action="store_true",
                    help="strong scaling: ONE seeded problem of the workload's size, its (batch, head) pairs split over "
                         "the ranks (no collective in the timed region); afterwards the ranks' results are gathered "
                         "over NCCL and rank 0 checks them bit for bit against its own unsharded run")
    ap.add_argument("--lazy-compare", action="store_true",
                    help="instead of the attention step: Lazy Attention of this library against the reference's Triton "
                         "module on the same GPU (needs oracle/_ref, see oracle/make_ref.py)")
    ap.add_argument("--rows-table", action="store_true",
                    help="instead of the attention step: bandwidth of the stand-alone row entmax per shape")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.rows_table:
        rows_table(args.steps, args.warmup)
        return
    if args.lazy_compare:
        lazy_compare(args.steps, args.warmup)
        return

    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    import flash_lazy_attention_b200 as fla
    from flash_lazy_attention_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # stdout carries the one JSON line; NCCL's version banner (NCCL_DEBUG=VERSION) would precede it
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    _lib.check(_lib.load().fla_device_supported(local), "device check")
    fla.set_flags(args.flags)

    B, H, L, D, alpha, causal = WORKLOADS[args.workload]
    if args.alpha is not None and alpha is not None:
        alpha = args.alpha
    is_lazy = alpha is None
    gen = torch.Generator(device=dev).manual_seed(rank)

    def rope(x):  # rotate-half RoPE, base 10000, positions 0..L-1, applied in fp32
        half = D // 2
        inv = 1.0 / (10000.0 ** (torch.arange(half, device=dev, dtype=torch.float32) / half))
        ang = torch.arange(L, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
        rot = torch.cat([-x[..., half:], x[..., :half]], -1)
        return x * cos + rot * sin

    centres = None
    if args.clusters > 0 and not is_lazy:
        centres = torch.nn.functional.normalize(torch.randn(args.clusters, D, generator=gen, device=dev), dim=-1) * 12.0
        centres = centres[(torch.arange(L, device=dev) // args.seg) % args.clusters]

    def make(i):
        x = torch.randn(B, H, L, D, generator=gen, device=dev, dtype=torch.float32)
        if is_lazy and i < 2:
            x = rope(x)
        if centres is not None and i < 2:
            x = centres + 0.3 * x
        return x.to(torch.bfloat16)

    Bg, Hg = B, H                      # the global problem (partition mode shards it)
    pieces = None
    if args.partition:
        if is_lazy or args.workload == "config3" or args.clusters:
            raise SystemExit("--partition: entmax workloads without varlen only")
        from flash_lazy_attention_b200.shard import bh_shard, gather_pairs, take_shard

        def make_pairs(pairs):
            """q, k, v, dO of the given (h, b) pairs, every pair from its own seed: [n, 1, L, D] each."""
            outs = [[], [], [], []]
            for (hh, bb) in pairs:
                gp = torch.Generator(device=dev).manual_seed(100003 * hh + bb + 1)
                for i in range(4):
                    outs[i].append(torch.randn(1, 1, L, D, generator=gp, device=dev, dtype=torch.float32).to(torch.bfloat16))
            return [torch.cat(o, dim=0) for o in outs]

        pieces = bh_shard(Bg, Hg, rank, world)
        q, k, v, do = make_pairs([(hh, bb) for (hh, b0, b1) in pieces for bb in range(b0, b1)])
        B, H = q.shape[0], 1           # this rank's shard: every pair its own batch entry
    else:
        q, k, v, do = (make(i) for i in range(4))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    varlen = None
    if args.workload == "config3":
        varlen = torch.randint(512, 8193, (B,), generator=torch.Generator().manual_seed(0)).to(dev)
    if is_lazy:
        bias = (torch.randn(H, 512, generator=gen, device=dev) * 0.02).requires_grad_(not args.frozen)
        tau_p = torch.full((H,), -1.0, device=dev).requires_grad_(not args.frozen)
    lens = varlen.double().cpu() if varlen is not None else torch.full((B,), float(L), dtype=torch.float64)
    F_fwd = 4.0 * H * D * float((lens * lens).sum()) * (0.5 if causal else 1.0)   # of this rank's work
    F_step = 3.5 * F_fwd
    F_job = 3.5 * flops_fwd(Bg, Hg, L, D, causal) if args.partition else world * F_step

    def forward():
        if is_lazy:
            return fla.lazy_attention_triton(q, k, v, bias.to(q.dtype), tau_p.to(q.dtype), window_size=512)
        return fla.adasplash(q, k, v, alpha=alpha, niter=args.niter, is_causal=causal, varlen=varlen)

    def step():
        q.grad = k.grad = v.grad = None
        if is_lazy:
            bias.grad = tau_p.grad = None
        out = forward()
        out.backward(do)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # the sampler starts before the warm-up (nvidia-smi needs up to a second for its first line on an 8-GPU box);
    # only the samples read during the timed region count
    with ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid)) as clocks:
        for _ in range(args.warmup):
            step()
        barrier()
        fla.read_status(dev, reset=True)
        barrier()
        t_start = time.monotonic()
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        barrier()
        t_end = time.monotonic()
        status = fla.read_status(dev)
        if clocks.window(t_start, t_end + 0.05) < 2:
            # a timed region shorter than two sampling periods: the same steps again, untimed, for the sampler
            clocks.rows, clocks.stamps = [], []
            t_more = time.monotonic()
            while time.monotonic() - t_more < 0.7:
                step()
                torch.cuda.synchronize()
            clocks.window(t_more + 0.1, time.monotonic() + 0.05)
            clocks.note = "the same steps repeated untimed right after the timed region (it was shorter than two samples)"
    ms = ev0.elapsed_time(ev1) / args.steps
    if status["error"]:
        raise RuntimeError(f"a kernel reported an expired wait: {status}")
    path = fla.last_call_info()["path"]
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = F_job / (ms * 1e-3) / 1e12

    # ---- partition mode: gather the shards' results and compare with the unsharded run (outside any timing)
    partition_check = None
    if args.partition:
        mine = [step().detach(), q.grad, k.grad, v.grad]
        gathered = [gather_pairs(t, Bg, Hg) for t in mine] if world > 1 else None      # [Bg, Hg, L, D] on every rank
        if rank == 0:
            diffs = {}
            if world > 1:
                # rank 0 runs the whole problem itself, pair by pair in the same layout as its shards
                worst = 0.0
                identical = True
                chunk = max(1, (Bg * Hg) // world)
                allp = [(hh, bb) for hh in range(Hg) for bb in range(Bg)]
                for c0 in range(0, len(allp), chunk):
                    sub = allp[c0:c0 + chunk]
                    fq, fk, fv, fdo = make_pairs(sub)
                    fq.requires_grad_(True), fk.requires_grad_(True), fv.requires_grad_(True)
                    fo = fla.adasplash(fq, fk, fv, alpha=alpha, niter=args.niter, is_causal=causal)
                    fo.backward(fdo)
                    for name, full, ref in zip(("out", "dq", "dk", "dv"), gathered, (fo.detach(), fq.grad, fk.grad, fv.grad)):
                        got = torch.stack([full[bb, hh] for (hh, bb) in sub]).unsqueeze(1)
                        d = float((got.float() - ref.float()).abs().max())
                        diffs[name] = max(diffs.get(name, 0.0), d)
                        identical = identical and torch.equal(got, ref)
                        worst = max(worst, d)
                partition_check = {"bit_identical": identical, "max_abs_diff": diffs, "pairs": Bg * Hg,
                                   "gathered_with": "NCCL all_gather (outside the timed region)"}
            else:
                partition_check = {"bit_identical": None, "note": "one rank: nothing to gather"}
        del gathered

    # ---- per-kernel and per-phase timing, live ----------------------------------------------------------------
    # Phases: CUDA events between the two halves of whole steps, on the stream the library launches on.
    # Kernels: every tensor-core kernel writes the global-timer time of its first CTA's start and its last
    # CTA's end into the status words (one launch of each per step between two clears), so the three
    # durations come from the same steps, without a profiler.
    reps = max(3, min(args.steps, 10))
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(reps)]
    per_kernel = {"fwd": [], "dq": [], "dkdv": []}
    cta_ms = {"fwd": [], "dq": [], "dkdv": []}
    n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
    torch.cuda.synchronize()
    for ev in marks:
        q.grad = k.grad = v.grad = None
        fla.read_status(dev, reset=True)
        ev[0].record()
        out = forward()
        ev[1].record()
        out.backward(do)
        ev[2].record()
        torch.cuda.synchronize()
        st_now = fla.read_status(dev)
        for name, val in st_now["kernel_ms"].items():
            if val is not None:
                per_kernel[name].append(val)
                cta_ms[name].append(st_now["cta_ms"][name])
    fwd_ms = sum(ev[0].elapsed_time(ev[1]) for ev in marks) / reps
    bwd_ms = sum(ev[1].elapsed_time(ev[2]) for ev in marks) / reps
    peak, peak_sustained, peak_kind = measured_peaks()
    executed = status["tile_mmas"] * 2.0 * 128 * 128 * D / max(args.steps, 1)
    # Credit per kernel in units of one masked L x L x D contraction (F_fwd / 2): the forward computes S and P.V
    # (2); the backward is credited 5 (S, dP, dV, dK, dQ), of which S and dP are needed once for both of its
    # kernels and are split evenly: dQ kernel 1 + 1, dK/dV kernel 2 + 1.
    unit = F_fwd / 2.0
    credit = {"fwd": 2.0, "dq": 2.0, "dkdv": 3.0}
    labels = {"fwd": "forward kernel (row max, row thresholds, S, P.V)", "dq": "dQ kernel (delta sweep, S, dP, dQ)",
              "dkdv": "dK/dV kernel (S^T, dP^T, dV, dK)"}
    traffic_file = os.path.join(ROOT, "profiles", "dram_traffic.json")
    traffic_tab = {}
    if os.path.exists(traffic_file):
        with open(traffic_file) as fh:
            traffic_tab = json.load(fh)
    kernels = {}
    for name, vals in per_kernel.items():
        if not vals:
            continue
        kms = statistics.median(vals)
        ktf = credit[name] * unit / (kms * 1e-3) / 1e12
        # share of the launch during which the SMs held a CTA of the kernel (one CTA per SM): what is missing
        # from 1 is dispatch gaps between CTAs plus the tail of the grid, the most a persistent scheduler could win
        busy = statistics.median(c / (n_sm * m) for c, m in zip(cta_ms[name], vals))
        kernels[name] = {"what": labels[name], "ms": kms, "credited_units": credit[name], "tflops": ktf,
                         "frac": ktf / peak_sustained, "sm_occupied_frac": busy}
        # DRAM bytes per launch: an ncu capture of a smaller workload of the same kernel, scaled by the number of
        # (batch, head, row) units (the (batch, head)-major grid keeps shared tiles in L2, so traffic follows the
        # tensor sizes); entmax kernels at D = 128 without varlen only
        t = traffic_tab.get("kernels", {}).get(name)
        if t and not is_lazy and D == 128 and varlen is None:
            kernels[name]["traffic"] = (t["dram_read_bytes"] + t["dram_write_bytes"]) * (B * H * L) / float(traffic_tab["units"])
    dom = max(kernels, key=lambda n: kernels[n]["ms"]) if kernels else None
    roofline = {"bound": "tensor", "achieved": value / world, "peak": peak_sustained, "unit": "TFLOP/s",
                "frac": value / world / peak_sustained,
                "traffic": sum(kv.get("traffic", 0.0) for kv in kernels.values()) or None,
                "kernel": "whole step (forward + dQ + dK/dV kernels) per GPU; dominant single kernel: "
                          + (labels[dom] if dom else "n/a"),
                "dominant_kernel": dom, "kernels": kernels, "peak_kind": f"{peak_kind}, sustained",
                "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
                "fwd_tflops": F_fwd / (fwd_ms * 1e-3) / 1e12, "bwd_tflops": 2.5 * F_fwd / (bwd_ms * 1e-3) / 1e12,
                "executed_tflops": executed / (ms * 1e-3) / 1e12 if executed else None,
                "executed_units_per_step": executed / unit if executed else None,
                "list_ctas": status.get("list_ctas"), "pass_ctas": status.get("pass_ctas"),
                "frac_of_burst_peak": value / world / peak, "frac_of_nominal_2250": value / world / 2250.0}

    # ---- end to end from pinned host buffers -------------------------------------------------------
    e2e = None
    e2e_ready = not args.no_e2e
    if e2e_ready:
        # 8 pinned host buffers and 4 device buffers of the size of q; if any rank cannot get them, every
        # rank skips the end-to-end leg (the ranks meet in barriers inside it)
        try:
            hq, hk, hv, hdo = (t.detach().cpu().pin_memory() for t in (q, k, v, do))
            hout, hdq, hdk, hdv = (torch.empty_like(hq).pin_memory() for _ in range(4))
            dq_, dk_, dv_, ddo_ = (torch.empty_like(do) for _ in range(4))
            alloc_error = None
        except RuntimeError as exc:   # out of (pinned) memory
            alloc_error = str(exc).splitlines()[0]
        flag = torch.tensor([0 if alloc_error else 1], device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            e2e_ready = False
            e2e = {"value": None, "unit": "TFLOP/s", "error": alloc_error or "another rank could not allocate its buffers"}
    if e2e_ready:

        # One step = every batch element's q, k, v, dO copied host->device, forward + backward through the
        # operator API, out, dq, dk, dv copied device->host.  The batch elements are independent, so the step is
        # pipelined over them on three streams: while element b computes, element b+1 is on its way in and
        # element b-1 on its way out (PCIe is full duplex).  Nothing is skipped and nothing is kept on the device
        # between steps; events order the reuse of every device slice.
        s_in, s_comp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        ev_in = [torch.cuda.Event() for _ in range(B)]      # inputs of element b are on the device
        ev_comp = [torch.cuda.Event() for _ in range(B)]    # its forward + backward are done
        ev_out = [torch.cuda.Event() for _ in range(B)]     # its results are on the host
        keep = []                                           # results whose device->host copy may still run
        bias_c = bias.detach().to(q.dtype) if is_lazy else None
        tau_c = tau_p.detach().to(q.dtype) if is_lazy else None
        state = {"first": True}

        def e2e_step():
            cur = torch.cuda.current_stream(dev)
            if state["first"]:
                for st in (s_in, s_comp, s_out):
                    st.wait_stream(cur)
            held = []
            for bi in range(B):
                sl = slice(bi, bi + 1)
                with torch.cuda.stream(s_in):
                    if not state["first"]:
                        s_in.wait_event(ev_comp[bi])      # last step's kernels have read this slice
                    dq_[sl].copy_(hq[sl], non_blocking=True), dk_[sl].copy_(hk[sl], non_blocking=True)
                    dv_[sl].copy_(hv[sl], non_blocking=True), ddo_[sl].copy_(hdo[sl], non_blocking=True)
                    ev_in[bi].record(s_in)
                with torch.cuda.stream(s_comp):
                    s_comp.wait_event(ev_in[bi])
                    a, b_, c = (t[sl].detach().requires_grad_(True) for t in (dq_, dk_, dv_))
                    vl = None if varlen is None else varlen[sl]
                    if is_lazy:
                        o = fla.lazy_attention_triton(a, b_, c, bias_c, tau_c, window_size=512)
                    else:
                        o = fla.adasplash(a, b_, c, alpha=alpha, niter=args.niter, is_causal=causal, varlen=vl)
                    o.backward(ddo_[sl])
                    ev_comp[bi].record(s_comp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_comp[bi])
                    if not state["first"]:
                        pass   # the host slices are rewritten in stream order on s_out
                    res = (o.detach(), a.grad, b_.grad, c.grad)
                    for t in res:
                        t.record_stream(s_out)
                    hout[sl].copy_(res[0], non_blocking=True), hdq[sl].copy_(res[1], non_blocking=True)
                    hdk[sl].copy_(res[2], non_blocking=True), hdv[sl].copy_(res[3], non_blocking=True)
                    ev_out[bi].record(s_out)
                held.append(res)
            keep[:] = held
            state["first"] = False

        def e2e_join():
            cur = torch.cuda.current_stream(dev)
            for st in (s_in, s_comp, s_out):
                cur.wait_stream(st)

        e2e_step()
        e2e_join()
        barrier()
        n_e2e = max(2, min(args.steps, 5))
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        state["first"] = True
        t0.record()
        for _ in range(n_e2e):
            e2e_step()
        e2e_join()
        t1.record()
        barrier()
        e2e_ms = t0.elapsed_time(t1) / n_e2e
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        nbytes = q.numel() * q.element_size()
        # the pipelined step must have produced what the resident step produces (last batch element: out and dq)
        with torch.no_grad():
            chk = max(float((hout[B - 1:].to(dev).float() - out[B - 1:].float()).abs().max()),
                      float((hdq[B - 1:].to(dev).float() - q.grad[B - 1:].float()).abs().max()))
        # The same bytes with no kernel at all: q, k, v, dO host->device on one stream while out, dq, dk, dv go
        # device->host on another (one cudaMemcpyAsync per tensor): the ceiling the host side allows this rank
        # while all ranks copy at the same time.
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(n_e2e):
            with torch.cuda.stream(s_in):
                dq_.copy_(hq, non_blocking=True), dk_.copy_(hk, non_blocking=True)
                dv_.copy_(hv, non_blocking=True), ddo_.copy_(hdo, non_blocking=True)
            with torch.cuda.stream(s_out):
                hout.copy_(do, non_blocking=True), hdq.copy_(do, non_blocking=True)
                hdk.copy_(do, non_blocking=True), hdv.copy_(do, non_blocking=True)
        e2e_join()
        c1.record()
        barrier()
        copy_ms = c0.elapsed_time(c1) / n_e2e
        if world > 1:
            t = torch.tensor([copy_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            copy_ms = float(t.item())
        e2e = {"value": F_job / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 4 * nbytes, "d2h_bytes_per_step": 4 * nbytes,
               "pipeline": f"{B} batch elements on three streams (copy in / compute / copy out)",
               "copies_only_ms_per_step": copy_ms, "fraction_of_copies_only": copy_ms / e2e_ms,
               "max_abs_diff_vs_resident_step": chk}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        Ls = min(L, args.cpu_len)
        tf, sec, threads = cpu_reference(Ls, D, alpha if alpha is not None else 1.5, causal, 3, 1)
        cpu = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "seconds_per_pair": sec,
               "sample": f"1 of {B * H} (batch, head) pairs at L={Ls} (dense fp32, bisection n_iter=10 + Jacobian backward), "
                         "mean of 3 after 1 warm-up",
               "config1": cpu_config1()}

    sparsity = None
    if centres is not None:
        # share of (128-row, 64-key) blocks the forward found non-empty, and the share of 128 x 128 tile
        # products the kernels issued against the dense count
        with torch.no_grad():
            mask = fla.entmax_attention_forward(q[:1], k[:1], v[:1], alpha, 10, causal, None, use_block_mask=True)[-1]
        blocks = fla.unpack_block_mask(mask, L)
        tr, tc_ = blocks.shape[-2], blocks.shape[-1]   # 128-row query blocks x 64-key blocks
        dense_blocks = tr * (tr + 1) if causal else tr * tc_
        sparsity = {"clusters": args.clusters, "seg": args.seg,
                    "nonempty_block_share": float(blocks.float().sum(dim=(-1, -2)).mean()) / dense_blocks}

    if rank == 0:
        # library kernels per step: forward, dQ, dK/dV (tensor-core family); the SIMT family adds the delta pre-pass
        # forward, dQ, dK/dV (the SIMT family adds its row pre-pass; a Lazy backward with trained bias and tau ends
        # with the small kernel that converts the fixed-point dbias / dtau sums)
        launches_per_step = {"tcgen05": 3, "simt": 4}.get(path, 3) + (1 if is_lazy and not args.frozen else 0)
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "strong" if args.partition else "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": (f"{args.workload}: B={Bg} H={Hg} L={L} D={D} alpha={alpha} niter={args.niter} causal={causal} "
                                        + ("in total, its (batch, head) pairs split over the GPUs" if args.partition else "per GPU")
                                        + ", fwd+bwd, seeded N(0,1) q,k,v,dO"),
                           "partition_check": partition_check,
                           "inputs": sparsity or "unstructured",
                           "kernel_family": path, "l2": "inputs larger than L2 (4 x %d MiB)" % (q.numel() * 2 >> 20),
                           "parallelism": f"(batch, head) shards on {world} GPU(s), no data-path collective"},
                "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
                "roofline": roofline, "cpu_baseline": cpu}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
