"""Benchmark of the gated-delta-rule chunked prefill on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c1_fwd|c3_fwdbwd|...] [--scaling weak|strong]

One "step" is one pass of the hot path over one synthetic batch.  Default workload: the fixed
length forward prefill B=4, T=8192, H_q=H_v=16, K=V=128 (bf16 inputs, fp32 gates) on every GPU.
Rank 0 prints one JSON line.  Under torchrun every rank runs its own shard, all ranks meet at a
barrier on both sides of the timed region and the slowest rank's device time is used.

``--impl reference`` times the CPU implementation of the same operator (the PyTorch port of the
reference's ``tests/ref_gdr.py`` algorithm in ``oracle/``; the reference's TileLang kernels are
Python that needs its own package name and a JIT, and do not travel with this repository) on a
bounded sample of the workload using all host threads.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Algorithmic work per (token, value head) at K=V=128, chunk 64 (2 FLOP per multiply-add).
FWD_FLOP = 163_840
FWDBWD_FLOP = 655_360

WORKLOADS = {
    # name: dict(B, T, Hq, Hv, mode, varlen)
    "c1_fwd": dict(B=4, T=8192, Hq=16, Hv=16, mode="fwd", varlen=None, h0=False),
    "c1_fwdbwd": dict(B=4, T=8192, Hq=16, Hv=16, mode="fwdbwd", varlen=None, h0=False),
    "c2_fwd": dict(B=1, T=None, Hq=8, Hv=8, mode="fwd", varlen="uniform64", h0=True),
    "c3_fwdbwd": dict(B=1, T=32768, Hq=16, Hv=32, mode="fwdbwd", varlen="lognormal", h0=True),
    "c4_fwdbwd": dict(B=1, T=262144, Hq=8, Hv=8, mode="fwdbwd", varlen=None, h0=False),
    "c4_fwd": dict(B=1, T=262144, Hq=8, Hv=8, mode="fwd", varlen=None, h0=False),
    # a quarter of c1 (one sequence): small enough for a full ncu capture, inputs still > L2
    "c1_quarter_fwd": dict(B=1, T=8192, Hq=16, Hv=16, mode="fwd", varlen=None, h0=False),
    "c1_quarter_fwdbwd": dict(B=1, T=8192, Hq=16, Hv=16, mode="fwdbwd", varlen=None, h0=False),
}


def make_lengths(kind: str, seed: int, total: int | None):
    gen = torch.Generator().manual_seed(seed)
    if kind == "uniform64":
        lens = torch.randint(128, 4097, (64,), generator=gen).tolist()
    elif kind == "lognormal":
        lens, acc = [], 0
        while acc < total:
            n = int(torch.exp(torch.randn((), generator=gen) + 6.931471805599453).item())
            n = min(max(n, 64), 8192, total - acc)
            lens.append(n)
            acc += n
    else:
        raise ValueError(kind)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    return cu


def make_batch(w, device, seed, heads_q=None, heads_v=None, batch=None):
    """Seeded synthetic inputs with the benchmark configuration's shapes and distributions."""
    Hq, Hv = heads_q or w["Hq"], heads_v or w["Hv"]
    cu = None
    B, T = batch or w["B"], w["T"]
    if w["varlen"]:
        cu = make_lengths(w["varlen"], seed, w["T"])
        B, T = 1, cu[-1]
    gen = torch.Generator(device=device).manual_seed(seed)

    def rn(*s):
        return torch.randn(*s, device=device, generator=gen, dtype=torch.float32)

    q = torch.nn.functional.normalize(rn(B, T, Hq, 128), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(rn(B, T, Hq, 128), dim=-1).bfloat16()
    v = rn(B, T, Hv, 128).bfloat16()
    g = torch.nn.functional.logsigmoid(rn(B, T, Hv))
    beta = torch.sigmoid(rn(B, T, Hv)).bfloat16()
    N = B if cu is None else len(cu) - 1
    h0 = 0.1 * rn(N, Hv, 128, 128) if w["h0"] else None
    do = rn(B, T, Hv, 128).bfloat16()
    dht = 0.1 * rn(N, Hv, 128, 128)
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32, device=device)
    return dict(q=q, k=k, v=v, g=g, beta=beta, h0=h0, do=do, dht=dht, cu=cu_t, tokens=B * T,
                Hv=Hv, Hq=Hq)


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=fd, stderr=subprocess.DEVNULL)
            os.close(fd)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons))
        return out


def run_ours(args):
    import torch.distributed as dist

    import flashqla_b200 as fq
    from flashqla_b200 import _lib, cp, ops

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = WORKLOADS[args.workload]
    tshard = False
    if args.scaling == "strong" and world > 1:
        if w["B"] == 1 and not w["varlen"]:
            # one long sequence: shard along T, boundary states handed over by one all-gather
            tshard = True
            w_loc = dict(w, T=w["T"] // world)
            x = make_batch(w_loc, dev, 1234 + rank)
            x["h0"] = None
        else:
            # shard by value head (and the matching q/k heads): no communication
            hv = max(w["Hv"] // world, 1)
            hq = max(w["Hq"] // world, 1)
            x = make_batch(w, dev, 1234 + rank, heads_q=hq, heads_v=hv)
    else:
        x = make_batch(w, dev, 1234 + rank)
    tokens = x["tokens"]
    bwd = w["mode"] == "fwdbwd"

    def step(inp):
        if tshard:
            from flashqla_b200 import distributed as fd

            g_cum, A, o, ht, saved = fd.fwd_tsharded(inp["q"], inp["k"], inp["v"], inp["g"],
                                                     inp["beta"], None, None)
            if not bwd:
                return o, ht
            grads = fd.bwd_tsharded(inp["q"], inp["k"], inp["v"], g_cum, inp["beta"], A,
                                    inp["do"], inp["dht"], None, saved)
            return (o, ht) + tuple(grads)
        g_cum, A, o, _, ht, cache = fq.chunk_gated_delta_rule_fwd(
            inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], None, inp["h0"], inp["cu"],
            output_final_state=True, enable_fwd_cp_cache=bwd)
        if not bwd:
            return o, ht
        grads = fq.chunk_gated_delta_rule_bwd(
            inp["q"], inp["k"], inp["v"], g_cum, inp["beta"], A, inp["do"], inp["dht"], None,
            inp["h0"], inp["cu"], cp_cache=cache)
        return (o, ht) + tuple(t for t in grads if t is not None)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    with ClockSampler(local) as clocks:
        for _ in range(max(args.warmup, 3)):
            step(x)
        if not args.kernel_only:
            # keep the GPU under the same load until the clock sampler has come up
            torch.cuda.synchronize()
            t_up = time.time() + 0.6
            while time.time() < t_up:
                step(x)
                torch.cuda.synchronize()
        launches0 = _lib.launch_count
        ms = timed(lambda: step(x), args.steps)
        launches = _lib.launch_count - launches0
        if not args.kernel_only:
            t_up = time.time() + 0.3  # a few more samples under load after the timed steps
            while time.time() < t_up:
                step(x)
                torch.cuda.synchronize()
    ms_per_step = ms / args.steps
    value = tokens * world / (ms_per_step * 1e-3)

    # ---- end to end: pinned host inputs -> device, operator, result back to host
    names = ["q", "k", "v", "g", "beta"] + (["do", "dht"] if bwd else []) + \
            (["h0"] if x["h0"] is not None else [])
    host = {n: x[n].cpu().pin_memory() for n in names}
    dev_in = {n: torch.empty_like(x[n]) for n in names}
    outs = step(x)
    host_out = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in outs]
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    # A fixed-length batch is fed sequence by sequence: the copy-in of sequence b+1 and the
    # copy-out of sequence b-1 overlap the kernels of sequence b (PCIe is full duplex).
    n_slices = x["q"].shape[0] if (x["cu"] is None and not tshard and x["q"].shape[0] > 1) else 1
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def e2e_step():
        cur = torch.cuda.current_stream()
        if n_slices == 1:
            for n in names:
                dev_in[n].copy_(host[n], non_blocking=True)
            inp = dict(x)
            inp.update(dev_in)
            res = step(inp)
            for dst, src in zip(host_out, res):
                dst.copy_(src, non_blocking=True)
            return
        s_in.wait_stream(cur)
        ready = []
        for b in range(n_slices):
            with torch.cuda.stream(s_in):
                for n in names:
                    dev_in[n][b:b + 1].copy_(host[n][b:b + 1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
                ready.append(ev)
        for b in range(n_slices):
            cur.wait_event(ready[b])
            inp = dict(x)
            inp.update({n: dev_in[n][b:b + 1] for n in names})
            res = step(inp)
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for dst, src in zip(host_out, res):
                    src.record_stream(s_out)
                    dst[b:b + 1].copy_(src, non_blocking=True)
        cur.wait_stream(s_out)

    e2e_steps = max(2, min(args.steps, 5))
    if args.kernel_only:
        e2e_ms = float("nan")
    else:
        e2e_step()
        e2e_ms = timed(e2e_step, e2e_steps) / e2e_steps
    e2e_value = tokens * world / (e2e_ms * 1e-3)

    # ---- dominant kernel alone, launched exactly as inside the step (same segment plan),
    # timed with CUDA events on the launching stream
    g_cum = ops.chunk_local_cumsum(x["g"], 64, x["cu"])
    A = ops.kkt_solve(x["k"], x["beta"], g_cum, x["cu"])
    scale = 128 ** -0.5
    B_, T_ = x["q"].shape[:2]
    tables = ops.SeqTables(B_, T_, x["cu"])
    plan = cp.plan_segments(tables, x["Hv"], device=x["q"].device)
    run_tables, run_h0 = tables, x["h0"]
    if plan is not None:
        run_tables = plan.seg_tables
        run_h0 = cp.forward_segment_states(plan, x["k"], x["v"], A, g_cum, x["beta"], scale, x["h0"])
    G = x["Hv"] // x["Hq"]
    if not bwd:
        kernel_name = "fwd_tc_kernel"

        def dominant():
            ops.fwd_seq(x["q"], x["k"], x["v"], A, g_cum, x["beta"], scale, run_h0,
                        output_final_state=True, tables=run_tables)

        # per (token, value head): q,k / v / A / g / beta / o
        bytes_per_th = 2 * 128 * 2 / G + 2 * 128 + 2 * 64 + 4 + 2 + 2 * 128
        flop_per_th = 147_456
    else:
        kernel_name = "bwd_main_tc_kernel"
        fw = ops.fwd_seq(None, x["k"], x["v"], A, g_cum, x["beta"], scale, run_h0, output_o=False,
                         output_h=True, output_vnew=True, tables=run_tables, operand_tiles=True)
        bw = ops.bwd_dh(x["q"], x["k"], A, g_cum, x["beta"], x["do"], scale, None,
                        tables=run_tables, operand_tiles=True)

        def dominant():
            ops.bwd_main(x["q"], x["k"], x["v"], fw["vnew"], A, g_cum, x["beta"], x["do"],
                         bw["du"], fw["h"], bw["dh"], scale, tables=run_tables,
                         operand_tiles=True)

        # per (token, value head): q,k / v,vnew,do,du / A / h,dh (2 x 32 KiB per 64 tokens) /
        # g,beta / dq,dk,dv / dg,db
        bytes_per_th = 2 * 128 * 2 / G + 4 * 256 + 128 + 2 * 32768 / 64 + 6 + 3 * 256 + 8
        # 16 tile products per chunk: 3 of 64x128x128, 5 of 64x64x128, 6 of 64x128x64, 2 of 64x64x64
        flop_per_th = 2 * (3 * 128 * 128 + 5 * 64 * 128 + 6 * 128 * 64 + 2 * 64 * 64)

    for _ in range(3):
        dominant()
    k_ms = timed(dominant, args.steps) / args.steps
    # DRAM bytes per (token, value head) of one launch, from the ncu capture of the quarter-size
    # workload (profiles/kernels__c1_quarter.md: read + write counters / 131072 pairs); traffic
    # grows in proportion to the pairs processed
    traffic_per_th = {"fwd_tc_kernel": 143.4e6 / 131072, "bwd_main_tc_kernel": 432.7e6 / 131072}
    traffic = traffic_per_th[kernel_name] * tokens * x["Hv"] if G == 1 else None
    alg_bytes = tokens * x["Hv"] * bytes_per_th
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = json.load(open(peaks_path))["hbm_gbs"], "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    achieved = alg_bytes / (k_ms * 1e-3) / 1e9
    roofline = {"kernel": kernel_name, "bound": "hbm", "achieved": round(achieved, 1),
                "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                "frac": round(achieved / peak, 4),
                "traffic": None if traffic is None else round(traffic),
                "traffic_source": "ncu dram__bytes_read+write on c1_quarter, scaled by (token, head) pairs",
                "algorithmic_bytes": round(alg_bytes),
                "kernel_ms": round(k_ms, 4),
                "tensor_tflops": round(tokens * x["Hv"] * flop_per_th / (k_ms * 1e-3) / 1e12, 1)}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    cpu = cpu_baseline(w, seconds=12.0) if world == 1 and not args.kernel_only else None
    flop = (FWDBWD_FLOP if bwd else FWD_FLOP) * tokens * x["Hv"] * world
    line = {
        "metric": f"gdn_{w['mode']}_tokens_per_s", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, **{k: v for k, v in w.items()},
                   "sharding": ("T" if tshard else "head") if args.scaling == "strong" and world > 1
                   else "replicated workload per GPU (independent sequences)",
                   "tokens_per_gpu": tokens, "Hq_per_gpu": x["Hq"], "Hv_per_gpu": x["Hv"],
                   "K": 128, "V": 128, "chunk": 64,
                   "l2": "inputs larger than L2 (no flush needed)"},
        "achieved_tflops": round(flop / (ms_per_step * 1e-3) / 1e12, 1),
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 3),
                "pipelined_slices": n_slices},
        "gpu_launches": launches,
        "roofline": roofline,
        "clocks": clocks.summary(),
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def cpu_sample(w):
    """A bounded sample of the workload for the CPU implementation: all heads of the workload,
    1024 tokens of one sequence (16 chunks)."""
    from oracle import gdr_oracle as orc

    T = 1024
    x = orc.make_inputs(1, T, w["Hq"], w["Hv"], 128, 128, seed=1234, with_h0=w["h0"])
    return x, T


def cpu_run(w, x):
    from oracle import gdr_oracle as orc

    if w["mode"] == "fwd":
        orc.chunk_gdr_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], None, x["h0"])
    else:
        orc.chunk_gdr_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], x["dht"], None,
                          x["h0"])


def _use_all_host_threads():
    """The CPU implementation gets every core the process may run on.  (torchrun exports
    OMP_NUM_THREADS=1 to its workers, which would otherwise leave it with one thread.)"""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_baseline(w, seconds):
    threads = _use_all_host_threads()
    x, T = cpu_sample(w)
    cpu_run(w, x)
    times, t_end = [], time.time() + seconds
    while time.time() < t_end or len(times) < 3:
        t0 = time.perf_counter()
        cpu_run(w, x)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": round(T / med, 1), "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"B=1 T={T} Hq={w['Hq']} Hv={w['Hv']} K=V=128 fp32, {w['mode']}, "
                      f"median of {len(times)} runs; os.cpu_count()={os.cpu_count()}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    threads = _use_all_host_threads()
    x, T = cpu_sample(w)
    for _ in range(max(args.warmup, 1)):
        cpu_run(w, x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_run(w, x)
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    value = T / (ms * 1e-3)
    sample = (f"each step = B=1 T={T} Hq={w['Hq']} Hv={w['Hv']} K=V=128 fp32 {w['mode']} on "
              f"{threads} host threads (PyTorch CPU port of the reference's tests/ref_gdr.py)")
    print(json.dumps({
        "impl": "reference", "metric": f"gdn_{w['mode']}_tokens_per_s", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": int(os.environ.get("WORLD_SIZE", 1)), "steps": args.steps,
        "warmup": max(args.warmup, 1), "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, **{k: v for k, v in w.items()}},
        "cpu_baseline": {"value": round(value, 1), "unit": "tokens/s", "cores": threads,
                         "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1_fwd", choices=sorted(WORKLOADS))
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU legs (for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
