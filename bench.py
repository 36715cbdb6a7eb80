"""Benchmark of the gated-delta-rule chunked prefill on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c1_fwd|c3_fwdbwd|...] [--scaling strong|weak]

One "step" is one pass of the hot path over one synthetic batch.  Default workload: the fixed
length forward prefill B=4, T=8192, H_q=H_v=16, K=V=128 (bf16 inputs, fp32 gates).  Rank 0 prints
ONE JSON line.  Under torchrun (N > 1) the same 32768 tokens are sharded over the ranks by value
head (no communication; ``"scaling": "strong"``), all ranks meet at a barrier on both sides of the
timed region and the slowest rank's device time is used.  The line also carries, measured in the
same run: ``fwdbwd`` (the training workload, forward + backward), ``tshard`` (the single
262144-token sequence: on one GPU at N = 1, sharded along T with the boundary-state exchange over
NCCL at N > 1), the roofline of the dominant kernel, the CPU baseline and, on one GPU, the
reference's own TileLang kernels on the same inputs (``reference_tilelang``).

``--impl reference`` times the reference's CPU implementation of the same operator
(``tests/ref_gdr.py`` of the reference, copied unmodified into the git-ignored ``oracle/_ref/`` by
``oracle/build_ref.py``; the PyTorch port in ``oracle/gdr_oracle.py`` when that copy is absent)
on a bounded sample of the workload using all host threads, and on the reference's own
CPU-sized configuration (B=1, T=512, H=4, K=V=64) exactly.
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
    sys.path.append(ROOT)

# Algorithmic work per (token, value head) at K=V=128, chunk 64 (2 FLOP per multiply-add).
FWD_FLOP = 163_840
FWDBWD_FLOP = 655_360
L2_BYTES = 126 * 1024 * 1024

WORKLOADS = {
    # name: dict(B, T, Hq, Hv, mode, varlen)
    "c1_fwd": dict(B=4, T=8192, Hq=16, Hv=16, mode="fwd", varlen=None, h0=False),
    "c1_fwdbwd": dict(B=4, T=8192, Hq=16, Hv=16, mode="fwdbwd", varlen=None, h0=False),
    "c2_fwd": dict(B=1, T=None, Hq=8, Hv=8, mode="fwd", varlen="uniform64", h0=True),
    "c3_fwdbwd": dict(B=1, T=32768, Hq=16, Hv=32, mode="fwdbwd", varlen="lognormal", h0="zeros"),
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


def make_batch(w, device, seed, batch=None):
    """Seeded synthetic inputs with the benchmark configuration's shapes and distributions."""
    Hq, Hv = w["Hq"], w["Hv"]
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
    if w["h0"] == "zeros":  # an initial state that is present (its gradient is wanted) but zero
        h0.zero_()
    do = rn(B, T, Hv, 128).bfloat16()
    dht = 0.1 * rn(N, Hv, 128, 128)
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32, device=device)
    return dict(q=q, k=k, v=v, g=g, beta=beta, h0=h0, do=do, dht=dht, cu=cu_t, tokens=B * T,
                Hv=Hv, Hq=Hq)


def shard_batch_by_head(x, rank, world):
    """This rank's value heads (and their q/k heads) of a full batch: no communication needed."""
    from flashqla_b200.distributed import shard_heads

    Hv = x["Hv"]
    q, k, v, g, beta, h0 = shard_heads(x["q"], x["k"], x["v"], x["g"], x["beta"], rank, world,
                                       x["h0"])
    hv = Hv // world
    sl = slice(rank * hv, (rank + 1) * hv)
    return dict(q=q, k=k, v=v, g=g, beta=beta, h0=h0, do=x["do"][:, :, sl].contiguous(),
                dht=x["dht"][:, sl].contiguous(), cu=x["cu"], tokens=x["tokens"], Hv=hv,
                Hq=q.shape[2])


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


def input_bytes(x):
    return sum(t.numel() * t.element_size() for t in x.values() if isinstance(t, torch.Tensor))


class Timer:
    """Device timing of a step function: CUDA events on the launching stream, a barrier and a
    device synchronize on both sides, the maximum over ranks.  When a step's working set is
    smaller than twice the L2, a 256 MiB write flushes the L2 before every timed step (each step
    is then timed by its own pair of events and the flush stays outside them)."""

    def __init__(self, dev, world):
        import torch.distributed as dist

        self.dev, self.world, self.dist = dev, world, dist
        self.flush_buf = None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def run(self, fn, steps, flush):
        if flush and self.flush_buf is None:
            self.flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=self.dev)
        self.barrier()
        if not flush:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            self.barrier()
            ms = e0.elapsed_time(e1)
        else:
            pairs = []
            for _ in range(steps):
                self.flush_buf.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                pairs.append((e0, e1))
            self.barrier()
            ms = sum(a.elapsed_time(b) for a, b in pairs)
        if self.world > 1:
            t = torch.tensor([ms], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps


def capture_graph(fn):
    """One step as a CUDA graph (what the reference's own benchmark replays), or None when the
    capture does not work; the caller then times eager launches."""
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            keep = fn()
        graph._keep_outputs = keep
        graph.replay()
        torch.cuda.synchronize()
        return graph
    except Exception as e:  # noqa: BLE001
        print(f"[bench] CUDA graph capture failed, timing eager launches: {e}", file=sys.stderr)
        torch.cuda.synchronize()
        return None


def make_step(fq, x, bwd):
    def step(inp=x):
        g_cum, A, o, _, ht, cache = fq.chunk_gated_delta_rule_fwd(
            inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], None, inp["h0"], inp["cu"],
            output_final_state=True, enable_fwd_cp_cache=bwd)
        if not bwd:
            return o, ht
        grads = fq.chunk_gated_delta_rule_bwd(
            inp["q"], inp["k"], inp["v"], g_cum, inp["beta"], A, inp["do"], inp["dht"], None,
            inp["h0"], inp["cu"], cp_cache=cache)
        return (o, ht) + tuple(t for t in grads if t is not None)

    return step


def make_tshard_step(x, bwd):
    from flashqla_b200 import distributed as fd

    def step(inp=x):
        g_cum, A, o, ht, saved = fd.fwd_tsharded(inp["q"], inp["k"], inp["v"], inp["g"],
                                                 inp["beta"], None, None, for_backward=bwd)
        if not bwd:
            return o, ht
        grads = fd.bwd_tsharded(inp["q"], inp["k"], inp["v"], g_cum, inp["beta"], A, inp["do"],
                                inp["dht"], None, saved)
        return (o, ht) + tuple(grads)

    return step


def time_step(timer, step, x, steps, warmup, use_graph):
    """ms per step of ``step`` (after warm-up), the timing mode, and launches per step."""
    from flashqla_b200 import _lib

    for _ in range(max(warmup, 3)):
        step()
    n0 = _lib.launch_count
    step()
    launches = _lib.launch_count - n0
    flush = input_bytes(x) < 2 * L2_BYTES
    graph = capture_graph(step) if use_graph else None
    fn = graph.replay if graph is not None else step
    for _ in range(3):
        fn()
    ms = timer.run(fn, steps, flush)
    mode = ("cuda graph replay" if graph is not None else "eager launches") + \
           (", L2 flushed before every step (256 MiB write)" if flush
            else ", inputs larger than L2 (no flush needed)")
    return ms, mode, launches


# per (token, value head), forward, G = Hv / Hq:  q,k / v / g / beta / o  (each operand once) ...
def fwd_min_bytes(G):
    return 2 * 128 * 2 / G + 2 * 128 + 4 + 2 + 2 * 128


# ... and what fwd_tc_kernel itself moves: the same plus the A tile written by kkt_solve
def fwd_kernel_bytes(G):
    return fwd_min_bytes(G) + 2 * 64


def bwd_main_kernel_bytes(G):
    # q,k / v,vnew,do,du / A / h,dh (2 x 32 KiB per 64 tokens) / g,beta / dq,dk,dv / dg,db
    return 2 * 128 * 2 / G + 4 * 256 + 128 + 2 * 32768 / 64 + 6 + 3 * 256 + 8


def measured_traffic(kernel, G, pairs):
    """DRAM bytes of one launch, scaled from the committed ncu capture of a smaller case by the
    (token, value head) pairs processed (every tile is read once, so traffic is proportional)."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if G != 1 or not os.path.exists(path):
        return None, None
    entry = json.load(open(path)).get(kernel)
    if not entry:
        return None, None
    return entry["dram_bytes"] / entry["pairs"] * pairs, entry["source"]


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path))["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def dominant_kernel_roofline(timer, x, bwd, steps):
    """The dominant kernel alone, launched exactly as inside the step (same segment plan), timed
    with CUDA events on the launching stream."""
    from flashqla_b200 import cp, ops

    g_cum, A = ops.kkt_solve(x["k"], x["beta"], x["g"], x["cu"], raw_gate=True)
    scale = 128 ** -0.5
    B_, T_ = x["q"].shape[:2]
    tables = ops.SeqTables(B_, T_, x["cu"])
    plan = cp.plan_segments(tables, x["Hv"], device=x["q"].device)
    run_tables, run_h0, lead = tables, x["h0"], None
    if plan is not None:
        run_tables = plan.seg_tables
        run_h0, lead = cp.forward_start(plan, x["k"], x["v"], A, g_cum, x["beta"], scale, x["h0"])
    G = x["Hv"] // x["Hq"]
    pairs = x["tokens"] * x["Hv"]
    if not bwd:
        kernel_name = "fwd_tc_kernel"

        def dominant():
            ops.fwd_seq(x["q"], x["k"], x["v"], A, g_cum, x["beta"], scale, run_h0,
                        output_final_state=True, tables=run_tables, lead_chunks=lead)

        min_bytes, kernel_bytes, flop_per_pair = fwd_min_bytes(G), fwd_kernel_bytes(G), 147_456
    else:
        kernel_name = "bwd_main_tc_kernel"
        fw = ops.fwd_seq(None, x["k"], x["v"], A, g_cum, x["beta"], scale, run_h0, output_o=False,
                         output_h=True, output_vnew=True, tables=run_tables, operand_tiles=True,
                         lead_chunks=lead)
        bw = ops.bwd_dh(x["q"], x["k"], A, g_cum, x["beta"], x["do"], scale, None,
                        tables=run_tables, operand_tiles=True)

        def dominant():
            ops.bwd_main(x["q"], x["k"], x["v"], fw["vnew"], A, g_cum, x["beta"], x["do"],
                         bw["du"], fw["h"], bw["dh"], scale, tables=run_tables,
                         operand_tiles=True)

        # the backward's minimum (each operand once, no h round trip): q,k,v,do,A,g,beta in;
        # dq,dk,dv,dg,db out
        min_bytes = 2 * 256 / G + 2 * 256 + 128 + 6 + 3 * 256 + 8
        kernel_bytes = bwd_main_kernel_bytes(G)
        # 16 tile products per chunk: 3 of 64x128x128, 5 of 64x64x128, 6 of 64x128x64, 2 of 64x64x64
        flop_per_pair = 2 * (3 * 128 * 128 + 5 * 64 * 128 + 6 * 128 * 64 + 2 * 64 * 64)
    for _ in range(3):
        dominant()
    k_ms = timer.run(dominant, steps, input_bytes(x) < 2 * L2_BYTES)
    peak, peak_src = hbm_peak()
    achieved = pairs * min_bytes / (k_ms * 1e-3) / 1e9
    achieved_kernel = pairs * kernel_bytes / (k_ms * 1e-3) / 1e9
    traffic, traffic_src = measured_traffic(kernel_name, G, pairs)
    return {"kernel": kernel_name, "bound": "hbm", "achieved": round(achieved, 1), "peak": peak,
            "peak_source": peak_src, "unit": "GB/s", "frac": round(achieved / peak, 4),
            "bytes_per_token_head": round(min_bytes, 1),
            "bytes_note": "each operand of the operator once (q,k,v,g,beta in; o out)" if not bwd
            else "each operand of the backward once, no per-chunk state round trip",
            "kernel_bytes_per_token_head": round(kernel_bytes, 1),
            "achieved_kernel_bytes": round(achieved_kernel, 1),
            "frac_kernel_bytes": round(achieved_kernel / peak, 4),
            "traffic": None if traffic is None else round(traffic), "traffic_source": traffic_src,
            "algorithmic_bytes": round(pairs * min_bytes), "kernel_ms": round(k_ms, 4),
            "tensor_tflops": round(pairs * flop_per_pair / (k_ms * 1e-3) / 1e12, 1)}


def run_ours(args):
    import torch.distributed as dist

    import flashqla_b200 as fq

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        from flashqla_b200 import distributed as fd

        if args.reserve_sms is not None:
            fd.RESERVE_SMS = args.reserve_sms
        dist.init_process_group("nccl", device_id=dev)
    timer = Timer(dev, world)
    w = WORKLOADS[args.workload]
    bwd = w["mode"] == "fwdbwd"
    single_long = w["B"] == 1 and not w["varlen"]
    strong = args.scaling == "strong"

    def build(wl, seed_rank=True):
        """This rank's part of workload ``wl`` under the chosen scaling."""
        if world == 1 or not strong:
            return make_batch(wl, dev, 1234 + (rank if seed_rank else 0)), "none"
        if wl["B"] == 1 and not wl["varlen"]:
            shard = make_batch(dict(wl, T=wl["T"] // world), dev, 1234 + rank)
            shard["h0"] = None
            return shard, "T"
        if wl["Hv"] % world or (wl["Hq"] % world and world % wl["Hq"]):
            raise SystemExit(f"{wl['Hv']} value / {wl['Hq']} q heads do not shard over {world} ranks")
        full = make_batch(wl, dev, 1234)
        return shard_batch_by_head(full, rank, world), "head"

    x, sharding = build(w)
    hq_gpu, hv_gpu = x["Hq"], x["Hv"]
    if sharding == "T":
        step = make_tshard_step(x, bwd)
        tokens_total = x["tokens"] * world
    else:
        step = make_step(fq, x, bwd)
        tokens_total = x["tokens"] * (world if sharding == "none" else 1)

    with ClockSampler(local) as clocks:
        # keep the GPU under load until the clock sampler has come up
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        if not args.kernel_only:
            t_up = time.time() + 0.6
            while time.time() < t_up:
                step()
                torch.cuda.synchronize()
        ms_per_step, mode, launches = time_step(timer, step, x, args.steps, args.warmup,
                                                use_graph=not args.eager)
        if not args.kernel_only:
            t_up = time.time() + 0.3  # a few more samples under load after the timed steps
            while time.time() < t_up:
                step()
                torch.cuda.synchronize()
    value = tokens_total / (ms_per_step * 1e-3)

    # ---- end to end: pinned host inputs -> device, operator, result back to host
    e2e = None
    if not args.kernel_only:
        names = ["q", "k", "v", "g", "beta"] + (["do", "dht"] if bwd else []) + \
                (["h0"] if x["h0"] is not None else [])
        host = {n: x[n].cpu().pin_memory() for n in names}
        dev_in = {n: torch.empty_like(x[n]) for n in names}
        outs = step()
        host_out = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in outs]
        h2d = sum(t.numel() * t.element_size() for t in host.values())
        d2h = sum(t.numel() * t.element_size() for t in host_out)
        # A fixed-length batch is fed sequence by sequence: the copy-in of sequence b+1 and the
        # copy-out of sequence b-1 overlap the kernels of sequence b (PCIe is full duplex).
        n_slices = x["q"].shape[0] if (x["cu"] is None and sharding != "T" and x["q"].shape[0] > 1) else 1
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
        e2e_step()
        e2e_ms = timer.run(e2e_step, e2e_steps, False)
        e2e = {"value": round(tokens_total / (e2e_ms * 1e-3), 1), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": round(e2e_ms, 3), "pipelined_slices": n_slices}
        del host, dev_in, host_out

    roofline = dominant_kernel_roofline(timer, x, bwd, args.steps)

    # ---- the other headline workloads, in the same run (every rank takes part) --------------
    extra = {}
    if args.workload == "c1_fwd" and not args.kernel_only and not args.no_extras:
        sub_steps = max(3, min(args.steps, 10))
        del x
        torch.cuda.empty_cache()
        # training workload: forward + backward, GVA, packed log-normal lengths
        w3 = WORKLOADS["c3_fwdbwd"]
        x3, sh3 = build(w3)
        ms3, mode3, _ = time_step(timer, make_step(fq, x3, True), x3, sub_steps, 3, not args.eager)
        rl3 = dominant_kernel_roofline(timer, x3, True, sub_steps)
        tok3 = x3["tokens"] * (world if sh3 == "none" else 1)
        extra["fwdbwd"] = {"workload": "c3_fwdbwd", "sharding": sh3, "ms_per_step": round(ms3, 4),
                           "tokens_per_s": round(tok3 / (ms3 * 1e-3), 1), "timing": mode3,
                           "achieved_tflops": round(FWDBWD_FLOP * tok3 * w3["Hv"] /
                                                    (ms3 * 1e-3) / 1e12, 1),
                           "roofline": rl3}
        del x3
        torch.cuda.empty_cache()
        # the single long sequence: forward, and forward + backward
        ts = {}
        for name in ("c4_fwd", "c4_fwdbwd"):
            w4 = WORKLOADS[name]
            b4 = w4["mode"] == "fwdbwd"
            x4, sh4 = build(w4)
            st4 = make_tshard_step(x4, b4) if sh4 == "T" else make_step(fq, x4, b4)
            # (the T-sharded step holds one NCCL all-gather per direction; it is captured too)
            ms4, mode4, _ = time_step(timer, st4, x4, sub_steps, 3, use_graph=not args.eager)
            tok4 = w4["T"] if sh4 == "T" else x4["tokens"] * (world if sh4 == "none" else 1)
            ts[name] = {"ms_per_step": round(ms4, 4), "tokens_per_s": round(tok4 / (ms4 * 1e-3), 1),
                        "sharding": "T over %d ranks, one all-gather of boundary states per "
                                    "direction" % world if sh4 == "T" else sh4,
                        "timing": mode4}
            del x4, st4
            torch.cuda.empty_cache()
        extra["tshard"] = ts

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    flop = (FWDBWD_FLOP if bwd else FWD_FLOP) * tokens_total * w["Hv"]
    line = {
        "metric": f"gdn_{w['mode']}_tokens_per_s", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, **{k: v for k, v in w.items()},
                   "sharding": {"none": "one full workload per GPU (independent sequences)"
                                if world > 1 else "one GPU",
                                "head": "value heads (and their q/k heads) split over the ranks, "
                                        "no communication",
                                "T": "tokens of the one sequence split over the ranks, boundary "
                                     "states by one all-gather per direction"}[sharding],
                   "tokens_total": tokens_total, "Hq_per_gpu": hq_gpu, "Hv_per_gpu": hv_gpu,
                   "K": 128, "V": 128, "chunk": 64, "timing": mode},
        "achieved_tflops": round(flop / (ms_per_step * 1e-3) / 1e12, 1),
        "gpu_launches": launches * args.steps,
        "roofline": roofline,
        "clocks": clocks.summary(),
    }
    if e2e is not None:
        line["e2e"] = e2e
    line.update(extra)
    if world == 1 and not args.kernel_only:
        line["cpu_baseline"] = cpu_baseline_subprocess(args.workload)
        if not args.no_tilelang:
            line["reference_tilelang"] = tilelang_subprocess(
                ["c1_fwd", "c3_fwdbwd"] if args.workload == "c1_fwd" else [args.workload])
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---- the reference's own implementations, each in a process of its own ------------------------

def _last_json_line(text):
    for ln in reversed(text.strip().splitlines()):
        ln = ln.strip()
        if ln.startswith("{"):
            try:
                return json.loads(ln)
            except ValueError:
                continue
    return None


def cpu_baseline_subprocess(workload):
    """The CPU arm (``--impl reference``) run in a child process: the reference's file imports
    ``flash_qla.utils``, a name this process has already bound to the drop-in package."""
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "OMP_NUM_THREADS"):
        env.pop(k, None)
    try:
        res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                              "--workload", workload, "--steps", "3", "--warmup", "1",
                              "--cpu-seconds", "10"], capture_output=True, text=True, timeout=240,
                             env=env, cwd=ROOT)
        line = _last_json_line(res.stdout)
        if line is None:
            return {"error": (res.stderr or res.stdout)[-300:]}
        return line["cpu_baseline"]
    except subprocess.TimeoutExpired:
        return {"error": "CPU baseline did not finish within 240 s"}


def tilelang_subprocess(workloads):
    out = {}
    dump = tempfile.mkdtemp(prefix="fqla_tl_")
    for name in workloads:
        try:
            res = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "tilelang_ref.py"),
                                  "--workload", name, "--reps", "20", "--dump", dump],
                                 capture_output=True, text=True, timeout=420, cwd=ROOT)
            line = _last_json_line(res.stdout) or {"unavailable": "unavailable on this box: " +
                                                   (res.stderr or res.stdout)[-300:]}
        except subprocess.TimeoutExpired:
            line = {"unavailable": "unavailable on this box: no result within 420 s (JIT compile)"}
        if "dump" in line:
            line["parity_vs_ours"] = compare_with_tilelang(name, line.pop("dump"))
        out[name] = line
    return out


def compare_with_tilelang(name, path):
    """Normalised difference between this library's forward and the reference's TileLang forward
    on the same seeded inputs (every 64th row of o, and the final state)."""
    import flashqla_b200 as fq

    try:
        ref = torch.load(path)
        x = make_batch(WORKLOADS[name], torch.device("cuda", torch.cuda.current_device()), 1234)
        _, _, o, _, ht, _ = fq.chunk_gated_delta_rule_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"],
                                                          None, x["h0"], x["cu"])
        rel = lambda a, b: float((a.double() - b.double()).norm() / b.double().norm())  # noqa: E731
        return {"o_rows": round(rel(o[:, ::64].float().cpu(), ref["o_rows"]), 6),
                "final_state": round(rel(ht.float().cpu(), ref["ht"]), 6)}
    except Exception as e:  # noqa: BLE001
        return {"error": f"{type(e).__name__}: {str(e)[:200]}"}


# ---- CPU arm ---------------------------------------------------------------------------------------

def _use_all_host_threads():
    """The CPU implementation gets every core the process may run on.  (torchrun exports
    OMP_NUM_THREADS=1 to its workers, which would otherwise leave it with one thread.)"""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


class CpuImpl:
    """The reference's ``tests/ref_gdr.py`` when its copy is present, else the port."""

    def __init__(self):
        from oracle import ref_loader

        self.ref = ref_loader.load() if ref_loader.available() else None
        self.kind = "reference" if self.ref is not None else "port"
        self.what = ("the reference's own tests/ref_gdr.py (unmodified copy in oracle/_ref)"
                     if self.ref is not None else
                     "PyTorch port of the reference's tests/ref_gdr.py (oracle/gdr_oracle.py)")

    def fwd(self, x):
        if self.ref is not None:
            return self.ref.chunk_gated_delta_rule_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"],
                                                       None, x["h0"], None)
        from oracle import gdr_oracle as orc

        return orc.chunk_gdr_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], None, x["h0"])

    def fwdbwd(self, x):
        if self.ref is not None:
            leaves = {n: x[n].clone().requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
            h0 = None if x["h0"] is None else x["h0"].clone().requires_grad_(True)
            o, ht = self.ref.chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"],
                                                    leaves["g"], leaves["beta"], None, h0, True)
            ((o * x["do"]).sum() + (ht * x["dht"]).sum()).backward()
            return leaves["q"].grad
        from oracle import gdr_oracle as orc

        return orc.chunk_gdr_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], x["dht"],
                                 None, x["h0"])


def _median_time(fn, seconds, min_runs=3):
    fn()
    times, t_end = [], time.time() + seconds
    while time.time() < t_end or len(times) < min_runs:
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return statistics.median(times), len(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    from oracle import gdr_oracle as orc

    w = WORKLOADS[args.workload]
    threads = _use_all_host_threads()
    impl = CpuImpl()
    bwd = w["mode"] == "fwdbwd"
    # bounded sample of the workload: all its heads, K = V = 128, 1024 tokens of one sequence
    T = 1024
    x = orc.make_inputs(1, T, w["Hq"], w["Hv"], 128, 128, seed=1234, with_h0=w["h0"])
    run = (lambda: impl.fwdbwd(x)) if bwd else (lambda: impl.fwd(x))
    for _ in range(max(args.warmup, 1)):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    value = T / (ms * 1e-3)
    # the reference's own CPU-sized configuration, exactly: B=1, T=512, H=4, K=V=64, with h0
    x0 = orc.make_inputs(1, 512, 4, 4, 64, 64, seed=1234, with_h0=True, round_to=None)
    budget = max(args.cpu_seconds / 2, 1.0)
    f_med, f_n = _median_time(lambda: impl.fwd(x0), budget)
    b_med, b_n = _median_time(lambda: impl.fwdbwd(x0), budget)
    sample = (f"each step = B=1 T={T} Hq={w['Hq']} Hv={w['Hv']} K=V=128 fp32 {w['mode']}"
              f"{' with h0' if w['h0'] else ''} on {threads} host threads: {impl.what}")
    cpu = {"value": round(value, 1), "unit": "tokens/s", "cores": threads, "kind": impl.kind,
           "sample": sample + f"; os.cpu_count()={os.cpu_count()}",
           "config0": {"shape": "B=1 T=512 Hq=Hv=4 K=V=64 chunk 64 fp32 with h0 (exact)",
                       "fwd_tokens_per_s": round(512 / f_med, 1), "fwd_ms": round(f_med * 1e3, 3),
                       "fwd_runs": f_n, "fwdbwd_tokens_per_s": round(512 / b_med, 1),
                       "fwdbwd_ms": round(b_med * 1e3, 3), "fwdbwd_runs": b_n}}
    print(json.dumps({
        "impl": "reference", "metric": f"gdn_{w['mode']}_tokens_per_s", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": int(os.environ.get("WORLD_SIZE", 1)), "steps": args.steps,
        "warmup": max(args.warmup, 1), "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload,
                   "ran": {"B": 1, "T": T, "Hq": w["Hq"], "Hv": w["Hv"], "K": 128, "V": 128,
                           "mode": w["mode"], "h0": w["h0"]},
                   "note": "a bounded sample of the named workload (its heads and head size, 1024 "
                           "tokens); throughput in tokens/s is what compares"},
        "cpu_baseline": cpu,
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
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="strong: one fixed workload sharded over the ranks (by value head, or "
                         "along T for the single long sequence); weak: one full workload per GPU")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end, CPU and extra legs (for profiler captures)")
    ap.add_argument("--eager", action="store_true", help="time eager launches, no CUDA graph")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the fwd+bwd and long-sequence blocks of the default line")
    ap.add_argument("--reserve-sms", type=int, default=None,
                    help="N > 1: SMs the T-sharded recurrence leaves to the exchange "
                         "(default: the library's RESERVE_SMS)")
    ap.add_argument("--no-tilelang", action="store_true",
                    help="skip timing the reference's TileLang kernels")
    ap.add_argument("--cpu-seconds", type=float, default=10.0,
                    help="CPU arm: time budget of the exact-config-0 measurement")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
