"""Time the reference's own sm_100 TileLang kernels on this GPU, on the benchmark's seeded inputs.

    python baseline/tilelang_ref.py --workload c1_fwd [--reps 20] [--dump DIR]

Runs in a process of its own because the unmodified reference (installed into
``baseline/_ref`` by ``__graft_entry__.build()``; git-ignored) has the same package name,
``flash_qla``, as this repository's drop-in.  Prints one JSON line: per-call time of the
reference's ``chunk_gated_delta_rule_fwd`` (and ``_bwd`` for a forward+backward workload) with
CUDA events, eager and, when capture works, as CUDA-graph replay (the method of the reference's
own benchmark).  ``--dump DIR`` also stores a sample of the reference's outputs (every 64th row of
``o`` and the final state) so that the caller can compare its own kernels with them.
On any failure (TileLang missing, JIT error) the line is ``{"unavailable": "..."}``.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.path.join(HERE, "_ref")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c1_fwd")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--dump", default=None)
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(REF, "flash_qla")):
        print(json.dumps({"unavailable": "baseline/_ref is not populated (reference not installed)"}))
        return
    sys.path.insert(0, REF)
    import torch

    try:
        import flash_qla  # the reference package (first on the path)

        assert os.path.realpath(flash_qla.__file__).startswith(os.path.realpath(REF))
        ref_fwd, ref_bwd = flash_qla.chunk_gated_delta_rule_fwd, flash_qla.chunk_gated_delta_rule_bwd
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"unavailable": f"import of the reference failed: {type(e).__name__}: "
                                         f"{str(e)[:300]}"}))
        return
    sys.path.append(ROOT)
    import bench  # workload table and seeded input builder only (imports nothing of ours)

    w = bench.WORKLOADS[args.workload]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    x = bench.make_batch(w, dev, 1234)
    bwd = w["mode"] == "fwdbwd"
    out = {"workload": args.workload, "tokens": x["tokens"], "reps": args.reps,
           "tilelang": getattr(__import__("tilelang"), "__version__", "?")}

    def run(beta):
        def fwd():
            return ref_fwd(x["q"], x["k"], x["v"], x["g"], beta, None, x["h0"], x["cu"],
                           output_final_state=True, output_h=False, auto_cp=True)

        res = fwd()
        g_cum, A = res[0], res[1]

        def bwd_call():
            return ref_bwd(x["q"], x["k"], x["v"], g_cum, beta, A, x["do"], x["dht"], None,
                           x["h0"], x["cu"], False, True)

        def timed(fn, reps):
            for _ in range(5):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps

        def graphed(fn, reps):
            try:
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    for _ in range(3):
                        fn()
                torch.cuda.current_stream().wait_stream(s)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    fn()
                return timed(graph.replay, reps)
            except Exception as e:  # noqa: BLE001
                out.setdefault("graph_error", f"{type(e).__name__}: {str(e)[:200]}")
                return None

        out["fwd_ms"] = timed(fwd, args.reps)
        out["fwd_graph_ms"] = graphed(fwd, args.reps)
        if bwd:
            bwd_call()
            out["bwd_ms"] = timed(bwd_call, args.reps)
            out["bwd_graph_ms"] = graphed(bwd_call, args.reps)
        return res

    try:
        try:
            res = run(x["beta"])
            out["beta_dtype"] = str(x["beta"].dtype)
        except Exception as e:  # noqa: BLE001  (the reference's tests and bench pass fp32 beta)
            out["bf16_beta_error"] = f"{type(e).__name__}: {str(e)[:200]}"
            res = run(x["beta"].float())
            out["beta_dtype"] = "torch.float32"
    except Exception as e:  # noqa: BLE001
        traceback.print_exc(file=sys.stderr)
        print(json.dumps({"unavailable": f"reference kernels failed on this box: "
                                         f"{type(e).__name__}: {str(e)[:300]}"}))
        return
    best_f = min(t for t in (out["fwd_ms"], out.get("fwd_graph_ms")) if t)
    total = best_f
    if bwd:
        total += min(t for t in (out["bwd_ms"], out.get("bwd_graph_ms")) if t)
    out["ms_per_step"] = total
    out["tokens_per_s"] = x["tokens"] / (total * 1e-3)
    if args.dump:
        os.makedirs(args.dump, exist_ok=True)
        torch.save({"o_rows": res[2][:, ::64].float().cpu(), "ht": res[4].float().cpu()},
                   os.path.join(args.dump, f"tilelang_{args.workload}.pt"))
        out["dump"] = os.path.join(args.dump, f"tilelang_{args.workload}.pt")
    print(json.dumps(out))


if __name__ == "__main__":
    main()
