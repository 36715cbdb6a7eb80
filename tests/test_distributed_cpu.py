"""Host logic of the multi-GPU paths on CPU ranks (gloo, world size 2): the boundary-state
exchange of T sharding against the oracle, the reverse (gradient) chain, head sharding, and a
rank that never joins (failure on the host, no GPU involved)."""

import datetime
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def cpu_merge(local, M, use_m, raw, seg_begin, reverse=False):
    """Torch stand-in for the CUDA merge kernel, same contract as ``ops.merge_states``."""
    out = torch.empty_like(local)
    for r in range(seg_begin.numel() - 1):
        s0, s1 = int(seg_begin[r]), int(seg_begin[r + 1])
        cur = raw[r].clone() if raw is not None else torch.zeros_like(local[0])
        order = range(s1 - 1, s0 - 1, -1) if reverse else range(s0, s1)
        for n, i in enumerate(order):
            out[i] = cur
            if n == s1 - s0 - 1:
                break
            m = M[i].transpose(-1, -2) if reverse else M[i]
            gate = (use_m[i] != 0).to(local.dtype)[:, None, None]
            cur = local[i] + gate * (m @ cur)
    return out


def _init(rank, world, port, timeout_s=60):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))


def _worker_tshard(rank, world, port, out):
    from flashqla_b200 import distributed as fd
    from oracle import gdr_oracle as orc

    _init(rank, world, port)
    T, H, D = 256, 2, 32
    x = orc.make_inputs(1, T, H, H, D, D, seed=5, dtype=torch.float64, round_to=None, gate="weak")
    # the truth: one pass over the whole sequence; h[c] is the state entering chunk c
    _, _, o_full, h_full, ht_full = orc.chunk_gdr_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"],
                                                      None, x["h0"])
    per = T // world
    sl = slice(rank * per, (rank + 1) * per)
    q, k, v, g, b = (x[n][:, sl] for n in ("q", "k", "v", "g", "beta"))
    # this rank's summary from a zero state, and its transition matrix (state = identity, v = 0)
    local = orc.chunk_gdr_fwd(q, k, v, g, b, None, None)[4]
    eye = torch.eye(D, dtype=torch.float64).expand(1, H, D, D)
    M = orc.chunk_gdr_fwd(q, k, torch.zeros_like(v), g, b, None, eye)[4]
    use_m = torch.ones(1, H, dtype=torch.int32)
    # only the owning rank passes the edge state: the collective sequence must not depend on it
    start = fd.exchange_forward(local, M, use_m, x["h0"] if rank == 0 else None, merge_fn=cpu_merge)
    want = h_full[0, rank * per // 64].unsqueeze(0)
    err_state = float((start - want).norm() / want.norm())
    # running the shard from the exchanged state reproduces the unsplit outputs
    _, _, o, _, ht = orc.chunk_gdr_fwd(q, k, v, g, b, None, start)
    err_o = float((o - o_full[:, sl]).norm() / o_full[:, sl].norm())
    err_ht = float((ht - ht_full).norm() / ht_full.norm()) if rank == world - 1 else 0.0
    # reverse chain on random summaries against an explicit loop
    gen = torch.Generator().manual_seed(100 + rank)
    loc_b = torch.randn(1, H, D, D, generator=gen, dtype=torch.float64)
    dht = torch.randn(1, H, D, D, generator=torch.Generator().manual_seed(7), dtype=torch.float64)
    end = fd.exchange_backward(loc_b, M, use_m, dht if rank == world - 1 else None,
                               merge_fn=cpu_merge)
    locs = [torch.randn(1, H, D, D, generator=torch.Generator().manual_seed(100 + r),
                        dtype=torch.float64) for r in range(world)]
    Ms = [torch.empty_like(M) for _ in range(world)]
    dist.all_gather(Ms, M)
    cur = dht
    for r in range(world - 1, rank, -1):
        cur = locs[r] + Ms[r].transpose(-1, -2) @ cur
    err_b = float((end - cur).norm() / cur.norm())
    # the spare step of the chain: the final state of the sequence (forward) and the gradient of
    # its initial state (reverse) on EVERY rank, without a second collective
    rec = fd._record_from(local, M, use_m, x["h0"] if rank == 0 else None, rank == 0)
    chained = fd._exchange(rec, H, D, 0, False, None, cpu_merge)
    assert chained.shape[0] == world + 1
    err_final = float((chained[world] - ht_full[0]).norm() / ht_full.norm())
    rec_b = fd._record_from(loc_b, M, use_m, dht if rank == world - 1 else None,
                            rank == world - 1)
    chained_b = fd._exchange(rec_b, H, D, world - 1, True, None, cpu_merge)
    first = dht
    for r in range(world - 1, -1, -1):
        first = locs[r] + Ms[r].transpose(-1, -2) @ first
    err_first = float((chained_b[0] - first[0]).norm() / first.norm())
    out[rank] = (err_state, err_o, err_ht, err_b, err_final, err_first)
    dist.destroy_process_group()


def test_tshard_exchange_matches_oracle_on_two_cpu_ranks():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker_tshard, args=(world, port, out), nprocs=world, join=True)
        for rank in range(world):
            assert max(out[rank]) < 1e-10, (rank, out[rank])


def test_shard_heads_covers_every_head_once():
    from flashqla_b200.distributed import shard_heads

    B, T, Hq, Hv, D = 2, 8, 4, 8, 4
    q = torch.arange(B * T * Hq * D, dtype=torch.float32).reshape(B, T, Hq, D)
    v = torch.arange(B * T * Hv * D, dtype=torch.float32).reshape(B, T, Hv, D)
    g = torch.arange(B * T * Hv, dtype=torch.float32).reshape(B, T, Hv)
    h0 = torch.arange(B * Hv * D * D, dtype=torch.float32).reshape(B, Hv, D, D)
    for world in (1, 2, 4, 8):
        vs, qs = [], []
        for r in range(world):
            ql, kl, vl, gl, bl, hl = shard_heads(q, q, v, g, g, r, world, h0)
            assert vl.shape[2] == Hv // world and gl.shape[2] == Hv // world
            assert hl.shape[1] == Hv // world and vl.shape[2] % ql.shape[2] == 0
            # every local value head still sees its own q/k head
            G_loc = vl.shape[2] // ql.shape[2]
            for j in range(vl.shape[2]):
                gv = r * (Hv // world) + j
                assert torch.equal(ql[:, :, j // G_loc], q[:, :, gv // (Hv // Hq)])
            vs.append(vl)
            qs.append(ql)
        assert torch.equal(torch.cat(vs, 2), v)
    with pytest.raises(ValueError):
        shard_heads(q, q, v, g, g, 0, 3)


def _worker_missing_rank(rank, world, port, out):
    from flashqla_b200 import distributed as fd

    try:
        _init(rank, world, port, timeout_s=5)
    except Exception as e:  # rendezvous itself may time out when the peer never comes
        out[rank] = type(e).__name__
        return
    x = torch.zeros(1, 1, 4, 4, dtype=torch.float64)
    try:
        fd.exchange_forward(x, x, torch.ones(1, 1, dtype=torch.int32), None, merge_fn=cpu_merge)
        out[rank] = "no error"
    except Exception as e:
        out[rank] = type(e).__name__


def test_rank_that_never_joins_is_a_host_error():
    """World size 2 but only rank 0 starts: the exchange (or the rendezvous before it) must end
    with an exception on the host within the process-group timeout."""
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker_missing_rank, args=(2, port, out), nprocs=1, join=True)
        assert out[0] != "no error"
