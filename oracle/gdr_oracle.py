"""CPU oracle for the gated-delta-rule chunked prefill (forward and backward).

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file; it is used by
``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of ``bench.py`` as the
checker / the timed CPU port, never as the thing shipped.

Parity pin: ``tests/golden/*.npz`` hold outputs of the reference's own pure-PyTorch
implementation (``tests/ref_gdr.py`` of the reference, run on CPU in fp64 by
``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks every function here against
those vectors.

Three independent statements of the same operator:

* ``recurrent_gdr``  - the token-by-token recurrence (chunk-size agnostic), which is what the
  reference's chunked code is algebraically equal to:
  ``S <- exp(g_t) S;  r = v_t - k_t S;  S <- S + beta_t k_t^T r;  o_t = scale q_t S``.
* ``chunk_gdr_fwd``  - the chunked algorithm, restating the reference's
  ``tests/ref_gdr.py:603-658`` pipeline (cumsum ``:50-74``, gated ``beta K K^T`` ``:77-113``,
  triangular solve ``:116-140``, WY factors ``:143-183``, state recurrence ``:186-245``,
  chunk output ``:248-299``).
* ``chunk_gdr_bwd``  - gradients ``(dq, dk, dv, db, dg, dh0)`` with the contract of
  ``tests/ref_gdr.py:661-746``, obtained by differentiating ``chunk_gdr_fwd`` with autograd
  (the reference hand-writes the same derivative).

Layouts follow the reference: q, k ``[B, T, Hq, K]``; v, o ``[B, T, Hv, V]``; g, beta
``[B, T, Hv]``; states ``[N, Hv, K, V]``; with ``cu_seqlens`` the batch is 1 and sequences are
packed along T.  ``Hv`` must be a multiple of ``Hq`` (grouped value attention).
"""

from __future__ import annotations

import torch

CHUNK = 64


def _seq_bounds(B, T, cu_seqlens):
    """(batch index, start, end) of every sequence."""
    if cu_seqlens is None:
        return [(b, 0, T) for b in range(B)]
    b = [int(x) for x in cu_seqlens.tolist()]
    return [(0, s, e) for s, e in zip(b[:-1], b[1:])]


def _expand_heads(x, Hv):
    """Repeat each q/k head over its group of v heads (``tests/ref_gdr.py:92-93``)."""
    G = Hv // x.shape[-2]
    return x if G == 1 else x.repeat_interleave(G, dim=-2)


def chunk_local_cumsum(g, cu_seqlens=None, chunk_size=CHUNK, reverse=False):
    """Prefix (or suffix) sum of ``g`` inside each chunk; chunks start at each sequence start
    (``tests/ref_gdr.py:50-74``)."""
    B, T = g.shape[:2]
    out = torch.zeros_like(g)
    for b, s, e in _seq_bounds(B, T, cu_seqlens):
        for c0 in range(s, e, chunk_size):
            c1 = min(c0 + chunk_size, e)
            blk = g[b, c0:c1]
            if reverse:
                out[b, c0:c1] = blk.flip(0).cumsum(0).flip(0)
            else:
                out[b, c0:c1] = blk.cumsum(0)
    return out


def recurrent_gdr(q, k, v, g, beta, scale=None, initial_state=None, cu_seqlens=None):
    """Token-level recurrence in the dtype of the inputs.  Returns ``(o, final_state)``."""
    B, T, Hv, V = v.shape
    K = q.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    q, k = _expand_heads(q, Hv), _expand_heads(k, Hv)
    o = torch.zeros_like(v)
    finals = []
    for n, (b, s, e) in enumerate(_seq_bounds(B, T, cu_seqlens)):
        S = (
            torch.zeros(Hv, K, V, dtype=v.dtype)
            if initial_state is None
            else initial_state[n].to(v.dtype).clone()
        )
        for t in range(s, e):
            S = S * g[b, t].exp()[:, None, None]
            r = v[b, t] - torch.einsum("hk,hkv->hv", k[b, t], S)
            S = S + torch.einsum("hk,hv->hkv", k[b, t] * beta[b, t][:, None], r)
            o[b, t] = scale * torch.einsum("hk,hkv->hv", q[b, t], S)
        finals.append(S)
    return o, torch.stack(finals)


def _chunk_one_sequence(q, k, v, g, beta, scale, S, C):
    """One sequence, heads already expanded.  q,k ``[T,H,K]``, v ``[T,H,V]``, g,beta ``[T,H]``,
    S ``[H,K,V]``.  Returns ``(g_cum [T,H], A [T,H,C], o [T,H,V], h [n,H,K,V], S_final)``."""
    T, H, K = q.shape
    V = v.shape[-1]
    n = (T + C - 1) // C
    pad = n * C - T

    def chunked(x):  # [T,H,...] -> [n,H,C,...]; zero rows pad the last chunk
        x = torch.cat([x, x.new_zeros((pad, *x.shape[1:]))]) if pad else x
        return x.reshape(n, C, *x.shape[1:]).transpose(1, 2)

    qc, kc, vc, bc = chunked(q), chunked(k), chunked(v), chunked(beta)
    # zero-padded g keeps the last valid running sum on the pad rows (ref_gdr.py:98)
    gc = chunked(g).cumsum(-1)  # [n,H,C]
    decay = (gc[..., :, None] - gc[..., None, :]).tril().exp().tril()  # exp(g_s-g_t), s>=t
    kk = kc @ kc.transpose(-1, -2)
    # (I + strict_lower(diag(beta) K K^T * decay))^-1, i.e. ref_gdr.py:100-109 + :116-140
    L = (bc[..., :, None] * kk * decay).tril(-1)
    eye = torch.eye(C, dtype=q.dtype).expand_as(L)
    A = torch.linalg.solve_triangular(eye + L, eye, upper=False)
    gamma = gc.exp()
    w = A @ (kc * (bc * gamma)[..., None])  # ref_gdr.py:165-175
    u = A @ (vc * bc[..., None])
    attn = scale * (qc @ kc.transpose(-1, -2)) * decay  # ref_gdr.py:281-292
    g_last = gc[..., -1]
    k_tail = kc * (g_last[..., None] - gc).exp()[..., None]  # ref_gdr.py:230

    hs, os_ = [], []
    for i in range(n):
        hs.append(S)
        v_new = u[i] - w[i] @ S  # ref_gdr.py:225
        os_.append(scale * (qc[i] * gamma[i][..., None]) @ S + attn[i] @ v_new)  # :293-294
        S = S * g_last[i].exp()[:, None, None] + k_tail[i].transpose(-1, -2) @ v_new  # :227-232
    o = torch.stack(os_).transpose(1, 2).reshape(n * C, H, V)[:T]
    g_cum = gc.transpose(1, 2).reshape(n * C, H)[:T]
    A_rows = A.transpose(1, 2).reshape(n * C, H, C)[:T]
    return g_cum, A_rows, o, torch.stack(hs), S


def chunk_gdr_fwd(q, k, v, g, beta, scale=None, initial_state=None, cu_seqlens=None,
                  chunk_size=CHUNK):
    """Chunked forward.  Returns ``(g_cum, A, o, h, final_state)`` with ``A`` the *gated*
    inverse (row t of the tensor is row ``t mod C`` of its chunk's matrix) and ``h`` the state
    entering each chunk, ``[B, NT, Hv, K, V]`` (varlen: ``[1, total chunks, Hv, K, V]``)."""
    B, T, Hv, V = v.shape
    K = q.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    qe, ke = _expand_heads(q, Hv), _expand_heads(k, Hv)
    g_out, A_out, o_out, h_out, finals = [], [], [], [], []
    for n, (b, s, e) in enumerate(_seq_bounds(B, T, cu_seqlens)):
        S0 = (
            torch.zeros(Hv, K, V, dtype=v.dtype)
            if initial_state is None
            else initial_state[n].to(v.dtype)
        )
        if e == s:  # zero-length sequence: no rows, no chunks, the state passes through
            finals.append(S0)
            g_out.append(g[b, s:e]), A_out.append(g.new_zeros(0, Hv, chunk_size))
            o_out.append(v[b, s:e]), h_out.append(v.new_zeros(0, Hv, K, V))
            continue
        gc, A, o, h, S = _chunk_one_sequence(
            qe[b, s:e], ke[b, s:e], v[b, s:e], g[b, s:e], beta[b, s:e], scale, S0, chunk_size
        )
        g_out.append(gc), A_out.append(A), o_out.append(o), h_out.append(h), finals.append(S)
    if cu_seqlens is None:
        stack = torch.stack
    else:
        def stack(xs):
            return torch.cat(xs).unsqueeze(0)
    return stack(g_out), stack(A_out), stack(o_out), stack(h_out), torch.stack(finals)


def chunk_gdr_bwd(q, k, v, g, beta, do, dht=None, scale=None, initial_state=None,
                  cu_seqlens=None, chunk_size=CHUNK):
    """Gradients of ``sum(o*do) + sum(final_state*dht)`` with respect to the *raw* inputs
    ``(q, k, v, beta, g, initial_state)``; ``g`` here is the raw per-token log gate (not its
    cumsum).  Same six results, in the same order, as ``tests/ref_gdr.py:661-746``."""
    leaves = [x.detach().clone().requires_grad_(True) for x in (q, k, v, beta, g)]
    h0 = None if initial_state is None else initial_state.detach().clone().requires_grad_(True)
    ql, kl, vl, bl, gl = leaves
    _, _, o, _, ht = chunk_gdr_fwd(ql, kl, vl, gl, bl, scale, h0, cu_seqlens, chunk_size)
    loss = (o * do[:, : o.shape[1]]).sum()  # rows past the last packed sequence carry no loss
    if dht is not None:
        loss = loss + (ht * dht).sum()
    wanted = leaves + ([h0] if h0 is not None else [])
    grads = torch.autograd.grad(loss, wanted)
    dq, dk, dv, db, dg = grads[:5]
    dh0 = grads[5] if h0 is not None else None
    return dq, dk, dv, db, dg, dh0


def make_inputs(B, T, Hq, Hv, K, V, seed, cu_seqlens=None, with_h0=True, dtype=torch.float32,
                round_to=torch.bfloat16, gate="logsigmoid"):
    """Seeded synthetic inputs with the value distributions of the benchmark configurations:
    q, k ~ N(0,1) L2-normalised over K; v ~ N(0,1); g = logsigmoid(N(0,1)); beta =
    sigmoid(N(0,1)); h0 ~ 0.1 N(0,1); do ~ N(0,1); dht ~ 0.1 N(0,1).  q, k, v, beta, do are
    rounded through ``round_to`` so that a bf16 kernel sees exactly the same numbers.
    ``gate="hard"`` uses the reference tests' per-head ``-A softplus`` gate with one
    decay-free head and one extreme-decay head (reference ``tests/test_gdr_unit.py:107-115``)."""
    gen = torch.Generator().manual_seed(seed)

    def rn(*shape):
        return torch.randn(*shape, generator=gen, dtype=torch.float32)

    def rt(x):
        return (x.to(round_to) if round_to is not None else x).to(dtype)

    q = rt(torch.nn.functional.normalize(rn(B, T, Hq, K), dim=-1))
    k = rt(torch.nn.functional.normalize(rn(B, T, Hq, K), dim=-1))
    v = rt(rn(B, T, Hv, V))
    if gate == "logsigmoid":
        g = torch.nn.functional.logsigmoid(rn(B, T, Hv)).to(dtype)
    elif gate == "hard":
        a = torch.rand(Hv, generator=gen) * 16
        a[0], a[-1] = 0.0, 16.0
        g = (-a * torch.nn.functional.softplus(rn(B, T, Hv) * 0.5 + 1.0)).to(dtype)
    elif gate == "weak":  # reference benchmark recipe: slow decay, a quarter of heads gate-free
        g = torch.nn.functional.logsigmoid(rn(B, T, Hv)) / 16
        g[..., : max(Hv // 4, 1)] = 0
        g = g.to(dtype)
    else:
        raise ValueError(gate)
    beta = rt(torch.sigmoid(rn(B, T, Hv)))
    N = B if cu_seqlens is None else len(cu_seqlens) - 1
    h0 = (0.1 * rn(N, Hv, K, V)).to(dtype) if with_h0 else None
    do = rt(rn(B, T, Hv, V))
    dht = (0.1 * rn(N, Hv, K, V)).to(dtype)
    return dict(q=q, k=k, v=v, g=g, beta=beta, h0=h0, do=do, dht=dht)


def rel_err(x, ref):
    """Normalised error ``||x - ref|| / ||ref||`` in fp64 (the parity metric)."""
    x, ref = x.detach().double().cpu(), ref.detach().double().cpu()
    return float((x - ref).norm() / ref.norm().clamp_min(1e-30))
