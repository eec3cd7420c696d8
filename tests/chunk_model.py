"""CPU model of the chunked (WY / UT-transform) PKDA pipeline, stage by stage.

TEST INFRASTRUCTURE.  The CUDA kernels in
``delta_feedback_experiment_b200/csrc`` implement exactly these stages; this
file restates them with plain torch matrix operations for one (row, head) at a
time so that (a) the algebra -- including the hand-derived backward -- can be
checked against the autograd oracle on the CPU, (b) the effect of rounding the
intermediates to bf16 can be measured without a GPU, and (c) GPU tests can
compare individual kernel outputs with the matching stage here.

Notation for one chunk of C tokens with entry state S0 [K,V]:
  G      chunk-local cumulative log-decay [C,K];  Gam = exp(G)
  M[i,j] = sum_c k[i,c] kt[j,c] exp(G[i,c]-G[j,c])   (i>j)
  P[i,j] = sum_c q[i,c] kt[j,c] exp(G[i,c]-G[j,c])   (i>=j)
  Tm     = (I + tril(M,-1) diag(beta))^-1
  W = Tm (k*Gam),  U = Tm v,  E = U - W S0,  F = beta*E
  O = s (q*Gam) S0 + s P F
  S1 = diag(Gam[last]) S0 + (kt*exp(G[last]-G))^T F
where kt is the preconditioned write key.  exp(G_i - G_j) is never formed from
exp(G_i)*exp(-G_j) (overflow); ``gated_pairs`` uses a binary hierarchy of
reference points so every factor is <= 1.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

C = 64
LEVELS = (32, 16, 8, 4, 2, 1)


def rnd(t, dtype):
    """Round through a storage dtype (None = keep)."""
    return t if dtype is None else t.to(dtype).to(t.dtype)


def level_factors(G, lvl):
    """Row factor exp(G_i - G_ref) for rows in the upper half of their 2*lvl
    block, column factor exp(G_ref - G_j) for rows in the lower half; zero
    elsewhere.  ref = first row of the upper half."""
    n = G.shape[0]
    idx = torch.arange(n)
    ref = (idx // (2 * lvl)) * (2 * lvl) + lvl
    upper = (idx & lvl) != 0
    refc = ref.clamp(max=n - 1)
    Gref = G[refc]
    rowf = torch.where(upper[:, None], torch.exp(G - Gref), torch.zeros_like(G))
    # columns whose reference lies beyond the chunk never pair with a valid row
    colok = (~upper) & (ref < n)
    colf = torch.where(colok[:, None], torch.exp(Gref - G), torch.zeros_like(G))
    return rowf, colf


def level_mask(n, lvl):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return ((i // (2 * lvl)) == (j // (2 * lvl))) & ((i & lvl) != 0) & ((j & lvl) == 0)


DIRECT = 1
"""Direct block size b (a power of two, 1..64): pairs inside the same b-block use
one reference row (the block's first row) instead of hierarchy levels < b.  Only
valid while the decay across a b-block stays far inside the exponent range; the
kernels pick the largest admissible b per (chunk, head)."""


def direct_factors(G, b):
    n = G.shape[0]
    ref = (torch.arange(n) // b) * b
    Gref = G[ref]
    return torch.exp(G - Gref), torch.exp(Gref - G)


def direct_mask(n, b):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return ((i // b) == (j // b)) & (j < i)


def gated_pairs(X, Y, G, diag, op_dtype=None):
    """sum_c X[i,c] Y[j,c] exp(G[i,c]-G[j,c]) for i>j (and i==j if diag)."""
    n = X.shape[0]
    out = torch.zeros(n, n, dtype=X.dtype)
    if DIRECT > 1:
        rowf, colf = direct_factors(G, DIRECT)
        out += torch.where(direct_mask(n, DIRECT),
                           rnd(X * rowf, op_dtype) @ rnd(Y * colf, op_dtype).T, 0.0)
    for lvl in LEVELS:
        if lvl >= n or lvl < DIRECT:
            continue
        rowf, colf = level_factors(G, lvl)
        out += torch.where(level_mask(n, lvl),
                           rnd(X * rowf, op_dtype) @ rnd(Y * colf, op_dtype).T, 0.0)
    if diag:
        out += torch.diag((rnd(X, op_dtype) * rnd(Y, op_dtype)).sum(-1))
    return out


def gated_pairs_bwd(dOut, X, Y, G, diag, op_dtype=None):
    """Given d(out) (already masked to the valid triangle) returns
    dX[i] = sum_j dOut[i,j] Y[j] e^{G_i-G_j},  dY[j] = sum_i dOut[i,j] X[i] e^{G_i-G_j}
    and the matching contribution to dG, X*dX - Y*dY, formed from the SAME
    rounded operands on both sides so that each pair's +/- terms cancel exactly
    under the later reverse cumulative sum."""
    n = X.shape[0]
    dX = torch.zeros_like(X)
    dY = torch.zeros_like(Y)
    dG = torch.zeros_like(X)
    for lvl in (0,) + LEVELS:
        if lvl == 0:
            if DIRECT <= 1:
                continue
            rowf, colf = direct_factors(G, DIRECT)
            mask = direct_mask(n, DIRECT)
        else:
            if lvl >= n or lvl < DIRECT:
                continue
            rowf, colf = level_factors(G, lvl)
            mask = level_mask(n, lvl)
        dm = rnd(torch.where(mask, dOut, 0.0), op_dtype)
        Xl, Yl = rnd(X * rowf, op_dtype), rnd(Y * colf, op_dtype)
        dXl = dm @ Yl
        dYl = dm.T @ Xl
        dX += rowf * dXl
        dY += colf * dYl
        dG += Xl * dXl - Yl * dYl
    if diag:
        d = torch.diagonal(dOut)[:, None]
        dX += d * Y
        dY += d * X
    return dX, dY, dG


def log_decay(raw, a_log, dt_bias):
    """g = -exp(A_log) softplus(raw + dt_bias) for one head: raw [T,K]."""
    return -math.exp(float(a_log)) * F.softplus(raw + dt_bias)


def atk_forward(k, gP, bP, c, x, eps, A0):
    """Preconditioner scan for one (row, head): returns write keys kt [T,K],
    the state A before every token [T,K] and the final state."""
    T, K = k.shape
    A = A0.clone()
    kt = torch.empty_like(k)
    Aprev = torch.empty_like(k)
    lnx = math.log(x)
    for t in range(T):
        Aprev[t] = A
        A = torch.exp(gP[t]) * A + bP[t] * k[t] * k[t]
        dev = torch.log(A + eps) - c
        kt[t] = k[t] * torch.exp(-lnx * dev / (1 + dev.abs()))
    return kt, Aprev, A


def atk_backward(dkt, k, gP, bP, c, x, eps, A0):
    """Reverse scan: gradients of k (through the write key), gP, bP, c, A0."""
    T, K = k.shape
    _, Aprev, _ = atk_forward(k, gP, bP, c, x, eps, A0)
    lnx = math.log(x)
    lam = torch.zeros(K, dtype=k.dtype)  # d loss / d A_t carried from later tokens
    dk = torch.zeros_like(k)
    dgP = torch.zeros(T, dtype=k.dtype)
    dbP = torch.zeros(T, dtype=k.dtype)
    dc = torch.zeros((), dtype=k.dtype)
    for t in reversed(range(T)):
        dec = torch.exp(gP[t])
        A = dec * Aprev[t] + bP[t] * k[t] * k[t]
        dev = torch.log(A + eps) - c
        Bf = torch.exp(-lnx * dev / (1 + dev.abs()))
        dk[t] += dkt[t] * Bf
        ddev = (-lnx) * dkt[t] * k[t] * Bf / (1 + dev.abs()) ** 2
        dc -= ddev.sum()
        lam = lam + ddev / (A + eps)
        dbP[t] = (lam * k[t] * k[t]).sum()
        dk[t] += 2 * lam * bP[t] * k[t]
        dgP[t] = (lam * dec * Aprev[t]).sum()
        lam = lam * dec
    return dk, dgP, dbP, dc, lam


def chunk_forward(q, k, v, raw, gP, bP, beta, a_log, dt_bias, c, scale, x, eps,
                  S0, A0, act=None, keep=False):
    """Forward for one (row, head).  ``act`` = storage dtype of intermediates
    that the kernels keep in bf16 (None: exact).  Returns (o, S_T, A_T, saved)."""
    T, K = q.shape
    V = v.shape[1]
    dt = q.dtype
    kt_full, _, A_T = atk_forward(k, gP, bP, c, x, eps, A0)
    kt_full = rnd(kt_full, act)
    g = log_decay(raw, a_log, dt_bias)
    S = S0.clone()
    o = torch.empty(T, V, dtype=dt)
    saved = []
    for lo in range(0, T, C):
        hi = min(T, lo + C)
        n = hi - lo
        Q, Kc, Kt, Vc, b = q[lo:hi], k[lo:hi], kt_full[lo:hi], v[lo:hi], beta[lo:hi]
        G = torch.cumsum(g[lo:hi], 0)
        Gam = torch.exp(G)
        M = gated_pairs(Kc, Kt, G, False, act)
        P = gated_pairs(Q, Kt, G, True, act) * scale
        L = torch.tril(M, -1) * b[None, :]
        Tm = torch.linalg.solve_triangular(torch.eye(n, dtype=dt) + L,
                                           torch.eye(n, dtype=dt), upper=False)
        Tm_s, P_s = rnd(Tm, act), rnd(P, act)
        W = rnd(Tm_s @ rnd(Kc * Gam, act), act)
        U = rnd(Tm_s @ rnd(Vc, act), act)
        Kg = rnd(Kt * torch.exp(G[-1:] - G), act)
        Qd = rnd(Q * Gam * scale, act)
        gC = Gam[-1]
        # ---- sequential part
        h = rnd(S, act)
        E = rnd(U - W @ h, act)
        Fm = rnd(b[:, None] * E, act)
        o[lo:hi] = Qd @ h + P_s @ Fm
        S = gC[:, None] * S + Kg.T @ Fm
        if keep:
            saved.append(dict(lo=lo, hi=hi, G=G, Tm=Tm_s, P=P_s, W=W, U=U, Kg=Kg, Qd=Qd,
                              gC=gC, h=h, E=E, Kt=Kt))
    return o, S, A_T, saved


def chunk_backward(do, dS_T, q, k, v, raw, gP, bP, beta, a_log, dt_bias, c, scale, x,
                   eps, S0, A0, act=None):
    """Hand-derived backward for one (row, head); mirrors the two backward
    kernels (reverse state scan, then the chunk-parallel part) and the two
    elementwise tails (gate, preconditioner)."""
    T, K = q.shape
    dt = q.dtype
    _, _, _, saved = chunk_forward(q, k, v, raw, gP, bP, beta, a_log, dt_bias, c, scale, x,
                                   eps, S0, A0, act, keep=True)
    g = log_decay(raw, a_log, dt_bias)
    dS = dS_T.clone()
    dq = torch.zeros_like(q)
    dk = torch.zeros_like(k)
    dkt = torch.zeros_like(k)
    dv = torch.zeros_like(v)
    dbeta = torch.zeros_like(beta)
    dg = torch.zeros_like(g)
    do_s = rnd(do, act)
    # ---- reverse scan over chunks
    for ch in reversed(saved):
        lo, hi = ch["lo"], ch["hi"]
        b = beta[lo:hi]
        dSC = rnd(dS, act)
        ch["dSC"] = dSC
        dF = rnd(ch["Kg"] @ dSC + ch["P"].T @ do_s[lo:hi], act)
        ch["dF"] = dF
        dE = rnd(b[:, None] * dF, act)
        dS = ch["gC"][:, None] * dS + ch["Qd"].T @ do_s[lo:hi] - ch["W"].T @ dE
    dS0 = dS
    # ---- chunk-parallel part
    for ch in saved:
        lo, hi = ch["lo"], ch["hi"]
        n = hi - lo
        Q, Kc, Kt, b = q[lo:hi], k[lo:hi], ch["Kt"], beta[lo:hi]
        G, Tm, E, h, dSC, dF = ch["G"], ch["Tm"], ch["E"], ch["h"], ch["dSC"], ch["dF"]
        dO = do_s[lo:hi]
        Gam = torch.exp(G)
        tail = torch.exp(G[-1:] - G)
        Fm = rnd(b[:, None] * E, act)
        dE = rnd(b[:, None] * dF, act)
        dbeta[lo:hi] = (dF * E).sum(-1)
        dQ = scale * Gam * (dO @ h.T)
        dPs = rnd(scale * torch.tril(dO @ Fm.T), act)
        dKt_a = tail * (Fm @ dSC.T)
        dR = Tm.T @ dE
        dv[lo:hi] = dR
        dR_s = rnd(dR, act)
        dK = -Gam * (dR_s @ h.T)
        dLn = rnd(torch.tril(dR_s @ E.T, -1), act)  # dL = -dLn
        # gated products
        dQ_b, dKt_c, dG_p = gated_pairs_bwd(dPs, Q, Kt, G, True, act)
        dM = rnd(-dLn * b[None, :], act)
        dK_b, dKt_b, dG_m = gated_pairs_bwd(dM, Kc, Kt, G, False, act)
        dbeta[lo:hi] += (Kt * dKt_b).sum(-1) / b
        dG = Q * dQ + Kc * dK - Kt * dKt_a + dG_p + dG_m
        dG[-1] += (Kt * dKt_a).sum(0) + ch["gC"] * (h * dSC).sum(-1)
        dQ = dQ + dQ_b
        dK = dK + dK_b
        dKt = dKt_a + dKt_b + dKt_c
        dg[lo:hi] = torch.flip(torch.cumsum(torch.flip(dG, [0]), 0), [0])
        dq[lo:hi] = dQ
        dk[lo:hi] = dK
        dkt[lo:hi] = dKt
    # ---- gate tail
    ea = math.exp(float(a_log))
    draw = dg * (-ea) * torch.sigmoid(raw + dt_bias)
    dA_log = (dg * g).sum()
    ddt_bias = draw.sum(0)
    # ---- preconditioner tail
    dk2, dgP, dbP, dc, dA0 = atk_backward(dkt, k, gP, bP, c, x, eps, A0)
    return dict(dq=dq, dk=dk + dk2, dv=dv, dg=draw, dg_atk=dgP, dbeta_atk=dbP, dbeta=dbeta,
                dA_log=dA_log, ddt_bias=ddt_bias, dlog_atk_scale=dc,
                dinitial_state=dS0, dinitial_A_state=dA0)


def model_forward_backward(inputs, do, scale=None, x=1.5, eps=1e-6, S0=None, A0=None,
                           dS_T=None, act=None, dtype=torch.float64):
    """Whole-tensor driver: loops rows and heads, returns the same dict as
    ``oracle.pkda_oracle.pkda_oracle_with_grads``."""
    q, k, v, raw, gP, bP, beta, A_log, dt_bias, c = [t.to(dtype) for t in inputs]
    B, T, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    do = do.to(dtype)
    res = {n: torch.zeros_like(t) for n, t in
           zip(("dq", "dk", "dv", "dg", "dg_atk", "dbeta_atk", "dbeta", "dA_log", "ddt_bias",
                "dlog_atk_scale"), (q, k, v, raw, gP, bP, beta, A_log, dt_bias, c))}
    res["o"] = torch.zeros(B, T, H, V, dtype=dtype)
    res["final_state"] = torch.zeros(B, H, K, V, dtype=dtype)
    res["final_A_state"] = torch.zeros(B, H, K, dtype=dtype)
    res["dinitial_state"] = torch.zeros(B, H, K, V, dtype=dtype)
    res["dinitial_A_state"] = torch.zeros(B, H, K, dtype=dtype)
    for b in range(B):
        for h in range(H):
            s0 = torch.zeros(K, V, dtype=dtype) if S0 is None else S0[b, h].to(dtype)
            a0 = torch.zeros(K, dtype=dtype) if A0 is None else A0[b, h].to(dtype)
            dst = torch.zeros(K, V, dtype=dtype) if dS_T is None else dS_T[b, h].to(dtype)
            args = (q[b, :, h], k[b, :, h], v[b, :, h], raw[b, :, h], gP[b, :, h], bP[b, :, h],
                    beta[b, :, h], A_log[h], dt_bias.view(H, K)[h], c[h], scale, x, eps, s0, a0)
            o, S, A, _ = chunk_forward(*args, act=act)
            res["o"][b, :, h], res["final_state"][b, h], res["final_A_state"][b, h] = o, S, A
            gr = chunk_backward(do[b, :, h], dst, *args, act=act)
            for n in ("dq", "dk", "dv", "dg", "dg_atk", "dbeta_atk", "dbeta"):
                res[n][b, :, h] = gr[n]
            res["dA_log"][h] += gr["dA_log"]
            res["ddt_bias"].view(H, K)[h] += gr["ddt_bias"]
            res["dlog_atk_scale"][h] += gr["dlog_atk_scale"]
            res["dinitial_state"][b, h] = gr["dinitial_state"]
            res["dinitial_A_state"][b, h] = gr["dinitial_A_state"]
    return res
