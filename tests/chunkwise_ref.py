"""fp64 torch model of the chunkwise algebra (test infrastructure): the per-chunk quantities the
chunk-parallel CUDA stage writes, used to check that stage on its own, and helpers that decode the
swizzled tile pack."""
import torch

BT = 64
TP = dict(W=0, QG=16384, KG=32768, AQK=49152, DECAY=57344, U0=57856, U1=66048, BYTES=74240)


def unswizzle(raw, rows, cols, dtype):
    """raw: uint8 tensor [..., rows*cols*2] holding a 2-byte matrix whose 16-byte column groups are
    XOR-swizzled by (row & 7). Returns [..., rows, cols] in `dtype`."""
    m = raw.reshape(*raw.shape[:-1], rows, cols // 8, 16)
    r = torch.arange(rows, device=raw.device).view(rows, 1)
    c = torch.arange(cols // 8, device=raw.device).view(1, -1)
    phys = (c ^ (r & 7)).expand(rows, cols // 8)
    idx = phys.reshape(*([1] * (m.dim() - 3)), rows, cols // 8, 1).expand(*m.shape)
    return torch.gather(m, -2, idx).reshape(*raw.shape[:-1], rows, cols * 2).contiguous().view(dtype)


def decode_tiles(tiles, n_tiles):
    t = tiles.view(n_tiles, TP["BYTES"])
    out = dict(
        w=unswizzle(t[:, TP["W"]:TP["QG"]], 64, 128, torch.float16).float(),
        qg=unswizzle(t[:, TP["QG"]:TP["KG"]], 64, 128, torch.float16).float(),
        kg=unswizzle(t[:, TP["KG"]:TP["AQK"]], 64, 128, torch.float16).float(),
        aqk=unswizzle(t[:, TP["AQK"]:TP["DECAY"]], 64, 64, torch.float16).float(),
        decay=t[:, TP["DECAY"]:TP["U0"]].contiguous().view(torch.float32),
    )
    u0 = unswizzle(t[:, TP["U0"]:TP["U1"]], 64, 64, torch.float16).float()
    u1 = unswizzle(t[:, TP["U1"]:TP["BYTES"]], 64, 64, torch.float16).float()
    out["u"] = torch.cat([u0, u1], dim=-1)
    return out


def chunk_quantities(q, k, v, a, beta, scale):
    """One sequence, one head. q,k [T,K] (already normalised), v [T,V], a [T,K] natural-log decay,
    beta [T]; all float64. Returns per-chunk lists padded to 64 rows with zeros."""
    T, K = q.shape
    out = []
    for s in range(0, T, BT):
        n = min(BT, T - s)
        pad = lambda x: torch.cat([x[s:s + n], x.new_zeros(BT - n, *x.shape[1:])])
        qc, kc, vc, bc = pad(q), pad(k), pad(v), pad(beta)
        G = torch.cumsum(pad(a), 0)          # padding rows add 0 -> repeat the last real value
        glast = G[-1]
        diff = G[:, None, :] - G[None, :, :]                 # [i, j, d]
        mask_le = torch.tril(torch.ones(BT, BT, dtype=torch.bool))
        E = torch.where(mask_le[:, :, None], diff, torch.zeros_like(diff)).exp() * mask_le[:, :, None]
        P = torch.einsum("id,jd,ijd->ij", qc, kc, E)
        Lm = torch.einsum("id,jd,ijd->ij", kc, kc, E)
        aqk = scale * torch.tril(P)
        L = torch.tril(bc[:, None] * Lm, -1)
        akk = torch.linalg.inv(torch.eye(BT, dtype=q.dtype) + L)
        w = akk @ (bc[:, None] * kc * G.exp())
        u = akk @ (bc[:, None] * vc)
        kg = kc * (glast[None] - G).exp()
        qg = scale * qc * G.exp()
        out.append(dict(w=w, u=u, kg=kg, qg=qg, aqk=aqk, decay=glast.exp(), akk=akk))
    return out


# -------------------------------------------------------------------------------------------------
# fp64 model of the chunkwise forward + backward for ONE (sequence, head): the executable
# specification the backward kernels are checked against, itself checked against autograd of the
# token recurrence in tests/test_chunkwise_model.py.
# -------------------------------------------------------------------------------------------------
def chunk_forward_backward(q, k, v, a, beta, scale, h0, do, dht):
    """q,k [T,K] normalised; v [T,V]; a [T,K] natural-log decay; beta [T]; h0 [K,V]; do [T,V]; dht [K,V].
    Returns dict with o, ht, per-chunk intermediates and gradients w.r.t. q,k,v,a,beta,h0."""
    T, K = q.shape
    V = v.shape[1]
    dt = q.dtype
    nchunks = (T + BT - 1) // BT
    eye = torch.eye(BT, dtype=dt)
    tril = torch.tril(torch.ones(BT, BT, dtype=torch.bool))
    stril = torch.tril(torch.ones(BT, BT, dtype=torch.bool), -1)
    fw = []
    S = h0.clone()
    o = torch.zeros(T, V, dtype=dt)
    for c in range(nchunks):
        s0, n = c * BT, min(BT, T - c * BT)
        pad = lambda x: torch.cat([x[s0:s0 + n], x.new_zeros(BT - n, *x.shape[1:])])
        qc, kc, vc, bc = pad(q), pad(k), pad(v), pad(beta)
        G = torch.cumsum(pad(a), 0)
        glast = G[-1]
        diff = G[:, None, :] - G[None, :, :]
        E = torch.where(tril[:, :, None], diff, torch.zeros_like(diff)).exp() * tril[:, :, None]   # e^{G_i-G_j}, j<=i
        P = torch.einsum("id,jd,ijd->ij", qc, kc, E)
        M = torch.einsum("id,jd,ijd->ij", kc, kc, E)
        Aqk = scale * P * tril
        L = bc[:, None] * M * stril
        A = torch.linalg.inv(eye + L)
        X = bc[:, None] * kc * G.exp()
        Y = bc[:, None] * vc
        W, U = A @ X, A @ Y
        Kg = kc * (glast[None] - G).exp()
        Qg = scale * qc * G.exp()
        D = glast.exp()
        Vn = U - W @ S
        oc = Qg @ S + Aqk @ Vn
        o[s0:s0 + n] = oc[:n]
        fw.append(dict(n=n, s0=s0, qc=qc, kc=kc, vc=vc, bc=bc, G=G, E=E, P=P, M=M, Aqk=Aqk, L=L, A=A, X=X, Y=Y, W=W,
                       U=U, Kg=Kg, Qg=Qg, D=D, Vn=Vn, S=S.clone()))
        S = D[:, None] * S + Kg.T @ Vn
    ht = S
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    da, dbeta = torch.zeros_like(a), torch.zeros_like(beta)
    dSn = dht.clone()                     # gradient w.r.t. the state leaving the current chunk
    inter = [None] * nchunks
    for c in reversed(range(nchunks)):
        f = fw[c]
        n, s0 = f["n"], f["s0"]
        dO = torch.cat([do[s0:s0 + n], do.new_zeros(BT - n, V)])
        # (B1)+(B2): reverse scan
        dVn = f["Kg"] @ dSn + f["Aqk"].T @ dO
        dS_in = f["D"][:, None] * dSn + f["Qg"].T @ dO - f["W"].T @ dVn
        # (B3) dense part
        dQg = dO @ f["S"].T
        dKg = f["Vn"] @ dSn.T
        dD = (f["S"] * dSn).sum(1)
        dW = -dVn @ f["S"].T
        Zu = f["A"].T @ dVn
        Zw = f["A"].T @ dW
        dA = (dVn @ f["Y"].T + dW @ f["X"].T) * stril
        dL = -(f["A"].T @ dA @ f["A"].T) * stril
        dPs = (dO @ f["Vn"].T) * tril          # gradient w.r.t. Aqk
        dvc = f["bc"][:, None] * Zu
        dbc = (Zu * f["vc"]).sum(1) + (Zw * f["kc"] * f["G"].exp()).sum(1) + (dL * f["M"]).sum(1)
        # (B4) gated Gram VJPs with pairwise factors E_ijd = e^{G_i - G_j}
        dP = scale * dPs
        R = f["bc"][:, None] * dL
        qc, kc, E, G = f["qc"], f["kc"], f["E"], f["G"]
        dq_P = torch.einsum("ij,jd,ijd->id", dP, kc, E)
        dk_Pj = torch.einsum("ij,id,ijd->jd", dP, qc, E)
        dk_Ri = torch.einsum("ij,jd,ijd->id", R, kc, E)
        dk_Rj = torch.einsum("ij,id,ijd->jd", R, kc, E)
        eG, eKg = G.exp(), (f["G"][-1][None] - G).exp()
        dkp = f["bc"][:, None] * Zw                         # gradient w.r.t. K+ = k e^G coming through X
        dqc = scale * dQg * eG + dq_P
        dkc = dkp * eG + dKg * eKg + dk_Pj + dk_Ri + dk_Rj
        dG = dQg * f["Qg"] + qc * dq_P + dkp * kc * eG + kc * dk_Ri - kc * dk_Pj - kc * dk_Rj - dKg * f["Kg"]
        dglast = (dKg * f["Kg"]).sum(0) + f["D"] * dD
        dG[BT - 1] += dglast          # padding rows repeat the last real value, so row 63 carries g_last ...
        dac = torch.flip(torch.cumsum(torch.flip(dG, [0]), 0), [0])    # ... and the reverse cumsum folds it back
        dq[s0:s0 + n], dk[s0:s0 + n], dv[s0:s0 + n] = dqc[:n], dkc[:n], dvc[:n]
        da[s0:s0 + n], dbeta[s0:s0 + n] = dac[:n], dbc[:n]
        inter[c] = dict(dVn=dVn, dSn=dSn.clone(), dQg=dQg, dKg=dKg, dD=dD, Zu=Zu, Zw=Zw, dL=dL, dPs=dPs, dG=dG)
        dSn = dS_in
    return dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, da=da, dbeta=dbeta, dh0=dSn, fw=fw, bw=inter)
