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
