"""Helpers for the GPU parity tests: run one link-prediction step through the C ABI on a workloads.BatchCase."""
from __future__ import annotations

import numpy as np
import torch


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-30))


def dev(a, device, dtype=None):
    if a is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(device)


def run_lp_step(capi, case, device, precision="fp32", filter_mode="pairs", indirect=False, dump_scores=True):
    """Returns a dict of numpy outputs.  filter_mode: 'pairs' | 'deg_rows' | 'none'.  indirect: node_emb is a larger table
    addressed through row_index (the fused pipeline's way)."""
    B, C, N, D, R, U = case.dims
    has_rel = case.rel is not None
    S = 2 if (has_rel and case.inv_rel is not None and case.src_negs is not None) else 1
    npc = -(-B // C)
    Bp = npc * C
    edges = dev(case.edges, device)
    emb_np = case.emb
    row_index = None
    if indirect:
        rng = np.random.default_rng(1234)
        rows = rng.permutation(U * 3)[:U].astype(np.int64)
        table = np.zeros((U * 3, D), np.float32)
        table[rows] = case.emb
        emb_np = table
        row_index = dev(rows, device)
    emb = dev(emb_np, device)
    out = dict(
        node_grad=torch.full((U, D), 7.0, device=device),  # must be overwritten
        loss=torch.full((1,), -1.0, device=device),
        status=torch.zeros(1, dtype=torch.int32, device=device),
    )
    rel = dev(case.rel, device)
    inv_rel = dev(case.inv_rel, device)
    rel_grad = torch.zeros((R, D), device=device) if has_rel else None
    inv_rel_grad = torch.zeros((R, D), device=device) if S == 2 else None
    if dump_scores:
        out["pos_scores"] = torch.zeros(Bp, device=device)
        out["neg_scores"] = torch.zeros((Bp, N), device=device)
        if S == 2:
            out["inv_pos_scores"] = torch.zeros(Bp, device=device)
            out["inv_neg_scores"] = torch.zeros((Bp, N), device=device)
    filt = dev(case.filt, device) if (filter_mode == "pairs" and len(case.filt)) else None
    deg_rows = dev(case.deg_rows, device) if (filter_mode == "deg_rows" and case.deg_rows is not None) else None
    cols = case.edges.shape[1]
    dst_negs, src_negs = dev(case.dst_negs, device), dev(case.src_negs, device) if S == 2 else None
    d = capi.make_lp_desc(
        decoder=case.kind, precision=precision, B=B, Cn=C, N=N, D=D, R=max(R, 0), U=U, node_emb=emb, row_index=row_index,
        src_ids=edges, dst_ids=edges[:, cols - 1], rel_ids=edges[:, 1] if has_rel else None, edge_stride=cols, rel_stride=cols,
        dst_negs=dst_negs, src_negs=src_negs, dst_filter=filt, src_filter=filt if S == 2 else None,
        deg_sample_rows=deg_rows, n_deg=0 if deg_rows is None else deg_rows.shape[1], rel=rel, inv_rel=inv_rel if S == 2 else None,
        node_grad=out["node_grad"], rel_grad=rel_grad, inv_rel_grad=inv_rel_grad, loss=out["loss"],
        pos_scores=out.get("pos_scores"), neg_scores=out.get("neg_scores"), inv_pos_scores=out.get("inv_pos_scores"),
        inv_neg_scores=out.get("inv_neg_scores"), status=out["status"])
    ws = torch.empty(capi.lp_workspace_bytes(d), dtype=torch.uint8, device=device)
    d.workspace, d.workspace_bytes = ws.data_ptr(), ws.numel()
    capi.lp_step(d)
    torch.cuda.synchronize()
    res = {k: v.cpu().numpy() for k, v in out.items()}
    if rel_grad is not None:
        res["rel_grad"] = rel_grad.cpu().numpy()
    if inv_rel_grad is not None:
        res["inv_rel_grad"] = inv_rel_grad.cpu().numpy()
    res["loss"] = float(res["loss"][0])
    res["status"] = int(res["status"][0])
    return res
