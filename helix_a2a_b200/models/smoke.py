"""Tiny end-to-end check on one GPU: exchange + fused combine with every rank played by one launch."""
from __future__ import annotations

import torch


def run() -> None:
    import helix_a2a_b200 as helix
    from helix_a2a_b200.ops import reference_math as rm
    from helix_a2a_b200.ops._ext import ops
    torch.cuda.set_device(0)
    cp, B, H, D = 2, 4, 16, 128
    ws = helix.allocate_workspace(cp, 0)
    helix.init_workspace_all_rows(ws, cp)
    outs = torch.randn(cp, B, H, D, device="cuda").bfloat16()
    lses = torch.randn(cp, B, H, device="cuda")
    got, _ = ops().alltoall_combine(outs, lses, ws, 0, cp, 0, False, False, 0, True, 0, 0)
    torch.cuda.synchronize()
    want = rm.head_scatter_combine_reference(outs, lses)
    err = (got.float() - want).abs().max().item()
    assert err < 2e-2, err
    print(f"smoke ok: exchange+combine max err {err:.3e}")
