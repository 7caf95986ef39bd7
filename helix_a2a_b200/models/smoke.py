"""Tiny end-to-end check on one GPU: a 2-layer Llama-architecture decode stack (attention ->
o_proj) against the fp32 oracle, plus the exchange + fused combine with every rank played by one
launch."""
from __future__ import annotations

import torch


def run() -> None:
    import helix_a2a_b200 as helix
    from helix_a2a_b200.models.llama_decode import HelixDecodeStack, LlamaDecodeConfig
    from helix_a2a_b200.ops import reference_math as rm
    from helix_a2a_b200.ops._ext import ops
    from helix_a2a_b200.ops.oproj import check_compute_status
    torch.cuda.set_device(0)

    cfg = LlamaDecodeConfig.tiny()
    stack = HelixDecodeStack(cfg, batch=2, local_ctx=200, device="cuda")
    q = torch.randn(cfg.n_layers, 2, cfg.n_q_heads, cfg.head_dim, device="cuda").bfloat16()
    y = stack.decode_step(q)
    torch.cuda.synchronize()
    check_compute_status(q)
    for l in range(cfg.n_layers):
        o, _ = rm.paged_decode_attention_reference(q[l].float(), stack.k_cache[l].float(), stack.v_cache[l].float(),
                                                   stack.block_table, stack.seq_lens, stack.scale)
        ref = rm.oproj_reference(o.reshape(2, -1), stack.w_o[l])
        err = (y[l].float() - ref).abs().max().item()
        assert err < 3e-2, err

    cp, B, H, D = 2, 4, 16, 128
    ws = helix.allocate_workspace(cp, 0)
    helix.init_workspace_all_rows(ws, cp)
    outs = torch.randn(cp, B, H, D, device="cuda").bfloat16()
    lses = torch.randn(cp, B, H, device="cuda")
    got, _ = ops().alltoall_combine(outs, lses, ws, 0, cp, 0, False, False, 0, True, 0, 0)
    torch.cuda.synchronize()
    want = rm.head_scatter_combine_reference(outs, lses)
    err2 = (got.float() - want).abs().max().item()
    assert err2 < 2e-2, err2
    print(f"smoke ok: decode stack max err {err:.3e}, exchange+combine max err {err2:.3e}")
