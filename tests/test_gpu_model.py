"""Decode stack on one GPU: kernels chained by PDL and replayed from a CUDA graph give the eager result,
and the result matches the fp32 oracle."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_decode_stack_matches_oracle_and_graph_pdl_replay(native_built):
    from helix_a2a_b200.models.llama_decode import HelixDecodeStack, LlamaDecodeConfig
    from helix_a2a_b200.ops import reference_math as rm
    from helix_a2a_b200.ops.oproj import check_compute_status
    cfg = LlamaDecodeConfig.tiny(n_layers=3, hidden=512)
    stack = HelixDecodeStack(cfg, batch=3, local_ctx=1000, device="cuda")
    q = torch.randn(cfg.n_layers, 3, cfg.n_q_heads, cfg.head_dim, device="cuda").bfloat16()
    y = stack.decode_step(q)
    for l in range(cfg.n_layers):
        o, _ = rm.paged_decode_attention_reference(q[l].float(), stack.k_cache[l].float(), stack.v_cache[l].float(),
                                                   stack.block_table, stack.seq_lens, stack.scale)
        ref = rm.oproj_reference(o.reshape(3, -1), stack.w_o[l])
        assert (y[l].float() - ref).abs().max() < 3e-2
    eager_last = stack.decode_step_device(q).clone()
    os.environ["HELIX_A2A_ENABLE_PDL"] = "1"
    try:
        stack.capture(q)
        for _ in range(3):
            got = stack.decode_step_device(q)
        torch.cuda.synchronize()
        assert torch.equal(got, eager_last)
        pinned = q.cpu().pin_memory()
        host = stack.decode_step_host(pinned)
        assert torch.equal(host.cuda(), eager_last)
    finally:
        del os.environ["HELIX_A2A_ENABLE_PDL"]
    check_compute_status(q)
