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
        # the step is two graphs and the later layers' queries are copied under the first one: alternate two
        # inputs so that a tail graph that started before its copy landed would show the other input's result
        q2 = torch.randn_like(q)
        pinned2 = q2.cpu().pin_memory()
        want = {0: eager_last}
        for it in range(6):
            host = stack.decode_step_host(pinned2 if it % 2 else pinned)
            if it % 2 and 1 not in want:
                want[1] = host.cuda().clone()
                assert not torch.equal(want[1], eager_last)
            assert torch.equal(host.cuda(), want[it % 2])
    finally:
        del os.environ["HELIX_A2A_ENABLE_PDL"]
    check_compute_status(q)


def test_mla_decode_stack_matches_oracle(native_built):
    from helix_a2a_b200.models.deepseek_mla_decode import MlaDecodeConfig, MlaDecodeStack
    from helix_a2a_b200.ops import reference_math as rm
    cfg = MlaDecodeConfig.tiny()
    stack = MlaDecodeStack(cfg, batch=2, local_ctx=300, device="cuda")
    qn = (torch.randn(cfg.n_layers, 2, 128, 512, device="cuda") * 0.3).bfloat16()
    qp = (torch.randn(cfg.n_layers, 2, 128, 64, device="cuda") * 0.3).bfloat16()
    y = stack.decode_step(qn, qp)
    l = cfg.n_layers - 1
    lat = rm.dequantize_fp8_blockscaled(stack.ckv[l], stack.scales[l], 128)
    outs = []
    for b in range(2):
        idx = stack.block_table[b].long()
        c = lat[idx].reshape(-1, 512)[:300]
        k = stack.kpe[l][idx].reshape(-1, 64)[:300].float()
        o, _ = rm.mla_partial_attention(qn[l, b:b + 1].float(), qp[l, b:b + 1].float(), c, k, stack.scale)
        outs.append(o)
    ref = rm.oproj_reference(torch.cat(outs).reshape(2, -1).bfloat16(), stack.w_o[l])
    assert (y.float() - ref).abs().max() < 5e-2 * max(1.0, ref.abs().max().item())
