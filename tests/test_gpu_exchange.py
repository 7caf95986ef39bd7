"""Exchange / fused combine on ONE GPU: a single cooperative launch plays every rank.

All workspace rows live in one tensor, so the multi-rank protocol (LL128 lines, ring wrap,
flow control, bounded waits) runs exactly as between GPUs, with local stores in place of
NVLink stores.  Numerics are checked against the fp32 oracles.
"""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def helix(native_built):
    import helix_a2a_b200 as h
    from helix_a2a_b200.ops._ext import ext
    ext()
    return h


def _ws(helix, cp):
    ws = helix.allocate_workspace(cp, 0)
    helix.init_workspace_all_rows(ws, cp)
    return ws


def _ops():
    return torch.ops.helix_a2a_b200


def test_workspace_size_matches_sm_count(helix):
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    for cp in (2, 4, 8):
        ch = max(sm // (((cp + 7) // 8) * 2), 1)
        assert helix.workspace_size(cp) == 512 * 1024 * cp * ch + 2 * 256 * cp * ch


def test_init_pattern(helix):
    cp = 4
    ws = helix.allocate_workspace(cp, 0)
    helix.init_workspace(ws, 0, cp)
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    ch = max(sm // 2, 1)
    fifo_u64 = 512 * 1024 * cp * ch // 8
    assert (ws[0, :fifo_u64] == -1).all()
    assert (ws[0, fifo_u64:] == 0).all()
    assert (ws[1] == 0).all()          # other rows untouched


def test_input_validation(helix):
    cp = 4
    ws = helix.allocate_workspace(cp, 0)
    o = torch.randn(2, cp, 128, dtype=torch.bfloat16, device="cuda")
    s = torch.randn(2, cp, 2, dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError):
        helix.alltoall(o.float(), s, ws, 0, cp)
    with pytest.raises(RuntimeError):
        helix.alltoall(o, s.half(), ws, 0, cp)
    with pytest.raises(RuntimeError):
        helix.alltoall(torch.randn(2, 3, 128, dtype=torch.bfloat16, device="cuda"), s, ws, 0, cp)
    with pytest.raises(RuntimeError):
        helix.alltoall(o, torch.randn(2, cp, 3, device="cuda"), ws, 0, cp)
    with pytest.raises(RuntimeError):
        helix.alltoall(torch.randn(2, cp, 4, dtype=torch.bfloat16, device="cuda"), s, ws, 0, cp)  # 8-byte rows
    with pytest.raises(RuntimeError):
        helix.alltoall(o, s, ws[:2], 0, cp)


@pytest.mark.parametrize("cp", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,S", [(128, 2), (512, 2), (64, 6), (1536, 4)])
def test_exchange_bit_exact(helix, cp, dtype, D, S):
    torch.manual_seed(cp * 1000 + D)
    ws = _ws(helix, cp)
    E = 37
    o = torch.randn(cp, E, cp, D, device="cuda").to(dtype)
    s = torch.randn(cp, E, cp, S, device="cuda")
    ro, rs = _ops().alltoall_debug(o, s, ws, 0, cp, True, 0, 0)
    torch.cuda.synchronize()
    assert torch.equal(ro, o.transpose(0, 2).contiguous())
    assert torch.equal(rs, s.transpose(0, 2).contiguous())
    for r in range(cp):
        assert helix.check_status(ws, r, cp)["code"] == 0


@pytest.mark.parametrize("cp", [2, 4, 8])
@pytest.mark.parametrize("B,H,D", [(1, 128, 512), (8, 64, 128), (33, 16, 256), (3, 8, 1024)])
@pytest.mark.parametrize("base2", [False, True])
def test_fused_combine_native_layout(helix, cp, B, H, D, base2):
    from helix_a2a_b200.ops import reference_math as rm
    torch.manual_seed(B * 31 + D)
    ws = _ws(helix, cp)
    outs = torch.randn(cp, B, H, D, device="cuda").bfloat16()
    lses = torch.randn(cp, B, H, device="cuda") * 3
    got, glse = _ops().alltoall_combine(outs, lses, ws, 0, cp, 0, True, base2, 0, True, 0, 0)
    torch.cuda.synchronize()
    want, wlse = rm.head_scatter_combine_reference(outs, lses, return_lse=True, base2=base2)
    assert got.shape == (cp, B, H // cp, D)
    assert (got.float() - want).abs().max() < 2e-2
    assert (glse - wlse).abs().max() < 1e-4


@pytest.mark.parametrize("cp", [2, 4, 8])
def test_fused_combine_bulk_call(helix, cp):
    """Hundreds of lines per channel: the auto-tuner gives 10 (cp = 8: 9) of a CTA's 16 warps to receiving."""
    from helix_a2a_b200.ops import reference_math as rm
    from helix_a2a_b200.ops._ext import ext
    B, H, D = 32 * cp, 128, 512          # >= 22 entries per channel of 9 lines each, whatever the rank count
    torch.manual_seed(cp)
    ws = _ws(helix, cp)
    outs = torch.randn(cp, B, H, D, device="cuda").bfloat16()
    lses = torch.randn(cp, B, H, device="cuda") * 3
    for _ in range(2):
        got, glse = _ops().alltoall_combine(outs, lses, ws, 0, cp, 0, True, False, 0, True, 0, 0)
    torch.cuda.synchronize()
    info = ext().last_launch_info()
    assert info["recv_warps"] > 8 and info["send_warps"] + info["recv_warps"] == 16
    want, wlse = rm.head_scatter_combine_reference(outs, lses, return_lse=True)
    assert (got.float() - want).abs().max() < 2e-2
    assert (glse - wlse).abs().max() < 1e-4
    for r in range(cp):
        assert helix.check_status(ws, r, cp)["code"] == 0


@pytest.mark.parametrize("stats_mode", ["lse", "max_sumexp"])
def test_fused_combine_entries_layout_and_stats_modes(helix, stats_mode):
    from helix_a2a_b200.ops import reference_math as rm
    cp, T, H, D = 4, 5, 8, 512
    ws = _ws(helix, cp)
    po = torch.randn(cp, T, H, cp, D, device="cuda").bfloat16()
    st = torch.stack([torch.randn(cp, T, H, cp, device="cuda") * 3,
                      torch.rand(cp, T, H, cp, device="cuda") * 63 + 1], -1)
    got, _ = _ops().alltoall_combine(po, st, ws, 0, cp, 1, False, False, 0 if stats_mode == "lse" else 1, True, 0, 0)
    torch.cuda.synchronize()
    ro, rs = rm.alltoall_reference(po.flatten(1, 2), st.flatten(1, 2))       # [recv, E, sender, *]
    l = rm.stats_to_lse(rs, stats_mode)
    want = rm.lse_combine(ro.permute(2, 0, 1, 3), l.permute(2, 0, 1))         # N, recv(B), E(H), D
    assert (got.flatten(1, 2).float() - want).abs().max() < 2e-2


def test_combine_edge_cases_nan_inf(helix):
    from helix_a2a_b200.ops import reference_math as rm
    cp, B, H, D = 4, 2, 8, 128
    ws = _ws(helix, cp)
    outs = torch.randn(cp, B, H, D, device="cuda").bfloat16()
    lses = torch.randn(cp, B, H, device="cuda")
    lses[0, 0, 0] = float("-inf")
    lses[1, 0, 1] = float("nan")
    lses[2, 0, 2] = float("inf")
    lses[:, 1, 3] = float("-inf")
    got, glse = _ops().alltoall_combine(outs, lses, ws, 0, cp, 0, True, False, 0, True, 0, 0)
    want, wlse = rm.head_scatter_combine_reference(outs, lses, return_lse=True)
    assert torch.isfinite(got.float()).all()
    assert (got.float() - want).abs().max() < 2e-2
    # every shard empty: output 0 and LSE -inf
    r, hl = 3 // (H // cp), 3 % (H // cp)
    assert (got[r, 1, hl] == 0).all() and glse[r, 1, hl] == float("-inf")
    fin = torch.isfinite(wlse)
    assert (glse[fin] - wlse[fin]).abs().max() < 1e-4


def test_many_calls_without_reinit_and_ring_wrap(helix):
    """> 2048 lines per ring across calls: rings wrap, nothing is re-initialised."""
    from helix_a2a_b200.ops import reference_math as rm
    cp, B, H, D = 2, 16, 32, 512
    ws = _ws(helix, cp)
    os.environ["HELIX_A2A_CHANNEL_COUNT"] = "2"      # 128 messages x 9 lines per ring per call
    try:
        for it in range(12):
            outs = torch.randn(cp, B, H, D, device="cuda").bfloat16()
            lses = torch.randn(cp, B, H, device="cuda")
            got, _ = _ops().alltoall_combine(outs, lses, ws, 0, cp, 0, False, False, 0, True, 0, 0)
            want = rm.head_scatter_combine_reference(outs, lses)
            assert (got.float() - want).abs().max() < 2e-2, f"call {it}"
        from helix_a2a_b200.ops._ext import ext
        assert ext().last_launch_info()["channels"] == 2
    finally:
        del os.environ["HELIX_A2A_CHANNEL_COUNT"]
    assert helix.check_status(ws, 0, cp)["code"] == 0


def test_single_call_larger_than_ring(helix):
    """One call that puts ~5 ring laps on one channel: in-call flow control (tail publishes)."""
    cp, E, D = 2, 1200, 512
    ws = _ws(helix, cp)
    os.environ["HELIX_A2A_CHANNEL_COUNT"] = "1"
    try:
        o = torch.randn(cp, E, cp, D, device="cuda").bfloat16()
        s = torch.randn(cp, E, cp, 2, device="cuda")
        ro, rs = _ops().alltoall_debug(o, s, ws, 0, cp, True, 0, 0)
        assert torch.equal(ro, o.transpose(0, 2).contiguous()) and torch.equal(rs, s.transpose(0, 2).contiguous())
        got, _ = _ops().alltoall_combine(o, s, ws, 0, cp, 1, False, False, 0, True, 0, 0)
        from helix_a2a_b200.ops import reference_math as rm
        ro2, rs2 = rm.alltoall_reference(o, s)
        want = rm.lse_combine(ro2.permute(2, 0, 1, 3), rs2[..., 0].permute(2, 0, 1))
        assert (got.float() - want).abs().max() < 2e-2
    finally:
        del os.environ["HELIX_A2A_CHANNEL_COUNT"]
    assert helix.check_status(ws, 0, cp)["code"] == 0


def test_timeout_returns_status_and_gpu_stays_usable(helix):
    """A sender that never sends: the receiver's wait runs out, the kernel returns, status is set."""
    cp = 2
    ws = _ws(helix, cp)
    o = torch.randn(cp, 4, cp, 128, device="cuda").bfloat16()
    s = torch.randn(cp, 4, cp, 2, device="cuda")
    # rank 0's sender skips peer 1 -> rank 1 never receives
    _ops().alltoall_debug(o, s, ws, 0, cp, True, 0b10, 50)
    torch.cuda.synchronize()
    st1 = helix.check_status(ws, 1, cp, raise_on_error=False)
    assert st1["code"] == 1 and st1["peer"] == 0
    with pytest.raises(helix.HelixTimeoutError):
        helix.check_status(ws, 1, cp)
    # recovery: re-init, then the same workspace works again
    helix.init_workspace_all_rows(ws, cp)
    ro, _ = _ops().alltoall_debug(o, s, ws, 0, cp, True, 0, 0)
    assert torch.equal(ro, o.transpose(0, 2).contiguous())
    assert helix.check_status(ws, 1, cp)["code"] == 0


def test_timeout_in_combine_mode_leaves_nan_rows_and_hook_raises(helix):
    """Combine mode with a sender that stays silent: the rows that could not be completed come out as NaN
    (never as stale memory) and the serving hook's status check raises."""
    from helix_a2a_b200.vllm_patch import dcp_alltoall_helix as hook
    cp, B, H, D = 2, 4, 16, 128
    ws = _ws(helix, cp)
    outs = torch.randn(cp, B, H, D, device="cuda").bfloat16()
    lses = torch.randn(cp, B, H, device="cuda")
    got, glse = _ops().alltoall_combine(outs, lses, ws, 0, cp, 0, True, False, 0, True, 0b10, 50)
    torch.cuda.synchronize()
    assert torch.isnan(got[1].float()).all() and torch.isnan(glse[1]).all()      # rank 1 never heard from rank 0
    old = hook._workspace, hook._workspace_key
    try:
        hook._workspace, hook._workspace_key = ws, (cp, 1, "cuda")
        with pytest.raises(helix.HelixTimeoutError):
            hook.dcp_a2a_check_status()
        assert hook.dcp_a2a_check_status(raise_on_error=False)["code"] == 1
        # the non-blocking poll the import hook runs once per engine step: the first call only requests a copy of
        # the status block, a later one (the copy has arrived by then) raises
        assert hook.dcp_a2a_poll_status() is None
        torch.cuda.synchronize()
        with pytest.raises(helix.HelixTimeoutError):
            hook.dcp_a2a_poll_status()
    finally:
        hook._workspace, hook._workspace_key = old
        hook._poller = None
    helix.init_workspace_all_rows(ws, cp)
    got, _ = _ops().alltoall_combine(outs, lses, ws, 0, cp, 0, False, False, 0, True, 0, 0)
    from helix_a2a_b200.ops import reference_math as rm
    assert (got.float() - rm.head_scatter_combine_reference(outs, lses)).abs().max() < 2e-2
    poller = helix.StatusPoller(ws, 1, cp)            # a clean workspace polls clean
    assert poller.poll() is None
    torch.cuda.synchronize()
    assert poller.poll()["code"] == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("N,B,H,D", [(2, 3, 8, 128), (8, 5, 16, 512), (4, 1, 4, 64), (3, 7, 2, 1024)])
@pytest.mark.parametrize("base2", [False, True])
def test_lse_combine_kernel_matches_fp32_reference(helix, dtype, N, B, H, D, base2):
    """Stand-alone combine kernel against the torch oracle, both layouts, including the -inf / NaN rules."""
    from helix_a2a_b200.ops import reference_math as rm
    torch.manual_seed(N * 100 + D)
    o = torch.randn(N, B, H, D, device="cuda").to(dtype)
    l = torch.randn(N, B, H, device="cuda") * 3
    l[0, 0, 0] = float("-inf")
    l[1, 0, 1] = float("nan")
    l[:, -1, -1] = float("-inf")                      # a row nobody contributes to
    if N > 2:
        l[2, 0, 0] = float("inf")
    want, wl = rm.lse_combine(o.float(), l, return_lse=True, base2=base2)
    got, gl = helix.lse_combine(o, l, return_lse=True, base2=base2)
    assert got.dtype == dtype and got.shape == (B, H, D)
    assert (got.float() - want).abs().max() < 2e-2
    fin = torch.isfinite(wl)
    assert (gl[fin] - wl[fin]).abs().max() < 1e-4 and torch.equal(torch.isfinite(gl), fin)
    assert (got[-1, -1] == 0).all() and gl[-1, -1] == float("-inf")
    # the layout `alltoall` returns: [..., N, D] with the LSE in slot 0 of the stats pair
    ro = o.permute(1, 2, 0, 3).contiguous()
    rs = torch.stack([l.permute(1, 2, 0), torch.zeros(B, H, N, device="cuda")], dim=-1).contiguous()
    got2 = helix.lse_combine(ro, rs[..., 0], base2=base2, layout="BHND")
    assert torch.equal(got2, got)


def test_cuda_graph_replay(helix):
    from helix_a2a_b200.ops import reference_math as rm
    cp, B, H, D = 4, 8, 64, 128
    ws = _ws(helix, cp)
    outs = torch.randn(cp, B, H, D, device="cuda").bfloat16()
    lses = torch.randn(cp, B, H, device="cuda")
    g = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        _ops().alltoall_combine(outs, lses, ws, 0, cp, 0, False, False, 0, True, 0, 0)
        with torch.cuda.graph(g, stream=stream):
            got, _ = _ops().alltoall_combine(outs, lses, ws, 0, cp, 0, False, False, 0, True, 0, 0)
    for _ in range(5):
        outs.copy_(torch.randn_like(outs))
        g.replay()
        torch.cuda.synchronize()
        want = rm.head_scatter_combine_reference(outs, lses)
        assert (got.float() - want).abs().max() < 2e-2


def test_public_api_cp1(helix):
    ws = helix.allocate_workspace(1, 0)
    helix.init_workspace(ws, 0, 1)
    o = torch.randn(5, 1, 128, device="cuda").bfloat16()
    s = torch.randn(5, 1, 2, device="cuda")
    ro, rs = helix.alltoall(o, s, ws, 0, 1)
    assert torch.equal(ro, o) and torch.equal(rs, s)
    os.environ["HELIX_A2A_ENABLE_PDL"] = "1"       # launch attribute for programmatic dependent launch
    try:
        for _ in range(3):
            ro, rs = helix.alltoall(o, s, ws, 0, 1)
        assert torch.equal(ro, o) and torch.equal(rs, s)
    finally:
        del os.environ["HELIX_A2A_ENABLE_PDL"]
    out = helix.alltoall_combine(torch.randn(3, 8, 128, device="cuda").bfloat16(), torch.randn(3, 8, device="cuda"),
                                 ws, 0, 1)
    assert out.shape == (3, 8, 128)
    info = helix.debug_info(ws)
    assert info["workspace_kind"] == "device"


@pytest.mark.parametrize("cp,B,H,D,hidden", [(2, 8, 16, 128, 512), (4, 3, 32, 128, 1024), (2, 64, 16, 128, 256),
                                              (4, 64, 16, 128, 512), (8, 8, 64, 128, 1024), (8, 33, 64, 128, 256),
                                              (2, 5, 8, 64, 384), (3, 2, 12, 192, 128),
                                              # many rows: the slabs of a head group share them, token-sliced fold
                                              (2, 64, 16, 128, 1024), (4, 40, 32, 128, 1024), (2, 17, 32, 128, 512),
                                              (2, 20, 12, 128, 256)])      # three heads per group
def test_fused_exchange_combine_oproj(helix, cp, B, H, D, hidden):
    """One launch: exchange + combine + tcgen05 o_proj, all ranks played on one GPU."""
    from helix_a2a_b200.ops import reference_math as rm
    torch.manual_seed(B + hidden)
    ws = _ws(helix, cp)
    K = (H // cp) * D
    outs = torch.randn(cp, B, H, D, device="cuda").bfloat16()
    lses = torch.randn(cp, B, H, device="cuda") * 2
    w = (torch.randn(cp, hidden, K, device="cuda") * 0.05).bfloat16()
    for it in range(3):                               # counters re-arm themselves between launches
        y, x = _ops().alltoall_combine_oproj(outs, lses, w, ws, 0, cp, False, True, 0)
        torch.cuda.synchronize()
        want_x = rm.head_scatter_combine_reference(outs, lses)                     # [cp, B, Hl, D]
        assert (x.float().view(cp, B, H // cp, D) - want_x).abs().max() < 2e-2
        for r in range(cp):
            ref = rm.oproj_reference(x[r], w[r])
            assert (y[r].float() - ref).abs().max() < 3e-2 * max(1.0, ref.abs().max().item()), (it, r)
    for r in range(cp):
        assert helix.check_status(ws, r, cp)["code"] == 0


def test_debug_bounds_checks_pass_on_valid_calls(helix, monkeypatch):
    """HELIX_A2A_DEBUG=1 also checks every message's source and destination span on the device; valid calls must
    come through with a clean status and unchanged results (invalid strides are exercised on the host only)."""
    from helix_a2a_b200.ops import reference_math as rm
    monkeypatch.setenv("HELIX_A2A_DEBUG", "1")
    for cp in (2, 4, 8):
        ws = _ws(helix, cp)
        o = torch.randn(cp, 9, cp, 128, device="cuda").bfloat16()
        s = torch.randn(cp, 9, cp, 4, device="cuda")
        ro, rs = _ops().alltoall_debug(o, s, ws, 0, cp, True, 0, 0)
        assert torch.equal(ro, o.transpose(0, 2).contiguous()) and torch.equal(rs, s.transpose(0, 2).contiguous())
        outs = torch.randn(cp, 6, 16 * cp, 128, device="cuda").bfloat16()
        lses = torch.randn(cp, 6, 16 * cp, device="cuda")
        got, glse = _ops().alltoall_combine(outs, lses, ws, 0, cp, 0, True, False, 0, True, 0, 0)
        want, wl = rm.head_scatter_combine_reference(outs, lses, return_lse=True)
        assert (got.float() - want).abs().max() < 2e-2 and (glse - wl).abs().max() < 1e-4
        for r in range(cp):
            assert helix.check_status(ws, r, cp)["code"] == 0


def test_debug_mode_poison_and_nvtx(helix):
    """HELIX_A2A_DEBUG=1 pre-fills outputs with NaN and verifies every row was written; NVTX ranges are harmless."""
    cp = 2
    ws = _ws(helix, 1)
    o = torch.randn(5, 1, 128, device="cuda").bfloat16()
    s = torch.randn(5, 1, 2, device="cuda")
    os.environ["HELIX_A2A_DEBUG"] = "1"
    os.environ["HELIX_A2A_NVTX"] = "1"
    try:
        ro, rs = helix.alltoall(o, s, ws, 0, 1)
        assert torch.equal(ro, o) and torch.equal(rs, s)
        from helix_a2a_b200.utils.tracing import check_written
        with pytest.raises(RuntimeError):
            check_written(torch.full((2, 2), float("nan"), device="cuda"), "poisoned tensor")
    finally:
        del os.environ["HELIX_A2A_DEBUG"], os.environ["HELIX_A2A_NVTX"]
    del cp
