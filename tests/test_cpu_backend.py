"""CPU / gloo correctness: world size 2, fp32, result equals single-device full attention to 1e-5.

Random q [T=4, H=8, D=128], K/V [S=256, 8, 128] split into two contiguous halves; each rank
computes its partial attention, then exchange + LSE combine through the public API.
"""
import pytest
import torch

from _mp import run_ranks


def _config1(rank, world):
    import helix_a2a_b200 as helix
    from helix_a2a_b200.ops import reference_math as rm
    import torch.distributed as dist
    torch.manual_seed(1234)                      # same tensors on every rank
    T, H, D, S = 4, 8, 128, 256
    q = torch.randn(T, H, D)
    k, v = torch.randn(S, 8, D), torch.randn(S, 8, D)
    full = rm.full_attention(q, k, v)
    ks, vs = k.chunk(world)[rank], v.chunk(world)[rank]
    o, lse = rm.partial_attention(q, ks, vs)

    ws = helix.allocate_workspace(world, rank, device="cpu", cpu_group=dist.group.WORLD)
    helix.init_workspace(ws, rank, world)
    dist.barrier()
    # fused path, native layout
    out, glse = helix.alltoall_combine(o, lse, ws, rank, world, return_lse=True)
    Hl = H // world
    err = (out - full[:, rank * Hl:(rank + 1) * Hl]).abs().max().item()
    _, lse_full = rm.partial_attention(q, k, v)
    err_lse = (glse - lse_full[:, rank * Hl:(rank + 1) * Hl]).abs().max().item()

    # reference contract: exchange, then combine by hand
    po = o.view(T, world, Hl, D).permute(0, 2, 1, 3).contiguous()            # [T, Hl, N, D]
    st = torch.stack([lse, torch.zeros_like(lse)], -1).view(T, world, Hl, 2).permute(0, 2, 1, 3).contiguous()
    ro, rs = helix.alltoall(po, st, ws, rank, world)
    comb = rm.lse_combine(ro.permute(2, 0, 1, 3), rs[..., 0].permute(2, 0, 1))
    err2 = (comb - full[:, rank * Hl:(rank + 1) * Hl]).abs().max().item()
    # entries layout of the fused call
    out3 = helix.alltoall_combine(po, st, ws, rank, world, layout="entries")
    err3 = (out3 - full[:, rank * Hl:(rank + 1) * Hl]).abs().max().item()
    return err, err_lse, err2, err3


def test_config1_world2_matches_full_attention():
    for err, err_lse, err2, err3 in run_ranks(_config1, 2):
        assert err < 1e-5 and err2 < 1e-5 and err3 < 1e-5
        assert err_lse < 1e-4


def test_world4():
    for err, err_lse, err2, err3 in run_ranks(_config1, 4):
        assert max(err, err2, err3) < 1e-5


def _exchange_contract(rank, world):
    import helix_a2a_b200 as helix
    import torch.distributed as dist
    torch.manual_seed(42)
    B, D, S = 4, 16, 4
    full_o = torch.randn(B, world, world, D)
    full_s = torch.randn(B, world, world, S)
    ws = helix.allocate_workspace(world, rank, device="cpu", cpu_group=dist.group.WORLD)
    ro, rs = helix.alltoall(full_o[:, :, rank].contiguous(), full_s[:, :, rank].contiguous(), ws, rank, world)
    # rank r receives from sender i the slice sender i had at [:, r, :]
    want_o = full_o[:, rank, :, :]
    want_s = full_s[:, rank, :, :]
    return (ro - want_o).abs().max().item(), (rs - want_s).abs().max().item()


def test_exchange_contract_world3():
    for eo, es in run_ranks(_exchange_contract, 3):
        assert eo == 0 and es == 0


def test_cp1_passthrough():
    import helix_a2a_b200 as helix
    ws = helix.allocate_workspace(1, 0, device="cpu")
    o, s = torch.randn(3, 1, 8), torch.randn(3, 1, 2)
    ro, rs = helix.alltoall(o, s, ws, 0, 1)
    assert torch.equal(ro, o) and torch.equal(rs, s)
    with pytest.raises(RuntimeError):
        helix.alltoall(torch.randn(3, 2, 8), s, ws, 0, 1)
