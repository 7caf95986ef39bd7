"""Failure detection without any GPU fault: every failure is made on the host.

* a CPU (gloo) rank that never joins the exchange: its peer's call ends with an error after a short
  process-group timeout instead of hanging;
* a rank that raises while the others wait in the handle exchange;
* argument / policy errors of the allocator surface as Python exceptions on every rank;
* the status block decoding used after a device-side timeout.
(The device-side path -- a receiver whose bounded wait runs out and returns a status -- is exercised on
a GPU in tests/test_gpu_exchange.py::test_timeout_returns_status_and_gpu_stays_usable.)
"""
from datetime import timedelta

import pytest
import torch

from _mp import run_ranks


def _absent_peer(rank, world):
    import torch.distributed as dist
    import helix_a2a_b200 as helix
    g = dist.new_group(backend="gloo", timeout=timedelta(seconds=2))
    ws = helix.allocate_workspace(world, rank, device="cpu", cpu_group=g)
    o, s = torch.randn(2, world, 8), torch.randn(2, world, 2)
    if rank == 1:
        return "skipped"                 # this rank never sends
    try:
        helix.alltoall(o, s, ws, rank, world)
    except Exception as e:  # noqa: BLE001
        return "error:" + type(e).__name__
    return "completed"


def test_absent_cpu_rank_ends_with_error_not_hang():
    res = run_ranks(_absent_peer, 2, timeout=60)
    assert res[1] == "skipped"
    assert res[0].startswith("error:")


def _raising_rank(rank, world):
    import torch.distributed as dist
    from helix_a2a_b200.parallel import workspace as wsm
    g = dist.new_group(backend="gloo", timeout=timedelta(seconds=2))
    if rank == 0:
        try:
            raise RuntimeError("simulated failure before the handle exchange")
        except RuntimeError:
            return "raised"
    try:
        wsm._allgather(("pid", 1), g)      # the exchange step the healthy rank is waiting in
    except Exception as e:  # noqa: BLE001
        return "error:" + type(e).__name__
    return "completed"


def test_rank_raising_during_handle_exchange_is_detected():
    res = run_ranks(_raising_rank, 2, timeout=60)
    assert res[0] == "raised" and res[1].startswith("error:")


def test_allocator_argument_errors():
    from helix_a2a_b200.parallel import workspace as wsm
    with pytest.raises(ValueError):
        wsm.workspace_bytes(0)
    assert wsm.should_use_mnnvl(None, False) is False
    assert wsm.should_use_mnnvl(None, True) is True
    assert wsm.should_use_mnnvl(None, "auto") is False       # no group, no env: private device memory


def test_mnnvl_env_policy(monkeypatch):
    from helix_a2a_b200.parallel import workspace as wsm
    monkeypatch.setenv("HELIX_A2A_USE_MNNVL", "1")
    assert wsm.should_use_mnnvl(None, "auto") is True
    monkeypatch.setenv("HELIX_A2A_USE_MNNVL", "off")
    assert wsm.should_use_mnnvl(None, "auto") is False
    monkeypatch.setenv("HELIX_A2A_USE_MNNVL", "auto")
    assert wsm.should_use_mnnvl(None, "auto") is False


def test_timeout_error_carries_location():
    import helix_a2a_b200 as helix
    e = helix.HelixTimeoutError(1, 3, 17, 42)
    assert e.code == 1 and e.peer == 3 and e.channel == 17 and e.entry == 42
    assert "peer=3" in str(e) and "never saw" in str(e)
    ws = helix.allocate_workspace(2, 0, device="cpu")
    assert helix.check_status(ws, 0, 2)["code"] == 0


def test_env_knobs(monkeypatch):
    from helix_a2a_b200.utils import env
    monkeypatch.setenv("HELIX_A2A_ENABLE_PDL", "1")
    monkeypatch.setenv("HELIX_A2A_CHANNEL_COUNT", "12")
    monkeypatch.setenv("HELIX_A2A_BACKEND", "NATIVE")
    monkeypatch.setenv("HELIX_A2A_TIMEOUT_MS", "50")
    assert env.enable_pdl() and env.channel_count() == 12 and env.backend() == "native" and env.timeout_ms() == 50
    monkeypatch.setenv("HELIX_A2A_CHANNEL_COUNT", "junk")
    assert env.channel_count() == 0
