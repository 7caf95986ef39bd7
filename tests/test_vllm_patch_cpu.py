"""The vLLM hook on CPU ranks (gloo): native and nccl backends agree with the fp32 oracle."""
import os

import pytest
import torch

from _mp import run_ranks


class _Group:
    def __init__(self, rank, world, group):
        self.rank_in_group, self.world_size = rank, world
        self.device_group = self.cpu_group = group


def _hook(rank, world, backend, base_e):
    os.environ["HELIX_A2A_BACKEND"] = backend
    import torch.distributed as dist
    from helix_a2a_b200.ops import reference_math as rm
    from helix_a2a_b200.vllm_patch import dcp_alltoall_helix as hook
    torch.manual_seed(0)
    B, H, D = 3, 8, 32
    outs, lses = torch.randn(world, B, H, D), torch.randn(world, B, H) * 2
    cp = _Group(rank, world, dist.group.WORLD)
    hook.dcp_a2a_ensure_initialized(cp, torch.device("cpu"))
    got, glse = hook.dcp_a2a_lse_reduce(outs[rank], lses[rank], cp, return_lse=True, is_lse_base_on_e=base_e)
    want, wlse = rm.head_scatter_combine_reference(outs, lses, return_lse=True, base2=not base_e)
    only = hook.dcp_a2a_lse_reduce(outs[rank], lses[rank], cp, is_lse_base_on_e=base_e)
    return (got - want[rank]).abs().max().item(), (glse - wlse[rank]).abs().max().item(), tuple(only.shape)


@pytest.mark.parametrize("backend", ["native", "nccl"])
@pytest.mark.parametrize("base_e", [True, False])
def test_hook_matches_oracle(backend, base_e):
    for e, el, shape in run_ranks(_hook, 2, (backend, base_e)):
        assert e < 1e-5 and el < 1e-4 and shape == (3, 4, 32)


def test_world_size_one_is_passthrough():
    from helix_a2a_b200.vllm_patch import dcp_alltoall_helix as hook
    o, l = torch.randn(2, 4, 8), torch.randn(2, 4)
    assert hook.dcp_a2a_lse_reduce(o, l, _Group(0, 1, None)) is o
    r = hook.dcp_a2a_lse_reduce(o, l, _Group(0, 1, None), return_lse=True)
    assert r[0] is o and r[1] is l


def test_signature_matches_installed_vllm():
    import inspect
    from helix_a2a_b200.vllm_patch import dcp_alltoall_helix as hook
    want = ["cp_attn_out", "cp_attn_lse", "cp_group", "ctx", "return_lse", "is_lse_base_on_e"]
    assert list(inspect.signature(hook.dcp_a2a_lse_reduce).parameters) == want


def test_installer_dry_run(tmp_path, capsys):
    from helix_a2a_b200.vllm_patch import install
    ops = tmp_path / "v1" / "attention" / "ops"
    ops.mkdir(parents=True)
    (ops / "dcp_alltoall.py").write_text("def dcp_a2a_lse_reduce(*a, **k):\n    return 'stock'\n")
    assert install.main(["--vllm-dir", str(tmp_path), "--dry-run"]) == 0
    assert (ops / "dcp_alltoall.py").read_text().startswith("def dcp_a2a")
    assert install.main(["--vllm-dir", str(tmp_path)]) == 0
    assert (ops / "dcp_alltoall.py.orig").exists() and "helix_a2a_b200" in (ops / "dcp_alltoall.py").read_text()
    assert install.main(["--vllm-dir", str(tmp_path), "--uninstall"]) == 0
    assert (ops / "dcp_alltoall.py").read_text().startswith("def dcp_a2a")


def test_hook_status_check_raises_and_combine_name_parity(monkeypatch):
    """The serving hook turns a recorded device-side timeout into an exception; the reference's public
    combine name exists and agrees with the oracle on CPU tensors."""
    import helix_a2a_b200 as helix
    from helix_a2a_b200.ops import reference_math as rm
    from helix_a2a_b200.vllm_patch import dcp_alltoall_helix as hook
    assert hook.dcp_a2a_check_status()["code"] == 0            # no workspace yet: nothing to report
    monkeypatch.setattr(hook, "_workspace", object())
    monkeypatch.setattr(hook, "_workspace_key", (2, 1, "cuda"))

    def fake_status(ws, rank, size, raise_on_error=True):
        assert (rank, size) == (1, 2)
        if raise_on_error:
            raise helix.HelixTimeoutError(1, 0, 3, 7)
        return {"code": 1, "peer": 0, "channel": 3, "entry": 7}

    monkeypatch.setattr(hook._helix, "check_status", fake_status)
    with pytest.raises(helix.HelixTimeoutError):
        hook.dcp_a2a_check_status()
    assert hook.dcp_a2a_check_status(raise_on_error=False)["code"] == 1
    o, l = torch.randn(3, 2, 4, 16), torch.randn(3, 2, 4)
    got, gl = hook.dcp_lse_combine_triton(o, l, return_lse=True, is_lse_base_on_e=False)
    want, wl = rm.lse_combine(o, l, return_lse=True, base2=True)
    assert (got - want).abs().max() < 1e-6 and (gl - wl).abs().max() < 1e-6


def test_import_hook_checks_status_after_each_step(monkeypatch):
    """Worker.execute_model is wrapped so that a failed exchange stops the engine after the step it happened in."""
    import types
    from helix_a2a_b200.vllm_patch import import_hook, dcp_alltoall_helix as hook
    calls = []

    class Worker:
        def compile_or_warm_up_model(self):
            return "warm"

        def execute_model(self, x):
            return x + 1

    mod = types.SimpleNamespace(Worker=Worker)
    import_hook._patch_worker_module(mod)
    monkeypatch.setenv("HELIX_A2A_BACKEND", "native")
    monkeypatch.delenv("HELIX_A2A_HOOK_CHECK", raising=False)
    monkeypatch.setattr(hook, "dcp_a2a_check_status", lambda raise_on_error=True: calls.append(("sync", raise_on_error)))
    monkeypatch.setattr(hook, "dcp_a2a_poll_status", lambda raise_on_error=True: calls.append(("poll", raise_on_error)))
    # default: the status is polled without waiting for the GPU
    assert Worker().execute_model(1) == 2 and calls == [("poll", True)]
    monkeypatch.setenv("HELIX_A2A_HOOK_CHECK", "sync")
    assert Worker().execute_model(1) == 2 and calls == [("poll", True), ("sync", True)]
    monkeypatch.setenv("HELIX_A2A_HOOK_CHECK", "0")
    assert Worker().execute_model(1) == 2 and len(calls) == 2


def test_status_poller_on_cpu_workspace_is_a_no_op():
    import helix_a2a_b200 as helix
    ws = helix.allocate_workspace(1, 0, device="cpu")
    poller = helix.StatusPoller(ws, 0, 1)
    assert poller.poll()["code"] == 0
