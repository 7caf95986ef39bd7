"""Build / import smoke tests (mirrors the reference's tests/test_build.py:5-26)."""
import helix_a2a_b200 as helix


def test_public_names():
    for name in ("workspace_size", "allocate_workspace", "init_workspace", "alltoall",
                 "alltoall_combine", "check_status", "reset_workspace"):
        assert callable(getattr(helix, name))
    assert helix.__version__ == "0.1.0"


def test_reference_package_name():
    import helix_a2a
    for name in ("workspace_size", "allocate_workspace", "init_workspace", "alltoall"):
        assert callable(getattr(helix_a2a, name))
    assert helix_a2a.__version__ == "0.1.0"


def test_workspace_size_formula():
    # B200: 148 SMs -> maxCh = 74 for cp <= 8 (values of the reference's formula)
    assert helix.workspace_size(2) == 77_670_400
    assert helix.workspace_size(4) == 155_340_800
    assert helix.workspace_size(8) == 310_681_600
    assert helix.workspace_size(4) != 16_778_240   # the stale stub value in the reference's docstring
    for cp in (1, 2, 4, 8, 16):
        assert helix.workspace_size(cp) > 0


def test_extension_builds(native_built):
    from helix_a2a_b200.ops._ext import ext
    C = ext()
    lay = C.layout(8, 148)
    assert lay["max_channels"] == 148
    assert lay["row_bytes"] == 310_681_600
    assert lay["status_offset"] + 256 <= lay["row_bytes"]
    # MLA message: 1024 B row + 8 B stats -> 9 lines; GQA: 256 + 8 -> 3 lines
    assert C.wire_bytes(1032) == 9 * 128
    assert C.wire_bytes(264) == 3 * 128


def test_one_kernel_path_shape_rules(native_built):
    """The launcher's "does this shape run as one kernel" rules, as the model stacks query them (148 SMs)."""
    from helix_a2a_b200.ops._ext import ext
    fits = ext().fused_oproj_fits            # (tokens, heads per rank, head dim, hidden, cp)
    assert fits(8, 8, 128, 8192, 8)          # Llama-3-70B at cp = 8: 64 slabs x 2 head groups = 128 GEMM CTAs
    assert fits(64, 8, 128, 8192, 8)
    assert not fits(65, 8, 128, 8192, 8)     # more than 64 tokens
    assert not fits(8, 32, 128, 8192, 2)     # cp = 2: 64 slabs x 8 groups do not fit the device at once
    assert fits(8, 32, 128, 2048, 2)
    assert not fits(8, 16, 512, 7168, 8)     # MLA rows (512 dims) are 9 lines, more than one warp-wide load
    assert not fits(8, 8, 128, 8192, 16)     # at most 8 ranks
    assert not fits(8, 64, 128, 8192, 1)     # a single rank has nothing to exchange


def test_bench_defaults_and_config_keys(monkeypatch):
    """bench.py without flags: one GPU, at least three warm-up steps, the two-kernel chain; both arms print the same
    ``config`` keys (they share the function that builds it); --fuse-oproj alone means "on"."""
    import sys
    import bench
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    a = bench.parse()
    assert a.gpus == 1 and a.warmup >= 3 and a.steps >= 1 and a.impl == "helix" and a.fuse_oproj == "off"
    monkeypatch.setattr(sys, "argv", ["bench.py", "--fuse-oproj", "--impl", "reference"])
    a = bench.parse()
    assert a.fuse_oproj == "on" and a.impl == "reference"
    cfg = bench.bench_config(80, 8, 131072, 8, 16, 16384, 42_900_000_000, True)
    assert {"model", "global_batch", "seq_len", "parallelism"} <= set(cfg) and cfg["parallelism"] == "cp8"
    import inspect
    from benchmarks import reference_arm
    assert "bench_config(" in inspect.getsource(reference_arm)


def test_exchange_auto_tuner_plans(native_built):
    """The launch shapes the auto-tuner picks (csrc/exchange.cu::plan_launch), without a GPU.  The reference derives
    its channel count from the SM count alone (csrc/helix_alltoall.cu:524-530); here it follows the entry count."""
    from helix_a2a_b200.ops._ext import ext
    plan = ext().plan_info                     # (cp, SMs, outer, heads per rank, row bytes, stats words, combine)
    # one decode token at cp = 2: one entry per channel, every sender warp on the single peer, one receiver warp
    p = plan(2, 148, 1, 32, 256, 1, True)
    assert (p["channels"], p["send_warps"], p["recv_warps"], p["lines_per_message"]) == (32, 8, 1, 3)
    # cp = 8, one entry per channel: four receiver warps share the entry's seven peers
    p = plan(8, 148, 8, 8, 256, 1, True)
    assert (p["channels"], p["send_warps"], p["group_warps"], p["recv_warps"]) == (64, 7, 4, 4)
    # many lines per channel: 4 (two ranks) or 6 of the CTA's 16 warps send, the rest receive (cp = 8: one per peer, 7 + 9)
    for cp, want in ((2, (4, 12)), (4, (6, 10)), (8, (7, 9))):
        p = plan(cp, 148, 256, 128 // cp, 1024, 1, True)
        assert p["channels"] == 148 and (p["send_warps"], p["recv_warps"]) == want and p["lines_per_message"] == 9
    # exchange-only mode keeps eight receiver warps
    assert plan(4, 148, 64, 32, 1024, 4, False)["recv_warps"] == 8
