"""Serving drivers and the import-time vLLM hook, on CPU: a fake OpenAI server, a fake vLLM tree."""
import asyncio
import json
import os
import subprocess
import sys
import textwrap

import pytest

from benchmarks.serving import correctness_check, loadgen, serve_sweep
from benchmarks.serving.server import ServerConfig, build_vllm_cmd, server_env
from benchmarks.serving.tiny_model import synthetic_prompt, write_tiny_model

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_parse_configs_and_modes():
    cfgs = serve_sweep.parse_configs("2:32768:a2a:;1:32768::;4:65536:a2a:2;8:1048576")
    assert cfgs == [(2, 32768, "a2a", ""), (1, 32768, "", ""), (4, 65536, "a2a", "2"), (8, 1048576, "", "")]
    assert ServerConfig("m", dcp=2, comm="a2a").mode_name == "dcp2_a2a"
    assert ServerConfig("m", dcp=1).mode_name == "dcp1"
    assert ServerConfig("m", dcp=4, comm="", tpa="2").mode_name == "dcp4_ag_rs_tpa2"
    assert serve_sweep.format_context(1048576) == "1M" and serve_sweep.format_context(32768) == "32K"
    for bad in ("2", "0:1024", "2:1024:tcp", "1:2:3:4:5"):
        with pytest.raises(ValueError):
            serve_sweep.parse_configs(bad)


def test_vllm_command_line():
    cmd = build_vllm_cmd(ServerConfig("/m", tp=4, dcp=2, comm="a2a", max_model_len=4096, load_format="dummy",
                                      attention_backend="FLASH_ATTN", enforce_eager=True, extra_args="--seed 7"))
    s = " ".join(cmd)
    assert "serve /m --tensor-parallel-size 4 --max-model-len 4096" in s
    assert "--decode-context-parallel-size 2 --dcp-comm-backend a2a" in s
    assert "--load-format dummy" in s and "--enforce-eager" in s and s.endswith("--seed 7")
    plain = " ".join(build_vllm_cmd(ServerConfig("/m", dcp=1, comm="a2a")))
    assert "--decode-context-parallel-size" not in plain
    env = server_env("native", {"PYTHONPATH": "/x"})
    parts = env["PYTHONPATH"].split(os.pathsep)
    assert parts[0].endswith(os.path.join("vllm_patch", "autoload")) and parts[1] == REPO and parts[-1] == "/x"
    assert env["HELIX_A2A_BACKEND"] == "native" and env["MASTER_ADDR"] == "127.0.0.1"


def test_sweep_dry_run_and_resume(tmp_path, capsys):
    results = str(tmp_path / "res")
    args = ["--model", "/models/tiny", "--configs", "2:4096:a2a:;2:8192:a2a:;1:4096::", "--concurrency", "1,2",
            "--results", results, "--dry-run", "--helix-backend", "native"]
    assert serve_sweep.main(args) == 0
    out = capsys.readouterr().out
    # one server start per distinct dcp:comm:tpa, the second context re-uses it
    assert out.count("[dry-run] HELIX_A2A_BACKEND=native") == 2 and "reusing server (2:a2a:)" in out
    assert out.count("benchmarks.serving.loadgen") == 6 and "all configs processed (3/3)" in out
    # points that exist are skipped; a configuration whose points all exist does not start a server
    for c in (1, 2):
        p = serve_sweep.point_path(results, "tiny", 2, "native", "dcp2_a2a", 4096, c)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        open(p, "w").write("{}")
    assert serve_sweep.main(args) == 0
    out = capsys.readouterr().out
    assert "SKIP: all points exist" in out and out.count("benchmarks.serving.loadgen") == 4
    # deadline: nothing new starts when too little time is left
    assert serve_sweep.main(args + ["--deadline-min", "1", "--min-config-min", "5", "--force"]) == 0
    assert "TIME:" in capsys.readouterr().out
    # sanity mode: one concurrency level, three requests
    assert serve_sweep.main(args + ["--sanity"]) == 0
    out = capsys.readouterr().out
    assert "--request-count 3" in out and "--concurrency 2" not in out


def _fake_openai_app(n_tokens_default=5, delay=0.002):
    from aiohttp import web

    async def completions(request):
        body = await request.json()
        n = int(body.get("max_tokens", n_tokens_default))
        if not body.get("stream"):
            return web.json_response({"choices": [{"text": " ".join(f"w{i}" for i in range(n))}]})
        resp = web.StreamResponse(headers={"Content-Type": "text/event-stream"})
        await resp.prepare(request)
        for i in range(n):
            await asyncio.sleep(delay)
            await resp.write(f"data: {json.dumps({'choices': [{'text': f' w{i}'}]})}\n\n".encode())
        await resp.write(f"data: {json.dumps({'choices': [], 'usage': {'completion_tokens': n}})}\n\n".encode())
        await resp.write(b"data: [DONE]\n\n")
        return resp

    async def health(request):
        return web.Response(text="ok")

    app = web.Application()
    app.router.add_post("/v1/completions", completions)
    app.router.add_get("/health", health)
    return app


def test_loadgen_against_fake_server():
    from aiohttp import web

    async def go():
        runner = web.AppRunner(_fake_openai_app())
        await runner.setup()
        site = web.TCPSite(runner, "127.0.0.1", 0)
        await site.start()
        port = site._server.sockets[0].getsockname()[1]
        try:
            return await loadgen.run_load(f"http://127.0.0.1:{port}", "m", synthetic_prompt(16), output_tokens=8,
                                          concurrency=3, request_count=7, warmup_request_count=2, timeout_s=30)
        finally:
            await runner.cleanup()

    res = asyncio.run(go())
    assert res["completed"] == 7 and res["failed"] == 0
    assert res["inter_token_latency_ms"]["n"] == 7 * 7 and res["inter_token_latency_ms"]["mean"] > 0
    assert res["output_token_throughput_per_s"] > 0 and res["time_to_first_token_ms"]["p50"] > 0
    assert res["sample_text"].split()[:2] == ["w0", "w1"]


def test_loadgen_counts_failures():
    res = asyncio.run(loadgen.run_load("http://127.0.0.1:9", "m", "x", output_tokens=2, concurrency=2,
                                       request_count=3, timeout_s=5))
    assert res["completed"] == 0 and res["failed"] == 3 and res["errors"]


def test_percentiles():
    xs = [1.0, 2.0, 3.0, 4.0, 5.0]
    assert loadgen.percentile(xs, 0.5) == 3.0 and loadgen.percentile(xs, 1.0) == 5.0
    assert loadgen.stats(xs, 1e3)["mean"] == 3000.0 and loadgen.stats([])["n"] == 0


def test_compare_outputs():
    a = ["w1 w2 w3 w4", "w5 w6"]
    r = correctness_check.compare(a, list(a), 0)
    assert r["all_match"] and r["matched"] == 2
    r = correctness_check.compare(a, ["w1 w2 w9 w4", "w5 w6"], 0)
    assert not r["all_match"] and r["rows"][0]["common_prefix_tokens"] == 2
    assert correctness_check.compare(a, ["w1 w2 w9 w4", "w5 w6"], 2)["all_match"]


def test_tiny_model_directory(tmp_path):
    d = write_tiny_model(str(tmp_path / "tiny"), layers=2, hidden=256, heads=2, vocab=512)
    cfg = json.load(open(os.path.join(d, "config.json")))
    assert cfg["num_key_value_heads"] == 1 and cfg["head_dim"] == 128 and cfg["architectures"] == ["LlamaForCausalLM"]
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(d)
    p = synthetic_prompt(33, seed=3, vocab=512)
    ids = tok(p)["input_ids"]
    assert len(ids) == 33 and tok.decode(ids) == p


def _write_fake_vllm(root):
    files = {
        "vllm/__init__.py": "",
        "vllm/v1/__init__.py": "", "vllm/v1/attention/__init__.py": "", "vllm/v1/attention/ops/__init__.py": "",
        "vllm/v1/attention/backends/__init__.py": "", "vllm/v1/worker/__init__.py": "",
        "vllm/distributed/__init__.py": "",
        "vllm/distributed/parallel_state.py": "def get_dcp_group():\n    raise AssertionError('no dcp group')\n",
        "vllm/v1/attention/ops/dcp_alltoall.py": "def dcp_a2a_lse_reduce(*a, **k):\n    return 'stock'\n",
        "vllm/v1/attention/backends/flash_attn.py": "from vllm.v1.attention.ops.dcp_alltoall import dcp_a2a_lse_reduce\n",
        "vllm/v1/worker/gpu_worker.py": "class Worker:\n    def compile_or_warm_up_model(self):\n        return 'warm'\n",
    }
    for rel, text in files.items():
        p = os.path.join(root, rel)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        open(p, "w").write(text)


def test_import_hook_in_child_interpreter(tmp_path):
    """With the autoload directory on PYTHONPATH a fresh interpreter swaps the hook in before the
    attention backend binds the stock function, keeps the stock one reachable, and wraps the warm-up."""
    from helix_a2a_b200.vllm_patch.import_hook import autoload_env
    _write_fake_vllm(str(tmp_path))
    env = autoload_env({**os.environ, "PYTHONPATH": str(tmp_path), "HELIX_A2A_BACKEND": "native"})
    code = textwrap.dedent("""
        import sys
        assert "torch" not in sys.modules, "the start-up shim must stay light"
        import vllm.v1.attention.backends.flash_attn as fa
        import vllm.v1.attention.ops.dcp_alltoall as stock
        from helix_a2a_b200.vllm_patch import dcp_alltoall_helix as hx
        assert fa.dcp_a2a_lse_reduce is hx.dcp_a2a_lse_reduce, fa.dcp_a2a_lse_reduce
        assert stock.dcp_a2a_ensure_initialized is hx.dcp_a2a_ensure_initialized
        assert hx._stock_reduce is not None and hx._stock_reduce() == "stock"
        import vllm.v1.worker.gpu_worker as w
        assert getattr(w.Worker.compile_or_warm_up_model, "__helix_hooked__", False)
        assert w.Worker().compile_or_warm_up_model() == "warm"     # no DCP group: the wrapper just passes through
        print("HOOKED")
    """)
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "HOOKED" in r.stdout, r.stdout + r.stderr
    # switched off: the stock function stays
    env["HELIX_A2A_VLLM_HOOK"] = "0"
    r = subprocess.run([sys.executable, "-c", "import vllm.v1.attention.backends.flash_attn as fa; print(fa.dcp_a2a_lse_reduce())"],
                       env=env, capture_output=True, text=True, timeout=120)
    assert r.stdout.strip() == "stock", r.stdout + r.stderr


def test_import_hook_install_is_idempotent():
    from helix_a2a_b200.vllm_patch import import_hook
    try:
        first = import_hook.install()
        assert import_hook.install() is False
        assert sum(isinstance(f, import_hook.HelixHookFinder) for f in sys.meta_path) == 1
        assert first in (True, False)
    finally:
        import_hook.uninstall()
    assert not any(isinstance(f, import_hook.HelixHookFinder) for f in sys.meta_path)
