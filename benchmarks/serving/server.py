"""Start / stop one ``vllm serve`` process with the Helix DCP hook loaded in every worker.

Covers what the reference's job scripts do around the server
(``benchmark/sbatch/run_gb200_aiperf_v3.sbatch:284-305`` builds the command line,
``benchmark/scripts/correctness_check.sh:162-216`` starts, health-checks and stops it): the hook is
loaded through ``PYTHONPATH`` (``helix_a2a_b200.vllm_patch.import_hook.autoload_env``) instead of
overwriting vLLM's file, and the server is stopped by signalling the process group this module
created - never by matching command lines.
"""
from __future__ import annotations

import os
import signal
import subprocess
import sys
import time
import urllib.request
from dataclasses import dataclass
from typing import List, Optional


@dataclass
class ServerConfig:
    model: str
    tp: int = 1
    dcp: int = 1
    comm: str = ""              # "" / "ag_rs" (vLLM default) or "a2a"
    tpa: str = ""               # attention tensor-parallel size (only forks of vLLM know this flag)
    max_model_len: int = 32768
    attention_backend: str = ""
    load_format: str = ""       # "dummy": random weights, no checkpoint needed
    port: int = 8000
    quantization: str = ""
    gpu_memory_utilization: float = 0.0
    enforce_eager: bool = False
    extra_args: str = ""

    @property
    def key(self) -> str:
        """Server identity: a sweep restarts the server only when this changes."""
        return f"{self.dcp}:{self.comm}:{self.tpa}"

    @property
    def mode_name(self) -> str:
        if self.dcp <= 1:
            return "dcp1"
        name = f"dcp{self.dcp}_{self.comm or 'ag_rs'}"
        return name + (f"_tpa{self.tpa}" if self.tpa else "")


def build_vllm_cmd(cfg: ServerConfig) -> List[str]:
    cmd = [sys.executable, "-m", "vllm.entrypoints.cli.main", "serve", cfg.model,
           "--tensor-parallel-size", str(cfg.tp), "--max-model-len", str(cfg.max_model_len),
           "--host", "127.0.0.1", "--port", str(cfg.port), "--disable-log-stats", "--enable-prefix-caching"]
    if cfg.attention_backend:
        cmd += ["--attention-config.backend", cfg.attention_backend]
    if cfg.quantization:
        cmd += ["--quantization", cfg.quantization]
    if cfg.dcp > 1:
        cmd += ["--decode-context-parallel-size", str(cfg.dcp)]
    if cfg.comm and cfg.comm != "ag_rs":
        cmd += ["--dcp-comm-backend", cfg.comm]
    if cfg.tpa:
        cmd += ["--tensor-parallel-size-attention", str(cfg.tpa)]
    if cfg.load_format:
        cmd += ["--load-format", cfg.load_format]
    if cfg.gpu_memory_utilization > 0:
        cmd += ["--gpu-memory-utilization", str(cfg.gpu_memory_utilization)]
    if cfg.enforce_eager:
        cmd += ["--enforce-eager"]
    if cfg.extra_args:
        import shlex
        cmd += shlex.split(cfg.extra_args)
    return cmd


def server_env(helix_backend: str, base=None) -> dict:
    """Environment of the server: hook autoload, backend choice, loopback rendezvous."""
    from helix_a2a_b200.vllm_patch.import_hook import autoload_env
    env = autoload_env(base)
    env["HELIX_A2A_BACKEND"] = helix_backend
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    env.setdefault("VLLM_HOST_IP", "127.0.0.1")
    env.setdefault("VLLM_WORKER_MULTIPROC_METHOD", "spawn")
    # no network on the test machines: never wait for the hub or for usage reporting
    env.setdefault("HF_HUB_OFFLINE", "1")
    env.setdefault("TRANSFORMERS_OFFLINE", "1")
    env.setdefault("VLLM_NO_USAGE_STATS", "1")
    env.setdefault("DO_NOT_TRACK", "1")
    # Ranks drift apart by many seconds while vLLM warms up (one rank compiling a kernel the other has cached),
    # so the device-side waits get a limit as patient as a collective library would be; a real hang still ends.
    env.setdefault("HELIX_A2A_TIMEOUT_MS", "120000")
    return env


class Server:
    def __init__(self, cfg: ServerConfig, helix_backend: str, log_path: str):
        self.cfg, self.helix_backend, self.log_path = cfg, helix_backend, log_path
        self.proc: Optional[subprocess.Popen] = None
        self._log = None

    @property
    def url(self) -> str:
        return f"http://127.0.0.1:{self.cfg.port}"

    def start(self, ready_timeout_s: float = 1200.0) -> bool:
        os.makedirs(os.path.dirname(os.path.abspath(self.log_path)) or ".", exist_ok=True)
        self._log = open(self.log_path, "ab")
        self.proc = subprocess.Popen(build_vllm_cmd(self.cfg), env=server_env(self.helix_backend),
                                     stdout=self._log, stderr=subprocess.STDOUT, start_new_session=True)
        deadline = time.time() + ready_timeout_s
        while time.time() < deadline:
            if self.proc.poll() is not None:
                return False
            try:
                with urllib.request.urlopen(self.url + "/health", timeout=2) as r:
                    if r.status == 200:
                        return True
            except Exception:  # noqa: BLE001  (not up yet)
                pass
            time.sleep(2.0)
        return False

    def stop(self, grace_s: float = 30.0) -> None:
        """SIGTERM, then SIGKILL, to the session this object started - nothing else."""
        if self.proc is None:
            return
        pgid = self.proc.pid            # start_new_session: the child leads its own process group
        for sig, wait in ((signal.SIGTERM, grace_s), (signal.SIGKILL, 10.0)):
            try:
                os.killpg(pgid, sig)
            except ProcessLookupError:
                break
            t_end = time.time() + wait
            while time.time() < t_end and self.proc.poll() is None:
                time.sleep(0.5)
            if self.proc.poll() is not None:
                # children of the leader share the group: give them the same signal once more, then move on
                try:
                    os.killpg(pgid, sig)
                except ProcessLookupError:
                    pass
                break
        if self._log:
            self._log.close()
        self.proc = None
