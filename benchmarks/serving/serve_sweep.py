"""End-to-end serving sweep on one box: vLLM with decode context parallelism, NCCL or Helix exchange.

Same job logic as the reference's SLURM script (``benchmark/sbatch/run_gb200_aiperf_v3.sbatch``),
for one machine and without SLURM / Ray / AIPerf:

* ``--configs "dcp:ctx:comm:tpa;..."`` - one entry per (server shape, context length); every
  ``--concurrency`` level runs for each entry (``:864-916``);
* the server is restarted only when ``dcp:comm:tpa`` changes (``:889-903``);
* every (mode, context, concurrency) point writes its own JSON; existing points are skipped unless
  ``--force`` - a killed sweep resumes where it stopped (``:307-311``, ``:811-813``);
* ``--deadline-min``: no new configuration starts when less than ``--min-config-min`` is left (``:883-887``);
* ``--sanity``: concurrency 1, 3 requests; ``--dry-run``: print commands, start nothing (``:72-84``);
* ``HELIX_A2A_BACKEND`` (``--helix-backend``) selects NCCL or the native kernel inside the hook.

    python -m benchmarks.serving.serve_sweep --model DIR --tp 2 --configs "2:32768:a2a:;1:32768::" \
        --concurrency 1,4 --helix-backend native --results results/serving [--load-format dummy] [--dry-run]
"""
from __future__ import annotations

import argparse
import json
import os
import shlex
import subprocess
import sys
import time
from typing import List, Tuple

from .server import Server, ServerConfig, build_vllm_cmd


def parse_configs(text: str) -> List[Tuple[int, int, str, str]]:
    out = []
    for entry in [e.strip() for e in text.split(";") if e.strip()]:
        parts = entry.split(":")
        if len(parts) < 2 or len(parts) > 4:
            raise ValueError(f"config entry '{entry}' is not dcp:ctx[:comm[:tpa]]")
        parts += [""] * (4 - len(parts))
        dcp, ctx = int(parts[0]), int(parts[1])
        if dcp < 1 or ctx < 1:
            raise ValueError(f"config entry '{entry}': dcp and ctx must be positive")
        if parts[2] not in ("", "ag_rs", "a2a"):
            raise ValueError(f"config entry '{entry}': comm must be empty, ag_rs or a2a")
        out.append((dcp, ctx, parts[2], parts[3]))
    return out


def format_context(ctx: int) -> str:
    return f"{ctx // 1048576}M" if ctx >= 1048576 and ctx % 1048576 == 0 else f"{ctx // 1024}K" if ctx >= 1024 else str(ctx)


def point_path(results: str, model_short: str, tp: int, backend: str, mode: str, ctx: int, conc: int) -> str:
    return os.path.join(results, f"{model_short}_tp{tp}_{mode}_{backend}", f"load_ctx{ctx}_c{conc}.json")


def loadgen_cmd(a, url: str, ctx: int, conc: int, out: str) -> List[str]:
    input_len = max(ctx - a.output_tokens - 100, 1)
    count = conc * (3 if a.sanity else a.requests_per_conc)
    return [sys.executable, "-m", "benchmarks.serving.loadgen", "--url", url, "--model", a.model,
            "--input-tokens", str(input_len), "--output-tokens", str(a.output_tokens), "--concurrency", str(conc),
            "--request-count", str(count), "--warmup-request-count", str(conc), "--vocab", str(a.vocab),
            "--seed", str(a.seed), "--out", out]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--configs", default="2:32768:a2a:;1:32768::")
    ap.add_argument("--concurrency", default="1,2,4,8")
    ap.add_argument("--requests-per-conc", type=int, default=5)
    ap.add_argument("--output-tokens", type=int, default=256)
    ap.add_argument("--max-model-len", type=int, default=0, help="0: the largest context of --configs")
    ap.add_argument("--helix-backend", default=os.environ.get("HELIX_A2A_BACKEND", "native"), choices=["nccl", "native"])
    ap.add_argument("--attention-backend", default="")
    ap.add_argument("--load-format", default="")
    ap.add_argument("--quantization", default="")
    ap.add_argument("--vocab", type=int, default=2048)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--results", default="results/serving")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--sanity", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--deadline-min", type=float, default=0.0, help="stop starting configurations after this many minutes")
    ap.add_argument("--min-config-min", type=float, default=10.0)
    ap.add_argument("--ready-timeout-s", type=float, default=1200.0)
    ap.add_argument("--extra-server-args", default="")
    a = ap.parse_args(argv)

    configs = parse_configs(a.configs)
    concs = [1] if a.sanity else [int(c) for c in a.concurrency.split(",") if c.strip()]
    force = a.force or a.sanity
    model_short = os.path.basename(os.path.normpath(a.model))
    max_len = a.max_model_len or max(c[1] for c in configs)
    t_start = time.time()
    total_points = len(configs) * len(concs)
    server = None
    prev_key = ""
    point = done_cfgs = 0
    summary = []
    try:
        for idx, (dcp, ctx, comm, tpa) in enumerate(configs):
            cfg = ServerConfig(model=a.model, tp=a.tp, dcp=dcp, comm=comm, tpa=tpa, max_model_len=max_len,
                               attention_backend=a.attention_backend, load_format=a.load_format, port=a.port,
                               quantization=a.quantization, extra_args=a.extra_server_args)
            mode = cfg.mode_name
            print(f"======== [{idx + 1}/{len(configs)}] {mode} ctx={format_context(ctx)} backend={a.helix_backend} ========", flush=True)
            paths = [point_path(a.results, model_short, a.tp, a.helix_backend, mode, ctx, c) for c in concs]
            if not force and all(os.path.isfile(p) for p in paths):
                print("SKIP: all points exist", flush=True)
                point += len(concs)
                done_cfgs += 1
                continue
            if a.deadline_min > 0:
                left = a.deadline_min - (time.time() - t_start) / 60.0
                if left < a.min_config_min:
                    print(f"TIME: {left:.1f} min left < {a.min_config_min} min needed; stopping", flush=True)
                    break
            if cfg.key != prev_key:
                if server is not None:
                    print(f"server key changed: {prev_key} -> {cfg.key}", flush=True)
                    server.stop()
                    server = None
                log = os.path.join(a.results, "logs", f"vllm_{mode}_{a.helix_backend}.log")
                if a.dry_run:
                    print("[dry-run] HELIX_A2A_BACKEND=" + a.helix_backend + " " + " ".join(shlex.quote(x) for x in build_vllm_cmd(cfg)), flush=True)
                else:
                    server = Server(cfg, a.helix_backend, log)
                    if not server.start(a.ready_timeout_s):
                        print(f"ERROR: vLLM did not come up for {mode} (see {log}); skipping", flush=True)
                        server.stop()
                        server, prev_key = None, ""
                        continue
                prev_key = cfg.key
            else:
                print(f"reusing server ({cfg.key})", flush=True)
            for conc, path in zip(concs, paths):
                point += 1
                print(f"--- [{point}/{total_points}] {mode} ctx={format_context(ctx)} c={conc} ---", flush=True)
                if os.path.isfile(path) and not force:
                    print("  SKIP: already exists", flush=True)
                    continue
                cmd = loadgen_cmd(a, f"http://127.0.0.1:{a.port}", ctx, conc, path)
                if a.dry_run:
                    print("  [dry-run] " + " ".join(shlex.quote(x) for x in cmd), flush=True)
                    continue
                os.makedirs(os.path.dirname(path), exist_ok=True)
                t0 = time.time()
                r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                took = time.time() - t0
                res = json.load(open(path)) if os.path.isfile(path) else None
                if res is not None and res.get("completed", 0) == 0:
                    os.remove(path)          # a point without one completed request is not a result: re-run on resume
                    print(f"  FAILED: no request completed ({took:.0f}s): {res.get('errors')}", flush=True)
                elif res is not None:
                    summary.append({"mode": mode, "ctx": ctx, "concurrency": conc,
                                    "tok_per_s": res["output_token_throughput_per_s"],
                                    "itl_ms_mean": res["inter_token_latency_ms"].get("mean"),
                                    "ttft_ms_mean": res["time_to_first_token_ms"].get("mean")})
                    print(f"  OK ({took:.0f}s): {res['output_token_throughput_per_s']:.1f} tok/s", flush=True)
                else:
                    print(f"  FAILED exit={r.returncode} ({took:.0f}s)\n    " + "\n    ".join(r.stdout.strip().splitlines()[-5:]), flush=True)
            done_cfgs += 1
    finally:
        if server is not None:
            server.stop()
    print(f"all configs processed ({done_cfgs}/{len(configs)})", flush=True)
    if summary:
        print(json.dumps({"backend": a.helix_backend, "points": summary}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
