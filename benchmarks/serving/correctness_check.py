"""End-to-end check: the same prompts, greedy decoding, served once with the NCCL exchange and once
with the Helix kernel; the generated texts must be identical.

Counterpart of ``benchmark/scripts/correctness_check.sh:162-283`` for one box.  Every prompt is
sent with ``temperature 0`` and a fixed seed; the two runs are compared string by string, and the
share of matching prompts plus the first differing position are reported.  With random (dummy)
weights the logits are nearly flat, so a last-bit difference between the two combine
implementations can flip an argmax late in a generation: ``--min-match-tokens`` says how long the
common prefix must be for a prompt to count as matching (default: the whole generation).

    python -m benchmarks.serving.correctness_check --model DIR --tp 2 --dcp 2 --load-format dummy \
        --prompts 8 --input-tokens 2048 --output-tokens 32 --out result.json
"""
from __future__ import annotations

import argparse
import json
import os
import shlex
import urllib.request
from typing import List

from .server import Server, ServerConfig, build_vllm_cmd
from .tiny_model import synthetic_prompt


def complete(url: str, model: str, prompt: str, max_tokens: int, timeout_s: float = 600.0) -> str:
    body = json.dumps({"model": model, "prompt": prompt, "max_tokens": max_tokens, "temperature": 0.0, "seed": 0,
                       "ignore_eos": True}).encode()
    req = urllib.request.Request(url.rstrip("/") + "/v1/completions", data=body, headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout_s) as r:
        return json.loads(r.read())["choices"][0]["text"]


def common_prefix_words(a: str, b: str) -> int:
    n = 0
    for x, y in zip(a.split(), b.split()):
        if x != y:
            break
        n += 1
    return n


def compare(texts_a: List[str], texts_b: List[str], min_match_tokens: int) -> dict:
    rows, matched = [], 0
    for i, (x, y) in enumerate(zip(texts_a, texts_b)):
        same = x == y
        pre = common_prefix_words(x, y)
        ok = same or (min_match_tokens > 0 and pre >= min_match_tokens)
        matched += ok
        rows.append({"prompt": i, "identical": same, "common_prefix_tokens": pre, "ok": ok})
    return {"prompts": len(rows), "matched": matched, "all_match": matched == len(rows), "rows": rows}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--dcp", type=int, default=2)
    ap.add_argument("--comm", default="a2a")
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--input-tokens", type=int, default=2048)
    ap.add_argument("--output-tokens", type=int, default=32)
    ap.add_argument("--min-match-tokens", type=int, default=0)
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--attention-backend", default="")
    ap.add_argument("--load-format", default="")
    ap.add_argument("--vocab", type=int, default=2048)
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--backends", default="nccl,native")
    ap.add_argument("--logs", default="results/serving/logs")
    ap.add_argument("--ready-timeout-s", type=float, default=1200.0)
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.0)
    ap.add_argument("--extra-server-args", default="")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)

    cfg = ServerConfig(model=a.model, tp=a.tp, dcp=a.dcp, comm=a.comm, max_model_len=a.max_model_len,
                       attention_backend=a.attention_backend, load_format=a.load_format, port=a.port,
                       enforce_eager=a.enforce_eager, gpu_memory_utilization=a.gpu_memory_utilization,
                       extra_args=a.extra_server_args)
    prompts = [synthetic_prompt(a.input_tokens, seed=1000 + i, vocab=a.vocab) for i in range(a.prompts)]
    backends = [b.strip() for b in a.backends.split(",") if b.strip()]
    outputs = {}
    for backend in backends:
        if a.dry_run:
            print(f"[dry-run] HELIX_A2A_BACKEND={backend} " + " ".join(shlex.quote(x) for x in build_vllm_cmd(cfg)))
            print(f"[dry-run] {len(prompts)} prompts x {a.input_tokens} tokens, {a.output_tokens} generated, temperature 0")
            continue
        log = os.path.join(a.logs, f"correctness_{backend}.log")
        server = Server(cfg, backend, log)
        try:
            if not server.start(a.ready_timeout_s):
                print(f"ERROR: server with backend {backend} did not come up; see {log}")
                return 2
            outputs[backend] = [complete(server.url, a.model, p, a.output_tokens) for p in prompts]
            print(f"{backend}: {len(outputs[backend])} completions; first: {outputs[backend][0][:80]!r}", flush=True)
        finally:
            server.stop()
    if a.dry_run:
        return 0
    res = compare(outputs[backends[0]], outputs[backends[-1]], a.min_match_tokens)
    res.update({"backends": backends, "tp": a.tp, "dcp": a.dcp, "comm": a.comm, "input_tokens": a.input_tokens,
                "output_tokens": a.output_tokens})
    line = json.dumps(res)
    if a.out:
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        with open(a.out, "w") as f:
            f.write(line + "\n")
    print(line)
    print("PASS: outputs match" if res["all_match"] else f"MISMATCH: {res['prompts'] - res['matched']} of {res['prompts']} prompts differ")
    return 0 if res["all_match"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
