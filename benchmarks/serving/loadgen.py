"""Closed-loop load generator for an OpenAI-compatible ``/v1/completions`` endpoint (streaming).

Stands in for the AIPerf runs of the reference's end-to-end benchmark
(``benchmark/sbatch/run_gb200_aiperf_v3.sbatch:797-851``): a fixed synthetic prompt of
``--input-tokens`` tokens, ``--output-tokens`` generated tokens per request (``ignore_eos``),
``--concurrency`` requests in flight, ``--request-count`` timed requests after
``--warmup-request-count`` untimed ones.  Per request it records time to first token, the gaps
between streamed chunks and the total latency; the summary (mean / p50 / p90 / p99, output
tokens per second, request rate) is written as one JSON file.

    python -m benchmarks.serving.loadgen --url http://127.0.0.1:8000 --model MODEL \
        --input-tokens 32000 --output-tokens 256 --concurrency 8 --request-count 40 --out result.json
"""
from __future__ import annotations

import argparse
import asyncio
import json
import time
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class RequestRecord:
    ok: bool
    ttft_s: float = 0.0
    latency_s: float = 0.0
    gaps_s: List[float] = field(default_factory=list)
    output_tokens: int = 0
    text: str = ""
    error: str = ""


def percentile(xs: List[float], q: float) -> float:
    if not xs:
        return float("nan")
    s = sorted(xs)
    k = (len(s) - 1) * q
    lo, hi = int(k), min(int(k) + 1, len(s) - 1)
    return s[lo] + (s[hi] - s[lo]) * (k - lo)


def stats(xs: List[float], scale: float = 1.0) -> dict:
    if not xs:
        return {"n": 0}
    return {"n": len(xs), "mean": sum(xs) / len(xs) * scale, "p50": percentile(xs, 0.5) * scale,
            "p90": percentile(xs, 0.9) * scale, "p99": percentile(xs, 0.99) * scale,
            "min": min(xs) * scale, "max": max(xs) * scale}


async def one_request(session, url: str, payload: dict, timeout_s: float) -> RequestRecord:
    import aiohttp
    t0 = time.perf_counter()
    last = t0
    rec = RequestRecord(ok=False)
    pieces = []
    try:
        async with session.post(url.rstrip("/") + "/v1/completions", json=payload,
                                timeout=aiohttp.ClientTimeout(total=timeout_s)) as resp:
            if resp.status != 200:
                rec.error = f"http {resp.status}: {(await resp.text())[:200]}"
                return rec
            usage_tokens: Optional[int] = None
            chunks = 0
            async for raw in resp.content:
                line = raw.decode("utf-8", "replace").strip()
                if not line.startswith("data:"):
                    continue
                body = line[5:].strip()
                if body == "[DONE]":
                    break
                msg = json.loads(body)
                if msg.get("usage") and msg["usage"].get("completion_tokens") is not None:
                    usage_tokens = int(msg["usage"]["completion_tokens"])
                choices = msg.get("choices") or []
                if not choices:
                    continue
                now = time.perf_counter()
                if chunks == 0:
                    rec.ttft_s = now - t0
                else:
                    rec.gaps_s.append(now - last)
                last = now
                chunks += 1
                pieces.append(choices[0].get("text") or "")
            rec.latency_s = time.perf_counter() - t0
            rec.output_tokens = usage_tokens if usage_tokens is not None else chunks
            rec.text = "".join(pieces)
            rec.ok = chunks > 0
            if not rec.ok:
                rec.error = "empty stream"
    except Exception as e:  # noqa: BLE001  (a failed request is a data point, not a crash)
        rec.error = f"{type(e).__name__}: {e}"
    return rec


async def run_load(url: str, model: str, prompt, *, output_tokens: int, concurrency: int, request_count: int,
                   warmup_request_count: int = 0, temperature: float = 0.0, seed: int = 42,
                   timeout_s: float = 3600.0) -> dict:
    import aiohttp
    payload = {"model": model, "prompt": prompt, "max_tokens": output_tokens, "temperature": temperature,
               "stream": True, "ignore_eos": True, "seed": seed, "stream_options": {"include_usage": True}}
    conn = aiohttp.TCPConnector(limit=0)
    async with aiohttp.ClientSession(connector=conn) as session:
        async def phase(n: int) -> List[RequestRecord]:
            out: List[RequestRecord] = []
            todo = iter(range(n))

            async def worker():
                for _ in todo:
                    out.append(await one_request(session, url, payload, timeout_s))

            await asyncio.gather(*[worker() for _ in range(max(1, min(concurrency, n)))])
            return out

        if warmup_request_count > 0:
            await phase(warmup_request_count)
        t0 = time.perf_counter()
        recs = await phase(request_count)
        wall = time.perf_counter() - t0
    good = [r for r in recs if r.ok]
    gaps = [g for r in good for g in r.gaps_s]
    out_tokens = sum(r.output_tokens for r in good)
    return {
        "url": url, "model": model, "concurrency": concurrency, "request_count": request_count,
        "warmup_request_count": warmup_request_count, "output_tokens_per_request": output_tokens,
        "completed": len(good), "failed": len(recs) - len(good),
        "errors": sorted({r.error for r in recs if not r.ok})[:5],
        "wall_s": wall,
        "output_token_throughput_per_s": out_tokens / wall if wall > 0 else 0.0,
        "request_throughput_per_s": len(good) / wall if wall > 0 else 0.0,
        "time_to_first_token_ms": stats([r.ttft_s for r in good], 1e3),
        "inter_token_latency_ms": stats(gaps, 1e3),
        "request_latency_ms": stats([r.latency_s for r in good], 1e3),
        "sample_text": good[0].text[:200] if good else "",
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", required=True)
    ap.add_argument("--input-tokens", type=int, default=1024)
    ap.add_argument("--output-tokens", type=int, default=128)
    ap.add_argument("--concurrency", type=int, default=1)
    ap.add_argument("--request-count", type=int, default=5)
    ap.add_argument("--warmup-request-count", type=int, default=0)
    ap.add_argument("--vocab", type=int, default=2048, help="vocabulary of the word-level synthetic prompt")
    ap.add_argument("--prompt-file", default="", help="use this text instead of the synthetic prompt")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--timeout-s", type=float, default=3600.0)
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    if a.prompt_file:
        prompt = open(a.prompt_file).read()
    else:
        from .tiny_model import synthetic_prompt
        prompt = synthetic_prompt(a.input_tokens, a.seed, a.vocab)
    res = asyncio.run(run_load(a.url, a.model, prompt, output_tokens=a.output_tokens, concurrency=a.concurrency,
                               request_count=a.request_count, warmup_request_count=a.warmup_request_count,
                               seed=a.seed, timeout_s=a.timeout_s))
    res["input_tokens"] = a.input_tokens
    line = json.dumps(res)
    if a.out:
        tmp = a.out + ".tmp"
        with open(tmp, "w") as f:
            f.write(line + "\n")
        import os
        os.replace(tmp, a.out)       # a result file either exists completely or not at all (resumable sweeps)
    print(line)
    return 0 if res["completed"] > 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
