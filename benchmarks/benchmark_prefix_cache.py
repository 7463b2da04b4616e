#!/usr/bin/env python
"""Serving-level check of the host-tier restore behind an OpenAI-compatible endpoint.

The same long prompt is sent three times to a running vLLM or SGLang server that was started with the
flexkv_b200 connector:

  1. cold          nothing cached anywhere: full prefill;
  2. engine hit    the engine's own prefix cache in HBM answers;
  3. restore hit   the engine's prefix cache was flushed in between (`--flush-url`), so the prefix comes back
                   from the host tier through the connector.

The generated text of the three requests must be identical (greedy decoding); latencies to the first token
are reported. Same purpose as the reference's benchmarks/benchmark_prefix_cache.py. Needs a running server,
so nothing here is exercised by the test suite.

    python benchmarks/benchmark_prefix_cache.py --model <served name> --port 8000 \
        --flush-url http://127.0.0.1:8000/flush_cache            # SGLang
        --flush-url http://127.0.0.1:8000/reset_prefix_cache     # vLLM (server in dev mode)
"""
import argparse
import json
import random
import sys
import time

import requests


def first_token_and_text(base: str, model: str, prompt: str, max_tokens: int, timeout: float):
    """Streams one completion; returns (seconds to the first token, seconds in total, text)."""
    body = {"model": model, "prompt": prompt, "max_tokens": max_tokens, "temperature": 0.0, "stream": True}
    t0 = time.perf_counter()
    first, parts = None, []
    with requests.post(base + "/v1/completions", json=body, stream=True, timeout=timeout) as r:
        r.raise_for_status()
        for line in r.iter_lines():
            if not line or not line.startswith(b"data:"):
                continue
            payload = line[5:].strip()
            if payload == b"[DONE]":
                break
            piece = json.loads(payload)["choices"][0].get("text", "")
            if piece and first is None:
                first = time.perf_counter() - t0
            parts.append(piece)
    return first if first is not None else float("nan"), time.perf_counter() - t0, "".join(parts)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True, help="model name as the server knows it")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--prompt-words", type=int, default=6000, help="length of the synthetic prompt")
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--flush-url", default="", help="POSTed between request 2 and 3 to drop the engine's HBM prefix cache")
    ap.add_argument("--settle-s", type=float, default=2.0, help="wait after request 1 so that the offload completes")
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    base = f"http://{a.host}:{a.port}"
    rng = random.Random(a.seed)
    words = ["".join(rng.choice("abcdefghijklmnopqrstuvwxyz") for _ in range(rng.randint(3, 9)))
             for _ in range(a.prompt_words)]
    prompt = " ".join(words) + "\nSummarise the text above in one sentence:"
    rows = []
    for name in ("cold", "engine_hit", "restore_hit"):
        if name == "restore_hit":
            if not a.flush_url:
                print("no --flush-url: the third request would hit the engine's own cache again; stopping after two",
                      file=sys.stderr)
                break
            requests.post(a.flush_url, timeout=60).raise_for_status()
        ttft, total, text = first_token_and_text(base, a.model, prompt, a.max_tokens, a.timeout)
        rows.append(dict(request=name, ttft_s=round(ttft, 4), total_s=round(total, 4), text=text))
        if name == "cold":
            time.sleep(a.settle_s)
    same = len({r["text"] for r in rows}) == 1
    out = dict(benchmark="prefix_cache_three_requests", model=a.model, prompt_words=a.prompt_words,
               requests=[{k: v for k, v in r.items() if k != "text"} for r in rows], outputs_identical=same)
    if len(rows) == 3:
        out["restore_over_cold_ttft"] = round(rows[2]["ttft_s"] / rows[0]["ttft_s"], 3)
    print(json.dumps(out))
    return 0 if same else 1


if __name__ == "__main__":
    sys.exit(main())
