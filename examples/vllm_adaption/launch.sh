#!/bin/bash
# Serves a model with vLLM and flexkv_b200 as its KV connector, without patching vLLM: vLLM's built-in
# FlexKVConnectorV1 imports `flexkv.integration.vllm.vllm_v1_adapter`, which the alias package under compat/
# maps onto this implementation.
#
#   MODEL=/models/Qwen3-8B TP=1 ./launch.sh
set -euo pipefail
REPO="$(cd "$(dirname "$0")/../.." && pwd)"
export PYTHONPATH="$REPO/compat:$REPO:${PYTHONPATH:-}"
export FLEXKV_CONFIG_PATH="${FLEXKV_CONFIG_PATH:-$REPO/examples/flexkv_config.yml}"
export FLEXKV_ENABLE_METRICS="${FLEXKV_ENABLE_METRICS:-1}"        # Prometheus on :8080 (Python) and :8081 (native)
MODEL="${MODEL:?set MODEL to a model path or name}"
TP="${TP:-1}"
PORT="${PORT:-8000}"

exec vllm serve "$MODEL" \
  --tensor-parallel-size "$TP" \
  --port "$PORT" \
  --enable-prefix-caching \
  --kv-transfer-config '{"kv_connector":"FlexKVConnectorV1","kv_role":"kv_both"}' \
  "$@"
