#!/usr/bin/env bash
# ./run_tests.sh          CPU tier (host stand-ins for GPUs, gloo, child processes)
# ./run_tests.sh gpu      GPU tier on the visible B200s
set -euo pipefail
cd "$(dirname "$0")"
./build.sh
if [ "${1:-cpu}" = "gpu" ]; then
  python -m pytest tests -q -m gpu
else
  python -m pytest tests -q -m "not gpu"
fi
