#!/usr/bin/env bash
# Start the OpenAI-compatible server.
#   ./run_server.sh Qwen/Qwen-Image --ulysses-degree 4 --cfg-parallel-size 2        (diffusion)
#   ./run_server.sh Qwen/Qwen3-Omni-30B-A3B-Instruct --omni                         (three stages)
set -euo pipefail
MODEL="${1:?model name or path}"
shift
exec python -m vllm_omni_b200.entrypoints.cli.main serve "$MODEL" --host 127.0.0.1 --port 8000 "$@"
