#!/usr/bin/env bash
# One 8 x B200 node: trainer TP=2 x DP=4 colocated with a TP=2 rollout engine.
set -euo pipefail
cd "$(dirname "$0")/../../.."
python -m gcore_b200.build_native
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${GPUS:-8}" --master-addr 127.0.0.1 \
    --master-port "${PORT:-29500}" -m gcore_b200.entry.train_lm_grpo \
    --config "${CONFIG:-tasks/math_rl/yaml/grpo_qwen2.5_7b.yaml}" "$@"
