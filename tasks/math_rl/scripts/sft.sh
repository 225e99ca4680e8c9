#!/usr/bin/env bash
set -euo pipefail
cd "$(dirname "$0")/../../.."
python -m gcore_b200.build_native
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${GPUS:-8}" --master-addr 127.0.0.1 \
    --master-port "${PORT:-29500}" -m gcore_b200.entry.train_lm_finetune \
    --config "${CONFIG:-tasks/math_rl/yaml/sft_long_context_cp4_tp2.yaml}" "$@"
