#!/usr/bin/env bash
# HF safetensors -> torch_dist (and back): convert_ckpt.sh hf2mcore qwen2.5-7b /path/hf /path/ckpt
set -euo pipefail
cd "$(dirname "$0")/../../.."
exec python -m gcore_b200.tools.ckpt_convert "$1" --model "$2" --src "$3" --dst "$4"
