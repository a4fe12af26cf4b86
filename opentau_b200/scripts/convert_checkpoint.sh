#!/usr/bin/env bash
# Consolidate the per-rank optimizer shards of a training checkpoint into one fp32 safetensors file
# (counterpart of the reference's convert_checkpoint.sh, which calls DeepSpeed's zero_to_fp32.py).
#
#   convert_checkpoint.sh <output_dir>/checkpoints/000040 [--moments]
set -euo pipefail
ckpt="${1:?usage: convert_checkpoint.sh <checkpoint_dir> [--moments]}"
shift
python -m opentau_b200.scripts.zero_to_fp32 "$ckpt" "$ckpt/model_fp32.safetensors" "$@"
