#!/usr/bin/env bash
# Launch GPT-MoE training on the GPUs of this node (counterpart of the reference's scripts/run_real_moe.sh,
# without Megatron).  Knobs come from the environment, as there:
#   MODEL           recipe name (launch/recipes.py); default gpt_moe_1b        NUM_LAYERS   depth override
#   NPROC           GPUs to use (default: all visible)                         GPUS_PER_NODE ranks per logical domain
#   EPLB_MODE       off | observe | apply (default apply)                      EPLB_N_SLOT  total expert slots per rank
#   ROUTER_SKEW     scale of the drifting router-logit bias                    EPLB_TRACE_OUT/MAX/EVERY  routing trace
#   ROUTER_BALANCING none (default: the skew reaches the dispatcher) | aux_loss (switch-style auxiliary loss)
#   EPLB_ADAPTER    fused (default) | alltoall                                  SKIP_PREFLIGHT=1 skips the validation
#   TRAIN_ITERS, MICRO_BATCH, NUM_MICRO_BATCHES, SEQ_LEN, LR, SAVE, LOAD, SAVE_INTERVAL, DATA, MASTER_PORT
# Extra arguments are passed to ep_balance_b200.launch.train_gpt_moe unchanged.
set -euo pipefail
NPROC="${NPROC:-$(python -c 'import torch; print(max(torch.cuda.device_count(), 1))')}"
export MODEL="${MODEL:-gpt_moe_1b}"
export EPLB_MODE="${EPLB_MODE:-apply}"
export GPUS_PER_NODE="${GPUS_PER_NODE:-$NPROC}"
# Reject knob combinations that cannot work before any process starts (launch/preflight.py).
if [ "${SKIP_PREFLIGHT:-0}" = "0" ]; then
  NPROC="$NPROC" python -m ep_balance_b200.launch.preflight --nproc "$NPROC"
fi
args=(--steps "${TRAIN_ITERS:-20}" --micro-batch "${MICRO_BATCH:-4}" --num-micro-batches "${NUM_MICRO_BATCHES:-1}"
      --seq-len "${SEQ_LEN:-2048}" --lr "${LR:-1e-4}")
[ -n "${SAVE:-}" ] && args+=(--save "$SAVE" --save-interval "${SAVE_INTERVAL:-0}")
[ -n "${LOAD:-}" ] && args+=(--load "$LOAD")
[ -n "${DATA:-}" ] && args+=(--data "$DATA")
if [ "$NPROC" -gt 1 ]; then
  exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NPROC" --master-addr 127.0.0.1 \
       --master-port "${MASTER_PORT:-29521}" -m ep_balance_b200.launch.train_gpt_moe "${args[@]}" "$@"
else
  exec python -m ep_balance_b200.launch.train_gpt_moe "${args[@]}" "$@"
fi
