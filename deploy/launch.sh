#!/usr/bin/env bash
# Starts one rank per GPU on this node of a (multi-node) job (counterpart of the reference's deploy/ scripts, which build
# the tree and launch a Legion job; here there is nothing to build per node beyond `python build.py`).
#
#   deploy/launch.sh <nnodes> <node_rank> <master_addr> <script.py | -m module> [args...]
#
# Single node: deploy/launch.sh 1 0 127.0.0.1 -m flexflow_train_b200.bin.run_model --model transformer_lm ...
# Every node runs the same command with its own <node_rank>; GPUS_PER_NODE and MASTER_PORT can be set in the environment.
set -euo pipefail
if [ "$#" -lt 4 ]; then
  sed -n '2,9p' "$0"
  exit 2
fi
NNODES=$1; NODE_RANK=$2; MASTER_ADDR=$3; shift 3
GPUS_PER_NODE=${GPUS_PER_NODE:-$(python -c 'import torch; print(torch.cuda.device_count())')}
MASTER_PORT=${MASTER_PORT:-29500}
cd "$(dirname "$0")/.."
[ -f flexflow_train_b200/libffk.so ] || python build.py
exec python -m torch.distributed.run --nnodes "$NNODES" --node-rank "$NODE_RANK" --nproc-per-node "$GPUS_PER_NODE" \
  --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" "$@"
