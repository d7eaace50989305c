#!/usr/bin/env bash
# Launch one node of a training job (counterpart of the reference's test_script.sh / test_script_imagenet.sh).
#   ./run_train.sh --master-ip-address 10.0.0.1 --my-ip-address 10.0.0.2 --world-size 2 --num-gpus 8 --rank 1 [-- extra train.py flags]
set -euo pipefail
MASTER_IP=127.0.0.1; MY_IP=127.0.0.1; WORLD=1; GPUS=$(python -c 'import torch; print(max(1, torch.cuda.device_count()))'); NODE_RANK=0
MODEL=${TEST_MODEL:-resnet152}; DATASET=dummy; EPOCHS=1
while [[ $# -gt 0 ]]; do
  case "$1" in
    --master-ip-address) MASTER_IP=$2; shift 2;;
    --my-ip-address) MY_IP=$2; shift 2;;
    --world-size) WORLD=$2; shift 2;;
    --num-gpus) GPUS=$2; shift 2;;
    --rank) NODE_RANK=$2; shift 2;;
    --imagenet) DATASET=imagenet100; EPOCHS=100; shift;;
    --) shift; break;;
    *) echo "unknown flag $1" >&2; exit 2;;
  esac
done
export MASTER_ADDR=$MASTER_IP PUBLIC_IP=$MY_IP MASTER_PORT=${MASTER_PORT:-5555} WORLD_SIZE=$WORLD NUM_GPUS=$GPUS RANK=$NODE_RANK
cd "$(dirname "$0")"
exec python -m stellatrain_b200.train --model="$MODEL" --dataset="$DATASET" --num-epochs="$EPOCHS" \
  --local-world-size="$GPUS" --batch-size=72 --compression=0.95 --scale-lr "$@"
