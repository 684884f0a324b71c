#!/bin/bash
# Usage: ./profile_models.sh <autocast_dtype> <sequence_length> <port> [model names...]
# Profiles one transformer block per model on this machine's GPU and updates
# data/model_latencies.json (input of zorse_planner.py).
set -e
DTYPE=${1:-bfloat16}
SEQ=${2:-4096}
PORT=${3:-29533}
shift 3 || true
MODELS=("$@")
if [ ${#MODELS[@]} -eq 0 ]; then
  MODELS=(llama2_7b llama3.2_1b mistral_7b opt_13b deepspeedllama_tiny deepspeedllama_13b)
fi
for m in "${MODELS[@]}"; do
  python -m torch.distributed.run --nnodes=1 --nproc_per_node=1 --master-addr 127.0.0.1 --master-port "$PORT" \
    -m bench.bench_layer --seq_length "$SEQ" --profile_batches 4 --autocast_dtype "$DTYPE" --reduce_dtype float32 --model_name "$m"
done
