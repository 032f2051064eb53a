#!/bin/bash
# Dense 0.25B-class GPT on real text (fineweb-edu through pretrain_example.py; needs network or a local copy). Same environment-variable interface as the
# reference launcher of the same name:
#   NUM_NODES NUM_GPUS NODE_RANK MASTER_ADDR MASTER_PORT LR_WARMUP_STEPS MAX_LR MIN_LR
#   SEED BATCH_SIZE SEQ_LEN GBS SEP_SIZE USE_COMPILE DEBUG DETER_MODE
set -euo pipefail
cd "$(dirname "$0")/../.."

NUM_NODES=${NUM_NODES:-1}
NUM_GPUS=${NUM_GPUS:-8}
NODE_RANK=${NODE_RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-29500}
LR_WARMUP_STEPS=${LR_WARMUP_STEPS:-2}
MAX_LR=${MAX_LR:-6e-4}
MIN_LR=${MIN_LR:-6e-5}
SEED=${SEED:-1337}
BATCH_SIZE=${BATCH_SIZE:-8}          # sequences per GPU
SEQ_LEN=${SEQ_LEN:-4096}
GBS=${GBS:-1024}                     # global batch in sequences
SEP_SIZE=${SEP_SIZE:-1}
USE_COMPILE=${USE_COMPILE:-1}
DEBUG=${DEBUG:-1}
DETER_MODE=${DETER_MODE:-1}

TOTAL_BATCH_SIZE=$((GBS * SEQ_LEN))
BATCH_SIZE_PER_DP_RANK=$((BATCH_SIZE * SEP_SIZE))   # a DP rank is a whole SEP group

ARGS="--exp_name example_gpt_0.25b --seed $SEED --log_dir ./log \
  --total_batch_size $TOTAL_BATCH_SIZE --batch_size $BATCH_SIZE_PER_DP_RANK --seq_len $SEQ_LEN \
  --max_lr $MAX_LR --min_lr $MIN_LR --weight_decay 0.1 --grad_clip_value 1.0 --warmup_steps $LR_WARMUP_STEPS \
  --max_epochs 1 --do_save --save_every_steps 500 \
  --sep_size $SEP_SIZE --use_distributed_optimizer \
  --block_size 4096 --vocab_size 50304 --num_layer 12 --num_attention_heads 32 --num_key_value_heads 4 \
  --hidden_size 1024 --intermediate_size 4096 --tied_lm_head --dropout 0.0"
[ "$DEBUG" -eq 1 ] && ARGS="$ARGS --debug"
[ "$USE_COMPILE" -eq 1 ] && ARGS="$ARGS --use_compile"
[ "$DETER_MODE" -eq 1 ] && ARGS="$ARGS --deterministic"

python -m train_large_model_from_scratch_b200.build_ext
exec python -m torch.distributed.run --nnodes "$NUM_NODES" --nproc-per-node "$NUM_GPUS" --node-rank "$NODE_RANK" \
  --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" pretrain_example.py $ARGS
