#!/bin/bash
# GPT-MoE pre-training with Megatron-LM core_r0.9.0 + planmoe experts on one node.
GPUS_PER_NODE=${GPUS_PER_NODE:-4}
MEGATRON=${MEGATRON:-./Megatron-LM}
DATA=${DATA:-./data/gpt2_text_document}
torchrun --nproc_per_node $GPUS_PER_NODE --nnodes 1 --master_addr 127.0.0.1 --master_port 6000 \
  $MEGATRON/pretrain_gpt.py \
  --num-layers 24 --hidden-size 1024 --ffn-hidden-size 4096 --num-attention-heads 16 \
  --seq-length 1024 --max-position-embeddings 1024 \
  --num-experts 8 --moe-router-topk 2 --moe-expert-capacity-factor 1.5 --expert-model-parallel-size $GPUS_PER_NODE \
  --tensor-model-parallel-size 1 --pipeline-model-parallel-size 1 \
  --micro-batch-size 2 --global-batch-size 32 --train-iters 500000 --lr 1.5e-4 --min-lr 1.0e-5 \
  --lr-decay-style cosine --weight-decay 1e-2 --clip-grad 1.0 --bf16 \
  --data-path $DATA --vocab-file ./data/gpt2-vocab.json --merge-file ./data/gpt2-merges.txt --split 949,50,1 \
  --log-interval 10 --save-interval 10000 --eval-interval 1000 --eval-iters 10 \
  --schemoe --schemoe-overlap-degree ${DEGREE:-auto} --schemoe-compress-name ${CODEC:-no} --schemoe-comm-name ${COMM:-naive}
