#!/bin/bash
# transformer_lm_gpt2_tiny with every MOE-th decoder layer as a planmoe moe_layer (top-2, dynamic capacity).
MOE=${MOE:-1} L_AUX_WT=${L_AUX_WT:-0.01} NO_OVERFLOW=${NO_OVERFLOW:-0} \
python3 -m planmoe_b200.launcher.run fairseq-train ${DATA:-./wikitext-103} \
  --task language_modeling --arch transformer_lm_gpt2_tiny --ddp-backend legacy_ddp \
  --share-decoder-input-output-embed --dropout 0.1 --optimizer adam --adam-betas '(0.9, 0.98)' \
  --weight-decay 0.01 --clip-norm 0.0 --lr 0.0005 --lr-scheduler inverse_sqrt --warmup-updates 4000 \
  --warmup-init-lr 1e-07 --tokens-per-sample 256 --sample-break-mode none --batch-size 8 --fp16 \
  --max-update 50000 --save-dir ./checkpoints
