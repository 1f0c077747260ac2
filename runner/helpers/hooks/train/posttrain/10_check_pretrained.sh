#!/usr/bin/env bash
# Stage hook (train posttrain): supervised fine-tuning normally starts from a checkpoint; warn when none is named.
for a in "$@"; do
  [[ "$a" == --load* || "$a" == load=* || "$a" == --pretrained_checkpoint* ]] && exit 0
done
echo "no --load / --pretrained_checkpoint given: fine-tuning starts from random weights"
