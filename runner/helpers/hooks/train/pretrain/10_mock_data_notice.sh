#!/usr/bin/env bash
# Stage hook (train pretrain): without --data_path the run uses the synthetic token stream; say so once.
for a in "$@"; do
  [[ "$a" == --data_path* || "$a" == data_path=* ]] && exit 0
done
echo "no --data_path given: pre-training runs on mock data (NullTokenizer)"
