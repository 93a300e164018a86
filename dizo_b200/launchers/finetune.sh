#!/bin/bash
# Usage (same variables as the reference's large_models/finetune.sh):
#   MODEL=/path/to/opt-13b TASK=SST2 MODE=ft ENHANCED=zo NUM_GPU=1 bash finetune.sh [extra run arguments]
exec python -m dizo_b200.launch finetune "$@"
