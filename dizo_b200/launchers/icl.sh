#!/bin/bash
# Usage (same variables as the reference's large_models/icl.sh):
#   MODEL=/path/to/opt-13b TASK=SST2 MODE=ft ENHANCED=zo NUM_GPU=1 bash icl.sh [extra run arguments]
exec python -m dizo_b200.launch icl "$@"
