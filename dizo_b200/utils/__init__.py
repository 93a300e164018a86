"""Helpers: prompt encoding, collators, callbacks (``common``) and checkpoints (``checkpoint``)."""
from .common import (DataCollatorForTokenClassification, DataCollatorWithPaddingAndNesting,
                     EnhancedJSONEncoder, ICLCollator, NondiffCollator, Prediction, SIGUSR1Callback,
                     StubTokenizer, TrainerCallback, TrainerControl, count_time, encode_prompt,
                     pad_sequences, temp_seed, write_metrics_to_file, write_predictions_to_file)

__all__ = ["DataCollatorForTokenClassification", "DataCollatorWithPaddingAndNesting",
           "EnhancedJSONEncoder", "ICLCollator", "NondiffCollator", "Prediction", "SIGUSR1Callback",
           "StubTokenizer", "TrainerCallback", "TrainerControl", "count_time", "encode_prompt",
           "pad_sequences", "temp_seed", "write_metrics_to_file", "write_predictions_to_file"]
