"""Batch-dictionary keys and sentinel values shared by loaders, models and plugins
(same names and values as the reference's ``utils/constants.py:3-29``; they are part of the batch contract)."""
from __future__ import annotations

IGNORE_INDEX = -100      # label value that does not contribute to the loss
PAD_SEQUENCE_ID = -1     # sequence id of padding tokens in packed batches

INPUT_IDS_KEY = "input_ids"
LABELS_KEY = "labels"
POSITION_IDS_KEY = "position_ids"
SEQUENCE_IDS_KEY = "sequence_ids"
POSITION_OFFSET_KEY = "position_offset"
LOSS_WEIGHT_KEY = "loss_weight"
#: per-row ``[rows, 2]`` (local targets, targets over the whole context-parallel group) behind ``loss_weight``: lets a
#: pipeline runner that cuts the batch into micro-batches give every piece its own exact weight
LOSS_TARGET_COUNTS_KEY = "loss_target_counts"
#: weight of token-count based auxiliary losses (expert load balance) of a rank that holds ``1 / cp`` of every sequence:
#: context-parallel gradients are SUMMED over the group, so an unweighted local term would count ``cp`` times
AUX_LOSS_WEIGHT_KEY = "auxiliary_loss_weight"
#: 0-dim tensor: this rank's targets x data-parallel size / targets of all data-parallel ranks in this micro-step
#: (``runtime/plugins/token_weighted_loss.py``); multiplies the cross-entropy so that the data-parallel gradient average is
#: the mean over TARGETS rather than the mean of the ranks' means
LOSS_SCALE_KEY = "loss_scale"
HIDDEN_STATES_KEY = "hidden_states"

MODEL_BATCH_KEYS = (
    INPUT_IDS_KEY, LABELS_KEY, POSITION_IDS_KEY, SEQUENCE_IDS_KEY,
    POSITION_OFFSET_KEY, LOSS_WEIGHT_KEY, AUX_LOSS_WEIGHT_KEY, LOSS_SCALE_KEY, HIDDEN_STATES_KEY,
)
SFT_BATCH_KEYS = (INPUT_IDS_KEY, LABELS_KEY, POSITION_IDS_KEY, SEQUENCE_IDS_KEY)
