"""Per-module incremental-state bookkeeping.

Same contract as the reference's ``with_incremental_state`` mixin
(fairseq/incremental_decoding_utils.py:12-50): every module instance owns a random id and
stores its buffers in the shared ``incremental_state`` dict under ``"<id>.<key>"``.
"""
import uuid
from typing import Dict, Optional

from torch import Tensor

StateDict = Dict[str, Dict[str, Optional[Tensor]]]


class IncrementalStateMixin:
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.init_incremental_state()

    def init_incremental_state(self):
        self._incremental_state_id = str(uuid.uuid4())

    def _get_full_incremental_state_key(self, key: str) -> str:
        return "%s.%s" % (self._incremental_state_id, key)

    def get_incremental_state(self, incremental_state: Optional[StateDict], key: str):
        if incremental_state is None:
            return None
        return incremental_state.get(self._get_full_incremental_state_key(key))

    def set_incremental_state(self, incremental_state: Optional[StateDict], key: str, value):
        if incremental_state is not None:
            incremental_state[self._get_full_incremental_state_key(key)] = value
        return incremental_state

    def _reorder_buffer(self, incremental_state, key, new_order):
        buf = self.get_incremental_state(incremental_state, key)
        if buf is not None:
            for k, v in buf.items():
                if v is not None:
                    buf[k] = v.index_select(0, new_order)
            self.set_incremental_state(incremental_state, key, buf)
        return incremental_state


def require_no_grad(*tensors):
    """Entry points that carry an incremental state (decode helpers) are inference-only."""
    import torch
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors):
        raise NotImplementedError(
            "this entry point is an inference helper (incremental state, single-step update): call it "
            "under torch.no_grad(); the differentiable path is the module's forward")
